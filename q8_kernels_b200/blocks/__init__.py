"""Drop-in for ``q8_kernels.blocks`` (reference: q8_kernels/blocks/)."""
from .ltx_transformer_block import LTXTransformerBlock

__all__ = ["LTXTransformerBlock"]

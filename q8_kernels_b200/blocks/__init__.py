"""Drop-in for ``q8_kernels.blocks`` (reference: q8_kernels/blocks/) plus the 28-block stack."""
from .ltx_transformer_block import LTXTransformerBlock
from .ltx_stack import LTXStack, LTXStackConfig, latent_grid, precompute_freqs_cis, random_init_

__all__ = ["LTXTransformerBlock", "LTXStack", "LTXStackConfig", "latent_grid", "precompute_freqs_cis", "random_init_"]

"""Drop-in for ``q8_kernels.functional`` (reference: q8_kernels/functional/__init__.py)."""
from . import fast_hadamard, flash_attention, fma, linear, quantizer, rms_norm, rope

__all__ = ["fast_hadamard", "flash_attention", "fma", "linear", "quantizer", "rms_norm", "rope"]

"""q8_kernels_b200 -- B200 (sm_100a) implementation of the q8_kernels 8-bit DiT
inference path, behind the reference's ``q8_kernels.functional`` /
``q8_kernels.modules`` / ``q8_kernels.blocks`` API.

Importing the package loads ``libq8k_b200.so`` (built by
``python q8_kernels_b200/build.py``) and fails if it is missing; there is no CPU
or eager fallback.
"""
from . import _lib, native  # noqa: F401  (loads the native library, fails loudly if absent)
from . import functional, modules, blocks, utils, graph  # noqa: F401
from ._lib import Q8KernelError, check_status, read_status  # noqa: F401  (the device status word, see _lib)

__version__ = "0.1.0"

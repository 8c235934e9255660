"""maryml_b200: B200 (sm_100a) kernels behind maryml's quantized-inference op surface.

The package is a thin host layer over libmary_b200.so (the C ABI of
include/mary_b200.h). Importing it loads the library; there is no fallback.
"""
from . import _lib
from ._lib import Context, MaryError, context
from .nvfp4 import Nvfp4, PromptLane, linear

__all__ = ["Context", "MaryError", "context", "Nvfp4", "PromptLane", "linear"]

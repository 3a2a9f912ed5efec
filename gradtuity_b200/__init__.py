"""gradtuity_b200: the B200-native GEMM path of the Gradtuity autograd engine.

Importing the package does not touch the GPU; the first tensor allocation or GEMM call loads
libgt_b200.so (see `_lib.load_library`) and creates the device context.  There is no CPU
fallback: without the library or without an sm_100 GPU those calls raise.
"""

from .tensor import Tensor, empty_tensor  # noqa: F401

__all__ = ["Tensor", "empty_tensor"]

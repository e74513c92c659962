"""B200-native (sm_100a) kernels for the e3nn message-passing hot path, behind e3nn's own API.

    from e3nn_b200 import o3
    tp = o3.FullyConnectedTensorProduct("32x0e+32x1o", "0e+1o", "32x0e+32x1o").cuda()

CUDA only: there is no CPU implementation and no fallback to PyTorch operators.
"""
from . import o3
from ._lib import E3BError, check_status, last_status_code
from .message_passing import conv_uvu, csr_from_dst

__version__ = "0.2.0"
__all__ = ["o3", "conv_uvu", "csr_from_dst", "check_status", "last_status_code", "E3BError"]

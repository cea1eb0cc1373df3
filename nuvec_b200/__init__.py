"""nuvec_b200: a B200 (sm_100a) backend for nuvec's quantized-matmul path.

The computation lives in ``libnuvec_cuda.so`` (hand-written CUDA behind the C ABI of
``include/nuvec_cuda.h``); this package is the host-side mirror of the reference's operator
interface.  Build the library with ``python -m nuvec_b200.build``.
"""
from .ops import *  # noqa: F401,F403
from .ops import BF16, F16, F32, I32, U8, U32  # noqa: F401

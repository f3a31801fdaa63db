"""B200 (sm_100a) decode kernels behind the ``crossdsl_kernels`` op signatures.

Four forward decode ops -- fused residual RMSNorm, the FP32 small-M projection,
fused RoPE + paged K/V append, and the W4A16 INT4 projection -- implemented as
hand-written CUDA in ``libxdk_b200.so`` (C ABI: include/xdk_b200.h) and reached
from Python through ctypes.  There is no CPU or alternative-backend path.
"""

__version__ = "0.1.0"

__all__ = ["__version__"]

"""B200-native replacement for mongoose's fused quantized decode path.

The product is ``libmongoose_kernels.so`` (CUDA, sm_100a, plain C ABI declared
in ``include/mongoose_kernels.h``).  This package only builds it
(``mongoose_b200.build``) and binds it with ctypes (``_lib``, ``kernels``,
``fused_infer``); it contains no arithmetic of its own and no fallback.
"""
from .configs import CONFIGS, FMT_F16, FMT_Q4_0, FMT_Q8_0, ModelConfig  # noqa: F401

"""B200-native fp32 GEMM and im2col convolution behind DECX's entry points.

The product is the C-ABI CUDA library ``libdecxb.so`` (``include/decxb.h``) and the C++
``de::`` layer over it (``include/decx/``).  This package is a thin Python binding used by
the test-suite and the benchmark: it loads the library, mirrors its entry points and passes
raw device/host pointers.  There is no CPU fallback: if the library is missing or no
sm_100 device is present, calls fail loudly.
"""
from .lib import (  # noqa: F401
    Comm,
    Context,
    DecxbError,
    GEMM_1XTF32,
    GEMM_3XTF32,
    GEMM_3XTF32_STRICT,
    GEMM_TF32_2XBF16,
    GEMM_DEFAULT,
    ACT_NONE,
    ACT_RELU,
    ACT_SIGMOID,
    ACT_TANH,
    CONV_EXPLICIT,
    CONV_IMPLICIT,
    CONV_NO_COMPENSATE,
    CONV_ZERO_COMPENSATE,
    TILE_AUTO,
    TILE_1CTA_128x128,
    TILE_2CTA_256x256,
    TILE_1CTA_128x256,
    TILE_1CTA_128x64,
    conv_geometry,
    library_path,
    load_library,
    shard_range,
)

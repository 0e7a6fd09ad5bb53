"""B200-native quantized GEMM operators (W8A8, W4A16, W4A8) behind the call signatures of the
tile-ai/tilelang-ascend examples ``quant_batch_matmul`` and ``dequantize_gemm``.

The kernels are hand-written CUDA for sm_100a in ``csrc/`` and are reached through the C ABI of
``libqgemm.so`` (``include/qgemm.h``).  There is no CPU or library fallback.
"""
from .ops import (  # noqa: F401
    act_quant,
    act_quant_kernel_int8_optimized,
    build_block_metadata,
    grouped_quant_gemm,
    grouped_quant_matmul,
    dequant_gemm_fp16_wrapper,
    dequant_gemm_int8_wrapper,
    quant_matmul,
    release_workspaces,
    simple_quant_batch_matmul,
    simple_quant_matmul,
    unpack_int4,
    w4a16_gemm,
    w4a8_gemm_cv,
    w4a8_gemm_act_quant,
)
from .quantize import (  # noqa: F401
    deinterleave_weight_int4_f16,
    gen_quant4,
    general_compress,
    interleave_weight,
    pack_int4,
    quantize_int4_groupwise,
    unpack_qzeros,
)
from ._lib import QGemmError  # noqa: F401

__version__ = "0.1.0"

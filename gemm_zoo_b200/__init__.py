"""gemm_zoo_b200 — B200-native dense GEMM (D = alpha*A*B + beta*C) behind the
call surface of AD2605/gemm-zoo's ``nvidia/kernel_functors``.

The product is the C ABI in ``include/gemmzoo/gemm.h`` (``libgemmzoo.so``) and
the C++ functor over it (``nvidia/kernel_functors/sm100_gemm.cuh``).  This
Python package is a thin ctypes binding used by the tests and by ``bench.py``;
torch is used only for device memory and streams.  There is no CPU or
library fallback: if the shared library is missing, importing ``lib()`` raises.
"""
from .api import (  # noqa: F401
    CFG_AUTO, CFG_1CTA_N256, CFG_1CTA_N128, CFG_1CTA_N64, CFG_2CTA_N256, CFG_2CTA_N128, CFG_SIMT,
    CFG_SWAP_M16, CFG_SWAP_M32, CFG_SWAP_M64, CFG_SWAP_M128, CFG_2CTA_M512_N256,
    COL_MAJOR, ROW_MAJOR, DT_BF16, DT_F16, DT_F32, DT_S8, DT_S32, DT_E4M3, DT_E5M2,
    FLAG_EPILOGUE_DIRECT, FLAG_EPILOGUE_TMA, FLAG_TEST_WITHHOLD_ACC_READY, FLAG_NO_SPLIT_K, FLAG_SPLIT_K, FLAG_BROADCAST_A, FLAG_BROADCAST_B,
    GemmDesc, GzError, Plan, PlanInfo, Sm100Gemm, fill, lib, lib_path, partition_columns,
    status_string, tile_coords, validate, EXPORTED_SYMBOLS, gemm_skinny_static, static_device_status, classify_dies, device_placement, FLAG_NO_DIE_ORDER, PROFILE_WORDS_PER_CTA,
    STATIC_SCRATCH_BYTES,
    ACT_NONE, ACT_RELU, ACT_GELU, ACT_GELU_TANH, ACT_SILU, Epilogue,
)

__all__ = [n for n in dir() if not n.startswith("_")]

from . import sm120_gated_gemm_nvfp4, sm120_mm_fp8_1d2d  # noqa: F401

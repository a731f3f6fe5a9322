from . import sm100_gemm_rs, sm100_mm_bf16, sm100_mm_mxfp8, sm100_mm_nvfp4  # noqa: F401

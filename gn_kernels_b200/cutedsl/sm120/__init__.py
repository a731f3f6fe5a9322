from . import sm120_mm_fp8_1d2d  # noqa: F401

"""gn_kernels_b200: hand-written sm_100a (B200) kernels behind the gn_kernels Python API.

Same public names as upstream `gn_kernels/__init__.py:1-23`; every function runs a CUDA
kernel from libgnk.so through a `gnk::` torch custom op.  There is no Triton, no CuteDSL,
no backend dispatch and no CPU fallback: CPU tensors or a missing library raise.
"""

from . import cutedsl
from .quant_utils import (
    absmax,
    dequantize_mx,
    dequantize_nvfp4,
    permute_nv_sf,
    quantize_mx,
    quantize_nvfp4,
    quantize_nvfp4_triton,
    quantize_rowwise,
    unpermute_nv_sf,
)
from .triton_attn import triton_attn, triton_varlen_attn
from .triton_mm import triton_mm

__all__ = [
    "absmax",
    "cutedsl",
    "dequantize_mx",
    "dequantize_nvfp4",
    "permute_nv_sf",
    "quantize_mx",
    "quantize_nvfp4",
    "quantize_nvfp4_triton",
    "quantize_rowwise",
    "triton_attn",
    "triton_mm",
    "triton_varlen_attn",
    "unpermute_nv_sf",
]

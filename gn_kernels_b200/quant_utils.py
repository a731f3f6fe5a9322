"""Quantizers and scale-factor layout helpers: the API of upstream gn_kernels/quant_utils.py
on CUDA kernels.  Byte-for-byte the values of the upstream torch reference functions.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import _lib, ops

_MX_KIND = {
    torch.float8_e4m3fn: _lib.Q_E4M3,
    torch.float8_e5m2: _lib.Q_E5M2,
    torch.float4_e2m1fn_x2: _lib.Q_E2M1,
}


def absmax(x: Tensor) -> Tensor:
    """max |x| as a 0-dim fp32 tensor (the reduction callers of quantize_nvfp4 run first,
    upstream tests/test_quant_utils.py:10)."""
    return ops.absmax(x)


def permute_nv_sf(scales: Tensor) -> Tensor:
    """[M, Ks] scales -> the 128x4-atom layout tcgen05 / cuBLAS read, zero-padded to
    multiples of (128, 4).  Upstream gn_kernels/quant_utils.py:21-30."""
    return ops.sf_swizzle(scales.view(torch.uint8), True).view(scales.dtype)


def unpermute_nv_sf(scales: Tensor) -> Tensor:
    """Inverse of permute_nv_sf on the padded shape.  Upstream gn_kernels/quant_utils.py:33-36."""
    M, Ks = scales.shape
    assert M % 128 == 0 and Ks % 4 == 0, (M, Ks)
    return ops.sf_swizzle(scales.view(torch.uint8), False).view(scales.dtype)


def quantize_mx(x: Tensor, dtype: torch.dtype, compute_scale_method: str = "ocp", *, swizzled_scales: bool = False):
    """MX quantizer, one E8M0 scale per 32 elements of the last dim.
    Upstream gn_kernels/quant_utils.py:93-117.  Returns (xq, scales float8_e8m0fnu [..., K/32]).
    `swizzled_scales=True` (extension) returns the scales already in permute_nv_sf layout."""
    assert dtype in _MX_KIND
    if compute_scale_method not in ("ocp", "nv"):
        raise ValueError(f"Unsupported {compute_scale_method=}")
    assert x.shape[-1] % 32 == 0
    rule = _lib.MX_OCP if compute_scale_method == "ocp" else _lib.MX_NV
    return ops.quant_mx(x, _MX_KIND[dtype], rule, swizzled_scales)


def dequantize_mx(xq: Tensor, scales: Tensor) -> Tensor:
    """fp32 values of an MX tensor (row-major scales).  Upstream gn_kernels/quant_utils.py:120-152;
    the FP4 branch inverts this package's packer (even element in the high nibble)."""
    assert scales.dtype == torch.float8_e8m0fnu
    return ops.dequant_block(xq, scales.view(torch.uint8), 32, None)


def quantize_nvfp4(x: Tensor, tensor_scale: Tensor | None = None, eps: float = 1e-12):
    """NVFP4 quantizer with row-major E4M3 scales [M, K/16].
    Upstream gn_kernels/quant_utils.py:156-171.  Returns (xq fp4x2 [M, K/2], scales, tensor_scale)."""
    assert x.ndim == 2 and x.shape[1] % 16 == 0
    if tensor_scale is None:
        tensor_scale = ops.absmax(x, 448.0 * 6.0)  # one kernel; torch's scalar division on CUDA is not IEEE
    elif not isinstance(tensor_scale, Tensor):
        tensor_scale = torch.tensor(float(tensor_scale), dtype=torch.float32, device=x.device)
    xq, sf = ops.quant_nvfp4(x, tensor_scale, eps, False)
    return xq, sf, tensor_scale


def quantize_nvfp4_triton(x: Tensor, tensor_scale: Tensor, eps: float = 1e-12):
    """Same quantizer, scales written directly as 128x4 atoms with rows padded to 128.
    Upstream gn_kernels/quant_utils.py:242-252 (name kept; the kernel is CUDA, and unlike
    upstream it divides exactly, so it equals quantize_nvfp4 on every input)."""
    M, N = x.shape
    assert N % 64 == 0
    if not isinstance(tensor_scale, Tensor):
        tensor_scale = torch.tensor(float(tensor_scale), dtype=torch.float32, device=x.device)
    return ops.quant_nvfp4(x, tensor_scale, eps, True)


def dequantize_nvfp4(xq: Tensor, scales: Tensor, tensor_scale: Tensor | None = None) -> Tensor:
    """fp32 values of an NVFP4 tensor with row-major scales (extension; upstream has no such helper)."""
    return ops.dequant_block(xq, scales.view(torch.uint8), 16, tensor_scale)


def quantize_rowwise(x: Tensor, dtype: torch.dtype, *, transpose_scales: bool = False):
    """Row-wise absmax quantizer over the last dim (upstream benchmark_attn.py:39-51).
    Returns (xq, scale fp32 x.shape[:-1]).  For a [B, L, H, D] input, transpose_scales=True
    returns the scale as contiguous [B, H, L] (what triton_attn takes, benchmark_attn.py:77-80)."""
    assert dtype in (torch.int8, torch.float8_e4m3fn)
    qkind = _lib.Q_INT8 if dtype == torch.int8 else _lib.Q_E4M3
    if transpose_scales:
        B, L, H, _ = x.shape
        q, s = ops.quant_rowwise(x, qkind, H, L)
        return q, s.view(B, H, L)
    q, s = ops.quant_rowwise(x, qkind, 0, 0)
    return q, s.view(x.shape[:-1])

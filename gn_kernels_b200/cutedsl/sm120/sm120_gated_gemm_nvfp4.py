"""SwiGLU-gated dual NVFP4 GEMM with an optional re-quantising epilogue.
Upstream gn_kernels/cutedsl/sm120/sm120_gated_gemm_nvfp4.py:513-555 (an sm_120 mma.sync kernel); the
module path and call are kept, the kernel underneath is the tcgen05 block-scaled GEMM for sm_100a
with both weight matrices in one 2-CTA tile."""

import torch

from ... import ops


def mm(
    X: torch.Tensor,
    SFX: torch.Tensor,
    SFX_tensor: torch.Tensor,
    W1: torch.Tensor,
    SFW1: torch.Tensor,
    SFW1_tensor: torch.Tensor,
    W3: torch.Tensor,
    SFW3: torch.Tensor,
    SFW3_tensor: torch.Tensor,
    SFC_tensor: torch.Tensor | None = None,
):
    """out = silu(X W1^T) * (X W3^T) with NVFP4 operands: X [M, K/2], W1 / W3 [N, K/2]
    float4_e2m1fn_x2, SF* float8_e4m3fn block scales in permute_nv_sf layout, SF*_tensor the fp32
    per-tensor scales (device tensors; each product is multiplied by the two tensor scales before the
    gate).  Without SFC_tensor: returns bf16 [M, N].  With SFC_tensor (the per-tensor scale of the
    output): returns (C float4_e2m1fn_x2 [M, N/2], SFC float8_e4m3fn [ceil128(M), N/16] in
    permute_nv_sf layout), equal to quantize_nvfp4_triton(bf16 output, SFC_tensor)."""
    M, _ = X.shape
    N, _ = W1.shape
    assert W3.shape == W1.shape and X.shape[1] == W1.shape[1]
    u8 = lambda t: t.view(torch.uint8)  # noqa: E731
    f32 = lambda t: t.to(torch.float32).reshape(1)  # noqa: E731
    args = (u8(X), u8(SFX), f32(SFX_tensor), u8(W1), u8(SFW1), f32(SFW1_tensor), u8(W3), u8(SFW3), f32(SFW3_tensor))
    if SFC_tensor is None:
        return ops.gated_mm_nvfp4(*args)
    C, SFC = ops.gated_mm_nvfp4_quant(*args, f32(SFC_tensor))
    return C.view(torch.float4_e2m1fn_x2), SFC.view(torch.float8_e4m3fn)

"""NVFP4 GEMM.  Upstream gn_kernels/cutedsl/sm100/sm100_mm_nvfp4.py:383-386."""

import torch

from ... import ops


def mm(A: torch.Tensor, B: torch.Tensor, SFA: torch.Tensor, SFB: torch.Tensor, alpha=1.0) -> torch.Tensor:
    """C[M,N] bf16 = alpha * dequant(A[M,K/2], SFA) @ dequant(B[N,K/2], SFB)^T.  A, B
    float4_e2m1fn_x2; SFA, SFB float8_e4m3fn in permute_nv_sf layout.  alpha (extension,
    default 1 = upstream behaviour) is tensor_scale_A * tensor_scale_B, applied to the fp32
    accumulator as upstream's gated kernel does (sm120_gated_gemm_nvfp4.py:317-319)."""
    if isinstance(alpha, torch.Tensor):
        alpha = float(alpha)
    return ops.mm_nvfp4(A.view(torch.uint8), B.view(torch.uint8), SFA.view(torch.uint8), SFB.view(torch.uint8), alpha)

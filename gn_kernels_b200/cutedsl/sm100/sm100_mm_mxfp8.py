"""MXFP8 GEMM.  Upstream gn_kernels/cutedsl/sm100/sm100_mm_mxfp8.py:380-383."""

import torch

from ... import ops


def mm(A: torch.Tensor, B: torch.Tensor, SFA: torch.Tensor, SFB: torch.Tensor) -> torch.Tensor:
    """C[M,N] bf16 = dequant(A[M,K], SFA) @ dequant(B[N,K], SFB)^T.  A, B float8_e4m3fn, K
    contiguous; SFA, SFB float8_e8m0fnu in permute_nv_sf layout."""
    return ops.mm_mxfp8(A, B, SFA.view(torch.uint8), SFB.view(torch.uint8))

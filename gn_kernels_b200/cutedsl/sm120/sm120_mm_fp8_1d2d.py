"""FP8 GEMM with 1x128 (A) and 128x128 (B) fp32 block scales, DeepSeek-V3 style.
Upstream gn_kernels/cutedsl/sm120/sm120_mm_fp8_1d2d.py:307-333 (an sm_120 mma.sync kernel); the
module path and call are kept, the kernel underneath is a tcgen05 kernel for sm_100a."""

import torch

from ... import ops


def mm(
    A: torch.Tensor,
    SFA: torch.Tensor,
    B: torch.Tensor,
    SFB: torch.Tensor,
    bias: torch.Tensor | None = None,
    add: torch.Tensor | None = None,
) -> torch.Tensor:
    """C[M,N] bf16 = sum_kb (A[:, kb] @ B[:, kb]^T) * SFA[:, kb] * SFB[n // 128, kb] (+ add) (+ bias).

    A [M,K], B [N,K] float8_e4m3fn with K contiguous; SFA fp32 [M, K/128] stored M-major
    (stride (1, >= M)), SFB [N/128, K/128]; bias bf16 [N]; add bf16 [M,N]."""
    return ops.mm_f8_block128(A, SFA, B, SFB, bias, add)

"""BF16 GEMM.  Upstream gn_kernels/cutedsl/sm100/sm100_mm_bf16.py:252-255."""

import torch

from ... import ops


def mm(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """C[M,N] bf16 = A[M,K] @ B[K,N]; B is the transposed view of an [N,K] row-major buffer."""
    return ops.mm_bf16(A, B.T)

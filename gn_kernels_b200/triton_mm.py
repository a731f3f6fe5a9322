"""`triton_mm`: the row-scaled INT8 / FP8 (and plain BF16) matmul entry point of upstream
gn_kernels/triton_mm.py:128-171, on tcgen05 kernels.  The name is kept so callers need no edit."""

from __future__ import annotations

import torch
from torch import Tensor

from . import ops


def triton_mm(
    A: Tensor,
    B: Tensor,
    bias: Tensor | None = None,
    *,
    scale_A: Tensor | None = None,
    scale_B: Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    acc_dtype: torch.dtype | None = None,
):
    """C[M,N] = A[M,K] @ B[K,N] with the fused epilogue acc*scale_A[m] -> *scale_B[n] -> +bias[n].

    int8 inputs accumulate exactly in int32 (int32 output when unscaled, else bf16); e4m3 and
    bf16 inputs accumulate in fp32 (bf16 output); fp16 inputs give fp16 output, accumulated in
    fp32 or, with acc_dtype=torch.float16, in the tensor core's fp16 accumulator.  B is normally the transposed view of an
    [N, K] row-major buffer; other layouts are copied into that form first."""
    assert A.shape[1] == B.shape[0]
    M, K = A.shape
    _, N = B.shape
    if scale_A is not None:
        assert scale_A.shape == (M, 1) and scale_A.is_contiguous()
    if scale_B is not None:
        assert scale_B.shape == (1, N) and scale_B.is_contiguous()
    if bias is not None:
        assert bias.shape == (N,) and bias.is_contiguous()
    if acc_dtype not in (None, torch.float32, torch.int32, torch.float16):
        raise NotImplementedError(f"acc_dtype {acc_dtype}")
    if acc_dtype == torch.float16 and A.dtype != torch.float16:
        # the tensor core's F16 accumulator belongs to kind::f16; for fp16 operands it is upstream's
        # `acc_dtype=torch.float16` (triton_mm.py:164-165)
        raise NotImplementedError("acc_dtype=float16 needs float16 A and B")

    scaled = scale_A is not None or scale_B is not None
    if out_dtype is None:  # upstream rule, triton_mm.py:155-161
        if A.dtype in (torch.float32, torch.float16, torch.bfloat16):
            out_dtype = A.dtype
        elif A.is_floating_point() or scaled:
            out_dtype = torch.bfloat16
        else:
            out_dtype = torch.int32

    Bt = B.T  # [N, K]
    if A.dtype == torch.int8:
        if out_dtype == torch.int32:
            if scaled or bias is not None:
                raise NotImplementedError("int32 output with scales or bias")
            return ops.mm_i8(A, Bt, None, None, None, True)
        assert out_dtype == torch.bfloat16
        return ops.mm_i8(A, Bt, scale_A, scale_B, bias, False)
    if A.dtype == torch.float8_e4m3fn:
        assert out_dtype == torch.bfloat16
        return ops.mm_f8(A, Bt, scale_A, scale_B, bias)
    if A.dtype == torch.bfloat16 and not scaled and bias is None and out_dtype == torch.bfloat16:
        return ops.mm_bf16(A, Bt)
    if A.dtype == torch.float16 and B.dtype == torch.float16 and not scaled and bias is None and out_dtype == torch.float16:
        return ops.mm_f16(A, Bt, acc_dtype == torch.float16)
    raise NotImplementedError(f"triton_mm: no sm_100a kernel for {A.dtype} inputs with this epilogue")

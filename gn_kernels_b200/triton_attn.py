"""`triton_attn` and `triton_varlen_attn`: GQA attention forward (upstream gn_kernels/triton_attn.py:268-325
and :462-517) on one tcgen05 kernel family.  The names are kept so callers need no edit."""

from __future__ import annotations

import torch
from torch import Tensor

from . import ops


def _acc16(q: Tensor, v: Tensor, qk_fp16_acc: bool, pv_fp16_acc: bool) -> int:
    """fp16 accumulation is a property of the tensor-core instruction (kind::f16 with an F16
    accumulator): it exists for fp16 operands, which is also the only case where upstream's option
    (triton_attn.py:311-312) leaves the operand precision."""
    if qk_fp16_acc and q.dtype != torch.float16:
        raise NotImplementedError("qk_fp16_acc needs float16 q and k")
    if pv_fp16_acc and v.dtype != torch.float16:
        raise NotImplementedError("pv_fp16_acc needs float16 v")
    return int(bool(qk_fp16_acc)) | (int(bool(pv_fp16_acc)) << 1)


def triton_attn(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    scale_q: Tensor | None = None,
    scale_k: Tensor | None = None,
    *,
    causal: bool = False,
    qk_fp16_acc: bool = False,
    pv_fp16_acc: bool = False,
):
    """O[B,Lq,Hq,D] = softmax((Q K^T) * scale_q * scale_k * D^-1/2 [causal, lower-right aligned]) V.

    q, k [B, L, H, D] (D = 128, last dim contiguous): int8 or float8_e4m3fn codes, with scale_q
    [B, Hq, Lq] and scale_k [B, Hkv, Lk] fp32 (both or neither), or bf16 / fp16 without scales.
    v: bf16 or fp16 (for 16-bit q, k: the same type); the output has v's type.  QK accumulates
    exactly (int32) or in fp32 (fp16 with qk_fp16_acc), softmax runs in fp32 with exp2, P is
    rounded to v's type before P @ V (fp32 accumulate, fp16 with pv_fp16_acc)."""
    BS, Q_LEN, Q_HEADS, QK_DIM = q.shape
    _, KV_LEN, KV_HEADS, V_DIM = v.shape
    assert Q_HEADS % KV_HEADS == 0
    assert k.shape == (BS, KV_LEN, KV_HEADS, QK_DIM)
    assert v.shape == (BS, KV_LEN, KV_HEADS, V_DIM)
    assert q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    if QK_DIM != 128 or V_DIM != 128:
        raise NotImplementedError("the sm_100a attention kernel is built for head dimension 128")
    if (scale_q is None) != (scale_k is None):
        raise ValueError("scale_q and scale_k must be given together")
    if scale_q is not None:
        if q.dtype in (torch.bfloat16, torch.float16):
            raise NotImplementedError("scale_q / scale_k go with int8 or float8_e4m3fn q and k")
        assert scale_q.shape == (BS, Q_HEADS, Q_LEN) and scale_q.is_contiguous()
        assert scale_k.shape == (BS, KV_HEADS, KV_LEN) and scale_k.is_contiguous()
    return ops.attn_fwd(q, k, v, scale_q, scale_k, causal, _acc16(q, v, qk_fp16_acc, pv_fp16_acc))


def triton_varlen_attn(
    q: Tensor,
    k: Tensor,
    v: Tensor,
    q_offsets: Tensor,
    kv_offsets: Tensor,
    max_q_len: int,
    *,
    causal: bool = False,
    qk_fp16_acc: bool = False,
    pv_fp16_acc: bool = False,
):
    """Attention over packed sequences: q [Lq_total, Hq, D], k / v [Lkv_total, Hkv, D] (bf16 or fp16,
    D = 128), sequence b = rows [offsets[b], offsets[b+1]) of each tensor; `max_q_len` bounds the
    longest query sequence.  The causal mask is lower-right aligned per sequence."""
    Q_LEN_TOTAL, Q_HEADS, QK_DIM = q.shape
    KV_LEN_TOTAL, KV_HEADS, V_DIM = v.shape
    BS = q_offsets.shape[0] - 1
    assert Q_HEADS % KV_HEADS == 0
    assert k.shape == (KV_LEN_TOTAL, KV_HEADS, QK_DIM)
    assert kv_offsets.shape[0] == BS + 1
    assert q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    assert q_offsets.is_contiguous() and kv_offsets.is_contiguous()
    if QK_DIM != 128 or V_DIM != 128:
        raise NotImplementedError("the sm_100a attention kernel is built for head dimension 128")
    return ops.attn_varlen_fwd(q, k, v, q_offsets, kv_offsets, int(max_q_len), causal, _acc16(q, v, qk_fp16_acc, pv_fp16_acc))

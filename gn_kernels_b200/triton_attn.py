"""`triton_attn`: GQA attention forward with INT8 / FP8 QK (upstream gn_kernels/triton_attn.py:268-325)
on a tcgen05 kernel.  The name is kept so callers need no edit."""

from __future__ import annotations

from torch import Tensor

from . import ops


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

    q, k: int8 or float8_e4m3fn [B, L, H, D] (D = 128, last dim contiguous); v: bf16; scale_q
    [B, Hq, Lq] and scale_k [B, Hkv, Lk] fp32, both or neither.  QK accumulates exactly (int32) or
    in fp32, softmax runs in fp32 with exp2, P is rounded to bf16 before P @ V (fp32 accumulate)."""
    BS, Q_LEN, Q_HEADS, QK_DIM = q.shape
    _, KV_LEN, KV_HEADS, V_DIM = v.shape
    assert Q_HEADS % KV_HEADS == 0
    assert k.shape == (BS, KV_LEN, KV_HEADS, QK_DIM)
    assert q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
    if qk_fp16_acc or pv_fp16_acc:
        raise NotImplementedError("fp16 accumulation has no tcgen05 kernel in this package")
    if QK_DIM != 128 or V_DIM != 128:
        raise NotImplementedError("the sm_100a attention kernel is built for head dimension 128")
    if (scale_q is None) != (scale_k is None):
        raise ValueError("scale_q and scale_k must be given together")
    if scale_q is not None:
        assert scale_q.shape == (BS, Q_HEADS, Q_LEN) and scale_q.is_contiguous()
        assert scale_k.shape == (BS, KV_HEADS, KV_LEN) and scale_k.is_contiguous()
    return ops.attn_fwd(q, k, v, scale_q, scale_k, causal)

"""`triton_attn`: GQA attention forward with INT8 / FP8 QK (upstream gn_kernels/triton_attn.py:268-325)."""

from __future__ import annotations

from torch import Tensor


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
    from . import ops

    if not hasattr(ops, "attn_fwd"):
        raise NotImplementedError("the sm_100a attention kernel is not built into this library yet")
    return ops.attn_fwd(q, k, v, scale_q, scale_k, causal)

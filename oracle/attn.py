"""Attention oracle (CPU torch, fp32).  Test infrastructure only, never imported by the package.

Restates the arithmetic of upstream `triton_attn` (gn_kernels/triton_attn.py:82-241, inner
loop :9-76) as "dequantise Q and K, exact softmax in fp32, P @ V":

    S[i, j] = (q_i . k_j) * scale_q[i] * scale_k[j] * D**-0.5
    visible(i, j) = (not causal) or (j <= i + (KV_LEN - Q_LEN))          (:165-181, :212)
    O[i] = softmax_j(S[i, visible]) @ V            rows that see nothing -> 0   (:236-237)

GQA: kv head = q_head // (Q_HEADS // KV_HEADS) (:112).  Layout [B, L, H, D] (:281-286).
This is the same comparison the upstream benchmark makes (benchmark_attn.py:94-97,130-138:
sdpa(dequant(Q), dequant(K), V.float()).bfloat16()) with the mask of
tests/test_triton_attn.py:11-22 (causal_lower_right).  The query axis is processed in
chunks so no [Lq, Lkv] score tensor for more than one (batch, head) is alive at a time.
"""

from __future__ import annotations

import numpy as np
import torch

from . import quant


def _f32(x) -> torch.Tensor:
    if isinstance(x, np.ndarray):
        return torch.from_numpy(np.ascontiguousarray(x)).float()
    return x.detach().cpu().float()


def attention_f32(q, k, v, *, causal: bool, sm_scale: float | None = None, q_chunk: int = 1024) -> torch.Tensor:
    """q [B,Lq,Hq,D], k [B,Lk,Hkv,D], v [B,Lk,Hkv,Dv], any float dtype -> fp32 [B,Lq,Hq,Dv]."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, Lq, Hq, D = q.shape
    _, Lk, Hkv, Dv = v.shape
    group = Hq // Hkv
    sm_scale = D**-0.5 if sm_scale is None else sm_scale
    out = torch.zeros(B, Lq, Hq, Dv)
    jj = torch.arange(Lk)
    for b in range(B):
        for h in range(Hq):
            kh = k[b, :, h // group, :]  # [Lk, D]
            vh = v[b, :, h // group, :]
            for i0 in range(0, Lq, q_chunk):
                i1 = min(Lq, i0 + q_chunk)
                s = (q[b, i0:i1, h, :] @ kh.T) * sm_scale
                if causal:
                    ii = torch.arange(i0, i1).unsqueeze(1)
                    vis = jj.unsqueeze(0) <= ii + (Lk - Lq)
                    s = s.masked_fill(~vis, float("-inf"))
                    dead = ~vis.any(dim=1)
                else:
                    dead = torch.zeros(i1 - i0, dtype=torch.bool)
                m = s.max(dim=1, keepdim=True).values
                m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
                p = torch.exp(s - m)
                o = (p @ vh) / p.sum(dim=1, keepdim=True).clamp_min(1e-38)
                o[dead] = 0.0
                out[b, i0:i1, h, :] = o
    return out


def attention_qk_quantized(q_codes, k_codes, v, scale_q, scale_k, *, kind: str, causal: bool) -> torch.Tensor:
    """q_codes/k_codes: int8 values or uint8 E4M3 encodings in [B,L,H,D]; scale_q [B,Hq,Lq],
    scale_k [B,Hkv,Lk] fp32 (the transposed layout triton_attn takes, :316-319).
    Returns bf16 [B,Lq,Hq,Dv] (output takes V's dtype, :291)."""
    sq = _f32(scale_q).permute(0, 2, 1)  # -> [B, L, H]
    sk = _f32(scale_k).permute(0, 2, 1)
    qf = torch.from_numpy(quant.dequantize_rowwise(np.asarray(q_codes), sq.numpy(), kind))
    kf = torch.from_numpy(quant.dequantize_rowwise(np.asarray(k_codes), sk.numpy(), kind))
    return attention_f32(qf, kf, v, causal=causal).bfloat16()

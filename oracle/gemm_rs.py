"""GEMM + reduce-scatter oracle (CPU torch).  Test infrastructure only.

Upstream: gn_kernels/cutedsl/sm100/sm100_gemm_rs.py:458-496 (entry), :393-397 (partials are
rounded to bf16 before the reduction), :27-60 (the reduction adds in fp32), :194,305,404
(rank r owns rows [r*M/W, (r+1)*M/W)).

    output_r[M/W, N] = bf16( sum_ranks f32( bf16( x_s @ w_s^T ) )[rows of r] )
"""

from __future__ import annotations

import torch


def gemm_rs(xs, ws, *, round_partials: bool = True):
    """xs[s]: [M, K/W], ws[s]: [N, K/W] for every rank s.  Returns the list of per-rank
    outputs [M/W, N] (bf16).  round_partials=False gives the unrounded fp32 sum, the
    tighter target a fused kernel may also be compared with."""
    W = len(xs)
    M = xs[0].shape[0]
    total = None
    for x, w in zip(xs, ws):
        p = x.detach().cpu().float() @ w.detach().cpu().float().T
        if round_partials:
            p = p.bfloat16().float()
        total = p if total is None else total + p
    rows = M // W
    return [total[r * rows : (r + 1) * rows].bfloat16() for r in range(W)]


def gemm_ar(xs, ws, *, round_partials: bool = True):
    """The all-reduce form of the same sum (no upstream function): every rank ends with all M rows,
    i.e. the reduce-scatter outputs of all ranks stacked.  Returns one [M, N] bf16 tensor."""
    return torch.cat(gemm_rs(xs, ws, round_partials=round_partials), dim=0)


def gemm_rs_f8(xs, ws, alphas):
    """E4M3 operands with one dequantisation factor per rank (no upstream function; the statement of
    gn_kernels_b200's gnk_gemm_rs_f8): xs[s] [M, K/W], ws[s] [N, K/W] float8_e4m3fn (or their exact
    fp32 values), alphas[s] = scale_x * scale_w of rank s.
        output_r = bf16( sum_ranks f32( bf16( alpha_s * (f32(x_s) @ f32(w_s)^T) ) )[rows of r] )"""
    W = len(xs)
    M = xs[0].shape[0]
    total = None
    for x, w, a in zip(xs, ws, alphas):
        p = (x.detach().cpu().float() @ w.detach().cpu().float().T) * float(a)
        p = p.bfloat16().float()
        total = p if total is None else total + p
    rows = M // W
    return [total[r * rows : (r + 1) * rows].bfloat16() for r in range(W)]

"""Helpers shared by the GPU parity tests: seeded inputs, bit views, oracle adapters."""

from __future__ import annotations

import numpy as np
import torch

from oracle import quant as oq

SEED_MM = 2025 * 2024 + 2027  # upstream benchmark_mm.py:36
SEED_ATTN = 2025 * 2026  # upstream benchmark_attn.py:66


def u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.uint8).cpu().numpy()


def f32np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def randn_bf16(shape, seed, device="cuda", scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).bfloat16().to(device)


def wide_range_bf16(M, K, seed, device="cuda"):
    """Per-16-block magnitudes spread over 2^-12 .. 2^5 plus the usual edge rows."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    x = x * torch.exp2(torch.randint(-12, 6, (M, K // 16, 1), generator=g).float()).expand(M, K // 16, 16).reshape(M, K)
    if M >= 6 and K >= 32:
        x[0, :32] = 0.0
        x[1, :32] = 1e-30
        x[2, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
        x[3, :32] = 449.0
        x[4, :32] = torch.linspace(-500, 500, 32)
        x[5, :32] = -0.0
    return x.bfloat16().to(device)


def swizzle_np(s: np.ndarray) -> np.ndarray:
    return oq.permute_nv_sf(s)


def rel_err(out: torch.Tensor, ref: torch.Tensor) -> float:
    out = out.detach().double().cpu()
    ref = ref.detach().double().cpu()
    return float((out - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


def assert_parity(out: torch.Tensor, ref: torch.Tensor, tol: float = 1e-2, atol_frac: float = 1e-3, elem_rtol: float | None = None,
                  atol_abs: float | None = None) -> None:
    """The two readings of "max relative error <= 1e-2" for floating-point outputs, both asserted:
    global   max|out - ref| <= tol * max|ref|
    element  |out - ref| <= elem_rtol * |ref| + atol   for every element, atol = atol_frac * max|ref|
             (or the fixed atol_abs), elem_rtol = tol unless given
    The absolute term covers elements near zero, where one bf16 rounding of a cancelling sum is large
    relative to the element itself; upstream's own checks use rtol 1e-2 (GEMM, benchmark_mm.py:81-95)
    or 1.6e-2 (attention, tests/test_triton_attn.py:41) with a fixed atol."""
    o = out.detach().double().cpu()
    r = ref.detach().double().cpu()
    scale = float(r.abs().max().clamp_min(1e-30))
    diff = (o - r).abs()
    worst = float(diff.max())
    assert worst <= tol * scale, f"global relative error {worst / scale:.3e} > {tol}"
    rt = tol if elem_rtol is None else elem_rtol
    at = atol_frac * scale if atol_abs is None else atol_abs
    excess = diff - (rt * r.abs() + at)
    bad = int((excess > 0).sum())
    assert bad == 0, f"{bad} elements outside |out-ref| <= {rt}*|ref| + {at:.2e} (worst excess {float(excess.max()):.3e}, max|ref| {scale:.3e})"

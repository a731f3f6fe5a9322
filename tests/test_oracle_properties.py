"""Size-independent properties of the oracle (CPU only): round trips, idempotence, linearity,
bijections.  The same properties are what the full-size GPU cases lean on where an element-wise
comparison with the oracle would take too long."""

import numpy as np
import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from oracle import gemm_rs as ors
from oracle import mm as omm
from oracle import quant as oq


def _rand(shape, seed, spread=4.0):
    g = np.random.default_rng(seed)
    x = g.standard_normal(shape).astype(np.float32) * np.exp2(g.integers(-int(spread), int(spread) + 1, size=shape)).astype(np.float32)
    return torch.from_numpy(x).bfloat16().float().numpy()  # bf16-representable, like the kernels' inputs


@settings(max_examples=25, deadline=None)
@given(st.integers(1, 300), st.integers(1, 40))
def test_scale_factor_swizzle_is_a_bijection_onto_the_padded_buffer(M, Ks):
    Mp, Kp = (M + 127) // 128 * 128, (Ks + 3) // 4 * 4
    offs = {oq.sf_swizzled_offset(r, c, Kp) for r in range(0, Mp, max(1, Mp // 64)) for c in range(Kp)}
    rows = len(range(0, Mp, max(1, Mp // 64)))
    assert len(offs) == rows * Kp and min(offs) >= 0 and max(offs) < Mp * Kp


@pytest.mark.parametrize("M,Ks", [(128, 4), (200, 6), (1, 1), (129, 5), (384, 64)])
def test_permute_then_unpermute_is_identity_on_the_valid_region(M, Ks):
    g = np.random.default_rng(M * 131 + Ks)
    s = g.integers(0, 256, size=(M, Ks), dtype=np.uint8)
    Mp, Kp = (M + 127) // 128 * 128, (Ks + 3) // 4 * 4
    padded = np.zeros((Mp, Kp), dtype=np.uint8)
    padded[:M, :Ks] = s
    back = oq.unpermute_nv_sf(oq.permute_nv_sf(padded))
    assert np.array_equal(np.asarray(back).reshape(Mp, Kp)[:M, :Ks], s)
    # element (r, c) sits where the offset function says
    flat = np.asarray(oq.permute_nv_sf(padded)).reshape(-1)
    for r, c in [(0, 0), (M - 1, Ks - 1), (M // 2, Ks // 2)]:
        assert flat[oq.sf_swizzled_offset(r, c, Kp)] == s[r, c]


@pytest.mark.parametrize("kind,method", [("e4m3", "ocp"), ("e4m3", "nv"), ("e5m2", "ocp"), ("e2m1", "ocp"), ("e2m1", "nv")])
def test_quantize_mx_is_idempotent_on_its_own_output(kind, method):
    x = _rand((16, 128), 7)
    q, s = oq.quantize_mx(x, kind, method)
    deq = oq.dequantize_mx(q, s, kind)
    q2, s2 = oq.quantize_mx(deq, kind, method)
    deq2 = oq.dequantize_mx(q2, s2, kind)
    # quantising a tensor that is already on the grid may pick a smaller shared exponent, never other values
    assert np.array_equal(deq2, deq)


def test_nvfp4_round_trip_error_is_bounded_by_the_block_scale():
    x = _rand((32, 256), 11, spread=2.0)
    packed, sf, ts = oq.quantize_nvfp4(x)
    deq = oq.dequantize_nvfp4(packed, sf, ts)
    scale = oq.e4m3_to_f32(sf).astype(np.float32) * np.float32(ts)       # one per 16 elements
    step = np.repeat(scale, 16, axis=1)                                   # e2m1 grid spacing is at most 2 * scale
    assert np.all(np.abs(deq - x) <= step * 1.0 + 1e-30)                  # half of the widest spacing (2) times the scale
    # idempotence on the grid
    packed2, sf2, _ = oq.quantize_nvfp4(deq, ts)
    assert np.array_equal(oq.dequantize_nvfp4(packed2, sf2, ts), deq)


def test_pack_unpack_e2m1_round_trip_and_nibble_order():
    codes = np.arange(16, dtype=np.uint8).repeat(2)[None, :]
    packed = oq.pack_e2m1_pairs(codes)
    table = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)
    vals = oq.unpack_e2m1_pairs(packed)  # decoded values, element order restored
    assert np.array_equal(vals, table[codes]) and np.array_equal(np.signbit(vals), np.signbit(table[codes]))
    two = oq.pack_e2m1_pairs(np.array([[0x3, 0xA]], dtype=np.uint8))
    assert two[0, 0] == 0x3A  # even element in the HIGH nibble


@settings(max_examples=20, deadline=None)
@given(st.integers(1, 40), st.integers(1, 24), st.integers(1, 96), st.integers(0, 2**31 - 1))
def test_int8_mm_is_exact_and_linear(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    A = torch.randint(-128, 128, (M, K), dtype=torch.int8, generator=g)
    A2 = torch.randint(-64, 64, (M, K), dtype=torch.int8, generator=g)
    Bt = torch.randint(-128, 128, (N, K), dtype=torch.int8, generator=g)
    ref = (A.to(torch.int64) @ Bt.to(torch.int64).T).to(torch.int32)
    assert torch.equal(omm.int8_mm_exact(A, Bt), ref)
    # linearity in A (kept in int16 range so the sum is still int8-free arithmetic in the check)
    lhs = (A.to(torch.int64) + A2.to(torch.int64)) @ Bt.to(torch.int64).T
    rhs = omm.int8_mm_exact(A, Bt).to(torch.int64) + omm.int8_mm_exact(A2, Bt).to(torch.int64)
    assert torch.equal(lhs, rhs)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_gemm_rs_is_the_row_slice_of_the_summed_bf16_partials(world):
    M, N, Kl = 64 * world, 48, 40
    g = torch.Generator().manual_seed(world)
    xs = [(torch.randn(M, Kl, generator=g) / 8).bfloat16() for _ in range(world)]
    ws = [(torch.randn(N, Kl, generator=g) / 8).bfloat16() for _ in range(world)]
    outs = ors.gemm_rs(xs, ws)
    partials = [(x.float() @ w.float().T).bfloat16().float() for x, w in zip(xs, ws)]
    full = sum(partials[1:], partials[0]).bfloat16()
    rows = M // world
    assert len(outs) == world
    for r, o in enumerate(outs):
        assert o.shape == (rows, N) and torch.equal(o, full[r * rows : (r + 1) * rows])
    # with one rank the op is the plain bf16 GEMM
    if world == 1:
        assert torch.equal(outs[0], omm.mm_bf16(xs[0], ws[0]))


def test_mxfp8_mm_equals_dequantise_then_matmul():
    A, Bt = _rand((24, 96), 3, 2.0), _rand((40, 96), 4, 2.0)
    Aq, sa = oq.quantize_mx(A, "e4m3")
    Bq, sb = oq.quantize_mx(Bt, "e4m3")
    ref = (torch.from_numpy(oq.dequantize_mx(Aq, sa, "e4m3")) @ torch.from_numpy(oq.dequantize_mx(Bq, sb, "e4m3")).T).bfloat16()
    assert torch.equal(omm.mm_mxfp8(Aq, Bq, sa, sb), ref)

"""GPU parity: quantizer kernels vs the CPU oracle (bit-exact bytes and scales), through the
public Python API (torch custom ops -> C ABI)."""

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits
from gpu_util import f32np, randn_bf16, u8, wide_range_bf16
from oracle import quant as oq

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gk():
    import gn_kernels_b200 as g

    return g


def test_library_loaded_and_arch(gk):
    from gn_kernels_b200 import _lib

    assert _lib.lib().gnk_version() == 100
    assert torch.cuda.get_device_capability()[0] == 10


@pytest.mark.parametrize("n", [1, 7, 8, 1000, 4096 * 33 + 5, 8192 * 8192])
def test_absmax(gk, n):
    g = torch.Generator().manual_seed(n)
    x = torch.randn(n, generator=g).bfloat16().cuda()
    got = gk.absmax(x)
    assert float(got) == float(x.float().abs().max())
    # the scratch ticket is restored: a second call gives the same answer
    assert float(gk.absmax(x)) == float(got)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_absmax_dtypes(gk, dtype):
    x = torch.randn(3, 1000, generator=torch.Generator().manual_seed(3)).to(dtype).cuda()
    assert float(gk.absmax(x)) == float(x.float().abs().max())


@pytest.mark.parametrize("name", ["a", "b"])
def test_nvfp4_golden(gk, golden_quant, name):
    g = golden_quant
    x = bf16_from_bits(g[f"nvfp4_{name}_x"]).cuda()
    ts = torch.tensor(float(g[f"nvfp4_{name}_ts"]), device="cuda")
    q, sf, _ = gk.quantize_nvfp4(x, ts)
    np.testing.assert_array_equal(u8(sf), g[f"nvfp4_{name}_sf"])
    np.testing.assert_array_equal(u8(q), g[f"nvfp4_{name}_q"])
    q2, sf2, ts2 = gk.quantize_nvfp4(x)
    assert float(ts2) == float(g[f"nvfp4_{name}_auto_ts"])
    np.testing.assert_array_equal(u8(sf2), g[f"nvfp4_{name}_auto_sf"])
    np.testing.assert_array_equal(u8(q2), g[f"nvfp4_{name}_auto_q"])


@pytest.mark.parametrize("M,N", [(256, 128), (196, 256)])  # the upstream test's shapes (tests/test_quant_utils.py:7)
def test_nvfp4_swizzled_equals_rowmajor(gk, M, N):
    x = randn_bf16((M, N), 11 + M)
    ts = x.abs().amax().float()
    q_ref, sf_ref, _ = gk.quantize_nvfp4(x, ts)
    q, sf = gk.quantize_nvfp4_triton(x, ts)
    assert sf.shape == (-(-M // 128) * 128, N // 16)
    np.testing.assert_array_equal(u8(q), u8(q_ref))
    np.testing.assert_array_equal(u8(gk.unpermute_nv_sf(sf))[:M], u8(sf_ref))
    # padding rows of the swizzled buffer are zero
    assert not u8(gk.unpermute_nv_sf(sf))[M:].any()
    want_q, want_sf, _ = oq.quantize_nvfp4(f32np(x), np.float32(float(ts)))
    np.testing.assert_array_equal(u8(q), want_q)
    np.testing.assert_array_equal(u8(sf_ref), want_sf)


def test_nvfp4_edge_cases(gk, golden_quant):
    g = golden_quant
    x = bf16_from_bits(g["tricky_x"]).cuda()
    q, sf, ts = gk.quantize_nvfp4(x)
    assert float(ts) == float(g["tricky_nvfp4_ts"])
    np.testing.assert_array_equal(u8(sf), g["tricky_nvfp4_sf"])
    np.testing.assert_array_equal(u8(q), g["tricky_nvfp4_q"])


def test_nvfp4_all_zero_and_tiny(gk):
    x = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    q, sf, ts = gk.quantize_nvfp4(x)
    assert float(ts) == 0 and not u8(q).any() and not u8(sf).any()
    x = torch.full((16, 64), 1e-35, dtype=torch.bfloat16, device="cuda")
    q, sf, ts = gk.quantize_nvfp4(x)
    wq, wsf, wts = oq.quantize_nvfp4(f32np(x))
    assert float(ts) == float(wts)
    np.testing.assert_array_equal(u8(q), wq)
    np.testing.assert_array_equal(u8(sf), wsf)


@pytest.mark.parametrize("M,K,seed", [(8, 16, 1), (5, 48, 2), (130, 4096, 3), (1024, 1024, 4)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_nvfp4_random_wide_range(gk, M, K, seed, dtype):
    x = wide_range_bf16(M, K, seed).to(dtype)
    if dtype == torch.float32:  # values off the bf16 grid
        x = x * (1 + torch.rand_like(x) * 1e-3)
    q, sf, ts = gk.quantize_nvfp4(x)
    wq, wsf, wts = oq.quantize_nvfp4(f32np(x))
    assert float(ts) == float(wts)
    np.testing.assert_array_equal(u8(sf), wsf)
    np.testing.assert_array_equal(u8(q), wq)


def test_nvfp4_full_size_bit_exact(gk):
    # the benchmark configuration: 8192 x 8192 bf16 N(0,1), ts = amax / (6 * 448)
    x = randn_bf16((8192, 8192), 2025 * 2024 + 2027)
    q, sf, ts = gk.quantize_nvfp4(x)
    # oracle on row slabs (bounded CPU time): 3 slabs of 256 rows, same tensor scale
    xf = x.float().cpu().numpy()
    assert float(ts) == float(oq.nvfp4_tensor_scale(xf))
    qh, sfh = u8(q), u8(sf)
    for r0 in (0, 4096 - 128, 8192 - 256):
        wq, wsf, _ = oq.quantize_nvfp4(xf[r0 : r0 + 256], np.float32(float(ts)))
        np.testing.assert_array_equal(qh[r0 : r0 + 256], wq)
        np.testing.assert_array_equal(sfh[r0 : r0 + 256], wsf)
    # size-independent property: dequantised values reproduce x within half an E2M1 step of the block scale
    deq = gk.dequantize_nvfp4(q, sf, ts)
    err = (deq - x.float()).abs().view(8192, -1, 16).amax(-1)
    step = sf.float() * ts  # value of one unit; largest E2M1 gap is 2 units
    assert bool((err <= step * 1.0 + 1e-12).all())


@pytest.mark.parametrize("method", ["ocp", "nv"])
@pytest.mark.parametrize("dt,kind", [(torch.float8_e4m3fn, "e4m3"), (torch.float8_e5m2, "e5m2"), (torch.float4_e2m1fn_x2, "e2m1")])
def test_quantize_mx(gk, golden_quant, method, dt, kind):
    tag = {"e4m3": "mxfp8", "e5m2": "mxe5m2", "e2m1": "mxfp4"}[kind]
    g = golden_quant
    x = bf16_from_bits(g["tricky_x"]).cuda()
    q, sf = gk.quantize_mx(x, dt, method)
    np.testing.assert_array_equal(u8(sf), g[f"tricky_{tag}_{method}_sf"])
    np.testing.assert_array_equal(u8(q), g[f"tricky_{tag}_{method}_q"])
    for M, K, seed in [(3, 32, 5), (257, 2048, 6)]:
        x = wide_range_bf16(M, K, seed)
        q, sf = gk.quantize_mx(x, dt, method)
        wq, wsf = oq.quantize_mx(f32np(x), kind, method)
        np.testing.assert_array_equal(u8(sf), wsf)
        np.testing.assert_array_equal(u8(q), wq)


def test_quantize_mx_full_size_and_dequant(gk):
    x = randn_bf16((8192, 8192), 7)
    q, sf = gk.quantize_mx(x, torch.float8_e4m3fn)
    xf = x.float().cpu().numpy()
    qh, sfh = u8(q), u8(sf)
    for r0 in (0, 5000, 8192 - 128):
        wq, wsf = oq.quantize_mx(xf[r0 : r0 + 128], "e4m3", "ocp")
        np.testing.assert_array_equal(qh[r0 : r0 + 128], wq)
        np.testing.assert_array_equal(sfh[r0 : r0 + 128], wsf)
    deq = gk.dequantize_mx(q, sf)
    want = oq.dequantize_mx(qh[:64], sfh[:64], "e4m3")
    np.testing.assert_array_equal(f32np(deq[:64]), want)
    # swizzled scales from the quantizer == permute_nv_sf of the row-major ones
    q2, sf2 = gk.quantize_mx(x, torch.float8_e4m3fn, swizzled_scales=True)
    assert torch.equal(q2.view(torch.uint8), q.view(torch.uint8))
    assert torch.equal(sf2.view(torch.uint8), gk.permute_nv_sf(sf).view(torch.uint8))


def test_dequantize_mx_fp4_roundtrip(gk):
    x = wide_range_bf16(64, 256, 9)
    q, sf = gk.quantize_mx(x, torch.float4_e2m1fn_x2)
    deq = gk.dequantize_mx(q, sf)
    want = oq.dequantize_mx(u8(q), u8(sf), "e2m1")
    np.testing.assert_array_equal(f32np(deq), want)


@pytest.mark.parametrize("M,Ks", [(200, 6), (256, 8), (1, 1), (129, 5), (8192, 256)])
def test_permute_nv_sf(gk, M, Ks):
    s = torch.randint(0, 256, (M, Ks), dtype=torch.uint8, generator=torch.Generator().manual_seed(M)).cuda()
    p = gk.permute_nv_sf(s)
    np.testing.assert_array_equal(u8(p), oq.permute_nv_sf(u8(s)))
    back = gk.unpermute_nv_sf(p)
    np.testing.assert_array_equal(u8(back)[:M, :Ks], u8(s))


def test_permute_nv_sf_golden(gk, golden_quant):
    g = golden_quant
    p = gk.permute_nv_sf(torch.from_numpy(g["sf_raw"]).cuda())
    np.testing.assert_array_equal(u8(p), g["sf_perm"])


@pytest.mark.parametrize("dt,kind", [(torch.int8, "int8"), (torch.float8_e4m3fn, "e4m3")])
def test_rowwise_golden_and_random(gk, golden_quant, dt, kind):
    g = golden_quant
    x = bf16_from_bits(g["row_x"]).cuda()
    q, s = gk.quantize_rowwise(x, dt)
    np.testing.assert_array_equal(f32np(s), g[f"row_{kind}_s"])
    np.testing.assert_array_equal(u8(q), g[f"row_{kind}_q"])
    for shape, seed in [((2, 64, 8, 128), 1), ((1024, 1024), 2), ((3, 8), 3), ((17, 8192), 4)]:
        gen = torch.Generator().manual_seed(seed)
        x = (torch.randn(*shape, generator=gen) * 3).cuda()  # fp32 input as in upstream cfg1
        q, s = gk.quantize_rowwise(x, dt)
        wq, ws = oq.quantize_rowwise(f32np(x), kind)
        np.testing.assert_array_equal(f32np(s), ws)
        np.testing.assert_array_equal(u8(q), wq.view(np.uint8))


def test_rowwise_transposed_scales(gk):
    x = randn_bf16((2, 48, 4, 128), 21)
    q, s = gk.quantize_rowwise(x, torch.float8_e4m3fn, transpose_scales=True)
    q2, s2 = gk.quantize_rowwise(x, torch.float8_e4m3fn)
    assert s.shape == (2, 4, 48)
    assert torch.equal(s, s2.transpose(1, 2).contiguous())
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8))


def test_cpu_tensor_raises(gk):
    with pytest.raises(RuntimeError):
        gk.quantize_mx(torch.randn(4, 32), torch.float8_e4m3fn)
    with pytest.raises((ValueError, AssertionError)):
        gk.quantize_nvfp4(torch.randn(4, 24, device="cuda").bfloat16())

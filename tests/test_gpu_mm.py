"""GPU parity: tcgen05 GEMM family vs the CPU oracle, through the public Python API.

INT8 results (int32 accumulators and the row-scaled bf16 epilogue) must be bit-exact.
Floating-point kinds are bounded against the fp32 dequantise-then-matmul oracle both globally
(max|out-ref| <= 1e-2 * max|ref|) and element by element (|out-ref| <= 1e-2*|ref| + 1e-3*max|ref|);
observed errors are ~2e-3: one bf16 rounding of the output.
"""

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits
from gpu_util import SEED_MM, assert_parity, f32np, randn_bf16, u8
from oracle import mm as omm
from oracle import quant as oq

pytestmark = pytest.mark.gpu

TOL = 1e-2
TILES = [-1, 0, 1, 2, 3]  # automatic, 2-CTA 256x256, 128x256, 128x128, 128x64
SHAPES = [(128, 128, 128), (256, 256, 512), (384, 512, 1024), (200, 136, 160), (1, 8, 32), (513, 264, 4096)]


@pytest.fixture(scope="module")
def gk():
    import gn_kernels_b200 as g

    return g


@pytest.fixture(autouse=True)
def _tile_reset_and_status():
    from gn_kernels_b200 import _lib

    yield
    _lib.lib().gnk_debug_force_tile(-1)
    _lib.lib().gnk_debug_staged(-1)
    _lib.raise_on_device_error()


def force(tile):
    from gn_kernels_b200 import _lib

    assert _lib.lib().gnk_debug_force_tile(tile) == 0


def rand_i8(shape, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(-128, 128, shape, dtype=torch.int8, generator=g)


@pytest.mark.parametrize("tile", TILES)
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_bf16(gk, tile, M, N, K):
    K = max(K, 8) // 8 * 8
    force(tile)
    A = randn_bf16((M, K), 1, "cpu")
    Bt = randn_bf16((N, K), 2, "cpu")
    out = gk.cutedsl.sm100.sm100_mm_bf16.mm(A.cuda(), Bt.cuda().T)
    assert_parity(out, omm.mm_bf16(A, Bt))
    out2 = gk.triton_mm(A.cuda(), Bt.cuda().T)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("tile", TILES)
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_int8_exact(gk, tile, M, N, K):
    K = max(K, 16) // 16 * 16
    force(tile)
    A, Bt = rand_i8((M, K), 3), rand_i8((N, K), 4)
    out = gk.triton_mm(A.cuda(), Bt.cuda().T)
    assert out.dtype == torch.int32
    ref = omm.int8_mm_exact(A, Bt)
    assert torch.equal(out.cpu(), ref)
    g = torch.Generator().manual_seed(5)
    sA = torch.randn(M, 1, generator=g).div(128)
    sB = torch.randn(1, N, generator=g).div(128)
    bias = torch.randn(N, generator=g)
    out = gk.triton_mm(A.cuda(), Bt.cuda().T, scale_A=sA.cuda(), scale_B=sB.cuda())
    assert out.dtype == torch.bfloat16
    assert torch.equal(out.cpu(), omm.mm_i8_row_scaled(A, Bt, sA, sB))
    out = gk.triton_mm(A.cuda(), Bt.cuda().T, bias.cuda(), scale_A=sA.cuda(), scale_B=sB.cuda())
    assert torch.equal(out.cpu(), omm.mm_i8_row_scaled(A, Bt, sA, sB, bias))
    out = gk.triton_mm(A.cuda(), Bt.cuda().T, scale_B=sB.cuda())
    assert torch.equal(out.cpu(), omm.mm_i8_row_scaled(A, Bt, None, sB))


@pytest.mark.parametrize("tile", TILES)
@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("acc16", [False, True])
def test_fp16_and_fp16_accumulate(gk, tile, M, N, K, acc16):
    """fp16 operands (upstream triton_mm.py:155-161: output takes A's dtype) with fp32 accumulation, and
    `acc_dtype=torch.float16` (:164-165).  The fp16-accumulated result is compared with the emulation
    upstream uses for that mode (tests/test_cuda_mm.py:66-75: fp32 products of one MMA K step added into
    an fp16 sum) and, loosely, with the fp32 result: the tensor core may keep more bits inside an
    instruction than the emulation does, never fewer."""
    K = max(K, 8) // 8 * 8
    force(tile)
    g = torch.Generator().manual_seed(M + 3 * N + K)
    A = (torch.randn(M, K, generator=g) / K**0.25).half()
    Bt = (torch.randn(N, K, generator=g) / K**0.25).half()
    out = gk.triton_mm(A.cuda(), Bt.cuda().T, acc_dtype=torch.float16 if acc16 else None)
    assert out.dtype == torch.float16
    exact = A.float() @ Bt.float().T
    if not acc16:
        assert_parity(out, exact.half())
        return
    emu = torch.zeros(M, N, dtype=torch.float16)
    for k0 in range(0, K, 16):  # one kind::f16 instruction covers 16 elements of K
        emu = (emu.float() + A[:, k0 : k0 + 16].float() @ Bt[:, k0 : k0 + 16].float().T).half()
    scale = float(exact.abs().max())
    err_emu = float((out.float().cpu() - emu.float()).abs().max()) / scale
    err_exact = float((out.float().cpu() - exact).abs().max()) / scale
    emu_exact = float((emu.float() - exact).abs().max()) / scale
    assert err_exact <= max(2.0 * emu_exact, 2e-3), (err_exact, emu_exact)
    assert err_emu <= max(2.0 * emu_exact, 2e-3), (err_emu, emu_exact)


def test_int8_golden_and_config1(gk, golden_mm):
    g = golden_mm
    A, Bt = torch.from_numpy(g["i8_A"]), torch.from_numpy(g["i8_Bt"])
    out = gk.triton_mm(A.cuda(), Bt.cuda().T)
    np.testing.assert_array_equal(out.cpu().numpy(), g["i8_acc"])
    sA, sB = torch.from_numpy(g["i8_sA"]).reshape(-1, 1), torch.from_numpy(g["i8_sB"]).reshape(1, -1)
    out = gk.triton_mm(A.cuda(), Bt.cuda().T, scale_A=sA.cuda(), scale_B=sB.cuda())
    torch.testing.assert_close(out.cpu(), bf16_from_bits(g["i8_scaled_ref"]), atol=4e-4, rtol=1e-2)  # upstream's own tolerance
    # configuration 1 end to end: fp32 N(0,1) 1024^3 -> row-wise int8 -> row-scaled GEMM, all on the GPU
    gen = torch.Generator().manual_seed(SEED_MM)
    A32, B32 = torch.randn(1024, 1024, generator=gen), torch.randn(1024, 1024, generator=gen)
    Aq, sA = gk.quantize_rowwise(A32.cuda(), torch.int8)
    Bq, sB = gk.quantize_rowwise(B32.cuda(), torch.int8)
    wAq, wsA = oq.quantize_rowwise(A32.numpy(), "int8")
    wBq, wsB = oq.quantize_rowwise(B32.numpy(), "int8")
    np.testing.assert_array_equal(Aq.cpu().numpy(), wAq)
    np.testing.assert_array_equal(f32np(sB), wsB)
    acc = gk.triton_mm(Aq, Bq.T)
    assert torch.equal(acc.cpu(), omm.int8_mm_exact(wAq, wBq))
    out = gk.triton_mm(Aq, Bq.T, scale_A=sA.view(-1, 1), scale_B=sB.view(1, -1))
    assert torch.equal(out.cpu(), omm.mm_i8_row_scaled(wAq, wBq, wsA, wsB))


@pytest.mark.parametrize("tile", TILES)
@pytest.mark.parametrize("M,N,K", SHAPES)
def test_fp8_row_scaled(gk, tile, M, N, K):
    K = max(K, 16) // 16 * 16
    force(tile)
    g = torch.Generator().manual_seed(6)
    A = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn)
    Bt = torch.randn(N, K, generator=g).to(torch.float8_e4m3fn)
    sA = torch.rand(M, 1, generator=g) + 0.5
    sB = torch.rand(1, N, generator=g) + 0.5
    out = gk.triton_mm(A.cuda(), Bt.cuda().T)
    assert_parity(out, omm.mm_f8_row_scaled(u8(A), u8(Bt)))
    out = gk.triton_mm(A.cuda(), Bt.cuda().T, scale_A=sA.cuda(), scale_B=sB.cuda())
    assert_parity(out, omm.mm_f8_row_scaled(u8(A), u8(Bt), sA, sB))


def test_fp8_golden(gk, golden_mm):
    g = golden_mm
    A = torch.from_numpy(g["f8_A"]).view(torch.float8_e4m3fn).cuda()
    Bt = torch.from_numpy(g["f8_Bt"]).view(torch.float8_e4m3fn).cuda()
    out = gk.triton_mm(A, Bt.T)
    assert_parity(out, bf16_from_bits(g["f8_plain_ref"]))
    sA, sB = torch.from_numpy(g["f8_sA"]).reshape(-1, 1).cuda(), torch.from_numpy(g["f8_sB"]).reshape(1, -1).cuda()
    out = gk.triton_mm(A, Bt.T, scale_A=sA, scale_B=sB)
    torch.testing.assert_close(out.cpu(), bf16_from_bits(g["f8_scaled_ref"]), atol=4e-4, rtol=1e-2)


BS_TILES = [-1, 0, 1, 2, 3, 4]  # 4: the 2-CTA 256x192 tile of the block-scaled kinds
BS_SHAPES = [(128, 128, 128), (256, 256, 512), (384, 512, 1024), (200, 136, 160), (16, 256, 2048), (513, 264, 4096)]


@pytest.mark.parametrize("tile", BS_TILES)
@pytest.mark.parametrize("M,N,K", BS_SHAPES)
def test_mxfp8(gk, tile, M, N, K):
    force(tile)
    A = randn_bf16((M, K), 7)
    Bt = randn_bf16((N, K), 8)
    # give blocks different exponents so a misplaced scale factor cannot go unnoticed
    A = (A.float() * torch.exp2(torch.randint(-3, 4, (M, K // 32, 1), device="cuda").float()).expand(M, K // 32, 32).reshape(M, K)).bfloat16()
    Aq, sfa = gk.quantize_mx(A, torch.float8_e4m3fn)
    Bq, sfb = gk.quantize_mx(Bt, torch.float8_e4m3fn)
    out = gk.cutedsl.sm100.sm100_mm_mxfp8.mm(Aq, Bq, gk.permute_nv_sf(sfa), gk.permute_nv_sf(sfb))
    ref = omm.mm_mxfp8(u8(Aq), u8(Bq), u8(sfa), u8(sfb))
    assert_parity(out, ref)


def test_mxfp8_golden(gk, golden_mm):
    g = golden_mm
    A = torch.from_numpy(g["mx_A"]).view(torch.float8_e4m3fn).cuda()
    Bt = torch.from_numpy(g["mx_Bt"]).view(torch.float8_e4m3fn).cuda()
    sfa = torch.from_numpy(g["mx_sfa"]).view(torch.float8_e8m0fnu).cuda()
    sfb = torch.from_numpy(g["mx_sfb"]).view(torch.float8_e8m0fnu).cuda()
    out = gk.cutedsl.sm100.sm100_mm_mxfp8.mm(A, Bt, gk.permute_nv_sf(sfa), gk.permute_nv_sf(sfb))
    assert_parity(out, bf16_from_bits(g["mx_ref"]))


@pytest.mark.parametrize("tile", BS_TILES)
@pytest.mark.parametrize("M,N,K", BS_SHAPES)
def test_nvfp4(gk, tile, M, N, K):
    K = max(K, 64) // 64 * 64
    force(tile)
    A = randn_bf16((M, K), 9)
    Bt = randn_bf16((N, K), 10)
    A = (A.float() * torch.exp2(torch.randint(-3, 4, (M, K // 16, 1), device="cuda").float()).expand(M, K // 16, 16).reshape(M, K)).bfloat16()
    Aq, sfa, tsa = gk.quantize_nvfp4(A)
    Bq, sfb, tsb = gk.quantize_nvfp4(Bt)
    alpha = float(tsa) * float(tsb)
    out = gk.cutedsl.sm100.sm100_mm_nvfp4.mm(Aq, Bq, gk.permute_nv_sf(sfa), gk.permute_nv_sf(sfb), alpha)
    ref = omm.mm_nvfp4(u8(Aq), u8(Bq), u8(sfa), u8(sfb), np.float32(float(tsa)) * np.float32(float(tsb)))
    assert_parity(out, ref)
    # the swizzled-scale quantizer feeds the GEMM directly
    Aq2, sfa2 = gk.quantize_nvfp4_triton(A, tsa) if K % 64 == 0 else (Aq, gk.permute_nv_sf(sfa))
    out2 = gk.cutedsl.sm100.sm100_mm_nvfp4.mm(Aq2, Bq, sfa2, gk.permute_nv_sf(sfb), alpha)
    assert torch.equal(out, out2)


def _sampled_rows(M, n=64, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.sort(torch.randperm(M, generator=g)[:n]).values


@pytest.mark.parametrize("kind", ["bf16", "int8", "fp8", "mxfp8", "nvfp4"])
@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (384, 512, 1024), (1000, 1024, 512), (2048, 2304, 4096)])
def test_pair_tile_epilogue_modes(gk, kind, M, N, K):
    """The 256 x 256 pair tile writes bf16 through bulk tensor stores from swizzled staging (default)
    or straight from registers; both must give the same bits (ragged M, many tiles per cluster)."""
    from gn_kernels_b200 import _lib

    force(0)
    A = randn_bf16((M, K), 31)
    Bt = randn_bf16((N, K), 32)
    if kind == "bf16":
        run = lambda: gk.triton_mm(A, Bt.T)
    elif kind == "int8":
        Ai, Bi = rand_i8((M, K), 33).cuda(), rand_i8((N, K), 34).cuda()
        sa, sb = torch.rand(M, 1, device="cuda") + 0.5, torch.rand(1, N, device="cuda") + 0.5
        bias = torch.randn(N, device="cuda")
        run = lambda: gk.triton_mm(Ai, Bi.T, bias, scale_A=sa, scale_B=sb)
    elif kind == "fp8":
        Af, Bf = A.to(torch.float8_e4m3fn), Bt.to(torch.float8_e4m3fn)
        sa, sb = torch.rand(M, 1, device="cuda") + 0.5, torch.rand(1, N, device="cuda") + 0.5
        run = lambda: gk.triton_mm(Af, Bf.T, scale_A=sa, scale_B=sb)
    elif kind == "mxfp8":
        Aq, sfa = gk.quantize_mx(A, torch.float8_e4m3fn, swizzled_scales=True)
        Bq, sfb = gk.quantize_mx(Bt, torch.float8_e4m3fn, swizzled_scales=True)
        run = lambda: gk.cutedsl.sm100.sm100_mm_mxfp8.mm(Aq, Bq, sfa, sfb)
    else:
        ts = gk.ops.absmax(A, 2688.0)
        Aq, sfa = gk.quantize_nvfp4_triton(A, ts)
        Bq, sfb = gk.quantize_nvfp4_triton(Bt, ts)
        run = lambda: gk.cutedsl.sm100.sm100_mm_nvfp4.mm(Aq, Bq, sfa, sfb, float(ts) ** 2)
    outs = []
    for mode in (0, 1):
        _lib.lib().gnk_debug_staged(mode)
        outs.append(run().clone())
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("kind", ["int8", "mxfp8", "nvfp4", "bf16", "fp8", "fp8_block128", "fp8_block128_deepseek"])
def test_full_size_8192(gk, kind):
    """Benchmark-size problems: oracle on 64 sampled rows x all columns, and every row block written."""
    M = N = K = 8192
    if kind == "fp8_block128_deepseek":
        M, N, K = 4096, 7168, 2048  # a DeepSeek-V3 projection shape (hidden 7168)
    rows = _sampled_rows(M)
    if kind in ("fp8", "fp8_block128", "fp8_block128_deepseek"):
        g = torch.Generator().manual_seed(SEED_MM + 7)
        A = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn)
        Bt = torch.randn(N, K, generator=g).to(torch.float8_e4m3fn)
        if kind == "fp8":
            sA, sB = torch.rand(M, 1, generator=g) + 0.5, torch.rand(1, N, generator=g) + 0.5
            out = gk.triton_mm(A.cuda(), Bt.cuda().T, scale_A=sA.cuda(), scale_B=sB.cuda())
            ref = omm.mm_f8_row_scaled(u8(A[rows]), u8(Bt), sA[rows], sB)
        else:
            sfa = (torch.rand(K // 128, M, generator=g) + 0.25).T  # M-major view [M, K/128]
            sfb = torch.rand(N // 128, K // 128, generator=g) + 0.25
            out = gk.cutedsl.sm120.sm120_mm_fp8_1d2d.mm(A.cuda(), sfa.cuda(), Bt.cuda(), sfb.cuda())
            ref = omm.mm_f8_block128(u8(A[rows]), sfa[rows], u8(Bt), sfb)
        assert_parity(out[rows.cuda()], ref)
        assert bool((out.float().abs().amax(dim=1) > 0).all())
        return
    if kind == "int8":
        A, Bt = rand_i8((M, K), 11), rand_i8((N, K), 12)
        out = gk.triton_mm(A.cuda(), Bt.cuda().T)
        assert torch.equal(out[rows.cuda()].cpu(), omm.int8_mm_exact(A[rows], Bt))
        return
    A = randn_bf16((M, K), SEED_MM)
    Bt = randn_bf16((N, K), SEED_MM + 1)
    if kind == "bf16":
        out = gk.cutedsl.sm100.sm100_mm_bf16.mm(A, Bt.T)
        ref = omm.mm_bf16(A[rows.cuda()].cpu(), Bt.cpu())
    elif kind == "mxfp8":
        Aq, sfa = gk.quantize_mx(A, torch.float8_e4m3fn)
        Bq, sfb = gk.quantize_mx(Bt, torch.float8_e4m3fn)
        out = gk.cutedsl.sm100.sm100_mm_mxfp8.mm(Aq, Bq, gk.permute_nv_sf(sfa), gk.permute_nv_sf(sfb))
        r = rows.cuda()
        ref = omm.mm_mxfp8(u8(Aq[r]), u8(Bq), u8(sfa[r]), u8(sfb))
    else:
        Aq, sfa, tsa = gk.quantize_nvfp4(A)
        Bq, sfb, tsb = gk.quantize_nvfp4(Bt)
        alpha = float(tsa) * float(tsb)
        out = gk.cutedsl.sm100.sm100_mm_nvfp4.mm(Aq, Bq, gk.permute_nv_sf(sfa), gk.permute_nv_sf(sfb), alpha)
        r = rows.cuda()
        ref = omm.mm_nvfp4(u8(Aq.view(torch.uint8)[r]), u8(Bq), u8(sfa[r]), u8(sfb), np.float32(float(tsa)) * np.float32(float(tsb)))
    assert_parity(out[rows.cuda()], ref)
    # every row block was written (no tile skipped): no row of the output is all zero
    assert bool((out.float().abs().amax(dim=1) > 0).all())


@pytest.mark.parametrize("M", [1, 16, 64, 128])
def test_mxfp8_skinny_decode_shapes(gk, M):
    N = K = 8192
    A = randn_bf16((M, K), 31)
    Bt = randn_bf16((N, K), 32)
    Aq, sfa = gk.quantize_mx(A, torch.float8_e4m3fn)
    Bq, sfb = gk.quantize_mx(Bt, torch.float8_e4m3fn)
    out = gk.cutedsl.sm100.sm100_mm_mxfp8.mm(Aq, Bq, gk.permute_nv_sf(sfa), gk.permute_nv_sf(sfb))
    ref = omm.mm_mxfp8(u8(Aq), u8(Bq), u8(sfa), u8(sfb))
    assert_parity(out, ref)


@pytest.mark.parametrize("M,N,K", [(16, 2048, 4096), (100, 1024, 4096 + 384), (128, 4096 + 64, 8192), (8, 512, 6144 + 128)])
def test_skinny_dense_kinds_deep_stages(gk, M, N, K):
    """The same pipeline for the kinds without block scales: INT8 stays exact (int32 sums in any order),
    FP8 row-scaled and BF16 stay within the parity bound and within one output step of the one-slice pipeline."""
    from gn_kernels_b200 import _lib

    L = _lib.lib()
    A8, B8 = rand_i8((M, K), 71), rand_i8((N, K), 72)
    g = torch.Generator().manual_seed(73)
    sA, sB = torch.randn(M, 1, generator=g).div(128), torch.randn(1, N, generator=g).div(128)
    Ab, Bb = randn_bf16((M, K), 74, "cpu"), randn_bf16((N, K), 75, "cpu")
    Af, sAf = gk.quantize_rowwise(Ab.cuda(), torch.float8_e4m3fn)
    Bf, sBf = gk.quantize_rowwise(Bb.cuda(), torch.float8_e4m3fn)

    def run():
        return (gk.triton_mm(A8.cuda(), B8.cuda().T), gk.triton_mm(A8.cuda(), B8.cuda().T, scale_A=sA.cuda(), scale_B=sB.cuda()),
                gk.triton_mm(Af, Bf.T, scale_A=sAf.view(M, 1), scale_B=sBf.view(1, N)), gk.triton_mm(Ab.cuda(), Bb.cuda().T))

    try:
        assert L.gnk_debug_force_tile(3) == 0
        deep = run()
        assert L.gnk_debug_deep_stage(0) == 0
        one = run()
    finally:
        L.gnk_debug_deep_stage(1)
        L.gnk_debug_force_tile(-1)
    assert torch.equal(deep[0].cpu(), omm.int8_mm_exact(A8, B8))
    assert torch.equal(deep[1].cpu(), omm.mm_i8_row_scaled(A8, B8, sA, sB))
    assert torch.equal(deep[0], one[0]) and torch.equal(deep[1], one[1])
    assert_parity(deep[3], omm.mm_bf16(Ab, Bb))
    for d, o in ((deep[2], one[2]), (deep[3], one[3])):
        assert float((d.float() - o.float()).abs().max()) <= 2.0**-7 * float(o.float().abs().max())


def test_back_to_back_dependent_decode_gemms(gk):
    """The decode-shaped kernels are launched with programmatic stream serialization: the next kernel's
    set-up may run under the previous one's tail, but it must not read or write global memory before its
    predecessor has finished.  A chain in which every GEMM consumes the previous one's output (and the
    last overwrites the first's input buffer) gives the same bits as the same chain with a host
    synchronisation after every launch."""
    M, D = 16, 4096
    g = torch.Generator().manual_seed(81)
    x0 = (torch.randn(M, D, generator=g)).bfloat16().cuda()
    Ws = [(torch.randn(D, D, generator=g) / D**0.5).bfloat16().cuda() for _ in range(4)]

    def chain(sync):
        x = x0.clone()
        for rep in range(3):
            for W in Ws:
                x = gk.cutedsl.sm100.sm100_mm_bf16.mm(x, W.T)
                if sync:
                    torch.cuda.synchronize()
        return x

    ref = chain(True)
    for _ in range(5):
        assert torch.equal(chain(False), ref)
    # and against the oracle for the first link
    assert_parity(gk.cutedsl.sm100.sm100_mm_bf16.mm(x0, Ws[0].T), omm.mm_bf16(x0.cpu(), Ws[0].cpu()))


@pytest.mark.parametrize("kind", ["mxfp8", "nvfp4"])
@pytest.mark.parametrize("M,N,K", [(16, 2048, 4096), (100, 1024, 4096 + 384), (128, 4096 + 64, 8192), (8, 512, 6144 + 128)])
def test_skinny_four_k_slices_per_stage(gk, kind, M, N, K):
    """One tile per CTA and a long K take the pipeline with four (few rows) or two 128-byte K slices per
    stage (rank-3 boxes) and two issuing threads, each with an accumulator of its own; the sum of the
    two differs from the one-slice pipeline's single accumulator by fp32 rounding only.  K that is not
    a multiple of the stage depth ends in zero-filled slices."""
    from gn_kernels_b200 import _lib

    L = _lib.lib()
    A = randn_bf16((M, K), 61)
    Bt = randn_bf16((N, K), 62)
    if kind == "mxfp8":
        Aq, sfa = gk.quantize_mx(A, torch.float8_e4m3fn)
        Bq, sfb = gk.quantize_mx(Bt, torch.float8_e4m3fn)
        run = lambda: gk.cutedsl.sm100.sm100_mm_mxfp8.mm(Aq, Bq, gk.permute_nv_sf(sfa), gk.permute_nv_sf(sfb))  # noqa: E731
        ref = omm.mm_mxfp8(u8(Aq), u8(Bq), u8(sfa), u8(sfb))
    else:
        Aq, sfa, tsa = gk.quantize_nvfp4(A)
        Bq, sfb, tsb = gk.quantize_nvfp4(Bt)
        alpha = float(tsa) * float(tsb)
        run = lambda: gk.cutedsl.sm100.sm100_mm_nvfp4.mm(Aq, Bq, gk.permute_nv_sf(sfa), gk.permute_nv_sf(sfb), alpha)  # noqa: E731
        ref = omm.mm_nvfp4(u8(Aq), u8(Bq), u8(sfa), u8(sfb), np.float32(float(tsa)) * np.float32(float(tsb)))
    try:
        assert L.gnk_debug_force_tile(3) == 0  # the 128 x 64 tile, as the automatic choice makes for these shapes
        out = run()
        assert L.gnk_debug_deep_stage(0) == 0
        one_slice = run()
    finally:
        L.gnk_debug_deep_stage(1)
        L.gnk_debug_force_tile(-1)
    assert_parity(out, ref)
    assert_parity(one_slice, ref)
    # the same products summed in another order: a few outputs move by one bf16 step
    assert float((out.float() - one_slice.float()).abs().max()) <= 2.0**-7 * float(ref.float().abs().max())


def test_strided_and_unaligned_operands(gk):
    # column-major A and row-major [K,N] B are legal for triton_mm (copied into K-major form)
    A = rand_i8((96, 80), 41).cuda()
    B = rand_i8((80, 72), 42).cuda()  # [K, N] contiguous: NOT the fast layout
    out = gk.triton_mm(A.T.contiguous().T, B)
    assert torch.equal(out.cpu(), omm.int8_mm_exact(A.cpu(), B.T.contiguous().cpu()))
    # K not a multiple of 16 bytes: padded copy
    A = rand_i8((40, 50), 43).cuda()
    Bt = rand_i8((24, 50), 44).cuda()
    out = gk.triton_mm(A, Bt.T)
    assert torch.equal(out.cpu(), omm.int8_mm_exact(A.cpu(), Bt.cpu()))


def test_bad_arguments(gk):
    A = torch.zeros(16, 32, dtype=torch.int8, device="cuda")
    with pytest.raises(AssertionError):
        gk.triton_mm(A, torch.zeros(16, 32, dtype=torch.int8, device="cuda"))
    with pytest.raises(NotImplementedError):
        gk.triton_mm(A.float(), A.float().T)
    with pytest.raises(NotImplementedError):  # the fp16 accumulator goes with fp16 operands
        gk.triton_mm(A.bfloat16(), A.bfloat16().T, acc_dtype=torch.float16)
    with pytest.raises(RuntimeError):
        gk.triton_mm(A.cpu(), A.cpu().T)


def test_fp8_block128_golden(gk, golden_mm):
    g = golden_mm
    A = torch.from_numpy(g["blk_A"]).view(torch.float8_e4m3fn).cuda()
    Bt = torch.from_numpy(g["blk_Bt"]).view(torch.float8_e4m3fn).cuda()
    sfa = torch.from_numpy(g["blk_sfa"]).cuda()
    sfb = torch.from_numpy(g["blk_sfb"]).cuda()
    out = gk.cutedsl.sm120.sm120_mm_fp8_1d2d.mm(A, sfa.T.contiguous().T, Bt, sfb)  # SFA stored M-major as upstream wants
    assert_parity(out, bf16_from_bits(g["blk_ref"]))


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (200, 256, 512), (1, 128, 1024), (1024, 1536, 7168 // 4)])
@pytest.mark.parametrize("extras", [False, True])
def test_fp8_block128(gk, M, N, K, extras):
    g = torch.Generator().manual_seed(M + N + K)
    A = torch.randn(M, K, generator=g).to(torch.float8_e4m3fn)
    Bt = torch.randn(N, K, generator=g).to(torch.float8_e4m3fn)
    sfa = (torch.rand(K // 128, M, generator=g) + 0.25).T  # M-major view [M, K/128]
    sfb = torch.rand(N // 128, K // 128, generator=g) + 0.25
    bias = torch.randn(N, generator=g).bfloat16() if extras else None
    add = torch.randn(M, N, generator=g).bfloat16() if extras else None
    out = gk.cutedsl.sm120.sm120_mm_fp8_1d2d.mm(A.cuda(), sfa.cuda(), Bt.cuda(), sfb.cuda(),
                                                bias.cuda() if extras else None, add.cuda() if extras else None)
    ref = omm.mm_f8_block128(u8(A), sfa, u8(Bt), sfb, bias, add)
    assert_parity(out, ref)

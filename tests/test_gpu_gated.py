"""GPU parity: SwiGLU-gated dual NVFP4 GEMM and its re-quantising epilogue
(upstream gn_kernels/cutedsl/sm120/sm120_gated_gemm_nvfp4.py, test tests/test_sm120_gated_gemm_nvfp4.py:29-53).

As upstream's test does: the bf16 output is compared with silu(X W1^T) * (X W3^T) on the dequantised
operands, and the quantised output must equal the NVFP4 quantizer applied to that bf16 output, byte
for byte (packed codes and block scales)."""

import numpy as np
import pytest
import torch

from gpu_util import assert_parity, u8
from oracle import mm as omm
from oracle import quant as oq

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gk():
    import gn_kernels_b200 as g

    return g


@pytest.fixture(autouse=True)
def _status():
    from gn_kernels_b200 import _lib

    yield
    _lib.lib().gnk_debug_force_tile(-1)
    _lib.raise_on_device_error()


def make_input(gk, rows, K, seed):
    """upstream's make_input: N(0,1)/sqrt(K) bf16, tensor scale = absmax (its choice, :33-34), swizzled block scales"""
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, K, generator=g) * K**-0.5).bfloat16().cuda()
    ts = x.abs().amax().float()
    xq, sf = gk.quantize_nvfp4_triton(x, ts)
    xq_rm, sf_rm, _ = gk.quantize_nvfp4(x, ts)  # row-major scales for the oracle
    assert torch.equal(xq.view(torch.uint8), xq_rm.view(torch.uint8))
    return (xq, sf, ts), (u8(xq_rm), u8(sf_rm), np.float32(float(ts)))


@pytest.mark.parametrize("tile", [-1, 0, 1])  # automatic, CTA-pair 256-row tiles, single-CTA 128-row tiles
@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (128, 128, 64), (200, 384, 320), (1000, 512, 1024), (2048, 2304, 512)])
def test_gated_gemm_and_quantised_epilogue(gk, tile, M, N, K):
    from gn_kernels_b200 import _lib
    from gn_kernels_b200.cutedsl.sm120 import sm120_gated_gemm_nvfp4

    assert _lib.lib().gnk_debug_force_tile(tile) == 0
    X, Xo = make_input(gk, M, K, 1)
    W1, W1o = make_input(gk, N, K, 2)
    W3, W3o = make_input(gk, N, K, 3)

    out = sm120_gated_gemm_nvfp4.mm(*X, *W1, *W3)
    assert out.shape == (M, N) and out.dtype == torch.bfloat16
    ref = omm.gated_mm_nvfp4(*Xo, *W1o, *W3o)
    assert_parity(out, ref)

    # quantised case: equals the quantizer run on the bf16 output (upstream :47-53)
    ts_out = out.abs().amax().float()
    q_ref, sf_ref = gk.quantize_nvfp4_triton(out, ts_out)
    q, sf = sm120_gated_gemm_nvfp4.mm(*X, *W1, *W3, ts_out)
    assert q.dtype == torch.float4_e2m1fn_x2 and sf.dtype == torch.float8_e4m3fn
    assert q.shape == (M, N // 2) and sf.shape == sf_ref.shape
    np.testing.assert_array_equal(u8(q), u8(q_ref))
    np.testing.assert_array_equal(u8(sf), u8(sf_ref))
    # and, through the CPU oracle, the torch reference quantizer on the same bf16 values
    wq, wsf, _ = oq.quantize_nvfp4(out.float().cpu().numpy(), np.float32(float(ts_out)))
    np.testing.assert_array_equal(u8(q), wq)
    np.testing.assert_array_equal(u8(gk.unpermute_nv_sf(sf))[:M], wsf)


def test_gated_gemm_rejects_bad_shapes(gk):
    from gn_kernels_b200.cutedsl.sm120 import sm120_gated_gemm_nvfp4

    X, _ = make_input(gk, 128, 64, 1)
    W, _ = make_input(gk, 64, 64, 2)  # N = 64 is not a multiple of 128
    with pytest.raises(ValueError):
        sm120_gated_gemm_nvfp4.mm(*X, *W, *W)

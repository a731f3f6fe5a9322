"""Regenerates tests/golden/*.npz by running the UPSTREAM Python reference on CPU.

Run only where the upstream checkout is available:

    python tests/golden/make_golden.py /path/to/gn-kernels

The fixtures hold seeded inputs and the outputs the upstream torch path produced for
them, so the oracle (and, through it, the CUDA kernels) can be pinned on machines that do
not have the upstream checkout.  bf16 / fp8 tensors are stored as raw integer bit
patterns (numpy has no such dtypes).
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def bits8(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint8).numpy()


def tricky_matrix(M: int, K: int, gen: torch.Generator) -> torch.Tensor:
    """bf16 matrix that hits the quantizers' edge cases: wide dynamic range per block,
    all-zero blocks, subnormal-tiny blocks, exact rounding ties, a block above 448."""
    x = torch.randn(M, K, generator=gen) * torch.exp2(torch.randint(-12, 6, (M, K // 16, 1), generator=gen).float()).expand(
        M, K // 16, 16
    ).reshape(M, K)
    x[0, :32] = 0.0
    x[1, :32] = 1e-30
    x[2, :16] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    x[3, :32] = 449.0
    x[4, :32] = torch.linspace(-500, 500, 32)
    x[5, :32] = -0.0
    return x.bfloat16()


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    from torch.nn.attention.bias import causal_lower_right

    import benchmark_attn  # noqa: E402  (upstream, has a __main__ guard)
    import benchmark_mm  # noqa: E402
    from gn_kernels import quant_utils as Q  # noqa: E402

    g = torch.Generator().manual_seed(2025 * 2024 + 2027)

    # ---------------- quantizers ----------------
    out = {}
    for name, (M, K) in {"a": (256, 128), "b": (196, 256)}.items():
        x = torch.randn(M, K, generator=g).bfloat16()
        ts = x.abs().amax().float()  # the upstream test passes amax itself as tensor_scale
        xq, sf, _ = Q.quantize_nvfp4(x, ts)
        out[f"nvfp4_{name}_x"] = bits16(x)
        out[f"nvfp4_{name}_ts"] = ts.numpy()
        out[f"nvfp4_{name}_q"] = bits8(xq)
        out[f"nvfp4_{name}_sf"] = bits8(sf)
        xq2, sf2, ts2 = Q.quantize_nvfp4(x)  # tensor scale computed by the callee
        out[f"nvfp4_{name}_auto_ts"] = ts2.numpy()
        out[f"nvfp4_{name}_auto_q"] = bits8(xq2)
        out[f"nvfp4_{name}_auto_sf"] = bits8(sf2)

    xt = tricky_matrix(64, 256, g)
    out["tricky_x"] = bits16(xt)
    xq, sf, ts = Q.quantize_nvfp4(xt)
    out["tricky_nvfp4_q"], out["tricky_nvfp4_sf"], out["tricky_nvfp4_ts"] = bits8(xq), bits8(sf), ts.numpy()
    for method in ("ocp", "nv"):
        xq, sf = Q.quantize_mx(xt, torch.float8_e4m3fn, method)
        out[f"tricky_mxfp8_{method}_q"], out[f"tricky_mxfp8_{method}_sf"] = bits8(xq), bits8(sf)
        out[f"tricky_mxfp8_{method}_deq"] = Q.dequantize_mx(xq, sf).numpy()
        xq, sf = Q.quantize_mx(xt, torch.float4_e2m1fn_x2, method)
        out[f"tricky_mxfp4_{method}_q"], out[f"tricky_mxfp4_{method}_sf"] = bits8(xq), bits8(sf)
        xq, sf = Q.quantize_mx(xt, torch.float8_e5m2, method)
        out[f"tricky_mxe5m2_{method}_q"], out[f"tricky_mxe5m2_{method}_sf"] = bits8(xq), bits8(sf)

    sfr = torch.randint(0, 256, (200, 6), generator=g, dtype=torch.uint8)
    out["sf_raw"] = sfr.numpy()
    out["sf_perm"] = Q.permute_nv_sf(sfr).numpy()
    sfr2 = torch.randint(0, 256, (256, 8), generator=g, dtype=torch.uint8)
    out["sf2_raw"] = sfr2.numpy()
    out["sf2_perm"] = Q.permute_nv_sf(sfr2).numpy()
    out["sf2_unperm_of_perm"] = Q.unpermute_nv_sf(Q.permute_nv_sf(sfr2)).numpy()

    xr = torch.randn(2, 24, 3, 64, generator=g).bfloat16()
    xr[0, 0, 0] = 0.0
    out["row_x"] = bits16(xr)
    for kind, dt in (("int8", torch.int8), ("e4m3", torch.float8_e4m3fn)):
        q, s = benchmark_attn.quantize(xr, dt)
        out[f"row_{kind}_q"] = bits8(q)
        out[f"row_{kind}_s"] = s.numpy()
        out[f"row_{kind}_deq"] = benchmark_attn.dequantize(q, s).numpy()
    np.savez_compressed(os.path.join(HERE, "quant.npz"), **out)

    # ---------------- matmuls ----------------
    out = {}
    M = N = K = 128
    A = torch.randn(M, K, generator=g)
    Bt = torch.randn(N, K, generator=g)
    A_i8, sA = benchmark_attn.quantize(A, torch.int8)
    B_i8, sB = benchmark_attn.quantize(Bt, torch.int8)
    out["i8_A"], out["i8_Bt"] = A_i8.numpy(), B_i8.numpy()
    out["i8_sA"], out["i8_sB"] = sA.numpy(), sB.numpy()
    out["i8_acc"] = torch._int_mm(A_i8, B_i8.T.contiguous()).numpy()
    out["i8_scaled_ref"] = bits16(benchmark_mm.scaled_mm_ref(A_i8, B_i8.T, sA.reshape(M, 1), sB.reshape(1, N)))
    A_f8, sA8 = benchmark_attn.quantize(A, torch.float8_e4m3fn)
    B_f8, sB8 = benchmark_attn.quantize(Bt, torch.float8_e4m3fn)
    out["f8_A"], out["f8_Bt"] = bits8(A_f8), bits8(B_f8)
    out["f8_sA"], out["f8_sB"] = sA8.numpy(), sB8.numpy()
    out["f8_plain_ref"] = bits16((A_f8.float() @ B_f8.float().T).bfloat16())
    out["f8_scaled_ref"] = bits16(benchmark_mm.scaled_mm_ref(A_f8, B_f8.T, sA8.reshape(M, 1), sB8.reshape(1, N)))
    # 2-D block scaling through the same upstream helper (scales repeat over 128-blocks)
    M2, N2, K2 = 128, 256, 256
    A2 = torch.randn(M2, K2, generator=g).to(torch.float8_e4m3fn)
    B2 = torch.randn(N2, K2, generator=g).to(torch.float8_e4m3fn)
    sfa2 = torch.rand(M2, K2 // 128, generator=g) + 0.5
    sfb2 = torch.rand(N2 // 128, K2 // 128, generator=g) + 0.5
    out["blk_A"], out["blk_Bt"], out["blk_sfa"], out["blk_sfb"] = bits8(A2), bits8(B2), sfa2.numpy(), sfb2.numpy()
    out["blk_ref"] = bits16(benchmark_mm.scaled_mm_ref(A2, B2.T, sfa2, sfb2.T))
    # MXFP8: upstream quantize -> upstream dequantize -> fp32 matmul
    Am = torch.randn(128, 256, generator=g).bfloat16()
    Bm = torch.randn(128, 256, generator=g).bfloat16()
    Aq, Asf = Q.quantize_mx(Am, torch.float8_e4m3fn)
    Bq, Bsf = Q.quantize_mx(Bm, torch.float8_e4m3fn)
    out["mx_A"], out["mx_Bt"], out["mx_sfa"], out["mx_sfb"] = bits8(Aq), bits8(Bq), bits8(Asf), bits8(Bsf)
    out["mx_ref"] = bits16((Q.dequantize_mx(Aq, Asf) @ Q.dequantize_mx(Bq, Bsf).T).bfloat16())
    np.savez_compressed(os.path.join(HERE, "mm.npz"), **out)

    # ---------------- attention (upstream test oracle: SDPA + causal_lower_right) ----------------
    out = {}
    bs, hq, hkv, d = 1, 4, 2, 128
    for q_len, kv_len in [(64, 256), (128, 32), (33, 123), (257, 39)]:
        q = torch.randn(bs, q_len, hq, d, generator=g).bfloat16()
        k = torch.randn(bs, kv_len, hkv, d, generator=g).bfloat16()
        v = torch.randn(bs, kv_len, hkv, d, generator=g).bfloat16()
        tag = f"{q_len}x{kv_len}"
        out[f"{tag}_q"], out[f"{tag}_k"], out[f"{tag}_v"] = bits16(q), bits16(k), bits16(v)
        for causal in (False, True):
            o = F.scaled_dot_product_attention(
                q.float().transpose(1, 2),
                k.float().transpose(1, 2),
                v.float().transpose(1, 2),
                attn_mask=causal_lower_right(q_len, kv_len) if causal else None,
                enable_gqa=True,
            ).transpose(1, 2)
            o = torch.nan_to_num(o, nan=0.0)  # rows that see no key: upstream kernel writes 0
            out[f"{tag}_o_{int(causal)}"] = bits16(o.bfloat16())
    np.savez_compressed(os.path.join(HERE, "attn.npz"), **out)
    print("wrote quant.npz mm.npz attn.npz")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/gn-kernels")
    main(sys.argv[1])

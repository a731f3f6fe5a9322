"""Matmul oracle (CPU torch / numpy).  Test infrastructure only, never imported by the package.

"Dequantise, then matmul in fp32" restatements of the upstream entry points:

* scaled_mm_ref                         benchmark_mm.py:23-27
* triton_mm epilogue order              gn_kernels/triton_mm.py:110-125, dtype rule :155-161
* MXFP8 / NVFP4 A[M,K] x B[N,K]^T       gn_kernels/cutedsl/sm100/sm100_mm_mxfp8.py:380-383,
                                        gn_kernels/cutedsl/sm100/sm100_mm_nvfp4.py:383-386
* per-tensor NVFP4 alpha                gn_kernels/cutedsl/sm120/sm120_gated_gemm_nvfp4.py:317-319
* FP8 1x128 / 128x128 block scaling     gn_kernels/cutedsl/sm120/sm120_mm_fp8_1d2d.py:166-224
* SwiGLU-gated dual NVFP4 GEMM          gn_kernels/cutedsl/sm120/sm120_gated_gemm_nvfp4.py:317-319,398-404,513-555
* bf16 mm                               gn_kernels/cutedsl/sm100/sm100_mm_bf16.py:252-255

Convention everywhere: A is [M, K] K-contiguous; "Bt" is the [N, K] K-contiguous buffer
whose transpose is the logical [K, N] right operand.
"""

from __future__ import annotations

import numpy as np
import torch

from . import quant


def _t(a) -> torch.Tensor:
    if isinstance(a, np.ndarray):
        return torch.from_numpy(np.ascontiguousarray(a))
    return a.detach().cpu()


def int8_mm_exact(A_i8, Bt_i8) -> torch.Tensor:
    """INT8 x INT8 -> INT32, exact (what torch._int_mm returns; benchmark_mm.py:77).

    fp64 products and sums of int8 values are exact far beyond any K used here."""
    A = _t(A_i8).double()
    Bt = _t(Bt_i8).double()
    return (A @ Bt.T).to(torch.int32)


def row_scaled_epilogue(acc: torch.Tensor, scale_A=None, scale_B=None, bias=None, out_dtype=torch.bfloat16):
    """fp32(acc) * scale_A[m], then * scale_B[n], then + bias[n], one final rounding
    (triton_mm.py:110-125)."""
    out = acc.float() if (scale_A is not None or scale_B is not None or bias is not None) else acc
    if scale_A is not None:
        out = out * _t(scale_A).float().reshape(-1, 1)
    if scale_B is not None:
        out = out * _t(scale_B).float().reshape(1, -1)
    if bias is not None:
        out = out + _t(bias).float().reshape(1, -1)
    return out.to(out_dtype)


def mm_i8_row_scaled(A_i8, Bt_i8, scale_A=None, scale_B=None, bias=None):
    acc = int8_mm_exact(A_i8, Bt_i8)
    if scale_A is None and scale_B is None and bias is None:
        return acc
    return row_scaled_epilogue(acc, scale_A, scale_B, bias)


def mm_f8_row_scaled(A_e4m3_codes, Bt_e4m3_codes, scale_A=None, scale_B=None, bias=None):
    """E4M3 operands (uint8 encodings), fp32 accumulate, same epilogue."""
    A = torch.from_numpy(quant.e4m3_to_f32(np.asarray(A_e4m3_codes)))
    Bt = torch.from_numpy(quant.e4m3_to_f32(np.asarray(Bt_e4m3_codes)))
    acc = A @ Bt.T
    return row_scaled_epilogue(acc, scale_A, scale_B, bias)


def scaled_mm_ref(A_f32, B_f32_kn, scale_A, scale_B):
    """benchmark_mm.py:23-27: scales broadcast by repetition along both dims (covers
    row-scaled and 2-D block-scaled), operands scaled in fp32 BEFORE the matmul."""
    A = _t(A_f32).float()
    B = _t(B_f32_kn).float()
    sA = _t(scale_A).float()
    sB = _t(scale_B).float()
    for d in (0, 1):
        sA = sA.repeat_interleave(A.shape[d] // sA.shape[d], d)
        sB = sB.repeat_interleave(B.shape[d] // sB.shape[d], d)
    return ((A * sA) @ (B * sB)).bfloat16()


def mm_bf16(A, Bt):
    return (_t(A).float() @ _t(Bt).float().T).bfloat16()


def mm_mxfp8(A_codes, Bt_codes, sfa_u8, sfb_u8):
    """A, Bt: uint8 E4M3 [M,K], [N,K]; sfa/sfb: uint8 E8M0 [M,K/32], [N,K/32] (row-major,
    NOT swizzled).  Returns bf16 [M,N]."""
    A = torch.from_numpy(quant.dequantize_mx(np.asarray(A_codes), np.asarray(sfa_u8), "e4m3"))
    Bt = torch.from_numpy(quant.dequantize_mx(np.asarray(Bt_codes), np.asarray(sfb_u8), "e4m3"))
    return (A @ Bt.T).bfloat16()


def mm_nvfp4(A_packed, Bt_packed, sfa_codes, sfb_codes, alpha: float = 1.0):
    """A, Bt: uint8 packed E2M1 [M,K/2], [N,K/2]; sfa/sfb: uint8 E4M3 [M,K/16], [N,K/16]
    row-major; alpha = tensor_scale_A * tensor_scale_B applied to the fp32 accumulator."""
    A = torch.from_numpy(quant.dequantize_nvfp4(np.asarray(A_packed), np.asarray(sfa_codes), 1.0))
    Bt = torch.from_numpy(quant.dequantize_nvfp4(np.asarray(Bt_packed), np.asarray(sfb_codes), 1.0))
    return ((A @ Bt.T) * np.float32(alpha)).bfloat16()


def gated_mm_nvfp4(X_packed, sfx_codes, ts_x, W1_packed, sfw1_codes, ts_w1, W3_packed, sfw3_codes, ts_w3):
    """SwiGLU-gated dual NVFP4 GEMM, gn_kernels/cutedsl/sm120/sm120_gated_gemm_nvfp4.py:513-555 with
    the epilogue arithmetic of :317-319 and :398-404, in fp32:
        o1 = (X W1^T) * (ts_w1 * ts_x);  o3 = (X W3^T) * (ts_w3 * ts_x);  out = bf16((o1 * o3) * sigmoid(o1))
    (tests/test_sm120_gated_gemm_nvfp4.py:43-44 states the same as silu(mm1) * mm3).  Packed operands
    and row-major E4M3 block scales as in mm_nvfp4."""
    X = torch.from_numpy(quant.dequantize_nvfp4(np.asarray(X_packed), np.asarray(sfx_codes), 1.0))
    W1 = torch.from_numpy(quant.dequantize_nvfp4(np.asarray(W1_packed), np.asarray(sfw1_codes), 1.0))
    W3 = torch.from_numpy(quant.dequantize_nvfp4(np.asarray(W3_packed), np.asarray(sfw3_codes), 1.0))
    a1 = np.float32(ts_w1) * np.float32(ts_x)
    a3 = np.float32(ts_w3) * np.float32(ts_x)
    o1 = (X @ W1.T) * a1
    o3 = (X @ W3.T) * a3
    return ((o1 * o3) * torch.sigmoid(o1)).bfloat16()


def mm_f8_block128(A_codes, sfa, Bt_codes, sfb, bias=None, add=None):
    """DeepSeek-style scaling: sfa fp32 [M, K/128] (one per row per 128 K), sfb fp32
    [N/128, K/128].  C = sum_kb (A_kb @ Bt_kb^T) * (sfa[:,kb] * sfb[nb,kb]) (+add) (+bias)."""
    A = torch.from_numpy(quant.e4m3_to_f32(np.asarray(A_codes)))
    Bt = torch.from_numpy(quant.e4m3_to_f32(np.asarray(Bt_codes)))
    sfa = _t(sfa).float()
    sfb = _t(sfb).float()
    M, K = A.shape
    N = Bt.shape[0]
    out = torch.zeros(M, N)
    sfb_full = sfb.repeat_interleave(128, 0)[:N]  # [N, K/128]
    for kb in range(K // 128):
        p = A[:, kb * 128 : (kb + 1) * 128] @ Bt[:, kb * 128 : (kb + 1) * 128].T
        out += p * (sfa[:, kb : kb + 1] * sfb_full[:, kb].reshape(1, -1))
    if add is not None:
        out = out + _t(add).float()
    if bias is not None:
        out = out + _t(bias).float().reshape(1, -1)
    return out.bfloat16()


def max_rel_err(out, ref) -> float:
    """max |out - ref| / max |ref|: the relative-error figure the parity tests bound by 1e-2."""
    out = _t(out).double()
    ref = _t(ref).double()
    return float((out - ref).abs().max() / ref.abs().max().clamp_min(1e-30))

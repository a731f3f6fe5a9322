"""torch custom ops (namespace `gnk::`) over the C ABI of libgnk.so.

Each op allocates its outputs with torch (so the caching allocator and stream semantics
hold), passes raw device pointers and the current CUDA stream to the library, and raises
on a non-zero status.  Fake (meta) implementations give shapes and dtypes for tracing.
Tensors must live on a CUDA device; there is no CPU path.
"""

from __future__ import annotations

import ctypes

import torch
from torch import Tensor

from . import _lib
from ._lib import check, lib

_DT = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}
_QK = {
    torch.int8: _lib.Q_INT8,
    torch.float8_e4m3fn: _lib.Q_E4M3,
    torch.float8_e5m2: _lib.Q_E5M2,
    torch.float4_e2m1fn_x2: _lib.Q_E2M1,
}
_QK_INV = {v: k for k, v in _QK.items()}


def _p(t: Tensor | None):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream(t: Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _need_cuda(*ts: Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("gn_kernels_b200 ops need CUDA tensors (there is no CPU implementation)")


def _ceil(a: int, b: int) -> int:
    return -(-a // b) * b


# ------------------------------------------------------------------ quantizers
@torch.library.custom_op("gnk::absmax", mutates_args=())
def absmax(x: Tensor, divisor: float = 1.0) -> Tensor:
    """max |x| / divisor (correctly rounded fp32 division) as a 0-dim tensor."""
    _need_cuda(x)
    x = x.contiguous()
    out = torch.empty((), dtype=torch.float32, device=x.device)
    scratch = torch.zeros(lib().gnk_absmax_scratch_bytes(x.numel()) // 4, dtype=torch.int32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib().gnk_absmax(_p(x), _DT[x.dtype], x.numel(), divisor, _p(out), _p(scratch), _stream(x)), "gnk_absmax")
    return out


@absmax.register_fake
def _(x, divisor=1.0):
    return x.new_empty((), dtype=torch.float32)


@torch.library.custom_op("gnk::quant_rowwise", mutates_args=())
def quant_rowwise(x: Tensor, qkind: int, perm_h: int, perm_l: int) -> tuple[Tensor, Tensor]:
    """x [..., cols] -> (codes [..., cols] int8/e4m3, scale fp32 [rows] in (optionally permuted) row order)."""
    _need_cuda(x)
    cols = x.shape[-1]
    x2 = x.reshape(-1, cols)
    if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16 != 0:
        x2 = x2.contiguous()
    rows = x2.shape[0]
    q = torch.empty(x.shape, dtype=_QK_INV[qkind], device=x.device)
    s = torch.empty(rows, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(
            lib().gnk_quant_rowwise(_p(x2), _DT[x.dtype], rows, cols, x2.stride(0), qkind, _p(q), _p(s), perm_h, perm_l, _stream(x)),
            "gnk_quant_rowwise",
        )
    return q, s


@quant_rowwise.register_fake
def _(x, qkind, perm_h, perm_l):
    return x.new_empty(x.shape, dtype=_QK_INV[qkind]), x.new_empty(x.numel() // x.shape[-1], dtype=torch.float32)


@torch.library.custom_op("gnk::quant_mx", mutates_args=())
def quant_mx(x: Tensor, qkind: int, rule: int, swizzled: bool) -> tuple[Tensor, Tensor]:
    _need_cuda(x)
    K = x.shape[-1]
    x2 = x.reshape(-1, K)
    if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16 != 0:
        x2 = x2.contiguous()
    M = x2.shape[0]
    qcols = K // 2 if qkind == _lib.Q_E2M1 else K
    q = torch.empty((*x.shape[:-1], qcols), dtype=_QK_INV[qkind], device=x.device)
    if swizzled:
        sf = torch.empty((_ceil(M, 128), _ceil(K // 32, 4)), dtype=torch.float8_e8m0fnu, device=x.device)
    else:
        sf = torch.empty((*x.shape[:-1], K // 32), dtype=torch.float8_e8m0fnu, device=x.device)
    with torch.cuda.device(x.device):
        check(
            lib().gnk_quant_mx(_p(x2), _DT[x.dtype], M, K, x2.stride(0), qkind, rule, _p(q), _p(sf), int(swizzled), _stream(x)),
            "gnk_quant_mx",
        )
    return q, sf


@quant_mx.register_fake
def _(x, qkind, rule, swizzled):
    K = x.shape[-1]
    M = x.numel() // K
    qcols = K // 2 if qkind == _lib.Q_E2M1 else K
    q = x.new_empty((*x.shape[:-1], qcols), dtype=_QK_INV[qkind])
    shape = (_ceil(M, 128), _ceil(K // 32, 4)) if swizzled else (*x.shape[:-1], K // 32)
    return q, x.new_empty(shape, dtype=torch.float8_e8m0fnu)


@torch.library.custom_op("gnk::quant_nvfp4", mutates_args=())
def quant_nvfp4(x: Tensor, tensor_scale: Tensor, eps: float, swizzled: bool) -> tuple[Tensor, Tensor]:
    _need_cuda(x, tensor_scale)
    M, K = x.shape
    if x.stride(-1) != 1 or (x.stride(0) * x.element_size()) % 16 != 0:
        x = x.contiguous()
    ts = tensor_scale.to(torch.float32).reshape(1).contiguous()
    q = torch.empty((M, K // 2), dtype=torch.float4_e2m1fn_x2, device=x.device)
    shape = (_ceil(M, 128), _ceil(K // 16, 4)) if swizzled else (M, K // 16)
    sf = torch.empty(shape, dtype=torch.float8_e4m3fn, device=x.device)
    with torch.cuda.device(x.device):
        check(
            lib().gnk_quant_nvfp4(_p(x), _DT[x.dtype], M, K, x.stride(0), _p(ts), eps, _p(q), _p(sf), int(swizzled), _stream(x)),
            "gnk_quant_nvfp4",
        )
    return q, sf


@quant_nvfp4.register_fake
def _(x, tensor_scale, eps, swizzled):
    M, K = x.shape
    shape = (_ceil(M, 128), _ceil(K // 16, 4)) if swizzled else (M, K // 16)
    return x.new_empty((M, K // 2), dtype=torch.float4_e2m1fn_x2), x.new_empty(shape, dtype=torch.float8_e4m3fn)


@torch.library.custom_op("gnk::sf_swizzle", mutates_args=())
def sf_swizzle(sf: Tensor, to_swizzled: bool) -> Tensor:
    _need_cuda(sf)
    M, Ks = sf.shape
    sf = sf.contiguous()
    out = torch.empty((_ceil(M, 128), _ceil(Ks, 4)), dtype=sf.dtype, device=sf.device)
    with torch.cuda.device(sf.device):
        check(lib().gnk_sf_swizzle(_p(sf), _p(out), M, Ks, int(to_swizzled), _stream(sf)), "gnk_sf_swizzle")
    return out


@sf_swizzle.register_fake
def _(sf, to_swizzled):
    M, Ks = sf.shape
    return sf.new_empty((_ceil(M, 128), _ceil(Ks, 4)))


@torch.library.custom_op("gnk::dequant_block", mutates_args=())
def dequant_block(q: Tensor, sf: Tensor, block: int, tensor_scale: Tensor | None) -> Tensor:
    _need_cuda(q, sf)
    qkind = _QK[q.dtype]
    K = q.shape[-1] * (2 if qkind == _lib.Q_E2M1 else 1)
    M = q.numel() // q.shape[-1]
    q = q.contiguous()
    sf = sf.contiguous()
    out = torch.empty((*q.shape[:-1], K), dtype=torch.float32, device=q.device)
    ts = tensor_scale.to(torch.float32).reshape(1).contiguous() if tensor_scale is not None else None
    with torch.cuda.device(q.device):
        check(lib().gnk_dequant_block(_p(q), _p(sf), M, K, qkind, block, _p(ts), _p(out), _stream(q)), "gnk_dequant_block")
    return out


@dequant_block.register_fake
def _(q, sf, block, tensor_scale):
    K = q.shape[-1] * (2 if q.dtype == torch.float4_e2m1fn_x2 else 1)
    return q.new_empty((*q.shape[:-1], K), dtype=torch.float32)


# ------------------------------------------------------------------ matmuls
def _k_major(t: Tensor, k_pad: int = 0) -> Tensor:
    """Returns t ([rows, K]) with K contiguous, a 16-byte aligned base and row pitch, and
    `k_pad` extra zero columns (a device copy is made only when one of these does not hold)."""
    ok = t.stride(-1) == 1 and (t.stride(0) * t.element_size()) % 16 == 0 and t.data_ptr() % 16 == 0
    if ok and k_pad == 0:
        return t
    if k_pad == 0:
        return t.contiguous()
    rows, K = t.shape
    buf = torch.zeros((rows, K + k_pad), dtype=torch.uint8, device=t.device).view(t.dtype) if t.element_size() == 1 else torch.zeros(
        (rows, K + k_pad), dtype=t.dtype, device=t.device
    )
    buf[:, :K].copy_(t)
    return buf


def _prep_ab(A: Tensor, Bt: Tensor, k_multiple: int) -> tuple[Tensor, Tensor, int]:
    """K-major operands whose K is a multiple of `k_multiple` elements (zero padding adds nothing to the product)."""
    K = A.shape[1]
    pad = (-K) % k_multiple
    return _k_major(A, pad), _k_major(Bt, pad), K + pad


@torch.library.custom_op("gnk::mm_bf16", mutates_args=())
def mm_bf16(A: Tensor, Bt: Tensor) -> Tensor:
    _need_cuda(A, Bt)
    M, K = A.shape
    N = Bt.shape[0]
    A, Bt, K = _prep_ab(A, Bt, 8)
    C = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    with torch.cuda.device(A.device):
        check(lib().gnk_mm_bf16(_p(A), A.stride(0), _p(Bt), Bt.stride(0), _p(C), N, M, N, K, _stream(A)), "gnk_mm_bf16")
    return C


@mm_bf16.register_fake
def _(A, Bt):
    return A.new_empty((A.shape[0], Bt.shape[0]), dtype=torch.bfloat16)


@torch.library.custom_op("gnk::mm_f16", mutates_args=())
def mm_f16(A: Tensor, Bt: Tensor, acc_f16: bool) -> Tensor:
    _need_cuda(A, Bt)
    M, K = A.shape
    N = Bt.shape[0]
    A, Bt, K = _prep_ab(A, Bt, 8)
    C = torch.empty((M, N), dtype=torch.float16, device=A.device)
    with torch.cuda.device(A.device):
        check(lib().gnk_mm_f16(_p(A), A.stride(0), _p(Bt), Bt.stride(0), _p(C), N, M, N, K, int(acc_f16), _stream(A)), "gnk_mm_f16")
    return C


@mm_f16.register_fake
def _(A, Bt, acc_f16):
    return A.new_empty((A.shape[0], Bt.shape[0]), dtype=torch.float16)


@torch.library.custom_op("gnk::mm_i8", mutates_args=())
def mm_i8(A: Tensor, Bt: Tensor, scale_A: Tensor | None, scale_B: Tensor | None, bias: Tensor | None, out_i32: bool) -> Tensor:
    _need_cuda(A, Bt)
    M, K = A.shape
    N = Bt.shape[0]
    A, Bt, K = _prep_ab(A, Bt, 16)
    C = torch.empty((M, N), dtype=torch.int32 if out_i32 else torch.bfloat16, device=A.device)
    f = lambda t: t.to(torch.float32).contiguous() if t is not None else None  # noqa: E731
    sa, sb, bi = f(scale_A), f(scale_B), f(bias)
    with torch.cuda.device(A.device):
        check(
            lib().gnk_mm_i8(_p(A), A.stride(0), _p(Bt), Bt.stride(0), _p(C), N, M, N, K, _p(sa), _p(sb), _p(bi),
                            _lib.OUT_I32 if out_i32 else _lib.OUT_BF16, _stream(A)),
            "gnk_mm_i8",
        )
    return C


@mm_i8.register_fake
def _(A, Bt, scale_A, scale_B, bias, out_i32):
    return A.new_empty((A.shape[0], Bt.shape[0]), dtype=torch.int32 if out_i32 else torch.bfloat16)


@torch.library.custom_op("gnk::mm_f8", mutates_args=())
def mm_f8(A: Tensor, Bt: Tensor, scale_A: Tensor | None, scale_B: Tensor | None, bias: Tensor | None) -> Tensor:
    _need_cuda(A, Bt)
    M, K = A.shape
    N = Bt.shape[0]
    A, Bt, K = _prep_ab(A, Bt, 16)
    C = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    f = lambda t: t.to(torch.float32).contiguous() if t is not None else None  # noqa: E731
    sa, sb, bi = f(scale_A), f(scale_B), f(bias)
    with torch.cuda.device(A.device):
        check(
            lib().gnk_mm_f8(_p(A), A.stride(0), _p(Bt), Bt.stride(0), _p(C), N, M, N, K, _p(sa), _p(sb), _p(bi), _stream(A)),
            "gnk_mm_f8",
        )
    return C


@mm_f8.register_fake
def _(A, Bt, scale_A, scale_B, bias):
    return A.new_empty((A.shape[0], Bt.shape[0]), dtype=torch.bfloat16)


@torch.library.custom_op("gnk::mm_mxfp8", mutates_args=())
def mm_mxfp8(A: Tensor, Bt: Tensor, SFA: Tensor, SFB: Tensor) -> Tensor:
    _need_cuda(A, Bt, SFA, SFB)
    M, K = A.shape
    N = Bt.shape[0]
    A, Bt = _k_major(A), _k_major(Bt)
    SFA, SFB = SFA.contiguous(), SFB.contiguous()
    need_a = _ceil(M, 128) * _ceil(K // 32, 4)
    need_b = _ceil(N, 128) * _ceil(K // 32, 4)
    if SFA.numel() < need_a or SFB.numel() < need_b:
        raise ValueError(f"swizzled scale buffers too small: need {need_a} / {need_b} bytes, got {SFA.numel()} / {SFB.numel()}")
    C = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    with torch.cuda.device(A.device):
        check(
            lib().gnk_mm_mxfp8(_p(A), A.stride(0), _p(Bt), Bt.stride(0), _p(SFA), _p(SFB), _p(C), N, M, N, K, _stream(A)),
            "gnk_mm_mxfp8",
        )
    return C


@mm_mxfp8.register_fake
def _(A, Bt, SFA, SFB):
    return A.new_empty((A.shape[0], Bt.shape[0]), dtype=torch.bfloat16)


@torch.library.custom_op("gnk::mm_nvfp4", mutates_args=())
def mm_nvfp4(A: Tensor, Bt: Tensor, SFA: Tensor, SFB: Tensor, alpha: float) -> Tensor:
    _need_cuda(A, Bt, SFA, SFB)
    M, Kh = A.shape
    K = Kh * 2
    N = Bt.shape[0]
    A, Bt = _k_major(A), _k_major(Bt)
    SFA, SFB = SFA.contiguous(), SFB.contiguous()
    need_a = _ceil(M, 128) * _ceil(K // 16, 4)
    need_b = _ceil(N, 128) * _ceil(K // 16, 4)
    if SFA.numel() < need_a or SFB.numel() < need_b:
        raise ValueError(f"swizzled scale buffers too small: need {need_a} / {need_b} bytes, got {SFA.numel()} / {SFB.numel()}")
    C = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    with torch.cuda.device(A.device):
        check(
            lib().gnk_mm_nvfp4(_p(A), A.stride(0), _p(Bt), Bt.stride(0), _p(SFA), _p(SFB), float(alpha), _p(C), N, M, N, K, _stream(A)),
            "gnk_mm_nvfp4",
        )
    return C


@mm_nvfp4.register_fake
def _(A, Bt, SFA, SFB, alpha):
    return A.new_empty((A.shape[0], Bt.shape[0]), dtype=torch.bfloat16)


def _gated_common(X, SFX, W1, SFW1, W3, SFW3):
    _need_cuda(X, SFX, W1, SFW1, W3, SFW3)
    M, Kh = X.shape
    K = Kh * 2
    N = W1.shape[0]
    if N % 128 != 0 or K % 32 != 0:
        raise ValueError(f"gated NVFP4 GEMM needs N % 128 == 0 and K % 32 == 0 (got N={N}, K={K})")
    X, W1, W3 = _k_major(X), _k_major(W1), _k_major(W3)
    SFX, SFW1, SFW3 = SFX.contiguous(), SFW1.contiguous(), SFW3.contiguous()
    need_x = _ceil(M, 128) * _ceil(K // 16, 4)
    need_w = _ceil(N, 128) * _ceil(K // 16, 4)
    if SFX.numel() < need_x or SFW1.numel() < need_w or SFW3.numel() < need_w:
        raise ValueError(f"swizzled scale buffers too small: need {need_x} / {need_w} bytes")
    return X, SFX, W1, SFW1, W3, SFW3, M, N, K


@torch.library.custom_op("gnk::gated_mm_nvfp4", mutates_args=())
def gated_mm_nvfp4(X: Tensor, SFX: Tensor, ts_x: Tensor, W1: Tensor, SFW1: Tensor, ts_w1: Tensor, W3: Tensor, SFW3: Tensor,
                   ts_w3: Tensor) -> Tensor:
    X, SFX, W1, SFW1, W3, SFW3, M, N, K = _gated_common(X, SFX, W1, SFW1, W3, SFW3)
    C = torch.empty((M, N), dtype=torch.bfloat16, device=X.device)
    with torch.cuda.device(X.device):
        check(
            lib().gnk_gated_mm_nvfp4(_p(X), X.stride(0), _p(SFX), _p(ts_x), _p(W1), _p(SFW1), _p(ts_w1), _p(W3), _p(SFW3), _p(ts_w3),
                                     W1.stride(0), None, _p(C), N, None, M, N, K, _stream(X)),
            "gnk_gated_mm_nvfp4",
        )
    return C


@gated_mm_nvfp4.register_fake
def _(X, SFX, ts_x, W1, SFW1, ts_w1, W3, SFW3, ts_w3):
    return X.new_empty((X.shape[0], W1.shape[0]), dtype=torch.bfloat16)


@torch.library.custom_op("gnk::gated_mm_nvfp4_quant", mutates_args=())
def gated_mm_nvfp4_quant(X: Tensor, SFX: Tensor, ts_x: Tensor, W1: Tensor, SFW1: Tensor, ts_w1: Tensor, W3: Tensor, SFW3: Tensor,
                         ts_w3: Tensor, ts_out: Tensor) -> tuple[Tensor, Tensor]:
    X, SFX, W1, SFW1, W3, SFW3, M, N, K = _gated_common(X, SFX, W1, SFW1, W3, SFW3)
    C = torch.empty((M, N // 2), dtype=torch.uint8, device=X.device)
    SFC = torch.zeros((_ceil(M, 128), _ceil(N // 16, 4)), dtype=torch.uint8, device=X.device)  # padding rows stay 0
    with torch.cuda.device(X.device):
        check(
            lib().gnk_gated_mm_nvfp4(_p(X), X.stride(0), _p(SFX), _p(ts_x), _p(W1), _p(SFW1), _p(ts_w1), _p(W3), _p(SFW3), _p(ts_w3),
                                     W1.stride(0), _p(ts_out), _p(C), N // 2, _p(SFC), M, N, K, _stream(X)),
            "gnk_gated_mm_nvfp4",
        )
    return C, SFC


@gated_mm_nvfp4_quant.register_fake
def _(X, SFX, ts_x, W1, SFW1, ts_w1, W3, SFW3, ts_w3, ts_out):
    M, N = X.shape[0], W1.shape[0]
    return X.new_empty((M, N // 2), dtype=torch.uint8), X.new_empty((_ceil(M, 128), _ceil(N // 16, 4)), dtype=torch.uint8)


# ------------------------------------------------------------------ attention
def _blhd_ok(t: Tensor) -> bool:
    es = t.element_size()
    return t.stride(-1) == 1 and all((t.stride(i) * es) % 16 == 0 for i in range(3)) and t.data_ptr() % 16 == 0


_ATTN_QK = {torch.int8: _lib.Q_INT8, torch.float8_e4m3fn: _lib.Q_E4M3, torch.bfloat16: _lib.Q_BF16, torch.float16: _lib.Q_F16}


@torch.library.custom_op("gnk::attn_fwd", mutates_args=())
def attn_fwd(q: Tensor, k: Tensor, v: Tensor, scale_q: Tensor | None, scale_k: Tensor | None, causal: bool, acc16: int = 0) -> Tensor:
    """q [B,Lq,Hq,D], k [B,Lk,Hkv,D]: int8 / float8_e4m3fn codes (optionally with fp32 scales [B,H,L]) or
    bf16 / fp16; v [B,Lk,Hkv,D] bf16 or fp16 (the type of the output).  acc16: bit 0 = fp16 Q K^T
    accumulation, bit 1 = fp16 P V accumulation (fp16 operands only)."""
    _need_cuda(q, k, v)
    B, Lq, Hq, D = q.shape
    _, Lk, Hkv, _ = k.shape
    if q.dtype not in _ATTN_QK or k.dtype != q.dtype:
        raise NotImplementedError(f"attention needs int8, float8_e4m3fn, bfloat16 or float16 Q and K of one type (got {q.dtype}, {k.dtype})")
    if v.dtype not in (torch.bfloat16, torch.float16):
        raise NotImplementedError("attention needs bf16 or fp16 V")
    if q.dtype in (torch.bfloat16, torch.float16) and v.dtype != q.dtype:
        raise NotImplementedError("16-bit Q and K need V of the same type")
    q = q if _blhd_ok(q) else q.contiguous()
    k = k if _blhd_ok(k) else k.contiguous()
    v = v if _blhd_ok(v) else v.contiguous()
    sq = scale_q.to(torch.float32).contiguous() if scale_q is not None else None
    sk = scale_k.to(torch.float32).contiguous() if scale_k is not None else None
    o = torch.empty((B, Lq, Hq, D), dtype=v.dtype, device=q.device)
    I3 = ctypes.c_int64 * 3
    strides = [I3(*t.stride()[:3]) for t in (q, k, v, o)]
    with torch.cuda.device(q.device):
        check(
            lib().gnk_attn_fwd(_p(q), _p(k), _p(v), _p(o), _p(sq), _p(sk), _ATTN_QK[q.dtype], _DT[v.dtype], acc16, B, Lq, Lk, Hq, Hkv, D,
                               strides[0], strides[1], strides[2], strides[3], int(causal), _stream(q)),
            "gnk_attn_fwd",
        )
    return o


@attn_fwd.register_fake
def _(q, k, v, scale_q, scale_k, causal, acc16=0):
    B, Lq, Hq, D = q.shape
    return q.new_empty((B, Lq, Hq, D), dtype=v.dtype)


def _lhd_ok(t: Tensor) -> bool:
    es = t.element_size()
    return t.stride(-1) == 1 and all((t.stride(i) * es) % 16 == 0 for i in range(2)) and t.data_ptr() % 16 == 0


@torch.library.custom_op("gnk::attn_varlen_fwd", mutates_args=())
def attn_varlen_fwd(q: Tensor, k: Tensor, v: Tensor, q_offsets: Tensor, kv_offsets: Tensor, max_q_len: int, causal: bool, acc16: int = 0) -> Tensor:
    """Packed sequences: q [Lq_total,Hq,D], k / v [Lk_total,Hkv,D], all bf16 or all fp16; offsets int32 [B+1]."""
    _need_cuda(q, k, v, q_offsets, kv_offsets)
    Lq_total, Hq, D = q.shape
    Lk_total, Hkv, _ = k.shape
    if q.dtype not in (torch.bfloat16, torch.float16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise NotImplementedError(f"packed attention needs bf16 or fp16 q, k, v of one type (got {q.dtype}, {k.dtype}, {v.dtype})")
    q = q if _lhd_ok(q) else q.contiguous()
    k = k if _lhd_ok(k) else k.contiguous()
    v = v if _lhd_ok(v) else v.contiguous()
    qo = q_offsets.to(torch.int32).contiguous()
    ko = kv_offsets.to(torch.int32).contiguous()
    B = qo.numel() - 1
    o = torch.empty((Lq_total, Hq, D), dtype=v.dtype, device=q.device)
    I2 = ctypes.c_int64 * 2
    strides = [I2(*t.stride()[:2]) for t in (q, k, v, o)]
    with torch.cuda.device(q.device):
        check(
            lib().gnk_attn_varlen_fwd(_p(q), _p(k), _p(v), _p(o), _p(qo), _p(ko), _ATTN_QK[q.dtype], acc16, B, max_q_len, Lq_total, Lk_total,
                                      Hq, Hkv, D, strides[0], strides[1], strides[2], strides[3], int(causal), _stream(q)),
            "gnk_attn_varlen_fwd",
        )
    return o


@attn_varlen_fwd.register_fake
def _(q, k, v, q_offsets, kv_offsets, max_q_len, causal, acc16=0):
    return q.new_empty(q.shape, dtype=v.dtype)


@torch.library.custom_op("gnk::mm_f8_block128", mutates_args=())
def mm_f8_block128(A: Tensor, SFA: Tensor, Bt: Tensor, SFB: Tensor, bias: Tensor | None, add: Tensor | None) -> Tensor:
    _need_cuda(A, Bt, SFA, SFB)
    M, K = A.shape
    N = Bt.shape[0]
    A, Bt = _k_major(A), _k_major(Bt)
    # SFA M-major: element (m, kb) at kb * ld + m
    sfa = SFA.to(torch.float32)
    if not (sfa.stride(0) == 1 and sfa.stride(1) >= M):
        sfa = sfa.T.contiguous().T
    sfb = SFB.to(torch.float32).contiguous()
    bi = bias.to(torch.bfloat16).contiguous() if bias is not None else None
    ad = add.to(torch.bfloat16) if add is not None else None
    if ad is not None and ad.stride(1) != 1:
        ad = ad.contiguous()
    C = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    with torch.cuda.device(A.device):
        check(
            lib().gnk_mm_f8_block128(_p(A), A.stride(0), _p(sfa), sfa.stride(1) if sfa.shape[1] > 1 else max(M, 1), _p(Bt), Bt.stride(0), _p(sfb), sfb.stride(0),
                                     _p(bi), _p(ad), ad.stride(0) if ad is not None else 0, _p(C), N, M, N, K, _stream(A)),
            "gnk_mm_f8_block128",
        )
    return C


@mm_f8_block128.register_fake
def _(A, SFA, Bt, SFB, bias, add):
    return A.new_empty((A.shape[0], Bt.shape[0]), dtype=torch.bfloat16)

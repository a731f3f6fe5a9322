"""Quantizer oracle (numpy).  Test infrastructure only, never imported by the package.

Restates, with explicit bit arithmetic, the upstream torch reference quantizers:

* row-wise absmax quantizer       benchmark_attn.py:39-55
* E8M0 scale rules (OCP / NV)     gn_kernels/quant_utils.py:40-59
* quantize_mx / dequantize_mx     gn_kernels/quant_utils.py:93-152
* fp32 -> packed E2M1 pairs       gn_kernels/quant_utils.py:62-90
* quantize_nvfp4                  gn_kernels/quant_utils.py:156-171
* 128x4 scale-factor swizzle      gn_kernels/quant_utils.py:21-36

All inputs are float32 numpy arrays (bf16 / fp16 tensors convert exactly).  Packed
outputs are uint8 arrays holding the raw encodings.
"""

from __future__ import annotations

import numpy as np

F32 = np.float32

E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=F32)


def to_f32(x) -> np.ndarray:
    """Accept a torch tensor (any float dtype) or an array; return float32 numpy."""
    if hasattr(x, "detach"):
        x = x.detach().cpu().float().numpy()
    return np.ascontiguousarray(x, dtype=F32)


# ----------------------------------------------------------------------------------------
# scalar format conversions
# ----------------------------------------------------------------------------------------
def f32_to_e4m3(x: np.ndarray) -> np.ndarray:
    """float32 -> E4M3 (fn: no inf, max 448) encodings, round-to-nearest-even.

    Mirrors what `tensor.to(torch.float8_e4m3fn)` does for |x| <= 448, which is the only
    range the reference feeds it (every call site clips first: quant_utils.py:109,166,
    benchmark_attn.py:50).  Values above 448 saturate to 448 here.
    """
    x = np.ascontiguousarray(x, dtype=F32)
    bits = x.view(np.uint32)
    sign = ((bits >> 31) & 1).astype(np.uint8) << 7
    a = np.abs(x)
    a = np.minimum(a, F32(448.0))
    abits = a.view(np.uint32)
    # normal range of E4M3 starts at 2^-6
    # round the 23-bit mantissa to 3 bits, ties to even, by the add-and-truncate trick
    lsb = (abits >> 20) & 1
    rounded = (abits + np.uint32(0x7FFFF) + lsb) >> 20  # exponent(8) | mantissa(3)
    # rebias 127 -> 7
    normal = rounded.astype(np.int64) - ((127 - 7) << 3)
    # subnormal range: multiples of 2^-9, np.rint is ties-to-even; 8 carries into the
    # first normal encoding 0x08 on its own
    sub = np.rint(a.astype(np.float64) * 512.0).astype(np.int64)
    mag = np.where(a < F32(2.0**-6), sub, normal)
    mag = np.clip(mag, 0, 0x7E)
    out = mag.astype(np.uint8) | sign
    out = np.where(np.isnan(x), np.uint8(0x7F), out)
    return out.astype(np.uint8)


def _e4m3_table() -> np.ndarray:
    b = np.arange(256, dtype=np.int32)
    sign = np.where(b & 0x80, -1.0, 1.0)
    e = (b >> 3) & 0xF
    m = b & 0x7
    val = np.where(e == 0, m * 2.0**-9, (1.0 + m / 8.0) * np.exp2(e.astype(np.float64) - 7))
    val = np.where((b & 0x7F) == 0x7F, np.nan, val)
    return (sign * val).astype(F32)


_E4M3_LUT = _e4m3_table()


def e4m3_to_f32(b: np.ndarray) -> np.ndarray:
    """E4M3 encodings -> float32 (sign, 4-bit exponent biased by 7, 3-bit mantissa; 0x7F/0xFF are NaN)."""
    return _E4M3_LUT[np.asarray(b, dtype=np.uint8)]


def f32_to_e5m2(x: np.ndarray) -> np.ndarray:
    """float32 -> E5M2, RNE, inputs assumed clipped to +-57344."""
    x = np.ascontiguousarray(x, dtype=F32)
    bits = x.view(np.uint32)
    sign = ((bits >> 31) & 1).astype(np.uint8) << 7
    a = np.minimum(np.abs(x), F32(57344.0))
    abits = a.view(np.uint32)
    lsb = (abits >> 21) & 1
    rounded = (abits + np.uint32(0xFFFFF) + lsb) >> 21
    normal = rounded.astype(np.int64) - ((127 - 15) << 2)
    sub = np.rint(a.astype(np.float64) * 2.0**16).astype(np.int64)  # step 2^-16
    mag = np.where(a < F32(2.0**-14), sub, normal)
    mag = np.clip(mag, 0, 0x7B)
    return (mag.astype(np.uint8) | sign).astype(np.uint8)


def e5m2_to_f32(b: np.ndarray) -> np.ndarray:
    b = np.asarray(b, dtype=np.uint8)
    return (b.astype(np.uint16) << 8).view(np.float16).astype(F32)


def f32_to_e2m1(x: np.ndarray) -> np.ndarray:
    """float32 -> 4-bit E2M1 codes (sign in bit 3), one code per element.

    Thresholds are the reference's (quant_utils.py:68-77): ties go to the even mantissa,
    NaN lands on code 7, the sign bit is copied from the input even for zero.
    """
    x = np.ascontiguousarray(x, dtype=F32)
    sign = ((x.view(np.uint32) >> 31) & 1).astype(np.uint8)
    a = np.abs(x)
    code = np.full(a.shape, 7, dtype=np.uint8)
    code[a <= F32(5.0)] = 6
    code[a < F32(3.5)] = 5
    code[a <= F32(2.5)] = 4
    code[a < F32(1.75)] = 3
    code[a <= F32(1.25)] = 2
    code[a < F32(0.75)] = 1
    code[a <= F32(0.25)] = 0
    return (sign << 3) | code


def pack_e2m1_pairs(codes: np.ndarray) -> np.ndarray:
    """Pack 4-bit codes two per byte along the last axis: EVEN index -> HIGH nibble.

    This is the reference's order (quant_utils.py:80-89: byte0 = code[1] | code[0] << 4).
    """
    assert codes.shape[-1] % 2 == 0
    return ((codes[..., 0::2] << 4) | codes[..., 1::2]).astype(np.uint8)


def unpack_e2m1_pairs(packed: np.ndarray) -> np.ndarray:
    """Inverse of pack_e2m1_pairs -> float32 values, last axis doubled."""
    packed = np.asarray(packed, dtype=np.uint8)
    hi = packed >> 4
    lo = packed & 0xF
    codes = np.stack([hi, lo], axis=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    mag = E2M1_VALUES[codes & 7]
    return np.where(codes & 8, -mag, mag).astype(F32)


# ----------------------------------------------------------------------------------------
# row-wise absmax quantizer (one scale per last-dim row)
# ----------------------------------------------------------------------------------------
def quantize_rowwise(x, kind: str):
    """kind in {"int8", "e4m3"}.  Returns (codes, scale float32[...]).

    benchmark_attn.py:39-51: scale = amax/qmax (qmax 127 or 448); x / clip(scale, 1e-6);
    int8 rounds half-to-even then clips to [-128, 127]; e4m3 clips to +-448 then casts.
    Integer output is int8, E4M3 output is the uint8 encoding.
    """
    x = to_f32(x)
    amax = np.abs(x).max(axis=-1)
    qmax = F32(127.0) if kind == "int8" else F32(448.0)
    scale = (amax / qmax).astype(F32)
    y = (x / np.maximum(scale, F32(1e-6))[..., None]).astype(F32)
    if kind == "int8":
        q = np.clip(np.rint(y), -128, 127).astype(np.int8)
    elif kind == "e4m3":
        q = f32_to_e4m3(np.clip(y, F32(-448.0), F32(448.0)))
    else:
        raise ValueError(kind)
    return q, scale


def dequantize_rowwise(q, scale, kind: str) -> np.ndarray:
    """benchmark_attn.py:54-55."""
    v = q.astype(F32) if kind == "int8" else e4m3_to_f32(q)
    return (v * np.asarray(scale, dtype=F32)[..., None]).astype(F32)


# ----------------------------------------------------------------------------------------
# MX (E8M0 shared exponent per 32)
# ----------------------------------------------------------------------------------------
_MX_POW2_LOG = {"e4m3": 8, "e5m2": 15, "e2m1": 2}  # log2 of 256 / 32768 / 4
_MX_AMAX = {"e4m3": 448.0, "e5m2": 57344.0, "e2m1": 6.0}


def mx_scale_bits_ocp(amax: np.ndarray, kind: str) -> np.ndarray:
    """OCP floor rule (quant_utils.py:55-59): power-of-two floor of amax divided by the
    largest power of two of the element type, biased exponent of the fp32 result."""
    amax = np.ascontiguousarray(amax, dtype=F32)
    p2 = (amax.view(np.uint32) & np.uint32(0x7F800000)).view(F32)
    q = (p2 / F32(2.0 ** _MX_POW2_LOG[kind])).astype(F32)
    return (q.view(np.uint32) >> 23).astype(np.int32)


def mx_scale_bits_nv(amax: np.ndarray, kind: str) -> np.ndarray:
    """cuBLAS round-up rule (quant_utils.py:40-51)."""
    amax = np.ascontiguousarray(amax, dtype=F32)
    s = (amax / F32(_MX_AMAX[kind])).astype(F32)
    bits = s.view(np.uint32).astype(np.int64)
    e = bits >> 23
    m = bits & 0x7FFFFF
    bump = ((e > 0) & (e < 254) & (m > 0)) | ((e == 0) & (m > 0x400000))
    return np.where(bump, e + 1, e).astype(np.int32)


def quantize_mx(x, kind: str = "e4m3", method: str = "ocp"):
    """quant_utils.py:93-117.  Returns (codes uint8, scales uint8 [..., K/32]).

    kind "e4m3"/"e5m2": codes [..., K]; kind "e2m1": packed pairs [..., K/2].
    """
    x = to_f32(x)
    assert x.shape[-1] % 32 == 0
    blk = x.reshape(*x.shape[:-1], -1, 32)
    amax = np.abs(blk).max(axis=-1)
    ebits = (mx_scale_bits_ocp if method == "ocp" else mx_scale_bits_nv)(amax, kind)
    scales = (ebits & 0xFF).astype(np.uint8)
    denom = (ebits.astype(np.uint32) << 23).view(F32)
    denom = np.maximum(denom, F32(1e-12))
    y = (blk / denom[..., None]).astype(F32)
    lim = F32(_MX_AMAX[kind])
    y = np.clip(y, -lim, lim)
    if kind == "e4m3":
        q = f32_to_e4m3(y)
    elif kind == "e5m2":
        q = f32_to_e5m2(y)
    else:
        q = pack_e2m1_pairs(f32_to_e2m1(y).reshape(*x.shape))
        return q, scales
    return q.reshape(x.shape), scales


def dequantize_mx(q: np.ndarray, scales: np.ndarray, kind: str = "e4m3") -> np.ndarray:
    """quant_utils.py:120-124 for FP8.  For E2M1 the upstream branch (:126-152) raises on a
    shape error and unpacks nibbles in the opposite order to its own packer; the FP4 branch
    here is the inverse of pack_e2m1_pairs instead (even element = high nibble)."""
    if kind == "e4m3":
        v = e4m3_to_f32(q)
    elif kind == "e5m2":
        v = e5m2_to_f32(q)
    else:
        v = unpack_e2m1_pairs(q)
    s = (np.asarray(scales, dtype=np.uint8).astype(np.uint32) << 23).view(F32)
    out = v.reshape(*v.shape[:-1], -1, 32) * s[..., None]
    return out.reshape(v.shape).astype(F32)


# ----------------------------------------------------------------------------------------
# NVFP4 (E2M1 pairs, E4M3 scale per 16, fp32 per-tensor scale)
# ----------------------------------------------------------------------------------------
def nvfp4_tensor_scale(x) -> np.float32:
    """quant_utils.py:162: amax / (448 * 6) in float32."""
    x = to_f32(x)
    return (np.abs(x).max().astype(F32) / F32(448.0 * 6.0)).astype(F32)


def quantize_nvfp4(x, tensor_scale=None, eps: float = 1e-12):
    """quant_utils.py:156-171.  Returns (packed uint8 [M, K/2], scales uint8 E4M3 [M, K/16],
    tensor_scale float32).  All divisions are IEEE float32 divisions."""
    x = to_f32(x)
    assert x.ndim == 2 and x.shape[-1] % 16 == 0
    ts = nvfp4_tensor_scale(x) if tensor_scale is None else F32(tensor_scale)
    blk = x.reshape(x.shape[0], -1, 16)
    amax = np.abs(blk).max(axis=-1)
    d0 = np.maximum(F32(6.0) * ts, F32(1e-12)).astype(F32)
    s_f32 = (amax / d0).astype(F32)
    s_codes = f32_to_e4m3(np.clip(s_f32, F32(-448.0), F32(448.0)))
    d1 = np.maximum((ts * e4m3_to_f32(s_codes)).astype(F32), F32(eps))
    y = (blk / d1[..., None]).astype(F32)
    packed = pack_e2m1_pairs(f32_to_e2m1(y).reshape(x.shape))
    return packed, s_codes, ts


def dequantize_nvfp4(packed, s_codes, tensor_scale) -> np.ndarray:
    v = unpack_e2m1_pairs(packed)
    s = e4m3_to_f32(s_codes) * F32(tensor_scale)
    return (v.reshape(v.shape[0], -1, 16) * s[..., None]).reshape(v.shape).astype(F32)


# ----------------------------------------------------------------------------------------
# 128x4 swizzled scale-factor layout
# ----------------------------------------------------------------------------------------
def permute_nv_sf(s: np.ndarray) -> np.ndarray:
    """quant_utils.py:21-30.  [M, Ks] bytes -> zero-padded to (128, 4) multiples, then each
    (128 rows x 4 scales) block becomes one 512-byte atom whose 16-byte rows hold rows
    r, r+32, r+64, r+96.  Returned with the padded [M', Ks'] shape (a flat reinterpretation)."""
    s = np.asarray(s, dtype=np.uint8)
    M, Ks = s.shape
    Mp, Kp = -(-M // 128) * 128, -(-Ks // 4) * 4
    buf = np.zeros((Mp, Kp), dtype=np.uint8)
    buf[:M, :Ks] = s
    t = buf.reshape(Mp // 128, 4, 32, Kp // 4, 4)  # [mb, quad, r, kb, j]
    return np.ascontiguousarray(t.transpose(0, 3, 2, 1, 4)).reshape(Mp, Kp)


def unpermute_nv_sf(s: np.ndarray) -> np.ndarray:
    """quant_utils.py:33-36 (inverse of the above, padded shape kept)."""
    s = np.asarray(s, dtype=np.uint8)
    Mp, Kp = s.shape
    t = s.reshape(Mp // 128, Kp // 4, 32, 4, 4)  # [mb, kb, r, quad, j]
    return np.ascontiguousarray(t.transpose(0, 3, 2, 1, 4)).reshape(Mp, Kp)


def sf_swizzled_offset(row: int, kcol: int, Ks_padded: int) -> int:
    """Byte offset of scale (row, kcol) inside the swizzled buffer; closed form of the
    permutation above, used to test kernels that write atoms directly."""
    mb, r = divmod(row, 128)
    quad, r32 = divmod(r, 32)
    kb, j = divmod(kcol, 4)
    return ((mb * (Ks_padded // 4) + kb) * 32 + r32) * 16 + quad * 4 + j

// Quantizer kernels: per-tensor absmax, row-wise INT8/E4M3, MX (E8M0 per 32) and NVFP4
// (E4M3 per 16 + fp32 tensor scale), scale-factor swizzle, block dequantizer.
//
// All of them are one-pass, HBM-bound byte producers: 128-bit loads, block maxima in
// registers (shuffles only where a block spans lanes), 64/128-bit stores, packed f32x2 arithmetic.
// The arithmetic that makes the bytes equal the torch reference bit for bit lives in gnk_quant_math.cuh.
#include <mutex>
#include <type_traits>

#include "gnk_quant_math.cuh"

namespace gnk {
namespace {

// ------------------------------------------------------------------------------------
// per-tensor absmax: partial maxima per CTA in scratch, last CTA (ticket) folds them
// ------------------------------------------------------------------------------------
constexpr int kAbsmaxMaxCtas = 2048;
constexpr int kAbsmaxThreads = 256;

template <typename T>
__device__ __forceinline__ float absmax_partial(const T* __restrict__ x, int64_t n) {
  float m = 0.f;
  const int64_t nvec = n >> 3;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  for (; i + 3 * stride < nvec; i += 4 * stride) {  // four independent 16-byte loads in flight
    float v[4][8];
#pragma unroll
    for (int j = 0; j < 4; ++j) load8<T>(x + (i + j * stride) * 8, v[j]);
#pragma unroll
    for (int j = 0; j < 4; ++j) m = fmaxf(m, amax8(v[j]));
  }
  for (; i < nvec; i += stride) {
    float v[8];
    load8<T>(x + i * 8, v);
    m = fmaxf(m, amax8(v));
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 7)) m = fmaxf(m, fabsf(to_f32<T>(x[(nvec << 3) + threadIdx.x])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  return m;
}

// scratch[0] = ticket (zero on entry, zero again on exit), scratch[1 + cta] = partial maxima
template <typename T>
__global__ void __launch_bounds__(kAbsmaxThreads) absmax_kernel(const T* __restrict__ x, int64_t n,
                                                                float* __restrict__ out, float divisor,
                                                                unsigned int* __restrict__ scratch) {
  __shared__ float warp_max[kAbsmaxThreads / 32];
  __shared__ bool is_last;
  float m = absmax_partial<T>(x, n);
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float b = warp_max[0];
    for (int i = 1; i < kAbsmaxThreads / 32; ++i) b = fmaxf(b, warp_max[i]);
    reinterpret_cast<float*>(scratch)[1 + blockIdx.x] = b;
    __threadfence();
    is_last = atomicAdd(&scratch[0], 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  float f = 0.f;
  for (int i = threadIdx.x; i < gridDim.x; i += blockDim.x)
    f = fmaxf(f, reinterpret_cast<volatile float*>(scratch)[1 + i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) f = fmaxf(f, __shfl_xor_sync(0xffffffffu, f, o));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = f;
  __syncthreads();
  if (threadIdx.x == 0) {
    float b = warp_max[0];
    for (int i = 1; i < kAbsmaxThreads / 32; ++i) b = fmaxf(b, warp_max[i]);
    out[0] = __fdiv_rn(b, divisor);
    scratch[0] = 0u;
  }
}

// ------------------------------------------------------------------------------------
// row-wise quantizer: LPR lanes share a row; pass 1 amax, pass 2 (row now in L1/L2) encode
// ------------------------------------------------------------------------------------
template <typename T, int QKIND, int LPR>
__global__ void __launch_bounds__(256) quant_rowwise_kernel(const T* __restrict__ x, int64_t rows, int64_t cols,
                                                            int64_t ldx, uint8_t* __restrict__ q,
                                                            float* __restrict__ scale, int64_t perm_h,
                                                            int64_t perm_l) {
  const int lane = threadIdx.x & 31;
  const int sub = lane % LPR;
  const int64_t rows_per_cta = (256 / LPR);
  const float qmax = QKIND == GNK_Q_INT8 ? 127.f : 448.f;
  const bool one_shot = cols <= LPR * 8;  // the row is one 8-element group per lane: read it once
  // persistent CTAs walk over groups of rows_per_cta rows
  for (int64_t rg = blockIdx.x; rg * rows_per_cta < rows; rg += gridDim.x) {
    const int64_t row = rg * rows_per_cta + threadIdx.x / LPR;
    const bool live = row < rows;
    const T* xr = x + (live ? row : 0) * ldx;
    float first[8];
    float m = 0.f;
    if (live) {
      if (one_shot) {
        if (sub * 8 < cols) {
          load8<T>(xr + sub * 8, first);
          m = amax8(first);
        }
      } else {
        int64_t c = sub * 8;
        for (; c + 3 * LPR * 8 < cols; c += 4 * LPR * 8) {  // four independent loads in flight
          float v[4][8];
#pragma unroll
          for (int j = 0; j < 4; ++j) load8<T>(xr + c + j * LPR * 8, v[j]);
#pragma unroll
          for (int j = 0; j < 4; ++j) m = fmaxf(m, amax8(v[j]));
        }
        for (; c < cols; c += LPR * 8) {
          float v[8];
          load8<T>(xr + c, v);
          m = fmaxf(m, amax8(v));
        }
      }
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (!live) continue;

    const float s = __fdiv_rn(m, qmax);
    const float d = fmaxf(s, 1e-6f);
    const float r = __frcp_rn(d);
    const bool safe = m >= 1e-30f;  // quotients are <= qmax * (1 + eps) then; tiny rows take the slow path
    if (sub == 0) {
      int64_t idx = row;
      if (perm_h > 0) {
        const int64_t h = row % perm_h, bl = row / perm_h, l = bl % perm_l, b = bl / perm_l;
        idx = (b * perm_h + h) * perm_l + l;
      }
      scale[idx] = s;
    }
    uint8_t* qr = q + row * cols;
    auto encode = [&](float (&v)[8], int64_t c) {
      divide_exact8(v, d, r, safe);
      uint2 out;
      if constexpr (QKIND == GNK_Q_INT8) {
        uint32_t b[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float t = fminf(fmaxf(rintf(v[i]), -128.f), 127.f);
          b[i] = static_cast<uint32_t>(static_cast<int>(t)) & 0xFFu;
        }
        out.x = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
        out.y = b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24);
      } else {
        out.x = cvt_e4m3x2(v[0], v[1]) | (cvt_e4m3x2(v[2], v[3]) << 16);
        out.y = cvt_e4m3x2(v[4], v[5]) | (cvt_e4m3x2(v[6], v[7]) << 16);
      }
      *reinterpret_cast<uint2*>(qr + c) = out;
    };
    if (one_shot) {
      if (sub * 8 < cols) encode(first, sub * 8);
      continue;
    }
    int64_t c = sub * 8;
    for (; c + 3 * LPR * 8 < cols; c += 4 * LPR * 8) {  // the row is in L1/L2 now
      float v[4][8];
#pragma unroll
      for (int j = 0; j < 4; ++j) load8<T>(xr + c + j * LPR * 8, v[j]);
#pragma unroll
      for (int j = 0; j < 4; ++j) encode(v[j], c + j * LPR * 8);
    }
    for (; c < cols; c += LPR * 8) {
      float v[8];
      load8<T>(xr + c, v);
      encode(v, c);
    }
  }
}

// Row-wise quantizer for rows of up to G * 32 elements: G threads share a row and hold it in registers
// (up to four 8-element groups each, group j of thread `sub` at column (j * G + sub) * 8, so a warp's
// loads are contiguous), so x is read from memory exactly once.  G <= 32: the row maximum is folded by
// shuffles; larger G: through shared memory.
template <int QKIND>
__device__ __forceinline__ void rowwise_encode8(float (&v)[8], float d, float r, bool safe, uint8_t* dst) {
  divide_exact8(v, d, r, safe);
  uint2 out;
  if constexpr (QKIND == GNK_Q_INT8) {
    uint32_t b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float t = fminf(fmaxf(rintf(v[i]), -128.f), 127.f);
      b[i] = static_cast<uint32_t>(static_cast<int>(t)) & 0xFFu;
    }
    out.x = b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24);
    out.y = b[4] | (b[5] << 8) | (b[6] << 16) | (b[7] << 24);
  } else {
    out.x = cvt_e4m3x2(v[0], v[1]) | (cvt_e4m3x2(v[2], v[3]) << 16);
    out.y = cvt_e4m3x2(v[4], v[5]) | (cvt_e4m3x2(v[6], v[7]) << 16);
  }
  *reinterpret_cast<uint2*>(dst) = out;
}

template <typename T, int QKIND, int G>
__global__ void __launch_bounds__(256) quant_rowwise_reg_kernel(const T* __restrict__ x, int64_t rows, int64_t cols,
                                                                int64_t ldx, uint8_t* __restrict__ q,
                                                                float* __restrict__ scale, int64_t perm_h,
                                                                int64_t perm_l) {
  constexpr int kRowsPerCta = 256 / G;
  constexpr int kWarpsPerRow = G > 32 ? G / 32 : 1;
  __shared__ float warp_max[8];
  const int sub = threadIdx.x % G;
  const float qmax = QKIND == GNK_Q_INT8 ? 127.f : 448.f;
  for (int64_t rg = blockIdx.x; rg * kRowsPerCta < rows; rg += gridDim.x) {
    const int64_t row = rg * kRowsPerCta + threadIdx.x / G;
    const bool live = row < rows;
    const T* xr = x + (live ? row : 0) * ldx;
    float v[4][8];
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t c = static_cast<int64_t>(j * G + sub) * 8;
      if (live && c < cols) {
        load8<T>(xr + c, v[j]);
        m = fmaxf(m, amax8(v[j]));
      }
    }
#pragma unroll
    for (int o = (G < 32 ? G : 32) / 2; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if constexpr (G > 32) {
      __syncthreads();  // the previous row group's maxima have been read
      if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
      __syncthreads();
      const int w0 = (threadIdx.x >> 5) / kWarpsPerRow * kWarpsPerRow;
      m = warp_max[w0];
#pragma unroll
      for (int i = 1; i < kWarpsPerRow; ++i) m = fmaxf(m, warp_max[w0 + i]);
    }
    if (!live) continue;
    const float s = __fdiv_rn(m, qmax);
    const float d = fmaxf(s, 1e-6f);
    const float r = __frcp_rn(d);
    const bool safe = m >= 1e-30f;  // quotients are <= qmax * (1 + eps) then; tiny rows take the slow path
    if (sub == 0) {
      int64_t idx = row;
      if (perm_h > 0) {
        const int64_t h = row % perm_h, bl = row / perm_h, l = bl % perm_l, b = bl / perm_l;
        idx = (b * perm_h + h) * perm_l + l;
      }
      scale[idx] = s;
    }
    uint8_t* qr = q + row * cols;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t c = static_cast<int64_t>(j * G + sub) * 8;
      if (c < cols) rowwise_encode8<QKIND>(v[j], d, r, safe, qr + c);
    }
  }
}

// ------------------------------------------------------------------------------------
// MX quantizer: one thread per 32-element block
// ------------------------------------------------------------------------------------
template <typename T, int QKIND, int RULE>
__global__ void __launch_bounds__(256) quant_mx_kernel(const T* __restrict__ x, int64_t M, int64_t K, int64_t ldx,
                                                       uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                                       int swizzled, int64_t rows_out, int64_t ks_out, int ks_shift) {
  const int64_t ks = K >> 5;
  const unsigned idx = blockIdx.x * blockDim.x + threadIdx.x;  // the launcher keeps rows_out * ks_out below 2^31
  if (idx >= static_cast<unsigned>(rows_out * ks_out)) return;
  const unsigned urow = ks_shift >= 0 ? idx >> ks_shift : idx / static_cast<unsigned>(ks_out);
  const int64_t row = urow, kb = idx - urow * static_cast<unsigned>(ks_out);
  if (row >= M || kb >= ks) {  // padding of the swizzled layout
    sf[sf_offset(row, kb, ks_out, true, ks)] = 0;
    return;
  }
  const T* p = x + row * ldx + kb * 32;
  float v[4][8];
#pragma unroll
  for (int j = 0; j < 4; ++j) load8<T>(p + j * 8, v[j]);
  float m = fmaxf(fmaxf(amax8(v[0]), amax8(v[1])), fmaxf(amax8(v[2]), amax8(v[3])));

  constexpr float kPow2 = QKIND == GNK_Q_E4M3 ? 256.f : QKIND == GNK_Q_E5M2 ? 32768.f : 4.f;
  constexpr float kAmax = QKIND == GNK_Q_E4M3 ? 448.f : QKIND == GNK_Q_E5M2 ? 57344.f : 6.f;
  uint32_t ebits;
  if constexpr (RULE == GNK_MX_OCP) {
    const float p2 = __uint_as_float(__float_as_uint(m) & 0x7F800000u);
    ebits = __float_as_uint(__fdiv_rn(p2, kPow2)) >> 23;
  } else {
    const uint32_t b = __float_as_uint(__fdiv_rn(m, kAmax));
    const uint32_t e = b >> 23, man = b & 0x7FFFFFu;
    const bool bump = (e > 0 && e < 254 && man > 0) || (e == 0 && man > 0x400000u);
    ebits = bump ? e + 1 : e;
  }
  sf[sf_offset(row, kb, ks_out, swizzled != 0, ks)] = static_cast<uint8_t>(ebits);

  const float denom = __uint_as_float(ebits << 23);
  const bool clipped = !(denom >= 1e-12f);
  // 1 / 2^(e-127) is exact (a subnormal for e = 254), so the product equals the quotient
  const float recip = __uint_as_float(ebits >= 254 ? 0x00400000u : (254u - ebits) << 23);
  // The clip to +-kAmax of the reference is what the saturating conversions below do for every
  // finite value, so only the scaling is left here.
  if (clipped) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) v[j][i] = fminf(fmaxf(__fdiv_rn(v[j][i], 1e-12f), -kAmax), kAmax);
  } else {
    const uint64_t recip2 = f2_pack(recip, recip);
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < 8; i += 2) f2_unpack(f2_mul(f2_pack(v[j][i], v[j][i + 1]), recip2), v[j][i], v[j][i + 1]);
  }
  if constexpr (QKIND == GNK_Q_E2M1) {
    uint4 out = make_uint4(cvt_e2m1x8(v[0]), cvt_e2m1x8(v[1]), cvt_e2m1x8(v[2]), cvt_e2m1x8(v[3]));
    *reinterpret_cast<uint4*>(q + row * (K >> 1) + kb * 16) = out;
  } else {
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if constexpr (QKIND == GNK_Q_E4M3) {
        w[2 * j] = cvt_e4m3x2(v[j][0], v[j][1]) | (cvt_e4m3x2(v[j][2], v[j][3]) << 16);
        w[2 * j + 1] = cvt_e4m3x2(v[j][4], v[j][5]) | (cvt_e4m3x2(v[j][6], v[j][7]) << 16);
      } else {
        w[2 * j] = cvt_e5m2x2(v[j][0], v[j][1]) | (cvt_e5m2x2(v[j][2], v[j][3]) << 16);
        w[2 * j + 1] = cvt_e5m2x2(v[j][4], v[j][5]) | (cvt_e5m2x2(v[j][6], v[j][7]) << 16);
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(q + row * K + kb * 32);
    dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
    dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// ------------------------------------------------------------------------------------
// NVFP4 quantizer: one thread per 16-element block
// ------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) quant_nvfp4_kernel(const T* __restrict__ x, int64_t M, int64_t K, int64_t ldx,
                                                          const float* __restrict__ tensor_scale, float eps,
                                                          uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                                          int swizzled, int64_t rows_out, int64_t ks_out, int ks_shift) {
  const int64_t ks = K >> 4;
  const unsigned idx = blockIdx.x * blockDim.x + threadIdx.x;  // the launcher keeps rows_out * ks_out below 2^31
  if (idx >= static_cast<unsigned>(rows_out * ks_out)) return;
  const unsigned urow = ks_shift >= 0 ? idx >> ks_shift : idx / static_cast<unsigned>(ks_out);
  const int64_t row = urow, kb = idx - urow * static_cast<unsigned>(ks_out);
  if (row >= M || kb >= ks) {
    sf[sf_offset(row, kb, ks_out, true, ks)] = 0;
    return;
  }
  const T* p = x + row * ldx + kb * 16;
  float v[2][8];
  load8<T>(p, v[0]);
  load8<T>(p + 8, v[1]);
  const float ts = __ldg(tensor_scale);
  const float d0 = fmaxf(__fmul_rn(6.f, ts), 1e-12f);
  const float r0 = __frcp_rn(d0);
  uint32_t code;
  const uint2 out = nvfp4_encode16(v, ts, d0, r0, eps, code);
  sf[sf_offset(row, kb, ks_out, swizzled != 0, ks)] = static_cast<uint8_t>(code);
  *reinterpret_cast<uint2*>(q + row * (K >> 1) + kb * 8) = out;
}

// ------------------------------------------------------------------------------------
// scale-factor swizzle / unswizzle, block dequantizer
// ------------------------------------------------------------------------------------
__global__ void sf_swizzle_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t M, int64_t Ks,
                                  int64_t Mp, int64_t Kp, int to_swizzled) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= Mp * Kp) return;
  const int64_t row = i / Kp, kc = i % Kp;
  const size_t sw = sf_offset(row, kc, Kp, true, Kp);
  if (to_swizzled)
    dst[sw] = (row < M && kc < Ks) ? src[row * Ks + kc] : 0;
  else
    dst[i] = src[sw];
}

__global__ void dequant_block_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sf, int64_t M,
                                     int64_t K, int qkind, int block, const float* __restrict__ tensor_scale,
                                     float* __restrict__ out) {
  const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (i >= M * K) return;
  const int64_t row = i / K, c = i % K;
  float v;
  if (qkind == GNK_Q_E2M1) {
    const uint32_t byte = q[row * (K >> 1) + (c >> 1)];
    v = e2m1_to_f32((c & 1) ? (byte & 0xF) : (byte >> 4));
  } else if (qkind == GNK_Q_E4M3) {
    v = e4m3_to_f32(q[i]);
  } else {
    v = e5m2_to_f32(q[i]);
  }
  const uint32_t s = sf[row * (K / block) + c / block];
  float sv = block == 32 ? __uint_as_float(s << 23) : e4m3_to_f32(s);
  if (tensor_scale) sv = __fmul_rn(sv, __ldg(tensor_scale));
  out[i] = __fmul_rn(v, sv);
}

// log2(n) when n is a power of two (the kernels then index with a shift instead of a division), else -1
inline int pow2_shift(int64_t n) {
  if (n <= 0 || (n & (n - 1))) return -1;
  int s = 0;
  while ((int64_t{1} << s) < n) ++s;
  return s;
}

template <typename F>
int dispatch_dtype(int dtype, F&& f) {
  switch (dtype) {
    case GNK_BF16: return f(static_cast<const __nv_bfloat16*>(nullptr));
    case GNK_F16: return f(static_cast<const __half*>(nullptr));
    case GNK_F32: return f(static_cast<const float*>(nullptr));
    default: return GNK_ERR_BAD_ARG;
  }
}

}  // namespace
}  // namespace gnk

using namespace gnk;

extern "C" size_t gnk_absmax_scratch_bytes(int64_t) { return sizeof(unsigned int) * (1 + kAbsmaxMaxCtas); }

extern "C" int gnk_absmax(const void* x, int dtype, int64_t n, float divisor, float* out, void* scratch,
                          gnk_stream_t stream) {
  if (!x || !out || !scratch || n <= 0 || !(divisor > 0.f)) return GNK_ERR_BAD_ARG;
  if (!aligned16(x)) return GNK_ERR_BAD_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int64_t want = (n / 8 + kAbsmaxThreads - 1) / kAbsmaxThreads;
  int grid = static_cast<int>(want < 1 ? 1 : (want > kAbsmaxMaxCtas ? kAbsmaxMaxCtas : want));
  int cap = num_sms() * 8;
  if (grid > cap) grid = cap;
  if (grid > kAbsmaxMaxCtas) grid = kAbsmaxMaxCtas;
  return dispatch_dtype(dtype, [&](auto* tag) -> int {
    using T = std::remove_cv_t<std::remove_pointer_t<decltype(tag)>>;
    absmax_kernel<T><<<grid, kAbsmaxThreads, 0, st>>>(static_cast<const T*>(x), n, out, divisor,
                                                       static_cast<unsigned int*>(scratch));
    GNK_LAUNCH_OK();
    return (int)GNK_OK;
  });
}

template <typename T, int QKIND>
static int launch_rowwise(const T* x, int64_t rows, int64_t cols, int64_t ldx, uint8_t* q, float* scale,
                          int64_t perm_h, int64_t perm_l, cudaStream_t st) {
  const int64_t cap8 = static_cast<int64_t>(num_sms()) * 8;  // persistent: 8 CTAs of 256 threads per SM
  if (cols <= 256 * 32) {
    // the row fits the registers of G threads (32 elements each): read x once
    const int g = cols <= 4 * 32 ? 4 : cols <= 16 * 32 ? 16 : cols <= 64 * 32 ? 64 : 256;
    const int64_t groups_r = (rows + 256 / g - 1) / (256 / g);
    const unsigned grid_r = static_cast<unsigned>(groups_r < cap8 ? groups_r : cap8);
    switch (g) {
      case 4: quant_rowwise_reg_kernel<T, QKIND, 4><<<grid_r, 256, 0, st>>>(x, rows, cols, ldx, q, scale, perm_h, perm_l); break;
      case 16: quant_rowwise_reg_kernel<T, QKIND, 16><<<grid_r, 256, 0, st>>>(x, rows, cols, ldx, q, scale, perm_h, perm_l); break;
      case 64: quant_rowwise_reg_kernel<T, QKIND, 64><<<grid_r, 256, 0, st>>>(x, rows, cols, ldx, q, scale, perm_h, perm_l); break;
      default: quant_rowwise_reg_kernel<T, QKIND, 256><<<grid_r, 256, 0, st>>>(x, rows, cols, ldx, q, scale, perm_h, perm_l); break;
    }
    GNK_LAUNCH_OK();
    return GNK_OK;
  }
  const int lpr = 32;  // longer rows: two passes, the second one from L1/L2
  const int64_t rows_per_cta = 256 / lpr;
  const int64_t groups = (rows + rows_per_cta - 1) / rows_per_cta;
  const int64_t cap = static_cast<int64_t>(num_sms()) * 8;  // persistent: 8 CTAs of 256 threads per SM
  const unsigned grid = static_cast<unsigned>(groups < cap ? groups : cap);
#define GNK_RW(L)                                                                                          \
  case L:                                                                                                  \
    quant_rowwise_kernel<T, QKIND, L><<<grid, 256, 0, st>>>(x, rows, cols, ldx, q, scale, perm_h, perm_l); \
    break;
  switch (lpr) {
    GNK_RW(32)
  }
#undef GNK_RW
  GNK_LAUNCH_OK();
  return GNK_OK;
}

extern "C" int gnk_quant_rowwise(const void* x, int dtype, int64_t rows, int64_t cols, int64_t ldx, int qkind,
                                 void* q, float* scale, int64_t perm_h, int64_t perm_l, gnk_stream_t stream) {
  if (!x || !q || !scale || rows <= 0 || cols <= 0) return GNK_ERR_BAD_ARG;
  if (qkind != GNK_Q_INT8 && qkind != GNK_Q_E4M3) return GNK_ERR_BAD_ARG;
  if (cols % 8 != 0 || ldx % 8 != 0) return GNK_ERR_BAD_SHAPE;
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 7)) return GNK_ERR_BAD_ALIGN;
  if (perm_h > 0 && (perm_l <= 0 || rows % (perm_h * perm_l) != 0)) return GNK_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dispatch_dtype(dtype, [&](auto* tag) -> int {
    using T = std::remove_cv_t<std::remove_pointer_t<decltype(tag)>>;
    if (qkind == GNK_Q_INT8)
      return launch_rowwise<T, GNK_Q_INT8>(static_cast<const T*>(x), rows, cols, ldx, static_cast<uint8_t*>(q), scale,
                                           perm_h, perm_l, st);
    return launch_rowwise<T, GNK_Q_E4M3>(static_cast<const T*>(x), rows, cols, ldx, static_cast<uint8_t*>(q), scale,
                                         perm_h, perm_l, st);
  });
}

extern "C" int gnk_quant_mx(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx, int qkind, int rule, void* q,
                            uint8_t* sf, int sf_swizzled, gnk_stream_t stream) {
  if (!x || !q || !sf || M <= 0 || K <= 0) return GNK_ERR_BAD_ARG;
  if (qkind != GNK_Q_E4M3 && qkind != GNK_Q_E5M2 && qkind != GNK_Q_E2M1) return GNK_ERR_BAD_ARG;
  if (rule != GNK_MX_OCP && rule != GNK_MX_NV) return GNK_ERR_BAD_ARG;
  if (K % 32 != 0 || ldx % 8 != 0) return GNK_ERR_BAD_SHAPE;
  if (!aligned16(x) || !aligned16(q)) return GNK_ERR_BAD_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t ks = K / 32;
  const int64_t rows_out = sf_swizzled ? (M + 127) / 128 * 128 : M;
  const int64_t ks_out = sf_swizzled ? (ks + 3) / 4 * 4 : ks;
  const int64_t nblk = (rows_out * ks_out + 255) / 256;
  if (nblk > 0x7FFFFFFF / 256) return GNK_ERR_TOO_LARGE;
  const unsigned grid = static_cast<unsigned>(nblk);
  const int ks_shift = pow2_shift(ks_out);
  return dispatch_dtype(dtype, [&](auto* tag) -> int {
    using T = std::remove_cv_t<std::remove_pointer_t<decltype(tag)>>;
    const T* xp = static_cast<const T*>(x);
    uint8_t* qp = static_cast<uint8_t*>(q);
#define GNK_MXK(QK, RL) quant_mx_kernel<T, QK, RL><<<grid, 256, 0, st>>>(xp, M, K, ldx, qp, sf, sf_swizzled, rows_out, ks_out, ks_shift)
    if (rule == GNK_MX_OCP) {
      if (qkind == GNK_Q_E4M3) GNK_MXK(GNK_Q_E4M3, GNK_MX_OCP);
      else if (qkind == GNK_Q_E5M2) GNK_MXK(GNK_Q_E5M2, GNK_MX_OCP);
      else GNK_MXK(GNK_Q_E2M1, GNK_MX_OCP);
    } else {
      if (qkind == GNK_Q_E4M3) GNK_MXK(GNK_Q_E4M3, GNK_MX_NV);
      else if (qkind == GNK_Q_E5M2) GNK_MXK(GNK_Q_E5M2, GNK_MX_NV);
      else GNK_MXK(GNK_Q_E2M1, GNK_MX_NV);
    }
#undef GNK_MXK
    GNK_LAUNCH_OK();
    return (int)GNK_OK;
  });
}

extern "C" int gnk_quant_nvfp4(const void* x, int dtype, int64_t M, int64_t K, int64_t ldx,
                               const float* tensor_scale, float eps, void* q, uint8_t* sf, int sf_swizzled,
                               gnk_stream_t stream) {
  if (!x || !q || !sf || !tensor_scale || M <= 0 || K <= 0) return GNK_ERR_BAD_ARG;
  if (K % 16 != 0 || ldx % 8 != 0) return GNK_ERR_BAD_SHAPE;
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 7)) return GNK_ERR_BAD_ALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t ks = K / 16;
  const int64_t rows_out = sf_swizzled ? (M + 127) / 128 * 128 : M;
  const int64_t ks_out = sf_swizzled ? (ks + 3) / 4 * 4 : ks;
  const int64_t nblk = (rows_out * ks_out + 255) / 256;
  if (nblk > 0x7FFFFFFF / 256) return GNK_ERR_TOO_LARGE;
  const unsigned grid = static_cast<unsigned>(nblk);
  const int ks_shift = pow2_shift(ks_out);
  return dispatch_dtype(dtype, [&](auto* tag) -> int {
    using T = std::remove_cv_t<std::remove_pointer_t<decltype(tag)>>;
    quant_nvfp4_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(x), M, K, ldx, tensor_scale, eps,
                                                 static_cast<uint8_t*>(q), sf, sf_swizzled, rows_out, ks_out, ks_shift);
    GNK_LAUNCH_OK();
    return (int)GNK_OK;
  });
}

extern "C" int gnk_sf_swizzle(const uint8_t* src, uint8_t* dst, int64_t M, int64_t Ks, int to_swizzled,
                              gnk_stream_t stream) {
  if (!src || !dst || M <= 0 || Ks <= 0) return GNK_ERR_BAD_ARG;
  const int64_t Mp = (M + 127) / 128 * 128, Kp = (Ks + 3) / 4 * 4;
  if (!to_swizzled && (M != Mp || Ks != Kp)) return GNK_ERR_BAD_SHAPE;
  const int64_t n = Mp * Kp;
  sf_swizzle_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, dst, M, Ks, Mp, Kp, to_swizzled);
  GNK_LAUNCH_OK();
  return GNK_OK;
}

extern "C" int gnk_dequant_block(const void* q, const uint8_t* sf, int64_t M, int64_t K, int qkind, int block,
                                 const float* tensor_scale, float* out, gnk_stream_t stream) {
  if (!q || !sf || !out || M <= 0 || K <= 0) return GNK_ERR_BAD_ARG;
  if ((block != 16 && block != 32) || K % block != 0) return GNK_ERR_BAD_SHAPE;
  if (qkind != GNK_Q_E4M3 && qkind != GNK_Q_E5M2 && qkind != GNK_Q_E2M1) return GNK_ERR_BAD_ARG;
  const int64_t n = M * K;
  dequant_block_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(q), sf, M, K, qkind, block, tensor_scale, out);
  GNK_LAUNCH_OK();
  return GNK_OK;
}

// ---------------------------------------------------------------------------------------------
// gnk_absmax_static: the same reduction for callers that cannot provide scratch memory.
//
// Some hosts of this library hold no allocator they could call for it: a serving runtime that
// has handed every byte of device memory to its own arena, or a plugin boundary that passes
// raw input/output pointers and nothing else.  Calling cudaMalloc from such a place is either
// impossible (no memory left outside the arena) or unwelcome (it synchronises the device in the
// middle of a latency-critical loop).  For them the scratch lives in the library image itself:
// a fixed array in device global memory that every GPU loading the library carries until the
// process exits.
// ---------------------------------------------------------------------------------------------
namespace gnk {
namespace {

constexpr int64_t kStaticAbsmaxMaxElems = 1ll << 32;  // documented limit of gnk_absmax_static
// ticket word + one partial maximum per CTA (the kernel never launches more than kAbsmaxMaxCtas CTAs)
static __device__ __align__(256) unsigned int g_static_absmax_scratch[1 + kAbsmaxMaxCtas];

// Device address of the array above, per device.  The array's name is only a host-side handle;
// the address a kernel can use has to be asked for with the owning device current.
std::mutex g_static_mu;
unsigned int* g_static_ptr[64];

int static_scratch_for_current_device(unsigned int** out) {
  int dev = 0;
  GNK_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return GNK_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    GNK_CUDA_OK(cudaGetSymbolAddress(&p, g_static_absmax_scratch));
    g_static_ptr[dev] = static_cast<unsigned int*>(p);
  }
  *out = g_static_ptr[dev];
  return GNK_OK;
}

}  // namespace
}  // namespace gnk

extern "C" int64_t gnk_absmax_static_max_elems(void) { return kStaticAbsmaxMaxElems; }

extern "C" int gnk_absmax_static(const void* x, int dtype, int64_t n, float divisor, float* out,
                                 gnk_stream_t stream) {
  if (!x || !out || n <= 0 || !(divisor > 0.f)) return GNK_ERR_BAD_ARG;
  if (n > kStaticAbsmaxMaxElems) return GNK_ERR_TOO_LARGE;  // beyond what the built-in scratch is specified for
  if (!aligned16(x)) return GNK_ERR_BAD_ALIGN;
  unsigned int* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc != GNK_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left.  Only the ticket word has to start at zero;
  // the partial maxima are overwritten before they are read.
  GNK_CUDA_OK(cudaMemsetAsync(scratch, 0, sizeof(unsigned int), st));
  int64_t want = (n / 8 + kAbsmaxThreads - 1) / kAbsmaxThreads;
  int grid = static_cast<int>(want < 1 ? 1 : (want > kAbsmaxMaxCtas ? kAbsmaxMaxCtas : want));
  const int cap = num_sms() * 8;
  if (grid > cap) grid = cap;
  if (grid > kAbsmaxMaxCtas) grid = kAbsmaxMaxCtas;
  return dispatch_dtype(dtype, [&](auto* tag) -> int {
    using T = std::remove_cv_t<std::remove_pointer_t<decltype(tag)>>;
    absmax_kernel<T><<<grid, kAbsmaxThreads, 0, st>>>(static_cast<const T*>(x), n, out, divisor, scratch);
    GNK_LAUNCH_OK();
    return (int)GNK_OK;
  });
}

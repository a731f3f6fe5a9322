// GQA attention forward with 8-bit QK (E4M3 or INT8 codes + per-row fp32 scales), bf16 V,
// online softmax in fp32, P rounded to bf16 for P*V, lower-right causal mask.  D = 128.
//
// One CTA per (batch, query head, 256 query rows) = two 128-row tiles "A" and "B" that share
// every K/V tile; heavy (late) query blocks of a causal problem are scheduled first.  Warps:
//   warps 0-3 / 4-7  softmax + epilogue of tile A / tile B (thread = query row).  Two passes over
//              the S tile in TMEM keep the register count low: pass 1 finds the row maximum of
//              (S * scale_q*D^-1/2*log2e) * scale_k[col] under the mask, pass 2 forms
//              P = exp2(. - max), sums it and writes it as bf16 into shared memory in the
//              128-byte-swizzled K-major layout the tensor core reads.  O lives in TMEM and is
//              rescaled only when a row maximum grows by more than 2^8 (decided per warp).
//   warp 8     MMA: S_T = Q_T K_j^T (tcgen05 kind::f8f6f4 or kind::i8, N = 128) and
//              O_T += P_T V_j (kind::f16, V consumed N-major straight from its TMA tile), issued
//              A, B, A, B ... so that the tensor core works on one tile while the softmax
//              warps of the other tile run
//   warp 9     producer: TMA loads of both Q tiles (once), K and V tiles (2-stage rings)
// TMEM: S_A [0,128) S_B [128,256) O_A [256,384) O_B [384,512).
// Every barrier wait is bounded (see mbar_wait); no thread ever spins without a limit.
#include <atomic>
#include <type_traits>

#include "gnk_common.cuh"

namespace gnk {
namespace {

constexpr int kBM = 128;  // query rows per tile (two tiles per CTA)
constexpr int kBN = 128;  // keys per tile
constexpr int kD = 128;   // head dimension (QK and V)
constexpr float kLazyRescale = 8.f;  // log2 units: O is rescaled only when a row max grows by more than this

constexpr int kQBytes = kBM * kD;          // 8-bit Q tile
constexpr int kKBytes = kBN * kD;          // 8-bit K tile
constexpr int kVHalfBytes = kBN * 128;     // bf16 V tile, 64 of the 128 D columns (one 128-byte swizzle row per key)
constexpr int kVBytes = 2 * kVHalfBytes;
constexpr int kPHalfBytes = kBM * 128;     // bf16 P tile, 64 of the 128 key columns
constexpr int kPBytes = 2 * kPHalfBytes;
constexpr int kSmemBytes = 1024 + 2 * kQBytes + 2 * kKBytes + 2 * kVBytes + 2 * kPBytes + 2 * kBN * 4 + 256;
constexpr int kThreads = 320;

struct AttnArgs {
  int Lq, Lk, Hq, Hkv, group, causal, q_blocks;
  float qk_scale;  // D^-1/2 * log2(e) in fp32
  const float* scale_q;
  const float* scale_k;
  __nv_bfloat16* o;
  int64_t o_sb, o_sl, o_sh;
  long long* trace;  // debug: clock64 stamps of CTA 0, softmax warps 0 and 4, 8 per key tile (null = off)
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// shared-memory descriptor for an N-major (MN-major) bf16 operand stored as two 64-column
// halves of [rows x 128 bytes], 128-byte swizzle: 8-row groups 1024 bytes apart (SBO), the
// second 64-column half `lbo_bytes` after the first (LBO).
__device__ __forceinline__ uint64_t sdesc_mn128(uint32_t smem_addr, uint32_t lbo_bytes) {
  return (uint64_t)((smem_addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}

// key tiles a 128-row query tile starting at row0 has to visit (0 when it sees no key at all)
__device__ __forceinline__ int kv_tiles_for(int row0, const AttnArgs& a) {
  if (row0 >= a.Lq) return 0;
  const int last_row = min(row0 + kBM - 1, a.Lq - 1);
  const int max_col = a.causal ? min(a.Lk - 1, last_row + (a.Lk - a.Lq)) : a.Lk - 1;
  return max_col >= 0 ? max_col / kBN + 1 : 0;
}

template <int QK>
__global__ void __launch_bounds__(kThreads, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const AttnArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sm_q = base;                     // Q_A, Q_B
  const uint32_t sm_k = sm_q + 2 * kQBytes;       // 2 stages
  const uint32_t sm_v = sm_k + 2 * kKBytes;       // 2 stages
  const uint32_t sm_p = sm_v + 2 * kVBytes;       // P_A, P_B
  const uint32_t sm_sk = sm_p + 2 * kPBytes;      // key scales of the current tile, one copy per query tile
  const uint32_t bars = sm_sk + 2 * kBN * 4;
  const uint32_t bar_q = bars;
  auto bar_kfull = [&](int s) { return bars + 8 * (1 + s); };
  auto bar_kempty = [&](int s) { return bars + 8 * (3 + s); };
  auto bar_vfull = [&](int s) { return bars + 8 * (5 + s); };
  auto bar_vempty = [&](int s) { return bars + 8 * (7 + s); };
  auto bar_sfull = [&](int t) { return bars + 8 * (9 + t); };    // per query tile
  auto bar_pready = [&](int t) { return bars + 8 * (11 + t); };
  auto bar_pvdone = [&](int t) { return bars + 8 * (13 + t); };
  const uint32_t tmem_slot = bars + 8 * 15;
  float* sk_ptr = reinterpret_cast<float*>(smem_raw + (sm_sk - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.z;
  const int qb = a.q_blocks - 1 - static_cast<int>(blockIdx.y);  // heavy causal blocks first
  const int hk = h / a.group;
  const int shift = a.Lk - a.Lq;  // lower-right alignment: query i sees keys j <= i + shift
  const int n_t[2] = {kv_tiles_for(qb * 2 * kBM, a), kv_tiles_for(qb * 2 * kBM + kBM, a)};
  const int n_max = max(n_t[0], n_t[1]);

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_kfull(s), 1);
      mbar_init(bar_kempty(s), 1);
      mbar_init(bar_vfull(s), 1);
      mbar_init(bar_vempty(s), 1);
      mbar_init(bar_sfull(s), 1);
      mbar_init(bar_pready(s), 4);  // one arrival per softmax warp of the tile
      mbar_init(bar_pvdone(s), 1);
    }
    fence_mbar_init();
  }
  if (warp == 9 && lane == 0) {
    tma_prefetch_desc(&tm_q);
    tma_prefetch_desc(&tm_k);
    tma_prefetch_desc(&tm_v);
  }
  if (warp == 8) {
    tmem_alloc<1>(tmem_slot, 512);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  if (warp == 9) {
    // ------------------------------ producer ------------------------------
    const bool leader = elect_one();
    if (n_max > 0 && leader) {
      mbar_expect_tx(bar_q, 2 * kQBytes);
      tma_load_4d(sm_q, &tm_q, bar_q, 0, h, qb * 2 * kBM, b);
      tma_load_4d(sm_q + kQBytes, &tm_q, bar_q, 0, h, qb * 2 * kBM + kBM, b);
    }
    for (int j = 0; j < n_max; ++j) {
      const int st = j & 1;
      const uint32_t par = ((j >> 1) & 1) ^ 1;
      if (!mbar_wait(bar_kempty(st), par, (0x11u << 24) | (1u << 16) | j)) break;
      if (leader) {
        mbar_expect_tx(bar_kfull(st), kKBytes);
        tma_load_4d(sm_k + st * kKBytes, &tm_k, bar_kfull(st), 0, hk, j * kBN, b);
      }
      if (!mbar_wait(bar_vempty(st), par, (0x11u << 24) | (2u << 16) | j)) break;
      if (leader) {
        mbar_expect_tx(bar_vfull(st), kVBytes);
        tma_load_4d(sm_v + st * kVBytes, &tm_v, bar_vfull(st), 0, hk, j * kBN, b);
        tma_load_4d(sm_v + st * kVBytes + kVHalfBytes, &tm_v, bar_vfull(st), 64, hk, j * kBN, b);
      }
      __syncwarp();
    }
  } else if (warp == 8) {
    // ------------------------------ MMA issuer ------------------------------
    const bool leader = elect_one();
    constexpr uint32_t kIdescS = QK == GNK_Q_INT8 ? idesc_dense(2, 1, 1, kBM, kBN) : idesc_dense(1, 0, 0, kBM, kBN);
    constexpr uint32_t kIdescO = idesc_dense(1, 1, 1, kBM, kD, 0, 1);  // bf16 x bf16, B (= V) N-major
    bool ok = n_max > 0 && mbar_wait(bar_q, 0, (0x12u << 24) | (1u << 16));
    // S_T(j) = Q_T K_j^T.  The K stage is released by the last tile that reads it.
    auto issue_s = [&](int t, int j) -> bool {
      const int st = j & 1;
      if (!mbar_wait(bar_kfull(st), (j >> 1) & 1, (0x12u << 24) | (2u << 16) | j)) return false;
      tc_fence_after();
      const uint64_t q_desc = sdesc_k128(sm_q + t * kQBytes);
      const uint64_t k_desc = sdesc_k128(sm_k + st * kKBytes);
      const uint32_t d = tmem_base + t * kBN;
      const bool last_user = (t == 1) || (j >= n_t[1]);
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          if constexpr (QK == GNK_Q_INT8)
            tc_mma<MmaKind::I8, 1>(d, q_desc + 2 * kk, k_desc + 2 * kk, kIdescS, kk != 0);
          else
            tc_mma<MmaKind::F8F6F4, 1>(d, q_desc + 2 * kk, k_desc + 2 * kk, kIdescS, kk != 0);
        }
        if (last_user) tc_commit<1>(bar_kempty(st));
        tc_commit<1>(bar_sfull(t));
      }
      __syncwarp();
      return true;
    };
    // O_T += P_T(j) V_j.  The V stage is released by the last tile that reads it.
    auto issue_pv = [&](int t, int j) -> bool {
      const int st = j & 1;
      if (!mbar_wait(bar_pready(t), j & 1, (0x12u << 24) | (4u << 16) | j)) return false;
      if (!mbar_wait(bar_vfull(st), (j >> 1) & 1, (0x12u << 24) | (5u << 16) | j)) return false;
      tc_fence_after();
      const uint32_t p_addr = sm_p + t * kPBytes;
      const uint32_t v_addr = sm_v + st * kVBytes;
      const uint32_t d = tmem_base + 256 + t * kD;
      const bool last_user = (t == 1) || (j >= n_t[1]);
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // A: 16 key columns of P (K-major, half kk/4, 32 bytes per step); B: 16 key rows of V (N-major)
          const uint64_t p_desc = sdesc_k128(p_addr + (kk >> 2) * kPHalfBytes) + 2 * (kk & 3);
          const uint64_t v_desc = sdesc_mn128(v_addr + kk * 16 * 128, kVHalfBytes);
          tc_mma<MmaKind::F16, 1>(d, p_desc, v_desc, kIdescO, (j | kk) != 0);
        }
        if (last_user) tc_commit<1>(bar_vempty(st));
        tc_commit<1>(bar_pvdone(t));
      }
      __syncwarp();
      return true;
    };
    if (ok && n_t[0] > 0) ok = issue_s(0, 0);
    if (ok && n_t[1] > 0) ok = issue_s(1, 0);
    for (int j = 0; j < n_max && ok; ++j) {
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (!ok || j >= n_t[t]) continue;
        ok = issue_pv(t, j);                                  // needs P_t(j): the softmax of tile t has finished S_t(j)
        if (ok && j + 1 < n_t[t]) ok = issue_s(t, j + 1);     // so S_t can be overwritten at once
      }
    }
  } else {
    // ------------------------------ softmax + epilogue (tile A: warps 0-3, tile B: warps 4-7) ------------------------------
    const int t = warp >> 2;
    const int r = (warp & 3) * 32 + lane;  // row inside the tile = TMEM lane
    const int row0 = qb * 2 * kBM + t * kBM;
    const int row = row0 + r;
    const int nt = n_t[t];
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tm_s = tmem_base + lane_sel + t * kBN;
    const uint32_t tm_o = tmem_base + lane_sel + 256 + t * kD;
    const bool row_live = row < a.Lq;
    const float sq = (a.scale_q && row_live) ? __ldg(a.scale_q + (static_cast<int64_t>(b) * a.Hq + h) * a.Lq + row) : 1.f;
    const float qs = __fmul_rn(a.qk_scale, sq);
    const float* skg = a.scale_k ? a.scale_k + (static_cast<int64_t>(b) * a.Hkv + hk) * a.Lk : nullptr;
    const int limit = a.causal ? min(row + shift, a.Lk - 1) : a.Lk - 1;  // last visible key of this row
    float* sk = sk_ptr + t * kBN;
    const uint32_t p_row = sm_p + t * kPBytes + (r >> 3) * 1024 + (r & 7) * 128;
    float m_used = -1e38f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nt; ++j) {
      long long* tr = (a.trace && blockIdx.x == 0 && (warp & 3) == 0 && lane == 0 && j < 32) ? a.trace + (t * 32 + j) * 8 : nullptr;
      if (tr) tr[0] = clock64();
      // stage the tile's key scales (one per thread of this group), 0 beyond the sequence
      {
        const int col = j * kBN + r;
        const float v = col < a.Lk ? (skg ? __ldg(skg + col) : 1.f) : 0.f;
        asm volatile("bar.sync %0, 128;" ::"r"(1 + t) : "memory");  // everyone is done with the previous tile's scales
        sk[r] = v;
        asm volatile("bar.sync %0, 128;" ::"r"(1 + t) : "memory");
      }
      // A wait that runs out does not leave the loop: the four warps of the group meet at the named
      // barrier above every iteration, so a warp that left alone would strand the other three there.
      // It stops waiting instead (every later wait is skipped), keeps arriving, and the rows it owns
      // are written as zeros at the end; the status word tells the host.
      if (ok && !mbar_wait(bar_sfull(t), j & 1, (0x13u << 24) | (1u << 16) | j)) ok = false;
      tc_fence_after();
      if (tr) tr[1] = clock64();
      const int col0 = j * kBN;
      const bool need_mask = col0 + kBN - 1 > min(row0 + shift, a.Lk - 1) && (a.causal || col0 + kBN > a.Lk);
      // ---- pass 1: row maximum of x = S * scale_k[col]; the positive row factor qs is applied once at the end ----
      float xmax = -INFINITY;
      auto pass1 = [&](auto masked) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t raw[32];
          tmem_ld32(tm_s + c * 32, raw);
          tc_wait_ld();
#pragma unroll
          for (int i4 = 0; i4 < 8; ++i4) {
            const float4 k4 = *reinterpret_cast<const float4*>(sk + c * 32 + i4 * 4);
            const float kk[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = i4 * 4 + e;
              const float s0 = QK == GNK_Q_INT8 ? __int2float_rn(static_cast<int>(raw[i])) : __uint_as_float(raw[i]);
              float x = s0 * kk[e];
              if (decltype(masked)::value && col0 + c * 32 + i > limit) x = -INFINITY;
              xmax = fmaxf(xmax, x);
            }
          }
        }
      };
      if (need_mask) pass1(std::true_type{}); else pass1(std::false_type{});
      if (tr) tr[2] = clock64();
      // qs >= 0 (absmax scales), so max(qs * x) = qs * max(x); a fully masked row keeps the old maximum
      const float mt = fmaxf(m_used, xmax == -INFINITY ? -INFINITY : qs * xmax);
      // lazy rescale, decided per warp so the TMEM traffic stays warp-collective
      const bool grow = mt > m_used + kLazyRescale;
      const bool rescale = __any_sync(0xffffffffu, grow) || j == 0;
      // O and the P buffer may only be touched once the previous P*V of this tile has retired
      if (j > 0 && ok && !mbar_wait(bar_pvdone(t), (j - 1) & 1, (0x13u << 24) | (2u << 16) | j)) ok = false;
      if (rescale) {
        const float alpha = fast_exp2(m_used - mt);
        m_used = mt;
        l *= alpha;
        if (j > 0) {
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld32(tm_o + c * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(tm_o + c * 32, o);
          }
          tc_wait_st();
        }
      }
      // ---- pass 2: P = exp2(qs * x - max), row sum, bf16 P into shared memory ----
      if (tr) tr[3] = clock64();
      float rs = 0.f;
      const float neg_m = -m_used;
      auto pass2 = [&](auto masked) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t raw[32];
          tmem_ld32(tm_s + c * 32, raw);
          tc_wait_ld();
          float p[32];
#pragma unroll
          for (int i4 = 0; i4 < 8; ++i4) {
            const float4 k4 = *reinterpret_cast<const float4*>(sk + c * 32 + i4 * 4);
            const float kk[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = i4 * 4 + e;
              const float s0 = QK == GNK_Q_INT8 ? __int2float_rn(static_cast<int>(raw[i])) : __uint_as_float(raw[i]);
              float ex = fmaf(qs, s0 * kk[e], neg_m);
              if (decltype(masked)::value && col0 + c * 32 + i > limit) ex = -INFINITY;
              p[i] = fast_exp2(ex);
              rs += p[i];
            }
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int cc = c * 4 + q4;  // 16-byte chunk index 0..15 along the 128 keys
            const uint32_t addr = p_row + (cc >> 3) * kPHalfBytes + (((cc & 7) ^ (r & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pack_bf16x2(p[q4 * 8], p[q4 * 8 + 1])),
                         "r"(pack_bf16x2(p[q4 * 8 + 2], p[q4 * 8 + 3])), "r"(pack_bf16x2(p[q4 * 8 + 4], p[q4 * 8 + 5])),
                         "r"(pack_bf16x2(p[q4 * 8 + 6], p[q4 * 8 + 7]))
                         : "memory");
          }
        }
      };
      if (need_mask) pass2(std::true_type{}); else pass2(std::false_type{});
      if (tr) tr[4] = clock64();
      l += rs;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pready(t));
      if (tr) tr[5] = clock64();
    }

    // epilogue: O / l -> bf16
    if (nt > 0 && ok) ok = mbar_wait(bar_pvdone(t), (nt - 1) & 1, (0x13u << 24) | (4u << 16));
    tc_fence_after();
    __nv_bfloat16* orow = a.o + b * a.o_sb + static_cast<int64_t>(row) * a.o_sl + h * a.o_sh;
    const bool has_sum = l > 0.f && nt > 0 && ok;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t o[32];
      if (nt > 0) {
        tmem_ld32(tm_o + c * 32, o);
        tc_wait_ld();
      }
      if (row_live) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = has_sum ? __fdiv_rn(__uint_as_float(o[i + e]), l) : 0.f;
          *reinterpret_cast<uint4*>(orow + c * 32 + i) =
              make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

GNK_DEFINE_STATUS_READER(attn_status_reader)

}  // namespace
}  // namespace gnk

using namespace gnk;

namespace {
std::atomic<long long*> g_attn_trace{nullptr};
}
// Test hook: device buffer of 2 * 32 * 8 int64 receiving clock64 stamps (see AttnArgs::trace); NULL = off.
extern "C" int gnk_debug_attn_trace(void* device_buffer) {
  g_attn_trace = static_cast<long long*>(device_buffer);
  return GNK_OK;
}

extern "C" int gnk_attn_fwd(const void* q, const void* k, const void* v, void* o, const float* scale_q,
                            const float* scale_k, int qk_kind, int64_t B, int64_t Lq, int64_t Lk, int64_t Hq,
                            int64_t Hkv, int64_t D, const int64_t* q_strides, const int64_t* k_strides,
                            const int64_t* v_strides, const int64_t* o_strides, int causal, gnk_stream_t stream) {
  if (!q || !k || !v || !o || !q_strides || !k_strides || !v_strides || !o_strides) return GNK_ERR_BAD_ARG;
  if (B <= 0 || Lq <= 0 || Lk <= 0 || Hq <= 0 || Hkv <= 0) return GNK_ERR_BAD_ARG;
  if (qk_kind != GNK_Q_E4M3 && qk_kind != GNK_Q_INT8) return GNK_ERR_BAD_ARG;
  if ((scale_q == nullptr) != (scale_k == nullptr)) return GNK_ERR_BAD_ARG;
  if (D != kD) return GNK_ERR_UNSUPPORTED;
  if (Hq % Hkv != 0) return GNK_ERR_BAD_SHAPE;
  if (B > 65535 || (Lq + 2 * kBM - 1) / (2 * kBM) > 65535) return GNK_ERR_TOO_LARGE;
  if ((o_strides[0] | o_strides[1] | o_strides[2]) & 7) return GNK_ERR_BAD_ALIGN;
  if (!aligned16(o)) return GNK_ERR_BAD_ALIGN;
  int rc = check_arch();
  if (rc != GNK_OK) return rc;

  // [B, L, H, D] seen by TMA as (D, H, L, B), strides in bytes for H, L, B
  auto make = [&](CUtensorMap* m, const void* p, int64_t L, int64_t H, const int64_t* s, int elem, uint32_t box_d,
                  uint32_t box_rows, CUtensorMapDataType dt) {
    const uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(H), static_cast<uint64_t>(L),
                              static_cast<uint64_t>(B)};
    const uint64_t str[3] = {static_cast<uint64_t>(s[2] * elem), static_cast<uint64_t>(s[1] * elem),
                             static_cast<uint64_t>(s[0] * elem)};
    const uint32_t box[4] = {box_d, 1, box_rows, 1};
    return make_tmap_4d(m, dt, p, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
  };
  CUtensorMap tm_q, tm_k, tm_v;
  if ((rc = make(&tm_q, q, Lq, Hq, q_strides, 1, 128, kBM, CU_TENSOR_MAP_DATA_TYPE_UINT8)) != GNK_OK) return rc;
  if ((rc = make(&tm_k, k, Lk, Hkv, k_strides, 1, 128, kBN, CU_TENSOR_MAP_DATA_TYPE_UINT8)) != GNK_OK) return rc;
  if ((rc = make(&tm_v, v, Lk, Hkv, v_strides, 2, 64, kBN, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16)) != GNK_OK) return rc;

  AttnArgs a{};
  a.trace = g_attn_trace.load();
  a.Lq = static_cast<int>(Lq);
  a.Lk = static_cast<int>(Lk);
  a.Hq = static_cast<int>(Hq);
  a.Hkv = static_cast<int>(Hkv);
  a.group = static_cast<int>(Hq / Hkv);
  a.causal = causal != 0;
  a.q_blocks = static_cast<int>((Lq + 2 * kBM - 1) / (2 * kBM));
  a.qk_scale = static_cast<float>((1.0 / sqrt(static_cast<double>(D))) * 1.44269504);  // as the reference folds it
  a.scale_q = scale_q;
  a.scale_k = scale_k;
  a.o = static_cast<__nv_bfloat16*>(o);
  a.o_sb = o_strides[0];
  a.o_sl = o_strides[1];
  a.o_sh = o_strides[2];

  dim3 grid(static_cast<unsigned>(Hq), static_cast<unsigned>(a.q_blocks), static_cast<unsigned>(B));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (qk_kind == GNK_Q_INT8) {
    GNK_CUDA_OK(cudaFuncSetAttribute(attn_fwd_kernel<GNK_Q_INT8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attn_fwd_kernel<GNK_Q_INT8><<<grid, kThreads, kSmemBytes, st>>>(tm_q, tm_k, tm_v, a);
  } else {
    GNK_CUDA_OK(cudaFuncSetAttribute(attn_fwd_kernel<GNK_Q_E4M3>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    attn_fwd_kernel<GNK_Q_E4M3><<<grid, kThreads, kSmemBytes, st>>>(tm_q, tm_k, tm_v, a);
  }
  GNK_LAUNCH_OK();
  return GNK_OK;
}

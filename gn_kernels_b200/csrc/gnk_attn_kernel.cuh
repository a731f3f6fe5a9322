// GQA attention forward on tcgen05 tensor cores: online softmax in fp32, lower-right causal mask,
// D = 128.  Q and K are 8-bit codes (E4M3 or INT8) with per-row fp32 scales, or plain bf16 / fp16;
// V, P and O are bf16 or fp16.  Batched [B, L, H, D] tensors or packed variable-length sequences.
//
// One CTA per (batch, query head, 256 query rows) = two 128-row tiles "A" and "B" that share every
// K/V tile; heavy (late) query blocks of a causal problem are scheduled first.  Warps:
//   warps 0-3 / 4-7  softmax + epilogue of tile A / tile B (thread = query row).  The whole 128-wide
//              score row is read from TMEM once (four 32-column loads in flight together), scaled
//              ((S * scale_k[col]) * (scale_q * D^-1/2 * log2e)), masked, reduced to the row maximum
//              with three-input max, exponentiated (ex2), summed, rounded to the 16-bit type of V
//              and written BACK INTO TMEM over the first 64 columns of the score tile, from where
//              the tensor core reads it as the A operand of P*V.  P never touches shared memory.
//              O lives in TMEM and is rescaled only when a row maximum grows by more than 2^8
//              (decided per warp); only then does the softmax wait for the previous P*V.
//   warp 8     MMA: S_T = Q_T K_j^T (kind::f8f6f4, kind::i8 or kind::f16, N = 128) and
//              O_T += P_T V_j (kind::f16, A from TMEM, V consumed N-major straight from its TMA
//              tile), issued A, B, A, B ... so that the tensor core works on one tile while the
//              softmax warps of the other tile run.  S_T(j+1) overwrites P_T(j): safe because the
//              tensor core executes the MMAs of one issuing thread in order.
//   warp 9     producer: TMA loads of both Q tiles (once), K and V tiles (rings of kStages)
//   warps 10-11 idle (they complete the warpgroup whose registers are handed to the softmax warps)
// TMEM: S_A / P_A [0,128) S_B / P_B [128,256) O_A [256,384) O_B [384,512).
// A variant with 64-key score sub-tiles (two score buffers per query tile, Q K^T two sub-tiles ahead of
// the softmax so that the chain softmax -> P V -> Q K^T -> softmax no longer contains the tensor core)
// was built and measured: correct, but slower (771 / 928 against 868 / 1069 TFLOP/s causal / full):
// the softmax is bound by dependent-issue latency (ncu: 9 instructions per score element, 0.42 issued
// per scheduler cycle with two softmax warps per scheduler, stall reason "wait"), and halving the step
// doubles its fixed costs (TMEM round trips, barrier hand-shakes, votes) without removing instructions.
// So was a variant with two threads per score row (16 softmax warps of 64 columns each, four per
// scheduler instead of two, row maxima exchanged through shared memory): correct, 669 / 764 TFLOP/s:
// at the 112 registers such a thread can have it spills, and the extra warps contend instead of
// filling each other's stalls.
// And so was one MMA issuer warp PER query tile (each blocking on its own tile's barriers only; K / V stages
// handed back by two arrivals), with or without the P V product split into two halves of 64 keys (the first
// issued half-way through the softmax's second pass): correct, 772 TFLOP/s causal against 865-877.  The
// single issuer that serves the tiles strictly in turn is what keeps the two softmax groups in anti-phase;
// with independent issuers they drift into phase and then share the tensor pipe and the special-function
// unit at the same moments.
// Every barrier wait is bounded (see mbar_wait); a softmax warp whose wait runs out stops waiting
// but keeps arriving at the barriers of its group, so the CTA always reaches its end.
#pragma once

#include <type_traits>

#include "gnk_common.cuh"

namespace gnk {
namespace attn {

constexpr int kBM = 128;  // query rows per tile (two tiles per CTA)
constexpr int kBN = 128;  // keys per tile
constexpr int kD = 128;   // head dimension (QK and V)
constexpr float kLazyRescale = 8.f;  // log2 units: O is rescaled only when a row max grows by more than this
// 12 warps: 0-7 softmax, 8 MMA, 9 producer, 10-11 idle.  Warp w runs on SM sub-partition w % 4, each with
// 16384 registers; three warps per sub-partition cap every thread at 168 registers at launch.  The
// role warps (one whole warpgroup, hence the two idle warps) give registers back and the softmax
// warps, which hold a full 128-element score row each, take them.  The CTA owns what it was launched
// with, 3 x 168 = 504 registers per lane of a sub-partition, and setmaxnreg.inc waits WITHOUT a limit
// until its request fits, so the split must stay inside that: 2 x 224 + 56 = 504.
constexpr int kThreads = 384;
// Every 4th pair of probabilities is exponentiated by polynomial (0 = never).  Measured at B=4, Hq=32,
// L=4096, FP8 QK (TFLOP/s causal / full): none 797 / 973, 1 in 4 868 / 1069, 1 in 3 851 / 1006, 1 in 2
// 837 / 998, all 683 / 781; the same with scalar instead of packed f32x2 arithmetic: 772 / 926 at 1 in 4.
constexpr int kPolyPeriod = 4;
constexpr int kSoftmaxRegs = 224, kRoleRegs = 56;
static_assert(2 * kSoftmaxRegs + kRoleRegs <= 3 * 168, "register split exceeds the launch allocation: setmaxnreg.inc would never return");

// element kinds of Q and K (gnk_qkind values)
constexpr int kQkInt8 = GNK_Q_INT8, kQkE4m3 = GNK_Q_E4M3, kQkBf16 = GNK_Q_BF16, kQkF16 = GNK_Q_F16;

template <int QK>
struct QkInfo {
  static constexpr int kElemBytes = (QK == kQkBf16 || QK == kQkF16) ? 2 : 1;
  static constexpr int kTileBytes = kBM * kD * kElemBytes;   // one Q or K tile
  static constexpr int kHalves = kElemBytes;                 // 128-byte-wide column blocks per tile
  static constexpr int kStages = kElemBytes == 1 ? 3 : 2;    // K / V ring depth
};
constexpr int kVHalfBytes = kBN * 128;  // 16-bit V tile, 64 of the 128 D columns (one 128-byte swizzle row per key)
constexpr int kVBytes = 2 * kVHalfBytes;

template <int QK>
constexpr int smem_bytes() {
  return 1024 + 2 * QkInfo<QK>::kTileBytes + QkInfo<QK>::kStages * (QkInfo<QK>::kTileBytes + kVBytes) + 2 * kBN * 4 + 512;
}

struct AttnArgs {
  int Lq, Lk, Hq, Hkv, group, causal, q_blocks;
  float qk_scale;  // D^-1/2 * log2(e) in fp32
  const float* scale_q;
  const float* scale_k;
  void* o;
  int64_t o_sb, o_sl, o_sh;
  const int32_t* q_offsets;   // packed variable-length sequences: [B + 1] row offsets (null = batched)
  const int32_t* kv_offsets;
  long long* trace;  // debug: clock64 stamps of CTA 0, softmax warps 0 and 4, 8 per key tile (null = off)
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// 2^t for a pair of fp32 values on the FMA and integer pipes instead of the special-function unit
// (which delivers only 16 results per clock per SM and is the attention kernel's tightest resource).
// t is clamped at -126, split into n = round(t) (magic-number addition) and f = t - n in [-0.5, 0.5],
// 2^f is a degree-3 polynomial (relative error 7.5e-5, far below the 2^-9 rounding P gets next), and
// n goes straight into the exponent field.
__device__ __forceinline__ void exp2_poly_pair(uint64_t t2, float& p0, float& p1) {
  float t0, t1;
  f2_unpack(t2, t0, t1);
  t0 = fmaxf(t0, -126.f);
  t1 = fmaxf(t1, -126.f);
  const uint64_t tc = f2_pack(t0, t1);
  const uint64_t magic = f2_pack(12582912.f, 12582912.f);  // 1.5 * 2^23: the sum's low mantissa bits hold round(t)
  const uint64_t r2 = f2_add(tc, magic);
  const uint64_t f2 = f2_sub(tc, f2_sub(r2, magic));
  uint64_t q = f2_fma(f2, f2_pack(0.0551716648f, 0.0551716648f), f2_pack(0.2426111251f, 0.2426111251f));
  q = f2_fma(q, f2, f2_pack(0.6932609677f, 0.6932609677f));
  q = f2_fma(q, f2, f2_pack(0.9999280572f, 0.9999280572f));
  float q0, q1, r0, r1;
  f2_unpack(q, q0, q1);
  f2_unpack(r2, r0, r1);
  p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(r0) << 23));
  p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(r1) << 23));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <int VT>
__device__ __forceinline__ uint32_t pack16x2(float lo, float hi) {
  if constexpr (VT == GNK_F16) return pack_half2(lo, hi);
  else return pack_bf16x2(lo, hi);
}

// shared-memory descriptor for an N-major (MN-major) 16-bit operand stored as two 64-column
// halves of [rows x 128 bytes], 128-byte swizzle: 8-row groups 1024 bytes apart (SBO), the
// second 64-column half `lbo_bytes` after the first (LBO).
__device__ __forceinline__ uint64_t sdesc_mn128(uint32_t smem_addr, uint32_t lbo_bytes) {
  return (uint64_t)((smem_addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}

// D[tmem] (+)= A[tmem] * B[smem desc], kind::f16: A is read from TMEM (lane = row, each 32-bit
// column holds two consecutive 16-bit K elements, even element in the low half).
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// key tiles a 128-row query tile starting at row0 has to visit (0 when it sees no key at all)
__device__ __forceinline__ int kv_tiles_for(int row0, int Lq, int Lk, int causal) {
  if (row0 >= Lq) return 0;
  const int last_row = min(row0 + kBM - 1, Lq - 1);
  const int max_col = causal ? min(Lk - 1, last_row + (Lk - Lq)) : Lk - 1;
  return max_col >= 0 ? max_col / kBN + 1 : 0;
}

// QK: element kind of Q and K.  VT: GNK_BF16 or GNK_F16, the type of V, P and O.  ACC16: bit 0 =
// S accumulates in fp16, bit 1 = O accumulates in fp16 (tcgen05 stores an fp16 accumulator in the
// low half of each 32-bit TMEM column).
template <int QK, int VT, int ACC16>
__global__ void __launch_bounds__(kThreads, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const AttnArgs a) {
  using QI = QkInfo<QK>;
  constexpr int kQBytes = QI::kTileBytes, kKBytes = QI::kTileBytes, kStages = QI::kStages;
  constexpr bool kQk16 = QI::kElemBytes == 2;
  constexpr bool kSAcc16 = (ACC16 & 1) != 0, kOAcc16 = (ACC16 & 2) != 0;
  using OutT = std::conditional_t<VT == GNK_F16, __half, __nv_bfloat16>;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sm_q = base;                          // Q_A, Q_B
  const uint32_t sm_k = sm_q + 2 * kQBytes;            // kStages
  const uint32_t sm_v = sm_k + kStages * kKBytes;      // kStages
  const uint32_t sm_sk = sm_v + kStages * kVBytes;     // key scales of the current tile, one copy per query tile
  const uint32_t bars = sm_sk + 2 * kBN * 4;
  const uint32_t bar_q = bars;
  auto bar_kfull = [&](int s) { return bars + 8 * (1 + s); };
  auto bar_kempty = [&](int s) { return bars + 8 * (1 + kStages + s); };
  auto bar_vfull = [&](int s) { return bars + 8 * (1 + 2 * kStages + s); };
  auto bar_vempty = [&](int s) { return bars + 8 * (1 + 3 * kStages + s); };
  auto bar_sfull = [&](int t) { return bars + 8 * (1 + 4 * kStages + t); };    // per query tile
  auto bar_pready = [&](int t) { return bars + 8 * (3 + 4 * kStages + t); };
  auto bar_pvdone = [&](int t) { return bars + 8 * (5 + 4 * kStages + t); };
  auto bar_sread = [&](int t) { return bars + 8 * (7 + 4 * kStages + t); };    // the tile's score row is in registers
  const uint32_t tmem_slot = bars + 8 * (9 + 4 * kStages);
  float* sk_ptr = reinterpret_cast<float*>(smem_raw + (sm_sk - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, b = blockIdx.z;
  const int qb = a.q_blocks - 1 - static_cast<int>(blockIdx.y);  // heavy causal blocks first
  const int hk = h / a.group;
  // batched: every sequence has a.Lq / a.Lk rows and its own batch coordinate; packed: the batch's
  // rows are [offsets[b], offsets[b + 1]) of one long sequence (batch coordinate 0)
  int Lq = a.Lq, Lk = a.Lk, q_start = 0, k_start = 0, bc = b;
  if (a.q_offsets) {
    q_start = __ldg(a.q_offsets + b);
    Lq = __ldg(a.q_offsets + b + 1) - q_start;
    k_start = __ldg(a.kv_offsets + b);
    Lk = __ldg(a.kv_offsets + b + 1) - k_start;
    bc = 0;
  }
  const int shift = Lk - Lq;  // lower-right alignment: query i sees keys j <= i + shift
  const int n_t[2] = {kv_tiles_for(qb * 2 * kBM, Lq, Lk, a.causal), kv_tiles_for(qb * 2 * kBM + kBM, Lq, Lk, a.causal)};
  const int n_max = max(n_t[0], n_t[1]);

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_kfull(s), 1);
      mbar_init(bar_kempty(s), 1);
      mbar_init(bar_vfull(s), 1);
      mbar_init(bar_vempty(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_sfull(s), 1);
      mbar_init(bar_pready(s), 4);  // one arrival per softmax warp of the tile
      mbar_init(bar_pvdone(s), 1);
      mbar_init(bar_sread(s), 4);   // one arrival per softmax warp of the tile
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

  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRoleRegs));
  if (warp == 9) {
    // ------------------------------ producer ------------------------------
    const bool leader = elect_one();
    // a Q or K tile is one 128-byte-wide box (8-bit) or two 64-column halves (16-bit)
    auto load_qk = [&](uint32_t dst, const CUtensorMap* tm, uint32_t bar, int head, int row) {
#pragma unroll
      for (int hf = 0; hf < QI::kHalves; ++hf) tma_load_4d(dst + hf * (kBM * 128), tm, bar, hf * 64, head, row, bc);
    };
    if (n_max > 0 && leader) {
      mbar_expect_tx(bar_q, 2 * kQBytes);
      load_qk(sm_q, &tm_q, bar_q, h, q_start + qb * 2 * kBM);
      load_qk(sm_q + kQBytes, &tm_q, bar_q, h, q_start + qb * 2 * kBM + kBM);
    }
    uint32_t st = 0, par = 1;
    for (int j = 0; j < n_max; ++j) {
      if (!mbar_wait(bar_kempty(st), par, (0x11u << 24) | (1u << 16) | j)) break;
      if (leader) {
        mbar_expect_tx(bar_kfull(st), kKBytes);
        load_qk(sm_k + st * kKBytes, &tm_k, bar_kfull(st), hk, k_start + j * kBN);
      }
      if (!mbar_wait(bar_vempty(st), par, (0x11u << 24) | (2u << 16) | j)) break;
      if (leader) {
        mbar_expect_tx(bar_vfull(st), kVBytes);
        tma_load_4d(sm_v + st * kVBytes, &tm_v, bar_vfull(st), 0, hk, k_start + j * kBN, bc);
        tma_load_4d(sm_v + st * kVBytes + kVHalfBytes, &tm_v, bar_vfull(st), 64, hk, k_start + j * kBN, bc);
      }
      __syncwarp();
      if (++st == kStages) { st = 0; par ^= 1; }
    }
  } else if (warp == 8) {
    // ------------------------------ MMA issuer ------------------------------
    const bool leader = elect_one();
    constexpr uint32_t kSFmt = kSAcc16 ? 0u : 1u;  // accumulator format: 0 = F16, 1 = F32
    constexpr uint32_t kIdescS = QK == kQkInt8   ? idesc_dense(2, 1, 1, kBM, kBN)
                                 : QK == kQkE4m3 ? idesc_dense(1, 0, 0, kBM, kBN)
                                 : QK == kQkBf16 ? idesc_dense(kSFmt, 1, 1, kBM, kBN)
                                                 : idesc_dense(kSFmt, 0, 0, kBM, kBN);
    constexpr uint32_t kVFmt = VT == GNK_F16 ? 0u : 1u;
    constexpr uint32_t kIdescO = idesc_dense(kOAcc16 ? 0u : 1u, kVFmt, kVFmt, kBM, kD, 0, 1);  // B (= V) N-major
    bool ok = n_max > 0 && mbar_wait(bar_q, 0, (0x12u << 24) | (1u << 16));
    // S_T(j) = Q_T K_j^T.  The K stage is released by the last tile that reads it.
    // waits for K_j; done ahead of the wait for P wherever possible: a barrier wait costs ~100 cycles even
    // when its phase has long completed, and everything after P is ready sits on the tile's critical path
    auto wait_k = [&](int j) -> bool {
      return mbar_wait(bar_kfull(j % kStages), (j / kStages) & 1, (0x12u << 24) | (2u << 16) | j);
    };
    // `part`: 0 = all 128 key columns; 1 = key columns 64..127 only, without signalling (they do not overlap P,
    // which sits in score columns 0..63, so they may be computed while the softmax of the previous key tile
    // still runs, as soon as that softmax has its score row in registers); 2 = key columns 0..63, which must
    // follow the P V product that reads P, then the signals for the whole tile.
    constexpr uint32_t kIdescSHalf = (kIdescS & ~(0x3Fu << 17)) | ((64u >> 3) << 17);
    auto issue_s = [&](int t, int j, bool k_waited, int part) -> bool {
      const int st = j % kStages;
      if (!k_waited && !wait_k(j)) return false;
      tc_fence_after();
      const int key0 = part == 1 ? 64 : 0;  // first key row / score column of this part
      const uint32_t q_addr = sm_q + t * kQBytes, k_addr = sm_k + st * kKBytes + key0 * 128;
      const uint32_t d = tmem_base + t * kBN + key0;
      const uint32_t idesc = part == 0 ? kIdescS : kIdescSHalf;
      const bool last_user = (t == 1) || (j >= n_t[1]);
      if (leader) {
        if constexpr (kQk16) {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {  // 16 elements of D per step, half kk / 4
            const uint64_t q_desc = sdesc_k128(q_addr + (kk >> 2) * (kBM * 128)) + 2 * (kk & 3);
            const uint64_t k_desc = sdesc_k128(k_addr + (kk >> 2) * (kBN * 128)) + 2 * (kk & 3);
            tc_mma<MmaKind::F16, 1>(d, q_desc, k_desc, idesc, kk != 0);
          }
        } else {
          const uint64_t q_desc = sdesc_k128(q_addr), k_desc = sdesc_k128(k_addr);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            if constexpr (QK == kQkInt8) tc_mma<MmaKind::I8, 1>(d, q_desc + 2 * kk, k_desc + 2 * kk, idesc, kk != 0);
            else tc_mma<MmaKind::F8F6F4, 1>(d, q_desc + 2 * kk, k_desc + 2 * kk, idesc, kk != 0);
          }
        }
        if (part != 1) {
          if (last_user) tc_commit<1>(bar_kempty(st));
          tc_commit<1>(bar_sfull(t));
        }
      }
      __syncwarp();
      return true;
    };
    // O_T += P_T(j) V_j.  P is read from TMEM (the first 64 columns of the tile's score region).
    auto issue_pv = [&](int t, int j) -> bool {
      const int st = j % kStages;
      // V_j first (it landed long ago), P_t(j) last: nothing but the issue itself follows the moment P is ready
      if (!mbar_wait(bar_vfull(st), (j / kStages) & 1, (0x12u << 24) | (5u << 16) | j)) return false;
      const uint32_t p_tmem = tmem_base + t * kBN;
      const uint32_t v_addr = sm_v + st * kVBytes;
      const uint32_t d = tmem_base + 256 + t * kD;
      const bool last_user = (t == 1) || (j >= n_t[1]);
      const uint64_t v_desc0 = sdesc_mn128(v_addr, kVHalfBytes);
      if (!mbar_wait(bar_pready(t), j & 1, (0x12u << 24) | (4u << 16) | j)) return false;
      tc_fence_after();
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // A: 16 key columns of P = 8 TMEM columns; B: 16 key rows of V (N-major, both 64-column halves):
          // 16 rows of 128 bytes further on per step (the address field counts 16-byte units)
          tc_mma_f16_ts(d, p_tmem + kk * 8, v_desc0 + kk * ((16 * 128) >> 4), kIdescO, (j | kk) != 0);
        }
        if (last_user) tc_commit<1>(bar_vempty(st));
        tc_commit<1>(bar_pvdone(t));
      }
      __syncwarp();
      return true;
    };
    if (ok && n_t[0] > 0) ok = issue_s(0, 0, false, 0);
    if (ok && n_t[1] > 0) ok = issue_s(1, 0, false, 0);
    for (int j = 0; j < n_max && ok; ++j) {
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (!ok || j >= n_t[t]) continue;
        const bool has_next = j + 1 < n_t[t];
        if (has_next) {
          // K_(j+1) and "S_t(j) is in registers" come long before P_t(j): the upper half of S_t(j+1) runs meanwhile
          ok = wait_k(j + 1) && mbar_wait(bar_sread(t), j & 1, (0x12u << 24) | (6u << 16) | j);
          if (ok) ok = issue_s(t, j + 1, true, 1);
        }
        if (ok) ok = issue_pv(t, j);                          // needs P_t(j): the softmax of tile t has consumed S_t(j)
        if (ok && has_next) ok = issue_s(t, j + 1, true, 2);  // executes after P_t(j) has been read (in-order pipe)
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
    // ------------------------------ softmax + epilogue (tile A: warps 0-3, tile B: warps 4-7) ------------------------------
    const int t = warp >> 2;
    const int r = (warp & 3) * 32 + lane;  // row inside the tile = TMEM lane
    const int row0 = qb * 2 * kBM + t * kBM;
    const int row = row0 + r;
    const int nt = n_t[t];
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tm_s = tmem_base + lane_sel + t * kBN;
    const uint32_t tm_o = tmem_base + lane_sel + 256 + t * kD;
    const bool row_live = row < Lq;
    const bool scaled = a.scale_q != nullptr;
    const float sq = (scaled && row_live) ? __ldg(a.scale_q + (static_cast<int64_t>(b) * a.Hq + h) * Lq + row) : 1.f;
    const float qs = __fmul_rn(a.qk_scale, sq);
    const float* skg = scaled ? a.scale_k + (static_cast<int64_t>(b) * a.Hkv + hk) * Lk : nullptr;
    const int limit = a.causal ? min(row + shift, Lk - 1) : Lk - 1;  // last visible key of this row
    float* sk = sk_ptr + t * kBN;
    float m_used = -1e38f, l = 0.f;
    bool ok = true;

    auto s_value = [](uint32_t raw) -> float {
      if constexpr (QK == kQkInt8) return __int2float_rn(static_cast<int>(raw));
      else if constexpr (kSAcc16) return __half2float(__ushort_as_half(static_cast<unsigned short>(raw & 0xFFFFu)));
      else return __uint_as_float(raw);
    };
    auto o_value = [](uint32_t raw) -> float {
      if constexpr (kOAcc16) return __half2float(__ushort_as_half(static_cast<unsigned short>(raw & 0xFFFFu)));
      else return __uint_as_float(raw);
    };
    auto o_raw = [](float v) -> uint32_t {
      if constexpr (kOAcc16) return static_cast<uint32_t>(__half_as_ushort(__float2half_rn(v)));
      else return __float_as_uint(v);
    };

    for (int j = 0; j < nt; ++j) {
      long long* tr = (a.trace && blockIdx.x == 0 && (warp & 3) == 0 && lane == 0 && j < 32) ? a.trace + (t * 32 + j) * 8 : nullptr;
      if (tr) tr[0] = clock64();
      if (scaled) {
        // stage the tile's key scales (one per thread of this group), 0 beyond the sequence
        const int col = j * kBN + r;
        const float v = col < Lk ? __ldg(skg + col) : 0.f;
        asm volatile("bar.sync %0, 128;" ::"r"(1 + t) : "memory");  // everyone is done with the previous tile's scales
        sk[r] = v;
        asm volatile("bar.sync %0, 128;" ::"r"(1 + t) : "memory");
      }
      // A wait that runs out does not leave the loop: the four warps of the group meet at the named
      // barriers above every iteration, so a warp that left alone would strand the other three.
      // It stops waiting instead, keeps arriving, and its rows are written as zeros at the end.
      if (ok && !mbar_wait(bar_sfull(t), j & 1, (0x13u << 24) | (1u << 16) | j)) ok = false;
      tc_fence_after();
      if (tr) tr[1] = clock64();
      const int col0 = j * kBN;
      const bool need_mask = col0 + kBN - 1 > min(row0 + shift, Lk - 1) && (a.causal || col0 + kBN > Lk);

      // ---- the whole score row: four loads in flight, one wait ----
      uint32_t raw[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tm_s + c * 32, raw[c]);
      tc_wait_ld();
      // from here on the score region may be overwritten: columns 64..127 by the next key tile's scores
      // (the MMA warp waits for this signal), columns 0..63 with P
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_sread(t));
      float x[4][32];
      // independent partial maxima / sums per 32-column chunk: one serial chain over the whole row
      // would cost ~4 cycles per link and is exactly what a latency-bound softmax thread cannot afford
      float xm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      auto scale_and_max = [&](auto masked) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int i4 = 0; i4 < 8; ++i4) {
            float kk[4] = {1.f, 1.f, 1.f, 1.f};
            if (scaled) {
              const float4 k4 = *reinterpret_cast<const float4*>(sk + c * 32 + i4 * 4);
              kk[0] = k4.x; kk[1] = k4.y; kk[2] = k4.z; kk[3] = k4.w;
            }
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
              const int i = i4 * 4 + e;
              float v0 = s_value(raw[c][i]), v1 = s_value(raw[c][i + 1]);
              if (scaled) f2_unpack(f2_mul(f2_pack(v0, v1), f2_pack(kk[e], kk[e + 1])), v0, v1);
              if (decltype(masked)::value && col0 + c * 32 + i > limit) v0 = -INFINITY;
              if (decltype(masked)::value && col0 + c * 32 + i + 1 > limit) v1 = -INFINITY;
              x[c][i] = v0;
              x[c][i + 1] = v1;
            }
            xm[c] = max3(xm[c], max3(x[c][i4 * 4], x[c][i4 * 4 + 1], x[c][i4 * 4 + 2]), x[c][i4 * 4 + 3]);
          }
        }
      };
      if (need_mask) scale_and_max(std::true_type{}); else scale_and_max(std::false_type{});
      const float xmax = fmaxf(fmaxf(xm[0], xm[1]), fmaxf(xm[2], xm[3]));
      if (tr) tr[2] = clock64();
      // qs >= 0 (absmax scales), so max(qs * x) = qs * max(x); a fully masked row keeps the old maximum
      const float mt = fmaxf(m_used, xmax == -INFINITY ? -INFINITY : qs * xmax);
      // lazy rescale, decided per warp so the TMEM traffic stays warp-collective
      const bool grow = mt > m_used + kLazyRescale;
      const bool rescale = __any_sync(0xffffffffu, grow) || j == 0;
      if (rescale) {
        const float alpha = fast_exp2(m_used - mt);
        m_used = mt;
        l *= alpha;
        if (j > 0) {
          // O may only be touched once the previous P*V of this tile has retired
          if (ok && !mbar_wait(bar_pvdone(t), (j - 1) & 1, (0x13u << 24) | (2u << 16) | j)) ok = false;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld32(tm_o + c * 32, o);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = o_raw(o_value(o[i]) * alpha);
            tmem_st32(tm_o + c * 32, o);
          }
        }
      }
      // ---- P = exp2(qs * x - max), row sum, 16-bit P back into TMEM ----
      if (tr) tr[3] = clock64();
      uint64_t rs2[4] = {f2_pack(0.f, 0.f), f2_pack(0.f, 0.f), f2_pack(0.f, 0.f), f2_pack(0.f, 0.f)};
      const uint64_t qs2 = f2_pack(qs, qs), negm2 = f2_pack(-m_used, -m_used);
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        uint32_t pk[32];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = c2 * 2 + cc;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint64_t t2 = f2_fma(qs2, f2_pack(x[c][i], x[c][i + 1]), negm2);
            float p0, p1;
            // one pair in kPolyPeriod takes the polynomial route, the others the special-function unit
            if (kPolyPeriod > 0 && ((i >> 1) % (kPolyPeriod > 0 ? kPolyPeriod : 1)) == 0) {
              exp2_poly_pair(t2, p0, p1);
            } else {
              float t0, t1;
              f2_unpack(t2, t0, t1);
              p0 = fast_exp2(t0);
              p1 = fast_exp2(t1);
            }
            rs2[c] = f2_add(rs2[c], f2_pack(p0, p1));
            pk[cc * 16 + (i >> 1)] = pack16x2<VT>(p0, p1);
          }
        }
        tmem_st32(tm_s + c2 * 32, pk);
      }
      float rs0, rs1;
      f2_unpack(f2_add(f2_add(rs2[0], rs2[1]), f2_add(rs2[2], rs2[3])), rs0, rs1);
      l += rs0 + rs1;
      tc_wait_st();
      if (tr) tr[4] = clock64();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_pready(t));
      if (tr) tr[5] = clock64();
    }

    // epilogue: O / l -> 16-bit output
    if (nt > 0 && ok) ok = mbar_wait(bar_pvdone(t), (nt - 1) & 1, (0x13u << 24) | (4u << 16));
    tc_fence_after();
    OutT* orow = static_cast<OutT*>(a.o) + (a.q_offsets ? 0 : b * a.o_sb) + static_cast<int64_t>(q_start + row) * a.o_sl + h * a.o_sh;
    // a row that sees no key at all is written as zeros (its masked probabilities are 0 from the
    // special-function unit but 2^-126 from the polynomial route, so the row sum cannot tell)
    const bool has_sum = l > 0.f && nt > 0 && ok && limit >= 0;
    const float inv_guard = has_sum ? l : 1.f;
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
          for (int e = 0; e < 8; ++e) f[e] = has_sum ? __fdiv_rn(o_value(o[i + e]), inv_guard) : 0.f;
          *reinterpret_cast<uint4*>(orow + c * 32 + i) =
              make_uint4(pack16x2<VT>(f[0], f[1]), pack16x2<VT>(f[2], f[3]), pack16x2<VT>(f[4], f[5]), pack16x2<VT>(f[6], f[7]));
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

// ---- host side shared by the entry points ----------------------------------------------------
struct AttnProblem {
  const void *q, *k, *v;
  void* o;
  const float *scale_q, *scale_k;
  const int32_t *q_offsets, *kv_offsets;  // packed sequences (both or neither)
  int qk_kind, v_dtype, acc16;
  int64_t B, Lq, Lk;                      // packed: Lq = longest query sequence, Lk unused
  int64_t Lq_total, Lk_total;             // packed: rows of the packed tensors
  int64_t Hq, Hkv, D;
  int64_t q_strides[3], k_strides[3], v_strides[3], o_strides[3];  // batch, seq, head (elements)
  int causal;
  long long* trace;
};

template <int QK, int VT, int ACC16>
int launch_attn(const AttnProblem& p, cudaStream_t st) {
  using QI = QkInfo<QK>;
  const bool packed = p.q_offsets != nullptr;
  // [B, L, H, D] seen by TMA as (D, H, L, B), strides in bytes for H, L, B; a packed tensor is one batch
  auto make = [&](CUtensorMap* m, const void* ptr, int64_t L, int64_t H, const int64_t* s, int elem, uint32_t box_d, uint32_t box_rows,
                  CUtensorMapDataType dt) {
    const uint64_t nb = packed ? 1 : static_cast<uint64_t>(p.B);
    const uint64_t dims[4] = {static_cast<uint64_t>(p.D), static_cast<uint64_t>(H), static_cast<uint64_t>(L), nb};
    const uint64_t batch_stride = packed ? static_cast<uint64_t>(s[1]) * static_cast<uint64_t>(L) : static_cast<uint64_t>(s[0]);
    const uint64_t str[3] = {static_cast<uint64_t>(s[2] * elem), static_cast<uint64_t>(s[1] * elem), batch_stride * elem};
    const uint32_t box[4] = {box_d, 1, box_rows, 1};
    return make_tmap_4d(m, dt, ptr, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
  };
  const CUtensorMapDataType dt16 = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;  // any 16-bit type: TMA only moves the bytes
  CUtensorMap tm_q, tm_k, tm_v;
  int rc;
  const int64_t lq_rows = packed ? p.Lq_total : p.Lq, lk_rows = packed ? p.Lk_total : p.Lk;
  if constexpr (QI::kElemBytes == 1) {
    if ((rc = make(&tm_q, p.q, lq_rows, p.Hq, p.q_strides, 1, 128, kBM, CU_TENSOR_MAP_DATA_TYPE_UINT8)) != GNK_OK) return rc;
    if ((rc = make(&tm_k, p.k, lk_rows, p.Hkv, p.k_strides, 1, 128, kBN, CU_TENSOR_MAP_DATA_TYPE_UINT8)) != GNK_OK) return rc;
  } else {
    if ((rc = make(&tm_q, p.q, lq_rows, p.Hq, p.q_strides, 2, 64, kBM, dt16)) != GNK_OK) return rc;
    if ((rc = make(&tm_k, p.k, lk_rows, p.Hkv, p.k_strides, 2, 64, kBN, dt16)) != GNK_OK) return rc;
  }
  if ((rc = make(&tm_v, p.v, lk_rows, p.Hkv, p.v_strides, 2, 64, kBN, dt16)) != GNK_OK) return rc;

  AttnArgs a{};
  a.trace = p.trace;
  a.Lq = static_cast<int>(p.Lq);
  a.Lk = static_cast<int>(p.Lk);
  a.Hq = static_cast<int>(p.Hq);
  a.Hkv = static_cast<int>(p.Hkv);
  a.group = static_cast<int>(p.Hq / p.Hkv);
  a.causal = p.causal != 0;
  a.q_blocks = static_cast<int>((p.Lq + 2 * kBM - 1) / (2 * kBM));
  a.qk_scale = static_cast<float>((1.0 / sqrt(static_cast<double>(p.D))) * 1.44269504);  // as the reference folds it
  a.scale_q = p.scale_q;
  a.scale_k = p.scale_k;
  a.o = p.o;
  a.o_sb = p.o_strides[0];
  a.o_sl = p.o_strides[1];
  a.o_sh = p.o_strides[2];
  a.q_offsets = p.q_offsets;
  a.kv_offsets = p.kv_offsets;

  dim3 grid(static_cast<unsigned>(p.Hq), static_cast<unsigned>(a.q_blocks), static_cast<unsigned>(p.B));
  auto kern = attn_fwd_kernel<QK, VT, ACC16>;
  constexpr int kSmem = smem_bytes<QK>();
  GNK_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  kern<<<grid, kThreads, kSmem, st>>>(tm_q, tm_k, tm_v, a);
  GNK_LAUNCH_OK();
  return GNK_OK;
}

// argument checks shared by the entry points
inline int check_attn(const AttnProblem& p) {
  if (!p.q || !p.k || !p.v || !p.o) return GNK_ERR_BAD_ARG;
  if (p.B <= 0 || p.Lq <= 0 || p.Hq <= 0 || p.Hkv <= 0) return GNK_ERR_BAD_ARG;
  if (!p.q_offsets && p.Lk <= 0) return GNK_ERR_BAD_ARG;
  if ((p.q_offsets == nullptr) != (p.kv_offsets == nullptr)) return GNK_ERR_BAD_ARG;
  if ((p.scale_q == nullptr) != (p.scale_k == nullptr)) return GNK_ERR_BAD_ARG;
  if (p.v_dtype != GNK_BF16 && p.v_dtype != GNK_F16) return GNK_ERR_BAD_ARG;
  if (p.acc16 < 0 || p.acc16 > 3) return GNK_ERR_BAD_ARG;
  if (p.D != kD) return GNK_ERR_UNSUPPORTED;
  if (p.Hq % p.Hkv != 0) return GNK_ERR_BAD_SHAPE;
  if (p.B > 65535 || (p.Lq + 2 * kBM - 1) / (2 * kBM) > 65535) return GNK_ERR_TOO_LARGE;
  if (p.Lq > (1ll << 30) || p.Lk > (1ll << 30) || p.Lq_total > (1ll << 30) || p.Lk_total > (1ll << 30)) return GNK_ERR_TOO_LARGE;
  if ((p.o_strides[0] | p.o_strides[1] | p.o_strides[2]) & 7) return GNK_ERR_BAD_ALIGN;
  if (!aligned16(p.o)) return GNK_ERR_BAD_ALIGN;
  return check_arch();
}

}  // namespace attn
}  // namespace gnk

// tcgen05 GEMM family: C[M,N] = A[M,K] * Bt[N,K]^T for BF16, INT8, E4M3 (dense kinds) and
// MXFP8 / NVFP4 (block-scaled kinds), with fused epilogues (bf16 cast, alpha, row scales +
// bias, raw int32).
//
// One persistent, warp-specialised kernel template:
//   warps 0-3  epilogue: TMEM -> registers (tcgen05.ld, lane = row) -> scale/cast -> global
//   warp  4    producer: one lane issues the TMA loads of a K stage (A, B, and for the
//              block-scaled kinds the 512-byte scale-factor atoms) onto a full barrier
//   warp  5    MMA: one lane copies scale atoms smem -> TMEM (tcgen05.cp) and issues four
//              tcgen05.mma per stage (32 bytes of K each); tcgen05.commit frees the stage
// Accumulators live in TMEM, two in flight so the epilogue of tile i overlaps the main
// loop of tile i+1.  When two BN-wide accumulators plus the scale columns do not fit the
// 512 TMEM columns (block-scaled, BN = 256) the two accumulators overlap by a few columns:
// the epilogue drains the shared columns first and releases them through a third barrier.
// CG = 2 pairs two CTAs (a cluster) on a 256 x BN tile: each loads its 128 rows of A and
// its half of B, CTA 0 issues cta_group::2 MMAs for both, and completion is multicast to
// the barriers of both CTAs.  No TMA load here uses cluster multicast.
// Every barrier wait is bounded; a wait that runs out sets the device status word and the
// role leaves its loop, after which the CTA tears down normally.
#include "gnk_common.cuh"

namespace gnk {
namespace {

enum Epi { EPI_BF16 = 0, EPI_ROWSCALED = 1, EPI_I32 = 2 };
constexpr int kTraceEvents = 256;  // stages recorded per (CTA, role) when tracing

template <MmaKind K> struct KindInfo;
template <> struct KindInfo<MmaKind::F16> { static constexpr bool kBlockScaled = false; static constexpr int kSfPerStage = 0; };
template <> struct KindInfo<MmaKind::I8> { static constexpr bool kBlockScaled = false; static constexpr int kSfPerStage = 0; };
template <> struct KindInfo<MmaKind::F8F6F4> { static constexpr bool kBlockScaled = false; static constexpr int kSfPerStage = 0; };
// scale bytes per operand row per K stage: 128 fp8 / 32 = 4, 256 fp4 / 16 = 16
template <> struct KindInfo<MmaKind::MXF8F6F4> { static constexpr bool kBlockScaled = true; static constexpr int kSfPerStage = 4; };
template <> struct KindInfo<MmaKind::MXF4NVF4> { static constexpr bool kBlockScaled = true; static constexpr int kSfPerStage = 16; };

struct GemmArgs {
  int M, N;
  int k_iters;           // K stages of 128 bytes
  int tiles_m, tiles_n;  // cluster tiles: (128 * CG) x BN
  void* C;
  int64_t ldc;
  const float* scale_a;
  const float* scale_b;
  const float* bias;
  float alpha;
  int vec_ok;  // C rows 16-byte aligned: vector stores allowed
  long long* trace;  // debug: per-stage clock64 stamps of CTAs 0 and 1 (null = off)
};

template <MmaKind KIND, int BN, int CG>
struct Cfg {
  using KI = KindInfo<KIND>;
  static constexpr int kABytes = 128 * 128;
  static constexpr int kBBytes = (BN / CG) * 128;
  static constexpr int kSfAtomBytes = 128 * KI::kSfPerStage;           // one 128-row group, one stage
  static constexpr int kSfaBytes = kSfAtomBytes;
  static constexpr int kSfbGroups = BN >= 128 ? BN / 128 : 1;
  static constexpr int kSfbBytes = kSfAtomBytes * kSfbGroups;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kSmemBudget = 227 * 1024 - 2048;                // barriers + alignment slack
  static constexpr int kStagesRaw = kSmemBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kSmemBytes = kStages * kStageBytes + 2048;
  // TMEM columns
  static constexpr int kSfaCols = KI::kSfPerStage;                      // 4 bytes per column, 128 rows -> 4 columns per 4 scales
  static constexpr int kSfbCols = KI::kSfPerStage * kSfbGroups;
  static constexpr int kSfCols = KI::kBlockScaled ? ((kSfaCols + kSfbCols + 15) / 16) * 16 : 0;
  static constexpr bool kOverlap = 2 * BN + kSfCols > 512;
  static constexpr int kAccStride = kOverlap ? (512 - kSfCols - BN) : BN;
  static constexpr int kOverlapCols = BN - kAccStride;                  // 0 when the accumulators are disjoint
  static constexpr int kSfBase = kOverlap ? 512 - kSfCols : 2 * BN;
  static constexpr int kTmemCols = 512;
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int kGroup = 8;
  const int width = kGroup * tiles_n;
  const int gid = t / width;
  const int first = gid * kGroup;
  const int gsz = min(tiles_m - first, kGroup);
  const int in = t - gid * width;
  tm = first + in % gsz;
  tn = in / gsz;
}

// ---- epilogue: W (16 or 32) consecutive accumulator columns of one row ------------------
template <MmaKind KIND, int EPI, int W>
__device__ __forceinline__ void store_cols(const uint32_t* r, const GemmArgs& g, int row, int col0, float sa) {
  if (row >= g.M || col0 >= g.N) return;
  const bool full = (col0 + W <= g.N) && g.vec_ok;
  if constexpr (EPI == EPI_I32) {
    int32_t* dst = static_cast<int32_t*>(g.C) + static_cast<int64_t>(row) * g.ldc + col0;
    if (full) {
#pragma unroll
      for (int i = 0; i < W; i += 4) *reinterpret_cast<uint4*>(dst + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
    } else {
      for (int i = 0; i < W && col0 + i < g.N; ++i) dst[i] = static_cast<int32_t>(r[i]);
    }
  } else {
    float f[W];
#pragma unroll
    for (int i = 0; i < W; ++i) {
      float v = KIND == MmaKind::I8 ? static_cast<float>(static_cast<int32_t>(r[i])) : __uint_as_float(r[i]);
      if constexpr (EPI == EPI_ROWSCALED) {
        // order fixed by the reference epilogue: * scale_A[m], * scale_B[n], + bias[n], each rounded
        const int c = min(col0 + i, g.N - 1);
        if (g.scale_a) v = __fmul_rn(v, sa);
        if (g.scale_b) v = __fmul_rn(v, __ldg(g.scale_b + c));
        if (g.bias) v = __fadd_rn(v, __ldg(g.bias + c));
      } else if constexpr (KIND == MmaKind::MXF4NVF4) {
        v = __fmul_rn(v, g.alpha);
      }
      f[i] = v;
    }
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(g.C) + static_cast<int64_t>(row) * g.ldc + col0;
    if (full) {
#pragma unroll
      for (int i = 0; i < W; i += 8)
        *reinterpret_cast<uint4*>(dst + i) = make_uint4(pack_bf16x2(f[i], f[i + 1]), pack_bf16x2(f[i + 2], f[i + 3]),
                                                        pack_bf16x2(f[i + 4], f[i + 5]), pack_bf16x2(f[i + 6], f[i + 7]));
    } else {
      for (int i = 0; i < W && col0 + i < g.N; ++i) dst[i] = __float2bfloat16_rn(f[i]);
    }
  }
}

// drains accumulator columns [c0, c1) (multiples of 16) of this warp's 32 rows
template <MmaKind KIND, int EPI>
__device__ __forceinline__ void drain_cols(uint32_t taddr_row, int c0, int c1, const GemmArgs& g, int row, int ncol0,
                                           float sa) {
  int c = c0;
  for (; c + 32 <= c1; c += 32) {
    uint32_t r[32];
    tmem_ld32(taddr_row + c, r);
    tc_wait_ld();
    store_cols<KIND, EPI, 32>(r, g, row, ncol0 + c, sa);
  }
  for (; c + 16 <= c1; c += 16) {
    uint32_t r[16];
    tmem_ld16(taddr_row + c, r);
    tc_wait_ld();
    store_cols<KIND, EPI, 16>(r, g, row, ncol0 + c, sa);
  }
}

template <MmaKind KIND, int BN, int CG, int EPI>
__global__ void __cluster_dims__(CG, 1, 1) __launch_bounds__(192, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                const __grid_constant__ CUtensorMap tm_sfa, const __grid_constant__ CUtensorMap tm_sfb,
                const GemmArgs g) {
  using C = Cfg<KIND, BN, CG>;
  constexpr bool kBS = C::KI::kBlockScaled;
  constexpr int S = C::kStages;
  constexpr int kInner = KIND == MmaKind::F16 ? 64 : 128;  // tensor-map elements per 128-byte K stage

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // [stage][A | B | SFA | SFB]; A and B stage buffers stay 1024-byte aligned (sizes are multiples of 1024... SF after them)
  auto stage_a = [&](int s) { return smem_base + s * (C::kABytes + C::kBBytes); };
  auto stage_b = [&](int s) { return stage_a(s) + C::kABytes; };
  const uint32_t sf_base = smem_base + S * (C::kABytes + C::kBBytes);
  auto stage_sfa = [&](int s) { return sf_base + s * (C::kSfaBytes + C::kSfbBytes); };
  auto stage_sfb = [&](int s) { return stage_sfa(s) + C::kSfaBytes; };
  const uint32_t bar_base = sf_base + S * (C::kSfaBytes + C::kSfbBytes);
  auto bar_full = [&](int s) { return bar_base + 8 * s; };
  auto bar_empty = [&](int s) { return bar_base + 8 * (S + s); };
  auto bar_tfull = [&](int s) { return bar_base + 8 * (2 * S + s); };
  auto bar_tempty = [&](int s) { return bar_base + 8 * (2 * S + 2 + s); };
  const uint32_t bar_partial = bar_base + 8 * (2 * S + 4);
  const uint32_t tmem_slot = bar_base + 8 * (2 * S + 5);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int trace_it = 0;
  const uint32_t cta_rank = CG == 2 ? cluster_ctarank() : 0u;
  const int cluster_id = blockIdx.x / CG;
  const int num_clusters = gridDim.x / CG;
  const int num_tiles = g.tiles_m * g.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full(s), CG);  // one expect_tx arrival per CTA of the pair
      mbar_init(bar_empty(s), 1);  // one tcgen05.commit
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull(s), 1);
      mbar_init(bar_tempty(s), 4 * CG);  // one arrival per epilogue warp of every CTA
    }
    mbar_init(bar_partial, 4 * CG);
    fence_mbar_init();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
    if constexpr (kBS) {
      tma_prefetch_desc(&tm_sfa);
      tma_prefetch_desc(&tm_sfb);
    }
  }
  if (warp == 5) {
    tmem_alloc<CG>(tmem_slot, C::kTmemCols);
    tmem_relinquish<CG>();
  }
  tc_fence_before();
  if constexpr (CG == 2) cluster_sync_all(); else __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  // Producer and MMA warps run their loops warp-uniformly (all 32 lanes wait on the barriers and
  // compute addresses and descriptors, which keeps those values in uniform registers); one
  // elected lane executes the TMA / tcgen05 issue instructions.
  if (warp == 4) {
    // ------------------------------ producer ------------------------------
    const bool leader = elect_one();
    uint32_t stage = 0, parity = 1;
    bool ok = true;
    // both CTAs of a pair count their bytes on CTA 0's barrier
    const uint32_t full0 = CG == 2 ? map_to_cta(bar_full(0), 0) : bar_full(0);
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
      int tm, tn;
      tile_coords(t, g.tiles_m, g.tiles_n, tm, tn);
      const int a_row = (tm * CG + cta_rank) * 128;
      const int b_row = tn * BN + cta_rank * (BN / CG);
      const int sfa_row = tm * CG + cta_rank;
      const int sfb_row = (tn * BN) / 128;
      for (int k = 0; k < g.k_iters; ++k) {
        const long long tr0 = g.trace ? clock64() : 0;
        if (!mbar_wait(bar_empty(stage), parity, (1u << 24) | (1u << 16) | stage)) { ok = false; break; }
        const long long tr1 = g.trace ? clock64() : 0;
        const uint32_t full = full0 + 8 * stage;
        const uint32_t sa = stage_a(stage), sb = stage_b(stage);
        if (leader) {
          if constexpr (CG == 2) {
            mbar_expect_tx_cluster(full, C::kStageBytes);
            tma_load_2d_pair(sa, &tm_a, full, k * kInner, a_row);
            tma_load_2d_pair(sb, &tm_b, full, k * kInner, b_row);
            if constexpr (kBS) {
              tma_load_2d_pair(stage_sfa(stage), &tm_sfa, full, k * (C::kSfAtomBytes / 8), sfa_row);
              tma_load_2d_pair(stage_sfb(stage), &tm_sfb, full, k * (C::kSfAtomBytes / 8), sfb_row);
            }
          } else {
            mbar_expect_tx(full, C::kStageBytes);
            tma_load_2d(sa, &tm_a, full, k * kInner, a_row);
            tma_load_2d(sb, &tm_b, full, k * kInner, b_row);
            if constexpr (kBS) {
              tma_load_2d(stage_sfa(stage), &tm_sfa, full, k * (C::kSfAtomBytes / 8), sfa_row);
              tma_load_2d(stage_sfb(stage), &tm_sfb, full, k * (C::kSfAtomBytes / 8), sfb_row);
            }
          }
          if (g.trace && blockIdx.x < 2 && trace_it < kTraceEvents) {
            long long* tp = g.trace + ((blockIdx.x * 2 + 0) * kTraceEvents + trace_it) * 3;
            tp[0] = tr0; tp[1] = tr1; tp[2] = clock64();
          }
        }
        ++trace_it;
        __syncwarp();
        if (++stage == S) { stage = 0; parity ^= 1; }
      }
    }
  } else if (warp == 5) {
    // ------------------------------ MMA issuer ------------------------------
    if (cta_rank == 0) {
      const bool leader = elect_one();
      uint32_t stage = 0, parity = 0, acc = 0, acc_parity = 1, iter = 0;
      bool ok = true;
      constexpr uint32_t kIdesc = KIND == MmaKind::F16      ? idesc_dense(1, 1, 1, 128 * CG, BN)
                                  : KIND == MmaKind::I8     ? idesc_dense(2, 1, 1, 128 * CG, BN)
                                  : KIND == MmaKind::F8F6F4 ? idesc_dense(1, 0, 0, 128 * CG, BN)
                                  : KIND == MmaKind::MXF8F6F4 ? idesc_block_scaled(0, 1, 128 * CG, BN)
                                                              : idesc_block_scaled(1, 0, 128 * CG, BN);
      const uint32_t sf_tmem = tmem_base + C::kSfBase;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++iter) {
        if (!mbar_wait(bar_tempty(acc), acc_parity, (2u << 24) | (2u << 16) | acc)) { ok = false; break; }
        if constexpr (C::kOverlap) {
          if (iter > 0 && !mbar_wait(bar_partial, (iter - 1) & 1, (2u << 24) | (3u << 16))) { ok = false; break; }
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * C::kAccStride;
        for (int k = 0; k < g.k_iters; ++k) {
          const long long tr0 = g.trace ? clock64() : 0;
          if (!mbar_wait(bar_full(stage), parity, (2u << 24) | (4u << 16) | stage)) { ok = false; break; }
          const long long tr1 = g.trace ? clock64() : 0;
          tc_fence_after();
          const uint64_t a_desc = sdesc_k128(stage_a(stage));
          const uint64_t b_desc = sdesc_k128(stage_b(stage));
          const uint64_t sfa_desc = sdesc_sf(stage_sfa(stage));
          const uint64_t sfb_desc = sdesc_sf(stage_sfb(stage));
          const uint32_t empty = bar_empty(stage);
          if (leader) {
            if constexpr (kBS) {
              constexpr int kAtoms = C::kSfAtomBytes / 512;  // atoms per 128-row group per stage: 1 (mxfp8) or 4 (nvfp4)
#pragma unroll
              for (int a = 0; a < kAtoms; ++a) {
                tc_cp_sf<CG>(sf_tmem + 4 * a, sfa_desc + (512 >> 4) * a);
#pragma unroll
                for (int j = 0; j < C::kSfbGroups; ++j)
                  tc_cp_sf<CG>(sf_tmem + C::kSfaCols + (a * C::kSfbGroups + j) * 4,
                               sfb_desc + ((j * C::kSfAtomBytes + 512 * a) >> 4));
              }
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint32_t accum = (k | kk) != 0;
              if constexpr (!kBS) {
                tc_mma<KIND, CG>(d_tmem, a_desc + 2 * kk, b_desc + 2 * kk, kIdesc, accum);
              } else if constexpr (KIND == MmaKind::MXF8F6F4) {
                // the four K steps of a stage read bytes 0..3 of the same scale columns (scale ids in the descriptor)
                tc_mma_bs<KIND, CG>(d_tmem, a_desc + 2 * kk, b_desc + 2 * kk, kIdesc | (kk << 4) | (kk << 29), sf_tmem,
                                    sf_tmem + C::kSfaCols, accum);
              } else {
                // each K step (64 fp4) has its own scale columns (4 scales = one 32-bit column per row group)
                tc_mma_bs<KIND, CG>(d_tmem, a_desc + 2 * kk, b_desc + 2 * kk, kIdesc, sf_tmem + 4 * kk,
                                    sf_tmem + C::kSfaCols + kk * C::kSfbGroups * 4, accum);
              }
            }
            if constexpr (CG == 2) tc_commit_pair(empty, 3); else tc_commit<1>(empty);
            if (g.trace && blockIdx.x < 2 && trace_it < kTraceEvents) {
              long long* tp = g.trace + ((blockIdx.x * 2 + 1) * kTraceEvents + trace_it) * 3;
              tp[0] = tr0; tp[1] = tr1; tp[2] = clock64();
            }
          }
          ++trace_it;
          __syncwarp();
          if (++stage == S) { stage = 0; parity ^= 1; }
        }
        if (!ok) break;
        if (leader) {
          if constexpr (CG == 2) tc_commit_pair(bar_tfull(acc), 3); else tc_commit<1>(bar_tfull(acc));
        }
        __syncwarp();
        acc ^= 1;
        if (acc == 0) acc_parity ^= 1;
      }
    }
  } else {
    // ------------------------------ epilogue (warps 0-3) ------------------------------
    uint32_t acc = 0, parity = 0;
    const uint32_t tempty0 = CG == 2 ? map_to_cta(bar_tempty(0), 0) : bar_tempty(0);
    const uint32_t partial = CG == 2 ? map_to_cta(bar_partial, 0) : bar_partial;
    bool ok = true;
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
      int tm, tn;
      tile_coords(t, g.tiles_m, g.tiles_n, tm, tn);
      if (!mbar_wait(bar_tfull(acc), parity, (3u << 24) | (5u << 16) | acc)) { ok = false; break; }
      tc_fence_after();
      const int row = (tm * CG + cta_rank) * 128 + warp * 32 + lane;
      const int ncol0 = tn * BN;
      const float sa = (EPI == EPI_ROWSCALED && g.scale_a && row < g.M) ? __ldg(g.scale_a + row) : 1.f;
      const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + acc * C::kAccStride;
      if constexpr (C::kOverlap) {
        // the columns shared with the other accumulator go first and are released at once
        const int o0 = acc == 0 ? C::kAccStride : 0;
        const int o1 = o0 + C::kOverlapCols;
        drain_cols<KIND, EPI>(taddr_row, o0, o1, g, row, ncol0, sa);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(partial);
        if (acc == 0) drain_cols<KIND, EPI>(taddr_row, 0, o0, g, row, ncol0, sa);
        else drain_cols<KIND, EPI>(taddr_row, o1, BN, g, row, ncol0, sa);
      } else {
        drain_cols<KIND, EPI>(taddr_row, 0, BN, g, row, ncol0, sa);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty0 + 8 * acc);
      acc ^= 1;
      if (acc == 0) parity ^= 1;
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  if constexpr (CG == 2) cluster_sync_all(); else __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc<CG>(tmem_base, C::kTmemCols);
  }
}

long long* g_trace = nullptr;  // test hook (gnk_debug_trace): device buffer of 2*2*256*3 int64
int g_max_clusters = 0;  // test hook (gnk_debug_max_clusters): cap on the persistent grid, 0 = none

template <MmaKind KIND>
struct ElemInfo {
  // bytes per K element as a rational: bf16 2/1, 8-bit 1/1, fp4 1/2
  static constexpr int kNum = KIND == MmaKind::F16 ? 2 : 1;
  static constexpr int kDen = KIND == MmaKind::MXF4NVF4 ? 2 : 1;
  static constexpr int kSfBlock = KIND == MmaKind::MXF8F6F4 ? 32 : 16;
};

template <MmaKind KIND, int BN, int CG, int EPI>
int launch(const void* A, int64_t lda, const void* Bt, int64_t ldb, const uint8_t* SFA, const uint8_t* SFB,
           GemmArgs g, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
  using C = Cfg<KIND, BN, CG>;
  using EI = ElemInfo<KIND>;
  const int64_t k_bytes = K * EI::kNum / EI::kDen;
  const int64_t lda_b = lda * EI::kNum;  // ld counts stored elements (bytes for packed fp4)
  const int64_t ldb_b = ldb * EI::kNum;
  CUtensorMap tm_a, tm_b, tm_sfa, tm_sfb;
  const CUtensorMapDataType dt = KIND == MmaKind::F16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const uint64_t k_elems_tm = KIND == MmaKind::F16 ? K : k_bytes;  // tensor-map inner extent in its own elements
  const uint32_t box_inner = KIND == MmaKind::F16 ? 64 : 128;
  int rc = make_tmap_2d(&tm_a, dt, A, M, k_elems_tm, lda_b, 128, box_inner, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != GNK_OK) return rc;
  rc = make_tmap_2d(&tm_b, dt, Bt, N, k_elems_tm, ldb_b, BN / CG, box_inner, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != GNK_OK) return rc;
  if constexpr (C::KI::kBlockScaled) {
    // swizzled scale buffer seen as [row groups of 128][K/(4 scales) atoms of 512 bytes], in 8-byte words
    const int64_t ks = (K + EI::kSfBlock - 1) / EI::kSfBlock;
    const int64_t atoms = (ks + 3) / 4;
    rc = make_tmap_2d(&tm_sfa, CU_TENSOR_MAP_DATA_TYPE_UINT64, SFA, (M + 127) / 128, atoms * 64, atoms * 512, 1,
                      C::kSfAtomBytes / 8, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != GNK_OK) return rc;
    rc = make_tmap_2d(&tm_sfb, CU_TENSOR_MAP_DATA_TYPE_UINT64, SFB, (N + 127) / 128, atoms * 64, atoms * 512,
                      C::kSfbGroups, C::kSfAtomBytes / 8, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != GNK_OK) return rc;
  } else {
    tm_sfa = tm_a;
    tm_sfb = tm_b;
  }
  g.k_iters = static_cast<int>((k_bytes + 127) / 128);
  g.tiles_m = static_cast<int>((M + 128 * CG - 1) / (128 * CG));
  g.tiles_n = static_cast<int>((N + BN - 1) / BN);
  const int tiles = g.tiles_m * g.tiles_n;
  auto kern = gemm_kernel<KIND, BN, CG, EPI>;
  // Persistent grid = the number of clusters that can be resident at once.  For 2-CTA
  // clusters this can be below SMs / 2 (both CTAs must land on one SM pair), and a cluster
  // that does not fit the first wave would run its whole share of tiles after everyone else.
  static int resident[64];  // per instantiation, per device; 0 = not yet queried
  int dev = 0;
  GNK_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return GNK_ERR_UNSUPPORTED;
  if (resident[dev] == 0) {
    GNK_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    int n = num_sms() / CG;
    if (CG > 1) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(static_cast<unsigned>(num_sms() / CG * CG));
      cfg.blockDim = dim3(192);
      cfg.dynamicSmemBytes = C::kSmemBytes;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = CG;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      int q = 0;
      GNK_CUDA_OK(cudaOccupancyMaxActiveClusters(&q, kern, &cfg));
      if (q > 0 && q < n) n = q;
    }
    resident[dev] = n;
  }
  int clusters = resident[dev];
  if (g_max_clusters > 0 && clusters > g_max_clusters) clusters = g_max_clusters;
  if (clusters > tiles) clusters = tiles;
  kern<<<clusters * CG, 192, C::kSmemBytes, st>>>(tm_a, tm_b, tm_sfa, tm_sfb, g);
  GNK_LAUNCH_OK();
  return GNK_OK;
}

// Tile choice: the largest tile that still gives every SM work; 2-CTA 256x256 for big problems.
enum TileSel { T_2x256, T_1x256, T_1x128, T_1x64 };
int g_force_tile = -1;  // test hook (gnk_debug_force_tile)

TileSel pick_tile(int64_t M, int64_t N, bool block_scaled) {
  if (g_force_tile >= 0) return static_cast<TileSel>(g_force_tile);
  const int sms = num_sms();
  auto ctas = [&](int64_t bm, int64_t bn) { return ((M + bm - 1) / bm) * ((N + bn - 1) / bn); };
  if (ctas(256, 256) * 2 >= sms) return T_2x256;
  if (ctas(128, 256) >= sms) return T_1x256;
  if (block_scaled || ctas(128, 128) >= sms) return T_1x128;
  return T_1x64;
}

template <MmaKind KIND, int EPI>
int dispatch_tile(const void* A, int64_t lda, const void* Bt, int64_t ldb, const uint8_t* SFA, const uint8_t* SFB,
                  const GemmArgs& g, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
  constexpr bool kBS = KindInfo<KIND>::kBlockScaled;
  switch (pick_tile(M, N, kBS)) {
    case T_2x256: return launch<KIND, 256, 2, EPI>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K, st);
    case T_1x256: return launch<KIND, 256, 1, EPI>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K, st);
    case T_1x128: return launch<KIND, 128, 1, EPI>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K, st);
    case T_1x64:
      if constexpr (!kBS) return launch<KIND, 64, 1, EPI>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K, st);
      return launch<KIND, 128, 1, EPI>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K, st);
  }
  return GNK_ERR_UNSUPPORTED;
}

int check_common(const void* A, const void* Bt, const void* C, int64_t M, int64_t N, int64_t K, int64_t lda_bytes,
                 int64_t ldb_bytes) {
  if (!A || !Bt || !C || M <= 0 || N <= 0 || K <= 0) return GNK_ERR_BAD_ARG;
  if (M > (1ll << 30) || N > (1ll << 30) || K > (1ll << 30)) return GNK_ERR_TOO_LARGE;
  if (!aligned16(A) || !aligned16(Bt)) return GNK_ERR_BAD_ALIGN;
  if ((lda_bytes & 15) || (ldb_bytes & 15)) return GNK_ERR_BAD_ALIGN;
  return check_arch();
}

GemmArgs base_args(void* C, int64_t ldc, int64_t M, int64_t N, int out_elem_bytes) {
  GemmArgs g{};
  g.M = static_cast<int>(M);
  g.N = static_cast<int>(N);
  g.C = C;
  g.ldc = ldc;
  g.alpha = 1.f;
  g.vec_ok = aligned16(C) && ((ldc * out_elem_bytes) % 16 == 0);
  g.trace = g_trace;
  return g;
}

GNK_DEFINE_STATUS_READER(gemm_status_reader)

}  // namespace
}  // namespace gnk

using namespace gnk;

// Test hook: force a tile configuration (0: 2-CTA 256x256, 1: 128x256, 2: 128x128, 3: 128x64; -1: automatic).
extern "C" int gnk_debug_force_tile(int sel) {
  if (sel < -1 || sel > 3) return GNK_ERR_BAD_ARG;
  g_force_tile = sel;
  return GNK_OK;
}

// Debug: device buffer (2 CTAs x 2 roles x 256 stages x 3 int64 clock stamps) or NULL to stop tracing.
extern "C" int gnk_debug_trace(void* device_buffer) {
  g_trace = static_cast<long long*>(device_buffer);
  return GNK_OK;
}

extern "C" int gnk_debug_max_clusters(int n) {
  g_max_clusters = n < 0 ? 0 : n;
  return GNK_OK;
}

extern "C" int gnk_mm_bf16(const void* A, int64_t lda, const void* Bt, int64_t ldb, void* C, int64_t ldc, int64_t M,
                           int64_t N, int64_t K, gnk_stream_t stream) {
  int rc = check_common(A, Bt, C, M, N, K, lda * 2, ldb * 2);
  if (rc != GNK_OK) return rc;
  if (K % 8 != 0) return GNK_ERR_BAD_SHAPE;
  GemmArgs g = base_args(C, ldc, M, N, 2);
  return dispatch_tile<MmaKind::F16, EPI_BF16>(A, lda, Bt, ldb, nullptr, nullptr, g, M, N, K,
                                               static_cast<cudaStream_t>(stream));
}

extern "C" int gnk_mm_i8(const void* A, int64_t lda, const void* Bt, int64_t ldb, void* C, int64_t ldc, int64_t M,
                         int64_t N, int64_t K, const float* scale_A, const float* scale_B, const float* bias,
                         int out_kind, gnk_stream_t stream) {
  int rc = check_common(A, Bt, C, M, N, K, lda, ldb);
  if (rc != GNK_OK) return rc;
  if (K % 16 != 0) return GNK_ERR_BAD_SHAPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_kind == GNK_OUT_I32) {
    if (scale_A || scale_B || bias) return GNK_ERR_BAD_ARG;
    GemmArgs g = base_args(C, ldc, M, N, 4);
    return dispatch_tile<MmaKind::I8, EPI_I32>(A, lda, Bt, ldb, nullptr, nullptr, g, M, N, K, st);
  }
  if (out_kind != GNK_OUT_BF16) return GNK_ERR_BAD_ARG;
  GemmArgs g = base_args(C, ldc, M, N, 2);
  g.scale_a = scale_A;
  g.scale_b = scale_B;
  g.bias = bias;
  return dispatch_tile<MmaKind::I8, EPI_ROWSCALED>(A, lda, Bt, ldb, nullptr, nullptr, g, M, N, K, st);
}

extern "C" int gnk_mm_f8(const void* A, int64_t lda, const void* Bt, int64_t ldb, void* C, int64_t ldc, int64_t M,
                         int64_t N, int64_t K, const float* scale_A, const float* scale_B, const float* bias,
                         gnk_stream_t stream) {
  int rc = check_common(A, Bt, C, M, N, K, lda, ldb);
  if (rc != GNK_OK) return rc;
  if (K % 16 != 0) return GNK_ERR_BAD_SHAPE;
  GemmArgs g = base_args(C, ldc, M, N, 2);
  g.scale_a = scale_A;
  g.scale_b = scale_B;
  g.bias = bias;
  return dispatch_tile<MmaKind::F8F6F4, EPI_ROWSCALED>(A, lda, Bt, ldb, nullptr, nullptr, g, M, N, K,
                                                       static_cast<cudaStream_t>(stream));
}

extern "C" int gnk_mm_mxfp8(const void* A, int64_t lda, const void* Bt, int64_t ldb, const uint8_t* SFA,
                            const uint8_t* SFB, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                            gnk_stream_t stream) {
  int rc = check_common(A, Bt, C, M, N, K, lda, ldb);
  if (rc != GNK_OK) return rc;
  if (!SFA || !SFB) return GNK_ERR_BAD_ARG;
  if (!aligned16(SFA) || !aligned16(SFB)) return GNK_ERR_BAD_ALIGN;
  if (K % 32 != 0) return GNK_ERR_BAD_SHAPE;
  GemmArgs g = base_args(C, ldc, M, N, 2);
  return dispatch_tile<MmaKind::MXF8F6F4, EPI_BF16>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K,
                                                    static_cast<cudaStream_t>(stream));
}

extern "C" int gnk_mm_nvfp4(const void* A, int64_t lda, const void* Bt, int64_t ldb, const uint8_t* SFA,
                            const uint8_t* SFB, float alpha, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                            gnk_stream_t stream) {
  int rc = check_common(A, Bt, C, M, N, K, lda, ldb);
  if (rc != GNK_OK) return rc;
  if (!SFA || !SFB) return GNK_ERR_BAD_ARG;
  if (!aligned16(SFA) || !aligned16(SFB)) return GNK_ERR_BAD_ALIGN;
  if (K % 32 != 0) return GNK_ERR_BAD_SHAPE;
  GemmArgs g = base_args(C, ldc, M, N, 2);
  g.alpha = alpha;
  return dispatch_tile<MmaKind::MXF4NVF4, EPI_BF16>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K,
                                                    static_cast<cudaStream_t>(stream));
}

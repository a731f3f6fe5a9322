// tcgen05 GEMM kernel template shared by the single-GPU GEMM entry points and the fused
// GEMM + reduce-scatter.  See gnk_gemm.cu for the description of the warp roles.
#pragma once

#include "gnk_quant_math.cuh"

namespace gnk {
namespace gemm {

enum Epi { EPI_BF16 = 0, EPI_ROWSCALED = 1, EPI_I32 = 2, EPI_RS = 3, EPI_GATED = 4 };
constexpr int kMaxWorld = 8;  // ranks of one NVLink domain the reduce-scatter variant addresses
constexpr int kTraceEvents = 256;  // stages recorded per (CTA, role) when tracing
constexpr int kTraceSpanAt = 2 * 2 * kTraceEvents * 3;  // then 4 words: clock64 / globaltimer at entry and exit of CTA 0

template <MmaKind K> struct KindInfo;
template <> struct KindInfo<MmaKind::F16> { static constexpr bool kBlockScaled = false; static constexpr int kSfPerStage = 0; };
template <> struct KindInfo<MmaKind::I8> { static constexpr bool kBlockScaled = false; static constexpr int kSfPerStage = 0; };
template <> struct KindInfo<MmaKind::F8F6F4> { static constexpr bool kBlockScaled = false; static constexpr int kSfPerStage = 0; };
// scale bytes per operand row per K stage: 128 fp8 / 32 = 4, 256 fp4 / 16 = 16
template <> struct KindInfo<MmaKind::MXF8F6F4> { static constexpr bool kBlockScaled = true; static constexpr int kSfPerStage = 4; };
template <> struct KindInfo<MmaKind::MXF4NVF4> { static constexpr bool kBlockScaled = true; static constexpr int kSfPerStage = 16; };

struct GemmArgs {
  int M, N;
  int k_iters;           // pipeline stages along K (128 bytes of K per row each, times the kernel's KD)
  int tiles_m, tiles_n;  // cluster tiles: (128 * CG) x BN
  void* C;
  int64_t ldc;
  const float* scale_a;
  const float* scale_b;
  const float* bias;
  float alpha;
  int vec_ok;  // C rows 16-byte aligned: vector stores allowed
  long long* trace;  // debug: per-stage clock64 stamps of CTAs 0 and 1, then the kernel span of CTA 0 (null = off)
  int a_rows;        // rows of A one stage load brings in (the tensor map's box; 128 unless M < 128)
  int stages;        // pipeline depth (the launcher's choice: fewer A rows per stage leave room for more stages)
  int f16;           // kind::f16 only: bit 0 = operands are fp16 (else bf16), bit 1 = fp16 accumulator, bit 2 = fp16 output
  // Gated dual GEMM (EPI_GATED): the B tile holds 128 rows of W1 and the matching 128 rows of W3, so
  // accumulator columns [0,128) are X W1^T and [128,256) X W3^T for the same 128 output columns.
  // out = (o1 * o3) * sigmoid(o1) with o1 = acc1 * (ts_w1 * ts_x), o3 = acc3 * (ts_w3 * ts_x); written
  // as bf16 (C, ldc in elements), or, when ts_out is set, quantised to NVFP4 (C = packed E2M1, ldc in
  // bytes; sfc = E4M3 block scales in the swizzled layout with N/16 columns).
  struct {
    const float* ts_x;
    const float* ts_w1;
    const float* ts_w3;
    const float* ts_out;
    uint8_t* sfc;
    float eps;
  } gated;
  // Reduce-scatter variant (EPI_RS): K-sharded partial tiles are pushed to the rank that owns
  // their rows and summed there.  staging[r] / flags[r] are rank r's buffers as mapped on
  // THIS GPU.  Flag words: per owned 128 x BN unit one arrival and one progress word, then a CTA
  // ticket, the exit counter (peers' "I have finished reducing" signals) and the count of calls
  // whose exit wait was deferred.
  struct {
    int world, rank;
    int lagged_exit;       // 1: this call signals its exit but leaves the wait to the next call's first store
    int rows_per_owner;    // M / world
    int tiles_per_owner;   // cluster tiles along M per owner
    unsigned int timeout_ms;
    __nv_bfloat16* staging[kMaxWorld];
    unsigned int* flags[kMaxWorld];
    __nv_bfloat16* out;
    int64_t ldo;
    // Pull variant: the multicast address of the ranks' [M, N] partial buffers (staging[] are then the
    // same buffers seen per rank).  Null selects the push variant.
    const __nv_bfloat16* mc_partial;
    // All-reduce variant (pull only): the multicast address of the ranks' [M, N] output buffers.  The owner
    // then stores every reduced piece through it (one multimem.st reaches all ranks) instead of into `out`,
    // so every rank ends with all M rows.  Null = reduce-scatter.
    __nv_bfloat16* mc_out;
    // debug: 8 words per CTA (globaltimer ns): start, epilogue end, reducer end, reducer wait total,
    // MMA end, epilogue store+signal total, epilogue wait-for-accumulator total (null = off)
    unsigned long long* trace;
  } rs;
};

// Tensor maps of the epilogue.  The reduce-scatter variant has one per owner rank, over
// this rank's slot in that owner's staging buffer ([rows_per_owner, N] bf16, 64 x 32 boxes, 128-byte
// swizzle), used for bulk tensor STORES of finished tiles into peer memory.
template <int EPI>
struct EpiMaps {
  CUtensorMap c;  // the bf16 output [M, N], 64 x 32 boxes, 128-byte swizzle (bulk-store epilogue only)
};
template <>
struct EpiMaps<EPI_RS> {
  CUtensorMap slot[kMaxWorld];
  CUtensorMap local;  // pull variant: this rank's own [M, N] partial
};
template <>
struct EpiMaps<EPI_GATED> {
  CUtensorMap c;     // unused
  CUtensorMap b3;    // W3 [N, K] (tm_b is W1), 128-row boxes
  CUtensorMap sfb3;  // its scale atoms (tm_sfb is W1's), one 128-row group per box
};
template <int EPI>
__device__ __forceinline__ const CUtensorMap* output_map(const EpiMaps<EPI>& m) {
  return &m.c;
}
template <>
__device__ __forceinline__ const CUtensorMap* output_map<EPI_RS>(const EpiMaps<EPI_RS>& m) {
  return &m.slot[0];  // never used: the reduce-scatter variant stores through slot[owner]
}

// KD = 128-byte K slices per pipeline stage.  A problem that is one stream of a weight matrix past a
// few rows of activations (one tile per CTA) is bound by the per-stage cost of the producer and issuer
// loops (barrier round trips, TMA issue), not by bytes or math: KD = 4 moves 512 bytes of K per row
// with the same number of operations (one rank-3 box per operand).
template <MmaKind KIND, int BN, int CG, int EPI = EPI_BF16, int STG = 1, int KD = 1>
struct Cfg {
  using KI = KindInfo<KIND>;
  static_assert(KD == 1 || (CG == 1 && BN <= 128), "deep stages are for the small single-CTA tiles");
  // bf16 outputs of the 256-wide pair tile leave through per-warp shared-memory staging and bulk
  // tensor stores.  Plain GEMMs (STG != 0): two 4 KB buffers per warp, one 64-column block each,
  // so only 32 KB of pipeline space is given up.  The reduce-scatter variant stages the whole
  // 32 x 256 piece (16 KB per warp) because it waits for completion once per tile.
  static constexpr bool kStaged = EPI == EPI_RS && BN == 256 && CG == 2;
  static constexpr bool kBulkC = STG != 0 && (BN == 256 || BN == 192) && CG == 2 && EPI != EPI_I32 && EPI != EPI_RS && EPI != EPI_GATED;
  static constexpr int kEpiBytes = kStaged ? 4 * 32 * BN * 2 : kBulkC ? 4 * 2 * 4096 : 0;
  static constexpr int kABytes = 128 * 128 * KD;
  static constexpr int kBSliceBytes = (BN / CG) * 128;                 // one 128-byte K slice of the B tile
  static constexpr int kBBytes = kBSliceBytes * KD;
  static constexpr int kSfAtomBytes = 128 * KI::kSfPerStage;           // one 128-row group, one K slice
  static constexpr int kSfaBytes = kSfAtomBytes * KD;
  // a 192-wide tile starts at row 0 or 64 of a 128-row scale group and touches two groups either way
  static constexpr int kSfbGroups = BN >= 128 ? (BN + 127) / 128 : 1;
  static constexpr int kSfbBytes = kSfAtomBytes * kSfbGroups * KD;
  static constexpr int kSfLoadsPerStage = (kSfaBytes / 8 + 255) / 256;  // TMA boxes are at most 256 elements wide
  static_assert(KD == 1 || kSfbGroups == 1, "deep stages load the scale atoms of one 128-row group of B");
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kSmemBudget = 227 * 1024 - 2048 - kEpiBytes;    // barriers + alignment slack
  static constexpr int kStagesRaw = kSmemBudget / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  // deep stages are coarse (up to 100 KB): they get the whole budget rather than a multiple of the full-size stage
  static constexpr int kSmemBytes = KD > 1 ? kSmemBudget + 2048 + kEpiBytes : kStages * kStageBytes + 2048 + kEpiBytes;
  static constexpr int kMaxStages = 24;  // barrier words stay well inside the 2 KB reserve
  // pipeline depth when a stage holds only a_rows rows of A.  The MMA still reads 128 rows (16 KB) from
  // the start of every A slice, whatever a_rows is: with few rows and a narrow B tile that read runs past
  // the end of its own stage, which is harmless inside the pipeline buffers but must not leave the
  // shared-memory allocation from the last stage (an out-of-range shared address faults the kernel).
  static int stages_for(int a_rows) {
    if (a_rows >= 128 && KD == 1) return kStages;
    const int pool = KD > 1 ? kSmemBudget : kStages * kStageBytes;
    const int stage = kStageBytes - (128 - a_rows) * 128 * KD;
    int n = pool / stage;
    while (n > 1 && (n - 1) * stage + (KD - 1) * a_rows * 128 + 128 * 128 > pool) --n;
    return n > kMaxStages ? kMaxStages : n;
  }
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

// Reduce-scatter tile order.  Sequence index i -> owner (rank + 1 + i) % W, so that at any moment
// every rank pushes to a different owner (each NVLink ingress sees one sender), and all ranks
// produce local tile q = i / W of every owner within the same round of W tiles, which lets the
// owners reduce right behind production.
__host__ __device__ __forceinline__ void rs_local_tile(int q, int tiles_per_owner, int tiles_n, int world, int& lm,
                                                        int& tn) {
  // inside an owner: groups of up to 8 / world tile rows, tile row fastest inside a group, so that a
  // wave of concurrently running tiles (all owners together) touches ~8 row blocks and ~9 column blocks
  int grp_rows = 8 / world;
  if (grp_rows < 1) grp_rows = 1;
  if (grp_rows > tiles_per_owner) grp_rows = tiles_per_owner;
  const int per = grp_rows * tiles_n;
  const int grp = q / per, rem = q - grp * per;
  const int first = grp * grp_rows;
  const int gsz = tiles_per_owner - first < grp_rows ? tiles_per_owner - first : grp_rows;
  lm = first + rem % gsz;
  tn = rem / gsz;
}
__device__ __forceinline__ void tile_coords_rs(int i, const GemmArgs& g, int& tm, int& tn) {
  const int owner = (g.rs.rank + 1 + i) % g.rs.world;
  int lm;
  rs_local_tile(i / g.rs.world, g.rs.tiles_per_owner, g.tiles_n, g.rs.world, lm, tn);
  tm = owner * g.rs.tiles_per_owner + lm;
}
template <int EPI>
__device__ __forceinline__ void map_tile(int t, const GemmArgs& g, int& tm, int& tn) {
  if constexpr (EPI == EPI_RS) tile_coords_rs(t, g, tm, tn);
  else tile_coords(t, g.tiles_m, g.tiles_n, tm, tn);
}

// Streaming accesses of the reducer: every staging line is read once and every output line written
// once, so both are marked evict-first in L2 and leave the GEMM operands (which are re-read by many
// tiles) in place.  The load stays L2-only (.cg): the lines were written by other GPUs.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint4 ld_cg_hint(const uint4* ptr, uint64_t pol) {
  uint4 v;
  asm volatile("ld.global.cg.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr), "l"(pol)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_hint(uint4* ptr, uint4 v, uint64_t pol) {
  asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1, %2, %3, %4}, %5;" ::"l"(ptr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w), "l"(pol)
               : "memory");
}

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(unsigned int* p, unsigned int v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded poll of a flag word another GPU increments.  Returns false (and records `detail`) on give-up.
__device__ __forceinline__ bool wait_flag_eq(const unsigned int* p, unsigned int want, unsigned int timeout_ms,
                                             uint32_t detail) {
  if (ld_acquire_sys(p) == want) return true;
  const uint64_t t0 = globaltimer_ns();
  const uint64_t budget = static_cast<uint64_t>(timeout_ms) * 1000000ull;
  while (ld_acquire_sys(p) != want) {
    __nanosleep(64);
    if (globaltimer_ns() - t0 > budget) {
      report_timeout(detail);
      return false;
    }
  }
  return true;
}
// The same for a counter that only grows: done when it has reached `want`.
__device__ __forceinline__ bool wait_flag_ge(const unsigned int* p, unsigned int want, unsigned int timeout_ms,
                                             uint32_t detail) {
  if (ld_acquire_sys(p) >= want) return true;
  const uint64_t t0 = globaltimer_ns();
  const uint64_t budget = static_cast<uint64_t>(timeout_ms) * 1000000ull;
  while (ld_acquire_sys(p) < want) {
    __nanosleep(64);
    if (globaltimer_ns() - t0 > budget) {
      report_timeout(detail);
      return false;
    }
  }
  return true;
}

// fp32/int32 accumulator values of W consecutive columns -> finished fp32 values (epilogue math)
template <MmaKind KIND, int EPI, int W>
__device__ __forceinline__ void finish_cols(const uint32_t* r, const GemmArgs& g, int col0, float sa, float* f) {
#pragma unroll
  for (int i = 0; i < W; ++i) {
    float v = KIND == MmaKind::I8 ? static_cast<float>(static_cast<int32_t>(r[i])) : __uint_as_float(r[i]);
    if constexpr (KIND == MmaKind::F16 && EPI == EPI_BF16) {
      // an fp16 accumulator sits in the low half of its 32-bit TMEM column
      if (g.f16 & 2) v = __half2float(__ushort_as_half(static_cast<unsigned short>(r[i] & 0xFFFFu)));
    }
    if constexpr (EPI == EPI_ROWSCALED) {
      const int c = min(col0 + i, g.N - 1);
      if (g.scale_a) v = __fmul_rn(v, sa);
      if (g.scale_b) v = __fmul_rn(v, __ldg(g.scale_b + c));
      if (g.bias) v = __fadd_rn(v, __ldg(g.bias + c));
    } else if constexpr (KIND == MmaKind::MXF4NVF4 || (KIND == MmaKind::F8F6F4 && EPI == EPI_RS)) {
      v = __fmul_rn(v, g.alpha);
    }
    f[i] = v;
  }
}

// two finished values -> one 32-bit word of the 16-bit output type (bf16, or fp16 for the fp16 GEMM)
template <MmaKind KIND, int EPI>
__device__ __forceinline__ uint32_t pack_out(const GemmArgs& g, float lo, float hi) {
  if constexpr (KIND == MmaKind::F16 && EPI == EPI_BF16) {
    if (g.f16 & 4) {
      __half2 h = __floats2half2_rn(lo, hi);
      return *reinterpret_cast<uint32_t*>(&h);
    }
  }
  return pack_bf16x2(lo, hi);
}

// ---- epilogue: W (16 or 32) consecutive accumulator columns of one row ------------------
template <MmaKind KIND, int EPI, int W>
__device__ __forceinline__ void store_cols(const uint32_t* r, const GemmArgs& g, int row, int col0, float sa,
                                           void* rowptr) {
  if (row >= g.M || col0 >= g.N) return;
  const bool full = (col0 + W <= g.N) && g.vec_ok;
  if constexpr (EPI == EPI_I32) {
    int32_t* dst = static_cast<int32_t*>(rowptr) + col0;
    if (full) {
#pragma unroll
      for (int i = 0; i < W; i += 4) *reinterpret_cast<uint4*>(dst + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
    } else {
      for (int i = 0; i < W && col0 + i < g.N; ++i) dst[i] = static_cast<int32_t>(r[i]);
    }
  } else {
    float f[W];
    finish_cols<KIND, EPI, W>(r, g, col0, sa, f);
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(rowptr) + col0;
    if (full) {
#pragma unroll
      for (int i = 0; i < W; i += 8)
        *reinterpret_cast<uint4*>(dst + i) =
            make_uint4(pack_out<KIND, EPI>(g, f[i], f[i + 1]), pack_out<KIND, EPI>(g, f[i + 2], f[i + 3]),
                       pack_out<KIND, EPI>(g, f[i + 4], f[i + 5]), pack_out<KIND, EPI>(g, f[i + 6], f[i + 7]));
    } else {
      for (int i = 0; i < W && col0 + i < g.N; ++i)
        reinterpret_cast<uint16_t*>(dst)[i] = static_cast<uint16_t>(pack_out<KIND, EPI>(g, f[i], 0.f) & 0xFFFFu);
    }
  }
}

// drains accumulator columns [c0, c1) (multiples of 16) of this warp's 32 rows
template <MmaKind KIND, int EPI>
__device__ __forceinline__ void drain_cols(uint32_t taddr_row, int c0, int c1, const GemmArgs& g, int row, int ncol0,
                                           float sa, void* rowptr) {
  int c = c0;
  for (; c + 32 <= c1; c += 32) {
    uint32_t r[32];
    tmem_ld32(taddr_row + c, r);
    tc_wait_ld();
    store_cols<KIND, EPI, 32>(r, g, row, ncol0 + c, sa, rowptr);
  }
  for (; c + 16 <= c1; c += 16) {
    uint32_t r[16];
    tmem_ld16(taddr_row + c, r);
    tc_wait_ld();
    store_cols<KIND, EPI, 16>(r, g, row, ncol0 + c, sa, rowptr);
  }
}

// the same for a result that two issuing threads accumulated in two places: columns [0, c1) of the
// accumulator at taddr_row plus the same columns `other` columns further on
template <MmaKind KIND, int EPI>
__device__ __forceinline__ void drain_cols_sum2(uint32_t taddr_row, uint32_t other, int c1, const GemmArgs& g, int row,
                                                int ncol0, float sa, void* rowptr) {
  for (int c = 0; c + 32 <= c1; c += 32) {
    uint32_t r[32], q[32];
    tmem_ld32(taddr_row + c, r);
    tmem_ld32(taddr_row + other + c, q);
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if constexpr (KIND == MmaKind::I8) r[i] += q[i];  // int32 accumulators: exact in any order
      else r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(q[i]));
    }
    store_cols<KIND, EPI, 32>(r, g, row, ncol0 + c, sa, rowptr);
  }
}

// Reducer: one chunk of PB * 128 / (BN / 8) rows x BN columns of this rank's output.  Each of the 128
// reducer threads owns PB 16-byte pieces; the loads of all slots of all its pieces are in flight
// together (PB * world <= 16), the fp32 sums run in rank order, the result is rounded to bf16 once.
template <int BN, int PB>
__device__ __forceinline__ void reduce_chunk(const GemmArgs& g, const __nv_bfloat16* my_stage, int lr0, int c0, int ct,
                                             uint64_t stream_pol) {
  constexpr int kPiecesPerRow = BN / 8;
  constexpr int kSlots = 16 / PB;  // most ranks this instantiation serves
  uint4 v[PB][kSlots];
  int rr[PB], cc[PB];
#pragma unroll
  for (int q = 0; q < PB; ++q) {
    const int piece = ct + q * 128;
    rr[q] = lr0 + piece / kPiecesPerRow;
    cc[q] = c0 + (piece % kPiecesPerRow) * 8;
#pragma unroll
    for (int sr = 0; sr < kSlots; ++sr)
      if (sr < g.rs.world) {  // L2-only loads: the lines were written by other GPUs during this kernel
        const uint4* src = reinterpret_cast<const uint4*>(
            my_stage + (static_cast<int64_t>(sr) * g.rs.rows_per_owner + rr[q]) * g.N + cc[q]);
        v[q][sr] = ld_cg_hint(src, stream_pol);
      }
  }
#pragma unroll
  for (int q = 0; q < PB; ++q) {
    float acc8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int sr = 0; sr < kSlots; ++sr)
      if (sr < g.rs.world) {
        const uint32_t w[4] = {v[q][sr].x, v[q][sr].y, v[q][sr].z, v[q][sr].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc8[2 * e] += __uint_as_float(w[e] << 16);
          acc8[2 * e + 1] += __uint_as_float(w[e] & 0xFFFF0000u);
        }
      }
    st_hint(reinterpret_cast<uint4*>(g.rs.out + static_cast<int64_t>(rr[q]) * g.rs.ldo + cc[q]),
            make_uint4(pack_bf16x2(acc8[0], acc8[1]), pack_bf16x2(acc8[2], acc8[3]), pack_bf16x2(acc8[4], acc8[5]),
                       pack_bf16x2(acc8[6], acc8[7])),
            stream_pol);
  }
}

// Pull variant of the reducer: the same chunk, but every 16-byte piece is ONE load from the multicast
// address of the ranks' partial buffers; NVSwitch fetches the piece from every rank, adds the bf16
// values in fp32 and returns the rounded sum, so only the reduced data enters this SM.
template <int BN, int PB>
__device__ __forceinline__ void reduce_chunk_multimem(const GemmArgs& g, int lr0, int c0, int ct, uint64_t stream_pol) {
  constexpr int kPiecesPerRow = BN / 8;
  uint4 v[PB];
  int rr[PB], cc[PB];
#pragma unroll
  for (int q = 0; q < PB; ++q) {
    const int piece = ct + q * 128;
    rr[q] = lr0 + piece / kPiecesPerRow;
    cc[q] = c0 + (piece % kPiecesPerRow) * 8;
    const __nv_bfloat16* src =
        g.rs.mc_partial + (static_cast<int64_t>(g.rs.rank) * g.rs.rows_per_owner + rr[q]) * g.N + cc[q];
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v[q].x), "=r"(v[q].y), "=r"(v[q].z), "=r"(v[q].w)
                 : "l"(src)
                 : "memory");
  }
  if (g.rs.mc_out) {
    // all-reduce: this rank's rows of the result go to every rank's output in one store through the switch
#pragma unroll
    for (int q = 0; q < PB; ++q) {
      __nv_bfloat16* dst =
          g.rs.mc_out + (static_cast<int64_t>(g.rs.rank) * g.rs.rows_per_owner + rr[q]) * g.rs.ldo + cc[q];
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst),
                   "f"(__uint_as_float(v[q].x)), "f"(__uint_as_float(v[q].y)), "f"(__uint_as_float(v[q].z)),
                   "f"(__uint_as_float(v[q].w))
                   : "memory");
    }
    return;
  }
#pragma unroll
  for (int q = 0; q < PB; ++q)
    st_hint(reinterpret_cast<uint4*>(g.rs.out + static_cast<int64_t>(rr[q]) * g.rs.ldo + cc[q]), v[q], stream_pol);
}

// Staging for a bulk tensor store: the warp's 32 x BN tile as BN/64 column blocks of [32 rows][128 bytes]
// in the 128-byte swizzle (16-byte piece index XOR row % 8), the layout a 64 x 32 box store reads.
template <MmaKind KIND, int EPI, int BN>
__device__ __forceinline__ void drain_to_smem_sw128(uint32_t taddr_row, int c0, int c1, const GemmArgs& g, int ncol0,
                                                    float sa, uint32_t stg, int r, uint32_t blk_stride = 4096) {
  for (int c = c0; c < c1; c += 16) {
    uint32_t raw[16];
    tmem_ld16(taddr_row + c, raw);
    tc_wait_ld();
    float f[16];
    finish_cols<KIND, EPI, 16>(raw, g, ncol0 + c, sa, f);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int piece = (c >> 3) + j;  // 16-byte piece of the row
      const uint32_t addr = stg + (piece >> 3) * blk_stride + r * 128 + (((piece & 7) ^ (r & 7)) << 4);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pack_out<KIND, EPI>(g, f[8 * j], f[8 * j + 1])),
                   "r"(pack_out<KIND, EPI>(g, f[8 * j + 2], f[8 * j + 3])), "r"(pack_out<KIND, EPI>(g, f[8 * j + 4], f[8 * j + 5])),
                   "r"(pack_out<KIND, EPI>(g, f[8 * j + 6], f[8 * j + 7]))
                   : "memory");
    }
  }
}

// Epilogue of the gated dual GEMM for one thread (= one output row): 128 output columns in eight
// 16-column chunks, each from 16 columns of X W1^T (accumulator columns c..c+15) and the matching 16
// of X W3^T (128 + c..).  The chunks whose accumulator columns are shared with the other TMEM
// accumulator are taken first and released at once (acc 0 shares its last 48 columns, the X W3^T
// chunks 5-7; acc 1 its first 48, the X W1^T chunks 0-2).  bf16 output: 32 bytes per chunk.  NVFP4
// output: a chunk is exactly one scale block, quantised from the bf16-rounded values with the
// quantizer's own arithmetic, 8 bytes of codes per chunk and the eight scale bytes of the row in
// two 4-byte stores (the swizzled layout keeps four consecutive blocks of a row together).
template <int BN, int ACC_STRIDE, int OVERLAP_COLS>
__device__ __forceinline__ void gated_epilogue(uint32_t taddr_row, uint32_t acc, const GemmArgs& g, int row, int ocol0,
                                               uint32_t partial_bar, uint32_t tempty_bar, int lane) {
  static_assert(BN == 256 && OVERLAP_COLS == 48 && ACC_STRIDE == 208, "chunk order below is written for the NVFP4 256-wide tile");
  const float a1 = __fmul_rn(__ldg(g.gated.ts_w1), __ldg(g.gated.ts_x));
  const float a3 = __fmul_rn(__ldg(g.gated.ts_w3), __ldg(g.gated.ts_x));
  const bool fp4 = g.gated.ts_out != nullptr;
  float ts = 0.f, d0 = 1.f, r0 = 1.f;
  if (fp4) {
    ts = __ldg(g.gated.ts_out);
    d0 = fmaxf(__fmul_rn(6.f, ts), 1e-12f);
    r0 = __frcp_rn(d0);
  }
  const bool live = row < g.M;
  uint32_t sf_lo = 0, sf_hi = 0;  // scale codes of chunks 0-3 and 4-7
  const int first = acc == 0 ? 5 : 0;
#pragma unroll 1
  for (int idx = 0; idx < 8; ++idx) {
    const int c = (first + idx) & 7;
    uint32_t r1[16], r3[16];
    tmem_ld16(taddr_row + c * 16, r1);
    tmem_ld16(taddr_row + 128 + c * 16, r3);
    tc_wait_ld();
    if (idx == 2) {  // the three chunks read so far covered every column shared with the other accumulator
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(partial_bar);
    }
    float f[2][8];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float o1 = __fmul_rn(__uint_as_float(r1[i]), a1);
      const float o3 = __fmul_rn(__uint_as_float(r3[i]), a3);
      const float sig = __frcp_rn(1.f + __expf(-o1));
      f[i >> 3][i & 7] = __fmul_rn(__fmul_rn(o1, o3), sig);
    }
    if (!fp4) {
      if (live) {
        __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(g.C) + static_cast<int64_t>(row) * g.ldc + ocol0 + c * 16;
#pragma unroll
        for (int j = 0; j < 2; ++j)
          *reinterpret_cast<uint4*>(dst + 8 * j) = make_uint4(pack_bf16x2(f[j][0], f[j][1]), pack_bf16x2(f[j][2], f[j][3]),
                                                              pack_bf16x2(f[j][4], f[j][5]), pack_bf16x2(f[j][6], f[j][7]));
      }
    } else {
      // the quantizer sees the bf16 output, exactly as a separate quantizer kernel after this GEMM would
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) f[j][i] = __bfloat162float(__float2bfloat16_rn(f[j][i]));
      uint32_t code;
      const uint2 q = nvfp4_encode16(f, ts, d0, r0, g.gated.eps, code);
      if (live)
        *reinterpret_cast<uint2*>(static_cast<uint8_t*>(g.C) + static_cast<int64_t>(row) * g.ldc + (ocol0 + c * 16) / 2) = q;
      if (c < 4) sf_lo |= code << (8 * c);
      else sf_hi |= code << (8 * (c - 4));
    }
  }
  tc_fence_before();
  __syncwarp();
  if (lane == 0) mbar_arrive_cluster(tempty_bar);
  if (fp4 && live) {
    const int64_t ks = g.N >> 4;  // scale columns of the output (N % 128 == 0, so no padding columns)
    const int64_t kcol0 = ocol0 >> 4;
    uint8_t* sfc = g.gated.sfc;
    *reinterpret_cast<uint32_t*>(sfc + sf_offset(row, kcol0, ks, true, ks)) = sf_lo;
    *reinterpret_cast<uint32_t*>(sfc + sf_offset(row, kcol0 + 4, ks, true, ks)) = sf_hi;
  }
}

// The same staging for 16 accumulator columns that are already in registers.
template <MmaKind KIND, int EPI>
__device__ __forceinline__ void stage_cols16_sw128(const uint32_t (&raw)[16], int c, const GemmArgs& g, int ncol0, float sa,
                                                   uint32_t stg, int r) {
  float f[16];
  finish_cols<KIND, EPI, 16>(raw, g, ncol0 + c, sa, f);
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int piece = (c >> 3) + j;
    const uint32_t addr = stg + (piece >> 3) * 4096 + r * 128 + (((piece & 7) ^ (r & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pack_out<KIND, EPI>(g, f[8 * j], f[8 * j + 1])),
                 "r"(pack_out<KIND, EPI>(g, f[8 * j + 2], f[8 * j + 3])), "r"(pack_out<KIND, EPI>(g, f[8 * j + 4], f[8 * j + 5])),
                 "r"(pack_out<KIND, EPI>(g, f[8 * j + 6], f[8 * j + 7]))
                 : "memory");
  }
}

template <MmaKind KIND, int BN, int CG, int EPI, int STG = 1, int KD = 1>
__global__ void __cluster_dims__(CG, 1, 1) __launch_bounds__(EPI == EPI_RS ? 320 : 192, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                const __grid_constant__ CUtensorMap tm_sfa, const __grid_constant__ CUtensorMap tm_sfb,
                const __grid_constant__ EpiMaps<EPI> epi_maps, const GemmArgs g) {
  using C = Cfg<KIND, BN, CG, EPI, STG, KD>;
  constexpr bool kBS = C::KI::kBlockScaled;
  // Deep stages have TWO issuing threads.  One thread issues a tcgen05 instruction every ~35 cycles, and
  // a weight stream past a few rows of activations needs K/32 MMAs plus the scale copies per CTA whatever
  // the tile width: that issue time, not bytes or math, bounds the kernel.  Warp 5 takes the first half
  // of a stage's K slices into accumulator 0, warp 3 (idle until its epilogue) the second half into
  // accumulator 1 with scale columns of its own; the epilogue adds the two.  Such a CTA has one tile.
  constexpr int kIssuers = KD > 1 ? 2 : 1;
  // A problem with fewer than 128 rows loads and holds only those rows of A per stage (rows beyond
  // them read stale shared memory and only feed accumulator rows that are never stored).  A skinny
  // GEMM is the DRAM stream of B, and its rate is set by the bytes in flight: the space saved on A
  // goes into more pipeline stages.
  const int S = g.stages;
  const uint32_t a_slice = static_cast<uint32_t>(g.a_rows) * 128u;  // one 128-byte K slice of the A tile
  const uint32_t a_bytes = a_slice * KD;
  constexpr int kInner = KIND == MmaKind::F16 ? 64 : 128;  // tensor-map elements per 128-byte K stage

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  // [stage][A | B | SFA | SFB]; A and B stage buffers stay 1024-byte aligned (sizes are multiples of 1024... SF after them)
  // the bulk-store staging (read by TMA in the 128-byte swizzle, hence 1024-byte aligned) comes first
  constexpr bool kEpiFirst = C::kBulkC || (EPI == EPI_RS && C::kStaged);
  const uint32_t ab_base = smem_base + (kEpiFirst ? C::kEpiBytes : 0);
  auto stage_a = [&](int s) { return ab_base + s * (a_bytes + C::kBBytes); };
  auto stage_b = [&](int s) { return stage_a(s) + a_bytes; };
  const uint32_t sf_base = ab_base + S * (a_bytes + C::kBBytes);
  auto stage_sfa = [&](int s) { return sf_base + s * (C::kSfaBytes + C::kSfbBytes); };
  auto stage_sfb = [&](int s) { return stage_sfa(s) + C::kSfaBytes; };
  const uint32_t bar_base = sf_base + S * (C::kSfaBytes + C::kSfbBytes);
  auto bar_full = [&](int s) { return bar_base + 8 * s; };
  auto bar_empty = [&](int s) { return bar_base + 8 * (S + s); };
  auto bar_tfull = [&](int s) { return bar_base + 8 * (2 * S + s); };
  auto bar_tempty = [&](int s) { return bar_base + 8 * (2 * S + 2 + s); };
  const uint32_t bar_partial = bar_base + 8 * (2 * S + 4);
  const uint32_t tmem_slot = bar_base + 8 * (2 * S + 5);
  const uint32_t epi_smem = kEpiFirst ? smem_base : (tmem_slot + 8 + 127u) & ~127u;  // epilogue staging (if any)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  int trace_it = 0;
  const uint32_t cta_rank = CG == 2 ? cluster_ctarank() : 0u;
  const int cluster_id = blockIdx.x / CG;
  const int num_clusters = gridDim.x / CG;
  const int num_tiles = g.tiles_m * g.tiles_n;
  // tracing: SM cycle counter and wall clock at entry and exit of CTA 0 (their ratio is the SM clock
  // the kernel really ran at)
  long long* const kspan = g.trace && blockIdx.x == 0 && threadIdx.x == 0 ? g.trace + kTraceSpanAt : nullptr;
  if (kspan) { kspan[0] = clock64(); kspan[1] = static_cast<long long>(globaltimer_ns()); }

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full(s), CG);  // one expect_tx arrival per CTA of the pair
      mbar_init(bar_empty(s), kIssuers);  // one tcgen05.commit per issuing thread
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull(s), kIssuers);
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
    if constexpr (EPI == EPI_GATED) {
      tma_prefetch_desc(&epi_maps.b3);
      tma_prefetch_desc(&epi_maps.sfb3);
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
  if constexpr (KD > 1) {
    // launched with programmatic stream serialization: the set-up above may have run under the previous
    // kernel's tail; let the next kernel start its own, then wait for everything this one depends on
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }
  unsigned long long* rs_tr = nullptr;
  if constexpr (EPI == EPI_RS) {
    if (g.rs.trace) {
      rs_tr = g.rs.trace + blockIdx.x * 8;
      if (threadIdx.x == 0) rs_tr[0] = globaltimer_ns();
    }
  }

  constexpr uint32_t kIdesc = KIND == MmaKind::F16      ? idesc_dense(1, 1, 1, 128 * CG, BN)
                              : KIND == MmaKind::I8     ? idesc_dense(2, 1, 1, 128 * CG, BN)
                              : KIND == MmaKind::F8F6F4 ? idesc_dense(1, 0, 0, 128 * CG, BN)
                              : KIND == MmaKind::MXF8F6F4 ? idesc_block_scaled(0, 1, 128 * CG, BN)
                                                          : idesc_block_scaled(1, 0, 128 * CG, BN);
  uint32_t idesc = kIdesc;
  if constexpr (KIND == MmaKind::F16 && EPI == EPI_BF16) {
    if (g.f16 & 1) idesc &= ~((7u << 7) | (7u << 10));  // operand formats: F16 = 0 (BF16 = 1)
    if (g.f16 & 2) idesc &= ~(3u << 4);                 // accumulator format: F16 = 0 (F32 = 1)
  }
  // The tcgen05 instructions of K slices [d0, d1) of a stage: scale copies, then four MMAs per slice, then
  // the commit that frees the stage.  Called by all 32 lanes: the descriptors are computed warp-uniformly
  // and only the issue instructions sit in the elected lane's region.
  auto issue_slices = [&](bool leader, uint32_t stage, int k, int d0, int d1, uint32_t d_tmem, uint32_t sf_tmem,
                          uint32_t sfb_half) {
    uint64_t a_desc[KD], b_desc[KD], sfa_desc[KD], sfb_desc[KD];
#pragma unroll
    for (int d = 0; d < KD; ++d) {
      a_desc[d] = sdesc_k128(stage_a(stage) + d * a_slice);
      b_desc[d] = sdesc_k128(stage_b(stage) + d * C::kBSliceBytes);
      // scale atoms of a stage: [row group][K slice]
      sfa_desc[d] = sdesc_sf(stage_sfa(stage) + d * C::kSfAtomBytes);
      sfb_desc[d] = sdesc_sf(stage_sfb(stage) + d * C::kSfAtomBytes);
    }
    const uint32_t empty = bar_empty(stage);
    if (leader) {
#pragma unroll
      for (int d = 0; d < KD; ++d) {
        if (d < d0 || d >= d1) continue;
        if constexpr (kBS) {
          constexpr int kAtoms = C::kSfAtomBytes / 512;  // atoms per 128-row group per K slice: 1 (mxfp8) or 4 (nvfp4)
#pragma unroll
          for (int a = 0; a < kAtoms; ++a) {
            tc_cp_sf<CG>(sf_tmem + 4 * a, sfa_desc[d] + (512 >> 4) * a);
#pragma unroll
            for (int j = 0; j < C::kSfbGroups; ++j)
              tc_cp_sf<CG>(sf_tmem + C::kSfaCols + (a * C::kSfbGroups + j) * 4,
                           sfb_desc[d] + ((j * C::kSfAtomBytes * KD + 512 * a) >> 4));
          }
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint32_t accum = (k | (d - d0) | kk) != 0;
          if constexpr (!kBS) {
            tc_mma<KIND, CG>(d_tmem, a_desc[d] + 2 * kk, b_desc[d] + 2 * kk, idesc, accum);
          } else if constexpr (KIND == MmaKind::MXF8F6F4) {
            // the four K steps of a slice read bytes 0..3 of the same scale columns (scale ids in the descriptor)
            tc_mma_bs<KIND, CG>(d_tmem, a_desc[d] + 2 * kk, b_desc[d] + 2 * kk, idesc | (kk << 4) | (kk << 29), sf_tmem,
                                sf_tmem + C::kSfaCols + sfb_half, accum);
          } else {
            // each K step (64 fp4) has its own scale columns (4 scales = one 32-bit column per row group)
            tc_mma_bs<KIND, CG>(d_tmem, a_desc[d] + 2 * kk, b_desc[d] + 2 * kk, idesc, sf_tmem + 4 * kk,
                                sf_tmem + C::kSfaCols + kk * C::kSfbGroups * 4 + sfb_half, accum);
          }
        }
      }
      if constexpr (CG == 2) tc_commit_pair(empty, 3); else tc_commit<1>(empty);
    }
  };

  // Producer and MMA warps run their loops warp-uniformly (all 32 lanes wait on the barriers and
  // compute addresses and descriptors, which keeps those values in uniform registers); one
  // elected lane executes the TMA / tcgen05 issue instructions.
  if (warp == 4) {
    // ------------------------------ producer ------------------------------
    const bool leader = elect_one();
    uint32_t stage = 0, parity = 1;
    bool ok = true;
    const uint32_t stage_tx = C::kStageBytes - (128 - g.a_rows) * 128 * KD;
    // both CTAs of a pair count their bytes on CTA 0's barrier
    const uint32_t full0 = CG == 2 ? map_to_cta(bar_full(0), 0) : bar_full(0);
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
      int tm, tn;
      map_tile<EPI>(t, g, tm, tn);
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
          if constexpr (EPI == EPI_GATED) {
            // 128 rows of W1 and the same 128 rows of W3 form the 256-row B tile; with a CTA pair each
            // CTA fetches one of them, and both fetch both scale-atom groups
            const int w_row = tn * 128;
            if constexpr (CG == 2) {
              mbar_expect_tx_cluster(full, stage_tx);
              tma_load_2d_pair(sa, &tm_a, full, k * kInner, a_row);
              tma_load_2d_pair(sb, cta_rank == 0 ? &tm_b : &epi_maps.b3, full, k * kInner, w_row);
              tma_load_2d_pair(stage_sfa(stage), &tm_sfa, full, k * (C::kSfAtomBytes / 8), sfa_row);
              tma_load_2d_pair(stage_sfb(stage), &tm_sfb, full, k * (C::kSfAtomBytes / 8), tn);
              tma_load_2d_pair(stage_sfb(stage) + C::kSfAtomBytes, &epi_maps.sfb3, full, k * (C::kSfAtomBytes / 8), tn);
            } else {
              mbar_expect_tx(full, stage_tx);
              tma_load_2d(sa, &tm_a, full, k * kInner, a_row);
              tma_load_2d(sb, &tm_b, full, k * kInner, w_row);
              tma_load_2d(sb + 128 * 128, &epi_maps.b3, full, k * kInner, w_row);
              tma_load_2d(stage_sfa(stage), &tm_sfa, full, k * (C::kSfAtomBytes / 8), sfa_row);
              tma_load_2d(stage_sfb(stage), &tm_sfb, full, k * (C::kSfAtomBytes / 8), tn);
              tma_load_2d(stage_sfb(stage) + C::kSfAtomBytes, &epi_maps.sfb3, full, k * (C::kSfAtomBytes / 8), tn);
            }
          } else if constexpr (CG == 2) {
            mbar_expect_tx_cluster(full, stage_tx);
            tma_load_2d_pair(sa, &tm_a, full, k * kInner, a_row);
            tma_load_2d_pair(sb, &tm_b, full, k * kInner, b_row);
            if constexpr (kBS) {
              tma_load_2d_pair(stage_sfa(stage), &tm_sfa, full, k * (C::kSfAtomBytes / 8), sfa_row);
              tma_load_2d_pair(stage_sfb(stage), &tm_sfb, full, k * (C::kSfAtomBytes / 8), sfb_row);
            }
          } else if constexpr (KD > 1) {
            // rank-3 boxes (128 bytes of K, rows, KD slices): the slices land one after the other, each in
            // the layout of an ordinary stage; the scale atoms of consecutive slices are contiguous anyway
            mbar_expect_tx(full, stage_tx);
            tma_load_4d(sa, &tm_a, full, 0, a_row, k * KD, 0);
            tma_load_4d(sb, &tm_b, full, 0, b_row, k * KD, 0);
            if constexpr (kBS) {
              // a box is at most 256 eight-byte words wide: all KD atoms of MXFP8 in one, one per slice for NVFP4
              constexpr int kSfLoads = C::kSfLoadsPerStage;
#pragma unroll
              for (int q = 0; q < kSfLoads; ++q) {
                tma_load_2d(stage_sfa(stage) + q * (C::kSfaBytes / kSfLoads), &tm_sfa, full,
                            (k * kSfLoads + q) * (C::kSfaBytes / kSfLoads / 8), sfa_row);
                tma_load_2d(stage_sfb(stage) + q * (C::kSfaBytes / kSfLoads), &tm_sfb, full,
                            (k * kSfLoads + q) * (C::kSfaBytes / kSfLoads / 8), sfb_row);
              }
            }
          } else {
            mbar_expect_tx(full, stage_tx);
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
      const uint32_t sf_tmem = tmem_base + C::kSfBase;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++iter) {
        if (!mbar_wait(bar_tempty(acc), acc_parity, (2u << 24) | (2u << 16) | acc)) { ok = false; break; }
        if constexpr (C::kOverlap) {
          if (iter > 0 && !mbar_wait(bar_partial, (iter - 1) & 1, (2u << 24) | (3u << 16))) { ok = false; break; }
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * C::kAccStride;
        // a 64-wide tile uses half of a 128-row scale atom of B: rows 64..127 sit in TMEM columns 2 and 3;
        // every second 192-wide tile starts at row 64 of its first scale group in the same way
        uint32_t sfb_half = 0;
        if constexpr (kBS && (BN == 64 || BN == 192)) {
          int tm, tn;
          map_tile<EPI>(t, g, tm, tn);
          sfb_half = 2u * (tn & 1);
        }
        for (int k = 0; k < g.k_iters; ++k) {
          const long long tr0 = g.trace ? clock64() : 0;
          if (!mbar_wait(bar_full(stage), parity, (2u << 24) | (4u << 16) | stage)) { ok = false; break; }
          const long long tr1 = g.trace ? clock64() : 0;
          tc_fence_after();
          issue_slices(leader, stage, k, 0, KD / kIssuers, d_tmem, sf_tmem, sfb_half);
          if (leader) {
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
      if (rs_tr && leader) rs_tr[4] = globaltimer_ns();
    }
  } else if (warp < 4) {
    if constexpr (kIssuers == 2) {
      // second issuing thread (see kIssuers): the upper half of every stage's K slices, accumulator 1,
      // scale columns 32 further on; then this warp joins the epilogue like the others
      if (warp == 3 && cluster_id < num_tiles) {
        const bool leader = elect_one();
        uint32_t stage = 0, parity = 0;
        int tm, tn;
        map_tile<EPI>(cluster_id, g, tm, tn);
        const uint32_t sfb_half = (kBS && BN == 64) ? 2u * (tn & 1) : 0u;
        bool ok = true;
        for (int k = 0; k < g.k_iters; ++k) {
          if (!mbar_wait(bar_full(stage), parity, (2u << 24) | (9u << 16) | stage)) { ok = false; break; }
          tc_fence_after();
          issue_slices(leader, stage, k, KD / 2, KD, tmem_base + C::kAccStride, tmem_base + C::kSfBase + 32, sfb_half);
          __syncwarp();
          if (++stage == S) { stage = 0; parity ^= 1; }
        }
        if (ok && leader) tc_commit<1>(bar_tfull(0));
        __syncwarp();
      }
    }
    unsigned long long tr_store = 0, tr_wait = 0;
    unsigned int* pending_flag = nullptr;  // lane 0: flag of the piece whose bulk stores are still in flight
    // ------------------------------ epilogue (warps 0-3) ------------------------------
    uint32_t acc = 0, parity = 0;
    const uint32_t tempty0 = CG == 2 ? map_to_cta(bar_tempty(0), 0) : bar_tempty(0);
    const uint32_t partial = CG == 2 ? map_to_cta(bar_partial, 0) : bar_partial;
    bool ok = true;
    [[maybe_unused]] uint32_t stage_turn = 0;  // bulk-store epilogue: which of the warp's two staging buffers comes next
    [[maybe_unused]] bool first_tile = true;
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
      int tm, tn;
      map_tile<EPI>(t, g, tm, tn);
      const unsigned long long trw0 = rs_tr ? globaltimer_ns() : 0;
      if (!mbar_wait(bar_tfull(acc), parity, (3u << 24) | (5u << 16) | acc)) { ok = false; break; }
      if (rs_tr) tr_wait += globaltimer_ns() - trw0;
      if constexpr (EPI == EPI_RS) {
        // Entry half of a deferred exit barrier: earlier calls on these buffers may have left without
        // waiting for their peers.  Nothing of this call may become visible to a peer (tile data, flag
        // signals) before every peer has finished reducing the previous one; the first tile's main loop
        // has run in the meantime.
        if (first_tile) {
          first_tile = false;
          if (lane == 0 && g.rs.world > 1) {
            const int units = (g.rs.rows_per_owner / 128) * g.tiles_n;
            const unsigned int* my_flags = g.rs.flags[g.rs.rank];
            const unsigned int deferred = *reinterpret_cast<const volatile unsigned int*>(my_flags + 2 * units + 2);
            if (deferred != 0u && !status_is_set())
              wait_flag_ge(my_flags + 2 * units + 1, deferred * (g.rs.world - 1), g.rs.timeout_ms, (3u << 24) | (8u << 16));
          }
          __syncwarp();
        }
        // Signal the warp's previous piece: by now its bulk stores have long completed, so this
        // wait returns at once; it also frees the staging area for this tile.
        if (lane == 0 && pending_flag) {
          tma_store_wait_all<0>();
          asm volatile("fence.proxy.async;" ::: "memory");
          red_release_sys_add(pending_flag, 1u);
          pending_flag = nullptr;
        }
        __syncwarp();
      }
      tc_fence_after();
      const int row = (tm * CG + cta_rank) * 128 + warp * 32 + lane;
      const int ncol0 = tn * BN;
      const float sa = (EPI == EPI_ROWSCALED && g.scale_a && row < g.M) ? __ldg(g.scale_a + row) : 1.f;
      void* rowptr;
      unsigned int* rs_flag = nullptr;
      if constexpr (EPI == EPI_RS) {
        // this rank's slot in the staging buffer of the rank that owns the row
        const int owner = row / g.rs.rows_per_owner;
        const int lrow = row - owner * g.rs.rows_per_owner;
        if (g.rs.mc_partial)  // pull variant: the row's place in this rank's own [M, N] partial
          rowptr = g.rs.staging[g.rs.rank] + static_cast<int64_t>(row) * g.N;
        else
          rowptr = g.rs.staging[owner] + (static_cast<int64_t>(g.rs.rank) * g.rs.rows_per_owner + lrow) * g.N;
        const int lrow0 = (tm * CG + cta_rank) * 128 - owner * g.rs.rows_per_owner;
        rs_flag = g.rs.flags[owner] + (lrow0 / 128) * g.tiles_n + tn;
      } else if constexpr (EPI == EPI_I32) {
        rowptr = static_cast<int32_t*>(g.C) + static_cast<int64_t>(row) * g.ldc;
      } else {
        rowptr = static_cast<__nv_bfloat16*>(g.C) + static_cast<int64_t>(row) * g.ldc;
      }
      const uint32_t taddr_row = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + acc * C::kAccStride;
      // bulk-store path: full-width tiles of an output with 16-byte aligned rows
      bool staged = false;
      // the reduce-scatter pair tile always covers whole 256 x 256 blocks of one owner's rows
      constexpr bool kBulkStore = EPI == EPI_RS && C::kStaged && !C::kOverlap;
      const uint32_t stg = epi_smem + warp * (C::kBulkC ? 2 * 4096 : 32 * BN * 2);
      if constexpr (C::kBulkC) staged = g.vec_ok && (ncol0 + BN <= g.N);
      if (C::kBulkC && staged) {
        // 64-column blocks, each: wait until the buffer's previous store has read it, drain the
        // block into it (swizzled), hand it to a bulk tensor store (rows beyond M are clipped).  With
        // overlapping accumulators the block holding the shared columns goes first.
        const int row0 = (tm * CG + cta_rank) * 128 + warp * 32;
        const int first = (C::kOverlap && acc == 0) ? 3 : 0;
        constexpr int kBlocks = BN / 64;
#pragma unroll 1
        for (int i = 0; i < kBlocks; ++i) {
          const int cb = C::kOverlap ? (first + i) & 3 : i;
          // the two buffers alternate across tiles too (a 192-wide tile has an odd number of blocks)
          const uint32_t buf = stg + (stage_turn++ & 1) * 4096;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          if (C::kOverlap && i == 0) {
            const int o0 = acc == 0 ? C::kAccStride : 0;
            const int o1 = o0 + C::kOverlapCols;
            // The MMA warp cannot start the next tile before these columns are free, so they are pulled
            // into registers in one go (all loads in flight, one wait) and released at once; converting
            // and staging them happens afterwards.
            constexpr int kShared16 = C::kOverlapCols / 16;
            uint32_t shared_raw[kShared16 > 0 ? kShared16 : 1][16];
#pragma unroll
            for (int q = 0; q < kShared16; ++q) tmem_ld16(taddr_row + o0 + q * 16, shared_raw[q]);
            tc_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(partial);
#pragma unroll
            for (int q = 0; q < kShared16; ++q)
              stage_cols16_sw128<KIND, EPI>(shared_raw[q], o0 + q * 16, g, ncol0, sa, buf - cb * 4096, lane);
            if (acc == 0) drain_to_smem_sw128<KIND, EPI, BN>(taddr_row, 192, o0, g, ncol0, sa, buf - cb * 4096, lane);
            else drain_to_smem_sw128<KIND, EPI, BN>(taddr_row, o1, 64, g, ncol0, sa, buf - cb * 4096, lane);
          } else {
            drain_to_smem_sw128<KIND, EPI, BN>(taddr_row, cb * 64, cb * 64 + 64, g, ncol0, sa, buf - cb * 4096, lane);
          }
          if (i == kBlocks - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(tempty0 + 8 * acc);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(output_map<EPI>(epi_maps), buf, ncol0 + cb * 64, row0);
            tma_store_commit();
          }
        }
      } else if constexpr (EPI == EPI_GATED) {
        gated_epilogue<BN, C::kAccStride, C::kOverlapCols>(taddr_row, acc, g, row, tn * 128, partial, tempty0 + 8 * acc, lane);
      } else {
      if constexpr (C::kOverlap) {
        // the columns shared with the other accumulator go first and are released at once
        const int o0 = acc == 0 ? C::kAccStride : 0;
        const int o1 = o0 + C::kOverlapCols;
        drain_cols<KIND, EPI>(taddr_row, o0, o1, g, row, ncol0, sa, rowptr);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(partial);
        const int p0 = acc == 0 ? 0 : o1, p1 = acc == 0 ? o0 : BN;
        drain_cols<KIND, EPI>(taddr_row, p0, p1, g, row, ncol0, sa, rowptr);
      } else {
        if constexpr (kBulkStore) drain_to_smem_sw128<KIND, EPI, BN>(taddr_row, 0, BN, g, ncol0, sa, stg, lane);
        else if constexpr (kIssuers == 2) drain_cols_sum2<KIND, EPI>(taddr_row, C::kAccStride, BN, g, row, ncol0, sa, rowptr);
        else drain_cols<KIND, EPI>(taddr_row, 0, BN, g, row, ncol0, sa, rowptr);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty0 + 8 * acc);
      }
      const unsigned long long trs0 = rs_tr ? globaltimer_ns() : 0;
      if constexpr (kBulkStore) {
        // TMEM is already released.  The warp's 32 x BN piece leaves as BN/64 bulk tensor stores (into
        // the owner's staging slot, or into this rank's own partial in the pull variant).  Its flag
        // signal needs the writes complete, not only shared memory read; that wait is deferred to the
        // start of the warp's next tile (see above), when it no longer costs anything.
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int row0 = (tm * CG + cta_rank) * 128 + warp * 32;
          const int owner = row0 / g.rs.rows_per_owner;
          if (g.rs.mc_partial) {
#pragma unroll
            for (int cb = 0; cb < BN / 64; ++cb) tma_store_2d(&epi_maps.local, stg + cb * 4096, ncol0 + cb * 64, row0);
          } else {
#pragma unroll
            for (int cb = 0; cb < BN / 64; ++cb)
              tma_store_2d(&epi_maps.slot[owner], stg + cb * 4096, ncol0 + cb * 64, row0 - owner * g.rs.rows_per_owner);
          }
          tma_store_commit();
          pending_flag = rs_flag;
        }
        __syncwarp();
      } else if constexpr (EPI == EPI_RS) {
        // plain stores by every lane: each lane orders its own, then one signal per warp
        __threadfence_system();
        __syncwarp();
        if (lane == 0) red_release_sys_add(rs_flag, 1u);
      }
      if (rs_tr) tr_store += globaltimer_ns() - trs0;
      acc ^= 1;
      if (acc == 0) parity ^= 1;
    }
    if constexpr (EPI == EPI_RS) {
      if (lane == 0 && pending_flag) {  // the warp's last tile
        tma_store_wait_all<0>();
        asm volatile("fence.proxy.async;" ::: "memory");
        red_release_sys_add(pending_flag, 1u);
      }
      __syncwarp();
    }
    if (rs_tr && threadIdx.x == 0) {
      rs_tr[1] = globaltimer_ns();
      rs_tr[5] = tr_store;
      rs_tr[6] = tr_wait;
    }
    // shared memory must outlive the bulk stores that still read it
    if constexpr (C::kBulkC) {
      if (lane == 0) tma_store_wait_all<0>();
      __syncwarp();
    }
  } else {
    // ------------------------------ reducer (warps 6-9, reduce-scatter variant only) ------------------------------
    if constexpr (EPI == EPI_RS) {
      const int ct = threadIdx.x - 192;
      const int units = (g.rs.rows_per_owner / 128) * g.tiles_n;  // 128 x BN units this rank owns
      unsigned int* my_flags = g.rs.flags[g.rs.rank];
      const __nv_bfloat16* my_stage = g.rs.staging[g.rs.rank];
      const uint64_t stream_pol = l2_evict_first_policy();
      __shared__ int rs_ok;
      // Work item = (unit, span of row chunks), in the order in which the ranks produce the owner's
      // tiles, so a CTA waits for its items roughly in arrival order.
      //  pull variant: a chunk is one batch of 8 multicast loads per thread (32 rows of a 256-wide
      //    unit) and every chunk is an item of its own, so the chunks of a unit go to different CTAs
      //    and every SM takes part when the last tiles of all ranks arrive together;
      //  push variant: a chunk is one batch of 2 pieces x world slots per thread and one item covers
      //    the whole unit (the slots are read through this SM's L2 port, which the operand loads of
      //    the main loop already keep busy: a more aggressive reducer only slows the GEMM down).
      const bool pull = g.rs.mc_partial != nullptr;
      const int pb = pull ? 8 : 2;  // 16-byte pieces per thread and batch
      const int chunk_rows = pb * 128 / (BN / 8);
      const int chunks = 128 / chunk_rows;
      const int span = pull ? 1 : chunks;  // chunks per item
      const int parts = chunks / span;     // items per unit
      const int items = units * parts;
      unsigned int* done = my_flags + units;  // items finished per unit
      unsigned long long red_wait = 0;
      bool rs_dead = false;  // thread ct == 0 only: a flag wait of this CTA has run out
      for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int q = item / (CG * parts), rem = item - q * (CG * parts);
        int lm, tn;
        rs_local_tile(q, g.rs.tiles_per_owner, g.tiles_n, g.rs.world, lm, tn);
        const int rb = lm * CG + rem / parts;  // 128-row block inside the owner's rows
        const int u = rb * g.tiles_n + tn;
        const int c0 = tn * BN;
        if (ct == 0) {
          const unsigned long long w0 = rs_tr ? globaltimer_ns() : 0;
          // every rank's four epilogue warps signal their 32-row pieces of the unit separately.
          // Giving up is paid once: after the first wait of this CTA (or of any CTA, through the
          // sticky status word) has run out, the remaining items are skipped without polling.
          if (rs_dead || status_is_set()) {
            rs_ok = 0;
          } else {
            rs_ok = wait_flag_eq(my_flags + u, 4u * g.rs.world, g.rs.timeout_ms, (4u << 24) | (6u << 16) | (u & 0xFFFF));
            if (!rs_ok) rs_dead = true;
          }
          if (rs_tr) red_wait += globaltimer_ns() - w0;
        }
        asm volatile("bar.sync 3, 128;" ::: "memory");
        if (rs_ok) {
          for (int c = 0; c < span; ++c) {
            const int lr0 = rb * 128 + ((rem % parts) * span + c) * chunk_rows;
            if (pull) reduce_chunk_multimem<BN, 8>(g, lr0, c0, ct, stream_pol);
            else reduce_chunk<BN, 2>(g, my_stage, lr0, c0, ct, stream_pol);
          }
        }
        asm volatile("bar.sync 3, 128;" ::: "memory");
        // the last item of a unit clears its words for the next call (peers cannot signal again
        // before the exit barrier)
        if (ct == 0 && rs_ok && atomicAdd(done + u, 1u) == static_cast<unsigned int>(parts - 1)) {
          my_flags[u] = 0u;
          done[u] = 0u;
        }
      }
      if (rs_tr && ct == 0) {
        rs_tr[2] = globaltimer_ns();
        rs_tr[3] = red_wait;
      }
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  if constexpr (CG == 2) cluster_sync_all(); else __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc<CG>(tmem_base, C::kTmemCols);
  }
  if (kspan) { kspan[2] = clock64(); kspan[3] = static_cast<long long>(globaltimer_ns()); }
  if constexpr (EPI == EPI_RS) {
    // Exit barrier across ranks: a rank may overwrite what its peers read (its partial, or its slots
    // in their staging buffers) only after every peer has finished reducing this call.  The last CTA
    // of this rank tells every peer.  It then either waits (bounded) for the world - 1 peers to tell
    // it, and leaves the words zero; or, with `lagged_exit`, returns at once and counts the call, and
    // the NEXT call on these buffers does the wait before its first store (see the epilogue), by
    // which time the slowest peer has normally long finished.  The exit word only grows while waits
    // are deferred: call number c is over everywhere when it holds c * (world - 1).
    if (threadIdx.x == 0) {
      const int units = (g.rs.rows_per_owner / 128) * g.tiles_n;
      unsigned int* my_flags = g.rs.flags[g.rs.rank];
      __threadfence();
      // flag words: [units] arrivals, [units] finished chunks, CTA ticket, exit counter, deferred calls
      const unsigned int ticket = atomicAdd(my_flags + 2 * units, 1u);
      if (ticket == gridDim.x - 1) {
        my_flags[2 * units] = 0u;
        const unsigned int calls = my_flags[2 * units + 2] + 1u;
        __threadfence_system();
        for (int p = 0; p < g.rs.world; ++p)
          if (p != g.rs.rank) red_release_sys_add(g.rs.flags[p] + 2 * units + 1, 1u);
        if (g.rs.lagged_exit) {
          my_flags[2 * units + 2] = calls;
        } else if (!status_is_set() &&
                   wait_flag_ge(my_flags + 2 * units + 1, calls * (g.rs.world - 1), g.rs.timeout_ms, (4u << 24) | (7u << 16))) {
          // a call that has already given up somewhere does not wait a second time: the flag words are
          // then left as they are and the caller re-zeroes them (see gnk_gemm_rs_bf16 in gnk.h)
          my_flags[2 * units + 1] = 0u;
          my_flags[2 * units + 2] = 0u;
        }
      }
    }
  }
}

}  // namespace gemm
}  // namespace gnk

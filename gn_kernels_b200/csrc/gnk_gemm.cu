// tcgen05 GEMM family: C[M,N] = A[M,K] * Bt[N,K]^T for BF16, INT8, E4M3 (dense kinds) and
// MXFP8 / NVFP4 (block-scaled kinds), with fused epilogues (bf16 cast, alpha, row scales +
// bias, raw int32).
//
// One persistent, warp-specialised kernel template:
//   warps 0-3  epilogue: TMEM -> registers (tcgen05.ld, lane = row) -> scale/cast -> global.  The
//              256 x 256 pair tile stages bf16 output in two swizzled 4 KB buffers per warp and
//              writes it with bulk tensor stores (cp.async.bulk.tensor shared -> global); the
//              other tiles store from registers
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
// Decode-shaped problems (one 128 x 64 tile per CTA, at least 1 KB of K per row) take a variant of the
// same template with 4 or 2 128-byte K slices per pipeline stage (rank-3 TMA boxes) and TWO issuing
// threads (warp 5 and warp 3, which is idle until its epilogue), each with an accumulator of its own that
// the epilogue adds: at these shapes the per-stage cost of the producer and issuer loops, not bytes or
// math, sets the pace.  These kernels are launched with programmatic stream serialization and wait for
// their predecessors (griddepcontrol.wait) before their first global access.
// Every barrier wait is bounded; a wait that runs out sets the device status word and the
// role leaves its loop, after which the CTA tears down normally.
#include <atomic>

#include "gnk_gemm_kernel.cuh"

namespace gnk {
namespace {

using namespace gnk::gemm;

std::atomic<long long*> g_trace{nullptr};  // test hook (gnk_debug_trace): device buffer of 2*2*256*3 + 4 int64
std::atomic<int> g_pdl{1};           // test hook (gnk_debug_deep_stage bit 1 clear = no programmatic dependent launch)
std::atomic<int> g_max_clusters{0};  // test hook (gnk_debug_max_clusters): cap on the persistent grid, 0 = none

template <MmaKind KIND>
struct ElemInfo {
  // bytes per K element as a rational: bf16 2/1, 8-bit 1/1, fp4 1/2
  static constexpr int kNum = KIND == MmaKind::F16 ? 2 : 1;
  static constexpr int kDen = KIND == MmaKind::MXF4NVF4 ? 2 : 1;
  static constexpr int kSfBlock = KIND == MmaKind::MXF8F6F4 ? 32 : 16;
};

template <MmaKind KIND, int BN, int CG, int EPI, int STG = 1, int KD = 1>
int launch(const void* A, int64_t lda, const void* Bt, int64_t ldb, const uint8_t* SFA, const uint8_t* SFB,
           GemmArgs g, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
  using C = Cfg<KIND, BN, CG, EPI, STG, KD>;
  using EI = ElemInfo<KIND>;
  const int64_t k_bytes = K * EI::kNum / EI::kDen;
  const int64_t lda_b = lda * EI::kNum;  // ld counts stored elements (bytes for packed fp4)
  const int64_t ldb_b = ldb * EI::kNum;
  CUtensorMap tm_a, tm_b, tm_sfa, tm_sfb;
  const CUtensorMapDataType dt = KIND == MmaKind::F16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const uint64_t k_elems_tm = KIND == MmaKind::F16 ? K : k_bytes;  // tensor-map inner extent in its own elements
  const uint32_t box_inner = KIND == MmaKind::F16 ? 64 : 128;
  g.a_rows = M < 128 ? static_cast<int>((M + 7) / 8 * 8) : 128;
  g.stages = C::stages_for(g.a_rows);
  int rc;
  if constexpr (KD > 1) {
    // the operand seen as (128 bytes of K, rows, K slices): one box brings KD slices of the tile's rows
    if (k_bytes % 128 != 0) return GNK_ERR_BAD_SHAPE;
    const uint64_t slices = static_cast<uint64_t>(k_bytes / 128);
    const uint64_t dims_a[4] = {box_inner, static_cast<uint64_t>(M), slices, 1};
    const uint64_t dims_b[4] = {box_inner, static_cast<uint64_t>(N), slices, 1};
    const uint64_t str_a[3] = {static_cast<uint64_t>(lda_b), 128, static_cast<uint64_t>(lda_b)};
    const uint64_t str_b[3] = {static_cast<uint64_t>(ldb_b), 128, static_cast<uint64_t>(ldb_b)};
    const uint32_t box_a[4] = {box_inner, static_cast<uint32_t>(g.a_rows), KD, 1};
    const uint32_t box_b[4] = {box_inner, BN / CG, KD, 1};
    if ((rc = make_tmap_4d(&tm_a, dt, A, dims_a, str_a, box_a, CU_TENSOR_MAP_SWIZZLE_128B)) != GNK_OK) return rc;
    if ((rc = make_tmap_4d(&tm_b, dt, Bt, dims_b, str_b, box_b, CU_TENSOR_MAP_SWIZZLE_128B)) != GNK_OK) return rc;
  } else {
    rc = make_tmap_2d(&tm_a, dt, A, M, k_elems_tm, lda_b, g.a_rows, box_inner, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != GNK_OK) return rc;
    rc = make_tmap_2d(&tm_b, dt, Bt, N, k_elems_tm, ldb_b, BN / CG, box_inner, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != GNK_OK) return rc;
  }
  if constexpr (C::KI::kBlockScaled) {
    // swizzled scale buffer seen as [row groups of 128][K/(4 scales) atoms of 512 bytes], in 8-byte words
    const int64_t ks = (K + EI::kSfBlock - 1) / EI::kSfBlock;
    const int64_t atoms = (ks + 3) / 4;
    rc = make_tmap_2d(&tm_sfa, CU_TENSOR_MAP_DATA_TYPE_UINT64, SFA, (M + 127) / 128, atoms * 64, atoms * 512, 1,
                      C::kSfaBytes / C::kSfLoadsPerStage / 8, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != GNK_OK) return rc;
    rc = make_tmap_2d(&tm_sfb, CU_TENSOR_MAP_DATA_TYPE_UINT64, SFB, (N + 127) / 128, atoms * 64, atoms * 512,
                      C::kSfbGroups, C::kSfaBytes / C::kSfLoadsPerStage / 8, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != GNK_OK) return rc;
  } else {
    tm_sfa = tm_a;
    tm_sfb = tm_b;
  }
  g.k_iters = static_cast<int>((k_bytes + 128 * KD - 1) / (128 * KD));
  g.tiles_m = static_cast<int>((M + 128 * CG - 1) / (128 * CG));
  g.tiles_n = static_cast<int>((N + BN - 1) / BN);
  const int tiles = g.tiles_m * g.tiles_n;
  auto kern = gemm_kernel<KIND, BN, CG, EPI, STG, KD>;
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
  const int cap = g_max_clusters.load();
  if (cap > 0 && clusters > cap) clusters = cap;
  if (clusters > tiles) clusters = tiles;
  EpiMaps<EPI> maps;
  if (C::kBulkC && g.vec_ok) {
    rc = make_tmap_2d(&maps.c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, g.C, M, N, g.ldc * 2, 32, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != GNK_OK) return rc;
  } else {
    maps.c = tm_a;
  }
  if constexpr (KD > 1) {
    // Decode-shaped problems are short kernels issued back to back (one per layer): launched with
    // programmatic stream serialization, the next kernel's CTAs may start their set-up (barriers, TMEM,
    // descriptor prefetch) while this one drains; every such kernel waits for its predecessors
    // (griddepcontrol.wait) before it touches global memory, so the stream order of all data is kept.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(clusters * CG));
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = g_pdl.load() ? 1 : 0;
    GNK_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, tm_a, tm_b, tm_sfa, tm_sfb, maps, g));
  } else {
    kern<<<clusters * CG, 192, C::kSmemBytes, st>>>(tm_a, tm_b, tm_sfa, tm_sfb, maps, g);
  }
  GNK_LAUNCH_OK();
  return GNK_OK;
}

// Persistent grid size of a kernel: the number of clusters that can be resident at once (cached per
// instantiation and device by the caller).
template <typename K>
int resident_clusters(K kern, int cg, int threads, int smem_bytes, int* out) {
  GNK_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  int n = num_sms() / cg;
  if (cg > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(num_sms() / cg * cg));
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem_bytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = cg;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int q = 0;
    GNK_CUDA_OK(cudaOccupancyMaxActiveClusters(&q, kern, &cfg));
    if (q > 0 && q < n) n = q;
  }
  *out = n;
  return GNK_OK;
}

// Gated dual NVFP4 GEMM: X [M, K/2], W1 / W3 [N, K/2] packed E2M1; the B tile of output columns
// [128 t, 128 t + 128) is rows of W1 followed by the same rows of W3.
template <int CG>
int launch_gated(const void* X, int64_t ldx, const uint8_t* SFX, const void* W1, const uint8_t* SFW1, const void* W3,
                 const uint8_t* SFW3, int64_t ldw, GemmArgs g, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
  using C = Cfg<MmaKind::MXF4NVF4, 256, CG, EPI_GATED, 0>;
  const int64_t k_bytes = K / 2;
  CUtensorMap tm_a, tm_b, tm_sfa, tm_sfb;
  EpiMaps<EPI_GATED> maps;
  const CUtensorMapDataType u8 = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  g.a_rows = M < 128 ? static_cast<int>((M + 7) / 8 * 8) : 128;
  g.stages = C::stages_for(g.a_rows);
  int rc = make_tmap_2d(&tm_a, u8, X, M, k_bytes, ldx, g.a_rows, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != GNK_OK) return rc;
  if ((rc = make_tmap_2d(&tm_b, u8, W1, N, k_bytes, ldw, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B)) != GNK_OK) return rc;
  if ((rc = make_tmap_2d(&maps.b3, u8, W3, N, k_bytes, ldw, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B)) != GNK_OK) return rc;
  const int64_t atoms = ((K + 15) / 16 + 3) / 4;
  const CUtensorMapDataType u64 = CU_TENSOR_MAP_DATA_TYPE_UINT64;
  if ((rc = make_tmap_2d(&tm_sfa, u64, SFX, (M + 127) / 128, atoms * 64, atoms * 512, 1, C::kSfAtomBytes / 8, CU_TENSOR_MAP_SWIZZLE_NONE)) != GNK_OK) return rc;
  if ((rc = make_tmap_2d(&tm_sfb, u64, SFW1, (N + 127) / 128, atoms * 64, atoms * 512, 1, C::kSfAtomBytes / 8, CU_TENSOR_MAP_SWIZZLE_NONE)) != GNK_OK) return rc;
  if ((rc = make_tmap_2d(&maps.sfb3, u64, SFW3, (N + 127) / 128, atoms * 64, atoms * 512, 1, C::kSfAtomBytes / 8, CU_TENSOR_MAP_SWIZZLE_NONE)) != GNK_OK) return rc;
  maps.c = tm_a;
  g.k_iters = static_cast<int>((k_bytes + 127) / 128);
  g.tiles_m = static_cast<int>((M + 128 * CG - 1) / (128 * CG));
  g.tiles_n = static_cast<int>(N / 128);
  auto kern = gemm_kernel<MmaKind::MXF4NVF4, 256, CG, EPI_GATED, 0>;
  static int resident[64];
  int dev = 0;
  GNK_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return GNK_ERR_UNSUPPORTED;
  if (resident[dev] == 0) {
    int n = 0;
    if ((rc = resident_clusters(kern, CG, 192, C::kSmemBytes, &n)) != GNK_OK) return rc;
    resident[dev] = n;
  }
  int clusters = resident[dev];
  const int tiles = g.tiles_m * g.tiles_n;
  if (clusters > tiles) clusters = tiles;
  kern<<<clusters * CG, 192, C::kSmemBytes, st>>>(tm_a, tm_b, tm_sfa, tm_sfb, maps, g);
  GNK_LAUNCH_OK();
  return GNK_OK;
}

// Tile choice: the largest tile that still gives every SM work; 2-CTA 256x256 for big problems.
enum TileSel { T_2x256, T_1x256, T_1x128, T_1x64, T_2x192 };
std::atomic<int> g_force_tile{-1};  // test hook (gnk_debug_force_tile)
std::atomic<int> g_staged{-1};      // test hook (gnk_debug_staged)
std::atomic<int> g_deep_stage{1};   // test hook (gnk_debug_deep_stage): 0 keeps one K slice per stage everywhere

TileSel pick_tile(int64_t M, int64_t N, bool block_scaled) {
  const int forced = g_force_tile.load();
  if (forced >= 0) return static_cast<TileSel>(forced);
  const int sms = num_sms();
  auto ctas = [&](int64_t bm, int64_t bn) { return ((M + bm - 1) / bm) * ((N + bn - 1) / bn); };
  // T_2x192 (block-scaled kinds, by request only): two 192-wide accumulators plus the scale columns fit the
  // 512 TMEM columns side by side, so the next tile's first MMA never waits for the epilogue to free
  // shared columns.  Measured at 8192^3 it needs MORE cycles per launch than the overlapped 256-wide
  // tiles (NVFP4 314 k against 280 k, MXFP8 529 k against 506 k): a third more tiles and operand traffic
  // cost more than the hand-over they avoid.
  (void)block_scaled;
  if (ctas(256, 256) * 2 >= sms) return T_2x256;
  if (ctas(128, 256) >= sms) return T_1x256;
  if (ctas(128, 128) >= sms) return T_1x128;
  return T_1x64;
}

template <MmaKind KIND, int EPI>
int dispatch_tile(const void* A, int64_t lda, const void* Bt, int64_t ldb, const uint8_t* SFA, const uint8_t* SFB,
                  const GemmArgs& g, int64_t M, int64_t N, int64_t K, cudaStream_t st) {
  constexpr bool kBS = KindInfo<KIND>::kBlockScaled;
  switch (pick_tile(M, N, kBS)) {
    case T_2x256:
      // g_staged: 0 = direct stores from registers, anything else = bulk tensor stores through staging
      if (g_staged.load() == 0) return launch<KIND, 256, 2, EPI, 0>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K, st);
      return launch<KIND, 256, 2, EPI, 2>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K, st);
    case T_2x192:
      if constexpr (kBS) return launch<KIND, 192, 2, EPI, 2>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K, st);
      else return launch<KIND, 256, 2, EPI, 2>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K, st);
    case T_1x256: return launch<KIND, 256, 1, EPI>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K, st);
    case T_1x128: return launch<KIND, 128, 1, EPI>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K, st);
    case T_1x64:
      // One tile per CTA, a long K: the weight stream of a decode step.  The pipeline then moves
      // four (or two) 128-byte K slices per pipeline stage (rank-3 boxes), which divides the per-byte cost
      // of the producer and issuer loops that bound this shape.
      if constexpr (EPI != EPI_GATED && EPI != EPI_RS) {
        const int64_t k_bytes = K * ElemInfo<KIND>::kNum / ElemInfo<KIND>::kDen;
        const int64_t tiles = ((M + 127) / 128) * ((N + 63) / 64);
        // (not with an fp16 accumulator: the two issuing threads' partial sums are added as fp32 words)
        if (g_deep_stage.load() != 0 && !(g.f16 & 2) && k_bytes % 128 == 0 && k_bytes >= 1024 && tiles <= num_sms()) {
          // the rows of A share the stage with the weight slices: few rows leave room for four slices
          // per stage, more rows for two (the bytes of B in flight are what hides the DRAM latency)
          if (M <= 32) return launch<KIND, 64, 1, EPI, 1, 4>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K, st);
          return launch<KIND, 64, 1, EPI, 1, 2>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K, st);
        }
      }
      return launch<KIND, 64, 1, EPI>(A, lda, Bt, ldb, SFA, SFB, g, M, N, K, st);
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
  g.trace = g_trace.load();
  return g;
}

GNK_DEFINE_STATUS_READER(gemm_status_reader)

}  // namespace
}  // namespace gnk

using namespace gnk;

// Test hook: force a tile configuration (0: 2-CTA 256x256, 1: 128x256, 2: 128x128, 3: 128x64; -1: automatic).
extern "C" int gnk_debug_force_tile(int sel) {
  if (sel < -1 || sel > 4) return GNK_ERR_BAD_ARG;
  g_force_tile = sel;
  return GNK_OK;
}

// Debug: device buffer (2 CTAs x 2 roles x 256 stages x 3 int64 clock stamps + 4 int64 kernel span) or NULL to stop tracing.
extern "C" int gnk_debug_trace(void* device_buffer) {
  g_trace = static_cast<long long*>(device_buffer);
  return GNK_OK;
}

// Debug: 0 = the 64-wide tile always moves one 128-byte K slice per stage, 1 (default) = four slices per
// stage where the shape qualifies.
extern "C" int gnk_debug_deep_stage(int on) {
  g_deep_stage = on & 1;
  g_pdl = (on & 2) ? 0 : 1;  // bit 1: launch the deep-stage kernels without programmatic stream serialization
  return GNK_OK;
}

// Debug: staged epilogue of the 256x256 pair tile: -1 = default per kind, 0 = direct stores, 1 = staged.
extern "C" int gnk_debug_staged(int mode) {
  g_staged = mode;
  return GNK_OK;
}

// Host-side pipeline plan of one kernel configuration, for tests of the shared-memory arithmetic:
// out[0] = stages, out[1] = bytes per stage, out[2] = bytes the stages may use, out[3] = bytes from the start of
// the LAST stage to the end of the 128-row read the MMA makes from its last A slice (must be <= out[2] + the part
// of the last stage in front of it, i.e. (stages - 1) * out[1] + out[3] <= out[2]).
// kind: 0 bf16/fp16, 1 int8, 2 fp8, 3 mxfp8, 4 nvfp4; tile as in gnk_debug_force_tile; kd = K slices per stage.
namespace {
template <MmaKind KIND, int BN, int CG, int KD>
int stage_plan(int a_rows, int32_t* out) {
  using C = Cfg<KIND, BN, CG, EPI_BF16, 1, KD>;
  const int stage = C::kStageBytes - (128 - a_rows) * 128 * KD;
  out[0] = C::stages_for(a_rows);
  out[1] = stage;
  out[2] = KD > 1 ? C::kSmemBudget : C::kStages * C::kStageBytes;
  out[3] = (KD - 1) * a_rows * 128 + 128 * 128;
  return GNK_OK;
}
template <MmaKind KIND>
int stage_plan_kind(int tile, int kd, int a_rows, int32_t* out) {
  if (kd == 1) {
    switch (tile) {
      case 0: return stage_plan<KIND, 256, 2, 1>(a_rows, out);
      case 1: return stage_plan<KIND, 256, 1, 1>(a_rows, out);
      case 2: return stage_plan<KIND, 128, 1, 1>(a_rows, out);
      case 3: return stage_plan<KIND, 64, 1, 1>(a_rows, out);
      case 4: return stage_plan<KIND, 192, 2, 1>(a_rows, out);
    }
  } else if (tile == 3 && kd == 2) {
    return stage_plan<KIND, 64, 1, 2>(a_rows, out);
  } else if (tile == 3 && kd == 4) {
    return stage_plan<KIND, 64, 1, 4>(a_rows, out);
  }
  return GNK_ERR_BAD_ARG;
}
}  // namespace

extern "C" int gnk_debug_stage_plan(int kind, int tile, int kd, int a_rows, int32_t* out) {
  if (!out || a_rows < 8 || a_rows > 128 || a_rows % 8) return GNK_ERR_BAD_ARG;
  switch (kind) {
    case 0: return stage_plan_kind<MmaKind::F16>(tile, kd, a_rows, out);
    case 1: return stage_plan_kind<MmaKind::I8>(tile, kd, a_rows, out);
    case 2: return stage_plan_kind<MmaKind::F8F6F4>(tile, kd, a_rows, out);
    case 3: return stage_plan_kind<MmaKind::MXF8F6F4>(tile, kd, a_rows, out);
    case 4: return stage_plan_kind<MmaKind::MXF4NVF4>(tile, kd, a_rows, out);
  }
  return GNK_ERR_BAD_ARG;
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

extern "C" int gnk_mm_f16(const void* A, int64_t lda, const void* Bt, int64_t ldb, void* C, int64_t ldc, int64_t M,
                          int64_t N, int64_t K, int acc_f16, gnk_stream_t stream) {
  int rc = check_common(A, Bt, C, M, N, K, lda * 2, ldb * 2);
  if (rc != GNK_OK) return rc;
  if (K % 8 != 0) return GNK_ERR_BAD_SHAPE;
  GemmArgs g = base_args(C, ldc, M, N, 2);
  g.f16 = 1 | 4 | (acc_f16 ? 2 : 0);
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

extern "C" int gnk_gated_mm_nvfp4(const void* X, int64_t ldx, const uint8_t* SFX, const float* ts_x, const void* W1,
                                  const uint8_t* SFW1, const float* ts_w1, const void* W3, const uint8_t* SFW3,
                                  const float* ts_w3, int64_t ldw, const float* ts_out, void* C, int64_t ldc, uint8_t* SFC,
                                  int64_t M, int64_t N, int64_t K, gnk_stream_t stream) {
  if (!W3 || !SFX || !SFW1 || !SFW3 || !ts_x || !ts_w1 || !ts_w3) return GNK_ERR_BAD_ARG;
  int rc = check_common(X, W1, C, M, N, K, ldx, ldw);
  if (rc != GNK_OK) return rc;
  if (!aligned16(W3) || !aligned16(SFX) || !aligned16(SFW1) || !aligned16(SFW3) || !aligned16(C)) return GNK_ERR_BAD_ALIGN;
  if (K % 32 != 0 || N % 128 != 0) return GNK_ERR_BAD_SHAPE;
  if ((ts_out != nullptr) != (SFC != nullptr)) return GNK_ERR_BAD_ARG;
  if (ts_out ? (ldc % 8 != 0 || (reinterpret_cast<uintptr_t>(SFC) & 3)) : (ldc % 8 != 0)) return GNK_ERR_BAD_ALIGN;
  GemmArgs g = base_args(C, ldc, M, N, 2);
  g.gated.ts_x = ts_x;
  g.gated.ts_w1 = ts_w1;
  g.gated.ts_w3 = ts_w3;
  g.gated.ts_out = ts_out;
  g.gated.sfc = SFC;
  g.gated.eps = 1e-12f;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // pair tiles (256 rows) once they give every SM work, single-CTA 128-row tiles below that
  const int64_t pair_ctas = ((M + 255) / 256) * (N / 128) * 2;
  if (g_force_tile.load() != 1 && (g_force_tile.load() == 0 || pair_ctas >= num_sms()))
    return launch_gated<2>(X, ldx, SFX, W1, SFW1, W3, SFW3, ldw, g, M, N, K, st);
  return launch_gated<1>(X, ldx, SFX, W1, SFW1, W3, SFW3, ldw, g, M, N, K, st);
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

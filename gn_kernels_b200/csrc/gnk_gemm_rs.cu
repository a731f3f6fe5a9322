// BF16 GEMM fused with a reduce-scatter over NVLink peer memory (K sharded across ranks).
//
// Every rank computes its [M, N] partial tile by tile with the tcgen05 GEMM kernel; each epilogue
// warp rounds its 32 x 256 piece to bf16, stages it in shared memory and hands it to bulk tensor
// stores.  Push variant: the stores go straight into the staging slot (indexed by the sending
// rank) of the rank that owns those rows.  The warp signals the owner's flag word for the
// 128 x 256 unit (system-scope release, one signal per warp) once the stores have completed;
// that wait is deferred to the start of the warp's next tile, where it costs nothing.  Four extra
// warps per CTA on the owner take work items in the order the tiles are produced, wait (bounded)
// until a unit's flag shows all warps of all ranks, add the slots in fp32 from the owner's own
// HBM and write the bf16 output rows; the last item of a unit clears its words.  The kernel ends
// with a cross-rank exit barrier so that the next call cannot overwrite staging that a slower
// rank is still reducing.  The 128-wide fallback tile uses plain peer stores.  Only stores and
// atomics cross NVLink in this variant: every load is local, no TMA load names peer memory and
// none uses cluster multicast.
//
// Pull variant (gnk_gemm_rs_bf16_pull, for buffers that also have an NVLink multicast address):
// a finished tile stays in the rank's OWN [M, N] partial; only the flag update crosses NVLink.  The
// owner's reducer warps read each 16-byte piece once through the multicast address with
// multimem.ld_reduce (NVSwitch fetches it from every rank and adds in fp32), so an SM receives
// only the reduced data: world times less than the push variant's slot reads, which compete
// with the main loop's operand loads for the SM's L2 port.
#include <atomic>

#include "gnk_gemm_kernel.cuh"

namespace gnk {
namespace {

using namespace gnk::gemm;

GNK_DEFINE_STATUS_READER(gemm_rs_status_reader)

// test hook (gnk_debug_rs_trace): caller-owned device buffer receiving 8 globaltimer words per CTA
std::atomic<unsigned long long*> g_rs_trace{nullptr};

struct RsPlan {
  int cg, bn;
  int tiles_m, tiles_n, tiles_per_owner, rows_per_owner, units;
};

int make_plan(int64_t M, int64_t N, int world, RsPlan* p) {
  if (world < 1 || world > kMaxWorld || M <= 0 || N <= 0) return GNK_ERR_BAD_ARG;
  if (M % world != 0) return GNK_ERR_BAD_SHAPE;
  const int64_t rpo = M / world;
  if (rpo % 256 == 0 && N % 256 == 0) {
    p->cg = 2;
    p->bn = 256;
  } else if (rpo % 128 == 0 && N % 128 == 0) {
    p->cg = 1;
    p->bn = 128;
  } else {
    return GNK_ERR_BAD_SHAPE;
  }
  p->rows_per_owner = static_cast<int>(rpo);
  p->tiles_m = static_cast<int>(M / (128 * p->cg));
  p->tiles_n = static_cast<int>(N / p->bn);
  p->tiles_per_owner = p->tiles_m / world;
  p->units = static_cast<int>(rpo / 128) * p->tiles_n;
  return GNK_OK;
}

// KIND: F16 (bf16 operands) or F8F6F4 (E4M3 operands, the partial product times g.alpha before its bf16 rounding)
template <MmaKind KIND, int BN, int CG>
int launch_rs(const void* x, int64_t ldx, const void* w, int64_t ldw, GemmArgs g, int64_t M, int64_t N, int64_t K,
              cudaStream_t st) {
  using C = Cfg<KIND, BN, CG, EPI_RS>;
  constexpr bool kBf16 = KIND == MmaKind::F16;
  constexpr int kElem = kBf16 ? 2 : 1;
  const CUtensorMapDataType dt = kBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUtensorMap tm_a, tm_b;
  int rc = make_tmap_2d(&tm_a, dt, x, M, K, ldx * kElem, 128, 128 / kElem, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != GNK_OK) return rc;
  rc = make_tmap_2d(&tm_b, dt, w, N, K, ldw * kElem, BN / CG, 128 / kElem, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != GNK_OK) return rc;
  g.k_iters = static_cast<int>((K * kElem + 127) / 128);
  g.a_rows = 128;
  g.stages = C::kStages;
  auto kern = gemm_kernel<KIND, BN, CG, EPI_RS>;
  static int resident[64];
  int dev = 0;
  GNK_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return GNK_ERR_UNSUPPORTED;
  if (resident[dev] == 0) {
    GNK_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    int n = num_sms() / CG;
    if (CG > 1) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(static_cast<unsigned>(num_sms() / CG * CG));
      cfg.blockDim = dim3(320);
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
  const int tiles = g.tiles_m * g.tiles_n;
  if (clusters > tiles) clusters = tiles;
  // this rank's slot in every owner's staging buffer, as the target of the epilogue's bulk stores
  EpiMaps<EPI_RS> maps;
  for (int r = 0; r < kMaxWorld; ++r) {
    const int o = r < g.rs.world ? r : 0;
    __nv_bfloat16* slot = g.rs.staging[o] + static_cast<int64_t>(g.rs.rank) * g.rs.rows_per_owner * N;
    rc = make_tmap_2d(&maps.slot[r], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, slot, g.rs.rows_per_owner, N, N * 2, 32, 64,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != GNK_OK) return rc;
  }
  // pull variant: finished tiles go to this rank's own [M, N] partial
  rc = make_tmap_2d(&maps.local, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, g.rs.staging[g.rs.rank], M, N, N * 2, 32, 64,
                    CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != GNK_OK) return rc;
  g.rs.trace = g_rs_trace.load();
  kern<<<clusters * CG, 320, C::kSmemBytes, st>>>(tm_a, tm_b, tm_a, tm_b, maps, g);
  GNK_LAUNCH_OK();
  return GNK_OK;
}

}  // namespace
}  // namespace gnk

using namespace gnk;

// Debug: per-CTA timeline of the next reduce-scatter calls.  `device_buffer` (caller-owned, zeroed by the
// caller, 8 uint64 per CTA, room for 160 CTAs) receives globaltimer stamps: start, epilogue end,
// reducer end, reducer wait total, MMA end, epilogue store+signal total, epilogue wait total.  NULL = off.
extern "C" int gnk_debug_rs_trace(void* device_buffer) {
  g_rs_trace = static_cast<unsigned long long*>(device_buffer);
  return GNK_OK;
}

extern "C" int64_t gnk_gemm_rs_flag_words(int64_t M, int64_t N, int world) {
  RsPlan p;
  if (make_plan(M, N, world, &p) != GNK_OK) return -1;
  return 2 * p.units + 3;  // arrivals and finished-chunk counts per unit, CTA ticket, exit counter, deferred calls
}

// Host-side restatement of the device tile order, for tests: sequence index i -> the 128 x BN
// units (owner, unit index) a cluster tile signals.  out[0..3] = {owner, tm, tn, first unit},
// out[4] = units signalled by this tile (1 or 2).  Returns the number of cluster tiles.
extern "C" int64_t gnk_gemm_rs_plan(int64_t M, int64_t N, int world, int rank, int64_t i, int32_t* out) {
  RsPlan p;
  if (make_plan(M, N, world, &p) != GNK_OK) return -1;
  const int64_t total = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  if (out && i >= 0 && i < total) {
    const int owner = static_cast<int>((rank + 1 + i) % world);
    int lm, tn;
    rs_local_tile(static_cast<int>(i / world), p.tiles_per_owner, p.tiles_n, world, lm, tn);
    const int tm = owner * p.tiles_per_owner + lm;
    const int lrow0 = tm * p.cg * 128 - owner * p.rows_per_owner;
    out[0] = owner;
    out[1] = tm;
    out[2] = tn;
    out[3] = (lrow0 / 128) * p.tiles_n + tn;
    out[4] = p.cg;  // the second CTA of a pair signals unit out[3] + tiles_n
  }
  return total;
}

namespace {
int gemm_rs_impl(const void* x, int64_t ldx, const void* w, int64_t ldw, void* const* staging, const void* multicast,
                 int32_t* const* flags, void* output, int64_t ldo, int64_t M, int64_t N, int64_t K_local, int rank,
                 int world, uint32_t timeout_ms, int lagged_exit, gnk_stream_t stream, void* output_multicast = nullptr,
                 bool fp8 = false, float alpha = 1.f) {
  if (!x || !w || !output || M <= 0 || N <= 0 || K_local <= 0) return GNK_ERR_BAD_ARG;
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return GNK_ERR_BAD_ARG;
  if (!aligned16(x) || !aligned16(w) || !aligned16(output)) return GNK_ERR_BAD_ALIGN;
  const int k_align = fp8 ? 16 : 8;  // 16-byte rows for TMA
  if (K_local % k_align != 0 || ldx % k_align != 0 || ldw % k_align != 0 || ldo % 8 != 0) return GNK_ERR_BAD_SHAPE;
  int rc = check_arch();
  if (rc != GNK_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (world == 1) {  // nothing to exchange: the GEMM writes the output rows itself
    if (fp8) return GNK_ERR_UNSUPPORTED;  // the single-GPU FP8 entries take row scales, not one factor
    return gnk_mm_bf16(x, ldx, w, ldw, output, ldo, M, N, K_local, stream);
  }
  if (!staging || !flags) return GNK_ERR_BAD_ARG;
  RsPlan p;
  rc = make_plan(M, N, world, &p);
  if (rc != GNK_OK) return rc;
  GemmArgs g{};
  g.M = static_cast<int>(M);
  g.N = static_cast<int>(N);
  g.tiles_m = p.tiles_m;
  g.tiles_n = p.tiles_n;
  g.alpha = alpha;
  g.vec_ok = 1;
  g.rs.world = world;
  g.rs.rank = rank;
  g.rs.rows_per_owner = p.rows_per_owner;
  g.rs.tiles_per_owner = p.tiles_per_owner;
  g.rs.timeout_ms = timeout_ms ? timeout_ms : 20000u;
  g.rs.lagged_exit = lagged_exit ? 1 : 0;
  for (int r = 0; r < world; ++r) {
    if (!staging[r] || !flags[r] || !aligned16(staging[r])) return GNK_ERR_BAD_ARG;
    g.rs.staging[r] = static_cast<__nv_bfloat16*>(staging[r]);
    g.rs.flags[r] = reinterpret_cast<unsigned int*>(flags[r]);
  }
  g.rs.mc_partial = static_cast<const __nv_bfloat16*>(multicast);
  g.rs.mc_out = static_cast<__nv_bfloat16*>(output_multicast);
  g.rs.out = static_cast<__nv_bfloat16*>(output);
  g.rs.ldo = ldo;
  if (fp8) {
    if (p.cg == 2) return launch_rs<MmaKind::F8F6F4, 256, 2>(x, ldx, w, ldw, g, M, N, K_local, st);
    return launch_rs<MmaKind::F8F6F4, 128, 1>(x, ldx, w, ldw, g, M, N, K_local, st);
  }
  if (p.cg == 2) return launch_rs<MmaKind::F16, 256, 2>(x, ldx, w, ldw, g, M, N, K_local, st);
  return launch_rs<MmaKind::F16, 128, 1>(x, ldx, w, ldw, g, M, N, K_local, st);
}
}  // namespace

extern "C" int gnk_gemm_rs_bf16(const void* x, int64_t ldx, const void* w, int64_t ldw, void* const* staging,
                                int32_t* const* flags, void* output, int64_t ldo, int64_t M, int64_t N,
                                int64_t K_local, int rank, int world, uint32_t timeout_ms, int lagged_exit,
                                gnk_stream_t stream) {
  return gemm_rs_impl(x, ldx, w, ldw, staging, nullptr, flags, output, ldo, M, N, K_local, rank, world, timeout_ms,
                      lagged_exit, stream);
}

extern "C" int gnk_gemm_rs_bf16_pull(const void* x, int64_t ldx, const void* w, int64_t ldw, void* const* partial,
                                     const void* partial_multicast, int32_t* const* flags, void* output, int64_t ldo,
                                     int64_t M, int64_t N, int64_t K_local, int rank, int world, uint32_t timeout_ms,
                                     int lagged_exit, gnk_stream_t stream) {
  if (world > 1 && (!partial_multicast || !aligned16(partial_multicast))) return GNK_ERR_BAD_ARG;
  return gemm_rs_impl(x, ldx, w, ldw, partial, partial_multicast, flags, output, ldo, M, N, K_local, rank, world,
                      timeout_ms, lagged_exit, stream);
}

// GEMM + all-reduce: the pull variant whose owners store the reduced rows through the multicast address of
// the ranks' [M, N] outputs, so every rank ends with the whole sum.  The exit barrier always waits: a rank's
// output is complete only when every owner has finished.
extern "C" int gnk_gemm_ar_bf16(const void* x, int64_t ldx, const void* w, int64_t ldw, void* const* partial,
                                const void* partial_multicast, int32_t* const* flags, void* output,
                                void* output_multicast, int64_t ldo, int64_t M, int64_t N, int64_t K_local, int rank,
                                int world, uint32_t timeout_ms, gnk_stream_t stream) {
  if (!output) return GNK_ERR_BAD_ARG;
  if (world > 1 && (!partial_multicast || !aligned16(partial_multicast) || !output_multicast ||
                    !aligned16(output_multicast)))
    return GNK_ERR_BAD_ARG;
  return gemm_rs_impl(x, ldx, w, ldw, partial, partial_multicast, flags, output, ldo, M, N, K_local, rank, world,
                      timeout_ms, 0, stream, world > 1 ? output_multicast : nullptr);
}

// The reduce-scatter with E4M3 operands and one dequantisation factor per rank (tensor-wise scales):
// partial_r = bf16(alpha * (x_r w_r^T)) with fp32 accumulation.  partial_multicast null = push variant.
extern "C" int gnk_gemm_rs_f8(const void* x, int64_t ldx, const void* w, int64_t ldw, float alpha, void* const* partial,
                              const void* partial_multicast, int32_t* const* flags, void* output, int64_t ldo,
                              int64_t M, int64_t N, int64_t K_local, int rank, int world, uint32_t timeout_ms,
                              int lagged_exit, gnk_stream_t stream) {
  if (partial_multicast && !aligned16(partial_multicast)) return GNK_ERR_BAD_ARG;
  return gemm_rs_impl(x, ldx, w, ldw, partial, partial_multicast, flags, output, ldo, M, N, K_local, rank, world,
                      timeout_ms, lagged_exit, stream, nullptr, true, alpha);
}

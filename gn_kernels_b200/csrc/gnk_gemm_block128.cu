// FP8 (E4M3) GEMM with DeepSeek-style scaling: one fp32 scale per row of A per 128 K elements
// (SFA, stored M-major) and one per 128 x 128 block of B (SFB).  The tensor core cannot apply
// fp32 scales, so every 128-deep partial product is formed on its own in TMEM (tcgen05
// kind::f8f6f4, accumulate off at the block start) and promoted into fp32 registers:
//   acc[m][n] += partial[m][n] * (SFA[m][kb] * SFB[n/128][kb])
// The promotion, not the tensor core, sets the pace of such a kernel, so it gets most of the SM:
//   warps 0-7  promotion + store.  Warp w owns rows 32 (w & 3) .. +31 of the 128-row tile and the 128-column
//              half (w >> 2) of the 256-column tile: exactly one 128 x 128 scale block of B per warp, 128 fp32
//              accumulators per thread (packed f32x2 FMAs, TMEM read 64 columns per instruction)
//   warp 8     TMA producer (A 128 x 128, B 256 x 128 bytes per K block, 4 stages)
//   warp 9     MMA issuer: four M = 128, N = 256, K = 32 MMAs per K block into one of two 256-column
//              TMEM buffers, so the MMA of block kb + 1 overlaps the promotion of kb
//   warps 10-11 idle: they complete the warpgroup that hands its registers to the promotion warps
//              (setmaxnreg: 224 for warps 0-7, 56 for the rest)
// Persistent CTAs over 128 x 256 output tiles.  All barrier waits are bounded.
// Tried and measured slower at 8192^3: 128 x 192 tiles with TWELVE promotion warps (warp = 32 rows x 64 columns,
// one 64-column TMEM read per K block instead of two, buffer released before the FMAs, 152 registers): 1251
// TFLOP/s against 1644 for this layout, 1318 cycles per K block against 1113.  A K block costs about what the
// tcgen05.ld of its accumulator columns costs (128 KB here at ~120 bytes per clock), however the reads are
// spread over warps: the TMEM read path, not the round-trip latency of one warp, is the limit.
#include "gnk_common.cuh"

namespace gnk {
namespace {

constexpr int kTileM = 128, kTileN = 256;
constexpr int kABytes = kTileM * 128, kBBytes = kTileN * 128;
constexpr int kStageBytes = kABytes + kBBytes;  // A and B tiles of one 128-element K block
constexpr int kStages = 4;
constexpr int kSmem = kStages * kStageBytes + 2048;
constexpr int kThreads = 384;
constexpr int kPromoteRegs = 224, kRoleRegs = 56;
static_assert(2 * kPromoteRegs + kRoleRegs <= 3 * 168, "register split exceeds the launch allocation");

struct Blk128Args {
  int M, N, k_blocks, tiles_m, tiles_n;
  const float* sfa;
  int64_t ld_sfa;
  const float* sfb;
  int64_t ld_sfb;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* add;
  int64_t ld_add;
  __nv_bfloat16* C;
  int64_t ldc;
  int vec_ok;
};

__global__ void __launch_bounds__(kThreads, 1)
    gemm_block128_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                         const Blk128Args g) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  auto stage_a = [&](int s) { return base + s * kStageBytes; };
  auto stage_b = [&](int s) { return base + s * kStageBytes + kABytes; };
  const uint32_t bars = base + kStages * kStageBytes;
  auto bar_full = [&](int s) { return bars + 8 * s; };
  auto bar_empty = [&](int s) { return bars + 8 * (kStages + s); };
  auto bar_tfull = [&](int s) { return bars + 8 * (2 * kStages + s); };
  auto bar_tempty = [&](int s) { return bars + 8 * (2 * kStages + 2 + s); };
  const uint32_t tmem_slot = bars + 8 * (2 * kStages + 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = g.tiles_m * g.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_empty(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull(s), 1);
      mbar_init(bar_tempty(s), 8);  // one arrival per promotion warp
    }
    fence_mbar_init();
  }
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&tm_a);
    tma_prefetch_desc(&tm_b);
  }
  if (warp == 9) {
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
    if (warp == 8) {
      const bool leader = elect_one();
      uint32_t stage = 0, parity = 1;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int tm = t % g.tiles_m, tn = t / g.tiles_m;
        for (int kb = 0; kb < g.k_blocks; ++kb) {
          if (!mbar_wait(bar_empty(stage), parity, (0x21u << 24) | (1u << 16) | stage)) { ok = false; break; }
          if (leader) {
            mbar_expect_tx(bar_full(stage), kStageBytes);
            tma_load_2d(stage_a(stage), &tm_a, bar_full(stage), kb * 128, tm * kTileM);
            tma_load_2d(stage_b(stage), &tm_b, bar_full(stage), kb * 128, tn * kTileN);  // rows beyond N read as zero
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; parity ^= 1; }
        }
      }
    } else if (warp == 9) {
      const bool leader = elect_one();
      constexpr uint32_t kIdesc = idesc_dense(1, 0, 0, kTileM, kTileN);
      uint32_t stage = 0, parity = 0, it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < g.k_blocks; ++kb, ++it) {
          const uint32_t buf = it & 1;
          if (!mbar_wait(bar_tempty(buf), ((it >> 1) & 1) ^ 1, (0x22u << 24) | (2u << 16))) { ok = false; break; }
          if (!mbar_wait(bar_full(stage), parity, (0x22u << 24) | (3u << 16) | stage)) { ok = false; break; }
          tc_fence_after();
          const uint64_t a_desc = sdesc_k128(stage_a(stage));
          const uint64_t b_desc = sdesc_k128(stage_b(stage));
          const uint32_t d = tmem_base + buf * kTileN;
          if (leader) {
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              tc_mma<MmaKind::F8F6F4, 1>(d, a_desc + 2 * kk, b_desc + 2 * kk, kIdesc, kk != 0);
            tc_commit<1>(bar_empty(stage));
            tc_commit<1>(bar_tfull(buf));
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; parity ^= 1; }
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kPromoteRegs));
    const int quad = warp & 3, half = warp >> 2;
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const int tm = t % g.tiles_m, tn = t / g.tiles_m;
      const int row = tm * kTileM + quad * 32 + lane;
      const int rowc = min(row, g.M - 1);
      const int col0 = tn * kTileN + half * 128;  // this warp's 128 columns = one scale block of B
      const int nb = min(col0 / 128, g.N / 128 - 1);
      uint64_t acc[64];  // 128 fp32 accumulators as packed pairs
#pragma unroll
      for (int i = 0; i < 64; ++i) acc[i] = 0ull;
      // scales are fetched one K block ahead: their global-memory latency would otherwise sit in front
      // of every promotion
      const float* sfa_p = g.sfa + rowc;
      const float* sfb_p = g.sfb + nb * g.ld_sfb;
      float sa_next = __ldg(sfa_p), sb_next = __ldg(sfb_p);
      for (int kb = 0; kb < g.k_blocks; ++kb, ++it) {
        const uint32_t buf = it & 1;
        const float sf = __fmul_rn(sa_next, sb_next);
        if (kb + 1 < g.k_blocks) {
          sa_next = __ldg(sfa_p + (kb + 1) * g.ld_sfa);
          sb_next = __ldg(sfb_p + kb + 1);
        }
        const uint64_t sf2 = f2_pack(sf, sf);
        if (!mbar_wait(bar_tfull(buf), (it >> 1) & 1, (0x23u << 24) | (4u << 16))) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * kTileN + half * 128;
        // two 64-column reads per K block: the TMEM round trip (a few hundred cycles) is what a promotion
        // warp waits for, so fewer, wider reads beat more, overlapped ones
        uint32_t r[64];
        auto accumulate = [&](int c) {
#pragma unroll
          for (int i = 0; i < 64; i += 2)
            acc[c * 32 + (i >> 1)] = f2_fma(f2_pack(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), sf2, acc[c * 32 + (i >> 1)]);
        };
        tmem_ld64(taddr, r);
        tc_wait_ld();
        accumulate(0);
        tmem_ld64(taddr + 64, r);
        tc_wait_ld();
        // every column of the buffer has been read: hand it back before the last half is accumulated
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty(buf));
        accumulate(1);
      }
      if (!ok || row >= g.M || col0 >= g.N) continue;
      __nv_bfloat16* crow = g.C + static_cast<int64_t>(row) * g.ldc + col0;
#pragma unroll
      for (int i = 0; i < 128; i += 8) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; e += 2) f2_unpack(acc[(i + e) >> 1], f[e], f[e + 1]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int c = min(col0 + i + e, g.N - 1);
          if (g.add) f[e] += __bfloat162float(g.add[static_cast<int64_t>(row) * g.ld_add + c]);
          if (g.bias) f[e] += __bfloat162float(g.bias[c]);
        }
        if (g.vec_ok && col0 + i + 8 <= g.N) {
          *reinterpret_cast<uint4*>(crow + i) =
              make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
        } else {
          for (int e = 0; e < 8 && col0 + i + e < g.N; ++e) crow[i + e] = __float2bfloat16_rn(f[e]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

GNK_DEFINE_STATUS_READER(blk128_status_reader)

}  // namespace
}  // namespace gnk

using namespace gnk;

extern "C" int gnk_mm_f8_block128(const void* A, int64_t lda, const float* SFA, int64_t ld_sfa, const void* Bt,
                                  int64_t ldb, const float* SFB, int64_t ld_sfb, const void* bias, const void* add,
                                  int64_t ld_add, void* C, int64_t ldc, int64_t M, int64_t N, int64_t K,
                                  gnk_stream_t stream) {
  if (!A || !Bt || !C || !SFA || !SFB || M <= 0 || N <= 0 || K <= 0) return GNK_ERR_BAD_ARG;
  if (K % 128 != 0 || N % 128 != 0) return GNK_ERR_BAD_SHAPE;
  if (!aligned16(A) || !aligned16(Bt) || (lda & 15) || (ldb & 15)) return GNK_ERR_BAD_ALIGN;
  if (ld_sfa < M || ld_sfb < K / 128) return GNK_ERR_BAD_SHAPE;
  int rc = check_arch();
  if (rc != GNK_OK) return rc;
  CUtensorMap tm_a, tm_b;
  rc = make_tmap_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, A, M, K, lda, kTileM, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != GNK_OK) return rc;
  rc = make_tmap_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, Bt, N, K, ldb, kTileN, 128, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != GNK_OK) return rc;
  Blk128Args g{};
  g.M = static_cast<int>(M);
  g.N = static_cast<int>(N);
  g.k_blocks = static_cast<int>(K / 128);
  g.tiles_m = static_cast<int>((M + kTileM - 1) / kTileM);
  g.tiles_n = static_cast<int>((N + kTileN - 1) / kTileN);
  g.sfa = SFA;
  g.ld_sfa = ld_sfa;
  g.sfb = SFB;
  g.ld_sfb = ld_sfb;
  g.bias = static_cast<const __nv_bfloat16*>(bias);
  g.add = static_cast<const __nv_bfloat16*>(add);
  g.ld_add = ld_add;
  g.C = static_cast<__nv_bfloat16*>(C);
  g.ldc = ldc;
  g.vec_ok = aligned16(C) && (ldc % 8 == 0);
  GNK_CUDA_OK(cudaFuncSetAttribute(gemm_block128_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  int grid = num_sms();
  const int tiles = g.tiles_m * g.tiles_n;
  if (grid > tiles) grid = tiles;
  gemm_block128_kernel<<<grid, kThreads, kSmem, static_cast<cudaStream_t>(stream)>>>(tm_a, tm_b, g);
  GNK_LAUNCH_OK();
  return GNK_OK;
}

// Library core: version / error text, CUDA error capture, device checks, TMA descriptor
// encoding through the driver entry point (no link-time libcuda dependency), and the
// registry of per-translation-unit device status words.
#include <cudaTypedefs.h>

#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "gnk_common.cuh"

namespace gnk {

static thread_local char tl_cuda_error[256] = "";

void set_cuda_error(cudaError_t e, const char* where) {
  snprintf(tl_cuda_error, sizeof(tl_cuda_error), "%s: %s (%s)", where, cudaGetErrorString(e), cudaGetErrorName(e));
}

int check_arch() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return GNK_ERR_CUDA;
  static int cached_major[64];
  static bool have[64];
  if (dev < 0 || dev >= 64) return GNK_ERR_ARCH;
  if (!have[dev]) {
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return GNK_ERR_CUDA;
    cached_major[dev] = major;
    have[dev] = true;
  }
  return cached_major[dev] == 10 ? GNK_OK : GNK_ERR_ARCH;
}

int num_sms() {
  int dev = 0;
  static int cached[64];
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  });
  return fn;
}

// Descriptor cache.  A tiled tensor map is a pure function of the arguments it is encoded from, so a
// map built once for (base, extents, strides, box, type, swizzle) can be handed out again: steady-state
// callers (the same weights, activations of the same shape in the same buffers) then pay a 128-byte
// copy under a mutex instead of a driver call per operand.  Direct-mapped, 512 entries.
namespace {
struct TmapKey {
  uint64_t base, dims[4], strides[3];
  uint32_t box[4], dt, swz, rank, pad;
  bool operator==(const TmapKey& o) const { return memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
struct TmapEntry {
  TmapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int kTmapCacheSize = 512;
TmapEntry g_tmap_cache[kTmapCacheSize];
std::mutex g_tmap_mutex;

inline uint32_t tmap_slot(const TmapKey& k) {
  uint64_t h = 1469598103934665603ull;
  const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
  for (size_t i = 0; i < sizeof(TmapKey) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
  return static_cast<uint32_t>((h ^ (h >> 29)) % kTmapCacheSize);
}
bool tmap_lookup(const TmapKey& k, CUtensorMap* out) {
  TmapEntry& e = g_tmap_cache[tmap_slot(k)];
  std::lock_guard<std::mutex> lock(g_tmap_mutex);
  if (!e.used || !(e.key == k)) return false;
  memcpy(out, &e.map, sizeof(CUtensorMap));
  return true;
}
void tmap_insert(const TmapKey& k, const CUtensorMap* m) {
  TmapEntry& e = g_tmap_cache[tmap_slot(k)];
  std::lock_guard<std::mutex> lock(g_tmap_mutex);
  e.key = k;
  memcpy(&e.map, m, sizeof(CUtensorMap));
  e.used = true;
}
}  // namespace

int make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t rows, uint64_t cols,
                 uint64_t ld_bytes, uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz) {
  TmapKey key;
  memset(&key, 0, sizeof(key));
  key.base = reinterpret_cast<uint64_t>(base);
  key.dims[0] = cols; key.dims[1] = rows;
  key.strides[0] = ld_bytes;
  key.box[0] = box_cols; key.box[1] = box_rows;
  key.dt = static_cast<uint32_t>(dt); key.swz = static_cast<uint32_t>(swz); key.rank = 2;
  if (tmap_lookup(key, map)) return GNK_OK;
  auto fn = encode_fn();
  if (!fn) {
    snprintf(tl_cuda_error, sizeof(tl_cuda_error), "cuTensorMapEncodeTiled entry point not found");
    return GNK_ERR_CUDA;
  }
  if (!aligned16(base) || (ld_bytes & 15)) return GNK_ERR_BAD_ALIGN;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estride[2] = {1, 1};
  CUresult r = fn(map, dt, 2, const_cast<void*>(base), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(tl_cuda_error, sizeof(tl_cuda_error),
             "cuTensorMapEncodeTiled failed (%d): rows=%llu cols=%llu ld=%llu box=%ux%u", (int)r,
             (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld_bytes, box_rows, box_cols);
    return GNK_ERR_CUDA;
  }
  tmap_insert(key, map);
  return GNK_OK;
}

int make_tmap_4d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, const uint64_t dims[4],
                 const uint64_t strides_bytes[3], const uint32_t box[4], CUtensorMapSwizzle swz) {
  TmapKey key;
  memset(&key, 0, sizeof(key));
  key.base = reinterpret_cast<uint64_t>(base);
  for (int i = 0; i < 4; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
  for (int i = 0; i < 3; ++i) key.strides[i] = strides_bytes[i];
  key.dt = static_cast<uint32_t>(dt); key.swz = static_cast<uint32_t>(swz); key.rank = 4;
  if (tmap_lookup(key, map)) return GNK_OK;
  auto fn = encode_fn();
  if (!fn) {
    snprintf(tl_cuda_error, sizeof(tl_cuda_error), "cuTensorMapEncodeTiled entry point not found");
    return GNK_ERR_CUDA;
  }
  if (!aligned16(base)) return GNK_ERR_BAD_ALIGN;
  for (int i = 0; i < 3; ++i)
    if (strides_bytes[i] & 15) return GNK_ERR_BAD_ALIGN;
  cuuint64_t gdim[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t gstride[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t bx[4] = {box[0], box[1], box[2], box[3]};
  cuuint32_t estride[4] = {1, 1, 1, 1};
  CUresult r = fn(map, dt, 4, const_cast<void*>(base), gdim, gstride, bx, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(tl_cuda_error, sizeof(tl_cuda_error), "cuTensorMapEncodeTiled (rank 4) failed (%d)", (int)r);
    return GNK_ERR_CUDA;
  }
  tmap_insert(key, map);
  return GNK_OK;
}

static std::vector<status_reader_t>& readers() {
  static std::vector<status_reader_t> v;
  return v;
}
void register_status_reader(status_reader_t fn) { readers().push_back(fn); }

}  // namespace gnk

extern "C" int gnk_version(void) { return GNK_VERSION; }

extern "C" const char* gnk_strerror(int status) {
  switch (status) {
    case GNK_OK: return "ok";
    case GNK_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or unknown enum)";
    case GNK_ERR_BAD_SHAPE: return "shape violates a divisibility rule of the op";
    case GNK_ERR_BAD_ALIGN: return "pointer or stride not aligned as the op needs (16 bytes)";
    case GNK_ERR_ARCH: return "current device is not compute capability 10.x (sm_100a kernels only)";
    case GNK_ERR_CUDA: return "CUDA call failed (see gnk_last_cuda_error)";
    case GNK_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case GNK_ERR_TOO_LARGE: return "size beyond a documented maximum";
    case GNK_ERR_UNSUPPORTED: return "no kernel in this build for the request";
    default: return "unknown status";
  }
}

extern "C" const char* gnk_last_cuda_error(void) { return gnk::tl_cuda_error; }

extern "C" int gnk_device_status(int* status, uint32_t* detail, int clear) {
  if (!status) return GNK_ERR_BAD_ARG;
  if (cudaDeviceSynchronize() != cudaSuccess) {
    gnk::set_cuda_error(cudaGetLastError(), "cudaDeviceSynchronize");
    return GNK_ERR_CUDA;
  }
  *status = GNK_OK;
  if (detail) *detail = 0;
  for (auto fn : gnk::readers()) {
    unsigned int w[2] = {0, 0};
    if (fn(w, clear) != 0) return GNK_ERR_CUDA;
    if (w[0] && *status == GNK_OK) {
      *status = GNK_ERR_TIMEOUT;
      if (detail) *detail = w[1];
    }
  }
  return GNK_OK;
}

// Attention entry points.  The kernel template lives in gnk_attn_kernel.cuh; this file holds the
// instantiations with 8-bit Q and K (E4M3 or INT8 codes, with per-row fp32 scales or unscaled); the
// 16-bit ones (bf16 / fp16 operands, packed variable-length sequences, fp16 accumulation) are
// compiled in gnk_attn16.cu.
#include <atomic>

#include "gnk_attn_kernel.cuh"

namespace gnk {
namespace {
GNK_DEFINE_STATUS_READER(attn_status_reader)
std::atomic<long long*> g_attn_trace{nullptr};
}  // namespace

// defined in gnk_attn16.cu
int attn_fwd_16bit(const attn::AttnProblem& p, cudaStream_t st);

}  // namespace gnk

using namespace gnk;

// Test hook: device buffer of 2 * 32 * 8 int64 receiving clock64 stamps (see AttnArgs::trace); NULL = off.
extern "C" int gnk_debug_attn_trace(void* device_buffer) {
  g_attn_trace = static_cast<long long*>(device_buffer);
  return GNK_OK;
}

namespace {
void fill_strides(attn::AttnProblem& p, const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os) {
  for (int i = 0; i < 3; ++i) {
    p.q_strides[i] = qs[i];
    p.k_strides[i] = ks[i];
    p.v_strides[i] = vs[i];
    p.o_strides[i] = os[i];
  }
}

int dispatch(const attn::AttnProblem& p, cudaStream_t st) {
  using namespace gnk::attn;
  if (p.qk_kind == GNK_Q_BF16 || p.qk_kind == GNK_Q_F16) return attn_fwd_16bit(p, st);
  if (p.acc16) return GNK_ERR_UNSUPPORTED;      // fp16 accumulation is built for fp16 operands only
  if (p.q_offsets) return GNK_ERR_UNSUPPORTED;  // packed sequences: 16-bit Q and K only (as upstream)
  if (p.qk_kind == GNK_Q_INT8)
    return p.v_dtype == GNK_F16 ? launch_attn<kQkInt8, GNK_F16, 0>(p, st) : launch_attn<kQkInt8, GNK_BF16, 0>(p, st);
  if (p.qk_kind == GNK_Q_E4M3)
    return p.v_dtype == GNK_F16 ? launch_attn<kQkE4m3, GNK_F16, 0>(p, st) : launch_attn<kQkE4m3, GNK_BF16, 0>(p, st);
  return GNK_ERR_BAD_ARG;
}
}  // namespace

extern "C" int gnk_attn_fwd(const void* q, const void* k, const void* v, void* o, const float* scale_q,
                            const float* scale_k, int qk_kind, int v_dtype, int acc16, int64_t B, int64_t Lq, int64_t Lk,
                            int64_t Hq, int64_t Hkv, int64_t D, const int64_t* q_strides, const int64_t* k_strides,
                            const int64_t* v_strides, const int64_t* o_strides, int causal, gnk_stream_t stream) {
  if (!q_strides || !k_strides || !v_strides || !o_strides) return GNK_ERR_BAD_ARG;
  attn::AttnProblem p{};
  p.q = q; p.k = k; p.v = v; p.o = o;
  p.scale_q = scale_q; p.scale_k = scale_k;
  p.qk_kind = qk_kind; p.v_dtype = v_dtype; p.acc16 = acc16;
  p.B = B; p.Lq = Lq; p.Lk = Lk; p.Hq = Hq; p.Hkv = Hkv; p.D = D;
  p.causal = causal;
  p.trace = g_attn_trace.load();
  fill_strides(p, q_strides, k_strides, v_strides, o_strides);
  int rc = attn::check_attn(p);
  if (rc != GNK_OK) return rc;
  if ((qk_kind == GNK_Q_BF16 || qk_kind == GNK_Q_F16) && scale_q) return GNK_ERR_UNSUPPORTED;  // scales go with 8-bit codes
  return dispatch(p, static_cast<cudaStream_t>(stream));
}

extern "C" int gnk_attn_varlen_fwd(const void* q, const void* k, const void* v, void* o, const int32_t* q_offsets,
                                   const int32_t* kv_offsets, int qk_kind, int acc16, int64_t B, int64_t max_q_len,
                                   int64_t Lq_total, int64_t Lk_total, int64_t Hq, int64_t Hkv, int64_t D,
                                   const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                                   const int64_t* o_strides, int causal, gnk_stream_t stream) {
  if (!q_strides || !k_strides || !v_strides || !o_strides || !q_offsets || !kv_offsets) return GNK_ERR_BAD_ARG;
  if (qk_kind != GNK_Q_BF16 && qk_kind != GNK_Q_F16) return GNK_ERR_UNSUPPORTED;
  if (Lq_total <= 0 || Lk_total <= 0) return GNK_ERR_BAD_ARG;
  attn::AttnProblem p{};
  p.q = q; p.k = k; p.v = v; p.o = o;
  p.q_offsets = q_offsets; p.kv_offsets = kv_offsets;
  p.qk_kind = qk_kind; p.v_dtype = qk_kind == GNK_Q_F16 ? GNK_F16 : GNK_BF16; p.acc16 = acc16;
  p.B = B; p.Lq = max_q_len; p.Lk = 0; p.Lq_total = Lq_total; p.Lk_total = Lk_total;
  p.Hq = Hq; p.Hkv = Hkv; p.D = D;
  p.causal = causal;
  p.trace = g_attn_trace.load();
  // packed tensors are [L_total, H, D]: strides (seq, head); the batch stride slot is unused
  const int64_t qs[3] = {0, q_strides[0], q_strides[1]}, ks[3] = {0, k_strides[0], k_strides[1]};
  const int64_t vs[3] = {0, v_strides[0], v_strides[1]}, os[3] = {0, o_strides[0], o_strides[1]};
  fill_strides(p, qs, ks, vs, os);
  int rc = attn::check_attn(p);
  if (rc != GNK_OK) return rc;
  return dispatch(p, static_cast<cudaStream_t>(stream));
}

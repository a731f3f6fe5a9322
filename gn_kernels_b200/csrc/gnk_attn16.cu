// Attention instantiations with 16-bit Q and K (bf16 or fp16, unscaled): batched and packed
// variable-length sequences, and for fp16 operands the fp16-accumulation options.  V, P and O have
// the type of Q and K.
#include "gnk_attn_kernel.cuh"

namespace gnk {
namespace {
GNK_DEFINE_STATUS_READER(attn16_status_reader)
}

int attn_fwd_16bit(const attn::AttnProblem& p, cudaStream_t st) {
  using namespace gnk::attn;
  if (p.qk_kind == GNK_Q_BF16) {
    if (p.v_dtype != GNK_BF16) return GNK_ERR_UNSUPPORTED;
    if (p.acc16) return GNK_ERR_UNSUPPORTED;  // the tensor core has no bf16 accumulator; fp16 accumulation goes with fp16 operands
    return launch_attn<kQkBf16, GNK_BF16, 0>(p, st);
  }
  if (p.v_dtype != GNK_F16) return GNK_ERR_UNSUPPORTED;
  switch (p.acc16) {
    case 0: return launch_attn<kQkF16, GNK_F16, 0>(p, st);
    case 1: return launch_attn<kQkF16, GNK_F16, 1>(p, st);
    case 2: return launch_attn<kQkF16, GNK_F16, 2>(p, st);
    default: return launch_attn<kQkF16, GNK_F16, 3>(p, st);
  }
}

}  // namespace gnk

// Tensor-core (tcgen05 / TMEM / TMA) MLA flash-decode for the H=128, dC=512, dHR=64 shape.
#include "common.cuh"
#include "internal.h"
#include "splitkv.h"

namespace relux {

bool mla_sm100_eligible(const Pool* p, const relux_attn_args& a) { return false; }

int32_t launch_mla_decode_sm100(Pool* p, const SeqBatch& sb, const relux_attn_args& a, const SplitPlan& plan, const uint16_t* q_abs) {
  set_error("tensor-core MLA kernel not built");
  return RELUX_ERR_UNSUPPORTED;
}

}  // namespace relux

// Instantiates the persistent LayerNormLSTM bwd recurrence kernels for bf16 storage
// (one translation unit per combination so that they compile in parallel).
#include "recurrent_ln_kernels.cuh"

namespace hb {
namespace rec {
int run_ln_bwd_bf16(LnBwdParams& p, const Geometry& g, cudaStream_t s) { return run_ln_bwd<4, 1, __nv_bfloat16>(p, g, s); }
}  // namespace rec
}  // namespace hb

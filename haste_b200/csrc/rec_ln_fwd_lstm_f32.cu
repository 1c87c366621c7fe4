// Instantiates the persistent LayerNormLSTM fwd recurrence kernels for f32 storage
// (one translation unit per combination so that they compile in parallel).
#include "recurrent_ln_kernels.cuh"

namespace hb {
namespace rec {
int run_ln_fwd_f32(LnFwdParams& p, const Geometry& g, cudaStream_t s) { return run_ln_fwd<4, 2, float>(p, g, s); }
}  // namespace rec
}  // namespace hb

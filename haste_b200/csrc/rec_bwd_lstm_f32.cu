// Instantiates the persistent lstm bwd recurrence kernels for f32 storage
// (one translation unit per combination so that they compile in parallel).
#include "recurrent_kernels.cuh"

namespace hb {
namespace rec {
int run_bwd_lstm_f32(BwdParams& p, const Geometry& g, cudaStream_t s) { return run_bwd<4, 2, float>(p, g, s); }
}  // namespace rec
}  // namespace hb

// Instantiates the persistent lstm fwd recurrence kernels for f32 storage
// (one translation unit per combination so that they compile in parallel).
#include "recurrent_kernels.cuh"

namespace hb {
namespace rec {
int run_fwd_lstm_f32(FwdParams& p, const Geometry& g, cudaStream_t s) { return run_fwd<4, 2, float>(p, g, s); }
}  // namespace rec
}  // namespace hb

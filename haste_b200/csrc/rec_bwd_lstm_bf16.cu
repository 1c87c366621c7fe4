// Instantiates the persistent lstm bwd recurrence kernels for bf16 storage
// (one translation unit per combination so that they compile in parallel).
#include "recurrent_kernels.cuh"

namespace hb {
namespace rec {
int run_bwd_lstm_bf16(BwdParams& p, const Geometry& g, cudaStream_t s) { return run_bwd<4, 1, __nv_bfloat16>(p, g, s); }
}  // namespace rec
}  // namespace hb

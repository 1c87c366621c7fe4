// Instantiates the persistent gru bwd recurrence kernels for f16 storage: the two-plane
// arithmetic of the fp32 kernels (a __half splits exactly into two bf16 planes) on __half
// tensors (one translation unit per combination so that they compile in parallel).
#include "recurrent_kernels.cuh"

namespace hb {
namespace rec {
int run_bwd_gru_f16(BwdParams& p, const Geometry& g, cudaStream_t s) { return run_bwd<3, 2, __half>(p, g, s); }
}  // namespace rec
}  // namespace hb

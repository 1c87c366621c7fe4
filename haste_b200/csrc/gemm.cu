// hb::gemm dispatcher: tcgen05/TMA kernel when the operands qualify, CUDA cores otherwise.
#include "cells.cuh"

namespace hb {

int gemm_sm100(const GemmDesc& g, cudaStream_t stream);  // gemm_sm100.cu

int gemm(const GemmDesc& g, cudaStream_t stream) {
  const int path = gemm_path();
  if (path != HASTE_B200_GEMM_SIMT) {
    const int st_ = gemm_sm100(g, stream);
    if (st_ != HASTE_B200_ERR_UNSUPPORTED) return st_;
    if (path == HASTE_B200_GEMM_TCGEN05 || path == HASTE_B200_GEMM_TCGEN05_SINGLE) return st_;  // forced: report rather than fall through
  }
  return gemm_simt(g, stream);
}

}  // namespace hb

#include "cells.cuh"
namespace hb {
int gemm_sm100(const GemmDesc& g, cudaStream_t stream) {
  set_last_error("gemm_sm100: not available for this operand layout");
  return HASTE_B200_ERR_UNSUPPORTED;
}
}  // namespace hb

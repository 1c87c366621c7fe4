#include "cells.cuh"
namespace hb {
int lstm_forward_persistent(const LstmFwd&, cudaStream_t) { return HASTE_B200_ERR_UNSUPPORTED; }
int lstm_backward_persistent(const LstmBwd&, float*, float*, cudaStream_t) { return HASTE_B200_ERR_UNSUPPORTED; }
int gru_forward_persistent(const GruFwd&, cudaStream_t) { return HASTE_B200_ERR_UNSUPPORTED; }
int gru_backward_persistent(const GruBwd&, float*, cudaStream_t) { return HASTE_B200_ERR_UNSUPPORTED; }
}  // namespace hb

// Argument blocks and driver entry points of the six cells (internal C++ layer
// directly under the C ABI of include/haste_b200.h; field meanings are documented
// there).
#pragma once

#include "common.cuh"
#include "util.cuh"

namespace hb {

struct LstmFwd {
  int dtype, training, T, N, C, H;
  const void *W, *R, *b, *x;
  void *h, *c, *v, *tmp_Rh;
  float zoneout_prob;
  const void* zoneout_mask;
  // Single-step form (T == 1, the reference's Iterate): new state goes to separate [N,H]
  // buffers instead of slot 1 of h / c.
  void *h_out = nullptr, *c_out = nullptr;
};
struct LstmBwd {
  int dtype, transposed_inputs, T, N, C, H;
  const void *W, *R, *b, *x, *h, *c, *dh_new, *dc_new;
  void *dx, *dW, *dR, *db, *dh, *dc, *v;
  const void* zoneout_mask;
  // Single-step form (T == 1): h, c, dh_new, dc_new are the step's own [N,H] buffers and
  // c_new is the cell state the forward step produced.
  int iterate = 0;
  const void* c_new = nullptr;
};
struct GruFwd {
  int dtype, training, T, N, C, H;
  const void *W, *R, *bx, *br, *x;
  void *h, *v, *tmp_Wx, *tmp_Rh;
  float zoneout_prob;
  const void* zoneout_mask;
  void* h_out = nullptr;  // single-step form (T == 1): new state, [N,H]
};
struct GruBwd {
  int dtype, transposed_inputs, T, N, C, H;
  const void *W, *R, *bx, *br, *x, *h, *v, *dh_new;
  void *dx, *dW, *dR, *dbx, *dbr, *dh, *dp, *dq;
  const void* zoneout_mask;
  int iterate = 0;  // single-step form (T == 1): dh_new is the step's own [N,H] buffer
};
struct IndrnnFwd {
  int dtype, training, T, N, C, H;
  const void *W, *u, *b, *x;
  void *h, *workspace;
  float zoneout_prob;
  const void* zoneout_mask;
  // LayerNorm variant only (gamma == nullptr selects the plain cell)
  const void* gamma;
  void *act_Wx, *cache_Wx;
};
struct IndrnnBwd {
  int dtype, transposed_inputs, T, N, C, H;
  const void *W, *u, *b, *x, *h, *dh_new;
  void *dx, *dW, *du, *db, *dh, *workspace;
  const void* zoneout_mask;
  const void* gamma;
  void* dgamma;
  const void *act_Wx, *cache_Wx;
};
struct LnLstmFwd {
  int dtype, training, T, N, C, H;
  const void *W, *R, *b, *gamma_Wx, *gamma_Rh, *gamma_h, *beta_h, *x;
  void *h, *c, *act_Wx, *act_Wx_norm, *cache_Wx, *act_Rh, *cache_Rh, *act_c_norm, *cache_c,
      *tmp_Rh;
  float zoneout_prob;
  const void* zoneout_mask;
};
struct LnLstmBwd {
  int dtype, transposed_inputs, T, N, C, H;
  const void *W, *R, *b, *gamma_Wx, *gamma_Rh, *gamma_h, *beta_h, *x, *h, *c, *dh_new, *dc_new;
  void *dx, *dW, *dR, *db, *dgamma_Wx, *dgamma_Rh, *dgamma_h, *dbeta_h, *dh, *dc, *act_Wx, *act_Wx_norm;
  const void* cache_Wx;
  void* act_Rh;
  const void* cache_Rh;
  void* act_c_norm;
  const void* cache_c;
  const void* zoneout_mask;
};
struct LnGruFwd {
  int dtype, training, T, N, C, H;
  const void *W, *R, *bx, *br, *gamma_Wx, *gamma_Rh, *x;
  void *h, *v, *act_Wx, *cache_Wx, *tmp_Wx_norm, *act_Rh, *cache_Rh, *tmp_Rh_norm;
  float zoneout_prob;
  const void* zoneout_mask;
};
struct LnGruBwd {
  int dtype, transposed_inputs, T, N, C, H;
  const void *W, *R, *bx, *br, *gamma_Wx, *gamma_Rh, *x, *h, *v, *dh_new;
  void *dx, *dW, *dR, *dbx, *dbr, *dgamma_Wx, *dgamma_Rh, *dh, *dp, *dq;
  const void *act_Wx, *cache_Wx;
  void* act_Rh;  // overwritten with d(h.R)
  const void* cache_Rh;
  const void* zoneout_mask;
};

int lstm_forward(const LstmFwd& a, cudaStream_t s);
int lstm_backward(const LstmBwd& a, cudaStream_t s);
int gru_forward(const GruFwd& a, cudaStream_t s);
int gru_backward(const GruBwd& a, cudaStream_t s);
int indrnn_forward(const IndrnnFwd& a, cudaStream_t s);
int indrnn_backward(const IndrnnBwd& a, cudaStream_t s);
int layer_norm_lstm_forward(const LnLstmFwd& a, cudaStream_t s);
int layer_norm_lstm_backward(const LnLstmBwd& a, cudaStream_t s);
int layer_norm_gru_forward(const LnGruFwd& a, cudaStream_t s);
int layer_norm_gru_backward(const LnGruBwd& a, cudaStream_t s);

// Persistent-kernel implementations of the recurrences (recurrent_kernels.cuh).
// Each returns HASTE_B200_ERR_UNSUPPORTED (without touching any buffer) when the
// shape does not fit, in which case the caller runs its step-wise path.
// Forward: the input projection is already in a.v (LSTM) / a.tmp_Wx (GRU).
// Backward: carries are fp32 [N,H] buffers, read at entry and written at exit.
int lstm_forward_persistent(const LstmFwd& a, cudaStream_t s);
// single-step (Iterate) forward in one launch (iterate_fused.cu); UNSUPPORTED: take the general path
int lstm_forward_step_fused(const LstmFwd& a, cudaStream_t s);
int gru_forward_step_fused(const GruFwd& a, cudaStream_t s);
// Optional bf16 (hi, lo) planes of the gate gradients, written by the persistent backward
// kernels in fp32 mode (p: dv / dp, p2: dq; lo plane `stride` elements after hi).
struct GradPlanes {
  __nv_bfloat16* p = nullptr;
  __nv_bfloat16* p2 = nullptr;
  long long stride = 0;
};
int lstm_backward_persistent(const LstmBwd& a, float* dh_carry, float* dc_carry,
                             const GradPlanes& planes, cudaStream_t s);
int gru_forward_persistent(const GruFwd& a, cudaStream_t s);
int gru_backward_persistent(const GruBwd& a, float* dh_carry, const GradPlanes& planes,
                            cudaStream_t s);
// Tensor-core recurrence for bf16 batches of about a hundred rows and more (rec_tc_gru.cu);
// same contract, except that the backward kernel does not sum the bias gradients.
int gru_forward_tc(const GruFwd& a, cudaStream_t s);
int gru_backward_tc(const GruBwd& a, float* dh_carry, cudaStream_t s);
// LayerNormLSTM: forward expects LN(x.W) in a.act_Wx_norm; backward adds the LayerNorm
// parameter gradients of the recurrence into the fp32 accumulators acc = [dgamma_Rh 4H |
// dgamma_h H | dbeta_h H]; planes.p / p2 receive the gate gradient and d(h.R).
int layer_norm_lstm_forward_persistent(const LnLstmFwd& a, cudaStream_t s);
int layer_norm_lstm_backward_persistent(const LnLstmBwd& a, float* dh_carry, float* dc_carry,
                                        float* acc, const GradPlanes& planes, cudaStream_t s);
// LayerNormGRU: forward expects LN(x.W) in a.tmp_Wx_norm; backward adds dgamma_Rh into the
// fp32 accumulator acc [3H] and leaves d(h.R) in a.act_Rh.
int layer_norm_gru_forward_persistent(const LnGruFwd& a, cudaStream_t s);
int layer_norm_gru_backward_persistent(const LnGruBwd& a, float* dh_carry, float* acc,
                                       const GradPlanes& planes, cudaStream_t s);

// Exchange-only probe (recurrent_host.cu): device microseconds per step of the forward
// recurrence's hand-off alone, for the tiling (N, H) would get.
int exchange_probe(int N, int H, int steps, float* us_per_step, cudaStream_t s);

// Per-step contraction (M = batch rows).  Small products are launch-bound and stay on the
// CUDA-core kernel; from 2^26 multiply-adds up the tensor-core kernel pays for its set-up
// (operand split and tensor maps) even with a partly empty 128-row tile.
inline int gemm_small(const GemmDesc& g, cudaStream_t s) {
  if (g.M >= 32 && (long long)g.M * g.N * g.K >= (1LL << 26)) return gemm(g, s);
  return gemm_simt(g, s);
}

// Process-wide knobs (set through the C ABI).
int recurrence_path();
int sm_budget();  // 0: the whole GPU; else the SMs one recurrence launch may occupy
int gemm_path();

}  // namespace hb

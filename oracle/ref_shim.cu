// TEST INFRASTRUCTURE (not product code): a C-callable face on the REFERENCE's own
// libhaste classes, so that tests and the benchmark can run the reference's CUDA
// build on the same device buffers as haste_b200 and compare / time it.
//
// Built only by oracle/build_ref.py, from the reference sources where they lie,
// into oracle/_ref/libhaste_ref.so.  fp32 only.  The reference's pre-transposed
// argument convention (x_t, W_t, R_t) is kept as is.
#include <cublas_v2.h>
#include <cuda_runtime_api.h>

#include "haste.h"

namespace {
cublasHandle_t handle() {
  static cublasHandle_t h = nullptr;
  if (!h) cublasCreate(&h);
  return h;
}
}  // namespace

using namespace haste::v0;

extern "C" {

int ref_lstm_forward(int training, int T, int N, int C, int H, const float* W, const float* R,
                     const float* b, const float* x, float* h, float* c, float* v, float* tmp_Rh,
                     float zoneout_prob, const float* mask) {
  {
    lstm::ForwardPass<float> fw(training != 0, N, C, H, handle(), 0);
    fw.Run(T, W, R, b, x, h, c, v, tmp_Rh, zoneout_prob, mask);
  }
  return (int)cudaGetLastError();
}

int ref_lstm_backward(int T, int N, int C, int H, const float* W_t, const float* R_t,
                      const float* b, const float* x_t, const float* h, const float* c,
                      const float* dh_new, const float* dc_new, float* dx, float* dW, float* dR,
                      float* db, float* dh, float* dc, float* v, const float* mask) {
  {
    lstm::BackwardPass<float> bw(N, C, H, handle(), 0);
    bw.Run(T, W_t, R_t, b, x_t, h, c, dh_new, dc_new, dx, dW, dR, db, dh, dc, v, mask);
  }
  return (int)cudaGetLastError();
}

int ref_gru_forward(int training, int T, int N, int C, int H, const float* W, const float* R,
                    const float* bx, const float* br, const float* x, float* h, float* v,
                    float* tmp_Wx, float* tmp_Rh, float zoneout_prob, const float* mask) {
  {
    gru::ForwardPass<float> fw(training != 0, N, C, H, handle(), 0);
    fw.Run(T, W, R, bx, br, x, h, v, tmp_Wx, tmp_Rh, zoneout_prob, mask);
  }
  return (int)cudaGetLastError();
}

int ref_gru_backward(int T, int N, int C, int H, const float* W_t, const float* R_t,
                     const float* bx, const float* br, const float* x_t, const float* h,
                     const float* v, const float* dh_new, float* dx, float* dW, float* dR,
                     float* dbx, float* dbr, float* dh, float* dp, float* dq, const float* mask) {
  {
    gru::BackwardPass<float> bw(N, C, H, handle(), 0);
    bw.Run(T, W_t, R_t, bx, br, x_t, h, v, dh_new, dx, dW, dR, dbx, dbr, dh, dp, dq, mask);
  }
  return (int)cudaGetLastError();
}

int ref_indrnn_forward(int training, int T, int N, int C, int H, const float* W, const float* u,
                       const float* b, const float* x, float* h, float* workspace,
                       float zoneout_prob, const float* mask) {
  {
    indrnn::ForwardPass<float> fw(training != 0, N, C, H, handle(), 0);
    fw.Run(T, W, u, b, x, h, workspace, zoneout_prob, mask);
  }
  return (int)cudaGetLastError();
}

int ref_indrnn_backward(int T, int N, int C, int H, const float* W_t, const float* u,
                        const float* b, const float* x_t, const float* h, const float* dh_new,
                        float* dx, float* dW, float* du, float* db, float* dh, float* workspace,
                        const float* mask) {
  {
    indrnn::BackwardPass<float> bw(N, C, H, handle(), 0);
    bw.Run(T, W_t, u, b, x_t, h, dh_new, dx, dW, du, db, dh, workspace, mask);
  }
  return (int)cudaGetLastError();
}

// ---- LayerNorm cells.  The reference passes the LayerNorm parameters, statistic caches and
// gradient accumulators inside layer_norm::ForwardPass / BackwardPass objects; they are
// constructed here the way its PyTorch glue constructs them (frameworks/pytorch/
// layer_norm_lstm.cc:76-131,204-262, layer_norm_gru.cc, layer_norm_indrnn.cc:65-92,134-171).
// gamma / dgamma are [2, G*H] (row 0: x.W, row 1: h.R).

int ref_layer_norm_lstm_forward(int training, int T, int N, int C, int H, const float* W,
                                const float* R, const float* b, const float* gamma,
                                const float* gamma_h, const float* beta_h, const float* x,
                                float* h, float* c, float* act_Wx, float* act_Wx_norm,
                                float* cache_Wx, float* act_Rh, float* cache_Rh, float* act_c_norm,
                                float* cache_c, float* tmp_Rh, float zoneout_prob,
                                const float* mask) {
  {
    layer_norm::ForwardPass<float> ln1(T * N, 4 * H, gamma, nullptr, cache_Wx);
    layer_norm::ForwardPass<float> ln2(T * N, 4 * H, gamma + 4 * H, nullptr, cache_Rh);
    layer_norm::ForwardPass<float> ln3(T * N, H, gamma_h, beta_h, cache_c);
    layer_norm_lstm::ForwardPass<float> fw(training != 0, N, C, H, handle(), 0);
    fw.Run(T, W, R, b, x, h, c, act_Wx, tmp_Rh, ln1, act_Wx_norm, act_Rh, ln2, ln3, act_c_norm,
           zoneout_prob, mask);
  }
  return (int)cudaGetLastError();
}

int ref_layer_norm_lstm_backward(int T, int N, int C, int H, const float* W_t, const float* R_t,
                                 const float* b, const float* gamma, const float* gamma_h,
                                 const float* beta_h, const float* x_t, const float* h,
                                 const float* c, const float* dh_new, const float* dc_new,
                                 float* dx, float* dW, float* dR, float* db, float* dgamma,
                                 float* dgamma_h, float* dbeta_h, float* dh, float* dc,
                                 float* act_Wx, float* act_Wx_norm, float* cache_Wx, float* act_Rh,
                                 float* cache_Rh, float* act_c_norm, float* cache_c,
                                 const float* mask) {
  {
    layer_norm::BackwardPass<float> ln1(T * N, 4 * H, gamma, nullptr, act_Wx, dgamma, nullptr,
                                        cache_Wx);
    layer_norm::BackwardPass<float> ln2(T * N, 4 * H, gamma + 4 * H, nullptr, act_Rh,
                                        dgamma + 4 * H, nullptr, cache_Rh);
    layer_norm::BackwardPass<float> ln3(T * N, H, gamma_h, beta_h, c + (size_t)N * H, dgamma_h,
                                        dbeta_h, cache_c);
    layer_norm_lstm::BackwardPass<float> bw(N, C, H, handle(), 0);
    bw.Run(T, W_t, R_t, b, x_t, h, c, dh_new, dc_new, dx, dW, dR, db, dh, dc, act_Wx, ln1,
           act_Wx_norm, act_Rh, ln2, ln3, act_c_norm, mask);
  }
  return (int)cudaGetLastError();
}

int ref_layer_norm_gru_forward(int training, int T, int N, int C, int H, const float* W,
                               const float* R, const float* bx, const float* br,
                               const float* gamma, const float* x, float* h, float* v,
                               float* act_Wx, float* cache_Wx, float* tmp_Wx_norm, float* act_Rh,
                               float* cache_Rh, float* tmp_Rh_norm, float zoneout_prob,
                               const float* mask) {
  {
    layer_norm::ForwardPass<float> ln1(T * N, 3 * H, gamma, nullptr, cache_Wx);
    layer_norm::ForwardPass<float> ln2(T * N, 3 * H, gamma + 3 * H, nullptr, cache_Rh);
    layer_norm_gru::ForwardPass<float> fw(training != 0, N, C, H, handle(), 0);
    fw.Run(T, W, R, bx, br, x, h, v, act_Wx, ln1, tmp_Wx_norm, act_Rh, ln2, tmp_Rh_norm,
           zoneout_prob, mask);
  }
  return (int)cudaGetLastError();
}

int ref_layer_norm_gru_backward(int T, int N, int C, int H, const float* W_t, const float* R_t,
                                const float* bx, const float* br, const float* gamma,
                                const float* x_t, const float* h, const float* v,
                                const float* dh_new, float* dx, float* dW, float* dR, float* dbx,
                                float* dbr, float* dgamma, float* dh, float* dp, float* dq,
                                const float* act_Wx, float* cache_Wx, const float* act_Rh,
                                float* cache_Rh, const float* mask) {
  {
    layer_norm::BackwardPass<float> ln1(T * N, 3 * H, gamma, nullptr, act_Wx, dgamma, nullptr,
                                        cache_Wx);
    layer_norm::BackwardPass<float> ln2(T * N, 3 * H, gamma + 3 * H, nullptr, act_Rh,
                                        dgamma + 3 * H, nullptr, cache_Rh);
    layer_norm_gru::BackwardPass<float> bw(N, C, H, handle(), 0);
    bw.Run(T, W_t, R_t, bx, br, x_t, h, v, dh_new, dx, dW, dR, dbx, dbr, dh, dp, dq, ln1, ln2,
           mask);
  }
  return (int)cudaGetLastError();
}

int ref_layer_norm_indrnn_forward(int training, int T, int N, int C, int H, const float* W,
                                  const float* u, const float* b, const float* gamma,
                                  const float* x, float* h, float* workspace, float* act_Wx,
                                  float* cache_Wx, float zoneout_prob, const float* mask) {
  {
    layer_norm::ForwardPass<float> ln1(T * N, H, gamma, nullptr, cache_Wx);
    layer_norm_indrnn::ForwardPass<float> fw(training != 0, N, C, H, handle(), 0);
    fw.Run(T, W, u, b, x, h, workspace, act_Wx, ln1, zoneout_prob, mask);
  }
  return (int)cudaGetLastError();
}

int ref_layer_norm_indrnn_backward(int T, int N, int C, int H, const float* W_t, const float* u,
                                   const float* b, const float* gamma, const float* x_t,
                                   const float* h, const float* dh_new, float* dx, float* dW,
                                   float* du, float* db, float* dgamma, float* dh,
                                   float* workspace, const float* act_Wx, float* cache_Wx,
                                   const float* mask) {
  {
    layer_norm::BackwardPass<float> ln1(T * N, H, gamma, nullptr, act_Wx, dgamma, nullptr,
                                        cache_Wx);
    layer_norm_indrnn::BackwardPass<float> bw(N, C, H, handle(), 0);
    bw.Run(T, W_t, u, b, x_t, h, dh_new, dx, dW, du, db, dh, workspace, ln1, mask);
  }
  return (int)cudaGetLastError();
}

}  // extern "C"

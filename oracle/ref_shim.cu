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

}  // extern "C"

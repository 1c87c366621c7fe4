// extern "C" surface of libhaste_b200.so (declared in include/haste_b200.h).
// Each function packs its arguments into the driver's argument block and forwards.
#include <atomic>

#include "cells.cuh"

namespace hb {
const char* last_error();
long long launch_count();
static std::atomic<int> g_rec_path{HASTE_B200_PATH_AUTO};
static std::atomic<int> g_gemm_path{HASTE_B200_GEMM_AUTO};
static std::atomic<int> g_sm_budget{0};
int recurrence_path() { return g_rec_path.load(); }
int sm_budget() { return g_sm_budget.load(); }
int gemm_path() { return g_gemm_path.load(); }
}  // namespace hb

using namespace hb;

namespace {
// A kernel that abandoned a bounded wait can only leave a code in the pinned error word; the
// asynchronous entry point that launched it has long returned.  Every compute entry point
// therefore looks at the word first (a plain host read, no synchronisation): a time-out of an
// earlier launch surfaces at the next call instead of at some unrelated later check.
int report_timeout() {
  int d[4] = {0, 0, 0, 0};
  const int code = hb::take_error_word(d);
  if (code == 0) return HASTE_B200_OK;
  hb::set_last_error("a kernel gave up on a bounded wait (code %d, detail %d %d %d 0x%x); "
                     "results are incomplete", code, d[0], d[1], d[2], (unsigned)d[3]);
  return HASTE_B200_ERR_TIMEOUT;
}
#define HB_ENTRY() HB_TRY(report_timeout())
}  // namespace

extern "C" {

const char* haste_b200_last_error(void) { return hb::last_error(); }
const char* haste_b200_version(void) { return "0.1.0"; }
long long haste_b200_launch_count(void) { return hb::launch_count(); }

int haste_b200_profile_enable(int on) {
  hb::profile_enable(on != 0);
  return HASTE_B200_OK;
}
int haste_b200_profile_read(float* ms, int n) {
  if (!ms || n < 0) return HASTE_B200_ERR_INVALID;
  hb::profile_read(ms, n);
  return HASTE_B200_OK;
}

int haste_b200_sync_check(void* stream) {
  HB_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
  return report_timeout();
}

int haste_b200_set_recurrence_path(int path) {
  if (path < 0 || path > 3) return HASTE_B200_ERR_INVALID;
  g_rec_path.store(path);
  return HASTE_B200_OK;
}
int haste_b200_set_sm_budget(int sms) {
  if (sms < 0) return HASTE_B200_ERR_INVALID;
  g_sm_budget.store(sms);
  return HASTE_B200_OK;
}
int haste_b200_set_gemm_path(int path) {
  if (path < 0 || path > 3) return HASTE_B200_ERR_INVALID;
  g_gemm_path.store(path);
  return HASTE_B200_OK;
}

int haste_b200_lstm_forward(int dtype, int training, int T, int N, int C, int H, const void* W,
                            const void* R, const void* b, const void* x, void* h, void* c,
                            void* v, void* tmp_Rh, float zoneout_prob, const void* zoneout_mask,
                            void* stream) {
  HB_ENTRY();
  LstmFwd a{dtype, training, T, N, C, H, W, R, b, x, h, c, v, tmp_Rh, zoneout_prob, zoneout_mask};
  return lstm_forward(a, (cudaStream_t)stream);
}

int haste_b200_lstm_backward(int dtype, int transposed_inputs, int T, int N, int C, int H,
                             const void* W, const void* R, const void* b, const void* x,
                             const void* h, const void* c, const void* dh_new,
                             const void* dc_new, void* dx, void* dW, void* dR, void* db, void* dh,
                             void* dc, void* v, const void* zoneout_mask, void* stream) {
  HB_ENTRY();
  LstmBwd a{dtype, transposed_inputs, T, N, C, H, W, R, b, x, h, c, dh_new, dc_new,
            dx, dW, dR, db, dh, dc, v, zoneout_mask};
  return lstm_backward(a, (cudaStream_t)stream);
}

int haste_b200_probe_exchange_latency(int N, int H, int steps, float* us_per_step, void* stream) {
  HB_ENTRY();
  return exchange_probe(N, H, steps, us_per_step, (cudaStream_t)stream);
}

int haste_b200_lstm_forward_iterate(int dtype, int training, int N, int C, int H, const void* W,
                                    const void* R, const void* b, const void* x, const void* h,
                                    const void* c, void* h_out, void* c_out, void* v,
                                    void* tmp_Rh, float zoneout_prob, const void* zoneout_mask,
                                    void* stream) {
  HB_ENTRY();
  HB_REQUIRE(h_out && c_out, "h_out/c_out is null");
  LstmFwd a{dtype, training, 1, N, C, H, W, R, b, x, const_cast<void*>(h), const_cast<void*>(c),
            v, tmp_Rh, zoneout_prob, zoneout_mask, h_out, c_out};
  return lstm_forward(a, (cudaStream_t)stream);
}

int haste_b200_lstm_backward_iterate(int dtype, int transposed_inputs, int N, int C, int H,
                                     const void* W, const void* R, const void* b, const void* x,
                                     const void* h, const void* c, const void* c_new,
                                     const void* dh_new, const void* dc_new, void* dx, void* dW,
                                     void* dR, void* db, void* dh, void* dc, void* v,
                                     const void* zoneout_mask, void* stream) {
  HB_ENTRY();
  HB_REQUIRE(c_new, "c_new is null");
  LstmBwd a{dtype, transposed_inputs, 1, N, C, H, W, R, b, x, h, c, dh_new, dc_new,
            dx, dW, dR, db, dh, dc, v, zoneout_mask, 1, c_new};
  return lstm_backward(a, (cudaStream_t)stream);
}

int haste_b200_gru_forward_iterate(int dtype, int training, int N, int C, int H, const void* W,
                                   const void* R, const void* bx, const void* br, const void* x,
                                   const void* h, void* h_out, void* v, void* tmp_Wx,
                                   void* tmp_Rh, float zoneout_prob, const void* zoneout_mask,
                                   void* stream) {
  HB_ENTRY();
  HB_REQUIRE(h_out, "h_out is null");
  GruFwd a{dtype, training, 1, N, C, H, W, R, bx, br, x, const_cast<void*>(h), v, tmp_Wx, tmp_Rh,
           zoneout_prob, zoneout_mask, h_out};
  return gru_forward(a, (cudaStream_t)stream);
}

int haste_b200_gru_backward_iterate(int dtype, int transposed_inputs, int N, int C, int H,
                                    const void* W, const void* R, const void* bx, const void* br,
                                    const void* x, const void* h, const void* v,
                                    const void* dh_new, void* dx, void* dW, void* dR, void* dbx,
                                    void* dbr, void* dh, void* dp, void* dq,
                                    const void* zoneout_mask, void* stream) {
  HB_ENTRY();
  GruBwd a{dtype, transposed_inputs, 1, N, C, H, W, R, bx, br, x, h, v, dh_new,
           dx, dW, dR, dbx, dbr, dh, dp, dq, zoneout_mask, 1};
  return gru_backward(a, (cudaStream_t)stream);
}

int haste_b200_gru_forward(int dtype, int training, int T, int N, int C, int H, const void* W,
                           const void* R, const void* bx, const void* br, const void* x, void* h,
                           void* v, void* tmp_Wx, void* tmp_Rh, float zoneout_prob,
                           const void* zoneout_mask, void* stream) {
  HB_ENTRY();
  GruFwd a{dtype, training, T, N, C, H, W, R, bx, br, x, h, v, tmp_Wx, tmp_Rh, zoneout_prob,
           zoneout_mask};
  return gru_forward(a, (cudaStream_t)stream);
}

int haste_b200_gru_backward(int dtype, int transposed_inputs, int T, int N, int C, int H,
                            const void* W, const void* R, const void* bx, const void* br,
                            const void* x, const void* h, const void* v, const void* dh_new,
                            void* dx, void* dW, void* dR, void* dbx, void* dbr, void* dh, void* dp,
                            void* dq, const void* zoneout_mask, void* stream) {
  HB_ENTRY();
  GruBwd a{dtype, transposed_inputs, T, N, C, H, W, R, bx, br, x, h, v, dh_new,
           dx, dW, dR, dbx, dbr, dh, dp, dq, zoneout_mask};
  return gru_backward(a, (cudaStream_t)stream);
}

int haste_b200_indrnn_forward(int dtype, int training, int T, int N, int C, int H, const void* W,
                              const void* u, const void* b, const void* x, void* h,
                              void* workspace, float zoneout_prob, const void* zoneout_mask,
                              void* stream) {
  HB_ENTRY();
  IndrnnFwd a{dtype, training, T, N, C, H, W, u, b, x, h, workspace, zoneout_prob, zoneout_mask,
              nullptr, nullptr, nullptr};
  return indrnn_forward(a, (cudaStream_t)stream);
}

int haste_b200_indrnn_backward(int dtype, int transposed_inputs, int T, int N, int C, int H,
                               const void* W, const void* u, const void* b, const void* x,
                               const void* h, const void* dh_new, void* dx, void* dW, void* du,
                               void* db, void* dh, void* workspace, const void* zoneout_mask,
                               void* stream) {
  HB_ENTRY();
  IndrnnBwd a{dtype, transposed_inputs, T, N, C, H, W, u, b, x, h, dh_new, dx, dW, du, db, dh,
              workspace, zoneout_mask, nullptr, nullptr, nullptr, nullptr};
  return indrnn_backward(a, (cudaStream_t)stream);
}

int haste_b200_layer_norm_forward(int dtype, int rows, int width, const void* gamma,
                                  const void* beta, const void* x, void* y, void* cache,
                                  void* stream) {
  HB_ENTRY();
  HB_REQUIRE(dtype == HASTE_B200_F32 || dtype == HASTE_B200_BF16, "dtype");
  HB_REQUIRE(rows >= 0 && width > 0, "rows,width");
  HB_REQUIRE(gamma && x && y && cache, "null pointer");
  return layer_norm_forward(dtype, rows, width, gamma, beta, x, y, cache, (cudaStream_t)stream);
}

int haste_b200_layer_norm_backward(int dtype, int rows, int width, const void* gamma,
                                   const void* x, const void* dy, void* dx, void* dgamma,
                                   void* dbeta, const void* cache, void* stream) {
  HB_ENTRY();
  HB_REQUIRE(dtype == HASTE_B200_F32 || dtype == HASTE_B200_BF16, "dtype");
  HB_REQUIRE(rows >= 0 && width > 0, "rows,width");
  HB_REQUIRE(gamma && x && dy && dx && dgamma && cache, "null pointer");
  if (rows == 0) return HASTE_B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const size_t f = layer_norm_backward_scratch_floats(rows, width);
  float* scratch = static_cast<float*>(workspace(s, f * sizeof(float)));
  if (!scratch) return HASTE_B200_ERR_CUDA;
  return layer_norm_backward(dtype, rows, width, gamma, x, dy, dx, dtype, dgamma, dbeta, cache,
                             scratch, s);
}

int haste_b200_layer_norm_lstm_forward(
    int dtype, int training, int T, int N, int C, int H, const void* W, const void* R,
    const void* b, const void* gamma_Wx, const void* gamma_Rh, const void* gamma_h,
    const void* beta_h, const void* x,
    void* h, void* c, void* act_Wx, void* act_Wx_norm, void* cache_Wx, void* act_Rh,
    void* cache_Rh, void* act_c_norm, void* cache_c, void* tmp_Rh, float zoneout_prob,
    const void* zoneout_mask, void* stream) {
  HB_ENTRY();
  LnLstmFwd a{dtype, training, T, N, C, H, W, R, b, gamma_Wx, gamma_Rh, gamma_h, beta_h, x, h, c, act_Wx,
              act_Wx_norm, cache_Wx, act_Rh, cache_Rh, act_c_norm, cache_c, tmp_Rh, zoneout_prob,
              zoneout_mask};
  return layer_norm_lstm_forward(a, (cudaStream_t)stream);
}

int haste_b200_layer_norm_lstm_backward(
    int dtype, int transposed_inputs, int T, int N, int C, int H, const void* W, const void* R,
    const void* b, const void* gamma_Wx, const void* gamma_Rh, const void* gamma_h,
    const void* beta_h, const void* x,
    const void* h, const void* c, const void* dh_new, const void* dc_new, void* dx, void* dW,
    void* dR, void* db, void* dgamma_Wx, void* dgamma_Rh, void* dgamma_h, void* dbeta_h, void* dh,
    void* dc,
    void* act_Wx, void* act_Wx_norm, const void* cache_Wx, void* act_Rh, const void* cache_Rh,
    void* act_c_norm, const void* cache_c, const void* zoneout_mask, void* stream) {
  HB_ENTRY();
  LnLstmBwd a{dtype, transposed_inputs, T, N, C, H, W, R, b, gamma_Wx, gamma_Rh, gamma_h, beta_h,
              x, h, c, dh_new, dc_new, dx, dW, dR, db, dgamma_Wx, dgamma_Rh, dgamma_h, dbeta_h, dh,
              dc, act_Wx,
              act_Wx_norm, cache_Wx, act_Rh, cache_Rh, act_c_norm, cache_c, zoneout_mask};
  return layer_norm_lstm_backward(a, (cudaStream_t)stream);
}

int haste_b200_layer_norm_gru_forward(
    int dtype, int training, int T, int N, int C, int H, const void* W, const void* R,
    const void* bx, const void* br, const void* gamma_Wx, const void* gamma_Rh, const void* x,
    void* h, void* v,
    void* act_Wx, void* cache_Wx, void* tmp_Wx_norm, void* act_Rh, void* cache_Rh,
    void* tmp_Rh_norm, float zoneout_prob, const void* zoneout_mask, void* stream) {
  HB_ENTRY();
  LnGruFwd a{dtype, training, T, N, C, H, W, R, bx, br, gamma_Wx, gamma_Rh, x, h, v, act_Wx, cache_Wx,
             tmp_Wx_norm, act_Rh, cache_Rh, tmp_Rh_norm, zoneout_prob, zoneout_mask};
  return layer_norm_gru_forward(a, (cudaStream_t)stream);
}

int haste_b200_layer_norm_gru_backward(
    int dtype, int transposed_inputs, int T, int N, int C, int H, const void* W, const void* R,
    const void* bx, const void* br, const void* gamma_Wx, const void* gamma_Rh, const void* x,
    const void* h, const void* v, const void* dh_new, void* dx, void* dW, void* dR, void* dbx,
    void* dbr, void* dgamma_Wx, void* dgamma_Rh, void* dh, void* dp, void* dq, const void* act_Wx,
    const void* cache_Wx,
    void* act_Rh, const void* cache_Rh, const void* zoneout_mask, void* stream) {
  HB_ENTRY();
  LnGruBwd a{dtype, transposed_inputs, T, N, C, H, W, R, bx, br, gamma_Wx, gamma_Rh, x, h, v,
             dh_new, dx, dW, dR, dbx, dbr, dgamma_Wx, dgamma_Rh, dh, dp, dq, act_Wx, cache_Wx, act_Rh, cache_Rh, zoneout_mask};
  return layer_norm_gru_backward(a, (cudaStream_t)stream);
}

int haste_b200_layer_norm_indrnn_forward(
    int dtype, int training, int T, int N, int C, int H, const void* W, const void* u,
    const void* b, const void* gamma, const void* x, void* h, void* workspace, void* act_Wx,
    void* cache_Wx, float zoneout_prob, const void* zoneout_mask, void* stream) {
  HB_ENTRY();
  HB_REQUIRE(gamma, "gamma is null");
  IndrnnFwd a{dtype, training, T, N, C, H, W, u, b, x, h, workspace, zoneout_prob, zoneout_mask,
              gamma, act_Wx, cache_Wx};
  return indrnn_forward(a, (cudaStream_t)stream);
}

int haste_b200_layer_norm_indrnn_backward(
    int dtype, int transposed_inputs, int T, int N, int C, int H, const void* W, const void* u,
    const void* b, const void* gamma, const void* x, const void* h, const void* dh_new, void* dx,
    void* dW, void* du, void* db, void* dgamma, void* dh, void* workspace, const void* act_Wx,
    const void* cache_Wx, const void* zoneout_mask, void* stream) {
  HB_ENTRY();
  HB_REQUIRE(gamma, "gamma is null");
  IndrnnBwd a{dtype, transposed_inputs, T, N, C, H, W, u, b, x, h, dh_new, dx, dW, du, db, dh,
              workspace, zoneout_mask, gamma, dgamma, act_Wx, cache_Wx};
  return indrnn_backward(a, (cudaStream_t)stream);
}

int haste_b200_gemm(int dtype, int M, int N, int K, const void* a, long long a_rs, long long a_cs,
                    const void* b, long long b_rs, long long b_cs, void* c, long long ldc,
                    int accumulate, void* stream) {
  HB_ENTRY();
  HB_REQUIRE(dtype == HASTE_B200_F32 || dtype == HASTE_B200_BF16 || dtype == HASTE_B200_F16,
             "dtype");
  HB_REQUIRE(M >= 0 && N >= 0 && K >= 0, "M,N,K");
  HB_REQUIRE(a && b && c, "null pointer");
  GemmDesc g{dtype, dtype, M, N, K, a, a_rs, a_cs, b, b_rs, b_cs, c, ldc, accumulate};
  return gemm(g, (cudaStream_t)stream);
}

}  // extern "C"

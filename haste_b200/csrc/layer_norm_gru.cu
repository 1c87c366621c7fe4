// LayerNormGRU: the GRU of gru.cu fed with LN(x.W; gamma0) + bx and
// LN(h.R; gamma1) + br (biases are added after the normalisation).
// Follows lib/layer_norm_gru_forward_gpu.cu.cc:25-83,150-305 and
// lib/layer_norm_gru_backward_gpu.cu.cc:25-95,160-310.
//
// One deliberate difference in buffer use: the reference normalises dq in place,
// which forces its pointwise kernel to accumulate the recurrent-bias gradient with
// atomics beforehand.  Here LayerNorm 2's input gradient is written over act_Rh[t]
// (dead after this step), dq keeps the pre-norm gradient, and both bias gradients are
// deterministic column sums after the loop.
#include "cells.cuh"

namespace hb {

template <typename T>
int gru_launch_pointwise_fwd(bool training, bool zo, int N, int H, const T* Wx, const T* Rh,
                             const T* bx, const T* br, const T* h_prev, T* h_out, T* v,
                             float zoneout_prob, const T* mask, cudaStream_t s);
template <typename T>
int gru_launch_pointwise_bwd(int N, int H, const T* h_prev, const T* v, const T* dh_new,
                             float* dh_carry, T* dp, T* dq, const T* mask, cudaStream_t s);

namespace {

template <typename T>
int forward_steps(const LnGruFwd& a, cudaStream_t s) {
  const int N = a.N, H = a.H;
  const long long NH = (long long)N * H;
  const size_t es = sizeof(T);
  T* h = (T*)a.h;
  T* v = (T*)a.v;
  T* act_Rh = (T*)a.act_Rh;
  const T* Wx = (const T*)a.tmp_Wx_norm;
  const T* gamma1 = (const T*)a.gamma_Rh;
  const T* mask = (const T*)a.zoneout_mask;
  const bool zo = a.zoneout_prob != 0.0f && mask != nullptr;
  for (int t = 0; t < a.T; ++t) {
    T* Rh_t = act_Rh + t * NH * 3;
    GemmDesc g{a.dtype, a.dtype, N, 3 * H, H, h + t * NH, H, 1, a.R, 3LL * H, 1, Rh_t, 3LL * H, 0};
    g.precise = 1;  // LayerNorm follows: keep the product at fp32 accuracy
    HB_TRY(gemm_small(g, s));
    HB_TRY(layer_norm_forward(a.dtype, N, 3 * H, gamma1, nullptr, Rh_t, a.tmp_Rh_norm,
                              (char*)a.cache_Rh + (size_t)t * N * 2 * es, s));
    HB_TRY(gru_launch_pointwise_fwd<T>(a.training != 0, zo, N, H, Wx + t * NH * 3,
                                       (const T*)a.tmp_Rh_norm, (const T*)a.bx, (const T*)a.br,
                                       h + t * NH, h + (t + 1) * NH, v ? v + t * NH * 4 : nullptr,
                                       a.zoneout_prob, zo ? mask + t * NH : nullptr, s));
  }
  return HASTE_B200_OK;
}

template <typename T>
int backward_steps(const LnGruBwd& a, float* dh_carry, void* dgamma1, float* lns, cudaStream_t s) {
  const int N = a.N, H = a.H;
  const long long NH = (long long)N * H;
  const size_t es = sizeof(T);
  const T* h = (const T*)a.h;
  const T* v = (const T*)a.v;
  T* dp = (T*)a.dp;
  T* dq = (T*)a.dq;
  T* act_Rh = (T*)a.act_Rh;
  const T* gamma1 = (const T*)a.gamma_Rh;
  const T* mask = (const T*)a.zoneout_mask;
  const long long r_rs = a.transposed_inputs ? H : 1;
  const long long r_cs = a.transposed_inputs ? 1 : 3LL * H;
  for (int t = a.T - 1; t >= 0; --t) {
    HB_TRY(gru_launch_pointwise_bwd<T>(N, H, h + t * NH, v + t * NH * 4,
                                       (const T*)a.dh_new + (t + 1) * NH, dh_carry,
                                       dp + t * NH * 3, dq + t * NH * 3,
                                       mask ? mask + t * NH : nullptr, s));
    T* Rh_t = act_Rh + t * NH * 3;
    HB_TRY(layer_norm_backward(a.dtype, N, 3 * H, gamma1, Rh_t, dq + t * NH * 3, Rh_t,
                               HASTE_B200_F32, dgamma1, nullptr,
                               (const char*)a.cache_Rh + (size_t)t * N * 2 * es, lns, s));
    GemmDesc g{a.dtype, HASTE_B200_F32, N, H, 3 * H, Rh_t, 3LL * H, 1, a.R, r_rs, r_cs, dh_carry,
               H, 1};
    g.precise = 1;  // LayerNorm follows: keep the product at fp32 accuracy
    HB_TRY(gemm_small(g, s));
  }
  return HASTE_B200_OK;
}

}  // namespace

int layer_norm_gru_forward(const LnGruFwd& a, cudaStream_t s) {
  HB_REQUIRE(a.dtype == HASTE_B200_F32 || a.dtype == HASTE_B200_BF16, "dtype");
  HB_REQUIRE(a.T >= 0 && a.N > 0 && a.C > 0 && a.H > 0, "T,N,C,H");
  HB_REQUIRE(a.W && a.R && a.bx && a.br && a.gamma_Wx && a.gamma_Rh && a.h && a.act_Wx && a.cache_Wx &&
                 a.tmp_Wx_norm && a.act_Rh && a.cache_Rh && a.tmp_Rh_norm, "null pointer");
  HB_REQUIRE(!a.training || a.v, "v is required when training");
  if (a.T == 0) return HASTE_B200_OK;
  HB_REQUIRE(a.x, "x is null");
  const long long TN = (long long)a.T * a.N;
  HB_REQUIRE(TN < (1LL << 31), "T*N too large");
  GemmDesc g{a.dtype, a.dtype, (int)TN, 3 * a.H, a.C, a.x, a.C, 1, a.W, 3LL * a.H, 1, a.act_Wx,
             3LL * a.H, 0};
  g.precise = 1;
  HB_TRY(gemm(g, s));
  HB_TRY(layer_norm_forward(a.dtype, (int)TN, 3 * a.H, a.gamma_Wx, nullptr, a.act_Wx, a.tmp_Wx_norm,
                            a.cache_Wx, s));
  {
    const int st_ = layer_norm_gru_forward_persistent(a, s);
    if (st_ != HASTE_B200_ERR_UNSUPPORTED) return st_;
  }
  if (a.dtype == HASTE_B200_F32) return forward_steps<float>(a, s);
  return forward_steps<__nv_bfloat16>(a, s);
}

int layer_norm_gru_backward(const LnGruBwd& a, cudaStream_t s) {
  HB_REQUIRE(a.dtype == HASTE_B200_F32 || a.dtype == HASTE_B200_BF16, "dtype");
  HB_REQUIRE(a.T >= 0 && a.N > 0 && a.C > 0 && a.H > 0, "T,N,C,H");
  HB_REQUIRE(a.W && a.R && a.gamma_Wx && a.gamma_Rh && a.h && a.v && a.dh_new && a.dW && a.dR && a.dbx && a.dbr &&
                 a.dgamma_Wx && a.dgamma_Rh && a.dh && a.dp && a.dq && a.act_Wx && a.cache_Wx && a.act_Rh &&
                 a.cache_Rh, "null pointer");
  if (a.T == 0) return HASTE_B200_OK;
  HB_REQUIRE(a.x && a.dx, "x/dx is null");
  const int N = a.N, H = a.H, C = a.C;
  const long long TN = (long long)a.T * N;
  HB_REQUIRE(TN < (1LL << 31), "T*N too large");
  const size_t NH = (size_t)N * H;
  const bool bf = a.dtype == HASTE_B200_BF16;
  const size_t es = dtype_size(a.dtype);
  const size_t csf = colsum_scratch_floats((int)TN, 3 * H);
  const size_t lnf = layer_norm_backward_scratch_floats((int)TN, 3 * H);
  Arena ws;
  HB_TRY(make_arena(&ws, s, Arena::pad(NH * 4) + Arena::pad(csf * 4) + Arena::pad(lnf * 4) +
                                Arena::pad(3 * H * 4) + 2048));
  float* dh_carry = ws.take<float>(NH);
  float* cs = ws.take<float>(csf);
  float* lns = ws.take<float>(lnf);
  float* acc = ws.take<float>(3 * H);
  HB_REQUIRE(dh_carry && cs && lns && acc, "scratch arena");
  HB_TRY(to_float(a.dtype, a.dh, dh_carry, NH, s));
  // Persistent recurrence first; it adds dgamma_Rh into `acc`.
  HB_CUDA_OK(cudaMemsetAsync(acc, 0, 3 * H * sizeof(float), s));
  int st_ = layer_norm_gru_backward_persistent(a, dh_carry, acc, GradPlanes{}, s);
  bool use_acc = st_ == HASTE_B200_OK;
  if (st_ == HASTE_B200_ERR_UNSUPPORTED) {
    void* dgamma1 = a.dgamma_Rh;
    if (bf) {
      dgamma1 = acc;
      use_acc = true;
    }
    st_ = bf ? backward_steps<__nv_bfloat16>(a, dh_carry, dgamma1, lns, s)
             : backward_steps<float>(a, dh_carry, dgamma1, lns, s);
  }
  HB_TRY(st_);
  if (use_acc) HB_TRY(add_float_into(a.dtype, acc, a.dgamma_Rh, 3 * H, s));
  HB_TRY(from_float(a.dtype, dh_carry, a.dh, NH, s));

  // dp/dq hold gradients w.r.t. the normalised projections (+ bias).
  HB_TRY(colsum(a.dtype, a.dp, 3LL * H, (int)TN, 3 * H, a.dtype, a.dbx, 1, cs, s));
  HB_TRY(colsum(a.dtype, a.dq, 3LL * H, (int)TN, 3 * H, a.dtype, a.dbr, 1, cs, s));
  // LayerNorm 1 backward over all steps, in place on dp.
  HB_TRY(layer_norm_backward(a.dtype, (int)TN, 3 * H, a.gamma_Wx, a.act_Wx, a.dp, a.dp, a.dtype,
                             a.dgamma_Wx, nullptr, a.cache_Wx, lns, s));
  const bool tr = a.transposed_inputs != 0;
  GemmDesc gx{a.dtype, a.dtype, (int)TN, C, 3 * H, a.dp, 3LL * H, 1, a.W, tr ? C : 1,
              tr ? 1 : 3LL * H, a.dx, C, 0};
  HB_TRY(gemm(gx, s));
  GemmDesc gr{a.dtype, a.dtype, H, 3 * H, (int)TN, a.h, 1, H, a.act_Rh, 3LL * H, 1, a.dR,
              3LL * H, 1};
  HB_TRY(gemm(gr, s));
  GemmDesc gw{a.dtype, a.dtype, C, 3 * H, (int)TN, a.x, tr ? TN : 1, tr ? 1 : C, a.dp, 3LL * H, 1,
              a.dW, 3LL * H, 1};
  HB_TRY(gemm(gw, s));
  return HASTE_B200_OK;
}

}  // namespace hb

// LSTM forward / backward drivers and their step-wise kernels.
//
// Two implementations of the recurrence sit behind each driver:
//   * the persistent kernels of recurrent_kernels.cuh (one launch per layer pass,
//     recurrent weights resident on chip, tensor-core step product), used
//     whenever the shape fits; and
//   * the step-wise path in this file (one contraction + one pointwise launch per
//     time step), which handles every shape.
// The time-parallel contractions (x.W, dW, dR, dx) go through hb::gemm.
//
// Math follows lib/lstm_forward_gpu.cu.cc:27-87 and lib/lstm_backward_gpu.cu.cc:27-96.
#include "cells.cuh"

namespace hb {
namespace {

template <typename T, bool Training, bool Zoneout>
__global__ void lstm_pointwise_fwd(int N, int H, const T* Wx, const T* __restrict__ Rh,
                                   const T* __restrict__ b, const T* __restrict__ h_prev,
                                   const T* __restrict__ c_prev, T* __restrict__ h_out,
                                   T* __restrict__ c_out, T* v_out, float zoneout_prob,
                                   const T* __restrict__ mask) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = blockIdx.y;
  if (j >= H) return;
  const long long g0 = (long long)n * 4 * H + j;
  const long long o0 = (long long)n * H + j;
  const float i = sigmoidf_(ld(Wx + g0 + 0 * H) + ld(Rh + g0 + 0 * H) + ld(b + j + 0 * H));
  const float g = tanhf(ld(Wx + g0 + 1 * H) + ld(Rh + g0 + 1 * H) + ld(b + j + 1 * H));
  const float f = sigmoidf_(ld(Wx + g0 + 2 * H) + ld(Rh + g0 + 2 * H) + ld(b + j + 2 * H));
  const float o = sigmoidf_(ld(Wx + g0 + 3 * H) + ld(Rh + g0 + 3 * H) + ld(b + j + 3 * H));
  if (Training) {
    st(v_out + g0 + 0 * H, i);
    st(v_out + g0 + 1 * H, g);
    st(v_out + g0 + 2 * H, f);
    st(v_out + g0 + 3 * H, o);
  }
  const float c_new = f * ld(c_prev + o0) + i * g;
  float h_new = o * tanhf(c_new);
  if (Zoneout) {
    const float hp = ld(h_prev + o0);
    h_new = zoneout<Training>(h_new, hp, zoneout_prob, Training ? ld(mask + o0) : 0.f);
  }
  st(c_out + o0, c_new);
  st(h_out + o0, h_new);
}

// One reverse-time step.  dh/dc carries are fp32 whatever the storage type.
template <typename T, bool Zoneout>
__global__ void lstm_pointwise_bwd(int N, int H, const T* __restrict__ c_prev, T* v,
                                   const T* __restrict__ c_new, const T* __restrict__ dh_new,
                                   const T* __restrict__ dc_new, float* __restrict__ dh_carry,
                                   float* __restrict__ dc_carry, const T* __restrict__ mask) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = blockIdx.y;
  if (j >= H) return;
  const long long g0 = (long long)n * 4 * H + j;
  const long long o0 = (long long)n * H + j;
  float dc_total = ld(dc_new + o0) + dc_carry[o0];
  float dh_total = ld(dh_new + o0) + dh_carry[o0];
  const float c_tanh = tanhf(ld(c_new + o0));
  const float i = ld(v + g0 + 0 * H), g = ld(v + g0 + 1 * H);
  const float f = ld(v + g0 + 2 * H), o = ld(v + g0 + 3 * H);
  if (Zoneout) {
    const float m = ld(mask + o0);
    dh_carry[o0] = (1.0f - m) * dh_total;
    dh_total = m * dh_total;
  } else {
    dh_carry[o0] = 0.0f;
  }
  const float d_o = c_tanh * dh_total;
  dc_total += d_tanh(c_tanh) * (o * dh_total);
  const float df = ld(c_prev + o0) * dc_total;
  const float di = g * dc_total;
  const float dg = i * dc_total;
  dc_carry[o0] = f * dc_total;
  st(v + g0 + 0 * H, d_sigmoid(i) * di);
  st(v + g0 + 1 * H, d_tanh(g) * dg);
  st(v + g0 + 2 * H, d_sigmoid(f) * df);
  st(v + g0 + 3 * H, d_sigmoid(o) * d_o);
}

template <typename T>
int lstm_forward_stepwise(const LstmFwd& a, cudaStream_t s) {
  const int N = a.N, H = a.H;
  const long long NH = (long long)N * H;
  const T* R = (const T*)a.R;
  T* h = (T*)a.h;
  T* c = (T*)a.c;
  T* v = (T*)a.v;
  const T* mask = (const T*)a.zoneout_mask;
  const bool zo = a.zoneout_prob != 0.0f && mask != nullptr;
  dim3 block(128), grid(ceil_div(H, 128), N);
  for (int t = 0; t < a.T; ++t) {
    GemmDesc g{a.dtype, a.dtype, N, 4 * H, H, h + t * NH, H, 1, R, 4LL * H, 1, a.tmp_Rh,
               4LL * H, 0};
    HB_TRY(gemm_small(g, s));
    T* vt = v + t * NH * 4;
    const T* mt = zo ? mask + t * NH : nullptr;
    T* h_next = a.h_out ? (T*)a.h_out : h + (t + 1) * NH;
    T* c_next = a.c_out ? (T*)a.c_out : c + (t + 1) * NH;
#define HB_ARGS N, H, vt, (const T*)a.tmp_Rh, (const T*)a.b, h + t * NH, c + t * NH, \
                h_next, c_next, vt, a.zoneout_prob, mt
    if (a.training) {
      if (zo) lstm_pointwise_fwd<T, true, true><<<grid, block, 0, s>>>(HB_ARGS);
      else    lstm_pointwise_fwd<T, true, false><<<grid, block, 0, s>>>(HB_ARGS);
    } else {
      if (zo) lstm_pointwise_fwd<T, false, true><<<grid, block, 0, s>>>(HB_ARGS);
      else    lstm_pointwise_fwd<T, false, false><<<grid, block, 0, s>>>(HB_ARGS);
    }
#undef HB_ARGS
    HB_LAUNCH_OK();
    count_launch(1);
  }
  return HASTE_B200_OK;
}

template <typename T>
int lstm_backward_stepwise(const LstmBwd& a, float* dh_carry, float* dc_carry, cudaStream_t s) {
  const int N = a.N, H = a.H;
  const long long NH = (long long)N * H;
  const T* c = (const T*)a.c;
  T* v = (T*)a.v;
  const T* mask = (const T*)a.zoneout_mask;
  dim3 block(128), grid(ceil_div(H, 128), N);
  // R^T as a strided view: B(k = gate column, n = hidden unit)
  const long long r_rs = a.transposed_inputs ? H : 1;
  const long long r_cs = a.transposed_inputs ? 1 : 4LL * H;
  for (int t = a.T - 1; t >= 0; --t) {
    T* vt = v + t * NH * 4;
    const T* dh_new = (const T*)a.dh_new + (a.iterate ? 0 : (t + 1) * NH);
    const T* dc_new = (const T*)a.dc_new + (a.iterate ? 0 : (t + 1) * NH);
    const T* c_new = a.iterate ? (const T*)a.c_new : c + (t + 1) * NH;
    if (mask)
      lstm_pointwise_bwd<T, true><<<grid, block, 0, s>>>(N, H, c + t * NH, vt, c_new,
                                                         dh_new, dc_new, dh_carry, dc_carry,
                                                         mask + t * NH);
    else
      lstm_pointwise_bwd<T, false><<<grid, block, 0, s>>>(N, H, c + t * NH, vt, c_new,
                                                          dh_new, dc_new, dh_carry, dc_carry,
                                                          nullptr);
    HB_LAUNCH_OK();
    count_launch(1);
    GemmDesc g{a.dtype, HASTE_B200_F32, N, H, 4 * H, vt, 4LL * H, 1, a.R, r_rs, r_cs, dh_carry,
               H, 1};
    HB_TRY(gemm_small(g, s));
  }
  return HASTE_B200_OK;
}

}  // namespace

int lstm_forward(const LstmFwd& a, cudaStream_t s) {
  HB_REQUIRE(a.dtype == HASTE_B200_F32 || a.dtype == HASTE_B200_BF16, "dtype");
  HB_REQUIRE(a.T >= 0 && a.N > 0 && a.C > 0 && a.H > 0, "T,N,C,H");
  if (a.T == 0) return HASTE_B200_OK;  // nothing to do; scratch pointers may be null
  HB_REQUIRE(a.W && a.R && a.b && a.h && a.c && a.v && a.tmp_Rh, "null pointer");
  HB_REQUIRE(a.T == 0 || a.x, "x is null");
  if (a.T == 0) return HASTE_B200_OK;
  const long long TN = (long long)a.T * a.N;
  HB_REQUIRE(TN < (1LL << 31), "T*N too large");
  if (a.T == 1 && a.h_out && recurrence_path() != HASTE_B200_PATH_STEPWISE) {
    // the per-step (Iterate) form: one fused launch for small batches
    ProfScope p(PH_REC_FWD, s);
    const int st_ = lstm_forward_step_fused(a, s);
    if (st_ != HASTE_B200_ERR_UNSUPPORTED) return st_;
  }
  // v = x . W for all steps at once
  GemmDesc g{a.dtype, a.dtype, (int)TN, 4 * a.H, a.C, a.x, a.C, 1, a.W, 4LL * a.H, 1, a.v,
             4LL * a.H, 0};
  {
    ProfScope p(PH_PROJ, s);
    HB_TRY(gemm(g, s));
  }
  ProfScope p(PH_REC_FWD, s);
  int st_ = (a.h_out || a.c_out) ? HASTE_B200_ERR_UNSUPPORTED : lstm_forward_persistent(a, s);
  if (st_ != HASTE_B200_ERR_UNSUPPORTED) return st_;
  if (a.dtype == HASTE_B200_F32) return lstm_forward_stepwise<float>(a, s);
  return lstm_forward_stepwise<__nv_bfloat16>(a, s);
}

int lstm_backward(const LstmBwd& a, cudaStream_t s) {
  HB_REQUIRE(a.dtype == HASTE_B200_F32 || a.dtype == HASTE_B200_BF16, "dtype");
  HB_REQUIRE(a.T >= 0 && a.N > 0 && a.C > 0 && a.H > 0, "T,N,C,H");
  if (a.T == 0) return HASTE_B200_OK;  // nothing to do; scratch pointers may be null
  HB_REQUIRE(a.W && a.R && a.h && a.c && a.dh_new && a.dc_new && a.dW && a.dR && a.db &&
                 a.dh && a.dc && a.v, "null pointer");
  if (a.T == 0) return HASTE_B200_OK;
  HB_REQUIRE(a.x && a.dx, "x/dx is null");
  const int N = a.N, H = a.H, C = a.C;
  const long long TN = (long long)a.T * N;
  HB_REQUIRE(TN < (1LL << 31), "T*N too large");
  const size_t NH = (size_t)N * H;

  Arena ws;
  HB_TRY(make_arena(&ws, s, Arena::pad(2 * NH * 4) * 2 + Arena::pad(colsum_scratch_floats((int)TN, 4 * H) * 4) + 1024));
  float* dh_carry = ws.take<float>(NH);
  float* dc_carry = ws.take<float>(NH);
  float* cs = ws.take<float>(colsum_scratch_floats((int)TN, 4 * H));
  HB_REQUIRE(dh_carry && dc_carry && cs, "scratch arena");
  HB_TRY(to_float(a.dtype, a.dh, dh_carry, NH, s));
  HB_TRY(to_float(a.dtype, a.dc, dc_carry, NH, s));

  // fp32: room for the gate gradients as bf16 planes (written by the persistent kernel)
  GradPlanes planes;
  bool have_planes = false, persistent_ran = false;
  if (a.dtype == HASTE_B200_F32 && ((4 * H) % 8) == 0) {
    const size_t pe = Arena::pad((size_t)TN * 4 * H * 2) / 2;  // elements per plane
    void* pw = workspace(s, 2 * pe * 2 + 256, /*slot=*/3);
    if (pw) {
      planes.p = static_cast<__nv_bfloat16*>(pw);
      planes.stride = (long long)pe;
    }
  }
  int st_;
  {
    ProfScope p(PH_REC_BWD, s);
    st_ = a.iterate ? HASTE_B200_ERR_UNSUPPORTED
                    : lstm_backward_persistent(a, dh_carry, dc_carry, planes, s);
    have_planes = st_ == HASTE_B200_OK && planes.p != nullptr;
    persistent_ran = st_ == HASTE_B200_OK;
    if (st_ == HASTE_B200_ERR_UNSUPPORTED) {
    st_ = (a.dtype == HASTE_B200_F32) ? lstm_backward_stepwise<float>(a, dh_carry, dc_carry, s)
                                      : lstm_backward_stepwise<__nv_bfloat16>(a, dh_carry, dc_carry, s);
    }
  }
  HB_TRY(st_);
  HB_TRY(from_float(a.dtype, dh_carry, a.dh, NH, s));
  HB_TRY(from_float(a.dtype, dc_carry, a.dc, NH, s));

  // v now holds dv = d(loss)/d(pre-activation) for every step.
  // (the persistent kernel summed the bias gradient itself)
  if (!persistent_ran)
    HB_TRY(colsum(a.dtype, a.v, 4LL * H, (int)TN, 4 * H, a.dtype, a.db, 1, cs, s));
  const bool tr = a.transposed_inputs != 0;
  // dW[C,4H] += x^T . dv
  GemmDesc gw{a.dtype, a.dtype, C, 4 * H, (int)TN, a.x, tr ? TN : 1, tr ? 1 : C, a.v, 4LL * H, 1,
              a.dW, 4LL * H, 1};
  // dR[H,4H] += h[0:T]^T . dv
  GemmDesc gr{a.dtype, a.dtype, H, 4 * H, (int)TN, a.h, 1, H, a.v, 4LL * H, 1, a.dR, 4LL * H, 1};
  // dx[T*N,C] = dv . W^T
  GemmDesc gx{a.dtype, a.dtype, (int)TN, C, 4 * H, a.v, 4LL * H, 1, a.W, tr ? C : 1,
              tr ? 1 : 4LL * H, a.dx, C, 0};
  if (have_planes) {  // dv was already split into bf16 planes by the recurrence kernel
    gw.b_pl = planes.p; gw.b_pl_ld = 4LL * H; gw.b_pl_stride = planes.stride;
    gr.b_pl = planes.p; gr.b_pl_ld = 4LL * H; gr.b_pl_stride = planes.stride;
    gx.a_pl = planes.p; gx.a_pl_ld = 4LL * H; gx.a_pl_stride = planes.stride;
  }
  {
    ProfScope p(PH_WGRAD, s);
    HB_TRY(gemm(gw, s));
  }
  {
    ProfScope p(PH_WGRAD, s);
    HB_TRY(gemm(gr, s));
  }
  {
    ProfScope p(PH_DGRAD, s);
    HB_TRY(gemm(gx, s));
  }
  return HASTE_B200_OK;
}

}  // namespace hb

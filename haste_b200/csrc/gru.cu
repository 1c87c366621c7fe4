// GRU forward / backward drivers and their step-wise kernels
// (reset-after variant: g = tanh(Wx_g + r * (Rh_g + br_g) + bx_g)).
// Math follows lib/gru_forward_gpu.cu.cc:27-85 and lib/gru_backward_gpu.cu.cc:26-96.
// The same pointwise kernels serve the LayerNorm variant (layer_norm_gru.cu), which
// feeds them normalised projections.
#include "cells.cuh"

namespace hb {

template <typename T, bool Training, bool Zoneout>
__global__ void gru_pointwise_fwd(int N, int H, const T* __restrict__ Wx,
                                  const T* __restrict__ Rh, const T* __restrict__ bx,
                                  const T* __restrict__ br, const T* __restrict__ h_prev,
                                  T* __restrict__ h_out, T* __restrict__ v, float zoneout_prob,
                                  const T* __restrict__ mask) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = blockIdx.y;
  if (j >= H) return;
  const long long w0 = (long long)n * 3 * H + j;
  const long long o0 = (long long)n * H + j;
  const float z = sigmoidf_(ld(Wx + w0) + ld(Rh + w0) + ld(bx + j) + ld(br + j));
  const float r = sigmoidf_(ld(Wx + w0 + H) + ld(Rh + w0 + H) + ld(bx + j + H) + ld(br + j + H));
  const float q_g = ld(Rh + w0 + 2 * H) + ld(br + j + 2 * H);
  const float g = tanhf(ld(Wx + w0 + 2 * H) + r * q_g + ld(bx + j + 2 * H));
  if (Training) {
    const long long v0 = (long long)n * 4 * H + j;
    st(v + v0 + 0 * H, z);
    st(v + v0 + 1 * H, r);
    st(v + v0 + 2 * H, g);
    st(v + v0 + 3 * H, q_g);
  }
  const float hp = ld(h_prev + o0);
  float h_new = z * hp + (1.0f - z) * g;
  if (Zoneout) h_new = zoneout<Training>(h_new, hp, zoneout_prob, Training ? ld(mask + o0) : 0.f);
  st(h_out + o0, h_new);
}

template <typename T, bool Zoneout>
__global__ void gru_pointwise_bwd(int N, int H, const T* __restrict__ h_prev,
                                  const T* __restrict__ v, const T* __restrict__ dh_new,
                                  float* __restrict__ dh_carry, T* __restrict__ dp,
                                  T* __restrict__ dq, const T* __restrict__ mask) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = blockIdx.y;
  if (j >= H) return;
  const long long o0 = (long long)n * H + j;
  const long long v0 = (long long)n * 4 * H + j;
  float dh_total = ld(dh_new + o0) + dh_carry[o0];
  const float z = ld(v + v0), r = ld(v + v0 + H), g = ld(v + v0 + 2 * H), q_g = ld(v + v0 + 3 * H);
  float carry;
  if (Zoneout) {
    const float m = ld(mask + o0);
    carry = (1.0f - m) * dh_total;
    dh_total = m * dh_total;
    carry += z * dh_total;
  } else {
    carry = z * dh_total;
  }
  dh_carry[o0] = carry;
  const float dg = (1.0f - z) * dh_total;
  const float dz = (ld(h_prev + o0) - g) * dh_total;
  const float dp_g = d_tanh(g) * dg;
  const float dq_g = dp_g * r;
  const float dr = dp_g * q_g;
  const float dp_r = d_sigmoid(r) * dr;
  const float dp_z = d_sigmoid(z) * dz;
  const long long w0 = (long long)n * 3 * H + j;
  st(dp + w0, dp_z);
  st(dp + w0 + H, dp_r);
  st(dp + w0 + 2 * H, dp_g);
  st(dq + w0, dp_z);
  st(dq + w0 + H, dp_r);
  st(dq + w0 + 2 * H, dq_g);
}

// Launch helpers shared with layer_norm_gru.cu.
template <typename T>
int gru_launch_pointwise_fwd(bool training, bool zo, int N, int H, const T* Wx, const T* Rh,
                             const T* bx, const T* br, const T* h_prev, T* h_out, T* v,
                             float zoneout_prob, const T* mask, cudaStream_t s) {
  dim3 block(128), grid(ceil_div(H, 128), N);
#define HB_ARGS N, H, Wx, Rh, bx, br, h_prev, h_out, v, zoneout_prob, mask
  if (training) {
    if (zo) gru_pointwise_fwd<T, true, true><<<grid, block, 0, s>>>(HB_ARGS);
    else    gru_pointwise_fwd<T, true, false><<<grid, block, 0, s>>>(HB_ARGS);
  } else {
    if (zo) gru_pointwise_fwd<T, false, true><<<grid, block, 0, s>>>(HB_ARGS);
    else    gru_pointwise_fwd<T, false, false><<<grid, block, 0, s>>>(HB_ARGS);
  }
#undef HB_ARGS
  HB_LAUNCH_OK();
  count_launch(1);
  return HASTE_B200_OK;
}

template <typename T>
int gru_launch_pointwise_bwd(int N, int H, const T* h_prev, const T* v, const T* dh_new,
                             float* dh_carry, T* dp, T* dq, const T* mask, cudaStream_t s) {
  dim3 block(128), grid(ceil_div(H, 128), N);
  if (mask)
    gru_pointwise_bwd<T, true><<<grid, block, 0, s>>>(N, H, h_prev, v, dh_new, dh_carry, dp, dq, mask);
  else
    gru_pointwise_bwd<T, false><<<grid, block, 0, s>>>(N, H, h_prev, v, dh_new, dh_carry, dp, dq,
                                                       nullptr);
  HB_LAUNCH_OK();
  count_launch(1);
  return HASTE_B200_OK;
}

template int gru_launch_pointwise_fwd<float>(bool, bool, int, int, const float*, const float*,
                                             const float*, const float*, const float*, float*,
                                             float*, float, const float*, cudaStream_t);
template int gru_launch_pointwise_fwd<__nv_bfloat16>(bool, bool, int, int, const __nv_bfloat16*,
                                                     const __nv_bfloat16*, const __nv_bfloat16*,
                                                     const __nv_bfloat16*, const __nv_bfloat16*,
                                                     __nv_bfloat16*, __nv_bfloat16*, float,
                                                     const __nv_bfloat16*, cudaStream_t);
template int gru_launch_pointwise_bwd<float>(int, int, const float*, const float*, const float*,
                                             float*, float*, float*, const float*, cudaStream_t);
template int gru_launch_pointwise_bwd<__nv_bfloat16>(int, int, const __nv_bfloat16*,
                                                     const __nv_bfloat16*, const __nv_bfloat16*,
                                                     float*, __nv_bfloat16*, __nv_bfloat16*,
                                                     const __nv_bfloat16*, cudaStream_t);
template int gru_launch_pointwise_fwd<__half>(bool, bool, int, int, const __half*, const __half*,
                                              const __half*, const __half*, const __half*, __half*,
                                              __half*, float, const __half*, cudaStream_t);
template int gru_launch_pointwise_bwd<__half>(int, int, const __half*, const __half*, const __half*,
                                              float*, __half*, __half*, const __half*, cudaStream_t);

namespace {

template <typename T>
int gru_forward_stepwise(const GruFwd& a, cudaStream_t s) {
  const int N = a.N, H = a.H;
  const long long NH = (long long)N * H;
  T* h = (T*)a.h;
  T* v = (T*)a.v;
  const T* Wx = (const T*)a.tmp_Wx;
  const T* mask = (const T*)a.zoneout_mask;
  const bool zo = a.zoneout_prob != 0.0f && mask != nullptr;
  for (int t = 0; t < a.T; ++t) {
    GemmDesc g{a.dtype, a.dtype, N, 3 * H, H, h + t * NH, H, 1, a.R, 3LL * H, 1, a.tmp_Rh,
               3LL * H, 0};
    HB_TRY(gemm_small(g, s));
    HB_TRY(gru_launch_pointwise_fwd<T>(a.training != 0, zo, N, H, Wx + t * NH * 3,
                                       (const T*)a.tmp_Rh, (const T*)a.bx, (const T*)a.br,
                                       h + t * NH, a.h_out ? (T*)a.h_out : h + (t + 1) * NH,
                                       v ? v + t * NH * 4 : nullptr,
                                       a.zoneout_prob, zo ? mask + t * NH : nullptr, s));
  }
  return HASTE_B200_OK;
}

template <typename T>
int gru_backward_stepwise(const GruBwd& a, float* dh_carry, cudaStream_t s) {
  const int N = a.N, H = a.H;
  const long long NH = (long long)N * H;
  const T* h = (const T*)a.h;
  const T* v = (const T*)a.v;
  T* dp = (T*)a.dp;
  T* dq = (T*)a.dq;
  const T* mask = (const T*)a.zoneout_mask;
  const long long r_rs = a.transposed_inputs ? H : 1;
  const long long r_cs = a.transposed_inputs ? 1 : 3LL * H;
  for (int t = a.T - 1; t >= 0; --t) {
    HB_TRY(gru_launch_pointwise_bwd<T>(N, H, h + t * NH, v + t * NH * 4,
                                       (const T*)a.dh_new + (a.iterate ? 0 : (t + 1) * NH),
                                       dh_carry, dp + t * NH * 3, dq + t * NH * 3,
                                       mask ? mask + t * NH : nullptr, s));
    GemmDesc g{a.dtype, HASTE_B200_F32, N, H, 3 * H, dq + t * NH * 3, 3LL * H, 1, a.R, r_rs, r_cs,
               dh_carry, H, 1};
    HB_TRY(gemm_small(g, s));
  }
  return HASTE_B200_OK;
}

}  // namespace

int gru_forward(const GruFwd& a, cudaStream_t s) {
  HB_REQUIRE(a.dtype == HASTE_B200_F32 || a.dtype == HASTE_B200_BF16 || a.dtype == HASTE_B200_F16,
             "dtype");
  HB_REQUIRE(a.T >= 0 && a.N > 0 && a.C > 0 && a.H > 0, "T,N,C,H");
  if (a.T == 0) return HASTE_B200_OK;  // nothing to do; scratch pointers may be null
  HB_REQUIRE(a.W && a.R && a.bx && a.br && a.h && a.tmp_Wx && a.tmp_Rh, "null pointer");
  HB_REQUIRE(!a.training || a.v, "v is required when training");
  if (a.T == 0) return HASTE_B200_OK;
  HB_REQUIRE(a.x, "x is null");
  const long long TN = (long long)a.T * a.N;
  HB_REQUIRE(TN < (1LL << 31), "T*N too large");
  if (a.T == 1 && a.h_out && recurrence_path() != HASTE_B200_PATH_STEPWISE) {
    // the per-step (Iterate) form: one fused launch for small batches
    ProfScope p(PH_REC_FWD, s);
    const int st_ = gru_forward_step_fused(a, s);
    if (st_ != HASTE_B200_ERR_UNSUPPORTED) return st_;
  }
  GemmDesc g{a.dtype, a.dtype, (int)TN, 3 * a.H, a.C, a.x, a.C, 1, a.W, 3LL * a.H, 1, a.tmp_Wx,
             3LL * a.H, 0};
  {
    ProfScope p(PH_PROJ, s);
    HB_TRY(gemm(g, s));
  }
  ProfScope p(PH_REC_FWD, s);
  // large bf16 batches: the tensor-core recurrence; small batches: the register-resident one
  int st_ = gru_forward_tc(a, s);
  if (st_ != HASTE_B200_ERR_UNSUPPORTED) return st_;
  st_ = a.h_out ? HASTE_B200_ERR_UNSUPPORTED : gru_forward_persistent(a, s);
  if (st_ != HASTE_B200_ERR_UNSUPPORTED) return st_;
  if (a.dtype == HASTE_B200_F32) return gru_forward_stepwise<float>(a, s);
  if (a.dtype == HASTE_B200_F16) return gru_forward_stepwise<__half>(a, s);
  return gru_forward_stepwise<__nv_bfloat16>(a, s);
}

int gru_backward(const GruBwd& a, cudaStream_t s) {
  HB_REQUIRE(a.dtype == HASTE_B200_F32 || a.dtype == HASTE_B200_BF16 || a.dtype == HASTE_B200_F16,
             "dtype");
  HB_REQUIRE(a.T >= 0 && a.N > 0 && a.C > 0 && a.H > 0, "T,N,C,H");
  if (a.T == 0) return HASTE_B200_OK;  // nothing to do; scratch pointers may be null
  HB_REQUIRE(a.W && a.R && a.h && a.v && a.dh_new && a.dW && a.dR && a.dbx && a.dbr && a.dh &&
                 a.dp && a.dq, "null pointer");
  if (a.T == 0) return HASTE_B200_OK;
  HB_REQUIRE(a.x && a.dx, "x/dx is null");
  const int N = a.N, H = a.H, C = a.C;
  const long long TN = (long long)a.T * N;
  HB_REQUIRE(TN < (1LL << 31), "T*N too large");
  const size_t NH = (size_t)N * H;
  Arena ws;
  const size_t csf = colsum_scratch_floats((int)TN, 3 * H);
  HB_TRY(make_arena(&ws, s, Arena::pad(NH * 4) + Arena::pad(csf * 4) + 1024));
  float* dh_carry = ws.take<float>(NH);
  float* cs = ws.take<float>(csf);
  HB_REQUIRE(dh_carry && cs, "scratch arena");
  HB_TRY(to_float(a.dtype, a.dh, dh_carry, NH, s));
  GradPlanes planes;
  bool have_planes = false, persistent_ran = false;
  if (a.dtype == HASTE_B200_F32 && ((3 * H) % 8) == 0) {
    const size_t pe = Arena::pad((size_t)TN * 3 * H * 2) / 2;  // elements per plane
    void* pw = workspace(s, 4 * pe * 2 + 256, /*slot=*/3);
    if (pw) {
      planes.p = static_cast<__nv_bfloat16*>(pw);
      planes.p2 = planes.p + 2 * pe;
      planes.stride = (long long)pe;
    }
  }
  int st_;
  {
    ProfScope p(PH_REC_BWD, s);
    st_ = gru_backward_tc(a, dh_carry, s);
    if (st_ == HASTE_B200_OK) {
      // the tensor-core kernel leaves the recurrent contribution of the last processed step
      // (t = 0) out of dh: dh += dq_0 . R^T
      GemmDesc gd{a.dtype, HASTE_B200_F32, N, H, 3 * H, a.dq, 3LL * H, 1, a.R,
                  a.transposed_inputs ? H : 1, a.transposed_inputs ? 1 : 3LL * H, dh_carry, H, 1};
      st_ = gemm_small(gd, s);
    } else if (st_ == HASTE_B200_ERR_UNSUPPORTED) {
      st_ = a.iterate ? HASTE_B200_ERR_UNSUPPORTED
                      : gru_backward_persistent(a, dh_carry, planes, s);
      have_planes = st_ == HASTE_B200_OK && planes.p != nullptr;
      persistent_ran = st_ == HASTE_B200_OK;
    }
    if (st_ == HASTE_B200_ERR_UNSUPPORTED) {
    st_ = (a.dtype == HASTE_B200_F32)   ? gru_backward_stepwise<float>(a, dh_carry, s)
          : (a.dtype == HASTE_B200_F16) ? gru_backward_stepwise<__half>(a, dh_carry, s)
                                        : gru_backward_stepwise<__nv_bfloat16>(a, dh_carry, s);
    }
  }
  HB_TRY(st_);
  HB_TRY(from_float(a.dtype, dh_carry, a.dh, NH, s));
  if (!persistent_ran) {  // (the persistent kernel summed the bias gradients itself)
    HB_TRY(colsum(a.dtype, a.dp, 3LL * H, (int)TN, 3 * H, a.dtype, a.dbx, 1, cs, s));
    HB_TRY(colsum(a.dtype, a.dq, 3LL * H, (int)TN, 3 * H, a.dtype, a.dbr, 1, cs, s));
  }
  const bool tr = a.transposed_inputs != 0;
  GemmDesc gx{a.dtype, a.dtype, (int)TN, C, 3 * H, a.dp, 3LL * H, 1, a.W, tr ? C : 1,
              tr ? 1 : 3LL * H, a.dx, C, 0};
  if (have_planes) {  // dp was already split into bf16 planes by the recurrence kernel
    gx.a_pl = planes.p; gx.a_pl_ld = 3LL * H; gx.a_pl_stride = planes.stride;
  }
  {
    ProfScope p(PH_DGRAD, s);
    HB_TRY(gemm(gx, s));
  }
  GemmDesc gr{a.dtype, a.dtype, H, 3 * H, (int)TN, a.h, 1, H, a.dq, 3LL * H, 1, a.dR, 3LL * H, 1};
  if (have_planes) {
    gr.b_pl = planes.p2; gr.b_pl_ld = 3LL * H; gr.b_pl_stride = planes.stride;
  }
  {
    ProfScope p(PH_WGRAD, s);
    HB_TRY(gemm(gr, s));
  }
  GemmDesc gw{a.dtype, a.dtype, C, 3 * H, (int)TN, a.x, tr ? TN : 1, tr ? 1 : C, a.dp, 3LL * H, 1,
              a.dW, 3LL * H, 1};
  if (have_planes) {
    gw.b_pl = planes.p; gw.b_pl_ld = 3LL * H; gw.b_pl_stride = planes.stride;
  }
  {
    ProfScope p(PH_WGRAD, s);
    HB_TRY(gemm(gw, s));
  }
  return HASTE_B200_OK;
}

}  // namespace hb

// LayerNormLSTM: v = LN(x.W; gamma0) + LN(h.R; gamma1) + b, c' = f*c + i*g,
// h' = o * tanh(LN(c'; gamma_h, beta_h)), with zoneout on h.
//
// Buffers and their reuse follow the reference so that the saved-tensor contract is
// the same (lib/layer_norm_lstm_forward_gpu.cu.cc:26-109,191-340 and
// lib/layer_norm_lstm_backward_gpu.cu.cc:27-118,207-352):
//   forward : act_Wx = x.W, act_Wx_norm = LN1(act_Wx) then overwritten per step with
//             the gate activations, act_Rh[t] = h_t.R (pre-norm), c = un-normalised
//             cell state, act_c_norm[t] = LN3(c[t+1]).
//   backward: act_c_norm[t] is overwritten with d/dLN3, then d/dc'; act_Wx_norm[t]
//             with the gate pre-activation gradients; act_Rh[t] with d/d(h.R);
//             act_Wx with d/d(x.W).
#include "cells.cuh"

namespace hb {
namespace {

template <typename T, bool Training>
__global__ void lnlstm_cell_state(int N, int H, T* v, const T* __restrict__ Rh_norm,
                                  const T* __restrict__ b, const T* __restrict__ c_prev,
                                  T* __restrict__ c_out, float* c_carry) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = blockIdx.y;
  if (j >= H) return;
  const long long g0 = (long long)n * 4 * H + j;
  const long long o0 = (long long)n * H + j;
  const float i = sigmoidf_(ld(v + g0 + 0 * H) + ld(Rh_norm + g0 + 0 * H) + ld(b + j + 0 * H));
  const float g = tanhf(ld(v + g0 + 1 * H) + ld(Rh_norm + g0 + 1 * H) + ld(b + j + 1 * H));
  const float f = sigmoidf_(ld(v + g0 + 2 * H) + ld(Rh_norm + g0 + 2 * H) + ld(b + j + 2 * H));
  const float o = sigmoidf_(ld(v + g0 + 3 * H) + ld(Rh_norm + g0 + 3 * H) + ld(b + j + 3 * H));
  if (Training) {
    st(v + g0 + 0 * H, i);
    st(v + g0 + 1 * H, g);
    st(v + g0 + 2 * H, f);
  }
  st(v + g0 + 3 * H, o);
  // bf16 storage: the running cell state is carried in fp32 (c_carry) and only its
  // saved copy is rounded
  const float cp = c_carry ? c_carry[o0] : ld(c_prev + o0);
  const float cn = f * cp + i * g;
  if (c_carry) c_carry[o0] = cn;
  st(c_out + o0, cn);
}

template <typename T, bool Training, bool Zoneout>
__global__ void lnlstm_cell_output(int N, int H, const T* __restrict__ h_prev,
                                   const T* __restrict__ c_norm, const T* __restrict__ v,
                                   T* __restrict__ h_out, float zoneout_prob,
                                   const T* __restrict__ mask) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = blockIdx.y;
  if (j >= H) return;
  const long long o0 = (long long)n * H + j;
  const float o = ld(v + (long long)n * 4 * H + j + 3 * H);
  float h_new = o * tanhf(ld(c_norm + o0));
  if (Zoneout) {
    const float hp = ld(h_prev + o0);
    h_new = zoneout<Training>(h_new, hp, zoneout_prob, Training ? ld(mask + o0) : 0.f);
  }
  st(h_out + o0, h_new);
}

// Backward, first half: through h' = o * tanh(c_norm).  Writes d/dc_norm over
// c_norm and d/d(pre-activation of o) over v.o.
template <typename T, bool Zoneout>
__global__ void lnlstm_output_grad(int N, int H, T* c_norm, const T* __restrict__ dh_new,
                                   float* __restrict__ dh_carry, T* v,
                                   const T* __restrict__ mask) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = blockIdx.y;
  if (j >= H) return;
  const long long o0 = (long long)n * H + j;
  const long long oi = (long long)n * 4 * H + j + 3 * H;
  float dh_total = ld(dh_new + o0) + dh_carry[o0];
  if (Zoneout) {
    const float m = ld(mask + o0);
    dh_carry[o0] = (1.0f - m) * dh_total;
    dh_total = m * dh_total;
  } else {
    dh_carry[o0] = 0.0f;
  }
  const float c_tanh = tanhf(ld(c_norm + o0));
  const float o = ld(v + oi);
  st(c_norm + o0, d_tanh(c_tanh) * (o * dh_total));
  st(v + oi, d_sigmoid(o) * (c_tanh * dh_total));
}

// Backward, second half: through c' = f*c + i*g.  `dln` holds d/dc' from LayerNorm 3.
template <typename T>
__global__ void lnlstm_gate_grad(int N, int H, const T* __restrict__ c_prev, T* v,
                                 const T* __restrict__ dc_new, const T* __restrict__ dln,
                                 float* __restrict__ dc_carry) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = blockIdx.y;
  if (j >= H) return;
  const long long g0 = (long long)n * 4 * H + j;
  const long long o0 = (long long)n * H + j;
  const float i = ld(v + g0 + 0 * H), g = ld(v + g0 + 1 * H), f = ld(v + g0 + 2 * H);
  const float dc_total = ld(dc_new + o0) + dc_carry[o0] + ld(dln + o0);
  const float df = ld(c_prev + o0) * dc_total;
  const float di = g * dc_total;
  const float dg = i * dc_total;
  dc_carry[o0] = f * dc_total;
  st(v + g0 + 0 * H, d_sigmoid(i) * di);
  st(v + g0 + 1 * H, d_tanh(g) * dg);
  st(v + g0 + 2 * H, d_sigmoid(f) * df);
  // v.o already holds its pre-activation gradient
}

template <typename T>
int forward_steps(const LnLstmFwd& a, float* rh_f32, float* c_f32, cudaStream_t s) {
  const int N = a.N, H = a.H;
  const long long NH = (long long)N * H;
  const size_t es = sizeof(T);
  T* h = (T*)a.h;
  T* c = (T*)a.c;
  T* v = (T*)a.act_Wx_norm;
  T* act_Rh = (T*)a.act_Rh;
  T* c_norm = (T*)a.act_c_norm;
  const T* gamma1 = (const T*)a.gamma_Rh;
  const T* mask = (const T*)a.zoneout_mask;
  const bool zo = a.zoneout_prob != 0.0f && mask != nullptr;
  dim3 block(128), grid(ceil_div(H, 128), N);
  for (int t = 0; t < a.T; ++t) {
    T* Rh_t = act_Rh + t * NH * 4;
    if (rh_f32) {
      // bf16 storage: keep h.R and c' in fp32 between the kernels of one step
      GemmDesc g{a.dtype, HASTE_B200_F32, N, 4 * H, H, h + t * NH, H, 1, a.R, 4LL * H, 1, rh_f32,
                 4LL * H, 0};
      g.precise = 1;  // LayerNorm follows: keep the product at fp32 accuracy
      HB_TRY(gemm_small(g, s));
      HB_TRY(layer_norm_forward_from(HASTE_B200_F32, a.dtype, N, 4 * H, gamma1, nullptr, rh_f32,
                                     a.tmp_Rh, (char*)a.cache_Rh + (size_t)t * N * 2 * es, Rh_t, s));
    } else {
      GemmDesc g{a.dtype, a.dtype, N, 4 * H, H, h + t * NH, H, 1, a.R, 4LL * H, 1, Rh_t, 4LL * H, 0};
      g.precise = 1;  // LayerNorm follows: keep the product at fp32 accuracy
      HB_TRY(gemm_small(g, s));
      HB_TRY(layer_norm_forward(a.dtype, N, 4 * H, gamma1, nullptr, Rh_t, a.tmp_Rh,
                                (char*)a.cache_Rh + (size_t)t * N * 2 * es, s));
    }
    T* vt = v + t * NH * 4;
    if (a.training)
      lnlstm_cell_state<T, true><<<grid, block, 0, s>>>(
          N, H, vt, (const T*)a.tmp_Rh, (const T*)a.b, c + t * NH, c + (t + 1) * NH, c_f32);
    else
      lnlstm_cell_state<T, false><<<grid, block, 0, s>>>(
          N, H, vt, (const T*)a.tmp_Rh, (const T*)a.b, c + t * NH, c + (t + 1) * NH, c_f32);
    HB_LAUNCH_OK();
    if (c_f32)
      HB_TRY(layer_norm_forward_from(HASTE_B200_F32, a.dtype, N, H, a.gamma_h, a.beta_h, c_f32,
                                     c_norm + t * NH, (char*)a.cache_c + (size_t)t * N * 2 * es,
                                     nullptr, s));
    else
      HB_TRY(layer_norm_forward(a.dtype, N, H, a.gamma_h, a.beta_h, c + (t + 1) * NH,
                                c_norm + t * NH, (char*)a.cache_c + (size_t)t * N * 2 * es, s));
    const T* mt = zo ? mask + t * NH : nullptr;
#define HB_ARGS N, H, h + t * NH, c_norm + t * NH, vt, h + (t + 1) * NH, a.zoneout_prob, mt
    if (a.training) {
      if (zo) lnlstm_cell_output<T, true, true><<<grid, block, 0, s>>>(HB_ARGS);
      else    lnlstm_cell_output<T, true, false><<<grid, block, 0, s>>>(HB_ARGS);
    } else {
      if (zo) lnlstm_cell_output<T, false, true><<<grid, block, 0, s>>>(HB_ARGS);
      else    lnlstm_cell_output<T, false, false><<<grid, block, 0, s>>>(HB_ARGS);
    }
#undef HB_ARGS
    HB_LAUNCH_OK();
    count_launch(2);
  }
  return HASTE_B200_OK;
}

template <typename T>
int backward_steps(const LnLstmBwd& a, float* dh_carry, float* dc_carry, void* dgamma1,
                   void* dgamma_h, void* dbeta_h, int acc_dtype, float* lns, cudaStream_t s) {
  const int N = a.N, H = a.H;
  const long long NH = (long long)N * H;
  const size_t es = sizeof(T);
  const T* c = (const T*)a.c;
  T* v = (T*)a.act_Wx_norm;
  T* act_Rh = (T*)a.act_Rh;
  T* c_norm = (T*)a.act_c_norm;
  const T* gamma1 = (const T*)a.gamma_Rh;
  const T* mask = (const T*)a.zoneout_mask;
  const long long r_rs = a.transposed_inputs ? H : 1;
  const long long r_cs = a.transposed_inputs ? 1 : 4LL * H;
  dim3 block(128), grid(ceil_div(H, 128), N);
  for (int t = a.T - 1; t >= 0; --t) {
    T* vt = v + t * NH * 4;
    T* cn = c_norm + t * NH;
    const T* dh_new = (const T*)a.dh_new + (t + 1) * NH;
    if (mask)
      lnlstm_output_grad<T, true><<<grid, block, 0, s>>>(N, H, cn, dh_new, dh_carry, vt,
                                                         mask + t * NH);
    else
      lnlstm_output_grad<T, false><<<grid, block, 0, s>>>(N, H, cn, dh_new, dh_carry, vt, nullptr);
    HB_LAUNCH_OK();
    // LayerNorm 3 backward: input was c[t+1]; d/dLN3 -> d/dc' in place.
    HB_TRY(layer_norm_backward(a.dtype, N, H, a.gamma_h, c + (t + 1) * NH, cn, cn, acc_dtype,
                               dgamma_h, dbeta_h, (const char*)a.cache_c + (size_t)t * N * 2 * es,
                               lns, s));
    lnlstm_gate_grad<T><<<grid, block, 0, s>>>(N, H, c + t * NH, vt,
                                               (const T*)a.dc_new + (t + 1) * NH, cn, dc_carry);
    HB_LAUNCH_OK();
    count_launch(2);
    // LayerNorm 2 backward: input was act_Rh[t]; result replaces it.
    T* Rh_t = act_Rh + t * NH * 4;
    HB_TRY(layer_norm_backward(a.dtype, N, 4 * H, gamma1, Rh_t, vt, Rh_t, acc_dtype, dgamma1,
                               nullptr, (const char*)a.cache_Rh + (size_t)t * N * 2 * es, lns, s));
    GemmDesc g{a.dtype, HASTE_B200_F32, N, H, 4 * H, Rh_t, 4LL * H, 1, a.R, r_rs, r_cs, dh_carry,
               H, 1};
    g.precise = 1;  // LayerNorm follows: keep the product at fp32 accuracy
    HB_TRY(gemm_small(g, s));
  }
  return HASTE_B200_OK;
}

// Recurrence part of the forward pass: LN(x.W) is in a.act_Wx_norm.
int forward_recurrence(const LnLstmFwd& a, cudaStream_t s) {
  ProfScope prec(PH_REC_FWD, s);
  {
    const int st_ = layer_norm_lstm_forward_persistent(a, s);
    if (st_ != HASTE_B200_ERR_UNSUPPORTED) return st_;
  }
  if (a.dtype == HASTE_B200_F32) return forward_steps<float>(a, nullptr, nullptr, s);
  const size_t NH = (size_t)a.N * a.H;
  Arena ws;
  HB_TRY(make_arena(&ws, s, Arena::pad(NH * 4 * 4) + Arena::pad(NH * 4) + 512));
  float* rh_f32 = ws.take<float>(NH * 4);
  float* c_f32 = ws.take<float>(NH);
  HB_REQUIRE(rh_f32 && c_f32, "scratch arena");
  HB_TRY(to_float(a.dtype, a.c, c_f32, NH, s));
  return forward_steps<__nv_bfloat16>(a, rh_f32, c_f32, s);
}

int backward_core(const LnLstmBwd& a, cudaStream_t s);

// ---- HASTE_B200_BF16_WIDE --------------------------------------------------------------
// bf16 tensors at the interface (x, parameters, h, c, masks, incoming and outgoing gradients),
// fp32 everywhere a value is carried from one step to the next or saved for the backward
// pass.  Three LayerNorms per step amplify a relative perturbation of their inputs about
// tenfold and the recurrence feeds it back, so rounding x.W, LN(x.W) or the running h to bf16
// moves outputs and gradients by 2e-2 .. 1e-1 over a few dozen steps however exact the
// arithmetic is.  In this mode only the copies of h and c handed to the caller are rounded:
// the pass converts the bf16 operands to fp32 scratch once and runs the fp32 kernels on them.
constexpr int kWideSlot = 4;

int forward_wide(const LnLstmFwd& a, cudaStream_t s) {
  const int T = a.T, N = a.N, C = a.C, H = a.H;
  const long long TN = (long long)T * N;
  const size_t NH = (size_t)N * H, RW = (size_t)H * 4 * H;
  const bool zo = a.zoneout_prob != 0.0f && a.zoneout_mask != nullptr;
  const int BF = HASTE_B200_BF16;
  Arena ws;
  const size_t bytes = Arena::pad(RW * 4) + 3 * Arena::pad((size_t)4 * H * 4) +
                       2 * Arena::pad((size_t)H * 4) + 2 * Arena::pad((T + 1) * NH * 4) +
                       (zo ? Arena::pad(T * NH * 4) : 0) + 4096;
  HB_TRY(make_arena(&ws, s, bytes, kWideSlot));
  float* R = ws.take<float>(RW);
  float* b = ws.take<float>(4 * H);
  float* gWx = ws.take<float>(4 * H);
  float* gRh = ws.take<float>(4 * H);
  float* gh = ws.take<float>(H);
  float* bh = ws.take<float>(H);
  float* h = ws.take<float>((T + 1) * NH);
  float* c = ws.take<float>((T + 1) * NH);
  float* mask = zo ? ws.take<float>(T * NH) : nullptr;
  HB_REQUIRE(R && b && gWx && gRh && gh && bh && h && c && (!zo || mask), "scratch arena");
  HB_TRY(to_float(BF, a.R, R, RW, s));
  HB_TRY(to_float(BF, a.b, b, 4 * H, s));
  HB_TRY(to_float(BF, a.gamma_Wx, gWx, 4 * H, s));
  HB_TRY(to_float(BF, a.gamma_Rh, gRh, 4 * H, s));
  HB_TRY(to_float(BF, a.gamma_h, gh, H, s));
  HB_TRY(to_float(BF, a.beta_h, bh, H, s));
  HB_TRY(to_float(BF, a.h, h, NH, s));  // slot 0: the initial state
  HB_TRY(to_float(BF, a.c, c, NH, s));
  if (zo) HB_TRY(to_float(BF, a.zoneout_mask, mask, T * NH, s));
  // x.W: bf16 operands are exact in the tensor-core product; the fp32 accumulator is stored
  // unrounded
  GemmDesc g{BF, HASTE_B200_F32, (int)TN, 4 * H, C, a.x, C, 1, a.W, 4LL * H, 1, a.act_Wx,
             4LL * H, 0};
  {
    ProfScope p(PH_PROJ, s);
    HB_TRY(gemm(g, s));
  }
  {
    ProfScope p(PH_OTHER, s);
    HB_TRY(layer_norm_forward(HASTE_B200_F32, (int)TN, 4 * H, gWx, nullptr, a.act_Wx,
                              a.act_Wx_norm, a.cache_Wx, s));
  }
  LnLstmFwd f = a;
  f.dtype = HASTE_B200_F32;
  f.R = R; f.b = b; f.gamma_Wx = gWx; f.gamma_Rh = gRh; f.gamma_h = gh; f.beta_h = bh;
  f.h = h; f.c = c; f.zoneout_mask = mask;
  HB_TRY(forward_recurrence(f, s));
  HB_TRY(from_float(BF, h + NH, static_cast<char*>(a.h) + NH * 2, (size_t)T * NH, s));
  HB_TRY(from_float(BF, c + NH, static_cast<char*>(a.c) + NH * 2, (size_t)T * NH, s));
  return HASTE_B200_OK;
}

int backward_wide(const LnLstmBwd& a, cudaStream_t s) {
  const int T = a.T, N = a.N, C = a.C, H = a.H;
  const size_t NH = (size_t)N * H, RW = (size_t)H * 4 * H, WW = (size_t)C * 4 * H;
  const size_t XN = (size_t)T * N * C, SN = (size_t)(T + 1) * NH;
  const int BF = HASTE_B200_BF16;
  Arena ws;
  const size_t bytes = 2 * Arena::pad(RW * 4) + 2 * Arena::pad(WW * 4) +
                       5 * Arena::pad((size_t)4 * H * 4) + 4 * Arena::pad((size_t)H * 4) +
                       2 * Arena::pad(XN * 4) + 4 * Arena::pad(SN * 4) + 2 * Arena::pad(NH * 4) +
                       (a.zoneout_mask ? Arena::pad((size_t)T * NH * 4) : 0) + 8192;
  HB_TRY(make_arena(&ws, s, bytes, kWideSlot));
  float* R = ws.take<float>(RW);
  float* dR = ws.take<float>(RW);
  float* W = ws.take<float>(WW);
  float* dW = ws.take<float>(WW);
  float* gWx = ws.take<float>(4 * H);
  float* gRh = ws.take<float>(4 * H);
  float* db = ws.take<float>(4 * H);
  float* dgWx = ws.take<float>(4 * H);
  float* dgRh = ws.take<float>(4 * H);
  float* gh = ws.take<float>(H);
  float* bh = ws.take<float>(H);
  float* dgh = ws.take<float>(H);
  float* dbh = ws.take<float>(H);
  float* x = ws.take<float>(XN);
  float* dx = ws.take<float>(XN);
  float* h = ws.take<float>(SN);
  float* c = ws.take<float>(SN);
  float* dhn = ws.take<float>(SN);
  float* dcn = ws.take<float>(SN);
  float* dh = ws.take<float>(NH);
  float* dc = ws.take<float>(NH);
  float* mask = a.zoneout_mask ? ws.take<float>((size_t)T * NH) : nullptr;
  HB_REQUIRE(R && dR && W && dW && gWx && gRh && db && dgWx && dgRh && gh && bh && dgh && dbh &&
                 x && dx && h && c && dhn && dcn && dh && dc && (!a.zoneout_mask || mask),
             "scratch arena");
  HB_TRY(to_float(BF, a.R, R, RW, s));
  HB_TRY(to_float(BF, a.W, W, WW, s));
  HB_TRY(to_float(BF, a.gamma_Wx, gWx, 4 * H, s));
  HB_TRY(to_float(BF, a.gamma_Rh, gRh, 4 * H, s));
  HB_TRY(to_float(BF, a.gamma_h, gh, H, s));
  if (a.beta_h) HB_TRY(to_float(BF, a.beta_h, bh, H, s));
  HB_TRY(to_float(BF, a.x, x, XN, s));
  HB_TRY(to_float(BF, a.h, h, SN, s));
  HB_TRY(to_float(BF, a.c, c, SN, s));
  HB_TRY(to_float(BF, a.dh_new, dhn, SN, s));
  HB_TRY(to_float(BF, a.dc_new, dcn, SN, s));
  HB_TRY(to_float(BF, a.dh, dh, NH, s));
  HB_TRY(to_float(BF, a.dc, dc, NH, s));
  if (mask) HB_TRY(to_float(BF, a.zoneout_mask, mask, (size_t)T * NH, s));
  // accumulated outputs: the fp32 pass adds into zeroed scratch, the sums go into the
  // caller's bf16 tensors afterwards
  HB_CUDA_OK(cudaMemsetAsync(dR, 0, RW * 4, s));
  HB_CUDA_OK(cudaMemsetAsync(dW, 0, WW * 4, s));
  HB_CUDA_OK(cudaMemsetAsync(db, 0, (size_t)4 * H * 4, s));
  HB_CUDA_OK(cudaMemsetAsync(dgWx, 0, (size_t)4 * H * 4, s));
  HB_CUDA_OK(cudaMemsetAsync(dgRh, 0, (size_t)4 * H * 4, s));
  HB_CUDA_OK(cudaMemsetAsync(dgh, 0, (size_t)H * 4, s));
  HB_CUDA_OK(cudaMemsetAsync(dbh, 0, (size_t)H * 4, s));
  LnLstmBwd f = a;
  f.dtype = HASTE_B200_F32;
  f.W = W; f.R = R; f.gamma_Wx = gWx; f.gamma_Rh = gRh; f.gamma_h = gh;
  f.beta_h = a.beta_h ? bh : nullptr;
  f.x = x; f.h = h; f.c = c; f.dh_new = dhn; f.dc_new = dcn; f.dx = dx; f.dW = dW; f.dR = dR;
  f.db = db; f.dgamma_Wx = dgWx; f.dgamma_Rh = dgRh; f.dgamma_h = dgh; f.dbeta_h = dbh;
  f.dh = dh; f.dc = dc; f.zoneout_mask = mask;
  HB_TRY(backward_core(f, s));
  HB_TRY(from_float(BF, dx, a.dx, XN, s));
  HB_TRY(from_float(BF, dh, a.dh, NH, s));
  HB_TRY(from_float(BF, dc, a.dc, NH, s));
  HB_TRY(add_float_into(BF, dW, a.dW, WW, s));
  HB_TRY(add_float_into(BF, dR, a.dR, RW, s));
  HB_TRY(add_float_into(BF, db, a.db, 4 * H, s));
  HB_TRY(add_float_into(BF, dgWx, a.dgamma_Wx, 4 * H, s));
  HB_TRY(add_float_into(BF, dgRh, a.dgamma_Rh, 4 * H, s));
  HB_TRY(add_float_into(BF, dgh, a.dgamma_h, H, s));
  HB_TRY(add_float_into(BF, dbh, a.dbeta_h, H, s));
  return HASTE_B200_OK;
}

}  // namespace

int layer_norm_lstm_forward(const LnLstmFwd& a, cudaStream_t s) {
  HB_REQUIRE(a.dtype == HASTE_B200_F32 || a.dtype == HASTE_B200_BF16 ||
                 a.dtype == HASTE_B200_BF16_WIDE, "dtype");
  HB_REQUIRE(a.T >= 0 && a.N > 0 && a.C > 0 && a.H > 0, "T,N,C,H");
  HB_REQUIRE(a.W && a.R && a.b && a.gamma_Wx && a.gamma_Rh && a.gamma_h && a.beta_h && a.h && a.c && a.act_Wx &&
                 a.act_Wx_norm && a.cache_Wx && a.act_Rh && a.cache_Rh && a.act_c_norm &&
                 a.cache_c && a.tmp_Rh, "null pointer");
  if (a.T == 0) return HASTE_B200_OK;
  HB_REQUIRE(a.x, "x is null");
  const long long TN = (long long)a.T * a.N;
  HB_REQUIRE(TN < (1LL << 31), "T*N too large");
  if (a.dtype == HASTE_B200_BF16_WIDE) return forward_wide(a, s);
  GemmDesc g{a.dtype, a.dtype, (int)TN, 4 * a.H, a.C, a.x, a.C, 1, a.W, 4LL * a.H, 1, a.act_Wx,
             4LL * a.H, 0};
  g.precise = 1;
  {
    ProfScope p(PH_PROJ, s);
    HB_TRY(gemm(g, s));
  }
  {
    ProfScope p(PH_OTHER, s);
    HB_TRY(layer_norm_forward(a.dtype, (int)TN, 4 * a.H, a.gamma_Wx, nullptr, a.act_Wx,
                              a.act_Wx_norm, a.cache_Wx, s));
  }
  return forward_recurrence(a, s);
}

int layer_norm_lstm_backward(const LnLstmBwd& a, cudaStream_t s) {
  HB_REQUIRE(a.dtype == HASTE_B200_F32 || a.dtype == HASTE_B200_BF16 ||
                 a.dtype == HASTE_B200_BF16_WIDE, "dtype");
  HB_REQUIRE(a.T >= 0 && a.N > 0 && a.C > 0 && a.H > 0, "T,N,C,H");
  HB_REQUIRE(a.W && a.R && a.gamma_Wx && a.gamma_Rh && a.gamma_h && a.h && a.c && a.dh_new && a.dc_new && a.dW &&
                 a.dR && a.db && a.dgamma_Wx && a.dgamma_Rh && a.dgamma_h && a.dbeta_h && a.dh && a.dc &&
                 a.act_Wx && a.act_Wx_norm && a.cache_Wx && a.act_Rh && a.cache_Rh &&
                 a.act_c_norm && a.cache_c, "null pointer");
  if (a.T == 0) return HASTE_B200_OK;
  HB_REQUIRE(a.x && a.dx, "x/dx is null");
  HB_REQUIRE((long long)a.T * a.N < (1LL << 31), "T*N too large");
  if (a.dtype == HASTE_B200_BF16_WIDE) return backward_wide(a, s);
  return backward_core(a, s);
}

namespace {
int backward_core(const LnLstmBwd& a, cudaStream_t s) {
  const int N = a.N, H = a.H, C = a.C;
  const long long TN = (long long)a.T * N;
  const size_t NH = (size_t)N * H;
  const bool bf = a.dtype == HASTE_B200_BF16;
  const size_t csf = colsum_scratch_floats((int)TN, 4 * H);
  const size_t lnf = layer_norm_backward_scratch_floats((int)TN, 4 * H);
  Arena ws;
  HB_TRY(make_arena(&ws, s, 2 * Arena::pad(NH * 4) + Arena::pad(csf * 4) + Arena::pad(lnf * 4) +
                                Arena::pad(6 * H * 4) + 2048));
  float* dh_carry = ws.take<float>(NH);
  float* dc_carry = ws.take<float>(NH);
  float* cs = ws.take<float>(csf);
  float* lns = ws.take<float>(lnf);
  float* acc = ws.take<float>(6 * H);  // fp32 accumulators for bf16 runs: dgamma1, dgamma_h, dbeta_h
  HB_REQUIRE(dh_carry && dc_carry && cs && lns && acc, "scratch arena");
  HB_TRY(to_float(a.dtype, a.dh, dh_carry, NH, s));
  HB_TRY(to_float(a.dtype, a.dc, dc_carry, NH, s));

  // Persistent recurrence first; it adds its LayerNorm parameter gradients into `acc`.
  HB_CUDA_OK(cudaMemsetAsync(acc, 0, 6 * H * sizeof(float), s));
  if (profile_enabled()) profile_mark(PH_REC_BWD, true, s);
  int st_ = layer_norm_lstm_backward_persistent(a, dh_carry, dc_carry, acc, GradPlanes{}, s);
  bool use_acc = st_ == HASTE_B200_OK;
  if (st_ == HASTE_B200_ERR_UNSUPPORTED) {
    void* dgamma1 = a.dgamma_Rh;
    void* dgamma_h = a.dgamma_h;
    void* dbeta_h = a.dbeta_h;
    if (bf) {
      dgamma1 = acc;
      dgamma_h = acc + 4 * H;
      dbeta_h = acc + 5 * H;
      use_acc = true;
    }
    st_ = bf ? backward_steps<__nv_bfloat16>(a, dh_carry, dc_carry, dgamma1, dgamma_h, dbeta_h,
                                             HASTE_B200_F32, lns, s)
             : backward_steps<float>(a, dh_carry, dc_carry, dgamma1, dgamma_h, dbeta_h,
                                     HASTE_B200_F32, lns, s);
  }
  if (profile_enabled()) profile_mark(PH_REC_BWD, false, s);
  HB_TRY(st_);
  if (use_acc) {
    HB_TRY(add_float_into(a.dtype, acc, a.dgamma_Rh, 4 * H, s));
    HB_TRY(add_float_into(a.dtype, acc + 4 * H, a.dgamma_h, H, s));
    HB_TRY(add_float_into(a.dtype, acc + 5 * H, a.dbeta_h, H, s));
  }
  HB_TRY(from_float(a.dtype, dh_carry, a.dh, NH, s));
  HB_TRY(from_float(a.dtype, dc_carry, a.dc, NH, s));

  {
    ProfScope p(PH_OTHER, s);
    // act_Wx_norm now holds the gradient w.r.t. (LN1(x.W) + LN2(h.R) + b).
    HB_TRY(colsum(a.dtype, a.act_Wx_norm, 4LL * H, (int)TN, 4 * H, a.dtype, a.db, 1, cs, s));
    // LayerNorm 1 backward over all steps: act_Wx <- d/d(x.W).
    HB_TRY(layer_norm_backward(a.dtype, (int)TN, 4 * H, a.gamma_Wx, a.act_Wx, a.act_Wx_norm,
                               a.act_Wx, a.dtype, a.dgamma_Wx, nullptr, a.cache_Wx, lns, s));
  }
  const bool tr = a.transposed_inputs != 0;
  GemmDesc gw{a.dtype, a.dtype, C, 4 * H, (int)TN, a.x, tr ? TN : 1, tr ? 1 : C, a.act_Wx,
              4LL * H, 1, a.dW, 4LL * H, 1};
  {
    ProfScope p(PH_WGRAD, s);
    HB_TRY(gemm(gw, s));
  }
  GemmDesc gr{a.dtype, a.dtype, H, 4 * H, (int)TN, a.h, 1, H, a.act_Rh, 4LL * H, 1, a.dR,
              4LL * H, 1};
  {
    ProfScope p(PH_WGRAD, s);
    HB_TRY(gemm(gr, s));
  }
  GemmDesc gx{a.dtype, a.dtype, (int)TN, C, 4 * H, a.act_Wx, 4LL * H, 1, a.W, tr ? C : 1,
              tr ? 1 : 4LL * H, a.dx, C, 0};
  {
    ProfScope p(PH_DGRAD, s);
    HB_TRY(gemm(gx, s));
  }
  return HASTE_B200_OK;
}

}  // namespace

}  // namespace hb

// haste_pytorch_lib: the compiled PyTorch extension of the reference, over the haste_b200 C ABI.
//
// The reference's Python modules bind to a pybind11 module of this name
// (frameworks/pytorch/lstm.py:19 `import haste_pytorch_lib as LIB`, built by
// build/setup.pytorch.py:43-49 from frameworks/pytorch/{lstm,gru,indrnn,layer_norm_lstm,
// layer_norm_gru,layer_norm_indrnn,support}.cc).  This file provides the same twelve
// functions - names, argument order, returned lists and the released GIL - so that those
// modules run unchanged on top of libhaste_b200.so.  Like the reference's glue, every op
// allocates its outputs and scratch with torch, selects the device of `x` and runs on torch's
// current CUDA stream; the backward ops receive x, kernel and recurrent_kernel pre-transposed,
// as the reference's autograd functions pass them (frameworks/pytorch/lstm.py:84-86).
// Additions: bfloat16 tensors (and float16 for the GRU) are accepted; LayerNormLSTM with
// bfloat16 tensors keeps its saved activations in float32 (the library's BF16_WIDE mode).
#include <torch/extension.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>

#include <vector>

#include "haste_b200.h"

namespace {

using at::Tensor;
namespace py = pybind11;

int dtype_of(const Tensor& t) {
  switch (t.scalar_type()) {
    case at::kFloat: return HASTE_B200_F32;
    case at::kBFloat16: return HASTE_B200_BF16;
    case at::kHalf: return HASTE_B200_F16;
    default:
      TORCH_CHECK(false, "haste_b200 supports float32, bfloat16 and (GRU only) float16 tensors");
  }
  return -1;
}

void check(std::initializer_list<const Tensor*> ts) {
  const Tensor* first = nullptr;
  for (const Tensor* t : ts) {
    // same wording as the reference's CHECK_INPUT (frameworks/pytorch/support.h:20-22)
    TORCH_CHECK(t->is_cuda(), "tensor must be a CUDA tensor");
    TORCH_CHECK(t->is_contiguous(), "tensor must be contiguous");
    if (!t->numel()) continue;
    if (!first) first = t;
    TORCH_CHECK(t->device() == first->device() && t->scalar_type() == first->scalar_type(),
                "all tensors must share one device and dtype");
  }
}

const void* ptr(const Tensor& t) { return t.numel() ? t.data_ptr() : nullptr; }
void* mptr(Tensor& t) { return t.numel() ? t.data_ptr() : nullptr; }

void* stream() { return (void*)c10::cuda::getCurrentCUDAStream().stream(); }

void ok(int status) {
  TORCH_CHECK(status == HASTE_B200_OK, "haste_b200: ", haste_b200_last_error());
}

// (mask pointer, probability) as the library wants them: zoneout is on only with both
struct Zoneout {
  const void* mask;
  float prob;
  Zoneout(float p, const Tensor& m) {
    const bool on = p != 0.0f && m.numel() > 0;
    mask = on ? m.data_ptr() : nullptr;
    prob = on ? p : 0.0f;
  }
};

struct Dims { int T, N, C, H; };
Dims dims_fwd(const Tensor& x, int64_t H) {
  return {(int)x.size(0), (int)x.size(1), (int)x.size(2), (int)H};
}
Dims dims_bwd(const Tensor& x_t, const Tensor& h) {  // x_t [C,T,N]
  return {(int)x_t.size(1), (int)x_t.size(2), (int)x_t.size(0), (int)h.size(2)};
}

// ---------------------------------------------------------------- LSTM
std::vector<Tensor> lstm_forward(bool training, float zoneout_prob, Tensor x, Tensor h0, Tensor c0,
                                 Tensor kernel, Tensor recurrent_kernel, Tensor bias,
                                 Tensor zoneout_mask) {
  check({&x, &h0, &c0, &kernel, &recurrent_kernel, &bias, &zoneout_mask});
  const Dims d = dims_fwd(x, recurrent_kernel.size(0));
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor h = at::empty({d.T + 1, d.N, d.H}, x.options());
  Tensor c = at::empty({d.T + 1, d.N, d.H}, x.options());
  h[0].copy_(h0);
  c[0].copy_(c0);
  Tensor cache = at::empty({d.T, d.N, 4 * d.H}, x.options());
  Tensor tmp_Rh = at::empty({d.N, 4 * d.H}, x.options());
  const Zoneout z(zoneout_prob, zoneout_mask);
  ok(haste_b200_lstm_forward(dtype_of(x), training, d.T, d.N, d.C, d.H, ptr(kernel),
                             ptr(recurrent_kernel), ptr(bias), ptr(x), mptr(h), mptr(c),
                             mptr(cache), mptr(tmp_Rh), z.prob, z.mask, stream()));
  return {h, c, cache};
}

std::vector<Tensor> lstm_backward(Tensor x_t, Tensor kernel_t, Tensor recurrent_kernel_t,
                                  Tensor bias, Tensor zoneout_mask, Tensor h, Tensor c,
                                  Tensor cache, Tensor dh_new, Tensor dc_new) {
  check({&x_t, &kernel_t, &recurrent_kernel_t, &bias, &zoneout_mask, &h, &c, &cache, &dh_new,
         &dc_new});
  const Dims d = dims_bwd(x_t, h);
  const c10::cuda::CUDAGuard guard(h.device());
  Tensor dx = at::empty({d.T, d.N, d.C}, h.options());
  Tensor dW = at::zeros({d.C, 4 * d.H}, h.options());
  Tensor dR = at::zeros({d.H, 4 * d.H}, h.options());
  Tensor db = at::zeros({4 * d.H}, h.options());
  Tensor dh = at::zeros({d.N, d.H}, h.options());
  Tensor dc = at::zeros({d.N, d.H}, h.options());
  ok(haste_b200_lstm_backward(dtype_of(h), 1, d.T, d.N, d.C, d.H, ptr(kernel_t),
                              ptr(recurrent_kernel_t), ptr(bias), ptr(x_t), ptr(h), ptr(c),
                              ptr(dh_new), ptr(dc_new), mptr(dx), mptr(dW), mptr(dR), mptr(db),
                              mptr(dh), mptr(dc), mptr(cache), ptr(zoneout_mask), stream()));
  return {dx, dh, dc, dW, dR, db};
}

// ---------------------------------------------------------------- GRU
std::vector<Tensor> gru_forward(bool training, float zoneout_prob, Tensor x, Tensor h0,
                                Tensor kernel, Tensor recurrent_kernel, Tensor bias,
                                Tensor recurrent_bias, Tensor zoneout_mask) {
  check({&x, &h0, &kernel, &recurrent_kernel, &bias, &recurrent_bias, &zoneout_mask});
  const Dims d = dims_fwd(x, recurrent_kernel.size(0));
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor h = at::empty({d.T + 1, d.N, d.H}, x.options());
  h[0].copy_(h0);
  Tensor cache = training ? at::empty({d.T, d.N, 4 * d.H}, x.options()) : at::empty({0}, x.options());
  Tensor tmp_Wx = at::empty({d.T, d.N, 3 * d.H}, x.options());
  Tensor tmp_Rh = at::empty({d.N, 3 * d.H}, x.options());
  const Zoneout z(zoneout_prob, zoneout_mask);
  ok(haste_b200_gru_forward(dtype_of(x), training, d.T, d.N, d.C, d.H, ptr(kernel),
                            ptr(recurrent_kernel), ptr(bias), ptr(recurrent_bias), ptr(x),
                            mptr(h), mptr(cache), mptr(tmp_Wx), mptr(tmp_Rh), z.prob, z.mask,
                            stream()));
  return {h, cache};
}

std::vector<Tensor> gru_backward(Tensor x_t, Tensor kernel_t, Tensor recurrent_kernel_t,
                                 Tensor bias, Tensor recurrent_bias, Tensor zoneout_mask, Tensor h,
                                 Tensor cache, Tensor dh_new) {
  check({&x_t, &kernel_t, &recurrent_kernel_t, &bias, &recurrent_bias, &zoneout_mask, &h, &cache,
         &dh_new});
  const Dims d = dims_bwd(x_t, h);
  const c10::cuda::CUDAGuard guard(h.device());
  Tensor dx = at::empty({d.T, d.N, d.C}, h.options());
  Tensor dW = at::zeros({d.C, 3 * d.H}, h.options());
  Tensor dR = at::zeros({d.H, 3 * d.H}, h.options());
  Tensor dbx = at::zeros({3 * d.H}, h.options());
  Tensor dbr = at::zeros({3 * d.H}, h.options());
  Tensor dh = at::zeros({d.N, d.H}, h.options());
  Tensor dp = at::empty({d.T, d.N, 3 * d.H}, h.options());
  Tensor dq = at::empty({d.T, d.N, 3 * d.H}, h.options());
  ok(haste_b200_gru_backward(dtype_of(h), 1, d.T, d.N, d.C, d.H, ptr(kernel_t),
                             ptr(recurrent_kernel_t), ptr(bias), ptr(recurrent_bias), ptr(x_t),
                             ptr(h), ptr(cache), ptr(dh_new), mptr(dx), mptr(dW), mptr(dR),
                             mptr(dbx), mptr(dbr), mptr(dh), mptr(dp), mptr(dq),
                             ptr(zoneout_mask), stream()));
  return {dx, dh, dW, dR, dbx, dbr};
}

// ---------------------------------------------------------------- IndRNN
Tensor indrnn_forward(bool training, float zoneout_prob, Tensor x, Tensor h0, Tensor kernel,
                      Tensor recurrent_scale, Tensor bias, Tensor zoneout_mask) {
  check({&x, &h0, &kernel, &recurrent_scale, &bias, &zoneout_mask});
  const Dims d = dims_fwd(x, kernel.size(1));
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor h = at::empty({d.T + 1, d.N, d.H}, x.options());
  h[0].copy_(h0);
  Tensor workspace = at::empty({d.T, d.N, d.H}, x.options());
  const Zoneout z(zoneout_prob, zoneout_mask);
  ok(haste_b200_indrnn_forward(dtype_of(x), training, d.T, d.N, d.C, d.H, ptr(kernel),
                               ptr(recurrent_scale), ptr(bias), ptr(x), mptr(h), mptr(workspace),
                               z.prob, z.mask, stream()));
  return h;
}

std::vector<Tensor> indrnn_backward(Tensor x_t, Tensor kernel_t, Tensor recurrent_scale,
                                    Tensor bias, Tensor zoneout_mask, Tensor h, Tensor dh_new) {
  check({&x_t, &kernel_t, &recurrent_scale, &bias, &zoneout_mask, &h, &dh_new});
  const Dims d = dims_bwd(x_t, h);
  const c10::cuda::CUDAGuard guard(h.device());
  Tensor dx = at::empty({d.T, d.N, d.C}, h.options());
  Tensor dW = at::zeros({d.C, d.H}, h.options());
  Tensor du = at::zeros({d.H}, h.options());
  Tensor db = at::zeros({d.H}, h.options());
  Tensor dh = at::zeros({d.N, d.H}, h.options());
  Tensor workspace = at::empty({d.T, d.N, d.H}, h.options());
  ok(haste_b200_indrnn_backward(dtype_of(h), 1, d.T, d.N, d.C, d.H, ptr(kernel_t),
                                ptr(recurrent_scale), ptr(bias), ptr(x_t), ptr(h), ptr(dh_new),
                                mptr(dx), mptr(dW), mptr(du), mptr(db), mptr(dh), mptr(workspace),
                                ptr(zoneout_mask), stream()));
  return {dx, dh, dW, du, db};
}

// ---------------------------------------------------------------- LayerNormLSTM
// The saved activations are float32 also for bfloat16 layers (BF16_WIDE).
at::TensorOptions saved_options(const Tensor& t) {
  return t.scalar_type() == at::kBFloat16 ? t.options().dtype(at::kFloat) : t.options();
}
int ln_lstm_dtype(const Tensor& t, const Tensor& saved) {
  if (t.scalar_type() == at::kBFloat16 && saved.scalar_type() == at::kFloat)
    return HASTE_B200_BF16_WIDE;
  TORCH_CHECK(t.scalar_type() == saved.scalar_type(),
              "LayerNormLSTM saved activations must be float32 or the layer's own dtype");
  return dtype_of(t);
}

std::vector<Tensor> layer_norm_lstm_forward(bool training, float zoneout_prob, Tensor x, Tensor h0,
                                            Tensor c0, Tensor kernel, Tensor recurrent_kernel,
                                            Tensor bias, Tensor gamma, Tensor gamma_h,
                                            Tensor beta_h, Tensor zoneout_mask) {
  check({&x, &h0, &c0, &kernel, &recurrent_kernel, &bias, &gamma, &gamma_h, &beta_h,
         &zoneout_mask});
  const Dims d = dims_fwd(x, recurrent_kernel.size(0));
  const c10::cuda::CUDAGuard guard(x.device());
  const auto so = saved_options(x);
  Tensor h = at::empty({d.T + 1, d.N, d.H}, x.options());
  Tensor c = at::empty({d.T + 1, d.N, d.H}, x.options());
  h[0].copy_(h0);
  c[0].copy_(c0);
  Tensor act_Wx = at::empty({d.T, d.N, 4 * d.H}, so);
  Tensor act_Wx_norm = at::empty({d.T, d.N, 4 * d.H}, so);
  Tensor cache_Wx = at::empty({d.T, d.N, 2}, so);
  Tensor act_Rh = at::empty({d.T, d.N, 4 * d.H}, so);
  Tensor cache_Rh = at::empty({d.T, d.N, 2}, so);
  Tensor act_c_norm = at::empty({d.T, d.N, d.H}, so);
  Tensor cache_c = at::empty({d.T, d.N, 2}, so);
  Tensor tmp_Rh = at::empty({d.N, 4 * d.H}, so);
  Tensor g0 = gamma[0], g1 = gamma[1];
  const Zoneout z(zoneout_prob, zoneout_mask);
  ok(haste_b200_layer_norm_lstm_forward(
      ln_lstm_dtype(x, act_Wx), training, d.T, d.N, d.C, d.H, ptr(kernel), ptr(recurrent_kernel),
      ptr(bias), ptr(g0), ptr(g1), ptr(gamma_h), ptr(beta_h), ptr(x), mptr(h), mptr(c),
      mptr(act_Wx), mptr(act_Wx_norm), mptr(cache_Wx), mptr(act_Rh), mptr(cache_Rh),
      mptr(act_c_norm), mptr(cache_c), mptr(tmp_Rh), z.prob, z.mask, stream()));
  return {h, c, act_Wx, act_Wx_norm, cache_Wx, act_Rh, cache_Rh, act_c_norm, cache_c};
}

std::vector<Tensor> layer_norm_lstm_backward(
    Tensor x_t, Tensor kernel_t, Tensor recurrent_kernel_t, Tensor bias, Tensor gamma,
    Tensor gamma_h, Tensor beta_h, Tensor zoneout_mask, Tensor h, Tensor c, Tensor act_Wx,
    Tensor act_Wx_norm, Tensor act_Wx_norm_cache, Tensor act_Rh, Tensor act_Rh_cache,
    Tensor act_c_norm, Tensor act_c_norm_cache, Tensor dh_new, Tensor dc_new) {
  check({&x_t, &kernel_t, &recurrent_kernel_t, &bias, &gamma, &gamma_h, &beta_h, &zoneout_mask,
         &h, &c, &dh_new, &dc_new});
  check({&act_Wx, &act_Wx_norm, &act_Wx_norm_cache, &act_Rh, &act_Rh_cache, &act_c_norm,
         &act_c_norm_cache});
  const Dims d = dims_bwd(x_t, h);
  const c10::cuda::CUDAGuard guard(h.device());
  Tensor dx = at::empty({d.T, d.N, d.C}, h.options());
  Tensor dW = at::zeros({d.C, 4 * d.H}, h.options());
  Tensor dR = at::zeros({d.H, 4 * d.H}, h.options());
  Tensor db = at::zeros({4 * d.H}, h.options());
  Tensor dgamma = at::zeros_like(gamma);
  Tensor dgamma_h = at::zeros_like(gamma_h);
  Tensor dbeta_h = at::zeros_like(beta_h);
  Tensor dh = at::zeros({d.N, d.H}, h.options());
  Tensor dc = at::zeros({d.N, d.H}, h.options());
  Tensor g0 = gamma[0], g1 = gamma[1], dg0 = dgamma[0], dg1 = dgamma[1];
  ok(haste_b200_layer_norm_lstm_backward(
      ln_lstm_dtype(h, act_Wx), 1, d.T, d.N, d.C, d.H, ptr(kernel_t), ptr(recurrent_kernel_t),
      ptr(bias), ptr(g0), ptr(g1), ptr(gamma_h), ptr(beta_h), ptr(x_t), ptr(h), ptr(c),
      ptr(dh_new), ptr(dc_new), mptr(dx), mptr(dW), mptr(dR), mptr(db), mptr(dg0), mptr(dg1),
      mptr(dgamma_h), mptr(dbeta_h), mptr(dh), mptr(dc), mptr(act_Wx), mptr(act_Wx_norm),
      ptr(act_Wx_norm_cache), mptr(act_Rh), ptr(act_Rh_cache), mptr(act_c_norm),
      ptr(act_c_norm_cache), ptr(zoneout_mask), stream()));
  return {dx, dh, dc, dW, dR, db, dgamma, dgamma_h, dbeta_h};
}

// ---------------------------------------------------------------- LayerNormGRU
std::vector<Tensor> layer_norm_gru_forward(bool training, float zoneout_prob, Tensor x, Tensor h0,
                                           Tensor kernel, Tensor recurrent_kernel, Tensor bias,
                                           Tensor recurrent_bias, Tensor gamma,
                                           Tensor zoneout_mask) {
  check({&x, &h0, &kernel, &recurrent_kernel, &bias, &recurrent_bias, &gamma, &zoneout_mask});
  const Dims d = dims_fwd(x, recurrent_kernel.size(0));
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor h = at::empty({d.T + 1, d.N, d.H}, x.options());
  h[0].copy_(h0);
  Tensor cache = training ? at::empty({d.T, d.N, 4 * d.H}, x.options()) : at::empty({0}, x.options());
  Tensor act_Wx = at::empty({d.T, d.N, 3 * d.H}, x.options());
  Tensor tmp_Wx_norm = at::empty({d.T, d.N, 3 * d.H}, x.options());
  Tensor cache_Wx = at::empty({d.T, d.N, 2}, x.options());
  Tensor act_Rh = at::empty({d.T, d.N, 3 * d.H}, x.options());
  Tensor tmp_Rh_norm = at::empty({d.N, 3 * d.H}, x.options());
  Tensor cache_Rh = at::empty({d.T, d.N, 2}, x.options());
  Tensor g0 = gamma[0], g1 = gamma[1];
  const Zoneout z(zoneout_prob, zoneout_mask);
  ok(haste_b200_layer_norm_gru_forward(
      dtype_of(x), training, d.T, d.N, d.C, d.H, ptr(kernel), ptr(recurrent_kernel), ptr(bias),
      ptr(recurrent_bias), ptr(g0), ptr(g1), ptr(x), mptr(h), mptr(cache), mptr(act_Wx),
      mptr(cache_Wx), mptr(tmp_Wx_norm), mptr(act_Rh), mptr(cache_Rh), mptr(tmp_Rh_norm), z.prob,
      z.mask, stream()));
  return {h, cache, act_Wx, cache_Wx, act_Rh, cache_Rh};
}

std::vector<Tensor> layer_norm_gru_backward(Tensor x_t, Tensor kernel_t, Tensor recurrent_kernel_t,
                                            Tensor bias, Tensor recurrent_bias, Tensor gamma,
                                            Tensor zoneout_mask, Tensor h, Tensor cache,
                                            Tensor act_Wx, Tensor act_Wx_norm_cache, Tensor act_Rh,
                                            Tensor act_Rh_norm_cache, Tensor dh_new) {
  check({&x_t, &kernel_t, &recurrent_kernel_t, &bias, &recurrent_bias, &gamma, &zoneout_mask, &h,
         &cache, &act_Wx, &act_Wx_norm_cache, &act_Rh, &act_Rh_norm_cache, &dh_new});
  const Dims d = dims_bwd(x_t, h);
  const c10::cuda::CUDAGuard guard(h.device());
  Tensor dx = at::empty({d.T, d.N, d.C}, h.options());
  Tensor dW = at::zeros({d.C, 3 * d.H}, h.options());
  Tensor dR = at::zeros({d.H, 3 * d.H}, h.options());
  Tensor dbx = at::zeros({3 * d.H}, h.options());
  Tensor dbr = at::zeros({3 * d.H}, h.options());
  Tensor dh = at::zeros({d.N, d.H}, h.options());
  Tensor dp = at::empty({d.T, d.N, 3 * d.H}, h.options());
  Tensor dq = at::empty({d.T, d.N, 3 * d.H}, h.options());
  Tensor dgamma = at::zeros_like(gamma);
  Tensor g0 = gamma[0], g1 = gamma[1], dg0 = dgamma[0], dg1 = dgamma[1];
  ok(haste_b200_layer_norm_gru_backward(
      dtype_of(h), 1, d.T, d.N, d.C, d.H, ptr(kernel_t), ptr(recurrent_kernel_t), ptr(bias),
      ptr(recurrent_bias), ptr(g0), ptr(g1), ptr(x_t), ptr(h), ptr(cache), ptr(dh_new), mptr(dx),
      mptr(dW), mptr(dR), mptr(dbx), mptr(dbr), mptr(dg0), mptr(dg1), mptr(dh), mptr(dp), mptr(dq),
      ptr(act_Wx), ptr(act_Wx_norm_cache), mptr(act_Rh), ptr(act_Rh_norm_cache),
      ptr(zoneout_mask), stream()));
  return {dx, dh, dW, dR, dbx, dbr, dgamma};
}

// ---------------------------------------------------------------- LayerNormIndRNN
std::vector<Tensor> layer_norm_indrnn_forward(bool training, float zoneout_prob, Tensor x,
                                              Tensor h0, Tensor kernel, Tensor recurrent_scale,
                                              Tensor bias, Tensor gamma, Tensor zoneout_mask) {
  check({&x, &h0, &kernel, &recurrent_scale, &bias, &gamma, &zoneout_mask});
  const Dims d = dims_fwd(x, kernel.size(1));
  const c10::cuda::CUDAGuard guard(x.device());
  Tensor h = at::empty({d.T + 1, d.N, d.H}, x.options());
  h[0].copy_(h0);
  Tensor workspace = at::empty({d.T, d.N, d.H}, x.options());
  Tensor act_Wx = at::empty({d.T, d.N, d.H}, x.options());
  Tensor cache_Wx = at::empty({d.T, d.N, 2}, x.options());
  const Zoneout z(zoneout_prob, zoneout_mask);
  // gamma is [2,H]; only its first row is used (frameworks/pytorch/layer_norm_indrnn.cc:67-72)
  ok(haste_b200_layer_norm_indrnn_forward(dtype_of(x), training, d.T, d.N, d.C, d.H, ptr(kernel),
                                          ptr(recurrent_scale), ptr(bias), ptr(gamma), ptr(x),
                                          mptr(h), mptr(workspace), mptr(act_Wx), mptr(cache_Wx),
                                          z.prob, z.mask, stream()));
  return {h, act_Wx, cache_Wx};
}

std::vector<Tensor> layer_norm_indrnn_backward(Tensor x_t, Tensor kernel_t, Tensor recurrent_scale,
                                               Tensor bias, Tensor gamma, Tensor zoneout_mask,
                                               Tensor h, Tensor act_Wx, Tensor act_Wx_norm_cache,
                                               Tensor dh_new) {
  check({&x_t, &kernel_t, &recurrent_scale, &bias, &gamma, &zoneout_mask, &h, &act_Wx,
         &act_Wx_norm_cache, &dh_new});
  const Dims d = dims_bwd(x_t, h);
  const c10::cuda::CUDAGuard guard(h.device());
  Tensor dx = at::empty({d.T, d.N, d.C}, h.options());
  Tensor dW = at::zeros({d.C, d.H}, h.options());
  Tensor du = at::zeros({d.H}, h.options());
  Tensor db = at::zeros({d.H}, h.options());
  Tensor dh = at::zeros({d.N, d.H}, h.options());
  Tensor dgamma = at::zeros_like(gamma);
  Tensor workspace = at::empty({d.T, d.N, d.H}, h.options());
  ok(haste_b200_layer_norm_indrnn_backward(
      dtype_of(h), 1, d.T, d.N, d.C, d.H, ptr(kernel_t), ptr(recurrent_scale), ptr(bias),
      ptr(gamma), ptr(x_t), ptr(h), ptr(dh_new), mptr(dx), mptr(dW), mptr(du), mptr(db),
      mptr(dgamma), mptr(dh), mptr(workspace), ptr(act_Wx), ptr(act_Wx_norm_cache),
      ptr(zoneout_mask), stream()));
  return {dx, dh, dW, du, db, dgamma};
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  using guard = py::call_guard<py::gil_scoped_release>;
  m.def("lstm_forward", &lstm_forward, "LSTM forward", guard());
  m.def("lstm_backward", &lstm_backward, "LSTM backward", guard());
  m.def("gru_forward", &gru_forward, "GRU forward", guard());
  m.def("gru_backward", &gru_backward, "GRU backward", guard());
  m.def("indrnn_forward", &indrnn_forward, "IndRNN forward", guard());
  m.def("indrnn_backward", &indrnn_backward, "IndRNN backward", guard());
  m.def("layer_norm_lstm_forward", &layer_norm_lstm_forward, "LayerNormLSTM forward", guard());
  m.def("layer_norm_lstm_backward", &layer_norm_lstm_backward, "LayerNormLSTM backward", guard());
  m.def("layer_norm_gru_forward", &layer_norm_gru_forward, "LayerNormGRU forward", guard());
  m.def("layer_norm_gru_backward", &layer_norm_gru_backward, "LayerNormGRU backward", guard());
  m.def("layer_norm_indrnn_forward", &layer_norm_indrnn_forward, "LayerNormIndRNN forward", guard());
  m.def("layer_norm_indrnn_backward", &layer_norm_indrnn_backward, "LayerNormIndRNN backward", guard());
}

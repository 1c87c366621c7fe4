// Drop-in C++ API: the `haste::v0::<cell>::{ForwardPass,BackwardPass}<T>` classes of
// lmnt-com/haste's libhaste (lib/haste/{lstm,gru,indrnn,layer_norm,layer_norm_lstm,
// layer_norm_gru,layer_norm_indrnn}.h), as header-only wrappers over the haste_b200 C ABI
// (include/haste_b200.h).  Constructor and Run() argument lists are the reference's, so code
// written against libhaste compiles against this header and links libhaste_b200.so instead.
//
//  * T is float or __nv_bfloat16 (the reference's double / half instantiations do not exist).
//  * The cublasHandle_t parameter is accepted for signature compatibility and ignored:
//    no cuBLAS call is made.  `blas_handle_t` is an opaque pointer type so that this header
//    does not need cublas_v2.h; pass your cublasHandle_t as is.
//  * All work is issued on the stream given to the constructor, in order.
//  * The reference's methods return void and check nothing; here a failed call throws
//    std::runtime_error carrying haste_b200_last_error().
//  * The per-step Iterate() methods exist for the LSTM and GRU passes (the cells for which the
//    reference has them in working order); the LayerNorm cells and IndRNN have Run() only.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime_api.h>

#include <stdexcept>
#include <string>

#include "../haste_b200.h"

namespace haste {
namespace v0 {

using blas_handle_t = void*;

namespace detail {
template <typename T> struct dtype_of;
template <> struct dtype_of<float> { static constexpr int value = HASTE_B200_F32; };
template <> struct dtype_of<__nv_bfloat16> { static constexpr int value = HASTE_B200_BF16; };
// __half: the gru classes only (as in the reference, lib/gru_forward_gpu.cu.cc:373)
template <> struct dtype_of<__half> { static constexpr int value = HASTE_B200_F16; };
inline void check(int status) {
  if (status != HASTE_B200_OK)
    throw std::runtime_error(std::string("haste_b200: ") + haste_b200_last_error());
}
}  // namespace detail

// ---- layer_norm (lib/haste/layer_norm.h:24-91) -------------------------------------------
namespace layer_norm {

template <typename T>
class ForwardPass {
 public:
  ForwardPass(const int batch_size, const int hidden_size, const T* gamma, const T* beta, T* cache)
      : batch_size_(batch_size), hidden_size_(hidden_size), gamma_(gamma), beta_(beta),
        cache_(cache), partial_(0) {}
  void Run(const cudaStream_t& stream, const T* x, T* y) { RunPartial(stream, batch_size_, x, y); }
  // Normalises the next `minibatch` rows; the cache cursor advances as in the reference
  // (lib/layer_norm_forward_gpu.cu.cc:113-150).
  void RunPartial(const cudaStream_t& stream, const int minibatch, const T* x, T* y) {
    detail::check(haste_b200_layer_norm_forward(detail::dtype_of<T>::value, minibatch,
                                                hidden_size_, gamma_, beta_, x, y,
                                                cache_ + partial_ * 2, stream));
    partial_ += minibatch;
  }
  const T* gamma() const { return gamma_; }
  const T* beta() const { return beta_; }
  T* cache() const { return cache_; }

 private:
  const int batch_size_, hidden_size_;
  const T* gamma_;
  const T* beta_;
  T* cache_;
  int partial_;
};

template <typename T>
class BackwardPass {
 public:
  BackwardPass(const int batch_size, const int hidden_size, const T* gamma, const T* beta,
               const T* x, T* dgamma, T* dbeta, T* cache)
      : batch_size_(batch_size), hidden_size_(hidden_size), gamma_(gamma), beta_(beta), x_(x),
        dgamma_(dgamma), dbeta_(dbeta), cache_(cache), partial_(batch_size) {}
  void Run(const cudaStream_t& stream, const T* dy, T* dx) { RunPartial(stream, batch_size_, dy, dx); }
  // Processes the previous `minibatch` rows (the cursor retreats,
  // lib/layer_norm_backward_gpu.cu.cc:127-165).
  void RunPartial(const cudaStream_t& stream, const int minibatch, const T* dy, T* dx) {
    partial_ -= minibatch;
    detail::check(haste_b200_layer_norm_backward(
        detail::dtype_of<T>::value, minibatch, hidden_size_, gamma_,
        x_ + (long long)partial_ * hidden_size_, dy, dx, dgamma_, beta_ ? dbeta_ : nullptr,
        cache_ + partial_ * 2, stream));
  }
  const T* gamma() const { return gamma_; }
  const T* x() const { return x_; }
  T* dgamma() const { return dgamma_; }
  T* dbeta() const { return dbeta_; }
  T* cache() const { return cache_; }

 private:
  const int batch_size_, hidden_size_;
  const T* gamma_;
  const T* beta_;
  const T* x_;
  T* dgamma_;
  T* dbeta_;
  T* cache_;
  int partial_;
};

}  // namespace layer_norm

// ---- lstm (lib/haste/lstm.h:25-281) ---------------------------------------------------------
namespace lstm {

template <typename T>
class ForwardPass {
 public:
  ForwardPass(const bool training, const int batch_size, const int input_size,
              const int hidden_size, const blas_handle_t& = nullptr, const cudaStream_t& stream = 0)
      : training_(training), N_(batch_size), C_(input_size), H_(hidden_size), stream_(stream) {}
  void Run(const int steps, const T* W, const T* R, const T* b, const T* x, T* h, T* c, T* v,
           T* tmp_Rh, const float zoneout_prob, const T* zoneout_mask) {
    detail::check(haste_b200_lstm_forward(detail::dtype_of<T>::value, training_, steps, N_, C_, H_,
                                          W, R, b, x, h, c, v, tmp_Rh, zoneout_prob, zoneout_mask,
                                          stream_));
  }
  // One step (lib/haste/lstm.h:73-86).  x [N,C], h, c, h_out, c_out [N,H], v, tmp_Rh [N,4H].
  // The work runs on `stream` when one is given (the reference orders its private streams
  // against it), else on the stream the object was built with.
  void Iterate(const cudaStream_t& stream, const T* W, const T* R, const T* b, const T* x,
               const T* h, const T* c, T* h_out, T* c_out, T* v, T* tmp_Rh,
               const float zoneout_prob, const T* zoneout_mask) {
    detail::check(haste_b200_lstm_forward_iterate(detail::dtype_of<T>::value, training_, N_, C_, H_,
                                                  W, R, b, x, h, c, h_out, c_out, v, tmp_Rh,
                                                  zoneout_prob, zoneout_mask,
                                                  stream ? stream : stream_));
  }

 private:
  bool training_;
  int N_, C_, H_;
  cudaStream_t stream_;
};

template <typename T>
class BackwardPass {
 public:
  BackwardPass(const int batch_size, const int input_size, const int hidden_size,
               const blas_handle_t& = nullptr, const cudaStream_t& stream = 0)
      : N_(batch_size), C_(input_size), H_(hidden_size), stream_(stream) {}
  // W_t [4H,C], R_t [4H,H], x_t [C,T,N]: pre-transposed, as in the reference.
  void Run(const int steps, const T* W_t, const T* R_t, const T* b, const T* x_t, const T* h,
           const T* c, const T* dh_new, const T* dc_new, T* dx, T* dW, T* dR, T* db, T* dh, T* dc,
           T* v, const T* zoneout_mask) {
    detail::check(haste_b200_lstm_backward(detail::dtype_of<T>::value, 1, steps, N_, C_, H_, W_t,
                                           R_t, b, x_t, h, c, dh_new, dc_new, dx, dW, dR, db, dh,
                                           dc, v, zoneout_mask, stream_));
  }
  // One step (lib/haste/lstm.h:201-219).  x_t [C,N]; h, c: state before the step; c_new: cell
  // state after it; dh_new, dc_new, dh, dc [N,H]; v [N,4H] from the matching forward step.
  void Iterate(const cudaStream_t& stream, const T* W_t, const T* R_t, const T* b, const T* x_t,
               const T* h, const T* c, const T* c_new, const T* dh_new, const T* dc_new, T* dx,
               T* dW, T* dR, T* db, T* dh, T* dc, T* v, const T* zoneout_mask) {
    detail::check(haste_b200_lstm_backward_iterate(detail::dtype_of<T>::value, 1, N_, C_, H_, W_t,
                                                   R_t, b, x_t, h, c, c_new, dh_new, dc_new, dx, dW,
                                                   dR, db, dh, dc, v, zoneout_mask,
                                                   stream ? stream : stream_));
  }

 private:
  int N_, C_, H_;
  cudaStream_t stream_;
};

}  // namespace lstm

// ---- gru (lib/haste/gru.h:25-226) -----------------------------------------------------------
namespace gru {

template <typename T>
class ForwardPass {
 public:
  ForwardPass(const bool training, const int batch_size, const int input_size,
              const int hidden_size, const blas_handle_t& = nullptr, const cudaStream_t& stream = 0)
      : training_(training), N_(batch_size), C_(input_size), H_(hidden_size), stream_(stream) {}
  void Run(const int steps, const T* W, const T* R, const T* bx, const T* br, const T* x, T* h,
           T* v, T* tmp_Wx, T* tmp_Rh, const float zoneout_prob, const T* zoneout_mask) {
    detail::check(haste_b200_gru_forward(detail::dtype_of<T>::value, training_, steps, N_, C_, H_,
                                         W, R, bx, br, x, h, v, tmp_Wx, tmp_Rh, zoneout_prob,
                                         zoneout_mask, stream_));
  }
  // One step (lib/haste/gru.h:72-84).  x [N,C], h, h_out [N,H], v [N,4H], tmp_Wx, tmp_Rh [N,3H].
  void Iterate(const T* W, const T* R, const T* bx, const T* br, const T* x, const T* h, T* h_out,
               T* v, T* tmp_Wx, T* tmp_Rh, const float zoneout_prob, const T* zoneout_mask) {
    detail::check(haste_b200_gru_forward_iterate(detail::dtype_of<T>::value, training_, N_, C_, H_,
                                                 W, R, bx, br, x, h, h_out, v, tmp_Wx, tmp_Rh,
                                                 zoneout_prob, zoneout_mask, stream_));
  }

 private:
  bool training_;
  int N_, C_, H_;
  cudaStream_t stream_;
};

template <typename T>
class BackwardPass {
 public:
  BackwardPass(const int batch_size, const int input_size, const int hidden_size,
               const blas_handle_t& = nullptr, const cudaStream_t& stream = 0)
      : N_(batch_size), C_(input_size), H_(hidden_size), stream_(stream) {}
  void Run(const int steps, const T* W_t, const T* R_t, const T* bx, const T* br, const T* x_t,
           const T* h, const T* v, const T* dh_new, T* dx, T* dW, T* dR, T* dbx, T* dbr, T* dh,
           T* dp, T* dq, const T* zoneout_mask) {
    detail::check(haste_b200_gru_backward(detail::dtype_of<T>::value, 1, steps, N_, C_, H_, W_t,
                                          R_t, bx, br, x_t, h, v, dh_new, dx, dW, dR, dbx, dbr, dh,
                                          dp, dq, zoneout_mask, stream_));
  }
  // One step (lib/haste/gru.h:172-189).  x_t [C,N]; h: state before the step; dh_new, dh [N,H].
  void Iterate(const T* W_t, const T* R_t, const T* bx, const T* br, const T* x_t, const T* h,
               const T* v, const T* dh_new, T* dx, T* dW, T* dR, T* dbx, T* dbr, T* dh, T* dp,
               T* dq, const T* zoneout_mask) {
    detail::check(haste_b200_gru_backward_iterate(detail::dtype_of<T>::value, 1, N_, C_, H_, W_t,
                                                  R_t, bx, br, x_t, h, v, dh_new, dx, dW, dR, dbx,
                                                  dbr, dh, dp, dq, zoneout_mask, stream_));
  }

 private:
  int N_, C_, H_;
  cudaStream_t stream_;
};

}  // namespace gru

// ---- indrnn (lib/haste/indrnn.h:25-85) ------------------------------------------------------
namespace indrnn {

template <typename T>
class ForwardPass {
 public:
  ForwardPass(const bool training, const int batch_size, const int input_size,
              const int hidden_size, const blas_handle_t& = nullptr, const cudaStream_t& stream = 0)
      : training_(training), N_(batch_size), C_(input_size), H_(hidden_size), stream_(stream) {}
  void Run(const int steps, const T* W, const T* u, const T* b, const T* x, T* h, T* workspace,
           const float zoneout_prob, const T* zoneout_mask) {
    detail::check(haste_b200_indrnn_forward(detail::dtype_of<T>::value, training_, steps, N_, C_,
                                            H_, W, u, b, x, h, workspace, zoneout_prob,
                                            zoneout_mask, stream_));
  }

 private:
  bool training_;
  int N_, C_, H_;
  cudaStream_t stream_;
};

template <typename T>
class BackwardPass {
 public:
  BackwardPass(const int batch_size, const int input_size, const int hidden_size,
               const blas_handle_t& = nullptr, const cudaStream_t& stream = 0)
      : N_(batch_size), C_(input_size), H_(hidden_size), stream_(stream) {}
  void Run(const int steps, const T* W_t, const T* u, const T* b, const T* x_t, const T* h,
           const T* dh_new, T* dx, T* dW, T* du, T* db, T* dh, T* workspace,
           const T* zoneout_mask) {
    detail::check(haste_b200_indrnn_backward(detail::dtype_of<T>::value, 1, steps, N_, C_, H_, W_t,
                                             u, b, x_t, h, dh_new, dx, dW, du, db, dh, workspace,
                                             zoneout_mask, stream_));
  }

 private:
  int N_, C_, H_;
  cudaStream_t stream_;
};

}  // namespace indrnn

#include "haste_layer_norm_cells.hpp"

}  // namespace v0
}  // namespace haste

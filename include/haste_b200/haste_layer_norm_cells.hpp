// LayerNorm cells of the drop-in C++ API (included by haste.hpp, inside namespace haste::v0).
// Signatures follow lib/haste/layer_norm_lstm.h:25-203, lib/haste/layer_norm_gru.h:25-202 and
// lib/haste/layer_norm_indrnn.h:25-88: the LayerNorm parameters, statistics caches and
// gradient accumulators travel inside the layer_norm::ForwardPass / BackwardPass objects the
// caller constructs, exactly as with the reference.
#pragma once

namespace layer_norm_lstm {

template <typename T>
class ForwardPass {
 public:
  ForwardPass(const bool training, const int batch_size, const int input_size,
              const int hidden_size, const blas_handle_t& = nullptr, const cudaStream_t& stream = 0)
      : training_(training), N_(batch_size), C_(input_size), H_(hidden_size), stream_(stream) {}
  void Run(const int steps, const T* W, const T* R, const T* b, const T* x, T* h, T* c, T* act_Wx,
           T* tmp_Rh, layer_norm::ForwardPass<T>& layer_norm1, T* act_Wx_norm, T* act_Rh,
           layer_norm::ForwardPass<T>& layer_norm2, layer_norm::ForwardPass<T>& layer_norm3,
           T* act_c_norm, const float zoneout_prob, const T* zoneout_mask) {
    detail::check(haste_b200_layer_norm_lstm_forward(
        detail::dtype_of<T>::value, training_, steps, N_, C_, H_, W, R, b, layer_norm1.gamma(),
        layer_norm2.gamma(), layer_norm3.gamma(), layer_norm3.beta(), x, h, c, act_Wx, act_Wx_norm,
        layer_norm1.cache(), act_Rh, layer_norm2.cache(), act_c_norm, layer_norm3.cache(), tmp_Rh,
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
  void Run(const int steps, const T* W_t, const T* R_t, const T* b, const T* x_t, const T* h,
           const T* c, const T* dh_new, const T* dc_new, T* dx, T* dW, T* dR, T* db, T* dh, T* dc,
           T* act_Wx, layer_norm::BackwardPass<T>& layer_norm1, T* act_Wx_norm, T* act_Rh,
           layer_norm::BackwardPass<T>& layer_norm2, layer_norm::BackwardPass<T>& layer_norm3,
           T* act_c_norm, const T* zoneout_mask) {
    detail::check(haste_b200_layer_norm_lstm_backward(
        detail::dtype_of<T>::value, 1, steps, N_, C_, H_, W_t, R_t, b, layer_norm1.gamma(),
        layer_norm2.gamma(), layer_norm3.gamma(), nullptr, x_t, h, c, dh_new, dc_new, dx, dW, dR,
        db, layer_norm1.dgamma(), layer_norm2.dgamma(), layer_norm3.dgamma(), layer_norm3.dbeta(),
        dh, dc, act_Wx, act_Wx_norm, layer_norm1.cache(), act_Rh, layer_norm2.cache(), act_c_norm,
        layer_norm3.cache(), zoneout_mask, stream_));
  }

 private:
  int N_, C_, H_;
  cudaStream_t stream_;
};

}  // namespace layer_norm_lstm

namespace layer_norm_gru {

template <typename T>
class ForwardPass {
 public:
  ForwardPass(const bool training, const int batch_size, const int input_size,
              const int hidden_size, const blas_handle_t& = nullptr, const cudaStream_t& stream = 0)
      : training_(training), N_(batch_size), C_(input_size), H_(hidden_size), stream_(stream) {}
  void Run(const int steps, const T* W, const T* R, const T* bx, const T* br, const T* x, T* h,
           T* v, T* act_Wx, layer_norm::ForwardPass<T>& layer_norm1, T* tmp_Wx_norm, T* act_Rh,
           layer_norm::ForwardPass<T>& layer_norm2, T* tmp_Rh_norm, const float zoneout_prob,
           const T* zoneout_mask) {
    detail::check(haste_b200_layer_norm_gru_forward(
        detail::dtype_of<T>::value, training_, steps, N_, C_, H_, W, R, bx, br, layer_norm1.gamma(),
        layer_norm2.gamma(), x, h, v, act_Wx, layer_norm1.cache(), tmp_Wx_norm, act_Rh,
        layer_norm2.cache(), tmp_Rh_norm, zoneout_prob, zoneout_mask, stream_));
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
  // layer_norm1.x() is act_Wx and layer_norm2.x() is act_Rh, as the reference's glue sets them
  // up (frameworks/pytorch/layer_norm_gru.cc:169-188).  act_Rh is overwritten.
  void Run(const int steps, const T* W_t, const T* R_t, const T* bx, const T* br, const T* x_t,
           const T* h, const T* v, const T* dh_new, T* dx, T* dW, T* dR, T* dbx, T* dbr, T* dh,
           T* dp, T* dq, layer_norm::BackwardPass<T>& layer_norm1,
           layer_norm::BackwardPass<T>& layer_norm2, const T* zoneout_mask) {
    detail::check(haste_b200_layer_norm_gru_backward(
        detail::dtype_of<T>::value, 1, steps, N_, C_, H_, W_t, R_t, bx, br, layer_norm1.gamma(),
        layer_norm2.gamma(), x_t, h, v, dh_new, dx, dW, dR, dbx, dbr, layer_norm1.dgamma(),
        layer_norm2.dgamma(), dh, dp, dq, layer_norm1.x(), layer_norm1.cache(),
        const_cast<T*>(layer_norm2.x()), layer_norm2.cache(), zoneout_mask, stream_));
  }

 private:
  int N_, C_, H_;
  cudaStream_t stream_;
};

}  // namespace layer_norm_gru

namespace layer_norm_indrnn {

template <typename T>
class ForwardPass {
 public:
  ForwardPass(const bool training, const int batch_size, const int input_size,
              const int hidden_size, const blas_handle_t& = nullptr, const cudaStream_t& stream = 0)
      : training_(training), N_(batch_size), C_(input_size), H_(hidden_size), stream_(stream) {}
  void Run(const int steps, const T* W, const T* u, const T* b, const T* x, T* h, T* workspace,
           T* act_Wx, layer_norm::ForwardPass<T>& layer_norm1, const float zoneout_prob,
           const T* zoneout_mask) {
    detail::check(haste_b200_layer_norm_indrnn_forward(
        detail::dtype_of<T>::value, training_, steps, N_, C_, H_, W, u, b, layer_norm1.gamma(), x, h,
        workspace, act_Wx, layer_norm1.cache(), zoneout_prob, zoneout_mask, stream_));
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
           layer_norm::BackwardPass<T>& layer_norm1, const T* zoneout_mask) {
    detail::check(haste_b200_layer_norm_indrnn_backward(
        detail::dtype_of<T>::value, 1, steps, N_, C_, H_, W_t, u, b, layer_norm1.gamma(), x_t, h,
        dh_new, dx, dW, du, db, layer_norm1.dgamma(), dh, workspace, layer_norm1.x(),
        layer_norm1.cache(), zoneout_mask, stream_));
  }

 private:
  int N_, C_, H_;
  cudaStream_t stream_;
};

}  // namespace layer_norm_indrnn

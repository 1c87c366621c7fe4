"""ctypes access to the reference's own CUDA build (oracle/_ref/libhaste_ref.so).

TEST INFRASTRUCTURE: used by the GPU parity tests and by the benchmark's
reference-CUDA timing only.  `available()` is False where the library was not built.
Tensors are fp32 CUDA tensors; the reference's backward wants x, W, R pre-transposed,
which this wrapper does (and `lstm_fwd_bwd` reports whether that is inside the timing).
"""
import ctypes
import os

import torch

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libhaste_ref.so")
_lib = None


def available():
    return os.path.exists(_PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_PATH)
    return _lib


def _p(t):
    return ctypes.c_void_p(None if t is None or t.numel() == 0 else t.data_ptr())


def _chk(code, what):
    if code != 0:
        raise RuntimeError(f"reference {what} reported CUDA error {code}")


def lstm_forward(training, zp, x, h0, c0, W, R, b, mask):
    T, N, C = x.shape
    H = R.shape[0]
    h = x.new_zeros(T + 1, N, H); c = x.new_zeros(T + 1, N, H)
    h[0] = h0; c[0] = c0
    v = x.new_empty(T, N, 4 * H); tmp = x.new_empty(N, 4 * H)
    torch.cuda.current_stream().synchronize()
    _chk(lib().ref_lstm_forward(int(training), T, N, C, H, _p(W), _p(R), _p(b), _p(x), _p(h), _p(c),
                                _p(v), _p(tmp), ctypes.c_float(zp if mask is not None else 0.0),
                                _p(mask)), "lstm_forward")
    return h, c, v


def lstm_backward(x, W, R, b, mask, h, c, v, dh_new, dc_new):
    T, N, C = x.shape
    H = R.shape[0]
    x_t = x.permute(2, 0, 1).contiguous(); W_t = W.t().contiguous(); R_t = R.t().contiguous()
    dx = x.new_empty(T, N, C); dW = x.new_zeros(C, 4 * H); dR = x.new_zeros(H, 4 * H)
    db = x.new_zeros(4 * H); dh = x.new_zeros(N, H); dc = x.new_zeros(N, H)
    torch.cuda.current_stream().synchronize()
    _chk(lib().ref_lstm_backward(T, N, C, H, _p(W_t), _p(R_t), _p(b), _p(x_t), _p(h), _p(c),
                                 _p(dh_new), _p(dc_new), _p(dx), _p(dW), _p(dR), _p(db), _p(dh),
                                 _p(dc), _p(v), _p(mask)), "lstm_backward")
    torch.cuda.synchronize()
    return {"x": dx, "h0": dh, "c0": dc, "W": dW, "R": dR, "b": db}


def gru_forward(training, zp, x, h0, W, R, bx, br, mask):
    T, N, C = x.shape
    H = R.shape[0]
    h = x.new_zeros(T + 1, N, H); h[0] = h0
    v = x.new_empty(T, N, 4 * H); tw = x.new_empty(T, N, 3 * H); tr = x.new_empty(N, 3 * H)
    torch.cuda.current_stream().synchronize()
    _chk(lib().ref_gru_forward(int(training), T, N, C, H, _p(W), _p(R), _p(bx), _p(br), _p(x),
                               _p(h), _p(v), _p(tw), _p(tr),
                               ctypes.c_float(zp if mask is not None else 0.0), _p(mask)),
         "gru_forward")
    torch.cuda.synchronize()
    return h, v


def gru_backward(x, W, R, bx, br, mask, h, v, dh_new):
    T, N, C = x.shape
    H = R.shape[0]
    x_t = x.permute(2, 0, 1).contiguous(); W_t = W.t().contiguous(); R_t = R.t().contiguous()
    dx = x.new_empty(T, N, C); dW = x.new_zeros(C, 3 * H); dR = x.new_zeros(H, 3 * H)
    dbx = x.new_zeros(3 * H); dbr = x.new_zeros(3 * H); dh = x.new_zeros(N, H)
    dp = x.new_empty(T, N, 3 * H); dq = x.new_empty(T, N, 3 * H)
    torch.cuda.current_stream().synchronize()
    _chk(lib().ref_gru_backward(T, N, C, H, _p(W_t), _p(R_t), _p(bx), _p(br), _p(x_t), _p(h), _p(v),
                                _p(dh_new), _p(dx), _p(dW), _p(dR), _p(dbx), _p(dbr), _p(dh),
                                _p(dp), _p(dq), _p(mask)), "gru_backward")
    torch.cuda.synchronize()
    return {"x": dx, "h0": dh, "W": dW, "R": dR, "bx": dbx, "br": dbr}


def indrnn_forward(training, zp, x, h0, W, u, b, mask):
    T, N, C = x.shape
    H = W.shape[1]
    h = x.new_zeros(T + 1, N, H); h[0] = h0
    ws = x.new_empty(T, N, H)
    torch.cuda.current_stream().synchronize()
    _chk(lib().ref_indrnn_forward(int(training), T, N, C, H, _p(W), _p(u), _p(b), _p(x), _p(h),
                                  _p(ws), ctypes.c_float(zp if mask is not None else 0.0),
                                  _p(mask)), "indrnn_forward")
    torch.cuda.synchronize()
    return h


def indrnn_backward(x, W, u, b, mask, h, dh_new):
    T, N, C = x.shape
    H = W.shape[1]
    x_t = x.permute(2, 0, 1).contiguous(); W_t = W.t().contiguous()
    dx = x.new_empty(T, N, C); dW = x.new_zeros(C, H); du = x.new_zeros(H); db = x.new_zeros(H)
    dh = x.new_zeros(N, H); ws = x.new_empty(T, N, H)
    torch.cuda.current_stream().synchronize()
    _chk(lib().ref_indrnn_backward(T, N, C, H, _p(W_t), _p(u), _p(b), _p(x_t), _p(h), _p(dh_new),
                                   _p(dx), _p(dW), _p(du), _p(db), _p(dh), _p(ws), _p(mask)),
         "indrnn_backward")
    torch.cuda.synchronize()
    return {"x": dx, "h0": dh, "W": dW, "u": du, "b": db}


# ---- LayerNorm cells (gamma is the module's [2, G*H] parameter) -------------------------
def layer_norm_lstm_forward(training, zp, x, h0, c0, W, R, b, gamma, gamma_h, beta_h, mask):
    T, N, C = x.shape
    H = R.shape[0]
    h = x.new_zeros(T + 1, N, H); c = x.new_zeros(T + 1, N, H)
    h[0] = h0; c[0] = c0
    e = lambda *s: x.new_empty(*s)
    saved = dict(act_Wx=e(T, N, 4 * H), act_Wx_norm=e(T, N, 4 * H), cache_Wx=e(T, N, 2),
                 act_Rh=e(T, N, 4 * H), cache_Rh=e(T, N, 2), act_c_norm=e(T, N, H),
                 cache_c=e(T, N, 2))
    tmp = e(N, 4 * H)
    torch.cuda.current_stream().synchronize()
    _chk(lib().ref_layer_norm_lstm_forward(
        int(training), T, N, C, H, _p(W), _p(R), _p(b), _p(gamma), _p(gamma_h), _p(beta_h), _p(x),
        _p(h), _p(c), _p(saved["act_Wx"]), _p(saved["act_Wx_norm"]), _p(saved["cache_Wx"]),
        _p(saved["act_Rh"]), _p(saved["cache_Rh"]), _p(saved["act_c_norm"]), _p(saved["cache_c"]),
        _p(tmp), ctypes.c_float(zp if mask is not None else 0.0), _p(mask)), "layer_norm_lstm_forward")
    torch.cuda.synchronize()
    return h, c, saved


def layer_norm_lstm_backward(x, W, R, b, gamma, gamma_h, beta_h, mask, h, c, saved, dh_new, dc_new):
    T, N, C = x.shape
    H = R.shape[0]
    x_t = x.permute(2, 0, 1).contiguous(); W_t = W.t().contiguous(); R_t = R.t().contiguous()
    z = lambda *s: x.new_zeros(*s)
    dx = x.new_empty(T, N, C); dW = z(C, 4 * H); dR = z(H, 4 * H); db = z(4 * H)
    dgamma = torch.zeros_like(gamma); dgh = torch.zeros_like(gamma_h); dbh = torch.zeros_like(beta_h)
    dh = z(N, H); dc = z(N, H)
    torch.cuda.current_stream().synchronize()
    _chk(lib().ref_layer_norm_lstm_backward(
        T, N, C, H, _p(W_t), _p(R_t), _p(b), _p(gamma), _p(gamma_h), _p(beta_h), _p(x_t), _p(h),
        _p(c), _p(dh_new), _p(dc_new), _p(dx), _p(dW), _p(dR), _p(db), _p(dgamma), _p(dgh),
        _p(dbh), _p(dh), _p(dc), _p(saved["act_Wx"]), _p(saved["act_Wx_norm"]),
        _p(saved["cache_Wx"]), _p(saved["act_Rh"]), _p(saved["cache_Rh"]), _p(saved["act_c_norm"]),
        _p(saved["cache_c"]), _p(mask)), "layer_norm_lstm_backward")
    torch.cuda.synchronize()
    return {"x": dx, "h0": dh, "c0": dc, "W": dW, "R": dR, "b": db, "gamma": dgamma,
            "gamma_h": dgh, "beta_h": dbh}


def layer_norm_gru_forward(training, zp, x, h0, W, R, bx, br, gamma, mask):
    T, N, C = x.shape
    H = R.shape[0]
    h = x.new_zeros(T + 1, N, H); h[0] = h0
    e = lambda *s: x.new_empty(*s)
    saved = dict(v=e(T, N, 4 * H), act_Wx=e(T, N, 3 * H), cache_Wx=e(T, N, 2),
                 act_Rh=e(T, N, 3 * H), cache_Rh=e(T, N, 2))
    twn = e(T, N, 3 * H); trn = e(N, 3 * H)
    torch.cuda.current_stream().synchronize()
    _chk(lib().ref_layer_norm_gru_forward(
        int(training), T, N, C, H, _p(W), _p(R), _p(bx), _p(br), _p(gamma), _p(x), _p(h),
        _p(saved["v"]), _p(saved["act_Wx"]), _p(saved["cache_Wx"]), _p(twn), _p(saved["act_Rh"]),
        _p(saved["cache_Rh"]), _p(trn), ctypes.c_float(zp if mask is not None else 0.0), _p(mask)),
         "layer_norm_gru_forward")
    torch.cuda.synchronize()
    return h, saved


def layer_norm_gru_backward(x, W, R, bx, br, gamma, mask, h, saved, dh_new):
    T, N, C = x.shape
    H = R.shape[0]
    x_t = x.permute(2, 0, 1).contiguous(); W_t = W.t().contiguous(); R_t = R.t().contiguous()
    z = lambda *s: x.new_zeros(*s)
    dx = x.new_empty(T, N, C); dW = z(C, 3 * H); dR = z(H, 3 * H); dbx = z(3 * H); dbr = z(3 * H)
    dgamma = torch.zeros_like(gamma); dh = z(N, H)
    dp = x.new_empty(T, N, 3 * H); dq = x.new_empty(T, N, 3 * H)
    torch.cuda.current_stream().synchronize()
    _chk(lib().ref_layer_norm_gru_backward(
        T, N, C, H, _p(W_t), _p(R_t), _p(bx), _p(br), _p(gamma), _p(x_t), _p(h), _p(saved["v"]),
        _p(dh_new), _p(dx), _p(dW), _p(dR), _p(dbx), _p(dbr), _p(dgamma), _p(dh), _p(dp), _p(dq),
        _p(saved["act_Wx"]), _p(saved["cache_Wx"]), _p(saved["act_Rh"]), _p(saved["cache_Rh"]),
        _p(mask)), "layer_norm_gru_backward")
    torch.cuda.synchronize()
    return {"x": dx, "h0": dh, "W": dW, "R": dR, "bx": dbx, "br": dbr, "gamma": dgamma}


def layer_norm_indrnn_forward(training, zp, x, h0, W, u, b, gamma, mask):
    T, N, C = x.shape
    H = W.shape[1]
    h = x.new_zeros(T + 1, N, H); h[0] = h0
    ws = x.new_empty(T, N, H)
    saved = dict(act_Wx=x.new_empty(T, N, H), cache_Wx=x.new_empty(T, N, 2))
    torch.cuda.current_stream().synchronize()
    _chk(lib().ref_layer_norm_indrnn_forward(
        int(training), T, N, C, H, _p(W), _p(u), _p(b), _p(gamma), _p(x), _p(h), _p(ws),
        _p(saved["act_Wx"]), _p(saved["cache_Wx"]),
        ctypes.c_float(zp if mask is not None else 0.0), _p(mask)), "layer_norm_indrnn_forward")
    torch.cuda.synchronize()
    return h, saved


def layer_norm_indrnn_backward(x, W, u, b, gamma, mask, h, saved, dh_new):
    T, N, C = x.shape
    H = W.shape[1]
    x_t = x.permute(2, 0, 1).contiguous(); W_t = W.t().contiguous()
    dx = x.new_empty(T, N, C); dW = x.new_zeros(C, H); du = x.new_zeros(H); db = x.new_zeros(H)
    dgamma = torch.zeros_like(gamma); dh = x.new_zeros(N, H); ws = x.new_empty(T, N, H)
    torch.cuda.current_stream().synchronize()
    _chk(lib().ref_layer_norm_indrnn_backward(
        T, N, C, H, _p(W_t), _p(u), _p(b), _p(gamma), _p(x_t), _p(h), _p(dh_new), _p(dx), _p(dW),
        _p(du), _p(db), _p(dgamma), _p(dh), _p(ws), _p(saved["act_Wx"]), _p(saved["cache_Wx"]),
        _p(mask)), "layer_norm_indrnn_backward")
    torch.cuda.synchronize()
    return {"x": dx, "h0": dh, "W": dW, "u": du, "b": db, "gamma": dgamma}

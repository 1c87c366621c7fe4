"""ctypes binding of libhaste_b200.so (the C ABI declared in include/haste_b200.h).

The library is built in-tree by `haste_b200.build`.  There is no fallback: if the
shared object is missing or a call fails, an exception is raised.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# HASTE_B200_LIBRARY selects another build of the library (a debug or experiment build)
LIB_PATH = os.environ.get("HASTE_B200_LIBRARY") or os.path.join(_HERE, "libhaste_b200.so")

F32, BF16, F16, BF16_WIDE = 0, 1, 2, 3
PATH_AUTO, PATH_STEPWISE, PATH_PERSISTENT, PATH_NO_TENSOR_CORE = 0, 1, 2, 3
GEMM_AUTO, GEMM_SIMT, GEMM_TCGEN05, GEMM_TCGEN05_SINGLE = 0, 1, 2, 3

_i, _f, _p, _ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

# name -> argument types, in the order of include/haste_b200.h
SIGNATURES = {
    "haste_b200_lstm_forward": [_i] * 6 + [_p] * 8 + [_f, _p, _p],
    "haste_b200_lstm_backward": [_i] * 6 + [_p] * 17,
    "haste_b200_probe_exchange_latency": [_i] * 3 + [_p, _p],
    "haste_b200_lstm_forward_iterate": [_i] * 5 + [_p] * 10 + [_f, _p, _p],
    "haste_b200_lstm_backward_iterate": [_i] * 5 + [_p] * 18,
    "haste_b200_gru_forward_iterate": [_i] * 5 + [_p] * 10 + [_f, _p, _p],
    "haste_b200_gru_backward_iterate": [_i] * 5 + [_p] * 18,
    "haste_b200_gru_forward": [_i] * 6 + [_p] * 9 + [_f, _p, _p],
    "haste_b200_gru_backward": [_i] * 6 + [_p] * 18,
    "haste_b200_indrnn_forward": [_i] * 6 + [_p] * 6 + [_f, _p, _p],
    "haste_b200_indrnn_backward": [_i] * 6 + [_p] * 14,
    "haste_b200_layer_norm_forward": [_i] * 3 + [_p] * 6,
    "haste_b200_layer_norm_backward": [_i] * 3 + [_p] * 8,
    "haste_b200_layer_norm_backward_noalloc": [_i] * 3 + [_p] * 8,
    "haste_b200_layer_norm_lstm_forward": [_i] * 6 + [_p] * 18 + [_f, _p, _p],
    "haste_b200_layer_norm_lstm_backward": [_i] * 6 + [_p] * 31,
    "haste_b200_layer_norm_gru_forward": [_i] * 6 + [_p] * 15 + [_f, _p, _p],
    "haste_b200_layer_norm_gru_backward": [_i] * 6 + [_p] * 26,
    "haste_b200_layer_norm_indrnn_forward": [_i] * 6 + [_p] * 9 + [_f, _p, _p],
    "haste_b200_layer_norm_indrnn_backward": [_i] * 6 + [_p] * 18,
    "haste_b200_gemm": [_i] * 4 + [_p, _ll, _ll, _p, _ll, _ll, _p, _ll, _i, _p],
    "haste_b200_set_recurrence_path": [_i],
    "haste_b200_set_gemm_path": [_i],
    "haste_b200_set_sm_budget": [_i],
    "haste_b200_sync_check": [_p],
    "haste_b200_profile_enable": [_i],
    "haste_b200_profile_read": [_p, _i],
}
OTHER_SYMBOLS = ["haste_b200_last_error", "haste_b200_version", "haste_b200_launch_count"]

_lib = None


class HasteError(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} not found: build it with `python -m haste_b200.build` "
                "(there is no CPU or PyTorch fallback)")
        L = ctypes.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = _i
        L.haste_b200_last_error.restype = ctypes.c_char_p
        L.haste_b200_version.restype = ctypes.c_char_p
        L.haste_b200_launch_count.restype = _ll
        _lib = L
    return _lib


def call(name, *args):
    L = lib()
    status = getattr(L, name)(*args)
    if status != 0:
        msg = L.haste_b200_last_error().decode()
        raise HasteError(f"{name} failed with status {status}: {msg}")


def launch_count():
    return int(lib().haste_b200_launch_count())


def set_recurrence_path(path):
    call("haste_b200_set_recurrence_path", path)


def set_sm_budget(sms):
    """SMs one persistent recurrence launch may occupy (0 = all); see the header."""
    call("haste_b200_set_sm_budget", int(sms))


def set_gemm_path(path):
    call("haste_b200_set_gemm_path", path)


def sync_check(stream=None):
    """Synchronises `stream` (a raw cudaStream_t or None) and raises if a kernel timed out."""
    call("haste_b200_sync_check", stream)


PHASES = ["input_projection", "recurrence_fwd", "recurrence_bwd", "weight_grad", "input_grad",
          "other"]


def profile_enable(on=True):
    call("haste_b200_profile_enable", int(on))


def probe_exchange_latency(N, H, steps=2000, stream=None):
    """Device microseconds per step of the forward recurrence's hand-off alone (see the header)."""
    out = ctypes.c_float(0.0)
    call("haste_b200_probe_exchange_latency", int(N), int(H), int(steps),
         ctypes.cast(ctypes.byref(out), ctypes.c_void_p), stream)
    return float(out.value)


def profile_read():
    """ms per phase since the last read, as a dict keyed by PHASES."""
    buf = (ctypes.c_float * len(PHASES))()
    call("haste_b200_profile_read", ctypes.cast(buf, ctypes.c_void_p), len(PHASES))
    return dict(zip(PHASES, [float(v) for v in buf]))

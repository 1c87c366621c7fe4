"""The twelve tensor-level ops of the reference's `haste_pytorch_lib` extension,
re-implemented over the haste_b200 C ABI.

Names, argument order and returned lists mirror the reference's pybind functions
(frameworks/pytorch/{lstm,gru,indrnn,layer_norm_lstm,layer_norm_gru,layer_norm_indrnn}.cc);
like them, each op allocates its outputs and scratch with torch and runs on torch's
current CUDA stream.  Additions: bfloat16 tensors are accepted, and every
`*_backward` takes `transposed=` - True (the reference's convention) means `x`,
`kernel` and `recurrent_kernel` arrive pre-transposed as `[C,T,N]`, `[G*H,C]`,
`[G*H,H]`; False means they arrive in forward layout and are used without a copy.
"""
import torch

from . import _C


def _dtype(t):
    if t.dtype == torch.float32:
        return _C.F32
    if t.dtype == torch.bfloat16:
        return _C.BF16
    if t.dtype == torch.float16:
        return _C.F16  # accepted by the GRU ops and gemm only; other entry points reject it
    raise TypeError(f"haste_b200 supports float32, bfloat16 and (GRU only) float16 tensors, "
                    f"got {t.dtype}")


def _ln_lstm_dtype(t, saved):
    """Library dtype of a LayerNormLSTM call: bfloat16 tensors with float32 saved activations
    are the BF16_WIDE mode."""
    d = _dtype(t)
    if saved.dtype == t.dtype:
        return d
    if d == _C.BF16 and saved.dtype == torch.float32:
        return _C.BF16_WIDE
    raise RuntimeError("haste_b200: LayerNormLSTM saved activations must be float32 or the "
                       "layer's own dtype")


def _check(*tensors):
    dev, dt = tensors[0].device, tensors[0].dtype
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("haste_b200: tensor must be a CUDA tensor")
        if not t.is_contiguous():
            raise RuntimeError("haste_b200: tensor must be contiguous")
        if t.numel() and (t.device != dev or t.dtype != dt):
            raise RuntimeError("haste_b200: all tensors must share one device and dtype")


def _p(t):
    return None if t is None or t.numel() == 0 else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _mask_ptr(zoneout_prob, mask):
    has = bool(zoneout_prob) and mask is not None and mask.numel() > 0
    return (mask.data_ptr() if has else None), (float(zoneout_prob) if has else 0.0)


def _zeros(grads, like, *shape):
    """A zeroed parameter-gradient output: a view of the caller's `GradientBucket` when one is
    given (`haste_b200.data_parallel`), else a fresh tensor."""
    if grads is None:
        return like.new_zeros(*shape)
    if grads.dtype != like.dtype or grads.flat.device != like.device:
        raise ValueError("gradient bucket has the wrong dtype or device")
    return grads.take(*shape)


def _dims_fwd(x, recurrent):
    T, N, C = x.shape
    return T, N, C, recurrent.shape[0]


def _dims_bwd(x, transposed, H):
    if transposed:
        C, T, N = x.shape
    else:
        T, N, C = x.shape
    return T, N, C, H


# ---------------------------------------------------------------- LSTM
def lstm_forward(training, zoneout_prob, x, h0, c0, kernel, recurrent_kernel, bias, zoneout_mask):
    _check(x, h0, c0, kernel, recurrent_kernel, bias, zoneout_mask)
    T, N, C, H = _dims_fwd(x, recurrent_kernel)
    with torch.cuda.device(x.device):
        h = x.new_empty(T + 1, N, H)
        c = x.new_empty(T + 1, N, H)
        h[0] = h0
        c[0] = c0
        cache = x.new_empty(T, N, 4 * H)
        tmp_Rh = x.new_empty(N, 4 * H)
        mp, zp = _mask_ptr(zoneout_prob, zoneout_mask)
        _C.call("haste_b200_lstm_forward", _dtype(x), int(training), T, N, C, H, _p(kernel),
                _p(recurrent_kernel), _p(bias), _p(x), _p(h), _p(c), _p(cache), _p(tmp_Rh),
                zp, mp, _stream())
    return [h, c, cache]


def lstm_backward(x, kernel, recurrent_kernel, bias, zoneout_mask, h, c, cache, dh_new, dc_new,
                  transposed=True, grads=None):
    _check(x, kernel, recurrent_kernel, bias, zoneout_mask, h, c, cache, dh_new, dc_new)
    H = h.shape[2]
    T, N, C, H = _dims_bwd(x, transposed, H)
    with torch.cuda.device(h.device):
        dx = h.new_empty(T, N, C)
        dW = _zeros(grads, h, C, 4 * H)
        dR = _zeros(grads, h, H, 4 * H)
        db = _zeros(grads, h, 4 * H)
        dh = h.new_zeros(N, H)
        dc = h.new_zeros(N, H)
        _C.call("haste_b200_lstm_backward", _dtype(h), int(transposed), T, N, C, H, _p(kernel),
                _p(recurrent_kernel), _p(bias), _p(x), _p(h), _p(c), _p(dh_new), _p(dc_new),
                _p(dx), _p(dW), _p(dR), _p(db), _p(dh), _p(dc), _p(cache), _p(zoneout_mask),
                _stream())
    return [dx, dh, dc, dW, dR, db]


_copy_streams = {}


def lstm_forward_from_host(training, zoneout_prob, x_host, h0, c0, kernel, recurrent_kernel, bias,
                           zoneout_mask, chunks=8):
    """`lstm_forward` for an input that still lives in pinned HOST memory.

    The sequence is cut into `chunks` pieces along time; while the GPU runs the projection and
    the recurrence of one piece, the next piece is copied host->device on a second stream, so
    only the first copy is exposed.  Every piece is a C-ABI call on slices of the same
    `[T+1,N,H]` / `[T,N,4H]` buffers (the state slot a piece ends on is the initial state of
    the next), so the result equals one call on the whole sequence up to the rounding of the
    input projection (a short piece may take the CUDA-core contraction path).
    The default of 8 pieces measured best at T=1000, N=64, C=H=512 in fp32, where the copy of
    the whole input takes about as long as the forward pass (fwd+bwd step with host input:
    1 piece 9.98 ms, 2: 8.83, 4: 8.34, 8: 8.21, 16: 8.43, 24: 8.88; each piece costs ~50 us of
    launches and start-up).
    Returns [h, c, cache, x_device].
    """
    _check(h0, c0, kernel, recurrent_kernel, bias, zoneout_mask)
    if x_host.is_cuda or not x_host.is_pinned():
        raise RuntimeError("haste_b200: x_host must be a pinned CPU tensor")
    T, N, C = x_host.shape
    H = recurrent_kernel.shape[0]
    dev = h0.device
    with torch.cuda.device(dev):
        main = torch.cuda.current_stream()
        side = _copy_streams.get(dev.index)
        if side is None:
            side = _copy_streams[dev.index] = torch.cuda.Stream(device=dev)
        x = torch.empty(T, N, C, device=dev, dtype=h0.dtype)
        h = h0.new_empty(T + 1, N, H)
        c = h0.new_empty(T + 1, N, H)
        h[0] = h0
        c[0] = c0
        cache = h0.new_empty(T, N, 4 * H)
        tmp_Rh = h0.new_empty(N, 4 * H)
        mp, zp = _mask_ptr(zoneout_prob, zoneout_mask)
        es = x.element_size()
        bounds = [round(i * T / chunks) for i in range(chunks + 1)]
        side.wait_stream(main)
        x.record_stream(side)
        events = []
        with torch.cuda.stream(side):
            for k in range(chunks):
                t0, t1 = bounds[k], bounds[k + 1]
                if t1 > t0:
                    x[t0:t1].copy_(x_host[t0:t1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(side)
                events.append(ev)
        for k in range(chunks):
            t0, t1 = bounds[k], bounds[k + 1]
            if t1 == t0:
                continue
            main.wait_event(events[k])
            _C.call("haste_b200_lstm_forward", _dtype(h0), int(training), t1 - t0, N, C, H,
                    _p(kernel), _p(recurrent_kernel), _p(bias), x.data_ptr() + t0 * N * C * es,
                    h.data_ptr() + t0 * N * H * es, c.data_ptr() + t0 * N * H * es,
                    cache.data_ptr() + t0 * N * 4 * H * es, _p(tmp_Rh), zp,
                    (mp + t0 * N * H * es) if mp else None, main.cuda_stream)
    return [h, c, cache, x]


_host_stage = {}  # (device, shape, dtype) -> [device buffer, event of its last reader]


def lstm_backward_from_host(x, kernel, recurrent_kernel, bias, zoneout_mask, h, c, cache,
                            dh_new_host, dc_new, chunks=4, grads=None):
    """`lstm_backward(..., transposed=False)` for an incoming gradient `dh_new_host`
    `[T+1,N,H]` that still lives in pinned HOST memory.

    The backward pass consumes the gradient from the last time step down, so it is copied in
    `chunks` pieces in that order on the copy stream while the GPU is still busy with the
    forward pass, and the pass itself runs as one C-ABI call per piece, latest piece first: the
    carried `dh`, `dc` go from call to call through the `[N,H]` in/out buffers, `dW`, `dR`, `db`
    accumulate, and each call assigns its own slice of `dx`.  The result equals one call on the
    whole sequence up to the summation order of the weight gradients.  The device copy of the
    gradient is kept between calls (one buffer per device and shape), guarded by an event of
    its last reader.
    Returns [dx, dh, dc, dW, dR, db].
    """
    _check(x, kernel, recurrent_kernel, bias, zoneout_mask, h, c, cache, dc_new)
    if dh_new_host.is_cuda or not dh_new_host.is_pinned():
        raise RuntimeError("haste_b200: dh_new_host must be a pinned CPU tensor")
    T, N, C = x.shape
    H = h.shape[2]
    dev = h.device
    with torch.cuda.device(dev):
        main = torch.cuda.current_stream()
        side = _copy_streams.get(dev.index)
        if side is None:
            side = _copy_streams[dev.index] = torch.cuda.Stream(device=dev)
        key = (dev.index, tuple(dh_new_host.shape), h.dtype)
        slot = _host_stage.get(key)
        if slot is None:
            slot = _host_stage[key] = [torch.empty(T + 1, N, H, device=dev, dtype=h.dtype), None]
        dh_new = slot[0]
        if slot[1] is not None:
            side.wait_event(slot[1])  # the previous call's kernels have read the buffer
        bounds = [round(i * T / chunks) for i in range(chunks + 1)]
        events = [None] * chunks
        with torch.cuda.stream(side):
            for k in reversed(range(chunks)):
                t0, t1 = bounds[k], bounds[k + 1]
                if t1 > t0:  # steps t0..t1-1 read the gradient slots t0+1..t1
                    dh_new[t0 + 1:t1 + 1].copy_(dh_new_host[t0 + 1:t1 + 1], non_blocking=True)
                events[k] = torch.cuda.Event()
                events[k].record(side)
        dx = h.new_empty(T, N, C)
        dW = _zeros(grads, h, C, 4 * H)
        dR = _zeros(grads, h, H, 4 * H)
        db = _zeros(grads, h, 4 * H)
        dh = h.new_zeros(N, H)
        dc = h.new_zeros(N, H)
        es = h.element_size()
        mp = _p(zoneout_mask)
        for k in reversed(range(chunks)):
            t0, t1 = bounds[k], bounds[k + 1]
            if t1 == t0:
                continue
            main.wait_event(events[k])
            o = t0 * N * es
            _C.call("haste_b200_lstm_backward", _dtype(h), 0, t1 - t0, N, C, H, _p(kernel),
                    _p(recurrent_kernel), _p(bias), x.data_ptr() + o * C, h.data_ptr() + o * H,
                    c.data_ptr() + o * H, dh_new.data_ptr() + o * H, dc_new.data_ptr() + o * H,
                    dx.data_ptr() + o * C, _p(dW), _p(dR), _p(db), _p(dh), _p(dc),
                    cache.data_ptr() + o * 4 * H, (mp + o * H) if mp else None,
                    main.cuda_stream)
        slot[1] = torch.cuda.Event()
        slot[1].record(main)
    return [dx, dh, dc, dW, dR, db]


# ---------------------------------------------------------------- GRU
def gru_forward(training, zoneout_prob, x, h0, kernel, recurrent_kernel, bias, recurrent_bias,
                zoneout_mask):
    _check(x, h0, kernel, recurrent_kernel, bias, recurrent_bias, zoneout_mask)
    T, N, C, H = _dims_fwd(x, recurrent_kernel)
    with torch.cuda.device(x.device):
        h = x.new_empty(T + 1, N, H)
        h[0] = h0
        cache = x.new_empty(T, N, 4 * H) if training else x.new_empty(0)
        tmp_Wx = x.new_empty(T, N, 3 * H)
        tmp_Rh = x.new_empty(N, 3 * H)
        mp, zp = _mask_ptr(zoneout_prob, zoneout_mask)
        _C.call("haste_b200_gru_forward", _dtype(x), int(training), T, N, C, H, _p(kernel),
                _p(recurrent_kernel), _p(bias), _p(recurrent_bias), _p(x), _p(h), _p(cache),
                _p(tmp_Wx), _p(tmp_Rh), zp, mp, _stream())
    return [h, cache]


def gru_backward(x, kernel, recurrent_kernel, bias, recurrent_bias, zoneout_mask, h, cache,
                 dh_new, transposed=True, grads=None):
    _check(x, kernel, recurrent_kernel, bias, recurrent_bias, zoneout_mask, h, cache, dh_new)
    H = h.shape[2]
    T, N, C, H = _dims_bwd(x, transposed, H)
    with torch.cuda.device(h.device):
        dx = h.new_empty(T, N, C)
        dW = _zeros(grads, h, C, 3 * H)
        dR = _zeros(grads, h, H, 3 * H)
        dbx = _zeros(grads, h, 3 * H)
        dbr = _zeros(grads, h, 3 * H)
        dh = h.new_zeros(N, H)
        dp = h.new_empty(T, N, 3 * H)
        dq = h.new_empty(T, N, 3 * H)
        _C.call("haste_b200_gru_backward", _dtype(h), int(transposed), T, N, C, H, _p(kernel),
                _p(recurrent_kernel), _p(bias), _p(recurrent_bias), _p(x), _p(h), _p(cache),
                _p(dh_new), _p(dx), _p(dW), _p(dR), _p(dbx), _p(dbr), _p(dh), _p(dp), _p(dq),
                _p(zoneout_mask), _stream())
    return [dx, dh, dW, dR, dbx, dbr]


# ---------------------------------------------------------------- IndRNN
def indrnn_forward(training, zoneout_prob, x, h0, kernel, recurrent_scale, bias, zoneout_mask):
    _check(x, h0, kernel, recurrent_scale, bias, zoneout_mask)
    T, N, C = x.shape
    H = kernel.shape[1]
    with torch.cuda.device(x.device):
        h = x.new_empty(T + 1, N, H)
        h[0] = h0
        workspace = x.new_empty(T, N, H)
        mp, zp = _mask_ptr(zoneout_prob, zoneout_mask)
        _C.call("haste_b200_indrnn_forward", _dtype(x), int(training), T, N, C, H, _p(kernel),
                _p(recurrent_scale), _p(bias), _p(x), _p(h), _p(workspace), zp, mp, _stream())
    return h


def indrnn_backward(x, kernel, recurrent_scale, bias, zoneout_mask, h, dh_new, transposed=True, grads=None):
    _check(x, kernel, recurrent_scale, bias, zoneout_mask, h, dh_new)
    H = h.shape[2]
    T, N, C, H = _dims_bwd(x, transposed, H)
    with torch.cuda.device(h.device):
        dx = h.new_empty(T, N, C)
        dW = _zeros(grads, h, C, H)
        du = _zeros(grads, h, H)
        db = _zeros(grads, h, H)
        dh = h.new_zeros(N, H)
        workspace = h.new_empty(T, N, H)
        _C.call("haste_b200_indrnn_backward", _dtype(h), int(transposed), T, N, C, H, _p(kernel),
                _p(recurrent_scale), _p(bias), _p(x), _p(h), _p(dh_new), _p(dx), _p(dW), _p(du),
                _p(db), _p(dh), _p(workspace), _p(zoneout_mask), _stream())
    return [dx, dh, dW, du, db]


# ---------------------------------------------------------------- LayerNormLSTM
def layer_norm_lstm_forward(training, zoneout_prob, x, h0, c0, kernel, recurrent_kernel, bias,
                            gamma, gamma_h, beta_h, zoneout_mask, saved_dtype=torch.float32):
    _check(x, h0, c0, kernel, recurrent_kernel, bias, gamma, gamma_h, beta_h, zoneout_mask)
    T, N, C, H = _dims_fwd(x, recurrent_kernel)
    with torch.cuda.device(x.device):
        h = x.new_empty(T + 1, N, H)
        c = x.new_empty(T + 1, N, H)
        h[0] = h0
        c[0] = c0
        # what the forward pass leaves for the backward pass is float32 whatever the layer's
        # dtype: with bfloat16 tensors the op runs in the library's BF16_WIDE mode (see the
        # header), because rounding these to bfloat16 alone costs 2e-2 .. 1e-1 of accuracy.
        # saved_dtype=torch.bfloat16 selects the library's all-bfloat16 mode instead (the
        # one a C++ caller with __nv_bfloat16 buffers gets).
        sd = saved_dtype if x.dtype == torch.bfloat16 else x.dtype
        act_Wx = x.new_empty(T, N, 4 * H, dtype=sd)
        act_Wx_norm = x.new_empty(T, N, 4 * H, dtype=sd)
        cache_Wx = x.new_empty(T, N, 2, dtype=sd)
        act_Rh = x.new_empty(T, N, 4 * H, dtype=sd)
        cache_Rh = x.new_empty(T, N, 2, dtype=sd)
        act_c_norm = x.new_empty(T, N, H, dtype=sd)
        cache_c = x.new_empty(T, N, 2, dtype=sd)
        tmp_Rh = x.new_empty(N, 4 * H, dtype=sd)
        mp, zp = _mask_ptr(zoneout_prob, zoneout_mask)
        _C.call("haste_b200_layer_norm_lstm_forward", _ln_lstm_dtype(x, act_Wx), int(training), T, N, C, H,
                _p(kernel), _p(recurrent_kernel), _p(bias), _p(gamma[0]), _p(gamma[1]), _p(gamma_h),
                _p(beta_h),
                _p(x), _p(h), _p(c), _p(act_Wx), _p(act_Wx_norm), _p(cache_Wx), _p(act_Rh),
                _p(cache_Rh), _p(act_c_norm), _p(cache_c), _p(tmp_Rh), zp, mp, _stream())
    return [h, c, act_Wx, act_Wx_norm, cache_Wx, act_Rh, cache_Rh, act_c_norm, cache_c]


def layer_norm_lstm_backward(x, kernel, recurrent_kernel, bias, gamma, gamma_h, beta_h,
                             zoneout_mask, h, c, act_Wx, act_Wx_norm, cache_Wx, act_Rh, cache_Rh,
                             act_c_norm, cache_c, dh_new, dc_new, transposed=True, grads=None):
    _check(x, kernel, recurrent_kernel, bias, gamma, gamma_h, beta_h, zoneout_mask, h, c, dh_new,
           dc_new)
    _check(act_Wx, act_Wx_norm, cache_Wx, act_Rh, cache_Rh, act_c_norm, cache_c)
    H = h.shape[2]
    T, N, C, H = _dims_bwd(x, transposed, H)
    with torch.cuda.device(h.device):
        dx = h.new_empty(T, N, C)
        dW = _zeros(grads, h, C, 4 * H)
        dR = _zeros(grads, h, H, 4 * H)
        db = _zeros(grads, h, 4 * H)
        dgamma = _zeros(grads, h, *gamma.shape)
        dgamma_h = _zeros(grads, h, *gamma_h.shape)
        dbeta_h = _zeros(grads, h, *beta_h.shape)
        dh = h.new_zeros(N, H)
        dc = h.new_zeros(N, H)
        _C.call("haste_b200_layer_norm_lstm_backward", _ln_lstm_dtype(h, act_Wx), int(transposed), T, N, C, H,
                _p(kernel), _p(recurrent_kernel), _p(bias), _p(gamma[0]), _p(gamma[1]), _p(gamma_h),
                _p(beta_h),
                _p(x), _p(h), _p(c), _p(dh_new), _p(dc_new), _p(dx), _p(dW), _p(dR), _p(db),
                _p(dgamma[0]), _p(dgamma[1]), _p(dgamma_h), _p(dbeta_h), _p(dh), _p(dc), _p(act_Wx),
                _p(act_Wx_norm), _p(cache_Wx), _p(act_Rh), _p(cache_Rh), _p(act_c_norm),
                _p(cache_c), _p(zoneout_mask), _stream())
    return [dx, dh, dc, dW, dR, db, dgamma, dgamma_h, dbeta_h]


# ---------------------------------------------------------------- LayerNormGRU
def layer_norm_gru_forward(training, zoneout_prob, x, h0, kernel, recurrent_kernel, bias,
                           recurrent_bias, gamma, zoneout_mask):
    _check(x, h0, kernel, recurrent_kernel, bias, recurrent_bias, gamma, zoneout_mask)
    T, N, C, H = _dims_fwd(x, recurrent_kernel)
    with torch.cuda.device(x.device):
        h = x.new_empty(T + 1, N, H)
        h[0] = h0
        cache = x.new_empty(T, N, 4 * H) if training else x.new_empty(0)
        act_Wx = x.new_empty(T, N, 3 * H)
        tmp_Wx_norm = x.new_empty(T, N, 3 * H)
        cache_Wx = x.new_empty(T, N, 2)
        act_Rh = x.new_empty(T, N, 3 * H)
        tmp_Rh_norm = x.new_empty(N, 3 * H)
        cache_Rh = x.new_empty(T, N, 2)
        mp, zp = _mask_ptr(zoneout_prob, zoneout_mask)
        _C.call("haste_b200_layer_norm_gru_forward", _dtype(x), int(training), T, N, C, H,
                _p(kernel), _p(recurrent_kernel), _p(bias), _p(recurrent_bias), _p(gamma[0]),
                _p(gamma[1]), _p(x),
                _p(h), _p(cache), _p(act_Wx), _p(cache_Wx), _p(tmp_Wx_norm), _p(act_Rh),
                _p(cache_Rh), _p(tmp_Rh_norm), zp, mp, _stream())
    return [h, cache, act_Wx, cache_Wx, act_Rh, cache_Rh]


def layer_norm_gru_backward(x, kernel, recurrent_kernel, bias, recurrent_bias, gamma,
                            zoneout_mask, h, cache, act_Wx, cache_Wx, act_Rh, cache_Rh, dh_new,
                            transposed=True, grads=None):
    _check(x, kernel, recurrent_kernel, bias, recurrent_bias, gamma, zoneout_mask, h, cache,
           act_Wx, cache_Wx, act_Rh, cache_Rh, dh_new)
    H = h.shape[2]
    T, N, C, H = _dims_bwd(x, transposed, H)
    with torch.cuda.device(h.device):
        dx = h.new_empty(T, N, C)
        dW = _zeros(grads, h, C, 3 * H)
        dR = _zeros(grads, h, H, 3 * H)
        dbx = _zeros(grads, h, 3 * H)
        dbr = _zeros(grads, h, 3 * H)
        dh = h.new_zeros(N, H)
        dp = h.new_empty(T, N, 3 * H)
        dq = h.new_empty(T, N, 3 * H)
        dgamma = _zeros(grads, h, *gamma.shape)
        _C.call("haste_b200_layer_norm_gru_backward", _dtype(h), int(transposed), T, N, C, H,
                _p(kernel), _p(recurrent_kernel), _p(bias), _p(recurrent_bias), _p(gamma[0]),
                _p(gamma[1]), _p(x),
                _p(h), _p(cache), _p(dh_new), _p(dx), _p(dW), _p(dR), _p(dbx), _p(dbr),
                _p(dgamma[0]), _p(dgamma[1]), _p(dh), _p(dp), _p(dq), _p(act_Wx), _p(cache_Wx), _p(act_Rh),
                _p(cache_Rh), _p(zoneout_mask), _stream())
    return [dx, dh, dW, dR, dbx, dbr, dgamma]


# ---------------------------------------------------------------- LayerNormIndRNN
def layer_norm_indrnn_forward(training, zoneout_prob, x, h0, kernel, recurrent_scale, bias, gamma,
                              zoneout_mask):
    _check(x, h0, kernel, recurrent_scale, bias, gamma, zoneout_mask)
    T, N, C = x.shape
    H = kernel.shape[1]
    with torch.cuda.device(x.device):
        h = x.new_empty(T + 1, N, H)
        h[0] = h0
        workspace = x.new_empty(T, N, H)
        act_Wx = x.new_empty(T, N, H)
        cache_Wx = x.new_empty(T, N, 2)
        mp, zp = _mask_ptr(zoneout_prob, zoneout_mask)
        # gamma is [2,H]; only row 0 is used (frameworks/pytorch/layer_norm_indrnn.cc:67-72)
        _C.call("haste_b200_layer_norm_indrnn_forward", _dtype(x), int(training), T, N, C, H,
                _p(kernel), _p(recurrent_scale), _p(bias), _p(gamma), _p(x), _p(h),
                _p(workspace), _p(act_Wx), _p(cache_Wx), zp, mp, _stream())
    return [h, act_Wx, cache_Wx]


def layer_norm_indrnn_backward(x, kernel, recurrent_scale, bias, gamma, zoneout_mask, h, act_Wx,
                               cache_Wx, dh_new, transposed=True, grads=None):
    _check(x, kernel, recurrent_scale, bias, gamma, zoneout_mask, h, act_Wx, cache_Wx, dh_new)
    H = h.shape[2]
    T, N, C, H = _dims_bwd(x, transposed, H)
    with torch.cuda.device(h.device):
        dx = h.new_empty(T, N, C)
        dW = _zeros(grads, h, C, H)
        du = _zeros(grads, h, H)
        db = _zeros(grads, h, H)
        dh = h.new_zeros(N, H)
        dgamma = _zeros(grads, h, *gamma.shape)
        workspace = h.new_empty(T, N, H)
        _C.call("haste_b200_layer_norm_indrnn_backward", _dtype(h), int(transposed), T, N, C, H,
                _p(kernel), _p(recurrent_scale), _p(bias), _p(gamma), _p(x), _p(h), _p(dh_new),
                _p(dx), _p(dW), _p(du), _p(db), _p(dgamma), _p(dh), _p(workspace), _p(act_Wx),
                _p(cache_Wx), _p(zoneout_mask), _stream())
    return [dx, dh, dW, du, db, dgamma]


# ---------------------------------------------------------------- helpers for tests/bench
def gemm(a, b, out=None, accumulate=False):
    """out (+)= a @ b for 2-D CUDA tensors with arbitrary strides (views allowed)."""
    M, K = a.shape
    K2, N = b.shape
    assert K == K2
    if out is None:
        out = a.new_zeros(M, N)
    with torch.cuda.device(a.device):
        _C.call("haste_b200_gemm", _dtype(a), M, N, K, a.data_ptr(), a.stride(0), a.stride(1),
                b.data_ptr(), b.stride(0), b.stride(1), out.data_ptr(), out.stride(0),
                int(accumulate), _stream())
    return out

"""CPU oracle for the fused RNN layers (TEST INFRASTRUCTURE, not product code).

This file restates, in plain torch-on-CPU arithmetic, the algorithm of the
reference's CPU path for every cell, so that the CUDA kernels can be checked
against it on a machine where the reference itself is not present.  Nothing in
the `haste_b200` package imports it; only the tests, the smoke check and the
benchmark's CPU-baseline leg do.

Parity pin: every function here is checked against outputs and autograd
gradients of the reference's own Python functions (generated once, with the
reference imported, by `tests/golden/make_golden.py`; fixtures committed under
`tests/golden/`).  The reference has no golden vectors of its own.

Reference citations (paths inside lmnt-com/haste):
  lstm              frameworks/pytorch/lstm.py:33-66   (LSTMScript)
  gru               frameworks/pytorch/gru.py:33-66    (GRUScript)
  indrnn            frameworks/pytorch/indrnn.py:33-54 (IndRNNScript)
  layer_norm_lstm   frameworks/pytorch/layer_norm_lstm.py:33-69
  layer_norm_gru    frameworks/pytorch/layer_norm_gru.py:33-67
  layer_norm_indrnn frameworks/pytorch/layer_norm_indrnn.py:33-56
  layer_norm        lib/layer_norm_forward_gpu.cu.cc:22-88 (biased variance, eps 1e-5)
  zoneout           lib/lstm_forward_gpu.cu.cc:77-83
  bidirectional     frameworks/tf/base_rnn.py:115-121 (flip, run, flip back)

All state tensors follow the reference layout: `h`/`c` are `[T+1, N, H]` with
slot 0 holding the initial state; gate order is i,g,f,o (LSTM) and z,r,g (GRU).
Gradients come from autograd over these forward functions, exactly as in the
reference's CPU path.
"""

import torch

LN_EPS = 1e-5


def layer_norm(x, gamma, beta=None):
    """Row LayerNorm over the last axis: biased variance, eps inside the sqrt."""
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    y = (x - mean) * torch.rsqrt(var + LN_EPS) * gamma
    if beta is not None:
        y = y + beta
    return y


def _zoneout(h_new, h_prev, training, zoneout_prob, mask_t):
    if not zoneout_prob:
        return h_new
    if training:
        return (h_new - h_prev) * mask_t + h_prev
    return zoneout_prob * h_prev + (1 - zoneout_prob) * h_new


def _has_mask(zoneout_prob, mask):
    return bool(zoneout_prob) and mask is not None and mask.numel() > 0


def lstm(training, zoneout_prob, x, h0, c0, W, R, b, mask=None):
    T = x.shape[0]
    H = R.shape[0]
    zp = zoneout_prob if (not training or _has_mask(zoneout_prob, mask)) else 0.0
    h, c = [h0], [c0]
    Wx = x @ W
    for t in range(T):
        v = h[t] @ R + Wx[t] + b
        i = torch.sigmoid(v[:, 0 * H:1 * H])
        g = torch.tanh(v[:, 1 * H:2 * H])
        f = torch.sigmoid(v[:, 2 * H:3 * H])
        o = torch.sigmoid(v[:, 3 * H:4 * H])
        c_new = f * c[t] + i * g
        h_new = o * torch.tanh(c_new)
        h_new = _zoneout(h_new, h[t], training, zp, mask[t] if zp and training else None)
        c.append(c_new)
        h.append(h_new)
    return torch.stack(h), torch.stack(c)


def gru(training, zoneout_prob, x, h0, W, R, bx, br, mask=None):
    T = x.shape[0]
    H = R.shape[0]
    zp = zoneout_prob if (not training or _has_mask(zoneout_prob, mask)) else 0.0
    h = [h0]
    Wx = x @ W + bx
    for t in range(T):
        Rh = h[t] @ R + br
        z = torch.sigmoid(Wx[t][:, 0:H] + Rh[:, 0:H])
        r = torch.sigmoid(Wx[t][:, H:2 * H] + Rh[:, H:2 * H])
        g = torch.tanh(Wx[t][:, 2 * H:3 * H] + r * Rh[:, 2 * H:3 * H])
        h_new = z * h[t] + (1 - z) * g
        h_new = _zoneout(h_new, h[t], training, zp, mask[t] if zp and training else None)
        h.append(h_new)
    return torch.stack(h)


def indrnn(training, zoneout_prob, x, h0, W, u, b, mask=None):
    T = x.shape[0]
    zp = zoneout_prob if (not training or _has_mask(zoneout_prob, mask)) else 0.0
    h = [h0]
    Wx = x @ W + b
    for t in range(T):
        h_new = torch.tanh(Wx[t] + h[t] * u)
        h_new = _zoneout(h_new, h[t], training, zp, mask[t] if zp and training else None)
        h.append(h_new)
    return torch.stack(h)


def layer_norm_lstm(training, zoneout_prob, x, h0, c0, W, R, b, gamma, gamma_h, beta_h, mask=None):
    T = x.shape[0]
    H = R.shape[0]
    zp = zoneout_prob if (not training or _has_mask(zoneout_prob, mask)) else 0.0
    h, c = [h0], [c0]
    Wx = layer_norm(x @ W, gamma[0])
    for t in range(T):
        v = layer_norm(h[t] @ R, gamma[1]) + Wx[t] + b
        i = torch.sigmoid(v[:, 0 * H:1 * H])
        g = torch.tanh(v[:, 1 * H:2 * H])
        f = torch.sigmoid(v[:, 2 * H:3 * H])
        o = torch.sigmoid(v[:, 3 * H:4 * H])
        c_new = f * c[t] + i * g
        h_new = o * torch.tanh(layer_norm(c_new, gamma_h, beta_h))
        h_new = _zoneout(h_new, h[t], training, zp, mask[t] if zp and training else None)
        c.append(c_new)
        h.append(h_new)
    return torch.stack(h), torch.stack(c)


def layer_norm_gru(training, zoneout_prob, x, h0, W, R, bx, br, gamma, mask=None):
    T = x.shape[0]
    H = R.shape[0]
    zp = zoneout_prob if (not training or _has_mask(zoneout_prob, mask)) else 0.0
    h = [h0]
    Wx = layer_norm(x @ W, gamma[0]) + bx
    for t in range(T):
        Rh = layer_norm(h[t] @ R, gamma[1]) + br
        z = torch.sigmoid(Wx[t][:, 0:H] + Rh[:, 0:H])
        r = torch.sigmoid(Wx[t][:, H:2 * H] + Rh[:, H:2 * H])
        g = torch.tanh(Wx[t][:, 2 * H:3 * H] + r * Rh[:, 2 * H:3 * H])
        h_new = z * h[t] + (1 - z) * g
        h_new = _zoneout(h_new, h[t], training, zp, mask[t] if zp and training else None)
        h.append(h_new)
    return torch.stack(h)


def layer_norm_indrnn(training, zoneout_prob, x, h0, W, u, b, gamma, mask=None):
    T = x.shape[0]
    zp = zoneout_prob if (not training or _has_mask(zoneout_prob, mask)) else 0.0
    h = [h0]
    Wx = layer_norm(x @ W, gamma[0]) + b
    for t in range(T):
        h_new = torch.tanh(Wx[t] + h[t] * u)
        h_new = _zoneout(h_new, h[t], training, zp, mask[t] if zp and training else None)
        h.append(h_new)
    return torch.stack(h)


# name -> (function, names of differentiable inputs in call order, has cell state)
CELLS = {
    "lstm": (lstm, ["x", "h0", "c0", "W", "R", "b"], True),
    "gru": (gru, ["x", "h0", "W", "R", "bx", "br"], False),
    "indrnn": (indrnn, ["x", "h0", "W", "u", "b"], False),
    "layer_norm_lstm": (layer_norm_lstm,
                        ["x", "h0", "c0", "W", "R", "b", "gamma", "gamma_h", "beta_h"], True),
    "layer_norm_gru": (layer_norm_gru, ["x", "h0", "W", "R", "bx", "br", "gamma"], False),
    "layer_norm_indrnn": (layer_norm_indrnn, ["x", "h0", "W", "u", "b", "gamma"], False),
}

GATES = {"lstm": 4, "gru": 3, "indrnn": 1,
         "layer_norm_lstm": 4, "layer_norm_gru": 3, "layer_norm_indrnn": 1}


def make_inputs(cell, T, N, C, H, seed=0, dtype=torch.float64, zoneout=0.0, scale=1.0):
    """Seeded inputs and weights for one layer of `cell` (CPU tensors).

    Weight distributions follow the reference modules' `reset_parameters`
    in magnitude (xavier-uniform input kernel, unit-scale recurrent kernel) but
    every bias/gamma/beta is randomised so that each gradient path is exercised.
    """
    g = torch.Generator().manual_seed(seed)
    G = GATES[cell]

    def rnd(*shape, s=1.0):
        return (torch.randn(*shape, generator=g, dtype=torch.float64) * s).to(dtype)

    d = {}
    d["x"] = rnd(T, N, C, s=scale)
    d["h0"] = rnd(N, H, s=0.5)
    if CELLS[cell][2]:
        d["c0"] = rnd(N, H, s=0.5)
    bound = (6.0 / (C + H)) ** 0.5
    d["W"] = ((torch.rand(C, G * H, generator=g, dtype=torch.float64) * 2 - 1) * bound).to(dtype)
    if "indrnn" in cell:
        d["u"] = torch.rand(H, generator=g, dtype=torch.float64).to(dtype)
        d["b"] = rnd(H, s=0.1)
    else:
        d["R"] = rnd(H, G * H, s=1.0 / H ** 0.5)
        if "lstm" in cell:
            d["b"] = rnd(G * H, s=0.1)
        else:
            d["bx"] = rnd(G * H, s=0.1)
            d["br"] = rnd(G * H, s=0.1)
    if cell.startswith("layer_norm"):
        d["gamma"] = (1.0 + rnd(2, G * H, s=0.1))
        if cell == "layer_norm_lstm":
            d["gamma_h"] = (1.0 + rnd(H, s=0.1))
            d["beta_h"] = rnd(H, s=0.1)
    if zoneout:
        d["mask"] = torch.bernoulli(torch.full((T, N, H), 1.0 - zoneout, dtype=torch.float64),
                                    generator=g).to(dtype)
    else:
        d["mask"] = None
    # upstream gradients for every state slot 1..T
    d["dh"] = rnd(T + 1, N, H)
    if CELLS[cell][2]:
        d["dc"] = rnd(T + 1, N, H)
    return d


def forward(cell, d, training=True, zoneout=0.0):
    fn, names, has_c = CELLS[cell]
    args = [d[k] for k in names]
    out = fn(training, zoneout, *args, d.get("mask"))
    return out if has_c else (out,)


def forward_backward(cell, d, zoneout=0.0):
    """Returns ({'h':…, 'c':…}, {name: grad}) with grads of sum(h*dh)+sum(c*dc).

    As in the reference's backward, the upstream gradient of slot 0 is ignored
    (lib/lstm_backward_gpu.cu.cc:362-363 start reading at index i+1).
    """
    fn, names, has_c = CELLS[cell]
    leaves = {k: d[k].detach().clone().requires_grad_(True) for k in names}
    out = fn(True, zoneout, *[leaves[k] for k in names], d.get("mask"))
    if has_c:
        h, c = out
        loss = (h[1:] * d["dh"][1:]).sum() + (c[1:] * d["dc"][1:]).sum()
    else:
        h = out
        loss = (h[1:] * d["dh"][1:]).sum()
    grads = torch.autograd.grad(loss, [leaves[k] for k in names])
    res = {"h": h.detach()}
    if has_c:
        res["c"] = c.detach()
    return res, {k: g for k, g in zip(names, grads)}


def max_rel_err(a, b):
    """max|a-b| / max(max|b|, 1e-6): the parity metric (b is the oracle)."""
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    return float((a - b).abs().max() / max(float(b.abs().max()), 1e-6))

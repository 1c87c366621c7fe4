"""Why LayerNormLSTM has its own bf16 bar: rounding only the tensors that the interface
stores in bf16 and that feed the forward pass (x.W, LN(x.W), h), with all arithmetic exact
(float64), already moves outputs and gradients by more than the generic 2e-2 bf16 bar.  No
implementation with bf16 storage can be closer to the unrounded oracle than this."""
import torch

import haste_oracle as oracle
from helpers import TOL_BF16, TOL_BF16_LN_LSTM


class _Stored(torch.autograd.Function):
    """bf16 rounding of a stored tensor; gradients pass straight through."""

    @staticmethod
    def forward(ctx, a):
        return a.to(torch.bfloat16).to(torch.float64)

    @staticmethod
    def backward(ctx, g):
        return g


def _run(d, T, N, C, H, stored_in_bf16):
    r = _Stored.apply if stored_in_bf16 else (lambda a: a)
    names = ["x", "W", "R", "b", "gamma", "gamma_h", "beta_h"]
    L = {k: d[k].clone().requires_grad_(True) for k in names}
    g = L["gamma"]
    h, c = d["h0"], d["c0"]
    wx = r(L["x"].reshape(T * N, C) @ L["W"])                     # act_Wx
    wxn = r(oracle.layer_norm(wx, g[0])).reshape(T, N, 4 * H)     # act_Wx_norm
    hs, cs = [h], [c]
    for t in range(T):
        v = oracle.layer_norm(h @ L["R"], g[1]) + wxn[t] + L["b"]
        i, gg, f, o = v.chunk(4, 1)
        c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(gg)
        h = r(torch.sigmoid(o) * torch.tanh(oracle.layer_norm(c, L["gamma_h"], L["beta_h"])))
        hs.append(h)
        cs.append(c)
    hs, cs = torch.stack(hs), torch.stack(cs)
    loss = (hs * d["dh"]).sum() + (cs * d["dc"]).sum()
    grads = torch.autograd.grad(loss, [L[k] for k in names])
    return hs.detach(), dict(zip(names, grads))


def _inputs(T, N, C, H, seed):
    d = oracle.make_inputs("layer_norm_lstm", T, N, C, H, seed=seed, zoneout=0.0)
    return {k: (v.to(torch.bfloat16).to(torch.float64) if v is not None else None)
            for k, v in d.items()}


def test_storage_rounding_alone_exceeds_the_generic_bf16_bar():
    T, N, C, H = 20, 64, 64, 512
    d = _inputs(T, N, C, H, seed=H)
    exact_h, exact_g = _run(d, T, N, C, H, False)
    ref_out, ref_g = oracle.forward_backward("layer_norm_lstm", d, zoneout=0.0)
    # the restatement above is the oracle's math
    assert oracle.max_rel_err(exact_h, ref_out["h"]) < 1e-12
    assert oracle.max_rel_err(exact_g["W"], ref_g["W"]) < 1e-10
    h, _ = _run(d, T, N, C, H, True)
    floor = oracle.max_rel_err(h, exact_h)
    assert TOL_BF16 < floor < TOL_BF16_LN_LSTM, floor


def test_storage_rounding_floor_of_the_parameter_gradients():
    T, N, C, H = 16, 32, 64, 64
    d = _inputs(T, N, C, H, seed=77 + H)
    _, exact_g = _run(d, T, N, C, H, False)
    _, g = _run(d, T, N, C, H, True)
    floor = max(oracle.max_rel_err(g[k], exact_g[k]) for k in g)
    assert TOL_BF16 < floor < TOL_BF16_LN_LSTM, floor

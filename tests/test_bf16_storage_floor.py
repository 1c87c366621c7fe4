"""Why LayerNormLSTM has its own bf16 bar: rounding only the tensors that the interface
stores in bf16, with all arithmetic exact (float64), already moves the result by more than
the generic 2e-2 bf16 bar.  No implementation with bf16 storage can be closer than this."""
import torch

import haste_oracle as oracle
from helpers import TOL_BF16, TOL_BF16_LN_LSTM


def _bf(a):
    return a.to(torch.bfloat16).to(torch.float64)


def _forward(d, T, N, C, H, stored_in_bf16):
    r = _bf if stored_in_bf16 else (lambda a: a)
    g = d["gamma"]
    h, c = d["h0"], d["c0"]
    wx = r(d["x"].reshape(T * N, C) @ d["W"])                     # act_Wx
    wxn = r(oracle.layer_norm(wx, g[0])).reshape(T, N, 4 * H)     # act_Wx_norm
    hs = [h]
    for t in range(T):
        v = oracle.layer_norm(h @ d["R"], g[1]) + wxn[t] + d["b"]
        i, gg, f, o = v.chunk(4, 1)
        c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(gg)
        h = r(torch.sigmoid(o) * torch.tanh(oracle.layer_norm(c, d["gamma_h"], d["beta_h"])))
        hs.append(h)
    return torch.stack(hs)


def test_storage_rounding_alone_exceeds_the_generic_bf16_bar():
    T, N, C, H = 20, 64, 64, 512
    d = oracle.make_inputs("layer_norm_lstm", T, N, C, H, seed=H, zoneout=0.0)
    d = {k: (_bf(v) if v is not None else None) for k, v in d.items()}
    exact = _forward(d, T, N, C, H, False)
    ref_h, _ = oracle.forward("layer_norm_lstm", d, training=True, zoneout=0.0)
    assert oracle.max_rel_err(exact, ref_h) < 1e-12  # the restatement above is the oracle's math
    floor = oracle.max_rel_err(_forward(d, T, N, C, H, True), exact)
    assert TOL_BF16 < floor < TOL_BF16_LN_LSTM, floor

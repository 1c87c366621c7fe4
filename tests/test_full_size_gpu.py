"""Full-size cases of the benchmark configurations.

The headline workload (LSTM N=64, C=H=512, T=1000, fp32) is compared with the CPU oracle
directly (run in float32: a few seconds of CPU time) and, like the larger
configurations the oracle cannot finish quickly, through properties that hold at any size:
causality (a prefix of the sequence gives the prefix of the outputs), independence of batch
rows, and linearity of the backward pass in the incoming gradient."""
import pytest
import torch

import haste_oracle as oracle
from helpers import TOL_F32, assert_close, run_cuda

pytestmark = pytest.mark.gpu


def _config0_style(cell, T, N, C, H, seed):
    """Inputs as the benchmark configurations draw them: x ~ N(0,1), orthogonal recurrent
    blocks, xavier-uniform input blocks, zero biases."""
    d = oracle.make_inputs(cell, T, N, C, H, seed=seed)
    g = torch.Generator().manual_seed(seed + 1)
    G = d["R"].shape[1] // H
    R = torch.empty(H, G * H, dtype=torch.float64)
    W = torch.empty(C, G * H, dtype=torch.float64)
    for k in range(G):
        q, _ = torch.linalg.qr(torch.randn(H, H, generator=g, dtype=torch.float64))
        R[:, k * H:(k + 1) * H] = q
        lim = (6.0 / (C + H)) ** 0.5
        W[:, k * H:(k + 1) * H] = (torch.rand(C, H, generator=g, dtype=torch.float64) * 2 - 1) * lim
    d["R"], d["W"] = R, W
    d["x"] = torch.randn(T, N, C, generator=g, dtype=torch.float64)
    for k in ("b", "bx", "br"):
        if k in d:
            d[k] = torch.zeros_like(d[k])
    return d


def test_headline_lstm_full_size_against_oracle():
    T, N, C, H = 1000, 64, 512, 512
    d = _config0_style("lstm", T, N, C, H, seed=0)
    # float32 oracle at this size (the float64 one needs minutes of CPU time); its own
    # rounding error, ~1e-6, is far inside the bar
    d = {k: (v.float() if v is not None else None) for k, v in d.items()}
    ref_out, ref_grads = oracle.forward_backward("lstm", d)
    out, grads = run_cuda("lstm", d)
    assert_close(out["h"], ref_out["h"], TOL_F32, "h")
    assert_close(out["c"], ref_out["c"], TOL_F32, "c")
    for k, ref in ref_grads.items():
        assert_close(grads[k], ref, TOL_F32, "d" + k)


@pytest.mark.parametrize("cell,T,N,C,H", [("lstm", 1000, 64, 512, 512), ("gru", 1000, 128, 512, 512),
                                          ("layer_norm_lstm", 400, 64, 80, 512)])
def test_full_size_causality_batch_independence_and_linearity(cell, T, N, C, H):
    d = _config0_style(cell, T, N, C, H, seed=3)
    out, grads = run_cuda(cell, d)

    # causality: the first T/4 steps do not depend on what follows
    Tp = T // 4
    dp = dict(d)
    dp["x"] = d["x"][:Tp]
    for k in ("dh", "dc"):
        if k in d and d[k] is not None:
            dp[k] = d[k][:Tp + 1]
    if d.get("mask") is not None:
        dp["mask"] = d["mask"][:Tp]
    out_p, _ = run_cuda(cell, dp, backward=False)
    assert_close(out_p["h"], out["h"][:Tp + 1], 1e-6, "prefix h")

    # batch rows are independent: half of the batch alone gives the same rows
    Nh = N // 2
    dh_ = {k: (v[:, :Nh] if (v is not None and v.dim() == 3) else
               (v[:Nh] if (v is not None and k in ("h0", "c0")) else v)) for k, v in d.items()}
    out_h, grads_h = run_cuda(cell, dh_)
    assert_close(out_h["h"], out["h"][:, :Nh], 1e-5, "half-batch h")
    assert_close(grads_h["x"], grads["x"][:, :Nh], 2e-5, "half-batch dx")

    # the backward pass is linear in the incoming gradient: scaling it scales every gradient
    d2 = dict(d)
    d2["dh"] = d["dh"] * 2.0
    if d.get("dc") is not None:
        d2["dc"] = d["dc"] * 2.0
    _, grads2 = run_cuda(cell, d2)
    for k in grads:
        assert_close(grads2[k], 2.0 * grads[k].double(), 2e-5, "linearity d" + k)

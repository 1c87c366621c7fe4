"""Single-step entry points (the reference's Iterate API): stepping through a sequence one
call at a time must give the oracle's outputs and gradients."""
import pytest
import torch

import haste_oracle as oracle
from helpers import TOL_F32, assert_close

pytestmark = pytest.mark.gpu


def _p(t):
    return t.data_ptr() if t is not None else None


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("zoneout", [0.0, 0.3])
def test_lstm_iterate_matches_oracle(zoneout, transposed):
    from haste_b200 import _C
    T, N, C, H = 7, 5, 12, 24
    d = oracle.make_inputs("lstm", T, N, C, H, seed=21, zoneout=zoneout)
    ref_out, ref_g = oracle.forward_backward("lstm", d, zoneout=zoneout)
    cu = lambda t: t.float().cuda().contiguous()
    x, W, R, b = cu(d["x"]), cu(d["W"]), cu(d["R"]), cu(d["b"])
    mask = cu(d["mask"]) if zoneout else None
    s = torch.cuda.current_stream().cuda_stream
    h = [cu(d["h0"])] + [torch.empty(N, H, device="cuda") for _ in range(T)]
    c = [cu(d["c0"])] + [torch.empty(N, H, device="cuda") for _ in range(T)]
    v = [torch.empty(N, 4 * H, device="cuda") for _ in range(T)]
    tmp = torch.empty(N, 4 * H, device="cuda")
    for t in range(T):
        _C.call("haste_b200_lstm_forward_iterate", _C.F32, 1, N, C, H, _p(W), _p(R), _p(b),
                _p(x[t]), _p(h[t]), _p(c[t]), _p(h[t + 1]), _p(c[t + 1]), _p(v[t]), _p(tmp),
                float(zoneout), _p(mask[t]) if zoneout else None, s)
    assert_close(torch.stack(h), ref_out["h"], TOL_F32, "h")
    assert_close(torch.stack(c), ref_out["c"], TOL_F32, "c")

    dhn, dcn = cu(d["dh"]), cu(d["dc"])
    dW, dR, db = torch.zeros_like(W), torch.zeros_like(R), torch.zeros_like(b)
    dh, dc = torch.zeros(N, H, device="cuda"), torch.zeros(N, H, device="cuda")
    dx = torch.empty(T, N, C, device="cuda")
    Wa = W.t().contiguous() if transposed else W
    Ra = R.t().contiguous() if transposed else R
    for t in reversed(range(T)):
        xt = x[t].t().contiguous() if transposed else x[t]
        _C.call("haste_b200_lstm_backward_iterate", _C.F32, int(transposed), N, C, H, _p(Wa),
                _p(Ra), _p(b), _p(xt), _p(h[t]), _p(c[t]), _p(c[t + 1]), _p(dhn[t + 1]),
                _p(dcn[t + 1]), _p(dx[t]), _p(dW), _p(dR), _p(db), _p(dh), _p(dc), _p(v[t]),
                _p(mask[t]) if zoneout else None, s)
    _C.sync_check(s)
    got = {"x": dx, "W": dW, "R": dR, "b": db, "h0": dh, "c0": dc}
    for k, ref in ref_g.items():
        assert_close(got[k], ref, TOL_F32, "d" + k)


@pytest.mark.parametrize("zoneout", [0.0, 0.3])
def test_gru_iterate_matches_oracle(zoneout):
    from haste_b200 import _C
    T, N, C, H = 6, 4, 10, 40
    d = oracle.make_inputs("gru", T, N, C, H, seed=22, zoneout=zoneout)
    ref_out, ref_g = oracle.forward_backward("gru", d, zoneout=zoneout)
    cu = lambda t: t.float().cuda().contiguous()
    x, W, R, bx, br = cu(d["x"]), cu(d["W"]), cu(d["R"]), cu(d["bx"]), cu(d["br"])
    mask = cu(d["mask"]) if zoneout else None
    s = torch.cuda.current_stream().cuda_stream
    h = [cu(d["h0"])] + [torch.empty(N, H, device="cuda") for _ in range(T)]
    v = [torch.empty(N, 4 * H, device="cuda") for _ in range(T)]
    tmp_wx, tmp_rh = torch.empty(N, 3 * H, device="cuda"), torch.empty(N, 3 * H, device="cuda")
    for t in range(T):
        _C.call("haste_b200_gru_forward_iterate", _C.F32, 1, N, C, H, _p(W), _p(R), _p(bx), _p(br),
                _p(x[t]), _p(h[t]), _p(h[t + 1]), _p(v[t]), _p(tmp_wx), _p(tmp_rh), float(zoneout),
                _p(mask[t]) if zoneout else None, s)
    assert_close(torch.stack(h), ref_out["h"], TOL_F32, "h")

    dhn = cu(d["dh"])
    dW, dR = torch.zeros_like(W), torch.zeros_like(R)
    dbx, dbr = torch.zeros_like(bx), torch.zeros_like(br)
    dh = torch.zeros(N, H, device="cuda")
    dx = torch.empty(T, N, C, device="cuda")
    dp, dq = torch.empty(N, 3 * H, device="cuda"), torch.empty(N, 3 * H, device="cuda")
    for t in reversed(range(T)):
        _C.call("haste_b200_gru_backward_iterate", _C.F32, 0, N, C, H, _p(W), _p(R), _p(bx),
                _p(br), _p(x[t]), _p(h[t]), _p(v[t]), _p(dhn[t + 1]), _p(dx[t]), _p(dW), _p(dR),
                _p(dbx), _p(dbr), _p(dh), _p(dp), _p(dq), _p(mask[t]) if zoneout else None, s)
    _C.sync_check(s)
    got = {"x": dx, "W": dW, "R": dR, "bx": dbx, "br": dbr, "h0": dh}
    for k, ref in ref_g.items():
        assert_close(got[k], ref, TOL_F32, "d" + k)

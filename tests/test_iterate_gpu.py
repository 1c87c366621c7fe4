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


@pytest.mark.parametrize("cell", ["lstm", "gru"])
@pytest.mark.parametrize("N,C,H", [(1, 12, 24), (7, 100, 50), (64, 512, 512), (24, 80, 1024),
                                   (64, 1024, 1024)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("training", [True, False])
def test_fused_single_launch_step_equals_the_general_path(cell, N, C, H, dtype, training):
    """Up to 64 rows a forward Iterate call is ONE launch (x.W + h.R + the cell fused); the
    step-wise path (two contractions and a pointwise kernel) is the check, plus the oracle."""
    from haste_b200 import _C
    zoneout = 0.25
    d = oracle.make_inputs(cell, 1, N, C, H, seed=N + H, zoneout=zoneout)
    bf16 = dtype == torch.bfloat16
    if bf16:
        d = {k: (v.to(dtype).to(v.dtype) if v is not None else None) for k, v in d.items()}
    cu = lambda t: t.to(dtype).cuda().contiguous()
    x, W, R, h0, mask = cu(d["x"][0]), cu(d["W"]), cu(d["R"]), cu(d["h0"]), cu(d["mask"][0])
    s = torch.cuda.current_stream().cuda_stream
    dt = _C.BF16 if bf16 else _C.F32
    G = 4 if cell == "lstm" else 3
    outs = {}
    launches = {}
    try:
        for name, path in (("fused", _C.PATH_AUTO), ("stepwise", _C.PATH_STEPWISE)):
            _C.set_recurrence_path(path)
            h1 = torch.empty(N, H, device="cuda", dtype=dtype)
            v = torch.zeros(N, 4 * H, device="cuda", dtype=dtype)
            tmp = torch.empty(N, G * H, device="cuda", dtype=dtype)
            n0 = _C.launch_count()
            if cell == "lstm":
                c0, b = cu(d["c0"]), cu(d["b"])
                c1 = torch.empty(N, H, device="cuda", dtype=dtype)
                _C.call("haste_b200_lstm_forward_iterate", dt, int(training), N, C, H, _p(W), _p(R),
                        _p(b), _p(x), _p(h0), _p(c0), _p(h1), _p(c1), _p(v), _p(tmp), zoneout,
                        _p(mask), s)
                outs[name] = (h1, c1, v)
            else:
                bx, br = cu(d["bx"]), cu(d["br"])
                tmp2 = torch.empty(N, G * H, device="cuda", dtype=dtype)
                _C.call("haste_b200_gru_forward_iterate", dt, int(training), N, C, H, _p(W), _p(R),
                        _p(bx), _p(br), _p(x), _p(h0), _p(h1), _p(v), _p(tmp), _p(tmp2), zoneout,
                        _p(mask), s)
                outs[name] = (h1, v)
            _C.sync_check(s)
            launches[name] = _C.launch_count() - n0
    finally:
        _C.set_recurrence_path(_C.PATH_AUTO)
    # (the largest case is beyond the size up to which the fused launch is faster)
    if N * (C + H) * H <= 64 * 1024 * 512:
        assert launches["fused"] == 1 and launches["stepwise"] > 1, launches
    tol = 2e-2 if bf16 else 2e-5
    for a, b in zip(outs["fused"], outs["stepwise"]):
        if training or a.shape[1] == H:  # the gate cache is written only when training
            assert_close(a, b, tol, "fused vs step-wise")
    if training:
        ref_out, _ = oracle.forward_backward(cell, d, zoneout=zoneout)
        assert_close(outs["fused"][0], ref_out["h"][1], tol if bf16 else TOL_F32, "h vs oracle")

"""haste_b200 against the REFERENCE's own CUDA build on the same device buffers.

The reference library is built out of tree by oracle/build_ref.py (only where the
reference checkout exists); these tests skip when it is absent."""
import pytest
import torch

import haste_oracle as oracle
from helpers import TOL_F32, assert_close, run_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    import ref_cuda
    if not ref_cuda.available():
        pytest.skip("reference CUDA build not present")
    return ref_cuda


def _cuda(d):
    return {k: (v.float().cuda().contiguous() if v is not None else None) for k, v in d.items()}


@pytest.mark.parametrize("zoneout", [0.0, 0.2])
@pytest.mark.parametrize("shape", [(20, 8, 16, 32), (50, 32, 128, 256)])
def test_lstm_matches_reference_cuda(ref, shape, zoneout):
    T, N, C, H = shape
    d = oracle.make_inputs("lstm", T, N, C, H, seed=1, zoneout=zoneout)
    t = _cuda(d)
    h, c, v = ref.lstm_forward(True, zoneout, t["x"], t["h0"], t["c0"], t["W"], t["R"], t["b"], t["mask"])
    g = ref.lstm_backward(t["x"], t["W"], t["R"], t["b"], t["mask"], h, c, v, t["dh"], t["dc"])
    out, grads = run_cuda("lstm", d, zoneout=zoneout)
    assert_close(out["h"], h, TOL_F32, "h")
    assert_close(out["c"], c, TOL_F32, "c")
    for k in g:
        assert_close(grads[k], g[k], TOL_F32, "d" + k)


@pytest.mark.parametrize("zoneout", [0.0, 0.2])
@pytest.mark.parametrize("shape", [(20, 8, 16, 32), (50, 32, 128, 256)])
def test_gru_matches_reference_cuda(ref, shape, zoneout):
    T, N, C, H = shape
    d = oracle.make_inputs("gru", T, N, C, H, seed=2, zoneout=zoneout)
    t = _cuda(d)
    h, v = ref.gru_forward(True, zoneout, t["x"], t["h0"], t["W"], t["R"], t["bx"], t["br"], t["mask"])
    g = ref.gru_backward(t["x"], t["W"], t["R"], t["bx"], t["br"], t["mask"], h, v, t["dh"])
    out, grads = run_cuda("gru", d, zoneout=zoneout)
    assert_close(out["h"], h, TOL_F32, "h")
    for k in g:
        assert_close(grads[k], g[k], TOL_F32, "d" + k)


def test_indrnn_matches_reference_cuda(ref):
    T, N, C, H = 40, 16, 64, 128
    d = oracle.make_inputs("indrnn", T, N, C, H, seed=3, zoneout=0.1)
    t = _cuda(d)
    h = ref.indrnn_forward(True, 0.1, t["x"], t["h0"], t["W"], t["u"], t["b"], t["mask"])
    g = ref.indrnn_backward(t["x"], t["W"], t["u"], t["b"], t["mask"], h, t["dh"])
    out, grads = run_cuda("indrnn", d, zoneout=0.1)
    assert_close(out["h"], h, TOL_F32, "h")
    for k in g:
        assert_close(grads[k], g[k], TOL_F32, "d" + k)

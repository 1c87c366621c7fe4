"""haste_b200 against the REFERENCE's own CUDA build on the same device buffers.

The reference library is built out of tree by oracle/build_ref.py (only where the
reference checkout exists); these tests skip when it is absent.

The reference's GRU runs its cuBLAS calls under CUBLAS_TENSOR_OP_MATH
(lib/gru_forward_gpu.cu.cc:331), which on current cuBLAS means TF32 products, so the
reference CUDA build is itself only ~5e-4 close to exact arithmetic there.  Each check
is therefore: ours is within the parity bar of the float64 oracle, and ours is as close
to the reference build as the reference build is to the oracle (plus the bar)."""
import pytest
import torch

import haste_oracle as oracle
from helpers import TOL_F32, max_rel_err, run_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    import ref_cuda
    if not ref_cuda.available():
        pytest.skip("reference CUDA build not present")
    return ref_cuda


def _cuda(d):
    return {k: (v.float().cuda().contiguous() if v is not None else None) for k, v in d.items()}


def _check(cell, d, zoneout, ref_h, ref_g, ref_c=None):
    o_out, o_g = oracle.forward_backward(cell, d, zoneout=zoneout)
    out, grads = run_cuda(cell, d, zoneout=zoneout)
    pairs = [("h", out["h"], ref_h, o_out["h"])]
    if ref_c is not None:
        pairs.append(("c", out["c"], ref_c, o_out["c"]))
    pairs += [("d" + k, grads[k], ref_g[k], o_g[k]) for k in ref_g]
    for name, ours, theirs, exact in pairs:
        e_ours = max_rel_err(ours, exact)
        e_ref = max_rel_err(theirs, exact)
        e_pair = max_rel_err(ours, theirs)
        assert e_ours < TOL_F32, f"{name}: ours vs oracle {e_ours:.2e}"
        assert e_pair < TOL_F32 + 2 * e_ref, \
            f"{name}: ours vs reference CUDA {e_pair:.2e} (reference vs oracle {e_ref:.2e})"


@pytest.mark.parametrize("zoneout", [0.0, 0.2])
@pytest.mark.parametrize("shape", [(20, 8, 16, 32), (50, 32, 128, 256)])
def test_lstm_matches_reference_cuda(ref, shape, zoneout):
    T, N, C, H = shape
    d = oracle.make_inputs("lstm", T, N, C, H, seed=1, zoneout=zoneout)
    t = _cuda(d)
    h, c, v = ref.lstm_forward(True, zoneout, t["x"], t["h0"], t["c0"], t["W"], t["R"], t["b"], t["mask"])
    g = ref.lstm_backward(t["x"], t["W"], t["R"], t["b"], t["mask"], h, c, v, t["dh"], t["dc"])
    _check("lstm", d, zoneout, h, g, c)


@pytest.mark.parametrize("zoneout", [0.0, 0.2])
@pytest.mark.parametrize("shape", [(20, 8, 16, 32), (50, 32, 128, 256)])
def test_gru_matches_reference_cuda(ref, shape, zoneout):
    T, N, C, H = shape
    d = oracle.make_inputs("gru", T, N, C, H, seed=2, zoneout=zoneout)
    t = _cuda(d)
    h, v = ref.gru_forward(True, zoneout, t["x"], t["h0"], t["W"], t["R"], t["bx"], t["br"], t["mask"])
    g = ref.gru_backward(t["x"], t["W"], t["R"], t["bx"], t["br"], t["mask"], h, v, t["dh"])
    _check("gru", d, zoneout, h, g)


def test_indrnn_matches_reference_cuda(ref):
    T, N, C, H = 40, 16, 64, 128
    d = oracle.make_inputs("indrnn", T, N, C, H, seed=3, zoneout=0.1)
    t = _cuda(d)
    h = ref.indrnn_forward(True, 0.1, t["x"], t["h0"], t["W"], t["u"], t["b"], t["mask"])
    g = ref.indrnn_backward(t["x"], t["W"], t["u"], t["b"], t["mask"], h, t["dh"])
    _check("indrnn", d, 0.1, h, g)


@pytest.mark.parametrize("zoneout", [0.0, 0.2])
@pytest.mark.parametrize("shape", [(12, 8, 16, 32), (30, 32, 80, 256)])
def test_layer_norm_lstm_matches_reference_cuda(ref, shape, zoneout):
    T, N, C, H = shape
    d = oracle.make_inputs("layer_norm_lstm", T, N, C, H, seed=4, zoneout=zoneout)
    t = _cuda(d)
    h, c, saved = ref.layer_norm_lstm_forward(True, zoneout, t["x"], t["h0"], t["c0"], t["W"], t["R"],
                                              t["b"], t["gamma"], t["gamma_h"], t["beta_h"], t["mask"])
    g = ref.layer_norm_lstm_backward(t["x"], t["W"], t["R"], t["b"], t["gamma"], t["gamma_h"],
                                     t["beta_h"], t["mask"], h, c, saved, t["dh"], t["dc"])
    _check("layer_norm_lstm", d, zoneout, h, g, c)


@pytest.mark.parametrize("zoneout", [0.0, 0.2])
@pytest.mark.parametrize("shape", [(12, 8, 16, 32), (30, 32, 80, 256)])
def test_layer_norm_gru_matches_reference_cuda(ref, shape, zoneout):
    T, N, C, H = shape
    d = oracle.make_inputs("layer_norm_gru", T, N, C, H, seed=5, zoneout=zoneout)
    t = _cuda(d)
    h, saved = ref.layer_norm_gru_forward(True, zoneout, t["x"], t["h0"], t["W"], t["R"], t["bx"],
                                          t["br"], t["gamma"], t["mask"])
    g = ref.layer_norm_gru_backward(t["x"], t["W"], t["R"], t["bx"], t["br"], t["gamma"], t["mask"],
                                    h, saved, t["dh"])
    _check("layer_norm_gru", d, zoneout, h, g)


def test_layer_norm_indrnn_matches_reference_cuda(ref):
    T, N, C, H = 40, 16, 64, 128
    d = oracle.make_inputs("layer_norm_indrnn", T, N, C, H, seed=6, zoneout=0.1)
    t = _cuda(d)
    h, saved = ref.layer_norm_indrnn_forward(True, 0.1, t["x"], t["h0"], t["W"], t["u"], t["b"],
                                             t["gamma"], t["mask"])
    g = ref.layer_norm_indrnn_backward(t["x"], t["W"], t["u"], t["b"], t["gamma"], t["mask"], h,
                                       saved, t["dh"])
    # row 1 of gamma is unused by this cell on both sides
    g["gamma"] = g["gamma"][0]
    o_out, o_g = oracle.forward_backward("layer_norm_indrnn", d, zoneout=0.1)
    out, grads = run_cuda("layer_norm_indrnn", d, zoneout=0.1)
    grads["gamma"] = grads["gamma"][0]
    o_g["gamma"] = o_g["gamma"][0]
    for name, ours, theirs, exact in [("h", out["h"], h, o_out["h"])] + \
            [("d" + k, grads[k], g[k], o_g[k]) for k in g]:
        e_ours, e_ref = max_rel_err(ours, exact), max_rel_err(theirs, exact)
        assert e_ours < TOL_F32, f"{name}: ours vs oracle {e_ours:.2e}"
        assert max_rel_err(ours, theirs) < TOL_F32 + 2 * e_ref, name

"""The oracle must reproduce the reference-generated fixtures (CPU only)."""
import os

import pytest
import torch

import haste_oracle as oracle
from helpers import golden_files, load_golden, max_rel_err


@pytest.mark.parametrize("path", golden_files(), ids=os.path.basename)
def test_oracle_matches_reference_fixture(path):
    cell, dims, zo, d, out, grads = load_golden(path, torch.float64)
    res, g = oracle.forward_backward(cell, d, zoneout=zo)
    assert max_rel_err(res["h"], out["h"]) < 1e-12
    if "c" in out:
        assert max_rel_err(res["c"], out["c"]) < 1e-12
    for k, ref in grads.items():
        assert max_rel_err(g[k], ref) < 1e-10, k
    with torch.no_grad():
        h_inf = oracle.forward(cell, d, training=False, zoneout=zo)[0]
    assert max_rel_err(h_inf, out["h_inference"]) < 1e-12


@pytest.mark.parametrize("path", golden_files()[:4], ids=os.path.basename)
def test_oracle_float32_close_to_fixture(path):
    cell, dims, zo, d, out, grads = load_golden(path, torch.float32)
    res, g = oracle.forward_backward(cell, d, zoneout=zo)
    assert max_rel_err(res["h"], out["h"]) < 1e-5
    for k, ref in grads.items():
        assert max_rel_err(g[k], ref) < 1e-4, k

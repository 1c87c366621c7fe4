"""The compiled PyTorch extension `haste_pytorch_lib` (haste_b200/torch_ext): the module name,
function names, argument order and returned lists of the reference's extension
(frameworks/pytorch/*.cc, bound by `import haste_pytorch_lib as LIB` in frameworks/pytorch/lstm.py:19),
over the haste_b200 C ABI.

CPU: the module builds, imports, exports the twelve functions and rejects CPU tensors with the
reference's error.  GPU: every op called the way the reference's autograd functions call it
(pre-transposed x, kernel, recurrent_kernel; an empty mask tensor for "no zoneout") returns
bit-identical tensors to `haste_b200.ops` and matches the oracle.
"""
import os
import sys

import pytest
import torch

import haste_oracle as oracle
from helpers import TOL_BF16, TOL_F32, assert_close, run_cuda

NAMES = [c + p for c in ("lstm", "gru", "indrnn", "layer_norm_lstm", "layer_norm_gru",
                         "layer_norm_indrnn") for p in ("_forward", "_backward")]


@pytest.fixture(scope="module")
def LIB():
    from haste_b200 import build
    # the module is built in-tree by `python -m haste_b200.build --torch-ext` (and by the
    # repository's build entry point); build it here only if that has not happened
    path = build.TORCH_EXT if os.path.exists(build.TORCH_EXT) else build.build_torch_ext()
    d = os.path.dirname(path)
    if d not in sys.path:
        sys.path.insert(0, d)
    import haste_pytorch_lib
    return haste_pytorch_lib


def test_module_exports_the_reference_functions(LIB):
    for n in NAMES:
        assert callable(getattr(LIB, n)), n


def test_cpu_tensors_are_rejected_like_the_reference(LIB):
    z = torch.zeros(2, 2, 2)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        LIB.lstm_forward(True, 0.0, z, z[0], z[0], z[0], z[0], z[0, 0], z)


@pytest.mark.gpu
@pytest.mark.parametrize("cell", list(oracle.CELLS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["fp32", "bf16"])
@pytest.mark.parametrize("zoneout", [0.0, 0.2])
def test_compiled_ops_equal_ctypes_ops_and_oracle(LIB, cell, dtype, zoneout):
    T, N, C, H = 12, 5, 24, 32
    d = oracle.make_inputs(cell, T, N, C, H, seed=3, zoneout=zoneout)
    bf16 = dtype == torch.bfloat16
    if bf16:
        d = {k: (v.to(dtype).to(v.dtype) if v is not None else None) for k, v in d.items()}
    out_c, g_c = run_cuda(cell, d, zoneout=zoneout, dtype=dtype, lib=LIB)
    out_p, g_p = run_cuda(cell, d, zoneout=zoneout, dtype=dtype, transposed=True)
    for k in out_p:
        assert torch.equal(out_c[k], out_p[k]), k
    for k in g_p:
        assert torch.equal(g_c[k], g_p[k]), "d" + k
    ref_out, ref_g = oracle.forward_backward(cell, d, zoneout=zoneout)
    tol = TOL_BF16 if bf16 else TOL_F32
    assert_close(out_c["h"], ref_out["h"], tol, "h")
    for k in ref_g:
        assert_close(g_c[k], ref_g[k], tol, "d" + k)

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


def _reference_root():
    env = os.environ.get("HASTE_REFERENCE_ROOT")
    here = os.path.dirname(os.path.abspath(__file__))
    sibling = os.path.join(os.path.dirname(os.path.dirname(here)), "reference")
    root = env or sibling
    return root if os.path.isdir(os.path.join(root, "frameworks", "pytorch")) else None


@pytest.mark.skipif(_reference_root() is None, reason="needs a checkout of the reference")
def test_the_reference_python_package_binds_to_the_compiled_module(LIB):
    """`import haste_pytorch_lib as LIB` in the reference's own modules resolves to this
    repository's compiled module: the package imports unchanged (only its generated version
    file is stood in for) and every LIB.<op> its autograd functions call exists here."""
    import importlib.util
    import re
    import types
    pkg_dir = os.path.join(_reference_root(), "frameworks", "pytorch")
    saved = {k: sys.modules.get(k) for k in ("haste_pytorch", "haste_pytorch._version")}
    try:
        ver = types.ModuleType("haste_pytorch._version")
        ver.__version__ = "reference"
        sys.modules["haste_pytorch._version"] = ver
        spec = importlib.util.spec_from_file_location(
            "haste_pytorch", os.path.join(pkg_dir, "__init__.py"),
            submodule_search_locations=[pkg_dir])
        mod = importlib.util.module_from_spec(spec)
        sys.modules["haste_pytorch"] = mod
        spec.loader.exec_module(mod)
        assert mod.lstm.LIB is LIB and mod.layer_norm_gru.LIB is LIB
        called = set()
        for name in ("lstm", "gru", "indrnn", "layer_norm_lstm", "layer_norm_gru", "layer_norm_indrnn"):
            with open(os.path.join(pkg_dir, name + ".py")) as f:
                called |= set(re.findall(r"LIB\.(\w+)\(", f.read()))
        assert called == set(NAMES), called ^ set(NAMES)
        # a CPU model of the reference still runs (its own fallback path), so the import is whole
        m = mod.LSTM(4, 6)
        y, _ = m(torch.zeros(3, 2, 4))
        assert y.shape == (3, 2, 6)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
        for k in [k for k in sys.modules if k.startswith("haste_pytorch.")]:
            sys.modules.pop(k, None)

"""CPU-side checks of the C ABI: the library loads and exports every declared symbol."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "haste_b200.h")


@pytest.fixture(scope="module")
def built_lib():
    from haste_b200 import build
    return build.build()


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(haste_b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_all_cells():
    syms = declared_symbols()
    for cell in ["lstm", "gru", "indrnn", "layer_norm_lstm", "layer_norm_gru",
                 "layer_norm_indrnn", "layer_norm"]:
        assert f"haste_b200_{cell}_forward" in syms
        assert f"haste_b200_{cell}_backward" in syms


def test_library_exports_every_declared_symbol(built_lib):
    L = ctypes.CDLL(built_lib)
    for name in declared_symbols():
        assert hasattr(L, name), name


def test_binding_table_matches_header(built_lib):
    from haste_b200 import _C
    bound = set(_C.SIGNATURES) | set(_C.OTHER_SYMBOLS)
    assert bound == set(declared_symbols())
    # argument counts in the ctypes table match the header's parameter lists
    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    for name, args in _C.SIGNATURES.items():
        m = re.search(name + r"\s*\((.*?)\)\s*;", text, flags=re.S)
        params = [p for p in m.group(1).split(",") if p.strip() and p.strip() != "void"]
        assert len(params) == len(args), name


def test_version_and_error_calls_work_without_gpu(built_lib):
    from haste_b200 import _C
    L = _C.lib()
    assert L.haste_b200_version().decode().count(".") == 2
    assert _C.launch_count() >= 0
    # argument validation happens before any CUDA call
    status = L.haste_b200_lstm_forward(0, 1, 4, 0, 3, 5, None, None, None, None, None, None,
                                       None, None, 0.0, None, None)
    assert status == 1
    assert b"invalid argument" in L.haste_b200_last_error()
    with pytest.raises(_C.HasteError):
        _C.call("haste_b200_set_gemm_path", 17)

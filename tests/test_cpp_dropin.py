"""The drop-in C++ API (include/haste_b200/haste.hpp): it must compile against the reference's
calling convention (CPU check), and one LSTM forward+backward driven from C++ must give the
same numbers as the same computation driven through the Python ops (GPU check)."""
import math
import os
import subprocess

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "dropin_api.cu")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")


@pytest.fixture(scope="module")
def binary(tmp_path_factory):
    from haste_b200 import build
    lib = build.build()
    out = str(tmp_path_factory.mktemp("cpp") / "dropin_api")
    libdir = os.path.dirname(lib)
    r = subprocess.run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-I",
                        os.path.join(ROOT, "include"), SRC, "-o", out, "-L", libdir,
                        "-lhaste_b200", "-Xlinker", "-rpath=" + libdir],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return out


def test_cpp_api_compiles_and_links(binary):
    assert os.path.exists(binary)


BENCH_SRC = os.path.join(ROOT, "haste_b200", "examples", "benchmark_rnn.cu")


@pytest.fixture(scope="module")
def bench_binary(tmp_path_factory):
    from haste_b200 import build
    lib = build.build()
    out = str(tmp_path_factory.mktemp("cppbench") / "benchmark_rnn")
    libdir = os.path.dirname(lib)
    r = subprocess.run([NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-I",
                        os.path.join(ROOT, "include"), BENCH_SRC, "-o", out, "-L", libdir,
                        "-lhaste_b200", "-Xlinker", "-rpath=" + libdir],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return out


def test_cpp_benchmark_driver_compiles(bench_binary):
    assert os.path.exists(bench_binary)


@pytest.mark.gpu
@pytest.mark.parametrize("extra", [[], ["--inference"], ["--cell", "gru"]])
def test_cpp_benchmark_driver_prints_the_reference_csv(bench_binary, extra):
    r = subprocess.run([bench_binary, "--point", "32,128,64", "--sample_size", "2",
                        "--time_steps", "20"] + extra, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    rows = [l for l in r.stdout.splitlines() if l and not l.startswith("#")]
    assert len(rows) == 1
    n, h, c, ms = rows[0].split(",")
    assert (int(n), int(h), int(c)) == (32, 128, 64) and 0.0 < float(ms) < 1000.0


def _fill(n, phase, scale):
    return torch.tensor([scale * math.sin(0.37 * i + phase) for i in range(n)], dtype=torch.float32)


def _checksum(t):
    t = t.detach().double().cpu().reshape(-1)
    w = (torch.arange(t.numel()) % 7 + 1).double()
    return float((t * w).sum())


@pytest.mark.gpu
def test_cpp_api_matches_python_ops(binary):
    from haste_b200 import ops
    r = subprocess.run([binary], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    got = {k: float(v) for k, v in (line.split() for line in r.stdout.strip().splitlines())}
    T, N, C, H = 6, 5, 7, 12
    x = _fill(T * N * C, 0.1, 1.0).reshape(T, N, C).cuda()
    W = _fill(C * 4 * H, 0.2, 0.4).reshape(C, 4 * H).cuda()
    R = _fill(H * 4 * H, 0.3, 0.3).reshape(H, 4 * H).cuda()
    b = _fill(4 * H, 0.4, 0.1).cuda()
    dh = _fill((T + 1) * N * H, 0.5, 1.0).reshape(T + 1, N, H).cuda()
    dc = _fill((T + 1) * N * H, 0.6, 1.0).reshape(T + 1, N, H).cuda()
    z = torch.zeros(N, H, device="cuda")
    nomask = torch.empty(0, 0, 0, device="cuda")
    h, c, cache = ops.lstm_forward(True, 0.0, x, z, z, W, R, b, nomask)
    dx, dh0, dc0, dW, dR, db = ops.lstm_backward(x, W, R, b, nomask, h, c, cache, dh, dc,
                                                 transposed=False)
    want = {"h": h, "dx": dx, "dW": dW, "dR": dR, "db": db, "dh": dh0, "dc": dc0}
    for k, t in want.items():
        ref = _checksum(t)
        assert abs(got[k] - ref) <= 1e-4 * max(1.0, abs(ref)), (k, got[k], ref)

"""GPU parity tests: the CUDA path (through the C ABI) against the reference-generated
fixtures and against the CPU oracle.  Bars: 1e-4 (fp32), 2e-2 (bf16), max|a-b|/max|b|."""
import os

import pytest
import torch

import haste_oracle as oracle
from helpers import (TOL_BF16, TOL_BF16_ALL_STORAGE_LN_LSTM, TOL_F16, TOL_F32, assert_close,
                     golden_files, load_golden, run_cuda)

pytestmark = pytest.mark.gpu

CELLS = list(oracle.CELLS)


def _compare(cell, d, out, grads, ref_out, ref_grads, tol):
    assert_close(out["h"], ref_out["h"], tol, f"{cell} h")
    if "c" in ref_out:
        assert_close(out["c"], ref_out["c"], tol, f"{cell} c")
    for k, ref in ref_grads.items():
        got = grads[k]
        if k == "gamma" and cell == "layer_norm_indrnn":
            got, ref = got[0], ref[0]  # row 1 of gamma is unused by this cell
        assert_close(got, ref, tol, f"{cell} d{k}")


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("path", golden_files(), ids=os.path.basename)
def test_against_reference_fixture(path, transposed):
    cell, dims, zo, d, ref_out, ref_grads = load_golden(path, torch.float64)
    out, grads = run_cuda(cell, d, zoneout=zo, dtype=torch.float32, transposed=transposed)
    _compare(cell, d, out, grads, ref_out, ref_grads, TOL_F32)


@pytest.mark.parametrize("path", golden_files(), ids=os.path.basename)
def test_inference_against_reference_fixture(path):
    cell, dims, zo, d, ref_out, _ = load_golden(path, torch.float64)
    out, _ = run_cuda(cell, d, zoneout=zo, training=False, backward=False)
    assert_close(out["h"], ref_out["h_inference"], TOL_F32, f"{cell} inference h")


# (T, N, C, H): ragged and tile-unfriendly shapes as well as aligned ones
SHAPES = [(9, 1, 5, 7), (6, 3, 16, 24), (12, 17, 33, 40), (16, 32, 64, 64), (10, 64, 128, 128)]


@pytest.mark.parametrize("zoneout", [0.0, 0.25])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "T%d_N%d_C%d_H%d" % s)
@pytest.mark.parametrize("cell", CELLS)
def test_fp32_against_oracle(cell, shape, zoneout):
    T, N, C, H = shape
    d = oracle.make_inputs(cell, T, N, C, H, seed=T * 1000 + H, zoneout=zoneout)
    ref_out, ref_grads = oracle.forward_backward(cell, d, zoneout=zoneout)
    out, grads = run_cuda(cell, d, zoneout=zoneout, dtype=torch.float32)
    _compare(cell, d, out, grads, ref_out, ref_grads, TOL_F32)


@pytest.mark.parametrize("shape", [(6, 3, 16, 24), (16, 32, 64, 64)],
                         ids=lambda s: "T%d_N%d_C%d_H%d" % s)
@pytest.mark.parametrize("cell", CELLS)
def test_bf16_against_oracle(cell, shape):
    T, N, C, H = shape
    zoneout = 0.25
    d = oracle.make_inputs(cell, T, N, C, H, seed=77 + H, zoneout=zoneout)
    # the oracle sees the bf16-rounded inputs, so only arithmetic differences remain
    dq = {k: (v.to(torch.bfloat16).to(torch.float64) if v is not None else None)
          for k, v in d.items()}
    ref_out, ref_grads = oracle.forward_backward(cell, dq, zoneout=zoneout)
    out, grads = run_cuda(cell, dq, zoneout=zoneout, dtype=torch.bfloat16)
    _compare(cell, dq, out, grads, ref_out, ref_grads, TOL_BF16)


@pytest.mark.parametrize("shape", [(6, 3, 16, 24), (16, 32, 64, 64), (20, 64, 64, 512)],
                         ids=lambda s: "T%d_N%d_C%d_H%d" % s)
def test_layer_norm_lstm_all_bf16_storage_mode(shape):
    """The C ABI's HASTE_B200_BF16 mode of LayerNormLSTM (every buffer bf16, what a C++ caller
    with __nv_bfloat16 buffers gets): held to the bar that the rounding of those interface
    buffers alone allows."""
    T, N, C, H = shape
    d = oracle.make_inputs("layer_norm_lstm", T, N, C, H, seed=77 + H, zoneout=0.25)
    dq = {k: (v.to(torch.bfloat16).to(torch.float64) if v is not None else None)
          for k, v in d.items()}
    ref_out, ref_grads = oracle.forward_backward("layer_norm_lstm", dq, zoneout=0.25)
    out, grads = run_cuda("layer_norm_lstm", dq, zoneout=0.25, dtype=torch.bfloat16,
                          fwd_kwargs={"saved_dtype": torch.bfloat16})
    _compare("layer_norm_lstm", dq, out, grads, ref_out, ref_grads, TOL_BF16_ALL_STORAGE_LN_LSTM)


@pytest.mark.parametrize("cell", CELLS)
def test_repeated_runs_are_bit_identical(cell):
    d = oracle.make_inputs(cell, 8, 5, 12, 16, seed=5, zoneout=0.3)
    runs = [run_cuda(cell, d, zoneout=0.3) for _ in range(3)]
    for out, grads in runs[1:]:
        assert torch.equal(out["h"], runs[0][0]["h"])
        for k in grads:
            assert torch.equal(grads[k], runs[0][1][k]), k


def test_long_sequence_stays_within_tolerance():
    # error must not build up over a long recurrence
    for cell in ["lstm", "gru"]:
        d = oracle.make_inputs(cell, 300, 8, 32, 64, seed=9)
        ref_out, ref_grads = oracle.forward_backward(cell, d)
        out, grads = run_cuda(cell, d)
        _compare(cell, d, out, grads, ref_out, ref_grads, TOL_F32)


def test_zero_steps_and_error_reporting():
    from haste_b200 import _C, ops
    x = torch.zeros(0, 2, 3, device="cuda")
    h0 = torch.zeros(2, 4, device="cuda")
    W = torch.zeros(3, 16, device="cuda")
    R = torch.zeros(4, 16, device="cuda")
    b = torch.zeros(16, device="cuda")
    h, c, _ = ops.lstm_forward(True, 0.0, x, h0, h0, W, R, b, torch.empty(0, 0, 0, device="cuda"))
    assert h.shape == (1, 2, 4) and torch.equal(h[0], h0)
    with pytest.raises(RuntimeError):
        ops.lstm_forward(True, 0.0, x.cpu(), h0, h0, W, R, b, torch.empty(0, 0, 0, device="cuda"))
    with pytest.raises(TypeError):
        ops.lstm_forward(True, 0.0, x.double(), h0.double(), h0.double(), W.double(), R.double(),
                         b.double(), torch.empty(0, 0, 0, device="cuda").double())
    assert _C.launch_count() >= 0


# shapes that exercise several hidden slices, several batch slices and multi-tile CTAs
REC_SHAPES = [(12, 40, 32, 80), (20, 64, 64, 512), (6, 130, 48, 512), (9, 3, 16, 200)]


@pytest.mark.parametrize("path", ["stepwise", "persistent"])
@pytest.mark.parametrize("shape", REC_SHAPES, ids=lambda s: "T%d_N%d_C%d_H%d" % s)
@pytest.mark.parametrize("cell", ["lstm", "gru", "layer_norm_lstm", "layer_norm_gru"])
def test_both_recurrence_paths_fp32(cell, shape, path):
    from haste_b200 import _C
    T, N, C, H = shape
    d = oracle.make_inputs(cell, T, N, C, H, seed=T + H, zoneout=0.2)
    ref_out, ref_grads = oracle.forward_backward(cell, d, zoneout=0.2)
    _C.set_recurrence_path(_C.PATH_STEPWISE if path == "stepwise" else _C.PATH_AUTO)
    try:
        n0 = _C.launch_count()
        out, grads = run_cuda(cell, d, zoneout=0.2)
        _C.sync_check(torch.cuda.current_stream().cuda_stream)
        launches = _C.launch_count() - n0
    finally:
        _C.set_recurrence_path(_C.PATH_AUTO)
    _compare(cell, d, out, grads, ref_out, ref_grads, TOL_F32)
    if path == "persistent":
        # a fixed number of launches per pass, none per time step
        assert launches < 64, launches
    else:
        assert launches >= 4 * T


@pytest.mark.parametrize("shape", [(20, 64, 64, 512), (8, 128, 64, 1024)],
                         ids=lambda s: "T%d_N%d_C%d_H%d" % s)
@pytest.mark.parametrize("cell", ["lstm", "gru", "layer_norm_lstm", "layer_norm_gru"])
def test_persistent_path_bf16(cell, shape):
    from haste_b200 import _C
    T, N, C, H = shape
    d = oracle.make_inputs(cell, T, N, C, H, seed=H, zoneout=0.1)
    dq = {k: (v.to(torch.bfloat16).to(torch.float64) if v is not None else None)
          for k, v in d.items()}
    ref_out, ref_grads = oracle.forward_backward(cell, dq, zoneout=0.1)
    out, grads = run_cuda(cell, dq, zoneout=0.1, dtype=torch.bfloat16)
    _C.sync_check(torch.cuda.current_stream().cuda_stream)
    _compare(cell, dq, out, grads, ref_out, ref_grads, TOL_BF16)


# large bf16 batches can take the tensor-core recurrence (tcgen05 step product, TMA-streamed
# h / dq): 64-row and 128-row tiles, one and two tiles per CTA, ragged last tiles, several row
# groups; with and without the SM budget that makes two directions co-resident.  The forward
# pass takes it by itself; the backward pass when a budget is set or the persistent path is
# requested.
TC_SHAPES = [(20, 128, 64, 1024, 0), (20, 256, 48, 512, 0), (20, 200, 32, 256, 0),
             (16, 700, 32, 512, 0), (16, 512, 64, 1024, 0), (24, 96, 16, 64, 0),
             (12, 128, 64, 1024, 74), (12, 256, 32, 1024, 74), (10, 300, 32, 512, 74)]


@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("shape", TC_SHAPES, ids=lambda s: "T%d_N%d_C%d_H%d_sms%d" % s)
def test_gru_tensor_core_recurrence_bf16(shape, transposed):
    from haste_b200 import _C
    T, N, C, H, budget = shape
    d = oracle.make_inputs("gru", T, N, C, H, seed=N + H, zoneout=0.1)
    dq = {k: (v.to(torch.bfloat16).to(torch.float64) if v is not None else None)
          for k, v in d.items()}
    ref_out, ref_grads = oracle.forward_backward("gru", dq, zoneout=0.1)
    _C.set_sm_budget(budget)
    _C.set_recurrence_path(_C.PATH_PERSISTENT)
    try:
        n0 = _C.launch_count()
        out, grads = run_cuda("gru", dq, zoneout=0.1, dtype=torch.bfloat16, transposed=transposed)
        _C.sync_check(torch.cuda.current_stream().cuda_stream)
        assert _C.launch_count() - n0 < 48  # one launch per pass, nothing per time step
        _compare("gru", dq, out, grads, ref_out, ref_grads, TOL_BF16)
        # inference (no gate cache, expectation form of zoneout)
        ref_inf = oracle.forward("gru", dq, training=False, zoneout=0.1)[0]
        out_inf, _ = run_cuda("gru", dq, zoneout=0.1, dtype=torch.bfloat16, training=False,
                              backward=False)
        assert_close(out_inf["h"], ref_inf, TOL_BF16, "inference h")
    finally:
        _C.set_sm_budget(0)
        _C.set_recurrence_path(_C.PATH_AUTO)


@pytest.mark.parametrize("path", ["stepwise", "persistent"])
@pytest.mark.parametrize("shape", [(6, 3, 16, 24), (16, 32, 64, 64), (20, 64, 64, 512), (6, 130, 48, 512)],
                         ids=lambda s: "T%d_N%d_C%d_H%d" % s)
def test_gru_float16_against_oracle(shape, path):
    """The reference's one reduced-precision type (half GRU): __half storage, oracle on the
    fp16-rounded inputs."""
    from haste_b200 import _C
    T, N, C, H = shape
    zoneout = 0.2
    d = oracle.make_inputs("gru", T, N, C, H, seed=31 + H, zoneout=zoneout)
    dq = {k: (v.to(torch.float16).to(torch.float64) if v is not None else None)
          for k, v in d.items()}
    ref_out, ref_grads = oracle.forward_backward("gru", dq, zoneout=zoneout)
    _C.set_recurrence_path(_C.PATH_STEPWISE if path == "stepwise" else _C.PATH_AUTO)
    try:
        out, grads = run_cuda("gru", dq, zoneout=zoneout, dtype=torch.float16)
        _C.sync_check(torch.cuda.current_stream().cuda_stream)
    finally:
        _C.set_recurrence_path(_C.PATH_AUTO)
    _compare("gru", dq, out, grads, ref_out, ref_grads, TOL_F16)


def test_float16_is_rejected_outside_the_gru():
    from haste_b200 import ops
    h = torch.zeros(2, 4, device="cuda", dtype=torch.float16)
    x = torch.zeros(3, 2, 3, device="cuda", dtype=torch.float16)
    W = torch.zeros(3, 16, device="cuda", dtype=torch.float16)
    R = torch.zeros(4, 16, device="cuda", dtype=torch.float16)
    b = torch.zeros(16, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError):
        ops.lstm_forward(True, 0.0, x, h, h, W, R, b, torch.empty(0, 0, 0, device="cuda", dtype=torch.float16))


@pytest.mark.parametrize("cell", ["lstm", "gru", "layer_norm_lstm", "layer_norm_gru"])
def test_hidden_size_beyond_the_persistent_kernels_falls_back_and_stays_correct(cell):
    """fp32 H > 512 does not fit the register-resident recurrence; the step-wise path takes
    over without the caller noticing anything but the launch count."""
    from haste_b200 import _C
    T, N, C, H = 5, 6, 24, 640
    d = oracle.make_inputs(cell, T, N, C, H, seed=H, zoneout=0.1)
    ref_out, ref_grads = oracle.forward_backward(cell, d, zoneout=0.1)
    n0 = _C.launch_count()
    out, grads = run_cuda(cell, d, zoneout=0.1)
    _C.sync_check(torch.cuda.current_stream().cuda_stream)
    assert _C.launch_count() - n0 >= 4 * T
    _compare(cell, d, out, grads, ref_out, ref_grads, TOL_F32)


def test_sequence_too_long_for_32_bit_row_index_is_rejected():
    from haste_b200 import _C
    # T*N >= 2^31 rows: rejected before anything is launched (pointers are never touched)
    with pytest.raises(RuntimeError):
        _C.call("haste_b200_lstm_forward", _C.F32, 1, 1 << 20, 1 << 11, 8, 8, 1, 1, 1, 1, 1, 1, 1,
                1, 0.0, None, None)

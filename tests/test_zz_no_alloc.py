"""LayerNorm backward without allocation (haste_b200_layer_norm_backward_noalloc).

Some callers of this library cannot allocate device memory when they call it: their own
arena owns the whole GPU, or they sit inside a stream-capture region, or they cannot take the
device-wide stall of a cudaMalloc.  The no-alloc entry point keeps its scratch in a fixed
array inside the library.  This test calls it through the C ABI twice in a row (the second
call reuses the array with whatever the first one left in it, and uses a different shape) and
requires bit-identical results to the ordinary entry point (both run the same three kernels),
the CPU oracle's LayerNorm gradient within the fp32 bar, and an unchanged amount of free
device memory across the second call.  It is collected last on purpose and must also pass
when run alone in a fresh process."""
import pytest
import torch

import haste_oracle as oracle
from helpers import TOL_F32, assert_close

pytestmark = pytest.mark.gpu


def _run(entry, rows, width, seed, with_beta):
    from haste_b200 import _C
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, width, generator=g, device="cuda") * 1.5 + 0.3
    gamma = 1 + 0.1 * torch.randn(width, generator=g, device="cuda")
    dy = torch.randn(rows, width, generator=g, device="cuda")
    y = torch.empty_like(x)
    cache = torch.empty(rows, 2, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    _C.call("haste_b200_layer_norm_forward", _C.F32, rows, width, gamma.data_ptr(), None,
            x.data_ptr(), y.data_ptr(), cache.data_ptr(), s)
    dx = torch.empty_like(x)
    dgamma = torch.zeros(width, device="cuda")
    dbeta = torch.zeros(width, device="cuda") if with_beta else None
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    _C.call(entry, _C.F32, rows, width, gamma.data_ptr(), x.data_ptr(), dy.data_ptr(),
            dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr() if with_beta else None,
            cache.data_ptr(), s)
    torch.cuda.synchronize()
    free_after = torch.cuda.mem_get_info()[0]
    # the oracle's gradient of the same LayerNorm (float64 autograd on the CPU)
    xl = x.double().cpu().requires_grad_(True)
    gl = gamma.double().cpu().requires_grad_(True)
    bl = torch.zeros(width, dtype=torch.float64, requires_grad=True) if with_beta else None
    yl = oracle.layer_norm(xl, gl, bl)
    ref = torch.autograd.grad((yl * dy.double().cpu()).sum(), [xl, gl] + ([bl] if with_beta else []))
    return (dx, dgamma, dbeta), ref, free_before - free_after


def test_noalloc_matches_ordinary_entry_point_twice_in_a_row():
    # the first call on the device looks the array's address up (and loads the module if
    # nothing else did); the second call is the one that must not move free memory at all
    for i, (rows, width, seed, with_beta) in enumerate([(300, 2048, 1, True), (77, 513, 2, False)]):
        want, _, _ = _run("haste_b200_layer_norm_backward", rows, width, seed, with_beta)
        got, ref, used = _run("haste_b200_layer_norm_backward_noalloc", rows, width, seed, with_beta)
        assert torch.equal(got[0], want[0]), "dx differs from the ordinary entry point"
        assert torch.equal(got[1], want[1]), "dgamma differs from the ordinary entry point"
        assert_close(got[0], ref[0], TOL_F32, "dx vs oracle")
        assert_close(got[1], ref[1], TOL_F32, "dgamma vs oracle")
        if with_beta:
            assert torch.equal(got[2], want[2]), "dbeta differs from the ordinary entry point"
            assert_close(got[2], ref[2], TOL_F32, "dbeta vs oracle")
        if i == 1:
            assert used == 0, f"free device memory moved by {used} bytes across the call"


def test_noalloc_rejects_widths_beyond_the_built_in_scratch():
    from haste_b200 import _C
    t = torch.zeros(4, 5000, device="cuda")
    v = torch.zeros(5000, device="cuda")
    c = torch.zeros(4, 2, device="cuda")
    with pytest.raises(_C.HasteError, match="exceeds the built-in scratch"):
        _C.call("haste_b200_layer_norm_backward_noalloc", _C.F32, 4, 5000, v.data_ptr(),
                t.data_ptr(), t.data_ptr(), t.data_ptr(), v.data_ptr(), None, c.data_ptr(), None)

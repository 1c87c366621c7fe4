"""GPU tests of the building blocks: contraction, LayerNorm, and the module API."""
import pytest
import torch

import haste_oracle as oracle
from helpers import TOL_BF16, TOL_F32, assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (7, 5, 3), (64, 64, 64), (130, 70, 257),
                                   (256, 512, 128), (512, 2048, 1024), (1000, 96, 40)])
@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_gemm_all_layouts(M, N, K, ta, tb, dtype):
    from haste_b200 import ops
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N)
    a = torch.randn((K, M) if ta else (M, K), generator=g, device="cuda").to(dtype)
    b = torch.randn((N, K) if tb else (K, N), generator=g, device="cuda").to(dtype)
    av = a.t() if ta else a
    bv = b.t() if tb else b
    want = av.double() @ bv.double()
    # float16 operands are used exactly (two bf16 planes); only the fp16 result is rounded
    tol = {torch.float32: TOL_F32, torch.bfloat16: TOL_BF16, torch.float16: 2e-3}[dtype]
    got = ops.gemm(av, bv)
    assert_close(got, want, tol, "gemm")
    c0 = torch.randn(M, N, generator=g, device="cuda").to(dtype)
    got = ops.gemm(av, bv, out=c0.clone(), accumulate=True)
    assert_close(got, want + c0.double(), tol, "gemm accumulate")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("M,N,K,ta,tb", [(256, 256, 64, False, False), (700, 520, 200, False, True),
                                         (1000, 456, 200, True, False), (2048, 1024, 4096, False, False),
                                         (512, 2048, 16384, True, False), (1024, 3072, 1024, False, False),
                                         (4000, 264, 520, True, True)])
def test_gemm_pair_and_single_cta_kernels(M, N, K, ta, tb, dtype):
    """Outputs of at least 192 x 192 take the CTA-pair kernel (256 x 256 tiles, cta_group::2);
    HASTE_B200_GEMM_TCGEN05_SINGLE keeps the single-CTA kernel.  Both against float64, ragged
    edges, every operand layout, long K (split along K) and many tiles per pair included."""
    from haste_b200 import _C, ops
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn((K, M) if ta else (M, K), generator=g, device="cuda").to(dtype)
    b = torch.randn((N, K) if tb else (K, N), generator=g, device="cuda").to(dtype)
    av = a.t() if ta else a
    bv = b.t() if tb else b
    want = av.double() @ bv.double()
    tol = TOL_F32 if dtype == torch.float32 else TOL_BF16
    try:
        for path in (_C.GEMM_AUTO, _C.GEMM_TCGEN05_SINGLE):
            _C.set_gemm_path(path)
            n0 = _C.launch_count()
            got = ops.gemm(av, bv)
            torch.cuda.synchronize()
            _C.sync_check(torch.cuda.current_stream().cuda_stream)
            assert _C.launch_count() > n0
            assert_close(got, want, tol, f"gemm path {path}")
            c0 = torch.randn(M, N, generator=g, device="cuda").to(dtype)
            got = ops.gemm(av, bv, out=c0.clone(), accumulate=True)
            assert_close(got, want + c0.double(), tol, f"gemm accumulate path {path}")
    finally:
        _C.set_gemm_path(_C.GEMM_AUTO)


@pytest.mark.parametrize("rows,width", [(1, 1), (5, 7), (33, 96), (256, 2048), (100, 1536)])
@pytest.mark.parametrize("with_beta", [False, True])
def test_layer_norm_forward_backward(rows, width, with_beta):
    from haste_b200 import _C
    g = torch.Generator().manual_seed(rows + width)
    x = torch.randn(rows, width, generator=g, dtype=torch.float64) * 2 + 0.5
    gamma = 1 + 0.1 * torch.randn(width, generator=g, dtype=torch.float64)
    beta = 0.1 * torch.randn(width, generator=g, dtype=torch.float64) if with_beta else None
    dy = torch.randn(rows, width, generator=g, dtype=torch.float64)
    xl, gl = x.clone().requires_grad_(True), gamma.clone().requires_grad_(True)
    bl = beta.clone().requires_grad_(True) if with_beta else None
    y = oracle.layer_norm(xl, gl, bl)
    grads = torch.autograd.grad((y * dy).sum(), [xl, gl] + ([bl] if with_beta else []))

    cu = lambda t: t.float().cuda().contiguous()
    xc, gc, dyc = cu(x), cu(gamma), cu(dy)
    bc = cu(beta) if with_beta else None
    yc = torch.empty_like(xc)
    cache = torch.empty(rows, 2, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    _C.call("haste_b200_layer_norm_forward", _C.F32, rows, width, gc.data_ptr(),
            bc.data_ptr() if with_beta else None, xc.data_ptr(), yc.data_ptr(), cache.data_ptr(), s)
    assert_close(yc, y, TOL_F32, "ln y")
    dg = torch.zeros(width, device="cuda")
    db = torch.zeros(width, device="cuda") if with_beta else None
    dx = dyc.clone()  # in place: dx aliases dy
    _C.call("haste_b200_layer_norm_backward", _C.F32, rows, width, gc.data_ptr(), xc.data_ptr(),
            dx.data_ptr(), dx.data_ptr(), dg.data_ptr(), db.data_ptr() if with_beta else None,
            cache.data_ptr(), s)
    assert_close(dx, grads[0], TOL_F32, "ln dx")
    assert_close(dg, grads[1], TOL_F32, "ln dgamma")
    if with_beta:
        assert_close(db, grads[2], TOL_F32, "ln dbeta")


def _copy_params(layer, d, cell):
    names = {"W": "kernel", "R": "recurrent_kernel", "b": "bias", "bx": "bias",
             "br": "recurrent_bias", "u": "recurrent_scale", "gamma": "gamma",
             "gamma_h": "gamma_h", "beta_h": "beta_h"}
    with torch.no_grad():
        for k, attr in names.items():
            if k in d and hasattr(layer, attr):
                getattr(layer, attr).copy_(d[k].float())


@pytest.mark.parametrize("cell,cls", [("lstm", "LSTM"), ("gru", "GRU"), ("indrnn", "IndRNN"),
                                      ("layer_norm_lstm", "LayerNormLSTM"),
                                      ("layer_norm_gru", "LayerNormGRU"),
                                      ("layer_norm_indrnn", "LayerNormIndRNN")])
def test_module_matches_oracle_with_explicit_masks(cell, cls):
    import haste_b200 as haste
    T, N, C, H = 7, 4, 6, 8
    zo, dc = 0.3, 0.2
    d = oracle.make_inputs(cell, T, N, C, H, seed=3, zoneout=zo)
    kw = dict(zoneout=zo)
    has_R = "indrnn" not in cell
    if has_R:
        kw["dropout"] = dc
    layer = getattr(haste, cls)(C, H, **kw).cuda()
    _copy_params(layer, d, cell)
    layer.train()
    g = torch.Generator().manual_seed(11)
    call_kw = {"zoneout_mask": d["mask"].float().cuda()}
    dq = dict(d)
    if has_R:
        keep = torch.bernoulli(torch.full(d["R"].shape, 1 - dc, dtype=torch.float64), generator=g)
        call_kw["dropconnect_mask"] = keep.cuda()
        dq["R"] = (d["R"] * keep / (1 - dc))
    x = d["x"].float().cuda().requires_grad_(True)
    h0 = d["h0"].float().cuda()[None]
    state = (h0, d["c0"].float().cuda()[None]) if "lstm" in cell else h0
    y, st = layer(x, state, **call_kw)
    (y * d["dh"][1:].float().cuda()).sum().backward()
    # oracle with the effective (masked, rescaled) recurrent matrix and no cell-state grads
    dq["dc"] = torch.zeros_like(d["dh"])
    ref_out, ref_g = oracle.forward_backward(cell, dq, zoneout=zo)
    assert_close(y, ref_out["h"][1:], TOL_F32, "module y")
    hn = st[0] if isinstance(st, tuple) else st
    assert_close(hn[0], ref_out["h"][-1], TOL_F32, "module h_n")
    assert_close(x.grad, ref_g["x"], TOL_F32, "module dx")
    assert_close(layer.kernel.grad, ref_g["W"], TOL_F32, "module dW")
    if has_R:
        # autograd routes dR through the DropConnect mask
        assert_close(layer.recurrent_kernel.grad, ref_g["R"] * keep / (1 - dc), TOL_F32, "module dR")
    # eval mode must refuse backward and use the expectation form of zoneout
    layer.eval()
    y2, _ = layer(x.detach(), state)
    with torch.no_grad():
        dq2 = dict(d)
        h_inf = oracle.forward(cell, dq2, training=False, zoneout=zo)[0]
    assert_close(y2, h_inf[1:], TOL_F32, "module eval y")


def test_lstm_and_gru_match_torch_nn_through_native_weights():
    import haste_b200 as haste
    T, N, C, H = 11, 5, 12, 16
    torch.manual_seed(0)
    x = torch.randn(T, N, C, device="cuda")
    for ours, theirs in [(haste.LSTM(C, H), torch.nn.LSTM(C, H)), (haste.GRU(C, H), torch.nn.GRU(C, H))]:
        ours, theirs = ours.cuda(), theirs.cuda()
        ours.from_native_weights(theirs.weight_ih_l0, theirs.weight_hh_l0, theirs.bias_ih_l0,
                                 theirs.bias_hh_l0)
        y1, _ = ours(x)
        # torch.nn on CPU in float64: the cuDNN path may use TF32 and is itself only
        # ~3e-4 accurate
        y2, _ = theirs.double().cpu()(x.double().cpu())
        theirs.float().cuda()
        assert_close(y1, y2, TOL_F32, type(ours).__name__ + " vs torch.nn")
        w = ours.to_native_weights()
        assert_close(w[0], theirs.weight_ih_l0, 1e-6, "round trip")


def test_state_validation_and_options():
    import haste_b200 as haste
    layer = haste.GRU(4, 6, batch_first=True, return_state_sequence=True).cuda()
    x = torch.randn(3, 5, 4, device="cuda")  # [N,T,C]
    y, st = layer(x)
    assert y.shape == (3, 5, 6) and st.shape == (1, 3, 5, 6)
    with pytest.raises(ValueError):
        layer(x, torch.zeros(1, 2, 6, device="cuda"))
    with pytest.raises(ValueError):
        haste.LSTM(4, 6, zoneout=1.5)
    layer2 = haste.LSTM(4, 6).cuda()
    xt = torch.randn(5, 3, 4, device="cuda")
    lengths = torch.tensor([5, 2, 4], device="cuda")
    y, (hn, cn) = layer2(xt, lengths=lengths)
    for n, L in enumerate([5, 2, 4]):
        assert torch.equal(hn[0, n], y[L - 1, n])
    with pytest.raises(RuntimeError):
        haste.LSTM(4, 6)(xt.cpu())


def test_bidirectional_stack_matches_oracle_composition():
    import haste_b200 as haste
    T, N, C, H = 6, 3, 5, 8
    net = haste.Stack(haste.LayerNormLSTM, C, H, num_layers=2, bidirectional=True).cuda()
    torch.manual_seed(4)
    with torch.no_grad():
        for p in net.parameters():
            p.add_(0.05 * torch.randn_like(p))
    x = torch.randn(T, N, C, device="cuda", requires_grad=True)
    y = net(x)
    dy = torch.randn_like(y)
    (y * dy).sum().backward()

    # the same network from oracle layers: flip / run / flip back, concat features
    xo = x.detach().double().cpu().requires_grad_(True)
    inp = xo
    leaves = []
    for level in net.layers:
        outs = []
        for d_, layer in enumerate(level):
            p = {k: v.detach().double().cpu().requires_grad_(True) for k, v in layer.named_parameters()}
            leaves.append(p)
            xi = torch.flip(inp, [0]) if d_ == 1 else inp
            z = torch.zeros(N, H, dtype=torch.float64)
            h, _ = oracle.layer_norm_lstm(True, 0.0, xi, z, z, p["kernel"], p["recurrent_kernel"],
                                          p["bias"], p["gamma"], p["gamma_h"], p["beta_h"])
            yo = h[1:]
            outs.append(torch.flip(yo, [0]) if d_ == 1 else yo)
        inp = torch.cat(outs, -1)
    (inp * dy.double().cpu()).sum().backward()
    assert_close(y, inp, TOL_F32, "stack y")
    assert_close(x.grad, xo.grad, TOL_F32, "stack dx")
    i = 0
    for level in net.layers:
        for layer in level:
            for k, v in layer.named_parameters():
                assert_close(v.grad, leaves[i][k].grad, TOL_F32, f"stack d{k}")
            i += 1


def test_streamed_host_input_equals_single_call():
    from haste_b200 import ops
    T, N, C, H = 37, 16, 32, 64
    d = oracle.make_inputs("lstm", T, N, C, H, seed=8, zoneout=0.2)
    cu = lambda t: t.float().cuda().contiguous()
    args = [cu(d[k]) for k in ("h0", "c0", "W", "R", "b", "mask")]
    want = ops.lstm_forward(True, 0.2, cu(d["x"]), *args)
    x_host = d["x"].float().pin_memory()
    for chunks in (1, 3, 5):
        got = ops.lstm_forward_from_host(True, 0.2, x_host, *args, chunks=chunks)
        torch.cuda.synchronize()
        # pieces may take a different contraction path than the whole (by size), so the
        # match is to rounding, not bit-for-bit
        for a, b in zip(got[:3], want):
            assert_close(a, b, 2e-5, "streamed vs single call")
        assert torch.equal(got[3], cu(d["x"]))


def test_streamed_host_gradient_equals_single_call():
    """The backward pass fed with an incoming gradient in pinned host memory (copied and
    consumed in pieces, latest first) equals one call on the whole sequence."""
    from haste_b200 import ops
    T, N, C, H = 37, 16, 32, 64
    d = oracle.make_inputs("lstm", T, N, C, H, seed=9, zoneout=0.2)
    cu = lambda t: t.float().cuda().contiguous()
    x, mask = cu(d["x"]), cu(d["mask"])
    W, R, b = cu(d["W"]), cu(d["R"]), cu(d["b"])
    dh_new, dc_new = cu(d["dh"]), cu(d["dc"])
    dh_host = d["dh"].float().pin_memory()

    def forward():
        return ops.lstm_forward(True, 0.2, x, cu(d["h0"]), cu(d["c0"]), W, R, b, mask)

    h, c, cache = forward()
    want = ops.lstm_backward(x, W, R, b, mask, h, c, cache, dh_new, dc_new, transposed=False)
    for chunks in (1, 3, 4, 4):  # the repeated count reuses the staged device buffer
        h, c, cache = forward()  # the backward pass overwrites the cache
        got = ops.lstm_backward_from_host(x, W, R, b, mask, h, c, cache, dh_host, dc_new,
                                          chunks=chunks)
        torch.cuda.synchronize()
        for a, e, name in zip(got, want, ["dx", "dh", "dc", "dW", "dR", "db"]):
            assert_close(a, e, 2e-5, f"streamed {name} ({chunks} pieces)")


@pytest.mark.parametrize("cell", ["lstm", "gru", "indrnn", "layer_norm_lstm", "layer_norm_gru",
                                  "layer_norm_indrnn"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parameter_gradients_written_into_a_bucket(cell, dtype):
    """With `grads=bucket` the backward op's parameter gradients are views of the caller's
    flat buffer (what the gradient all-reduce then sums) and equal the separately allocated
    ones bit for bit."""
    from haste_b200.data_parallel import GradientBucket
    from helpers import run_cuda
    T, N, C, H = 9, 32, 24, 64
    d = oracle.make_inputs(cell, T, N, C, H, seed=21, zoneout=0.1)
    _, want = run_cuda(cell, d, zoneout=0.1, dtype=dtype)
    bucket = GradientBucket.for_cell(cell, C, H, dtype, "cuda")
    for _ in range(2):  # the second pass reuses the buffer
        bucket.reset()
        _, got = run_cuda(cell, d, zoneout=0.1, dtype=dtype, grads=bucket)
        lo = bucket.flat.data_ptr()
        hi = lo + bucket.flat.numel() * bucket.flat.element_size()
        for k, v in got.items():
            assert torch.equal(v, want[k]), k
            if k not in ("x", "h0", "c0"):
                assert lo <= v.data_ptr() < hi and v.data_ptr() % 16 == 0, k

"""The benchmark configurations at their stated composition, against the CPU oracle.

  * 3-layer bidirectional LayerNormLSTM, C=80, H=512, N=64, zoneout 0.1 and DropConnect 0.05
    with masks drawn per layer and direction from torch.Generator(1234 + layer*2 + dir) and
    passed explicitly; fp32 and bf16 (2e-2); T=50 (outputs and all gradients) and the full
    T=400 (outputs; gradients through linearity) against the float64 oracle.  This stack amplifies float32 rounding (the reference's own float32 path is
    3e-4 .. 4e-4 from the float64 result), so the fp32 bar per tensor is 1e-4 plus twice the
    distance of the reference's float32 path from the float64 result.
  * 6-layer IndRNN and LayerNormIndRNN, C=H=1024, N=128, u ~ U(0,1), zoneout 0.1: T=200
    against the float64 oracle, and at the full T=2000 the properties that need no oracle
    (causality of a prefix, linearity of the backward pass).
  * 4-layer bidirectional GRU in bf16, C=512, H=1024, N=128, T=50, oracle on the bf16-rounded
    tensors.
  * The batch-sharded data-parallel step: the gradients of the shards, written into the
    per-layer buckets and summed, equal the gradients of the whole batch.

Outputs, the input gradient and every parameter gradient of every layer and direction are
compared (`helpers.compare_stack`).
"""
import pytest
import torch

from helpers import (TOL_BF16, TOL_F32, assert_close, compare_stack, oracle_stack,
                     oracle_stack_forward, seeded_masks)

pytestmark = pytest.mark.gpu


def _to_device(masks, dtype):
    return [[{k: v.to("cuda", dtype) for k, v in m.items()} for m in level] for level in masks]


def _perturb(net, seed, scale=0.05):
    """Moves every parameter off its initial value (gains off 1, biases off 0) so that each
    gradient path carries signal."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in net.parameters():
            p.add_((scale * torch.randn(p.shape, generator=g)).to(p.device, p.dtype))


def _run_stack(net, x, dy, masks):
    for p in net.parameters():
        p.grad = None
    x = x.detach().clone().requires_grad_(True)
    y = net(x, masks=masks)
    (y * dy).sum().backward()
    torch.cuda.synchronize()
    from haste_b200 import _C
    _C.sync_check(torch.cuda.current_stream().cuda_stream)
    return y.detach(), x.grad


# ------------------------------------------------------------------ configuration 2
def _config2(T, dtype, seed=11):
    import haste_b200 as hb
    N, C, H = 64, 80, 512
    torch.manual_seed(seed)
    net = hb.Stack(hb.LayerNormLSTM, C, H, num_layers=3, bidirectional=True, zoneout=0.1,
                   dropout=0.05)
    _perturb(net, seed)
    net = net.cuda().to(dtype)
    net.train()
    g = torch.Generator().manual_seed(seed + 1)
    x = torch.randn(T, N, C, generator=g).to("cuda", dtype)
    dy = torch.randn(T, N, 2 * H, generator=g).to("cuda", dtype)
    masks = seeded_masks(3, 2, T, N, H, 4, zoneout=0.1, dropconnect=0.05)
    return net, x, dy, masks


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_F32), (torch.bfloat16, TOL_BF16)],
                         ids=["fp32", "bf16"])
def test_config2_three_layer_bidirectional_layer_norm_lstm_with_masks(dtype, tol):
    T = 50
    net, x, dy, masks = _config2(T, dtype)
    y, dx = _run_stack(net, x, dy, _to_device(masks, dtype))
    ref = oracle_stack(net, "layer_norm_lstm", x, dy, masks, dropconnect=0.05, zoneout=0.1,
                       bf16=dtype == torch.bfloat16)
    native = None
    if dtype == torch.float32:
        # three LayerNorms per step and six layer passes amplify float32 rounding: the
        # reference's own float32 path is 3e-4 .. 4e-4 from the float64 result here
        native = oracle_stack(net, "layer_norm_lstm", x, dy, masks, dropconnect=0.05, zoneout=0.1,
                              dtype=torch.float32)
    compare_stack(net, y, dx, ref, tol, "config 2 T=50", ref_native=native)


def test_config2_full_length_fp32():
    """All T=400 steps.  Over 400 steps of three normalised layers the gradients of this
    network grow by ten orders of magnitude and the reference's own float32 path is several
    hundred percent from the float64 result on them, so no gradient can be compared with an
    oracle at this length; the outputs can (with the float32-path rule), and the backward
    pass is checked through its linearity in the incoming gradient."""
    T = 400
    net, x, dy, masks = _config2(T, torch.float32, seed=12)
    dm = _to_device(masks, torch.float32)
    y, dx = _run_stack(net, x, dy, dm)
    grads = [p.grad.clone() for p in net.parameters()]
    import haste_oracle as oracle
    with torch.no_grad():
        ref = oracle_stack_forward(net, "layer_norm_lstm", x, masks, 0.05, 0.1, torch.float64)
        native = oracle_stack_forward(net, "layer_norm_lstm", x, masks, 0.05, 0.1, torch.float32)
    bar = TOL_F32 + 2.0 * oracle.max_rel_err(native, ref)
    assert_close(y, ref, bar, "config 2 T=400 y")
    assert torch.isfinite(dx).all()
    y2, dx2 = _run_stack(net, x, 2.0 * dy, dm)
    assert torch.equal(y2, y)
    assert_close(dx2, 2.0 * dx.double(), 2e-5, "linearity dx")
    for p, g0 in zip(net.parameters(), grads):
        assert_close(p.grad, 2.0 * g0.double(), 2e-5, "linearity of a parameter gradient")


# ------------------------------------------------------------------ configuration 3
def _config3(cls_name, T, seed=21):
    import haste_b200 as hb
    N, C, H = 128, 1024, 1024
    torch.manual_seed(seed)
    net = hb.Stack(getattr(hb, cls_name), C, H, num_layers=6, zoneout=0.1)
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for level in net.layers:
            level[0].recurrent_scale.copy_(torch.rand(H, generator=g))  # u ~ U(0,1)
    net = net.cuda()
    net.train()
    x = torch.randn(T, N, C, generator=g).cuda()
    dy = torch.randn(T, N, H, generator=g).cuda()
    masks = seeded_masks(6, 1, T, N, H, 1, zoneout=0.1, dropconnect=0.0)
    return net, x, dy, masks


@pytest.mark.parametrize("cls_name,cell", [("IndRNN", "indrnn"), ("LayerNormIndRNN", "layer_norm_indrnn")])
def test_config3_six_layer_indrnn(cls_name, cell):
    T = 200
    net, x, dy, masks = _config3(cls_name, T)
    y, dx = _run_stack(net, x, dy, _to_device(masks, torch.float32))
    ref = oracle_stack(net, cell, x, dy, masks, zoneout=0.1)
    compare_stack(net, y, dx, ref, TOL_F32, f"config 3 {cls_name} T=200")


@pytest.mark.parametrize("cls_name", ["IndRNN", "LayerNormIndRNN"])
def test_config3_full_length_properties(cls_name):
    T = 2000
    net, x, dy, masks = _config3(cls_name, T, seed=22)
    dm = _to_device(masks, torch.float32)
    y, dx = _run_stack(net, x, dy, dm)
    assert torch.isfinite(y).all() and torch.isfinite(dx).all()
    grads = [p.grad.clone() for p in net.parameters()]
    # causality: the first quarter of the sequence gives the first quarter of the outputs
    Tp = T // 4
    mp = [[{k: v[:Tp] for k, v in m.items()} for m in level] for level in dm]
    with torch.no_grad():
        yp = net(x[:Tp].contiguous(), masks=mp)
    assert_close(yp, y[:Tp], 1e-6, "prefix y")
    # the backward pass is linear in the incoming gradient
    y2, dx2 = _run_stack(net, x, 2.0 * dy, dm)
    assert torch.equal(y2, y)
    assert_close(dx2, 2.0 * dx.double(), 2e-5, "linearity dx")
    for p, g0 in zip(net.parameters(), grads):
        if p.grad is not None and g0.abs().max() > 0:
            assert_close(p.grad, 2.0 * g0.double(), 2e-5, "linearity of a parameter gradient")


# ------------------------------------------------------------------ configuration 4
def _config4(T, N, seed=31):
    import haste_b200 as hb
    C, H = 512, 1024
    torch.manual_seed(seed)
    net = hb.Stack(hb.GRU, C, H, num_layers=4, bidirectional=True)
    _perturb(net, seed, 0.02)
    net = net.cuda().to(torch.bfloat16)
    net.train()
    g = torch.Generator().manual_seed(seed + 1)
    x = torch.randn(T, N, C, generator=g).to("cuda", torch.bfloat16)
    dy = torch.randn(T, N, 2 * H, generator=g).to("cuda", torch.bfloat16)
    return net, x, dy


def test_config4_four_layer_bidirectional_gru_bf16():
    T, N = 50, 128
    net, x, dy = _config4(T, N)
    y, dx = _run_stack(net, x, dy, None)
    ref = oracle_stack(net, "gru", x, dy, None, bf16=True)
    compare_stack(net, y, dx, ref, TOL_BF16, "config 4 T=50")


def test_config4_sharded_batch_gradients_equal_whole_batch_gradients():
    """The data-parallel step on one device: every shard's backward pass writes into the
    per-layer gradient buckets (`data_parallel.attach`), the shard sums are what an all-reduce
    would give, and they equal the whole-batch gradients within the bf16 bar."""
    from haste_b200 import data_parallel
    T, N, world = 24, 128, 4
    net, x, dy = _config4(T, N, seed=41)
    _run_stack(net, x, dy, None)
    want = {k: v.grad.detach().float().clone() for k, v in net.named_parameters()}
    dp = data_parallel.attach(net)
    total = {k: torch.zeros_like(v) for k, v in want.items()}
    for rank in range(world):
        dp.zero_grad()
        xs = data_parallel.shard(x, rank, world).requires_grad_(True)
        ys = net(xs)
        (ys * data_parallel.shard(dy, rank, world)).sum().backward()
        dp.finish()
        lo = {h.bucket.flat.data_ptr() for h in dp.hooks}
        for k, v in net.named_parameters():
            total[k] += v.grad.float()
        # the gradients the layers hold ARE the buckets (no copy in between)
        for h in dp.hooks:
            assert h.layer.kernel.grad.data_ptr() in lo
    dp.detach()
    for k in want:
        assert_close(total[k], want[k], TOL_BF16, f"sharded d{k}")

"""Host-side logic of the multi-GPU path, run as two gloo ranks on CPU: batch sharding,
shared DropConnect masks, parameter broadcast and the bucketed gradient all-reduce.  The
per-rank computation is the CPU oracle (test infrastructure); what is under test is
haste_b200.data_parallel."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import haste_oracle as oracle

WORLD = 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, port, cell, results):
    from haste_b200 import data_parallel as dp
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        torch.set_num_threads(1)
        T, N, C, H = 5, 6, 4, 8
        d = oracle.make_inputs(cell, T, N, C, H, seed=5, zoneout=0.2)
        # the same DropConnect mask on every rank, from the seed alone
        keep = dp.dropconnect_mask(d["R"].shape, 0.25, seed=77, dtype=torch.float64)
        gathered = [torch.empty_like(keep) for _ in range(WORLD)]
        dist.all_gather(gathered, keep)
        assert all(torch.equal(g, keep) for g in gathered)
        d["R"] = d["R"] * keep / 0.75
        ref_out, ref_g = oracle.forward_backward(cell, d, zoneout=0.2)

        # rank-local shard of everything that carries a batch axis
        ds = dict(d)
        for k in ("x", "mask", "dh", "dc"):
            if d.get(k) is not None:
                ds[k] = dp.shard(d[k], rank, WORLD, batch_dim=1)
        for k in ("h0", "c0"):
            if k in d:
                ds[k] = dp.shard(d[k], rank, WORLD, batch_dim=0)
        out, g = oracle.forward_backward(cell, ds, zoneout=0.2)
        per = N // WORLD
        assert torch.allclose(out["h"], ref_out["h"][:, rank * per:(rank + 1) * per], atol=1e-12)

        # parameter gradients: summed over ranks in flat buckets; tiny buckets force several
        weights = [k for k in g if k not in ("x", "h0", "c0")]
        tensors = [g[k].clone() for k in weights]
        finish = dp.all_reduce_tensors(tensors, bucket_bytes=256, async_op=True)
        finish()
        for k, t in zip(weights, tensors):
            assert torch.allclose(t, ref_g[k], rtol=1e-10, atol=1e-12), k
        # per-sample gradients stay local and equal the matching slice
        assert torch.allclose(g["x"], ref_g["x"][:, rank * per:(rank + 1) * per], atol=1e-12)

        # module form: broadcast, then all_reduce_gradients on .grad
        lin = torch.nn.Linear(3, 2).double()
        with torch.no_grad():
            for p in lin.parameters():
                p.add_(rank + 1.0)
        dp.broadcast_parameters(lin, src=0)
        ref = [p.detach().clone() for p in lin.parameters()]
        gathered = [torch.empty_like(ref[0]) for _ in range(WORLD)]
        dist.all_gather(gathered, ref[0])
        assert torch.equal(gathered[0], gathered[1])
        for p in lin.parameters():
            p.grad = torch.full_like(p, float(rank + 1))
        dp.all_reduce_gradients(lin)
        for p in lin.parameters():
            assert torch.equal(p.grad, torch.full_like(p, 3.0))

        # gradient bucket: the outputs are views of one flat buffer, summed by one collective
        bucket = dp.GradientBucket.for_cell(cell, C, H, torch.float64, "cpu")
        for _ in range(2):  # a second step reuses the buffer after reset()
            bucket.reset()
            views = [bucket.take(*g[k].shape) for k in weights]
            base = bucket.flat.untyped_storage().data_ptr()
            for v, k in zip(views, weights):
                assert v.untyped_storage().data_ptr() == base and v.data_ptr() % 256 == base % 256
                assert not v.any()
                v.add_(g[k])  # what a backward op does: accumulate into its zeroed output
            work = bucket.all_reduce(async_op=True)
            work.wait()
            for v, k in zip(views, weights):
                assert torch.allclose(v, ref_g[k], rtol=1e-10, atol=1e-12), k
        with pytest.raises(ValueError):
            bucket.take(1 << 20)
        _check_attach(rank)
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


class GRU(torch.nn.Module):
    """Stand-in with the attributes `data_parallel.attach` uses of a haste_b200.GRU (the real
    layers need a GPU): its "backward pass" takes the gradient views from the bucket, adds a
    rank-dependent value and reports them ready, like the autograd glue does."""

    def __init__(self, C, H):
        super().__init__()
        self.input_size, self.hidden_size, self._dp = C, H, None
        self.kernel = torch.nn.Parameter(torch.zeros(C, 3 * H, dtype=torch.float64))
        self.recurrent_kernel = torch.nn.Parameter(torch.zeros(H, 3 * H, dtype=torch.float64))
        self.bias = torch.nn.Parameter(torch.zeros(3 * H, dtype=torch.float64))
        self.recurrent_bias = torch.nn.Parameter(torch.zeros(3 * H, dtype=torch.float64))

    def fake_backward(self, value, scale=None):
        names = ["kernel", "recurrent_kernel", "bias", "recurrent_bias"]
        views = {k: self._dp.bucket.take(*getattr(self, k).shape) for k in names}
        for v in views.values():
            v.add_(value)
        self._dp.recurrent_scale = scale
        self._dp.gradients_ready(views)


def _check_attach(rank):
    """attach(): buckets per layer, all-reduce issued from the backward pass (or in finish()),
    DropConnect scale applied after the sum, .grad aliases the bucket."""
    from haste_b200 import data_parallel as dp
    net = torch.nn.ModuleList([GRU(3, 4), GRU(8, 4)])
    for overlap in (True, False):
        d = dp.attach(net, overlap=overlap)
        assert len(d.hooks) == 2 and d.bucket_bytes() > 0
        for step in range(2):
            d.zero_grad()
            scale = torch.full((4, 12), 2.0, dtype=torch.float64)
            net[1].fake_backward(float(rank + 1) * 10)           # upper layer finishes first
            net[0].fake_backward(float(rank + 1), scale=scale)
            d.finish()
            assert torch.equal(net[1].kernel.grad, torch.full((8, 12), 30.0, dtype=torch.float64))
            assert torch.equal(net[0].bias.grad, torch.full((12,), 3.0, dtype=torch.float64))
            assert torch.equal(net[0].recurrent_kernel.grad, torch.full((4, 12), 6.0, dtype=torch.float64))
            assert net[1].kernel.grad.data_ptr() == net[1]._dp.bucket.flat.data_ptr()
        d.detach()
        assert net[0]._dp is None


@pytest.mark.parametrize("cell", ["lstm", "layer_norm_gru"])
def test_two_gloo_ranks_reproduce_the_single_process_gradients(cell):
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, port, cell, results)) for r in range(WORLD)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    for p in procs:
        if p.is_alive():
            p.terminate()
            pytest.fail("rank did not finish")
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert dict(results) == {0: "ok", 1: "ok"}


def _failing_rank_main(rank, port, results):
    """Rank 1 leaves between steps (it raises on the host before its all-reduce); rank 0's
    all-reduce then ends with an error inside the process group's short time-out instead of
    waiting for ever."""
    import datetime
    import time
    from haste_b200 import data_parallel as dp
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD,
                            timeout=datetime.timedelta(seconds=5))
    t = torch.ones(8, dtype=torch.float64) * (rank + 1)
    dp.all_reduce_tensors([t])  # a step both ranks complete
    assert torch.equal(t, torch.full((8,), 3.0, dtype=torch.float64))
    if rank == 1:
        results[1] = "left"
        os._exit(0)  # no collective in flight
    t0 = time.time()
    try:
        dp.all_reduce_tensors([t])
        results[0] = "no error"
    except Exception as e:  # gloo reports the lost peer or the time-out
        results[0] = f"error after {time.time() - t0:.1f}s: {type(e).__name__}"
    os._exit(0)  # the group is unusable; skip its destructor


def test_a_rank_that_leaves_ends_the_others_all_reduce_with_an_error():
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_failing_rank_main, args=(r, port, results)) for r in range(WORLD)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    for p in procs:
        if p.is_alive():
            p.terminate()
            pytest.fail("a rank hung on the lost peer")
    assert results.get(1) == "left"
    assert str(results.get(0, "")).startswith("error after"), dict(results)


def test_shard_rejects_ragged_batches_and_is_identity_for_one_rank():
    from haste_b200 import data_parallel as dp
    x = torch.arange(24.0).reshape(2, 6, 2)
    assert torch.equal(dp.shard(x, 0, 1), x)
    assert torch.equal(dp.shard(x, 1, 3), x[:, 2:4])
    assert dp.shard(None, 0, 2) is None
    with pytest.raises(ValueError):
        dp.shard(x, 0, 4)
    # without a process group the collectives are no-ops
    t = torch.ones(3)
    assert dp.all_reduce_tensors([t]) is None and torch.equal(t, torch.ones(3))
    dp.all_reduce_tensors([t], async_op=True)()

"""Batch-sharded data parallelism on real devices: two ranks, one GPU each, NCCL.

Each rank runs its half of the batch through a bidirectional GRU stack wired with
`data_parallel.attach` (per-layer gradient buckets, all-reduce issued from inside the backward
pass); rank 0 then checks the summed gradients against a single-GPU run of the whole batch.
Needs two GPUs; skipped otherwise."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, overlap, out):
    import torch.distributed as dist
    import haste_b200 as hb
    from haste_b200 import _C, data_parallel
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        T, N, C, H = 20, 64, 64, 256
        torch.manual_seed(5)
        net = hb.Stack(hb.GRU, C, H, num_layers=3, bidirectional=True, dropout=0.1).to(dev)
        net = net.to(torch.bfloat16)
        net.train()
        data_parallel.broadcast_parameters(net)
        g = torch.Generator().manual_seed(6)
        x = torch.randn(T, N, C, generator=g).to(dev, torch.bfloat16)
        dy = torch.randn(T, N, 2 * H, generator=g).to(dev, torch.bfloat16)
        # DropConnect masks are shared by all ranks: drawn from a seed, not from device state
        masks = [[{"dropconnect_mask": data_parallel.dropconnect_mask((H, 3 * H), 0.1, 100 + 2 * l + d,
                                                                      device=dev)}
                  for d in range(2)] for l in range(3)]
        want = None
        if rank == 0:  # the whole batch on one GPU
            y = net(x.clone().requires_grad_(True), masks=masks)
            (y * dy).sum().backward()
            want = {k: v.grad.float().clone() for k, v in net.named_parameters()}
        dp = data_parallel.attach(net, overlap=overlap)
        for _ in range(2):  # the second step reuses the buckets
            dp.zero_grad()
            xs = data_parallel.shard(x, rank, world).requires_grad_(True)
            ys = net(xs, masks=masks)
            (ys * data_parallel.shard(dy, rank, world)).sum().backward()
            dp.finish()
        torch.cuda.synchronize()
        _C.sync_check(torch.cuda.current_stream().cuda_stream)
        if rank == 0:
            worst = 0.0
            for k, v in net.named_parameters():
                err = float((v.grad.float() - want[k]).abs().max() / max(float(want[k].abs().max()), 1e-6))
                worst = max(worst, err)
            out.put(worst)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("overlap", [True, False])
def test_two_rank_gradients_equal_single_gpu_gradients(overlap):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, overlap, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
    for p in procs:
        if p.is_alive():
            p.kill()  # exactly the process this test started
            pytest.fail("a rank did not finish")
        assert p.exitcode == 0
    worst = out.get(timeout=10)
    assert worst < 2e-2, worst

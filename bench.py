"""Headline benchmark: LSTM forward+backward throughput, N=64, H=C=512, T=1000, fp32.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one forward + backward pass of one LSTM layer over one synthetic batch
(x ~ N(0,1), dy ~ N(0,1), xavier-uniform W, orthogonal R, b = 0) through the haste_b200
C ABI.  The metric is batch*steps per second = N*T / time(fwd+bwd).  Prints ONE JSON line.

 * `value`      inputs resident in HBM, CUDA-event timed over exactly K steps.
 * `e2e`        the same step driven from pinned HOST buffers: every step copies x
                host->device and reads the final state and bias gradient back.
 * `roofline`   dominant kernel (by summed device time, measured live with the
                library's per-phase CUDA events): algorithmic HBM bytes per launch /
                its mean duration, against the measured copy bandwidth.
 * `cpu_baseline` the CPU oracle (a port of the reference's CPU path) on a bounded
                sample of the same workload, on rank 0 at N=1 only.
 * `--impl reference` times that CPU implementation instead, on all host threads.

With N>1 (torchrun, one rank per GPU) every rank runs the full per-GPU batch (weak
scaling) and the weight gradients are all-reduced over NCCL inside the timed step.
Working sets (x 131 MB, gate cache 524 MB) exceed the 126 MB L2, so no explicit flush
is needed between iterations.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(cell="lstm", N=64, C=512, H=512, T=1000)
METRIC = "LSTM fwd+bwd batch*steps/sec (N=64,H=512,T=1000)"
UNIT = "batch*steps/s"


def make_weights(C, H, device, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    W = torch.empty(C, 4 * H)
    R = torch.empty(H, 4 * H)
    for i in range(4):
        torch.nn.init.xavier_uniform_(W[:, i * H:(i + 1) * H], generator=g)
        torch.nn.init.orthogonal_(R[:, i * H:(i + 1) * H], generator=g)
    b = torch.zeros(4 * H)
    return [t.to(device=device, dtype=dtype) for t in (W, R, b)]


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.stop = index, [], threading.Event()
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        # NVML (read-only queries) gives a sample every few milliseconds; nvidia-smi, at one
        # process per sample, is the fallback.
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            bits = [("hw_slowdown", nv.nvmlClocksEventReasonHwSlowdown),
                    ("hw_thermal_slowdown", nv.nvmlClocksEventReasonHwThermalSlowdown),
                    ("sw_thermal_slowdown", nv.nvmlClocksEventReasonSwThermalSlowdown),
                    ("sw_power_cap", nv.nvmlClocksEventReasonSwPowerCap)]
            mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            while not self.stop.is_set():
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                self.samples.append([str(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)), str(mx)] +
                                    ["Active" if r & b else "Not Active" for _, b in bits])
                self.stop.wait(0.005)
            return
        except Exception:
            pass
        while not self.stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                      "--format=csv,noheader,nounits"], capture_output=True,
                                     text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([p.strip() for p in out.split(",")])
            except Exception:
                pass
            self.stop.wait(0.2)

    def __enter__(self):
        self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.thread.join(timeout=6)

    def summary(self):
        mhz = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[2:6]) if v == "Active"})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def cpu_oracle_step(T, N, C, H, threads, seed=0):
    """One fwd+bwd of the CPU oracle (float32) on a T-step sample; returns seconds."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import haste_oracle as oracle
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, N, C, generator=g)
    dy = torch.randn(T, N, H, generator=g)
    W, R, b = make_weights(C, H, "cpu", torch.float32)
    leaves = [t.requires_grad_(True) for t in (x, W, R, b)]
    h0 = torch.zeros(N, H)
    t0 = time.perf_counter()
    h, c = oracle.lstm(True, 0.0, leaves[0], h0, h0, leaves[1], leaves[2], leaves[3])
    (h[1:] * dy).sum().backward()
    return time.perf_counter() - t0


def run_reference_arm(args):
    """The reference's CPU path (oracle port) on the box's host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOAD
    threads = os.cpu_count() or 1
    sample_T = 100
    for _ in range(max(args.warmup, 1)):
        cpu_oracle_step(sample_T, w["N"], w["C"], w["H"], threads)
    times = [cpu_oracle_step(sample_T, w["N"], w["C"], w["H"], threads) for _ in range(args.steps)]
    sec = sum(times) / len(times)
    value = w["N"] * sample_T / sec
    sample = f"T={sample_T} of {w['T']} steps per timed step, same N/C/H, float32 torch CPU"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "lstm_N64_C512_H512_T1000_f32_fwd_bwd", "per_gpu_batch": 64,
                   "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="haste_b200")
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16"])
    ap.add_argument("--T", type=int, default=WORKLOAD["T"], help="override steps per sequence (tests)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ref-cuda", action="store_true",
                    help="also time the reference's own CUDA build if oracle/_ref holds it")
    ap.add_argument("--workload", default="headline",
                    help="headline (default) | grid-<lstm|gru>-N<n>-H<h> | config2 | "
                         "config3-indrnn | config3-lnindrnn | config4-N<n>: the other benchmark "
                         "configurations, one JSON line each (single GPU)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.workload != "headline":
        run_config_workload(args)
        return

    from haste_b200 import _C, data_parallel, ops
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    w = dict(WORKLOAD, T=args.T)
    T, N, C, H = w["T"], w["N"], w["C"], w["H"]
    dtype = torch.float32 if args.dtype == "f32" else torch.bfloat16
    W, R, b = make_weights(C, H, dev, dtype)
    g = torch.Generator().manual_seed(100 + rank)
    x_host = torch.randn(T, N, C, generator=g).to(dtype).pin_memory()
    x = x_host.to(dev)
    dy = torch.cat([torch.zeros(1, N, H), torch.randn(T, N, H, generator=g)]).to(dev, dtype)
    dc = torch.zeros(T + 1, N, H, device=dev, dtype=dtype)
    h0 = torch.zeros(N, H, device=dev, dtype=dtype)
    nomask = torch.empty(0, 0, 0, device=dev, dtype=dtype)
    res_host = torch.empty(N * H + 4 * H, dtype=dtype).pin_memory()
    # dW, dR and db are views of one flat buffer: the backward pass writes into it and the
    # gradient sum over the ranks is one collective on that buffer, with no pack or scatter
    bucket = data_parallel.GradientBucket.for_cell("lstm", C, H, dtype, dev)

    def step(x_dev):
        h, c, cache = ops.lstm_forward(True, 0.0, x_dev, h0, h0, W, R, b, nomask)
        bucket.reset()
        dx, dh, dc0, dW, dR, db = ops.lstm_backward(x_dev, W, R, b, nomask, h, c, cache, dy, dc,
                                                    transposed=False, grads=bucket)
        bucket.all_reduce()
        return h, db

    def e2e_step():
        # host-resident input: the public streamed-input op overlaps the copy with compute
        h, c, cache, x_dev = ops.lstm_forward_from_host(True, 0.0, x_host, h0, h0, W, R, b, nomask)
        bucket.reset()
        dx, dh, dc0, dW, dR, db = ops.lstm_backward(x_dev, W, R, b, nomask, h, c, cache, dy, dc,
                                                    transposed=False, grads=bucket)
        bucket.all_reduce()
        res_host[:N * H].copy_(h[-1].reshape(-1), non_blocking=True)
        res_host[N * H:].copy_(db, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        step(x)
    for _ in range(2):
        e2e_step()
    barrier()

    launches0 = _C.launch_count()
    with ClockSampler(local) as clocks:
        ms_total = timed(lambda: step(x), args.steps)
    launches = _C.launch_count() - launches0
    ms_e2e = timed(e2e_step, args.steps)

    # per-phase device time, measured live (a separate pass so event overhead stays
    # out of the headline number)
    _C.profile_enable(True)
    _C.profile_read()
    for _ in range(args.steps):
        step(x)
    torch.cuda.synchronize()
    phases = {k: v / args.steps for k, v in _C.profile_read().items()}
    _C.profile_enable(False)

    try:
        exchange_us = _C.probe_exchange_latency(N, H, 2000, torch.cuda.current_stream().cuda_stream)
    except Exception:
        exchange_us = None  # shape does not fit the probe's one-CTA-per-SM tiling
    ms_step = ms_total / args.steps
    value = world * N * T / (ms_step * 1e-3)
    e2e_value = world * N * T / (ms_e2e / args.steps * 1e-3)

    # roofline of the dominant kernel
    es = 4 if args.dtype == "f32" else 2
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peaks, peak_src = json.load(open(peaks_path)), "measured"
    else:
        peaks, peak_src = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"
    alg_bytes = {
        # forward recurrence: read x.W (4H), write h, c, gate cache (4H)
        "recurrence_fwd": es * T * N * (4 * H + 2 * H + 4 * H),
        # backward recurrence: read gate cache, c (twice), dh_new, dc_new; write dv
        "recurrence_bwd": es * T * N * (4 * H + 2 * H + 2 * H + 4 * H),
    }
    flops = {
        "input_projection": 2.0 * T * N * C * 4 * H,
        "weight_grad": 2.0 * T * N * 4 * H * (C + H),
        "input_grad": 2.0 * T * N * C * 4 * H,
    }
    # DRAM bytes per time step of the fp32 N=64 H=512 recurrence launches, from one ncu
    # --set full capture at T=200 (dram__bytes_read.sum + dram__bytes_write.sum over 200
    # steps; the summary is profiles/rec_kernels_and_gemm_T200_full_capture.md).  Every
    # step touches its own slice of the activations once, so a launch's traffic is this
    # times T.
    ncu_bytes_per_step = {"recurrence_fwd": (109.377024e6 + 108.569600e6) / 200,
                          "recurrence_bwd": (188.644096e6 + 166.822912e6) / 200}
    dom = max(phases, key=phases.get)
    if dom in alg_bytes:
        ach = alg_bytes[dom] / (phases[dom] * 1e-3) / 1e9
        captured = args.dtype == "f32" and (N, H) == (64, 512)
        roof = {"kernel": dom, "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                "traffic": ncu_bytes_per_step[dom] * T if captured else None,
                "algorithmic_bytes": alg_bytes[dom],
                "peak_source": peak_src,
                "us_per_timestep": phases[dom] * 1e3 / T}
    else:
        ach = flops.get(dom, 0.0) / (phases[dom] * 1e-3) / 1e12
        roof = {"kernel": dom, "bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"],
                "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops"], "traffic": None,
                "peak_source": peak_src}

    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
        "config": {"workload": f"lstm_N{N}_C{C}_H{H}_T{T}_{args.dtype}_fwd_bwd",
                   "per_gpu_batch": N, "l2": "inputs larger than L2 (x 131 MB, cache 524 MB)",
                   "grad_allreduce": world > 1},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * es,
                "d2h_bytes_per_step": res_host.numel() * es},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "roofline": roof,
        # The recurrence is bound by its step-to-step dependency, not by a throughput roofline:
        # measured time per step of both passes beside the time per step of the inter-CTA
        # hand-off alone (exchange-only probe kernel, same tiling, measured in this run).
        "latency": {"fwd_us_per_step": phases["recurrence_fwd"] * 1e3 / T,
                    "bwd_us_per_step": phases["recurrence_bwd"] * 1e3 / T,
                    "exchange_only_us_per_step": exchange_us},
        "phases_ms": phases,
        "phase_tflops": {k: flops[k] / (phases[k] * 1e-3) / 1e12 for k in flops if phases.get(k)},
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        sample_T = 100
        cpu_oracle_step(sample_T, N, C, H, threads)
        secs = sorted(cpu_oracle_step(sample_T, N, C, H, threads) for _ in range(3))
        out["cpu_baseline"] = {"value": N * sample_T / secs[1], "unit": UNIT, "cores": threads,
                               "kind": "port",
                               "sample": f"T={sample_T} of {T} steps, same N/C/H, float32 torch CPU, "
                                         "median of 3"}
    if rank == 0 and world == 1 and args.ref_cuda:
        out["reference_cuda"] = time_reference_cuda(T, N, C, H, x, W, R, b, dy, dc, h0, args.steps)
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def _event_ms(fn, steps, warmup):
    for _ in range(max(warmup, 1)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def _wall_ms(fn, steps, warmup):
    for _ in range(max(warmup, 1)):
        fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) / steps * 1e3


def run_config_workload(args):
    """The benchmark configurations other than the headline, on one GPU, synthetic seeded
    inputs of the configuration's shapes.  One JSON line; `value` is batch*steps/s of a
    forward+backward pass of the whole (possibly stacked, bidirectional) network."""
    import re
    import haste_b200 as hb
    from haste_b200 import ops
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    dtype = torch.float32 if args.dtype == "f32" else torch.bfloat16
    steps, warmup = args.steps, max(args.warmup, 3)
    name = args.workload
    torch.manual_seed(1234)
    out = {"workload": name, "unit": UNIT, "steps": steps, "warmup": warmup, "n_gpus": 1,
           "dtype": args.dtype, "data": "synthetic", "higher_is_better": True}

    def stack_step(net, x):
        def f():
            y = net(x)
            y.backward(torch.ones_like(y))
        return f

    m = re.fullmatch(r"grid-(lstm|gru)-N(\d+)-H(\d+)", name)
    if m:
        cell, N, H = m.group(1), int(m.group(2)), int(m.group(3))
        T, C = 1000, H
        G = 4 if cell == "lstm" else 3
        g = torch.Generator().manual_seed(7)
        x = torch.randn(T, N, C, generator=g).to(dev, dtype)
        W = ((torch.rand(C, G * H, generator=g) * 2 - 1) * (6.0 / (C + H)) ** 0.5).to(dev, dtype)
        R = torch.cat([torch.linalg.qr(torch.randn(H, H, generator=g))[0] for _ in range(G)], 1)
        R = R.contiguous().to(dev, dtype)
        bz = torch.zeros(G * H, device=dev, dtype=dtype)
        h0 = torch.zeros(N, H, device=dev, dtype=dtype)
        dy = torch.cat([torch.zeros(1, N, H), torch.randn(T, N, H, generator=g)]).to(dev, dtype)
        dc = torch.zeros(T + 1, N, H, device=dev, dtype=dtype)
        nomask = torch.empty(0, 0, 0, device=dev, dtype=dtype)
        if cell == "lstm":
            def train():
                h, c, v = ops.lstm_forward(True, 0.0, x, h0, h0, W, R, bz, nomask)
                ops.lstm_backward(x, W, R, bz, nomask, h, c, v, dy, dc, transposed=False)
            infer = lambda: ops.lstm_forward(False, 0.0, x, h0, h0, W, R, bz, nomask)
        else:
            def train():
                h, v = ops.gru_forward(True, 0.0, x, h0, W, R, bz, bz, nomask)
                ops.gru_backward(x, W, R, bz, bz, nomask, h, v, dy, transposed=False)
            infer = lambda: ops.gru_forward(False, 0.0, x, h0, W, R, bz, bz, nomask)
        ms, ms_inf = _event_ms(train, steps, warmup), _event_ms(infer, steps, warmup)
        out.update(metric=f"{cell.upper()} fwd+bwd batch*steps/sec (N={N},H=C={H},T={T})",
                   value=N * T / (ms * 1e-3), ms_per_step=ms,
                   forward_only={"value": N * T / (ms_inf * 1e-3), "ms_per_step": ms_inf})
        if args.ref_cuda:
            sys.path.insert(0, os.path.join(ROOT, "oracle"))
            import ref_cuda
            if ref_cuda.available() and dtype == torch.float32:
                if cell == "lstm":
                    def rtrain():
                        h, c, v = ref_cuda.lstm_forward(True, 0.0, x, h0, h0, W, R, bz, None)
                        ref_cuda.lstm_backward(x, W, R, bz, None, h, c, v, dy, dc)
                    rinfer = lambda: ref_cuda.lstm_forward(False, 0.0, x, h0, h0, W, R, bz, None)
                else:
                    def rtrain():
                        h, v = ref_cuda.gru_forward(True, 0.0, x, h0, W, R, bz, bz, None)
                        ref_cuda.gru_backward(x, W, R, bz, bz, None, h, v, dy)
                    rinfer = lambda: ref_cuda.gru_forward(False, 0.0, x, h0, W, R, bz, bz, None)
                r, ri = _wall_ms(rtrain, min(steps, 3), 1), _wall_ms(rinfer, min(steps, 3), 1)
                out["reference_cuda"] = {"ms_per_step": r, "forward_only_ms": ri,
                                         "value": N * T / (r * 1e-3),
                                         "timing": "host wall clock around synchronous calls"}
            else:
                out["reference_cuda"] = {"unavailable": "oracle/_ref not built or dtype not fp32"}
    elif name == "config2":
        T, N, C, H = 400, 64, 80, 512
        net = hb.Stack(hb.LayerNormLSTM, C, H, num_layers=3, bidirectional=True, zoneout=0.1,
                       dropout=0.05).to(dev).to(dtype)
        net.train()
        x = torch.randn(T, N, C, device=dev, dtype=dtype, requires_grad=True)
        ms = _event_ms(stack_step(net, x), steps, warmup)
        out.update(metric="3-layer bidirectional LayerNormLSTM fwd+bwd batch*steps/sec "
                          "(N=64,C=80,H=512,T=400, zoneout 0.1, DropConnect 0.05)",
                   value=N * T / (ms * 1e-3), ms_per_step=ms)
    elif name in ("config3-indrnn", "config3-lnindrnn"):
        T, N, C, H = 2000, 128, 1024, 1024
        cls = hb.IndRNN if name.endswith("-indrnn") and "ln" not in name else hb.LayerNormIndRNN
        net = hb.Stack(cls, C, H, num_layers=6, zoneout=0.1).to(dev).to(dtype)
        net.train()
        x = torch.randn(T, N, C, device=dev, dtype=dtype, requires_grad=True)
        ms = _event_ms(stack_step(net, x), steps, warmup)
        out.update(metric=f"6-layer {cls.__name__} fwd+bwd batch*steps/sec (N=128,C=H=1024,T=2000)",
                   value=N * T / (ms * 1e-3), ms_per_step=ms)
    elif re.fullmatch(r"config4-N(\d+)", name):
        N = int(name.split("N")[1])
        T, C, H = 500, 512, 1024
        dtype = torch.bfloat16
        out["dtype"] = "bf16"
        net = hb.Stack(hb.GRU, C, H, num_layers=4, bidirectional=True).to(dev).to(dtype)
        net.train()
        x = torch.randn(T, N, C, device=dev, dtype=dtype, requires_grad=True)
        ms = _event_ms(stack_step(net, x), steps, warmup)
        out.update(metric=f"4-layer bidirectional GRU bf16 fwd+bwd batch*steps/sec "
                          f"(per-GPU N={N},C=512,H=1024,T=500)",
                   value=N * T / (ms * 1e-3), ms_per_step=ms)
    else:
        raise SystemExit(f"unknown workload {name!r}")
    print(json.dumps(out))


def time_reference_cuda(T, N, C, H, x, W, R, b, dy, dc, h0, steps):
    """Times the reference's own CUDA build (fp32) on the same buffers, including the
    three transposes its backward needs (as its own benchmark does)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_cuda
    if not ref_cuda.available() or x.dtype != torch.float32:
        return {"unavailable": "oracle/_ref/libhaste_ref.so not built or dtype not fp32"}

    def one():
        h, c, v = ref_cuda.lstm_forward(True, 0.0, x, h0, h0, W, R, b, None)
        ref_cuda.lstm_backward(x, W, R, b, None, h, c, v, dy, dc)

    for _ in range(2):
        one()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        one()
    torch.cuda.synchronize()
    sec = (time.perf_counter() - t0) / steps
    return {"value": N * T / sec, "unit": UNIT, "ms_per_step": sec * 1e3,
            "timing": "host wall clock around synchronous calls (the reference blocks the host)"}


if __name__ == "__main__":
    main()

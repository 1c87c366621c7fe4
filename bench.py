"""Headline benchmark: LSTM forward+backward throughput, N=64, H=C=512, T=1000, fp32.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one forward + backward pass of one LSTM layer over one synthetic batch
(x ~ N(0,1), dy ~ N(0,1), xavier-uniform W, orthogonal R, b = 0) through the haste_b200
C ABI.  The metric is batch*steps per second = N*T / time(fwd+bwd).  Prints ONE JSON line.

 * `value`      inputs resident in HBM, CUDA-event timed over exactly K steps.
 * `e2e`        the same step driven from pinned HOST buffers: every step copies x and
                the incoming gradient dy host->device (overlapped with compute by the
                streamed ops) and reads the final state and bias gradient back.  The
                process is first bound to the CPUs local to its GPU (NVML affinity
                query), so the pinned buffers are NUMA-local; `h2d_gbs_per_rank` is
                each rank's plain copy rate with all ranks copying at once.
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


def bind_near_gpu(index):
    """Restricts this process to the CPUs NVML reports as local to GPU `index` (a read-only
    query), so that the pinned host buffers allocated afterwards land on that GPU's NUMA node
    and the copy-issuing thread runs next to them.  Returns the number of CPUs kept (0: not
    bound)."""
    try:
        import pynvml as nv
        nv.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(index).uuid)
        try:
            h = nv.nvmlDeviceGetHandleByUUID(("GPU-" + uuid).encode())
        except Exception:
            h = nv.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = nv.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (int(w) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return 0
        os.sched_setaffinity(0, cpus)
        return len(cpus)
    except Exception:
        return 0


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.stop = index, [], threading.Event()
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.nv = self.handle = None
        # NVML (read-only queries) gives a sample every few milliseconds; nvidia-smi, at one
        # process per sample, is the fallback.  NVML is set up here, outside the timed region.
        try:
            import pynvml as nv
            nv.nvmlInit()
            self.handle = nv.nvmlDeviceGetHandleByIndex(index)
            self.bits = [nv.nvmlClocksEventReasonHwSlowdown, nv.nvmlClocksEventReasonHwThermalSlowdown,
                         nv.nvmlClocksEventReasonSwThermalSlowdown, nv.nvmlClocksEventReasonSwPowerCap]
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self.handle, nv.NVML_CLOCK_SM)
            self.nv = nv
        except Exception:
            self.nv = None

    def _sample(self):
        if self.nv is not None:
            nv, h = self.nv, self.handle
            r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
            self.samples.append([str(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)), str(self.max_mhz)] +
                                ["Active" if r & b else "Not Active" for b in self.bits])
            return
        out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                              "--format=csv,noheader,nounits"], capture_output=True,
                             text=True, timeout=5).stdout.strip()
        if out:
            self.samples.append([p.strip() for p in out.split(",")])

    def _run(self):
        while not self.stop.is_set():
            try:
                self._sample()
            except Exception:
                pass
            self.stop.wait(0.005 if self.nv is not None else 0.2)

    def __enter__(self):
        self.thread.start()
        t0 = time.perf_counter()  # the sampler is running before the timed region starts
        while not self.samples and time.perf_counter() - t0 < 1.0:
            time.sleep(0.001)
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


def _cpu_sample_length(T, N, C, H, threads, steps_wanted, budget_s):
    """Longest sample of the workload (all T steps if possible) whose `steps_wanted` timed
    steps fit `budget_s` seconds of host time.  Each candidate is tried once (that run is
    the warm-up of the length finally used); returns (T_sample, seconds of that run)."""
    sec = None
    for cand in [t for t in (T, T // 2, T // 4, T // 10) if t >= 1]:
        sec = cpu_oracle_step(cand, N, C, H, threads)
        if sec * steps_wanted <= budget_s or cand == T // 10:
            return cand, sec
        budget_s = max(budget_s - sec, 0.0)
    return max(T // 10, 1), sec


def run_reference_arm(args):
    """The reference's CPU path (oracle port) on the box's host cores, all threads.  Every
    timed step is the whole workload when `--steps` of them fit about four minutes on this
    host; otherwise a prefix of the sequence (same N, C, H), and the line says which."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = dict(WORKLOAD, T=args.T)
    threads = os.cpu_count() or 1
    sample_T, _ = _cpu_sample_length(w["T"], w["N"], w["C"], w["H"], threads,
                                     args.steps + max(args.warmup - 1, 0), 240.0)
    for _ in range(max(args.warmup - 1, 0)):
        cpu_oracle_step(sample_T, w["N"], w["C"], w["H"], threads)
    times = [cpu_oracle_step(sample_T, w["N"], w["C"], w["H"], threads) for _ in range(args.steps)]
    sec = sum(times) / len(times)
    value = w["N"] * sample_T / sec
    whole = sample_T == w["T"]
    sample = (("all" if whole else f"the first {sample_T} of") + f" T={w['T']} steps per timed step, "
              f"N={w['N']}, C={w['C']}, H={w['H']}, float32 torch CPU, all host threads")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": f"lstm_N{w['N']}_C{w['C']}_H{w['H']}_T{w['T']}_f32_fwd_bwd",
                   "per_gpu_batch": w["N"], "sample": sample, "whole_workload": whole},
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
    ap.add_argument("--no-ref-cuda", action="store_true",
                    help="skip timing the reference's own CUDA build (oracle/_ref), which is "
                         "timed by default wherever that library exists")
    ap.add_argument("--ref-cuda", action="store_true", help=argparse.SUPPRESS)  # old spelling
    ap.add_argument("--no-dp-parity", action="store_true",
                    help="config4: skip the single-GPU whole-batch run that checks the reduced "
                         "gradients (it needs the whole batch on rank 0)")
    ap.add_argument("--rec-path", type=int, default=0,
                    help="recurrence implementation (haste_b200_set_recurrence_path): 0 automatic, "
                         "1 step-wise, 3 automatic without the tensor-core recurrence")
    ap.add_argument("--sequential-directions", action="store_true",
                    help="bidirectional workloads: give each direction the whole GPU in turn "
                         "instead of half of it at the same time")
    ap.add_argument("--no-overlap", action="store_true",
                    help="config4: issue the gradient all-reduces after the backward pass "
                         "instead of from inside it")
    ap.add_argument("--workload", default="headline",
                    help="headline (default) | grid-<lstm|gru>-N<n>-H<h> | config2 | "
                         "config3-indrnn | config3-lnindrnn | config4 (global batch 1024 sharded "
                         "over the ranks, under torchrun) | config4-N<n> (per-GPU batch n): the "
                         "other benchmark configurations, one JSON line each")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.rec_path:
        from haste_b200 import _C as _c
        _c.set_recurrence_path(args.rec_path)
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
    cpus_bound = bind_near_gpu(local)  # before the pinned buffers are allocated
    x_host = torch.randn(T, N, C, generator=g).to(dtype).pin_memory()
    x = x_host.to(dev)
    dy_host = torch.cat([torch.zeros(1, N, H), torch.randn(T, N, H, generator=g)]).to(dtype).pin_memory()
    dy = dy_host.to(dev)
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
        # host-resident input and incoming gradient: the public streamed ops overlap both
        # copies with compute (x piece by piece under the forward pass, dy under it as well,
        # latest steps first, consumed piece by piece by the backward pass)
        h, c, cache, x_dev = ops.lstm_forward_from_host(True, 0.0, x_host, h0, h0, W, R, b, nomask)
        bucket.reset()
        dx, dh, dc0, dW, dR, db = ops.lstm_backward_from_host(x_dev, W, R, b, nomask, h, c, cache,
                                                              dy_host, dc, grads=bucket)
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

    # host-to-device rate of this rank while every rank copies at once (the ranks share the
    # host's memory and PCIe paths): the plain copy of x, best of three
    stage = torch.empty_like(x)
    h2d = []
    for _ in range(3):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        stage.copy_(x_host, non_blocking=True)
        e1.record()
        torch.cuda.synchronize()
        h2d.append(x_host.numel() * x_host.element_size() / (e0.elapsed_time(e1) * 1e-3) / 1e9)
    del stage
    h2d_rates = [max(h2d)]
    if world > 1:
        t = torch.tensor([max(h2d)], device=dev)
        allr = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allr, t)
        h2d_rates = [float(v.item()) for v in allr]

    launches0 = _C.launch_count()
    with ClockSampler(local) as clocks:
        ms_total = timed(lambda: step(x), args.steps)
    launches = _C.launch_count() - launches0
    _C.sync_check(torch.cuda.current_stream().cuda_stream)  # raises if a kernel gave up a wait
    ms_e2e = timed(e2e_step, args.steps)
    _C.sync_check(torch.cuda.current_stream().cuda_stream)

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
    # capture of each kernel at T=200 (dram__bytes_read.sum + dram__bytes_write.sum over
    # the 200 steps).  Every step touches its own slice of the activations once, so a
    # launch's traffic is this times T.
    ncu_bytes_per_step = {"recurrence_fwd": (109.424896e6 + 103.794944e6) / 200,
                          "recurrence_bwd": (188.525568e6 + 169.723648e6) / 200}
    dom = max(phases, key=phases.get)
    if dom in alg_bytes:
        ach = alg_bytes[dom] / (phases[dom] * 1e-3) / 1e9
        captured = args.dtype == "f32" and (N, H) == (64, 512)
        roof = {"kernel": dom, "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                "traffic": ncu_bytes_per_step[dom] * T if captured else None,
                "traffic_source": ("ncu capture of this kernel at T=200 (dram bytes read + "
                                   "written), scaled by T") if captured else None,
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
        "e2e": {"value": e2e_value, "unit": UNIT,
                "h2d_bytes_per_step": (x_host.numel() + dy_host.numel()) * es,
                "d2h_bytes_per_step": res_host.numel() * es,
                "inputs_from_host": ["x", "dy"],
                "h2d_gbs_per_rank": [round(v, 1) for v in h2d_rates],
                "cpus_bound_near_gpu": cpus_bound},
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
        # a bounded sample, 10-20 s of host time: the first quarter of the sequence, one warm-up
        # and three timed runs (the whole workload is what `--impl reference` times; the CPU
        # path slows down more than in proportion to T, so a shorter sample reads faster)
        threads = os.cpu_count() or 1
        sample_T = max(T // 4, 1)
        cpu_oracle_step(sample_T, N, C, H, threads)
        secs = sorted(cpu_oracle_step(sample_T, N, C, H, threads) for _ in range(3))
        out["cpu_baseline"] = {"value": N * sample_T / secs[len(secs) // 2], "unit": UNIT,
                               "cores": threads, "kind": "port",
                               "sample": (f"all T={T} steps" if sample_T == T else
                                          f"the first {sample_T} of T={T} steps") +
                                         f", float32 torch CPU, median of {len(secs)} runs"}
    if rank == 0 and world == 1 and not args.no_ref_cuda:
        # the reference's own CUDA build on the same buffers: the denominator of the
        # ">= 2x the reference CUDA build" target
        out["reference_cuda"] = time_reference_cuda(T, N, C, H, x, W, R, b, dy, dc, h0,
                                                    min(args.steps, 5))
        if "ms_per_step" in out["reference_cuda"]:
            out["reference_cuda"]["speedup"] = out["reference_cuda"]["ms_per_step"] / ms_step
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


def _event_and_wall_ms(fn, steps, warmup):
    """(device ms, host wall ms) per call of `fn`, which launches on the legacy default stream
    (the reference's own CUDA build does): events are recorded there."""
    for _ in range(max(warmup, 1)):
        fn()
    torch.cuda.synchronize()
    legacy = torch.cuda.default_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record(legacy)
    for _ in range(steps):
        fn()
    e1.record(legacy)
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) / steps * 1e3
    return e0.elapsed_time(e1) / steps, wall


def _wall_ms(fn, steps, warmup):
    for _ in range(max(warmup, 1)):
        fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) / steps * 1e3


# ---------------------------------------------------------------------------------------
# The other benchmark configurations
# ---------------------------------------------------------------------------------------
def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path)), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def _phases_of(fn, steps):
    """Per-phase device milliseconds of one call of `fn` (library phase events)."""
    from haste_b200 import _C
    _C.profile_enable(True)
    _C.profile_read()
    for _ in range(steps):
        fn()
    torch.cuda.synchronize()
    ph = {k: v / steps for k, v in _C.profile_read().items()}
    _C.profile_enable(False)
    return ph


def _roofline(phases, alg_bytes, flops):
    """Roofline entry of the phase that takes the most device time: HBM bytes for the
    recurrence / scan phases, tensor FLOPs for the contraction phases."""
    peaks, src = _peaks()
    live = {k: v for k, v in phases.items() if v > 0 and (k in alg_bytes or k in flops)}
    if not live:
        return None
    dom = max(live, key=live.get)
    if dom in alg_bytes:
        ach = alg_bytes[dom] / (phases[dom] * 1e-3) / 1e9
        return {"kernel": dom, "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "traffic": None,
                "algorithmic_bytes": alg_bytes[dom], "peak_source": src}
    ach = flops[dom] / (phases[dom] * 1e-3) / 1e12
    return {"kernel": dom, "bound": "tensor", "achieved": ach, "peak": peaks["bf16_tflops"],
            "unit": "TFLOP/s", "frac": ach / peaks["bf16_tflops"], "traffic": None,
            "algorithmic_flops": flops[dom], "peak_source": src}


def _stack_work(cell, T, N, C, H, layers, dirs, es):
    """Algorithmic HBM bytes of the recurrence phases and FLOPs of the contraction phases of
    a whole stack (formulas per layer and direction, summed)."""
    G = {"lstm": 4, "gru": 3, "indrnn": 1}[cell.replace("layer_norm_", "")]
    ab = {"recurrence_fwd": 0.0, "recurrence_bwd": 0.0}
    fl = {"input_projection": 0.0, "weight_grad": 0.0, "input_grad": 0.0}
    for l in range(layers):
        c = C if l == 0 else H * dirs
        for _ in range(dirs):
            if "indrnn" in cell:
                # scan forward: read x.W and mask, write h; backward: read h, dh, mask, write dk
                ab["recurrence_fwd"] += es * T * N * 3 * H
                ab["recurrence_bwd"] += es * T * N * 4 * H
                fl["weight_grad"] += 2.0 * T * N * H * c
            else:
                # forward: read x.W (G*H), write h (+c) and the gate cache; backward: read the
                # cache, states and incoming gradients, write the gate gradients
                states = 2 if "lstm" in cell else 1
                cache = 4 * H
                ab["recurrence_fwd"] += es * T * N * (G * H + states * H + cache)
                ab["recurrence_bwd"] += es * T * N * (cache + 2 * states * H + (2 if G == 3 else 1) * G * H)
                fl["weight_grad"] += 2.0 * T * N * G * H * (c + H)
            fl["input_projection"] += 2.0 * T * N * G * H * c
            fl["input_grad"] += 2.0 * T * N * G * H * c
    return ab, fl


def _ref_stack_step(cell, net, x, dy, dropconnect):
    """One forward+backward of the same stack through the REFERENCE's own CUDA build, composed
    from its single layers the way a user composes them (flip / run / flip back, concatenate),
    fp32 only.  Returns a callable, or None where the reference has no such cell."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_cuda
    if not ref_cuda.available() or x.dtype != torch.float32:
        return None
    fwd = getattr(ref_cuda, cell + "_forward")
    bwd = getattr(ref_cuda, cell + "_backward")
    has_c = "lstm" in cell

    def params(layer):
        p = dict(layer.named_parameters())
        if "indrnn" in cell:
            a = [p["kernel"], p["recurrent_scale"], p["bias"]]
        elif "gru" in cell:
            a = [p["kernel"], p["recurrent_kernel"], p["bias"], p["recurrent_bias"]]
        else:
            a = [p["kernel"], p["recurrent_kernel"], p["bias"]]
        a += [p[k] for k in ("gamma", "gamma_h", "beta_h") if k in p]
        return [t.detach() for t in a]

    def step():
        inp, tape = x, []
        for level in net.layers:
            outs, H = [], level[0].hidden_size
            for d_, layer in enumerate(level):
                xi = torch.flip(inp, [0]).contiguous() if d_ == 1 else inp
                a = params(layer)
                if dropconnect and "indrnn" not in cell:
                    a[1] = a[1] * (torch.bernoulli(torch.full_like(a[1], 1 - dropconnect)) / (1 - dropconnect))
                N = xi.shape[1]
                z = xi.new_zeros(N, H)
                mask = torch.bernoulli(torch.full((xi.shape[0], N, H), 0.9, device=xi.device)) \
                    if layer.zoneout else None
                st = (z, z) if has_c else (z,)
                res = fwd(True, layer.zoneout, xi, *st, *a, mask)
                res = (res,) if torch.is_tensor(res) else res
                tape.append((xi, a, mask, res))
                y = res[0][1:]
                outs.append(torch.flip(y, [0]) if d_ == 1 else y)
            inp = torch.cat(outs, -1) if len(outs) > 1 else outs[0]
        g = dy
        for level in reversed(net.layers):
            H, dxs = level[0].hidden_size, []
            for d_ in reversed(range(len(level))):
                xi, a, mask, res = tape.pop()
                gd = g[..., d_ * H:(d_ + 1) * H] if len(level) > 1 else g
                gd = torch.flip(gd, [0]) if d_ == 1 else gd
                dh = torch.cat([torch.zeros_like(gd[:1]), gd]).contiguous()
                if has_c:
                    grads = bwd(xi, *a, mask, *res, dh, torch.zeros_like(dh))
                else:
                    grads = bwd(xi, *a, mask, *res, dh)
                dxi = grads["x"]
                dxs.append(torch.flip(dxi, [0]) if d_ == 1 else dxi)
            g = dxs[0] if len(dxs) == 1 else dxs[0] + dxs[1]
    return step


def run_config_workload(args):
    """The benchmark configurations other than the headline, synthetic seeded inputs of the
    configuration's shapes.  One JSON line: `value` is batch*steps/s of a forward+backward pass
    of the whole (possibly stacked, bidirectional) network, with `phases_ms`, the `roofline`
    of the dominant phase and, where the reference has the cell in fp32, `reference_cuda`."""
    import re
    import haste_b200 as hb
    from haste_b200 import _C, ops
    name = args.workload
    if re.fullmatch(r"config4(-N\d+)?", name):
        return run_config4(args)
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    dtype = torch.float32 if args.dtype == "f32" else torch.bfloat16
    es = 4 if dtype == torch.float32 else 2
    steps, warmup = args.steps, max(args.warmup, 3)
    torch.manual_seed(1234)
    out = {"workload": name, "unit": UNIT, "steps": steps, "warmup": warmup, "n_gpus": 1,
           "dtype": args.dtype, "data": "synthetic", "higher_is_better": True}
    ref_step = None

    def stack_step(net, x, dy):
        def f():
            y = net(x)
            y.backward(dy)
        return f

    m = re.fullmatch(r"grid-(lstm|gru)-N(\d+)-H(\d+)", name)
    if m:
        cell, N, H = m.group(1), int(m.group(2)), int(m.group(3))
        T, C = args.T, H
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
        ms_inf = _event_ms(infer, steps, warmup)
        out.update(metric=f"{cell.upper()} fwd+bwd batch*steps/sec (N={N},H=C={H},T={T})",
                   forward_only={"value": N * T / (ms_inf * 1e-3), "ms_per_step": ms_inf})
        step, layers, dirs = train, 1, 1
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import ref_cuda
        if ref_cuda.available() and dtype == torch.float32 and not args.no_ref_cuda:
            if cell == "lstm":
                def ref_step():
                    h, c, v = ref_cuda.lstm_forward(True, 0.0, x, h0, h0, W, R, bz, None)
                    ref_cuda.lstm_backward(x, W, R, bz, None, h, c, v, dy, dc)
            else:
                def ref_step():
                    h, v = ref_cuda.gru_forward(True, 0.0, x, h0, W, R, bz, bz, None)
                    ref_cuda.gru_backward(x, W, R, bz, bz, None, h, v, dy)
    elif name == "config2":
        T, N, C, H = (400 if args.T == WORKLOAD["T"] else args.T), 64, 80, 512
        cell, layers, dirs = "layer_norm_lstm", 3, 2
        net = hb.Stack(hb.LayerNormLSTM, C, H, num_layers=3, bidirectional=True, zoneout=0.1,
                       dropout=0.05,
                       concurrent_directions=not args.sequential_directions).to(dev).to(dtype)
        net.train()
        x = torch.randn(T, N, C, device=dev, dtype=dtype, requires_grad=True)
        dy = torch.randn(T, N, 2 * H, device=dev, dtype=dtype)
        step = stack_step(net, x, dy)
        out["metric"] = ("3-layer bidirectional LayerNormLSTM fwd+bwd batch*steps/sec "
                         f"(N=64,C=80,H=512,T={T}, zoneout 0.1, DropConnect 0.05)")
        if not args.no_ref_cuda:
            ref_step = _ref_stack_step(cell, net, x.detach(), dy, 0.05)
    elif name in ("config3-indrnn", "config3-lnindrnn"):
        T, N, C, H = (2000 if args.T == WORKLOAD["T"] else args.T), 128, 1024, 1024
        cell = "indrnn" if name == "config3-indrnn" else "layer_norm_indrnn"
        layers, dirs = 6, 1
        cls = hb.IndRNN if cell == "indrnn" else hb.LayerNormIndRNN
        net = hb.Stack(cls, C, H, num_layers=6, zoneout=0.1).to(dev).to(dtype)
        with torch.no_grad():
            for level in net.layers:
                level[0].recurrent_scale.uniform_(0.0, 1.0)
        net.train()
        x = torch.randn(T, N, C, device=dev, dtype=dtype, requires_grad=True)
        dy = torch.randn(T, N, H, device=dev, dtype=dtype)
        step = stack_step(net, x, dy)
        out["metric"] = f"6-layer {cls.__name__} fwd+bwd batch*steps/sec (N=128,C=H=1024,T={T})"
        if not args.no_ref_cuda:
            ref_step = _ref_stack_step(cell, net, x.detach(), dy, 0.0)
    else:
        raise SystemExit(f"unknown workload {name!r}")

    ms = _event_ms(step, steps, warmup)
    _C.sync_check(torch.cuda.current_stream().cuda_stream)
    phases = _phases_of(step, min(steps, 3))
    ab, fl = _stack_work(cell, T, N, C, H, layers, dirs, es)
    out.update(value=N * T / (ms * 1e-3), ms_per_step=ms, phases_ms=phases,
               roofline=_roofline(phases, ab, fl),
               phase_tflops={k: fl[k] / (phases[k] * 1e-3) / 1e12 for k in fl if phases.get(k)},
               phase_gbs={k: ab[k] / (phases[k] * 1e-3) / 1e9 for k in ab if phases.get(k)})
    if ref_step is not None:
        rms, rwall = _event_and_wall_ms(ref_step, min(steps, 3), 1)
        out["reference_cuda"] = {"ms_per_step": rms, "wall_ms_per_step": rwall,
                                 "value": N * T / (rms * 1e-3), "speedup": rms / ms,
                                 "timing": "CUDA events on the legacy default stream"}
    elif not args.no_ref_cuda:
        out["reference_cuda"] = {"unavailable": "oracle/_ref not built, or the reference has no "
                                                "such cell in this dtype"}
    print(json.dumps(out))


def run_config4(args):
    """Configuration 4: a data-parallel training step of a 4-layer bidirectional GRU in bf16,
    C=512, H=1024, T=500.  `config4` shards a GLOBAL batch of 1024 evenly over the ranks
    (strong scaling; launch under torchrun for more than one GPU); `config4-N<n>` runs a
    per-GPU batch of n on one GPU.  Parameter gradients are written by each layer's backward
    pass into that layer's bucket and all-reduced over NCCL from inside the backward pass, so
    the collectives overlap the backward passes of the layers below."""
    import haste_b200 as hb
    from haste_b200 import _C, data_parallel
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    T, C, H, layers = (500 if args.T == WORKLOAD["T"] else args.T), 512, 1024, 4
    fixed = "-N" in args.workload
    n_global = int(args.workload.split("N")[1]) * world if fixed else 1024
    n_local = n_global // world
    dtype = torch.bfloat16
    torch.manual_seed(4321)  # same parameters on every rank
    net = hb.Stack(hb.GRU, C, H, num_layers=layers, bidirectional=True,
                   concurrent_directions=not args.sequential_directions).to(dev).to(dtype)
    net.train()
    data_parallel.broadcast_parameters(net)
    # the whole global batch is drawn on every rank's own GPU from the same seed (identical
    # devices give identical values), then cut: no host-side generation of gigabytes
    g = torch.Generator(device=dev).manual_seed(99)
    x_all = torch.randn(T, n_global, C, generator=g, device=dev).to(dtype)
    dy_all = torch.randn(T, n_global, 2 * H, generator=g, device=dev).to(dtype)
    x = data_parallel.shard(x_all, rank, world).clone().requires_grad_(True)
    dy = data_parallel.shard(dy_all, rank, world).clone()
    if world > 1 and (rank != 0 or args.no_dp_parity):
        del x_all, dy_all
    steps, warmup = args.steps, max(args.warmup, 3)

    def make_step(dp):
        def f():
            dp.zero_grad()
            y = net(x)
            y.backward(dy)
            dp.finish()
        return f

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, k, warm=warmup):
        for _ in range(warm):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(k):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / k], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    dp = data_parallel.attach(net, overlap=not args.no_overlap)
    step = make_step(dp)
    for _ in range(warmup):
        step()
    launches0 = _C.launch_count()
    with ClockSampler(local) as clocks:
        ms = timed(step, steps, warm=0)
    launches = _C.launch_count() - launches0
    _C.sync_check(torch.cuda.current_stream().cuda_stream)
    grads = {k: v.grad.float().clone() for k, v in net.named_parameters()}
    bucket_bytes = dp.bucket_bytes()
    dp.detach()
    # the same step without any collective: what communication adds when it is exposed
    dp0 = data_parallel.attach(net, reduce=False)
    ms_nocomm = timed(make_step(dp0), max(2, steps // 2)) if world > 1 else ms
    dp0.detach()
    phases = _phases_of(make_step(data_parallel.attach(net, reduce=False)), 2)
    for m_ in net.modules():
        if hasattr(m_, "_dp"):
            m_._dp = None

    # parity of the reduced gradients with a single-GPU run of the whole batch (rank 0)
    dp_err = None
    if world > 1 and rank == 0 and not args.no_dp_parity:
        for p in net.parameters():
            p.grad = None
        xf = x_all.requires_grad_(True)
        net(xf).backward(dy_all)
        torch.cuda.synchronize()
        dp_err = 0.0
        for k, v in net.named_parameters():
            want = v.grad.float()
            dp_err = max(dp_err, float((grads[k] - want).abs().max() / max(float(want.abs().max()), 1e-6)))
    ab, fl = _stack_work("gru", T, n_local, C, H, layers, 2, 2)
    total_flops = 6.0 * T * n_global * 3 * H * ((C + H) + (layers - 1) * (2 * H + H)) * 2
    peaks, src = _peaks()
    out = {
        "workload": args.workload, "metric": "4-layer bidirectional GRU bf16 data-parallel fwd+bwd "
        f"batch*steps/sec (global N={n_global}, C=512, H=1024, T={T})",
        "value": n_global * T / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak" if fixed else "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": args.workload, "global_batch": n_global, "per_gpu_batch": n_local,
                   "layers": layers, "bidirectional": True,
                   "grad_allreduce": "per layer and direction, issued from inside the backward pass"
                   if not args.no_overlap else "after the backward pass",
                   "bucket_bytes_per_step": bucket_bytes,
                   "l2": "inputs larger than L2"},
        "gpu_launches": int(launches), "clocks": clocks.summary(),
        "ms_per_step_without_allreduce": ms_nocomm,
        "exposed_communication_ms": max(ms - ms_nocomm, 0.0),
        "dp_parity_err": dp_err,
        "tflops": total_flops / (ms * 1e-3) / 1e12,
        "tensor_frac_of_peak": total_flops / world / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
        "phases_ms": phases, "roofline": _roofline(phases, ab, fl),
        "phase_tflops": {k: fl[k] / (phases[k] * 1e-3) / 1e12 for k in fl if phases.get(k)},
    }
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def time_reference_cuda(T, N, C, H, x, W, R, b, dy, dc, h0, steps):
    """Times the reference's own CUDA build (fp32) on the same buffers, including the three
    transposes its backward pass needs (its own benchmark charges them too).  Device time by
    CUDA events on the stream the reference runs on, host wall clock beside it (the
    reference's LSTM passes block the host when they are destroyed)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ref_cuda
    if not ref_cuda.available():
        return {"unavailable": "oracle/_ref/libhaste_ref.so is not built on this machine"}
    if x.dtype != torch.float32:
        return {"unavailable": "the reference has no bf16 build"}

    def one():
        h, c, v = ref_cuda.lstm_forward(True, 0.0, x, h0, h0, W, R, b, None)
        ref_cuda.lstm_backward(x, W, R, b, None, h, c, v, dy, dc)

    ms, wall = _event_and_wall_ms(one, steps, 2)
    return {"value": N * T / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "wall_ms_per_step": wall,
            "steps": steps,
            "timing": "CUDA events on the legacy default stream the reference launches on; "
                      "includes its three transposes"}


if __name__ == "__main__":
    main()

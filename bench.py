"""Benchmark of the fused conv2d hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c3]

A step is one pass of the fused conv -> bias -> ReLU graph over one batch of
synthetic input.  The default workload is the 3x3 256-channel layer the
headline target is quoted on; --workload picks the 1x1, stem or fp32 layers.
With N > 1 (launched under torchrun, one rank per GPU) every rank runs the
same batch-sized problem on its own GPU — the path shards along the batch with
replicated filters and needs no collective — so the scaling is weak.

One JSON line is printed by rank 0:
  value     device-resident throughput (TFLOP/s over all ranks): inputs already
            in HBM, steps replayed from a CUDA graph, operands rotated through
            more buffers than L2 holds so every step reads from DRAM;
  e2e       the same metric through the public API from pinned HOST buffers,
            host->device and device->host copies inside the timed region;
  roofline  the implicit-GEMM kernel against the measured tensor (or HBM) peak;
  cpu_baseline  the reference's CPU path (torch.nn.functional.conv2d + relu,
            what src/flag_dnn/graph/registry.py:1357-1365,1426 runs on CPU
            tensors) on a bounded sample, all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# name: (N, C, H, K, R, stride, pad, dtype, layout, x distribution, roofline bound)
WORKLOADS = {
    "c3": dict(desc="3x3 conv+bias+ReLU bf16 NHWC N=256 C=K=256 H=W=14 s1 p1", n=256, c=256, hw=14, k=256, r=3,
               stride=1, pad=1, dtype="bfloat16", layout="nhwc", dist="normal", bound="tensor"),
    "c2": dict(desc="1x1 conv+bias+ReLU bf16 NHWC N=256 C=256 H=W=56 K=64", n=256, c=256, hw=56, k=64, r=1,
               stride=1, pad=0, dtype="bfloat16", layout="nhwc", dist="normal", bound="hbm"),
    "c4": dict(desc="7x7 s2 stem conv+bias+ReLU bf16 NHWC N=256 C=3 H=W=224 K=64", n=256, c=3, hw=224, k=64, r=7,
               stride=2, pad=3, dtype="bfloat16", layout="nhwc", dist="uniform", bound="hbm"),
    "c1": dict(desc="3x3 conv+bias fp32 NCHW N=4 C=64 H=W=56 K=64 s1 p1 (split TF32)", n=4, c=64, hw=56, k=64, r=3,
               stride=1, pad=1, dtype="float32", layout="nchw", dist="normal", bound="tensor"),
}

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the implicit-GEMM
# kernel, from the ncu captures summarised under profiles/ (None = not captured).
NCU_TRAFFIC_BYTES = {"c3": 26.98e6, "c2": 495.9e6, "c4": 435.0e6, "c1": None}

# the arithmetic type as the JSON line names it (fp32 tensors run as 3xTF32 with fp32 accumulation)
SHORT_DTYPE = {"bfloat16": "bf16", "float16": "f16", "float32": "f32"}

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            data = json.load(fh)
        return {k: float(data[k]) for k in FALLBACK_PEAKS}, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


def out_dim(size, pad, r, stride):
    return (size + 2 * pad - (r - 1) - 1) // stride + 1


def workload_numbers(wl):
    oh = out_dim(wl["hw"], wl["pad"], wl["r"], wl["stride"])
    es = 2 if wl["dtype"] != "float32" else 4
    flops = 2.0 * wl["n"] * oh * oh * wl["k"] * wl["c"] * wl["r"] * wl["r"]
    x_bytes = wl["n"] * wl["c"] * wl["hw"] * wl["hw"] * es
    w_bytes = wl["k"] * wl["c"] * wl["r"] * wl["r"] * es
    y_bytes = wl["n"] * wl["k"] * oh * oh * es
    return dict(oh=oh, flops=flops, x_bytes=x_bytes, w_bytes=w_bytes, y_bytes=y_bytes,
                bytes=x_bytes + w_bytes + y_bytes + wl["k"] * es)


def make_inputs(wl, n, seed, device, torch):
    """Seeded synthetic tensors with the configuration's shapes and distributions."""
    dtype = getattr(torch, wl["dtype"])
    g = torch.Generator(device=device).manual_seed(seed)
    shape = (n, wl["c"], wl["hw"], wl["hw"])
    if wl["dist"] == "uniform":
        x = torch.rand(shape, generator=g, device=device) * 2 - 1
    else:
        x = torch.randn(shape, generator=g, device=device)
    fan_in = wl["c"] * wl["r"] * wl["r"]
    w = torch.randn((wl["k"], wl["c"], wl["r"], wl["r"]), generator=g, device=device) * fan_in ** -0.5
    b = torch.randn((wl["k"],), generator=g, device=device) * 0.1
    x, w, b = x.to(dtype), w.to(dtype), b.to(dtype)
    if wl["layout"] == "nhwc":
        x = x.contiguous(memory_format=torch.channels_last)
        w = w.contiguous(memory_format=torch.channels_last)
    return x, w, b


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while a region runs (every 2 ms, plus on request)."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
            self._bits = {
                "hw_slowdown": getattr(pynvml, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                "sw_power_cap": getattr(pynvml, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
                "hw_thermal_slowdown": getattr(pynvml, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(pynvml, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                "hw_power_brake": getattr(pynvml, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
            }
        except Exception:
            self._nvml = None

    def sample(self):
        """One reading now; a region shorter than the sampling period calls this right after its launches are
        queued (the GPU is then under that load) and once more before it synchronises."""
        nv = self._nvml
        if nv is None:
            return
        try:
            self.samples.append(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
            mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
            for name, bit in self._bits.items():
                if mask & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def _loop(self):
        while not self._stop.is_set():
            self.sample()
            time.sleep(0.002)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        return False

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def use_all_host_threads(torch):
    """torchrun pins OMP_NUM_THREADS=1; the CPU legs are meant to use every core the process may run on."""
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    torch.set_num_threads(max(1, cores))
    return torch.get_num_threads()


def time_cpu_calls(fn, warmup, steps=None, min_seconds=None, min_warm_seconds=3.0, max_warm_seconds=20.0):
    """Wall-clock times of repeated calls of `fn` on the host.  The warm-up makes at least `warmup` calls, lasts at
    least `min_warm_seconds` and goes on until two consecutive calls agree within 5 %: a bf16 convolution on the
    host cores keeps getting faster for about a second of back-to-back calls (2.3x on this pool's hosts: thread
    pool, matrix-unit clocks, page placement), and only the steady state is a fair baseline.  Then exactly `steps`
    calls are timed, or as many as fit `min_seconds`."""
    prev, calls, t_warm = None, 0, time.perf_counter()
    while True:
        t0 = time.perf_counter()
        fn()
        now = time.perf_counter()
        dt = now - t0
        calls += 1
        steady = prev is not None and abs(dt - prev) <= 0.05 * max(dt, prev)
        if calls >= max(warmup, 2) and ((now - t_warm >= min_warm_seconds and steady) or now - t_warm >= max_warm_seconds):
            break
        prev = dt
    times, t_all = [], time.perf_counter()
    while True:
        if steps is not None and len(times) >= steps:
            break
        if steps is None and len(times) >= 3 and (time.perf_counter() - t_all >= min_seconds or len(times) >= 5000):
            break
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    return times


def _cpu_layer_call(wl, torch, sample_n):
    """The reference's CPU path for one workload on `sample_n` images: the oracle's torch call, used here as the
    timed CPU baseline (test-infrastructure code as the checker's timer, never on the product path)."""
    import oracle

    x, w, b = make_inputs(wl, sample_n, 0, "cpu", torch)
    relu = wl["dtype"] != "float32"
    cdt = getattr(torch, wl["dtype"])  # the reference runs F.conv2d in the tensors' own dtype
    return lambda: oracle.conv2d_torch_cpu(x, w, b, wl["stride"], wl["pad"], 1, 1, relu=relu, compute_dtype=cdt)


def cpu_baseline_leg(wl, torch, sample_n, min_seconds=10.0):
    """The reference's CPU path timed on the host cores for about `min_seconds`; median of the steady-state calls."""
    use_all_host_threads(torch)
    times = time_cpu_calls(_cpu_layer_call(wl, torch, sample_n), warmup=3, min_seconds=min_seconds)
    med = statistics.median(times)
    nums = workload_numbers(dict(wl, n=sample_n))
    return dict(value=nums["flops"] / med / 1e12, unit="TFLOP/s", cores=torch.get_num_threads(), kind="port",
                sample=f"{sample_n} of {wl['n']} images, {len(times)} repeats, median; torch.nn.functional.conv2d+relu "
                       f"in {wl['dtype']} on CPU (the call the reference's CPU graph path makes)",
                ms_per_sample=med * 1e3, ms_per_sample_mean=statistics.fmean(times) * 1e3)


def run_reference(args):
    """The reference arm: the reference's CPU path on the host cores (rank 0 only), exactly --steps timed calls of a
    bounded sample after a warm-up that runs until the call time is steady; the line's value is the median."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    use_all_host_threads(torch)
    wl = WORKLOADS[args.workload]
    sample_n = min(wl["n"], 32)
    nums = workload_numbers(dict(wl, n=sample_n))
    steps = max(1, args.steps)
    times = time_cpu_calls(_cpu_layer_call(wl, torch, sample_n), warmup=max(args.warmup, 3), steps=steps)
    med, mean = statistics.median(times), statistics.fmean(times)
    value = nums["flops"] / med / 1e12
    sample = (f"each step = {sample_n} of {wl['n']} images through torch.nn.functional.conv2d+relu in {wl['dtype']} "
              f"on the host CPU (the reference's CPU graph path); {steps} steps timed after a warm-up of at least 3 s of "
              f"back-to-back calls that ended when two consecutive calls agreed within 5 %; value from the median step")
    line = {
        "impl": "reference", "metric": "fused_conv2d_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": med * 1e3,
        "ms_per_step_mean": mean * 1e3, "value_from_mean": nums["flops"] / mean / 1e12,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": SHORT_DTYPE[wl["dtype"]], "data": "synthetic",
        "config": {"workload": args.workload, "description": wl["desc"], "sample_images": sample_n},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def init_ranks(torch, cpu_leg=None):
    """Device selection and, under torchrun, the NCCL process group.  `cpu_leg` (rank 0 only) runs BEFORE the
    group is created: the other ranks then sit in the rendezvous, a blocking socket wait, instead of spinning in
    an NCCL barrier on the host cores the CPU baseline is being timed on."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU path for this library)")
    torch.cuda.set_device(local_rank)
    cpu = cpu_leg() if (cpu_leg is not None and rank == 0) else None
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    return rank, world, local_rank, dist, cpu


def hold_gpu(torch, stream=None, micros=150):
    """Keeps the GPU busy for about `micros` so that the launches of a short timed region are already queued when
    the GPU reaches the region's first event: the CPU's launch latency (10-20 us for a graph launch) then does not
    sit between that event and the first kernel.  Nothing but a spin kernel; caches and clocks are untouched."""
    try:
        if stream is None:
            torch.cuda._sleep(int(micros * 2000))
        else:
            with torch.cuda.stream(stream):
                torch.cuda._sleep(int(micros * 2000))
    except Exception:
        pass


def max_over_ranks(torch, dist, device, values):
    if dist is None:
        return list(values)
    t = torch.tensor(list(values), device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t.tolist()]


def count_true_over_ranks(torch, dist, device, flag):
    if dist is None:
        return int(bool(flag))
    t = torch.tensor([1.0 if flag else 0.0], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return int(round(float(t.item())))


def run_ours(args):
    import torch

    import flagdnn_b200 as fd

    wl = WORKLOADS[args.workload]
    rank, world, local_rank, dist, cpu = init_ranks(
        torch, None if args.kernel_only else (lambda: cpu_baseline_leg(wl, torch, sample_n=min(wl["n"], 32))))
    device = torch.device("cuda", local_rank)
    nums = workload_numbers(wl)
    peaks, peak_src = load_peaks()
    relu = wl["dtype"] != "float32"

    # ---- operands: enough rotating (x, y) sets that a set is evicted from L2 before it is reused
    l2_bytes = 126 * 1024 * 1024
    per_set = nums["x_bytes"] + nums["y_bytes"]
    n_sets = max(2, min(64, -(-3 * l2_bytes // per_set)))
    xs = []
    w = b = None
    for i in range(n_sets):
        x, w_i, b_i = make_inputs(wl, wl["n"], 100 * rank + i, device, torch)
        xs.append(x)
        if w is None:
            w, b = w_i, b_i

    @fd.graph
    def layer(x, weight, bias):
        y = fd.conv2d(x, weight, stride=wl["stride"], padding=wl["pad"])
        y = fd.bias_add(y, bias)
        return fd.relu(y) if relu else y

    compiled = fd.compile(layer, inputs=[xs[0], w, b], options={"cache": None})
    node_types = [n.op_type for n in compiled.graph.nodes]
    plan = fd.conv2d_plan(xs[0], w, stride=wl["stride"], padding=wl["pad"])
    launches_per_step = plan["launches"]

    # first calls through the eager API (pack the filter, set kernel attributes); not the counted warm-up
    for i in range(3):
        compiled.run(xs[i % n_sets], w, b)
    torch.cuda.synchronize()

    # ---- device-resident leg.  Step i runs on operand set i % n_sets.  One CUDA graph holds a whole cycle of
    # n_sets steps; a second, shorter graph holds the steps % n_sets steps that remain, so that exactly --steps
    # (and exactly --warmup) steps run while consecutive launches stay inside a graph.
    stream = torch.cuda.Stream()
    outs = []

    class _EagerSteps:
        def __init__(self, count):
            self.count = count

        def replay(self):
            for i in range(self.count):
                compiled.run(xs[i], w, b)

    def capture(count, keep=None):
        if count == 0:
            return None
        if args.eager:
            return _EagerSteps(count)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for i in range(count):
                y = compiled.run(xs[i], w, b)
                if keep is not None:
                    keep.append(y)
        return g

    steps, warmup = max(1, args.steps), max(3, args.warmup)
    one_graph_limit = 4096   # up to this many steps a region is ONE graph (consecutive launches overlap their set-up
                             # with the previous launch's tail only inside a graph); longer regions replay cycles
    with torch.cuda.stream(stream):
        for i in range(n_sets):
            out = compiled.run(xs[i], w, b)
            if args.eager:
                outs.append(out)
        stream.synchronize()
        cycle = capture(n_sets, outs)
        tails = {}
        for r in {steps % n_sets, warmup % n_sets}:
            tails[r] = capture(r)
        whole = {}
        if not args.eager:
            for count in {steps, warmup}:
                if count <= one_graph_limit:
                    g_ = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g_, stream=stream):
                        for i in range(count):
                            compiled.run(xs[i % n_sets], w, b)
                    whole[count] = g_
        # a CUDA graph is uploaded to the device by its first launch: launch each one once here, before the
        # counted warm-up, so that neither the warm-up nor the timed region contains a first launch
        for g_ in [cycle] + [t for t in tails.values() if t is not None] + list(whole.values()):
            g_.replay()
        stream.synchronize()

    def run_steps(count):
        if count in whole:
            whole[count].replay()
            return
        for _ in range(count // n_sets):
            cycle.replay()
        if count % n_sets:
            tails[count % n_sets].replay()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        run_steps(warmup)
        stream.synchronize()
        barrier()
        with ClockSampler(local_rank) as clocks:
            hold_gpu(torch, stream)
            e0.record(stream)
            run_steps(steps)
            e1.record(stream)
            clocks.sample()   # the launches are queued: the GPU is executing them now
            stream.synchronize()
            clocks.sample()
        barrier()
    elapsed_ms = max_over_ranks(torch, dist, device, [e0.elapsed_time(e1)])[0]
    ms_per_step = elapsed_ms / steps
    value = world * nums["flops"] / (ms_per_step * 1e-3) / 1e12

    # ---- a region of at least 100 ms of the same steps when the requested one was shorter than 50 ms: the clock
    # sampler then sees the GPU under sustained load (power cap); reported beside `value`, never instead of it
    sustained = None
    if elapsed_ms < 50.0 and not args.eager:
        long_steps = int(-(-120.0 // ms_per_step))
        long_steps = -(-long_steps // n_sets) * n_sets
        with torch.cuda.stream(stream):
            barrier()
            with ClockSampler(local_rank) as long_clocks:
                e0.record(stream)
                run_steps(long_steps)
                e1.record(stream)
                stream.synchronize()
            barrier()
        long_ms = max_over_ranks(torch, dist, device, [e0.elapsed_time(e1)])[0]
        sustained = {"steps": long_steps, "ms_per_step": long_ms / long_steps,
                     "value": world * nums["flops"] / (long_ms / long_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                     "clocks": long_clocks.summary()}

    # ---- the same steps with two streams: independent batches overlap, so the SMs that idle through the last
    # partial wave of tiles of one launch start the next launch's tiles (reported beside `value`, not as it:
    # `value` and the roofline stay the serial per-launch figures)
    concurrent = None
    if not args.eager and n_sets >= 2:
        side = torch.cuda.Stream()
        graph2 = torch.cuda.CUDAGraph()
        replays = max(1, steps // n_sets)
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph2, stream=stream):
                side.wait_stream(stream)
                for i in range(n_sets):
                    with torch.cuda.stream(side if i % 2 else stream):
                        compiled.run(xs[i], w, b)
                stream.wait_stream(side)
            graph2.replay()
            stream.synchronize()
            barrier()
            e0.record(stream)
            for _ in range(replays):
                graph2.replay()
            e1.record(stream)
            stream.synchronize()
            barrier()
        c_ms = max_over_ranks(torch, dist, device, [e0.elapsed_time(e1)])[0]
        c_steps = replays * n_sets
        concurrent = {"streams": 2, "steps": c_steps, "ms_per_step": c_ms / c_steps,
                      "value": world * nums["flops"] / (c_ms / c_steps * 1e-3) / 1e12, "unit": "TFLOP/s"}

    # ---- every step through the eager API (no CUDA graph): what a caller without graphs pays per call
    eager = None
    if not args.eager and not args.kernel_only:
        e_steps = 300
        for i in range(300):   # the host side of a call keeps getting faster for its first few hundred calls
            compiled.run(xs[i % n_sets], w, b)
        torch.cuda.synchronize()
        barrier()
        e0.record()
        for i in range(e_steps):
            compiled.run(xs[i % n_sets], w, b)
        e1.record()
        torch.cuda.synchronize()
        barrier()
        eg_ms = max_over_ranks(torch, dist, device, [e0.elapsed_time(e1)])[0]
        t_host = time.perf_counter()
        for i in range(e_steps):
            compiled.run(xs[i % n_sets], w, b)
        host_us = (time.perf_counter() - t_host) / e_steps * 1e6
        torch.cuda.synchronize()
        eager = {"steps": e_steps, "ms_per_step": eg_ms / e_steps, "host_enqueue_us_per_call": host_us,
                 "note": "every step one call of the compiled graph through the Python API, no CUDA graph; "
                         "300 untimed calls first"}

    # ---- parity of what was timed: image 0 of this rank's first operand set against the CPU oracle (outside
    # every timed region; the oracle is the checker here)
    import oracle

    ref = oracle.conv2d_torch_cpu(xs[0][:1], w, b, wl["stride"], wl["pad"], 1, 1, relu=relu)
    tol = 1e-4 if wl["dtype"] == "float32" else 1e-2
    parity_ok = bool(torch.allclose(outs[0][:1].float().cpu(), ref.float(), rtol=tol, atol=tol))
    parity_ranks = count_true_over_ranks(torch, dist, device, parity_ok)

    e2e = None
    if not args.kernel_only:
        e2e = _e2e_leg(args, torch, dist, device, compiled, xs, outs, w, b, nums, world, barrier, wl)
    stack = None
    if args.workload == "c3" and not args.kernel_only and not args.eager and not args.no_stack:
        del xs, outs, cycle, tails
        torch.cuda.empty_cache()
        stack = _stack_record(args, torch, fd, dist, device, rank, world, local_rank, peaks)
    status_word = fd.device_status()
    if rank == 0:
        _report(args, world, wl, nums, peaks, peak_src, ms_per_step, value, steps, warmup, n_sets, per_set, node_types,
                plan, launches_per_step, clocks, status_word, e2e, concurrent, sustained, eager, cpu, parity_ranks, stack)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def _e2e_leg(args, torch, dist, device, compiled, xs, outs, w, b, nums, world, barrier, wl):
    """Pinned host buffers -> device -> fused op -> host, copies inside the timed region."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # Every step copies its own input from pinned host memory and its own result back; the three
    # legs of consecutive steps overlap on three streams (input copy / compute / output copy) with
    # two buffers each, as a caller streaming batches through the API would do.
    x_host = xs[0].cpu().pin_memory()
    y_host = [torch.empty_like(outs[0], device="cpu").pin_memory() for _ in range(2)]
    x_dev = [torch.empty_like(xs[0]) for _ in range(2)]
    e2e_steps = max(3, min(args.steps, 40))
    compute = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]       # x_dev[b] holds the step's input
    ev_comp = [torch.cuda.Event() for _ in range(2)]     # the step's kernel has consumed x_dev[b]
    ev_out = [torch.cuda.Event() for _ in range(2)]      # y_host[b] holds the step's result

    def e2e_step(i):
        b_ = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_comp[b_])                  # the step two back no longer reads x_dev[b]
            x_dev[b_].copy_(x_host, non_blocking=True)
            ev_in[b_].record(s_in)
        compute.wait_event(ev_in[b_])
        y = compiled.run(x_dev[b_], w, b)
        ev_comp[b_].record(compute)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[b_])
            s_out.wait_event(ev_out[b_])
            y.record_stream(s_out)
            y_host[b_].copy_(y, non_blocking=True)
            ev_out[b_].record(s_out)

    def e2e_step_serial(i):
        x_dev[0].copy_(x_host, non_blocking=True)
        y = compiled.run(x_dev[0], w, b)
        y_host[0].copy_(y, non_blocking=True)

    def timed(step_fn):
        for i in range(4):
            step_fn(i)
        torch.cuda.synchronize()
        barrier()
        e0.record(compute)
        s_in.wait_event(e0)
        for i in range(e2e_steps):
            step_fn(i)
        compute.wait_stream(s_out)
        compute.wait_stream(s_in)
        e1.record(compute)
        torch.cuda.synchronize()
        barrier()
        return e0.elapsed_time(e1)

    # both orders of the same work are legitimate callers; keep the faster one
    candidates = max_over_ranks(torch, dist, device, [timed(e2e_step), timed(e2e_step_serial)])
    e2e_ms = min(candidates)
    result = {"value": world * nums["flops"] / (e2e_ms / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
              "h2d_bytes_per_step": nums["x_bytes"], "d2h_bytes_per_step": nums["y_bytes"], "steps": e2e_steps,
              "ms_per_step": e2e_ms / e2e_steps,
              "schedule": "copies overlapped with the neighbouring steps" if candidates[0] <= candidates[1] else "serial"}
    # the C ABI's own host-buffer entry point, fdnn_conv2d_fwd_host: serial and synchronising by contract
    # (copy in, pack when the plan asks for it, run, copy out, wait), from the same pinned buffers
    try:
        result["c_abi_host_ms"] = _c_abi_host_call_ms(torch, xs[0], x_host, w, b, y_host[0], wl)
    except Exception as exc:  # reported, never hidden: the Python-API figure above stands on its own
        result["c_abi_host_ms"] = None
        result["c_abi_host_error"] = str(exc)[:200]
    return result


def _c_abi_host_call_ms(torch, x_dev, x_host, w, b, y_host, wl, repeats=5):
    import ctypes

    from flagdnn_b200 import _native as nat

    lib = nat.load()
    d = nat.ConvDesc()
    d.dtype = {"bfloat16": nat.BF16, "float16": nat.F16, "float32": nat.F32}[wl["dtype"]]
    d.n, d.c, d.h, d.w = x_dev.shape
    d.k, _, d.r, d.s = w.shape
    d.stride_h = d.stride_w = wl["stride"]
    d.pad_top = d.pad_bottom = d.pad_left = d.pad_right = wl["pad"]
    d.dil_h = d.dil_w = 1
    d.groups = 1
    d.algo = nat.ALGO_AUTO
    w_host, b_host = w.cpu().pin_memory(), b.cpu().pin_memory()
    for i in range(4):
        d.x_strides[i], d.w_strides[i], d.y_strides[i] = x_host.stride(i), w_host.stride(i), y_host.stride(i)
    need = ctypes.c_int64(0)
    nat.check(lib.fdnn_conv2d_host_arena_bytes(ctypes.byref(d), ctypes.byref(need)))
    arena = torch.empty(need.value, dtype=torch.uint8, device=x_dev.device)
    stream = torch.cuda.current_stream().cuda_stream
    act = nat.ACT_RELU if wl["dtype"] != "float32" else nat.ACT_NONE
    times = []
    for _ in range(repeats + 1):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        nat.check(lib.fdnn_conv2d_fwd_host(ctypes.byref(d), x_host.data_ptr(), w_host.data_ptr(), b_host.data_ptr(), None,
                                           act, y_host.data_ptr(), arena.data_ptr(), need.value, stream))
        times.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(times[1:])


def _report(args, world, wl, nums, peaks, peak_src, ms_per_step, value, steps, warmup, n_sets, per_set, node_types,
            plan, launches_per_step, clocks, status_word, e2e, concurrent, sustained, eager, cpu, parity_ranks, stack):
    # ---- roofline of the dominant kernel (the implicit-GEMM kernel; one launch per step)
    if wl["bound"] == "tensor":
        achieved = nums["flops"] / (ms_per_step * 1e-3) / 1e12
        peak, unit = peaks["bf16_tflops"], "TFLOP/s"
        extra = {"frac_of_sustained_peak": achieved / peaks["bf16_tflops_sustained"]}
    else:
        achieved = nums["bytes"] / (ms_per_step * 1e-3) / 1e9
        peak, unit = peaks["hbm_gbs"], "GB/s"
        extra = {}
    roofline = {"bound": wl["bound"], "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES.get(args.workload), "peak_source": f"of {peak_src}",
                "kernel": "conv_igemm_pair_kernel" if plan["algo"] == 3 else "conv_igemm_kernel",
                "algorithmic_flops_per_launch": nums["flops"], "algorithmic_bytes_per_launch": nums["bytes"], **extra}
    if stack is not None:
        roofline["c5_strong"] = stack
    cycled_mib = n_sets * per_set / 2 ** 20
    l2_note = (f"{n_sets} rotating (x, y) sets = {cycled_mib:.0f} MiB "
               + ("> 126 MiB L2 (cold L2 every step)" if cycled_mib > 126 else "<= 126 MiB L2: WARM L2")
               + "; filter and bias shared")
    line = {
        "metric": "fused_conv2d_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": SHORT_DTYPE[wl["dtype"]], "data": "synthetic",
        "config": {"workload": args.workload, "description": wl["desc"], "graph_nodes": node_types,
                   "launch": "eager_api_calls" if args.eager else "cuda_graph_replay (each graph launched once after "
                   "capture to upload it, before the counted warm-up)", "l2": l2_note,
                   "timing": "CUDA events on the launching stream around exactly the counted steps; a 150 us spin kernel "
                             "ahead of the first event lets the CPU queue the region's launches before the GPU reaches it",
                   "per_gpu_batch": wl["n"], "parallelism": f"batch-sharded replicas x{world}, no collective",
                   "tile": [plan["tile_m"], plan["tile_n"], plan["tile_k"]], "stages": plan["stages"],
                   "grid": plan["grid"], "parity_checked_ranks": parity_ranks},
        "pct_of_bf16_peak": 100.0 * (value / world) / peaks["bf16_tflops"],
        "roofline": roofline, "cpu_baseline": cpu,
        "e2e": e2e,
        "sustained": sustained,
        "two_stream_throughput": concurrent,
        "eager_api": eager,
        "parity_checked_ranks": parity_ranks,
        "gpu_launches": steps * launches_per_step * world,
        "clocks": clocks.summary(), "device_status_word": status_word,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------ ResNet-50 conv stack (workload c5)
def stack_roofline_seconds(layers, batch, peaks):
    """Sum over layers of max(flops / tensor peak, bytes / HBM peak): the mixed roofline of the stack."""
    return sum(max(l.flops(batch) / (peaks["bf16_tflops"] * 1e12), l.bytes(batch) / (peaks["hbm_gbs"] * 1e9))
               for l in layers)


def cpu_stack_leg(torch, images, repeats=2):
    """The reference's CPU path (F.conv2d -> scale -> bias -> relu in bf16) over all 53 layers of a small batch."""
    import oracle
    from flagdnn_b200.convstack import make_layer_params, resnet50_conv_layers, stack_totals

    use_all_host_threads(torch)
    layers = resnet50_conv_layers()
    params = [make_layer_params(l, i, "cpu") for i, l in enumerate(layers)]
    g = torch.Generator().manual_seed(0)
    inputs = [torch.randn(images, l.cin, l.hw_in, l.hw_in, generator=g).to(torch.bfloat16)
              .contiguous(memory_format=torch.channels_last) for l in layers]

    def once():
        for l, (w, sc, b), x in zip(layers, params, inputs):
            oracle.conv2d_torch_cpu(x, w, b, l.stride, l.pad, 1, 1, scale=sc, relu=l.relu, compute_dtype=torch.bfloat16)

    once()
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        once()
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    return stack_totals(layers, images)["flops"] / med / 1e12, med


def _stack_device_leg(args, torch, dist, device, rank, world, local_rank, steps, warmup):
    """The 53 convolutions of this rank's batch slice replayed from one CUDA graph; returns the timing (max over
    ranks) and everything the callers report from."""
    from flagdnn_b200.convstack import make_layer_params, resnet50_conv_layers, run_layer
    from flagdnn_b200.sharding import batch_slice

    total_batch = args.batch
    b0, b1 = batch_slice(total_batch, rank, world)
    batch = b1 - b0
    layers = resnet50_conv_layers()
    params = [make_layer_params(l, i, device) for i, l in enumerate(layers)]
    # one shared pool of random activations, viewed per layer as its NHWC input
    max_in = max(batch * l.cin * l.hw_in ** 2 for l in layers)
    g = torch.Generator(device=device).manual_seed(1000 + rank)
    pool = torch.randn(max_in, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    inputs = [pool[: batch * l.cin * l.hw_in ** 2].view(batch, l.hw_in, l.hw_in, l.cin).permute(0, 3, 1, 2)
              for l in layers]

    def step(keep=None):
        out = None
        for l, prm, x in zip(layers, params, inputs):
            out = run_layer(l, x, prm)
            if keep is not None:
                keep.append(out)
        return out

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    outputs = []
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            last = step(outputs)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            graph.replay()
        stream.synchronize()
        barrier()
        with ClockSampler(local_rank) as clocks:
            e0.record(stream)
            for _ in range(steps):
                graph.replay()
            e1.record(stream)
            clocks.sample()
            stream.synchronize()
            clocks.sample()
        barrier()
    elapsed_ms = max_over_ranks(torch, dist, device, [e0.elapsed_time(e1)])[0]

    # parity of what was timed: image 0 of a spread of layers (every resolution, both filter sizes, the stem)
    # against the CPU oracle, outside the timed region
    import oracle

    parity_ok = True
    picks = {"stem", "s1b0.conv2", "s2b0.conv2", "s2b1.conv1", "s3b1.conv2", "s3b0.conv3", "s4b0.conv2", "s4b1.conv1",
             "s4b1.conv2", "s4b0.proj"}
    for l, (w_, sc, bi), x, y in zip(layers, params, inputs, outputs):
        if l.name not in picks:
            continue
        ref = oracle.conv2d_torch_cpu(x[:1], w_, bi, l.stride, l.pad, 1, 1, scale=sc, relu=l.relu)
        parity_ok = parity_ok and bool(torch.allclose(y[:1].float().cpu(), ref, rtol=1e-2, atol=1e-2))
    parity_ranks = count_true_over_ranks(torch, dist, device, parity_ok)
    return dict(ms_per_step=elapsed_ms / steps, batch=batch, total_batch=total_batch, layers=layers, params=params,
                inputs=inputs, last=last, clocks=clocks, barrier=barrier, parity_ranks=parity_ranks,
                parity_layers=len(picks))


def _stack_record(args, torch, fd, dist, device, rank, world, local_rank, peaks):
    """Compact strong-scaled record of the ResNet-50 stack (batch 1024 over all ranks) for the default line."""
    from flagdnn_b200.convstack import stack_totals

    leg = _stack_device_leg(args, torch, dist, device, rank, world, local_rank, steps=10, warmup=3)
    totals = stack_totals(leg["layers"], leg["total_batch"])
    roof_s = stack_roofline_seconds(leg["layers"], leg["batch"], peaks)
    ms = leg["ms_per_step"]
    return {"workload": "c5", "scaling": "strong", "total_batch": leg["total_batch"], "per_gpu_batch": leg["batch"],
            "n_gpus": world, "steps": 10, "warmup": 3, "ms_per_step": ms,
            "value": totals["flops"] / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
            "frac_of_mixed_roofline": roof_s * 1e3 / ms, "mixed_roofline_ms": roof_s * 1e3,
            "parity_checked_ranks": leg["parity_ranks"], "parity_checked_layers": leg["parity_layers"],
            "clocks": leg["clocks"].summary()}


def run_stack(args):
    """All 53 ResNet-50 convolutions (scale + bias + ReLU fused), batch 1024 split over the ranks (strong scaling).
    Every layer runs on an independently generated N(0,1) input of its own shape, so only convolutions are timed."""
    import torch

    import flagdnn_b200 as fd
    from flagdnn_b200.convstack import run_layer, stack_totals

    rank, world, local_rank, dist, cpu_stack = init_ranks(torch, lambda: cpu_stack_leg(torch, images=2))
    device = torch.device("cuda", local_rank)
    peaks, peak_src = load_peaks()
    steps = max(1, args.steps)
    leg = _stack_device_leg(args, torch, dist, device, rank, world, local_rank, steps=steps, warmup=max(args.warmup, 3))
    layers, params, inputs, last, clocks, barrier = (leg[k] for k in ("layers", "params", "inputs", "last", "clocks", "barrier"))
    batch, total_batch, ms_per_step = leg["batch"], leg["total_batch"], leg["ms_per_step"]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    totals = stack_totals(layers, total_batch)
    value = totals["flops"] / (ms_per_step * 1e-3) / 1e12

    # per-shape times (rank 0, outside the timed region) for the breakdown
    shape_ms = {}
    if rank == 0:
        for l, prm, x in zip(layers, params, inputs):
            if l.shape_key in shape_ms:
                continue
            run_layer(l, x, prm)
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(3):
                run_layer(l, x, prm)
            b.record()
            torch.cuda.synchronize()
            shape_ms[l.shape_key] = (l, a.elapsed_time(b) / 3)

    # end to end: images from pinned host memory in, the real chained forward (max-pool after the stem, each
    # block's shortcut add + ReLU inside its last convolution), last activation back out
    from flagdnn_b200.convstack import ResNet50ConvStack

    chain = ResNet50ConvStack.__new__(ResNet50ConvStack)
    chain.layers, chain.params = layers, params
    x_host = inputs[0].contiguous(memory_format=torch.channels_last).cpu().pin_memory()
    x_dev = torch.empty_like(x_host, device=device)
    y_host = torch.empty(last.shape, dtype=last.dtype).contiguous(memory_format=torch.channels_last).pin_memory()

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)
        y_host.copy_(chain.forward(x_dev, fuse_residual=True), non_blocking=True)

    e2e_step()
    barrier()
    e2e_steps = 3
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps

    # the same steps with the copies on their own streams and two input / output buffers, so that the copy-in of
    # step i+1 and the copy-out of step i-1 overlap the forward of step i (every step still copies in and out)
    comp, s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    x_bufs = [x_dev, torch.empty_like(x_dev)]
    y_hosts = [y_host, torch.empty_like(y_host).pin_memory()]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def piped_step(i):
        b_ = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_done[b_])                      # the forward two steps back has consumed x_bufs[b_]
            x_bufs[b_].copy_(x_host, non_blocking=True)
            ev_in[b_].record(s_in)
        with torch.cuda.stream(comp):
            comp.wait_event(ev_in[b_])
            y = chain.forward(x_bufs[b_], fuse_residual=True)
            ev_done[b_].record(comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[b_])
            s_out.wait_event(ev_out[b_])
            y.record_stream(s_out)
            y_hosts[b_].copy_(y, non_blocking=True)
            ev_out[b_].record(s_out)

    piped_steps = 6
    for i in range(2):
        piped_step(i)
    torch.cuda.synchronize()
    barrier()
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p0.record(comp)
    s_in.wait_event(p0)
    for i in range(piped_steps):
        piped_step(i)
    comp.wait_stream(s_in)
    comp.wait_stream(s_out)
    p1.record(comp)
    torch.cuda.synchronize()
    barrier()
    piped_ms = p0.elapsed_time(p1) / piped_steps
    e2e_mode = "serial"
    if piped_ms < e2e_ms:
        e2e_ms, e2e_steps, e2e_mode = piped_ms, piped_steps, "copies overlapped with the neighbouring steps' forward"
    e2e_ms = max_over_ranks(torch, dist, device, [e2e_ms])[0]
    status_word = fd.device_status()

    if rank == 0:
        roof_s = stack_roofline_seconds(layers, batch, peaks)
        launches = sum(fd.conv2d_plan(x, p_[0], stride=l.stride, padding=l.pad)["launches"]
                       for l, p_, x in zip(layers, params, inputs))
        slow = sorted(shape_ms.values(), key=lambda t: -t[1])[:6]
        cpu_value, cpu_s = cpu_stack
        line = {
            "metric": "fused_conv2d_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "c5", "description": "ResNet-50 forward conv stack, 53 convs with folded scale+bias(+ReLU), "
                       f"bf16 NHWC 224x224, batch {total_batch} sharded along N", "per_gpu_batch": batch,
                       "inputs": "each layer reads independently generated N(0,1) activations of its shape; "
                                 "no pooling / residual glue in the timed region",
                       "launch": "cuda_graph_replay", "l2": "activations of every layer exceed the 126 MiB L2",
                       "parallelism": f"batch-sharded replicas x{world}, no collective",
                       "parity_checked_ranks": leg["parity_ranks"], "parity_checked_layers": leg["parity_layers"]},
            "pct_of_bf16_peak": 100.0 * (value / world) / peaks["bf16_tflops"],
            "parity_checked_ranks": leg["parity_ranks"],
            "roofline": {"bound": "mixed", "achieved": roof_s * 1e3, "peak": ms_per_step, "unit": "ms",
                         "frac": roof_s * 1e3 / ms_per_step, "traffic": None, "peak_source": f"of {peak_src}",
                         "note": "achieved = sum over layers of max(flops/tensor peak, bytes/HBM peak) for this rank's "
                                 "batch; peak = measured ms per step; frac = roofline time / measured time",
                         "slowest_shapes_ms": [{"layer": l.name, "cin": l.cin, "hw": l.hw_in, "cout": l.cout, "k": l.k,
                                                "stride": l.stride, "ms": ms,
                                                "tflops": l.flops(batch) / ms / 1e9} for l, ms in slow]},
            "cpu_baseline": {"value": cpu_value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": f"2 of {total_batch} images through all 53 layers, F.conv2d*scale+bias+relu in "
                                       f"bf16 on CPU, median of 2 ({cpu_s:.2f} s per pass)"},
            "e2e": {"value": totals["flops"] / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": y_host.numel() * 2,
                    "steps": e2e_steps, "ms_per_step": e2e_ms,
                    "path": "chained forward: stem, max-pool, 16 blocks with the shortcut add + ReLU fused into "
                            "each block's last convolution", "schedule": e2e_mode},
            "gpu_launches": steps * launches * world, "clocks": clocks.summary(), "device_status_word": status_word,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_stack_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch

    value, seconds = cpu_stack_leg(torch, images=2, repeats=max(1, min(args.steps, 3)))
    sample = ("each step = 2 images through all 53 ResNet-50 convolutions, F.conv2d*scale+bias+relu in bf16 on the host CPU")
    print(json.dumps({
        "impl": "reference", "metric": "fused_conv2d_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": max(1, min(args.steps, 3)), "warmup": 1, "ms_per_step": seconds * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "c5", "sample_images": 2},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}))


# ------------------------------------------------------------------ rows next to the path: block tail, mm
EXTRA = {
    # a ResNet block's last layer: 1x1 conv 64->256 at 56x56, folded scale + bias, shortcut add, ReLU, one kernel
    "res": dict(desc="1x1 conv 64->256 56x56 N=256 bf16 NHWC + scale + bias + shortcut add + ReLU (one kernel)",
                bound="hbm"),
    # mm on the same kernels: a 1x1 convolution over a row of M pixels
    "mm": dict(desc="mm bf16 [8192 x 4096] @ [4096 x 4096] as a 1x1 convolution over a row of M pixels",
               bound="tensor"),
    # depthwise 3x3 at 64 channels, 56 x 56 (the shape of benchmark/test_conv2d_perf.py:51 of the reference at a
    # batch larger than L2), NCHW as the reference benchmarks it and channels-last
    "dw": dict(desc="depthwise 3x3 conv (groups = C = K = 64) 56x56 N=256 bf16 NCHW + bias, stride 1 pad 1",
               bound="hbm"),
    "dwcl": dict(desc="depthwise 3x3 conv (groups = C = K = 64) 56x56 N=256 bf16 channels-last + bias, stride 1 pad 1",
                 bound="hbm"),
    # a grouped layer the reference times (benchmark/test_conv2d_perf.py:48) at a batch larger than L2: two groups
    # of 32 -> 64 channels, one tensor-core launch per group
    "grp": dict(desc="grouped 3x3 conv 64->128, groups = 2, 56x56 N=256 bf16 channels-last + bias, stride 1 pad 1",
                bound="hbm"),
}


def run_extra(args):
    """One JSON line for a row next to the hot path, same timing rules (cold L2, CUDA graph, events, clocks)."""
    import torch

    import flagdnn_b200 as fd

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise RuntimeError("the 'res', 'mm' and 'dw' workloads are single-GPU measurements")
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    wl = EXTRA[args.workload]
    peaks, peak_src = load_peaks()
    bf = torch.bfloat16
    g = torch.Generator(device=device).manual_seed(0)

    def rnd(*shape, std=1.0):
        return (torch.randn(*shape, generator=g, device=device) * std).to(bf)

    if args.workload == "res":
        n, c, hw, k = 256, 64, 56, 256
        w = rnd(k, 1, 1, c, std=c ** -0.5).permute(0, 3, 1, 2)
        scale, bias = (torch.rand(k, generator=g, device=device) + 0.5).to(bf), rnd(k, std=0.1)
        per_set = 2 * n * hw * hw * (c + 2 * k)
        n_sets = max(2, -(-3 * 126 * 2 ** 20 // per_set))
        sets = [(rnd(n, hw, hw, c).permute(0, 3, 1, 2), rnd(n, hw, hw, k).permute(0, 3, 1, 2)) for _ in range(n_sets)]
        flops = 2.0 * n * hw * hw * k * c
        nbytes = per_set + 2 * (k * c + 2 * k)

        def step(i):
            x, shortcut = sets[i]
            return fd.conv2d_bias_act(x, w, bias, scale=scale, relu=True, residual=shortcut)

        def cpu_once(m):
            import oracle

            x, shortcut = sets[0][0][:m].cpu(), sets[0][1][:m].cpu()
            wc, sc, bc = w.cpu(), scale.cpu(), bias.cpu()

            def run():
                y = oracle.conv2d_torch_cpu(x, wc, bc, 1, 0, 1, 1, scale=sc, compute_dtype=bf)
                return torch.relu(y + shortcut)
            return run, 2.0 * m * hw * hw * k * c, f"{m} of {n} images, conv2d*scale+bias, add, relu in bf16 on CPU"
        h2d, d2h = 2 * n * hw * hw * (c + k), 2 * n * hw * hw * k
        host_in = [t.contiguous(memory_format=torch.channels_last).cpu().pin_memory() for t in sets[0]]
    elif args.workload in ("dw", "dwcl", "grp"):
        n, c, hw = 256, 64, 56
        cl = args.workload != "dw"
        groups, k = (2, 128) if args.workload == "grp" else (c, c)
        w = rnd(k, c // groups, 3, 3, std=(9 * c // groups) ** -0.5)
        if cl:
            w = w.contiguous(memory_format=torch.channels_last)
        bias = rnd(k, std=0.1)
        per_set = 2 * n * (c + k) * hw * hw
        n_sets = max(2, -(-3 * 126 * 2 ** 20 // per_set))

        def make_x():
            x = rnd(n, c, hw, hw)
            return x.contiguous(memory_format=torch.channels_last) if cl else x
        sets = [(make_x(),) for _ in range(n_sets)]
        flops = 2.0 * n * k * (c // groups) * hw * hw * 9
        nbytes = per_set + 2 * (k * (c // groups) * 9 + k)

        def step(i):
            return fd.conv2d(sets[i][0], w, bias, stride=1, padding=1, groups=groups)

        def cpu_once(m):
            import oracle

            x, wc, bc = sets[0][0][:m].cpu(), w.cpu(), bias.cpu()
            return ((lambda: oracle.conv2d_torch_cpu(x, wc, bc, 1, 1, 1, groups, compute_dtype=bf)),
                    2.0 * m * k * (c // groups) * hw * hw * 9,
                    f"{m} of {n} images, F.conv2d(groups={groups}) in bf16 on CPU")
        h2d, d2h = 2 * n * c * hw * hw, 2 * n * k * hw * hw
        host_in = [sets[0][0].cpu().pin_memory()]
    else:
        m_, k_, n_ = 8192, 4096, 4096
        b_mat = rnd(k_, n_, std=k_ ** -0.5)
        per_set = 2 * (m_ * k_ + m_ * n_)
        n_sets = max(2, -(-3 * 126 * 2 ** 20 // per_set))
        sets = [(rnd(m_, k_),) for _ in range(n_sets)]
        flops = 2.0 * m_ * k_ * n_
        nbytes = per_set + 2 * k_ * n_

        def step(i):
            return fd.mm(sets[i][0], b_mat)

        def cpu_once(m):
            a, bc = sets[0][0][:m].cpu(), b_mat.cpu()
            return (lambda: torch.mm(a, bc)), 2.0 * m * k_ * n_, f"{m} of {m_} rows, torch.mm in bf16 on CPU"
        h2d, d2h = 2 * m_ * k_, 2 * m_ * n_
        host_in = [sets[0][0].cpu().pin_memory()]

    for i in range(n_sets):
        out = step(i)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        step(0)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(n_sets):
                out = step(i)
        replays = max(1, -(-min(args.steps, 400) // n_sets))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(max(1, -(-max(args.warmup, 3) // n_sets))):
            graph.replay()
        stream.synchronize()
        with ClockSampler(0) as clocks:
            e0.record(stream)
            for _ in range(replays):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
    steps = replays * n_sets
    ms_per_step = e0.elapsed_time(e1) / steps

    # end to end: operands from pinned host memory, the result back, every step
    dev_in = [torch.empty_like(t, device=device) for t in host_in]
    host_out = torch.empty_like(out, device="cpu").pin_memory()   # keeps the result's memory format

    def e2e_step():
        for d, h in zip(dev_in, host_in):
            d.copy_(h, non_blocking=True)
        if args.workload == "res":
            y = fd.conv2d_bias_act(dev_in[0], w, bias, scale=scale, relu=True, residual=dev_in[1])
        elif args.workload in ("dw", "dwcl", "grp"):
            y = fd.conv2d(dev_in[0], w, bias, stride=1, padding=1, groups=groups)
        else:
            y = fd.mm(dev_in[0], b_mat)
        host_out.copy_(y, non_blocking=True)

    e2e_step()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(5):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / 5

    use_all_host_threads(torch)
    run, cpu_flops, sample = cpu_once(256 if args.workload == "mm" else 8)
    run()
    times, t_all = [], time.perf_counter()
    while len(times) < 3 or time.perf_counter() - t_all < 10.0:
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
    cpu_med = statistics.median(times)

    value = flops / (ms_per_step * 1e-3) / 1e12
    if wl["bound"] == "tensor":
        achieved, peak, unit = value, peaks["bf16_tflops"], "TFLOP/s"
    else:
        achieved, peak, unit = nbytes / (ms_per_step * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
    print(json.dumps({
        "metric": "fused_conv2d_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": args.workload, "description": wl["desc"], "launch": "cuda_graph_replay",
                   "l2": f"{n_sets} rotating operand sets = {n_sets * per_set / 2**20:.0f} MiB > 126 MiB L2"},
        "roofline": {"bound": wl["bound"], "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                     "traffic": None, "peak_source": f"of {peak_src}", "algorithmic_flops_per_launch": flops,
                     "algorithmic_bytes_per_launch": nbytes},
        "cpu_baseline": {"value": cpu_flops / cpu_med / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": f"{sample}, {len(times)} repeats, median"},
        "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": 5, "ms_per_step": e2e_ms},
        "gpu_launches": steps, "clocks": clocks.summary(),
        "device_status_word": fd.device_status(),
    }))


# ------------------------------------------------------------------ the reference's own GPU path (informative arm)
def _import_reference_gpu():
    """Imports the UNMODIFIED reference from baseline/_ref (installed there with pip, not tracked).  Three things it
    needs are supplied from outside without touching its files: an empty stand-in for the `sqlalchemy` package (its
    autotune cache is the only user), FLAGGEMS_DB_URL and DNN_VENDOR=nvidia; its SQL-backed store of tuned
    configurations is then replaced by a dict-backed one with the same interface (utils/models/model.py:9-88)."""
    import tempfile
    from pathlib import Path

    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "flag_dnn")):
        raise FileNotFoundError("baseline/_ref/flag_dnn is missing (pip install --target baseline/_ref <reference>)")
    stub_dir = tempfile.mkdtemp(prefix="sqlalchemy_stub_")
    any_src = ("class _Any:\n    def __init__(self, *a, **k): pass\n    def __call__(self, *a, **k): return _Any()\n"
               "    def __getattr__(self, n): return _Any()\n    def __getitem__(self, n): return _Any()\n"
               "def __getattr__(name): return _Any()\n")
    for sub in ("", "orm", "ext", "ext/automap", "engine", "exc", "schema"):
        d = Path(stub_dir) / "sqlalchemy" / sub
        d.mkdir(parents=True, exist_ok=True)
        (d / "__init__.py").write_text(any_src)
    (Path(stub_dir) / "sqlalchemy" / "orm" / "__init__.py").write_text(any_src + "class DeclarativeBase: pass\nclass Session: pass\n")
    (Path(stub_dir) / "sqlalchemy" / "exc" / "__init__.py").write_text(any_src + "class IntegrityError(Exception): pass\n")
    os.environ.setdefault("FLAGGEMS_DB_URL", "sqlite:///" + os.path.join(stub_dir, "tune.db"))
    os.environ.setdefault("DNN_VENDOR", "nvidia")
    sys.dont_write_bytecode = True
    sys.path.insert(0, stub_dir)
    sys.path.insert(0, ref_dir)
    import importlib

    import flag_dnn

    libentry = importlib.import_module("flag_dnn.utils.libentry")
    from flag_dnn.utils.models.model import PersistantModel

    class DictModel(PersistantModel):
        def __init__(self):
            super().__init__()
            self.configs, self.benchmarks = {}, {}

        def get_config(self, name, key):
            return self.configs.get((name, tuple(key)))

        def put_config(self, name, keys, config):
            self.configs[(name, tuple(keys))] = config

        def get_benchmark(self, name, keys, config):
            return self.benchmarks.get((name, tuple(keys), str(config)))

        def put_benchmark(self, name, keys, config, benchmark):
            self.benchmarks[(name, tuple(keys), str(config))] = benchmark

    model = DictModel()
    libentry.libcache.model = model
    for cache in list(libentry.libcache.config_cache_pool.values()) + list(libentry.libcache.benchmark_cache_pool.values()):
        cache.model = model
    return flag_dnn


def run_reference_gpu(args):
    """The reference's own kernels on this GPU, for the record beside ours: eager flag_dnn.ops.conv2d for the fp32
    configuration (src/flag_dnn/ops/conv2d.py:3575, autotuned Triton kernels), the compiled conv -> bias_add -> relu
    graph for the others (src/flag_dnn/graph/capture.py:127 -> src/flag_dnn/graph/kernels/fused_conv.py:62, one
    Triton kernel with a fixed 64x32x32 tile).  Same seeded inputs, rotating operand sets and CUDA events as our arm;
    first calls (JIT compilation and autotuning) are outside the timed region."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch

    wl = WORKLOADS[args.workload]
    base = {"impl": "reference-gpu", "metric": "fused_conv2d_tflops", "unit": "TFLOP/s", "n_gpus": 1,
            "higher_is_better": True, "dtype": SHORT_DTYPE[wl["dtype"]], "data": "synthetic",
            "config": {"workload": args.workload, "description": wl["desc"]}}
    try:
        flag_dnn = _import_reference_gpu()
    except Exception as exc:
        print(json.dumps(dict(base, unavailable=f"{type(exc).__name__}: {str(exc)[:200]}")))
        return
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    nums = workload_numbers(wl)
    relu = wl["dtype"] != "float32"
    per_set = nums["x_bytes"] + nums["y_bytes"]
    n_sets = max(2, min(64, -(-3 * 126 * 2 ** 20 // per_set)))
    xs, w, b = [], None, None
    for i in range(n_sets):
        x, w_i, b_i = make_inputs(wl, wl["n"], i, device, torch)
        xs.append(x)
        if w is None:
            w, b = w_i, b_i
    try:
        if relu:
            def layer(x, weight, bias):
                return flag_dnn.relu(flag_dnn.bias_add(flag_dnn.conv2d(x, weight, stride=wl["stride"], padding=wl["pad"]), bias))

            compiled = flag_dnn.compile(layer, inputs=[xs[0], w, b], options={"cache": None})
            nodes = [n.op_type for n in compiled.graph.nodes]
            call = lambda x: compiled.run(x, w, b)
        else:
            nodes = ["eager conv2d"]
            call = lambda x: flag_dnn.ops.conv2d(x, w, b, stride=wl["stride"], padding=wl["pad"])
        t_first = time.perf_counter()
        y0 = call(xs[0])
        torch.cuda.synchronize()
        first_call_s = time.perf_counter() - t_first
        for i in range(max(3, args.warmup)):
            call(xs[i % n_sets])
        torch.cuda.synchronize()
        steps = max(1, min(args.steps, 400))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(0) as clocks:
            e0.record()
            for i in range(steps):
                call(xs[i % n_sets])
            e1.record()
            clocks.sample()
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
    except Exception as exc:
        print(json.dumps(dict(base, unavailable=f"the reference's GPU path failed: {type(exc).__name__}: {str(exc)[:300]}")))
        return
    import oracle

    ref = oracle.conv2d_torch_cpu(xs[0][:1], w, b, wl["stride"], wl["pad"], 1, 1, relu=relu)
    err = float((y0[:1].float().cpu() - ref).abs().max())
    peaks, peak_src = load_peaks()
    value = nums["flops"] / (ms * 1e-3) / 1e12
    print(json.dumps(dict(
        base, value=value, steps=steps, warmup=max(3, args.warmup), ms_per_step=ms, scaling="weak", vs_baseline=None,
        graph_nodes=nodes, first_call_seconds=first_call_s, launch="eager calls through the reference's public API",
        l2=f"{n_sets} rotating (x, y) sets", pct_of_bf16_peak=100.0 * value / peaks["bf16_tflops"],
        hbm_gbs=nums["bytes"] / (ms * 1e-3) / 1e9, max_abs_err_image0_vs_fp32_oracle=err,
        note="single-pass TF32 for fp32 tensors (src/flag_dnn/ops/conv2d.py:1471), so the fp32 configuration does "
             "not meet 1e-4 against the fp32 oracle by design" if not relu else None,
        clocks=clocks.summary(), gpu_launches=0)))


def run_reference_gpu_extra(args):
    """The reference's eager conv2d on the depthwise / grouped workloads (its Triton depthwise kernels,
    src/flag_dnn/ops/conv2d.py:2613 and :3089, and its grouped path), same tensors and timing as run_extra."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    import torch

    base = {"impl": "reference-gpu", "metric": "fused_conv2d_tflops", "unit": "TFLOP/s", "n_gpus": 1,
            "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.workload, "description": EXTRA[args.workload]["desc"]}}
    try:
        flag_dnn = _import_reference_gpu()
    except Exception as exc:
        print(json.dumps(dict(base, unavailable=f"{type(exc).__name__}: {str(exc)[:200]}")))
        return
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    g = torch.Generator(device=device).manual_seed(4321)
    n, c, hw = 256, 64, 56
    cl = args.workload != "dw"
    groups, k = (2, 128) if args.workload == "grp" else (c, c)

    def rnd(*shape, std=1.0):
        return (torch.randn(*shape, generator=g, device=device) * std).to(torch.bfloat16)

    w = rnd(k, c // groups, 3, 3, std=(9 * c // groups) ** -0.5)
    if cl:
        w = w.contiguous(memory_format=torch.channels_last)
    bias = rnd(k, std=0.1)
    per_set = 2 * n * (c + k) * hw * hw
    n_sets = max(2, -(-3 * 126 * 2 ** 20 // per_set))
    xs = [rnd(n, c, hw, hw) for _ in range(n_sets)]
    if cl:
        xs = [x.contiguous(memory_format=torch.channels_last) for x in xs]
    try:
        call = lambda x: flag_dnn.ops.conv2d(x, w, bias, stride=1, padding=1, groups=groups)
        t_first = time.perf_counter()
        y0 = call(xs[0])
        torch.cuda.synchronize()
        first_call_s = time.perf_counter() - t_first
        for i in range(max(3, args.warmup)):
            call(xs[i % n_sets])
        torch.cuda.synchronize()
        steps = max(1, min(args.steps, 200))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            call(xs[i % n_sets])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
    except Exception as exc:
        print(json.dumps(dict(base, unavailable=f"the reference's GPU path failed: {type(exc).__name__}: {str(exc)[:300]}")))
        return
    import oracle

    ref = oracle.conv2d_torch_cpu(xs[0][:1], w, bias, 1, 1, 1, groups)
    err = float((y0[:1].float().cpu() - ref).abs().max())
    flops = 2.0 * n * k * (c // groups) * hw * hw * 9
    nbytes = per_set + 2 * (k * (c // groups) * 9 + k)
    print(json.dumps(dict(
        base, value=flops / (ms * 1e-3) / 1e12, steps=steps, warmup=max(3, args.warmup), ms_per_step=ms,
        scaling="weak", vs_baseline=None, first_call_seconds=first_call_s,
        launch="eager calls through the reference's public API", l2=f"{n_sets} rotating x sets",
        hbm_gbs=nbytes / (ms * 1e-3) / 1e9, max_abs_err_image0_vs_fp32_oracle=err, gpu_launches=0)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS) + ["c5"] + sorted(EXTRA))
    ap.add_argument("--batch", type=int, default=1024, help="total batch of the c5 workload (split over the ranks)")
    ap.add_argument("--eager", action="store_true",
                    help="launch every step through the API instead of replaying a CUDA graph (for profilers)")
    ap.add_argument("--no-stack", action="store_true",
                    help="default workload only: leave out the nested strong-scaled ResNet-50 record (roofline.c5_strong)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end and CPU-baseline legs (short runs under a profiler)")
    args = ap.parse_args()
    if args.impl == "reference-gpu":
        if args.workload in ("dw", "dwcl", "grp"):
            run_reference_gpu_extra(args)
            return
        if args.workload not in WORKLOADS:
            raise SystemExit("--impl reference-gpu measures the single-layer workloads c1..c4, dw, dwcl and grp")
        run_reference_gpu(args)
        return
    if args.workload in EXTRA:
        if args.impl == "reference":
            raise SystemExit("the 'res' and 'mm' workloads report their CPU leg in the same line (cpu_baseline)")
        run_extra(args)
    elif args.workload == "c5":
        if args.impl == "reference":
            run_stack_reference(args)
        else:
            if args.steps == 2000:
                args.steps = 20  # a pass over the whole stack takes milliseconds, not microseconds
            run_stack(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

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
NCU_TRAFFIC_BYTES = {"c3": 26.96e6, "c2": 495.5e6, "c4": 459.0e6, "c1": None}

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
    """Samples SM clock and throttle reasons through NVML while a region runs."""

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
        except Exception:
            self._nvml = None

    def _loop(self):
        nv = self._nvml
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
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


def cpu_baseline_leg(wl, torch, sample_n, min_seconds=10.0):
    """The reference's CPU path timed on the host cores; test-infrastructure code (oracle/) as the checker's timer."""
    import oracle

    use_all_host_threads(torch)

    x, w, b = make_inputs(wl, sample_n, 0, "cpu", torch)
    relu = wl["dtype"] != "float32"
    cdt = getattr(torch, wl["dtype"])  # the reference runs F.conv2d in the tensors' own dtype
    oracle.conv2d_torch_cpu(x, w, b, wl["stride"], wl["pad"], 1, 1, relu=relu, compute_dtype=cdt)
    times, t_all = [], time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t_all < min_seconds and len(times) < 5000):
        t0 = time.perf_counter()
        oracle.conv2d_torch_cpu(x, w, b, wl["stride"], wl["pad"], 1, 1, relu=relu, compute_dtype=cdt)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    nums = workload_numbers(dict(wl, n=sample_n))
    return dict(value=nums["flops"] / med / 1e12, unit="TFLOP/s", cores=torch.get_num_threads(), kind="port",
                sample=f"{sample_n} of {wl['n']} images, {len(times)} repeats, median; torch.nn.functional.conv2d+relu "
                       f"in {wl['dtype']} on CPU (the call the reference's CPU graph path makes)",
                ms_per_sample=med * 1e3)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    use_all_host_threads(torch)
    wl = WORKLOADS[args.workload]
    sample_n = min(wl["n"], 32)
    nums = workload_numbers(dict(wl, n=sample_n))
    import oracle

    x, w, b = make_inputs(wl, sample_n, 0, "cpu", torch)
    relu = wl["dtype"] != "float32"
    cdt = getattr(torch, wl["dtype"])
    for _ in range(max(args.warmup, 1)):
        oracle.conv2d_torch_cpu(x, w, b, wl["stride"], wl["pad"], 1, 1, relu=relu, compute_dtype=cdt)
    steps = max(1, min(args.steps, 50))
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.conv2d_torch_cpu(x, w, b, wl["stride"], wl["pad"], 1, 1, relu=relu, compute_dtype=cdt)
    dt = (time.perf_counter() - t0) / steps
    value = nums["flops"] / dt / 1e12
    sample = (f"each step = {sample_n} of {wl['n']} images through torch.nn.functional.conv2d+relu in {wl['dtype']} "
              f"on the host CPU (the reference's CPU graph path); {steps} steps timed")
    line = {
        "impl": "reference", "metric": "fused_conv2d_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": SHORT_DTYPE[wl["dtype"]], "data": "synthetic",
        "config": {"workload": args.workload, "description": wl["desc"], "sample_images": sample_n},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def run_ours(args):
    import torch

    import flagdnn_b200 as fd

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU path for this library)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    device = torch.device("cuda", local_rank)
    wl = WORKLOADS[args.workload]
    nums = workload_numbers(wl)
    peaks, peak_src = load_peaks()
    relu = wl["dtype"] != "float32"

    # ---- operands: enough rotating (x, y) sets that a set is evicted from L2 before it is reused
    l2_bytes = 126 * 1024 * 1024
    per_set = nums["x_bytes"] + nums["y_bytes"]
    n_sets = max(2, min(16, -(-3 * l2_bytes // per_set)))
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

    # warm-up through the eager API (also packs the filter and sets kernel attributes)
    for i in range(max(args.warmup, 3)):
        compiled.run(xs[i % n_sets], w, b)
    torch.cuda.synchronize()

    # ---- device-resident leg: one CUDA graph holding one step per operand set
    stream = torch.cuda.Stream()
    outs = []

    class _EagerCycle:
        def replay(self):
            for i in range(n_sets):
                compiled.run(xs[i], w, b)

    with torch.cuda.stream(stream):
        for i in range(n_sets):
            out = compiled.run(xs[i], w, b)
            if args.eager:
                outs.append(out)
        stream.synchronize()
        if args.eager:
            graph = _EagerCycle()
        else:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(n_sets):
                    outs.append(compiled.run(xs[i], w, b))
    replays = max(1, -(-args.steps // n_sets))
    steps = replays * n_sets
    warm_replays = max(1, -(-max(args.warmup, 3) // n_sets))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        for _ in range(warm_replays):
            graph.replay()
        stream.synchronize()
        barrier()
        with ClockSampler(local_rank) as clocks:
            e0.record(stream)
            for _ in range(replays):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
        barrier()
    elapsed_ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / steps
    value = world * nums["flops"] / (ms_per_step * 1e-3) / 1e12

    # ---- the same steps with two streams: independent batches overlap, so the SMs that idle through the last
    # partial wave of tiles of one launch start the next launch's tiles (reported beside `value`, not as it:
    # `value` and the roofline stay the serial per-launch figures)
    concurrent = None
    if not args.eager and n_sets >= 2:
        side = torch.cuda.Stream()
        graph2 = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph2, stream=stream):
                side.wait_stream(stream)
                for i in range(n_sets):
                    with torch.cuda.stream(side if i % 2 else stream):
                        compiled.run(xs[i], w, b)
                stream.wait_stream(side)
            for _ in range(warm_replays):
                graph2.replay()
            stream.synchronize()
            barrier()
            e0.record(stream)
            for _ in range(replays):
                graph2.replay()
            e1.record(stream)
            stream.synchronize()
            barrier()
        c_ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([c_ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            c_ms = float(t.item())
        concurrent = {"streams": 2, "ms_per_step": c_ms / steps,
                      "value": world * nums["flops"] / (c_ms / steps * 1e-3) / 1e12, "unit": "TFLOP/s"}

    e2e_value = e2e_ms = None
    e2e_steps = 0
    if not args.kernel_only:
        e2e_value, e2e_ms, e2e_steps = _e2e_leg(args, torch, dist, device, compiled, xs, outs, w, b, nums, world, barrier)
    status_word = fd.device_status()
    _report(args, torch, rank, world, wl, nums, peaks, peak_src, ms_per_step, value, steps, warm_replays, n_sets,
            per_set, node_types, plan, launches_per_step, clocks, status_word, e2e_value, e2e_ms, e2e_steps, concurrent)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def _e2e_leg(args, torch, dist, device, compiled, xs, outs, w, b, nums, world, barrier):
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
    e2e_ms_candidates = [timed(e2e_step), timed(e2e_step_serial)]
    if dist is not None:
        t = torch.tensor(e2e_ms_candidates, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms_candidates = [float(v) for v in t.tolist()]
    e2e_ms = min(e2e_ms_candidates)
    e2e_value = world * nums["flops"] / (e2e_ms / e2e_steps * 1e-3) / 1e12
    return e2e_value, e2e_ms, e2e_steps


def _report(args, torch, rank, world, wl, nums, peaks, peak_src, ms_per_step, value, steps, warm_replays, n_sets,
            per_set, node_types, plan, launches_per_step, clocks, status_word, e2e_value, e2e_ms, e2e_steps,
            concurrent=None):
    if rank == 0:
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
                    "kernel": "conv_igemm_pair_kernel" if plan["algo"] == 3 else "conv_igemm_kernel", "algorithmic_flops_per_launch": nums["flops"],
                    "algorithmic_bytes_per_launch": nums["bytes"], **extra}
        cpu = None if args.kernel_only else cpu_baseline_leg(wl, torch, sample_n=min(wl["n"], 32))
        e2e = None if e2e_value is None else {
            "value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": nums["x_bytes"],
            "d2h_bytes_per_step": nums["y_bytes"], "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps}
        line = {
            "metric": "fused_conv2d_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warm_replays * n_sets, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": SHORT_DTYPE[wl["dtype"]], "data": "synthetic",
            "config": {"workload": args.workload, "description": wl["desc"], "graph_nodes": node_types,
                       "launch": "eager_api_calls" if args.eager else "cuda_graph_replay", "l2": f"{n_sets} rotating (x, y) sets = "
                       f"{n_sets * per_set / 2**20:.0f} MiB > 126 MiB L2; filter and bias shared",
                       "per_gpu_batch": wl["n"], "parallelism": f"batch-sharded replicas x{world}, no collective",
                       "tile": [plan["tile_m"], plan["tile_n"], plan["tile_k"]], "stages": plan["stages"],
                       "grid": plan["grid"]},
            "pct_of_bf16_peak": 100.0 * (value / world) / peaks["bf16_tflops"],
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": e2e,
            "two_stream_throughput": concurrent,
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


def run_stack(args):
    """All 53 ResNet-50 convolutions (scale + bias + ReLU fused), batch 1024 split over the ranks (strong scaling).
    Every layer runs on an independently generated N(0,1) input of its own shape, so only convolutions are timed."""
    import torch

    import flagdnn_b200 as fd
    from flagdnn_b200.convstack import make_layer_params, resnet50_conv_layers, run_layer, stack_totals

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    device = torch.device("cuda", local_rank)
    from flagdnn_b200.sharding import batch_slice

    total_batch = args.batch
    b0, b1 = batch_slice(total_batch, rank, world)
    batch = b1 - b0
    layers = resnet50_conv_layers()
    params = [make_layer_params(l, i, device) for i, l in enumerate(layers)]
    peaks, peak_src = load_peaks()
    # one shared pool of random activations, viewed per layer as its NHWC input
    max_in = max(batch * l.cin * l.hw_in ** 2 for l in layers)
    g = torch.Generator(device=device).manual_seed(1000 + rank)
    pool = torch.randn(max_in, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    inputs = [pool[: batch * l.cin * l.hw_in ** 2].view(batch, l.hw_in, l.hw_in, l.cin).permute(0, 3, 1, 2)
              for l in layers]

    def step():
        out = None
        for l, prm, x in zip(layers, params, inputs):
            out = run_layer(l, x, prm)
        return out

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            last = step()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    steps = max(1, args.steps)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        stream.synchronize()
        barrier()
        with ClockSampler(local_rank) as clocks:
            e0.record(stream)
            for _ in range(steps):
                graph.replay()
            e1.record(stream)
            stream.synchronize()
        barrier()
    elapsed_ms = e0.elapsed_time(e1)
    if dist is not None:
        t = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / steps
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
    if dist is not None:
        t = torch.tensor([e2e_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    status_word = fd.device_status()

    if rank == 0:
        roof_s = stack_roofline_seconds(layers, batch, peaks)
        launches = sum(fd.conv2d_plan(x, p_[0], stride=l.stride, padding=l.pad)["launches"]
                       for l, p_, x in zip(layers, params, inputs))
        slow = sorted(shape_ms.values(), key=lambda t: -t[1])[:6]
        cpu_value, cpu_s = cpu_stack_leg(torch, images=2)
        line = {
            "metric": "fused_conv2d_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "c5", "description": "ResNet-50 forward conv stack, 53 convs with folded scale+bias(+ReLU), "
                       f"bf16 NHWC 224x224, batch {total_batch} sharded along N", "per_gpu_batch": batch,
                       "inputs": "each layer reads independently generated N(0,1) activations of its shape; "
                                 "no pooling / residual glue in the timed region",
                       "launch": "cuda_graph_replay", "l2": "activations of every layer exceed the 126 MiB L2",
                       "parallelism": f"batch-sharded replicas x{world}, no collective"},
            "pct_of_bf16_peak": 100.0 * (value / world) / peaks["bf16_tflops"],
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
}


def run_extra(args):
    """One JSON line for a row next to the hot path, same timing rules (cold L2, CUDA graph, events, clocks)."""
    import torch

    import flagdnn_b200 as fd

    if int(os.environ.get("WORLD_SIZE", "1")) != 1:
        raise RuntimeError("the 'res' and 'mm' workloads are single-GPU measurements")
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
    host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    if args.workload == "res":
        host_out = torch.empty(out.shape, dtype=out.dtype).contiguous(memory_format=torch.channels_last).pin_memory()

    def e2e_step():
        for d, h in zip(dev_in, host_in):
            d.copy_(h, non_blocking=True)
        if args.workload == "res":
            y = fd.conv2d_bias_act(dev_in[0], w, bias, scale=scale, relu=True, residual=dev_in[1])
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
    run, cpu_flops, sample = cpu_once(8 if args.workload == "res" else 256)
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS) + ["c5"] + sorted(EXTRA))
    ap.add_argument("--batch", type=int, default=1024, help="total batch of the c5 workload (split over the ranks)")
    ap.add_argument("--eager", action="store_true",
                    help="launch every step through the API instead of replaying a CUDA graph (for profilers)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end and CPU-baseline legs (short runs under a profiler)")
    args = ap.parse_args()
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

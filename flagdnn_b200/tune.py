"""Measure the planner's choice against every alternative it could have made.

The reference fixes launch configurations per shape from a table its autotuner fills
(src/flag_dnn/utils/libentry.py:499-579, tune_configs.yaml:1326-1466).  This library has a planner instead:
a cost model picks the kernel family (one CTA per tile, or CTA pairs), the tile width and whether narrow
layers group output pixels.  This tool is the check on that model: for every distinct convolution of
ResNet-50 at a given batch it times the planner's choice and each forced alternative (through the
``FDNN_ALGO_FLAG_TILE_N_*`` / ``FDNN_ALGO_FLAG_NO_PIXEL_GROUP`` flags and the forced kernel families) and
prints one line per layer plus the totals, so that a choice that loses to an alternative shows up as a ratio.

    python -m flagdnn_b200.tune --batch 128            # the batch a rank holds when 1024 images are split over 8
    python -m flagdnn_b200.tune --batch 1024 --json out.json

Timing: each configuration is captured into a CUDA graph of ``--reps`` launches over rotating input sets (so
that consecutive launches do not find their operands in L2), replayed once untimed and then timed with CUDA
events on the launching stream; L2 is flushed before every replay.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Dict, List, Optional

import torch

from . import _native as nat
from . import conv_host
from .convstack import ConvLayer, make_layer_params, resnet50_conv_layers, run_layer

CANDIDATES = [
    ("auto", nat.ALGO_AUTO),
    ("cta64", nat.ALGO_IGEMM | nat.ALGO_FLAG_TILE_N_64 | nat.ALGO_FLAG_NO_PIXEL_GROUP),
    ("cta128", nat.ALGO_IGEMM | nat.ALGO_FLAG_TILE_N_128 | nat.ALGO_FLAG_NO_PIXEL_GROUP),
    ("cta256", nat.ALGO_IGEMM | nat.ALGO_FLAG_TILE_N_256 | nat.ALGO_FLAG_NO_PIXEL_GROUP),
    ("cta+group", nat.ALGO_IGEMM),
    ("pair", nat.ALGO_IGEMM_PAIR),
    ("pair+split", nat.ALGO_IGEMM_PAIR | nat.ALGO_FLAG_STREAM_K),   # reduction steps shared evenly between the pairs
]


def _time_config(layer: ConvLayer, xs: List[torch.Tensor], params, reps: int, replays: int,
                 flush: torch.Tensor) -> Optional[float]:
    """Microseconds per launch, or None when the forced configuration does not apply to this layer."""
    try:
        for x in xs[:2]:
            run_layer(layer, x, params)
    except NotImplementedError:
        return None
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for i in range(reps):
                run_layer(layer, xs[i % len(xs)], params)
    torch.cuda.synchronize()
    graph.replay()   # the first launch uploads the graph
    torch.cuda.synchronize()
    times = []
    for _ in range(replays):
        flush.zero_()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop) * 1e3 / reps)
    times.sort()
    return times[len(times) // 2]


def sweep(batch: int, dtype: torch.dtype, reps: int, replays: int, only: Optional[str] = None) -> List[Dict]:
    device = torch.device("cuda", torch.cuda.current_device())
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    seen, rows = set(), []
    for layer in resnet50_conv_layers():
        if layer.shape_key in seen or (only and only not in layer.name):
            continue
        seen.add(layer.shape_key)
        count = sum(1 for l in resnet50_conv_layers() if l.shape_key == layer.shape_key)
        params = make_layer_params(layer, 1, device, dtype)
        x_bytes = batch * layer.cin * layer.hw_in ** 2 * 2
        sets = max(2, min(8, (192 << 20) // max(x_bytes, 1) + 1))
        g = torch.Generator().manual_seed(2)
        xs = [torch.randn(batch, layer.cin, layer.hw_in, layer.hw_in, generator=g).to(dtype).to(device)
              .contiguous(memory_format=torch.channels_last) for _ in range(sets)]
        row = {"layer": layer.name, "shape": f"{layer.cin}->{layer.cout} {layer.k}x{layer.k}/{layer.stride} @{layer.hw_in}",
               "count": count, "us": {}}
        for name, algo in CANDIDATES:
            prev = conv_host.set_algo(algo)
            try:
                if name == "auto":
                    plan = conv_host.conv2d_plan(xs[0], params[0], stride=layer.stride, padding=layer.pad)
                    row["plan"] = {"algo": {1: "direct", 2: "cta", 3: "pair"}.get(plan["algo"], plan["algo"]),
                                   "tile_n": plan["tile_n"], "pixel_group": plan["pixel_group"],
                                   "low_channel": plan["low_channel"], "grid": plan["grid"]}
                us = _time_config(layer, xs, params, reps, replays, flush)
            finally:
                conv_host.set_algo(prev)
            if us is not None:
                row["us"][name] = round(us, 2)
        best = min(row["us"], key=row["us"].get)
        row["best"] = best
        row["auto_over_best"] = round(row["us"]["auto"] / row["us"][best], 3)
        rows.append(row)
        del xs
        torch.cuda.empty_cache()
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float16"])
    ap.add_argument("--reps", type=int, default=16, help="launches per captured graph")
    ap.add_argument("--replays", type=int, default=7, help="timed replays (the median is reported)")
    ap.add_argument("--only", default=None, help="substring of the layer names to keep")
    ap.add_argument("--json", default=None, help="also write the rows to this file")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("flagdnn_b200.tune needs a CUDA device", file=sys.stderr)
        return 2
    rows = sweep(args.batch, getattr(torch, args.dtype), args.reps, args.replays, args.only)
    names = [n for n, _ in CANDIDATES]
    print(f"batch {args.batch} {args.dtype}: microseconds per launch (median of {args.replays} replays of {args.reps})")
    print(f"{'layer':<12}{'shape':<26}{'x':>3} {'plan':<22}" + "".join(f"{n:>10}" for n in names) + f"{'best':>10}{'auto/best':>10}")
    tot_auto = tot_best = 0.0
    for r in rows:
        p = r["plan"]
        plan = f"{p['algo']} n{p['tile_n']} g{p['pixel_group']} lc{p['low_channel']}"
        cells = "".join(f"{r['us'].get(n, float('nan')):>10.1f}" for n in names)
        print(f"{r['layer']:<12}{r['shape']:<26}{r['count']:>3} {plan:<22}{cells}{r['best']:>10}{r['auto_over_best']:>10.3f}")
        tot_auto += r["us"]["auto"] * r["count"]
        tot_best += r["us"][r["best"]] * r["count"]
    print(f"whole stack ({sum(r['count'] for r in rows)} launches): planner {tot_auto:.0f} us, best per layer {tot_best:.0f} us, "
          f"ratio {tot_auto / tot_best:.3f}")
    if args.json:
        with open(args.json, "w") as f:
            json.dump({"batch": args.batch, "dtype": args.dtype, "rows": rows}, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())

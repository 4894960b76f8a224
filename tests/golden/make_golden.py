"""Generates tests/golden/*.npz by running the UNMODIFIED reference on CPU.

Run from the repository root on a machine that has the reference checked out:

    python tests/golden/make_golden.py /path/to/FlagDNN

The reference's CPU path is its compiled graph executed on CPU tensors
(src/flag_dnn/graph/backend.py:154-159 picks the torch backend when no device
is present; src/flag_dnn/graph/registry.py:1357-1365, 1426 then run
torch.nn.functional.conv2d and relu).  For every case this script records the
seeded inputs, what the reference's fusion pass made of the graph, and the
reference's output, so that the tests can replay them without the reference.

Three things the reference needs to import on a machine without a GPU are
supplied from outside, without touching its files: an empty stand-in for the
`sqlalchemy` package (only used by its autotune cache), FLAGGEMS_DB_URL (so it
does not ask CUDA for a device name) and DNN_VENDOR=nvidia (so it does not
shell out to nvidia-smi).

Shape lists: tests/test_conv2d.py:18-39 and tests_graph/consts.py:58-82 of the
reference (shape tuples only), plus scaled-down versions of the benchmark
configurations.
"""
from __future__ import annotations

import os
import sys
import tempfile
import types
from pathlib import Path

import numpy as np
import torch

OUT_DIR = Path(__file__).resolve().parent

# (input_shape, weight_shape, bias?, stride, padding, dilation, groups) — tests/test_conv2d.py:18-39
EAGER_CASES = [
    ((1, 3, 8, 8), (4, 3, 3, 3), True, 1, 0, 1, 1),
    ((2, 3, 16, 16), (8, 3, 3, 3), False, 1, 1, 1, 1),
    ((2, 3, 15, 17), (6, 3, 5, 5), True, 2, 2, 1, 1),
    ((1, 3, 13, 11), (5, 3, 1, 1), True, 1, 0, 1, 1),
    ((1, 3, 17, 17), (4, 3, 3, 3), True, 1, 2, 2, 1),
    ((2, 3, 19, 21), (7, 3, 3, 3), False, 2, 2, 2, 1),
    ((1, 4, 12, 12), (8, 2, 3, 3), True, 1, 1, 1, 2),
    ((2, 4, 18, 14), (6, 2, 5, 5), False, 2, 2, 1, 2),
    ((1, 4, 10, 11), (4, 1, 3, 3), True, 1, 1, 1, 4),
    ((2, 8, 16, 16), (8, 1, 5, 5), False, 1, 2, 1, 8),
    ((1, 2, 9, 9), (4, 2, 3, 3), True, 1, "same", 1, 1),
    ((1, 4, 13, 13), (8, 2, 3, 3), False, 1, "same", 2, 2),
    ((1, 3, 12, 12), (6, 3, 3, 3), True, 1, "valid", 1, 1),
    ((2, 4, 20, 18), (8, 2, 5, 5), False, 2, "valid", 1, 2),
]

# (input_shape, weight_shape, stride, padding, dilation) — tests_graph/consts.py:71-82
FUSED_CASES = [
    ((2, 8, 16, 16), (16, 8, 3, 3), 1, 1, 1),
    ((1, 4, 15, 17), (6, 4, 3, 5), (2, 1), (1, 2), 1),
    ((2, 3, 8, 8), (5, 3, 1, 1), 1, 0, 1),
    ((1, 6, 20, 18), (8, 6, 5, 3), (1, 2), (2, 1), 1),
    ((2, 4, 12, 10), (7, 4, 3, 3), 2, 1, 1),
    ((1, 5, 19, 21), (9, 5, 3, 3), 1, 2, 2),
    ((1, 3, 32, 32), (8, 3, 3, 3), 1, 1, 1),
    ((2, 8, 9, 11), (4, 8, 1, 1), 1, 0, 1),
    ((1, 4, 18, 18), (4, 4, 3, 3), 1, 0, 1),
    ((2, 12, 13, 15), (10, 12, 3, 3), 1, 1, 1),
    # scaled-down benchmark configurations (same kernel / stride / padding, fewer images and pixels)
    ((1, 64, 14, 14), (64, 64, 3, 3), 1, 1, 1),      # fp32 NCHW 3x3 configuration
    ((2, 256, 7, 7), (64, 256, 1, 1), 1, 0, 1),      # 1x1 bottleneck reduce
    ((1, 128, 6, 6), (128, 128, 3, 3), 1, 1, 1),     # 3x3 headline layer at half width
    ((1, 3, 30, 30), (64, 3, 7, 7), 2, 3, 1),        # 7x7 stride-2 stem
]


def _import_reference(ref_root: str):
    stub_dir = tempfile.mkdtemp(prefix="sqlalchemy_stub_")
    pkg = Path(stub_dir) / "sqlalchemy"
    any_src = (
        "class _Any:\n"
        "    def __init__(self, *a, **k): pass\n"
        "    def __call__(self, *a, **k): return _Any()\n"
        "    def __getattr__(self, n): return _Any()\n"
        "def __getattr__(name): return _Any()\n"
    )
    for sub in ("", "orm", "ext", "ext/automap", "engine", "exc", "schema"):
        d = pkg / sub
        d.mkdir(parents=True, exist_ok=True)
        (d / "__init__.py").write_text(any_src)
    (pkg / "orm" / "__init__.py").write_text(
        any_src + "class DeclarativeBase: pass\nclass Session: pass\n"
    )
    (pkg / "exc" / "__init__.py").write_text(any_src + "class IntegrityError(Exception): pass\n")
    os.environ.setdefault("FLAGGEMS_DB_URL", "sqlite:///" + os.path.join(stub_dir, "tune.db"))
    os.environ.setdefault("DNN_VENDOR", "nvidia")
    sys.dont_write_bytecode = True
    sys.path.insert(0, stub_dir)
    sys.path.insert(0, os.path.join(ref_root, "src"))
    import flag_dnn  # noqa: E402

    return flag_dnn


def _seeded(shape, seed, dist="normal", std=1.0):
    g = torch.Generator().manual_seed(seed)
    if dist == "uniform":
        return torch.rand(shape, generator=g) * 2 - 1
    return torch.randn(shape, generator=g) * std


def main() -> None:
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/FlagDNN")
    ref_root = sys.argv[1]
    flag_dnn = _import_reference(ref_root)
    records = {}

    # ---- fused graph cases: conv2d -> bias_add -> relu through flag_dnn.compile on CPU
    for idx, (ishape, wshape, stride, padding, dilation) in enumerate(FUSED_CASES):
        seed = 1000 + idx
        fan_in = wshape[1] * wshape[2] * wshape[3]
        x = _seeded(ishape, seed)
        w = _seeded(wshape, seed + 100, std=fan_in ** -0.5)
        b = _seeded((wshape[0],), seed + 200, std=0.1)

        @flag_dnn.graph
        def fn(x, weight, bias, _s=stride, _p=padding, _d=dilation):
            y = flag_dnn.conv2d(x, weight, stride=_s, padding=_p, dilation=_d, groups=1)
            y = flag_dnn.bias_add(y, bias)
            return flag_dnn.relu(y)

        compiled = flag_dnn.compile(fn, inputs=[x, w, b], options={"cache": None})
        nodes = [n.op_type for n in compiled.graph.nodes]
        assert nodes == ["fused_conv2d_bias_relu"], nodes
        assert compiled.plan.debug_info["fusion"]["conv2d_bias_activation_fused"] == 1
        y = compiled.run(x.clone(), w.clone(), b.clone())
        key = f"fused_{idx:02d}"
        records[key + "_x"] = x.numpy()
        records[key + "_w"] = w.numpy()
        records[key + "_b"] = b.numpy()
        records[key + "_y"] = y.numpy()
        records[key + "_meta"] = np.array(
            [*(_pair(stride)), *(_pair(padding)), *(_pair(dilation))], dtype=np.int64
        )

    # ---- eager-surface cases: conv2d (+bias folded by the fusion pass) through the CPU graph
    for idx, (ishape, wshape, has_bias, stride, padding, dilation, groups) in enumerate(EAGER_CASES):
        seed = 2000 + idx
        x = _seeded(ishape, seed)
        w = _seeded(wshape, seed + 100)
        b = _seeded((wshape[0],), seed + 200) if has_bias else None

        if has_bias:
            @flag_dnn.graph
            def fn(x, weight, bias, _s=stride, _p=padding, _d=dilation, _g=groups):
                return flag_dnn.conv2d(x, weight, bias, stride=_s, padding=_p, dilation=_d, groups=_g)

            compiled = flag_dnn.compile(fn, inputs=[x, w, b], options={"cache": None})
            y = compiled.run(x.clone(), w.clone(), b.clone())
        else:
            @flag_dnn.graph
            def fn(x, weight, _s=stride, _p=padding, _d=dilation, _g=groups):
                return flag_dnn.conv2d(x, weight, stride=_s, padding=_p, dilation=_d, groups=_g)

            compiled = flag_dnn.compile(fn, inputs=[x, w], options={"cache": None})
            y = compiled.run(x.clone(), w.clone())
        assert [n.op_type for n in compiled.graph.nodes] == ["conv2d"]
        key = f"eager_{idx:02d}"
        records[key + "_x"] = x.numpy()
        records[key + "_w"] = w.numpy()
        if has_bias:
            records[key + "_b"] = b.numpy()
        records[key + "_y"] = y.numpy()

    np.savez_compressed(OUT_DIR / "reference_cpu_outputs.npz", **records)
    print("wrote", OUT_DIR / "reference_cpu_outputs.npz", len(records), "arrays")
    _write_next_rows(flag_dnn)


# Graphs next to the conv -> bias -> ReLU path, as the unmodified reference runs them on CPU: a residual
# block's tail (conv, per-channel scale, bias, shortcut add, ReLU), conv -> bias -> GELU in both forms, mm.
TAIL_CASES = [((2, 16, 12, 12), (24, 16, 1, 1), 1, 0), ((2, 8, 10, 10), (8, 8, 3, 3), 1, 1),
              ((1, 32, 9, 9), (40, 32, 3, 3), 2, 1)]
GELU_CASES = [((2, 8, 10, 10), (12, 8, 3, 3), 1, 1, "none"), ((1, 16, 7, 7), (16, 16, 1, 1), 1, 0, "tanh")]
MM_CASES = [(2, 3, 4), (7, 5, 3), (16, 17, 15), (32, 64, 16), (64, 128, 96)]


def _write_next_rows(flag_dnn) -> None:
    records = {}
    for idx, (ishape, wshape, stride, padding) in enumerate(TAIL_CASES):
        seed = 3000 + idx
        fan_in = wshape[1] * wshape[2] * wshape[3]
        x = _seeded(ishape, seed)
        w = _seeded(wshape, seed + 100, std=fan_in ** -0.5)
        s = torch.rand(wshape[0], 1, 1, generator=torch.Generator().manual_seed(seed + 150)) + 0.5
        b = _seeded((wshape[0],), seed + 200, std=0.1)
        oh = (ishape[2] + 2 * padding - wshape[2]) // stride + 1
        shortcut = _seeded((ishape[0], wshape[0], oh, oh), seed + 300)

        @flag_dnn.graph
        def tail(x, weight, scale, bias, shortcut, _s=stride, _p=padding):
            y = flag_dnn.conv2d(x, weight, stride=_s, padding=_p)
            y = flag_dnn.bias_add(flag_dnn.mul(y, scale), bias)
            return flag_dnn.relu(flag_dnn.add(y, shortcut))

        compiled = flag_dnn.compile(tail, inputs=[x, w, s, b, shortcut], options={"cache": None})
        y = compiled.run(x.clone(), w.clone(), s.clone(), b.clone(), shortcut.clone())
        key = f"tail_{idx:02d}"
        for name, t in (("x", x), ("w", w), ("s", s), ("b", b), ("r", shortcut), ("y", y)):
            records[f"{key}_{name}"] = t.numpy()
        records[key + "_meta"] = np.array([stride, padding], dtype=np.int64)

    for idx, (ishape, wshape, stride, padding, approximate) in enumerate(GELU_CASES):
        seed = 4000 + idx
        fan_in = wshape[1] * wshape[2] * wshape[3]
        x = _seeded(ishape, seed)
        w = _seeded(wshape, seed + 100, std=fan_in ** -0.5)
        b = _seeded((wshape[0],), seed + 200, std=0.5)

        @flag_dnn.graph
        def act(x, weight, bias, _s=stride, _p=padding, _a=approximate):
            return flag_dnn.gelu(flag_dnn.bias_add(flag_dnn.conv2d(x, weight, stride=_s, padding=_p), bias),
                                 approximate=_a)

        compiled = flag_dnn.compile(act, inputs=[x, w, b], options={"cache": None})
        y = compiled.run(x.clone(), w.clone(), b.clone())
        key = f"gelu_{idx:02d}"
        for name, t in (("x", x), ("w", w), ("b", b), ("y", y)):
            records[f"{key}_{name}"] = t.numpy()
        records[key + "_meta"] = np.array([stride, padding, int(approximate == "tanh")], dtype=np.int64)

    for idx, (m, k, n) in enumerate(MM_CASES):
        a = _seeded((m, k), 5000 + idx, dist="uniform")
        bm = _seeded((k, n), 5100 + idx, dist="uniform")

        @flag_dnn.graph
        def matmul(a, b):
            return flag_dnn.mm(a, b)

        compiled = flag_dnn.compile(matmul, inputs=[a, bm], options={"cache": None})
        y = compiled.run(a.clone(), bm.clone())
        key = f"mm_{idx:02d}"
        records[key + "_a"], records[key + "_b"], records[key + "_y"] = a.numpy(), bm.numpy(), y.numpy()

    np.savez_compressed(OUT_DIR / "reference_cpu_outputs_next.npz", **records)
    print("wrote", OUT_DIR / "reference_cpu_outputs_next.npz", len(records), "arrays")


def _pair(v):
    return (v, v) if isinstance(v, int) else tuple(v)


if __name__ == "__main__":
    main()

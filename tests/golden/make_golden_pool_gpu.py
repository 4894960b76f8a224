"""Generates tests/golden/reference_gpu_pool_outputs.npz: outputs of the UNMODIFIED reference's pooling operators.

The reference has no CPU path for max_pool2d / adaptive_avg_pool2d (src/flag_dnn/ops/max_pool2d.py:174,
src/flag_dnn/ops/adaptive_avg_pool2d.py:456 launch Triton kernels only), so these fixtures come from a run of the
reference itself on a GPU: it is imported from baseline/_ref (a pip --target install of the reference, not tracked)
through the same shims the benchmark's reference arm uses, fed seeded fp32 inputs, and its results are stored next
to the inputs.  Run once on a machine with a GPU:

    python tests/golden/make_golden_pool_gpu.py [output.npz]

The tests then hold both this library's kernels and the CPU oracle (torch's pooling) to these outputs.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

# (input shape, kernel, stride, padding, dilation, ceil_mode): the reference's own cases
# (tests/test_max_pool2d.py:9-16) in both rounding modes where they differ, and two more
MAXPOOL = [
    ((2, 3, 32, 32), 2, 2, 0, 1, False),
    ((1, 16, 28, 28), 3, 1, 1, 1, False),
    ((4, 8, 15, 15), 3, 2, 1, 1, False),
    ((4, 8, 15, 15), 3, 2, 1, 1, True),
    ((2, 4, 32, 32), (3, 5), (2, 1), 0, 1, False),
    ((2, 3, 32, 32), 3, 2, 0, 2, True),
    ((16, 14, 14), 2, 2, 0, 1, False),
    ((2, 72, 19, 23), (2, 3), (2, 2), (1, 1), 1, True),
]
# (input shape, output size): the reference's cases (tests/test_adaptive_avg_pool2d.py) and one ragged one
AVGPOOL = [
    ((2, 3, 32, 32), (1, 1)),
    ((1, 16, 28, 28), 14),
    ((4, 8, 15, 15), (7, 5)),
    ((2, 4, 32, 32), (None, 16)),
    ((16, 14, 14), (2, 2)),
    ((2, 64, 20, 13), (3, 4)),
]


def main(out_path):
    import bench

    flag_dnn = bench._import_reference_gpu()
    from flag_dnn.ops.adaptive_avg_pool2d import adaptive_avg_pool2d
    from flag_dnn.ops.max_pool2d import max_pool2d

    data = {}
    for i, (shape, kernel, stride, padding, dilation, ceil_mode) in enumerate(MAXPOOL):
        x = torch.randn(shape, generator=torch.Generator().manual_seed(500 + i))
        y, idx = max_pool2d(x.cuda(), kernel, stride, padding, dilation, ceil_mode, return_indices=True)
        data[f"max_{i:02d}_x"] = x.numpy()
        data[f"max_{i:02d}_y"] = y.cpu().numpy()
        data[f"max_{i:02d}_idx"] = idx.cpu().numpy().astype(np.int64)
    for i, (shape, size) in enumerate(AVGPOOL):
        x = torch.randn(shape, generator=torch.Generator().manual_seed(600 + i))
        y = adaptive_avg_pool2d(x.cuda(), size)
        data[f"avg_{i:02d}_x"] = x.numpy()
        data[f"avg_{i:02d}_y"] = y.cpu().numpy()
    torch.cuda.synchronize()
    np.savez_compressed(out_path, **data)
    print(f"wrote {out_path}: {len(data)} arrays from flag_dnn {getattr(flag_dnn, '__version__', '?')}")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden", "reference_gpu_pool_outputs.npz"))

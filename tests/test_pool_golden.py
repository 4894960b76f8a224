"""Pooling against outputs of the unmodified reference's own (GPU-only) operators, stored in
tests/golden/reference_gpu_pool_outputs.npz by tests/golden/make_golden_pool_gpu.py:

* without a GPU: the CPU oracle (torch's pooling, which the reference's tests use as theirs,
  tests/test_max_pool2d.py:49-58, tests/test_adaptive_avg_pool2d.py:46-60) reproduces those outputs;
* on the GPU: this library's kernels reproduce them, values and argmax indices.
"""
import importlib.util
import os

import numpy as np
import pytest
import torch

from conftest import ROOT

_spec = importlib.util.spec_from_file_location("make_golden_pool_gpu",
                                               os.path.join(ROOT, "tests", "golden", "make_golden_pool_gpu.py"))
_cases = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_cases)   # the case tables only; nothing runs at import
MAXPOOL, AVGPOOL = _cases.MAXPOOL, _cases.AVGPOOL


@pytest.fixture(scope="module")
def pool_golden():
    with np.load(os.path.join(ROOT, "tests", "golden", "reference_gpu_pool_outputs.npz")) as data:
        return {k: data[k] for k in data.files}


@pytest.mark.parametrize("i", range(len(MAXPOOL)))
def test_oracle_max_pool_reproduces_reference_outputs(pool_golden, i):
    shape, kernel, stride, padding, dilation, ceil_mode = MAXPOOL[i]
    x = torch.from_numpy(pool_golden[f"max_{i:02d}_x"])
    assert tuple(x.shape) == shape
    y, idx = torch.nn.functional.max_pool2d(x, kernel, stride, padding, dilation, ceil_mode, return_indices=True)
    assert torch.equal(y, torch.from_numpy(pool_golden[f"max_{i:02d}_y"]))
    assert torch.equal(idx, torch.from_numpy(pool_golden[f"max_{i:02d}_idx"]))


@pytest.mark.parametrize("i", range(len(AVGPOOL)))
def test_oracle_adaptive_avg_pool_reproduces_reference_outputs(pool_golden, i):
    shape, size = AVGPOOL[i]
    x = torch.from_numpy(pool_golden[f"avg_{i:02d}_x"])
    y = torch.nn.functional.adaptive_avg_pool2d(x, size)
    torch.testing.assert_close(y, torch.from_numpy(pool_golden[f"avg_{i:02d}_y"]), rtol=1e-6, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("channels_last", [False, True])
@pytest.mark.parametrize("i", range(len(MAXPOOL)))
def test_library_max_pool_reproduces_reference_outputs(native_lib, pool_golden, i, channels_last):
    import flagdnn_b200 as fd

    shape, kernel, stride, padding, dilation, ceil_mode = MAXPOOL[i]
    x = torch.from_numpy(pool_golden[f"max_{i:02d}_x"]).cuda()
    if channels_last:
        if x.dim() != 4:
            pytest.skip("channels-last needs a batch dimension")
        x = x.contiguous(memory_format=torch.channels_last)
    y, idx = fd.max_pool2d(x, kernel, stride, padding, dilation, ceil_mode, return_indices=True)
    assert torch.equal(y.cpu(), torch.from_numpy(pool_golden[f"max_{i:02d}_y"]))
    assert torch.equal(idx.cpu(), torch.from_numpy(pool_golden[f"max_{i:02d}_idx"]))
    for dtype in (torch.bfloat16, torch.float16):     # 16-bit: the maximum of rounded values is the rounded maximum
        got = fd.max_pool2d(x.to(dtype), kernel, stride, padding, dilation, ceil_mode)
        want = torch.nn.functional.max_pool2d(x.to(dtype).float().cpu(), kernel, stride, padding, dilation, ceil_mode)
        assert torch.equal(got.float().cpu(), want)


@pytest.mark.gpu
@pytest.mark.parametrize("i", range(len(AVGPOOL)))
def test_library_adaptive_avg_pool_reproduces_reference_outputs(native_lib, pool_golden, i):
    import flagdnn_b200 as fd

    shape, size = AVGPOOL[i]
    x = torch.from_numpy(pool_golden[f"avg_{i:02d}_x"]).cuda()
    y = fd.adaptive_avg_pool2d(x, size)
    torch.testing.assert_close(y.cpu(), torch.from_numpy(pool_golden[f"avg_{i:02d}_y"]), rtol=1e-6, atol=1e-6)

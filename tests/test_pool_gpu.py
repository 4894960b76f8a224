"""max_pool2d / adaptive_avg_pool2d on the library's CUDA kernels against torch on CPU (the reference's own
oracle for these operators, tests/test_max_pool2d.py:49-58, tests/test_adaptive_avg_pool2d.py:46-60)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

# the reference's cases (tests/test_max_pool2d.py:9-16) plus the ResNet stem pool and a wide channels-last case
MAXPOOL = [
    ((2, 3, 32, 32), 2, 2, 0, 1),
    ((1, 16, 28, 28), 3, 1, 1, 1),
    ((4, 8, 15, 15), 3, 2, 1, 1),
    ((2, 4, 32, 32), (3, 5), (2, 1), 0, 1),
    ((2, 3, 32, 32), 3, 2, 0, 2),
    ((16, 14, 14), 2, 2, 0, 1),
    ((3, 64, 112, 112), 3, 2, 1, 1),
    ((2, 72, 19, 23), (2, 3), (2, 2), (1, 1), 1),
]
AVGPOOL = [
    ((2, 3, 32, 32), (1, 1)),
    ((1, 16, 28, 28), 14),
    ((4, 8, 15, 15), (7, 5)),
    ((2, 4, 32, 32), (None, 16)),
    ((16, 14, 14), (2, 2)),
    ((5, 2048, 7, 7), 1),
    ((2, 64, 20, 13), (3, 4)),
]
DTYPES = ["float32", "bfloat16", "float16", "float64"]


@pytest.fixture(scope="module")
def fd(native_lib):
    import flagdnn_b200

    assert torch.cuda.is_available()
    return flagdnn_b200


def _layouts(shape):
    return [False, True] if len(shape) == 4 else [False]


@pytest.mark.parametrize("ceil_mode", [False, True])
@pytest.mark.parametrize("dtype_name", DTYPES)
@pytest.mark.parametrize("case", MAXPOOL, ids=[str(i) for i in range(len(MAXPOOL))])
def test_max_pool2d_matches_torch_cpu(fd, case, dtype_name, ceil_mode):
    shape, kernel, stride, padding, dilation = case
    dtype = getattr(torch, dtype_name)
    x_cpu = torch.randn(shape, generator=torch.Generator().manual_seed(len(shape) + sum(shape))).to(dtype)
    ref, ref_idx = torch.nn.functional.max_pool2d(x_cpu.float() if dtype_name != "float64" else x_cpu, kernel, stride,
                                                  padding, dilation, ceil_mode, return_indices=True)
    for channels_last in _layouts(shape):
        x = x_cpu.cuda()
        if channels_last:
            x = x.contiguous(memory_format=torch.channels_last)
        got = fd.max_pool2d(x, kernel, stride, padding, dilation, ceil_mode)
        assert got.dtype == dtype and got.shape == ref.shape
        assert torch.equal(got.cpu().to(ref.dtype), ref)          # a maximum of exact values is exact
        if channels_last:
            assert got.is_contiguous(memory_format=torch.channels_last)
        vals, idx = fd.max_pool2d(x, kernel, stride, padding, dilation, ceil_mode, return_indices=True)
        assert torch.equal(vals, got) and idx.dtype == torch.int64
        assert torch.equal(idx.cpu(), ref_idx)


def test_max_pool2d_nan_and_checks(fd):
    x = torch.randn(2, 8, 9, 9, device="cuda", dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    x[1, 3, 4, 4] = float("nan")
    got = fd.max_pool2d(x, 3, 2, 1)
    ref = torch.nn.functional.max_pool2d(x.float().cpu(), 3, 2, 1)
    assert torch.equal(torch.isnan(got.cpu()), torch.isnan(ref)) and int(torch.isnan(ref).sum()) > 0
    scalar = fd.max_pool2d(x[:, :5], 3, 2, 1)                      # 5 channels: the per-element kernel
    assert torch.equal(torch.isnan(scalar.cpu()), torch.isnan(ref[:, :5]))
    with pytest.raises(RuntimeError, match="pad should be at most half"):
        fd.max_pool2d(x, 2, 2, 2)
    with pytest.raises(NotImplementedError, match="requires CUDA input"):
        fd.max_pool2d(x.cpu(), 2)
    with pytest.raises(AssertionError, match="3D or 4D"):
        fd.max_pool2d(x[0, 0], 2)
    assert fd.max_pool2d(x[:0], 2).shape == (0, 8, 4, 4)


@pytest.mark.parametrize("dtype_name", DTYPES)
@pytest.mark.parametrize("case", AVGPOOL, ids=[str(i) for i in range(len(AVGPOOL))])
def test_adaptive_avg_pool2d_matches_torch_cpu(fd, case, dtype_name):
    shape, size = case
    dtype = getattr(torch, dtype_name)
    x_cpu = torch.randn(shape, generator=torch.Generator().manual_seed(sum(shape))).to(dtype)
    cdt = torch.float64 if dtype_name == "float64" else torch.float32
    ref = torch.nn.functional.adaptive_avg_pool2d(x_cpu.to(cdt), size)
    tol = {"float32": 1e-5, "float64": 1e-12, "bfloat16": 1e-2, "float16": 2e-3}[dtype_name]
    for channels_last in _layouts(shape):
        x = x_cpu.cuda()
        if channels_last:
            x = x.contiguous(memory_format=torch.channels_last)
        got = fd.adaptive_avg_pool2d(x, size)
        assert got.dtype == dtype and got.shape == ref.shape
        torch.testing.assert_close(got.cpu().to(cdt), ref, rtol=tol, atol=tol)


def test_pooling_in_a_captured_graph(fd):
    """stem conv -> ReLU -> max pool -> global average, compiled once; pooling nodes run on the library."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 3, 64, 64, generator=g).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    w = (torch.randn(64, 3, 7, 7, generator=g) * 0.08).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    b = torch.randn(64, generator=g).to(torch.bfloat16).cuda()

    @fd.graph
    def head(x, w, b):
        y = fd.relu(fd.bias_add(fd.conv2d(x, w, stride=2, padding=3), b))
        return fd.adaptive_avg_pool2d(fd.max_pool2d(y, 3, 2, 1), 1)

    compiled = fd.compile(head, inputs=[x, w, b], options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["fused_conv2d_bias_relu", "max_pool2d", "adaptive_avg_pool2d"]
    got = compiled.run(x, w, b)
    y = torch.relu(torch.nn.functional.conv2d(x.float().cpu(), w.float().cpu(), b.float().cpu(), 2, 3)).to(torch.bfloat16)
    ref = torch.nn.functional.adaptive_avg_pool2d(torch.nn.functional.max_pool2d(y.float(), 3, 2, 1), 1)
    torch.testing.assert_close(got.float().cpu(), ref, rtol=2e-2, atol=2e-2)
    assert fd.device_status() == 0

"""Parity of the CUDA path with the oracle, through the public API (which
calls the C ABI).  Modelled on the reference's own tests: eager conv2d against
an upcast torch result (tests/test_conv2d.py:56-116) and the compiled
conv -> bias -> ReLU graph against a second implementation
(tests_graph/test_graph_conv_bias_relu.py:113-145), here the CPU oracle."""
import pytest
import torch

import oracle
from cases import EAGER_CASES, FUSED_CASES, TOL

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16,
          "float64": torch.float64}


@pytest.fixture(scope="module")
def fd(native_lib):
    import flagdnn_b200

    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    yield flagdnn_b200
    flagdnn_b200.set_algo("auto")
    assert flagdnn_b200.device_status() == 0, "a kernel recorded a bounded-wait incident"


def _to_dev(t, dtype, channels_last):
    if t is None:
        return None
    t = t.to(dtype).cuda()
    if channels_last and t.dim() == 4:
        t = t.contiguous(memory_format=torch.channels_last)
    return t


def _check(out, ref, dtype_name):
    assert out.shape == ref.shape
    torch.testing.assert_close(out.detach().float().cpu() if dtype_name != "float64" else out.cpu(),
                               ref.float() if dtype_name != "float64" else ref, **TOL[dtype_name])


@pytest.mark.parametrize("algo", ["igemm", "pair", "direct"])
@pytest.mark.parametrize("channels_last", [True, False])
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16", "float16"])
@pytest.mark.parametrize("idx", range(len(FUSED_CASES)))
def test_fused_graph_matches_oracle(fd, golden, idx, dtype_name, channels_last, algo):
    if algo == "pair" and (dtype_name == "float32" or not channels_last):
        pytest.skip("the CTA-pair kernel takes 16-bit tensors and writes channels-last outputs")
    ishape, wshape, stride, padding, dilation = FUSED_CASES[idx]
    key = f"fused_{idx:02d}"
    dtype = DTYPES[dtype_name]
    x, w, b = (torch.from_numpy(golden[key + s]) for s in ("_x", "_w", "_b"))
    xd, wd, bd = _to_dev(x, dtype, channels_last), _to_dev(w, dtype, channels_last), _to_dev(b, dtype, False)

    @fd.graph
    def fn(x, weight, bias):
        y = fd.conv2d(x, weight, stride=stride, padding=padding, dilation=dilation, groups=1)
        return fd.relu(fd.bias_add(y, bias))

    compiled = fd.compile(fn, inputs=[fd.TensorSpec.from_tensor(xd, "x"), fd.TensorSpec.from_tensor(wd, "weight"),
                                      fd.TensorSpec.from_tensor(bd, "bias")], options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["fused_conv2d_bias_relu"]
    assert compiled.plan.debug_info["fusion"]["conv2d_bias_activation_fused"] == 1
    if algo == "pair" and wshape[0] % 8 != 0:
        # y rows of K elements must be 16-byte multiples for the pair kernel's TMA stores;
        # forcing it on such a shape is refused, which the graph layer turns into its fallback
        fd.set_algo("pair")
        try:
            with pytest.raises(NotImplementedError):
                fd.fused_conv2d_bias_relu(xd, wd, bd, stride=stride, padding=padding, dilation=dilation)
        finally:
            fd.set_algo("auto")
        return
    fd.set_algo(algo)
    try:
        out = compiled.run(xd.clone(), wd.clone(), bd.clone())
    finally:
        fd.set_algo("auto")
    assert out.dtype == dtype
    assert out.is_contiguous(memory_format=torch.channels_last) == (xd.stride(1) == 1) or out.shape[1] == 1
    # oracle on the very bits the GPU saw
    ref = oracle.conv2d_torch_cpu(xd, wd, bd, stride, padding, dilation, 1, relu=True)
    _check(out, ref, dtype_name)
    if dtype_name == "float32":  # the stored output of the reference itself
        _check(out, torch.from_numpy(golden[key + "_y"]), dtype_name)


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16", "float16", "float64"])
@pytest.mark.parametrize("idx", range(len(EAGER_CASES)))
def test_eager_conv2d_matches_oracle(fd, golden, idx, dtype_name):
    ishape, wshape, has_bias, stride, padding, dilation, groups = EAGER_CASES[idx]
    key = f"eager_{idx:02d}"
    dtype = DTYPES[dtype_name]
    x, w = torch.from_numpy(golden[key + "_x"]), torch.from_numpy(golden[key + "_w"])
    b = torch.from_numpy(golden[key + "_b"]) if has_bias else None
    xd, wd, bd = _to_dev(x, dtype, False), _to_dev(w, dtype, False), _to_dev(b, dtype, False)
    for algo in ("auto", "igemm", "direct"):
        if algo == "igemm" and (groups != 1 or dtype_name == "float64"):
            continue
        fd.set_algo(algo)
        try:
            out = fd.conv2d(xd, wd, bd, stride=stride, padding=padding, dilation=dilation, groups=groups)
        finally:
            fd.set_algo("auto")
        cdt = torch.float64 if dtype_name == "float64" else torch.float32
        ref = oracle.conv2d_torch_cpu(xd, wd, bd, stride, padding, dilation, groups, compute_dtype=cdt)
        _check(out, ref, dtype_name)
        if dtype_name == "float32":
            _check(out, torch.from_numpy(golden[key + "_y"]), dtype_name)


# (input_shape, weight_shape, bias?, stride, padding, dilation, groups, unbatched, noncontiguous):
# the shape list of the reference's tests/test_conv1d.py:18-30
CONV1D_CASES = [
    ((2, 3, 16), (4, 3, 3), True, 1, 1, 1, 1, False, False),
    ((1, 3, 17), (5, 3, 1), True, 1, 0, 1, 1, False, False),
    ((2, 4, 31), (8, 4, 5), False, 2, 2, 1, 1, False, False),
    ((1, 3, 29), (4, 3, 3), True, 1, 2, 2, 1, False, False),
    ((2, 4, 23), (6, 2, 3), True, 1, 1, 1, 2, False, False),
    ((2, 8, 33), (8, 1, 5), False, 1, 2, 1, 8, False, False),
    ((1, 2, 19), (4, 2, 4), True, 1, "same", 1, 1, False, False),
    ((2, 4, 25), (8, 2, 3), False, 1, "same", 2, 2, False, False),
    ((2, 3, 21), (5, 3, 3), True, 2, "valid", 1, 1, False, False),
    ((3, 13), (4, 3, 3), True, 1, 1, 1, 1, True, False),
    ((2, 3, 18), (4, 3, 3), True, 1, 1, 1, 1, False, True),
    ((8, 64, 4096), (128, 64, 5), True, 1, 2, 1, 1, False, False),   # large enough for the tensor-core path
]


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16", "float16", "float64"])
@pytest.mark.parametrize("case", CONV1D_CASES, ids=[str(i) for i in range(len(CONV1D_CASES))])
def test_conv1d_matches_torch_cpu(fd, case, dtype_name):
    ishape, wshape, has_bias, stride, padding, dilation, groups, unbatched, noncontig = case
    dtype = DTYPES[dtype_name]
    g = torch.Generator().manual_seed(5)
    if noncontig:
        x = torch.randn(tuple(ishape[:-1]) + (ishape[-1] * 2,), generator=g).to(dtype).cuda()[..., ::2]
    else:
        x = torch.randn(ishape, generator=g).to(dtype).cuda()
    fan_in = wshape[1] * wshape[2]
    w = (torch.randn(wshape, generator=g) * fan_in ** -0.5).to(dtype).cuda()
    b = (torch.randn(wshape[0], generator=g) * 0.1).to(dtype).cuda() if has_bias else None
    out = fd.conv1d(x, w, b, stride=stride, padding=padding, dilation=dilation, groups=groups)
    cdt = torch.float64 if dtype_name == "float64" else torch.float32
    ref = torch.nn.functional.conv1d(x.cpu().to(cdt), w.cpu().to(cdt), None if b is None else b.cpu().to(cdt),
                                     stride=stride, padding=padding, dilation=dilation, groups=groups)
    assert out.shape == ref.shape and out.dtype == dtype and out.is_contiguous()
    _check(out, ref, dtype_name)


MM_CASES = [(0, 3, 4), (2, 0, 4), (2, 3, 0), (2, 3, 4), (7, 5, 3), (16, 17, 15), (32, 64, 16),   # the reference's
            (300, 256, 520), (4096, 1024, 256), (129, 72, 8)]


@pytest.mark.parametrize("use_out", [False, True])
@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16", "float16", "float64"])
@pytest.mark.parametrize("case", MM_CASES, ids=["x".join(map(str, c)) for c in MM_CASES])
def test_mm_matches_torch_cpu(fd, case, dtype_name, use_out):
    """mm as a 1x1 convolution over a row of M pixels, the reference's cases (tests/test_mm.py:9-17) and larger."""
    m, k, n = case
    dtype = getattr(torch, dtype_name)
    a = torch.empty(m, k).uniform_(-1, 1, generator=torch.Generator().manual_seed(5)).to(dtype).cuda()
    b = torch.empty(k, n).uniform_(-1, 1, generator=torch.Generator().manual_seed(6)).to(dtype).cuda()
    a0, b0 = a.clone(), b.clone()
    cdt = torch.float64 if dtype_name == "float64" else torch.float32
    ref = torch.mm(a.cpu().to(cdt), b.cpu().to(cdt))
    if use_out:
        buf = torch.empty(m, n, dtype=dtype, device="cuda")
        got = fd.mm(a, b, out=buf)
        assert got.data_ptr() == buf.data_ptr()
    else:
        got = fd.mm(a, b)
    assert got.shape == (m, n) and got.dtype == dtype
    # the reference's own test allows atol = 1e-4 * K (tests/test_mm.py:27-30 with reduce_dim=k); here the
    # absolute part grows with sqrt(K) only, the relative part is the dtype's usual one
    tol = dict(TOL[dtype_name])
    tol["atol"] = tol["atol"] * max(1.0, k ** 0.5)
    torch.testing.assert_close(got.cpu().to(cdt), ref, **tol)
    assert torch.equal(a, a0) and torch.equal(b, b0)


@pytest.mark.parametrize("use_out", [False, True])
@pytest.mark.parametrize("dtype_name", ["bfloat16", "float16"])
@pytest.mark.parametrize("case", MM_CASES, ids=["x".join(map(str, c)) for c in MM_CASES])
def test_mm_float32_result_from_16_bit_operands(fd, case, dtype_name, use_out):
    """out_dtype=torch.float32 with fp16 / bf16 operands (src/flag_dnn/ops/mm.py:123-131): the fp32 accumulators
    are stored unrounded, so the result is within fp32 summation-order error of an fp32 product of the same
    (already rounded) operands, far inside what a 16-bit output could hold."""
    m, k, n = case
    dtype = getattr(torch, dtype_name)
    a = torch.empty(m, k).uniform_(-1, 1, generator=torch.Generator().manual_seed(7)).to(dtype).cuda()
    b = torch.empty(k, n).uniform_(-1, 1, generator=torch.Generator().manual_seed(8)).to(dtype).cuda()
    ref = torch.mm(a.cpu().double(), b.cpu().double())
    if use_out:
        buf = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
        got = fd.mm(a, b, torch.float32, out=buf)
        assert got.data_ptr() == buf.data_ptr()
    else:
        got = fd.mm(a, b, out_dtype=torch.float32)
    assert got.shape == (m, n) and got.dtype == torch.float32
    torch.testing.assert_close(got.cpu().double(), ref, rtol=1e-5, atol=2e-6 * max(1.0, k ** 0.5))
    if m * n * k:
        # and it is not the 16-bit result widened: a rounded output differs from this one
        narrow = fd.mm(a, b).float()
        assert (narrow - got).abs().max().item() > 0 or k == 1


def test_mm_strided_operands_and_checks(fd):
    a = torch.randn(64, 96, device="cuda")[:, ::2]            # non-contiguous left operand
    b = torch.randn(40, 48, device="cuda").t()                # transposed right operand: [48, 40]
    torch.testing.assert_close(fd.mm(a, b).cpu(), torch.mm(a.cpu(), b.cpu()), rtol=1e-4, atol=1e-4)
    out = torch.empty(40, 64, device="cuda").t()              # non-contiguous out: result is copied back
    got = fd.mm(a, b, out=out)
    assert got is out
    torch.testing.assert_close(out.cpu(), torch.mm(a.cpu(), b.cpu()), rtol=1e-4, atol=1e-4)
    with pytest.raises(RuntimeError, match="self must be a matrix"):
        fd.mm(torch.randn(2, 3, 4, device="cuda"), b)
    with pytest.raises(RuntimeError, match="cannot be multiplied"):
        fd.mm(torch.randn(2, 3, device="cuda"), torch.randn(4, 5, device="cuda"))
    with pytest.raises(RuntimeError, match="same dtype"):
        fd.mm(torch.randn(2, 3, device="cuda"), torch.randn(3, 5, device="cuda", dtype=torch.float16))
    with pytest.raises(NotImplementedError):
        fd.mm(torch.randn(2, 3, device="cuda", dtype=torch.complex64), torch.randn(3, 5, device="cuda", dtype=torch.complex64))
    with pytest.raises(RuntimeError, match="Expected out tensor to have dtype torch.float32"):
        fd.mm(torch.randn(2, 3, device="cuda", dtype=torch.float16), torch.randn(3, 5, device="cuda", dtype=torch.float16),
              out_dtype=torch.float32, out=torch.empty(2, 5, device="cuda", dtype=torch.float16))
    with pytest.raises(RuntimeError, match="out_dtype must be"):
        fd.mm(torch.randn(2, 3, device="cuda"), torch.randn(3, 5, device="cuda"), out_dtype=torch.float16)


def test_aten_override_routes_functional_conv2d(fd):
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 16, 12, 12, generator=g).cuda()
    w = torch.randn(8, 16, 3, 3, generator=g).cuda()
    b = torch.randn(8, generator=g).cuda()
    with fd.use_dnn():
        out = torch.nn.functional.conv2d(x, w, b, stride=1, padding=1)
    ref = oracle.conv2d_torch_cpu(x, w, b, 1, 1, 1, 1)
    _check(out, ref, "float32")


def _rand(shape, seed, std=1.0, dist="normal"):
    g = torch.Generator().manual_seed(seed)
    if dist == "uniform":
        return torch.rand(shape, generator=g) * 2 - 1
    return torch.randn(shape, generator=g) * std


# Benchmark configurations at a batch the CPU oracle finishes in seconds.
BENCH_SMALL = [
    # name, N, C, H, K, R, stride, pad, dtype, layout, x dist
    ("c1_fp32_nchw_3x3", 4, 64, 56, 64, 3, 1, 1, "float32", "nchw", "normal"),
    ("c2_bf16_1x1", 8, 256, 56, 64, 1, 1, 0, "bfloat16", "nhwc", "normal"),
    ("c3_bf16_3x3_256", 8, 256, 14, 256, 3, 1, 1, "bfloat16", "nhwc", "normal"),
    ("c4_bf16_stem_7x7", 4, 3, 224, 64, 7, 2, 3, "bfloat16", "nhwc", "uniform"),
]


@pytest.mark.parametrize("cfg", BENCH_SMALL, ids=[c[0] for c in BENCH_SMALL])
def test_benchmark_configs_reduced_batch(fd, cfg):
    name, n, c, hw, k, r, stride, pad, dtype_name, layout, dist = cfg
    dtype = DTYPES[dtype_name]
    x = _rand((n, c, hw, hw), 0, dist=dist)
    w = _rand((k, c, r, r), 1, std=(c * r * r) ** -0.5)
    b = _rand((k,), 2, std=0.1)
    cl = layout == "nhwc"
    xd, wd, bd = _to_dev(x, dtype, cl), _to_dev(w, dtype, cl), _to_dev(b, dtype, False)
    plan = fd.conv2d_plan(xd, wd, stride=stride, padding=pad)
    assert plan["algo"] in (2, 3), "benchmark configurations must take the tensor-core path"
    out = fd.fused_conv2d_bias_relu(xd, wd, bd, stride=stride, padding=pad)
    ref = oracle.conv2d_torch_cpu(xd, wd, bd, stride, pad, 1, 1, relu=True)
    _check(out, ref, dtype_name)
    # second, independent oracle leg on one image (plain loops, double accumulate)
    ref_loops = oracle.conv2d_loops(xd[:1], wd, bd, stride, pad, 1, 1, relu=True)
    _check(out[:1], ref_loops, dtype_name)


FULL = [
    ("c2_bf16_1x1", 256, 256, 56, 64, 1, 1, 0),
    ("c3_bf16_3x3_256", 256, 256, 14, 256, 3, 1, 1),
    ("c4_bf16_stem_7x7", 256, 3, 224, 64, 7, 2, 3),
]


@pytest.mark.parametrize("cfg", FULL, ids=[c[0] for c in FULL])
def test_benchmark_configs_full_size_properties(fd, cfg):
    """At the benchmark batch: every image against the reference's CPU call in the tensors' own dtype
    (torch.nn.functional.conv2d + relu in bf16, src/flag_dnn/graph/registry.py:1357-1365, 1426 — fast on the host's
    matrix units, its own result rounded to bf16), sampled images against the fp32 oracle, and the
    size-independent properties: images are independent (a batch slice run alone gives the same answer), the
    result is deterministic, ReLU output is non-negative, the convolution is linear."""
    name, n, c, hw, k, r, stride, pad = cfg
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((n, c, hw, hw), generator=g, device="cuda", dtype=torch.float32)
    x = x.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    w = (_rand((k, c, r, r), 1, std=(c * r * r) ** -0.5)).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    b = _rand((k,), 2, std=0.1).to(torch.bfloat16).cuda()
    out = fd.fused_conv2d_bias_relu(x, w, b, stride=stride, padding=pad)
    again = fd.fused_conv2d_bias_relu(x, w, b, stride=stride, padding=pad)
    assert torch.equal(out, again)
    assert (out >= 0).all()
    picks = [0, n // 2 + 1, n - 1]
    plan_full = fd.conv2d_plan(x, w, stride=stride, padding=pad)
    for i in picks:
        alone = fd.fused_conv2d_bias_relu(x[i:i + 1], w, b, stride=stride, padding=pad)
        plan_one = fd.conv2d_plan(x[i:i + 1], w, stride=stride, padding=pad)
        if (plan_one["low_channel"], plan_one["pixel_group"]) == (plan_full["low_channel"], plan_full["pixel_group"]):
            # same reduction order in both kernels: bit for bit
            assert torch.equal(alone, out[i:i + 1])
        else:
            # one image alone takes another operand layout (the stem: 4 stored channels instead of 3), which adds
            # the same products in another order: fp32 sums differ in the last bits, outputs by one bf16 step at most
            a, bb = alone.float(), out[i:i + 1].float()
            assert (a - bb).abs().max() <= 2.0 ** -7 * bb.abs().max() and (alone != out[i:i + 1]).float().mean() < 1e-2
    # two different batch slices of the full plan's own size class agree bit for bit
    half = fd.fused_conv2d_bias_relu(x[n // 2:], w, b, stride=stride, padding=pad)
    if fd.conv2d_plan(x[n // 2:], w, stride=stride, padding=pad)["low_channel"] == plan_full["low_channel"]:
        assert torch.equal(half, out[n // 2:])
    ref = oracle.conv2d_torch_cpu(x[picks], w, b, stride, pad, 1, 1, relu=True)
    _check(out[picks], ref, "bfloat16")
    # all n images, in chunks, against the CPU call in bf16: both sides round once to bf16, so they may differ by
    # one bf16 step (2^-8 relative) where the fp32 values straddle a rounding boundary
    out_cpu = out.cpu()
    for i0 in range(0, n, 32):
        ref16 = oracle.conv2d_torch_cpu(x[i0:i0 + 32], w, b, stride, pad, 1, 1, relu=True, compute_dtype=torch.bfloat16)
        torch.testing.assert_close(out_cpu[i0:i0 + 32].float(), ref16.float(), rtol=1e-2, atol=1e-2)
    # linearity of the convolution part: conv(2x) == 2 conv(x) exactly in binary floating point
    y1 = fd.conv2d(x[:4], w, None, stride=stride, padding=pad)
    y2 = fd.conv2d(x[:4] * 2, w, None, stride=stride, padding=pad)
    assert torch.equal(y2, y1 * 2)


def test_scale_bias_epilogue_variants(fd):
    x = _rand((3, 32, 10, 9), 10).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    w = _rand((40, 32, 3, 3), 11, std=0.06).to(torch.bfloat16).cuda()
    b = _rand((40,), 12, std=0.1).to(torch.bfloat16).cuda()
    s = (torch.rand(40, generator=torch.Generator().manual_seed(13)) + 0.5).to(torch.bfloat16).cuda()
    for algo in ("igemm", "pair", "direct"):
        fd.set_algo(algo)
        try:
            got = fd.fused_conv2d_bias_relu(x, w, b, padding=1, scale=s)
            ref = oracle.conv2d_torch_cpu(x, w, b, 1, 1, 1, 1, scale=s, relu=True)
            _check(got, ref, "bfloat16")
            got = fd.fused_conv2d_bias_relu(x, w, b, padding=1, scale=s, activation="none")
            ref = oracle.conv2d_torch_cpu(x, w, b, 1, 1, 1, 1, scale=s, relu=False)
            _check(got, ref, "bfloat16")
            got = fd.conv2d(x, w, None, padding=1)
            ref = oracle.conv2d_torch_cpu(x, w, None, 1, 1, 1, 1)
            _check(got, ref, "bfloat16")
        finally:
            fd.set_algo("auto")


@pytest.mark.parametrize("shape", [(5, 192, 20, 20, 320, 3, 1, 1), (2, 64, 40, 33, 256, 1, 1, 0), (3, 128, 17, 17, 600, 3, 2, 1)])
def test_pair_kernel_matches_single_cta_kernel_bitwise(fd, shape):
    """Both tensor-core kernels accumulate the same products in the same order."""
    n, c, h, w_, k, r, stride, pad = shape
    x = _rand((n, c, h, w_), 50).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    w = _rand((k, c, r, r), 51, std=(c * r * r) ** -0.5).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    b = _rand((k,), 52, std=0.1).to(torch.bfloat16).cuda()
    outs = {}
    for algo in ("igemm", "pair"):
        fd.set_algo(algo)
        try:
            outs[algo] = fd.fused_conv2d_bias_relu(x, w, b, stride=stride, padding=pad)
        finally:
            fd.set_algo("auto")
    assert torch.equal(outs["igemm"], outs["pair"])
    _check(outs["pair"], oracle.conv2d_torch_cpu(x, w, b, stride, pad, 1, 1, relu=True), "bfloat16")


def _pair2(v):
    return (v, v) if isinstance(v, int) else tuple(v)


LOWC = [
    # n, c, h, w, k, r, s, stride, pad, dtype
    (2, 3, 32, 32, 64, 7, 7, 2, 3, "bfloat16"),            # the stem at a small image
    (3, 3, 40, 24, 16, 3, 3, 1, 1, "bfloat16"),            # stride 1, 4*K = 64 GEMM columns
    (2, 4, 19, 64, 40, 3, 5, (1, 2), (1, 2), "float16"),   # 4 channels, rectangular filter, odd left padding
    (1, 2, 9, 16, 8, 1, 1, 1, 0, "bfloat16"),              # 1x1 filter, one tile
    (2, 2, 33, 48, 32, 5, 4, 2, (2, 2), "float16"),        # 25 output columns: not whole quads, generic path
    (2, 1, 33, 52, 32, 5, 4, 2, (2, 2), "float16"),        # one channel (torch then reports an NCHW-like view)
    (1, 3, 70, 520, 8, 3, 3, (3, 1), 1, "bfloat16"),       # 130 quads per row: more than one tile may hold
    (3, 3, 40, 48, 32, 3, 3, 2, 1, "float16"),             # 3x3 stride 2: 128 GEMM columns, 32 window elements used
    (2, 3, 37, 128, 64, 5, 5, 2, 2, "bfloat16"),           # 5x5 stride 2, 19 output rows in tiles of 8: ragged last tile
    (5, 3, 64, 64, 64, 7, 7, 2, 3, "bfloat16"),            # the stem, an odd number of tiles for the pairs
]


@pytest.mark.parametrize("algo", ["igemm", "pair"])
@pytest.mark.parametrize("case", LOWC, ids=[f"c{c[1]}_{c[5]}x{c[6]}_k{c[4]}_w{c[3]}" for c in LOWC])
def test_low_channel_path_matches_oracle(fd, case, algo):
    """C <= 4 with channels-last tensors: pixel quads become GEMM rows over 16-pixel input windows."""
    n, c, h, w_, k, r, s_, stride, pad, dtype_name = case
    dtype = DTYPES[dtype_name]
    x = _rand((n, c, h, w_), 60, dist="uniform").to(dtype).cuda().contiguous(memory_format=torch.channels_last)
    w = _rand((k, c, r, s_), 61, std=(c * r * s_) ** -0.5).to(dtype).cuda().contiguous(memory_format=torch.channels_last)
    b = _rand((k,), 62, std=0.1).to(dtype).cuda()
    sc = (torch.rand(k, generator=torch.Generator().manual_seed(63)) + 0.5).to(dtype).cuda()
    channels_last_out = x.stride(1) == 1  # the output follows the input's layout
    if algo == "pair" and not channels_last_out:
        pytest.skip("the CTA-pair kernel writes channels-last outputs only")
    fd.set_algo(algo)
    try:
        plan = fd.conv2d_plan(x, w, stride=stride, padding=pad)
        got = fd.fused_conv2d_bias_relu(x, w, b, stride=stride, padding=pad, scale=sc)
        again = fd.fused_conv2d_bias_relu(x, w, b, stride=stride, padding=pad, scale=sc)
    finally:
        fd.set_algo("auto")
    expect_lowc = channels_last_out and (got.shape[3] % 4 == 0) and got.shape[3] // 4 <= 128
    assert bool(plan["low_channel"]) == expect_lowc
    # on CTA pairs a dense 3-channel input with an even W-stride is read without the relayout pass (mode 2)
    fused3 = algo == "pair" and c == 3 and expect_lowc and _pair2(stride)[1] % 2 == 0 and (3 * w_) % 8 == 0
    assert plan["low_channel"] == (2 if fused3 else int(expect_lowc))
    assert torch.equal(got, again)
    _check(got, oracle.conv2d_torch_cpu(x, w, b, stride, pad, 1, 1, scale=sc, relu=True), dtype_name)


def test_stem_without_relayout_many_tiles_and_unaligned_input(fd):
    """The 3-channel mode of the pair kernel over enough tiles that every CTA reuses both of its scratch slots
    several times (slot hand-over between the converter warps, the copy-issuing thread and the MMA issuer), and on
    an input whose first element is not 16-byte aligned (pieces are then read element by element)."""
    n, hw, k = 96, 112, 64
    store = _rand((n * hw * hw * 3 + 8,), 64, dist="uniform").to(torch.bfloat16).cuda()
    w = _rand((k, 3, 7, 7), 65, std=147 ** -0.5).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    b = _rand((k,), 66, std=0.1).to(torch.bfloat16).cuda()
    fd.set_algo("pair")
    try:
        for offset in (0, 1):
            x = store[offset:offset + n * hw * hw * 3].view(n, hw, hw, 3).permute(0, 3, 1, 2)
            assert (x.data_ptr() % 16 != 0) == bool(offset)
            plan = fd.conv2d_plan(x, w, stride=2, padding=3)
            assert plan["low_channel"] == 2 and plan["launches"] == 1 and plan["x_repacked"] == 0
            assert plan["grid"] == 148 and n * 56 * 56 // 4 // 112 > 4 * 148, "several tiles per CTA"
            got = fd.fused_conv2d_bias_relu(x, w, b, stride=2, padding=3)
            again = fd.fused_conv2d_bias_relu(x, w, b, stride=2, padding=3)
            assert torch.equal(got, again)
            ref16 = oracle.conv2d_torch_cpu(x, w, b, 2, 3, 1, 1, relu=True, compute_dtype=torch.bfloat16)
            torch.testing.assert_close(got.float().cpu(), ref16.float(), rtol=1e-2, atol=1e-2)
            picks = [0, 17, n - 1]
            _check(got[picks], oracle.conv2d_torch_cpu(x[picks], w, b, 2, 3, 1, 1, relu=True), "bfloat16")
    finally:
        fd.set_algo("auto")


GROUPED = [
    # n, c, hw, k, r, stride, pad, expected pixel group
    (20, 64, 56, 64, 3, 1, 1, 4),     # ResNet stage-1 3x3: four pixels per GEMM row, 256 columns
    (24, 128, 56, 128, 3, 2, 1, 2),   # stride-2 3x3 at 128 channels: pairs
    (40, 128, 28, 128, 3, 1, 1, 2),
    (24, 64, 54, 64, 3, 1, 1, 2),     # 54 output columns: pairs divide, quads do not
]


@pytest.mark.parametrize("case", GROUPED, ids=[f"c{c[1]}_hw{c[2]}_s{c[5]}" for c in GROUPED])
def test_pixel_grouped_narrow_layers_match_oracle(fd, case):
    """Narrow layers run as an equivalent convolution whose rows are groups of output pixels."""
    n, c, hw, k, r, stride, pad, group = case
    x = _rand((n, c, hw, hw), 70).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    w = _rand((k, c, r, r), 71, std=(c * r * r) ** -0.5).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    b = _rand((k,), 72, std=0.1).to(torch.bfloat16).cuda()
    sc = (torch.rand(k, generator=torch.Generator().manual_seed(73)) + 0.5).to(torch.bfloat16).cuda()
    plan = fd.conv2d_plan(x, w, stride=stride, padding=pad)
    assert plan["pixel_group"] == group and plan["w_packed"] == 1
    got = fd.fused_conv2d_bias_relu(x, w, b, stride=stride, padding=pad, scale=sc)
    fd.set_algo("direct")  # the plain CUDA-core kernel as an in-library second opinion
    try:
        plain = fd.fused_conv2d_bias_relu(x[:2], w, b, stride=stride, padding=pad, scale=sc)
    finally:
        fd.set_algo("auto")
    torch.testing.assert_close(got[:2].float(), plain.float(), rtol=1e-2, atol=1e-2)
    picks = [0, n // 2, n - 1]
    ref = oracle.conv2d_torch_cpu(x[picks], w, b, stride, pad, 1, 1, scale=sc, relu=True)
    _check(got[picks], ref, "bfloat16")
    # every image, against the library's own ungrouped result on a different batch split
    alone = fd.fused_conv2d_bias_relu(x[3:4], w, b, stride=stride, padding=pad, scale=sc)  # small: not grouped
    assert torch.equal(alone, got[3:4])


RESIDUAL = [
    # name, (n, c, hw, k, r, stride, pad, groups), dtype, channels_last, algo, residual layout matches
    ("nhwc_bf16", (6, 64, 28, 256, 1, 1, 0, 1), "bfloat16", True, "igemm", True),
    ("nhwc_f16_ragged_k", (3, 40, 19, 72, 3, 1, 1, 1), "float16", True, "igemm", True),   # 72 columns: partial group
    ("nhwc_f32", (2, 32, 17, 96, 3, 2, 1, 1), "float32", True, "igemm", True),
    ("pair_bf16", (5, 128, 20, 512, 1, 1, 0, 1), "bfloat16", True, "pair", True),
    ("nchw_bf16", (3, 24, 15, 40, 3, 1, 1, 1), "bfloat16", False, "igemm", True),          # strided per-element epilogue
    ("nchw_f32", (2, 16, 12, 20, 3, 1, 1, 1), "float32", False, "igemm", True),
    ("direct_groups", (2, 16, 12, 24, 3, 1, 1, 4), "float16", True, "auto", True),
    ("direct_f64", (2, 8, 9, 12, 3, 1, 1, 1), "float64", False, "auto", True),
    ("grouped_pixels", (20, 64, 56, 64, 3, 1, 1, 1), "bfloat16", True, "auto", True),      # pixel-grouped layer
    ("low_channel", (4, 3, 64, 32, 7, 2, 3, 1), "bfloat16", True, "auto", True),           # separate add + ReLU steps
    ("other_layout", (3, 64, 14, 128, 1, 1, 0, 1), "bfloat16", True, "igemm", False),      # NCHW shortcut, NHWC output
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", RESIDUAL, ids=[c[0] for c in RESIDUAL])
def test_residual_add_in_the_epilogue(fd, case):
    """act(conv * scale + bias + shortcut) against the fp32/fp64 CPU answer for the same bits."""
    _, (n, c, hw, k, r, stride, pad, groups), dtype_name, channels_last, algo, same_layout = case
    dtype = getattr(torch, dtype_name)
    x = _to_dev(_rand((n, c, hw, hw), 90), dtype, channels_last)
    w = _to_dev(_rand((k, c // groups, r, r), 91, std=(c // groups * r * r) ** -0.5), dtype, channels_last)
    b = _rand((k,), 92, std=0.1).to(dtype).cuda()
    sc = (torch.rand(k, generator=torch.Generator().manual_seed(93)) + 0.5).to(dtype).cuda()
    oh = (hw + 2 * pad - r) // stride + 1
    shortcut = _to_dev(_rand((n, k, oh, oh), 94), dtype, channels_last == same_layout)
    fd.set_algo(algo)
    try:
        for relu in (True, False):
            for use_scale, use_bias in ((True, True), (False, False)):
                got = fd.conv2d_bias_act(x, w, b if use_bias else None, stride=stride, padding=pad, groups=groups,
                                         scale=sc if use_scale else None, relu=relu, residual=shortcut)
                cdt = torch.float64 if dtype_name == "float64" else torch.float32
                ref = oracle.conv2d_torch_cpu(x, w, b if use_bias else None, stride, pad, 1, groups,
                                              scale=sc if use_scale else None, compute_dtype=cdt)
                ref = ref + shortcut.cpu().to(cdt)
                if relu:
                    ref = torch.relu(ref)
                _check(got, ref, dtype_name)
                assert got.stride() == fd.conv2d(x, w, None, stride, pad, 1, groups).stride()
    finally:
        fd.set_algo("auto")


@pytest.mark.gpu
def test_residual_contract(fd):
    x = torch.randn(2, 16, 8, 8, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(24, 16, 3, 3, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="residual must have the shape"):
        fd.conv2d_bias_act(x, w, None, padding=1, residual=torch.zeros(2, 24, 8, 7, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(RuntimeError, match="residual must have the shape"):
        fd.conv2d_bias_act(x, w, None, padding=1, residual=torch.zeros(2, 24, 8, 8, device="cuda", dtype=torch.float16))
    # NaN in the shortcut survives the ReLU, as torch.relu(conv + shortcut) would keep it
    shortcut = torch.zeros(2, 24, 8, 8, device="cuda", dtype=torch.bfloat16)
    shortcut[1, 5, 2, 3] = float("nan")
    for cl in (True, False):
        xs = x.contiguous(memory_format=torch.channels_last) if cl else x
        sh = shortcut.contiguous(memory_format=torch.channels_last) if cl else shortcut
        out = fd.conv2d_bias_act(xs, w, None, padding=1, relu=True, residual=sh)
        assert torch.isnan(out[1, 5, 2, 3]) and int(torch.isnan(out).sum()) == 1


@pytest.mark.parametrize("approximate", ["none", "tanh"])
@pytest.mark.parametrize("dtype_name,channels_last,groups", [("bfloat16", True, 1), ("float16", False, 1),
                                                             ("float32", True, 1), ("float64", False, 1),
                                                             ("float16", True, 4)])
def test_gelu_epilogue(fd, dtype_name, channels_last, groups, approximate):
    """gelu(conv * scale + bias) in the epilogue of every kernel family, both GELU forms, through the graph."""
    dtype = getattr(torch, dtype_name)
    n, c, hw, k = 3, 32, 13, 72
    x = _to_dev(_rand((n, c, hw, hw), 120), dtype, channels_last)
    w = _to_dev(_rand((k, c // groups, 3, 3), 121, std=(c // groups * 9) ** -0.5), dtype, channels_last)
    b = _rand((k,), 122, std=0.5).to(dtype).cuda()
    cdt = torch.float64 if dtype_name == "float64" else torch.float32
    ref = torch.nn.functional.gelu(oracle.conv2d_torch_cpu(x, w, b, 1, 1, 1, groups, compute_dtype=cdt),
                                   approximate=approximate)

    @fd.graph
    def layer(x, w, b):
        return fd.gelu(fd.bias_add(fd.conv2d(x, w, padding=1, groups=groups), b), approximate=approximate)

    compiled = fd.compile(layer, inputs=[x, w, b], options={"cache": None})
    assert [nd.op_type for nd in compiled.graph.nodes] == ["fused_conv2d_bias_gelu"]
    _check(compiled.run(x, w, b), ref, dtype_name)
    got = fd.conv2d_bias_act(x, w, b, padding=1, groups=groups,
                             activation="gelu_tanh" if approximate == "tanh" else "gelu")
    _check(got, ref, dtype_name)
    if dtype_name == "bfloat16":
        x_nan = x.clone()
        x_nan[0, 0, 0, 0] = float("nan")
        out = fd.conv2d_bias_act(x_nan, w, b, padding=1, activation="gelu")
        assert torch.isnan(out[0, :, 0, 0]).all() and not torch.isnan(out[1:]).any()


@pytest.mark.parametrize("dtype_name", ["float32", "bfloat16", "float16"])
def test_next_rows_match_reference_cpu_outputs(fd, golden_next, dtype_name):
    """Block tails, conv->bias->GELU and mm against what the unmodified reference computed on CPU."""
    dtype = getattr(torch, dtype_name)

    def dev(name, channels_last=True):
        return _to_dev(torch.from_numpy(golden_next[name]), dtype, channels_last)

    def cpu32(t):
        return t.detach().float().cpu()

    for idx in range(3):
        key = f"tail_{idx:02d}"
        x, w, r = dev(key + "_x"), dev(key + "_w"), dev(key + "_r")
        s, b = dev(key + "_s", False), dev(key + "_b", False)
        stride, padding = (int(v) for v in golden_next[key + "_meta"])

        @fd.graph
        def tail(x, weight, scale, bias, shortcut):
            y = fd.bias_add(fd.conv2d(x, weight, stride=stride, padding=padding) * scale, bias)
            return fd.relu(y + shortcut)

        compiled = fd.compile(tail, inputs=[x, w, s, b, r], options={"cache": None})
        assert [n.op_type for n in compiled.graph.nodes] == ["fused_conv2d_bias_add_relu"]
        got = compiled.run(x, w, s, b, r)
        # the reference saw fp32 inputs; here they were rounded to `dtype` first, so compare with the oracle
        # on the rounded bits and, for fp32, with the stored reference output itself
        ref = torch.relu(oracle.conv2d_torch_cpu(x, w, b, stride, padding, 1, 1, scale=s.reshape(-1)) + cpu32(r))
        _check(got, ref, dtype_name)
        if dtype_name == "float32":
            _check(got, torch.from_numpy(golden_next[key + "_y"]), dtype_name)

    for idx in range(2):
        key = f"gelu_{idx:02d}"
        x, w, b = dev(key + "_x"), dev(key + "_w"), dev(key + "_b", False)
        stride, padding, tanh = (int(v) for v in golden_next[key + "_meta"])
        got = fd.conv2d_bias_act(x, w, b, stride=stride, padding=padding, activation="gelu_tanh" if tanh else "gelu")
        ref = torch.nn.functional.gelu(oracle.conv2d_torch_cpu(x, w, b, stride, padding, 1, 1),
                                       approximate="tanh" if tanh else "none")
        _check(got, ref, dtype_name)
        if dtype_name == "float32":
            _check(got, torch.from_numpy(golden_next[key + "_y"]), dtype_name)

    for idx in range(5):
        key = f"mm_{idx:02d}"
        a, b = dev(key + "_a", False), dev(key + "_b", False)
        got = fd.mm(a, b)
        _check(got, torch.mm(cpu32(a), cpu32(b)), dtype_name)
        if dtype_name == "float32":
            _check(got, torch.from_numpy(golden_next[key + "_y"]), dtype_name)


def test_scaled_graph_folds_into_one_node(fd):
    x = _rand((2, 16, 8, 8), 20).to(torch.float16).cuda().contiguous(memory_format=torch.channels_last)
    w = _rand((24, 16, 3, 3), 21, std=0.08).to(torch.float16).cuda()
    s = (torch.rand(24, generator=torch.Generator().manual_seed(22)) + 0.5).to(torch.float16).cuda()
    b = _rand((24,), 23, std=0.1).to(torch.float16).cuda()

    @fd.graph
    def fn(x, w, s, b):
        return fd.relu(fd.bias_add(fd.conv2d(x, w, padding=1) * s, b))

    compiled = fd.compile(fn, inputs=[x, w, s.reshape(1, 24, 1, 1), b], options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["fused_conv2d_bias_relu"]
    out = compiled.run(x, w, s.reshape(1, 24, 1, 1), b)
    ref = oracle.conv2d_torch_cpu(x, w, b, 1, 1, 1, 1, scale=s, relu=True)
    _check(out, ref, "float16")


def test_ragged_and_strided_inputs(fd):
    # M not a multiple of the 128-row tile, channels not a multiple of 8, output
    # channels not a multiple of 32, and a non-dense channels-last view.
    base = _rand((3, 24, 13, 17), 30).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    x = base[:, :16]  # channel slice: unit channel stride, pixel stride 24
    w = _rand((37, 16, 3, 3), 31, std=0.08).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    b = _rand((37,), 32, std=0.1).to(torch.bfloat16).cuda()
    for algo in ("igemm", "direct"):  # 37 output channels: no 16-byte rows, so not the pair kernel
        fd.set_algo(algo)
        try:
            got = fd.fused_conv2d_bias_relu(x, w, b, stride=(2, 1), padding=(1, 2), dilation=(1, 2))
        finally:
            fd.set_algo("auto")
        ref = oracle.conv2d_torch_cpu(x, w, b, (2, 1), (1, 2), (1, 2), 1, relu=True)
        _check(got, ref, "bfloat16")
    x5 = _rand((2, 5, 9, 9), 33).to(torch.float16).cuda()
    w5 = _rand((3, 5, 2, 4), 34, std=0.2).to(torch.float16).cuda()
    fd.set_algo("igemm")
    try:
        got = fd.conv2d(x5, w5, None, padding=(1, 3))
    finally:
        fd.set_algo("auto")
    _check(got, oracle.conv2d_torch_cpu(x5, w5, None, 1, (1, 3), 1, 1), "float16")


def test_empty_and_degenerate_outputs(fd):
    w = torch.randn(4, 3, 3, 3, device="cuda")
    out = fd.conv2d(torch.randn(0, 3, 8, 8, device="cuda"), w, None, padding=1)
    assert out.shape == (0, 4, 8, 8)
    out = fd.conv2d(torch.randn(2, 3, 2, 9, device="cuda"), w, None)  # kernel taller than the image
    assert out.shape == (2, 4, 0, 7)
    with pytest.raises(RuntimeError, match="negative"):
        fd.conv2d(torch.randn(2, 3, 1, 9, device="cuda"), torch.randn(4, 3, 5, 5, device="cuda"), None)


def test_fused_entry_contract_errors(fd):
    x = torch.randn(1, 4, 8, 8, device="cuda")
    w = torch.randn(4, 2, 3, 3, device="cuda")
    b = torch.randn(4, device="cuda")
    with pytest.raises(NotImplementedError):
        fd.fused_conv2d_bias_relu(x, w, b, groups=2)
    with pytest.raises(NotImplementedError):
        fd.fused_conv2d_bias_relu(x.double(), torch.randn(4, 4, 3, 3, device="cuda").double(), b.double())
    with pytest.raises(RuntimeError):
        fd.fused_conv2d_bias_relu(x, torch.randn(4, 4, 3, 3, device="cuda").half(), b)

    # the graph executor still runs a grouped fused node, through the direct kernel
    @fd.graph
    def fn(x, w, b):
        return fd.relu(fd.bias_add(fd.conv2d(x, w, padding=1, groups=2), b))

    compiled = fd.compile(fn, inputs=[x, w, b], options={"cache": None})
    assert [n.op_type for n in compiled.graph.nodes] == ["fused_conv2d_bias_relu"]
    _check(compiled.run(x, w, b), oracle.conv2d_torch_cpu(x, w, b, 1, 1, 1, 2, relu=True), "float32")


def test_host_buffer_entry_point(fd, native_lib):
    """fdnn_conv2d_fwd_host: host pointers in, host pointer out."""
    import ctypes

    from flagdnn_b200 import _native as nat

    x = _rand((2, 16, 9, 9), 40).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    w = _rand((24, 16, 3, 3), 41, std=0.1).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    b = _rand((24,), 42, std=0.1).to(torch.bfloat16)
    y = torch.empty((2, 24, 9, 9), dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    d = nat.ConvDesc()
    d.dtype = nat.BF16
    d.n, d.c, d.h, d.w = x.shape
    d.k, _, d.r, d.s = w.shape
    d.stride_h = d.stride_w = d.dil_h = d.dil_w = d.groups = 1
    d.pad_top = d.pad_bottom = d.pad_left = d.pad_right = 1
    d.algo = nat.ALGO_IGEMM
    for i in range(4):
        d.x_strides[i], d.w_strides[i], d.y_strides[i] = x.stride(i), w.stride(i), y.stride(i)
    need = ctypes.c_int64(0)
    nat.check(native_lib.fdnn_conv2d_host_arena_bytes(ctypes.byref(d), ctypes.byref(need)))
    arena = torch.empty(need.value, dtype=torch.uint8, device="cuda")
    nat.check(native_lib.fdnn_conv2d_fwd_host(ctypes.byref(d), x.data_ptr(), w.data_ptr(), b.data_ptr(), None,
                                              nat.ACT_RELU, y.data_ptr(), arena.data_ptr(), need.value, None))
    _check(y, oracle.conv2d_torch_cpu(x, w, b, 1, 1, 1, 1, relu=True), "bfloat16")


DEPTHWISE = [
    # n, c, h, w, r, s, stride, pad, dilation, dtype, channels_last
    (4, 32, 112, 112, 3, 3, 1, 1, 1, "bfloat16", False),     # the reference's depthwise perf shapes (benchmark/test_conv2d_perf.py:50-52)
    (4, 64, 56, 56, 3, 3, 1, 1, 1, "bfloat16", False),
    (4, 128, 28, 28, 5, 5, 1, 2, 1, "float16", False),
    (4, 64, 56, 56, 3, 3, 1, 1, 1, "bfloat16", True),
    (3, 128, 28, 28, 5, 5, 1, 2, 1, "float16", True),
    (2, 40, 31, 29, 3, 3, 2, 1, 1, "bfloat16", True),        # stride 2, odd sizes, odd output width
    (2, 24, 20, 23, 3, 5, (1, 2), (2, 3), (2, 1), "float32", True),   # dilation, rectangular filter, fp32 vectors of 4
    (2, 16, 17, 19, 3, 3, 1, 1, (1, 2), "float32", False),   # dilation along W on planes
    (2, 12, 14, 14, 3, 3, 1, 1, 1, "bfloat16", True),        # 12 channels: not whole 16-byte vectors -> plane kernel
    (1, 8, 9, 11, 7, 7, 1, 3, 1, "float16", False),
    (2, 16, 32, 32, 3, 3, 2, 1, 1, "bfloat16", False),       # NCHW rows as 16-byte vectors, stride 2
    (2, 16, 24, 24, 5, 5, 2, 2, 1, "float16", False),        # output rows of 12: 8-byte vectors
    (2, 8, 16, 16, 3, 3, 1, 1, 1, "float32", False),         # fp32 rows, vectors of 4
    (2, 8, 10, 6, 3, 3, 1, 1, 1, "float32", False),          # rows of 24 bytes: fp32 vectors of 2
    (3, 24, 28, 28, 3, 3, 1, 1, 1, "bfloat16", False),       # rows of 56 bytes: 8-byte vectors
    (1, 4096, 9, 9, 3, 3, 1, 1, 1, "bfloat16", True),        # more channels than one block's shared memory holds
    (32, 64, 56, 56, 3, 3, 1, 1, 1, "bfloat16", True),       # more units than the resident blocks take in one round
    (2, 1024, 14, 14, 3, 3, 1, 1, 1, "float16", True),
    (2, 64, 14, 14, 3, 3, 1, 1, 1, "bfloat16", False),        # rows of 28 bytes: 4-byte vectors
    (2, 32, 14, 14, 5, 5, 2, 2, 1, "float16", False),
    (2, 32, 30, 30, 5, 5, 2, 2, 1, "bfloat16", True),
]


@pytest.mark.parametrize("case", DEPTHWISE, ids=[f"c{c[1]}_{c[4]}x{c[5]}_{c[9]}_{'cl' if c[10] else 'nchw'}" for c in DEPTHWISE])
def test_depthwise_kernels_match_oracle_and_direct_kernel(fd, case):
    """groups == C == K: the channels-last and the per-plane depthwise kernels against the oracle and against
    the one-thread-per-output direct kernel they replace, with scale, bias, a residual and ReLU."""
    n, c, h, w_, r, s_, stride, pad, dil, dtype_name, cl = case
    dtype = DTYPES[dtype_name]
    x = _to_dev(_rand((n, c, h, w_), 80), dtype, cl)
    w = _to_dev(_rand((c, 1, r, s_), 81, std=(r * s_) ** -0.5), dtype, False)
    b = _to_dev(_rand((c,), 82, std=0.1), dtype, False)
    sc = (torch.rand(c, generator=torch.Generator().manual_seed(83)) + 0.5).to(dtype).cuda()
    got = fd.conv2d(x, w, b, stride=stride, padding=pad, dilation=dil, groups=c)
    ref = oracle.conv2d_torch_cpu(x, w, b, stride, pad, dil, c)
    _check(got, ref, dtype_name)
    assert got.is_contiguous(memory_format=torch.channels_last) == cl or c == 1
    fd.set_algo("direct")
    try:
        plain = fd.conv2d(x, w, b, stride=stride, padding=pad, dilation=dil, groups=c)
    finally:
        fd.set_algo("auto")
    torch.testing.assert_close(got.float(), plain.float(), **TOL[dtype_name])
    shortcut = _to_dev(_rand(tuple(got.shape), 84), dtype, cl)
    fused = fd.conv2d_bias_act(x, w, b, stride=stride, padding=pad, dilation=dil, groups=c, scale=sc, relu=True,
                               residual=shortcut)
    ref = torch.relu(oracle.conv2d_torch_cpu(x, w, b, stride, pad, dil, c, scale=sc) + shortcut.float().cpu())
    _check(fused, ref, dtype_name)
    assert fd.device_status() == 0


GROUPED = [
    # n, c, h, w, k, r, groups, stride, pad, dtype, channels_last
    (4, 64, 56, 56, 128, 3, 2, 1, 1, "bfloat16", True),       # the reference's grouped perf shapes at a smaller batch
    (8, 128, 28, 28, 128, 3, 8, 1, 1, "bfloat16", True),      # (benchmark/test_conv2d_perf.py:48-49)
    (4, 64, 56, 56, 128, 3, 2, 1, 1, "float16", False),       # NCHW: every group's channels are relaid out
    (4, 64, 30, 30, 96, 3, 2, 2, 1, "float32", True),         # fp32 (split TF32), stride 2, 48 filters per group
    (4, 512, 14, 14, 512, 1, 4, 1, 0, "bfloat16", True),      # 1x1, 128 -> 128 per group
    (3, 96, 17, 19, 48, 5, 3, 1, 2, "bfloat16", True),        # three groups of 32 -> 16, ragged sizes
    (8, 256, 28, 28, 256, 3, 16, 1, 1, "bfloat16", True),     # sixteen groups: one launch per group
    (8, 256, 28, 28, 512, 3, 16, 1, 1, "float16", False),     # ... from NCHW tensors
    (16, 8, 64, 64, 32, 3, 2, 1, 1, "bfloat16", True),        # two groups of 4 -> 16 channels: dense 8 -> 32
]


@pytest.mark.parametrize("case", GROUPED, ids=[f"c{c[1]}k{c[4]}g{c[6]}_{c[9]}_{'cl' if c[10] else 'nchw'}" for c in GROUPED])
def test_grouped_layers_on_the_tensor_core_path_match_oracle(fd, case):
    """groups > 1, not depthwise: up to eight groups run as one dense convolution with a block-diagonal filter, more
    groups as one tensor-core launch per group on views of x, w and y; against the oracle, against the direct
    kernel, and with the full epilogue."""
    n, c, h, w_, k, r, groups, stride, pad, dtype_name, cl = case
    dtype = DTYPES[dtype_name]
    x = _to_dev(_rand((n, c, h, w_), 90), dtype, cl)
    w = _to_dev(_rand((k, c // groups, r, r), 91, std=(c // groups * r * r) ** -0.5), dtype, cl)
    b = _to_dev(_rand((k,), 92, std=0.1), dtype, False)
    sc = (torch.rand(k, generator=torch.Generator().manual_seed(93)) + 0.5).to(dtype).cuda()
    plan = fd.conv2d_plan(x, w, stride=stride, padding=pad, groups=groups)
    assert plan["algo"] != 1, "expected a tensor-core route"
    if groups > 8:
        assert plan["launches"] % groups == 0, "expected one launch per group"
    got = fd.conv2d(x, w, b, stride=stride, padding=pad, groups=groups)
    ref = oracle.conv2d_torch_cpu(x, w, b, stride, pad, 1, groups)
    _check(got, ref, dtype_name)
    fd.set_algo("direct")
    try:
        plain = fd.conv2d(x, w, b, stride=stride, padding=pad, groups=groups)
    finally:
        fd.set_algo("auto")
    torch.testing.assert_close(got.float(), plain.float(), **TOL[dtype_name])
    shortcut = _to_dev(_rand(tuple(got.shape), 94), dtype, cl)
    fused = fd.conv2d_bias_act(x, w, b, stride=stride, padding=pad, groups=groups, scale=sc, relu=True,
                               residual=shortcut)
    ref = torch.relu(oracle.conv2d_torch_cpu(x, w, b, stride, pad, 1, groups, scale=sc) + shortcut.float().cpu())
    _check(fused, ref, dtype_name)
    assert fd.device_status() == 0

"""Seeded random sweep over the operator surface: shapes, strides, paddings, dilations, groups, dtypes,
layouts, epilogues.  Every case is checked against the CPU oracle on the same bits; the planner decides
which kernel family runs (direct, single-CTA, CTA pairs, low-channel, pixel-grouped), so the sweep also
walks the boundaries between them."""
import random

import pytest
import torch

import oracle
from cases import TOL

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fd(native_lib):
    import flagdnn_b200

    assert torch.cuda.is_available()
    yield flagdnn_b200
    assert flagdnn_b200.device_status() == 0, "a kernel recorded a bounded-wait incident"


def _case(rng: random.Random):
    groups = rng.choice([1, 1, 1, 1, 2, 4])
    c = groups * rng.choice([1, 2, 3, 4, 8, 16, 24, 40, 64, 96])
    k = groups * rng.choice([1, 2, 4, 8, 16, 20, 32, 64, 72, 128])
    r, s = rng.choice([(1, 1), (3, 3), (3, 3), (1, 3), (5, 5), (7, 7), (2, 2), (3, 1)])
    stride = (rng.choice([1, 1, 2, 3]), rng.choice([1, 1, 2]))
    dil = (rng.choice([1, 1, 1, 2]), rng.choice([1, 1, 2]))
    pad = (rng.randint(0, r // 2 + 1), rng.randint(0, s // 2 + 1))
    h = rng.randint(max(1, dil[0] * (r - 1) + 1 - 2 * pad[0]), 40)
    w = rng.randint(max(1, dil[1] * (s - 1) + 1 - 2 * pad[1]), 40)
    n = rng.choice([1, 2, 3, 5, 8, 33])
    # a few large problems so that the tensor-core paths (and pixel grouping / CTA pairs) are reached
    if rng.random() < 0.3:
        n, h, w = rng.choice([16, 32, 48]), rng.choice([28, 32, 56]), rng.choice([28, 32, 56])
    return n, c, h, w, k, r, s, stride, pad, dil, groups


@pytest.mark.parametrize("seed", range(60))
def test_random_case_matches_oracle(fd, seed):
    rng = random.Random(1234 + seed)
    n, c, h, w, k, r, s, stride, pad, dil, groups = _case(rng)
    dtype_name = rng.choice(["bfloat16", "bfloat16", "float16", "float32", "float64"])
    if dtype_name == "float64" and n * k * h * w * c * r * s // groups > 2e9:
        dtype_name = "float32"
    channels_last = rng.random() < 0.6
    epilogue = rng.choice(["none", "bias", "bias_relu", "scale_bias_relu", "residual_relu", "gelu"])
    dtype = getattr(torch, dtype_name)
    g = torch.Generator().manual_seed(seed)

    def make(shape, std=1.0):
        t = (torch.randn(shape, generator=g) * std).to(dtype).cuda()
        return t.contiguous(memory_format=torch.channels_last) if channels_last and t.dim() == 4 else t

    x = make((n, c, h, w))
    wt = make((k, c // groups, r, s), std=(c // groups * r * s) ** -0.5)
    bias = None if epilogue == "none" else make((k,), std=0.2)
    scale = (torch.rand(k, generator=g) + 0.5).to(dtype).cuda() if epilogue == "scale_bias_relu" else None
    oh = (h + 2 * pad[0] - dil[0] * (r - 1) - 1) // stride[0] + 1
    ow = (w + 2 * pad[1] - dil[1] * (s - 1) - 1) // stride[1] + 1
    assert oh >= 1 and ow >= 1
    residual = make((n, k, oh, ow)) if epilogue == "residual_relu" else None
    activation = {"none": "none", "bias": "none", "bias_relu": "relu", "scale_bias_relu": "relu",
                  "residual_relu": "relu", "gelu": "gelu"}[epilogue]

    got = fd.conv2d_bias_act(x, wt, bias, stride=stride, padding=pad, dilation=dil, groups=groups, scale=scale,
                             residual=residual, activation=activation)
    cdt = torch.float64 if dtype_name == "float64" else torch.float32
    ref = oracle.conv2d_torch_cpu(x, wt, bias, stride, pad, dil, groups, scale=scale, compute_dtype=cdt)
    if residual is not None:
        ref = ref + residual.cpu().to(cdt)
    if activation == "relu":
        ref = torch.relu(ref)
    elif activation == "gelu":
        ref = torch.nn.functional.gelu(ref)
    assert got.shape == ref.shape and got.dtype == dtype
    tol = TOL[dtype_name]
    what = f"n{n} c{c} h{h} w{w} k{k} r{r}x{s} stride{stride} pad{pad} dil{dil} g{groups} {dtype_name} cl={channels_last} {epilogue}"
    torch.testing.assert_close(got.cpu().to(cdt), ref, rtol=tol["rtol"], atol=tol["atol"], msg=lambda m: f"{what}: {m}")


def _grouped_case(rng: random.Random):
    """Depthwise layers (own kernels per layout and alignment), depthwise with a channel multiplier (direct
    kernel), and layers with many groups (one tensor-core launch per group when the groups are wide enough)."""
    kind = rng.choice(["depthwise", "depthwise", "depthwise", "multiplier", "many_groups"])
    if kind == "many_groups":
        groups = rng.choice([16, 32])
        c = groups * rng.choice([8, 16])
        k = groups * rng.choice([8, 16, 24])
    else:
        c = rng.choice([2, 6, 8, 12, 16, 32, 64, 96, 144, 256])
        groups = c
        k = c * (2 if kind == "multiplier" else 1)
    r, s = rng.choice([(3, 3), (3, 3), (3, 3), (5, 5), (5, 5), (7, 7), (3, 5), (2, 2), (1, 3)])
    st = rng.choice([1, 1, 2, 3])
    stride = (st, st) if rng.random() < 0.8 else (st, rng.choice([1, 2]))
    dil = (1, 1) if rng.random() < 0.8 else (rng.choice([1, 2]), rng.choice([1, 2]))
    pad = (r // 2, s // 2) if rng.random() < 0.7 else (rng.randint(0, r // 2 + 1), rng.randint(0, s // 2 + 1))
    h = rng.choice([7, 8, 14, 15, 16, 28, 30, 56])
    w = rng.choice([7, 8, 14, 16, 20, 28, 31, 56])
    h = max(h, dil[0] * (r - 1) + 1 - 2 * pad[0])
    w = max(w, dil[1] * (s - 1) + 1 - 2 * pad[1])
    n = rng.choice([1, 2, 3, 8, 16])
    if kind == "many_groups":
        n, h, w = rng.choice([8, 16]), rng.choice([28, 32]), rng.choice([28, 32])
    return n, c, h, w, k, r, s, stride, pad, dil, groups


@pytest.mark.parametrize("seed", range(48))
def test_random_depthwise_and_grouped_case_matches_oracle(fd, seed):
    rng = random.Random(9000 + seed)
    n, c, h, w, k, r, s, stride, pad, dil, groups = _grouped_case(rng)
    dtype_name = rng.choice(["bfloat16", "bfloat16", "float16", "float32"])
    channels_last = rng.random() < 0.5
    epilogue = rng.choice(["none", "bias", "bias_relu", "scale_bias_relu", "residual_relu", "gelu"])
    dtype = getattr(torch, dtype_name)
    g = torch.Generator().manual_seed(seed)

    def make(shape, std=1.0):
        t = (torch.randn(shape, generator=g) * std).to(dtype).cuda()
        return t.contiguous(memory_format=torch.channels_last) if channels_last and t.dim() == 4 else t

    x = make((n, c, h, w))
    wt = make((k, c // groups, r, s), std=(c // groups * r * s) ** -0.5)
    bias = None if epilogue == "none" else make((k,), std=0.2)
    scale = (torch.rand(k, generator=g) + 0.5).to(dtype).cuda() if epilogue == "scale_bias_relu" else None
    oh = (h + 2 * pad[0] - dil[0] * (r - 1) - 1) // stride[0] + 1
    ow = (w + 2 * pad[1] - dil[1] * (s - 1) - 1) // stride[1] + 1
    assert oh >= 1 and ow >= 1
    residual = make((n, k, oh, ow)) if epilogue == "residual_relu" else None
    activation = {"none": "none", "bias": "none", "bias_relu": "relu", "scale_bias_relu": "relu",
                  "residual_relu": "relu", "gelu": "gelu"}[epilogue]
    got = fd.conv2d_bias_act(x, wt, bias, stride=stride, padding=pad, dilation=dil, groups=groups, scale=scale,
                             residual=residual, activation=activation)
    ref = oracle.conv2d_torch_cpu(x, wt, bias, stride, pad, dil, groups, scale=scale)
    if residual is not None:
        ref = ref + residual.float().cpu()
    if activation == "relu":
        ref = torch.relu(ref)
    elif activation == "gelu":
        ref = torch.nn.functional.gelu(ref)
    assert got.shape == ref.shape and got.dtype == dtype
    torch.testing.assert_close(got.float().cpu(), ref, **TOL[dtype_name])

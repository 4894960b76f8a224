"""Reduction splitting across CTA pairs: layers whose tiles do not fill whole rounds of the GPU's pairs are
computed with the (tile, reduction step) space shared evenly and fp32 partial sums exchanged through scratch.
Checked against the oracle, against the unsplit schedule of the same kernel, for determinism, with several
contributors per tile, with two column tiles, with a folded scale and a residual, and call after call on the
same scratch buffer."""
import pytest
import torch

import oracle
from flagdnn_b200 import _native as nat

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _rand(shape, seed, std=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * std


def _nhwc(t):
    return t.contiguous(memory_format=torch.channels_last)


# n, c, hw, k, r, stride, pad, what the case exercises
CASES = [
    (40, 256, 14, 256, 3, 1, 1, "31 tiles on 74 pairs: every tile split once or twice"),
    (128, 512, 7, 512, 3, 1, 1, "50 tiles of 72 steps, two column tiles: up to three pieces per tile"),
    (100, 256, 14, 256, 3, 1, 1, "77 tiles: one round and a sliver"),
    (120, 1024, 14, 256, 1, 1, 0, "1x1 with a long reduction: 92 tiles of 16 steps"),
    (81, 256, 15, 320, 3, 2, 1, "stride 2: ragged last tile, ragged second column tile"),
]


@pytest.mark.parametrize("case", CASES, ids=[c[-1].split(":")[0].replace(" ", "_") for c in CASES])
def test_split_reduction_matches_oracle_and_unsplit_schedule(native_lib, case):
    import flagdnn_b200 as fd

    n, c, hw, k, r, stride, pad, _ = case
    x = _nhwc(_rand((n, c, hw, hw), 1).to(BF).cuda())
    w = _nhwc(_rand((k, c, r, r), 2, std=(c * r * r) ** -0.5).to(BF).cuda())
    b = _rand((k,), 3, std=0.1).to(BF).cuda()
    s = (torch.rand(k, generator=torch.Generator().manual_seed(4)) + 0.5).to(BF).cuda()
    fd.set_algo("pair")
    fd.set_stream_k(True)
    try:
        plan = fd.conv2d_plan(x, w, stride=stride, padding=pad)
        assert plan["algo"] == nat.ALGO_IGEMM_PAIR and plan["stream_k"] == 1, "the case must plan a split"
        assert plan["streamk_bytes"] == nat.STREAMK_FLAG_BYTES + plan["grid"] * 128 * 256 * 4
        split = fd.fused_conv2d_bias_relu(x, w, b, stride=stride, padding=pad, scale=s)
        again = fd.fused_conv2d_bias_relu(x, w, b, stride=stride, padding=pad, scale=s)   # same scratch, flags back at zero
        fd.set_stream_k(False)
        assert fd.conv2d_plan(x, w, stride=stride, padding=pad)["stream_k"] == 0
        whole = fd.fused_conv2d_bias_relu(x, w, b, stride=stride, padding=pad, scale=s)
    finally:
        fd.set_stream_k(False)
        fd.set_algo("auto")
    torch.cuda.synchronize()
    assert fd.device_status() == 0
    assert torch.equal(split, again), "the split schedule is a function of the problem, not of timing"
    # the unsplit schedule adds the same products in one chain: fp32 sums may differ in the last bit, outputs by
    # at most one bf16 step, and only a few of them
    a, bb = split.float(), whole.float()
    assert (a - bb).abs().max() <= 2.0 ** -7 * bb.abs().max()
    assert (split != whole).float().mean() < 2e-3
    # every image against the reference's CPU call in bf16, sampled images against the fp32 oracle
    out_cpu = split.cpu()
    for i0 in range(0, n, 32):
        ref16 = oracle.conv2d_torch_cpu(x[i0:i0 + 32], w, b, stride, pad, 1, 1, scale=s, relu=True, compute_dtype=BF)
        torch.testing.assert_close(out_cpu[i0:i0 + 32].float(), ref16.float(), rtol=1.6e-2, atol=1e-2)
    picks = [0, n // 2, n - 1]
    ref = oracle.conv2d_torch_cpu(x[picks], w, b, stride, pad, 1, 1, scale=s, relu=True)
    torch.testing.assert_close(out_cpu[picks].float(), ref, rtol=1e-2, atol=1e-2)


def test_split_reduction_with_residual_and_in_a_cuda_graph(native_lib):
    import flagdnn_b200 as fd

    n, c, hw, k = 40, 256, 14, 256
    x = _nhwc(_rand((n, c, hw, hw), 5).to(BF).cuda())
    w = _nhwc(_rand((k, c, 3, 3), 6, std=(c * 9) ** -0.5).to(BF).cuda())
    b = _rand((k,), 7, std=0.1).to(BF).cuda()
    shortcut = _nhwc(_rand((n, k, hw, hw), 8).to(BF).cuda())
    assert fd.conv2d_plan(x, w, padding=1)["stream_k"] == 0, "off unless asked for"
    fd.set_stream_k(True)
    try:
        _residual_and_graph(fd, x, w, b, shortcut)
    finally:
        fd.set_stream_k(False)


def _residual_and_graph(fd, x, w, b, shortcut):
    plan = fd.conv2d_plan(x, w, padding=1)
    assert plan["stream_k"] == 1 and plan["algo"] == nat.ALGO_IGEMM_PAIR, "with the option on, planned automatically"
    eager = fd.conv2d_bias_act(x, w, b, padding=1, relu=True, residual=shortcut)
    ref = torch.relu(oracle.conv2d_torch_cpu(x[:3], w, b, 1, 1, 1, 1) + shortcut[:3].float().cpu())
    torch.testing.assert_close(eager[:3].float().cpu(), ref, rtol=1e-2, atol=1e-2)
    # replayed from a CUDA graph on a side stream: the scratch of that stream is created before the capture
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        fd.conv2d_bias_act(x, w, b, padding=1, relu=True, residual=shortcut)
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            outs = [fd.conv2d_bias_act(x, w, b, padding=1, relu=True, residual=shortcut) for _ in range(3)]
        for _ in range(3):
            g.replay()
        stream.synchronize()
    for o in outs:
        assert torch.equal(o, eager)
    assert fd.device_status() == 0


def test_c_abi_runs_whole_tiles_without_the_scratch_and_splits_with_it(native_lib):
    """fdnn_conv2d_fwd never splits; fdnn_conv2d_fwd_ex does when handed zeroed scratch of plan.streamk_bytes."""
    import ctypes

    lib = native_lib
    n, c, hw, k = 40, 256, 14, 256
    x = _nhwc(_rand((n, c, hw, hw), 9).to(BF).cuda())
    w = _nhwc(_rand((k, c, 3, 3), 10, std=(c * 9) ** -0.5).to(BF).cuda())
    b = _rand((k,), 11, std=0.1).to(BF).cuda()
    y0 = torch.empty((n, k, hw, hw), dtype=BF, device="cuda", memory_format=torch.channels_last)
    y1, y2 = torch.empty_like(y0), torch.empty_like(y0)
    d = nat.ConvDesc()
    d.dtype = nat.BF16
    d.n, d.c, d.h, d.w, d.k, d.r, d.s = n, c, hw, hw, k, 3, 3
    d.stride_h = d.stride_w = d.dil_h = d.dil_w = d.groups = 1
    d.pad_top = d.pad_bottom = d.pad_left = d.pad_right = 1
    d.algo = nat.ALGO_AUTO
    for i in range(4):
        d.x_strides[i], d.w_strides[i], d.y_strides[i] = x.stride(i), w.stride(i), y0.stride(i)
    plan = nat.ConvPlan()
    nat.check(lib.fdnn_conv2d_query(ctypes.byref(d), x.data_ptr(), w.data_ptr(), y0.data_ptr(), ctypes.byref(plan)))
    assert plan.stream_k == 0 and plan.streamk_bytes == 0, "the plain descriptor never splits"
    d.algo = nat.ALGO_AUTO | nat.ALGO_FLAG_STREAM_K
    nat.check(lib.fdnn_conv2d_query(ctypes.byref(d), x.data_ptr(), w.data_ptr(), y0.data_ptr(), ctypes.byref(plan)))
    assert plan.stream_k == 1 and plan.workspace_bytes == 0 and plan.w_packed == 0
    nat.check(lib.fdnn_conv2d_fwd(ctypes.byref(d), x.data_ptr(), w.data_ptr(), None, b.data_ptr(), None, nat.ACT_RELU,
                                  y0.data_ptr(), None, 0, None))
    scratch = torch.empty(plan.streamk_bytes, dtype=torch.uint8, device="cuda")
    scratch[: nat.STREAMK_FLAG_BYTES].zero_()
    for y in (y1, y2):
        nat.check(lib.fdnn_conv2d_fwd_ex(ctypes.byref(d), x.data_ptr(), w.data_ptr(), None, b.data_ptr(), None, None,
                                         nat.ACT_RELU, y.data_ptr(), None, 0, scratch.data_ptr(), scratch.numel(), None))
    torch.cuda.synchronize()
    assert (scratch[: nat.STREAMK_FLAG_BYTES] == 0).all(), "every launch lowers the flags it raised"
    assert torch.equal(y1, y2)
    assert (scratch[nat.STREAMK_FLAG_BYTES:].view(torch.float32).abs().sum() > 0), "partial sums went through the scratch"
    ref = oracle.conv2d_torch_cpu(x[:4], w, b, 1, 1, 1, 1, relu=True)
    for y in (y0, y1):
        torch.testing.assert_close(y[:4].float().cpu(), ref, rtol=1e-2, atol=1e-2)
    too_small = lib.fdnn_conv2d_fwd_ex(ctypes.byref(d), x.data_ptr(), w.data_ptr(), None, b.data_ptr(), None, None,
                                       nat.ACT_RELU, y2.data_ptr(), None, 0, scratch.data_ptr() + 8, 1024, None)
    assert too_small == nat.FDNN_BAD_PARAM      # misaligned scratch is refused, not ignored

"""Hazards at the C boundary, each pinned by a GPU test that calls through the C ABI:

* a packed filter handed to a forward call whose plan reads another layout is refused, not misread;
* an activation tensor smaller than 128 KiB read in place by an im2col-mode tensor map (the case the
  library adjusts the encoded map for) gives the oracle's answer, like the relaid-out route;
* a bounded device-side wait that runs out makes the kernel return, is reported once by
  fdnn_device_status, and leaves the device usable.
"""
import ctypes

import pytest
import torch

import oracle
from flagdnn_b200 import _native as nat

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _desc(x, w, y, stride, pad, algo=nat.ALGO_AUTO):
    d = nat.ConvDesc()
    d.dtype = {torch.float32: nat.F32, torch.bfloat16: nat.BF16, torch.float16: nat.F16}[x.dtype]
    d.n, d.c, d.h, d.w = x.shape
    d.k, _, d.r, d.s = w.shape
    d.stride_h = d.stride_w = stride
    d.pad_top = d.pad_bottom = d.pad_left = d.pad_right = pad
    d.dil_h = d.dil_w = 1
    d.groups = 1
    d.algo = algo
    for i in range(4):
        d.x_strides[i], d.w_strides[i], d.y_strides[i] = x.stride(i), w.stride(i), y.stride(i)
    return d


def _rand(shape, seed, std=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * std


def _nhwc(t):
    return t.contiguous(memory_format=torch.channels_last)


def _unaligned_nhwc_output(n, k, oh, ow, dtype):
    """A dense channels-last [n, k, oh, ow] view that starts 2 bytes into its storage (8-byte misaligned for TMA)."""
    store = torch.zeros(n * k * oh * ow + 8, dtype=dtype, device="cuda")
    y = store[1:1 + n * oh * ow * k].view(n, oh, ow, k).permute(0, 3, 1, 2)
    assert y.data_ptr() % 16 != 0
    return store, y


# (name, x shape, w shape, stride, pad, attribute of the aligned plan that an unaligned y switches off)
GUARD_CASES = [
    ("stem_low_channel", (4, 3, 64, 64), (32, 3, 7, 7), 2, 3, "low_channel"),
    ("narrow_3x3_pixel_group", (18, 64, 56, 56), (64, 64, 3, 3), 1, 1, "pixel_group"),
]


@pytest.mark.parametrize("case", GUARD_CASES, ids=[c[0] for c in GUARD_CASES])
def test_packed_filter_of_another_layout_is_refused(native_lib, case):
    lib = native_lib
    _, xs, ws, stride, pad, attr = case
    x = _nhwc(_rand(xs, 1).to(BF).cuda())
    w = _nhwc(_rand(ws, 2, std=(ws[1] * ws[2] * ws[3]) ** -0.5).to(BF).cuda())
    b = _rand((ws[0],), 3, std=0.1).to(BF).cuda()
    oh = (xs[2] + 2 * pad - ws[2]) // stride + 1
    y_al = torch.empty((xs[0], ws[0], oh, oh), dtype=BF, device="cuda", memory_format=torch.channels_last)
    store, y_un = _unaligned_nhwc_output(xs[0], ws[0], oh, oh, BF)
    d = _desc(x, w, y_al, stride, pad)
    plan_al, plan_un = nat.ConvPlan(), nat.ConvPlan()
    nat.check(lib.fdnn_conv2d_query(ctypes.byref(d), x.data_ptr(), 1, y_al.data_ptr(), ctypes.byref(plan_al)))
    nat.check(lib.fdnn_conv2d_query(ctypes.byref(d), x.data_ptr(), 1, y_un.data_ptr(), ctypes.byref(plan_un)))
    assert getattr(plan_al, attr) >= 1 and getattr(plan_un, attr) <= (1 if attr == "pixel_group" else 0), \
        "the case must plan differently for the aligned and the unaligned output"

    def run(packed, plan, y):
        ws_buf = torch.empty(max(int(plan.workspace_bytes), 256), dtype=torch.uint8, device="cuda")
        return lib.fdnn_conv2d_fwd(ctypes.byref(d), x.data_ptr(), w.data_ptr(), packed.data_ptr(), b.data_ptr(), None,
                                   nat.ACT_RELU, y.data_ptr(), ws_buf.data_ptr(), ws_buf.numel(), None)

    size = max(int(plan_al.packed_weight_bytes), int(plan_un.packed_weight_bytes))
    packed_al = torch.empty(size, dtype=torch.uint8, device="cuda")
    packed_un = torch.empty(size, dtype=torch.uint8, device="cuda")
    nat.check(lib.fdnn_conv2d_pack_weight(ctypes.byref(d), w.data_ptr(), y_al.data_ptr(), packed_al.data_ptr(), size, None))
    nat.check(lib.fdnn_conv2d_pack_weight(ctypes.byref(d), w.data_ptr(), y_un.data_ptr(), packed_un.data_ptr(), size, None))
    # the mismatched pairings are refused before anything is launched ...
    y_un.fill_(-7.0)
    assert run(packed_al, plan_un, y_un) == nat.FDNN_BAD_PARAM
    assert b"packed filter" in lib.fdnn_last_error() and b"pack again" in lib.fdnn_last_error()
    assert run(packed_un, plan_al, y_al) == nat.FDNN_BAD_PARAM
    torch.cuda.synchronize()
    assert (y_un == -7.0).all(), "a refused call must not write"
    # ... and the matching ones give the oracle's answer, also into the unaligned output
    nat.check(run(packed_al, plan_al, y_al))
    nat.check(run(packed_un, plan_un, y_un))
    torch.cuda.synchronize()
    ref = oracle.conv2d_torch_cpu(x, w, b, stride, pad, 1, 1, relu=True)
    torch.testing.assert_close(y_al.float().cpu(), ref, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(y_un.float().cpu(), ref, rtol=1e-2, atol=1e-2)
    assert store[0] == 0 and store[-1] == 0, "bytes around the unaligned output were touched"


def test_python_api_handles_an_output_view_offset_by_two_bytes(native_lib):
    """The host wrapper packs for the output it is given: a stem and a narrow 3x3 layer into `out` views that
    start 2 bytes into their storage take the generic path and still match the oracle."""
    import flagdnn_b200 as fd

    for _, xs, ws, stride, pad, _attr in GUARD_CASES:
        x = _nhwc(_rand(xs, 4).to(BF).cuda())
        w = _nhwc(_rand(ws, 5, std=(ws[1] * ws[2] * ws[3]) ** -0.5).to(BF).cuda())
        b = _rand((ws[0],), 6, std=0.1).to(BF).cuda()
        oh = (xs[2] + 2 * pad - ws[2]) // stride + 1
        _, y_un = _unaligned_nhwc_output(xs[0], ws[0], oh, oh, BF)
        got_un = fd.fused_conv2d_bias_relu(x, w, b, stride=stride, padding=pad, out=y_un)
        got_al = fd.fused_conv2d_bias_relu(x, w, b, stride=stride, padding=pad)
        ref = oracle.conv2d_torch_cpu(x, w, b, stride, pad, 1, 1, relu=True)
        torch.testing.assert_close(got_un.float().cpu(), ref, rtol=1e-2, atol=1e-2)
        torch.testing.assert_close(got_al.float().cpu(), ref, rtol=1e-2, atol=1e-2)


# activations under 128 KiB: [n, c, h, w] bf16 channels-last, read in place by the im2col-mode map
SMALL_IM2COL = [
    ((1, 64, 14, 14), (64, 64, 3, 3), 1, 1),      # 25 KB
    ((2, 128, 14, 14), (128, 128, 3, 3), 1, 1),   # 100 KB
    ((1, 256, 7, 7), (512, 256, 3, 3), 1, 1),     # 25 KB, wide filter
    ((4, 64, 15, 15), (96, 64, 3, 3), 2, 1),      # 115 KB, stride 2, ragged tile
    ((1, 512, 8, 8), (256, 512, 1, 1), 1, 0),     # 64 KB, 1x1
    ((2, 256, 16, 16), (64, 256, 3, 3), 1, 1),    # 256 KB: just above the threshold, for contrast
]


@pytest.mark.parametrize("case", SMALL_IM2COL, ids=[f"{c[0][0]}x{c[0][1]}x{c[0][2]}_k{c[1][0]}_r{c[1][2]}_s{c[2]}" for c in SMALL_IM2COL])
def test_small_activation_in_place_equals_relaid_out_route_and_oracle(native_lib, case):
    import flagdnn_b200 as fd

    xs, ws, stride, pad = case
    x = _nhwc(_rand(xs, 7).to(BF).cuda())
    w = _nhwc(_rand(ws, 8, std=(ws[1] * ws[2] * ws[3]) ** -0.5).to(BF).cuda())
    b = _rand((ws[0],), 9, std=0.1).to(BF).cuda()
    fd.set_algo("igemm")
    try:
        plan = fd.conv2d_plan(x, w, stride=stride, padding=pad)
        assert plan["algo"] == nat.ALGO_IGEMM and plan["x_repacked"] == 0, "x must be consumed in place"
        in_place = fd.fused_conv2d_bias_relu(x, w, b, stride=stride, padding=pad)
        # the same values as an NCHW tensor are first rewritten into the workspace (a fresh dense NHWC copy)
        x_nchw = x.contiguous()
        plan2 = fd.conv2d_plan(x_nchw, w, stride=stride, padding=pad)
        assert plan2["x_repacked"] == 1
        relaid = fd.fused_conv2d_bias_relu(x_nchw, w, b, stride=stride, padding=pad)
    finally:
        fd.set_algo("auto")
    ref = oracle.conv2d_torch_cpu(x, w, b, stride, pad, 1, 1, relu=True)
    torch.testing.assert_close(in_place.float().cpu(), ref, rtol=1e-2, atol=1e-2)
    assert torch.equal(in_place.contiguous(), relaid.contiguous()), "both routes feed the same kernel the same values"


@pytest.mark.parametrize("algo", ["igemm", "pair"])
def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable(native_lib, algo):
    """No copy is issued, so the MMA issuer's first wait for data runs out after ~0.1 ms of clocks: the kernel
    records its incident, every role leaves its loop, tensor memory is freed and the launch returns."""
    import flagdnn_b200 as fd

    lib = native_lib
    x = _nhwc(_rand((2, 64, 16, 16), 10).to(BF).cuda())
    w = _nhwc(_rand((256, 64, 3, 3), 11, std=1 / 24).to(BF).cuda())
    b = _rand((256,), 12, std=0.1).to(BF).cuda()
    fd.set_algo(algo)
    try:
        good = fd.fused_conv2d_bias_relu(x, w, b, padding=1)
        torch.cuda.synchronize()
        assert fd.device_status() == 0
        nat.check(lib.fdnn_debug_set_wait_limit(200_000, 1))
        try:
            fd.fused_conv2d_bias_relu(x, w, b, padding=1)
            torch.cuda.synchronize()            # returns: the kernel gave up instead of spinning
        finally:
            nat.check(lib.fdnn_debug_set_wait_limit(0, 0))
        word = ctypes.c_uint32(0)
        assert lib.fdnn_device_status(ctypes.byref(word)) == nat.FDNN_DEVICE_TIMEOUT
        assert word.value in (2, 4), "issuer's wait for data (2) or, in the partner CTA, the epilogue's wait (4)"
        assert b"incident" in lib.fdnn_last_error()
        assert lib.fdnn_device_status(ctypes.byref(word)) == nat.FDNN_OK and word.value == 0, "the word clears"
        again = fd.fused_conv2d_bias_relu(x, w, b, padding=1)
        torch.cuda.synchronize()
        assert torch.equal(again, good)
        ref = oracle.conv2d_torch_cpu(x, w, b, 1, 1, 1, 1, relu=True)
        torch.testing.assert_close(again.float().cpu(), ref, rtol=1e-2, atol=1e-2)
        assert fd.device_status() == 0
    finally:
        fd.set_algo("auto")


def _map_counters(lib):
    reused, encoded = ctypes.c_int64(0), ctypes.c_int64(0)
    assert lib.fdnn_debug_tensor_map_counters(ctypes.byref(reused), ctypes.byref(encoded)) == nat.FDNN_OK
    return reused.value, encoded.value


@pytest.mark.parametrize("shape", [((8, 64, 28, 28), (128, 64, 3, 3), 1, 1), ((4, 3, 64, 64), (32, 3, 7, 7), 2, 3),
                                   ((16, 256, 14, 14), (256, 256, 3, 3), 1, 1)],
                         ids=["generic", "stem", "pairs"])
def test_a_repeated_layer_encodes_no_tensor_map(native_lib, shape):
    """The steady state of an eager loop: the same layer on the same buffers takes every tensor map from the
    library's table (no driver call), a new output buffer encodes only the maps that name it, and the results
    stay those of the first call."""
    import flagdnn_b200 as fd

    xs, ws, stride, pad = shape
    x = _nhwc(_rand(xs, 21).to(BF).cuda())
    w = _nhwc(_rand(ws, 22, std=(ws[1] * ws[2] * ws[3]) ** -0.5).to(BF).cuda())
    b = _rand((ws[0],), 23, std=0.1).to(BF).cuda()
    out = fd.fused_conv2d_bias_relu(x, w, b, stride=stride, padding=pad)
    first = out.clone()
    buf = torch.empty_like(out)
    fd.conv2d_bias_act(x, w, b, stride=stride, padding=pad, relu=True, out=buf)      # maps over `buf` are new
    r0, e0 = _map_counters(native_lib)
    for _ in range(3):
        fd.conv2d_bias_act(x, w, b, stride=stride, padding=pad, relu=True, out=buf)
    r1, e1 = _map_counters(native_lib)
    assert e1 == e0, "a repeated call went back to the driver for a tensor map"
    assert r1 > r0
    assert torch.equal(buf, first)
    other = torch.empty_like(out)
    fd.conv2d_bias_act(x, w, b, stride=stride, padding=pad, relu=True, out=other)
    r2, e2 = _map_counters(native_lib)
    assert 0 < e2 - e1 <= 3, "only the maps over the new output are encoded"
    assert torch.equal(other, first)
    ref = oracle.conv2d_torch_cpu(x, w, b, stride, pad, 1, 1, relu=True)
    torch.testing.assert_close(first.float().cpu(), ref, rtol=1e-2, atol=1e-2)

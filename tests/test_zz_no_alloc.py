"""fdnn_conv2d_fwd_static_scratch: the forward entry point for hosts that are
not allowed to allocate device memory while they run (a serving process whose
arena was sized at start-up, a plug-in inside another framework's pool, a job
under a fixed memory quota).  Its scratch is an array inside the library, so
the call itself must not change the amount of free device memory, and its
result must equal the regular entry point's, call after call.

Collected last on purpose: if it fails, a run that stops at the first failure
has already run every other test.
"""
import ctypes

import pytest
import torch

import oracle
from flagdnn_b200 import _native as nat

pytestmark = pytest.mark.gpu


def _desc(x, w, y, stride, pad, algo=nat.ALGO_IGEMM):
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


def _problem(dtype, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(3, 20, 17, 19, generator=g).to(dtype).cuda()            # NCHW: x must be relaid out
    w = (torch.randn(40, 20, 3, 3, generator=g) / 13).to(dtype).cuda()
    b = (torch.randn(40, generator=g) * 0.1).to(dtype).cuda()
    s = (torch.rand(40, generator=g) + 0.5).to(dtype).cuda()
    return x, w, b, s


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_matches_regular_entry_point_twice(native_lib, dtype):
    lib = native_lib
    x, w, b, s = _problem(dtype, 5)
    y_ref = torch.empty(3, 40, 17, 19, dtype=dtype, device="cuda")
    d = _desc(x, w, y_ref, 1, 1)
    plan = nat.ConvPlan()
    nat.check(lib.fdnn_conv2d_query(ctypes.byref(d), x.data_ptr(), 1, y_ref.data_ptr(), ctypes.byref(plan)))
    assert plan.algo == nat.ALGO_IGEMM and plan.workspace_bytes > 0, "the case must need scratch"
    assert plan.workspace_bytes <= lib.fdnn_static_scratch_bytes()
    # buffers the caller owns either way: packed filter, and a workspace for the regular call
    packed = torch.empty(plan.packed_weight_bytes, dtype=torch.uint8, device="cuda")
    nat.check(lib.fdnn_conv2d_pack_weight(ctypes.byref(d), w.data_ptr(), y_ref.data_ptr(), packed.data_ptr(), packed.numel(), None))
    ws = torch.empty(plan.workspace_bytes, dtype=torch.uint8, device="cuda")
    nat.check(lib.fdnn_conv2d_fwd(ctypes.byref(d), x.data_ptr(), w.data_ptr(), packed.data_ptr(), b.data_ptr(),
                                  s.data_ptr(), nat.ACT_RELU, y_ref.data_ptr(), ws.data_ptr(), ws.numel(), None))
    torch.cuda.synchronize()

    outs = [torch.full_like(y_ref, float("nan")) for _ in range(2)]
    # first call on the device performs the one-time address lookup
    nat.check(lib.fdnn_conv2d_fwd_static_scratch(ctypes.byref(d), x.data_ptr(), w.data_ptr(), packed.data_ptr(),
                                                 b.data_ptr(), s.data_ptr(), nat.ACT_RELU, outs[0].data_ptr(), None))
    torch.cuda.synchronize()
    # second call in a row, on a different input so stale scratch contents would show
    x2 = (x * 0.5 + 1).contiguous()
    y_ref2 = torch.empty_like(y_ref)
    nat.check(lib.fdnn_conv2d_fwd(ctypes.byref(d), x2.data_ptr(), w.data_ptr(), packed.data_ptr(), b.data_ptr(),
                                  s.data_ptr(), nat.ACT_RELU, y_ref2.data_ptr(), ws.data_ptr(), ws.numel(), None))
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    nat.check(lib.fdnn_conv2d_fwd_static_scratch(ctypes.byref(d), x2.data_ptr(), w.data_ptr(), packed.data_ptr(),
                                                 b.data_ptr(), s.data_ptr(), nat.ACT_RELU, outs[1].data_ptr(), None))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the call changed the amount of free device memory"

    # same kernels on the same values, only the scratch differs: bit for bit the regular entry point's result
    assert torch.equal(outs[0], y_ref) and torch.equal(outs[1], y_ref2)
    # and the oracle's, within the tolerances of the other parity tests
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    for got, x_in in ((outs[0], x), (outs[1], x2)):
        ref = oracle.conv2d_torch_cpu(x_in, w, b, 1, 1, 1, 1, scale=s, relu=True)
        torch.testing.assert_close(got.float().cpu(), ref, **tol)


def test_static_scratch_refuses_oversized_problems(native_lib):
    lib = native_lib
    # 64 x 64 x 128 x 128 fp32: the split copy of x needs 2 x 268 MB, far beyond the built-in array
    x = torch.empty(64, 64, 128, 128, dtype=torch.float32, device="meta")
    w = torch.empty(64, 64, 3, 3, dtype=torch.float32, device="meta")
    y = torch.empty(64, 64, 128, 128, dtype=torch.float32, device="meta")
    d = _desc(x, w, y, 1, 1)
    status = lib.fdnn_conv2d_fwd_static_scratch(ctypes.byref(d), 0x1000, 0x2000, 0x3000, None, None, nat.ACT_NONE,
                                                0x4000, None)
    assert status == nat.FDNN_WORKSPACE_TOO_SMALL
    text = lib.fdnn_static_scratch_last_error().decode()
    assert "scratch" in text and str(lib.fdnn_static_scratch_bytes()) in text

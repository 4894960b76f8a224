"""The C-ABI library builds, loads, exports every function the header declares
and validates descriptors — all without a GPU (no compute is launched)."""
import ctypes
import os
import re

import pytest

from conftest import ROOT
from flagdnn_b200 import _native as nat


def _header_functions():
    text = open(os.path.join(ROOT, "include", "flagdnn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fdnn_[a-z0-9_]+)\s*\(", text)))


def _desc(dtype=nat.BF16, n=2, c=64, h=14, w=14, k=64, r=3, s=3, stride=1, pad=1, dil=1, groups=1,
          algo=nat.ALGO_AUTO, channels_last=True):
    d = nat.ConvDesc()
    d.dtype = dtype
    d.n, d.c, d.h, d.w, d.k, d.r, d.s = n, c, h, w, k, r, s
    d.stride_h = d.stride_w = stride
    d.pad_top = d.pad_bottom = d.pad_left = d.pad_right = pad
    d.dil_h = d.dil_w = dil
    d.groups = groups
    d.algo = algo
    oh = (h + 2 * pad - dil * (r - 1) - 1) // stride + 1
    ow = (w + 2 * pad - dil * (s - 1) - 1) // stride + 1
    cg = c // groups
    if channels_last:
        xs, ws, ys = (h * w * c, 1, w * c, c), (r * s * cg, 1, s * cg, cg), (oh * ow * k, 1, ow * k, k)
    else:
        xs, ws, ys = (c * h * w, h * w, w, 1), (cg * r * s, r * s, s, 1), (k * oh * ow, oh * ow, ow, 1)
    for i in range(4):
        d.x_strides[i], d.w_strides[i], d.y_strides[i] = xs[i], ws[i], ys[i]
    return d


def test_library_exports_every_declared_symbol(native_lib):
    declared = _header_functions()
    assert declared == sorted(nat.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(native_lib, name), f"{name} is declared in the header but not exported"
    assert native_lib.fdnn_abi_version() == 2
    assert native_lib.fdnn_status_string(0) == b"ok"
    assert b"unknown" in native_lib.fdnn_status_string(12345)


def test_struct_layout_matches_header():
    # 18 int32 + 3 x 4 int64
    assert ctypes.sizeof(nat.ConvDesc) == 18 * 4 + 12 * 8
    assert ctypes.sizeof(nat.ConvPlan) == 16 * 4 + 4 * 8 + 2 * 8  # 16 ints, 4 int64, 2 doubles


def test_query_plans_headline_configs(native_lib):
    plan = nat.ConvPlan()
    # 3x3 256-channel headline layer: in place, 256 x 256 tiles on CTA pairs, one CTA per SM
    d = _desc(n=256, c=256, h=14, w=14, k=256)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
    assert (plan.algo, plan.tile_m, plan.tile_n, plan.x_repacked, plan.w_packed) == (nat.ALGO_IGEMM_PAIR, 256, 256, 0, 0)
    d.algo = nat.ALGO_IGEMM  # the single-CTA kernel can still be asked for
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
    assert (plan.algo, plan.tile_m, plan.tile_n, plan.stages) == (nat.ALGO_IGEMM, 128, 256, 3)
    assert plan.workspace_bytes == 0 and plan.packed_weight_bytes == 0
    assert plan.oh == 14 and plan.ow == 14 and plan.block == 384 and plan.grid == 148
    assert plan.flops == pytest.approx(59.190e9, rel=1e-3)
    assert plan.bytes == pytest.approx(52.56e6, rel=1e-2)
    # 1x1 bottleneck reduce: narrow tile so the activations are read once
    d = _desc(n=256, c=256, h=56, w=56, k=64, r=1, s=1, pad=0)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
    assert plan.tile_n == 64 and plan.flops == pytest.approx(26.307e9, rel=1e-3)
    # fp32 NCHW: repacked and split, two launches
    d = _desc(dtype=nat.F32, n=4, c=64, h=56, w=56, k=64, channels_last=False)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
    assert plan.algo == nat.ALGO_IGEMM and plan.x_repacked == 1 and plan.w_packed == 1 and plan.launches == 2
    assert plan.workspace_bytes == 2 * 4 * 56 * 56 * 64 * 4
    assert plan.packed_weight_bytes == 2 * 64 * 9 * 64 * 4
    # stem on CTA pairs: dense 3-channel input read in place (no relayout pass): pixel quads as GEMM rows
    # (4 x 64 = 256 columns), 48-element windows, two scratch slots of 13 input rows per CTA
    d = _desc(n=256, c=3, h=224, w=224, k=64, r=7, s=7, stride=2, pad=3)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
    assert plan.algo == nat.ALGO_IGEMM_PAIR and plan.low_channel == 2 and plan.c_padded == 3
    assert plan.x_repacked == 0 and plan.w_packed == 1 and plan.launches == 1 and plan.tile_k == 48
    assert plan.oh == 112 and plan.tile_n == 256
    assert plan.workspace_bytes == 148 * 2 * 18688               # 13 rows x 712 elements, rounded to 256 bytes
    assert plan.packed_weight_bytes == 256 * 7 * 64 * 2
    # the single-CTA kernel keeps the relayout: 3 channels stored as 4, rows padded to 232 stored pixels
    d.algo = nat.ALGO_IGEMM
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
    assert plan.low_channel == 1 and plan.c_padded == 4 and plan.x_repacked == 1 and plan.w_packed == 1
    assert plan.launches == 2 and plan.workspace_bytes == 256 * 224 * 232 * 4 * 2
    assert plan.packed_weight_bytes == 256 * 7 * 64 * 2
    # the same layer with an NCHW output cannot use it and falls back to 8-channel padding
    d = _desc(n=256, c=3, h=224, w=224, k=64, r=7, s=7, stride=2, pad=3, channels_last=False)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
    assert plan.low_channel == 0 and plan.c_padded == 8


def test_query_routes_unsupported_geometry_to_direct(native_lib):
    plan = nat.ConvPlan()
    for d in (_desc(groups=2, n=1), _desc(dtype=nat.F64), _desc(stride=9, h=40, w=40), _desc(pad=200, h=8, w=8)):
        assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
        assert plan.algo == nat.ALGO_DIRECT and plan.workspace_bytes == 0
    d = _desc(groups=16, algo=nat.ALGO_IGEMM)     # four channels per group: no tensor-core view of a group
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_NOT_SUPPORTED
    d = _desc(algo=nat.ALGO_IGEMM_PAIR, channels_last=False)  # NCHW output cannot go through the pair kernel
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_NOT_SUPPORTED
    d = _desc(algo=nat.ALGO_IGEMM_PAIR, dtype=nat.F32)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_NOT_SUPPORTED
    with pytest.raises(NotImplementedError):
        nat.check(nat.FDNN_NOT_SUPPORTED)


def test_query_float32_output_flag(native_lib):
    """FDNN_ALGO_FLAG_OUT_F32: 16-bit operands only, single-CTA tensor-core kernel, no pixel groups / quads."""
    plan, wide = nat.ConvPlan(), nat.ConvPlan()
    d = _desc(n=1, c=1024, h=1, w=4096, k=256, r=1, s=1, pad=0)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
    d.algo = nat.ALGO_FLAG_OUT_F32
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(wide)) == nat.FDNN_OK
    assert wide.algo == nat.ALGO_IGEMM and wide.low_channel == 0 and wide.pixel_group <= 1
    assert wide.bytes == plan.bytes + 2.0 * 4096 * 256          # y costs four bytes an element
    d = _desc(algo=nat.ALGO_FLAG_OUT_F32, c=3, h=32, w=32, k=64, r=7, s=7, stride=2, pad=3)   # a stem: no quads
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(wide)) == nat.FDNN_OK
    assert wide.algo == nat.ALGO_IGEMM and wide.low_channel == 0
    d = _desc(dtype=nat.F32, algo=nat.ALGO_FLAG_OUT_F32)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(wide)) == nat.FDNN_BAD_PARAM
    for algo in (nat.ALGO_DIRECT, nat.ALGO_IGEMM_PAIR):
        d = _desc(algo=algo | nat.ALGO_FLAG_OUT_F32)
        assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(wide)) == nat.FDNN_NOT_SUPPORTED
    d = _desc(groups=2, algo=nat.ALGO_FLAG_OUT_F32)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(wide)) == nat.FDNN_NOT_SUPPORTED


def test_query_tile_override_flags(native_lib):
    """FDNN_ALGO_FLAG_TILE_N_* fix the single-CTA kernel's tile width, FDNN_ALGO_FLAG_NO_PIXEL_GROUP keeps a
    narrow layer ungrouped; without them the planner's own choice stands."""
    plan = nat.ConvPlan()
    for flag, width in ((nat.ALGO_FLAG_TILE_N_64, 64), (nat.ALGO_FLAG_TILE_N_128, 128), (nat.ALGO_FLAG_TILE_N_256, 256)):
        d = _desc(n=128, c=512, h=7, w=7, k=512, algo=nat.ALGO_IGEMM | flag)
        assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
        assert plan.algo == nat.ALGO_IGEMM and plan.tile_n == width
        assert plan.grid == min(148, 49 * (512 // width))
    d = _desc(dtype=nat.F32, n=8, c=64, h=28, w=28, k=256, algo=nat.ALGO_IGEMM | nat.ALGO_FLAG_TILE_N_256)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
    assert plan.tile_n == 128                                    # fp32 tiles stop at 128 columns
    narrow = dict(n=256, c=64, h=56, w=56, k=64, r=3, s=3, pad=1)
    d = _desc(**narrow)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
    grouped = plan.pixel_group
    d = _desc(algo=nat.ALGO_FLAG_NO_PIXEL_GROUP, **narrow)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
    assert plan.pixel_group <= 1 and grouped > 1, "the 64-channel 3x3 layer is the case pixel grouping exists for"


def test_query_grouped_layers_take_a_tensor_core_route(native_lib):
    """groups > 1, not depthwise.  Up to eight groups: one dense convolution with a block-diagonal filter (the dense
    plan, plus room for the dense filter in front of the packed one).  More groups with at least 8 channels and
    16-byte multiples of channels per group: the plan of one group, launched once per group, one packed filter per
    group.  Depthwise, narrow groups and a forced direct kernel stay direct."""
    dense, one, plan = nat.ConvPlan(), nat.ConvPlan(), nat.ConvPlan()
    d = _desc(n=16, c=64, h=56, w=56, k=128, groups=2)                    # a grouped shape the reference times
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, 0x1002, None, ctypes.byref(plan)) == nat.FDNN_OK
    v = _desc(n=16, c=64, h=56, w=56, k=128)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(v), None, None, None, ctypes.byref(dense)) == nat.FDNN_OK
    assert plan.algo == dense.algo and plan.algo != nat.ALGO_DIRECT and plan.launches == dense.launches
    assert (plan.tile_n, plan.pixel_group, plan.grid) == (dense.tile_n, dense.pixel_group, dense.grid)
    assert plan.w_packed == 1 and plan.packed_weight_bytes == 128 * 9 * 64 * 2 + dense.packed_weight_bytes
    assert plan.flops == 2.0 * 16 * 56 * 56 * 128 * 32 * 9                # the layer's work, not the dense GEMM's
    d = _desc(n=16, c=128, h=28, w=28, k=128, groups=8)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
    assert plan.algo != nat.ALGO_DIRECT and plan.packed_weight_bytes >= 128 * 9 * 128 * 2

    sub = _desc(n=16, c=16, h=28, w=28, k=32, algo=nat.ALGO_IGEMM)
    sub.w_strides[0] = 3 * 3 * 16
    assert native_lib.fdnn_conv2d_query(ctypes.byref(sub), None, 0x1002, None, ctypes.byref(one)) == nat.FDNN_OK
    d = _desc(n=16, c=256, h=28, w=28, k=512, groups=16, algo=nat.ALGO_IGEMM)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, 0x1002, None, ctypes.byref(plan)) == nat.FDNN_OK
    assert plan.algo == nat.ALGO_IGEMM
    assert plan.launches == 16 * one.launches and plan.packed_weight_bytes == 16 * one.packed_weight_bytes
    for d in (_desc(n=16, c=64, h=56, w=56, k=64, groups=64), _desc(n=16, c=64, h=56, w=56, k=64, groups=16),
              _desc(n=16, c=64, h=56, w=56, k=128, groups=2, algo=nat.ALGO_DIRECT),
              _desc(dtype=nat.F32, n=16, c=160, h=56, w=56, k=160, groups=16)):     # 10 fp32 channels: 40 bytes
        assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_OK
        assert plan.algo == nat.ALGO_DIRECT


def test_query_unaligned_pointer_forces_repack(native_lib):
    plan = nat.ConvPlan()
    d = _desc()
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), 0x1000, 0x2000, None, ctypes.byref(plan)) == nat.FDNN_OK
    assert plan.x_repacked == 0 and plan.w_packed == 0
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), 0x1002, 0x2004, None, ctypes.byref(plan)) == nat.FDNN_OK
    assert plan.x_repacked == 1 and plan.w_packed == 1


@pytest.mark.parametrize("field,value,fragment", [
    ("groups", 0, "groups must be a positive integer"),
    ("stride_h", 0, "stride must be positive"),
    ("dil_w", 0, "dilation must be positive"),
    ("pad_left", -1, "negative padding is not supported"),
    ("groups", 3, "channels must be divisible by groups"),
    ("dtype", 9, "Unsupported dtype"),
])
def test_query_rejects_bad_descriptors(native_lib, field, value, fragment):
    d = _desc()
    setattr(d, field, value)
    plan = nat.ConvPlan()
    status = native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan))
    assert status in (nat.FDNN_BAD_PARAM, nat.FDNN_NOT_SUPPORTED)
    assert fragment in native_lib.fdnn_last_error().decode()
    with pytest.raises((RuntimeError, NotImplementedError)):
        nat.check(status)


def test_negative_output_and_null_arguments(native_lib):
    plan = nat.ConvPlan()
    d = _desc(h=1, w=9, r=5, s=5, pad=0)
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, ctypes.byref(plan)) == nat.FDNN_BAD_PARAM
    assert b"negative" in native_lib.fdnn_last_error()
    assert native_lib.fdnn_conv2d_query(None, None, None, None, ctypes.byref(plan)) == nat.FDNN_BAD_PARAM
    d = _desc()
    assert native_lib.fdnn_conv2d_query(ctypes.byref(d), None, None, None, None) == nat.FDNN_BAD_PARAM
    # fwd with missing buffers is refused before anything is launched
    assert native_lib.fdnn_conv2d_fwd(ctypes.byref(d), None, None, None, None, None, 0, None, None, 0, None) == nat.FDNN_BAD_PARAM
    assert native_lib.fdnn_conv2d_fwd(ctypes.byref(d), 0x1000, 0x2000, None, None, None, 7, 0x3000, None, 0, None) == nat.FDNN_BAD_PARAM
    need = ctypes.c_int64(0)
    assert native_lib.fdnn_conv2d_host_arena_bytes(ctypes.byref(d), ctypes.byref(need)) == nat.FDNN_OK
    assert need.value > 0

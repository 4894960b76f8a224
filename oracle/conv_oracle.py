"""CPU oracle for conv2d / conv -> (scale) -> bias -> ReLU.  TEST INFRASTRUCTURE.

Two independent legs:

* ``conv2d_torch_cpu`` — the reference's own CPU path.  On CPU tensors the
  reference's graph executor runs ``torch.nn.functional.conv2d`` followed by
  ``torch.nn.functional.relu`` (src/flag_dnn/graph/registry.py:1357-1365, 1426;
  bias_add is ``x + bias.reshape(1,-1,1,1)``, registry.py:1007-1009).  The
  arithmetic lives in PyTorch (pinned ``torch>=2.6.0`` by the reference's
  pyproject.toml:23; 2.11.0 in this image), not in the reference's tree.
* ``conv2d_loops`` — plain C loops (conv_oracle.c) following the index math of
  src/flag_dnn/graph/kernels/fused_conv.py:249-299, accumulating in double.

Both are pinned against outputs of the reference itself (tests/golden/*.npz,
produced by tests/golden/make_golden.py running the unmodified reference on
CPU); tests/test_oracle_golden.py checks that.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path
from typing import Optional, Sequence, Tuple, Union

import numpy as np
import torch

_DIR = Path(__file__).resolve().parent
_LIB_PATH = _DIR / "libconv_oracle.so"
_lib = None


class _Desc(ctypes.Structure):
    _fields_ = (
        [(n, ctypes.c_int) for n in (
            "n", "c", "h", "w", "k", "r", "s",
            "stride_h", "stride_w", "pad_top", "pad_left", "dil_h", "dil_w", "groups",
            "oh", "ow", "relu")]
        + [("xs", ctypes.c_int64 * 4), ("ws", ctypes.c_int64 * 4), ("ys", ctypes.c_int64 * 4)]
    )


def build(force: bool = False) -> Path:
    """Compile conv_oracle.c with gcc if the library is missing or stale."""
    src = _DIR / "conv_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        cc = os.environ.get("CC", "gcc")
        subprocess.run([cc, "-O2", "-fPIC", "-shared", "-o", str(_LIB_PATH), str(src)], check=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        _lib.oracle_conv_out_dim.restype = ctypes.c_int
    return _lib


def _pair(v) -> Tuple[int, int]:
    if isinstance(v, int):
        return v, v
    return int(v[0]), int(v[1])


def conv_out_dim(size: int, pad_before: int, pad_after: int, dilation: int, kernel: int, stride: int) -> int:
    """src/flag_dnn/ops/conv2d.py:52-62."""
    return (size + pad_before + pad_after - dilation * (kernel - 1) - 1) // stride + 1


def normalize_padding(weight_shape, stride, padding, dilation) -> Tuple[int, int, int, int]:
    """(top, bottom, left, right), the rule of src/flag_dnn/ops/conv2d.py:65-87."""
    if isinstance(padding, str):
        if padding == "valid":
            return 0, 0, 0, 0
        if padding == "same":
            if tuple(stride) != (1, 1):
                raise RuntimeError("padding='same' is not supported for strided convolutions")
            kh, kw = weight_shape[2], weight_shape[3]
            ph = max(dilation[0] * (kh - 1), 0)
            pw = max(dilation[1] * (kw - 1), 0)
            return ph // 2, ph - ph // 2, pw // 2, pw - pw // 2
        raise RuntimeError("padding must be 'valid', 'same', int, or tuple")
    ph, pw = _pair(padding)
    return ph, ph, pw, pw


def conv2d_torch_cpu(
    x: torch.Tensor,
    w: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    stride=1,
    padding: Union[str, int, Sequence[int]] = 0,
    dilation=1,
    groups: int = 1,
    scale: Optional[torch.Tensor] = None,
    relu: bool = False,
    compute_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    """The reference's CPU path: F.conv2d (+ bias) then F.relu, on CPU.

    16-bit inputs are upcast exactly to ``compute_dtype`` first, so the result
    is the fp32 (or fp64) answer for the very bits the GPU kernel sees.  The
    optional BN-folded ``scale`` has no counterpart in the reference; it is
    applied as ``conv(x, w) * scale[k]`` before the bias.
    """
    xd = x.detach().cpu().to(compute_dtype)
    wd = w.detach().cpu().to(compute_dtype)
    bd = None if bias is None else bias.detach().cpu().to(compute_dtype)
    pad = padding if isinstance(padding, str) else _pair(padding)
    if scale is None:
        y = torch.nn.functional.conv2d(xd, wd, bias=bd, stride=_pair(stride), padding=pad,
                                       dilation=_pair(dilation), groups=groups)
    else:
        y = torch.nn.functional.conv2d(xd, wd, bias=None, stride=_pair(stride), padding=pad,
                                       dilation=_pair(dilation), groups=groups)
        y = y * scale.detach().cpu().to(compute_dtype).reshape(1, -1, 1, 1)
        if bd is not None:
            y = y + bd.reshape(1, -1, 1, 1)
    if relu:
        y = torch.nn.functional.relu(y)
    return y


def conv2d_loops(
    x: torch.Tensor,
    w: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    stride=1,
    padding: Union[str, int, Sequence[int]] = 0,
    dilation=1,
    groups: int = 1,
    scale: Optional[torch.Tensor] = None,
    relu: bool = False,
    double: bool = False,
) -> torch.Tensor:
    """Plain-loop restatement (C, double accumulate).  Returns fp32 (or fp64) NCHW-shaped output."""
    lib = _load()
    np_t = np.float64 if double else np.float32
    t_t = torch.float64 if double else torch.float32
    xa = np.ascontiguousarray(x.detach().cpu().to(t_t).numpy())
    wa = np.ascontiguousarray(w.detach().cpu().to(t_t).numpy())
    ba = None if bias is None else np.ascontiguousarray(bias.detach().cpu().to(t_t).numpy())
    sa = None if scale is None else np.ascontiguousarray(scale.detach().cpu().to(t_t).numpy())
    stride = _pair(stride)
    dilation = _pair(dilation)
    pt, pb, pl, pr = normalize_padding(wa.shape, stride, padding, dilation)
    n, c, h, wd_ = xa.shape
    k, cg, r, s = wa.shape
    oh = conv_out_dim(h, pt, pb, dilation[0], r, stride[0])
    ow = conv_out_dim(wd_, pl, pr, dilation[1], s, stride[1])
    ya = np.zeros((n, k, max(oh, 0), max(ow, 0)), dtype=np_t)
    if oh <= 0 or ow <= 0 or n == 0:
        return torch.from_numpy(ya)
    d = _Desc()
    d.n, d.c, d.h, d.w, d.k, d.r, d.s = n, c, h, wd_, k, r, s
    d.stride_h, d.stride_w = stride
    d.pad_top, d.pad_left = pt, pl
    d.dil_h, d.dil_w = dilation
    d.groups = groups
    d.oh, d.ow, d.relu = oh, ow, int(relu)
    item = xa.itemsize
    for i in range(4):
        d.xs[i] = xa.strides[i] // item
        d.ws[i] = wa.strides[i] // item
        d.ys[i] = ya.strides[i] // item
    fn = lib.oracle_conv2d_f64 if double else lib.oracle_conv2d_f32
    ptr = lambda a: None if a is None else a.ctypes.data_as(ctypes.c_void_p)
    rc = fn(ctypes.byref(d), ptr(xa), ptr(wa), ptr(ba), ptr(sa), ptr(ya))
    if rc != 0:
        raise RuntimeError(f"oracle returned {rc}")
    return torch.from_numpy(ya)

"""Host side of the pooling operators next to the convolution path.

``max_pool2d`` and ``adaptive_avg_pool2d`` keep the reference's signatures
(src/flag_dnn/ops/max_pool2d.py:174-182, src/flag_dnn/ops/adaptive_avg_pool2d.py:456-459)
and run on this library's CUDA kernels through the C ABI.  Unlike the reference,
which asserts a contiguous NCHW input, channels-last inputs are taken as they
are and produce channels-last outputs, so that a ResNet's stem -> pool -> blocks
-> pool chain stays in one layout.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple, Union

import torch

from . import _native as nat

_DTYPE_IDS = {torch.float16: nat.F16, torch.bfloat16: nat.BF16, torch.float32: nat.F32, torch.float64: nat.F64}


def _pair(v) -> Tuple[int, int]:
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def _prepare(input: torch.Tensor, what: str):
    assert input.ndim in [3, 4], "Input must be 3D or 4D"
    if input.dtype not in _DTYPE_IDS:
        raise NotImplementedError(f"flag_dnn {what} does not support dtype={input.dtype}")
    if not input.is_cuda:
        raise NotImplementedError(f"flag_dnn {what} CUDA implementation requires CUDA input")
    is_3d = input.ndim == 3
    return (input.unsqueeze(0) if is_3d else input), is_3d


def _empty_like_layout(x: torch.Tensor, shape, dtype=None) -> torch.Tensor:
    channels_last = x.dim() == 4 and x.stride(1) == 1 and x.shape[1] > 1
    return torch.empty(shape, dtype=dtype or x.dtype, device=x.device,
                       memory_format=torch.channels_last if channels_last else torch.contiguous_format)


def _desc(x: torch.Tensor, y: torch.Tensor) -> "nat.PoolDesc":
    d = nat.PoolDesc()
    d.dtype = _DTYPE_IDS[x.dtype]
    d.n, d.c, d.h, d.w = x.shape
    d.oh, d.ow = y.shape[2], y.shape[3]
    d.kernel_h = d.kernel_w = d.stride_h = d.stride_w = d.dil_h = d.dil_w = 1
    d.pad_h = d.pad_w = 0
    for i in range(4):
        d.x_strides[i] = x.stride(i)
        d.y_strides[i] = y.stride(i)
    return d


def max_pool2d(
    input: torch.Tensor,
    kernel_size: Union[int, Tuple[int, int]],
    stride: Optional[Union[int, Tuple[int, int]]] = None,
    padding: Union[int, Tuple[int, int]] = 0,
    dilation: Union[int, Tuple[int, int]] = 1,
    ceil_mode: bool = False,
    return_indices: bool = False,
):
    """Drop-in for ``flag_dnn.ops.max_pool2d`` (src/flag_dnn/ops/max_pool2d.py:174); output sizes follow
    its rule (src/flag_dnn/ops/max_pool2d.py:201-230), values and indices torch.nn.functional.max_pool2d."""
    kernel = _pair(kernel_size)
    stride2 = _pair(stride) if stride is not None else kernel
    pad = _pair(padding)
    dil = _pair(dilation)
    x, is_3d = _prepare(input, "max_pool2d")
    n, c, h, w = x.shape
    if min(kernel) <= 0 or min(stride2) <= 0 or min(dil) <= 0 or min(pad) < 0:
        raise RuntimeError("kernel_size, stride and dilation must be positive and padding non-negative")
    if 2 * pad[0] > kernel[0] or 2 * pad[1] > kernel[1]:
        raise RuntimeError("pad should be at most half of effective kernel size")

    def out_size(length, p, d, k, s):
        out = (length + 2 * p - d * (k - 1) - 1) / s + 1
        out = math.ceil(out) if ceil_mode else math.floor(out)
        if ceil_mode and (out - 1) * s >= length + p:
            out -= 1
        return max(int(out), 0)

    oh = out_size(h, pad[0], dil[0], kernel[0], stride2[0])
    ow = out_size(w, pad[1], dil[1], kernel[1], stride2[1])
    y = _empty_like_layout(x, (n, c, oh, ow))
    idx = _empty_like_layout(x, (n, c, oh, ow), torch.int64) if return_indices else None
    if y.numel() > 0:
        d = _desc(x, y)
        d.kernel_h, d.kernel_w = kernel
        d.stride_h, d.stride_w = stride2
        d.pad_h, d.pad_w = pad
        d.dil_h, d.dil_w = dil
        with torch.cuda.device(x.device):
            nat.check(nat.load().fdnn_max_pool2d_fwd(
                ctypes.byref(d), x.data_ptr(), y.data_ptr(), None if idx is None else idx.data_ptr(),
                torch.cuda.current_stream().cuda_stream))
    if is_3d:
        y = y.squeeze(0)
        idx = None if idx is None else idx.squeeze(0)
    return (y, idx) if return_indices else y


def adaptive_avg_pool2d(
    input: torch.Tensor,
    output_size: Union[int, Tuple[Optional[int], Optional[int]]],
) -> torch.Tensor:
    """Drop-in for ``flag_dnn.ops.adaptive_avg_pool2d`` (src/flag_dnn/ops/adaptive_avg_pool2d.py:456)."""
    if isinstance(output_size, int):
        oh = ow = int(output_size)
    else:
        assert len(output_size) == 2, "output_size for adaptive_avg_pool2d must have 2 elements"
        oh = int(output_size[0]) if output_size[0] is not None else input.shape[-2]
        ow = int(output_size[1]) if output_size[1] is not None else input.shape[-1]
    x, is_3d = _prepare(input, "adaptive_avg_pool2d")
    n, c, h, w = x.shape
    y = _empty_like_layout(x, (n, c, oh, ow))
    if y.numel() > 0:
        if h == 0 or w == 0:
            raise RuntimeError("adaptive_avg_pool2d: the input plane must not be empty")
        d = _desc(x, y)
        with torch.cuda.device(x.device):
            nat.check(nat.load().fdnn_adaptive_avg_pool2d_fwd(
                ctypes.byref(d), x.data_ptr(), y.data_ptr(), torch.cuda.current_stream().cuda_stream))
    return y.squeeze(0) if is_3d else y

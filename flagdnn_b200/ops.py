"""The ``flag_dnn.ops`` names on the convolution path.

Each function records a node while a graph is being captured and runs eagerly
otherwise, like the reference's wrappers (src/flag_dnn/graph/wrappers.py:49-87).
``conv2d`` always runs through the native library; ``bias_add`` / ``relu`` /
``add`` / ``sub`` / ``mul`` are the glue ops of the conv -> bias -> ReLU graphs.
"""
from __future__ import annotations

from typing import Any

import torch

from . import conv_host as _conv
from . import pool_host as _pool
from .graph.compiler import current_capture


def _capturable(op_type: str, eager):
    def wrapper(*args: Any, **kwargs: Any):
        ctx = current_capture()
        if ctx is not None:
            return ctx.add_op_call(op_type, args, kwargs)
        return eager(*args, **kwargs)

    wrapper.__name__ = op_type
    wrapper.__doc__ = eager.__doc__
    return wrapper


def _eager_bias_add(x: torch.Tensor, bias: torch.Tensor, **_: Any) -> torch.Tensor:
    """x + bias broadcast along dim 1 (src/flag_dnn/graph/wrappers.py:82-87)."""
    if bias.dim() == 1 and x.dim() >= 2:
        shape = [1] * x.dim()
        shape[1] = bias.numel()
        bias = bias.reshape(shape)
    return x + bias


def _eager_relu(x: torch.Tensor, inplace: bool = False, **_: Any) -> torch.Tensor:
    return torch.relu_(x) if inplace else torch.relu(x)


def _eager_gelu(x: torch.Tensor, approximate: str = "none", **_: Any) -> torch.Tensor:
    return torch.nn.functional.gelu(x, approximate=approximate)


def _eager_binary(fn):
    def run(x, y, **_: Any):
        return fn(x, y)
    return run


conv2d = _capturable("conv2d", _conv.conv2d)
bias_add = _capturable("bias_add", _eager_bias_add)
relu = _capturable("relu", _eager_relu)
gelu = _capturable("gelu", _eager_gelu)
max_pool2d = _capturable("max_pool2d", _pool.max_pool2d)
adaptive_avg_pool2d = _capturable("adaptive_avg_pool2d", _pool.adaptive_avg_pool2d)
add = _capturable("add", _eager_binary(torch.add))
sub = _capturable("sub", _eager_binary(torch.sub))
mul = _capturable("mul", _eager_binary(torch.mul))
conv1d = _conv.conv1d  # eager only: the graph registry has no conv1d node, as in the reference
mm = _conv.mm          # eager only
fused_conv2d_bias_relu = _conv.fused_conv2d_bias_relu

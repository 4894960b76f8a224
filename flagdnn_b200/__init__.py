"""flagdnn_b200 — the conv2d / conv->bias->ReLU hot path of FlagDNN, rebuilt
for B200 (sm_100a) behind FlagDNN's own Python call signatures.

    import flagdnn_b200 as flag_dnn
    y = flag_dnn.conv2d(x, w, b, stride=1, padding=1)          # eager
    compiled = flag_dnn.compile(fn, inputs=[...])               # graph API
    with flag_dnn.use_dnn(): torch.nn.functional.conv2d(...)    # aten override

Everything that computes a convolution goes through the native library
(``libflagdnn_b200.so``, C ABI in ``include/flagdnn_b200.h``); importing this
package does not need a GPU, calling a convolution does.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import ops  # noqa: F401
from .conv_host import (  # noqa: F401
    conv2d_bias_act,
    conv2d_plan,
    device_status,
    fused_conv2d_bias_relu,
    set_algo,
    set_stream_k,
)
from .graph import (  # noqa: F401
    CompiledGraph,
    GraphTensor,
    PlanCache,
    TensorSpec,
    compile,
    graph,
)
from .ops import (  # noqa: F401
    adaptive_avg_pool2d, add, bias_add, conv1d, conv2d, gelu, max_pool2d, mm, mul, relu, sub,
)

__version__ = "0.1.0"

device = "cuda"

_ATEN_LIB: Optional[torch.library.Library] = None


def _aten_conv2d(input, weight, bias=None, stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups=1):
    from . import conv_host as native

    return native.conv2d(input, weight, bias, tuple(stride), tuple(padding), tuple(dilation), groups)


def enable() -> None:
    """Route ``aten::conv2d`` on CUDA tensors to this library
    (src/flag_dnn/__init__.py:195-232 registers conv2d the same way)."""
    global _ATEN_LIB
    if _ATEN_LIB is not None:
        return
    lib = torch.library.Library("aten", "IMPL")
    lib.impl("conv2d", _aten_conv2d, "CUDA")
    _ATEN_LIB = lib


def disable() -> None:
    global _ATEN_LIB
    if _ATEN_LIB is not None:
        _ATEN_LIB._destroy()
        _ATEN_LIB = None


class use_dnn:
    """Context manager form of ``enable`` (src/flag_dnn/__init__.py:294-343)."""

    def __enter__(self):
        enable()
        return self

    def __exit__(self, exc_type, exc, tb):
        disable()
        return False

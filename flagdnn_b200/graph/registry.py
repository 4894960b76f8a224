"""Op schemas for the graph API: how a call is recorded (normalize), what it
produces (infer) and how it executes (run).

Only the ops on or next to the convolution path are registered: conv2d,
bias_add, relu, the element-wise add / sub / mul used as glue, and the fused
nodes the fusion pass creates.  Counterpart of the conv-related entries of
src/flag_dnn/graph/registry.py (normalize 777-812, shape 436-479, run_fns
1343-1428, registrations 1563-1580).

Convolution nodes execute through the native library only.  A convolution
node fed CPU tensors raises NotImplementedError: this package carries no CPU
implementation of the hot path.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch

from .spec import TensorSpec

RunFn = Callable[[list, dict], Any]


@dataclass
class OpSchema:
    name: str
    normalize: Callable[[Any, tuple, dict], tuple]
    infer: Callable[[list, dict], TensorSpec]
    run: RunFn


_SCHEMAS: dict[str, OpSchema] = {}


def register_op(schema: OpSchema) -> None:
    _SCHEMAS[schema.name] = schema


def get_op_schema(name: str) -> OpSchema:
    try:
        return _SCHEMAS[name]
    except KeyError:
        raise NotImplementedError(f"graph op {name!r} is not registered") from None


def _public(attrs: dict) -> dict:
    return {k: v for k, v in attrs.items() if not k.startswith("_")}


def _pair(v) -> tuple:
    return (v, v) if isinstance(v, int) else (int(v[0]), int(v[1]))


# ------------------------------------------------------------------ conv2d
_CONV_ARG_NAMES = ["input", "weight", "bias", "stride", "padding", "dilation", "groups"]
_CONV_DEFAULTS = {"bias": None, "stride": 1, "padding": 0, "dilation": 1, "groups": 1}


def _normalize_conv2d(ctx: Any, args: tuple, kwargs: dict) -> tuple:
    if len(args) > len(_CONV_ARG_NAMES):
        raise TypeError("conv2d got too many positional args")
    params = dict(_CONV_DEFAULTS)
    params.update(kwargs)
    for name, arg in zip(_CONV_ARG_NAMES, args):
        if name in kwargs:
            raise TypeError(f"conv2d got multiple values for {name}")
        params[name] = arg
    input_ids = [ctx.as_value(params.pop("input"), "input"), ctx.as_value(params.pop("weight"), "weight")]
    bias = params.pop("bias")
    if bias is not None:
        input_ids.append(ctx.as_value(bias, "bias"))
    return input_ids, params


def _padding4(weight_shape, stride, padding, dilation) -> tuple:
    if isinstance(padding, str):
        if padding == "valid":
            return (0, 0, 0, 0)
        if padding == "same":
            if stride != (1, 1):
                raise RuntimeError("padding='same' is not supported for strided convolutions")
            ph = max(dilation[0] * (weight_shape[2] - 1), 0)
            pw = max(dilation[1] * (weight_shape[3] - 1), 0)
            return (ph // 2, ph - ph // 2, pw // 2, pw - pw // 2)
        raise RuntimeError("padding must be 'valid', 'same', int, or tuple")
    ph, pw = _pair(padding)
    return (ph, ph, pw, pw)


def _infer_conv2d(specs: list, attrs: dict) -> TensorSpec:
    x, weight = specs[0], specs[1]
    if len(x.shape) != 4 or len(weight.shape) != 4:
        raise RuntimeError("graph conv2d expects 4D input and weight")
    stride = _pair(attrs.get("stride", 1))
    dilation = _pair(attrs.get("dilation", 1))
    pt, pb, pl, pr = _padding4(weight.shape, stride, attrs.get("padding", 0), dilation)
    groups = int(attrs.get("groups", 1))
    n, c_in, h, w = x.shape
    c_out, c_per_group, kh, kw = weight.shape
    if c_in % groups != 0:
        raise RuntimeError("graph conv2d input channels must divide groups")
    if c_per_group != c_in // groups:
        raise RuntimeError("graph conv2d weight channel mismatch")
    oh = (h + pt + pb - dilation[0] * (kh - 1) - 1) // stride[0] + 1
    ow = (w + pl + pr - dilation[1] * (kw - 1) - 1) // stride[1] + 1
    if oh < 0 or ow < 0:
        raise RuntimeError("computed graph conv2d output size is negative")
    return TensorSpec("", (n, c_out, max(oh, 0), max(ow, 0)), x.dtype, layout=x.layout, device=x.device)


def _on_device(inputs: list) -> bool:
    return any(isinstance(t, torch.Tensor) and t.is_cuda for t in inputs)


def _require_device(inputs: list, what: str) -> None:
    if not _on_device(inputs):
        raise NotImplementedError(
            f"{what}: this build runs convolution nodes on CUDA tensors only (no CPU implementation)")


def _run_conv2d(inputs: list, attrs: dict) -> torch.Tensor:
    from .. import conv_host as native

    _require_device(inputs, "conv2d")
    a = _public(attrs)
    bias = inputs[2] if len(inputs) > 2 else None
    scale = inputs[3].reshape(-1) if len(inputs) > 3 else None
    out = attrs.get("_out")   # the executor's workspace slice for this node's output, if it planned one
    if scale is None:
        return native.conv2d(inputs[0], inputs[1], bias, a.get("stride", 1), a.get("padding", 0),
                             a.get("dilation", 1), a.get("groups", 1), out=out)
    return native.fused_conv2d_bias_relu(inputs[0], inputs[1], bias, stride=a.get("stride", 1),
                                         padding=a.get("padding", 0), dilation=a.get("dilation", 1),
                                         groups=a.get("groups", 1), scale=scale, activation="none", out=out)


def _run_fused_conv2d_bias_relu(inputs: list, attrs: dict) -> torch.Tensor:
    from .. import conv_host as native

    _require_device(inputs, "fused_conv2d_bias_relu")
    a = _public(attrs)
    scale = inputs[3].reshape(-1) if len(inputs) > 3 else None  # captured as (K,1,1) or (1,K,1,1)
    kw = dict(stride=a.get("stride", 1), padding=a.get("padding", 0), dilation=a.get("dilation", 1))
    try:
        return native.fused_conv2d_bias_relu(inputs[0], inputs[1], inputs[2], groups=a.get("groups", 1),
                                             config=attrs.get("_kernel_config"), scale=scale, out=attrs.get("_out"),
                                             **kw)
    except NotImplementedError:
        # Outside the fused entry's contract (grouped convolution, fp64): the
        # same native library still fuses bias and ReLU through its direct kernel.
        return native.conv2d_bias_act(inputs[0], inputs[1], inputs[2], groups=a.get("groups", 1),
                                      scale=scale, relu=True, out=attrs.get("_out"), **kw)


def _gelu_code(attrs: dict) -> str:
    return "gelu_tanh" if attrs.get("approximate", "none") == "tanh" else "gelu"


def _run_fused_conv2d_bias_gelu(inputs: list, attrs: dict) -> torch.Tensor:
    """inputs: x, w, bias[, scale]; gelu(conv * scale + bias) in the convolution's epilogue."""
    from .. import conv_host as native

    _require_device(inputs, "fused_conv2d_bias_gelu")
    a = _public(attrs)
    scale = inputs[3].reshape(-1) if len(inputs) > 3 else None
    return native.conv2d_bias_act(inputs[0], inputs[1], inputs[2], stride=a.get("stride", 1),
                                  padding=a.get("padding", 0), dilation=a.get("dilation", 1),
                                  groups=a.get("groups", 1), scale=scale, activation=_gelu_code(attrs),
                                  out=attrs.get("_out"))


def _run_fused_conv2d_bias_add_relu(inputs: list, attrs: dict) -> torch.Tensor:
    """inputs: x, w, residual[, bias[, scale]]; relu(conv * scale + bias + residual) in one kernel."""
    from .. import conv_host as native

    _require_device(inputs, "fused_conv2d_bias_add_relu")
    a = _public(attrs)
    bias = inputs[3] if len(inputs) > 3 else None
    scale = inputs[4].reshape(-1) if len(inputs) > 4 else None
    return native.conv2d_bias_act(inputs[0], inputs[1], bias, stride=a.get("stride", 1), padding=a.get("padding", 0),
                                  dilation=a.get("dilation", 1), groups=a.get("groups", 1), scale=scale,
                                  relu=a.get("activation", "relu") == "relu", residual=inputs[2],
                                  out=attrs.get("_out"))


def _normalize_conv2d_residual(ctx: Any, args: tuple, kwargs: dict) -> tuple:
    raise NotImplementedError("fused_conv2d_bias_add_relu nodes are created by the fusion pass only")


def _infer_conv2d_residual(specs: list, attrs: dict) -> TensorSpec:
    return _infer_conv2d([specs[0], specs[1]], attrs)


# ---------------------------------------------------------------- pooling
_MAXPOOL_ARG_NAMES = ["input", "kernel_size", "stride", "padding", "dilation", "ceil_mode", "return_indices"]


def _normalize_max_pool2d(ctx: Any, args: tuple, kwargs: dict) -> tuple:
    params = {"stride": None, "padding": 0, "dilation": 1, "ceil_mode": False, "return_indices": False}
    params.update(kwargs)
    for name, arg in zip(_MAXPOOL_ARG_NAMES, args):
        params[name] = arg
    if params.get("return_indices"):
        raise NotImplementedError("graph max_pool2d returns values only (return_indices=False)")
    if "input" not in params or "kernel_size" not in params:
        raise TypeError("max_pool2d expects an input and a kernel_size")
    return [ctx.as_value(params.pop("input"), "input")], params


def _infer_max_pool2d(specs: list, attrs: dict) -> TensorSpec:
    import math

    x = specs[0]
    if len(x.shape) != 4:
        raise RuntimeError("graph max_pool2d expects a 4D input")
    kernel = _pair(attrs["kernel_size"])
    stride = _pair(attrs["stride"]) if attrs.get("stride") is not None else kernel
    pad, dil = _pair(attrs.get("padding", 0)), _pair(attrs.get("dilation", 1))
    ceil_mode = bool(attrs.get("ceil_mode", False))

    def out(length, p, d, k, s):
        o = (length + 2 * p - d * (k - 1) - 1) / s + 1
        o = math.ceil(o) if ceil_mode else math.floor(o)
        if ceil_mode and (o - 1) * s >= length + p:
            o -= 1
        return max(int(o), 0)

    n, c, h, w = x.shape
    return TensorSpec("", (n, c, out(h, pad[0], dil[0], kernel[0], stride[0]), out(w, pad[1], dil[1], kernel[1], stride[1])),
                      x.dtype, layout=x.layout, device=x.device)


def _run_max_pool2d(inputs: list, attrs: dict) -> torch.Tensor:
    from .. import pool_host

    a = _public(attrs)
    if not _on_device(inputs):   # glue on CPU specs (shape checks, tests); device tensors use the library
        return torch.nn.functional.max_pool2d(inputs[0], a["kernel_size"], a.get("stride"), a.get("padding", 0),
                                              a.get("dilation", 1), bool(a.get("ceil_mode", False)))
    return pool_host.max_pool2d(inputs[0], a["kernel_size"], a.get("stride"), a.get("padding", 0),
                                a.get("dilation", 1), bool(a.get("ceil_mode", False)))


def _normalize_adaptive_avg_pool2d(ctx: Any, args: tuple, kwargs: dict) -> tuple:
    params = dict(kwargs)
    for name, arg in zip(["input", "output_size"], args):
        params[name] = arg
    if "input" not in params or "output_size" not in params:
        raise TypeError("adaptive_avg_pool2d expects an input and an output_size")
    return [ctx.as_value(params.pop("input"), "input")], params


def _infer_adaptive_avg_pool2d(specs: list, attrs: dict) -> TensorSpec:
    x = specs[0]
    if len(x.shape) != 4:
        raise RuntimeError("graph adaptive_avg_pool2d expects a 4D input")
    size = attrs["output_size"]
    oh, ow = (size, size) if isinstance(size, int) else size
    oh = x.shape[2] if oh is None else int(oh)
    ow = x.shape[3] if ow is None else int(ow)
    return TensorSpec("", (x.shape[0], x.shape[1], oh, ow), x.dtype, layout=x.layout, device=x.device)


def _run_adaptive_avg_pool2d(inputs: list, attrs: dict) -> torch.Tensor:
    from .. import pool_host

    a = _public(attrs)
    if not _on_device(inputs):
        return torch.nn.functional.adaptive_avg_pool2d(inputs[0], a["output_size"])
    return pool_host.adaptive_avg_pool2d(inputs[0], a["output_size"])


# -------------------------------------------------------------- glue ops
def _normalize_unary(name: str):
    def normalize(ctx: Any, args: tuple, kwargs: dict) -> tuple:
        if len(args) < 1:
            raise TypeError(f"{name} expects a tensor")
        attrs = dict(kwargs)
        return [ctx.as_value(args[0], "input")], attrs
    return normalize


def _normalize_binary(name: str):
    def normalize(ctx: Any, args: tuple, kwargs: dict) -> tuple:
        if len(args) != 2:
            raise TypeError(f"{name} expects two operands")
        attrs = dict(kwargs)
        ids = [ctx.as_value(args[0], "input")]
        if ctx.is_tensor_like(args[1]):
            ids.append(ctx.as_value(args[1], "other"))
        else:
            attrs["other"] = args[1]
        return ids, attrs
    return normalize


def _infer_same(specs: list, attrs: dict) -> TensorSpec:
    x = specs[0]
    return TensorSpec("", x.shape, x.dtype, layout=x.layout, device=x.device)


def _infer_broadcast(specs: list, attrs: dict) -> TensorSpec:
    x = specs[0]
    if len(specs) == 1:
        return _infer_same(specs, attrs)
    shape = tuple(torch.broadcast_shapes(tuple(x.shape), tuple(specs[1].shape)))
    return TensorSpec("", shape, x.dtype, layout=x.layout, device=x.device)


def _format_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    if bias.dim() == 1 and x.dim() >= 2:
        shape = [1] * x.dim()
        shape[1] = bias.numel()
        return bias.reshape(shape)
    return bias


def _usable_out(attrs: dict, *operands) -> Optional[torch.Tensor]:
    """The planned output slice, if every tensor operand has its dtype (no type promotion in play)."""
    out = attrs.get("_out")
    if out is None or any(isinstance(t, torch.Tensor) and t.dtype != out.dtype for t in operands):
        return None
    return out


def _run_bias_add(inputs: list, attrs: dict) -> torch.Tensor:
    x, bias = inputs
    out = _usable_out(attrs, x, bias)
    if out is not None and tuple(out.shape) == tuple(x.shape):
        return torch.add(x, _format_bias(x, bias), out=out)
    return x + _format_bias(x, bias)


def _run_relu(inputs: list, attrs: dict) -> torch.Tensor:
    out = _usable_out(attrs, inputs[0])
    if out is not None and tuple(out.shape) == tuple(inputs[0].shape):
        return torch.clamp_min(inputs[0], 0, out=out)   # NaN stays NaN, like torch.relu
    return torch.relu(inputs[0])


def _run_fused_bias_relu(inputs: list, attrs: dict) -> torch.Tensor:
    return torch.relu_(_run_bias_add(inputs, attrs)) if attrs.get("_out") is not None else \
        torch.relu(_run_bias_add(inputs, attrs))


def _run_gelu(inputs: list, attrs: dict) -> torch.Tensor:
    return torch.nn.functional.gelu(inputs[0], approximate=attrs.get("approximate", "none"))


def _run_fused_bias_gelu(inputs: list, attrs: dict) -> torch.Tensor:
    return torch.nn.functional.gelu(_run_bias_add(inputs, attrs), approximate=attrs.get("approximate", "none"))


def _binary_runner(fn):
    def run(inputs: list, attrs: dict) -> torch.Tensor:
        other = inputs[1] if len(inputs) > 1 else attrs["other"]
        if attrs.get("reverse") and len(inputs) == 1:
            return fn(torch.as_tensor(other, dtype=inputs[0].dtype, device=inputs[0].device), inputs[0])
        out = _usable_out(attrs, inputs[0], other)
        if out is not None and isinstance(other, torch.Tensor) and \
                tuple(out.shape) == tuple(torch.broadcast_shapes(inputs[0].shape, other.shape)):
            return fn(inputs[0], other, out=out)
        return fn(inputs[0], other)
    return run


def _register_defaults() -> None:
    register_op(OpSchema("conv2d", _normalize_conv2d, _infer_conv2d, _run_conv2d))
    register_op(OpSchema("fused_conv2d_bias_relu", _normalize_conv2d, _infer_conv2d, _run_fused_conv2d_bias_relu))
    register_op(OpSchema("fused_conv2d_bias_add_relu", _normalize_conv2d_residual, _infer_conv2d_residual,
                         _run_fused_conv2d_bias_add_relu))
    register_op(OpSchema("max_pool2d", _normalize_max_pool2d, _infer_max_pool2d, _run_max_pool2d))
    register_op(OpSchema("adaptive_avg_pool2d", _normalize_adaptive_avg_pool2d, _infer_adaptive_avg_pool2d,
                         _run_adaptive_avg_pool2d))
    register_op(OpSchema("bias_add", _normalize_binary("bias_add"), _infer_same, _run_bias_add))
    register_op(OpSchema("relu", _normalize_unary("relu"), _infer_same, _run_relu))
    register_op(OpSchema("fused_bias_relu", _normalize_binary("fused_bias_relu"), _infer_same, _run_fused_bias_relu))
    register_op(OpSchema("gelu", _normalize_unary("gelu"), _infer_same, _run_gelu))
    register_op(OpSchema("fused_bias_gelu", _normalize_binary("fused_bias_gelu"), _infer_same, _run_fused_bias_gelu))
    register_op(OpSchema("fused_conv2d_bias_gelu", _normalize_conv2d, _infer_conv2d, _run_fused_conv2d_bias_gelu))
    register_op(OpSchema("add", _normalize_binary("add"), _infer_broadcast, _binary_runner(torch.add)))
    register_op(OpSchema("sub", _normalize_binary("sub"), _infer_broadcast, _binary_runner(torch.sub)))
    register_op(OpSchema("mul", _normalize_binary("mul"), _infer_broadcast, _binary_runner(torch.mul)))


_register_defaults()

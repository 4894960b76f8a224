"""Host side of the conv2d hot path: same signatures, checks and exceptions as
the reference's ``flag_dnn.ops.conv2d`` (src/flag_dnn/ops/conv2d.py:3575-3611)
and ``fused_conv2d_bias_relu`` (src/flag_dnn/graph/kernels/fused_conv.py:62-130),
with the Triton launches replaced by calls into the C ABI
(include/flagdnn_b200.h).  There is no CPU fallback: CPU tensors raise
``NotImplementedError`` exactly as the reference does.
"""
from __future__ import annotations

import ctypes
import weakref
from collections import OrderedDict
from typing import Any, Optional, Sequence, Tuple, Union

import torch

from . import _native as nat

_DTYPE_IDS = {
    torch.float16: nat.F16,
    torch.bfloat16: nat.BF16,
    torch.float32: nat.F32,
    torch.float64: nat.F64,
}

# Packed filters are kept in a small LRU keyed on tensor identity and version,
# validated with a weak reference, like src/flag_dnn/ops/conv2d.py:24-32, 154-190.
_PACKED_WEIGHT_CACHE: "OrderedDict[tuple, tuple[weakref.ReferenceType, torch.Tensor]]" = OrderedDict()
_PACKED_WEIGHT_CACHE_MAX = 32

# Plans are pure functions of geometry, strides and pointer alignment.
_PLAN_CACHE: "OrderedDict[tuple, tuple[nat.ConvDesc, nat.ConvPlan]]" = OrderedDict()
_PLAN_CACHE_MAX = 256

_FORCED_ALGO = nat.ALGO_AUTO

# Scratch for reduction splitting on CTA pairs (include/flagdnn_b200.h, FDNN_STREAMK_FLAG_BYTES): one buffer per
# (device, stream), flags zeroed when it is created; every launch leaves them zero, and launches on one stream
# do not overlap, so the buffer is simply reused.
_STREAMK_SCRATCH: "dict[tuple, torch.Tensor]" = {}
_STREAM_K = False


def set_stream_k(enabled: bool) -> bool:
    """Switch reduction splitting on CTA pairs on or off for subsequent calls; returns the previous setting.
    Off (the default), every tile is computed whole by one pair, and an image's result does not depend on the
    batch it is computed in down to the last bit.  On, layers whose tiles do not fill whole rounds of the GPU's
    pairs share the reduction steps evenly; on B200 that measured no faster (the layers are bound by operand
    traffic from L2, which the split does not reduce), which is why it is off."""
    global _STREAM_K
    prev, _STREAM_K = _STREAM_K, bool(enabled)
    return prev


def _streamk_scratch(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    key = (device.index, stream)
    buf = _STREAMK_SCRATCH.get(key)
    if buf is not None and buf.numel() >= nbytes:
        return buf
    buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
    buf[: nat.STREAMK_FLAG_BYTES].zero_()
    if not torch.cuda.is_current_stream_capturing():
        # a buffer created during a stream capture belongs to that graph's memory pool and is zeroed by a node
        # of that graph on every replay: it serves that call only
        _STREAMK_SCRATCH[key] = buf
    return buf


_WORKSPACE: "OrderedDict[tuple, torch.Tensor]" = OrderedDict()
_WORKSPACE_KEEP_BYTES = 256 << 20
_WORKSPACE_KEEP_STREAMS = 8


def _workspace(device: torch.device, stream: int, nbytes: int) -> torch.Tensor:
    """Scratch for one call's relayouts.  Calls on one stream run in order, so they share one buffer per
    (device, stream) that grows to the largest request up to 256 MiB; larger requests, and requests made while
    the stream is being captured into a graph, get a buffer of their own from the caching allocator."""
    if torch.cuda.is_current_stream_capturing():
        # the graph keeps the address: the buffer must come from the graph's own memory pool
        return torch.empty(nbytes, dtype=torch.uint8, device=device)
    key = (device.index, stream)
    buf = _WORKSPACE.get(key)
    if buf is not None and buf.numel() >= nbytes:
        _WORKSPACE.move_to_end(key)
        return buf
    buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
    if nbytes <= _WORKSPACE_KEEP_BYTES:
        _WORKSPACE[key] = buf
        while len(_WORKSPACE) > _WORKSPACE_KEEP_STREAMS:   # the streams used longest ago give their buffers back
            _WORKSPACE.popitem(last=False)
    return buf


def set_algo(algo: Union[int, str]) -> int:
    """Force the kernel family for subsequent calls: "auto", "direct", "igemm"
    (one CTA per tile) or "pair" (CTA pairs).

    Returns the previous setting.  Meant for tests and benchmarks.
    """
    global _FORCED_ALGO
    names = {"auto": nat.ALGO_AUTO, "direct": nat.ALGO_DIRECT, "igemm": nat.ALGO_IGEMM,
             "pair": nat.ALGO_IGEMM_PAIR}
    prev = _FORCED_ALGO
    _FORCED_ALGO = names[algo] if isinstance(algo, str) else int(algo)
    return prev


def _pair(v: Union[int, Sequence[int]]) -> Tuple[int, int]:
    if isinstance(v, int):
        return v, v
    if len(v) != 2:
        raise RuntimeError(f"expected length 2, but got {v}")
    return int(v[0]), int(v[1])


def _conv_out_dim(size: int, pad_before: int, pad_after: int, dilation: int, kernel: int, stride: int) -> int:
    return (size + pad_before + pad_after - dilation * (kernel - 1) - 1) // stride + 1


def _normalize_padding(weight, stride, padding, dilation) -> Tuple[int, int, int, int]:
    """(top, bottom, left, right); rule of src/flag_dnn/ops/conv2d.py:65-87."""
    if isinstance(padding, str):
        if padding == "valid":
            return (0, 0, 0, 0)
        if padding == "same":
            if stride != (1, 1):
                raise RuntimeError("padding='same' is not supported for strided convolutions")
            kh, kw = weight.shape[2], weight.shape[3]
            pad_h = max(dilation[0] * (kh - 1), 0)
            pad_w = max(dilation[1] * (kw - 1), 0)
            return (pad_h // 2, pad_h - pad_h // 2, pad_w // 2, pad_w - pad_w // 2)
        raise RuntimeError("padding must be 'valid', 'same', int, or tuple")
    pad_h, pad_w = _pair(padding)
    return (pad_h, pad_h, pad_w, pad_w)


def _check_conv2d_inputs(input, weight, bias, stride, padding, dilation, groups) -> None:
    """Same checks and messages as src/flag_dnn/ops/conv2d.py:90-135."""
    if input.dim() != 4 or weight.dim() != 4:
        raise RuntimeError("flag_dnn conv2d expects 4D input and weight")
    if input.dtype not in _DTYPE_IDS:
        raise NotImplementedError(f"Unsupported dtype: {input.dtype}")
    if weight.dtype != input.dtype:
        raise RuntimeError("input and weight must have the same dtype")
    if input.device != weight.device:
        raise RuntimeError("input and weight must be on the same device")
    if bias is not None:
        if bias.dtype != input.dtype:
            raise RuntimeError("bias must have the same dtype as input")
        if bias.device != input.device:
            raise RuntimeError("bias must be on the same device as input")
    if groups <= 0:
        raise RuntimeError("groups must be a positive integer")
    if stride[0] <= 0 or stride[1] <= 0:
        raise RuntimeError("stride must be positive")
    if dilation[0] <= 0 or dilation[1] <= 0:
        raise RuntimeError("dilation must be positive")
    if min(padding) < 0:
        raise RuntimeError("negative padding is not supported")
    c_in = input.shape[1]
    c_out, c_per_group = weight.shape[0], weight.shape[1]
    if c_in % groups != 0 or c_out % groups != 0:
        raise RuntimeError("channels must be divisible by groups")
    if c_per_group != c_in // groups:
        raise RuntimeError("weight.shape[1] must match input_channels // groups")
    if bias is not None and (bias.dim() != 1 or bias.numel() != c_out):
        raise RuntimeError(f"bias shape mismatch, expected ({c_out},)")


def _current_stream(device: torch.device) -> int:
    """The raw handle of torch's current stream on `device` (the accessor the stream object is built from;
    an order of magnitude cheaper than building the object on every call)."""
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None and device.index is not None:
        return raw(device.index)
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t: torch.Tensor) -> int:
    return 0 if t.device.type == "meta" else t.data_ptr()


def _plan_for(input, weight, out, stride, padding4, dilation, groups, algo):
    key = (
        input.dtype, tuple(input.shape), tuple(input.stride()), tuple(weight.shape), tuple(weight.stride()),
        tuple(out.stride()), stride, padding4, dilation, groups, algo,
        _ptr(input) % 16, _ptr(weight) % 16, _ptr(out) % 16,
    )
    hit = _PLAN_CACHE.get(key)
    if hit is not None:
        _PLAN_CACHE.move_to_end(key)
        return hit
    lib = nat.load()
    d = nat.ConvDesc()
    d.dtype = _DTYPE_IDS[input.dtype]
    d.n, d.c, d.h, d.w = input.shape
    d.k, _, d.r, d.s = weight.shape
    d.stride_h, d.stride_w = stride
    d.pad_top, d.pad_bottom, d.pad_left, d.pad_right = padding4
    d.dil_h, d.dil_w = dilation
    d.groups = groups
    d.algo = algo
    for i in range(4):
        d.x_strides[i] = input.stride(i)
        d.w_strides[i] = weight.stride(i)
        d.y_strides[i] = out.stride(i)
    plan = nat.ConvPlan()
    nat.check(lib.fdnn_conv2d_query(ctypes.byref(d), _ptr(input) or None, _ptr(weight) or None,
                                    _ptr(out) or None, ctypes.byref(plan)))
    _PLAN_CACHE[key] = (d, plan)
    while len(_PLAN_CACHE) > _PLAN_CACHE_MAX:
        _PLAN_CACHE.popitem(last=False)
    return d, plan


def _packed_weight(weight: torch.Tensor, d: nat.ConvDesc, plan: nat.ConvPlan, stream: int, y_ptr: int) -> torch.Tensor:
    version = int(getattr(weight, "_version", 0))
    # the packed layout depends on the plan: generic [K,R,S,Cpad] or the low-channel quad layout
    if plan.pixel_group > 1:
        layout = ("grouped", plan.pixel_group, d.stride_w)
    elif plan.low_channel:
        layout = ("lowc", plan.low_channel, d.stride_w)
    else:
        layout = ("krsc", plan.c_padded)
    key = (layout, id(weight), weight.data_ptr(), tuple(weight.shape), tuple(weight.stride()),
           str(weight.dtype), weight.device.type, weight.device.index, version)
    entry = _PACKED_WEIGHT_CACHE.get(key)
    if entry is not None:
        owner_ref, value = entry
        if owner_ref() is weight:
            _PACKED_WEIGHT_CACHE.move_to_end(key)
            return value
        del _PACKED_WEIGHT_CACHE[key]
    packed = torch.empty(plan.packed_weight_bytes, dtype=torch.uint8, device=weight.device)
    # y_ptr: only its alignment matters (it selects the plan, and with it the packed layout, as in _plan_for)
    nat.check(nat.load().fdnn_conv2d_pack_weight(ctypes.byref(d), weight.data_ptr(), y_ptr, packed.data_ptr(),
                                                 plan.packed_weight_bytes, stream))
    _PACKED_WEIGHT_CACHE[key] = (weakref.ref(weight), packed)
    while len(_PACKED_WEIGHT_CACHE) > _PACKED_WEIGHT_CACHE_MAX:
        _PACKED_WEIGHT_CACHE.popitem(last=False)
    return packed


def conv2d_plan(input, weight, stride=1, padding=0, dilation=1, groups=1, algo=None) -> dict:
    """What the library would do for this call (kernel family, tile, scratch sizes)."""
    stride = _pair(stride)
    dilation = _pair(dilation)
    padding4 = _normalize_padding(weight, stride, padding, dilation)
    n, _, h, w = input.shape
    c_out, _, kh, kw = weight.shape
    oh = max(_conv_out_dim(h, padding4[0], padding4[1], dilation[0], kh, stride[0]), 0)
    ow = max(_conv_out_dim(w, padding4[2], padding4[3], dilation[1], kw, stride[1]), 0)
    out = _empty_output(input, n, c_out, oh, ow, meta=True)
    _, plan = _plan_for(input, weight, out, stride, padding4, dilation, groups,
                        (_FORCED_ALGO if algo is None else algo) | (nat.ALGO_FLAG_STREAM_K if _STREAM_K else 0))
    return plan.as_dict()


_ACTIVATIONS = {"none": nat.ACT_NONE, "relu": nat.ACT_RELU, "gelu": nat.ACT_GELU, "gelu_tanh": nat.ACT_GELU_TANH}


def _empty_output(input, n, c_out, oh, ow, meta=False):
    # channels_last output iff the input has unit channel stride
    # (src/flag_dnn/ops/conv2d.py:3729-3738, fused_conv.py:120-130); fp64 always
    # produces a contiguous NCHW tensor (conv2d.py:3631-3633).
    use_cl = input.dim() == 4 and input.stride(1) == 1 and input.dtype != torch.float64
    return torch.empty(
        (n, c_out, oh, ow),
        device="meta" if meta else input.device,
        dtype=input.dtype,
        memory_format=torch.channels_last if use_cl else torch.contiguous_format,
    )


def _run(input, weight, bias, scale, stride, padding4, dilation, groups, activation, residual=None,
         out=None, out_f32=False) -> torch.Tensor:
    n, _, h, w = input.shape
    c_out, _, kh, kw = weight.shape
    oh = _conv_out_dim(h, padding4[0], padding4[1], dilation[0], kh, stride[0])
    ow = _conv_out_dim(w, padding4[2], padding4[3], dilation[1], kw, stride[1])
    if oh < 0 or ow < 0:
        raise RuntimeError("computed output size is negative")
    if oh == 0 or ow == 0:
        return torch.empty((n, c_out, max(oh, 0), max(ow, 0)), device=input.device, dtype=input.dtype)
    if bias is not None and not bias.is_contiguous():
        bias = bias.contiguous()
    if scale is not None and not scale.is_contiguous():
        scale = scale.contiguous()
    lib = nat.load()
    with torch.cuda.device(input.device):
        if out is None:
            out = _empty_output(input, n, c_out, oh, ow)
        elif (tuple(out.shape) != (n, c_out, oh, ow) or out.device != input.device
              or out.dtype != (torch.float32 if out_f32 else input.dtype)):
            raise RuntimeError(f"out must be a {torch.float32 if out_f32 else input.dtype} tensor of shape "
                               f"{(n, c_out, oh, ow)} on {input.device}")
        if n == 0:
            return out
        if residual is not None:
            if residual.shape != out.shape or residual.dtype != out.dtype or residual.device != out.device:
                raise RuntimeError("residual must have the shape, dtype and device of the convolution's output")
            fusable = (residual.stride() == out.stride() and residual.data_ptr() % 16 == out.data_ptr() % 16)
        # a float32 result from 16-bit operands has one kernel family (the request for another is dropped)
        algo = nat.ALGO_FLAG_OUT_F32 if out_f32 else (_FORCED_ALGO | (nat.ALGO_FLAG_STREAM_K if _STREAM_K else 0))
        d, plan = _plan_for(input, weight, out, stride, padding4, dilation, groups, algo)
        stream = _current_stream(input.device)
        packed_ptr = None
        packed = None
        if plan.algo != nat.ALGO_DIRECT and plan.w_packed:
            packed = _packed_weight(weight, d, plan, stream, out.data_ptr())
            packed_ptr = packed.data_ptr()
        ws_ptr = None
        ws = None
        if plan.workspace_bytes > 0:
            ws = _workspace(input.device, stream, plan.workspace_bytes)
            ws_ptr = ws.data_ptr()
        sk_ptr, sk_bytes = None, 0
        if plan.stream_k:
            sk = _streamk_scratch(input.device, stream, plan.streamk_bytes)
            sk_ptr, sk_bytes = sk.data_ptr(), sk.numel()
        fused_residual = residual is not None and fusable and not plan.low_channel
        nat.check(lib.fdnn_conv2d_fwd_ex(
            ctypes.byref(d), input.data_ptr(), weight.data_ptr(), packed_ptr,
            None if bias is None else bias.data_ptr(),
            None if scale is None else scale.data_ptr(),
            residual.data_ptr() if fused_residual else None,
            activation if (residual is None or fused_residual) else nat.ACT_NONE,
            out.data_ptr(), ws_ptr, plan.workspace_bytes, sk_ptr, sk_bytes, stream))
        if fused_residual:
            return out
        if residual is not None:
            # the residual's layout differs from the output's (or the low-channel path ran): the add
            # and the activation follow as device-side elementwise steps
            out.add_(residual)
            if activation == nat.ACT_RELU:
                out.relu_()
            elif activation in (nat.ACT_GELU, nat.ACT_GELU_TANH):
                out.copy_(torch.nn.functional.gelu(out, approximate="tanh" if activation == nat.ACT_GELU_TANH else "none"))
        # `ws` goes back to torch's caching allocator when this frame ends; the
        # allocator orders reuse on the stream the kernels were queued on.
    return out


def conv2d(
    input: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    stride: Union[int, Tuple[int, int]] = 1,
    padding: Union[str, int, Tuple[int, int]] = 0,
    dilation: Union[int, Tuple[int, int]] = 1,
    groups: int = 1,
    *,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Drop-in for ``flag_dnn.ops.conv2d`` (src/flag_dnn/ops/conv2d.py:3575).  ``out`` (not in the
    reference) receives the result: any strides, the output's shape and the input's dtype."""
    stride = _pair(stride)
    dilation = _pair(dilation)
    padding4 = _normalize_padding(weight, stride, padding, dilation)
    _check_conv2d_inputs(input, weight, bias, stride, padding4, dilation, groups)
    if not input.is_cuda:
        raise NotImplementedError("flag_dnn conv2d CUDA implementation requires CUDA input")
    return _run(input, weight, bias, None, stride, padding4, dilation, groups, nat.ACT_NONE, out=out)


def fused_conv2d_bias_relu(
    input: torch.Tensor,
    weight: torch.Tensor,
    bias: torch.Tensor,
    *,
    stride: Union[int, Tuple[int, int]] = 1,
    padding: Union[str, int, Tuple[int, int]] = 0,
    dilation: Union[int, Tuple[int, int]] = 1,
    groups: int = 1,
    config: Optional[dict[str, Any]] = None,
    scale: Optional[torch.Tensor] = None,
    activation: str = "relu",
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Drop-in for the reference's fused op (src/flag_dnn/graph/kernels/fused_conv.py:62-72).

    ``config`` (the reference's Triton tile override) is accepted and ignored.
    Two additions the reference's callers never pass: ``scale`` (BN-folded
    per-channel multiplier applied before the bias) and ``activation`` ("relu",
    "none", "gelu" or "gelu_tanh").
    """
    del config
    if not (isinstance(input, torch.Tensor) and input.is_cuda):
        raise NotImplementedError("fused_conv2d_bias_relu requires runtime device input")
    if groups != 1:
        raise NotImplementedError("fused_conv2d_bias_relu currently supports groups=1")
    if input.dim() != 4 or weight.dim() != 4 or bias.dim() != 1:
        raise RuntimeError("fused_conv2d_bias_relu expects 4D input/weight and 1D bias")
    if input.dtype != weight.dtype or input.dtype != bias.dtype:
        raise RuntimeError("input, weight, and bias must have the same dtype")
    if input.dtype not in (torch.float16, torch.bfloat16, torch.float32):
        raise NotImplementedError(f"fused_conv2d_bias_relu does not support dtype={input.dtype}")
    if input.device != weight.device or input.device != bias.device:
        raise RuntimeError("input, weight, and bias must be on the same device")
    if scale is not None and (scale.dtype != input.dtype or scale.device != input.device or scale.dim() != 1):
        raise RuntimeError("scale must be a 1D tensor with the dtype and device of input")
    if activation not in _ACTIVATIONS:
        raise NotImplementedError(f"unsupported activation {activation!r}")
    stride = _pair(stride)
    dilation = _pair(dilation)
    padding4 = _normalize_padding(weight, stride, padding, dilation)
    c_in = input.shape[1]
    c_out, c_per_group = weight.shape[0], weight.shape[1]
    if c_per_group != c_in:
        raise RuntimeError("weight.shape[1] must match input channels for groups=1")
    if bias.numel() != c_out:
        raise RuntimeError(f"bias shape mismatch, expected ({c_out},)")
    if scale is not None and scale.numel() != c_out:
        raise RuntimeError(f"scale shape mismatch, expected ({c_out},)")
    return _run(input, weight, bias, scale, stride, padding4, dilation, 1, _ACTIVATIONS[activation], out=out)


def conv2d_bias_act(
    input: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    *,
    stride: Union[int, Tuple[int, int]] = 1,
    padding: Union[str, int, Tuple[int, int]] = 0,
    dilation: Union[int, Tuple[int, int]] = 1,
    groups: int = 1,
    scale: Optional[torch.Tensor] = None,
    relu: bool = False,
    residual: Optional[torch.Tensor] = None,
    activation: Optional[str] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """conv2d with the full epilogue (scale, bias, residual add, ReLU) and conv2d's
    argument range (any groups, fp64): ``act(conv(x, w) * scale + bias + residual)``
    computed in fp32 and rounded once.  The graph executor uses it for fused nodes
    that fall outside ``fused_conv2d_bias_relu``'s contract and for a block's last
    convolution with its shortcut add (``residual`` has the output's shape; when it
    also has the output's strides the add happens in the kernel's epilogue)."""
    stride = _pair(stride)
    dilation = _pair(dilation)
    padding4 = _normalize_padding(weight, stride, padding, dilation)
    _check_conv2d_inputs(input, weight, bias, stride, padding4, dilation, groups)
    if not input.is_cuda:
        raise NotImplementedError("flag_dnn conv2d CUDA implementation requires CUDA input")
    if scale is not None and (scale.dtype != input.dtype or scale.device != input.device
                              or scale.dim() != 1 or scale.numel() != weight.shape[0]):
        raise RuntimeError("scale must be a 1D tensor of length C_out with the dtype and device of input")
    if activation is None:
        activation = "relu" if relu else "none"
    if activation not in _ACTIVATIONS:
        raise NotImplementedError(f"unsupported activation {activation!r}")
    return _run(input, weight, bias, scale, stride, padding4, dilation, groups, _ACTIVATIONS[activation], residual,
                out=out)


def conv1d(
    input: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    stride: Union[int, Tuple[int]] = 1,
    padding: Union[str, int, Tuple[int]] = 0,
    dilation: Union[int, Tuple[int]] = 1,
    groups: int = 1,
) -> torch.Tensor:
    """Drop-in for ``flag_dnn.ops.conv1d`` (src/flag_dnn/ops/conv1d.py:416): a convolution over
    [N, C, L] (or unbatched [C, L]) is the 2-D path with H = R = 1, so it runs on the same kernels.
    Checks and messages follow src/flag_dnn/ops/conv1d.py:21-66, 90-150, 436-446."""
    def single(v, name):
        if isinstance(v, int):
            return int(v)
        if len(v) != 1:
            raise RuntimeError(f"{name} must be an int or a length-1 tuple")
        return int(v[0])

    stride_w = single(stride, "stride")
    dilation_w = single(dilation, "dilation")
    if input.dim() not in (2, 3) or weight.dim() != 3:
        raise RuntimeError("flag_dnn conv1d expects 2D/3D input and 3D weight")
    if not input.is_cuda:
        raise NotImplementedError("flag_dnn conv1d only supports CUDA input")
    if weight.device != input.device:
        raise RuntimeError("input and weight must be on the same device")
    if bias is not None and bias.device != input.device:
        raise RuntimeError("input and bias must be on the same device")
    if input.dtype not in _DTYPE_IDS:
        raise NotImplementedError(f"Unsupported dtype: {input.dtype}")
    if weight.dtype != input.dtype:
        raise RuntimeError("input and weight must have the same dtype")
    if bias is not None and bias.dtype != input.dtype:
        raise RuntimeError("input and bias must have the same dtype")
    if any(t is not None and t.requires_grad for t in (input, weight, bias)) and torch.is_grad_enabled():
        raise NotImplementedError("flag_dnn conv1d is forward-only")
    if groups <= 0:
        raise RuntimeError("groups must be a positive integer")
    if stride_w <= 0:
        raise RuntimeError("stride must be positive")
    if dilation_w <= 0:
        raise RuntimeError("dilation must be positive")
    kw = weight.shape[2]
    if isinstance(padding, str):
        if padding == "valid":
            pad_left = pad_right = 0
        elif padding == "same":
            if stride_w != 1:
                raise RuntimeError("padding='same' is not supported for strided convolutions")
            total = max(dilation_w * (kw - 1), 0)
            pad_left, pad_right = total // 2, total - total // 2
        else:
            raise RuntimeError("padding must be 'valid', 'same', int, or tuple")
    else:
        pad_left = pad_right = single(padding, "padding")
        if pad_left < 0:
            raise RuntimeError("negative padding is not supported")
    batched = input.dim() == 3
    c_in, length = input.shape[-2], input.shape[-1]
    c_out, c_per_group = weight.shape[0], weight.shape[1]
    if c_in <= 0 or c_out <= 0 or c_per_group <= 0 or kw <= 0:
        raise RuntimeError("input and weight dimensions must be non-empty")
    if c_in % groups != 0 or c_out % groups != 0:
        raise RuntimeError("channels must be divisible by groups")
    if c_per_group != c_in // groups:
        raise RuntimeError("weight.shape[1] must match input_channels // groups")
    if bias is not None and (bias.dim() != 1 or bias.numel() != c_out):
        raise RuntimeError(f"bias shape mismatch, expected ({c_out},)")
    if length + pad_left + pad_right < dilation_w * (kw - 1) + 1:
        raise RuntimeError("kernel size can't be greater than input size")
    if _conv_out_dim(length, pad_left, pad_right, dilation_w, kw, stride_w) <= 0:
        raise RuntimeError("computed output size is not positive")
    x4 = (input if batched else input.unsqueeze(0)).unsqueeze(2)   # [N, C, 1, L]
    w4 = weight.unsqueeze(2)                                        # [K, C/g, 1, S]
    y4 = _run(x4, w4, bias, None, (1, stride_w), (0, 0, pad_left, pad_right), (1, dilation_w), groups, nat.ACT_NONE)
    y = y4.squeeze(2)
    return y if batched else y.squeeze(0)


def device_status() -> int:
    """Synchronise the current device and return its incident word (0 = clean)."""
    word = ctypes.c_uint32(0)
    lib = nat.load()
    status = lib.fdnn_device_status(ctypes.byref(word))
    if status not in (nat.FDNN_OK, nat.FDNN_DEVICE_TIMEOUT):
        nat.check(status)
    return int(word.value)


def mm(
    input: torch.Tensor,
    mat2: torch.Tensor,
    out_dtype: Optional[torch.dtype] = None,
    *,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Drop-in for ``flag_dnn.ops.mm`` (src/flag_dnn/ops/mm.py:336) on real tensors: ``input @ mat2`` is a
    1x1 convolution over a row of M pixels with K channels whose filter is ``mat2`` transposed, so it runs
    on the same kernels (fp64 on the direct one).  Checks and messages follow src/flag_dnn/ops/mm.py:100-140,
    the ``out`` handling src/flag_dnn/ops/mm.py:153-181.  ``out_dtype=torch.float32`` with fp16 / bf16 operands
    stores the fp32 accumulators unrounded.  Complex tensors are not implemented on this path."""
    if input.dim() != 2:
        raise RuntimeError("self must be a matrix")
    if mat2.dim() != 2:
        raise RuntimeError("mat2 must be a matrix")
    if input.shape[1] != mat2.shape[0]:
        raise RuntimeError("mat1 and mat2 shapes cannot be multiplied "
                           f"({input.shape[0]}x{input.shape[1]} and {mat2.shape[0]}x{mat2.shape[1]})")
    if input.device != mat2.device:
        raise RuntimeError(f"mm: input and mat2 must be on the same device, but got {input.device} and {mat2.device}")
    if input.dtype != mat2.dtype:
        raise RuntimeError(f"expected mat1 and mat2 to have the same dtype, but got: {input.dtype} != {mat2.dtype}")
    if input.layout != torch.strided or mat2.layout != torch.strided:
        raise NotImplementedError("flag_dnn mm supports dense strided tensors only")
    if input.dtype in (torch.complex64, torch.complex128):
        raise NotImplementedError("flag_dnn mm: complex tensors are not implemented on the convolution kernels")
    if input.dtype not in (torch.float16, torch.bfloat16, torch.float32, torch.float64):
        raise NotImplementedError(f"flag_dnn mm does not support dtype={input.dtype}")
    wide = False
    if out_dtype is not None and out_dtype != input.dtype:
        if not (input.dtype in (torch.float16, torch.bfloat16) and out_dtype == torch.float32):
            raise RuntimeError("out_dtype must be the same as input dtype or fp32 for fp16/bf16 inputs")
        wide = True
    y_dtype = torch.float32 if wide else input.dtype
    if not input.is_cuda:
        raise NotImplementedError("flag_dnn mm CUDA implementation requires CUDA input")
    m, k = input.shape
    n = mat2.shape[1]
    if out is not None:
        if out.device != input.device:
            raise RuntimeError(f"mm out tensor device mismatch: expected {input.device}, got {out.device}")
        if out.dtype != y_dtype:
            raise RuntimeError(f"Expected out tensor to have dtype {y_dtype}, but got {out.dtype} instead")
        if out.dim() != 2 or tuple(out.shape) != (m, n):
            out.resize_((m, n))
    y = out if out is not None and out.is_contiguous() else torch.empty((m, n), dtype=y_dtype, device=input.device)
    if y.numel() > 0:
        if k == 0:
            y.zero_()
        else:
            # one image of one row of M pixels with K channels (row m of `input` is pixel m), so that a tile's
            # 128 GEMM rows are 128 neighbouring pixels of a row; the result [1, N, 1, M] is y transposed
            x4 = input.t().unsqueeze(0).unsqueeze(2)               # [1, K, 1, M]
            w4 = mat2.t().unsqueeze(-1).unsqueeze(-1)              # [N, K, 1, 1]: the filter is mat2 transposed
            _run(x4, w4, None, None, (1, 1), (0, 0, 0, 0), (1, 1), 1, nat.ACT_NONE,
                 out=y.t().unsqueeze(0).unsqueeze(2), out_f32=wide)   # [1, N, 1, M] over y's memory
    if out is not None and y is not out:
        out.copy_(y)
        return out
    return y

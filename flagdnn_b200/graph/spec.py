"""Static tensor descriptions and the symbolic tensor handed to captured
functions.  Field names and methods follow the reference's ``TensorSpec`` /
``GraphTensor`` (src/flag_dnn/graph/tensor.py:113-299) so user code and tests
written against it keep working."""
from __future__ import annotations

from dataclasses import dataclass, replace
from functools import reduce
from operator import mul
from typing import Any, Optional, Tuple

import torch

_DTYPE_NAMES = {
    torch.float16: "float16", torch.bfloat16: "bfloat16", torch.float32: "float32",
    torch.float64: "float64", torch.int32: "int32", torch.int64: "int64", torch.bool: "bool",
    torch.int8: "int8", torch.uint8: "uint8", torch.int16: "int16",
}
_NAME_TO_DTYPE = {v: k for k, v in _DTYPE_NAMES.items()}
_ALIASES = {"half": "float16", "fp16": "float16", "bf16": "bfloat16", "float": "float32",
            "fp32": "float32", "double": "float64", "fp64": "float64"}


def canonical_dtype(dtype: Any) -> str:
    if isinstance(dtype, torch.dtype):
        return _DTYPE_NAMES.get(dtype, str(dtype).replace("torch.", ""))
    name = str(dtype).replace("torch.", "").lower()
    return _ALIASES.get(name, name)


def torch_dtype(name: str) -> torch.dtype:
    return _NAME_TO_DTYPE[canonical_dtype(name)]


def dtype_itemsize(name: str) -> int:
    return torch.empty((), dtype=torch_dtype(name)).element_size()


def infer_layout(tensor: torch.Tensor) -> str:
    if tensor.dim() == 4 and tensor.is_contiguous(memory_format=torch.channels_last):
        return "nhwc"
    return "contiguous" if tensor.is_contiguous() else "strided"


def contiguous_strides(shape: Tuple[int, ...]) -> Tuple[int, ...]:
    out, acc = [], 1
    for dim in reversed(shape):
        out.append(acc)
        acc *= max(int(dim), 1)
    return tuple(reversed(out))


def channels_last_strides(shape: Tuple[int, ...]) -> Tuple[int, ...]:
    n, c, h, w = shape
    return (h * w * c, 1, w * c, c)


@dataclass(frozen=True)
class TensorSpec:
    name: str
    shape: Tuple[int, ...]
    dtype: str
    stride: Optional[Tuple[int, ...]] = None
    layout: Optional[str] = None
    device: Optional[str] = None
    is_input: bool = False
    is_output: bool = False
    contiguous: Optional[bool] = None

    def __post_init__(self) -> None:
        object.__setattr__(self, "shape", tuple(int(d) for d in self.shape))
        object.__setattr__(self, "dtype", canonical_dtype(self.dtype))
        if self.stride is not None:
            object.__setattr__(self, "stride", tuple(int(s) for s in self.stride))
        if self.device is not None:
            object.__setattr__(self, "device", str(self.device))

    @classmethod
    def from_tensor(cls, tensor: torch.Tensor, name: str = "") -> "TensorSpec":
        return cls(name=name, shape=tuple(tensor.shape), dtype=tensor.dtype, stride=tuple(tensor.stride()),
                   layout=infer_layout(tensor), device=tensor.device, contiguous=tensor.is_contiguous())

    def with_name(self, name: str) -> "TensorSpec":
        return replace(self, name=name)

    def as_input(self) -> "TensorSpec":
        return replace(self, is_input=True)

    def as_output(self) -> "TensorSpec":
        return replace(self, is_output=True)

    def numel(self) -> int:
        return reduce(mul, self.shape, 1)

    def nbytes(self) -> int:
        return self.numel() * dtype_itemsize(self.dtype)

    def signature(self) -> dict:
        return {"shape": tuple(self.shape), "dtype": self.dtype, "stride": self.stride,
                "layout": self.layout, "device": self.device, "contiguous": self.contiguous}


class GraphTensor:
    """Symbolic value seen by a function while it is being captured."""

    def __init__(self, value_id: int, graph: Any):
        self.value_id = value_id
        self.graph = graph

    @property
    def spec(self) -> TensorSpec:
        return self.graph.values[self.value_id].spec

    @property
    def shape(self):
        return self.spec.shape

    @property
    def dtype(self) -> str:
        return self.spec.dtype

    @property
    def device(self):
        return self.spec.device

    def dim(self) -> int:
        return len(self.spec.shape)

    def numel(self) -> int:
        return self.spec.numel()

    def _binary(self, op_type: str, other: Any, reverse: bool = False):
        from .compiler import current_capture

        ctx = current_capture()
        if ctx is None:
            raise RuntimeError("GraphTensor operation used outside capture")
        return ctx.add_binary_op(op_type, self, other, reverse=reverse)

    def __add__(self, other):
        return self._binary("add", other)

    def __radd__(self, other):
        return self._binary("add", other, reverse=True)

    def __sub__(self, other):
        return self._binary("sub", other)

    def __rsub__(self, other):
        return self._binary("sub", other, reverse=True)

    def __mul__(self, other):
        return self._binary("mul", other)

    def __rmul__(self, other):
        return self._binary("mul", other, reverse=True)

    def __repr__(self) -> str:
        return f"GraphTensor(value_id={self.value_id}, shape={self.spec.shape}, dtype={self.spec.dtype})"

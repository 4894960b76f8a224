"""ctypes binding of the C ABI declared in include/flagdnn_b200.h.

The library is loaded from this package directory.  There is no fallback: if
the library is missing, or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
from pathlib import Path
from typing import Optional

_PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = _PKG_DIR / "libflagdnn_b200.so"

FDNN_OK = 0
FDNN_BAD_PARAM = 1
FDNN_NOT_SUPPORTED = 2
FDNN_ARCH_MISMATCH = 3
FDNN_WORKSPACE_TOO_SMALL = 4
FDNN_CUDA_ERROR = 5
FDNN_DEVICE_TIMEOUT = 6

F16, BF16, F32, F64 = 0, 1, 2, 3
ALGO_AUTO, ALGO_DIRECT, ALGO_IGEMM, ALGO_IGEMM_PAIR = 0, 1, 2, 3
ACT_NONE, ACT_RELU, ACT_GELU, ACT_GELU_TANH = 0, 1, 2, 3
STREAMK_FLAG_BYTES = 8192
ALGO_FLAG_STREAM_K = 0x100
ALGO_FLAG_OUT_F32 = 0x200
ALGO_FLAG_TILE_N_64 = 0x400
ALGO_FLAG_TILE_N_128 = 0x800
ALGO_FLAG_TILE_N_256 = 0xC00
ALGO_FLAG_NO_PIXEL_GROUP = 0x1000

EXPORTED_SYMBOLS = (
    "fdnn_abi_version",
    "fdnn_status_string",
    "fdnn_last_error",
    "fdnn_conv2d_query",
    "fdnn_conv2d_pack_weight",
    "fdnn_conv2d_fwd",
    "fdnn_conv2d_fwd_residual",
    "fdnn_conv2d_fwd_ex",
    "fdnn_max_pool2d_fwd",
    "fdnn_adaptive_avg_pool2d_fwd",
    "fdnn_conv2d_fwd_host",
    "fdnn_conv2d_host_arena_bytes",
    "fdnn_device_status",
    "fdnn_debug_set_profile_buffer",
    "fdnn_debug_set_wait_limit",
    "fdnn_debug_tensor_map_counters",
    "fdnn_conv2d_fwd_static_scratch",
    "fdnn_static_scratch_bytes",
    "fdnn_static_scratch_last_error",
)


class ConvDesc(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32),
        ("n", ctypes.c_int32), ("c", ctypes.c_int32), ("h", ctypes.c_int32), ("w", ctypes.c_int32),
        ("k", ctypes.c_int32), ("r", ctypes.c_int32), ("s", ctypes.c_int32),
        ("stride_h", ctypes.c_int32), ("stride_w", ctypes.c_int32),
        ("pad_top", ctypes.c_int32), ("pad_bottom", ctypes.c_int32),
        ("pad_left", ctypes.c_int32), ("pad_right", ctypes.c_int32),
        ("dil_h", ctypes.c_int32), ("dil_w", ctypes.c_int32),
        ("groups", ctypes.c_int32),
        ("algo", ctypes.c_int32),
        ("x_strides", ctypes.c_int64 * 4),
        ("w_strides", ctypes.c_int64 * 4),
        ("y_strides", ctypes.c_int64 * 4),
    ]


class ConvPlan(ctypes.Structure):
    _fields_ = [
        ("algo", ctypes.c_int32),
        ("oh", ctypes.c_int32), ("ow", ctypes.c_int32),
        ("tile_m", ctypes.c_int32), ("tile_n", ctypes.c_int32), ("tile_k", ctypes.c_int32),
        ("stages", ctypes.c_int32),
        ("x_repacked", ctypes.c_int32),
        ("w_packed", ctypes.c_int32),
        ("c_padded", ctypes.c_int32),
        ("grid", ctypes.c_int32), ("block", ctypes.c_int32),
        ("launches", ctypes.c_int32),
        ("low_channel", ctypes.c_int32),
        ("pixel_group", ctypes.c_int32),
        ("stream_k", ctypes.c_int32),
        ("workspace_bytes", ctypes.c_int64),
        ("streamk_bytes", ctypes.c_int64),
        ("packed_weight_bytes", ctypes.c_int64),
        ("smem_bytes", ctypes.c_int64),
        ("flops", ctypes.c_double),
        ("bytes", ctypes.c_double),
    ]

    def as_dict(self) -> dict:
        return {name: getattr(self, name) for name, _ in self._fields_}


class PoolDesc(ctypes.Structure):
    _fields_ = [(name, ctypes.c_int32) for name in
                ("dtype", "n", "c", "h", "w", "oh", "ow", "kernel_h", "kernel_w", "stride_h", "stride_w",
                 "pad_h", "pad_w", "dil_h", "dil_w")] + \
               [("x_strides", ctypes.c_int64 * 4), ("y_strides", ctypes.c_int64 * 4)]


class NativeError(RuntimeError):
    """A non-OK status that maps to RuntimeError in the reference's convention."""


_lib: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    """Load libflagdnn_b200.so (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m flagdnn_b200.build` "
            "(there is no CPU or Triton fallback for this path)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    lib.fdnn_abi_version.restype = i32
    lib.fdnn_status_string.restype = ctypes.c_char_p
    lib.fdnn_status_string.argtypes = [i32]
    lib.fdnn_last_error.restype = ctypes.c_char_p
    lib.fdnn_conv2d_query.restype = i32
    lib.fdnn_conv2d_query.argtypes = [ctypes.POINTER(ConvDesc), vp, vp, vp, ctypes.POINTER(ConvPlan)]
    lib.fdnn_conv2d_pack_weight.restype = i32
    lib.fdnn_conv2d_pack_weight.argtypes = [ctypes.POINTER(ConvDesc), vp, vp, vp, i64, vp]
    lib.fdnn_conv2d_fwd.restype = i32
    lib.fdnn_conv2d_fwd.argtypes = [ctypes.POINTER(ConvDesc), vp, vp, vp, vp, vp, i32, vp, vp, i64, vp]
    lib.fdnn_max_pool2d_fwd.restype = i32
    lib.fdnn_max_pool2d_fwd.argtypes = [ctypes.POINTER(PoolDesc), vp, vp, vp, vp]
    lib.fdnn_adaptive_avg_pool2d_fwd.restype = i32
    lib.fdnn_adaptive_avg_pool2d_fwd.argtypes = [ctypes.POINTER(PoolDesc), vp, vp, vp]
    lib.fdnn_conv2d_fwd_residual.restype = i32
    lib.fdnn_conv2d_fwd_residual.argtypes = [ctypes.POINTER(ConvDesc), vp, vp, vp, vp, vp, vp, i32, vp, vp, i64, vp]
    lib.fdnn_conv2d_fwd_ex.restype = i32
    lib.fdnn_conv2d_fwd_ex.argtypes = [ctypes.POINTER(ConvDesc), vp, vp, vp, vp, vp, vp, i32, vp, vp, i64, vp, i64, vp]
    lib.fdnn_conv2d_fwd_host.restype = i32
    lib.fdnn_conv2d_fwd_host.argtypes = [ctypes.POINTER(ConvDesc), vp, vp, vp, vp, i32, vp, vp, i64, vp]
    lib.fdnn_conv2d_host_arena_bytes.restype = i32
    lib.fdnn_conv2d_host_arena_bytes.argtypes = [ctypes.POINTER(ConvDesc), ctypes.POINTER(i64)]
    lib.fdnn_conv2d_fwd_static_scratch.restype = i32
    lib.fdnn_conv2d_fwd_static_scratch.argtypes = [ctypes.POINTER(ConvDesc), vp, vp, vp, vp, vp, i32, vp, vp]
    lib.fdnn_static_scratch_bytes.restype = i64
    lib.fdnn_static_scratch_last_error.restype = ctypes.c_char_p
    lib.fdnn_debug_set_profile_buffer.restype = i32
    lib.fdnn_debug_set_profile_buffer.argtypes = [vp]
    lib.fdnn_debug_set_wait_limit.restype = i32
    lib.fdnn_debug_set_wait_limit.argtypes = [i64, i32]
    lib.fdnn_debug_tensor_map_counters.restype = i32
    lib.fdnn_debug_tensor_map_counters.argtypes = [ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]
    lib.fdnn_device_status.restype = i32
    lib.fdnn_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint32)]
    _lib = lib
    return lib


def check(status: int) -> None:
    """Translate a status code into the exception the reference would raise."""
    if status == FDNN_OK:
        return
    lib = load()
    detail = lib.fdnn_last_error().decode("utf-8", "replace")
    text = lib.fdnn_status_string(status).decode()
    msg = f"{detail} [{text}]" if detail else text
    if status in (FDNN_NOT_SUPPORTED, FDNN_ARCH_MISMATCH):
        raise NotImplementedError(msg)
    raise NativeError(msg)

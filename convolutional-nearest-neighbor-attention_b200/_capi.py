"""ctypes binding of libconvnn_b200.so (declared in include/convnn_b200.h).

The library is the product: there is no Python or CPU fallback.  ``lib()`` raises when
the shared object is missing and cannot be built, and every call raises on a non-zero
status with the library's own message.
"""
from __future__ import annotations

import ctypes
import os
import threading

from . import build as _build

c_i32, c_i64, c_void, c_size = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t

F32, BF16 = 0, 1
METRIC = {"cosine": 0, "matmul": 1, "euclidean": 2}
CONV = {"depthwise": 0, "standard": 1, "depthwise-separable": 2}

OK = 0
E_INVALID, E_UNSUPPORTED, E_NULL, E_ALIGN, E_WORKSPACE, E_CUDA, E_DEVICE, E_TOPK_RANGE, E_SEQ_LENGTH = range(-1, -10, -1)


class ConvnnDesc(ctypes.Structure):
    """Mirror of ``struct convnn_desc``."""
    _fields_ = [(n, c_i32) for n in ("B", "T", "S", "D", "H", "K", "dtype", "metric", "sampled",
                                     "conv_type", "softmax", "coord", "seq_length", "reserved")]


# name -> (restype, argtypes); must list every symbol the header declares
SIGNATURES = {
    "convnn_b200_abi_version": (ctypes.c_int, []),
    "convnn_b200_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "convnn_b200_last_error": (ctypes.c_char_p, []),
    "convnn_b200_launch_count": (ctypes.c_uint64, []),
    "convnn_b200_device_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_int)]),
    "convnn_b200_selftest_wait_timeout": (ctypes.c_int, [ctypes.c_uint32, c_void, c_void, c_void]),
    "convnn_b200_head_channels": (ctypes.c_int, [ctypes.POINTER(ConvnnDesc)]),
    "convnn_b200_workspace_bytes": (c_size, [ctypes.POINTER(ConvnnDesc)]),
    "convnn_b200_stage_scratch_bytes": (c_size, [ctypes.POINTER(ConvnnDesc)]),
    "convnn_b200_qkv_proj": (ctypes.c_int, [ctypes.POINTER(ConvnnDesc), c_void, c_i64, c_void, c_void, c_void,
                                            c_void, c_void, c_void, c_void, c_void, c_void]),
    "convnn_b200_sim_topk": (ctypes.c_int, [ctypes.POINTER(ConvnnDesc), c_void, c_void, c_void, c_void, c_void,
                                            c_void, c_void, c_void]),
    "convnn_b200_gather_conv": (ctypes.c_int, [ctypes.POINTER(ConvnnDesc), c_void, c_void, c_void, c_void, c_void,
                                               c_void, c_void, c_void]),
    "convnn_b200_out_proj": (ctypes.c_int, [ctypes.POINTER(ConvnnDesc), c_void, c_void, c_void, c_i64, c_void, c_i64,
                                            c_void, c_void]),
    "convnn_b200_forward": (ctypes.c_int, [ctypes.POINTER(ConvnnDesc), c_void, c_i64, c_void, c_void, c_void, c_void,
                                           c_void, c_void, c_i64, c_void, c_i64, c_void, c_size, c_void]),
    "convnn_b200_noalloc_capacity": (c_size, []),
    "convnn_b200_forward_noalloc": (ctypes.c_int, [ctypes.POINTER(ConvnnDesc), c_void, c_i64, c_void, c_void, c_void,
                                                   c_void, c_void, c_void, c_i64, c_void, c_i64, c_void]),
    "convnn_b200_layernorm": (ctypes.c_int, [ctypes.c_int, c_void, c_i64, c_void, c_void, ctypes.c_float, c_void,
                                             c_i64, c_i64, c_i32, c_void]),
    "convnn_b200_linear": (ctypes.c_int, [ctypes.c_int, c_void, c_i64, c_void, c_void, c_void, c_i64, c_void, c_i64,
                                          c_i64, c_i32, c_i32, c_i32, c_void]),
    "convnn_b200_patchify": (ctypes.c_int, [ctypes.c_int, c_void, c_void, c_i32, c_i32, c_i32, c_i32, c_i32, c_void]),
    "convnn_b200_patchify_u8": (ctypes.c_int, [ctypes.c_int, c_void, c_void, c_void, c_void, c_i32, c_i32, c_i32, c_i32,
                                               c_i32, c_void]),
    "convnn_b200_embed_tokens": (ctypes.c_int, [ctypes.c_int, c_void, c_void, c_void, ctypes.c_float, c_void, c_void,
                                                c_void, c_i32, c_i32, c_i32, c_void]),
    "convnn_b200_moment_planes": (ctypes.c_int, [c_i32]),
    "convnn_b200_moment_stride": (c_i64, [c_i64]),
    "convnn_b200_prenorm_linear_supported": (ctypes.c_int, [c_i32, c_i32, c_i32]),
    "convnn_b200_prenorm_forward_supported": (ctypes.c_int, [ctypes.POINTER(ConvnnDesc)]),
    "convnn_b200_row_moments": (ctypes.c_int, [c_void, c_i64, c_i64, c_i32, c_void, c_void]),
    "convnn_b200_fold_layernorm": (ctypes.c_int, [c_void, c_void, c_void, c_void, c_i32, c_i32, c_void, c_void,
                                                  c_void]),
    "convnn_b200_prenorm_linear": (ctypes.c_int, [c_void, c_i64, c_void, c_i32, ctypes.c_float, c_void, c_void, c_void,
                                                  c_i64, c_i64, c_i32, c_i32, c_i32, c_void]),
    "convnn_b200_linear_moments": (ctypes.c_int, [c_void, c_i64, c_void, c_void, c_void, c_i64, c_void, c_i64, c_i64,
                                                  c_i32, c_i32, c_void, c_void]),
    "convnn_b200_prenorm_forward": (ctypes.c_int, [ctypes.POINTER(ConvnnDesc), c_void, c_i64, c_void, c_i32,
                                                   ctypes.c_float, c_void, c_void, c_void, c_void, c_void, c_void, c_i64,
                                                   c_void, c_i64, c_void, c_void, c_size, c_void]),
    "convnn_b200_prenorm_mlp_supported": (ctypes.c_int, [c_i32, c_i32, c_i32]),
    "convnn_b200_prenorm_mlp_moment_planes": (ctypes.c_int, []),
    "convnn_b200_prenorm_mlp": (ctypes.c_int, [c_void, c_i64, c_void, c_i32, ctypes.c_float, c_void, c_void, c_void,
                                               c_void, c_void, c_i64, c_i64, c_i32, c_i32, c_void, c_void]),
    "convnn_b200_outproj_mlp": (ctypes.c_int, [c_void, c_i64, c_void, c_void, c_i64, ctypes.c_float, c_void, c_void, c_void,
                                               c_void, c_void, c_i64, c_i64, c_i32, c_i32, c_void, c_void]),
    "convnn_b200_embed_tokens_moments": (ctypes.c_int, [ctypes.c_int, c_void, c_void, c_void, ctypes.c_float, c_void, c_void,
                                                        c_void, c_i32, c_i32, c_i32, c_void, c_void]),
    "convnn_b200_attention_workspace_bytes": (c_size, [ctypes.c_int, c_i32, c_i32, c_i32]),
    "convnn_b200_softmax_attention": (ctypes.c_int, [ctypes.c_int, c_void, c_i64, c_void, c_void, c_void, c_i64, c_i32,
                                                     c_i32, c_i32, c_i32, c_void, c_size, c_void]),
    "convnn_b200_conv1d_attention_workspace_bytes": (c_size, [ctypes.c_int, c_i32, c_i32, c_i32, c_i32]),
    "convnn_b200_conv1d_attention": (ctypes.c_int, [ctypes.c_int, c_void, c_i64, c_void, c_void, c_void, c_void, c_void,
                                                    c_void, c_void, c_i64, c_i32, c_i32, c_i32, c_i32, c_i32, c_void,
                                                    c_size, c_void]),
}

_lock = threading.Lock()
_lib = None


def library_path() -> str:
    return _build.LIB


def lib() -> ctypes.CDLL:
    """Load (building first if the sources are newer and nvcc is present) the library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.LIB
        if os.environ.get("CONVNN_B200_NO_BUILD") != "1":
            try:
                if _build.stale():
                    _build.build()
            except RuntimeError:
                if not os.path.exists(path):
                    raise
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: build it with convnn_b200.build.build(); there is no fallback path")
        handle = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)          # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        if handle.convnn_b200_abi_version() != 1:
            raise RuntimeError("libconvnn_b200.so ABI version mismatch")
        _lib = handle
        return _lib


class ConvnnError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def check(status: int) -> None:
    """Raise the Python exception the reference would have raised for this failure
    (ValueError for bad arguments, RuntimeError otherwise)."""
    if status == OK:
        return
    L = lib()
    detail = (L.convnn_b200_last_error() or b"").decode() or L.convnn_b200_status_string(status).decode()
    if status == E_INVALID:
        raise ValueError(detail)
    raise ConvnnError(status, detail)


def make_desc(B, T, S, D, H, K, dtype, metric, sampled, conv_type, softmax, coord, seq_length) -> ConvnnDesc:
    return ConvnnDesc(B, T, S, D, H, K, dtype, METRIC[metric] if isinstance(metric, str) else metric,
                      int(bool(sampled)), CONV[conv_type] if isinstance(conv_type, str) else conv_type,
                      int(bool(softmax)), int(bool(coord)), int(seq_length), 0)


def ptr(t) -> int:
    """Device pointer of a torch tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


def device_status() -> int:
    """Error latch of the tensor-core kernels (0 = clean); synchronises the device."""
    code = ctypes.c_int(0)
    check(lib().convnn_b200_device_status(ctypes.byref(code)))
    return code.value

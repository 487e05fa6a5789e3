"""ctypes binding of the C-ABI library (``include/luna_b200.h``).

The library is the product: there is no Python or CPU fallback.  If the shared object is missing, or an entry
point fails, callers get an exception.  The reference reaches its own generated kernels through pybind11
(``src/utils/extension.py:38-70``) and has a ctypes precedent for plain C libraries (``src/utils/jit.py:64-98``).
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

_PACKAGE_DIR = os.path.dirname(os.path.abspath(__file__))
# LUNA_B200_LIBRARY selects another build of the same library (kernel tuning experiments).
LIBRARY_PATH = os.environ.get("LUNA_B200_LIBRARY") or os.path.join(_PACKAGE_DIR, "_lib", "libluna_b200.so")

LUNA_OK = 0
LUNA_ERR_INVALID_ARGUMENT = -1
LUNA_ERR_UNSUPPORTED = -2
LUNA_ERR_CUDA = -3
LUNA_ERR_MISALIGNED = -4
LUNA_ERR_SCRATCH = -5
LUNA_ERR_DEVICE_TIMEOUT = -6
LUNA_ERR_OVERFLOW = -7

LUNA_F32, LUNA_F64 = 0, 1

_EXCEPTIONS = {
    LUNA_ERR_INVALID_ARGUMENT: ValueError,
    LUNA_ERR_UNSUPPORTED: NotImplementedError,
    LUNA_ERR_CUDA: RuntimeError,
    LUNA_ERR_MISALIGNED: ValueError,
    LUNA_ERR_SCRATCH: RuntimeError,
    LUNA_ERR_DEVICE_TIMEOUT: RuntimeError,
    LUNA_ERR_OVERFLOW: OverflowError,
}


class UvuPath(ctypes.Structure):
    _fields_ = [(name, ctypes.c_int32) for name in (
        "x_offset", "y_offset", "out_offset", "weight_offset", "weight_stride", "channels",
        "l1", "l2", "l3", "term_begin", "term_end")]


class UvuDesc(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32), ("in1_dim", ctypes.c_int32), ("in2_dim", ctypes.c_int32),
        ("out_dim", ctypes.c_int32), ("weight_numel", ctypes.c_int32), ("num_paths", ctypes.c_int32),
        ("paths", ctypes.POINTER(UvuPath)), ("num_terms", ctypes.c_int32),
        ("term_i", ctypes.POINTER(ctypes.c_int32)), ("term_j", ctypes.POINTER(ctypes.c_int32)),
        ("term_k", ctypes.POINTER(ctypes.c_int32)), ("term_c", ctypes.POINTER(ctypes.c_double)),
    ]


class Graph(ctypes.Structure):
    _fields_ = [
        ("num_nodes", ctypes.c_int64), ("num_src_nodes", ctypes.c_int64), ("num_edges", ctypes.c_int64),
        ("src", ctypes.c_void_p), ("dst", ctypes.c_void_p), ("dst_rowptr", ctypes.c_void_p),
        ("src_rowptr", ctypes.c_void_p), ("edge_ids_by_src", ctypes.c_void_p),
    ]


class GraphOut(ctypes.Structure):
    _fields_ = [(name, ctypes.c_void_p) for name in (
        "src", "dst", "dst_rowptr", "src_rowptr", "edge_ids_by_src", "node_order", "source_node_order")]


class ShDesc(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32), ("num_degrees", ctypes.c_int32), ("degrees", ctypes.c_int32 * 32),
        ("normalize", ctypes.c_int32), ("normalization", ctypes.c_int32),
    ]


# name -> (restype, argtypes); mirrors include/luna_b200.h
_P = ctypes.c_void_p
_SIGNATURES = {
    "luna_last_error": (ctypes.c_char_p, []),
    "luna_version": (ctypes.c_int, []),
    "luna_compiled_sm": (ctypes.c_int, []),
    "luna_uvu_plan_create": (ctypes.c_int, [ctypes.POINTER(UvuDesc), ctypes.POINTER(_P)]),
    "luna_uvu_plan_destroy": (None, [_P]),
    "luna_uvu_plan_query": (ctypes.c_int64, [_P, ctypes.c_int]),
    "luna_uvu_plan_set_generic": (ctypes.c_int, [_P, ctypes.c_int]),
    "luna_uvu_conv_scratch_bytes": (ctypes.c_int64, [_P, ctypes.c_int64, ctypes.c_int64]),
    "luna_uvu_conv_fwd": (ctypes.c_int, [_P, ctypes.POINTER(Graph), _P, _P, _P, _P, _P]),
    "luna_uvu_conv_bwd": (ctypes.c_int, [_P, ctypes.POINTER(Graph), _P, _P, _P, _P, _P, _P, _P, _P,
                                         ctypes.c_int64, _P]),
    "luna_uvu_conv_bwd_add_gx": (ctypes.c_int, [_P, ctypes.POINTER(Graph), _P, _P, _P, _P, _P, _P, _P, _P,
                                                ctypes.c_int64, _P]),
    "luna_uvu_conv_noalloc_max_scratch_bytes": (ctypes.c_int64, []),
    "luna_uvu_conv_noalloc_prepare": (ctypes.c_int, [_P]),
    "luna_uvu_conv_bwd_noalloc": (ctypes.c_int, [_P, ctypes.POINTER(Graph), _P, _P, _P, _P, _P, _P, _P, _P]),
    "luna_uvu_conv_dbl_bwd": (ctypes.c_int, [_P, ctypes.POINTER(Graph), _P, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                                             _P, _P, ctypes.c_int64, _P]),
    "luna_uvu_check_status": (ctypes.c_int, [_P, _P]),
    "luna_graph_scratch_bytes": (ctypes.c_int64, [ctypes.c_int64, ctypes.c_int64]),
    "luna_graph_bounds": (ctypes.c_int, [_P, _P, ctypes.c_int, ctypes.c_int64, ctypes.POINTER(ctypes.c_int64),
                                         ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64),
                                         ctypes.POINTER(ctypes.c_int), _P, ctypes.c_int64, _P]),
    "luna_graph_build": (ctypes.c_int, [_P, _P, ctypes.c_int, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,
                                        ctypes.POINTER(GraphOut), _P, ctypes.c_int64, _P]),
    "luna_probe_fma": (ctypes.c_int, [ctypes.c_int, ctypes.c_int, _P, ctypes.POINTER(ctypes.c_double), _P]),
    "luna_sh_fwd": (ctypes.c_int, [ctypes.POINTER(ShDesc), _P, _P, ctypes.c_int64, _P]),
    "luna_sh_bwd": (ctypes.c_int, [ctypes.POINTER(ShDesc), _P, _P, _P, ctypes.c_int64, _P]),
    "luna_sh_dbl_bwd": (ctypes.c_int, [ctypes.POINTER(ShDesc), _P, _P, _P, _P, _P, ctypes.c_int64, _P]),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lock = threading.Lock()
_library = None


def library() -> ctypes.CDLL:
    """Load the shared object once.  Raises if it has not been built: there is no fallback path."""
    global _library
    if _library is not None:
        return _library
    with _lock:
        if _library is None:
            if not os.path.exists(LIBRARY_PATH):
                raise RuntimeError(
                    f"{LIBRARY_PATH} is missing: build it with `python -m lunaequivariance_b200.build` "
                    "(needs nvcc; the kernels target sm_100a and have no CPU or PyTorch fallback)."
                )
            handle = ctypes.CDLL(LIBRARY_PATH)
            for name, (restype, argtypes) in _SIGNATURES.items():
                function = getattr(handle, name)
                function.restype = restype
                function.argtypes = argtypes
            _library = handle
    return _library


def last_error() -> str:
    return library().luna_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Map a luna_status to the exception class the reference would raise for the same condition."""
    if status == LUNA_OK:
        return
    raise _EXCEPTIONS.get(status, RuntimeError)(last_error() or f"luna_b200 call failed with status {status}")


def pointer(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def current_stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return LUNA_F32
    if dtype == torch.float64:
        return LUNA_F64
    raise ValueError(f"float32 or float64 required, got {dtype}")


__all__ = ["library", "check", "last_error", "pointer", "current_stream", "dtype_code", "UvuPath", "UvuDesc",
           "Graph", "GraphOut", "ShDesc", "EXPORTED_SYMBOLS", "LIBRARY_PATH"]

"""ctypes binding of libtqb200.so (the C ABI declared in include/tqb200.h).

This is the only module that touches the shared library.  Tensors are passed as raw device
pointers together with the current CUDA stream of their device; outputs and workspaces are torch
allocations made by the callers in this package.  There is no CPU implementation behind these
functions: a missing library or a machine without CUDA raises immediately.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libtqb200.so")
_lib = None

F32, F16, BF16 = 0, 1, 2
_DTYPE_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}
SCAN_MAX_K = 256

c_void_p, c_int, c_int64, c_size_t, c_float = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64,
                                               ctypes.c_size_t, ctypes.c_float)


class RowMap(ctypes.Structure):
    """struct tqb_rowmap of include/tqb200.h."""
    _fields_ = [("inner", c_int64), ("stride_a", c_int64), ("stride_b", c_int64), ("offset", c_int64),
                ("pos", c_void_p), ("pos_div", c_int64), ("slots", c_void_p), ("block_size", ctypes.c_int32)]


def lib():
    """Load the library once.  Fails loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python turboquant-kv_b200/csrc/build.py` "
                "(nvcc, sm_100a).  This package has no CPU or Triton fallback.")
        L = ctypes.CDLL(_LIB_PATH)
        L.tqb_last_error.restype = ctypes.c_char_p
        L.tqb_launch_count.restype = c_int64
        L.tqb_abi_version.restype = c_int
        L.tqb_decode_attention_workspace_bytes.restype = c_size_t
        L.tqb_decode_attention_workspace_bytes.argtypes = [c_int, c_int, c_int, c_int, c_int64]
        L.tqb_scan_records_ctas_per_group.restype = c_int
        L.tqb_scan_records_ctas_per_group.argtypes = [c_int, c_int64, c_int]
        L.tqb_scan_topk_workspace_bytes.restype = c_size_t
        L.tqb_scan_topk_workspace_bytes.argtypes = [c_int, c_int64, c_int, c_int, c_int]
        L.tqb_pack_codes.argtypes = [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]
        L.tqb_unpack_codes.argtypes = [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]
        L.tqb_quantize_mse.argtypes = [c_void_p, c_int, c_int64, c_int, c_int64, c_void_p, c_void_p, c_int,
                                       c_void_p, c_void_p, ctypes.POINTER(RowMap), c_void_p]
        L.tqb_quantize_status.argtypes = [c_void_p]
        L.tqb_dequantize_mse.argtypes = [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int,
                                         c_void_p, c_int, c_void_p]
        L.tqb_quantize_prod.argtypes = [c_void_p, c_int, c_int64, c_int, c_int64, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        L.tqb_dequantize_prod.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p,
                                          c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p]
        L.tqb_attention_scores_packed.argtypes = [c_void_p, c_int64, c_int, c_void_p, c_void_p, c_int64,
                                                  c_void_p, c_void_p, c_int, c_void_p, c_void_p]
        L.tqb_attention_values_packed.argtypes = [c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p,
                                                  c_void_p, c_void_p, c_int, c_void_p, c_void_p]
        L.tqb_kv_record_bytes.restype = c_int64
        L.tqb_kv_record_bytes.argtypes = [c_int, c_int, c_int]
        L.tqb_kv_append.argtypes = [c_void_p, c_void_p, c_int, c_int64, c_int, c_int64, c_void_p, c_void_p,
                                    c_int, c_void_p, c_void_p, c_int, c_void_p, ctypes.POINTER(RowMap), c_void_p]
        L.tqb_kv_export.argtypes = [c_void_p, c_int64, c_int, c_int, c_int, ctypes.POINTER(RowMap), c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_void_p]
        L.tqb_kv_import.argtypes = [c_void_p, c_int64, c_int, c_int, c_int, ctypes.POINTER(RowMap), c_void_p,
                                    c_void_p, c_void_p, c_void_p, c_void_p]
        L.tqb_decode_attention.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int64,
                                           c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                                           c_void_p, c_void_p, c_int, c_float, c_void_p, c_size_t, c_void_p,
                                           c_int, c_void_p]
        L.tqb_decode_step.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_int,
                                      c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                      c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_size_t, c_void_p,
                                      c_int, c_void_p]
        L.tqb_scan_topk_prod_workspace_bytes.restype = c_size_t
        L.tqb_scan_topk_prod_workspace_bytes.argtypes = [c_int, c_int64, c_int, c_int, c_int]
        L.tqb_scan_topk_prod.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                                         c_void_p, c_void_p, c_void_p, c_int, c_int64, c_void_p, c_size_t, c_void_p,
                                         c_void_p, c_void_p]
        L.tqb_scan_topk.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
                                    c_void_p, c_int, c_int64, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p]
        L.tqb_scan_records_workspace_bytes.restype = c_size_t
        L.tqb_scan_records_workspace_bytes.argtypes = [c_int, c_int, c_int, c_int]
        L.tqb_scan_records_topk.argtypes = [c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p,
                                            c_int, c_int64, c_void_p, c_size_t, c_void_p, c_void_p, c_void_p]
        L.tqb_topk_merge.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        msg = lib().tqb_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"turboquant (libtqb200): {msg} [code {rc}]")


def launch_count() -> int:
    return int(lib().tqb_launch_count())


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("turboquant_kv (B200 build) computes on a CUDA device only; none is available "
                           "and there is no CPU fallback")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise RuntimeError(f"unsupported dtype {dtype}; use float32, float16 or bfloat16") from None


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def stream_of(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


def to_device(t: torch.Tensor, device=None) -> torch.Tensor:
    """Host tensors are staged on the GPU (that is the only way anything is computed here)."""
    if t.is_cuda:
        return t
    require_cuda()
    return t.to(device if device is not None else torch.device("cuda", torch.cuda.current_device()),
                non_blocking=True)


def f32c(t: torch.Tensor, device) -> torch.Tensor:
    """float32, contiguous, on `device` (no copy when already so)."""
    return t.to(device=device, dtype=torch.float32).contiguous()


def dense_rowmap() -> RowMap:
    return RowMap(1, 1, 0, 0, None, 1, None, 1)

"""ctypes binding of ``libmoc_b200.so``.

The product has no CPU path: importing this module never builds or falls back; :func:`lib` raises
``RuntimeError`` if the shared library has not been built (``python -m memory_b200.build``).
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

from .build import LIB_PATH

MOC_F32, MOC_BF16 = 0, 1
ATTN_BWD_STATIC_MAX_FLOATS = 1 << 20   # MOC_ATTN_BWD_STATIC_MAX_FLOATS in include/moc_b200.h
NORM_NONE, NORM_RMS, NORM_LAYERNORM = 0, 1, 2
NORM_CODES = {None: NORM_NONE, "none": NORM_NONE, "rms": NORM_RMS, "layernorm": NORM_LAYERNORM}
KERNEL_TAGS = {1: "gemm_tc.cu", 2: "attn_tc_fwd.cu", 3: "attn_tc_bwd.cu", 4: "host_util.cu",
               5: "token_mix_tc.cu"}
DEV_STATUS_TEXT = {1: "a bounded device wait timed out", 2: "a chapter index was out of range"}


class RouterShape(C.Structure):
    _fields_ = [("batch", C.c_int32), ("seq", C.c_int32), ("hidden_dim", C.c_int32),
                ("num_chapters", C.c_int32), ("top_k", C.c_int32), ("num_shared", C.c_int32),
                ("routed_scale", C.c_float), ("h_dtype", C.c_int32)]


class GemmDesc(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("c_dtype", C.c_int32), ("m", C.c_int32), ("n", C.c_int32),
                ("k", C.c_int32), ("a_kmajor", C.c_int32), ("b_kmajor", C.c_int32),
                ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64),
                ("accumulate", C.c_int32), ("split_k", C.c_int32), ("scale_block_rows", C.c_int32),
                ("a_block_rows", C.c_int32), ("a_stored_rows", C.c_int64),
                ("residual", C.c_void_p), ("ldr", C.c_int64)]


class AttnShape(C.Structure):
    _fields_ = [("batch", C.c_int32), ("seq", C.c_int32), ("n_sel", C.c_int32), ("num_heads", C.c_int32),
                ("num_kv_heads", C.c_int32), ("head_dim", C.c_int32), ("scale", C.c_float),
                ("dtype", C.c_int32)]


class SparseAttnShape(C.Structure):
    _fields_ = [("batch", C.c_int32), ("tq", C.c_int32), ("tk", C.c_int32), ("hq", C.c_int32),
                ("h", C.c_int32), ("head_dim", C.c_int32), ("n_select", C.c_int32),
                ("block_size", C.c_int32), ("scale", C.c_float), ("dtype", C.c_int32)]


class DecodeShape(C.Structure):
    _fields_ = [("batch", C.c_int32), ("n_q", C.c_int32), ("num_heads", C.c_int32), ("num_kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("n_chapters", C.c_int32), ("tokens_per_chapter", C.c_int32),
                ("scale", C.c_float)]


P = C.c_void_p
_PROTOTYPES = {
    "moc_last_error": (C.c_char_p, []),
    "moc_abi_version": (C.c_int, []),
    "moc_peer_barrier": (C.c_int, [P, C.c_int32, C.c_int32, C.c_uint32, C.c_uint32, P, P]),
    "moc_router_workspace_bytes": (C.c_size_t, [C.POINTER(RouterShape)]),
    "moc_router_workspace_bytes_parts": (C.c_size_t, [C.POINTER(RouterShape), C.c_int32, C.c_int32]),
    "moc_router_fwd": (C.c_int, [C.POINTER(RouterShape)] + [P] * 13 + [P, C.c_size_t, P, P]),
    "moc_router_fwd_parts": (C.c_int, [C.POINTER(RouterShape)] + [P] * 13 + [P, C.c_size_t, C.c_int32, P, P]),
    "moc_router_bwd": (C.c_int, [C.POINTER(RouterShape)] + [P] * 16 + [C.c_int32, P, C.c_size_t, P, P]),
    "moc_router_bwd_parts": (C.c_int, [C.POINTER(RouterShape)] + [P] * 16 + [C.c_int32, P, C.c_size_t, C.c_int32, P, P]),
    "moc_pool_weighted_fwd": (C.c_int, [P, C.c_int32, P, P, C.c_int32, C.c_int32, C.c_int32, P, C.c_size_t, P]),
    "moc_pool_weighted_bwd": (C.c_int, [P, P, P, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, P]),
    "moc_wait_probe": (C.c_int, [C.c_int32, C.c_int32, C.c_uint32, P, P, P]),
    "moc_gather_rows_fwd": (C.c_int, [P, C.c_int32, C.c_int64, C.c_int32, C.c_int32, P, P, C.c_int32,
                                      C.c_int32, C.c_int32, C.c_float, P, C.c_int32, P, P, P]),
    "moc_chapter_segments": (C.c_int, [P, C.c_int32, C.c_int32, P, P, P, P, P, P, P]),
    "moc_gather_rows_bwd": (C.c_int, [P, C.c_int32, P, C.c_int32, C.c_int64, C.c_int32, C.c_int32, P, P,
                                      C.c_int32, C.c_int32, C.c_int32, C.c_float, P, P, P, P, P, P, P, P, P, P]),
    "moc_bank_grad_merge": (C.c_int, [P, C.c_int32, C.c_int32, P, P, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                      C.c_float, P, P, P, P, P, P, C.c_int64, P, P]),
    "moc_bank_grad_merge_to": (C.c_int, [P, C.c_int32, C.c_int32, P, P, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                         C.c_float, P, P, P, P, P, P, C.c_int32, C.c_int64, P, P]),
    "moc_scatter_bank_grad": (C.c_int, [P, P, P, C.c_int32, C.c_int32, C.c_int32, P, C.c_int64, P, P]),
    "moc_gemm": (C.c_int, [C.POINTER(GemmDesc), P, P, P, P, P, P, P]),
    "moc_attn_fwd": (C.c_int, [C.POINTER(AttnShape), P, P, P, P, P, P]),
    "moc_attn_bwd": (C.c_int, [C.POINTER(AttnShape), P, P, P, P, P, P, P, P, P, P]),
    "moc_attn_bwd_parts": (C.c_int, [C.POINTER(AttnShape), P, P, P, P, P, P, P, P, C.c_int32, P, P]),
    "moc_attn_bwd_scaled": (C.c_int, [C.POINTER(AttnShape), P, P, P, P, P, P, P, P, P, P, P, P]),
    "moc_attn_bwd_scaled_parts": (C.c_int, [C.POINTER(AttnShape), P, P, P, P, P, P, P, P, P, P, C.c_int32, P, P]),
    "moc_gemm_gather_b": (C.c_int, [C.POINTER(GemmDesc), P, P, P, P, P, C.c_int32, C.c_int64, P, P]),
    "moc_row_inv_rms": (C.c_int, [P, C.c_int32, C.c_int64, C.c_int32, C.c_float, P, P]),
    "moc_chapter_row_scale": (C.c_int, [P, P, P, C.c_int64, C.c_int32, C.c_int32, P, P, P]),
    "moc_gather_rows_bwd_prescaled": (C.c_int, [P, C.c_int32, P, C.c_int32, C.c_int64, C.c_int32, C.c_int32, P, P,
                                                C.c_int32, P, P, P, P, P, P, P, P, P, P]),
    "moc_attn_bwd_static": (C.c_int, [C.POINTER(AttnShape), P, P, P, P, P, P, P, P, P]),
    "moc_sparse_attn_fwd": (C.c_int, [C.POINTER(SparseAttnShape), P, P, P, P, P, P, P, P]),
    "moc_sparse_attn_bwd": (C.c_int, [C.POINTER(SparseAttnShape), P, P, P, P, P, P, P, P, P, P, P, P]),
    "moc_sparse_attn_weighted_fwd": (C.c_int, [C.POINTER(SparseAttnShape), P, P, P, C.c_int64, P, P, P, C.c_float,
                                               P, P, P, P]),
    "moc_sparse_attn_weighted_bwd": (C.c_int, [C.POINTER(SparseAttnShape), P, P, P, C.c_int64, P, P, C.c_float, P,
                                               P, P, C.c_int32, P, P, C.c_int64, P, P, P]),
    "moc_token_mix_workspace_bytes": (C.c_size_t, [C.POINTER(SparseAttnShape), C.c_int32]),
    "moc_token_mix_index": (C.c_int, [C.POINTER(SparseAttnShape), C.c_int32, P, P, P, P]),
    "moc_token_mix_fwd": (C.c_int, [C.POINTER(SparseAttnShape), C.c_int32, P, P, P, C.c_int64, P, P, P, C.c_float,
                                    P, P, P, P, P, P]),
    "moc_token_mix_bwd": (C.c_int, [C.POINTER(SparseAttnShape), C.c_int32, P, P, P, C.c_int64, P, P, C.c_float, P, P,
                                    P, P, P, P, P, P, C.c_int64, P, P, P]),
    "moc_bank_adamw_workspace_bytes": (C.c_size_t, [C.c_int32]),
    "moc_bank_adamw_step": (C.c_int, [P, P, P, C.c_int64, C.c_int32, C.c_int32, P, P, C.c_int32, P, C.c_float,
                                      C.c_float, C.c_float, C.c_float, C.c_float, C.c_float, C.c_int64, P, P,
                                      C.c_size_t, P, P]),
    "moc_rows_sqnorm": (C.c_int, [P, P, C.c_int32, C.c_int32, P, P, C.c_size_t, P]),
    "moc_row_dot": (C.c_int, [P, P, C.c_int32, P, C.c_int64, C.c_int32, P]),
    "moc_col_sum": (C.c_int, [P, P, C.c_int64, C.c_int32, P]),
    "moc_cast_f32_to_bf16": (C.c_int, [P, P, C.c_int64, P]),
    "moc_cast_bf16_to_f32": (C.c_int, [P, P, C.c_int64, P]),
    "moc_split_bf16": (C.c_int, [P, P, C.c_int64, C.c_int32, P]),
    "moc_sum_terms": (C.c_int, [P, P, P, C.c_int64, C.c_int32, C.c_int32, C.c_int32, P]),
    "moc_transpose": (C.c_int, [P, C.c_int32, P, C.c_int32, C.c_int32, C.c_int32, P]),
    "moc_pack_weights": (C.c_int, [C.c_int32, P, C.c_int32, P, P, P, P, P, P]),
    "moc_decode_attn": (C.c_int, [P, P, P, C.c_int64, P, P, P, P, P, P]),
    "moc_norm_bwd_workspace_bytes": (C.c_size_t, [C.c_int64, C.c_int32]),
    "moc_norm_fwd": (C.c_int, [P, P, P, C.c_int32, C.c_float, C.c_int64, C.c_int32, P, P, P, P]),
    "moc_norm_bwd": (C.c_int, [P, P, P, P, P, C.c_int32, C.c_int64, C.c_int32, P, P, P, P, P]),
}
# symbols every build must export (checked by the CPU test-suite against include/moc_b200.h)
EXPORTED = tuple(_PROTOTYPES)

_lock = threading.Lock()
_lib = None
_status = {}


def lib() -> C.CDLL:
    """The loaded library.  Raises if it is missing: there is no fallback implementation."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: build it with `python -m memory_b200.build` "
                        "(the CUDA library is the only implementation of these operators)")
                handle = C.CDLL(LIB_PATH)
                for name, (res, args) in _PROTOTYPES.items():
                    if not hasattr(handle, name):
                        continue
                    fn = getattr(handle, name)
                    fn.restype = res
                    fn.argtypes = args
                _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().moc_last_error().decode("utf-8", "replace")
        if rc == -1:
            raise ValueError(f"{what}: {msg}")
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")


def ptr(t) -> int:
    """Device pointer of a tensor (None -> NULL)."""
    if t is None:
        return None
    return t.data_ptr()


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def status_word(device) -> torch.Tensor:
    """Per-device int32 the kernels raise on device-side errors."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", key))
        _status[key] = t
    return t


def check_device_status(device, clear: bool = True) -> None:
    """Synchronising read of the device status word; raises if a kernel reported an error."""
    t = status_word(device)
    v = int(t.item())
    if clear and v != 0:
        t.zero_()
    if v != 0:
        code, tag, line = v & 0xFF, (v >> 8) & 0xF, v >> 12
        where = f" ({KERNEL_TAGS.get(tag, 'kernel file %d' % tag)}, source line {line})" if (tag or line) else ""
        raise RuntimeError(f"device-side error {code}: {DEV_STATUS_TEXT.get(code, 'unknown')}{where}")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return MOC_F32
    if dt == torch.bfloat16:
        return MOC_BF16
    raise TypeError(f"unsupported dtype {dt}; the kernels take float32 or bfloat16")


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("memory_b200 operators run on CUDA tensors only (there is no CPU path)")

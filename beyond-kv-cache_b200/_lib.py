"""ctypes binding of ``libbkv_sm100.so`` (the C ABI declared in ``include/bkv_sm100.h``).

There is no fallback: if the library is missing or a call returns a non-zero status
the caller gets an exception.  Tensors cross the boundary as raw device pointers
(``tensor.data_ptr()``), sizes, element strides and the current CUDA stream handle.
"""

from __future__ import annotations

import ctypes
import os
import threading

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libbkv_sm100.so")

BKV_F16, BKV_BF16, BKV_F32 = 0, 1, 2
LAYOUT_HEAD_WORD_TOKEN, LAYOUT_HND_TOKEN_WORD = 1, 2
FLAG_PDL_TRIGGER, FLAG_PDL_WAIT, FLAG_LINEAR_SEARCH, FLAG_KLEVELS_LANE_MAJOR, FLAG_BINNED_TABLES = 1, 2, 4, 8, 16
ERR_ARG, ERR_UNSUPPORTED, ERR_ALIGN, ERR_CUDA, ERR_LIMIT = -1, -2, -3, -4, -5

_c = ctypes
_P, _I, _L, _F = _c.c_void_p, _c.c_int, _c.c_int64, _c.c_float

# name -> argtypes, in the order of include/bkv_sm100.h
SIGNATURES = {
    "bkv_abi_version": [],
    "bkv_status_string": [_I],
    "bkv_last_cuda_error": [],
    "bkv_encode_sm100": [_P, _P, _L, _L, _L, _L, _I, _P, _I, _L, _L, _I, _P, _L, _L, _I, _I, _I,
                         _P, _P, _P, _P, _I, _I, _I, _P, _P, _L, _L, _L, _L, _I, _P],
    "bkv_decode_sm100": [_P, _L, _I, _P, _L, _L, _I, _I, _I, _P, _L, _P, _P, _P, _I, _P, _I, _P,
                         _P, _P, _P, _I, _I, _I, _I, _F, _I, _P],
    "bkv_decode_noalloc_sm100": [_P, _L, _I, _P, _L, _L, _I, _I, _I, _P, _L, _P, _P, _P, _I, _P, _I, _P,
                                 _I, _I, _I, _I, _F, _I, _P],
    "bkv_decode_stream_sm100": [_P, _L, _I, _P, _L, _L, _I, _I, _I, _P, _L, _P, _P, _P, _I, _P, _I, _P,
                                _P, _L, _P, _I, _I, _I, _F, _I, _I, _P],
    "bkv_decode_stream_workspace_bytes": [],
    "bkv_decode_stream_workspace_init": [_P, _L, _P],
    "bkv_decode_tables_bytes": [_I],
    "bkv_decode_tables_sm100": [_P, _P, _I, _I, _I, _P, _L, _P],
    "bkv_selftest_partition": [_P, _I, _I, _I, _I],
    "bkv_selftest_division_sm100": [_c.c_uint64, _L, _I, _P, _P],
    "bkv_decode_device_status": [_P],
    "bkv_combine_sm100": [_P, _P, _P, _I, _L, _P, _I, _P, _P],
    "bkv_decode_range_sm100": [_P, _L, _I, _P, _L, _L, _I, _I, _I, _P, _L, _P, _P, _P, _I, _P, _P,
                               _P, _I, _I, _I, _I, _F, _I, _P],
    "bkv_combine_packed_sm100": [_P, _I, _L, _P, _I, _P, _P],
    "bkv_decode_range_stream_sm100": [_P, _L, _I, _P, _L, _L, _I, _I, _I, _P, _L, _P, _P, _P, _I, _P, _P,
                                      _P, _P, _L, _P, _I, _I, _I, _I, _F, _I, _I, _P],
    "bkv_kv_exchange_bytes": [_I, _L],
    "bkv_kv_exchange_alloc": [_L, _P, _P],
    "bkv_kv_exchange_open": [_P, _P],
    "bkv_kv_exchange_close": [_P],
    "bkv_kv_exchange_free": [_P],
    "bkv_kv_exchange_merge_sm100": [_P, _L, _P, _I, _I, _I, _L, _P, _I, _P, _P, _P],
    "bkv_readback_sm100": [_P, _L, _L, _I, _I, _I, _P, _L, _L, _P, _P, _I, _I, _P, _P, _I, _I, _I,
                           _P, _P, _I, _P],
    "bkv_decode_dense_sm100": [_P, _L, _I, _P, _P, _I, _L, _I, _I, _P, _L, _P, _P, _I, _P, _P, _P,
                               _I, _I, _I, _I, _F, _P],
    "bkv_derive_slots_sm100": [_P, _P, _L, _L, _I, _I, _P, _P],
}

_lock = threading.Lock()
_lib = None


class BkvError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn: str, status: int, detail: str):
        super().__init__(f"{fn} failed with status {status}: {detail}")
        self.status = status


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python beyond-kv-cache_b200/build.py` "
                "(nvcc, sm_100a). There is no CPU or library fallback for this path."
            )
        lib = ctypes.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is not exported
            fn.argtypes = argtypes
            if name in ("bkv_status_string", "bkv_last_cuda_error"):
                fn.restype = _c.c_char_p
            elif name in ("bkv_decode_stream_workspace_bytes", "bkv_decode_tables_bytes", "bkv_kv_exchange_bytes"):
                fn.restype = _L
            else:
                fn.restype = _I
        _lib = lib
        return lib


def call(name: str, *args) -> None:
    """Invoke an entry point and convert a non-zero status into an exception
    (``ValueError`` for argument/shape problems, ``BkvError`` otherwise)."""
    lib = load()
    status = getattr(lib, name)(*args)
    if status == 0:
        return
    detail = lib.bkv_status_string(status).decode()
    if status == ERR_CUDA:
        detail += " — " + lib.bkv_last_cuda_error().decode()
    if status in (ERR_ARG, ERR_ALIGN, ERR_LIMIT):
        raise ValueError(f"{name}: {detail}")
    raise BkvError(name, status, detail)


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float16:
        return BKV_F16
    if dtype == torch.bfloat16:
        return BKV_BF16
    if dtype == torch.float32:
        return BKV_F32
    raise TypeError(f"unsupported dtype {dtype}")


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def current_stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def stream_workspace(device: torch.device) -> torch.Tensor:
    """Scratch of the persistent decode schedule for ``device``, prepared for its first use
    (the request counters at its head start at zero; the kernels leave them at zero)."""
    with torch.cuda.device(device):
        nbytes = int(load().bkv_decode_stream_workspace_bytes())
    return torch.zeros((nbytes,), dtype=torch.uint8, device=device)

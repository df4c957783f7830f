"""Loads the CUDA kernel library and declares its C entry points.

The library is the only implementation of these operations: there is no CPU or library fallback.
`load()` raises `KernelLibraryError` when the library cannot be built or loaded, and every wrapper
raises `KernelError` with the library's own message when a call is refused.
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Optional

from . import build as _build

F32, BF16 = 0, 1  # dtype codes of csrc/common.cuh

ERR_BAD_PAGE, ERR_BAD_TOKEN, ERR_WAIT_TIMEOUT, ERR_INTERNAL = 1, 2, 4, 8


class KernelLibraryError(RuntimeError):
    """The CUDA kernel library is missing and could not be built."""


class KernelError(RuntimeError):
    """A kernel entry point refused its arguments or failed to launch."""


class KvView(C.Structure):
    """Mirror of IbKvView in csrc/kv_view.cuh."""
    _fields_ = [
        ("base", C.c_void_p),
        ("page_stride", C.c_longlong),
        ("v_offset", C.c_longlong),
        ("block_table", C.c_void_p),
        ("table_stride", C.c_int),
        ("page_size", C.c_int),
        ("num_pages", C.c_int),
        ("kv_heads", C.c_int),
        ("head_dim", C.c_int),
        ("dtype", C.c_int),
    ]


_p, _i, _f, _ll = C.c_void_p, C.c_int, C.c_float, C.c_longlong

_SIGNATURES = {
    "ib_embed": [_p, _i, _p, _p, _i, _i, _i, _p, _p],
    "ib_add_rmsnorm": [_p, _p, _i, _ll, _p, _p, _i, _p, _i, _i, _f, _i, _p],
    "ib_rope_table": [_p, _p, _p, _p, _i, _i, _p],
    "ib_silu_mul": [_p, _i, _ll, _p, _i, _i, _i, _p],
    "ib_qk_norm_rope_kv": [_p, _i, _ll, _p, _p, _f, _p, _p, _i, _p, _p, _p, _i, C.POINTER(KvView), _i, _i, _i, _p, _p],
    "ib_attention_generic": [_p, _i, C.POINTER(KvView), _p, _p, _i, _f, _p, _i, _i, _p, _p],
    "ib_gemm_simt": [_p, _i, _p, _i, _p, _i, _i, _i, _p],
    "ib_sample_rows": [_p, _i, _i, _p, _p, _p, _p, _p],
    "ib_advance_rows": [_p, _p, _p, _p, _p, _p, _p, _i, _i, _p],
}

_lib: Optional[C.CDLL] = None
_lock = threading.Lock()


def load() -> C.CDLL:
    """Build (if needed) and load the kernel library; fails loudly."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        try:
            path = _build.build()
            lib = C.CDLL(str(path))
        except (OSError, _build.BuildError) as e:
            raise KernelLibraryError(f"the CUDA kernel library is not available: {e}") from e
        lib.ib_last_error.restype = C.c_char_p
        lib.ib_last_error.argtypes = []
        for name, argtypes in _SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError as e:
                raise KernelLibraryError(f"{path} has no symbol {name}; rebuild it") from e
            fn.argtypes = argtypes
            fn.restype = C.c_int
        _lib = lib
        return lib


def register(name: str, argtypes: list) -> None:
    """Declare another entry point (used by kernel files added later)."""
    _SIGNATURES[name] = argtypes
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = C.c_int


launches = 0   # kernels launched so far through `call`


KERNELS_PER_CALL = {"ib_sample_rows": 3, "ib_attention_decode": 2, "ib_attention_decode_stream": 2, "ib_attention_decode_fused": 2}


_entry: dict = {}   # name -> (function, kernels it launches)


def call(name: str, *args) -> None:
    global launches
    e = _entry.get(name)
    if e is None:
        e = _entry[name] = (getattr(load(), name), KERNELS_PER_CALL.get(name, 1))
    launches += e[1]
    if e[0](*args) != 0:
        raise KernelError(load().ib_last_error().decode(errors="replace"))

"""The host-side C++ library (csrc/host/*.cpp), loaded with ctypes: page pools, block tables and the scheduler's decisions."""
from __future__ import annotations

import ctypes as C
from typing import Optional

_lib: Optional[C.CDLL] = None

_i, _p = C.c_int, C.c_void_p
_SIGNATURES = {
    "ibh_last_error": (C.c_char_p, []),
    "ibh_pool_new": (_p, [_i]), "ibh_pool_free": (None, [_p]), "ibh_pool_num_pages": (_i, [_p]), "ibh_pool_free_pages": (_i, [_p]),
    "ibh_pool_allocate": (_i, [_p]), "ibh_pool_share": (_i, [_p, _i]), "ibh_pool_release": (_i, [_p, _i]), "ibh_pool_refcount": (_i, [_p, _i]),
    "ibh_pool_check": (_i, [_p]),
    "ibh_cache_new": (_p, [_i, C.POINTER(_i), _i, _i, _i, _i]), "ibh_cache_free": (None, [_p]), "ibh_cache_pool": (_p, [_p, _i]),
    "ibh_cache_tables": (C.POINTER(_i), [_p]), "ibh_cache_table_width": (_i, [_p]), "ibh_cache_free_slots": (_i, [_p]),
    "ibh_cache_admit": (_i, [_p]), "ibh_cache_length": (_i, [_p, _i]), "ibh_cache_pages_missing": (None, [_p, _i, _i, _i, C.POINTER(_i)]),
    "ibh_cache_extend": (_i, [_p, _i, _i]), "ibh_cache_shrink_to_committed": (_i, [_p, _i]), "ibh_cache_commit": (_i, [_p, _i, _i]),
    "ibh_cache_release": (_i, [_p, _i]), "ibh_cache_fill_rows": (_i, [_p, C.POINTER(_i), _i, C.POINTER(_i), C.POINTER(C.POINTER(_i))]),
    "ibh_cache_check": (_i, [_p]),
    "ibh_sched_new": (_p, [_p, _i, _i, _i, _i, _i]), "ibh_sched_free": (None, [_p]), "ibh_sched_submit": (_i, [_p, _i, _i]),
    "ibh_sched_cancel": (_i, [_p, _i]), "ibh_sched_n_waiting": (_i, [_p]), "ibh_sched_n_running": (_i, [_p]), "ibh_sched_steady": (_i, [_p]),
    "ibh_sched_waiting": (None, [_p, C.POINTER(_i)]), "ibh_sched_running": (None, [_p, C.POINTER(_i)]),
    "ibh_sched_total_preemptions": (C.c_longlong, [_p]), "ibh_sched_get": (None, [_p, _i, C.POINTER(C.c_longlong)]),
    "ibh_sched_plan": (None, [_p, C.POINTER(_i), C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]), "ibh_sched_computed": (None, [_p, _i, _i]),
    "ibh_sched_accept": (_i, [_p, _i, _i]),
}


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        from ..kernels.build import build_host
        lib = C.CDLL(str(build_host()))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def last_error() -> str:
    return (load().ibh_last_error() or b"").decode()

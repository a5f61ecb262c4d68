"""ctypes bindings of the host core (pulsarlm_b200/csrc_host): the library is built
with g++ on first use; there is no Python fallback for what it does."""

from __future__ import annotations

import ctypes
import threading

from ..kernels import build

_I32, _I64, _PTR = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p
_lib = None
_lock = threading.Lock()
ABI_VERSION = 5

# return codes of csrc_host/host_core.hpp
OK, NO_ROOM = 0, 1
UNKNOWN_REQUEST, ALREADY_OPEN, SHRINK, NOT_RESERVED, BAD_PAGE, BAD_ARGUMENT = -1, -2, -3, -4, -5, -6
NO_SLOT = -100
REASONS = {0: "stop", 1: "length", 2: "cancelled", 3: "oom"}

_SIGNATURES = {
    "plh_pool_create": ([_I32], _PTR),
    "plh_pool_destroy": ([_PTR], None),
    "plh_pool_take": ([_PTR, _I32, _PTR], _I32),
    "plh_pool_give": ([_PTR, _PTR, _I32], _I32),
    "plh_pool_stat": ([_PTR, _I32], _I32),
    "plh_pool_is_held": ([_PTR, _I32], _I32),
    "plh_cache_create": ([_I32, _PTR, _I32, _PTR, _I32, _I32], _PTR),
    "plh_cache_destroy": ([_PTR], None),
    "plh_cache_open": ([_PTR, _I64], _I32),
    "plh_cache_is_open": ([_PTR, _I64], _I32),
    "plh_cache_slot": ([_PTR, _I64], _I32),
    "plh_cache_length": ([_PTR, _I64], _I64),
    "plh_cache_reserve": ([_PTR, _I64, _I64], _I32),
    "plh_cache_commit": ([_PTR, _I64, _I64], _I32),
    "plh_cache_close": ([_PTR, _I64], _I32),
    "plh_cache_pages_needed": ([_PTR, _I64, _I64], _I32),
    "plh_cache_table_row": ([_PTR, _I32, _I64, _PTR, _I32], _I32),
    "plh_cache_held_pages": ([_PTR, _I32, _I64, _PTR, _I32], _I32),
    "plh_cache_take_fresh": ([_PTR, _I32, _PTR, _I32], _I32),
    "plh_cache_free_pages": ([_PTR], _I32),
    "plh_cache_slots_used": ([_PTR], _I32),
    "plh_cache_pool_stat": ([_PTR, _I32, _I32], _I32),
    "plh_cache_pool_is_held": ([_PTR, _I32, _I32], _I32),
    "plh_cache_open_requests": ([_PTR, _PTR, _I32], _I32),
    "plh_cache_fill_tables": ([_PTR, _I32, _PTR, _I32, _PTR, _I32, _PTR], _I32),
    "plh_fill_random": ([_PTR, _I64, _I32, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_float, ctypes.c_float], _I32),
    "plh_decode_work_items": ([_PTR, _I32, _I32, _I32, _I32, _I32, _PTR, _I32, _PTR], _I32),
    "plh_cache_reserve_many": ([_PTR, _PTR, _PTR, _I32, _PTR, _PTR, _PTR], _I32),
    "plh_cache_commit_many": ([_PTR, _PTR, _PTR, _I32], _I32),
    "plh_sched_create": ([_PTR, _I32, _I32], _PTR),
    "plh_sched_destroy": ([_PTR], None),
    "plh_sched_set_stop_ids": ([_PTR, _PTR, _I32], None),
    "plh_sched_add": ([_PTR, _I64, _I32, _I64, _I32], _I32),
    "plh_sched_cancel": ([_PTR, _I64], _I32),
    "plh_sched_has_work": ([_PTR], _I32),
    "plh_sched_preemptions": ([_PTR], _I32),
    "plh_sched_plan": ([_PTR, _PTR, _PTR, _PTR, _I32, _PTR], _I32),
    "plh_sched_finish_step": ([_PTR, _PTR, _PTR, _I32, _PTR, _I32], _I32),
    "plh_sched_advance": ([_PTR, _PTR, _I32], None),
    "plh_sched_settle": ([_PTR, _PTR, _PTR, _I32, _PTR, _I32], _I32),
}


def library() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            lib = ctypes.CDLL(build.host_library_path(build=True))
            lib.plh_abi_version.restype = _I32
            if lib.plh_abi_version() != ABI_VERSION:
                raise RuntimeError("the host core's ABI version does not match the package; delete the build folder")
            for name, (argtypes, restype) in _SIGNATURES.items():
                fn = getattr(lib, name)
                fn.argtypes = argtypes
                fn.restype = restype
            _lib = lib
    return _lib

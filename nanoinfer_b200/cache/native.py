"""The compiled host runtime behind the cache and scheduler classes (csrc/host_runtime.cpp),
loaded once."""
from __future__ import annotations

import ctypes

_I, _LL, _P = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
_IP = ctypes.POINTER(ctypes.c_int32)
_LP = ctypes.POINTER(ctypes.c_longlong)

_SIGNATURES = {
    "ni_pool_create": ([_I], _P),
    "ni_pool_destroy": ([_P], None),
    "ni_pool_num_free": ([_P], _I),
    "ni_pool_is_taken": ([_P, _I], _I),
    "ni_pool_take": ([_P, _I, _IP], _I),
    "ni_pool_give_back": ([_P, _IP, _I], _I),
    "ni_pool_last_error": ([_P], ctypes.c_char_p),
    "ni_cache_create": ([_I, _IP, _IP, _I, _I, _I], _P),
    "ni_cache_destroy": ([_P], None),
    "ni_cache_last_error": ([_P], ctypes.c_char_p),
    "ni_cache_table_width": ([_P], _I),
    "ni_cache_table_version": ([_P], _LL),
    "ni_cache_mirror": ([_P, _I], _IP),
    "ni_cache_has": ([_P, _LL], _I),
    "ni_cache_num_free_slots": ([_P], _I),
    "ni_cache_admit": ([_P, _LL], _I),
    "ni_cache_slot": ([_P, _LL], _I),
    "ni_cache_length": ([_P, _LL], _I),
    "ni_cache_pages_needed": ([_P, _LL, _I, _IP], _I),
    "ni_cache_append": ([_P, _LL, _I], _I),
    "ni_cache_needs_page_for_one": ([_P, _LL], _I),
    "ni_cache_append_one": ([_P, _LL], _I),
    "ni_cache_release_passed": ([_P, _LL], _I),
    "ni_cache_free": ([_P, _LL], _I),
    "ni_cache_check": ([_P], _I),
    "ni_cache_pool_num_pages": ([_P, _I], _I),
    "ni_cache_pool_num_free": ([_P, _I], _I),
    "ni_cache_pool_is_taken": ([_P, _I, _I], _I),
    "ni_cache_block_table": ([_P, _LL, _I, _IP, _I], _I),
    "ni_sched_create": ([_P, _I, _I, _I, _I], _P),
    "ni_sched_destroy": ([_P], None),
    "ni_sched_add": ([_P, _LL, _I, _I], _I),
    "ni_sched_has_work": ([_P], _I),
    "ni_sched_schedule": ([_P], _I),
    "ni_sched_result": ([_P, _I, _LP, _I], _I),
    "ni_sched_advance": ([_P, _I, _LP, _IP, _I, _LP], _I),
    "ni_sched_commit": ([_P, _LL, _I], _I),
    "ni_sched_abort": ([_P, _LL], _I),
    "ni_sched_can_continue": ([_P, _LP, _I], _I),
    "ni_sched_get": ([_P, _LL, _I], _I),
    "ni_sched_stat": ([_P, _I], _LL),
}

ERR_ARGUMENT, ERR_OUT_OF_PAGES, ERR_PAGE, ERR_LIMIT, ERR_NO_SLOT, ERR_INCONSISTENT = -1, -2, -3, -4, -5, -6

_lib = None


def lib() -> ctypes.CDLL:
    """The host library, compiled at its first use (a C++17 compiler, no CUDA needed)."""
    global _lib
    if _lib is None:
        from ..kernels import build
        handle = ctypes.CDLL(build.ensure_built(["host_runtime"])["host_runtime"])
        for name, (argtypes, restype) in _SIGNATURES.items():
            f = getattr(handle, name)
            f.argtypes, f.restype = argtypes, restype
        _lib = handle
    return _lib

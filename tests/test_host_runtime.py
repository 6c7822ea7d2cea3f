"""The compiled host runtime through its C interface (what the Python classes wrap): error codes
leave the books unchanged, the scheduler's decisions are read back as plain arrays."""
import ctypes

import pytest

from nanoinfer_b200.cache import native


def _cache(lib, pages=(8,), windows=(-1,), page_size=4, max_requests=3, max_tokens=32):
    n = len(pages)
    return lib.ni_cache_create(n, (ctypes.c_int32 * n)(*pages), (ctypes.c_int32 * n)(*windows), page_size,
                               max_requests, max_tokens)


def test_cache_error_codes_change_nothing():
    lib = native.lib()
    c = _cache(lib)
    assert lib.ni_cache_admit(c, 7) == 0                 # slots, like pages, are handed out from 0 upwards
    assert lib.ni_cache_admit(c, 7) == native.ERR_ARGUMENT and b"already" in lib.ni_cache_last_error(c)
    assert lib.ni_cache_append(c, 99, 1) == native.ERR_ARGUMENT          # unknown request
    assert lib.ni_cache_append(c, 7, 33) == native.ERR_LIMIT
    assert lib.ni_cache_append(c, 7, 30) == 0 and lib.ni_cache_pool_num_free(c, 0) == 0
    version = lib.ni_cache_table_version(c)
    assert lib.ni_cache_admit(c, 8) == 1
    assert lib.ni_cache_append(c, 8, 1) == native.ERR_OUT_OF_PAGES
    assert lib.ni_cache_length(c, 8) == 0 and lib.ni_cache_pool_num_free(c, 0) == 0
    assert lib.ni_cache_table_version(c) == version + 1                  # the admission only
    assert lib.ni_cache_check(c) == 0
    assert lib.ni_cache_free(c, 7) == 0 and lib.ni_cache_free(c, 7) == native.ERR_ARGUMENT
    assert lib.ni_cache_pool_num_free(c, 0) == 8 and lib.ni_cache_num_free_slots(c) == 2
    out = (ctypes.c_int32 * 8)()
    assert lib.ni_cache_append(c, 8, 5) == 0 and lib.ni_cache_block_table(c, 8, 0, out, 8) == 2
    assert list(out[:2]) == [7, 6]                                       # freed pages come back last in, first out
    lib.ni_cache_destroy(c)
    assert _cache(lib, pages=(0,)) is None and _cache(lib, page_size=0) is None


def test_windowed_group_gives_pages_back_through_the_c_interface():
    lib = native.lib()
    c = _cache(lib, pages=(16, 16), windows=(-1, 6), page_size=4, max_tokens=64)
    lib.ni_cache_admit(c, 1)
    assert lib.ni_cache_append(c, 1, 20) == 0
    assert lib.ni_cache_release_passed(c, 1) == 3        # keys below 20 - 6 + 1 = 15: pages 0, 1, 2 of the windowed group
    assert lib.ni_cache_pool_num_free(c, 0) == 11 and lib.ni_cache_pool_num_free(c, 1) == 14
    out = (ctypes.c_int32 * 16)()
    assert lib.ni_cache_block_table(c, 1, 1, out, 16) == 5 and list(out[:5])[:3] == [-1, -1, -1]
    assert lib.ni_cache_check(c) == 0
    assert lib.ni_cache_free(c, 1) == 0 and lib.ni_cache_pool_num_free(c, 1) == 16
    lib.ni_cache_destroy(c)


def test_scheduler_decisions_as_arrays():
    lib = native.lib()
    c = _cache(lib, pages=(64,), max_requests=4, max_tokens=128)
    s = lib.ni_sched_create(c, 8, 4, 8, 12)              # batch 8, sequences 4, portions of 8, budget 12
    assert lib.ni_sched_add(s, 0, 20, 3) == 0 and lib.ni_sched_add(s, 1, 5, 3) == 0
    assert lib.ni_sched_add(s, 1, 5, 3) == native.ERR_ARGUMENT and lib.ni_sched_add(s, 2, 0, 3) == native.ERR_ARGUMENT
    buf = (ctypes.c_longlong * 8)()
    assert lib.ni_sched_schedule(s) == 2
    assert lib.ni_sched_result(s, 0, buf, 8) == 2 and list(buf[:2]) == [0, 1]
    assert lib.ni_sched_result(s, 1, buf, 8) == 2 and list(buf[:2]) == [8, 4]      # 12 tokens: 8 for the first, 4 left
    assert lib.ni_sched_result(s, 2, buf, 8) == 0 and lib.ni_sched_result(s, 3, buf, 8) == 0
    assert lib.ni_sched_get(s, 0, 0) == 1 and lib.ni_sched_get(s, 0, 5) == 20     # running, 20 tokens to go
    ids = (ctypes.c_longlong * 2)(0, 1)
    counts = (ctypes.c_int32 * 2)(8, 4)
    assert lib.ni_sched_advance(s, 2, ids, counts, 0, ids) == 0
    assert lib.ni_sched_get(s, 0, 1) == 8 and lib.ni_sched_get(s, 1, 5) == 1
    assert lib.ni_sched_commit(s, 1, 0) == native.ERR_ARGUMENT                    # nothing on the way for request 1
    assert lib.ni_sched_stat(s, 0) == 2 and lib.ni_sched_stat(s, 3) == 2 and lib.ni_sched_has_work(s) == 1
    lib.ni_sched_destroy(s)
    lib.ni_cache_destroy(c)

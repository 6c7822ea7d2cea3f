"""Cache manager on the host: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back early; slots."""
import random

import numpy as np
import pytest

from nanoinfer_b200.cache import (CacheError, CacheManager, GroupSpec, OutOfPages, PagePool,
                                  PagePoolError)


def test_pool_order_reuse_and_errors():
    pool = PagePool(4)
    assert pool.take(3) == [0, 1, 2]            # first pops are 0, 1, 2 (block_manager.cpp:23-28)
    pool.give_back([1])
    assert pool.take(1) == [1]                  # a page given back is the next one handed out
    with pytest.raises(OutOfPages):
        pool.take(2)
    assert pool.num_free == 1                   # a refused request takes nothing
    with pytest.raises(PagePoolError):
        pool.give_back([3])                     # never taken
    pool.give_back([0])
    with pytest.raises(PagePoolError):
        pool.give_back([0])                     # freed twice
    with pytest.raises(PagePoolError):
        pool.give_back([2, 2])                  # twice in one call: nothing changes
    assert pool.is_taken(2)
    with pytest.raises(PagePoolError):
        pool.give_back([9])


def test_append_takes_pages_on_demand():
    cm = CacheManager([GroupSpec(2, 16)], [8], page_size=4, max_requests=2, max_tokens_per_request=32)
    slot = cm.admit("a")
    assert cm.pages_needed("a", 5) == [2]
    cm.append("a", 5)
    assert cm.block_table("a") == [0, 1] and cm.length("a") == 5
    cm.append("a", 3)                            # fills page 1 exactly
    assert cm.block_table("a") == [0, 1]
    cm.append("a", 1)
    assert cm.block_table("a") == [0, 1, 2]
    assert list(cm.mirror[0][slot, :4]) == [0, 1, 2, -1]
    cm.admit("b")
    with pytest.raises(OutOfPages):
        cm.append("b", 4 * 6)                    # needs 6, 5 free: nothing taken
    assert cm.length("b") == 0 and cm.num_free_pages() == 5
    with pytest.raises(CacheError, match="max_tokens_per_request"):
        cm.append("a", 100)
    with pytest.raises(CacheError, match="no free request slot"):
        cm.admit("c")
    with pytest.raises(CacheError, match="already admitted"):
        cm.admit("a")
    cm.free("a")
    with pytest.raises(CacheError, match="not admitted"):
        cm.free("a")
    cm.check_consistency()
    assert cm.num_free_pages() == 8 and np.all(cm.mirror[0][slot] == -1)


def test_window_gives_pages_back_early():
    cm = CacheManager([GroupSpec(1, 16, None), GroupSpec(1, 16, 6)], [64, 64], page_size=4,
                      max_requests=1, max_tokens_per_request=128)
    cm.admit("a")
    peak = 0
    for step in range(40):
        cm.append("a", 3)
        peak = max(peak, cm.pools[1].num_taken)
        cm.release_passed("a")
        cm.check_consistency()
        n = cm.length("a")
        table = cm.block_table("a", 1)
        first_needed = max(0, n - 6 + 1) // 4           # page of the oldest key the next query sees
        assert all(p == -1 for p in table[:first_needed]) and all(p >= 0 for p in table[first_needed:])
    assert cm.pools[0].num_taken == 30                  # the full group keeps everything
    assert peak <= 4                                    # window 6 + portion 3, pages of 4
    cm.free("a")
    assert cm.pools[0].num_free == 64 and cm.pools[1].num_free == 64


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    cm = CacheManager([GroupSpec(2, 16, None), GroupSpec(2, 16, 10)], [40, 12], page_size=4,
                      max_requests=5, max_tokens_per_request=64)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and cm.num_free_slots > 0:
            cm.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.8 and live:
            r = rng.choice(list(live))
            n = rng.randint(1, 9)
            if live[r] + n > 64:
                with pytest.raises(CacheError):
                    cm.append(r, n)
            elif cm.can_append(r, n):
                cm.append(r, n)
                live[r] += n
                cm.release_passed(r)
            else:
                before = [p.num_free for p in cm.pools]
                with pytest.raises(OutOfPages):
                    cm.append(r, n)
                assert before == [p.num_free for p in cm.pools] and cm.length(r) == live[r]
        elif live:
            r = rng.choice(list(live))
            cm.free(r)
            del live[r]
        cm.check_consistency()
        for r, n in live.items():
            assert cm.length(r) == n
            assert len(cm.block_table(r, 0)) == -(-n // 4)
    for r in list(live):
        cm.free(r)
    assert all(p.num_free == p.num_pages for p in cm.pools) and cm.num_free_slots == 5

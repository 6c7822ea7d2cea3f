"""Host-side launch decisions that need no GPU: how the decode attention cuts a context into
splits, and which prefill attention kernel takes which head layout."""
import itertools

import pytest

from nanoinfer_b200.kernels import ops


@pytest.mark.parametrize("head_dim", [64, 128])
def test_decode_splits_are_bounded_and_leave_no_empty_split(head_dim):
    for n_items, n_kv, ctx in itertools.product([1, 2, 3, 8, 16, 19, 24, 32, 37, 40, 56, 64, 96, 128, 300],
                                                [1, 2, 8], [1, 63, 64, 65, 500, 2112, 3072, 4096, 16384, 131072]):
        s = ops.decode_splits(n_items, n_kv, head_dim, ctx, n_sms=148)
        assert 1 <= s <= 64
        chunks = -(-ctx // 64)
        assert s <= chunks                                  # a split holds at least one 64-key chunk
        per_split = -(-chunks // s)                          # the kernel's own cut of the longest context
        assert -(-chunks // per_split) == s                  # ... leaves no split of it empty
        if s > 1:
            assert per_split * 64 >= 256 or s == chunks      # no splits of a handful of keys


def test_decode_splits_follow_the_resident_blocks():
    # few pairs: as many fat blocks as fit at three per SM, of at least 256 / 384 keys
    assert ops.decode_splits(1, 8, 64, 3072, n_sms=148) == 12
    assert ops.decode_splits(8, 8, 64, 3072, n_sms=148) == 6
    assert 8 * 8 * ops.decode_splits(8, 8, 64, 131072, n_sms=148) <= 3 * 148
    # middle batches of 64-wide heads: lean blocks, four per SM
    assert ops.decode_splits(32, 8, 64, 3072, n_sms=148) == 2 and 32 * 8 * 2 <= 4 * 148
    assert ops.decode_splits(24, 8, 64, 3072, n_sms=148) == 3
    # large batches: one block per pair with heads of 64; with heads of 128 the last wave is filled
    assert ops.decode_splits(64, 8, 64, 3072, n_sms=148) == 1
    assert ops.decode_splits(64, 8, 128, 7168, n_sms=148) == 4
    assert ops.decode_splits(64, 8, 128, 300, n_sms=148) == 1           # too short to split
    assert ops.decode_splits(32, 8, 128, 3072, n_sms=148) == 1          # three per SM: 256 blocks are one wave


def test_tensor_core_prefill_attention_cases():
    assert ops.attention_prefill_tc_supports(32, 8, 64, 16)
    assert ops.attention_prefill_tc_supports(24, 8, 128, 16)        # odd group of three
    assert ops.attention_prefill_tc_supports(5, 1, 64, 128)
    assert not ops.attention_prefill_tc_supports(8, 8, 64, 16)      # one query head per kv head
    assert not ops.attention_prefill_tc_supports(8, 3, 64, 16)      # heads do not divide
    assert not ops.attention_prefill_tc_supports(8, 2, 96, 16)      # head size
    assert not ops.attention_prefill_tc_supports(8, 2, 64, 4)       # page size
    assert not ops.attention_prefill_tc_supports(8, 2, 64, 48)

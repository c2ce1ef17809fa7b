"""Key splits of the decode attention: chosen from the batch size and the context class, within bounds, and as measured."""
from functools import partial

from imp_b200.ops.attention import DECODE_MAX_SPLITS
from imp_b200.ops.attention import decode_splits as device_splits

SMS = 148                                               # a B200; another count is tried below
decode_splits = partial(device_splits, sm_count=SMS)


def test_splits_fill_the_device_for_small_batches_and_stop_for_large_ones():
    slots = 2 * SMS
    for batch in range(1, 300):
        s = decode_splits(batch, 8, 4, 16)
        assert 1 <= s <= DECODE_MAX_SPLITS
        base = batch * 8
        if base <= slots:
            assert base * s <= slots and s & (s - 1) == 0           # resident at once, a power of two
            assert base * s * 2 > slots or s == DECODE_MAX_SPLITS   # and no further doubling would fit
    # measured at 8 kv heads of 128, context 4096: 64 sequences unsplit beat 4 splits, 40 and 48 do not
    assert decode_splits(64, 8, 4, 16) == 1
    assert decode_splits(32, 8, 4, 16) == 1
    assert decode_splits(40, 8, 4, 16) > 1 and decode_splits(48, 8, 4, 16) > 1
    assert decode_splits(8, 8, 4, 16) == 4 and decode_splits(1, 8, 4, 16) == 32


def test_groups_above_sixteen_count_as_several_row_tiles():
    assert decode_splits(4, 2, 40, 16) == decode_splits(4, 6, 4, 16)


def test_other_page_sizes_use_the_direct_kernel_rule():
    assert decode_splits(1, 8, 4, 3) >= 1
    assert decode_splits(1000, 8, 4, 3) == 1


def test_the_rule_scales_with_the_number_of_sms():
    for sms in (132, 74, 20):
        slots = 2 * sms
        for batch in (1, 3, 8, 17):
            s = device_splits(batch, 8, 4, 16, sm_count=sms)
            base = batch * 8
            if base <= slots:
                assert base * s <= slots and (base * s * 2 > slots or s == DECODE_MAX_SPLITS)
    assert device_splits(8, 8, 4, 16, sm_count=74) == 2


def test_large_batches_split_by_context_as_measured():
    """Whole decode steps of the 8B shape (8 kv heads of 128) were timed at 36 to 112 sequences with 1 to 8 splits:
    at contexts of 1,024 the unsplit kernel won everywhere; at 4,096 splits won where the last wave of CTAs is short."""
    for batch in (36, 40, 48, 56, 72, 80, 96, 112, 128):
        assert decode_splits(batch, 8, 4, 16, context=1024) == 1
        assert decode_splits(batch, 8, 4, 16, context=256) == 1
    fastest = {36: 1, 40: 3, 48: 2, 72: 1, 80: 2, 96: 1, 112: 2}
    for batch, splits in fastest.items():
        assert decode_splits(batch, 8, 4, 16, context=4096) == splits
        assert decode_splits(batch, 8, 4, 16) == splits                  # no context given: 4,096
    # long contexts: the fixed cost of a split vanishes, a short last wave is always worth splitting
    assert decode_splits(40, 8, 4, 16, context=32768) > 1
    assert decode_splits(74, 8, 4, 16, context=32768) == 1               # 592 CTAs: two full waves


def test_short_contexts_get_fewer_splits_at_small_batches():
    assert decode_splits(1, 8, 4, 16, context=256) == 2 and decode_splits(1, 8, 4, 16, context=1024) == 8
    assert decode_splits(1, 8, 4, 16, context=4096) == 32 and decode_splits(8, 8, 4, 16, context=128) == 1

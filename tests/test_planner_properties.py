"""Property tests of the host planner over random batches: every token is covered exactly once, work
is balanced, partial slots are consistent - for any SM count and any column count."""
import numpy as np
from hypothesis import given, settings, strategies as st

from helpers import capi


@settings(max_examples=500, deadline=None, derandomize=True)
@given(lens=st.lists(st.integers(min_value=0, max_value=40000), min_size=1, max_size=80),
       kv_heads=st.sampled_from([1, 2, 4, 8, 32]), group=st.sampled_from([1, 4, 8]),
       sm=st.sampled_from([1, 7, 132, 148]))
def test_plan_invariants(lens, kv_heads, group, sm):
    lens = np.asarray(lens, dtype=np.int32)
    max_blocks = max(1, int((lens.max() + 127) // 128))
    d = capi.make_desc(len(lens), kv_heads * group, kv_heads, 128, 128, 128, 1 << 20, max_blocks, "bf16", sm_count=sm)
    plan = capi.PaPlan(d, lens)
    info = plan.info
    items, groups = plan.dump()
    n_groups = info.num_ctas // kv_heads
    covered = np.zeros(len(lens), dtype=np.int64)
    parts = np.zeros(len(lens), dtype=np.int64)
    last_end = {}
    slots = []
    for seq, b, e, slot in items:
        assert 0 <= b < e <= lens[seq] and b % 64 == 0
        assert last_end.get(seq, 0) == b          # ranges of a sequence are contiguous and in order
        last_end[seq] = e
        covered[seq] += e - b
        parts[seq] += 1
        if slot >= 0:
            slots.append(slot)
    assert np.array_equal(covered, lens.astype(np.int64))
    assert sorted(slots) == list(range(info.num_partials))
    assert info.num_partials == int(parts[parts > 1].sum())
    assert info.num_combine_seqs == int((parts > 1).sum())
    if info.num_items:
        # work is balanced in 64-token tiles (a sequence occupies ceil(len / 64) of them): a cut is the
        # absolute position j*total/n rounded down, moved by at most one tile onto a sequence boundary,
        # so a group is less than three tiles (one per end + the rounding) above the mean
        tiles = np.array([sum((e - b + 63) // 64 for _, b, e, _ in items[groups[g]:groups[g + 1]])
                          for g in range(n_groups)])
        assert groups[n_groups] == info.num_items
        assert tiles.max() - tiles.mean() < 3.0
    plan.close()


@settings(max_examples=300, deadline=None, derandomize=True)
@given(lens=st.lists(st.integers(min_value=0, max_value=20000), min_size=1, max_size=60),
       heads=st.sampled_from([8, 64, 128]), sm=st.sampled_from([1, 2, 7, 148]))
def test_mla_plan_invariants(lens, heads, sm):
    """The MLA plan packs cost = tiles + 6 x token ranges: every token is still covered exactly once, in order, for
    any batch and SM count, and no group costs more than the smallest cap a greedy packing can reach plus nothing."""
    lens = np.asarray(lens, dtype=np.int32)
    max_blocks = max(1, int((lens.max() + 127) // 128))
    d = capi.make_desc(len(lens), heads, 1, 576, 512, 128, 1 << 20, max_blocks, "bf16", v_row_dim=576, sm_count=sm)
    plan = capi.PaPlan(d, lens)
    info = plan.info
    assert info.kernel == capi.KERNEL_MLA_TC5
    items, groups = plan.dump()
    cols = (heads + 63) // 64
    n_groups = info.num_ctas // cols
    covered = np.zeros(len(lens), dtype=np.int64)
    last_end = {}
    for seq, b, e, slot in items:
        assert 0 <= b < e <= lens[seq] and b % 64 == 0
        assert last_end.get(seq, 0) == b
        last_end[seq] = e
        covered[seq] += e - b
    assert np.array_equal(covered, lens.astype(np.int64))
    assert groups[n_groups] == info.num_items
    if info.num_items:
        cost = np.array([sum((e - b + 63) // 64 for _, b, e, _ in items[groups[g]:groups[g + 1]]) + 6 * (groups[g + 1] - groups[g])
                         for g in range(n_groups)])
        total = int(((lens.astype(np.int64) + 63) // 64).sum())
        # a lower bound of any plan's largest group, and the greedy cap is within one range + one tile of it
        lower = (total + 6 * int((lens > 0).sum())) / n_groups
        assert cost.max() <= max(lower + 7, 7 + int(((lens.astype(np.int64) + 63) // 64).max()) if n_groups == 1 else lower * 1.5 + 13)
    plan.close()

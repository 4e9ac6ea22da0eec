"""The host-side cut of a step into attention work items: every packed row of every entry is
covered exactly once per split, by a tile of the right kind."""

from __future__ import annotations

import numpy as np
import pytest

from rapid_llm_b200.ops import kernels
from rapid_llm_b200.parts.attention import DEFAULT_DECODE_CLUSTERS, DEFAULT_SMS, MAX_SPLITS, AttentionItems
from rapid_llm_b200.parts.base import StepShape


def covered(items: np.ndarray, tile_rows: int, rows_of_entry: np.ndarray, splits: int) -> dict:
    seen: dict[tuple[int, int, int], int] = {}
    for entry, row0, split, _ in items.tolist():
        assert 0 <= split < splits and row0 % tile_rows == 0 and row0 < rows_of_entry[entry]
        for row in range(row0, min(row0 + tile_rows, int(rows_of_entry[entry]))):
            seen[(entry, row, split)] = seen.get((entry, row, split), 0) + 1
    return seen


@pytest.mark.parametrize("group,kv_heads", [(1, 4), (2, 2), (4, 8), (6, 1), (20, 2)])
@pytest.mark.parametrize("seed", range(5))
def test_every_row_is_covered_once_per_split(group, kv_heads, seed):
    rng = np.random.default_rng(seed)
    entries = int(rng.integers(1, 9))
    lengths = rng.choice([1, 1, 1, 2, 3, 16, 17, 100, 700], size=entries).astype(np.int32)
    starts = rng.integers(0, 3000, size=entries).astype(np.int32)
    planner = AttentionItems(group, kv_heads)
    plan = planner.plan(StepShape(lengths, starts, decode_only=bool(lengths.max() == 1)))
    splits = plan["splits"]
    assert 1 <= splits <= MAX_SPLITS
    rows = lengths.astype(np.int64) * group
    seen = covered(plan["chunk_items"], kernels.CHUNK_TILE_ROWS, rows, splits)
    for key, count in covered(plan["decode_items"], kernels.DECODE_TILE_ROWS, rows, splits).items():
        seen[key] = seen.get(key, 0) + count
    assert all(count == 1 for count in seen.values())
    assert len(seen) == int(rows.sum()) * splits
    words = 4 * (len(plan["chunk_items"]) + len(plan["decode_items"]))
    assert words <= planner.capacity(int(lengths.sum()), entries)
    for entry in plan["decode_items"][:, 0]:
        assert lengths[entry] == 1 or rows[entry] <= kernels.DECODE_TILE_ROWS
    for entry in plan["chunk_items"][:, 0]:
        assert lengths[entry] > 1 and rows[entry] > kernels.DECODE_TILE_ROWS


def test_a_decode_only_step_splits_by_the_number_of_entries_alone():
    planner = AttentionItems(4, 8)
    short = planner.plan(StepShape(np.ones(4, np.int32), np.full(4, 3, np.int32), decode_only=True))
    long = planner.plan(StepShape(np.ones(4, np.int32), np.full(4, 7000, np.int32), decode_only=True))
    assert short["splits"] == long["splits"] == min(MAX_SPLITS, DEFAULT_SMS // (4 * 8))
    assert np.array_equal(short["decode_items"], long["decode_items"])
    full = planner.plan(StepShape(np.ones(64, np.int32), np.full(64, 1000, np.int32), decode_only=True))
    assert full["splits"] == 1


def test_decode_steps_of_the_cluster_kernel_take_the_largest_cluster_that_runs_in_one_round():
    planner = AttentionItems(4, 8, 128)      # 8 kv heads: a request is 8 tiles
    for entries, want in [(1, 10), (2, 6), (3, 5), (4, 4), (5, 3), (6, 2), (8, 2), (9, 2), (10, 1), (16, 1)]:
        plan = planner.plan(StepShape(np.ones(entries, np.int32), np.full(entries, 5000, np.int32), True, page_size=16))
        assert plan["splits"] == want, entries
        assert DEFAULT_DECODE_CLUSTERS[want] >= entries * 8          # all of the step's clusters run at one time
    # another GPU's table: few clusters of any size above two
    small = AttentionItems(4, 8, 128, decode_clusters={1: 60, 2: 30, 3: 4})
    assert small.plan(StepShape(np.ones(1, np.int32), np.full(1, 5000, np.int32), True, page_size=16))["splits"] == 2
    other_page = planner.plan(StepShape(np.ones(1, np.int32), np.full(1, 500, np.int32), True, page_size=24))
    assert other_page["splits"] == MAX_SPLITS            # the mma.sync tiles merge in a kernel of their own


def test_padding_rows_of_a_decode_bucket_do_not_count_as_clusters():
    planner = AttentionItems(4, 8, 128)
    lengths, starts = np.ones(8, np.int32), np.array([5000] * 5 + [0] * 3, np.int32)
    padded = planner.plan(StepShape(lengths, starts, True, page_size=16, padding=3))
    full = planner.plan(StepShape(lengths, np.full(8, 5000, np.int32), True, page_size=16))
    assert (padded["splits"], full["splits"]) == (3, 2)
    short = planner.plan(StepShape(lengths, np.array([1000] * 5 + [0] * 3, np.int32), True, page_size=16, padding=3))
    assert short["splits"] == 2                     # on short contexts the extra round of padding clusters costs more
    assert len(padded["decode_items"]) == 8 * 3 and list(padded["decode_items"][-9:, 0]) == [5, 5, 5, 6, 6, 6, 7, 7, 7]


def test_decode_steps_of_the_cluster_kernel_split_no_finer_than_the_context_has_blocks():
    planner = AttentionItems(4, 8, 128)
    seen = []
    for context in (1, 100, 127, 128, 300, 511, 512, 1000, 1023, 1024, 2047, 2048, 30000):
        plan = planner.plan(StepShape(np.ones(1, np.int32), np.full(1, context, np.int32), True, page_size=16))
        seen.append(plan["splits"])
    assert seen == [1, 1, 1, 2, 2, 4, 4, 8, 8, 8, 10, 10, 10]    # the new token's key counts: 129 keys are two blocks
    assert len(set(seen)) <= 5                                    # so few graphs per batch size


def test_short_contexts_are_not_split_in_a_mixed_step():
    planner = AttentionItems(4, 8)
    plan = planner.plan(StepShape(np.array([30, 1], np.int32), np.array([0, 100], np.int32), decode_only=False))
    assert plan["splits"] == 1
    plan = planner.plan(StepShape(np.array([30, 1], np.int32), np.array([4000, 100], np.int32), decode_only=False))
    assert plan["splits"] > 1


def test_chunk_tiles_follow_the_kernel_that_will_run():
    planner = AttentionItems(4, 8, 128)
    whole = StepShape(np.asarray([2048], dtype=np.int32), np.asarray([0], dtype=np.int32), False, page_size=16)
    plan = planner.plan(whole)
    assert plan["chunk_rows"] == kernels.CHUNK_TILE_ROWS_TC and plan["splits"] == 1
    assert len(plan["chunk_items"]) == 2048 * 4 // 256
    # the longest tiles first
    assert list(plan["chunk_items"][:, 1]) == sorted(plan["chunk_items"][:, 1], reverse=True)
    # a short portion far into a long context wants its key range split: the mma.sync tiles take it
    late = StepShape(np.asarray([40], dtype=np.int32), np.asarray([6000], dtype=np.int32), False, page_size=16)
    plan = planner.plan(late)
    assert plan["splits"] > 1 and plan["chunk_rows"] == kernels.CHUNK_TILE_ROWS
    # medium portions, also deep into a context, stay on the tcgen05 kernel, unsplit; so do short
    # portions of a short context
    for count, start in [(512, 0), (1024, 3072), (512, 7000), (100, 500), (32, 600)]:
        plan = planner.plan(StepShape(np.asarray([count], dtype=np.int32), np.asarray([start], dtype=np.int32), False, page_size=16))
        assert plan["chunk_rows"] == kernels.CHUNK_TILE_ROWS_TC and plan["splits"] == 1, (count, start)
    # a decode token beside such a portion gets key ranges of its own, merged in the decode kernel's clusters: eight
    # tiles (one per kv head) run as clusters of ten; the portion's tiles stay unsplit
    mixed = StepShape(np.asarray([700, 1], dtype=np.int32), np.asarray([0, 3000], dtype=np.int32), False, page_size=16)
    plan = planner.plan(mixed)
    assert plan["chunk_rows"] == kernels.CHUNK_TILE_ROWS_TC and plan["splits"] == 1
    assert plan["decode_splits"] == 10 and len(plan["decode_items"]) == 10 and len(plan["chunk_items"]) == -(-700 * 4 // 256)
    assert list(plan["decode_items"][:, 2]) == list(range(10)) and set(plan["decode_items"][:, 0]) == {1}
    # ... as many as its context has blocks of 128 keys, rounded down to a power of two; none for a short one
    for start, want in [(100, 1), (300, 2), (1100, 8)]:
        near = StepShape(np.asarray([700, 1], dtype=np.int32), np.asarray([0, start], dtype=np.int32), False, page_size=16)
        assert planner.plan(near)["decode_splits"] == want, start
    # sixty-four decode tokens beside a portion are 512 tiles: no cluster size runs that many at one time
    lengths = np.asarray([700] + [1] * 64, dtype=np.int32)
    starts = np.asarray([0] + [5000] * 64, dtype=np.int32)
    assert planner.plan(StepShape(lengths, starts, False, page_size=16))["decode_splits"] == 1
    # other head sizes or page sizes: the mma.sync tiles
    assert AttentionItems(4, 8, 64).plan(whole)["chunk_rows"] == kernels.CHUNK_TILE_ROWS
    odd = StepShape(np.asarray([2048], dtype=np.int32), np.asarray([0], dtype=np.int32), False, page_size=4)
    assert planner.plan(odd)["chunk_rows"] == kernels.CHUNK_TILE_ROWS

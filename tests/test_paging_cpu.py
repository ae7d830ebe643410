"""Host logic on the caller's side of the paged KV cache (tlaloc_b200/paging.py): the page pool's rules
(triton/backend/sequence_mode.h:315-336) and the derivation of a step's integer inputs
(triton/backend/sequence_mode.cc:2584-2604; padding constants ir/.../DecodeGraphSpec.kt:989-1004)."""
import numpy as np
import pytest

from tlaloc_b200 import paging, sharding


def test_page_zero_is_never_handed_out_and_pages_come_lowest_first():
    pool = paging.PagePool(8)
    assert pool.capacity == 7 and pool.free_count == 7
    assert pool.take(3) == [1, 2, 3]
    assert pool.take(5) is None and pool.free_count == 4  # nothing taken when fewer are free
    pool.give([2])
    assert pool.take(2) == [2, 4]
    with pytest.raises(ValueError):
        pool.give([0])
    with pytest.raises(ValueError):
        pool.give([7])  # free: nobody holds it
    assert pool.take(0) == []


def test_a_shared_page_is_freed_only_by_its_last_holder():
    pool = paging.PagePool(6)
    prefix = pool.take(2)
    pool.share(prefix)  # a second sequence starts from the cached prefix
    pool.share(prefix[:1])  # and a third from its first page
    pool.give(prefix)
    assert pool.free_count == 3
    pool.give(prefix)
    assert pool.free_count == 4 and 1 not in pool._free
    pool.give(prefix[:1])
    assert pool.free_count == 5


def test_step_inputs_follow_the_reference_derivation():
    bs, M = 4, 6
    pool = paging.PagePool(32)
    a, b = paging.Sequence(), paging.Sequence()
    assert a.reserve(pool, 7, bs) and a.pages == [1, 2]
    assert b.reserve(pool, 2, bs) and b.pages == [3]
    work = [(a, [11, 12, 13, 14, 15, 16, 17]), (b, [21, 22])]
    step = paging.stage_step(work, rows=4, width=8, max_blocks=M, block_size=bs)
    # tokens right-aligned: the last column holds each row's newest token
    assert step.token_ids[0].tolist() == [0, 11, 12, 13, 14, 15, 16, 17]
    assert step.token_ids[1].tolist() == [0, 0, 0, 0, 0, 0, 21, 22]
    assert step.positions[0].tolist() == [0, 0, 1, 2, 3, 4, 5, 6]
    assert step.slot_mapping[0].tolist() == [-1, 4, 5, 6, 7, 8, 9, 10]  # page 1 slots 4..7, page 2 slots 8..
    assert step.slot_mapping[1].tolist() == [-1] * 6 + [12, 13]
    assert step.block_tables[0].tolist() == [1, 2, 0, 0, 0, 0] and step.block_tables[1].tolist() == [3, 0, 0, 0, 0, 0]
    assert step.seq_lens.tolist() == [7, 2, 1, 1]
    # padding rows: slot -1, length 1, page 0
    assert np.all(step.slot_mapping[2:] == -1) and np.all(step.block_tables[2:] == 0)
    paging.commit_step(work)
    assert (a.length, b.length) == (7, 2)
    # one decode token each: a needs no new page for position 7, then one for position 8
    assert a.reserve(pool, 1, bs) and a.pages == [1, 2]
    step = paging.stage_step([(a, [31]), (b, [32])], rows=2, width=1, max_blocks=M, block_size=bs)
    assert step.positions[:, 0].tolist() == [7, 2] and step.slot_mapping[:, 0].tolist() == [2 * bs + 3, 3 * bs + 2]
    assert step.seq_lens.tolist() == [8, 3]
    # the decode-only form agrees with the helper the decoder tests use
    tables = step.block_tables
    assert np.array_equal(sharding.slot_mapping(tables, step.positions[:, 0], bs), step.slot_mapping[:, 0])
    paging.commit_step([(a, [31]), (b, [32])])
    assert a.reserve(pool, 1, bs) and a.pages == [1, 2, 4]


def test_refusals():
    bs = 4
    pool = paging.PagePool(3)
    s = paging.Sequence()
    assert not s.reserve(pool, 9, bs) and s.pages == [] and pool.free_count == 2  # 3 pages needed, 2 exist
    assert s.reserve(pool, 8, bs)
    with pytest.raises(ValueError):
        paging.stage_step([(s, list(range(9)))], rows=1, width=16, max_blocks=4, block_size=bs)  # pages do not cover it
    with pytest.raises(ValueError):
        paging.stage_step([(s, [1, 2, 3])], rows=1, width=2, max_blocks=4, block_size=bs)  # too many tokens for the row
    with pytest.raises(ValueError):
        paging.stage_step([(s, [1]), (s, [2])], rows=1, width=1, max_blocks=4, block_size=bs)
    s.release(pool)
    assert pool.free_count == 2 and s.length == 0
    with pytest.raises(ValueError):
        paging.PagePool(1)

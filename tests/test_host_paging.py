"""Host logic of the page allocator and the scheduler (no GPU): the unit tests of the reference's
BlockManager (paged_kv.rs:1227-1321) and scheduler gates (serving.rs:3425, :3689) restated."""
import numpy as np
import pytest

from wukong_b200.paged import BlockManager, Scheduler, OutOfBlocks


def test_append_allocates_only_on_block_boundary():
    m = BlockManager(8, 4, 2, 4)
    assert m.free_blocks() == 8
    assert m.append(0) == (0, 0)           # fresh pool hands out ascending pages
    assert m.free_blocks() == 7
    for off in (1, 2, 3):
        assert m.append(0) == (0, off)
    assert m.free_blocks() == 7
    assert m.append(0) == (1, 0)
    assert m.context_len(0) == 5 and m.used_blocks() == 2


def test_reserve_bulk_and_locate_matches_append():
    m = BlockManager(16, 4, 3, 8)
    assert m.reserve(1, 10) == 0 and m.context_len(1) == 10 and m.used_blocks() == 3
    seen = [m.locate(1, p) for p in range(10)]
    m2 = BlockManager(16, 4, 3, 8)
    assert seen == [m2.append(1) for _ in range(10)]
    assert all(0 <= off < 4 for _, off in seen)
    assert m.reserve(1, 2) == 10 and m.used_blocks() == 3  # fits the last page


def test_free_relayouts_lifo_and_epoch_moves():
    m = BlockManager(4, 2, 2, 4)
    e0 = m.layout_epoch()
    m.reserve(0, 4)            # pages 0, 1
    m.reserve(1, 2)            # page 2
    assert m.layout_epoch() > e0
    e1 = m.layout_epoch()
    m.free(0)
    assert m.layout_epoch() > e1 and m.free_blocks() == 3 and m.context_len(0) == 0
    assert m.append(1)[1] == 0 and m.locate(1, 2)[0] == 1   # last freed page comes back first
    e2 = m.layout_epoch()
    m.append(1)                # same page: no table change
    assert m.layout_epoch() == e2


def test_out_of_blocks_is_reported_and_table_width_cap():
    m = BlockManager(2, 2, 2, 4)
    m.reserve(0, 4)
    with pytest.raises(OutOfBlocks):
        m.append(1)
    assert m.context_len(1) == 0 and m.free_blocks() == 0
    assert not m.can_grow(1, 1)
    m2 = BlockManager(100, 2, 1, 3)
    m2.reserve(0, 6)
    with pytest.raises(OutOfBlocks):
        m2.append(0)           # would need a 4th table column
    with pytest.raises(OutOfBlocks):
        m2.reserve(0, 1)
    assert m2.context_len(0) == 6


def test_flat_table_is_padded_row_major():
    m = BlockManager(8, 2, 3, 4)
    m.reserve(0, 3); m.reserve(2, 1)
    t = m.flat_block_table()
    assert t.shape == (3, 4) and list(t[0]) == [0, 1, 0, 0] and list(t[1]) == [0, 0, 0, 0] and list(t[2]) == [2, 0, 0, 0]
    assert list(m.ctx_lens()) == [3, 0, 1]


def _drain(s, sample=lambda slot, step: (slot * 7 + step) % 50):
    steps = 0
    while not s.is_idle():
        n = s.plan_step()
        assert n > 0
        s.commit_step([sample(i, steps) for i in range(s.bcap)])
        steps += 1
        assert steps < 10000
    return steps


def test_scheduler_drains_and_conserves_blocks():
    s = Scheduler(bcap=4, num_blocks=64, block_size=4, max_blocks_per_seq=16, max_rows=16, prefill_chunk=5)
    rng = np.random.default_rng(0)
    want = []
    for _ in range(11):
        L, g = int(rng.integers(1, 20)), int(rng.integers(1, 9))
        want.append((s.enqueue(rng.integers(0, 50, L), g), g))
    _drain(s)
    assert s.completed() == 11 == s.admitted() and s.free_blocks() == 64 and s.num_active() == 0
    assert s.emitted() == sum(g for _, g in want)
    for rid, g in want:
        assert s.output(rid).size == g


def test_scheduler_rows_positions_and_feedback():
    s = Scheduler(bcap=2, num_blocks=16, block_size=4, max_blocks_per_seq=8, max_rows=8, prefill_chunk=3)
    r0 = s.enqueue([10, 11, 12, 13], 3)
    n = s.plan_step()                       # first prefill chunk: 3 rows, nothing sampled
    assert n == 3 and list(s.row_token[:3]) == [10, 11, 12] and list(s.row_pos[:3]) == [0, 1, 2]
    assert list(s.row_ctx[:3]) == [1, 2, 3] and list(s.row_slot[:3]) == [0, 0, 0] and s.sample_row[0] == -1
    assert s.commit_step([99, 99]) == 0
    n = s.plan_step()                       # last prompt token: sampled
    assert n == 1 and s.row_token[0] == 13 and s.row_pos[0] == 3 and s.sample_row[0] == 0
    assert s.commit_step([42, 0]) == 1
    n = s.plan_step()                       # decode: feeds the sampled token back at the next position
    assert n == 1 and s.row_token[0] == 42 and s.row_pos[0] == 4 and s.row_ctx[0] == 5
    s.commit_step([43, 0])
    s.plan_step(); s.commit_step([44, 0])
    assert s.is_idle() and list(s.output(r0)) == [42, 43, 44] and s.free_blocks() == 16


def test_failed_plan_leaves_allocator_unchanged():
    s = Scheduler(bcap=2, num_blocks=2, block_size=2, max_blocks_per_seq=4, max_rows=4, prefill_chunk=4)
    s.enqueue([1, 2], 4); s.enqueue([3, 4], 4)
    assert s.plan_step() == 4               # both prompts fill both pages
    s.commit_step([5, 6])
    free, ctx = s.free_blocks(), list(s.manager.ctx_lens())
    with pytest.raises(OutOfBlocks):
        s.plan_step()                       # both slots need a new page, none is free
    assert s.free_blocks() == free and list(s.manager.ctx_lens()) == ctx
    with pytest.raises(ValueError):
        s.enqueue([1] * 7, 4)               # can never fit a block-table row


def test_admission_lookahead_skips_oversized_head():
    s = Scheduler(bcap=2, num_blocks=4, block_size=2, max_blocks_per_seq=4, max_rows=8, prefill_chunk=8)
    big = s.enqueue([1] * 6, 1)             # needs 3 pages
    s.enqueue([2] * 4, 1)                   # 2 pages
    small = s.enqueue([3] * 2, 1)           # 1 page
    s.plan_step()
    # slot 0 takes the first that fits (big, 3 pages), slot 1 skips the 2-page request for the 1-page one
    assert s.num_active() == 2 and s.pending() == 1
    s.commit_step([0, 0])
    assert s.output(big).size == 1 and s.output(small).size == 1


def test_starved_slots_sit_out_and_resume_when_pages_are_released():
    """A pool smaller than bcap * (prompt + gen_len): a slot whose next row needs a page that is not free is left out of
    the step (decode rows are served before prompt chunks) and continues once another sequence retires."""
    s = Scheduler(bcap=3, num_blocks=5, block_size=2, max_blocks_per_seq=4, max_rows=6, prefill_chunk=2)
    ids = [s.enqueue([1, 2], 5), s.enqueue([3, 4], 3), s.enqueue([5, 6], 2)]
    sat_out = 0
    steps = 0
    while not s.is_idle():
        n = s.plan_step()
        assert n > 0
        live = s.num_active()
        planned_slots = len(set(s.row_slot[:n].tolist()))
        sat_out += live - planned_slots
        assert s.manager.used_blocks() <= 5
        s.commit_step([7, 8, 9])
        steps += 1
        assert steps < 100
    assert sat_out > 0                                   # the pool did run short at some step
    assert [s.output(i).size for i in ids] == [5, 3, 2] and s.free_blocks() == 5 and s.completed() == 3

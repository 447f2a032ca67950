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


def test_scheduler_invariants_under_random_load():
    """Random geometries and request streams, pools that run short: at every step the rows of a slot are consecutive
    positions that continue its context, causal (ctx = pos + 1), prompt tokens come back in order and each sampled token
    is fed back exactly once as the next decode row; no page holds tokens of two slots; used + free pages = the pool; every
    request ends with exactly gen_len tokens, the ones this "model" drew for it."""
    for seed in range(25):
        rng = np.random.default_rng(seed)
        bcap = int(rng.integers(1, 6))
        bs = int(rng.choice([1, 2, 4, 16]))
        mbps = int(rng.integers(2, 9))
        cap_tokens = bs * mbps
        nblk = int(rng.integers(mbps, bcap * mbps + 1))            # at least one full row of pages, often fewer than bcap rows
        max_rows = int(rng.integers(bcap, 4 * bcap + 4))
        chunk = int(rng.integers(1, 8))
        s = Scheduler(bcap=bcap, num_blocks=nblk, block_size=bs, max_blocks_per_seq=mbps, max_rows=max_rows, prefill_chunk=chunk)
        reqs = {}
        for _ in range(int(rng.integers(1, 12))):
            L = int(rng.integers(1, max(2, cap_tokens)))
            g = int(rng.integers(1, max(2, cap_tokens - L + 1)))
            if L + g - 1 > cap_tokens:                             # the last sampled token is never written back
                continue
            prompt = rng.integers(0, 1000, L).astype(np.int32)
            reqs[s.enqueue(prompt, g)] = (prompt, g, [])
        slot_req = {}                                               # slot -> (request id known to the test) via its prompt
        fed = {}                                                    # slot -> tokens seen so far for the current occupant
        pending_feedback = {}                                       # slot -> sampled token that must come back next
        drawn = {}                                                  # slot -> tokens drawn for the current occupant
        steps = 0
        while not s.is_idle():
            try:
                n = s.plan_step()
            except OutOfBlocks:
                # every resident slot needs a page and none is free: legal only when nothing can move
                assert s.free_blocks() < s.num_active() or s.free_blocks() == 0
                break
            assert 0 < n <= max_rows
            slots = s.row_slot[:n].tolist()
            pos = s.row_pos[:n].tolist()
            ctxs = s.row_ctx[:n].tolist()
            toks = s.row_token[:n].tolist()
            ctx_now = s.manager.ctx_lens()
            for sl in set(slots):
                idx = [i for i in range(n) if slots[i] == sl]
                assert idx == list(range(idx[0], idx[-1] + 1))       # a slot's rows are contiguous in the step
                p = [pos[i] for i in idx]
                assert p == list(range(p[0], p[0] + len(p)))
                assert [ctxs[i] for i in idx] == [q + 1 for q in p]
                assert ctx_now[sl] == p[-1] + 1                      # pages are reserved up to the last row of the step
                if p[0] == 0:                                        # a new occupant
                    fed[sl], drawn[sl] = [], []
                    pending_feedback.pop(sl, None)
                assert len(fed[sl]) == p[0]
                if sl in pending_feedback:
                    assert len(idx) == 1 and toks[idx[0]] == pending_feedback.pop(sl)
                fed[sl].extend(toks[i] for i in idx)
            # no page in two slots; accounting adds up
            table = s.manager.flat_block_table()
            owned = []
            for sl in range(bcap):
                owned.extend(table[sl, :(ctx_now[sl] + bs - 1) // bs].tolist())
            # (admission reserves a prompt's pages ahead of its rows, so more pages may be in use than the contexts cover)
            assert len(owned) == len(set(owned)) <= s.manager.used_blocks()
            assert all(0 <= pg < nblk for pg in owned)
            assert s.manager.used_blocks() + s.free_blocks() == nblk
            sampled = np.zeros(bcap, np.int32)
            for sl in range(bcap):
                r = int(s.sample_row[sl])
                if r >= 0:
                    assert slots[r] == sl and (r == n - 1 or slots[r + 1] != sl)   # the slot's last row of the step
                    sampled[sl] = int(rng.integers(1000, 2000))
                    pending_feedback[sl] = int(sampled[sl])
                    drawn[sl].append(int(sampled[sl]))
            s.commit_step(sampled)
            # a slot that retired leaves its prompt + drawn tokens behind: match them to a request
            for sl in list(drawn):
                if ctx_now[sl] > 0 and s.manager.ctx_lens()[sl] == 0:
                    hit = [rid for rid, (pr, g, got) in reqs.items() if not got and len(drawn[sl]) == g and fed[sl][:len(pr)] == pr.tolist()]
                    assert hit, (seed, sl)
                    reqs[hit[0]][2].extend(drawn[sl])
                    pending_feedback.pop(sl, None)
                    del drawn[sl]
            steps += 1
            assert steps < 5000
        if s.is_idle():
            assert s.free_blocks() == nblk and s.completed() == len(reqs)
            for rid, (pr, g, got) in reqs.items():
                assert s.output(rid).tolist() == got and len(got) == g

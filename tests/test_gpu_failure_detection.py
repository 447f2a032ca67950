"""Failure detection on the GPU without any fault: waits that run out report a status and return, a host-side
deadline turns a slow stream into an error, and the paged-KV kernels refuse positions past the block table.

Nothing here traps, faults or leaves a kernel waiting: the "peer that never answers" is a flag nobody sets and the
wait limit is a few milliseconds; the "launch that does not finish in time" is a kernel that sleeps for a bounded
time and ends by itself.  The reference's one failure mechanism is its `sync_within` deadline
(crates/wukong_codegen_gpu/src/gpu.rs:250-262, :302)."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch
    from wukong_b200 import _lib, lib, device
    _lib.require_gpu()
    return torch, lib(), device


def _tp_call(torch, L, parts, flags, step, phase, x, out, rows, cols):
    arr = (ctypes.c_void_p * 2)(parts[0].data_ptr(), parts[1].data_ptr())
    farr = (ctypes.c_void_p * 2)(flags[0].data_ptr(), flags[1].data_ptr())
    return L.wkb_tp_reduce_add_rmsnorm(arr, farr, 0, 2, step.data_ptr(), phase, 2, x.data_ptr(), None, out.data_ptr(), rows, cols, 1e-5,
                                       torch.cuda.current_stream().cuda_stream)


def test_tp_reduce_wait_runs_out_reports_and_leaves_x_untouched(env):
    """Two-rank reduce on one GPU whose second "rank" is plain local memory that never publishes its flag."""
    torch, L, dev = env
    rows, cols = 8, 1024
    parts = [torch.full((rows, cols), 1.0, device="cuda"), torch.full((rows, cols), 2.0, device="cuda")]
    flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(2)]
    step = torch.zeros(1, dtype=torch.int32, device="cuda")
    x = torch.full((rows, cols), 5.0, device="cuda")
    out = torch.full((rows, cols), 9.0, device="cuda", dtype=torch.bfloat16)
    assert dev.gemm_status() == 0
    L.wkb_tp_set_wait_limit_ms(5)
    try:
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        assert _tp_call(torch, L, parts, flags, step, 0, x, out, rows, cols) == 0
        t1.record()
        torch.cuda.synchronize()
        assert t0.elapsed_time(t1) < 500.0                  # the kernel came back by itself, near its 5 ms limit
        assert dev.gemm_status() == 21                      # "flag wait ran out"
        assert bool((x == 5.0).all()) and bool((out.float() == 9.0).all())      # the sum was skipped
        # rank 0 published its own flag to the peer before waiting, then marked itself dead everywhere
        assert int(flags[1][0].item()) == -1 and int(flags[0][0].item()) == -1
        # a dead rank ends every later phase at once with code 22, still without touching x
        assert _tp_call(torch, L, parts, flags, step, 1, x, out, rows, cols) == 0
        torch.cuda.synchronize()
        assert dev.gemm_status() == 22 and bool((x == 5.0).all())
        # zeroed flag rows start again; with the peer's flag published the same call sums in rank order
        for f in flags:
            f.zero_()
        flags[0][1] = 1                                      # the peer's sequence number for step 0, phase 0
        assert _tp_call(torch, L, parts, flags, step, 0, x, out, rows, cols) == 0
        torch.cuda.synchronize()
        assert dev.gemm_status() == 0
        assert bool((x == 8.0).all())                        # 5 + (1 + 2)
        assert torch.allclose(out.float(), torch.ones_like(x), atol=1e-2)      # rmsnorm of a constant row
    finally:
        L.wkb_tp_set_wait_limit_ms(0)


def test_stream_deadline_reports_a_slow_stream_and_nothing_is_lost(env):
    torch, L, dev = env
    st = torch.cuda.Stream()
    assert L.wkb_stream_sync_within(st.cuda_stream, 5) == 0            # idle stream
    assert L.wkb_device_sleep_ms(60, st.cuda_stream) == 0
    marker = torch.zeros(1, device="cuda")
    with torch.cuda.stream(st):
        marker.add_(1.0)                                               # work queued behind the sleeping kernel
    assert L.wkb_stream_sync_within(st.cuda_stream, 5) == -1           # deadline passed, work still in flight
    assert L.wkb_stream_sync_within(st.cuda_stream, 2000) == 0         # it ends by itself
    assert float(marker.item()) == 1.0


def test_engine_step_deadline_raises_and_the_step_can_still_be_finished(env):
    torch, L, dev = env
    from wukong_b200.serving import GPT2Config, synth_weights, Engine, StepTimeout
    cfg = GPT2Config(n_layer=2, d_model=128, n_head=2, d_ff=256, vocab=500, n_pos=128)
    w = synth_weights(cfg, 0)
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, 500, 9).tolist(), rng.integers(0, 500, 4).tolist()]

    def run(slow):
        eng = Engine(cfg, w, bcap=2, num_pages=32, max_blocks_per_seq=4, step_timeout_ms=20 if slow else None)
        ids = [eng.enqueue(p, 5) for p in prompts]
        timeouts = 0
        for it in range(100):
            if eng.sched.is_idle():
                break
            if slow and it == 2:
                assert L.wkb_device_sleep_ms(150, eng.stream.cuda_stream) == 0     # the step queues behind a slow kernel
                with pytest.raises(StepTimeout):
                    eng.step()
                timeouts += 1
                with pytest.raises(RuntimeError):
                    eng.step()                                                  # a new step may not start over a pending one
                eng.finish_step(2000)                                           # keep waiting: the step completes and commits
            else:
                eng.step()
        return [eng.sched.output(i).tolist() for i in ids], timeouts

    plain, _ = run(False)
    slow, timeouts = run(True)
    assert timeouts == 1 and slow == plain


def test_kv_append_and_decode_refuse_positions_past_the_block_table(env, orc):
    """A row whose position lies past its block-table row is skipped by every append kernel (cache bytes unchanged,
    status 31); decode attention clamps the visible keys to what the table covers; the device-side feedback parks a row
    that reaches the last covered position."""
    torch, L, dev = env
    s = torch.cuda.current_stream().cuda_stream
    kvh, hd, page, mbps, pages = 2, 64, 16, 2, 8
    kv = dev.PagedKV(1, pages, kvh, hd, page)
    kv.k.fill_(3.0); kv.v.fill_(3.0)
    bt = torch.tensor([[1, 2], [3, 4]], dtype=torch.int32, device="cuda")
    src = torch.randn(2, 2 * kvh * hd, device="cuda")
    row_slot = torch.tensor([0, 1], dtype=torch.int32, device="cuda")
    row_pos = torch.tensor([mbps * page, 5], dtype=torch.int32, device="cuda")          # row 0 is one past the table
    assert dev.gemm_status() == 0
    dev.paged_kv_append(kv, 0, src, src[:, kvh * hd:], src.stride(0), bt, row_slot, row_pos, 2, mbps)
    torch.cuda.synchronize()
    assert dev.gemm_status() == 31
    k = kv.k[0].float()
    assert bool((k[[0, 1, 2, 4, 5, 6, 7]] == 3.0).all())                               # only page 3 (slot 1, position 5) changed
    assert bool((k[3][:, 5] != 3.0).any()) and bool((k[3][:, :5] == 3.0).all()) and bool((k[3][:, 6:] == 3.0).all())
    # int8 cache append
    kv8 = dev.PagedKVInt8(1, pages, kvh, hd, page)
    dev.paged_kv_append_int8(kv8, 0, src, src[:, kvh * hd:], src.stride(0), bt, row_slot, row_pos, 2, mbps)
    torch.cuda.synchronize()
    assert dev.gemm_status() == 31
    assert bool((kv8.k[0][[0, 1, 2, 4, 5, 6, 7]] == 0).all())
    # RoPE + append fused
    qh, half = 2, hd // 2
    qkv = torch.randn(2, (qh + 2 * kvh) * hd, device="cuda")
    before = qkv.clone()
    inv = torch.rand(half, device="cuda")
    kv.k.fill_(3.0); kv.v.fill_(3.0)
    assert L.wkb_rope_qk_paged_append(qkv.data_ptr(), qkv.stride(0), inv.data_ptr(), bt.data_ptr(), row_slot.data_ptr(), row_pos.data_ptr(),
                                      kv.k[0].data_ptr(), kv.v[0].data_ptr(), 2, qh, kvh, half, page, mbps, s) == 0
    torch.cuda.synchronize()
    assert dev.gemm_status() == 31
    assert torch.equal(qkv[0], before[0])                                              # the skipped row is untouched, q included
    assert bool((kv.k[0].float()[[0, 1, 2, 4, 5, 6, 7]] == 3.0).all())
    # decode attention: a context length past the table is read as the table's capacity
    kv.k.normal_(); kv.v.normal_()
    q = torch.randn(2, qh * hd, device="cuda")
    scratch = dev.paged_attn_scratch(2, qh, hd, 4096)
    out_big = torch.empty(2, qh * hd, device="cuda")
    out_cap = torch.empty(2, qh * hd, device="cuda")
    big = torch.tensor([4000, 20], dtype=torch.int32, device="cuda")
    cap = torch.tensor([mbps * page, 20], dtype=torch.int32, device="cuda")
    dev.paged_attn_decode(q, qh * hd, kv, 0, bt, row_slot, big, out_big, 2, qh, mbps, 4096, 0.125, scratch)
    dev.paged_attn_decode(q, qh * hd, kv, 0, bt, row_slot, cap, out_cap, 2, qh, mbps, 4096, 0.125, scratch)
    torch.cuda.synchronize()
    assert torch.equal(out_big, out_cap) and not bool(torch.isnan(out_big).any())
    # feedback: a row at the last covered position is parked instead of moving on
    tok = torch.zeros(2, dtype=torch.int32, device="cuda")
    pos = torch.tensor([mbps * page - 1, 7], dtype=torch.int32, device="cuda")
    ctx = pos + 1
    nxt = torch.tensor([11, 12], dtype=torch.int32, device="cuda")
    assert L.wkb_decode_advance(tok.data_ptr(), pos.data_ptr(), ctx.data_ptr(), nxt.data_ptr(), 2, mbps * page - 1, s) == 0
    torch.cuda.synchronize()
    assert pos.tolist() == [-1, 8] and ctx.tolist() == [0, 9] and tok.tolist() == [11, 12]

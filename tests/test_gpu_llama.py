"""GPU parity of the Llama-shape int4 decode model against the CPU oracle model, unsharded and with the
tensor-parallel split emulated on one device."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch
    from wukong_b200 import _lib, llama
    _lib.require_gpu()
    return torch, llama


def small_cfg(llama):
    return llama.LlamaConfig(n_layer=2, d_model=512, n_head=4, n_kv_head=2, d_ff=1408, vocab=1024)


def drive(torch, models_forward, set_rows, read_logits, oracle, cfg, prompts, steps, page_perm):
    """Feed the same tokens (the oracle's greedy continuation) to both models; return per-step (oracle logits, ours)."""
    S = len(prompts)
    kc, vc = zip(*[oracle.new_cache(steps + 1) for _ in range(S)])
    mbps = 4
    table = np.zeros((S, mbps), np.int32)
    for s in range(S):
        table[s] = page_perm[s * mbps:(s + 1) * mbps]
    toks = [p[0] for p in prompts]
    hist = []
    for t in range(steps):
        poss = [t] * S
        nxt, ref_logits = oracle.step(toks, poss, kc, vc)
        i32 = lambda a: torch.tensor(np.asarray(a, np.int32), device="cuda")
        set_rows(i32(toks), i32(poss), i32(np.arange(S)), i32([t + 1] * S), torch.from_numpy(table).cuda())
        ours_tok = models_forward(S)
        torch.cuda.synchronize()
        hist.append((ref_logits, read_logits(), np.asarray(nxt), ours_tok.cpu().numpy()[:S]))
        toks = [prompts[s][t + 1] if t + 1 < len(prompts[s]) else int(nxt[s]) for s in range(S)]
    return hist


def check_hist(hist, rel):
    """|ours - oracle| <= rel * (|oracle| + rms of the row's logits) (tests/tolerances.py says why the floor is the
    row's rms); tokens equal wherever the oracle's winner leads by more than both allowances."""
    from tolerances import check_logits, clear_winner
    for ref, got, ref_tok, got_tok in hist:
        check_logits(got, ref, rel)
        clear = clear_winner(ref, rel)
        assert np.array_equal(got_tok[clear], ref_tok[clear])


def test_llama_int4_decode_matches_oracle(env, orc):
    torch, llama = env
    from oracle.llama_model import OracleLlama
    from wukong_b200 import device as dev
    cfg = small_cfg(llama)
    w = llama.synth_llama_raw(cfg, seed=11, sigma=0.008)
    S, steps = 3, 6
    model = llama.LlamaDecodeModel(cfg, llama.LlamaRankWeights.from_raw(cfg, w), 0, 1, bcap=S, num_pages=64, max_blocks_per_seq=4)

    def set_rows(tok, pos, slot, ctx, table):
        model.row_token.copy_(tok); model.row_pos.copy_(pos); model.row_slot.copy_(slot); model.row_ctx.copy_(ctx)
        model.block_table.copy_(table)

    rng = np.random.default_rng(5)
    prompts = [list(rng.integers(0, cfg.vocab, 3)) for _ in range(S)]
    perm = rng.permutation(64).astype(np.int32)
    # (1) the same model with every weight held as the bf16 operand the tensor core multiplies: what is left is
    #     accumulation order and activations that round to the neighbouring bf16 value (one such flip is 2^-8 of
    #     that activation and spreads through the following layers)
    hist = drive(torch, model.forward, set_rows, lambda: model.logits.cpu().numpy()[:S], OracleLlama(cfg, w, orc, "bf16"), cfg,
                 prompts, steps, perm)
    assert dev.gemm_status() == 0
    check_hist(hist, 8e-3)
    # (2) the exact dequantisation: the stated bar of the half-precision paths, rtol 2e-2 on the logits
    hist = drive(torch, model.forward, set_rows, lambda: model.logits.cpu().numpy()[:S], OracleLlama(cfg, w, orc), cfg, prompts,
                 steps, perm)
    check_hist(hist, 2e-2)


def test_llama_tensor_parallel_split_matches_unsharded(env, orc):
    torch, llama = env
    from oracle.llama_model import OracleLlama
    cfg = small_cfg(llama)
    w = llama.synth_llama_raw(cfg, seed=12, sigma=0.008)
    oracle = OracleLlama(cfg, w, orc, "bf16")
    S, steps = 2, 4
    tp = llama.LocalTensorParallel(cfg, w, 2, bcap=S, num_pages=64, max_blocks_per_seq=4)
    rng = np.random.default_rng(6)
    prompts = [list(rng.integers(0, cfg.vocab, 2)) for _ in range(S)]

    def logits():
        return np.concatenate([m.logits.cpu().numpy()[:S] for m in tp.models], axis=1)

    hist = drive(torch, tp.forward, tp.set_rows, logits, oracle, cfg, prompts, steps, rng.permutation(64).astype(np.int32))
    check_hist(hist, 8e-3)
    # each rank holds half of the KV heads and half of the weight bytes
    assert tp.models[0].kv.k[0].shape[1] == cfg.n_kv_head // 2
    full = llama.LlamaRankWeights.from_raw(cfg, w).q4_bytes()
    assert sum(m.w.q4_bytes() for m in tp.models) == full


def test_llama_chunked_prefill_matches_token_by_token_oracle(env, orc):
    """Prompt chunks (several positions of a sequence in one step, on the tiled prefill attention) give the logits the
    oracle computes token by token, and the decode steps that follow continue from the same cache."""
    torch, llama = env
    from oracle.llama_model import OracleLlama
    from wukong_b200 import device as dev
    cfg = small_cfg(llama)
    w = llama.synth_llama_raw(cfg, seed=11, sigma=0.008)
    rng = np.random.default_rng(9)
    lens = [9, 3, 5]                                    # prompt lengths: 17 rows in the first step
    prompts = [list(rng.integers(0, cfg.vocab, n)) for n in lens]
    S, R, mbps = len(lens), 24, 4
    model = llama.LlamaDecodeModel(cfg, llama.LlamaRankWeights.from_raw(cfg, w), 0, 1, bcap=R, num_pages=64, max_blocks_per_seq=mbps)
    oracle = OracleLlama(cfg, w, orc, "bf16")
    table = np.zeros((R, mbps), np.int32)
    table[:S] = rng.permutation(64).astype(np.int32)[:S * mbps].reshape(S, mbps)
    model.block_table.copy_(torch.from_numpy(table).cuda())
    # the oracle, one token at a time
    kc, vc = zip(*[oracle.new_cache(16) for _ in range(S)])
    ref = {}
    for t in range(max(lens)):
        live = [s for s in range(S) if t < lens[s]]
        _, lg = oracle.step([prompts[s][t] for s in live], [t] * len(live), [kc[s] for s in live], [vc[s] for s in live])
        for i, s in enumerate(live):
            ref[(s, t)] = lg[i]
    # ours: the whole prompts in one step
    slot = np.concatenate([np.full(n, s, np.int32) for s, n in enumerate(lens)])
    pos = np.concatenate([np.arange(n, dtype=np.int32) for n in lens])
    tok = np.concatenate([np.asarray(p, np.int32) for p in prompts])
    n = slot.shape[0]
    i32 = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.int32)).cuda()
    pad = lambda a, fill: np.concatenate([np.asarray(a, np.int32), np.full(R - len(a), fill, np.int32)])
    model.row_token.copy_(i32(pad(tok, 0))); model.row_pos.copy_(i32(pad(pos, -1)))
    model.row_slot.copy_(i32(pad(slot, 0))); model.row_ctx.copy_(i32(pad(pos + 1, 0)))
    model.set_prefill_rows(slot)
    model.forward(n)
    torch.cuda.synchronize()
    assert dev.gemm_status() == 0
    got = model.logits.cpu().numpy()[:n]
    want = np.stack([ref[(int(slot[r]), int(pos[r]))] for r in range(n)])
    check_hist([(want, got, want.argmax(1), got.argmax(1))], 8e-3)
    # decode continues from the cache the chunks wrote
    model.set_prefill_rows(None)
    toks = [int(ref[(s, lens[s] - 1)].argmax()) for s in range(S)]
    for step in range(2):
        poss = [lens[s] + step for s in range(S)]
        nxt, lg = oracle.step(toks, poss, list(kc), list(vc))
        model.row_token.copy_(i32(pad(np.asarray(toks), 0))); model.row_pos.copy_(i32(pad(np.asarray(poss), -1)))
        model.row_slot.copy_(i32(pad(np.arange(S), 0))); model.row_ctx.copy_(i32(pad(np.asarray(poss) + 1, 0)))
        model.forward(S)
        torch.cuda.synchronize()
        check_hist([(lg, model.logits.cpu().numpy()[:S], np.asarray(nxt), model.next_tok.cpu().numpy()[:S])], 8e-3)
        toks = [int(t) for t in nxt]


def test_fused_rank_sum_with_eight_local_partials_adds_in_rank_order():
    """The fused tensor-parallel reduce on one GPU: the "ranks" are local buffers whose flags are already published.
    x must come out as x + (((p0 + p1) + p2) + ...), bit for bit, for 3, 4 and 8 ranks (every rank's piece is loaded
    before the first add; the adds stay in rank order), and the normed row must match the fp32 formula."""
    import ctypes
    import torch
    from wukong_b200 import _lib, lib, device as dev
    _lib.require_gpu()
    L = lib()
    torch.manual_seed(0)
    for world, rows, cols in [(8, 16, 4096), (8, 64, 4096), (4, 64, 4096), (3, 5, 1024), (8, 7, 8192)]:
        parts = [torch.randn(rows, cols, device="cuda") for _ in range(world)]
        flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(world)]
        flags[0][:world] = 1                                  # every peer's sequence number for step 0, phase 0
        step = torch.zeros(1, dtype=torch.int32, device="cuda")
        x = torch.randn(rows, cols, device="cuda")
        x0 = x.clone()
        gamma = torch.rand(cols, device="cuda") + 0.5
        out = torch.empty(rows, cols, device="cuda", dtype=torch.bfloat16)
        arr = (ctypes.c_void_p * world)(*[p.data_ptr() for p in parts])
        farr = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
        rc = L.wkb_tp_reduce_add_rmsnorm(arr, farr, 0, world, step.data_ptr(), 0, 2, x.data_ptr(), gamma.data_ptr(), out.data_ptr(), rows, cols,
                                         ctypes.c_float(1e-5), torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert rc == 0 and dev.gemm_status() == 0
        s = parts[0].clone()
        for p in range(1, world):
            s += parts[p]
        ref = x0 + s
        assert torch.equal(x, ref)
        normed = ref.double() * torch.rsqrt((ref.double() ** 2).mean(1, keepdim=True) + 1e-5) * gamma.double()
        assert torch.allclose(out.double(), normed, rtol=2 ** -7, atol=1e-6)

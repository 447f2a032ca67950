"""Tensor-parallel algebra of the Llama-shape block on CPU ranks (gloo, world size 2), with the oracle model
doing the arithmetic: each rank computes its contribution to the attention and MLP sub-blocks from its own
heads / FFN columns, a gloo all-reduce sums them, and the result is compared with the unsharded block.
Mirrors the reference's one-GPU validation of the same split (crates/wukong_codegen_gpu/src/serving.rs:
4161-4240): a split by output rows reproduces the unsharded values exactly, a split by input columns
differs only by the re-association of one sum."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def small_cfg():
    from wukong_b200.llama import LlamaConfig
    return LlamaConfig(n_layer=2, d_model=256, n_head=4, n_kv_head=2, d_ff=512, vocab=320)


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import binding as orc
    from oracle.llama_model import OracleLlama
    from wukong_b200.llama import synth_llama_raw
    cfg = small_cfg()
    model = OracleLlama(cfg, synth_llama_raw(cfg, seed=3), orc)
    toks, steps = [5, 17, 300], 3
    kc, vc = zip(*[model.new_cache(8) for _ in toks])
    x_hist = []
    for t in range(steps):
        poss = [t] * len(toks)
        x = model.embed[np.asarray(toks)].astype(np.float32)
        for li in range(cfg.n_layer):
            part = torch.from_numpy(model.attn_partial(li, x, poss, kc, vc, rank, world).copy())
            dist.all_reduce(part)
            x = (x + part.numpy()).astype(np.float32)
            part = torch.from_numpy(model.mlp_partial(li, x, rank, world).copy())
            dist.all_reduce(part)
            x = (x + part.numpy()).astype(np.float32)
        x_hist.append(x)
        toks = [(int(v) * 7 + t) % cfg.vocab for v in toks]
    if rank == 0:
        out.put(np.stack(x_hist))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_block_matches_unsharded(orc):
    from oracle.llama_model import OracleLlama
    from wukong_b200.llama import synth_llama_raw
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29900 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = out.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    cfg = small_cfg()
    model = OracleLlama(cfg, synth_llama_raw(cfg, seed=3), orc)
    toks = [5, 17, 300]
    kc, vc = zip(*[model.new_cache(8) for _ in toks])
    for t in range(3):
        poss = [t] * len(toks)
        x = model.embed[np.asarray(toks)].astype(np.float32)
        for li in range(cfg.n_layer):
            x = (x + model.attn_partial(li, x, poss, kc, vc)).astype(np.float32)
            x = (x + model.mlp_partial(li, x)).astype(np.float32)
        # the sum over input-column slices re-associates one fp32 sum per element
        scale = np.abs(x).max()
        assert np.all(np.abs(got[t] - x) <= 2e-5 * scale), float(np.abs(got[t] - x).max() / scale)
        toks = [(int(v) * 7 + t) % cfg.vocab for v in toks]


def test_row_split_is_exact_and_column_split_reassociates(orc):
    """The two halves of the algebra on one linear: output-row shards concatenate to the full product bit for
    bit; input-column shards sum to it within one re-association."""
    from oracle.llama_model import dequant_rows
    from wukong_b200.llama import synth_q4_raw, shard_rows, shard_cols
    rng = np.random.default_rng(0)
    n, k = 96, 256
    raw = synth_q4_raw(rng, n, k)
    w = dequant_rows(orc, raw, n, k).astype(np.float64)
    x = orc.from_bf16_bits(orc.to_bf16_bits(rng.standard_normal((4, k)).astype(np.float32))).reshape(4, k).astype(np.float64)
    full = (x @ w.T).astype(np.float32)
    rows = [(x @ dequant_rows(orc, shard_rows(raw, r, 2), n // 2, k).astype(np.float64).T).astype(np.float32) for r in range(2)]
    assert np.array_equal(np.concatenate(rows, axis=1), full)
    cols = [(x[:, r * k // 2:(r + 1) * k // 2] @ dequant_rows(orc, shard_cols(raw, r, 2), n, k // 2).astype(np.float64).T).astype(np.float32)
            for r in range(2)]
    assert np.all(np.abs((cols[0] + cols[1]) - full) <= 4e-7 * np.abs(x) @ np.abs(w).T + 1e-7)

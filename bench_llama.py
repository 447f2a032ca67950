"""Second benchmark workload: the Llama-7B-shape Q4_0 block stack, batch 64 decode at context 2048,
tensor-parallel over the GPUs of one node (python bench.py --workload llama_int4 --gpus N ...).

A step is one decode step of the 64 sequences (64 tokens for the whole job, whatever the GPU count:
tensor parallelism splits one model, so scaling is strong).  Weights are seeded synthetic Q4_0 blocks of
the named shapes; the KV cache is filled with seeded normal values standing for the 2048-token prefill
(the timed region is decode; a real prefill of the same cache changes none of its work).
`value` replays a captured CUDA graph of whole steps with the token feedback on the device; `e2e` goes
through host buffers every step (rows up, tokens down)."""
import json
import os
import sys
import time

import bench as B

BATCH, CTX0, PAGE = 64, 2048, 16


def llama_config_dict(cfg, world, batch, ctx0, how=""):
    return {"workload": "Llama-7B-shape Q4_0 block stack, batch %d decode at context %d after a synthetic-fill prefill" % (batch, ctx0),
            "layers": cfg.n_layer, "d_model": cfg.d_model, "heads": cfg.n_head, "kv_heads": cfg.n_kv_head, "d_ff": cfg.d_ff,
            "vocab": cfg.vocab, "batch": batch, "context": ctx0, "weights": "Q4_0 (18 B per 32 weights), activations bf16",
            "kv": "paged bf16, %d-token pages, synthetic fill standing for the prefill" % PAGE,
            "parallelism": "tp%d (heads / FFN columns / vocabulary split, 2 sums over ranks per layer%s)" % (world, how),
            "l2": "per-step inputs (weights + KV, several GB per GPU) exceed the 126 MB L2; no flush needed"}


def cpu_llama_tok_s(cfg, batch, ctx, threads):
    """CPU port on a bounded sample: ONE layer of the stack at the benchmark's batch and context -- the seven
    Q4_0 linears through the reference-contract GEMV (one call per row, rows in parallel inside the kernel),
    RoPE, GQA attention over `ctx` bf16 keys, SwiGLU -- timed once after a warm-up on a quarter of the rows;
    the step time is that x n_layer (the LM head and norms are left out, which flatters the CPU)."""
    import numpy as np
    from oracle import binding as orc
    from wukong_b200.llama import synth_q4_raw
    orc.set_threads(threads)
    rng = np.random.default_rng(0)
    d, hd, F = cfg.d_model, cfg.head_dim, cfg.d_ff
    shapes = {"q": (cfg.n_head * hd, d), "k": (cfg.n_kv_head * hd, d), "v": (cfg.n_kv_head * hd, d), "o": (d, cfg.n_head * hd),
              "gate": (F, d), "up": (F, d), "down": (d, F)}
    w = {k: synth_q4_raw(rng, n, kk).reshape(-1) for k, (n, kk) in shapes.items()}
    kc = rng.standard_normal((batch, ctx, cfg.n_kv_head, hd)).astype(np.float32)
    vc = rng.standard_normal((batch, ctx, cfg.n_kv_head, hd)).astype(np.float32)
    x = rng.standard_normal((batch, d)).astype(np.float32)
    inv = (1.0 / (10000.0 ** (np.arange(hd // 2, dtype=np.float32) * 2.0 / hd))).astype(np.float32)

    def lin(name, a):
        n = shapes[name][0]
        return np.stack([orc.gemv_q(w[name], a[r], n)[1] for r in range(a.shape[0])])

    def layer(rows):
        xs = x[:rows]
        xn = orc.norm_affine(xs, np.ones(d, np.float32), np.zeros(d, np.float32), 2, 1e-5)
        q, k, v = lin("q", xn), lin("k", xn), lin("v", xn)
        pos = np.full(rows, ctx, np.int32)
        q, k = orc.rope_pos(q, inv, pos, cfg.n_head), orc.rope_pos(k, inv, pos, cfg.n_kv_head)
        g = cfg.n_head // cfg.n_kv_head
        qh = q.reshape(rows, cfg.n_kv_head, g, hd)
        sc = np.einsum("bkgd,btkd->bkgt", qh, kc[:rows]) * (1.0 / np.sqrt(hd))
        e = np.exp(sc - sc.max(-1, keepdims=True))
        att = np.einsum("bkgt,btkd->bkgd", e / e.sum(-1, keepdims=True), vc[:rows]).reshape(rows, -1).astype(np.float32)
        xs = xs + lin("o", att)
        xn = orc.norm_affine(xs, np.ones(d, np.float32), np.zeros(d, np.float32), 2, 1e-5)
        gt, up = lin("gate", xn), lin("up", xn)
        return xs + lin("down", (gt / (1.0 + np.exp(-gt)) * up).astype(np.float32))

    layer(max(1, batch // 4))
    t0 = time.perf_counter()
    layer(batch)
    dt = time.perf_counter() - t0
    return batch / (dt * cfg.n_layer), "1 of %d layers at batch %d, context %d, timed once (%.1f s); step = layer x %d" % (
        cfg.n_layer, batch, ctx, dt, cfg.n_layer)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from wukong_b200.llama import LlamaConfig
    cfg = LlamaConfig()
    threads = os.cpu_count() or 1
    tok_s, sample = cpu_llama_tok_s(cfg, BATCH, CTX0, threads)
    line = {"impl": "reference", "metric": B.METRIC, "value": tok_s, "unit": B.UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * BATCH / tok_s, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int4 weights x int8 activations (reference GEMV contract), f32 accumulate", "data": "synthetic",
            "config": llama_config_dict(cfg, 1, BATCH, CTX0),
            "cpu_baseline": {"value": tok_s, "unit": B.UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": tok_s, "unit": B.UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


class _Dist:
    def __init__(self, world, rank, local):
        self.world, self.rank, self.local = world, rank, local


def _barrier(D):
    import torch
    torch.cuda.synchronize()
    if D.world > 1:
        import torch.distributed as dist
        dist.barrier()
        torch.cuda.synchronize()


def _status_over_ranks(D):
    """The library's device status word, worst over the ranks (a rank whose flag wait ran out must not be hidden by
    rank 0 printing its own clean status)."""
    import torch
    from wukong_b200 import device as dev
    st = int(dev.gemm_status())
    if D.world > 1:
        import torch.distributed as dist
        t = torch.tensor([st], dtype=torch.int32, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        st = int(t.item())
    return st


def check_fused_reduce_equals_nccl(D, cfg_full, weights, note):
    """Before anything is timed on several ranks: two layers of the stack at full width, three decode steps, once
    through NCCL and once with the fused peer-memory reduce + add + RMSNorm kernel.  Tokens and residual streams must be
    equal bit for bit.  The fused kernel adds the ranks' partials in rank order; NCCL's all-reduce adds in an order of its
    own, which gives the same bits only for two terms, so on more than two ranks the NCCL side of this check gathers the
    partials (all_gather) and adds them in rank order too.  (Against the plain all-reduce the streams drift like any two
    bf16 evaluations of the stack: 2.4e-4 of the largest element after two layers on 8 ranks.)  Returns the largest row difference
    over row rms (0.0); raises on a mismatch."""
    import torch
    import torch.distributed as dist
    from wukong_b200.llama import LlamaConfig, LlamaDecodeModel, PeerReduce
    device = "cuda:%d" % D.local
    cfg = LlamaConfig(n_layer=2, d_model=cfg_full.d_model, n_head=cfg_full.n_head, n_kv_head=cfg_full.n_kv_head, d_ff=cfg_full.d_ff,
                      vocab=cfg_full.vocab, rope_base=cfg_full.rope_base, eps=cfg_full.eps)

    class TwoLayers:                       # a view of the first two layers of the resident weights
        layers, embed, norm_f, lm_head = weights.layers[:2], weights.embed, weights.norm_f, weights.lm_head
    Bc, mbps = 16, 4

    def sum_in_rank_order(t):
        if D.world == 2:
            dist.all_reduce(t)
            return
        parts = torch.empty((D.world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(parts, t.contiguous())
        acc = parts[0].clone()
        for r in range(1, D.world):
            acc += parts[r]
        t.copy_(acc)

    def make(peer):
        m = LlamaDecodeModel(cfg, TwoLayers, D.rank, D.world, Bc, Bc * mbps, mbps, PAGE, device, sum_in_rank_order,
                             lambda a, b: dist.all_gather_into_tensor(b, a), peer)
        g = torch.Generator(device=device)
        g.manual_seed(5 + D.rank)
        m.kv.k.normal_(generator=g)
        m.kv.v.normal_(generator=g)
        m.block_table.copy_(torch.arange(Bc * mbps, dtype=torch.int32, device=device).view(Bc, mbps))
        m.row_token.copy_(torch.arange(Bc, dtype=torch.int32, device=device) * 37 % cfg.vocab)
        m.row_pos.fill_(20)
        m.row_ctx.fill_(21)
        return m

    peer = PeerReduce(D.rank, D.world, Bc, cfg.d_model, device)
    ma, mb = make(None), make(peer)
    worst = 0.0
    _barrier(D)                            # every rank's buffers and mappings exist before the first peer kernel starts
    for _ in range(3):
        ta = ma.forward(Bc).clone()
        ma.advance(Bc)
        tb = mb.forward(Bc).clone()
        mb.advance(Bc)
        torch.cuda.synchronize()
        if _status_over_ranks(D) != 0:
            raise RuntimeError("a kernel reported an expired wait during the fused-reduce check")
        if not torch.equal(ta, tb):
            raise RuntimeError("tokens differ between the NCCL and the fused peer-memory path")
        xa, xb = ma.x[:Bc].float(), mb.x[:Bc].float()
        rel = ((xa - xb).pow(2).mean(1).sqrt() / xa.pow(2).mean(1).sqrt().clamp_min(1e-30)).max().item()
        worst = max(worst, rel)
        if rel > 0.0 or not torch.equal(ma.x[:Bc], mb.x[:Bc]):
            raise RuntimeError("residual streams differ between the NCCL and the fused path: %g of a row's rms" % rel)
    _barrier(D)
    peer.close()
    del ma, mb, peer
    return worst
    torch.cuda.empty_cache()
    note("fused peer-memory reduce == NCCL all-reduce path on %d ranks (2 layers, 3 steps)" % D.world)


def measure(args, D, clocks, note, use_nccl, cfg, weights):
    """The Llama-shape int4 decode benchmark on the initialised process group: e2e region, device-resident region and
    the two HBM streams timed alone.  Returns the pieces of a bench line (rank-reduced times)."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from wukong_b200._lib import lib, check
    from wukong_b200.llama import LlamaDecodeModel, DecodeStepRunner, PeerReduce

    world, rank, local = D.world, D.rank, D.local
    device = "cuda:%d" % local
    K, W = args.steps, args.warmup
    positions = CTX0 + 2 * (K + W) + 8          # the e2e region and the resident loop both move every sequence on
    mbps = (positions + PAGE - 1) // PAGE
    num_pages = BATCH * mbps
    reduce = (lambda t: dist.all_reduce(t)) if world > 1 else None
    gather = (lambda pairs, allp: dist.all_gather_into_tensor(allp, pairs)) if world > 1 else None
    peer = PeerReduce(rank, world, BATCH, cfg.d_model, device) if (world > 1 and not use_nccl) else None
    m = LlamaDecodeModel(cfg, weights, rank, world, BATCH, num_pages, mbps, PAGE, device, reduce, gather, peer)
    g = torch.Generator(device=device)
    g.manual_seed(1 + rank)
    m.kv.k.normal_(generator=g)
    m.kv.v.normal_(generator=g)
    rng = np.random.default_rng(0)                 # same rows and block table on every rank
    table = rng.permutation(num_pages).astype(np.int32).reshape(BATCH, mbps)
    m.block_table.copy_(torch.from_numpy(table))
    h_rows = torch.zeros(3 * BATCH, dtype=torch.int32).pin_memory()
    h_next = torch.zeros(BATCH, dtype=torch.int32).pin_memory()
    d_rows = m.rows[:3 * BATCH]                    # the model's row block: token | position | visible keys (| slot)
    hr = h_rows.numpy()
    hr[:BATCH] = rng.integers(0, cfg.vocab, BATCH)
    hr[BATCH:2 * BATCH] = CTX0
    hr[2 * BATCH:] = CTX0 + 1
    stream = torch.cuda.Stream(device=device)

    note("weights and KV resident on %d rank(s)" % world)
    _barrier(D)                                    # no rank starts a peer kernel before every rank's buffers exist
    with torch.cuda.stream(stream):
        d_rows.copy_(h_rows, non_blocking=True)
        for _ in range(2):
            m.forward(BATCH)           # eager warm-up: first-use attribute calls, process-group channel setup
    stream.synchronize()
    note("eager forward done")
    with torch.cuda.stream(stream):
        fwd = DecodeStepRunner(m, BATCH, stream, with_advance=False)
        resident = DecodeStepRunner(m, BATCH, stream, with_advance=True)
    stream.synchronize()
    note("step graphs captured (%d segment(s) per step)" % len(fwd.segments))

    def e2e_step():
        with torch.cuda.stream(stream):
            d_rows.copy_(h_rows, non_blocking=True)
            fwd.run()
            h_next.copy_(m.next_tok, non_blocking=True)
        stream.synchronize()
        hr[:BATCH] = h_next.numpy()
        hr[BATCH:] += 1

    for _ in range(W):
        e2e_step()
    _barrier(D)
    clocks.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(K):
        e2e_step()
    e1.record(stream)
    _barrier(D)
    clocks.stop()
    e2e_ms = B.max_over_ranks_ms(e0.elapsed_time(e1), world, "cuda")

    note("e2e region done")
    # ---- device-resident loop: forward + on-device feedback per step
    with torch.cuda.stream(stream):
        d_rows.copy_(h_rows, non_blocking=True)
        for _ in range(W):
            resident.run()
    _barrier(D)
    clocks.start()
    d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        d0.record(stream)
        for _ in range(K):
            resident.run()
        d1.record(stream)
    _barrier(D)
    clocks.stop()
    dev_ms = B.max_over_ranks_ms(d0.elapsed_time(d1), world, "cuda")
    status = _status_over_ranks(D)
    if status != 0:
        raise SystemExit("a kernel reported status %d (expired wait or refused KV position) on some rank" % status)

    # ---- the two HBM streams timed alone on the same state: paged attention (KV) and the four linears (weights)
    p = lambda t: t.data_ptr()
    hd = cfg.head_dim

    def timed(fn, reps=3):
        with torch.cuda.stream(stream):
            fn()
            stream.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=stream):
                fn()
            run = gr.replay
            run()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record(stream)
            for _ in range(reps):
                run()
            a1.record(stream)
        stream.synchronize()
        return a0.elapsed_time(a1) / reps

    def all_attn():
        s = torch.cuda.current_stream().cuda_stream
        for li in range(cfg.n_layer):
            check(lib().wkb_paged_attn_decode(p(m.qkv), m.qkv_w, p(m.kv.k[li]), p(m.kv.v[li]), p(m.block_table), p(m.row_slot),
                                              p(m.row_ctx), p(m.att), 1, m.hq * hd, BATCH, m.hq, m.hkv, hd, PAGE, mbps, m.max_ctx,
                                              m.scale, p(m.scratch), s), "attention")

    def all_gemm():
        for lw in weights.layers:
            m._gemm(lw["wqkv"], m.xn, cfg.d_model, m.qkv, m.qkv_w, 0, BATCH, "qkv")
            m._gemm(lw["wo"], m.att, m.hq * hd, m.part, cfg.d_model, 0, BATCH, "o_proj")
            m._gemm(lw["wgu"], m.xn, cfg.d_model, m.h, m.f, 2, BATCH, "gate_up")
            m._gemm(lw["wdown"], m.h, m.f, m.part, cfg.d_model, 0, BATCH, "down")

    attn_ms = timed(all_attn) / cfg.n_layer
    gemm_ms = timed(all_gemm) / cfg.n_layer
    ctx_now = float(m.row_ctx.float().mean().item())
    attn_bytes = BATCH * ctx_now * 2 * m.hkv * hd * 2 + BATCH * m.hq * hd * (4 + 2) + BATCH * mbps * 4
    layer_w_bytes = sum(lw[k].n * (lw[k].k // 32) * 18 for lw in weights.layers[:1] for k in ("wqkv", "wo", "wgu", "wdown"))
    gemm_bytes = layer_w_bytes + BATCH * (2 * cfg.d_model + m.hq * hd + m.f) * 2 + BATCH * (m.qkv_w + 2 * cfg.d_model) * 4 + BATCH * m.f * 2
    peak, peak_kind = B.hbm_peak()
    step_ms = dev_ms / K
    a_gbs, g_gbs = attn_bytes / (attn_ms * 1e-3) / 1e9, gemm_bytes / (gemm_ms * 1e-3) / 1e9
    # DRAM bytes per attention launch: an ncu capture of this kernel on the batch-64, ctx U[128,4096] case of the
    # micro-suite read and wrote 1.02 x its algorithmic bytes; the traffic grows with the visible tokens
    roofline = {"kernel": "paged GQA decode attention, group of %d" % (m.hq // m.hkv), "bound": "hbm", "achieved": a_gbs,
                "peak": peak, "peak_source": "of " + peak_kind, "unit": "GB/s", "frac": a_gbs / peak,
                "traffic": 1.02 * attn_bytes, "traffic_source": "ncu on the micro-suite's paged_attn case, scaled by visible tokens",
                "algorithmic_bytes_per_launch": attn_bytes, "ms_per_launch": attn_ms, "share_of_step": attn_ms * cfg.n_layer / step_ms,
                "second_stream": {"kernel": "W4A16 GEMM (4 linears of a layer)", "bound": "hbm", "achieved": g_gbs, "unit": "GB/s",
                                  "frac": g_gbs / peak, "algorithmic_bytes_per_layer": gemm_bytes, "ms_per_layer": gemm_ms,
                                  "share_of_step": gemm_ms * cfg.n_layer / step_ms}}
    how = "" if world == 1 else (": NCCL all-reduce" if peer is None else ": fused peer-memory reduce + add + RMSNorm kernel")
    out = {"value": BATCH * K / (dev_ms * 1e-3), "ms_per_step": step_ms, "e2e_value": BATCH * K / (e2e_ms * 1e-3), "e2e_ms_per_step": e2e_ms / K,
           "h2d": int(h_rows.numel() * 4), "d2h": int(h_next.numel() * 4), "launches_per_step": m.launches_per_forward + 1,
           "segments": len(resident.segments), "roofline": roofline, "how": how,
           "weights_bytes_per_gpu": int(weights.q4_bytes()), "kv_bytes_read_per_step_per_gpu": attn_bytes * cfg.n_layer}
    _barrier(D)
    if peer is not None:
        peer.close()
    del fwd, resident, m
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return out


def measure_both(args, D, clocks, note):
    """The `tp_llama_int4` key of the serving benchmark's line: the tensor-parallel step on the same GPUs, with the
    fused reduce (checked against the NCCL path first) and with NCCL all-reduces."""
    import torch
    from wukong_b200.llama import LlamaConfig, LlamaRankWeights
    cfg = LlamaConfig(n_layer=args.layers) if args.layers else LlamaConfig()
    weights = LlamaRankWeights.synth_device(cfg, D.rank, D.world, 0, "cuda:%d" % D.local)
    res = {"metric": B.METRIC, "unit": B.UNIT, "scaling": "strong", "n_gpus": D.world,
           "config": llama_config_dict(cfg, D.world, BATCH, CTX0)}
    if D.world > 1:
        res["fused_vs_nccl_row_rms_diff"] = check_fused_reduce_equals_nccl(D, cfg, weights, note)
        res["fused_equals_nccl"] = True
    r = measure(args, D, clocks, note, False, cfg, weights)
    res.update({"value": r["value"], "ms_per_step": r["ms_per_step"], "e2e_value": r["e2e_value"], "roofline": r["roofline"],
                "reduce": r["how"].lstrip(": ") or "none (one rank)", "graph_segments_per_step": r["segments"]})
    if D.world > 1:
        n = measure(args, D, clocks, note, True, cfg, weights)
        res["nccl_allreduce"] = {"value": n["value"], "ms_per_step": n["ms_per_step"], "e2e_value": n["e2e_value"],
                                 "graph_segments_per_step": n["segments"]}
    del weights
    torch.cuda.empty_cache()
    return res


def run_ours(args):
    import torch
    import torch.distributed as dist
    from wukong_b200 import _lib
    from wukong_b200.llama import LlamaConfig, LlamaRankWeights

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    _lib.require_gpu()
    torch.cuda.set_device(local)
    clocks = B.ClockSampler(local)
    clocks.launch()                 # streams from here on; start() / stop() mark the timed regions
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    D = _Dist(world, rank, local)

    def note(msg):
        if rank == 0:
            print("[llama_int4] " + msg, file=sys.stderr, flush=True)

    cfg = LlamaConfig(n_layer=args.layers) if args.layers else LlamaConfig()
    weights = LlamaRankWeights.synth_device(cfg, rank, world, 0, "cuda:%d" % local)
    if world > 1 and not args.nccl_allreduce:
        check_fused_reduce_equals_nccl(D, cfg, weights, note)
    r = measure(args, D, clocks, note, args.nccl_allreduce, cfg, weights)
    clocks.close()
    K, W = args.steps, args.warmup
    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            tok_s, sample = cpu_llama_tok_s(cfg, BATCH, CTX0, threads)
            cpu = {"value": tok_s, "unit": B.UNIT, "cores": threads, "kind": "port", "sample": sample}
        line = {"metric": B.METRIC, "value": r["value"], "unit": B.UNIT, "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "bf16 (Q4_0 weights dequantised in-register, fp32 accumulate)", "data": "synthetic",
                "config": llama_config_dict(cfg, world, BATCH, CTX0, r["how"]),
                "e2e": {"value": r["e2e_value"], "unit": B.UNIT, "h2d_bytes_per_step": r["h2d"],
                        "d2h_bytes_per_step": r["d2h"], "ms_per_step": r["e2e_ms_per_step"]},
                "gpu_launches": int(r["launches_per_step"] * K), "graph_segments_per_step": r["segments"], "roofline": r["roofline"],
                "cpu_baseline": cpu, "clocks": clocks.summary(),
                "weights_bytes_per_gpu": r["weights_bytes_per_gpu"], "kv_bytes_read_per_step_per_gpu": r["kv_bytes_read_per_step_per_gpu"]}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()

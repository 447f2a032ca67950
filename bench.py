"""Benchmark of the decode hot path: GPT-2-124M-shape batched greedy decode serving, bf16 weights,
paged KV with 16-token pages, 512 concurrent sequences per GPU (prompts uniform in [32, 512]).

    python bench.py --gpus N --steps K --warmup W            # this library (one replica per GPU)
    python bench.py --impl reference --steps K --warmup W    # the CPU port of the reference kernels
    python bench.py --workload llama_int4 --gpus N ...        # second workload: tensor-parallel Q4_0 Llama-shape stack

A step is one decode step of every resident sequence (one token each).  `value` is measured with
all inputs resident in HBM (a self-feeding CUDA graph per step); `e2e` is measured through the public
serving API (`Engine.step`: pinned-host row / block-table upload, graph replay, token download, host
scheduling).  Weights, prompts and their values are synthetic (seeded) stand-ins of the same shapes.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SEQS_PER_GPU = 512
PROMPT_LO, PROMPT_HI = 32, 512
GEN_NOMINAL = 128
PAGE = 16
MBPS = 56                      # block-table columns: 896 tokens per sequence at most
METRIC, UNIT = "decode_tokens_per_s", "tok/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seqs", type=int, default=SEQS_PER_GPU, help="sequences per GPU (default: the named workload)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="gpt2_serving", choices=["gpt2_serving", "llama_int4"],
                    help="gpt2_serving: the headline workload (sequence-sharded replicas); llama_int4: the tensor-parallel Q4_0 stack")
    ap.add_argument("--nccl-allreduce", action="store_true",
                    help="llama_int4 only: sum over ranks with NCCL all-reduce instead of the fused peer-memory kernel")
    ap.add_argument("--layers", type=int, default=0, help="llama_int4 only: run a shorter stack (0: the named 32 layers)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    a.steps = max(a.steps, 1)
    return a


def workload_config(args, n_gpus):
    return {
        "workload": "GPT-2-124M-shape batched greedy decode serving (BASELINE configs[3])",
        "layers": 12, "d_model": 768, "heads": 12, "d_ff": 3072, "vocab": 50257,
        "sequences_per_gpu": args.seqs, "global_sequences": args.seqs * n_gpus,
        "prompt_len": "uniform[%d,%d]" % (PROMPT_LO, PROMPT_HI), "greedy_steps_nominal": GEN_NOMINAL,
        "kv": "paged bf16, %d-token pages" % PAGE, "parallelism": "replicas x%d (sequence sharded, no collective)" % n_gpus,
        "l2": "per-step inputs (249 MB weights + multi-GB KV) exceed the 126 MB L2; no flush needed",
    }


# ------------------------------------------------------------------------------------------------
# clocks: sampled with nvidia-smi while a timed region runs
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None
        self.t_begin = self.t_end = None

    def launch(self):
        """Start nvidia-smi streaming samples (it needs a moment to come up, so this is called well before the
        timed region; `start` / `stop` then mark the region whose samples count)."""
        if self.proc is not None:
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def start(self):
        self.launch()
        self.t_begin = time.perf_counter()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append((time.perf_counter(), parts))

    def stop(self):
        self.t_end = time.perf_counter()
        if self.proc:
            time.sleep(0.06)            # let the sample that covers the end of the region arrive
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [p for (t, p) in self.samples if self.t_begin is not None and self.t_begin <= t <= (self.t_end or t) + 0.06]
        # a region shorter than the sampling period may hold no sample: then the nearest ones around it stand in
        chosen = inside or [p for (_, p) in self.samples[-3:]]
        for p in chosen:
            try:
                sm.append(int(p[0]))
                mx = max(mx, int(p[1]))
            except ValueError:
                continue
            for nm, v in zip(names, p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU port of the reference kernels (the oracle), timed on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_decode_tok_s(weights, cfg, steps, warmup, seqs, threads):
    """Decode steps of `seqs` sequences on the CPU oracle model; contexts drawn from the workload's
    distribution at mid-generation, KV caches pre-filled with seeded random bf16 values (only the
    decode step is timed).  Returns (tok/s, seconds, description)."""
    import numpy as np
    from oracle import binding as orc
    from oracle.gpt2_model import OracleGPT2
    orc.set_threads(threads)
    model = OracleGPT2(cfg, weights, orc)
    rng = np.random.default_rng(1234)
    ctx = rng.integers(PROMPT_LO, PROMPT_HI + 1, seqs) + GEN_NOMINAL // 2
    caches = [model.new_cache(int(c) + steps + warmup + 2) for c in ctx]
    for kc, vc in caches:
        for l in range(cfg.n_layer):
            kc[l][:] = orc.to_bf16_bits(rng.standard_normal(kc[l].shape, dtype=np.float32))
            vc[l][:] = orc.to_bf16_bits(rng.standard_normal(vc[l].shape, dtype=np.float32))
    toks = rng.integers(0, cfg.vocab, seqs).tolist()
    pos = [int(c) for c in ctx]
    kcs, vcs = [c[0] for c in caches], [c[1] for c in caches]
    t0 = None
    for it in range(warmup + steps):
        if it == warmup:
            t0 = time.perf_counter()
        nxt, _ = model.step(toks, pos, kcs, vcs)
        toks = [int(t) for t in nxt]
        pos = [p + 1 for p in pos]
    dt = time.perf_counter() - t0
    desc = "%d sequences x %d decode steps, ctx uniform[%d,%d]+%d, random bf16 KV" % (seqs, steps, PROMPT_LO, PROMPT_HI, GEN_NOMINAL // 2)
    return seqs * steps / dt, dt, desc


def run_reference(args):
    """The reference arm: the reference's CPU implementation cannot be compiled here (Rust), so the
    C++ port of its kernels (the oracle) is what runs, on every host thread."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from wukong_b200.serving import GPT2Config, synth_weights
    cfg = GPT2Config()
    weights = synth_weights(cfg, 0)
    threads = os.cpu_count() or 1
    total = args.steps + args.warmup
    seqs = max(1, min(8, int(150.0 / (total * 0.05))))     # ~0.05 s per token-forward on 8 threads: stay within minutes
    tok_s, dt, desc = cpu_decode_tok_s(weights, cfg, args.steps, args.warmup, seqs, threads)
    n_gpus = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    line = {
        "impl": "reference", "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": n_gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args, n_gpus),
        "cpu_baseline": {"value": tok_s, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": tok_s, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# this library, one replica per GPU
# ------------------------------------------------------------------------------------------------
def shard_prompts(rank, seqs, vocab):
    """This rank's shard of the workload: `seqs` prompts drawn from a rank-specific seeded stream, so
    the global job is world x seqs distinct sequences and no two ranks share one (replicas exchange
    nothing on the data path)."""
    import numpy as np
    rng = np.random.default_rng(100 + rank)
    lens = rng.integers(PROMPT_LO, PROMPT_HI + 1, seqs)
    return [rng.integers(0, vocab, int(L)) for L in lens]


def max_over_ranks_ms(ms, world, device):
    """Whole-job time of a region = the slowest rank's device time."""
    if world == 1:
        return ms
    import torch
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from wukong_b200 import _lib, device as dev
    from wukong_b200._lib import lib, check
    from wukong_b200.serving import GPT2Config, synth_weights, Engine

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    _lib.require_gpu()
    torch.cuda.set_device(local)
    clocks = ClockSampler(local)
    clocks.launch()                 # streams from here on; start() / stop() mark the timed regions
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    K, W, S = args.steps, args.warmup, args.seqs

    cfg = GPT2Config()
    weights = synth_weights(cfg, 0)
    num_pages = S * MBPS
    eng = Engine(cfg, weights, bcap=S, num_pages=num_pages, max_blocks_per_seq=MBPS, max_rows=max(8192, S),
                 prefill_chunk=512, page_tokens=PAGE, device="cuda:%d" % local)
    m, sched = eng.model, eng.sched
    prompts = shard_prompts(rank, S, cfg.vocab)
    lens = np.array([p.size for p in prompts])
    budget = MBPS * PAGE - PROMPT_HI - 8          # decode positions available to every sequence
    need = 2 * (K + W) + 40
    if need > budget:
        raise SystemExit("steps + warmup too large for the block-table width: need %d decode positions, have %d" % (need, budget))
    gen_len = max(GEN_NOMINAL, need + 64)         # nobody retires inside the measurement
    for pr in prompts:
        eng.enqueue(pr, gen_len)

    # ---- prefill (untimed): run engine steps until every sequence is decoding
    t_pre = time.perf_counter()
    pre_steps = 0
    while True:
        n = sched.plan_step()
        decode_only = n <= S and np.array_equal(sched.sample_row[sched.row_slot[:n]], np.arange(n, dtype=np.int32)) and n == S
        # undo is impossible, so run this planned step through the engine's own machinery
        sched_commit_via_engine(eng, n)
        pre_steps += 1
        if decode_only:
            break
        if pre_steps > 4096:
            raise SystemExit("prefill did not converge")
    torch.cuda.synchronize()
    t_pre = time.perf_counter() - t_pre

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms):
        return max_over_ranks_ms(ms, world, "cuda")


    # ---- e2e: the public serving API, host buffers in and out every step
    for _ in range(W):
        eng.step()
    h2d0, d2h0 = eng.h2d_bytes, eng.d2h_bytes
    barrier()
    clocks.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(eng.stream)
    emitted = 0
    for _ in range(K):
        emitted += eng.step()
    e1.record(eng.stream)
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1))
    h2d_step, d2h_step = (eng.h2d_bytes - h2d0) // K, (eng.d2h_bytes - d2h0) // K
    assert emitted == S * K, (emitted, S * K)

    # ---- device-resident loop: extend every block table ahead, then self-feeding graph replays
    for slot in range(S):
        sched.manager.reserve(slot, K + W + 2)
    sched.manager.flat_block_table(eng.h_table.numpy().view(np.uint32).reshape(S, -1))
    with torch.cuda.stream(eng.stream):
        m.block_table.view(-1).copy_(eng.h_table, non_blocking=True)
        # rows for the next step, as the scheduler would lay them out (slot i -> row i)
        hr = eng.h_rows.numpy()
        R = m.max_rows
        ctx_now = sched.manager.ctx_lens().astype(np.int32) - (K + W + 2)
        hr[0 * R:0 * R + S] = eng.h_next.numpy()[:S]
        hr[1 * R:1 * R + S] = ctx_now
        hr[2 * R:2 * R + S] = np.arange(S)
        hr[3 * R:3 * R + S] = ctx_now + 1
        hr[4 * R:4 * R + S] = np.arange(S)
        eng.d_rows.copy_(eng.h_rows, non_blocking=True)
    eng.stream.synchronize()
    graph = eng.capture_resident_loop()
    with torch.cuda.stream(eng.stream):
        for _ in range(W):
            graph.replay()
    barrier()
    d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(eng.stream):
        d0.record(eng.stream)
        for _ in range(K):
            graph.replay()
        d1.record(eng.stream)
    barrier()
    clocks.stop()
    dev_ms = max_over_ranks(d0.elapsed_time(d1))
    if dev.gemm_status() != 0:
        raise SystemExit("tensor-core GEMM reported an expired pipeline wait")
    launches_per_step = m.launches_per_forward + 1

    # ---- dominant kernel (paged decode attention) timed alone on the same state, same stream
    ctx_end = (ctx_now + 1 + K + W).astype(np.int64)           # visible keys per row during this loop
    d = cfg.d_model
    reps = 5
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    p = lambda t: t.data_ptr()
    with torch.cuda.stream(eng.stream):
        def attn(li):
            s = torch.cuda.current_stream().cuda_stream
            check(lib().wkb_paged_attn_decode(p(m.qkv), 3 * d, p(m.kv.k[li]), p(m.kv.v[li]), p(m.block_table), p(m.row_slot), p(m.row_ctx),
                                              p(m.att), 1, d, S, cfg.n_head, cfg.n_head, cfg.head_dim, PAGE, MBPS, m.max_ctx, m.scale,
                                              p(m.scratch), s), "attn")
        for li in range(cfg.n_layer):
            attn(li)
        eng.stream.synchronize()
        ag = torch.cuda.CUDAGraph()
        with torch.cuda.graph(ag, stream=eng.stream):
            for li in range(cfg.n_layer):
                attn(li)
        ag.replay()
        a0.record(eng.stream)
        for _ in range(reps):
            ag.replay()
        a1.record(eng.stream)
    eng.stream.synchronize()
    attn_ms = a0.elapsed_time(a1) / (reps * cfg.n_layer)
    # algorithmic bytes of one launch: K and V of every visible token (bf16) + q in (f32) + out (bf16)
    attn_bytes = float(ctx_end.sum()) * 2 * d * 2 + S * d * (4 + 2) + S * 4 * 2
    peak, peak_kind = hbm_peak()
    achieved = attn_bytes / (attn_ms * 1e-3) / 1e9
    # DRAM traffic per launch: 1.04 x the algorithmic bytes, from the ncu capture summarised in
    # profiles/paged_attn_decode_ncu.md (taken at 128 sequences; traffic grows with the visible tokens)
    roofline = {"kernel": "paged_attn_decode_kernel<64,1> (+ chunk merge)", "bound": "hbm", "achieved": achieved, "peak": peak,
                "peak_source": "of " + peak_kind, "unit": "GB/s", "frac": achieved / peak, "traffic": 1.04 * attn_bytes,
                "traffic_source": "ncu at 128 sequences, scaled by visible tokens",
                "algorithmic_bytes_per_launch": attn_bytes, "ms_per_launch": attn_ms,
                "share_of_step": attn_ms * cfg.n_layer / (dev_ms / K)}

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            tok_s, dt, desc = cpu_decode_tok_s(weights, cfg, 64, 1, 16, threads)      # about 10-15 s of host work
            cpu = {"value": tok_s, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc, "seconds": dt}
        line = {
            "metric": METRIC, "value": world * S * K / (dev_ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": dev_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(args, world),
            "e2e": {"value": world * S * K / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": int(h2d_step),
                    "d2h_bytes_per_step": int(d2h_step), "ms_per_step": e2e_ms / K},
            "gpu_launches": int(launches_per_step * K), "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks.summary(),
            "prefill": {"steps": pre_steps, "seconds": t_pre, "prompt_tokens": int(lens.sum())},
            "mean_ctx": float(ctx_end.mean()),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def sched_commit_via_engine(eng, n_planned):
    """Run a step whose rows were already planned (used by the prefill loop, which inspects the plan
    before running it)."""
    eng._planned = n_planned
    eng.step()


if __name__ == "__main__":
    a = parse()
    if a.workload == "llama_int4":
        import bench_llama
        (bench_llama.run_reference if a.impl == "reference" else bench_llama.run_ours)(a)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)

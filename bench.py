"""Benchmark of the decode hot path: GPT-2-124M-shape batched greedy decode serving, bf16 weights, paged KV with
16-token pages, 512 concurrent sequences (prompts uniform in [32, 512]) sharded by sequence over the GPUs.

    python bench.py --gpus N --steps K --warmup W            # this library, one replica per GPU
    python bench.py --impl reference --steps K --warmup W    # the CPU port of the reference kernels
    python bench.py --workload llama_int4 --gpus N ...       # only the second workload: tensor-parallel Q4_0 Llama-shape stack

A step is one decode step of every resident sequence (one token each).  The job is the fixed 512-sequence batch:
with N GPUs every rank serves 512 / N of them as an independent replica (no collective on the data path), so
`value` is a strong-scaling number; the per-GPU-512 (weak) figure is reported beside it under `weak` when N > 1.
`value` is measured with all inputs resident in HBM (a self-feeding CUDA graph per step); `e2e` through the public
serving API (`Engine.step`: pinned-host row / block-table upload, graph replay, token download, host scheduling).
Extra keys of the line: `continuous_batching` (a second timed region with admissions, prompt chunks and retirements
inside it), `tp_llama_int4` (the tensor-parallel Llama-shape int4 step on the same N GPUs: fused peer-memory reduce
and the NCCL all-reduce baseline) and, at N = 1, `microsuite` (per-kernel roofline fractions of the kernel
micro-suite).  Weights, prompts and their values are synthetic (seeded) stand-ins of the same shapes.
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

GLOBAL_SEQS = 512
PROMPT_LO, PROMPT_HI = 32, 512
GEN_NOMINAL = 128
PAGE = 16
N_POS = 1024                   # learned positions of the GPT-2 shape: no sequence may grow past this
CPU_SAMPLE_SEQS = 64           # the one CPU sample definition: a step = one decode step of 64 of the workload's sequences, run as one batch
METRIC, UNIT = "decode_tokens_per_s", "tok/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=48)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seqs", type=int, default=0, help="sequences per GPU (default: 512 / number of GPUs, the named workload)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the continuous-batching region, the tensor-parallel "
                    "Llama-shape step, the weak-scaling figure and the micro-suite (for profiling runs)")
    ap.add_argument("--workload", default="gpt2_serving", choices=["gpt2_serving", "llama_int4"],
                    help="gpt2_serving: the headline workload (sequence-sharded replicas); llama_int4: only the tensor-parallel Q4_0 stack")
    ap.add_argument("--nccl-allreduce", action="store_true",
                    help="llama_int4 only: sum over ranks with NCCL all-reduce instead of the fused peer-memory kernel")
    ap.add_argument("--layers", type=int, default=0, help="llama_int4 only: run a shorter stack (0: the named 32 layers)")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    a.steps = max(a.steps, 1)
    return a


def workload_config(seqs_per_gpu, n_gpus):
    return {
        "workload": "GPT-2-124M-shape batched greedy decode serving, %d concurrent sequences sharded over the GPUs" % (seqs_per_gpu * n_gpus),
        "layers": 12, "d_model": 768, "heads": 12, "d_ff": 3072, "vocab": 50257,
        "sequences_per_gpu": seqs_per_gpu, "global_sequences": seqs_per_gpu * n_gpus,
        "prompt_len": "uniform[%d,%d]" % (PROMPT_LO, PROMPT_HI), "greedy_steps_nominal": GEN_NOMINAL,
        "kv": "paged bf16, %d-token pages" % PAGE, "parallelism": "replicas x%d (sequence sharded, no collective)" % n_gpus,
        "l2": "per-step inputs (249 MB weights + KV of every resident sequence) exceed the 126 MB L2; no flush needed",
    }


# ------------------------------------------------------------------------------------------------
# clocks: sampled with nvidia-smi while a timed region runs
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None
        self.regions = []

    def launch(self):
        """Start nvidia-smi streaming samples (it needs a moment to come up, so this is called well before the
        timed regions; `start` / `stop` then mark the regions whose samples count)."""
        if self.proc is not None:
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def start(self):
        self.launch()
        self.regions.append([time.perf_counter(), None])

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append((time.perf_counter(), parts))

    def stop(self):
        if self.regions and self.regions[-1][1] is None:
            self.regions[-1][1] = time.perf_counter()

    def close(self):
        if self.proc:
            time.sleep(0.05)            # let the sample that covers the end of the last region arrive
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass
            self.proc = None

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside = [p for (t, p) in self.samples if any(b <= t <= (e or t) + 0.03 for b, e in self.regions)]
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
def cpu_decode_tok_s(weights, cfg, steps, warmup, threads):
    """Decode steps of CPU_SAMPLE_SEQS sequences on the CPU oracle model, batched the way the reference's CPU path runs
    them: every GEMM over all the sequences' rows at once (weights read once per call), dense fp32 KV caches, one call to
    the batched KV-cache attention kernel per layer.  Contexts are drawn from the workload's distribution at
    mid-generation, the caches pre-filled with seeded random bf16 values (only the decode step is timed).  Returns
    (tok/s, seconds, description).  Both the `cpu_baseline` key of this library's line and the reference arm time exactly
    this sample."""
    import numpy as np
    from oracle import binding as orc
    from oracle.gpt2_model import OracleGPT2
    orc.set_threads(threads)
    seqs = CPU_SAMPLE_SEQS
    model = OracleGPT2(cfg, weights, orc)
    rng = np.random.default_rng(1234)
    ctx = rng.integers(PROMPT_LO, PROMPT_HI + 1, seqs) + GEN_NOMINAL // 2
    cap = (int(ctx.max()) + steps + warmup + 2 + 15) // 16 * 16
    K = [orc.from_bf16_bits(orc.to_bf16_bits(rng.standard_normal((seqs, cap, cfg.d_model), dtype=np.float32))).reshape(seqs, cap, cfg.d_model)
         for _ in range(cfg.n_layer)]
    V = [orc.from_bf16_bits(orc.to_bf16_bits(rng.standard_normal((seqs, cap, cfg.d_model), dtype=np.float32))).reshape(seqs, cap, cfg.d_model)
         for _ in range(cfg.n_layer)]
    toks = rng.integers(0, cfg.vocab, seqs).tolist()
    pos = [int(c) for c in ctx]
    t0 = None
    for it in range(warmup + steps):
        if it == warmup:
            t0 = time.perf_counter()
        nxt, _ = model.step_dense_cache(toks, pos, K, V)
        toks = [int(t) for t in nxt]
        pos = [p + 1 for p in pos]
    dt = time.perf_counter() - t0
    desc = "%d of the workload's sequences x %d decode steps as one batch, ctx uniform[%d,%d]+%d, random bf16-valued fp32 KV" % (
        seqs, steps, PROMPT_LO, PROMPT_HI, GEN_NOMINAL // 2)
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
    steps = min(args.steps, 64)             # about 0.2 s per 64-sequence step: the run stays within a few minutes
    tok_s, dt, desc = cpu_decode_tok_s(weights, cfg, steps, min(args.warmup, 3), threads)
    n_gpus = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    line = {
        "impl": "reference", "metric": METRIC, "value": tok_s, "unit": UNIT, "n_gpus": n_gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(GLOBAL_SEQS // n_gpus, n_gpus),
        "cpu_baseline": {"value": tok_s, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc, "seconds": dt},
        "e2e": {"value": tok_s, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# this library, one replica per GPU
# ------------------------------------------------------------------------------------------------
def shard_prompts(rank, seqs, vocab, stream=0):
    """This rank's shard of the workload: `seqs` prompts drawn from a rank-specific seeded stream, so
    the global job is world x seqs distinct sequences and no two ranks share one (replicas exchange
    nothing on the data path)."""
    import numpy as np
    rng = np.random.default_rng(100 + rank + 1000 * stream)
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


class Dist:
    """The few process-group calls the bench needs (barrier, max over ranks); one rank: no-ops."""

    def __init__(self, world, rank, local):
        self.world, self.rank, self.local = world, rank, local

    def barrier(self):
        import torch
        torch.cuda.synchronize()
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
            torch.cuda.synchronize()

    def max_ms(self, ms):
        return max_over_ranks_ms(ms, self.world, "cuda")

    def sum_int(self, v):
        if self.world == 1:
            return int(v)
        import torch
        import torch.distributed as dist
        t = torch.tensor([int(v)], dtype=torch.int64, device="cuda")
        dist.all_reduce(t)
        return int(t.item())


def measure_serving(args, S, D, weights, cfg, clocks, label):
    """The decode benchmark on this rank's S sequences: prefill (untimed), the e2e region through Engine.step, the
    device-resident region, and the dominant kernel timed alone.  Returns a dict of rank-reduced results."""
    import numpy as np
    import torch
    from wukong_b200 import device as dev
    from wukong_b200._lib import lib, check
    from wukong_b200.serving import Engine

    K, W = args.steps, args.warmup
    need = 2 * (K + W) + 40                        # decode positions the two timed regions consume per sequence
    gen_len = max(GEN_NOMINAL, need + 64)          # nobody retires inside these two regions (the continuous-batching region is separate)
    if PROMPT_HI + gen_len > N_POS:
        raise SystemExit("steps + warmup too large for the %d learned positions: need %d decode positions" % (N_POS, need))
    mbps = max(56, (PROMPT_HI + gen_len + 8 + PAGE - 1) // PAGE)
    eng = Engine(cfg, weights, bcap=S, num_pages=S * mbps, max_blocks_per_seq=mbps, max_rows=max(8192, S),
                 prefill_chunk=512, page_tokens=PAGE, device="cuda:%d" % D.local)
    m, sched = eng.model, eng.sched
    prompts = shard_prompts(D.rank, S, cfg.vocab)
    lens = np.array([p.size for p in prompts])
    for pr in prompts:
        eng.enqueue(pr, gen_len)

    # ---- prefill (untimed): engine steps until every sequence is decoding
    t_pre = time.perf_counter()
    pre_steps = 0
    while True:
        n = sched.plan_step()
        decode_only = n == S and np.array_equal(sched.sample_row[sched.row_slot[:n]], np.arange(n, dtype=np.int32))
        eng._planned = n                           # the plan was inspected first; the engine runs exactly this plan
        eng.step()
        pre_steps += 1
        if decode_only:
            break
        if pre_steps > 4096:
            raise SystemExit("prefill did not converge")
    torch.cuda.synchronize()
    t_pre = time.perf_counter() - t_pre

    # ---- e2e: the public serving API, host buffers in and out every step
    for _ in range(W):
        eng.step()
    h2d0, d2h0 = eng.h2d_bytes, eng.d2h_bytes
    D.barrier()
    clocks.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(eng.stream)
    emitted = 0
    for _ in range(K):
        emitted += eng.step()
    e1.record(eng.stream)
    D.barrier()
    clocks.stop()
    e2e_ms = D.max_ms(e0.elapsed_time(e1))
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
    D.barrier()
    clocks.start()
    d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(eng.stream):
        d0.record(eng.stream)
        for _ in range(K):
            graph.replay()
        d1.record(eng.stream)
    D.barrier()
    clocks.stop()
    dev_ms = D.max_ms(d0.elapsed_time(d1))
    if dev.gemm_status() != 0:
        raise SystemExit("a kernel reported an expired wait or a refused KV position")
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
            check(lib().wkb_paged_attn_decode(p(m.q), d, p(m.kv.k[li]), p(m.kv.v[li]), p(m.block_table), p(m.row_slot), p(m.row_ctx),
                                              p(m.att), 1, d, S, cfg.n_head, cfg.n_head, cfg.head_dim, PAGE, mbps, m.max_ctx, m.scale,
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
    # DRAM traffic per launch: an ncu capture of this kernel at 128 sequences read and wrote 1.04 x its algorithmic
    # bytes (every K/V byte once, plus the output rows); the traffic grows with the visible tokens, so that factor is
    # applied to this launch's algorithmic bytes
    roofline = {"kernel": "paged_attn_decode_kernel<64,1>", "bound": "hbm", "achieved": achieved, "peak": peak,
                "peak_source": "of " + peak_kind, "unit": "GB/s", "frac": achieved / peak, "traffic": 1.04 * attn_bytes,
                "traffic_source": "ncu at 128 sequences, scaled by visible tokens",
                "algorithmic_bytes_per_launch": attn_bytes, "ms_per_launch": attn_ms,
                "share_of_step": attn_ms * cfg.n_layer / (dev_ms / K)}
    # whole-step algorithmic bytes: every weight once + K/V of every visible token over the 12 layers
    step_bytes = 2.0 * cfg.n_params() - 2.0 * cfg.n_pos * d + float(ctx_end.sum()) * 2 * d * 2 * cfg.n_layer
    total_seqs = D.sum_int(S)
    out = {"label": label, "seqs_per_gpu": S, "global_seqs": total_seqs, "dev_ms": dev_ms, "e2e_ms": e2e_ms,
           "value": total_seqs * K / (dev_ms * 1e-3), "e2e_value": total_seqs * K / (e2e_ms * 1e-3),
           "h2d": int(h2d_step), "d2h": int(d2h_step), "launches_per_step": int(launches_per_step), "roofline": roofline,
           "whole_step_hbm_frac": step_bytes / (dev_ms / K * 1e-3) / 1e9 / peak,
           "prefill": {"steps": pre_steps, "seconds": t_pre, "prompt_tokens": int(lens.sum())}, "mean_ctx": float(ctx_end.mean())}
    del graph, ag, eng, m, sched
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return out


def measure_continuous_batching(args, S, D, weights, cfg, clocks):
    """A second timed region in which the scheduler does its whole job: 2 x S requests of 128 greedy tokens each against
    S slots, so prompt chunks, admissions into freed slots and retirements all happen inside the timing (the reference's
    goodput bench has the same shape: crates/wukong_codegen_gpu/src/serving.rs:3845-3992).  Goodput counts generated
    tokens only; the prompt tokens pushed through the model in the same time are reported beside it."""
    import numpy as np
    import torch
    from wukong_b200 import device as dev
    from wukong_b200.serving import Engine
    mbps = (PROMPT_HI + GEN_NOMINAL + 8 + PAGE - 1) // PAGE
    eng = Engine(cfg, weights, bcap=S, num_pages=S * mbps, max_blocks_per_seq=mbps, max_rows=max(8192, S),
                 prefill_chunk=512, page_tokens=PAGE, device="cuda:%d" % D.local)
    warm = shard_prompts(D.rank, min(S, 8), cfg.vocab, stream=2)
    for pr in warm:                                # untimed warm-up: captures the graph, touches every kernel
        eng.enqueue(pr, 4)
    eng.run_until_idle()
    prompts = shard_prompts(D.rank, 2 * S, cfg.vocab, stream=1)
    for pr in prompts:
        eng.enqueue(pr, GEN_NOMINAL)
    base_emitted, base_done = eng.sched.emitted(), eng.sched.completed()
    D.barrier()
    clocks.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(eng.stream)
    steps = eng.run_until_idle()
    e1.record(eng.stream)
    D.barrier()
    clocks.stop()
    ms = D.max_ms(e0.elapsed_time(e1))
    gen = D.sum_int(eng.sched.emitted() - base_emitted)
    prompt_tokens = D.sum_int(int(sum(p.size for p in prompts)))
    done = D.sum_int(eng.sched.completed() - base_done)
    if dev.gemm_status() != 0:
        raise SystemExit("a kernel reported an expired wait or a refused KV position")
    out = {"value": gen / (ms * 1e-3), "unit": "generated tok/s (whole job, admissions, prompt chunks and retirements inside the timed region)",
           "requests": done, "generated_tokens": gen, "prompt_tokens": prompt_tokens, "prompt_tok_per_s": prompt_tokens / (ms * 1e-3),
           "engine_steps_rank0": steps, "seconds": ms * 1e-3, "slots_per_gpu": S, "requests_per_gpu": 2 * S, "tokens_per_request": GEN_NOMINAL}
    del eng
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist
    from wukong_b200 import _lib
    from wukong_b200.serving import GPT2Config, synth_weights

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    _lib.require_gpu()
    torch.cuda.set_device(local)
    clocks = ClockSampler(local)
    clocks.launch()                 # streams from here on; start() / stop() mark the timed regions
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    D = Dist(world, rank, local)
    K, W = args.steps, args.warmup
    S = args.seqs or max(1, GLOBAL_SEQS // world)
    cfg = GPT2Config()
    weights = synth_weights(cfg, 0)

    def note(msg):
        if rank == 0:
            print("[bench] " + msg, file=sys.stderr, flush=True)

    main = measure_serving(args, S, D, weights, cfg, clocks, "strong")
    note("serving regions done: %.3f ms/step" % (main["dev_ms"] / K))
    extras = {}
    if not args.no_extras:
        if world > 1 and not args.seqs:
            weak = measure_serving(args, GLOBAL_SEQS, D, weights, cfg, clocks, "weak")
            extras["weak"] = {"value": weak["value"], "unit": UNIT, "sequences_per_gpu": GLOBAL_SEQS, "global_sequences": weak["global_seqs"],
                              "ms_per_step": weak["dev_ms"] / K, "e2e_value": weak["e2e_value"], "roofline_frac": weak["roofline"]["frac"],
                              "whole_step_hbm_frac": weak["whole_step_hbm_frac"]}
            note("weak-scaling figure done")
        extras["continuous_batching"] = measure_continuous_batching(args, S, D, weights, cfg, clocks)
        note("continuous-batching region done")
        import bench_llama
        try:
            extras["tp_llama_int4"] = bench_llama.measure_both(args, D, clocks, note)
        except Exception as exc:            # the headline line must still be printed
            extras["tp_llama_int4"] = {"error": "%s: %s" % (type(exc).__name__, exc)}
        if world == 1:
            from wukong_b200 import microbench
            try:
                with open(os.devnull, "w") as sink:
                    res = microbench.run(out=sink)
                extras["microsuite"] = [{k: r[k] for k in ("case", "shape", "us", "achieved", "unit", "bound", "frac", "peak_source") if k in r} for r in res]
            except Exception as exc:
                extras["microsuite"] = {"error": "%s: %s" % (type(exc).__name__, exc)}
            note("micro-suite done")
    clocks.close()

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            tok_s, dt, desc = cpu_decode_tok_s(weights, cfg, min(K, 64), 3, threads)      # the reference arm's sample definition
            cpu = {"value": tok_s, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc, "seconds": dt}
        line = {
            "metric": METRIC, "value": main["value"], "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": main["dev_ms"] / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(S, world),
            "e2e": {"value": main["e2e_value"], "unit": UNIT, "h2d_bytes_per_step": main["h2d"],
                    "d2h_bytes_per_step": main["d2h"], "ms_per_step": main["e2e_ms"] / K},
            "gpu_launches": int(main["launches_per_step"] * K), "roofline": main["roofline"], "cpu_baseline": cpu, "clocks": clocks.summary(),
            "whole_step_hbm_frac": main["whole_step_hbm_frac"], "prefill": main["prefill"], "mean_ctx": main["mean_ctx"],
        }
        line.update(extras)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    a = parse()
    if a.workload == "llama_int4":
        import bench_llama
        (bench_llama.run_reference if a.impl == "reference" else bench_llama.run_ours)(a)
    elif a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)

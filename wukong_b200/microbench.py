"""Kernel micro-suite: per-kernel throughput against the measured roofline.

    python -m wukong_b200.microbench            # prints one JSON line per case

Cases (seeded synthetic inputs of the named shapes):
  gemm_bf16      C = A.B^T, M = N = K in {1024, 4096, 8192}, inputs ~N(0,1), fp32 accumulate
  gemv_q4_0      y = W.x, W 4096x4096 and 11008x4096 Q4_0 (f16 scale ~|N(0,0.02)|, nibbles uniform),
                 reference contract (Q8 activation, exact block dots) and bf16-activation variant
  rmsnorm/softmax  8192 rows x 4096, bf16
  gemm_q4_0_bf16 batch 64 against the three linear shapes of a 7B-shape block (fused QKV 6144x4096, gate/up
                 22016x4096 with the SwiGLU epilogue, down projection 4096x11008), tensor-core W4A16
  paged_attn     batch 64, ctx uniform [128, 4096], 32 q heads / 8 kv heads, d = 128, bf16, 16-token pages
Memory-bound kernels rotate through enough distinct operand sets to exceed the 126 MB L2; every case
is timed with CUDA events over one CUDA graph of `reps` launches after warm-up.
"""
import json
import math
import os
import sys

import numpy as np
import torch

from . import device as dev
from ._lib import lib, check, require_gpu

L2_BYTES = 126 << 20


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as fh:
            p = json.load(fh)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def sustained_tensor_peak():
    """The measured bf16 throughput of a seconds-long GEMM loop under the power cap (None when the file is absent)."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as fh:
            return float(json.load(fh)["bf16_tflops_sustained"])
    except Exception:
        return None


def time_graph(fn, reps, warm=3):
    """Average microseconds per call of `fn(i)`, i = 0..reps-1, replayed as one CUDA graph."""
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for i in range(min(warm, reps)):
            fn(i)
        st.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for i in range(reps):
                fn(i)
        g.replay()
        st.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        g.replay()
        e1.record(st)
        st.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def _s():
    return torch.cuda.current_stream().cuda_stream


def case_gemm(size, hbm, tf, src):
    a = torch.randn(size, size, device="cuda").to(torch.bfloat16)
    b = torch.randn(size, size, device="cuda").to(torch.bfloat16)
    c = torch.empty(size, size, device="cuda")
    # Ten launches back to back as one graph (no launch overhead; under the board's power cap the SM clock settles near
    # 1.35 GHz within a few milliseconds of dense tensor work, the regime the sustained peak was measured in), and the launch
    # alone (best of 10 single launches bracketed by CUDA events, the way the burst peak was taken; launch latency makes this
    # one meaningless below about 100 us).
    us = time_graph(lambda i: dev.gemm_bf16_nt(a, b, out=c), 10)
    best = float("inf")
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        dev.gemm_bf16_nt(a, b, out=c)
        e1.record()
        e1.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e3)
    t = 2 * size ** 3 / us / 1e6
    out = {"case": "gemm_bf16", "shape": [size] * 3, "us": us, "achieved": t, "unit": "TFLOP/s", "bound": "tensor", "peak": tf,
           "frac": t / tf, "peak_source": "of " + src, "single_launch_us": best, "single_launch_tflops": 2 * size ** 3 / best / 1e6}
    sustained = sustained_tensor_peak()
    if sustained:
        out["frac_of_sustained_peak"] = t / sustained
    return out


def case_decode_gemms(hbm, tf, src):
    """The dense GEMMs of one GPT-2-124M-shape layer at a decode batch of 512 rows, launched the way the serving step
    launches them: O projection as a residual update with its K slices summed inside a cluster, FC (+bias, GELU, bf16 out),
    down projection as a residual update.  Weights rotate over 12 layer copies (170 MB), activations stay in L2.  The
    figure is the time of the three launches; they are bound by their latency chains (dependency wait, first tile,
    K steps at TMA latency / ring depth, epilogue), not by the 10.6 MB of weights they stream."""
    L = lib()
    rows, d, ff, layers = 512, 768, 3072, 12
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    w_o = [(torch.randn(d, d, device="cuda", generator=g) * 0.02).to(torch.bfloat16) for _ in range(layers)]
    w_fc = [(torch.randn(ff, d, device="cuda", generator=g) * 0.02).to(torch.bfloat16) for _ in range(layers)]
    w_pr = [(torch.randn(d, ff, device="cuda", generator=g) * 0.02).to(torch.bfloat16) for _ in range(layers)]
    b_d = torch.zeros(d, device="cuda")
    b_ff = torch.zeros(ff, device="cuda")
    att = torch.randn(rows, d, device="cuda", generator=g).to(torch.bfloat16)
    h = torch.randn(rows, d, device="cuda", generator=g).to(torch.bfloat16)
    x = torch.zeros(rows, d, device="cuda")
    ffb = torch.empty(rows, ff, device="cuda", dtype=torch.bfloat16)
    assert L.wkb_gemm_bf16_addto_slices(rows, d, d) > 0 and L.wkb_gemm_bf16_addto_slices(rows, d, ff) > 0
    prev = L.wkb_gemm_b_static(1)

    def seq(i):
        j = i % layers
        s = _s()
        check(L.wkb_gemm_bf16_nt_addto(att.data_ptr(), d, w_o[j].data_ptr(), d, x.data_ptr(), d, rows, d, d, b_d.data_ptr(), s), "addto")
        dev.gemm_bf16_nt(h, w_fc[j], bias=b_ff, act=2, out=ffb)
        check(L.wkb_gemm_bf16_nt_addto(ffb.data_ptr(), ff, w_pr[j].data_ptr(), ff, x.data_ptr(), d, rows, d, ff, b_d.data_ptr(), s), "addto")

    try:
        us = time_graph(seq, 24)
    finally:
        L.wkb_gemm_b_static(prev)
    bytes_w = 2.0 * (d * d + 2 * d * ff)
    gbs = bytes_w / us / 1e3
    return {"case": "decode_gemms", "shape": {"rows": rows, "d_model": d, "d_ff": ff}, "us": us, "achieved": gbs, "unit": "GB/s", "bound": "hbm",
            "peak": hbm, "frac": gbs / hbm, "algorithmic_bytes": bytes_w, "launches": 3, "peak_source": "of " + src,
            "note": "three dependent launches of 4-6 us each; latency-bound"}


def q4_weights(n, k, rng):
    nb = k // 32
    raw = rng.integers(0, 256, (n * nb, 18), dtype=np.uint8)
    sc = np.abs(rng.standard_normal(n * nb) * 0.02).astype(np.float16).view(np.uint16)
    raw[:, 0] = sc & 0xFF
    raw[:, 1] = sc >> 8
    return raw.reshape(-1)


def case_gemv_q4(n, k, variant, hbm, tf, src):
    rng = np.random.default_rng(0)
    nb = k // 32
    bytes_w = n * nb * 18
    copies = max(2, L2_BYTES * 3 // bytes_w + 1)
    planes = []
    raw = torch.from_numpy(q4_weights(n, k, rng)).cuda()
    for _ in range(copies):
        planes.append(dev.q_split(raw, n * nb, q4=True))
    x = torch.randn(k, device="cuda")
    xb = x.to(torch.bfloat16)
    y = torch.empty(n, device="cuda")
    xq, dx, sx = dev.quantize_act(x)
    if variant == "contract":
        def fn(i):
            qs, d = planes[i % copies]
            check(lib().wkb_quantize_act(x.data_ptr(), k, xq.data_ptr(), dx.data_ptr(), sx.data_ptr(), _s()), "qact")
            dev.gemv_q_contract(qs, d, xq, dx, sx, n, k, out=y)
    else:
        def fn(i):
            qs, d = planes[i % copies]
            dev.gemv_q4_0_bf16x(qs, d, xb, n, k, out=y)
    us = time_graph(fn, copies * 2)
    alg = bytes_w + 2 * k + 4 * n
    gbs = alg / us / 1e3
    return {"case": "gemv_q4_0_" + variant, "shape": [n, k], "us": us, "achieved": gbs, "unit": "GB/s", "bound": "hbm", "peak": hbm,
            "frac": gbs / hbm, "algorithmic_bytes": alg, "rotating_copies": copies, "peak_source": "of " + src}


def case_gemm_q4(m, n, k, mode, hbm, tf, src):
    """W4A16 tensor-core GEMM at decode batch m: bound by the weight stream (18 B per 32 weights)."""
    rng = np.random.default_rng(0)
    nb = k // 32
    bytes_w = n * nb * 18
    copies = max(2, L2_BYTES * 3 // bytes_w + 1)
    raw = torch.from_numpy(q4_weights(n, k, rng)).cuda()
    ws_ = [dev.Q4Weight.from_raw(raw, n, k) for _ in range(copies)]
    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    out = torch.empty(m, n // 2 if mode == 2 else n, dtype=torch.float32 if mode == 0 else torch.bfloat16, device="cuda")
    work = dev.gemm_q4_workspace(n, k)
    us = time_graph(lambda i: dev.gemm_q4_0_bf16_nt(ws_[i % copies], x, mode=mode, out=out, workspace=work), copies * 2)
    alg = bytes_w + 2 * m * k + out.numel() * out.element_size()
    gbs = alg / us / 1e3
    return {"case": "gemm_q4_0_bf16" + ("_swiglu" if mode == 2 else ""), "shape": [m, n, k], "us": us, "achieved": gbs, "unit": "GB/s",
            "bound": "hbm", "peak": hbm, "frac": gbs / hbm, "algorithmic_bytes": alg, "tflops": 2 * m * n * k / us / 1e6,
            "rotating_copies": copies, "peak_source": "of " + src}


def case_norm(op, hbm, tf, src):
    rows, cols = 8192, 4096
    copies = 4                                   # 4 x 64 MB inputs
    xs = [torch.randn(rows, cols, device="cuda").to(torch.bfloat16) for _ in range(copies)]
    out = torch.empty(rows, cols, dtype=torch.bfloat16, device="cuda")
    g = torch.ones(cols, device="cuda")
    us = time_graph(lambda i: dev.norm_fast(xs[i % copies], op, 1e-5, g if op else None, None, out=out), 12)
    alg = 2 * rows * cols * 2 + (cols * 4 if op else 0)
    gbs = alg / us / 1e3
    return {"case": {0: "softmax_bf16", 2: "rmsnorm_bf16", 1: "layernorm_bf16"}[op], "shape": [rows, cols], "us": us, "achieved": gbs,
            "unit": "GB/s", "bound": "hbm", "peak": hbm, "frac": gbs / hbm, "algorithmic_bytes": alg, "peak_source": "of " + src}


def build_paged_attn_case(seed=0, torch_seed=None):
    """The paged GQA decode-attention case of the micro-suite: batch 64, context lengths uniform in [128, 4096], 32 query
    heads over 8 KV heads of dim 128, bf16 K/V ~N(0,1) in 16-token pages handed out as a seeded random permutation of
    a shared 65 536-page pool.  Returns a dict of the device tensors and the host copies of table and contexts."""
    rng = np.random.default_rng(seed)
    B, H, HKV, D, page, pool = 64, 32, 8, 128, 16, 65536
    ctx = rng.integers(128, 4097, B).astype(np.int32)
    mbps = 256
    perm = rng.permutation(pool).astype(np.uint32)
    table = np.zeros((B, mbps), np.uint32)
    nxt = 0
    for b in range(B):
        n = (int(ctx[b]) + page - 1) // page
        table[b, :n] = perm[nxt:nxt + n]
        nxt += n
    gen = None
    if torch_seed is not None:
        gen = torch.Generator(device="cuda")
        gen.manual_seed(torch_seed)
    kv = dev.PagedKV(1, pool, HKV, D, page)
    kv.k.normal_(generator=gen)
    kv.v.normal_(generator=gen)
    q = torch.randn(B, H * D, device="cuda", generator=gen)
    return dict(B=B, H=H, HKV=HKV, D=D, page=page, pool=pool, mbps=mbps, max_ctx=4096, ctx=ctx, table=table, kv=kv, q=q,
                bt=torch.from_numpy(table.view(np.int32)).cuda(), row_slot=torch.arange(B, dtype=torch.int32, device="cuda"),
                row_ctx=torch.from_numpy(ctx).cuda(), scale=1.0 / math.sqrt(D), pages_used=nxt)


def case_paged_attn(hbm, tf, src):
    c = build_paged_attn_case()
    B, H, HKV, D, mbps, ctx, kv, q, bt, row_slot, row_ctx = (c[k] for k in ("B", "H", "HKV", "D", "mbps", "ctx", "kv", "q", "bt", "row_slot", "row_ctx"))
    out = torch.empty(B, H * D, dtype=torch.bfloat16, device="cuda")
    scratch = dev.paged_attn_scratch(B, H, D, 4096)
    fn = lambda i: dev.paged_attn_decode(q, H * D, kv, 0, bt, row_slot, row_ctx, out, B, H, mbps, 4096, c["scale"], scratch)
    us = time_graph(fn, 10)
    alg = float(ctx.sum()) * 2 * HKV * D * 2 + B * H * D * (4 + 2) + B * mbps * 4
    gbs = alg / us / 1e3
    return {"case": "paged_attn_decode", "shape": {"batch": B, "q_heads": H, "kv_heads": HKV, "d": D, "ctx": "U[128,4096]"}, "us": us,
            "achieved": gbs, "unit": "GB/s", "bound": "hbm", "peak": hbm, "frac": gbs / hbm, "algorithmic_bytes": alg,
            "note": "555 MB of KV per launch exceeds L2", "peak_source": "of " + src}


def build_paged_attn_int8_case(seed=0, torch_seed=None, pool=65536):
    """The paged_attn_decode case over the int8 cache: the same batch, heads and context draw as the bf16 case, int8 values
    uniform in [-127, 127] with f32 scales uniform in [0.005, 0.03] per (token, KV head), pages a seeded permutation of a
    `pool`-page pool.  Returns a dict of the device tensors and the host copies of table and contexts."""
    rng = np.random.default_rng(seed)
    B, H, HKV, D, page = 64, 32, 8, 128, 16
    ctx = rng.integers(128, 4097, B).astype(np.int32)
    mbps = 256
    perm = rng.permutation(pool).astype(np.uint32)
    table = np.zeros((B, mbps), np.uint32)
    nxt = 0
    for b in range(B):
        n = (int(ctx[b]) + page - 1) // page
        table[b, :n] = perm[nxt:nxt + n]
        nxt += n
    if torch_seed is not None:
        torch.manual_seed(torch_seed)
    kv = dev.PagedKVInt8(1, pool, HKV, D, page)
    kv.k.copy_(torch.randint(-127, 128, kv.k.shape, dtype=torch.int8, device="cuda"))
    kv.v.copy_(torch.randint(-127, 128, kv.v.shape, dtype=torch.int8, device="cuda"))
    kv.k_scale.uniform_(0.005, 0.03)
    kv.v_scale.uniform_(0.005, 0.03)
    q = torch.randn(B, H * D, device="cuda")
    return {"B": B, "H": H, "HKV": HKV, "D": D, "page": page, "pool": pool, "mbps": mbps, "ctx": ctx, "table": table, "kv": kv, "q": q,
            "bt": torch.from_numpy(table.view(np.int32)).cuda(), "row_slot": torch.arange(B, dtype=torch.int32, device="cuda"),
            "row_ctx": torch.from_numpy(ctx).cuda(), "max_ctx": 4096, "scale": 1.0 / math.sqrt(D), "pages_used": nxt}


def case_paged_attn_int8(hbm, tf, src):
    """The paged_attn_decode case over the int8 cache (same batch, heads and context draw)."""
    c = build_paged_attn_int8_case()
    B, H, HKV, D, mbps, kv, q, bt, row_slot, row_ctx, ctx = (c[k] for k in ("B", "H", "HKV", "D", "mbps", "kv", "q", "bt", "row_slot", "row_ctx", "ctx"))
    out = torch.empty(B, H * D, dtype=torch.bfloat16, device="cuda")
    scratch = dev.paged_attn_scratch(B, H, D, 4096)
    fn = lambda i: dev.paged_attn_decode_int8(q, H * D, kv, 0, bt, row_slot, row_ctx, out, B, H, mbps, 4096, 1.0 / math.sqrt(D), scratch)
    us = time_graph(fn, 10)
    alg = float(ctx.sum()) * 2 * HKV * (D + 4) + B * H * D * (4 + 2) + B * mbps * 4
    gbs = alg / us / 1e3
    return {"case": "paged_attn_decode_int8", "shape": {"batch": B, "q_heads": H, "kv_heads": HKV, "d": D, "ctx": "U[128,4096]"}, "us": us,
            "achieved": gbs, "unit": "GB/s", "bound": "hbm", "peak": hbm, "frac": gbs / hbm, "algorithmic_bytes": alg,
            "note": "int8 values + f32 scale per (token, kv head): 286 MB per launch, above L2", "peak_source": "of " + src}


def case_paged_prefill(H, HKV, D, seqs, hist, chunk, hbm, tf, src):
    """Prompt chunks of `chunk` tokens on top of `hist` cached tokens, `seqs` sequences: the tiled kernel, with the
    row-per-token kernel it replaces timed beside it.  Rated against the tensor peak (useful flops: QK^T and PV over
    the causal triangle, 4 * head_dim per (query, visible key, head)) and by the key bytes it streams."""
    rng = np.random.default_rng(0)
    page = 16
    total = hist + chunk
    mbps = (total + page - 1) // page
    pool = seqs * mbps
    table = rng.permutation(pool).astype(np.uint32).reshape(seqs, mbps)
    kv = dev.PagedKV(1, pool, HKV, D, page)
    kv.k.normal_()
    kv.v.normal_()
    rows = seqs * chunk
    q = torch.randn(rows, H * D, device="cuda")
    bt = torch.from_numpy(table.view(np.int32)).cuda()
    rs = np.repeat(np.arange(seqs, dtype=np.int32), chunk)
    rc = np.tile(np.arange(hist + 1, total + 1, dtype=np.int32), seqs)
    tile_rows = int(lib().wkb_paged_attn_prefill_tile_rows(H, HKV))
    tiles = dev.prefill_tiles(rs, tile_rows)
    row_slot, row_ctx, d_tiles = torch.from_numpy(rs).cuda(), torch.from_numpy(rc).cuda(), torch.from_numpy(tiles).cuda()
    out = torch.empty(rows, H * D, dtype=torch.bfloat16, device="cuda")
    scale = 1.0 / math.sqrt(D)
    us = time_graph(lambda i: dev.paged_attn_prefill(q, H * D, kv, 0, bt, row_slot, row_ctx, d_tiles, out, H, mbps, scale), 10)
    scratch = dev.paged_attn_scratch(rows, H, D, total)
    us_rows = time_graph(lambda i: dev.paged_attn_decode(q, H * D, kv, 0, bt, row_slot, row_ctx, out, rows, H, mbps, total, scale, scratch), 5)
    pairs = float(rc.sum())                                   # (query, visible key) pairs per head
    flops = pairs * H * 4 * D
    key_bytes = float(sum(int(rc[r0:r0 + n].max()) for r0, n in tiles)) * HKV * 2 * D * 2
    return {"case": "paged_attn_prefill", "shape": {"q_heads": H, "kv_heads": HKV, "d": D, "sequences": seqs, "cached": hist, "chunk": chunk},
            "us": us, "achieved": flops / us / 1e6, "unit": "TFLOP/s", "bound": "tensor", "peak": tf, "frac": flops / us / 1e6 / tf,
            "useful_flops": flops, "key_bytes_streamed": key_bytes, "key_stream_gbs": key_bytes / us / 1e3, "prompt_tok_per_s": rows / us * 1e6,
            "row_per_token_us": us_rows, "speedup_vs_row_per_token": us_rows / us,
            "note": "tcgen05 (S = Q.K^T with q as bf16 hi + lo, P.V with P in tensor memory): 1.5x the useful flops are issued, "
                    "plus the masked part of the diagonal blocks", "peak_source": "of " + src}


def run(out=sys.stdout, only=None, reps_scale=1.0):
    """Run the suite (or the cases whose name contains `only`) and print one JSON line per case."""
    require_gpu()
    hbm, tf, src = peaks()
    plan = []
    for size in (1024, 4096, 8192):
        plan.append(("gemm_bf16", lambda size=size: case_gemm(size, hbm, tf, src)))
    for (n, k) in ((4096, 4096), (11008, 4096)):
        for variant in ("contract", "bf16x"):
            plan.append(("gemv_q4_0_" + variant, lambda n=n, k=k, variant=variant: case_gemv_q4(n, k, variant, hbm, tf, src)))
    for (n, k, mode) in ((6144, 4096, 0), (22016, 4096, 2), (4096, 11008, 0)):
        plan.append(("gemm_q4_0_bf16", lambda n=n, k=k, mode=mode: case_gemm_q4(64, n, k, mode, hbm, tf, src)))
    for op, name in ((2, "rmsnorm_bf16"), (0, "softmax_bf16"), (1, "layernorm_bf16")):
        plan.append((name, lambda op=op: case_norm(op, hbm, tf, src)))
    plan.append(("paged_attn_decode", lambda: case_paged_attn(hbm, tf, src)))
    plan.append(("paged_attn_decode_int8", lambda: case_paged_attn_int8(hbm, tf, src)))
    for (H, HKV, D, seqs, hist, chunk) in ((12, 12, 64, 64, 0, 512), (32, 8, 128, 16, 0, 512), (32, 8, 128, 16, 2048, 256)):
        plan.append(("paged_attn_prefill", lambda a=(H, HKV, D, seqs, hist, chunk): case_paged_prefill(*a, hbm, tf, src)))
    plan.append(("decode_gemms", lambda: case_decode_gemms(hbm, tf, src)))
    results = []
    for name, fn in plan:
        if only and only not in name:
            continue
        r = fn()
        results.append(r)
        print(json.dumps(r), file=out, flush=True)
    if dev.gemm_status() != 0:
        raise RuntimeError("tensor-core GEMM reported an expired pipeline wait")
    return results


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default=None, help="run only the cases whose name contains this string")
    run(only=ap.parse_args().case)

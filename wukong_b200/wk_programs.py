"""Dispatch-trace driver: replays the builtin-call sequence that a `.wk` program lowers to.

The compiler that turns `.wk` source into these calls is Rust and cannot be built here, so a program
is represented by its trace: the same builtins, in the same order, with the same operands, as
`crates/wukong_mir_build/src/builtins.rs:245-433` / `decode_builtins.rs:117-230` emit for it.  The
scalar statements between the builtin calls (embedding sums, residual adds, the GELU loop, the
arg-max loop) are the language's own f32 arithmetic, one IEEE operation per source operator, and are
executed here with numpy float32 in the source's operator order.

`rt` is any namespace with the builtin names of `wukong_b200.runtime` (the GPU library through the
reference C ABI); the tests pass an oracle-backed namespace with the same names to obtain the
reference result of the identical trace.
"""
import numpy as np

F = np.float32


class GPT2Flat:
    """Weights in the order `examples/gpt2_generate.wk` slices them out of its flat blob: per layer
    ln1 g/b, Wq/bq, Wk/bk, Wv/bv, Wo/bo, ln2 g/b, W1/b1, W2/b2 (all `[out, in]` f32); wte, wpe, lnf."""

    def __init__(self, n_layer, d, n_head, d_ff, vocab, n_pos, seed=0):
        rng = np.random.default_rng(seed)
        n = lambda *s: (rng.standard_normal(s, dtype=np.float32) * F(0.02))
        self.n_layer, self.d, self.n_head, self.d_ff, self.vocab, self.n_pos = n_layer, d, n_head, d_ff, vocab, n_pos
        self.wte, self.wpe = n(vocab, d), n(n_pos, d)
        self.lnf_g, self.lnf_b = np.ones(d, F), np.zeros(d, F)
        self.layers = []
        for _ in range(n_layer):
            self.layers.append(dict(ln1_g=np.ones(d, F), ln1_b=np.zeros(d, F), wq=n(d, d), bq=n(d), wk=n(d, d), bk=n(d),
                                    wv=n(d, d), bv=n(d), wo=n(d, d), bo=n(d), ln2_g=np.ones(d, F), ln2_b=np.zeros(d, F),
                                    w1=n(d_ff, d), b1=n(d_ff), w2=n(d, d_ff), b2=n(d)))


def scalar_gelu_loop(ff, rt):
    """`u = 0.7978845608*(ff + 0.044715*ff*ff*ff); th = 1 - 2/(exp(2u)+1); ff = 0.5*ff*(1+th)`:
    the scalar loop of gpt2_generate.wk:214-218, one rounding per operator, `exp` = the runtime's."""
    t = (F(0.044715) * ff) * ff * ff
    u = F(0.7978845608) * (ff + t)
    e = np.empty_like(u)
    rt.exp(np.ascontiguousarray(F(2.0) * u), e)
    th = F(1.0) - F(2.0) / (e + F(1.0))
    return ((F(0.5) * ff) * (F(1.0) + th)).astype(F)


def gpt2_generate(rt, w, prompt0, prompt1, nsteps, join1=2, maxt=None, collect_logits=False):
    """The trace of examples/gpt2_generate.wk:111-275: two sequences in one padded batch, the second
    joining at step `join1`; per step and layer `layernorm`, 3x `linear`, 2-4x `kv_append`,
    `sdpa_kv_batch::<2,1,MAXT,H,H,hd>`, `linear`, residual, `layernorm`, `linear`, GELU loop, `linear`,
    residual; then `layernorm`, `matmul_nt` against wte and a strict `>` arg-max.
    Returns (tokens of sequence 0, tokens of sequence 1[, logits per step])."""
    d, H, dff, V, L = w.d, w.n_head, w.d_ff, w.vocab, w.n_layer
    hd = d // H
    maxt = maxt or nsteps
    toks0 = list(prompt0) + [0] * (nsteps + 1)
    toks1 = list(prompt1) + [0] * (nsteps + 1)
    cache = 2 * maxt * d
    kc = [np.zeros(cache, F) for _ in range(L)]
    vc = [np.zeros(cache, F) for _ in range(L)]
    x, nrm, q, krow, vrow, att, a = (np.zeros((2, d), F) for _ in range(7))
    ff = np.zeros((2, dff), F)
    logits = np.zeros((2, V), F)
    lens, pos = np.zeros(2, np.int32), np.zeros(2, np.int32)
    scale = float(F(1.0) / np.sqrt(F(hd)))
    trace = []
    for t in range(nsteps):
        p0, p1 = t, t - join1
        live1 = p1 >= 0
        lens[0], pos[0] = p0 + 1, p0
        if live1:
            lens[1], pos[1] = p1 + 1, p1
        x[0] = w.wte[toks0[p0]] + w.wpe[p0]
        x[1] = 0.0
        if live1:
            x[1] = w.wte[toks1[p1]] + w.wpe[p1]
        for l, lw in enumerate(w.layers):
            rt.layernorm(x, lw["ln1_g"], lw["ln1_b"], nrm, 2, d, 1e-5)
            rt.linear(nrm, lw["wq"], lw["bq"], q, 2, d, d)
            rt.linear(nrm, lw["wk"], lw["bk"], krow, 2, d, d)
            rt.linear(nrm, lw["wv"], lw["bv"], vrow, 2, d, d)
            rt.kv_append(kc[l], krow[0], p0, d)
            rt.kv_append(vc[l], vrow[0], p0, d)
            if live1:
                rt.kv_append(kc[l], krow[1], maxt + p1, d)
                rt.kv_append(vc[l], vrow[1], maxt + p1, d)
            rt.sdpa_kv_batch(q, kc[l], vc[l], att, lens, pos, scale, True, 2, 1, maxt, H, H, hd)
            rt.linear(att, lw["wo"], lw["bo"], a, 2, d, d)
            a[:] = x + a
            rt.layernorm(a, lw["ln2_g"], lw["ln2_b"], nrm, 2, d, 1e-5)
            rt.linear(nrm, lw["w1"], lw["b1"], ff, 2, d, dff)
            ff[:] = scalar_gelu_loop(ff, rt)
            rt.linear(ff, lw["w2"], lw["b2"], x, 2, dff, d)
            x[:] = a + x
        rt.layernorm(x, w.lnf_g, w.lnf_b, nrm, 2, d, 1e-5)
        rt.matmul_nt(nrm, w.wte, logits, 2, d, V)
        if collect_logits:
            trace.append(logits.copy())
        if p0 + 1 >= len(prompt0):
            toks0[p0 + 1] = _strict_argmax(logits[0])
        if live1 and p1 + 1 >= len(prompt1):
            toks1[p1 + 1] = _strict_argmax(logits[1])
    out = (toks0[len(prompt0):nsteps + 1], toks1[len(prompt1):max(len(prompt1), nsteps - join1 + 1)])
    return out + (trace,) if collect_logits else out


def _strict_argmax(row):
    """`best = row[0]; for v: if row[v] > best {best = row[v]; bi = v}` (gpt2_generate.wk:250-255)."""
    best, bi = row[0], 0
    # vectorised form of the strict scan: the first index holding the maximum (NaNs never win unless at 0)
    if np.isnan(best):
        return 0
    m = np.nanmax(row)
    return int(np.flatnonzero(row == m)[0]) if m > best else bi


def llama_block_inputs():
    """The deterministic operands of examples/llama_block.wk:183-204."""
    i512, i4096, i16384, i64_ = (np.arange(n) for n in (512, 4096, 16384, 64))
    f = lambda v: v.astype(F)
    x = f(i512 % 13) * F(0.02) - F(0.12)
    wq = f(i4096 % 7) * F(0.01) - F(0.03)
    wk = f(i4096 % 11) * F(0.008) - F(0.04)
    wv = f(i4096 % 5) * F(0.012) - F(0.024)
    wo = f(i4096 % 9) * F(0.009) - F(0.036)
    wg = f(i16384 % 17) * F(0.004) - F(0.032)
    wu = f(i16384 % 19) * F(0.003) - F(0.027)
    wd = f(i16384 % 23) * F(0.0025) - F(0.0275)
    rg1 = F(1.0) + f(i64_ % 3) * F(0.1)
    rg2 = F(1.0) - f(i64_ % 4) * F(0.05)
    return dict(x=x.astype(F), rg1=rg1.astype(F), wq=wq.astype(F), wk=wk.astype(F), wv=wv.astype(F), wo=wo.astype(F),
                rg2=rg2.astype(F), wg=wg.astype(F), wu=wu.astype(F), wd=wd.astype(F))


def llama_block(rt, x, rg1, wq, wk, wv, wo, rg2, wg, wu, wd):
    """The trace of examples/llama_block.wk:35-181 (S = 8, D = 64, 4 heads of 16, Dff = 256): two affine
    RMSNorms, seven `sgemm_nt`, one `vmath(silu)` and one Hadamard `velem` are dispatched; the
    interleaved-pair RoPE and the per-head causal softmax attention are plain loops in the source and run
    here as float32 numpy in the same operator order."""
    S, D, H, hd, Dff = 8, 64, 4, 16, 256
    nrm = np.zeros((S, D), F)
    rt.rmsnorm(x.reshape(S, D).copy(), rg1, nrm, S, D, 1e-5)
    q, k, v = (np.zeros((S, D), F) for _ in range(3))
    rt.matmul_nt(nrm, wq, q, S, D, D)
    rt.matmul_nt(nrm, wk, k, S, D, D)
    rt.matmul_nt(nrm, wv, v, S, D, D)
    # RoPE, interleaved pairs (2p, 2p+1): freq = 10000^(-2p/hd), theta = pos * freq
    p = np.arange(hd // 2)
    freq = np.power(F(10000.0), -(2 * p).astype(F) / F(16.0)).astype(F)
    theta = (np.arange(S, dtype=F)[:, None] * freq[None, :]).astype(F)
    c, sn = np.cos(theta).astype(F), np.sin(theta).astype(F)
    for t in (q, k):
        tv = t.reshape(S, H, hd // 2, 2)
        t0, t1 = tv[..., 0].copy(), tv[..., 1].copy()
        tv[..., 0] = t0 * c[:, None, :] - t1 * sn[:, None, :]
        tv[..., 1] = t0 * sn[:, None, :] + t1 * c[:, None, :]
    attn = np.zeros((S, D), F)
    for hh in range(H):
        sl = slice(hh * hd, (hh + 1) * hd)
        sc = ((q[:, sl] @ k[:, sl].T) * F(0.25)).astype(F)
        sc[np.triu_indices(S, 1)] = F(-1.0e30)
        e = np.exp(sc - sc.max(1, keepdims=True)).astype(F)
        attn[:, sl] = ((e * (F(1.0) / e.sum(1, keepdims=True))) @ v[:, sl]).astype(F)
    a = np.zeros((S, D), F)
    rt.matmul_nt(attn, wo, a, S, D, D)
    a[:] = x.reshape(S, D) + a
    rt.rmsnorm(a.copy(), rg2, nrm, S, D, 1e-5)
    gate, up, h = (np.zeros((S, Dff), F) for _ in range(3))
    rt.matmul_nt(nrm, wg, gate, S, D, Dff)
    rt.matmul_nt(nrm, wu, up, S, D, Dff)
    rt.silu(gate, gate)
    rt.hadamard(gate, up, h)
    out = np.zeros((S, D), F)
    rt.matmul_nt(h, wd, out, S, Dff, D)
    out[:] = a + out
    return out.reshape(-1)

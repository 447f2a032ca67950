"""CPU model of the Llama-shape int4 decode block stack (test infrastructure).

Recipe (the W4A16 one: Q4_0 weights, bf16 activations): every linear is y = x . W^T with W the *exact*
dequantisation d * (nib - 8) of its Q4_0 blocks (crates/wukong_runtime/src/quant.rs:13-16; the exact
dequant is also the gate the reference holds its own W4A16 GPU kernels to, crates/wukong_codegen_gpu/
src/ptx_int4.rs:11-14), x rounded to bf16, accumulation in float64 and one rounding to fp32.
RMSNorm (norm.rs:50-54, op 2, affine) and the SwiGLU product are rounded once to bf16, K / V are cached
as bf16, RoPE is the half-split pairing of rope.rs:54-71 at the row's own position, attention is GQA
over the visible keys, the residual stream and the logits are fp32, and the token is the arg-max with
the lowest index winning ties.

Tensor parallelism (`world` > 1) follows the split the reference validates in
crates/wukong_codegen_gpu/src/serving.rs:4161-4240: QKV / gate / up / LM head by output rows (heads,
FFN columns, vocabulary), O / down by input columns, one sum over ranks after attention and one after
the MLP; `attn_partial` / `mlp_partial` return what one rank contributes so a test can do the sum itself.

`operand="bf16"` evaluates the same model with every weight rounded the way a bf16 x bf16 tensor-core path
holds it; comparing a GPU run with that variant isolates kernel faults from the operand rounding, whose size
the comparison with the exact variant then bounds."""
import math

import numpy as np


def dequant_rows(orc, raw, n, k, operand="exact"):
    """f32 weights of raw Q4_0 rows.  operand "exact": d * (nib - 8), exact in f32.  operand "bf16": that value as a
    bf16 tensor-core operand holding it, bf16(bf16(d) * (nib - 8)) -- what a bf16 x bf16 MMA path multiplies."""
    q, s = orc.unpack_q4_0(np.ascontiguousarray(raw).reshape(-1))
    d = s.view(np.float16).astype(np.float32).reshape(n, k // 32, 1)
    q = q.astype(np.float32).reshape(n, k // 32, 32)
    if operand == "bf16":
        rnd = lambda a: orc.from_bf16_bits(orc.to_bf16_bits(np.ascontiguousarray(a, np.float32).ravel())).reshape(a.shape)
        return rnd(rnd(d) * q).reshape(n, k)
    return (d * q).reshape(n, k)


class OracleLlama:
    def __init__(self, cfg, weights, orc, operand="exact"):
        """weights: dict with f32 `embed` [V, d], `norm_f` [d], raw Q4_0 `lm_head` [V, d/32, 18] and per layer
        `norm1`, `norm2` (f32 [d]) and raw Q4_0 `wq`, `wk`, `wv`, `wo`, `wgate`, `wup`, `wdown`."""
        self.cfg, self.orc = cfg, orc
        d, hd, F = cfg.d_model, cfg.head_dim, cfg.d_ff
        dq = lambda raw, n, k: dequant_rows(orc, raw, n, k, operand).astype(np.float64)
        self.embed, self.norm_f = weights["embed"], weights["norm_f"]
        self.lm_head = dq(weights["lm_head"], cfg.vocab, d)
        self.layers = []
        for lw in weights["layers"]:
            self.layers.append(dict(norm1=lw["norm1"], norm2=lw["norm2"], wq=dq(lw["wq"], cfg.n_head * hd, d),
                                    wk=dq(lw["wk"], cfg.n_kv_head * hd, d), wv=dq(lw["wv"], cfg.n_kv_head * hd, d),
                                    wo=dq(lw["wo"], d, cfg.n_head * hd), wgate=dq(lw["wgate"], F, d), wup=dq(lw["wup"], F, d),
                                    wdown=dq(lw["wdown"], d, F)))
        half = hd // 2
        self.inv_freq = (1.0 / (np.float32(cfg.rope_base) ** (np.arange(half, dtype=np.float32) * np.float32(2.0 / hd)))).astype(np.float32)

    def _bf(self, x):
        return self.orc.from_bf16_bits(self.orc.to_bf16_bits(np.ascontiguousarray(x, np.float32))).reshape(np.shape(x))

    def _rms(self, x, gamma):
        return self._bf(self.orc.norm_affine(x, gamma, np.zeros_like(gamma), 2, self.cfg.eps))

    @staticmethod
    def _lin(x, w):
        return (x.astype(np.float64) @ w.T).astype(np.float32)

    def attn_partial(self, li, x, poss, kcs, vcs, rank=0, world=1):
        """Rank's contribution to the attention sub-block output (before the residual add); appends this
        rank's KV heads at poss.  kcs[s][li] / vcs[s][li]: float32 [capacity, n_kv_head * hd] holding bf16 values."""
        cfg, lw, orc = self.cfg, self.layers[li], self.orc
        hd, S = cfg.head_dim, x.shape[0]
        hq, hkv = cfg.n_head // world, cfg.n_kv_head // world
        q0, k0 = rank * hq * hd, rank * hkv * hd
        xn = self._rms(x, lw["norm1"])
        q = self._lin(xn, lw["wq"][q0:q0 + hq * hd])
        k = self._lin(xn, lw["wk"][k0:k0 + hkv * hd])
        v = self._lin(xn, lw["wv"][k0:k0 + hkv * hd])
        pos = np.asarray(poss, np.int32)
        q = orc.rope_pos(q, self.inv_freq, pos, hq)
        k = orc.rope_pos(k, self.inv_freq, pos, hkv)
        att = np.zeros((S, hq * hd), np.float32)
        scale = 1.0 / math.sqrt(hd)
        for s in range(S):
            p = int(poss[s])
            kcs[s][li][p, k0:k0 + hkv * hd] = self._bf(k[s])
            vcs[s][li][p, k0:k0 + hkv * hd] = self._bf(v[s])
            n = p + 1
            K = kcs[s][li][:n, k0:k0 + hkv * hd].reshape(n, hkv, hd).astype(np.float64)
            V = vcs[s][li][:n, k0:k0 + hkv * hd].reshape(n, hkv, hd).astype(np.float64)
            qs = q[s].reshape(hq, hd).astype(np.float64)
            for h in range(hq):
                g = h // (hq // hkv)
                sc = (K[:, g, :] @ qs[h]) * scale
                e = np.exp(sc - sc.max())
                att[s, h * hd:(h + 1) * hd] = (e / e.sum()) @ V[:, g, :]
        a = self._bf(att)
        return self._lin(a, lw["wo"][:, q0:q0 + hq * hd])

    def mlp_partial(self, li, x, rank=0, world=1):
        cfg, lw = self.cfg, self.layers[li]
        f = cfg.d_ff // world
        f0 = rank * f
        xn = self._rms(x, lw["norm2"])
        g = self._lin(xn, lw["wgate"][f0:f0 + f]).astype(np.float64)
        u = self._lin(xn, lw["wup"][f0:f0 + f]).astype(np.float64)
        h = self._bf((g / (1.0 + np.exp(-g)) * u).astype(np.float32))
        return self._lin(h, lw["wdown"][:, f0:f0 + f])

    def step(self, toks, poss, kcs, vcs, world=1, reduce=None):
        """One decode step for S rows.  `reduce(list_of_partials)` sums the per-rank contributions (default:
        in rank order in fp32).  Returns (tokens, logits)."""
        cfg = self.cfg
        reduce = reduce or (lambda parts: np.sum(np.stack(parts), axis=0, dtype=np.float32) if len(parts) > 1 else parts[0])
        x = self.embed[np.asarray(toks)].astype(np.float32)
        for li in range(cfg.n_layer):
            x = (x + reduce([self.attn_partial(li, x, poss, kcs, vcs, r, world) for r in range(world)])).astype(np.float32)
            x = (x + reduce([self.mlp_partial(li, x, r, world) for r in range(world)])).astype(np.float32)
        xn = self._rms(x, self.norm_f)
        logits = self._lin(xn, self.lm_head)
        return self.orc.rowargmax(logits), logits

    def new_cache(self, capacity):
        z = lambda: [np.zeros((capacity, self.cfg.n_kv_head * self.cfg.head_dim), np.float32) for _ in range(self.cfg.n_layer)]
        return z(), z()

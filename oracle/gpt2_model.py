"""CPU model of the GPT-2-shape decode path in the library's precision recipe, built only from the
oracle's kernels (test infrastructure; also the timed CPU baseline of the benchmark).

Recipe: weights and KV cache bf16, residual stream fp32, every GEMM bf16 x bf16 with fp32
accumulation in the reference's order contract, norm / attention / MLP-hidden outputs rounded once
to bf16, logits fp32, greedy arg-max with the lowest index winning ties.  The layer sequence is the
one the reference's examples/gpt2_generate.wk:137-255 lowers to (norm_affine, sgemm_nt_epi x4-6,
kv_append, attention over the cache, GELU, residual adds, tied LM head, strict arg-max)."""
import math

import numpy as np


class OracleGPT2:
    def __init__(self, cfg, weights, orc):
        self.cfg, self.w, self.orc = cfg, weights, orc

    def _round(self, x):
        return self.orc.to_bf16_bits(np.ascontiguousarray(x, np.float32))

    def step(self, toks, poss, kcs, vcs, want_logits=True):
        """One decode step for S sequences: row s has token toks[s] at position poss[s]; kcs[s][layer]
        / vcs[s][layer] are [capacity, d_model] bf16-bit caches holding positions < poss[s].  Appends
        the new K/V rows and returns (next tokens, logits)."""
        cfg, w, orc = self.cfg, self.w, self.orc
        d, H, hd, S = cfg.d_model, cfg.n_head, cfg.head_dim, len(toks)
        x = np.stack([orc.from_bf16_bits(w["wte"][t]) + orc.from_bf16_bits(w["wpe"][p]) for t, p in zip(toks, poss)]).astype(np.float32)
        for li, lw in enumerate(w["layers"]):
            h = self._round(orc.norm_affine(x, lw["ln1_g"], lw["ln1_b"], 1, cfg.eps))
            qkv = orc.sgemm_half_nt(h, lw["w_qkv"], S, d, 3 * d, bias=lw["b_qkv"], act=0)
            att = np.empty((S, d), np.float32)
            for s in range(S):
                pos = poss[s]
                kcs[s][li][pos] = self._round(qkv[s, d:2 * d])
                vcs[s][li][pos] = self._round(qkv[s, 2 * d:])
                n = pos + 1
                npg = (n + 15) // 16
                # a contiguous cache is consecutive pages of the slab order [page, token, head, dim]
                att[s] = orc.paged_attn_decode(qkv[s:s + 1, :d], kcs[s][li], vcs[s][li], 1,
                                               np.arange(npg, dtype=np.uint32).reshape(1, npg), [n], 1, H, H, hd, 16, npg,
                                               1.0 / math.sqrt(hd), layout=0)
            a = self._round(att)
            x = (orc.sgemm_half_nt(a, lw["w_o"], S, d, d, bias=lw["b_o"], act=0) + x).astype(np.float32)
            h2 = self._round(orc.norm_affine(x, lw["ln2_g"], lw["ln2_b"], 1, cfg.eps))
            ff = self._round(orc.sgemm_half_nt(h2, lw["w_fc"], S, d, cfg.d_ff, bias=lw["b_fc"], act=2))
            x = (orc.sgemm_half_nt(ff, lw["w_proj"], S, cfg.d_ff, d, bias=lw["b_proj"], act=0) + x).astype(np.float32)
        if not want_logits:
            return None, None
        hf = self._round(orc.norm_affine(x, w["lnf_g"], w["lnf_b"], 1, cfg.eps))
        logits = orc.sgemm_half_nt(hf, w["wte"], S, d, cfg.vocab)
        return orc.rowargmax(logits), logits

    def step_dense_cache(self, toks, poss, K, V, want_logits=True):
        """The same decode step over dense fp32 caches, the way the reference's CPU path keeps them: K[layer] / V[layer] are
        [S, capacity, d_model] fp32 arrays holding the (bf16-rounded) rows of positions < poss[s]; attention is ONE call
        per layer to the reference's batched KV-cache kernel (wko_attention_kv_batch_f32: attention_kv.rs entries
        :1157-1250) instead of one f64 model evaluation per sequence.  This is the form the timed CPU baseline runs."""
        cfg, w, orc = self.cfg, self.w, self.orc
        d, H, hd, S = cfg.d_model, cfg.n_head, cfg.head_dim, len(toks)
        pos = np.asarray(poss, np.int64)
        rows = np.arange(S)
        cap = K[0].shape[1]
        x = (orc.from_bf16_bits(w["wte"][np.asarray(toks)]) + orc.from_bf16_bits(w["wpe"][pos])).astype(np.float32)
        for li, lw in enumerate(w["layers"]):
            h = self._round(orc.norm_affine(x, lw["ln1_g"], lw["ln1_b"], 1, cfg.eps))
            qkv = orc.sgemm_half_nt(h, lw["w_qkv"], S, d, 3 * d, bias=lw["b_qkv"], act=0)
            K[li][rows, pos] = orc.from_bf16_bits(self._round(qkv[:, d:2 * d]))
            V[li][rows, pos] = orc.from_bf16_bits(self._round(qkv[:, 2 * d:]))
            st, att = orc.attention_kv_batch(np.ascontiguousarray(qkv[:, :d]), K[li], V[li], pos + 1, pos, S, 1, cap, H, H, hd,
                                             1.0 / math.sqrt(hd), True)
            if st != 0:
                raise RuntimeError("attention_kv_batch refused its plan: %d" % st)
            a = self._round(att.reshape(S, d))
            x = (orc.sgemm_half_nt(a, lw["w_o"], S, d, d, bias=lw["b_o"], act=0) + x).astype(np.float32)
            h2 = self._round(orc.norm_affine(x, lw["ln2_g"], lw["ln2_b"], 1, cfg.eps))
            ff = self._round(orc.sgemm_half_nt(h2, lw["w_fc"], S, d, cfg.d_ff, bias=lw["b_fc"], act=2))
            x = (orc.sgemm_half_nt(ff, lw["w_proj"], S, cfg.d_ff, d, bias=lw["b_proj"], act=0) + x).astype(np.float32)
        if not want_logits:
            return None, None
        hf = self._round(orc.norm_affine(x, w["lnf_g"], w["lnf_b"], 1, cfg.eps))
        logits = orc.sgemm_half_nt(hf, w["wte"], S, d, cfg.vocab)
        return orc.rowargmax(logits), logits

    def new_cache(self, capacity):
        cap = (capacity + 15) // 16 * 16
        z = lambda: [np.zeros((cap, self.cfg.d_model), np.uint16) for _ in range(self.cfg.n_layer)]
        return z(), z()

    def generate(self, prompt, gen_len, return_margins=False):
        total = len(prompt) + gen_len
        kc, vc = self.new_cache(total)
        toks, out, margins = list(prompt), [], []
        for pos in range(total - 1):
            sample = pos >= len(prompt) - 1
            nxt, logits = self.step([toks[pos]], [pos], [kc], [vc], want_logits=sample)
            if sample:
                srt = np.sort(logits[0])
                margins.append(float(srt[-1] - srt[-2]))
                out.append(int(nxt[0]))
                if len(toks) <= pos + 1:
                    toks.append(int(nxt[0]))
        return (out, margins) if return_margins else out

"""CPU model of the GPT-2-shape decode path in the library's precision recipe, built only from the
oracle's kernels (test infrastructure).  One sequence at a time, contiguous KV cache."""
import math

import numpy as np


class OracleGPT2:
    def __init__(self, cfg, weights, orc):
        self.cfg, self.w, self.orc = cfg, weights, orc

    def _round(self, x):
        return self.orc.to_bf16_bits(np.ascontiguousarray(x, np.float32))

    def generate(self, prompt, gen_len, return_margins=False):
        cfg, w, orc = self.cfg, self.w, self.orc
        d, H, hd = cfg.d_model, cfg.n_head, cfg.head_dim
        total = len(prompt) + gen_len
        kc = [np.zeros((total, d), np.uint16) for _ in range(cfg.n_layer)]
        vc = [np.zeros((total, d), np.uint16) for _ in range(cfg.n_layer)]
        toks, out, margins = list(prompt), [], []
        wte_f = None
        for pos in range(total - 1):
            tok = toks[pos]
            x = (orc.from_bf16_bits(w["wte"][tok]) + orc.from_bf16_bits(w["wpe"][pos])).astype(np.float32).reshape(1, d)
            for li, lw in enumerate(w["layers"]):
                h = self._round(orc.norm_affine(x, lw["ln1_g"], lw["ln1_b"], 1, cfg.eps))
                qkv = orc.sgemm_half_nt(h, lw["w_qkv"], 1, d, 3 * d, bias=lw["b_qkv"], act=0)[0]
                kc[li][pos] = self._round(qkv[d:2 * d])
                vc[li][pos] = self._round(qkv[2 * d:])
                n = pos + 1
                # contiguous cache == consecutive pages of the reference slab order [page, token, head, dim]
                npg = (n + 15) // 16
                kpad = np.zeros((npg * 16, d), np.uint16); kpad[:n] = kc[li][:n]
                vpad = np.zeros((npg * 16, d), np.uint16); vpad[:n] = vc[li][:n]
                att = orc.paged_attn_decode(qkv[:d].reshape(1, d), kpad, vpad, 1, np.arange(npg, dtype=np.uint32).reshape(1, npg),
                                            [n], 1, H, H, hd, 16, npg, 1.0 / math.sqrt(hd), layout=0)
                a = self._round(att)
                x = (orc.sgemm_half_nt(a, lw["w_o"], 1, d, d, bias=lw["b_o"], act=0) + x).astype(np.float32)
                h2 = self._round(orc.norm_affine(x, lw["ln2_g"], lw["ln2_b"], 1, cfg.eps))
                ff = self._round(orc.sgemm_half_nt(h2, lw["w_fc"], 1, d, cfg.d_ff, bias=lw["b_fc"], act=2))
                x = (orc.sgemm_half_nt(ff, lw["w_proj"], 1, cfg.d_ff, d, bias=lw["b_proj"], act=0) + x).astype(np.float32)
            if pos >= len(prompt) - 1:
                hf = self._round(orc.norm_affine(x, w["lnf_g"], w["lnf_b"], 1, cfg.eps))
                logits = orc.sgemm_half_nt(hf, w["wte"], 1, d, cfg.vocab)[0]
                t = int(orc.rowargmax(logits.reshape(1, -1))[0])
                srt = np.sort(logits)
                margins.append(float(srt[-1] - srt[-2]))
                out.append(t)
                if len(toks) <= pos + 1:
                    toks.append(t)
        return (out, margins) if return_margins else out

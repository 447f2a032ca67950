"""The CPU model's two decode-step forms agree: per-sequence f64 paged attention over bf16 caches (the checker the GPU
engine is compared with) and the batched fp32 KV-cache kernel over dense caches (the form the benchmark's CPU baseline
times).  Same tokens; logits equal to the difference between an f64 and an fp32 softmax."""
import numpy as np

from oracle import binding as orc
from oracle.gpt2_model import OracleGPT2
from wukong_b200.serving import GPT2Config, synth_weights


def test_dense_cache_step_matches_paged_step():
    cfg = GPT2Config(n_layer=2, d_model=256, n_head=4, d_ff=512, vocab=500, n_pos=128)
    w = synth_weights(cfg, 3)
    model = OracleGPT2(cfg, w, orc)
    rng = np.random.default_rng(0)
    S, cap = 5, 48
    ctx = [3, 17, 32, 1, 40]
    # caches holding `ctx` earlier positions of bf16-exact values
    kcs, vcs = [], []
    K = [np.zeros((S, cap, cfg.d_model), np.float32) for _ in range(cfg.n_layer)]
    V = [np.zeros((S, cap, cfg.d_model), np.float32) for _ in range(cfg.n_layer)]
    for s in range(S):
        kc, vc = model.new_cache(cap)
        for l in range(cfg.n_layer):
            kb = orc.to_bf16_bits(rng.standard_normal((ctx[s], cfg.d_model), dtype=np.float32))
            vb = orc.to_bf16_bits(rng.standard_normal((ctx[s], cfg.d_model), dtype=np.float32))
            kc[l][:ctx[s]] = kb
            vc[l][:ctx[s]] = vb
            K[l][s, :ctx[s]] = orc.from_bf16_bits(kb)
            V[l][s, :ctx[s]] = orc.from_bf16_bits(vb)
        kcs.append(kc)
        vcs.append(vc)
    toks = rng.integers(0, cfg.vocab, S).tolist()
    pos = list(ctx)
    for _ in range(3):
        ta, la = model.step(toks, pos, kcs, vcs)
        tb, lb = model.step_dense_cache(toks, pos, K, V)
        assert np.array_equal(ta, tb)
        assert np.allclose(la, lb, rtol=2e-2, atol=2e-2 * float(np.sqrt((la ** 2).mean())))
        # both forms appended the same bf16-rounded K / V rows
        for l in range(cfg.n_layer):
            for s in range(S):
                assert np.array_equal(orc.from_bf16_bits(kcs[s][l][pos[s]]), K[l][s, pos[s]])
        toks = [int(t) for t in ta]
        pos = [p + 1 for p in pos]

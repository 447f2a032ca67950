"""The dispatch trace of examples/gpt2_generate.wk through the reference C ABI on the GPU, against the
identical trace on the CPU oracle: fp32, every logit bit for bit, greedy tokens equal."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _both(orc, w, p0, p1, nsteps, join1):
    from wukong_b200 import _lib, runtime, wk_programs
    from oracle_rt import OracleRT
    _lib.require_gpu()
    got = wk_programs.gpt2_generate(runtime, w, p0, p1, nsteps, join1=join1, collect_logits=True)
    want = wk_programs.gpt2_generate(OracleRT(orc), w, p0, p1, nsteps, join1=join1, collect_logits=True)
    return got, want


def test_reduced_twin_full_run(orc):
    """The reference gates its oracle on a reduced twin of the model (examples/README.md:104-105):
    D = 64, 4 heads, 2 layers; here with the program's own constants (16 steps, joins at 2)."""
    from wukong_b200.wk_programs import GPT2Flat
    orc.set_threads(8)
    w = GPT2Flat(n_layer=2, d=64, n_head=4, d_ff=256, vocab=997, n_pos=32, seed=3)
    got, want = _both(orc, w, [11, 5, 900, 3, 42], [7, 7, 1], 16, 2)
    assert got[0] == want[0] and got[1] == want[1]
    for a, b in zip(got[2], want[2]):
        assert a[0].tobytes() == b[0].tobytes()
    for t in range(2, 16):                      # row 1 is live from the join on
        assert got[2][t][1].tobytes() == want[2][t][1].tobytes()
    assert len(got[0]) == 12 and len(got[1]) == 12


def test_gpt2_124m_shape_fp32(orc):
    """configs[0] at full width (12 layers, 768, 12 heads, 3072, vocab 50257), a short run the CPU
    oracle finishes in seconds: prompt 4 + 4 greedy steps for sequence 0, a second sequence joining."""
    from wukong_b200.wk_programs import GPT2Flat
    orc.set_threads(8)
    w = GPT2Flat(n_layer=12, d=768, n_head=12, d_ff=3072, vocab=50257, n_pos=1024, seed=0)
    rng = np.random.default_rng(0)
    p0, p1 = rng.integers(0, 50257, 4).tolist(), rng.integers(0, 50257, 2).tolist()
    got, want = _both(orc, w, p0, p1, 7, 2)
    assert got[0] == want[0] and got[1] == want[1]
    for t in range(7):
        assert got[2][t][0].tobytes() == want[2][t][0].tobytes(), t
    orc.set_threads(1)


def test_llama_block_example(orc):
    """examples/llama_block.wk through the C ABI: the reference's golden values, and every output lane
    equal to the oracle's run of the same trace."""
    from wukong_b200 import _lib, runtime, wk_programs
    from oracle_rt import OracleRT
    import fixtures_wk as fx
    _lib.require_gpu()
    ins = wk_programs.llama_block_inputs()
    got = wk_programs.llama_block(runtime, **ins)
    want = wk_programs.llama_block(OracleRT(orc), **ins)
    assert [int(t) for t in fx.rust_round(got[[0, 64, 256, 511]] * np.float32(10000.0))] == [-1227, 1204, 593, -404]
    assert got.tobytes() == want.tobytes()

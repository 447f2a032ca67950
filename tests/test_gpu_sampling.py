"""GPU parity of top-k / argsort / categorical sampling / Philox fill with the CPU oracle: every result is unique under
the reference's total orders and index-order f64 sums, so the comparison is exact."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    from wukong_b200 import _lib, runtime
    _lib.require_gpu()
    return runtime


def awkward(n, seed):
    """Many duplicates, signed zeros, NaNs and infinities (the shape of the reference's own selection test)."""
    rng = np.random.default_rng(seed)
    x = rng.integers(-5, 6, n).astype(np.float32)
    x[rng.random(n) < 0.05] = np.nan
    x[rng.random(n) < 0.05] = -0.0
    x[rng.random(n) < 0.02] = np.inf
    x[rng.random(n) < 0.02] = -np.inf
    return x


def test_topk_and_argsort_match_the_total_order(rt, orc):
    for n, k, seed in [(8, 5, 0), (97, 97, 1), (1000, 40, 2), (50257, 50, 3), (5000, 300, 4), (3, 8, 5)]:
        x = awkward(n, seed) if seed % 2 else np.random.default_rng(seed).standard_normal(n).astype(np.float32)
        vals, idx = np.full(k, 9.0, np.float32), np.full(k, 9, np.int64)
        got = rt.topk(x, vals, idx)
        want, wv, wi = orc.topk(x, k)
        assert got == want and np.array_equal(idx, wi)
        assert vals[:got].tobytes() == wv[:want].tobytes() or np.array_equal(np.isnan(vals[:got]), np.isnan(wv[:want]))
        assert np.array_equal(vals[got:], wv[want:])           # past k: untouched
        for desc in (False, True):
            m = min(n, 64) if n > 1000 else n
            gi = np.full(m, 9, np.int64)
            assert rt.argsort(x, gi, desc) == orc.argsort(x, m, desc)[0]
            assert np.array_equal(gi, orc.argsort(x, m, desc)[1]), (n, desc)
    # outputs may overlap the input: the selection sees the original values
    x = np.array([0.5, 2.0, 1.0], np.float32)
    idx = np.zeros(3, np.int64)
    assert rt.topk(x, x, idx) == 3 and x.tolist() == [2.0, 1.0, 0.5] and idx.tolist() == [1, 2, 0]
    assert rt.topk(np.zeros(0, np.float32), np.zeros(2, np.float32), np.zeros(2, np.int64)) == 0


def test_sample_categorical_is_bit_for_bit_the_index_order_f64_cdf(rt, orc):
    rng = np.random.default_rng(7)
    p = np.array([0.0, 1.0, np.nan, 2.0, -4.0, np.inf, 1.0], np.float32)
    for u in (0.0, 0.2499, 0.25, 0.7499, 0.75, 1.0, 7.0, -3.0, float("nan")):
        assert rt.sample_categorical(p, u) == orc.sample_categorical(p, u)
    assert rt.sample_categorical(np.array([0.0, -1.0, np.nan], np.float32), 0.5) == -1
    assert rt.sample_categorical(np.zeros(0, np.float32), 0.5) == -1
    # a softmax-like row over a vocabulary, spanning ~40 binades: the running sum rounds, so the order of the adds matters
    w = np.exp(rng.standard_normal(50257).astype(np.float32) * 6).astype(np.float32)
    for u in rng.random(40).astype(np.float32):
        assert rt.sample_categorical(w, float(u)) == orc.sample_categorical(w, float(u))


def test_rand_fill_is_the_philox_stream(rt, orc):
    for n, seed, ctr0 in [(5, 42, -2), (1000, 0, 0), (257, -1, 3), (1, 0xDEADBEEF, 1 << 40)]:
        out = np.full(n, 7.0, np.float32)
        rt.rand_fill(out, seed, ctr0)
        assert out.tobytes() == orc.rand_fill(n, seed, ctr0).tobytes()
    untouched = np.full(2, 7.0, np.float32)
    rt.rand_fill(untouched[:0], 1, 1)
    assert untouched.tolist() == [7.0, 7.0]


def test_device_rows_api(orc):
    import torch
    from wukong_b200._lib import lib, check, require_gpu
    require_gpu()
    rng = np.random.default_rng(11)
    rows, cols, k = 6, 4099, 17
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    x[2, 5] = np.nan
    xt = torch.from_numpy(x).cuda()
    vals = torch.zeros(rows, k, device="cuda")
    idx = torch.zeros(rows, k, dtype=torch.int64, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    check(lib().wkb_topk_rows_f32(xt.data_ptr(), cols, rows, cols, k, vals.data_ptr(), idx.data_ptr(), s), "topk_rows")
    w = np.abs(x)
    u = rng.random(rows).astype(np.float32)
    out = torch.zeros(rows, dtype=torch.int64, device="cuda")
    wt, ut = torch.from_numpy(w).cuda(), torch.from_numpy(u).cuda()
    check(lib().wkb_sample_categorical_rows_f32(wt.data_ptr(), cols, rows, cols, ut.data_ptr(), out.data_ptr(), s), "sample_rows")
    torch.cuda.synchronize()
    for r in range(rows):
        assert np.array_equal(idx[r].cpu().numpy(), orc.topk(x[r], k)[2])
        assert int(out[r]) == orc.sample_categorical(w[r], float(u[r]))

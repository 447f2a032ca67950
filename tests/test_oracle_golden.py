"""The CPU oracle against the reference's own golden vectors (tests/run/*.wk EXPECT-OUT lines and
the constructions of its unit tests).  No GPU, no product code."""
import math

import numpy as np
import pytest

import fixtures_wk as fx

EXP, LOG, TANH, SIGMOID, RELU, SILU, GELU = range(7)
SOFTMAX, LAYERNORM, RMSNORM, LOGSOFTMAX, L2NORM = range(5)


def ints(lines):
    return [int(float(s)) for s in lines]


def floats(lines):
    return [float(s) for s in lines]


def test_activations_fixture(orc, golden):
    x, xp = fx.activations_x()
    got = []
    got += list(fx.rust_round(orc.vmath(x, EXP).astype(np.float64) * 100.0))
    got += list(fx.rust_round(orc.vmath(xp, LOG) * np.float32(1000.0)))
    for op in (TANH, SIGMOID, SILU, GELU, RELU):
        got += list(fx.rust_round(orc.vmath(x, op) * np.float32(1000.0)))
    assert [int(g) for g in got] == ints(golden["builtin_activations"])


def test_exp_log_tanh_accuracy_claims(orc):
    # vmath.rs:164-166, :213-215: exp <= 2 ULP on [-87, 88.37], log <= 12 ULP, tanh <= 1 ULP.
    L = orc.lib()
    rng = np.random.default_rng(0)
    xs = rng.uniform(-87.0, 88.37, 20000).astype(np.float32)
    worst = 0.0
    for x in xs:
        ref = math.exp(float(x))
        worst = max(worst, abs(L.wko_exp1(float(x)) - ref) / ref)
    assert worst <= 1.7e-7
    assert L.wko_exp1(0.0) == 1.0
    assert L.wko_exp1(-88.37626) == 0.0
    assert L.wko_exp1(float("-inf")) == 0.0 and L.wko_exp1(float("inf")) == float("inf")
    worst = 0.0
    for x in np.exp(rng.uniform(-80, 80, 20000)).astype(np.float32):
        ref = math.log(float(x))
        if ref != 0.0:
            worst = max(worst, abs(L.wko_log1(float(x)) - ref) / abs(ref))
    assert worst <= 7e-7
    for x in rng.uniform(-12, 12, 20000).astype(np.float32):
        ref = np.float32(math.tanh(float(x)))
        got = np.float32(L.wko_tanh1(float(x)))
        assert abs(int(got.view(np.int32)) - int(ref.view(np.int32))) <= 1


def test_norms_fixture(orc, golden):
    want = ints(golden["builtin_norms"])
    x = np.array([[1, 2, 3, 4], [0, 0, 0, 0]], np.float32)
    v = (np.arange(13, dtype=np.float32) * np.float32(0.5) - np.float32(3.0)).reshape(1, 13)
    xl = np.array([[1, 2, 3, 4], [-2, 0, 2, 8]], np.float32)
    got = []
    show = lambda y: [int(t) for t in fx.rust_round(y.ravel() * np.float32(10000.0))]
    got += show(orc.norm(x, SOFTMAX))
    got += show(orc.norm(v, SOFTMAX))
    got += show(orc.norm(x, LOGSOFTMAX))
    got += show(orc.norm(x[:1], SOFTMAX))
    got += show(orc.norm_affine(xl, [1, 2, 0.5, -1], [0, 1, -1, 0.5], LAYERNORM, 1e-5))
    got += show(orc.norm_affine(xl, [1, 1, 2, 0.5], None, RMSNORM, 1e-5))
    got += show(orc.norm_affine(xl, [1, 1, 2, 0.5], None, RMSNORM, 1e-5))
    assert got == want


def test_norm_blocked_every_lane(orc, golden):
    want = ints(golden["norm_blocked_every_lane"])
    a = np.array([((i * 3) % 7) + 1 for i in range(100)], np.float32).reshape(1, -1)
    b = np.array([((i * 3) % 7) + 1 for i in range(112)], np.float32).reshape(1, -1)
    got = [int(t) for t in fx.rust_round(orc.norm(a, L2NORM, 1e-5).ravel() * np.float32(400.0))]
    got += [int(t) for t in fx.rust_round(orc.norm(b, LAYERNORM, 1e-5).ravel() * np.float32(1000.0))]
    assert got == want


def test_norm_matches_f64(orc):
    rng = np.random.default_rng(1)
    for cols in (1, 7, 8, 63, 64, 65, 100, 112, 768, 4096):
        x = rng.standard_normal((3, cols)).astype(np.float32)
        g = rng.standard_normal(cols).astype(np.float32)
        b = rng.standard_normal(cols).astype(np.float32)
        x64 = x.astype(np.float64)
        e = np.exp(x64 - x64.max(1, keepdims=True))
        np.testing.assert_allclose(orc.norm(x, SOFTMAX), e / e.sum(1, keepdims=True), rtol=2e-6, atol=1e-9)
        mu = x64.mean(1, keepdims=True)
        var = ((x64 - mu) ** 2).mean(1, keepdims=True)
        ln = (x64 - mu) / np.sqrt(var + 1e-5) * g + b
        np.testing.assert_allclose(orc.norm_affine(x, g, b, LAYERNORM, 1e-5), ln, rtol=1e-4, atol=1e-5)
        rms = x64 / np.sqrt((x64 ** 2).mean(1, keepdims=True) + 1e-5) * g
        np.testing.assert_allclose(orc.norm_affine(x, g, None, RMSNORM, 1e-5), rms, rtol=1e-5, atol=1e-6)


def test_matmul_fixture(orc, golden):
    want = floats(golden["builtin_matmul"])
    a = np.array([1, 2, 3, 4, 5, 6], np.float32)
    b = np.arange(1, 13, dtype=np.float32)
    w = np.array([1, 0, 0, 0, 1, 0, 0, 0, 1, 1, 1, 1], np.float32)
    at = np.array([1, 4, 2, 5, 3, 6], np.float32)
    got = []
    ab = orc.sgemm(a, b, 2, 3, 4, "nn").ravel()
    got += list(ab) + list(ab)
    got += list(orc.sgemm(a, w, 2, 3, 4, "nt").ravel())
    got += list(orc.sgemm(at, b, 2, 3, 4, "tn").ravel())
    got += list(orc.sgemm(a, w, 2, 3, 4, bias=[0.5, -1, 2, 0], act=0).ravel())
    got += list(a.reshape(2, 3).T.ravel())  # transpose: pure data movement, not a hot-path kernel
    got += list(orc.sgemm([1, 2, 3, 4], [5, 6, 7, 8], 2, 2, 2, "nn").ravel())
    got += list(ab)
    # K = 0: the kernel writes nothing (sentinels survive); the builtin's lowering fills zeros / bias.
    z = orc.sgemm(np.zeros(0, np.float32), np.zeros(0, np.float32), 2, 0, 2, "nn", c=np.full((2, 2), 7.0))
    assert (z == 7.0).all()
    got += [0.0] * 4 + [1.5, -2.0, 1.5, -2.0] + [0.0] * 4
    got += list(ab)
    assert got == want


def test_select_kc_partition(orc):
    # gemm.rs:253-256: round_up(ceil(k / ceil(k/384)), 4), result in [4, 384].
    L = orc.lib()
    assert [L.wko_select_kc(k) for k in (1, 4, 384, 385, 512, 768, 1024, 4096, 11008)] == \
        [4, 4, 384, 196, 256, 384, 344, 376, 380]


def test_sgemm_order_contract_vs_f64(orc):
    rng = np.random.default_rng(2)
    for (m, k, n) in [(1, 1, 1), (7, 17, 13), (6, 16, 5), (13, 19, 4), (13, 391, 19), (5, 805, 9)]:
        a = rng.standard_normal((m, k)).astype(np.float32)
        b = rng.standard_normal((n, k)).astype(np.float32)
        bias = rng.standard_normal(n).astype(np.float32)
        c = orc.sgemm(a, b, m, k, n, "nt")
        exact = a.astype(np.float64) @ b.astype(np.float64).T
        kc = orc.lib().wko_select_kc(k)
        r = kc + (k + kc - 1) // kc - 1
        u = 2.0 ** -24
        bound = (r * u / (1 - r * u)) * (np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64).T)
        assert (np.abs(c - exact) <= bound + 1e-30).all()
        # fused epilogue == unfused, bit for bit (gemm.rs module docs)
        fused = orc.sgemm(a, b, m, k, n, bias=bias, act=2)
        unf = orc.vmath((c + bias).astype(np.float32), GELU).reshape(m, n)
        assert fused.tobytes() == unf.tobytes()
        # nn / tn agree with nt on transposed storage
        assert orc.sgemm(a, np.ascontiguousarray(b.T), m, k, n, "nn").tobytes() == c.tobytes()
        assert orc.sgemm(np.ascontiguousarray(a.T), np.ascontiguousarray(b.T), m, k, n, "tn").tobytes() == c.tobytes()


def test_gemv_half_fixture(orc, golden):
    want = floats(golden["decode_gemv_half"])
    w, x = fx.gemv_half_operands()
    wb = orc.to_bf16_bits(w.ravel())
    wh = (w.ravel() * np.float32(0.25)).astype(np.float16).view(np.uint16)
    st, y = orc.sgemv_half(wb, x, 11, bf16=True)
    st2, z = orc.sgemv_half(wh, x, 11, bf16=False)
    assert st == 0 and st2 == 0
    assert list(y) + list(z) == want
    # bad extent: nothing written
    st, y = orc.sgemv_half(wb[:-1], x, 11)
    assert st == -2 and (y == 7.0).all()
    # M = 1 row of the half GEMM with a widened x (gemv_half.rs module docs)
    xb = orc.to_bf16_bits(x)
    c = orc.sgemm_half_nt(xb, wb, 1, 13, 11, bf16=True)
    st, y = orc.sgemv_half(wb, orc.from_bf16_bits(xb), 11)
    assert c.ravel().tobytes() == y.tobytes()


def test_gemv_quant_fixture(orc, golden):
    want = ints(golden["decode_gemv_quant"])
    w8, w4, x = fx.gemv_quant_operands()
    q8 = orc.quantize(w8, 40, q4=False)
    q4 = orc.quantize(w4, 40, q4=True)
    st, y8 = orc.gemv_q(q8, x, 9, q4=False)
    st2, y4 = orc.gemv_q(q4, x, 9, q4=True)
    assert st == 0 and st2 == 0
    got = [int(b) for b in q8[:4]] + [int(v) for v in y8] + [int(b) for b in q4[:36]] + [int(v) for v in y4]
    assert got == want
    assert q8.size == 612 and q4.size == 324


def test_quant_unit_constructions(orc):
    # quant.rs:880-1099: NaN -> nibble 8 / quant 0, padding -> zero nibble, bad extents, K = 0.
    x = np.zeros(32, np.float32)
    x[0] = np.nan
    x[1] = -8.0
    q = orc.quantize(x, 32, q4=True)
    assert q[0] == 0x00 and q[1] == 0x3C  # scale 1.0
    assert q[2] & 0x0F == 8 and q[3] & 0x0F == 0
    st, y = orc.gemv_q(np.zeros(0, np.uint8), np.zeros(0, np.float32), 3)
    assert st == 0 and (y == 0.0).all()
    st, y = orc.gemv_q(np.zeros(17, np.uint8), np.zeros(32, np.float32), 1)
    assert st == -2 and (y == 7.0).all()
    # dequantised weights x exact activations reproduce the integer dot (quant.rs:969-999)
    rng = np.random.default_rng(3)
    for (n, k) in [(1, 1), (7, 31), (8, 32), (9, 33), (17, 100), (40, 257)]:
        w = rng.uniform(-1, 1, (n, k)).astype(np.float32)
        xv = rng.uniform(-1, 1, k).astype(np.float32)
        qw = orc.quantize(w, k)
        st, y = orc.gemv_q(qw, xv, n)
        assert st == 0
        quants, scales = orc.unpack_q4_0(qw)
        nb = (k + 31) // 32
        deq = (quants.reshape(n, nb, 32).astype(np.float64)
               * scales.view(np.float16).astype(np.float64).reshape(n, nb, 1)).reshape(n, nb * 32)[:, :k]
        ref = deq @ xv.astype(np.float64)
        amax = np.abs(xv).max()
        tol = np.abs(deq).sum(1) * (amax / 127.0) * 0.5 + 1e-6  # half a Q8 step per element
        assert (np.abs(y - ref) <= tol).all()


def test_int4_dequant_fixture(orc, golden):
    L = orc.lib()
    w = np.array([0x7F, 0x80, 0x21, 0xED, 0x3C], np.uint8)
    s = np.array([0.5, 0.25, -2.0], np.float32)
    zr = np.array([8.0, 7.5, 0.0], np.float32)
    a = np.zeros(10, np.float32)
    assert L.wko_dequant_i4_f32(orc.p(w), 5, orc.p(s), 3, 4, orc.p(a), 10) == 0
    b = np.zeros(10, np.float32)
    assert L.wko_dequant_u4_f32(orc.p(w), 5, orc.p(s), 3, orc.p(zr), 3, 4, orc.p(b), 10) == 0
    odd = np.zeros(9, np.float32)
    assert L.wko_dequant_u4_f32(orc.p(w), 5, orc.p(s), 3, orc.p(zr), 3, 4, orc.p(odd), 9) == 0
    one = np.array([0.125], np.float32)
    c = np.zeros(10, np.float32)
    assert L.wko_dequant_i4_f32(orc.p(w), 5, orc.p(one), 1, 10, orc.p(c), 10) == 0
    fmt = lambda v: "[" + ", ".join(repr(float(t)) for t in v) + "]"
    assert [fmt(a), fmt(b), fmt(odd), fmt(c), fmt(a)] == golden["int4_dequant"]
    assert L.wko_dequant_i4_f32(orc.p(w), 4, orc.p(s), 3, 4, orc.p(a), 10) == -2


def test_kv_attention_fixture(orc, golden):
    want = floats(golden["decode_kv_attention"])
    kc, vc, steps, q2 = fx.kv_attention_steps()
    L = orc.lib()
    got = []
    for s in steps:
        t = s["t"]
        assert L.wko_kv_append_f32(orc.p(kc), 32, orc.p(s["krow"]), 8, t, 8) == 0
        assert L.wko_kv_append_f32(orc.p(vc), 32, orc.p(s["vrow"]), 8, t, 8) == 0
        st, o = orc.attention_kv(s["q"], kc, vc, 1, t + 1, 4, t, 4, 2, 16, 8, 1.0, True, o_init=0.0)
        assert st == 0
        got += list(o)
    st, o2 = orc.attention_kv(q2, kc, vc, 2, 4, 4, 2, 4, 2, 20, 8, 1.0, True)
    assert st == 0
    got += list(o2)
    assert got == want


def test_kv_batch_fixtures(orc, golden):
    for name, ops in (("decode_kv_batch", fx.kv_batch_operands()), ("decode_kv_batch_gqa", fx.kv_batch_gqa_operands())):
        st, o = orc.attention_kv_batch(ops["q"], ops["k"], ops["v"], ops["lens"], ops["pos"], *ops["geo"], 1.0, True)
        assert st == 0
        want = floats(golden[name])
        assert list(o) == want[: o.size]
        if len(want) > o.size:
            assert list(o) == want[o.size:]  # the _parallel twin prints the same lanes


def test_kv_status_codes(orc):
    q = np.zeros(16, np.float32)
    kv = np.zeros(8, np.float32)
    assert orc.attention_kv(q, kv, kv, 1, 1, 4, 0, 4, 3, 16, 8, 1.0, True)[0] == -1  # heads not divisible
    assert orc.attention_kv(q, kv, kv, 1, 2, 4, 0, 4, 2, 16, 8, 1.0, True)[0] == -2  # short cache
    assert orc.attention_kv(q, kv, kv, 0, 1, 4, 0, 4, 2, 16, 8, 1.0, True)[0] == 0   # nothing to do
    st, o = orc.attention_kv_batch(q, kv, kv, [2], [0], 1, 1, 1, 4, 2, 4, 1.0, True)
    assert st == -1 and (o == -1.0).all()  # kv_len > skv, nothing written
    L = orc.lib()
    c = np.zeros(8, np.float32)
    r = np.ones(4, np.float32)
    assert L.wko_kv_append_f32(orc.p(c), 8, orc.p(r), 4, 2, 4) == -2
    assert L.wko_kv_append_f32(orc.p(c), 8, orc.p(r), 4, 1, 3) == -1
    assert L.wko_kv_append_f32(orc.p(c), 8, orc.p(r), 4, 1, 4) == 0 and (c[4:] == 1).all()


def test_kv_attention_geometries_vs_f64(orc):
    # attention_kv.rs:1375-1392, tolerance :1528-1530 (1e-4 + 1e-4*|w|).
    rng = np.random.default_rng(4)
    geos = [(1, 5, 8, 4, 4, 4, 0, 0), (1, 70, 12, 69, 8, 2, 3, 5), (3, 130, 16, 127, 6, 6, 0, 0),
            (2, 64, 5, 62, 12, 1, 0, 2), (1, 65, 128, 64, 32, 8, 0, 0)]
    for (sq, skv, d, p0, h, hkv, qpad, kvpad) in geos:
        qs, ks = h * d + qpad, hkv * d + kvpad
        q = rng.standard_normal(sq * qs).astype(np.float32)
        k = rng.standard_normal(skv * ks).astype(np.float32)
        v = rng.standard_normal(skv * ks).astype(np.float32)
        scale = 1.0 / math.sqrt(d)
        st, o = orc.attention_kv(q, k, v, sq, skv, d, p0, h, hkv, qs, ks, scale, True)
        assert st == 0
        for i in range(sq):
            keys = min(skv, p0 + i + 1)
            for hh in range(h):
                g = hh // (h // hkv)
                qv = q[i * qs + hh * d: i * qs + hh * d + d].astype(np.float64)
                kk = np.stack([k[j * ks + g * d: j * ks + g * d + d] for j in range(keys)]).astype(np.float64)
                vv = np.stack([v[j * ks + g * d: j * ks + g * d + d] for j in range(keys)]).astype(np.float64)
                s = kk @ qv * scale
                w = np.exp(s - s.max())
                ref = (w / w.sum()) @ vv
                got = o[i * qs + hh * d: i * qs + hh * d + d]
                assert (np.abs(got - ref) <= 1e-4 + 1e-4 * np.abs(ref)).all()
            if qpad:
                assert (o[i * qs + h * d: (i + 1) * qs] == -1.0).all()


def test_sdpa_fixture(orc, golden):
    want = golden["sdpa"]
    o = orc.attention([1, 0, 0, 1], [1, 0, 0, 1], [1, 2, 3, 4], 2, 2, 1.0, 0)
    got = [str(int(np.float32(t) * np.float32(10000.0))) for t in o]
    o2 = orc.attention([2, 3, 1, 4], [3, 1, 3, 1], [5, 7, 100, 200], 2, 2, 1.0, 1)
    got += [repr(float(t)).rstrip("0").rstrip(".") if float(t).is_integer() else repr(float(t)) for t in o2]
    assert got == want


def test_rope_fixture(orc, golden):
    x = np.array([[1, 2, 3, 4], [1, 2, 3, 4]], np.float32)
    out = orc.rope(x, [1.0, 0.5])
    assert [int(np.float32(t) * np.float32(1000.0)) for t in out.ravel()] == ints(golden["rope"])
    # positions as a vector: row r at pos r reproduces the row-index entry bit for bit
    out2 = orc.rope_pos(x, [1.0, 0.5], [0, 1], heads=1)
    assert out2.tobytes() == out.tobytes()


def test_embedding_rowargmax_fixtures(orc, golden):
    w = np.array([[v * 10 + d for d in range(3)] for v in range(4)], np.float32)
    out = orc.embedding(w, [2, 0, 3, 0])
    assert [int(t) for t in out.ravel()] == ints(golden["embedding"])
    assert (orc.embedding(w, [4, -1]) == 0.0).all()  # out-of-range id -> zero row
    x = np.array([[1, 3, 2, 0], [5, 1, 9, 4], [2, 2, 2, 8]], np.float32)
    assert list(orc.rowargmax(x)) == ints(golden["rowargmax"])[:3]
    assert list(orc.rowargmax(np.array([[np.nan, 5, 6], [1, np.nan, 0], [2, 2, 2]], np.float32))) == [0, 0, 0]


def test_f8_codec_all_codes(orc, golden):
    L = orc.lib()
    for line in golden["f8_code_round_trip"]:
        c, r4, r5, m4, m5 = (int(t) for t in line.split())
        assert L.wko_f32_to_f8e4m3(L.wko_f8e4m3_to_f32(c)) == r4 == m4
        v5 = L.wko_f8e5m2_to_f32(c)
        assert L.wko_f32_to_f8e5m2(v5) == r5 == m5
    assert L.wko_f32_to_f8e4m3(1000.0) == 0x7E and L.wko_f8e4m3_to_f32(0x7E) == 448.0  # saturating
    assert L.wko_f32_to_f8e5m2(1e6) == 0x7C  # overflow to +inf


def test_half_codecs(orc):
    L = orc.lib()
    rng = np.random.default_rng(5)
    xs = np.concatenate([rng.standard_normal(2000).astype(np.float32) * 100, np.array([0.0, -0.0, np.inf, 65504.0, 1e-8], np.float32)])
    for x in xs:
        assert L.wko_f32_to_f16_bits(float(x)) == int(np.float16(x).view(np.uint16))
    import torch
    t = torch.from_numpy(xs.copy()).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert (orc.to_bf16_bits(xs) == t).all()
    assert all(L.wko_f32_to_bf16_bits(float(x)) == int(b) for x, b in zip(xs, t))


def test_tiny_lm_decode(orc, golden):
    """The whole toy decode loop of the reference's decode_tiny_lm fixture: tokens 6 3 0 7 4 1."""
    L = orc.lib()
    wk = np.zeros((12, 20), np.float32); wv = np.zeros((12, 20), np.float32); wq = np.zeros((24, 20), np.float32)
    for i in range(12):
        wk[i, 8 + i] = 1.0
        if i < 8:
            wv[i, i] = 1.0
        if i + 2 < 12:
            wq[i, 8 + i + 2] = 200.0
        if i + 3 < 12:
            wq[12 + i, 8 + i + 3] = 200.0
    wo = np.zeros((8, 24), np.float32)
    for c in range(8):
        src = (c + 7) % 8
        wo[c, src] = 2.0
        wo[c, 12 + src] = 1.0
    woq = orc.quantize(wo, 24, q4=False)
    assert woq.size == 272
    kc = np.zeros(144, np.float32); vc = np.zeros(144, np.float32)
    toks = [5, 2, 7] + [0] * 9
    out = []
    for p in range(8):
        h = np.zeros(20, np.float32)
        h[toks[p]] = 1.0
        h[8 + p] = 1.0
        _, krow = orc.sgemv_half(orc.to_bf16_bits(wk.ravel()), h, 12)
        _, vrow = orc.sgemv_half(orc.to_bf16_bits(wv.ravel()), h, 12)
        assert L.wko_kv_append_f32(orc.p(kc), 144, orc.p(krow), 12, p, 12) == 0
        assert L.wko_kv_append_f32(orc.p(vc), 144, orc.p(vrow), 12, p, 12) == 0
        if p >= 2:
            _, q = orc.sgemv_half(orc.to_bf16_bits(wq.ravel()), h, 24)
            st, att = orc.attention_kv(q, kc, vc, 1, p + 1, 12, p, 2, 1, 24, 12, 1.0, True)
            assert st == 0
            st, logits = orc.gemv_q(woq, att, 8, q4=False)
            assert st == 0
            best = int(orc.rowargmax(logits.reshape(1, 8))[0])
            out.append(best)
            toks[p + 1] = best
    assert out == ints(golden["decode_tiny_lm"])


def test_paged_model_layout_invariance(orc):
    """Two physical page layouts of one logical KV history give identical bits (the property the
    reference pins on its GPU path, serving.rs:2944 / paged_attention.rs:32-47)."""
    rng = np.random.default_rng(6)
    slots, qh, kvh, hd, bs, mbps, nblk = 3, 8, 2, 16, 4, 6, 40
    ctx = np.array([9, 0, 24], np.int32)
    kflat = [rng.standard_normal((c, kvh, hd)).astype(np.float32) for c in ctx]
    vflat = [rng.standard_normal((c, kvh, hd)).astype(np.float32) for c in ctx]
    q = rng.standard_normal((slots, qh * hd)).astype(np.float32)
    outs = []
    for seed in (0, 1):
        perm = np.random.default_rng(seed).permutation(nblk)
        kc = np.full((nblk, bs, kvh, hd), np.nan, np.float32)
        vc = np.full((nblk, bs, kvh, hd), np.nan, np.float32)
        bt = np.zeros((slots, mbps), np.uint32)
        nxt = 0
        for b in range(slots):
            for t in range(ctx[b]):
                if t % bs == 0:
                    bt[b, t // bs] = perm[nxt]; nxt += 1
                kc[bt[b, t // bs], t % bs] = kflat[b][t]
                vc[bt[b, t // bs], t % bs] = vflat[b][t]
        outs.append(orc.paged_attn_decode(q, kc, vc, 0, bt, ctx, slots, qh, kvh, hd, bs, mbps, 0.25))
    assert outs[0].tobytes() == outs[1].tobytes()
    assert (outs[0][1] == 0.0).all()
    assert not np.isnan(outs[0]).any()
    # equals the padded-cache kernel to its tolerance on the same logical history
    skv = int(ctx.max())
    kp = np.zeros((slots, skv, kvh, hd), np.float32); vp_ = np.zeros_like(kp)
    for b in range(slots):
        kp[b, :ctx[b]] = kflat[b]; vp_[b, :ctx[b]] = vflat[b]
    st, o = orc.attention_kv_batch(q, kp, vp_, ctx, ctx - 1, slots, 1, skv, qh, kvh, hd, 0.25, True)
    assert st == 0
    np.testing.assert_allclose(o.reshape(slots, -1), outs[0], rtol=1e-4, atol=1e-4)


def test_llama_block_example_golden(orc):
    """examples/llama_block.wk of the reference: `EXPECT-OUT-VALUES: -1227 1204 593 -404`
    (round(out[k] * 10000) for k = 0, 64, 256, 511), derived there from an independent f64 evaluation."""
    from oracle_rt import OracleRT
    from wukong_b200 import wk_programs
    out = wk_programs.llama_block(OracleRT(orc), **wk_programs.llama_block_inputs())
    assert [int(t) for t in fx.rust_round(out[[0, 64, 256, 511]] * np.float32(10000.0))] == [-1227, 1204, 593, -404]


# ---- selection, sampling and the counter-based RNG (crates/wukong_runtime/src/topk.rs, random.rs) ----------
def test_philox_known_answers_and_builtin_mapping(orc):
    """Random123's published known-answer vectors for philox4x32-10 and the (seed, counter) mapping the reference
    pins in random.rs:109-155."""
    M = 0xFFFFFFFF
    kat = [([0, 0, 0, 0], [0, 0], [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]),
           ([M] * 4, [M] * 2, [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]),
           ([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0], [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1])]
    for ctr, key, want in kat:
        assert [int(v) for v in orc.philox4x32_10(ctr, key)] == want
    assert orc.rand_u32(0, 0) == 0x6627e8d5 and orc.rand_u32(0, 1) == 0xf8e4cca4 and orc.rand_u32(1, 0) == 0xe3e80670
    assert orc.rand_u32(42, 7) == 0x5bbd83b1 and orc.rand_u32(0xDEADBEEFCAFEF00D, 0x123456789ABCDEF0) == 0xdecbb6f2
    assert orc.rand_u32(0xFFFFFFFFFFFFFFFF, 3) == 0x8e8fd014
    f = orc.rand_fill(5, 42, -2)                      # the counter wraps: lane 2 is counter 0
    assert f[2] == np.float32((orc.rand_u32(42, 0) >> 8) / 16777216.0)
    assert orc.rand_fill(1, 0, 0)[0] == np.float32(6694888.0 / 16777216.0)
    assert orc.rand_fill(1, 42, 7)[0] == np.float32(6012291.0 / 16777216.0)
    assert orc.rand_fill(0, 1, 1).size == 0


def test_topk_argsort_total_order(orc):
    """topk.rs:244-286: NaN largest, ties (signed zeros, NaNs) to the lower index; ascending sort is stable, NaN last."""
    nan = np.nan
    x = np.array([1.0, nan, 3.0, -0.0, 3.0, 0.0, nan, -5.0], np.float32)
    k, vals, idx = orc.topk(x, 5)
    assert k == 5 and idx.tolist() == [1, 6, 2, 4, 0]
    assert np.isnan(vals[:2]).all() and vals[2:].tolist() == [3.0, 3.0, 1.0]
    k, vals, idx = orc.topk(np.array([0.0, -0.0, 0.0], np.float32), 3)
    assert idx.tolist() == [0, 1, 2] and np.signbit(vals[1])
    assert orc.topk(np.zeros(0, np.float32), 3)[0] == 0
    y = np.array([2.0, nan, -1.0, 2.0, 0.5, -1.0], np.float32)
    assert orc.argsort(y, 6)[1].tolist() == [2, 5, 4, 0, 3, 1]
    assert orc.argsort(y, 6, True)[1].tolist() == [1, 0, 3, 4, 2, 5]
    m, short = orc.argsort(y, 2)
    assert m == 2 and short.tolist() == [2, 5]
    m, long = orc.argsort(y[:3], 8)
    assert m == 3 and long.tolist() == [2, 0, 1, 9, 9, 9, 9, 9]


def test_sample_categorical_inverse_cdf(orc):
    """topk.rs:309-323: mass = the weight when positive and finite, first index whose running mass exceeds u * total."""
    p = [0.0, 1.0, np.nan, 2.0, -4.0, np.inf, 1.0]
    want = {0.0: 1, 0.2499: 1, 0.25: 3, 0.7499: 3, 0.75: 6, 1.0: 6, 7.0: 6, -3.0: 1}
    for u, i in want.items():
        assert orc.sample_categorical(p, u) == i, u
    assert orc.sample_categorical(p, np.nan) == 1
    assert orc.sample_categorical([0.0, -1.0, np.nan], 0.5) == -1
    assert orc.sample_categorical([], 0.5) == -1

"""Parity of the CUDA path (called through the C ABI with host buffers) against the CPU oracle and
the reference's golden vectors.  fp32 entries are bit-exact; tolerances are stated where they are not."""
import math

import numpy as np
import pytest

import fixtures_wk as fx

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    import wukong_b200
    from wukong_b200 import _lib, runtime
    _lib.require_gpu()
    return runtime


def bits_equal(a, b):
    return np.ascontiguousarray(a).tobytes() == np.ascontiguousarray(b).tobytes()


def assert_bits(a, b, what=""):
    """Bit equality on every lane; a NaN lane must be a NaN lane (GPU arithmetic returns the
    canonical NaN instead of propagating an operand's payload, so NaN payload bits are not compared)."""
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    if a.tobytes() != b.tobytes():
        diff = a.view(np.uint32).ravel() != b.view(np.uint32).ravel()
        if a.dtype == np.float32:
            diff &= ~(np.isnan(a.ravel()) & np.isnan(b.ravel()))
        bad = np.flatnonzero(diff)
        if bad.size == 0:
            return
        raise AssertionError("%s: %d of %d lanes differ, first %d: %r vs %r" % (
            what, bad.size, a.size, bad[0], a.ravel()[bad[0]], b.ravel()[bad[0]]))


def test_vmath_bit_exact(rt, orc):
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(100003).astype(np.float32) * 4,
                        np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 88.4, -88.4, 1e-40, -1e-40, 0.75, 10.0], np.float32)])
    for name, op in (("exp", 0), ("tanh", 2), ("sigmoid", 3), ("relu", 4), ("silu", 5), ("gelu", 6)):
        out = np.empty_like(x)
        getattr(rt, name)(x, out)
        assert_bits(out, orc.vmath(x, op), name)
    xp = np.abs(x) + np.float32(1e-3)
    out = np.empty_like(xp)
    rt.log(xp, out)
    assert_bits(out, orc.vmath(xp, 1), "log")
    for op in (15, 16):
        xs = (rng.standard_normal(5000) * 300).astype(np.float32)
        from wukong_b200 import lib
        out = np.empty_like(xs)
        lib().wukong_vmath_f32(xs.ctypes.data, out.ctypes.data, xs.size, op)
        assert_bits(out, orc.vmath(xs, op), "sincos")
    a, b = x[:5000].copy(), rng.standard_normal(5000).astype(np.float32)
    out = np.empty_like(a)
    rt.silu_gate(a, b, out)
    assert_bits(out, orc.vmath2(a, b, 9), "silu_gate")
    # in place
    y = x.copy()
    rt.gelu(y, y)
    assert_bits(y, orc.vmath(x, 6), "gelu in place")


def test_activations_golden(rt, golden):
    x, xp = fx.activations_x()
    got = []
    y = np.empty_like(x)
    rt.exp(x, y); got += list(fx.rust_round(y.astype(np.float64) * 100.0))
    rt.log(xp, y); got += list(fx.rust_round(y * np.float32(1000)))
    for f in (rt.tanh, rt.sigmoid, rt.silu, rt.gelu, rt.relu):
        f(x, y); got += list(fx.rust_round(y * np.float32(1000)))
    assert [int(g) for g in got] == [int(s) for s in golden["builtin_activations"]]


def test_velem_bit_exact(rt, orc):
    from wukong_b200 import lib
    rng = np.random.default_rng(1)
    x = rng.standard_normal(10007).astype(np.float32)
    y = rng.standard_normal(10007).astype(np.float32)
    for (a, b, c, op) in [(1.0, 1.0, 0.0, 256), (2.5, -0.5, 0.25, 256 | 1), (1.0, 0.0, 0.0, 0), (3.0, 0.0, 1.0, 2),
                          (1.0, 1.0, 0.0, 512), (1.0, 1.0, 0.0, 1024)]:
        out = np.empty_like(x)
        lib().wukong_velem_f32(x.ctypes.data, y.ctypes.data, out.ctypes.data, x.size, a, b, c, op)
        assert_bits(out, orc.velem(x, y, a, b, c, op), "velem %d" % op)


def test_norms_bit_exact(rt, orc, golden):
    rng = np.random.default_rng(2)
    for rows, cols in [(3, 1), (2, 7), (5, 8), (3, 63), (4, 64), (3, 65), (2, 100), (2, 112), (9, 768), (3, 4096), (2, 50257)]:
        x = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
        g = rng.standard_normal(cols).astype(np.float32)
        b = rng.standard_normal(cols).astype(np.float32)
        out = np.empty_like(x)
        rt.softmax(x, out, rows, cols); assert_bits(out, orc.norm(x, 0), "softmax %d" % cols)
        rt.log_softmax(x, out, rows, cols); assert_bits(out, orc.norm(x, 3), "log_softmax %d" % cols)
        rt.layernorm(x, g, b, out, rows, cols, 1e-5); assert_bits(out, orc.norm_affine(x, g, b, 1, 1e-5), "layernorm %d" % cols)
        rt.rmsnorm(x, g, out, rows, cols, 1e-5); assert_bits(out, orc.norm_affine(x, g, None, 2, 1e-5), "rmsnorm %d" % cols)
        from wukong_b200 import lib
        lib().wukong_norm_f32(x.ctypes.data, out.ctypes.data, rows, cols, rt.eps_bits(1e-5), 4)
        assert_bits(out, orc.norm(x, 4, 1e-5), "l2norm %d" % cols)
        lib().wukong_norm_f32(x.ctypes.data, out.ctypes.data, rows, cols, rt.eps_bits(1e-5), 1)
        assert_bits(out, orc.norm(x, 1, 1e-5), "plain layernorm %d" % cols)
    # NaN / -inf rows follow ordinary exceptional arithmetic, identically
    x = rng.standard_normal((3, 100)).astype(np.float32)
    x[0, 70] = np.nan; x[1, :] = -np.inf; x[2, 3] = np.inf
    out = np.empty_like(x)
    rt.softmax(x, out, 3, 100)
    ref = orc.norm(x, 0)
    assert np.array_equal(np.isnan(out), np.isnan(ref))
    # in place
    y = x.copy(); y[:] = rng.standard_normal((3, 100)).astype(np.float32); y0 = y.copy()
    rt.softmax(y, y, 3, 100); assert_bits(y, orc.norm(y0, 0), "softmax in place")
    # golden fixture
    xl = np.array([[1, 2, 3, 4], [-2, 0, 2, 8]], np.float32)
    o = np.empty_like(xl)
    rt.layernorm(xl, np.array([1, 2, 0.5, -1], np.float32), np.array([0, 1, -1, 0.5], np.float32), o, 2, 4, 1e-5)
    assert [int(t) for t in fx.rust_round(o.ravel() * np.float32(10000))] == [int(s) for s in golden["builtin_norms"][33:41]]
    # unknown code: nothing written
    o[:] = 7.0
    lib().wukong_norm_f32(xl.ctypes.data, o.ctypes.data, 2, 4, 0, 9)
    assert (o == 7.0).all()


def test_gemm_bit_exact(rt, orc, golden):
    rng = np.random.default_rng(3)
    from wukong_b200 import lib
    for (m, k, n) in [(1, 1, 1), (7, 17, 13), (6, 16, 5), (13, 19, 4), (150, 20, 20), (13, 391, 19), (13, 805, 19),
                      (64, 768, 96), (1, 768, 300), (130, 64, 70)]:
        a = rng.standard_normal((m, k)).astype(np.float32)
        b = rng.standard_normal((n, k)).astype(np.float32)
        bias = rng.standard_normal(n).astype(np.float32)
        c = np.zeros((m, n), np.float32)
        rt.matmul_nt(a, b, c, m, k, n); assert_bits(c, orc.sgemm(a, b, m, k, n, "nt"), "nt %s" % ((m, k, n),))
        bn = np.ascontiguousarray(b.T)
        rt.matmul(a, bn, c, m, k, n); assert_bits(c, orc.sgemm(a, bn, m, k, n, "nn"), "nn")
        at = np.ascontiguousarray(a.T)
        rt.matmul_tn(at, bn, c, m, k, n); assert_bits(c, orc.sgemm(at, bn, m, k, n, "tn"), "tn")
        for act in ("identity", "relu", "gelu", "silu"):
            rt.linear(a, b, bias, c, m, k, n, act)
            assert_bits(c, orc.sgemm(a, b, m, k, n, bias=bias, act=rt.ACT[act]), "linear " + act)
        c0 = rng.standard_normal((m, n)).astype(np.float32)
        c1 = c0.copy()
        lib().wukong_sgemm_nt(a.ctypes.data, b.ctypes.data, c1.ctypes.data, m, k, n, 1)
        assert_bits(c1, orc.sgemm(a, b, m, k, n, "nt", beta=1, c=c0), "beta")
        lib().wukong_sgemm_nt_alpha(a.ctypes.data, b.ctypes.data, c1.ctypes.data, m, k, n, 0, 0.125)
        assert_bits(c1, orc.sgemm(a, b, m, k, n, alpha=0.125), "alpha")
        ab, bb = orc.to_bf16_bits(a), orc.to_bf16_bits(b)
        lib().wukong_sgemm_bf16_nt(ab.ctypes.data, bb.ctypes.data, c1.ctypes.data, m, k, n, 0)
        assert_bits(c1, orc.sgemm_half_nt(ab, bb, m, k, n), "bf16 nt")
        ah, bh = a.astype(np.float16).view(np.uint16), b.astype(np.float16).view(np.uint16)
        lib().wukong_sgemm_f16_nt(ah.ctypes.data, bh.ctypes.data, c1.ctypes.data, m, k, n, 0)
        assert_bits(c1, orc.sgemm_half_nt(ah, bh, m, k, n, bf16=False), "f16 nt")
    # the golden fixture lanes, incl. the empty contraction handled by the builtin layer
    a = np.array([1, 2, 3, 4, 5, 6], np.float32); b = np.arange(1, 13, dtype=np.float32)
    c = np.zeros(8, np.float32)
    rt.matmul(a, b, c, 2, 3, 4)
    assert list(c) == [float(s) for s in golden["builtin_matmul"][:8]]
    z = np.full(4, 7.0, np.float32)
    rt.linear(np.zeros(0, np.float32), np.zeros(0, np.float32), np.array([1.5, -2.0], np.float32), z, 2, 0, 2)
    assert list(z) == [1.5, -2.0, 1.5, -2.0]
    z[:] = 7.0
    lib().wukong_sgemm(a.ctypes.data, b.ctypes.data, z.ctypes.data, 2, 0, 2, 0)
    assert (z == 7.0).all()


def test_gemv_bit_exact(rt, orc, golden):
    rng = np.random.default_rng(4)
    for (m, n) in [(1, 1), (5, 7), (9, 8), (11, 33), (40, 257), (3, 768), (17, 4096)]:
        a = rng.standard_normal((m, n)).astype(np.float32)
        x = rng.standard_normal(n).astype(np.float32)
        y = np.empty(m, np.float32)
        rt.gemv(a, x, y, m, n); assert_bits(y, orc.sgemv(a, x), "sgemv %s" % ((m, n),))
        rt.gemv(a, x, y, m, n, 0.5); assert_bits(y, orc.sgemv(a, x, 0.5), "sgemv alpha")
    w, x = fx.gemv_half_operands()
    wb = orc.to_bf16_bits(w.ravel()); wh = (w.ravel() * np.float32(0.25)).astype(np.float16).view(np.uint16)
    y = np.full(11, 7.0, np.float32); z = np.full(11, 7.0, np.float32)
    rt.gemv_bf16(wb, x, y); rt.gemv_f16(wh, x, z)
    assert list(y) + list(z) == [float(s) for s in golden["decode_gemv_half"]]
    for (n, k) in [(11, 13), (40, 257), (300, 768), (64, 1000)]:
        wv = orc.to_bf16_bits(rng.standard_normal(n * k).astype(np.float32))
        xv = rng.standard_normal(k).astype(np.float32)
        y = np.empty(n, np.float32)
        rt.gemv_bf16(wv, xv, y)
        assert_bits(y, orc.sgemv_half(wv, xv, n)[1], "gemv_bf16 %s" % ((n, k),))
    with pytest.raises(Exception):
        rt.gemv_bf16(wb[:-1], x, y[:11].copy())


def test_quant_bit_exact(rt, orc, golden):
    rng = np.random.default_rng(5)
    w8, w4, x = fx.gemv_quant_operands()
    q8 = np.zeros(612, np.uint8); q4 = np.zeros(324, np.uint8)
    rt.quantize_q8_0(w8.ravel(), q8, 40); rt.quantize_q4_0(w4.ravel(), q4, 40)
    y8 = np.zeros(9, np.float32); y4 = np.zeros(9, np.float32)
    rt.gemv_q8_0(q8, x, y8); rt.gemv_q4_0(q4, x, y4)
    got = [int(b) for b in q8[:4]] + [int(v) for v in y8] + [int(b) for b in q4[:36]] + [int(v) for v in y4]
    assert got == [int(s) for s in golden["decode_gemv_quant"]]
    for (n, k) in [(1, 1), (7, 31), (8, 32), (9, 33), (17, 100), (40, 257), (128, 4096), (33, 11008)]:
        w = rng.uniform(-1, 1, (n, k)).astype(np.float32)
        if n * k > 64:
            w.ravel()[5] = np.nan
            w.ravel()[17] = np.inf
        xv = rng.standard_normal(k).astype(np.float32)
        for q4f in (True, False):
            bb = 18 if q4f else 34
            q = np.zeros(n * ((k + 31) // 32) * bb, np.uint8)
            (rt.quantize_q4_0 if q4f else rt.quantize_q8_0)(w.ravel(), q, k)
            assert bits_equal(q, orc.quantize(w, k, q4=q4f)), ("packer", n, k, q4f)
            wc = np.where(np.isfinite(w), w, 0).astype(np.float32)
            q = orc.quantize(wc, k, q4=q4f)
            y = np.empty(n, np.float32)
            (rt.gemv_q4_0 if q4f else rt.gemv_q8_0)(q, xv, y)
            assert_bits(y, orc.gemv_q(q, xv, n, q4=q4f)[1], "gemv_q %s q4=%s" % ((n, k), q4f))
    # group int4
    w = np.array([0x7F, 0x80, 0x21, 0xED, 0x3C], np.uint8)
    a = np.zeros(10, np.float32); b = np.zeros(10, np.float32)
    rt.dequant_i4(w, np.array([0.5, 0.25, -2.0], np.float32), 4, a)
    rt.dequant_u4(w, np.array([0.5, 0.25, -2.0], np.float32), np.array([8.0, 7.5, 0.0], np.float32), 4, b)
    assert list(a) == [-0.5, 3.5, 0.0, -4.0, 0.25, 0.5, -0.75, -0.5, 8.0, -6.0]
    assert list(b) == [3.5, -0.5, -4.0, 0.0, -1.625, -1.375, 1.375, 1.625, -24.0, -6.0]


def test_q4_unpack_bit_exact_and_bf16x_variant(orc):
    """Every nibble and scale bit survives the resident layout; the bf16-activation GEMV agrees with
    the f64 evaluation of its defining formula to rtol 1e-4 (fp32 accumulate, exact products)."""
    import torch
    from wukong_b200 import device as dev
    rng = np.random.default_rng(6)
    for (n, k) in [(8, 32), (17, 100), (64, 4096), (40, 11008)]:
        nb = (k + 31) // 32
        raw = rng.integers(0, 256, n * nb * 18, dtype=np.uint8)
        scale = np.abs(rng.standard_normal(n * nb) * 0.02).astype(np.float16).view(np.uint16)
        raw.reshape(-1, 18)[:, 0] = scale & 0xFF
        raw.reshape(-1, 18)[:, 1] = scale >> 8
        if k % 32:
            # padded elements of the last block hold the zero nibble, as the packer leaves them
            blk = raw.reshape(n, nb, 18)[:, -1, 2:]
            for e in range(k % 32, 32):
                j, hi = e % 16, e >= 16
                blk[:, j] = (blk[:, j] & (0x0F if hi else 0xF0)) | ((8 << 4) if hi else 8)
        qs, d = dev.q_split(torch.from_numpy(raw).cuda(), n * nb, q4=True)
        got_q = qs.cpu().numpy().reshape(-1, 16)
        quants, scales = orc.unpack_q4_0(raw)
        lo = (got_q & 0x0F).astype(np.int8) - 8
        hi = (got_q >> 4).astype(np.int8) - 8
        assert np.array_equal(np.concatenate([lo, hi], 1).ravel(), quants)
        assert np.array_equal(d.cpu().numpy().view(np.uint16).ravel(), scales)
        xb = orc.to_bf16_bits(rng.standard_normal(k).astype(np.float32))
        y = dev.gemv_q4_0_bf16x(qs, d, torch.from_numpy(xb.view(np.int16)).cuda(), n, k).cpu().numpy()
        ref = orc.gemv_q4_bf16x(raw, xb, n)
        deq_abs = np.abs(quants.reshape(n, -1).astype(np.float64)) * np.repeat(scales.view(np.float16).astype(np.float64).reshape(n, nb), 32, 1)
        bound = 1e-4 * np.abs(ref) + 1e-5 * (deq_abs[:, :k] @ np.abs(orc.from_bf16_bits(xb)).astype(np.float64)) + 1e-7
        assert (np.abs(y - ref) <= bound).all(), (n, k, np.abs(y - ref).max())


def test_kv_attention_bit_exact(rt, orc, golden):
    kc, vc, steps, q2 = fx.kv_attention_steps()
    got = []
    for s in steps:
        t = s["t"]
        rt.kv_append(kc, s["krow"], t, 8); rt.kv_append(vc, s["vrow"], t, 8)
        o = np.zeros(16, np.float32)
        rt.sdpa_kv(s["q"], kc, vc, o, 1, t + 1, 4, t, 4, 2, 16, 8, 1.0, True)
        got += list(o)
    o2 = np.full(40, -1.0, np.float32)
    rt.sdpa_kv(q2, kc, vc, o2, 2, 4, 4, 2, 4, 2, 20, 8, 1.0, True)
    got += list(o2)
    assert got == [float(s) for s in golden["decode_kv_attention"]]
    for name, ops in (("decode_kv_batch", fx.kv_batch_operands()), ("decode_kv_batch_gqa", fx.kv_batch_gqa_operands())):
        o = np.full(ops["q"].size, -1.0, np.float32)
        rt.sdpa_kv_batch(ops["q"], ops["k"], ops["v"], o, np.array(ops["lens"], np.int32), np.array(ops["pos"], np.int32),
                         1.0, True, *ops["geo"])
        assert list(o) == [float(s) for s in golden[name]][: o.size]
    rng = np.random.default_rng(7)
    geos = [(1, 5, 8, 4, 4, 4, 0, 0), (1, 70, 12, 69, 8, 2, 3, 5), (3, 130, 16, 127, 6, 6, 0, 0),
            (2, 64, 5, 62, 12, 1, 0, 2), (1, 65, 128, 64, 32, 8, 0, 0), (1, 300, 64, 299, 12, 12, 0, 0)]
    for (sq, skv, d, p0, h, hkv, qpad, kvpad) in geos:
        qs, ks = h * d + qpad, hkv * d + kvpad
        q = rng.standard_normal(sq * qs).astype(np.float32)
        k = rng.standard_normal(skv * ks).astype(np.float32)
        v = rng.standard_normal(skv * ks).astype(np.float32)
        o = np.full(q.size, -1.0, np.float32)
        rt.sdpa_kv(q, k, v, o, sq, skv, d, p0, h, hkv, qs, ks, 1.0 / math.sqrt(d), True)
        assert_bits(o, orc.attention_kv(q, k, v, sq, skv, d, p0, h, hkv, qs, ks, 1.0 / math.sqrt(d), True)[1], "sdpa_kv")
    # batch with ragged lengths, padding full of NaN
    B, SQ, SKV, H, HKV, D = 5, 1, 200, 8, 2, 64
    q = rng.standard_normal(B * SQ * H * D).astype(np.float32)
    k = rng.standard_normal(B * SKV * HKV * D).astype(np.float32)
    v = rng.standard_normal(B * SKV * HKV * D).astype(np.float32)
    lens = np.array([200, 1, 0, 77, 64], np.int32)
    for b in range(B):
        k.reshape(B, SKV, -1)[b, lens[b]:] = np.nan
        v.reshape(B, SKV, -1)[b, lens[b]:] = np.nan
    o = np.full(q.size, -1.0, np.float32)
    rt.sdpa_kv_batch(q, k, v, o, lens, lens - 1, 0.125, True, B, SQ, SKV, H, HKV, D)
    assert_bits(o, orc.attention_kv_batch(q, k, v, lens, lens - 1, B, SQ, SKV, H, HKV, D, 0.125, True)[1], "batch")
    assert not np.isnan(o).any()
    with pytest.raises(Exception):
        rt.sdpa_kv_batch(q, k, v, o, lens + 1000, lens, 0.125, True, B, SQ, SKV, H, HKV, D)


def test_sdpa_rope_embedding_argmax(rt, orc, golden):
    o = np.zeros(4, np.float32)
    rt.sdpa(np.array([2, 3, 1, 4], np.float32), np.array([3, 1, 3, 1], np.float32), np.array([5, 7, 100, 200], np.float32), o, 2, 2, 1.0, 1)
    assert list(o) == [5.0, 7.0, 52.5, 103.5]
    rng = np.random.default_rng(8)
    q = rng.standard_normal((20, 16)).astype(np.float32); k = rng.standard_normal((20, 16)).astype(np.float32)
    v = rng.standard_normal((20, 16)).astype(np.float32); o = np.zeros((20, 16), np.float32)
    rt.sdpa(q, k, v, o, 20, 16, 0.25, 1)
    assert_bits(o.ravel(), orc.attention(q, k, v, 20, 16, 0.25, 1), "sdpa")
    x = rng.standard_normal((50, 128)).astype(np.float32)
    inv = (10000.0 ** (-np.arange(64) / 64.0)).astype(np.float32)
    out = np.empty_like(x)
    rt.rope(x, inv, out, 50, 64)
    assert_bits(out, orc.rope(x, inv), "rope")
    xg = np.array([[1, 2, 3, 4], [1, 2, 3, 4]], np.float32); og = np.empty_like(xg)
    rt.rope(xg, np.array([1.0, 0.5], np.float32), og, 2, 2)
    assert [int(np.float32(t) * np.float32(1000)) for t in og.ravel()] == [int(s) for s in golden["rope"]]
    w = rng.standard_normal((100, 24)).astype(np.float32)
    ids = np.array([3, 99, 0, 100, -1, 50], np.int32)
    out = np.full((6, 24), -1.0, np.float32)
    rt.embedding(out, w, ids, 6, 24, 100)
    assert_bits(out, orc.embedding(w, ids), "embedding")
    xs = rng.standard_normal((7, 50257)).astype(np.float32)
    xs[1, 0] = np.nan; xs[2, 5] = np.nan; xs[3, 100] = xs[3].max(); xs[3, 40000] = xs[3].max(); xs[4, :] = 2.0
    am = np.empty(7, np.int32)
    rt.rowargmax(xs, am, 7, 50257)
    assert list(am) == list(orc.rowargmax(xs))


def test_tiny_lm_tokens(rt, orc, golden):
    """The reference's toy decode loop through the C ABI: greedy tokens 6 3 0 7 4 1."""
    wk = np.zeros((12, 20), np.float32); wv = np.zeros((12, 20), np.float32); wq = np.zeros((24, 20), np.float32)
    for i in range(12):
        wk[i, 8 + i] = 1.0
        if i < 8: wv[i, i] = 1.0
        if i + 2 < 12: wq[i, 8 + i + 2] = 200.0
        if i + 3 < 12: wq[12 + i, 8 + i + 3] = 200.0
    wo = np.zeros((8, 24), np.float32)
    for c in range(8):
        wo[c, (c + 7) % 8] = 2.0; wo[c, 12 + (c + 7) % 8] = 1.0
    woq = np.zeros(272, np.uint8)
    rt.quantize_q8_0(wo.ravel(), woq, 24)
    wkb, wvb, wqb = (orc.to_bf16_bits(t.ravel()) for t in (wk, wv, wq))
    kc = np.zeros(144, np.float32); vc = np.zeros(144, np.float32)
    toks = [5, 2, 7] + [0] * 9
    out = []
    for p in range(8):
        h = np.zeros(20, np.float32); h[toks[p]] = 1.0; h[8 + p] = 1.0
        krow = np.zeros(12, np.float32); vrow = np.zeros(12, np.float32)
        rt.gemv_bf16(wkb, h, krow); rt.gemv_bf16(wvb, h, vrow)
        rt.kv_append(kc, krow, p, 12); rt.kv_append(vc, vrow, p, 12)
        if p >= 2:
            q = np.zeros(24, np.float32); att = np.zeros(24, np.float32); logits = np.zeros(8, np.float32)
            rt.gemv_bf16(wqb, h, q)
            rt.sdpa_kv(q, kc, vc, att, 1, p + 1, 12, p, 2, 1, 24, 12, 1.0, True)
            rt.gemv_q8_0(woq, att, logits)
            best = np.zeros(1, np.int32)
            rt.rowargmax(logits, best, 1, 8)
            out.append(int(best[0])); toks[p + 1] = int(best[0])
    assert out == [int(s) for s in golden["decode_tiny_lm"]]

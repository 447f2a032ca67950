"""ctypes binding of the CPU oracle (test infrastructure).

Every wrapper takes and returns numpy arrays and calls the `wko_*` export of the same name; see
`wk_oracle.h` for the reference file:line each one restates.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libwk_oracle.so")


def build(force=False):
    """Compile the oracle with its Makefile (gcc only)."""
    if force or not os.path.exists(_SO):
        subprocess.check_call(["make", "-s", "-C", _HERE])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _declare(_lib)
    return _lib


i64, f32, vp = C.c_int64, C.c_float, C.c_void_p


def _declare(L):
    for name in ("wko_exp1", "wko_log1", "wko_tanh1", "wko_gelu1", "wko_silu1", "wko_sigmoid1"):
        getattr(L, name).restype = f32
        getattr(L, name).argtypes = [f32]
    L.wko_sincos1.restype = f32
    L.wko_sincos1.argtypes = [f32, C.c_int]
    L.wko_f32_to_bf16_bits.restype = C.c_uint16
    L.wko_f32_to_bf16_bits.argtypes = [f32]
    L.wko_bf16_bits_to_f32.restype = f32
    L.wko_bf16_bits_to_f32.argtypes = [C.c_uint16]
    L.wko_f32_to_f16_bits.restype = C.c_uint16
    L.wko_f32_to_f16_bits.argtypes = [f32]
    L.wko_f16_bits_to_f32.restype = f32
    L.wko_f16_bits_to_f32.argtypes = [C.c_uint16]
    for n in ("wko_f32_to_f8e4m3", "wko_f32_to_f8e5m2"):
        getattr(L, n).restype = C.c_uint8
        getattr(L, n).argtypes = [f32]
    for n in ("wko_f8e4m3_to_f32", "wko_f8e5m2_to_f32"):
        getattr(L, n).restype = f32
        getattr(L, n).argtypes = [C.c_uint8]
    L.wko_select_kc.restype = i64
    L.wko_select_kc.argtypes = [i64]
    sig = {
        "wko_vmath_f32": (None, [vp, vp, i64, i64]),
        "wko_vmath2_f32": (None, [vp, vp, vp, i64, i64]),
        "wko_velem_f32": (None, [vp, vp, vp, i64, f32, f32, f32, i64]),
        "wko_norm_f32": (None, [vp, vp, i64, i64, i64, i64]),
        "wko_norm_affine_f32": (None, [vp, vp, vp, vp, i64, i64, i64, i64]),
        "wko_sgemm": (None, [vp, vp, vp, i64, i64, i64, i64]),
        "wko_sgemm_nt": (None, [vp, vp, vp, i64, i64, i64, i64]),
        "wko_sgemm_tn": (None, [vp, vp, vp, i64, i64, i64, i64]),
        "wko_sgemm_nt_epi": (None, [vp, vp, vp, i64, i64, i64, i64, vp, i64]),
        "wko_sgemm_nt_alpha": (None, [vp, vp, vp, i64, i64, i64, i64, f32]),
        "wko_sgemm_bf16_nt": (None, [vp, vp, vp, i64, i64, i64, i64]),
        "wko_sgemm_f16_nt": (None, [vp, vp, vp, i64, i64, i64, i64]),
        "wko_sgemm_bf16_nt_epi": (None, [vp, vp, vp, i64, i64, i64, i64, vp, i64]),
        "wko_sgemv": (None, [vp, vp, vp, i64, i64]),
        "wko_sgemv_alpha": (None, [vp, vp, vp, i64, i64, f32]),
        "wko_sgemv_bf16": (i64, [vp, i64, vp, i64, vp, i64]),
        "wko_sgemv_f16": (i64, [vp, i64, vp, i64, vp, i64]),
        "wko_quantize_q8_0_f32": (i64, [vp, i64, vp, i64, i64]),
        "wko_quantize_q4_0_f32": (i64, [vp, i64, vp, i64, i64]),
        "wko_gemv_q8_0_f32": (i64, [vp, i64, vp, i64, vp, i64]),
        "wko_gemv_q4_0_f32": (i64, [vp, i64, vp, i64, vp, i64]),
        "wko_gemv_q4_0_bf16x_f64": (i64, [vp, i64, vp, i64, vp, i64]),
        "wko_unpack_q4_0": (None, [vp, i64, vp, vp]),
        "wko_dequant_i4_f32": (i64, [vp, i64, vp, i64, i64, vp, i64]),
        "wko_dequant_u4_f32": (i64, [vp, i64, vp, i64, vp, i64, i64, vp, i64]),
        "wko_attention_kv_f32": (i64, [vp, i64, vp, i64, vp, i64, vp, i64] + [i64] * 8 + [f32, i64]),
        "wko_attention_kv_batch_f32": (i64, [vp, i64, vp, i64, vp, i64, vp, i64, vp, i64, vp, i64] + [i64] * 6 + [f32, i64]),
        "wko_kv_append_f32": (i64, [vp, i64, vp, i64, i64, i64]),
        "wko_attention_f32": (None, [vp, vp, vp, vp, i64, i64, f32, i64]),
        "wko_paged_attn_decode_f64": (i64, [vp, vp, vp, C.c_int, C.c_int, vp, vp, vp] + [i64] * 6 + [f32]),
        "wko_rope_f32": (None, [vp, vp, vp, i64, i64]),
        "wko_rope_pos_f32": (None, [vp, vp, vp, vp, i64, i64, i64]),
        "wko_embedding_f32": (None, [vp, vp, vp, i64, i64, i64]),
        "wko_rowargmax_i32": (None, [vp, vp, i64, i64]),
        "wko_philox4x32_10": (None, [vp, vp, vp]),
        "wko_rand_u32": (C.c_uint32, [C.c_uint64, C.c_uint64]),
        "wko_rand_fill_f32": (None, [vp, i64, i64, i64]),
        "wko_topk_f32": (i64, [vp, i64, vp, i64, vp, i64]),
        "wko_argsort_f32": (i64, [vp, i64, vp, i64, i64]),
        "wko_sample_categorical_f32": (i64, [vp, i64, C.c_float]),
        "wko_set_threads": (None, [C.c_int]),
        "wko_get_threads": (C.c_int, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args


def p(a):
    """Raw pointer of a numpy array (None -> NULL)."""
    return None if a is None else a.ctypes.data_as(vp)


def f32a(x):
    return np.ascontiguousarray(x, dtype=np.float32)


def eps_bits(eps):
    return int(np.float32(eps).view(np.uint32))


def set_threads(n):
    lib().wko_set_threads(int(n))


# ---- array-level conveniences used by the tests --------------------------------------------------

def vmath(x, op):
    x = f32a(x)
    out = np.empty_like(x)
    lib().wko_vmath_f32(p(x), p(out), x.size, op)
    return out


def vmath2(x, y, op):
    x, y = f32a(x), f32a(y)
    out = np.empty_like(x)
    lib().wko_vmath2_f32(p(x), p(y), p(out), x.size, op)
    return out


def velem(x, y, a, b, c, op):
    x = f32a(x)
    y = None if y is None else f32a(y)
    out = np.empty_like(x)
    lib().wko_velem_f32(p(x), p(y), p(out), x.size, a, b, c, op)
    return out


def norm(x, op, eps=0.0):
    x = f32a(x)
    rows, cols = x.shape
    out = np.empty_like(x)
    lib().wko_norm_f32(p(x), p(out), rows, cols, eps_bits(eps), op)
    return out


def norm_affine(x, gamma, beta, op, eps):
    x = f32a(x)
    rows, cols = x.shape
    g = None if gamma is None else f32a(gamma)
    b = None if beta is None else f32a(beta)
    out = np.empty_like(x)
    lib().wko_norm_affine_f32(p(x), p(out), p(g), p(b), rows, cols, eps_bits(eps), op)
    return out


def sgemm(a, b, m, k, n, kind="nn", beta=0, c=None, bias=None, act=None, alpha=None):
    a, b = f32a(a), f32a(b)
    c = np.zeros((m, n), np.float32) if c is None else f32a(c).copy()
    L = lib()
    if bias is not None or act is not None:
        bb = None if bias is None else f32a(bias)
        L.wko_sgemm_nt_epi(p(a), p(b), p(c), m, k, n, beta, p(bb), act or 0)
    elif alpha is not None:
        L.wko_sgemm_nt_alpha(p(a), p(b), p(c), m, k, n, beta, alpha)
    else:
        {"nn": L.wko_sgemm, "nt": L.wko_sgemm_nt, "tn": L.wko_sgemm_tn}[kind](p(a), p(b), p(c), m, k, n, beta)
    return c


def sgemm_half_nt(a_bits, b_bits, m, k, n, bf16=True, bias=None, act=None):
    a = np.ascontiguousarray(a_bits, np.uint16)
    b = np.ascontiguousarray(b_bits, np.uint16)
    c = np.zeros((m, n), np.float32)
    L = lib()
    if bias is not None or act is not None:
        assert bf16
        bb = None if bias is None else f32a(bias)
        L.wko_sgemm_bf16_nt_epi(p(a), p(b), p(c), m, k, n, 0, p(bb), act or 0)
    else:
        (L.wko_sgemm_bf16_nt if bf16 else L.wko_sgemm_f16_nt)(p(a), p(b), p(c), m, k, n, 0)
    return c


def sgemv(a, x, alpha=1.0):
    a, x = f32a(a), f32a(x)
    m, n = a.shape
    y = np.empty(m, np.float32)
    lib().wko_sgemv_alpha(p(a), p(x), p(y), m, n, alpha)
    return y


def sgemv_half(w_bits, x, n, bf16=True):
    w = np.ascontiguousarray(w_bits, np.uint16)
    x = f32a(x)
    y = np.full(n, 7.0, np.float32)
    fn = lib().wko_sgemv_bf16 if bf16 else lib().wko_sgemv_f16
    st = fn(p(w), w.size, p(x), x.size, p(y), n)
    return st, y


def quantize(x, k, q4=True):
    x = f32a(x).ravel()
    rows = x.size // k
    bb = 18 if q4 else 34
    q = np.zeros(rows * ((k + 31) // 32) * bb, np.uint8)
    fn = lib().wko_quantize_q4_0_f32 if q4 else lib().wko_quantize_q8_0_f32
    st = fn(p(x), x.size, p(q), q.size, k)
    assert st == 0, st
    return q


def gemv_q(w, x, n, q4=True):
    w = np.ascontiguousarray(w, np.uint8)
    x = f32a(x)
    y = np.full(n, 7.0, np.float32)
    fn = lib().wko_gemv_q4_0_f32 if q4 else lib().wko_gemv_q8_0_f32
    st = fn(p(w), w.size, p(x), x.size, p(y), n)
    return st, y


def gemv_q4_bf16x(w, x_bits, n):
    w = np.ascontiguousarray(w, np.uint8)
    xb = np.ascontiguousarray(x_bits, np.uint16)
    y = np.empty(n, np.float32)
    st = lib().wko_gemv_q4_0_bf16x_f64(p(w), w.size, p(xb), xb.size, p(y), n)
    assert st == 0
    return y


def unpack_q4_0(w):
    w = np.ascontiguousarray(w, np.uint8)
    nb = w.size // 18
    quants = np.empty(nb * 32, np.int8)
    scales = np.empty(nb, np.uint16)
    lib().wko_unpack_q4_0(p(w), nb, p(quants), p(scales))
    return quants, scales


def attention_kv_batch(q, k, v, kv_lens, q_pos, batch, sq, skv, h, hkv, d, scale, causal, o_init=-1.0):
    q, k, v = f32a(q), f32a(k), f32a(v)
    lens = np.ascontiguousarray(kv_lens, np.int32)
    pos = np.ascontiguousarray(q_pos, np.int32)
    o = np.full(q.size, o_init, np.float32)
    st = lib().wko_attention_kv_batch_f32(p(q), q.size, p(k), k.size, p(v), v.size, p(o), o.size, p(lens),
                                          lens.size, p(pos), pos.size, batch, sq, skv, h, hkv, d, scale,
                                          int(causal))
    return st, o


def attention_kv(q, k, v, sq, skv, d, q_pos0, h, hkv, q_stride, kv_stride, scale, causal, o_init=-1.0):
    q, k, v = f32a(q), f32a(k), f32a(v)
    o = np.full(q.size, o_init, np.float32)
    st = lib().wko_attention_kv_f32(p(q), q.size, p(k), k.size, p(v), v.size, p(o), o.size, sq, skv, d, q_pos0,
                                    h, hkv, q_stride, kv_stride, scale, int(causal))
    return st, o


def attention(q, k, v, s, d, scale, causal):
    q, k, v = f32a(q), f32a(k), f32a(v)
    o = np.zeros(s * d, np.float32)
    lib().wko_attention_f32(p(q), p(k), p(v), p(o), s, d, scale, int(causal))
    return o


def paged_attn_decode(q, kcache, vcache, kv_dtype, block_table, ctx_lens, slots, q_heads, kv_heads, hd, bs, mbps, scale,
                      layout=0):
    q = f32a(q)
    bt = np.ascontiguousarray(block_table, np.uint32)
    cl = np.ascontiguousarray(ctx_lens, np.int32)
    o = np.empty(slots * q_heads * hd, np.float32)
    st = lib().wko_paged_attn_decode_f64(p(q), p(kcache), p(vcache), kv_dtype, layout, p(bt), p(cl), p(o), slots, q_heads,
                                         kv_heads, hd, bs, mbps, scale)
    assert st == 0
    return o.reshape(slots, q_heads * hd)


def rope(x, inv_freq):
    x = f32a(x)
    rows, dim = x.shape
    inv = f32a(inv_freq)
    out = np.empty_like(x)
    lib().wko_rope_f32(p(x), p(inv), p(out), rows, dim // 2)
    return out


def rope_pos(x, inv_freq, pos, heads):
    x = f32a(x)
    rows = x.shape[0]
    inv = f32a(inv_freq)
    pv = np.ascontiguousarray(pos, np.int32)
    out = np.empty_like(x)
    lib().wko_rope_pos_f32(p(x), p(inv), p(pv), p(out), rows, heads, inv.size)
    return out


def embedding(weight, ids):
    w = f32a(weight)
    v, h = w.shape
    idv = np.ascontiguousarray(ids, np.int32)
    out = np.full((idv.size, h), -1.0, np.float32)
    lib().wko_embedding_f32(p(out), p(w), p(idv), idv.size, h, v)
    return out


def rowargmax(x):
    x = f32a(x)
    rows, cols = x.shape
    out = np.empty(rows, np.int32)
    lib().wko_rowargmax_i32(p(x), p(out), rows, cols)
    return out


def to_bf16_bits(x):
    """Round-to-nearest-even f32 -> bf16 bits with NaN quieting (vectorised restatement)."""
    x = f32a(x)
    bits = x.view(np.uint32)
    nan = np.isnan(x)
    bias = np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
    out = ((bits + bias) >> np.uint32(16)).astype(np.uint16)
    out[nan] = ((bits[nan] >> np.uint32(16)) | np.uint32(0x40)).astype(np.uint16)
    return out


def from_bf16_bits(b):
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def philox4x32_10(ctr4, key2):
    c, k, o = np.asarray(ctr4, np.uint32), np.asarray(key2, np.uint32), np.zeros(4, np.uint32)
    lib().wko_philox4x32_10(p(c), p(k), p(o))
    return o


def rand_u32(seed, ctr):
    return int(lib().wko_rand_u32(seed & 0xFFFFFFFFFFFFFFFF, ctr & 0xFFFFFFFFFFFFFFFF))


def rand_fill(n, seed, ctr0):
    out = np.full(max(n, 0), 7.0, np.float32)
    lib().wko_rand_fill_f32(p(out), n, seed, ctr0)
    return out


def topk(x, k):
    x = f32a(x).ravel()
    vals, idx = np.full(k, 9.0, np.float32), np.full(k, 9, np.int64)
    got = lib().wko_topk_f32(p(x), x.size, p(vals), k, p(idx), k)
    return int(got), vals, idx


def argsort(x, m, descending=False):
    x = f32a(x).ravel()
    idx = np.full(m, 9, np.int64)
    got = lib().wko_argsort_f32(p(x), x.size, p(idx), m, int(descending))
    return int(got), idx


def sample_categorical(w, u):
    w = f32a(w).ravel()
    return int(lib().wko_sample_categorical_f32(p(w) if w.size else None, w.size, float(u)))

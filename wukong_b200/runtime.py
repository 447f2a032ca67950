"""The language's tensor builtins over HOST buffers, through the reference's C ABI.

Function names, argument order and error behaviour follow the builtins of the reference
(crates/wukong_sema/src/builtins.rs:14-24, decode_builtins.rs:5-7,82-85): the checked builtins
raise when the kernel returns a non-zero status (the reference's lowering turns that into an assert
failure), and the empty-contraction fill of `matmul` / `linear` is done here as the lowering does it
(crates/wukong_mir_build/src/builtins.rs:738-766), because the kernels write nothing for K <= 0.
Every call runs on the GPU.
"""
import numpy as np

from ._lib import lib, vp, WukongB200Error

ACT = {"identity": 0, "relu": 1, "gelu": 2, "silu": 3}
VM = {"exp": 0, "log": 1, "tanh": 2, "sigmoid": 3, "relu": 4, "silu": 5, "gelu": 6, "sin": 15, "cos": 16}
NORM_SOFTMAX, NORM_LAYERNORM, NORM_RMSNORM, NORM_LOGSOFTMAX, NORM_L2 = range(5)


def _p(a):
    return None if a is None else a.ctypes.data_as(vp)


def _f32(a):
    a = np.asarray(a)
    if a.dtype != np.float32 or not a.flags["C_CONTIGUOUS"]:
        raise TypeError("builtin operands are contiguous f32 buffers")
    return a


def _status(code, name):
    if code != 0:
        raise WukongB200Error("%s: status %d (the reference asserts on a non-zero status)" % (name, code))


def eps_bits(eps):
    return int(np.float32(eps).view(np.uint32))


# ---- GEMM family -------------------------------------------------------------------------------
def matmul(a, b, c, m, k, n):
    if k <= 0:
        c.reshape(-1)[: m * n] = 0.0
        return
    lib().wukong_sgemm(_p(_f32(a)), _p(_f32(b)), _p(_f32(c)), m, k, n, 0)


def matmul_nt(a, b, c, m, k, n):
    if k <= 0:
        c.reshape(-1)[: m * n] = 0.0
        return
    lib().wukong_sgemm_nt(_p(_f32(a)), _p(_f32(b)), _p(_f32(c)), m, k, n, 0)


def matmul_tn(a, b, c, m, k, n):
    if k <= 0:
        c.reshape(-1)[: m * n] = 0.0
        return
    lib().wukong_sgemm_tn(_p(_f32(a)), _p(_f32(b)), _p(_f32(c)), m, k, n, 0)


def linear(x, w, bias, out, m, k, n, act="identity"):
    if k <= 0:
        out.reshape(m, n)[:] = 0.0 if bias is None else np.asarray(bias, np.float32)
        return
    lib().wukong_sgemm_nt_epi(_p(_f32(x)), _p(_f32(w)), _p(_f32(out)), m, k, n, 0,
                              _p(None if bias is None else _f32(bias)), ACT[act])


def gemv_bf16(w_bits, x, y):
    _status(lib().wukong_sgemv_bf16(_p(w_bits), w_bits.size, _p(_f32(x)), x.size, _p(_f32(y)), y.size), "gemv_bf16")


def gemv_f16(w_bits, x, y):
    _status(lib().wukong_sgemv_f16(_p(w_bits), w_bits.size, _p(_f32(x)), x.size, _p(_f32(y)), y.size), "gemv_f16")


def gemv(a, x, y, m, n, alpha=1.0):
    lib().wukong_sgemv_alpha(_p(_f32(a)), _p(_f32(x)), _p(_f32(y)), m, n, alpha)


# ---- quantised -----------------------------------------------------------------------------------
def quantize_q8_0(x, q, k):
    _status(lib().wukong_quantize_q8_0_f32(_p(_f32(x)), x.size, _p(q), q.size, k), "quantize_q8_0")


def quantize_q4_0(x, q, k):
    _status(lib().wukong_quantize_q4_0_f32(_p(_f32(x)), x.size, _p(q), q.size, k), "quantize_q4_0")


def gemv_q8_0(w, x, y):
    _status(lib().wukong_gemv_q8_0_f32(_p(w), w.size, _p(_f32(x)), x.size, _p(_f32(y)), y.size), "gemv_q8_0")


def gemv_q4_0(w, x, y):
    _status(lib().wukong_gemv_q4_0_f32(_p(w), w.size, _p(_f32(x)), x.size, _p(_f32(y)), y.size), "gemv_q4_0")


def dequant_i4(q, scale, group, out):
    _status(lib().wukong_dequant_i4_f32(_p(q), q.size, _p(_f32(scale)), scale.size, group, _p(_f32(out)), out.size),
            "dequant_i4")


def dequant_u4(q, scale, zero, group, out):
    _status(lib().wukong_dequant_u4_f32(_p(q), q.size, _p(_f32(scale)), scale.size, _p(_f32(zero)), zero.size, group,
                                        _p(_f32(out)), out.size), "dequant_u4")


# ---- elementwise and norms ----------------------------------------------------------------------
def _act(name):
    def f(x, out):
        lib().wukong_vmath_f32(_p(_f32(x)), _p(_f32(out)), x.size, VM[name])
    f.__name__ = name
    return f


exp, log, tanh, sigmoid, relu, silu, gelu = (_act(n) for n in ("exp", "log", "tanh", "sigmoid", "relu", "silu", "gelu"))


def silu_gate(a, b, out):
    lib().wukong_vmath2_f32(_p(_f32(a)), _p(_f32(b)), _p(_f32(out)), a.size, 9)


def hadamard(x, y, out):
    """out = x * y, the `VE_HADAMARD` form of wukong_velem_f32 (velem.rs:46)."""
    lib().wukong_velem_f32(_p(_f32(x)), _p(_f32(y)), _p(_f32(out)), x.size, 1.0, 1.0, 0.0, 512)


def residual_add(x, y, out):
    """out = x + y, the `VE_USE_Y` affine form with a = b = 1, c = 0 (velem.rs:44)."""
    lib().wukong_velem_f32(_p(_f32(x)), _p(_f32(y)), _p(_f32(out)), x.size, 1.0, 1.0, 0.0, 256)


def softmax(x, out, rows, cols):
    lib().wukong_norm_f32(_p(_f32(x)), _p(_f32(out)), rows, cols, 0, NORM_SOFTMAX)


def log_softmax(x, out, rows, cols):
    lib().wukong_norm_f32(_p(_f32(x)), _p(_f32(out)), rows, cols, 0, NORM_LOGSOFTMAX)


def layernorm(x, gamma, beta, out, rows, cols, eps):
    lib().wukong_norm_affine_f32(_p(_f32(x)), _p(_f32(out)), _p(gamma), _p(beta), rows, cols, eps_bits(eps), NORM_LAYERNORM)


def rmsnorm(x, gamma, out, rows, cols, eps):
    lib().wukong_norm_affine_f32(_p(_f32(x)), _p(_f32(out)), _p(gamma), None, rows, cols, eps_bits(eps), NORM_RMSNORM)


# ---- decode attention -----------------------------------------------------------------------------
def sdpa_kv(q, k, v, o, sq, skv, d, q_pos0, n_heads, n_kv_heads, q_stride, kv_stride, scale, causal):
    _status(lib().wukong_attention_kv_f32(_p(_f32(q)), q.size, _p(_f32(k)), k.size, _p(_f32(v)), v.size, _p(_f32(o)),
                                          o.size, sq, skv, d, q_pos0, n_heads, n_kv_heads, q_stride, kv_stride, scale,
                                          int(bool(causal))), "sdpa_kv")


def sdpa_kv_batch(q, k, v, o, kv_lens, q_pos, scale, causal, B, SQ, SKV, H, HKV, D):
    _status(lib().wukong_attention_kv_batch_f32(_p(_f32(q)), q.size, _p(_f32(k)), k.size, _p(_f32(v)), v.size,
                                                _p(_f32(o)), o.size, _p(kv_lens), kv_lens.size, _p(q_pos), q_pos.size,
                                                B, SQ, SKV, H, HKV, D, scale, int(bool(causal))), "sdpa_kv_batch")


def kv_append(cache, row, pos, stride):
    _status(lib().wukong_kv_append_f32(_p(_f32(cache)), cache.size, _p(_f32(row)), row.size, pos, stride), "kv_append")


def sdpa(q, k, v, out, s, d, scale, causal):
    lib().wukong_attention_f32(_p(_f32(q)), _p(_f32(k)), _p(_f32(v)), _p(_f32(out)), s, d, scale, int(causal))


def rope(x, inv_freq, out, rows, half):
    lib().wukong_rope_f32(_p(_f32(x)), _p(_f32(inv_freq)), _p(_f32(out)), rows, half)


def embedding(out, weight, ids, t, h, v):
    lib().wukong_embedding_f32(_p(_f32(out)), _p(_f32(weight)), _p(ids), t, h, v)


def rowargmax(x, out, rows, cols):
    lib().wukong_rowargmax_i32(_p(_f32(x)), _p(out), rows, cols)


# ---- selection / sampling / RNG builtins (topk_f32, argsort_f32, sample_categorical, rand_fill_f32) ----
def topk(x, vals, idx):
    """Writes the k = min(len(x), len(vals), len(idx)) largest elements (value, int64 index) in descending order; returns k."""
    return int(lib().wukong_topk_f32(_p(_f32(x)), x.size, _p(_f32(vals)), vals.size, _p(idx), idx.size))


def argsort(x, idx, descending=False):
    return int(lib().wukong_argsort_f32(_p(_f32(x)), x.size, _p(idx), idx.size, int(descending)))


def sample_categorical(p, u):
    p = _f32(p)
    return int(lib().wukong_sample_categorical_f32(_p(p) if p.size else None, p.size, float(u)))


def rand_fill(out, seed, ctr0):
    lib().wukong_rand_fill_f32(_p(_f32(out)), out.size, seed, ctr0)

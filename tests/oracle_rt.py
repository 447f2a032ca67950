"""The builtin namespace of `wukong_b200.runtime`, backed by the CPU oracle (test infrastructure):
lets one dispatch trace run once on the GPU library and once on the oracle."""
import numpy as np


class OracleRT:
    ACT = {"identity": 0, "relu": 1, "gelu": 2, "silu": 3}

    def __init__(self, orc):
        self.o = orc

    def layernorm(self, x, g, b, out, rows, cols, eps):
        out[:] = self.o.norm_affine(x.reshape(rows, cols), g, b, 1, eps).reshape(out.shape)

    def rmsnorm(self, x, g, out, rows, cols, eps):
        out[:] = self.o.norm_affine(x.reshape(rows, cols), g, None, 2, eps).reshape(out.shape)

    def linear(self, x, w, bias, out, m, k, n, act="identity"):
        out[:] = self.o.sgemm(x, w, m, k, n, bias=bias, act=self.ACT[act]).reshape(out.shape)

    def matmul_nt(self, a, b, c, m, k, n):
        c[:] = self.o.sgemm(a, b, m, k, n, "nt").reshape(c.shape)

    def kv_append(self, cache, row, pos, stride):
        st = self.o.lib().wko_kv_append_f32(self.o.p(cache), cache.size, self.o.p(np.ascontiguousarray(row)), row.size, pos, stride)
        assert st == 0

    def sdpa_kv_batch(self, q, k, v, o, kv_lens, q_pos, scale, causal, B, SQ, SKV, H, HKV, D):
        st, out = self.o.attention_kv_batch(q, k, v, kv_lens, q_pos, B, SQ, SKV, H, HKV, D, scale, causal)
        assert st == 0
        o[:] = out.reshape(o.shape)

    def exp(self, x, out):
        out[:] = self.o.vmath(x, 0).reshape(out.shape)

    def silu(self, x, out):
        out[:] = self.o.vmath(x, 5).reshape(out.shape)

    def hadamard(self, x, y, out):
        out[:] = self.o.velem(x, y, 1.0, 1.0, 0.0, 512).reshape(out.shape)

// Oracle (test infrastructure): decode attention over a KV cache, the square sdpa recurrence, the
// KV append, and an f64 paged-attention model.
// Follows crates/wukong_runtime/src/attention_kv.rs of the reference (plans :153-311, the portable
// twin :423-549, entries :922-1360), attention.rs (`attention_scalar` :158-215) and, for the paged
// model, crates/wukong_codegen_gpu/src/paged_attention.rs (`reference_decode_attn_gqa` :2047-2119)
// with the slab indexing of paged_kv.rs (`KvConfig::elem_offset` :139-151).
#include "oracle_internal.h"
#include <cmath>
#include <vector>

namespace wko {

static const size_t KV_BC = 64;

// attention_kv.rs:423-443.
static float dot_contract(const float* a, const float* b, size_t d, size_t dv) {
  float lane[8] = {};
  size_t t = 0;
  while (t < dv) {
    for (int l = 0; l < 8; ++l) lane[l] = fmaf(a[t + l], b[t + l], lane[l]);
    t += 8;
  }
  float tree = ((lane[0] + lane[1]) + (lane[2] + lane[3])) + ((lane[4] + lane[5]) + (lane[6] + lane[7]));
  if (t == d) return tree;
  float tail = 0.0f;
  while (t < d) { tail = fmaf(a[t], b[t], tail); ++t; }
  return tree + tail;
}
static inline float max_rule(float a, float b) { return a > b ? a : b; }

// attention_kv.rs:456-478.
static float row_max(const float* row, size_t n, float init) {
  size_t nv = n & ~(size_t)7;
  float best = init;
  if (nv) {
    float lane[8];
    for (auto& l : lane) l = init;
    for (size_t c = 0; c < nv; c += 8)
      for (int l = 0; l < 8; ++l) lane[l] = max_rule(lane[l], row[c + l]);
    float a[4] = {max_rule(lane[0], lane[4]), max_rule(lane[1], lane[5]), max_rule(lane[2], lane[6]),
                  max_rule(lane[3], lane[7])};
    best = max_rule(max_rule(a[0], a[2]), max_rule(a[1], a[3]));
  }
  for (size_t i = nv; i < n; ++i) best = max_rule(best, row[i]);
  return best;
}

// attention_kv.rs:481-503.
static float exp_row(float* row, size_t n, float mn) {
  size_t nv = n & ~(size_t)7;
  float sv[8] = {};
  for (size_t c = 0; c < nv; c += 8)
    for (int l = 0; l < 8; ++l) {
      float p = exp1(row[c + l] - mn);
      row[c + l] = p;
      sv[l] += p;
    }
  float rs = 0.0f;
  if (nv) {
    float s[4] = {sv[0] + sv[4], sv[1] + sv[5], sv[2] + sv[6], sv[3] + sv[7]};
    rs = (s[0] + s[1]) + (s[2] + s[3]);
  }
  for (size_t i = nv; i < n; ++i) {
    float p = exp1(row[i] - mn);
    row[i] = p;
    rs += p;
  }
  return rs;
}

// attention_kv.rs:511-549: one (row, head).
static void attend_row(const float* qv, const float* k, const float* v, size_t stride, size_t keys,
                       size_t d, float scale, float* out) {
  size_t dv = d & ~(size_t)7;
  float m = -INFINITY, l = 0.0f;
  std::vector<float> acc(d, 0.0f);
  float sc[KV_BC];
  size_t j0 = 0;
  while (j0 < keys) {
    size_t kb = keys - j0 < KV_BC ? keys - j0 : KV_BC;
    for (size_t jj = 0; jj < kb; ++jj) sc[jj] = dot_contract(qv, k + (j0 + jj) * stride, d, dv) * scale;
    float mn = row_max(sc, kb, m);
    float corr = (m == mn) ? 1.0f : exp1(m - mn);
    float sum = exp_row(sc, kb, mn);
    l = l * corr + sum;
    m = mn;
    for (size_t t = 0; t < d; ++t) {
      float a = acc[t] * corr;
      for (size_t jj = 0; jj < kb; ++jj) a = fmaf(sc[jj], v[(j0 + jj) * stride + t], a);
      acc[t] = a;
    }
    j0 += kb;
  }
  float inv = l != 0.0f ? 1.0f / l : 0.0f;
  for (size_t t = 0; t < d; ++t) out[t] = acc[t] * inv;
}

struct Walk {
  size_t batch, sq, d, n_heads, n_kv_heads, q_stride, kv_stride, q_bstride, kv_bstride;
};

// Number of leading keys row i sees (attention_kv.rs:139-146, :343-351).
static size_t visible(size_t len, __int128 pos, size_t i, bool causal) {
  if (!causal) return len;
  __int128 vis = pos + (__int128)i + 1;
  if (vis < 0) vis = 0;
  if (vis > (__int128)len) vis = (__int128)len;
  return (size_t)vis;
}

static void run_walk(const Walk& w, const float* q, const float* k, const float* v, float* o,
                     const std::vector<size_t>& lens, const std::vector<i64>& pos, float scale, bool causal) {
  size_t group = w.n_heads / w.n_kv_heads;
  i64 units = (i64)(w.batch * w.sq * w.n_heads);
  par_for(units, 1, [&](i64 lo, i64 hi) {
    for (i64 u = lo; u < hi; ++u) {
      size_t h = (size_t)u % w.n_heads;
      size_t i = ((size_t)u / w.n_heads) % w.sq;
      size_t b = (size_t)u / (w.n_heads * w.sq);
      size_t g = h / group;
      size_t keys = visible(lens[b], pos[b], i, causal);
      size_t qoff = b * w.q_bstride + i * w.q_stride + h * w.d;
      attend_row(q + qoff, k + b * w.kv_bstride + g * w.d, v + b * w.kv_bstride + g * w.d, w.kv_stride, keys,
                 w.d, scale, o + qoff);
    }
  });
}

}  // namespace wko

using namespace wko;

extern "C" {

// attention_kv.rs:153-203 (plan), :973-1046 (value semantics + entry).
i64 wko_attention_kv_f32(const float* q, i64 nq, const float* k, i64 nk, const float* v, i64 nv, float* o,
                         i64 no, i64 sq, i64 skv, i64 d, i64 q_pos0, i64 n_heads, i64 n_kv_heads,
                         i64 q_stride, i64 kv_stride, float scale, i64 causal) {
  i64 geo[8] = {sq, skv, d, q_pos0, n_heads, n_kv_heads, q_stride, kv_stride};
  for (i64 g : geo) if (g < 0) return -1;
  if (nq < 0 || nk < 0 || nv < 0 || no < 0) return -1;
  if (sq == 0 || n_heads == 0 || d == 0) return 0;
  if (n_kv_heads == 0 || n_heads % n_kv_heads != 0) return -1;
  __int128 q_row = (__int128)n_heads * d, kv_row = (__int128)n_kv_heads * d;
  if ((__int128)q_stride < q_row || (skv > 0 && (__int128)kv_stride < kv_row)) return -1;
  __int128 q_extent = ((__int128)sq - 1) * q_stride + q_row;
  __int128 kv_extent = skv == 0 ? 0 : ((__int128)skv - 1) * kv_stride + kv_row;
  if (q_extent > nq || q_extent > no || kv_extent > nk || kv_extent > nv) return -2;
  Walk w{1, (size_t)sq, (size_t)d, (size_t)n_heads, (size_t)n_kv_heads, (size_t)q_stride, (size_t)kv_stride,
         (size_t)q_extent, (size_t)kv_extent};
  // Value semantics: compute into scratch that starts as a copy of `o` (elements between heads stay
  // untouched), then copy back.
  std::vector<float> qc(q, q + (size_t)q_extent), kc(k, k + (size_t)kv_extent), vc(v, v + (size_t)kv_extent);
  std::vector<float> oc(o, o + (size_t)q_extent);
  run_walk(w, qc.data(), kc.data(), vc.data(), oc.data(), {(size_t)skv}, {q_pos0}, scale, causal != 0);
  // Only head lanes are written back.
  for (size_t i = 0; i < (size_t)sq; ++i)
    for (size_t e = 0; e < (size_t)q_row; ++e) o[i * (size_t)q_stride + e] = oc[i * (size_t)q_stride + e];
  return 0;
}

// attention_kv.rs:254-311 (plan + lens check), :1157-1250.
i64 wko_attention_kv_batch_f32(const float* q, i64 nq, const float* k, i64 nk, const float* v, i64 nv,
                               float* o, i64 no, const int32_t* kv_lens, i64 nl, const int32_t* q_pos,
                               i64 np, i64 batch, i64 sq, i64 skv, i64 n_heads, i64 n_kv_heads, i64 d,
                               float scale, i64 causal) {
  i64 geo[6] = {batch, sq, skv, n_heads, n_kv_heads, d};
  for (i64 g : geo) if (g < 0) return -1;
  if (nq < 0 || nk < 0 || nv < 0 || no < 0 || nl < 0 || np < 0) return -1;
  if (batch == 0 || sq == 0 || n_heads == 0 || d == 0) return 0;
  if (n_kv_heads == 0 || n_heads % n_kv_heads != 0) return -1;
  __int128 q_extent = (__int128)batch * sq * n_heads * d;
  __int128 kv_extent = (__int128)batch * skv * n_kv_heads * d;
  if (q_extent > nq || q_extent > no || kv_extent > nk || kv_extent > nv || batch > nl || batch > np) return -2;
  std::vector<size_t> lens((size_t)batch);
  std::vector<i64> pos((size_t)batch);
  for (i64 b = 0; b < batch; ++b) {
    if (kv_lens[b] < 0 || (i64)kv_lens[b] > skv) return -1;
    lens[(size_t)b] = (size_t)kv_lens[b];
    pos[(size_t)b] = q_pos[b];
  }
  size_t q_row = (size_t)(n_heads * d), kv_row = (size_t)(n_kv_heads * d);
  Walk w{(size_t)batch, (size_t)sq, (size_t)d, (size_t)n_heads, (size_t)n_kv_heads, q_row, kv_row,
         (size_t)sq * q_row, (size_t)skv * kv_row};
  std::vector<float> oc((size_t)q_extent);
  run_walk(w, q, k, v, oc.data(), lens, pos, scale, causal != 0);
  for (size_t i = 0; i < (size_t)q_extent; ++i) o[i] = oc[i];
  return 0;
}

// attention_kv.rs:1301-1360.
i64 wko_kv_append_f32(float* cache, i64 ncache, const float* row, i64 nrow, i64 pos, i64 stride) {
  if (ncache < 0 || nrow < 0 || pos < 0 || stride < 0) return -1;
  if (nrow == 0) return 0;
  if (stride < nrow) return -1;
  __int128 off = (__int128)pos * stride;
  if (off + nrow > (__int128)ncache) return -2;
  memmove(cache + (size_t)off, row, (size_t)nrow * 4);
  return 0;
}

// attention.rs:158-215: the per-key online softmax of the square single-head kernel.
void wko_attention_f32(const float* q, const float* k, const float* v, float* o, i64 s_, i64 d_, float scale,
                       i64 causal) {
  if (s_ <= 0 || d_ <= 0) return;
  size_t s = (size_t)s_, d = (size_t)d_;
  par_for((i64)s, 1, [&](i64 lo, i64 hi) {
    std::vector<float> acc(d);
    for (i64 ii = lo; ii < hi; ++ii) {
      size_t i = (size_t)ii;
      const float* qi = q + i * d;
      size_t jmax = causal ? i + 1 : s;
      float m = -INFINITY, l = 0.0f;
      for (auto& a : acc) a = 0.0f;
      for (size_t j = 0; j < jmax; ++j) {
        const float* kj = k + j * d;
        float x = 0.0f;
        for (size_t t = 0; t < d; ++t) x += qi[t] * kj[t];
        x *= scale;
        float mn = m > x ? m : x;
        float corr = (m == mn) ? 1.0f : exp1(m - mn);
        float p = exp1(x - mn);
        l = l * corr + p;
        const float* vj = v + j * d;
        for (size_t t = 0; t < d; ++t) acc[t] = acc[t] * corr + p * vj[t];
        m = mn;
      }
      float inv = l != 0.0f ? 1.0f / l : 0.0f;
      for (size_t t = 0; t < d; ++t) o[i * d + t] = acc[t] * inv;
    }
  });
}

// f64 full-softmax model of paged GQA decode attention.  Parity unpinned (property pinned).
i64 wko_paged_attn_decode_f64(const float* q, const void* kcache, const void* vcache, int kv_dtype, int layout,
                              const uint32_t* block_table, const int32_t* ctx_lens, float* o, i64 slots,
                              i64 q_heads, i64 kv_heads, i64 hd, i64 bs, i64 mbps, float scale) {
  if (slots < 0 || q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads || hd <= 0 || bs <= 0 || mbps < 0) return -1;
  auto load = [&](const void* base, size_t idx) -> double {
    if (kv_dtype == 0) return (double)((const float*)base)[idx];
    u16 b = ((const u16*)base)[idx];
    return (double)(kv_dtype == 1 ? bf16_bits_to_f32(b) : f16_bits_to_f32(b));
  };
  size_t group = (size_t)(q_heads / kv_heads), qd = (size_t)(q_heads * hd);
  par_for(slots * q_heads, 1, [&](i64 lo, i64 hi) {
    for (i64 u = lo; u < hi; ++u) {
      size_t b = (size_t)(u / q_heads), h = (size_t)(u % q_heads), kvh = h / group;
      size_t ctx = ctx_lens[b] > 0 ? (size_t)ctx_lens[b] : 0;
      float* out = o + b * qd + h * (size_t)hd;
      if (ctx == 0) { for (i64 t = 0; t < hd; ++t) out[t] = 0.0f; continue; }
      std::vector<double> sc(ctx);
      double mx = -INFINITY;
      auto off = [&](size_t t) {
        size_t phys = block_table[b * (size_t)mbps + t / (size_t)bs];
        if (layout == 1)  // [page][kv_head][token][dim]
          return ((phys * (size_t)kv_heads + kvh) * (size_t)bs + t % (size_t)bs) * (size_t)hd;
        return ((phys * (size_t)bs + t % (size_t)bs) * (size_t)kv_heads + kvh) * (size_t)hd;
      };
      for (size_t t = 0; t < ctx; ++t) {
        size_t base = off(t);
        double acc = 0.0;
        for (i64 e = 0; e < hd; ++e) acc += (double)q[b * qd + h * (size_t)hd + (size_t)e] * load(kcache, base + (size_t)e);
        sc[t] = acc * (double)scale;
        if (sc[t] > mx) mx = sc[t];
      }
      double denom = 0.0;
      for (size_t t = 0; t < ctx; ++t) { sc[t] = std::exp(sc[t] - mx); denom += sc[t]; }
      for (i64 e = 0; e < hd; ++e) {
        double acc = 0.0;
        for (size_t t = 0; t < ctx; ++t) acc += sc[t] * load(vcache, off(t) + (size_t)e);
        out[e] = (float)(acc / denom);
      }
    }
  });
  return 0;
}
}

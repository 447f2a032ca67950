// Test infrastructure: CPU restatement of the reference's selection / sampling / RNG kernels.
//   topk, argsort, sample_categorical : crates/wukong_runtime/src/topk.rs:22-136 (one strict total order:
//       descending = NaN largest, larger first, ties (-0.0 vs +0.0 and NaN vs NaN included) to the lower index;
//       ascending = smaller first, NaN last, ties to the lower index; categorical = inverse CDF over the positive
//       finite weights with the running mass summed in f64 in index order)
//   Philox4x32-10 and the (seed, counter) mapping of rand_u32 / rand_f32 / rand_fill : crates/wukong_runtime/
//       src/random.rs:24-104
// Because the order is total every result is unique, so a plain full sort of the indices is a valid restatement.
#include "wk_oracle.h"

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <vector>

namespace {

bool desc_before(const float* x, i64 a, i64 b) {
  const float xa = x[a], xb = x[b];
  const bool na = std::isnan(xa), nb = std::isnan(xb);
  if (na != nb) return na;                // NaN first
  if (!na && xa != xb) return xa > xb;    // -0.0 == +0.0 ties
  return a < b;
}
bool asc_before(const float* x, i64 a, i64 b) {
  const float xa = x[a], xb = x[b];
  const bool na = std::isnan(xa), nb = std::isnan(xb);
  if (na != nb) return nb;                // NaN last
  if (!na && xa != xb) return xa < xb;
  return a < b;
}
std::vector<i64> ranked_prefix(const float* x, i64 n, i64 m, bool descending) {
  std::vector<i64> idx((size_t)n);
  for (i64 i = 0; i < n; ++i) idx[(size_t)i] = i;
  if (descending) std::sort(idx.begin(), idx.end(), [&](i64 a, i64 b) { return desc_before(x, a, b); });
  else std::sort(idx.begin(), idx.end(), [&](i64 a, i64 b) { return asc_before(x, a, b); });
  idx.resize((size_t)m);
  return idx;
}

void philox_round(uint32_t (&c)[4], const uint32_t (&k)[2]) {
  const uint64_t p0 = (uint64_t)0xD2511F53u * c[0], p1 = (uint64_t)0xCD9E8D57u * c[2];
  const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k[0], n1 = (uint32_t)p1, n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k[1], n3 = (uint32_t)p0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

}  // namespace

extern "C" {

void wko_philox4x32_10(const uint32_t* ctr4, const uint32_t* key2, uint32_t* out4) {
  uint32_t c[4] = {ctr4[0], ctr4[1], ctr4[2], ctr4[3]}, k[2] = {key2[0], key2[1]};
  for (int r = 0; r < 10; ++r) {
    if (r > 0) { k[0] += 0x9E3779B9u; k[1] += 0xBB67AE85u; }
    philox_round(c, k);
  }
  for (int i = 0; i < 4; ++i) out4[i] = c[i];
}

uint32_t wko_rand_u32(uint64_t seed, uint64_t ctr) {
  const uint32_t c[4] = {(uint32_t)ctr, (uint32_t)(ctr >> 32), 0u, 0u}, k[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
  uint32_t o[4];
  wko_philox4x32_10(c, k, o);
  return o[0];
}

void wko_rand_fill_f32(float* out, i64 n, i64 seed, i64 ctr0) {
  for (i64 i = 0; i < n; ++i) out[i] = (float)(wko_rand_u32((uint64_t)seed, (uint64_t)ctr0 + (uint64_t)i) >> 8) * (1.0f / 16777216.0f);
}

i64 wko_topk_f32(const float* x, i64 n, float* vals, i64 nv, i64* idx, i64 ni) {
  if (n < 0) n = 0;
  const i64 k = std::min(n, std::min(nv < 0 ? 0 : nv, ni < 0 ? 0 : ni));
  std::vector<float> xs(x, x + n);   // outputs may overlap the input
  const std::vector<i64> order = ranked_prefix(xs.data(), n, k, true);
  for (i64 j = 0; j < k; ++j) { vals[j] = xs[(size_t)order[(size_t)j]]; idx[j] = order[(size_t)j]; }
  return k;
}

i64 wko_argsort_f32(const float* x, i64 n, i64* idx, i64 ni, i64 descending) {
  if (n < 0) n = 0;
  const i64 m = std::min(n, ni < 0 ? 0 : ni);
  std::vector<float> xs(x, x + n);
  const std::vector<i64> order = ranked_prefix(xs.data(), n, m, descending != 0);
  for (i64 j = 0; j < m; ++j) idx[j] = order[(size_t)j];
  return m;
}

i64 wko_sample_categorical_f32(const float* p, i64 n, float u) {
  auto mass = [](float w) -> double { return (w > 0.0f && std::isfinite(w)) ? (double)w : 0.0; };
  double total = 0.0;
  for (i64 i = 0; i < n; ++i) total += mass(p[i]);
  if (!(total > 0.0)) return -1;
  const float uc = std::isnan(u) ? 0.0f : std::min(1.0f, std::max(0.0f, u));
  const double target = (double)uc * total;
  double acc = 0.0;
  i64 last = -1;
  for (i64 i = 0; i < n; ++i) {
    const double m = mass(p[i]);
    if (m > 0.0) {
      acc += m;
      last = i;
      if (acc > target) return last;
    }
  }
  return last;
}

}  // extern "C"

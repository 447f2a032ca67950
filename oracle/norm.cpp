// Oracle (test infrastructure): row-wise softmax / log-softmax / LayerNorm / RMSNorm / L2-norm.
// Follows the scalar twins of crates/wukong_runtime/src/norm.rs of the reference: 8 accumulators
// of 8 lanes over 64-element blocks, a single-accumulator remainder, a lane tail, fixed trees.
#include "oracle_internal.h"
#include <cmath>

namespace wko {

// norm.rs:60-62.
static inline float hsum8(const float a[8]) {
  return ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
}
// Rust f32::max (maxNum): returns the non-NaN operand.
static inline float maxnum(float a, float b) {
  if (a != a) return b;
  if (b != b) return a;
  return a > b ? a : b;
}
// norm.rs:71-73.
static inline float hmax8(const float a[8]) {
  return maxnum(maxnum(maxnum(a[0], a[1]), maxnum(a[2], a[3])),
                maxnum(maxnum(a[4], a[5]), maxnum(a[6], a[7])));
}
// norm.rs:85-91.
static inline float maxps(float a, float b) { return a > b ? a : b; }

// norm.rs:132-147: halving tree (0,4)(1,5)(2,6)(3,7), (0,2)(1,3), (0,1).
static inline void combine8(float a[8][8]) {
  for (int w = 8; w > 1; w /= 2) {
    int h = w / 2;
    for (int t = 0; t < h; ++t)
      for (int j = 0; j < 8; ++j) a[t][j] += a[t + h][j];
  }
}

enum Red { SSQ, SUM, DEV2 };

// norm.rs:152-240 (ssq8_scalar / sum8_scalar / dev2_8_scalar share one block structure).
template <Red R>
static void reduce8(const float* x, size_t n, float mean, float out[8]) {
  float a[8][8] = {};
  size_t i = 0;
  auto step = [&](float& acc, float v) {
    if (R == SSQ) acc = fmaf(v, v, acc);
    else if (R == SUM) acc += v;
    else { float d = v - mean; acc = fmaf(d, d, acc); }
  };
  while (i + 64 <= n) {
    for (int t = 0; t < 8; ++t)
      for (int j = 0; j < 8; ++j) step(a[t][j], x[i + 8 * t + j]);
    i += 64;
  }
  while (i + 8 <= n) {
    for (int j = 0; j < 8; ++j) step(a[0][j], x[i + j]);
    i += 8;
  }
  combine8(a);
  for (int j = 0; j < 8; ++j) out[j] = a[0][j];
  for (size_t j = 0; j < n - i; ++j) step(out[j], x[i + j]);
}

// norm.rs:379-413.
static void rowmax8(const float* x, size_t n, float out[8]) {
  float a[8][8];
  for (auto& r : a) for (auto& v : r) v = -INFINITY;
  size_t i = 0;
  while (i + 64 <= n) {
    for (int t = 0; t < 8; ++t)
      for (int j = 0; j < 8; ++j) a[t][j] = maxps(a[t][j], x[i + 8 * t + j]);
    i += 64;
  }
  while (i + 8 <= n) {
    for (int j = 0; j < 8; ++j) a[0][j] = maxps(a[0][j], x[i + j]);
    i += 8;
  }
  for (int w = 8; w > 1; w /= 2) {
    int h = w / 2;
    for (int t = 0; t < h; ++t)
      for (int j = 0; j < 8; ++j) a[t][j] = maxps(a[t + h][j], a[t][j]);  // higher chain first
  }
  for (int j = 0; j < 8; ++j) out[j] = a[0][j];
  for (size_t j = 0; j < n - i; ++j) out[j] = maxnum(out[j], x[i + j]);
}

// norm.rs:466-490.
static void softmax_row(const float* x, float* out, size_t n) {
  float mx[8];
  rowmax8(x, n, mx);
  float m = hmax8(mx);
  size_t nb = n / 8, t = nb * 8;
  float sm[8] = {};
  for (size_t s = 0; s < nb; ++s)
    for (int j = 0; j < 8; ++j) {
      float e = exp1(x[s * 8 + j] - m);
      out[s * 8 + j] = e;
      sm[j] += e;
    }
  for (size_t j = 0; j < n - t; ++j) {
    float e = exp1(x[t + j] - m);
    out[t + j] = e;
    sm[j] += e;
  }
  float inv = 1.0f / hsum8(sm);
  for (size_t i = 0; i < n; ++i) out[i] *= inv;
}

// norm.rs:512-532.
static void logsoftmax_row(const float* x, float* out, size_t n) {
  float mx[8];
  rowmax8(x, n, mx);
  float m = hmax8(mx);
  size_t nb = n / 8, t = nb * 8;
  float sm[8] = {};
  for (size_t s = 0; s < nb; ++s)
    for (int j = 0; j < 8; ++j) sm[j] += exp1(x[s * 8 + j] - m);
  for (size_t j = 0; j < n - t; ++j) sm[j] += exp1(x[t + j] - m);
  float off = m + log1(hsum8(sm));
  for (size_t i = 0; i < n; ++i) out[i] = x[i] - off;
}

// norm.rs:538-576 (plain) and :757-796 (affine).  gamma/beta null => 1 / 0; `affine` selects the
// fma writeback of the affine entries.
static void norm_row(const float* x, float* out, const float* g, const float* b, size_t n, float eps,
                     i64 op, bool affine) {
  float acc[8];
  float invn = 1.0f / (float)n;
  float mean = 0.0f, inv;
  if (op == 1) {
    reduce8<SUM>(x, n, 0.0f, acc);
    mean = hsum8(acc) * invn;
    reduce8<DEV2>(x, n, mean, acc);
    inv = 1.0f / sqrtf(hsum8(acc) * invn + eps);
  } else if (op == 2) {
    reduce8<SSQ>(x, n, 0.0f, acc);
    inv = 1.0f / sqrtf(hsum8(acc) * invn + eps);
  } else {  // L2
    reduce8<SSQ>(x, n, 0.0f, acc);
    inv = 1.0f / sqrtf(hsum8(acc) + eps);
  }
  for (size_t i = 0; i < n; ++i) {
    float nv = (op == 1) ? (x[i] - mean) * inv : x[i] * inv;
    if (affine) {
      float gi = g ? g[i] : 1.0f, bi = b ? b[i] : 0.0f;
      out[i] = fmaf(nv, gi, bi);
    } else {
      out[i] = nv;
    }
  }
}

}  // namespace wko

using namespace wko;

extern "C" {
// norm.rs:991-1020.
void wko_norm_f32(const float* x, float* out, i64 rows, i64 cols, i64 eps_bits, i64 op) {
  if (rows <= 0 || cols <= 0) return;
  float eps = u2f((uint32_t)eps_bits);
  size_t n = (size_t)cols;
  par_for(rows, 1, [&](i64 lo, i64 hi) {
    for (i64 r = lo; r < hi; ++r) {
      const float* xr = x + (size_t)r * n;
      float* orow = out + (size_t)r * n;
      switch (op) {
        case 0: softmax_row(xr, orow, n); break;
        case 3: logsoftmax_row(xr, orow, n); break;
        case 1: case 2: case 4: norm_row(xr, orow, nullptr, nullptr, n, eps, op, false); break;
        default: break;  // unknown code: nothing written
      }
    }
  });
}

// norm.rs:1102-1150: only LAYERNORM / RMSNORM; any other code silently does nothing.
void wko_norm_affine_f32(const float* x, float* out, const float* gamma, const float* beta, i64 rows,
                         i64 cols, i64 eps_bits, i64 op) {
  if (rows <= 0 || cols <= 0) return;
  if (op != 1 && op != 2) return;
  float eps = u2f((uint32_t)eps_bits);
  size_t n = (size_t)cols;
  par_for(rows, 1, [&](i64 lo, i64 hi) {
    for (i64 r = lo; r < hi; ++r)
      norm_row(x + (size_t)r * n, out + (size_t)r * n, gamma, beta, n, eps, op, true);
  });
}
}

// Oracle (test infrastructure): GGML Q8_0 / Q4_0 block quantisation, the quantised GEMV, and
// group-wise int4 dequantisation.  Follows crates/wukong_runtime/src/quant.rs of the reference:
// packers :154-197, activation quantiser :201-212, `row_dot` :227-239, checked entries :408-480,
// group int4 :628-730.
#include "oracle_internal.h"
#include <cmath>
#include <vector>

namespace wko {

static const size_t QK = 32, Q8B = 34, Q4B = 18;

static inline float block_amax(const float* blk, size_t len) {
  float amax = 0.0f;
  for (size_t i = 0; i < len; ++i) {
    float a = fabsf(blk[i]);
    if (a > amax) amax = a;  // false for NaN
  }
  return amax;
}

// round half away from zero, clamp to [-127, 127], NaN -> 0 (Rust `as i8` saturates, NaN -> 0).
static inline int8_t q8_quant(float v) {
  if (v != v) return 0;
  float r = roundf(v);
  if (r < -127.0f) r = -127.0f;
  if (r > 127.0f) r = 127.0f;
  return (int8_t)r;
}

static void quantize_row_q8_0(const float* x, size_t len, u8* out, size_t nblocks) {
  for (size_t b = 0; b < nblocks; ++b) {
    u8* o = out + b * Q8B;
    size_t lo = b * QK < len ? b * QK : len;
    size_t bl = (lo + QK < len ? lo + QK : len) - lo;
    float d = block_amax(x + lo, bl) / 127.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    u16 h = f32_to_f16_bits(d);
    o[0] = (u8)(h & 0xff);
    o[1] = (u8)(h >> 8);
    for (size_t e = 0; e < QK; ++e) o[2 + e] = (u8)(e < bl ? q8_quant(x[lo + e] * id) : 0);
  }
}

static void quantize_row_q4_0(const float* x, size_t len, u8* out, size_t nblocks) {
  for (size_t b = 0; b < nblocks; ++b) {
    u8* o = out + b * Q4B;
    size_t lo = b * QK < len ? b * QK : len;
    size_t bl = (lo + QK < len ? lo + QK : len) - lo;
    float amax = 0.0f, mx = 0.0f;
    for (size_t i = 0; i < bl; ++i) {
      float v = x[lo + i];
      if (amax < fabsf(v)) { amax = fabsf(v); mx = v; }
    }
    float d = mx / -8.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    u16 h = f32_to_f16_bits(d);
    o[0] = (u8)(h & 0xff);
    o[1] = (u8)(h >> 8);
    auto nib = [&](size_t e) -> u8 {
      float v = (e < bl ? x[lo + e] : 0.0f) * id;
      if (v != v) return 8;
      float t = v + 8.5f;
      // Rust `as i8`: truncate toward zero, saturate.
      int iv = t >= 127.0f ? 127 : (t <= -128.0f ? -128 : (int)t);
      if (iv > 15) iv = 15;
      return (u8)(int8_t)iv;
    };
    for (size_t j = 0; j < QK / 2; ++j) o[2 + j] = (u8)(nib(j) | (nib(j + QK / 2) << 4));
  }
}

static inline int weight_quant(bool q4, const u8* qs, size_t e) {
  if (!q4) return (int)(int8_t)qs[e];
  u8 byte = qs[e % 16];
  int nibv = e < 16 ? (byte & 0x0F) : (byte >> 4);
  return nibv - 8;
}

static i64 need_bytes(i64 rows, i64 k, size_t bb, bool& ok) {
  __int128 v = (__int128)rows * (__int128)((k + 31) / 32) * (__int128)bb;
  ok = v <= (__int128)INT64_MAX;
  return (i64)v;
}

static i64 gemv_q(const u8* w, i64 nw, const float* x, i64 nx, float* y, i64 ny, bool q4) {
  if (nw < 0 || nx < 0 || ny < 0) return -2;
  size_t bb = q4 ? Q4B : Q8B;
  bool ok;
  i64 need = need_bytes(ny, nx, bb, ok);
  if (!ok || need != nw) return -2;
  size_t n = (size_t)ny, k = (size_t)nx;
  if (n == 0) return 0;
  if (k == 0) {
    for (size_t j = 0; j < n; ++j) y[j] = 0.0f;
    return 0;
  }
  size_t nb = (k + QK - 1) / QK;
  std::vector<int8_t> xq(nb * QK, 0);
  std::vector<float> dx(nb, 0.0f);
  for (size_t b = 0; b < nb; ++b) {  // quant.rs:201-212: exact f32 scale
    size_t lo = b * QK, bl = (lo + QK < k ? lo + QK : k) - lo;
    float d = block_amax(x + lo, bl) / 127.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    dx[b] = d;
    for (size_t e = 0; e < bl; ++e) xq[b * QK + e] = q8_quant(x[lo + e] * id);
  }
  size_t row_bytes = nb * bb;
  std::vector<float> out(n);
  par_for((i64)n, 8, [&](i64 lo, i64 hi) {
    for (i64 r = lo; r < hi; ++r) {
      const u8* wrow = w + (size_t)r * row_bytes;
      float acc = 0.0f;
      for (size_t b = 0; b < nb; ++b) {
        const u8* blk = wrow + b * bb;
        int isum = 0;
        for (size_t e = 0; e < QK; ++e) isum += weight_quant(q4, blk + 2, e) * (int)xq[b * QK + e];
        float dw = f16_bits_to_f32((u16)(blk[0] | (blk[1] << 8)));
        acc = acc + (dw * dx[b]) * (float)isum;  // two multiplies and one add, each rounded once
      }
      out[(size_t)r] = acc;
    }
  });
  for (size_t j = 0; j < n; ++j) y[j] = out[j];
  return 0;
}

static i64 quantize(const float* x, i64 nx, u8* q, i64 nq, i64 k, bool q4) {
  if (nx < 0 || nq < 0 || k <= 0) return -2;
  if (nx % k != 0) return -2;
  i64 rows = nx / k;
  size_t bb = q4 ? Q4B : Q8B;
  bool ok;
  i64 need = need_bytes(rows, k, bb, ok);
  if (!ok || need != nq) return -2;
  if (rows == 0) return 0;
  size_t nb = (size_t)(k + 31) / 32;
  std::vector<float> src(x, x + nx);  // value semantics
  for (i64 r = 0; r < rows; ++r) {
    if (q4) quantize_row_q4_0(src.data() + r * k, (size_t)k, q + (size_t)r * nb * bb, nb);
    else quantize_row_q8_0(src.data() + r * k, (size_t)k, q + (size_t)r * nb * bb, nb);
  }
  return 0;
}

// quant.rs:628-730.
static i64 dequant_int4(const u8* q, i64 nq, const float* scale, i64 ns, const float* zero, i64 nz,
                        i64 group, float* out, i64 nout) {
  if (nq < 0 || ns < 0 || nout < 0 || group < 1) return -2;
  uint64_t n = (uint64_t)nout, g = (uint64_t)group;
  uint64_t groups = (n + g - 1) / g;
  if ((uint64_t)nq != (n + 1) / 2 || (uint64_t)ns != groups || (nz >= 0 && (uint64_t)nz != groups)) return -2;
  if (n == 0) return 0;
  std::vector<float> tmp(n);
  for (uint64_t i = 0; i < n; ++i) {
    u8 b = q[i >> 1];
    u8 nibv = (i & 1) == 0 ? (b & 0x0f) : (b >> 4);
    float s = scale[i / g];
    if (nz < 0) {
      int8_t sv = (int8_t)(nibv << 4);
      sv = (int8_t)(sv >> 4);
      tmp[i] = (float)sv * s;
    } else {
      tmp[i] = ((float)nibv - zero[i / g]) * s;
    }
  }
  for (uint64_t i = 0; i < n; ++i) out[i] = tmp[i];
  return 0;
}

}  // namespace wko

using namespace wko;

extern "C" {
i64 wko_quantize_q8_0_f32(const float* x, i64 nx, u8* q, i64 nq, i64 k) { return quantize(x, nx, q, nq, k, false); }
i64 wko_quantize_q4_0_f32(const float* x, i64 nx, u8* q, i64 nq, i64 k) { return quantize(x, nx, q, nq, k, true); }
i64 wko_gemv_q8_0_f32(const u8* w, i64 nw, const float* x, i64 nx, float* y, i64 ny) {
  return gemv_q(w, nw, x, nx, y, ny, false);
}
i64 wko_gemv_q4_0_f32(const u8* w, i64 nw, const float* x, i64 nx, float* y, i64 ny) {
  return gemv_q(w, nw, x, nx, y, ny, true);
}
i64 wko_dequant_i4_f32(const u8* q, i64 nq, const float* scale, i64 ns, i64 group, float* out, i64 nout) {
  return dequant_int4(q, nq, scale, ns, nullptr, -1, group, out, nout);
}
i64 wko_dequant_u4_f32(const u8* q, i64 nq, const float* scale, i64 ns, const float* zero, i64 nz, i64 group,
                       float* out, i64 nout) {
  if (nz < 0) return -2;
  return dequant_int4(q, nq, scale, ns, zero, nz, group, out, nout);
}

// Decode every Q4_0 block: 32 signed quants in element order (byte j -> element j low nibble,
// element j+16 high nibble; quant.rs:13-16, :215-223) and the raw f16 scale bits.
void wko_unpack_q4_0(const u8* w, i64 nblocks, int8_t* quants, u16* scale_bits) {
  for (i64 b = 0; b < nblocks; ++b) {
    const u8* blk = w + (size_t)b * Q4B;
    scale_bits[b] = (u16)(blk[0] | (blk[1] << 8));
    for (size_t e = 0; e < QK; ++e) quants[(size_t)b * QK + e] = (int8_t)weight_quant(true, blk + 2, e);
  }
}

// The in-register-dequant GEMV with bf16 activations: defining formula in f64.
i64 wko_gemv_q4_0_bf16x_f64(const u8* w, i64 nw, const u16* xb, i64 nx, float* y, i64 ny) {
  if (nw < 0 || nx < 0 || ny < 0) return -2;
  bool ok;
  i64 need = need_bytes(ny, nx, Q4B, ok);
  if (!ok || need != nw) return -2;
  size_t n = (size_t)ny, k = (size_t)nx, nb = (k + QK - 1) / QK;
  par_for((i64)n, 8, [&](i64 lo, i64 hi) {
    for (i64 r = lo; r < hi; ++r) {
      const u8* wrow = w + (size_t)r * nb * Q4B;
      double acc = 0.0;
      for (size_t b = 0; b < nb; ++b) {
        const u8* blk = wrow + b * Q4B;
        double d = (double)f16_bits_to_f32((u16)(blk[0] | (blk[1] << 8)));
        double s = 0.0;
        for (size_t e = 0; e < QK && b * QK + e < k; ++e)
          s += (double)weight_quant(true, blk + 2, e) * (double)bf16_bits_to_f32(xb[b * QK + e]);
        acc += d * s;
      }
      y[(size_t)r] = (float)acc;
    }
  });
  return 0;
}
}

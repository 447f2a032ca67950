// Oracle (test infrastructure): scalar transcendental and elementwise kernels.
// Follows crates/wukong_runtime/src/vmath.rs (scalar twins) and velem.rs of the reference.
#include "wk_oracle.h"
#include "oracle_internal.h"
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace wko {

// vmath.rs:139-146 (Cephes constants) and :176-202 (8-bucket exp table).
static const float EXP_MAGIC = 12582912.0f;
static const float EXP_C1 = 0.6933594f;
static const float EXP_C2 = -2.1219444e-4f;
static const float EXP_HI = 88.37626f;
static const float EXP_LO = -88.37626f;
static const float INV_2P23 = 1.0f / 8388608.0f;
static const float EXP_TBL_SCALE = (float)(8.0 / 0.693147180559945309417232121458176568);
static const float EXP_TBL_C1 = EXP_C1 / 8.0f;
static const float EXP_TBL_C2 = EXP_C2 / 8.0f;
static const int32_t EXP_TBL_MBIAS = 0x4B400000 - 1016;
static const float EXP_TBL_T[8] = {1.0f,       1.0905077f, 1.1892071f, 1.2968396f,
                                   1.4142135f, 1.5422108f, 1.6817929f, 1.8340081f};
static const float EXP_TBL_P2 = 0.5000648f;
static const float EXP_TBL_P3 = 1.0f / 6.0f;

// vmath.rs:321-356.
float exp1(float x) {
  uint32_t bits = f2u(x);
  uint32_t mag = bits & 0x7fffffffu;
  if (mag > 0x7f800000u) return u2f(bits | 0x00400000u);
  if (mag == 0x7f800000u) return bits == 0x7f800000u ? x : 0.0f;
  x = x < EXP_HI ? x : EXP_HI;  // min then max, the vector order
  x = x > EXP_LO ? x : EXP_LO;
  float t = fmaf(x, EXP_TBL_SCALE, EXP_MAGIC);
  float n = t - EXP_MAGIC;
  int32_t m = (int32_t)(f2u(t) - (uint32_t)EXP_TBL_MBIAS);
  float r = fmaf(n, -EXP_TBL_C1, x);
  r = fmaf(n, -EXP_TBL_C2, r);
  float tj = EXP_TBL_T[m & 7];
  float q = fmaf(r, EXP_TBL_P3, EXP_TBL_P2);
  q = fmaf(r, q, 1.0f);
  float p = fmaf(r, q, 1.0f);
  int32_t mm = m > 0 ? m : 0;
  float pow2 = u2f(((uint32_t)(mm >> 3)) << 23);
  return (tj * p) * pow2;
}

// vmath.rs:220-249 (tables), :369-420.
static const int32_t LOG_OFF = 0x3F320000;
static const float LOG_TBL_R[8] = {1.3763441f, 1.2673267f, 1.1743119f, 1.0940171f,
                                   1.0f,       0.92753625f, 0.83116883f, 0.7529412f};
static const float LOG_TBL_L[8] = {-0.31943077f, -0.23690973f, -0.16068234f, -0.08985638f,
                                   0.0f,         0.0752234f,   0.18492234f,  0.28376815f};
static const float LOG_C1 = -0.5f, LOG_C2 = 0.33333334f, LOG_C3 = -0.25f, LOG_C4 = 0.2f;

float log1(float x) {
  uint32_t ob = f2u(x);
  uint32_t mag = ob & 0x7fffffffu;
  if (mag > 0x7f800000u) return u2f(ob | 0x00400000u);
  if (mag == 0) return -INFINITY;
  if (ob & 0x80000000u) return NAN;
  if (mag == 0x7f800000u) return INFINITY;
  bool sub = mag < 0x00800000u;
  if (sub) x = x * 8388608.0f;
  int32_t bits = (int32_t)f2u(x);
  int32_t tmp = (int32_t)((uint32_t)bits - (uint32_t)LOG_OFF);
  int32_t kbits = tmp & (int32_t)0xFF800000u;
  int32_t iz = (int32_t)((uint32_t)bits - (uint32_t)kbits);
  float z = u2f((uint32_t)iz);
  float e = ((float)kbits) * INV_2P23 - (sub ? 23.0f : 0.0f);
  int j = (int)((((uint32_t)tmp) >> 20) & 7);
  float r = LOG_TBL_R[j], l = LOG_TBL_L[j];
  float s = fmaf(z, r, -1.0f);
  float w = s * s;
  float q0 = fmaf(LOG_C2, s, LOG_C1);
  float q1 = fmaf(LOG_C4, s, LOG_C3);
  float p = fmaf(q1, w, q0);
  p = p * w;
  float t = l + p;
  float y = fmaf(e, EXP_C2, t);
  float r2 = s + y;
  return fmaf(e, EXP_C1, r2);
}

// vmath.rs:429-431: the exp-composed tanh used inside gelu.
static inline float tanh_exp1(float x) { return 1.0f - 2.0f / (exp1(2.0f * x) + 1.0f); }

// vmath.rs:474-496 (constants), :504-546.
static const float TANH_XC = 0.75f, TANH_EXP_CLAMP = 10.0f;
static const float TANH_P[6] = {-0.33333316f, 0.13332695f,   -0.053892724f,
                                0.021452034f, -0.0076572555f, 0.0017369358f};
static const int32_t TANH_EXP_MBIAS = 0x4B400000 - 1020;
static const float TANH_EXP_Q3 = 1.0f / 6.0f, TANH_EXP_Q4 = 1.0f / 24.0f;

float tanh1(float x) {
  const float T[8] = {EXP_TBL_T[4] * 0.5f, EXP_TBL_T[5] * 0.5f, EXP_TBL_T[6] * 0.5f, EXP_TBL_T[7] * 0.5f,
                      EXP_TBL_T[0],        EXP_TBL_T[1],        EXP_TBL_T[2],        EXP_TBL_T[3]};
  uint32_t sgn = f2u(x) & 0x80000000u;
  float ax = u2f(f2u(x) & 0x7fffffffu);
  float t = ax * ax;
  float p = fmaf(t, TANH_P[5], TANH_P[4]);
  p = fmaf(t, p, TANH_P[3]);
  p = fmaf(t, p, TANH_P[2]);
  p = fmaf(t, p, TANH_P[1]);
  p = fmaf(t, p, TANH_P[0]);
  float w = ax * t;
  float y_poly = fmaf(w, p, ax);
  // Rust's f32::min returns the non-NaN operand; on the NaN path the polynomial side is taken.
  float axc = (ax != ax) ? TANH_EXP_CLAMP : (ax < TANH_EXP_CLAMP ? ax : TANH_EXP_CLAMP);
  float x2 = axc + axc;
  float tt = fmaf(x2, EXP_TBL_SCALE, EXP_MAGIC);
  float n = tt - EXP_MAGIC;
  int32_t m = (int32_t)(f2u(tt) - (uint32_t)TANH_EXP_MBIAS);
  float r = fmaf(n, -EXP_TBL_C1, x2);
  r = fmaf(n, -EXP_TBL_C2, r);
  float tj = T[m & 7];
  float q = fmaf(r, TANH_EXP_Q4, TANH_EXP_Q3);
  q = fmaf(r, q, 0.5f);
  q = fmaf(r, q, 1.0f);
  float pm1 = r * q;
  float mm = fmaf(tj, pm1, tj);
  float pow2 = u2f(((uint32_t)(m >> 3)) << 23);
  float d = fmaf(mm, pow2, 1.0f);
  float rr = 1.0f / d;
  float y_exp = fmaf(-2.0f, rr, 1.0f);
  float y = ax > TANH_XC ? y_exp : y_poly;
  return u2f((f2u(y) & 0x7fffffffu) | sgn);
}

// vmath.rs:549-582.
float sigmoid1(float x) { return 1.0f / (1.0f + exp1(-x)); }
float silu1(float x) {
  if (x != x) return u2f(f2u(x) | 0x00400000u);
  return x * sigmoid1(x);
}
static const float GELU_C0 = 0.7978846f, GELU_C1 = 0.044715f;
float gelu1(float x) {
  float x3 = x * x * x;
  float inner = GELU_C0 * fmaf(GELU_C1, x3, x);
  return (0.5f * x) * (1.0f + tanh_exp1(inner));
}

// vmath.rs:255-275 (constants), :706-760.
static const float TWO_OVER_PI = (float)0.636619772367581343075535053490057448;
static const float PIO2_1 = (float)1.5703125, PIO2_2 = (float)4.837512969970703e-4,
                   PIO2_3 = (float)7.54978995489188e-8;
static const float TRIG_FAST_LIMIT = 4096.0f;
static const float SIN_P[3] = {(float)-1.9515295891e-4, (float)8.3321608736e-3, (float)-1.6666654611e-1};
static const float COS_P[3] = {(float)2.443315711809948e-5, (float)-1.388731625493765e-3,
                               (float)4.166664568298827e-2};

float sincos1(float x, bool is_cos) {
  if (!std::isfinite(x)) return (x != x) ? u2f(f2u(x) | 0x00400000u) : NAN;
  if (fabsf(x) >= TRIG_FAST_LIMIT) return is_cos ? cosf(x) : sinf(x);
  if (x == 0.0f) return is_cos ? 1.0f : x;
  float tt = fmaf(x, TWO_OVER_PI, EXP_MAGIC);
  float qf = tt - EXP_MAGIC;
  float r = fmaf(qf, -PIO2_1, x);
  r = fmaf(qf, -PIO2_2, r);
  r = fmaf(qf, -PIO2_3, r);
  float z = r * r;
  float s = SIN_P[0];
  s = fmaf(s, z, SIN_P[1]);
  s = fmaf(s, z, SIN_P[2]);
  float sz = s * z;
  float sin_p = fmaf(sz, r, r);
  float c = COS_P[0];
  c = fmaf(c, z, COS_P[1]);
  c = fmaf(c, z, COS_P[2]);
  float z2 = z * z;
  float cz2 = c * z2;
  float hz = fmaf(-0.5f, z, 1.0f);
  float cos_p = hz + cz2;
  float quad = (float)(((int32_t)qf) & 3);
  float neg_sin = sin_p * -1.0f, neg_cos = cos_p * -1.0f;
  float a0, a1, a2, a3;
  if (is_cos) { a0 = cos_p; a1 = neg_sin; a2 = neg_cos; a3 = sin_p; }
  else        { a0 = sin_p; a1 = cos_p;  a2 = neg_sin; a3 = neg_cos; }
  float sel23 = quad == 2.0f ? a2 : a3;
  float sel123 = quad == 1.0f ? a1 : sel23;
  return quad == 0.0f ? a0 : sel123;
}

[[noreturn]] void unsupported(const char* what, i64 code) {
  fprintf(stderr, "wk_oracle: %s code %lld is outside the restated hot path\n", what, (long long)code);
  abort();
}

// vmath.rs:1000-1046 (apply1), restricted to the codes the decode path uses.
float apply1(i64 op, float x) {
  switch (op) {
    case 0: return exp1(x);
    case 1: return log1(x);
    case 2: return tanh1(x);
    case 3: return sigmoid1(x);
    case 4: return x > 0.0f ? x : 0.0f;
    case 5: return silu1(x);
    case 6: return gelu1(x);
    case 15: return sincos1(x, false);
    case 16: return sincos1(x, true);
    default: unsupported("vmath op", op);
  }
}

}  // namespace wko

using namespace wko;

extern "C" {
float wko_exp1(float x) { return exp1(x); }
float wko_log1(float x) { return log1(x); }
float wko_tanh1(float x) { return tanh1(x); }
float wko_gelu1(float x) { return gelu1(x); }
float wko_silu1(float x) { return silu1(x); }
float wko_sigmoid1(float x) { return sigmoid1(x); }
float wko_sincos1(float x, int is_cos) { return sincos1(x, is_cos != 0); }

// vmath.rs:1063-1090: out[i] = f(x[i]); in place allowed.
void wko_vmath_f32(const float* x, float* out, i64 n, i64 op) {
  if (n <= 0) return;
  par_for(n, 16384, [&](i64 lo, i64 hi) {
    for (i64 i = lo; i < hi; ++i) out[i] = apply1(op, x[i]);
  });
}

// vmath.rs:1506-1512, :2022-2050: gated forms out = act(a) * b.
void wko_vmath2_f32(const float* x, const float* y, float* out, i64 n, i64 op) {
  if (n <= 0) return;
  par_for(n, 16384, [&](i64 lo, i64 hi) {
    for (i64 i = lo; i < hi; ++i) {
      float a = x[i], b = y[i];
      switch (op) {
        case 9: out[i] = silu1(a) * b; break;
        case 10: out[i] = gelu1(a) * b; break;
        case 11: out[i] = sigmoid1(a) * b; break;
        default: unsupported("vmath2 op", op);
      }
    }
  });
}

// velem.rs:39-53 (codes), :134-168 (act1, elem1), :212-236 (entry).
void wko_velem_f32(const float* x, const float* y, float* out, i64 n, float a, float b, float c, i64 op) {
  if (n <= 0) return;
  const i64 USE_Y = 256, HAD = 512, DIV = 1024;
  par_for(n, 8192, [&](i64 lo, i64 hi) {
    for (i64 i = lo; i < hi; ++i) {
      float base;
      if (op & HAD) base = x[i] * y[i];
      else if (op & DIV) base = x[i] / y[i];
      else if (!(op & USE_Y) && a == 1.0f && c == 0.0f) base = x[i];
      else {
        float inner = (op & USE_Y) ? fmaf(b, y[i], c) : c;
        base = fmaf(a, x[i], inner);
      }
      switch (op & 0xff) {
        case 1: base = base > 0.0f ? base : 0.0f; break;
        case 2: base = base > 0.0f ? base : 0.0f; base = base < 6.0f ? base : 6.0f; break;
        default: break;
      }
      out[i] = base;
    }
  });
}
}

// Shared device helpers for the sm_100a kernels: correctly-rounded float primitives that the
// compiler can never contract or reorder, the scalar transcendental sequences of the runtime ABI
// (same operation order as crates/wukong_runtime/src/vmath.rs of the reference, so fp32 results
// are bit-identical to its CPU kernels), half-precision codecs and launch utilities.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

typedef int64_t i64;
typedef uint8_t u8;
typedef uint16_t u16;

#define WKB_SM_COUNT 148

// Codes of the library's device status word beyond the pipeline-wait codes of the tensor-core kernels (read and cleared
// by wkb_gemm_status): a KV append met a position past its block-table row (the row was skipped, nothing written).
#define WKB_STATUS_KV_POS_RANGE 31
// ... or a bounded wait on an asynchronous K/V copy of the paged attention ran out (the unit's output was not written).
#define WKB_STATUS_ATTN_WAIT 41

// Fatal-error policy of the `void` entry points: the runtime ABI has no status to return there, and
// a kernel library that silently computes nothing is worse than one that stops (the reference's own
// entries abort rather than unwind).  Checked entries return their status instead.
#define WKB_CUDA_CHECK(expr)                                                                      \
  do {                                                                                            \
    cudaError_t _e = (expr);                                                                      \
    if (_e != cudaSuccess) {                                                                      \
      fprintf(stderr, "wukong_b200: CUDA error %s at %s:%d: %s\n", cudaGetErrorName(_e), __FILE__, \
              __LINE__, cudaGetErrorString(_e));                                                  \
      abort();                                                                                    \
    }                                                                                             \
  } while (0)

namespace wkb {

__device__ __forceinline__ float fmul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float fadd(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float fsub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float ffma(float a, float b, float c) { return __fmaf_rn(a, b, c); }
__device__ __forceinline__ float fdiv(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float fsqrt(float a) { return __fsqrt_rn(a); }
__device__ __forceinline__ uint32_t f2u(float x) { return __float_as_uint(x); }
__device__ __forceinline__ float u2f(uint32_t u) { return __uint_as_float(u); }

// MAXPS rule: the first operand only when strictly greater (NaN in `b` wins, NaN in `a` is dropped).
__device__ __forceinline__ float maxps(float a, float b) { return a > b ? a : b; }
// maxNum: the non-NaN operand.
__device__ __forceinline__ float maxnum(float a, float b) {
  if (a != a) return b;
  if (b != b) return a;
  return a > b ? a : b;
}

// ---- exp: 8-bucket table reduction (vmath.rs:176-202, :321-356) ----
// 2^(j/8) rounded once to f32.
static __constant__ float c_exp_tbl[8] = {1.0f,       1.0905077f, 1.1892071f, 1.2968396f,
                                          1.4142135f, 1.5422108f, 1.6817929f, 1.8340081f};
static __constant__ float c_log_r[8] = {1.3763441f, 1.2673267f,  1.1743119f,  1.0940171f,
                                        1.0f,       0.92753625f, 0.83116883f, 0.7529412f};
static __constant__ float c_log_l[8] = {-0.31943077f, -0.23690973f, -0.16068234f, -0.08985638f,
                                        0.0f,         0.0752234f,   0.18492234f,  0.28376815f};
__device__ __forceinline__ float exp_tbl(int j) { return c_exp_tbl[j]; }
#define WKB_EXP_MAGIC 12582912.0f
#define WKB_EXP_C1 0.6933594f
#define WKB_EXP_C2 (-2.1219444e-4f)
#define WKB_EXP_TBL_SCALE 11.541560327111707f /* (f32)(8/ln2) */
#define WKB_EXP_TBL_C1 (0.6933594f / 8.0f)
#define WKB_EXP_TBL_C2 (-2.1219444e-4f / 8.0f)

__device__ __forceinline__ float exp1(float x) {
  uint32_t bits = f2u(x), mag = bits & 0x7fffffffu;
  if (mag > 0x7f800000u) return u2f(bits | 0x00400000u);
  if (mag == 0x7f800000u) return bits == 0x7f800000u ? x : 0.0f;
  x = x < 88.37626f ? x : 88.37626f;
  x = x > -88.37626f ? x : -88.37626f;
  float t = ffma(x, WKB_EXP_TBL_SCALE, WKB_EXP_MAGIC);
  float n = fsub(t, WKB_EXP_MAGIC);
  int32_t m = (int32_t)(f2u(t) - (uint32_t)(0x4B400000 - 1016));
  float r = ffma(n, -WKB_EXP_TBL_C1, x);
  r = ffma(n, -WKB_EXP_TBL_C2, r);
  float tj = exp_tbl(m & 7);
  float q = ffma(r, 1.0f / 6.0f, 0.5000648f);
  q = ffma(r, q, 1.0f);
  float p = ffma(r, q, 1.0f);
  int32_t mm = m > 0 ? m : 0;
  float pow2 = u2f(((uint32_t)(mm >> 3)) << 23);
  return fmul(fmul(tj, p), pow2);
}

// ---- log (vmath.rs:220-249, :369-420) ----
__device__ __forceinline__ float log1(float x) {
  uint32_t ob = f2u(x), mag = ob & 0x7fffffffu;
  if (mag > 0x7f800000u) return u2f(ob | 0x00400000u);
  if (mag == 0) return -INFINITY;
  if (ob & 0x80000000u) return u2f(0x7fc00000u);
  if (mag == 0x7f800000u) return INFINITY;
  bool sub = mag < 0x00800000u;
  if (sub) x = fmul(x, 8388608.0f);
  int32_t bits = (int32_t)f2u(x);
  int32_t tmp = (int32_t)((uint32_t)bits - 0x3F320000u);
  int32_t kbits = tmp & (int32_t)0xFF800000u;
  float z = u2f((uint32_t)bits - (uint32_t)kbits);
  float e = fsub(fmul((float)kbits, 1.0f / 8388608.0f), sub ? 23.0f : 0.0f);
  int j = (int)((((uint32_t)tmp) >> 20) & 7);
  float s = ffma(z, c_log_r[j], -1.0f);
  float w = fmul(s, s);
  float q0 = ffma(0.33333334f, s, -0.5f);
  float q1 = ffma(0.2f, s, -0.25f);
  float p = fmul(ffma(q1, w, q0), w);
  float t = fadd(c_log_l[j], p);
  float y = ffma(e, WKB_EXP_C2, t);
  float r2 = fadd(s, y);
  return ffma(e, WKB_EXP_C1, r2);
}

// exp-composed tanh used inside gelu (vmath.rs:429-431).
__device__ __forceinline__ float tanh_exp1(float x) {
  return fsub(1.0f, fdiv(2.0f, fadd(exp1(fmul(2.0f, x)), 1.0f)));
}

// <= 1 ULP tanh (vmath.rs:474-546).
__device__ __forceinline__ float tanh1(float x) {
  const float P[6] = {-0.33333316f, 0.13332695f, -0.053892724f, 0.021452034f, -0.0076572555f, 0.0017369358f};
  uint32_t sgn = f2u(x) & 0x80000000u;
  float ax = u2f(f2u(x) & 0x7fffffffu);
  float t = fmul(ax, ax);
  float p = ffma(t, P[5], P[4]);
  p = ffma(t, p, P[3]);
  p = ffma(t, p, P[2]);
  p = ffma(t, p, P[1]);
  p = ffma(t, p, P[0]);
  float w = fmul(ax, t);
  float y_poly = ffma(w, p, ax);
  float axc = (ax != ax) ? 10.0f : (ax < 10.0f ? ax : 10.0f);
  float x2 = fadd(axc, axc);
  float tt = ffma(x2, WKB_EXP_TBL_SCALE, WKB_EXP_MAGIC);
  float n = fsub(tt, WKB_EXP_MAGIC);
  int32_t m = (int32_t)(f2u(tt) - (uint32_t)(0x4B400000 - 1020));
  float r = ffma(n, -WKB_EXP_TBL_C1, x2);
  r = ffma(n, -WKB_EXP_TBL_C2, r);
  int idx = m & 7;
  float tj = idx < 4 ? fmul(exp_tbl(idx + 4), 0.5f) : exp_tbl(idx - 4);
  float q = ffma(r, 1.0f / 24.0f, 1.0f / 6.0f);
  q = ffma(r, q, 0.5f);
  q = ffma(r, q, 1.0f);
  float pm1 = fmul(r, q);
  float mm = ffma(tj, pm1, tj);
  float pow2 = u2f(((uint32_t)(m >> 3)) << 23);
  float d = ffma(mm, pow2, 1.0f);
  float rr = fdiv(1.0f, d);
  float y_exp = ffma(-2.0f, rr, 1.0f);
  float y = ax > 0.75f ? y_exp : y_poly;
  return u2f((f2u(y) & 0x7fffffffu) | sgn);
}

__device__ __forceinline__ float sigmoid1(float x) { return fdiv(1.0f, fadd(1.0f, exp1(-x))); }
__device__ __forceinline__ float silu1(float x) {
  if (x != x) return u2f(f2u(x) | 0x00400000u);
  return fmul(x, sigmoid1(x));
}
__device__ __forceinline__ float gelu1(float x) {
  float x3 = fmul(fmul(x, x), x);
  float inner = fmul(0.7978846f, ffma(0.044715f, x3, x));
  return fmul(fmul(0.5f, x), fadd(1.0f, tanh_exp1(inner)));
}

// Cephes sin/cos with the 3-part pi/2 reduction (vmath.rs:255-275, :706-760).  For |x| >= 4096 the
// reference defers to libm; the CUDA libm stands in there (parity by tolerance beyond that range).
__device__ __forceinline__ float sincos1(float x, bool is_cos) {
  uint32_t mag = f2u(x) & 0x7fffffffu;
  if (mag >= 0x7f800000u) return mag > 0x7f800000u ? u2f(f2u(x) | 0x00400000u) : u2f(0x7fc00000u);
  if (fabsf(x) >= 4096.0f) return is_cos ? cosf(x) : sinf(x);
  if (x == 0.0f) return is_cos ? 1.0f : x;
  float tt = ffma(x, 0.636619772367581343f, WKB_EXP_MAGIC);
  float qf = fsub(tt, WKB_EXP_MAGIC);
  float r = ffma(qf, -1.5703125f, x);
  r = ffma(qf, -4.837512969970703e-4f, r);
  r = ffma(qf, -7.54978995489188e-8f, r);
  float z = fmul(r, r);
  float s = -1.9515295891e-4f;
  s = ffma(s, z, 8.3321608736e-3f);
  s = ffma(s, z, -1.6666654611e-1f);
  float sin_p = ffma(fmul(s, z), r, r);
  float c = 2.443315711809948e-5f;
  c = ffma(c, z, -1.388731625493765e-3f);
  c = ffma(c, z, 4.166664568298827e-2f);
  float cos_p = fadd(ffma(-0.5f, z, 1.0f), fmul(c, fmul(z, z)));
  int quad = ((int)qf) & 3;
  float neg_sin = fmul(sin_p, -1.0f), neg_cos = fmul(cos_p, -1.0f);
  if (is_cos) return quad == 0 ? cos_p : quad == 1 ? neg_sin : quad == 2 ? neg_cos : sin_p;
  return quad == 0 ? sin_p : quad == 1 ? cos_p : quad == 2 ? neg_sin : neg_cos;
}

// Activation codes of the fused GEMM epilogue (gemm.rs:726-733) and of vmath (vmath.rs:81-116).
__device__ __forceinline__ float act_apply(int act, float y) {
  switch (act) {
    case 1: return y > 0.0f ? y : 0.0f;
    case 2: return gelu1(y);
    case 3: return silu1(y);
    default: return y;
  }
}
__device__ __forceinline__ float vmath_apply(int op, float x) {
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
    default: return x;
  }
}

// bf16 <-> f32 exactly as the runtime defines them (lib.rs:287-302): RNE with NaN quieting.
__device__ __host__ __forceinline__ u16 f32_to_bf16_bits(float x) {
  uint32_t bits;
#ifdef __CUDA_ARCH__
  bits = __float_as_uint(x);
#else
  memcpy(&bits, &x, 4);
#endif
  if (x != x) return (u16)((bits >> 16) | 0x0040);
  uint32_t bias = 0x00007fffu + ((bits >> 16) & 1u);
  return (u16)((bits + bias) >> 16);
}
__device__ __forceinline__ float bf16_bits_to_f32(u16 b) { return __uint_as_float(((uint32_t)b) << 16); }
__device__ __forceinline__ float f16_bits_to_f32(u16 b) { return __half2float(__ushort_as_half(b)); }
// f32 -> IEEE f16 bits, round to nearest even, in integer arithmetic (equals F16C / the `half`
// crate).  Integer-only on purpose: a byte store fed directly by the hardware convert's 16-bit
// result register came out with a wrong low byte on sm_100a builds.
__device__ __forceinline__ u16 f32_to_f16_bits(float f) {
  uint32_t x = __float_as_uint(f);
  uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7fffffffu;
  if (x > 0x7f800000u) return (u16)(sign | 0x7e00u | ((x >> 13) & 0x03ffu));
  int e = (int)(x >> 23);
  if (e >= 143) return (u16)(sign | 0x7c00u);
  uint32_t m = (x & 0x007fffffu) | 0x00800000u;
  if (e < 113) {
    int sh = 126 - e;
    if (sh >= 25) return (u16)sign;
    uint32_t q = m >> sh, rem = m & ((1u << sh) - 1u), half = 1u << (sh - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q;
    return (u16)(sign | q);
  }
  uint32_t q = ((uint32_t)(e - 112) << 10) | ((m & 0x007fffffu) >> 13);
  uint32_t rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) ++q;
  return (u16)(sign | q);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- programmatic dependent launch -------------------------------------------------------------------------------
// The kernels of a decode step are short (5-100 us) and strictly ordered on one stream, so the gap between two of them
// (drain, launch, block scheduling, prologue) is a visible share of the step.  A kernel launched through launch_pdl
// may become resident while its predecessor is still running; it must call pdl_wait() -- every thread, before its
// first access to global memory -- which returns once the predecessor has completed and its writes are visible, and
// it calls pdl_trigger() to let its own successor be scheduled early.  With WKB_PDL=0 in the environment launch_pdl
// is a plain launch and both calls are no-ops in effect.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
inline bool pdl_enabled() {
  static const bool on = [] { const char* e = getenv("WKB_PDL"); return !(e && e[0] == '0'); }();
  return on;
}
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

static inline int ceil_div_i(i64 a, i64 b) { return (int)((a + b - 1) / b); }
static inline cudaStream_t as_stream(void* s) { return (cudaStream_t)s; }

}  // namespace wkb

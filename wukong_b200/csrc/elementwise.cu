// Elementwise kernels: activations (vmath), gated activations (vmath2), affine/Hadamard (velem).
// fp32 forms follow the scalar operation order of the runtime ABI, so results are bit-identical to
// the reference CPU kernels (vmath.rs:1000-1090, :1506-1512, velem.rs:134-168).  bf16 forms
// (GELU / SiLU-gate for the half-precision decode path) widen, compute in fp32 and round once.
// All are HBM-bound: 128-bit loads/stores, grid sized in multiples of the SM count.
#include "common.cuh"
#include "wkb_device.h"

namespace wkb {

__global__ void __launch_bounds__(256) vmath_f32_kernel(const float* __restrict__ x, float* __restrict__ out,
                                                        i64 n, int op) {
  i64 n4 = n >> 2;
  i64 stride = (i64)gridDim.x * blockDim.x;
  bool al = ((((uintptr_t)x) | ((uintptr_t)out)) & 15) == 0;
  i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (al) {
    for (i64 v = i; v < n4; v += stride) {
      float4 a = reinterpret_cast<const float4*>(x)[v];
      a.x = vmath_apply(op, a.x);
      a.y = vmath_apply(op, a.y);
      a.z = vmath_apply(op, a.z);
      a.w = vmath_apply(op, a.w);
      reinterpret_cast<float4*>(out)[v] = a;
    }
    for (i64 e = (n4 << 2) + i; e < n; e += stride) out[e] = vmath_apply(op, x[e]);
  } else {
    for (i64 e = i; e < n; e += stride) out[e] = vmath_apply(op, x[e]);
  }
}

__global__ void __launch_bounds__(256) vmath2_f32_kernel(const float* __restrict__ x, const float* __restrict__ y,
                                                         float* __restrict__ out, i64 n, int op) {
  i64 stride = (i64)gridDim.x * blockDim.x;
  for (i64 e = (i64)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    float a = x[e], b = y[e], r;
    switch (op) {
      case 9: r = fmul(silu1(a), b); break;
      case 10: r = fmul(gelu1(a), b); break;
      default: r = fmul(sigmoid1(a), b); break;  // 11
    }
    out[e] = r;
  }
}

__global__ void __launch_bounds__(256) velem_f32_kernel(const float* __restrict__ x, const float* __restrict__ y,
                                                        float* __restrict__ out, i64 n, float a, float b, float c,
                                                        int op) {
  i64 stride = (i64)gridDim.x * blockDim.x;
  for (i64 e = (i64)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) {
    float base;
    if (op & 512) base = fmul(x[e], y[e]);
    else if (op & 1024) base = fdiv(x[e], y[e]);
    else if (!(op & 256) && a == 1.0f && c == 0.0f) base = x[e];
    else {
      float inner = (op & 256) ? ffma(b, y[e], c) : c;
      base = ffma(a, x[e], inner);
    }
    int act = op & 0xff;
    if (act == 1) base = base > 0.0f ? base : 0.0f;
    else if (act == 2) { base = base > 0.0f ? base : 0.0f; base = base < 6.0f ? base : 6.0f; }
    out[e] = base;
  }
}

// bf16 activation: out = act(x) (op 5 silu, 6 gelu, 4 relu) or out = act(x) * y when y != null.
__global__ void __launch_bounds__(256) act_bf16_kernel(const __nv_bfloat16* __restrict__ x,
                                                       const __nv_bfloat16* __restrict__ y,
                                                       __nv_bfloat16* __restrict__ out, i64 n, int op) {
  i64 n8 = n >> 3;
  i64 stride = (i64)gridDim.x * blockDim.x;
  i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  for (i64 v = i; v < n8; v += stride) {
    uint4 xa = reinterpret_cast<const uint4*>(x)[v];
    uint4 ya = y ? reinterpret_cast<const uint4*>(y)[v] : make_uint4(0, 0, 0, 0);
    uint32_t xs[4] = {xa.x, xa.y, xa.z, xa.w}, ys[4] = {ya.x, ya.y, ya.z, ya.w}, os[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float lo = vmath_apply(op, bf16_bits_to_f32((u16)(xs[k] & 0xffff)));
      float hi = vmath_apply(op, bf16_bits_to_f32((u16)(xs[k] >> 16)));
      if (y) {
        lo = fmul(lo, bf16_bits_to_f32((u16)(ys[k] & 0xffff)));
        hi = fmul(hi, bf16_bits_to_f32((u16)(ys[k] >> 16)));
      }
      os[k] = (uint32_t)f32_to_bf16_bits(lo) | ((uint32_t)f32_to_bf16_bits(hi) << 16);
    }
    reinterpret_cast<uint4*>(out)[v] = make_uint4(os[0], os[1], os[2], os[3]);
  }
  const u16* xb = reinterpret_cast<const u16*>(x);
  const u16* yb = reinterpret_cast<const u16*>(y);
  u16* ob = reinterpret_cast<u16*>(out);
  for (i64 e = (n8 << 3) + i; e < n; e += stride) {
    float r = vmath_apply(op, bf16_bits_to_f32(xb[e]));
    if (y) r = fmul(r, bf16_bits_to_f32(yb[e]));
    ob[e] = f32_to_bf16_bits(r);
  }
}

static inline int ew_grid(i64 work_items) {
  i64 blocks = (work_items + 255) / 256;
  i64 cap = (i64)WKB_SM_COUNT * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

}  // namespace wkb

using namespace wkb;

extern "C" {

int wkb_vmath_f32(const float* x, float* out, i64 n, i64 op, void* stream) {
  if (n <= 0) return 0;
  vmath_f32_kernel<<<ew_grid((n + 3) / 4), 256, 0, as_stream(stream)>>>(x, out, n, (int)op);
  return (int)cudaGetLastError();
}

int wkb_vmath2_f32(const float* x, const float* y, float* out, i64 n, i64 op, void* stream) {
  if (n <= 0) return 0;
  vmath2_f32_kernel<<<ew_grid(n), 256, 0, as_stream(stream)>>>(x, y, out, n, (int)op);
  return (int)cudaGetLastError();
}

int wkb_velem_f32(const float* x, const float* y, float* out, i64 n, float a, float b, float c, i64 op,
                  void* stream) {
  if (n <= 0) return 0;
  velem_f32_kernel<<<ew_grid(n), 256, 0, as_stream(stream)>>>(x, y, out, n, a, b, c, (int)op);
  return (int)cudaGetLastError();
}

int wkb_act_bf16(const void* x, const void* y_gate_or_null, void* out, i64 n, i64 op, void* stream) {
  if (n <= 0) return 0;
  if (((((uintptr_t)x) | ((uintptr_t)out) | ((uintptr_t)y_gate_or_null)) & 15) != 0) return (int)cudaErrorMisalignedAddress;
  act_bf16_kernel<<<ew_grid((n + 7) / 8), 256, 0, as_stream(stream)>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)y_gate_or_null, (__nv_bfloat16*)out, n, (int)op);
  return (int)cudaGetLastError();
}
}

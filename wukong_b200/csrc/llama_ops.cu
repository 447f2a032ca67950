// Row-wise glue of the Llama-shape decode block: residual add fused with RMSNorm, and RoPE applied
// in place to the query / key heads of a fused QKV row.
//
// add_rmsnorm: x[r, :] += delta[r, :] (when delta is given), then out[r, :] = bf16(x * inv * gamma) with
//   inv = 1 / sqrt(mean(x^2) + eps) -- the RMSNORM op of crates/wukong_runtime/src/norm.rs:50-54 on the
//   updated residual stream, in the precision recipe of the half-precision path (fp32 statistics, one
//   rounding on the way out).  The same row is read by the add and by the norm, so fusing them saves one
//   pass over the residual stream per sub-block.
// rope_qk: half-split pairs (x[j], x[j + half]) rotated by theta = pos[r] * inv_freq[j] with the
//   runtime's own sin / cos sequence (crates/wukong_runtime/src/rope.rs:54-71); the position comes from
//   a vector because a decode row sits at an arbitrary position of its sequence.
#include "common.cuh"
#include "wkb_device.h"

namespace wkb {

__global__ void __launch_bounds__(256) add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                                          const float* __restrict__ gamma, u16* __restrict__ out,
                                                          i64 rows, int cols, float eps) {
  __shared__ float red[8];
  const int nvec = cols >> 2;
  for (i64 r = blockIdx.x; r < rows; r += gridDim.x) {
    float4* xr = reinterpret_cast<float4*>(x + r * (i64)cols);
    const float4* dr = delta ? reinterpret_cast<const float4*>(delta + r * (i64)cols) : nullptr;
    float q = 0.0f;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      float4 v = xr[i];
      if (dr) {
        const float4 d = dr[i];
        v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
        xr[i] = v;
      }
      q = fmaf(v.x, v.x, q); q = fmaf(v.y, v.y, q); q = fmaf(v.z, v.z, q); q = fmaf(v.w, v.w, q);
    }
    q = warp_sum(q);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = q;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w];
    const float inv = rsqrtf(tot / (float)cols + eps);
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
      const float4 v = xr[i];  // this thread's own earlier write
      const float4 g = gamma ? reinterpret_cast<const float4*>(gamma)[i] : make_float4(1.f, 1.f, 1.f, 1.f);
      uint2 o;
      o.x = (uint32_t)f32_to_bf16_bits(v.x * inv * g.x) | ((uint32_t)f32_to_bf16_bits(v.y * inv * g.y) << 16);
      o.y = (uint32_t)f32_to_bf16_bits(v.z * inv * g.z) | ((uint32_t)f32_to_bf16_bits(v.w * inv * g.w) << 16);
      reinterpret_cast<uint2*>(out + r * (i64)cols)[i] = o;
    }
  }
}

__global__ void __launch_bounds__(256) rope_qk_kernel(float* x, i64 row_stride, const float* __restrict__ inv_freq,
                                                      const int* __restrict__ pos, i64 rows, i64 heads, i64 half) {
  const i64 total = rows * heads * half;
  const i64 stride = (i64)gridDim.x * blockDim.x;
  for (i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const i64 j = idx % half, rh = idx / half, r = rh / heads, hh = rh % heads;
    const float theta = fmul((float)pos[r], inv_freq[j]);
    const float c = sincos1(theta, true), s = sincos1(theta, false);
    float* p = x + r * row_stride + hh * 2 * half;
    const float a = p[j], b = p[j + half];
    p[j] = ffma(b, -s, fmul(a, c));
    p[j + half] = ffma(a, s, fmul(b, c));
  }
}

// Vocabulary-parallel greedy sampling: each rank packs (value bits, global column) of its local arg-max;
// after the gather the pick applies the arg-max rule across ranks (greater value wins, equal values keep
// the lower column, a NaN never wins unless it sits in global column 0, which pins the row to 0).
__global__ void __launch_bounds__(128) argmax_pack_kernel(const float* __restrict__ logits, i64 ld, const int* __restrict__ idx,
                                                          int col_offset, i64 rows, int* __restrict__ pairs) {
  const i64 r = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int i = idx[r];
  pairs[2 * r] = __float_as_int(logits[r * ld + i]);
  pairs[2 * r + 1] = i + col_offset;
}

__global__ void __launch_bounds__(128) argmax_pick_kernel(const int* __restrict__ pairs, int world, i64 rows, int* __restrict__ out) {
  const i64 r = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  float bv = 0.0f;
  int bi = -1;
  for (int g = 0; g < world; ++g) {
    const float v = __int_as_float(pairs[(g * rows + r) * 2]);
    const int i = pairs[(g * rows + r) * 2 + 1];
    if (i == 0 && v != v) { bi = 0; break; }
    if (v != v) continue;
    if (bi < 0 || v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  }
  out[r] = bi < 0 ? 0 : bi;
}

}  // namespace wkb

using namespace wkb;

extern "C" {

int wkb_add_rmsnorm_bf16(float* x, const float* delta_or_null, const float* gamma_or_null, void* out_bf16, i64 rows,
                         i64 cols, float eps, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 4 != 0) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)x) | ((uintptr_t)delta_or_null) | ((uintptr_t)gamma_or_null) | ((uintptr_t)out_bf16)) & 15)
    return (int)cudaErrorMisalignedAddress;
  const int grid = (int)(rows < (i64)WKB_SM_COUNT * 8 ? rows : (i64)WKB_SM_COUNT * 8);
  add_rmsnorm_kernel<<<grid, 256, 0, as_stream(stream)>>>(x, delta_or_null, gamma_or_null, (u16*)out_bf16, rows, (int)cols, eps);
  return (int)cudaGetLastError();
}

int wkb_rope_qk_f32(float* x, i64 row_stride, const float* inv_freq, const int* pos, i64 rows, i64 heads, i64 half,
                    void* stream) {
  if (rows <= 0 || heads <= 0 || half <= 0) return 0;
  if (!pos || row_stride < heads * 2 * half) return (int)cudaErrorInvalidValue;
  const i64 total = rows * heads * half;
  i64 grid = (total + 255) / 256;
  if (grid > (i64)WKB_SM_COUNT * 16) grid = (i64)WKB_SM_COUNT * 16;
  rope_qk_kernel<<<(int)grid, 256, 0, as_stream(stream)>>>(x, row_stride, inv_freq, pos, rows, heads, half);
  return (int)cudaGetLastError();
}

int wkb_argmax_pack(const float* logits, i64 ld, const int* idx_local, i64 col_offset, i64 rows, int* pairs, void* stream) {
  if (rows <= 0) return 0;
  argmax_pack_kernel<<<(int)((rows + 127) / 128), 128, 0, as_stream(stream)>>>(logits, ld, idx_local, (int)col_offset, rows, pairs);
  return (int)cudaGetLastError();
}

int wkb_argmax_pick(const int* pairs, i64 world, i64 rows, int* out, void* stream) {
  if (rows <= 0 || world <= 0) return 0;
  argmax_pick_kernel<<<(int)((rows + 127) / 128), 128, 0, as_stream(stream)>>>(pairs, (int)world, rows, out);
  return (int)cudaGetLastError();
}

}  // extern "C"

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

int* gemm_status_word();   // the library's device status word (gemm_tc.cu)

// One CTA per row; a thread keeps its NV float4 of the row in registers between the statistic and the write-back,
// so the row is read once (x and delta) and written once (x and the bf16 normed row).
template <int NV>
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta,
                                                           const float* __restrict__ gamma, u16* __restrict__ out,
                                                           i64 rows, int cols, float eps, int nsl, i64 slice_stride, i64 dld) {
  __shared__ float red[32];
  const int nvec = cols >> 2, nwarps = blockDim.x >> 5;
  pdl_wait();
  pdl_trigger();
  for (i64 r = blockIdx.x; r < rows; r += gridDim.x) {
    float4* xr = reinterpret_cast<float4*>(x + r * (i64)cols);
    // delta: nsl planes of pitch dld, added in plane order (the K-slice partials of a split GEMM, or one plain matrix)
    const float4* dr = delta ? reinterpret_cast<const float4*>(delta + r * dld) : nullptr;
    float4 v[NV];
    float q = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < nvec) {
        v[k] = xr[i];
        if (dr) {
          float4 d = __ldcg(dr + i);
          for (int sl = 1; sl < nsl; ++sl) {
            const float4 e = __ldcg(reinterpret_cast<const float4*>(delta + sl * slice_stride + r * dld) + i);
            d.x += e.x; d.y += e.y; d.z += e.z; d.w += e.w;
          }
          v[k].x += d.x; v[k].y += d.y; v[k].z += d.z; v[k].w += d.w;
        }
        q = fmaf(v[k].x, v[k].x, q); q = fmaf(v[k].y, v[k].y, q); q = fmaf(v[k].z, v[k].z, q); q = fmaf(v[k].w, v[k].w, q);
      }
    }
    q = warp_sum(q);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = q;
    __syncthreads();
    float tot = 0.0f;
    for (int w = 0; w < nwarps; ++w) tot += red[w];
    const float inv = rsqrtf(tot / (float)cols + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < nvec) {
        if (dr) xr[i] = v[k];
        const float4 g = gamma ? reinterpret_cast<const float4*>(gamma)[i] : make_float4(1.f, 1.f, 1.f, 1.f);
        uint2 o;
        o.x = (uint32_t)f32_to_bf16_bits(v[k].x * inv * g.x) | ((uint32_t)f32_to_bf16_bits(v[k].y * inv * g.y) << 16);
        o.y = (uint32_t)f32_to_bf16_bits(v[k].z * inv * g.z) | ((uint32_t)f32_to_bf16_bits(v[k].w * inv * g.w) << 16);
        reinterpret_cast<uint2*>(out + r * (i64)cols)[i] = o;
      }
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

// RoPE and the KV append in one pass over a fused QKV row: a thread owns the pair (j, j + half) of one head.
// Query heads are rotated in place; key heads are rotated and rounded straight into their page; value heads are
// rounded into theirs.  Same pairing, sin / cos and page addressing as rope_qk_kernel and paged_kv_append_kernel
// (pages are bf16 [page][kv_head][token][dim]); a row with pos < 0 is inactive and touches nothing.
__global__ void __launch_bounds__(256) rope_append_kernel(float* qkv, i64 row_stride, const float* __restrict__ src, int nsl,
                                                          i64 slice_stride, i64 sld, const float* __restrict__ inv_freq,
                                                          const uint32_t* __restrict__ block_table, const int* __restrict__ row_slot,
                                                          const int* __restrict__ row_pos, u16* __restrict__ kcache,
                                                          u16* __restrict__ vcache, i64 rows, int hq, int hkv, int half,
                                                          int page_tokens, int mbps, int* __restrict__ status) {
  const int heads = hq + 2 * hkv, hd = 2 * half;
  const i64 total = rows * heads * half;
  pdl_wait();
  pdl_trigger();
  for (i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    const int j = (int)(idx % half);
    const i64 rh = idx / half;
    const int hh = (int)(rh % heads);
    const i64 r = rh / heads;
    const int pos = row_pos[r];
    if (pos < 0) continue;
    if (pos / page_tokens >= mbps) {   // beyond the block-table row: the row is skipped whole and reported
      if (j == 0 && hh == 0 && status) atomicExch(status, WKB_STATUS_KV_POS_RANGE);
      continue;
    }
    float* p = qkv + r * row_stride + (i64)hh * hd;
    float a, b;
    if (src) {
      // the projection's K-slice partials, added in slice order
      const float* sp = src + r * sld + (i64)hh * hd;
      a = __ldcg(sp + j); b = __ldcg(sp + j + half);
      for (int sl = 1; sl < nsl; ++sl) { a += __ldcg(sp + sl * slice_stride + j); b += __ldcg(sp + sl * slice_stride + j + half); }
    } else {
      a = p[j]; b = p[j + half];
    }
    if (hh < hq + hkv) {
      const float theta = fmul((float)pos, inv_freq[j]);
      const float c = sincos1(theta, true), s = sincos1(theta, false);
      const float ra = ffma(b, -s, fmul(a, c)), rb = ffma(a, s, fmul(b, c));
      a = ra; b = rb;
    }
    if (hh < hq) {
      p[j] = a; p[j + half] = b;
    } else {
      const int kvh = hh < hq + hkv ? hh - hq : hh - hq - hkv;
      const uint32_t page = block_table[(i64)row_slot[r] * mbps + pos / page_tokens];
      const i64 dst = (((i64)page * hkv + kvh) * page_tokens + pos % page_tokens) * hd;
      u16* cache = hh < hq + hkv ? kcache : vcache;
      cache[dst + j] = f32_to_bf16_bits(a);
      cache[dst + j + half] = f32_to_bf16_bits(b);
    }
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

static int launch_add_rmsnorm(float* x, const float* delta, int nsl, i64 slice_stride, i64 dld, const float* gamma, void* out_bf16, i64 rows,
                              i64 cols, float eps, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (cols % 4 != 0 || dld % 4 != 0 || slice_stride % 4 != 0) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)x) | ((uintptr_t)delta) | ((uintptr_t)gamma) | ((uintptr_t)out_bf16)) & 15) return (int)cudaErrorMisalignedAddress;
  const int grid = (int)(rows < (i64)WKB_SM_COUNT * 2 ? rows : (i64)WKB_SM_COUNT * 2);
  const i64 nvec = cols / 4;
  // as many threads as the row has float4 (up to 1024), then 2 or 4 or 8 vectors per thread
  int threads = (int)(((nvec < 1024 ? nvec : 1024) + 31) / 32 * 32);
  const i64 per = (nvec + threads - 1) / threads;
  cudaStream_t st = as_stream(stream);
  u16* o = (u16*)out_bf16;
#define WKB_ARN(NV_) launch_pdl(add_rmsnorm_kernel<NV_>, grid, threads, 0, st, x, delta, gamma, o, rows, (int)cols, eps, nsl, slice_stride, dld)
  if (per <= 1) WKB_ARN(1);
  else if (per <= 2) WKB_ARN(2);
  else if (per <= 4) WKB_ARN(4);
  else if (per <= 8) WKB_ARN(8);
  else return (int)cudaErrorInvalidValue;   // rows wider than 32768 columns
#undef WKB_ARN
  return (int)cudaGetLastError();
}

int wkb_add_rmsnorm_bf16(float* x, const float* delta_or_null, const float* gamma_or_null, void* out_bf16, i64 rows,
                         i64 cols, float eps, void* stream) {
  return launch_add_rmsnorm(x, delta_or_null, 1, 0, cols, gamma_or_null, out_bf16, rows, cols, eps, stream);
}

int wkb_add_slices_rmsnorm_bf16(float* x, const float* slices, i64 nslices, i64 slice_stride, i64 ld, const float* gamma_or_null,
                                void* out_bf16, i64 rows, i64 cols, float eps, void* stream) {
  if (nslices < 1 || !slices) return (int)cudaErrorInvalidValue;
  return launch_add_rmsnorm(x, slices, (int)nslices, slice_stride, ld, gamma_or_null, out_bf16, rows, cols, eps, stream);
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

int wkb_rope_qk_paged_append(float* qkv, i64 row_stride, const float* inv_freq, const uint32_t* block_table, const int* row_slot,
                             const int* row_pos, void* kcache, void* vcache, i64 rows, i64 q_heads, i64 kv_heads, i64 half,
                             i64 page_tokens, i64 max_blocks_per_seq, void* stream) {
  if (rows <= 0) return 0;
  if (q_heads < 0 || kv_heads <= 0 || half <= 0 || page_tokens <= 0 || row_stride < (q_heads + 2 * kv_heads) * 2 * half)
    return (int)cudaErrorInvalidValue;
  const i64 total = rows * (q_heads + 2 * kv_heads) * half;
  i64 grid = (total + 255) / 256;
  if (grid > (i64)WKB_SM_COUNT * 16) grid = (i64)WKB_SM_COUNT * 16;
  return (int)launch_pdl(rope_append_kernel, (int)grid, 256, 0, as_stream(stream), qkv, row_stride, (const float*)nullptr, 0, (i64)0, (i64)0, inv_freq,
                         block_table, row_slot, row_pos, (u16*)kcache, (u16*)vcache, rows, (int)q_heads, (int)kv_heads, (int)half,
                         (int)page_tokens, (int)max_blocks_per_seq, gemm_status_word());
}

int wkb_rope_qk_paged_append_slices(float* q_out, i64 row_stride, const float* slices, i64 nslices, i64 slice_stride, i64 ld,
                                    const float* inv_freq, const uint32_t* block_table, const int* row_slot, const int* row_pos,
                                    void* kcache, void* vcache, i64 rows, i64 q_heads, i64 kv_heads, i64 half, i64 page_tokens,
                                    i64 max_blocks_per_seq, void* stream) {
  if (rows <= 0) return 0;
  if (!slices || nslices < 1 || q_heads < 0 || kv_heads <= 0 || half <= 0 || page_tokens <= 0 || row_stride < q_heads * 2 * half ||
      ld < (q_heads + 2 * kv_heads) * 2 * half)
    return (int)cudaErrorInvalidValue;
  const i64 total = rows * (q_heads + 2 * kv_heads) * half;
  i64 grid = (total + 255) / 256;
  if (grid > (i64)WKB_SM_COUNT * 16) grid = (i64)WKB_SM_COUNT * 16;
  return (int)launch_pdl(rope_append_kernel, (int)grid, 256, 0, as_stream(stream), q_out, row_stride, slices, (int)nslices, slice_stride, ld, inv_freq,
                         block_table, row_slot, row_pos, (u16*)kcache, (u16*)vcache, rows, (int)q_heads, (int)kv_heads, (int)half,
                         (int)page_tokens, (int)max_blocks_per_seq, gemm_status_word());
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

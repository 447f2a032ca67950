// Decode attention over a padded KV cache (fp32), the square single-head sdpa, and the KV append.
//
// `attention_kv_exact_kernel` reproduces the reference's per-(row, head) numeric contract
// (crates/wukong_runtime/src/attention_kv.rs:52-69, portable twin :423-549): key blocks of 64 from
// key 0; each score is eight FMA lanes over d folded ((l0+l1)+(l2+l3))+((l4+l5)+(l6+l7)) plus an
// FMA tail, times scale; block max by the MAXPS rule on eight lanes seeded with the running max;
// weights exp1(s-m) summed on eight lanes then a fixed tree; acc = acc*corr then one FMA per key
// in key order; o = acc*(1/l), exactly +0.0 for a row that sees no key.  Masked keys are never
// read.  One CTA per (sequence, query row, head); outputs are bit-identical to the CPU kernel.
#include "common.cuh"
#include "wkb_device.h"

namespace wkb {

constexpr int KV_BC = 64;
constexpr int ATT_NT = 128;
constexpr int ATT_MAXD = 512;

struct AttGeo {
  i64 batch, sq, d, n_heads, n_kv_heads, q_stride, kv_stride, q_bstride, kv_bstride;
  i64 skv_single, q_pos0_single;  // used when kv_lens == nullptr
  float scale;
  int causal;
};

__global__ void __launch_bounds__(ATT_NT) attention_kv_exact_kernel(const float* __restrict__ q,
                                                                    const float* __restrict__ k,
                                                                    const float* __restrict__ v, float* __restrict__ o,
                                                                    const int* __restrict__ kv_lens,
                                                                    const int* __restrict__ q_pos, AttGeo g) {
  __shared__ float sc[KV_BC];
  __shared__ float bc[2];  // corr, unused
  __shared__ float qs[ATT_MAXD];
  const int tid = threadIdx.x;
  const i64 units = g.batch * g.sq * g.n_heads;
  const int d = (int)g.d, dv = d & ~7;
  const i64 group = g.n_heads / g.n_kv_heads;
  for (i64 u = blockIdx.x; u < units; u += gridDim.x) {
    i64 h = u % g.n_heads, i = (u / g.n_heads) % g.sq, b = u / (g.n_heads * g.sq);
    i64 len = kv_lens ? (i64)kv_lens[b] : g.skv_single;
    i64 pos = q_pos ? (i64)q_pos[b] : g.q_pos0_single;
    i64 keys = len;
    if (g.causal) {
      i64 vis = pos + i + 1;
      keys = vis < 0 ? 0 : (vis > len ? len : vis);
    }
    const float* qv = q + b * g.q_bstride + i * g.q_stride + h * g.d;
    float* out = o + b * g.q_bstride + i * g.q_stride + h * g.d;
    const float* kb = k + b * g.kv_bstride + (h / group) * g.d;
    const float* vb = v + b * g.kv_bstride + (h / group) * g.d;
    __syncthreads();
    for (int t = tid; t < d; t += ATT_NT) qs[t] = qv[t];
    float acc[ATT_MAXD / ATT_NT];
#pragma unroll
    for (int a = 0; a < ATT_MAXD / ATT_NT; ++a) acc[a] = 0.0f;
    float m = -INFINITY, l = 0.0f;
    __syncthreads();
    for (i64 j0 = 0; j0 < keys; j0 += KV_BC) {
      int kbn = (int)(keys - j0 < KV_BC ? keys - j0 : KV_BC);
      // scores: 8 threads per key, thread `ln` runs FMA lane `ln`
      for (int item = tid; item < KV_BC * 8; item += ATT_NT) {
        int jj = item >> 3, ln = item & 7;
        float lane_acc = 0.0f;
        if (jj < kbn) {
          const float* kr = kb + (j0 + jj) * g.kv_stride;
          for (int t = ln; t < dv; t += 8) lane_acc = ffma(qs[t], kr[t], lane_acc);
        }
        float s1 = fadd(lane_acc, __shfl_xor_sync(0xffffffffu, lane_acc, 1));
        float s2 = fadd(s1, __shfl_xor_sync(0xffffffffu, s1, 2));
        float tree = fadd(s2, __shfl_xor_sync(0xffffffffu, s2, 4));
        if (ln == 0 && jj < kbn) {
          if (dv != d) {
            const float* kr = kb + (j0 + jj) * g.kv_stride;
            float tail = 0.0f;
            for (int t = dv; t < d; ++t) tail = ffma(qs[t], kr[t], tail);
            tree = fadd(tree, tail);
          }
          sc[jj] = fmul(tree, g.scale);
        }
      }
      __syncthreads();
      // block max, exp weights and their sum: the eight-lane chains and trees, on one warp
      if (tid < 32) {
        int nv = kbn & ~7;
        float lane_m = m;
        if (tid < 8) for (int c = 0; c < nv; c += 8) lane_m = maxps(lane_m, sc[c + tid]);
        float l0 = __shfl_sync(0xffffffffu, lane_m, 0), l1 = __shfl_sync(0xffffffffu, lane_m, 1);
        float l2 = __shfl_sync(0xffffffffu, lane_m, 2), l3 = __shfl_sync(0xffffffffu, lane_m, 3);
        float l4 = __shfl_sync(0xffffffffu, lane_m, 4), l5 = __shfl_sync(0xffffffffu, lane_m, 5);
        float l6 = __shfl_sync(0xffffffffu, lane_m, 6), l7 = __shfl_sync(0xffffffffu, lane_m, 7);
        float best = m;
        if (nv) best = maxps(maxps(maxps(l0, l4), maxps(l2, l6)), maxps(maxps(l1, l5), maxps(l3, l7)));
        for (int c = nv; c < kbn; ++c) best = maxps(best, sc[c]);
        float mn = best;
        // weights
        float p0 = 0.0f, p1 = 0.0f;
        if (tid < kbn) { p0 = exp1(fsub(sc[tid], mn)); }
        if (tid + 32 < kbn) { p1 = exp1(fsub(sc[tid + 32], mn)); }
        __syncwarp();
        if (tid < kbn) sc[tid] = p0;
        if (tid + 32 < kbn) sc[tid + 32] = p1;
        __syncwarp();
        float sv = 0.0f;
        if (tid < 8) for (int c = 0; c < nv; c += 8) sv = fadd(sv, sc[c + tid]);
        float s0 = __shfl_sync(0xffffffffu, sv, 0), s1 = __shfl_sync(0xffffffffu, sv, 1);
        float s2 = __shfl_sync(0xffffffffu, sv, 2), s3 = __shfl_sync(0xffffffffu, sv, 3);
        float s4 = __shfl_sync(0xffffffffu, sv, 4), s5 = __shfl_sync(0xffffffffu, sv, 5);
        float s6 = __shfl_sync(0xffffffffu, sv, 6), s7 = __shfl_sync(0xffffffffu, sv, 7);
        float rs = 0.0f;
        if (nv) rs = fadd(fadd(fadd(s0, s4), fadd(s1, s5)), fadd(fadd(s2, s6), fadd(s3, s7)));
        for (int c = nv; c < kbn; ++c) rs = fadd(rs, sc[c]);
        if (tid == 0) { bc[0] = mn; bc[1] = rs; }
      }
      __syncthreads();
      float mn = bc[0], rs = bc[1];
      float corr = (m == mn) ? 1.0f : exp1(fsub(m, mn));
      l = fadd(fmul(l, corr), rs);
      m = mn;
#pragma unroll
      for (int a = 0; a < ATT_MAXD / ATT_NT; ++a) {
        int t = tid + a * ATT_NT;
        if (t < d) {
          float av = fmul(acc[a], corr);
          const float* vr = vb + j0 * g.kv_stride + t;
          for (int jj = 0; jj < kbn; ++jj) av = ffma(sc[jj], vr[(i64)jj * g.kv_stride], av);
          acc[a] = av;
        }
      }
      __syncthreads();
    }
    float inv = l != 0.0f ? fdiv(1.0f, l) : 0.0f;
#pragma unroll
    for (int a = 0; a < ATT_MAXD / ATT_NT; ++a) {
      int t = tid + a * ATT_NT;
      if (t < d) out[t] = fmul(acc[a], inv);
    }
  }
}

// Square single-head attention (attention.rs:158-215): per-key online softmax, unfused multiply-add.
// One warp per query row; lane t owns output lanes t, t+32, ...; the dot is a plain in-order sum,
// so it is computed redundantly by every lane (d is small for this builtin's uses).
__global__ void __launch_bounds__(128) sdpa_square_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                          const float* __restrict__ v, float* __restrict__ o, i64 s,
                                                          i64 d, float scale, int causal) {
  int lane = threadIdx.x & 31;
  i64 warp = ((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = ((i64)gridDim.x * blockDim.x) >> 5;
  for (i64 i = warp; i < s; i += nw) {
    const float* qi = q + i * d;
    i64 jmax = causal ? i + 1 : s;
    float m = -INFINITY, l = 0.0f;
    float acc[8];
#pragma unroll
    for (int a = 0; a < 8; ++a) acc[a] = 0.0f;
    for (i64 j = 0; j < jmax; ++j) {
      const float* kj = k + j * d;
      float x = 0.0f;
      for (i64 t = 0; t < d; ++t) x = fadd(x, fmul(qi[t], kj[t]));
      x = fmul(x, scale);
      float mn = m > x ? m : x;
      float corr = (m == mn) ? 1.0f : exp1(fsub(m, mn));
      float p = exp1(fsub(x, mn));
      l = fadd(fmul(l, corr), p);
      const float* vj = v + j * d;
#pragma unroll
      for (int a = 0; a < 8; ++a) {
        i64 t = lane + 32 * a;
        if (t < d) acc[a] = fadd(fmul(acc[a], corr), fmul(p, vj[t]));
      }
      m = mn;
    }
    float inv = l != 0.0f ? fdiv(1.0f, l) : 0.0f;
#pragma unroll
    for (int a = 0; a < 8; ++a) {
      i64 t = lane + 32 * a;
      if (t < d) o[i * d + t] = fmul(acc[a], inv);
    }
  }
}

__global__ void copy_f32_kernel(const float* __restrict__ src, float* __restrict__ dst, i64 n) {
  i64 stride = (i64)gridDim.x * blockDim.x;
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = src[i];
}

}  // namespace wkb

using namespace wkb;

extern "C" {

// Geometry must already be validated (the host entries run the reference's plan checks).
int wkb_attention_kv_f32(const float* q, const float* k, const float* v, float* o, const int* kv_lens,
                         const int* q_pos, i64 batch, i64 sq, i64 skv, i64 d, i64 q_pos0, i64 n_heads,
                         i64 n_kv_heads, i64 q_stride, i64 kv_stride, i64 q_bstride, i64 kv_bstride, float scale,
                         i64 causal, void* stream) {
  if (batch <= 0 || sq <= 0 || n_heads <= 0 || d <= 0) return 0;
  if (d > ATT_MAXD) return (int)cudaErrorInvalidValue;
  AttGeo g{batch, sq, d, n_heads, n_kv_heads, q_stride, kv_stride, q_bstride, kv_bstride, skv, q_pos0, scale, causal != 0};
  i64 units = batch * sq * n_heads;
  int grid = (int)(units < (i64)WKB_SM_COUNT * 16 ? units : (i64)WKB_SM_COUNT * 16);
  attention_kv_exact_kernel<<<grid, ATT_NT, 0, as_stream(stream)>>>(q, k, v, o, kv_lens, q_pos, g);
  return (int)cudaGetLastError();
}

int wkb_attention_f32(const float* q, const float* k, const float* v, float* o, i64 s, i64 d, float scale,
                      i64 causal, void* stream) {
  if (s <= 0 || d <= 0) return 0;
  if (d > 256) return (int)cudaErrorInvalidValue;
  int grid = (int)((s + 3) / 4 < (i64)WKB_SM_COUNT * 8 ? (s + 3) / 4 : (i64)WKB_SM_COUNT * 8);
  sdpa_square_kernel<<<grid, 128, 0, as_stream(stream)>>>(q, k, v, o, s, d, scale, causal != 0);
  return (int)cudaGetLastError();
}

int wkb_kv_append_f32(float* cache, const float* row, i64 nrow, i64 pos, i64 stride, void* stream) {
  if (nrow <= 0) return 0;
  int grid = (int)((nrow + 255) / 256 < 1024 ? (nrow + 255) / 256 : 1024);
  copy_f32_kernel<<<grid, 256, 0, as_stream(stream)>>>(row, cache + pos * stride, nrow);
  return (int)cudaGetLastError();
}
}

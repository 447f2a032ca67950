// Selection, sampling and the counter-based RNG used for decoding beyond greedy arg-max.
//
// Semantics are the reference runtime's (crates/wukong_runtime/src/topk.rs:1-136, random.rs:1-104):
//   * ONE strict total order per direction, so every result is unique whatever the algorithm:
//       descending: NaN largest, larger value first, ties (-0.0 vs +0.0, NaN vs NaN) to the lower index;
//       ascending : smaller value first, NaN last, ties to the lower index (a stable sort).
//     Both are expressed here as a 64-bit sort key that is sorted ASCENDING: the high word is an order-
//     preserving image of the value (complemented for the descending order), the low word the index.
//   * categorical sampling is the inverse CDF over the positive finite weights, the running mass summed in
//     f64 IN INDEX ORDER -- the comparison `acc > u * total` is sensitive to the rounding of that sum, so the
//     device kernel adds in the same order (one thread per row; rows in parallel) and is bit-for-bit the CPU's;
//   * Philox4x32-10 with key (seed lo, seed hi) and counter (ctr lo, ctr hi, 0, 0); rand_f32 = top 24 bits * 2^-24.
// top-k for the small k of decoding runs k rounds of a block-wide minimum over the row held in shared memory;
// a full argsort is a bitonic network over the padded key array.
#include "common.cuh"
#include "wkb_device.h"

namespace wkb {

typedef unsigned long long u64;

__device__ __forceinline__ uint32_t value_key(float v) {   // ascending numeric order, -0.0 == +0.0, NaN above +inf
  if (v != v) return 0xFFFFFFFFu;
  uint32_t b = __float_as_uint(v == 0.0f ? 0.0f : v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ u64 sort_key(float v, uint32_t idx, bool descending) {
  const uint32_t k = value_key(v);
  return ((u64)(descending ? ~k : k) << 32) | idx;
}

__global__ void __launch_bounds__(256) make_keys_kernel(const float* __restrict__ x, i64 n, i64 n_pad, int descending, u64* __restrict__ keys) {
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n_pad; i += (i64)gridDim.x * blockDim.x)
    keys[i] = i < n ? sort_key(x[i], (uint32_t)i, descending != 0) : ~0ull;
}
__global__ void __launch_bounds__(256) bitonic_step_kernel(u64* __restrict__ keys, i64 n_pad, i64 j, i64 k) {
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n_pad; i += (i64)gridDim.x * blockDim.x) {
    const i64 p = i ^ j;
    if (p > i) {
      const u64 a = keys[i], b = keys[p];
      const bool up = (i & k) == 0;
      if ((a > b) == up) { keys[i] = b; keys[p] = a; }
    }
  }
}
__global__ void __launch_bounds__(256) take_sorted_kernel(const u64* __restrict__ keys, const float* __restrict__ x, i64 m,
                                                          float* __restrict__ vals, i64* __restrict__ idx) {
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < m; i += (i64)gridDim.x * blockDim.x) {
    const uint32_t id = (uint32_t)keys[i];
    idx[i] = (i64)id;
    if (vals) vals[i] = x[id];
  }
}

// One CTA per row: k rounds, each the minimum sort key above the previous round's.
__global__ void __launch_bounds__(256) topk_rounds_kernel(const float* __restrict__ x, i64 ld, int cols, int k, float* __restrict__ vals,
                                                          i64* __restrict__ idx, int in_smem) {
  extern __shared__ float row_s[];
  __shared__ u64 red[8];
  __shared__ u64 s_prev;
  const float* xr = x + (i64)blockIdx.x * ld;
  if (in_smem) {
    for (int i = threadIdx.x; i < cols; i += blockDim.x) row_s[i] = xr[i];
    __syncthreads();
  }
  const float* src = in_smem ? row_s : xr;
  u64 prev = 0;
  for (int r = 0; r < k; ++r) {
    u64 best = ~0ull;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
      const u64 key = sort_key(src[i], (uint32_t)i, true);
      if ((r == 0 || key > prev) && key < best) best = key;
    }
#pragma unroll
    for (int ofs = 16; ofs > 0; ofs >>= 1) {
      const u64 o = __shfl_xor_sync(0xffffffffu, best, ofs);
      best = o < best ? o : best;
    }
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
      u64 b = red[0];
      for (int w = 1; w < 8; ++w) b = red[w] < b ? red[w] : b;
      s_prev = b;
      const uint32_t id = (uint32_t)b;
      vals[(i64)blockIdx.x * k + r] = src[id];
      idx[(i64)blockIdx.x * k + r] = (i64)id;
    }
    __syncthreads();
    prev = s_prev;
  }
}

// One thread per row, sequential f64 sums in index order (the reference's arithmetic, hence its bits).
__global__ void __launch_bounds__(128) sample_categorical_kernel(const float* __restrict__ p, i64 ld, i64 rows, i64 cols,
                                                                 const float* __restrict__ u, i64* __restrict__ out) {
  const i64 r = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const float* pr = p + r * ld;
  double total = 0.0;
  for (i64 i = 0; i < cols; ++i) {
    const float w = pr[i];
    if (w > 0.0f && w <= 3.402823466e+38f) total = __dadd_rn(total, (double)w);
  }
  if (!(total > 0.0)) { out[r] = -1; return; }
  float uc = u[r];
  uc = uc != uc ? 0.0f : fminf(1.0f, fmaxf(0.0f, uc));
  const double target = __dmul_rn((double)uc, total);
  double acc = 0.0;
  i64 last = -1;
  for (i64 i = 0; i < cols; ++i) {
    const float w = pr[i];
    if (w > 0.0f && w <= 3.402823466e+38f) {
      acc = __dadd_rn(acc, (double)w);
      last = i;
      if (acc > target) break;
    }
  }
  out[r] = last;
}

__device__ __forceinline__ uint32_t philox_word0(u64 seed, u64 ctr) {
  uint32_t c0 = (uint32_t)ctr, c1 = (uint32_t)(ctr >> 32), c2 = 0u, c3 = 0u;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    if (r > 0) { k0 += 0x9E3779B9u; k1 += 0xBB67AE85u; }
    const u64 p0 = (u64)0xD2511F53u * c0, p1 = (u64)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1, n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t)p0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
  }
  return c0;
}
__global__ void __launch_bounds__(256) rand_fill_kernel(float* __restrict__ out, i64 n, u64 seed, u64 ctr0) {
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (i64)gridDim.x * blockDim.x)
    out[i] = (float)(philox_word0(seed, ctr0 + (u64)i) >> 8) * (1.0f / 16777216.0f);
}

static int grid_of(i64 n) {
  i64 g = (n + 255) / 256;
  if (g > (i64)WKB_SM_COUNT * 16) g = (i64)WKB_SM_COUNT * 16;
  return (int)(g < 1 ? 1 : g);
}

}  // namespace wkb

using namespace wkb;

extern "C" {

int wkb_rand_fill_f32(float* out, i64 n, i64 seed, i64 ctr0, void* stream) {
  if (n <= 0) return 0;
  rand_fill_kernel<<<grid_of(n), 256, 0, as_stream(stream)>>>(out, n, (u64)seed, (u64)ctr0);
  return (int)cudaGetLastError();
}

int wkb_topk_rows_f32(const float* x, i64 ld, i64 rows, i64 cols, i64 k, float* vals, i64* idx, void* stream) {
  if (rows <= 0 || k <= 0) return 0;
  if (cols <= 0 || k > cols || cols > 0x7fffffff || k > 4096) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)cols * 4;
  const int in_smem = smem <= 200 * 1024 ? 1 : 0;
  if (in_smem) {
    cudaError_t e = cudaFuncSetAttribute(topk_rounds_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return (int)e;
  }
  topk_rounds_kernel<<<(unsigned)rows, 256, in_smem ? smem : 0, as_stream(stream)>>>(x, ld, (int)cols, (int)k, vals, idx, in_smem);
  return (int)cudaGetLastError();
}

i64 wkb_argsort_scratch_bytes(i64 n) {
  i64 p = 1;
  while (p < n) p <<= 1;
  return p * 8;
}

// Full order of x[0..n): idx[0..m) (and vals, if given) receive its first m positions.
int wkb_argsort_f32(const float* x, i64 n, float* vals_or_null, i64* idx, i64 m, i64 descending, void* scratch, void* stream) {
  if (n <= 0 || m <= 0) return 0;
  if (m > n || n > 0x7fffffff) return (int)cudaErrorInvalidValue;
  i64 n_pad = 1;
  while (n_pad < n) n_pad <<= 1;
  u64* keys = (u64*)scratch;
  cudaStream_t st = as_stream(stream);
  make_keys_kernel<<<grid_of(n_pad), 256, 0, st>>>(x, n, n_pad, (int)(descending != 0), keys);
  for (i64 k = 2; k <= n_pad; k <<= 1)
    for (i64 j = k >> 1; j > 0; j >>= 1) bitonic_step_kernel<<<grid_of(n_pad), 256, 0, st>>>(keys, n_pad, j, k);
  take_sorted_kernel<<<grid_of(m), 256, 0, st>>>(keys, x, m, vals_or_null, idx);
  return (int)cudaGetLastError();
}

int wkb_sample_categorical_rows_f32(const float* p, i64 ld, i64 rows, i64 cols, const float* u, i64* out, void* stream) {
  if (rows <= 0) return 0;
  sample_categorical_kernel<<<(unsigned)((rows + 127) / 128), 128, 0, as_stream(stream)>>>(p, ld, rows, cols < 0 ? 0 : cols, u, out);
  return (int)cudaGetLastError();
}

}  // extern "C"

// RoPE, embedding gather, per-row arg-max.
// rope: half-split pairs, out[j] = fma(b,-s,a*c), out[j+half] = fma(a,s,b*c), theta = pos*inv_freq[j]
// with the shared Cephes sin/cos (rope.rs:54-71 of the reference runtime) -- bit-identical in fp32.
// embedding: in-range ids copy the row, any other id writes zeros (embedding.rs:118-186).
// rowargmax: ascending scan semantics, strict compare, lowest index on a tie, a NaN at column 0 pins
// the result to 0 and later NaNs never win (rowarg.rs:1-30, reduce.rs:631-639).
#include "common.cuh"
#include <chrono>
#include <thread>
#include "wkb_device.h"

namespace wkb {

// x/out: [rows, heads, 2*half]; position of row r is pos[r] when pos != null, else r (heads == 1 in
// the reference entry).
__global__ void __launch_bounds__(256) rope_f32_kernel(const float* x, const float* __restrict__ inv_freq,
                                                       const int* __restrict__ pos, float* out, i64 rows, i64 heads,
                                                       i64 half) {
  i64 total = rows * heads * half;
  i64 stride = (i64)gridDim.x * blockDim.x;
  for (i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    i64 j = idx % half, rh = idx / half, r = rh / heads;
    float p = pos ? (float)pos[r] : (float)r;
    float theta = fmul(p, inv_freq[j]);
    float c = sincos1(theta, true), s = sincos1(theta, false);
    i64 base = rh * 2 * half;
    float a = x[base + j], b = x[base + j + half];
    out[base + j] = ffma(b, -s, fmul(a, c));
    out[base + j + half] = ffma(a, s, fmul(b, c));
  }
}

// bf16 storage, fp32 math, one rounding on the way out; in place allowed.
__global__ void __launch_bounds__(256) rope_bf16_kernel(const u16* x, const float* __restrict__ inv_freq,
                                                        const int* __restrict__ pos, u16* out, i64 rows, i64 heads,
                                                        i64 half, i64 row_stride) {
  i64 total = rows * heads * half;
  i64 stride = (i64)gridDim.x * blockDim.x;
  for (i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    i64 j = idx % half, rh = idx / half, r = rh / heads, hh = rh % heads;
    float theta = fmul((float)pos[r], inv_freq[j]);
    float c = sincos1(theta, true), s = sincos1(theta, false);
    i64 base = r * row_stride + hh * 2 * half;
    float a = bf16_bits_to_f32(x[base + j]), b = bf16_bits_to_f32(x[base + j + half]);
    out[base + j] = f32_to_bf16_bits(ffma(b, -s, fmul(a, c)));
    out[base + j + half] = f32_to_bf16_bits(ffma(a, s, fmul(b, c)));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) embedding_kernel(T* __restrict__ out, const T* __restrict__ weight,
                                                        const int* __restrict__ ids, i64 t, i64 h, i64 v) {
  pdl_wait();
  pdl_trigger();
  i64 total = t * h;
  i64 stride = (i64)gridDim.x * blockDim.x;
  for (i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    i64 r = idx / h, c = idx % h;
    int id = ids[r];
    out[idx] = (id >= 0 && (i64)id < v) ? weight[(i64)id * h + c] : (T)0;
  }
}

// GPT-2 style input embedding for the half-precision decode path: out[r] = wte[id[r]] + wpe[pos[r]]
// in fp32 (the residual stream is fp32), weights bf16.  Rows whose id is out of range give zeros.
__global__ void __launch_bounds__(256) embed_tok_pos_kernel(float* __restrict__ out, const u16* __restrict__ wte,
                                                            const u16* __restrict__ wpe, const int* __restrict__ ids,
                                                            const int* __restrict__ pos, i64 t, i64 h, i64 v,
                                                            i64 npos) {
  pdl_wait();
  pdl_trigger();
  i64 total = t * h;
  i64 stride = (i64)gridDim.x * blockDim.x;
  for (i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    i64 r = idx / h, c = idx % h;
    int id = ids[r], p = pos[r];
    float a = (id >= 0 && (i64)id < v) ? bf16_bits_to_f32(wte[(i64)id * h + c]) : 0.0f;
    float b = (p >= 0 && (i64)p < npos) ? bf16_bits_to_f32(wpe[(i64)p * h + c]) : 0.0f;
    out[idx] = a + b;
  }
}

// One CTA per row.  Candidates fold with (strictly greater) or (equal and lower index); NaNs past
// column 0 never enter; a NaN at column 0 wins outright.
__global__ void __launch_bounds__(256) rowargmax_kernel(const float* __restrict__ x, int* __restrict__ out, i64 rows,
                                                        i64 cols, i64 ld) {
  __shared__ float sv[8];
  __shared__ long long si[8];
  for (i64 r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* row = x + r * ld;
    float bv = -INFINITY;
    i64 bi = cols;  // "no candidate yet"
    for (i64 j = threadIdx.x; j < cols; j += blockDim.x) {
      float val = row[j];
      if (val != val) continue;
      if (bi == cols || val > bv) { bv = val; bi = j; }
    }
    // warp fold
    for (int ofs = 16; ofs > 0; ofs >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, bv, ofs);
      long long oi = __shfl_xor_sync(0xffffffffu, (long long)bi, ofs);
      bool take = (oi != cols) && (bi == cols || ov > bv || (ov == bv && oi < bi));
      if (take) { bv = ov; bi = oi; }
    }
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      float fv = sv[0];
      i64 fi = si[0];
      for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
        float ov = sv[w];
        i64 oi = si[w];
        bool take = (oi != cols) && (fi == cols || ov > fv || (ov == fv && oi < fi));
        if (take) { fv = ov; fi = oi; }
      }
      float first = row[0];
      int res = (first != first || fi == cols) ? 0 : (int)fi;
      out[r] = res;
    }
  }
}

// out = a + b over fp32 (the residual add of the half-precision decode path when it is not fused).
__global__ void __launch_bounds__(256) add_f32_kernel(const float* a, const float* b, float* out, i64 n) {
  i64 stride = (i64)gridDim.x * blockDim.x;
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = a[i] + b[i];
}

// Device-side feedback of a decode step: the sampled token becomes the next input and the row moves
// one position on (inactive rows, pos < 0, stay inactive).  Lets a run of decode steps replay with
// no host round trip (the block table must already cover the positions ahead).
// A row whose next position would pass max_pos (the last position its block-table row covers) is parked instead:
// pos = -1, ctx = 0, so every later step skips it.
__global__ void decode_advance_kernel(int* row_token, int* row_pos, int* row_ctx, const int* next_tok, int n, int max_pos) {
  pdl_wait();
  pdl_trigger();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && row_pos[i] >= 0) {
    row_token[i] = next_tok[i];
    if (row_pos[i] >= max_pos) { row_pos[i] = -1; row_ctx[i] = 0; }
    else { row_pos[i] += 1; row_ctx[i] += 1; }
  }
}

// One thread that sleeps until `ns` nanoseconds have passed on the device clock (at most 2 s; the poll count is
// bounded as well).  It exists so that the host-side deadline of wkb_stream_sync_within can be exercised without
// any kernel that fails to finish.
__global__ void device_sleep_kernel(unsigned long long ns) {
  unsigned long long t0, now;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (unsigned it = 0; it < (1u << 22); ++it) {
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (now - t0 >= ns) break;
    __nanosleep(1000);
  }
}

static inline int grid_for(i64 items, int per_block) {
  i64 b = (items + per_block - 1) / per_block;
  i64 cap = (i64)WKB_SM_COUNT * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace wkb

using namespace wkb;

extern "C" {

int wkb_rope_f32(const float* x, const float* inv_freq, const int* pos_or_null, float* out, i64 rows, i64 heads,
                 i64 half, void* stream) {
  if (rows <= 0 || half <= 0 || heads <= 0) return 0;
  rope_f32_kernel<<<grid_for(rows * heads * half, 256), 256, 0, as_stream(stream)>>>(x, inv_freq, pos_or_null, out,
                                                                                      rows, heads, half);
  return (int)cudaGetLastError();
}

int wkb_rope_bf16(const void* x, const float* inv_freq, const int* pos, void* out, i64 rows, i64 heads, i64 half,
                  i64 row_stride, void* stream) {
  if (rows <= 0 || half <= 0 || heads <= 0) return 0;
  rope_bf16_kernel<<<grid_for(rows * heads * half, 256), 256, 0, as_stream(stream)>>>(
      (const u16*)x, inv_freq, pos, (u16*)out, rows, heads, half, row_stride);
  return (int)cudaGetLastError();
}

int wkb_embedding_f32(float* out, const float* weight, const int* ids, i64 t, i64 h, i64 v, void* stream) {
  if (t <= 0 || h <= 0) return 0;
  launch_pdl(embedding_kernel<float>, grid_for(t * h, 256), 256, 0, as_stream(stream), out, weight, ids, t, h, v < 0 ? 0 : v);
  return (int)cudaGetLastError();
}

int wkb_embed_tok_pos_bf16(float* out, const void* wte, const void* wpe, const int* ids, const int* pos, i64 t, i64 h,
                           i64 v, i64 npos, void* stream) {
  if (t <= 0 || h <= 0) return 0;
  launch_pdl(embed_tok_pos_kernel, grid_for(t * h, 256), 256, 0, as_stream(stream), out, (const u16*)wte, (const u16*)wpe, ids, pos, t, h, v,
             npos);
  return (int)cudaGetLastError();
}

int wkb_rowargmax_i32(const float* x, int* out, i64 rows, i64 cols, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  int grid = (int)(rows < (i64)WKB_SM_COUNT * 8 ? rows : (i64)WKB_SM_COUNT * 8);
  rowargmax_kernel<<<grid, 256, 0, as_stream(stream)>>>(x, out, rows, cols, cols);
  return (int)cudaGetLastError();
}

int wkb_rowargmax_strided_i32(const float* x, int* out, i64 rows, i64 cols, i64 ld, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  int grid = (int)(rows < (i64)WKB_SM_COUNT * 8 ? rows : (i64)WKB_SM_COUNT * 8);
  rowargmax_kernel<<<grid, 256, 0, as_stream(stream)>>>(x, out, rows, cols, ld);
  return (int)cudaGetLastError();
}

int wkb_decode_advance(int* row_token, int* row_pos, int* row_ctx, const int* next_tok, i64 n, i64 max_pos, void* stream) {
  if (n <= 0) return 0;
  if (max_pos < 0 || max_pos > 0x7ffffffe) max_pos = 0x7ffffffe;
  launch_pdl(decode_advance_kernel, (int)((n + 255) / 256), 256, 0, as_stream(stream), row_token, row_pos, row_ctx, next_tok, (int)n, (int)max_pos);
  return (int)cudaGetLastError();
}

// Host-side deadline on a stream (the counterpart of the reference's `sync_within`, crates/wukong_codegen_gpu/src/
// gpu.rs:250-262, :302, which turns a launch that does not finish into an error instead of a hung process): polls
// the stream without blocking in the driver.  0 = everything queued on the stream has completed; -1 = the deadline
// passed with work still in flight (the stream is left as it is: the caller decides whether to keep waiting, tear
// the context down or report); > 0 = the CUDA error the stream reported.
int wkb_stream_sync_within(void* stream, i64 timeout_ms) {
  const auto t0 = std::chrono::steady_clock::now();
  const auto limit = std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms);
  for (unsigned spins = 0;; ++spins) {
    const cudaError_t e = cudaStreamQuery(as_stream(stream));
    if (e == cudaSuccess) return 0;
    if (e != cudaErrorNotReady) return (int)e;
    if (std::chrono::steady_clock::now() - t0 >= limit) return -1;
    if (spins > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50));   // spin first: steps last ~2 ms
  }
}

// The live prefix of several equally long row vectors in one call: `height` runs of `width_bytes` bytes, `pitch_bytes` apart in
// both buffers, host (pinned) to device.  One driver call instead of one copy per vector: the per-call overhead was a visible
// part of a 1.8 ms serving step.
int wkb_upload_rows(void* dst_dev, const void* src_host, i64 pitch_bytes, i64 width_bytes, i64 height, void* stream) {
  if (width_bytes <= 0 || height <= 0) return 0;
  if (width_bytes > pitch_bytes) return (int)cudaErrorInvalidValue;
  return (int)cudaMemcpy2DAsync(dst_dev, (size_t)pitch_bytes, src_host, (size_t)pitch_bytes, (size_t)width_bytes, (size_t)height,
                                cudaMemcpyHostToDevice, as_stream(stream));
}

// Queues a kernel that occupies the stream for about `ms` milliseconds (clamped to [0, 2000]).
int wkb_device_sleep_ms(i64 ms, void* stream) {
  if (ms < 0) ms = 0;
  if (ms > 2000) ms = 2000;
  device_sleep_kernel<<<1, 1, 0, as_stream(stream)>>>((unsigned long long)ms * 1000000ull);
  return (int)cudaGetLastError();
}

int wkb_add_f32(const float* a, const float* b, float* out, i64 n, void* stream) {
  if (n <= 0) return 0;
  add_f32_kernel<<<grid_for(n, 256), 256, 0, as_stream(stream)>>>(a, b, out, n);
  return (int)cudaGetLastError();
}
}

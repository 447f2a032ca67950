// fp32-accumulate GEMM / GEMV under the reference's per-element order contract.
//
// gemm.rs:30-58 of the reference runtime: for each (i, j) K is cut into ceil(K/select_kc(K))
// blocks; a block is an ascending-p chain acc = fma(a, b, acc) from +0.0; the first block honours
// beta (a 0 / non-0 flag), later blocks add into C with one rounding; the epilogue
// act(alpha*x + bias[j]) runs once on the last block (gemm.rs:751-780).  A SIMT tiled GEMM keeps
// exactly this order per output element as long as K tiles never straddle a select_kc block, so
// the results are bit-identical to the CPU kernels for every transpose form and for half-storage
// operands (which widen losslessly; gemm.rs:1436-1480, gemv_half.rs:73-110).
//
// gemv.rs:28-88: the f32 GEMV instead uses four 8-lane accumulators over 32-element steps -- one
// warp lane per accumulator lane here -- with the fixed trees and an unfused scalar tail.
#include "common.cuh"
#include "wkb_device.h"

namespace wkb {

template <typename T> __device__ __forceinline__ float widen(T v);
template <> __device__ __forceinline__ float widen<float>(float v) { return v; }
struct bf16raw { u16 b; };
struct f16raw { u16 b; };
template <> __device__ __forceinline__ float widen<bf16raw>(bf16raw v) { return bf16_bits_to_f32(v.b); }
template <> __device__ __forceinline__ float widen<f16raw>(f16raw v) { return f16_bits_to_f32(v.b); }

__host__ __device__ inline i64 select_kc(i64 k) {
  i64 nblocks = (k + 383) / 384;
  if (nblocks < 1) nblocks = 1;
  i64 per = (k + nblocks - 1) / nblocks;
  return (per + 3) / 4 * 4;
}

constexpr int TM = 64, TN = 64, TK = 16;

template <typename TA, typename TB>
__global__ void __launch_bounds__(256) sgemm_contract_kernel(const TA* __restrict__ a, const TB* __restrict__ b,
                                                             float* c, i64 M, i64 K, i64 N, int beta, int at, int bt,
                                                             const float* __restrict__ bias, int act, float alpha,
                                                             int has_epi) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const i64 i0 = (i64)blockIdx.y * TM, j0 = (i64)blockIdx.x * TN;
  const i64 kcap = select_kc(K);
  float cval[4][4];
#pragma unroll
  for (int ii = 0; ii < 4; ++ii)
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) cval[ii][jj] = 0.0f;
  for (i64 pc = 0; pc < K; pc += kcap) {
    i64 kc = K - pc < kcap ? K - pc : kcap;
    float acc[4][4];
#pragma unroll
    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) acc[ii][jj] = 0.0f;
    for (i64 p0 = pc; p0 < pc + kc; p0 += TK) {
      int tk = (int)(pc + kc - p0 < TK ? pc + kc - p0 : TK);
      __syncthreads();
      for (int e = threadIdx.x; e < TK * TM; e += 256) {
        int kk, ii;
        if (at) { ii = e % TM; kk = e / TM; } else { kk = e % TK; ii = e / TK; }
        i64 gi = i0 + ii, gp = p0 + kk;
        float v = 0.0f;
        if (gi < M && kk < tk) v = widen<TA>(at ? a[gp * M + gi] : a[gi * K + gp]);
        As[kk][ii] = v;
      }
      for (int e = threadIdx.x; e < TK * TN; e += 256) {
        int kk, jj;
        if (bt) { kk = e % TK; jj = e / TK; } else { jj = e % TN; kk = e / TN; }
        i64 gj = j0 + jj, gp = p0 + kk;
        float v = 0.0f;
        if (gj < N && kk < tk) v = widen<TB>(bt ? b[gj * K + gp] : b[gp * N + gj]);
        Bs[kk][jj] = v;
      }
      __syncthreads();
      for (int kk = 0; kk < tk; ++kk) {
        float av[4], bv[4];
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) av[ii] = As[kk][ty * 4 + ii];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) bv[jj] = Bs[kk][tx * 4 + jj];
#pragma unroll
        for (int ii = 0; ii < 4; ++ii)
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) acc[ii][jj] = ffma(av[ii], bv[jj], acc[ii][jj]);
      }
    }
    bool first = pc == 0, last = pc + kc == K;
#pragma unroll
    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        i64 gi = i0 + ty * 4 + ii, gj = j0 + tx * 4 + jj;
        if (gi < M && gj < N) {
          float val;
          if (first) val = beta ? fadd(c[gi * N + gj], acc[ii][jj]) : acc[ii][jj];
          else val = fadd(cval[ii][jj], acc[ii][jj]);
          if (last && has_epi) {
            float y = (alpha != 1.0f) ? fmul(alpha, val) : val;
            if (bias) y = fadd(y, bias[gj]);
            val = act_apply(act, y);
          }
          cval[ii][jj] = val;
          if (last) c[gi * N + gj] = val;
        }
      }
  }
}

// f32 GEMV, y[i] = alpha * sum_j a[i, j] x[j]; one warp per row.
__global__ void __launch_bounds__(256) sgemv_exact_kernel(const float* __restrict__ a, const float* __restrict__ x,
                                                          float* __restrict__ y, i64 m, i64 n, float alpha) {
  int lane = threadIdx.x & 31;
  i64 warp = ((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = ((i64)gridDim.x * blockDim.x) >> 5;
  for (i64 i = warp; i < m; i += nw) {
    const float* row = a + i * n;
    float c = 0.0f;  // accumulator (lane / 8), vector lane (lane % 8)
    i64 j = 0;
    for (; j + 32 <= n; j += 32) c = ffma(row[j + lane], x[j + lane], c);
    for (; j + 8 <= n; j += 8)
      if (lane < 8) c = ffma(row[j + lane], x[j + lane], c);
    int l = lane & 7;
    float c0 = __shfl_sync(0xffffffffu, c, l), c1 = __shfl_sync(0xffffffffu, c, l + 8);
    float c2 = __shfl_sync(0xffffffffu, c, l + 16), c3 = __shfl_sync(0xffffffffu, c, l + 24);
    float v = fadd(fadd(c0, c1), fadd(c2, c3));
    float v0 = __shfl_sync(0xffffffffu, v, 0), v1 = __shfl_sync(0xffffffffu, v, 1);
    float v2 = __shfl_sync(0xffffffffu, v, 2), v3 = __shfl_sync(0xffffffffu, v, 3);
    float v4 = __shfl_sync(0xffffffffu, v, 4), v5 = __shfl_sync(0xffffffffu, v, 5);
    float v6 = __shfl_sync(0xffffffffu, v, 6), v7 = __shfl_sync(0xffffffffu, v, 7);
    float s = fadd(fadd(fadd(v0, v4), fadd(v1, v5)), fadd(fadd(v2, v6), fadd(v3, v7)));
    if (lane == 0) {
      for (; j < n; ++j) s = fadd(s, fmul(row[j], x[j]));
      y[i] = (alpha != 1.0f) ? fmul(s, alpha) : s;
    }
  }
}

template <typename TA, typename TB>
static int launch_gemm(const void* a, const void* b, float* c, i64 m, i64 k, i64 n, i64 beta, int at, int bt,
                       const float* bias, i64 act, float alpha, int has_epi, cudaStream_t st) {
  if (m <= 0 || k <= 0 || n <= 0) return 0;
  dim3 grid((unsigned)((n + TN - 1) / TN), (unsigned)((m + TM - 1) / TM));
  if (grid.y > 65535) return (int)cudaErrorInvalidValue;
  sgemm_contract_kernel<TA, TB><<<grid, 256, 0, st>>>((const TA*)a, (const TB*)b, c, m, k, n, beta != 0, at, bt, bias,
                                                      (int)act, alpha, has_epi);
  return (int)cudaGetLastError();
}

}  // namespace wkb

using namespace wkb;

extern "C" {

// a_dtype / b_dtype: 0 = f32, 1 = bf16 bits, 2 = f16 bits.
int wkb_sgemm_contract(const void* a, int a_dtype, const void* b, int b_dtype, float* c, i64 m, i64 k, i64 n,
                       i64 beta, int at, int bt, const float* bias, i64 act, float alpha, int has_epi, void* stream) {
  cudaStream_t st = as_stream(stream);
  if (a_dtype == 0 && b_dtype == 0) return launch_gemm<float, float>(a, b, c, m, k, n, beta, at, bt, bias, act, alpha, has_epi, st);
  if (a_dtype == 1 && b_dtype == 1) return launch_gemm<bf16raw, bf16raw>(a, b, c, m, k, n, beta, at, bt, bias, act, alpha, has_epi, st);
  if (a_dtype == 2 && b_dtype == 2) return launch_gemm<f16raw, f16raw>(a, b, c, m, k, n, beta, at, bt, bias, act, alpha, has_epi, st);
  if (a_dtype == 0 && b_dtype == 1) return launch_gemm<float, bf16raw>(a, b, c, m, k, n, beta, at, bt, bias, act, alpha, has_epi, st);
  if (a_dtype == 0 && b_dtype == 2) return launch_gemm<float, f16raw>(a, b, c, m, k, n, beta, at, bt, bias, act, alpha, has_epi, st);
  return (int)cudaErrorInvalidValue;
}

int wkb_sgemv_f32(const float* a, const float* x, float* y, i64 m, i64 n, float alpha, void* stream) {
  if (m <= 0 || n <= 0) return 0;
  i64 blocks = (m + 7) / 8;
  if (blocks > (i64)WKB_SM_COUNT * 8) blocks = (i64)WKB_SM_COUNT * 8;
  sgemv_exact_kernel<<<(int)blocks, 256, 0, as_stream(stream)>>>(a, x, y, m, n, alpha);
  return (int)cudaGetLastError();
}
}

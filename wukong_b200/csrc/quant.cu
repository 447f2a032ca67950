// GGML Q4_0 / Q8_0 block-quantised weights: packers, layout split, the weight-only quantised GEMV
// and group-wise int4 dequantisation.
//
// Reference semantics (crates/wukong_runtime/src/quant.rs): a 32-value block is a little-endian f16
// scale `d` followed by its quants; Q4_0 byte j holds element j (low nibble) and element j+16 (high
// nibble), value d*(nibble-8) (:13-16).  The GEMV quantises the activation per call to Q8 blocks
// with an exact f32 scale (:201-212), takes exact i32 block dots, and accumulates
// `acc = acc + (dw*dx)*f32(isum)` in block order with every operation rounded once (:21-37,
// :227-239).  `gemv_q_contract_kernel` reproduces exactly that, so y is bit-identical to the CPU
// kernel: dp4a gives the exact integer dots, and the float recurrence runs in block order.
//
// Device layout.  The raw rows are 18 (34) bytes per block, so nothing in them is 16-byte aligned.
// Resident weights are therefore held as two planes -- quants [N, nb] x 16 B (Q8: 32 B) and scales
// [N, nb] x f16 -- produced by a pure byte permutation (`split_kernel`); the algorithmic bytes per
// block are unchanged (18 / 34) and every nibble and scale bit survives, which the tests check.
#include "common.cuh"
#include "wkb_device.h"

namespace wkb {

// ---- layout split: raw [rows, nb*BB] bytes -> quant plane + scale plane -------------------------
template <int BB>
__global__ void __launch_bounds__(256) split_kernel(const u8* __restrict__ raw, u8* __restrict__ qs,
                                                    u16* __restrict__ d, i64 nblocks) {
  constexpr int QB = BB - 2;  // quant bytes per block
  i64 stride = (i64)gridDim.x * blockDim.x;
  // one thread per 2-byte unit of a block (BB/2 units: unit 0 is the scale)
  i64 units = nblocks * (BB / 2);
  for (i64 u = (i64)blockIdx.x * blockDim.x + threadIdx.x; u < units; u += stride) {
    i64 b = u / (BB / 2);
    int w = (int)(u % (BB / 2));
    u16 v = (u16)raw[b * BB + 2 * w] | ((u16)raw[b * BB + 2 * w + 1] << 8);
    if (w == 0) d[b] = v;
    else reinterpret_cast<u16*>(qs + b * QB)[w - 1] = v;
  }
}

// ---- activation quantiser (quant.rs:132-146, :201-212) ------------------------------------------
// One warp per block.  xq: [nb][32] int8 (zero padded), dx: [nb] f32, sx: [nb] i32 = sum of quants.
__global__ void __launch_bounds__(128) quantize_act_kernel(const float* __restrict__ x, i64 k, int8_t* __restrict__ xq,
                                                           float* __restrict__ dx, int* __restrict__ sx, i64 nb) {
  int lane = threadIdx.x & 31;
  i64 warp = ((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  i64 nwarps = ((i64)gridDim.x * blockDim.x) >> 5;
  for (i64 b = warp; b < nb; b += nwarps) {
    i64 e = b * 32 + lane;
    float v = e < k ? x[e] : 0.0f;
    float a = fabsf(v);
    if (a != a) a = 0.0f;  // `|x| > amax` is false for NaN
    float amax = warp_max(a);
    float dd = fdiv(amax, 127.0f);
    float id = dd != 0.0f ? fdiv(1.0f, dd) : 0.0f;
    float s = fmul(v, id);
    int q;
    if (s != s) q = 0;
    else {
      float r = roundf(s);  // half away from zero
      r = r < -127.0f ? -127.0f : (r > 127.0f ? 127.0f : r);
      q = (int)r;
    }
    if (e >= k) q = 0;
    xq[b * 32 + lane] = (int8_t)q;
    int tot = q;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    if (lane == 0) { dx[b] = dd; sx[b] = tot; }
  }
}

// ---- the contract GEMV ---------------------------------------------------------------------------
// A CTA of 8 warps owns 32 consecutive rows at a time, 4 per warp; lane l owns blocks l, l+32, ...  Per block: the
// exact integer dot by dp4a, the term (dw*dx)*f32(isum) with each product rounded once, parked in shared memory.
// Then ONE warp adds the 32 rows' terms in block order, a lane per row -- the part of the contract that cannot be
// re-associated: nb dependent adds, paid once per 32 rows with all 32 lanes busy and the loads issued eight ahead
// of the adds (it used to be paid per 4 rows by 4 lanes of every warp).
constexpr int GQ_RB = 4, GQ_WARPS = 8, GQ_ROWS = GQ_RB * GQ_WARPS;

template <bool Q4, int U>
__global__ void __launch_bounds__(GQ_WARPS * 32) gemv_q_contract_kernel(const uint4* __restrict__ qs, const u16* __restrict__ d,
                                                                        const int8_t* __restrict__ xq, const float* __restrict__ dx,
                                                                        const int* __restrict__ sx, float* __restrict__ y, i64 n,
                                                                        int nb) {
  extern __shared__ __align__(16) unsigned char smem[];
  // x words transposed: xs[w][b], w = 0..7 (32-bit word of the block's 32 quants)
  int* xs = reinterpret_cast<int*>(smem);
  float* dxs = reinterpret_cast<float*>(xs + 8 * nb);
  int* sxs = reinterpret_cast<int*>(dxs + nb);
  float* terms = reinterpret_cast<float*>(sxs + nb);      // [32 rows][nb]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int QW = Q4 ? 1 : 2;  // uint4 words per block
  // U: blocks per lane whose loads are in flight together (a pass covers 32 * U blocks of every row)
  const i64 nbatches = (n + GQ_ROWS - 1) / GQ_ROWS;
  uint4 wq[U][GQ_RB][QW];
  u16 dw[U][GQ_RB];
  // all the loads of a pass are issued before any of them is used: one trip to HBM per pass instead of one per block
  auto load_pass = [&](i64 r0, int b0) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int b = b0 + 32 * u;
      if (b < nb) {
#pragma unroll
        for (int r = 0; r < GQ_RB; ++r) {
          const i64 row = r0 + r < n ? r0 + r : n - 1;
          const uint4* p = qs + (row * nb + b) * QW;
#pragma unroll
          for (int h = 0; h < QW; ++h) wq[u][r][h] = p[h];
          dw[u][r] = d[row * nb + b];
        }
      }
    }
  };
  // the first pass of the first batch does not depend on the activations: its loads travel while x is staged
  const bool preloaded = (i64)blockIdx.x < nbatches && (i64)blockIdx.x * GQ_ROWS + warp * GQ_RB < n;
  if (preloaded) load_pass((i64)blockIdx.x * GQ_ROWS + warp * GQ_RB, lane);
  for (int i = threadIdx.x; i < nb * 8; i += blockDim.x) {
    int b = i >> 3, w = i & 7;
    xs[w * nb + b] = reinterpret_cast<const int*>(xq)[i];
  }
  for (int i = threadIdx.x; i < nb; i += blockDim.x) { dxs[i] = dx[i]; sxs[i] = sx[i]; }
  __syncthreads();
  for (i64 batch = blockIdx.x; batch < nbatches; batch += gridDim.x) {
    const i64 rbase = batch * GQ_ROWS;
    const i64 r0 = rbase + warp * GQ_RB;
    if (r0 < n) {
      for (int b0 = lane; b0 < nb; b0 += 32 * U) {
        if (!(preloaded && batch == (i64)blockIdx.x && b0 == lane)) load_pass(r0, b0);
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int b = b0 + 32 * u;
          if (b < nb) {
            int xw[8];
#pragma unroll
            for (int w = 0; w < 8; ++w) xw[w] = xs[w * nb + b];
            const float dxb = dxs[b];
            const int sxb = sxs[b];
#pragma unroll
            for (int r = 0; r < GQ_RB; ++r) {
              int isum = 0;
              if (Q4) {
                uint32_t ws[4] = {wq[u][r][0].x, wq[u][r][0].y, wq[u][r][0].z, wq[u][r][0].w};
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                  int lo = (int)(ws[w] & 0x0f0f0f0fu), hi = (int)((ws[w] >> 4) & 0x0f0f0f0fu);
                  isum = __dp4a(lo, xw[w], isum);       // elements 4w..4w+3
                  isum = __dp4a(hi, xw[w + 4], isum);   // elements 16+4w..16+4w+3
                }
                isum -= 8 * sxb;  // sum (nib-8)*x = sum nib*x - 8*sum x, all exact integers
              } else {
                uint32_t ws[8] = {wq[u][r][0].x, wq[u][r][0].y, wq[u][r][0].z, wq[u][r][0].w,
                                  wq[u][r][QW - 1].x, wq[u][r][QW - 1].y, wq[u][r][QW - 1].z, wq[u][r][QW - 1].w};
#pragma unroll
                for (int w = 0; w < 8; ++w) isum = __dp4a((int)ws[w], xw[w], isum);
              }
              float term = fmul(fmul(f16_bits_to_f32(dw[u][r]), dxb), (float)isum);
              terms[(warp * GQ_RB + r) * nb + b] = term;
            }
          }
        }
      }
    }
    __syncthreads();
    if (warp == 0 && rbase + lane < n) {
      const float* t = terms + lane * nb;
      float acc = 0.0f;
      int b = 0;
      for (; b + 8 <= nb; b += 8) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = t[b + e];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc = fadd(acc, v[e]);
      }
      for (; b < nb; ++b) acc = fadd(acc, t[b]);
      y[rbase + lane] = acc;
    }
    __syncthreads();
  }
}

// ---- packers (quant.rs:154-197): one thread per block, the scalar scan order --------------------
template <bool Q4>
__global__ void __launch_bounds__(128) quantize_kernel(const float* __restrict__ x, u8* __restrict__ q, i64 rows,
                                                       i64 k, i64 nb) {
  constexpr int BB = Q4 ? 18 : 34;
  i64 total = rows * nb;
  i64 stride = (i64)gridDim.x * blockDim.x;
  for (i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += stride) {
    i64 r = t / nb, b = t % nb;
    const float* xr = x + r * k;
    i64 lo = b * 32;
    int bl = (int)((lo + 32 < k ? lo + 32 : k) - lo);
    if (bl < 0) bl = 0;
    u8* o = q + t * BB;
    float amax = 0.0f, mx = 0.0f;
    for (int e = 0; e < bl; ++e) {
      float v = xr[lo + e];
      if (Q4) { if (amax < fabsf(v)) { amax = fabsf(v); mx = v; } }
      else    { if (fabsf(v) > amax) amax = fabsf(v); }
    }
    float dd = Q4 ? fdiv(mx, -8.0f) : fdiv(amax, 127.0f);
    float id = dd != 0.0f ? fdiv(1.0f, dd) : 0.0f;
    unsigned int h = (unsigned int)f32_to_f16_bits(dd);
    o[0] = (u8)(h & 0xffu);
    o[1] = (u8)((h >> 8) & 0xffu);
    if (Q4) {
      for (int j = 0; j < 16; ++j) {
        u8 nibs[2];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          int e = j + 16 * s;
          float v = fmul(e < bl ? xr[lo + e] : 0.0f, id);
          int iv;
          if (v != v) iv = 8;
          else {
            float tt = fadd(v, 8.5f);
            iv = tt >= 127.0f ? 127 : (tt <= -128.0f ? -128 : (int)tt);  // truncating, saturating cast
            if (iv > 15) iv = 15;
          }
          nibs[s] = (u8)(int8_t)iv;
        }
        o[2 + j] = (u8)(nibs[0] | (nibs[1] << 4));
      }
    } else {
      for (int e = 0; e < 32; ++e) {
        int qv = 0;
        if (e < bl) {
          float s = fmul(xr[lo + e], id);
          if (s == s) {
            float rr = roundf(s);
            rr = rr < -127.0f ? -127.0f : (rr > 127.0f ? 127.0f : rr);
            qv = (int)rr;
          }
        }
        o[2 + e] = (u8)(int8_t)qv;
      }
    }
  }
}

// ---- group-wise int4 (quant.rs:607-688) -----------------------------------------------------------
__global__ void __launch_bounds__(256) dequant_int4_kernel(const u8* __restrict__ q, const float* __restrict__ scale,
                                                           const float* __restrict__ zero, i64 group,
                                                           float* __restrict__ out, i64 n) {
  i64 stride = (i64)gridDim.x * blockDim.x;
  for (i64 i = (i64)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    u8 b = q[i >> 1];
    u8 nib = (i & 1) == 0 ? (b & 0x0f) : (b >> 4);
    float s = scale[i / group];
    float v;
    if (!zero) {
      int sv = (int)(int8_t)(nib << 4) >> 4;
      v = fmul((float)sv, s);
    } else {
      v = fmul(fsub((float)nib, zero[i / group]), s);
    }
    out[i] = v;
  }
}

// ---- scratch of the allocation-free GEMV entry ----------------------------------------------------
// The per-call Q8 activation (quants, block scales, block sums) lives in this fixed array instead of
// caller- or runtime-allocated memory.  Every GPU that loads the library holds it until exit.
constexpr i64 NOALLOC_MAX_K = 32768;
constexpr i64 NOALLOC_MAX_NB = NOALLOC_MAX_K / 32;
constexpr i64 NOALLOC_XQ_BYTES = NOALLOC_MAX_K;                // i8 quants
constexpr i64 NOALLOC_DX_OFF = NOALLOC_XQ_BYTES;               // f32 scales
constexpr i64 NOALLOC_SX_OFF = NOALLOC_DX_OFF + NOALLOC_MAX_NB * 4;  // i32 sums
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SX_OFF + NOALLOC_MAX_NB * 4];

static size_t contract_smem(int nb) { return (size_t)nb * (32 + 4 + 4) + (size_t)GQ_ROWS * nb * 4; }

// ---- y = W x, bf16 activation, every load issued before any arithmetic -----------------------------------------
// A GEMV of these sizes (9-25 MB of weights) lasts a few microseconds at HBM speed, so what matters is that the
// whole matrix is in flight at once: a warp owns R rows, a lane owns blocks lane, lane+32, ... of each, and all of
// a pass's 16-byte block loads (and scale loads) are issued first; x (8-22 KB, L2-resident) is read straight from
// global by the lane that needs it, 64 B per block, with no shared-memory staging and no barrier.
// Per block: sum_e (16 + nib_e) * x_e in f32 (the nibble becomes the mantissa of 16 + nib, exact), minus 24 * sum_e x_e,
// times the f16 scale.
template <int R, int BPL>
__global__ void __launch_bounds__(128, 4) gemv_q4_lean_kernel(const uint4* __restrict__ qs, const u16* __restrict__ d,
                                                           const uint4* __restrict__ xb, float* __restrict__ y, i64 n, int nb, i64 k) {
  const int lane = threadIdx.x & 31;
  const i64 warp = ((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const i64 r0 = warp * R;
  if (r0 >= n) return;
  float acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = 0.0f;
  for (int b0 = 0; b0 < nb; b0 += 32 * BPL) {
    uint4 wq[R][BPL];
    u16 dw[R][BPL];
    uint4 xv[BPL][4];
#pragma unroll
    for (int i = 0; i < BPL; ++i) {
      const int b = min(b0 + lane + 32 * i, nb - 1);
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const i64 row = r0 + r < n ? r0 + r : n - 1;
        wq[r][i] = __ldcs(qs + row * nb + b);
        dw[r][i] = d[row * nb + b];
      }
    }
#pragma unroll
    for (int i = 0; i < BPL; ++i) {
      const int b = min(b0 + lane + 32 * i, nb - 1);
      if ((i64)(b + 1) * 32 <= k) {
#pragma unroll
        for (int c = 0; c < 4; ++c) xv[i][c] = xb[(i64)b * 4 + c];
      } else {
        // ragged last block: elements past k count as zero
        const u16* xs = reinterpret_cast<const u16*>(xb);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t ww[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const i64 i0 = (i64)b * 32 + 8 * c + 2 * e;
            ww[e] = (i0 < k ? (uint32_t)xs[i0] : 0u) | ((i0 + 1 < k ? (uint32_t)xs[i0 + 1] : 0u) << 16);
          }
          xv[i][c] = make_uint4(ww[0], ww[1], ww[2], ww[3]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < BPL; ++i) {
      const bool live = b0 + lane + 32 * i < nb;
      float xf[32];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t ww[4] = {xv[i][c].x, xv[i][c].y, xv[i][c].z, xv[i][c].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { xf[8 * c + 2 * e] = u2f(ww[e] << 16); xf[8 * c + 2 * e + 1] = u2f(ww[e] & 0xffff0000u); }
      }
      float sx = 0.0f;
#pragma unroll
      for (int e = 0; e < 32; ++e) sx += xf[e];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint32_t words[4] = {wq[r][i].x, wq[r][i].y, wq[r][i].z, wq[r][i].w};
        float part = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w)
#pragma unroll
          for (int p = 0; p < 8; ++p) {
            const int e = 4 * w + (p >> 1) + ((p & 1) ? 16 : 0);   // nibble p of word w is element e of the block
            const int sh = 19 - 4 * p;
            const uint32_t pos = sh >= 0 ? (words[w] << sh) : (words[w] >> (-sh));
            part = fmaf(u2f((pos & 0x00780000u) | 0x41800000u), xf[e], part);
          }
        const float term = f16_bits_to_f32(dw[r][i]) * (part - 24.0f * sx);
        acc[r] += live ? term : 0.0f;
      }
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const float v = warp_sum(acc[r]);
    if (lane == 0 && r0 + r < n) y[r0 + r] = v;
  }
}

}  // namespace wkb

using namespace wkb;

extern "C" {

int wkb_q_split(const u8* raw, void* qs, void* d, i64 nblocks, int q4, void* stream) {
  if (nblocks <= 0) return 0;
  i64 units = nblocks * (q4 ? 9 : 17);
  int grid = (int)((units + 255) / 256 < (i64)WKB_SM_COUNT * 16 ? (units + 255) / 256 : (i64)WKB_SM_COUNT * 16);
  if (q4) split_kernel<18><<<grid, 256, 0, as_stream(stream)>>>(raw, (u8*)qs, (u16*)d, nblocks);
  else split_kernel<34><<<grid, 256, 0, as_stream(stream)>>>(raw, (u8*)qs, (u16*)d, nblocks);
  return (int)cudaGetLastError();
}

int wkb_quantize_act(const float* x, i64 k, void* xq, float* dx, int* sx, void* stream) {
  i64 nb = (k + 31) / 32;
  if (nb <= 0) return 0;
  int grid = (int)((nb + 3) / 4 < (i64)WKB_SM_COUNT * 8 ? (nb + 3) / 4 : (i64)WKB_SM_COUNT * 8);
  quantize_act_kernel<<<grid, 128, 0, as_stream(stream)>>>(x, k, (int8_t*)xq, dx, sx, nb);
  return (int)cudaGetLastError();
}

// y = W x under the reference contract.  qs/d are the split planes; xq/dx/sx come from
// wkb_quantize_act.  Bit-identical to the CPU kernel.
int wkb_gemv_q_contract(const void* qs, const void* d, const void* xq, const float* dx, const int* sx, float* y,
                        i64 n, i64 k, int q4, void* stream) {
  if (n <= 0 || k <= 0) return 0;
  int nb = (int)((k + 31) / 32);
  size_t sm = contract_smem(nb);
  if (sm > 200 * 1024) return (int)cudaErrorInvalidValue;
  i64 blocks = (n + GQ_ROWS - 1) / GQ_ROWS;
  if (blocks > (i64)WKB_SM_COUNT * 8) blocks = (i64)WKB_SM_COUNT * 8;
  // a grid that fits the machine once keeps 4 blocks per lane in flight (one trip to HBM for a 4096-wide row); a larger one
  // runs more CTAs per SM on half the registers
  const bool deep = q4 && blocks <= (i64)WKB_SM_COUNT;
  auto kern = q4 ? (deep ? gemv_q_contract_kernel<true, 4> : gemv_q_contract_kernel<true, 2>) : gemv_q_contract_kernel<false, 2>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  if (e != cudaSuccess) return (int)e;
  kern<<<(int)blocks, GQ_WARPS * 32, sm, as_stream(stream)>>>((const uint4*)qs, (const u16*)d, (const int8_t*)xq, dx, sx, y, n, nb);
  return (int)cudaGetLastError();
}

int wkb_gemv_q4_0_bf16x(const void* qs, const void* d, const void* x_bf16, float* y, i64 n, i64 k, void* stream) {
  if (n <= 0 || k <= 0) return 0;
  if ((((uintptr_t)qs) | ((uintptr_t)x_bf16)) & 15) return (int)cudaErrorMisalignedAddress;
  const int nb = (int)((k + 31) / 32);
  // two rows per warp; few rows: one row per warp so that the grid still covers the SMs
  const bool one = n < (i64)WKB_SM_COUNT * 16;
  const i64 warps = one ? n : (n + 1) / 2;
  // CTAs of four warps held to 128 registers: four are resident per SM, so that 4096 rows (512 CTAs) are one wave
  const i64 blocks = (warps + 3) / 4;
  if (one) gemv_q4_lean_kernel<1, 4><<<(int)blocks, 128, 0, as_stream(stream)>>>((const uint4*)qs, (const u16*)d, (const uint4*)x_bf16, y, n, nb, k);
  else gemv_q4_lean_kernel<2, 4><<<(int)blocks, 128, 0, as_stream(stream)>>>((const uint4*)qs, (const u16*)d, (const uint4*)x_bf16, y, n, nb, k);
  return (int)cudaGetLastError();
}

int wkb_quantize_q(const float* x, u8* q, i64 rows, i64 k, int q4, void* stream) {
  if (rows <= 0 || k <= 0) return 0;
  i64 nb = (k + 31) / 32, total = rows * nb;
  int grid = (int)((total + 127) / 128 < (i64)WKB_SM_COUNT * 16 ? (total + 127) / 128 : (i64)WKB_SM_COUNT * 16);
  if (q4) quantize_kernel<true><<<grid, 128, 0, as_stream(stream)>>>(x, q, rows, k, nb);
  else quantize_kernel<false><<<grid, 128, 0, as_stream(stream)>>>(x, q, rows, k, nb);
  return (int)cudaGetLastError();
}

int wkb_dequant_int4(const u8* q, const float* scale, const float* zero_or_null, i64 group, float* out, i64 n,
                     void* stream) {
  if (n <= 0) return 0;
  int grid = (int)((n + 255) / 256 < (i64)WKB_SM_COUNT * 16 ? (n + 255) / 256 : (i64)WKB_SM_COUNT * 16);
  dequant_int4_kernel<<<grid, 256, 0, as_stream(stream)>>>(q, scale, zero_or_null, group, out, n);
  return (int)cudaGetLastError();
}

// y = W x for resident Q4_0 weights, bit-identical to wkb_gemv_q_contract, for callers that cannot
// allocate device memory (a runtime that owns every byte of its arena up front, a plug-in called
// inside someone else's memory-managed region, code running where a cudaMalloc would synchronise the
// device at the wrong moment).  The Q8 activation scratch is the library's fixed device array, so
// K is limited to 32768.  The first call on each device looks the array's device address up (make it
// before any stream capture starts); no call allocates or frees anything.  All calls share the one
// array: it is fully rewritten by each call (nothing needs to start at zero), and two calls whose
// kernels overlap on the GPU -- different streams, or different host threads -- race on it.
int wkb_gemv_q4_0_f32_noalloc(const void* qs, const void* d, const float* x, float* y, i64 n, i64 k, void* stream) {
  if (n <= 0 || k <= 0) return 0;
  if (k > NOALLOC_MAX_K) {
    fprintf(stderr, "wkb_gemv_q4_0_f32_noalloc: K = %lld exceeds the fixed scratch (max %lld); use wkb_gemv_q_contract\n",
            (long long)k, (long long)NOALLOC_MAX_K);
    return (int)cudaErrorInvalidValue;
  }
  static unsigned char* base[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
  if (!base[dev]) {
    // the array's name is a host-side stand-in here; this is its address on the current device
    unsigned char* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    base[dev] = p;
  }
  unsigned char* s = base[dev];
  int rc = wkb_quantize_act(x, k, s, reinterpret_cast<float*>(s + NOALLOC_DX_OFF), reinterpret_cast<int*>(s + NOALLOC_SX_OFF), stream);
  if (rc) return rc;
  return wkb_gemv_q_contract(qs, d, s, reinterpret_cast<const float*>(s + NOALLOC_DX_OFF),
                             reinterpret_cast<const int*>(s + NOALLOC_SX_OFF), y, n, k, 1, stream);
}
}

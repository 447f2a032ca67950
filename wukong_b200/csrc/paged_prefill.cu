// Paged prefill attention: many query tokens of one sequence against the paged bf16 KV cache (causal, GQA).
//
// The reference's counterpart is its flash prefill over the paged cache (crates/wukong_codegen_gpu/src/ptx_flash.rs,
// chunked prefill of crates/wukong_codegen_gpu/src/serving.rs:1346-1595): the tokens of a prompt chunk attend to
// everything already in the sequence's pages plus the chunk's own earlier tokens.  The decode kernel treats every
// query token as a row of its own and streams that row's keys once per row; here a warp owns a TILE of 16 / G
// consecutive query tokens of one sequence (G = query heads per KV head) and streams the keys once per tile, so a
// prompt chunk reads its keys 16 / G times less often.
//
// One warp = (tile, kv head).  The 16 rows of the tensor-core A operand are (token, head-of-group) pairs,
// token-major.  Per 16 keys: scores = q . K^T on mma.sync m16n8k16 (q split into bf16 hi + lo so the scores carry
// ~16 bits, K fragments are 128-bit loads from the page with a fixed dim permutation that is applied to q as well),
// masked per row by that row's visible-key count, online softmax in base 2 (the weights are rounded to bf16 and the
// normaliser sums the rounded weights), then out += P . V with V fragments byte-permuted from two token rows.
// Every index depends on the LOGICAL key position only, so the page layout cannot change a bit of the result.
// Algorithmic bytes per (tile, kv head, key) = 2 * head_dim * 2; the kernel is bound by L2 / HBM for long contexts
// and by the legacy tensor path for short ones.
#include "common.cuh"
#include "wkb_device.h"

namespace wkb {

int paged_attn_prefill_tc(const float*, i64, const void*, const void*, const uint32_t*, const int*, const int*, const int*, i64, void*, int, i64, i64,
                          i64, i64, i64, float, cudaStream_t);

struct PrefillGeo {
  int n_tiles, q_heads, kv_heads, page_tokens, page_shift, mbps;
  i64 q_row_stride, out_row_stride;
};

__device__ __forceinline__ void mma_bf16_full(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pf_pack2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t pf_perm(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

constexpr int PF_WARPS = 4;
constexpr int PF_SUBS = 8;   // 16-row sub-tiles of a 128-row tile

template <int HD, int G>
__global__ void __launch_bounds__(PF_WARPS * 32, HD == 64 ? 3 : 1) paged_attn_prefill_kernel(
    const float* __restrict__ q, const uint4* __restrict__ kcache, const uint4* __restrict__ vcache,
    const uint32_t* __restrict__ block_table, const int* __restrict__ row_slot, const int* __restrict__ row_ctx,
    const int2* __restrict__ tiles, void* __restrict__ out, int out_dtype, PrefillGeo g, float scale_log2e) {
  constexpr int LPT = HD / 8;      // uint4 per token row
  constexpr int NJ = HD / 32;      // 32-dim groups of the score contraction
  constexpr int NSL = HD / 64;     // 64-dim slabs of the output
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gi = lane >> 2, t = lane & 3;
  // a caller's tile holds up to 128 / G rows; a warp takes one of its PF_SUBS sub-tiles of 16 / G rows
  const i64 unit = (i64)blockIdx.x * PF_WARPS + warp;
  if (unit >= (i64)g.n_tiles * PF_SUBS * g.kv_heads) return;
  const int kvh = (int)(unit % g.kv_heads);
  const i64 ts = unit / g.kv_heads;
  const int2 tile = tiles[ts / PF_SUBS];
  const int sub = (int)(ts % PF_SUBS);
  const int row0 = tile.x + sub * (16 / G), nrows = min(min(tile.y, 128 / G) - sub * (16 / G), 16 / G);
  if (nrows <= 0) return;
  // this lane's two A rows: (token, head-of-group) = (a / G, a % G) for a = gi and gi + 8
  int tok[2], hd[2], ctx[2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int a = gi + 8 * rr;
    tok[rr] = a / G;
    hd[rr] = kvh * G + a % G;
    ctx[rr] = tok[rr] < nrows ? min(row_ctx[row0 + tok[rr]], g.mbps * g.page_tokens) : 0;
  }
  int kmax = max(ctx[0], ctx[1]);
  kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, 4));
  kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, 8));
  kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, 16));
  if (kmax <= 0) return;
  const int last_tok = kmax - 1;
  const uint32_t* bt = block_table + (i64)row_slot[row0] * g.mbps;
  const i64 page_units = (i64)g.kv_heads * g.page_tokens * LPT;
  const i64 head_off = (i64)kvh * g.page_tokens * LPT;
  auto row_index = [&](int key) {   // uint4 index of the first 8 dims of a (clamped) key's row
    key = min(key, last_tok);
    return (i64)bt[key >> g.page_shift] * page_units + head_off + (i64)(key & (g.page_tokens - 1)) * LPT;
  };
  // query fragments of both rows: k-steps (j, h), bf16 hi and lo of q * scale * log2(e)
  uint32_t qh[2][NJ][2][2], ql[2][NJ][2][2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr)
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      float f[8];
      if (tok[rr] < nrows) {
        const float* qp = q + (i64)(row0 + tok[rr]) * g.q_row_stride + (i64)hd[rr] * HD + 32 * j + 8 * t;
        const float4 a = *reinterpret_cast<const float4*>(qp), b = *reinterpret_cast<const float4*>(qp + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = 0.0f;
      }
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const float x0 = f[4 * h + 2 * c] * scale_log2e, x1 = f[4 * h + 2 * c + 1] * scale_log2e;
          const uint32_t hi = pf_pack2(x0, x1);
          qh[rr][j][h][c] = hi;
          ql[rr][j][h][c] = pf_pack2(x0 - u2f(hi << 16), x1 - u2f(hi & 0xffff0000u));
        }
    }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float acc[NSL][8][4];
#pragma unroll
  for (int sl = 0; sl < NSL; ++sl)
#pragma unroll
    for (int jj = 0; jj < 8; ++jj)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[sl][jj][c] = 0.0f;

  auto load_k = [&](int tile0, uint4 (&kw)[2][NJ]) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const i64 base = row_index(tile0 + 8 * u + gi);
#pragma unroll
      for (int j = 0; j < NJ; ++j) kw[u][j] = kcache[base + 4 * j + t];
    }
  };
  uint4 kcur[2][NJ];
  load_k(0, kcur);
  for (int tile0 = 0; tile0 < kmax; tile0 += 16) {
    // this tile's V rows (keys 2t, 2t+1, 2t+8, 2t+9; dims 64*sl + 8*gi .. +8)
    uint4 vw[4][NSL];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const i64 base = row_index(tile0 + 2 * t + (a & 1) + 8 * (a >> 1));
#pragma unroll
      for (int sl = 0; sl < NSL; ++sl) vw[a][sl] = vcache[base + 8 * sl + gi];
    }
    // ---- scores: sc[u] = rows {gi, gi + 8} x keys tile0 + 8u + 2t + {0, 1}
    float sc[2][4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
#pragma unroll
      for (int c = 0; c < 4; ++c) sc[u][c] = 0.0f;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const uint32_t kr[4] = {kcur[u][j].x, kcur[u][j].y, kcur[u][j].z, kcur[u][j].w};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          mma_bf16_full(sc[u], qh[0][j][h][0], qh[1][j][h][0], qh[0][j][h][1], qh[1][j][h][1], kr[2 * h], kr[2 * h + 1]);
          mma_bf16_full(sc[u], ql[0][j][h][0], ql[1][j][h][0], ql[0][j][h][1], ql[1][j][h][1], kr[2 * h], kr[2 * h + 1]);
        }
      }
    }
    if (tile0 + 16 < kmax) load_k(tile0 + 16, kcur);   // the next tile's K rows travel during the softmax and P.V
    uint32_t pa[2][2];   // [row][u]: the row's weights of keys 8u + 2t + {0, 1}
    float corr[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      float s4[4];
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int c = 0; c < 2; ++c) s4[2 * u + c] = (tile0 + 8 * u + 2 * t + c < ctx[rr]) ? sc[u][2 * rr + c] : -INFINITY;
      float tm = fmaxf(fmaxf(s4[0], s4[1]), fmaxf(s4[2], s4[3]));
      tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
      tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
      const float mn = fmaxf(m[rr], tm);
      const float ms = mn == -INFINITY ? 0.0f : mn;    // a row that sees no key yet: weights 0, nothing rescaled
      corr[rr] = exp2f(m[rr] - ms);
      m[rr] = mn;
      pa[rr][0] = pf_pack2(exp2f(s4[0] - ms), exp2f(s4[1] - ms));
      pa[rr][1] = pf_pack2(exp2f(s4[2] - ms), exp2f(s4[3] - ms));
      l[rr] = l[rr] * corr[rr] + ((u2f(pa[rr][0] << 16) + u2f(pa[rr][0] & 0xffff0000u)) + (u2f(pa[rr][1] << 16) + u2f(pa[rr][1] & 0xffff0000u)));
    }
#pragma unroll
    for (int sl = 0; sl < NSL; ++sl)
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        acc[sl][jj][0] *= corr[0]; acc[sl][jj][1] *= corr[0];
        acc[sl][jj][2] *= corr[1]; acc[sl][jj][3] *= corr[1];
      }
    // ---- values: two keys of one dim per B register
#pragma unroll
    for (int sl = 0; sl < NSL; ++sl) {
      const uint32_t x0[4] = {vw[0][sl].x, vw[0][sl].y, vw[0][sl].z, vw[0][sl].w};   // key 2t
      const uint32_t x1[4] = {vw[1][sl].x, vw[1][sl].y, vw[1][sl].z, vw[1][sl].w};   // key 2t+1
      const uint32_t y0[4] = {vw[2][sl].x, vw[2][sl].y, vw[2][sl].z, vw[2][sl].w};   // key 2t+8
      const uint32_t y1[4] = {vw[3][sl].x, vw[3][sl].y, vw[3][sl].z, vw[3][sl].w};   // key 2t+9
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        mma_bf16_full(acc[sl][2 * e], pa[0][0], pa[1][0], pa[0][1], pa[1][1], pf_perm(x0[e], x1[e], 0x5410u), pf_perm(y0[e], y1[e], 0x5410u));
        mma_bf16_full(acc[sl][2 * e + 1], pa[0][0], pa[1][0], pa[0][1], pa[1][1], pf_perm(x0[e], x1[e], 0x7632u), pf_perm(y0[e], y1[e], 0x7632u));
      }
    }
  }
  // ---- lane (gi, t) owns dims [64*sl + 16*t, +16) of rows gi and gi + 8: value 2*rr of pair jj is dim +jj, 2*rr + 1 is dim +8+jj
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    float lt = l[rr] + __shfl_xor_sync(0xffffffffu, l[rr], 1);
    lt += __shfl_xor_sync(0xffffffffu, lt, 2);
    if (tok[rr] >= nrows || ctx[rr] <= 0) continue;
    const float inv = 1.0f / lt;
    const i64 o = (i64)(row0 + tok[rr]) * g.out_row_stride + (i64)hd[rr] * HD;
#pragma unroll
    for (int sl = 0; sl < NSL; ++sl) {
      float v[16];
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) { v[jj] = acc[sl][jj][2 * rr] * inv; v[8 + jj] = acc[sl][jj][2 * rr + 1] * inv; }
      const i64 at = o + 64 * sl + 16 * t;
      if (out_dtype == 0) {
        float4* d = reinterpret_cast<float4*>(static_cast<float*>(out) + at);
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) d[k4] = make_float4(v[4 * k4], v[4 * k4 + 1], v[4 * k4 + 2], v[4 * k4 + 3]);
      } else {
        uint4* d = reinterpret_cast<uint4*>(static_cast<u16*>(out) + at);
        d[0] = make_uint4(pf_pack2(v[0], v[1]), pf_pack2(v[2], v[3]), pf_pack2(v[4], v[5]), pf_pack2(v[6], v[7]));
        d[1] = make_uint4(pf_pack2(v[8], v[9]), pf_pack2(v[10], v[11]), pf_pack2(v[12], v[13]), pf_pack2(v[14], v[15]));
      }
    }
  }
}

template <int HD, int G>
static int launch_prefill(const float* q, const void* kc, const void* vc, const uint32_t* bt, const int* row_slot, const int* row_ctx,
                          const int* tiles, void* out, int out_dtype, PrefillGeo g, float scale, cudaStream_t st) {
  const i64 units = (i64)g.n_tiles * PF_SUBS * g.kv_heads;
  const i64 blocks = (units + PF_WARPS - 1) / PF_WARPS;
  if (blocks > 0x7fffffff) return (int)cudaErrorInvalidValue;
  paged_attn_prefill_kernel<HD, G><<<(unsigned)blocks, PF_WARPS * 32, 0, st>>>(
      q, (const uint4*)kc, (const uint4*)vc, bt, row_slot, row_ctx, (const int2*)tiles, out, out_dtype, g, scale * 1.4426950408889634f);
  return (int)cudaGetLastError();
}

}  // namespace wkb

using namespace wkb;

extern "C" {

// Query tokens per tile: the 128 rows of the tensor-core operand hold (token, head-of-group) pairs.
i64 wkb_paged_attn_prefill_tile_rows(i64 q_heads, i64 kv_heads) {
  if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0) return 0;
  const i64 G = q_heads / kv_heads;
  return (G == 1 || G == 2 || G == 4 || G == 8) ? 128 / G : 0;
}

int wkb_paged_attn_prefill(const float* q, i64 q_row_stride, const void* kcache, const void* vcache, const uint32_t* block_table,
                           const int* row_slot, const int* row_ctx, const int* tiles, i64 n_tiles, void* out, int out_dtype,
                           i64 out_row_stride, i64 q_heads, i64 kv_heads, i64 head_dim, i64 page_tokens, i64 max_blocks_per_seq,
                           float scale, void* stream) {
  if (n_tiles <= 0) return 0;
  if (wkb_paged_attn_prefill_tile_rows(q_heads, kv_heads) == 0) return (int)cudaErrorInvalidValue;
  if (page_tokens < 4 || (page_tokens & (page_tokens - 1)) != 0 || n_tiles > 0x7fffffff) return (int)cudaErrorInvalidValue;
  int page_shift = 0;
  while ((1 << page_shift) < page_tokens) ++page_shift;
  if ((q_row_stride % 4) != 0 || ((((uintptr_t)q) | ((uintptr_t)kcache) | ((uintptr_t)vcache)) & 15) != 0 || (((uintptr_t)tiles) & 7) != 0)
    return (int)cudaErrorMisalignedAddress;
  if (out_row_stride % 8 != 0 || (((uintptr_t)out) & 15) != 0 || (out_dtype != 0 && out_dtype != 1)) return (int)cudaErrorMisalignedAddress;
  PrefillGeo g{(int)n_tiles, (int)q_heads, (int)kv_heads, (int)page_tokens, page_shift, (int)max_blocks_per_seq, q_row_stride, out_row_stride};
  const int G = (int)(q_heads / kv_heads);
  cudaStream_t st = as_stream(stream);
  // 16-token pages: both contractions on tcgen05, K / V pages landed by TMA; other page sizes: the mma.sync kernel
  static const bool use_tc = [] { const char* e = getenv("WKB_PREFILL_TC"); return !(e && e[0] == '0'); }();
  if (page_tokens == 16 && use_tc && (head_dim == 64 || head_dim == 128))
    return paged_attn_prefill_tc(q, q_row_stride, kcache, vcache, block_table, row_slot, row_ctx, tiles, n_tiles, out, out_dtype, out_row_stride,
                                 q_heads, kv_heads, head_dim, max_blocks_per_seq, scale, st);
#define WKB_PF_CASE(HD_, G_) \
  if (head_dim == HD_ && G == G_) return launch_prefill<HD_, G_>(q, kcache, vcache, block_table, row_slot, row_ctx, tiles, out, out_dtype, g, scale, st);
  WKB_PF_CASE(64, 1) WKB_PF_CASE(64, 2) WKB_PF_CASE(64, 4) WKB_PF_CASE(64, 8)
  WKB_PF_CASE(128, 1) WKB_PF_CASE(128, 2) WKB_PF_CASE(128, 4) WKB_PF_CASE(128, 8)
#undef WKB_PF_CASE
  return (int)cudaErrorInvalidValue;
}

}  // extern "C"

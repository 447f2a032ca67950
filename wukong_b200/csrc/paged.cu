// Paged KV cache: append (scatter through the block table) and single-query GQA decode attention.
//
// Behaviour follows the reference's GPU serving stack (crates/wukong_codegen_gpu/src/paged_kv.rs
// :84-151 geometry, :428-628 block table; paged_attention.rs:395-534 decode, :1343-1410 append):
// a padded row-major block table [slots, max_blocks_per_seq] of u32 physical pages, per-row context
// lengths, query head h reads KV head h / (q_heads / kv_heads), a row with no visible key gives a
// zero row, inactive rows never scatter.  The kernels themselves are new.
//
// HBM layout (this library's own): per layer, K and V slabs of bf16
//     [num_pages][kv_heads][page_tokens][head_dim]
// so one (page, head) is a single contiguous page_tokens*head_dim*2-byte run (2 KiB at d=64, 4 KiB at
// d=128) and a warp step reads 512 contiguous bytes.
//
// Decode kernel.  The unit of work is (row, kv head, 128-token chunk of the logical sequence), one
// warp each.  A lane owns 8 head dims (one 128-bit load) of one token; 32/(d/8) tokens per step.
// Partial dots are reduce-scattered so each lane ends up owning one token's score; softmax runs in
// base 2 on those; each lane then accumulates its 8 output dims over its tokens.  All query heads
// of a GQA group share each K/V load.  Chunk boundaries and every reduction tree depend on the
// LOGICAL token position only, so two physical page layouts of the same history give identical
// bits.  A second kernel merges a row's chunks in ascending order.
//
// Both are HBM-bound: algorithmic bytes per (row, kv head, token) = 2 * head_dim * 2.
#include "common.cuh"
#include "wkb_device.h"

namespace wkb {

constexpr int PA_CHUNK_MIN = 128;   // smallest split of the logical sequence (sizes the scratch)
constexpr int PA_WARPS = 4;

__device__ __forceinline__ void unpack8(const uint4& w, float f[8]) {
  f[0] = u2f(w.x << 16); f[1] = u2f(w.x & 0xffff0000u);
  f[2] = u2f(w.y << 16); f[3] = u2f(w.y & 0xffff0000u);
  f[4] = u2f(w.z << 16); f[5] = u2f(w.z & 0xffff0000u);
  f[6] = u2f(w.w << 16); f[7] = u2f(w.w & 0xffff0000u);
}

struct PagedGeo {
  int rows, q_heads, kv_heads, page_tokens, page_shift, mbps, max_chunks, chunk_tokens;
  i64 q_row_stride;
};

// scratch layout: [row][q_head][chunk] x (HD + 4) floats: acc[HD], m, l, 2 pad (keeps records 16-byte aligned)
template <int HD, int G>
__global__ void __launch_bounds__(PA_WARPS * 32) paged_attn_decode_kernel(
    const float* __restrict__ q, const uint4* __restrict__ kcache, const uint4* __restrict__ vcache,
    const uint32_t* __restrict__ block_table, const int* __restrict__ row_slot, const int* __restrict__ row_ctx,
    float* __restrict__ scratch, PagedGeo g, float scale_log2e) {
  constexpr int LPT = HD / 8;       // lanes per token
  constexpr int TPW = 32 / LPT;     // tokens per warp step
  constexpr int STEPS = LPT;        // steps per tile (so the reduce-scatter is square)
  constexpr int TILE = STEPS * TPW; // 32 tokens
  constexpr bool PREFETCH_V = (HD == 64) || (G <= 2);
  constexpr bool DOUBLE_BUFFER = (HD == 64 && G <= 2) || (HD == 128 && G == 1);
  static_assert(TILE == 32, "tile is one token per lane");
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = lane / LPT, j = lane % LPT;
  const i64 unit = (i64)blockIdx.x * PA_WARPS + warp;
  const i64 units = (i64)g.rows * g.kv_heads * g.max_chunks;
  if (unit >= units) return;
  // chunk is the slowest-varying index: CTAs of a late chunk are (almost) all empty and retire at
  // once instead of pinning idle warps beside busy ones
  const int chunk = (int)(unit / ((i64)g.rows * g.kv_heads));
  const int kvh = (int)(unit % g.kv_heads);
  const int row = (int)((unit / g.kv_heads) % g.rows);
  const int ctx = row_ctx[row];
  const int t0 = chunk * g.chunk_tokens;
  float* sbase = scratch + (((i64)row * g.q_heads + (i64)kvh * G) * g.max_chunks + chunk) * (HD + 4);
  const i64 head_stride = (i64)g.max_chunks * (HD + 4);
  if (t0 >= ctx) {  // nothing visible in this chunk: mark it empty
    if (lane < G) { float* s = sbase + lane * head_stride; s[HD] = -INFINITY; s[HD + 1] = 0.0f; }
    return;
  }
  const int t1 = min(ctx, t0 + g.chunk_tokens);
  const uint32_t* bt = block_table + (i64)row_slot[row] * g.mbps;
  // this lane's 8 query dims for each head of the group, pre-scaled by scale*log2(e)
  float qv[G][8];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    const float* qp = q + (i64)row * g.q_row_stride + ((i64)kvh * G + h) * HD + j * 8;
    float4 a = *reinterpret_cast<const float4*>(qp), b = *reinterpret_cast<const float4*>(qp + 4);
    qv[h][0] = a.x * scale_log2e; qv[h][1] = a.y * scale_log2e; qv[h][2] = a.z * scale_log2e; qv[h][3] = a.w * scale_log2e;
    qv[h][4] = b.x * scale_log2e; qv[h][5] = b.y * scale_log2e; qv[h][6] = b.z * scale_log2e; qv[h][7] = b.w * scale_log2e;
  }
  float m[G], l[G], acc[G][8];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    m[h] = -INFINITY; l[h] = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[h][e] = 0.0f;
  }
  const i64 page_units = (i64)g.kv_heads * g.page_tokens * LPT;  // uint4 per page
  const i64 head_off = (i64)kvh * g.page_tokens * LPT;
  // Tokens past the visible end are clamped onto the last visible token: their loads are real
  // (finite) data and their weight is forced to zero, which keeps the loops free of branches.
  const int last_tok = t1 - 1;
  const int last_page = last_tok >> g.page_shift;
  // Issue every K (and, when registers allow, V) load of one 32-token tile.  The tile's page ids (at
  // most 8 for 4-token pages) are fetched by the first lanes in one go and handed out by shuffle, so
  // no K/V load waits on its own table lookup.
  auto load_tile = [&](int tile0, uint4 (&kw)[STEPS], uint4 (&vw)[PREFETCH_V ? STEPS : 1], uint32_t& my_page) {
    const int first_page = tile0 >> g.page_shift;
    my_page = bt[min(first_page + (lane & 7), last_page)];
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      int tok = min(tile0 + s * TPW + grp, last_tok);
      uint32_t page = __shfl_sync(0xffffffffu, my_page, (tok >> g.page_shift) - first_page);
      i64 idx = (i64)page * page_units + head_off + (i64)(tok & (g.page_tokens - 1)) * LPT + j;
      kw[s] = kcache[idx];
      if (PREFETCH_V) vw[PREFETCH_V ? s : 0] = vcache[idx];
    }
  };
  auto compute_tile = [&](int tile0, uint4 (&kw)[STEPS], uint4 (&vw)[PREFETCH_V ? STEPS : 1], uint32_t my_page) {
    const int first_page = tile0 >> g.page_shift;
    (void)first_page; (void)my_page;
    // ---- scores: partial dots of this lane's 8 dims, for token (s*TPW + grp) at each step s
    float part[G][STEPS];
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      float kf[8];
      unpack8(kw[s], kf);
#pragma unroll
      for (int h = 0; h < G; ++h) {
        float d = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) d = fmaf(qv[h][e], kf[e], d);
        part[h][s] = d;
      }
    }
    // ---- reduce-scatter over the LPT lanes of a token: lane j ends with the full dot of step j
#pragma unroll
    for (int hh = STEPS / 2; hh >= 1; hh >>= 1) {
      bool upper = (j & hh) != 0;
#pragma unroll
      for (int h = 0; h < G; ++h) {
#pragma unroll
        for (int i = 0; i < hh; ++i) {
          float send = upper ? part[h][i] : part[h][i + hh];
          float keep = upper ? part[h][i + hh] : part[h][i];
          part[h][i] = keep + __shfl_xor_sync(0xffffffffu, send, hh);
        }
      }
    }
    // lane (grp, j) now owns token tile0 + j*TPW + grp
    int mytok = tile0 + j * TPW + grp;
    bool mine = mytok < t1;
    float p[G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
      float s = mine ? part[h][0] : -INFINITY;
      float tm = warp_max(s);
      float mn = fmaxf(m[h], tm);  // finite: the tile has at least one visible token
      float corr = exp2f(m[h] - mn);
      p[h] = exp2f(s - mn);
      l[h] = l[h] * corr + p[h];   // per-lane partial sum; lanes are combined at the end
      m[h] = mn;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[h][e] *= corr;
    }
    // ---- values: acc[dims of this lane] += p(token) * v(token)
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      uint4 vcur;
      if (PREFETCH_V) {
        vcur = vw[PREFETCH_V ? s : 0];
      } else {
        int tok = min(tile0 + s * TPW + grp, last_tok);
        uint32_t page = __shfl_sync(0xffffffffu, my_page, (tok >> g.page_shift) - first_page);
        vcur = vcache[(i64)page * page_units + head_off + (i64)(tok & (g.page_tokens - 1)) * LPT + j];
      }
      float vf[8];
      unpack8(vcur, vf);
#pragma unroll
      for (int h = 0; h < G; ++h) {
        float pt = __shfl_sync(0xffffffffu, p[h], grp * LPT + s);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[h][e] = fmaf(pt, vf[e], acc[h][e]);
      }
    }
  };
  if constexpr (DOUBLE_BUFFER) {
    // Two register buffers: the next tile's loads are in flight while the current tile is reduced.
    uint4 kwA[STEPS], vwA[PREFETCH_V ? STEPS : 1], kwB[STEPS], vwB[PREFETCH_V ? STEPS : 1];
    uint32_t pgA = 0, pgB = 0;
    load_tile(t0, kwA, vwA, pgA);
    for (int tile0 = t0; tile0 < t1; tile0 += 2 * TILE) {
      if (tile0 + TILE < t1) load_tile(tile0 + TILE, kwB, vwB, pgB);
      compute_tile(tile0, kwA, vwA, pgA);
      if (tile0 + TILE < t1) {
        if (tile0 + 2 * TILE < t1) load_tile(tile0 + 2 * TILE, kwA, vwA, pgA);
        compute_tile(tile0 + TILE, kwB, vwB, pgB);
      }
    }
  } else {
    uint4 kw[STEPS], vw[PREFETCH_V ? STEPS : 1];
    uint32_t pg = 0;
    for (int tile0 = t0; tile0 < t1; tile0 += TILE) {
      load_tile(tile0, kw, vw, pg);
      compute_tile(tile0, kw, vw, pg);
    }
  }
  // ---- combine the token groups (fixed xor tree over the group bits), then the lane sums of l
#pragma unroll
  for (int h = 0; h < G; ++h) {
#pragma unroll
    for (int ofs = LPT; ofs < 32; ofs <<= 1) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[h][e] += __shfl_xor_sync(0xffffffffu, acc[h][e], ofs);
    }
    float lt = warp_sum(l[h]);
    float* s = sbase + h * head_stride;
    if (grp == 0) {
      *reinterpret_cast<float4*>(s + j * 8) = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
      *reinterpret_cast<float4*>(s + j * 8 + 4) = make_float4(acc[h][4], acc[h][5], acc[h][6], acc[h][7]);
    }
    if (lane == 0) { s[HD] = m[h]; s[HD + 1] = lt; }
  }
}

// Merge a row-head's chunks in ascending order; out_dtype 0 = f32, 1 = bf16.
template <int HD>
__global__ void __launch_bounds__(128) paged_attn_merge_kernel(const float* __restrict__ scratch, void* __restrict__ out,
                                                               int out_dtype, i64 out_row_stride,
                                                               const int* __restrict__ row_ctx, int rows, int q_heads,
                                                               int max_chunks, int chunk_tokens) {
  i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  i64 total = (i64)rows * q_heads * (HD / 4);
  if (idx >= total) return;
  int dq = (int)(idx % (HD / 4));
  i64 rh = idx / (HD / 4);
  int row = (int)(rh / q_heads), h = (int)(rh % q_heads);
  int ctx = row_ctx[row];
  int nch = ctx <= 0 ? 0 : (ctx + chunk_tokens - 1) / chunk_tokens;
  if (nch > max_chunks) nch = max_chunks;
  const float* s = scratch + rh * (i64)max_chunks * (HD + 4);
  float mm = -INFINITY;
  for (int c = 0; c < nch; ++c) mm = fmaxf(mm, s[(i64)c * (HD + 4) + HD]);
  float lsum = 0.0f;
  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c = 0; c < nch; ++c) {
    const float* sc = s + (i64)c * (HD + 4);
    float w = exp2f(sc[HD] - mm);
    lsum = fmaf(sc[HD + 1], w, lsum);
    float4 a = *reinterpret_cast<const float4*>(sc + dq * 4);
    o.x = fmaf(a.x, w, o.x); o.y = fmaf(a.y, w, o.y); o.z = fmaf(a.z, w, o.z); o.w = fmaf(a.w, w, o.w);
  }
  float inv = lsum != 0.0f ? 1.0f / lsum : 0.0f;
  o.x *= inv; o.y *= inv; o.z *= inv; o.w *= inv;
  i64 off = (i64)row * out_row_stride + (i64)h * HD + dq * 4;
  if (out_dtype == 0) {
    *reinterpret_cast<float4*>((float*)out + off) = o;
  } else {
    uint2 pk;
    pk.x = (uint32_t)f32_to_bf16_bits(o.x) | ((uint32_t)f32_to_bf16_bits(o.y) << 16);
    pk.y = (uint32_t)f32_to_bf16_bits(o.z) | ((uint32_t)f32_to_bf16_bits(o.w) << 16);
    *reinterpret_cast<uint2*>((u16*)out + off) = pk;
  }
}

// Scatter new K/V rows (f32, rounded to bf16) into their pages.  One thread per 8 dims.
// Rows with row_pos < 0 are inactive and write nothing.
__global__ void __launch_bounds__(256) paged_kv_append_kernel(const float* __restrict__ ksrc, const float* __restrict__ vsrc,
                                                              i64 src_row_stride, u16* __restrict__ kcache,
                                                              u16* __restrict__ vcache, const uint32_t* __restrict__ block_table,
                                                              const int* __restrict__ row_slot, const int* __restrict__ row_pos,
                                                              int rows, int kv_heads, int hd, int page_tokens, int mbps) {
  int per_row = kv_heads * hd / 8;
  i64 total = (i64)rows * per_row;
  i64 stride = (i64)gridDim.x * blockDim.x;
  for (i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    int row = (int)(idx / per_row), c = (int)(idx % per_row);
    int pos = row_pos[row];
    if (pos < 0) continue;
    int head = (c * 8) / hd, d0 = (c * 8) % hd;
    uint32_t page = block_table[(i64)row_slot[row] * mbps + pos / page_tokens];
    i64 dst = (((i64)page * kv_heads + head) * page_tokens + pos % page_tokens) * hd + d0;
    const float* ks = ksrc + (i64)row * src_row_stride + c * 8;
    const float* vs = vsrc + (i64)row * src_row_stride + c * 8;
    uint32_t kw[4], vw[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      kw[e] = (uint32_t)f32_to_bf16_bits(ks[2 * e]) | ((uint32_t)f32_to_bf16_bits(ks[2 * e + 1]) << 16);
      vw[e] = (uint32_t)f32_to_bf16_bits(vs[2 * e]) | ((uint32_t)f32_to_bf16_bits(vs[2 * e + 1]) << 16);
    }
    *reinterpret_cast<uint4*>(kcache + dst) = make_uint4(kw[0], kw[1], kw[2], kw[3]);
    *reinterpret_cast<uint4*>(vcache + dst) = make_uint4(vw[0], vw[1], vw[2], vw[3]);
  }
}

template <int HD, int G>
static int launch_decode(const float* q, const void* kc, const void* vc, const uint32_t* bt, const int* row_slot,
                         const int* row_ctx, float* scratch, void* out, int out_dtype, i64 out_row_stride, PagedGeo g,
                         float scale, cudaStream_t st) {
  i64 units = (i64)g.rows * g.kv_heads * g.max_chunks;
  i64 blocks = (units + PA_WARPS - 1) / PA_WARPS;
  if (blocks > 0x7fffffff) return (int)cudaErrorInvalidValue;
  paged_attn_decode_kernel<HD, G><<<(unsigned)blocks, PA_WARPS * 32, 0, st>>>(
      q, (const uint4*)kc, (const uint4*)vc, bt, row_slot, row_ctx, scratch, g, scale * 1.4426950408889634f);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  i64 total = (i64)g.rows * g.q_heads * (HD / 4);
  paged_attn_merge_kernel<HD><<<(unsigned)((total + 127) / 128), 128, 0, st>>>(scratch, out, out_dtype, out_row_stride,
                                                                                row_ctx, g.rows, g.q_heads, g.max_chunks, g.chunk_tokens);
  return (int)cudaGetLastError();
}

}  // namespace wkb

using namespace wkb;

extern "C" {

i64 wkb_paged_attn_scratch_bytes(i64 rows, i64 q_heads, i64 head_dim, i64 max_ctx) {
  i64 chunks = (max_ctx + PA_CHUNK_MIN - 1) / PA_CHUNK_MIN;   // worst case: the smallest split
  if (chunks < 1) chunks = 1;
  return rows * q_heads * chunks * (head_dim + 4) * 4;
}

int wkb_paged_attn_decode(const float* q, i64 q_row_stride, const void* kcache, const void* vcache,
                          const uint32_t* block_table, const int* row_slot, const int* row_ctx, void* out,
                          int out_dtype, i64 out_row_stride, i64 rows, i64 q_heads, i64 kv_heads, i64 head_dim,
                          i64 page_tokens, i64 max_blocks_per_seq, i64 max_ctx, float scale, float* scratch,
                          void* stream) {
  if (rows <= 0) return 0;
  if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0) return (int)cudaErrorInvalidValue;
  if (page_tokens < 4 || (page_tokens & (page_tokens - 1)) != 0) return (int)cudaErrorInvalidValue;  // power of two, >= 4
  int page_shift = 0;
  while ((1 << page_shift) < page_tokens) ++page_shift;
  if ((q_row_stride % 4) != 0 || ((((uintptr_t)q) | ((uintptr_t)scratch) | ((uintptr_t)kcache) | ((uintptr_t)vcache)) & 15) != 0)
    return (int)cudaErrorMisalignedAddress;
  if (out_row_stride % 4 != 0 || (((uintptr_t)out) & 15) != 0) return (int)cudaErrorMisalignedAddress;
  // How finely a sequence is split depends on the launch shape only (never on the data): few
  // (row, kv head) pairs need the split for parallelism, many pairs are better off amortising the
  // per-unit set-up over longer runs.
  // Aim for about 4096 units at full context, between 128 and 512 tokens each.
  i64 want = rows * kv_heads * (max_ctx > 0 ? max_ctx : 1) / 4096;
  int chunk_tokens = PA_CHUNK_MIN;
  while (chunk_tokens < 512 && chunk_tokens * 2 <= want) chunk_tokens *= 2;
  i64 chunks = (max_ctx + chunk_tokens - 1) / chunk_tokens;
  if (chunks < 1) chunks = 1;
  PagedGeo g{(int)rows, (int)q_heads, (int)kv_heads, (int)page_tokens, page_shift, (int)max_blocks_per_seq, (int)chunks, chunk_tokens, q_row_stride};
  int G = (int)(q_heads / kv_heads);
  cudaStream_t st = as_stream(stream);
#define WKB_PA_CASE(HD_, G_) \
  if (head_dim == HD_ && G == G_) return launch_decode<HD_, G_>(q, kcache, vcache, block_table, row_slot, row_ctx, scratch, out, out_dtype, out_row_stride, g, scale, st);
  WKB_PA_CASE(64, 1) WKB_PA_CASE(64, 2) WKB_PA_CASE(64, 4)
  WKB_PA_CASE(128, 1) WKB_PA_CASE(128, 2) WKB_PA_CASE(128, 4) WKB_PA_CASE(128, 8)
#undef WKB_PA_CASE
  return (int)cudaErrorInvalidValue;
}

int wkb_paged_kv_append(const float* ksrc, const float* vsrc, i64 src_row_stride, void* kcache, void* vcache,
                        const uint32_t* block_table, const int* row_slot, const int* row_pos, i64 rows, i64 kv_heads,
                        i64 head_dim, i64 page_tokens, i64 max_blocks_per_seq, void* stream) {
  if (rows <= 0) return 0;
  if (head_dim % 8 != 0) return (int)cudaErrorInvalidValue;
  i64 total = rows * kv_heads * head_dim / 8;
  i64 blocks = (total + 255) / 256;
  if (blocks > (i64)WKB_SM_COUNT * 16) blocks = (i64)WKB_SM_COUNT * 16;
  paged_kv_append_kernel<<<(int)blocks, 256, 0, as_stream(stream)>>>(ksrc, vsrc, src_row_stride, (u16*)kcache, (u16*)vcache,
                                                                     block_table, row_slot, row_pos, (int)rows, (int)kv_heads,
                                                                     (int)head_dim, (int)page_tokens, (int)max_blocks_per_seq);
  return (int)cudaGetLastError();
}
}

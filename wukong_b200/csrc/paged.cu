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
#include "tc_common.cuh"

namespace wkb {

constexpr int PA_CHUNK_MIN = 128;   // smallest split of the logical sequence (sizes the scratch)
constexpr int PA_WARPS = 4;
int* gemm_status_word();   // the library's device status word (gemm_tc.cu)

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
    float* __restrict__ scratch, PagedGeo g, float scale_log2e, void* __restrict__ out, int out_dtype, i64 out_row_stride) {
  // out != nullptr: the launch has one chunk per row, so the unit normalises and writes the row itself (the arithmetic
  // of the merge kernel for a single chunk) and no scratch record or merge launch is needed
  constexpr int LPT = HD / 8;       // lanes per token
  constexpr int TPW = 32 / LPT;     // tokens per warp step
  constexpr int STEPS = LPT;        // steps per tile (so the reduce-scatter is square)
  constexpr int TILE = STEPS * TPW; // 32 tokens
  constexpr bool PREFETCH_V = (HD == 64) || (G <= 2);
  constexpr bool DOUBLE_BUFFER = (HD == 64 && G <= 2) || (HD == 128 && G == 1);
  static_assert(TILE == 32, "tile is one token per lane");
  pdl_wait();
  pdl_trigger();
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
  const int ctx = min(row_ctx[row], g.mbps * g.page_tokens);   // never walk past the block-table row
  const int t0 = chunk * g.chunk_tokens;
  float* sbase = scratch + (((i64)row * g.q_heads + (i64)kvh * G) * g.max_chunks + chunk) * (HD + 4);
  const i64 head_stride = (i64)g.max_chunks * (HD + 4);
  auto write_row = [&](int h, const float (&v)[8]) {   // 8 dims j*8.. of head kvh*G + h, by the lanes of token group 0
    const i64 off = (i64)row * out_row_stride + ((i64)kvh * G + h) * HD + j * 8;
    if (out_dtype == 0) {
      float4* d = reinterpret_cast<float4*>(static_cast<float*>(out) + off);
      d[0] = make_float4(v[0], v[1], v[2], v[3]);
      d[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      uint4 pk;
      pk.x = (uint32_t)f32_to_bf16_bits(v[0]) | ((uint32_t)f32_to_bf16_bits(v[1]) << 16);
      pk.y = (uint32_t)f32_to_bf16_bits(v[2]) | ((uint32_t)f32_to_bf16_bits(v[3]) << 16);
      pk.z = (uint32_t)f32_to_bf16_bits(v[4]) | ((uint32_t)f32_to_bf16_bits(v[5]) << 16);
      pk.w = (uint32_t)f32_to_bf16_bits(v[6]) | ((uint32_t)f32_to_bf16_bits(v[7]) << 16);
      *reinterpret_cast<uint4*>(static_cast<u16*>(out) + off) = pk;
    }
  };
  if (t0 >= ctx) {  // nothing visible in this chunk: mark it empty
    if (out) {
      const float zero[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (grp == 0)
        for (int h = 0; h < G; ++h) write_row(h, zero);
    } else if (lane < G) { float* s = sbase + lane * head_stride; s[HD] = -INFINITY; s[HD + 1] = 0.0f; }
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
    if (out) {
      const float inv = lt != 0.0f ? 1.0f / lt : 0.0f;
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = acc[h][e] * inv;
      if (grp == 0) write_row(h, v);
      continue;
    }
    float* s = sbase + h * head_stride;
    if (grp == 0) {
      *reinterpret_cast<float4*>(s + j * 8) = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
      *reinterpret_cast<float4*>(s + j * 8 + 4) = make_float4(acc[h][4], acc[h][5], acc[h][6], acc[h][7]);
    }
    if (lane == 0) { s[HD] = m[h]; s[HD + 1] = lt; }
  }
}

// ---- the same unit of work with K / V staged in shared memory by asynchronous bulk copies ---------------------
// The register kernel above keeps its bytes in flight in registers (two tile buffers, 185 registers, 8 warps per SM)
// and every unit starts with a serial chain row -> block table -> first tile during which its warp streams nothing.
// Here a (page, kv head) run -- 16 tokens x head_dim bf16, one contiguous 2 or 4 KiB piece of HBM -- is brought in by
// ONE cp.async.bulk issued by lane 0 (global -> this CTA's shared memory, completion counted on an mbarrier; never a
// multicast, never another GPU's memory), into a ring of NST tile slots per warp.  A tile is 32 tokens = two pages of
// K and two of V.  Bytes in flight cost shared memory instead of registers (NST x 8 KiB per warp at head_dim 64), the
// warp needs ~80 registers, and the arithmetic, the reduction trees and therefore the output bits are those of the
// register kernel.  Warps are independent (own ring, own barriers, no __syncthreads), so ragged context lengths cost
// nothing beyond the launch tail.  Every barrier wait is bounded; a wait that runs out records
// WKB_STATUS_ATTN_WAIT, waits (bounded) for the copies still in flight and leaves the unit unwritten.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <int HD, int G, int NST, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) paged_attn_decode_staged_kernel(
    const float* __restrict__ q, const uint8_t* __restrict__ kcache, const uint8_t* __restrict__ vcache,
    const uint32_t* __restrict__ block_table, const int* __restrict__ row_slot, const int* __restrict__ row_ctx,
    float* __restrict__ scratch, PagedGeo g, float scale_log2e, void* __restrict__ out, int out_dtype, i64 out_row_stride,
    int* __restrict__ status) {
  constexpr int LPT = HD / 8, TPW = 32 / LPT, STEPS = LPT, TILE = 32;
  constexpr int ROW_BYTES = HD * 2, PAGE_BYTES = 16 * ROW_BYTES, STAGE_BYTES = 4 * PAGE_BYTES;   // K a, K b, V a, V b
  extern __shared__ __align__(128) uint8_t pa_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = lane / LPT, j = lane % LPT;
  const uint32_t ring = smem_u32(pa_smem) + (uint32_t)warp * (NST * STAGE_BYTES);
  const uint32_t bars = smem_u32(pa_smem) + (uint32_t)WARPS * (NST * STAGE_BYTES) + (uint32_t)warp * (NST * 8);
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NST; ++s) mbar_init(bars + 8u * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  pdl_wait();
  pdl_trigger();
  const i64 unit = (i64)blockIdx.x * WARPS + warp;
  const i64 units = (i64)g.rows * g.kv_heads * g.max_chunks;
  if (unit >= units) return;
  const int chunk = (int)(unit / ((i64)g.rows * g.kv_heads));
  const int kvh = (int)(unit % g.kv_heads);
  const int row = (int)((unit / g.kv_heads) % g.rows);
  const int ctx = min(row_ctx[row], g.mbps * g.page_tokens);
  const int t0 = chunk * g.chunk_tokens;
  float* sbase = scratch + (((i64)row * g.q_heads + (i64)kvh * G) * g.max_chunks + chunk) * (HD + 4);
  const i64 head_stride = (i64)g.max_chunks * (HD + 4);
  auto write_row = [&](int h, const float (&v)[8]) {
    const i64 off = (i64)row * out_row_stride + ((i64)kvh * G + h) * HD + j * 8;
    if (out_dtype == 0) {
      float4* d = reinterpret_cast<float4*>(static_cast<float*>(out) + off);
      d[0] = make_float4(v[0], v[1], v[2], v[3]);
      d[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      uint4 pk;
      pk.x = (uint32_t)f32_to_bf16_bits(v[0]) | ((uint32_t)f32_to_bf16_bits(v[1]) << 16);
      pk.y = (uint32_t)f32_to_bf16_bits(v[2]) | ((uint32_t)f32_to_bf16_bits(v[3]) << 16);
      pk.z = (uint32_t)f32_to_bf16_bits(v[4]) | ((uint32_t)f32_to_bf16_bits(v[5]) << 16);
      pk.w = (uint32_t)f32_to_bf16_bits(v[6]) | ((uint32_t)f32_to_bf16_bits(v[7]) << 16);
      *reinterpret_cast<uint4*>(static_cast<u16*>(out) + off) = pk;
    }
  };
  if (t0 >= ctx) {  // nothing visible in this chunk (no copy has been issued yet)
    if (out) {
      const float zero[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (grp == 0)
        for (int h = 0; h < G; ++h) write_row(h, zero);
    } else if (lane < G) { float* s = sbase + lane * head_stride; s[HD] = -INFINITY; s[HD + 1] = 0.0f; }
    return;
  }
  const int t1 = min(ctx, t0 + g.chunk_tokens);
  const int ntiles = (t1 - t0 + TILE - 1) / TILE;
  const uint32_t* bt = block_table + (i64)row_slot[row] * g.mbps;
  const int first_page = t0 >> 4, last_page = (t1 - 1) >> 4;
  // page ids of the unit, 32 at a time in the lanes (a window of 16 tiles); handed to lane 0 by shuffle
  uint32_t my_page = bt[min(first_page + lane, last_page)];
  const i64 page_stride = (i64)g.kv_heads * PAGE_BYTES;
  const i64 head_off = (i64)kvh * PAGE_BYTES;
  // issue the copies of tile i into its ring slot (all lanes take part in the shuffles, lane 0 issues)
  auto issue = [&](int i) {
    const int tile0 = t0 + i * TILE;
    const int pa = (tile0 >> 4) - first_page;                 // page index inside the unit
    const uint32_t pg_a = __shfl_sync(0xffffffffu, my_page, pa & 31);
    const uint32_t pg_b = __shfl_sync(0xffffffffu, my_page, (pa + 1) & 31);
    if (lane == 0) {
      const int na = min(16, t1 - tile0), nb = min(16, max(0, t1 - tile0 - 16));   // visible tokens in the two pages
      const uint32_t slot = ring + (uint32_t)(i % NST) * STAGE_BYTES, bar = bars + 8u * (i % NST);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the slot's last readers (generic proxy) are done
      mbar_expect_tx(bar, (uint32_t)(na + nb) * ROW_BYTES * 2);
      const i64 src_a = (i64)pg_a * page_stride + head_off;
      bulk_g2s(slot, kcache + src_a, (uint32_t)na * ROW_BYTES, bar);
      bulk_g2s(slot + 2 * PAGE_BYTES, vcache + src_a, (uint32_t)na * ROW_BYTES, bar);
      if (nb > 0) {
        const i64 src_b = (i64)pg_b * page_stride + head_off;
        bulk_g2s(slot + PAGE_BYTES, kcache + src_b, (uint32_t)nb * ROW_BYTES, bar);
        bulk_g2s(slot + 3 * PAGE_BYTES, vcache + src_b, (uint32_t)nb * ROW_BYTES, bar);
      }
    }
  };
  const int pre = min(NST, ntiles);
  for (int i = 0; i < pre; ++i) issue(i);
  // this lane's 8 query dims for each head of the group, pre-scaled by scale*log2(e) (these loads overlap the copies)
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
  bool ok = true;
  int issued = pre;
  for (int i = 0; i < ntiles; ++i) {
    const int tile0 = t0 + i * TILE;
    if (!mbar_wait(bars + 8u * (i % NST), (uint32_t)((i / NST) & 1))) { ok = false; break; }
    const uint32_t slot = ring + (uint32_t)(i % NST) * STAGE_BYTES;
    // tokens past the visible end are clamped onto the last visible token of the tile (real, finite data in the slot)
    // and their weight is forced to zero
    const int last_local = min(TILE, t1 - tile0) - 1;
    // ---- scores
    float part[G][STEPS];
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      const int tl = min(s * TPW + grp, last_local);
      uint4 kw;
      asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(kw.x), "=r"(kw.y), "=r"(kw.z), "=r"(kw.w)
                   : "r"(slot + (uint32_t)tl * ROW_BYTES + (uint32_t)j * 16u));
      float kf[8];
      unpack8(kw, kf);
#pragma unroll
      for (int h = 0; h < G; ++h) {
        float d = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) d = fmaf(qv[h][e], kf[e], d);
        part[h][s] = d;
      }
    }
#pragma unroll
    for (int hh = STEPS / 2; hh >= 1; hh >>= 1) {
      bool upper = (j & hh) != 0;
#pragma unroll
      for (int h = 0; h < G; ++h) {
#pragma unroll
        for (int ii = 0; ii < hh; ++ii) {
          float send = upper ? part[h][ii] : part[h][ii + hh];
          float keep = upper ? part[h][ii + hh] : part[h][ii];
          part[h][ii] = keep + __shfl_xor_sync(0xffffffffu, send, hh);
        }
      }
    }
    const int mytok = tile0 + j * TPW + grp;
    const bool mine = mytok < t1;
    float p[G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
      float s = mine ? part[h][0] : -INFINITY;
      float tm = warp_max(s);
      float mn = fmaxf(m[h], tm);
      float corr = exp2f(m[h] - mn);
      p[h] = exp2f(s - mn);
      l[h] = l[h] * corr + p[h];
      m[h] = mn;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[h][e] *= corr;
    }
    // ---- values
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      const int tl = min(s * TPW + grp, last_local);
      uint4 vw;
      asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(vw.x), "=r"(vw.y), "=r"(vw.z), "=r"(vw.w)
                   : "r"(slot + 2u * PAGE_BYTES + (uint32_t)tl * ROW_BYTES + (uint32_t)j * 16u));
      float vf[8];
      unpack8(vw, vf);
#pragma unroll
      for (int h = 0; h < G; ++h) {
        float pt = __shfl_sync(0xffffffffu, p[h], grp * LPT + s);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[h][e] = fmaf(pt, vf[e], acc[h][e]);
      }
    }
    __syncwarp();                       // every lane has read the slot
    if (i + NST < ntiles) {
      if (((i + NST) & 15) == 0) {      // the next window of page ids (32 pages = 16 tiles)
        const int base_page = first_page + 2 * (i + NST);
        my_page = bt[min(base_page + lane, last_page)];
      }
      issue(i + NST);
      ++issued;
    }
  }
  if (!ok) {
    if (lane == 0) atomicExch(status, WKB_STATUS_ATTN_WAIT);
    // the copies still in flight target this CTA's shared memory: wait for them (bounded) before the warp leaves
    for (int i2 = 0; i2 < issued; ++i2)
      if (i2 + NST >= issued) mbar_wait(bars + 8u * (i2 % NST), (uint32_t)((i2 / NST) & 1));
    return;
  }
#pragma unroll
  for (int h = 0; h < G; ++h) {
#pragma unroll
    for (int ofs = LPT; ofs < 32; ofs <<= 1) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[h][e] += __shfl_xor_sync(0xffffffffu, acc[h][e], ofs);
    }
    float lt = warp_sum(l[h]);
    if (out) {
      const float inv = lt != 0.0f ? 1.0f / lt : 0.0f;
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = acc[h][e] * inv;
      if (grp == 0) write_row(h, v);
      continue;
    }
    float* s = sbase + h * head_stride;
    if (grp == 0) {
      *reinterpret_cast<float4*>(s + j * 8) = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
      *reinterpret_cast<float4*>(s + j * 8 + 4) = make_float4(acc[h][4], acc[h][5], acc[h][6], acc[h][7]);
    }
    if (lane == 0) { s[HD] = m[h]; s[HD + 1] = lt; }
  }
}

// ---- tensor-core variant for head_dim 128 with a GQA group of 2..8 query heads ------------------------------
// At a group of 4 the lane-per-8-dims kernel above spends ~3 lane-instructions per KV byte (unpack + 4 heads of
// FMAs + the reduce-scatter) and is bound by instruction issue at half the HBM rate.  Here the same unit of work
// (row, kv head, chunk) per warp runs on mma.sync.m16n8k16 (bf16 x bf16 -> f32): the group's query heads are the
// rows of the A operand, and the K / V fragments are exactly what 128-bit loads bring in:
//   scores  S[head, token] : B fragment of lane (g, t) = K[token 8u+g][dims 32j+8t+4h .. +4]; the dim order inside a
//           k-step is a fixed permutation applied to q as well (a dot product does not care).  q is split into
//           bf16 hi + lo so the scores carry ~16 bits.
//   output  O[head, dim]   : A fragment = the tile's probabilities straight from the S accumulators (rounded to bf16,
//           and the same rounded values feed the normaliser); B fragment (tokens x dims) needs two tokens of one dim in
//           a register: two byte-permutes of the rows of tokens 2t, 2t+1 loaded for dims 64s+8g..+8.
// Lane (g, t) ends up owning dims [64s+16t, +16) of head g.  Everything is indexed by logical token position.
// D(rows 0-7) += A(rows 0-7) . B for an A operand whose rows 8-15 are zero: only c0 / c1 are live accumulators, the
// lower half of the result is discarded.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[2], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  float z0, z1;
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %5}, {%7, %8}, {%0, %1, %9, %9};"
               : "+f"(d[0]), "+f"(d[1]), "=f"(z0), "=f"(z1) : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1), "f"(0.0f));
}
// The same instruction with the hi parts of the A operand in rows 0-7 (registers a0, a2) and the lo parts in rows 8-15
// (a1, a3), which a group of at most 8 heads leaves free: one instruction multiplies both parts, rows g and g + 8 of the
// result land in the same thread and are added there.  The legacy tensor path is what bounds these kernels once the
// pages arrive through shared memory, so halving the score instructions is worth the two additions.
__device__ __forceinline__ void mma_bf16_hilo(float (&d)[2], uint32_t a_hi0, uint32_t a_lo0, uint32_t a_hi8, uint32_t a_lo8, uint32_t b0, uint32_t b1) {
  float l0, l1;
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %10, %10};"
               : "+f"(d[0]), "+f"(d[1]), "=f"(l0), "=f"(l1) : "r"(a_hi0), "r"(a_lo0), "r"(a_hi8), "r"(a_lo8), "r"(b0), "r"(b1), "f"(0.0f));
  d[0] += l0;
  d[1] += l1;
}
__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t byte_perm(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

template <int G>
__global__ void __launch_bounds__(PA_WARPS * 32, 2) paged_attn_decode_mma_kernel(
    const float* __restrict__ q, const uint4* __restrict__ kcache, const uint4* __restrict__ vcache,
    const uint32_t* __restrict__ block_table, const int* __restrict__ row_slot, const int* __restrict__ row_ctx,
    float* __restrict__ scratch, PagedGeo g, float scale_log2e) {
  constexpr int HD = 128, LPT = HD / 8;   // 16 uint4 per token row
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gi = lane >> 2, t = lane & 3;
  const i64 unit = (i64)blockIdx.x * PA_WARPS + warp;
  const i64 units = (i64)g.rows * g.kv_heads * g.max_chunks;
  if (unit >= units) return;
  const int chunk = (int)(unit / ((i64)g.rows * g.kv_heads));
  const int kvh = (int)(unit % g.kv_heads);
  const int row = (int)((unit / g.kv_heads) % g.rows);
  const int ctx = min(row_ctx[row], g.mbps * g.page_tokens);   // never walk past the block-table row
  const int t0 = chunk * g.chunk_tokens;
  float* sbase = scratch + (((i64)row * g.q_heads + (i64)kvh * G) * g.max_chunks + chunk) * (HD + 4);
  const i64 head_stride = (i64)g.max_chunks * (HD + 4);
  if (t0 >= ctx) {
    if (lane < G) { float* s = sbase + lane * head_stride; s[HD] = -INFINITY; s[HD + 1] = 0.0f; }
    return;
  }
  const int t1 = min(ctx, t0 + g.chunk_tokens);
  const int last_tok = t1 - 1;
  const uint32_t* bt = block_table + (i64)row_slot[row] * g.mbps;
  const i64 page_units = (i64)g.kv_heads * g.page_tokens * LPT;
  const i64 head_off = (i64)kvh * g.page_tokens * LPT;
  auto row_index = [&](int tok) {   // uint4 index of the first 8 dims of a (clamped) token's row
    tok = min(tok, last_tok);
    return (i64)bt[tok >> g.page_shift] * page_units + head_off + (i64)(tok & (g.page_tokens - 1)) * LPT;
  };
  // query fragments: head gi (zero rows past the group), 8 k-steps (j, h), bf16 hi and lo of q * scale * log2(e)
  uint32_t qh[4][2][2], ql[4][2][2];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float f[8];
    if (gi < G) {
      const float* qp = q + (i64)row * g.q_row_stride + ((i64)kvh * G + gi) * HD + 32 * j + 8 * t;
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
        const uint32_t hi = pack2_bf16(x0, x1);
        qh[j][h][c] = hi;
        ql[j][h][c] = pack2_bf16(x0 - u2f(hi << 16), x1 - u2f(hi & 0xffff0000u));
      }
  }
  float m = -INFINITY, l = 0.0f;
  float acc[2][8][2];
#pragma unroll
  for (int sl = 0; sl < 2; ++sl)
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) { acc[sl][jj][0] = 0.0f; acc[sl][jj][1] = 0.0f; }

  auto load_k = [&](int tile0, uint4 (&kw)[2][4]) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const i64 base = row_index(tile0 + 8 * u + gi);
#pragma unroll
      for (int j = 0; j < 4; ++j) kw[u][j] = kcache[base + 4 * j + t];
    }
  };
  uint4 kcur[2][4];
  load_k(t0, kcur);
  for (int tile0 = t0; tile0 < t1; tile0 += 16) {
    // this tile's V rows (tokens 2t, 2t+1, 2t+8, 2t+9; dims 64*sl + 8*gi .. +8) and the next tile's K rows
    uint4 vw[4][2];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const i64 base = row_index(tile0 + 2 * t + (a & 1) + 8 * (a >> 1));
#pragma unroll
      for (int sl = 0; sl < 2; ++sl) vw[a][sl] = vcache[base + 8 * sl + gi];
    }
    // ---- scores of 16 tokens for the group's heads
    float sc[2][2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      sc[u][0] = 0.0f; sc[u][1] = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t kr[4] = {kcur[u][j].x, kcur[u][j].y, kcur[u][j].z, kcur[u][j].w};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          mma_bf16_hilo(sc[u], qh[j][h][0], ql[j][h][0], qh[j][h][1], ql[j][h][1], kr[2 * h], kr[2 * h + 1]);
        }
      }
    }
    // the K registers are free again: the next tile's K rows travel while this tile's softmax and values run
    if (tile0 + 16 < t1) load_k(tile0 + 16, kcur);
    // lane (gi, t) holds head gi's scores of tokens tile0 + 8u + 2t + {0, 1}
    float s4[4];
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int c = 0; c < 2; ++c) s4[2 * u + c] = (tile0 + 8 * u + 2 * t + c < t1) ? sc[u][c] : -INFINITY;
    float tm = fmaxf(fmaxf(s4[0], s4[1]), fmaxf(s4[2], s4[3]));
    tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
    tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
    const float mn = fmaxf(m, tm);           // finite: every tile has a visible token
    const float corr = exp2f(m - mn);
    m = mn;
    const uint32_t p01 = pack2_bf16(exp2f(s4[0] - mn), exp2f(s4[1] - mn));
    const uint32_t p23 = pack2_bf16(exp2f(s4[2] - mn), exp2f(s4[3] - mn));
    // the normaliser sums the same rounded weights the values are multiplied by
    l = l * corr + ((u2f(p01 << 16) + u2f(p01 & 0xffff0000u)) + (u2f(p23 << 16) + u2f(p23 & 0xffff0000u)));
    if (__any_sync(0xffffffffu, corr != 1.0f)) {         // most tiles do not move the maximum
#pragma unroll
      for (int sl = 0; sl < 2; ++sl)
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) { acc[sl][jj][0] *= corr; acc[sl][jj][1] *= corr; }
    }
    // ---- values: 8 dims per slab and register pair, two tokens of one dim per B register
#pragma unroll
    for (int sl = 0; sl < 2; ++sl) {
      const uint32_t x0[4] = {vw[0][sl].x, vw[0][sl].y, vw[0][sl].z, vw[0][sl].w};   // token 2t
      const uint32_t x1[4] = {vw[1][sl].x, vw[1][sl].y, vw[1][sl].z, vw[1][sl].w};   // token 2t+1
      const uint32_t y0[4] = {vw[2][sl].x, vw[2][sl].y, vw[2][sl].z, vw[2][sl].w};   // token 2t+8
      const uint32_t y1[4] = {vw[3][sl].x, vw[3][sl].y, vw[3][sl].z, vw[3][sl].w};   // token 2t+9
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        mma_bf16_16816(acc[sl][2 * e], p01, p23, byte_perm(x0[e], x1[e], 0x5410u), byte_perm(y0[e], y1[e], 0x5410u));
        mma_bf16_16816(acc[sl][2 * e + 1], p01, p23, byte_perm(x0[e], x1[e], 0x7632u), byte_perm(y0[e], y1[e], 0x7632u));
      }
    }
  }
  // ---- lane (gi, t) owns dims [64*sl + 16*t, +16) of head gi: c0 of pair jj is dim +jj, c1 is dim +8+jj
  float lt = l + __shfl_xor_sync(0xffffffffu, l, 1);
  lt += __shfl_xor_sync(0xffffffffu, lt, 2);
  if (gi < G) {
    float* s = sbase + gi * head_stride;
#pragma unroll
    for (int sl = 0; sl < 2; ++sl) {
      float* d = s + 64 * sl + 16 * t;
      *reinterpret_cast<float4*>(d) = make_float4(acc[sl][0][0], acc[sl][1][0], acc[sl][2][0], acc[sl][3][0]);
      *reinterpret_cast<float4*>(d + 4) = make_float4(acc[sl][4][0], acc[sl][5][0], acc[sl][6][0], acc[sl][7][0]);
      *reinterpret_cast<float4*>(d + 8) = make_float4(acc[sl][0][1], acc[sl][1][1], acc[sl][2][1], acc[sl][3][1]);
      *reinterpret_cast<float4*>(d + 12) = make_float4(acc[sl][4][1], acc[sl][5][1], acc[sl][6][1], acc[sl][7][1]);
    }
    if (t == 0) { s[HD] = m; s[HD + 1] = lt; }
  }
}

// The tensor-core unit with its K / V pages staged in shared memory by TMA.  The cache of a layer is described to the
// TMA unit as a matrix [token row][head_dim] (token row = (page * kv_heads + head) * 16 + token); a ring slot holds one
// 16-token page of K and of V as four boxes of 16 rows x 64 dims (2 KiB each, 128-byte swizzle, this GPU's own memory,
// no multicast): four copies per 8 KiB, issued by lane 0 and counted on the slot's mbarrier.  With the swizzle, row r
// keeps its 16-byte chunk c at position c ^ (r & 7).  The tokens of a tile are assigned to the MMA's column / k positions
// through a fixed permutation (position n of an 8-token group holds token SIGMA[n]), chosen so that the two token rows a
// quarter warp reads for a K fragment differ in bit 2 and the four it reads for a V fragment are all even or all odd:
// every fragment load is then free of bank conflicts.  A permutation of the keys inside a tile changes neither the
// scores nor the weighted sum; the mask and the value rows follow the same assignment.
__device__ __forceinline__ int pa_sigma(int n) {   // 0 5 2 7 4 1 6 3
  return (n & 1) ? ((n + 4) & 7) : n;
}

template <int G, int NST>
__global__ void __launch_bounds__(32) paged_attn_decode_mma_staged_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const float* __restrict__ q,
    const uint32_t* __restrict__ block_table, const int* __restrict__ row_slot, const int* __restrict__ row_ctx,
    float* __restrict__ scratch, PagedGeo g, float scale_log2e, int* __restrict__ status) {
  constexpr int HD = 128, BOX = 2048, SLOT = 4 * BOX;      // K dims 0-63 | K dims 64-127 | V dims 0-63 | V dims 64-127
  extern __shared__ uint8_t pa_smem_raw[];
  const int lane = threadIdx.x & 31;
  const int gi = lane >> 2, t = lane & 3;
  const uint32_t ring = (smem_u32(pa_smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = ring + NST * SLOT;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NST; ++s) mbar_init(bars + 8u * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  __syncwarp();
  pdl_wait();
  pdl_trigger();
  const i64 unit = blockIdx.x;
  const int chunk = (int)(unit / ((i64)g.rows * g.kv_heads));
  const int kvh = (int)(unit % g.kv_heads);
  const int row = (int)((unit / g.kv_heads) % g.rows);
  const int ctx = min(row_ctx[row], g.mbps * g.page_tokens);
  const int t0 = chunk * g.chunk_tokens;
  float* sbase = scratch + (((i64)row * g.q_heads + (i64)kvh * G) * g.max_chunks + chunk) * (HD + 4);
  const i64 head_stride = (i64)g.max_chunks * (HD + 4);
  if (t0 >= ctx) {
    if (lane < G) { float* s = sbase + lane * head_stride; s[HD] = -INFINITY; s[HD + 1] = 0.0f; }
    return;
  }
  const int t1 = min(ctx, t0 + g.chunk_tokens);
  const int ntiles = (t1 - t0 + 15) >> 4;
  const uint32_t* bt = block_table + (i64)row_slot[row] * g.mbps;
  const int first_page = t0 >> 4, last_page = (t1 - 1) >> 4;
  uint32_t my_page = bt[min(first_page + lane, last_page)];      // page ids of the next 32 tiles, one per lane
  auto issue = [&](int i) {
    const uint32_t pg = __shfl_sync(0xffffffffu, my_page, i & 31);
    if (lane == 0) {
      const uint32_t slot = ring + (uint32_t)(i % NST) * SLOT, bar = bars + 8u * (i % NST);
      const int y = (int)(((i64)pg * g.kv_heads + kvh) * 16);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the slot's last readers (generic proxy) are done
      mbar_expect_tx(bar, SLOT);
      tma_load_2d(slot, &map_k, bar, 0, y);
      tma_load_2d(slot + BOX, &map_k, bar, 64, y);
      tma_load_2d(slot + 2 * BOX, &map_v, bar, 0, y);
      tma_load_2d(slot + 3 * BOX, &map_v, bar, 64, y);
    }
  };
  const int pre = min(NST, ntiles);
  for (int i = 0; i < pre; ++i) issue(i);
  // query fragments: head gi (zero rows past the group), 8 k-steps (j, h), bf16 hi and lo of q * scale * log2(e)
  uint32_t qh[4][2][2], ql[4][2][2];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float f[8];
    if (gi < G) {
      const float* qp = q + (i64)row * g.q_row_stride + ((i64)kvh * G + gi) * HD + 32 * j + 8 * t;
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
        const uint32_t hi = pack2_bf16(x0, x1);
        qh[j][h][c] = hi;
        ql[j][h][c] = pack2_bf16(x0 - u2f(hi << 16), x1 - u2f(hi & 0xffff0000u));
      }
  }
  float m = -INFINITY, l = 0.0f;
  float acc[2][8][2];
#pragma unroll
  for (int sl = 0; sl < 2; ++sl)
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) { acc[sl][jj][0] = 0.0f; acc[sl][jj][1] = 0.0f; }
  auto lds128 = [](uint32_t addr) {
    uint4 w;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "r"(addr));
    return w;
  };
  // token (inside the 16-token tile) behind this lane's score columns 2t, 2t+1 of group u, and behind its K column gi
  const int tokA = pa_sigma(2 * t), tokB = pa_sigma(2 * t + 1), tokK = pa_sigma(gi);
  bool ok = true;
  int issued = pre;
  for (int i = 0; i < ntiles; ++i) {
    const int tile0 = t0 + 16 * i;
    if (!mbar_wait(bars + 8u * (i % NST), (uint32_t)((i / NST) & 1))) { ok = false; break; }
    const uint32_t kslot = ring + (uint32_t)(i % NST) * SLOT, vslot = kslot + 2 * BOX;
    const int last_local = min(16, t1 - tile0) - 1;     // rows past it may never have been written: clamp onto it (weight forced to zero)
    // ---- scores of 16 tokens for the group's heads
    float sc[2][2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      sc[u][0] = 0.0f; sc[u][1] = 0.0f;
      const int r = min(8 * u + tokK, last_local);
      const uint32_t rowaddr = kslot + (uint32_t)r * 128u;
      const uint32_t sw = (uint32_t)(r & 7);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        // 16-byte chunk 4j + t of the 256-byte row: half j >> 1, position ((4 (j & 1) + t) ^ (r & 7)) inside it
        const uint4 kw = lds128(rowaddr + (uint32_t)(j >> 1) * BOX + ((((uint32_t)(4 * (j & 1) + t)) ^ sw) << 4));
        const uint32_t kr[4] = {kw.x, kw.y, kw.z, kw.w};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          mma_bf16_hilo(sc[u], qh[j][h][0], ql[j][h][0], qh[j][h][1], ql[j][h][1], kr[2 * h], kr[2 * h + 1]);
        }
      }
    }
    float s4[4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      s4[2 * u] = (tile0 + 8 * u + tokA < t1) ? sc[u][0] : -INFINITY;
      s4[2 * u + 1] = (tile0 + 8 * u + tokB < t1) ? sc[u][1] : -INFINITY;
    }
    float tm = fmaxf(fmaxf(s4[0], s4[1]), fmaxf(s4[2], s4[3]));
    tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
    tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
    const float mn = fmaxf(m, tm);           // finite: every tile has a visible token
    const float corr = exp2f(m - mn);
    m = mn;
    const uint32_t p01 = pack2_bf16(exp2f(s4[0] - mn), exp2f(s4[1] - mn));
    const uint32_t p23 = pack2_bf16(exp2f(s4[2] - mn), exp2f(s4[3] - mn));
    l = l * corr + ((u2f(p01 << 16) + u2f(p01 & 0xffff0000u)) + (u2f(p23 << 16) + u2f(p23 & 0xffff0000u)));
    if (__any_sync(0xffffffffu, corr != 1.0f)) {         // most tiles do not move the maximum
#pragma unroll
      for (int sl = 0; sl < 2; ++sl)
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) { acc[sl][jj][0] *= corr; acc[sl][jj][1] *= corr; }
    }
    // ---- values: k positions 2t, 2t+1, 2t+8, 2t+9 hold tokens tokA, tokB, 8 + tokA, 8 + tokB; dims 64 * sl + 8 * gi .. +8
    uint32_t vrow[4], vsw[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int r = min(((a & 1) ? tokB : tokA) + 8 * (a >> 1), last_local);
      vrow[a] = vslot + (uint32_t)r * 128u;
      vsw[a] = (((uint32_t)gi) ^ (uint32_t)(r & 7)) << 4;
    }
#pragma unroll
    for (int sl = 0; sl < 2; ++sl) {
      const uint4 v0 = lds128(vrow[0] + sl * BOX + vsw[0]), v1 = lds128(vrow[1] + sl * BOX + vsw[1]);
      const uint4 v2 = lds128(vrow[2] + sl * BOX + vsw[2]), v3 = lds128(vrow[3] + sl * BOX + vsw[3]);
      const uint32_t x0[4] = {v0.x, v0.y, v0.z, v0.w}, x1[4] = {v1.x, v1.y, v1.z, v1.w};
      const uint32_t y0[4] = {v2.x, v2.y, v2.z, v2.w}, y1[4] = {v3.x, v3.y, v3.z, v3.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        mma_bf16_16816(acc[sl][2 * e], p01, p23, byte_perm(x0[e], x1[e], 0x5410u), byte_perm(y0[e], y1[e], 0x5410u));
        mma_bf16_16816(acc[sl][2 * e + 1], p01, p23, byte_perm(x0[e], x1[e], 0x7632u), byte_perm(y0[e], y1[e], 0x7632u));
      }
    }
    __syncwarp();                       // every lane has read the slot
    if (i + NST < ntiles) {
      if (((i + NST) & 31) == 0) my_page = bt[min(first_page + i + NST + lane, last_page)];
      issue(i + NST);
      ++issued;
    }
  }
  if (!ok) {
    if (lane == 0) atomicExch(status, WKB_STATUS_ATTN_WAIT);
    for (int i2 = 0; i2 < issued; ++i2)
      if (i2 + NST >= issued) mbar_wait(bars + 8u * (i2 % NST), (uint32_t)((i2 / NST) & 1));
    return;
  }
  float lt = l + __shfl_xor_sync(0xffffffffu, l, 1);
  lt += __shfl_xor_sync(0xffffffffu, lt, 2);
  if (gi < G) {
    float* s = sbase + gi * head_stride;
#pragma unroll
    for (int sl = 0; sl < 2; ++sl) {
      float* d = s + 64 * sl + 16 * t;
      *reinterpret_cast<float4*>(d) = make_float4(acc[sl][0][0], acc[sl][1][0], acc[sl][2][0], acc[sl][3][0]);
      *reinterpret_cast<float4*>(d + 4) = make_float4(acc[sl][4][0], acc[sl][5][0], acc[sl][6][0], acc[sl][7][0]);
      *reinterpret_cast<float4*>(d + 8) = make_float4(acc[sl][0][1], acc[sl][1][1], acc[sl][2][1], acc[sl][3][1]);
      *reinterpret_cast<float4*>(d + 12) = make_float4(acc[sl][4][1], acc[sl][5][1], acc[sl][6][1], acc[sl][7][1]);
    }
    if (t == 0) { s[HD] = m; s[HD + 1] = lt; }
  }
}

// Merge a row-head's chunks in ascending order; out_dtype 0 = f32, 1 = bf16.
template <int HD>
__global__ void __launch_bounds__(128) paged_attn_merge_kernel(const float* __restrict__ scratch, void* __restrict__ out,
                                                               int out_dtype, i64 out_row_stride,
                                                               const int* __restrict__ row_ctx, int rows, int q_heads,
                                                               int max_chunks, int chunk_tokens, int table_tokens) {
  pdl_wait();
  pdl_trigger();
  i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x;
  i64 total = (i64)rows * q_heads * (HD / 4);
  if (idx >= total) return;
  int dq = (int)(idx % (HD / 4));
  i64 rh = idx / (HD / 4);
  int row = (int)(rh / q_heads), h = (int)(rh % q_heads);
  int ctx = min(row_ctx[row], table_tokens);
  int nch = ctx <= 0 ? 0 : (ctx + chunk_tokens - 1) / chunk_tokens;
  if (nch > max_chunks) nch = max_chunks;
  const float* s = scratch + rh * (i64)max_chunks * (HD + 4);
  float mm = -INFINITY;
#pragma unroll 4
  for (int c = 0; c < nch; ++c) mm = fmaxf(mm, s[(i64)c * (HD + 4) + HD]);
  float lsum = 0.0f;
  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
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
                                                              int rows, int kv_heads, int hd, int page_tokens, int mbps, int* __restrict__ status) {
  pdl_wait();
  pdl_trigger();
  int per_row = kv_heads * hd / 8;
  i64 total = (i64)rows * per_row;
  i64 stride = (i64)gridDim.x * blockDim.x;
  for (i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    int row = (int)(idx / per_row), c = (int)(idx % per_row);
    int pos = row_pos[row];
    if (pos < 0) continue;
    if (pos / page_tokens >= mbps) {   // beyond the block-table row: skip the row, report it
      if (c == 0 && status) atomicExch(status, WKB_STATUS_KV_POS_RANGE);
      continue;
    }
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

// One layer's cache as a matrix [token rows][head_dim] of bf16 for the TMA unit; box = one page of one head (16 rows) x 64
// dims, 128-byte swizzle.  The row extent is left open: the kernels only address pages named by the block table.
static int make_kv_page_map(CUtensorMap* map, const void* cache, i64 head_dim) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)1 << 31};
  cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
  cuuint32_t box[2] = {64, 16};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int G>
static int launch_decode_mma(const float* q, const void* kc, const void* vc, const uint32_t* bt, const int* row_slot,
                             const int* row_ctx, float* scratch, void* out, int out_dtype, i64 out_row_stride, PagedGeo g,
                             float scale, cudaStream_t st) {
  i64 units = (i64)g.rows * g.kv_heads * g.max_chunks;
  i64 blocks = (units + PA_WARPS - 1) / PA_WARPS;
  if (blocks > 0x7fffffff || units > 0x7fffffff) return (int)cudaErrorInvalidValue;
  cudaError_t e;
  static const int staged_cfg = [] { const char* s = getenv("WKB_PA_MMA_STAGED"); return s ? atoi(s) : 31; }();
  int* status = g.page_tokens == 16 && staged_cfg > 0 ? gemm_status_word() : nullptr;
  if (status) {
    // one warp per CTA, K / V pages staged in shared memory by TMA (16-token pages only)
    CUtensorMap mk, mv;
    int rc = make_kv_page_map(&mk, kc, 128);
    if (rc) return rc;
    rc = make_kv_page_map(&mv, vc, 128);
    if (rc) return rc;
    constexpr int SLOT = 4 * 2048;
#define WKB_PA_MMA_STAGED(NST_) launch_pdl(paged_attn_decode_mma_staged_kernel<G, NST_>, (unsigned)units, 32, (size_t)(NST_ * SLOT + NST_ * 8 + 1024), st, mk, mv, q, \
    bt, row_slot, row_ctx, scratch, g, scale * 1.4426950408889634f, status)
    switch (staged_cfg / 10) {
      case 3: e = WKB_PA_MMA_STAGED(3); break;
      case 4: e = WKB_PA_MMA_STAGED(4); break;
      default: e = WKB_PA_MMA_STAGED(2); break;
    }
#undef WKB_PA_MMA_STAGED
  } else {
    e = launch_pdl(paged_attn_decode_mma_kernel<G>, (unsigned)blocks, PA_WARPS * 32, 0, st, q, (const uint4*)kc, (const uint4*)vc, bt,
                   row_slot, row_ctx, scratch, g, scale * 1.4426950408889634f);
  }
  if (e != cudaSuccess) return (int)e;
  i64 total = (i64)g.rows * g.q_heads * (128 / 4);
  return (int)launch_pdl(paged_attn_merge_kernel<128>, (unsigned)((total + 127) / 128), 128, 0, st, (const float*)scratch, out, out_dtype,
                         out_row_stride, row_ctx, g.rows, g.q_heads, g.max_chunks, g.chunk_tokens, g.mbps * g.page_tokens);
}

// Launch of the staged kernel for one (NST, WARPS) shape; the dynamic shared memory limit is raised once per device.
template <int HD, int G, int NST, int WARPS>
static cudaError_t launch_staged_cfg(const float* q, const void* kc, const void* vc, const uint32_t* bt, const int* row_slot,
                                     const int* row_ctx, float* scratch, void* out, int out_dtype, i64 out_row_stride, PagedGeo g,
                                     float scale, cudaStream_t st, int* status) {
  constexpr int SMEM = WARPS * NST * (4 * 16 * HD * 2) + WARPS * NST * 8;
  auto kern = paged_attn_decode_staged_kernel<HD, G, NST, WARPS>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (SMEM > 48 * 1024 && !attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return e;
    attr_set[dev & 63] = true;
  }
  const i64 units = (i64)g.rows * g.kv_heads * g.max_chunks;
  const i64 blocks = (units + WARPS - 1) / WARPS;
  if (blocks > 0x7fffffff) return cudaErrorInvalidValue;
  return launch_pdl(kern, (unsigned)blocks, WARPS * 32, (size_t)SMEM, st, q, (const uint8_t*)kc, (const uint8_t*)vc, bt, row_slot, row_ctx,
                    scratch, g, scale * 1.4426950408889634f, out, out_dtype, out_row_stride, status);
}

template <int HD, int G>
static int launch_decode(const float* q, const void* kc, const void* vc, const uint32_t* bt, const int* row_slot,
                         const int* row_ctx, float* scratch, void* out, int out_dtype, i64 out_row_stride, PagedGeo g,
                         float scale, cudaStream_t st) {
  i64 units = (i64)g.rows * g.kv_heads * g.max_chunks;
  i64 blocks = (units + PA_WARPS - 1) / PA_WARPS;
  if (blocks > 0x7fffffff) return (int)cudaErrorInvalidValue;
  // one unit per (row, kv head): it writes the row itself (128-bit stores: a bf16 row pitch must be a multiple of 8)
  const bool direct = g.max_chunks == 1 && (out_dtype == 0 || out_row_stride % 8 == 0);
  cudaError_t e;
  static const int staged_cfg = [] { const char* s = getenv("WKB_PA_STAGED"); return s ? atoi(s) : 1; }();   // 0: the register-path kernel
  int* status = g.page_tokens == 16 && staged_cfg > 0 ? gemm_status_word() : nullptr;
  if (status) {
    // K / V pages staged in shared memory by bulk copies (16-token pages only)
    void* o = direct ? out : (void*)nullptr;
#define WKB_PA_STAGED(NST_, WARPS_) launch_staged_cfg<HD, G, NST_, WARPS_>(q, kc, vc, bt, row_slot, row_ctx, scratch, o, out_dtype, out_row_stride, g, scale, st, status)
    if constexpr (HD == 64 && G == 1) {
      // two ring slots and one warp per CTA were the fastest of the shapes tried (2 - 6 slots, 1 / 2 / 4 warps per CTA) on
      // 512 rows x 12 heads with contexts up to 640
      e = WKB_PA_STAGED(2, 1);
    } else if constexpr (HD == 64) {
      e = WKB_PA_STAGED(3, 1);
    } else {
      e = WKB_PA_STAGED(2, 1);
    }
#undef WKB_PA_STAGED
  } else {
    e = launch_pdl(paged_attn_decode_kernel<HD, G>, (unsigned)blocks, PA_WARPS * 32, 0, st, q, (const uint4*)kc, (const uint4*)vc, bt,
                   row_slot, row_ctx, scratch, g, scale * 1.4426950408889634f, direct ? out : (void*)nullptr, out_dtype,
                   out_row_stride);
  }
  if (e != cudaSuccess || direct) return (int)e;
  i64 total = (i64)g.rows * g.q_heads * (HD / 4);
  return (int)launch_pdl(paged_attn_merge_kernel<HD>, (unsigned)((total + 127) / 128), 128, 0, st, (const float*)scratch, out, out_dtype,
                         out_row_stride, row_ctx, g.rows, g.q_heads, g.max_chunks, g.chunk_tokens, g.mbps * g.page_tokens);
}

}  // namespace wkb

using namespace wkb;

// How finely a sequence is split depends on the launch shape only (never on the data): few (row, kv head) pairs need
// the split for parallelism, many pairs are better off amortising the per-unit set-up over longer runs.
static void pa_plan(i64 rows, i64 kv_heads, i64 head_dim, int G, i64 max_ctx, int* chunk_tokens_out, i64* chunks_out) {
  // Aim for about 1024 units at full context, between 128 and 512 tokens each (measured on batch 64 x 8 KV heads at
  // context 2048: 128 / 256 / 512 / 1024-token units give 128 / 122 / 115 / 112 us per launch, 2048 gives 197 us; on
  // ragged contexts up to 4096, 512 beats 1024; with 4 or 2 KV heads per GPU, 256 / 512-token units beat 128 / 256).
  i64 want = rows * kv_heads * (max_ctx > 0 ? max_ctx : 1) / 1024;
  int chunk_tokens = PA_CHUNK_MIN;
  while (chunk_tokens < 512 && chunk_tokens * 2 <= want) chunk_tokens *= 2;
  // Two chunks of 512 where one of 1024 would do (contexts up to 1024 with plenty of rows): take the single chunk --
  // the SIMT kernels then write the rows themselves and the merge launch disappears (same time per launch measured
  // on 512 rows x 12 heads with contexts up to 896).
  const bool simt = head_dim == 64 || G == 1;
  if (simt) {
    // The SIMT kernels stage K / V in shared memory and keep about 2000 single-warp CTAs resident: they want the fewest
    // chunks that still give some 3000 units (measured on 12 heads of 64, contexts up to 640: 512 rows -- one
    // 1024-token chunk, no merge launch, 96.7 us; 64 rows -- 256-token chunks 19.4 us against 23.4 us unsplit).
    const i64 pairs = rows * kv_heads > 0 ? rows * kv_heads : 1;
    const i64 chunks_wanted = (3000 + pairs - 1) / pairs;
    chunk_tokens = 1024;
    while (chunk_tokens > 256 && (max_ctx + chunk_tokens - 1) / chunk_tokens < chunks_wanted) chunk_tokens /= 2;
  }
  i64 chunks = (max_ctx + chunk_tokens - 1) / chunk_tokens;
  if (chunks < 1) chunks = 1;
  *chunk_tokens_out = chunk_tokens;
  *chunks_out = chunks;
}

extern "C" {

i64 wkb_paged_attn_scratch_bytes(i64 rows, i64 q_heads, i64 head_dim, i64 max_ctx) {
  i64 chunks = (max_ctx + PA_CHUNK_MIN - 1) / PA_CHUNK_MIN;   // worst case: the smallest split
  if (chunks < 1) chunks = 1;
  return rows * q_heads * chunks * (head_dim + 4) * 4;
}

// Kernels one wkb_paged_attn_decode call launches: 1 when every row is a single unit that writes its own output
// (SIMT kernels, one chunk), else 2 (units + chunk merge).
i64 wkb_paged_attn_decode_launches(i64 rows, i64 q_heads, i64 kv_heads, i64 head_dim, i64 max_ctx, int out_dtype, i64 out_row_stride) {
  if (rows <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0) return 0;
  const int G = (int)(q_heads / kv_heads);
  int chunk_tokens;
  i64 chunks;
  pa_plan(rows, kv_heads, head_dim, G, max_ctx, &chunk_tokens, &chunks);
  const bool simt = head_dim == 64 || G == 1;
  return (simt && chunks == 1 && (out_dtype == 0 || out_row_stride % 8 == 0)) ? 1 : 2;
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
  int G = (int)(q_heads / kv_heads);
  int chunk_tokens;
  i64 chunks;
  pa_plan(rows, kv_heads, head_dim, G, max_ctx, &chunk_tokens, &chunks);
  PagedGeo g{(int)rows, (int)q_heads, (int)kv_heads, (int)page_tokens, page_shift, (int)max_blocks_per_seq, (int)chunks, chunk_tokens, q_row_stride};
  cudaStream_t st = as_stream(stream);
#define WKB_PA_CASE(HD_, G_) \
  if (head_dim == HD_ && G == G_) return launch_decode<HD_, G_>(q, kcache, vcache, block_table, row_slot, row_ctx, scratch, out, out_dtype, out_row_stride, g, scale, st);
  WKB_PA_CASE(64, 1) WKB_PA_CASE(64, 2) WKB_PA_CASE(64, 4)
  WKB_PA_CASE(128, 1)
#undef WKB_PA_CASE
  if (head_dim == 128 && chunk_tokens % 16 == 0) {
    if (G == 2) return launch_decode_mma<2>(q, kcache, vcache, block_table, row_slot, row_ctx, scratch, out, out_dtype, out_row_stride, g, scale, st);
    if (G == 4) return launch_decode_mma<4>(q, kcache, vcache, block_table, row_slot, row_ctx, scratch, out, out_dtype, out_row_stride, g, scale, st);
    if (G == 8) return launch_decode_mma<8>(q, kcache, vcache, block_table, row_slot, row_ctx, scratch, out, out_dtype, out_row_stride, g, scale, st);
  }
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
  return (int)launch_pdl(paged_kv_append_kernel, (int)blocks, 256, 0, as_stream(stream), ksrc, vsrc, src_row_stride, (u16*)kcache,
                         (u16*)vcache, block_table, row_slot, row_pos, (int)rows, (int)kv_heads, (int)head_dim, (int)page_tokens,
                         (int)max_blocks_per_seq, gemm_status_word());
}
}

#include "paged_int8.cuh"

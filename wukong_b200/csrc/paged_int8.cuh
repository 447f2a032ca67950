// int8 KV cache: append (quantize + scatter) and decode attention.  Included at the end of paged.cu, whose geometry,
// scratch records and chunk-merge kernel it shares.
//
// The reference's lossy storage option (crates/wukong_codegen_gpu/src/paged_attention.rs:1305-1326 quantizer,
// crates/wukong_codegen_gpu/src/paged_kv.rs:153-178 slabs): per (token, KV head) scale = max|x| / 127 (1 for an
// all-zero row), value = round(x / scale) half away from zero, clamped to +-127; attention reads int8 * scale.
// HBM layout here: int8 [num_pages][kv_heads][page_tokens][head_dim] and f32 scales
// [num_pages][kv_heads][page_tokens], so a (page, head) run of values is contiguous and its 16 scales are one
// 64-byte line.  Algorithmic bytes per (row, kv head, token) = 2 * (head_dim + 4): about half the bf16 cache's.
#pragma once

namespace wkb {

// One warp per (row, kv head): K then V.  The quantized bytes and the scale are exactly the reference's.
template <int HD>
__global__ void __launch_bounds__(256) paged_kv_append_i8_kernel(const float* __restrict__ ksrc, const float* __restrict__ vsrc,
                                                                 i64 src_row_stride, int8_t* __restrict__ kq, int8_t* __restrict__ vq,
                                                                 float* __restrict__ kscale, float* __restrict__ vscale,
                                                                 const uint32_t* __restrict__ block_table, const int* __restrict__ row_slot,
                                                                 const int* __restrict__ row_pos, int rows, int kv_heads, int page_tokens,
                                                                 int page_shift, int mbps, int* __restrict__ status) {
  constexpr int EPL = HD / 32;     // elements per lane: 2 or 4
  const int lane = threadIdx.x & 31;
  const i64 unit = ((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (unit >= (i64)rows * kv_heads) return;
  const int row = (int)(unit / kv_heads), h = (int)(unit % kv_heads);
  const int pos = row_pos[row];
  if (pos < 0) return;
  if ((pos >> page_shift) >= mbps) {   // beyond the block-table row: skip the row, report it
    if (lane == 0 && h == 0 && status) atomicExch(status, WKB_STATUS_KV_POS_RANGE);
    return;
  }
  const uint32_t page = block_table[(i64)row_slot[row] * mbps + (pos >> page_shift)];
  const i64 tok = ((i64)page * kv_heads + h) * page_tokens + (pos & (page_tokens - 1));
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const float* src = (which ? vsrc : ksrc) + (i64)row * src_row_stride + (i64)h * HD + lane * EPL;
    float x[EPL];
    float amax = 0.0f;
#pragma unroll
    for (int e = 0; e < EPL; ++e) { x[e] = src[e]; amax = fmaxf(amax, fabsf(x[e])); }
    amax = warp_max(amax);
    const float scale = amax > 0.0f ? fdiv(amax, 127.0f) : 1.0f;
    uint32_t packed = 0;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      const float r = fminf(fmaxf(roundf(fdiv(x[e], scale)), -127.0f), 127.0f);
      packed |= ((uint32_t)(int)r & 0xFFu) << (8 * e);
    }
    int8_t* dst = (which ? vq : kq) + tok * HD + lane * EPL;
    if (EPL == 4) *reinterpret_cast<uint32_t*>(dst) = packed;
    else *reinterpret_cast<uint16_t*>(dst) = (uint16_t)packed;
    if (lane == 0) (which ? vscale : kscale)[tok] = scale;
  }
}

__device__ __forceinline__ void unpack8_i8(const uint2& w, float f[8]) {
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    f[e] = (float)(int)(int8_t)(w.x >> (8 * e));
    f[4 + e] = (float)(int)(int8_t)(w.y >> (8 * e));
  }
}

// The decode kernel's unit of work and reduction trees (one warp per (row, kv head, chunk); a lane owns 8 head dims of
// one token; 32 tokens per tile; scratch records merged by paged_attn_merge_kernel) over the int8 cache: a token's dot
// is taken over the raw int8 values and multiplied by its scale once, a token's weight is multiplied by its V scale.
template <int HD, int G>
__global__ void __launch_bounds__(PA_WARPS * 32) paged_attn_decode_i8_kernel(
    const float* __restrict__ q, const uint2* __restrict__ kq, const uint2* __restrict__ vq, const float* __restrict__ kscale,
    const float* __restrict__ vscale, const uint32_t* __restrict__ block_table, const int* __restrict__ row_slot,
    const int* __restrict__ row_ctx, float* __restrict__ scratch, PagedGeo g, float scale_log2e) {
  constexpr int LPT = HD / 8, TPW = 32 / LPT, STEPS = LPT, TILE = STEPS * TPW;
  static_assert(TILE == 32, "tile is one token per lane");
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grp = lane / LPT, j = lane % LPT;
  const i64 unit = (i64)blockIdx.x * PA_WARPS + warp;
  if (unit >= (i64)g.rows * g.kv_heads * g.max_chunks) return;
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
  const int last_tok = t1 - 1;
  const uint32_t* bt = block_table + (i64)row_slot[row] * g.mbps;
  float qv[G][8];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    const float* qp = q + (i64)row * g.q_row_stride + ((i64)kvh * G + h) * HD + j * 8;
    const float4 a = *reinterpret_cast<const float4*>(qp), b = *reinterpret_cast<const float4*>(qp + 4);
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
  for (int tile0 = t0; tile0 < t1; tile0 += TILE) {
    uint2 kw[STEPS], vw[STEPS];
    float ks[STEPS], vs[STEPS];
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      const int tok = min(tile0 + s * TPW + grp, last_tok);      // clamped: real data, weight forced to zero below
      const i64 trow = ((i64)bt[tok >> g.page_shift] * g.kv_heads + kvh) * g.page_tokens + (tok & (g.page_tokens - 1));
      kw[s] = kq[trow * LPT + j];
      vw[s] = vq[trow * LPT + j];
      ks[s] = kscale[trow];
      vs[s] = vscale[trow];
    }
    float part[G][STEPS];
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      float kf[8];
      unpack8_i8(kw[s], kf);
#pragma unroll
      for (int h = 0; h < G; ++h) {
        float d = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) d = fmaf(qv[h][e], kf[e], d);
        part[h][s] = d * ks[s];
      }
    }
#pragma unroll
    for (int hh = STEPS / 2; hh >= 1; hh >>= 1) {
      const bool upper = (j & hh) != 0;
#pragma unroll
      for (int h = 0; h < G; ++h)
#pragma unroll
        for (int i = 0; i < hh; ++i) {
          const float send = upper ? part[h][i] : part[h][i + hh];
          const float keep = upper ? part[h][i + hh] : part[h][i];
          part[h][i] = keep + __shfl_xor_sync(0xffffffffu, send, hh);
        }
    }
    const bool mine = tile0 + j * TPW + grp < t1;       // lane (grp, j) owns token tile0 + j*TPW + grp
    float p[G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
      const float sc = mine ? part[h][0] : -INFINITY;
      const float mn = fmaxf(m[h], warp_max(sc));
      const float corr = exp2f(m[h] - mn);
      p[h] = exp2f(sc - mn);
      l[h] = l[h] * corr + p[h];
      m[h] = mn;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[h][e] *= corr;
    }
#pragma unroll
    for (int s = 0; s < STEPS; ++s) {
      float vf[8];
      unpack8_i8(vw[s], vf);
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const float pt = __shfl_sync(0xffffffffu, p[h], grp * LPT + s) * vs[s];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[h][e] = fmaf(pt, vf[e], acc[h][e]);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < G; ++h) {
#pragma unroll
    for (int ofs = LPT; ofs < 32; ofs <<= 1)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[h][e] += __shfl_xor_sync(0xffffffffu, acc[h][e], ofs);
    const float lt = warp_sum(l[h]);
    float* s = sbase + h * head_stride;
    if (grp == 0) {
      *reinterpret_cast<float4*>(s + j * 8) = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
      *reinterpret_cast<float4*>(s + j * 8 + 4) = make_float4(acc[h][4], acc[h][5], acc[h][6], acc[h][7]);
    }
    if (lane == 0) { s[HD] = m[h]; s[HD + 1] = lt; }
  }
}


// ---- tensor-core unit over the int8 cache (head_dim 128, GQA group of 2-8, 16-token pages) --------------------------------
// The same unit of work, scratch records and chunk merge as the bf16 tensor-core kernel, with the page of K and of V
// (16 tokens x 128 int8 = 2 KiB each) landed in shared memory by one TMA copy each (the cache seen as a matrix
// [token row][128 bytes], box = 16 rows, 128-byte swizzle, this GPU's memory, no multicast) and the two 64-byte runs of
// scales by bulk copies on the same mbarrier.  int8 -> f16 is exact and costs one byte permute and one subtraction per pair:
// (0x6400 | (v ^ 0x80)) is the f16 number 1024 + (v + 128), minus 1152.  The MMAs are m16n8k16 f16 x f16 -> f32: scores are
// taken over the raw integers with the query as f16 hi + lo (about 22 bits) and multiplied by the token's K scale once; a
// token's weight times its V scale, relative to the largest V scale met so far (a running reference, handled like the
// running maximum: the accumulator is rescaled when it grows, so the operand stays in [0, 1] whatever the scales' range),
// goes into the P . V product over the raw integers as f16 hi + lo; the normaliser sums the unrounded weights.  Tokens sit at the MMA's column / k
// positions through the same fixed permutation as in the bf16 kernel, which keeps every fragment load conflict-free.
// Rows of a partly filled page are never clamped: stale int8 values are finite, and a stale scale only ever meets a select.
// m16n8k16 with the hi parts of the A operand in rows 0-7 (registers a0, a2) and the lo parts in rows 8-15 (a1, a3), which a
// group of at most 8 heads leaves free: ONE instruction multiplies both parts, rows g and g + 8 of the result land in the
// same thread (d0, d1 and d2, d3) and are added there.  The legacy tensor path is what bounds this kernel (about one
// m16n8k16 per 6 clocks per SM), so halving the instruction count matters more than the two additions.
__device__ __forceinline__ void mma_f16_hilo(float (&d)[2], uint32_t a_hi0, uint32_t a_lo0, uint32_t a_hi8, uint32_t a_lo8, uint32_t b0, uint32_t b1) {
  float l0, l1;
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %10, %10};"
               : "+f"(d[0]), "+f"(d[1]), "=f"(l0), "=f"(l1) : "r"(a_hi0), "r"(a_lo0), "r"(a_hi8), "r"(a_lo8), "r"(b0), "r"(b1), "f"(0.0f));
  d[0] += l0;
  d[1] += l1;
}
__device__ __forceinline__ uint32_t pack2_f16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float f16_lo(uint32_t w) { float f; asm("{\n .reg .b16 l, h;\n mov.b32 {l, h}, %1;\n cvt.f32.f16 %0, l;\n}" : "=f"(f) : "r"(w)); return f; }
__device__ __forceinline__ float f16_hi(uint32_t w) { float f; asm("{\n .reg .b16 l, h;\n mov.b32 {l, h}, %1;\n cvt.f32.f16 %0, h;\n}" : "=f"(f) : "r"(w)); return f; }
// two offset-binary bytes (already ^ 0x80) picked by `sel` against the 0x64 filler -> f16x2 of the signed values
__device__ __forceinline__ uint32_t i8pair_f16(uint32_t biased, uint32_t sel) {
  uint32_t r;
  asm("{\n .reg .b32 t;\n prmt.b32 t, %1, %2, %3;\n sub.rn.f16x2 %0, t, %4;\n}" : "=r"(r) : "r"(biased), "r"(0x64646464u), "r"(sel), "r"(0x64806480u));
  return r;
}

template <int G, int NST>
__global__ void __launch_bounds__(32) paged_attn_decode_i8_mma_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const float* __restrict__ q,
    const float* __restrict__ kscale, const float* __restrict__ vscale, const uint32_t* __restrict__ block_table,
    const int* __restrict__ row_slot, const int* __restrict__ row_ctx, float* __restrict__ scratch, PagedGeo g, float scale_log2e,
    int* __restrict__ status) {
  constexpr int HD = 128, BOX = 2048, SLOT = 2 * BOX, SC = 128;      // slot: K page | V page; scales: 16 K | 16 V (f32)
  extern __shared__ uint8_t pa8_smem_raw[];
  const int lane = threadIdx.x & 31;
  const int gi = lane >> 2, t = lane & 3;
  const uint32_t ring = (smem_u32(pa8_smem_raw) + 1023u) & ~1023u;
  const uint32_t scales = ring + NST * SLOT;
  const uint32_t bars = scales + NST * SC;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NST; ++s) mbar_init(bars + 8u * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  __syncwarp();
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
      const uint32_t slot = ring + (uint32_t)(i % NST) * SLOT, sc = scales + (uint32_t)(i % NST) * SC, bar = bars + 8u * (i % NST);
      const i64 trow = ((i64)pg * g.kv_heads + kvh) * 16;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the slot's last readers (generic proxy) are done
      mbar_expect_tx(bar, SLOT + SC);
      tma_load_2d(slot, &map_k, bar, 0, (int)trow);
      tma_load_2d(slot + BOX, &map_v, bar, 0, (int)trow);
      bulk_g2s(sc, kscale + trow, 64, bar);
      bulk_g2s(sc + 64, vscale + trow, 64, bar);
    }
  };
  const int pre = min(NST, ntiles);
  for (int i = 0; i < pre; ++i) issue(i);
  // query fragments of head gi (zero rows past the group): the lane's K chunk j covers dims 16 (4j + t) .. +16, word h of it
  // feeds one MMA with k positions (2t, 2t+1) <- bytes (4h, 4h+1) and (2t+8, 2t+9) <- bytes (4h+2, 4h+3); f16 hi + lo of
  // q * scale * log2(e), clamped to the f16 range
  uint32_t qh[2][4][2], ql[2][4][2];
#pragma unroll
  for (int j = 0; j < 2; ++j)
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      if (gi < G) a = *reinterpret_cast<const float4*>(q + (i64)row * g.q_row_stride + ((i64)kvh * G + gi) * HD + 16 * (4 * j + t) + 4 * h);
      const float f[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const float x0 = fminf(fmaxf(f[2 * c] * scale_log2e, -65504.0f), 65504.0f), x1 = fminf(fmaxf(f[2 * c + 1] * scale_log2e, -65504.0f), 65504.0f);
        const uint32_t hi = pack2_f16(x0, x1);
        qh[j][h][c] = hi;
        ql[j][h][c] = pack2_f16(x0 - f16_lo(hi), x1 - f16_hi(hi));
      }
    }
  float m = -INFINITY, l = 0.0f, vref = 0.0f;     // vref: largest V scale of the tokens seen so far; acc is in units of it
  float acc[16][2];
#pragma unroll
  for (int e = 0; e < 16; ++e) { acc[e][0] = 0.0f; acc[e][1] = 0.0f; }
  auto lds128 = [](uint32_t addr) {
    uint4 w;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w) : "r"(addr));
    return w;
  };
  auto lds32f = [](uint32_t addr) {
    float f;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(f) : "r"(addr));
    return f;
  };
  // token (inside the 16-token tile) behind this lane's score columns 2t, 2t+1 of group u, and behind its K column gi
  const int tokA = pa_sigma(2 * t), tokB = pa_sigma(2 * t + 1), tokK = pa_sigma(gi);
  bool ok = true;
  int issued = pre;
  for (int i = 0; i < ntiles; ++i) {
    const int tile0 = t0 + 16 * i;
    if (!mbar_wait(bars + 8u * (i % NST), (uint32_t)((i / NST) & 1))) { ok = false; break; }
    const uint32_t kslot = ring + (uint32_t)(i % NST) * SLOT, vslot = kslot + BOX, sc_addr = scales + (uint32_t)(i % NST) * SC;
    // ---- scores of 16 tokens for the group's heads, over the raw integers
    float sc[2][2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      sc[u][0] = 0.0f; sc[u][1] = 0.0f;
      const int r = 8 * u + tokK;
      const uint32_t rowaddr = kslot + (uint32_t)r * 128u;
      const uint32_t sw = (uint32_t)(r & 7);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const uint4 kw = lds128(rowaddr + ((((uint32_t)(4 * j + t)) ^ sw) << 4));
        const uint32_t kr[4] = {kw.x ^ 0x80808080u, kw.y ^ 0x80808080u, kw.z ^ 0x80808080u, kw.w ^ 0x80808080u};
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const uint32_t b0 = i8pair_f16(kr[h], 0x7170u), b1 = i8pair_f16(kr[h], 0x7372u);
          mma_f16_hilo(sc[u], qh[j][h][0], ql[j][h][0], qh[j][h][1], ql[j][h][1], b0, b1);
        }
      }
    }
    // lane (gi, t) holds head gi's scores of tokens 8u + tokA, 8u + tokB; a token past the chunk's end is masked by select
    float s4[4], vs4[4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const bool va = tile0 + 8 * u + tokA < t1, vb = tile0 + 8 * u + tokB < t1;
      const float ka = lds32f(sc_addr + 4u * (uint32_t)(8 * u + tokA)), kb = lds32f(sc_addr + 4u * (uint32_t)(8 * u + tokB));
      s4[2 * u] = va ? sc[u][0] * ka : -INFINITY;
      s4[2 * u + 1] = vb ? sc[u][1] * kb : -INFINITY;
      vs4[2 * u] = va ? lds32f(sc_addr + 64u + 4u * (uint32_t)(8 * u + tokA)) : 0.0f;
      vs4[2 * u + 1] = vb ? lds32f(sc_addr + 64u + 4u * (uint32_t)(8 * u + tokB)) : 0.0f;
    }
    float tm = fmaxf(fmaxf(s4[0], s4[1]), fmaxf(s4[2], s4[3]));
    tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
    tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
    const float mn = fmaxf(m, tm);           // finite: every tile has a visible token
    const float corr = exp2f(m - mn);
    m = mn;
    float p[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) p[e] = exp2f(s4[e] - mn);      // 0 for a masked token
    l = l * corr + ((p[0] + p[1]) + (p[2] + p[3]));
    // weights times the tokens' V scales (a masked token's scale was replaced by 0 above, whatever the stale word holds),
    // relative to the running reference scale, as f16 hi + lo
    float vt = fmaxf(fmaxf(vs4[0], vs4[1]), fmaxf(vs4[2], vs4[3]));
    vt = fmaxf(vt, __shfl_xor_sync(0xffffffffu, vt, 1));
    vt = fmaxf(vt, __shfl_xor_sync(0xffffffffu, vt, 2));
    const float vnew = fmaxf(vref, vt);
    const float vinv = vnew > 0.0f ? 1.0f / vnew : 0.0f;
    const float corr_all = corr * (vnew > 0.0f ? vref * vinv : 1.0f);
    vref = vnew;
    float pv[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) pv[e] = p[e] * (vs4[e] * vinv);
    const uint32_t p01 = pack2_f16(pv[0], pv[1]), p23 = pack2_f16(pv[2], pv[3]);
    const uint32_t r01 = pack2_f16(pv[0] - f16_lo(p01), pv[1] - f16_hi(p01)), r23 = pack2_f16(pv[2] - f16_lo(p23), pv[3] - f16_hi(p23));
    if (__any_sync(0xffffffffu, corr_all != 1.0f)) {      // most tiles move neither the maximum nor the reference scale
#pragma unroll
      for (int e = 0; e < 16; ++e) { acc[e][0] *= corr_all; acc[e][1] *= corr_all; }
    }
    // ---- values: k positions 2t, 2t+1, 2t+8, 2t+9 hold tokens tokA, tokB, 8 + tokA, 8 + tokB; the lane supplies dims
    // 16 gi .. +16 (column gi of output block e is dim 16 gi + e)
    const uint4 v0 = lds128(vslot + (uint32_t)tokA * 128u + ((((uint32_t)gi) ^ (uint32_t)(tokA & 7)) << 4));
    const uint4 v1 = lds128(vslot + (uint32_t)tokB * 128u + ((((uint32_t)gi) ^ (uint32_t)(tokB & 7)) << 4));
    const uint4 v2 = lds128(vslot + (uint32_t)(8 + tokA) * 128u + ((((uint32_t)gi) ^ (uint32_t)(tokA & 7)) << 4));
    const uint4 v3 = lds128(vslot + (uint32_t)(8 + tokB) * 128u + ((((uint32_t)gi) ^ (uint32_t)(tokB & 7)) << 4));
    const uint32_t x0[4] = {v0.x ^ 0x80808080u, v0.y ^ 0x80808080u, v0.z ^ 0x80808080u, v0.w ^ 0x80808080u};
    const uint32_t x1[4] = {v1.x ^ 0x80808080u, v1.y ^ 0x80808080u, v1.z ^ 0x80808080u, v1.w ^ 0x80808080u};
    const uint32_t y0[4] = {v2.x ^ 0x80808080u, v2.y ^ 0x80808080u, v2.z ^ 0x80808080u, v2.w ^ 0x80808080u};
    const uint32_t y1[4] = {v3.x ^ 0x80808080u, v3.y ^ 0x80808080u, v3.z ^ 0x80808080u, v3.w ^ 0x80808080u};
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      // bytes of the two token rows interleaved: (a.b0, b.b0, a.b1, b.b1) and (a.b2, b.b2, a.b3, b.b3)
      const uint32_t xa = byte_perm(x0[w], x1[w], 0x5140u), xb = byte_perm(x0[w], x1[w], 0x7362u);
      const uint32_t ya = byte_perm(y0[w], y1[w], 0x5140u), yb = byte_perm(y0[w], y1[w], 0x7362u);
      const uint32_t bx[4] = {i8pair_f16(xa, 0x7170u), i8pair_f16(xa, 0x7372u), i8pair_f16(xb, 0x7170u), i8pair_f16(xb, 0x7372u)};
      const uint32_t by[4] = {i8pair_f16(ya, 0x7170u), i8pair_f16(ya, 0x7372u), i8pair_f16(yb, 0x7170u), i8pair_f16(yb, 0x7372u)};
#pragma unroll
      for (int e = 0; e < 4; ++e) mma_f16_hilo(acc[4 * w + e], p01, r01, p23, r23, bx[e], by[e]);
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
  // ---- lane (gi, t) owns, of head gi, dims 32 t + e (c0 of output block e) and 32 t + 16 + e (c1): output column n is dim 16 n + e
  float lt = l + __shfl_xor_sync(0xffffffffu, l, 1);
  lt += __shfl_xor_sync(0xffffffffu, lt, 2);
  if (gi < G) {
    float* s = sbase + gi * head_stride;
    float* d = s + 32 * t;
#pragma unroll
    for (int e = 0; e < 16; e += 4) {
      *reinterpret_cast<float4*>(d + e) = make_float4(acc[e][0] * vref, acc[e + 1][0] * vref, acc[e + 2][0] * vref, acc[e + 3][0] * vref);
      *reinterpret_cast<float4*>(d + 16 + e) = make_float4(acc[e][1] * vref, acc[e + 1][1] * vref, acc[e + 2][1] * vref, acc[e + 3][1] * vref);
    }
    if (t == 0) { s[HD] = m; s[HD + 1] = lt; }
  }
}

// One layer's int8 cache as a matrix [token rows][128 bytes] for the TMA unit; box = one page of one head (16 rows), 128-byte swizzle.
static int make_kv8_page_map(CUtensorMap* map, const void* cache) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {128, (cuuint64_t)1 << 31};
  cuuint64_t strides[1] = {128};
  cuuint32_t box[2] = {128, 16};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(cache), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int G>
static int launch_decode_i8_mma(const float* q, const void* kq, const void* vq, const float* ks, const float* vs, const uint32_t* bt,
                                const int* row_slot, const int* row_ctx, float* scratch, void* out, int out_dtype, i64 out_row_stride,
                                PagedGeo g, float scale, cudaStream_t st) {
  constexpr int NST = 3, SMEM = NST * (4096 + 128) + NST * 8 + 1024;
  const i64 units = (i64)g.rows * g.kv_heads * g.max_chunks;
  if (units > 0x7fffffff) return (int)cudaErrorInvalidValue;
  CUtensorMap mk, mv;
  int rc = make_kv8_page_map(&mk, kq);
  if (rc) return rc;
  rc = make_kv8_page_map(&mv, vq);
  if (rc) return rc;
  int* status = gemm_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  paged_attn_decode_i8_mma_kernel<G, NST><<<(unsigned)units, 32, SMEM, st>>>(mk, mv, q, ks, vs, bt, row_slot, row_ctx, scratch, g,
                                                                          scale * 1.4426950408889634f, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  const i64 total = (i64)g.rows * g.q_heads * (128 / 4);
  paged_attn_merge_kernel<128><<<(unsigned)((total + 127) / 128), 128, 0, st>>>(scratch, out, out_dtype, out_row_stride, row_ctx, g.rows,
                                                                                 g.q_heads, g.max_chunks, g.chunk_tokens, g.mbps * g.page_tokens);
  return (int)cudaGetLastError();
}

template <int HD, int G>
static int launch_decode_i8(const float* q, const void* kq, const void* vq, const float* ks, const float* vs, const uint32_t* bt,
                            const int* row_slot, const int* row_ctx, float* scratch, void* out, int out_dtype, i64 out_row_stride,
                            PagedGeo g, float scale, cudaStream_t st) {
  const i64 units = (i64)g.rows * g.kv_heads * g.max_chunks;
  const i64 blocks = (units + PA_WARPS - 1) / PA_WARPS;
  if (blocks > 0x7fffffff) return (int)cudaErrorInvalidValue;
  paged_attn_decode_i8_kernel<HD, G><<<(unsigned)blocks, PA_WARPS * 32, 0, st>>>(
      q, (const uint2*)kq, (const uint2*)vq, ks, vs, bt, row_slot, row_ctx, scratch, g, scale * 1.4426950408889634f);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  const i64 total = (i64)g.rows * g.q_heads * (HD / 4);
  paged_attn_merge_kernel<HD><<<(unsigned)((total + 127) / 128), 128, 0, st>>>(scratch, out, out_dtype, out_row_stride, row_ctx, g.rows,
                                                                                g.q_heads, g.max_chunks, g.chunk_tokens, g.mbps * g.page_tokens);
  return (int)cudaGetLastError();
}

}  // namespace wkb

extern "C" {

int wkb_paged_kv_append_int8(const float* ksrc, const float* vsrc, i64 src_row_stride, void* kq, void* vq, float* kscale, float* vscale,
                             const uint32_t* block_table, const int* row_slot, const int* row_pos, i64 rows, i64 kv_heads,
                             i64 head_dim, i64 page_tokens, i64 max_blocks_per_seq, void* stream) {
  using namespace wkb;
  if (rows <= 0) return 0;
  if (head_dim != 64 && head_dim != 128) return (int)cudaErrorInvalidValue;
  if (page_tokens < 4 || (page_tokens & (page_tokens - 1)) != 0) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)kq) | ((uintptr_t)vq)) & 3) return (int)cudaErrorMisalignedAddress;
  int page_shift = 0;
  while ((1 << page_shift) < page_tokens) ++page_shift;
  const i64 threads = rows * kv_heads * 32;
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  cudaStream_t st = as_stream(stream);
  if (head_dim == 64)
    paged_kv_append_i8_kernel<64><<<blocks, 256, 0, st>>>(ksrc, vsrc, src_row_stride, (int8_t*)kq, (int8_t*)vq, kscale, vscale, block_table,
                                                          row_slot, row_pos, (int)rows, (int)kv_heads, (int)page_tokens, page_shift,
                                                          (int)max_blocks_per_seq, gemm_status_word());
  else
    paged_kv_append_i8_kernel<128><<<blocks, 256, 0, st>>>(ksrc, vsrc, src_row_stride, (int8_t*)kq, (int8_t*)vq, kscale, vscale, block_table,
                                                           row_slot, row_pos, (int)rows, (int)kv_heads, (int)page_tokens, page_shift,
                                                           (int)max_blocks_per_seq, gemm_status_word());
  return (int)cudaGetLastError();
}

int wkb_paged_attn_decode_int8(const float* q, i64 q_row_stride, const void* kq, const void* vq, const float* kscale, const float* vscale,
                               const uint32_t* block_table, const int* row_slot, const int* row_ctx, void* out, int out_dtype,
                               i64 out_row_stride, i64 rows, i64 q_heads, i64 kv_heads, i64 head_dim, i64 page_tokens,
                               i64 max_blocks_per_seq, i64 max_ctx, float scale, float* scratch, void* stream) {
  using namespace wkb;
  if (rows <= 0) return 0;
  if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0) return (int)cudaErrorInvalidValue;
  if (page_tokens < 4 || (page_tokens & (page_tokens - 1)) != 0) return (int)cudaErrorInvalidValue;
  int page_shift = 0;
  while ((1 << page_shift) < page_tokens) ++page_shift;
  if ((q_row_stride % 4) != 0 || ((((uintptr_t)q) | ((uintptr_t)scratch)) & 15) != 0 || ((((uintptr_t)kq) | ((uintptr_t)vq)) & 7) != 0)
    return (int)cudaErrorMisalignedAddress;
  if (out_row_stride % 4 != 0 || (((uintptr_t)out) & 15) != 0) return (int)cudaErrorMisalignedAddress;
  i64 want = rows * kv_heads * (max_ctx > 0 ? max_ctx : 1) / 1024;      // the bf16 path's split rule
  int chunk_tokens = PA_CHUNK_MIN;
  while (chunk_tokens < 512 && chunk_tokens * 2 <= want) chunk_tokens *= 2;
  i64 chunks = (max_ctx + chunk_tokens - 1) / chunk_tokens;
  if (chunks < 1) chunks = 1;
  PagedGeo g{(int)rows, (int)q_heads, (int)kv_heads, (int)page_tokens, page_shift, (int)max_blocks_per_seq, (int)chunks, chunk_tokens, q_row_stride};
  const int G = (int)(q_heads / kv_heads);
  cudaStream_t st = as_stream(stream);
  // head_dim 128 with a GQA group on 16-token pages: the tensor-core unit (needs 16-byte aligned caches and scale planes)
  if (head_dim == 128 && page_tokens == 16 && (G == 2 || G == 4 || G == 8) &&
      ((((uintptr_t)kq) | ((uintptr_t)vq) | ((uintptr_t)kscale) | ((uintptr_t)vscale)) & 15) == 0) {
    // 16 single-warp CTAs are resident per SM: the largest chunk that still gives two waves of units (measured on batch 64 x 8
    // KV heads, contexts up to 4096: 128 / 256 / 512 / 1024-token units stream 2.88 / 3.02 / 2.76 / 2.46 TB/s)
    const i64 slots = (i64)WKB_SM_COUNT * 16;
    chunk_tokens = 512;
    while (chunk_tokens > 128 && rows * kv_heads * ((max_ctx + chunk_tokens - 1) / chunk_tokens) < 2 * slots) chunk_tokens /= 2;
    g.chunk_tokens = chunk_tokens;
    g.max_chunks = (int)((max_ctx + chunk_tokens - 1) / chunk_tokens);
    if (g.max_chunks < 1) g.max_chunks = 1;
    if (G == 2) return launch_decode_i8_mma<2>(q, kq, vq, kscale, vscale, block_table, row_slot, row_ctx, scratch, out, out_dtype, out_row_stride, g, scale, st);
    if (G == 4) return launch_decode_i8_mma<4>(q, kq, vq, kscale, vscale, block_table, row_slot, row_ctx, scratch, out, out_dtype, out_row_stride, g, scale, st);
    return launch_decode_i8_mma<8>(q, kq, vq, kscale, vscale, block_table, row_slot, row_ctx, scratch, out, out_dtype, out_row_stride, g, scale, st);
  }
#define WKB_PA8_CASE(HD_, G_) \
  if (head_dim == HD_ && G == G_) return launch_decode_i8<HD_, G_>(q, kq, vq, kscale, vscale, block_table, row_slot, row_ctx, scratch, out, out_dtype, out_row_stride, g, scale, st);
  WKB_PA8_CASE(64, 1) WKB_PA8_CASE(64, 2) WKB_PA8_CASE(64, 4)
  WKB_PA8_CASE(128, 1) WKB_PA8_CASE(128, 2) WKB_PA8_CASE(128, 4)
#undef WKB_PA8_CASE
  return (int)cudaErrorInvalidValue;
}

}  // extern "C"

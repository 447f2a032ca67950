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
#define WKB_PA8_CASE(HD_, G_) \
  if (head_dim == HD_ && G == G_) return launch_decode_i8<HD_, G_>(q, kq, vq, kscale, vscale, block_table, row_slot, row_ctx, scratch, out, out_dtype, out_row_stride, g, scale, st);
  WKB_PA8_CASE(64, 1) WKB_PA8_CASE(64, 2) WKB_PA8_CASE(64, 4)
  WKB_PA8_CASE(128, 1) WKB_PA8_CASE(128, 2) WKB_PA8_CASE(128, 4)
#undef WKB_PA8_CASE
  return (int)cudaErrorInvalidValue;
}

}  // extern "C"

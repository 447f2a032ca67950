// One decode / prefill-chunk step of the GPT-2-shape model behind the C ABI: the launch sequence a resident serving
// loop replays every step, issued from C++ so that any host (a Rust driver, Python, a C program) calls ONE entry and
// captures it into a CUDA graph if it wishes.
//
// Counterpart in the reference: `DecodeLayer::forward_step_on` (crates/wukong_codegen_gpu/src/serving.rs:684-937),
// `DecodeModel` (:942) and the body of `Scheduler::step_graphed` (:1536-1575): norm -> QKV projection -> KV append
// through the block table -> paged attention -> output projection + residual -> norm -> MLP + residual, 12-14 launches
// per layer there.  Here a layer is 7 launches:
//   1. QKV GEMM (tcgen05) whose epilogue rounds the new K / V rows straight into their pages (no append launch);
//   2. paged decode attention (plus the tiled prefill kernel when the step carries prompt chunks);
//   3. output projection as K-slice partial sums (every SM pulls operands even at 64 rows);
//   4. ONE row kernel: x += bias + sum of the slices (slice order), h = LayerNorm(x) in bf16 -- the residual add, the
//      split-K finish and the next norm in a single pass over the row;
//   5. FC GEMM with bias + GELU -> bf16;  6. down projection as K-slice partials;  7. the row kernel again, normalising
//      with the next layer's first norm (the final norm after the last layer).
// Then the sampled rows of h are gathered and the tied LM head runs with the arg-max fused into its epilogue.
//
// The model object owns no memory: weights, caches, row vectors and one workspace arena are the caller's device
// buffers (sizes from wkb_gpt2_workspace_bytes), so nothing is allocated while stepping.
#include "common.cuh"
#include "wkb_device.h"
#include <vector>

extern "C" {
int wkb_embed_tok_pos_bf16(float*, const void*, const void*, const int*, const int*, i64, i64, i64, i64, void*);
int wkb_gemm_bf16_nt_qkv_append(const void*, i64, const void*, i64, float*, i64, i64, i64, i64, const float*, i64, void*, void*, const uint32_t*,
                                const int*, const int*, i64, i64, i64, i64, void*);
int wkb_gemm_bf16_nt_partial(const void*, i64, const void*, i64, i64, i64, i64, void*, i64, void*);
void wkb_gemm_bf16_partial_layout(i64, i64, i64, i64*, i64*);
int wkb_gemm_bf16_nt_ws(const void*, i64, const void*, i64, void*, i64, int, i64, i64, i64, const float*, i64, const float*, i64, void*, i64, void*);
i64 wkb_gemm_workspace_bytes(i64, i64, i64);
int wkb_gemm_bf16_nt_argmax(const void*, i64, const void*, i64, i64, i64, i64, const float*, float*, int*, int*, void*);
i64 wkb_gemm_argmax_tiles(i64);
int wkb_rowargmax_strided_i32(const float*, int*, i64, i64, i64, void*);
i64 wkb_paged_attn_scratch_bytes(i64, i64, i64, i64);
i64 wkb_paged_attn_decode_launches(i64, i64, i64, i64, i64, int, i64);
int wkb_paged_attn_decode(const float*, i64, const void*, const void*, const uint32_t*, const int*, const int*, void*, int, i64, i64, i64, i64, i64,
                          i64, i64, i64, float, float*, void*);
int wkb_paged_attn_prefill(const float*, i64, const void*, const void*, const uint32_t*, const int*, const int*, const int*, i64, void*, int, i64,
                           i64, i64, i64, i64, i64, float, void*);
int wkb_decode_advance(int*, int*, int*, const int*, i64, i64, void*);
int wkb_gemm_init(void);
int wkb_gemm_b_static(int);
i64 wkb_gemm_bf16_addto_slices(i64, i64, i64);
int wkb_gemm_bf16_nt_addto(const void*, i64, const void*, i64, float*, i64, i64, i64, i64, const float*, void*);
}

namespace wkb {

__device__ __forceinline__ float block_sum_128(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const float r = lane < nw ? red[lane] : 0.0f;
  return warp_sum(r);
}

// x[r, :] += bias + sum_s slices[s][r, :] (slice order; either may be absent), then out[r, :] = bf16(LayerNorm(x[r, :])).
// One CTA of 128 threads per row, a thread keeps VPT 8-element vectors of the row in registers between the update, the
// two-pass statistics (mean, then centred variance -- the sequence of the bf16 LayerNorm kernel) and the write-back.
// (The narrow instantiation is held to 85 registers: all 512 one-row CTAs of a decode batch are then resident beside the
// CTAs of the GEMM that precedes them in the stream and start the moment it completes.)
template <int VPT>
__global__ void __launch_bounds__(128, VPT == 1 ? 6 : 1) add_slices_bias_layernorm_kernel(float* __restrict__ x, const float* __restrict__ slices, int nsl,
                                                                        i64 slice_stride, i64 ld, const float* __restrict__ bias,
                                                                        const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                        u16* __restrict__ out, i64 rows, int cols, float eps) {
  __shared__ float red[32];
  const int nvec = cols >> 3;
  const bool update = nsl > 0 || bias != nullptr;
  pdl_wait();
  pdl_trigger();
  for (i64 r = blockIdx.x; r < rows; r += gridDim.x) {
    float* xr = x + r * (i64)cols;
    float v[VPT][8];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vi = threadIdx.x + k * 128;
      if (vi < nvec) {
        const float4 a = *reinterpret_cast<const float4*>(xr + vi * 8), b = *reinterpret_cast<const float4*>(xr + vi * 8 + 4);
        v[k][0] = a.x; v[k][1] = a.y; v[k][2] = a.z; v[k][3] = a.w; v[k][4] = b.x; v[k][5] = b.y; v[k][6] = b.z; v[k][7] = b.w;
        if (update) {
          float d[8];
          if (nsl > 0) {
            // the loads of four slices are issued together (one trip to L2 per four slices instead of one per slice); the adds
            // run in slice order
            const float* sp = slices + r * ld + vi * 8;
#pragma unroll
            for (int e = 0; e < 8; ++e) d[e] = 0.0f;
            for (int s0 = 0; s0 < nsl; s0 += 4) {
              float4 p[4], q[4];
#pragma unroll
              for (int s = 0; s < 4; ++s) {
                if (s0 + s < nsl) {
                  p[s] = __ldcg(reinterpret_cast<const float4*>(sp + (s0 + s) * slice_stride));
                  q[s] = __ldcg(reinterpret_cast<const float4*>(sp + (s0 + s) * slice_stride + 4));
                }
              }
#pragma unroll
              for (int s = 0; s < 4; ++s) {
                if (s0 + s < nsl) {
                  if (s0 + s == 0) {
                    d[0] = p[s].x; d[1] = p[s].y; d[2] = p[s].z; d[3] = p[s].w; d[4] = q[s].x; d[5] = q[s].y; d[6] = q[s].z; d[7] = q[s].w;
                  } else {
                    d[0] += p[s].x; d[1] += p[s].y; d[2] += p[s].z; d[3] += p[s].w; d[4] += q[s].x; d[5] += q[s].y; d[6] += q[s].z; d[7] += q[s].w;
                  }
                }
              }
            }
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) d[e] = 0.0f;
          }
          if (bias) {
#pragma unroll
            for (int e = 0; e < 8; ++e) d[e] += bias[vi * 8 + e];
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) v[k][e] += d[e];
          *reinterpret_cast<float4*>(xr + vi * 8) = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
          *reinterpret_cast<float4*>(xr + vi * 8 + 4) = make_float4(v[k][4], v[k][5], v[k][6], v[k][7]);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[k][e] = 0.0f;
      }
    }
    if (!out) continue;
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; ++k)
#pragma unroll
      for (int e = 0; e < 8; ++e) s += v[k][e];
    const float mean = block_sum_128(s, red) / (float)cols;
    float q = 0.0f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      if (threadIdx.x + k * 128 < nvec) {
#pragma unroll
        for (int e = 0; e < 8; ++e) { const float dd = v[k][e] - mean; q = fmaf(dd, dd, q); }
      }
    }
    q = block_sum_128(q, red);
    const float scale = rsqrtf(q / (float)cols + eps);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int vi = threadIdx.x + k * 128;
      if (vi < nvec) {
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const float g0 = gamma ? gamma[vi * 8 + e] : 1.0f, g1 = gamma ? gamma[vi * 8 + e + 1] : 1.0f;
          const float b0 = beta ? beta[vi * 8 + e] : 0.0f, b1 = beta ? beta[vi * 8 + e + 1] : 0.0f;
          const float o0 = fmaf((v[k][e] - mean) * scale, g0, b0), o1 = fmaf((v[k][e + 1] - mean) * scale, g1, b1);
          pk[e >> 1] = (uint32_t)f32_to_bf16_bits(o0) | ((uint32_t)f32_to_bf16_bits(o1) << 16);
        }
        *reinterpret_cast<uint4*>(out + r * (i64)cols + vi * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
    }
  }
}

// out[i, :] = src[rows[i], :] for bf16 rows of `cols` elements (cols % 8 == 0); an index outside [0, nsrc) gives zeros.
__global__ void __launch_bounds__(256) gather_rows_bf16_kernel(u16* __restrict__ out, const u16* __restrict__ src, const int* __restrict__ rows,
                                                               i64 n, int cols, i64 nsrc) {
  pdl_wait();
  pdl_trigger();
  const int nvec = cols >> 3;
  const i64 total = n * nvec;
  for (i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    const i64 i = idx / nvec;
    const int vi = (int)(idx % nvec);
    const int r = rows[i];
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    if (r >= 0 && (i64)r < nsrc) w = *reinterpret_cast<const uint4*>(src + (i64)r * cols + vi * 8);
    *reinterpret_cast<uint4*>(out + i * cols + vi * 8) = w;
  }
}

struct Gpt2Layer {
  const float *ln1_g, *ln1_b;
  const void* w_qkv;
  const float* b_qkv;
  const void* w_o;
  const float* b_o;
  const float *ln2_g, *ln2_b;
  const void* w_fc;
  const float* b_fc;
  const void* w_proj;
  const float* b_proj;
};

struct Gpt2Model {
  i64 n_layer, d, n_head, hd, ff, vocab, n_pos, bcap, max_rows, num_pages, mbps, page_tokens;
  float eps, scale;
  const void *wte, *wpe;
  const float *lnf_g, *lnf_b;
  std::vector<Gpt2Layer> layers;
  u16 *kcache, *vcache;
  i64 layer_stride;   // elements between two layers' slabs
  uint32_t* block_table;
  int* rows;          // token | pos | slot | ctx | sample_rows | ctx_dec | tiles (2 vectors), each max_rows int32
  int* next_tok;
  float* logits;      // optional [bcap, ldl]
  i64 ldl;
  // workspace carve-up
  float* x;
  u16* h;
  float* q;
  u16* att;
  u16* ffb;
  u16* hs;
  float* part_val;
  int* part_idx;
  float* attn_scratch;
  float* gemm_ws;
  i64 gemm_ws_bytes;
  i64 attn_scratch_bytes;
  i64 launches;
  // Two-lane execution of a decode-only step: the rows are cut in two halves that run the layer sequence on two
  // streams (rows are independent of each other).  Paged attention is bound by HBM and needs few SM resources, the
  // GEMMs of a 256-512-row step are latency-bound and leave HBM idle: with two lanes one half's attention streams
  // K / V while the other half's GEMMs run.  The side stream and the two events are created with the model.
  cudaStream_t side;
  cudaEvent_t ev_fork, ev_join;
  int two_lanes;      // 0 = never (default), 1 = for decode-only steps of at least 256 rows
};

struct Gpt2Layout {
  i64 off[11], total, gemm_ws_bytes, attn_scratch_bytes;
};

static i64 align_up(i64 v) { return (v + 255) & ~(i64)255; }

static Gpt2Layout gpt2_layout(const i64* dims) {
  const i64 d = dims[1], n_head = dims[2], ff = dims[3], vocab = dims[4], bcap = dims[6], R = dims[7], mbps = dims[9], page = dims[10];
  Gpt2Layout L;
  // K-slice workspace: the largest slices * rows * n over every row count the step can see, for the two partial GEMMs
  // (n = d) and the split shapes of the FC GEMM
  i64 ws = 0;
  for (i64 m = 1; m <= R; ++m) {
    i64 s, st;
    wkb_gemm_bf16_partial_layout(m, d, d, &s, &st);
    if (s * st * 4 > ws) ws = s * st * 4;
    wkb_gemm_bf16_partial_layout(m, d, ff, &s, &st);
    if (s * st * 4 > ws) ws = s * st * 4;
    const i64 w2 = wkb_gemm_workspace_bytes(m, ff, d);
    if (w2 > ws) ws = w2;
  }
  L.gemm_ws_bytes = ws;
  L.attn_scratch_bytes = wkb_paged_attn_scratch_bytes(R, n_head, d / n_head, mbps * page);
  const i64 tiles = wkb_gemm_argmax_tiles(vocab);
  // the K-slice workspace and the attention scratch exist twice: one per lane of a two-lane step
  const i64 sizes[11] = {R * d * 4, R * d * 2, R * d * 4, R * d * 2, R * ff * 2, bcap * d * 2, bcap * tiles * 4, bcap * tiles * 4,
                         L.attn_scratch_bytes, ws, ws};
  i64 o = 0;
  for (int i = 0; i < 11; ++i) { L.off[i] = o; o += align_up(sizes[i]); }
  L.total = o;
  return L;
}

#define WKB_TRY(expr)      \
  do {                     \
    const int _rc = (expr); \
    if (_rc != 0) return _rc; \
  } while (0)

static int add_ln(Gpt2Model* m, float* x, i64 n, const float* slices, i64 nsl, i64 slice_stride, const float* bias, const float* g, const float* b,
                  u16* out, cudaStream_t st) {
  const i64 nvec = m->d / 8;
  const int grid = (int)(n < (i64)WKB_SM_COUNT * 8 ? n : (i64)WKB_SM_COUNT * 8);
  cudaError_t e;
  if (nvec <= 128)
    e = launch_pdl(add_slices_bias_layernorm_kernel<1>, grid, 128, 0, st, x, slices, (int)nsl, slice_stride, m->d, bias, g, b, out, n, (int)m->d, m->eps);
  else if (nvec <= 256)
    e = launch_pdl(add_slices_bias_layernorm_kernel<2>, grid, 128, 0, st, x, slices, (int)nsl, slice_stride, m->d, bias, g, b, out, n, (int)m->d, m->eps);
  else if (nvec <= 512)
    e = launch_pdl(add_slices_bias_layernorm_kernel<4>, grid, 128, 0, st, x, slices, (int)nsl, slice_stride, m->d, bias, g, b, out, n, (int)m->d, m->eps);
  else if (nvec <= 1024)
    e = launch_pdl(add_slices_bias_layernorm_kernel<8>, grid, 128, 0, st, x, slices, (int)nsl, slice_stride, m->d, bias, g, b, out, n, (int)m->d, m->eps);
  else
    return (int)cudaErrorInvalidValue;
  ++m->launches;
  return (int)e;
}

// The layer sequence over rows [r0, r0 + n) on one stream, with that lane's K-slice workspace and attention scratch.
static int run_layers(Gpt2Model* m, i64 r0, i64 n, i64 n_tiles, float* gemm_ws, float* attn_scratch, cudaStream_t st) {
  const i64 R = m->max_rows, d = m->d, ff = m->ff;
  void* stream = (void*)st;
  const int* row_pos = m->rows + R + r0;
  const int* row_slot = m->rows + 2 * R + r0;
  const int* row_ctx = m->rows + 3 * R + r0;
  const int* ctx_dec = n_tiles > 0 ? m->rows + 5 * R + r0 : row_ctx;
  const int* tiles = m->rows + 6 * R;
  float* x = m->x + r0 * d;
  u16* h = m->h + r0 * d;
  float* q = m->q + r0 * d;
  u16* att = m->att + r0 * d;
  u16* ffb = m->ffb + r0 * ff;
  for (i64 li = 0; li < m->n_layer; ++li) {
    const Gpt2Layer& L = m->layers[(size_t)li];
    u16* kc = m->kcache + li * m->layer_stride;
    u16* vc = m->vcache + li * m->layer_stride;
    WKB_TRY(wkb_gemm_bf16_nt_qkv_append(h, d, L.w_qkv, d, q, d, n, 3 * d, d, L.b_qkv, d, kc, vc, m->block_table, row_slot, row_pos, m->n_head, m->hd,
                                        m->page_tokens, m->mbps, stream));
    ++m->launches;
    WKB_TRY(wkb_paged_attn_decode(q, d, kc, vc, m->block_table, row_slot, ctx_dec, att, 1, d, n, m->n_head, m->n_head, m->hd, m->page_tokens, m->mbps,
                                  m->mbps * m->page_tokens, m->scale, attn_scratch, stream));
    m->launches += wkb_paged_attn_decode_launches(n, m->n_head, m->n_head, m->hd, m->mbps * m->page_tokens, 1, d);
    if (n_tiles > 0) {
      WKB_TRY(wkb_paged_attn_prefill(q, d, kc, vc, m->block_table, row_slot, row_ctx, tiles, n_tiles, att, 1, d, m->n_head, m->n_head, m->hd,
                                     m->page_tokens, m->mbps, m->scale, stream));
      ++m->launches;
    }
    i64 nsl, sst;
    // residual update x += att.Wo^T + b_o: K slices summed inside a cluster (then the row kernel only normalises), or as
    // partials that the row kernel adds up.  The cluster form pays from about 512 rows on, where the partials are 6-9 MB
    // of L2 traffic per GEMM (1.653 -> 1.636 ms per step at 512 rows); below that the cluster barrier and the
    // distributed-shared-memory sum cost more than the small partials (0.680 -> 0.705 ms per step at 64 rows).
    const bool in_cluster = n >= 512;
    if (in_cluster && wkb_gemm_bf16_addto_slices(n, d, d) > 0) {
      WKB_TRY(wkb_gemm_bf16_nt_addto(att, d, L.w_o, d, x, d, n, d, d, L.b_o, stream));
      ++m->launches;
      WKB_TRY(add_ln(m, x, n, nullptr, 0, 0, nullptr, L.ln2_g, L.ln2_b, h, st));
    } else {
      wkb_gemm_bf16_partial_layout(n, d, d, &nsl, &sst);
      WKB_TRY(wkb_gemm_bf16_nt_partial(att, d, L.w_o, d, n, d, d, gemm_ws, m->gemm_ws_bytes, stream));
      ++m->launches;
      WKB_TRY(add_ln(m, x, n, gemm_ws, nsl, sst, L.b_o, L.ln2_g, L.ln2_b, h, st));
    }
    WKB_TRY(wkb_gemm_bf16_nt_ws(h, d, L.w_fc, d, ffb, ff, 1, n, ff, d, L.b_fc, 2, nullptr, 0, gemm_ws, m->gemm_ws_bytes, stream));
    m->launches += wkb_gemm_workspace_bytes(n, ff, d) > 0 ? 2 : 1;
    const bool last = li + 1 == m->n_layer;
    const float* g = last ? m->lnf_g : m->layers[(size_t)li + 1].ln1_g;
    const float* b = last ? m->lnf_b : m->layers[(size_t)li + 1].ln1_b;
    if (in_cluster && wkb_gemm_bf16_addto_slices(n, d, ff) > 0) {
      WKB_TRY(wkb_gemm_bf16_nt_addto(ffb, ff, L.w_proj, ff, x, d, n, d, ff, L.b_proj, stream));
      ++m->launches;
      WKB_TRY(add_ln(m, x, n, nullptr, 0, 0, nullptr, g, b, h, st));
    } else {
      wkb_gemm_bf16_partial_layout(n, d, ff, &nsl, &sst);
      WKB_TRY(wkb_gemm_bf16_nt_partial(ffb, ff, L.w_proj, ff, n, d, ff, gemm_ws, m->gemm_ws_bytes, stream));
      ++m->launches;
      WKB_TRY(add_ln(m, x, n, gemm_ws, nsl, sst, L.b_proj, g, b, h, st));
    }
  }
  return 0;
}

}  // namespace wkb

using namespace wkb;

extern "C" {

// dims: n_layer, d_model, n_head, d_ff, vocab, n_pos, bcap, max_rows, num_pages, max_blocks_per_seq, page_tokens,
// eps (bits of the f32, zero extended).
i64 wkb_gpt2_workspace_bytes(const i64* dims) { return gpt2_layout(dims).total; }

// weights: wte, wpe (bf16), lnf_g, lnf_b (f32), then per layer ln1_g, ln1_b, w_qkv (bf16 [3d, d]), b_qkv, w_o (bf16 [d, d]),
// b_o, ln2_g, ln2_b, w_fc (bf16 [ff, d]), b_fc, w_proj (bf16 [d, ff]), b_proj -- 4 + 12 * n_layer device pointers in a HOST
// array.  kcache / vcache: bf16 [n_layer][num_pages][n_head][page_tokens][head_dim].  rows: int32 [8 * max_rows] (token |
// position | slot | visible keys | sampled rows | visible keys of the rows left to the row-per-token kernel | prefill tiles
// x 2).  next_tok: int32 [bcap].  logits_or_null: f32 [bcap, ldl] for keep_logits steps.  Returns null on bad geometry.
void* wkb_gpt2_new(const i64* dims, const void* const* weights, void* kcache, void* vcache, void* block_table, void* rows, void* next_tok,
                   void* workspace, void* logits_or_null, i64 ldl) {
  const i64 n_layer = dims[0], d = dims[1], n_head = dims[2], ff = dims[3], vocab = dims[4];
  if (n_layer <= 0 || d <= 0 || n_head <= 0 || d % n_head != 0 || d % 32 != 0 || ff % 8 != 0 || vocab <= 0 || dims[6] <= 0 || dims[7] < dims[6] ||
      dims[8] <= 0 || dims[9] <= 0 || dims[10] <= 0)
    return nullptr;
  const i64 hd = d / n_head;
  if (hd != 64 && hd != 128) return nullptr;
  if ((((uintptr_t)workspace) | ((uintptr_t)kcache) | ((uintptr_t)vcache)) & 255) return nullptr;
  Gpt2Model* m = new Gpt2Model();
  m->n_layer = n_layer; m->d = d; m->n_head = n_head; m->hd = hd; m->ff = ff; m->vocab = vocab; m->n_pos = dims[5];
  m->bcap = dims[6]; m->max_rows = dims[7]; m->num_pages = dims[8]; m->mbps = dims[9]; m->page_tokens = dims[10];
  m->eps = __builtin_bit_cast(float, (uint32_t)dims[11]);
  m->scale = 1.0f / sqrtf((float)hd);
  m->wte = weights[0]; m->wpe = weights[1]; m->lnf_g = (const float*)weights[2]; m->lnf_b = (const float*)weights[3];
  m->layers.resize((size_t)n_layer);
  for (i64 l = 0; l < n_layer; ++l) {
    const void* const* w = weights + 4 + 12 * l;
    Gpt2Layer& L = m->layers[(size_t)l];
    L.ln1_g = (const float*)w[0]; L.ln1_b = (const float*)w[1]; L.w_qkv = w[2]; L.b_qkv = (const float*)w[3]; L.w_o = w[4];
    L.b_o = (const float*)w[5]; L.ln2_g = (const float*)w[6]; L.ln2_b = (const float*)w[7]; L.w_fc = w[8]; L.b_fc = (const float*)w[9];
    L.w_proj = w[10]; L.b_proj = (const float*)w[11];
  }
  m->kcache = (u16*)kcache; m->vcache = (u16*)vcache;
  m->layer_stride = m->num_pages * n_head * m->page_tokens * hd;
  m->block_table = (uint32_t*)block_table; m->rows = (int*)rows; m->next_tok = (int*)next_tok;
  m->logits = (float*)logits_or_null; m->ldl = ldl;
  const Gpt2Layout L = gpt2_layout(dims);
  char* base = (char*)workspace;
  m->x = (float*)(base + L.off[0]); m->h = (u16*)(base + L.off[1]); m->q = (float*)(base + L.off[2]); m->att = (u16*)(base + L.off[3]);
  m->ffb = (u16*)(base + L.off[4]); m->hs = (u16*)(base + L.off[5]); m->part_val = (float*)(base + L.off[6]); m->part_idx = (int*)(base + L.off[7]);
  m->attn_scratch = (float*)(base + L.off[8]); m->gemm_ws = (float*)(base + L.off[9]); m->gemm_ws_bytes = L.gemm_ws_bytes;
  m->attn_scratch_bytes = L.attn_scratch_bytes;
  m->launches = 0;
  wkb_gemm_init();      // the status word exists before the first step (a step may be the first thing captured)
  m->side = nullptr; m->ev_fork = nullptr; m->ev_join = nullptr;
  // off unless asked for: measured on the 512-sequence serving step it lost (1.97 ms against 1.84 ms per step) -- a GEMM
  // CTA's 197 KB of shared memory keeps the attention CTAs of the other lane off its SM, and every GEMM is issued twice
  const char* env = getenv("WKB_TWO_LANES");
  m->two_lanes = env && env[0] == '1';
  {
    if (cudaStreamCreateWithFlags(&m->side, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&m->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&m->ev_join, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      m->two_lanes = 0;
      m->side = nullptr;
    }
  }
  return m;
}

void wkb_gpt2_delete(void* h) {
  Gpt2Model* m = (Gpt2Model*)h;
  if (!m) return;
  if (m->ev_fork) cudaEventDestroy(m->ev_fork);
  if (m->ev_join) cudaEventDestroy(m->ev_join);
  if (m->side) cudaStreamDestroy(m->side);
  delete m;
}

// 0 / 1: run decode-only steps of at least 256 rows as two lanes on two streams (default 0; the environment variable
// WKB_TWO_LANES=1 turns it on at creation).  Returns the previous setting.
int wkb_gpt2_set_two_lanes(void* h, int on) {
  Gpt2Model* m = (Gpt2Model*)h;
  const int prev = m->two_lanes;
  m->two_lanes = on && m->side ? 1 : 0;
  return prev;
}

// Activation buffers for tests and tools: which = 0 x (f32 [max_rows, d]), 1 h (bf16), 2 q (f32 [max_rows, d]), 3 att (bf16),
// 4 ff (bf16 [max_rows, d_ff]), 5 hs (bf16 [bcap, d]).  Returns the device pointer (null for an unknown code).
void* wkb_gpt2_buffer(void* h, i64 which) {
  Gpt2Model* m = (Gpt2Model*)h;
  switch (which) {
    case 0: return m->x;
    case 1: return m->h;
    case 2: return m->q;
    case 3: return m->att;
    case 4: return m->ffb;
    case 5: return m->hs;
    default: return nullptr;
  }
}

// Kernels the last wkb_gpt2_step call launched.
i64 wkb_gpt2_launches(void* h) { return ((Gpt2Model*)h)->launches; }

// One forward over the first n_rows rows of the row vectors; the n_sample rows listed in the sampled-rows vector reach
// the LM head and their greedy tokens land in next_tok[0 .. n_sample).  n_tiles > 0: the step carries prompt chunks --
// those rows (tile list in the rows block) go through the tiled prefill attention, the row-per-token kernel takes the
// rest (its visible-key vector has the tiled rows zeroed).  keep_logits != 0 materialises fp32 logits (needs the logits
// buffer) instead of fusing the arg-max into the LM head.  Launches only; the caller owns synchronisation.
int wkb_gpt2_step(void* h, i64 n_rows, i64 n_sample, i64 n_tiles, int keep_logits, void* stream) {
  Gpt2Model* m = (Gpt2Model*)h;
  if (n_rows <= 0) return 0;
  if (n_rows > m->max_rows || n_sample < 0 || n_sample > m->bcap || (keep_logits && !m->logits)) return (int)cudaErrorInvalidValue;
  cudaStream_t st = as_stream(stream);
  // every B operand of the step is a resident weight: the GEMMs may fetch it ahead of their stream dependency
  struct WeightsStatic {
    int was;
    WeightsStatic() : was(wkb_gemm_b_static(1)) {}
    ~WeightsStatic() { wkb_gemm_b_static(was); }
  } weights_static;
  const i64 R = m->max_rows, d = m->d, n = n_rows;
  int* row_token = m->rows;
  int* row_pos = m->rows + R;
  int* sample_rows = m->rows + 4 * R;
  m->launches = 0;
  WKB_TRY(wkb_embed_tok_pos_bf16(m->x, m->wte, m->wpe, row_token, row_pos, n, d, m->vocab, m->n_pos, stream));
  ++m->launches;
  WKB_TRY(add_ln(m, m->x, n, nullptr, 0, 0, nullptr, m->layers[0].ln1_g, m->layers[0].ln1_b, m->h, st));
  float* ws2 = (float*)((char*)m->gemm_ws + ((m->gemm_ws_bytes + 255) & ~(i64)255));
  if (m->two_lanes && n_tiles == 0 && n >= 256) {
    // two lanes: rows [0, n0) stay on the caller's stream, rows [n0, n) run on the side stream; fork / join by events
    // (the pattern is capturable: the side stream's work becomes a parallel branch of the caller's graph)
    const i64 n0 = ((n / 2) + 127) / 128 * 128;
    if (cudaEventRecord(m->ev_fork, st) != cudaSuccess || cudaStreamWaitEvent(m->side, m->ev_fork, 0) != cudaSuccess) return (int)cudaGetLastError();
    float* scratch2 = (float*)((char*)m->attn_scratch + wkb_paged_attn_scratch_bytes(n0, m->n_head, m->hd, m->mbps * m->page_tokens));
    WKB_TRY(run_layers(m, n0, n - n0, 0, ws2, scratch2, m->side));
    WKB_TRY(run_layers(m, 0, n0, 0, m->gemm_ws, m->attn_scratch, st));
    if (cudaEventRecord(m->ev_join, m->side) != cudaSuccess || cudaStreamWaitEvent(st, m->ev_join, 0) != cudaSuccess) return (int)cudaGetLastError();
  } else {
    WKB_TRY(run_layers(m, 0, n, n_tiles, m->gemm_ws, m->attn_scratch, st));
  }
  if (n_sample == 0) return 0;
  // LM head on the sampled rows only (LayerNorm is row-wise, so normalising every row and gathering afterwards equals
  // gathering first): gather -> tied head -> arg-max
  {
    const i64 total = n_sample * (d / 8);
    i64 grid = (total + 255) / 256;
    if (grid > (i64)WKB_SM_COUNT * 8) grid = (i64)WKB_SM_COUNT * 8;
    cudaError_t e = launch_pdl(gather_rows_bf16_kernel, (int)grid, 256, 0, st, m->hs, (const u16*)m->h, (const int*)sample_rows, n_sample, (int)d, n);
    if (e != cudaSuccess) return (int)e;
    ++m->launches;
  }
  if (keep_logits) {
    WKB_TRY(wkb_gemm_bf16_nt_ws(m->hs, d, m->wte, d, m->logits, m->ldl, 0, n_sample, m->vocab, d, nullptr, 0, nullptr, 0, m->gemm_ws, m->gemm_ws_bytes, stream));
    WKB_TRY(wkb_rowargmax_strided_i32(m->logits, m->next_tok, n_sample, m->vocab, m->ldl, stream));
  } else {
    WKB_TRY(wkb_gemm_bf16_nt_argmax(m->hs, d, m->wte, d, n_sample, m->vocab, d, nullptr, m->part_val, m->part_idx, m->next_tok, stream));
  }
  m->launches += 2;
  return 0;
}

// Device-side feedback between two decode steps of the first n rows: the sampled token becomes the next input, position
// and visible keys move on by one; a row at the last position its block-table row covers is parked.
int wkb_gpt2_advance(void* h, i64 n, void* stream) {
  Gpt2Model* m = (Gpt2Model*)h;
  const i64 R = m->max_rows;
  return wkb_decode_advance(m->rows, m->rows + R, m->rows + 3 * R, m->next_tok, n, m->mbps * m->page_tokens - 1, stream);
}
}

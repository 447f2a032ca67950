// One decode step of one tensor-parallel rank of the Llama-shape Q4_0 block stack behind the C ABI.
//
// The launch sequence per layer on a rank (reference: the tensor-parallel block validated in
// crates/wukong_codegen_gpu/src/serving.rs:4161-4240 and the decode layer of :684-937):
//   fused QKV W4A16 GEMM (this rank's query / KV heads) -> RoPE at the rows' positions fused with the paged K / V append
//   -> paged GQA decode attention (or the tiled prefill kernel for prompt chunks) -> O projection over this rank's K slice
//   -> [sum over ranks] -> residual add + RMSNorm -> gate / up GEMM with the SwiGLU epilogue -> down projection over this
//   rank's K slice -> [sum over ranks] -> residual add + RMSNorm with the next layer's gain.
// Then the vocabulary-split LM head, the local arg-max and its (value, index) pair; after the pairs of all ranks have
// been gathered, the pick.
//
// The step is cut into numbered phases so that a host that sums over ranks with a collective library can issue its
// collectives between two calls, and so that several ranks emulated on one device can be run in lockstep:
//   0                begin (embedding + first norm)
//   1 + 4 l          attention part of layer l (ends with this rank's O-projection partial)
//   2 + 4 l          after the sum over ranks: residual add + norm
//   3 + 4 l          MLP part of layer l (ends with this rank's down-projection partial)
//   4 + 4 l          after the sum over ranks: residual add + norm (next layer's gain, or the final norm)
//   1 + 4 L          LM head, local arg-max, pair
//   2 + 4 L          pick across ranks (+ step counter bump of the peer-memory reduce)
// With the peer-memory reduce configured (wkb_llama_set_peer) phases 2 + 4 l and 4 + 4 l are this library's fused
// reduce + add + RMSNorm kernel and the whole range 0 .. 1 + 4 L is one call.  On one rank with at most 64 rows the
// split-K second passes of the QKV, O and down projections are folded into the kernels that consume them.
// The object owns no device memory.
#include "common.cuh"
#include "wkb_device.h"
#include <vector>

extern "C" {
int wkb_embedding_f32(float*, const float*, const int*, i64, i64, i64, void*);
int wkb_add_rmsnorm_bf16(float*, const float*, const float*, void*, i64, i64, float, void*);
int wkb_add_slices_rmsnorm_bf16(float*, const float*, i64, i64, i64, const float*, void*, i64, i64, float, void*);
i64 wkb_gemm_q4_0_workspace_bytes(i64, i64);
void wkb_gemm_q4_0_partial_layout(i64, i64, i64*, i64*, i64*);
int wkb_gemm_q4_0_bf16_nt(const void*, const void*, i64, void*, i64, int, i64, i64, i64, void*, i64, void*);
int wkb_rope_qk_paged_append(float*, i64, const float*, const uint32_t*, const int*, const int*, void*, void*, i64, i64, i64, i64, i64, i64, void*);
int wkb_rope_qk_paged_append_slices(float*, i64, const float*, i64, i64, i64, const float*, const uint32_t*, const int*, const int*, void*, void*,
                                    i64, i64, i64, i64, i64, i64, void*);
i64 wkb_paged_attn_scratch_bytes(i64, i64, i64, i64);
int wkb_paged_attn_decode(const float*, i64, const void*, const void*, const uint32_t*, const int*, const int*, void*, int, i64, i64, i64, i64, i64,
                          i64, i64, i64, float, float*, void*);
int wkb_paged_attn_prefill(const float*, i64, const void*, const void*, const uint32_t*, const int*, const int*, const int*, i64, void*, int, i64,
                           i64, i64, i64, i64, i64, float, void*);
int wkb_tp_reduce_add_rmsnorm(const void* const*, void* const*, i64, i64, const void*, i64, i64, float*, const float*, void*, i64, i64, float, void*);
int wkb_tp_step_bump(void*, void*);
int wkb_rowargmax_strided_i32(const float*, int*, i64, i64, i64, void*);
int wkb_argmax_pack(const float*, i64, const int*, i64, i64, int*, void*);
int wkb_argmax_pick(const int*, i64, i64, int*, void*);
int wkb_decode_advance(int*, int*, int*, const int*, i64, i64, void*);
int wkb_gemm_init(void);
}

namespace wkb {

struct LlamaLayer {
  const float *norm1, *norm2;
  const void *wqkv, *wo, *wgu, *wdown;
};

struct LlamaModel {
  i64 n_layer, d, n_head, n_kv_head, hd, ff, vocab, rank, world, bcap, num_pages, mbps, page_tokens;
  i64 hq, hkv, f, vloc, qkv_w;
  float eps, scale;
  const float *embed, *norm_f, *inv_freq;
  const void* lm_head;
  std::vector<LlamaLayer> layers;
  u16 *kcache, *vcache;
  i64 layer_stride;
  uint32_t* block_table;
  int* rows;        // token | position | visible keys | slot, each bcap int32
  int* next_tok;
  float *x, *part, *qkv, *logits, *attn_scratch;
  u16 *xn, *att, *h;
  int *idx_local, *pairs, *all_pairs;
  char* gemm_ws;
  i64 gemm_ws_bytes;
  // peer-memory reduce (optional)
  bool peer;
  const void* part_ptrs[2][8];
  void* flag_ptrs[8];
  void* step_ptr;
  // prompt chunks (optional)
  const int* tiles;
  i64 n_tiles;
  bool fold_slices;   // one rank, <= 64 rows: the O / down split-K second passes are folded into the add + norm that follows
  bool fold_qkv;      // <= 64 rows (any rank count): the QKV projection's second pass is folded into RoPE + append
  i64 launches;
};

struct LlamaLayout {
  i64 off[12], total, gemm_ws_bytes;
};

static i64 ll_align(i64 v) { return (v + 255) & ~(i64)255; }

static void llama_derived(const i64* dims, i64* hq, i64* hkv, i64* f, i64* vloc, i64* qkv_w) {
  const i64 world = dims[7], hd = dims[1] / dims[2];
  *hq = dims[2] / world; *hkv = dims[3] / world; *f = dims[4] / world; *vloc = dims[5] / world;
  *qkv_w = (*hq + 2 * *hkv) * hd;
}

static LlamaLayout llama_layout(const i64* dims) {
  const i64 d = dims[1], hd = dims[1] / dims[2], world = dims[7], R = dims[8], mbps = dims[10], page = dims[11];
  i64 hq, hkv, f, vloc, qkv_w;
  llama_derived(dims, &hq, &hkv, &f, &vloc, &qkv_w);
  LlamaLayout L;
  i64 ws = wkb_gemm_q4_0_workspace_bytes(vloc, d);
  const i64 shapes[4][2] = {{qkv_w, d}, {d, hq * hd}, {2 * f, d}, {d, f}};
  for (auto& s : shapes) {
    const i64 b = wkb_gemm_q4_0_workspace_bytes(s[0], s[1]);
    if (b > ws) ws = b;
  }
  L.gemm_ws_bytes = ws;
  const i64 sizes[12] = {R * d * 4, R * d * 4, R * d * 2, R * qkv_w * 4, R * hq * hd * 2, R * f * 2, R * vloc * 4, R * 4, R * 2 * 4, world * R * 2 * 4,
                         wkb_paged_attn_scratch_bytes(R, hq, hd, mbps * page), ws};
  i64 o = 0;
  for (int i = 0; i < 12; ++i) { L.off[i] = o; o += ll_align(sizes[i]); }
  L.total = o;
  return L;
}

#define WKB_TRY(expr)         \
  do {                        \
    const int _rc = (expr);   \
    if (_rc != 0) return _rc; \
  } while (0)

static int ll_gemm(LlamaModel* m, const void* w, i64 wn, i64 wk, const void* x, i64 ldx, void* out, i64 ldo, int mode, i64 n, void* stream) {
  ++m->launches;
  return wkb_gemm_q4_0_bf16_nt(w, x, ldx, out, ldo, mode, n, wn, wk, m->gemm_ws, m->gemm_ws_bytes, stream);
}

static int ll_add_slices_norm(LlamaModel* m, i64 wn, i64 wk, const float* gain, i64 n, void* stream) {
  i64 nsl, sst, sld;
  wkb_gemm_q4_0_partial_layout(wn, wk, &nsl, &sst, &sld);
  ++m->launches;
  return wkb_add_slices_rmsnorm_bf16(m->x, (const float*)m->gemm_ws, nsl, sst, sld, gain, m->xn, n, m->d, m->eps, stream);
}

static int ll_phase(LlamaModel* m, i64 ph, i64 n, void* stream) {
  const i64 L = m->n_layer, d = m->d, hd = m->hd;
  int* row_token = m->rows;
  int* row_pos = m->rows + m->bcap;
  int* row_ctx = m->rows + 2 * m->bcap;
  int* row_slot = m->rows + 3 * m->bcap;
  if (ph == 0) {
    WKB_TRY(wkb_embedding_f32(m->x, m->embed, row_token, n, d, m->vocab, stream));
    WKB_TRY(wkb_add_rmsnorm_bf16(m->x, nullptr, m->layers[0].norm1, m->xn, n, d, m->eps, stream));
    m->launches += 2;
    return 0;
  }
  if (ph == 1 + 4 * L) {   // LM head on this rank's vocabulary rows
    WKB_TRY(ll_gemm(m, m->lm_head, m->vloc, d, m->xn, d, m->logits, m->vloc, 0, n, stream));
    WKB_TRY(wkb_rowargmax_strided_i32(m->logits, m->idx_local, n, m->vloc, m->vloc, stream));
    WKB_TRY(wkb_argmax_pack(m->logits, m->vloc, m->idx_local, m->rank * m->vloc, n, m->pairs, stream));
    m->launches += 2;
    return 0;
  }
  if (ph == 2 + 4 * L) {
    WKB_TRY(wkb_argmax_pick(m->all_pairs, m->world, m->bcap, m->next_tok, stream));
    ++m->launches;
    if (m->peer) { WKB_TRY(wkb_tp_step_bump(m->step_ptr, stream)); ++m->launches; }
    return 0;
  }
  const i64 li = (ph - 1) / 4, sub = (ph - 1) % 4;
  const LlamaLayer& lw = m->layers[(size_t)li];
  u16* kc = m->kcache + li * m->layer_stride;
  u16* vc = m->vcache + li * m->layer_stride;
  float* part_attn = m->peer ? (float*)m->part_ptrs[0][m->rank] : m->part;
  float* part_mlp = m->peer ? (float*)m->part_ptrs[1][m->rank] : m->part;
  switch (sub) {
    case 0: {   // attention part
      if (m->fold_qkv) {
        i64 nsl, sst, sld;
        wkb_gemm_q4_0_partial_layout(m->qkv_w, d, &nsl, &sst, &sld);
        WKB_TRY(ll_gemm(m, lw.wqkv, m->qkv_w, d, m->xn, d, m->qkv, m->qkv_w, 3, n, stream));
        WKB_TRY(wkb_rope_qk_paged_append_slices(m->qkv, m->qkv_w, (const float*)m->gemm_ws, nsl, sst, sld, m->inv_freq, m->block_table, row_slot,
                                                row_pos, kc, vc, n, m->hq, m->hkv, hd / 2, m->page_tokens, m->mbps, stream));
      } else {
        WKB_TRY(ll_gemm(m, lw.wqkv, m->qkv_w, d, m->xn, d, m->qkv, m->qkv_w, 0, n, stream));
        WKB_TRY(wkb_rope_qk_paged_append(m->qkv, m->qkv_w, m->inv_freq, m->block_table, row_slot, row_pos, kc, vc, n, m->hq, m->hkv, hd / 2,
                                         m->page_tokens, m->mbps, stream));
      }
      ++m->launches;
      if (m->tiles) {
        WKB_TRY(wkb_paged_attn_prefill(m->qkv, m->qkv_w, kc, vc, m->block_table, row_slot, row_ctx, m->tiles, m->n_tiles, m->att, 1, m->hq * hd,
                                       m->hq, m->hkv, hd, m->page_tokens, m->mbps, m->scale, stream));
        ++m->launches;
      } else {
        WKB_TRY(wkb_paged_attn_decode(m->qkv, m->qkv_w, kc, vc, m->block_table, row_slot, row_ctx, m->att, 1, m->hq * hd, n, m->hq, m->hkv, hd,
                                      m->page_tokens, m->mbps, m->mbps * m->page_tokens, m->scale, m->attn_scratch, stream));
        m->launches += 2;
      }
      return ll_gemm(m, lw.wo, d, m->hq * hd, m->att, m->hq * hd, part_attn, d, m->fold_slices ? 3 : 0, n, stream);
    }
    case 1: {   // after the sum over ranks
      ++m->launches;
      if (m->peer)
        return wkb_tp_reduce_add_rmsnorm(m->part_ptrs[0], m->flag_ptrs, m->rank, m->world, m->step_ptr, 2 * li, 2 * L, m->x, lw.norm2, m->xn, n, d,
                                         m->eps, stream);
      if (m->fold_slices) { --m->launches; return ll_add_slices_norm(m, d, m->hq * hd, lw.norm2, n, stream); }
      return wkb_add_rmsnorm_bf16(m->x, m->part, lw.norm2, m->xn, n, d, m->eps, stream);
    }
    case 2: {   // MLP part
      WKB_TRY(ll_gemm(m, lw.wgu, 2 * m->f, d, m->xn, d, m->h, m->f, 2, n, stream));
      return ll_gemm(m, lw.wdown, d, m->f, m->h, m->f, part_mlp, d, m->fold_slices ? 3 : 0, n, stream);
    }
    default: {  // after the sum over ranks
      const float* gain = li + 1 < L ? m->layers[(size_t)li + 1].norm1 : m->norm_f;
      ++m->launches;
      if (m->peer)
        return wkb_tp_reduce_add_rmsnorm(m->part_ptrs[1], m->flag_ptrs, m->rank, m->world, m->step_ptr, 2 * li + 1, 2 * L, m->x, gain, m->xn, n, d,
                                         m->eps, stream);
      if (m->fold_slices) { --m->launches; return ll_add_slices_norm(m, d, m->f, gain, n, stream); }
      return wkb_add_rmsnorm_bf16(m->x, m->part, gain, m->xn, n, d, m->eps, stream);
    }
  }
}

}  // namespace wkb

using namespace wkb;

extern "C" {

// dims: n_layer, d_model, n_head, n_kv_head, d_ff, vocab, rank, world, bcap, num_pages, max_blocks_per_seq, page_tokens,
// eps (bits of the f32, zero extended).
i64 wkb_llama_workspace_bytes(const i64* dims) { return llama_layout(dims).total; }

// weights: embed (f32 [vocab, d]), norm_f (f32 [d]), lm_head (tiled Q4_0 of this rank's vocab / world rows), inv_freq (f32
// [head_dim / 2]), then per layer norm1, norm2 (f32 [d]), wqkv, wo, wgu (gate / up rows interleaved), wdown (tiled Q4_0 of
// this rank's slices, wkb_q4_tile layout) -- 4 + 6 * n_layer device pointers in a HOST array.  kcache / vcache: bf16
// [n_layer][num_pages][n_kv_head / world][page_tokens][head_dim].  rows: int32 [4 * bcap] = token | position | visible
// keys | slot.  next_tok: int32 [bcap].  Returns null on a geometry the kernels do not take.
void* wkb_llama_new(const i64* dims, const void* const* weights, void* kcache, void* vcache, void* block_table, void* rows, void* next_tok,
                    void* workspace) {
  const i64 n_layer = dims[0], d = dims[1], n_head = dims[2], n_kv = dims[3], ffn = dims[4], vocab = dims[5], rank = dims[6], world = dims[7];
  if (n_layer <= 0 || d <= 0 || n_head <= 0 || n_kv <= 0 || d % n_head != 0 || world < 1 || world > 8 || rank < 0 || rank >= world) return nullptr;
  const i64 hd = d / n_head;
  if ((hd != 64 && hd != 128) || d % 32 != 0 || ffn % 32 != 0 || n_kv % world || n_head % world || vocab % world || (ffn / 32) % world) return nullptr;
  if (dims[8] <= 0 || dims[9] <= 0 || dims[10] <= 0 || dims[11] <= 0) return nullptr;
  if ((((uintptr_t)workspace) | ((uintptr_t)kcache) | ((uintptr_t)vcache)) & 255) return nullptr;
  LlamaModel* m = new LlamaModel();
  m->n_layer = n_layer; m->d = d; m->n_head = n_head; m->n_kv_head = n_kv; m->hd = hd; m->ff = ffn; m->vocab = vocab; m->rank = rank; m->world = world;
  m->bcap = dims[8]; m->num_pages = dims[9]; m->mbps = dims[10]; m->page_tokens = dims[11];
  m->eps = __builtin_bit_cast(float, (uint32_t)dims[12]);
  m->scale = 1.0f / sqrtf((float)hd);
  llama_derived(dims, &m->hq, &m->hkv, &m->f, &m->vloc, &m->qkv_w);
  m->embed = (const float*)weights[0]; m->norm_f = (const float*)weights[1]; m->lm_head = weights[2]; m->inv_freq = (const float*)weights[3];
  m->layers.resize((size_t)n_layer);
  for (i64 l = 0; l < n_layer; ++l) {
    const void* const* w = weights + 4 + 6 * l;
    m->layers[(size_t)l] = LlamaLayer{(const float*)w[0], (const float*)w[1], w[2], w[3], w[4], w[5]};
  }
  m->kcache = (u16*)kcache; m->vcache = (u16*)vcache;
  m->layer_stride = m->num_pages * m->hkv * m->page_tokens * hd;
  m->block_table = (uint32_t*)block_table; m->rows = (int*)rows; m->next_tok = (int*)next_tok;
  const LlamaLayout Lo = llama_layout(dims);
  char* b = (char*)workspace;
  m->x = (float*)(b + Lo.off[0]); m->part = (float*)(b + Lo.off[1]); m->xn = (u16*)(b + Lo.off[2]); m->qkv = (float*)(b + Lo.off[3]);
  m->att = (u16*)(b + Lo.off[4]); m->h = (u16*)(b + Lo.off[5]); m->logits = (float*)(b + Lo.off[6]); m->idx_local = (int*)(b + Lo.off[7]);
  m->pairs = (int*)(b + Lo.off[8]); m->all_pairs = (int*)(b + Lo.off[9]); m->attn_scratch = (float*)(b + Lo.off[10]);
  m->gemm_ws = b + Lo.off[11]; m->gemm_ws_bytes = Lo.gemm_ws_bytes;
  m->peer = false; m->step_ptr = nullptr; m->tiles = nullptr; m->n_tiles = 0;
  m->fold_slices = world == 1 && m->bcap <= 64;
  m->fold_qkv = m->bcap <= 64;
  m->launches = 0;
  wkb_gemm_init();
  return m;
}

void wkb_llama_delete(void* h) { delete (LlamaModel*)h; }

// Sum over ranks by this library's fused peer-memory kernel: parts0 / parts1 (HOST arrays of `world` device pointers, by
// rank) are every rank's fp32 [bcap, d] partial buffers for the attention and the MLP sum, flags every rank's flag row,
// step_ptr this rank's device step counter (see wkb_tp_reduce_add_rmsnorm).  The O / down projections then write straight
// into this rank's two buffers.  Null parts0 goes back to the host-summed path.
int wkb_llama_set_peer(void* h, const void* const* parts0, const void* const* parts1, void* const* flags, void* step_ptr) {
  LlamaModel* m = (LlamaModel*)h;
  if (!parts0) { m->peer = false; m->fold_slices = m->world == 1 && m->bcap <= 64; return 0; }
  if (!parts1 || !flags || !step_ptr) return (int)cudaErrorInvalidValue;
  for (i64 r = 0; r < m->world; ++r) { m->part_ptrs[0][r] = parts0[r]; m->part_ptrs[1][r] = parts1[r]; m->flag_ptrs[r] = flags[r]; }
  m->step_ptr = step_ptr;
  m->peer = true;
  m->fold_slices = false;
  return 0;
}

// Prompt chunks: the step's rows are laid out sequence by sequence and covered by `n_tiles` (first row, row count) pairs
// (DEVICE array, see wkb_paged_attn_prefill); attention then runs on the tiled prefill kernel.  Null: one row per sequence.
int wkb_llama_set_prefill_tiles(void* h, const int* tiles_dev, i64 n_tiles) {
  LlamaModel* m = (LlamaModel*)h;
  m->tiles = n_tiles > 0 ? tiles_dev : nullptr;
  m->n_tiles = n_tiles > 0 ? n_tiles : 0;
  return 0;
}

// Buffers a host needs between phases: 0 x (f32 [bcap, d]), 1 part (f32 [bcap, d]: this rank's partial when no peer
// reduce is configured -- sum it over the ranks in place), 2 xn (bf16), 3 qkv (f32 [bcap, qkv width]), 4 att (bf16),
// 5 h (bf16 [bcap, d_ff / world]), 6 logits (f32 [bcap, vocab / world]), 7 pairs (i32 [bcap, 2]), 8 all_pairs (i32 [world,
// bcap, 2]: gather every rank's pairs here before the last phase), 9 attention scratch.
void* wkb_llama_buffer(void* h, i64 which) {
  LlamaModel* m = (LlamaModel*)h;
  switch (which) {
    case 0: return m->x;
    case 1: return m->part;
    case 2: return m->xn;
    case 3: return m->qkv;
    case 4: return m->att;
    case 5: return m->h;
    case 6: return m->logits;
    case 7: return m->pairs;
    case 8: return m->all_pairs;
    case 9: return m->attn_scratch;
    default: return nullptr;
  }
}

i64 wkb_llama_num_phases(void* h) { return 3 + 4 * ((LlamaModel*)h)->n_layer; }
i64 wkb_llama_launches(void* h) { return ((LlamaModel*)h)->launches; }

// Runs phases [phase_begin, phase_end) of one step over the first n rows (see the numbering at the top of this file's
// counterpart in the header).  Launches only.
int wkb_llama_step(void* h, i64 n, i64 phase_begin, i64 phase_end, void* stream) {
  LlamaModel* m = (LlamaModel*)h;
  if (n <= 0 || n > m->bcap || phase_begin < 0 || phase_end > 3 + 4 * m->n_layer) return (int)cudaErrorInvalidValue;
  if (phase_begin == 0) m->launches = 0;
  for (i64 ph = phase_begin; ph < phase_end; ++ph) WKB_TRY(ll_phase(m, ph, n, stream));
  return 0;
}

int wkb_llama_advance(void* h, i64 n, void* stream) {
  LlamaModel* m = (LlamaModel*)h;
  return wkb_decode_advance(m->rows, m->rows + m->bcap, m->rows + 2 * m->bcap, m->next_tok, n, m->mbps * m->page_tokens - 1, stream);
}
}

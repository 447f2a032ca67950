// CPU oracle for the Wukong tensor-builtin hot path.
//
// THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It restates, in portable scalar C++, the numeric
// contracts of the reference's `wukong_runtime` kernels (file:line citations sit on each function
// in the .cpp files).  Only the test-suite, the smoke check and the CPU-baseline leg of the
// benchmark may load it; the CUDA library never links or calls anything declared here.
//
// Parity status: pinned.  Every function below is checked against the golden vectors of the
// reference's own end-to-end fixtures (tests/run/*.wk `EXPECT-OUT` lines, transcribed under
// tests/golden/) and against the constructions of its unit tests.  The two pieces with no
// CPU fixture in the reference -- paged attention values and an f8 GEMM -- are marked
// "parity unpinned (property pinned)" where they are defined.
//
// All exports use the `wko_` prefix so that the oracle and the CUDA library (which exports the
// reference's own `wukong_*` names) can be loaded into one process without symbol clashes.
// Build: -O2 -mavx2 -mfma -mf16c -ffp-contract=off (every fused multiply-add is an explicit fmaf).
#pragma once
#include <cstdint>
#include <cstddef>

#ifdef __cplusplus
extern "C" {
#endif

typedef int64_t i64;
typedef uint8_t u8;
typedef uint16_t u16;

// ---- scalar helpers (exposed for tests) ----
float wko_exp1(float x);
float wko_log1(float x);
float wko_tanh1(float x);
float wko_gelu1(float x);
float wko_silu1(float x);
float wko_sigmoid1(float x);
float wko_sincos1(float x, int is_cos);
u16 wko_f32_to_bf16_bits(float x);
float wko_bf16_bits_to_f32(u16 b);
u16 wko_f32_to_f16_bits(float x);
float wko_f16_bits_to_f32(u16 b);
u8 wko_f32_to_f8e4m3(float x);
float wko_f8e4m3_to_f32(u8 b);
u8 wko_f32_to_f8e5m2(float x);
float wko_f8e5m2_to_f32(u8 b);
i64 wko_select_kc(i64 k);

// ---- elementwise ----
void wko_vmath_f32(const float* x, float* out, i64 n, i64 op);
void wko_vmath2_f32(const float* x, const float* y, float* out, i64 n, i64 op);
void wko_velem_f32(const float* x, const float* y, float* out, i64 n, float a, float b, float c, i64 op);

// ---- norms ----
void wko_norm_f32(const float* x, float* out, i64 rows, i64 cols, i64 eps_bits, i64 op);
void wko_norm_affine_f32(const float* x, float* out, const float* gamma, const float* beta, i64 rows,
                         i64 cols, i64 eps_bits, i64 op);

// ---- GEMM / GEMV ----
void wko_sgemm(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta);
void wko_sgemm_nt(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta);
void wko_sgemm_tn(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta);
void wko_sgemm_nt_epi(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta,
                      const float* bias, i64 act);
void wko_sgemm_nt_alpha(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta, float alpha);
void wko_sgemm_bf16_nt(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta);
void wko_sgemm_f16_nt(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta);
void wko_sgemm_bf16_nt_epi(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta,
                           const float* bias, i64 act);
void wko_sgemv(const float* a, const float* x, float* y, i64 m, i64 n);
void wko_sgemv_alpha(const float* a, const float* x, float* y, i64 m, i64 n, float alpha);
i64 wko_sgemv_bf16(const u16* w, i64 nw, const float* x, i64 nx, float* y, i64 ny);
i64 wko_sgemv_f16(const u16* w, i64 nw, const float* x, i64 nx, float* y, i64 ny);

// ---- block quantisation ----
i64 wko_quantize_q8_0_f32(const float* x, i64 nx, u8* q, i64 nq, i64 k);
i64 wko_quantize_q4_0_f32(const float* x, i64 nx, u8* q, i64 nq, i64 k);
i64 wko_gemv_q8_0_f32(const u8* w, i64 nw, const float* x, i64 nx, float* y, i64 ny);
i64 wko_gemv_q4_0_f32(const u8* w, i64 nw, const float* x, i64 nx, float* y, i64 ny);
i64 wko_dequant_i4_f32(const u8* q, i64 nq, const float* scale, i64 ns, i64 group, float* out, i64 nout);
i64 wko_dequant_u4_f32(const u8* q, i64 nq, const float* scale, i64 ns, const float* zero, i64 nz,
                       i64 group, float* out, i64 nout);
// In-register-dequant variant with bf16 activations (no reference CPU kernel: the defining formula
// y[j] = sum_k f32(d)*(nib-8)*f32(x_bf16[k]) evaluated in f64 and rounded once to f32).
i64 wko_gemv_q4_0_bf16x_f64(const u8* w, i64 nw, const u16* x_bf16, i64 nx, float* y, i64 ny);
void wko_unpack_q4_0(const u8* w, i64 nblocks, int8_t* quants /*32 per block*/, u16* scale_bits);

// ---- attention ----
i64 wko_attention_kv_f32(const float* q, i64 nq, const float* k, i64 nk, const float* v, i64 nv, float* o,
                         i64 no, i64 sq, i64 skv, i64 d, i64 q_pos0, i64 n_heads, i64 n_kv_heads,
                         i64 q_stride, i64 kv_stride, float scale, i64 causal);
i64 wko_attention_kv_batch_f32(const float* q, i64 nq, const float* k, i64 nk, const float* v, i64 nv,
                               float* o, i64 no, const int32_t* kv_lens, i64 nl, const int32_t* q_pos,
                               i64 np, i64 batch, i64 sq, i64 skv, i64 n_heads, i64 n_kv_heads, i64 d,
                               float scale, i64 causal);
i64 wko_kv_append_f32(float* cache, i64 ncache, const float* row, i64 nrow, i64 pos, i64 stride);
void wko_attention_f32(const float* q, const float* k, const float* v, float* o, i64 s, i64 d, float scale,
                       i64 causal);
// Paged GQA decode attention, f64 accumulate, independent of the physical page layout.
// Parity unpinned (property pinned): the reference gates this path only on a GPU, by tolerance
// against an f64 model and by bit-identity across two physical layouts.
// kv_dtype: 0 = f32, 1 = bf16 bits, 2 = f16 bits.  layout 0: [num_blocks, block_size, kv_heads, head_dim]
// (the reference's slab order, paged_kv.rs:139-151); layout 1: [num_blocks, kv_heads, block_size, head_dim].
i64 wko_paged_attn_decode_f64(const float* q, const void* kcache, const void* vcache, int kv_dtype, int layout,
                              const uint32_t* block_table, const int32_t* ctx_lens, float* o, i64 slots,
                              i64 q_heads, i64 kv_heads, i64 head_dim, i64 block_size,
                              i64 max_blocks_per_seq, float scale);

// ---- positional / gather / argmax ----
void wko_rope_f32(const float* x, const float* inv_freq, float* out, i64 rows, i64 half);
// RoPE at explicit positions (no reference entry takes a position vector; same scalar formula).
void wko_rope_pos_f32(const float* x, const float* inv_freq, const int32_t* pos, float* out, i64 rows,
                      i64 heads, i64 half);
void wko_embedding_f32(float* out, const float* weight, const int32_t* ids, i64 t, i64 h, i64 v);
void wko_rowargmax_i32(const float* x, int32_t* out, i64 rows, i64 cols);

/* selection, sampling, RNG: topk.rs:22-136, random.rs:24-104 of the reference runtime */
void wko_philox4x32_10(const uint32_t* ctr4, const uint32_t* key2, uint32_t* out4);
uint32_t wko_rand_u32(uint64_t seed, uint64_t ctr);
void wko_rand_fill_f32(float* out, i64 n, i64 seed, i64 ctr0);
i64 wko_topk_f32(const float* x, i64 n, float* vals, i64 nv, i64* idx, i64 ni);
i64 wko_argsort_f32(const float* x, i64 n, i64* idx, i64 ni, i64 descending);
i64 wko_sample_categorical_f32(const float* p, i64 n, float u);

// ---- threading knob for the timed CPU baseline (rows/units split across threads; results are
// bit-identical to the single-thread run because units are independent) ----
void wko_set_threads(int n);
int wko_get_threads(void);

#ifdef __cplusplus
}
#endif

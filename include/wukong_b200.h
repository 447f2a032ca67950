/* wukong_b200 -- B200 (sm_100a) implementation of the tensor builtins of the Wukong runtime.
 *
 * PART 1 is the drop-in boundary: the `extern "C" wukong_*` symbols of the reference's kernel
 * library (crates/wukong_runtime), same names, argument order, aliasing classes and status codes;
 * the machine-readable signature table they were checked against is
 * crates/wukong_codegen_llvm/src/runtime_abi.rs:7-232.  Pointers are HOST pointers; each call
 * moves its operands to the GPU, runs the CUDA kernel and moves the result back.
 *
 * PART 2 is the device-resident API (`wkb_*`): the same kernels on DEVICE pointers with an explicit
 * stream (a `cudaStream_t` passed as `void*`), plus the pieces a resident decode loop needs that the
 * host ABI cannot express (bf16 storage, paged KV, dense tensor-core GEMM, block allocator,
 * continuous-batching scheduler).  All `wkb_*` functions return 0 on success, a `cudaError_t` value
 * (> 0) on a CUDA failure, or a negative status where documented.
 *
 * Every integer is `int64_t`, every float `float`, System V AMD64.  There is no CPU compute path in
 * this library: without a usable CUDA device PART 1 aborts with a message.
 */
#ifndef WUKONG_B200_H
#define WUKONG_B200_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ======================================= PART 1: runtime ABI ================================== */

/* Status codes of the checked entries (quant.rs:61-65, gemv_half.rs:53-57, attention_kv.rs:97-102). */
#define WUKONG_OK 0
#define WUKONG_KV_BAD_GEOMETRY (-1)
#define WUKONG_BAD_EXTENT (-2) /* QUANT_BAD_EXTENT, GEMV_BAD_EXTENT, KV_SHORT_OPERAND */

/* Activation codes of the fused epilogue (gemm.rs:726-733): 0 identity, 1 relu, 2 gelu(tanh), 3 silu.
 * vmath op codes (vmath.rs:81-116): 0 exp 1 log 2 tanh 3 sigmoid 4 relu 5 silu 6 gelu 15 sin 16 cos;
 * vmath2 (vmath.rs:1506-1512): 9 silu_gate 10 gelu_gate 11 sigmoid_gate (out = act(x) * y).
 * norm op codes (norm.rs:50-54): 0 softmax 1 layernorm 2 rmsnorm 3 log_softmax 4 l2norm.
 * velem op (velem.rs:39-53): low byte 0 id / 1 relu / 2 relu6; |256 use y; |512 Hadamard; |1024 divide. */

/* C[M,N] = A.B (gemm.rs:809), A.B^T (:839), A^T.B (:1245); beta is a 0 / non-0 accumulate flag.
 * Non-positive extents write nothing.  Bit-identical to the reference (order contract gemm.rs:30-58). */
void wukong_sgemm(const float* a, const float* b, float* c, int64_t m, int64_t k, int64_t n, int64_t beta);
void wukong_sgemm_nt(const float* a, const float* b, float* c, int64_t m, int64_t k, int64_t n, int64_t beta);
void wukong_sgemm_tn(const float* a, const float* b, float* c, int64_t m, int64_t k, int64_t n, int64_t beta);
/* c = act(A.B^T + bias[j]) (gemm.rs:873); bias may be null. */
void wukong_sgemm_nt_epi(const float* a, const float* b, float* c, int64_t m, int64_t k, int64_t n, int64_t beta,
                         const float* bias, int64_t act);
/* c = alpha * (A.B^T) (gemm.rs:924). */
void wukong_sgemm_nt_alpha(const float* a, const float* b, float* c, int64_t m, int64_t k, int64_t n, int64_t beta,
                           float alpha);
void wukong_sgemm_parallel(const float*, const float*, float*, int64_t, int64_t, int64_t, int64_t);
void wukong_sgemm_nt_parallel(const float*, const float*, float*, int64_t, int64_t, int64_t, int64_t);
void wukong_sgemm_tn_parallel(const float*, const float*, float*, int64_t, int64_t, int64_t, int64_t);
void wukong_sgemm_nt_epi_parallel(const float*, const float*, float*, int64_t, int64_t, int64_t, int64_t, const float*, int64_t);
void wukong_sgemm_nt_alpha_parallel(const float*, const float*, float*, int64_t, int64_t, int64_t, int64_t, float);

/* Half-storage operands (bf16 / f16 bits), f32 accumulate and output (gemm.rs:1490,1549,1639,1705,1811,1870). */
void wukong_sgemm_bf16_nt(const uint16_t* a, const uint16_t* b, float* c, int64_t m, int64_t k, int64_t n, int64_t beta);
void wukong_sgemm_f16_nt(const uint16_t* a, const uint16_t* b, float* c, int64_t m, int64_t k, int64_t n, int64_t beta);
void wukong_sgemm_bf16_nt_epi(const uint16_t* a, const uint16_t* b, float* c, int64_t m, int64_t k, int64_t n, int64_t beta, const float* bias, int64_t act);
void wukong_sgemm_f16_nt_epi(const uint16_t* a, const uint16_t* b, float* c, int64_t m, int64_t k, int64_t n, int64_t beta, const float* bias, int64_t act);
void wukong_sgemm_bf16_tn(const uint16_t* a, const uint16_t* b, float* c, int64_t m, int64_t k, int64_t n, int64_t beta);
void wukong_sgemm_f16_tn(const uint16_t* a, const uint16_t* b, float* c, int64_t m, int64_t k, int64_t n, int64_t beta);
void wukong_sgemm_bf16_nt_parallel(const uint16_t*, const uint16_t*, float*, int64_t, int64_t, int64_t, int64_t);
void wukong_sgemm_f16_nt_parallel(const uint16_t*, const uint16_t*, float*, int64_t, int64_t, int64_t, int64_t);
void wukong_sgemm_bf16_nt_epi_parallel(const uint16_t*, const uint16_t*, float*, int64_t, int64_t, int64_t, int64_t, const float*, int64_t);
void wukong_sgemm_f16_nt_epi_parallel(const uint16_t*, const uint16_t*, float*, int64_t, int64_t, int64_t, int64_t, const float*, int64_t);
void wukong_sgemm_bf16_tn_parallel(const uint16_t*, const uint16_t*, float*, int64_t, int64_t, int64_t, int64_t);
void wukong_sgemm_f16_tn_parallel(const uint16_t*, const uint16_t*, float*, int64_t, int64_t, int64_t, int64_t);

/* y[M] = (alpha *) A[M,N].x (gemv.rs:197,226): four 8-lane accumulators, fixed trees, unfused tail. */
void wukong_sgemv(const float* a, const float* x, float* y, int64_t m, int64_t n);
void wukong_sgemv_alpha(const float* a, const float* x, float* y, int64_t m, int64_t n, float alpha);
void wukong_sgemv_parallel(const float*, const float*, float*, int64_t, int64_t);
void wukong_sgemv_alpha_parallel(const float*, const float*, float*, int64_t, int64_t, float);
/* y[N] = W[N,K].x with half-storage W (gemv_half.rs:465-529); N = ny, K = nx, nw must be N*K.
 * Returns 0 or -2 (nothing touched).  K = 0 writes zeros. */
int64_t wukong_sgemv_bf16(const uint16_t* w, int64_t nw, const float* x, int64_t nx, float* y, int64_t ny);
int64_t wukong_sgemv_f16(const uint16_t* w, int64_t nw, const float* x, int64_t nx, float* y, int64_t ny);
int64_t wukong_sgemv_bf16_parallel(const uint16_t*, int64_t, const float*, int64_t, float*, int64_t);
int64_t wukong_sgemv_f16_parallel(const uint16_t*, int64_t, const float*, int64_t, float*, int64_t);

/* GGML Q8_0 / Q4_0 packers and GEMV (quant.rs:488-605).  GEMV: x is quantised per call to Q8 with
 * an exact f32 scale, block dots are exact i32, the row accumulates in block order.  Returns 0 / -2. */
int64_t wukong_quantize_q8_0_f32(const float* x, int64_t nx, uint8_t* q, int64_t nq, int64_t k);
int64_t wukong_quantize_q4_0_f32(const float* x, int64_t nx, uint8_t* q, int64_t nq, int64_t k);
int64_t wukong_gemv_q8_0_f32(const uint8_t* w, int64_t nw, const float* x, int64_t nx, float* y, int64_t ny);
int64_t wukong_gemv_q4_0_f32(const uint8_t* w, int64_t nw, const float* x, int64_t nx, float* y, int64_t ny);
int64_t wukong_gemv_q8_0_f32_parallel(const uint8_t*, int64_t, const float*, int64_t, float*, int64_t);
int64_t wukong_gemv_q4_0_f32_parallel(const uint8_t*, int64_t, const float*, int64_t, float*, int64_t);
/* Group-wise int4 (quant.rs:742-800): element i = nibble i&1 of byte i>>1. */
int64_t wukong_dequant_i4_f32(const uint8_t* q, int64_t nq, const float* scale, int64_t ns, int64_t group, float* out, int64_t nout);
int64_t wukong_dequant_u4_f32(const uint8_t* q, int64_t nq, const float* scale, int64_t ns, const float* zero, int64_t nz, int64_t group, float* out, int64_t nout);

/* Elementwise (vmath.rs:1063,1106,2022; velem.rs:212,537).  out may be exactly x. */
void wukong_vmath_f32(const float* x, float* out, int64_t n, int64_t op);
void wukong_vmath_f32_parallel(const float* x, float* out, int64_t n, int64_t op);
void wukong_vmath2_f32(const float* x, const float* y, float* out, int64_t n, int64_t op);
void wukong_velem_f32(const float* x, const float* y, float* out, int64_t n, float a, float b, float c, int64_t op);
void wukong_velem_f32_parallel(const float* x, const float* y, float* out, int64_t n, float a, float b, float c, int64_t op);

/* Row-wise norms (norm.rs:991,1041,1102,1157).  eps_bits = bits of the f32 eps, zero extended.
 * The affine entries take only layernorm / rmsnorm; gamma / beta may be null (1 / 0). */
void wukong_norm_f32(const float* x, float* out, int64_t rows, int64_t cols, int64_t eps_bits, int64_t op);
void wukong_norm_affine_f32(const float* x, float* out, const float* gamma, const float* beta, int64_t rows, int64_t cols, int64_t eps_bits, int64_t op);
void wukong_norm_f32_parallel(const float*, float*, int64_t, int64_t, int64_t, int64_t);
void wukong_norm_affine_f32_parallel(const float*, float*, const float*, const float*, int64_t, int64_t, int64_t, int64_t);

/* Decode attention over a padded KV cache (attention_kv.rs:1050,1099,1207,1255) and the cache
 * append (:1331).  Returns 0, -1 (bad geometry) or -2 (short operand); nothing written on refusal. */
int64_t wukong_attention_kv_f32(const float* q, int64_t nq, const float* k, int64_t nk, const float* v, int64_t nv,
                                float* o, int64_t no, int64_t sq, int64_t skv, int64_t d, int64_t q_pos0,
                                int64_t n_heads, int64_t n_kv_heads, int64_t q_stride, int64_t kv_stride, float scale,
                                int64_t causal);
int64_t wukong_attention_kv_f32_parallel(const float*, int64_t, const float*, int64_t, const float*, int64_t, float*, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, float, int64_t);
int64_t wukong_attention_kv_batch_f32(const float* q, int64_t nq, const float* k, int64_t nk, const float* v,
                                      int64_t nv, float* o, int64_t no, const int32_t* kv_lens, int64_t nl,
                                      const int32_t* q_pos, int64_t np, int64_t batch, int64_t sq, int64_t skv,
                                      int64_t n_heads, int64_t n_kv_heads, int64_t d, float scale, int64_t causal);
int64_t wukong_attention_kv_batch_f32_parallel(const float*, int64_t, const float*, int64_t, const float*, int64_t, float*, int64_t, const int32_t*, int64_t, const int32_t*, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, float, int64_t);
int64_t wukong_kv_append_f32(float* cache, int64_t ncache, const float* row, int64_t nrow, int64_t pos, int64_t stride);
/* Square single-head attention (attention.rs:107). */
void wukong_attention_f32(const float* q, const float* k, const float* v, float* o, int64_t s, int64_t d, float scale, int64_t causal);

/* RoPE half-split, position = row index (rope.rs:143,190); embedding gather (embedding.rs:161,202);
 * per-row arg-max, lowest index wins ties (rowarg.rs:210,227). */
void wukong_rope_f32(const float* x, const float* inv_freq, float* out, int64_t rows, int64_t half);
void wukong_rope_f32_parallel(const float* x, const float* inv_freq, float* out, int64_t rows, int64_t half);
void wukong_embedding_f32(float* out, const float* weight, const int32_t* ids, int64_t t, int64_t h, int64_t v);
void wukong_embedding_f32_parallel(float* out, const float* weight, const int32_t* ids, int64_t t, int64_t h, int64_t v);
void wukong_rowargmax_i32(const float* x, int32_t* out, int64_t rows, int64_t cols);
void wukong_rowargmax_i32_parallel(const float* x, int32_t* out, int64_t rows, int64_t cols);

/* Selection, sampling, RNG (crates/wukong_runtime/src/topk.rs:161-221, random.rs:88-104).  One strict total
 * order: descending = NaN largest, larger first, ties (signed zeros, NaNs) to the lower index; ascending = smaller
 * first, NaN last, stable.  topk writes k = min(n, nv, ni) (value, index) pairs and returns k; the input is read
 * before any output is written.  sample_categorical is the inverse CDF over the positive finite weights with the
 * running mass summed in f64 in index order (-1 when nothing has mass).  rand_fill: out[i] = top 24 bits of
 * Philox4x32-10(key = seed, counter = ctr0 + i) word 0, times 2^-24. */
int64_t wukong_topk_f32(const float* x, int64_t n, float* vals, int64_t nv, int64_t* idx, int64_t ni);
int64_t wukong_argsort_f32(const float* x, int64_t n, int64_t* idx, int64_t ni, int64_t descending);
int64_t wukong_sample_categorical_f32(const float* p, int64_t n, float u);
void wukong_rand_fill_f32(float* out, int64_t n, int64_t seed, int64_t ctr0);

/* ===================================== PART 2: device-resident API ============================ */
/* The reference's GPU path crosses host<->device on every call (crates/wukong_codegen_gpu/src/gpu.rs
 * :1647-1663); these entries are what replaces it.  All pointers are DEVICE pointers. */

int wkb_device_count(void);
const char* wkb_build_arch(void);

int wkb_vmath_f32(const float* x, float* out, int64_t n, int64_t op, void* stream);
int wkb_vmath2_f32(const float* x, const float* y, float* out, int64_t n, int64_t op, void* stream);
int wkb_velem_f32(const float* x, const float* y, float* out, int64_t n, float a, float b, float c, int64_t op, void* stream);
/* bf16 activation, optionally gated: out = act(x) [* y]; op as vmath (4 relu, 5 silu, 6 gelu). */
int wkb_act_bf16(const void* x, const void* y_gate_or_null, void* out, int64_t n, int64_t op, void* stream);

/* fp32 norms, bit-identical to PART 1 (affine != 0 selects the affine entry's semantics). */
int wkb_norm_f32(const float* x, float* out, const float* gamma, const float* beta, int64_t rows, int64_t cols,
                 int64_t eps_bits, int64_t op, int affine, void* stream);
/* Half-precision-path norms: dtype 0 = f32, 1 = bf16; op 0 softmax, 1 layernorm, 2 rmsnorm; f32 gamma /
 * beta (nullable); cols % 8 == 0, cols <= 8192.  Widen, fp32 math, one rounding on the way out. */
int wkb_norm_fast(const void* x, int in_dtype, void* out, int out_dtype, const float* gamma, const float* beta,
                  int64_t rows, int64_t cols, float eps, int64_t op, void* stream);

/* Order-contract GEMM on device operands; dtype 0 f32, 1 bf16 bits, 2 f16 bits (c is always f32). */
int wkb_sgemm_contract(const void* a, int a_dtype, const void* b, int b_dtype, float* c, int64_t m, int64_t k,
                       int64_t n, int64_t beta, int at, int bt, const float* bias, int64_t act, float alpha,
                       int has_epi, void* stream);
int wkb_sgemv_f32(const float* a, const float* x, float* y, int64_t m, int64_t n, float alpha, void* stream);

/* Q4_0 / Q8_0.  wkb_q_split permutes raw 18 / 34-byte blocks into the resident layout: a quant
 * plane (16 / 32 B per block) and an f16 scale plane.  wkb_quantize_act produces the per-call Q8
 * activation (xq [nb*32] i8, dx [nb] f32, sx [nb] i32).  wkb_gemv_q_contract is bit-identical to the
 * reference GEMV; wkb_gemv_q4_0_bf16x is the in-register-dequant form with bf16 activations. */
int wkb_q_split(const uint8_t* raw, void* qs, void* d, int64_t nblocks, int q4, void* stream);
int wkb_quantize_act(const float* x, int64_t k, void* xq, float* dx, int* sx, void* stream);
int wkb_gemv_q_contract(const void* qs, const void* d, const void* xq, const float* dx, const int* sx, float* y,
                        int64_t n, int64_t k, int q4, void* stream);
int wkb_gemv_q4_0_bf16x(const void* qs, const void* d, const void* x_bf16, float* y, int64_t n, int64_t k, void* stream);
/* No counterpart in the reference.  The Q4_0 contract GEMV for callers that must not allocate device
 * memory: the Q8 activation scratch is a fixed device array inside the library, so K <= 32768 (larger K
 * is refused with cudaErrorInvalidValue and a message).  The first call on a device resolves the array's
 * address and should precede any stream capture.  Calls share the array: overlapping calls race. */
int wkb_gemv_q4_0_f32_noalloc(const void* qs, const void* d, const float* x, float* y, int64_t n, int64_t k, void* stream);
int wkb_quantize_q(const float* x, uint8_t* q, int64_t rows, int64_t k, int q4, void* stream);
int wkb_dequant_int4(const uint8_t* q, const float* scale, const float* zero_or_null, int64_t group, float* out, int64_t n, void* stream);

/* fp32 decode attention on device operands (geometry already validated).  kv_lens / q_pos null
 * selects the single-sequence form with (skv, q_pos0). */
int wkb_attention_kv_f32(const float* q, const float* k, const float* v, float* o, const int* kv_lens,
                         const int* q_pos, int64_t batch, int64_t sq, int64_t skv, int64_t d, int64_t q_pos0,
                         int64_t n_heads, int64_t n_kv_heads, int64_t q_stride, int64_t kv_stride, int64_t q_bstride,
                         int64_t kv_bstride, float scale, int64_t causal, void* stream);
int wkb_attention_f32(const float* q, const float* k, const float* v, float* o, int64_t s, int64_t d, float scale, int64_t causal, void* stream);
int wkb_kv_append_f32(float* cache, const float* row, int64_t nrow, int64_t pos, int64_t stride, void* stream);

/* RoPE with an optional position vector (null: position = row); x is [rows, heads, 2*half]. */
int wkb_rope_f32(const float* x, const float* inv_freq, const int* pos_or_null, float* out, int64_t rows, int64_t heads, int64_t half, void* stream);
int wkb_rope_bf16(const void* x, const float* inv_freq, const int* pos, void* out, int64_t rows, int64_t heads, int64_t half, int64_t row_stride, void* stream);
/* RoPE in place on the leading `heads` heads (query heads then key heads) of each fused-QKV row of pitch
 * row_stride floats; same pairing and sin / cos sequence as wkb_rope_f32, position from pos[row]. */
int wkb_rope_qk_f32(float* x, int64_t row_stride, const float* inv_freq, const int* pos, int64_t rows, int64_t heads,
                    int64_t half, void* stream);
/* The two above fused with the paged KV append (wkb_paged_kv_append): one pass over fused QKV rows
 * [q heads | k heads | v heads]; q rotated in place, k rotated and v copied into their bf16 pages at row_pos
 * (which is also the RoPE position); rows with row_pos < 0 are untouched. */
int wkb_rope_qk_paged_append(float* qkv, int64_t row_stride, const float* inv_freq, const uint32_t* block_table, const int* row_slot,
                             const int* row_pos, void* kcache, void* vcache, int64_t rows, int64_t q_heads, int64_t kv_heads,
                             int64_t half, int64_t page_tokens, int64_t max_blocks_per_seq, void* stream);
/* wkb_rope_qk_paged_append reading the fused QKV row as the K-slice partials of its projection (out_mode 3 of
 * wkb_gemm_q4_0_bf16_nt): rotated q heads go to q_out (row pitch row_stride), k and v into their pages. */
int wkb_rope_qk_paged_append_slices(float* q_out, int64_t row_stride, const float* slices, int64_t nslices, int64_t slice_stride,
                                    int64_t ld, const float* inv_freq, const uint32_t* block_table, const int* row_slot,
                                    const int* row_pos, void* kcache, void* vcache, int64_t rows, int64_t q_heads, int64_t kv_heads,
                                    int64_t half, int64_t page_tokens, int64_t max_blocks_per_seq, void* stream);
/* Residual add fused with RMSNorm: x += delta (delta may be null), out = bf16(x / sqrt(mean(x^2) + eps) * gamma);
 * cols % 4 == 0.  The norm is the RMSNORM op of crates/wukong_runtime/src/norm.rs:50-54 in the
 * half-precision recipe (fp32 statistics, one rounding on the way out). */
int wkb_add_rmsnorm_bf16(float* x, const float* delta_or_null, const float* gamma_or_null, void* out_bf16, int64_t rows,
                         int64_t cols, float eps, void* stream);
/* The same with delta given as nslices planes (pitch ld, slice_stride apart) that are added in plane order. */
int wkb_add_slices_rmsnorm_bf16(float* x, const float* slices, int64_t nslices, int64_t slice_stride, int64_t ld,
                                const float* gamma_or_null, void* out_bf16, int64_t rows, int64_t cols, float eps, void* stream);
/* Tensor-parallel sum over ranks fused with the residual add and RMSNorm that follow it, over peer memory
 * (one kernel per rank instead of an all-reduce plus a norm; the reference's counterpart is the all-reduce of its
 * tensor-parallel block, crates/wukong_codegen_gpu/src/serving.rs:4161-4240).  parts[r] / flags[r] (HOST arrays
 * of `world` device pointers, by rank) are every rank's fp32 [rows, cols] partial for this phase and every rank's
 * flag row (>= world uint32, zeroed once), mapped into this process (wkb_ipc_* below, or any peer mapping).
 * x += sum_r parts[r] (rank order on every rank); out = bf16(x / sqrt(mean(x^2) + eps) * gamma).
 * `phase` in [0, phases_per_step) numbers the sums of one decode step; step_ptr is this rank's device step counter
 * (wkb_tp_step_bump once per step, after the step's last sum).  Each rank alternates between two partial buffers.
 * A wait that runs out (about a second) records 21 in the status word read by wkb_gemm_status. */
int wkb_tp_reduce_add_rmsnorm(const void* const* parts, void* const* flags, int64_t rank, int64_t world, const void* step_ptr,
                              int64_t phase, int64_t phases_per_step, float* x, const float* gamma_or_null, void* out_bf16,
                              int64_t rows, int64_t cols, float eps, void* stream);
int wkb_tp_step_bump(void* step_ptr, void* stream);
/* Flag-wait limit of later wkb_tp_reduce_add_rmsnorm launches (process-wide; <= 0: the default, one second).  A rank
 * whose wait runs out records 21, leaves x / out untouched and marks itself dead in every flag row, so every later
 * phase on every rank ends with 22 at once; zero the flag rows to start again. */
void wkb_tp_set_wait_limit_ms(int64_t ms);
/* CUDA IPC plumbing for the peer mappings: export the allocation containing `ptr` as a 64-byte handle plus the
 * offset of `ptr` inside it; map a peer's allocation (add the peer's offset to the returned base). */
int wkb_ipc_export(void* ptr, void* handle64, int64_t* offset);
void* wkb_ipc_import(const void* handle64);
int wkb_ipc_close(void* mapped_ptr);
/* Sampling beyond greedy on device rows: per-row top-k (k <= 4096; k rounds over the row held in shared memory),
 * full argsort (bitonic network; scratch of wkb_argsort_scratch_bytes(n)), per-row categorical draw with the
 * reference's f64 index-order sums, Philox fill.  Same total orders and bits as the PART 1 entries. */
int wkb_rand_fill_f32(float* out, int64_t n, int64_t seed, int64_t ctr0, void* stream);
int wkb_topk_rows_f32(const float* x, int64_t ld, int64_t rows, int64_t cols, int64_t k, float* vals, int64_t* idx, void* stream);
int64_t wkb_argsort_scratch_bytes(int64_t n);
int wkb_argsort_f32(const float* x, int64_t n, float* vals_or_null, int64_t* idx, int64_t m, int64_t descending, void* scratch, void* stream);
int wkb_sample_categorical_rows_f32(const float* p, int64_t ld, int64_t rows, int64_t cols, const float* u, int64_t* out, void* stream);
/* Greedy sampling with the vocabulary split over ranks: pack (value bits, idx_local + col_offset) of each
 * row's local arg-max into pairs[rows][2]; after gathering the ranks' pairs into [world][rows][2], pick the
 * row's token by the arg-max rule of wukong_rowargmax_i32 applied across ranks. */
int wkb_argmax_pack(const float* logits, int64_t ld, const int* idx_local, int64_t col_offset, int64_t rows, int* pairs, void* stream);
int wkb_argmax_pick(const int* pairs, int64_t world, int64_t rows, int* out, void* stream);
int wkb_embedding_f32(float* out, const float* weight, const int* ids, int64_t t, int64_t h, int64_t v, void* stream);
/* out[r] = wte[ids[r]] + wpe[pos[r]] (bf16 tables, f32 out): the GPT-2 input embedding. */
int wkb_embed_tok_pos_bf16(float* out, const void* wte, const void* wpe, const int* ids, const int* pos, int64_t t, int64_t h, int64_t v, int64_t npos, void* stream);
int wkb_rowargmax_i32(const float* x, int* out, int64_t rows, int64_t cols, void* stream);
/* Same with a row pitch ld >= cols (padded logits). */
int wkb_rowargmax_strided_i32(const float* x, int* out, int64_t rows, int64_t cols, int64_t ld, void* stream);
int wkb_add_f32(const float* a, const float* b, float* out, int64_t n, void* stream);
/* Host-side deadline on a stream, after the reference's `sync_within` (crates/wukong_codegen_gpu/src/gpu.rs:250-262,
 * :302): 0 = all work queued on the stream has completed, -1 = timeout_ms passed with work still in flight (nothing is
 * cancelled), > 0 = a CUDA error.  wkb_device_sleep_ms queues a kernel that holds the stream for about ms (<= 2000)
 * milliseconds and then ends by itself: a way to exercise the deadline. */
int wkb_stream_sync_within(void* stream, int64_t timeout_ms);
int wkb_device_sleep_ms(int64_t ms, void* stream);
/* Upload of the live prefix of a step's row vectors (token, position, slot, visible keys, ... stored `pitch_bytes` apart in a
 * pinned host block and in the device block alike): `height` vectors, `width_bytes` bytes of each, one asynchronous 2-D copy
 * (the host side of the reference's per-step upload, crates/wukong_codegen_gpu/src/serving.rs:1536-1575). */
int wkb_upload_rows(void* dst_dev, const void* src_host, int64_t pitch_bytes, int64_t width_bytes, int64_t height, void* stream);
/* Decode feedback on the device: row_token = next_tok, row_pos += 1, row_ctx += 1 for active rows.  A row already at
 * max_pos (the last position its block-table row covers; < 0: no limit) is parked instead: pos = -1, ctx = 0. */
int wkb_decode_advance(int* row_token, int* row_pos, int* row_ctx, const int* next_tok, int64_t n, int64_t max_pos, void* stream);

/* Paged KV cache (behaviour of crates/wukong_codegen_gpu/src/paged_kv.rs:84-151,428-628 and
 * paged_attention.rs:395-534,1343-1410; kernels and HBM layout are this library's own).
 * Per layer the K and V slabs are bf16 [num_pages][kv_heads][page_tokens][head_dim].
 * block_table is [slots, max_blocks_per_seq] u32, padded; a "row" is one query token:
 * row_slot[r] selects its table row, row_ctx[r] is how many leading keys it sees (0: zero output),
 * row_pos[r] is where its own K/V land (< 0: inactive, nothing written).
 * The decode call needs `scratch` of wkb_paged_attn_scratch_bytes(...) bytes; max_ctx bounds row_ctx.
 * head_dim in {64, 128}; q_heads / kv_heads in {1, 2, 4} (and 8 at head_dim 128); out_dtype 0 f32, 1 bf16. */
int64_t wkb_paged_attn_scratch_bytes(int64_t rows, int64_t q_heads, int64_t head_dim, int64_t max_ctx);
/* Kernels one wkb_paged_attn_decode call of this shape launches (1: every row is one unit that writes its own output; 2: units + chunk merge). */
int64_t wkb_paged_attn_decode_launches(int64_t rows, int64_t q_heads, int64_t kv_heads, int64_t head_dim, int64_t max_ctx, int out_dtype,
                                       int64_t out_row_stride);
int wkb_paged_attn_decode(const float* q, int64_t q_row_stride, const void* kcache, const void* vcache,
                          const uint32_t* block_table, const int* row_slot, const int* row_ctx, void* out,
                          int out_dtype, int64_t out_row_stride, int64_t rows, int64_t q_heads, int64_t kv_heads,
                          int64_t head_dim, int64_t page_tokens, int64_t max_blocks_per_seq, int64_t max_ctx,
                          float scale, float* scratch, void* stream);
/* int8 KV cache (the reference's lossy storage option: crates/wukong_codegen_gpu/src/paged_attention.rs:1305-1326,
 * paged_kv.rs:153-178): per (token, KV head) scale = max|x| / 127 (1 for an all-zero row), value = round(x / scale)
 * half away from zero, clamped to +-127 -- bytes and scales identical to the reference's quantizer.  Slabs per layer:
 * int8 [num_pages][kv_heads][page_tokens][head_dim], f32 scales [num_pages][kv_heads][page_tokens].  The decode call
 * has the contract of wkb_paged_attn_decode (same scratch); head_dim in {64, 128}; q_heads / kv_heads in {1, 2, 4}. */
int wkb_paged_kv_append_int8(const float* ksrc, const float* vsrc, int64_t src_row_stride, void* kq, void* vq, float* kscale,
                             float* vscale, const uint32_t* block_table, const int* row_slot, const int* row_pos, int64_t rows,
                             int64_t kv_heads, int64_t head_dim, int64_t page_tokens, int64_t max_blocks_per_seq, void* stream);
int wkb_paged_attn_decode_int8(const float* q, int64_t q_row_stride, const void* kq, const void* vq, const float* kscale,
                               const float* vscale, const uint32_t* block_table, const int* row_slot, const int* row_ctx,
                               void* out, int out_dtype, int64_t out_row_stride, int64_t rows, int64_t q_heads, int64_t kv_heads,
                               int64_t head_dim, int64_t page_tokens, int64_t max_blocks_per_seq, int64_t max_ctx, float scale,
                               float* scratch, void* stream);
/* Prefill / chunked prefill against the same cache (causal, GQA; the reference's counterpart is the flash prefill of
 * crates/wukong_codegen_gpu/src/ptx_flash.rs under the chunked scheduler of serving.rs:1346-1595).  `tiles` is a
 * DEVICE array of n_tiles (first row, row count) int32 pairs; the rows of a tile are consecutive query tokens of ONE
 * sequence, at most wkb_paged_attn_prefill_tile_rows(q_heads, kv_heads) = 128 / (q_heads / kv_heads) of them.  Row r
 * sees its sequence's first row_ctx[r] keys (0: the row is not written).  Keys are streamed once per tile instead of
 * once per row.  head_dim in {64, 128}; q_heads / kv_heads in {1, 2, 4, 8}; out_dtype 0 f32, 1 bf16. */
int64_t wkb_paged_attn_prefill_tile_rows(int64_t q_heads, int64_t kv_heads);
int wkb_paged_attn_prefill(const float* q, int64_t q_row_stride, const void* kcache, const void* vcache,
                           const uint32_t* block_table, const int* row_slot, const int* row_ctx, const int* tiles,
                           int64_t n_tiles, void* out, int out_dtype, int64_t out_row_stride, int64_t q_heads,
                           int64_t kv_heads, int64_t head_dim, int64_t page_tokens, int64_t max_blocks_per_seq, float scale,
                           void* stream);
int wkb_paged_kv_append(const float* ksrc, const float* vsrc, int64_t src_row_stride, void* kcache, void* vcache,
                        const uint32_t* block_table, const int* row_slot, const int* row_pos, int64_t rows,
                        int64_t kv_heads, int64_t head_dim, int64_t page_tokens, int64_t max_blocks_per_seq,
                        void* stream);

/* Page allocator (host; behaviour of paged_kv.rs:428-628): LIFO free list handing out ascending
 * pages on a fresh pool; append allocates only on a page boundary; -1 = out of pages, state unchanged. */
void* wkb_blockmgr_new(int64_t num_blocks, int64_t block_size, int64_t num_slots, int64_t max_blocks_per_seq);
void wkb_blockmgr_delete(void* h);
int64_t wkb_blockmgr_append(void* h, int64_t slot, uint32_t* phys, int64_t* off);
int64_t wkb_blockmgr_reserve(void* h, int64_t slot, int64_t tokens);
void wkb_blockmgr_release(void* h, int64_t slot);
int64_t wkb_blockmgr_can_grow(void* h, int64_t slot, int64_t tokens);
int64_t wkb_blockmgr_free_blocks(void* h);
int64_t wkb_blockmgr_used_blocks(void* h);
int64_t wkb_blockmgr_context_len(void* h, int64_t slot);
int64_t wkb_blockmgr_layout_epoch(void* h);
int64_t wkb_blockmgr_locate(void* h, int64_t slot, int64_t pos, uint32_t* phys, int64_t* off);
void wkb_blockmgr_flat_table(void* h, uint32_t* out);
void wkb_blockmgr_ctx_lens(void* h, int32_t* out);

/* Continuous-batching scheduler (host; behaviour of serving.rs:1346-1595): first-fit admission with
 * a 64-request look-ahead, plan -> run -> commit per step.  plan_step admits first (admission is kept whatever
 * follows), then plans the rows of every slot whose pages fit, decode rows before prompt chunks; a slot that cannot get
 * a page sits the step out.  It returns the row count, 0 when idle, -1 when sequences are resident but no row at all can
 * get a page (terminal unless the caller releases a slot), -3 when the previous step was not committed. */
void* wkb_sched_new(int64_t bcap, int64_t num_blocks, int64_t block_size, int64_t max_blocks_per_seq,
                    int64_t max_rows, int64_t prefill_chunk);
void wkb_sched_delete(void* h);
int64_t wkb_sched_enqueue(void* h, const int32_t* prompt, int64_t prompt_len, int64_t gen_len);
int64_t wkb_sched_plan_step(void* h, int32_t* row_token, int32_t* row_pos, int32_t* row_slot, int32_t* row_ctx,
                            int32_t* sample_row);
int64_t wkb_sched_commit_step(void* h, const int32_t* sampled);
void* wkb_sched_blockmgr(void* h);
int64_t wkb_sched_num_active(void* h);
int64_t wkb_sched_pending(void* h);
int64_t wkb_sched_emitted(void* h);
int64_t wkb_sched_admitted(void* h);
int64_t wkb_sched_completed(void* h);
int64_t wkb_sched_is_idle(void* h);
int64_t wkb_sched_output_len(void* h, int64_t request);
int64_t wkb_sched_output(void* h, int64_t request, int32_t* out, int64_t cap);

/* Dense bf16 GEMM on tcgen05 tensor cores with TMEM accumulators and TMA-fed operands:
 * C[M,N] = act(A[M,K].B[N,K]^T + bias[j]) (+ residual[i,j]); A, B bf16 with row pitches lda / ldb
 * (elements, multiples of 8), C f32 or bf16 (c_bf16) with pitch ldc; fp32 accumulate; K % 8 == 0.
 * Replaces the reference's wmma / wgmma NT families (ptx_wmma.rs, ptx_wgmma.rs) and their fused
 * epilogues.  wkb_gemm_status returns 0 unless a bounded pipeline wait expired (then 1, 2 or 3). */
int wkb_gemm_bf16_nt(const void* a, int64_t lda, const void* b, int64_t ldb, void* c, int64_t ldc, int c_bf16,
                     int64_t m, int64_t n, int64_t k, const float* bias, int64_t act, const float* residual,
                     int64_t ldr, void* stream);
/* Whether a shape splits K is a function of (m, n, k) only; a split shape keeps fp32 partials in a workspace.  This entry
 * uses one default workspace per device, shared by every stream and host thread: at most one split-shaped GEMM may be
 * in flight per device through it.  wkb_gemm_init allocates that workspace (32 MiB) and the status word; call it once
 * per device before capturing into a CUDA graph -- a split-shaped call that finds no workspace while its stream is
 * capturing returns cudaErrorNotReady (600) and launches nothing.  wkb_gemm_bf16_nt_ws is the same GEMM with a caller
 * workspace of at least wkb_gemm_workspace_bytes(m, n, k) bytes (0: the shape does not split), one per stream. */
int wkb_gemm_init(void);
int64_t wkb_gemm_workspace_bytes(int64_t m, int64_t n, int64_t k);
int wkb_gemm_bf16_nt_ws(const void* a, int64_t lda, const void* b, int64_t ldb, void* c, int64_t ldc, int c_bf16,
                        int64_t m, int64_t n, int64_t k, const float* bias, int64_t act, const float* residual,
                        int64_t ldr, void* workspace, int64_t workspace_bytes, void* stream);
/* K-slice partial sums of the same product, no epilogue: slice s goes to workspace + s * slice_stride as an fp32 [m, n]
 * plane, for a consumer that adds the planes in slice order while it does its own row-wise work.  The slice count
 * depends on the shape only (wkb_gemm_bf16_partial_layout); the workspace must hold slices * m * n floats; n % 4 == 0. */
void wkb_gemm_bf16_partial_layout(int64_t m, int64_t n, int64_t k, int64_t* slices, int64_t* slice_stride);
int wkb_gemm_bf16_nt_partial(const void* a, int64_t lda, const void* b, int64_t ldb, int64_t m, int64_t n, int64_t k,
                             void* workspace, int64_t workspace_bytes, void* stream);
/* The fused QKV projection of a decode step (the reference launches the projection and the cache append separately:
 * crates/wukong_codegen_gpu/src/serving.rs:684-937): C[:, :kv_col0] = A.B^T + bias in fp32 (the query heads); columns
 * [kv_col0, kv_col0 + 2 * kv_heads * head_dim) -- the new K rows, then the new V rows -- are rounded to bf16 straight into
 * their pages at row_pos through the block table (the work of wkb_paged_kv_append) and are not stored to C.
 * n = kv_col0 + 2 * kv_heads * head_dim; kv_col0 % 32 == 0 and head_dim % 32 == 0; caches and bias 16-byte aligned. */
int wkb_gemm_bf16_nt_qkv_append(const void* a, int64_t lda, const void* b, int64_t ldb, float* c, int64_t ldc, int64_t m,
                                int64_t n, int64_t k, const float* bias, int64_t kv_col0, void* kcache, void* vcache,
                                const uint32_t* block_table, const int* row_slot, const int* row_pos, int64_t kv_heads,
                                int64_t head_dim, int64_t page_tokens, int64_t max_blocks_per_seq, void* stream);
/* x[m, n] += A.B^T + bias (x f32 with row pitch ldx, updated in place) for decode-sized products: K is cut into 2, 4 or 8
 * slices that run as the CTAs of one thread-block cluster per 128 x 128 tile, and the slices are added -- in slice order,
 * then the bias, then x -- through distributed shared memory, so that no partial leaves the SMs (the residual update of
 * the O and down projections, crates/wukong_codegen_gpu/src/serving.rs:684-937).  wkb_gemm_bf16_addto_slices returns the
 * number of slices for a shape, 0 when the shape is not offered (too many tiles for one wave of clusters, K shorter than
 * three 64-wide steps per slice, n % 4 != 0): then wkb_gemm_bf16_nt_addto returns cudaErrorNotSupported and the caller
 * uses wkb_gemm_bf16_nt_partial.  Results equal the partial path's (same slice order) whenever the slice counts agree. */
int64_t wkb_gemm_bf16_addto_slices(int64_t m, int64_t n, int64_t k);
int wkb_gemm_bf16_nt_addto(const void* a, int64_t lda, const void* b, int64_t ldb, float* x, int64_t ldx, int64_t m,
                           int64_t n, int64_t k, const float* bias, void* stream);
/* Weight-resident hint for the dense tensor-core GEMMs (wkb_gemm_bf16_nt*, per calling thread; returns the previous
 * setting).  While it is non-zero the caller promises that the B operand of every GEMM it launches is not written by a
 * kernel still in flight on the launch's stream (resident model weights): the kernel then requests its first B tiles
 * before it waits for the preceding kernel of the stream, which hides the first weight fetch of a decode-sized GEMM
 * behind that kernel's tail.  A is always read after the preceding kernel.  wkb_gpt2_step sets it around its launches.
 * Results do not depend on the setting. */
int wkb_gemm_b_static(int on);
/* Reads and clears the library's device status word of the current device (synchronises): 0, or the code of the last
 * event -- 1-4 / 11-17 a bounded pipeline wait of the dense / W4A16 GEMM ran out, 21 the tensor-parallel reduce's flag
 * wait ran out (22: a peer had given up), 31 a KV append met a position past its block-table row (the row was skipped),
 * 41 a bounded wait on an asynchronous K/V copy of the paged attention ran out (that unit's output was not written).  The word is one per
 * device, shared by every stream and thread: concurrent users see each other's codes and the read clears them all. */
int wkb_gemm_status(void);

/* W4A16 GEMM on the tensor cores for batched decode: out[m, n] = x[m, k] . W[n, k]^T, x bf16 with row pitch ldx.
 * W is resident in the tiled layout that wkb_q4_tile builds from the reference's raw Q4_0 rows (n rows of k/32
 * 18-byte blocks, crates/wukong_runtime/src/quant.rs:13-16): [tile of 128 rows][stage of 256 K] -> one contiguous
 * 18 KB image (nibble rows, then f16 scales), zero beyond n and k, wkb_q4_tiled_bytes(n, k) bytes in all -- every
 * stage the kernel streams is one contiguous burst of HBM.  The weight the tensor core multiplies is exactly
 * bf16(bf16(d) * (nib - 8)); accumulation is fp32.  out_mode 0: f32 out[m, n]; 1: bf16 out[m, n];
 * 2: SwiGLU -- W rows interleaved (gate_0, up_0, gate_1, up_1, ...), bf16 out[m, n / 2] = silu(gate) * up.
 * Rows are processed 64 at a time.  `workspace` (at least wkb_gemm_q4_0_workspace_bytes(n, k), one per stream)
 * holds the K-slice partial sums, which a second pass adds in slice order: results are run-to-run identical.
 * Counterpart in the reference: the W4A16 tile kernels of crates/wukong_codegen_gpu/src/ptx_int4.rs. */
int64_t wkb_q4_tiled_bytes(int64_t n, int64_t k);
int wkb_q4_tile(const uint8_t* raw, int64_t n, int64_t k, void* tiled, void* stream);
int64_t wkb_gemm_q4_0_workspace_bytes(int64_t n, int64_t k);
/* out_mode 3 (m <= 64): no second pass -- the fp32 K-slice partials stay in the workspace as
 * [slices][64][ld] (this call reports the layout) for a consumer that adds them in slice order while it does its
 * own work: wkb_add_slices_rmsnorm_bf16, wkb_rope_qk_paged_append_slices.  `out` is ignored. */
void wkb_gemm_q4_0_partial_layout(int64_t n, int64_t k, int64_t* slices, int64_t* slice_stride, int64_t* ld);
int wkb_gemm_q4_0_bf16_nt(const void* w_tiled, const void* x_bf16, int64_t ldx, void* out, int64_t ldo, int out_mode,
                          int64_t m, int64_t n, int64_t k, void* workspace, int64_t workspace_bytes, void* stream);
/* The same GEMM over OCP E4M3FN codes (one byte per element, the codec of crates/wukong_runtime/src/fp8.rs
 * :66-164; the reference's GPU counterpart is ptx_fp8.rs `fp8_gemm_nt*`): tcgen05 kind::f8f6f4, fp32
 * accumulate, K % 16 == 0, pitches multiples of 16. */
int wkb_gemm_e4m3_nt(const void* a, int64_t lda, const void* b, int64_t ldb, void* c, int64_t ldc, int c_bf16,
                     int64_t m, int64_t n, int64_t k, const float* bias, int64_t act, const float* residual,
                     int64_t ldr, void* stream);
/* Greedy sampling fused into the LM-head GEMM: out[i] = argmax_j (A.B^T + bias)[i,j]; the logits are
 * never written.  part_val / part_idx are scratch of m * wkb_gemm_argmax_tiles(n) elements each. */
int64_t wkb_gemm_argmax_tiles(int64_t n);
int wkb_gemm_bf16_nt_argmax(const void* a, int64_t lda, const void* b, int64_t ldb, int64_t m, int64_t n, int64_t k,
                            const float* bias, float* part_val, int* part_idx, int* out, void* stream);

/* ---- the GPT-2-shape decode model step behind one call --------------------------------------------------------------
 * The per-step launch sequence of the resident serving loop (reference: `DecodeLayer::forward_step_on`,
 * crates/wukong_codegen_gpu/src/serving.rs:684-937, and the body `Scheduler::step_graphed` replays, :1536-1575), issued
 * by the library so that any host calls one entry per step and may capture it into a CUDA graph.  The object owns no
 * device memory.  dims = {n_layer, d_model, n_head, d_ff, vocab, n_pos, bcap, max_rows, num_pages, max_blocks_per_seq,
 * page_tokens, eps bits}.  weights = HOST array of 4 + 12 * n_layer device pointers: wte, wpe (bf16), lnf_g, lnf_b, then
 * per layer ln1_g, ln1_b, w_qkv (bf16 [3d, d]), b_qkv, w_o (bf16 [d, d]), b_o, ln2_g, ln2_b, w_fc (bf16 [ff, d]), b_fc,
 * w_proj (bf16 [d, ff]), b_proj (vectors f32).  kcache / vcache: bf16 [n_layer][num_pages][n_head][page_tokens][head_dim].
 * rows: int32 [8 * max_rows] = token | position | slot | visible keys | sampled rows | visible keys for the row-per-token
 * kernel | prefill tiles (2 vectors).  next_tok: int32 [bcap].  workspace: wkb_gpt2_workspace_bytes(dims) bytes, 256-byte
 * aligned.  logits_or_null: f32 [bcap, ldl] when steps with keep_logits are wanted.
 * wkb_gpt2_step runs the first n_rows rows; the n_sample rows named in the sampled-rows vector reach the LM head and
 * their greedy tokens land in next_tok[0 .. n_sample).  n_tiles > 0: the step carries prompt chunks (tile list in the rows
 * block, see wkb_paged_attn_prefill).  It only launches (no synchronisation, no allocation).  wkb_gpt2_advance is the
 * device-side token feedback between two decode steps (wkb_decode_advance on the model's own vectors). */
int64_t wkb_gpt2_workspace_bytes(const int64_t* dims);
void* wkb_gpt2_new(const int64_t* dims, const void* const* weights, void* kcache, void* vcache, void* block_table, void* rows,
                   void* next_tok, void* workspace, void* logits_or_null, int64_t ldl);
void wkb_gpt2_delete(void* h);
int wkb_gpt2_step(void* h, int64_t n_rows, int64_t n_sample, int64_t n_tiles, int keep_logits, void* stream);
int wkb_gpt2_advance(void* h, int64_t n, void* stream);
int64_t wkb_gpt2_launches(void* h);
/* Optional two-lane execution of decode-only steps of at least 256 rows: the rows are cut in two halves that walk the
 * layers on two streams (the caller's and one the model created), forked and joined by events, so one half's HBM-bound
 * attention can overlap the other half's latency-bound GEMMs; capturable into a CUDA graph as two parallel branches.
 * Off by default (it measured slower on the 512-sequence serving step); on = 1 or environment WKB_TWO_LANES=1 at creation
 * turns it on.  Returns the previous setting. */
int wkb_gpt2_set_two_lanes(void* h, int on);
/* Activation buffers inside the workspace, for tests and tools: 0 x (f32 [max_rows, d]), 1 h (bf16), 2 q (f32 [max_rows, d]),
 * 3 att (bf16), 4 ff (bf16 [max_rows, d_ff]), 5 hs (bf16 [bcap, d]). */
void* wkb_gpt2_buffer(void* h, int64_t which);

/* ---- one tensor-parallel rank of the Llama-shape Q4_0 decode stack behind one call -----------------------------------
 * The launch sequence of a decode step (reference: the tensor-parallel block validated in
 * crates/wukong_codegen_gpu/src/serving.rs:4161-4240 and the decode layer of :684-937), cut into phases at the two sums
 * over ranks of every layer so that a host can issue its collectives between calls:
 *   0 begin | 1 + 4l attention part of layer l | 2 + 4l add + norm after the sum | 3 + 4l MLP part | 4 + 4l add + norm after
 *   the sum | 1 + 4L LM head, local arg-max, (value, index) pair | 2 + 4L pick across ranks.
 * dims = {n_layer, d_model, n_head, n_kv_head, d_ff, vocab, rank, world, bcap, num_pages, max_blocks_per_seq, page_tokens,
 * eps bits}.  weights = HOST array of 4 + 6 * n_layer device pointers: embed (f32 [vocab, d]), norm_f, lm_head (this rank's
 * vocab / world rows, wkb_q4_tile layout), inv_freq (f32 [head_dim / 2]), then per layer norm1, norm2, wqkv, wo, wgu (gate /
 * up rows interleaved), wdown (this rank's slices, wkb_q4_tile layout).  kcache / vcache: bf16 [n_layer][num_pages]
 * [n_kv_head / world][page_tokens][head_dim].  rows: int32 [4 * bcap] = token | position | visible keys | slot.
 * Without wkb_llama_set_peer the host sums buffer 1 (this rank's fp32 partial) over the ranks after phases 1 + 4l and
 * 3 + 4l; with it those sums are the library's fused peer-memory kernel (wkb_tp_reduce_add_rmsnorm) and phases
 * 0 .. 1 + 4L are one call.  Before the last phase every rank's pairs (buffer 7) must have been gathered into buffer 8.
 * The object owns no device memory; a step only launches. */
int64_t wkb_llama_workspace_bytes(const int64_t* dims);
void* wkb_llama_new(const int64_t* dims, const void* const* weights, void* kcache, void* vcache, void* block_table, void* rows,
                    void* next_tok, void* workspace);
void wkb_llama_delete(void* h);
int wkb_llama_set_peer(void* h, const void* const* parts0, const void* const* parts1, void* const* flags, void* step_ptr);
int wkb_llama_set_prefill_tiles(void* h, const int* tiles_dev, int64_t n_tiles);
/* 0 x, 1 part, 2 xn (bf16), 3 qkv, 4 att (bf16), 5 h (bf16), 6 logits, 7 pairs, 8 all_pairs, 9 attention scratch. */
void* wkb_llama_buffer(void* h, int64_t which);
int64_t wkb_llama_num_phases(void* h);
int64_t wkb_llama_launches(void* h);
int wkb_llama_step(void* h, int64_t n, int64_t phase_begin, int64_t phase_end, void* stream);
int wkb_llama_advance(void* h, int64_t n, void* stream);

/* ---- checkpoint containers (GGUF versions 2 and 3, safetensors) ----------------------------------------------
 * Host readers with the names, arguments, check order and codes of the reference runtime entries
 * (crates/wukong_runtime/src/gguf.rs:809-851 read, :902-918 query, :1026-1062 metadata, :1086-1110 strings;
 * crates/wukong_runtime/src/safetensors.rs:379-407).  dtype codes: 0 f32, 1 f64, 2 f16, 3 bf16, 4 i8, 5 i16,
 * 6 i32, 7 i64, 8 u8, 9 u16, 10 u32, 11 u64 (crates/wukong_runtime/src/fileio.rs:45-67).  A read returns the
 * element count, or -1 (open), -2 (I/O), -3 (dtype), -4 (shape or count), -5 (no such name), -6 (malformed
 * header), -7 (a ggml type with no decoder); rank < 0 means a flat destination, else dims[0..rank) is its shape,
 * outermost first.  A block-quantized GGUF tensor dequantizes into f32 (Q4_0 Q4_1 Q5_0 Q5_1 Q8_0, the K-quants
 * Q2_K..Q6_K and Q8_K, IQ4_NL / IQ4_XS; ggml's reference arithmetic) or loads its raw block bytes into u8;
 * F16 / BF16 widen exactly into f32. */
int64_t wukong_rt_gguf_read(const char* path, const char* name, void* data, int64_t len, int64_t dtype, const int64_t* dims,
                            int64_t rank);
/* what: 0 find (index in the tensor table), 1 rank, 2 dim k (outermost first), 3 ggml type id. */
int64_t wukong_rt_gguf_query(const char* path, const char* name, int64_t what, int64_t k);
/* what: 0 value type id (9 for an array), 1 length (string bytes / array items / 1), 2 value i as i64 or dflt. */
int64_t wukong_rt_gguf_meta(const char* path, const char* key, int64_t what, int64_t i, int64_t dflt);
double wukong_rt_gguf_meta_f64(const char* path, const char* key, int64_t i, double dflt);
int64_t wukong_rt_gguf_meta_str(const char* path, const char* key, int64_t i, char* buf, int64_t len);
int64_t wukong_rt_st_read(const char* path, const char* name, void* data, int64_t len, int64_t dtype, const int64_t* dims,
                          int64_t rank);
/* The same reads with a DEVICE destination: the payload crosses PCIe as the file's own bytes (pinned double
 * buffer) and is dequantized or widened by a kernel on `stream`; values are bit-identical to the host readers'. */
int64_t wkb_gguf_read_device(const char* path, const char* name, void* dev_data, int64_t len, int64_t dtype, const int64_t* dims,
                             int64_t rank, void* stream);
int64_t wkb_st_read_device(const char* path, const char* name, void* dev_data, int64_t len, int64_t dtype, const int64_t* dims,
                           int64_t rank, void* stream);
/* Dequantize `blocks` device-resident blocks of a ggml type into f32 (the kernel the device reads use). */
int wkb_ggml_dequant_f32(int64_t ggml_type_id, const void* raw_dev, int64_t blocks, float* out_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* WUKONG_B200_H */

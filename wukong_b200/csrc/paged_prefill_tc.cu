// Paged prefill attention on the 5th-generation tensor cores: a tile of up to 128 query rows -- (token, head-of-group)
// pairs of consecutive prompt tokens of ONE sequence and one KV head -- against that sequence's paged bf16 K / V
// (causal through each row's visible-key count, GQA).  Same contract as the mma.sync kernel of paged_prefill.cu
// (counterpart in the reference: the flash prefill of crates/wukong_codegen_gpu/src/ptx_flash.rs:19-37 under the chunked
// scheduler of crates/wukong_codegen_gpu/src/serving.rs:1346-1595), with both contractions on tcgen05:
//
//   S = Q . K^T   A = the query tile in shared memory (bf16, pre-scaled by scale * log2 e, K-major, 128-byte swizzle);
//                 B = a block of 128 keys = 8 pages, each page landed by TMA (cp.async.bulk.tensor.2d over the cache seen
//                 as a [token row, head_dim] matrix; 128-byte swizzle; this GPU's memory; no multicast) exactly as the
//                 K-major operand wants it; accumulator: 128 lanes x 128 columns of tensor memory.
//   softmax       four warps, thread = query row = TMEM lane: tcgen05.ld the row's 128 scores, mask by the row's own
//                 visible-key count, online max / sum in base 2, probabilities rounded to bf16 (the normaliser sums the
//                 rounded values) and written back to tensor memory with tcgen05.st.
//   O += P . V    A = P from TENSOR MEMORY; B = the V pages as they lie in the cache ([key][dim], i.e. the MN-major form
//                 of the operand: no transpose pass), fp32 accumulator in tensor memory, rescaled in place when a
//                 row's running maximum moves.
// One CTA = (tile, KV head): 192 threads = TMA producer warp, MMA-issuing warp, four softmax / epilogue warps; K / V
// blocks go through a 2-deep ring.  Keys are streamed once per 128 / G query tokens.  Every index depends on the
// logical key position only.  Every mbarrier wait is bounded (status code WKB_STATUS_ATTN_WAIT, rows left unwritten).
#include "common.cuh"
#include "wkb_device.h"
#include "tc_common.cuh"

namespace wkb {
int* gemm_status_word();

namespace pftc {

constexpr int QROWS = 128, KBLK = 128, THREADS = 192, STAGES = 2;
constexpr int SUB_BYTES = 128 * 128;          // one 64-dim half of a 128-row operand tile: 128 rows x 128 B

struct Geo {
  int n_tiles, q_heads, kv_heads, mbps;
  i64 q_row_stride, out_row_stride;
};

// instruction descriptors, kind::f16: D f32, A = B = bf16; bit 16 = B operand MN-major
__host__ __device__ constexpr uint32_t idesc(int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(QROWS >> 4) << 24);
}
// MN-major operand, 128-byte swizzle: 64 contiguous MN elements (128 B) per K row, 8 K rows per 1024-byte atom;
// leading byte offset = distance between 64-element MN chunks, stride byte offset = distance between 8-row K groups
__device__ __forceinline__ uint64_t make_sdesc_mn(uint32_t saddr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t id, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(id), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tst32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
        "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Shared memory: Q tile | STAGES x (K block, V block) | barriers | tmem slot | tile-wide max of the visible-key counts
template <int HD>
struct Smem {
  static constexpr int NSUB = HD / 64;
  static constexpr int OP_BYTES = NSUB * SUB_BYTES;                 // one 128-row operand (Q, a K block or a V block)
  static constexpr int STAGE_BYTES = 2 * OP_BYTES;
  static constexpr int Q_BYTES = 2 * OP_BYTES;                      // the query tile twice: bf16 hi part and bf16 lo part
  static constexpr int BYTES = Q_BYTES + STAGES * STAGE_BYTES + 1024 /*align*/ + 256;
  static constexpr uint32_t TMEM_COLS = HD == 64 ? 256 : 512;
  static constexpr int S_COL = 0, P_COL = 128, O_COL = HD == 64 ? 192 : 256;
};

template <int HD, int G>
__global__ void __launch_bounds__(THREADS, HD == 64 ? 2 : 1)
paged_attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const float* __restrict__ q,
                             const uint32_t* __restrict__ block_table, const int* __restrict__ row_slot, const int* __restrict__ row_ctx,
                             const int2* __restrict__ tiles, void* __restrict__ out, int out_dtype, Geo g, float scale_log2e,
                             int* __restrict__ status) {
  using SM = Smem<HD>;
  constexpr int NSUB = SM::NSUB;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t q_base = base, ring = base + SM::Q_BYTES;
  const uint32_t bars = ring + STAGES * SM::STAGE_BYTES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + SM::Q_BYTES + STAGES * SM::STAGE_BYTES + 64);
  int* kmax_slot = reinterpret_cast<int*>(gen + SM::Q_BYTES + STAGES * SM::STAGE_BYTES + 72);
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  const uint32_t s_full = bars + 8u * (2 * STAGES), p_full = bars + 8u * (2 * STAGES + 1), o_full = bars + 8u * (2 * STAGES + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.x % g.kv_heads;
  const int2 tile = tiles[blockIdx.x / g.kv_heads];
  const int row0 = tile.x, nrows = min(tile.y, QROWS / G);
  const int live = nrows * G;                      // operand rows in use: a = token * G + head-of-group

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    mbar_init(s_full, 1); mbar_init(p_full, 4); mbar_init(o_full, 1);
    *kmax_slot = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(SM::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  __syncthreads();
  // ---- the query tile: fp32 rows -> bf16, pre-scaled, into the swizzled K-major operand image; rows past `live` are zero
  {
    constexpr int CH = HD / 8;                     // 16-byte chunks per operand row
    for (int idx = threadIdx.x; idx < QROWS * CH; idx += THREADS) {
      const int a = idx / CH, c = idx % CH;
      uint32_t hi[4] = {0u, 0u, 0u, 0u}, lo[4] = {0u, 0u, 0u, 0u};
      if (a < live) {
        const float* qp = q + (i64)(row0 + a / G) * g.q_row_stride + ((i64)kvh * G + a % G) * HD + c * 8;
        const float4 x = *reinterpret_cast<const float4*>(qp), y = *reinterpret_cast<const float4*>(qp + 4);
        const float f[8] = {x.x * scale_log2e, x.y * scale_log2e, x.z * scale_log2e, x.w * scale_log2e,
                            y.x * scale_log2e, y.y * scale_log2e, y.z * scale_log2e, y.w * scale_log2e};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          // q = hi + lo with both parts bf16: the scores then carry about 16 bits of the query
          hi[e] = pack2(f[2 * e], f[2 * e + 1]);
          lo[e] = pack2(f[2 * e] - u2f(hi[e] << 16), f[2 * e + 1] - u2f(hi[e] & 0xffff0000u));
        }
      }
      const uint32_t dst = q_base + (uint32_t)(c >> 3) * SUB_BYTES + (uint32_t)a * 128u + (uint32_t)(((c & 7) ^ (a & 7)) << 4);
      asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(hi[0]), "r"(hi[1]), "r"(hi[2]), "r"(hi[3]) : "memory");
      asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst + SM::OP_BYTES), "r"(lo[0]), "r"(lo[1]), "r"(lo[2]), "r"(lo[3]) : "memory");
    }
    // the tile-wide largest visible-key count decides how many key blocks every role walks
    if (threadIdx.x < QROWS) {
      const int a = threadIdx.x;
      const int c = a < live ? min(row_ctx[row0 + a / G], g.mbps * 16) : 0;
      if (c > 0) atomicMax(kmax_slot, c);
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the MMA reads the query image through the async proxy
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  const int kmax = *kmax_slot;
  const int nkb = (kmax + KBLK - 1) / KBLK;
  const uint32_t* bt = block_table + (i64)row_slot[row0] * g.mbps;

  if (warp == 0) {
    // ---------------- TMA producer: 8 K pages and 8 V pages per key block ----------------
    // lanes 0-7 take one page each (their block-table lookups run side by side, and the next block's are already in
    // flight while this block's ring slot is awaited)
    if (nkb > 0) {
      const int last_page = (kmax - 1) >> 4;
      const int p = lane & 7;
      bool ok = true;
      int kb = 0;
      // pages past the last visible key do not exist: the last real page stands in (its rows are masked / zeroed)
      uint32_t page = bt[min(p, last_page)];
      for (; kb < nkb && ok; ++kb) {
        const int s = kb % STAGES;
        const uint32_t page_next = kb + 1 < nkb ? bt[min(8 * (kb + 1) + p, last_page)] : 0u;
        int good = 1;
        if (lane == 0) {
          good = mbar_wait(empty_bar(s), ((kb / STAGES) & 1) ^ 1) ? 1 : 0;
          if (good) mbar_expect_tx(full_bar(s), SM::STAGE_BYTES);
          else atomicExch(status, WKB_STATUS_ATTN_WAIT);
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) { ok = false; break; }
        if (lane < 8) {
          const uint32_t kdst = ring + s * SM::STAGE_BYTES, vdst = kdst + SM::OP_BYTES;
          const int y = (int)(((i64)page * g.kv_heads + kvh) * 16);
#pragma unroll
          for (int h = 0; h < NSUB; ++h) {
            tma_load_2d(kdst + h * SUB_BYTES + p * 2048, &map_k, full_bar(s), 64 * h, y);
            tma_load_2d(vdst + h * SUB_BYTES + p * 2048, &map_v, full_bar(s), 64 * h, y);
          }
        }
        page = page_next;
      }
      if (!ok && lane == 0)
        for (int j = kb > STAGES ? kb - STAGES : 0; j < kb; ++j) mbar_wait(full_bar(j % STAGES), (j / STAGES) & 1);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t ID_S = idesc(KBLK, false), ID_O = idesc(HD, true);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        const int s = kb % STAGES;
        if (!mbar_wait(full_bar(s), (kb / STAGES) & 1)) { atomicExch(status, WKB_STATUS_ATTN_WAIT); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t kaddr = ring + s * SM::STAGE_BYTES, vaddr = kaddr + SM::OP_BYTES;
        // S = Q . K^T over head_dim in steps of 16 (the previous block's P . V, issued earlier, retires first)
#pragma unroll
        for (int part = 0; part < 2; ++part)
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) {
            const uint32_t off = (uint32_t)(k >> 2) * SUB_BYTES + (uint32_t)(k & 3) * 32u;
            umma_bf16(tmem + SM::S_COL, make_sdesc(q_base + part * SM::OP_BYTES + off), make_sdesc(kaddr + off), ID_S, (part > 0 || k > 0) ? 1u : 0u);
          }
        umma_commit(s_full);
        // O += P . V once the softmax warps have written P (and rescaled O, and zeroed the V rows past the last key)
        if (!mbar_wait(p_full, kb & 1)) { atomicExch(status, WKB_STATUS_ATTN_WAIT); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int k = 0; k < KBLK / 16; ++k)
          umma_ts(tmem + SM::O_COL, tmem + SM::P_COL + (uint32_t)(k * 8), make_sdesc_mn(vaddr + (uint32_t)k * 2048u, SUB_BYTES), ID_O,
                  (kb > 0 || k > 0) ? 1u : 0u);
        umma_commit(empty_bar(s));
        if (kb + 1 == nkb) umma_commit(o_full);
      }
    }
  } else {
    // ---------------- softmax and epilogue: thread = operand row a = TMEM lane ----------------
    const int quarter = warp & 3;
    const int a = quarter * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const int ctx = a < live ? min(row_ctx[row0 + a / G], g.mbps * 16) : 0;
    float m_run = -INFINITY, l_run = 0.0f;
    bool ok = true;
    for (int kb = 0; kb < nkb; ++kb) {
      int good = 1;
      if (lane == 0) good = mbar_wait(s_full, kb & 1) ? 1 : 0;
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) { if (lane == 0) atomicExch(status, WKB_STATUS_ATTN_WAIT); ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int key0 = kb * KBLK;
      const int vis = min(max(ctx - key0, 0), KBLK);          // visible keys of this row inside the block
      // pass 1: the row's maximum over its visible scores
      float bm = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < KBLK; c0 += 32) {
        uint32_t r[32];
        tld32(lane_base + SM::S_COL + c0, r);
#pragma unroll
        for (int e = 0; e < 32; ++e) bm = (c0 + e < vis) ? fmaxf(bm, __uint_as_float(r[e])) : bm;
      }
      const float m_new = fmaxf(m_run, bm);
      const float m_use = m_new == -INFINITY ? 0.0f : m_new;
      const float corr = exp2f(m_run - m_use);                 // 0 for a row that had seen nothing yet
      // pass 2: probabilities, rounded to bf16, into tensor memory as the A operand of P . V (a column = two keys)
      float rs = 0.0f;
#pragma unroll 1
      for (int c0 = 0; c0 < KBLK; c0 += 64) {
        uint32_t pk[32];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t r[32];
          tld32(lane_base + SM::S_COL + c0 + 32 * hh, r);
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const int c = c0 + 32 * hh + e;
            const float p0 = c < vis ? exp2f(__uint_as_float(r[e]) - m_use) : 0.0f;
            const float p1 = c + 1 < vis ? exp2f(__uint_as_float(r[e + 1]) - m_use) : 0.0f;
            const uint32_t w = pack2(p0, p1);
            rs += u2f(w << 16) + u2f(w & 0xffff0000u);
            pk[16 * hh + (e >> 1)] = w;
          }
        }
        tst32(lane_base + SM::P_COL + (c0 >> 1), pk);
      }
      l_run = l_run * corr + rs;
      m_run = m_new;
      // rescale the output accumulator when any row of this warp moved its maximum (the accumulator holds the blocks
      // before this one: their P . V retired before this block's scores did)
      if (kb > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t r[32];
          tld32(lane_base + SM::O_COL + c0, r);
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * corr);
          tst32(lane_base + SM::O_COL + c0, r);
        }
      }
      // the last block may hold key rows that were never written (a partly filled page): their probabilities are zero,
      // but 0 x NaN would still poison the product, so those V rows are zeroed in shared memory first
      if (kb + 1 == nkb && (kmax - key0) < KBLK) {
        const uint32_t vaddr = ring + (kb % STAGES) * SM::STAGE_BYTES + SM::OP_BYTES;
        const int first_bad = kmax - key0;
        for (int idx = (warp - 2) * 32 + lane; idx < (KBLK - first_bad) * NSUB * 8; idx += 128) {
          const int rrow = first_bad + idx / (NSUB * 8), rem = idx % (NSUB * 8);
          asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(vaddr + (uint32_t)(rem >> 3) * SUB_BYTES + (uint32_t)rrow * 128u + (uint32_t)((rem & 7) << 4)),
                       "r"(0u) : "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: normalise and write the rows
    if (ok && nkb > 0) {
      int good = 1;
      if (lane == 0) good = mbar_wait(o_full, 0) ? 1 : 0;
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) { if (lane == 0) atomicExch(status, WKB_STATUS_ATTN_WAIT); ok = false; }
    }
    if (ok && nkb > 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = l_run != 0.0f ? 1.0f / l_run : 0.0f;
      const i64 o = (i64)(row0 + a / G) * g.out_row_stride + ((i64)kvh * G + a % G) * HD;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t r[32];
        tld32(lane_base + SM::O_COL + c0, r);       // every lane of the warp takes part in the load
        if (ctx > 0) {
          if (out_dtype == 0) {
            float4* d = reinterpret_cast<float4*>(static_cast<float*>(out) + o + c0);
#pragma unroll
            for (int e = 0; e < 8; ++e)
              d[e] = make_float4(__uint_as_float(r[4 * e]) * inv, __uint_as_float(r[4 * e + 1]) * inv, __uint_as_float(r[4 * e + 2]) * inv,
                                 __uint_as_float(r[4 * e + 3]) * inv);
          } else {
            uint4* d = reinterpret_cast<uint4*>(static_cast<u16*>(out) + o + c0);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              d[e] = make_uint4(pack2(__uint_as_float(r[8 * e]) * inv, __uint_as_float(r[8 * e + 1]) * inv),
                                pack2(__uint_as_float(r[8 * e + 2]) * inv, __uint_as_float(r[8 * e + 3]) * inv),
                                pack2(__uint_as_float(r[8 * e + 4]) * inv, __uint_as_float(r[8 * e + 5]) * inv),
                                pack2(__uint_as_float(r[8 * e + 6]) * inv, __uint_as_float(r[8 * e + 7]) * inv));
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(SM::TMEM_COLS) : "memory");
  }
}

// The cache of one layer seen as a matrix [token rows][head_dim] of bf16 (token row = ((page * kv_heads + head) * 16 +
// token)); box = 16 rows (one page of one head) x 64 dims, 128-byte swizzle.  The row extent is left open: the kernel
// only addresses pages named by the block table.
static int make_kv_map(CUtensorMap* map, const void* cache, i64 head_dim) {
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

template <int HD, int G>
static int launch(const float* q, const void* kc, const void* vc, const uint32_t* bt, const int* row_slot, const int* row_ctx, const int* tiles,
                  void* out, int out_dtype, Geo g, float scale, cudaStream_t st) {
  CUtensorMap mk, mv;
  int rc = make_kv_map(&mk, kc, HD);
  if (rc) return rc;
  rc = make_kv_map(&mv, vc, HD);
  if (rc) return rc;
  int* status = gemm_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  auto kern = paged_attn_prefill_tc_kernel<HD, G>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<HD>::BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev & 63] = true;
  }
  const i64 blocks = (i64)g.n_tiles * g.kv_heads;
  if (blocks > 0x7fffffff) return (int)cudaErrorInvalidValue;
  kern<<<(unsigned)blocks, THREADS, Smem<HD>::BYTES, st>>>(mk, mv, q, bt, row_slot, row_ctx, (const int2*)tiles, out, out_dtype, g,
                                                           scale * 1.4426950408889634f, status);
  return (int)cudaGetLastError();
}

}  // namespace pftc

// Entry used by wkb_paged_attn_prefill for 16-token pages.  Tiles hold at most 128 / G rows.
int paged_attn_prefill_tc(const float* q, i64 q_row_stride, const void* kcache, const void* vcache, const uint32_t* block_table,
                          const int* row_slot, const int* row_ctx, const int* tiles, i64 n_tiles, void* out, int out_dtype, i64 out_row_stride,
                          i64 q_heads, i64 kv_heads, i64 head_dim, i64 max_blocks_per_seq, float scale, cudaStream_t st) {
  pftc::Geo g{(int)n_tiles, (int)q_heads, (int)kv_heads, (int)max_blocks_per_seq, q_row_stride, out_row_stride};
  const int G = (int)(q_heads / kv_heads);
#define WKB_PFTC_CASE(HD_, G_) \
  if (head_dim == HD_ && G == G_) return pftc::launch<HD_, G_>(q, kcache, vcache, block_table, row_slot, row_ctx, tiles, out, out_dtype, g, scale, st);
  WKB_PFTC_CASE(64, 1) WKB_PFTC_CASE(64, 2) WKB_PFTC_CASE(64, 4) WKB_PFTC_CASE(64, 8)
  WKB_PFTC_CASE(128, 1) WKB_PFTC_CASE(128, 2) WKB_PFTC_CASE(128, 4) WKB_PFTC_CASE(128, 8)
#undef WKB_PFTC_CASE
  return (int)cudaErrorInvalidValue;
}

}  // namespace wkb

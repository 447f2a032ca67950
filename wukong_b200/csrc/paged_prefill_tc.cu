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
//   softmax       eight warps, two threads per query row (= TMEM lane): tcgen05.ld the row's 128 scores, mask by the row's own
//                 visible-key count, online max / sum in base 2, probabilities rounded to bf16 (the normaliser sums the
//                 rounded values) and written back to tensor memory with tcgen05.st.
//   O += P . V    A = P from TENSOR MEMORY; B = the V pages as they lie in the cache ([key][dim], i.e. the MN-major form
//                 of the operand: no transpose pass), fp32 accumulator in tensor memory, rescaled in place when a
//                 row's running maximum moves.
// One CTA = (tile, KV head): 320 threads = TMA producer warp, MMA-issuing warp, eight softmax / epilogue warps (two
// threads per query row); K / V blocks go through a 2-deep ring.  Keys are streamed once per 128 / G query tokens.  Every index depends on the
// logical key position only.  Every mbarrier wait is bounded (status code WKB_STATUS_ATTN_WAIT, rows left unwritten).
#include "common.cuh"
#include "wkb_device.h"
#include "tc_common.cuh"

namespace wkb {
int* gemm_status_word();

namespace pftc {

constexpr int QROWS = 128, KBLK = 128, THREADS = 320, STAGES = 2;   // warps: TMA producer, MMA issuer, 8 x softmax
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
__device__ __forceinline__ void tld32_nowait(uint32_t taddr, uint32_t (&r)[32]) {
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

// Shared memory: Q tile | STAGES x (K block, V block) | barriers (thirteen, 104 bytes) | tmem slot (+128) | tile-wide max of the visible-key counts
template <int HD>
struct Smem {
  static constexpr int NSUB = HD / 64;
  static constexpr int OP_BYTES = NSUB * SUB_BYTES;                 // one 128-row operand (Q, a K block or a V block)
  static constexpr int STAGE_BYTES = 2 * OP_BYTES;
  static constexpr int Q_BYTES = 2 * OP_BYTES;                      // the query tile twice: bf16 hi part and bf16 lo part
  static constexpr int XCH_BYTES = 2 * (2 * 2 * 128 * 4);           // values + sequence numbers traded by the two threads of a row
  static constexpr int BYTES = Q_BYTES + STAGES * STAGE_BYTES + 1024 /*align*/ + 256 + XCH_BYTES;
  // head_dim 128 runs one CTA per SM and double-buffers the scores and the probabilities in tensor memory, so the next
  // block's Q . K^T runs while this block's softmax does; head_dim 64 fits two CTAs per SM (256 columns each), which
  // overlap each other instead
  static constexpr bool DB = HD == 128;
  static constexpr uint32_t TMEM_COLS = DB ? 512 : 256;
  static constexpr int S_COL0 = 0, S_COL1 = DB ? 128 : 0, P_COL0 = DB ? 256 : 128, P_COL1 = DB ? 320 : 128, O_COL = DB ? 384 : 192;
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
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + SM::Q_BYTES + STAGES * SM::STAGE_BYTES + 128);
  int* kmax_slot = reinterpret_cast<int*>(gen + SM::Q_BYTES + STAGES * SM::STAGE_BYTES + 136);
  float* xmax = reinterpret_cast<float*>(gen + SM::Q_BYTES + STAGES * SM::STAGE_BYTES + 256);
  // K and V of a key block travel separately: a K slot is free again once the block's Q . K^T has retired, a V slot once its
  // P . V has, so the load of the K block two ahead starts a whole block earlier than if the two shared a barrier
  auto kfull = [&](int s) { return bars + 8u * s; };
  auto kempty = [&](int s) { return bars + 8u * (STAGES + s); };
  auto vfull = [&](int s) { return bars + 8u * (2 * STAGES + s); };
  auto vempty = [&](int s) { return bars + 8u * (3 * STAGES + s); };
  const uint32_t s_full0 = bars + 8u * (4 * STAGES), p_full = bars + 8u * (4 * STAGES + 1), o_full = bars + 8u * (4 * STAGES + 2);
  const uint32_t s_full1 = bars + 8u * (4 * STAGES + 3), o_done = bars + 8u * (4 * STAGES + 4);
  // score / probability buffer and barrier phase of key block kb
  auto s_bar = [&](int kb) { return (SM::DB && (kb & 1)) ? s_full1 : s_full0; };
  auto s_par = [&](int kb) { return (uint32_t)(SM::DB ? (kb >> 1) & 1 : kb & 1); };
  auto s_col = [&](int kb) { return (uint32_t)((kb & 1) ? SM::S_COL1 : SM::S_COL0); };
  auto p_col = [&](int kb) { return (uint32_t)((kb & 1) ? SM::P_COL1 : SM::P_COL0); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.x % g.kv_heads;
  const int2 tile = tiles[blockIdx.x / g.kv_heads];
  const int row0 = tile.x, nrows = min(tile.y, QROWS / G);
  const int live = nrows * G;                      // operand rows in use: a = token * G + head-of-group

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(kfull(s), 1); mbar_init(kempty(s), 1); mbar_init(vfull(s), 1); mbar_init(vempty(s), 1); }
    mbar_init(s_full0, 1); mbar_init(s_full1, 1); mbar_init(p_full, 8); mbar_init(o_full, 1); mbar_init(o_done, 1);
    *kmax_slot = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(SM::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  // the tile-wide largest visible-key count decides how many key blocks every role walks
  if (threadIdx.x < QROWS) {
    const int a = threadIdx.x;
    const int c = a < live ? min(row_ctx[row0 + a / G], g.mbps * 16) : 0;
    if (c > 0) atomicMax(kmax_slot, c);
  }
  for (int i = threadIdx.x; i < 2 * 2 * QROWS; i += THREADS) reinterpret_cast<int*>(xmax + 2 * 2 * QROWS)[i] = 0;
  __syncthreads();
  const uint32_t tmem = *tmem_slot;
  const int kmax = *kmax_slot;
  const int nkb = (kmax + KBLK - 1) / KBLK;
  // ---- the query tile: fp32 rows -> bf16 hi + lo, pre-scaled, into the swizzled K-major operand image; rows past `live`
  // are zero.  Warps 1-9 do this while the producer warp already has the first key blocks under way.
  if (warp != 0) {
    constexpr int CH = HD / 8;                     // 16-byte chunks per operand row
    for (int idx = threadIdx.x - 32; idx < QROWS * CH; idx += THREADS - 32) {
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
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the MMA reads the query image through the async proxy
    asm volatile("bar.sync 1, %0;" ::"n"(THREADS - 32) : "memory");    // every thread of warps 1-9 gets here unconditionally
  }
  const uint32_t* bt = block_table + (i64)row_slot[row0] * g.mbps;

  if (warp == 0) {
    // ---------------- TMA producer: 8 K pages and 8 V pages per key block ----------------
    // lanes 0-7 take one page each (their block-table lookups run side by side, and the next block's are already in
    // flight while this block's ring slot is awaited)
    if (nkb > 0) {
      const int last_page = (kmax - 1) >> 4;
      const int p = lane & 7;
      bool ok = true;
      // one operand (K or V) of key block kb: lane 0 waits for the slot and arms the barrier, lanes 0-7 issue their page
      auto load = [&](int kb, bool is_v, uint32_t page) {
        const int s = kb % STAGES;
        const uint32_t fb = is_v ? vfull(s) : kfull(s), eb = is_v ? vempty(s) : kempty(s);
        int good = 1;
        if (lane == 0) {
          good = mbar_wait(eb, ((kb / STAGES) & 1) ^ 1) ? 1 : 0;
          if (good) mbar_expect_tx(fb, SM::OP_BYTES);
          else atomicExch(status, WKB_STATUS_ATTN_WAIT);
        }
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) return false;
        if (lane < 8) {
          const uint32_t dst = ring + s * SM::STAGE_BYTES + (is_v ? SM::OP_BYTES : 0);
          const int y = (int)(((i64)page * g.kv_heads + kvh) * 16);
#pragma unroll
          for (int h = 0; h < NSUB; ++h) tma_load_2d(dst + h * SUB_BYTES + p * 2048, is_v ? &map_v : &map_k, fb, 64 * h, y);
        }
        return true;
      };
      // pages past the last visible key do not exist: the last real page stands in (its rows are masked / zeroed)
      uint32_t page = bt[min(p, last_page)];
      int k_issued = 0, v_issued = 0;       // blocks whose K / V loads have been started
      if (SM::DB) {
        // K runs one block ahead of V, the order in which the MMA warp (which issues the next block's Q . K^T before this
        // block's P . V) frees the slots: K(0) K(1) V(0) K(2) V(1) ...
        ok = load(0, false, page);
        if (ok) k_issued = 1;
        for (int kb = 0; kb < nkb && ok; ++kb) {
          const uint32_t page_next = kb + 1 < nkb ? bt[min(8 * (kb + 1) + p, last_page)] : 0u;
          if (kb + 1 < nkb) {
            ok = load(kb + 1, false, page_next);
            if (!ok) break;
            k_issued = kb + 2;
          }
          ok = load(kb, true, page);
          if (!ok) break;
          v_issued = kb + 1;
          page = page_next;
        }
      } else {
        // K(0) V(0) K(1) V(1) ...; the next block's table entry is fetched while this block's slots are awaited
        for (int kb = 0; kb < nkb && ok; ++kb) {
          const uint32_t page_next = kb + 1 < nkb ? bt[min(8 * (kb + 1) + p, last_page)] : 0u;
          ok = load(kb, false, page);
          if (!ok) break;
          k_issued = kb + 1;
          ok = load(kb, true, page);
          if (!ok) break;
          v_issued = kb + 1;
          page = page_next;
        }
      }
      if (!ok && lane == 0) {
        // wait (bounded) for the copies already started before the CTA may exit
        for (int j = k_issued > STAGES ? k_issued - STAGES : 0; j < k_issued; ++j) mbar_wait(kfull(j % STAGES), (j / STAGES) & 1);
        for (int j = v_issued > STAGES ? v_issued - STAGES : 0; j < v_issued; ++j) mbar_wait(vfull(j % STAGES), (j / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t ID_S = idesc(KBLK, false), ID_O = idesc(HD, true);
      bool ok = true;
      // S(kb) = Q . K(kb)^T over head_dim in steps of 16, query hi part then lo part
      auto issue_scores = [&](int kb) {
        const int s = kb % STAGES;
        if (!mbar_wait(kfull(s), (kb / STAGES) & 1)) { atomicExch(status, WKB_STATUS_ATTN_WAIT); return false; }
        // Single-buffered scores: K and V of a block are requested together, so waiting for both here costs nothing and
        // tells the softmax warps (which zero the unwritten V rows of a ragged last block) that V has landed when the
        // scores arrive.  With double-buffered scores they wait for V themselves.
        if (!SM::DB && !mbar_wait(vfull(s), (kb / STAGES) & 1)) {
          atomicExch(status, WKB_STATUS_ATTN_WAIT);
          return false;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t kaddr = ring + s * SM::STAGE_BYTES;
#pragma unroll
        for (int part = 0; part < 2; ++part)
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) {
            const uint32_t off = (uint32_t)(k >> 2) * SUB_BYTES + (uint32_t)(k & 3) * 32u;
            umma_bf16(tmem + s_col(kb), make_sdesc(q_base + part * SM::OP_BYTES + off), make_sdesc(kaddr + off), ID_S, (part > 0 || k > 0) ? 1u : 0u);
          }
        umma_commit(s_bar(kb));
        umma_commit(kempty(s));
        return true;
      };
      if (SM::DB && nkb > 0) ok = issue_scores(0);
      for (int kb = 0; kb < nkb && ok; ++kb) {
        // double-buffered: the next block's scores are issued before this block's P . V, so they are computed while the
        // softmax warps work on this block (the buffer they go to was released with the block before this one)
        if (SM::DB) { if (kb + 1 < nkb) ok = issue_scores(kb + 1); }
        else ok = issue_scores(kb);
        if (!ok) break;
        // O += P . V once the softmax warps have written P (and rescaled O, and zeroed the V rows past the last key)
        if (!mbar_wait(p_full, kb & 1) || !mbar_wait(vfull(kb % STAGES), (kb / STAGES) & 1)) { atomicExch(status, WKB_STATUS_ATTN_WAIT); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t vaddr = ring + (kb % STAGES) * SM::STAGE_BYTES + SM::OP_BYTES;
#pragma unroll
        for (int k = 0; k < KBLK / 16; ++k)
          umma_ts(tmem + SM::O_COL, tmem + p_col(kb) + (uint32_t)(k * 8), make_sdesc_mn(vaddr + (uint32_t)k * 2048u, SUB_BYTES), ID_O,
                  (kb > 0 || k > 0) ? 1u : 0u);
        umma_commit(vempty(kb % STAGES));
        umma_commit(o_done);
        if (kb + 1 == nkb) umma_commit(o_full);
      }
    }
  } else {
    // ---------------- softmax and epilogue: eight warps, two threads per operand row ----------------
    // A warp reaches the 32 TMEM lanes of its quarter (warp % 4); warps w and w + 4 share a quarter and split a row's
    // 128 keys (and the output's columns) in two halves.  With one warp per scheduler the exponentials and the
    // dependent max / sum chains were the slowest part of a key block, so the halves double the warps in flight, the
    // scores of a half stay in registers (one pass, two loads in flight), the chains are split four ways and the
    // unmasked interior blocks skip the mask.
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int a = quarter * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const int ctx = a < live ? min(row_ctx[row0 + a / G], g.mbps * 16) : 0;
    const int sm_tid = (warp - 2) * 32 + lane;               // 0 .. 255 over the softmax warps
    float m_run = -INFINITY, l_run = 0.0f;                   // l_run: this thread's half of the row's normaliser
    bool ok = true;
    auto ex2 = [](float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; };
    // The two threads of a row trade one float per key block through shared memory: value, then a sequence number; the
    // reader polls the partner's sequence number a bounded number of times (no barrier instruction: a barrier that one
    // side never reaches cannot be bounded).  Slots alternate by block parity, so a writer two blocks ahead is the
    // earliest that could touch a slot again, and it cannot be two ahead before its partner has read this one.
    volatile float* xval = xmax;
    volatile int* xseq = reinterpret_cast<volatile int*>(xmax + 2 * 2 * QROWS);
    auto exchange = [&](int seq, float mine, float& theirs) {
      const int me = ((seq & 1) * 2 + half) * QROWS + a, them = ((seq & 1) * 2 + (half ^ 1)) * QROWS + a;
      xval[me] = mine;
      __threadfence_block();
      xseq[me] = seq + 1;
      for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
        if (xseq[them] == seq + 1) { __threadfence_block(); theirs = xval[them]; return true; }
      }
      return false;
    };
    for (int kb = 0; kb < nkb; ++kb) {
      int good = 1;
      if (lane == 0) good = mbar_wait(s_bar(kb), s_par(kb)) ? 1 : 0;
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) { if (lane == 0) atomicExch(status, WKB_STATUS_ATTN_WAIT); ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int key0 = kb * KBLK + 64 * half;
      const int vis = min(max(ctx - key0, 0), 64);            // visible keys of this row inside this thread's half block
      uint32_t r[64];
      {
        uint32_t (&r0)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[0]);
        uint32_t (&r1)[32] = *reinterpret_cast<uint32_t (*)[32]>(&r[32]);
        tld32_nowait(lane_base + s_col(kb) + 64 * half, r0);
        tld32_nowait(lane_base + s_col(kb) + 64 * half + 32, r1);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      }
      const bool interior = __all_sync(0xffffffffu, vis == 64);
      if (!interior) {
#pragma unroll
        for (int e = 0; e < 64; ++e) r[e] = e < vis ? r[e] : 0xff800000u;      // -inf
      }
      float b4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < 64; e += 4) {
        b4[0] = fmaxf(b4[0], __uint_as_float(r[e])); b4[1] = fmaxf(b4[1], __uint_as_float(r[e + 1]));
        b4[2] = fmaxf(b4[2], __uint_as_float(r[e + 2])); b4[3] = fmaxf(b4[3], __uint_as_float(r[e + 3]));
      }
      const float bm = fmaxf(fmaxf(b4[0], b4[1]), fmaxf(b4[2], b4[3]));
      // the other half's maximum
      float other;
      if (!exchange(kb, bm, other)) { if (lane == 0) atomicExch(status, WKB_STATUS_ATTN_WAIT); ok = false; break; }
      const float m_new = fmaxf(m_run, fmaxf(bm, other));
      const float m_use = m_new == -INFINITY ? 0.0f : m_new;
      const float corr = ex2(m_run - m_use);                   // 0 for a row that had seen nothing yet
      // probabilities, rounded to bf16, into tensor memory as the A operand of P . V (a column = two keys); the
      // normaliser sums the rounded values
      uint32_t pk[32];
      float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int e = 0; e < 64; e += 2) {
        const uint32_t w = pack2(ex2(__uint_as_float(r[e]) - m_use), ex2(__uint_as_float(r[e + 1]) - m_use));   // ex2(-inf) = 0
        pk[e >> 1] = w;
        s4[(e >> 1) & 1] += u2f(w << 16);
        s4[2 + ((e >> 1) & 1)] += u2f(w & 0xffff0000u);
      }
      tst32(lane_base + p_col(kb) + 32 * half, pk);
      l_run = l_run * corr + ((s4[0] + s4[1]) + (s4[2] + s4[3]));
      m_run = m_new;
      // rescale this thread's half of the output accumulator when a row of the warp moved its maximum; the accumulator
      // holds the blocks before this one, whose last P . V must have retired (with single-buffered scores it retired
      // before this block's scores did)
      if (SM::DB && kb > 0) {
        int od = 1;
        if (lane == 0) od = mbar_wait(o_done, (kb - 1) & 1) ? 1 : 0;
        od = __shfl_sync(0xffffffffu, od, 0);
        if (!od) { if (lane == 0) atomicExch(status, WKB_STATUS_ATTN_WAIT); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      if (kb > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll 1
        for (int c0 = 0; c0 < HD / 2; c0 += 32) {
          uint32_t o[32];
          tld32(lane_base + SM::O_COL + half * (HD / 2) + c0, o);
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * corr);
          tst32(lane_base + SM::O_COL + half * (HD / 2) + c0, o);
        }
      }
      // the last block may hold key rows that were never written (a partly filled page): their probabilities are zero,
      // but 0 x NaN would still poison the product, so those V rows are zeroed in shared memory first
      if (kb + 1 == nkb && (kmax - kb * KBLK) < KBLK) {
        if constexpr (SM::DB) {
          int vok = 1;
          if (lane == 0) vok = mbar_wait(vfull(kb % STAGES), (kb / STAGES) & 1) ? 1 : 0;     // the V block must have landed
          vok = __shfl_sync(0xffffffffu, vok, 0);
          if (!vok) { if (lane == 0) atomicExch(status, WKB_STATUS_ATTN_WAIT); ok = false; break; }
        }
        const uint32_t vaddr = ring + (kb % STAGES) * SM::STAGE_BYTES + SM::OP_BYTES;
        const int first_bad = kmax - kb * KBLK;
        for (int idx = sm_tid; idx < (KBLK - first_bad) * NSUB * 8; idx += 256) {
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
    // ---- epilogue: normalise and write this thread's half of the row
    if (ok && nkb > 0) {
      int good = 1;
      if (lane == 0) good = mbar_wait(o_full, 0) ? 1 : 0;
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) { if (lane == 0) atomicExch(status, WKB_STATUS_ATTN_WAIT); ok = false; }
    }
    // the two halves of the normaliser meet the same way
    float l_other = 0.0f;
    if (ok && nkb > 0 && !exchange(nkb, l_run, l_other)) { if (lane == 0) atomicExch(status, WKB_STATUS_ATTN_WAIT); ok = false; }
    const float l_tot = l_run + l_other;
    if (ok && nkb > 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = l_tot != 0.0f ? 1.0f / l_tot : 0.0f;
      const i64 o = (i64)(row0 + a / G) * g.out_row_stride + ((i64)kvh * G + a % G) * HD + half * (HD / 2);
#pragma unroll 1
      for (int c0 = 0; c0 < HD / 2; c0 += 32) {
        uint32_t rr[32];
        tld32(lane_base + SM::O_COL + half * (HD / 2) + c0, rr);       // every lane of the warp takes part in the load
        if (ctx > 0) {
          if (out_dtype == 0) {
            float4* d = reinterpret_cast<float4*>(static_cast<float*>(out) + o + c0);
#pragma unroll
            for (int e = 0; e < 8; ++e)
              d[e] = make_float4(__uint_as_float(rr[4 * e]) * inv, __uint_as_float(rr[4 * e + 1]) * inv, __uint_as_float(rr[4 * e + 2]) * inv,
                                 __uint_as_float(rr[4 * e + 3]) * inv);
          } else {
            uint4* d = reinterpret_cast<uint4*>(static_cast<u16*>(out) + o + c0);
#pragma unroll
            for (int e = 0; e < 4; ++e)
              d[e] = make_uint4(pack2(__uint_as_float(rr[8 * e]) * inv, __uint_as_float(rr[8 * e + 1]) * inv),
                                pack2(__uint_as_float(rr[8 * e + 2]) * inv, __uint_as_float(rr[8 * e + 3]) * inv),
                                pack2(__uint_as_float(rr[8 * e + 4]) * inv, __uint_as_float(rr[8 * e + 5]) * inv),
                                pack2(__uint_as_float(rr[8 * e + 6]) * inv, __uint_as_float(rr[8 * e + 7]) * inv));
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

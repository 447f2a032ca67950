// Dense bf16 GEMM on the 5th-generation tensor cores: C[M,N] = epilogue(A[M,K] . B[N,K]^T).
//
// This is the B200 replacement for the reference's tensor-core GEMM families
// (crates/wukong_codegen_gpu/src/ptx_wmma.rs `wmma_nt_bf16*` with fused bias / activation /
// residual epilogues, and the sm_90a-only ptx_wgmma.rs which cannot load on sm_100): same operand
// convention (both operands K-major, "NT"), fp32 accumulate, same epilogue menu
// act(alpha-free A.B^T + bias[j]) (+ residual), act codes 0 identity / 1 relu / 2 gelu / 3 silu.
//
// Design (persistent CTAs, one per SM, looping over 128 x 128 output tiles -- 128 x 256 or 128 x 64 in two instantiations;
// 320 threads):
//   warp 0   one elected lane issues TMA loads (cp.async.bulk.tensor.2d, 128-byte swizzle, no
//            multicast) of a 128x64 A tile and a 128x64 B tile per stage into a 192 KB ring (6 stages of 32 KB,
//            4 of 48 KB, 8 of 24 KB), completion counted on an mbarrier per stage; with the weight-resident hint the
//            first ring of B tiles is requested before the wait for the preceding kernel of the stream;
//   warp 1   allocates the TMEM columns of two accumulator buffers (before that wait), and one elected lane issues
//            tcgen05.mma (cta_group::1, kind::f16, M=128 N=128 K=16) four times per stage straight
//            from shared memory descriptors; tcgen05.commit releases the stage back to the producer
//            and, after a tile's last K step, hands the accumulator buffer to the epilogue;
//   warps 2-9 read the fp32 accumulator out of TMEM with tcgen05.ld (32 lanes x 32 columns per
//            instruction; warp w owns lanes 32*(w%4).., the two warps of a lane quarter take alternate column chunks),
//            release the buffer as soon as it is in
//            registers (so the next tile's MMAs overlap this tile's epilogue), transpose through
//            shared memory and store coalesced rows with bias / activation / residual applied, or
//            keep a per-row arg-max candidate instead of storing (greedy LM head), or write K / V rows into their
//            pages (fused QKV projection), or leave the partial tile in shared memory for the in-cluster K-slice sum.
// Every mbarrier wait is bounded: on expiry the kernel records a code in `status`, stops issuing,
// waits (bounded) for the copies it started, frees its TMEM and returns.
// Ragged M / N / K are handled by TMA zero fill and masked stores; K % 8 == 0 is required (the
// row pitch of a tensor map must be a multiple of 16 bytes).
// Accumulation order is the tensor core's own, so results agree with the order-contract GEMM to
// fp32 rounding (rtol 2e-2 is the stated bf16 bar; measured error is ~1e-6 relative to sum|a||b|).
#include "common.cuh"
#include "wkb_device.h"
#include "tc_common.cuh"

namespace wkb {

constexpr int BM = 128, BN = 128, STAGES = 6;
constexpr int BK_BYTES = 128;   // one 128-byte swizzle row of K per stage: 64 bf16 or 128 e4m3 elements
constexpr int UMMA_K_BYTES = 32;  // K extent of one tcgen05.mma: 16 bf16 or 32 e4m3 elements
constexpr int TILE_A_BYTES = BM * BK_BYTES, TILE_B_BYTES = BN * BK_BYTES;
constexpr int STAGE_BYTES = TILE_A_BYTES + TILE_B_BYTES;
constexpr int GEMM_THREADS = 320;                 // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue (two per TMEM lane quarter)
constexpr int EPI_STAGE_BYTES = 8 * 32 * 33 * 4;  // one 32 x 33 fp32 transpose pad per epilogue warp
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int BN_WIDE = 256;
constexpr int SMEM_BYTES_WIDE = 4 * (TILE_A_BYTES + BN_WIDE * BK_BYTES) + EPI_STAGE_BYTES + 1024 + 256;
// Instruction descriptor, kind::f16: D = f32 (1 << 4), A = B = bf16 (1 << 7, 1 << 10), both K-major,
// N >> 3 in bits 17-22, M >> 4 in bits 24-28.
// (kind::f8f6f4 with A = B = E4M3 uses format code 0 for both operands.)
__host__ __device__ constexpr uint32_t make_idesc(int bn, bool f8) {
  return (1u << 4) | (f8 ? 0u : ((1u << 7) | (1u << 10))) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

struct GemmEpi {
  const float* bias;       // [N] or null
  const float* residual;   // [M, ldr] f32 or null (added after the activation)
  i64 ldr;
  int act;                 // 0 identity, 1 relu, 2 gelu, 3 silu
  int out_bf16;            // 0: f32 C, 1: bf16 C
  int* arg_idx;            // arg-max mode: per-(row, column tile) winning column (values go to C)
  int ksplit;              // > 1: work item = (tile, K slice); slice s writes its raw fp32 partial at c + s * slice_stride
  i64 slice_stride;        // elements between the partial outputs of consecutive K slices
  // KVAPPEND instantiation (fused QKV projection of a decode step): columns [kv_col0, kv_col0 + 2 * kv_heads * kv_hd)
  // are the new K then V rows; they are rounded to bf16 straight into their pages (the paged_kv_append_kernel
  // addressing: bf16 [page][kv_head][token][dim]) instead of being stored to C.  Rows with row_pos < 0 or past the
  // block-table row write nothing (the latter is reported in the status word).
  u16* kcache;
  u16* vcache;
  const uint32_t* block_table;
  const int* row_slot;
  const int* row_pos;
  int kv_col0, kv_heads, kv_hd, page_tokens, mbps;
  // B (the weights) is not written by any kernel still in flight on the stream: the producer may request its first B
  // tiles before it waits for the preceding kernel (wkb_gemm_b_static)
  int b_static;
};

// Set by wkb_gemm_b_static on the calling thread; copied into every launch of gemm_bf16_tc_kernel from that thread.
static thread_local int g_b_static = 0;

// GELU for bf16 output: x * sigmoid(2u), u = sqrt(2/pi)(x + 0.044715 x^3), with the hardware exp2 and
// reciprocal.  Relative error ~1e-6, three orders below the bf16 rounding that follows; the exact
// sequence (gelu1) stays in use wherever fp32 values are returned.
__device__ __forceinline__ float gelu_fast(float x) {
  float u = 0.7978846f * fmaf(0.044715f * x * x, x, x);
  float e = exp2f(-2.8853900817779268f * u);  // exp(-2u)
  return __fdividef(x, 1.0f + e);
}

template <int ACT, bool OUT_BF16>
__device__ __forceinline__ float epi_act(float y) {
  if (ACT == 2 && OUT_BF16) return gelu_fast(y);
  return act_apply(ACT, y);
}

__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
// this CTA's shared-memory address -> the same offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_shared_f4(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Persistent kernel: CTA b works on tiles b, b + gridDim.x, ...; tile t is (m_tile = t % tiles_m,
// n_tile = t / tiles_m), so CTAs running side by side share one B (weight) tile through L2.
// ACT / OUT_BF16 / ARGMAX are compile-time so an identity epilogue carries no transcendental code.
// CLUSTERK instantiation (x += A.B^T + bias for a decode-sized product whose K is cut into slices): the CTAs of a thread-block
// cluster are the K slices of one tile (cluster rank = slice; the grid is exactly tiles x slices).  Each leaves its fp32
// partial tile in its own shared memory (the operand ring is free by then), the cluster meets at a barrier, and CTA r adds
// rows [r * 128 / slices, ...) of all the partials in slice order -- read through distributed shared memory -- plus the bias
// into x.  The partials never travel through L2, and the row kernel that follows reads x alone.
template <int ACT, bool OUT_BF16, bool ARGMAX, bool F8, bool WIDE, bool KVAPPEND = false, bool NARROW = false, bool CLUSTERK = false>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, void* c,
                    i64 ldc, int M, int N, int K, GemmEpi epi, int* status) {
  // tile shape of this instantiation: 128 x 128 with a 6-stage ring, 128 x 256 with 4 stages, or 128 x 64 with 8 (a problem with
  // fewer 128-wide tiles than half the SMs then still puts a CTA on most of them)
  static_assert(!(WIDE && NARROW), "one tile shape per instantiation");
  constexpr int BN = NARROW ? 64 : WIDE ? 256 : 128;
  constexpr int STAGES = NARROW ? 8 : WIDE ? 4 : 6;   // 192 KB of operand ring whatever the tile: the loop of a decode-sized GEMM runs at
                                                      // one stage per (TMA latency / stages)
  constexpr int TILE_B_BYTES = BN * BK_BYTES, STAGE_BYTES = TILE_A_BYTES + TILE_B_BYTES;
  constexpr int NUM_BARS = 2 * STAGES + 4;
  constexpr uint32_t TMEM_COLS = 2 * BN;       // two accumulator buffers
  // epilogue warps: two per TMEM lane quarter, taking alternate 32-column chunks (the arg-max epilogue leaves one candidate
  // per row, tile and warp of the pair)
  constexpr int EPI_WARPS = 8, CHUNK_STEP = 32 * (EPI_WARPS / 4);
  constexpr uint32_t IDESC_ = make_idesc(BN, F8);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  // layout: STAGES x (A tile, B tile) | epilogue staging 4 x 32 x 33 floats | barriers | tmem slot
  float* stage_all = reinterpret_cast<float*>(gen_base + STAGES * STAGE_BYTES);
  const uint32_t bars = base + STAGES * STAGE_BYTES + EPI_STAGE_BYTES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + STAGES * STAGE_BYTES + EPI_STAGE_BYTES + 8 * NUM_BARS);
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bars + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
  const int ksplit = epi.ksplit > 1 ? epi.ksplit : 1;
  const int num_tiles = tiles_m * tiles_n * ksplit;   // work items: the K slice is the fastest index
  constexpr int BK = F8 ? BK_BYTES : BK_BYTES / 2;  // elements of K per stage
  const int kiters_all = (K + BK - 1) / BK;
  const int kper = (kiters_all + ksplit - 1) / ksplit;   // the host picks ksplit so that no slice is empty

  int pre = 0;   // producer lane: stages whose B tile was requested before the dependency wait
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), EPI_WARPS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
    if (epi.b_static) {
      // the first ring of B tiles is on its way while the preceding kernel of the stream is still running: each barrier is
      // armed for the whole stage, the A tile follows after the wait below
      for (int w = blockIdx.x; w < num_tiles && pre < STAGES; w += gridDim.x) {
        const int t = w / ksplit, k0 = (w % ksplit) * kper, kiters = min(kper, kiters_all - k0);
        const int n0 = (t / tiles_m) * BN;
        for (int kk = 0; kk < kiters && pre < STAGES; ++kk, ++pre) {
          mbar_expect_tx(full_bar(pre), STAGE_BYTES);
          tma_load_2d(base + pre * STAGE_BYTES + TILE_A_BYTES, &map_b, full_bar(pre), (k0 + kk) * BK, n0);
        }
      }
    }
  }
  // Tensor memory is claimed before the wait for the preceding kernel as well: an allocation that meets a still-resident
  // CTA of that kernel simply blocks until its columns are freed (no kernel waits on its successor), and everything up to
  // here touches only this CTA's shared memory and (b_static) the weights.  A is read after the wait.
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  pdl_trigger();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int it = 0, issued_from = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_tiles && ok; w += gridDim.x) {
        const int t = w / ksplit, k0 = (w % ksplit) * kper, kiters = min(kper, kiters_all - k0);
        const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
        for (int kk = 0; kk < kiters; ++kk, ++it) {
          const int s = it % STAGES;
          const uint32_t sa = base + s * STAGE_BYTES, sb = sa + TILE_A_BYTES;
          if (it >= pre) {
            if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1)) { atomicExch(status, 1); ok = false; break; }
            mbar_expect_tx(full_bar(s), STAGE_BYTES);
            tma_load_2d(sb, &map_b, full_bar(s), (k0 + kk) * BK, n0);
          }
          tma_load_2d(sa, &map_a, full_bar(s), (k0 + kk) * BK, m0);
        }
      }
      if (!ok) {
        // wait (bounded) for the copies already started before the CTA may exit
        issued_from = it > STAGES ? it - STAGES : 0;
        for (int j = issued_from; j < it; ++j) mbar_wait(full_bar(j % STAGES), (j / STAGES) & 1);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int it = 0, local = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_tiles && ok; w += gridDim.x, ++local) {
        const int kiters = min(kper, kiters_all - (w % ksplit) * kper);
        const int buf = local & 1;
        // the epilogue must have drained this accumulator buffer (two tiles ago)
        if (!mbar_wait(tempty_bar(buf), ((local >> 1) & 1) ^ 1)) { atomicExch(status, 4); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN);
        for (int kk = 0; kk < kiters; ++kk, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(full_bar(s), (it / STAGES) & 1)) { atomicExch(status, 2); ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = base + s * STAGE_BYTES, sb = sa + TILE_A_BYTES;
#pragma unroll
          for (int k = 0; k < BK_BYTES / UMMA_K_BYTES; ++k) {
            const uint64_t ad = make_sdesc(sa + k * UMMA_K_BYTES), bd = make_sdesc(sb + k * UMMA_K_BYTES);
            if (F8) umma_e4m3(tmem_d, ad, bd, IDESC_, (kk > 0 || k > 0) ? 1u : 0u);
            else umma_bf16(tmem_d, ad, bd, IDESC_, (kk > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(tfull_bar(buf));
      }
    }
  } else if (warp < 2 + EPI_WARPS) {
    // ---------------- epilogue warps: TMEM lane quarter (warp % 4), column chunks c0 = 32 * half, + CHUNK_STEP, ... ----------------
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    float* stage = stage_all + (warp - 2) * (32 * 33);
    (void)stage;
    int local = 0;
    bool ok = true;
    void* const c_all = c;
    for (int w = blockIdx.x; w < num_tiles && ok; w += gridDim.x, ++local) {
      const int t = w / ksplit;
      // a K slice's partial goes to its own plane of the split workspace (fp32, identity epilogue)
      c = reinterpret_cast<float*>(c_all) + (i64)(w % ksplit) * epi.slice_stride;
      const int buf = local & 1;
      const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
      const int row = m0 + quarter * 32 + lane;
      // KVAPPEND: where this thread's row (the TMEM lane it reads) lands in the cache: element offset of its token row for
      // KV head 0 (-1: the row writes nothing).  Looked up while the tile is still being multiplied.
      i64 kv_dst = -1;
      (void)kv_dst;
      if (KVAPPEND && n0 + BN > epi.kv_col0 && row < M) {
        const int pos = epi.row_pos[row];
        if (pos >= 0) {
          const int lp = pos / epi.page_tokens;
          if (lp < epi.mbps) {
            const uint32_t page = epi.block_table[(i64)epi.row_slot[row] * epi.mbps + lp];
            kv_dst = ((i64)page * epi.kv_heads * epi.page_tokens + (pos % epi.page_tokens)) * epi.kv_hd;
          } else {
            atomicExch(status, WKB_STATUS_KV_POS_RANGE);
          }
        }
      }
      int good = 1;
      if (lane == 0) good = mbar_wait(tfull_bar(buf), (local >> 1) & 1) ? 1 : 0;
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) { if (lane == 0) atomicExch(status, 3); ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      float best_v = -INFINITY;
      int best_i = -1;
      bool pinned = false;
      (void)best_v; (void)best_i; (void)pinned;
#pragma unroll 1
      for (int c0 = 32 * half; c0 < BN; c0 += CHUNK_STEP) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c0);
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
        if (c0 + CHUNK_STEP >= BN) {
          // this warp's last chunk of the accumulator buffer is in registers: its share is handed back to the MMA warp
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty_bar(buf));
        }
        if (CLUSTERK) {
          // this thread's row of the partial tile, 32 columns: [row][BN + 4] floats at the base of the (idle) operand ring
          const uint32_t dst = base + (uint32_t)(((quarter * 32 + lane) * (BN + 4) + c0) * 4);
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            st_shared_f4(dst + e * 4, __uint_as_float(r[e]), __uint_as_float(r[e + 1]), __uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
        } else if (KVAPPEND && n0 + c0 >= epi.kv_col0) {
          // a K or V chunk (kv_col0 and the head size are multiples of 32, so the 32 columns are consecutive dims of one
          // head): the thread holds them for its own row and writes them as 64 contiguous bytes of that token's cache row --
          // no transpose, no exchange of destinations between lanes
          if (kv_dst >= 0 && n0 + c0 + 32 <= N) {
            const int kc = n0 + c0 - epi.kv_col0, kv_dim = epi.kv_heads * epi.kv_hd;
            u16* cache = kc < kv_dim ? epi.kcache : epi.vcache;
            const int cc = kc < kv_dim ? kc : kc - kv_dim;
            uint4* dst = reinterpret_cast<uint4*>(cache + kv_dst + (i64)(cc / epi.kv_hd) * epi.page_tokens * epi.kv_hd + (cc % epi.kv_hd));
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float b8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
              if (epi.bias) {
                const float4 b0 = *reinterpret_cast<const float4*>(epi.bias + n0 + c0 + 8 * v), b1 = *reinterpret_cast<const float4*>(epi.bias + n0 + c0 + 8 * v + 4);
                b8[0] = b0.x; b8[1] = b0.y; b8[2] = b0.z; b8[3] = b0.w; b8[4] = b1.x; b8[5] = b1.y; b8[6] = b1.z; b8[7] = b1.w;
              }
              uint32_t w4[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                w4[e] = (uint32_t)f32_to_bf16_bits(__uint_as_float(r[8 * v + 2 * e]) + b8[2 * e]) |
                        ((uint32_t)f32_to_bf16_bits(__uint_as_float(r[8 * v + 2 * e + 1]) + b8[2 * e + 1]) << 16);
              dst[v] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            }
          }
        } else if (ARGMAX) {
          // thread = row: ascending scan of its 32 columns keeps the lowest index on a tie; NaNs never
          // win, except that a NaN in global column 0 pins the row to 0 (the arg-max rule of the ABI)
          if (n0 + c0 + 32 <= N && n0 + c0 > 0 && !epi.bias) {
            // interior chunk: branch-free scan (a NaN fails `y > best_v`; column 0 is not in this chunk)
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const float y = __uint_as_float(r[e]);
              const bool take = !pinned && (y > best_v || (best_i < 0 && y == y));
              best_v = take ? y : best_v;
              best_i = take ? n0 + c0 + e : best_i;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int col = n0 + c0 + e;
              float y = __uint_as_float(r[e]);
              if (col < N) {
                if (epi.bias) y += epi.bias[col];
                if (col == 0 && y != y) { best_v = INFINITY; best_i = 0; pinned = true; }
                if (!pinned && y == y && (best_i < 0 || y > best_v)) { best_v = y; best_i = col; }
              }
            }
          }
        } else {
          // transpose through shared memory so that a lane owns a column and every global access is
          // one coalesced row segment; the residual rows are fetched first so their latency overlaps
          const int col = n0 + c0 + lane;
          const bool col_ok = col < N;
          const int row0 = m0 + quarter * 32;
          const int nrows = min(32, M - row0);  // rows of this warp inside the matrix (may be <= 0)
          const bool full = nrows == 32;        // warp-uniform: the straight-line path has no per-row branch
          float res[32];
          if (epi.residual && full && col_ok) {
            const float* rp = epi.residual + (i64)row0 * epi.ldr + col;
#pragma unroll
            for (int rr = 0; rr < 32; ++rr) res[rr] = rp[(i64)rr * epi.ldr];
          }
#pragma unroll
          for (int e = 0; e < 32; ++e) stage[lane * 33 + e] = __uint_as_float(r[e]);
          __syncwarp();
          const float bias_v = (col_ok && epi.bias) ? epi.bias[col] : 0.0f;
          if (col_ok) {
            if (full) {
              float vals[32];
#pragma unroll
              for (int rr = 0; rr < 32; ++rr) vals[rr] = epi_act<ACT, OUT_BF16>(stage[rr * 33 + lane] + bias_v);
              if (epi.residual) {
#pragma unroll
                for (int rr = 0; rr < 32; ++rr) vals[rr] += res[rr];
              }
              if (OUT_BF16) {
                u16* cp = reinterpret_cast<u16*>(c) + (i64)row0 * ldc + col;
#pragma unroll
                for (int rr = 0; rr < 32; ++rr) cp[(i64)rr * ldc] = f32_to_bf16_bits(vals[rr]);
              } else {
                float* cp = reinterpret_cast<float*>(c) + (i64)row0 * ldc + col;
#pragma unroll
                for (int rr = 0; rr < 32; ++rr) cp[(i64)rr * ldc] = vals[rr];
              }
            } else {
#pragma unroll 1
              for (int rr = 0; rr < nrows; ++rr) {
                const i64 grow = row0 + rr;
                float y = epi_act<ACT, OUT_BF16>(stage[rr * 33 + lane] + bias_v);
                if (epi.residual) y += epi.residual[grow * epi.ldr + col];
                if (OUT_BF16) reinterpret_cast<u16*>(c)[grow * ldc + col] = f32_to_bf16_bits(y);
                else reinterpret_cast<float*>(c)[grow * ldc + col] = y;
              }
            }
          }
          __syncwarp();
        }
      }
      if (ARGMAX && row < M) {
        // partial result of this warp's chunks of the column tile: [row][tile][half] (value, index); index -1 = no candidate
        const i64 slot = ((i64)row * tiles_n + (t / tiles_m)) * 2 + half;
        reinterpret_cast<float*>(c)[slot] = best_v;
        epi.arg_idx[slot] = best_i;
      }
    }
  }
  if (CLUSTERK) {
    cluster_sync_all();                              // every slice's partial tile is in its CTA's shared memory
    if (warp >= 2) {
      const int t = blockIdx.x / ksplit;
      const int m0 = (t % tiles_m) * BM, n0 = (t / tiles_m) * BN;
      const int rows_per = BM / ksplit, row_first = (int)cluster_rank() * rows_per;
      float* xg = reinterpret_cast<float*>(c);
      for (int idx = threadIdx.x - 64; idx < rows_per * (BN / 4); idx += GEMM_THREADS - 64) {
        const int rl = row_first + idx / (BN / 4), c4 = idx % (BN / 4);
        const int grow = m0 + rl, gcol = n0 + 4 * c4;
        if (grow < M && gcol < N) {                  // N is a multiple of 4: the four columns are inside together
          const uint32_t mine = base + (uint32_t)((rl * (BN + 4) + 4 * c4) * 4);
          // every slice's piece is requested before the first add; the adds run in slice order
          float4 p[8];
#pragma unroll
          for (int sl = 0; sl < 8; ++sl)
            if (sl < ksplit) p[sl] = ld_cluster_f4(map_to_cta(mine, (uint32_t)sl));
          float4 d = p[0];
#pragma unroll
          for (int sl = 1; sl < 8; ++sl)
            if (sl < ksplit) { d.x += p[sl].x; d.y += p[sl].y; d.z += p[sl].z; d.w += p[sl].w; }
          if (epi.bias) {
            const float4 bb = *reinterpret_cast<const float4*>(epi.bias + gcol);
            d.x += bb.x; d.y += bb.y; d.z += bb.z; d.w += bb.w;
          }
          float4* xp = reinterpret_cast<float4*>(xg + (i64)grow * ldc + gcol);
          float4 xv = *xp;
          xv.x += d.x; xv.y += d.y; xv.z += d.z; xv.w += d.w;
          *xp = xv;
        }
      }
    }
    cluster_sync_all();                              // nobody leaves while a peer may still read its tile
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}


// ---- CTA-pair kernel: one 256 x 256 tile per pair of CTAs (tcgen05.mma.cta_group::2) ---------------------------------
// A single CTA's 128 x 256 tile moves 96 KB through shared memory per 64-K step (48 KB written by TMA, 48 KB read by the
// MMA) for 4 MMAs of 72 ns: more than the shared memory delivers, which held the kernel above at 0.78 of the cuBLAS burst.
// Here the two CTAs of a cluster share a tile: each loads its own 128 rows of A and its own 128-column half of B (ordinary
// per-CTA TMA loads of this GPU's memory, no multicast), and one thread of the even CTA issues M = 256 MMAs that run on
// both SMs, each SM reading its A rows and both halves of B: 64 KB per CTA per step.
//   * full barriers live in the even CTA: it arms them for the bytes of both CTAs, and the odd CTA's loads complete on
//     them through their cluster address;
//   * a stage is released (and a finished accumulator announced) by two tcgen05.commit, one to each CTA's barrier;
//   * the odd CTA's epilogue warps hand an accumulator buffer back by a remote arrive on the even CTA's barrier;
//   * tensor memory is allocated and freed by both CTAs together (cta_group::2); the CTAs meet at a cluster barrier after
//     the barriers are initialised and before either may exit.
// Every mbarrier wait is bounded like in the kernel above.
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_TILE_BYTES = 128 * BK_BYTES;              // a 128-row operand tile of one stage
constexpr int PAIR_STAGE_BYTES = 2 * PAIR_TILE_BYTES;        // A tile + this CTA's half of B
constexpr int PAIR_THREADS = 192;                            // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue
constexpr int PAIR_EPI_STAGE_BYTES = 4 * 32 * 33 * 4;        // one 32 x 33 fp32 transpose pad per epilogue warp
constexpr int SMEM_BYTES_PAIR = PAIR_STAGES * PAIR_STAGE_BYTES + PAIR_EPI_STAGE_BYTES + 1024 + 256;
constexpr uint32_t IDESC_PAIR = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);

// TMA load into this CTA's shared memory whose bytes are counted on a barrier given by its cluster address
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster) : "memory");
}

template <int ACT, bool OUT_BF16>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, void* c, i64 ldc, int M, int N,
                      int K, GemmEpi epi, int* status) {
  constexpr int STAGES = PAIR_STAGES, BN2 = 256, BM2 = 256;
  constexpr int NUM_BARS = 2 * STAGES + 4;
  constexpr uint32_t TMEM_COLS = 2 * BN2;       // two accumulator buffers of 256 columns (this CTA's 128 rows of the tile)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  float* stage_all = reinterpret_cast<float*>(gen_base + STAGES * PAIR_STAGE_BYTES);
  const uint32_t bars = base + STAGES * PAIR_STAGE_BYTES + PAIR_EPI_STAGE_BYTES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + STAGES * PAIR_STAGE_BYTES + PAIR_EPI_STAGE_BYTES + 8 * NUM_BARS);
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bars + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bars + 8u * (2 * STAGES + 2 + b); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();                 // 0: the CTA that issues the MMAs
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int tiles_m = (M + BM2 - 1) / BM2, tiles_n = (N + BN2 - 1) / BN2;
  const int num_tiles = tiles_m * tiles_n;
  constexpr int BK = BK_BYTES / 2;
  const int kiters = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 8); }   // 4 epilogue warps of each CTA
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
  }
  pdl_wait();
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                                    // both CTAs' barriers exist before anything arrives on them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs): own A rows, own half of B; bytes counted on the even CTA's barrier ----------------
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += npairs) {
        const int m0 = (t % tiles_m) * BM2 + (int)rank * 128, n0 = (t / tiles_m) * BN2 + (int)rank * 128;
        for (int kk = 0; kk < kiters; ++kk, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1)) { atomicExch(status, 1); ok = false; break; }
          if (rank == 0) mbar_expect_tx(full_bar(s), 2 * PAIR_STAGE_BYTES);
          const uint32_t sa = base + s * PAIR_STAGE_BYTES, sb = sa + PAIR_TILE_BYTES;
          const uint32_t fb = map_to_cta(full_bar(s), 0);
          tma_load_2d_pair(sa, &map_a, fb, kk * BK, m0);
          tma_load_2d_pair(sb, &map_b, fb, kk * BK, n0);
        }
      }
      // (a failed wait leaves this CTA's copies to the other roles' own bounded waits: the pair ends through the cluster
      // barrier below only after every role of both CTAs has stopped)
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (lane == 0 && rank == 0) {
      int it = 0, local = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += npairs, ++local) {
        const int buf = local & 1;
        if (!mbar_wait(tempty_bar(buf), ((local >> 1) & 1) ^ 1)) { atomicExch(status, 4); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * BN2);
        for (int kk = 0; kk < kiters; ++kk, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(full_bar(s), (it / STAGES) & 1)) { atomicExch(status, 2); ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t sa = base + s * PAIR_STAGE_BYTES, sb = sa + PAIR_TILE_BYTES;
#pragma unroll
          for (int k = 0; k < BK_BYTES / UMMA_K_BYTES; ++k)
            umma_bf16_pair(tmem_d, make_sdesc(sa + k * UMMA_K_BYTES), make_sdesc(sb + k * UMMA_K_BYTES), IDESC_PAIR, (kk > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(empty_bar(s));                       // frees the stage in this CTA ...
          umma_commit_pair(map_to_cta(empty_bar(s), 1));        // ... and in the other one
        }
        if (ok) {
          umma_commit_pair(tfull_bar(buf));
          umma_commit_pair(map_to_cta(tfull_bar(buf), 1));
        }
      }
    }
  } else {
    // ---------------- epilogue warps 2..5 of both CTAs: this CTA's 128 rows of the tile ----------------
    const int quarter = warp & 3;
    float* stage = stage_all + (warp - 2) * (32 * 33);
    int local = 0;
    bool ok = true;
    const uint32_t tempty0[2] = {map_to_cta(tempty_bar(0), 0), map_to_cta(tempty_bar(1), 0)};
    for (int t = pair; t < num_tiles && ok; t += npairs, ++local) {
      const int buf = local & 1;
      const int m0 = (t % tiles_m) * BM2 + (int)rank * 128, n0 = (t / tiles_m) * BN2;
      int good = 1;
      if (lane == 0) good = mbar_wait(tfull_bar(buf), (local >> 1) & 1) ? 1 : 0;
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) { if (lane == 0) atomicExch(status, 3); ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c0 = 0; c0 < BN2; c0 += 32) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN2 + c0);
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
        if (c0 + 32 == BN2) {
          // this CTA's part of the accumulator buffer is in registers: hand it back to the MMA warp of the even CTA
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(tempty0[buf]);
        }
        // transpose through shared memory so that a lane owns a column and every global access is one coalesced row segment
        const int col = n0 + c0 + lane;
        const bool col_ok = col < N;
        const int row0 = m0 + quarter * 32;
        const int nrows = min(32, M - row0);   // rows of this warp inside the matrix (may be <= 0)
        const bool full = nrows == 32;
        float res[32];
        if (epi.residual && full && col_ok) {
          const float* rp = epi.residual + (i64)row0 * epi.ldr + col;
#pragma unroll
          for (int rr = 0; rr < 32; ++rr) res[rr] = rp[(i64)rr * epi.ldr];
        }
#pragma unroll
        for (int e = 0; e < 32; ++e) stage[lane * 33 + e] = __uint_as_float(r[e]);
        __syncwarp();
        const float bias_v = (col_ok && epi.bias) ? epi.bias[col] : 0.0f;
        if (col_ok) {
          if (full) {
            float vals[32];
#pragma unroll
            for (int rr = 0; rr < 32; ++rr) vals[rr] = epi_act<ACT, OUT_BF16>(stage[rr * 33 + lane] + bias_v);
            if (epi.residual) {
#pragma unroll
              for (int rr = 0; rr < 32; ++rr) vals[rr] += res[rr];
            }
            if (OUT_BF16) {
              u16* cp = reinterpret_cast<u16*>(c) + (i64)row0 * ldc + col;
#pragma unroll
              for (int rr = 0; rr < 32; ++rr) cp[(i64)rr * ldc] = f32_to_bf16_bits(vals[rr]);
            } else {
              float* cp = reinterpret_cast<float*>(c) + (i64)row0 * ldc + col;
#pragma unroll
              for (int rr = 0; rr < 32; ++rr) cp[(i64)rr * ldc] = vals[rr];
            }
          } else {
#pragma unroll 1
            for (int rr = 0; rr < nrows; ++rr) {
              const i64 grow = row0 + rr;
              float y = epi_act<ACT, OUT_BF16>(stage[rr * 33 + lane] + bias_v);
              if (epi.residual) y += epi.residual[grow * epi.ldr + col];
              if (OUT_BF16) reinterpret_cast<u16*>(c)[grow * ldc + col] = f32_to_bf16_bits(y);
              else reinterpret_cast<float*>(c)[grow * ldc + col] = y;
            }
          }
        }
        __syncwarp();
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();          // neither CTA leaves while the other may still read its shared memory or signal its barriers
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// 2-D tensor [rows, k] of bf16 (or 1-byte e4m3) with row pitch ld elements; box = [128 bytes of K,
// box_rows]; 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* ptr, i64 rows, i64 k, i64 ld, int box_rows, bool f8 = false) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * (f8 ? 1 : 2)};
  cuuint32_t box[2] = {(cuuint32_t)(f8 ? BK_BYTES : BK_BYTES / 2), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, f8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

// One warp per row folds the per-tile candidates: greater value wins, equal values keep the lower
// column, a pinned row (value +inf from a NaN at column 0, index 0) wins outright by its index rule.
__global__ void __launch_bounds__(128) argmax_tiles_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int tiles,
                                                           int* __restrict__ out, int rows) {
  pdl_wait();
  pdl_trigger();
  int lane = threadIdx.x & 31;
  int row = (int)(((i64)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  if (row >= rows) return;
  float bv = -INFINITY;
  int bi = -1;
  for (int t = lane; t < tiles; t += 32) {
    float v = pv[(i64)row * tiles + t];
    int i = pi[(i64)row * tiles + t];
    if (i >= 0 && (bi < 0 || v > bv || (v == bv && i < bi))) { bv = v; bi = i; }
  }
#pragma unroll
  for (int ofs = 16; ofs > 0; ofs >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, bv, ofs);
    int oi = __shfl_xor_sync(0xffffffffu, bi, ofs);
    bool take = oi >= 0 && (bi < 0 || ov > bv || (ov == bv && oi < bi));
    if (take) { bv = ov; bi = oi; }
  }
  if (lane == 0) out[row] = bi < 0 ? 0 : bi;
}

static i64 sm_count() {
  static int counts[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return WKB_SM_COUNT;
  if (!counts[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = WKB_SM_COUNT;
    counts[dev] = n;
  }
  return counts[dev];
}

int* gemm_status_word() {
  // one device word per device for the bounded-wait status; allocated at first use
  static int* words[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!words[dev]) {
    int* p = nullptr;
    if (cudaMalloc((void**)&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    words[dev] = p;
  }
  return words[dev];
}

// Split-K second pass of the dense GEMM: c = act(sum over slices (slice order) + bias) (+ residual), f32 or bf16.
__global__ void __launch_bounds__(256) gemm_splitk_finish_kernel(const float* __restrict__ ws, int ksplit, i64 slice_stride, int M, int N,
                                                                 void* __restrict__ c, i64 ldc, int c_bf16, const float* __restrict__ bias,
                                                                 int act, const float* __restrict__ residual, i64 ldr) {
  pdl_wait();
  pdl_trigger();
  const i64 quads = (i64)(N >> 2), total = (i64)M * quads;
  for (i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    const int m = (int)(idx / quads), n0 = (int)(idx % quads) << 2;
    const float4* src = reinterpret_cast<const float4*>(ws + (i64)m * N + n0);
    float4 v = __ldcg(src);
    for (int s = 1; s < ksplit; ++s) {
      const float4 p = __ldcg(reinterpret_cast<const float4*>(ws + (i64)s * slice_stride + (i64)m * N + n0));
      v.x += p.x; v.y += p.y; v.z += p.z; v.w += p.w;
    }
    float y[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float t = y[j] + (bias ? bias[n0 + j] : 0.0f);
      t = (act == 2 && c_bf16) ? gelu_fast(t) : act_apply(act, t);
      if (residual) t += residual[(i64)m * ldr + n0 + j];
      y[j] = t;
    }
    if (c_bf16) {
      uint2 o;
      o.x = (uint32_t)f32_to_bf16_bits(y[0]) | ((uint32_t)f32_to_bf16_bits(y[1]) << 16);
      o.y = (uint32_t)f32_to_bf16_bits(y[2]) | ((uint32_t)f32_to_bf16_bits(y[3]) << 16);
      *reinterpret_cast<uint2*>(reinterpret_cast<u16*>(c) + (i64)m * ldc + n0) = o;
    } else {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(c) + (i64)m * ldc + n0) = make_float4(y[0], y[1], y[2], y[3]);
    }
  }
}

// Default split-K workspace, one per device: allocated by wkb_gemm_init (or by the first eligible call that is not
// inside a stream capture).  Whether a shape splits is a pure function of (m, n, k); a split shape that finds no
// workspace is an error, never a silent change of algorithm (the summation order, hence the output bits, would
// otherwise depend on the call history).
constexpr size_t SPLITK_WS_BYTES = (size_t)32 << 20;
static float* splitk_workspace(cudaStream_t st, bool may_allocate) {
  static float* ws[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ws[dev] && may_allocate) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (st && (cudaStreamIsCapturing(st, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone)) return nullptr;
    float* p = nullptr;
    if (cudaMalloc((void**)&p, SPLITK_WS_BYTES) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    ws[dev] = p;
  }
  return ws[dev];
}

// K slices of a shape (1: no split).  Few 128 x 128 tiles and a long K (the decode MLP's down projection: 24 tiles,
// K = 3072): cut K so that most SMs pull operands.
static i64 splitk_slices(i64 m, i64 n, i64 k) {
  const i64 tiles = ((n + BN - 1) / BN) * ((m + BM - 1) / BM);
  const i64 tiles_wide = ((n + BN_WIDE - 1) / BN_WIDE) * ((m + BM - 1) / BM);
  const i64 kiters = (k + 63) / 64;
  if (tiles_wide >= 2 * sm_count() || tiles * 2 > sm_count() || kiters < 32 || n % 4 != 0) return 1;
  i64 ks = sm_count() / tiles;
  if (ks > 4) ks = 4;
  if (ks > kiters / 8) ks = kiters / 8;
  if (ks < 1) ks = 1;
  const i64 kper = (kiters + ks - 1) / ks;
  ks = (kiters + kper - 1) / kper;
  if (ks > 1 && (size_t)(ks * m * n * 4) > SPLITK_WS_BYTES) return 1;
  return ks;
}

i64 gemm_sm_count() { return sm_count(); }

}  // namespace wkb

using namespace wkb;

extern "C" {

// Shared body of the two bf16 entries.  `ws` holds the fp32 K-slice partials of a split shape (ws_bytes of it).
static int gemm_bf16_nt_impl(const void* a, i64 lda, const void* b, i64 ldb, void* c, i64 ldc, int c_bf16, i64 m, i64 n, i64 k,
                             const float* bias, i64 act, const float* residual, i64 ldr, float* ws, i64 ws_bytes, cudaStream_t st) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  if (k % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)a) | ((uintptr_t)b)) & 15) return (int)cudaErrorMisalignedAddress;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, a, m, k, lda, BM);
  if (rc) return rc;
  rc = make_map(&mb, b, n, k, ldb, BN);
  if (rc) return rc;
  int* status = gemm_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  if (act < 0 || act > 3) return (int)cudaErrorInvalidValue;
  typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, void*, i64, int, int, int, GemmEpi, int*);
  static const KernelFn table[4][2] = {
      {gemm_bf16_tc_kernel<0, false, false, false, false>, gemm_bf16_tc_kernel<0, true, false, false, false>},
      {gemm_bf16_tc_kernel<1, false, false, false, false>, gemm_bf16_tc_kernel<1, true, false, false, false>},
      {gemm_bf16_tc_kernel<2, false, false, false, false>, gemm_bf16_tc_kernel<2, true, false, false, false>},
      {gemm_bf16_tc_kernel<3, false, false, false, false>, gemm_bf16_tc_kernel<3, true, false, false, false>}};
  static const KernelFn table_wide[4][2] = {
      {gemm_bf16_tc_kernel<0, false, false, false, true>, gemm_bf16_tc_kernel<0, true, false, false, true>},
      {gemm_bf16_tc_kernel<1, false, false, false, true>, gemm_bf16_tc_kernel<1, true, false, false, true>},
      {gemm_bf16_tc_kernel<2, false, false, false, true>, gemm_bf16_tc_kernel<2, true, false, false, true>},
      {gemm_bf16_tc_kernel<3, false, false, false, true>, gemm_bf16_tc_kernel<3, true, false, false, true>}};
  // Large products: 256 x 256 tiles on CTA pairs, once every pair has at least two of them.
  const i64 tiles_pair = ((n + 255) / 256) * ((m + 255) / 256);
  static const bool pair_on = [] { const char* e = getenv("WKB_GEMM_PAIR"); return !(e && e[0] == '0'); }();
  if (pair_on && tiles_pair >= sm_count() && sm_count() >= 2) {
    rc = make_map(&mb, b, n, k, ldb, 128);
    if (rc) return rc;
    typedef void (*PairFn)(const CUtensorMap, const CUtensorMap, void*, i64, int, int, int, GemmEpi, int*);
    static const PairFn ptable[4][2] = {{gemm_bf16_pair_kernel<0, false>, gemm_bf16_pair_kernel<0, true>},
                                        {gemm_bf16_pair_kernel<1, false>, gemm_bf16_pair_kernel<1, true>},
                                        {gemm_bf16_pair_kernel<2, false>, gemm_bf16_pair_kernel<2, true>},
                                        {gemm_bf16_pair_kernel<3, false>, gemm_bf16_pair_kernel<3, true>}};
    PairFn pk = ptable[act][c_bf16 ? 1 : 0];
    static bool pattr[64][8] = {{false}};
    int pdev = 0;
    cudaGetDevice(&pdev);
    const int pslot = (int)act * 2 + (c_bf16 ? 1 : 0);
    if (!pattr[pdev & 63][pslot]) {
      cudaError_t e = cudaFuncSetAttribute(pk, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES_PAIR);
      if (e != cudaSuccess) return (int)e;
      pattr[pdev & 63][pslot] = true;
    }
    GemmEpi pepi{bias, residual, ldr, (int)act, c_bf16, nullptr};
    i64 pairs = sm_count() / 2;
    if (pairs > tiles_pair) pairs = tiles_pair;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(PAIR_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES_PAIR;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, pk, ma, mb, c, ldc, (int)m, (int)n, (int)k, pepi, status);
  }
  // 128 x 256 tiles halve the operand bytes per flop; they pay off once there are at least two waves of them
  const i64 tiles_wide = ((n + BN_WIDE - 1) / BN_WIDE) * ((m + BM - 1) / BM);
  const bool wide = tiles_wide >= 2 * sm_count();
  if (wide) {
    rc = make_map(&mb, b, n, k, ldb, BN_WIDE);
    if (rc) return rc;
  }
  KernelFn kern = wide ? table_wide[act][c_bf16 ? 1 : 0] : table[act][c_bf16 ? 1 : 0];
  const int smem = wide ? SMEM_BYTES_WIDE : SMEM_BYTES;
  static bool attr_set[64][16] = {{false}};
  int dev = 0;
  cudaGetDevice(&dev);
  int slot = (int)act * 2 + (c_bf16 ? 1 : 0) + (wide ? 8 : 0);
  if (!attr_set[dev & 63][slot]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev & 63][slot] = true;
  }
  GemmEpi epi{bias, residual, ldr, (int)act, c_bf16, nullptr};
  i64 tiles = wide ? tiles_wide : ((n + BN - 1) / BN) * ((m + BM - 1) / BM);
  // Split-K: fp32 partials of each K slice to the workspace, one finishing pass with the epilogue.  The decision
  // depends on the shape (and the pitches' alignment) only, and the slices are summed in slice order.
  const i64 ks = splitk_slices(m, n, k);
  if (ks > 1 && ldc % 4 == 0 && (residual == nullptr || ldr % 4 == 0)) {
    if (!ws || ws_bytes < ks * m * n * 4 || (((uintptr_t)ws) & 15)) return (int)cudaErrorInvalidValue;
    KernelFn plain = table[0][0];
    if (!attr_set[dev & 63][0]) {
      cudaError_t e = cudaFuncSetAttribute(plain, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
      if (e != cudaSuccess) return (int)e;
      attr_set[dev & 63][0] = true;
    }
    GemmEpi part{nullptr, nullptr, 0, 0, 0, nullptr, (int)ks, m * n};
    part.b_static = g_b_static;
    const i64 items = tiles * ks;
    cudaError_t e = launch_pdl(plain, (unsigned)(items < sm_count() ? items : sm_count()), GEMM_THREADS, SMEM_BYTES, st, ma, mb,
                               (void*)ws, n, (int)m, (int)n, (int)k, part, status);
    if (e != cudaSuccess) return (int)e;
    const i64 total = m * (n / 4);
    i64 g = (total + 255) / 256;
    if (g > sm_count() * 8) g = sm_count() * 8;
    return (int)launch_pdl(gemm_splitk_finish_kernel, (unsigned)g, 256, 0, st, (const float*)ws, (int)ks, m * n, (int)m, (int)n, c,
                           ldc, c_bf16, bias, (int)act, residual, ldr);
  }
  unsigned grid = (unsigned)(tiles < sm_count() ? tiles : sm_count());
  epi.b_static = g_b_static;
  return (int)launch_pdl(kern, grid, GEMM_THREADS, smem, st, ma, mb, c, ldc, (int)m, (int)n, (int)k, epi, status);
}

// Allocates this device's default split-K workspace (32 MiB) and the status word.  Call once per device before
// capturing wkb_gemm_bf16_nt into a CUDA graph; without it the first split-shaped call outside a capture allocates.
int wkb_gemm_init(void) {
  if (!gemm_status_word()) return (int)cudaErrorMemoryAllocation;
  return splitk_workspace(nullptr, true) ? 0 : (int)cudaErrorMemoryAllocation;
}

// Bytes of workspace wkb_gemm_bf16_nt_ws needs for this shape (0: the shape does not split K).
i64 wkb_gemm_workspace_bytes(i64 m, i64 n, i64 k) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  const i64 ks = splitk_slices(m, n, k);
  return ks > 1 ? ks * m * n * 4 : 0;
}

int wkb_gemm_bf16_nt_ws(const void* a, i64 lda, const void* b, i64 ldb, void* c, i64 ldc, int c_bf16, i64 m, i64 n, i64 k,
                        const float* bias, i64 act, const float* residual, i64 ldr, void* workspace, i64 workspace_bytes, void* stream) {
  return gemm_bf16_nt_impl(a, lda, b, ldb, c, ldc, c_bf16, m, n, k, bias, act, residual, ldr, (float*)workspace, workspace_bytes,
                           as_stream(stream));
}

// K-slice partials only (no epilogue): slice s of the product goes to workspace + s * m * n as an fp32 [m, n] plane, for a
// consumer that adds the planes in slice order while it does its own row-wise work (wkb_add_slices_layernorm_bf16).
// The number of slices depends on the shape only: as many as keep every SM busy, each at least three 64-element K steps
// long, at most 8.  wkb_gemm_bf16_partial_layout reports it; the workspace must hold slices * m * n floats.
static i64 partial_slices(i64 m, i64 n, i64 k) {
  const i64 tiles = ((n + BN - 1) / BN) * ((m + BM - 1) / BM);
  const i64 kiters = (k + 63) / 64;
  i64 ks = sm_count() / (tiles > 0 ? tiles : 1);
  if (ks > 8) ks = 8;
  if (ks > kiters / 3) ks = kiters / 3;
  if (ks < 1) ks = 1;
  const i64 kper = (kiters + ks - 1) / ks;
  return (kiters + kper - 1) / kper;
}

void wkb_gemm_bf16_partial_layout(i64 m, i64 n, i64 k, i64* slices, i64* slice_stride) {
  *slices = (m > 0 && n > 0 && k > 0) ? partial_slices(m, n, k) : 0;
  *slice_stride = m * n;
}

int wkb_gemm_bf16_nt_partial(const void* a, i64 lda, const void* b, i64 ldb, i64 m, i64 n, i64 k, void* workspace, i64 workspace_bytes,
                             void* stream) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  if (k % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || n % 4 != 0) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)workspace)) & 15) return (int)cudaErrorMisalignedAddress;
  const i64 ks = partial_slices(m, n, k);
  if (!workspace || workspace_bytes < ks * m * n * 4) return (int)cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, a, m, k, lda, BM);
  if (rc) return rc;
  rc = make_map(&mb, b, n, k, ldb, BN);
  if (rc) return rc;
  int* status = gemm_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  auto kern = gemm_bf16_tc_kernel<0, false, false, false, false>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev & 63] = true;
  }
  GemmEpi part{};
  part.ksplit = (int)ks;
  part.slice_stride = m * n;
  part.b_static = g_b_static;
  const i64 items = ((n + BN - 1) / BN) * ((m + BM - 1) / BM) * ks;
  return (int)launch_pdl(kern, (unsigned)(items < sm_count() ? items : sm_count()), GEMM_THREADS, SMEM_BYTES, as_stream(stream), ma, mb, workspace,
                         n, (int)m, (int)n, (int)k, part, status);
}

// x[m, n] += A.B^T + bias with the K slices of a tile summed inside a thread-block cluster (the CLUSTERK instantiation).
// Slices for a problem: 0 = not offered (the caller uses wkb_gemm_bf16_nt_partial and sums the slices itself).  The rule
// depends on the shape and the SM count only: 2, 4 or 8 slices, at least three 64-wide K steps each, all CTAs in one wave.
static i64 cluster_slices(i64 m, i64 n, i64 k) {
  static const bool off = getenv("WKB_GEMM_NO_CLUSTERK") != nullptr;   // switch for A/B timing: never offer the cluster form
  if (m <= 0 || n <= 0 || k <= 0 || n % 4 != 0 || off) return 0;
  const i64 tiles = ((n + BN - 1) / BN) * ((m + BM - 1) / BM);
  const i64 kiters = (k + 63) / 64;
  i64 ks = 8;
  // (the last slice must not be empty: slices are ceil(kiters / ks) steps long)
  while (ks >= 2 && (tiles * ks > sm_count() || kiters / ks < 3 || (ks - 1) * ((kiters + ks - 1) / ks) >= kiters)) ks >>= 1;
  return ks >= 2 ? ks : 0;
}

i64 wkb_gemm_bf16_addto_slices(i64 m, i64 n, i64 k) { return cluster_slices(m, n, k); }

int wkb_gemm_bf16_nt_addto(const void* a, i64 lda, const void* b, i64 ldb, float* x, i64 ldx, i64 m, i64 n, i64 k, const float* bias,
                           void* stream) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  if (k % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || n % 4 != 0 || ldx % 4 != 0) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)x) | ((uintptr_t)bias)) & 15) return (int)cudaErrorMisalignedAddress;
  const i64 ks = cluster_slices(m, n, k);
  if (ks == 0) return (int)cudaErrorNotSupported;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, a, m, k, lda, BM);
  if (rc) return rc;
  rc = make_map(&mb, b, n, k, ldb, BN);
  if (rc) return rc;
  int* status = gemm_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  auto kern = gemm_bf16_tc_kernel<0, false, false, false, false, false, false, true>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev & 63] = true;
  }
  GemmEpi epi{};
  epi.bias = bias;
  epi.ksplit = (int)ks;
  epi.slice_stride = 0;
  epi.b_static = g_b_static;
  const i64 tiles = ((n + BN - 1) / BN) * ((m + BM - 1) / BM);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * ks));
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = as_stream(stream);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)ks; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, ma, mb, (void*)x, ldx, (int)m, (int)n, (int)k, epi, status);
}

// The fused QKV projection of a decode step: C[:, :kv_col0] = A.B^T + bias (fp32, the query heads); columns
// [kv_col0, kv_col0 + 2 * kv_heads * head_dim) -- the new K rows, then the new V rows -- are rounded to bf16 straight
// into their pages at row_pos through the block table and are not stored to C (the work of wkb_paged_kv_append, without
// its launch and without the fp32 round trip).  n must be kv_col0 + 2 * kv_heads * head_dim; kv_col0 and head_dim are
// multiples of 32 (a 32-column piece of the accumulator is then 32 consecutive dims of one head), the caches and the bias
// 16-byte aligned.
int wkb_gemm_bf16_nt_qkv_append(const void* a, i64 lda, const void* b, i64 ldb, float* c, i64 ldc, i64 m, i64 n, i64 k, const float* bias,
                                i64 kv_col0, void* kcache, void* vcache, const uint32_t* block_table, const int* row_slot, const int* row_pos,
                                i64 kv_heads, i64 head_dim, i64 page_tokens, i64 max_blocks_per_seq, void* stream) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  if (k % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0) return (int)cudaErrorInvalidValue;
  if (kv_col0 < 0 || kv_col0 % 32 != 0 || kv_heads <= 0 || head_dim <= 0 || head_dim % 32 != 0 || page_tokens <= 0 || max_blocks_per_seq <= 0 ||
      n != kv_col0 + 2 * kv_heads * head_dim)
    return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)kcache) | ((uintptr_t)vcache) | ((uintptr_t)bias)) & 15) return (int)cudaErrorMisalignedAddress;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, a, m, k, lda, BM);
  if (rc) return rc;
  // 64-column tiles while they still fit one wave: a decode batch of 512 rows x 2304 columns is 72 tiles of 128 columns
  // (half the SMs idle) but 144 of 64
  const i64 tiles_narrow = ((n + 63) / 64) * ((m + BM - 1) / BM);
  static const bool keep_wide = getenv("WKB_QKV_WIDE") != nullptr;     // switch for A/B timing: always 128-column tiles
  const bool narrow = tiles_narrow <= sm_count() && !keep_wide;
  const int bn = narrow ? 64 : BN;
  rc = make_map(&mb, b, n, k, ldb, bn);
  if (rc) return rc;
  int* status = gemm_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  auto kern = narrow ? gemm_bf16_tc_kernel<0, false, false, false, false, true, true> : gemm_bf16_tc_kernel<0, false, false, false, false, true, false>;
  static bool attr_set[64][2] = {{false}};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63][narrow ? 1 : 0]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev & 63][narrow ? 1 : 0] = true;
  }
  GemmEpi epi{};
  epi.bias = bias;
  epi.kcache = (u16*)kcache;
  epi.vcache = (u16*)vcache;
  epi.block_table = block_table;
  epi.row_slot = row_slot;
  epi.row_pos = row_pos;
  epi.kv_col0 = (int)kv_col0;
  epi.kv_heads = (int)kv_heads;
  epi.kv_hd = (int)head_dim;
  epi.page_tokens = (int)page_tokens;
  epi.mbps = (int)max_blocks_per_seq;
  epi.b_static = g_b_static;
  const i64 tiles = ((n + bn - 1) / bn) * ((m + BM - 1) / BM);
  return (int)launch_pdl(kern, (unsigned)(tiles < sm_count() ? tiles : sm_count()), GEMM_THREADS, SMEM_BYTES, as_stream(stream), ma, mb, (void*)c, ldc,
                         (int)m, (int)n, (int)k, epi, status);
}

// The same with this device's default workspace, which every stream and host thread shares: only one split-shaped
// GEMM may be in flight per device through this entry (use wkb_gemm_bf16_nt_ws with a workspace per stream otherwise).
// A split-shaped call that finds no workspace while its stream is capturing returns cudaErrorNotReady: call
// wkb_gemm_init first.
int wkb_gemm_bf16_nt(const void* a, i64 lda, const void* b, i64 ldb, void* c, i64 ldc, int c_bf16, i64 m, i64 n, i64 k,
                     const float* bias, i64 act, const float* residual, i64 ldr, void* stream) {
  float* ws = nullptr;
  if (m > 0 && n > 0 && k > 0 && splitk_slices(m, n, k) > 1) {
    ws = splitk_workspace(as_stream(stream), true);
    if (!ws) return (int)cudaErrorNotReady;
  }
  return gemm_bf16_nt_impl(a, lda, b, ldb, c, ldc, c_bf16, m, n, k, bias, act, residual, ldr, ws, (i64)SPLITK_WS_BYTES, as_stream(stream));
}

// E4M3 x E4M3 -> fp32 accumulate: same kernel with kind::f8f6f4 MMAs and 128 elements of K per stage.
int wkb_gemm_e4m3_nt(const void* a, i64 lda, const void* b, i64 ldb, void* c, i64 ldc, int c_bf16, i64 m, i64 n, i64 k,
                     const float* bias, i64 act, const float* residual, i64 ldr, void* stream) {
  if (m <= 0 || n <= 0 || k <= 0) return 0;
  if (k % 16 != 0 || lda % 16 != 0 || ldb % 16 != 0) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)a) | ((uintptr_t)b)) & 15) return (int)cudaErrorMisalignedAddress;
  if (act < 0 || act > 3) return (int)cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, a, m, k, lda, BM, true);
  if (rc) return rc;
  rc = make_map(&mb, b, n, k, ldb, BN, true);
  if (rc) return rc;
  int* status = gemm_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, void*, i64, int, int, int, GemmEpi, int*);
  static const KernelFn table[4][2] = {
      {gemm_bf16_tc_kernel<0, false, false, true, false>, gemm_bf16_tc_kernel<0, true, false, true, false>},
      {gemm_bf16_tc_kernel<1, false, false, true, false>, gemm_bf16_tc_kernel<1, true, false, true, false>},
      {gemm_bf16_tc_kernel<2, false, false, true, false>, gemm_bf16_tc_kernel<2, true, false, true, false>},
      {gemm_bf16_tc_kernel<3, false, false, true, false>, gemm_bf16_tc_kernel<3, true, false, true, false>}};
  KernelFn kern = table[act][c_bf16 ? 1 : 0];
  static bool attr_set[64][8] = {{false}};
  int dev = 0;
  cudaGetDevice(&dev);
  int slot = (int)act * 2 + (c_bf16 ? 1 : 0);
  if (!attr_set[dev & 63][slot]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev & 63][slot] = true;
  }
  GemmEpi epi{bias, residual, ldr, (int)act, c_bf16, nullptr};
  i64 tiles = ((n + BN - 1) / BN) * ((m + BM - 1) / BM);
  unsigned grid = (unsigned)(tiles < sm_count() ? tiles : sm_count());
  kern<<<grid, GEMM_THREADS, SMEM_BYTES, as_stream(stream)>>>(ma, mb, c, ldc, (int)m, (int)n, (int)k, epi, status);
  return (int)cudaGetLastError();
}

i64 wkb_gemm_argmax_tiles(i64 n) { return 2 * ((n + BN - 1) / BN); }   // two candidates per 128-column tile

// out[i] = argmax_j (A.B^T + bias)[i, j] without materialising the product: every column tile leaves
// one (value, column) candidate per row in part_val / part_idx ([m, wkb_gemm_argmax_tiles(n)] each),
// then a small kernel folds them.  Ties and NaNs follow wkb_rowargmax_i32.
int wkb_gemm_bf16_nt_argmax(const void* a, i64 lda, const void* b, i64 ldb, i64 m, i64 n, i64 k, const float* bias,
                            float* part_val, int* part_idx, int* out, void* stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k <= 0 || k % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)a) | ((uintptr_t)b)) & 15) return (int)cudaErrorMisalignedAddress;
  CUtensorMap ma, mb;
  int rc = make_map(&ma, a, m, k, lda, BM);
  if (rc) return rc;
  // 256-column tiles once they still fill two waves: a tile then moves 48 KB through shared memory per K step for twice the
  // work of a 128-column one (32 KB); with two epilogue warps per lane quarter the scan of 256 columns keeps up
  const bool wide = ((n + BN_WIDE - 1) / BN_WIDE) * ((m + BM - 1) / BM) >= 2 * (i64)sm_count();
  const int bn = wide ? BN_WIDE : BN;
  rc = make_map(&mb, b, n, k, ldb, bn);
  if (rc) return rc;
  int* status = gemm_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  auto kern = wide ? gemm_bf16_tc_kernel<0, false, true, false, true> : gemm_bf16_tc_kernel<0, false, true, false, false>;
  const int smem = wide ? SMEM_BYTES_WIDE : SMEM_BYTES;
  static bool attr_set[64][2] = {{false}};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63][wide ? 1 : 0]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev & 63][wide ? 1 : 0] = true;
  }
  GemmEpi epi{bias, nullptr, 0, 0, 0, part_idx};
  epi.b_static = g_b_static;
  // (the candidate arrays hold wkb_gemm_argmax_tiles(n) entries per row, the count for 128-column tiles: an upper bound)
  i64 tiles_n = (n + bn - 1) / bn, tiles = tiles_n * ((m + BM - 1) / BM);
  unsigned grid = (unsigned)(tiles < sm_count() ? tiles : sm_count());
  cudaError_t e = launch_pdl(kern, grid, GEMM_THREADS, smem, as_stream(stream), ma, mb, (void*)part_val, (i64)0, (int)m, (int)n, (int)k, epi,
                             status);
  if (e != cudaSuccess) return (int)e;
  return (int)launch_pdl(argmax_tiles_kernel, (unsigned)((m * 32 + 127) / 128), 128, 0, as_stream(stream), (const float*)part_val,
                         (const int*)part_idx, (int)(2 * tiles_n), out, (int)m);
}

// While set (non-zero) on the calling thread, every dense tensor-core GEMM launched from it may read its B operand before
// the preceding kernel of the stream has completed: the caller promises that B (resident weights) is not written by any
// kernel still in flight on that stream.  A is always read after that kernel.  Returns the previous setting.
int wkb_gemm_b_static(int on) {
  const int was = g_b_static;
  g_b_static = on ? 1 : 0;
  return was;
}

// Reads (and clears) the bounded-wait status of the tensor-core GEMM on the current device:
// 0 = every wait completed; 1 / 2 / 3 / 4 = the producer / MMA-operand / epilogue / MMA-accumulator
// wait ran out.  Synchronises.
int wkb_gemm_status(void) {
  int* status = gemm_status_word();
  if (!status) return -1;
  int v = 0;
  if (cudaMemcpy(&v, status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  if (v) cudaMemset(status, 0, sizeof(int));
  return v;
}

}

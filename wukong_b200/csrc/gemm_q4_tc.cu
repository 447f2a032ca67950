// W4A16 GEMM on the tensor cores: out[M, N] = x[M, K] . W[N, K]^T for resident Q4_0 weights and bf16
// activations, M <= 64 rows per pass (batched decode).  Replaces the reference's int4 GEMM family
// (crates/wukong_codegen_gpu/src/ptx_int4.rs: dequantise-in-register W4A16 tiles over mma.sync) for
// sm_100a; block format and nibble order are the Q4_0 ones of crates/wukong_runtime/src/quant.rs:13-16.
//
// The kernel is bound by the weight stream (0.5625 B per weight) and, on this part, by the instructions it
// takes to turn nibbles into tensor-core operands, so it is built to keep both busy on every SM:
//   * the activation slice x[:, k-slice] (<= 1024 columns, 128 KB) is loaded once per CTA (one barrier per
//     256-K stage, so the first MMAs start when a quarter of it has landed) and stays in shared memory; a CTA owns one K slice and walks over weight-row tiles of 128 rows;
//   * warp 0 streams raw tiles (128 rows x 256 K: 16 KB of nibbles + 2 KB of f16 scales) through a
//     5-stage TMA ring (128-byte swizzle, no multicast);
//   * warps 4-19 dequantise, in two teams of eight (each feeding its own MMA warp, so a stage is handed over between
//     8 warps and one lane, not 16; the teams take alternate stages of the stream): thread = weight row, four 32-value
//     blocks of each stage, written as two half-stage buffers so that the MMAs of one half run while the
//     other half is converted; nibble -> bf16 with
//     one byte permute (0x4300 | nib = 128 + nib exactly), subtract 136, multiply by the block scale rounded
//     to bf16, all in bf16x2 (the reference's kernel does the same two operations per pair in f16x2, its
//     activations being f16).  The result is written with tcgen05.st straight into TENSOR MEMORY, where
//     lane = weight row and a column holds two consecutive K values: the MMA's A operand never touches
//     shared memory, so there is no swizzled store and no proxy fence; one 256-K stage of operand
//     buffering per team (two halves, recycled independently) sits beside the four accumulators in the 512
//     TMEM columns;
//   * warps 1 and 2 issue tcgen05.mma with A in tensor memory and B (activations) from shared memory
//     (M = 128 weight rows, N = 64 activation rows, K = 16) x 16 per stage; tcgen05.commit recycles the
//     operand stage.  One thread issues such an MMA about every 27-36 ns, the tensor pipe retires one every
//     19-20 ns (measured with two issuing warps), so two warps issue: stage s of the CTA's j-th tile belongs to team
//     (j + s) & 1, each team accumulates its stages of a tile into its own accumulator, and the epilogue adds the two
//     (team 0's sum + team 1's sum: a fixed order).  Both teams are busy whatever the number of tiles a CTA owns; one
//     team per tile left a team idle on a single or an odd last tile;
//   * warps 20-27 read the accumulators (four of them: two per tile, so a tile is finished while the next one
//     is multiplied; the two sets of four warps take alternate tiles; thread = weight row, 64 activation rows in
//     registers).
//     With one K slice they finish the tile directly.  With several, they write the partial tile to
//     the workspace and count arrivals per (tile, lane quarter); the last arriving warp adds the
//     slices in slice order (so the result does not depend on arrival order) and finishes.
//   Finishing = optional SwiGLU (rows interleaved gate, up, gate, up ...: silu(gate) * up), rounding to
//   bf16 if asked, and a store that is coalesced across lanes (consecutive n for one m).
// The weight value the tensor core sees is exactly bf16_rn(bf16_rn(d) * (nib - 8)); accumulation is
// fp32 in the tensor core's own order.
// The kernel is launched as a programmatic dependent: the weight stream does not depend on the kernel before it, so the
// first ring of raw stages is requested (and dequantised) while that kernel is still draining; only the activation load
// and the stores wait for it.
// Every mbarrier wait is bounded; on expiry a code is recorded in the status word, the role stops
// issuing, and the CTA drains and frees its TMEM.
#include "common.cuh"
#include "wkb_device.h"
#include "tc_common.cuh"

namespace wkb {
int* gemm_status_word();
i64 gemm_sm_count();

namespace q4tc {

constexpr int TN = 128;        // weight rows per tile (MMA M)
constexpr int TM = 64;         // activation rows per pass (MMA N)
constexpr int STAGE_K = 256;   // K per raw stage: 128 B of nibbles per row
constexpr int KS_MAX = 1024;   // K per resident activation slice
constexpr int RAW_STAGES = 5;
constexpr int RAW_BYTES = TN * 128, SCALE_BYTES = TN * 16, RAW_STAGE_BYTES = RAW_BYTES + SCALE_BYTES;
constexpr int X_SUB_BYTES = TM * 128;
constexpr int X_BYTES = (KS_MAX / 64) * X_SUB_BYTES;
// tensor memory: columns 0-255 four fp32 accumulators (64 activation rows each), 256-511 one stage buffer of
// dequantised weights per team (256 K as 128 columns of bf16 pairs, two halves of 64 columns; lane = weight row)
constexpr int A_STAGE_COLS = STAGE_K / 2, A_HALF_COLS = A_STAGE_COLS / 2, NUM_ACC = 4, A_COL0 = NUM_ACC * TM;
constexpr uint32_t TMEM_COLS = 512;
constexpr int X_STAGES = KS_MAX / STAGE_K;
constexpr int NUM_BARS = X_STAGES + 2 * RAW_STAGES + 8 + 2 * NUM_ACC;
constexpr int SMEM = X_BYTES + RAW_STAGES * RAW_STAGE_BYTES + 1024 + 256;
static_assert(8 * NUM_BARS + 8 <= 256, "barriers and the TMEM slot share 256 bytes");
// warps: 0 TMA producer, 1-2 MMA issuers, 3 TMEM allocation, 4-19 dequantisers (two teams of 8), 20-27 epilogue (two sets of 4)
constexpr int DEQ_WARP0 = 4, TEAM_WARPS = 8, EPI_WARP0 = DEQ_WARP0 + 2 * TEAM_WARPS, THREADS = 32 * (EPI_WARP0 + 8);
// instruction descriptor, kind::f16: D = f32, A = B = bf16 (the two operand formats must agree: an f16 A with a
// bf16 B is rejected by the hardware as an illegal instruction)
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TM >> 3) << 17) | ((uint32_t)(TN >> 4) << 24);

struct Plan {
  int n_tiles, kstages, ksplit, stages_per_slice, groups;
  int kstages_pitch;   // stages per tile row in the resident layout (>= kstages)
};

// Choose the K split: a slice holds at most KS_MAX / STAGE_K stages; among the feasible splits take
// the one with the fewest (rounds x (stages + 1)) -- the +1 stands for the per-tile fixed cost -- and,
// between equals, the one with fewer slices to add up.
inline Plan make_plan(i64 n, i64 k, i64 sms) {
  Plan p;
  p.n_tiles = (int)((n + TN - 1) / TN);
  p.kstages = (int)((k + STAGE_K - 1) / STAGE_K);
  int best_cost = 1 << 30;
  p.ksplit = 1; p.stages_per_slice = p.kstages; p.groups = 1; p.kstages_pitch = p.kstages;
  for (int sps = KS_MAX / STAGE_K; sps >= 1; --sps) {
    int ks = (p.kstages + sps - 1) / sps;
    if (ks > sms) continue;
    int groups = (int)(sms / ks);
    if (groups > p.n_tiles) groups = p.n_tiles;
    int rounds = (p.n_tiles + groups - 1) / groups;
    int cost = rounds * (sps + 1) * 8 + ks;
    if (cost < best_cost) { best_cost = cost; p.ksplit = ks; p.stages_per_slice = sps; p.groups = groups; }
  }
  return p;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
// two nibbles (already isolated in bytes, widened to 0x4300 | nib = 128 + nib in bf16) -> bf16x2 of
// d * (nib - 8): the subtraction is exact, the product is rounded once
__device__ __forceinline__ uint32_t deq2(uint32_t pair_bits, uint32_t d2) {
  uint32_t r;
  asm("{\n .reg .b32 t;\n sub.rn.bf16x2 t, %1, %2;\n mul.rn.bf16x2 %0, t, %3;\n}"
      : "=r"(r) : "r"(pair_bits), "r"(0x43084308u), "r"(d2));
  return r;
}
// one 32-value block (16 raw bytes: byte j = element j | element j + 16 << 4) -> 16 registers of bf16 pairs in
// element order
__device__ __forceinline__ void deq_block(const uint4 w, uint32_t d2, uint32_t* o) {
  const uint32_t lo[4] = {w.x & 0x0F0F0F0Fu, w.y & 0x0F0F0F0Fu, w.z & 0x0F0F0F0Fu, w.w & 0x0F0F0F0Fu};
  const uint32_t hi[4] = {(w.x >> 4) & 0x0F0F0F0Fu, (w.y >> 4) & 0x0F0F0F0Fu, (w.z >> 4) & 0x0F0F0F0Fu, (w.w >> 4) & 0x0F0F0F0Fu};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = deq2(prmt(lo[i], 0x43434343u, 0x4140u), d2);          // elements 4i, 4i+1
    o[2 * i + 1] = deq2(prmt(lo[i], 0x43434343u, 0x4342u), d2);      // 4i+2, 4i+3
    o[8 + 2 * i] = deq2(prmt(hi[i], 0x43434343u, 0x4140u), d2);      // 16+4i, 16+4i+1
    o[8 + 2 * i + 1] = deq2(prmt(hi[i], 0x43434343u, 0x4342u), d2);  // 16+4i+2, 16+4i+3
  }
}
// f16 scale bits -> the scale rounded to bf16 (nearest even), in both halves of a register
__device__ __forceinline__ uint32_t bf16x2_of_f16(uint32_t h) {
  uint32_t r;
  asm("{\n .reg .b16 t;\n .reg .f32 f;\n cvt.u16.u32 t, %1;\n cvt.f32.f16 f, t;\n cvt.rn.bf16x2.f32 %0, f, f;\n}" : "=r"(r) : "r"(h));
  return r;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
// 1-D bulk copy global -> shared, completion counted on an mbarrier (addresses and size multiples of 16 bytes)
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// MMA with the A operand in tensor memory (lane = row, a column holds two consecutive K elements)
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 registers -> 32 consecutive columns of this thread's TMEM lane; the caller waits for the store (tcgen05.wait::st)
// before it tells anyone about it
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
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

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
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

// 16 consecutive columns of this thread's TMEM lane, added to acc[0..15]
__device__ __forceinline__ void tmem_ld16_add(uint32_t taddr, float* acc) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int e = 0; e < 16; ++e) acc[e] += __uint_as_float(r[e]);
}

// Finish 32 activation rows (m0 .. m0+31) of weight row n held one per register.
// MODE 0: f32 out[m, n]; 1: bf16 out[m, n]; 2: SwiGLU, bf16 out[m, n / 2] from (gate = even n, up = odd n).
// (MODE 3 never finishes in the kernel: the K-slice partials are the result, left in the workspace for a consumer
// that adds them up itself.)
template <int MODE>
__device__ __forceinline__ void finish32(const float (&v)[32], int m0, int M, int n, int N, void* out, i64 ldo) {
  const int mcount = min(32, M - m0);
  if (MODE == 2) {
#pragma unroll
    for (int e = 0; e < 32; ++e) {
      const float up = __shfl_xor_sync(0xffffffffu, v[e], 1);
      if (e < mcount && n < N && !(n & 1)) {
        const float y = fmul(silu1(v[e]), up);
        reinterpret_cast<u16*>(out)[(i64)(m0 + e) * ldo + (n >> 1)] = f32_to_bf16_bits(y);
      }
    }
  } else if (n < N) {
    if (mcount == 32) {
      if (MODE == 1) {
        u16* p = reinterpret_cast<u16*>(out) + (i64)m0 * ldo + n;
#pragma unroll
        for (int e = 0; e < 32; ++e) p[(i64)e * ldo] = f32_to_bf16_bits(v[e]);
      } else {
        float* p = reinterpret_cast<float*>(out) + (i64)m0 * ldo + n;
#pragma unroll
        for (int e = 0; e < 32; ++e) p[(i64)e * ldo] = v[e];
      }
    } else {
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        if (e < mcount) {
          if (MODE == 1) reinterpret_cast<u16*>(out)[(i64)(m0 + e) * ldo + n] = f32_to_bf16_bits(v[e]);
          else reinterpret_cast<float*>(out)[(i64)(m0 + e) * ldo + n] = v[e];
        }
      }
    }
  }
}

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_q4_tc_kernel(const __grid_constant__ CUtensorMap map_x, const uint8_t* __restrict__ wt, void* out, i64 ldo, int M, int N,
                  Plan plan, float* ws, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t x_base = base, raw_base = base + X_BYTES;
  const uint32_t bars = raw_base + RAW_STAGES * RAW_STAGE_BYTES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + X_BYTES + RAW_STAGES * RAW_STAGE_BYTES + 8 * NUM_BARS);
  auto x_full = [&](int s) { return bars + 8u * s; };                                  // one per 256-K stage of the slice
  auto raw_full = [&](int s) { return bars + 8u * (X_STAGES + s); };
  auto raw_empty = [&](int s) { return bars + 8u * (X_STAGES + RAW_STAGES + s); };
  auto a_full = [&](int team, int half) { return bars + 8u * (X_STAGES + 2 * RAW_STAGES + team * 2 + half); };
  auto a_empty = [&](int team, int half) { return bars + 8u * (X_STAGES + 2 * RAW_STAGES + 4 + team * 2 + half); };
  auto t_full = [&](int b) { return bars + 8u * (X_STAGES + 2 * RAW_STAGES + 8 + b); };
  auto t_empty = [&](int b) { return bars + 8u * (X_STAGES + 2 * RAW_STAGES + 8 + NUM_ACC + b); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ks = blockIdx.x % plan.ksplit, group = blockIdx.x / plan.ksplit;
  const int stage0 = ks * plan.stages_per_slice;
  const int nstages = min(plan.stages_per_slice, plan.kstages - stage0);  // >= 1 by construction
  // This CTA's tiles are group, group + groups, ...; the producer streams them tile by tile, stage by stage.  Stage s of
  // local tile j belongs to team (j + s) & 1 (dequantiser warps 4-11 + MMA warp 1, or 12-19 + warp 2): the two teams work on
  // the SAME tile, on alternate stages, each into its own accumulator (2 * (j & 1) + team), and the epilogue adds the two.
  // Both teams are therefore busy whatever the number of tiles (a CTA with a single tile, or an odd one out, used to
  // leave one team idle), and they stay in step with the stream.
  const int ntl = group < plan.n_tiles ? (plan.n_tiles - group + plan.groups - 1) / plan.groups : 0;
  const int total_its = ntl * nstages;
  auto locate = [&](int it, int& j, int& s) { j = it / nstages; s = it - j * nstages; };
  auto position = [&](int j, int s) { return j * nstages + s; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < X_STAGES; ++s) mbar_init(x_full(s), 1);
    for (int s = 0; s < RAW_STAGES; ++s) { mbar_init(raw_full(s), 1); mbar_init(raw_empty(s), TEAM_WARPS); }
    for (int b = 0; b < 4; ++b) { mbar_init(a_full(b >> 1, b & 1), TEAM_WARPS); mbar_init(a_empty(b >> 1, b & 1), 1); }
    for (int b = 0; b < NUM_ACC; ++b) { mbar_init(t_full(b), 1); mbar_init(t_empty(b), 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
  }
  if (warp == 3) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_trigger();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      auto issue_raw = [&](int upto) {
        for (; it < upto && ok; ++it) {
          int j, st;
          locate(it, j, st);
          const int slot = it % RAW_STAGES;
          if (!mbar_wait_parked(raw_empty(slot), ((it / RAW_STAGES) & 1) ^ 1)) { atomicExch(status, 11); ok = false; break; }
          mbar_expect_tx(raw_full(slot), RAW_STAGE_BYTES);
          // one contiguous 18 KB stage image: (tile, stage) -> nibble rows already in their swizzled places, then scales
          bulk_load(raw_base + slot * RAW_STAGE_BYTES,
                    wt + ((i64)(group + j * plan.groups) * plan.kstages_pitch + stage0 + st) * RAW_STAGE_BYTES, RAW_STAGE_BYTES, raw_full(slot));
        }
      };
      // the resident weights do not depend on the kernel before this one: fill the ring first, then wait for that kernel
      // and fetch its output, the activation slice
      issue_raw(min(RAW_STAGES, total_its));
      pdl_wait();
      for (int xs = 0; xs < nstages; ++xs) {
        mbar_expect_tx(x_full(xs), 4u * X_SUB_BYTES);
        for (int j = 4 * xs; j < 4 * xs + 4; ++j) tma_load_2d(x_base + j * X_SUB_BYTES, &map_x, x_full(xs), stage0 * STAGE_K + j * 64, 0);
      }
      issue_raw(total_its);
      if (!ok) {
        // wait (bounded) for the copies already started before the CTA may exit
        for (int xs = 0; xs < nstages; ++xs) mbar_wait(x_full(xs), 0);
        for (int j = it > RAW_STAGES ? it - RAW_STAGES : 0; j < it; ++j) mbar_wait(raw_full(j % RAW_STAGES), (j / RAW_STAGES) & 1);
      }
    }
  } else if (warp <= 2) {
    // ---------------- MMA issuers: A (dequantised weights) from tensor memory, B (activations) from shared memory ----------------
    // warp 1 takes the even local tiles, warp 2 the odd ones
    if (lane == 0) {
      const int team = warp - 1;
      bool ok = true;
      int n = 0;                                    // stages this team has multiplied so far
      const uint64_t bdesc0 = make_sdesc(x_base);   // the start-address field counts 16-byte units: later operands are plain adds
      const uint32_t ta0 = tmem_base + (uint32_t)(A_COL0 + team * A_STAGE_COLS);
      for (int j = 0; j < ntl && ok; ++j) {
        const int s_first = (j + team) & 1;        // this team's stages of tile j: s_first, s_first + 2, ...
        if (s_first >= nstages) continue;          // a one-stage slice: the other team has the tile to itself
        const int acc = 2 * (j & 1) + team;
        if (!mbar_wait_parked(t_empty(acc), ((j >> 1) & 1) ^ 1)) { atomicExch(status, 13); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * TM);
        for (int s = s_first; s < nstages && ok; s += 2, ++n) {
          if (!mbar_wait_parked(x_full(s), 0)) { atomicExch(status, 12); ok = false; break; }   // completes once; later tiles pass at once
          const uint64_t bd = bdesc0 + (uint64_t)((s * 4 * X_SUB_BYTES) >> 4);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            if (!mbar_wait_parked(a_full(team, half), n & 1)) { atomicExch(status, 14); ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int k = 8 * half; k < 8 * half + 8; ++k)
              umma_bf16_ts(tmem_d, ta0 + (uint32_t)(k * 8), bd + (uint64_t)(((k >> 2) * X_SUB_BYTES + (k & 3) * 32) >> 4), IDESC,
                           (s == s_first && k == 0) ? 0u : 1u);   // this team's first K step of a tile overwrites its accumulator
            umma_commit(a_empty(team, half));
          }
        }
        if (ok) umma_commit(t_full(acc));
      }
    }
  } else if (warp == 3) {
    // nothing more: this warp owns the tensor-memory allocation
  } else if (warp < EPI_WARP0) {
    // ---------------- dequantisers: thread = weight row (its TMEM lane), four 32-value blocks of every 256-K stage of its team ----------------
    const int team = (warp - DEQ_WARP0) >> 3, quarter = warp & 3, part = ((warp - DEQ_WARP0) >> 2) & 1;   // a warp reaches only the TMEM lanes of its quarter
    const int r = quarter * 32 + lane;
    const uint32_t swz = (uint32_t)(r & 7);
    const uint32_t ta0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(A_COL0 + team * A_STAGE_COLS + part * 32);
    bool ok = true;
    int n = 0;            // stages this team has converted so far
    int pending = -1;     // half whose tcgen05.st has been issued but not yet announced
    // A store is announced to the MMA lane only after the next piece of work has been started: the thread then never sits in
    // tcgen05.wait::st right behind its own store.
    auto publish = [&]() {
      if (pending >= 0) {
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(a_full(team, pending));
        pending = -1;
      }
    };
    for (int j = 0; j < ntl && ok; ++j) {
      for (int s = (j + team) & 1; s < nstages && ok; s += 2, ++n) {
        const int it = position(j, s);
        const int slot = it % RAW_STAGES;
        if (!mbar_wait_parked(raw_full(slot), (it / RAW_STAGES) & 1)) { if (lane == 0) atomicExch(status, 15); ok = false; break; }
        const uint32_t rawp = raw_base + slot * RAW_STAGE_BYTES;
        // blocks 2*part, 2*part+1 (first half of the stage) and 4+2*part, 5+2*part (second half), with their f16 scales
        const uint4 q0 = lds128(rawp + r * 128 + (((uint32_t)(2 * part) ^ swz) << 4));
        const uint4 q1 = lds128(rawp + r * 128 + (((uint32_t)(2 * part + 1) ^ swz) << 4));
        const uint4 q2 = lds128(rawp + r * 128 + (((uint32_t)(4 + 2 * part) ^ swz) << 4));
        const uint4 q3 = lds128(rawp + r * 128 + (((uint32_t)(5 + 2 * part) ^ swz) << 4));
        const uint32_t sw0 = lds32(rawp + RAW_BYTES + r * 16 + part * 4);
        const uint32_t sw1 = lds32(rawp + RAW_BYTES + r * 16 + (2 + part) * 4);
        publish();                                                          // the previous stage's second half
        __syncwarp();
        if (lane == 0) mbar_arrive(raw_empty(slot));                        // the stage now lives in registers
        uint32_t v[32];
        deq_block(q0, bf16x2_of_f16(sw0 & 0xFFFFu), v);
        deq_block(q1, bf16x2_of_f16(sw0 >> 16), v + 16);
        if (!mbar_wait_parked(a_empty(team, 0), (n & 1) ^ 1)) { if (lane == 0) atomicExch(status, 16); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tmem_st32(ta0, v);
        pending = 0;
        uint32_t w[32];
        deq_block(q2, bf16x2_of_f16(sw1 & 0xFFFFu), w);
        deq_block(q3, bf16x2_of_f16(sw1 >> 16), w + 16);
        publish();                                                          // the first half, while its store had the second half's arithmetic to land behind
        if (!mbar_wait_parked(a_empty(team, 1), (n & 1) ^ 1)) { if (lane == 0) atomicExch(status, 16); ok = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        tmem_st32(ta0 + (uint32_t)A_HALF_COLS, w);
        pending = 1;
      }
    }
    publish();
  } else {
    // ---------------- epilogue warps: TMEM lane quarter (warp % 4), thread = weight row ----------------
    const int quarter = warp & 3;
    const i64 n_pad = (i64)plan.n_tiles * TN;
    bool ok = true;
    pdl_wait();
    const int set = (warp - EPI_WARP0) >> 2;                   // set 0: even local tiles, set 1: odd ones
    for (int local = set; local < ntl && ok; local += 2) {
      const int t = group + local * plan.groups;
      const int n = t * TN + quarter * 32 + lane;
      // the tile's two accumulators: team 0's (its stages local & 1, + 2, ...) and team 1's; a one-stage slice has only the
      // one of team local & 1
      const int acc0 = 2 * set, acc1 = 2 * set + 1;
      const bool has0 = (local & 1) < nstages, has1 = ((local + 1) & 1) < nstages;
      const uint32_t par = (uint32_t)((local >> 1) & 1);
      if (has0 && !mbar_wait_parked(t_full(acc0), par)) { if (lane == 0) atomicExch(status, 17); ok = false; break; }
      if (has1 && !mbar_wait_parked(t_full(acc1), par)) { if (lane == 0) atomicExch(status, 17); ok = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
      const uint32_t taddr = lane_base + (uint32_t)((has0 ? acc0 : acc1) * TM), taddr_b = lane_base + (uint32_t)(acc1 * TM);
      const bool both = has0 && has1;
      float* mine = ws + ((i64)ks * TM) * n_pad + n;
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        uint32_t rr[32];
        tmem_ld32(taddr + h * 32, rr);
        float v[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(rr[e]);
        if (both) {                                             // team 0's sum + team 1's sum, in that order
          tmem_ld16_add(taddr_b + h * 32, v);
          tmem_ld16_add(taddr_b + h * 32 + 16, v + 16);
        }
        if (h == 1) {
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            if (has0) mbar_arrive(t_empty(acc0));
            if (has1) mbar_arrive(t_empty(acc1));
          }
        }
        if (plan.ksplit == 1 && MODE != 3) {
          finish32<MODE>(v, h * 32, M, n, N, out, ldo);
        } else {
          // partial sums go to the workspace as [slice][activation row][weight row]; a separate pass adds the
          // slices in slice order, so the result does not depend on which CTA finished first
          const int mcount = min(32, M - h * 32);
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (e < mcount) __stcg(mine + (i64)(h * 32 + e) * n_pad, v[e]);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 3) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- split-K second pass: out = finish(sum over slices in slice order) ----------------------------------------
// One thread per (activation row, four consecutive weight rows): ksplit independent 16-byte loads, then the same
// finishing as the in-kernel path (MODE 2: two (gate, up) pairs -> two bf16 outputs).
template <int MODE>
__global__ void __launch_bounds__(256) q4_splitk_reduce_kernel(const float* __restrict__ ws, int ksplit, int M, int N, i64 n_pad,
                                                               void* out, i64 ldo) {
  const i64 quads = n_pad >> 2;
  const i64 total = (i64)M * quads;
  pdl_wait();
  pdl_trigger();
  for (i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    const int m = (int)(idx / quads);
    const i64 n0 = (idx % quads) << 2;
    if (n0 >= N) continue;
    const float4* src = reinterpret_cast<const float4*>(ws + (i64)m * n_pad + n0);
    const i64 slice = ((i64)TM * n_pad) >> 2;
    float4 v = __ldcg(src);
    for (int s0 = 1; s0 < ksplit; s0 += 4) {
      float4 p[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (s0 + j < ksplit) p[j] = __ldcg(src + (i64)(s0 + j) * slice);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (s0 + j < ksplit) { v.x = fadd(v.x, p[j].x); v.y = fadd(v.y, p[j].y); v.z = fadd(v.z, p[j].z); v.w = fadd(v.w, p[j].w); }
    }
    if (MODE == 2) {
      const float y0 = fmul(silu1(v.x), v.y), y1 = fmul(silu1(v.z), v.w);
      u16* o = reinterpret_cast<u16*>(out) + (i64)m * ldo + (n0 >> 1);
      o[0] = f32_to_bf16_bits(y0);
      if (n0 + 2 < N) o[1] = f32_to_bf16_bits(y1);
    } else {
      const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (n0 + j < N) {
          if (MODE == 1) reinterpret_cast<u16*>(out)[(i64)m * ldo + n0 + j] = f32_to_bf16_bits(vv[j]);
          else reinterpret_cast<float*>(out)[(i64)m * ldo + n0 + j] = vv[j];
        }
      }
    }
  }
}

// ---- resident layout: raw Q4_0 rows -> [tile of 128 rows][stage of 256 K][18 KB stage image] -----------------------
// A stage image is what the kernel wants in shared memory: 128 rows x 128 B of nibbles with the 16-byte block chunks
// already XOR-swizzled by (row & 7), then 128 rows x 8 f16 scales.  Rows past N and blocks past K are zero (scale 0).
__global__ void __launch_bounds__(256) q4_tile_kernel(const u8* __restrict__ raw, i64 n, i64 nb, i64 n_tiles, i64 kstages,
                                                      u8* __restrict__ out) {
  const i64 total = n_tiles * kstages * TN * 8;
  for (i64 idx = (i64)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (i64)gridDim.x * blockDim.x) {
    const int b = (int)(idx & 7), r = (int)((idx >> 3) & (TN - 1));
    const i64 ts = idx >> 10, s = ts % kstages, t = ts / kstages;
    const i64 row = t * TN + r, kb = s * 8 + b;
    u8* img = out + ts * RAW_STAGE_BYTES;
    u8* qdst = img + r * 128 + ((b ^ (r & 7)) << 4);
    u8* ddst = img + RAW_BYTES + r * 16 + b * 2;
    if (row < n && kb < nb) {
      const u8* src = raw + (row * nb + kb) * 18;
      ddst[0] = src[0]; ddst[1] = src[1];
#pragma unroll
      for (int j = 0; j < 16; ++j) qdst[j] = src[2 + j];
    } else {
      ddst[0] = 0; ddst[1] = 0;
#pragma unroll
      for (int j = 0; j < 16; ++j) qdst[j] = 0;
    }
  }
}

static int encode_x(CUtensorMap* map, const void* ptr, i64 k, i64 rows, i64 ldx) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return (int)cudaErrorNotSupported;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ldx * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)TM};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

}  // namespace q4tc
}  // namespace wkb

using namespace wkb;

extern "C" {

int64_t wkb_q4_tiled_bytes(int64_t n, int64_t k) {
  if (n <= 0 || k <= 0) return 0;
  return ((n + q4tc::TN - 1) / q4tc::TN) * ((k + q4tc::STAGE_K - 1) / q4tc::STAGE_K) * q4tc::RAW_STAGE_BYTES;
}

int wkb_q4_tile(const uint8_t* raw, int64_t n, int64_t k, void* tiled, void* stream) {
  if (n <= 0 || k <= 0) return 0;
  if (k % 32 != 0 || (((uintptr_t)tiled) & 15)) return (int)cudaErrorInvalidValue;
  const i64 n_tiles = (n + q4tc::TN - 1) / q4tc::TN, kstages = (k + q4tc::STAGE_K - 1) / q4tc::STAGE_K;
  const i64 total = n_tiles * kstages * q4tc::TN * 8;
  i64 grid = (total + 255) / 256;
  if (grid > gemm_sm_count() * 32) grid = gemm_sm_count() * 32;
  q4tc::q4_tile_kernel<<<(int)grid, 256, 0, as_stream(stream)>>>(raw, n, k / 32, n_tiles, kstages, (u8*)tiled);
  return (int)cudaGetLastError();
}

int64_t wkb_gemm_q4_0_workspace_bytes(int64_t n, int64_t k) {
  if (n <= 0 || k <= 0) return 256;
  q4tc::Plan p = q4tc::make_plan(n, k, gemm_sm_count());
  return (i64)p.ksplit * q4tc::TM * p.n_tiles * q4tc::TN * 4;   // one slice is the least: out_mode 3 always goes through it
}

void wkb_gemm_q4_0_partial_layout(int64_t n, int64_t k, int64_t* slices, int64_t* slice_stride, int64_t* ld) {
  q4tc::Plan p = q4tc::make_plan(n, k, gemm_sm_count());
  *slices = p.ksplit;
  *ld = (i64)p.n_tiles * q4tc::TN;
  *slice_stride = (i64)q4tc::TM * (*ld);
}

int wkb_gemm_q4_0_bf16_nt(const void* w_tiled, const void* x_bf16, int64_t ldx, void* out, int64_t ldo, int out_mode,
                          int64_t m, int64_t n, int64_t k, void* workspace, int64_t workspace_bytes, void* stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k <= 0 || k % 32 != 0 || ldx % 8 != 0) return (int)cudaErrorInvalidValue;
  if (out_mode < 0 || out_mode > 3 || (out_mode == 2 && (n & 1)) || (out_mode == 3 && m > q4tc::TM)) return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)w_tiled) | ((uintptr_t)x_bf16) | ((uintptr_t)workspace)) & 15) return (int)cudaErrorMisalignedAddress;
  if (!workspace || workspace_bytes < wkb_gemm_q4_0_workspace_bytes(n, k)) return (int)cudaErrorInvalidValue;
  int* status = gemm_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  q4tc::Plan plan = q4tc::make_plan(n, k, gemm_sm_count());
  typedef void (*KernelFn)(const CUtensorMap, const uint8_t*, void*, i64, int, int, q4tc::Plan, float*, int*);
  static const KernelFn table[4] = {q4tc::gemm_q4_tc_kernel<0>, q4tc::gemm_q4_tc_kernel<1>, q4tc::gemm_q4_tc_kernel<2>,
                                    q4tc::gemm_q4_tc_kernel<3>};
  static bool attr_set[64][4] = {{false}};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev][out_mode]) {
    cudaError_t e = cudaFuncSetAttribute(table[out_mode], cudaFuncAttributeMaxDynamicSharedMemorySize, q4tc::SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set[dev][out_mode] = true;
  }
  float* ws = reinterpret_cast<float*>(workspace);
  const i64 n_pad = (i64)plan.n_tiles * q4tc::TN;
  const int esz = out_mode == 0 ? 4 : 2;
  for (i64 m0 = 0; m0 < m; m0 += q4tc::TM) {
    const i64 mc = m - m0 < q4tc::TM ? m - m0 : q4tc::TM;
    CUtensorMap mx;
    int rc = q4tc::encode_x(&mx, (const u16*)x_bf16 + m0 * ldx, k, mc, ldx);
    if (rc) return rc;
    void* o = reinterpret_cast<uint8_t*>(out) + m0 * ldo * esz;
    cudaError_t e = launch_pdl(table[out_mode], plan.ksplit * plan.groups, q4tc::THREADS, (size_t)q4tc::SMEM, as_stream(stream), mx,
                               (const uint8_t*)w_tiled, o, ldo, (int)mc, (int)n, plan, ws, status);
    if (e != cudaSuccess) return (int)e;
    if (plan.ksplit > 1 && out_mode != 3) {
      const i64 total = mc * (n_pad >> 2);
      i64 grid = (total + 255) / 256;
      if (grid > gemm_sm_count() * 8) grid = gemm_sm_count() * 8;
      const float* cws = ws;
      if (out_mode == 0) e = launch_pdl(q4tc::q4_splitk_reduce_kernel<0>, (int)grid, 256, 0, as_stream(stream), cws, plan.ksplit, (int)mc, (int)n, n_pad, o, ldo);
      else if (out_mode == 1) e = launch_pdl(q4tc::q4_splitk_reduce_kernel<1>, (int)grid, 256, 0, as_stream(stream), cws, plan.ksplit, (int)mc, (int)n, n_pad, o, ldo);
      else e = launch_pdl(q4tc::q4_splitk_reduce_kernel<2>, (int)grid, 256, 0, as_stream(stream), cws, plan.ksplit, (int)mc, (int)n, n_pad, o, ldo);
      if (e != cudaSuccess) return (int)e;
    }
  }
  return 0;
}

}  // extern "C"

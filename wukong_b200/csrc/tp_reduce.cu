// Tensor-parallel sum over ranks fused with the residual add and RMSNorm that follow it, over peer memory.
//
// In the tensor-parallel Llama-shape block every rank ends its attention and its MLP with an fp32 [rows, d]
// partial that must be summed over the ranks (the all-reduce of crates/wukong_codegen_gpu/src/serving.rs:4161-4240)
// before `x += sum; xn = rmsnorm(x)`.  With NCCL that is a collective plus a norm kernel, and the collective cannot
// be part of the step's CUDA graph.  Here it is ONE kernel per rank:
//   1. block 0 publishes "my partial is complete" to every peer (a release store of the step's sequence number
//      into the peer's flag row; the partial was written by the preceding GEMM on the same stream);
//   2. every block waits (acquire loads, bounded) until all peers have published this sequence number;
//   3. a block then owns rows: it reads the row of every rank's partial -- plain loads through the peer mappings,
//      over NVLink -- adds them in rank order (so all ranks compute bit-identical sums and the replicated residual
//      stream stays identical), adds the residual, computes the RMS statistic and writes x and the bf16 normed row
//      (the row stays in registers between the statistic and the write-back).
// Buffers: each rank owns two partial buffers (attention, MLP) used alternately; a rank can run at most one phase
// ahead of its slowest peer (it cannot pass a phase without that peer's flag), so a partial buffer is never
// rewritten while a peer may still read it.  Sequence numbers come from a per-rank device step counter plus the
// phase index baked into the launch, so the launches can live in a CUDA graph.
// Peer memory is mapped with CUDA IPC (no multicast objects); loads are plain ld.global, never TMA.
// Waits are bounded (one second unless wkb_tp_set_wait_limit_ms says otherwise): on expiry the block records 21 in
// `status`, skips the sum (x and out are left untouched) and returns.  The rank that gave up also marks itself dead --
// a poison value in its own flag row and in its slot of every peer's -- so every later phase on every rank ends at once
// with code 22 instead of summing a buffer whose owner has moved on; the flag rows must be zeroed to start again.
#include "common.cuh"
#include "wkb_device.h"
#include <cstring>
#include <cuda.h>

namespace wkb {
int* gemm_status_word();

constexpr int TP_MAX_WORLD = 8;
constexpr uint32_t TP_POISON = 0xFFFFFFFFu;    // a sequence number no step reaches: "this rank gave up"
static unsigned long long g_tp_wait_ns = 1000000000ull;   // flag-wait limit, set by wkb_tp_set_wait_limit_ms

struct TpPeers {
  const float* part[TP_MAX_WORLD];   // every rank's partial buffer for this phase (own entry included), by rank
  uint32_t* flags[TP_MAX_WORLD];     // every rank's flag row: flags[r][sender] = last sequence number published
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

template <int NV>
__global__ void __launch_bounds__(1024) tp_reduce_add_rmsnorm_kernel(TpPeers peers, int rank, int world, const uint32_t* __restrict__ step_ptr,
                                                                    int phase, int phases_per_step, float* __restrict__ x,
                                                                    const float* __restrict__ gamma, u16* __restrict__ out, int rows,
                                                                    int cols, float eps, int* status, unsigned long long wait_ns) {
  __shared__ float red[32];
  __shared__ int s_ok;
  // a programmatic dependent of the GEMM that writes this rank's partial: nothing is read or published before that kernel
  // has completed
  pdl_wait();
  pdl_trigger();
  const uint32_t seq = (*step_ptr) * (uint32_t)phases_per_step + (uint32_t)phase + 1u;
  // slot [rank] of a rank's own flag row is its "gave up" mark
  const bool dead = ld_acquire_sys(peers.flags[rank] + rank) == TP_POISON;
  if (blockIdx.x == 0 && threadIdx.x < world && (int)threadIdx.x != rank) {
    __threadfence_system();
    st_release_sys(peers.flags[threadIdx.x] + rank, dead ? TP_POISON : seq);
  }
  if (threadIdx.x == 0) {
    int code = dead ? 22 : 0;
    unsigned long long t_begin;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_begin));
    // two limits: the clock, and a poll count in case the clock does not move
    const unsigned long long max_polls = wait_ns / 64 + 1024;
    for (int p = 0; p < world && !code; ++p) {
      if (p == rank) continue;
      const uint32_t* f = peers.flags[rank] + p;
      unsigned long long it = 0;
      for (;;) {
        const uint32_t v = ld_acquire_sys(f);
        if (v == TP_POISON) { code = 22; break; }        // that peer gave up earlier
        // sequence numbers only grow; a peer one phase ahead has already published a larger one
        if ((int32_t)(v - seq) >= 0) break;
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (now - t_begin > wait_ns || ++it > max_polls) { code = 21; break; }
        __nanosleep(200);
      }
    }
    if (code) atomicExch(status, code);
    if (code == 21) {
      // tell everyone, and remember it: this rank no longer takes part
      st_release_sys(peers.flags[rank] + rank, TP_POISON);
      for (int p = 0; p < world; ++p)
        if (p != rank) st_release_sys(peers.flags[p] + rank, TP_POISON);
    }
    s_ok = code == 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const int nvec = cols >> 2, nwarps = blockDim.x >> 5;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    float4* xr = reinterpret_cast<float4*>(x + (i64)r * cols);
    float4 v[NV];
    float q = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < nvec) {
        // every rank's piece is requested before the first add: one trip over NVLink, not one per rank (a loop over a
        // run-time rank count issues each load behind the previous add); the adds stay in rank order
        float4 d[TP_MAX_WORLD];
#pragma unroll
        for (int p = 0; p < TP_MAX_WORLD; ++p)
          if (p < world) d[p] = __ldcg(reinterpret_cast<const float4*>(peers.part[p] + (i64)r * cols) + i);
        float4 s = d[0];
#pragma unroll
        for (int p = 1; p < TP_MAX_WORLD; ++p)
          if (p < world) { s.x += d[p].x; s.y += d[p].y; s.z += d[p].z; s.w += d[p].w; }
        v[k] = xr[i];
        v[k].x += s.x; v[k].y += s.y; v[k].z += s.z; v[k].w += s.w;
        q = fmaf(v[k].x, v[k].x, q); q = fmaf(v[k].y, v[k].y, q); q = fmaf(v[k].z, v[k].z, q); q = fmaf(v[k].w, v[k].w, q);
      }
    }
    q = warp_sum(q);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = q;
    __syncthreads();
    float tot = 0.0f;
    for (int w = 0; w < nwarps; ++w) tot += red[w];
    const float inv = rsqrtf(tot / (float)cols + eps);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      if (i < nvec) {
        xr[i] = v[k];
        const float4 g = gamma ? reinterpret_cast<const float4*>(gamma)[i] : make_float4(1.f, 1.f, 1.f, 1.f);
        uint2 o;
        o.x = (uint32_t)f32_to_bf16_bits(v[k].x * inv * g.x) | ((uint32_t)f32_to_bf16_bits(v[k].y * inv * g.y) << 16);
        o.y = (uint32_t)f32_to_bf16_bits(v[k].z * inv * g.z) | ((uint32_t)f32_to_bf16_bits(v[k].w * inv * g.w) << 16);
        reinterpret_cast<uint2*>(out + (i64)r * cols)[i] = o;
      }
    }
  }
}

__global__ void tp_step_bump_kernel(uint32_t* step_ptr) { *step_ptr += 1u; }

}  // namespace wkb

using namespace wkb;

extern "C" {

// Export the allocation that contains `p`: the handle names the whole allocation, *offset is where p sits in it
// (memory handed out by a caching allocator is usually an interior pointer of a larger cudaMalloc block).
int wkb_ipc_export(void* p, void* handle64, i64* offset) {
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn range = nullptr;
  if (!range) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess)
      return (int)cudaErrorNotSupported;
    range = (RangeFn)fn;
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  if (range(&base, &size, (CUdeviceptr)p) != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, (void*)base);
  if (e != cudaSuccess) return (int)e;
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  *offset = (i64)((CUdeviceptr)p - base);
  return 0;
}
void* wkb_ipc_import(const void* handle64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return nullptr;
  return p;
}
int wkb_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

int wkb_tp_reduce_add_rmsnorm(const void* const* parts, void* const* flags, i64 rank, i64 world, const void* step_ptr, i64 phase,
                              i64 phases_per_step, float* x, const float* gamma_or_null, void* out_bf16, i64 rows, i64 cols, float eps,
                              void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (world < 1 || world > TP_MAX_WORLD || rank < 0 || rank >= world || cols % 4 != 0) return (int)cudaErrorInvalidValue;
  int* status = gemm_status_word();
  if (!status) return (int)cudaErrorMemoryAllocation;
  TpPeers peers;
  for (int p = 0; p < TP_MAX_WORLD; ++p) {
    peers.part[p] = p < world ? (const float*)parts[p] : nullptr;
    peers.flags[p] = p < world ? (uint32_t*)flags[p] : nullptr;
  }
  const int grid = (int)(rows < (i64)WKB_SM_COUNT ? rows : (i64)WKB_SM_COUNT);
  const i64 nvec = cols / 4;
  const int threads = (int)(((nvec < 1024 ? nvec : 1024) + 31) / 32 * 32);   // the thread layout (and with it the order of the row's sum of
                                                                            // squares) is the one of add_rmsnorm_kernel: the two paths agree bit for bit
  const i64 per = (nvec + threads - 1) / threads;
  cudaStream_t st = as_stream(stream);
#define WKB_TP_LAUNCH(NV_) launch_pdl(tp_reduce_add_rmsnorm_kernel<NV_>, grid, threads, 0, st, peers, (int)rank, (int)world, (const uint32_t*)step_ptr, \
    (int)phase, (int)phases_per_step, x, gamma_or_null, (u16*)out_bf16, (int)rows, (int)cols, eps, status, g_tp_wait_ns)
  if (per <= 1) WKB_TP_LAUNCH(1);
  else if (per <= 2) WKB_TP_LAUNCH(2);
  else if (per <= 4) WKB_TP_LAUNCH(4);
  else if (per <= 8) WKB_TP_LAUNCH(8);
  else return (int)cudaErrorInvalidValue;
#undef WKB_TP_LAUNCH
  return (int)cudaGetLastError();
}

// Limit of the flag wait of wkb_tp_reduce_add_rmsnorm launches made after this call (process-wide; <= 0 restores the
// default of one second).
void wkb_tp_set_wait_limit_ms(i64 ms) { g_tp_wait_ns = ms > 0 ? (unsigned long long)ms * 1000000ull : 1000000000ull; }

int wkb_tp_step_bump(void* step_ptr, void* stream) {
  tp_step_bump_kernel<<<1, 1, 0, as_stream(stream)>>>((uint32_t*)step_ptr);
  return (int)cudaGetLastError();
}

}  // extern "C"

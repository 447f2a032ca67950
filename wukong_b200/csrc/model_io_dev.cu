// Checkpoint tensors straight into device memory.
//
// wkb_gguf_read_device / wkb_st_read_device take the arguments of the host readers `wukong_rt_gguf_read` /
// `wukong_rt_st_read` (crates/wukong_runtime/src/gguf.rs:809-851, crates/wukong_runtime/src/safetensors.rs:379-407)
// with a DEVICE destination.  Every check runs first, in the same order with the same codes; then the payload
// crosses PCIe as the file's own bytes -- 18 B per 32 weights for Q4_0 instead of 128 B of f32 -- through two
// pinned staging buffers, and a kernel dequantizes (or widens) each chunk on the GPU while the next one is read.
// The device arithmetic is ggml's reference dequantization in f32 with every product and sum rounded once, so
// the values are bit-identical to the host reader's.
#include "common.cuh"
#include "model_io.h"

#include <algorithm>
#include <cstdio>
#include <mutex>

namespace wkb_io {

__device__ __forceinline__ float dev_half(const u8* b, int at) {
  return __half2float(__ushort_as_half((unsigned short)(b[at] | (unsigned)b[at + 1] << 8)));
}
__constant__ int8_t c_iq4nl[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

__device__ __forceinline__ void dev_scale_min_k4(int j, const u8* q, int* sc, int* mn) {
  if (j < 4) {
    *sc = q[j] & 63;
    *mn = q[j + 4] & 63;
  } else {
    *sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    *mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// Element e of one block of ggml type ID.
template <int ID>
__device__ __forceinline__ float dequant_elem(const u8* blk, int e) {
  using wkb::fadd;
  using wkb::fmul;
  using wkb::fsub;
  if constexpr (ID == 2) {            // Q4_0
    const u8 q = blk[2 + (e & 15)];
    return fmul((float)((int)(e < 16 ? (q & 0xF) : (q >> 4)) - 8), dev_half(blk, 0));
  } else if constexpr (ID == 3) {     // Q4_1
    const u8 q = blk[4 + (e & 15)];
    return fadd(fmul((float)(e < 16 ? (q & 0xF) : (q >> 4)), dev_half(blk, 0)), dev_half(blk, 2));
  } else if constexpr (ID == 6 || ID == 7) {   // Q5_0 / Q5_1
    constexpr int h = ID == 7 ? 4 : 2;
    const uint32_t qh = (uint32_t)blk[h] | (uint32_t)blk[h + 1] << 8 | (uint32_t)blk[h + 2] << 16 | (uint32_t)blk[h + 3] << 24;
    const u8 q = blk[h + 4 + (e & 15)];
    const int x = (int)(e < 16 ? (q & 0xF) : (q >> 4)) | (int)(((qh >> e) & 1u) << 4);
    if constexpr (ID == 7) return fadd(fmul((float)x, dev_half(blk, 0)), dev_half(blk, 2));
    else return fmul((float)(x - 16), dev_half(blk, 0));
  } else if constexpr (ID == 8) {     // Q8_0
    return fmul((float)(int8_t)blk[2 + e], dev_half(blk, 0));
  } else if constexpr (ID == 10 || ID == 11) {   // Q2_K / Q3_K share the element order
    const int n = e >> 7, r = e & 127, sh = r >> 5, h16 = (r & 31) >> 4, l = r & 15;
    const int is = n * 8 + sh * 2 + h16, at = l + 16 * h16;
    if constexpr (ID == 10) {
      const u8 sc = blk[is];
      const int v = (blk[16 + n * 32 + at] >> (2 * sh)) & 3;
      const float dl = fmul(dev_half(blk, 80), (float)(sc & 0xF)), ml = fmul(dev_half(blk, 82), (float)(sc >> 4));
      return fsub(fmul(dl, (float)v), ml);
    } else {
      const u8* sr = blk + 96;
      const int low = is < 8 ? (sr[is] & 0xF) : (sr[is - 8] >> 4);
      const int high = (sr[8 + is % 4] >> (2 * (is / 4))) & 3;
      const int s = (low | (high << 4)) - 32;
      const int m = 1 << (n * 4 + sh);
      const int v = (int)((blk[32 + n * 32 + at] >> (2 * sh)) & 3) - ((blk[at] & m) ? 0 : 4);
      return fmul(fmul(dev_half(blk, 108), (float)s), (float)v);
    }
  } else if constexpr (ID == 12 || ID == 13) {   // Q4_K / Q5_K
    const int c = e >> 6, hi = (e >> 5) & 1, l = e & 31;
    int sc, mn;
    dev_scale_min_k4(2 * c + hi, blk + 4, &sc, &mn);
    const u8 q = blk[(ID == 13 ? 48 : 16) + c * 32 + l];
    int v = hi ? (q >> 4) : (q & 0xF);
    if constexpr (ID == 13) v += (blk[16 + l] & ((hi ? 2 : 1) << (2 * c))) ? 16 : 0;
    const float d1 = fmul(dev_half(blk, 0), (float)sc), m1 = fmul(dev_half(blk, 2), (float)mn);
    return fsub(fmul(d1, (float)v), m1);
  } else if constexpr (ID == 14) {    // Q6_K
    const int n = e >> 7, r = e & 127, grp = r >> 5, l = r & 31;
    const u8 lowb = blk[n * 64 + l + 32 * (grp & 1)];
    const int q = (int)((grp >= 2 ? (lowb >> 4) : (lowb & 0xF)) | (((blk[128 + n * 32 + l] >> (2 * grp)) & 3) << 4)) - 32;
    const int sc = (int8_t)blk[192 + n * 8 + (l >> 4) + 2 * grp];
    return fmul(fmul(dev_half(blk, 208), (float)sc), (float)q);
  } else if constexpr (ID == 15) {    // Q8_K
    const uint32_t u = (uint32_t)blk[0] | (uint32_t)blk[1] << 8 | (uint32_t)blk[2] << 16 | (uint32_t)blk[3] << 24;
    return fmul(__uint_as_float(u), (float)(int8_t)blk[4 + e]);
  } else if constexpr (ID == 20) {    // IQ4_NL
    const u8 q = blk[2 + (e & 15)];
    return fmul(dev_half(blk, 0), (float)c_iq4nl[e < 16 ? (q & 0xF) : (q >> 4)]);
  } else {                            // IQ4_XS (23)
    const int ib = e >> 5, j = e & 31;
    const uint32_t scales_h = (uint32_t)blk[2] | (uint32_t)blk[3] << 8;
    const int lo = (blk[4 + ib / 2] >> (4 * (ib & 1))) & 0xF, hi = (int)((scales_h >> (2 * ib)) & 3);
    const float dl = fmul(dev_half(blk, 0), (float)((lo | (hi << 4)) - 32));
    const u8 q = blk[8 + ib * 16 + (j & 15)];
    return fmul(dl, (float)c_iq4nl[j < 16 ? (q & 0xF) : (q >> 4)]);
  }
}

// One thread per output element: consecutive threads write consecutive f32 (coalesced); the block bytes they
// share are served from L1.
template <int ID, int BLOCK, int BYTES>
__global__ void __launch_bounds__(256) dequant_blocks_kernel(const u8* __restrict__ raw, float* __restrict__ out, i64 elems) {
  for (i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x; t < elems; t += (i64)gridDim.x * blockDim.x)
    out[t] = dequant_elem<ID>(raw + (t / BLOCK) * BYTES, (int)(t % BLOCK));
}

__global__ void __launch_bounds__(256) widen_half_kernel(const u16* __restrict__ src, float* __restrict__ out, i64 elems, int is_bf16) {
  for (i64 t = (i64)blockIdx.x * blockDim.x + threadIdx.x; t < elems; t += (i64)gridDim.x * blockDim.x) {
    const u16 h = src[t];
    out[t] = is_bf16 ? __uint_as_float((uint32_t)h << 16) : __half2float(__ushort_as_half(h));
  }
}

static int grid_for(i64 elems) {
  const i64 want = (elems + 255) / 256;
  const i64 cap = (i64)WKB_SM_COUNT * 8;
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

static cudaError_t launch_dequant(uint32_t id, const u8* raw, float* out, i64 elems, cudaStream_t st) {
  const int g = grid_for(elems);
  switch (id) {
#define WKB_DQ(ID_, BLOCK_, BYTES_) case ID_: dequant_blocks_kernel<ID_, BLOCK_, BYTES_><<<g, 256, 0, st>>>(raw, out, elems); break
    WKB_DQ(2, 32, 18); WKB_DQ(3, 32, 20); WKB_DQ(6, 32, 22); WKB_DQ(7, 32, 24); WKB_DQ(8, 32, 34);
    WKB_DQ(10, 256, 84); WKB_DQ(11, 256, 110); WKB_DQ(12, 256, 144); WKB_DQ(13, 256, 176); WKB_DQ(14, 256, 210);
    WKB_DQ(15, 256, 292); WKB_DQ(20, 32, 18); WKB_DQ(23, 256, 136);
#undef WKB_DQ
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

// Two pinned host buffers and two device staging buffers, made on first use and kept for the process.
struct Staging {
  static constexpr size_t CHUNK = 16u << 20;
  std::mutex mu;
  u8* host[2] = {nullptr, nullptr};
  u8* dev[2] = {nullptr, nullptr};
  cudaEvent_t done[2] = {nullptr, nullptr};
  int device = -1;

  cudaError_t ready() {
    int cur = 0;
    cudaError_t e = cudaGetDevice(&cur);
    if (e != cudaSuccess) return e;
    if (device == cur) return cudaSuccess;
    release();
    for (int s = 0; s < 2; ++s) {
      if ((e = cudaHostAlloc((void**)&host[s], CHUNK, cudaHostAllocDefault)) != cudaSuccess) return e;
      if ((e = cudaMalloc((void**)&dev[s], CHUNK)) != cudaSuccess) return e;
      if ((e = cudaEventCreateWithFlags(&done[s], cudaEventDisableTiming)) != cudaSuccess) return e;
    }
    device = cur;
    return cudaSuccess;
  }
  void release() {
    for (int s = 0; s < 2; ++s) {
      if (done[s]) { cudaEventSynchronize(done[s]); cudaEventDestroy(done[s]); done[s] = nullptr; }
      if (host[s]) { cudaFreeHost(host[s]); host[s] = nullptr; }
      if (dev[s]) { cudaFree(dev[s]); dev[s] = nullptr; }
    }
    device = -1;
  }
};
static Staging g_staging;

// Stream the located payload to the device; the destination is written in stream order.
static int64_t transfer_device(const char* path, const Located& loc, void* dev_out, cudaStream_t st) {
  if (loc.count == 0) return 0;
  std::lock_guard<std::mutex> lock(g_staging.mu);
  if (g_staging.ready() != cudaSuccess) return IO_ERROR;
  FILE* f = fopen(path, "rb");
  if (!f) return IO_ERROR;
  int64_t rc = 0;
  if (fseeko(f, (off_t)loc.data_off, SEEK_SET) != 0) rc = IO_ERROR;
  const GgmlType* ty = loc.move == Move::Dequant ? ggml_type(loc.ggml_id) : nullptr;
  // bytes of payload and elements of output per unit that may not be split over two chunks
  const uint64_t unit_bytes = ty ? ty->bytes : (loc.move == Move::Widen ? 2 : 1);
  const uint64_t unit_elems = ty ? ty->block : 1;
  const uint64_t total_bytes = loc.move == Move::Verbatim ? loc.count * (uint64_t)dtype_size(loc.src_dt)
                               : loc.move == Move::Raw    ? loc.count
                                                          : loc.count / unit_elems * unit_bytes;
  const uint64_t chunk_bytes = Staging::CHUNK / unit_bytes * unit_bytes;
  uint64_t done_bytes = 0;
  for (int slot = 0; rc == 0 && done_bytes < total_bytes; slot ^= 1) {
    const uint64_t m = std::min<uint64_t>(chunk_bytes, total_bytes - done_bytes);
    if (cudaEventSynchronize(g_staging.done[slot]) != cudaSuccess) { rc = IO_ERROR; break; }   // the slot's last copy and kernel
    if (fread(g_staging.host[slot], 1, m, f) != m) { rc = IO_ERROR; break; }
    cudaError_t e;
    if (loc.move == Move::Verbatim || loc.move == Move::Raw) {
      e = cudaMemcpyAsync(static_cast<u8*>(dev_out) + done_bytes, g_staging.host[slot], m, cudaMemcpyHostToDevice, st);
    } else {
      e = cudaMemcpyAsync(g_staging.dev[slot], g_staging.host[slot], m, cudaMemcpyHostToDevice, st);
      float* out = static_cast<float*>(dev_out) + done_bytes / unit_bytes * unit_elems;
      const i64 elems = (i64)(m / unit_bytes * unit_elems);
      if (e == cudaSuccess) {
        if (ty) e = launch_dequant(ty->id, g_staging.dev[slot], out, elems, st);
        else {
          widen_half_kernel<<<grid_for(elems), 256, 0, st>>>((const u16*)g_staging.dev[slot], out, elems, loc.src_dt == DT_BF16);
          e = cudaGetLastError();
        }
      }
    }
    if (e == cudaSuccess) e = cudaEventRecord(g_staging.done[slot], st);
    if (e != cudaSuccess) rc = IO_ERROR;
    done_bytes += m;
  }
  fclose(f);
  return rc;
}

}  // namespace wkb_io

using namespace wkb_io;

extern "C" {

// Dequantize `blocks` blocks of ggml type `ggml_type_id` that already sit in device memory.
int wkb_ggml_dequant_f32(int64_t ggml_type_id, const void* raw_dev, int64_t blocks, float* out_dev, void* stream) {
  const GgmlType* ty = ggml_type_id >= 0 ? ggml_type((uint32_t)ggml_type_id) : nullptr;
  if (!ty || !ty->dequant || blocks < 0) return (int)cudaErrorInvalidValue;
  if (blocks == 0) return 0;
  return (int)launch_dequant(ty->id, static_cast<const u8*>(raw_dev), out_dev, blocks * (i64)ty->block, wkb::as_stream(stream));
}

int64_t wkb_gguf_read_device(const char* path, const char* name, void* dev_data, int64_t len, int64_t dtype, const int64_t* dims,
                             int64_t rank, void* stream) {
  Located loc;
  if (const int64_t rc = gguf_locate_for(path, name, dtype, len, dims, rank, &loc)) return rc;
  if (const int64_t rc = transfer_device(path, loc, dev_data, wkb::as_stream(stream))) return rc;
  return (int64_t)loc.count;
}

int64_t wkb_st_read_device(const char* path, const char* name, void* dev_data, int64_t len, int64_t dtype, const int64_t* dims,
                           int64_t rank, void* stream) {
  Located loc;
  if (const int64_t rc = st_locate_for(path, name, dtype, len, dims, rank, &loc)) return rc;
  if (const int64_t rc = transfer_device(path, loc, dev_data, wkb::as_stream(stream))) return rc;
  return (int64_t)loc.count;
}

}  // extern "C"

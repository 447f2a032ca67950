// The runtime ABI with HOST pointers: the exact `extern "C" wukong_*` symbols, argument meaning and
// status conventions of the reference's kernel library (crates/wukong_runtime; the signature table
// is crates/wukong_codegen_llvm/src/runtime_abi.rs:7-232), executed on the GPU.
//
// Each call validates its shape on the host with the reference's own plan rules (nothing is read or
// written on a refused call), uploads the operands into a per-thread device arena, launches the
// kernel on a per-thread stream, downloads the result and synchronises.  Inputs are snapshotted by
// the upload before any output byte is written back, which gives the "value semantics on overlap"
// the checked entries promise.  There is no CPU compute path: without a usable CUDA device the
// `void` entries abort with a message and the checked entries do the same (a status code cannot
// express "no device").  `_parallel` twins are the same functions: on the device every launch is
// parallel and the results are identical by construction.
#include "common.cuh"
#include "wkb_device.h"
#include <cstring>
#include <vector>

namespace {

// Staging memory and stream of one (host thread, device) pair.
struct Arena {
  char* base = nullptr;
  size_t cap = 0, used = 0;
  cudaStream_t stream = nullptr;
  void begin(size_t need) {
    if (!stream) WKB_CUDA_CHECK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    need += 4096;
    if (need > cap) {
      if (base) WKB_CUDA_CHECK(cudaFree(base));
      size_t ncap = cap ? cap : (size_t)1 << 20;
      while (ncap < need) ncap <<= 1;
      WKB_CUDA_CHECK(cudaMalloc((void**)&base, ncap));
      cap = ncap;
    }
    used = 0;
  }
  void* take(size_t bytes) {
    size_t off = (used + 255) & ~(size_t)255;
    used = off + bytes;
    if (used > cap) { fprintf(stderr, "wukong_b200: staging arena overflow\n"); abort(); }
    return base + off;
  }
  template <typename T> T* up(const T* host, size_t count) {
    if (!host || count == 0) return nullptr;
    T* d = (T*)take(count * sizeof(T));
    WKB_CUDA_CHECK(cudaMemcpyAsync(d, host, count * sizeof(T), cudaMemcpyHostToDevice, stream));
    return d;
  }
  template <typename T> T* out(size_t count) { return (T*)take(count * sizeof(T)); }
  template <typename T> void down(T* host, const T* dev, size_t count) {
    if (count) WKB_CUDA_CHECK(cudaMemcpyAsync(host, dev, count * sizeof(T), cudaMemcpyDeviceToHost, stream));
  }
  void sync() { WKB_CUDA_CHECK(cudaStreamSynchronize(stream)); }
};

// One arena per device for each host thread, kept when the thread switches devices and released at thread exit
// (with the owning device made current for the release).
struct ArenaSet {
  static constexpr int MAX_DEV = 64;
  Arena per_device[MAX_DEV];
  Arena& current() {
    int dev;
    WKB_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEV) { fprintf(stderr, "wukong_b200: device index %d out of range\n", dev); abort(); }
    return per_device[dev];
  }
  ~ArenaSet() {
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) return;   // the runtime is already gone (process exit)
    for (int d = 0; d < MAX_DEV; ++d) {
      Arena& a = per_device[d];
      if (!a.stream && !a.base) continue;
      if (cudaSetDevice(d) != cudaSuccess) continue;
      if (a.stream) { cudaStreamSynchronize(a.stream); cudaStreamDestroy(a.stream); }
      if (a.base) cudaFree(a.base);
    }
    cudaSetDevice(prev);
    cudaGetLastError();
  }
};
thread_local ArenaSet g_arenas;

static inline size_t pad(size_t b) { return (b + 255) & ~(size_t)255; }
static void check_launch(int code, const char* what) {
  if (code != 0) {
    fprintf(stderr, "wukong_b200: %s failed: %s\n", what, cudaGetErrorString((cudaError_t)code));
    abort();
  }
}
static inline bool same_buf(const void* a, const void* b) { return a == b; }

// ---- GEMM family -------------------------------------------------------------------------------
static void gemm_host(const void* a, int adt, const void* b, int bdt, float* c, i64 m, i64 k, i64 n, i64 beta, int at,
                      int bt, const float* bias, i64 act, float alpha, int has_epi) {
  if (m <= 0 || k <= 0 || n <= 0) return;  // gemm.rs:1018-1020: nothing written
  size_t ea = adt == 0 ? 4 : 2, eb = bdt == 0 ? 4 : 2;
  size_t na = (size_t)m * k, nbb = (size_t)k * n, nc = (size_t)m * n;
  Arena& A = g_arenas.current();
  A.begin(pad(na * ea) + pad(nbb * eb) + pad(nc * 4) + pad((size_t)n * 4));
  void* da = A.take(na * ea);
  void* db = A.take(nbb * eb);
  WKB_CUDA_CHECK(cudaMemcpyAsync(da, a, na * ea, cudaMemcpyHostToDevice, A.stream));
  WKB_CUDA_CHECK(cudaMemcpyAsync(db, b, nbb * eb, cudaMemcpyHostToDevice, A.stream));
  float* dc = A.out<float>(nc);
  if (beta != 0) WKB_CUDA_CHECK(cudaMemcpyAsync(dc, c, nc * 4, cudaMemcpyHostToDevice, A.stream));
  float* dbias = A.up(bias, (size_t)n);
  check_launch(wkb_sgemm_contract(da, adt, db, bdt, dc, m, k, n, beta, at, bt, dbias, act, alpha, has_epi, A.stream), "sgemm");
  A.down(c, dc, nc);
  A.sync();
}

static i64 gemv_half_host(const u16* w, i64 nw, const float* x, i64 nx, float* y, i64 ny, int dt) {
  if (nw < 0 || nx < 0 || ny < 0) return -2;            // gemv_half.rs:29-36 (gemv_half_plan)
  if ((__int128)ny * (__int128)nx != (__int128)nw) return -2;
  if (ny == 0) return 0;
  if (nx == 0) { memset(y, 0, (size_t)ny * 4); return 0; }
  Arena& A = g_arenas.current();
  A.begin(pad((size_t)nw * 2) + pad((size_t)nx * 4) + pad((size_t)ny * 4));
  u16* dw = A.up(w, (size_t)nw);
  float* dx = A.up(x, (size_t)nx);
  float* dy = A.out<float>((size_t)ny);
  // y[j] = sum_p x[p] w[j,p]: the M = 1 row of the half NT GEMM with an f32 activation.
  check_launch(wkb_sgemm_contract(dx, 0, dw, dt, dy, 1, nx, ny, 0, 0, 1, nullptr, 0, 1.0f, 0, A.stream), "sgemv_half");
  A.down(y, dy, (size_t)ny);
  A.sync();
  return 0;
}

// ---- quantised family --------------------------------------------------------------------------
static bool q_need(i64 rows, i64 k, i64 bb, i64 have) {
  __int128 v = (__int128)rows * (__int128)((k + 31) / 32) * (__int128)bb;
  return v == (__int128)have;
}

static i64 gemv_q_host(const u8* w, i64 nw, const float* x, i64 nx, float* y, i64 ny, int q4) {
  if (nw < 0 || nx < 0 || ny < 0) return -2;  // quant.rs:113-130
  i64 bb = q4 ? 18 : 34;
  if (!q_need(ny, nx, bb, nw)) return -2;
  if (ny == 0) return 0;
  if (nx == 0) { memset(y, 0, (size_t)ny * 4); return 0; }
  i64 nb = (nx + 31) / 32, nblocks = ny * nb;
  Arena& A = g_arenas.current();
  size_t qb = (size_t)nblocks * (bb - 2);
  A.begin(pad((size_t)nw) + pad(qb) + pad((size_t)nblocks * 2) + pad((size_t)nx * 4) + pad((size_t)nb * 32) +
          2 * pad((size_t)nb * 4) + pad((size_t)ny * 4));
  u8* draw = A.up(w, (size_t)nw);
  void* dqs = A.take(qb);
  void* dd = A.take((size_t)nblocks * 2);
  float* dxf = A.up(x, (size_t)nx);
  void* dxq = A.take((size_t)nb * 32);
  float* ddx = A.out<float>((size_t)nb);
  int* dsx = A.out<int>((size_t)nb);
  float* dy = A.out<float>((size_t)ny);
  check_launch(wkb_q_split(draw, dqs, dd, nblocks, q4, A.stream), "q_split");
  check_launch(wkb_quantize_act(dxf, nx, dxq, ddx, dsx, A.stream), "quantize_act");
  check_launch(wkb_gemv_q_contract(dqs, dd, dxq, ddx, dsx, dy, ny, nx, q4, A.stream), "gemv_q");
  A.down(y, dy, (size_t)ny);
  A.sync();
  return 0;
}

static i64 quantize_host(const float* x, i64 nx, u8* q, i64 nq, i64 k, int q4) {
  if (nx < 0 || nq < 0 || k <= 0) return -2;  // quant.rs:93-109
  if (nx % k != 0) return -2;
  i64 rows = nx / k;
  if (!q_need(rows, k, q4 ? 18 : 34, nq)) return -2;
  if (rows == 0) return 0;
  Arena& A = g_arenas.current();
  A.begin(pad((size_t)nx * 4) + pad((size_t)nq));
  float* dx = A.up(x, (size_t)nx);
  u8* dq = A.out<u8>((size_t)nq);
  check_launch(wkb_quantize_q(dx, dq, rows, k, q4, A.stream), "quantize");
  A.down(q, dq, (size_t)nq);
  A.sync();
  return 0;
}

static i64 dequant_int4_host(const u8* q, i64 nq, const float* scale, i64 ns, const float* zero, i64 nz, i64 group,
                             float* out, i64 nout) {
  if (nq < 0 || ns < 0 || nout < 0 || group < 1) return -2;  // quant.rs:628-647
  uint64_t n = (uint64_t)nout, g = (uint64_t)group, groups = (n + g - 1) / g;
  if ((uint64_t)nq != (n + 1) / 2 || (uint64_t)ns != groups || (nz >= 0 && (uint64_t)nz != groups)) return -2;
  if (n == 0) return 0;
  Arena& A = g_arenas.current();
  A.begin(pad((size_t)nq) + 2 * pad((size_t)groups * 4) + pad((size_t)n * 4));
  u8* dq = A.up(q, (size_t)nq);
  float* dsc = A.up(scale, (size_t)groups);
  float* dz = nz >= 0 ? A.up(zero, (size_t)groups) : nullptr;
  float* dout = A.out<float>((size_t)n);
  check_launch(wkb_dequant_int4(dq, dsc, dz, group, dout, (i64)n, A.stream), "dequant_int4");
  A.down(out, dout, (size_t)n);
  A.sync();
  return 0;
}

}  // namespace

extern "C" {

// ---- f32 GEMM (gemm.rs:809-960) ----
void wukong_sgemm(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta) {
  gemm_host(a, 0, b, 0, c, m, k, n, beta, 0, 0, nullptr, 0, 1.0f, 0);
}
void wukong_sgemm_nt(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta) {
  gemm_host(a, 0, b, 0, c, m, k, n, beta, 0, 1, nullptr, 0, 1.0f, 0);
}
void wukong_sgemm_tn(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta) {
  gemm_host(a, 0, b, 0, c, m, k, n, beta, 1, 0, nullptr, 0, 1.0f, 0);
}
void wukong_sgemm_nt_epi(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta, const float* bias,
                         i64 act) {
  gemm_host(a, 0, b, 0, c, m, k, n, beta, 0, 1, bias, act, 1.0f, 1);
}
void wukong_sgemm_nt_alpha(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta, float alpha) {
  gemm_host(a, 0, b, 0, c, m, k, n, beta, 0, 1, nullptr, 0, alpha, 1);
}
void wukong_sgemm_parallel(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta) { wukong_sgemm(a, b, c, m, k, n, beta); }
void wukong_sgemm_nt_parallel(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta) { wukong_sgemm_nt(a, b, c, m, k, n, beta); }
void wukong_sgemm_tn_parallel(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta) { wukong_sgemm_tn(a, b, c, m, k, n, beta); }
void wukong_sgemm_nt_epi_parallel(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta, const float* bias, i64 act) { wukong_sgemm_nt_epi(a, b, c, m, k, n, beta, bias, act); }
void wukong_sgemm_nt_alpha_parallel(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta, float alpha) { wukong_sgemm_nt_alpha(a, b, c, m, k, n, beta, alpha); }

// ---- half-storage GEMM (gemm.rs:1490-1900) ----
void wukong_sgemm_bf16_nt(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta) {
  gemm_host(a, 1, b, 1, c, m, k, n, beta, 0, 1, nullptr, 0, 1.0f, 0);
}
void wukong_sgemm_f16_nt(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta) {
  gemm_host(a, 2, b, 2, c, m, k, n, beta, 0, 1, nullptr, 0, 1.0f, 0);
}
void wukong_sgemm_bf16_nt_epi(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta, const float* bias, i64 act) {
  gemm_host(a, 1, b, 1, c, m, k, n, beta, 0, 1, bias, act, 1.0f, 1);
}
void wukong_sgemm_f16_nt_epi(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta, const float* bias, i64 act) {
  gemm_host(a, 2, b, 2, c, m, k, n, beta, 0, 1, bias, act, 1.0f, 1);
}
void wukong_sgemm_bf16_tn(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta) {
  gemm_host(a, 1, b, 1, c, m, k, n, beta, 1, 0, nullptr, 0, 1.0f, 0);
}
void wukong_sgemm_f16_tn(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta) {
  gemm_host(a, 2, b, 2, c, m, k, n, beta, 1, 0, nullptr, 0, 1.0f, 0);
}
void wukong_sgemm_bf16_nt_parallel(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta) { wukong_sgemm_bf16_nt(a, b, c, m, k, n, beta); }
void wukong_sgemm_f16_nt_parallel(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta) { wukong_sgemm_f16_nt(a, b, c, m, k, n, beta); }
void wukong_sgemm_bf16_nt_epi_parallel(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta, const float* bias, i64 act) { wukong_sgemm_bf16_nt_epi(a, b, c, m, k, n, beta, bias, act); }
void wukong_sgemm_f16_nt_epi_parallel(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta, const float* bias, i64 act) { wukong_sgemm_f16_nt_epi(a, b, c, m, k, n, beta, bias, act); }
void wukong_sgemm_bf16_tn_parallel(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta) { wukong_sgemm_bf16_tn(a, b, c, m, k, n, beta); }
void wukong_sgemm_f16_tn_parallel(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta) { wukong_sgemm_f16_tn(a, b, c, m, k, n, beta); }

// ---- GEMV (gemv.rs:197-326, gemv_half.rs:465-529) ----
void wukong_sgemv_alpha(const float* a, const float* x, float* y, i64 m, i64 n, float alpha) {
  if (m <= 0 || n <= 0) return;
  Arena& A = g_arenas.current();
  A.begin(pad((size_t)m * n * 4) + pad((size_t)n * 4) + pad((size_t)m * 4));
  float* da = A.up(a, (size_t)m * n);
  float* dx = A.up(x, (size_t)n);
  float* dy = A.out<float>((size_t)m);
  check_launch(wkb_sgemv_f32(da, dx, dy, m, n, alpha, A.stream), "sgemv");
  A.down(y, dy, (size_t)m);
  A.sync();
}
void wukong_sgemv(const float* a, const float* x, float* y, i64 m, i64 n) { wukong_sgemv_alpha(a, x, y, m, n, 1.0f); }
void wukong_sgemv_parallel(const float* a, const float* x, float* y, i64 m, i64 n) { wukong_sgemv(a, x, y, m, n); }
void wukong_sgemv_alpha_parallel(const float* a, const float* x, float* y, i64 m, i64 n, float alpha) { wukong_sgemv_alpha(a, x, y, m, n, alpha); }
i64 wukong_sgemv_bf16(const u16* w, i64 nw, const float* x, i64 nx, float* y, i64 ny) { return gemv_half_host(w, nw, x, nx, y, ny, 1); }
i64 wukong_sgemv_f16(const u16* w, i64 nw, const float* x, i64 nx, float* y, i64 ny) { return gemv_half_host(w, nw, x, nx, y, ny, 2); }
i64 wukong_sgemv_bf16_parallel(const u16* w, i64 nw, const float* x, i64 nx, float* y, i64 ny) { return gemv_half_host(w, nw, x, nx, y, ny, 1); }
i64 wukong_sgemv_f16_parallel(const u16* w, i64 nw, const float* x, i64 nx, float* y, i64 ny) { return gemv_half_host(w, nw, x, nx, y, ny, 2); }

// ---- block quantisation (quant.rs:488-800) ----
i64 wukong_quantize_q8_0_f32(const float* x, i64 nx, u8* q, i64 nq, i64 k) { return quantize_host(x, nx, q, nq, k, 0); }
i64 wukong_quantize_q4_0_f32(const float* x, i64 nx, u8* q, i64 nq, i64 k) { return quantize_host(x, nx, q, nq, k, 1); }
i64 wukong_gemv_q8_0_f32(const u8* w, i64 nw, const float* x, i64 nx, float* y, i64 ny) { return gemv_q_host(w, nw, x, nx, y, ny, 0); }
i64 wukong_gemv_q4_0_f32(const u8* w, i64 nw, const float* x, i64 nx, float* y, i64 ny) { return gemv_q_host(w, nw, x, nx, y, ny, 1); }
i64 wukong_gemv_q8_0_f32_parallel(const u8* w, i64 nw, const float* x, i64 nx, float* y, i64 ny) { return gemv_q_host(w, nw, x, nx, y, ny, 0); }
i64 wukong_gemv_q4_0_f32_parallel(const u8* w, i64 nw, const float* x, i64 nx, float* y, i64 ny) { return gemv_q_host(w, nw, x, nx, y, ny, 1); }
i64 wukong_dequant_i4_f32(const u8* q, i64 nq, const float* scale, i64 ns, i64 group, float* out, i64 nout) {
  return dequant_int4_host(q, nq, scale, ns, nullptr, -1, group, out, nout);
}
i64 wukong_dequant_u4_f32(const u8* q, i64 nq, const float* scale, i64 ns, const float* zero, i64 nz, i64 group,
                          float* out, i64 nout) {
  if (nz < 0) return -2;
  return dequant_int4_host(q, nq, scale, ns, zero, nz, group, out, nout);
}

// ---- elementwise (vmath.rs:1063-1130, :2022-2050; velem.rs:212-236) ----
void wukong_vmath_f32(const float* x, float* out, i64 n, i64 op) {
  if (n <= 0) return;
  Arena& A = g_arenas.current();
  A.begin(2 * pad((size_t)n * 4));
  float* dx = A.up(x, (size_t)n);
  float* dout = A.out<float>((size_t)n);
  check_launch(wkb_vmath_f32(dx, dout, n, op, A.stream), "vmath");
  A.down(out, dout, (size_t)n);
  A.sync();
}
void wukong_vmath_f32_parallel(const float* x, float* out, i64 n, i64 op) { wukong_vmath_f32(x, out, n, op); }
void wukong_vmath2_f32(const float* x, const float* y, float* out, i64 n, i64 op) {
  if (n <= 0) return;
  Arena& A = g_arenas.current();
  A.begin(3 * pad((size_t)n * 4));
  float* dx = A.up(x, (size_t)n);
  float* dy = A.up(y, (size_t)n);
  float* dout = A.out<float>((size_t)n);
  check_launch(wkb_vmath2_f32(dx, dy, dout, n, op, A.stream), "vmath2");
  A.down(out, dout, (size_t)n);
  A.sync();
}
void wukong_velem_f32(const float* x, const float* y, float* out, i64 n, float a, float b, float c, i64 op) {
  if (n <= 0) return;
  bool use_y = (op & (256 | 512 | 1024)) != 0;
  Arena& A = g_arenas.current();
  A.begin(3 * pad((size_t)n * 4));
  float* dx = A.up(x, (size_t)n);
  float* dy = use_y ? A.up(y, (size_t)n) : nullptr;
  float* dout = A.out<float>((size_t)n);
  check_launch(wkb_velem_f32(dx, dy, dout, n, a, b, c, op, A.stream), "velem");
  A.down(out, dout, (size_t)n);
  A.sync();
}
void wukong_velem_f32_parallel(const float* x, const float* y, float* out, i64 n, float a, float b, float c, i64 op) { wukong_velem_f32(x, y, out, n, a, b, c, op); }

// ---- norms (norm.rs:991-1200) ----
static void norm_host(const float* x, float* out, const float* gamma, const float* beta, i64 rows, i64 cols,
                      i64 eps_bits, i64 op, int affine) {
  if (rows <= 0 || cols <= 0) return;
  if (affine ? (op != 1 && op != 2) : (op < 0 || op > 4)) return;  // unknown code: nothing written
  size_t n = (size_t)rows * cols;
  Arena& A = g_arenas.current();
  A.begin(2 * pad(n * 4) + 2 * pad((size_t)cols * 4));
  float* dx = A.up(x, n);
  float* dg = A.up(gamma, (size_t)cols);
  float* db = A.up(beta, (size_t)cols);
  float* dout = A.out<float>(n);
  check_launch(wkb_norm_f32(dx, dout, dg, db, rows, cols, eps_bits, op, affine, A.stream), "norm");
  A.down(out, dout, n);
  A.sync();
}
void wukong_norm_f32(const float* x, float* out, i64 rows, i64 cols, i64 eps_bits, i64 op) {
  norm_host(x, out, nullptr, nullptr, rows, cols, eps_bits, op, 0);
}
void wukong_norm_affine_f32(const float* x, float* out, const float* gamma, const float* beta, i64 rows, i64 cols,
                            i64 eps_bits, i64 op) {
  norm_host(x, out, gamma, beta, rows, cols, eps_bits, op, 1);
}
void wukong_norm_f32_parallel(const float* x, float* out, i64 rows, i64 cols, i64 eps_bits, i64 op) { wukong_norm_f32(x, out, rows, cols, eps_bits, op); }
void wukong_norm_affine_f32_parallel(const float* x, float* out, const float* gamma, const float* beta, i64 rows, i64 cols, i64 eps_bits, i64 op) { wukong_norm_affine_f32(x, out, gamma, beta, rows, cols, eps_bits, op); }

// ---- attention over a KV cache (attention_kv.rs:153-311 plans, :1050-1360 entries) ----
i64 wukong_attention_kv_f32(const float* q, i64 nq, const float* k, i64 nk, const float* v, i64 nv, float* o, i64 no,
                            i64 sq, i64 skv, i64 d, i64 q_pos0, i64 n_heads, i64 n_kv_heads, i64 q_stride,
                            i64 kv_stride, float scale, i64 causal) {
  i64 geo[8] = {sq, skv, d, q_pos0, n_heads, n_kv_heads, q_stride, kv_stride};
  for (i64 g : geo) if (g < 0) return -1;
  if (nq < 0 || nk < 0 || nv < 0 || no < 0) return -1;
  if (sq == 0 || n_heads == 0 || d == 0) return 0;
  if (n_kv_heads == 0 || n_heads % n_kv_heads != 0) return -1;
  __int128 q_row = (__int128)n_heads * d, kv_row = (__int128)n_kv_heads * d;
  if ((__int128)q_stride < q_row || (skv > 0 && (__int128)kv_stride < kv_row)) return -1;
  __int128 q_ext = ((__int128)sq - 1) * q_stride + q_row;
  __int128 kv_ext = skv == 0 ? 0 : ((__int128)skv - 1) * kv_stride + kv_row;
  if (q_ext > nq || q_ext > no || kv_ext > nk || kv_ext > nv) return -2;
  Arena& A = g_arenas.current();
  A.begin(2 * pad((size_t)q_ext * 4) + 2 * pad((size_t)kv_ext * 4 + 16));
  float* dq = A.up(q, (size_t)q_ext);
  float* dk = kv_ext ? A.up(k, (size_t)kv_ext) : (float*)A.take(16);
  float* dv = kv_ext ? A.up(v, (size_t)kv_ext) : (float*)A.take(16);
  float* dob = A.up(o, (size_t)q_ext);  // lanes between heads keep their old contents
  check_launch(wkb_attention_kv_f32(dq, dk, dv, dob, nullptr, nullptr, 1, sq, skv, d, q_pos0, n_heads, n_kv_heads,
                                    q_stride, kv_stride, (i64)q_ext, (i64)kv_ext, scale, causal, A.stream), "attention_kv");
  A.down(o, dob, (size_t)q_ext);
  A.sync();
  return 0;
}
i64 wukong_attention_kv_f32_parallel(const float* q, i64 nq, const float* k, i64 nk, const float* v, i64 nv, float* o, i64 no, i64 sq, i64 skv, i64 d, i64 q_pos0, i64 n_heads, i64 n_kv_heads, i64 q_stride, i64 kv_stride, float scale, i64 causal) {
  return wukong_attention_kv_f32(q, nq, k, nk, v, nv, o, no, sq, skv, d, q_pos0, n_heads, n_kv_heads, q_stride, kv_stride, scale, causal);
}

i64 wukong_attention_kv_batch_f32(const float* q, i64 nq, const float* k, i64 nk, const float* v, i64 nv, float* o,
                                  i64 no, const int32_t* kv_lens, i64 nl, const int32_t* q_pos, i64 np, i64 batch,
                                  i64 sq, i64 skv, i64 n_heads, i64 n_kv_heads, i64 d, float scale, i64 causal) {
  i64 geo[6] = {batch, sq, skv, n_heads, n_kv_heads, d};
  for (i64 g : geo) if (g < 0) return -1;
  if (nq < 0 || nk < 0 || nv < 0 || no < 0 || nl < 0 || np < 0) return -1;
  if (batch == 0 || sq == 0 || n_heads == 0 || d == 0) return 0;
  if (n_kv_heads == 0 || n_heads % n_kv_heads != 0) return -1;
  __int128 q_ext = (__int128)batch * sq * n_heads * d, kv_ext = (__int128)batch * skv * n_kv_heads * d;
  if (q_ext > nq || q_ext > no || kv_ext > nk || kv_ext > nv || batch > nl || batch > np) return -2;
  for (i64 b = 0; b < batch; ++b)
    if (kv_lens[b] < 0 || (i64)kv_lens[b] > skv) return -1;
  Arena& A = g_arenas.current();
  A.begin(2 * pad((size_t)q_ext * 4) + 2 * pad((size_t)kv_ext * 4 + 16) + 2 * pad((size_t)batch * 4));
  float* dq = A.up(q, (size_t)q_ext);
  float* dk = kv_ext ? A.up(k, (size_t)kv_ext) : (float*)A.take(16);
  float* dv = kv_ext ? A.up(v, (size_t)kv_ext) : (float*)A.take(16);
  int* dl = A.up(kv_lens, (size_t)batch);
  int* dp = A.up(q_pos, (size_t)batch);
  float* dob = A.out<float>((size_t)q_ext);
  i64 q_row = n_heads * d, kv_row = n_kv_heads * d;
  check_launch(wkb_attention_kv_f32(dq, dk, dv, dob, dl, dp, batch, sq, skv, d, 0, n_heads, n_kv_heads, q_row, kv_row,
                                    sq * q_row, skv * kv_row, scale, causal, A.stream), "attention_kv_batch");
  A.down(o, dob, (size_t)q_ext);
  A.sync();
  return 0;
}
i64 wukong_attention_kv_batch_f32_parallel(const float* q, i64 nq, const float* k, i64 nk, const float* v, i64 nv, float* o, i64 no, const int32_t* kv_lens, i64 nl, const int32_t* q_pos, i64 np, i64 batch, i64 sq, i64 skv, i64 n_heads, i64 n_kv_heads, i64 d, float scale, i64 causal) {
  return wukong_attention_kv_batch_f32(q, nq, k, nk, v, nv, o, no, kv_lens, nl, q_pos, np, batch, sq, skv, n_heads, n_kv_heads, d, scale, causal);
}

// The cache of this entry lives in HOST memory, so the append is the host memmove the reference
// performs (attention_kv.rs:1301-1360); device-resident caches use wkb_kv_append_* instead.
i64 wukong_kv_append_f32(float* cache, i64 ncache, const float* row, i64 nrow, i64 pos, i64 stride) {
  if (ncache < 0 || nrow < 0 || pos < 0 || stride < 0) return -1;
  if (nrow == 0) return 0;
  if (stride < nrow) return -1;
  __int128 off = (__int128)pos * stride;
  if (off + nrow > (__int128)ncache) return -2;
  memmove(cache + (size_t)off, row, (size_t)nrow * 4);
  return 0;
}

void wukong_attention_f32(const float* q, const float* k, const float* v, float* o, i64 s, i64 d, float scale, i64 causal) {
  if (s <= 0 || d <= 0) return;
  size_t n = (size_t)s * d;
  Arena& A = g_arenas.current();
  A.begin(4 * pad(n * 4));
  float* dq = A.up(q, n);
  float* dk = A.up(k, n);
  float* dv = A.up(v, n);
  float* dob = A.out<float>(n);
  check_launch(wkb_attention_f32(dq, dk, dv, dob, s, d, scale, causal, A.stream), "attention");
  A.down(o, dob, n);
  A.sync();
}

// ---- RoPE, embedding, arg-max (rope.rs:143-230, embedding.rs:161-240, rowarg.rs:210-248) ----
void wukong_rope_f32(const float* x, const float* inv_freq, float* out, i64 rows, i64 half) {
  if (rows <= 0 || half <= 0) return;
  size_t n = (size_t)rows * half * 2;
  Arena& A = g_arenas.current();
  A.begin(2 * pad(n * 4) + pad((size_t)half * 4));
  float* dx = A.up(x, n);
  float* df = A.up(inv_freq, (size_t)half);
  float* dout = A.out<float>(n);
  check_launch(wkb_rope_f32(dx, df, nullptr, dout, rows, 1, half, A.stream), "rope");
  A.down(out, dout, n);
  A.sync();
}
void wukong_rope_f32_parallel(const float* x, const float* inv_freq, float* out, i64 rows, i64 half) { wukong_rope_f32(x, inv_freq, out, rows, half); }

void wukong_embedding_f32(float* out, const float* weight, const int32_t* ids, i64 t, i64 h, i64 v) {
  if (t <= 0 || h <= 0) return;
  i64 vv = v < 0 ? 0 : v;
  Arena& A = g_arenas.current();
  A.begin(pad((size_t)t * h * 4) + pad((size_t)vv * h * 4 + 16) + pad((size_t)t * 4));
  float* dw = vv ? A.up(weight, (size_t)vv * h) : (float*)A.take(16);
  int* di = A.up(ids, (size_t)t);
  float* dout = A.out<float>((size_t)t * h);
  check_launch(wkb_embedding_f32(dout, dw, di, t, h, vv, A.stream), "embedding");
  A.down(out, dout, (size_t)t * h);
  A.sync();
}
void wukong_embedding_f32_parallel(float* out, const float* weight, const int32_t* ids, i64 t, i64 h, i64 v) { wukong_embedding_f32(out, weight, ids, t, h, v); }

void wukong_rowargmax_i32(const float* x, int32_t* out, i64 rows, i64 cols) {
  if (rows <= 0 || cols <= 0) return;
  Arena& A = g_arenas.current();
  A.begin(pad((size_t)rows * cols * 4) + pad((size_t)rows * 4));
  float* dx = A.up(x, (size_t)rows * cols);
  int* dout = A.out<int>((size_t)rows);
  check_launch(wkb_rowargmax_i32(dx, dout, rows, cols, A.stream), "rowargmax");
  A.down(out, dout, (size_t)rows);
  A.sync();
}
void wukong_rowargmax_i32_parallel(const float* x, int32_t* out, i64 rows, i64 cols) { wukong_rowargmax_i32(x, out, rows, cols); }

// ---- selection / sampling / RNG (topk.rs:161-221, random.rs:88-104 of the reference runtime) ----
i64 wukong_topk_f32(const float* x, i64 n, float* vals, i64 nv, i64* idx, i64 ni) {
  if (n < 0) n = 0;
  i64 k = n;
  if (nv < k) k = nv < 0 ? 0 : nv;
  if (ni < k) k = ni < 0 ? 0 : ni;
  if (k <= 0) return 0;
  Arena& A = g_arenas.current();
  A.begin(pad((size_t)n * 4) + pad((size_t)k * 4) + pad((size_t)k * 8) + pad((size_t)wkb_argsort_scratch_bytes(n)));
  float* dx = A.up(x, (size_t)n);           // the input is snapshotted here: outputs may overlap it
  float* dv = A.out<float>((size_t)k);
  i64* di = A.out<i64>((size_t)k);
  if (k <= 64) {
    check_launch(wkb_topk_rows_f32(dx, n, 1, n, k, dv, di, A.stream), "topk");
  } else {
    void* scratch = A.take((size_t)wkb_argsort_scratch_bytes(n));
    check_launch(wkb_argsort_f32(dx, n, dv, di, k, 1, scratch, A.stream), "topk(sort)");
  }
  A.down(vals, dv, (size_t)k);
  A.down(idx, di, (size_t)k);
  A.sync();
  return k;
}

i64 wukong_argsort_f32(const float* x, i64 n, i64* idx, i64 ni, i64 descending) {
  if (n < 0) n = 0;
  i64 m = ni < n ? (ni < 0 ? 0 : ni) : n;
  if (m <= 0) return 0;
  Arena& A = g_arenas.current();
  A.begin(pad((size_t)n * 4) + pad((size_t)m * 8) + pad((size_t)wkb_argsort_scratch_bytes(n)));
  float* dx = A.up(x, (size_t)n);
  i64* di = A.out<i64>((size_t)m);
  void* scratch = A.take((size_t)wkb_argsort_scratch_bytes(n));
  check_launch(wkb_argsort_f32(dx, n, nullptr, di, m, descending, scratch, A.stream), "argsort");
  A.down(idx, di, (size_t)m);
  A.sync();
  return m;
}

i64 wukong_sample_categorical_f32(const float* p, i64 n, float u) {
  if (n <= 0 || !p) return -1;
  Arena& A = g_arenas.current();
  A.begin(pad((size_t)n * 4) + pad(8) + pad(8));
  float* dp = A.up(p, (size_t)n);
  float* du = A.up(&u, 1);
  i64* dout = A.out<i64>(1);
  check_launch(wkb_sample_categorical_rows_f32(dp, n, 1, n, du, dout, A.stream), "sample_categorical");
  i64 r = -1;
  A.down(&r, dout, 1);
  A.sync();
  return r;
}

void wukong_rand_fill_f32(float* out, i64 n, i64 seed, i64 ctr0) {
  if (n <= 0) return;
  Arena& A = g_arenas.current();
  A.begin(pad((size_t)n * 4));
  float* d = A.out<float>((size_t)n);
  check_launch(wkb_rand_fill_f32(d, n, seed, ctr0, A.stream), "rand_fill");
  A.down(out, d, (size_t)n);
  A.sync();
}

// Library identity / device probe used by the Python loader.
int wkb_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
  return n;
}
const char* wkb_build_arch(void) { return "sm_100a"; }
}

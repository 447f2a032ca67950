// Oracle (test infrastructure): RoPE, embedding gather, row arg-max, half / f8 codecs, and the
// thread fan-out of the timed CPU baseline.
// Follows crates/wukong_runtime/src/rope.rs (:54-71, :143-186), embedding.rs (:118-186),
// rowarg.rs (:1-60), reduce.rs (`arg_fold` :631-639), lib.rs (:287-333) and fp8.rs (:66-164).
#include "oracle_internal.h"
#include <cmath>
#include <thread>
#include <vector>
#include <atomic>
#include <unistd.h>
#include <condition_variable>
#include <mutex>
#include <immintrin.h>

namespace wko {

// IEEE f16 <-> f32, round to nearest even: the `half` crate's conversion equals F16C.
u16 f32_to_f16_bits(float x) { return (u16)_cvtss_sh(x, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC); }
float f16_bits_to_f32(u16 b) { return _cvtsh_ss(b); }

static std::atomic<int> g_threads{1};

// Persistent worker pool: the oracle's kernels are called a hundred times per model step, and starting a fresh set of
// std::threads for each call cost more than the kernels themselves once they were vectorised.  Workers sleep on a
// condition variable between calls; chunks are handed out through an atomic counter; the caller works too and returns
// when every worker has checked in.  A call that finds the pool busy (another host thread, or a nested call) runs serially.
namespace {
struct Pool {
  std::mutex m;
  std::condition_variable cv_start, cv_done;
  std::vector<std::thread> workers;
  const std::function<void(i64, i64)>* body = nullptr;
  std::atomic<i64> next{0};
  i64 nchunks = 0, chunk = 0, n = 0;
  unsigned long long gen = 0;
  int active = 0;
  bool stop = false;
  std::atomic_flag busy = ATOMIC_FLAG_INIT;

  void run_chunks() {
    for (;;) {
      const i64 c = next.fetch_add(1);
      if (c >= nchunks) return;
      const i64 lo = c * chunk, hi = lo + chunk < n ? lo + chunk : n;
      (*body)(lo, hi);
    }
  }
  void worker_main() {
    unsigned long long seen = 0;
    std::unique_lock<std::mutex> lk(m);
    for (;;) {
      cv_start.wait(lk, [&] { return stop || gen != seen; });
      if (stop) return;
      seen = gen;
      lk.unlock();
      run_chunks();
      lk.lock();
      if (--active == 0) cv_done.notify_one();
    }
  }
  void resize(int nworkers) {
    if ((int)workers.size() == nworkers) return;
    shutdown();
    stop = false;
    for (int t = 0; t < nworkers; ++t) workers.emplace_back([this] { worker_main(); });
  }
  void shutdown() {
    {
      std::lock_guard<std::mutex> lk(m);
      stop = true;
    }
    cv_start.notify_all();
    for (auto& t : workers) t.join();
    workers.clear();
  }
  ~Pool() { shutdown(); }
};
// The pool of this process.  A forked child inherits the object but none of its threads (and possibly a locked mutex):
// it is told apart by its pid and starts a pool of its own, leaving the inherited one alone.
Pool* g_pool_ptr = nullptr;
pid_t g_pool_pid = 0;
std::mutex g_pool_guard;
Pool& pool() {
  std::lock_guard<std::mutex> lk(g_pool_guard);
  const pid_t me = getpid();
  if (!g_pool_ptr || g_pool_pid != me) {
    g_pool_ptr = new Pool();      // an inherited pool is leaked on purpose: its threads do not exist here
    g_pool_pid = me;
  }
  return *g_pool_ptr;
}
struct PoolAtExit {
  ~PoolAtExit() {
    if (g_pool_ptr && g_pool_pid == getpid()) g_pool_ptr->shutdown();
  }
} g_pool_at_exit;
}  // namespace

void par_for(i64 n, i64 chunk, const std::function<void(i64, i64)>& body) {
  int nt = g_threads.load();
  if (chunk < 1) chunk = 1;
  i64 nchunks = (n + chunk - 1) / chunk;
  if (nt <= 1 || nchunks <= 1) { if (n > 0) body(0, n); return; }
  Pool& g_pool = pool();
  if (g_pool.busy.test_and_set(std::memory_order_acquire)) { body(0, n); return; }
  g_pool.resize(nt - 1);
  {
    std::lock_guard<std::mutex> lk(g_pool.m);
    g_pool.body = &body;
    g_pool.n = n; g_pool.chunk = chunk; g_pool.nchunks = nchunks;
    g_pool.next.store(0);
    g_pool.active = (int)g_pool.workers.size();
    ++g_pool.gen;
  }
  g_pool.cv_start.notify_all();
  g_pool.run_chunks();
  {
    std::unique_lock<std::mutex> lk(g_pool.m);
    g_pool.cv_done.wait(lk, [&] { return g_pool.active == 0; });
    g_pool.body = nullptr;
  }
  g_pool.busy.clear(std::memory_order_release);
}

// fp8.rs:66-164: OCP E4M3FN (bias 7, saturating, NaN S.1111.111) and E5M2 (bias 15, IEEE inf).
struct F8 { int mbits; int bias; double max; bool has_inf; };
static const F8 E4M3{3, 7, 448.0, false}, E5M2{2, 15, 57344.0, true};

static bool f8_decode(u8 b, const F8& f, double& out) {
  int ebits = 7 - f.mbits;
  unsigned emax = (1u << ebits) - 1;
  unsigned e = ((unsigned)b >> f.mbits) & emax;
  unsigned m = (unsigned)b & ((1u << f.mbits) - 1);
  double sign = (b & 0x80) ? -1.0 : 1.0;
  if (e == emax) {
    if (f.has_inf) { if (m == 0) { out = sign * INFINITY; return true; } return false; }
    if (m == (1u << f.mbits) - 1) return false;
  }
  double scale = (double)(1u << f.mbits);
  double mag = e == 0 ? (double)m / scale * std::ldexp(1.0, 1 - f.bias)
                      : (1.0 + (double)m / scale) * std::ldexp(1.0, (int)e - f.bias);
  out = sign * mag;
  return true;
}
static float f8_to_f32(u8 b, const F8& f) {
  double v;
  if (f8_decode(b, f, v)) return (float)v;
  uint32_t payload = f.has_inf ? ((uint32_t)(b & 3) << 21) : 0;
  return u2f(((uint32_t)(b & 0x80) << 24) | 0x7fc00000u | payload);
}
static u8 f8_encode(float xf, const F8& f) {
  double x = (double)xf;
  u8 sign = std::signbit(x) ? 0x80 : 0;
  if (x != x) return sign | (f.has_inf ? 0x7e : 0x7f);
  double a = std::fabs(x), rounded;
  int emin = 1 - f.bias;
  if (std::isinf(a)) rounded = INFINITY;
  else if (a == 0.0) rounded = 0.0;
  else {
    int e = std::ilogb(a);
    if (e < emin) e = emin;
    double ulp = std::ldexp(1.0, e - f.mbits);
    double qv = a / ulp, r = std::floor(qv), frac = qv - r;
    if (frac > 0.5 || (frac == 0.5 && std::fmod(r, 2.0) == 1.0)) r += 1.0;
    rounded = r * ulp;
  }
  double target = rounded > f.max ? (f.has_inf ? INFINITY : f.max) : rounded;
  for (unsigned c = 0; c < 0x80; ++c) {
    double v;
    if (f8_decode((u8)c, f, v) && v == target) return sign | (u8)c;
  }
  return sign;
}

}  // namespace wko

using namespace wko;

extern "C" {
void wko_set_threads(int n) { g_threads.store(n < 1 ? 1 : n); }
int wko_get_threads(void) { return g_threads.load(); }

u16 wko_f32_to_bf16_bits(float x) { return f32_to_bf16_bits(x); }
float wko_bf16_bits_to_f32(u16 b) { return bf16_bits_to_f32(b); }
u16 wko_f32_to_f16_bits(float x) { return f32_to_f16_bits(x); }
float wko_f16_bits_to_f32(u16 b) { return f16_bits_to_f32(b); }
u8 wko_f32_to_f8e4m3(float x) { return f8_encode(x, E4M3); }
float wko_f8e4m3_to_f32(u8 b) { return f8_to_f32(b, E4M3); }
u8 wko_f32_to_f8e5m2(float x) { return f8_encode(x, E5M2); }
float wko_f8e5m2_to_f32(u8 b) { return f8_to_f32(b, E5M2); }

// rope.rs:54-71, :143-186: half-split pairs, position = row index.
void wko_rope_f32(const float* x, const float* inv_freq, float* out, i64 rows, i64 half) {
  if (rows <= 0 || half <= 0) return;
  size_t h = (size_t)half, dim = 2 * h;
  par_for(rows, 1, [&](i64 lo, i64 hi) {
    for (i64 r = lo; r < hi; ++r) {
      float pos = (float)r;
      const float* xr = x + (size_t)r * dim;
      float* orow = out + (size_t)r * dim;
      for (size_t j = 0; j < h; ++j) {
        float theta = pos * inv_freq[j];
        float c = sincos1(theta, true), s = sincos1(theta, false);
        float a = xr[j], b = xr[j + h];
        orow[j] = fmaf(b, -s, a * c);
        orow[j + h] = fmaf(a, s, b * c);
      }
    }
  });
}

// The same rotation at an explicit per-row position, x laid out [rows, heads, 2*half].
void wko_rope_pos_f32(const float* x, const float* inv_freq, const int32_t* posv, float* out, i64 rows,
                      i64 heads, i64 half) {
  if (rows <= 0 || half <= 0 || heads <= 0) return;
  size_t h = (size_t)half, dim = 2 * h;
  for (i64 r = 0; r < rows; ++r) {
    float pos = (float)posv[r];
    for (i64 hh = 0; hh < heads; ++hh) {
      const float* xr = x + ((size_t)r * (size_t)heads + (size_t)hh) * dim;
      float* orow = out + ((size_t)r * (size_t)heads + (size_t)hh) * dim;
      for (size_t j = 0; j < h; ++j) {
        float theta = pos * inv_freq[j];
        float c = sincos1(theta, true), s = sincos1(theta, false);
        float a = xr[j], b = xr[j + h];
        orow[j] = fmaf(b, -s, a * c);
        orow[j + h] = fmaf(a, s, b * c);
      }
    }
  }
}

// embedding.rs:118-186: in-range ids copy the row; any other id writes a zero row.
void wko_embedding_f32(float* out, const float* weight, const int32_t* ids, i64 t, i64 h, i64 v) {
  if (t <= 0 || h <= 0) return;
  i64 vv = v < 0 ? 0 : v;
  for (i64 r = 0; r < t; ++r) {
    int32_t id = ids[r];
    float* orow = out + (size_t)r * (size_t)h;
    if (id >= 0 && (i64)id < vv) memcpy(orow, weight + (size_t)id * (size_t)h, (size_t)h * 4);
    else memset(orow, 0, (size_t)h * 4);
  }
}

// rowarg.rs:40-50 with reduce.rs:631-639: ascending scan, strict compare, lowest index on a tie.
void wko_rowargmax_i32(const float* x, int32_t* out, i64 rows, i64 cols) {
  if (rows <= 0 || cols <= 0) return;
  par_for(rows, 1, [&](i64 lo, i64 hi) {
    for (i64 r = lo; r < hi; ++r) {
      const float* row = x + (size_t)r * (size_t)cols;
      float bv = row[0];
      size_t bi = 0;
      for (size_t j = 1; j < (size_t)cols; ++j)
        if (row[j] > bv) { bv = row[j]; bi = j; }
      out[r] = (int32_t)bi;
    }
  });
}
}

// Oracle (test infrastructure): f32 / half GEMM and GEMV by the reference's per-element order
// contract.  Follows crates/wukong_runtime/src/gemm.rs (module docs :30-58, `select_kc` :253-256,
// `Epilogue::apply` :751-780, the portable twin `sgemm_scalar` :3234-3282), gemv.rs (:28-88,
// :141-180) and gemv_half.rs (`elem_scalar` :73-110, checked entries :440-529).
#include "oracle_internal.h"
#include <vector>
#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#endif
#include <cmath>

namespace wko {

struct Epi {
  const float* bias;
  uint32_t act;
  float alpha;
};

// gemm.rs:751-780.
static inline float epi_apply(const Epi& e, float x, size_t j) {
  float y = (e.alpha != 1.0f) ? e.alpha * x : x;
  if (e.bias) y += e.bias[j];
  switch (e.act) {
    case 1: y = y > 0.0f ? y : 0.0f; break;
    case 2: y = gelu1(y); break;
    case 3: y = silu1(y); break;
    default: break;
  }
  return y;
}

// gemm.rs:3234-3282: for each (i, j): K blocks of select_kc(k); every block is an ascending-p fma
// chain from +0.0; the first block honours beta (a 0 / non-0 flag), later blocks add into C; the
// epilogue runs once, on the last block, with the global column index.
template <typename LoadA, typename LoadB>
static void gemm_contract(LoadA la, LoadB lb, float* c, size_t m, size_t k, size_t n, float beta,
                          const Epi* epi) {
  const size_t kcap = (size_t)select_kc((i64)k);
  par_for((i64)m * (i64)n, 4096, [&](i64 lo, i64 hi) {
    for (i64 idx = lo; idx < hi; ++idx) {
      size_t i = (size_t)idx / n, j = (size_t)idx % n;
      float* cij = c + i * n + j;
      size_t pc = 0;
      while (pc < k) {
        size_t kc = (k - pc) < kcap ? (k - pc) : kcap;
        float acc = 0.0f;
        for (size_t p = pc; p < pc + kc; ++p) acc = fmaf(la(i, p), lb(p, j), acc);
        float beta_eff = (pc == 0) ? beta : 1.0f;
        float val = (beta_eff == 0.0f) ? acc : *cij + acc;
        *cij = (pc + kc == k && epi) ? epi_apply(*epi, val, j) : val;
        pc += kc;
      }
    }
  });
}

// The NT form with B read in its storage type.  Each (i, j) still runs exactly the chain of `gemm_contract` (ascending p
// per K block from +0.0, blocks folded in order, one fused multiply-add per step), so the bits are the same; what changes
// is which chains run side by side.  The eight lanes of a vector are eight ROWS of A (A is repacked once per call as
// [p][row panel][8 rows]); an element of B is widened, broadcast and multiplied into every row of the panel, so each weight
// is read once per call whatever the number of activation rows -- the traffic pattern of a register-blocked AVX2
// microkernel, which is what makes the timed CPU baseline a fair port of the reference's CPU path rather than a loop that
// streams the weight matrix once per activation row.  Four columns x two panels = eight independent chains per thread
// hide the FMA latency.
template <typename TB>
static inline float widen_b(TB v);
template <> inline float widen_b<float>(float v) { return v; }
struct Bf16B { u16 b; };
struct F16B { u16 b; };
template <> inline float widen_b<Bf16B>(Bf16B v) { return bf16_bits_to_f32(v.b); }
template <> inline float widen_b<F16B>(F16B v) { return f16_bits_to_f32(v.b); }

#if defined(__AVX2__) && defined(__FMA__)
// eight consecutive elements of B, widened exactly (bf16: the bits moved to the top half; f16: vcvtph2ps)
template <typename TB>
static inline __m256 widen8(const TB* p);
template <> inline __m256 widen8<float>(const float* p) { return _mm256_loadu_ps(p); }
template <> inline __m256 widen8<Bf16B>(const Bf16B* p) {
  return _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_cvtepu16_epi32(_mm_loadu_si128(reinterpret_cast<const __m128i*>(p))), 16));
}
template <> inline __m256 widen8<F16B>(const F16B* p) { return _mm256_cvtph_ps(_mm_loadu_si128(reinterpret_cast<const __m128i*>(p))); }
#endif

template <typename TB>
static void gemm_nt_fast(const float* a, const TB* b, float* c, size_t M, size_t K, size_t N, float beta,
                         const Epi* epi) {
  const size_t kcap = (size_t)select_kc((i64)K);
  constexpr size_t JB = 4, PB = 2;                 // columns and row panels in flight
  const size_t panels = (M + 7) / 8;
  // A^T in panels of 8 rows: at[(p * panels + panel) * 8 + lane] = a[panel * 8 + lane][p]; rows past M are zero
  std::vector<float> at(K * panels * 8, 0.0f);
  par_for((i64)panels, 1, [&](i64 lo, i64 hi) {
    for (i64 pn = lo; pn < hi; ++pn)
      for (size_t lane = 0; lane < 8; ++lane) {
        const size_t i = (size_t)pn * 8 + lane;
        if (i >= M) break;
        const float* ar = a + i * K;
        for (size_t p = 0; p < K; ++p) at[(p * panels + (size_t)pn) * 8 + lane] = ar[p];
      }
  });
  const size_t jblocks = (N + JB - 1) / JB;
  par_for((i64)jblocks, 4, [&](i64 lo, i64 hi) {
    for (i64 u = lo; u < hi; ++u) {
      const size_t j0 = (size_t)u * JB, nj = N - j0 < JB ? N - j0 : JB;
      const TB* br[JB];
      for (size_t jj = 0; jj < JB; ++jj) br[jj] = b + (j0 + (jj < nj ? jj : 0)) * K;
      for (size_t pn0 = 0; pn0 < panels; pn0 += PB) {
        const size_t np = panels - pn0 < PB ? panels - pn0 : PB;
        for (size_t pc = 0; pc < K; pc += kcap) {
          const size_t kc = K - pc < kcap ? K - pc : kcap;
          float acc[JB][PB][8];
#if defined(__AVX2__) && defined(__FMA__)
          __m256 v[JB][PB];
#pragma GCC unroll 4
          for (size_t jj = 0; jj < JB; ++jj) {
            v[jj][0] = _mm256_setzero_ps();
            v[jj][1] = _mm256_setzero_ps();
          }
          // eight consecutive K elements of a column are widened together and broadcast lane by lane from the register
          // (one shuffle per element instead of a scalar widen + move + broadcast); the chain of every (i, j) still takes
          // its products in ascending p
          size_t p = pc;
          for (; p + 8 <= pc + kc; p += 8) {
            __m256 bw[JB];
#pragma GCC unroll 4
            for (size_t jj = 0; jj < JB; ++jj) bw[jj] = widen8<TB>(br[jj] + p);
#pragma GCC unroll 8
            for (size_t e = 0; e < 8; ++e) {
              const float* ap = at.data() + ((p + e) * panels + pn0) * 8;
              const __m256 a0 = _mm256_loadu_ps(ap);
              const __m256 a1 = np > 1 ? _mm256_loadu_ps(ap + 8) : _mm256_setzero_ps();
              const __m256i idx = _mm256_set1_epi32((int)e);
#pragma GCC unroll 4
              for (size_t jj = 0; jj < JB; ++jj) {
                const __m256 bv = _mm256_permutevar8x32_ps(bw[jj], idx);
                v[jj][0] = _mm256_fmadd_ps(a0, bv, v[jj][0]);      // one fused multiply-add per lane: fmaf(a, b, acc)
                v[jj][1] = _mm256_fmadd_ps(a1, bv, v[jj][1]);
              }
            }
          }
          for (; p < pc + kc; ++p) {
            const float* ap = at.data() + (p * panels + pn0) * 8;
            const __m256 a0 = _mm256_loadu_ps(ap);
            const __m256 a1 = np > 1 ? _mm256_loadu_ps(ap + 8) : _mm256_setzero_ps();
#pragma GCC unroll 4
            for (size_t jj = 0; jj < JB; ++jj) {
              const __m256 bv = _mm256_set1_ps(widen_b<TB>(br[jj][p]));
              v[jj][0] = _mm256_fmadd_ps(a0, bv, v[jj][0]);
              v[jj][1] = _mm256_fmadd_ps(a1, bv, v[jj][1]);
            }
          }
#pragma GCC unroll 4
          for (size_t jj = 0; jj < JB; ++jj) {
            _mm256_storeu_ps(acc[jj][0], v[jj][0]);
            _mm256_storeu_ps(acc[jj][1], v[jj][1]);
          }
#else
          for (size_t jj = 0; jj < JB; ++jj)
            for (size_t q = 0; q < PB; ++q)
              for (size_t l = 0; l < 8; ++l) acc[jj][q][l] = 0.0f;
          for (size_t p = pc; p < pc + kc; ++p) {
            const float* ap = at.data() + (p * panels + pn0) * 8;
            for (size_t jj = 0; jj < JB; ++jj) {
              const float bv = widen_b<TB>(br[jj][p]);
              for (size_t q = 0; q < np; ++q)
                for (size_t l = 0; l < 8; ++l) acc[jj][q][l] = fmaf(ap[q * 8 + l], bv, acc[jj][q][l]);
            }
          }
#endif
          const float beta_eff = pc == 0 ? beta : 1.0f;
          const bool last = pc + kc == K;
          for (size_t q = 0; q < np; ++q)
            for (size_t l = 0; l < 8; ++l) {
              const size_t i = (pn0 + q) * 8 + l;
              if (i >= M) break;
              for (size_t jj = 0; jj < nj; ++jj) {
                float* cij = c + i * N + j0 + jj;
                const float val = beta_eff == 0.0f ? acc[jj][q][l] : *cij + acc[jj][q][l];
                *cij = (last && epi) ? epi_apply(*epi, val, j0 + jj) : val;
              }
            }
        }
      }
    }
  });
}

static void sgemm_f32(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta, bool at,
                      bool bt, const Epi* epi) {
  if (m <= 0 || k <= 0 || n <= 0) return;  // gemm.rs:1018-1020
  size_t M = (size_t)m, K = (size_t)k, N = (size_t)n;
  if (!at && bt) { gemm_nt_fast<float>(a, b, c, M, K, N, (float)beta, epi); return; }
  auto la = [=](size_t i, size_t p) { return at ? a[p * M + i] : a[i * K + p]; };
  auto lb = [=](size_t p, size_t j) { return bt ? b[j * K + p] : b[p * N + j]; };
  gemm_contract(la, lb, c, M, K, N, (float)beta, epi);
}

// gemm.rs:1436-1480: both half operands widen losslessly, then the f32 contract applies.
static void sgemm_half_nt(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta, bool bf16,
                          const Epi* epi) {
  if (m <= 0 || k <= 0 || n <= 0) return;
  size_t M = (size_t)m, K = (size_t)k, N = (size_t)n;
  std::vector<float> af(M * K);
  for (size_t i = 0; i < M * K; ++i) af[i] = bf16 ? bf16_bits_to_f32(a[i]) : f16_bits_to_f32(a[i]);
  if (bf16) gemm_nt_fast<Bf16B>(af.data(), reinterpret_cast<const Bf16B*>(b), c, M, K, N, (float)beta, epi);
  else gemm_nt_fast<F16B>(af.data(), reinterpret_cast<const F16B*>(b), c, M, K, N, (float)beta, epi);
}

// gemv.rs:60-88 with hsum256 (:28-38): four 8-lane fma accumulators over 32-element steps,
// leftover 8-blocks into the first, tree (c0+c1)+(c2+c3), horizontal
// ((v0+v4)+(v1+v5))+((v2+v6)+(v3+v7)), then an unfused scalar tail.
static float gemv_row(const float* a, const float* x, size_t n) {
  float c[4][8] = {};
  size_t j = 0;
  while (j + 32 <= n) {
    for (int t = 0; t < 4; ++t)
      for (int l = 0; l < 8; ++l) c[t][l] = fmaf(a[j + 8 * t + l], x[j + 8 * t + l], c[t][l]);
    j += 32;
  }
  while (j + 8 <= n) {
    for (int l = 0; l < 8; ++l) c[0][l] = fmaf(a[j + l], x[j + l], c[0][l]);
    j += 8;
  }
  float v[8];
  for (int l = 0; l < 8; ++l) v[l] = (c[0][l] + c[1][l]) + (c[2][l] + c[3][l]);
  float s = ((v[0] + v[4]) + (v[1] + v[5])) + ((v[2] + v[6]) + (v[3] + v[7]));
  while (j < n) {
    s += a[j] * x[j];
    ++j;
  }
  return s;
}

// gemv_half.rs:73-110 with beta = 0 and no epilogue (the checked GEMV entries).
static i64 sgemv_half(const u16* w, i64 nw, const float* x, i64 nx, float* y, i64 ny, bool bf16) {
  if (nw < 0 || nx < 0 || ny < 0) return -2;
  // gemv_half_plan: w_len must be exactly N*K.
  __int128 need = (__int128)ny * (__int128)nx;
  if (need != (__int128)nw) return -2;
  size_t N = (size_t)ny, K = (size_t)nx;
  if (N == 0) return 0;
  if (K == 0) {
    for (size_t j = 0; j < N; ++j) y[j] = 0.0f;
    return 0;
  }
  std::vector<float> xin(x, x + K);  // value semantics: inputs read as they were before the call
  std::vector<float> out(N);
  const size_t kcap = (size_t)select_kc((i64)K);
  par_for((i64)N, 64, [&](i64 lo, i64 hi) {
    for (i64 j = lo; j < hi; ++j) {
      const u16* row = w + (size_t)j * K;
      float cval = 0.0f;
      size_t pc = 0;
      while (pc < K) {
        size_t pend = pc + ((K - pc) < kcap ? (K - pc) : kcap);
        float acc = 0.0f;
        for (size_t p = pc; p < pend; ++p) {
          float wv = bf16 ? bf16_bits_to_f32(row[p]) : f16_bits_to_f32(row[p]);
          acc = fmaf(xin[p], wv, acc);
        }
        cval = (pc == 0) ? acc : cval + acc;
        pc = pend;
      }
      out[(size_t)j] = cval;
    }
  });
  for (size_t j = 0; j < N; ++j) y[j] = out[j];
  return 0;
}

}  // namespace wko

using namespace wko;

extern "C" {
i64 wko_select_kc(i64 k) { return select_kc(k); }

void wko_sgemm(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta) {
  sgemm_f32(a, b, c, m, k, n, beta, false, false, nullptr);
}
void wko_sgemm_nt(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta) {
  sgemm_f32(a, b, c, m, k, n, beta, false, true, nullptr);
}
void wko_sgemm_tn(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta) {
  sgemm_f32(a, b, c, m, k, n, beta, true, false, nullptr);
}
void wko_sgemm_nt_epi(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta,
                      const float* bias, i64 act) {
  Epi e{bias, (uint32_t)act, 1.0f};
  sgemm_f32(a, b, c, m, k, n, beta, false, true, &e);
}
void wko_sgemm_nt_alpha(const float* a, const float* b, float* c, i64 m, i64 k, i64 n, i64 beta, float alpha) {
  Epi e{nullptr, 0u, alpha};
  sgemm_f32(a, b, c, m, k, n, beta, false, true, &e);
}
void wko_sgemm_bf16_nt(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta) {
  sgemm_half_nt(a, b, c, m, k, n, beta, true, nullptr);
}
void wko_sgemm_f16_nt(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta) {
  sgemm_half_nt(a, b, c, m, k, n, beta, false, nullptr);
}
void wko_sgemm_bf16_nt_epi(const u16* a, const u16* b, float* c, i64 m, i64 k, i64 n, i64 beta,
                           const float* bias, i64 act) {
  Epi e{bias, (uint32_t)act, 1.0f};
  sgemm_half_nt(a, b, c, m, k, n, beta, true, &e);
}

// gemv.rs:160-226.
void wko_sgemv_alpha(const float* a, const float* x, float* y, i64 m, i64 n, float alpha) {
  if (m <= 0 || n <= 0) return;
  par_for(m, 16, [&](i64 lo, i64 hi) {
    for (i64 i = lo; i < hi; ++i) {
      float s = gemv_row(a + (size_t)i * (size_t)n, x, (size_t)n);
      y[i] = (alpha != 1.0f) ? s * alpha : s;
    }
  });
}
void wko_sgemv(const float* a, const float* x, float* y, i64 m, i64 n) { wko_sgemv_alpha(a, x, y, m, n, 1.0f); }

i64 wko_sgemv_bf16(const u16* w, i64 nw, const float* x, i64 nx, float* y, i64 ny) {
  return sgemv_half(w, nw, x, nx, y, ny, true);
}
i64 wko_sgemv_f16(const u16* w, i64 nw, const float* x, i64 nx, float* y, i64 ny) {
  return sgemv_half(w, nw, x, nx, y, ny, false);
}
}

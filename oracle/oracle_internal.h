// Oracle (test infrastructure): shared internals -- bit casts, the scalar math twins, and the
// fixed-unit thread fan-out used only by the timed CPU baseline.
#pragma once
#include "wk_oracle.h"
#include <cstring>
#include <functional>

namespace wko {
static inline uint32_t f2u(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float u2f(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

float exp1(float x);
float log1(float x);
float tanh1(float x);
float sigmoid1(float x);
float silu1(float x);
float gelu1(float x);
float sincos1(float x, bool is_cos);
float apply1(i64 op, float x);
[[noreturn]] void unsupported(const char* what, i64 code);

// lib.rs:287-333 of the reference runtime.
static inline u16 f32_to_bf16_bits(float x) {
  uint32_t bits = f2u(x);
  if (x != x) return (u16)((bits >> 16) | 0x0040);
  uint32_t bias = 0x00007fffu + ((bits >> 16) & 1u);
  return (u16)((bits + bias) >> 16);
}
static inline float bf16_bits_to_f32(u16 b) { return u2f(((uint32_t)b) << 16); }
u16 f32_to_f16_bits(float x);
float f16_bits_to_f32(u16 b);

// gemm.rs:253-256.
static inline i64 select_kc(i64 k) {
  const i64 KC = 384;
  i64 nblocks = (k + KC - 1) / KC;
  if (nblocks < 1) nblocks = 1;
  i64 per = (k + nblocks - 1) / nblocks;
  return (per + 3) / 4 * 4;
}

static inline bool bytes_overlap(const void* a, size_t na, const void* b, size_t nb) {
  if (na == 0 || nb == 0) return false;
  uintptr_t pa = (uintptr_t)a, pb = (uintptr_t)b;
  return pa < pb + nb && pb < pa + na;
}

// Split [0, n) into fixed `chunk`-sized spans and run them on the oracle's threads.  Spans never
// share an output, so thread count cannot change a bit.
void par_for(i64 n, i64 chunk, const std::function<void(i64, i64)>& body);
}  // namespace wko

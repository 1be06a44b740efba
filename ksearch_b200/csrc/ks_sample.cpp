// CPU logit sampling for the serve surface: softcap, temperature, min-p, multinomial draw
// (crates/ksearch_gemma/src/sample.rs:9-81).  The reference samples on the host from the logits the device
// produced; temperature < 1e-6 is the greedy arg-max after the softcap, the same choice the device kernel makes
// (crates/ksearch_kernels/src/lib.rs:1966).  Host code: no GPU is touched here.
#include <cmath>
#include <cstring>
#include <vector>

#include "ks_internal.h"

namespace {

// sample.rs:76-81
inline uint32_t splitmix32(uint32_t* state) {
  *state += 0x9E3779B9u;
  uint32_t z = *state;
  z = (z ^ (z >> 16)) * 0x7feb352du;
  z = (z ^ (z >> 15)) * 0x846ca68bu;
  return z ^ (z >> 16);
}

// crates/ksearch_gguf/src/lib.rs:20-35 f16_to_f32
inline float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1Fu, mant = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (mant == 0) {
      bits = sign;
    } else {  // subnormal: value = mant * 2^-24
      float f = (float)mant * 5.9604644775390625e-08f;
      memcpy(&bits, &f, 4);
      bits |= sign;
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (mant << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (mant << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

template <typename Get>
uint32_t sample_impl(size_t n, Get get, float cap, float temperature, float min_p, uint32_t seed) {
  uint32_t best_i = 0;
  float best_v = -INFINITY;
  std::vector<float> xs(n);
  for (size_t i = 0; i < n; i++) {
    const float x = get(i);
    const float y = cap > 0.0f ? cap * tanhf(x / cap) : x;
    xs[i] = y;
    if (y > best_v) {  // strict: the first of equal values stays
      best_v = y;
      best_i = (uint32_t)i;
    }
  }
  if (temperature < 1e-6f) return best_i;
  float sum = 0.0f;
  for (float& x : xs) {
    x = expf((x - best_v) / temperature);
    sum += x;
  }
  const float inv = 1.0f / fmaxf(sum, 1e-30f);
  float p_max = 0.0f;
  for (float& x : xs) {
    x *= inv;
    if (x > p_max) p_max = x;
  }
  const float threshold = p_max * fmaxf(min_p, 0.0f);
  float filtered = 0.0f;
  for (float& x : xs) {
    if (x < threshold) x = 0.0f;
    else filtered += x;
  }
  if (filtered <= 1e-9f) return best_i;
  uint32_t rng = seed | 1u;
  const float r = ((float)splitmix32(&rng) / 4294967296.0f) * filtered;
  float cdf = 0.0f;
  for (size_t i = 0; i < n; i++) {
    cdf += xs[i];
    if (r < cdf) return (uint32_t)i;
  }
  return (uint32_t)(n - 1);
}

}  // namespace

extern "C" {

// sample_softcap_min_p over f16 logit bits, as the reference takes them.  n >= 1; returns the token id.
uint32_t ks_sample_softcap_min_p(const uint16_t* logits_f16, size_t n, float cap, float temperature, float min_p, uint32_t seed) {
  if (!logits_f16 || n == 0) return 0;
  return sample_impl(n, [&](size_t i) { return half_to_float(logits_f16[i]); }, cap, temperature, min_p, seed);
}

// The same over f32 logits (what this library's f32 models produce).
uint32_t ks_sample_softcap_min_p_f32(const float* logits, size_t n, float cap, float temperature, float min_p, uint32_t seed) {
  if (!logits || n == 0) return 0;
  return sample_impl(n, [&](size_t i) { return logits[i]; }, cap, temperature, min_p, seed);
}

}  // extern "C"

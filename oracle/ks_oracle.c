/*
 * ks_oracle.c -- CPU restatement of the ksearch decode hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is
 * compared against; nothing in the shipped package calls it.  It restates, in
 * plain C, the arithmetic of the reference (paths are relative to the
 * reference project root):
 *
 *   crates/ksearch_gguf/src/lib.rs:20-75          f16 <-> f32 conversions
 *   crates/ksearch_gguf/src/gguf_impl.rs:563-573  get_scale_min_k4
 *   crates/ksearch_gguf/src/gguf_impl.rs:618-633  Q4_0 dequant
 *   crates/ksearch_gguf/src/gguf_impl.rs:690-721  Q4_K dequant
 *   crates/ksearch_gguf/src/gguf_impl.rs:761-791  Q6_K dequant
 *   crates/ksearch_gguf/src/gguf_impl.rs:803-1016 Q4_K reference quantizer
 *   crates/ksearch_kernels/examples/check_mul_mm.rs:60-71  dequant + f32 dot
 *   crates/ksearch_codegen/src/render.rs:1021-1059  Q4_0 pack (shader math)
 *   crates/ksearch_codegen/src/lower.rs:3926-4162   RMSNorm family
 *   crates/ksearch_codegen/src/lower.rs:4231-4702   per-head RMS + RoPE + pack
 *   crates/ksearch_codegen/src/lower.rs:4897-5359   online-softmax attention
 *   crates/ksearch_codegen/src/lower.rs:5367-6088   16-partition attention + merge
 *   crates/ksearch_codegen/src/lower.rs:2926-2954   tanh-GELU * up
 *   crates/ksearch_codegen/src/lower.rs:6090-6157   softcap argmax
 *   crates/ksearch_gemma/src/gemma_prim.rs:33-56    RoPE table
 *   crates/ksearch_gemma/src/gemma_prim.rs:881-1275 forward_token op order
 *
 * Pinning status.  The reference holds no byte-level golden vectors for this
 * path.  Its only CPU test touching the math (q4k_roundtrip_approx,
 * gguf_impl.rs:1022-1059) is reproduced by tests/ (quantize -> dequant of the
 * same signal, same thresholds, zero block exact), and the integer-pattern
 * matrices of check_mul_mm.rs are reproduced as known-answer inputs.  The
 * attention / norm / RoPE / GELU / argmax functions have no CPU twin in the
 * reference at all, so for those this oracle is a restatement of the shader
 * lowering: PARITY UNPINNED for those ops.
 *
 * Build: gcc -O2 -ffp-contract=off (no FMA contraction: the reference's Rust
 * never fuses a*b-c, and dequant must be bit-exact).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QK_K 256
#define Q4K_BS 144
#define Q6K_BS 210
#define Q40_BS 18

/* ---- f16 conversions (crates/ksearch_gguf/src/lib.rs:20-75) ------------- */

float kso_f16_to_f32(uint16_t h) {
  float sign = (float)(h >> 15) * -2.0f + 1.0f;
  int e = (h >> 10) & 0x1F;
  int mant = h & 0x3FF;
  if (e == 0) return sign * (float)mant * ldexpf(1.0f, -24);
  if (e == 31) return mant == 0 ? sign * INFINITY : NAN;
  return sign * (1.0f + (float)mant / 1024.0f) * ldexpf(1.0f, e - 15);
}

/* The reference's own f32->f16: adds 0x1000 to the mantissa (round half UP in
 * magnitude, not ties-to-even), lib.rs:39-75. Used by its host-side quantizer. */
uint16_t kso_f32_to_f16_ref(float v) {
  uint32_t bits;
  memcpy(&bits, &v, 4);
  uint16_t sign = (uint16_t)((bits >> 16) & 0x8000);
  int e = (int)((bits >> 23) & 0xFF);
  uint32_t mant = bits & 0x7FFFFF;
  if (e == 255) return mant == 0 ? (sign | 0x7C00) : (uint16_t)(sign | 0x7C00 | (mant >> 13));
  e -= 127;
  if (e > 15) return sign | 0x7C00;
  if (e < -14) {
    if (e < -24) return sign;
    mant |= 0x800000;
    uint32_t shift = (uint32_t)(-14 - e) + 13;
    uint32_t r = (mant + (1u << (shift - 1))) >> shift;
    return (uint16_t)(sign | r);
  }
  uint16_t he = (uint16_t)(e + 15);
  uint32_t hm = mant + 0x1000;
  if (hm & 0x800000) return (uint16_t)(sign | ((he + 1) << 10));
  return (uint16_t)(sign | (he << 10) | (hm >> 13));
}

/* IEEE round-to-nearest-even f32->f16: what a GPU `half(x)` store does
 * (the shader-side conversion, e.g. render.rs:1033 `half(scale)`). */
uint16_t kso_f32_to_f16_rne(float v) {
  uint32_t x;
  memcpy(&x, &v, 4);
  uint32_t sign = (x >> 16) & 0x8000;
  uint32_t ax = x & 0x7FFFFFFF;
  if (ax >= 0x7F800000) return (uint16_t)(sign | 0x7C00 | (ax > 0x7F800000 ? 0x200 : 0));
  if (ax >= 0x477FF000) return (uint16_t)(sign | 0x7C00); /* >= 65520 rounds to inf */
  if (ax < 0x33000001) return (uint16_t)sign;               /* <= 2^-25 rounds to 0 */
  int e = (int)(ax >> 23) - 127;
  uint32_t mant = (ax & 0x7FFFFF) | 0x800000;
  int shift = (e < -14) ? (13 + (-14 - e)) : 13;
  uint32_t half_m = mant >> shift;
  uint32_t rem = mant & ((1u << shift) - 1);
  uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (half_m & 1))) half_m++;
  uint32_t out;
  if (e < -14) out = half_m; /* subnormal; carry into exponent is naturally right */
  else out = ((uint32_t)(e + 15) << 10) + (half_m - 0x400);
  return (uint16_t)(sign | out);
}

void kso_f16_to_f32_n(const uint16_t* src, float* dst, size_t n) {
  for (size_t i = 0; i < n; i++) dst[i] = kso_f16_to_f32(src[i]);
}
void kso_f32_to_f16_rne_n(const float* src, uint16_t* dst, size_t n) {
  for (size_t i = 0; i < n; i++) dst[i] = kso_f32_to_f16_rne(src[i]);
}
void kso_f32_to_f16_ref_n(const float* src, uint16_t* dst, size_t n) {
  for (size_t i = 0; i < n; i++) dst[i] = kso_f32_to_f16_ref(src[i]);
}

static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* ---- 6-bit scale/min unpack (gguf_impl.rs:563-573) ---------------------- */
static inline void scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) {
  if (j < 4) {
    *d = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *d = (uint8_t)((q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4));
    *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
  }
}
void kso_scale_min_k4(int j, const uint8_t* q, uint8_t* d, uint8_t* m) { scale_min_k4(j, q, d, m); }

/* ---- dequant (gguf_impl.rs:618-633, 690-721, 761-791) ------------------- */
static void deq_q40_block(const uint8_t* blk, float* out) {
  float d = kso_f16_to_f32(rd16(blk));
  const uint8_t* qs = blk + 2;
  for (int i = 0; i < 16; i++) {
    int lo = (int)(qs[i] & 0x0F) - 8;
    int hi = (int)(qs[i] >> 4) - 8;
    out[i] = (float)lo * d;
    out[i + 16] = (float)hi * d;
  }
}

static void deq_q4k_block(const uint8_t* blk, float* out) {
  float d = kso_f16_to_f32(rd16(blk));
  float dmin = kso_f16_to_f32(rd16(blk + 2));
  const uint8_t* scales = blk + 4;
  const uint8_t* qs = blk + 16;
  int is = 0, qoff = 0;
  for (int y = 0; y < QK_K; y += 64) {
    uint8_t sc1, m1, sc2, m2;
    scale_min_k4(is, scales, &sc1, &m1);
    scale_min_k4(is + 1, scales, &sc2, &m2);
    float d1 = d * (float)sc1, mn1 = dmin * (float)m1;
    float d2 = d * (float)sc2, mn2 = dmin * (float)m2;
    for (int l = 0; l < 32; l++) out[y + l] = d1 * (float)(qs[qoff + l] & 0x0F) - mn1;
    for (int l = 0; l < 32; l++) out[y + 32 + l] = d2 * (float)(qs[qoff + l] >> 4) - mn2;
    qoff += 32;
    is += 2;
  }
}

/* gguf_impl.rs:722-760 */
static void deq_q5k_block(const uint8_t* blk, float* out) {
  float d = kso_f16_to_f32(rd16(blk));
  float dmin = kso_f16_to_f32(rd16(blk + 2));
  const uint8_t* scales = blk + 4;
  const uint8_t* qh = blk + 16;
  const uint8_t* qs = blk + 48;
  int is = 0, qoff = 0;
  uint8_t u1 = 1, u2 = 2;
  for (int y = 0; y < QK_K; y += 64) {
    uint8_t sc1, m1, sc2, m2;
    scale_min_k4(is, scales, &sc1, &m1);
    scale_min_k4(is + 1, scales, &sc2, &m2);
    float d1 = d * (float)sc1, mn1 = dmin * (float)m1;
    float d2 = d * (float)sc2, mn2 = dmin * (float)m2;
    for (int l = 0; l < 32; l++) {
      float hi = (qh[l] & u1) ? 16.0f : 0.0f;
      out[y + l] = d1 * ((float)(qs[qoff + l] & 0x0F) + hi) - mn1;
    }
    for (int l = 0; l < 32; l++) {
      float hi = (qh[l] & u2) ? 16.0f : 0.0f;
      out[y + 32 + l] = d2 * ((float)(qs[qoff + l] >> 4) + hi) - mn2;
    }
    qoff += 32;
    is += 2;
    u1 = (uint8_t)(u1 << 2);
    u2 = (uint8_t)(u2 << 2);
  }
}

static void deq_q6k_block(const uint8_t* blk, float* out) {
  const uint8_t* ql0 = blk;
  const uint8_t* qh0 = blk + 128;
  const int8_t* sc0 = (const int8_t*)(blk + 192);
  float d = kso_f16_to_f32(rd16(blk + 208));
  for (int half = 0; half < 2; half++) {
    const uint8_t* ql = ql0 + half * 64;
    const uint8_t* qh = qh0 + half * 32;
    const int8_t* sc = sc0 + half * 8;
    float* y = out + half * 128;
    for (int l = 0; l < 32; l++) {
      int is = l / 16;
      int q1 = ((ql[l] & 0x0F) | (((qh[l] >> 0) & 3) << 4)) - 32;
      int q2 = ((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32;
      int q3 = ((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
      int q4 = ((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
      y[l] = d * (float)sc[is] * (float)q1;
      y[l + 32] = d * (float)sc[is + 2] * (float)q2;
      y[l + 64] = d * (float)sc[is + 4] * (float)q3;
      y[l + 96] = d * (float)sc[is + 6] * (float)q4;
    }
  }
}

/* dtype codes shared with the CUDA library's public header */
enum { KS_F32 = 0, KS_F16 = 1, KS_Q4K = 2, KS_Q6K = 3, KS_Q40 = 4, KS_Q5K = 5 };

size_t kso_block_bytes(int dtype) {
  return dtype == KS_Q4K ? Q4K_BS : dtype == KS_Q6K ? Q6K_BS : dtype == KS_Q40 ? Q40_BS : dtype == KS_Q5K ? 176 : 0;
}
size_t kso_block_elems(int dtype) { return dtype == KS_Q40 ? 32 : QK_K; }

/* Dequantise nelem elements (a multiple of the block size). Returns 0 / -1. */
int kso_dequant(int dtype, const uint8_t* src, size_t nelem, float* dst) {
  if (dtype == KS_Q4K) {
    if (nelem % QK_K) return -1;
    for (size_t b = 0; b < nelem / QK_K; b++) deq_q4k_block(src + b * Q4K_BS, dst + b * QK_K);
  } else if (dtype == KS_Q6K) {
    if (nelem % QK_K) return -1;
    for (size_t b = 0; b < nelem / QK_K; b++) deq_q6k_block(src + b * Q6K_BS, dst + b * QK_K);
  } else if (dtype == KS_Q5K) {
    if (nelem % QK_K) return -1;
    for (size_t b = 0; b < nelem / QK_K; b++) deq_q5k_block(src + b * 176, dst + b * QK_K);
  } else if (dtype == KS_Q40) {
    if (nelem % 32) return -1;
    for (size_t b = 0; b < nelem / 32; b++) deq_q40_block(src + b * Q40_BS, dst + b * 32);
  } else if (dtype == KS_F16) {
    kso_f16_to_f32_n((const uint16_t*)src, dst, nelem);
  } else if (dtype == KS_F32) {
    memcpy(dst, src, nelem * 4);
  } else {
    return -1;
  }
  return 0;
}

/* ---- Q4_K reference quantizer (gguf_impl.rs:803-1016) ------------------- */
static inline int nearest_int(float f) {
  float v = f + 12582912.0f;
  int32_t i;
  memcpy(&i, &v, 4);
  return (i & 0x007fffff) - 0x00400000;
}
static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : v > hi ? hi : v; }

static float qkx2_search(int n, int nmax, const float* x, const float* w, uint8_t* L, float* the_min,
                         uint8_t* Laux, float rmin, float rdelta, int nstep) {
  float mn = x[0], mx = x[0];
  float sum_w = w[0], sum_x = sum_w * x[0];
  for (int i = 1; i < n; i++) {
    if (x[i] < mn) mn = x[i];
    if (x[i] > mx) mx = x[i];
    sum_w += w[i];
    sum_x += w[i] * x[i];
  }
  if (mn > 0.0f) mn = 0.0f;
  if (mx == mn) {
    for (int i = 0; i < n; i++) L[i] = 0;
    *the_min = -mn;
    return 0.0f;
  }
  float iscale = (float)nmax / (mx - mn);
  float scale = 1.0f / iscale;
  float best = 0.0f;
  for (int i = 0; i < n; i++) {
    int l = clampi(nearest_int(iscale * (x[i] - mn)), 0, nmax);
    L[i] = (uint8_t)l;
    float diff = scale * (float)l + mn - x[i];
    best += w[i] * (diff * diff);
  }
  if (nstep < 1) {
    *the_min = -mn;
    return scale;
  }
  for (int is = 0; is <= nstep; is++) {
    iscale = (rmin + rdelta * (float)is + (float)nmax) / (mx - mn);
    float sl = 0.0f, sl2 = 0.0f, sxl = 0.0f;
    for (int i = 0; i < n; i++) {
      int l = clampi(nearest_int(iscale * (x[i] - mn)), 0, nmax);
      Laux[i] = (uint8_t)l;
      float lf = (float)l;
      sl += w[i] * lf;
      sl2 += w[i] * lf * lf;
      sxl += w[i] * lf * x[i];
    }
    float D = sum_w * sl2 - sl * sl;
    if (D > 0.0f) {
      float ts = (sum_w * sxl - sum_x * sl) / D;
      float tm = (sl2 * sum_x - sl * sxl) / D;
      if (tm > 0.0f) {
        tm = 0.0f;
        ts = sxl / sl2;
      }
      float err = 0.0f;
      for (int i = 0; i < n; i++) {
        float diff = ts * (float)Laux[i] + tm - x[i];
        err += w[i] * (diff * diff);
      }
      if (err < best) {
        memcpy(L, Laux, (size_t)n);
        best = err;
        scale = ts;
        mn = tm;
      }
    }
  }
  *the_min = -mn;
  return scale;
}

/* elems: n f32 (n % 256 == 0) -> out: n/256*144 bytes. Returns 0 / -1. */
int kso_quantize_q4k(const float* elems, size_t n, uint8_t* out) {
  if (n % QK_K) return -1;
  size_t nb = n / QK_K;
  uint8_t L[QK_K], Laux[32];
  float weights[32], mins[8], scales[8];
  memset(out, 0, nb * Q4K_BS);
  for (size_t b = 0; b < nb; b++) {
    const float* x = elems + b * QK_K;
    uint8_t* blk = out + b * Q4K_BS;
    float max_scale = 0.0f, max_min = 0.0f;
    for (int j = 0; j < 8; j++) {
      const float* xs = x + 32 * j;
      float s2 = 0.0f;
      for (int t = 0; t < 32; t++) s2 += xs[t] * xs[t];
      float av = sqrtf(s2 / 32.0f);
      for (int t = 0; t < 32; t++) weights[t] = av + fabsf(xs[t]);
      scales[j] = qkx2_search(32, 15, xs, weights, L + 32 * j, &mins[j], Laux, -1.0f, 0.1f, 20);
      if (scales[j] > max_scale) max_scale = scales[j];
      if (mins[j] > max_min) max_min = mins[j];
    }
    float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
    float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
    uint16_t db = kso_f32_to_f16_ref(max_scale / 63.0f);
    uint16_t mb = kso_f32_to_f16_ref(max_min / 63.0f);
    blk[0] = (uint8_t)db; blk[1] = (uint8_t)(db >> 8);
    blk[2] = (uint8_t)mb; blk[3] = (uint8_t)(mb >> 8);
    uint8_t* sc = blk + 4;
    for (int j = 0; j < 8; j++) {
      uint8_t ls = (uint8_t)nearest_int(inv_scale * scales[j]);
      uint8_t lm = (uint8_t)nearest_int(inv_min * mins[j]);
      if (ls > 63) ls = 63;
      if (lm > 63) lm = 63;
      if (j < 4) {
        sc[j] = ls;
        sc[j + 4] = lm;
      } else {
        sc[j + 4] = (uint8_t)((ls & 0x0F) | ((lm & 0x0F) << 4));
        sc[j - 4] |= (uint8_t)((ls >> 4) << 6);
        sc[j] |= (uint8_t)((lm >> 4) << 6);
      }
    }
    float d = kso_f16_to_f32(rd16(blk));
    float dmin = kso_f16_to_f32(rd16(blk + 2));
    for (int j = 0; j < 8; j++) {
      uint8_t s, m;
      scale_min_k4(j, sc, &s, &m);
      float dj = d * (float)s;
      if (dj == 0.0f) continue;
      float dm = dmin * (float)m;
      for (int ii = 0; ii < 32; ii++)
        L[32 * j + ii] = (uint8_t)clampi(nearest_int((x[32 * j + ii] + dm) / dj), 0, 15);
    }
    uint8_t* qs = blk + 16;
    for (int j = 0, qoff = 0; j < QK_K; j += 64, qoff += 32)
      for (int t = 0; t < 32; t++) qs[qoff + t] = (uint8_t)(L[j + t] | (L[j + t + 32] << 4));
  }
  return 0;
}

/* ---- matvec: dequant then sequential f32 dot (check_mul_mm.rs:60-71) ---- */
/* y32: f32 sequential accumulation exactly as the reference's check does it;
 * y64: same products summed in f64 (the value both sides are judged against
 * when the tolerance is tighter than f32 summation noise). Either may be NULL.
 * x is [n_tok, cols], y is [n_tok, rows]. Row-parallel with OpenMP. */
int kso_matvec(int dtype, const uint8_t* W, size_t rows, size_t cols, const float* x, size_t n_tok,
               float* y32, double* y64) {
  size_t be = kso_block_elems(dtype), bb = kso_block_bytes(dtype);
  if (!bb || cols % be) return -1;
  size_t row_bytes = cols / be * bb;
  int rc = 0;
#pragma omp parallel
  {
    float* wd = (float*)malloc(cols * sizeof(float));
#pragma omp for schedule(static)
    for (long r = 0; r < (long)rows; r++) {
      if (kso_dequant(dtype, W + (size_t)r * row_bytes, cols, wd)) { rc = -1; continue; }
      for (size_t t = 0; t < n_tok; t++) {
        const float* xt = x + t * cols;
        if (y32) {
          float s = 0.0f;
          for (size_t c = 0; c < cols; c++) s += wd[c] * xt[c];
          y32[t * rows + r] = s;
        }
        if (y64) {
          double s = 0.0;
          for (size_t c = 0; c < cols; c++) s += (double)wd[c] * (double)xt[c];
          y64[t * rows + r] = s;
        }
      }
    }
    free(wd);
  }
  return rc;
}

/* Timed-baseline form "as the reference does it": dequantise the WHOLE matrix
 * to f32 first (wd must hold rows*cols floats), then dot (check_mul_mm.rs:61-71). */
int kso_matvec_two_pass(int dtype, const uint8_t* W, size_t rows, size_t cols, const float* x,
                        float* wd, float* y) {
  size_t be = kso_block_elems(dtype), bb = kso_block_bytes(dtype);
  if (!bb || cols % be) return -1;
  size_t row_bytes = cols / be * bb;
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows; r++) kso_dequant(dtype, W + (size_t)r * row_bytes, cols, wd + (size_t)r * cols);
#pragma omp parallel for schedule(static)
  for (long r = 0; r < (long)rows; r++) {
    float s = 0.0f;
    const float* wr = wd + (size_t)r * cols;
    for (size_t c = 0; c < cols; c++) s += wr[c] * x[c];
    y[r] = s;
  }
  return 0;
}

/* ---- tanh-GELU(gate) * up (lower.rs:2926-2954) -------------------------- */
float kso_gelu_mul(float g, float u) {
  float ax = fminf(20.0f, fmaxf(-20.0f, g));
  float t = 0.79788456f * (ax + 0.044715f * ((ax * ax) * ax));
  float gelu = (0.5f * ax) * (1.0f + tanhf(t));
  return gelu * u;
}
void kso_gelu_mul_n(const float* g, const float* u, float* out, size_t n) {
  for (size_t i = 0; i < n; i++) out[i] = kso_gelu_mul(g[i], u[i]);
}

/* ---- RMSNorm family (lower.rs:4079-4162): y = (x*inv)*w [+res] [*scale] - */
static float rms_inv(const float* x, size_t n, float eps) {
  double ss = 0.0; /* the shader's tree reduction has no CPU-defined order: sum in f64 */
  for (size_t i = 0; i < n; i++) ss += (double)(x[i] * x[i]);
  return 1.0f / sqrtf((float)ss / (float)n + eps);
}
void kso_rmsnorm(const float* x, const float* w, const float* res, int has_scale, float scale,
                 size_t n, size_t rows, float eps, float* y) {
  for (size_t r = 0; r < rows; r++) {
    const float* xr = x + r * n;
    float inv = rms_inv(xr, n, eps);
    for (size_t i = 0; i < n; i++) {
      float v = (xr[i] * inv) * (w ? w[i] : 1.0f);
      if (res) v = v + res[r * n + i];
      if (has_scale) v = scale * v;
      y[r * n + i] = v;
    }
  }
}
/* lower.rs:3926-4077: out_x = res + (y*inv)*w_post ; out_x2 = (out_x*inv2)*w_ffn */
void kso_rmsnorm_add_then_rmsnorm(const float* y, const float* w_post, const float* res,
                                  const float* w_ffn, size_t n, size_t rows, float eps,
                                  float* out_x, float* out_x2) {
  for (size_t r = 0; r < rows; r++) {
    const float* yr = y + r * n;
    float inv = rms_inv(yr, n, eps);
    float* ox = out_x + r * n;
    for (size_t i = 0; i < n; i++) ox[i] = res[r * n + i] + (yr[i] * inv) * w_post[i];
    float inv2 = rms_inv(ox, n, eps);
    for (size_t i = 0; i < n; i++) out_x2[r * n + i] = (ox[i] * inv2) * w_ffn[i];
  }
}

/* ---- Q4_0 pack (render.rs:1021-1059) ------------------------------------ */
/* through_half != 0: first round every value through f16 (the `_th` variant
 * used when packing from registers, render.rs:1046). */
void kso_pack_q40(const float* src, size_t n, int through_half, uint8_t* dst) {
  for (size_t b = 0; b < n / 32; b++) {
    float vals[32], max_abs = 0.0f;
    for (int d = 0; d < 32; d++) {
      float v = src[b * 32 + d];
      if (through_half) v = kso_f16_to_f32(kso_f32_to_f16_rne(v));
      vals[d] = v;
      max_abs = fmaxf(max_abs, fabsf(v));
    }
    float scale = max_abs > 0.0f ? max_abs / 7.0f : 1.0f;
    float inv = 1.0f / scale;
    uint8_t* blk = dst + b * Q40_BS;
    uint16_t hs = kso_f32_to_f16_rne(scale);
    blk[0] = (uint8_t)hs;
    blk[1] = (uint8_t)(hs >> 8);
    for (int i = 0; i < 16; i++) {
      int lo = clampi((int)roundf(vals[i] * inv) + 8, 0, 15);
      int hi = clampi((int)roundf(vals[i + 16] * inv) + 8, 0, 15);
      blk[2 + i] = (uint8_t)(lo | (hi << 4));
    }
  }
}

/* ---- RoPE table (gemma_prim.rs:33-56): per pos hd f32 = cos[half] || sin[half] */
void kso_rope_table(size_t max_seq, size_t hd, float theta, size_t rope_angles, float* out) {
  size_t half = hd / 2;
  if (rope_angles > half) rope_angles = half;
  for (size_t pos = 0; pos < max_seq; pos++) {
    for (size_t i = 0; i < half; i++) {
      if (i < rope_angles) {
        float freq = (float)(1.0 / pow((double)theta, (double)(2 * i) / (double)hd));
        float ang = (float)pos * freq;
        out[pos * hd + i] = cosf(ang);
        out[pos * hd + half + i] = sinf(ang);
      } else {
        out[pos * hd + i] = 1.0f;
        out[pos * hd + half + i] = 0.0f;
      }
    }
  }
}

/* ---- per-head RMS + RoPE (Q) / + Q4_0 pack (K, V) (lower.rs:4231-4702) --- */
/* q,k,v: [n_tok, heads, hd] f32. rope: table rows for these tokens, [n_tok, hd].
 * q_out f32 [n_tok, n_q, hd]; kv_k/kv_v: packed rows written at
 * kv_byte_off + (tok*n_kv + head) * hd/32*18.  V: RMS without weight. */
void kso_rmsnorm_per_head_qkv_q40(size_t n_q, size_t n_kv, size_t hd, size_t n_tok, float eps,
                                  const float* q, const float* qw, const float* rope,
                                  const float* k, const float* kw, const float* v, float* q_out,
                                  uint8_t* kv_k, uint8_t* kv_v, size_t kv_byte_off) {
  size_t half = hd / 2, rowb = hd / 32 * Q40_BS;
  float* tmp = (float*)malloc(hd * sizeof(float));
  for (size_t t = 0; t < n_tok; t++) {
    const float* cs = rope + t * hd;
    for (size_t h = 0; h < n_q; h++) {
      const float* xr = q + (t * n_q + h) * hd;
      float inv = rms_inv(xr, hd, eps);
      float* o = q_out + (t * n_q + h) * hd;
      for (size_t i = 0; i < half; i++) {
        float u = (xr[i] * inv) * qw[i];
        float w = (xr[half + i] * inv) * qw[half + i];
        float c = cs[i], s = cs[half + i];
        float lo = u * c - w * s, hi = u * s + w * c;
        o[i] = lo;
        o[half + i] = hi;
      }
    }
    for (size_t h = 0; h < n_kv; h++) {
      const float* xr = k + (t * n_kv + h) * hd;
      float inv = rms_inv(xr, hd, eps);
      for (size_t i = 0; i < half; i++) {
        float u = (xr[i] * inv) * kw[i];
        float w = (xr[half + i] * inv) * kw[half + i];
        float c = cs[i], s = cs[half + i];
        tmp[i] = u * c - w * s;
        tmp[half + i] = u * s + w * c;
      }
      kso_pack_q40(tmp, hd, 1, kv_k + kv_byte_off + (t * n_kv + h) * rowb);
      const float* vr = v + (t * n_kv + h) * hd;
      float invv = rms_inv(vr, hd, eps);
      for (size_t i = 0; i < hd; i++) tmp[i] = vr[i] * invv;
      kso_pack_q40(tmp, hd, 1, kv_v + kv_byte_off + (t * n_kv + h) * rowb);
    }
  }
  free(tmp);
}

/* ---- decode attention over a Q4_0 cache ---------------------------------- */
/* One query token. K/V logical layout [max_t, n_kv, hd] packed Q4_0.
 * Positions start..start+tlen-1.  Scores s = scale * (q . K_t); the reference
 * applies no scale (scale == 1, lower.rs:5284-5299).
 * nwg == 0: single-pass online softmax (lower.rs:4897-5359).
 * nwg  > 0: nwg partitions of ceil(tlen/nwg) positions, partials (m,l,O) with
 *           m initialised to -1e30, merged in partition order (lower.rs:5367-6088). */
static void attn_range(const float* qh, const uint8_t* K, const uint8_t* V, size_t n_kv, size_t kvh,
                       size_t hd, size_t start, size_t p0, size_t p1, float scale, float* m_io,
                       float* l_io, float* O, float* krow, float* vrow) {
  size_t rowb = hd / 32 * Q40_BS;
  float m = *m_io, l = *l_io;
  for (size_t t = p0; t < p1; t++) {
    size_t row = (start + t) * n_kv + kvh;
    kso_dequant(KS_Q40, K + row * rowb, hd, krow);
    kso_dequant(KS_Q40, V + row * rowb, hd, vrow);
    double acc = 0.0; /* lane-split + simd_sum order is device-specific: sum in f64 */
    for (size_t d = 0; d < hd; d++) acc += (double)(qh[d] * krow[d]);
    float s = (float)acc * scale;
    float m2 = fmaxf(m, s);
    float alpha = expf(m - m2);
    float e = expf(s - m2);
    l = l * alpha + e;
    m = m2;
    for (size_t d = 0; d < hd; d++) O[d] = O[d] * alpha + e * vrow[d];
  }
  *m_io = m;
  *l_io = l;
}

void kso_sdpa_decode(size_t n_q, size_t n_kv, size_t hd, const float* q, const uint8_t* K,
                     const uint8_t* V, size_t tlen, size_t start, float scale, size_t nwg,
                     float* out) {
  size_t groups = n_q / n_kv;
  float* krow = (float*)malloc(hd * 4);
  float* vrow = (float*)malloc(hd * 4);
  float* O = (float*)malloc(hd * 4);
  float* Op = (float*)malloc(hd * 4);
  for (size_t h = 0; h < n_q; h++) {
    size_t kvh = h / groups;
    const float* qh = q + h * hd;
    float m = -1.0e30f, l = 0.0f;
    for (size_t d = 0; d < hd; d++) O[d] = 0.0f;
    if (nwg == 0) {
      attn_range(qh, K, V, n_kv, kvh, hd, start, 0, tlen, scale, &m, &l, O, krow, vrow);
    } else {
      size_t chunk = (tlen + nwg - 1) / nwg;
      for (size_t p = 0; p < nwg; p++) {
        size_t p0 = p * chunk, p1 = p0 + chunk < tlen ? p0 + chunk : tlen;
        float mp = -1.0e30f, lp = 0.0f;
        for (size_t d = 0; d < hd; d++) Op[d] = 0.0f;
        if (p0 < p1) attn_range(qh, K, V, n_kv, kvh, hd, start, p0, p1, scale, &mp, &lp, Op, krow, vrow);
        float m2 = fmaxf(m, mp);
        float alpha = expf(m - m2), beta = expf(mp - m2);
        l = l * alpha + lp * beta;
        m = m2;
        for (size_t d = 0; d < hd; d++) O[d] = O[d] * alpha + Op[d] * beta;
      }
    }
    float inv_l = 1.0f / l;
    for (size_t d = 0; d < hd; d++) out[h * hd + d] = O[d] * inv_l;
  }
  free(krow); free(vrow); free(O); free(Op);
}

/* ---- embedding gather (lower.rs:3899-3924): dst = scale * deq(src)[id*n..] */
int kso_copy_scale_indexed(int dtype, const uint8_t* src, size_t n, const float* idx, size_t batch,
                           float scale, float* dst) {
  size_t be = kso_block_elems(dtype), bb = kso_block_bytes(dtype);
  for (size_t b = 0; b < batch; b++) {
    size_t id = (size_t)(uint32_t)idx[b];
    if (bb) {
      if (n % be) return -1;
      if (kso_dequant(dtype, src + id * (n / be * bb), n, dst + b * n)) return -1;
    } else if (dtype == KS_F16) {
      kso_f16_to_f32_n((const uint16_t*)src + id * n, dst + b * n, n);
    } else {
      memcpy(dst + b * n, (const float*)src + id * n, n * 4);
    }
    for (size_t i = 0; i < n; i++) dst[b * n + i] = scale * dst[b * n + i];
  }
  return 0;
}

/* ---- softcap argmax (lower.rs:6090-6157, render.rs:2346-2389) ------------ */
/* v = cap*tanh(x/cap); larger v wins, ties go to the LOWER index; the index is
 * returned as f32 like the shader writes it. best starts at (-1e30, 0). */
float kso_softcap_argmax(const float* x, size_t n, float cap, float* best_val) {
  float bv = -1.0e30f;
  size_t bi = 0;
  for (size_t i = 0; i < n; i++) {
    float v = cap * tanhf(x[i] / cap);
    if (v > bv) { bv = v; bi = i; }
  }
  if (best_val) *best_val = bv;
  return (float)bi;
}

/* ======================================================================== */
/* CPU fp32 decoder for the synthetic dense model: the op order of
 * forward_token (gemma_prim.rs:881-1275) for layers that own their KV, no
 * PLE, no sliding window.  Weights stay packed; activations f32.            */
typedef struct {
  int n_layers, hidden, ffn, n_q, n_kv, hd, vocab, max_seq;
  float eps, rope_theta, softcap, attn_scale;
  int embd_dtype;             /* KS_Q6K or KS_Q4K, tied lm_head */
  const uint8_t* token_embd;  /* [vocab, hidden] packed */
  const float* output_norm;   /* [hidden] */
  /* per layer arrays of pointers (length n_layers) */
  const uint8_t** wq; const uint8_t** wk; const uint8_t** wv; const uint8_t** wo;
  const uint8_t** wgate; const uint8_t** wup; const uint8_t** wdown;
  const float** attn_norm; const float** q_norm; const float** k_norm;
  const float** post_attn_norm; const float** ffn_norm; const float** post_ffw_norm;
  /* sliding-window layers (gemma_prim.rs:1009-1016): layer l with bit l of swa_layers set attends to the last
   * sliding_window positions only; 0 = every layer is full attention */
  int sliding_window;
  unsigned long long swa_layers;
} kso_model;

typedef struct {
  const kso_model* m;
  uint8_t** kv_k; uint8_t** kv_v; /* per layer [max_seq, n_kv, hd] Q4_0 */
  float* rope;                    /* [max_seq, hd] */
  float *x, *x2, *q, *k, *v, *o, *ff, *logits;
  int pos;
} kso_state;

kso_state* kso_state_new(const kso_model* m) {
  kso_state* s = (kso_state*)calloc(1, sizeof(kso_state));
  s->m = m;
  size_t rowb = (size_t)m->hd / 32 * Q40_BS;
  s->kv_k = (uint8_t**)calloc((size_t)m->n_layers, sizeof(void*));
  s->kv_v = (uint8_t**)calloc((size_t)m->n_layers, sizeof(void*));
  for (int l = 0; l < m->n_layers; l++) {
    s->kv_k[l] = (uint8_t*)calloc((size_t)m->max_seq * m->n_kv, rowb);
    s->kv_v[l] = (uint8_t*)calloc((size_t)m->max_seq * m->n_kv, rowb);
  }
  s->rope = (float*)malloc((size_t)m->max_seq * m->hd * 4);
  kso_rope_table((size_t)m->max_seq, (size_t)m->hd, m->rope_theta, (size_t)m->hd / 2, s->rope);
  s->x = (float*)calloc((size_t)m->hidden, 4);
  s->x2 = (float*)calloc((size_t)m->hidden, 4);
  s->q = (float*)calloc((size_t)m->n_q * m->hd, 4);
  s->k = (float*)calloc((size_t)m->n_kv * m->hd, 4);
  s->v = (float*)calloc((size_t)m->n_kv * m->hd, 4);
  s->o = (float*)calloc((size_t)m->n_q * m->hd, 4);
  s->ff = (float*)calloc((size_t)m->ffn * 2, 4);
  s->logits = (float*)calloc((size_t)m->vocab, 4);
  return s;
}
void kso_state_free(kso_state* s) {
  if (!s) return;
  for (int l = 0; l < s->m->n_layers; l++) { free(s->kv_k[l]); free(s->kv_v[l]); }
  free(s->kv_k); free(s->kv_v); free(s->rope);
  free(s->x); free(s->x2); free(s->q); free(s->k); free(s->v); free(s->o); free(s->ff); free(s->logits);
  free(s);
}
void kso_state_reset(kso_state* s) { s->pos = 0; }
const float* kso_state_logits(const kso_state* s) { return s->logits; }
const float* kso_state_hidden(const kso_state* s) { return s->x; }
/* the decoder's cache rows of one layer, [max_seq, n_kv, hd] Q4_0; which: 0 = K, 1 = V */
uint8_t* kso_state_kv(const kso_state* s, int layer, int which) { return which ? s->kv_v[layer] : s->kv_k[layer]; }

/* One token through all layers; returns the greedy next token (softcap argmax),
 * or -1 when pos >= max_seq ("max_seq exceeded", gemma_prim.rs:882-884).
 * Matvecs use f64 accumulation (see kso_matvec) rounded to f32. */
int kso_forward_token(kso_state* s, int token, int want_logits) {
  const kso_model* m = s->m;
  if (s->pos >= m->max_seq) return -1;
  size_t H = (size_t)m->hidden, hd = (size_t)m->hd, nq = (size_t)m->n_q, nkv = (size_t)m->n_kv;
  size_t F = (size_t)m->ffn;
  size_t rowb = hd / 32 * Q40_BS;
  double* acc = (double*)malloc((F > (size_t)m->vocab ? F : (size_t)m->vocab) * 2 * sizeof(double));
  float idx = (float)token;
  kso_copy_scale_indexed(m->embd_dtype, m->token_embd, H, &idx, 1, sqrtf((float)H), s->x);
  for (int l = 0; l < m->n_layers; l++) {
    kso_rmsnorm(s->x, m->attn_norm[l], NULL, 0, 0.0f, H, 1, m->eps, s->x2);
    kso_matvec(KS_Q4K, m->wq[l], nq * hd, H, s->x2, 1, NULL, acc);
    for (size_t i = 0; i < nq * hd; i++) s->q[i] = (float)acc[i];
    kso_matvec(KS_Q4K, m->wk[l], nkv * hd, H, s->x2, 1, NULL, acc);
    for (size_t i = 0; i < nkv * hd; i++) s->k[i] = (float)acc[i];
    kso_matvec(KS_Q4K, m->wv[l], nkv * hd, H, s->x2, 1, NULL, acc);
    for (size_t i = 0; i < nkv * hd; i++) s->v[i] = (float)acc[i];
    kso_rmsnorm_per_head_qkv_q40(nq, nkv, hd, 1, m->eps, s->q, m->q_norm[l],
                                 s->rope + (size_t)s->pos * hd, s->k, m->k_norm[l], s->v, s->q,
                                 s->kv_k[l], s->kv_v[l], (size_t)s->pos * nkv * rowb);
    {
      /* kv_len = pos + 1; a sliding-window layer starts at kv_len - window (gemma_prim.rs:1009-1016) */
      size_t kv_len = (size_t)s->pos + 1, start = 0;
      if (m->sliding_window > 0 && ((m->swa_layers >> l) & 1ull) && kv_len > (size_t)m->sliding_window)
        start = kv_len - (size_t)m->sliding_window;
      kso_sdpa_decode(nq, nkv, hd, s->q, s->kv_k[l], s->kv_v[l], kv_len - start, start, m->attn_scale, 0, s->o);
    }
    kso_matvec(KS_Q4K, m->wo[l], H, nq * hd, s->o, 1, NULL, acc);
    for (size_t i = 0; i < H; i++) s->x2[i] = (float)acc[i];
    kso_rmsnorm_add_then_rmsnorm(s->x2, m->post_attn_norm[l], s->x, m->ffn_norm[l], H, 1, m->eps,
                                 s->x, s->x2);
    kso_matvec(KS_Q4K, m->wgate[l], F, H, s->x2, 1, NULL, acc);
    kso_matvec(KS_Q4K, m->wup[l], F, H, s->x2, 1, NULL, acc + F);
    for (size_t i = 0; i < F; i++) s->ff[i] = kso_gelu_mul((float)acc[i], (float)acc[F + i]);
    kso_matvec(KS_Q4K, m->wdown[l], H, F, s->ff, 1, NULL, acc);
    for (size_t i = 0; i < H; i++) s->x2[i] = (float)acc[i];
    kso_rmsnorm(s->x2, m->post_ffw_norm[l], s->x, 0, 0.0f, H, 1, m->eps, s->x);
  }
  s->pos += 1;
  int best = 0;
  if (want_logits) {
    kso_rmsnorm(s->x, m->output_norm, NULL, 0, 0.0f, H, 1, m->eps, s->x2);
    kso_matvec(m->embd_dtype, m->token_embd, (size_t)m->vocab, H, s->x2, 1, NULL, acc);
    for (size_t i = 0; i < (size_t)m->vocab; i++) s->logits[i] = (float)acc[i];
    best = (int)kso_softcap_argmax(s->logits, (size_t)m->vocab, m->softcap, NULL);
  }
  free(acc);
  return best;
}

// Device helpers shared by the matvec kernels: streaming loads, f32x2 arithmetic, the
// nibble -> f32 extraction, scale unpacking and the staging of x in shared memory.
#pragma once
#include "ks_internal.h"

#ifndef KS_F32X2
#define KS_F32X2 1
#endif

namespace {

constexpr float kMagic = 8388608.0f;  // 2^23
constexpr uint32_t kMagicBits = 0x4B000000u;

__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_stream_u16x2(const void* p) {
  // 4 bytes at a 2-byte aligned address
  unsigned short a, b;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(a) : "l"(p));
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1+2];" : "=h"(b) : "l"(p));
  return (uint32_t)a | ((uint32_t)b << 16);
}
__device__ __forceinline__ uint32_t ldg_stream_u16(const void* p) {
  unsigned short a;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(a) : "l"(p));
  return a;
}

__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
#if KS_F32X2
  unsigned long long A, B, D;
  asm("mov.b64 %0, {%1, %2};" : "=l"(A) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(B) : "f"(b.x), "f"(b.y));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(D) : "l"(A), "l"(B));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(D));
  return d;
#else
  return make_float2(a.x + b.x, a.y + b.y);
#endif
}
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
#if KS_F32X2
  unsigned long long A, B, Cc, D;
  asm("mov.b64 %0, {%1, %2};" : "=l"(A) : "f"(a.x), "f"(a.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(B) : "f"(b.x), "f"(b.y));
  asm("mov.b64 %0, {%1, %2};" : "=l"(Cc) : "f"(c.x), "f"(c.y));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(D) : "l"(A), "l"(B), "l"(Cc));
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(D));
  return d;
#else
  return make_float2(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y));
#endif
}

template <typename T>
__device__ __forceinline__ float act_load(const T* p, size_t i);
template <>
__device__ __forceinline__ float act_load<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float act_load<__half>(const __half* p, size_t i) { return __half2float(p[i]); }
template <typename T>
__device__ __forceinline__ void act_store(T* p, size_t i, float v);
template <>
__device__ __forceinline__ void act_store<float>(float* p, size_t i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void act_store<__half>(__half* p, size_t i, float v) { p[i] = __float2half_rn(v); }

// tanh-GELU(gate) * up, gate clamped to +-20 (lower.rs:2926-2954).
__device__ __forceinline__ float gelu_mul(float g, float u) {
  float ax = fminf(20.0f, fmaxf(-20.0f, g));
  float t = 0.79788456f * (ax + 0.044715f * ((ax * ax) * ax));
  float gelu = (0.5f * ax) * (1.0f + tanhf(t));
  return gelu * u;
}

struct MvArgs {
  const uint8_t* W[3];
  void* y[3];
  unsigned rows[3];
  unsigned tile_start[4];  // first tile index of each segment; [n_seg] = total tiles
  int n_seg;
  unsigned nb;         // super-blocks per row
  unsigned row_bytes;
  unsigned cols;
  const void* x;
  int n_tok;
  unsigned y_stride;   // elements between tokens of y: rows of the segment
};

// Kernel parameters live in constant memory; indexing them with a run-time value would force a
// local copy, so segment fields are picked with selects.
__device__ __forceinline__ const uint8_t* seg_w(const MvArgs& a, int s) { return s == 0 ? a.W[0] : s == 1 ? a.W[1] : a.W[2]; }
__device__ __forceinline__ void* seg_y(const MvArgs& a, int s) { return s == 0 ? a.y[0] : s == 1 ? a.y[1] : a.y[2]; }
__device__ __forceinline__ unsigned seg_rows_of(const MvArgs& a, int s) { return s == 0 ? a.rows[0] : s == 1 ? a.rows[1] : a.rows[2]; }
__device__ __forceinline__ unsigned seg_tile0(const MvArgs& a, int s) { return s == 0 ? a.tile_start[0] : s == 1 ? a.tile_start[1] : a.tile_start[2]; }
__device__ __forceinline__ unsigned total_tiles_of(const MvArgs& a) {
  return a.n_seg == 1 ? a.tile_start[1] : a.n_seg == 2 ? a.tile_start[2] : a.tile_start[3];
}

// -------------------------------------------------------------------------------------------
// Q4_K.  A "unit" is one 64-element group of a super-block: 32 bytes of nibbles (low nibbles =
// sub-block 2g, high nibbles = sub-block 2g+1) plus that group's two scales and mins.
// LPR lanes share a row (each takes every LPR-th unit); 32/LPR rows run side by side in a
// warp, and each lane keeps R such row sets going so one x fragment serves R rows.
// Shared memory: xp[unit][l] = (x_lo[l]*s, x_hi[l]*s/16), s = 1 for even l, 1/256 for odd l;
//                sx[unit]    = (sum x_lo, sum x_hi).
// -------------------------------------------------------------------------------------------
// Stage x for the Q4_K kernels.  Thread i takes 4 consecutive elements (always one sub-block:
// 8 neighbouring lanes cover its 32 elements), so every load is issued before anything waits
// and the sub-block sums need three shuffles instead of a pass over shared memory.
// Shared-memory layout of a staged x (Q4_K), per token: units * Q4K_XS floats of (lo, hi) pairs --
// 64 used per unit, padded to 68 so that the 8 lanes of a row, which read consecutive units with
// 16-byte loads, fall on different banks -- then units * 2 floats of sub-block sums.
constexpr unsigned Q4K_XS = 68;
constexpr unsigned Q4K_XTOK = Q4K_XS + 2;  // floats per unit per token
template <typename XT>
__device__ __forceinline__ void q4k_stage_x(unsigned char* smem, const XT* x, unsigned cols, int n_tok) {
  const unsigned units = cols >> 6;
  const unsigned nchunk = cols >> 2;
  for (int t = 0; t < n_tok; t++) {
    float* xp = reinterpret_cast<float*>(smem) + (size_t)t * units * Q4K_XTOK;
    float* sx = xp + (size_t)units * Q4K_XS;
    const XT* xt = x + (size_t)t * cols;
    // cols is a multiple of 256, so nchunk is a multiple of 64 and whole warps run every trip
    const bool vec_ok = (reinterpret_cast<uintptr_t>(xt) & (sizeof(XT) * 4 - 1)) == 0;
#pragma unroll 4
    for (unsigned c = threadIdx.x; c < nchunk; c += blockDim.x) {
      const bool live = true;
      float v0, v1, v2, v3;
      if (!vec_ok) {
        v0 = act_load<XT>(xt, (size_t)c * 4);
        v1 = act_load<XT>(xt, (size_t)c * 4 + 1);
        v2 = act_load<XT>(xt, (size_t)c * 4 + 2);
        v3 = act_load<XT>(xt, (size_t)c * 4 + 3);
      } else if (sizeof(XT) == 4) {
        const float4 v = reinterpret_cast<const float4*>(xt)[c];
        v0 = v.x; v1 = v.y; v2 = v.z; v3 = v.w;
      } else {
        const uint2 raw = reinterpret_cast<const uint2*>(xt)[c];
        const __half2 a = *reinterpret_cast<const __half2*>(&raw.x), b = *reinterpret_cast<const __half2*>(&raw.y);
        v0 = __low2float(a); v1 = __high2float(a); v2 = __low2float(b); v3 = __high2float(b);
      }
      const unsigned e = c << 2;
      const unsigned u = e >> 6, hi = (e >> 5) & 1u, l = e & 31u;  // l is a multiple of 4: even, odd, even, odd
      float s = (v0 + v1) + (v2 + v3);
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      if (live) {
        const float k0 = hi ? (1.0f / 16.0f) : 1.0f, k1 = hi ? (1.0f / 4096.0f) : (1.0f / 256.0f);
        float* dst = xp + (size_t)u * Q4K_XS + l * 2 + hi;
        dst[0] = v0 * k0;
        dst[2] = v1 * k1;
        dst[4] = v2 * k0;
        dst[6] = v3 * k1;
        if ((threadIdx.x & 7u) == 0) sx[(size_t)u * 2 + hi] = s;
      }
    }
  }
}

__device__ __forceinline__ float4 lds_f4(const void* p) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"((uint32_t)__cvta_generic_to_shared(p)));
  return v;
}
__device__ __forceinline__ uint4 lds_u4(const void* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"((uint32_t)__cvta_generic_to_shared(p)));
  return v;
}
__device__ __forceinline__ float2 lds_f2(const void* p) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"((uint32_t)__cvta_generic_to_shared(p)));
  return v;
}

// Eight nibbles of one 32-bit word against four (lo, hi) x pairs.
__device__ __forceinline__ void q4_word(uint32_t w, const float2 x0, const float2 x1, const float2 x2,
                                        const float2 x3, float2& acc0, float2& acc1) {
  const uint32_t h = w >> 16;
  const float2 neg = make_float2(-kMagic, -kMagic);
  float2 f0 = make_float2(__uint_as_float((w & 0x000Fu) | kMagicBits), __uint_as_float((w & 0x00F0u) | kMagicBits));
  float2 f1 = make_float2(__uint_as_float((w & 0x0F00u) | kMagicBits), __uint_as_float((w & 0xF000u) | kMagicBits));
  float2 f2 = make_float2(__uint_as_float((h & 0x000Fu) | kMagicBits), __uint_as_float((h & 0x00F0u) | kMagicBits));
  float2 f3 = make_float2(__uint_as_float((h & 0x0F00u) | kMagicBits), __uint_as_float((h & 0xF000u) | kMagicBits));
  acc0 = ffma2(fadd2(f0, neg), x0, acc0);
  acc1 = ffma2(fadd2(f1, neg), x1, acc1);
  acc0 = ffma2(fadd2(f2, neg), x2, acc0);
  acc1 = ffma2(fadd2(f3, neg), x3, acc1);
}

// Scales and mins of group g from the 12 packed bytes (gguf_impl.rs:563-573), as
// (sc_lo, sc_hi, m_lo, m_hi) for sub-blocks 2g and 2g+1.
__device__ __forceinline__ void q4k_group_scales(const uint4 hdr, int g, float& dsc_lo, float& dsc_hi,
                                                 float& dm_lo, float& dm_hi) {
  const __half2 dd = *reinterpret_cast<const __half2*>(&hdr.x);
  const float d = __low2float(dd), dmin = __high2float(dd);
  // 16-bit words of the scale field: s16[0..5]
  const uint32_t w0 = hdr.y, w1 = hdr.z, w2 = hdr.w;
  // s16[g] and s16[g+2] for g<2 ; s16[g+2], s16[g-2], s16[g] for g>=2
  uint32_t a, b;
  if (g < 2) {
    const uint32_t sg = (g == 0) ? (w0 & 0xFFFFu) : (w0 >> 16);
    const uint32_t sg2 = (g == 0) ? (w1 & 0xFFFFu) : (w1 >> 16);
    a = sg & 0x3F3Fu;
    b = sg2 & 0x3F3Fu;
  } else {
    const uint32_t sg2 = (g == 2) ? (w2 & 0xFFFFu) : (w2 >> 16);  // s16[g+2]
    const uint32_t sgm = (g == 2) ? (w0 & 0xFFFFu) : (w0 >> 16);  // s16[g-2]
    const uint32_t sg = (g == 2) ? (w1 & 0xFFFFu) : (w1 >> 16);   // s16[g]
    a = (sg2 & 0x0F0Fu) | ((sgm & 0xC0C0u) >> 2);
    b = ((sg2 >> 4) & 0x0F0Fu) | ((sg & 0xC0C0u) >> 2);
  }
  dsc_lo = d * (float)(a & 0xFFu);
  dsc_hi = d * (float)(a >> 8);
  dm_lo = dmin * (float)(b & 0xFFu);
  dm_hi = dmin * (float)(b >> 8);
}

// Shared-memory layout of a staged x (Q6_K), per token: four planes k = 0..3 of units float4
// (x[128h + 32k + 4*l4 + j] * p(j), p = 1, 2^-8, 2^-16, 1), then units float4 of the four sums.
// Plane-major so that lanes reading consecutive units with 16-byte loads do not share banks.
constexpr unsigned Q6K_XTOK = 20;  // floats per unit per token
template <typename XT>
__device__ __forceinline__ void q6k_stage_x(unsigned char* smem, const XT* x, unsigned cols, int n_tok) {
  const unsigned units = cols >> 4;  // 16 units per 256-element block
  for (int t = 0; t < n_tok; t++) {
    float4* xq = reinterpret_cast<float4*>(smem) + (size_t)t * units * 5;
    const XT* xt = x + (size_t)t * cols;
    for (unsigned u = threadIdx.x; u < units; u += blockDim.x) {
      const unsigned blk = u >> 4, h = (u >> 3) & 1, l4 = u & 7;
      const size_t e0 = (size_t)blk * 256 + h * 128 + l4 * 4;
      float s[4];
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const float v0 = act_load<XT>(xt, e0 + 32 * k + 0);
        const float v1 = act_load<XT>(xt, e0 + 32 * k + 1);
        const float v2 = act_load<XT>(xt, e0 + 32 * k + 2);
        const float v3 = act_load<XT>(xt, e0 + 32 * k + 3);
        xq[(size_t)k * units + u] = make_float4(v0, v1 * (1.0f / 256.0f), v2 * (1.0f / 65536.0f), v3);
        s[k] = (v0 + v1) + (v2 + v3);
      }
      xq[(size_t)4 * units + u] = make_float4(s[0], s[1], s[2], s[3]);
    }
  }
}

// Four 6-bit values in the bytes of v against (x0, x1/256, x2/65536, x3).
__device__ __forceinline__ float q6_word(uint32_t v, const float4 x) {
  const float2 neg = make_float2(-kMagic, -kMagic);
  float2 f01 = make_float2(__uint_as_float((v & 0x3Fu) | kMagicBits), __uint_as_float((v & 0x3F00u) | kMagicBits));
  float2 f23 = make_float2(__uint_as_float((v & 0x3F0000u) | kMagicBits), __uint_as_float((v >> 24) | kMagicBits));
  float2 acc = ffma2(fadd2(f01, neg), make_float2(x.x, x.y), make_float2(0.0f, 0.0f));
  acc = ffma2(fadd2(f23, neg), make_float2(x.z, x.w), acc);
  return acc.x + acc.y;
}

}  // namespace

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

// ---- fused input prologue -----------------------------------------------------------------------
// The matvec can apply the norm that precedes it while it stages x, instead of a kernel of its own:
//   KS_PRO_NORM     x2 = (x*inv)*w                      (Eng::rmsnorm_matvec*, K:264-416)
//   KS_PRO_ADD_NORM x' = res + (y*inv)*w_post ; x2 = (x'*inv2)*w_next   (K:539 followed by a matvec)
// Every block computes the same x2 (same order, same result); block 0 also writes x' to out_x, which
// must not alias res (other blocks may still be reading it).
typedef ks_mv_pro MvPro;
constexpr int KS_PRO_MAXC = 4;  // 4-element chunks per thread: cols <= 16 * blockDim

template <typename XT>
__device__ __forceinline__ float4 ld_chunk(const XT* p, unsigned c) {
  if (sizeof(XT) == 4) return reinterpret_cast<const float4*>(p)[c];
  const uint2 raw = reinterpret_cast<const uint2*>(p)[c];
  const __half2 a = *reinterpret_cast<const __half2*>(&raw.x), b = *reinterpret_cast<const __half2*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}
template <typename XT>
__device__ __forceinline__ void st_chunk(XT* p, unsigned c, float4 v) {
  if (sizeof(XT) == 4) {
    reinterpret_cast<float4*>(p)[c] = v;
  } else {
    const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&a);
    raw.y = *reinterpret_cast<const uint32_t*>(&b);
    reinterpret_cast<uint2*>(p)[c] = raw;
  }
}
__device__ __forceinline__ float block_sum_f(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? red[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}
// One 4-element chunk of x into the Q4_K staging layout (scaled pairs + sub-block sums).
__device__ __forceinline__ void q4k_put_chunk(float* xp, float* sx, unsigned c, float4 v) {
  const unsigned e = c << 2;
  const unsigned u = e >> 6, hi = (e >> 5) & 1u, l = e & 31u;
  float s = (v.x + v.y) + (v.z + v.w);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  const float k0 = hi ? (1.0f / 16.0f) : 1.0f, k1 = hi ? (1.0f / 4096.0f) : (1.0f / 256.0f);
  float* dst = xp + (size_t)u * Q4K_XS + l * 2 + hi;
  dst[0] = v.x * k0;
  dst[2] = v.y * k1;
  dst[4] = v.z * k0;
  dst[6] = v.w * k1;
  if ((threadIdx.x & 7u) == 0) sx[(size_t)u * 2 + hi] = s;
}
// Stage x with the prologue applied.  x: the input (NORM) or the residual stream (ADD_NORM).
// Waits for the previous kernel itself (griddepcontrol.wait) after it has fetched the norm weights.
// All pointers 16-byte aligned (8 for f16); cols <= 16 * blockDim; red: 32 floats of shared memory.
template <typename XT>
__device__ __forceinline__ void q4k_stage_x_pro(unsigned char* smem, float* red, const MvPro& p, const XT* x,
                                                unsigned cols, int n_tok) {
  const unsigned units = cols >> 6;
  const unsigned nchunk = cols >> 2;
  const float invn = 1.0f / (float)cols;
  // The norm weights are constants of the model: fetch them before waiting for the previous kernel,
  // so that after the wait only ONE round trip to memory (y and x together) is left.
  float4 wv[KS_PRO_MAXC], wpv[KS_PRO_MAXC];
#pragma unroll
  for (int k = 0; k < KS_PRO_MAXC; k++) {
    const unsigned c = threadIdx.x + k * blockDim.x;
    if (c < nchunk) {
      wv[k] = ld_chunk<XT>(reinterpret_cast<const XT*>(p.w), c);
      if (p.mode == KS_PRO_ADD_NORM) wpv[k] = ld_chunk<XT>(reinterpret_cast<const XT*>(p.w_post), c);
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int t = 0; t < n_tok; t++) {
    float* xp = reinterpret_cast<float*>(smem) + (size_t)t * units * Q4K_XTOK;
    float* sx = xp + (size_t)units * Q4K_XS;
    const XT* xt = x + (size_t)t * cols;
    float4 v[KS_PRO_MAXC];
    float ss = 0.0f;
    if (p.mode == KS_PRO_ADD_NORM) {
      const XT* yt = reinterpret_cast<const XT*>(p.y) + (size_t)t * cols;
      float4 yv[KS_PRO_MAXC];
#pragma unroll
      for (int k = 0; k < KS_PRO_MAXC; k++) {
        const unsigned c = threadIdx.x + k * blockDim.x;
        if (c < nchunk) {
          yv[k] = ld_chunk<XT>(yt, c);
          v[k] = ld_chunk<XT>(xt, c);
          ss = fmaf(yv[k].x, yv[k].x, ss); ss = fmaf(yv[k].y, yv[k].y, ss);
          ss = fmaf(yv[k].z, yv[k].z, ss); ss = fmaf(yv[k].w, yv[k].w, ss);
        }
      }
      ss = block_sum_f(ss, red);
      const float inv = 1.0f / sqrtf(ss * invn + p.eps);
      ss = 0.0f;
#pragma unroll
      for (int k = 0; k < KS_PRO_MAXC; k++) {
        const unsigned c = threadIdx.x + k * blockDim.x;
        if (c < nchunk) {
          const float4 wp = wpv[k];
          float4 r = v[k];
          r.x = __fadd_rn(r.x, __fmul_rn(__fmul_rn(yv[k].x, inv), wp.x));
          r.y = __fadd_rn(r.y, __fmul_rn(__fmul_rn(yv[k].y, inv), wp.y));
          r.z = __fadd_rn(r.z, __fmul_rn(__fmul_rn(yv[k].z, inv), wp.z));
          r.w = __fadd_rn(r.w, __fmul_rn(__fmul_rn(yv[k].w, inv), wp.w));
          if (blockIdx.x == 0) st_chunk<XT>(reinterpret_cast<XT*>(p.out_x) + (size_t)t * cols, c, r);
          if (sizeof(XT) == 2) {  // the next norm reads what was stored
            r.x = __half2float(__float2half_rn(r.x)); r.y = __half2float(__float2half_rn(r.y));
            r.z = __half2float(__float2half_rn(r.z)); r.w = __half2float(__float2half_rn(r.w));
          }
          v[k] = r;
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < KS_PRO_MAXC; k++) {
        const unsigned c = threadIdx.x + k * blockDim.x;
        if (c < nchunk) v[k] = ld_chunk<XT>(xt, c);
      }
    }
#pragma unroll
    for (int k = 0; k < KS_PRO_MAXC; k++) {
      const unsigned c = threadIdx.x + k * blockDim.x;
      if (c < nchunk) {
        ss = fmaf(v[k].x, v[k].x, ss); ss = fmaf(v[k].y, v[k].y, ss);
        ss = fmaf(v[k].z, v[k].z, ss); ss = fmaf(v[k].w, v[k].w, ss);
      }
    }
    ss = block_sum_f(ss, red);
    const float inv2 = 1.0f / sqrtf(ss * invn + p.eps);
#pragma unroll
    for (int k = 0; k < KS_PRO_MAXC; k++) {
      const unsigned c = threadIdx.x + k * blockDim.x;
      if (c < nchunk) {  // nchunk is a multiple of 64: whole warps take this branch together
        const float4 w = wv[k];
        float4 r;
        r.x = __fmul_rn(__fmul_rn(v[k].x, inv2), w.x);
        r.y = __fmul_rn(__fmul_rn(v[k].y, inv2), w.y);
        r.z = __fmul_rn(__fmul_rn(v[k].z, inv2), w.z);
        r.w = __fmul_rn(__fmul_rn(v[k].w, inv2), w.w);
        if (sizeof(XT) == 2) {  // the unfused path stores x2 in f16 before the matvec reads it
          r.x = __half2float(__float2half_rn(r.x)); r.y = __half2float(__float2half_rn(r.y));
          r.z = __half2float(__float2half_rn(r.z)); r.w = __half2float(__float2half_rn(r.w));
        }
        q4k_put_chunk(xp, sx, c, r);
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

// ---- f32x2 values kept packed in 64-bit registers end to end ------------------------------------
// (x pairs are loaded as 64-bit words and accumulators stay 64-bit, so the only packing left is
// the two extracted nibbles of one pair, which the register allocator can place side by side.)
typedef unsigned long long u64;
__device__ __forceinline__ u64 pack2(uint32_t lo, uint32_t hi) {
  u64 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ float2 unpack2(u64 v) {
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(v));
  return d;
}
__device__ __forceinline__ u64 padd2(u64 a, u64 b) {
  u64 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ u64 pfma2(u64 a, u64 b, u64 c) {
  u64 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
// 16 bytes of shared memory as two packed pairs
__device__ __forceinline__ void lds_p2(const void* p, u64& a, u64& b) {
  asm volatile("ld.shared.v2.b64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
constexpr u64 kNegMagic2 = 0xCB000000CB000000ull;  // (-2^23, -2^23)
// Eight nibbles of one 32-bit word against four packed (lo, hi) x pairs.
__device__ __forceinline__ void q4_word_p(uint32_t w, u64 x0, u64 x1, u64 x2, u64 x3, u64& acc0, u64& acc1) {
  // The word is duplicated into both halves of a 64-bit register once; each pair of nibbles is then
  // one 64-bit and/or (two LOP3 on the register pair), which lands already packed for f32x2.
  constexpr u64 M2 = ((u64)kMagicBits << 32) | kMagicBits;
  const u64 ww = pack2(w, w);
  const u64 hh = pack2(w >> 16, w >> 16);
  const u64 f0 = (ww & 0x000000F00000000Full) | M2;
  const u64 f1 = (ww & 0x0000F00000000F00ull) | M2;
  const u64 f2 = (hh & 0x000000F00000000Full) | M2;
  const u64 f3 = (hh & 0x0000F00000000F00ull) | M2;
  acc0 = pfma2(padd2(f0, kNegMagic2), x0, acc0);
  acc1 = pfma2(padd2(f1, kNegMagic2), x1, acc1);
  acc0 = pfma2(padd2(f2, kNegMagic2), x2, acc0);
  acc1 = pfma2(padd2(f3, kNegMagic2), x3, acc1);
}
// Four 6-bit values in the bytes of v against (x0, x1/256) and (x2/65536, x3), packed.
__device__ __forceinline__ float q6_word_p(uint32_t v, u64 x01, u64 x23) {
  constexpr u64 M2 = ((u64)kMagicBits << 32) | kMagicBits;
  const u64 f01 = (pack2(v, v) & 0x00003F000000003Full) | M2;
  const u64 f23 = (pack2(v, v >> 8) & 0x003F0000003F0000ull) | M2;  // byte 2 in place, byte 3 moved to byte 2
  u64 acc = pfma2(padd2(f01, kNegMagic2), x01, 0ull);
  acc = pfma2(padd2(f23, kNegMagic2), x23, acc);
  const float2 r = unpack2(acc);
  return r.x + r.y;
}

// Shared loads through a 32-bit shared-space address plus a compile-time byte offset, so one
// address register serves a whole fragment.
template <int OFF>
__device__ __forceinline__ void lds_p2o(uint32_t a, u64& x, u64& y) {
  asm volatile("ld.shared.v2.b64 {%0,%1}, [%2+%3];" : "=l"(x), "=l"(y) : "r"(a), "n"(OFF));
}
template <int OFF>
__device__ __forceinline__ uint4 lds_u4o(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a), "n"(OFF));
  return v;
}
__device__ __forceinline__ float2 lds_f2a(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
  return v;
}

// Scales and mins of group g (sub-blocks 2g, 2g+1) without a branch: the 12 scale bytes are six
// 16-bit words h0..h5 (gguf_impl.rs:563-573); with p = g & 1,
//   g < 2 : (sc_lo, sc_hi) = h[p] & 0x3f3f,                      (m_lo, m_hi) = h[2+p] & 0x3f3f
//   g >= 2: (sc_lo, sc_hi) = (h[4+p] & 0x0f0f) | ((h[p] & 0xc0c0) >> 2),
//           (m_lo, m_hi)   = ((h[4+p] >> 4) & 0x0f0f) | ((h[2+p] & 0xc0c0) >> 2).
// Returns y += d*(sc_lo*a_lo + sc_hi*a_hi) - dmin*(m_lo*sx_lo + m_hi*sx_hi).
__device__ __forceinline__ float q4k_apply_scales(const uint4 hdr, int g, float a_lo, float a_hi, float sx_lo,
                                                  float sx_hi, float y) {
  const unsigned sh = (g & 1) * 16;
  const uint32_t hA = (hdr.y >> sh) & 0xFFFFu, hB = (hdr.z >> sh) & 0xFFFFu, hC = (hdr.w >> sh) & 0xFFFFu;
  const uint32_t a_small = hA & 0x3F3Fu, b_small = hB & 0x3F3Fu;
  const uint32_t a_big = (hC & 0x0F0Fu) | ((hA & 0xC0C0u) >> 2);
  const uint32_t b_big = ((hC >> 4) & 0x0F0Fu) | ((hB & 0xC0C0u) >> 2);
  const uint32_t av = g < 2 ? a_small : a_big, bv = g < 2 ? b_small : b_big;
  const __half2 dd = *reinterpret_cast<const __half2*>(&hdr.x);
  const float d = __low2float(dd), dmin = __high2float(dd);
  float t1 = (float)(av & 0xFFu) * a_lo;
  t1 = fmaf((float)(av >> 8), a_hi, t1);
  float t2 = (float)(bv & 0xFFu) * sx_lo;
  t2 = fmaf((float)(bv >> 8), sx_hi, t2);
  y = fmaf(d, t1, y);
  return fmaf(-dmin, t2, y);
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
// (x[128h + 32k + 4*l4 + j] * p(j), p = 1, 2^-8, 2^-16, 2^-16), then units float4 of the four sums.
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
        xq[(size_t)k * units + u] = make_float4(v0, v1 * (1.0f / 256.0f), v2 * (1.0f / 65536.0f), v3 * (1.0f / 65536.0f));
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
  float2 f23 = make_float2(__uint_as_float((v & 0x3F0000u) | kMagicBits), __uint_as_float(((v >> 8) & 0x3F0000u) | kMagicBits));
  float2 acc = ffma2(fadd2(f01, neg), make_float2(x.x, x.y), make_float2(0.0f, 0.0f));
  acc = ffma2(fadd2(f23, neg), make_float2(x.z, x.w), acc);
  return acc.x + acc.y;
}

}  // namespace

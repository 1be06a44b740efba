// Device helpers shared by the kernels that multiply Q4_K rows out of shared memory against a
// fixed-point x (the persistent decode kernel and the stand-alone fixed-point matvec): mbarrier and
// bulk-copy wrappers, the staging of x as three byte planes, and the lane-per-unit dot product.
#pragma once
#include "ks_mv_common.cuh"

namespace {

__device__ __forceinline__ uint32_t sm32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mb_init(uint32_t bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mb_expect(uint32_t bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mb_wait(uint32_t bar, unsigned parity, unsigned limit) {
  for (unsigned i = 0; i < limit; i++) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void bulk_in(uint32_t dst, const void* src, unsigned bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// ---- x as 24-bit block fixed point, weights x x as byte dot products ----------------------------
// Each 32-element sub-block of the staged vector shares a scale s; element i is the integer
// X_i = round(x_i / s), |X_i| <= 8e6, kept as three byte planes (X = l2*65536 + l1*256 + l0, l2
// signed).  Four neighbouring nibbles of a weight word, masked in place, are the other operand of a
// dp4a, so 4 weights cost 3 integer dot-product instructions instead of ~9 f32 instructions, and the
// shared-memory traffic for x drops from 4 bytes to 3/4 byte per weight.  Integer accumulation is
// exact; the only approximation is x to 24 bits of its sub-block's largest element (f32 has 24 bits
// per element), far inside the parity tolerance.
// Shared-memory layout: plane k (k = 0..2) at k * units * 80 bytes, unit u at u * 80 inside it (64
// used: words 0..7 = elements 0..31 of the low-nibble sub-block, 8..15 = the high-nibble one; the pad
// keeps the 8 lanes of a row on different banks), then units * 16 bytes of (sum_lo, sum_hi, s_lo, s_hi).
constexpr unsigned MG_XU = 80;        // bytes per unit and plane
// Chunk c = elements 4c..4c+3; the 8 lanes that hold one sub-block's chunks are neighbours, all 32 lanes call.
__device__ __noinline__ void fx_put_chunk(unsigned char* xs, unsigned units, unsigned c, float4 v) {
  const unsigned e = c << 2;
  const unsigned u = e >> 6, hi = (e >> 5) & 1u, l = e & 31u;
  float s = (v.x + v.y) + (v.z + v.w);
  float am = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
  for (int o = 1; o <= 4; o <<= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
  }
  const float inv = am > 0.0f ? __fdividef(8.0e6f, am) : 0.0f;
  const float sc = am > 0.0f ? am * (1.0f / 8.0e6f) : 1.0f;
  const int X0 = __float2int_rn(v.x * inv), X1 = __float2int_rn(v.y * inv), X2 = __float2int_rn(v.z * inv),
            X3 = __float2int_rn(v.w * inv);
  const unsigned wi = hi * 8u + (l >> 2);
  unsigned char* base = xs + (size_t)u * MG_XU + wi * 4u;
  const size_t plane = (size_t)units * MG_XU;
  *reinterpret_cast<uint32_t*>(base) = __byte_perm(__byte_perm(X0, X1, 0x0040), __byte_perm(X2, X3, 0x0040), 0x5410);
  *reinterpret_cast<uint32_t*>(base + plane) = __byte_perm(__byte_perm(X0, X1, 0x0051), __byte_perm(X2, X3, 0x0051), 0x5410);
  *reinterpret_cast<uint32_t*>(base + 2 * plane) = __byte_perm(__byte_perm(X0, X1, 0x0062), __byte_perm(X2, X3, 0x0062), 0x5410);
  if ((threadIdx.x & 7u) == 0) {
    float* mt = reinterpret_cast<float*>(xs + 3 * plane + (size_t)u * 16u);
    mt[hi] = s;
    mt[2 + hi] = sc;
  }
}
__device__ __forceinline__ unsigned dp4a_uu(unsigned a, unsigned b, unsigned c) {
  unsigned d;
  asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_us(unsigned a, unsigned b, int c) {  // a: unsigned bytes, b: signed bytes
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
template <int OFF>
__device__ __forceinline__ float4 lds_f4o(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4+%5];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a), "n"(OFF));
  return v;
}
// One byte plane of x for a unit (16 words: [0..7] low sub-block, [8..15] high sub-block) against the
// masked nibbles of a row's unit: lo[i] / hi[i] hold elements 4i..4i+3 of the low / high sub-block.
template <bool SIGNED>
__device__ __forceinline__ void fx_plane(const uint32_t (&lo)[8], const uint32_t (&hi)[8], const uint4 x0, const uint4 x1,
                                         const uint4 x2, const uint4 x3, int& alo, int& ahi) {
  if (SIGNED) {
    alo = dp4a_us(lo[0], x0.x, alo); alo = dp4a_us(lo[1], x0.y, alo); alo = dp4a_us(lo[2], x0.z, alo); alo = dp4a_us(lo[3], x0.w, alo);
    alo = dp4a_us(lo[4], x1.x, alo); alo = dp4a_us(lo[5], x1.y, alo); alo = dp4a_us(lo[6], x1.z, alo); alo = dp4a_us(lo[7], x1.w, alo);
    ahi = dp4a_us(hi[0], x2.x, ahi); ahi = dp4a_us(hi[1], x2.y, ahi); ahi = dp4a_us(hi[2], x2.z, ahi); ahi = dp4a_us(hi[3], x2.w, ahi);
    ahi = dp4a_us(hi[4], x3.x, ahi); ahi = dp4a_us(hi[5], x3.y, ahi); ahi = dp4a_us(hi[6], x3.z, ahi); ahi = dp4a_us(hi[7], x3.w, ahi);
  } else {
    unsigned a = (unsigned)alo, h = (unsigned)ahi;
    a = dp4a_uu(lo[0], x0.x, a); a = dp4a_uu(lo[1], x0.y, a); a = dp4a_uu(lo[2], x0.z, a); a = dp4a_uu(lo[3], x0.w, a);
    a = dp4a_uu(lo[4], x1.x, a); a = dp4a_uu(lo[5], x1.y, a); a = dp4a_uu(lo[6], x1.z, a); a = dp4a_uu(lo[7], x1.w, a);
    h = dp4a_uu(hi[0], x2.x, h); h = dp4a_uu(hi[1], x2.y, h); h = dp4a_uu(hi[2], x2.z, h); h = dp4a_uu(hi[3], x2.w, h);
    h = dp4a_uu(hi[4], x3.x, h); h = dp4a_uu(hi[5], x3.y, h); h = dp4a_uu(hi[6], x3.z, h); h = dp4a_uu(hi[7], x3.w, h);
    alo = (int)a;
    ahi = (int)h;
  }
}
// This lane's unit of the staged x: three byte planes of 16 words and (sum_lo, sum_hi, s_lo, s_hi).
struct XUnit {
  uint4 p[12];
  float4 mt;
};
__device__ __forceinline__ void fx_load_unit(XUnit& x, uint32_t xs_s, unsigned units, unsigned u) {
  const uint32_t plane = units * MG_XU;
  const uint32_t xa = xs_s + u * MG_XU;
#pragma unroll
  for (int k = 0; k < 3; k++) {
    x.p[4 * k + 0] = lds_u4o<0>(xa + k * plane);
    x.p[4 * k + 1] = lds_u4o<16>(xa + k * plane);
    x.p[4 * k + 2] = lds_u4o<32>(xa + k * plane);
    x.p[4 * k + 3] = lds_u4o<48>(xa + k * plane);
  }
  x.mt = lds_f4o<0>(xs_s + 3u * plane + u * 16u);
}
// R rows at once against the unit this lane holds: wa[r] is the shared address of row r's unit (its 32
// nibble bytes sit 16 bytes after the block header at wa[r] - g * 32).  The rows' instruction streams are
// independent, which is what keeps a warp busy while each row's dp4a chains and loads are in flight.
template <int R>
__device__ __forceinline__ void fx_rows(const uint32_t (&wa)[R], int g, const XUnit& x, float (&out)[R]) {
  uint32_t lo[R][8], hi[R][8];
  int a0l[R], a0h[R], a1l[R], a1h[R], a2l[R], a2h[R];
#pragma unroll
  for (int r = 0; r < R; r++) {
    const uint4 q0 = lds_u4o<16>(wa[r]), q1 = lds_u4o<32>(wa[r]);
    const uint32_t q[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int i = 0; i < 8; i++) {
      lo[r][i] = q[i] & 0x0F0F0F0Fu;
      hi[r][i] = (q[i] >> 4) & 0x0F0F0F0Fu;
    }
    a0l[r] = a0h[r] = a1l[r] = a1h[r] = a2l[r] = a2h[r] = 0;
  }
#pragma unroll
  for (int r = 0; r < R; r++) fx_plane<false>(lo[r], hi[r], x.p[0], x.p[1], x.p[2], x.p[3], a0l[r], a0h[r]);
#pragma unroll
  for (int r = 0; r < R; r++) fx_plane<false>(lo[r], hi[r], x.p[4], x.p[5], x.p[6], x.p[7], a1l[r], a1h[r]);
#pragma unroll
  for (int r = 0; r < R; r++) fx_plane<true>(lo[r], hi[r], x.p[8], x.p[9], x.p[10], x.p[11], a2l[r], a2h[r]);
#pragma unroll
  for (int r = 0; r < R; r++) {
    const uint4 hdr = lds_u4o<0>(wa[r] - (uint32_t)g * 32u);
    const float flo = fmaf((float)a2l[r], 65536.0f, fmaf((float)(unsigned)a1l[r], 256.0f, (float)(unsigned)a0l[r])) * x.mt.z;
    const float fhi = fmaf((float)a2h[r], 65536.0f, fmaf((float)(unsigned)a1h[r], 256.0f, (float)(unsigned)a0h[r])) * x.mt.w;
    out[r] = q4k_apply_scales(hdr, g, flo, fhi, x.mt.x, x.mt.y, 0.0f);
  }
}

}  // namespace

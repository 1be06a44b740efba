// The small ops of the decode path: bit-exact dequant, RMSNorm family, per-head
// RMS + RoPE + Q4_0 pack, embedding gather, softcap argmax, GELU*mul.
//
// Each kernel restates one lowering of the reference (file:line given at the
// kernel); arithmetic order follows the lowering so that results stay within
// rounding of its CPU restatement.
#include "ks_internal.h"

namespace {

template <typename T>
__device__ __forceinline__ float ld_act(const T* p, size_t i);
template <>
__device__ __forceinline__ float ld_act<float>(const float* p, size_t i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_act<__half>(const __half* p, size_t i) { return __half2float(p[i]); }
template <typename T>
__device__ __forceinline__ void st_act(T* p, size_t i, float v);
template <>
__device__ __forceinline__ void st_act<float>(float* p, size_t i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void st_act<__half>(__half* p, size_t i, float v) { p[i] = __float2half_rn(v); }

__device__ __forceinline__ float half_bits_to_float(unsigned short h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ unsigned short rd16(const uint8_t* p) { return (unsigned short)(p[0] | (p[1] << 8)); }

// ---- element-wise dequant, bit-exact with gguf_impl.rs:618-633 / 690-721 / 761-791 ----------
// __fmul_rn / __fsub_rn keep the compiler from contracting a*b-c into one FMA.
__device__ __forceinline__ float deq_q4k(const uint8_t* base, size_t idx) {
  const uint8_t* blk = base + (idx >> 8) * KS_Q4K_BLOCK_BYTES;
  const unsigned e = (unsigned)(idx & 255);
  const unsigned grp = e >> 6, within = e & 63, hi = within >> 5, l = within & 31;
  const float d = half_bits_to_float(rd16(blk));
  const float dmin = half_bits_to_float(rd16(blk + 2));
  const uint8_t* q = blk + 4;
  const unsigned j = grp * 2 + hi;
  unsigned sc, m;
  if (j < 4) {
    sc = q[j] & 63;
    m = q[j + 4] & 63;
  } else {
    sc = (q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4);
    m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
  const unsigned byte = blk[16 + grp * 32 + l];
  const unsigned nib = hi ? (byte >> 4) : (byte & 0x0F);
  const float d1 = __fmul_rn(d, (float)sc);
  const float mn = __fmul_rn(dmin, (float)m);
  return __fsub_rn(__fmul_rn(d1, (float)nib), mn);
}
__device__ __forceinline__ float deq_q6k(const uint8_t* base, size_t idx) {
  const uint8_t* blk = base + (idx >> 8) * KS_Q6K_BLOCK_BYTES;
  const unsigned e = (unsigned)(idx & 255);
  const unsigned half = e >> 7, r = e & 127, k = r >> 5, l = r & 31;
  const uint8_t* ql = blk + half * 64;
  const uint8_t* qh = blk + 128 + half * 32;
  const signed char* sc = reinterpret_cast<const signed char*>(blk + 192 + half * 8);
  const float d = half_bits_to_float(rd16(blk + 208));
  const unsigned qlb = ql[l + (k & 1) * 32];
  const unsigned lo4 = (k & 2) ? (qlb >> 4) : (qlb & 0x0F);
  const unsigned hi2 = (qh[l] >> (2 * k)) & 3;
  const int qv = (int)(lo4 | (hi2 << 4)) - 32;
  const int s = sc[(l >> 4) + 2 * k];
  return __fmul_rn(__fmul_rn(d, (float)s), (float)qv);
}
// Q5_K (gguf_impl.rs:722-760): d, dmin, 12 scale bytes, qh[32] (bit 2g / 2g + 1 of byte l: the fifth bit of element l
// of the low / high sub-block of 64-group g), qs[128] nibbles laid out as in Q4_K.
__device__ __forceinline__ float deq_q5k(const uint8_t* base, size_t idx) {
  const uint8_t* blk = base + (idx >> 8) * KS_Q5K_BLOCK_BYTES;
  const unsigned e = (unsigned)(idx & 255), grp = e >> 6, hi = (e >> 5) & 1u, l = e & 31u, j = 2u * grp + hi;
  const float d = half_bits_to_float(rd16(blk)), dmin = half_bits_to_float(rd16(blk + 2));
  const uint8_t* q = blk + 4;
  unsigned sc, m;
  if (j < 4) {
    sc = q[j] & 63;
    m = q[j + 4] & 63;
  } else {
    sc = (q[j + 4] & 0x0F) | ((q[j - 4] >> 6) << 4);
    m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
  const unsigned byte = blk[48 + grp * 32 + l];
  const unsigned nib = hi ? (byte >> 4) : (byte & 0x0F);
  const float fifth = (blk[16 + l] >> j) & 1u ? 16.0f : 0.0f;
  return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), __fadd_rn((float)nib, fifth)), __fmul_rn(dmin, (float)m));
}
__device__ __forceinline__ float deq_q40(const uint8_t* base, size_t idx) {
  const uint8_t* blk = base + (idx >> 5) * KS_Q40_BLOCK_BYTES;
  const unsigned j = (unsigned)(idx & 31);
  const float d = half_bits_to_float(rd16(blk));
  const unsigned byte = blk[2 + (j & 15)];
  const int qv = (j < 16) ? (int)(byte & 0x0F) - 8 : (int)(byte >> 4) - 8;
  return __fmul_rn((float)qv, d);
}
__device__ __forceinline__ float deq_any(int dtype, const void* base, size_t idx) {
  switch (dtype) {
    case KS_Q4K: return deq_q4k((const uint8_t*)base, idx);
    case KS_Q6K: return deq_q6k((const uint8_t*)base, idx);
    case KS_Q40: return deq_q40((const uint8_t*)base, idx);
    case KS_Q5K: return deq_q5k((const uint8_t*)base, idx);
    case KS_F16: return __half2float(((const __half*)base)[idx]);
    default: return ((const float*)base)[idx];
  }
}

__global__ void dequant_kernel(int dtype, const uint8_t* src, size_t n, float* dst) {
  ks_pdl_entry();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = deq_any(dtype, src, i);
}

// ---- f32 / packed -> Q4_K: the reference's load-time quantizer (gguf_impl.rs:803-1016) -----------------
// The model loader requantises Q6_K ffn_down / attn_v tensors (and f32 / bf16 ones) to Q4_K on the host
// (gemma_prim.rs:415-440); here the same arithmetic runs on the GPU, byte for byte: every float operation is an
// explicit round-to-nearest intrinsic in the reference's order (no fused multiply-add), sums run sequentially.
// One thread per 32-element sub-block; the 8 threads of a super-block are neighbouring lanes.
__device__ __forceinline__ int q4k_nearest_int(float f) {
  return (int)(__float_as_uint(__fadd_rn(f, 12582912.0f)) & 0x007fffffu) - 0x00400000;
}
__device__ __forceinline__ int q4k_clampi(int v, int lo, int hi) { return v < lo ? lo : v > hi ? hi : v; }
// f32 -> f16 as the reference's own converter rounds (lib.rs:39-75: half UP in magnitude, not ties-to-even).
__device__ __forceinline__ unsigned f32_to_f16_half_up(float v) {
  const unsigned bits = __float_as_uint(v), sign = (bits >> 16) & 0x8000u;
  int e = (int)((bits >> 23) & 0xFFu);
  unsigned mant = bits & 0x7FFFFFu;
  if (e == 255) return mant == 0 ? (sign | 0x7C00u) : (sign | 0x7C00u | (mant >> 13));
  e -= 127;
  if (e > 15) return sign | 0x7C00u;
  if (e < -14) {
    if (e < -24) return sign;
    mant |= 0x800000u;
    const unsigned shift = (unsigned)(-14 - e) + 13u;
    return sign | ((mant + (1u << (shift - 1u))) >> shift);
  }
  const unsigned he = (unsigned)(e + 15), hm = mant + 0x1000u;
  if (hm & 0x800000u) return sign | ((he + 1u) << 10);
  return sign | (he << 10) | (hm >> 13);
}
// make_qkx2_quants (gguf_impl.rs:803-905) for n = 32, nmax = 15, rmin = -1, rdelta = 0.1, nstep = 20.
__device__ float q4k_search(const float (&x)[32], const float (&w)[32], unsigned char (&L)[32], float* the_min) {
  float mn = x[0], mx = x[0];
  float sum_w = w[0], sum_x = __fmul_rn(sum_w, x[0]);
  for (int i = 1; i < 32; i++) {
    if (x[i] < mn) mn = x[i];
    if (x[i] > mx) mx = x[i];
    sum_w = __fadd_rn(sum_w, w[i]);
    sum_x = __fadd_rn(sum_x, __fmul_rn(w[i], x[i]));
  }
  if (mn > 0.0f) mn = 0.0f;
  if (mx == mn) {
    for (int i = 0; i < 32; i++) L[i] = 0;
    *the_min = -mn;
    return 0.0f;
  }
  float iscale = __fdiv_rn(15.0f, __fsub_rn(mx, mn));
  float scale = __fdiv_rn(1.0f, iscale);
  float best = 0.0f;
  for (int i = 0; i < 32; i++) {
    const int l = q4k_clampi(q4k_nearest_int(__fmul_rn(iscale, __fsub_rn(x[i], mn))), 0, 15);
    L[i] = (unsigned char)l;
    const float diff = __fsub_rn(__fadd_rn(__fmul_rn(scale, (float)l), mn), x[i]);
    best = __fadd_rn(best, __fmul_rn(w[i], __fmul_rn(diff, diff)));
  }
  unsigned char Laux[32];
  for (int is = 0; is <= 20; is++) {
    // mn is the best minimum found so far: the candidate grid moves with it, as in the reference
    iscale = __fdiv_rn(__fadd_rn(__fadd_rn(-1.0f, __fmul_rn(0.1f, (float)is)), 15.0f), __fsub_rn(mx, mn));
    float sl = 0.0f, sl2 = 0.0f, sxl = 0.0f;
    for (int i = 0; i < 32; i++) {
      const int l = q4k_clampi(q4k_nearest_int(__fmul_rn(iscale, __fsub_rn(x[i], mn))), 0, 15);
      Laux[i] = (unsigned char)l;
      const float lf = (float)l;
      sl = __fadd_rn(sl, __fmul_rn(w[i], lf));
      sl2 = __fadd_rn(sl2, __fmul_rn(__fmul_rn(w[i], lf), lf));
      sxl = __fadd_rn(sxl, __fmul_rn(__fmul_rn(w[i], lf), x[i]));
    }
    const float D = __fsub_rn(__fmul_rn(sum_w, sl2), __fmul_rn(sl, sl));
    if (D > 0.0f) {
      float ts = __fdiv_rn(__fsub_rn(__fmul_rn(sum_w, sxl), __fmul_rn(sum_x, sl)), D);
      float tm = __fdiv_rn(__fsub_rn(__fmul_rn(sl2, sum_x), __fmul_rn(sl, sxl)), D);
      if (tm > 0.0f) {
        tm = 0.0f;
        ts = __fdiv_rn(sxl, sl2);
      }
      float err = 0.0f;
      for (int i = 0; i < 32; i++) {
        const float diff = __fsub_rn(__fadd_rn(__fmul_rn(ts, (float)Laux[i]), tm), x[i]);
        err = __fadd_rn(err, __fmul_rn(w[i], __fmul_rn(diff, diff)));
      }
      if (err < best) {
        for (int i = 0; i < 32; i++) L[i] = Laux[i];
        best = err;
        scale = ts;
        mn = tm;
      }
    }
  }
  *the_min = -mn;
  return scale;
}
// quantize_f32_to_q4k (gguf_impl.rs:907-1016): n_sb super-blocks of 256 source elements -> 144 bytes each.
__global__ void quantize_q4k_kernel(int dtype, const uint8_t* src, size_t n_sb, uint8_t* dst) {
  ks_pdl_entry();
  const size_t gt = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  const size_t sb = gt >> 3;
  const unsigned j = (unsigned)(gt & 7u);
  const bool live = sb < n_sb;  // whole groups of 8 lanes are live or not; dead lanes still take part in the shuffles
  float x[32], w[32];
  unsigned char L[32];
  float scale = 0.0f, mnv = 0.0f;
  if (live) {
    float s2 = 0.0f;
    for (int t = 0; t < 32; t++) {
      x[t] = deq_any(dtype, src, sb * 256 + 32 * j + t);
      s2 = __fadd_rn(s2, __fmul_rn(x[t], x[t]));
    }
    const float av = __fsqrt_rn(__fdiv_rn(s2, 32.0f));
    for (int t = 0; t < 32; t++) w[t] = __fadd_rn(av, fabsf(x[t]));
    scale = q4k_search(x, w, L, &mnv);
  } else {
    for (int t = 0; t < 32; t++) L[t] = 0;
  }
  // the largest scale and minimum of the super-block (the reference starts both at 0 and keeps what compares greater)
  float max_scale = fmaxf(scale, 0.0f), max_min = fmaxf(mnv, 0.0f);
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) {
    max_scale = fmaxf(max_scale, __shfl_xor_sync(0xffffffffu, max_scale, o));
    max_min = fmaxf(max_min, __shfl_xor_sync(0xffffffffu, max_min, o));
  }
  const float inv_scale = max_scale > 0.0f ? __fdiv_rn(63.0f, max_scale) : 0.0f;
  const float inv_min = max_min > 0.0f ? __fdiv_rn(63.0f, max_min) : 0.0f;
  const unsigned db = f32_to_f16_half_up(__fdiv_rn(max_scale, 63.0f)), mb = f32_to_f16_half_up(__fdiv_rn(max_min, 63.0f));
  unsigned ls = (unsigned)q4k_nearest_int(__fmul_rn(inv_scale, scale)) & 0xFFu;  // the reference casts to u8, then clamps
  unsigned lm = (unsigned)q4k_nearest_int(__fmul_rn(inv_min, mnv)) & 0xFFu;
  if (ls > 63u) ls = 63u;
  if (lm > 63u) lm = 63u;
  // the 12 scale bytes (gguf_impl.rs:976-983), built by every lane from its neighbours' values
  const unsigned lane = threadIdx.x & 31u, base = lane & ~7u;
  unsigned sc[12];
#pragma unroll
  for (int i = 0; i < 12; i++) sc[i] = 0;
#pragma unroll
  for (unsigned jj = 0; jj < 8; jj++) {
    const unsigned s_ = __shfl_sync(0xffffffffu, ls, base + jj), m_ = __shfl_sync(0xffffffffu, lm, base + jj);
    if (jj < 4) {
      sc[jj] |= s_;
      sc[jj + 4] |= m_;
    } else {
      sc[jj + 4] |= (s_ & 0x0Fu) | ((m_ & 0x0Fu) << 4);
      sc[jj - 4] |= (s_ >> 4) << 6;
      sc[jj] |= (m_ >> 4) << 6;
    }
  }
  uint8_t* blk = dst + sb * KS_Q4K_BLOCK_BYTES;
  if (live && j == 0) {
    uint32_t* h = reinterpret_cast<uint32_t*>(blk);
    h[0] = db | (mb << 16);
    h[1] = sc[0] | (sc[1] << 8) | (sc[2] << 16) | (sc[3] << 24);
    h[2] = sc[4] | (sc[5] << 8) | (sc[6] << 16) | (sc[7] << 24);
    h[3] = sc[8] | (sc[9] << 8) | (sc[10] << 16) | (sc[11] << 24);
  }
  // final levels against the stored 6-bit scale and minimum (unpacking the bytes gives ls and lm back)
  if (live) {
    const float dj = __fmul_rn(half_bits_to_float((unsigned short)db), (float)ls);
    if (dj != 0.0f) {
      const float dm = __fmul_rn(half_bits_to_float((unsigned short)mb), (float)lm);
      for (int t = 0; t < 32; t++) L[t] = (unsigned char)q4k_clampi(q4k_nearest_int(__fdiv_rn(__fadd_rn(x[t], dm), dj)), 0, 15);
    }
  }
  // byte t of a 64-element group holds sub-block 2g's level in the low nibble and sub-block 2g + 1's in the high one
  uint32_t* qs = reinterpret_cast<uint32_t*>(blk + 16 + 32 * (j >> 1));
#pragma unroll
  for (int wd = 0; wd < 8; wd++) {
    const uint32_t mine = (uint32_t)L[4 * wd] | ((uint32_t)L[4 * wd + 1] << 8) | ((uint32_t)L[4 * wd + 2] << 16) | ((uint32_t)L[4 * wd + 3] << 24);
    const uint32_t next = __shfl_down_sync(0xffffffffu, mine, 1);
    if (live && !(j & 1u)) qs[wd] = mine | (next << 4);
  }
}

// ---- block reductions -----------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Sum over the block; every thread gets the result. red: >= 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // red may still be read from a previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? red[lane] : 0.0f;
  return warp_sum(t);
}

// ---- RMSNorm (lower.rs:4079-4162): y = (x*inv)*w [+ res] [* scale] ---------------------------
template <typename T>
__global__ void rmsnorm_kernel(unsigned n, float eps, const T* x, const T* w, const T* res, int has_scale,
                               float scale, T* y) {
  ks_pdl_entry();
  __shared__ float red[32];
  const size_t off = (size_t)blockIdx.x * n;
  float ss = 0.0f;
  for (unsigned i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = ld_act<T>(x, off + i);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (unsigned i = threadIdx.x; i < n; i += blockDim.x) {
    float v = __fmul_rn(__fmul_rn(ld_act<T>(x, off + i), inv), ld_act<T>(w, i));
    if (res) v = __fadd_rn(v, ld_act<T>(res, off + i));
    if (has_scale) v = __fmul_rn(scale, v);
    st_act<T>(y, off + i, v);
  }
}

// ---- lower.rs:3926-4077: out_x = res + (y*inv)*w_post ; out_x2 = (out_x*inv2)*w_ffn ----------
template <typename T>
__global__ void rmsnorm_add_then_rmsnorm_kernel(unsigned n, float eps, const T* y, const T* w_post, const T* res,
                                                const T* w_ffn, T* out_x, T* out_x2) {
  ks_pdl_entry();
  extern __shared__ float xs[];  // n floats: the new residual stream
  __shared__ float red[32];
  const size_t off = (size_t)blockIdx.x * n;
  float ss = 0.0f;
  for (unsigned i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = ld_act<T>(y, off + i);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  float ss2 = 0.0f;
  for (unsigned i = threadIdx.x; i < n; i += blockDim.x) {
    float v = __fadd_rn(ld_act<T>(res, off + i), __fmul_rn(__fmul_rn(ld_act<T>(y, off + i), inv), ld_act<T>(w_post, i)));
    st_act<T>(out_x, off + i, v);
    if (sizeof(T) == 2) v = __half2float(__float2half_rn(v));  // the second norm reads what was stored
    xs[i] = v;
    ss2 = fmaf(v, v, ss2);
  }
  ss2 = block_sum(ss2, red);
  const float inv2 = 1.0f / sqrtf(ss2 / (float)n + eps);
  for (unsigned i = threadIdx.x; i < n; i += blockDim.x)
    st_act<T>(out_x2, off + i, __fmul_rn(__fmul_rn(xs[i], inv2), ld_act<T>(w_ffn, i)));
}

// ---- Q4_0 pack of 32 values held one per lane (render.rs:1021-1059) --------------------------
__device__ __forceinline__ void pack_q40_warp(float v, uint8_t* blk, int lane) {
  const float amax = warp_max(fabsf(v));
  const float scale = amax > 0.0f ? amax / 7.0f : 1.0f;
  const float inv = 1.0f / scale;
  int q = (int)roundf(__fmul_rn(v, inv)) + 8;
  q = q < 0 ? 0 : q > 15 ? 15 : q;
  const int qhi = __shfl_down_sync(0xffffffffu, q, 16);
  if (lane < 16) blk[2 + lane] = (uint8_t)(q | (qhi << 4));
  // Q4_0 blocks are 18 bytes on an even base, so the fp16 scale is one aligned 16-bit store
  if (lane == 0) *reinterpret_cast<__half*>(blk) = __float2half_rn(scale);
}

template <typename T>
__global__ void quantize_q40_kernel(size_t nblocks, const T* src, uint8_t* dst) {
  ks_pdl_entry();
  const int lane = threadIdx.x & 31;
  const size_t warp = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t b = warp; b < nblocks; b += nwarps) pack_q40_warp(ld_act<T>(src, b * 32 + lane), dst + b * KS_Q40_BLOCK_BYTES, lane);
}

// ---- per-head RMS + RoPE (Q) / + Q4_0 pack (K) / RMS only + pack (V): lower.rs:4231-4702 -----
// One warp per (token, job): jobs 0..n_q-1 are Q heads, then n_kv K heads, then n_kv V heads.
// pos == nullptr: token t uses rope row t and KV row t (the reference's batch form, consecutive
// positions).  pos != nullptr: token t belongs to slot t at position pos[t]: rope row pos[t],
// KV row pos[t] of that slot's cache (slot_stride bytes apart).
template <typename T>
__global__ void per_head_qkv_q40_kernel(unsigned n_q, unsigned n_kv, unsigned hd, float eps, const T* q, const T* qw,
                                        const float* rope, const T* k, const T* kw, const T* v, T* q_out,
                                        uint8_t* kv_k, uint8_t* kv_v, const int* pos, size_t slot_stride) {
  ks_pdl_entry();
  extern __shared__ float tmp[];  // hd floats
  const int lane = threadIdx.x;
  const unsigned jobs = n_q + 2 * n_kv;
  const unsigned tok = blockIdx.x / jobs, job = blockIdx.x % jobs;
  const unsigned half = hd / 2;
  const size_t rowb = (size_t)(hd / 32) * KS_Q40_BLOCK_BYTES;
  const size_t p = pos ? (size_t)pos[tok] : (size_t)tok;
  const float* cs = rope + p * hd;
  const size_t kv_off = pos ? (size_t)tok * slot_stride + p * n_kv * rowb : p * n_kv * rowb;

  const T* src;
  const T* w;
  size_t base;
  int kind;  // 0 = Q, 1 = K, 2 = V
  if (job < n_q) {
    kind = 0; src = q; w = qw; base = ((size_t)tok * n_q + job) * hd;
  } else if (job < n_q + n_kv) {
    kind = 1; src = k; w = kw; base = ((size_t)tok * n_kv + (job - n_q)) * hd;
  } else {
    kind = 2; src = v; w = nullptr; base = ((size_t)tok * n_kv + (job - n_q - n_kv)) * hd;
  }
  float ss = 0.0f;
  for (unsigned i = lane; i < hd; i += 32) {
    const float x = ld_act<T>(src, base + i);
    ss = fmaf(x, x, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)hd + eps);

  if (kind == 2) {
    for (unsigned i = lane; i < hd; i += 32) tmp[i] = __fmul_rn(ld_act<T>(src, base + i), inv);
  } else {
    for (unsigned i = lane; i < half; i += 32) {
      const float u = __fmul_rn(__fmul_rn(ld_act<T>(src, base + i), inv), ld_act<T>(w, i));
      const float vv = __fmul_rn(__fmul_rn(ld_act<T>(src, base + half + i), inv), ld_act<T>(w, half + i));
      const float c = cs[i], s = cs[half + i];
      const float lo = __fsub_rn(__fmul_rn(u, c), __fmul_rn(vv, s));
      const float hi = __fadd_rn(__fmul_rn(u, s), __fmul_rn(vv, c));
      if (kind == 0) {
        st_act<T>(q_out, base + i, lo);
        st_act<T>(q_out, base + half + i, hi);
      } else {
        tmp[i] = lo;
        tmp[half + i] = hi;
      }
    }
  }
  if (kind == 0) return;
  __syncwarp();
  const unsigned head = (kind == 1) ? job - n_q : job - n_q - n_kv;
  uint8_t* dst = (kind == 1 ? kv_k : kv_v) + kv_off + (size_t)head * rowb;
  for (unsigned b = 0; b < hd / 32; b++) {
    // values pass through f16 before packing (render.rs:1046)
    const float val = __half2float(__float2half_rn(tmp[b * 32 + lane]));
    pack_q40_warp(val, dst + (size_t)b * KS_Q40_BLOCK_BYTES, lane);
  }
}

// ---- embedding gather (lower.rs:3899-3924): dst[b, i] = scale * deq(src)[uint(idx[b])*n + i] --
template <typename T>
__global__ void copy_scale_indexed_kernel(unsigned n, float scale, int dtype, const void* src, const float* idx, T* dst) {
  ks_pdl_entry();
  const size_t id = (size_t)(unsigned)idx[blockIdx.y];
  size_t row_elems = (size_t)id * n;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    st_act<T>(dst, (size_t)blockIdx.y * n + i, __fmul_rn(scale, deq_any(dtype, src, row_elems + i)));
}

// ---- softcap argmax (lower.rs:6090-6157, render.rs:2346-2389) --------------------------------
// Stage 1: every block scans a strided share and leaves its best (value, index) in ws; the block
// that finishes last merges them.  Larger value wins, equal values go to the lower index.
__device__ __forceinline__ void argmax_merge(float& bv, unsigned& bi, float ov, unsigned oi) {
  if (ov > bv || (ov == bv && oi < bi)) {
    bv = ov;
    bi = oi;
  }
}
template <typename T>
__global__ void softcap_argmax_kernel(unsigned n, float cap, const T* x, float* out_idx, float* ws_val,
                                      unsigned* ws_idx, unsigned* counter) {
  ks_pdl_entry();
  __shared__ float sv[32];
  __shared__ unsigned si[32];
  __shared__ bool last;
  float bv = -1.0e30f;
  unsigned bi = 0;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    const float v = cap * tanhf(ld_act<T>(x, i) / cap);
    if (v > bv) {
      bv = v;
      bi = i;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) argmax_merge(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if (lane == 0) {
    sv[warp] = bv;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    bv = lane < nwarp ? sv[lane] : -1.0e30f;
    bi = lane < nwarp ? si[lane] : 0xffffffffu;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) argmax_merge(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (lane == 0) {
      ws_val[blockIdx.x] = bv;
      ws_idx[blockIdx.x] = bi;
      __threadfence();
      last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    }
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  bv = -1.0e30f;
  bi = 0xffffffffu;
  for (unsigned b = threadIdx.x; b < gridDim.x; b += blockDim.x) argmax_merge(bv, bi, ((volatile float*)ws_val)[b], ((volatile unsigned*)ws_idx)[b]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) argmax_merge(bv, bi, __shfl_xor_sync(0xffffffffu, bv, o), __shfl_xor_sync(0xffffffffu, bi, o));
  __syncthreads();
  if (lane == 0) {
    sv[warp] = bv;
    si[warp] = bi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < nwarp; w++) argmax_merge(bv, bi, sv[w], si[w]);
    out_idx[0] = (float)(bi == 0xffffffffu ? 0u : bi);
    *counter = 0;  // ready for the next launch
  }
}

template <typename T>
__global__ void gelu_mul_kernel(size_t n, const T* g, const T* u, T* y) {
  ks_pdl_entry();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float ax = fminf(20.0f, fmaxf(-20.0f, ld_act<T>(g, i)));
    const float t = 0.79788456f * (ax + 0.044715f * ((ax * ax) * ax));
    st_act<T>(y, i, ((0.5f * ax) * (1.0f + tanhf(t))) * ld_act<T>(u, i));
  }
}

}  // namespace

// ---- launchers ----------------------------------------------------------------------------------

static int norm_threads(size_t n) { return n >= 4096 ? 1024 : n >= 1024 ? 512 : 256; }

int ks_launch_rmsnorm(ks_ctx* ctx, size_t n, size_t rows, float eps, ks_dtype act, const void* x, const void* w,
                      const void* res, int has_scale, float scale, void* y) {
  const int th = norm_threads(n);
  if (act == KS_F32)
    KS_LAUNCH(ctx, (rmsnorm_kernel<float>), (unsigned)rows, th, 0, (unsigned)n, eps, (const float*)x, (const float*)w,
                                                                 (const float*)res, has_scale, scale, (float*)y);
  else
    KS_LAUNCH(ctx, (rmsnorm_kernel<__half>), (unsigned)rows, th, 0, (unsigned)n, eps, (const __half*)x, (const __half*)w,
                                                                  (const __half*)res, has_scale, scale, (__half*)y);
  return ks_after_launch(ctx, "rmsnorm");
}

int ks_launch_rmsnorm_add_then_rmsnorm(ks_ctx* ctx, size_t n, size_t rows, float eps, ks_dtype act, const void* y,
                                       const void* w_post, const void* res, const void* w_ffn, void* out_x,
                                       void* out_x2) {
  const int th = norm_threads(n);
  const size_t smem = n * sizeof(float);
  if (act == KS_F32)
    KS_LAUNCH(ctx, (rmsnorm_add_then_rmsnorm_kernel<float>), (unsigned)rows, th, smem, 
        (unsigned)n, eps, (const float*)y, (const float*)w_post, (const float*)res, (const float*)w_ffn, (float*)out_x,
        (float*)out_x2);
  else
    KS_LAUNCH(ctx, (rmsnorm_add_then_rmsnorm_kernel<__half>), (unsigned)rows, th, smem, 
        (unsigned)n, eps, (const __half*)y, (const __half*)w_post, (const __half*)res, (const __half*)w_ffn,
        (__half*)out_x, (__half*)out_x2);
  return ks_after_launch(ctx, "rmsnorm_add_then_rmsnorm");
}

int ks_launch_per_head_qkv_q40(ks_ctx* ctx, size_t n_q, size_t n_kv, size_t hd, size_t n_tok, float eps, ks_dtype act,
                               const void* q, const void* qw, const float* rope, const void* k, const void* kw,
                               const void* v, void* q_out, uint8_t* kv_k, uint8_t* kv_v, const int* pos_dev,
                               size_t slot_stride_bytes) {
  const unsigned grid = (unsigned)(n_tok * (n_q + 2 * n_kv));
  const size_t smem = hd * sizeof(float);
  if (act == KS_F32)
    KS_LAUNCH(ctx, (per_head_qkv_q40_kernel<float>), grid, 32, smem, 
        (unsigned)n_q, (unsigned)n_kv, (unsigned)hd, eps, (const float*)q, (const float*)qw, rope, (const float*)k,
        (const float*)kw, (const float*)v, (float*)q_out, kv_k, kv_v, pos_dev, slot_stride_bytes);
  else
    KS_LAUNCH(ctx, (per_head_qkv_q40_kernel<__half>), grid, 32, smem, 
        (unsigned)n_q, (unsigned)n_kv, (unsigned)hd, eps, (const __half*)q, (const __half*)qw, rope, (const __half*)k,
        (const __half*)kw, (const __half*)v, (__half*)q_out, kv_k, kv_v, pos_dev, slot_stride_bytes);
  return ks_after_launch(ctx, "rmsnorm_per_head_qkv_q40");
}

int ks_launch_copy_scale_indexed(ks_ctx* ctx, size_t n, size_t batch, float scale, ks_dtype src_dtype, const void* src,
                                 const float* idx, ks_dtype act, void* dst) {
  dim3 grid((unsigned)((n + 255) / 256), (unsigned)batch);
  if (act == KS_F32)
    KS_LAUNCH(ctx, (copy_scale_indexed_kernel<float>), grid, 256, 0, (unsigned)n, scale, (int)src_dtype, src, idx, (float*)dst);
  else
    KS_LAUNCH(ctx, (copy_scale_indexed_kernel<__half>), grid, 256, 0, (unsigned)n, scale, (int)src_dtype, src, idx, (__half*)dst);
  return ks_after_launch(ctx, "copy_scale_indexed");
}

int ks_launch_softcap_argmax(ks_ctx* ctx, size_t n, float cap, ks_dtype act, const void* logits, float* out_idx) {
  // workspace layout: [0,1024) f32 values, [1024,2048) u32 indices, [2048] counter
  float* ws_val = (float*)ctx->ws;
  unsigned* ws_idx = (unsigned*)ctx->ws + 1024;
  unsigned* counter = (unsigned*)ctx->ws + 2048;
  unsigned grid = (unsigned)((n + 1023) / 1024);
  const unsigned cap_grid = (unsigned)(ctx->sm_count * 2) < 1024u ? (unsigned)(ctx->sm_count * 2) : 1024u;
  if (grid > cap_grid) grid = cap_grid;
  if (grid == 0) grid = 1;
  if (act == KS_F32)
    KS_LAUNCH(ctx, (softcap_argmax_kernel<float>), grid, 256, 0, (unsigned)n, cap, (const float*)logits, out_idx, ws_val, ws_idx, counter);
  else
    KS_LAUNCH(ctx, (softcap_argmax_kernel<__half>), grid, 256, 0, (unsigned)n, cap, (const __half*)logits, out_idx, ws_val, ws_idx, counter);
  return ks_after_launch(ctx, "softcap_argmax");
}

// ---- C ABI --------------------------------------------------------------------------------------
int ks_launch_quantize_q4k(ks_ctx* ctx, ks_dtype src_dtype, const void* src, size_t nelem, void* dst) {
  const size_t n_sb = nelem / 256, threads = n_sb * 8;
  if (nelem % 256 || (threads + 127) / 128 >= (1ull << 31)) return ks_fail(ctx, KS_ERR_INVALID, "quantize_q4k: bad element count %zu", nelem);
  if (n_sb == 0) return KS_OK;
  KS_LAUNCH(ctx, (quantize_q4k_kernel), (unsigned)((threads + 127) / 128), 128, 0, (int)src_dtype, (const uint8_t*)src, n_sb, (uint8_t*)dst);
  return ks_after_launch(ctx, "quantize_q4k");
}

extern "C" {

int ks_dequant(ks_ctx* ctx, ks_dtype dtype, const ks_buf* src, size_t src_byte_off, size_t nelem, ks_buf* dst,
               size_t dst_off) {
  if (!ctx) return KS_ERR_INVALID;
  KS_REQUIRE(ctx, dtype == KS_Q4K || dtype == KS_Q6K || dtype == KS_Q40 || dtype == KS_Q5K || dtype == KS_F16,
             "dequant: unsupported ggml type %d", (int)dtype);
  if (dtype != KS_F16) KS_REQUIRE(ctx, nelem % ks_block_elems(dtype) == 0, "dequant: nelem=%zu is not a whole number of blocks", nelem);
  KS_REQUIRE(ctx, ks_fits(src, src_byte_off, ks_nbytes(dtype, nelem)), "dequant: source buffer too small");
  KS_REQUIRE(ctx, ks_fits(dst, dst_off * 4, nelem * 4), "dequant: destination buffer too small");
  if (nelem == 0) return KS_OK;
  size_t blocks = (nelem + 255) / 256;
  if (blocks > (size_t)ctx->sm_count * 32) blocks = (size_t)ctx->sm_count * 32;
  KS_LAUNCH(ctx, (dequant_kernel), (unsigned)blocks, 256, 0, (int)dtype, (const uint8_t*)src->dptr + src_byte_off, nelem,
                                                            (float*)dst->dptr + dst_off);
  return ks_after_launch(ctx, "dequant");
}

int ks_quantize_q4k(ks_ctx* ctx, ks_dtype src_dtype, const ks_buf* src, size_t src_byte_off, size_t nelem, ks_buf* dst,
                    size_t dst_byte_off) {
  if (!ctx) return KS_ERR_INVALID;
  KS_REQUIRE(ctx, src_dtype == KS_Q6K || src_dtype == KS_Q5K || src_dtype == KS_Q4K || src_dtype == KS_F16 || src_dtype == KS_F32,
             "quantize_q4k: unsupported source type %d", (int)src_dtype);
  KS_REQUIRE(ctx, nelem % 256 == 0, "quantize_q4k: nelem=%zu is not a multiple of 256", nelem);
  KS_REQUIRE(ctx, src_byte_off % 4 == 0 && dst_byte_off % 4 == 0, "quantize_q4k: byte offsets must be multiples of 4");
  KS_REQUIRE(ctx, ks_fits(src, src_byte_off, ks_nbytes(src_dtype, nelem)), "quantize_q4k: source buffer too small");
  KS_REQUIRE(ctx, ks_fits(dst, dst_byte_off, nelem / 256 * KS_Q4K_BLOCK_BYTES), "quantize_q4k: destination buffer too small");
  return ks_launch_quantize_q4k(ctx, src_dtype, (const uint8_t*)src->dptr + src_byte_off, nelem, (uint8_t*)dst->dptr + dst_byte_off);
}

int ks_rmsnorm(ks_ctx* ctx, size_t n, size_t rows, float eps, ks_dtype act, const ks_buf* x, size_t x_off,
               const ks_buf* w, const ks_buf* res, size_t res_off, int has_scale, float scale, ks_buf* y, size_t y_off) {
  if (!ctx) return KS_ERR_INVALID;
  KS_REQUIRE(ctx, ks_is_act(act), "rmsnorm: activation dtype must be F32 or F16");
  KS_REQUIRE(ctx, n > 0 && rows > 0 && n < (1u << 24) && rows < (1u << 24), "rmsnorm: n=%zu rows=%zu out of range", n, rows);
  const size_t ab = ks_act_bytes(act);
  KS_REQUIRE(ctx, ks_fits(x, x_off * ab, rows * n * ab), "rmsnorm: x buffer too small");
  KS_REQUIRE(ctx, ks_fits(w, 0, n * ab), "rmsnorm: weight buffer too small");
  KS_REQUIRE(ctx, !res || ks_fits(res, res_off * ab, rows * n * ab), "rmsnorm: residual buffer too small");
  KS_REQUIRE(ctx, ks_fits(y, y_off * ab, rows * n * ab), "rmsnorm: y buffer too small");
  return ks_launch_rmsnorm(ctx, n, rows, eps, act, (const char*)x->dptr + x_off * ab, w->dptr,
                           res ? (const char*)res->dptr + res_off * ab : nullptr, has_scale, scale,
                           (char*)y->dptr + y_off * ab);
}

int ks_rmsnorm_add_then_rmsnorm(ks_ctx* ctx, size_t n, size_t rows, float eps, ks_dtype act, const ks_buf* y,
                                const ks_buf* w_post, const ks_buf* res, const ks_buf* w_ffn, ks_buf* out_x,
                                ks_buf* out_x2) {
  if (!ctx) return KS_ERR_INVALID;
  KS_REQUIRE(ctx, ks_is_act(act), "rmsnorm_add_then_rmsnorm: activation dtype must be F32 or F16");
  KS_REQUIRE(ctx, n > 0 && rows > 0 && rows < (1u << 24), "rmsnorm_add_then_rmsnorm: n=%zu rows=%zu out of range", n, rows);
  // the residual stream is staged in shared memory (the reference has the same limit, lower.rs:3934-3938)
  KS_REQUIRE(ctx, n * 4 <= 48 * 1024, "rmsnorm_add_then_rmsnorm requires LOCAL staging of residual stream (n=%zu too large)", n);
  const size_t ab = ks_act_bytes(act);
  KS_REQUIRE(ctx, ks_fits(y, 0, rows * n * ab) && ks_fits(res, 0, rows * n * ab) && ks_fits(out_x, 0, rows * n * ab) &&
                      ks_fits(out_x2, 0, rows * n * ab),
             "rmsnorm_add_then_rmsnorm: activation buffer too small");
  KS_REQUIRE(ctx, ks_fits(w_post, 0, n * ab) && ks_fits(w_ffn, 0, n * ab), "rmsnorm_add_then_rmsnorm: weight buffer too small");
  return ks_launch_rmsnorm_add_then_rmsnorm(ctx, n, rows, eps, act, y->dptr, w_post->dptr, res->dptr, w_ffn->dptr,
                                            out_x->dptr, out_x2->dptr);
}

int ks_rmsnorm_per_head_qkv_q40(ks_ctx* ctx, size_t n_q, size_t n_kv, size_t hd, size_t n_tok, float eps, ks_dtype act,
                                const ks_buf* q, const ks_buf* qw, const ks_buf* rope, size_t rope_off, const ks_buf* k,
                                const ks_buf* kw, const ks_buf* v, ks_buf* q_out, ks_buf* kv_k, ks_buf* kv_v,
                                size_t kv_byte_off) {
  if (!ctx) return KS_ERR_INVALID;
  KS_REQUIRE(ctx, ks_is_act(act), "rmsnorm_per_head_qkv_q40: activation dtype must be F32 or F16");
  KS_REQUIRE(ctx, hd >= 64 && hd % 64 == 0 && hd <= 1024, "rmsnorm_per_head_qkv_q40: hd=%zu must be a multiple of 64 in 64..1024", hd);
  KS_REQUIRE(ctx, n_q > 0 && n_kv > 0 && n_kv <= n_q && n_tok > 0 && n_tok < 65536, "rmsnorm_per_head_qkv_q40: bad head or token count");
  const size_t ab = ks_act_bytes(act);
  const size_t rowb = hd / 32 * KS_Q40_BLOCK_BYTES;
  KS_REQUIRE(ctx, ks_fits(q, 0, n_tok * n_q * hd * ab) && ks_fits(q_out, 0, n_tok * n_q * hd * ab), "rmsnorm_per_head_qkv_q40: q buffer too small");
  KS_REQUIRE(ctx, ks_fits(k, 0, n_tok * n_kv * hd * ab) && ks_fits(v, 0, n_tok * n_kv * hd * ab), "rmsnorm_per_head_qkv_q40: k/v buffer too small");
  KS_REQUIRE(ctx, ks_fits(qw, 0, hd * ab) && ks_fits(kw, 0, hd * ab), "rmsnorm_per_head_qkv_q40: norm weight too small");
  KS_REQUIRE(ctx, ks_fits(rope, rope_off * 4, n_tok * hd * 4), "rmsnorm_per_head_qkv_q40: rope table too small for offset %zu", rope_off);
  KS_REQUIRE(ctx, ks_fits(kv_k, kv_byte_off, n_tok * n_kv * rowb) && ks_fits(kv_v, kv_byte_off, n_tok * n_kv * rowb),
             "rmsnorm_per_head_qkv_q40: KV write at byte offset %zu exceeds the cache (max_seq exceeded)", kv_byte_off);
  KS_REQUIRE(ctx, kv_byte_off % 2 == 0, "rmsnorm_per_head_qkv_q40: odd KV byte offset");
  return ks_launch_per_head_qkv_q40(ctx, n_q, n_kv, hd, n_tok, eps, act, q->dptr, qw->dptr,
                                    (const float*)rope->dptr + rope_off, k->dptr, kw->dptr, v->dptr, q_out->dptr,
                                    (uint8_t*)kv_k->dptr + kv_byte_off, (uint8_t*)kv_v->dptr + kv_byte_off, nullptr, 0);
}

int ks_quantize_q40(ks_ctx* ctx, size_t n, ks_dtype act, const ks_buf* src, size_t src_off, ks_buf* dst,
                    size_t dst_byte_off) {
  if (!ctx) return KS_ERR_INVALID;
  KS_REQUIRE(ctx, ks_is_act(act), "quantize_q40: source dtype must be F32 or F16");
  KS_REQUIRE(ctx, n % 32 == 0, "quantize_q40: n=%zu is not a multiple of 32", n);
  const size_t ab = ks_act_bytes(act);
  KS_REQUIRE(ctx, ks_fits(src, src_off * ab, n * ab), "quantize_q40: source buffer too small");
  KS_REQUIRE(ctx, ks_fits(dst, dst_byte_off, n / 32 * KS_Q40_BLOCK_BYTES), "quantize_q40: destination buffer too small");
  KS_REQUIRE(ctx, dst_byte_off % 2 == 0, "quantize_q40: odd destination byte offset");
  if (n == 0) return KS_OK;
  const size_t nblocks = n / 32;
  size_t grid = (nblocks + 7) / 8;
  if (grid > (size_t)ctx->sm_count * 8) grid = (size_t)ctx->sm_count * 8;
  if (act == KS_F32)
    KS_LAUNCH(ctx, (quantize_q40_kernel<float>), (unsigned)grid, 256, 0, nblocks, (const float*)src->dptr + src_off,
                                                                        (uint8_t*)dst->dptr + dst_byte_off);
  else
    KS_LAUNCH(ctx, (quantize_q40_kernel<__half>), (unsigned)grid, 256, 0, nblocks, (const __half*)src->dptr + src_off,
                                                                         (uint8_t*)dst->dptr + dst_byte_off);
  return ks_after_launch(ctx, "quantize_q40");
}

int ks_copy_scale_indexed(ks_ctx* ctx, size_t n, size_t batch, float scale, ks_dtype src_dtype, const ks_buf* src,
                          const ks_buf* idx, size_t idx_off, ks_dtype act, ks_buf* dst) {
  if (!ctx) return KS_ERR_INVALID;
  KS_REQUIRE(ctx, src_dtype == KS_F32 || src_dtype == KS_F16 || src_dtype == KS_Q4K || src_dtype == KS_Q5K || src_dtype == KS_Q6K,
             "copy_scale_indexed: source dtype %d not wired", (int)src_dtype);
  KS_REQUIRE(ctx, ks_is_act(act), "copy_scale_indexed: destination dtype must be F32 or F16");
  KS_REQUIRE(ctx, n > 0 && batch > 0 && batch < 65536, "copy_scale_indexed: n=%zu batch=%zu out of range", n, batch);
  if (src_dtype == KS_Q4K || src_dtype == KS_Q5K || src_dtype == KS_Q6K) KS_REQUIRE(ctx, n % 256 == 0, "copy_scale_indexed: n=%zu must be a multiple of 256 for packed rows", n);
  KS_REQUIRE(ctx, src && src->dptr, "copy_scale_indexed: null source");
  KS_REQUIRE(ctx, ks_fits(idx, idx_off * 4, batch * 4), "copy_scale_indexed: index buffer too small");
  KS_REQUIRE(ctx, ks_fits(dst, 0, batch * n * ks_act_bytes(act)), "copy_scale_indexed: destination buffer too small");
  // Row ids live on the device and are not range-checked here (the reference does not either);
  // the caller sizes src for its vocabulary.
  return ks_launch_copy_scale_indexed(ctx, n, batch, scale, src_dtype, src->dptr, (const float*)idx->dptr + idx_off, act, dst->dptr);
}

int ks_softcap_argmax(ks_ctx* ctx, size_t n, float cap, ks_dtype act, const ks_buf* logits, ks_buf* out_idx, size_t out_off) {
  if (!ctx) return KS_ERR_INVALID;
  KS_REQUIRE(ctx, ks_is_act(act), "softcap_argmax: logits dtype must be F32 or F16");
  // 32-bit indices inside the kernel: n + one grid stride must not wrap; the index comes back as f32 (exact below 2^24)
  KS_REQUIRE(ctx, n > 0 && n <= (1ull << 31), "softcap_argmax: n=%zu out of range (1 .. 2^31)", n);
  KS_REQUIRE(ctx, cap > 0.0f, "softcap_argmax: cap must be > 0");
  KS_REQUIRE(ctx, ks_fits(logits, 0, n * ks_act_bytes(act)), "softcap_argmax: logits buffer too small");
  KS_REQUIRE(ctx, ks_fits(out_idx, out_off * 4, 4), "softcap_argmax: output buffer too small");
  return ks_launch_softcap_argmax(ctx, n, cap, act, logits->dptr, (float*)out_idx->dptr + out_off);
}

int ks_gelu_mul(ks_ctx* ctx, size_t n, ks_dtype act, const ks_buf* g, const ks_buf* u, ks_buf* y) {
  if (!ctx) return KS_ERR_INVALID;
  KS_REQUIRE(ctx, ks_is_act(act), "gelu_mul: dtype must be F32 or F16");
  const size_t ab = ks_act_bytes(act);
  KS_REQUIRE(ctx, ks_fits(g, 0, n * ab) && ks_fits(u, 0, n * ab) && ks_fits(y, 0, n * ab), "gelu_mul: buffer too small");
  if (n == 0) return KS_OK;
  size_t grid = (n + 255) / 256;
  if (grid > (size_t)ctx->sm_count * 8) grid = (size_t)ctx->sm_count * 8;
  if (act == KS_F32)
    KS_LAUNCH(ctx, (gelu_mul_kernel<float>), (unsigned)grid, 256, 0, n, (const float*)g->dptr, (const float*)u->dptr, (float*)y->dptr);
  else
    KS_LAUNCH(ctx, (gelu_mul_kernel<__half>), (unsigned)grid, 256, 0, n, (const __half*)g->dptr, (const __half*)u->dptr, (__half*)y->dptr);
  return ks_after_launch(ctx, "gelu_mul");
}

}  // extern "C"

// ---- arg-max for callers that must not allocate ---------------------------------------------------
// Some hosts hand this library device pointers but may not create device allocations themselves:
// a runtime that carved all of HBM into its own arena up front, a plugin loaded into a process
// whose memory budget is fixed, code running where cudaMalloc would synchronise a device it does
// not own.  ks_softcap_argmax needs a little global scratch for its cross-block reduction and takes
// it from the context, which cudaMalloc'ed it; this variant needs no context at all and keeps that
// scratch in a fixed array inside the library image instead.
#define KS_NOALLOC_MAX_N (1u << 22)   /* largest logits vector accepted */
#define KS_NOALLOC_MAX_BLOCKS 512
// [0, 512) f32 block maxima | [512, 1024) u32 block indices | [1024] u32 arrival counter
static __device__ __align__(256) unsigned ks_noalloc_scratch[KS_NOALLOC_MAX_BLOCKS * 2 + 64];

extern "C" int ks_softcap_argmax_noalloc(int device, void* stream, size_t n, float cap, const float* logits,
                                         float* out_idx) {
  // Device address of the array, per device.  The cache is not synchronised: like every entry point of
  // this library it expects one calling thread at a time (two racing first calls would both look the
  // address up and store the same value, but nothing here promises more than that).
  static void* scratch_addr[64] = {nullptr};
  char msg[256];
  if (!logits || !out_idx || n == 0 || !(cap > 0.0f) || device < 0 || device >= 64) {
    ks_set_global_error("softcap_argmax_noalloc: null pointer, n == 0, cap <= 0 or bad device index");
    return KS_ERR_INVALID;
  }
  if (n > KS_NOALLOC_MAX_N) {
    snprintf(msg, sizeof msg, "softcap_argmax_noalloc: n=%zu exceeds the fixed-scratch limit of %u elements", n, KS_NOALLOC_MAX_N);
    ks_set_global_error(msg);
    return KS_ERR_INVALID;
  }
  int prev = -1;
  cudaGetDevice(&prev);
  cudaError_t e = cudaSetDevice(device);
  if (e == cudaSuccess && !scratch_addr[device]) {
    // In host code the array's name is only a handle; the kernel needs the device-side address,
    // looked up once per device with that device current.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, ks_noalloc_scratch);
    if (e == cudaSuccess) scratch_addr[device] = p;
  }
  if (e != cudaSuccess) {
    snprintf(msg, sizeof msg, "softcap_argmax_noalloc: set-up on device %d failed: %s", device, cudaGetErrorString(e));
    ks_set_global_error(msg);
    if (prev >= 0) cudaSetDevice(prev);
    return KS_ERR_CUDA;
  }
  unsigned* base = (unsigned*)scratch_addr[device];
  float* ws_val = (float*)base;
  unsigned* ws_idx = base + KS_NOALLOC_MAX_BLOCKS;
  unsigned* counter = base + 2 * KS_NOALLOC_MAX_BLOCKS;
  cudaStream_t st = (cudaStream_t)stream;
  // the array keeps whatever the last call left: the arrival counter has to start at zero
  e = cudaMemsetAsync(counter, 0, sizeof(unsigned), st);
  unsigned grid = (unsigned)((n + 1023) / 1024);
  if (grid > KS_NOALLOC_MAX_BLOCKS) grid = KS_NOALLOC_MAX_BLOCKS;
  if (e == cudaSuccess) {
    softcap_argmax_kernel<float><<<grid, 256, 0, st>>>((unsigned)n, cap, logits, out_idx, ws_val, ws_idx, counter);
    e = cudaGetLastError();
  }
  if (prev >= 0 && prev != device) cudaSetDevice(prev);
  if (e != cudaSuccess) {
    snprintf(msg, sizeof msg, "softcap_argmax_noalloc: launch failed: %s", cudaGetErrorString(e));
    ks_set_global_error(msg);
    return KS_ERR_CUDA;
  }
  return KS_OK;
}

// Q4_K / Q6_K weights x a batch of 9..256 token rows on the 5th-generation tensor cores (tcgen05).
//
// The reference routes matvec_batch with more than 8 rows (crates/ksearch_kernels/src/lib.rs:1414) to its
// mul_mm kernel (crates/ksearch_codegen/src/render.rs:1073-1291: 64x32 tiles, weights dequantised to half in
// threadgroup memory, simdgroup 8x8 MMA).  Here one CTA owns 128 weight rows and ALL token rows:
//   D[weight row, token] (f32, in tensor memory)  +=  A[128 rows, 16 k] . B[tokens, 16 k]^T
// with the weight rows as the M side of the MMA, so 9 tokens cost as little tensor work as the instruction
// allows (N = 16) and 256 tokens fill it (N = 256).
//   * B (token rows) is prepared once per call by x_split_kernel: every f32 x is split into two f16 terms
//     (hi = rn(x), lo = rn(x - hi)) and stored k-step by k-step in exactly the shared-memory image the MMA wants
//     (8x8 core matrices, K-major, no swizzle; per 8-k chunk the hi rows of all tokens, then the lo rows), so a
//     k-step of B is ONE cp.async.bulk into the stage.
//   * A (weights) is dequantised by the CTA's 512 threads, a quarter of a row's k-step (16 weights) each.  Q4_K:
//     bit for bit as crates/ksearch_gguf/src/gguf_impl.rs:690-721 computes it in f32, scaled by 2^6 (exact; keeps
//     the low term out of the f16 denormal range), then split like x.  Q6_K (gguf_impl.rs:761-791): in half2
//     arithmetic straight from the packed bytes (see dequant_to_stage), two f16 terms that add up to the f32 weight
//     to 2^-17.  Both are stored as core matrices.
//   * Products: Ahi.Bhi + Ahi.Blo + Alo.Bhi; the dropped lo.lo term is below 2^-22 relative, so the result matches
//     f32 arithmetic (the reference's single half operands give ~1e-3).  Up to 128 token rows the first two are ONE
//     MMA over 2 NP rows of B (the hi and lo rows of a chunk are neighbours): the accumulator has 2 NP columns, the
//     epilogue adds the halves, and the tensor core fetches the A tile twice per 16 k instead of three times.
//   * Warp-specialised: 16 warps dequantise into two A stages and signal each one full on an mbarrier (one arrival
//     per warp); the first lane of a 17th warp waits for both operands of a step, issues its MMAs and lets
//     tcgen05.commit release the step's A and B stage on one mbarrier; the first lane of an 18th warp requests the
//     token rows (ring of two or four stages) as those mbarriers complete.  No block-wide barrier inside the k
//     loop; the packed weights are fetched two k-steps ahead into registers.  The accumulator is read back with
//     tcgen05.ld, scaled by 2^-6 and stored coalesced along the weight-row index.
// Every wait is bounded; on expiry the CTA raises the context's status word, waits (bounded) for what it has in
// flight, frees its tensor memory and returns.
#include <cuda_fp16.h>

#include <cstdlib>

#include "ks_fx.cuh"

namespace {

constexpr int GM_ROWS = 128;        // weight rows per CTA (M of the MMA)
constexpr int GM_KSTEP = 64;        // k per stage: one Q4_K scale pair, half of a Q6_K 128-run
constexpr int GM_THREADS = 512;     // dequantising threads: four per weight row and k-step (two more warps: MMAs, copies)
constexpr unsigned GM_A_BYTES = 2u * 8u * GM_ROWS * 16u;  // hi + lo, 8 k-chunks, 128 rows, 16 bytes: 32 KB
constexpr unsigned GM_WAIT = 1u << 20;
constexpr float GM_SCALE = 64.0f;   // weights carry 2^6: keeps the low f16 term of small weights out of the denormal
                                    // range and the high term finite up to |w| = 1000

struct GemmArgs {
  // up to three matrices over the same columns and token rows in one launch (q, k, v; gate, up): matrix i owns
  // the row tiles [tile0[i], tile0[i + 1])
  const uint8_t* W[3];
  float* y[3];            // y[i][token * ldy[i] + row]
  size_t ldy[3];
  size_t part_stride[3];  // floats between the outputs of consecutive k splits
  unsigned rows[3], tile0[4];
  size_t row_bytes;
  const __half* xt;   // [chunks of 8 k][2][NP][8] halves
  unsigned cols, n_tok, np;        // np: token count padded to a multiple of 16 (<= 256)
  unsigned tmem_cols;              // power of two >= max(32, accumulator columns)
  unsigned ksteps_per;             // k-steps per CTA (grid.y splits the k range)
  unsigned nb;                     // stages (2..4) of the A ring and of the B ring
  unsigned wait_limit;             // polls before a wait inside the kernel gives up
  unsigned test_stall;             // test hook: the token rows of k-step test_stall - 1 of every CTA are never requested
  unsigned* err;
};

// 1 in exactly one lane of a converged warp.
__device__ __forceinline__ unsigned elect_one() {
  unsigned pred;
  asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
  return pred;
}
__device__ __forceinline__ uint32_t pack_h2(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 as_h2(uint32_t v) { return *reinterpret_cast<__half2*>(&v); }
// Eight f32 values -> 16 bytes of hi and 16 bytes of lo halves (hi = rn(v), lo = rn(v - hi)).
__device__ __forceinline__ void split8(const float (&w)[8], uint4& hi, uint4& lo) {
  uint32_t h[4], l[4];
#pragma unroll
  for (int e = 0; e < 4; e++) {
    const __half2 hh = __floats2half2_rn(w[2 * e], w[2 * e + 1]);
    const float2 hf = __half22float2(hh);
    h[e] = pack_h2(hh);
    l[e] = pack_h2(__floats2half2_rn(w[2 * e] - hf.x, w[2 * e + 1] - hf.y));
  }
  hi = make_uint4(h[0], h[1], h[2], h[3]);
  lo = make_uint4(l[0], l[1], l[2], l[3]);
}
// Eight f32 values -> token t, chunk ck of the B image: chunk c (8 k), part p (0 hi, 1 lo), token t, 8 halves.  A
// chunk's hi and lo rows are neighbours, so one MMA can take both as 2 NP rows of B.
__device__ __forceinline__ void put_split8(__half* xt, unsigned np, unsigned t, unsigned ck, const float (&v)[8]) {
  uint4 hi, lo;
  split8(v, hi, lo);
  __half* base = xt + (size_t)ck * 2u * np * 8u + (size_t)t * 8u;
  *reinterpret_cast<uint4*>(base) = hi;
  *reinterpret_cast<uint4*>(base + (size_t)np * 8u) = lo;
}

// Range.  f16 ends at 65504 and loses its low term below ~1e-3 (the low half of a small value is a denormal);
// activations do neither.  Every token row is therefore stored as x * 2^-e with e = exponent(largest magnitude) - 14,
// so the scaled row peaks in [2^14, 2^15), and the GEMM multiplies that token's outputs by 2^e (both exact).
// The factors 2^e sit behind the image, one float per (padded) token row; an all-zero row keeps e = 0.
__device__ __host__ __forceinline__ size_t xt_scale_off(unsigned cols, unsigned np) { return (size_t)cols * np * 2u; }  // in halves
__device__ __forceinline__ float row_scale_down(float row_max, float* scale_up) {
  int e = 0;
  if (row_max > 0.0f && row_max < 3.0e38f) {
    e = (int)((__float_as_uint(row_max) >> 23) & 0xFFu) - 127 - 14;
    e = e < -100 ? -100 : e;  // 2^-e must stay a float
  }
  *scale_up = __uint_as_float((unsigned)(127 + e) << 23);
  return __uint_as_float((unsigned)(127 - e) << 23);
}
__device__ __forceinline__ float block_max_f(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? red[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
  return t;
}
__device__ __forceinline__ float absmax8(const float (&v)[8]) {
  return fmaxf(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))),
               fmaxf(fmaxf(fabsf(v[4]), fabsf(v[5])), fmaxf(fabsf(v[6]), fabsf(v[7]))));
}

// x[token, k] (f32, row stride ldx) -> the B image.  One block per (padded) token row; rows past n_tok become zeros.
__global__ void __launch_bounds__(1024) x_split_kernel(const float* x, size_t ldx, unsigned n_tok, unsigned np, unsigned cols, __half* xt) {
  ks_pdl_entry();
  __shared__ float red[32];
  const unsigned t = blockIdx.x, chunks = cols / 8u;
  const bool live = t < n_tok;
  const float* row = x + (size_t)t * ldx;
  float m = 0.0f;
  if (live)
    for (unsigned ck = threadIdx.x; ck < chunks; ck += blockDim.x) {
      const float4 a = *reinterpret_cast<const float4*>(row + (size_t)ck * 8u), b = *reinterpret_cast<const float4*>(row + (size_t)ck * 8u + 4u);
      const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
      m = fmaxf(m, absmax8(v));
    }
  m = block_max_f(m, red);
  float up;
  const float down = row_scale_down(m, &up);
  if (threadIdx.x == 0) reinterpret_cast<float*>(xt + xt_scale_off(cols, np))[t] = up;
  for (unsigned ck = threadIdx.x; ck < chunks; ck += blockDim.x) {
    float v[8];
    if (live) {
      const float4 a = *reinterpret_cast<const float4*>(row + (size_t)ck * 8u), b = *reinterpret_cast<const float4*>(row + (size_t)ck * 8u + 4u);
      v[0] = a.x * down; v[1] = a.y * down; v[2] = a.z * down; v[3] = a.w * down;
      v[4] = b.x * down; v[5] = b.y * down; v[6] = b.z * down; v[7] = b.w * down;
    } else {
#pragma unroll
      for (int e = 0; e < 8; e++) v[e] = 0.0f;
    }
    put_split8(xt, np, t, ck, v);
  }
}

// ---- tcgen05 wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ void tc_alloc(uint32_t slot_smem, unsigned cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, unsigned cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] . B[smem desc]^T, f16 inputs, f32 accumulation; one thread issues.
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 8 consecutive f32 columns of this warp's 32 lanes.
__device__ __forceinline__ void tc_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Shared-memory operand descriptor, K-major, no swizzle: 8-row x 16-byte core matrices; `lbo` = bytes between the
// two 8-k chunks of one MMA, `sbo` = bytes between 8-row groups.
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr, unsigned lbo, unsigned sbo) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) |
         (1ull << 46);
}

// The packed bytes one thread needs for one k-step, fetched two steps ahead of their use.  Thread (row, quarter qd)
// owns weights [64 ks + 16 qd, +16) of its row: chunks 2 qd and 2 qd + 1 of the stage.
template <int DT>
struct Raw;
template <>
struct Raw<KS_Q4K> {
  uint4 hdr, q;  // d, dmin, 12 scale bytes; 16 bytes that hold the quarter's nibbles
};
template <>
struct Raw<KS_Q6K> {
  uint32_t ql[4], qh[4];  // the 16 bytes that hold the quarter's nibbles, the 16 bytes that hold its bit pairs
  float ds;               // 2^6 d sc of the quarter's 16-run
};

// A read-only load the compiler must issue where it is written (it may not sink it towards the first use, which is
// two k-steps later): the weights have to be in flight while the steps before them are converted.
__device__ __forceinline__ uint4 ldg_now(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_now32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ void load_raw(const uint8_t* W, size_t row_bytes, unsigned row, unsigned qd, unsigned ks, Raw<KS_Q4K>& w) {
  const uint8_t* blk = W + (size_t)row * row_bytes + (size_t)(ks >> 2) * 144u;
  w.hdr = ldg_now(blk);
  w.q = ldg_now(blk + 16u + 32u * (ks & 3u) + 16u * (qd & 1u));
}
// 16 bytes from a 2-byte-aligned address: five aligned words, shifted into place (the fifth lies inside the same
// 210-byte block wherever this is used).
__device__ __forceinline__ void load16_a2(const uint8_t* p, uint32_t (&o)[4]) {
  const unsigned sh = 8u * (unsigned)((uintptr_t)p & 3u);
  const uint32_t* q = reinterpret_cast<const uint32_t*>(p - (sh >> 3));
  const uint32_t x0 = ldg_now32(q), x1 = ldg_now32(q + 1), x2 = ldg_now32(q + 2), x3 = ldg_now32(q + 3), x4 = ldg_now32(q + 4);
  o[0] = __funnelshift_r(x0, x1, sh);
  o[1] = __funnelshift_r(x1, x2, sh);
  o[2] = __funnelshift_r(x2, x3, sh);
  o[3] = __funnelshift_r(x3, x4, sh);
}
// Q6_K: block = ql[128] qh[64] scales[16] d; a 128-run holds four groups g of 32 (gguf_impl.rs:761-791):
// group g takes nibble g >> 1 of ql[32 (g & 1) + l] and bits 2g, 2g + 1 of qh[l]; scale index 2g + (l >> 4).
__device__ __forceinline__ void load_raw(const uint8_t* W, size_t row_bytes, unsigned row, unsigned qd, unsigned ks, Raw<KS_Q6K>& w) {
  const uint8_t* blk = W + (size_t)row * row_bytes + (size_t)(ks >> 2) * 210u;  // blocks are 2-byte aligned
  const unsigned n = (ks >> 1) & 1u, g = 2u * (ks & 1u) + (qd >> 1), sub = qd & 1u;
  load16_a2(blk + 64u * n + 32u * (g & 1u) + 16u * sub, w.ql);
  load16_a2(blk + 128u + 32u * n + 16u * sub, w.qh);
  const int8_t sc = *reinterpret_cast<const int8_t*>(blk + 192u + 8u * n + 2u * g + sub);
  w.ds = __half2float(*reinterpret_cast<const __half*>(blk + 208u)) * GM_SCALE * (float)sc;
}

// 2^6 d sc and 2^6 dmin m of the four sub-blocks 2j + h (j = 0..3) of a Q4_K super-block: get_scale_min_k4
// (gguf_impl.rs:563-573) for the half h this thread always works on, decoded once per super-block instead of once
// per k-step.
struct Q4Scales {
  float dsc[4], dm[4];
};
__device__ __forceinline__ void q4k_half_scales(const uint4 hdr, unsigned h, Q4Scales& o) {
  const __half2 dd = *reinterpret_cast<const __half2*>(&hdr.x);
  const float d = __low2float(dd) * GM_SCALE, dmin = __high2float(dd) * GM_SCALE;
  const unsigned sh = 8u * h;
  // bytes q[h], q[2+h] | q[4+h], q[6+h] | q[8+h], q[10+h] of the 12 scale bytes
  const unsigned a0 = (hdr.y >> sh) & 0xFFu, a2 = (hdr.y >> (16u + sh)) & 0xFFu;
  const unsigned b0 = (hdr.z >> sh) & 0xFFu, b2 = (hdr.z >> (16u + sh)) & 0xFFu;
  const unsigned c0 = (hdr.w >> sh) & 0xFFu, c2 = (hdr.w >> (16u + sh)) & 0xFFu;
  o.dsc[0] = d * (float)(a0 & 63u);
  o.dm[0] = dmin * (float)(b0 & 63u);
  o.dsc[1] = d * (float)(a2 & 63u);
  o.dm[1] = dmin * (float)(b2 & 63u);
  o.dsc[2] = d * (float)((c0 & 0xFu) | ((a0 >> 6) << 4));
  o.dm[2] = dmin * (float)((c0 >> 4) | ((b0 >> 6) << 4));
  o.dsc[3] = d * (float)((c2 & 0xFu) | ((a2 >> 6) << 4));
  o.dm[3] = dmin * (float)((c2 >> 4) | ((b2 >> 6) << 4));
}

// The thread's 16 weights into chunks 2 qd, 2 qd + 1 of the A stage (hi and lo halves).
template <int DT>
__device__ __forceinline__ void dequant_to_stage(const Raw<DT>& w, const Q4Scales& sc4, bool live, unsigned qd, unsigned ks,
                                                 unsigned char* A, unsigned r) {
  uint4* Ahi = reinterpret_cast<uint4*>(A) + (size_t)(2u * qd) * GM_ROWS + r;
  uint4* Alo = Ahi + (size_t)8u * GM_ROWS;
  if (!live) {  // rows past the matrix: zeros (their outputs are not stored)
#pragma unroll
    for (int cc = 0; cc < 2; cc++) {
      Ahi[(size_t)cc * GM_ROWS] = make_uint4(0, 0, 0, 0);
      Alo[(size_t)cc * GM_ROWS] = make_uint4(0, 0, 0, 0);
    }
    return;
  }
  if constexpr (DT == KS_Q4K) {
    // d*sc*q - dmin*m as gguf_impl.rs:690-721 rounds it (times 2^6), then the two f16 terms
    const unsigned h = qd >> 1, j = ks & 3u;  // selects, no dynamic indexing
    const float dsc = j == 0 ? sc4.dsc[0] : j == 1 ? sc4.dsc[1] : j == 2 ? sc4.dsc[2] : sc4.dsc[3];
    const float dm = j == 0 ? sc4.dm[0] : j == 1 ? sc4.dm[1] : j == 2 ? sc4.dm[2] : sc4.dm[3];
    const unsigned sh = 4u * h;
    const uint32_t nib[4] = {(w.q.x >> sh) & 0x0F0F0F0Fu, (w.q.y >> sh) & 0x0F0F0F0Fu, (w.q.z >> sh) & 0x0F0F0F0Fu, (w.q.w >> sh) & 0x0F0F0F0Fu};
#pragma unroll
    for (int cc = 0; cc < 2; cc++) {
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; e++) {
        // one byte permute puts nibble byte e under the exponent of 2^23: the float 2^23 + q, then an exact subtract
        const float q = __uint_as_float(__byte_perm(nib[2 * cc + (e >> 2)], 0x4B000000u, 0x7440u | (unsigned)(e & 3))) - 8388608.0f;
        v[e] = __fsub_rn(__fmul_rn(dsc, q), dm);
      }
      uint4 hi, lo;
      split8(v, hi, lo);
      Ahi[(size_t)cc * GM_ROWS] = hi;
      Alo[(size_t)cc * GM_ROWS] = lo;
    }
  } else {
    // (2^6 d sc) q in half2 arithmetic: the f32 scale A is cut into A1 = A rounded to 6 significant bits (A1 q is
    // exact in f16 for q in -32..31) and A2 = A - A1 (at most 11 significant bits: exact in f16); q + 32 comes out of
    // the packed bytes as the half 0x5400 | (q + 32) << 4 = 64 + (q + 32) by one byte permute and one OR; one exact
    // add makes it q, and two multiplies give hi = A1 q (exact) and lo = rn(A2 q): hi + lo is A q to 2^-17.
    const unsigned g = 2u * (ks & 1u) + (qd >> 1);
    const __half a1 = __float2half_rn(__uint_as_float((__float_as_uint(w.ds) + 0x00020000u) & 0xFFFC0000u));
    const __half2 s1 = __half2half2(a1), s2 = __half2half2(__float2half_rn(w.ds - __half2float(a1)));
    const __half2 bias = __float2half2_rn(-96.0f);
    const unsigned shl = 4u * (1u - (g >> 1)), shh = 2u * g;
    uint32_t hi[8], lo[8];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const uint32_t tl = (w.ql[k] << shl) & 0xF0F0F0F0u;   // the nibble at bits 4..7 of its byte
      const uint32_t th = (w.qh[k] >> shh) & 0x03030303u;   // the bit pair at bits 0..1: bits 8..9 of the half
      const __half2 p0 = __hadd2(as_h2(__byte_perm(tl, th, 0x5140u) | 0x54005400u), bias);
      const __half2 p1 = __hadd2(as_h2(__byte_perm(tl, th, 0x7362u) | 0x54005400u), bias);
      hi[2 * k] = pack_h2(__hmul2(p0, s1));
      hi[2 * k + 1] = pack_h2(__hmul2(p1, s1));
      lo[2 * k] = pack_h2(__hmul2(p0, s2));
      lo[2 * k + 1] = pack_h2(__hmul2(p1, s2));
    }
#pragma unroll
    for (int cc = 0; cc < 2; cc++) {
      Ahi[(size_t)cc * GM_ROWS] = make_uint4(hi[4 * cc], hi[4 * cc + 1], hi[4 * cc + 2], hi[4 * cc + 3]);
      Alo[(size_t)cc * GM_ROWS] = make_uint4(lo[4 * cc], lo[4 * cc + 1], lo[4 * cc + 2], lo[4 * cc + 3]);
    }
  }
}

// grid = (row tiles, k splits): CTA (bx, by) multiplies rows [128 bx, +128) over k-steps [by * per, (by + 1) * per)
// and stores its sums at y + by * part_stride (a partial when there is more than one split).
// Warps 0..15 dequantise; an elected lane of warp 16 issues the MMAs; an elected lane of warp 17 requests the token rows.  Step i uses
// stage i % nb of the A ring and of the B ring (nb = 2..4); its MMAs commit to free[i % nb], which releases both.
template <int DT>
__global__ void __launch_bounds__(GM_THREADS + 64, 2) gemm_kq_tc_kernel(const GemmArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  // [0,32): mbarriers fullB[4]; [32,64): free[4]; [64,72): done; [72,104): fullA[4]; [104,108): tensor-memory address;
  // [108,112): failure flag; from 1024: the A stages, then the B stages
  const uint32_t bars = sm32(smem);
  const uint32_t bar_free = bars + 32u, bar_done = bars + 64u, bar_fullA = bars + 72u;
  uint32_t* tslot = reinterpret_cast<uint32_t*>(smem + 104);
  volatile unsigned* fail = reinterpret_cast<volatile unsigned*>(smem + 108);  // a bounded wait gave up somewhere in the CTA
  const unsigned b_bytes = a.np * 256u;                 // 8 chunks, hi + lo, np tokens, 16 bytes
  unsigned char* A0 = smem + 1024;
  const unsigned nb = a.nb;
  unsigned char* B0 = A0 + (size_t)nb * GM_A_BYTES;
  const unsigned tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
  // a producer warp takes 8 rows x 4 quarters: its 32 loads of a k-step fall into 8 runs of contiguous bytes, and the
  // 8 lanes that store together (same quarter) write 128 contiguous bytes
  const unsigned r = ((warp << 3) | (tid & 7u)) & (GM_ROWS - 1), qd = (tid >> 3) & 3u;
  // which matrix this row tile belongs to (selects, no dynamic indexing of the parameter arrays)
  const unsigned bx = blockIdx.x;
  const int seg = (bx >= a.tile0[1]) + (bx >= a.tile0[2]);
  const uint8_t* W = seg == 0 ? a.W[0] : seg == 1 ? a.W[1] : a.W[2];
  const unsigned seg_rows = seg == 0 ? a.rows[0] : seg == 1 ? a.rows[1] : a.rows[2];
  const size_t ldy = seg == 0 ? a.ldy[0] : seg == 1 ? a.ldy[1] : a.ldy[2];
  const size_t part_stride = seg == 0 ? a.part_stride[0] : seg == 1 ? a.part_stride[1] : a.part_stride[2];
  const unsigned row_base = (bx - (seg == 0 ? a.tile0[0] : seg == 1 ? a.tile0[1] : a.tile0[2])) * GM_ROWS;
  const unsigned row = row_base + r;
  const bool live = row < seg_rows;
  const unsigned ks0 = blockIdx.y * a.ksteps_per, ks1 = min(ks0 + a.ksteps_per, a.cols / GM_KSTEP);
  const unsigned ksteps = ks1 - ks0;
  float* yout = (seg == 0 ? a.y[0] : seg == 1 ? a.y[1] : a.y[2]) + (size_t)blockIdx.y * part_stride;

  // weights do not depend on the kernels before this one: the first two k-steps are fetched right away
  const bool producer = warp < GM_THREADS / 32;
  Raw<DT> raw0, raw1;
  Q4Scales sc4{};
  if (producer && live) {
    load_raw(W, a.row_bytes, row, qd, ks0, raw0);
    if (ksteps > 1) load_raw(W, a.row_bytes, row, qd, ks0 + 1, raw1);
  }
  if (tid == 0) {
    for (int i = 0; i < 9; i++) mb_init(bars + 8u * i, 1);                    // fullB[4], free[4], done: one arrival each
    for (int i = 0; i < 4; i++) mb_init(bar_fullA + 8u * i, GM_THREADS / 32);  // fullA[4]: one arrival per producer warp
    *fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) tc_alloc(sm32(tslot), a.tmem_cols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tslot;
  ks_pdl_entry();  // the B image comes from the kernel before this one

  if (producer) {
    // ---- 16 warps: packed weights -> two f16 terms -> A stage; no block-wide barrier inside the loop
    for (unsigned i = 0; i < ksteps; i++) {
      const unsigned ks = ks0 + i, s = i % nb;
      unsigned char* A = A0 + (size_t)s * GM_A_BYTES;
      if (i >= nb && !mb_wait(bar_free + 8u * s, (i / nb - 1u) & 1u, a.wait_limit)) {  // the MMAs of step i - nb still read this stage
        *fail = 1;
        break;
      }
      const Raw<DT> cur = raw0;
      raw0 = raw1;
      if (live && i + 2 < ksteps) load_raw(W, a.row_bytes, row, qd, ks + 2, raw1);  // in flight while two steps are converted
      if constexpr (DT == KS_Q4K)
        if (i == 0 || (ks & 3u) == 0) q4k_half_scales(cur.hdr, qd >> 1, sc4);  // a new super-block
      dequant_to_stage<DT>(cur, sc4, live, qd, ks, A, r);
      __syncwarp();
      if (lane == 0) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the warp's generic-proxy stores of A, then the tensor core's reads
        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar_fullA + 8u * s) : "memory");
      }
    }
  } else if (warp == GM_THREADS / 32) {
    // ---- the MMAs of a step as soon as both operands are there.  The whole warp runs the loop, converged, and one
    // elected lane issues: the loop state and the 64-bit descriptors then live in uniform registers, which is where
    // tcgen05.mma reads them (computed inside a one-lane branch they are moved there one by one, ~150 cycles per MMA).
    const unsigned leader = elect_one();
    const uint32_t idesc = (1u << 4) | ((a.np >> 3) << 17) | ((unsigned)(GM_ROWS >> 4) << 24);  // f32 accumulate, f16 x f16, K-major both
    // up to 128 token rows: the hi and lo rows of B go through ONE instruction as 2 NP rows (columns [0, NP) take
    // Ahi.Bhi, columns [NP, 2 NP) Ahi.Blo), so the tensor core fetches the A tile twice per 16 k instead of three times
    const bool cat = a.np <= 128u;
    const uint32_t idesc2 = (1u << 4) | ((a.np >> 2) << 17) | ((unsigned)(GM_ROWS >> 4) << 24);
    // descriptors of the first chunk pair of stage 0; the address field counts 16-byte units and shared memory ends
    // below its 14 bits, so the other stages and chunks are plain additions
    const uint64_t a_desc0 = tc_desc(sm32(A0), GM_ROWS * 16u, 128u), b_desc0 = tc_desc(sm32(B0), 2u * a.np * 16u, 128u);
    bool ok = true;
    for (unsigned i = 0; i < ksteps; i++) {
      const unsigned t = i % nb, s = t;
      const bool got = mb_wait(bars + 8u * t, (i / nb) & 1u, a.wait_limit) && mb_wait(bar_fullA + 8u * s, (i / nb) & 1u, a.wait_limit);
      if (!__all_sync(0xffffffffu, got)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint64_t a_hi = a_desc0 + (uint64_t)(s * (GM_A_BYTES >> 4)), b_hi = b_desc0 + (uint64_t)(t * (b_bytes >> 4));
      if (leader) {
#pragma unroll
        for (unsigned j = 0; j < 4; j++) {  // 16 k each: chunks 2j, 2j+1
          const uint64_t ah = a_hi + (uint64_t)(2u * j * GM_ROWS);
          const uint64_t al = ah + (uint64_t)(8u * GM_ROWS);
          const uint64_t bh = b_hi + (uint64_t)(4u * j * a.np);  // chunk 2j: 2 NP rows of 16 bytes each
          if (cat) {
            tc_mma_f16(tmem, ah, bh, idesc2, (i | j) ? 1u : 0u);
          } else {
            tc_mma_f16(tmem, ah, bh, idesc, (i | j) ? 1u : 0u);
            tc_mma_f16(tmem, ah, bh + (uint64_t)a.np, idesc, 1u);
          }
          tc_mma_f16(tmem, al, bh, idesc, 1u);
        }
        tc_commit(bar_free + 8u * t);
        if (i + 1 == ksteps) tc_commit(bar_done);
      }
      __syncwarp();
    }
    if (!ok) {
      // every MMA issued so far must finish before shared and tensor memory go away (bounded): a fresh commit tracks them all
      if (leader) {
        *fail = 1;
        tc_commit(bar_done);
      }
      __syncwarp();
      mb_wait(bar_done, 0u, a.wait_limit);
    }
  } else if (warp == GM_THREADS / 32 + 1) {
    // ---- token rows of step j into B stage j % nb, as soon as the MMAs of step j - nb are done (whole warp in the
    // loop, one elected lane issues)
    const unsigned leader = elect_one();
    unsigned issued = 0;
    for (unsigned j = 0; j < ksteps; j++) {
      const bool got = j < nb || mb_wait(bar_free + 8u * (j % nb), (j / nb - 1u) & 1u, a.wait_limit);
      if (!__all_sync(0xffffffffu, got)) {
        if (leader) *fail = 1;
        break;
      }
      const bool withheld = a.test_stall && j + 1 == a.test_stall;  // test hook: this step's token rows never arrive
      if (leader) {
        const uint32_t fb = bars + 8u * (j % nb);
        mb_expect(fb, b_bytes);
        if (!withheld) bulk_in(sm32(B0 + (size_t)(j % nb) * b_bytes), a.xt + (size_t)(ks0 + j) * (b_bytes / 2u), b_bytes, fb);
      }
      if (withheld) break;  // nothing to wait for at the end either
      issued++;
      __syncwarp();
    }
    // the copies must have landed before this CTA's shared memory goes away (bounded; all done already unless a wait gave up)
    for (unsigned j = issued > nb ? issued - nb : 0u; j < issued; j++) mb_wait(bars + 8u * (j % nb), (j / nb) & 1u, a.wait_limit);
  }
  __syncthreads();
  bool ok = *fail == 0;
  // all MMAs done (tcgen05.commit tracks every MMA issued before it)
  if (ok && !mb_wait(bar_done, 0u, a.wait_limit)) ok = false;
  tc_fence_after();
  if (ok && producer) {
    // warp w reads lanes 32 (w % 4) .. +31; the four warps of a lane quarter take every fourth 8-column group
    const unsigned lane_base = (warp & 3u) * 32u;
    const unsigned out_row = row_base + lane_base + lane;
    const float* up = reinterpret_cast<const float*>(a.xt + xt_scale_off(a.cols, a.np));  // 2^e of every token row
    for (unsigned c0 = (warp >> 2) * 8u; c0 < a.np; c0 += 32u) {
      uint32_t v[8], v2[8];
      tc_ld8(tmem + (lane_base << 16) + c0, v);
      if (a.np <= 128u) {
        tc_ld8(tmem + (lane_base << 16) + a.np + c0, v2);  // the columns that took Ahi.Blo
      } else {
#pragma unroll
        for (unsigned e = 0; e < 8; e++) v2[e] = 0u;
      }
      if (out_row < seg_rows) {
#pragma unroll
        for (unsigned e = 0; e < 8; e++)
          if (c0 + e < a.n_tok)
            yout[(size_t)(c0 + e) * ldy + out_row] = (__uint_as_float(v[e]) + __uint_as_float(v2[e])) * ((1.0f / GM_SCALE) * up[c0 + e]);
      }
    }
  } else if (!ok && tid == 0) {
    atomicOr(a.err, 8u);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tc_dealloc(tmem, a.tmem_cols);
}

// Sum of the k-split partials in split order (the result does not depend on how the CTAs were scheduled), then
// the epilogue.  mode 0: up to three matrices, y[i] = sum of P[i]; mode 1: y[0] = gelu(sum of P[0]) * (sum of P[1])
// (lib.rs:953, the GeGLU of gate and up).
struct FinishArgs {
  const float* P[3];
  float* y[3];
  size_t ldy[3], part_stride[3];
  unsigned rows[3], n_seg, splits, n_tok;
  int mode;
};
__global__ void gemm_finish_kernel(const FinishArgs f) {
  ks_pdl_entry();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t n0 = (size_t)f.n_tok * f.rows[0], n1 = f.n_seg > 1 && f.mode == 0 ? (size_t)f.n_tok * f.rows[1] : 0,
               n2 = f.n_seg > 2 && f.mode == 0 ? (size_t)f.n_tok * f.rows[2] : 0;
  if (i >= n0 + n1 + n2) return;
  const int seg = (i >= n0) + (i >= n0 + n1);
  i -= seg == 0 ? 0 : seg == 1 ? n0 : n0 + n1;
  const unsigned rows = seg == 0 ? f.rows[0] : seg == 1 ? f.rows[1] : f.rows[2];
  const float* P = seg == 0 ? f.P[0] : seg == 1 ? f.P[1] : f.P[2];
  const size_t ps = seg == 0 ? f.part_stride[0] : seg == 1 ? f.part_stride[1] : f.part_stride[2];
  const unsigned t = (unsigned)(i / rows), r = (unsigned)(i % rows);
  const size_t at = (size_t)t * rows + r;  // partials are dense [split][token][row]
  float g = 0.0f;
  for (unsigned s = 0; s < f.splits; s++) g += P[(size_t)s * ps + at];
  if (f.mode == 1) {
    float u = 0.0f;
    for (unsigned s = 0; s < f.splits; s++) u += f.P[1][(size_t)s * f.part_stride[1] + at];
    g = gelu_mul(g, u);
  }
  float* y = seg == 0 ? f.y[0] : seg == 1 ? f.y[1] : f.y[2];
  y[(size_t)t * (seg == 0 ? f.ldy[0] : seg == 1 ? f.ldy[1] : f.ldy[2]) + r] = g;
}

}  // namespace

namespace {
// The sum of a matrix's k-split partials straight into what consumes it, one block per token row:
//   y = sum of partials;  x = res + rms(y) * w_post (lower.rs:3926-4077, the residual update of lib.rs:539);
//   the image of rms(x) * w_norm for the next GEMM.
// The f32 normed vector is not stored: on this path only a GEMM reads it.  Rows past n_tok become zeros.
struct EpiNormArgs {
  const float* P;
  size_t part_stride;
  unsigned splits, n_tok, np, rows;
  const float *res, *w_post, *w_norm;
  float eps;
  float* out_x;
  __half* xt;
};
__global__ void gemm_finish_norm_split_kernel(const EpiNormArgs e) {
  ks_pdl_entry();
  __shared__ float red[32];
  const unsigned t = blockIdx.x, ck = threadIdx.x, chunks = e.rows / 8u;
  const bool live = ck < chunks && t < e.n_tok;
  float y[8];
#pragma unroll
  for (int i = 0; i < 8; i++) y[i] = 0.0f;
  const size_t at = (size_t)t * e.rows + 8u * ck;
  if (live)
    for (unsigned s = 0; s < e.splits; s++) {
      const float4 a = *reinterpret_cast<const float4*>(e.P + (size_t)s * e.part_stride + at);
      const float4 b = *reinterpret_cast<const float4*>(e.P + (size_t)s * e.part_stride + at + 4);
      y[0] += a.x; y[1] += a.y; y[2] += a.z; y[3] += a.w; y[4] += b.x; y[5] += b.y; y[6] += b.z; y[7] += b.w;
    }
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; i++) ss = fmaf(y[i], y[i], ss);
  ss = block_sum_f(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)e.rows + e.eps);
  float v[8], ss2 = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; i++) v[i] = 0.0f;
  if (live) {
    const float4 r0 = *reinterpret_cast<const float4*>(e.res + at), r1 = *reinterpret_cast<const float4*>(e.res + at + 4);
    const float4 p0 = *reinterpret_cast<const float4*>(e.w_post + 8u * ck), p1 = *reinterpret_cast<const float4*>(e.w_post + 8u * ck + 4);
    const float rr[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w}, pp[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
    for (int i = 0; i < 8; i++) v[i] = __fadd_rn(rr[i], __fmul_rn(__fmul_rn(y[i], inv), pp[i]));
    *reinterpret_cast<float4*>(e.out_x + at) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(e.out_x + at + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
#pragma unroll
  for (int i = 0; i < 8; i++) ss2 = fmaf(v[i], v[i], ss2);
  ss2 = block_sum_f(ss2, red);
  const float inv2 = 1.0f / sqrtf(ss2 / (float)e.rows + e.eps);
  float xn[8];
#pragma unroll
  for (int i = 0; i < 8; i++) xn[i] = 0.0f;
  if (live) {
    const float4 n0 = *reinterpret_cast<const float4*>(e.w_norm + 8u * ck), n1 = *reinterpret_cast<const float4*>(e.w_norm + 8u * ck + 4);
    const float nn[8] = {n0.x, n0.y, n0.z, n0.w, n1.x, n1.y, n1.z, n1.w};
#pragma unroll
    for (int i = 0; i < 8; i++) xn[i] = __fmul_rn(__fmul_rn(v[i], inv2), nn[i]);
  }
  float up;
  const float down = row_scale_down(block_max_f(absmax8(xn), red), &up);
  if (threadIdx.x == 0) reinterpret_cast<float*>(e.xt + xt_scale_off(e.rows, e.np))[t] = up;
  if (ck < chunks) {
#pragma unroll
    for (int i = 0; i < 8; i++) xn[i] *= down;
    put_split8(e.xt, e.np, t, ck, xn);
  }
}

// gelu(sum of gate partials) * (sum of up partials) (lib.rs:953) straight into the image the down GEMM reads.
constexpr int GM_GELU_CHUNKS = 2;     // 8-value chunks per thread
constexpr int GM_ROW_THREADS = 1024;  // threads of a block that writes one token row of an image: rows up to 2 * 8 * 1024 = 16384
__global__ void __launch_bounds__(GM_ROW_THREADS) gemm_finish_gelu_split_kernel(const float* P0, const float* P1, size_t part_stride, unsigned splits, unsigned n_tok,
                                              unsigned np, unsigned rows, __half* xt) {
  ks_pdl_entry();
  __shared__ float red[32];
  const unsigned t = blockIdx.x, chunks = rows / 8u;  // one block per (padded) token row
  float v[GM_GELU_CHUNKS][8];
  float m = 0.0f;
#pragma unroll
  for (int kk = 0; kk < GM_GELU_CHUNKS; kk++) {
    const unsigned ck = threadIdx.x + (unsigned)kk * blockDim.x;
#pragma unroll
    for (int k = 0; k < 8; k++) v[kk][k] = 0.0f;
    if (t < n_tok && ck < chunks) {
      float g[8], u[8];
#pragma unroll
      for (int k = 0; k < 8; k++) g[k] = u[k] = 0.0f;
      const size_t at = (size_t)t * rows + 8u * ck;
      for (unsigned s = 0; s < splits; s++) {
        const float4 a = *reinterpret_cast<const float4*>(P0 + (size_t)s * part_stride + at);
        const float4 b = *reinterpret_cast<const float4*>(P0 + (size_t)s * part_stride + at + 4);
        const float4 c = *reinterpret_cast<const float4*>(P1 + (size_t)s * part_stride + at);
        const float4 d = *reinterpret_cast<const float4*>(P1 + (size_t)s * part_stride + at + 4);
        g[0] += a.x; g[1] += a.y; g[2] += a.z; g[3] += a.w; g[4] += b.x; g[5] += b.y; g[6] += b.z; g[7] += b.w;
        u[0] += c.x; u[1] += c.y; u[2] += c.z; u[3] += c.w; u[4] += d.x; u[5] += d.y; u[6] += d.z; u[7] += d.w;
      }
#pragma unroll
      for (int k = 0; k < 8; k++) v[kk][k] = gelu_mul(g[k], u[k]);
      m = fmaxf(m, absmax8(v[kk]));
    }
  }
  // gelu(gate) * up is where a random-weight model leaves the f16 range
  float up;
  const float down = row_scale_down(block_max_f(m, red), &up);
  if (threadIdx.x == 0) reinterpret_cast<float*>(xt + xt_scale_off(rows, np))[t] = up;
#pragma unroll
  for (int kk = 0; kk < GM_GELU_CHUNKS; kk++) {
    const unsigned ck = threadIdx.x + (unsigned)kk * blockDim.x;
    if (ck < chunks) {
#pragma unroll
      for (int k = 0; k < 8; k++) v[kk][k] *= down;
      put_split8(xt, np, t, ck, v[kk]);
    }
  }
}
}  // namespace

namespace {
unsigned gemm_np(int n_tok) { return ((unsigned)n_tok + 15u) / 16u * 16u; }
// Shared memory of one CTA and its stage count (A and B rings have the same depth): two stages when that lets two
// CTAs share an SM (measured: a third stage that still lets them does not pay), else as many (up to four) as one CTA fits.
size_t gemm_smem(const ks_ctx* ctx, unsigned np, unsigned* nb_out) {
  const size_t stage = (size_t)GM_A_BYTES + (size_t)np * 256, per_sm = ctx->smem_optin + 1024;  // the SM holds 1 KB more than a CTA may ask for
  auto bytes = [&](size_t n) { return 1024 + n * stage; };
  auto two_fit = [&](size_t n) { return 2 * (bytes(n) + 1024) <= per_sm; };  // each resident CTA costs 1 KB on top
  if (bytes(2) > ctx->smem_optin) return 0;
  size_t nb = 2;
  if (!two_fit(2))
    while (nb < 4 && bytes(nb + 1) <= ctx->smem_optin) nb++;
  if (nb_out) *nb_out = (unsigned)nb;
  return bytes(nb);
}
// k splits of a launch over `tiles` row tiles: the count that minimises rounds x (k-steps per CTA + a fixed
// start-up and epilogue cost of about three k-steps); two CTAs that share an SM cost each other about a fifth.
unsigned gemm_splits(const ks_ctx* ctx, size_t rows, size_t cols, int n_tok) {
  const unsigned tiles = (unsigned)((rows + GM_ROWS - 1) / GM_ROWS), ksteps = (unsigned)(cols / GM_KSTEP);
  const size_t smem = gemm_smem(ctx, gemm_np(n_tok), nullptr);
  const unsigned cps = smem && 2 * (smem + 1024) <= ctx->smem_optin + 1024 ? 2u : 1u;
  const unsigned sms = (unsigned)ctx->sm_count, slots = sms * cps;
  if (const char* f = getenv("KSEARCH_GEMM_SPLITS")) {  // measurement override
    const unsigned s = (unsigned)atoi(f);
    if (s >= 1 && s <= 16 && s * 2 <= (ksteps < 2 ? 2 : ksteps)) return s;
  }
  unsigned best = 1;
  double best_cost = 1e30;
  for (unsigned s = 1; s <= 16 && s * 2 <= (ksteps < 2 ? 2 : ksteps); s++) {
    const unsigned per = (ksteps + s - 1) / s, real = (ksteps + per - 1) / per;
    if (real != s) continue;  // this count leaves a split empty
    const unsigned ctas = tiles * s, rounds = (ctas + slots - 1) / slots;
    const double cost = (double)rounds * (per + 3) * (cps == 2 && ctas > sms ? 1.2 : 1.0);
    if (cost < best_cost * 0.97) {
      best_cost = cost;
      best = s;
    }
  }
  return best;
}
bool gemm_covers(ks_dtype wdtype, size_t cols, int n_tok) {
  return (wdtype == KS_Q4K || wdtype == KS_Q6K) && cols % 256 == 0 && n_tok >= 1 && n_tok <= 256;
}
}  // namespace

// Bytes of the B image of n_tok rows of `cols` values (hi + lo halves, token count padded to 16).
size_t ks_gemm_xt_bytes(size_t cols, int n_tok) { return cols * gemm_np(n_tok) * 4 + (size_t)gemm_np(n_tok) * 4; }  // image + one factor per row

// x[t * ldx + k] (f32) -> the B image in xt.
int ks_launch_gemm_split(ks_ctx* ctx, const float* x, size_t ldx, int n_tok, size_t cols, void* xt) {
  if (cols % 256 || n_tok < 1 || n_tok > 256 || ldx % 4) return ks_fail(ctx, KS_ERR_INVALID, "gemm: bad operand shape");
  const unsigned np = gemm_np(n_tok);
  KS_LAUNCH(ctx, (x_split_kernel), np, GM_ROW_THREADS, 0, x, ldx, (unsigned)n_tok, np, (unsigned)cols, (__half*)xt);
  return ks_after_launch(ctx, "x_split");
}

// Up to three matrices over the same columns in one launch.  With one k split matrix i's result goes straight to
// y[i] (row stride ldy[i]); otherwise the partials go to P (dense [split][token][row] per matrix, matrix after
// matrix) and a second launch sums them in split order into y.  mode 1 (two matrices, gate and up): y[0] =
// gelu(gate) * up, always through P.  `xt` is the image ks_launch_gemm_split made of the same token rows.
int ks_launch_gemm_segs(ks_ctx* ctx, ks_dtype wdtype, int n_seg, const uint8_t* const* W, const size_t* rows, size_t cols, const void* xt,
                        int n_tok, float* const* y, const size_t* ldy, float* P, int mode, const ks_gemm_epi* epi) {
  if (!gemm_covers(wdtype, cols, n_tok) || n_seg < 1 || n_seg > 3) return ks_fail(ctx, KS_ERR_UNSUPPORTED, "gemm: shape not covered");
  if ((mode == KS_GEMM_NORM_SPLIT && (n_seg != 1 || !epi || rows[0] % 8 || rows[0] > 8192)) ||
      (mode == KS_GEMM_GELU_SPLIT && (n_seg != 2 || !epi || rows[0] != rows[1] || rows[0] % 8 || rows[0] > 8u * GM_GELU_CHUNKS * GM_ROW_THREADS)))
    return ks_fail(ctx, KS_ERR_INVALID, "gemm: bad epilogue arguments");
  GemmArgs a{};
  FinishArgs f{};
  unsigned tiles = 0;
  size_t total_rows = 0;
  for (int i = 0; i < 3; i++) {
    a.tile0[i] = tiles;
    if (i < n_seg) {
      a.W[i] = W[i];
      a.rows[i] = (unsigned)rows[i];
      tiles += (unsigned)((rows[i] + GM_ROWS - 1) / GM_ROWS);
      total_rows += rows[i];
    }
  }
  a.tile0[3] = tiles;
  for (int i = n_seg; i < 3; i++) a.tile0[i] = 0xFFFFFFFFu;  // no tile reaches an absent matrix
  a.row_bytes = cols / 256 * (wdtype == KS_Q4K ? 144 : 210);
  a.xt = (const __half*)xt;
  a.cols = (unsigned)cols;
  a.n_tok = (unsigned)n_tok;
  a.np = gemm_np(n_tok);
  a.tmem_cols = 32;  // the accumulator: 2 NP columns up to 128 token rows (hi and lo products side by side), NP beyond
  while (a.tmem_cols < (a.np <= 128 ? 2 * a.np : a.np)) a.tmem_cols <<= 1;
  const unsigned ksteps = (unsigned)(cols / GM_KSTEP);
  unsigned splits = gemm_splits(ctx, total_rows, cols, n_tok);
  a.ksteps_per = (ksteps + splits - 1) / splits;
  splits = (ksteps + a.ksteps_per - 1) / a.ksteps_per;
  const bool direct = splits == 1 && mode == KS_GEMM_PLAIN;
  size_t poff = 0;
  for (int i = 0; i < n_seg; i++) {
    if (direct) {
      a.y[i] = y[i];
      a.ldy[i] = ldy[i];
      a.part_stride[i] = 0;
    } else {
      a.y[i] = P + poff;
      a.ldy[i] = rows[i];
      a.part_stride[i] = (size_t)n_tok * rows[i];
      f.P[i] = a.y[i];
      f.part_stride[i] = a.part_stride[i];
      f.rows[i] = (unsigned)rows[i];
      if (mode == KS_GEMM_PLAIN || mode == KS_GEMM_GELU) {
        f.y[i] = mode == KS_GEMM_GELU ? y[0] : y[i];
        f.ldy[i] = mode == KS_GEMM_GELU ? ldy[0] : ldy[i];
      }
      poff += (size_t)splits * n_tok * rows[i];
    }
  }
  a.err = (unsigned*)ctx->ws + KS_WS_ERR_WORD;
  a.wait_limit = GM_WAIT;
  if (const char* t = getenv("KSEARCH_GEMM_TEST_STALL")) {  // exercises the give-up path: short waits, one operand withheld
    a.test_stall = (unsigned)atoi(t);
    if (a.test_stall) a.wait_limit = 4000;
  }
  const size_t smem = gemm_smem(ctx, a.np, &a.nb);
  if (!smem) return ks_fail(ctx, KS_ERR_UNSUPPORTED, "gemm: %u token rows do not fit the shared memory", a.np);
  auto kern = wdtype == KS_Q4K ? gemm_kq_tc_kernel<KS_Q4K> : gemm_kq_tc_kernel<KS_Q6K>;
  static size_t smem_set[2][16] = {{0}};
  size_t& set = smem_set[wdtype == KS_Q4K ? 0 : 1][ctx->device & 15];
  if (smem > set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "gemm: cannot set %zu B shared memory: %s", smem, cudaGetErrorString(e));
    set = smem;
  }
  KS_LAUNCH(ctx, kern, dim3(tiles, splits), GM_THREADS + 64, smem, a);
  int rc = ks_after_launch(ctx, "gemm_kq_tc");
  if (rc || direct) return rc;
  if (mode == KS_GEMM_NORM_SPLIT) {
    EpiNormArgs e{};
    e.P = a.y[0];
    e.part_stride = a.part_stride[0];
    e.splits = splits;
    e.n_tok = (unsigned)n_tok;
    e.np = a.np;
    e.rows = (unsigned)rows[0];
    e.res = epi->res;
    e.w_post = epi->w_post;
    e.w_norm = epi->w_norm;
    e.eps = epi->eps;
    e.out_x = epi->out_x;
    e.xt = (__half*)epi->xt_out;
    KS_LAUNCH(ctx, (gemm_finish_norm_split_kernel), a.np, (unsigned)((rows[0] / 8 + 31) / 32 * 32), 0, e);
    return ks_after_launch(ctx, "gemm_finish_norm_split");
  }
  if (mode == KS_GEMM_GELU_SPLIT) {
    KS_LAUNCH(ctx, (gemm_finish_gelu_split_kernel), a.np, GM_ROW_THREADS, 0, (const float*)a.y[0], (const float*)a.y[1],
              a.part_stride[0], splits, (unsigned)n_tok, a.np, (unsigned)rows[0], (__half*)epi->xt_out);
    return ks_after_launch(ctx, "gemm_finish_gelu_split");
  }
  f.n_seg = (unsigned)n_seg;
  f.splits = splits;
  f.n_tok = (unsigned)n_tok;
  f.mode = mode;
  const size_t n = (size_t)n_tok * (mode == KS_GEMM_GELU ? rows[0] : total_rows);
  KS_LAUNCH(ctx, (gemm_finish_kernel), (unsigned)((n + 255) / 256), 256, 0, f);
  return ks_after_launch(ctx, "gemm_finish");
}

// Floats of partials ks_launch_gemm_segs may write for matrices of `total_rows` rows in all.
size_t ks_gemm_part_floats(const ks_ctx* ctx, size_t total_rows, size_t cols, int n_tok) {
  return (size_t)gemm_splits(ctx, total_rows, cols, n_tok) * (size_t)n_tok * total_rows;
}

// y[t * ldy + r] = sum_k W[r, k] x[t * ldx + k] for t < n_tok (<= 256), f32 x and y: operand split, GEMM and, when
// the k range was split, the ordered sum of the partials.  `scratch`: ks_gemm_xt_bytes + 4 * ks_gemm_part_floats.
int ks_launch_gemm_kq(ks_ctx* ctx, ks_dtype wdtype, size_t rows, size_t cols, const uint8_t* W, const float* x, size_t ldx, float* y,
                      size_t ldy, int n_tok, void* scratch) {
  if (!gemm_covers(wdtype, cols, n_tok) || ldx % 4) return 1;
  int rc = ks_launch_gemm_split(ctx, x, ldx, n_tok, cols, scratch);
  if (rc) return rc;
  float* P = (float*)((char*)scratch + ks_gemm_xt_bytes(cols, n_tok));
  return ks_launch_gemm_segs(ctx, wdtype, 1, &W, &rows, cols, scratch, n_tok, &y, &ldy, P, KS_GEMM_PLAIN, nullptr);
}

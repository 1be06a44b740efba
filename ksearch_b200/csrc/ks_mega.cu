// One persistent kernel for all layers of a decode token (single slot, f32 activations).
//
// The op order is forward_token's (crates/ksearch_gemma/src/gemma_prim.rs:923-1197) for dense,
// KV-owning layers; what changes is WHERE the boundaries between ops are.  On B200 a token is a
// chain of ~180 dependent steps, each a few hundred kilobytes to ten megabytes of weights, and a
// kernel boundary costs more than most of those steps take.  Here one block per SM stays resident
// for the whole token:
//   * the weight stream never stops: every warp owns a ring of shared-memory stages fed by
//     cp.async.bulk, and walks ONE item list for the whole token (all its row groups of all phases);
//     the copies of the next phases are already in flight while the block waits at a barrier;
//   * phases (qkv | attention | o-proj | gate-up | down, per layer) are separated by a grid barrier
//     on one global counter; activations cross it through global memory (L2), read with ld.cg;
//     one hop has no barrier: q/k/v go to the attention blocks as 64-bit (value, tag) words written
//     with relaxed stores and polled by their consumers (a hop of ~1 us instead of ~2 us);
//   * the norms are applied while x is staged; their weights are fetched BEFORE the barrier wait,
//     because the acquire that ends the wait drops the SM's L1 and every later plain load of a
//     constant would be a full round trip to L2;
//   * for the same reason nothing on the critical path reads a descriptor from global memory: the
//     five phase shapes and the per-layer pointers are copied to shared memory once;
//   * attention: per-head RMS + RoPE + Q4_0 pack of the new K/V row, split-context online softmax
//     and the merge of the splits (last arriving block) happen inside one phase.
// Every spin (barrier, tagged word, mbarrier) is bounded; on expiry the block raises the context's status word,
// drains its copies and leaves, and the other blocks time out the same way.
#include <utility>
#include <vector>

#include "ks_mv_common.cuh"

namespace {

enum { MG_MATVEC = 0, MG_GATE_UP = 1, MG_ATTN = 2 };
enum { PH_QKV = 0, PH_ATTN = 1, PH_OPROJ = 2, PH_GATEUP = 3, PH_DOWN = 4, PH_PER_LAYER = 5 };

struct MegaShape {          // one of the five phases of a layer; the same for every layer
  int type;
  int n_seg;                // matvec: 1 or 3 (q, k, v)
  unsigned rows[3];
  unsigned grp_start[4];    // first group of each segment, [n_seg] = total groups (0 for attention)
  unsigned cols, row_bytes, seg_blocks, n_cseg;
  int oct;                  // 1: a block owns runs of 8 consecutive groups (32 rows = one sub-block of the next phase's x)
  int split;                // gate-up only, 1: the gate rows and the up rows of a group are two items (rows too long for one slot)
};

struct MegaLayer {          // per-layer pointers, copied to shared memory when the kernel starts
  const uint8_t* W[7];      // wq, wk, wv, wo, wgate, wup, wdown (Q4_K)
  const float* norm[6];     // attn_norm, q_norm, k_norm, post_attn_norm, ffn_norm, post_ffw_norm
  uint8_t *kv_k, *kv_v;     // this slot's cache rows [max_seq, n_kv, hd] Q4_0
};

struct MegaArgs {
  const void* tables;       // MegaShape[5] then MegaLayer[n_layers], 16-byte aligned; copied to shared memory at start
  unsigned tables_bytes;    // multiple of 16
  int n_layers;
  int stages;               // ring slots per warp
  unsigned slot_bytes;      // bytes per ring slot
  unsigned x_bytes;         // staging area for x (also the attention scratch)
  unsigned n_q, n_kv, hd, n_splits;
  float eps, attn_scale;
  const float* rope;        // [max_seq, hd]
  const int* pos;           // [1]
  float *x_a, *x_b;         // residual stream: layers read x_a / write x_b at the FFN, the reverse at the next qkv
  float *yb, *q, *k, *v;
  unsigned char *ox, *ffx;  // attention output and GeGLU output, written by their producers in the staged fixed-point layout
  float* att_tmp;           // [n_q * n_splits * (hd + 2)]
  float4* nsum;             // [grid] per-block sums of the last o-proj / down phase: (sum y^2, sum x*y*wp, sum (y*wp)^2, sum x^2)
  unsigned* att_cnt;        // [n_q] arrival counters of the attention blocks, per head
  unsigned* bar;            // [0] running barrier counter, [1] its value when the previous token ended
  unsigned* err;
  unsigned long long* qkv_t;  // q | k | v rows of the current layer as (tag << 32 | f32 bits) words: the q/k/v phase hands
                              // them to the attention blocks without a grid barrier, consumers poll for the tag
  unsigned poll_limit;      // polls of the barrier counter (or of a tagged word) before a wait gives up
  unsigned test_stall;      // test hook: the barrier before phase 1 waits for this many arrivals more than ever come
  long long* prof;          // [2][phases][8] SM clocks of the first and last block: start, staged, computed, released
                            // (attention rows: 4..7 = q/k/v ready, positions done, folded, arrived)
};

__device__ __forceinline__ uint32_t sm32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mb_init(uint32_t bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mb_expect(uint32_t bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mb_wait(uint32_t bar, unsigned parity) {
  for (unsigned i = 0; i < (1u << 22); i++) {
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
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ldcg4(const float* p, unsigned c) { return __ldcg(reinterpret_cast<const float4*>(p) + c); }
// A value and its tag in one 64-bit word: single-copy atomic, so a consumer that sees the tag sees the value; no fence.
__device__ __forceinline__ void tag_store(unsigned long long* p, float v, unsigned tag) {
  const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
  asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long tag_load(const unsigned long long* p) {
  unsigned long long w;
  asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
  return w;
}
// Four tagged words per lane until every tag matches; false when the limit ran out.
__device__ __forceinline__ bool tag_wait4(const unsigned long long* base, int i0, int i1, int i2, int i3, unsigned tag, unsigned limit,
                                          float& o0, float& o1, float& o2, float& o3) {
  for (unsigned it = 0; it < limit; it++) {
    const unsigned long long w0 = tag_load(base + i0), w1 = tag_load(base + i1), w2 = tag_load(base + i2), w3 = tag_load(base + i3);
    if ((unsigned)(w0 >> 32) == tag && (unsigned)(w1 >> 32) == tag && (unsigned)(w2 >> 32) == tag && (unsigned)(w3 >> 32) == tag) {
      o0 = __uint_as_float((unsigned)w0);
      o1 = __uint_as_float((unsigned)w1);
      o2 = __uint_as_float((unsigned)w2);
      o3 = __uint_as_float((unsigned)w3);
      return true;
    }
  }
  o0 = o1 = o2 = o3 = 0.0f;
  return false;
}

// Grid-wide barrier on a monotonically increasing counter, in two halves so that loads which do not
// depend on other blocks can be issued in between.
// wsum != nullptr: the eight warps left their partial norm sums there; thread 0 folds them (fixed order) into nsum[block].
__device__ __forceinline__ void grid_arrive(unsigned* counter, const float4* wsum, float4* nsum) {
  __syncthreads();  // every store of this block is issued
  if (threadIdx.x == 0) {
    if (wsum) {
      float4 t = wsum[0];
#pragma unroll
      for (int w = 1; w < 8; w++) {
        const float4 u = wsum[w];
        t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
      }
      nsum[blockIdx.x] = t;
    }
    // release: everything this block wrote (ordered before by the barrier above) is visible to whoever
    // acquires the counter; nothing comes back, so the thread does not wait for a round trip
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(counter) : "memory");
  }
}
// Returns false when the wait gave up.
// Lane 0 of four warps polls: their loads drift apart in time, so the arrival of the last block is
// seen sooner than one poller's round trip allows.  sflag: 0 = waiting, 1 = released, 2 = gave up.
// Two flag words alternate between consecutive barriers, so a word is cleared a whole phase after its last reader.
__device__ __forceinline__ bool grid_wait(unsigned* counter, unsigned target, unsigned* err, int* flags, int parity, unsigned limit) {
  int* sflag = flags + parity;
  if (threadIdx.x == 0) flags[parity ^ 1] = 0;
  if ((threadIdx.x & 31) == 0 && threadIdx.x < 128) {
    volatile int* vf = sflag;
    int state = 0;
    for (unsigned i = 0; i < limit; i++) {  // a second or two of polling at most
      if ((int)(ld_acquire_u32(counter) - target) >= 0) {
        state = 1;
        break;
      }
      if (*vf == 1) {  // another poller saw it; take the acquire ourselves before reading what other blocks wrote
        if ((int)(ld_acquire_u32(counter) - target) >= 0) {
          state = 1;
          break;
        }
      }
    }
    if (state == 1) {
      *vf = 1;
    } else {
      atomicOr(err, 2u);
      *vf = 2;
    }
  }
  __syncthreads();
  return *sflag == 1;
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
constexpr int MG_RL = 4, MG_LPR = 8;  // 8 lanes per row, 4 rows side by side
constexpr unsigned MG_XU = 80;  // bytes per unit and plane
__device__ __forceinline__ void fx_put_chunk(unsigned char* xs, unsigned units, unsigned c, float4 v) {
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
// The same layout written to GLOBAL memory by a producer: the warp holds the 32 consecutive elements
// e0 .. e0+31 of one sub-block, one per lane (e0 a multiple of 32).
__device__ __forceinline__ void fx_store_subblock(unsigned char* dst, unsigned units, unsigned e0, float val, int lane) {
  float s = val, am = fabsf(val);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
  }
  const float inv = am > 0.0f ? __fdividef(8.0e6f, am) : 0.0f;
  const float sc = am > 0.0f ? am * (1.0f / 8.0e6f) : 1.0f;
  const int X = __float2int_rn(val * inv);
  const unsigned u = e0 >> 6, hi = (e0 >> 5) & 1u;
  const size_t plane = (size_t)units * MG_XU;
  unsigned char* base = dst + (size_t)u * MG_XU + hi * 32u + (unsigned)lane;
  base[0] = (unsigned char)(X & 0xFF);
  base[plane] = (unsigned char)((X >> 8) & 0xFF);
  base[2 * plane] = (unsigned char)((X >> 16) & 0xFF);
  if (lane == 0) {
    float* mt = reinterpret_cast<float*>(dst + 3 * plane + (size_t)u * 16u);
    mt[hi] = s;
    mt[2 + hi] = sc;
  }
}
// Bring a vector a producer left in that layout into shared memory (units * 256 bytes; the pad words travel too).
__device__ __forceinline__ void fx_copy_in(unsigned char* xs, const unsigned char* src, unsigned units) {
  const unsigned n16 = units * 16u;  // 3 planes of 80 bytes + 16 bytes of sums and scales per unit
  for (unsigned base = 0; base < n16; base += 6u * blockDim.x) {
    uint4 v[6];
#pragma unroll
    for (int k = 0; k < 6; k++) {
      const unsigned i = base + threadIdx.x + k * blockDim.x;
      if (i < n16) v[k] = __ldcg(reinterpret_cast<const uint4*>(src) + i);
    }
#pragma unroll
    for (int k = 0; k < 6; k++) {
      const unsigned i = base + threadIdx.x + k * blockDim.x;
      if (i < n16) reinterpret_cast<uint4*>(xs)[i] = v[k];
    }
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
// One weight word (8 nibbles: elements j..j+3 of the low and of the high sub-block) against the
// matching x words of the three planes.
__device__ __forceinline__ void fx_word(uint32_t w, unsigned xl0, unsigned xl1, unsigned xl2, unsigned xh0, unsigned xh1,
                                        unsigned xh2, unsigned (&alo)[2], int& alo2, unsigned (&ahi)[2], int& ahi2) {
  const unsigned lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
  alo[0] = dp4a_uu(lo, xl0, alo[0]);
  alo[1] = dp4a_uu(lo, xl1, alo[1]);
  alo2 = dp4a_us(lo, xl2, alo2);
  ahi[0] = dp4a_uu(hi, xh0, ahi[0]);
  ahi[1] = dp4a_uu(hi, xh1, ahi[1]);
  ahi2 = dp4a_us(hi, xh2, ahi2);
}
// Multiply-accumulate one item against the fixed-point x: MATS row slots per lane.
template <int MATS>
__device__ __forceinline__ void mg_item_compute_fx(uint32_t slot_addr, uint32_t xs_s, unsigned units, unsigned seg_blocks,
                                                   unsigned cs, int cl, int rl, float (&yacc)[2]) {
  const int g = cl & 3;
  const unsigned seg_bytes = seg_blocks * KS_Q4K_BLOCK_BYTES, seg_units = seg_blocks * 4, upl = seg_units / MG_LPR;
  const uint32_t plane = units * MG_XU;
  uint32_t waddr = slot_addr + (uint32_t)rl * seg_bytes + (uint32_t)(cl >> 2) * KS_Q4K_BLOCK_BYTES + (uint32_t)g * 32u;
  uint32_t xaddr = xs_s + (cs * seg_units + (unsigned)cl) * MG_XU;
  uint32_t maddr = xs_s + 3u * plane + (cs * seg_units + (unsigned)cl) * 16u;
  for (unsigned it = 0; it < upl; it++) {
    const float4 mt = lds_f4o<0>(maddr);
    // 16 words per plane: [0..7] low sub-block, [8..15] high sub-block
    const uint4 a0 = lds_u4o<0>(xaddr), a1 = lds_u4o<16>(xaddr), a2 = lds_u4o<32>(xaddr), a3 = lds_u4o<48>(xaddr);
    const uint4 b0 = lds_u4o<0>(xaddr + plane), b1 = lds_u4o<16>(xaddr + plane), b2 = lds_u4o<32>(xaddr + plane),
                b3 = lds_u4o<48>(xaddr + plane);
    const uint4 c0 = lds_u4o<0>(xaddr + 2 * plane), c1 = lds_u4o<16>(xaddr + 2 * plane), c2 = lds_u4o<32>(xaddr + 2 * plane),
                c3 = lds_u4o<48>(xaddr + 2 * plane);
#pragma unroll
    for (int r = 0; r < MATS; r++) {
      const uint32_t wa = waddr + (uint32_t)(r * MG_RL) * seg_bytes;
      const uint4 q0 = lds_u4o<16>(wa), q1 = lds_u4o<32>(wa);
      const uint4 hdr = lds_u4o<0>(wa - (uint32_t)g * 32u);
      unsigned alo[2] = {0u, 0u}, ahi[2] = {0u, 0u};
      int alo2 = 0, ahi2 = 0;
      fx_word(q0.x, a0.x, b0.x, c0.x, a2.x, b2.x, c2.x, alo, alo2, ahi, ahi2);
      fx_word(q0.y, a0.y, b0.y, c0.y, a2.y, b2.y, c2.y, alo, alo2, ahi, ahi2);
      fx_word(q0.z, a0.z, b0.z, c0.z, a2.z, b2.z, c2.z, alo, alo2, ahi, ahi2);
      fx_word(q0.w, a0.w, b0.w, c0.w, a2.w, b2.w, c2.w, alo, alo2, ahi, ahi2);
      fx_word(q1.x, a1.x, b1.x, c1.x, a3.x, b3.x, c3.x, alo, alo2, ahi, ahi2);
      fx_word(q1.y, a1.y, b1.y, c1.y, a3.y, b3.y, c3.y, alo, alo2, ahi, ahi2);
      fx_word(q1.z, a1.z, b1.z, c1.z, a3.z, b3.z, c3.z, alo, alo2, ahi, ahi2);
      fx_word(q1.w, a1.w, b1.w, c1.w, a3.w, b3.w, c3.w, alo, alo2, ahi, ahi2);
      const float flo = fmaf((float)alo2, 65536.0f, fmaf((float)alo[1], 256.0f, (float)alo[0])) * mt.z;
      const float fhi = fmaf((float)ahi2, 65536.0f, fmaf((float)ahi[1], 256.0f, (float)ahi[0])) * mt.w;
      yacc[r] = q4k_apply_scales(hdr, g, flo, fhi, mt.x, mt.y, yacc[r]);
    }
    waddr += (MG_LPR / 4) * KS_Q4K_BLOCK_BYTES;
    xaddr += MG_LPR * MG_XU;
    maddr += MG_LPR * 16u;
  }
}


// ---- staging of x (with the fused norm prologues), reads through L2 ---------------------------
// Norm weights of the next matvec phase, fetched into registers before the barrier wait.
template <int PC>
struct NormPre {  // PC chunks of 4 elements per thread: cols <= PC * 4 * blockDim
  float4 w[PC], wp[PC];
};
template <int PC>
__device__ __forceinline__ void mg_prefetch_norm(NormPre<PC>& n, int mode, const float* w, const float* wp, unsigned cols) {
  const unsigned nchunk = cols >> 2;
  if (mode == KS_PRO_NONE) return;
#pragma unroll
  for (int k = 0; k < PC; k++) {
    const unsigned c = threadIdx.x + k * blockDim.x;
    if (c < nchunk) {
      n.w[k] = reinterpret_cast<const float4*>(w)[c];
      if (mode == KS_PRO_ADD_NORM) n.wp[k] = reinterpret_cast<const float4*>(wp)[c];
    }
  }
}

constexpr int MG_XMAX = 8;  // plain staging keeps up to 8 chunks per thread in flight (cols <= 8192), loops beyond

// mode NONE: x' = x.  NORM: x' = rms(x)*w.  ADD_NORM: r = x + rms(y)*wp (block 0 stores r to out_x); x' = rms(r)*w.
template <int PC>
__device__ __forceinline__ void mg_stage_x(unsigned char* xs, float* red, int mode, unsigned cols, const float* x,
                                           const float* y, float* out_x, float eps, const NormPre<PC>& n) {
  const unsigned units = cols >> 6, nchunk = cols >> 2;
  if (mode == KS_PRO_NONE) {
    for (unsigned base = 0; base < nchunk; base += MG_XMAX * blockDim.x) {
      float4 v[MG_XMAX];
#pragma unroll
      for (int k = 0; k < MG_XMAX; k++) {
        const unsigned c = base + threadIdx.x + k * blockDim.x;
        if (c < nchunk) v[k] = ldcg4(x, c);
      }
#pragma unroll
      for (int k = 0; k < MG_XMAX; k++) {
        const unsigned c = base + threadIdx.x + k * blockDim.x;
        if (c < nchunk) fx_put_chunk(xs, units, c, v[k]);
      }
    }
    return;
  }
  const float invn = 1.0f / (float)cols;
  float4 v[PC], yv[PC];
  float ss = 0.0f;
  if (mode == KS_PRO_ADD_NORM) {
#pragma unroll
    for (int k = 0; k < PC; k++) {
      const unsigned c = threadIdx.x + k * blockDim.x;
      if (c < nchunk) {
        yv[k] = ldcg4(y, c);
        v[k] = ldcg4(x, c);
      }
    }
#pragma unroll
    for (int k = 0; k < PC; k++) {
      const unsigned c = threadIdx.x + k * blockDim.x;
      if (c < nchunk) {
        ss = fmaf(yv[k].x, yv[k].x, ss); ss = fmaf(yv[k].y, yv[k].y, ss);
        ss = fmaf(yv[k].z, yv[k].z, ss); ss = fmaf(yv[k].w, yv[k].w, ss);
      }
    }
    ss = block_sum_f(ss, red);
    const float inv = 1.0f / sqrtf(ss * invn + eps);
    ss = 0.0f;
#pragma unroll
    for (int k = 0; k < PC; k++) {
      const unsigned c = threadIdx.x + k * blockDim.x;
      if (c < nchunk) {
        const float4 p4 = n.wp[k];
        float4 r = v[k];
        r.x = __fadd_rn(r.x, __fmul_rn(__fmul_rn(yv[k].x, inv), p4.x));
        r.y = __fadd_rn(r.y, __fmul_rn(__fmul_rn(yv[k].y, inv), p4.y));
        r.z = __fadd_rn(r.z, __fmul_rn(__fmul_rn(yv[k].z, inv), p4.z));
        r.w = __fadd_rn(r.w, __fmul_rn(__fmul_rn(yv[k].w, inv), p4.w));
        if (blockIdx.x == 0) reinterpret_cast<float4*>(out_x)[c] = r;
        v[k] = r;
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < PC; k++) {
      const unsigned c = threadIdx.x + k * blockDim.x;
      if (c < nchunk) v[k] = ldcg4(x, c);
    }
  }
#pragma unroll
  for (int k = 0; k < PC; k++) {
    const unsigned c = threadIdx.x + k * blockDim.x;
    if (c < nchunk) {
      ss = fmaf(v[k].x, v[k].x, ss); ss = fmaf(v[k].y, v[k].y, ss);
      ss = fmaf(v[k].z, v[k].z, ss); ss = fmaf(v[k].w, v[k].w, ss);
    }
  }
  ss = block_sum_f(ss, red);
  const float inv2 = 1.0f / sqrtf(ss * invn + eps);
#pragma unroll
  for (int k = 0; k < PC; k++) {
    const unsigned c = threadIdx.x + k * blockDim.x;
    if (c < nchunk) {
      const float4 w4 = n.w[k];
      float4 r;
      r.x = __fmul_rn(__fmul_rn(v[k].x, inv2), w4.x);
      r.y = __fmul_rn(__fmul_rn(v[k].y, inv2), w4.y);
      r.z = __fmul_rn(__fmul_rn(v[k].z, inv2), w4.z);
      r.w = __fmul_rn(__fmul_rn(v[k].w, inv2), w4.w);
      fx_put_chunk(xs, units, c, r);
    }
  }
}

// ADD_NORM without any block-wide reduction: the blocks that produced y left the four sums that both
// norms need (K:539 expands to  sum r^2 = sum x^2 + 2 inv sum x y wp + inv^2 sum (y wp)^2,  r = x + inv y wp).
template <int PC>
__device__ __forceinline__ void mg_stage_addnorm(unsigned char* xs, unsigned cols, const float* x, const float* y, float* out_x,
                                                 float eps, const NormPre<PC>& n, const float4* nsum, unsigned nblocks) {
  const unsigned units = cols >> 6, nchunk = cols >> 2;
  const int lane = threadIdx.x & 31;
  float4 v[PC], yv[PC], ps[8];
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const unsigned i = (unsigned)lane + 32u * j;
    ps[j] = i < nblocks ? __ldcg(nsum + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int k = 0; k < PC; k++) {
    const unsigned c = threadIdx.x + k * blockDim.x;
    if (c < nchunk) {
      yv[k] = ldcg4(y, c);
      v[k] = ldcg4(x, c);
    }
  }
  float4 t = ps[0];
#pragma unroll
  for (int j = 1; j < 8; j++) {
    t.x += ps[j].x; t.y += ps[j].y; t.z += ps[j].z; t.w += ps[j].w;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    t.x += __shfl_xor_sync(0xffffffffu, t.x, o);
    t.y += __shfl_xor_sync(0xffffffffu, t.y, o);
    t.z += __shfl_xor_sync(0xffffffffu, t.z, o);
    t.w += __shfl_xor_sync(0xffffffffu, t.w, o);
  }
  const float invn = 1.0f / (float)cols;
  const float inv = __frsqrt_rn(t.x * invn + eps);
  const float rr = fmaf(inv * inv, t.z, fmaf(2.0f * inv, t.y, t.w));
  const float inv2 = __frsqrt_rn(fmaxf(rr, 0.0f) * invn + eps);
#pragma unroll
  for (int k = 0; k < PC; k++) {
    const unsigned c = threadIdx.x + k * blockDim.x;
    if (c < nchunk) {
      const float4 p4 = n.wp[k], w4 = n.w[k];
      float4 r = v[k];
      r.x = __fadd_rn(r.x, __fmul_rn(__fmul_rn(yv[k].x, inv), p4.x));
      r.y = __fadd_rn(r.y, __fmul_rn(__fmul_rn(yv[k].y, inv), p4.y));
      r.z = __fadd_rn(r.z, __fmul_rn(__fmul_rn(yv[k].z, inv), p4.z));
      r.w = __fadd_rn(r.w, __fmul_rn(__fmul_rn(yv[k].w, inv), p4.w));
      if (blockIdx.x == 0) reinterpret_cast<float4*>(out_x)[c] = r;
      float4 q;
      q.x = __fmul_rn(__fmul_rn(r.x, inv2), w4.x);
      q.y = __fmul_rn(__fmul_rn(r.y, inv2), w4.y);
      q.z = __fmul_rn(__fmul_rn(r.z, inv2), w4.z);
      q.w = __fmul_rn(__fmul_rn(r.w, inv2), w4.w);
      fx_put_chunk(xs, units, c, q);
    }
  }
}

// ---- the per-warp item list of a whole token -----------------------------------------------------
// Item = (phase, row group, column segment).

// The items of a warp repeat layer after layer (same shapes, other pointers), so the walk over the
// shapes is done once per kernel: each warp records its items of ONE layer, in phase order, and the
// issue and consume positions are (layer, entry) pairs.
constexpr int MG_MAX_ENT = 16;
struct ItemEnt {
  uint32_t src_off;  // byte offset of the first copy inside its weight matrix
  uint32_t pslot;    // index of this item among the block's items of the phase (where its partial sums go)
  uint16_t seg16;    // bytes of one row segment / 16
  uint8_t kind, seg, cs, valid;
  uint8_t widx;      // MegaLayer::W index of the first matrix
  uint8_t flags;     // bit 0: two matrices (gate, up) in one item; bit 1: whole rows (one copy per matrix);
                     // bit 2: this item is the second matrix (up) of a split gate-up group
};
struct ItemPos {
  int layer, e;
};
__device__ __forceinline__ void pos_next(ItemPos& c, int n_ent) {
  if (++c.e >= n_ent) {
    c.e = 0;
    c.layer++;
  }
}
// Groups of a phase go to blocks round-robin (block c owns groups c, c + grid, ...); the block's items
// -- its groups x the column segments -- go to its warps round-robin.  A row's column segments may
// therefore be multiplied by different warps; the partial sums meet in shared memory (slot pslot).
constexpr int MG_MAX_P = 64;  // items of one block in one phase
__device__ __forceinline__ unsigned block_groups(const MegaShape& sh) {
  const unsigned total = sh.type == MG_ATTN ? 0u : sh.grp_start[sh.n_seg];
  if (sh.oct) {
    const unsigned octs = (total + 7u) / 8u;
    return octs > blockIdx.x ? (octs - blockIdx.x + gridDim.x - 1) / gridDim.x * 8u : 0u;
  }
  return total > blockIdx.x ? (total - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u;
}
// global group index of this block's k-th group
__device__ __forceinline__ unsigned block_group_id(const MegaShape& sh, unsigned k) {
  return sh.oct ? (blockIdx.x + (k >> 3) * gridDim.x) * 8u + (k & 7u) : blockIdx.x + k * gridDim.x;
}
// lane 0 of each warp fills its table; returns the entry count (0 when the warp owns nothing, -1 on overflow)
__device__ __forceinline__ int build_items(ItemEnt* ent, const MegaShape* shapes, int warp) {
  int n = 0;
  for (int kind = 0; kind < PH_PER_LAYER; kind++) {
    const MegaShape& sh = shapes[kind];
    const unsigned C = sh.n_cseg, n_slots = block_groups(sh) * C;
    if (n_slots > (unsigned)MG_MAX_P) return -1;
    const unsigned seg_bytes = sh.seg_blocks * KS_Q4K_BLOCK_BYTES;
    const bool split = sh.type == MG_GATE_UP && sh.split;
    const int mats = (sh.type == MG_GATE_UP && !split) ? 2 : 1;
    const int w0 = kind == PH_QKV ? 0 : kind == PH_OPROJ ? 3 : kind == PH_GATEUP ? 4 : 6;
    const unsigned n_items = split ? n_slots * 2u : n_slots;
    for (unsigned jj = (unsigned)warp; jj < n_items; jj += 8u) {
      if (n >= MG_MAX_ENT) return -1;
      const unsigned j = split ? jj >> 1 : jj, second = split ? jj & 1u : 0u;
      const unsigned k = j / C, cs = j - k * C;
      const unsigned g = block_group_id(sh, k);
      if (g >= sh.grp_start[sh.n_seg]) continue;
      int seg = 0;
      if (sh.n_seg > 1 && g >= sh.grp_start[1]) seg = 1;
      if (sh.n_seg > 2 && g >= sh.grp_start[2]) seg = 2;
      const unsigned row0 = (g - sh.grp_start[seg]) * MG_RL;
      ItemEnt e;
      e.src_off = row0 * sh.row_bytes + cs * seg_bytes;
      e.pslot = j;
      e.seg16 = (uint16_t)(seg_bytes / 16u);
      e.kind = (uint8_t)kind;
      e.seg = (uint8_t)seg;
      e.cs = (uint8_t)cs;
      e.valid = (uint8_t)min((unsigned)MG_RL, sh.rows[seg] - row0);
      e.widx = (uint8_t)(w0 + (mats == 2 ? 0 : split ? second : seg));
      e.flags = (uint8_t)((mats == 2 ? 1 : 0) | (C == 1 ? 2 : 0) | (second ? 4 : 0));
      ent[n++] = e;
    }
  }
  return n;
}

// Start the copies of one item into a ring slot (all lanes call).
__device__ __forceinline__ void mg_issue_ent(const ItemEnt& e, const MegaLayer& L, unsigned row_bytes, uint32_t slot_addr,
                                             uint32_t bar, int lane) {
  const unsigned seg_bytes = (unsigned)e.seg16 * 16u, valid = e.valid;
  const int mats = (e.flags & 1) ? 2 : 1;
  if (lane == 0) mb_expect(bar, valid * mats * seg_bytes);
  if (e.flags & 2) {
    if (lane < mats)
      bulk_in(slot_addr + (uint32_t)lane * MG_RL * seg_bytes, L.W[e.widx + lane] + e.src_off, valid * seg_bytes, bar);
  } else if (lane < MG_RL * mats) {
    const int m = lane / MG_RL, rr = lane % MG_RL;
    if ((unsigned)rr < valid)
      bulk_in(slot_addr + (uint32_t)lane * seg_bytes, L.W[e.widx + m] + e.src_off + (size_t)rr * row_bytes, seg_bytes, bar);
  }
}

// Multiply-accumulate one item: MATS row slots per lane, units of this lane in the segment.
template <int MATS>
__device__ __forceinline__ void mg_item_compute(uint32_t slot_addr, uint32_t xs_s, unsigned units, unsigned seg_blocks,
                                                unsigned cs, int cl, int rl, float (&yacc)[2]) {
  const int g = cl & 3;
  const unsigned seg_bytes = seg_blocks * KS_Q4K_BLOCK_BYTES, seg_units = seg_blocks * 4, upl = seg_units / MG_LPR;
  uint32_t waddr = slot_addr + (uint32_t)rl * seg_bytes + (uint32_t)(cl >> 2) * KS_Q4K_BLOCK_BYTES + (uint32_t)g * 32u;
  uint32_t xaddr = xs_s + (cs * seg_units + (unsigned)cl) * (Q4K_XS * 4u);
  uint32_t saddr = xs_s + units * (Q4K_XS * 4u) + (cs * seg_units + (unsigned)cl) * 8u;
  for (unsigned it = 0; it < upl; it++) {
    const float2 sx = lds_f2a(saddr);
    u64 acc[MATS][2];
#pragma unroll
    for (int r = 0; r < MATS; r++) acc[r][0] = acc[r][1] = 0ull;
    {
      u64 xf[16];
      lds_p2o<0>(xaddr, xf[0], xf[1]);     lds_p2o<16>(xaddr, xf[2], xf[3]);
      lds_p2o<32>(xaddr, xf[4], xf[5]);    lds_p2o<48>(xaddr, xf[6], xf[7]);
      lds_p2o<64>(xaddr, xf[8], xf[9]);    lds_p2o<80>(xaddr, xf[10], xf[11]);
      lds_p2o<96>(xaddr, xf[12], xf[13]);  lds_p2o<112>(xaddr, xf[14], xf[15]);
#pragma unroll
      for (int r = 0; r < MATS; r++) {
        const uint4 q = lds_u4o<16>(waddr + (uint32_t)(r * MG_RL) * seg_bytes);
        q4_word_p(q.x, xf[0], xf[1], xf[2], xf[3], acc[r][0], acc[r][1]);
        q4_word_p(q.y, xf[4], xf[5], xf[6], xf[7], acc[r][0], acc[r][1]);
        q4_word_p(q.z, xf[8], xf[9], xf[10], xf[11], acc[r][0], acc[r][1]);
        q4_word_p(q.w, xf[12], xf[13], xf[14], xf[15], acc[r][0], acc[r][1]);
      }
    }
    {
      u64 xf[16];
      lds_p2o<128>(xaddr, xf[0], xf[1]);    lds_p2o<144>(xaddr, xf[2], xf[3]);
      lds_p2o<160>(xaddr, xf[4], xf[5]);    lds_p2o<176>(xaddr, xf[6], xf[7]);
      lds_p2o<192>(xaddr, xf[8], xf[9]);    lds_p2o<208>(xaddr, xf[10], xf[11]);
      lds_p2o<224>(xaddr, xf[12], xf[13]);  lds_p2o<240>(xaddr, xf[14], xf[15]);
#pragma unroll
      for (int r = 0; r < MATS; r++) {
        const uint4 q = lds_u4o<32>(waddr + (uint32_t)(r * MG_RL) * seg_bytes);
        q4_word_p(q.x, xf[0], xf[1], xf[2], xf[3], acc[r][0], acc[r][1]);
        q4_word_p(q.y, xf[4], xf[5], xf[6], xf[7], acc[r][0], acc[r][1]);
        q4_word_p(q.z, xf[8], xf[9], xf[10], xf[11], acc[r][0], acc[r][1]);
        q4_word_p(q.w, xf[12], xf[13], xf[14], xf[15], acc[r][0], acc[r][1]);
      }
    }
#pragma unroll
    for (int r = 0; r < MATS; r++) {
      const uint4 hdr = lds_u4o<0>(waddr + (uint32_t)(r * MG_RL) * seg_bytes - (uint32_t)g * 32u);
      const float2 a01 = unpack2(padd2(acc[r][0], acc[r][1]));
      yacc[r] = q4k_apply_scales(hdr, g, a01.x, a01.y, sx.x, sx.y, yacc[r]);
    }
    waddr += (MG_LPR / 4) * KS_Q4K_BLOCK_BYTES;
    xaddr += MG_LPR * Q4K_XS * 4u;
    saddr += MG_LPR * 8u;
  }
}

// ---- attention phase ------------------------------------------------------------------------------
constexpr float kNegInit = -1.0e30f;

__device__ __forceinline__ float mg_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float mg_warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Q4_0 pack of 32 values held one per lane (render.rs:1021-1059); blk is 2-byte aligned.
__device__ __forceinline__ void mg_pack_q40(float v, uint8_t* blk, int lane) {
  const float amax = mg_warp_max(fabsf(v));
  const float scale = amax > 0.0f ? amax / 7.0f : 1.0f;
  const float inv = 1.0f / scale;
  int q = (int)roundf(__fmul_rn(v, inv)) + 8;
  q = q < 0 ? 0 : q > 15 ? 15 : q;
  const int qhi = __shfl_down_sync(0xffffffffu, q, 16);
  if (lane < 16) blk[2 + lane] = (uint8_t)(q | (qhi << 4));
  if (lane == 0) *reinterpret_cast<__half*>(blk) = __float2half_rn(scale);
}

// This lane's share of one Q4_0 row, still packed: DPL/4 16-bit words of nibbles and the scale.
template <int DPL>
struct RawRow {
  unsigned short q[DPL / 4];
  unsigned short d;
};
template <int DPL>
__device__ __forceinline__ void raw_load(const uint8_t* row, int lane, RawRow<DPL>& r) {
  constexpr int BPL = DPL / 2, LPB = 16 / BPL;
  const uint8_t* blk = row + (lane / LPB) * KS_Q40_BLOCK_BYTES;
  r.d = *reinterpret_cast<const unsigned short*>(blk);
  const unsigned short* qs = reinterpret_cast<const unsigned short*>(blk + 2 + (lane % LPB) * BPL);
#pragma unroll
  for (int w = 0; w < BPL / 2; w++) r.q[w] = qs[w];
}
template <int DPL>
__device__ __forceinline__ void raw_decode(const RawRow<DPL>& r, float (&out)[DPL]) {
  constexpr int BPL = DPL / 2;
  const float d = __half2float(__ushort_as_half(r.d));
#pragma unroll
  for (int w = 0; w < BPL / 2; w++) {
    const unsigned v = r.q[w];
    out[2 * w] = (float)((int)(v & 0xF) - 8) * d;
    out[2 * w + 1] = (float)((int)((v >> 8) & 0xF) - 8) * d;
    out[BPL + 2 * w] = (float)((int)((v >> 4) & 0xF) - 8) * d;
    out[BPL + 2 * w + 1] = (float)((int)(v >> 12) - 8) * d;
  }
}
template <int DPL>
__device__ __forceinline__ int mg_lane_dim(int lane, int j) {
  constexpr int BPL = DPL / 2, LPB = 16 / BPL;
  const int base = (lane / LPB) * 32 + (lane % LPB) * BPL;
  return j < BPL ? base + j : base + 16 + (j - BPL);
}

constexpr int MG_MAX_SPLITS = 16;  // context splits per head (the final merge keeps one record per split in registers)

// Shared memory the attention phase needs (it reuses the x staging area).
__host__ __device__ inline unsigned mg_att_bytes(unsigned hd) {
  return 8u * (hd + 2u) * 4u + 2u * ((hd / 32u) * KS_Q40_BLOCK_BYTES + 16u) + 32u;
}

// Splits in use for a context of tlen positions: one row per warp (8 per block) until every split is
// in use, more rows per warp beyond that.
__host__ __device__ inline unsigned mg_active_splits(unsigned tlen, unsigned max_splits) {
  unsigned ns = (tlen + 7u) / 8u;
  return ns < 1u ? 1u : ns > max_splits ? max_splits : ns;
}

// One block per (query head, context split): the work of a short context is tiny, so it is spread
// as widely as the grid allows and every serial step stays short.
//   1. every warp builds the roped, normed, scaled q of the head in registers (no exchange needed);
//      in the blocks of the split that holds the newest position, warps 0.. pack the new K row and
//      warps 4.. the new V row to Q4_0 in shared memory (lower.rs:4231-4702), block pairs (b, b+NB/2)
//      per warp because RoPE pairs those halves; the block of the KV group's first head stores them;
//   2. warps take the positions of the split round-robin, online softmax per warp;
//   3. the eight warps' (m, l, O) meet in shared memory, thread d folds dimension d;
//   4. the block leaves a (m, l, O[hd]) record; the last block of a head to arrive merges the
//      head's records (lower.rs:5897-6088).
template <int DPL>
__device__ __forceinline__ void mg_attention(const MegaArgs& a, const MegaLayer& L, unsigned char* sm, int* sflag, long long* pf,
                                             unsigned tag) {
  constexpr int HD = DPL * 32, HALF = HD / 2, NB = HD / 32;
  constexpr unsigned ROWB = NB * KS_Q40_BLOCK_BYTES;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned NSMAX = a.n_splits;
  if (blockIdx.x >= a.n_q * NSMAX) return;
  const unsigned head = blockIdx.x / NSMAX, split = blockIdx.x % NSMAX;
  const unsigned G = a.n_q / a.n_kv, kvh = head / G;
  const unsigned pos = (unsigned)a.pos[0], tlen = pos + 1;
  const unsigned NS = mg_active_splits(tlen, NSMAX);
  if (split >= NS) return;
  const unsigned chunk = (tlen + NS - 1) / NS;
  const unsigned p0 = split * chunk, p1 = min(p0 + chunk, tlen);
  const bool owner = pos >= p0 && pos < p1;  // the split that holds the newest position
  float* part = reinterpret_cast<float*>(sm);     // [8][HD + 2]
  uint8_t* skrow = reinterpret_cast<uint8_t*>(part + 8 * (HD + 2));
  uint8_t* svrow = skrow + ROWB + 16u;
  const float* cs = a.rope + (size_t)pos * HD;

  float qr[DPL];
  {
    const int pb = warp & 3;  // block pair of the K / V job
    const bool kjob = owner && warp < 4 && pb < NB / 2, vjob = owner && warp >= 4 && pb < NB / 2;
    float qv[DPL], qw[DPL], qc[DPL], qs[DPL], rv[DPL], r_w0 = 0.f, r_w1 = 0.f, r_c = 0.f, r_s = 0.f;
    const float* qnw = L.norm[1];
#pragma unroll
    for (int j = 0; j < DPL; j++) {  // constants first: they are on their way while the tagged words are polled
      const int d = mg_lane_dim<DPL>(lane, j);
      qw[j] = qnw[d];
      qc[j] = cs[d & (HALF - 1)];
      qs[j] = cs[HALF + (d & (HALF - 1))];
    }
    // q (and, in the owner split, k / v) arrive as tagged words straight from the blocks that computed them
    bool got = true;
    {
      const unsigned long long* qsrc = a.qkv_t + (size_t)head * HD;
#pragma unroll
      for (int j = 0; j < DPL; j += 4)
        got = tag_wait4(qsrc, mg_lane_dim<DPL>(lane, j), mg_lane_dim<DPL>(lane, j + 1), mg_lane_dim<DPL>(lane, j + 2),
                        mg_lane_dim<DPL>(lane, j + 3), tag, a.poll_limit, qv[j], qv[j + 1], qv[j + 2], qv[j + 3]) && got;
    }
    if (kjob || vjob) {
      const unsigned long long* src = a.qkv_t + (size_t)a.n_q * HD + (kjob ? 0u : (size_t)a.n_kv * HD) + (size_t)kvh * HD;
#pragma unroll
      for (int j = 0; j < DPL; j += 4)
        got = tag_wait4(src, lane + 32 * j, lane + 32 * (j + 1), lane + 32 * (j + 2), lane + 32 * (j + 3), tag, a.poll_limit, rv[j],
                        rv[j + 1], rv[j + 2], rv[j + 3]) && got;
      if (kjob) {
        const float* w = L.norm[2];
        r_w0 = w[32 * pb + lane];
        r_w1 = w[HALF + 32 * pb + lane];
        r_c = cs[32 * pb + lane];
        r_s = cs[HALF + 32 * pb + lane];
      }
    }
    if (!got) atomicOr(a.err, 2u);  // a tagged word never came: the values are zeros, the status word tells the host
    {
      float ss = 0.0f;
#pragma unroll
      for (int j = 0; j < DPL; j++) ss = fmaf(qv[j], qv[j], ss);
      ss = mg_warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)HD + a.eps);
      // lanes 0..15 hold dims of the first half, lanes 16..31 their RoPE partners (dim + HD/2)
#pragma unroll
      for (int j = 0; j < DPL; j++) {
        const float u = __fmul_rn(__fmul_rn(qv[j], inv), qw[j]);
        const float pu = __shfl_xor_sync(0xffffffffu, u, 16);
        const float r = lane < 16 ? __fsub_rn(__fmul_rn(u, qc[j]), __fmul_rn(pu, qs[j]))
                                  : __fadd_rn(__fmul_rn(pu, qs[j]), __fmul_rn(u, qc[j]));
        qr[j] = r * a.attn_scale;
      }
    }
    if (kjob || vjob) {
      float ss = 0.0f;
#pragma unroll
      for (int j = 0; j < DPL; j++) ss = fmaf(rv[j], rv[j], ss);
      ss = mg_warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss / (float)HD + a.eps);
      float x0 = 0.f, x1 = 0.f;  // this lane's element of block pb and of block pb + NB/2
#pragma unroll
      for (int j = 0; j < DPL / 2; j++)
        if (j == pb) {
          x0 = rv[j];
          x1 = rv[j + DPL / 2];
        }
      float lo, hi;
      if (kjob) {
        const float u = __fmul_rn(__fmul_rn(x0, inv), r_w0), vv = __fmul_rn(__fmul_rn(x1, inv), r_w1);
        lo = __fsub_rn(__fmul_rn(u, r_c), __fmul_rn(vv, r_s));
        hi = __fadd_rn(__fmul_rn(u, r_s), __fmul_rn(vv, r_c));
      } else {
        lo = __fmul_rn(x0, inv);
        hi = __fmul_rn(x1, inv);
      }
      uint8_t* dst = kjob ? skrow : svrow;
      // values pass through f16 before packing (render.rs:1046)
      mg_pack_q40(__half2float(__float2half_rn(lo)), dst + pb * KS_Q40_BLOCK_BYTES, lane);
      mg_pack_q40(__half2float(__float2half_rn(hi)), dst + (pb + NB / 2) * KS_Q40_BLOCK_BYTES, lane);
    }
  }
  const size_t rowstride = (size_t)a.n_kv * ROWB;
  uint8_t* Kc = L.kv_k + (size_t)kvh * ROWB;
  uint8_t* Vc = L.kv_v + (size_t)kvh * ROWB;
  if (owner) {
    __syncthreads();
    if (head == kvh * G) {
      const unsigned n16 = ROWB / 2;
      if (threadIdx.x < n16)
        reinterpret_cast<unsigned short*>(Kc + (size_t)pos * rowstride)[threadIdx.x] = reinterpret_cast<const unsigned short*>(skrow)[threadIdx.x];
      else if (threadIdx.x < 2 * n16)
        reinterpret_cast<unsigned short*>(Vc + (size_t)pos * rowstride)[threadIdx.x - n16] =
            reinterpret_cast<const unsigned short*>(svrow)[threadIdx.x - n16];
    }
  }
  if (pf) pf[4] = clock64();

  float o[DPL], m = kNegInit, l = 0.0f;
#pragma unroll
  for (int j = 0; j < DPL; j++) o[j] = 0.0f;
  {
    RawRow<DPL> kn, vn;  // next row, in flight while the current one is processed
    unsigned t = p0 + warp;
    if (t < p1) {
      raw_load<DPL>(t == pos ? skrow : Kc + (size_t)t * rowstride, lane, kn);
      raw_load<DPL>(t == pos ? svrow : Vc + (size_t)t * rowstride, lane, vn);
    }
#pragma unroll 1
    for (; t < p1; t += 8) {
      const RawRow<DPL> kr = kn, vr = vn;
      const unsigned t2 = t + 8;
      if (t2 < p1) {
        raw_load<DPL>(t2 == pos ? skrow : Kc + (size_t)t2 * rowstride, lane, kn);
        raw_load<DPL>(t2 == pos ? svrow : Vc + (size_t)t2 * rowstride, lane, vn);
      }
      float kv[DPL];
      raw_decode<DPL>(kr, kv);
      float sc = 0.0f;
#pragma unroll
      for (int j = 0; j < DPL; j++) sc = fmaf(qr[j], kv[j], sc);
      sc = mg_warp_sum(sc);
      raw_decode<DPL>(vr, kv);
      const float m2 = fmaxf(m, sc);
      const float alpha = __expf(m - m2);
      const float e = __expf(sc - m2);
      l = l * alpha + e;
      m = m2;
#pragma unroll
      for (int j = 0; j < DPL; j++) o[j] = fmaf(e, kv[j], o[j] * alpha);
    }
  }
  {
    float* dst = part + warp * (HD + 2);
    if (lane == 0) {
      dst[0] = m;
      dst[1] = l;
    }
#pragma unroll
    for (int j = 0; j < DPL; j++) dst[2 + j * 32 + lane] = o[j];
  }
  __syncthreads();
  if (pf) pf[5] = clock64();
  // thread d folds head dimension d over the eight warps; it sits in slot j * 32 + lane of the warps' layout
  const int d = threadIdx.x;
  int dslot;
  {
    constexpr int BPL = DPL / 2, LPB = 16 / BPL;
    const int within = d & 31, hh = within >> 4, w16 = within & 15;
    dslot = (hh * BPL + (w16 % BPL)) * 32 + ((d >> 5) * LPB + w16 / BPL);
  }
  const unsigned ounits = (a.n_q * HD) >> 6;
  float M = kNegInit, Lsum = 0.0f, O = 0.0f;
  if (d < HD) {
    float mw[8];
#pragma unroll
    for (int w = 0; w < 8; w++) {
      mw[w] = part[w * (HD + 2)];
      M = fmaxf(M, mw[w]);
    }
#pragma unroll
    for (int w = 0; w < 8; w++) {
      const float f = __expf(mw[w] - M);
      Lsum = fmaf(part[w * (HD + 2) + 1], f, Lsum);
      O = fmaf(part[w * (HD + 2) + 2 + dslot], f, O);
    }
  }
  if (pf) pf[6] = clock64();
  if (NS == 1) {  // one split: this block's result is final
    if (d < HD) fx_store_subblock(a.ox, ounits, head * HD + (d & ~31), O / Lsum, lane);
    return;
  }
  float* rec = a.att_tmp + ((size_t)head * NSMAX + split) * (HD + 2);
  if (d < HD) {
    rec[2 + d] = O;  // records are kept in dimension order
    if (d == 0) {
      rec[0] = M;
      rec[1] = Lsum;
    }
    __threadfence();
  }
  __syncthreads();
  if (threadIdx.x == 0) *sflag = (atomicAdd(a.att_cnt + head, 1u) == NS - 1) ? 1 : 0;
  __syncthreads();
  if (pf) pf[7] = clock64();
  if (*sflag) {
    // last block of this head to arrive: merge the head's records, every load first
    __threadfence();
    if (d < HD) {
      const float* rec0 = a.att_tmp + (size_t)head * NSMAX * (HD + 2);
      float mp[MG_MAX_SPLITS], lp[MG_MAX_SPLITS], ov[MG_MAX_SPLITS];
#pragma unroll
      for (int p = 0; p < MG_MAX_SPLITS; p++) {
        if ((unsigned)p < NS) {
          const float* r = rec0 + (size_t)p * (HD + 2);
          mp[p] = __ldcg(r);
          lp[p] = __ldcg(r + 1);
          ov[p] = __ldcg(r + 2 + d);
        } else {
          mp[p] = kNegInit;
          lp[p] = 0.0f;
          ov[p] = 0.0f;
        }
      }
      float MM = kNegInit;
#pragma unroll
      for (int p = 0; p < MG_MAX_SPLITS; p++) MM = fmaxf(MM, mp[p]);
      float LL = 0.0f, OO = 0.0f;
#pragma unroll
      for (int p = 0; p < MG_MAX_SPLITS; p++) {
        const float f = __expf(mp[p] - MM);
        LL = fmaf(lp[p], f, LL);
        OO = fmaf(ov[p], f, OO);
      }
      fx_store_subblock(a.ox, ounits, head * HD + (d & ~31), OO / LL, lane);
    }
    if (threadIdx.x == 0) a.att_cnt[head] = 0u;
  }
}

// ---- the kernel -------------------------------------------------------------------------------------
struct MegaSmem {
  unsigned ring_off, bar_off, red_off, flag_off, tab_off, ent_off, total;
};
__host__ __device__ inline MegaSmem mg_smem(unsigned x_bytes, unsigned slot_bytes, int stages, unsigned tables_bytes) {
  MegaSmem L;
  L.ring_off = (x_bytes + 127u) & ~127u;
  L.bar_off = L.ring_off + 8u * (unsigned)stages * slot_bytes;
  L.red_off = (L.bar_off + 8u * 8u * (unsigned)stages + 15u) & ~15u;
  L.flag_off = L.red_off + 256u + MG_MAX_P * 32u;  // 32 floats for block sums, 8 float4 of per-warp norm sums, partial sums [MG_MAX_P][2][4]
  L.tab_off = L.flag_off + 48u;  // 4 flag words, then 8 words of per-kind group counts
  L.ent_off = L.tab_off + tables_bytes;
  L.total = L.ent_off + 8u * MG_MAX_ENT * (unsigned)sizeof(ItemEnt);
  return L;
}

template <int DPL, int PC>
__global__ void __launch_bounds__(256, 1) mega_kernel(const MegaArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cl = lane % MG_LPR, rl = lane / MG_LPR;
  const int S = a.stages;
  const MegaSmem SL = mg_smem(a.x_bytes, a.slot_bytes, S, a.tables_bytes);
  const uint32_t ring_s = sm32(smem + SL.ring_off) + (uint32_t)(warp * S) * a.slot_bytes;
  const uint32_t bars = sm32(smem + SL.bar_off) + (uint32_t)(warp * S) * 8u;
  float* red = reinterpret_cast<float*>(smem + SL.red_off);
  float4* wsum = reinterpret_cast<float4*>(smem + SL.red_off + 128u);
  float* psum = reinterpret_cast<float*>(smem + SL.red_off + 256u);
  int* sflag = reinterpret_cast<int*>(smem + SL.flag_off);
  const MegaShape* shapes = reinterpret_cast<const MegaShape*>(smem + SL.tab_off);
  const MegaLayer* layers = reinterpret_cast<const MegaLayer*>(smem + SL.tab_off + ((PH_PER_LAYER * sizeof(MegaShape) + 15u) & ~15u));
  const uint32_t xs_s = sm32(smem);
  const unsigned bar_base = a.bar[1];
  const int n_phases = a.n_layers * PH_PER_LAYER;

  for (unsigned i = threadIdx.x; i < a.tables_bytes / 16u; i += blockDim.x)
    reinterpret_cast<uint4*>(smem + SL.tab_off)[i] = reinterpret_cast<const uint4*>(a.tables)[i];
  if (threadIdx.x == 0) sflag[2] = sflag[3] = 0;  // barrier flag words ([0] belongs to the attention phase)
  unsigned* ngrp = reinterpret_cast<unsigned*>(smem + SL.flag_off + 16u);  // this block's group count per phase kind
  if (threadIdx.x < PH_PER_LAYER) ngrp[threadIdx.x] = 0;
  if (lane == 0) {
    for (int s = 0; s < S; s++) mb_init(bars + s * 8u, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x < PH_PER_LAYER) ngrp[threadIdx.x] = block_groups(shapes[threadIdx.x]);
  const unsigned H = shapes[PH_QKV].cols;

  ItemEnt* ent = reinterpret_cast<ItemEnt*>(smem + SL.ent_off) + warp * MG_MAX_ENT;
  int n_ent = 0;
  if (lane == 0) n_ent = build_items(ent, shapes, warp);
  n_ent = __shfl_sync(0xffffffffu, n_ent, 0);
  bool dead = false;  // this warp gave up (a copy never landed, or its item table overflowed): it keeps the block-level steps only
  if (n_ent < 0) {
    dead = true;
    if (lane == 0) atomicOr(a.err, 4u);
    n_ent = 0;
  }
  __syncwarp();
  ItemPos ic{n_ent > 0 ? 0 : a.n_layers, 0}, cc = ic;
  unsigned issued = 0, consumed = 0;
  while (issued < (unsigned)S && ic.layer < a.n_layers) {
    const ItemEnt e = ent[ic.e];
    mg_issue_ent(e, layers[ic.layer], shapes[e.kind].row_bytes, ring_s + issued * a.slot_bytes, bars + issued * 8u, lane);
    issued++;
    pos_next(ic, n_ent);
  }

  long long* prof = nullptr;
  if (threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1))
    prof = a.prof + (size_t)(blockIdx.x == 0 ? 0 : 1) * n_phases * 8;
  int p = 0, layer = 0, kind = 0;
  // tag of this token's words: position and layer; a slot reset clears the words, so a replayed position never
  // meets its own old tags
  const unsigned tag_base = (((unsigned)a.pos[0] + 1u) << 8) + 1u;
  for (; p < n_phases; p++) {
    const MegaLayer& L = layers[layer];
    // constants of this phase, fetched while the other blocks arrive at the barrier before it
    NormPre<PC> npre;
    if (kind == PH_QKV)
      mg_prefetch_norm(npre, layer == 0 ? KS_PRO_NORM : KS_PRO_ADD_NORM, L.norm[0], layers[layer > 0 ? layer - 1 : 0].norm[5], H);
    else if (kind == PH_GATEUP)
      mg_prefetch_norm(npre, KS_PRO_ADD_NORM, L.norm[4], L.norm[3], H);
    // No barrier in front of attention: its inputs are tagged words.  Every block still ARRIVES after every phase,
    // so the targets of the barriers that remain are unchanged; the flag word this wait would have cleared is
    // cleared all the same.  (The parity stays `p & 1`: written as a separate counter the same logic compiles into
    // a kernel that is 40 % slower.)
    if (p > 0 && kind == PH_ATTN) {
      if (threadIdx.x == 0) sflag[2 + ((p & 1) ^ 1)] = 0;
    } else if (p > 0) {
      if (!grid_wait(a.bar, bar_base + (unsigned)p * gridDim.x + (p == 2 ? a.test_stall : 0u), a.err, sflag + 2, p & 1, a.poll_limit)) break;
      if (prof) prof[(p - 1) * 8 + 3] = clock64();
    }
    if (prof) prof[p * 8 + 0] = clock64();
    if (kind == PH_ATTN) {
      mg_attention<DPL>(a, L, smem, sflag, prof ? prof + p * 8 : nullptr, tag_base + (unsigned)layer);
    } else {
      const MegaShape& sh = shapes[kind];
      // input, prologue and outputs of this phase
      int mode = KS_PRO_NONE;
      const float* x;
      const float* yin = a.yb;
      float* out_x = nullptr;
      if (kind == PH_QKV) {
        mode = layer == 0 ? KS_PRO_NORM : KS_PRO_ADD_NORM;
        x = layer == 0 ? a.x_a : a.x_b;
        out_x = a.x_a;
      } else if (kind == PH_OPROJ) {
        x = nullptr;
      } else if (kind == PH_GATEUP) {
        mode = KS_PRO_ADD_NORM;
        x = a.x_a;
        out_x = a.x_b;
      } else {
        x = nullptr;
      }
      if (kind == PH_OPROJ || kind == PH_DOWN)
        fx_copy_in(smem, kind == PH_OPROJ ? a.ox : a.ffx, sh.cols >> 6);
      else if (mode == KS_PRO_ADD_NORM)
        mg_stage_addnorm(smem, sh.cols, x, yin, out_x, a.eps, npre, a.nsum, gridDim.x);
      else
        mg_stage_x(smem, red, mode, sh.cols, x, yin, out_x, a.eps, npre);
      __syncthreads();
      if (prof) prof[p * 8 + 1] = clock64();
      const unsigned units = sh.cols >> 6;
      // o-proj and down feed a residual-add + norm: their rows also leave the sums that norm needs
      const bool sums = kind == PH_OPROJ || kind == PH_DOWN;
      // Thread f finishes row (f & 3) of this block's group (f >> 2): it adds the column segments'
      // partial sums in order, applies the epilogue and stores the row.
      const unsigned n_g = ngrp[kind], C = sh.n_cseg;
      unsigned frow = 0;
      int fseg = 0;
      bool fin = false;
      float xr = 0.0f, wpr = 0.0f;
      if ((threadIdx.x >> 2) < n_g) {
        const unsigned g = block_group_id(sh, threadIdx.x >> 2);
        if (sh.n_seg > 1 && g >= sh.grp_start[1]) fseg = 1;
        if (sh.n_seg > 2 && g >= sh.grp_start[2]) fseg = 2;
        frow = (g - sh.grp_start[fseg]) * MG_RL + (threadIdx.x & 3u);
        fin = g < sh.grp_start[sh.n_seg] && frow < sh.rows[fseg];
        if (fin && sums) {  // in flight while the items are multiplied
          xr = __ldcg((kind == PH_OPROJ ? a.x_a : a.x_b) + frow);
          wpr = (kind == PH_OPROJ ? L.norm[3] : L.norm[5])[frow];
        }
      }
      while (cc.layer == layer && !dead) {
        const ItemEnt e = ent[cc.e];
        if (e.kind != kind) break;
        const unsigned st = consumed % (unsigned)S;
        if (!mb_wait(bars + st * 8u, (consumed / (unsigned)S) & 1u)) {
          dead = true;
          if (lane == 0) atomicOr(a.err, 1u);
          break;
        }
        const uint32_t slot = ring_s + st * a.slot_bytes;
        float yacc[2] = {0.0f, 0.0f};
        if (e.flags & 1)
          mg_item_compute_fx<2>(slot, xs_s, units, sh.seg_blocks, e.cs, cl, rl, yacc);
        else
          mg_item_compute_fx<1>(slot, xs_s, units, sh.seg_blocks, e.cs, cl, rl, yacc);
        consumed++;
        float v0 = yacc[0], v1 = yacc[1];
#pragma unroll
        for (int o = MG_LPR / 2; o > 0; o >>= 1) {
          v0 += __shfl_xor_sync(0xffffffffu, v0, o);
          v1 += __shfl_xor_sync(0xffffffffu, v1, o);
        }
        if (cl == 0) {
          if (e.flags & 4) {
            psum[e.pslot * 8u + 4u + (unsigned)rl] = v0;  // the up rows of a split gate-up group
          } else {
            psum[e.pslot * 8u + (unsigned)rl] = v0;
            if (e.flags & 1) psum[e.pslot * 8u + 4u + (unsigned)rl] = v1;
          }
        }
        pos_next(cc, n_ent);
        // Refill now only when the next item of THIS phase is not in flight yet; everything else is
        // refilled after the barrier arrival below, off the critical path.
        if (ic.layer == layer && ent[ic.e].kind == kind) {
          __syncwarp();
          if (lane == 0) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the slot was read through the generic proxy
          __syncwarp();
          const ItemEnt ne = ent[ic.e];
          mg_issue_ent(ne, layers[ic.layer], sh.row_bytes, slot, bars + st * 8u, lane);
          issued++;
          pos_next(ic, n_ent);
        }
      }
      __syncthreads();  // the partial sums of every item of this block are in shared memory
      float ns0 = 0.0f, ns1 = 0.0f, ns2 = 0.0f, ns3 = 0.0f, fval = 0.0f;
      if (fin) {
        const float* ps = psum + (size_t)(threadIdx.x >> 2) * C * 8u + (threadIdx.x & 3u);
        float v0 = 0.0f, v1 = 0.0f;
        for (unsigned cs = 0; cs < C; cs++) {
          v0 += ps[cs * 8u];
          v1 += ps[cs * 8u + 4u];
        }
        fval = sh.type == MG_GATE_UP ? gelu_mul(v0, v1) : v0;
        const float val = fval;
        if (kind == PH_QKV) {  // handed to the attention blocks as tagged words (no barrier follows this phase)
          const size_t at = fseg == 0 ? 0u : fseg == 1 ? (size_t)a.n_q * a.hd : (size_t)(a.n_q + a.n_kv) * a.hd;
          tag_store(a.qkv_t + at + frow, val, tag_base + (unsigned)layer);
        } else if (kind != PH_GATEUP) {
          a.yb[frow] = val;
        }
        if (sums) {
          const float t = val * wpr;
          ns0 = val * val;
          ns1 = xr * t;
          ns2 = t * t;
          ns3 = xr * xr;
        }
      }
      if (kind == PH_GATEUP && (threadIdx.x >> 2) < n_g) {
        // this warp's 32 threads hold 32 consecutive rows (a run of 8 groups): one sub-block of the next phase's x
        const unsigned g0 = block_group_id(sh, (threadIdx.x >> 2) & ~7u);
        if (g0 < sh.grp_start[1]) fx_store_subblock(a.ffx, sh.rows[0] >> 6, g0 * MG_RL, fval, lane);
      }
      if (sums) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          ns0 += __shfl_xor_sync(0xffffffffu, ns0, o);
          ns1 += __shfl_xor_sync(0xffffffffu, ns1, o);
          ns2 += __shfl_xor_sync(0xffffffffu, ns2, o);
          ns3 += __shfl_xor_sync(0xffffffffu, ns3, o);
        }
        if (lane == 0) wsum[warp] = make_float4(ns0, ns1, ns2, ns3);
      }
    }
    if (prof) prof[p * 8 + 2] = clock64();
    if (p + 1 == n_phases) {  // the end of the kernel orders the last phase before whatever follows
      p++;
      break;
    }
    grid_arrive(a.bar, (kind == PH_OPROJ || kind == PH_DOWN) ? wsum : nullptr, a.nsum);
    // refill the ring while the other blocks arrive
    if (!dead && issued - consumed < (unsigned)S && ic.layer < a.n_layers) {
      if (lane == 0) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      while (issued - consumed < (unsigned)S && ic.layer < a.n_layers) {
        const unsigned st = issued % (unsigned)S;
        const ItemEnt ne = ent[ic.e];
        mg_issue_ent(ne, layers[ic.layer], shapes[ne.kind].row_bytes, ring_s + st * a.slot_bytes, bars + st * 8u, lane);
        issued++;
        pos_next(ic, n_ent);
      }
    }
    if (++kind == PH_PER_LAYER) {
      kind = 0;
      layer++;
    }
  }
  if (p == n_phases && blockIdx.x == 0 && threadIdx.x == 0) a.bar[1] = bar_base + (unsigned)(n_phases - 1) * gridDim.x;
  // copies still in flight must land before this block's shared memory goes away (bounded)
  for (unsigned j = consumed; j < issued; j++) mb_wait(bars + (j % (unsigned)S) * 8u, (j / (unsigned)S) & 1u);
}

}  // namespace

// ---- host side --------------------------------------------------------------------------------------
struct ks_mega {
  MegaArgs args{};
  void* d_tables = nullptr;
  unsigned* d_sync = nullptr;  // words 0..1 barrier (a 128-byte line of its own: every block polls it), 64..111 per-head
                               // attention arrival counters, from byte 512: per-block norm sums
  long long* d_prof = nullptr;
  unsigned long long* d_qkv = nullptr;  // tagged q | k | v words
  size_t qkv_words = 0;
  unsigned char* d_fx = nullptr;  // attention output and GeGLU output in the staged layout
  unsigned grid = 0;
  size_t smem = 0;
  int G = 0, dpl = 0, pc = 4;  // pc: 4-element chunks of the hidden vector per thread (2 up to 2048 columns)
  float* residual = nullptr;  // buffer that holds the residual stream when the kernel ends
};

namespace {
template <int DPL, int PC>
int mega_launch_t(ks_ctx* ctx, ks_mega* mg) {
  auto kern = mega_kernel<DPL, PC>;
  static size_t smem_set[16] = {0};
  if (mg->smem > smem_set[ctx->device & 15]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mg->smem);
    if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "decode kernel: cannot set %zu B shared memory: %s", mg->smem, cudaGetErrorString(e));
    smem_set[ctx->device & 15] = mg->smem;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(mg->grid);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = mg->smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // every block resident: the grid barrier needs it
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, mg->args);
  if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "decode kernel launch failed: %s", cudaGetErrorString(e));
  return ks_after_launch(ctx, "decode_layers");
}
}  // namespace

int ks_mega_launch(ks_ctx* ctx, ks_mega* mg) {
  if (mg->dpl == 4) return mg->pc == 2 ? mega_launch_t<4, 2>(ctx, mg) : mega_launch_t<4, 4>(ctx, mg);
  if (mg->dpl == 8) return mg->pc == 2 ? mega_launch_t<8, 2>(ctx, mg) : mega_launch_t<8, 4>(ctx, mg);
  return ks_fail(ctx, KS_ERR_UNSUPPORTED, "decode kernel: head size not supported");
}

float* ks_mega_residual(const ks_mega* mg) { return mg->residual; }

// Zero the barrier words and arrival counters (stream-ordered).  They only leave their rest state when
// a bounded wait gave up; a slot reset puts the kernel back in working order.
int ks_mega_reset(ks_ctx* ctx, ks_mega* mg) {
  cudaError_t e = cudaMemsetAsync(mg->d_sync, 0, 512, ctx->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(mg->d_qkv, 0, mg->qkv_words * sizeof(unsigned long long), ctx->stream);  // no stale tags
  if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "decode kernel: reset failed: %s", cudaGetErrorString(e));
  return KS_OK;
}
const long long* ks_mega_prof(const ks_mega* mg) { return mg->d_prof; }

// Test knobs (the next launch sees them; graphs captured before must be dropped by the caller):
// 0 = polls before a barrier wait gives up, 1 = make the first barrier of a token wait for `value`
// arrivals that never come (exercises the give-up path; 0 switches it off).  2 and 3 belong to the
// dataflow kernel (attention split point, stamps on or off) and are accepted without effect.
int ks_mega_set(ks_mega* mg, int what, unsigned value) {
  if (what == 0) mg->args.poll_limit = value ? value : 1u;
  else if (what == 1) mg->args.test_stall = value;
  else if (what != 2 && what != 3) return KS_ERR_INVALID;
  return KS_OK;
}

void ks_mega_destroy(ks_mega* mg) {
  if (!mg) return;
  if (mg->d_tables) cudaFree(mg->d_tables);
  if (mg->d_sync) cudaFree(mg->d_sync);
  if (mg->d_qkv) cudaFree(mg->d_qkv);
  if (mg->d_prof) cudaFree(mg->d_prof);
  if (mg->d_fx) cudaFree(mg->d_fx);
  delete mg;
}

// Returns KS_OK and *out == nullptr when the shape is outside what the kernel covers (the caller keeps
// the launch-per-op path), a negative code on a CUDA failure.
int ks_mega_create(ks_ctx* ctx, const ks_mega_desc* d, const ks_mega_layer* layers, ks_mega** out) {
  *out = nullptr;
  const unsigned H = d->hidden, F = d->ffn, hd = d->hd, nq = d->n_q, nkv = d->n_kv;
  const unsigned qn = nq * hd, kvn = nkv * hd;
  const unsigned G = nq / nkv;
  auto even_blocks = [](unsigned cols) { return cols % 512 == 0; };
  if (!even_blocks(H) || !even_blocks(F) || !even_blocks(qn)) return KS_OK;
  if (H > 16u * 256u) return KS_OK;  // the fused norms hold the vector in registers
  if (G < 1 || nq % nkv || !(hd == 128 || hd == 256)) return KS_OK;
  // one block per (query head, split): fewer splits than the caller's record layout allows if the grid is small
  unsigned n_splits = (unsigned)d->n_splits;
  if (n_splits > (unsigned)ctx->sm_count / nq) n_splits = (unsigned)ctx->sm_count / nq;
  if (n_splits > (unsigned)MG_MAX_SPLITS) n_splits = MG_MAX_SPLITS;
  if (n_splits < 1 || nq > 48) return KS_OK;
  if (d->n_layers < 1 || d->n_layers > 128) return KS_OK;

  const int stages = 3;
  const unsigned shapes_bytes = (unsigned)((PH_PER_LAYER * sizeof(MegaShape) + 15u) & ~15u);
  const unsigned tables_bytes = (unsigned)((shapes_bytes + d->n_layers * sizeof(MegaLayer) + 15u) & ~15u);
  unsigned maxcols = H > F ? H : F;
  if (qn > maxcols) maxcols = qn;
  unsigned x_bytes = (maxcols / 64u) * Q4K_XTOK * 4u;
  const unsigned att = mg_att_bytes(hd);
  if (att > x_bytes) x_bytes = att;
  const unsigned budget = (unsigned)ctx->smem_optin;
  const MegaSmem fixed = mg_smem(x_bytes, 0, stages, tables_bytes);
  if (fixed.total + 8u * stages * 4u * KS_Q4K_BLOCK_BYTES * 2u > budget) return KS_OK;
  unsigned slot_cap = (budget - fixed.total) / (8u * stages);
  slot_cap &= ~15u;
  if (slot_cap > 8192u) slot_cap = 8192u;
  // Blocks per column segment.  A block's items (its groups x column segments) are shared by its 8
  // warps, so more segments shorten the longest warp until the per-item overhead (measured: a little more
  // than one unit's worth of time) wins; segments hold an even number of blocks (8 lanes per row) and must fit a ring slot.
  const unsigned grid = (unsigned)ctx->sm_count;
  auto pick_seg = [&](unsigned cols, unsigned mats, unsigned total_groups, bool oct = false) {
    const unsigned nb = cols / 256u;
    const unsigned n_g = oct ? ((total_groups + 7) / 8 + grid - 1) / grid * 8 : (total_groups + grid - 1) / grid;
    unsigned best = 0;
    float best_cost = 0.f;
    for (unsigned C = 1; C <= nb; C++) {
      if (nb % C) continue;
      const unsigned sb = nb / C;
      if (sb % 2 || 4u * mats * sb * KS_Q4K_BLOCK_BYTES > slot_cap || n_g * C > (unsigned)MG_MAX_P) continue;
      const float cost = (float)((n_g * C + 7u) / 8u) * ((float)(sb * mats) * 0.5f + 1.2f);
      if (!best || cost < best_cost) {
        best = sb;
        best_cost = cost;
      }
    }
    return best;
  };
  const unsigned g_qkv = (qn + 3) / 4 + 2 * ((kvn + 3) / 4), g_h = (H + 3) / 4, g_f = (F + 3) / 4;
  if (g_qkv > 64u * grid || g_f > 64u * grid || g_h > 64u * grid) return KS_OK;  // a block finishes at most 64 groups per phase
  const unsigned sb_h = pick_seg(H, 1, g_qkv), sb_q = pick_seg(qn, 1, g_h), sb_f = pick_seg(F, 1, g_h);
  // gate-up: gate and up rows of a group in one item (x read once for both) when they fit a slot, else as two items
  unsigned sb_h2 = pick_seg(H, 2, g_f, true);
  bool gu_split = false;
  if (!sb_h2) {
    gu_split = true;
    const unsigned n_g = ((g_f + 7) / 8 + grid - 1) / grid * 8, nb = H / 256u;
    float best_cost = 0.f;
    for (unsigned C = 1; C <= nb; C++) {
      if (nb % C) continue;
      const unsigned sb = nb / C;
      if (sb % 2 || 4u * sb * KS_Q4K_BLOCK_BYTES > slot_cap || n_g * C > (unsigned)MG_MAX_P) continue;
      const float cost = (float)((n_g * C * 2u + 7u) / 8u) * ((float)sb * 0.5f + 1.2f);
      if (!sb_h2 || cost < best_cost) {
        sb_h2 = sb;
        best_cost = cost;
      }
    }
  }
  if (!sb_h || !sb_h2 || !sb_q || !sb_f) return KS_OK;
  unsigned slot_bytes = 0;
  auto upd = [&](unsigned sb, unsigned mats) {
    const unsigned b = 4u * mats * sb * KS_Q4K_BLOCK_BYTES;
    if (b > slot_bytes) slot_bytes = b;
  };
  upd(sb_h, 1); upd(sb_h2, gu_split ? 1 : 2); upd(sb_q, 1); upd(sb_f, 1);

  {  // every warp's items of one layer must fit its table
    auto per_warp = [&](unsigned total_groups, unsigned ncs) { return ((total_groups + grid - 1) / grid * ncs + 7u) / 8u; };
    const unsigned worst = per_warp(g_qkv, H / 256 / sb_h) + per_warp(g_h, qn / 256 / sb_q) +
                           (((g_f + 7) / 8 + grid - 1) / grid * 8 * (H / 256 / sb_h2) * (gu_split ? 2u : 1u) + 7u) / 8u +
                           per_warp(g_h, F / 256 / sb_f);
    if (worst > (unsigned)MG_MAX_ENT) return KS_OK;
  }
  std::vector<unsigned char> tab(tables_bytes, 0);
  MegaShape* sh = reinterpret_cast<MegaShape*>(tab.data());
  MegaLayer* ly = reinterpret_cast<MegaLayer*>(tab.data() + shapes_bytes);
  auto set_rows = [](MegaShape& p, unsigned cols, unsigned sb) {
    p.cols = cols;
    p.row_bytes = cols / 256u * KS_Q4K_BLOCK_BYTES;
    p.seg_blocks = sb;
    p.n_cseg = cols / 256u / sb;
    unsigned g0 = 0;
    for (int s = 0; s < p.n_seg; s++) {
      p.grp_start[s] = g0;
      g0 += (p.rows[s] + 3u) / 4u;
    }
    p.grp_start[p.n_seg] = g0;
  };
  sh[PH_QKV].type = MG_MATVEC; sh[PH_QKV].n_seg = 3;
  sh[PH_QKV].rows[0] = qn; sh[PH_QKV].rows[1] = kvn; sh[PH_QKV].rows[2] = kvn;
  set_rows(sh[PH_QKV], H, sb_h);
  sh[PH_ATTN].type = MG_ATTN; sh[PH_ATTN].n_seg = 1; sh[PH_ATTN].n_cseg = 1;
  sh[PH_OPROJ].type = MG_MATVEC; sh[PH_OPROJ].n_seg = 1; sh[PH_OPROJ].rows[0] = H;
  set_rows(sh[PH_OPROJ], qn, sb_q);
  sh[PH_GATEUP].type = MG_GATE_UP; sh[PH_GATEUP].n_seg = 1; sh[PH_GATEUP].rows[0] = F; sh[PH_GATEUP].oct = 1; sh[PH_GATEUP].split = gu_split ? 1 : 0;
  set_rows(sh[PH_GATEUP], H, sb_h2);
  sh[PH_DOWN].type = MG_MATVEC; sh[PH_DOWN].n_seg = 1; sh[PH_DOWN].rows[0] = H;
  set_rows(sh[PH_DOWN], F, sb_f);
  for (int l = 0; l < d->n_layers; l++) {
    const ks_mega_layer& L = layers[l];
    MegaLayer& o = ly[l];
    o.W[0] = (const uint8_t*)L.wq; o.W[1] = (const uint8_t*)L.wk; o.W[2] = (const uint8_t*)L.wv; o.W[3] = (const uint8_t*)L.wo;
    o.W[4] = (const uint8_t*)L.wgate; o.W[5] = (const uint8_t*)L.wup; o.W[6] = (const uint8_t*)L.wdown;
    o.norm[0] = (const float*)L.attn_norm; o.norm[1] = (const float*)L.q_norm; o.norm[2] = (const float*)L.k_norm;
    o.norm[3] = (const float*)L.post_attn_norm; o.norm[4] = (const float*)L.ffn_norm; o.norm[5] = (const float*)L.post_ffw_norm;
    o.kv_k = L.kv_k; o.kv_v = L.kv_v;
  }

  ks_mega* mg = new ks_mega();
  cudaSetDevice(ctx->device);
  const size_t n_phases = (size_t)d->n_layers * PH_PER_LAYER;
  if (cudaMalloc(&mg->d_tables, tables_bytes) != cudaSuccess || cudaMalloc((void**)&mg->d_sync, 512 + 16 * (size_t)ctx->sm_count) != cudaSuccess ||
      cudaMalloc((void**)&mg->d_prof, n_phases * 16 * sizeof(long long)) != cudaSuccess ||
      cudaMalloc((void**)&mg->d_fx, ((size_t)qn / 64 + (size_t)F / 64) * 256) != cudaSuccess ||
      cudaMalloc((void**)&mg->d_qkv, ((size_t)qn + 2 * (size_t)kvn) * sizeof(unsigned long long)) != cudaSuccess) {
    ks_mega_destroy(mg);
    return ks_fail(ctx, KS_ERR_OOM, "decode kernel: cannot allocate its tables");
  }
  cudaError_t e = cudaMemcpyAsync(mg->d_tables, tab.data(), tables_bytes, cudaMemcpyHostToDevice, ctx->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(mg->d_sync, 0, 512 + 16 * (size_t)ctx->sm_count, ctx->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(mg->d_fx, 0, ((size_t)qn / 64 + (size_t)F / 64) * 256, ctx->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(mg->d_prof, 0, n_phases * 16 * sizeof(long long), ctx->stream);
  mg->qkv_words = (size_t)qn + 2 * (size_t)kvn;
  if (e == cudaSuccess) e = cudaMemsetAsync(mg->d_qkv, 0, mg->qkv_words * sizeof(unsigned long long), ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);  // tab is a local
  if (e != cudaSuccess) {
    ks_mega_destroy(mg);
    return ks_fail(ctx, KS_ERR_CUDA, "decode kernel: table upload failed: %s", cudaGetErrorString(e));
  }
  MegaArgs& a = mg->args;
  a.tables = mg->d_tables;
  a.tables_bytes = tables_bytes;
  a.n_layers = d->n_layers;
  a.stages = stages;
  a.slot_bytes = slot_bytes;
  a.x_bytes = x_bytes;
  a.n_q = nq; a.n_kv = nkv; a.hd = hd; a.n_splits = n_splits;
  a.eps = d->eps; a.attn_scale = d->attn_scale;
  a.rope = d->rope; a.pos = d->pos;
  a.x_a = d->x_a; a.x_b = d->x_b;
  a.yb = d->yb; a.q = d->q; a.k = d->k; a.v = d->v;
  a.ox = mg->d_fx;
  a.ffx = mg->d_fx + (size_t)qn / 64 * 256;
  a.att_tmp = d->att_tmp;
  a.bar = mg->d_sync;
  a.qkv_t = mg->d_qkv;
  a.att_cnt = mg->d_sync + 64;
  a.nsum = reinterpret_cast<float4*>(mg->d_sync + 128);
  a.err = (unsigned*)ctx->ws + KS_WS_ERR_WORD;
  a.poll_limit = 1u << 21;
  a.test_stall = 0;
  a.prof = mg->d_prof;
  mg->grid = grid;
  mg->smem = mg_smem(x_bytes, slot_bytes, stages, tables_bytes).total;
  mg->G = (int)G;
  mg->dpl = (int)(hd / 32);
  mg->pc = H <= 2048 ? 2 : 4;
  mg->residual = d->x_b;
  *out = mg;
  return KS_OK;
}

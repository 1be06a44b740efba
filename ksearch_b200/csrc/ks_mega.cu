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
//   * the norms are applied while x is staged (same code path as the stand-alone fused matvec);
//   * attention: per-head RMS + RoPE + Q4_0 pack of the new K/V row, split-context online softmax
//     and the merge of the splits (last arriving block) happen inside one phase.
// Every spin (barrier, mbarrier) is bounded; on expiry the block raises the context's status word,
// drains its copies and leaves, and the other blocks time out the same way.
#include <vector>
#include <utility>

#include "ks_mv_common.cuh"

namespace {

enum { MG_MATVEC = 0, MG_GATE_UP = 1, MG_ATTN = 2 };

struct MegaPhase {
  int type;
  int n_seg;                // matvec: 1 or 3 (q, k, v)
  const uint8_t* W[3];
  float* y[3];
  unsigned rows[3];
  unsigned grp_start[4];    // first group of each segment, [n_seg] = total groups
  unsigned cols, row_bytes, seg_blocks, n_cseg;
  const float* x;           // input vector, or the residual stream for ADD_NORM
  ks_mv_pro pro;
  // attention only: this layer's KV cache (Q4_0 rows [max_seq, n_kv, hd]) and per-head norm weights
  uint8_t *kv_k, *kv_v;
  const float *q_norm, *k_norm;
};

struct MegaArgs {
  const MegaPhase* phases;
  int n_phases;
  int stages;               // ring slots per warp
  unsigned slot_bytes;      // bytes per ring slot
  unsigned x_bytes;         // staging area for x
  // attention
  unsigned n_q, n_kv, hd, n_splits;
  float eps, attn_scale;
  const float* rope;        // [max_seq, hd]
  const int* pos;           // [1]
  const float *q, *k, *v;   // outputs of the qkv phase
  float* o;                 // attention output [n_q * hd]
  float* att_tmp;           // [n_q * n_splits * (hd + 2)]
  unsigned* att_cnt;        // arrival counter of the attention blocks
  unsigned* bar;            // [0] running barrier counter, [1] its value when the previous token ended
  unsigned* err;
  long long* prof;          // [2][n_phases][4] SM clock stamps of the first and last block (start, staged, computed, released)
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

// Grid-wide barrier on a monotonically increasing counter.  Returns false when the wait gave up.
__device__ __forceinline__ bool grid_barrier(unsigned* counter, unsigned target, unsigned* err, int* sflag) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
    int ok = 0;
    for (unsigned i = 0; i < (1u << 21); i++) {  // a second or two of polling at most
      if ((int)(ld_acquire_u32(counter) - target) >= 0) {
        ok = 1;
        break;
      }
    }
    if (!ok) atomicOr(err, 2u);
    __threadfence();
    *sflag = ok;
  }
  __syncthreads();
  return *sflag != 0;
}

// ---- staging of x (with the fused norm prologues), reads through L2 ---------------------------
__device__ __forceinline__ void mg_stage_x(unsigned char* xs, float* red, const MegaPhase& ph) {
  const unsigned cols = ph.cols, units = cols >> 6, nchunk = cols >> 2;
  float* xp = reinterpret_cast<float*>(xs);
  float* sx = xp + (size_t)units * Q4K_XS;
  if (ph.pro.mode == KS_PRO_NONE) {
#pragma unroll 4
    for (unsigned c = threadIdx.x; c < nchunk; c += blockDim.x) q4k_put_chunk(xp, sx, c, ldcg4(ph.x, c));
    return;
  }
  const float invn = 1.0f / (float)cols;
  float4 v[KS_PRO_MAXC], yv[KS_PRO_MAXC];
  float ss = 0.0f;
  const float* w = reinterpret_cast<const float*>(ph.pro.w);
  if (ph.pro.mode == KS_PRO_ADD_NORM) {
    const float* y = reinterpret_cast<const float*>(ph.pro.y);
    const float* wp = reinterpret_cast<const float*>(ph.pro.w_post);
#pragma unroll
    for (int k = 0; k < KS_PRO_MAXC; k++) {
      const unsigned c = threadIdx.x + k * blockDim.x;
      if (c < nchunk) {
        yv[k] = ldcg4(y, c);
        v[k] = ldcg4(ph.x, c);
        ss = fmaf(yv[k].x, yv[k].x, ss); ss = fmaf(yv[k].y, yv[k].y, ss);
        ss = fmaf(yv[k].z, yv[k].z, ss); ss = fmaf(yv[k].w, yv[k].w, ss);
      }
    }
    ss = block_sum_f(ss, red);
    const float inv = 1.0f / sqrtf(ss * invn + ph.pro.eps);
    ss = 0.0f;
#pragma unroll
    for (int k = 0; k < KS_PRO_MAXC; k++) {
      const unsigned c = threadIdx.x + k * blockDim.x;
      if (c < nchunk) {
        const float4 p4 = reinterpret_cast<const float4*>(wp)[c];
        float4 r = v[k];
        r.x = __fadd_rn(r.x, __fmul_rn(__fmul_rn(yv[k].x, inv), p4.x));
        r.y = __fadd_rn(r.y, __fmul_rn(__fmul_rn(yv[k].y, inv), p4.y));
        r.z = __fadd_rn(r.z, __fmul_rn(__fmul_rn(yv[k].z, inv), p4.z));
        r.w = __fadd_rn(r.w, __fmul_rn(__fmul_rn(yv[k].w, inv), p4.w));
        if (blockIdx.x == 0) reinterpret_cast<float4*>(ph.pro.out_x)[c] = r;
        v[k] = r;
      }
    }
  } else {
#pragma unroll
    for (int k = 0; k < KS_PRO_MAXC; k++) {
      const unsigned c = threadIdx.x + k * blockDim.x;
      if (c < nchunk) v[k] = ldcg4(ph.x, c);
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
  const float inv2 = 1.0f / sqrtf(ss * invn + ph.pro.eps);
#pragma unroll
  for (int k = 0; k < KS_PRO_MAXC; k++) {
    const unsigned c = threadIdx.x + k * blockDim.x;
    if (c < nchunk) {
      const float4 w4 = reinterpret_cast<const float4*>(w)[c];
      float4 r;
      r.x = __fmul_rn(__fmul_rn(v[k].x, inv2), w4.x);
      r.y = __fmul_rn(__fmul_rn(v[k].y, inv2), w4.y);
      r.z = __fmul_rn(__fmul_rn(v[k].z, inv2), w4.z);
      r.w = __fmul_rn(__fmul_rn(v[k].w, inv2), w4.w);
      q4k_put_chunk(xp, sx, c, r);
    }
  }
}

// ---- the per-warp item list of a whole token -----------------------------------------------------
// Item = (phase, row group, column segment).  Warp gw owns groups gw, gw+GW, ... of every matvec
// phase.  Two cursors walk the same list: one issues copies, one consumes them.
struct Cursor {
  int p;
  unsigned g, cs;
};
__device__ __forceinline__ void cur_settle(Cursor& c, const MegaArgs& a, unsigned gw) {
  while (c.p < a.n_phases) {
    const MegaPhase& ph = a.phases[c.p];
    const unsigned total = ph.type == MG_ATTN ? 0u : ph.grp_start[ph.n_seg];
    if (c.g < total) return;
    c.p++;
    c.g = gw;
    c.cs = 0;
  }
}
__device__ __forceinline__ void cur_next(Cursor& c, const MegaArgs& a, unsigned gw, unsigned GW) {
  const MegaPhase& ph = a.phases[c.p];
  if (++c.cs >= ph.n_cseg) {
    c.cs = 0;
    c.g += GW;
  }
  cur_settle(c, a, gw);
}

constexpr int MG_RL = 4, MG_LPR = 8;  // 8 lanes per row, 4 rows side by side

// Start the copies of the item under the cursor into ring slot `slot` (all lanes call).
__device__ __forceinline__ void mg_issue(const MegaArgs& a, const Cursor& c, uint32_t slot_addr, uint32_t bar, int lane) {
  const MegaPhase& ph = a.phases[c.p];
  int seg = 0;
  if (ph.n_seg > 1 && c.g >= ph.grp_start[1]) seg = 1;
  if (ph.n_seg > 2 && c.g >= ph.grp_start[2]) seg = 2;
  const unsigned seg_rows = seg == 0 ? ph.rows[0] : seg == 1 ? ph.rows[1] : ph.rows[2];
  const unsigned g0 = seg == 0 ? ph.grp_start[0] : seg == 1 ? ph.grp_start[1] : ph.grp_start[2];
  const unsigned row0 = (c.g - g0) * MG_RL;
  const unsigned valid = min((unsigned)MG_RL, seg_rows - row0);
  const unsigned seg_bytes = ph.seg_blocks * KS_Q4K_BLOCK_BYTES;
  const int mats = ph.type == MG_GATE_UP ? 2 : 1;
  if (lane == 0) mb_expect(bar, valid * mats * seg_bytes);
  if (ph.n_cseg == 1) {
    if (lane < mats) {
      const uint8_t* base = ph.type == MG_GATE_UP ? (lane ? ph.W[1] : ph.W[0]) : (seg == 0 ? ph.W[0] : seg == 1 ? ph.W[1] : ph.W[2]);
      bulk_in(slot_addr + (uint32_t)lane * MG_RL * seg_bytes, base + (size_t)row0 * ph.row_bytes, valid * seg_bytes, bar);
    }
  } else if (lane < MG_RL * mats) {
    const int m = lane / MG_RL, rr = lane % MG_RL;
    if ((unsigned)rr < valid) {
      const uint8_t* base = ph.type == MG_GATE_UP ? (m ? ph.W[1] : ph.W[0]) : (seg == 0 ? ph.W[0] : seg == 1 ? ph.W[1] : ph.W[2]);
      bulk_in(slot_addr + (uint32_t)lane * seg_bytes, base + (size_t)(row0 + rr) * ph.row_bytes + (size_t)c.cs * seg_bytes,
              seg_bytes, bar);
    }
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

// Shared memory the attention phase needs (it reuses the x staging area).
__host__ __device__ inline unsigned mg_att_bytes(unsigned G, unsigned hd) {
  const unsigned area = 4u * G * (hd + 2u) > 8u * hd ? 4u * G * (hd + 2u) : 8u * hd;
  return (G * hd + area) * 4u + 2u * ((hd / 32u) * KS_Q40_BLOCK_BYTES + 16u) + 32u;
}

template <int G, int DPL>
__device__ __forceinline__ void mg_attention(const MegaArgs& a, const MegaPhase& ph, unsigned char* sm, int* sflag) {
  constexpr int HD = DPL * 32, HALF = HD / 2;
  constexpr unsigned ROWB = (HD / 32) * KS_Q40_BLOCK_BYTES;
  constexpr unsigned AREA = (4u * G * (HD + 2u) > 8u * HD) ? 4u * G * (HD + 2u) : 8u * HD;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned NS = a.n_splits, n_att = a.n_kv * NS;
  if (blockIdx.x >= n_att) return;
  const unsigned kvh = blockIdx.x / NS, split = blockIdx.x % NS;
  const unsigned pos = (unsigned)a.pos[0], tlen = pos + 1;
  const unsigned chunk = (tlen + NS - 1) / NS;
  const unsigned p0 = split * chunk, p1 = min(p0 + chunk, tlen);
  float* sq = reinterpret_cast<float*>(sm);       // [G][HD] roped, scaled q
  float* area = sq + G * HD;                      // warp scratch, then the merge tree
  uint8_t* skrow = reinterpret_cast<uint8_t*>(area + AREA);
  uint8_t* svrow = skrow + ROWB + 16u;
  const float* cs = a.rope + (size_t)pos * HD;

  // per-head RMS + RoPE of q, and the new K / V row (lower.rs:4231-4702), one warp per job
  for (int t = warp; t < G + 2; t += 8) {
    const int kind = t < G ? 0 : t == G ? 1 : 2;
    const float* src = kind == 0 ? a.q + ((size_t)kvh * G + t) * HD : kind == 1 ? a.k + (size_t)kvh * HD : a.v + (size_t)kvh * HD;
    const float* w = kind == 0 ? ph.q_norm : ph.k_norm;
    float xv[DPL];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < DPL; j++) {
      xv[j] = __ldcg(src + lane + 32 * j);
      ss = fmaf(xv[j], xv[j], ss);
    }
    ss = mg_warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)HD + a.eps);
    float* tmp = area + warp * HD;
    if (kind == 2) {
#pragma unroll
      for (int j = 0; j < DPL; j++) tmp[lane + 32 * j] = __fmul_rn(xv[j], inv);
    } else {
#pragma unroll
      for (int j = 0; j < DPL / 2; j++) {
        const int i = lane + 32 * j;
        const float u = __fmul_rn(__fmul_rn(xv[j], inv), w[i]);
        const float vv = __fmul_rn(__fmul_rn(xv[j + DPL / 2], inv), w[HALF + i]);
        const float c = cs[i], s = cs[HALF + i];
        const float lo = __fsub_rn(__fmul_rn(u, c), __fmul_rn(vv, s));
        const float hi = __fadd_rn(__fmul_rn(u, s), __fmul_rn(vv, c));
        if (kind == 0) {
          sq[t * HD + i] = lo * a.attn_scale;
          sq[t * HD + HALF + i] = hi * a.attn_scale;
        } else {
          tmp[i] = lo;
          tmp[HALF + i] = hi;
        }
      }
    }
    if (kind != 0) {
      __syncwarp();
      uint8_t* dst = kind == 1 ? skrow : svrow;
#pragma unroll
      for (int b = 0; b < HD / 32; b++) {
        const float val = __half2float(__float2half_rn(tmp[b * 32 + lane]));  // through f16 (render.rs:1046)
        mg_pack_q40(val, dst + b * KS_Q40_BLOCK_BYTES, lane);
      }
    }
  }
  __syncthreads();
  const size_t rowstride = (size_t)a.n_kv * ROWB;
  uint8_t* Kc = ph.kv_k + (size_t)kvh * ROWB;
  uint8_t* Vc = ph.kv_v + (size_t)kvh * ROWB;
  if (pos >= p0 && pos < p1) {  // the split that holds the newest position stores the new row
    const unsigned n16 = ROWB / 2;
    if (threadIdx.x < n16)
      reinterpret_cast<unsigned short*>(Kc + (size_t)pos * rowstride)[threadIdx.x] = reinterpret_cast<const unsigned short*>(skrow)[threadIdx.x];
    else if (threadIdx.x < 2 * n16)
      reinterpret_cast<unsigned short*>(Vc + (size_t)pos * rowstride)[threadIdx.x - n16] =
          reinterpret_cast<const unsigned short*>(svrow)[threadIdx.x - n16];
  }

  float qr[G][DPL], o[G][DPL], m[G], l[G];
#pragma unroll
  for (int g = 0; g < G; g++) {
#pragma unroll
    for (int j = 0; j < DPL; j++) {
      qr[g][j] = sq[g * HD + mg_lane_dim<DPL>(lane, j)];
      o[g][j] = 0.0f;
    }
    m[g] = kNegInit;
    l[g] = 0.0f;
  }
  auto fetch = [&](unsigned t, RawRow<DPL>& kr, RawRow<DPL>& vr) {
    if (t < p1) {
      const uint8_t* kp = t == pos ? skrow : Kc + (size_t)t * rowstride;
      const uint8_t* vp = t == pos ? svrow : Vc + (size_t)t * rowstride;
      raw_load<DPL>(kp, lane, kr);
      raw_load<DPL>(vp, lane, vr);
    }
  };
  auto process = [&](const RawRow<DPL>& kr, const RawRow<DPL>& vr) {
    float kv[DPL];
    raw_decode<DPL>(kr, kv);
    float s[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
      float acc = 0.0f;
#pragma unroll
      for (int j = 0; j < DPL; j++) acc = fmaf(qr[g][j], kv[j], acc);
      s[g] = acc;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
#pragma unroll
      for (int g = 0; g < G; g++) s[g] += __shfl_xor_sync(0xffffffffu, s[g], off);
    raw_decode<DPL>(vr, kv);
#pragma unroll
    for (int g = 0; g < G; g++) {
      const float m2 = fmaxf(m[g], s[g]);
      const float alpha = __expf(m[g] - m2);
      const float e = __expf(s[g] - m2);
      l[g] = l[g] * alpha + e;
      m[g] = m2;
#pragma unroll
      for (int j = 0; j < DPL; j++) o[g][j] = fmaf(e, kv[j], o[g][j] * alpha);
    }
  };
  {
    RawRow<DPL> kA, vA, kB, vB;
    unsigned t = p0 + warp;
    fetch(t, kA, vA);
    fetch(t + 8, kB, vB);
    while (t < p1) {
      const RawRow<DPL> k0 = kA, v0 = vA, k1 = kB, v1 = vB;
      fetch(t + 16, kA, vA);
      fetch(t + 24, kB, vB);
      process(k0, v0);
      if (t + 8 < p1) process(k1, v1);
      t += 16;
    }
  }
  __syncthreads();  // every warp is done with sq / its scratch: the area becomes the merge tree
  // fold the 8 warps pairwise: (4..7 -> 0..3), (2,3 -> 0,1), (1 -> 0)
#pragma unroll 1
  for (int half = 4; half >= 1; half >>= 1) {
    if (warp >= half && warp < 2 * half) {
      float* dst = area + (size_t)(warp - half) * G * (HD + 2);
#pragma unroll
      for (int g = 0; g < G; g++) {
        if (lane == 0) {
          dst[g * (HD + 2)] = m[g];
          dst[g * (HD + 2) + 1] = l[g];
        }
#pragma unroll
        for (int j = 0; j < DPL; j++) dst[g * (HD + 2) + 2 + j * 32 + lane] = o[g][j];
      }
    }
    __syncthreads();
    if (warp < half) {
      const float* srcm = area + (size_t)warp * G * (HD + 2);
#pragma unroll
      for (int g = 0; g < G; g++) {
        const float mp = srcm[g * (HD + 2)], lp = srcm[g * (HD + 2) + 1];
        const float m2 = fmaxf(m[g], mp);
        const float alpha = __expf(m[g] - m2), beta = __expf(mp - m2);
        l[g] = l[g] * alpha + lp * beta;
        m[g] = m2;
#pragma unroll
        for (int j = 0; j < DPL; j++) o[g][j] = o[g][j] * alpha + srcm[g * (HD + 2) + 2 + j * 32 + lane] * beta;
      }
    }
    __syncthreads();
  }
  if (warp == 0) {
#pragma unroll
    for (int g = 0; g < G; g++) {
      const unsigned head = kvh * G + g;
      float* rec = a.att_tmp + ((size_t)head * NS + split) * (HD + 2);
      if (lane == 0) {
        rec[0] = m[g];
        rec[1] = l[g];
      }
#pragma unroll
      for (int j = 0; j < DPL; j++) rec[2 + mg_lane_dim<DPL>(lane, j)] = o[g][j];
    }
    __threadfence();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned old = atomicAdd(a.att_cnt, 1u);
    *sflag = (old == n_att - 1) ? 1 : 0;
  }
  __syncthreads();
  if (*sflag) {
    // last block to arrive: merge the splits of every head (lower.rs:5897-6088)
    __threadfence();
    const unsigned total = a.n_q * HD;
    for (unsigned idx = threadIdx.x; idx < total; idx += blockDim.x) {
      const unsigned head = idx / HD, d = idx % HD;
      const float* rec0 = a.att_tmp + (size_t)head * NS * (HD + 2);
      float mm = kNegInit, ll = 0.0f, oo = 0.0f;
      for (unsigned p = 0; p < NS; p++) {
        const float* rec = rec0 + (size_t)p * (HD + 2);
        const float mp = __ldcg(rec), lp = __ldcg(rec + 1);
        const float m2 = fmaxf(mm, mp);
        const float alpha = __expf(mm - m2), beta = __expf(mp - m2);
        ll = ll * alpha + lp * beta;
        mm = m2;
        oo = oo * alpha + __ldcg(rec + 2 + d) * beta;
      }
      a.o[idx] = oo * (1.0f / ll);
    }
    if (threadIdx.x == 0) *a.att_cnt = 0u;
  }
}

// ---- the kernel -------------------------------------------------------------------------------------
struct MegaSmem {
  unsigned ring_off, bar_off, red_off, flag_off, total;
};
__host__ __device__ inline MegaSmem mg_smem(unsigned x_bytes, unsigned slot_bytes, int stages) {
  MegaSmem L;
  L.ring_off = (x_bytes + 127u) & ~127u;
  L.bar_off = L.ring_off + 8u * (unsigned)stages * slot_bytes;
  L.red_off = (L.bar_off + 8u * 8u * (unsigned)stages + 15u) & ~15u;
  L.flag_off = L.red_off + 128u;
  L.total = L.flag_off + 16u;
  return L;
}

template <int G, int DPL>
__global__ void __launch_bounds__(256, 1) mega_kernel(const MegaArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cl = lane % MG_LPR, rl = lane / MG_LPR;
  const int S = a.stages;
  const MegaSmem L = mg_smem(a.x_bytes, a.slot_bytes, S);
  const uint32_t ring_s = sm32(smem + L.ring_off) + (uint32_t)(warp * S) * a.slot_bytes;
  const uint32_t bars = sm32(smem + L.bar_off) + (uint32_t)(warp * S) * 8u;
  float* red = reinterpret_cast<float*>(smem + L.red_off);
  int* sflag = reinterpret_cast<int*>(smem + L.flag_off);
  const uint32_t xs_s = sm32(smem);
  // consecutive groups go to different blocks, so a phase with few groups still uses every SM
  const unsigned gw = (unsigned)warp * gridDim.x + blockIdx.x, GW = gridDim.x * 8u;
  const unsigned bar_base = a.bar[1];

  if (lane == 0) {
    for (int s = 0; s < S; s++) mb_init(bars + s * 8u, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  Cursor ic{0, gw, 0}, cc{0, gw, 0};
  cur_settle(ic, a, gw);
  cur_settle(cc, a, gw);
  unsigned issued = 0, consumed = 0;
  while (issued < (unsigned)S && ic.p < a.n_phases) {
    mg_issue(a, ic, ring_s + issued * a.slot_bytes, bars + issued * 8u, lane);
    issued++;
    cur_next(ic, a, gw, GW);
  }

  long long* prof = nullptr;
  if (threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1))
    prof = a.prof + (size_t)(blockIdx.x == 0 ? 0 : 1) * a.n_phases * 4;
  bool dead = false;  // this warp gave up on a copy: it keeps the block-level steps, skips its items
  int p = 0;
  for (; p < a.n_phases; p++) {
    const MegaPhase& ph = a.phases[p];
    if (prof) prof[p * 4 + 0] = clock64();
    if (ph.type == MG_ATTN) {
      mg_attention<G, DPL>(a, ph, smem, sflag);
    } else {
      mg_stage_x(smem, red, ph);
      __syncthreads();
      if (prof) prof[p * 4 + 1] = clock64();
      const unsigned units = ph.cols >> 6;
      float yacc[2] = {0.0f, 0.0f};
      while (cc.p == p && !dead) {
        const unsigned st = consumed % (unsigned)S;
        if (!mb_wait(bars + st * 8u, (consumed / (unsigned)S) & 1u)) {
          dead = true;
          if (lane == 0) atomicOr(a.err, 1u);
          break;
        }
        const uint32_t slot = ring_s + st * a.slot_bytes;
        if (ph.type == MG_GATE_UP)
          mg_item_compute<2>(slot, xs_s, units, ph.seg_blocks, cc.cs, cl, rl, yacc);
        else
          mg_item_compute<1>(slot, xs_s, units, ph.seg_blocks, cc.cs, cl, rl, yacc);
        __syncwarp();
        consumed++;
        const unsigned g = cc.g, cs = cc.cs;
        cur_next(cc, a, gw, GW);
        if (ic.p < a.n_phases) {
          if (lane == 0) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the slot was read through the generic proxy
          __syncwarp();
          mg_issue(a, ic, slot, bars + st * 8u, lane);
          issued++;
          cur_next(ic, a, gw, GW);
        }
        if (cs + 1 == ph.n_cseg) {
          int seg = 0;
          if (ph.n_seg > 1 && g >= ph.grp_start[1]) seg = 1;
          if (ph.n_seg > 2 && g >= ph.grp_start[2]) seg = 2;
          const unsigned seg_rows = seg == 0 ? ph.rows[0] : seg == 1 ? ph.rows[1] : ph.rows[2];
          const unsigned g0 = seg == 0 ? ph.grp_start[0] : seg == 1 ? ph.grp_start[1] : ph.grp_start[2];
          const unsigned row = (g - g0) * MG_RL + (unsigned)rl;
          float v0 = yacc[0], v1 = yacc[1];
#pragma unroll
          for (int o = MG_LPR / 2; o > 0; o >>= 1) {
            v0 += __shfl_xor_sync(0xffffffffu, v0, o);
            v1 += __shfl_xor_sync(0xffffffffu, v1, o);
          }
          if (cl == 0 && row < seg_rows) {
            float* y = seg == 0 ? ph.y[0] : seg == 1 ? ph.y[1] : ph.y[2];
            y[row] = ph.type == MG_GATE_UP ? gelu_mul(v0, v1) : v0;
          }
          yacc[0] = yacc[1] = 0.0f;
        }
      }
    }
    if (prof) prof[p * 4 + 2] = clock64();
    if (!grid_barrier(a.bar, bar_base + (unsigned)(p + 1) * gridDim.x, a.err, sflag)) break;
    if (prof) prof[p * 4 + 3] = clock64();
  }
  if (p == a.n_phases) {
    if (blockIdx.x == 0 && threadIdx.x == 0) a.bar[1] = bar_base + (unsigned)a.n_phases * gridDim.x;
  }
  // copies still in flight must land before this block's shared memory goes away (bounded)
  for (unsigned j = consumed; j < issued; j++) mb_wait(bars + (j % (unsigned)S) * 8u, (j / (unsigned)S) & 1u);
}

}  // namespace

// ---- host side --------------------------------------------------------------------------------------
struct ks_mega {
  MegaArgs args{};
  MegaPhase* d_phases = nullptr;
  unsigned* d_sync = nullptr;  // [0..1] barrier words, [2] attention arrival counter
  long long* d_prof = nullptr;
  unsigned grid = 0;
  size_t smem = 0;
  int G = 0, dpl = 0;
  float* residual = nullptr;  // buffer that holds the residual stream when the kernel ends
};

namespace {
template <int G, int DPL>
int mega_launch_t(ks_ctx* ctx, ks_mega* mg) {
  auto kern = mega_kernel<G, DPL>;
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
#define KS_MG(G_, D_) \
  if (mg->G == G_ && mg->dpl == D_) return mega_launch_t<G_, D_>(ctx, mg)
  KS_MG(1, 4); KS_MG(2, 4); KS_MG(4, 4); KS_MG(8, 4);
  KS_MG(1, 8); KS_MG(2, 8); KS_MG(4, 8); KS_MG(8, 8);
#undef KS_MG
  return ks_fail(ctx, KS_ERR_UNSUPPORTED, "decode kernel: head grouping not supported");
}

float* ks_mega_residual(const ks_mega* mg) { return mg->residual; }
const long long* ks_mega_prof(const ks_mega* mg) { return mg->d_prof; }

void ks_mega_destroy(ks_mega* mg) {
  if (!mg) return;
  if (mg->d_phases) cudaFree(mg->d_phases);
  if (mg->d_sync) cudaFree(mg->d_sync);
  if (mg->d_prof) cudaFree(mg->d_prof);
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
  if (!(G == 1 || G == 2 || G == 4 || G == 8) || !(hd == 128 || hd == 256)) return KS_OK;
  if (d->n_splits < 1 || nkv * (unsigned)d->n_splits > (unsigned)ctx->sm_count) return KS_OK;

  const int stages = 3;
  unsigned maxcols = H > F ? H : F;
  if (qn > maxcols) maxcols = qn;
  unsigned x_bytes = (maxcols / 64u) * Q4K_XTOK * 4u;
  const unsigned att = mg_att_bytes(G, hd);
  if (att > x_bytes) x_bytes = att;
  const unsigned budget = (unsigned)ctx->smem_optin;
  const MegaSmem fixed = mg_smem(x_bytes, 0, stages);
  if (fixed.total + 8u * stages * 4u * KS_Q4K_BLOCK_BYTES * 2u > budget) return KS_OK;
  unsigned slot_cap = (budget - fixed.total) / (8u * stages);
  slot_cap &= ~15u;
  if (slot_cap > 8192u) slot_cap = 8192u;
  // blocks per column segment: the largest even divisor of the row's block count that fits a slot
  auto pick_seg = [&](unsigned cols, unsigned mats) {
    const unsigned nb = cols / 256u;
    unsigned best = 0;
    for (unsigned c = 2; c <= nb; c += 2)
      if (nb % c == 0 && 4u * mats * c * KS_Q4K_BLOCK_BYTES <= slot_cap) best = c;
    return best;
  };
  const unsigned sb_h = pick_seg(H, 1), sb_h2 = pick_seg(H, 2), sb_q = pick_seg(qn, 1), sb_f = pick_seg(F, 1);
  if (!sb_h || !sb_h2 || !sb_q || !sb_f) return KS_OK;
  unsigned slot_bytes = 0;
  auto upd = [&](unsigned sb, unsigned mats) {
    const unsigned b = 4u * mats * sb * KS_Q4K_BLOCK_BYTES;
    if (b > slot_bytes) slot_bytes = b;
  };
  upd(sb_h, 1); upd(sb_h2, 2); upd(sb_q, 1); upd(sb_f, 1);

  std::vector<MegaPhase> ph;
  float* cur = d->x_a;
  float* oth = d->x_b;
  auto set_rows = [](MegaPhase& p, unsigned cols, unsigned sb) {
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
  for (int l = 0; l < d->n_layers; l++) {
    const ks_mega_layer& L = layers[l];
    MegaPhase a{};
    a.type = MG_MATVEC;
    a.n_seg = 3;
    a.W[0] = (const uint8_t*)L.wq; a.W[1] = (const uint8_t*)L.wk; a.W[2] = (const uint8_t*)L.wv;
    a.y[0] = d->q; a.y[1] = d->k; a.y[2] = d->v;
    a.rows[0] = qn; a.rows[1] = kvn; a.rows[2] = kvn;
    set_rows(a, H, sb_h);
    a.x = cur;
    a.pro.eps = d->eps;
    a.pro.w = L.attn_norm;
    if (l == 0) {
      a.pro.mode = KS_PRO_NORM;
    } else {
      a.pro.mode = KS_PRO_ADD_NORM;
      a.pro.y = d->yb;
      a.pro.w_post = layers[l - 1].post_ffw_norm;
      a.pro.out_x = oth;
    }
    ph.push_back(a);
    if (l > 0) std::swap(cur, oth);

    MegaPhase t{};
    t.type = MG_ATTN;
    t.kv_k = L.kv_k; t.kv_v = L.kv_v;
    t.q_norm = (const float*)L.q_norm; t.k_norm = (const float*)L.k_norm;
    ph.push_back(t);

    MegaPhase o{};
    o.type = MG_MATVEC;
    o.n_seg = 1;
    o.W[0] = (const uint8_t*)L.wo;
    o.y[0] = d->yb;
    o.rows[0] = H;
    set_rows(o, qn, sb_q);
    o.x = d->o;
    ph.push_back(o);

    MegaPhase gu{};
    gu.type = MG_GATE_UP;
    gu.n_seg = 1;
    gu.W[0] = (const uint8_t*)L.wgate; gu.W[1] = (const uint8_t*)L.wup;
    gu.y[0] = d->ff;
    gu.rows[0] = F;
    set_rows(gu, H, sb_h2);
    gu.x = cur;
    gu.pro.mode = KS_PRO_ADD_NORM;
    gu.pro.eps = d->eps;
    gu.pro.w = L.ffn_norm;
    gu.pro.y = d->yb;
    gu.pro.w_post = L.post_attn_norm;
    gu.pro.out_x = oth;
    ph.push_back(gu);
    std::swap(cur, oth);

    MegaPhase dn{};
    dn.type = MG_MATVEC;
    dn.n_seg = 1;
    dn.W[0] = (const uint8_t*)L.wdown;
    dn.y[0] = d->yb;
    dn.rows[0] = H;
    set_rows(dn, F, sb_f);
    dn.x = d->ff;
    ph.push_back(dn);
  }

  ks_mega* mg = new ks_mega();
  cudaSetDevice(ctx->device);
  if (cudaMalloc((void**)&mg->d_phases, ph.size() * sizeof(MegaPhase)) != cudaSuccess ||
      cudaMalloc((void**)&mg->d_sync, 64) != cudaSuccess ||
      cudaMalloc((void**)&mg->d_prof, ph.size() * 8 * sizeof(long long)) != cudaSuccess) {
    ks_mega_destroy(mg);
    return ks_fail(ctx, KS_ERR_OOM, "decode kernel: cannot allocate the phase table");
  }
  cudaError_t e = cudaMemcpyAsync(mg->d_phases, ph.data(), ph.size() * sizeof(MegaPhase), cudaMemcpyHostToDevice, ctx->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(mg->d_sync, 0, 64, ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);  // ph is a local
  if (e != cudaSuccess) {
    ks_mega_destroy(mg);
    return ks_fail(ctx, KS_ERR_CUDA, "decode kernel: phase table upload failed: %s", cudaGetErrorString(e));
  }
  MegaArgs& a = mg->args;
  a.phases = mg->d_phases;
  a.n_phases = (int)ph.size();
  a.stages = stages;
  a.slot_bytes = slot_bytes;
  a.x_bytes = x_bytes;
  a.n_q = nq; a.n_kv = nkv; a.hd = hd; a.n_splits = (unsigned)d->n_splits;
  a.eps = d->eps; a.attn_scale = d->attn_scale;
  a.rope = d->rope; a.pos = d->pos;
  a.q = d->q; a.k = d->k; a.v = d->v; a.o = d->o;
  a.att_tmp = d->att_tmp;
  a.bar = mg->d_sync;
  a.att_cnt = mg->d_sync + 2;
  a.err = (unsigned*)ctx->ws + KS_WS_ERR_WORD;
  a.prof = mg->d_prof;
  mg->grid = (unsigned)ctx->sm_count;
  mg->smem = mg_smem(x_bytes, slot_bytes, stages).total;
  mg->G = (int)G;
  mg->dpl = (int)(hd / 32);
  mg->residual = cur;
  *out = mg;
  return KS_OK;
}

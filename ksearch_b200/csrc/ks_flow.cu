// One persistent kernel for all layers of a decode token (single slot, f32 activations).
//
// The op order is forward_token's (crates/ksearch_gemma/src/gemma_prim.rs:923-1197) for dense,
// KV-owning layers; what changes is WHERE the boundaries between ops are and HOW a result reaches
// its consumers.  A token is a chain of ~175 dependent steps of a few hundred kilobytes to ten
// megabytes of weights each; neither a kernel boundary nor a grid-wide barrier is affordable
// between them.  One block per SM (8 warps) stays resident for the whole token:
//   * Dataflow instead of barriers.  Every activation that crosses blocks (q/k/v, attention
//     output, o-proj output, GeGLU output, down-proj output, attention split records) is written
//     as a 64-bit word (f32 value, 32-bit tag) with one relaxed store, tag = token epoch + layer.
//     A consumer polls the words it needs until their tags match.  Value and tag travel in one
//     single-copy-atomic word, so no fence, no flag and no second round trip is needed: a hop
//     between phases costs one store and one load through L2.  Buffers alternate by layer parity.
//   * Rows are split evenly: block b owns the contiguous rows [b*R/grid, (b+1)*R/grid) (in pairs)
//     of every matvec phase, so its weights are ONE contiguous byte range per matrix and phase.
//   * The weight stream never stops: those ranges are cut into pieces that fit a slot of a
//     block-wide shared-memory ring fed by cp.async.bulk (mbarrier completion).  The pieces of all
//     phases and layers form one sequence; when the block is done with a slot, a lane of its last warp
//     refills it with the piece n_slots further down the sequence, so the next phases' (and layer's)
//     weights arrive while the block computes or waits for its inputs.
//   * Inside a phase a task is one row x one 32-unit column segment (a lane owns one 64-weight unit
//     and keeps that unit of x in registers); each warp takes one contiguous run of the block's tasks,
//     two rows interleaved; row sums meet in shared memory, thread f finishes row f.
//   * x is staged once per phase and block as 24-bit block fixed point (three byte planes per
//     32-element sub-block) so weight nibbles x x are exact dp4a integer sums.
//   * The residual stream never leaves the block: every block applies the same residual-add + norm
//     to the same inputs in the same order, so each thread keeps its elements in registers.
//   * Attention: one block per (query head, context split); short contexts use one split (no
//     merge hop), long ones merge the split records in the head's first block.
// Every wait (tag poll, mbarrier) is bounded; on expiry the block raises the context's status
// word and carries on without waiting any more, so the kernel always ends; blocks that see the
// status word raised stop waiting too.
#include <cstdlib>
#include <cstring>
#include <utility>
#include <vector>

#include "ks_fx.cuh"

namespace {

enum { PH_QKV = 0, PH_OPROJ = 1, PH_GATEUP = 2, PH_DOWN = 3, PH_KINDS = 4 };
enum { PF_QKV = 0, PF_ATTN = 1, PF_OPROJ = 2, PF_GATEUP = 3, PF_DOWN = 4, PF_PER_LAYER = 5, PF_STAMPS = 8 };

#ifndef MG_NW_CFG
#define MG_NW_CFG 8
#endif
#ifndef MG_FN
#define MG_FN __forceinline__
#endif
constexpr int MG_NW = MG_NW_CFG, MG_THREADS = MG_NW * 32;  // warps per block (at least 8)
constexpr int MG_MAXPIECE = 64;   // pieces of one layer owned by one block
constexpr int MG_MAXROWS = 96;    // rows of one phase owned by one block
constexpr int MG_MAXC = 8;        // column segments per row
constexpr int MG_MAXSLOTS = 16;   // ring slots
constexpr int MG_MAX_SPLITS = 16; // context splits per head

struct MegaPhase {          // one matvec phase of a layer; the same for every layer
  unsigned n_seg;           // matrices laid end to end in the phase's row space (qkv: 3, else 1)
  unsigned mats;            // matrices multiplied per row (gate-up: 2, gate row i and up row i)
  unsigned seg_start[4];    // first row of each matrix in the row space; [n_seg] = total rows
  unsigned widx;            // MegaLayer::W index of the first matrix
  unsigned cols, row_bytes, seg_units, n_cseg, piece_rows;  // n_cseg column segments of seg_units (<= 32) 64-weight units
};

struct MegaLayer {          // per-layer pointers, copied to shared memory when the kernel starts
  const uint8_t* W[7];      // wq, wk, wv, wo, wgate, wup, wdown (Q4_K)
  const float* norm[6];     // attn_norm, q_norm, k_norm, post_attn_norm, ffn_norm, post_ffw_norm
  uint8_t *kv_k, *kv_v;     // this slot's cache rows [max_seq, n_kv, hd] Q4_0
};

struct Piece {              // a run of consecutive rows of one matrix (two for gate-up): one ring slot
  uint32_t src_off;         // byte offset of the first row inside its matrix
  uint32_t out0;            // index of the first row in the phase's output vector
  uint16_t nrows, row0;     // row0: index of the first row among the block's rows of the phase
  uint16_t item0, n_items;  // items are numbered through the phase; item j belongs to warp j % 16
  uint8_t kind, widx, pad[2];
};
struct PhInfo {
  uint16_t p0, np, nrows, nitems;
};

struct MegaArgs {
  const void* tables;       // MegaPhase[4] then MegaLayer[n_layers], 16-byte aligned; copied to shared memory at start
  unsigned tables_bytes;    // multiple of 16
  int n_layers;
  int n_slots;              // ring slots
  unsigned slot_bytes;      // bytes per ring slot (multiple of 128)
  unsigned x_bytes;         // staging area for x (also the attention scratch)
  unsigned n_q, n_kv, hd, n_splits;
  unsigned split_from;      // contexts longer than this are split across blocks
  float eps, attn_scale;
  const float* rope;        // [max_seq, hd]
  const int* pos;           // [1]
  const float* x_in;        // the token's embedding (residual stream on entry)
  float* resid_out;         // residual stream after the last layer's attention half
  float* y_out;             // last layer's down-proj output (the head applies the final residual update and norm)
  // tagged activation vectors, two of each (layer parity)
  u64 *ll_yd0, *ll_yd1, *ll_yo0, *ll_yo1, *ll_qkv0, *ll_qkv1, *ll_ox0, *ll_ox1, *ll_ff0, *ll_ff1, *ll_rec0, *ll_rec1;
  unsigned* epoch;          // tag base of this token; advanced by n_layers + 1 when the kernel ends
  unsigned* err;
  unsigned poll_limit;      // polls of one wait before it gives up
  unsigned test_stall;      // test hook: added to the tag the gate-up stage waits for (a tag nobody writes)
  long long* prof_all;      // optional [grid][n_layers][5][2]: thread 0 of every block, (phase entered, rows stored)
  long long* prof;          // optional [2][n_layers][5][8] SM clocks of the first and last block (thread 0): see the PF_* rows;
                            // matvec phases: entered, inputs arrived, x staged, tasks done, block joined, row stored; attention: entered, q arrived, q/k/v built, positions done, folded, -, stored, left
};

// ---- tagged words ---------------------------------------------------------------------------------
__device__ __forceinline__ void ll_store(u64* p, float v, unsigned tag) {
  const u64 w = ((u64)tag << 32) | (u64)__float_as_uint(v);
  asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void ll_load2(const u64* p, u64& a, u64& b) {
  asm volatile("ld.relaxed.gpu.global.v2.b64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ u64 ll_load1(const u64* p) {
  u64 a;
  asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
  return a;
}
__device__ __forceinline__ unsigned ld_relaxed_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ long long gtime() {  // nanoseconds, the same clock on every SM
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned ll_tag(u64 w) { return (unsigned)(w >> 32); }
__device__ __forceinline__ float ll_val(u64 w) { return __uint_as_float((unsigned)w); }

struct Poll {
  const unsigned* err;
  unsigned limit;
  bool gave_up;  // this thread stopped waiting (its own wait ran out, or it saw the status word raised)
};
// After a failed tag check: may the wait go on?
__device__ __noinline__ bool poll_again(Poll& pl, unsigned& it) {
  if (pl.gave_up) return false;
  if (++it >= pl.limit) {
    atomicOr(const_cast<unsigned*>(pl.err), 2u);
    pl.gave_up = true;
    return false;
  }
  if ((it & 127u) == 0u && ld_relaxed_u32(pl.err) != 0u) {
    pl.gave_up = true;
    return false;
  }
  return true;
}
// N chunks of 4 consecutive values (32 bytes, 16-byte aligned).  Every load is issued before any is checked,
// and every chunk that is still stale is re-read in the SAME round: a thread that came early pays one round
// trip per round, not one per chunk.
template <int N>
__device__ __forceinline__ void ll_wait_chunks(const u64* base, const unsigned (&c)[N], const bool (&live)[N], unsigned tag,
                                               float4 (&v)[N], Poll& pl) {
  u64 w[N][4];
#pragma unroll
  for (int k = 0; k < N; k++)
    if (live[k]) {
      ll_load2(base + (size_t)c[k] * 4, w[k][0], w[k][1]);
      ll_load2(base + (size_t)c[k] * 4 + 2, w[k][2], w[k][3]);
    }
  unsigned it = 0;
  for (;;) {
    bool stale[N], any = false;
#pragma unroll
    for (int k = 0; k < N; k++) {
      stale[k] = live[k] && !(ll_tag(w[k][0]) == tag && ll_tag(w[k][1]) == tag && ll_tag(w[k][2]) == tag && ll_tag(w[k][3]) == tag);
      any = any || stale[k];
    }
    if (!any || !poll_again(pl, it)) break;
#pragma unroll
    for (int k = 0; k < N; k++)
      if (stale[k]) {
        ll_load2(base + (size_t)c[k] * 4, w[k][0], w[k][1]);
        ll_load2(base + (size_t)c[k] * 4 + 2, w[k][2], w[k][3]);
      }
  }
#pragma unroll
  for (int k = 0; k < N; k++)
    if (live[k]) v[k] = make_float4(ll_val(w[k][0]), ll_val(w[k][1]), ll_val(w[k][2]), ll_val(w[k][3]));
}

// ---- staging of x ---------------------------------------------------------------------------------
// Sum four values over the block: every thread gets the same totals (fixed order).  red: 16 float4.
__device__ __forceinline__ float4 block_sum4(float4 v, float4* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    v.x += __shfl_xor_sync(0xffffffffu, v.x, o);
    v.y += __shfl_xor_sync(0xffffffffu, v.y, o);
    v.z += __shfl_xor_sync(0xffffffffu, v.z, o);
    v.w += __shfl_xor_sync(0xffffffffu, v.w, o);
  }
  __syncthreads();  // the previous use of red is over
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float4 t = red[0];
#pragma unroll 1
  for (int w = 1; w < MG_NW; w++) {
    const float4 u = red[w];
    t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
  }
  return t;
}

// Per-thread wait state, carried through the phase functions in one word (they are separate,
// non-inlined functions so that each gets the whole register budget; everything block-wide lives in
// shared memory): bits 0-7 ring slot of the next piece, bit 8 its mbarrier parity, bit 9 this warp
// stopped waiting for weight copies, bit 10 this thread stopped waiting for other blocks.
constexpr unsigned ST_DEAD = 1u << 9, ST_GAVE_UP = 1u << 10;

// The hidden vector of a phase that starts with a norm.  Thread t owns chunks t and t + 512 (4 elements
// each) of the residual stream; it keeps them in shared memory (xres) between phases.
//   add == false (first layer):  x' = rms(x) * w
//   add == true:  r = x + rms(y) * wp (K:539; both RMS factors come from ONE block-wide sum:
//                 sum r^2 = sum x^2 + 2 inv sum x y wp + inv^2 sum (y wp)^2);  x' = rms(r) * w;  xres = r.
template <int PC>
__device__ MG_FN unsigned mg_stage_hidden(unsigned char* xs, float4* red, float* xres, bool add, unsigned cols,
                                                 const u64* ysrc, unsigned tag, const float* w, const float* wp, float eps,
                                                 float* resid_out, const unsigned* err, unsigned limit, unsigned st, long long* pf) {
  Poll pl{err, limit, (st & ST_GAVE_UP) != 0u};
  const unsigned units = cols >> 6, nchunk = cols >> 2;
  unsigned c[PC];
  bool live[PC];
  float4 wv[PC], wpv[PC], yv[PC], xr[PC];
#pragma unroll
  for (int k = 0; k < PC; k++) {
    c[k] = threadIdx.x + k * MG_THREADS;
    live[k] = c[k] < nchunk;
    if (live[k]) {  // constants of the model: in flight while the inputs are awaited
      wv[k] = reinterpret_cast<const float4*>(w)[c[k]];
      if (add) wpv[k] = reinterpret_cast<const float4*>(wp)[c[k]];
      xr[k] = reinterpret_cast<const float4*>(xres)[c[k]];
    }
  }
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  if (add) {
    ll_wait_chunks<PC>(ysrc, c, live, tag, yv, pl);
#pragma unroll
    for (int k = 0; k < PC; k++)
      if (live[k]) {
        const float4 x = xr[k], y = yv[k], p = wpv[k];
        const float t0 = y.x * p.x, t1 = y.y * p.y, t2 = y.z * p.z, t3 = y.w * p.w;
        s.x = fmaf(y.x, y.x, s.x); s.x = fmaf(y.y, y.y, s.x); s.x = fmaf(y.z, y.z, s.x); s.x = fmaf(y.w, y.w, s.x);
        s.y = fmaf(x.x, t0, s.y); s.y = fmaf(x.y, t1, s.y); s.y = fmaf(x.z, t2, s.y); s.y = fmaf(x.w, t3, s.y);
        s.z = fmaf(t0, t0, s.z); s.z = fmaf(t1, t1, s.z); s.z = fmaf(t2, t2, s.z); s.z = fmaf(t3, t3, s.z);
        s.w = fmaf(x.x, x.x, s.w); s.w = fmaf(x.y, x.y, s.w); s.w = fmaf(x.z, x.z, s.w); s.w = fmaf(x.w, x.w, s.w);
      }
  } else {
#pragma unroll
    for (int k = 0; k < PC; k++)
      if (live[k]) {
        const float4 x = xr[k];
        s.w = fmaf(x.x, x.x, s.w); s.w = fmaf(x.y, x.y, s.w); s.w = fmaf(x.z, x.z, s.w); s.w = fmaf(x.w, x.w, s.w);
      }
  }
  if (pf) pf[1] = clock64();
  const float4 t = block_sum4(s, red);
  const float invn = 1.0f / (float)cols;
  float inv = 0.0f, inv2;
  if (add) {
    inv = __frsqrt_rn(t.x * invn + eps);
    const float rr = fmaf(inv * inv, t.z, fmaf(2.0f * inv, t.y, t.w));
    inv2 = __frsqrt_rn(fmaxf(rr, 0.0f) * invn + eps);
  } else {
    inv2 = 1.0f / sqrtf(t.w * invn + eps);
  }
#pragma unroll
  for (int k = 0; k < PC; k++)
    if (live[k]) {  // nchunk is a multiple of 64: whole warps take this branch together
      float4 r = xr[k];
      if (add) {
        const float4 y = yv[k], p = wpv[k];
        r.x = __fadd_rn(r.x, __fmul_rn(__fmul_rn(y.x, inv), p.x));
        r.y = __fadd_rn(r.y, __fmul_rn(__fmul_rn(y.y, inv), p.y));
        r.z = __fadd_rn(r.z, __fmul_rn(__fmul_rn(y.z, inv), p.z));
        r.w = __fadd_rn(r.w, __fmul_rn(__fmul_rn(y.w, inv), p.w));
        reinterpret_cast<float4*>(xres)[c[k]] = r;
        if (resid_out) reinterpret_cast<float4*>(resid_out)[c[k]] = r;
      }
      const float4 w4 = wv[k];
      float4 q;
      q.x = __fmul_rn(__fmul_rn(r.x, inv2), w4.x);
      q.y = __fmul_rn(__fmul_rn(r.y, inv2), w4.y);
      q.z = __fmul_rn(__fmul_rn(r.z, inv2), w4.z);
      q.w = __fmul_rn(__fmul_rn(r.w, inv2), w4.w);
      fx_put_chunk(xs, units, c[k], q);
    }
  return pl.gave_up ? (st | ST_GAVE_UP) : st;
}

// A vector other blocks produced (attention output, GeGLU output), staged as it is.
__device__ MG_FN unsigned mg_stage_plain(unsigned char* xs, unsigned cols, const u64* src, unsigned tag, const unsigned* err,
                                                unsigned limit, unsigned st, long long* pf) {
  Poll pl{err, limit, (st & ST_GAVE_UP) != 0u};
  constexpr int XC = 6;
  const unsigned units = cols >> 6, nchunk = cols >> 2;
  for (unsigned base = 0; base < nchunk; base += XC * MG_THREADS) {
    unsigned c[XC];
    bool live[XC];
    float4 v[XC];
#pragma unroll
    for (int k = 0; k < XC; k++) {
      c[k] = base + threadIdx.x + k * MG_THREADS;
      live[k] = c[k] < nchunk;
    }
    ll_wait_chunks<XC>(src, c, live, tag, v, pl);
    if (pf) pf[1] = clock64();
#pragma unroll
    for (int k = 0; k < XC; k++)
      if (live[k]) fx_put_chunk(xs, units, c[k], v[k]);
  }
  return pl.gave_up ? (st | ST_GAVE_UP) : st;
}

// ---- pieces -----------------------------------------------------------------------------------------
// Rows [lo, hi) of a phase's row space owned by this block: an even split in pairs of rows.
__device__ __forceinline__ void block_rows(const MegaPhase& ph, unsigned& lo, unsigned& hi) {
  const unsigned half = ph.seg_start[ph.n_seg] >> 1;
  lo = (unsigned)(((unsigned long long)blockIdx.x * half) / gridDim.x) * 2u;
  hi = (unsigned)(((unsigned long long)(blockIdx.x + 1) * half) / gridDim.x) * 2u;
}
// Thread 0 lists this block's pieces of one layer, in the order they are consumed.  Returns false when a table overflows.
__device__ __forceinline__ bool build_pieces(Piece* pieces, PhInfo* info, const MegaPhase* phases) {
  unsigned np = 0;
  for (int kind = 0; kind < PH_KINDS; kind++) {
    const MegaPhase& ph = phases[kind];
    unsigned lo, hi, rows = 0, items = 0;
    block_rows(ph, lo, hi);
    info[kind].p0 = (uint16_t)np;
    for (unsigned s = 0; s < ph.n_seg; s++) {
      const unsigned a = max(lo, ph.seg_start[s]), b = min(hi, ph.seg_start[s + 1]);
      for (unsigned r = a; r < b; r += ph.piece_rows) {
        if (np >= (unsigned)MG_MAXPIECE) return false;
        const unsigned n = min(ph.piece_rows, b - r);
        Piece p;
        p.src_off = (r - ph.seg_start[s]) * ph.row_bytes;
        p.out0 = r;
        p.nrows = (uint16_t)n;
        p.row0 = (uint16_t)rows;
        p.item0 = (uint16_t)items;
        p.n_items = 0;
        p.kind = (uint8_t)kind;
        p.widx = (uint8_t)(ph.widx + s);
        p.pad[0] = p.pad[1] = 0;
        pieces[np++] = p;
        rows += n;
        items += p.n_items;
      }
    }
    if (rows > (unsigned)MG_MAXROWS) return false;
    info[kind].np = (uint16_t)(np - info[kind].p0);
    info[kind].nrows = (uint16_t)rows;
    info[kind].nitems = (uint16_t)items;
  }
  return true;
}
// Start the copies of one piece into a ring slot (one thread).
__device__ __forceinline__ void issue_piece(const Piece& p, const MegaPhase& ph, const MegaLayer& L, uint32_t slot_addr, uint32_t bar) {
  const unsigned bytes = (unsigned)p.nrows * ph.row_bytes;
  mb_expect(bar, bytes * ph.mats);
  bulk_in(slot_addr, L.W[p.widx] + p.src_off, bytes, bar);
  if (ph.mats == 2) bulk_in(slot_addr + (((unsigned)p.nrows + 3u) & ~3u) * ph.row_bytes, L.W[p.widx + 1] + p.src_off, bytes, bar);
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

constexpr int MG_AB = 8;  // positions of one warp in flight together

// Shared memory the attention phase needs (it reuses the x staging area).
__host__ __device__ inline unsigned mg_att_bytes(unsigned hd) {
  const unsigned rowb = (hd / 32u) * KS_Q40_BLOCK_BYTES;
  return (unsigned)MG_NW * (hd + 2u) * 4u + 2u * (rowb + 16u) + 8u * MG_MAX_SPLITS + 12u * hd + 4u * MG_NW +
         (unsigned)MG_NW * MG_AB * 2u * rowb + 32u;
}

// Splits in use for a context of tlen positions: a warp walks at most four positions (one batch of
// loads in flight) until every split is in use.  A split costs a hop through L2 (records out, merge in
// the head's first block); contexts of up to split_from positions stay in one block.
__host__ __device__ inline unsigned mg_active_splits(unsigned tlen, unsigned max_splits, unsigned split_from) {
  if (tlen <= split_from) return 1u;
  unsigned ns = (tlen + 4u * MG_NW - 1u) / (4u * MG_NW);
  return ns < 1u ? 1u : ns > max_splits ? max_splits : ns;
}


// What the attention phase needs, block-wide (read from shared memory).
struct AttnArgs {
  unsigned n_q, n_kv, n_splits, split_from;
  float eps, attn_scale;
  const float* rope;
  const int* pos;
  const unsigned* err;
  unsigned limit;
};

// Sum of v over the first nw warps of the block (every thread of those warps calls, every thread gets the
// total); red: MG_NW floats of scratch.  Fixed order.
__device__ __forceinline__ float mg_rows_sum(float v, float* red, int nw) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = mg_warp_sum(v);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.0f;
  for (int w = 0; w < nw; w++) t += red[w];
  return t;
}

// One block per (query head, context split).  The code is kept small on purpose (rolled loops, one
// value per thread): it runs once per layer, so its instructions are fetched cold every time.
//   0. each warp starts the loads of its first positions' packed K/V rows (cp.async into the scratch):
//      they do not depend on this layer's q, so they travel while q is awaited;
//   1. thread d awaits q[d] of the head (and k[d], v[d] in the block(s) of the split that holds the newest
//      position), the block norms and ropes them (lower.rs:4231-4702): q stays in shared memory for the
//      dot products, the new K / V rows are packed to Q4_0 (one warp per 32-value block) and the block of
//      the KV group's first head stores them to the cache;
//   2. warps take the positions of the split round-robin, four rows in flight, online softmax per warp;
//   3. the warps' (m, l, O) meet in shared memory, thread d folds dimension d;
//   4. one split: thread d stores the head's output; several: the block leaves a tagged (m, l, O[hd])
//      record and the head's first block merges the records (lower.rs:5897-6088).
template <int DPL>
__device__ MG_FN unsigned mg_attention(const AttnArgs* ap, const MegaLayer* Lp, const u64* qkv, u64* ox, u64* rec, unsigned tag,
                                       unsigned char* sm, unsigned st, long long* pf) {
  constexpr int HD = DPL * 32, HALF = HD / 2, NB = HD / 32;
  constexpr unsigned ROWB = NB * KS_Q40_BLOCK_BYTES;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned NSMAX = ap->n_splits, n_q = ap->n_q, n_kv = ap->n_kv;
  if (blockIdx.x >= n_q * NSMAX) return st;
  const unsigned head = blockIdx.x / NSMAX, split = blockIdx.x % NSMAX;
  const unsigned G = n_q / n_kv, kvh = head / G;
  const unsigned pos = (unsigned)ap->pos[0], tlen = pos + 1;
  const unsigned NS = mg_active_splits(tlen, NSMAX, ap->split_from);
  if (split >= NS) return st;
  Poll pl{ap->err, ap->limit, (st & ST_GAVE_UP) != 0u};
  const unsigned chunk = (tlen + NS - 1) / NS;
  const unsigned p0 = split * chunk, p1 = min(p0 + chunk, tlen);
  const bool owner = pos >= p0 && pos < p1;  // the split that holds the newest position
  // scratch: part [NW][HD + 2] | skrow | svrow | ml [2 * MAX_SPLITS] | vec [3][HD] (q, k, v) | red [NW] | kvbuf
  float* part = reinterpret_cast<float*>(sm);
  uint8_t* skrow = reinterpret_cast<uint8_t*>(part + MG_NW * (HD + 2));
  uint8_t* svrow = skrow + ROWB + 16u;
  float* ml = reinterpret_cast<float*>(svrow + ROWB + 16u);
  float* vec = ml + 2 * MG_MAX_SPLITS;
  float* red = vec + 3 * HD;
  uint8_t* kvbuf = reinterpret_cast<uint8_t*>(red + MG_NW) + (size_t)warp * (MG_AB * 2u * ROWB);  // [MG_AB][K, V][ROWB]
  const float* cs = ap->rope + (size_t)pos * HD;
  const unsigned qn = n_q * HD, kvn = n_kv * HD;
  const size_t rowstride = (size_t)n_kv * ROWB;
  uint8_t* Kc = Lp->kv_k + (size_t)kvh * ROWB;
  uint8_t* Vc = Lp->kv_v + (size_t)kvh * ROWB;

  // 0. the first batch of cached rows (the newest position's row does not exist yet: it comes from skrow / svrow)
  auto prefetch_rows = [&](unsigned tb) {
#pragma unroll 1
    for (int i = 0; i < MG_AB; i++) {
      const unsigned t = tb + (unsigned)(MG_NW * i);
      if (t < p1 && t != pos && lane < (int)(ROWB / 8u)) {
        cp_async8(sm32(kvbuf + (size_t)(2 * i) * ROWB) + (uint32_t)lane * 8u, Kc + (size_t)t * rowstride + (size_t)lane * 8u);
        cp_async8(sm32(kvbuf + (size_t)(2 * i + 1) * ROWB) + (uint32_t)lane * 8u, Vc + (size_t)t * rowstride + (size_t)lane * 8u);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  prefetch_rows(p0 + (unsigned)warp);

  // 1. q (and the new k, v): one value per thread
  const int d = threadIdx.x;
  const bool has = d < HD;  // whole warps: HD is a multiple of 32
  {
    float qv = 0.f, kx = 0.f, vx = 0.f, qw = 0.f, kw = 0.f, c = 0.f, sn = 0.f;
    if (has) {
      qw = Lp->norm[1][d];
      c = cs[d & (HALF - 1)];
      sn = cs[HALF + (d & (HALF - 1))];
      if (owner) kw = Lp->norm[2][d];
      const u64* qp = qkv + (size_t)head * HD + d;
      const u64* kp = qkv + qn + (size_t)kvh * HD + d;
      const u64* vp = kp + kvn;
      u64 wq = ll_load1(qp), wk = 0, wv = 0;
      if (owner) {
        wk = ll_load1(kp);
        wv = ll_load1(vp);
      }
      unsigned it = 0;
      if (owner) {  // every stale word is re-read in the same round
        while (!(ll_tag(wq) == tag && ll_tag(wk) == tag && ll_tag(wv) == tag) && poll_again(pl, it)) {
          if (ll_tag(wq) != tag) wq = ll_load1(qp);
          if (ll_tag(wk) != tag) wk = ll_load1(kp);
          if (ll_tag(wv) != tag) wv = ll_load1(vp);
        }
        kx = ll_val(wk);
        vx = ll_val(wv);
      } else {
        while (ll_tag(wq) != tag && poll_again(pl, it)) wq = ll_load1(qp);
      }
      qv = ll_val(wq);
    }
    if (pf) pf[1] = clock64();
    if (warp < NB) {  // the warps that hold the HD values
      const float sq = mg_rows_sum(qv * qv, red, NB);
      const float invq = 1.0f / sqrtf(sq / (float)HD + ap->eps);
      vec[d] = __fmul_rn(__fmul_rn(qv, invq), qw);
      if (owner) {
        __syncthreads();
        const float sk = mg_rows_sum(kx * kx, red, NB);
        __syncthreads();
        const float sv = mg_rows_sum(vx * vx, red, NB);
        const float invk = 1.0f / sqrtf(sk / (float)HD + ap->eps), invv = 1.0f / sqrtf(sv / (float)HD + ap->eps);
        vec[HD + d] = __fmul_rn(__fmul_rn(kx, invk), kw);
        vx = __fmul_rn(vx, invv);
      }
    } else {  // the other warps only keep the barriers company
      __syncthreads();
      if (owner) {
        __syncthreads();
        __syncthreads();
        __syncthreads();
        __syncthreads();
      }
    }
    __syncthreads();  // u = normed q (and k) of every dimension is in vec
    float qrot = 0.f, krot = 0.f;
    if (has) {
      // dims of the first half pair with dim + HD/2 (gemma_prim.rs:33-56 cos / sin table)
      const float u = vec[d], pu = vec[d ^ HALF];
      qrot = d < HALF ? __fsub_rn(__fmul_rn(u, c), __fmul_rn(pu, sn)) : __fadd_rn(__fmul_rn(pu, sn), __fmul_rn(u, c));
      if (owner) {
        const float uk = vec[HD + d], pk = vec[HD + (d ^ HALF)];
        krot = d < HALF ? __fsub_rn(__fmul_rn(uk, c), __fmul_rn(pk, sn)) : __fadd_rn(__fmul_rn(pk, sn), __fmul_rn(uk, c));
      }
    }
    __syncthreads();  // every partner was read
    if (has) {
      vec[d] = qrot * ap->attn_scale;
      if (owner) {
        // values pass through f16 before packing (render.rs:1046); warp w holds block w of both rows
        mg_pack_q40(__half2float(__float2half_rn(krot)), skrow + warp * KS_Q40_BLOCK_BYTES, lane);
        mg_pack_q40(__half2float(__float2half_rn(vx)), svrow + warp * KS_Q40_BLOCK_BYTES, lane);
      }
    }
    __syncthreads();  // q and the packed rows are in shared memory
    if (owner && head == kvh * G) {
      const unsigned n16 = ROWB / 2;
      if (threadIdx.x < n16)
        reinterpret_cast<unsigned short*>(Kc + (size_t)pos * rowstride)[threadIdx.x] = reinterpret_cast<const unsigned short*>(skrow)[threadIdx.x];
      else if (threadIdx.x < 2 * n16)
        reinterpret_cast<unsigned short*>(Vc + (size_t)pos * rowstride)[threadIdx.x - n16] =
            reinterpret_cast<const unsigned short*>(svrow)[threadIdx.x - n16];
    }
  }
  if (pf) pf[2] = clock64();
  float qr[DPL];
#pragma unroll
  for (int j = 0; j < DPL; j++) qr[j] = vec[mg_lane_dim<DPL>(lane, j)];

  // 2. this warp's positions
  float o[DPL], m = kNegInit, l = 0.0f;
#pragma unroll
  for (int j = 0; j < DPL; j++) o[j] = 0.0f;
#pragma unroll 1
  for (unsigned tb = p0 + (unsigned)warp; tb < p1; tb += MG_NW * MG_AB) {
    if (tb != p0 + (unsigned)warp) {  // later batches (long contexts): the buffer is free again
      __syncwarp();
      prefetch_rows(tb);
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncwarp();
#pragma unroll 1
    for (int i = 0; i < MG_AB; i++) {
      const unsigned t = tb + (unsigned)(MG_NW * i);
      if (t >= p1) break;
      RawRow<DPL> kr, vr;
      raw_load<DPL>(t == pos ? skrow : kvbuf + (size_t)(2 * i) * ROWB, lane, kr);
      raw_load<DPL>(t == pos ? svrow : kvbuf + (size_t)(2 * i + 1) * ROWB, lane, vr);
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
  if (pf) pf[3] = clock64();
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
  // 3. thread d folds head dimension d over the warps; it sits in slot j * 32 + lane of the warps' layout
  int dslot;
  {
    constexpr int BPL = DPL / 2, LPB = 16 / BPL;
    const int within = d & 31, hh = within >> 4, w16 = within & 15;
    dslot = (hh * BPL + (w16 % BPL)) * 32 + (((d >> 5) & (NB - 1)) * LPB + w16 / BPL);
  }
  float M = kNegInit, Lsum = 0.0f, O = 0.0f;
  if (has) {
#pragma unroll 1
    for (int w = 0; w < MG_NW; w++) M = fmaxf(M, part[w * (HD + 2)]);
#pragma unroll 1
    for (int w = 0; w < MG_NW; w++) {
      const float f = __expf(part[w * (HD + 2)] - M);
      Lsum = fmaf(part[w * (HD + 2) + 1], f, Lsum);
      O = fmaf(part[w * (HD + 2) + 2 + dslot], f, O);
    }
  }
  if (pf) pf[4] = clock64();
  // 4.
  if (NS == 1) {  // one split: this block's result is final
    if (has) ll_store(ox + (size_t)head * HD + d, O / Lsum, tag);
  } else {
    u64* myrec = rec + ((size_t)head * NSMAX + split) * (HD + 2);
    if (split != 0) {
      if (has) {
        ll_store(myrec + 2 + d, O, tag);  // records are kept in dimension order
        if (d == 0) {
          ll_store(myrec, M, tag);
          ll_store(myrec + 1, Lsum, tag);
        }
      }
    } else {
      // The head's first block merges (lower.rs:5897-6088): its own record is in registers, the others are
      // awaited.  Thread p fetches (m, l) of split p for everybody; thread d fetches O[d], four splits at a time.
      const u64* rec0 = rec + (size_t)head * NSMAX * (HD + 2);
      if (d == 0) {
        ml[0] = M;
        ml[1] = Lsum;
      } else if ((unsigned)d < NS) {
        const u64* r = rec0 + (size_t)d * (HD + 2);
        u64 w0 = ll_load1(r), w1 = ll_load1(r + 1);
        unsigned it = 0;
        while (!(ll_tag(w0) == tag && ll_tag(w1) == tag) && poll_again(pl, it)) {
          w0 = ll_load1(r);
          w1 = ll_load1(r + 1);
        }
        ml[2 * d] = ll_val(w0);
        ml[2 * d + 1] = ll_val(w1);
      }
      __syncthreads();
      if (has) {
        float MM = kNegInit;
#pragma unroll 1
        for (unsigned p = 0; p < NS; p++) MM = fmaxf(MM, ml[2 * p]);
        float f0 = __expf(ml[0] - MM);
        float LL = ml[1] * f0, OO = O * f0;
#pragma unroll 1
        for (unsigned pb = 1; pb < NS; pb += 4) {
          u64 w[4];
#pragma unroll
          for (int k = 0; k < 4; k++)
            if (pb + k < NS) w[k] = ll_load1(rec0 + (size_t)(pb + k) * (HD + 2) + 2 + d);
          {
            unsigned it = 0;
            for (;;) {
              bool any = false;
#pragma unroll
              for (int k = 0; k < 4; k++) any = any || (pb + k < NS && ll_tag(w[k]) != tag);
              if (!any || !poll_again(pl, it)) break;
#pragma unroll
              for (int k = 0; k < 4; k++)
                if (pb + k < NS && ll_tag(w[k]) != tag) w[k] = ll_load1(rec0 + (size_t)(pb + k) * (HD + 2) + 2 + d);
            }
          }
#pragma unroll
          for (int k = 0; k < 4; k++)
            if (pb + k < NS) {
              const float f = __expf(ml[2 * (pb + k)] - MM);
              LL = fmaf(ml[2 * (pb + k) + 1], f, LL);
              OO = fmaf(ll_val(w[k]), f, OO);
            }
        }
        ll_store(ox + (size_t)head * HD + d, OO / LL, tag);
      }
    }
  }
  if (pf) pf[6] = clock64();
  __syncthreads();  // the scratch is the next phase's x staging area
  if (pf) pf[7] = clock64();
  return pl.gave_up ? (st | ST_GAVE_UP) : st;
}

// ---- the kernel -------------------------------------------------------------------------------------
struct MegaSmem {
  unsigned xs_off, xres_off, ring_off, bar_off, done_off, red_off, psum_off, rowtab_off, tab_off, piece_off, info_off, total;
};
__host__ __device__ inline MegaSmem mg_smem(unsigned x_bytes, unsigned hidden, unsigned slot_bytes, int n_slots, unsigned tables_bytes) {
  MegaSmem L;
  L.xs_off = 1024u;  // MegaShared first
  L.xres_off = L.xs_off + ((x_bytes + 127u) & ~127u);
  L.ring_off = L.xres_off + ((hidden * 4u + 127u) & ~127u);
  L.bar_off = L.ring_off + (unsigned)n_slots * slot_bytes;
  L.done_off = L.bar_off + MG_MAXSLOTS * 8u;
  L.red_off = L.done_off + MG_MAXSLOTS * 4u;      // 16 float4 of block sums
  L.psum_off = L.red_off + MG_NW * 16u;
  L.rowtab_off = L.psum_off + 2u * MG_MAXROWS * MG_MAXC * 4u;
  L.tab_off = L.rowtab_off + 2u * MG_MAXROWS * 4u;
  L.piece_off = L.tab_off + tables_bytes;
  L.info_off = L.piece_off + MG_MAXPIECE * (unsigned)sizeof(Piece);
  L.total = L.info_off + PH_KINDS * (unsigned)sizeof(PhInfo) + 16u;
  return L;
}

struct MegaShared {  // block-wide state at the start of dynamic shared memory
  MegaSmem SL;
  AttnArgs att;
  unsigned n_slots, slot_bytes, n_layers, poll_limit;
  unsigned NP, total_pieces;
  unsigned* err;
  int ok;
};
static_assert(sizeof(MegaShared) <= 1024, "MegaShared must fit its reserved kilobyte");

// One matvec phase after its input was staged.  A lane owns one 64-weight unit of a 32-unit column
// segment and keeps that unit of x in registers; a task is (segment, matrix, row); the tasks of a wave
// (the rows of up to half the ring's slots) are ordered segment-major and cut into one
// contiguous range per warp, so a warp loads x at most twice per wave and all warps get the same number
// of tasks (+-1); two tasks run interleaved.  Row sums meet in shared memory; after a block-wide barrier
// thread f finishes row f of the wave (segments added in order, epilogue, tagged store) while lanes of the
// last warp refill the wave's slots with the pieces n_slots further down the sequence (one lane per slot:
// issuing them one after the other from one thread cost 0.3 us each on the critical path).  Begins with
// the block-wide barrier that ends the staging of x.
__device__ MG_FN unsigned mg_phase(int kind, int layer, unsigned tag, u64* out, float* plain, long long* pf, unsigned st, long long* pa) {
  extern __shared__ __align__(128) unsigned char smem[];
  const MegaShared* S = reinterpret_cast<const MegaShared*>(smem);
  const MegaSmem& SL = S->SL;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t ring_s = sm32(smem + SL.ring_off), bars = sm32(smem + SL.bar_off), xs_s = sm32(smem + SL.xs_off);
  float* psum = reinterpret_cast<float*>(smem + SL.psum_off);
  uint32_t* rowaddr = reinterpret_cast<uint32_t*>(smem + SL.rowtab_off);  // shared address of each row of the wave (first matrix)
  uint32_t* rowmat2 = rowaddr + MG_MAXROWS;                               // distance to the same row of the second matrix
  const MegaPhase* phases = reinterpret_cast<const MegaPhase*>(smem + SL.tab_off);
  const MegaLayer* layers = reinterpret_cast<const MegaLayer*>(smem + SL.tab_off + ((PH_KINDS * sizeof(MegaPhase) + 15u) & ~15u));
  const Piece* pieces = reinterpret_cast<const Piece*>(smem + SL.piece_off);
  const PhInfo inf = reinterpret_cast<const PhInfo*>(smem + SL.info_off)[kind];
  const MegaPhase& ph = phases[kind];
  const unsigned n_slots = S->n_slots, slot_bytes = S->slot_bytes, NP = S->NP;
  unsigned slot = st & 0xFFu, par = (st >> 8) & 1u;
  bool dead = (st & ST_DEAD) != 0u;

  const unsigned NS = ph.n_cseg, units = ph.cols >> 6, seg_units = ph.seg_units;
  const unsigned row_bytes = ph.row_bytes, mats = ph.mats;
  const unsigned wave_max = n_slots > 1u ? n_slots / 2u : 1u;
  const bool active = (unsigned)lane < seg_units;
  XUnit x;
  int cur_s = -1;
  for (unsigned wp0 = inf.p0; wp0 < (unsigned)inf.p0 + inf.np; wp0 += wave_max) {
    const unsigned wp1 = min(wp0 + wave_max, (unsigned)inf.p0 + inf.np);
    const unsigned wr0 = pieces[wp0].row0, wr1 = (unsigned)pieces[wp1 - 1].row0 + pieces[wp1 - 1].nrows, rows_w = wr1 - wr0;
    if (threadIdx.x < rows_w) {
      const unsigned r = wr0 + threadIdx.x;
      unsigned pi = wp0;
      while (pi + 1 < wp1 && pieces[pi + 1].row0 <= r) pi++;
      unsigned sl = slot + (pi - wp0);
      if (sl >= n_slots) sl -= n_slots;
      rowaddr[threadIdx.x] = ring_s + sl * slot_bytes + (r - pieces[pi].row0) * row_bytes;
      rowmat2[threadIdx.x] = (((unsigned)pieces[pi].nrows + 3u) & ~3u) * row_bytes;
    }
    __syncthreads();  // x is staged (first wave), the row table is written
    if (pf && wp0 == inf.p0) pf[2] = clock64();
    if (pa && threadIdx.x == 0 && wp0 == inf.p0) pa[3] = gtime();
    // the wave's weights: one lane per piece asks the piece's mbarrier, the warp votes
    if (!dead) {
      bool ok = true;
      if ((unsigned)lane < wp1 - wp0) {
        unsigned sl = slot + (unsigned)lane, pr = par;
        if (sl >= n_slots) {
          sl -= n_slots;
          pr ^= 1u;
        }
        ok = mb_wait(bars + sl * 8u, pr, S->poll_limit);
      }
      if (!__all_sync(0xffffffffu, ok)) {
        dead = true;
        if (lane == 0) atomicOr(S->err, 1u);
      }
    }
    if (pa && threadIdx.x == 0 && wp0 == inf.p0) pa[4] = gtime();
    if (!dead) {
      const unsigned per_seg = mats * rows_w, T = NS * per_seg;
      const unsigned t0 = (unsigned)warp * T / MG_NW, t1 = (unsigned)(warp + 1) * T / MG_NW;
      unsigned t = t0, sg = t0 / per_seg, rem = t0 - sg * per_seg;
      // task (sg, rem): rem < rows_w is row rem of the first matrix, else row rem - rows_w of the second
      auto row_of = [&](unsigned q, uint32_t uoff, uint32_t& wa, unsigned& pidx) {
        const unsigned m = q >= rows_w ? 1u : 0u, r = q - m * rows_w;
        wa = rowaddr[r] + (m ? rowmat2[r] : 0u) + uoff;
        pidx = ((wr0 + r) * mats + m) * NS + sg;
      };
#pragma unroll 1
      while (t < t1) {
        const unsigned u = sg * seg_units + (unsigned)lane;
        if ((int)sg != cur_s) {
          if (active) fx_load_unit(x, xs_s, units, u);
          cur_s = (int)sg;
        }
        const uint32_t uoff = (u >> 2) * KS_Q4K_BLOCK_BYTES + (u & 3u) * 32u;
        unsigned n = min(t1 - t, per_seg - rem);  // my tasks left in this segment
        t += n;
#pragma unroll 1
        for (; n >= 2u; n -= 2u, rem += 2u) {  // two rows at a time: their instruction streams interleave
          uint32_t wa[2];
          unsigned pidx[2];
          row_of(rem, uoff, wa[0], pidx[0]);
          row_of(rem + 1u, uoff, wa[1], pidx[1]);
          float v[2] = {0.0f, 0.0f};
          if (active) fx_rows<2>(wa, (int)(u & 3u), x, v);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
            v[1] += __shfl_xor_sync(0xffffffffu, v[1], o);
          }
          if (lane == 0) {
            psum[pidx[0]] = v[0];
            psum[pidx[1]] = v[1];
          }
        }
        if (n) {
          uint32_t wa[1];
          unsigned pidx;
          row_of(rem, uoff, wa[0], pidx);
          float v[1] = {0.0f};
          if (active) fx_rows<1>(wa, (int)(u & 3u), x, v);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
          if (lane == 0) psum[pidx] = v[0];
          rem += 1u;
        }
        if (rem == per_seg) {
          rem = 0;
          sg++;
        }
      }
    }
    if (pf) pf[3] = clock64();
    if (pa && threadIdx.x == 0) pa[5] = gtime();
    __syncthreads();  // the wave's row sums are in shared memory and nobody reads its slots any more
    if (pf) pf[4] = clock64();
    if (pa && threadIdx.x == 0) pa[6] = gtime();
    // the last warp (never a finishing warp) refills the wave's slots with the pieces n_slots further on, one lane per slot
    if (warp == MG_NW - 1 && (unsigned)lane < wp1 - wp0) {
      const long long rt0 = pa ? gtime() : 0;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the slots were read through the generic proxy
      unsigned sl = slot + (unsigned)lane;
      if (sl >= n_slots) sl -= n_slots;
      unsigned npi = wp0 + (unsigned)lane + n_slots;
      unsigned nl = (unsigned)layer;
      while (npi >= NP) {
        npi -= NP;
        nl++;
      }
      if (nl < S->n_layers) {
        const Piece np_ = pieces[npi];
        issue_piece(np_, phases[np_.kind], layers[nl], ring_s + sl * slot_bytes, bars + sl * 8u);
      }
      if (pa && lane == 0) pa[7] = gtime() - rt0;
    }
    // thread f finishes row wr0 + f of the block: segments added in order, epilogue, tagged store
    if (threadIdx.x < rows_w) {
      const unsigned r = wr0 + threadIdx.x;
      unsigned pi = wp0;
      while (pi + 1 < wp1 && pieces[pi + 1].row0 <= r) pi++;
      const unsigned orow = pieces[pi].out0 + (r - pieces[pi].row0);
      const float* ps = psum + (size_t)r * mats * NS;
      float v0 = 0.0f;
      for (unsigned sg = 0; sg < NS; sg++) v0 += ps[sg];
      if (mats == 2) {
        float v1 = 0.0f;
        for (unsigned sg = 0; sg < NS; sg++) v1 += ps[NS + sg];
        v0 = gelu_mul(v0, v1);
      }
      ll_store(out + orow, v0, tag);
      if (plain) plain[orow] = v0;  // the head reads plain floats
    }
    if (pf) pf[5] = clock64();
    slot += wp1 - wp0;
    if (slot >= n_slots) {
      slot -= n_slots;
      par ^= 1u;
    }
  }
  return (st & ST_GAVE_UP) | slot | (par << 8) | (dead ? ST_DEAD : 0u);
}

template <int DPL, int PC>
__global__ void __launch_bounds__(MG_THREADS, 1) flow_kernel(const MegaArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  MegaShared* S = reinterpret_cast<MegaShared*>(smem);
  const unsigned H0 = reinterpret_cast<const MegaPhase*>(a.tables)[PH_QKV].cols;  // hidden size (tables are in global memory here)
  const MegaSmem SL = mg_smem(a.x_bytes, H0, a.slot_bytes, a.n_slots, a.tables_bytes);
  const uint32_t ring_s = sm32(smem + SL.ring_off);
  const uint32_t bars = sm32(smem + SL.bar_off);
  float4* red = reinterpret_cast<float4*>(smem + SL.red_off);
  float* xres = reinterpret_cast<float*>(smem + SL.xres_off);
  unsigned char* xs = smem + SL.xs_off;
  const MegaPhase* phases = reinterpret_cast<const MegaPhase*>(smem + SL.tab_off);
  const MegaLayer* layers = reinterpret_cast<const MegaLayer*>(smem + SL.tab_off + ((PH_KINDS * sizeof(MegaPhase) + 15u) & ~15u));
  Piece* pieces = reinterpret_cast<Piece*>(smem + SL.piece_off);
  PhInfo* info = reinterpret_cast<PhInfo*>(smem + SL.info_off);
  const unsigned n_slots = (unsigned)a.n_slots;

  for (unsigned i = threadIdx.x; i < a.tables_bytes / 16u; i += blockDim.x)
    reinterpret_cast<uint4*>(smem + SL.tab_off)[i] = reinterpret_cast<const uint4*>(a.tables)[i];
  if (threadIdx.x == 0) {
    S->SL = SL;
    S->att.n_q = a.n_q; S->att.n_kv = a.n_kv; S->att.n_splits = a.n_splits; S->att.split_from = a.split_from;
    S->att.eps = a.eps; S->att.attn_scale = a.attn_scale; S->att.rope = a.rope; S->att.pos = a.pos;
    S->att.err = a.err; S->att.limit = a.poll_limit;
    S->n_slots = n_slots; S->slot_bytes = a.slot_bytes; S->n_layers = (unsigned)a.n_layers; S->poll_limit = a.poll_limit;
    S->err = a.err;
    for (unsigned s = 0; s < n_slots; s++) mb_init(bars + s * 8u, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    S->ok = build_pieces(pieces, info, phases) ? 1 : 0;
    S->NP = (unsigned)info[PH_KINDS - 1].p0 + info[PH_KINDS - 1].np;
    S->total_pieces = S->NP * (unsigned)a.n_layers;
  }
  __syncthreads();
  if (!S->ok) {  // a table overflowed: the host's own check of the same arithmetic should have refused this shape
    if (threadIdx.x == 0) atomicOr(a.err, 4u);
    return;
  }
  const unsigned NP = S->NP, total_pieces = S->total_pieces;
  const unsigned epoch = *a.epoch;

  // fill the ring: piece n goes to slot n
  if (lane == 0)
    for (unsigned n = (unsigned)warp; n < n_slots && n < total_pieces; n += MG_NW) {
      const Piece p = pieces[n % NP];
      issue_piece(p, phases[p.kind], layers[n / NP], ring_s + n * a.slot_bytes, bars + n * 8u);
    }

  // the residual stream: thread t keeps chunks t and t + 512 (only ever touched by the same thread)
  const unsigned H = phases[PH_QKV].cols;
  for (unsigned c = threadIdx.x; c < (H >> 2); c += MG_THREADS)
    reinterpret_cast<float4*>(xres)[c] = reinterpret_cast<const float4*>(a.x_in)[c];

  long long* prof = nullptr;
  if (a.prof && threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1))
    prof = a.prof + (size_t)(blockIdx.x == 0 ? 0 : 1) * a.n_layers * PF_PER_LAYER * PF_STAMPS;

  long long* pall = (a.prof_all && (threadIdx.x == 0 || threadIdx.x == MG_THREADS - 32)) ? a.prof_all + (size_t)blockIdx.x * a.n_layers * PF_PER_LAYER * 8 : nullptr;
  unsigned st = 0u;  // ring position, wait state (see ST_*)
#pragma unroll 1
  for (int layer = 0; layer < a.n_layers; layer++) {
    const unsigned tag = epoch + (unsigned)layer + 1u;
    const int b = layer & 1;
    const bool last = layer + 1 == a.n_layers;
#pragma unroll 1
    for (int kind = 0; kind < PH_KINDS; kind++) {
      // kernel parameters are picked with selects (indexing them would force a local copy)
      u64* const yd = b ? a.ll_yd1 : a.ll_yd0;
      u64* const yo = b ? a.ll_yo1 : a.ll_yo0;
      u64* const qkv = b ? a.ll_qkv1 : a.ll_qkv0;
      u64* const ox = b ? a.ll_ox1 : a.ll_ox0;
      u64* const ff = b ? a.ll_ff1 : a.ll_ff0;
      // profile rows: qkv, attention, o-proj, gate-up, down
      long long* pf = prof ? prof + ((size_t)layer * PF_PER_LAYER + (kind == PH_QKV ? PF_QKV : kind + 1)) * PF_STAMPS : nullptr;
      const MegaLayer& L = layers[layer];
      if (kind == PH_OPROJ) {
        if (pall && threadIdx.x == 0) pall[((size_t)layer * PF_PER_LAYER + PF_ATTN) * 8] = gtime();
        if (pf) pf[-PF_STAMPS] = clock64();
        st = mg_attention<DPL>(&S->att, &L, qkv, ox, b ? a.ll_rec1 : a.ll_rec0, tag, xs, st, pf ? pf - PF_STAMPS : nullptr);
      }
      if (pall && threadIdx.x == 0) {
        if (kind == PH_OPROJ) pall[((size_t)layer * PF_PER_LAYER + PF_ATTN) * 8 + 1] = gtime();
        pall[((size_t)layer * PF_PER_LAYER + (kind == PH_QKV ? PF_QKV : kind + 1)) * 8] = gtime();
      }
      if (pf) pf[0] = clock64();
      // ---- this phase's input vector, staged in shared memory
      if (kind == PH_QKV || kind == PH_GATEUP) {
        // residual update (from the second phase on) + norm.  q/k/v: the previous layer's down-proj output
        // and post-FFN norm, then this layer's attention norm; gate/up: the o-proj output and post-attention
        // norm, then the FFN norm.
        const bool qk = kind == PH_QKV;
        st = mg_stage_hidden<PC>(xs, red, xres, !qk || layer > 0, H, qk ? (b ? a.ll_yd0 : a.ll_yd1) : yo,
                                 qk ? tag - 1u : tag + a.test_stall, qk ? L.norm[0] : L.norm[4],
                                 qk ? layers[layer > 0 ? layer - 1 : 0].norm[5] : L.norm[3], a.eps,
                                 (!qk && last && blockIdx.x == 0) ? a.resid_out : nullptr, a.err, a.poll_limit, st, pf);
      } else {
        st = mg_stage_plain(xs, phases[kind].cols, kind == PH_OPROJ ? ox : ff, tag, a.err, a.poll_limit, st, pf);
      }
      u64* const out = kind == PH_QKV ? qkv : kind == PH_OPROJ ? yo : kind == PH_GATEUP ? ff : yd;
      long long* pa = pall ? pall + ((size_t)layer * PF_PER_LAYER + (kind == PH_QKV ? PF_QKV : kind + 1)) * 8 : nullptr;
      if (pa && threadIdx.x == 0) pa[2] = gtime();
      st = mg_phase(kind, layer, tag, out, (kind == PH_DOWN && last) ? a.y_out : nullptr, pf, st, pa);
      if (pa && threadIdx.x == 0) pa[1] = gtime();
    }
  }
  // The next token's tags must differ from everything this one wrote.  Every block read the epoch before
  // block 0 can get here (its last phase needed rows from all of them).
  if (blockIdx.x == 0 && threadIdx.x == 0) *a.epoch = epoch + (unsigned)a.n_layers + 1u;
  // copies still in flight must land before this block's shared memory goes away (bounded; a no-op unless a warp gave up)
  __syncthreads();
  if (threadIdx.x == 0) {
    for (unsigned s = 0; s < n_slots && s < total_pieces; s++) {
      const unsigned n_last = s + ((total_pieces - 1u - s) / n_slots) * n_slots;
      mb_wait(bars + s * 8u, (n_last / n_slots) & 1u, a.poll_limit);
    }
  }
}

}  // namespace

// ---- host side --------------------------------------------------------------------------------------
struct ks_flow {
  MegaArgs args{};
  void* d_tables = nullptr;
  unsigned* d_sync = nullptr;     // word 0: the tag epoch
  long long* d_prof = nullptr;
  long long* d_prof_all = nullptr;
  u64* d_ll = nullptr;            // the tagged activation vectors
  size_t ll_bytes = 0;
  unsigned grid = 0;
  size_t smem = 0;
  int dpl = 0, pc = 1;            // pc: 4-element chunks of the hidden vector per thread
  float* residual = nullptr;      // buffer that holds the residual stream when the kernel ends
};

namespace {
template <int DPL, int PC>
int mega_launch_t(ks_ctx* ctx, ks_flow* mg) {
  auto kern = flow_kernel<DPL, PC>;
  static size_t smem_set[16] = {0};
  if (mg->smem > smem_set[ctx->device & 15]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mg->smem);
    if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "decode kernel: cannot set %zu B shared memory: %s", mg->smem, cudaGetErrorString(e));
    smem_set[ctx->device & 15] = mg->smem;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(mg->grid);
  cfg.blockDim = dim3(MG_THREADS);
  cfg.dynamicSmemBytes = mg->smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // every block resident: blocks wait for each other's rows
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, mg->args);
  if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "decode kernel launch failed: %s", cudaGetErrorString(e));
  return ks_after_launch(ctx, "decode_layers");
}
}  // namespace

int ks_flow_launch(ks_ctx* ctx, ks_flow* mg) {
  if (mg->dpl == 4) {
    switch (mg->pc) {
      case 1: return mega_launch_t<4, 1>(ctx, mg);
      case 2: return mega_launch_t<4, 2>(ctx, mg);
      case 3: return mega_launch_t<4, 3>(ctx, mg);
      case 4: return mega_launch_t<4, 4>(ctx, mg);
    }
  } else if (mg->dpl == 8) {
    switch (mg->pc) {
      case 1: return mega_launch_t<8, 1>(ctx, mg);
      case 2: return mega_launch_t<8, 2>(ctx, mg);
      case 3: return mega_launch_t<8, 3>(ctx, mg);
      case 4: return mega_launch_t<8, 4>(ctx, mg);
    }
  }
  return ks_fail(ctx, KS_ERR_UNSUPPORTED, "decode kernel: head size or hidden size not supported");
}

float* ks_flow_residual(const ks_flow* mg) { return mg->residual; }

// After a wait gave up the tagged vectors hold a mix of tokens; clearing them (tag 0 is never used)
// puts the kernel back in working order.  The epoch word keeps counting.  Stream-ordered.
int ks_flow_reset(ks_ctx* ctx, ks_flow* mg) {
  cudaError_t e = cudaMemsetAsync(mg->d_ll, 0, mg->ll_bytes, ctx->stream);
  if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "decode kernel: reset failed: %s", cudaGetErrorString(e));
  return KS_OK;
}
const long long* ks_flow_prof(const ks_flow* mg) { return mg->d_prof; }
const long long* ks_flow_prof_all(const ks_flow* mg) { return mg->d_prof_all; }

// Knobs that tests and the profiling reader set: 0 = polls before a wait gives up, 1 = make the gate-up stage
// of every layer wait for a tag nobody writes (0 = off), 2 = context length from which attention is split
// across blocks, 3 = record phase clocks (0 / 1).  The caller re-captures its graphs afterwards.
int ks_flow_set(ks_flow* mg, int what, unsigned value) {
  if (!mg) return KS_ERR_INVALID;
  switch (what) {
    case 0: mg->args.poll_limit = value ? value : 1u; return KS_OK;
    case 1: mg->args.test_stall = value; return KS_OK;
    case 2: mg->args.split_from = value; return KS_OK;
    case 3: mg->args.prof = value ? mg->d_prof : nullptr; mg->args.prof_all = value > 1 ? mg->d_prof_all : nullptr; return KS_OK;
    default: return KS_ERR_INVALID;
  }
}

void ks_flow_destroy(ks_flow* mg) {
  if (!mg) return;
  if (mg->d_tables) cudaFree(mg->d_tables);
  if (mg->d_sync) cudaFree(mg->d_sync);
  if (mg->d_prof) cudaFree(mg->d_prof);
  if (mg->d_prof_all) cudaFree(mg->d_prof_all);
  if (mg->d_ll) cudaFree(mg->d_ll);
  delete mg;
}

// Returns KS_OK and *out == nullptr when the shape is outside what the kernel covers (the caller keeps
// the launch-per-op path), a negative code on a CUDA failure.
int ks_flow_create(ks_ctx* ctx, const ks_mega_desc* d, const ks_mega_layer* layers, ks_flow** out) {
  *out = nullptr;
  const unsigned H = d->hidden, F = d->ffn, hd = d->hd, nq = d->n_q, nkv = d->n_kv;
  const unsigned qn = nq * hd, kvn = nkv * hd;
  if (H % 256u || F % 256u || qn % 256u) return KS_OK;
  if (H > 4u * 4u * MG_THREADS) return KS_OK;  // the norm stages hold at most four 4-element chunks per thread
  if (nq % nkv || !(hd == 128 || hd == 256)) return KS_OK;
  const unsigned grid = (unsigned)ctx->sm_count;
  // one block per (query head, split): fewer splits than the caller's record layout allows if the grid is small
  unsigned n_splits = (unsigned)d->n_splits;
  if (n_splits > grid / nq) n_splits = grid / nq;
  if (n_splits > (unsigned)MG_MAX_SPLITS) n_splits = MG_MAX_SPLITS;
  if (n_splits < 1) return KS_OK;
  if (d->n_layers < 1 || d->n_layers > 128) return KS_OK;

  const unsigned shapes_bytes = (unsigned)((PH_KINDS * sizeof(MegaPhase) + 15u) & ~15u);
  const unsigned tables_bytes = (unsigned)((shapes_bytes + d->n_layers * sizeof(MegaLayer) + 15u) & ~15u);
  unsigned maxcols = H > F ? H : F;
  if (qn > maxcols) maxcols = qn;
  unsigned x_bytes = (maxcols / 64u) * 256u;
  if (mg_att_bytes(hd) > x_bytes) x_bytes = mg_att_bytes(hd);

  std::vector<unsigned char> tab(tables_bytes, 0);
  MegaPhase* ph = reinterpret_cast<MegaPhase*>(tab.data());
  MegaLayer* ly = reinterpret_cast<MegaLayer*>(tab.data() + shapes_bytes);
  auto set_phase = [&](MegaPhase& p, unsigned n_seg, const unsigned* rows, unsigned mats, unsigned widx, unsigned cols) {
    p.n_seg = n_seg;
    p.mats = mats;
    p.seg_start[0] = 0;
    for (unsigned s = 0; s < n_seg; s++) p.seg_start[s + 1] = p.seg_start[s] + rows[s];
    p.widx = widx;
    p.cols = cols;
    p.row_bytes = cols / 256u * KS_Q4K_BLOCK_BYTES;
  };
  const unsigned r_qkv[3] = {qn, kvn, kvn}, r_h[1] = {H}, r_f[1] = {F};
  set_phase(ph[PH_QKV], 3, r_qkv, 1, 0, H);
  set_phase(ph[PH_OPROJ], 1, r_h, 1, 3, qn);
  set_phase(ph[PH_GATEUP], 1, r_f, 2, 4, H);
  set_phase(ph[PH_DOWN], 1, r_h, 1, 6, F);
  for (int k = 0; k < PH_KINDS; k++)
    if (ph[k].seg_start[ph[k].n_seg] % 4u || ph[k].seg_start[1] % 4u) return KS_OK;

  // ring: as many slots as give every phase room for at least one 4-row group (x 2 matrices for gate-up)
  const unsigned budget = (unsigned)ctx->smem_optin;
  unsigned need = 0;
  for (int k = 0; k < PH_KINDS; k++) need = std::max(need, 4u * ph[k].mats * ph[k].row_bytes);
  int n_slots = 8;
  if (const char* e = getenv("KSEARCH_MEGA_SLOTS")) n_slots = atoi(e);
  if (n_slots > MG_MAXSLOTS) n_slots = MG_MAXSLOTS;
  unsigned slot_bytes = 0;
  for (; n_slots >= 2; n_slots--) {
    const MegaSmem fixed = mg_smem(x_bytes, H, 0, n_slots, tables_bytes);
    if (fixed.total >= budget) continue;
    slot_bytes = ((budget - fixed.total) / (unsigned)n_slots) & ~127u;
    if (slot_bytes >= need) break;
  }
  if (n_slots < 2 || slot_bytes < need) return KS_OK;

  // rows of a phase owned by the fullest block
  auto max_rows = [&](const MegaPhase& p) {
    const unsigned half = p.seg_start[p.n_seg] / 2u;
    unsigned m = 0;
    for (unsigned b = 0; b < grid; b++) {
      const unsigned lo = (unsigned)(((unsigned long long)b * half) / grid) * 2u, hi = (unsigned)(((unsigned long long)(b + 1) * half) / grid) * 2u;
      m = std::max(m, hi - lo);
    }
    return m;
  };
  // Column segments per phase: a lane owns one 64-weight unit of a segment, so a segment has at most 32 units;
  // the units of a row are split evenly over as few segments as that allows.
  unsigned total_pieces = 0;
  for (int k = 0; k < PH_KINDS; k++) {
    MegaPhase& p = ph[k];
    const unsigned R = max_rows(p);
    if (R > (unsigned)MG_MAXROWS || R == 0) return KS_OK;
    // pieces: as few as fit the slot, of equal size
    unsigned cap_rows = (slot_bytes / (p.mats * p.row_bytes)) & ~3u;
    if (cap_rows > 64u) cap_rows = 64u;
    const unsigned n_pc = (R + cap_rows - 1u) / cap_rows;
    p.piece_rows = std::min(cap_rows, (((R + n_pc - 1u) / n_pc) + 3u) & ~3u);
    const unsigned U = p.cols / 64u;
    p.n_cseg = (U + 31u) / 32u;
    if (p.n_cseg > (unsigned)MG_MAXC || U % p.n_cseg) return KS_OK;
    p.seg_units = U / p.n_cseg;
    total_pieces += p.n_seg + (R + p.piece_rows - 1u) / p.piece_rows + 1u;
  }
  if (total_pieces > (unsigned)MG_MAXPIECE) return KS_OK;

  for (int l = 0; l < d->n_layers; l++) {
    const ks_mega_layer& L = layers[l];
    MegaLayer& o = ly[l];
    o.W[0] = (const uint8_t*)L.wq; o.W[1] = (const uint8_t*)L.wk; o.W[2] = (const uint8_t*)L.wv; o.W[3] = (const uint8_t*)L.wo;
    o.W[4] = (const uint8_t*)L.wgate; o.W[5] = (const uint8_t*)L.wup; o.W[6] = (const uint8_t*)L.wdown;
    o.norm[0] = (const float*)L.attn_norm; o.norm[1] = (const float*)L.q_norm; o.norm[2] = (const float*)L.k_norm;
    o.norm[3] = (const float*)L.post_attn_norm; o.norm[4] = (const float*)L.ffn_norm; o.norm[5] = (const float*)L.post_ffw_norm;
    o.kv_k = L.kv_k; o.kv_v = L.kv_v;
  }

  ks_flow* mg = new ks_flow();
  cudaSetDevice(ctx->device);
  const size_t prof_n = (size_t)2 * d->n_layers * PF_PER_LAYER * PF_STAMPS;
  // tagged vectors, two of each: yd, yo [H], qkv [qn + 2 kvn], ox [qn], ff [F], rec [n_q * n_splits * (hd + 2)]
  const size_t n_rec = (size_t)nq * n_splits * (hd + 2);
  auto up2 = [](size_t n) { return (n + 1) & ~size_t(1); };   // keep every vector 16-byte aligned
  const size_t ll_words = 2 * (up2(H) + up2(H) + up2(qn + 2 * kvn) + up2(qn) + up2(F) + up2(n_rec));
  mg->ll_bytes = ll_words * sizeof(u64);
  if (cudaMalloc(&mg->d_tables, tables_bytes) != cudaSuccess || cudaMalloc((void**)&mg->d_sync, 256) != cudaSuccess ||
      cudaMalloc((void**)&mg->d_prof, prof_n * sizeof(long long)) != cudaSuccess ||
      cudaMalloc((void**)&mg->d_prof_all, (size_t)grid * d->n_layers * PF_PER_LAYER * 8 * sizeof(long long)) != cudaSuccess ||
      cudaMalloc((void**)&mg->d_ll, mg->ll_bytes) != cudaSuccess) {
    ks_flow_destroy(mg);
    return ks_fail(ctx, KS_ERR_OOM, "decode kernel: cannot allocate its tables");
  }
  const unsigned epoch0[1] = {1u};
  cudaError_t e = cudaMemcpyAsync(mg->d_tables, tab.data(), tables_bytes, cudaMemcpyHostToDevice, ctx->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(mg->d_sync, 0, 256, ctx->stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(mg->d_sync, epoch0, sizeof epoch0, cudaMemcpyHostToDevice, ctx->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(mg->d_ll, 0, mg->ll_bytes, ctx->stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(mg->d_prof, 0, prof_n * sizeof(long long), ctx->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);  // tab and epoch0 are locals
  if (e != cudaSuccess) {
    ks_flow_destroy(mg);
    return ks_fail(ctx, KS_ERR_CUDA, "decode kernel: table upload failed: %s", cudaGetErrorString(e));
  }
  MegaArgs& a = mg->args;
  a.tables = mg->d_tables;
  a.tables_bytes = tables_bytes;
  a.n_layers = d->n_layers;
  a.n_slots = n_slots;
  a.slot_bytes = slot_bytes;
  a.x_bytes = x_bytes;
  a.n_q = nq; a.n_kv = nkv; a.hd = hd; a.n_splits = n_splits;
  a.split_from = MG_NW * MG_AB;  // one batch of rows per warp
  if (const char* e2 = getenv("KSEARCH_MEGA_SPLIT_FROM")) a.split_from = (unsigned)atoi(e2);
  a.eps = d->eps; a.attn_scale = d->attn_scale;
  a.rope = d->rope; a.pos = d->pos;
  a.x_in = d->x_a;
  a.resid_out = d->x_b;
  a.y_out = d->yb;
  {
    u64* p = mg->d_ll;
    auto take = [&](size_t n) { u64* r = p; p += up2(n); return r; };
    a.ll_yd0 = take(H); a.ll_yd1 = take(H);
    a.ll_yo0 = take(H); a.ll_yo1 = take(H);
    a.ll_qkv0 = take(qn + 2 * kvn); a.ll_qkv1 = take(qn + 2 * kvn);
    a.ll_ox0 = take(qn); a.ll_ox1 = take(qn);
    a.ll_ff0 = take(F); a.ll_ff1 = take(F);
    a.ll_rec0 = take(n_rec); a.ll_rec1 = take(n_rec);
  }
  a.epoch = mg->d_sync;
  a.err = (unsigned*)ctx->ws + KS_WS_ERR_WORD;
  a.poll_limit = 1u << 21;  // a second or two of polling at most
  a.test_stall = 0;
  a.prof = getenv("KSEARCH_PROFILE") ? mg->d_prof : nullptr;
  mg->grid = grid;
  mg->smem = mg_smem(x_bytes, H, slot_bytes, n_slots, tables_bytes).total;
  mg->dpl = (int)(hd / 32);
  mg->pc = (int)((H / 4u + MG_THREADS - 1u) / MG_THREADS);
  mg->residual = d->x_b;
  *out = mg;
  return KS_OK;
}

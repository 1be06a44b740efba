// Decode attention (one query token per slot) over a Q4_0 KV cache, split over
// the context.
//
// Stands in for the reference's two attention lowerings,
//   crates/ksearch_codegen/src/lower.rs:4897-5359  single-pass online softmax (short contexts)
//   crates/ksearch_codegen/src/lower.rs:5367-6088  16-partition pass + LSE merge (tlen >= 128)
// dispatched by Eng::sdpa_hybrid_kv (crates/ksearch_kernels/src/lib.rs:1157-1178).
//
// Layout.  K and V: [max_t, n_kv, hd] in Q4_0 (18-byte blocks of 32 values), per
// slot.  One block of the grid handles (split, kv head, slot); its warps take
// the positions of the split round-robin.  A warp serves ALL query heads of the
// KV head's group from one read of the K/V row: lane L owns the dims that live
// in bytes [ (L % LPB)*BPL, +BPL ) of Q4_0 block L / LPB (low nibbles = dims i,
// high nibbles = dims i+16), so a row is read once, 2 bytes at a time, and is
// never dequantised to memory.  Running (m, l, O) per head stay in registers;
// warps are merged through shared memory, splits through `tmp` with the
// reference's (m, l, O[hd]) record layout, stride hd+2, m initialised to -1e30.
#include <cstdlib>

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

constexpr int kWarps = 4;
constexpr float kNegInit = -1.0e30f;

// Load this lane's DPL values of one Q4_0 row: dims (lo nibbles) then dims+16 (hi nibbles).
template <int DPL>
__device__ __forceinline__ void load_row(const uint8_t* row, int lane, float (&out)[DPL]) {
  constexpr int BPL = DPL / 2;        // bytes per lane
  constexpr int LPB = 16 / BPL;       // lanes per 32-value block
  const uint8_t* blk = row + (lane / LPB) * KS_Q40_BLOCK_BYTES;
  const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(blk)));
  const unsigned short* qs = reinterpret_cast<const unsigned short*>(blk + 2 + (lane % LPB) * BPL);
#pragma unroll
  for (int w = 0; w < BPL / 2; w++) {
    const unsigned v = qs[w];
    out[2 * w] = (float)((int)(v & 0xF) - 8) * d;
    out[2 * w + 1] = (float)((int)((v >> 8) & 0xF) - 8) * d;
    out[BPL + 2 * w] = (float)((int)((v >> 4) & 0xF) - 8) * d;
    out[BPL + 2 * w + 1] = (float)((int)(v >> 12) - 8) * d;
  }
}
// The same DPL values as plain nibbles (0..15 as floats) and the block's scale: the -8 offset and the scale are
// applied once per (row, head) by the caller instead of once per value.
template <int DPL>
__device__ __forceinline__ float load_row_raw(const uint8_t* row, int lane, float (&out)[DPL]) {
  constexpr int BPL = DPL / 2;
  constexpr int LPB = 16 / BPL;
  const uint8_t* blk = row + (lane / LPB) * KS_Q40_BLOCK_BYTES;
  const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(blk)));
  const unsigned short* qs = reinterpret_cast<const unsigned short*>(blk + 2 + (lane % LPB) * BPL);
#pragma unroll
  for (int w = 0; w < BPL / 2; w++) {
    const unsigned v = qs[w];
    out[2 * w] = (float)(v & 0xF);
    out[2 * w + 1] = (float)((v >> 8) & 0xF);
    out[BPL + 2 * w] = (float)((v >> 4) & 0xF);
    out[BPL + 2 * w + 1] = (float)(v >> 12);
  }
  return d;
}
// Sum over the warp of G values per lane; every lane gets all G sums.  G == 4: the lanes first trade halves
// (each keeps two, then one, of the four values), so 10 shuffles do what 20 would.
template <int G>
__device__ __forceinline__ void warp_sum_g(float (&s)[G], int lane) {
  if (G == 4) {
    const bool hi = (lane & 16) != 0, h8 = (lane & 8) != 0;
    float k0 = hi ? s[2] : s[0], k1 = hi ? s[3] : s[1];
    const float t0 = hi ? s[0] : s[2], t1 = hi ? s[1] : s[3];
    k0 += __shfl_xor_sync(0xffffffffu, t0, 16);
    k1 += __shfl_xor_sync(0xffffffffu, t1, 16);
    float k = h8 ? k1 : k0;
    const float t = h8 ? k0 : k1;
    k += __shfl_xor_sync(0xffffffffu, t, 8);
    k += __shfl_xor_sync(0xffffffffu, k, 4);
    k += __shfl_xor_sync(0xffffffffu, k, 2);
    k += __shfl_xor_sync(0xffffffffu, k, 1);
#pragma unroll
    for (int g = 0; g < G; g++) s[g] = __shfl_sync(0xffffffffu, k, 8 * (g & 1) + 16 * (g >> 1));
  } else {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
#pragma unroll
      for (int g = 0; g < G; g++) s[g] += __shfl_xor_sync(0xffffffffu, s[g], off);
  }
}
// Dimension index (within the head) of this lane's j-th value.
template <int DPL>
__device__ __forceinline__ int lane_dim(int lane, int j) {
  constexpr int BPL = DPL / 2;
  constexpr int LPB = 16 / BPL;
  const int base = (lane / LPB) * 32 + (lane % LPB) * BPL;
  return j < BPL ? base + j : base + 16 + (j - BPL);
}

constexpr int kRing = 8;  // rows of one warp in flight (K and V each)

__device__ __forceinline__ void cp_async8(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}

// ASYNC: the rows of a warp travel through a ring of kRing shared-memory buffers filled by cp.async (8 bytes per
// lane), so kRing rows of K and V are in flight per warp while one is being multiplied; without it a warp waited
// out one full memory round trip per row.  Needs 8-byte aligned rows; the plain path takes the rest.
// G: query heads served by one block (at most 4: more would not leave registers for enough warps per SM); a KV head
// with a larger group is served by hpk / G blocks (blockIdx.y = kvh * (hpk / G) + group), each reading the rows itself.
template <int G, int DPL, typename T, bool ASYNC>
__global__ void __launch_bounds__(kWarps * 32)
sdpa_part_kernel(unsigned n_q, unsigned n_kv, float scale, const T* q, const uint8_t* K, const uint8_t* V,
                 size_t slot_stride, const float* meta, float* tmp, T* out, int n_splits) {
  ks_pdl_entry();
  constexpr int HD = DPL * 32;
  constexpr unsigned ROWB = (HD / 32) * KS_Q40_BLOCK_BYTES;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned hpk = n_q / n_kv, gpk = hpk / G;  // heads and blocks per KV head
  const int split = blockIdx.x, kvh = blockIdx.y / gpk, slot = blockIdx.z;
  const unsigned head0 = (unsigned)kvh * hpk + (blockIdx.y % gpk) * G;  // first query head of this block
  const unsigned tlen = (unsigned)meta[slot * 4 + 0];
  const unsigned start = (unsigned)meta[slot * 4 + 1];
  const unsigned chunk = (tlen + n_splits - 1) / n_splits;
  const unsigned p0 = split * chunk;
  const unsigned p1 = min(p0 + chunk, tlen);
  const size_t rowb = ROWB;
  const uint8_t* Ks = K + (size_t)slot * slot_stride;
  const uint8_t* Vs = V + (size_t)slot * slot_stride;
  __shared__ __align__(16) uint8_t ring[ASYNC ? kWarps * kRing * 2 * ROWB : 16];

  // qs8[g] = 8 * (sum of this lane's q values): the -8 of Q4_0 leaves the dot product as one term per (row, head);
  // c[g] gathers sum(e * d) the same way for V, and is taken off o at the end
  float qr[G][DPL], o[G][DPL], m[G], l[G], qs8[G], c[G];
#pragma unroll
  for (int g = 0; g < G; g++) {
    const size_t qb = ((size_t)slot * n_q + head0 + g) * HD;
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < DPL; j++) {
      qr[g][j] = ld_act<T>(q, qb + lane_dim<DPL>(lane, j)) * scale;
      sum += qr[g][j];
      o[g][j] = 0.0f;
    }
    qs8[g] = 8.0f * sum;
    c[g] = 0.0f;
    m[g] = kNegInit;
    l[g] = 0.0f;
  }

  // one position: scores of the G heads against the K row, then the online-softmax update with the V row
  auto step = [&](const uint8_t* krow, const uint8_t* vrow) {
    float kv[DPL];
    const float dk = load_row_raw<DPL>(krow, lane, kv);
    float s[G];
#pragma unroll
    for (int g = 0; g < G; g++) {
      float a = -qs8[g];
#pragma unroll
      for (int j = 0; j < DPL; j++) a = fmaf(qr[g][j], kv[j], a);
      s[g] = a * dk;
    }
    warp_sum_g<G>(s, lane);
    const float dv = load_row_raw<DPL>(vrow, lane, kv);
#pragma unroll
    for (int g = 0; g < G; g++) {
      if (s[g] > m[g]) {  // a new maximum (the same in every lane): rescale what was gathered so far
        const float alpha = __expf(m[g] - s[g]);
        l[g] *= alpha;
        c[g] *= alpha;
#pragma unroll
        for (int j = 0; j < DPL; j++) o[g][j] *= alpha;
        m[g] = s[g];
      }
      const float e = __expf(s[g] - m[g]);
      l[g] += e;
      const float ed = e * dv;
      c[g] += ed;
#pragma unroll
      for (int j = 0; j < DPL; j++) o[g][j] = fmaf(ed, kv[j], o[g][j]);
    }
  };

  if (ASYNC) {
    uint8_t* my = ring + (size_t)warp * (kRing * 2 * ROWB);
    const uint32_t my_s = (uint32_t)__cvta_generic_to_shared(my);
    auto fetch = [&](unsigned n) {  // the warp's n-th position into buffer n % kRing (an empty group past the end)
      const unsigned t = p0 + (unsigned)warp + n * kWarps;
      if (t < p1 && lane < (int)(ROWB / 8u)) {
        const size_t row = ((size_t)(start + t) * n_kv + kvh) * rowb + (size_t)lane * 8u;
        const uint32_t dst = my_s + (n % kRing) * (2u * ROWB) + (uint32_t)lane * 8u;
        cp_async8(dst, Ks + row);
        cp_async8(dst + ROWB, Vs + row);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll 1
    for (unsigned n = 0; n < (unsigned)kRing; n++) fetch(n);
    unsigned n = 0;
#pragma unroll 1
    for (unsigned t = p0 + warp; t < p1; t += kWarps, n++) {
      asm volatile("cp.async.wait_group %0;" ::"n"(kRing - 1) : "memory");
      __syncwarp();
      const uint8_t* buf = my + (size_t)(n % kRing) * (2u * ROWB);
      step(buf, buf + ROWB);
      __syncwarp();  // every lane is done with the buffer before it is refilled
      fetch(n + kRing);
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else {
    for (unsigned t = p0 + warp; t < p1; t += kWarps) {
      const size_t row = ((size_t)(start + t) * n_kv + kvh) * rowb;
      step(Ks + row, Vs + row);
    }
  }

#pragma unroll
  for (int g = 0; g < G; g++)
#pragma unroll
    for (int j = 0; j < DPL; j++) o[g][j] = fmaf(-8.0f, c[g], o[g][j]);

  // merge the warps of this block: warp w leaves (m, l, O) in shared memory, warp 0 folds them in order
  __shared__ float sm_ml[kWarps][G][2];
  __shared__ float sm_o[kWarps][G][HD];
  if (warp > 0) {
#pragma unroll
    for (int g = 0; g < G; g++) {
      if (lane == 0) {
        sm_ml[warp][g][0] = m[g];
        sm_ml[warp][g][1] = l[g];
      }
#pragma unroll
      for (int j = 0; j < DPL; j++) sm_o[warp][g][j * 32 + lane] = o[g][j];
    }
  }
  __syncthreads();
  if (warp != 0) return;
#pragma unroll
  for (int g = 0; g < G; g++) {
    for (int w = 1; w < kWarps; w++) {
      const float mp = sm_ml[w][g][0], lp = sm_ml[w][g][1];
      const float m2 = fmaxf(m[g], mp);
      const float alpha = __expf(m[g] - m2), beta = __expf(mp - m2);
      l[g] = l[g] * alpha + lp * beta;
      m[g] = m2;
#pragma unroll
      for (int j = 0; j < DPL; j++) o[g][j] = o[g][j] * alpha + sm_o[w][g][j * 32 + lane] * beta;
    }
    const unsigned head = head0 + g;
    if (n_splits == 1) {
      const float inv_l = 1.0f / l[g];
      const size_t ob = ((size_t)slot * n_q + head) * HD;
#pragma unroll
      for (int j = 0; j < DPL; j++) st_act<T>(out, ob + lane_dim<DPL>(lane, j), o[g][j] * inv_l);
    } else {
      float* rec = tmp + (((size_t)slot * n_q + head) * n_splits + split) * (HD + 2);
      if (lane == 0) {
        rec[0] = m[g];
        rec[1] = l[g];
      }
#pragma unroll
      for (int j = 0; j < DPL; j++) rec[2 + lane_dim<DPL>(lane, j)] = o[g][j];
    }
  }
}

// Merge the per-split records of one (slot, head): lower.rs:5897-6088.  The (m, l) pairs go through shared
// memory; 1024 / hd groups of threads share the splits, thread (group, d) adds O[d] of its splits eight loads at a
// time, and the groups' sums meet in shared memory in a fixed order.
template <typename T>
__global__ void __launch_bounds__(1024) sdpa_reduce_kernel(unsigned hd, const float* tmp, T* out, int n_splits) {
  ks_pdl_entry();
  __shared__ float sm[2 * KS_SDPA_MAX_SPLITS];
  __shared__ float part[1024];
  const size_t sh = blockIdx.x;  // slot * n_q + head
  const float* rec0 = tmp + sh * n_splits * (hd + 2);
  for (int p = threadIdx.x; p < n_splits; p += blockDim.x) {
    sm[2 * p] = rec0[(size_t)p * (hd + 2)];
    sm[2 * p + 1] = rec0[(size_t)p * (hd + 2) + 1];
  }
  __syncthreads();
  float M = kNegInit;
  for (int p = 0; p < n_splits; p++) M = fmaxf(M, sm[2 * p]);
  float L = 0.0f;
  for (int p = 0; p < n_splits; p++) L = fmaf(sm[2 * p + 1], __expf(sm[2 * p] - M), L);
  // thread (group, d): the splits p = group, group + groups, ... of dimension d, eight loads in flight at a time
  const unsigned groups = blockDim.x / hd, grp = threadIdx.x / hd, d = threadIdx.x % hd;
  float o = 0.0f;
  if (grp < groups) {
    for (int pb = (int)grp; pb < n_splits; pb += 8 * (int)groups) {
      float v[8];
#pragma unroll
      for (int k = 0; k < 8; k++) {  // an empty split (l = 0) left no O behind
        const int p = pb + k * (int)groups;
        v[k] = (p < n_splits && sm[2 * p + 1] != 0.0f) ? rec0[(size_t)p * (hd + 2) + 2 + d] : 0.0f;
      }
#pragma unroll
      for (int k = 0; k < 8; k++) {
        const int p = pb + k * (int)groups;
        if (p < n_splits) o = fmaf(v[k], __expf(sm[2 * p] - M), o);
      }
    }
    part[threadIdx.x] = o;
  }
  __syncthreads();
  if (threadIdx.x < hd) {
    float a = 0.0f;
    for (unsigned g2 = 0; g2 < groups; g2++) a += part[g2 * hd + threadIdx.x];  // fixed order
    st_act<T>(out, sh * hd + threadIdx.x, a / L);
  }
}

// ---- the tiled form: positions across lanes for q.k, dims across lanes for p.v ------------------------------
// One block of 256 threads per (split, KV head, slot) serves the query heads of the KV head (up to four; a group of
// eight is two blocks).  The split's rows come
// into shared memory 256 positions at a time (cp.async, 4 bytes per request, row stride ROWB + 4 bytes so that 32
// lanes reading 32 different rows hit 32 different banks).
//   scores   thread t owns position t of the tile: it walks its K row two Q4_0 blocks (nine words) at a time and
//            multiplies the 64 nibbles against q of every head (q and the per-block 8 * sum(q) sit in shared memory,
//            read as broadcasts) -- no shuffle, and the row is decoded once for all heads;
//   softmax  warp g owns head g: tile maximum, rescale factor of what was gathered before, probabilities in place;
//   values   lane L owns the dims of its nibbles (as in the per-row kernel above), the eight warps take positions
//            round-robin, the probabilities are shared-memory broadcasts.
// Per position and head this costs ~25 warp instructions where the per-row kernel needs ~70 (it pays five shuffles
// and an exp chain per row and head).  Records and the merge kernel are the same.
constexpr int kTP = 256;
constexpr int kMinChunk = 128;

__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

template <int G, int HD>
struct TileSmem {
  static constexpr unsigned ROWB = (HD / 32) * KS_Q40_BLOCK_BYTES, RP = ROWB + 4, NW = ROWB / 4, NB = HD / 32;
  static constexpr unsigned q_off = 0;                         // G * HD floats
  static constexpr unsigned st_off = q_off + G * HD * 4;       // m[G], l[G], alpha[G]
  static constexpr unsigned s_off = st_off + 3 * 8 * 4;        // G * kTP floats: scores, then probabilities
  static constexpr unsigned k_off = s_off + G * kTP * 4;       // kTP rows of K, then of V
  static constexpr unsigned v_off = k_off + kTP * RP;
  static constexpr unsigned tiles = 2 * kTP * RP, merge = 8 * G * HD * 4;  // the warps' partial O reuse the tiles
  static constexpr unsigned total = k_off + (tiles > merge ? tiles : merge);
};

template <int G, int HD, typename T>
__global__ void __launch_bounds__(kTP, 2)
sdpa_tile_kernel(unsigned n_q, unsigned n_kv, float scale, const T* q, const uint8_t* K, const uint8_t* V, size_t slot_stride,
                 const float* meta, float* tmp, T* out, int n_splits) {
  ks_pdl_entry();
  using S = TileSmem<G, HD>;
  constexpr int DPL = HD / 32;
  constexpr unsigned ROWB = S::ROWB, RP = S::RP, NW = S::NW, NB = S::NB;
  extern __shared__ __align__(16) unsigned char smem[];
  float* sq = reinterpret_cast<float*>(smem + S::q_off);
  float* sst = reinterpret_cast<float*>(smem + S::st_off);
  float* ss = reinterpret_cast<float*>(smem + S::s_off);
  unsigned char* kt = smem + S::k_off;
  unsigned char* vt = smem + S::v_off;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned hpk = n_q / n_kv, gpk = hpk / G;  // heads and blocks per KV head
  const int split = blockIdx.x, kvh = blockIdx.y / gpk, slot = blockIdx.z;
  const unsigned head0 = (unsigned)kvh * hpk + (blockIdx.y % gpk) * G;
  const unsigned tlen = (unsigned)meta[slot * 4 + 0], start = (unsigned)meta[slot * 4 + 1];
  // a split never holds fewer than kMinChunk positions: on a short context the later splits are empty and their
  // blocks leave after writing an empty record, so a split count sized for the longest context costs little
  const unsigned chunk = max((tlen + n_splits - 1) / n_splits, (unsigned)kMinChunk);
  const unsigned p0 = split * chunk, p1 = min(p0 + chunk, tlen);
  const uint8_t* Ks = K + (size_t)slot * slot_stride;
  const uint8_t* Vs = V + (size_t)slot * slot_stride;

  if (p0 >= p1 && n_splits > 1) {  // nothing to do: the empty record (m = -1e30, l = 0) is all the merge needs
    if (tid < G) {
      float* rec = tmp + (((size_t)slot * n_q + head0 + tid) * n_splits + split) * (HD + 2);
      rec[0] = kNegInit;
      rec[1] = 0.0f;
    }
    return;
  }
  for (int i = tid; i < G * HD; i += kTP) sq[i] = ld_act<T>(q, ((size_t)slot * n_q + head0) * HD + i) * scale;
  if (tid < 3 * 8) sst[tid] = tid < 8 ? kNegInit : 0.0f;
  __syncthreads();
  float o[G][DPL], c[G];
#pragma unroll
  for (int g = 0; g < G; g++) {
    c[g] = 0.0f;
#pragma unroll
    for (int j = 0; j < DPL; j++) o[g][j] = 0.0f;
  }
  const uint32_t kt_s = (uint32_t)__cvta_generic_to_shared(kt), vt_s = (uint32_t)__cvta_generic_to_shared(vt);

  for (unsigned t0 = p0; t0 < p1; t0 += kTP) {
    const unsigned n = min((unsigned)kTP, p1 - t0);
    __syncthreads();  // the previous tile is used up
    for (unsigned r = warp; r < n; r += kTP / 32) {  // a warp per row: lane = word, the first lanes take the tail
      const size_t src = ((size_t)(start + t0 + r) * n_kv + kvh) * ROWB + 4u * lane;
      const uint32_t dst = r * RP + 4u * lane;
      if ((unsigned)lane < NW) {
        cp_async4(kt_s + dst, Ks + src);
        cp_async4(vt_s + dst, Vs + src);
      }
      if (NW > 32 && (unsigned)lane + 32u < NW) {
        cp_async4(kt_s + dst + 128u, Ks + src + 128u);
        cp_async4(vt_s + dst + 128u, Vs + src + 128u);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    // ---- scores: thread = position; a short tile spreads the block pairs of a row over 2 or 4 neighbouring lanes
    const unsigned wshift = (n * 4u <= (unsigned)kTP && NB >= 8u) ? 2u : (n * 2u <= (unsigned)kTP && NB >= 4u) ? 1u : 0u;
    const unsigned pos_t = (unsigned)tid >> wshift, part = (unsigned)tid & ((1u << wshift) - 1u);
    {
      const uint32_t* kr = reinterpret_cast<const uint32_t*>(kt + (size_t)(pos_t < n ? pos_t : 0u) * RP);
      float sc[G];
#pragma unroll
      for (int g = 0; g < G; g++) sc[g] = 0.0f;
#pragma unroll 1
      for (unsigned pb = part; pb < NB / 2; pb += 1u << wshift) {
        uint32_t w[9];
#pragma unroll
        for (int i = 0; i < 9; i++) w[i] = kr[9 * pb + i];
        // two blocks of 18 bytes: [d0 | 16 nibble bytes][d1 | 16 nibble bytes]; the first one's bytes straddle the words
        uint32_t qw[2][4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
          qw[0][i] = __funnelshift_r(w[i], w[i + 1], 16);
          qw[1][i] = w[5 + i];
        }
        const float d01[2] = {__half2float(__ushort_as_half((unsigned short)(w[0] & 0xFFFFu))),
                              __half2float(__ushort_as_half((unsigned short)(w[4] >> 16)))};
#pragma unroll
        for (int b = 0; b < 2; b++) {
          float lo[16], hi[16];  // dims 0..15 and 16..31 of the block
#pragma unroll
          for (int i = 0; i < 4; i++)
#pragma unroll
            for (int k = 0; k < 4; k++) {
              // 2^23 + n as a float, minus (2^23 + 8): the signed nibble without an int-to-float conversion
              lo[4 * i + k] = __uint_as_float(((qw[b][i] >> (8 * k)) & 0xFu) | 0x4B000000u) - 8388616.0f;
              hi[4 * i + k] = __uint_as_float(((qw[b][i] >> (8 * k + 4)) & 0xFu) | 0x4B000000u) - 8388616.0f;
            }
          const unsigned blk = 2 * pb + b;
#pragma unroll
          for (int g = 0; g < G; g++) {
            const float4* q4 = reinterpret_cast<const float4*>(sq + (size_t)g * HD + blk * 32);
            float a = 0.0f;
#pragma unroll
            for (int i = 0; i < 4; i++) {
              const float4 ql = q4[i], qh = q4[4 + i];
              a = fmaf(ql.x, lo[4 * i], a); a = fmaf(ql.y, lo[4 * i + 1], a); a = fmaf(ql.z, lo[4 * i + 2], a); a = fmaf(ql.w, lo[4 * i + 3], a);
              a = fmaf(qh.x, hi[4 * i], a); a = fmaf(qh.y, hi[4 * i + 1], a); a = fmaf(qh.z, hi[4 * i + 2], a); a = fmaf(qh.w, hi[4 * i + 3], a);
            }
            sc[g] = fmaf(a, d01[b], sc[g]);
          }
        }
      }
      for (unsigned off = (1u << wshift) >> 1; off > 0; off >>= 1)
#pragma unroll
        for (int g = 0; g < G; g++) sc[g] += __shfl_xor_sync(0xffffffffu, sc[g], off);
      if (pos_t < n && part == 0) {
#pragma unroll
        for (int g = 0; g < G; g++) ss[g * kTP + pos_t] = sc[g];
      }
    }
    __syncthreads();
    // ---- softmax of the tile: warp = head
    if (warp < G) {
      float* sg = ss + warp * kTP;
      float mx = kNegInit;
      for (unsigned i = lane; i < n; i += 32) mx = fmaxf(mx, sg[i]);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const float m_old = sst[warp], m_new = fmaxf(m_old, mx);
      float sum = 0.0f;
      for (unsigned i = lane; i < n; i += 32) {
        const float e = __expf(sg[i] - m_new);
        sg[i] = e;
        sum += e;
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      if (lane == 0) {
        const float alpha = __expf(m_old - m_new);
        sst[warp] = m_new;
        sst[8 + warp] = sst[8 + warp] * alpha + sum;
        sst[16 + warp] = alpha;
      }
    }
    __syncthreads();
    // ---- values: lane = dims, warps take positions round-robin
#pragma unroll
    for (int g = 0; g < G; g++) {
      const float alpha = sst[16 + g];
      c[g] *= alpha;
#pragma unroll
      for (int j = 0; j < DPL; j++) o[g][j] *= alpha;
    }
    for (unsigned pos = warp; pos < n; pos += kTP / 32) {
      float vv[DPL];
      const float dv = load_row_raw<DPL>(vt + (size_t)pos * RP, lane, vv);
#pragma unroll
      for (int g = 0; g < G; g++) {
        const float ed = ss[g * kTP + pos] * dv;
        c[g] += ed;
#pragma unroll
        for (int j = 0; j < DPL; j++) o[g][j] = fmaf(ed, vv[j], o[g][j]);
      }
    }
  }
  __syncthreads();  // tiles are free: the warps' partial O meet there
  float* mo = reinterpret_cast<float*>(kt);  // [warp][g][dim]
#pragma unroll
  for (int g = 0; g < G; g++)
#pragma unroll
    for (int j = 0; j < DPL; j++) mo[((size_t)warp * G + g) * HD + lane_dim<DPL>(lane, j)] = fmaf(-8.0f, c[g], o[g][j]);
  __syncthreads();
  for (int i = tid; i < G * HD; i += kTP) {
    const int g = i / HD, d = i - g * HD;
    float a = 0.0f;
#pragma unroll
    for (int w = 0; w < kTP / 32; w++) a += mo[((size_t)w * G + g) * HD + d];
    const unsigned head = head0 + g;
    if (n_splits == 1) {
      st_act<T>(out, ((size_t)slot * n_q + head) * HD + d, a / sst[8 + g]);
    } else {
      float* rec = tmp + (((size_t)slot * n_q + head) * n_splits + split) * (HD + 2);
      if (d == 0) {
        rec[0] = sst[g];
        rec[1] = sst[8 + g];
      }
      rec[2 + d] = a;
    }
  }
}

template <int G, int HD, typename T>
int launch_tile(ks_ctx* ctx, dim3 grid, unsigned n_q, unsigned n_kv, float scale, const void* q, const uint8_t* K, const uint8_t* V,
                size_t slot_stride, const float* meta, float* tmp, void* out, int n_splits) {
  auto kern = sdpa_tile_kernel<G, HD, T>;
  constexpr size_t smem = TileSmem<G, HD>::total;
  static bool set[16] = {false};
  if (!set[ctx->device & 15]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "sdpa: cannot set %zu B shared memory: %s", smem, cudaGetErrorString(e));
    set[ctx->device & 15] = true;
  }
  KS_LAUNCH(ctx, kern, grid, kTP, smem, n_q, n_kv, scale, (const T*)q, K, V, slot_stride, meta, tmp, (T*)out, n_splits);
  return ks_after_launch(ctx, "sdpa_tile");
}
template <int HD, typename T>
int launch_tile_g(ks_ctx* ctx, int G, dim3 grid, unsigned n_q, unsigned n_kv, float scale, const void* q, const uint8_t* K,
                  const uint8_t* V, size_t slot_stride, const float* meta, float* tmp, void* out, int n_splits) {
  switch (G) {
    case 1: return launch_tile<1, HD, T>(ctx, grid, n_q, n_kv, scale, q, K, V, slot_stride, meta, tmp, out, n_splits);
    case 2: return launch_tile<2, HD, T>(ctx, grid, n_q, n_kv, scale, q, K, V, slot_stride, meta, tmp, out, n_splits);
    case 4: return launch_tile<4, HD, T>(ctx, grid, n_q, n_kv, scale, q, K, V, slot_stride, meta, tmp, out, n_splits);
    case 8:  // four heads per block, two blocks per KV head: no register spills, and twice the blocks
      grid.y *= 2;
      return launch_tile<4, HD, T>(ctx, grid, n_q, n_kv, scale, q, K, V, slot_stride, meta, tmp, out, n_splits);
  }
  return 1;
}

template <int G, int DPL, typename T>
int launch_part(ks_ctx* ctx, dim3 grid, unsigned n_q, unsigned n_kv, float scale, const void* q, const uint8_t* K,
                const uint8_t* V, size_t slot_stride, const float* meta, float* tmp, void* out, int n_splits) {
  const bool aligned = (((uintptr_t)K | (uintptr_t)V | (uintptr_t)slot_stride) & 7u) == 0;
  if (aligned)
    KS_LAUNCH(ctx, (sdpa_part_kernel<G, DPL, T, true>), grid, kWarps * 32, 0, n_q, n_kv, scale, (const T*)q, K, V, slot_stride, meta,
              tmp, (T*)out, n_splits);
  else
    KS_LAUNCH(ctx, (sdpa_part_kernel<G, DPL, T, false>), grid, kWarps * 32, 0, n_q, n_kv, scale, (const T*)q, K, V, slot_stride,
              meta, tmp, (T*)out, n_splits);
  return ks_after_launch(ctx, "sdpa_part");
}

template <int DPL, typename T>
int launch_part_g(ks_ctx* ctx, int G, dim3 grid, unsigned n_q, unsigned n_kv, float scale, const void* q, const uint8_t* K,
                  const uint8_t* V, size_t slot_stride, const float* meta, float* tmp, void* out, int n_splits) {
  switch (G) {
    case 1: return launch_part<1, DPL, T>(ctx, grid, n_q, n_kv, scale, q, K, V, slot_stride, meta, tmp, out, n_splits);
    case 2: return launch_part<2, DPL, T>(ctx, grid, n_q, n_kv, scale, q, K, V, slot_stride, meta, tmp, out, n_splits);
    case 4: return launch_part<4, DPL, T>(ctx, grid, n_q, n_kv, scale, q, K, V, slot_stride, meta, tmp, out, n_splits);
    case 8:
    case 16:  // four heads per block, G / 4 blocks per KV head
      grid.y *= (unsigned)(G / 4);
      return launch_part<4, DPL, T>(ctx, grid, n_q, n_kv, scale, q, K, V, slot_stride, meta, tmp, out, n_splits);
  }
  return ks_fail(ctx, KS_ERR_UNSUPPORTED, "sdpa: n_q/n_kv = %d not supported (1, 2, 4, 8, 16)", G);
}

}  // namespace

int ks_launch_sdpa(ks_ctx* ctx, size_t n_slots, size_t n_q, size_t n_kv, size_t hd, float scale, ks_dtype act,
                   const void* q, const uint8_t* K, const uint8_t* V, size_t slot_stride_bytes, const float* meta,
                   float* tmp, void* out, int n_splits) {
  const int G = (int)(n_q / n_kv);
  dim3 grid((unsigned)n_splits, (unsigned)n_kv, (unsigned)n_slots);
  int rc = 1;
  static const bool per_row = getenv("KSEARCH_SDPA_PER_ROW") != nullptr;  // keep the per-row kernel (comparison runs)
  const bool aligned4 = (((uintptr_t)K | (uintptr_t)V | (uintptr_t)slot_stride_bytes) & 3u) == 0;
  if (!per_row && aligned4 && G <= 8 && (hd == 256 || hd == 128)) {
    if (hd == 256)
      rc = act == KS_F32 ? launch_tile_g<256, float>(ctx, G, grid, (unsigned)n_q, (unsigned)n_kv, scale, q, K, V, slot_stride_bytes, meta, tmp, out, n_splits)
                         : launch_tile_g<256, __half>(ctx, G, grid, (unsigned)n_q, (unsigned)n_kv, scale, q, K, V, slot_stride_bytes, meta, tmp, out, n_splits);
    else
      rc = act == KS_F32 ? launch_tile_g<128, float>(ctx, G, grid, (unsigned)n_q, (unsigned)n_kv, scale, q, K, V, slot_stride_bytes, meta, tmp, out, n_splits)
                         : launch_tile_g<128, __half>(ctx, G, grid, (unsigned)n_q, (unsigned)n_kv, scale, q, K, V, slot_stride_bytes, meta, tmp, out, n_splits);
  }
  if (rc != 1) {
    // the tiled kernel took it
  } else if (hd == 256) {
    rc = act == KS_F32 ? launch_part_g<8, float>(ctx, G, grid, (unsigned)n_q, (unsigned)n_kv, scale, q, K, V, slot_stride_bytes, meta, tmp, out, n_splits)
                       : launch_part_g<8, __half>(ctx, G, grid, (unsigned)n_q, (unsigned)n_kv, scale, q, K, V, slot_stride_bytes, meta, tmp, out, n_splits);
  } else if (hd == 128) {
    rc = act == KS_F32 ? launch_part_g<4, float>(ctx, G, grid, (unsigned)n_q, (unsigned)n_kv, scale, q, K, V, slot_stride_bytes, meta, tmp, out, n_splits)
                       : launch_part_g<4, __half>(ctx, G, grid, (unsigned)n_q, (unsigned)n_kv, scale, q, K, V, slot_stride_bytes, meta, tmp, out, n_splits);
  } else {
    return ks_fail(ctx, KS_ERR_UNSUPPORTED, "sdpa: head_dim %zu not supported (128, 256)", hd);
  }
  if (rc || n_splits == 1) return rc;
  const unsigned blocks = (unsigned)(n_slots * n_q);
  if (act == KS_F32)
    KS_LAUNCH(ctx, (sdpa_reduce_kernel<float>), blocks, 1024, 0, (unsigned)hd, tmp, (float*)out, n_splits);
  else
    KS_LAUNCH(ctx, (sdpa_reduce_kernel<__half>), blocks, 1024, 0, (unsigned)hd, tmp, (__half*)out, n_splits);
  return ks_after_launch(ctx, "sdpa_reduce");
}

extern "C" {

size_t ks_sdpa_tmp_floats(size_t n_slots, size_t n_q, size_t hd, int n_splits) {
  if (n_splits <= 1) return 0;
  return n_slots * n_q * (size_t)n_splits * (hd + 2);
}

int ks_sdpa_pick_splits(const ks_ctx* ctx, size_t n_slots, size_t n_kv, size_t max_t) {
  // about 256 blocks in all (a block serves up to four query heads, so a slot has at least two per split), at least
  // 128 positions per split: measured best over 1..8 slots x 1024..16384 positions on B200
  (void)ctx;
  const size_t per_split = (n_slots ? n_slots : 1) * (n_kv > 2 ? n_kv : 2);
  size_t want = 256 / per_split;
  size_t by_len = (max_t + 127) / 128;
  size_t s = want < by_len ? want : by_len;
  if (s < 1) s = 1;
  if (s > KS_SDPA_MAX_SPLITS) s = KS_SDPA_MAX_SPLITS;
  return (int)s;
}

int ks_sdpa_decode(ks_ctx* ctx, size_t n_slots, size_t n_q, size_t n_kv, size_t hd, size_t max_t, ks_dtype kv_dtype,
                   float scale, ks_dtype act, const ks_buf* q, const ks_buf* K, const ks_buf* V, size_t kv_byte_off,
                   size_t slot_stride_bytes, const ks_buf* meta, ks_buf* tmp, ks_buf* out, int n_splits) {
  if (!ctx) return KS_ERR_INVALID;
  KS_REQUIRE(ctx, kv_dtype == KS_Q40, "sdpa: KV dtype %d not supported (Q40)", (int)kv_dtype);
  KS_REQUIRE(ctx, ks_is_act(act), "sdpa: activation dtype must be F32 or F16");
  KS_REQUIRE(ctx, n_slots > 0 && n_slots < 65536 && n_q > 0 && n_kv > 0 && n_kv < 65536, "sdpa: bad slot or head count");
  KS_REQUIRE(ctx, n_q % n_kv == 0, "sdpa: n_q=%zu is not a multiple of n_kv=%zu", n_q, n_kv);
  KS_REQUIRE(ctx, hd % 32 == 0, "sdpa hd must be multiple of 32");
  KS_REQUIRE(ctx, max_t > 0, "sdpa: max_t must be > 0");
  if (n_splits == 0) n_splits = ks_sdpa_pick_splits(ctx, n_slots, n_kv, max_t);
  KS_REQUIRE(ctx, n_splits >= 1 && n_splits <= KS_SDPA_MAX_SPLITS, "sdpa: n_splits=%d outside 1..%d", n_splits, KS_SDPA_MAX_SPLITS);
  const size_t ab = ks_act_bytes(act);
  const size_t rowb = hd / 32 * KS_Q40_BLOCK_BYTES;
  const size_t slot_bytes = max_t * n_kv * rowb;
  KS_REQUIRE(ctx, n_slots == 1 || slot_stride_bytes >= slot_bytes, "sdpa: slot stride smaller than one slot's cache");
  KS_REQUIRE(ctx, kv_byte_off % 2 == 0 && slot_stride_bytes % 2 == 0, "sdpa: odd KV offset or stride");
  const size_t kv_need = (n_slots - 1) * slot_stride_bytes + slot_bytes;
  KS_REQUIRE(ctx, ks_fits(K, kv_byte_off, kv_need) && ks_fits(V, kv_byte_off, kv_need), "sdpa: KV buffer too small for max_t=%zu", max_t);
  KS_REQUIRE(ctx, ks_fits(q, 0, n_slots * n_q * hd * ab) && ks_fits(out, 0, n_slots * n_q * hd * ab), "sdpa: q/out buffer too small");
  KS_REQUIRE(ctx, ks_fits(meta, 0, n_slots * 16), "sdpa: meta buffer too small (4 f32 per slot)");
  if (n_splits > 1)
    KS_REQUIRE(ctx, ks_fits(tmp, 0, ks_sdpa_tmp_floats(n_slots, n_q, hd, n_splits) * 4), "sdpa: tmp buffer too small for %d splits", n_splits);
  // (tlen, start) are device-resident and trusted to satisfy start + tlen <= max_t, as in the reference.
  return ks_launch_sdpa(ctx, n_slots, n_q, n_kv, hd, scale, act, q->dptr, (const uint8_t*)K->dptr + kv_byte_off,
                        (const uint8_t*)V->dptr + kv_byte_off, slot_stride_bytes, (const float*)meta->dptr,
                        n_splits > 1 ? (float*)tmp->dptr : nullptr, out->dptr, n_splits);
}

}  // extern "C"

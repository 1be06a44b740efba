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
// memory; thread d then adds O[d] of the splits eight at a time, every load of a batch issued before any is used
// (one after the other they cost a memory round trip per split).
template <typename T>
__global__ void sdpa_reduce_kernel(unsigned hd, const float* tmp, T* out, int n_splits) {
  ks_pdl_entry();
  __shared__ float sm[2 * KS_SDPA_MAX_SPLITS];
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
  const float inv_l = 1.0f / L;
  for (unsigned d = threadIdx.x; d < hd; d += blockDim.x) {
    float o = 0.0f;
    for (int pb = 0; pb < n_splits; pb += 8) {
      float v[8];
#pragma unroll
      for (int k = 0; k < 8; k++)
        if (pb + k < n_splits) v[k] = rec0[(size_t)(pb + k) * (hd + 2) + 2 + d];
#pragma unroll
      for (int k = 0; k < 8; k++)
        if (pb + k < n_splits) o = fmaf(v[k], __expf(sm[2 * (pb + k)] - M), o);
    }
    st_act<T>(out, sh * hd + d, o * inv_l);
  }
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
  int rc;
  if (hd == 256) {
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
    KS_LAUNCH(ctx, (sdpa_reduce_kernel<float>), blocks, 256, 0, (unsigned)hd, tmp, (float*)out, n_splits);
  else
    KS_LAUNCH(ctx, (sdpa_reduce_kernel<__half>), blocks, 256, 0, (unsigned)hd, tmp, (__half*)out, n_splits);
  return ks_after_launch(ctx, "sdpa_reduce");
}

extern "C" {

size_t ks_sdpa_tmp_floats(size_t n_slots, size_t n_q, size_t hd, int n_splits) {
  if (n_splits <= 1) return 0;
  return n_slots * n_q * (size_t)n_splits * (hd + 2);
}

int ks_sdpa_pick_splits(const ks_ctx* ctx, size_t n_slots, size_t n_kv, size_t max_t) {
  // enough (slot, kv head, split) blocks for two per SM, no split shorter than 32 positions
  size_t want = (size_t)ctx->sm_count * 2 / (n_slots * n_kv ? n_slots * n_kv : 1);
  size_t by_len = (max_t + 31) / 32;
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

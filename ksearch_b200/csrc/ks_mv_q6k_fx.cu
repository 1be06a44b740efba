// Q6_K matvec with the input vector as 24-bit block fixed point and byte dot products (dp4a).
//
// Stands in for the same reference lowering as the other Q6_K kernels
// (crates/ksearch_codegen/src/lower.rs:2086-2472; block layout gguf_impl.rs:756-826): the 262144-row
// tied lm_head of the decode step.  The f32 kernels spend ~4.4 instructions per weight rebuilding
// 6-bit values and converting them; here a lane owns 64 weights that share one x scale per 16 and one
// weight scale per 16 -- (block, half h, 16-position run `is`) x the four 32-groups k -- so the 6-bit
// values stay bytes, go through dp4a against three byte planes of x, and only 4 integer sums per 64
// weights are converted to f32.
//
// x: every 32-element sub-block shares a scale s; element i is X_i = round(x_i / s), |X_i| <= 8e6,
// stored as three byte planes (X = l2*65536 + l1*256 + l0, l2 signed).  Exact integer accumulation;
// x is rounded to 2^-23 of its sub-block's largest element.
// Shared memory: plane p at p * nbh * 160 bytes (nbh = 2 * blocks per row); inside, (block, h) at 160
// bytes (128 used: k * 32 + is * 16 + word * 4; the pad keeps the 8 lanes of a row on different banks);
// then nbh float4 of sub-block scales (k = 0..3) and 2 * nbh float4 of 16-element sums of x (the -32
// offset of Q6_K folds into them).
#include "ks_mv_common.cuh"

namespace {

constexpr unsigned Q6F_BH = 160;

struct Q6fArgs {
  const uint8_t* W;
  void* y;
  unsigned rows, cols, row_bytes;
  const void* x;
};

__device__ __forceinline__ uint32_t ldg_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(p));  // L1 keeps the sector for the neighbouring words
  return v;
}
__device__ __forceinline__ unsigned q6f_dp_uu(unsigned a, unsigned b, unsigned c) {
  unsigned d;
  asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int q6f_dp_us(unsigned a, unsigned b, int c) {  // a: unsigned bytes, b: signed bytes
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

template <typename XT>
__device__ __forceinline__ void q6f_stage_x(unsigned char* smem, const XT* x, unsigned cols) {
  const unsigned nbh = cols >> 7;  // (block, half) pairs per row
  const size_t plane = (size_t)nbh * Q6F_BH;
  float* scl = reinterpret_cast<float*>(smem + 3 * plane);
  float* s16 = scl + (size_t)nbh * 4;
  const unsigned nchunk = cols >> 2;  // a multiple of 64: whole warps run every trip
  for (unsigned c = threadIdx.x; c < nchunk; c += blockDim.x) {
    const float4 v = ld_chunk<XT>(x, c);
    const unsigned e = c << 2;
    const unsigned bh = e >> 7, k = (e >> 5) & 3u, l = e & 31u;
    float s = (v.x + v.y) + (v.z + v.w);
    float am = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
#pragma unroll
    for (int o = 1; o <= 4; o <<= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    const float inv = am > 0.0f ? __fdividef(8.0e6f, am) : 0.0f;
    const int X0 = __float2int_rn(v.x * inv), X1 = __float2int_rn(v.y * inv), X2 = __float2int_rn(v.z * inv),
              X3 = __float2int_rn(v.w * inv);
    unsigned char* base = smem + (size_t)bh * Q6F_BH + k * 32u + l;  // l = is * 16 + word * 4
    *reinterpret_cast<uint32_t*>(base) = __byte_perm(__byte_perm(X0, X1, 0x0040), __byte_perm(X2, X3, 0x0040), 0x5410);
    *reinterpret_cast<uint32_t*>(base + plane) = __byte_perm(__byte_perm(X0, X1, 0x0051), __byte_perm(X2, X3, 0x0051), 0x5410);
    *reinterpret_cast<uint32_t*>(base + 2 * plane) = __byte_perm(__byte_perm(X0, X1, 0x0062), __byte_perm(X2, X3, 0x0062), 0x5410);
    if ((threadIdx.x & 7u) == 0) scl[(size_t)bh * 4 + k] = am > 0.0f ? am * (1.0f / 8.0e6f) : 1.0f;
    if ((threadIdx.x & 3u) == 0) s16[((size_t)bh * 2 + (l >> 4)) * 4 + k] = s;
  }
}

// One aligned word of the packed rows: from global memory, or (SM) from the shared-memory stage they were copied to.
template <bool SM>
__device__ __forceinline__ uint32_t q6f_word(const uint32_t* p) {
  if (SM) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"((uint32_t)__cvta_generic_to_shared(p)));
    return v;
  }
  return ldg_u32(p);
}
template <bool SM>
__device__ __forceinline__ uint32_t q6f_half(const uint8_t* p) {
  if (SM) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"((uint32_t)__cvta_generic_to_shared(p)));
    return v;
  }
  return ldg_stream_u16(p);
}
// 16 bytes at a 2-byte aligned address as four words: aligned words around them plus a byte permute.
template <bool SM>
__device__ __forceinline__ void q6f_load16(const uint8_t* p, unsigned odd, uint32_t sel, uint32_t (&out)[4]) {
  const uint32_t* b = reinterpret_cast<const uint32_t*>(p - 2 * odd);
  const uint32_t w0 = q6f_word<SM>(b), w1 = q6f_word<SM>(b + 1), w2 = q6f_word<SM>(b + 2), w3 = q6f_word<SM>(b + 3);
  uint32_t w4 = 0;
  if (odd) w4 = q6f_word<SM>(b + 4);
  out[0] = __byte_perm(w0, w1, sel);
  out[1] = __byte_perm(w1, w2, sel);
  out[2] = __byte_perm(w2, w3, sel);
  out[3] = __byte_perm(w3, w4, sel);
}

// One tile: R row sets of 4 rows side by side (8 lanes per row), rowp[r] = this lane's row of set r (global memory,
// or SM: its copy in shared memory), against the staged x.  Leaves the lane's partial sums in yacc.
template <int R, bool SM>
__device__ __forceinline__ void q6f_tile(const uint8_t* const (&rowp)[R], unsigned units, unsigned nbh, uint32_t plane, uint32_t xs,
                                         const unsigned char* smem, int cl, float (&yacc)[R]) {
  constexpr int LPR = 8;
#pragma unroll
  for (int r = 0; r < R; r++) yacc[r] = 0.0f;
  for (unsigned u = cl; u < units; u += LPR) {
    const unsigned blk = u >> 2, h = (u >> 1) & 1u, is = u & 1u;
    uint32_t A[R][4], B[R][4], H[R][4], S01[R], S23[R], D[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
      const uint8_t* bp = rowp[r] + (size_t)blk * KS_Q6K_BLOCK_BYTES;
      const unsigned odd = (unsigned)((reinterpret_cast<uintptr_t>(bp) >> 1) & 1u);
      const uint32_t sel = odd ? 0x5432u : 0x3210u;
      q6f_load16<SM>(bp + 64 * h + 16 * is, odd, sel, A[r]);
      q6f_load16<SM>(bp + 64 * h + 32 + 16 * is, odd, sel, B[r]);
      q6f_load16<SM>(bp + 128 + 32 * h + 16 * is, odd, sel, H[r]);
      const uint32_t* sb = reinterpret_cast<const uint32_t*>(bp + 192 + 8 * h - 2 * odd);
      const uint32_t s0 = q6f_word<SM>(sb), s1 = q6f_word<SM>(sb + 1);
      uint32_t s2 = 0;
      if (odd) s2 = q6f_word<SM>(sb + 2);
      S01[r] = __byte_perm(s0, s1, sel);
      S23[r] = __byte_perm(s1, s2, sel);
      D[r] = q6f_half<SM>(bp + 208);
    }
    const uint32_t xa = xs + (blk * 2 + h) * Q6F_BH + is * 16u;
    const float4 sxv = lds_f4(reinterpret_cast<const void*>(smem + 3 * (size_t)plane + (size_t)(blk * 2 + h) * 16));
    const float4 s16v = lds_f4(reinterpret_cast<const void*>(smem + 3 * (size_t)plane + (size_t)nbh * 16 + (size_t)((blk * 2 + h) * 2 + is) * 16));
    float part[R];
#pragma unroll
    for (int r = 0; r < R; r++) part[r] = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      uint4 x0, x1, x2;
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(x0.x), "=r"(x0.y), "=r"(x0.z), "=r"(x0.w) : "r"(xa + k * 32u));
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(x1.x), "=r"(x1.y), "=r"(x1.z), "=r"(x1.w) : "r"(xa + plane + k * 32u));
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(x2.x), "=r"(x2.y), "=r"(x2.z), "=r"(x2.w) : "r"(xa + 2u * plane + k * 32u));
      const unsigned xw0[4] = {x0.x, x0.y, x0.z, x0.w}, xw1[4] = {x1.x, x1.y, x1.z, x1.w}, xw2[4] = {x2.x, x2.y, x2.z, x2.w};
      const float sxk = k == 0 ? sxv.x : k == 1 ? sxv.y : k == 2 ? sxv.z : sxv.w;
      const float s16k = k == 0 ? s16v.x : k == 1 ? s16v.y : k == 2 ? s16v.z : s16v.w;
#pragma unroll
      for (int r = 0; r < R; r++) {
        unsigned a0 = 0u, a1 = 0u;
        int a2 = 0;
#pragma unroll
        for (int w = 0; w < 4; w++) {
          const uint32_t q = (k & 1) ? B[r][w] : A[r][w];
          const uint32_t nib = ((k & 2) ? (q >> 4) : q) & 0x0F0F0F0Fu;
          const uint32_t hb = (k == 0 ? (H[r][w] << 4) : k == 1 ? (H[r][w] << 2) : k == 2 ? H[r][w] : (H[r][w] >> 2)) & 0x30303030u;
          const uint32_t v = nib | hb;
          a0 = q6f_dp_uu(v, xw0[w], a0);
          a1 = q6f_dp_uu(v, xw1[w], a1);
          a2 = q6f_dp_us(v, xw2[w], a2);
        }
        const float f = fmaf((float)a2, 65536.0f, fmaf((float)a1, 256.0f, (float)a0)) * sxk;
        // scale sc[8h + is + 2k]: byte (is + 2k) of the 8 scale bytes of this half
        const uint32_t sw = (k & 2) ? S23[r] : S01[r];
        const int sc = (int)(signed char)((sw >> (8u * (is + 2u * (k & 1)))) & 0xFFu);
        part[r] = fmaf((float)sc, fmaf(-32.0f, s16k, f), part[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < R; r++) yacc[r] = fmaf(__half2float(__ushort_as_half((unsigned short)D[r])), part[r], yacc[r]);
  }
}

template <int R, typename XT>
__global__ void __launch_bounds__(256) mv_q6k_fx_kernel(const Q6fArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  ks_pdl_entry();
  constexpr int RL = 4, LPR = 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int cl = lane % LPR, rl = lane / LPR;
  const unsigned nb = a.cols >> 8, units = nb * 4, nbh = nb * 2;
  const uint32_t plane = nbh * Q6F_BH;
  q6f_stage_x<XT>(smem, reinterpret_cast<const XT*>(a.x), a.cols);
  __syncthreads();
  const uint32_t xs = (uint32_t)__cvta_generic_to_shared(smem);
  const unsigned tiles = (a.rows + RL * R - 1) / (RL * R);

  for (unsigned tile = blockIdx.x * nwarp + warp; tile < tiles; tile += gridDim.x * nwarp) {
    const uint8_t* rowp[R];
    unsigned rowi[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
      rowi[r] = tile * (RL * R) + r * RL + rl;
      const unsigned lr = rowi[r] < a.rows ? rowi[r] : a.rows - 1;
      rowp[r] = a.W + (size_t)lr * a.row_bytes;
    }
    float yacc[R];
    q6f_tile<R, false>(rowp, units, nbh, plane, xs, smem, cl, yacc);
#pragma unroll
    for (int r = 0; r < R; r++) {
      float v = yacc[r];
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (cl == 0 && rowi[r] < a.rows) act_store<XT>(reinterpret_cast<XT*>(a.y), rowi[r], v);
    }
  }
}

// The same arithmetic with the rows streamed through shared memory (planner variant 4).  A tile is 4R consecutive
// rows = 840 R * (cols / 256) bytes, a multiple of 16 at a 16-byte aligned address (the launcher checks), so ONE
// cp.async.bulk brings it in;
// read straight from global memory the same rows cost 2.1x their bytes in L2 traffic, because the 16-byte fields of a
// 210-byte block sit at 2-byte alignment and straddle 32-byte sectors.  Every warp owns a ring of `stages` tiles
// (mbarrier completion, bounded waits); the copies of the first tiles are issued before griddepcontrol.wait.
template <int R, typename XT>
__global__ void __launch_bounds__(512) mv_q6k_ring_kernel(const Q6fArgs a, unsigned stages, unsigned x_bytes, unsigned* err) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int RL = 4, LPR = 8;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int cl = lane % LPR, rl = lane / LPR;
  const unsigned nb = a.cols >> 8, units = nb * 4, nbh = nb * 2;
  const uint32_t plane = nbh * Q6F_BH;
  const unsigned tile_bytes = RL * R * a.row_bytes;
  const unsigned tile_pad = (tile_bytes + 127u) & ~127u;
  const unsigned tiles = a.rows / (RL * R);  // the launcher takes only row counts that are multiples of the tile
  unsigned char* ring = smem + ((x_bytes + 127u) & ~127u) + (size_t)warp * stages * tile_pad;
  const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);
  const uint32_t bars = (uint32_t)__cvta_generic_to_shared(smem + ((x_bytes + 127u) & ~127u) + (size_t)nwarp * stages * tile_pad) +
                        (uint32_t)warp * stages * 8u;
  const unsigned t0 = blockIdx.x * nwarp + warp, tstep = gridDim.x * nwarp;
  const unsigned n_mine = t0 < tiles ? (tiles - t0 + tstep - 1) / tstep : 0u;
  if (lane == 0) {
    for (unsigned s = 0; s < stages; s++)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bars + s * 8u), "r"(1u) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();
  auto fetch = [&](unsigned n) {  // lane 0: my n-th tile into stage n % stages
    const unsigned st = n % stages;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bars + st * 8u), "r"(tile_bytes) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(ring_s + st * tile_pad),
                 "l"(a.W + (size_t)(t0 + n * tstep) * tile_bytes), "r"(tile_bytes), "r"(bars + st * 8u)
                 : "memory");
  };
  if (lane == 0)
    for (unsigned n = 0; n < stages && n < n_mine; n++) fetch(n);  // weights are constants: before the wait
  ks_pdl_entry();
  q6f_stage_x<XT>(smem, reinterpret_cast<const XT*>(a.x), a.cols);
  __syncthreads();
  const uint32_t xs = (uint32_t)__cvta_generic_to_shared(smem);
  bool dead = false;
  for (unsigned n = 0; n < n_mine && !dead; n++) {
    const unsigned st = n % stages, par = (n / stages) & 1u;
    bool ok = false;
    for (unsigned i = 0; i < (1u << 22) && !ok; i++) {
      unsigned done;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(done)
          : "r"(bars + st * 8u), "r"(par)
          : "memory");
      ok = done != 0;
    }
    if (!__all_sync(0xffffffffu, ok)) {  // the copy never landed: raise the status word and stop
      if (lane == 0) atomicOr(err, 1u);
      dead = true;
      break;
    }
    const unsigned char* stage = ring + (size_t)st * tile_pad;
    const uint8_t* rowp[R];
#pragma unroll
    for (int r = 0; r < R; r++) rowp[r] = stage + (size_t)(r * RL + rl) * a.row_bytes;
    float yacc[R];
    q6f_tile<R, true>(rowp, units, nbh, plane, xs, smem, cl, yacc);
    __syncwarp();  // every lane is done with the stage
    if (lane == 0 && n + stages < n_mine) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // it was read through the generic proxy
      fetch(n + stages);
    }
    const unsigned tile = t0 + n * tstep;
#pragma unroll
    for (int r = 0; r < R; r++) {
      float v = yacc[r];
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (cl == 0) act_store<XT>(reinterpret_cast<XT*>(a.y), tile * (RL * R) + r * RL + rl, v);
    }
  }
}

template <int R, typename XT>
int launch_q6f(ks_ctx* ctx, const Q6fArgs& a, unsigned grid, int nwarps, size_t smem) {
  auto kern = mv_q6k_fx_kernel<R, XT>;
  static size_t smem_set[16] = {0};
  if (smem > 48 * 1024 && smem > smem_set[ctx->device & 15]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "matvec: cannot set %zu B shared memory: %s", smem, cudaGetErrorString(e));
    smem_set[ctx->device & 15] = smem;
  }
  KS_LAUNCH(ctx, kern, grid, nwarps * 32, smem, a);
  return ks_after_launch(ctx, "matvec_q6k_fx");
}

}  // namespace

// Plan variant 2 of the Q6_K matvec.  Returns 1 (not an error) when the call is outside what this
// kernel takes -- several tokens, several segments, weights not 4-byte aligned -- and the caller
// falls back to the other variants.  plan: nr = rows per lane (1 or 2), nwarps, ctas_per_sm.
int ks_launch_matvec_q6k_fx(ks_ctx* ctx, const ks_mv_seg* segs, int n_seg, size_t cols, ks_dtype act, const void* x,
                            int n_tok, const ks_plan* plan) {
  if (n_tok != 1 || n_seg != 1 || ((uintptr_t)segs[0].W & 3) || cols % 256) return 1;
  if ((uintptr_t)x & (act == KS_F32 ? 15 : 7)) return 1;  // x is staged with 16-byte (8-byte) loads
  const unsigned nb = (unsigned)(cols / 256), nbh = nb * 2;
  const size_t smem = 3 * (size_t)nbh * Q6F_BH + (size_t)nbh * 16 + (size_t)nbh * 32;
  if (smem > (size_t)ctx->smem_optin) return 1;
  int nwarps = (plan && plan->nwarps > 0) ? plan->nwarps : 8;
  if (nwarps > 8) nwarps = 8;
  const int R = (!plan || plan->nr >= 2) ? 2 : 1;
  const int cps = (plan && plan->ctas_per_sm > 0) ? plan->ctas_per_sm : 6;
  Q6fArgs a{};
  a.W = segs[0].W;
  a.y = segs[0].y;
  a.rows = segs[0].rows;
  a.cols = (unsigned)cols;
  a.row_bytes = nb * KS_Q6K_BLOCK_BYTES;
  a.x = x;
  const unsigned tiles = (a.rows + 4 * R - 1) / (4 * R);
  unsigned grid = (tiles + nwarps - 1) / nwarps;
  const unsigned cap = (unsigned)(ctx->sm_count * cps);
  if (grid > cap) grid = cap;
  if (act == KS_F32) return R == 2 ? launch_q6f<2, float>(ctx, a, grid, nwarps, smem) : launch_q6f<1, float>(ctx, a, grid, nwarps, smem);
  return R == 2 ? launch_q6f<2, __half>(ctx, a, grid, nwarps, smem) : launch_q6f<1, __half>(ctx, a, grid, nwarps, smem);
}

// Plan variant 4 of the Q6_K matvec: the rows streamed through per-warp shared-memory rings.  Returns 1 when the
// call is outside what it takes (several tokens or segments, a row count that is not a multiple of the tile, tiles
// that are not a multiple of 16 bytes, rows too long for two stages per warp).  plan: nr = row sets per tile (1 or 2:
// tiles of 4 or 8 rows), nwarps (up to 16), stages (variant bits 8-15).
namespace {
template <int R>
int launch_q6_ring(ks_ctx* ctx, const Q6fArgs& a, ks_dtype act, unsigned grid, int nwarps, unsigned stages, unsigned x_bytes, size_t smem) {
  unsigned* err = (unsigned*)ctx->ws + KS_WS_ERR_WORD;
  static size_t smem_set[2][16] = {{0}};
  const int ti = act == KS_F32 ? 0 : 1;
  if (smem > smem_set[ti][ctx->device & 15]) {
    cudaError_t e = act == KS_F32 ? cudaFuncSetAttribute(mv_q6k_ring_kernel<R, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                                  : cudaFuncSetAttribute(mv_q6k_ring_kernel<R, __half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "matvec: cannot set %zu B shared memory: %s", smem, cudaGetErrorString(e));
    smem_set[ti][ctx->device & 15] = smem;
  }
  if (act == KS_F32)
    KS_LAUNCH(ctx, (mv_q6k_ring_kernel<R, float>), grid, nwarps * 32, smem, a, stages, x_bytes, err);
  else
    KS_LAUNCH(ctx, (mv_q6k_ring_kernel<R, __half>), grid, nwarps * 32, smem, a, stages, x_bytes, err);
  return ks_after_launch(ctx, "matvec_q6k_ring");
}
}  // namespace

int ks_launch_matvec_q6k_ring(ks_ctx* ctx, const ks_mv_seg* segs, int n_seg, size_t cols, ks_dtype act, const void* x, int n_tok,
                              const ks_plan* plan) {
  if (n_tok != 1 || n_seg != 1 || ((uintptr_t)segs[0].W & 15) || cols % 256) return 1;
  if ((uintptr_t)x & (act == KS_F32 ? 15 : 7)) return 1;
  const unsigned nb = (unsigned)(cols / 256), nbh = nb * 2;
  const unsigned R = (plan && plan->nr == 1) ? 1u : 2u;
  const unsigned tile_bytes = 4u * R * nb * KS_Q6K_BLOCK_BYTES;
  if (tile_bytes % 16u || segs[0].rows % (4u * R)) return 1;
  const unsigned x_bytes = 3u * nbh * Q6F_BH + nbh * 16u + nbh * 32u;
  const unsigned tile_pad = (tile_bytes + 127u) & ~127u;
  unsigned stages = plan ? (unsigned)((plan->variant >> 8) & 0xFF) : 0u;
  if (stages < 2u) stages = 2u;
  int nwarps = (plan && plan->nwarps > 0) ? plan->nwarps : 8;
  if (nwarps > 16) nwarps = 16;
  const unsigned budget = (unsigned)ctx->smem_optin;
  auto need = [&](int nw, unsigned st) { return ((x_bytes + 127u) & ~127u) + (unsigned)nw * st * tile_pad + (unsigned)nw * st * 8u + 128u; };
  while (stages > 2u && need(nwarps, stages) > budget) stages--;
  while (nwarps > 1 && need(nwarps, stages) > budget) nwarps--;
  if (need(nwarps, stages) > budget) return 1;
  Q6fArgs a{};
  a.W = segs[0].W;
  a.y = segs[0].y;
  a.rows = segs[0].rows;
  a.cols = (unsigned)cols;
  a.row_bytes = nb * KS_Q6K_BLOCK_BYTES;
  a.x = x;
  const unsigned tiles = a.rows / (4u * R);
  unsigned grid = (tiles + nwarps - 1) / nwarps;
  if (grid > (unsigned)ctx->sm_count) grid = (unsigned)ctx->sm_count;
  const size_t smem = need(nwarps, stages);
  return R == 2 ? launch_q6_ring<2>(ctx, a, act, grid, nwarps, stages, x_bytes, smem)
                : launch_q6_ring<1>(ctx, a, act, grid, nwarps, stages, x_bytes, smem);
}

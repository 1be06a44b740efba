// Streamed dequant-fused matvec for Q4_K / Q6_K on sm_100a: the weight stream is moved by the
// bulk-copy engine (cp.async.bulk global -> shared, completion on an mbarrier) and never passes
// through registers on its way in; every warp owns a private ring of stages and is its own
// producer, so there is no block-wide synchronisation after x has been staged.
//
// Stands in for the same reference lowerings as ks_matvec.cu
// (crates/ksearch_codegen/src/lower.rs:1763-2082, 2086-2472, 2673-2968, 3343-3464).
//
// Work decomposition.  Rows are cut into groups of RL*R rows (RL = 32/LPR rows side by side in
// a warp, R per lane) and every row into column segments of `seg_blocks` super-blocks.  One
// pipeline item = one row group x one column segment = RL*SLOTS bulk copies (one per row
// segment, each contiguous and 16-byte aligned).  Warp gw handles groups gw, gw+GW, ...; the
// partial sums of a group stay in registers across its segments.
//
// The kernel starts its first copies BEFORE it waits for the previous kernel in the stream
// (programmatic dependent launch): weights do not depend on anything a predecessor writes,
// x does.  Every wait on an mbarrier is bounded; when a wait gives up the warp raises the
// context's error word, drains its own copies (bounded too) and returns without storing.
#include "ks_mv_common.cuh"

namespace {

struct MvsArgs {
  const uint8_t* W[3];
  void* y[3];
  unsigned rows[3];
  unsigned grp_start[4];  // first row-group index of each segment; [n_seg] = total groups
  int n_seg;
  unsigned row_bytes;
  unsigned cols;
  const void* x;
  int n_tok;
  unsigned seg_blocks;  // super-blocks per column segment
  unsigned n_cseg;      // column segments per row
  int stages;
  unsigned* err;
  MvPro pro;
};

__device__ __forceinline__ const uint8_t* s_w(const MvsArgs& a, int s) { return s == 0 ? a.W[0] : s == 1 ? a.W[1] : a.W[2]; }
__device__ __forceinline__ void* s_y(const MvsArgs& a, int s) { return s == 0 ? a.y[0] : s == 1 ? a.y[1] : a.y[2]; }
__device__ __forceinline__ unsigned s_rows(const MvsArgs& a, int s) { return s == 0 ? a.rows[0] : s == 1 ? a.rows[1] : a.rows[2]; }
__device__ __forceinline__ unsigned s_g0(const MvsArgs& a, int s) { return s == 0 ? a.grp_start[0] : s == 1 ? a.grp_start[1] : a.grp_start[2]; }
__device__ __forceinline__ unsigned s_total(const MvsArgs& a) {
  return a.n_seg == 1 ? a.grp_start[1] : a.n_seg == 2 ? a.grp_start[2] : a.grp_start[3];
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: about a second of polling at most, then give up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, unsigned parity) {
  for (unsigned i = 0; i < (1u << 22); i++)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, unsigned bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Shared memory map (bytes): [x staging | pad to 128 | stage rings of all warps | mbarriers]
struct Layout {
  unsigned x_bytes, ring_off, stage_bytes, bar_off, red_off, total;
};
__host__ __device__ inline Layout make_layout(unsigned x_bytes, unsigned stage_bytes, int nwarps, int stages) {
  Layout L;
  L.x_bytes = x_bytes;
  L.ring_off = (x_bytes + 127u) & ~127u;
  L.stage_bytes = stage_bytes;
  L.bar_off = L.ring_off + stage_bytes * (unsigned)(nwarps * stages);
  L.red_off = (L.bar_off + 8u * (unsigned)(nwarps * stages) + 15u) & ~15u;  // 32 floats for block reductions
  L.total = L.red_off + 128u;
  return L;
}

// -----------------------------------------------------------------------------------------------
template <int LPR, int R, int NT, int EPI, typename XT>
__global__ void __launch_bounds__(256) mvs_q4k_kernel(const MvsArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int RL = 32 / LPR;
  constexpr int MATS = (EPI == KS_EPI_GATE_UP) ? 2 : 1;
  constexpr int SLOTS = R * MATS;  // rows a lane works on per item
  constexpr int GROWS = RL * R;    // logical rows per group
  constexpr int NCOPY = RL * SLOTS;
  static_assert(NCOPY <= 32, "one copy per lane");
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int cl = lane % LPR, rl = lane / LPR;
  const int g = cl & 3;
  const unsigned units = a.cols >> 6;
  const unsigned seg_bytes = a.seg_blocks * KS_Q4K_BLOCK_BYTES;
  const unsigned seg_units = a.seg_blocks * 4;
  const unsigned upl = seg_units / LPR;
  const int S = a.stages;
  const Layout L = make_layout((unsigned)a.n_tok * units * Q4K_XTOK * 4u, (unsigned)NCOPY * seg_bytes, nwarp, S);
  unsigned char* ring = smem + L.ring_off + (size_t)warp * S * L.stage_bytes;
  const uint32_t bars = smem_u32(smem + L.bar_off) + (uint32_t)(warp * S) * 8u;

  const unsigned total_groups = s_total(a);
  const unsigned gw = blockIdx.x * nwarp + warp, GW = gridDim.x * nwarp;
  const unsigned nk = gw < total_groups ? (total_groups - gw + GW - 1) / GW : 0;
  const unsigned n_items = nk * a.n_cseg;

  // Issue the copies of item i (all lanes call this; lanes < NCOPY each start one copy).
  auto issue = [&](unsigned i) {
    const unsigned k = i / a.n_cseg, cs = i - k * a.n_cseg;
    const unsigned grp = gw + k * GW;
    int seg = 0;
    if (a.n_seg > 1 && grp >= a.grp_start[1]) seg = 1;
    if (a.n_seg > 2 && grp >= a.grp_start[2]) seg = 2;
    const unsigned seg_rows = s_rows(a, seg);
    const unsigned row0 = (grp - s_g0(a, seg)) * GROWS;
    const unsigned valid = min((unsigned)GROWS, seg_rows - row0);
    const unsigned st = i % (unsigned)S;
    const uint32_t bar = bars + st * 8u;
    if (lane == 0) mbar_expect_tx(bar, valid * MATS * seg_bytes);
    if (a.n_cseg == 1 && (EPI == KS_EPI_PLAIN || R == 1)) {
      // whole rows: the rows of a group are contiguous in memory, one copy per matrix
      if (lane < MATS) {
        const uint8_t* base = (EPI == KS_EPI_GATE_UP) ? (lane ? a.W[1] : a.W[0]) : s_w(a, seg);
        bulk_g2s(smem_u32(ring + (size_t)st * L.stage_bytes + (size_t)lane * RL * seg_bytes),
                 base + (size_t)row0 * a.row_bytes, valid * seg_bytes, bar);
      }
    } else if (lane < NCOPY) {
      const int slot = lane / RL, rr = lane % RL;
      const unsigned j = (unsigned)(EPI == KS_EPI_GATE_UP ? (slot >> 1) : slot) * RL + rr;  // logical row in group
      if (j < valid) {
        const uint8_t* base = (EPI == KS_EPI_GATE_UP) ? ((slot & 1) ? a.W[1] : a.W[0]) : s_w(a, seg);
        const uint8_t* src = base + (size_t)(row0 + j) * a.row_bytes + (size_t)cs * seg_bytes;
        bulk_g2s(smem_u32(ring + (size_t)st * L.stage_bytes + (size_t)lane * seg_bytes), src, seg_bytes, bar);
      }
    }
  };

  pdl_launch_dependents();  // successors may start (and prefetch their own weights) right away
  if (lane == 0) {
    for (int s = 0; s < S; s++) mbar_init(bars + s * 8u, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  __syncwarp();
  for (unsigned i = 0; i < (unsigned)S && i < n_items; i++) issue(i);

  if (a.pro.mode == KS_PRO_NONE) {
    pdl_wait();  // x is written by the kernel before this one
    q4k_stage_x<XT>(smem, reinterpret_cast<const XT*>(a.x), a.cols, a.n_tok);
  } else
    q4k_stage_x_pro<XT>(smem, reinterpret_cast<float*>(smem + L.red_off), a.pro, reinterpret_cast<const XT*>(a.x), a.cols, a.n_tok);
  __syncthreads();

  float yacc[SLOTS][NT];
#pragma unroll
  for (int r = 0; r < SLOTS; r++)
#pragma unroll
    for (int t = 0; t < NT; t++) yacc[r][t] = 0.0f;
  const uint32_t ring_s = smem_u32(ring), xs_s = smem_u32(smem);
  const uint32_t tok_stride = units * Q4K_XTOK * 4u;

  bool ok = true;
  unsigned i = 0;
  for (; i < n_items; i++) {
    const unsigned k = i / a.n_cseg, cs = i - k * a.n_cseg;
    const unsigned st = i % (unsigned)S;
    if (!mbar_wait(bars + st * 8u, (i / (unsigned)S) & 1u)) {
      ok = false;
      break;
    }
    // 32-bit shared addresses that advance by constants per unit: this lane's first unit of the
    // segment in every row slot, and the matching x fragment / sums.
    uint32_t waddr = ring_s + st * L.stage_bytes + (uint32_t)rl * seg_bytes + (uint32_t)(cl >> 2) * KS_Q4K_BLOCK_BYTES +
                     (uint32_t)g * 32u;
    uint32_t xaddr = xs_s + (cs * seg_units + (unsigned)cl) * (Q4K_XS * 4u);
    uint32_t saddr = xs_s + units * (Q4K_XS * 4u) + (cs * seg_units + (unsigned)cl) * 8u;
    for (unsigned it = 0; it < upl; it++) {
      if constexpr (NT == 1) {
#pragma unroll
      for (int t = 0; t < NT; t++) {
        if (t < a.n_tok) {
          const uint32_t xt = xaddr + (uint32_t)t * tok_stride;
          const float2 sx = lds_f2a(saddr + (uint32_t)t * tok_stride);
          u64 acc[SLOTS][2];
#pragma unroll
          for (int r = 0; r < SLOTS; r++) acc[r][0] = acc[r][1] = 0ull;
          {
            u64 xf[16];  // 16 packed (lo, hi) pairs: l = 0..15
            lds_p2o<0>(xt, xf[0], xf[1]);     lds_p2o<16>(xt, xf[2], xf[3]);
            lds_p2o<32>(xt, xf[4], xf[5]);    lds_p2o<48>(xt, xf[6], xf[7]);
            lds_p2o<64>(xt, xf[8], xf[9]);    lds_p2o<80>(xt, xf[10], xf[11]);
            lds_p2o<96>(xt, xf[12], xf[13]);  lds_p2o<112>(xt, xf[14], xf[15]);
#pragma unroll
            for (int r = 0; r < SLOTS; r++) {
              const uint4 q = lds_u4o<16>(waddr + (uint32_t)(r * RL) * seg_bytes);
              q4_word_p(q.x, xf[0], xf[1], xf[2], xf[3], acc[r][0], acc[r][1]);
              q4_word_p(q.y, xf[4], xf[5], xf[6], xf[7], acc[r][0], acc[r][1]);
              q4_word_p(q.z, xf[8], xf[9], xf[10], xf[11], acc[r][0], acc[r][1]);
              q4_word_p(q.w, xf[12], xf[13], xf[14], xf[15], acc[r][0], acc[r][1]);
            }
          }
          {
            u64 xf[16];  // l = 16..31
            lds_p2o<128>(xt, xf[0], xf[1]);    lds_p2o<144>(xt, xf[2], xf[3]);
            lds_p2o<160>(xt, xf[4], xf[5]);    lds_p2o<176>(xt, xf[6], xf[7]);
            lds_p2o<192>(xt, xf[8], xf[9]);    lds_p2o<208>(xt, xf[10], xf[11]);
            lds_p2o<224>(xt, xf[12], xf[13]);  lds_p2o<240>(xt, xf[14], xf[15]);
#pragma unroll
            for (int r = 0; r < SLOTS; r++) {
              const uint4 q = lds_u4o<32>(waddr + (uint32_t)(r * RL) * seg_bytes);
              q4_word_p(q.x, xf[0], xf[1], xf[2], xf[3], acc[r][0], acc[r][1]);
              q4_word_p(q.y, xf[4], xf[5], xf[6], xf[7], acc[r][0], acc[r][1]);
              q4_word_p(q.z, xf[8], xf[9], xf[10], xf[11], acc[r][0], acc[r][1]);
              q4_word_p(q.w, xf[12], xf[13], xf[14], xf[15], acc[r][0], acc[r][1]);
            }
          }
#pragma unroll
          for (int r = 0; r < SLOTS; r++) {
            const uint4 hdr = lds_u4o<0>(waddr + (uint32_t)(r * RL) * seg_bytes - (uint32_t)g * 32u);
            const float2 a01 = unpack2(padd2(acc[r][0], acc[r][1]));
            yacc[r][t] = q4k_apply_scales(hdr, g, a01.x, a01.y, sx.x, sx.y, yacc[r][t]);
          }
        }
      }
      } else {
        // Several tokens: every nibble is turned into an f32 ONCE and then meets each token's x
        // (the conversion is two thirds of the single-token instruction count).
        u64 acc[SLOTS][NT][2];
#pragma unroll
        for (int r = 0; r < SLOTS; r++)
#pragma unroll
          for (int t = 0; t < NT; t++) acc[r][t][0] = acc[r][t][1] = 0ull;
#pragma unroll
        for (int half = 0; half < 2; half++) {
          constexpr u64 M2 = ((u64)kMagicBits << 32) | kMagicBits;
          u64 f[SLOTS][16];
#pragma unroll
          for (int r = 0; r < SLOTS; r++) {
            const uint4 q = half ? lds_u4o<32>(waddr + (uint32_t)(r * RL) * seg_bytes) : lds_u4o<16>(waddr + (uint32_t)(r * RL) * seg_bytes);
            const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int w = 0; w < 4; w++) {
              const u64 ww = pack2(qw[w], qw[w]), hh = pack2(qw[w] >> 16, qw[w] >> 16);
              f[r][4 * w + 0] = padd2((ww & 0x000000F00000000Full) | M2, kNegMagic2);
              f[r][4 * w + 1] = padd2((ww & 0x0000F00000000F00ull) | M2, kNegMagic2);
              f[r][4 * w + 2] = padd2((hh & 0x000000F00000000Full) | M2, kNegMagic2);
              f[r][4 * w + 3] = padd2((hh & 0x0000F00000000F00ull) | M2, kNegMagic2);
            }
          }
#pragma unroll
          for (int t = 0; t < NT; t++) {
            if (t < a.n_tok) {
              const uint32_t xt = xaddr + (uint32_t)t * tok_stride + (uint32_t)half * 128u;
              u64 xf[16];
              lds_p2o<0>(xt, xf[0], xf[1]);     lds_p2o<16>(xt, xf[2], xf[3]);
              lds_p2o<32>(xt, xf[4], xf[5]);    lds_p2o<48>(xt, xf[6], xf[7]);
              lds_p2o<64>(xt, xf[8], xf[9]);    lds_p2o<80>(xt, xf[10], xf[11]);
              lds_p2o<96>(xt, xf[12], xf[13]);  lds_p2o<112>(xt, xf[14], xf[15]);
#pragma unroll
              for (int r = 0; r < SLOTS; r++)
#pragma unroll
                for (int j = 0; j < 16; j++) acc[r][t][j & 1] = pfma2(f[r][j], xf[j], acc[r][t][j & 1]);
            }
          }
        }
#pragma unroll
        for (int r = 0; r < SLOTS; r++) {
          const uint4 hdr = lds_u4o<0>(waddr + (uint32_t)(r * RL) * seg_bytes - (uint32_t)g * 32u);
          float dsc_lo, dsc_hi, dm_lo, dm_hi;
          q4k_group_scales(hdr, g, dsc_lo, dsc_hi, dm_lo, dm_hi);
#pragma unroll
          for (int t = 0; t < NT; t++) {
            if (t < a.n_tok) {
              const float2 sx = lds_f2a(saddr + (uint32_t)t * tok_stride);
              const float2 a01 = unpack2(padd2(acc[r][t][0], acc[r][t][1]));
              float y = yacc[r][t];
              y = fmaf(dsc_lo, a01.x, y);
              y = fmaf(dsc_hi, a01.y, y);
              y = fmaf(-dm_lo, sx.x, y);
              yacc[r][t] = fmaf(-dm_hi, sx.y, y);
            }
          }
        }
      }
      waddr += (LPR / 4) * KS_Q4K_BLOCK_BYTES;
      xaddr += LPR * Q4K_XS * 4u;
      saddr += LPR * 8u;
    }
    __syncwarp();
    if (i + (unsigned)S < n_items) {
      if (lane == 0) fence_async_smem();  // the stage was read through the generic proxy
      __syncwarp();
      issue(i + (unsigned)S);
    }
    if (cs + 1 == a.n_cseg) {
      const unsigned grp = gw + k * GW;
      int seg = 0;
      if (a.n_seg > 1 && grp >= a.grp_start[1]) seg = 1;
      if (a.n_seg > 2 && grp >= a.grp_start[2]) seg = 2;
      const unsigned seg_rows = s_rows(a, seg);
      const unsigned row0 = (grp - s_g0(a, seg)) * GROWS;
#pragma unroll
      for (int r = 0; r < SLOTS; r++)
#pragma unroll
        for (int t = 0; t < NT; t++) {
          float v = yacc[r][t];
#pragma unroll
          for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          yacc[r][t] = v;
        }
      if (cl == 0) {
        if (EPI == KS_EPI_GATE_UP) {
#pragma unroll
          for (int r = 0; r < SLOTS; r += 2) {
            const unsigned lrow = row0 + (r >> 1) * RL + rl;
            if (lrow < seg_rows) {
#pragma unroll
              for (int t = 0; t < NT; t++)
                if (t < a.n_tok)
                  act_store<XT>(reinterpret_cast<XT*>(a.y[0]), (size_t)t * seg_rows + lrow, gelu_mul(yacc[r][t], yacc[r + 1][t]));
            }
          }
        } else {
#pragma unroll
          for (int r = 0; r < SLOTS; r++) {
            const unsigned lrow = row0 + r * RL + rl;
            if (lrow < seg_rows) {
#pragma unroll
              for (int t = 0; t < NT; t++)
                if (t < a.n_tok) act_store<XT>(reinterpret_cast<XT*>(s_y(a, seg)), (size_t)t * seg_rows + lrow, yacc[r][t]);
            }
          }
        }
      }
#pragma unroll
      for (int r = 0; r < SLOTS; r++)
#pragma unroll
        for (int t = 0; t < NT; t++) yacc[r][t] = 0.0f;
    }
  }
  if (!ok) {
    // A copy never landed.  Flag it, then give the copies still in flight a bounded chance to land
    // before this block's shared memory goes away.
    if (lane == 0) atomicOr(a.err, 1u);
    for (unsigned j = i; j < n_items && j < i + (unsigned)S; j++) mbar_wait(bars + (j % (unsigned)S) * 8u, (j / (unsigned)S) & 1u);
  }
}

template <int LPR, int R, int NT, int EPI, typename XT>
int launch_q4k(ks_ctx* ctx, const MvsArgs& a, unsigned grid, int nwarps, size_t smem) {
  auto kern = mvs_q4k_kernel<LPR, R, NT, EPI, XT>;
  static bool carve_set[16] = {false};
  if (!carve_set[ctx->device & 15]) {
    // Ask for the largest shared-memory carve-out, so that the blocks of two consecutive kernels can
    // be resident together (the next kernel prefetches its weights while this one computes).
    carve_set[ctx->device & 15] = true;
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  }
  static size_t smem_set[16] = {0};  // per device: largest opt-in size already granted to this kernel
  if (smem > 48 * 1024 && smem > smem_set[ctx->device & 15]) {
    smem_set[ctx->device & 15] = smem;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "matvec: cannot set %zu B shared memory: %s", smem, cudaGetErrorString(e));
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(nwarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
  if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "matvec launch failed: %s", cudaGetErrorString(e));
  return ks_after_launch(ctx, "matvec_q4k_stream");
}

template <int LPR, int R, int EPI, typename XT>
int launch_q4k_nt(ks_ctx* ctx, const MvsArgs& a, unsigned grid, int nwarps, size_t smem) {
  if (a.n_tok == 1) return launch_q4k<LPR, R, 1, EPI, XT>(ctx, a, grid, nwarps, smem);
  if (a.n_tok == 2) return launch_q4k<LPR, R, 2, EPI, XT>(ctx, a, grid, nwarps, smem);
  if (a.n_tok <= 4) return launch_q4k<LPR, R, 4, EPI, XT>(ctx, a, grid, nwarps, smem);
  return launch_q4k<LPR, R, 8, EPI, XT>(ctx, a, grid, nwarps, smem);
}

template <int LPR, int EPI, typename XT>
int launch_q4k_r(ks_ctx* ctx, const MvsArgs& a, int R, unsigned grid, int nwarps, size_t smem) {
  if (R >= 2 && EPI != KS_EPI_GATE_UP) return launch_q4k_nt<LPR, 2, EPI, XT>(ctx, a, grid, nwarps, smem);
  return launch_q4k_nt<LPR, 1, EPI, XT>(ctx, a, grid, nwarps, smem);
}

// -----------------------------------------------------------------------------------------------
// Q6_K.  210-byte blocks leave rows and blocks only 2-byte aligned, so a row group (4 rows) is
// moved as ONE bulk copy (4*row_bytes is a multiple of 16 when a row holds an even number of
// blocks) and the lanes read it back from shared memory at 2-byte granularity: every 32-bit
// field is assembled from the two aligned words around it with one byte permute.
// Lane layout: 8 lanes per row (RL = 4 rows side by side); a unit is 4 byte positions of one
// 128-element half (16 values, 4 int8 scales), as in the direct kernel.
__device__ __forceinline__ uint32_t lds_u32_unaligned2(const unsigned char* p) {
  // p is 2-byte aligned
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  const uint32_t* w = reinterpret_cast<const uint32_t*>(a & ~uintptr_t(3));
  return __byte_perm(w[0], w[1], (a & 2) ? 0x5432 : 0x3210);
}

template <int NT, typename XT>
__global__ void __launch_bounds__(256) mvs_q6k_kernel(const MvsArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int LPR = 8, RL = 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int cl = lane % LPR, rl = lane / LPR;
  const unsigned units = a.cols >> 4;  // 16 units per block
  const unsigned upl = units / LPR;
  const int S = a.stages;
  const unsigned stage_bytes = RL * a.row_bytes;
  const Layout L = make_layout((unsigned)a.n_tok * units * 80u, (stage_bytes + 15u) & ~15u, nwarp, S);
  unsigned char* ring = smem + L.ring_off + (size_t)warp * S * L.stage_bytes;
  const uint32_t bars = smem_u32(smem + L.bar_off) + (uint32_t)(warp * S) * 8u;
  const unsigned total_groups = s_total(a);
  const unsigned gw = blockIdx.x * nwarp + warp, GW = gridDim.x * nwarp;
  const unsigned n_items = gw < total_groups ? (total_groups - gw + GW - 1) / GW : 0;

  auto locate = [&](unsigned i, int& seg, unsigned& row0) {
    const unsigned grp = gw + i * GW;
    seg = 0;
    if (a.n_seg > 1 && grp >= a.grp_start[1]) seg = 1;
    if (a.n_seg > 2 && grp >= a.grp_start[2]) seg = 2;
    row0 = (grp - s_g0(a, seg)) * RL;
  };
  auto issue = [&](unsigned i) {
    if (lane == 0) {
      int seg;
      unsigned row0;
      locate(i, seg, row0);
      const unsigned st = i % (unsigned)S;
      const uint32_t bar = bars + st * 8u;
      mbar_expect_tx(bar, stage_bytes);
      bulk_g2s(smem_u32(ring + (size_t)st * L.stage_bytes), s_w(a, seg) + (size_t)row0 * a.row_bytes, stage_bytes, bar);
    }
  };

  pdl_launch_dependents();  // successors may start (and prefetch their own weights) right away
  if (lane == 0) {
    for (int s = 0; s < S; s++) mbar_init(bars + s * 8u, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  __syncwarp();
  for (unsigned i = 0; i < (unsigned)S && i < n_items; i++) issue(i);

  pdl_wait();
  q6k_stage_x<XT>(smem, reinterpret_cast<const XT*>(a.x), a.cols, a.n_tok);
  __syncthreads();

  bool ok = true;
  unsigned i = 0;
  for (; i < n_items; i++) {
    const unsigned st = i % (unsigned)S;
    if (!mbar_wait(bars + st * 8u, (i / (unsigned)S) & 1u)) {
      ok = false;
      break;
    }
    const unsigned char* row = ring + (size_t)st * L.stage_bytes + (size_t)rl * a.row_bytes;
    float yacc[NT];
#pragma unroll
    for (int t = 0; t < NT; t++) yacc[t] = 0.0f;
    for (unsigned it = 0; it < upl; it++) {
      const unsigned u = cl + LPR * it;
      const unsigned blk = u >> 4, h = (u >> 3) & 1, l4 = u & 7, is = l4 >> 2;
      const unsigned char* bp = row + (size_t)blk * KS_Q6K_BLOCK_BYTES;
      const uint32_t A = lds_u32_unaligned2(bp + 64 * h + 4 * l4);
      const uint32_t B = lds_u32_unaligned2(bp + 64 * h + 32 + 4 * l4);
      const uint32_t H = lds_u32_unaligned2(bp + 128 + 32 * h + 4 * l4);
      const uint32_t s01 = lds_u32_unaligned2(bp + 192 + 8 * h);
      const uint32_t s23 = lds_u32_unaligned2(bp + 196 + 8 * h);
      // scales sc[8h + is + {0,2,4,6}] = byte `is` of each 16-bit half of s01, s23
      const uint32_t Ssel = __byte_perm(s01, s23, is ? 0x7531 : 0x6420);
      const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(bp + 208)));
      const uint32_t v1 = (A & 0x0F0F0F0Fu) | ((H << 4) & 0x30303030u);
      const uint32_t v2 = (B & 0x0F0F0F0Fu) | ((H << 2) & 0x30303030u);
      const uint32_t v3 = ((A >> 4) & 0x0F0F0F0Fu) | (H & 0x30303030u);
      const uint32_t v4 = ((B >> 4) & 0x0F0F0F0Fu) | ((H >> 2) & 0x30303030u);
      const float s1 = (float)(int)(signed char)(Ssel & 0xFFu);
      const float s2 = (float)(int)(signed char)((Ssel >> 8) & 0xFFu);
      const float s3 = (float)(int)(signed char)((Ssel >> 16) & 0xFFu);
      const float s4 = (float)(int)(signed char)(Ssel >> 24);
#pragma unroll
      for (int t = 0; t < NT; t++) {
        if (t < a.n_tok) {
          const float4* xq = reinterpret_cast<const float4*>(smem) + (size_t)t * units * 5;
          const float4 sx = lds_f4(xq + (size_t)4 * units + u);
          u64 xa, xb;
          lds_p2(xq + u, xa, xb);
          float p = s1 * (q6_word_p(v1, xa, xb) - 32.0f * sx.x);
          lds_p2(xq + (size_t)units + u, xa, xb);
          p += s2 * (q6_word_p(v2, xa, xb) - 32.0f * sx.y);
          lds_p2(xq + (size_t)2 * units + u, xa, xb);
          p += s3 * (q6_word_p(v3, xa, xb) - 32.0f * sx.z);
          lds_p2(xq + (size_t)3 * units + u, xa, xb);
          p += s4 * (q6_word_p(v4, xa, xb) - 32.0f * sx.w);
          yacc[t] += d * p;
        }
      }
    }
    __syncwarp();
    if (i + (unsigned)S < n_items) {
      if (lane == 0) fence_async_smem();
      __syncwarp();
      issue(i + (unsigned)S);
    }
    int seg;
    unsigned row0;
    locate(i, seg, row0);
    const unsigned seg_rows = s_rows(a, seg);
#pragma unroll
    for (int t = 0; t < NT; t++) {
      float v = yacc[t];
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (cl == 0 && t < a.n_tok && row0 + rl < seg_rows)
        act_store<XT>(reinterpret_cast<XT*>(s_y(a, seg)), (size_t)t * seg_rows + row0 + rl, v);
    }
  }
  if (!ok) {
    if (lane == 0) atomicOr(a.err, 1u);
    for (unsigned j = i; j < n_items && j < i + (unsigned)S; j++) mbar_wait(bars + (j % (unsigned)S) * 8u, (j / (unsigned)S) & 1u);
  }
}

template <int NT, typename XT>
int launch_q6k(ks_ctx* ctx, const MvsArgs& a, unsigned grid, int nwarps, size_t smem) {
  auto kern = mvs_q6k_kernel<NT, XT>;
  static bool carve_set[16] = {false};
  if (!carve_set[ctx->device & 15]) {
    // Ask for the largest shared-memory carve-out, so that the blocks of two consecutive kernels can
    // be resident together (the next kernel prefetches its weights while this one computes).
    carve_set[ctx->device & 15] = true;
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  }
  static size_t smem_set[16] = {0};  // per device: largest opt-in size already granted to this kernel
  if (smem > 48 * 1024 && smem > smem_set[ctx->device & 15]) {
    smem_set[ctx->device & 15] = smem;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "matvec: cannot set %zu B shared memory: %s", smem, cudaGetErrorString(e));
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(nwarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
  if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "matvec launch failed: %s", cudaGetErrorString(e));
  return ks_after_launch(ctx, "matvec_q6k_stream");
}

}  // namespace

// Streamed Q4_K launch; plan fields: nr = rows per lane (1 or 2), nwarps, ctas_per_sm,
// variant bits 8..15 = stages (0 = default 3), bits 16..23 = blocks per column segment (0 = auto).
int ks_launch_matvec_stream_q4k(ks_ctx* ctx, const ks_mv_seg* segs, int n_seg, ks_mv_epilogue epi, size_t cols,
                                ks_dtype act, const void* x, int n_tok, const ks_plan* plan, const ks_mv_pro* pro) {
  const unsigned nb = (unsigned)(cols / 256);
  const int LPR = (nb % 2 == 0) ? 8 : 4;
  const int RL = 32 / LPR;
  int R = (plan && plan->nr > 0) ? plan->nr : 1;
  if (epi == KS_EPI_GATE_UP || n_tok > 2) R = 1;
  R = R >= 2 ? 2 : 1;
  const int mats = epi == KS_EPI_GATE_UP ? 2 : 1;
  int nwarps = (plan && plan->nwarps > 0) ? plan->nwarps : 8;
  if (nwarps > 8) nwarps = 8;
  int stages = plan ? (plan->variant >> 8) & 0xFF : 0;
  const bool auto_stages = stages <= 0;
  if (stages <= 0) stages = 3;
  unsigned seg_blocks = plan ? (unsigned)((plan->variant >> 16) & 0xFF) : 0;
  const unsigned step = LPR == 8 ? 2 : 1;  // segment units must divide among LPR lanes
  if (seg_blocks == 0 || nb % seg_blocks != 0 || seg_blocks % step != 0) {
    seg_blocks = step;
    for (unsigned c = step; c <= nb && c <= 12; c += step)
      if (nb % c == 0) seg_blocks = c;
  }
  MvsArgs a{};
  a.n_seg = (epi == KS_EPI_GATE_UP) ? 1 : n_seg;
  a.cols = (unsigned)cols;
  a.row_bytes = nb * KS_Q4K_BLOCK_BYTES;
  a.x = x;
  a.n_tok = n_tok;
  a.seg_blocks = seg_blocks;
  a.n_cseg = nb / seg_blocks;
  a.err = (unsigned*)ctx->ws + KS_WS_ERR_WORD;
  if (pro) a.pro = *pro;
  if (a.pro.mode != KS_PRO_NONE) {
    if (nwarps < (int)((cols + 511) / 512)) nwarps = (int)((cols + 511) / 512);  // 16 elements per thread
    KS_REQUIRE(ctx, nwarps <= 8, "matvec: fused norm needs cols <= 4096");
    const uintptr_t al = act == KS_F32 ? 15 : 7;
    KS_REQUIRE(ctx, (((uintptr_t)x | (uintptr_t)a.pro.w) & al) == 0, "matvec: fused norm needs aligned vectors");
    if (a.pro.mode == KS_PRO_ADD_NORM)
      KS_REQUIRE(ctx, a.pro.out_x != x && (((uintptr_t)a.pro.y | (uintptr_t)a.pro.w_post | (uintptr_t)a.pro.out_x) & al) == 0,
                 "matvec: fused residual update must not alias its input and needs aligned vectors");
  }
  // a fused norm holds the input vector in registers, 16 elements per thread: never run it with fewer warps
  const int min_warps = a.pro.mode != KS_PRO_NONE ? (int)((cols + 511) / 512) : 1;
  const unsigned grows = (unsigned)(RL * R);
  unsigned g0 = 0;
  for (int s = 0; s < n_seg; s++) {
    a.W[s] = segs[s].W;
    a.y[s] = segs[s].y;
    a.rows[s] = segs[s].rows;
  }
  for (int s = 0; s < a.n_seg; s++) {
    a.grp_start[s] = g0;
    g0 += (a.rows[s] + grows - 1) / grows;
  }
  a.grp_start[a.n_seg] = g0;
  const unsigned x_bytes = (unsigned)n_tok * (unsigned)(cols / 64) * Q4K_XTOK * 4u;
  const unsigned stage_bytes = (unsigned)(RL * R * mats) * seg_blocks * KS_Q4K_BLOCK_BYTES;
  const int cps = (plan && plan->ctas_per_sm > 0) ? plan->ctas_per_sm : 1;
  if (auto_stages) {
    // Enough stages for a warp to start ALL of its copies before it waits for its input (the whole
    // weight stream of a decode-sized matrix is then in flight while the previous kernel still
    // runs), inside HALF of an SM's shared memory so that the blocks of two consecutive kernels fit
    // side by side: fewer stages first, then fewer warps (not below 4).
    const unsigned half = 108u * 1024u;
    const bool pick_warps = !(plan && plan->nwarps > 0);
    for (;;) {
      const unsigned gw_total = (unsigned)(ctx->sm_count * cps * nwarps);
      const unsigned items = ((g0 + gw_total - 1) / gw_total) * a.n_cseg;
      stages = (int)(items < 2 ? 2 : items > 8 ? 8 : items);
      while (stages > 2 && make_layout(x_bytes, stage_bytes, nwarps, stages).total > half) stages--;
      if (make_layout(x_bytes, stage_bytes, nwarps, stages).total <= half || !pick_warps || nwarps <= 4 || nwarps <= min_warps) break;
      nwarps -= 1;
    }
  }
  // fit the rings into the shared memory budget: fewer stages first, then fewer warps
  Layout L = make_layout(x_bytes, stage_bytes, nwarps, stages);
  const unsigned budget = (unsigned)ctx->smem_optin;
  while (L.total > budget && stages > 2) L = make_layout(x_bytes, stage_bytes, nwarps, --stages);
  while (L.total > budget && nwarps > min_warps) L = make_layout(x_bytes, stage_bytes, --nwarps, stages);
  KS_REQUIRE(ctx, L.total <= budget, "matvec: needs %u B of shared memory (limit %u)", L.total, budget);
  a.stages = stages;
  unsigned grid = (g0 + nwarps - 1) / nwarps;
  const unsigned cap = (unsigned)(ctx->sm_count * cps);
  if (grid > cap) grid = cap;
#define KS_GO(LPR_)                                                                                                   \
  do {                                                                                                                \
    if (epi == KS_EPI_GATE_UP)                                                                                        \
      return act == KS_F32 ? launch_q4k_r<LPR_, KS_EPI_GATE_UP, float>(ctx, a, R, grid, nwarps, L.total)              \
                           : launch_q4k_r<LPR_, KS_EPI_GATE_UP, __half>(ctx, a, R, grid, nwarps, L.total);            \
    return act == KS_F32 ? launch_q4k_r<LPR_, KS_EPI_PLAIN, float>(ctx, a, R, grid, nwarps, L.total)                  \
                         : launch_q4k_r<LPR_, KS_EPI_PLAIN, __half>(ctx, a, R, grid, nwarps, L.total);                \
  } while (0)
  if (LPR == 8) KS_GO(8);
  KS_GO(4);
#undef KS_GO
}

// Streamed Q6_K launch.  Returns 1 (not an error) when the shape cannot be streamed -- a row holds
// an odd number of blocks, a segment's row count is not a multiple of 4, or a row group does not
// fit a stage -- and the caller falls back to the direct-load kernel.
int ks_launch_matvec_stream_q6k(ks_ctx* ctx, const ks_mv_seg* segs, int n_seg, size_t cols, ks_dtype act, const void* x,
                                int n_tok, const ks_plan* plan) {
  const unsigned nb = (unsigned)(cols / 256);
  const unsigned row_bytes = nb * KS_Q6K_BLOCK_BYTES;
  if (nb % 2) return 1;
  if (cols / 16 % 8) return 1;
  for (int s = 0; s < n_seg; s++)
    if (segs[s].rows % 4 || ((uintptr_t)segs[s].W & 15)) return 1;
  if (4u * row_bytes > 20480u) return 1;
  int nwarps = (plan && plan->nwarps > 0) ? plan->nwarps : 8;
  if (nwarps > 8) nwarps = 8;
  int stages = plan ? (plan->variant >> 8) & 0xFF : 0;
  if (stages <= 0) stages = 3;
  MvsArgs a{};
  a.n_seg = n_seg;
  a.cols = (unsigned)cols;
  a.row_bytes = row_bytes;
  a.x = x;
  a.n_tok = n_tok;
  a.err = (unsigned*)ctx->ws + KS_WS_ERR_WORD;
  unsigned g0 = 0;
  for (int s = 0; s < n_seg; s++) {
    a.W[s] = segs[s].W;
    a.y[s] = segs[s].y;
    a.rows[s] = segs[s].rows;
    a.grp_start[s] = g0;
    g0 += segs[s].rows / 4;
  }
  a.grp_start[n_seg] = g0;
  const unsigned x_bytes = (unsigned)n_tok * (unsigned)(cols / 16) * 80u;
  const unsigned stage_bytes = (4u * row_bytes + 15u) & ~15u;
  Layout L = make_layout(x_bytes, stage_bytes, nwarps, stages);
  const unsigned budget = (unsigned)ctx->smem_optin;
  while (L.total > budget && stages > 2) L = make_layout(x_bytes, stage_bytes, nwarps, --stages);
  while (L.total > budget && nwarps > 1) L = make_layout(x_bytes, stage_bytes, --nwarps, stages);
  if (L.total > budget) return 1;
  a.stages = stages;
  const int cps = (plan && plan->ctas_per_sm > 0) ? plan->ctas_per_sm : 1;
  unsigned grid = (g0 + nwarps - 1) / nwarps;
  const unsigned cap = (unsigned)(ctx->sm_count * cps);
  if (grid > cap) grid = cap;
#define KS_GO6(T_)                                                              \
  do {                                                                          \
    if (n_tok == 1) return launch_q6k<1, T_>(ctx, a, grid, nwarps, L.total);    \
    if (n_tok == 2) return launch_q6k<2, T_>(ctx, a, grid, nwarps, L.total);    \
    if (n_tok <= 4) return launch_q6k<4, T_>(ctx, a, grid, nwarps, L.total);    \
    return launch_q6k<8, T_>(ctx, a, grid, nwarps, L.total);                    \
  } while (0)
  if (act == KS_F32) KS_GO6(float);
  KS_GO6(__half);
#undef KS_GO6
}

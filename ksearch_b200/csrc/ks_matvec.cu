// Dequant-fused matvec for GGUF Q4_K / Q6_K weights on sm_100a.
//
// Replaces the reference's cooperative GEMV lowerings
//   crates/ksearch_codegen/src/lower.rs:1763-2082  (Q4_K, 4 rows per simdgroup)
//   crates/ksearch_codegen/src/lower.rs:2086-2472  (Q6_K)
//   crates/ksearch_codegen/src/lower.rs:2673-2968  (gate || up + GELU*mul)
//   crates/ksearch_codegen/src/lower.rs:3343-3464  (fused Q/K/V)
// and computes what crates/ksearch_gguf/src/gguf_impl.rs:690-721 / 761-791
// followed by a dot product computes.
//
// Arithmetic.  A Q4_K value is d*sc*n - dmin*m with n a 4-bit integer, so per
// 32-element sub-block   sum_i w_i x_i = (d*sc) * sum_i n_i x_i - (dmin*m) * sum_i x_i.
// sum_i x_i does not depend on the row: it is computed once per launch while x
// is staged in shared memory.  n_i is turned into an f32 without a shift or a
// convert: (word & (0xF << 4k)) | 0x4B000000 is the float 2^23 + n*16^k, one
// exact subtraction of 2^23 leaves n*16^k, and x is staged pre-divided by 16^k
// (exact, a power of two).  Products and sums are f32 (FMA), paired as f32x2.
// Q6_K works the same way on 6-bit values (q-32), the -32 folded into sum_i x_i.
#include "ks_mv_common.cuh"

namespace {

template <int LPR, int R, int NT, int EPI, typename XT, typename YT>
__global__ void __launch_bounds__(256) mv_q4k_kernel(const MvArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  constexpr int RL = 32 / LPR;       // rows side by side in a warp
  constexpr int TILE = RL * R;       // row slots per warp tile
  constexpr int LROWS = (EPI == KS_EPI_GATE_UP) ? TILE / 2 : TILE;  // logical rows per tile
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int cl = lane % LPR, rl = lane / LPR;
  const unsigned units = a.cols >> 6;
  const unsigned upl = units / LPR;  // units per lane (host guarantees divisibility)
  const int g = cl & 3;              // LPR is a multiple of 4, so the group index is fixed per lane
  const unsigned total_tiles = total_tiles_of(a);

  unsigned tile = blockIdx.x * nwarp + warp;
  const unsigned tile_step = gridDim.x * nwarp;

  // Row pointers of the first tile are resolved and its first loads issued before x is staged,
  // so the weight stream starts while x is still on its way.
  q4k_stage_x<XT>(smem, reinterpret_cast<const XT*>(a.x), a.cols, a.n_tok);
  __syncthreads();

  for (; tile < total_tiles; tile += tile_step) {
    int seg = 0;
    if (a.n_seg > 1 && tile >= a.tile_start[1]) seg = 1;
    if (a.n_seg > 2 && tile >= a.tile_start[2]) seg = 2;
    const unsigned ltile = tile - seg_tile0(a, seg);
    const unsigned seg_rows = seg_rows_of(a, seg);

    const uint8_t* rowp[R];
    unsigned lrow[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
      unsigned lr;
      const uint8_t* base;
      if (EPI == KS_EPI_GATE_UP) {
        lr = ltile * LROWS + (r >> 1) * RL + rl;
        base = (r & 1) ? a.W[1] : a.W[0];
      } else {
        lr = ltile * LROWS + r * RL + rl;
        base = seg_w(a, seg);
      }
      lrow[r] = lr;
      const unsigned lrc = lr < seg_rows ? lr : seg_rows - 1;  // clamp loads, mask the store
      rowp[r] = base + (size_t)lrc * a.row_bytes;
    }

    float yacc[R][NT];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
      for (int t = 0; t < NT; t++) yacc[r][t] = 0.0f;

    for (unsigned it = 0; it < upl; it++) {
      const unsigned u = cl + LPR * it;
      const unsigned blk = u >> 2;
      uint4 hdr[R], qa[R], qb[R];
#pragma unroll
      for (int r = 0; r < R; r++) {
        const uint8_t* bp = rowp[r] + (size_t)blk * KS_Q4K_BLOCK_BYTES;
        hdr[r] = ldg_stream16(bp);
        qa[r] = ldg_stream16(bp + 16 + g * 32);
        qb[r] = ldg_stream16(bp + 32 + g * 32);
      }
#pragma unroll
      for (int t = 0; t < NT; t++) {
        if (t < a.n_tok) {
          const float* xp = reinterpret_cast<const float*>(smem) + (size_t)t * units * Q4K_XTOK;
          const float2 sx = reinterpret_cast<const float2*>(xp + (size_t)units * Q4K_XS)[u];
          const float4* xv = reinterpret_cast<const float4*>(xp + (size_t)u * Q4K_XS);
          float2 acc[R][2];
#pragma unroll
          for (int r = 0; r < R; r++) acc[r][0] = acc[r][1] = make_float2(0.0f, 0.0f);
#pragma unroll
          for (int half = 0; half < 2; half++) {
            float4 xf[8];  // 16 (lo, hi) pairs: l = 16*half .. 16*half+15
#pragma unroll
            for (int i = 0; i < 8; i++) xf[i] = xv[half * 8 + i];
#pragma unroll
            for (int r = 0; r < R; r++) {
              const uint4 q = half ? qb[r] : qa[r];
              const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
              for (int j = 0; j < 4; j++) {
                q4_word(w[j], make_float2(xf[2 * j].x, xf[2 * j].y), make_float2(xf[2 * j].z, xf[2 * j].w),
                        make_float2(xf[2 * j + 1].x, xf[2 * j + 1].y), make_float2(xf[2 * j + 1].z, xf[2 * j + 1].w),
                        acc[r][0], acc[r][1]);
              }
            }
          }
#pragma unroll
          for (int r = 0; r < R; r++) {
            float dsc_lo, dsc_hi, dm_lo, dm_hi;
            q4k_group_scales(hdr[r], g, dsc_lo, dsc_hi, dm_lo, dm_hi);
            const float s_lo = acc[r][0].x + acc[r][1].x;
            const float s_hi = acc[r][0].y + acc[r][1].y;
            yacc[r][t] += (dsc_lo * s_lo + dsc_hi * s_hi) - (dm_lo * sx.x + dm_hi * sx.y);
          }
        }
      }
    }

    // reduce over the LPR lanes of each row
#pragma unroll
    for (int r = 0; r < R; r++)
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
        for (int r = 0; r < R; r += 2) {
          if (lrow[r] < seg_rows) {
#pragma unroll
            for (int t = 0; t < NT; t++)
              if (t < a.n_tok)
                act_store<YT>(reinterpret_cast<YT*>(a.y[0]), (size_t)t * seg_rows + lrow[r],
                              gelu_mul(yacc[r][t], yacc[r + 1][t]));
          }
        }
      } else {
#pragma unroll
        for (int r = 0; r < R; r++) {
          if (lrow[r] < seg_rows) {
#pragma unroll
            for (int t = 0; t < NT; t++)
              if (t < a.n_tok)
                act_store<YT>(reinterpret_cast<YT*>(seg_y(a, seg)), (size_t)t * seg_rows + lrow[r], yacc[r][t]);
          }
        }
      }
    }
  }
}

// -------------------------------------------------------------------------------------------
// Q6_K.  A unit is four consecutive byte positions l = 4*l4..4*l4+3 of one 128-element half h:
// one word of ql[l], one of ql[l+32], one of qh[l] -> 16 values under 4 int8 scales
// (gguf_impl.rs:761-791).  32 lanes share a row.  Blocks are only 2-byte aligned (210 bytes).
// Shared memory per unit: 16 floats xq[k][j] = x[128h + 32k + 4*l4 + j] * p(j), p = 1, 2^-8, 2^-16, 1
// and 4 floats sx[k] = sum_j x[...].
// -------------------------------------------------------------------------------------------
template <int R, int NT, typename XT, typename YT>
__global__ void __launch_bounds__(256) mv_q6k_kernel(const MvArgs a) {
  extern __shared__ __align__(16) unsigned char smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const unsigned units = a.cols >> 4;
  const unsigned total_tiles = total_tiles_of(a);

  q6k_stage_x<XT>(smem, reinterpret_cast<const XT*>(a.x), a.cols, a.n_tok);
  __syncthreads();

  for (unsigned tile = blockIdx.x * nwarp + warp; tile < total_tiles; tile += gridDim.x * nwarp) {
    int seg = 0;
    if (a.n_seg > 1 && tile >= a.tile_start[1]) seg = 1;
    if (a.n_seg > 2 && tile >= a.tile_start[2]) seg = 2;
    const unsigned ltile = tile - seg_tile0(a, seg);
    const unsigned seg_rows = seg_rows_of(a, seg);
    const uint8_t* rowp[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
      unsigned lr = ltile * R + r;
      lr = lr < seg_rows ? lr : seg_rows - 1;
      rowp[r] = seg_w(a, seg) + (size_t)lr * a.row_bytes;
    }
    float yacc[R][NT];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
      for (int t = 0; t < NT; t++) yacc[r][t] = 0.0f;

    for (unsigned u = lane; u < units; u += 32) {
      const unsigned blk = u >> 4, h = (u >> 3) & 1, l4 = u & 7;
      const unsigned is = l4 >> 2;
      uint32_t A[R], B[R], H[R], S[R], D[R];
#pragma unroll
      for (int r = 0; r < R; r++) {
        const uint8_t* bp = rowp[r] + (size_t)blk * KS_Q6K_BLOCK_BYTES;
        A[r] = ldg_stream_u16x2(bp + 64 * h + 4 * l4);
        B[r] = ldg_stream_u16x2(bp + 64 * h + 32 + 4 * l4);
        H[r] = ldg_stream_u16x2(bp + 128 + 32 * h + 4 * l4);
        // scales sc[8h + is + {0,2,4,6}]: bytes `is` of the four 16-bit words at 192 + 8h
        const uint32_t s01 = ldg_stream_u16x2(bp + 192 + 8 * h);
        const uint32_t s23 = ldg_stream_u16x2(bp + 192 + 8 * h + 4);
        const uint32_t sh = is * 8;
        S[r] = ((s01 >> sh) & 0xFFu) | (((s01 >> (16 + sh)) & 0xFFu) << 8) | (((s23 >> sh) & 0xFFu) << 16) |
               (((s23 >> (16 + sh)) & 0xFFu) << 24);
        D[r] = ldg_stream_u16(bp + 208);
      }
#pragma unroll
      for (int t = 0; t < NT; t++) {
        if (t < a.n_tok) {
          const float4* xq = reinterpret_cast<const float4*>(smem) + (size_t)t * units * 5;
          const float4 sx = xq[(size_t)4 * units + u];
          const float4 x1 = xq[u], x2 = xq[(size_t)units + u], x3 = xq[(size_t)2 * units + u], x4 = xq[(size_t)3 * units + u];
#pragma unroll
          for (int r = 0; r < R; r++) {
            const uint32_t v1 = (A[r] & 0x0F0F0F0Fu) | ((H[r] << 4) & 0x30303030u);
            const uint32_t v2 = (B[r] & 0x0F0F0F0Fu) | ((H[r] << 2) & 0x30303030u);
            const uint32_t v3 = ((A[r] >> 4) & 0x0F0F0F0Fu) | (H[r] & 0x30303030u);
            const uint32_t v4 = ((B[r] >> 4) & 0x0F0F0F0Fu) | ((H[r] >> 2) & 0x30303030u);
            const float d = __half2float(__ushort_as_half((unsigned short)D[r]));
            const float s1 = (float)(int)(signed char)(S[r] & 0xFFu);
            const float s2 = (float)(int)(signed char)((S[r] >> 8) & 0xFFu);
            const float s3 = (float)(int)(signed char)((S[r] >> 16) & 0xFFu);
            const float s4 = (float)(int)(signed char)(S[r] >> 24);
            float p = s1 * (q6_word(v1, x1) - 32.0f * sx.x);
            p += s2 * (q6_word(v2, x2) - 32.0f * sx.y);
            p += s3 * (q6_word(v3, x3) - 32.0f * sx.z);
            p += s4 * (q6_word(v4, x4) - 32.0f * sx.w);
            yacc[r][t] += d * p;
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
      for (int t = 0; t < NT; t++) {
        float v = yacc[r][t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && t < a.n_tok && ltile * R + r < seg_rows)
          act_store<YT>(reinterpret_cast<YT*>(seg_y(a, seg)), (size_t)t * seg_rows + ltile * R + r, v);
      }
  }
}

// ---- host-side dispatch --------------------------------------------------------------------

template <int LPR, int R, int NT, int EPI, typename T>
int launch_q4k_t(ks_ctx* ctx, const MvArgs& a, int grid, int threads, size_t smem) {
  auto kern = mv_q4k_kernel<LPR, R, NT, EPI, T, T>;
  static size_t smem_set[16] = {0};  // per device: largest opt-in size already granted to this kernel
  if (smem > 48 * 1024 && smem > smem_set[ctx->device & 15]) {
    smem_set[ctx->device & 15] = smem;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "matvec: cannot set %zu B shared memory: %s", smem, cudaGetErrorString(e));
  }
  kern<<<grid, threads, smem, ctx->stream>>>(a);
  return ks_after_launch(ctx, "matvec_q4k");
}

template <int LPR, int R, int EPI, typename T>
int launch_q4k_nt(ks_ctx* ctx, const MvArgs& a, int grid, int threads, size_t smem) {
  if (a.n_tok == 1) return launch_q4k_t<LPR, R, 1, EPI, T>(ctx, a, grid, threads, smem);
  if (a.n_tok == 2) return launch_q4k_t<LPR, R, 2, EPI, T>(ctx, a, grid, threads, smem);
  if (a.n_tok <= 4) return launch_q4k_t<LPR, R, 4, EPI, T>(ctx, a, grid, threads, smem);
  return launch_q4k_t<LPR, R, 8, EPI, T>(ctx, a, grid, threads, smem);
}

template <int LPR, int EPI, typename T>
int launch_q4k_r(ks_ctx* ctx, const MvArgs& a, int R, int grid, int threads, size_t smem) {
  if (EPI == KS_EPI_GATE_UP) {
    if (R >= 4) return launch_q4k_nt<LPR, 4, EPI, T>(ctx, a, grid, threads, smem);
    return launch_q4k_nt<LPR, 2, EPI, T>(ctx, a, grid, threads, smem);
  }
  if (R >= 4) return launch_q4k_nt<LPR, 4, EPI, T>(ctx, a, grid, threads, smem);
  if (R >= 2) return launch_q4k_nt<LPR, 2, EPI, T>(ctx, a, grid, threads, smem);
  return launch_q4k_nt<LPR, 1, EPI, T>(ctx, a, grid, threads, smem);
}

template <int R, typename T>
int launch_q6k_nt(ks_ctx* ctx, const MvArgs& a, int grid, int threads, size_t smem) {
#define KS_Q6_LAUNCH(NT_)                                                                           \
  do {                                                                                              \
    auto kern = mv_q6k_kernel<R, NT_, T, T>;                                                        \
    static size_t smem_set[16] = {0};                                                               \
    if (smem > 48 * 1024 && smem > smem_set[ctx->device & 15]) {                                    \
      smem_set[ctx->device & 15] = smem;                                                            \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "matvec: cannot set shared memory: %s", cudaGetErrorString(e)); \
    }                                                                                               \
    kern<<<grid, threads, smem, ctx->stream>>>(a);                                                  \
    return ks_after_launch(ctx, "matvec_q6k");                                                      \
  } while (0)
  if (a.n_tok == 1) KS_Q6_LAUNCH(1);
  if (a.n_tok == 2) KS_Q6_LAUNCH(2);
  if (a.n_tok <= 4) KS_Q6_LAUNCH(4);
  KS_Q6_LAUNCH(8);
#undef KS_Q6_LAUNCH
}

}  // namespace

bool ks_matvec_can_fuse_pro(ks_dtype wdtype, size_t cols) { return wdtype == KS_Q4K && cols % 256 == 0 && cols <= 4096; }

int ks_launch_matvec(ks_ctx* ctx, ks_dtype wdtype, const ks_mv_seg* segs, int n_seg, ks_mv_epilogue epi,
                     size_t cols, ks_dtype act, const void* x, int n_tok, const ks_mv_plan* plan, const ks_mv_pro* pro) {
  KS_REQUIRE(ctx, wdtype == KS_Q4K || wdtype == KS_Q6K, "matvec: weight dtype %d not supported (Q4K, Q6K)", (int)wdtype);
  KS_REQUIRE(ctx, ks_is_act(act), "matvec: activation dtype must be F32 or F16");
  KS_REQUIRE(ctx, n_seg >= 1 && n_seg <= 3, "matvec: 1..3 weight segments");
  KS_REQUIRE(ctx, cols > 0 && cols % 256 == 0, "matvec: cols=%zu must be a positive multiple of 256", cols);
  KS_REQUIRE(ctx, cols <= 65536, "matvec: cols=%zu exceeds 65536", cols);
  KS_REQUIRE(ctx, n_tok >= 1 && n_tok <= 8, "matvec: n_tok=%d outside 1..8 (larger batches belong to the prefill GEMM)", n_tok);
  KS_REQUIRE(ctx, epi == KS_EPI_PLAIN || (wdtype == KS_Q4K && n_seg == 2 && segs[0].rows == segs[1].rows),
             "matvec: gate/up epilogue needs two Q4K matrices of equal rows");
  for (int s = 0; s < n_seg; s++) {
    KS_REQUIRE(ctx, segs[s].rows > 0, "matvec: rows must be > 0");
    KS_REQUIRE(ctx, ((uintptr_t)segs[s].W & (wdtype == KS_Q4K ? 15 : 1)) == 0, "matvec: weight pointer misaligned");
  }

  if (ctx->has_override) {
    plan = &ctx->override_plan;
  } else if (!plan && !ctx->plans.empty()) {
    // the planner's table: op_rowsxcols[_bN]
    size_t total = 0;
    for (int s = 0; s < n_seg; s++) total += segs[s].rows;
    const char* op = epi == KS_EPI_GATE_UP ? "gu_q4k" : n_seg == 3 ? (wdtype == KS_Q4K ? "qkv_q4k" : "qkv_q6k")
                                                                  : (wdtype == KS_Q4K ? "mv_q4k" : "mv_q6k");
    plan = ks_plan_lookup(ctx, op, epi == KS_EPI_GATE_UP ? segs[0].rows : total, cols, n_tok);
  }
  if (pro && pro->mode != KS_PRO_NONE) {
    KS_REQUIRE(ctx, ks_matvec_can_fuse_pro(wdtype, cols), "matvec: no fused norm prologue for dtype %d, cols=%zu", (int)wdtype, cols);
    return ks_launch_matvec_stream_q4k(ctx, segs, n_seg, epi, cols, act, x, n_tok, plan, pro);
  }
  if (wdtype == KS_Q4K && plan && (plan->variant & 0xFF) == 3) {
    const int rc = ks_launch_matvec_q4k_fx(ctx, segs, n_seg, epi, cols, act, x, n_tok, plan);
    if (rc != 1) return rc;
  }
  if (wdtype == KS_Q4K && (!plan || (plan->variant & 0xFF) == 0 || (plan->variant & 0xFF) == 3))
    return ks_launch_matvec_stream_q4k(ctx, segs, n_seg, epi, cols, act, x, n_tok, plan, nullptr);
  if (wdtype == KS_Q6K && plan && (plan->variant & 0xFF) == 4) {
    const int rc = ks_launch_matvec_q6k_ring(ctx, segs, n_seg, cols, act, x, n_tok, plan);
    if (rc != 1) return rc;
  }
  if (wdtype == KS_Q6K && (!plan || (plan->variant & 0xFF) == 2 || (plan->variant & 0xFF) == 4)) {  // also the default: single-token calls take it, others fall through
    const int rc = ks_launch_matvec_q6k_fx(ctx, segs, n_seg, cols, act, x, n_tok, plan);
    if (rc != 1) return rc;
  }
  if (wdtype == KS_Q6K && (!plan || (plan->variant & 0xFF) == 0)) {
    const int rc = ks_launch_matvec_stream_q6k(ctx, segs, n_seg, cols, act, x, n_tok, plan);
    if (rc != 1) return rc;
  }
  MvArgs a{};
  a.n_seg = (epi == KS_EPI_GATE_UP) ? 1 : n_seg;
  a.cols = (unsigned)cols;
  a.nb = (unsigned)(cols / 256);
  a.row_bytes = (unsigned)(a.nb * ks_block_bytes(wdtype));
  a.x = x;
  a.n_tok = n_tok;
  for (int s = 0; s < n_seg; s++) {
    a.W[s] = segs[s].W;
    a.y[s] = segs[s].y;
    a.rows[s] = segs[s].rows;
  }

  const int nwarps = (plan && plan->nwarps > 0) ? plan->nwarps : 8;
  const int threads = nwarps * 32;
  KS_REQUIRE(ctx, nwarps >= 1 && nwarps <= 8, "matvec: plan.nwarps outside 1..8");

  if (wdtype == KS_Q4K) {
    const unsigned units = (unsigned)(cols / 64);
    const int LPR = (units % 32 == 0) ? 32 : (units % 16 == 0) ? 16 : (units % 8 == 0) ? 8 : 4;
    int R = (plan && plan->nr > 0) ? plan->nr : (n_tok > 2 ? 2 : 4);
    if (epi == KS_EPI_GATE_UP && R < 2) R = 2;
    R = R >= 4 ? 4 : R >= 2 ? 2 : 1;
    const unsigned RL = 32 / LPR;
    const unsigned lrows = (epi == KS_EPI_GATE_UP) ? RL * R / 2 : RL * R;
    unsigned t0 = 0;
    for (int s = 0; s < a.n_seg; s++) {
      a.tile_start[s] = t0;
      t0 += (a.rows[s] + lrows - 1) / lrows;
    }
    a.tile_start[a.n_seg] = t0;
    const size_t smem = (size_t)n_tok * units * Q4K_XTOK * sizeof(float);
    KS_REQUIRE(ctx, smem <= ctx->smem_optin, "matvec: x needs %zu B of shared memory (limit %zu); split the batch", smem, ctx->smem_optin);
    const int cps = (plan && plan->ctas_per_sm > 0) ? plan->ctas_per_sm : 2;
    unsigned grid = (t0 + nwarps - 1) / nwarps;
    const unsigned cap = (unsigned)(ctx->sm_count * cps);
    if (grid > cap) grid = cap;
#define KS_Q4_DISPATCH(LPR_)                                                                              \
  do {                                                                                                    \
    if (epi == KS_EPI_GATE_UP) {                                                                          \
      return act == KS_F32 ? launch_q4k_r<LPR_, KS_EPI_GATE_UP, float>(ctx, a, R, grid, threads, smem)    \
                           : launch_q4k_r<LPR_, KS_EPI_GATE_UP, __half>(ctx, a, R, grid, threads, smem);  \
    }                                                                                                     \
    return act == KS_F32 ? launch_q4k_r<LPR_, KS_EPI_PLAIN, float>(ctx, a, R, grid, threads, smem)        \
                         : launch_q4k_r<LPR_, KS_EPI_PLAIN, __half>(ctx, a, R, grid, threads, smem);      \
  } while (0)
    if (LPR == 32) KS_Q4_DISPATCH(32);
    if (LPR == 16) KS_Q4_DISPATCH(16);
    if (LPR == 8) KS_Q4_DISPATCH(8);
    KS_Q4_DISPATCH(4);
#undef KS_Q4_DISPATCH
  }

  // Q6_K
  const unsigned units = (unsigned)(cols / 16);
  int R = (plan && plan->nr > 0) ? plan->nr : 2;
  R = R >= 4 ? 4 : R >= 2 ? 2 : 1;
  unsigned t0 = 0;
  for (int s = 0; s < a.n_seg; s++) {
    a.tile_start[s] = t0;
    t0 += (a.rows[s] + R - 1) / R;
  }
  a.tile_start[a.n_seg] = t0;
  const size_t smem = (size_t)n_tok * units * 20 * sizeof(float);
  KS_REQUIRE(ctx, smem <= ctx->smem_optin, "matvec: x needs %zu B of shared memory (limit %zu); split the batch", smem, ctx->smem_optin);
  const int cps = (plan && plan->ctas_per_sm > 0) ? plan->ctas_per_sm : 4;
  unsigned grid = (t0 + nwarps - 1) / nwarps;
  const unsigned cap = (unsigned)(ctx->sm_count * cps);
  if (grid > cap) grid = cap;
  if (act == KS_F32) {
    if (R == 4) return launch_q6k_nt<4, float>(ctx, a, grid, threads, smem);
    if (R == 2) return launch_q6k_nt<2, float>(ctx, a, grid, threads, smem);
    return launch_q6k_nt<1, float>(ctx, a, grid, threads, smem);
  }
  if (R == 4) return launch_q6k_nt<4, __half>(ctx, a, grid, threads, smem);
  if (R == 2) return launch_q6k_nt<2, __half>(ctx, a, grid, threads, smem);
  return launch_q6k_nt<1, __half>(ctx, a, grid, threads, smem);
}

// ---- C ABI ------------------------------------------------------------------------------------

static int check_w(ks_ctx* ctx, const char* what, ks_dtype wd, const ks_buf* W, size_t off, size_t rows, size_t cols) {
  KS_REQUIRE(ctx, wd == KS_Q4K || wd == KS_Q6K, "%s: weight dtype %d not supported (Q4K, Q6K)", what, (int)wd);
  KS_REQUIRE(ctx, cols > 0 && cols % 256 == 0, "%s: cols=%zu must be a positive multiple of 256", what, cols);
  KS_REQUIRE(ctx, rows > 0 && rows < (1u << 31), "%s: rows=%zu out of range", what, rows);
  const size_t need = rows * (cols / 256) * ks_block_bytes(wd);
  KS_REQUIRE(ctx, ks_fits(W, off, need), "%s: weight buffer too small: need %zu B at offset %zu, have %zu", what, need, off,
             W ? W->bytes : 0);
  KS_REQUIRE(ctx, off % (wd == KS_Q4K ? 16 : 2) == 0, "%s: weight byte offset %zu misaligned", what, off);
  return KS_OK;
}

extern "C" {

int ks_matvec(ks_ctx* ctx, size_t rows, size_t cols, ks_dtype wdtype, const ks_buf* W, size_t w_byte_off,
              ks_dtype act, const ks_buf* x, size_t x_off, ks_buf* y, size_t y_off, int n_tok) {
  if (!ctx) return KS_ERR_INVALID;
  int rc = check_w(ctx, "matvec", wdtype, W, w_byte_off, rows, cols);
  if (rc) return rc;
  KS_REQUIRE(ctx, ks_is_act(act), "matvec: activation dtype must be F32 or F16");
  KS_REQUIRE(ctx, n_tok >= 1 && n_tok <= 256, "matvec: n_tok=%d outside 1..256", n_tok);
  const size_t ab = ks_act_bytes(act);
  KS_REQUIRE(ctx, ks_fits(x, x_off * ab, (size_t)n_tok * cols * ab), "matvec: x buffer too small");
  KS_REQUIRE(ctx, ks_fits(y, y_off * ab, (size_t)n_tok * rows * ab), "matvec: y buffer too small");
  if (n_tok > 8) {  // the reference's mul_mm route (lib.rs:1414): a tensor-core GEMM over all rows at once
    KS_REQUIRE(ctx, act == KS_F32 && (wdtype == KS_Q4K || wdtype == KS_Q6K) && cols % 256 == 0 && x_off % 4 == 0,
               "matvec: batches of more than 8 rows need f32 activations, Q4K/Q6K weights, cols %% 256 == 0 and x_off %% 4 == 0");
    void* scratch = nullptr;
    if ((rc = ks_ctx_gemm_scratch(ctx, ks_gemm_xt_bytes(cols, n_tok) + 4 * ks_gemm_part_floats(ctx, rows, cols, n_tok), &scratch))) return rc;
    rc = ks_launch_gemm_kq(ctx, wdtype, rows, cols, (const uint8_t*)W->dptr + w_byte_off, (const float*)x->dptr + x_off, cols,
                           (float*)y->dptr + y_off, rows, n_tok, scratch);
    return rc == 1 ? ks_fail(ctx, KS_ERR_UNSUPPORTED, "matvec: %zux%zu with %d rows does not fit the GEMM kernel", rows, cols, n_tok) : rc;
  }
  ks_mv_seg seg{(const uint8_t*)W->dptr + w_byte_off, (char*)y->dptr + y_off * ab, (unsigned)rows};
  return ks_launch_matvec(ctx, wdtype, &seg, 1, KS_EPI_PLAIN, cols, act, (const char*)x->dptr + x_off * ab, n_tok, nullptr);
}

int ks_matvec_qkv(ks_ctx* ctx, size_t q_rows, size_t kv_rows, size_t cols, ks_dtype dq, ks_dtype dk, ks_dtype dv,
                  const ks_buf* Wq, const ks_buf* Wk, const ks_buf* Wv, ks_dtype act, const ks_buf* x, ks_buf* q,
                  ks_buf* k, ks_buf* v) {
  if (!ctx) return KS_ERR_INVALID;
  int rc;
  if ((rc = check_w(ctx, "matvec_qkv(q)", dq, Wq, 0, q_rows, cols))) return rc;
  if ((rc = check_w(ctx, "matvec_qkv(k)", dk, Wk, 0, kv_rows, cols))) return rc;
  if ((rc = check_w(ctx, "matvec_qkv(v)", dv, Wv, 0, kv_rows, cols))) return rc;
  KS_REQUIRE(ctx, ks_is_act(act), "matvec_qkv: activation dtype must be F32 or F16");
  const size_t ab = ks_act_bytes(act);
  KS_REQUIRE(ctx, ks_fits(x, 0, cols * ab), "matvec_qkv: x buffer too small");
  KS_REQUIRE(ctx, ks_fits(q, 0, q_rows * ab) && ks_fits(k, 0, kv_rows * ab) && ks_fits(v, 0, kv_rows * ab),
             "matvec_qkv: output buffer too small");
  if (dq == dk && dk == dv) {
    ks_mv_seg segs[3] = {{(const uint8_t*)Wq->dptr, q->dptr, (unsigned)q_rows},
                         {(const uint8_t*)Wk->dptr, k->dptr, (unsigned)kv_rows},
                         {(const uint8_t*)Wv->dptr, v->dptr, (unsigned)kv_rows}};
    return ks_launch_matvec(ctx, dq, segs, 3, KS_EPI_PLAIN, cols, act, x->dptr, 1, nullptr);
  }
  // mixed packings (e.g. Q4K/Q4K/Q6K): one launch per dtype
  const ks_dtype dts[3] = {dq, dk, dv};
  const ks_buf* Ws[3] = {Wq, Wk, Wv};
  ks_buf* ys[3] = {q, k, v};
  const size_t rs[3] = {q_rows, kv_rows, kv_rows};
  for (int i = 0; i < 3; i++) {
    ks_mv_seg seg{(const uint8_t*)Ws[i]->dptr, ys[i]->dptr, (unsigned)rs[i]};
    if ((rc = ks_launch_matvec(ctx, dts[i], &seg, 1, KS_EPI_PLAIN, cols, act, x->dptr, 1, nullptr))) return rc;
  }
  return KS_OK;
}

int ks_matvec_gate_up_gelu(ks_ctx* ctx, size_t rows, size_t cols, ks_dtype wdtype, const ks_buf* Wg, const ks_buf* Wu,
                           ks_dtype act, const ks_buf* x, ks_buf* y) {
  if (!ctx) return KS_ERR_INVALID;
  KS_REQUIRE(ctx, wdtype == KS_Q4K, "matvec_gate_up_gelu: only Q4K weights are fused (got dtype %d)", (int)wdtype);
  int rc;
  if ((rc = check_w(ctx, "matvec_gate_up_gelu(gate)", wdtype, Wg, 0, rows, cols))) return rc;
  if ((rc = check_w(ctx, "matvec_gate_up_gelu(up)", wdtype, Wu, 0, rows, cols))) return rc;
  KS_REQUIRE(ctx, ks_is_act(act), "matvec_gate_up_gelu: activation dtype must be F32 or F16");
  const size_t ab = ks_act_bytes(act);
  KS_REQUIRE(ctx, ks_fits(x, 0, cols * ab), "matvec_gate_up_gelu: x buffer too small");
  KS_REQUIRE(ctx, ks_fits(y, 0, rows * ab), "matvec_gate_up_gelu: y buffer too small");
  ks_mv_seg segs[2] = {{(const uint8_t*)Wg->dptr, y->dptr, (unsigned)rows}, {(const uint8_t*)Wu->dptr, y->dptr, (unsigned)rows}};
  return ks_launch_matvec(ctx, wdtype, segs, 2, KS_EPI_GATE_UP, cols, act, x->dptr, 1, nullptr);
}

// Validates the fused-norm operands and fills the prologue descriptor.
static int make_pro(ks_ctx* ctx, const char* what, size_t cols, float eps, ks_dtype wdtype, ks_dtype act, const ks_buf* x,
                    const ks_buf* w_norm, const ks_buf* y_prev, const ks_buf* w_post, ks_buf* out_x, ks_mv_pro* pro) {
  KS_REQUIRE(ctx, ks_is_act(act), "%s: activation dtype must be F32 or F16", what);
  KS_REQUIRE(ctx, ks_matvec_can_fuse_pro(wdtype, cols), "%s: the norm can be fused only for Q4K weights with cols <= 4096", what);
  const size_t ab = ks_act_bytes(act);
  KS_REQUIRE(ctx, ks_fits(x, 0, cols * ab) && ks_fits(w_norm, 0, cols * ab), "%s: x or norm weight buffer too small", what);
  const bool add = y_prev || w_post || out_x;
  if (add) {
    KS_REQUIRE(ctx, y_prev && w_post && out_x, "%s: y_prev, w_post and out_x go together", what);
    KS_REQUIRE(ctx, ks_fits(y_prev, 0, cols * ab) && ks_fits(w_post, 0, cols * ab) && ks_fits(out_x, 0, cols * ab),
               "%s: residual-update buffer too small", what);
    KS_REQUIRE(ctx, out_x->dptr != x->dptr, "%s: out_x must not alias x", what);
  }
  pro->mode = add ? KS_PRO_ADD_NORM : KS_PRO_NORM;
  pro->eps = eps;
  pro->w = w_norm->dptr;
  pro->y = add ? y_prev->dptr : nullptr;
  pro->w_post = add ? w_post->dptr : nullptr;
  pro->out_x = add ? out_x->dptr : nullptr;
  return KS_OK;
}

int ks_rmsnorm_matvec(ks_ctx* ctx, size_t rows, size_t cols, float eps, ks_dtype wdtype, ks_dtype act, const ks_buf* x,
                      const ks_buf* w_norm, const ks_buf* W, ks_buf* y, const ks_buf* y_prev, const ks_buf* w_post,
                      ks_buf* out_x) {
  if (!ctx) return KS_ERR_INVALID;
  int rc;
  if ((rc = check_w(ctx, "rmsnorm_matvec", wdtype, W, 0, rows, cols))) return rc;
  ks_mv_pro pro{};
  if ((rc = make_pro(ctx, "rmsnorm_matvec", cols, eps, wdtype, act, x, w_norm, y_prev, w_post, out_x, &pro))) return rc;
  KS_REQUIRE(ctx, ks_fits(y, 0, rows * ks_act_bytes(act)), "rmsnorm_matvec: y buffer too small");
  ks_mv_seg seg{(const uint8_t*)W->dptr, y->dptr, (unsigned)rows};
  return ks_launch_matvec(ctx, wdtype, &seg, 1, KS_EPI_PLAIN, cols, act, x->dptr, 1, nullptr, &pro);
}

int ks_rmsnorm_matvec_qkv(ks_ctx* ctx, size_t q_rows, size_t kv_rows, size_t cols, float eps, ks_dtype wdtype,
                          ks_dtype act, const ks_buf* x, const ks_buf* w_norm, const ks_buf* Wq, const ks_buf* Wk,
                          const ks_buf* Wv, ks_buf* q, ks_buf* k, ks_buf* v, const ks_buf* y_prev, const ks_buf* w_post,
                          ks_buf* out_x) {
  if (!ctx) return KS_ERR_INVALID;
  int rc;
  if ((rc = check_w(ctx, "rmsnorm_matvec_qkv(q)", wdtype, Wq, 0, q_rows, cols))) return rc;
  if ((rc = check_w(ctx, "rmsnorm_matvec_qkv(k)", wdtype, Wk, 0, kv_rows, cols))) return rc;
  if ((rc = check_w(ctx, "rmsnorm_matvec_qkv(v)", wdtype, Wv, 0, kv_rows, cols))) return rc;
  ks_mv_pro pro{};
  if ((rc = make_pro(ctx, "rmsnorm_matvec_qkv", cols, eps, wdtype, act, x, w_norm, y_prev, w_post, out_x, &pro))) return rc;
  const size_t ab = ks_act_bytes(act);
  KS_REQUIRE(ctx, ks_fits(q, 0, q_rows * ab) && ks_fits(k, 0, kv_rows * ab) && ks_fits(v, 0, kv_rows * ab),
             "rmsnorm_matvec_qkv: output buffer too small");
  ks_mv_seg segs[3] = {{(const uint8_t*)Wq->dptr, q->dptr, (unsigned)q_rows},
                       {(const uint8_t*)Wk->dptr, k->dptr, (unsigned)kv_rows},
                       {(const uint8_t*)Wv->dptr, v->dptr, (unsigned)kv_rows}};
  return ks_launch_matvec(ctx, wdtype, segs, 3, KS_EPI_PLAIN, cols, act, x->dptr, 1, nullptr, &pro);
}

int ks_rmsnorm_matvec_gate_up_gelu(ks_ctx* ctx, size_t rows, size_t cols, float eps, ks_dtype wdtype, ks_dtype act,
                                   const ks_buf* x, const ks_buf* w_norm, const ks_buf* Wg, const ks_buf* Wu, ks_buf* y,
                                   const ks_buf* y_prev, const ks_buf* w_post, ks_buf* out_x) {
  if (!ctx) return KS_ERR_INVALID;
  int rc;
  if ((rc = check_w(ctx, "rmsnorm_matvec_gate_up_gelu(gate)", wdtype, Wg, 0, rows, cols))) return rc;
  if ((rc = check_w(ctx, "rmsnorm_matvec_gate_up_gelu(up)", wdtype, Wu, 0, rows, cols))) return rc;
  ks_mv_pro pro{};
  if ((rc = make_pro(ctx, "rmsnorm_matvec_gate_up_gelu", cols, eps, wdtype, act, x, w_norm, y_prev, w_post, out_x, &pro))) return rc;
  KS_REQUIRE(ctx, ks_fits(y, 0, rows * ks_act_bytes(act)), "rmsnorm_matvec_gate_up_gelu: y buffer too small");
  ks_mv_seg segs[2] = {{(const uint8_t*)Wg->dptr, y->dptr, (unsigned)rows}, {(const uint8_t*)Wu->dptr, y->dptr, (unsigned)rows}};
  return ks_launch_matvec(ctx, wdtype, segs, 2, KS_EPI_GATE_UP, cols, act, x->dptr, 1, nullptr, &pro);
}

int ks_matvec_host(ks_ctx* ctx, size_t rows, size_t cols, ks_dtype wdtype, const ks_buf* W, size_t w_byte_off,
                   const float* x_host, float* y_host, int n_tok) {
  if (!ctx) return KS_ERR_INVALID;
  KS_REQUIRE(ctx, x_host && y_host, "matvec_host: null host pointer");
  KS_REQUIRE(ctx, n_tok >= 1 && n_tok <= 8, "matvec_host: n_tok=%d outside 1..8", n_tok);
  const size_t xb = (size_t)n_tok * cols * 4, yb = (size_t)n_tok * rows * 4;
  if (!ctx->stage_x || ctx->stage_x->bytes < xb) {
    if (ctx->stage_x) ks_buf_free(ctx, ctx->stage_x);
    ctx->stage_x = ks_buf_alloc(ctx, xb);
    if (!ctx->stage_x) return KS_ERR_OOM;
  }
  if (!ctx->stage_y || ctx->stage_y->bytes < yb) {
    if (ctx->stage_y) ks_buf_free(ctx, ctx->stage_y);
    ctx->stage_y = ks_buf_alloc(ctx, yb);
    if (!ctx->stage_y) return KS_ERR_OOM;
  }
  int rc;
  if ((rc = ks_buf_upload_async(ctx, ctx->stage_x, 0, x_host, xb))) return rc;
  if ((rc = ks_matvec(ctx, rows, cols, wdtype, W, w_byte_off, KS_F32, ctx->stage_x, 0, ctx->stage_y, 0, n_tok))) return rc;
  return ks_buf_download(ctx, ctx->stage_y, 0, y_host, yb);
}

}  // extern "C"

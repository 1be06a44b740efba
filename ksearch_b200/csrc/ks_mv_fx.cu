// Q4_K matvec, one token, f32 x and y: the planner's variant 3.
//
// y = W x (crates/ksearch_kernels/src/lib.rs:137 matvec_wd; the G1 kernel of
// crates/ksearch_codegen/src/lower.rs:1763-2082) for matrices of a few megabytes, where a launch lasts
// only microseconds and latency, not bandwidth, decides.  Built like one phase of the persistent decode
// kernel:
//   * block b owns the contiguous rows [b*R/grid, (b+1)*R/grid) (in pairs): its weights are one byte range,
//     fetched with a handful of cp.async.bulk copies into a shared-memory ring.  The copies are issued
//     BEFORE griddepcontrol.wait: weights are constants, so under programmatic dependent launch they travel
//     while the previous kernel of the stream still runs, and two blocks fit an SM so the next launch's
//     blocks can take residence (and start their copies) while this launch computes;
//   * x is staged once per block as 24-bit block fixed point (three byte planes per 32 elements); a lane owns
//     one 64-weight unit of a 32-unit column segment and keeps that unit of x in registers; nibbles x x are
//     exact dp4a sums; a task is (segment, row); each warp takes one contiguous run of the block's tasks, two
//     rows interleaved; a row's segments meet in shared memory and thread f stores row f.
#include "ks_fx.cuh"

namespace {

constexpr int FXM_NW = 8, FXM_THREADS = FXM_NW * 32;
constexpr int FXM_MAXROWS = 128;  // rows of one block
constexpr int FXM_MAXSEG = 8;
constexpr int FXM_MAXSLOTS = 16;

struct FxmArgs {
  const uint8_t* W;
  const float* x;
  float* y;
  unsigned rows, cols, row_bytes;
  unsigned n_seg, seg_units;   // column segments of <= 32 units
  unsigned piece_rows;         // rows per ring slot (multiple of 4)
  unsigned n_slots, slot_bytes, x_bytes;
  unsigned* err;
};

struct FxmSmem {
  unsigned xs_off, ring_off, bar_off, psum_off, total;
};
__host__ __device__ inline FxmSmem fxm_smem(unsigned x_bytes, unsigned slot_bytes, unsigned n_slots) {
  FxmSmem L;
  L.xs_off = 0;
  L.ring_off = (x_bytes + 127u) & ~127u;
  L.bar_off = L.ring_off + n_slots * slot_bytes;
  L.psum_off = L.bar_off + FXM_MAXSLOTS * 8u;
  L.total = L.psum_off + FXM_MAXROWS * FXM_MAXSEG * 4u;
  return L;
}

__global__ void __launch_bounds__(FXM_THREADS, 2) mv_q4k_fx_kernel(const FxmArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const FxmSmem SL = fxm_smem(a.x_bytes, a.slot_bytes, a.n_slots);
  const uint32_t ring_s = sm32(smem + SL.ring_off), bars = sm32(smem + SL.bar_off), xs_s = sm32(smem + SL.xs_off);
  float* psum = reinterpret_cast<float*>(smem + SL.psum_off);
  // this block's rows: an even split in pairs
  const unsigned half = a.rows >> 1;
  const unsigned lo = (unsigned)(((unsigned long long)blockIdx.x * half) / gridDim.x) * 2u;
  unsigned hi = (unsigned)(((unsigned long long)(blockIdx.x + 1) * half) / gridDim.x) * 2u;
  if (blockIdx.x + 1 == gridDim.x) hi = a.rows;  // an odd last row
  const unsigned nrows = hi - lo;
  const unsigned np = (nrows + a.piece_rows - 1u) / a.piece_rows;  // pieces of this block, piece p -> slot p % n_slots

  auto issue = [&](unsigned p) {  // one thread
    const unsigned r0 = p * a.piece_rows, n = min(a.piece_rows, nrows - r0), sl = p % a.n_slots;
    mb_expect(bars + sl * 8u, n * a.row_bytes);
    bulk_in(ring_s + sl * a.slot_bytes, a.W + (size_t)(lo + r0) * a.row_bytes, n * a.row_bytes, bars + sl * 8u);
  };
  if (threadIdx.x == 0) {
    for (unsigned s = 0; s < a.n_slots; s++) mb_init(bars + s * 8u, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0 && (unsigned)lane < min(np, a.n_slots)) issue((unsigned)lane);  // weights are constants: before the wait
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // x: chunks of 4 elements, all loads first
  const unsigned units = a.cols >> 6, nchunk = a.cols >> 2;
  for (unsigned base = 0; base < nchunk; base += 4u * FXM_THREADS) {
    float4 v[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const unsigned c = base + threadIdx.x + k * FXM_THREADS;
      if (c < nchunk) v[k] = reinterpret_cast<const float4*>(a.x)[c];
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const unsigned c = base + threadIdx.x + k * FXM_THREADS;
      if (c < nchunk) fx_put_chunk(smem + SL.xs_off, units, c, v[k]);  // nchunk is a multiple of 64: whole warps
    }
  }
  __syncthreads();

  const bool active = (unsigned)lane < a.seg_units;
  XUnit x;
  int cur_s = -1;
  bool dead = false;
  const unsigned wave_max = a.n_slots;  // all slots: nothing else competes for the ring
  for (unsigned wp0 = 0; wp0 < np; wp0 += wave_max) {
    const unsigned wp1 = min(wp0 + wave_max, np);
    const unsigned wr0 = wp0 * a.piece_rows, wr1 = min(wp1 * a.piece_rows, nrows), rows_w = wr1 - wr0;
    const unsigned par = (wp0 / a.n_slots) & 1u;
    if (!dead) {
      bool ok = true;
      if ((unsigned)lane < wp1 - wp0) ok = mb_wait(bars + (((unsigned)lane + wp0) % a.n_slots) * 8u, par, 1u << 22);
      if (!__all_sync(0xffffffffu, ok)) {
        dead = true;
        if (lane == 0) atomicOr(a.err, 1u);
      }
    }
    if (!dead) {
      const unsigned T = a.n_seg * rows_w;
      const unsigned t0 = (unsigned)warp * T / FXM_NW, t1 = (unsigned)(warp + 1) * T / FXM_NW;
      unsigned t = t0, sg = t0 / rows_w, rem = t0 - sg * rows_w;
      auto row_addr = [&](unsigned r) {  // row r of the wave
        const unsigned p = wp0 + r / a.piece_rows;
        return ring_s + (p % a.n_slots) * a.slot_bytes + (r % a.piece_rows) * a.row_bytes;
      };
#pragma unroll 1
      while (t < t1) {
        const unsigned u = sg * a.seg_units + (unsigned)lane;
        if ((int)sg != cur_s) {
          if (active) fx_load_unit(x, xs_s, units, u);
          cur_s = (int)sg;
        }
        const uint32_t uoff = (u >> 2) * KS_Q4K_BLOCK_BYTES + (u & 3u) * 32u;
        unsigned n = min(t1 - t, rows_w - rem);
        t += n;
#pragma unroll 1
        for (; n >= 2u; n -= 2u, rem += 2u) {
          const uint32_t wa[2] = {row_addr(rem) + uoff, row_addr(rem + 1u) + uoff};
          float v[2] = {0.0f, 0.0f};
          if (active) fx_rows<2>(wa, (int)(u & 3u), x, v);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
            v[1] += __shfl_xor_sync(0xffffffffu, v[1], o);
          }
          if (lane == 0) {
            psum[(wr0 + rem) * a.n_seg + sg] = v[0];
            psum[(wr0 + rem + 1u) * a.n_seg + sg] = v[1];
          }
        }
        if (n) {
          const uint32_t wa[1] = {row_addr(rem) + uoff};
          float v[1] = {0.0f};
          if (active) fx_rows<1>(wa, (int)(u & 3u), x, v);
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
          if (lane == 0) psum[(wr0 + rem) * a.n_seg + sg] = v[0];
          rem += 1u;
        }
        if (rem == rows_w) {
          rem = 0;
          sg++;
        }
      }
    }
    __syncthreads();  // the wave's row sums are complete and nobody reads its slots any more
    if (warp == FXM_NW - 1 && wp1 < np && (unsigned)lane < min(np - wp1, a.n_slots)) {  // the next wave's pieces
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      issue(wp1 + (unsigned)lane);
    }
    if (threadIdx.x < rows_w) {
      const unsigned r = wr0 + threadIdx.x;
      float v = 0.0f;
      for (unsigned sg2 = 0; sg2 < a.n_seg; sg2++) v += psum[r * a.n_seg + sg2];
      a.y[lo + r] = v;
    }
  }
}

}  // namespace

// Returns 1 when the call is outside what this kernel takes (the caller picks another variant).
int ks_launch_matvec_q4k_fx(ks_ctx* ctx, const ks_mv_seg* segs, int n_seg, ks_mv_epilogue epi, size_t cols, ks_dtype act,
                            const void* x, int n_tok, const ks_plan* plan) {
  if (n_seg != 1 || epi != KS_EPI_PLAIN || act != KS_F32 || n_tok != 1) return 1;
  const unsigned U = (unsigned)(cols / 64);
  const unsigned S = (U + 31u) / 32u;
  if (S > (unsigned)FXM_MAXSEG || U % S) return 1;
  const unsigned rows = segs[0].rows, row_bytes = (unsigned)(cols / 256 * KS_Q4K_BLOCK_BYTES);
  if (rows < 2 || ((uintptr_t)x & 15u)) return 1;
  // grid: one or two blocks per SM, as long as every block keeps a few rows
  const int cps = (plan && plan->ctas_per_sm > 0) ? (plan->ctas_per_sm > 2 ? 2 : plan->ctas_per_sm) : 1;
  unsigned grid = (unsigned)(ctx->sm_count * cps);
  if (grid > rows / 2u) grid = rows / 2u;
  const unsigned max_rows = ((rows / 2u + grid - 1u) / grid) * 2u + 1u;
  if (max_rows > (unsigned)FXM_MAXROWS) return 1;
  // two blocks must fit an SM, so that the next launch's blocks can move in while this one computes
  const unsigned x_bytes = U * 256u;
  const unsigned budget = (unsigned)(ctx->smem_optin / 2u) - 2048u;
  const FxmSmem fixed = fxm_smem(x_bytes, 0, 0);
  if (fixed.total + 4u * row_bytes > budget) return 1;
  const unsigned room = budget - fixed.total;
  // pieces of about 8 KB (bulk copies of that size move at full speed), all of the block's rows in flight if they fit
  unsigned piece_rows = (8192u / row_bytes) & ~3u;
  if (piece_rows < 4u) piece_rows = 4u;
  unsigned slot_bytes = (piece_rows * row_bytes + 127u) & ~127u;
  unsigned n_slots = room / slot_bytes;
  if (n_slots < 1u) return 1;
  const unsigned need = (max_rows + piece_rows - 1u) / piece_rows;
  if (n_slots > need) n_slots = need;
  if (n_slots > (unsigned)FXM_MAXSLOTS) n_slots = FXM_MAXSLOTS;
  FxmArgs a{};
  a.W = segs[0].W;
  a.x = (const float*)x;
  a.y = (float*)segs[0].y;
  a.rows = rows;
  a.cols = (unsigned)cols;
  a.row_bytes = row_bytes;
  a.n_seg = S;
  a.seg_units = U / S;
  a.piece_rows = piece_rows;
  a.n_slots = n_slots;
  a.slot_bytes = slot_bytes;
  a.x_bytes = x_bytes;
  a.err = (unsigned*)ctx->ws + KS_WS_ERR_WORD;
  const size_t smem = fxm_smem(x_bytes, slot_bytes, n_slots).total;
  static size_t smem_set[16] = {0};
  if (smem > smem_set[ctx->device & 15]) {
    cudaError_t e = cudaFuncSetAttribute(mv_q4k_fx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "matvec (fixed point): cannot set %zu B shared memory: %s", smem, cudaGetErrorString(e));
    smem_set[ctx->device & 15] = smem;
  }
  KS_LAUNCH(ctx, (mv_q4k_fx_kernel), grid, FXM_THREADS, smem, a);
  return ks_after_launch(ctx, "matvec_q4k_fx");
}

// Internal declarations shared by the translation units of libksearch_cuda.so.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <cstdarg>
#include <cstdio>
#include <deque>
#include <map>
#include <string>

#include "../../include/ksearch_cuda.h"

struct ks_ctx {
  int device = 0;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  size_t smem_optin = 0;
  cudaStream_t stream = nullptr;
  bool pdl = false;  // launch kernels with programmatic stream serialization
  std::string err;
  std::string chip;
  std::deque<cudaEvent_t> inflight;  // commit points not yet known complete
  uint64_t launches = 0;
  cudaEvent_t t0 = nullptr, t1 = nullptr;  // stopwatch
  bool has_override = false;
  ks_plan override_plan{};
  std::map<std::string, ks_plan> plans;  // op_rowsxcols[_bN] -> plan (searched, loaded or set)
  void* ws = nullptr;  // small zero-initialised device workspace (cross-block reductions)
  void* gemm_ws = nullptr;  // token rows split into f16 terms for the tensor-core GEMM (grown outside stream capture)
  size_t gemm_ws_bytes = 0;
  // pinned staging for the *_host convenience calls
  void* stage_h = nullptr;
  size_t stage_h_bytes = 0;
  ks_buf* stage_x = nullptr;
  ks_buf* stage_y = nullptr;
};

struct ks_buf {
  void* dptr = nullptr;
  size_t bytes = 0;
  bool owned = true;
};

int ks_fail(ks_ctx* ctx, int code, const char* fmt, ...);
void ks_set_global_error(const char* msg);

#define KS_REQUIRE(ctx, cond, ...)                              \
  do {                                                          \
    if (!(cond)) return ks_fail((ctx), KS_ERR_INVALID, __VA_ARGS__); \
  } while (0)

#define KS_CUDA(ctx, call)                                                                     \
  do {                                                                                         \
    cudaError_t e__ = (call);                                                                  \
    if (e__ != cudaSuccess)                                                                    \
      return ks_fail((ctx), KS_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__));     \
  } while (0)

// Checks the last launch and counts it.
int ks_after_launch(ks_ctx* ctx, const char* what);

static inline size_t ks_act_bytes(ks_dtype a) { return a == KS_F16 ? 2 : 4; }
static inline bool ks_is_act(ks_dtype a) { return a == KS_F32 || a == KS_F16; }
static inline size_t ks_block_bytes(ks_dtype d) {
  return d == KS_Q4K ? KS_Q4K_BLOCK_BYTES : d == KS_Q6K ? KS_Q6K_BLOCK_BYTES : d == KS_Q40 ? KS_Q40_BLOCK_BYTES : d == KS_Q5K ? KS_Q5K_BLOCK_BYTES : 0;
}
static inline size_t ks_block_elems(ks_dtype d) { return d == KS_Q40 ? 32 : 256; }
// bytes of n elements of dtype d (n a multiple of the block size for packed types)
static inline size_t ks_nbytes(ks_dtype d, size_t n) {
  if (d == KS_F32) return n * 4;
  if (d == KS_F16) return n * 2;
  return n / ks_block_elems(d) * ks_block_bytes(d);
}

// Range check of (buffer, byte offset, byte extent).
static inline bool ks_fits(const ks_buf* b, size_t off, size_t extent) {
  return b && b->dptr && off <= b->bytes && extent <= b->bytes - off;
}

// ---- launchers on raw device pointers (used by the C ABI and by the decoder) --
struct ks_mv_seg {   // one weight matrix of a fused matvec launch
  const uint8_t* W;  // packed rows
  void* y;           // output vector base ([n_tok, rows])
  unsigned rows;
};

enum ks_mv_epilogue { KS_EPI_PLAIN = 0, KS_EPI_GATE_UP = 1 };

// Input prologue fused into a matvec (see ks_mv_common.cuh): none, RMSNorm, or
// residual-add-then-RMSNorm.  out_x must not alias the residual input.
enum { KS_PRO_NONE = 0, KS_PRO_NORM = 1, KS_PRO_ADD_NORM = 2 };
struct ks_mv_pro {
  int mode;
  float eps;
  const void* w;       // norm weight applied last (w or w_next)
  const void* y;       // ADD_NORM: the vector that is normed and added
  const void* w_post;  // ADD_NORM: its weight
  void* out_x;         // ADD_NORM: new residual stream (written by block 0)
};

// Launch tuning knobs of the matvec kernels (the planner's vocabulary, after
// OptSchedule in crates/ksearch_ir/src/kernel.rs:11-54).  Zero = default.
typedef ks_plan ks_mv_plan;

int ks_launch_matvec(ks_ctx* ctx, ks_dtype wdtype, const ks_mv_seg* segs, int n_seg, ks_mv_epilogue epi,
                     size_t cols, ks_dtype act, const void* x, int n_tok, const ks_mv_plan* plan,
                     const ks_mv_pro* pro = nullptr);
std::string ks_plan_key(const char* op, size_t rows, size_t cols, int n_tok);
const ks_plan* ks_plan_lookup(const ks_ctx* ctx, const char* op, size_t rows, size_t cols, int n_tok);
// True when a prologue can be fused for this shape (streamed Q4_K kernel, cols <= 4096, even block count).
bool ks_matvec_can_fuse_pro(ks_dtype wdtype, size_t cols);

// variant (plan->variant & 0xFF): 0 = streamed through the bulk-copy engine, 1 = direct register loads
int ks_launch_matvec_stream_q4k(ks_ctx* ctx, const ks_mv_seg* segs, int n_seg, ks_mv_epilogue epi, size_t cols,
                                ks_dtype act, const void* x, int n_tok, const ks_plan* plan, const ks_mv_pro* pro);
int ks_launch_matvec_stream_q6k(ks_ctx* ctx, const ks_mv_seg* segs, int n_seg, size_t cols, ks_dtype act, const void* x,
                                int n_tok, const ks_plan* plan);   // returns 1 when the shape must use the direct kernel
// variant 2 (Q6_K only): x as block fixed point, byte dot products; returns 1 when the call must use another variant
int ks_launch_matvec_q6k_fx(ks_ctx* ctx, const ks_mv_seg* segs, int n_seg, size_t cols, ks_dtype act, const void* x, int n_tok,
                            const ks_plan* plan);
// variant 4 (Q6_K): variant 2's arithmetic with the rows streamed through per-warp shared-memory rings; returns 1 when
// the call must use another variant
int ks_launch_matvec_q6k_ring(ks_ctx* ctx, const ks_mv_seg* segs, int n_seg, size_t cols, ks_dtype act, const void* x, int n_tok,
                              const ks_plan* plan);
// variant 3 (Q4_K, one token, f32): rows out of a shared-memory ring against a block fixed-point x (ks_mv_fx.cu);
// returns 1 when the call must use another variant
int ks_launch_matvec_q4k_fx(ks_ctx* ctx, const ks_mv_seg* segs, int n_seg, ks_mv_epilogue epi, size_t cols, ks_dtype act,
                            const void* x, int n_tok, const ks_plan* plan);
// Device error word raised by a kernel whose bounded wait gave up (index into ctx->ws, in words).
#define KS_WS_ERR_WORD 4000

int ks_launch_rmsnorm(ks_ctx* ctx, size_t n, size_t rows, float eps, ks_dtype act, const void* x, const void* w,
                      const void* res, int has_scale, float scale, void* y);
int ks_launch_rmsnorm_add_then_rmsnorm(ks_ctx* ctx, size_t n, size_t rows, float eps, ks_dtype act, const void* y,
                                       const void* w_post, const void* res, const void* w_ffn, void* out_x,
                                       void* out_x2);
int ks_launch_per_head_qkv_q40(ks_ctx* ctx, size_t n_q, size_t n_kv, size_t hd, size_t n_tok, float eps,
                               ks_dtype act, const void* q, const void* qw, const float* rope, const void* k,
                               const void* kw, const void* v, void* q_out, uint8_t* kv_k, uint8_t* kv_v,
                               const int* pos_dev, size_t slot_stride_bytes);
int ks_launch_sdpa(ks_ctx* ctx, size_t n_slots, size_t n_q, size_t n_kv, size_t hd, float scale, ks_dtype act,
                   const void* q, const uint8_t* K, const uint8_t* V, size_t slot_stride_bytes, const float* meta,
                   float* tmp, void* out, int n_splits);
int ks_launch_copy_scale_indexed(ks_ctx* ctx, size_t n, size_t batch, float scale, ks_dtype src_dtype,
                                 const void* src, const float* idx, ks_dtype act, void* dst);
int ks_launch_softcap_argmax(ks_ctx* ctx, size_t n, float cap, ks_dtype act, const void* logits, float* out_idx);

// ---- tensor-core GEMM for batches of more than 8 token rows (ks_gemm.cu) ---------------------------
// nelem (a multiple of 256) elements of src (Q6K, Q4K, F16, F32) -> Q4_K blocks, as the reference's load-time quantizer.
int ks_launch_quantize_q4k(ks_ctx* ctx, ks_dtype src_dtype, const void* src, size_t nelem, void* dst);
size_t ks_gemm_xt_bytes(size_t cols, int n_tok);  // bytes of the split image of n_tok rows of `cols` values
size_t ks_gemm_part_floats(const ks_ctx* ctx, size_t total_rows, size_t cols, int n_tok);  // k-split partials, at most
// The context's scratch, grown to `bytes` (fails inside a stream capture when it would have to grow).
int ks_ctx_gemm_scratch(ks_ctx* ctx, size_t bytes, void** out);
// x[t * ldx + k] (f32) -> the image the GEMM reads its token rows from.
int ks_launch_gemm_split(ks_ctx* ctx, const float* x, size_t ldx, int n_tok, size_t cols, void* xt);
// Up to three matrices over the same columns and token rows (q, k, v; gate, up) in one launch.  What becomes of
// the sums: PLAIN y[i] = W[i] x; GELU (two matrices) y[0] = gelu(W[0] x) * (W[1] x); NORM_SPLIT (one matrix)
// out_x = res + rms(W x) * w_post and the image of rms(out_x) * w_norm for the next GEMM in xt_out; GELU_SPLIT
// (two matrices) the image of gelu(W[0] x) * (W[1] x) in xt_out.  P: ks_gemm_part_floats(sum of rows) floats.
enum { KS_GEMM_PLAIN = 0, KS_GEMM_GELU = 1, KS_GEMM_NORM_SPLIT = 2, KS_GEMM_GELU_SPLIT = 3 };
struct ks_gemm_epi {
  const float *res, *w_post, *w_norm;  // NORM_SPLIT: residual rows [n_tok, rows], the two norm weights
  float eps;
  float* out_x;                        // NORM_SPLIT: the updated residual rows
  void* xt_out;                        // the image written for the next GEMM (may be the image this GEMM read)
};
int ks_launch_gemm_segs(ks_ctx* ctx, ks_dtype wdtype, int n_seg, const uint8_t* const* W, const size_t* rows, size_t cols, const void* xt,
                        int n_tok, float* const* y, const size_t* ldy, float* P, int mode, const ks_gemm_epi* epi);
// Split + GEMM for one matrix.  Returns 1 when the shape is not covered (cols not a multiple of 256, more than
// 256 rows).  scratch: ks_gemm_xt_bytes + 4 * ks_gemm_part_floats bytes.
int ks_launch_gemm_kq(ks_ctx* ctx, ks_dtype wdtype, size_t rows, size_t cols, const uint8_t* W, const float* x, size_t ldx, float* y,
                      size_t ldy, int n_tok, void* scratch);

// ---- all layers of one token as ONE persistent kernel (ks_mega.cu) --------------------------------
struct ks_mega_layer {
  const void *wq, *wk, *wv, *wo, *wgate, *wup, *wdown;  // Q4_K
  const void *attn_norm, *q_norm, *k_norm, *post_attn_norm, *ffn_norm, *post_ffw_norm;  // f32
  uint8_t *kv_k, *kv_v;  // this slot's cache rows [max_seq, n_kv, hd] Q4_0
};
struct ks_mega_desc {
  int n_layers;
  unsigned hidden, ffn, n_q, n_kv, hd;
  float eps, attn_scale;
  const float* rope;  // [max_seq, hd]
  const int* pos;     // device: position of the token being processed
  float *x_a, *x_b;   // residual stream ping-pong; the token's embedding is in x_a on entry
  float *yb, *q, *k, *v, *o, *ff;
  float* att_tmp;     // n_q * n_splits * (hd + 2) floats
  int n_splits;
};
// Two kernels take the same description.  ks_mega_* (ks_mega.cu): phases separated by grid-wide barriers,
// inputs staged from plain global vectors.  ks_flow_* (ks_flow.cu): no barriers, every value that crosses
// blocks travels as a tagged 64-bit word and consumers poll for the tags.
// *out == nullptr with KS_OK: shape not covered, keep the launch-per-op path.
struct ks_mega;
int ks_mega_create(ks_ctx* ctx, const ks_mega_desc* d, const ks_mega_layer* layers, ks_mega** out);
int ks_mega_launch(ks_ctx* ctx, ks_mega* mg);
float* ks_mega_residual(const ks_mega* mg);  // where the residual stream is when the kernel ends (yb holds the last down-proj)
const long long* ks_mega_prof(const ks_mega* mg);  // [2][5 * n_layers][8] clock64 stamps of the last token (first, last block)
int ks_mega_reset(ks_ctx* ctx, ks_mega* mg);  // barrier words back to their rest state (after a timed-out wait)
int ks_mega_set(ks_mega* mg, int what, unsigned value);  // test knobs: 0 poll limit, 1 stall one barrier
void ks_mega_destroy(ks_mega* mg);

struct ks_flow;
int ks_flow_create(ks_ctx* ctx, const ks_mega_desc* d, const ks_mega_layer* layers, ks_flow** out);
int ks_flow_launch(ks_ctx* ctx, ks_flow* mg);
float* ks_flow_residual(const ks_flow* mg);
const long long* ks_flow_prof(const ks_flow* mg);  // [2][n_layers][5][8] globaltimer stamps of the last token (first, last block)
const long long* ks_flow_prof_all(const ks_flow* mg);  // [grid][n_layers][5][8]: every block's stamps
int ks_flow_reset(ks_ctx* ctx, ks_flow* mg);  // working order again after a timed-out wait
int ks_flow_set(ks_flow* mg, int what, unsigned value);  // test / profiling knobs, see ks_flow.cu
void ks_flow_destroy(ks_flow* mg);

// ---- programmatic dependent launch --------------------------------------------------------------
// Every kernel of the library is launched through ks_launch_k.  When the context was created with
// flag bit 0, the launch carries the programmatic-stream-serialization attribute: the kernel may
// start while its predecessor in the stream still runs.  Each kernel therefore calls
// ks_pdl_entry() (or, for the streamed matvec, issues its weight copies first) before it touches
// anything a predecessor writes; griddepcontrol.wait returns at once when the launch carried no
// such attribute.
#ifdef __CUDACC__
#include <utility>
template <typename... KArgs, typename... Args>
static inline cudaError_t ks_launch_k(ks_ctx* ctx, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, std::forward<Args>(args)...);
}
#define KS_LAUNCH(ctx, kern, grid, block, smem, ...) (void)ks_launch_k((ctx), kern, dim3(grid), dim3(block), (smem), __VA_ARGS__)
// Let the next kernel in the stream start, then wait until everything before this kernel is done.
static __device__ __forceinline__ void ks_pdl_entry() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
#endif

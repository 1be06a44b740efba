/*
 * ksearch_cuda.h -- C ABI of libksearch_cuda.so, a B200 (sm_100a) backend for
 * the single-token decode path of ksearch.
 *
 * Each entry point names the reference interface it stands in for.  Paths are
 * relative to the reference project root; K = crates/ksearch_kernels/src/lib.rs
 * (the `Eng` op interface), M = crates/ksearch_metal/src/lib.rs (the device
 * runtime), GG = crates/ksearch_gguf/src/gguf_impl.rs, GP =
 * crates/ksearch_gemma/src/gemma_prim.rs, KV = crates/ksearch_gemma/src/kv_pool.rs,
 * CG = crates/ksearch_codegen/src/lib.rs.
 *
 * Conventions (the reference's, K:137-146, M:269-374):
 *   - every op only ENQUEUES work on the context's stream, in program order;
 *     nothing inside an op allocates or synchronises;
 *   - static dims first, then dtype tags, then (buffer, offset) pairs; offsets
 *     are in ELEMENTS for f32/f16 operands and in BYTES for packed operands;
 *   - outputs may alias inputs where the reference allows it (residual in/out);
 *   - return 0 on success, a negative ks_status otherwise; ks_last_error() gives
 *     the message.  Nothing aborts.  There is no CPU fallback: every op needs
 *     a CUDA device of compute capability 10.x.
 *   - one context per GPU, used from one thread at a time (M:20-22).
 */
#ifndef KSEARCH_CUDA_H
#define KSEARCH_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct ks_ctx ks_ctx;
typedef struct ks_buf ks_buf;

/* crates/ksearch_ir/src/lib.rs:17-74 (DType and packed byte sizes) */
typedef enum { KS_F32 = 0, KS_F16 = 1, KS_Q4K = 2, KS_Q6K = 3, KS_Q40 = 4, KS_Q5K = 5 } ks_dtype;  /* Q5K: dequant, row gather and load-time requantisation only */

typedef enum {
  KS_OK = 0,
  KS_ERR_INVALID = -1,     /* bad shape / alignment / range (anyhow::bail! in the reference) */
  KS_ERR_CUDA = -2,        /* a CUDA call failed */
  KS_ERR_OOM = -3,         /* allocation failed */
  KS_ERR_UNSUPPORTED = -4, /* dtype or device not supported */
  KS_ERR_STATE = -5,       /* e.g. max_seq exceeded (GP:882-884), slot pool full (KV:136-145) */
  KS_ERR_TIMEOUT = -6      /* a bounded device-side wait gave up */
} ks_status;

#define KS_Q4K_BLOCK_BYTES 144
#define KS_Q6K_BLOCK_BYTES 210
#define KS_Q40_BLOCK_BYTES 18
#define KS_Q5K_BLOCK_BYTES 176
#define KS_SDPA_MAX_SPLITS 128

/* ---- runtime: MetalContext (M:16-218) ----------------------------------- */
ks_ctx* ks_ctx_create(int device, uint64_t flags);          /* M:31-41  MetalContext::new */
void ks_ctx_destroy(ks_ctx* ctx);
const char* ks_last_error(const ks_ctx* ctx);               /* anyhow::Error text */
const char* ks_chip_name(const ks_ctx* ctx);                /* M device_name(); KSEARCH_CHIP overrides (CG:63-66) */
int ks_ctx_device(const ks_ctx* ctx);
int ks_ctx_sm_count(const ks_ctx* ctx);
void* ks_ctx_stream(const ks_ctx* ctx);                     /* the cudaStream_t ops are enqueued on */
/* Number of kernels this context has launched since creation (bench bookkeeping). */
uint64_t ks_ctx_launch_count(const ks_ctx* ctx);

ks_buf* ks_buf_alloc(ks_ctx* ctx, size_t bytes);            /* M:63-91  buffer_empty_* (zero-filled) */
void ks_buf_free(ks_ctx* ctx, ks_buf* buf);
size_t ks_buf_size(const ks_buf* buf);
void* ks_buf_device_ptr(const ks_buf* buf);
/* Wrap device memory owned by the caller (e.g. a torch tensor); never freed by the library. */
ks_buf* ks_buf_wrap(ks_ctx* ctx, void* device_ptr, size_t bytes);
int ks_buf_upload(ks_ctx* ctx, ks_buf* dst, size_t dst_off, const void* host, size_t bytes);   /* M:93-113 write_buffer (blocking) */
int ks_buf_download(ks_ctx* ctx, const ks_buf* src, size_t src_off, void* host, size_t bytes); /* M:115-135 read_* (synchronises first) */
int ks_buf_upload_async(ks_ctx* ctx, ks_buf* dst, size_t dst_off, const void* host, size_t bytes);   /* write_buffer_nosync */
int ks_buf_download_async(ks_ctx* ctx, const ks_buf* src, size_t src_off, void* host, size_t bytes); /* read_f32_nosync */
int ks_buf_zero(ks_ctx* ctx, ks_buf* buf, size_t off, size_t bytes);
void* ks_host_alloc_pinned(size_t bytes);
void ks_host_free_pinned(void* p);

int ks_flush(ks_ctx* ctx);                                  /* M:162   flush_async: mark a commit point */
int ks_wait_inflight_at_most(ks_ctx* ctx, int n);           /* M:173   wait until <= n commit points are pending */
int ks_synchronize(ks_ctx* ctx);                            /* M:205   synchronize */
int ks_has_gpu_work(ks_ctx* ctx);                           /* M:157   has_gpu_work */

/* Device-side stopwatch on the context's stream (the timed `run` of M:377-456 measures with
 * the host clock around commit+wait; CUDA events time the device itself). */
int ks_timer_begin(ks_ctx* ctx);
int ks_timer_end_ms(ks_ctx* ctx, float* ms);               /* synchronises, returns elapsed milliseconds */

/* Record the ops enqueued between begin and end into a replayable CUDA graph: the B200
 * counterpart of keeping one open encoder per token (M:137-155, M:308-312) -- one submission
 * replays a whole token.  Ops are capturable because none allocates or synchronises. */
typedef struct ks_graph ks_graph;
int ks_graph_begin(ks_ctx* ctx);
ks_graph* ks_graph_end(ks_ctx* ctx);                       /* NULL on failure (see ks_last_error) */
int ks_graph_launch(ks_ctx* ctx, ks_graph* g);
void ks_graph_free(ks_ctx* ctx, ks_graph* g);

/* ---- launch plans: OptSchedule {tg, vec, unroll, nsg, nr0} + ms of
 * crates/ksearch_ir/src/kernel.rs:11-54, retargeted to the knobs of the hand-written matvec
 * kernels.  A zero field means "kernel default". */
typedef struct {
  int variant;      /* bits 0-7 kernel family (0 streamed, 1 direct loads, 2 Q6_K fixed point, 3 Q4_K fixed point out of a shared-memory ring, 4 Q6_K fixed point out of shared-memory rings), 8-15 pipeline stages, 16-23 blocks per column segment (0 = auto) */
  int nr;           /* rows kept in flight per lane group (nr0) */
  int nwarps;       /* warps per block (nsg) */
  int ctas_per_sm;  /* grid = min(tiles, SMs * ctas_per_sm) */
  float ms;         /* measured time of the winning candidate, 0 if untimed */
} ks_plan;
/* Force every matvec launch of this context to use *plan (NULL clears): how the search times
 * a candidate through the ordinary op path (K:2015-2031). */
int ks_plan_override(ks_ctx* ctx, const ks_plan* plan);
/* Plan table of the context, keyed by (op, rows, cols, n_tok); op is "mv_q4k", "mv_q6k", "gu_q4k"
 * (gate||up, rows of one matrix) or "qkv_q4k" (rows = q_rows + 2*kv_rows).  plan_plan == NULL erases. */
int ks_plan_set(ks_ctx* ctx, const char* op, size_t rows, size_t cols, int n_tok, const ks_plan* plan);
int ks_plan_get(const ks_ctx* ctx, const char* op, size_t rows, size_t cols, int n_tok, ks_plan* out);
/* CG:178-246 beam_search_matvec + K:1985 Eng::beam_matvec: use the cached plan of this chip if there is
 * one, else time every candidate (beam.rs:26-65) on synthetic weights, keep and cache the fastest.
 * Allocates scratch: call at load time, not on the decode path.  kv_rows only for "qkv_*". */
int ks_plan_search(ks_ctx* ctx, const char* op, size_t rows, size_t kv_rows, size_t cols, int n_tok, ks_plan* best);
int ks_plan_candidates(const char* op, ks_plan* out, int max_out);     /* beam.rs:26-65 */
/* The on-disk plan cache (beam.rs:67-139, plan_cache.rs:9-38): <dir>/<key>_<hash(key,chip)>.txt holding
 * k=v lines.  dir == NULL: $KSEARCH_BEAM_CACHE or ~/.cache/ksearch/beam.  No GPU needed. */
int ks_plan_file_name(const char* key, const char* chip, char* out, size_t out_len);
int ks_plan_file_save(const char* dir, const char* key, const char* chip, const ks_plan* plan);
int ks_plan_file_load(const char* dir, const char* key, const char* chip, ks_plan* plan);

/* ---- dequant test hook: GG:577-794 dequant_blocks (Q4_0 / Q4_K / Q6_K) --- */
int ks_dequant(ks_ctx* ctx, ks_dtype dtype, const ks_buf* src, size_t src_byte_off, size_t nelem,
               ks_buf* dst_f32, size_t dst_off);

/* ---- load-time requantisation to Q4_K: GG:803-1016 make_qkx2_quants + quantize_f32_to_q4k ----
 * The reference's loader turns Q6_K ffn_down / attn_v tensors, and f32 / bf16 ones, into Q4_K on the host before
 * upload (GP:415-440 ensure_weight: dequant_to_f32, then quantize_f32_to_q4k).  The same arithmetic on the GPU,
 * byte for byte: nelem source elements (a multiple of 256; Q6K, Q4K, F16 or F32) -> nelem / 256 blocks of 144
 * bytes.  Byte offsets are multiples of 4. */
int ks_quantize_q4k(ks_ctx* ctx, ks_dtype src_dtype, const ks_buf* src, size_t src_byte_off, size_t nelem,
                    ks_buf* dst_q4k, size_t dst_byte_off);

/* ---- matvec family ------------------------------------------------------- */
/* y[t, r] = sum_c deq(W)[r, c] * x[t, c], t < n_tok (1..256).  x is [n_tok, cols],
 * y is [n_tok, rows].  K:137 matvec_wd, K:1446 matvec_wd_at (offsets),
 * K:1414 matvec_batch: up to 8 rows share one GEMV pass over the weights; 9..256 rows take the route the
 * reference gives to mul_mm (crates/ksearch_codegen/src/render.rs:1073-1291), here a tensor-core GEMM
 * (f32 activations, Q4K / Q6K weights, cols a multiple of 256, x_off a multiple of 4).  The first such call
 * grows a scratch buffer inside the context: make it outside any ks_graph capture. */
int ks_matvec(ks_ctx* ctx, size_t rows, size_t cols, ks_dtype wdtype, const ks_buf* W, size_t w_byte_off,
              ks_dtype act, const ks_buf* x, size_t x_off, ks_buf* y, size_t y_off, int n_tok);
/* K:227 matvec_qkv_wds: three outputs in one launch. */
int ks_matvec_qkv(ks_ctx* ctx, size_t q_rows, size_t kv_rows, size_t cols, ks_dtype dq, ks_dtype dk, ks_dtype dv,
                  const ks_buf* Wq, const ks_buf* Wk, const ks_buf* Wv, ks_dtype act, const ks_buf* x,
                  ks_buf* q, ks_buf* k, ks_buf* v);
/* K:953 matvec_gate_up_gelu_wd: out[i] = gelu_tanh(clamp(Wg[i].x, +-20)) * (Wu[i].x). */
int ks_matvec_gate_up_gelu(ks_ctx* ctx, size_t rows, size_t cols, ks_dtype wdtype, const ks_buf* Wg,
                           const ks_buf* Wu, ks_dtype act, const ks_buf* x, ks_buf* y);
/* RMSNorm fused into the matvec that follows it: K:278 rmsnorm_matvec_wd, K:379 rmsnorm_matvec_qkv_wds,
 * K:1004 rmsnorm_matvec_gate_up_gelu_wd.  The matvec applies x2 = (x*rsqrt(mean(x^2)+eps))*w_norm while
 * it stages its input (Q4K weights, cols <= 4096).  When y_prev != NULL the residual update of K:539 is
 * fused in front as well: x' = x + rms(y_prev)*w_post is written to out_x (which must not alias x) and
 * the norm is taken of x'.  y_prev, w_post, out_x are NULL together. */
int ks_rmsnorm_matvec(ks_ctx* ctx, size_t rows, size_t cols, float eps, ks_dtype wdtype, ks_dtype act, const ks_buf* x,
                      const ks_buf* w_norm, const ks_buf* W, ks_buf* y, const ks_buf* y_prev, const ks_buf* w_post,
                      ks_buf* out_x);
int ks_rmsnorm_matvec_qkv(ks_ctx* ctx, size_t q_rows, size_t kv_rows, size_t cols, float eps, ks_dtype wdtype,
                          ks_dtype act, const ks_buf* x, const ks_buf* w_norm, const ks_buf* Wq, const ks_buf* Wk,
                          const ks_buf* Wv, ks_buf* q, ks_buf* k, ks_buf* v, const ks_buf* y_prev,
                          const ks_buf* w_post, ks_buf* out_x);
int ks_rmsnorm_matvec_gate_up_gelu(ks_ctx* ctx, size_t rows, size_t cols, float eps, ks_dtype wdtype, ks_dtype act,
                                   const ks_buf* x, const ks_buf* w_norm, const ks_buf* Wg, const ks_buf* Wu, ks_buf* y,
                                   const ks_buf* y_prev, const ks_buf* w_post, ks_buf* out_x);

/* Blocking convenience for callers that hold HOST memory: copies x up, runs
 * ks_matvec, copies y back.  W must already be resident (a ks_buf). */
int ks_matvec_host(ks_ctx* ctx, size_t rows, size_t cols, ks_dtype wdtype, const ks_buf* W, size_t w_byte_off,
                   const float* x_host, float* y_host, int n_tok);

/* ---- RMSNorm family ------------------------------------------------------ */
/* K:456-535 rmsnorm / rmsnorm_at / rmsnorm_add / rmsnorm_add_scale and the
 * *_rows forms K:1478-1560: y = (x*rsqrt(mean(x^2)+eps))*w [+ res] [* scale].
 * res may be NULL; scale is applied only when has_scale != 0.  w: [n] in `act`. */
int ks_rmsnorm(ks_ctx* ctx, size_t n, size_t rows, float eps, ks_dtype act, const ks_buf* x, size_t x_off,
               const ks_buf* w, const ks_buf* res, size_t res_off, int has_scale, float scale, ks_buf* y,
               size_t y_off);
/* K:539 rmsnorm_add_then_rmsnorm: out_x = res + rms(y)*w_post; out_x2 = rms(out_x)*w_ffn. */
int ks_rmsnorm_add_then_rmsnorm(ks_ctx* ctx, size_t n, size_t rows, float eps, ks_dtype act, const ks_buf* y,
                                const ks_buf* w_post, const ks_buf* res, const ks_buf* w_ffn, ks_buf* out_x,
                                ks_buf* out_x2);
/* K:1257 rmsnorm_per_head_qkv_q40_off (n_tok == 1) and K:1750 .._batch:
 * Q: per-head RMS*w then RoPE -> q_out; K: RMS*w, RoPE, Q4_0 pack; V: RMS (no
 * weight), Q4_0 pack.  rope is f32 [*, hd] = cos[hd/2] || sin[hd/2] per position,
 * rope_off in elements.  Token t writes its KV rows at kv_byte_off +
 * t*n_kv*(hd/32*18). */
int ks_rmsnorm_per_head_qkv_q40(ks_ctx* ctx, size_t n_q, size_t n_kv, size_t hd, size_t n_tok, float eps,
                                ks_dtype act, const ks_buf* q, const ks_buf* qw, const ks_buf* rope,
                                size_t rope_off, const ks_buf* k, const ks_buf* kw, const ks_buf* v,
                                ks_buf* q_out, ks_buf* kv_k, ks_buf* kv_v, size_t kv_byte_off);

/* ---- decode attention over a Q4_0 cache ---------------------------------- */
/* K:1157 sdpa_hybrid_kv (one slot) and the slot-batched form used by serving.
 * q/out: [n_slots, n_q*hd].  K, V: slot s starts at kv_byte_off + s*slot_stride_bytes,
 * logical layout [max_t, n_kv, hd] in Q4_0.  meta: f32 [n_slots, 4] = (tlen, start, -, -)
 * read ON THE DEVICE (GP:636-644), so one captured launch serves every length.
 * Scores are scale*(q.k); the reference uses scale = 1.  n_splits partitions of
 * the context per KV head (1..KS_SDPA_MAX_SPLITS; 0 = pick from max_t); tmp must
 * hold ks_sdpa_tmp_floats() f32 when n_splits != 1 (K:1117 `tmp`). */
size_t ks_sdpa_tmp_floats(size_t n_slots, size_t n_q, size_t hd, int n_splits);
int ks_sdpa_pick_splits(const ks_ctx* ctx, size_t n_slots, size_t n_kv, size_t max_t);
int ks_sdpa_decode(ks_ctx* ctx, size_t n_slots, size_t n_q, size_t n_kv, size_t hd, size_t max_t,
                   ks_dtype kv_dtype, float scale, ks_dtype act, const ks_buf* q, const ks_buf* K,
                   const ks_buf* V, size_t kv_byte_off, size_t slot_stride_bytes, const ks_buf* meta,
                   ks_buf* tmp, ks_buf* out, int n_splits);

/* ---- small ops ------------------------------------------------------------ */
/* K:1181 quantize_q40: n values (n % 32 == 0) -> Q4_0 at dst + dst_byte_off. */
int ks_quantize_q40(ks_ctx* ctx, size_t n, ks_dtype act, const ks_buf* src, size_t src_off, ks_buf* dst,
                    size_t dst_byte_off);
/* K:1364 copy_scale_indexed_wd / K:1387 .._batch_wd: dst[b, i] = scale * deq(src)[uint(idx[b])*n + i];
 * idx holds token ids as f32.  src dtype: F32, F16, Q4K or Q6K. */
int ks_copy_scale_indexed(ks_ctx* ctx, size_t n, size_t batch, float scale, ks_dtype src_dtype, const ks_buf* src,
                          const ks_buf* idx, size_t idx_off, ks_dtype act, ks_buf* dst);
/* K:1966 softcap_argmax: index of max cap*tanh(x/cap), ties to the lower index, written as one f32
 * (like the reference, so the index is exact only below 2^24 = 16,777,216).  1 <= n <= 2^31. */
int ks_softcap_argmax(ks_ctx* ctx, size_t n, float cap, ks_dtype act, const ks_buf* logits, ks_buf* out_idx,
                      size_t out_off);
/* No counterpart in the reference.  The same arg-max as ks_softcap_argmax (f32 logits) for callers that
 * cannot allocate device memory and so cannot own a ks_ctx (whose creation allocates): a host runtime
 * that pre-carved all device memory into its own arena, a plugin under a fixed memory budget, code that
 * must not trigger the implicit synchronisation of cudaMalloc.  It takes raw device pointers and a
 * stream (NULL = the default stream) and allocates nothing: the cross-block scratch is a fixed array
 * inside the library image (about 4 KB; every GPU that loads the library holds it until exit).
 *  - n <= 4,194,304 (KS_ERR_INVALID beyond; message via ks_last_error(NULL)).
 *  - The first call on a device looks up the array's device address; make that first call outside
 *    any stream capture.
 *  - All calls share the array: two calls that may overlap on the GPU (different streams) race.
 *    Calls on one stream are safe; the arrival counter is cleared on the stream before each launch. */
int ks_softcap_argmax_noalloc(int device, void* stream, size_t n, float cap, const float* logits_dev,
                              float* out_idx_dev);
/* K:695 gelu_mul: y = gelu_tanh(clamp(g)) * u (the unfused fallback of the gate/up path). */
int ks_gelu_mul(ks_ctx* ctx, size_t n, ks_dtype act, const ks_buf* g, const ks_buf* u, ks_buf* y);

/* ---- decode driver: GemmaPrimModel (GP:76-132, 881-1275, 1616-1768) + KvPool (KV:24-230) ----
 * Dense layers that own their KV cache; no per-layer embeddings, sliding window or shared KV. */
typedef struct ks_model ks_model;

/* ---- CPU sampling of the serve surface (crates/ksearch_gemma/src/sample.rs:9-81); host code, no GPU needed ----
 * cap * tanh(x / cap) when cap > 0, then: temperature < 1e-6 -> greedy arg-max (first of equal values, the device
 * kernel's choice); otherwise softmax at that temperature, tokens below min_p * p_max dropped, one multinomial draw
 * from splitmix32(seed | 1).  Returns the token id. */
uint32_t ks_sample_softcap_min_p(const uint16_t* logits_f16, size_t n, float cap, float temperature, float min_p, uint32_t seed);
uint32_t ks_sample_softcap_min_p_f32(const float* logits, size_t n, float cap, float temperature, float min_p, uint32_t seed);

/* ---- GGUF container (GG:130-417 Gguf::open and accessors); host code, no GPU needed -------------------------
 * ks_gguf_open maps the file and parses header, key/value metadata and tensor infos; NULL on failure with the
 * reason in err ("not a GGUF file (bad magic)", "unsupported GGUF version N", "truncated GGUF file", ... — where the
 * reference panics).  ggml type ids as in the file (GG:20-31: F32 0, F16 1, Q4_0 2, Q4_K 12, Q5_K 13, Q6_K 14, BF16 30). */
typedef struct ks_gguf ks_gguf;
ks_gguf* ks_gguf_open(const char* path, char* err, size_t err_len);
void ks_gguf_close(ks_gguf* g);
int ks_gguf_version(const ks_gguf* g);
size_t ks_gguf_n_tensors(const ks_gguf* g);
size_t ks_gguf_n_kv(const ks_gguf* g);
uint64_t ks_gguf_data_offset(const ks_gguf* g);                       /* first byte of tensor data: aligned to general.alignment (default 32) */
const char* ks_gguf_tensor_name(const ks_gguf* g, size_t i);          /* file order; NULL past the end */
/* GG:262-324 tensor / tensor_type / tensor_file_offset: up to 4 dims (ne0 first), absolute file offset, byte length.
 * KS_ERR_INVALID when the tensor is not in the file. */
int ks_gguf_tensor(const ks_gguf* g, const char* name, uint32_t* ggml_type, uint32_t* n_dims, uint64_t* dims4,
                   uint64_t* file_offset, uint64_t* nbytes);
const void* ks_gguf_tensor_raw(const ks_gguf* g, const char* name);   /* GG:277 tensor_raw: bytes inside the mapping; NULL if unknown */
/* GG:326-417 metadata accessors with the reference's coercions; 1 = found, 0 = absent or of another type */
int ks_gguf_has_key(const ks_gguf* g, const char* key);
int ks_gguf_get_u32(const ks_gguf* g, const char* key, uint32_t* out);   /* U32, I32, U64, U16 */
int ks_gguf_get_u64(const ks_gguf* g, const char* key, uint64_t* out);   /* U64, U32, I32 */
int ks_gguf_get_f32(const ks_gguf* g, const char* key, float* out);      /* F32, F64 */
int ks_gguf_get_bool(const ks_gguf* g, const char* key, int* out);
const char* ks_gguf_get_str(const ks_gguf* g, const char* key);          /* NULL if absent */
long long ks_gguf_arr_len(const ks_gguf* g, const char* key, uint32_t* elem_type);   /* -1: absent or not an array */
long long ks_gguf_get_arr_u32(const ks_gguf* g, const char* key, uint32_t* out, size_t max);  /* element count, -1: other type */
long long ks_gguf_get_arr_i32(const ks_gguf* g, const char* key, int32_t* out, size_t max);
long long ks_gguf_get_arr_f32(const ks_gguf* g, const char* key, float* out, size_t max);
long long ks_gguf_get_arr_bool(const ks_gguf* g, const char* key, uint8_t* out, size_t max);
const char* ks_gguf_get_arr_str(const ks_gguf* g, const char* key, size_t i);
typedef struct {              /* the GemmaConfig fields the dense path uses (crates/ksearch_gemma/src/lib.rs:14-36) */
  int n_layers, hidden, ffn, n_q, n_kv, hd, vocab, max_seq;
  int n_slots;                /* KvPool max_batch (1..64): slots that can advance together */
  float eps, rope_theta, softcap, attn_scale;   /* attn_scale: the reference uses 1 */
  int embd_dtype;             /* ks_dtype of the tied token_embd / lm_head: KS_Q4K or KS_Q6K */
  int act;                    /* ks_dtype of activations and norm weights: KS_F32 or KS_F16 */
  int sliding_window;         /* GemmaConfig.sliding_window: positions a sliding-window layer attends to; 0 = every layer is full */
  unsigned long long swa_layers;  /* bit l set: layer l is a sliding-window layer (GemmaConfig.swa_pattern, lib.rs:137-147; <= 64 layers) */
} ks_model_config;
typedef struct {              /* GenerateStats (crates/ksearch_gemma/src/lib.rs:189-205), device-timed */
  int prefill_tokens, decode_tokens;
  float prefill_ms_device, decode_ms_device;
} ks_generate_stats;

ks_model* ks_model_create(ks_ctx* ctx, const ks_model_config* cfg);          /* GP:135-413 load, minus the GGUF file */
void ks_model_destroy(ks_model* m);
int ks_model_warm_plans(ks_model* m, int n_tok);                             /* GP:254-290 BEAM warm at load; returns plans found */
/* Tensor names are the GGUF names the reference loads (GP:149-183, 356-357): token_embd.weight,
 * output_norm.weight, blk.N.{attn_q,attn_k,attn_v,attn_output,ffn_gate,ffn_up,ffn_down}.weight (Q4_K),
 * blk.N.{attn_norm,attn_q_norm,attn_k_norm,post_attention_norm,ffn_norm,post_ffw_norm}.weight (act dtype). */
size_t ks_model_tensor_bytes(const ks_model* m, const char* name);           /* 0 if unknown */
int ks_model_upload_tensor(ks_model* m, const char* name, const void* host, size_t bytes);  /* GP:415-451 ensure_weight */
/* The same with the file's tensor type: bytes of the resident type are copied; a Q6K, F16 or F32 matrix whose resident
 * form is Q4_K is requantised on the device as the reference's loader does on the host (GP:422-440, GG:803-1016). */
int ks_model_upload_tensor_as(ks_model* m, const char* name, ks_dtype src_dtype, const void* host, size_t bytes);
/* Every tensor the model holds, by its GGUF name, out of an open file (GP:149-183, 356-357, 415-451): element counts
 * are checked against the model's shapes, F32 / F16 / Q4_K / Q6_K tensors are uploaded or requantised as
 * ks_model_upload_tensor_as does, F32 norm weights are narrowed with the reference's own f32 -> f16 (GGL:39-75)
 * when the model keeps f16 activations.  KS_ERR_INVALID "tensor not found: NAME" when one is missing. */
int ks_model_load_gguf(ks_model* m, const ks_gguf* g);
const void* ks_model_tensor_ptr(const ks_model* m, const char* name);      /* device address of a resident tensor, NULL if unknown */
size_t ks_model_weight_bytes(const ks_model* m);
int ks_model_slot_alloc(ks_model* m);                                        /* KV:136 alloc -> slot id, or KS_ERR_STATE "KvPool full" */
int ks_model_slot_free(ks_model* m, int slot);                               /* KV:168 free */
int ks_model_slot_reset(ks_model* m, int slot);                              /* KV:147 clear_slot + GP:1644 reset */
int ks_model_slot_seq_len(const ks_model* m, int slot);                      /* KV:161 seq_len */
int ks_model_slot_active(const ks_model* m);                                 /* KV:179 active_batch().len() */
int ks_model_forward(ks_model* m, int first_slot, int n_slots, const int* tokens, int want_logits);   /* GP:881 forward_token, enqueue only */
/* Prompt tokens of one slot without logits, up to 128 per pass over the weights (the rows of a chunk attend
 * causally inside the chunk).  GemmaPrimModel::prefill_chunk (crates/ksearch_gemma/src/gemma_prim.rs:1305-1315):
 * chunks of more than 8 rows run every matrix through the tensor-core GEMM (the reference's mul_mm), shorter
 * ones through the batch GEMV (crates/ksearch_kernels/src/lib.rs:1414).  The slot advances by n_tokens;
 * enqueues only, apart from the wait for the pinned staging words between chunks. */
int ks_model_prefill(ks_model* m, int slot, const int* tokens, int n_tokens);
int ks_model_decode_token(ks_model* m, int first_slot, int n_slots, const int* tokens, int* next);    /* GP:1616 decode_token, blocking */
int ks_model_generate(ks_model* m, int slot, const int* prompt, int n_prompt, int n_new, int max_inflight,
                      int* out, ks_generate_stats* stats);                   /* GP:1658 generate_timed */
const void* ks_model_debug_ptr(const ks_model* m, int which, int slot);      /* test hook: 0 residual x, 1 logits, 2 phase stamps (first, last block), 3 every block's stamps */
/* Knobs of a slot's persistent decode kernel (tests, profiling): what = 0 polls before a device-side wait gives
 * up, 1 = make one wait of the token (a grid barrier; with KSEARCH_DECODE_KERNEL=2 one stage of every layer) wait
 * for something nobody writes (exercises the KS_ERR_TIMEOUT path; 0 = off); KSEARCH_DECODE_KERNEL=2 only: 2 =
 * context length from which attention is split across blocks, 3 = record per-phase time stamps (the counterpart
 * of KSEARCH_PROFILE, GP:885,924-929,1260-1273; also switched on by that environment variable; the default
 * kernel always records its stamps). */
int ks_model_debug_set(ks_model* m, int slot, int what, unsigned value);
/* One slot's rows of a layer's KV cache on the device, [max_seq, n_kv, hd] in Q4_0 (KV:24-60 holds one such
 * buffer per owning layer); which: 0 = K, 1 = V.  For tests and for hosts that snapshot or restore a slot. */
void* ks_model_kv_ptr(const ks_model* m, int layer, int which, int slot);
size_t ks_model_kv_slot_bytes(const ks_model* m);                            /* bytes of one slot in one layer's K (or V) */

/* ---- row-sharded matvec over the GPUs of one box -------------------------------------------------
 * No counterpart in the reference: crates/ksearch_metal/src/lib.rs:33 takes the system default device and
 * nothing there spans devices.  One process and one ks_ctx per GPU.  The matrices served are the reference's
 * largest matvecs, the tied lm_head (GP:1222-1242) and the FFN projections (GP:1130-1157); rank k owns a
 * contiguous run of rows = a contiguous byte range of the GGUF tensor, x is replicated, ONE exchange follows.
 * Everything is enqueued on the context's stream (no host synchronisation; capturable in a ks_graph). */
typedef struct ks_comm ks_comm;
#define KS_COMM_ID_BYTES 128
enum { KS_GATHER_NONE = 0, KS_GATHER_NCCL = 1 };
/* Rank 0 creates the 128-byte rendezvous id and hands it to the other ranks over any host channel. */
int ks_comm_unique_id(void* id_out);
/* Collective: every rank calls it with the same id.  n_ranks == 1 needs no id and no NCCL. */
ks_comm* ks_comm_init(ks_ctx* ctx, int n_ranks, int rank, const void* unique_id);
void ks_comm_destroy(ks_comm* comm);
/* Optional: the arg-max exchange over peer memory (NVLink) instead of NCCL.  Every rank creates its mailbox and
 * gets a 64-byte handle; the host gathers the handles of all ranks (rank r's at r * 64) and every rank opens them.
 * From then on ks_argmax_sharded is one kernel that stores this rank's (value, index) word into every peer's
 * mailbox, waits (bounded; KS_ERR_TIMEOUT through the status word) for the peers' words and merges them.
 * ks_comm_set: what 0 = use peer memory (1, default once open) or NCCL (0); 1 = poll limit of the peer wait;
 * 2 = zero this rank's mailbox and step counter (all ranks, nothing in flight). */
#define KS_COMM_P2P_HANDLE_BYTES 64
int ks_comm_p2p_handle(ks_comm* comm, void* handle_out);
int ks_comm_p2p_open(ks_comm* comm, const void* all_handles);
int ks_comm_set(ks_comm* comm, int what, unsigned value);
int ks_comm_rank(const ks_comm* comm);
int ks_comm_size(const ks_comm* comm);
/* all[all_off + r*count .. ] of every rank <- rank r's slot of the same buffer (in-place all-gather, f32). */
int ks_comm_all_gather_f32(ks_comm* comm, ks_buf* all, size_t all_off, size_t count);
/* y_all[y_off + rank*rows_per_rank + i] = W_local[i] . x for this rank's rows_local (<= rows_per_rank) rows,
 * then (gather == KS_GATHER_NCCL) the in-place all-gather of the slots.  f32 x and y, one token. */
int ks_matvec_sharded(ks_comm* comm, size_t rows_local, size_t rows_per_rank, size_t cols, ks_dtype wdtype,
                      const ks_buf* W_local, size_t w_byte_off, const ks_buf* x, size_t x_off, ks_buf* y_all,
                      size_t y_off, int gather);
/* Greedy token from row-sharded logits (K:1966 softcap_argmax over the whole vocabulary): arg-max of this
 * rank's rows_local logits, all-gather of one (value, index) pair per rank, merge with ties to the lower
 * index (crates/ksearch_codegen/src/render.rs:2355).  row0: global index of this rank's first logit.
 * Every rank gets the same index, as one f32. */
int ks_argmax_sharded(ks_comm* comm, size_t rows_local, size_t row0, float cap, const ks_buf* logits_local,
                      size_t logits_off, ks_buf* out_idx, size_t out_off);

#ifdef __cplusplus
}
#endif
#endif /* KSEARCH_CUDA_H */

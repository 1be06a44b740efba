// Decode driver: the op sequence of GemmaPrimModel::forward_token
// (crates/ksearch_gemma/src/gemma_prim.rs:881-1275) for dense layers that own
// their KV cache, the slot pool of crates/ksearch_gemma/src/kv_pool.rs:24-230,
// and the generate loop of gemma_prim.rs:1658-1768.
//
// What differs from the reference, by design for this GPU:
//   * the position, the (tlen, start) attention record and the token id all
//     live on the device (the reference already keeps the token id there,
//     gemma_prim.rs:1237-1242), so ONE captured CUDA graph replays any token;
//   * up to 8 slots advance together through one pass over the weights
//     (the reference runs slots serially, scheduler.rs:163-231);
//   * the residual update after the FFN and the next layer's attention norm
//     run as one launch (the same two-output kernel as after attention).
// Per-layer embeddings, sliding windows and shared-KV layers of real Gemma-4
// checkpoints are not part of this driver.
#include <cmath>
#include <cstdlib>
#include <utility>
#include <cstring>
#include <map>
#include <string>
#include <atomic>
#include <chrono>
#include <vector>

#include "ks_internal.h"

namespace {

// (tlen, start) of a row with kv_len cached positions: everything for a full-attention layer, the last `window`
// positions for a sliding-window layer (gemma_prim.rs:1009-1016).  meta_swa may be null (no such layers).
__device__ __forceinline__ void write_meta_pair(float* meta, float* meta_swa, int row, int kv_len, int window) {
  meta[row * 4 + 0] = (float)kv_len;
  meta[row * 4 + 1] = 0.0f;
  meta[row * 4 + 2] = 0.0f;
  meta[row * 4 + 3] = 0.0f;
  if (meta_swa) {
    const int start = kv_len > window ? kv_len - window : 0;
    meta_swa[row * 4 + 0] = (float)(kv_len - start);
    meta_swa[row * 4 + 1] = (float)start;
    meta_swa[row * 4 + 2] = 0.0f;
    meta_swa[row * 4 + 3] = 0.0f;
  }
}
__global__ void begin_token_kernel(int n, const int* pos, float* meta, float* meta_swa, int window) {
  ks_pdl_entry();
  const int s = threadIdx.x;
  if (s < n) write_meta_pair(meta, meta_swa, s, pos[s] + 1, window);
}
__global__ void end_token_kernel(int n, int* pos) {
  ks_pdl_entry();
  const int s = threadIdx.x;
  if (s < n) pos[s] += 1;
}
// What a blocking step brings back: the n next-token ids and, behind them, whether a device-side wait gave up.
// `host` (pinned host memory, may be null): the same values where the host can see them without a copy — ids at
// [0, n), the flag at [n_slots], and last, behind a system-wide fence, the request word the host left at
// [n_slots + 2] echoed to [n_slots + 1]: a host that spins on the echo needs neither a copy nor a stream wait.
__global__ void collect_kernel(int n, const float* tok, const unsigned* err_word, float* ret, float* host, int n_slots) {
  ks_pdl_entry();
  const int s = threadIdx.x;
  if (s < n) {
    ret[s] = tok[s];
    if (host) host[s] = tok[s];
  }
  if (s == n) {
    const float f = err_word[0] ? 1.0f : 0.0f;
    ret[n] = f;
    if (host) host[n_slots] = f;
  }
  if (host) {
    __threadfence_system();
    __syncthreads();
    if (s == 0) {
      volatile unsigned* w = reinterpret_cast<volatile unsigned*>(host);
      w[n_slots + 1] = w[n_slots + 2];
    }
  }
}
__global__ void set_state_kernel(int slot, int pos_value, int* pos) { ks_pdl_entry(); pos[slot] = pos_value; }
// A prompt chunk: row t of the chunk sits at position base + t of ONE slot (causal: it sees base + t + 1 positions).
__global__ void begin_chunk_kernel(int n, const int* base, int* cpos, float* meta, float* meta_swa, int window) {
  ks_pdl_entry();
  const int t = threadIdx.x;
  if (t < n) {
    cpos[t] = base[0] + t;
    write_meta_pair(meta, meta_swa, t, base[0] + t + 1, window);
  }
}
__global__ void end_chunk_kernel(int n, int* base) {
  ks_pdl_entry();
  if (threadIdx.x == 0) base[0] += n;
}

struct Tensor {
  void* dptr = nullptr;
  size_t bytes = 0;
  bool set = false;
  int dtype = KS_F32;  // what the resident bytes are
};

struct Layer {
  Tensor wq, wk, wv, wo, wgate, wup, wdown;
  Tensor attn_norm, q_norm, k_norm, post_attn_norm, ffn_norm, post_ffw_norm;
};

}  // namespace

struct ks_model {
  ks_ctx* ctx = nullptr;
  ks_model_config cfg{};
  std::vector<Layer> layers;
  Tensor token_embd, output_norm;
  std::map<std::string, Tensor*> by_name;
  void* arena = nullptr;  // all weights, one allocation
  size_t arena_bytes = 0;
  // KV pool: per layer K and V, [n_slots, max_seq, n_kv, hd] Q4_0
  std::vector<uint8_t*> kv_k, kv_v;
  size_t slot_stride = 0;
  std::vector<char> occupied;
  std::vector<int> seq_len;
  // activations, n_slots rows each
  void *xb = nullptr, *xn = nullptr;  // second residual buffer (fused chain ping-pong), normed x for the head
  bool fused = false;                 // norms folded into the matvec prologues
  void *x = nullptr, *x2 = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *o = nullptr, *ff = nullptr,
       *logits = nullptr;
  float* rope = nullptr;
  float* tok = nullptr;   // [2][n_slots] f32 token ids, ping-pong (gemma_prim.rs:98-99)
  int* pos = nullptr;     // [n_slots]
  float* meta = nullptr;  // [n_slots][4]
  float* meta_swa = nullptr;  // the same for sliding-window layers; null when the model has none
  float* attn_tmp = nullptr;
  int n_splits = 1;
  float* ret = nullptr;       // [n_slots][n_slots + 1] per first slot: next ids + status flag of the last blocking step
  float* host_tok = nullptr;  // pinned ring for token read-back
  float* host_ret = nullptr;  // pinned: what collect_kernel leaves for a blocking step (ids, flag, echo, request word)
  unsigned req_id = 0;        // the last request word handed to collect_kernel
  int solo_max = 2;           // up to this many slots step as one persistent-kernel pass each
  size_t host_tok_n = 0;
  // graphs keyed by (first slot, n slots, src parity, want_logits)
  std::map<uint64_t, cudaGraphExec_t> graphs;
  std::map<uint64_t, size_t> graph_nodes;
  std::vector<void*> owned;
  std::vector<char> tok_src;  // per slot: which half of the ping-pong holds its next input id
  // ids that come from the host are read by the embedding kernel straight out of this pinned, device-visible array
  // (one word per slot; source index 2): no staging copy in front of the step
  float* host_ids = nullptr;
  // one persistent decode kernel per slot (both null: shape not covered, tried once); decode_kernel
  // picks which of the two is built: 1 = grid barriers (ks_mega.cu), 2 = tagged-word dataflow (ks_flow.cu)
  struct Mega {
    ks_mega* bar = nullptr;
    ks_flow* flow = nullptr;
    explicit operator bool() const { return bar || flow; }
  };
  std::map<int, Mega> mega;
  bool use_mega = false;
  int decode_kernel = 1;
  // prompt chunks (ks_model_prefill): KS_PREFILL_CHUNK rows of activations of their own
  void *cx = nullptr, *cxb = nullptr, *cx2 = nullptr, *cq = nullptr, *ck = nullptr, *cv = nullptr, *co = nullptr, *cff = nullptr;
  float* ctok = nullptr;
  int* cpos = nullptr;
  float* cmeta = nullptr;
  float* cmeta_swa = nullptr;
  float* cattn_tmp = nullptr;
  int chunk = 1;  // tokens per prompt chunk: as many as the matvec kernels can stage side by side (<= KS_PREFILL_CHUNK)
  // rows per pass through the tensor-core GEMM (0: not available, activations are not f32); its scratch inside the
  // context's GEMM workspace: the split operand image, two sets of k-split partials
  int gemm_chunk = 0;
  void* gemm_xt = nullptr;
  float* gemm_p0 = nullptr;
};

namespace {

size_t act_b(const ks_model* m) { return ks_act_bytes((ks_dtype)m->cfg.act); }

int dev_alloc(ks_model* m, void** p, size_t bytes) {
  cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
  if (e != cudaSuccess) return ks_fail(m->ctx, KS_ERR_OOM, "model: cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
  cudaMemsetAsync(*p, 0, bytes ? bytes : 16, m->ctx->stream);
  m->owned.push_back(*p);
  return KS_OK;
}

constexpr int KS_PREFILL_CHUNK = 8;  // tokens per pass over the weights (the matvec kernels take up to 8)
constexpr int KS_GEMM_CHUNK = 256;   // rows per pass when the tensor-core GEMM takes the matrices (f32 activations)
constexpr size_t KS_STAGE_IDS = 256; // pinned words that stage host token ids

// Where a forward pass reads and writes: n rows of activations, their positions, and the KV caches
// behind them.  Decode steps map row s to slot first + s (one cache per row); a prompt chunk maps
// row t to position base + t of ONE slot (every row shares that slot's cache, kv_stride = 0).
struct Lane {
  char *x, *xb, *x2, *xn, *q, *k, *v, *o, *ff, *logits;
  const float* tok_in;
  float* tok_out;
  float* ret;        // where a blocking step's ids and status flag are collected
  int* pos;          // device, one per row
  float* meta;       // device, (tlen, start, -, -) per row
  float* meta_swa;   // the same for sliding-window layers (null: none)
  float* attn_tmp;
  size_t kv_off;     // byte offset of row 0's cache inside every layer's K / V allocation
  size_t kv_stride;  // bytes between the caches of consecutive rows
  int* chunk_base;   // prompt chunk: the slot's position word (rows take base, base + 1, ...); else nullptr
};

Lane slot_lane(ks_model* m, int first, int src) {
  const ks_model_config& g = m->cfg;
  const size_t ab = act_b(m), H = g.hidden, F = g.ffn, qn = (size_t)g.n_q * g.hd, kvn = (size_t)g.n_kv * g.hd;
  Lane L{};
  L.x = (char*)m->x + (size_t)first * H * ab;
  L.xb = (char*)m->xb + (size_t)first * H * ab;
  L.x2 = (char*)m->x2 + (size_t)first * H * ab;
  L.xn = (char*)m->xn + (size_t)first * H * ab;
  L.q = (char*)m->q + (size_t)first * qn * ab;
  L.k = (char*)m->k + (size_t)first * kvn * ab;
  L.v = (char*)m->v + (size_t)first * kvn * ab;
  L.o = (char*)m->o + (size_t)first * qn * ab;
  L.ff = (char*)m->ff + (size_t)first * F * ab;
  L.logits = (char*)m->logits + (size_t)first * g.vocab * ab;
  L.tok_in = src == 2 ? m->host_ids + first : m->tok + (size_t)src * g.n_slots + first;
  L.tok_out = m->tok + (size_t)(src == 2 ? 1 : src ^ 1) * g.n_slots + first;
  L.ret = m->ret + (size_t)first * (g.n_slots + 1);
  L.pos = m->pos + first;
  L.meta = m->meta + (size_t)first * 4;
  L.meta_swa = m->meta_swa ? m->meta_swa + (size_t)first * 4 : nullptr;
  L.attn_tmp = m->attn_tmp;
  L.kv_off = (size_t)first * m->slot_stride;
  L.kv_stride = m->slot_stride;
  return L;
}

Lane chunk_lane(ks_model* m, int slot) {
  Lane L{};
  L.x = (char*)m->cx; L.xb = (char*)m->cxb; L.x2 = (char*)m->cx2; L.xn = nullptr;
  L.q = (char*)m->cq; L.k = (char*)m->ck; L.v = (char*)m->cv; L.o = (char*)m->co; L.ff = (char*)m->cff;
  L.logits = nullptr;
  L.tok_in = m->ctok;
  L.tok_out = nullptr;
  L.pos = m->cpos;
  L.meta = m->cmeta;
  L.meta_swa = m->cmeta_swa;
  L.attn_tmp = m->cattn_tmp;
  L.kv_off = (size_t)slot * m->slot_stride;
  L.kv_stride = 0;
  L.chunk_base = m->pos + slot;
  return L;
}

// Context splits of an attention launch over n rows: the rows themselves spread the work over the chip, so each
// row's context is split only as far as about 256 blocks in all need (never beyond what the scratch was sized for).
int att_splits_for(const ks_model* m, int n) {
  int s = ks_sdpa_pick_splits(m->ctx, (size_t)n, (size_t)m->cfg.n_kv, (size_t)m->cfg.max_seq);
  return s > m->n_splits ? m->n_splits : s;
}

unsigned row_threads(int n) { return (unsigned)((n + 1 + 31) / 32 * 32); }  // one thread per row and one more

int lane_begin(ks_model* m, const Lane& L, int n) {
  if (L.chunk_base)
    KS_LAUNCH(m->ctx, (begin_chunk_kernel), 1, row_threads(n), 0, n, (const int*)L.chunk_base, L.pos, L.meta, L.meta_swa, (int)m->cfg.sliding_window);
  else
    KS_LAUNCH(m->ctx, (begin_token_kernel), 1, row_threads(n), 0, n, (const int*)L.pos, L.meta, L.meta_swa, (int)m->cfg.sliding_window);
  return ks_after_launch(m->ctx, "begin_token");
}
int lane_end(ks_model* m, const Lane& L, int n) {
  if (L.chunk_base)
    KS_LAUNCH(m->ctx, (end_chunk_kernel), 1, 32, 0, n, L.chunk_base);
  else
    KS_LAUNCH(m->ctx, (end_token_kernel), 1, row_threads(n), 0, n, L.pos);
  return ks_after_launch(m->ctx, "end_token");
}

// Does any layer attend to a window shorter than the cache?
bool has_window(const ks_model_config& g) { return g.sliding_window > 0 && g.sliding_window < g.max_seq && g.swa_layers != 0; }

// The (tlen, start) rows layer l's attention reads: the sliding-window ones for a sliding-window layer.
const float* layer_meta(const ks_model* m, const Lane& L, int l) {
  return L.meta_swa && ((m->cfg.swa_layers >> l) & 1ull) ? L.meta_swa : L.meta;
}

// One token per row through every layer.
int enqueue_forward(ks_model* m, const Lane& L_, int n, bool want_logits) {
  ks_ctx* c = m->ctx;
  const ks_model_config& g = m->cfg;
  const ks_dtype act = (ks_dtype)g.act;
  const size_t ab = act_b(m);
  const size_t H = g.hidden, F = g.ffn, hd = g.hd, nq = g.n_q, nkv = g.n_kv;
  const size_t qn = nq * hd, kvn = nkv * hd;
  char *x = L_.x, *x2 = L_.x2, *q = L_.q, *k = L_.k, *v = L_.v, *o = L_.o, *ff = L_.ff, *logits = L_.logits;
  const float* tok_in = L_.tok_in;
  float* tok_out = L_.tok_out;
  int* pos = L_.pos;
  int rc;

  if ((rc = lane_begin(m, L_, n))) return rc;
  // embed: x = sqrt(hidden) * deq(token_embd[id])   (gemma_prim.rs:681-683)
  if ((rc = ks_launch_copy_scale_indexed(c, H, n, sqrtf((float)H), (ks_dtype)g.embd_dtype, m->token_embd.dptr, tok_in, act, x))) return rc;
  if ((rc = ks_launch_rmsnorm(c, H, n, g.eps, act, x, m->layers[0].attn_norm.dptr, nullptr, 0, 0.f, x2))) return rc;

  for (int l = 0; l < g.n_layers; l++) {
    const Layer& L = m->layers[l];
    ks_mv_seg qkv[3] = {{(const uint8_t*)L.wq.dptr, q, (unsigned)qn},
                        {(const uint8_t*)L.wk.dptr, k, (unsigned)kvn},
                        {(const uint8_t*)L.wv.dptr, v, (unsigned)kvn}};
    if ((rc = ks_launch_matvec(c, KS_Q4K, qkv, 3, KS_EPI_PLAIN, H, act, x2, n, nullptr))) return rc;
    uint8_t* kk = m->kv_k[l] + L_.kv_off;
    uint8_t* kv = m->kv_v[l] + L_.kv_off;
    if ((rc = ks_launch_per_head_qkv_q40(c, nq, nkv, hd, n, g.eps, act, q, L.q_norm.dptr, m->rope, k, L.k_norm.dptr, v, q,
                                         kk, kv, pos, L_.kv_stride)))
      return rc;
    if ((rc = ks_launch_sdpa(c, n, nq, nkv, hd, g.attn_scale, act, q, kk, kv, L_.kv_stride, layer_meta(m, L_, l), L_.attn_tmp, o, att_splits_for(m, n))))
      return rc;
    ks_mv_seg so{(const uint8_t*)L.wo.dptr, x2, (unsigned)H};
    if ((rc = ks_launch_matvec(c, KS_Q4K, &so, 1, KS_EPI_PLAIN, qn, act, o, n, nullptr))) return rc;
    if ((rc = ks_launch_rmsnorm_add_then_rmsnorm(c, H, n, g.eps, act, x2, L.post_attn_norm.dptr, x, L.ffn_norm.dptr, x, x2))) return rc;
    ks_mv_seg gu[2] = {{(const uint8_t*)L.wgate.dptr, ff, (unsigned)F}, {(const uint8_t*)L.wup.dptr, ff, (unsigned)F}};
    if ((rc = ks_launch_matvec(c, KS_Q4K, gu, 2, KS_EPI_GATE_UP, H, act, x2, n, nullptr))) return rc;
    ks_mv_seg sd{(const uint8_t*)L.wdown.dptr, x2, (unsigned)H};
    if ((rc = ks_launch_matvec(c, KS_Q4K, &sd, 1, KS_EPI_PLAIN, F, act, ff, n, nullptr))) return rc;
    // x += rms(down)*w_post_ffw, then the NEXT norm (next layer's attn_norm, or output_norm) in the same launch
    const void* next_norm = (l + 1 < g.n_layers) ? m->layers[l + 1].attn_norm.dptr : m->output_norm.dptr;
    if ((rc = ks_launch_rmsnorm_add_then_rmsnorm(c, H, n, g.eps, act, x2, L.post_ffw_norm.dptr, x, next_norm, x, x2))) return rc;
  }
  if ((rc = lane_end(m, L_, n))) return rc;
  if (!want_logits) return KS_OK;
  // head: logits = token_embd . rms(x, output_norm); next id = softcap argmax (gemma_prim.rs:1222-1242)
  ks_mv_seg sh{(const uint8_t*)m->token_embd.dptr, logits, (unsigned)g.vocab};
  if ((rc = ks_launch_matvec(c, (ks_dtype)g.embd_dtype, &sh, 1, KS_EPI_PLAIN, H, act, x2, n, nullptr))) return rc;
  for (int s = 0; s < n; s++)
    if ((rc = ks_launch_softcap_argmax(c, g.vocab, g.softcap, act, logits + (size_t)s * g.vocab * ab, tok_out + s))) return rc;
  KS_LAUNCH(c, (collect_kernel), 1, row_threads(n), 0, n, (const float*)tok_out, (const unsigned*)c->ws + KS_WS_ERR_WORD, L_.ret, (float*)m->host_ret, (int)g.n_slots);
  return ks_after_launch(c, "collect");
}

// The same op order for 9..KS_GEMM_CHUNK rows (a prompt chunk, or more slots than the batch matvec stages side by
// side): the matrices go through the tensor-core GEMM, the reference's mul_mm route (forward_prefill_chunk,
// gemma_prim.rs:1317-1607); norms, RoPE/KV pack, attention and GELU are the row-wise kernels above.  f32 only.
int enqueue_forward_gemm(ks_model* m, const Lane& L_, int n, bool want_logits) {
  ks_ctx* c = m->ctx;
  const ks_model_config& g = m->cfg;
  const ks_dtype act = KS_F32;
  const size_t H = g.hidden, F = g.ffn, hd = g.hd, nq = g.n_q, nkv = g.n_kv;
  const size_t qn = nq * hd, kvn = nkv * hd;
  char *x = L_.x, *x2 = L_.x2, *q = L_.q, *k = L_.k, *v = L_.v, *o = L_.o, *logits = L_.logits;
  float* tok_out = L_.tok_out;
  int rc;
  const int att_splits = att_splits_for(m, n);
  if ((rc = lane_begin(m, L_, n))) return rc;
  if ((rc = ks_launch_copy_scale_indexed(c, H, n, sqrtf((float)H), (ks_dtype)g.embd_dtype, m->token_embd.dptr, L_.tok_in, act, x))) return rc;
  if ((rc = ks_launch_rmsnorm(c, H, n, g.eps, act, x, m->layers[0].attn_norm.dptr, nullptr, 0, 0.f, x2))) return rc;
  if ((rc = ks_launch_gemm_split(c, (const float*)x2, H, n, H, m->gemm_xt))) return rc;
  // From here on the normed rows exist only as the image the next GEMM reads: the sums of the o-proj and
  // down-proj partials go straight through the residual update and the next norm into that image.
  ks_gemm_epi epi{};
  epi.eps = g.eps;
  epi.res = (const float*)x;
  epi.out_x = (float*)x;
  epi.xt_out = m->gemm_xt;
  for (int l = 0; l < g.n_layers; l++) {
    const Layer& L = m->layers[l];
    {  // q, k and v rows in one launch (lib.rs:227)
      const uint8_t* Ws[3] = {(const uint8_t*)L.wq.dptr, (const uint8_t*)L.wk.dptr, (const uint8_t*)L.wv.dptr};
      float* ys[3] = {(float*)q, (float*)k, (float*)v};
      const size_t rs[3] = {qn, kvn, kvn};
      if ((rc = ks_launch_gemm_segs(c, KS_Q4K, 3, Ws, rs, H, m->gemm_xt, n, ys, rs, m->gemm_p0, KS_GEMM_PLAIN, nullptr))) return rc;
    }
    uint8_t* kk = m->kv_k[l] + L_.kv_off;
    uint8_t* kv = m->kv_v[l] + L_.kv_off;
    if ((rc = ks_launch_per_head_qkv_q40(c, nq, nkv, hd, n, g.eps, act, q, L.q_norm.dptr, m->rope, k, L.k_norm.dptr, v, q,
                                         kk, kv, L_.pos, L_.kv_stride)))
      return rc;
    if ((rc = ks_launch_sdpa(c, n, nq, nkv, hd, g.attn_scale, act, q, kk, kv, L_.kv_stride, layer_meta(m, L_, l), L_.attn_tmp, o, att_splits)))
      return rc;
    if ((rc = ks_launch_gemm_split(c, (const float*)o, qn, n, qn, m->gemm_xt))) return rc;
    {  // o-proj, x += rms(.) * w_post_attn, image of rms(x) * w_ffn_norm (lib.rs:539)
      const uint8_t* Ws[1] = {(const uint8_t*)L.wo.dptr};
      float* ys[1] = {nullptr};
      epi.w_post = (const float*)L.post_attn_norm.dptr;
      epi.w_norm = (const float*)L.ffn_norm.dptr;
      if ((rc = ks_launch_gemm_segs(c, KS_Q4K, 1, Ws, &H, qn, m->gemm_xt, n, ys, &H, m->gemm_p0, KS_GEMM_NORM_SPLIT, &epi))) return rc;
    }
    {  // gate and up share the operand image; their partials meet in the GeGLU epilogue (lib.rs:953)
      const uint8_t* Ws[2] = {(const uint8_t*)L.wgate.dptr, (const uint8_t*)L.wup.dptr};
      float* ys[2] = {nullptr, nullptr};
      const size_t rs[2] = {F, F};
      if ((rc = ks_launch_gemm_segs(c, KS_Q4K, 2, Ws, rs, H, m->gemm_xt, n, ys, rs, m->gemm_p0, KS_GEMM_GELU_SPLIT, &epi))) return rc;
    }
    {  // down-proj, x += rms(.) * w_post_ffw, image of the NEXT norm (next layer's attn norm, or the output norm)
      const uint8_t* Ws[1] = {(const uint8_t*)L.wdown.dptr};
      float* ys[1] = {nullptr};
      epi.w_post = (const float*)L.post_ffw_norm.dptr;
      epi.w_norm = (const float*)((l + 1 < g.n_layers) ? m->layers[l + 1].attn_norm.dptr : m->output_norm.dptr);
      if ((rc = ks_launch_gemm_segs(c, KS_Q4K, 1, Ws, &H, F, m->gemm_xt, n, ys, &H, m->gemm_p0, KS_GEMM_NORM_SPLIT, &epi))) return rc;
    }
  }
  if ((rc = lane_end(m, L_, n))) return rc;
  if (!want_logits) return KS_OK;
  {
    const uint8_t* Ws[1] = {(const uint8_t*)m->token_embd.dptr};
    float* ys[1] = {(float*)logits};
    const size_t V = (size_t)g.vocab;
    if ((rc = ks_launch_gemm_segs(c, (ks_dtype)g.embd_dtype, 1, Ws, &V, H, m->gemm_xt, n, ys, &V, m->gemm_p0, KS_GEMM_PLAIN, nullptr))) return rc;
  }
  for (int s = 0; s < n; s++)
    if ((rc = ks_launch_softcap_argmax(c, g.vocab, g.softcap, act, logits + (size_t)s * g.vocab * 4, tok_out + s))) return rc;
  KS_LAUNCH(c, (collect_kernel), 1, row_threads(n), 0, n, (const float*)tok_out, (const unsigned*)c->ws + KS_WS_ERR_WORD, L_.ret, (float*)m->host_ret, (int)g.n_slots);
  return ks_after_launch(c, "collect");
}

// The same token with the norms folded into the matvecs that consume them: five launches per layer
// (qkv, per-head norm/rope/KV, attention, o-proj, gate/up, down -> six with the attention pair).
// The residual stream alternates between two buffers because the block that writes the updated
// stream must not overwrite what the other blocks of the same launch still read.
int enqueue_forward_fused(ks_model* m, const Lane& L_, int n, bool want_logits) {
  ks_ctx* c = m->ctx;
  const ks_model_config& g = m->cfg;
  const ks_dtype act = (ks_dtype)g.act;
  const size_t ab = act_b(m);
  const size_t H = g.hidden, F = g.ffn, hd = g.hd, nq = g.n_q, nkv = g.n_kv;
  const size_t qn = nq * hd, kvn = nkv * hd;
  char *cur = L_.x, *oth = L_.xb, *yb = L_.x2, *xn = L_.xn, *q = L_.q, *k = L_.k, *v = L_.v, *o = L_.o, *ff = L_.ff,
       *logits = L_.logits;
  const float* tok_in = L_.tok_in;
  float* tok_out = L_.tok_out;
  int* pos = L_.pos;
  int rc;

  if ((rc = lane_begin(m, L_, n))) return rc;
  if ((rc = ks_launch_copy_scale_indexed(c, H, n, sqrtf((float)H), (ks_dtype)g.embd_dtype, m->token_embd.dptr, tok_in, act, cur))) return rc;
  for (int l = 0; l < g.n_layers; l++) {
    const Layer& L = m->layers[l];
    ks_mv_pro pro{};
    pro.eps = g.eps;
    pro.w = L.attn_norm.dptr;
    if (l == 0) {
      pro.mode = KS_PRO_NORM;
    } else {
      pro.mode = KS_PRO_ADD_NORM;  // x += rms(down)*w_post_ffw of the previous layer, then this layer's attn norm
      pro.y = yb;
      pro.w_post = m->layers[l - 1].post_ffw_norm.dptr;
      pro.out_x = oth;
    }
    ks_mv_seg qkv[3] = {{(const uint8_t*)L.wq.dptr, q, (unsigned)qn},
                        {(const uint8_t*)L.wk.dptr, k, (unsigned)kvn},
                        {(const uint8_t*)L.wv.dptr, v, (unsigned)kvn}};
    if ((rc = ks_launch_matvec(c, KS_Q4K, qkv, 3, KS_EPI_PLAIN, H, act, cur, n, nullptr, &pro))) return rc;
    if (l > 0) std::swap(cur, oth);
    uint8_t* kk = m->kv_k[l] + L_.kv_off;
    uint8_t* kv = m->kv_v[l] + L_.kv_off;
    if ((rc = ks_launch_per_head_qkv_q40(c, nq, nkv, hd, n, g.eps, act, q, L.q_norm.dptr, m->rope, k, L.k_norm.dptr, v, q,
                                         kk, kv, pos, L_.kv_stride)))
      return rc;
    if ((rc = ks_launch_sdpa(c, n, nq, nkv, hd, g.attn_scale, act, q, kk, kv, L_.kv_stride, layer_meta(m, L_, l), L_.attn_tmp, o, att_splits_for(m, n))))
      return rc;
    ks_mv_seg so{(const uint8_t*)L.wo.dptr, yb, (unsigned)H};
    if ((rc = ks_launch_matvec(c, KS_Q4K, &so, 1, KS_EPI_PLAIN, qn, act, o, n, nullptr))) return rc;
    ks_mv_pro p2{};
    p2.mode = KS_PRO_ADD_NORM;  // x += rms(attn)*w_post_attn, then the FFN norm (K:539)
    p2.eps = g.eps;
    p2.w = L.ffn_norm.dptr;
    p2.y = yb;
    p2.w_post = L.post_attn_norm.dptr;
    p2.out_x = oth;
    ks_mv_seg gu[2] = {{(const uint8_t*)L.wgate.dptr, ff, (unsigned)F}, {(const uint8_t*)L.wup.dptr, ff, (unsigned)F}};
    if ((rc = ks_launch_matvec(c, KS_Q4K, gu, 2, KS_EPI_GATE_UP, H, act, cur, n, nullptr, &p2))) return rc;
    std::swap(cur, oth);
    ks_mv_seg sd{(const uint8_t*)L.wdown.dptr, yb, (unsigned)H};
    if ((rc = ks_launch_matvec(c, KS_Q4K, &sd, 1, KS_EPI_PLAIN, F, act, ff, n, nullptr))) return rc;
  }
  if ((rc = lane_end(m, L_, n))) return rc;
  if (!want_logits) return KS_OK;
  // last residual update and the output norm, then the head (gemma_prim.rs:1222-1242)
  if ((rc = ks_launch_rmsnorm_add_then_rmsnorm(c, H, n, g.eps, act, yb, m->layers[g.n_layers - 1].post_ffw_norm.dptr, cur,
                                               m->output_norm.dptr, cur, xn)))
    return rc;
  ks_mv_seg sh{(const uint8_t*)m->token_embd.dptr, logits, (unsigned)g.vocab};
  if ((rc = ks_launch_matvec(c, (ks_dtype)g.embd_dtype, &sh, 1, KS_EPI_PLAIN, H, act, xn, n, nullptr))) return rc;
  for (int s = 0; s < n; s++)
    if ((rc = ks_launch_softcap_argmax(c, g.vocab, g.softcap, act, logits + (size_t)s * g.vocab * ab, tok_out + s))) return rc;
  KS_LAUNCH(c, (collect_kernel), 1, row_threads(n), 0, n, (const float*)tok_out, (const unsigned*)c->ws + KS_WS_ERR_WORD, L_.ret, (float*)m->host_ret, (int)g.n_slots);
  return ks_after_launch(c, "collect");
}

int mega_reset(ks_ctx* c, const ks_model::Mega& mg) { return mg.bar ? ks_mega_reset(c, mg.bar) : ks_flow_reset(c, mg.flow); }

// Rows that share one pass over the weights when `left` rows are waiting: what the batch matvec stages side by
// side, or, for more rows than that, a tensor-core GEMM chunk.
int pass_rows(const ks_model* m, int left) { return left > m->chunk && m->gemm_chunk ? m->gemm_chunk : m->chunk; }

// One slot's token with every layer inside one persistent kernel; embedding before, head after.
int enqueue_forward_mega(ks_model* m, const ks_model::Mega& mg, int first, int src, bool want_logits) {
  ks_ctx* c = m->ctx;
  const ks_model_config& g = m->cfg;
  const size_t H = g.hidden;
  float* cur = (float*)m->x + (size_t)first * H;
  float* yb = (float*)m->x2 + (size_t)first * H;
  float* xn = (float*)m->xn + (size_t)first * H;
  float* logits = (float*)m->logits + (size_t)first * g.vocab;
  const float* tok_in = src == 2 ? m->host_ids + first : m->tok + (size_t)src * g.n_slots + first;
  float* tok_out = m->tok + (size_t)(src == 2 ? 1 : src ^ 1) * g.n_slots + first;
  int* pos = m->pos + first;
  int rc;
  if ((rc = ks_launch_copy_scale_indexed(c, H, 1, sqrtf((float)H), (ks_dtype)g.embd_dtype, m->token_embd.dptr, tok_in, KS_F32, cur))) return rc;
  if ((rc = mg.bar ? ks_mega_launch(c, mg.bar) : ks_flow_launch(c, mg.flow))) return rc;
  KS_LAUNCH(c, (end_token_kernel), 1, 32, 0, 1, pos);
  if ((rc = ks_after_launch(c, "end_token"))) return rc;
  if (!want_logits) return KS_OK;
  float* res = mg.bar ? ks_mega_residual(mg.bar) : ks_flow_residual(mg.flow);
  if ((rc = ks_launch_rmsnorm_add_then_rmsnorm(c, H, 1, g.eps, KS_F32, yb, m->layers[g.n_layers - 1].post_ffw_norm.dptr, res,
                                               m->output_norm.dptr, res, xn)))
    return rc;
  ks_mv_seg sh{(const uint8_t*)m->token_embd.dptr, logits, (unsigned)g.vocab};
  if ((rc = ks_launch_matvec(c, (ks_dtype)g.embd_dtype, &sh, 1, KS_EPI_PLAIN, H, KS_F32, xn, 1, nullptr))) return rc;
  if ((rc = ks_launch_softcap_argmax(c, g.vocab, g.softcap, KS_F32, logits, tok_out))) return rc;
  KS_LAUNCH(c, (collect_kernel), 1, 32, 0, 1, (const float*)tok_out, (const unsigned*)c->ws + KS_WS_ERR_WORD,
            m->ret + (size_t)first * (g.n_slots + 1), (float*)m->host_ret, (int)g.n_slots);
  return ks_after_launch(c, "collect");
}

// The persistent kernel of slot `first`, built on first use (outside any stream capture).
int get_mega(ks_model* m, int first, ks_model::Mega* out) {
  *out = ks_model::Mega();
  if (!m->use_mega) return KS_OK;
  auto it = m->mega.find(first);
  if (it != m->mega.end()) {
    *out = it->second;
    return KS_OK;
  }
  const ks_model_config& g = m->cfg;
  const size_t H = g.hidden, F = g.ffn, qn = (size_t)g.n_q * g.hd, kvn = (size_t)g.n_kv * g.hd;
  ks_mega_desc d{};
  d.n_layers = g.n_layers;
  d.hidden = (unsigned)H; d.ffn = (unsigned)F; d.n_q = (unsigned)g.n_q; d.n_kv = (unsigned)g.n_kv; d.hd = (unsigned)g.hd;
  d.eps = g.eps; d.attn_scale = g.attn_scale;
  d.rope = m->rope;
  d.pos = m->pos + first;
  d.x_a = (float*)m->x + (size_t)first * H;
  d.x_b = (float*)m->xb + (size_t)first * H;
  d.yb = (float*)m->x2 + (size_t)first * H;
  d.q = (float*)m->q + (size_t)first * qn;
  d.k = (float*)m->k + (size_t)first * kvn;
  d.v = (float*)m->v + (size_t)first * kvn;
  d.o = (float*)m->o + (size_t)first * qn;
  d.ff = (float*)m->ff + (size_t)first * F;
  d.att_tmp = m->attn_tmp + (size_t)first * g.n_q * m->n_splits * (g.hd + 2);
  d.n_splits = m->n_splits;
  std::vector<ks_mega_layer> ls(g.n_layers);
  for (int l = 0; l < g.n_layers; l++) {
    const Layer& L = m->layers[l];
    ks_mega_layer& o = ls[l];
    o.wq = L.wq.dptr; o.wk = L.wk.dptr; o.wv = L.wv.dptr; o.wo = L.wo.dptr;
    o.wgate = L.wgate.dptr; o.wup = L.wup.dptr; o.wdown = L.wdown.dptr;
    o.attn_norm = L.attn_norm.dptr; o.q_norm = L.q_norm.dptr; o.k_norm = L.k_norm.dptr;
    o.post_attn_norm = L.post_attn_norm.dptr; o.ffn_norm = L.ffn_norm.dptr; o.post_ffw_norm = L.post_ffw_norm.dptr;
    o.kv_k = m->kv_k[l] + (size_t)first * m->slot_stride;
    o.kv_v = m->kv_v[l] + (size_t)first * m->slot_stride;
  }
  ks_model::Mega mg;
  int rc = m->decode_kernel == 2 ? ks_flow_create(m->ctx, &d, ls.data(), &mg.flow) : ks_mega_create(m->ctx, &d, ls.data(), &mg.bar);
  if (rc) return rc;
  m->mega[first] = mg;
  *out = mg;
  return KS_OK;
}

// Launch the forward pass through a cached graph (captured on first use).
int run_forward(ks_model* m, int first, int n, int src, bool want_logits) {
  ks_ctx* c = m->ctx;
  const uint64_t key = ((uint64_t)first << 32) | ((uint64_t)n << 8) | ((uint64_t)src << 1) | (want_logits ? 1 : 0);
  auto it = m->graphs.find(key);
  if (it == m->graphs.end()) {
    ks_model::Mega mg;
    if (n == 1) {  // (with sliding-window layers get_mega leaves mg empty: the launch-per-op path runs)
      int rcm = get_mega(m, first, &mg);
      if (rcm) return rcm;
    }
    cudaGraph_t graph = nullptr;
    KS_CUDA(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    const uint64_t before = c->launches;
    const Lane lane = slot_lane(m, first, src);
    int rc = mg ? enqueue_forward_mega(m, mg, first, src, want_logits)
             : n > m->chunk ? enqueue_forward_gemm(m, lane, n, want_logits)
             : m->fused ? enqueue_forward_fused(m, lane, n, want_logits)
                        : enqueue_forward(m, lane, n, want_logits);
    cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
    c->launches = before;  // captured launches are counted when the graph replays
    if (rc) {
      if (graph) cudaGraphDestroy(graph);
      return rc;
    }
    if (e != cudaSuccess) return ks_fail(c, KS_ERR_CUDA, "model: graph capture failed: %s", cudaGetErrorString(e));
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    size_t nodes = 0;
    cudaGraphGetNodes(graph, nullptr, &nodes);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return ks_fail(c, KS_ERR_CUDA, "model: graph instantiate failed: %s", cudaGetErrorString(e));
    m->graphs[key] = exec;
    m->graph_nodes[key] = nodes;
    it = m->graphs.find(key);
  }
  KS_CUDA(c, cudaGraphLaunch(it->second, c->stream));
  c->launches += m->graph_nodes[key];
  return KS_OK;
}

// A chunk of n prompt tokens of one slot (ids already in m->ctok) through every layer, no head.
int run_prefill_chunk(ks_model* m, int slot, int n) {
  ks_ctx* c = m->ctx;
  const uint64_t key = (1ull << 63) | ((uint64_t)slot << 32) | ((uint64_t)n << 8);
  auto it = m->graphs.find(key);
  if (it == m->graphs.end()) {
    cudaGraph_t graph = nullptr;
    KS_CUDA(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    const uint64_t before = c->launches;
    const Lane lane = chunk_lane(m, slot);
    int rc = n > m->chunk ? enqueue_forward_gemm(m, lane, n, false)
             : m->fused   ? enqueue_forward_fused(m, lane, n, false)
                          : enqueue_forward(m, lane, n, false);
    cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
    c->launches = before;
    if (rc) {
      if (graph) cudaGraphDestroy(graph);
      return rc;
    }
    if (e != cudaSuccess) return ks_fail(c, KS_ERR_CUDA, "model: graph capture failed: %s", cudaGetErrorString(e));
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    size_t nodes = 0;
    cudaGraphGetNodes(graph, nullptr, &nodes);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return ks_fail(c, KS_ERR_CUDA, "model: graph instantiate failed: %s", cudaGetErrorString(e));
    m->graphs[key] = exec;
    m->graph_nodes[key] = nodes;
    it = m->graphs.find(key);
  }
  KS_CUDA(c, cudaGraphLaunch(it->second, c->stream));
  c->launches += m->graph_nodes[key];
  return KS_OK;
}

}  // namespace

// ---- C ABI ------------------------------------------------------------------------------------
extern "C" {

ks_model* ks_model_create(ks_ctx* ctx, const ks_model_config* cfg) {
  if (!ctx || !cfg) return nullptr;
  const ks_model_config& g = *cfg;
  auto bad = [&](const char* why) -> ks_model* {
    ks_fail(ctx, KS_ERR_INVALID, "model_create: %s", why);
    return nullptr;
  };
  if (g.n_layers < 1 || g.hidden < 256 || g.hidden % 256 || g.ffn < 256 || g.ffn % 256) return bad("hidden and ffn must be positive multiples of 256");
  if (g.n_q < 1 || g.n_kv < 1 || g.n_q % g.n_kv) return bad("n_q must be a multiple of n_kv");
  if (g.hd != 128 && g.hd != 256) return bad("head_dim must be 128 or 256");
  if ((g.n_q * g.hd) % 256) return bad("n_q*head_dim must be a multiple of 256");
  if (g.vocab < 1 || g.max_seq < 1 || g.n_slots < 1 || g.n_slots > 64) return bad("vocab, max_seq >= 1 and 1 <= n_slots <= 64 required");
  if (g.embd_dtype != KS_Q4K && g.embd_dtype != KS_Q6K) return bad("token_embd must be Q4K or Q6K");
  if (g.act != KS_F32 && g.act != KS_F16) return bad("activation dtype must be F32 or F16");
  if (!(g.softcap > 0.0f)) return bad("softcap must be > 0");
  if (g.sliding_window < 0) return bad("sliding_window must be >= 0");
  if (g.n_layers > 64 && g.sliding_window > 0 && g.swa_layers) return bad("sliding-window layers are flagged in a 64-bit mask: at most 64 layers");
  cudaSetDevice(ctx->device);

  ks_model* m = new ks_model();
  m->ctx = ctx;
  m->cfg = g;
  m->layers.resize(g.n_layers);
  const size_t ab = ks_act_bytes((ks_dtype)g.act);
  const size_t H = g.hidden, F = g.ffn, qn = (size_t)g.n_q * g.hd, kvn = (size_t)g.n_kv * g.hd;
  // weight arena
  size_t off = 0;
  auto place = [&](Tensor& t, size_t bytes, const std::string& name) {
    off = (off + 255) & ~size_t(255);
    t.dptr = (void*)off;  // offset for now
    t.bytes = bytes;
    t.dtype = name == "token_embd.weight" ? g.embd_dtype : name.find("norm") != std::string::npos ? g.act : (int)KS_Q4K;
    off += bytes;
    m->by_name[name] = &t;
  };
  place(m->token_embd, ks_nbytes((ks_dtype)g.embd_dtype, (size_t)g.vocab * H), "token_embd.weight");
  place(m->output_norm, H * ab, "output_norm.weight");
  for (int l = 0; l < g.n_layers; l++) {
    Layer& L = m->layers[l];
    const std::string p = "blk." + std::to_string(l) + ".";
    place(L.wq, ks_nbytes(KS_Q4K, qn * H), p + "attn_q.weight");
    place(L.wk, ks_nbytes(KS_Q4K, kvn * H), p + "attn_k.weight");
    place(L.wv, ks_nbytes(KS_Q4K, kvn * H), p + "attn_v.weight");
    place(L.wo, ks_nbytes(KS_Q4K, H * qn), p + "attn_output.weight");
    place(L.wgate, ks_nbytes(KS_Q4K, F * H), p + "ffn_gate.weight");
    place(L.wup, ks_nbytes(KS_Q4K, F * H), p + "ffn_up.weight");
    place(L.wdown, ks_nbytes(KS_Q4K, H * F), p + "ffn_down.weight");
    place(L.attn_norm, H * ab, p + "attn_norm.weight");
    place(L.q_norm, (size_t)g.hd * ab, p + "attn_q_norm.weight");
    place(L.k_norm, (size_t)g.hd * ab, p + "attn_k_norm.weight");
    place(L.post_attn_norm, H * ab, p + "post_attention_norm.weight");
    place(L.ffn_norm, H * ab, p + "ffn_norm.weight");
    place(L.post_ffw_norm, H * ab, p + "post_ffw_norm.weight");
  }
  m->arena_bytes = off + 256;
  bool ok = dev_alloc(m, &m->arena, m->arena_bytes) == KS_OK;
  if (ok)
    for (auto& kv : m->by_name) kv.second->dptr = (char*)m->arena + (size_t)kv.second->dptr;

  const size_t rowb = (size_t)g.hd / 32 * KS_Q40_BLOCK_BYTES;
  m->slot_stride = (size_t)g.max_seq * g.n_kv * rowb;
  m->kv_k.resize(g.n_layers);
  m->kv_v.resize(g.n_layers);
  for (int l = 0; ok && l < g.n_layers; l++) {
    ok = dev_alloc(m, (void**)&m->kv_k[l], m->slot_stride * g.n_slots) == KS_OK &&
         dev_alloc(m, (void**)&m->kv_v[l], m->slot_stride * g.n_slots) == KS_OK;
  }
  m->occupied.assign(g.n_slots, 0);
  m->seq_len.assign(g.n_slots, 0);
  m->tok_src.assign(g.n_slots, 0);
  const size_t S = g.n_slots;
  m->fused = ks_matvec_can_fuse_pro(KS_Q4K, H) && !getenv("KSEARCH_UNFUSED");
  // Single-slot steps run all layers inside one persistent kernel.  KSEARCH_DECODE_KERNEL: 0 keeps one
  // launch per op (the path every multi-slot step takes anyway), 1 = the kernel whose phases meet at grid
  // barriers (default), 2 = the kernel whose blocks exchange tagged words instead of meeting.
  const char* dk = getenv("KSEARCH_DECODE_KERNEL");
  // (the persistent kernels attend to the whole context: a model with sliding-window layers takes one launch per op)
  m->use_mega = m->fused && g.act == KS_F32 && !(dk && dk[0] == '0') && !has_window(g);
  m->decode_kernel = dk && dk[0] == '2' ? 2 : 1;
  // Two slots step faster as two persistent-kernel passes than side by side through one launch per op (same
  // measurement: E2B 938 against 1074 us, E4B 1157 against 1378); from three slots on the GEMM path wins.
  m->solo_max = 2;
  if (const char* sm = getenv("KSEARCH_SOLO_SLOTS")) m->solo_max = atoi(sm) < 1 ? 1 : atoi(sm);
  ok = ok && dev_alloc(m, &m->xb, S * H * ab) == KS_OK && dev_alloc(m, &m->xn, S * H * ab) == KS_OK;
  ok = ok && dev_alloc(m, &m->x, S * H * ab) == KS_OK && dev_alloc(m, &m->x2, S * H * ab) == KS_OK &&
       dev_alloc(m, &m->q, S * qn * ab) == KS_OK && dev_alloc(m, &m->k, S * kvn * ab) == KS_OK &&
       dev_alloc(m, &m->v, S * kvn * ab) == KS_OK && dev_alloc(m, &m->o, S * qn * ab) == KS_OK &&
       dev_alloc(m, &m->ff, S * F * ab) == KS_OK && dev_alloc(m, &m->logits, S * (size_t)g.vocab * ab) == KS_OK &&
       dev_alloc(m, (void**)&m->tok, 2 * S * sizeof(float)) == KS_OK && dev_alloc(m, (void**)&m->pos, S * sizeof(int)) == KS_OK &&
       dev_alloc(m, (void**)&m->meta, S * 4 * sizeof(float)) == KS_OK &&
       (!has_window(g) || dev_alloc(m, (void**)&m->meta_swa, S * 4 * sizeof(float)) == KS_OK) &&
       dev_alloc(m, (void**)&m->ret, S * (S + 1) * sizeof(float)) == KS_OK &&
       dev_alloc(m, (void**)&m->rope, (size_t)g.max_seq * g.hd * sizeof(float)) == KS_OK;
  {
    // every token of a chunk keeps its staged input vector in shared memory (280 bytes per 64 columns);
    // leave 64 KB for the weight stages
    size_t maxcols = H > F ? H : F;
    if (qn > maxcols) maxcols = qn;
    m->chunk = KS_PREFILL_CHUNK;
    while (m->chunk > 1 && (size_t)m->chunk * (maxcols / 64) * 280 + (64u << 10) > ctx->smem_optin) m->chunk--;
    // f32 activations and block-aligned columns: larger batches go through the tensor-core GEMM
    if (g.act == KS_F32 && H % 256 == 0 && F % 256 == 0 && qn % 256 == 0 && !getenv("KSEARCH_NO_GEMM")) {
      const int G = KS_GEMM_CHUNK;
      m->gemm_chunk = G;
      // one launch each: q|k|v, o, gate|up, down, head
      const size_t rows_of[5] = {qn + 2 * kvn, H, 2 * F, H, (size_t)g.vocab}, cols_of[5] = {H, qn, H, F, H};
      size_t xt = 0, part = 0;
      for (int i = 0; i < 5; i++) {
        const size_t a = ks_gemm_xt_bytes(cols_of[i], G), b = 4 * ks_gemm_part_floats(ctx, rows_of[i], cols_of[i], G);
        xt = a > xt ? a : xt;
        part = b > part ? b : part;
      }
      xt = (xt + 255) & ~(size_t)255;
      void* ws = nullptr;
      if (ks_ctx_gemm_scratch(ctx, xt + part, &ws) != KS_OK) {
        ok = false;
      } else {
        m->gemm_xt = ws;
        m->gemm_p0 = (float*)((char*)ws + xt);
        // Measured on both model shapes (12 layers + head, one round of n slots): the GEMM path costs about the same
        // for 3 rows as for 16 and beats the batch matvec from 3 rows on (E2B 3 / 4 / 6 rows: 1264 / 1232 / 1307 us
        // against 1485 / 1748 / 2348; E4B 3 rows: 1501 against 1787), so only pairs still share a batch-matvec pass.
        // KSEARCH_BATCH_ROWS moves the limit (measurement).
        int limit = 2;
        if (const char* br = getenv("KSEARCH_BATCH_ROWS")) limit = atoi(br) < 1 ? 1 : atoi(br);
        if (limit < m->chunk) m->chunk = limit;
      }
    }
    const size_t C = m->gemm_chunk > KS_PREFILL_CHUNK ? m->gemm_chunk : KS_PREFILL_CHUNK;
    ok = ok && dev_alloc(m, &m->cx, C * H * ab) == KS_OK && dev_alloc(m, &m->cxb, C * H * ab) == KS_OK &&
         dev_alloc(m, &m->cx2, C * H * ab) == KS_OK && dev_alloc(m, &m->cq, C * qn * ab) == KS_OK &&
         dev_alloc(m, &m->ck, C * kvn * ab) == KS_OK && dev_alloc(m, &m->cv, C * kvn * ab) == KS_OK &&
         dev_alloc(m, &m->co, C * qn * ab) == KS_OK && dev_alloc(m, &m->cff, C * F * ab) == KS_OK &&
         dev_alloc(m, (void**)&m->ctok, C * sizeof(float)) == KS_OK && dev_alloc(m, (void**)&m->cpos, C * sizeof(int)) == KS_OK &&
         dev_alloc(m, (void**)&m->cmeta, C * 4 * sizeof(float)) == KS_OK &&
         (!has_window(g) || dev_alloc(m, (void**)&m->cmeta_swa, C * 4 * sizeof(float)) == KS_OK);
  }
  if (ok) {
    m->n_splits = ks_sdpa_pick_splits(ctx, 1, g.n_kv, g.max_seq);
    const size_t C = m->gemm_chunk > KS_PREFILL_CHUNK ? m->gemm_chunk : KS_PREFILL_CHUNK;
    ok = dev_alloc(m, (void**)&m->cattn_tmp, (C * g.n_q * (size_t)m->n_splits * (g.hd + 2) + 4) * sizeof(float)) == KS_OK;
  }
  if (ok) {
    ok = dev_alloc(m, (void**)&m->attn_tmp, (S * g.n_q * (size_t)m->n_splits * (g.hd + 2) + 4) * sizeof(float)) == KS_OK;
  }
  if (ok) {
    // RoPE table: per position hd f32 = cos[hd/2] || sin[hd/2], freq_i = theta^(-2i/hd) (gemma_prim.rs:33-56)
    std::vector<float> t((size_t)g.max_seq * g.hd);
    const int half = g.hd / 2;
    for (int p = 0; p < g.max_seq; p++)
      for (int i = 0; i < half; i++) {
        const float freq = (float)(1.0 / pow((double)g.rope_theta, (double)(2 * i) / (double)g.hd));
        const float ang = (float)p * freq;
        t[(size_t)p * g.hd + i] = cosf(ang);
        t[(size_t)p * g.hd + half + i] = sinf(ang);
      }
    ok = cudaMemcpyAsync(m->rope, t.data(), t.size() * sizeof(float), cudaMemcpyHostToDevice, ctx->stream) == cudaSuccess &&
         cudaStreamSynchronize(ctx->stream) == cudaSuccess;
    if (!ok) ks_fail(ctx, KS_ERR_CUDA, "model_create: rope upload failed");
  }
  if (ok && cudaMallocHost((void**)&m->host_ids, (size_t)g.n_slots * sizeof(float)) != cudaSuccess) {
    ks_fail(ctx, KS_ERR_OOM, "model_create: pinned allocation failed");
    m->host_ids = nullptr;
    ok = false;
  }
  if (ok && cudaMallocHost((void**)&m->host_ret, ((size_t)g.n_slots + 4) * sizeof(float)) != cudaSuccess) {
    ks_fail(ctx, KS_ERR_OOM, "model_create: pinned allocation failed");
    m->host_ret = nullptr;
    ok = false;
  }
  if (m->host_ret) memset(m->host_ret, 0, ((size_t)g.n_slots + 4) * sizeof(float));
  m->host_tok_n = 8192;
  if (ok && cudaMallocHost((void**)&m->host_tok, m->host_tok_n * sizeof(float)) != cudaSuccess) {
    ks_fail(ctx, KS_ERR_OOM, "model_create: pinned allocation failed");
    ok = false;
  }
  if (!ok) {
    ks_model_destroy(m);
    return nullptr;
  }
  return m;
}

// Search (or load from the per-chip cache) the launch plan of every matvec shape of this model:
// the load-time BEAM warm of gemma_prim.rs:254-290.  Honours KSEARCH_SKIP_BEAM.
int ks_model_warm_plans(ks_model* m, int n_tok) {
  if (!m) return KS_ERR_INVALID;
  ks_ctx* c = m->ctx;
  const ks_model_config& g = m->cfg;
  const size_t H = g.hidden, F = g.ffn, qn = (size_t)g.n_q * g.hd, kvn = (size_t)g.n_kv * g.hd;
  if (n_tok < 1) n_tok = 1;
  int found = 0;
  found += ks_plan_search(c, "qkv_q4k", qn, kvn, H, n_tok, nullptr) == KS_OK;
  found += ks_plan_search(c, "mv_q4k", H, 0, qn, n_tok, nullptr) == KS_OK;
  found += ks_plan_search(c, "gu_q4k", F, 0, H, n_tok, nullptr) == KS_OK;
  found += ks_plan_search(c, "mv_q4k", H, 0, F, n_tok, nullptr) == KS_OK;
  found += ks_plan_search(c, g.embd_dtype == KS_Q6K ? "mv_q6k" : "mv_q4k", (size_t)g.vocab, 0, H, n_tok, nullptr) == KS_OK;
  // plans change the captured launches: drop graphs recorded before
  cudaStreamSynchronize(c->stream);
  for (auto& kv : m->graphs) cudaGraphExecDestroy(kv.second);
  m->graphs.clear();
  m->graph_nodes.clear();
  return found;
}

void ks_model_destroy(ks_model* m) {
  if (!m) return;
  cudaSetDevice(m->ctx->device);
  cudaStreamSynchronize(m->ctx->stream);
  for (auto& kv : m->graphs) cudaGraphExecDestroy(kv.second);
  for (auto& kv : m->mega) {
    if (kv.second.bar) ks_mega_destroy(kv.second.bar);
    if (kv.second.flow) ks_flow_destroy(kv.second.flow);
  }
  for (void* p : m->owned) cudaFree(p);
  if (m->host_tok) cudaFreeHost(m->host_tok);
  if (m->host_ret) cudaFreeHost(m->host_ret);
  if (m->host_ids) cudaFreeHost(m->host_ids);
  delete m;
}

size_t ks_model_tensor_bytes(const ks_model* m, const char* name) {
  if (!m || !name) return 0;
  auto it = m->by_name.find(name);
  return it == m->by_name.end() ? 0 : it->second->bytes;
}

int ks_model_upload_tensor(ks_model* m, const char* name, const void* host, size_t bytes) {
  if (!m) return KS_ERR_INVALID;
  ks_ctx* c = m->ctx;
  KS_REQUIRE(c, name && host, "model_upload_tensor: null argument");
  auto it = m->by_name.find(name);
  KS_REQUIRE(c, it != m->by_name.end(), "missing tensor %s", name);
  KS_REQUIRE(c, bytes == it->second->bytes, "tensor %s: got %zu bytes, expected %zu", name, bytes, it->second->bytes);
  KS_CUDA(c, cudaMemcpyAsync(it->second->dptr, host, bytes, cudaMemcpyHostToDevice, c->stream));
  KS_CUDA(c, cudaStreamSynchronize(c->stream));
  it->second->set = true;
  return KS_OK;
}

// ensure_weight (gemma_prim.rs:415-451) with the file's tensor type: a tensor stored as it is resident is copied; a
// Q6_K, F16 or F32 tensor whose resident form is Q4_K (the reference requantises Q6_K ffn_down / attn_v and every
// f32 / bf16 matrix on the host) is staged on the device and requantised there by the same arithmetic.
int ks_model_upload_tensor_as(ks_model* m, const char* name, ks_dtype src_dtype, const void* host, size_t bytes) {
  if (!m) return KS_ERR_INVALID;
  ks_ctx* c = m->ctx;
  KS_REQUIRE(c, name && host, "model_upload_tensor: null argument");
  auto it = m->by_name.find(name);
  KS_REQUIRE(c, it != m->by_name.end(), "missing tensor %s", name);
  Tensor& t = *it->second;
  if ((int)src_dtype == t.dtype) return ks_model_upload_tensor(m, name, host, bytes);
  KS_REQUIRE(c, t.dtype == KS_Q4K && (src_dtype == KS_Q6K || src_dtype == KS_Q5K || src_dtype == KS_F16 || src_dtype == KS_F32),
             "tensor %s: no conversion from ggml type %d to the resident type %d", name, (int)src_dtype, t.dtype);
  const size_t nelem = t.bytes / KS_Q4K_BLOCK_BYTES * 256;
  KS_REQUIRE(c, bytes == ks_nbytes(src_dtype, nelem), "tensor %s: got %zu bytes, expected %zu", name, bytes, ks_nbytes(src_dtype, nelem));
  void* stage = nullptr;
  if (cudaMalloc(&stage, bytes) != cudaSuccess) return ks_fail(c, KS_ERR_OOM, "tensor %s: cannot stage %zu bytes", name, bytes);
  cudaError_t e = cudaMemcpyAsync(stage, host, bytes, cudaMemcpyHostToDevice, c->stream);
  int rc = e == cudaSuccess ? ks_launch_quantize_q4k(c, src_dtype, stage, nelem, t.dptr) : KS_ERR_CUDA;
  if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
  cudaFree(stage);
  if (e != cudaSuccess) return ks_fail(c, KS_ERR_CUDA, "tensor %s: upload failed: %s", name, cudaGetErrorString(e));
  if (rc) return rc;
  t.set = true;
  return KS_OK;
}

// f32 -> f16 as the reference's converter rounds (crates/ksearch_gguf/src/lib.rs:39-75: half UP in magnitude).
static uint16_t f32_to_f16_half_up(float v) {
  uint32_t bits;
  memcpy(&bits, &v, 4);
  const uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
  int e = (int)((bits >> 23) & 0xFFu);
  uint32_t mant = bits & 0x7FFFFFu;
  if (e == 255) return mant == 0 ? (uint16_t)(sign | 0x7C00u) : (uint16_t)(sign | 0x7C00u | (mant >> 13));
  e -= 127;
  if (e > 15) return (uint16_t)(sign | 0x7C00u);
  if (e < -14) {
    if (e < -24) return sign;
    mant |= 0x800000u;
    const uint32_t shift = (uint32_t)(-14 - e) + 13u;
    return (uint16_t)(sign | ((mant + (1u << (shift - 1u))) >> shift));
  }
  const uint32_t he = (uint32_t)(e + 15), hm = mant + 0x1000u;
  if (hm & 0x800000u) return (uint16_t)(sign | ((he + 1u) << 10));
  return (uint16_t)(sign | (he << 10) | (hm >> 13));
}

int ks_model_load_gguf(ks_model* m, const ks_gguf* g) {
  if (!m) return KS_ERR_INVALID;
  ks_ctx* c = m->ctx;
  KS_REQUIRE(c, g, "model_load_gguf: null file");
  for (auto& kv : m->by_name) {
    const char* name = kv.first.c_str();
    const Tensor& t = *kv.second;
    uint32_t type = 0, n_dims = 0;
    uint64_t dims[4], off = 0, nbytes = 0;
    if (ks_gguf_tensor(g, name, &type, &n_dims, dims, &off, &nbytes)) return ks_fail(c, KS_ERR_INVALID, "tensor not found: %s", name);
    ks_dtype src;
    switch (type) {  // gguf_impl.rs:20-31
      case 0: src = KS_F32; break;
      case 1: src = KS_F16; break;
      case 12: src = KS_Q4K; break;
      case 13: src = KS_Q5K; break;
      case 14: src = KS_Q6K; break;
      default: return ks_fail(c, KS_ERR_UNSUPPORTED, "tensor %s: ggml type %u is not supported", name, type);
    }
    const size_t nelem = t.dtype == KS_F32 ? t.bytes / 4 : t.dtype == KS_F16 ? t.bytes / 2 : t.bytes / ks_block_bytes((ks_dtype)t.dtype) * 256;
    uint64_t have = 1;
    for (uint32_t d = 0; d < n_dims && d < 4; d++) have *= dims[d];
    KS_REQUIRE(c, n_dims <= 4 && have == nelem, "tensor %s: the file holds %llu elements, the model expects %zu", name,
               (unsigned long long)have, nelem);
    const void* raw = ks_gguf_tensor_raw(g, name);
    KS_REQUIRE(c, raw, "tensor %s: no data", name);
    int rc;
    if (src == KS_F32 && t.dtype == KS_F16) {  // norm weights of an f16 model
      std::vector<uint16_t> h(nelem);
      const float* f = static_cast<const float*>(raw);
      for (size_t i = 0; i < nelem; i++) h[i] = f32_to_f16_half_up(f[i]);
      rc = ks_model_upload_tensor(m, name, h.data(), nelem * 2);
    } else {
      rc = ks_model_upload_tensor_as(m, name, src, raw, (size_t)nbytes);
    }
    if (rc) return rc;
  }
  return KS_OK;
}

const void* ks_model_tensor_ptr(const ks_model* m, const char* name) {
  if (!m || !name) return nullptr;
  auto it = m->by_name.find(name);
  return it == m->by_name.end() ? nullptr : it->second->dptr;
}

size_t ks_model_weight_bytes(const ks_model* m) {
  if (!m) return 0;
  size_t n = 0;
  for (auto& kv : m->by_name) n += kv.second->bytes;
  return n;
}

// ---- slot pool (kv_pool.rs:136-230) ---------------------------------------------------------
int ks_model_slot_alloc(ks_model* m) {
  if (!m) return KS_ERR_INVALID;
  for (int s = 0; s < m->cfg.n_slots; s++)
    if (!m->occupied[s]) {
      m->occupied[s] = 1;
      m->seq_len[s] = 0;
      KS_LAUNCH(m->ctx, (set_state_kernel), 1, 1, 0, s, 0, m->pos);
      return s;
    }
  return ks_fail(m->ctx, KS_ERR_STATE, "KvPool full (max_batch=%d)", m->cfg.n_slots);
}

int ks_model_slot_free(ks_model* m, int slot) {
  if (!m) return KS_ERR_INVALID;
  if (slot < 0 || slot >= m->cfg.n_slots) return ks_fail(m->ctx, KS_ERR_STATE, "bad SlotId");
  m->occupied[slot] = 0;
  m->seq_len[slot] = 0;
  return KS_OK;
}

int ks_model_slot_seq_len(const ks_model* m, int slot) {
  if (!m || slot < 0 || slot >= m->cfg.n_slots) return KS_ERR_STATE;
  return m->seq_len[slot];
}

int ks_model_slot_active(const ks_model* m) {
  int n = 0;
  if (m)
    for (char o : m->occupied) n += o ? 1 : 0;
  return n;
}

// Zero a slot's K/V rows and rewind it (gemma_prim.rs:1644-1656 reset, kv_pool.rs:147-160 clear_slot).
int ks_model_slot_reset(ks_model* m, int slot) {
  if (!m) return KS_ERR_INVALID;
  ks_ctx* c = m->ctx;
  if (slot < 0 || slot >= m->cfg.n_slots) return ks_fail(c, KS_ERR_STATE, "bad SlotId");
  for (int l = 0; l < m->cfg.n_layers; l++) {
    KS_CUDA(c, cudaMemsetAsync(m->kv_k[l] + (size_t)slot * m->slot_stride, 0, m->slot_stride, c->stream));
    KS_CUDA(c, cudaMemsetAsync(m->kv_v[l] + (size_t)slot * m->slot_stride, 0, m->slot_stride, c->stream));
  }
  KS_LAUNCH(c, (set_state_kernel), 1, 1, 0, slot, 0, m->pos);
  m->seq_len[slot] = 0;
  m->occupied[slot] = 1;
  auto it = m->mega.find(slot);
  if (it != m->mega.end() && it->second) {
    const int rc = mega_reset(c, it->second);
    if (rc) return rc;
  }
  return ks_after_launch(c, "slot_reset");
}

static int check_ready(ks_model* m) {
  for (auto& kv : m->by_name)
    if (!kv.second->set) return ks_fail(m->ctx, KS_ERR_STATE, "missing tensor %s", kv.first.c_str());
  return KS_OK;
}

static int check_slots(ks_model* m, int first, int n) {
  ks_ctx* c = m->ctx;
  if (first < 0 || n < 1 || first + n > m->cfg.n_slots) return ks_fail(c, KS_ERR_STATE, "bad SlotId");
  for (int s = first; s < first + n; s++) {
    if (!m->occupied[s]) return ks_fail(c, KS_ERR_STATE, "slot not occupied");
    if (m->seq_len[s] >= m->cfg.max_seq) return ks_fail(c, KS_ERR_STATE, "max_seq exceeded");
  }
  return KS_OK;
}

// Rows per pass of a decode step over slots [first, first + n).  A few slots are faster as one persistent-kernel
// pass each (all layers of a slot's token in one launch) than side by side through one launch per op.
int step_rows(ks_model* m, int first, int n) {
  if (n > 1 && n <= m->solo_max) {
    bool all = true;
    for (int s = first; s < first + n && all; s++) {
      ks_model::Mega mg;
      all = get_mega(m, s, &mg) == 0 && mg;
    }
    if (all) return 1;
  }
  return pass_rows(m, n);
}

// Enqueue one token for slots first..first+n-1.  tokens != NULL: ids are written from the host
// first (decode_token_sampled, gemma_prim.rs:1622-1634); NULL: ids already on the device from the
// previous step's argmax.  Nothing is read back and nothing waits.
int ks_model_forward(ks_model* m, int first, int n, const int* tokens, int want_logits) {
  if (!m) return KS_ERR_INVALID;
  ks_ctx* c = m->ctx;
  int rc;
  if ((rc = check_ready(m)) || (rc = check_slots(m, first, n))) return rc;
  // Ids chained on the device sit in the half of the ping-pong each slot's last head wrote; slots that
  // step together must agree on it (they do when they always step together, or when ids come from the host).
  int src = m->tok_src[first];
  if (!tokens)
    for (int s = first + 1; s < first + n; s++)
      if (m->tok_src[s] != src)
        return ks_fail(c, KS_ERR_STATE, "slots %d..%d hold their device-side token ids in different buffers; pass host ids", first, first + n - 1);
  if (tokens) {
    src = 2;  // the step's embedding kernel reads the ids from pinned host memory
    for (int s = 0; s < n; s++)
      KS_REQUIRE(c, tokens[s] >= 0 && tokens[s] < m->cfg.vocab, "token id %d outside the vocabulary", tokens[s]);
    KS_CUDA(c, cudaStreamSynchronize(c->stream));     // an earlier step may not have read its ids yet
    for (int s = 0; s < n; s++) m->host_ids[first + s] = (float)tokens[s];
  }
  // The slots share one pass over the weights as long as their staged input vectors fit the matvec kernels'
  // shared memory side by side (m->chunk of them); a larger batch takes several passes.
  const int per_pass = step_rows(m, first, n);
  for (int s0 = 0; s0 < n; s0 += per_pass) {
    const int nn = n - s0 < per_pass ? n - s0 : per_pass;
    if ((rc = run_forward(m, first + s0, nn, src, want_logits != 0))) return rc;
  }
  for (int s = first; s < first + n; s++) {
    m->seq_len[s] += 1;
    m->tok_src[s] = (char)(want_logits ? (src == 2 ? 1 : src ^ 1) : (src == 2 ? 0 : src));
  }
  return KS_OK;
}

// After a blocking wait: did a bounded device-side wait give up during the steps just run?  `status`
// is the pinned word the context's status word was copied to behind them.  When it is set, the token
// ids that came back are meaningless: the status word is cleared, the persistent kernel's barrier
// words are put back to rest, the slots are rewound by `steps` positions and KS_ERR_TIMEOUT is returned,
// so the context stays usable.
static int check_device_status(ks_model* m, const unsigned* status, int first, int n, int steps) {
  if (!*status) return KS_OK;
  ks_ctx* c = m->ctx;
  const unsigned flag = *status;
  cudaMemsetAsync((unsigned*)c->ws + KS_WS_ERR_WORD, 0, sizeof(unsigned), c->stream);
  for (int s = first; s < first + n; s++) {
    m->seq_len[s] = m->seq_len[s] >= steps ? m->seq_len[s] - steps : 0;
    KS_LAUNCH(c, (set_state_kernel), 1, 1, 0, s, m->seq_len[s], m->pos);
    auto it = m->mega.find(s);
    if (it != m->mega.end() && it->second) mega_reset(c, it->second);
  }
  cudaStreamSynchronize(c->stream);
  return ks_fail(c, KS_ERR_TIMEOUT, "a device-side wait gave up during decode (status word 0x%x); the slots were rewound", flag);
}

// Prompt tokens of one slot, KS_PREFILL_CHUNK at a time: the rows of a chunk share one pass over the
// weights (the batch form of the matvec kernels, K:1414) and attend causally inside the chunk.  This is
// the reference's GEMV fallback for prompts (forward_prefill_chunk, gemma_prim.rs:1317-1607, runs its
// mul_mm GEMM instead); no logits are produced.  Enqueues only, apart from the wait for the pinned
// staging words between chunks.
int ks_model_prefill(ks_model* m, int slot, const int* tokens, int n_tokens) {
  if (!m) return KS_ERR_INVALID;
  ks_ctx* c = m->ctx;
  KS_REQUIRE(c, tokens || n_tokens == 0, "prefill: null tokens");
  KS_REQUIRE(c, n_tokens >= 0, "prefill: negative token count");
  int rc;
  if ((rc = check_ready(m)) || (rc = check_slots(m, slot, 1))) return rc;
  if (m->seq_len[slot] + n_tokens > m->cfg.max_seq) return ks_fail(c, KS_ERR_STATE, "max_seq exceeded");
  float* stage = m->host_tok + m->host_tok_n - 16 - KS_STAGE_IDS;
  for (int t0 = 0; t0 < n_tokens;) {
    const int per_pass = pass_rows(m, n_tokens - t0);
    const int n = n_tokens - t0 < per_pass ? n_tokens - t0 : per_pass;
    KS_CUDA(c, cudaStreamSynchronize(c->stream));  // the staging words may still be in flight
    for (int t = 0; t < n; t++) {
      KS_REQUIRE(c, tokens[t0 + t] >= 0 && tokens[t0 + t] < m->cfg.vocab, "token id %d outside the vocabulary", tokens[t0 + t]);
      stage[t] = (float)tokens[t0 + t];
    }
    KS_CUDA(c, cudaMemcpyAsync(m->ctok, stage, n * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    if ((rc = run_prefill_chunk(m, slot, n))) return rc;
    m->seq_len[slot] += n;
    t0 += n;
  }
  return KS_OK;
}

// Blocking greedy step with host ids in and out: the serve path's decode_token
// (gemma_prim.rs:1616-1635).  4*n bytes go up, 4*n bytes come back, every call.
int ks_model_decode_token(ks_model* m, int first, int n, const int* tokens, int* next) {
  if (!m) return KS_ERR_INVALID;
  ks_ctx* c = m->ctx;
  KS_REQUIRE(c, tokens && next, "decode_token: null argument");
  // the request word the step's last kernel echoes into pinned memory once ids and flag are there
  volatile unsigned* hw = reinterpret_cast<volatile unsigned*>(m->host_ret);
  const int ns = m->cfg.n_slots;
  const unsigned req = ++m->req_id ? m->req_id : ++m->req_id;
  hw[ns + 2] = req;
  int rc = ks_model_forward(m, first, n, tokens, 1);
  if (rc) return rc;
  float* back = m->host_tok;  // n ids, then the status flag
  if (n <= step_rows(m, first, n)) {  // one pass: its last kernel left ids and flag in pinned memory; wait for its echo
    const auto t0 = std::chrono::steady_clock::now();
    bool seen = false;
    for (unsigned spin = 0;; spin++) {
      if (hw[ns + 1] == req) {
        seen = true;
        break;
      }
      if ((spin & 0xFFFu) == 0xFFFu) {  // a look at the clock and at the stream now and then: an error must not spin forever
        if (cudaStreamQuery(c->stream) != cudaErrorNotReady) break;
        if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(10)) break;
      }
    }
    if (seen) {
      std::atomic_thread_fence(std::memory_order_acquire);
      for (int s = 0; s < n; s++) back[s] = m->host_ret[s];
      back[n] = m->host_ret[ns];
      if (back[n] == 0.0f) {
        for (int s = 0; s < n; s++) next[s] = (int)back[s];
        return KS_OK;
      }
    }
    // not seen (the stream ended or failed first) or a wait gave up on the device: the plain route below
    KS_CUDA(c, cudaMemcpyAsync(back, m->ret + (size_t)first * (m->cfg.n_slots + 1), (n + 1) * sizeof(float), cudaMemcpyDeviceToHost,
                               c->stream));
  } else {                    // several passes: ids from the token buffer, the flag as any non-zero status word
    KS_CUDA(c, cudaMemcpyAsync(back, m->tok + (size_t)m->tok_src[first] * m->cfg.n_slots + first, n * sizeof(float),
                               cudaMemcpyDeviceToHost, c->stream));
    KS_CUDA(c, cudaMemcpyAsync(back + n, (unsigned*)c->ws + KS_WS_ERR_WORD, sizeof(unsigned), cudaMemcpyDeviceToHost, c->stream));
  }
  KS_CUDA(c, cudaStreamSynchronize(c->stream));
  if (back[n] != 0.0f) {
    unsigned flag = 0;
    cudaMemcpy(&flag, (unsigned*)c->ws + KS_WS_ERR_WORD, sizeof flag, cudaMemcpyDeviceToHost);
    if ((rc = check_device_status(m, &flag, first, n, 1))) return rc;
  }
  for (int s = 0; s < n; s++) next[s] = (int)back[s];
  return KS_OK;
}

// generate_timed (gemma_prim.rs:1658-1768) for one slot: rewind, run prompt[0..n-2] in chunks without
// logits, then n_new greedy steps starting from the last prompt token.  The token id never
// leaves the device between steps; each step's id is copied to pinned host memory behind the
// step and the host waits only once more than `max_inflight` steps are pending
// (wait_inflight_at_most, gemma_prim.rs:1688-1691).  Times are host wall clock like the
// reference's; decode_ms_device is the device time of the decode steps (CUDA events).
int ks_model_generate(ks_model* m, int slot, const int* prompt, int n_prompt, int n_new, int max_inflight, int* out,
                      ks_generate_stats* stats) {
  if (!m) return KS_ERR_INVALID;
  ks_ctx* c = m->ctx;
  KS_REQUIRE(c, prompt && n_prompt >= 1, "empty prompt");
  KS_REQUIRE(c, n_new >= 0 && (size_t)n_new <= m->host_tok_n - 32 - KS_STAGE_IDS, "generate: n_new out of range");
  KS_REQUIRE(c, out || n_new == 0, "generate: null output");
  int rc;
  if ((rc = ks_model_slot_reset(m, slot))) return rc;
  if (n_prompt - 1 + n_new > m->cfg.max_seq) return ks_fail(c, KS_ERR_STATE, "max_seq exceeded");
  cudaEvent_t e0, e1, e2;
  KS_CUDA(c, cudaEventCreate(&e0));
  KS_CUDA(c, cudaEventCreate(&e1));
  KS_CUDA(c, cudaEventCreate(&e2));
  cudaEventRecord(e0, c->stream);
  if ((rc = ks_model_prefill(m, slot, prompt, n_prompt - 1))) return rc;
  KS_CUDA(c, cudaStreamSynchronize(c->stream));
  int last = prompt[n_prompt - 1];
  cudaEventRecord(e1, c->stream);
  std::vector<cudaEvent_t> done;
  if (max_inflight < 0) max_inflight = 0;
  for (int i = 0; i < n_new; i++) {
    if ((rc = ks_model_forward(m, slot, 1, i == 0 ? &last : nullptr, 1))) return rc;
    KS_CUDA(c, cudaMemcpyAsync(m->host_tok + i, m->tok + (size_t)m->tok_src[slot] * m->cfg.n_slots + slot, sizeof(float),
                               cudaMemcpyDeviceToHost, c->stream));
    cudaEvent_t ev;
    KS_CUDA(c, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    cudaEventRecord(ev, c->stream);
    done.push_back(ev);
    const int wait_upto = i - max_inflight;  // steps <= this index must have finished
    if (wait_upto >= 0) KS_CUDA(c, cudaEventSynchronize(done[wait_upto]));
  }
  cudaEventRecord(e2, c->stream);
  unsigned* status = reinterpret_cast<unsigned*>(m->host_tok + m->host_tok_n - 9);
  KS_CUDA(c, cudaMemcpyAsync(status, (unsigned*)c->ws + KS_WS_ERR_WORD, sizeof(unsigned), cudaMemcpyDeviceToHost, c->stream));
  KS_CUDA(c, cudaStreamSynchronize(c->stream));
  for (cudaEvent_t ev : done) cudaEventDestroy(ev);
  if ((rc = check_device_status(m, status, slot, 1, n_new))) {
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaEventDestroy(e2);
    return rc;
  }
  for (int i = 0; i < n_new; i++) out[i] = (int)m->host_tok[i];
  if (stats) {
    float a = 0, b = 0;
    cudaEventElapsedTime(&a, e0, e1);
    cudaEventElapsedTime(&b, e1, e2);
    stats->prefill_tokens = n_prompt - 1;
    stats->decode_tokens = n_new;
    stats->prefill_ms_device = a;
    stats->decode_ms_device = b;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaEventDestroy(e2);
  return KS_OK;
}

// Device pointers of the slot's state, for tests and profiling: 0 = residual x, 1 = logits, 2 = phase clocks.
const void* ks_model_debug_ptr(const ks_model* m, int which, int slot) {
  if (!m || slot < 0 || slot >= m->cfg.n_slots) return nullptr;
  const size_t ab = ks_act_bytes((ks_dtype)m->cfg.act);
  if (which == 0) return (const char*)m->x + (size_t)slot * m->cfg.hidden * ab;
  if (which == 1) return (const char*)m->logits + (size_t)slot * m->cfg.vocab * ab;
  if (which == 2) {  // phase stamps of the persistent decode kernel, first and last block: [2][n_layers][5][8] int64
    auto it = m->mega.find(slot);  // (clock64 ticks from the barrier kernel, globaltimer ns from the dataflow one)
    if (it == m->mega.end() || !it->second) return nullptr;
    return it->second.bar ? (const void*)ks_mega_prof(it->second.bar) : (const void*)ks_flow_prof(it->second.flow);
  }
  if (which == 3) {  // every block's stamps [grid][n_layers][5][8] int64; the dataflow kernel only
    auto it = m->mega.find(slot);
    return it == m->mega.end() || !it->second.flow ? nullptr : (const void*)ks_flow_prof_all(it->second.flow);
  }
  return nullptr;
}

// Knobs of a slot's persistent decode kernel, for tests and for the phase-clock reader: what = 0 polls before
// a device-side wait gives up, 1 = make one stage of every layer wait for a tag nobody writes (exercises the
// give-up path; 0 switches it off), 2 = context length from which attention is split across blocks,
// 3 = record phase clocks (0 / 1).  Builds the kernel if the slot has none yet; drops the captured graphs.
int ks_model_debug_set(ks_model* m, int slot, int what, unsigned value) {
  if (!m) return KS_ERR_INVALID;
  ks_ctx* c = m->ctx;
  if (slot < 0 || slot >= m->cfg.n_slots) return ks_fail(c, KS_ERR_STATE, "bad SlotId");
  ks_model::Mega mg;
  int rc = get_mega(m, slot, &mg);
  if (rc) return rc;
  if (!mg) return ks_fail(c, KS_ERR_UNSUPPORTED, "this model shape does not use the persistent decode kernel");
  if ((rc = mg.bar ? ks_mega_set(mg.bar, what, value) : ks_flow_set(mg.flow, what, value)))
    return ks_fail(c, rc, "debug_set: unknown knob %d", what);
  cudaStreamSynchronize(c->stream);
  for (auto& kv : m->graphs) cudaGraphExecDestroy(kv.second);
  m->graphs.clear();
  m->graph_nodes.clear();
  return KS_OK;
}

// Device address of one slot's rows of a layer's cache ([max_seq, n_kv, hd] Q4_0); which: 0 = K, 1 = V.
void* ks_model_kv_ptr(const ks_model* m, int layer, int which, int slot) {
  if (!m || layer < 0 || layer >= m->cfg.n_layers || slot < 0 || slot >= m->cfg.n_slots || which < 0 || which > 1) return nullptr;
  return (which ? m->kv_v[layer] : m->kv_k[layer]) + (size_t)slot * m->slot_stride;
}
size_t ks_model_kv_slot_bytes(const ks_model* m) { return m ? m->slot_stride : 0; }

}  // extern "C"

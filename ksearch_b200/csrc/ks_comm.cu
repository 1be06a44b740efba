// Row-sharded matvec across the GPUs of one box: one process and one context per GPU, NCCL over
// NVLink for the one exchange that follows the local rows.
//
// The reference has no multi-device code (crates/ksearch_metal/src/lib.rs:33 takes the system default
// device), so nothing here replaces a reference entry point; the shapes it serves are the reference's
// largest matvecs: the tied lm_head (crates/ksearch_gemma/src/gemma_prim.rs:1222-1242) and the FFN
// projections (gemma_prim.rs:1130-1157).  A K-quant matrix is row-major over blocks, so rank k's rows
// are one contiguous byte range of the GGUF tensor: sharding needs no repacking.  x is replicated.
//   ks_matvec_sharded  local rows straight into this rank's slot of the gathered vector, then an in-place
//                      ncclAllGather on the context's stream (no host synchronisation, capturable);
//   ks_argmax_sharded  the lm_head form: soft-capped arg-max of the local logits, an all-gather of ONE
//                      (value, index) pair per rank, merge with ties to the lower index
//                      (crates/ksearch_codegen/src/render.rs:2355) -- 8 bytes per rank instead of 1 MiB.
// NCCL is loaded at run time (dlopen), preferring a copy the process already holds (the one torch
// brought), so the library itself keeps no link dependency on it.
#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>

#include "ks_internal.h"

namespace {

struct NcclApi {
  void* handle = nullptr;
  decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
  decltype(&ncclCommInitRank) CommInitRank = nullptr;
  decltype(&ncclAllGather) AllGather = nullptr;
  decltype(&ncclCommDestroy) CommDestroy = nullptr;
  decltype(&ncclGetErrorString) GetErrorString = nullptr;
  decltype(&ncclGetVersion) GetVersion = nullptr;
  bool ok = false;
};

NcclApi& nccl_api() {
  static NcclApi api;
  if (api.handle) return api;
  const char* names[4] = {getenv("KSEARCH_NCCL_LIB"), "libnccl.so.2", "libnccl.so", nullptr};
  for (int pass = 0; pass < 2 && !api.handle; pass++)  // pass 0: only a copy that is already loaded
    for (int i = 0; i < 3 && !api.handle; i++)
      if (names[i]) api.handle = dlopen(names[i], RTLD_NOW | RTLD_LOCAL | (pass == 0 ? RTLD_NOLOAD : 0));
  if (!api.handle) return api;
  api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(api.handle, "ncclGetUniqueId");
  api.CommInitRank = (decltype(api.CommInitRank))dlsym(api.handle, "ncclCommInitRank");
  api.AllGather = (decltype(api.AllGather))dlsym(api.handle, "ncclAllGather");
  api.CommDestroy = (decltype(api.CommDestroy))dlsym(api.handle, "ncclCommDestroy");
  api.GetErrorString = (decltype(api.GetErrorString))dlsym(api.handle, "ncclGetErrorString");
  api.GetVersion = (decltype(api.GetVersion))dlsym(api.handle, "ncclGetVersion");
  api.ok = api.GetUniqueId && api.CommInitRank && api.AllGather && api.CommDestroy && api.GetErrorString;
  return api;
}

// (soft-capped value, global index) of this rank's best logit: pair[0] = cap*tanh(x[i]/cap), pair[1] = row0 + i.
__global__ void argmax_pair_kernel(const float* logits, const float* local_idx, float cap, unsigned row0, float* pair) {
  ks_pdl_entry();
  if (threadIdx.x == 0) {
    const unsigned i = (unsigned)local_idx[0];
    pair[0] = cap * tanhf(logits[i] / cap);
    pair[1] = (float)(row0 + i);
  }
}
// Merge of one pair per rank: largest value, ties to the lower index.
__global__ void argmax_merge_kernel(const float* pairs, int n_ranks, float* out_idx) {
  ks_pdl_entry();
  if (threadIdx.x == 0) {
    float bv = pairs[0], bi = pairs[1];
    for (int r = 1; r < n_ranks; r++) {
      const float v = pairs[2 * r], i = pairs[2 * r + 1];
      if (v > bv || (v == bv && i < bi)) {
        bv = v;
        bi = i;
      }
    }
    out_idx[0] = bi;
  }
}

// ---- the same exchange over peer memory (NVLink), fused with the merge -----------------------------------------
// Every rank owns a mailbox of 2 x n_ranks 64-bit words that its peers can write (cudaIpc mapping).  One kernel per
// call: lane r stores this rank's (value, index, step) word into rank r's mailbox with one 8-byte system-scope store
// -- value and tag travel in one single-copy-atomic word, so no fence and no flag -- then lane r polls its own
// mailbox word r until the tag shows this step, and the warp merges the n_ranks candidates (largest value, ties to
// the lower index).  No NCCL launch: the exchange costs one store and one poll across NVLink instead of the
// ~20 us latency of a tiny all-gather.  The word: value bits << 32 | index << 8 | step & 0xFF; mailboxes alternate
// by step parity, so a rank that is one step ahead never overwrites a word a slower rank still waits for.  The
// poll is bounded: on expiry the context's status word is raised and the rank's own candidate is written.
constexpr int KS_P2P_MAX_RANKS = 32;
struct P2pArgs {
  unsigned long long* box[KS_P2P_MAX_RANKS];  // box[r]: rank r's mailbox as mapped into this process (own: local)
  unsigned* step;                             // this rank's step counter (device)
  unsigned n_ranks, rank, row0, poll_limit;
  float cap;
  const float* logits;
  const float* local_idx;
  float* out_idx;
  unsigned* err;
};
__global__ void argmax_p2p_kernel(const P2pArgs a) {
  ks_pdl_entry();
  const unsigned lane = threadIdx.x;
  unsigned step = 0;
  if (lane == 0) step = a.step[0] + 1u;
  step = __shfl_sync(0xffffffffu, step, 0);
  const unsigned i = (unsigned)a.local_idx[0];
  const float v = a.cap * tanhf(a.logits[i] / a.cap);
  const unsigned long long word =
      ((unsigned long long)__float_as_uint(v) << 32) | ((unsigned long long)(a.row0 + i) << 8) | (unsigned long long)(step & 0xFFu);
  const unsigned slot = (step & 1u) * a.n_ranks;
  unsigned long long* peer_box = nullptr;
#pragma unroll
  for (int r = 0; r < KS_P2P_MAX_RANKS; r++)
    if (lane == (unsigned)r) peer_box = a.box[r];  // selects: no dynamic indexing of the parameter array
  if (lane < a.n_ranks)
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(peer_box + slot + a.rank), "l"(word) : "memory");
  // own mailbox: word `lane` comes from rank `lane`
  unsigned long long got = word;
  bool ok = true;
  if (lane < a.n_ranks) {
    const unsigned long long* mine = a.box[0];
#pragma unroll
    for (int r = 1; r < KS_P2P_MAX_RANKS; r++)
      if (a.rank == (unsigned)r) mine = a.box[r];
    ok = false;
    for (unsigned n = 0; n < a.poll_limit; n++) {
      asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(got) : "l"(mine + slot + lane) : "memory");
      if ((unsigned)(got & 0xFFull) == (step & 0xFFu)) {
        ok = true;
        break;
      }
    }
    if (!ok) got = word;  // gave up: fall back to the local candidate, the status word tells the host
  }
  if (__any_sync(0xffffffffu, !ok) && lane == 0) atomicOr(a.err, 16u);
  float bv = lane < a.n_ranks ? __uint_as_float((unsigned)(got >> 32)) : -3.0e38f;
  unsigned bi = lane < a.n_ranks ? (unsigned)((got >> 8) & 0xFFFFFFu) : 0xFFFFFFFFu;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
    const unsigned oi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
  if (lane == 0) {
    a.out_idx[0] = (float)bi;
    a.step[0] = step;
  }
}

}  // namespace

struct ks_comm {
  ks_ctx* ctx = nullptr;
  ncclComm_t comm = nullptr;
  int n_ranks = 1, rank = 0;
  float* pair_local = nullptr;  // [2] this rank's (value, index), then [2 * n_ranks] gathered
  float* idx_local = nullptr;   // [1]
  // peer-memory exchange: this rank's mailbox (2 x n_ranks words) + step counter, and the peers' mailboxes as mapped here
  unsigned long long* box_local = nullptr;
  unsigned* step = nullptr;
  unsigned long long* box[KS_P2P_MAX_RANKS] = {nullptr};
  bool p2p = false, use_p2p = true;
  unsigned poll_limit = 1u << 23;  // several seconds of polling: the peers are other processes
};

extern "C" {

int ks_comm_unique_id(void* id_out) {
  if (!id_out) return KS_ERR_INVALID;
  NcclApi& api = nccl_api();
  if (!api.ok) {
    ks_set_global_error("ks_comm: libnccl.so.2 could not be loaded (set KSEARCH_NCCL_LIB to its path)");
    return KS_ERR_UNSUPPORTED;
  }
  static_assert(sizeof(ncclUniqueId) == KS_COMM_ID_BYTES, "NCCL unique id size");
  ncclUniqueId id;
  ncclResult_t r = api.GetUniqueId(&id);
  if (r != ncclSuccess) {
    ks_set_global_error(api.GetErrorString(r));
    return KS_ERR_CUDA;
  }
  memcpy(id_out, &id, sizeof id);
  return KS_OK;
}

ks_comm* ks_comm_init(ks_ctx* ctx, int n_ranks, int rank, const void* unique_id) {
  if (!ctx) return nullptr;
  if (n_ranks < 1 || rank < 0 || rank >= n_ranks || (!unique_id && n_ranks > 1)) {
    ks_fail(ctx, KS_ERR_INVALID, "comm_init: bad rank %d of %d or null id", rank, n_ranks);
    return nullptr;
  }
  ks_comm* c = new ks_comm();
  c->ctx = ctx;
  c->n_ranks = n_ranks;
  c->rank = rank;
  cudaSetDevice(ctx->device);
  if (cudaMalloc((void**)&c->pair_local, (2 + 2 * (size_t)n_ranks + 2) * sizeof(float)) != cudaSuccess) {
    ks_fail(ctx, KS_ERR_OOM, "comm_init: cudaMalloc failed");
    delete c;
    return nullptr;
  }
  c->idx_local = c->pair_local + 2 + 2 * (size_t)n_ranks;
  if (n_ranks > 1) {
    NcclApi& api = nccl_api();
    if (!api.ok) {
      ks_fail(ctx, KS_ERR_UNSUPPORTED, "comm_init: libnccl.so.2 could not be loaded (set KSEARCH_NCCL_LIB to its path)");
      ks_comm_destroy(c);
      return nullptr;
    }
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof id);
    ncclResult_t r = api.CommInitRank(&c->comm, n_ranks, id, rank);
    if (r != ncclSuccess) {
      ks_fail(ctx, KS_ERR_CUDA, "comm_init: ncclCommInitRank failed: %s", api.GetErrorString(r));
      c->comm = nullptr;
      ks_comm_destroy(c);
      return nullptr;
    }
  }
  return c;
}

void ks_comm_destroy(ks_comm* c) {
  if (!c) return;
  cudaSetDevice(c->ctx->device);
  cudaStreamSynchronize(c->ctx->stream);
  for (int r = 0; r < c->n_ranks && r < KS_P2P_MAX_RANKS; r++)
    if (r != c->rank && c->box[r]) cudaIpcCloseMemHandle(c->box[r]);
  if (c->box_local) cudaFree(c->box_local);
  if (c->comm) nccl_api().CommDestroy(c->comm);
  if (c->pair_local) cudaFree(c->pair_local);
  delete c;
}

// This rank's mailbox, created on first use, as a 64-byte handle the other ranks open (any host channel carries it).
int ks_comm_p2p_handle(ks_comm* c, void* handle_out) {
  if (!c || !handle_out) return KS_ERR_INVALID;
  ks_ctx* ctx = c->ctx;
  static_assert(sizeof(cudaIpcMemHandle_t) == KS_COMM_P2P_HANDLE_BYTES, "IPC handle size");
  KS_REQUIRE(ctx, c->n_ranks <= KS_P2P_MAX_RANKS, "comm_p2p: at most %d ranks", KS_P2P_MAX_RANKS);
  cudaSetDevice(ctx->device);
  if (!c->box_local) {
    const size_t bytes = 256 + 2 * (size_t)c->n_ranks * sizeof(unsigned long long);
    KS_CUDA(ctx, cudaMalloc((void**)&c->box_local, bytes));
    KS_CUDA(ctx, cudaMemset(c->box_local, 0, bytes));
    c->step = reinterpret_cast<unsigned*>(c->box_local + 2 * (size_t)c->n_ranks);
  }
  cudaIpcMemHandle_t h;
  KS_CUDA(ctx, cudaIpcGetMemHandle(&h, c->box_local));
  memcpy(handle_out, &h, sizeof h);
  return KS_OK;
}
// all_handles: n_ranks x 64 bytes, rank r's handle at r * 64 (this rank's own entry is ignored).  Collective in the
// sense that every rank must have created its mailbox first.  From then on ks_argmax_sharded exchanges over peer memory.
int ks_comm_p2p_open(ks_comm* c, const void* all_handles) {
  if (!c || !all_handles) return KS_ERR_INVALID;
  ks_ctx* ctx = c->ctx;
  KS_REQUIRE(ctx, c->box_local, "comm_p2p_open: call ks_comm_p2p_handle first");
  cudaSetDevice(ctx->device);
  for (int r = 0; r < c->n_ranks; r++) {
    if (r == c->rank) {
      c->box[r] = c->box_local;
      continue;
    }
    cudaIpcMemHandle_t h;
    memcpy(&h, (const char*)all_handles + (size_t)r * sizeof h, sizeof h);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "comm_p2p_open: rank %d's mailbox cannot be mapped: %s", r, cudaGetErrorString(e));
    c->box[r] = (unsigned long long*)p;
  }
  c->p2p = true;
  return KS_OK;
}
// what = 0: 1 exchanges over peer memory when the mailboxes are open (default), 0 always NCCL; what = 1: polls before
// the peer wait gives up; what = 2: zero this rank's mailbox and step counter (every rank, with no step in flight,
// after a wait gave up).
int ks_comm_set(ks_comm* c, int what, unsigned value) {
  if (!c) return KS_ERR_INVALID;
  if (what == 0) c->use_p2p = value != 0;
  else if (what == 1) c->poll_limit = value ? value : 1u;
  else if (what == 2 && c->box_local) {
    cudaSetDevice(c->ctx->device);
    cudaStreamSynchronize(c->ctx->stream);
    cudaMemset(c->box_local, 0, 256 + 2 * (size_t)c->n_ranks * sizeof(unsigned long long));
  } else if (what != 2) return KS_ERR_INVALID;
  return KS_OK;
}

int ks_comm_rank(const ks_comm* c) { return c ? c->rank : -1; }
int ks_comm_size(const ks_comm* c) { return c ? c->n_ranks : 0; }

int ks_comm_all_gather_f32(ks_comm* c, ks_buf* all, size_t all_off, size_t count) {
  if (!c) return KS_ERR_INVALID;
  ks_ctx* ctx = c->ctx;
  KS_REQUIRE(ctx, count > 0, "all_gather: count must be > 0");
  KS_REQUIRE(ctx, ks_fits(all, all_off * 4, (size_t)c->n_ranks * count * 4), "all_gather: gathered buffer too small");
  if (c->n_ranks == 1) return KS_OK;
  float* base = (float*)all->dptr + all_off;
  ncclResult_t r = nccl_api().AllGather(base + (size_t)c->rank * count, base, count, ncclFloat32, c->comm, ctx->stream);
  if (r != ncclSuccess) return ks_fail(ctx, KS_ERR_CUDA, "ncclAllGather failed: %s", nccl_api().GetErrorString(r));
  return KS_OK;
}

int ks_matvec_sharded(ks_comm* c, size_t rows_local, size_t rows_per_rank, size_t cols, ks_dtype wdtype, const ks_buf* W_local,
                      size_t w_byte_off, const ks_buf* x, size_t x_off, ks_buf* y_all, size_t y_off, int gather) {
  if (!c) return KS_ERR_INVALID;
  ks_ctx* ctx = c->ctx;
  KS_REQUIRE(ctx, gather == KS_GATHER_NCCL || gather == KS_GATHER_NONE,
             "matvec_sharded: gather mode %d is not built (KS_GATHER_NCCL or KS_GATHER_NONE)", gather);
  KS_REQUIRE(ctx, rows_local <= rows_per_rank && rows_per_rank > 0, "matvec_sharded: rows_local %zu exceeds the per-rank slot %zu",
             rows_local, rows_per_rank);
  KS_REQUIRE(ctx, ks_fits(y_all, y_off * 4, (size_t)c->n_ranks * rows_per_rank * 4), "matvec_sharded: gathered buffer too small");
  int rc = KS_OK;
  if (rows_local)
    rc = ks_matvec(ctx, rows_local, cols, wdtype, W_local, w_byte_off, KS_F32, x, x_off, y_all, y_off + (size_t)c->rank * rows_per_rank, 1);
  if (rc || gather == KS_GATHER_NONE) return rc;
  return ks_comm_all_gather_f32(c, y_all, y_off, rows_per_rank);
}

int ks_argmax_sharded(ks_comm* c, size_t rows_local, size_t row0, float cap, const ks_buf* logits_local, size_t logits_off,
                      ks_buf* out_idx, size_t out_off) {
  if (!c) return KS_ERR_INVALID;
  ks_ctx* ctx = c->ctx;
  KS_REQUIRE(ctx, rows_local > 0 && rows_local <= (1ull << 24) && row0 + rows_local <= (1ull << 24),
             "argmax_sharded: indices must stay below 2^24 (they travel as f32)");
  KS_REQUIRE(ctx, cap > 0.0f, "argmax_sharded: cap must be > 0");
  KS_REQUIRE(ctx, ks_fits(logits_local, logits_off * 4, rows_local * 4), "argmax_sharded: logits buffer too small");
  KS_REQUIRE(ctx, ks_fits(out_idx, out_off * 4, 4), "argmax_sharded: output buffer too small");
  const float* lg = (const float*)logits_local->dptr + logits_off;
  int rc = ks_launch_softcap_argmax(ctx, rows_local, cap, KS_F32, lg, c->idx_local);
  if (rc) return rc;
  if (c->p2p && c->use_p2p && c->n_ranks > 1) {  // one kernel: store to every peer, poll the own mailbox, merge
    P2pArgs a{};
    for (int r = 0; r < c->n_ranks; r++) a.box[r] = c->box[r];
    a.step = c->step;
    a.n_ranks = (unsigned)c->n_ranks;
    a.rank = (unsigned)c->rank;
    a.row0 = (unsigned)row0;
    a.poll_limit = c->poll_limit;
    a.cap = cap;
    a.logits = lg;
    a.local_idx = c->idx_local;
    a.out_idx = (float*)out_idx->dptr + out_off;
    a.err = (unsigned*)ctx->ws + KS_WS_ERR_WORD;
    KS_LAUNCH(ctx, (argmax_p2p_kernel), 1, 32, 0, a);
    return ks_after_launch(ctx, "argmax_p2p");
  }
  float* pairs = c->pair_local + 2;  // gathered pairs; this rank's own pair is written in place
  KS_LAUNCH(ctx, (argmax_pair_kernel), 1, 32, 0, lg, (const float*)c->idx_local, cap, (unsigned)row0, pairs + 2 * (size_t)c->rank);
  if ((rc = ks_after_launch(ctx, "argmax_pair"))) return rc;
  if (c->n_ranks > 1) {
    ncclResult_t r = nccl_api().AllGather(pairs + 2 * (size_t)c->rank, pairs, 2, ncclFloat32, c->comm, ctx->stream);
    if (r != ncclSuccess) return ks_fail(ctx, KS_ERR_CUDA, "ncclAllGather failed: %s", nccl_api().GetErrorString(r));
  }
  KS_LAUNCH(ctx, (argmax_merge_kernel), 1, 32, 0, (const float*)pairs, c->n_ranks, (float*)out_idx->dptr + out_off);
  return ks_after_launch(ctx, "argmax_merge");
}

}  // extern "C"

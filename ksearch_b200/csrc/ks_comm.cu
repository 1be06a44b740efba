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

}  // namespace

struct ks_comm {
  ks_ctx* ctx = nullptr;
  ncclComm_t comm = nullptr;
  int n_ranks = 1, rank = 0;
  float* pair_local = nullptr;  // [2] this rank's (value, index), then [2 * n_ranks] gathered
  float* idx_local = nullptr;   // [1]
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
  if (c->comm) nccl_api().CommDestroy(c->comm);
  if (c->pair_local) cudaFree(c->pair_local);
  delete c;
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

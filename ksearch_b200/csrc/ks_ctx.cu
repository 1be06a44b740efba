// Context, buffers and stream-ordering calls: the CUDA counterpart of the
// reference's device runtime (crates/ksearch_metal/src/lib.rs:16-218).
#include <cstdlib>
#include <cstring>

#include "ks_internal.h"

int ks_fail(ks_ctx* ctx, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) ctx->err = buf;
  return code;
}

int ks_after_launch(ks_ctx* ctx, const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return ks_fail(ctx, KS_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
  ctx->launches++;
  return KS_OK;
}

static thread_local std::string g_create_err;

// Message for calls that have no context to hang an error on; read back with ks_last_error(NULL).
void ks_set_global_error(const char* msg) { g_create_err = msg ? msg : ""; }

extern "C" {

ks_ctx* ks_ctx_create(int device, uint64_t flags) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) {
    g_create_err = std::string("no CUDA device: ") + cudaGetErrorString(e);
    return nullptr;
  }
  if (device < 0 || device >= n) {
    g_create_err = "device index out of range";
    return nullptr;
  }
  cudaDeviceProp p;
  if (cudaGetDeviceProperties(&p, device) != cudaSuccess) {
    g_create_err = "cudaGetDeviceProperties failed";
    return nullptr;
  }
  if (p.major != 10) {
    g_create_err = "this library is built for sm_100a only (compute capability 10.x required)";
    return nullptr;
  }
  if (cudaSetDevice(device) != cudaSuccess) {
    g_create_err = "cudaSetDevice failed";
    return nullptr;
  }
  ks_ctx* c = new ks_ctx();
  c->device = device;
  c->sm_count = p.multiProcessorCount;
  c->cc_major = p.major;
  c->cc_minor = p.minor;
  c->smem_optin = p.sharedMemPerBlockOptin;
  c->pdl = (flags & 1u) != 0;
  const char* chip = getenv("KSEARCH_CHIP");
  c->chip = chip && *chip ? chip : p.name;
  if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) {
    g_create_err = "cudaStreamCreate failed";
    delete c;
    return nullptr;
  }
  if (cudaMalloc(&c->ws, 16384) != cudaSuccess || cudaMemset(c->ws, 0, 16384) != cudaSuccess) {
    g_create_err = "workspace allocation failed";
    cudaStreamDestroy(c->stream);
    delete c;
    return nullptr;
  }
  return c;
}

void ks_ctx_destroy(ks_ctx* c) {
  if (!c) return;
  cudaSetDevice(c->device);
  cudaStreamSynchronize(c->stream);
  for (cudaEvent_t ev : c->inflight) cudaEventDestroy(ev);
  if (c->stage_h) cudaFreeHost(c->stage_h);
  if (c->stage_x) ks_buf_free(c, c->stage_x);
  if (c->stage_y) ks_buf_free(c, c->stage_y);
  if (c->ws) cudaFree(c->ws);
  if (c->gemm_ws) cudaFree(c->gemm_ws);
  if (c->t0) cudaEventDestroy(c->t0);
  if (c->t1) cudaEventDestroy(c->t1);
  cudaStreamDestroy(c->stream);
  delete c;
}

const char* ks_last_error(const ks_ctx* c) { return c ? c->err.c_str() : g_create_err.c_str(); }
const char* ks_chip_name(const ks_ctx* c) { return c->chip.c_str(); }
int ks_ctx_device(const ks_ctx* c) { return c->device; }
int ks_ctx_sm_count(const ks_ctx* c) { return c->sm_count; }
void* ks_ctx_stream(const ks_ctx* c) { return (void*)c->stream; }
uint64_t ks_ctx_launch_count(const ks_ctx* c) { return c->launches; }

ks_buf* ks_buf_alloc(ks_ctx* c, size_t bytes) {
  if (!c) return nullptr;
  cudaSetDevice(c->device);
  ks_buf* b = new ks_buf();
  size_t n = bytes ? bytes : 16;
  n = (n + 255) & ~size_t(255);  // keep 16-byte vector loads of a ragged tail in bounds
  cudaError_t e = cudaMalloc(&b->dptr, n);
  if (e != cudaSuccess) {
    ks_fail(c, KS_ERR_OOM, "cudaMalloc(%zu) failed: %s", n, cudaGetErrorString(e));
    delete b;
    return nullptr;
  }
  cudaMemsetAsync(b->dptr, 0, n, c->stream);
  b->bytes = bytes;
  b->owned = true;
  return b;
}

ks_buf* ks_buf_wrap(ks_ctx* c, void* dptr, size_t bytes) {
  if (!c || !dptr) return nullptr;
  ks_buf* b = new ks_buf();
  b->dptr = dptr;
  b->bytes = bytes;
  b->owned = false;
  return b;
}

void ks_buf_free(ks_ctx* c, ks_buf* b) {
  if (!b) return;
  if (b->owned && b->dptr) {
    if (c) {
      cudaSetDevice(c->device);
      cudaStreamSynchronize(c->stream);
    }
    cudaFree(b->dptr);
  }
  delete b;
}

size_t ks_buf_size(const ks_buf* b) { return b ? b->bytes : 0; }
void* ks_buf_device_ptr(const ks_buf* b) { return b ? b->dptr : nullptr; }

int ks_buf_upload_async(ks_ctx* c, ks_buf* dst, size_t off, const void* host, size_t bytes) {
  KS_REQUIRE(c, ks_fits(dst, off, bytes), "upload: %zu bytes at offset %zu exceed buffer of %zu", bytes, off,
             dst ? dst->bytes : 0);
  KS_REQUIRE(c, host || !bytes, "upload: null host pointer");
  KS_CUDA(c, cudaMemcpyAsync((char*)dst->dptr + off, host, bytes, cudaMemcpyHostToDevice, c->stream));
  return KS_OK;
}
int ks_buf_download_async(ks_ctx* c, const ks_buf* src, size_t off, void* host, size_t bytes) {
  KS_REQUIRE(c, ks_fits(src, off, bytes), "download: %zu bytes at offset %zu exceed buffer of %zu", bytes, off,
             src ? src->bytes : 0);
  KS_REQUIRE(c, host || !bytes, "download: null host pointer");
  KS_CUDA(c, cudaMemcpyAsync(host, (const char*)src->dptr + off, bytes, cudaMemcpyDeviceToHost, c->stream));
  return KS_OK;
}
int ks_buf_upload(ks_ctx* c, ks_buf* dst, size_t off, const void* host, size_t bytes) {
  int rc = ks_buf_upload_async(c, dst, off, host, bytes);
  if (rc) return rc;
  KS_CUDA(c, cudaStreamSynchronize(c->stream));
  return KS_OK;
}
int ks_buf_download(ks_ctx* c, const ks_buf* src, size_t off, void* host, size_t bytes) {
  int rc = ks_buf_download_async(c, src, off, host, bytes);
  if (rc) return rc;
  KS_CUDA(c, cudaStreamSynchronize(c->stream));
  return KS_OK;
}
int ks_buf_zero(ks_ctx* c, ks_buf* b, size_t off, size_t bytes) {
  KS_REQUIRE(c, ks_fits(b, off, bytes), "zero: range exceeds buffer");
  KS_CUDA(c, cudaMemsetAsync((char*)b->dptr + off, 0, bytes, c->stream));
  return KS_OK;
}

void* ks_host_alloc_pinned(size_t bytes) {
  void* p = nullptr;
  if (cudaMallocHost(&p, bytes ? bytes : 1) != cudaSuccess) return nullptr;
  return p;
}
void ks_host_free_pinned(void* p) {
  if (p) cudaFreeHost(p);
}

// A "commit point" stands for one committed command buffer of the reference
// runtime: an event recorded behind everything enqueued so far.
int ks_flush(ks_ctx* c) {
  cudaEvent_t ev;
  KS_CUDA(c, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  cudaError_t e = cudaEventRecord(ev, c->stream);
  if (e != cudaSuccess) {
    cudaEventDestroy(ev);
    return ks_fail(c, KS_ERR_CUDA, "cudaEventRecord failed: %s", cudaGetErrorString(e));
  }
  c->inflight.push_back(ev);
  return KS_OK;
}

static void reap(ks_ctx* c) {
  while (!c->inflight.empty() && cudaEventQuery(c->inflight.front()) == cudaSuccess) {
    cudaEventDestroy(c->inflight.front());
    c->inflight.pop_front();
  }
}

int ks_wait_inflight_at_most(ks_ctx* c, int n) {
  if (n < 0) n = 0;
  reap(c);
  while ((int)c->inflight.size() > n) {
    KS_CUDA(c, cudaEventSynchronize(c->inflight.front()));
    cudaEventDestroy(c->inflight.front());
    c->inflight.pop_front();
  }
  return KS_OK;
}

int ks_synchronize(ks_ctx* c) {
  KS_CUDA(c, cudaStreamSynchronize(c->stream));
  for (cudaEvent_t ev : c->inflight) cudaEventDestroy(ev);
  c->inflight.clear();
  // a kernel whose bounded wait gave up leaves a mark instead of hanging
  unsigned flag = 0;
  KS_CUDA(c, cudaMemcpy(&flag, (unsigned*)c->ws + KS_WS_ERR_WORD, sizeof flag, cudaMemcpyDeviceToHost));
  if (flag) {
    cudaMemset((unsigned*)c->ws + KS_WS_ERR_WORD, 0, sizeof flag);
    return ks_fail(c, KS_ERR_TIMEOUT, "a device-side wait gave up (status word 0x%x)", flag);
  }
  return KS_OK;
}

int ks_timer_begin(ks_ctx* c) {
  if (!c->t0) {
    KS_CUDA(c, cudaEventCreate(&c->t0));
    KS_CUDA(c, cudaEventCreate(&c->t1));
  }
  KS_CUDA(c, cudaEventRecord(c->t0, c->stream));
  return KS_OK;
}

int ks_timer_end_ms(ks_ctx* c, float* ms) {
  KS_REQUIRE(c, c->t0 && ms, "timer_end without timer_begin");
  KS_CUDA(c, cudaEventRecord(c->t1, c->stream));
  KS_CUDA(c, cudaEventSynchronize(c->t1));
  KS_CUDA(c, cudaEventElapsedTime(ms, c->t0, c->t1));
  return KS_OK;
}

struct ks_graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
};

int ks_graph_begin(ks_ctx* c) {
  KS_CUDA(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
  return KS_OK;
}

ks_graph* ks_graph_end(ks_ctx* c) {
  ks_graph* g = new ks_graph();
  cudaError_t e = cudaStreamEndCapture(c->stream, &g->graph);
  if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
  if (e != cudaSuccess) {
    ks_fail(c, KS_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
    return nullptr;
  }
  return g;
}

int ks_graph_launch(ks_ctx* c, ks_graph* g) {
  KS_REQUIRE(c, g && g->exec, "graph_launch: null graph");
  KS_CUDA(c, cudaGraphLaunch(g->exec, c->stream));
  return KS_OK;
}

void ks_graph_free(ks_ctx* c, ks_graph* g) {
  if (!g) return;
  if (c) cudaStreamSynchronize(c->stream);
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  delete g;
}

int ks_plan_override(ks_ctx* c, const ks_plan* plan) {
  if (!c) return KS_ERR_INVALID;
  c->has_override = plan != nullptr;
  if (plan) c->override_plan = *plan;
  return KS_OK;
}

int ks_has_gpu_work(ks_ctx* c) {
  reap(c);
  if (!c->inflight.empty()) return 1;
  return cudaStreamQuery(c->stream) == cudaErrorNotReady ? 1 : 0;
}

}  // extern "C"

int ks_ctx_gemm_scratch(ks_ctx* c, size_t bytes, void** out) {
  if (bytes > c->gemm_ws_bytes) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(c->stream, &st);
    if (st != cudaStreamCaptureStatusNone)
      return ks_fail(c, KS_ERR_STATE, "gemm: scratch of %zu bytes must exist before the stream is captured", bytes);
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);  // launches that still read the old scratch
    if (c->gemm_ws) cudaFree(c->gemm_ws);
    c->gemm_ws = nullptr;
    c->gemm_ws_bytes = 0;
    if (cudaMalloc(&c->gemm_ws, bytes) != cudaSuccess) return ks_fail(c, KS_ERR_OOM, "gemm: cudaMalloc(%zu) failed", bytes);
    c->gemm_ws_bytes = bytes;
  }
  *out = c->gemm_ws;
  return KS_OK;
}

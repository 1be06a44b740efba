// TMA bulk streaming throughput vs copy size (per-warp rings), serialized graph launches
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
__device__ __forceinline__ uint32_t s32(const void* p){return (uint32_t)__cvta_generic_to_shared(p);}
__global__ void __launch_bounds__(256) tk(const uint8_t* src, size_t total, unsigned cs, int stages, unsigned* out) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  unsigned char* ring = smem + (size_t)warp * stages * cs;
  uint32_t bars = s32(smem + (size_t)nw * stages * cs) + warp * stages * 8;
  if (lane == 0) { for (int s = 0; s < stages; s++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bars + s*8)); asm volatile("fence.mbarrier_init.release.cluster;"); asm volatile("fence.proxy.async.shared::cta;"); }
  __syncwarp();
  size_t ncopy = total / cs; unsigned gw = blockIdx.x * nw + warp, GW = gridDim.x * nw;
  unsigned n = gw < ncopy ? (unsigned)((ncopy - gw + GW - 1) / GW) : 0;
  auto issue = [&](unsigned i){ if (lane == 0) { uint32_t bar = bars + (i % stages) * 8; asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(cs));
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" :: "r"(s32(ring + (size_t)(i % stages) * cs)), "l"(src + ((size_t)gw + (size_t)i * GW) * cs), "r"(cs), "r"(bar) : "memory"); } };
  for (unsigned i = 0; i < (unsigned)stages && i < n; i++) issue(i);
  unsigned acc = 0;
  for (unsigned i = 0; i < n; i++) {
    uint32_t bar = bars + (i % stages) * 8; unsigned par = (i / stages) & 1, ok = 0;
    for (int it = 0; it < (1 << 22) && !ok; it++) asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0,1,0,p;\n}" : "=r"(ok) : "r"(bar), "r"(par) : "memory");
    acc += ring[(size_t)(i % stages) * cs + lane * 4];
    __syncwarp();
    if (i + stages < n) { if (lane == 0) asm volatile("fence.proxy.async.shared::cta;"); __syncwarp(); issue(i + stages); }
  }
  if (acc == 0x7fffffff) out[0] = acc;
}
int main() {
  size_t total = 10616832; int ncopies = 40;
  uint8_t* buf; cudaMalloc(&buf, total * ncopies); cudaMemset(buf, 1, total * ncopies);
  unsigned* out; cudaMalloc(&out, 4);
  cudaStream_t s; cudaStreamCreate(&s); cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  cudaFuncSetAttribute(tk, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  for (unsigned cs : {864u, 1728u, 3456u, 6912u, 13824u}) for (int nw : {4, 8}) for (int cps : {1, 2}) {
    int stages = (int)(90 * 1024 / cps / (nw * cs)); if (stages > 8) stages = 8; if (stages < 1) continue;
    size_t smem = (size_t)nw * stages * cs + nw * stages * 8 + 128;
    cudaGraph_t g; cudaGraphExec_t ge;
    cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal);
    for (int c = 0; c < ncopies; c++) tk<<<148 * cps, nw * 32, smem, s>>>(buf + (size_t)c * total, total, cs, stages, out);
    cudaStreamEndCapture(s, &g); cudaGraphInstantiate(&ge, g, 0);
    cudaGraphLaunch(ge, s); cudaStreamSynchronize(s);
    cudaEventRecord(e0, s); for (int r = 0; r < 3; r++) cudaGraphLaunch(ge, s); cudaEventRecord(e1, s); cudaStreamSynchronize(s);
    float ms; cudaEventElapsedTime(&ms, e0, e1); double us = ms * 1e3 / (3.0 * ncopies);
    printf("cs %5u nw %d cps %d stages %d smem %6zu: %6.2f us  %7.1f GB/s (%s)\n", cs, nw, cps, stages, smem, us, total / us / 1e3, cudaGetErrorString(cudaGetLastError()));
    cudaGraphExecDestroy(ge); cudaGraphDestroy(g);
  }
  return 0;
}

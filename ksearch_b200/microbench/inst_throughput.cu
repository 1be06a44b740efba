// instruction throughput microbench: ops per clock per SM
#include <cstdio>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#define ITERS 4096
#define ILP 8
template <int OP>
__global__ void k(unsigned* out, long long* cyc, unsigned seed) {
  unsigned r[ILP]; float f[ILP]; float2 f2[ILP]; unsigned long long p[ILP];
  for (int i = 0; i < ILP; i++) { r[i] = seed + threadIdx.x * 31 + i; f[i] = r[i] * 1e-9f; f2[i] = make_float2(f[i], f[i] + 1.f); p[i] = ((unsigned long long)r[i] << 32) | r[i]; }
  float c1 = seed * 1e-7f + 1.0f, c2 = seed * 1e-8f;
  unsigned long long pc1 = ((unsigned long long)__float_as_uint(c1) << 32) | __float_as_uint(c1);
  unsigned long long pc2 = ((unsigned long long)__float_as_uint(c2) << 32) | __float_as_uint(c2);
  __syncthreads();
  long long t0 = clock64();
  #pragma unroll 1
  for (int it = 0; it < ITERS; it++) {
    #pragma unroll
    for (int i = 0; i < ILP; i++) {
      if (OP == 0) f[i] = fmaf(f[i], c1, c2);
      if (OP == 1) asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(p[i]) : "l"(pc1), "l"(pc2));
      if (OP == 2) asm volatile("add.rn.f32x2 %0, %0, %1;" : "+l"(p[i]) : "l"(pc2));
      if (OP == 3) asm volatile("lop3.b32 %0, %0, %1, %2, 0xEA;" : "+r"(r[i]) : "r"(seed), "r"(0x4B000000u));
      if (OP == 4) asm volatile("prmt.b32 %0, %0, %1, 0x7250;" : "+r"(r[i]) : "r"(seed));
      if (OP == 5) asm volatile("shf.r.clamp.b32 %0, %0, %1, 3;" : "+r"(r[i]) : "r"(seed));
      if (OP == 6) asm volatile("dp4a.u32.s32 %0, %0, %1, %0;" : "+r"(r[i]) : "r"(seed));
      if (OP == 7) { float t; asm volatile("cvt.rn.f32.u32 %0, %1;" : "=f"(t) : "r"(r[i])); r[i] = __float_as_uint(t) ^ seed; }
      if (OP == 8) asm volatile("fma.rn.f16x2 %0, %0, %1, %2;" : "+r"(r[i]) : "r"(seed), "r"(0x3c003c00u));
      if (OP == 9) asm volatile("mad.lo.u32 %0, %0, %1, %2;" : "+r"(r[i]) : "r"(seed), "r"(7u));
      if (OP == 10) { // my inner loop mix: 2 lop3 + fadd2 + ffma2 per 2 weights
        unsigned a, b; asm volatile("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(a) : "r"(r[i]), "r"(0xFu), "r"(0x4B000000u));
        asm volatile("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(b) : "r"(r[i]), "r"(0xF0u), "r"(0x4B000000u));
        unsigned long long q; asm volatile("mov.b64 %0, {%1,%2};" : "=l"(q) : "r"(a), "r"(b));
        asm volatile("add.rn.f32x2 %0, %0, %1;" : "+l"(q) : "l"(pc2));
        asm volatile("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(p[i]) : "l"(q), "l"(pc1));
      }
      if (OP == 11) { float t; asm volatile("cvt.rn.f32.s32 %0, %1;" : "=f"(t) : "r"(r[i])); f[i] = fmaf(t, c1, f[i]); }
      if (OP == 12) asm volatile("add.u32 %0, %0, %1;" : "+r"(r[i]) : "r"(seed));
    }
  }
  long long t1 = clock64();
  unsigned acc = 0;
  for (int i = 0; i < ILP; i++) acc ^= r[i] ^ __float_as_uint(f[i]) ^ (unsigned)p[i] ^ (unsigned)(p[i] >> 32) ^ __float_as_uint(f2[i].x);
  out[blockIdx.x * blockDim.x + threadIdx.x] = acc;
  if (threadIdx.x == 0) cyc[blockIdx.x] = t1 - t0;
}
template <int OP> void run(const char* name, int ops_per_iter_lane, int threads) {
  unsigned* out; long long* cyc; int nb = 148;
  cudaMalloc(&out, nb * threads * 4); cudaMalloc(&cyc, nb * 8);
  k<OP><<<nb, threads>>>(out, cyc, 3); cudaDeviceSynchronize();
  k<OP><<<nb, threads>>>(out, cyc, 5); cudaDeviceSynchronize();
  long long h[148]; cudaMemcpy(h, cyc, nb * 8, cudaMemcpyDeviceToHost);
  double c = 0; for (int i = 0; i < nb; i++) c += h[i]; c /= nb;
  double ops = (double)threads * ITERS * ILP * ops_per_iter_lane;
  printf("%-28s threads=%4d  %.1f lane-ops/clk/SM  (%.1f warp-instr/clk/SM)\n", name, threads, ops / c, ops / c / 32);
  cudaFree(out); cudaFree(cyc);
}
int main() {
  for (int th : {512, 1024}) {
    run<0>("ffma", 1, th); run<1>("fma.f32x2 (instr)", 1, th); run<2>("add.f32x2 (instr)", 1, th);
    run<3>("lop3", 1, th); run<4>("prmt", 1, th); run<5>("shf", 1, th); run<6>("dp4a", 1, th);
    run<7>("cvt.f32.u32 (+xor)", 2, th); run<8>("hfma2", 1, th); run<9>("imad", 1, th); run<12>("iadd", 1, th);
    run<10>("mix 2lop3+add2+fma2 (4 instr)", 4, th); run<11>("i2f+ffma", 2, th);
  }
  return 0;
}

// Instruction-cache capacity probe: a loop whose body is K blocks of 256 straight-line FFMAs (4 KiB of code
// each).  Prints cycles per instruction and warp for 1 and 148 blocks of 1, 4 and 8 warps.
// Build: nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o icache_probe icache_probe.cu
#include <cstdio>
#include <cuda_runtime.h>
#define F1 asm volatile("fma.rn.f32 %0, %0, %1, %2;" : "+f"(a) : "f"(b), "f"(c)); asm volatile("fma.rn.f32 %0, %0, %1, %2;" : "+f"(d) : "f"(b), "f"(c)); asm volatile("fma.rn.f32 %0, %0, %1, %2;" : "+f"(e) : "f"(b), "f"(c)); asm volatile("fma.rn.f32 %0, %0, %1, %2;" : "+f"(f) : "f"(b), "f"(c));
#define F4 F1 F1 F1 F1
#define F16 F4 F4 F4 F4
#define F64 F16 F16 F16 F16
template <int K>
__global__ void probe(float* out, int iters, long long* cyc) {
  float a = threadIdx.x, b = 1.0001f, c = 0.5f, d = 1.f, e = 2.f, f = 3.f;
  long long t0 = clock64();
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int k = 0; k < K; ++k) { F64 if (cyc == nullptr) return; }   // 256 instructions = 4 KiB per block
  }
  long long t1 = clock64();
  if (threadIdx.x == 0) cyc[blockIdx.x] = t1 - t0;
  out[blockIdx.x * blockDim.x + threadIdx.x] = a + d + e + f;
}
template <int K>
void run(int blocks, int threads) {
  float* out; long long* cyc;
  cudaMalloc(&out, blocks * threads * 4); cudaMalloc(&cyc, blocks * 8);
  int iters = 8192 / K; if (iters < 16) iters = 16;
  probe<K><<<blocks, threads>>>(out, iters, cyc);
  probe<K><<<blocks, threads>>>(out, iters, cyc);
  cudaDeviceSynchronize();
  long long h[148]; cudaMemcpy(h, cyc, blocks * 8, cudaMemcpyDeviceToHost);
  long long mx = 0, mn = 1ll << 60; for (int i = 0; i < blocks; ++i) { if (h[i] > mx) mx = h[i]; if (h[i] < mn) mn = h[i]; }
  double n = (double)iters * K * 256;
  printf("code %4d KiB blocks %3d threads %3d : cycles/instr/warp min %.3f max %.3f  err=%d\n", K * 4, blocks, threads, mn / n, mx / n, (int)cudaGetLastError());
  cudaFree(out); cudaFree(cyc);
}
int main() {
  for (int blocks : {1, 148}) for (int threads : {32, 128, 256}) {
    run<2>(blocks, threads); run<4>(blocks, threads); run<6>(blocks, threads); run<8>(blocks, threads); run<12>(blocks, threads);
    run<16>(blocks, threads); run<24>(blocks, threads); run<32>(blocks, threads); run<48>(blocks, threads); run<64>(blocks, threads);
  }
  return 0;
}

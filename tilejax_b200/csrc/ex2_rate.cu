// Throughput of the exponential instruction in its f32, f16x2 and bf16x2 forms, as the attention kernel's softmax would
// use them: cycles per warp instruction per SM sub-partition with four warps on each (148 CTAs x 512 threads), eight
// independent chains a thread. A standalone timing program, not part of the library:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o ex2_rate tilejax_b200/csrc/ex2_rate.cu && ./ex2_rate
// Measured on a B200: 8.0 cycles for ex2.approx.ftz.f32 (32 results), 16.0 for ex2.approx.f16x2 and
// ex2.approx.ftz.bf16x2 (64 results): the same four results a cycle per sub-partition in every format.
#include <cstdio>
#include <cuda_runtime.h>
template <int MODE>
__global__ void rate(unsigned* out, long long* cyc, int iters) {
  float a[8];
  unsigned h[8];
  for (int i = 0; i < 8; ++i) a[i] = -0.001f * (threadIdx.x + i), h[i] = (MODE == 1 ? 0xB800B800u : 0xBF00BF00u);
  const long long t0 = clock64();
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (MODE == 0) asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(a[i]));
      if (MODE == 1) asm volatile("ex2.approx.f16x2 %0, %0;" : "+r"(h[i]));
      if (MODE == 2) asm volatile("ex2.approx.ftz.bf16x2 %0, %0;" : "+r"(h[i]));
    }
  }
  const long long t1 = clock64();
  unsigned acc = 0;
  for (int i = 0; i < 8; ++i) acc ^= h[i] ^ __float_as_uint(a[i]);
  out[blockIdx.x * blockDim.x + threadIdx.x] = acc;
  if (threadIdx.x == 0) cyc[blockIdx.x] = t1 - t0;
}
template <int MODE>
void run(const char* name) {
  const int ctas = 148, threads = 512, iters = 2000;
  unsigned* out;
  long long* cyc;
  cudaMalloc(&out, ctas * threads * 4);
  cudaMalloc(&cyc, ctas * 8);
  rate<MODE><<<ctas, threads>>>(out, cyc, 10);
  rate<MODE><<<ctas, threads>>>(out, cyc, iters);
  long long host[148];
  cudaMemcpy(host, cyc, sizeof(host), cudaMemcpyDeviceToHost);
  double mean = 0;
  for (int i = 0; i < ctas; ++i) mean += host[i];
  mean /= ctas;
  const double per = mean / (4.0 * 8 * iters);  // four warps a sub-partition, eight instructions an iteration
  printf("%s: %.2f cycles per warp instruction per sub-partition (%s) err=%s\n", name, per,
         MODE == 0 ? "32 results" : "64 results", cudaGetErrorString(cudaGetLastError()));
  cudaFree(out), cudaFree(cyc);
}
int main() {
  run<0>("ex2.approx.ftz.f32");
  run<1>("ex2.approx.f16x2");
  run<2>("ex2.approx.ftz.bf16x2");
  return 0;
}

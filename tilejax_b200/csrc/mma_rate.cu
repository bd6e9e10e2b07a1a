// A standalone timing program, not part of the library: cycles per tcgen05.mma (kind::f16, bf16 operands, f32
// accumulation, cta_group::1) for several tile shapes, with both operands in shared memory or A in tensor memory.
// Every CTA (one per SM) issues 320 MMAs of a shape back to back from one elected lane, commits once and waits for the
// commit (a bounded wait), twice; the second pass is reported, averaged over the CTAs: "issue" = cycles until the last
// MMA was issued, "complete" = until the commit arrived. Operands are whatever shared / tensor memory holds (zeros);
// results are discarded. What it showed on a B200: an MMA takes max(N / 2 cycles whether M is 64 or 128, bytes of its
// shared-memory operands / 128 B per cycle) plus ~4 (64 x 32 x 16: 27.6 cycles from shared memory, 19.9 with A in TMEM).
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_rate tilejax_b200/csrc/mma_rate.cu -lcuda
//   ./mma_rate
#include <cstdio>
#include "tjx_ptx.cuh"
using namespace tjx;
struct Cfg { int m, n, a_mn, ts; };
constexpr int NCFG = 20;
__constant__ Cfg cfgs[NCFG] = {{64, 32, 0, 0}, {64, 64, 0, 0}, {64, 128, 0, 0}, {64, 256, 0, 0}, {128, 32, 0, 0}, {128, 64, 0, 0},
                               {128, 128, 0, 0}, {128, 256, 0, 0}, {128, 64, 1, 0}, {64, 64, 1, 0}, {64, 256, 0, 1}, {128, 256, 0, 1},
                               {64, 48, 0, 0}, {128, 48, 0, 0}, {64, 32, 0, 1}, {64, 48, 0, 1}, {64, 64, 0, 1}, {64, 32, 0, 2}, {64, 64, 0, 2}, {128, 64, 0, 1}};
__global__ void __launch_bounds__(64, 1) rate_kernel(long long* out, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* bp = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t a_base = base, b_base = base + 80 * 1024, bar = base + 160 * 1024;
  volatile uint32_t* holder = reinterpret_cast<volatile uint32_t*>(bp + 160 * 1024 + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bp + 160 * 1024 + 24);
  for (int i = threadIdx.x; i < 160 * 1024 / 16; i += blockDim.x) reinterpret_cast<uint4*>(bp)[i] = make_uint4(0, 0, 0, 0);
  const int warp = uniform_warp_index();
  if (threadIdx.x == 0) { mbar_init(bar, 1); *abort_flag = 0; mbar_fence_init(); }
  if (warp == 0) { tmem_alloc(smem_u32(const_cast<uint32_t*>(holder)), 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = __shfl_sync(0xFFFFFFFFu, *holder, 0);
  if (warp == 0) {
    uint32_t phase = 0;
    for (int c = 0; c < NCFG; ++c) {
      const Cfg cf = cfgs[c];
      const uint32_t idesc = idesc_bf16_f32(cf.m, cf.n, cf.a_mn, 0);
      for (int rep = 0; rep < 2; ++rep) {
        const long long t0 = clock64();
        for (int blk = 0; blk < 10; ++blk) {   // ten 64-k blocks, as a 640-wide score product walks them
          // K-major A: m rows x 128 B per block (8 KB for 64 rows); B: n rows x 128 B.
          const uint64_t a0 = cf.a_mn ? smem_desc_sw128(a_base + (blk & 3) * 16384, 8192, 1024) : smem_desc_sw128(a_base + blk * 8192, 16, 1024);
          const uint64_t b0 = smem_desc_sw128(b_base + (blk & 1) * 32768, 16, 1024);  // 256 rows x 128 B = 32 KB: stays inside the 80 KB B region
          for (int half = 0; half < 4; ++half) {  // 4 x 8 = 32 MMAs per block -> 320 in all
            uint64_t ad[8], bd[8];
            uint32_t at[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              ad[k] = a0 + (cf.a_mn ? (k & 3) * (2048 >> 4) : (k & 3) * (32 >> 4));
              bd[k] = b0 + (k & 3) * (32 >> 4);
              at[k] = tmem + (cf.ts == 2 ? (16u << 16) : 0u) + 256 + (k & 3) * 8;
            }
            if (cf.ts) {
              const uint32_t dd = tmem + (cf.ts == 2 ? (16u << 16) : 0u);
              mma_ts_x4(dd, at, bd, idesc, 1u);
              mma_ts_x4(dd, at + 4, bd + 4, idesc, 1u);
            } else {
              mma_ss_x8(tmem, ad, bd, idesc, 1u);
            }
          }
        }
        const long long t1 = clock64();
        mma_commit_elected(bar);
        const bool ok = __all_sync(0xFFFFFFFFu, mbar_wait(bar, phase, abort_flag, status, TJX_ERR_WAIT_OTHER));
        phase ^= 1u;
        const long long t2 = clock64();
        if (!ok) { c = NCFG; break; }
        if (rep == 1 && threadIdx.x == 0) {
          out[(blockIdx.x * NCFG + c) * 2] = t1 - t0;
          out[(blockIdx.x * NCFG + c) * 2 + 1] = t2 - t0;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}
int main() {
  long long* out; int* status;
  const int grid = 148;
  cudaMalloc(&out, grid * NCFG * 2 * sizeof(long long)); cudaMemset(out, 0, grid * NCFG * 2 * sizeof(long long));
  cudaMalloc(&status, 8); cudaMemset(status, 0, 8);
  const int smem = 160 * 1024 + 1024 + 64;
  cudaFuncSetAttribute(rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  for (int i = 0; i < 2; ++i) rate_kernel<<<grid, 64, smem>>>(out, status);
  cudaError_t e = cudaDeviceSynchronize();
  printf("sync: %s\n", cudaGetErrorString(e));
  static long long h[148 * NCFG * 2]; int st[2];
  cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost); cudaMemcpy(st, status, 8, cudaMemcpyDeviceToHost);
  printf("status %d\n", st[0]);
  Cfg hc[NCFG]; cudaMemcpyFromSymbol(hc, cfgs, sizeof(hc));
  for (int c = 0; c < NCFG; ++c) {
    double issue = 0, total = 0;
    for (int b = 0; b < grid; ++b) issue += h[(b * NCFG + c) * 2], total += h[(b * NCFG + c) * 2 + 1];
    printf("M %3d N %3d a_mn %d ts %d: issue %.1f cycles/MMA, complete %.1f cycles/MMA (ideal %.1f)\n", hc[c].m, hc[c].n, hc[c].a_mn,
           hc[c].ts, issue / grid / 320, total / grid / 320, 2.0 * hc[c].m * hc[c].n * 16 / 8192);
  }
  return 0;
}

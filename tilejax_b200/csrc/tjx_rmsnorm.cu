// RMSNorm fused with the projection after it: out = rmsnorm(x) @ w, the loop nest `rmsnorm_matmul`
// (examples/rmsnorm_matmul.py:31-47). The row scale commutes with the matmul,
//     rmsnorm(x) @ w = rsqrt(mean(x^2) + eps) * ((x * gamma) @ w),
// so the work is one bandwidth pass over x and one matmul:
//   rmsnorm_prepare_kernel   reads x once: writes xg = bf16(f32(x) * f32(gamma)) — the operand the reference feeds
//                            its `@` (examples/rmsnorm_matmul.py:44) — and each row's scale rsqrt(sum(x^2) / D + eps)
//   the matmul step loop     (tjx_gemm.cu) on xg and w, its epilogue multiplying row r of the f32 accumulator by
//                            scale[r] before the one rounding to the output dtype (examples/rmsnorm_matmul.py:45-46)
// The normalised activations are never written; xg (the gamma-scaled ones) and the scales live in the caller's
// workspace. HBM traffic beyond the matmul's: 2 M D bytes read + 2 M D + 4 M bytes written.
#include <algorithm>

#include "tjx_host.cuh"
#include "tjx_ptx.cuh"

#include "../../include/tilejax_b200.h"

namespace tjx {

int gemm_launch(const void* x, const void* y, void* out, int M, int N, int K, int y_transposed, int tm, int tn, int tk,
                int stages, int out_f32, int causal, const int32_t* tile_i, const int32_t* tile_j, int n_tiles,
                const int32_t* fill_i, const int32_t* fill_j, int n_fills, const float* row_scale, int activation,
                tjx_stream_t stream);

constexpr int RMS_WARPS = 8;  // rows per CTA: a warp per row

// One warp per row: 16 bytes (8 bf16) per lane per pass, coalesced; the sum of squares in f32, lanes combined by
// shuffles. D is a multiple of 8.
__global__ void __launch_bounds__(RMS_WARPS * 32)
    rmsnorm_prepare_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                           __nv_bfloat16* __restrict__ xg, float* __restrict__ scale, int M, int D, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * RMS_WARPS + warp;
  if (row >= M) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * D);
  const uint4* g = reinterpret_cast<const uint4*>(gamma);
  uint4* dst = reinterpret_cast<uint4*>(xg + static_cast<size_t>(row) * D);
  float sum = 0.f;
  for (int u = lane; u < D / 8; u += 32) {
    const uint4 a = src[u], b = __ldg(g + u);
    const uint32_t av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float x0 = bf16_lo(av[i]), x1 = bf16_hi(av[i]);
      sum = fmaf(x0, x0, sum);
      sum = fmaf(x1, x1, sum);
      r[i] = pack_bf16(x0 * bf16_lo(bv[i]), x1 * bf16_hi(bv[i]));
    }
    dst[u] = make_uint4(r[0], r[1], r[2], r[3]);
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
  if (lane == 0) scale[row] = rsqrtf(sum / static_cast<float>(D) + eps);
  chain_release();  // the matmul chained behind may be scheduled once every CTA is here (or gone): it sets itself up
                    // beside this kernel's tail and waits for the rows on the device
}

static size_t rms_align256(size_t n) { return (n + 255) & ~static_cast<size_t>(255); }

}  // namespace tjx

extern "C" {

size_t tjx_rmsnorm_gemm_workspace_bytes(int M, int D) {
  if (M <= 0 || D <= 0) return 0;
  return tjx::rms_align256(static_cast<size_t>(M) * D * 2) + tjx::rms_align256(static_cast<size_t>(M) * sizeof(float));
}

int tjx_rmsnorm_gemm_bf16(const void* x, const void* gamma, const void* w, void* out, int M, int N, int D, float eps,
                          int tm, int tn, int tk, int out_f32, void* workspace, size_t workspace_bytes,
                          tjx_stream_t stream) {
  using namespace tjx;
  if (int rc = check_device()) return rc;
  if (!x || !gamma || !w || !out) return fail(TJX_E_ARG, "x, gamma, w or out is null");
  if (M <= 0 || N <= 0 || D <= 0 || D % 8 != 0) return fail(TJX_E_ARG, "M, N, D must be positive and D a multiple of 8");
  if (!(eps >= 0.f)) return fail(TJX_E_ARG, "eps must not be negative");
  const uintptr_t ptrs[] = {reinterpret_cast<uintptr_t>(x), reinterpret_cast<uintptr_t>(gamma)};
  for (uintptr_t a : ptrs)
    if (a & 15u) return fail(TJX_E_ARG, "x and gamma must be 16-byte aligned");
  const size_t need = tjx_rmsnorm_gemm_workspace_bytes(M, D);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(TJX_E_ARG, "workspace is null or smaller than tjx_rmsnorm_gemm_workspace_bytes");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(TJX_E_ARG, "workspace must be 256-byte aligned");
  __nv_bfloat16* xg = static_cast<__nv_bfloat16*>(workspace);
  float* scale = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + rms_align256(static_cast<size_t>(M) * D * 2));
  const int grid = (M + RMS_WARPS - 1) / RMS_WARPS;
  rmsnorm_prepare_kernel<<<grid, RMS_WARPS * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(gamma), xg, scale, M, D, eps);
  TJX_CUDA(cudaGetLastError());
  LaunchChain chain(CHAIN_WAITS);
  return gemm_launch(xg, w, out, M, N, D, 0, tm, tn, tk, 0, out_f32, 0, nullptr, nullptr, 0, nullptr, nullptr, 0, scale, 0,
                     stream);
}

}  // extern "C"

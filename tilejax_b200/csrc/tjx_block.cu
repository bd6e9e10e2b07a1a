// A whole attention block: causal multi-head attention, the RMSNorm after it and the feed-forward layer, the loop
// nest `attention_block` (examples/attention_block.py:49-85):
//     a   = the heads of softmax(q_h k_h^T + causal mask) v_h side by side     (B * S, D), D = H * Dh, f32
//     n   = bf16(a * rsqrt(mean(a^2) + eps) * gamma)
//     out = bf16(gelu(n @ w_up)) @ w_down                                      (B * S, D)
// The reference keeps a query block's `a`, `n` and hidden activations in on-chip memory across two reduction
// phases. A 128-row block of `a` at D = 2048 is 1 MB, four times an SM's shared memory, so here the phases are four
// launches on one stream and the intermediates go through the caller's workspace, which at these sizes stays in the
// 126 MB L2:
//   attention_kernel        (tjx_attention.cu) with its epilogue writing a's rows in f32, heads side by side
//   rmsnorm_rows_kernel     a warp per row: the sum of squares, then n in bf16
//   the matmul step loop    (tjx_gemm.cu) n @ w_up with tanh GELU on the f32 accumulator before the one rounding
//   the matmul step loop    hidden @ w_down
// The user's block_f only decides in which order the reference adds the hidden units' contributions in f32; the
// second matmul adds them in its own order (blocks of 64).
#include <algorithm>

#include "tjx_host.cuh"
#include "tjx_ptx.cuh"

#include "../../include/tilejax_b200.h"

namespace tjx {

int gemm_launch(const void* x, const void* y, void* out, int M, int N, int K, int y_transposed, int tm, int tn, int tk,
                int stages, int out_f32, int causal, const int32_t* tile_i, const int32_t* tile_j, int n_tiles,
                const int32_t* fill_i, const int32_t* fill_j, int n_fills, const float* row_scale, int activation,
                tjx_stream_t stream);
int attention_launch(const void* q, const void* k, const void* v, void* out, float* out_heads, int B, int H, int S,
                     int D, int block_q, int block_kv, const int32_t* step_tile, const int32_t* step_code,
                     int pattern_steps, int pattern_tiles, tjx_stream_t stream);

constexpr int ROWS_WARPS = 8;  // rows per CTA: a warp per row

// n[r, :] = bf16(a[r, :] * rsqrt(mean(a[r, :]^2) + eps) * gamma): two passes over the row (the second one hits L1/L2),
// 16 bytes of a per lane per load. D is a multiple of 8.
__global__ void __launch_bounds__(ROWS_WARPS * 32)
    rmsnorm_rows_kernel(const float* __restrict__ a, const __nv_bfloat16* __restrict__ gamma,
                        __nv_bfloat16* __restrict__ n, int M, int D, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * ROWS_WARPS + warp;
  chain_wait();  // launched behind the attention kernel, whose rows it reads
  if (row >= M) return;
  const float4* src = reinterpret_cast<const float4*>(a + static_cast<size_t>(row) * D);
  float sum = 0.f;
  for (int u = lane; u < D / 4; u += 32) {
    const float4 x = src[u];
    sum = fmaf(x.x, x.x, sum), sum = fmaf(x.y, x.y, sum), sum = fmaf(x.z, x.z, sum), sum = fmaf(x.w, x.w, sum);
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, d);
  const float scale = rsqrtf(sum / static_cast<float>(D) + eps);
  const uint2* g = reinterpret_cast<const uint2*>(gamma);
  uint2* dst = reinterpret_cast<uint2*>(n + static_cast<size_t>(row) * D);
  for (int u = lane; u < D / 4; u += 32) {
    const float4 x = src[u];
    const uint2 gv = __ldg(g + u);
    dst[u] = make_uint2(pack_bf16(x.x * scale * bf16_lo(gv.x), x.y * scale * bf16_hi(gv.x)),
                        pack_bf16(x.z * scale * bf16_lo(gv.y), x.w * scale * bf16_hi(gv.y)));
  }
  chain_release();  // (a CTA that has written its rows: the matmul behind is scheduled when every CTA is here or gone)
}

static size_t block_align256(size_t n) { return (n + 255) & ~static_cast<size_t>(255); }

// The largest matmul tile edge of 512, 256, 128 that divides n (n is a multiple of 128 here).
static int tile_edge(int n) { return n % 512 == 0 ? 512 : n % 256 == 0 ? 256 : 128; }

}  // namespace tjx

extern "C" {

size_t tjx_attention_block_workspace_bytes(int B, int H, int S, int Dh, int F) {
  if (B <= 0 || H <= 0 || S <= 0 || Dh <= 0 || F <= 0) return 0;
  const size_t rows = static_cast<size_t>(B) * S, D = static_cast<size_t>(H) * Dh;
  return tjx::block_align256(rows * D * 4) + tjx::block_align256(rows * D * 2) + tjx::block_align256(rows * F * 2);
}

int tjx_attention_block_bf16(const void* q, const void* k, const void* v, const void* gamma, const void* w_up,
                             const void* w_down, void* out, int B, int H, int S, int Dh, int F, int block_q,
                             int block_kv, float eps, const int32_t* step_tile, const int32_t* step_code,
                             int pattern_steps, int pattern_tiles, void* workspace, size_t workspace_bytes,
                             tjx_stream_t stream) {
  using namespace tjx;
  if (int rc = check_device()) return rc;
  if (!q || !k || !v || !gamma || !w_up || !w_down || !out) return fail(TJX_E_ARG, "an input or out is null");
  if (B <= 0 || H <= 0 || S <= 0 || F <= 0) return fail(TJX_E_ARG, "sizes must be positive");
  if (Dh != 128) return fail(TJX_E_ARG, "head dimension must be 128");
  if (S % 128 != 0) return fail(TJX_E_ARG, "S must be a multiple of 128");
  if (F % 128 != 0) return fail(TJX_E_ARG, "the hidden width must be a multiple of 128");
  if (static_cast<long long>(B) * S >= (1ll << 31) / 128) return fail(TJX_E_LIMIT, "B * S * 128 must fit in int32");
  const size_t need = tjx_attention_block_workspace_bytes(B, H, S, Dh, F);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(TJX_E_ARG, "the workspace is smaller than tjx_attention_block_workspace_bytes says");
  if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return fail(TJX_E_ARG, "the workspace must be 256-byte aligned");
  const int M = B * S, D = H * Dh;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* a = reinterpret_cast<float*>(ws);
  __nv_bfloat16* normed = reinterpret_cast<__nv_bfloat16*>(ws + block_align256(static_cast<size_t>(M) * D * 4));
  __nv_bfloat16* hidden = reinterpret_cast<__nv_bfloat16*>(ws + block_align256(static_cast<size_t>(M) * D * 4) +
                                                           block_align256(static_cast<size_t>(M) * D * 2));
  // The four launches are chained: each may be scheduled while the one in front of it still runs, sets itself up
  // (barriers, tensor memory, descriptors) beside that kernel's tail and waits for its results on the device.
  {
    LaunchChain chain(CHAIN_RELEASES);
    if (int rc = attention_launch(q, k, v, nullptr, a, B, H, S, Dh, block_q, block_kv, step_tile, step_code,
                                  pattern_steps, pattern_tiles, stream))
      return rc;
  }
  {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((M + ROWS_WARPS - 1) / ROWS_WARPS), cfg.blockDim = dim3(ROWS_WARPS * 32);
    cfg.dynamicSmemBytes = 0, cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr, cfg.numAttrs = 1;
    TJX_CUDA(cudaLaunchKernelEx(&cfg, rmsnorm_rows_kernel, static_cast<const float*>(a),
                                static_cast<const __nv_bfloat16*>(gamma), normed, M, D, eps));
  }
  const int tm = tile_edge(M);
  {
    LaunchChain chain(CHAIN_WAITS | CHAIN_RELEASES);
    if (int rc = gemm_launch(normed, w_up, hidden, M, F, D, 0, tm, tile_edge(F), 512, 0, 0, 0, nullptr, nullptr, 0,
                             nullptr, nullptr, 0, nullptr, 1, stream))
      return rc;
  }
  LaunchChain chain(CHAIN_WAITS);
  return gemm_launch(hidden, w_down, out, M, D, F, 0, tm, tile_edge(D), 512, 0, 0, 0, nullptr, nullptr, 0, nullptr, nullptr,
                     0, nullptr, 0, stream);
}

}  // extern "C"

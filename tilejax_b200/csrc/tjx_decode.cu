// Ragged paged GQA decode attention on sm_100a, bound by HBM bandwidth: every valid K/V page is read once,
// with 16-byte coalesced loads straight into registers, f32 FMAs and warp-shuffle reductions (no tensor cores).
//
// The work is the device step table (tjx_steps.cu): the steps that run, one K/V page each, in tile (sequence)
// order. It is cut into chunks of CHUNK consecutive steps, a CTA per chunk, so ragged lengths balance by
// themselves. Inside a CTA warp w owns KV head w and its 4 query heads: a lane holds 8 of the 128 head
// dimensions (one 16-byte load) for one of two tokens, so one warp-wide load covers two tokens' K (or V) rows
// of that head. A chunk may cover the end of one sequence and the start of the next; every (sequence, chunk)
// piece writes an online-softmax partial (max, sum, accumulator) to scratch, and a small second kernel merges
// a sequence's partials, normalises and writes bf16.
//
// Follows `paged_gqa_decode` (examples/decode.py:199-223): positions >= lengths[b] masked to -1e30, the
// probabilities rounded to bf16 before multiplying V, 1 / max(row_sum, 1e-30), zeros for an empty sequence.
#include "tjx_host.cuh"
#include "tjx_ptx.cuh"

#include <mutex>
#include <string>

#include "../../include/tilejax_b200.h"

namespace tjx {

int launch_build_steps_lengths(const int32_t* lengths, int n_lengths, const int32_t* tile_values, int tiles,
                               int blocks, int value0, int value_step, int32_t* step_tile, int32_t* step_code,
                               int32_t* step_count, int32_t* tile_first, cudaStream_t stream);

constexpr int DEC_D = 128;         // head dimension
constexpr int DEC_SUB = 16;        // tokens a warp handles at a time (a page is a whole number of these)
constexpr int DEC_CHUNK = 8;       // steps (pages) per CTA
constexpr int DEC_WARPS = 8;       // KV heads per CTA
constexpr float DEC_MASK = -1e30f;

struct DecodeParams {
  const __nv_bfloat16* q;        // [B, 1, H, D]
  const __nv_bfloat16* k_pages;  // [num_pages, PAGE, Hkv * D]
  const __nv_bfloat16* v_pages;
  const int32_t* block_tables;   // [B, pages_per_seq]
  const int32_t* lengths;        // [B]
  const int32_t* step_tile;
  const int32_t* step_code;
  const int32_t* step_count;
  const int32_t* tile_first;     // [B + 1]
  float* ws_m;                   // [B, slots, H]
  float* ws_l;                   // [B, slots, H]
  float* ws_acc;                 // [B, slots, H, D]
  __nv_bfloat16* out;            // [B, 1, H, D]
  int B, H, Hkv, page_size, pages_per_seq, num_pages, slots;
};

__device__ __forceinline__ uint4 ld_nc_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

template <int DEC_GROUP>
__global__ void __launch_bounds__(DEC_WARPS * 32) decode_chunks_kernel(const DecodeParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.y * DEC_WARPS + warp;
  if (kvh >= p.Hkv) return;
  const int n_steps = p.step_count[0];
  const int chunk = blockIdx.x;
  const int s_begin = chunk * DEC_CHUNK;
  if (s_begin >= n_steps) return;
  const int s_end = min(s_begin + DEC_CHUNK, n_steps);

  const int half = lane >> 4;        // which of the two tokens a warp-wide load covers
  const int d0 = (lane & 15) * 8;    // this lane's 8 head dimensions
  const size_t row_elems = static_cast<size_t>(p.Hkv) * DEC_D;

  float q[DEC_GROUP][8];
  float acc[DEC_GROUP][8];
  float m[DEC_GROUP], l[DEC_GROUP];
  int cur = -1, cur_len = 0;

  auto flush = [&]() {
    if (cur < 0) return;
    const int slot = chunk - p.tile_first[cur] / DEC_CHUNK;
    const size_t base = (static_cast<size_t>(cur) * p.slots + slot) * p.H + kvh * DEC_GROUP;
#pragma unroll
    for (int h = 0; h < DEC_GROUP; ++h) {
      const float l_all = l[h] + __shfl_xor_sync(0xFFFFFFFFu, l[h], 16);
      float a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = acc[h][j] + __shfl_xor_sync(0xFFFFFFFFu, acc[h][j], 16);
      if (half == 0) {
        float4* dst = reinterpret_cast<float4*>(p.ws_acc + (base + h) * DEC_D + d0);
        dst[0] = make_float4(a[0], a[1], a[2], a[3]);
        dst[1] = make_float4(a[4], a[5], a[6], a[7]);
      }
      if (lane == 0) {
        p.ws_m[base + h] = m[h];
        p.ws_l[base + h] = l_all;
      }
    }
  };

  for (int s = s_begin; s < s_end; ++s) {
    const int t = p.step_tile[s];
    const int code = p.step_code[s];
    if (t != cur) {
      flush();
      cur = t;
      cur_len = p.lengths[t];
      const __nv_bfloat16* qp = p.q + (static_cast<size_t>(t) * p.H + kvh * DEC_GROUP) * DEC_D + d0;
#pragma unroll
      for (int h = 0; h < DEC_GROUP; ++h) {
        const uint4 u = *reinterpret_cast<const uint4*>(qp + h * DEC_D);
        q[h][0] = bf16_lo(u.x), q[h][1] = bf16_hi(u.x), q[h][2] = bf16_lo(u.y), q[h][3] = bf16_hi(u.y);
        q[h][4] = bf16_lo(u.z), q[h][5] = bf16_hi(u.z), q[h][6] = bf16_lo(u.w), q[h][7] = bf16_hi(u.w);
        m[h] = DEC_MASK, l[h] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[h][j] = 0.f;
      }
    }
    if (code & 4) continue;  // an empty step: the sequence has no valid position
    const int pg = code >> 3;
    int page = p.block_tables[static_cast<size_t>(t) * p.pages_per_seq + pg];
    page = min(max(page, 0), p.num_pages - 1);
    for (int sub = 0; sub < p.page_size; sub += DEC_SUB) {
    if (pg * p.page_size + sub >= cur_len) break;  // the rest of the page holds no valid position
    const size_t page_off =
        (static_cast<size_t>(page) * p.page_size + sub + half) * row_elems + kvh * DEC_D + d0;
    const __nv_bfloat16* kp = p.k_pages + page_off;
    const __nv_bfloat16* vp = p.v_pages + page_off;

    uint4 kr[DEC_SUB / 2], vr[DEC_SUB / 2];
#pragma unroll
    for (int i = 0; i < DEC_SUB / 2; ++i) kr[i] = ld_nc_16(kp + static_cast<size_t>(2 * i) * row_elems);
#pragma unroll
    for (int i = 0; i < DEC_SUB / 2; ++i) vr[i] = ld_nc_16(vp + static_cast<size_t>(2 * i) * row_elems);

    // Scores of this lane's token of each pair against the 4 query heads, summed over the 16 lanes that
    // share the token.
    float sc[DEC_GROUP][DEC_SUB / 2];
#pragma unroll
    for (int i = 0; i < DEC_SUB / 2; ++i) {
      const float k0 = bf16_lo(kr[i].x), k1 = bf16_hi(kr[i].x), k2 = bf16_lo(kr[i].y), k3 = bf16_hi(kr[i].y);
      const float k4 = bf16_lo(kr[i].z), k5 = bf16_hi(kr[i].z), k6 = bf16_lo(kr[i].w), k7 = bf16_hi(kr[i].w);
#pragma unroll
      for (int h = 0; h < DEC_GROUP; ++h) {
        float a = q[h][0] * k0;
        a = fmaf(q[h][1], k1, a), a = fmaf(q[h][2], k2, a), a = fmaf(q[h][3], k3, a);
        a = fmaf(q[h][4], k4, a), a = fmaf(q[h][5], k5, a), a = fmaf(q[h][6], k6, a), a = fmaf(q[h][7], k7, a);
        sc[h][i] = a;
      }
    }
#pragma unroll
    for (int i = 0; i < DEC_SUB / 2; ++i)
#pragma unroll
      for (int h = 0; h < DEC_GROUP; ++h) {
        float a = sc[h][i];
        a += __shfl_xor_sync(0xFFFFFFFFu, a, 8);
        a += __shfl_xor_sync(0xFFFFFFFFu, a, 4);
        a += __shfl_xor_sync(0xFFFFFFFFu, a, 2);
        a += __shfl_xor_sync(0xFFFFFFFFu, a, 1);
        const int pos = pg * p.page_size + sub + 2 * i + half;
        sc[h][i] = pos < cur_len ? a : DEC_MASK;
      }

    // Online softmax over the page; the probabilities are rounded to bf16 before they multiply V.
#pragma unroll
    for (int h = 0; h < DEC_GROUP; ++h) {
      float mx = sc[h][0];
#pragma unroll
      for (int i = 1; i < DEC_SUB / 2; ++i) mx = fmaxf(mx, sc[h][i]);
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 16));
      const float m_new = fmaxf(m[h], mx);
      const float alpha = __expf(m[h] - m_new);
      m[h] = m_new;
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < DEC_SUB / 2; ++i) {
        const float pr = __expf(sc[h][i] - m_new);
        sum += pr;
        sc[h][i] = __bfloat162float(__float2bfloat16_rn(pr));
      }
      l[h] = l[h] * alpha + sum;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[h][j] *= alpha;
    }
#pragma unroll
    for (int i = 0; i < DEC_SUB / 2; ++i) {
      const float v0 = bf16_lo(vr[i].x), v1 = bf16_hi(vr[i].x), v2 = bf16_lo(vr[i].y), v3 = bf16_hi(vr[i].y);
      const float v4 = bf16_lo(vr[i].z), v5 = bf16_hi(vr[i].z), v6 = bf16_lo(vr[i].w), v7 = bf16_hi(vr[i].w);
#pragma unroll
      for (int h = 0; h < DEC_GROUP; ++h) {
        const float pr = sc[h][i];
        acc[h][0] = fmaf(pr, v0, acc[h][0]), acc[h][1] = fmaf(pr, v1, acc[h][1]);
        acc[h][2] = fmaf(pr, v2, acc[h][2]), acc[h][3] = fmaf(pr, v3, acc[h][3]);
        acc[h][4] = fmaf(pr, v4, acc[h][4]), acc[h][5] = fmaf(pr, v5, acc[h][5]);
        acc[h][6] = fmaf(pr, v6, acc[h][6]), acc[h][7] = fmaf(pr, v7, acc[h][7]);
      }
    }
    }  // sub-blocks of the page
  }
  flush();
}

// Merge a sequence's partials: one warp per (sequence, query head), a lane per 4 head dimensions.
__global__ void __launch_bounds__(256) decode_combine_kernel(const DecodeParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= p.B * p.H) return;
  const int b = warp / p.H, h = warp - b * p.H;
  const int first = p.tile_first[b], next = p.tile_first[b + 1];
  const int n = (next - 1) / DEC_CHUNK - first / DEC_CHUNK + 1;  // a tile takes at least one step
  const size_t base = static_cast<size_t>(b) * p.slots * p.H + h;
  float mx = DEC_MASK;
  for (int i = 0; i < n; ++i) mx = fmaxf(mx, p.ws_m[base + static_cast<size_t>(i) * p.H]);
  float lsum = 0.f;
  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i = 0; i < n; ++i) {
    const size_t idx = base + static_cast<size_t>(i) * p.H;
    const float w = __expf(p.ws_m[idx] - mx);
    lsum += w * p.ws_l[idx];
    const float4 a = *reinterpret_cast<const float4*>(p.ws_acc + idx * DEC_D + lane * 4);
    o.x = fmaf(w, a.x, o.x), o.y = fmaf(w, a.y, o.y), o.z = fmaf(w, a.z, o.z), o.w = fmaf(w, a.w, o.w);
  }
  const float inv = 1.0f / fmaxf(lsum, 1e-30f);
  uint2 r;
  r.x = pack_bf16(o.x * inv, o.y * inv);
  r.y = pack_bf16(o.z * inv, o.w * inv);
  *reinterpret_cast<uint2*>(p.out + (static_cast<size_t>(b) * p.H + h) * DEC_D + lane * 4) = r;
}

static int decode_slots(int pages_per_seq) { return (pages_per_seq + DEC_CHUNK - 1) / DEC_CHUNK + 1; }

static size_t align256(size_t n) { return (n + 255) & ~static_cast<size_t>(255); }

}  // namespace tjx

extern "C" {

size_t tjx_paged_gqa_decode_workspace_bytes(int B, int H, int D, int pages_per_seq) {
  if (B <= 0 || H <= 0 || D <= 0 || pages_per_seq <= 0) return 0;
  const size_t rows = static_cast<size_t>(B) * tjx::decode_slots(pages_per_seq) * H;
  return 2 * tjx::align256(rows * sizeof(float)) + tjx::align256(rows * D * sizeof(float));
}

int tjx_paged_gqa_decode_bf16(const void* q, const void* k_pages, const void* v_pages, const int32_t* block_tables,
                              const int32_t* lengths, void* out, int B, int H, int Hkv, int D, int page_size,
                              int pages_per_seq, int num_pages, int32_t* step_tile, int32_t* step_code,
                              int32_t* step_count, int32_t* tile_first, void* workspace, size_t workspace_bytes,
                              tjx_stream_t stream) {
  using namespace tjx;
  if (int rc = check_device()) return rc;
  if (!q || !k_pages || !v_pages || !block_tables || !lengths || !out)
    return fail(TJX_E_ARG, "an input or output pointer is null");
  if (!step_tile || !step_code || !step_count || !tile_first)
    return fail(TJX_E_ARG, "a step table pointer is null");
  if (B <= 0 || H <= 0 || Hkv <= 0 || pages_per_seq <= 0 || num_pages <= 0)
    return fail(TJX_E_ARG, "sizes must be positive");
  if (D != DEC_D) return fail(TJX_E_ARG, "head dimension must be 128");
  if (page_size <= 0 || page_size % DEC_SUB != 0) return fail(TJX_E_ARG, "page size must be a multiple of 16");
  if (H % Hkv != 0) return fail(TJX_E_ARG, "H must be a multiple of Hkv");
  const int group = H / Hkv;
  if (group != 1 && group != 2 && group != 4 && group != 8)
    return fail(TJX_E_ARG, "H / Hkv must be 1, 2, 4 or 8");
  const size_t need = tjx_paged_gqa_decode_workspace_bytes(B, H, D, pages_per_seq);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(TJX_E_ARG, "workspace is null or smaller than tjx_paged_gqa_decode_workspace_bytes");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(TJX_E_ARG, "workspace must be 256-byte aligned");
  const uintptr_t ptrs[] = {reinterpret_cast<uintptr_t>(q), reinterpret_cast<uintptr_t>(k_pages),
                            reinterpret_cast<uintptr_t>(v_pages), reinterpret_cast<uintptr_t>(out)};
  for (uintptr_t a : ptrs)
    if (a & 15u) return fail(TJX_E_ARG, "q, k_pages, v_pages and out must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  if (int rc = launch_build_steps_lengths(lengths, B, nullptr, B, pages_per_seq, 0, page_size, step_tile, step_code,
                                          step_count, tile_first, s))
    return rc;

  DecodeParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_pages = static_cast<const __nv_bfloat16*>(k_pages);
  p.v_pages = static_cast<const __nv_bfloat16*>(v_pages);
  p.block_tables = block_tables, p.lengths = lengths;
  p.step_tile = step_tile, p.step_code = step_code, p.step_count = step_count, p.tile_first = tile_first;
  p.B = B, p.H = H, p.Hkv = Hkv, p.page_size = page_size, p.pages_per_seq = pages_per_seq, p.num_pages = num_pages;
  p.slots = decode_slots(pages_per_seq);
  const size_t rows = static_cast<size_t>(B) * p.slots * H;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  p.ws_m = reinterpret_cast<float*>(ws);
  p.ws_l = reinterpret_cast<float*>(ws + align256(rows * sizeof(float)));
  p.ws_acc = reinterpret_cast<float*>(ws + 2 * align256(rows * sizeof(float)));
  p.out = static_cast<__nv_bfloat16*>(out);

  const long long capacity = static_cast<long long>(B) * pages_per_seq;
  const int chunks = static_cast<int>((capacity + DEC_CHUNK - 1) / DEC_CHUNK);
  dim3 grid(chunks, (Hkv + DEC_WARPS - 1) / DEC_WARPS);
  switch (group) {
    case 1: decode_chunks_kernel<1><<<grid, DEC_WARPS * 32, 0, s>>>(p); break;
    case 2: decode_chunks_kernel<2><<<grid, DEC_WARPS * 32, 0, s>>>(p); break;
    case 4: decode_chunks_kernel<4><<<grid, DEC_WARPS * 32, 0, s>>>(p); break;
    default: decode_chunks_kernel<8><<<grid, DEC_WARPS * 32, 0, s>>>(p); break;
  }
  TJX_CUDA(cudaGetLastError());
  const int warps = B * H;
  decode_combine_kernel<<<(warps * 32 + 255) / 256, 256, 0, s>>>(p);
  TJX_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------------------
// Decode without any allocation by anyone: the partials live in a fixed array inside the library's image.

namespace tjx {

constexpr size_t STATIC_SCRATCH_BYTES = static_cast<size_t>(TJX_STATIC_SCRATCH_BYTES);

// Scratch for tjx_paged_gqa_decode_bf16_static. Every GPU that loads the library carries these 36 MiB until the
// process exits. In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_decode_scratch[STATIC_SCRATCH_BYTES];

static void* g_decode_scratch_addr[64];  // per device, filled on the device's first call
static std::mutex g_decode_scratch_mutex;

// The array's address on the current device, looked up once per device with that device current.
static int static_scratch_address(void** out) {
  int dev = 0;
  TJX_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(TJX_E_ARG, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_decode_scratch_mutex);
  if (g_decode_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_decode_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_decode_scratch)");
    if (ptr == nullptr) return fail(TJX_E_CUDA, "cudaGetSymbolAddress returned a null address");
    g_decode_scratch_addr[dev] = ptr;
  }
  *out = g_decode_scratch_addr[dev];
  return 0;
}

}  // namespace tjx

extern "C" {

size_t tjx_paged_gqa_decode_static_scratch_bytes(void) { return tjx::STATIC_SCRATCH_BYTES; }

int tjx_paged_gqa_decode_bf16_static(const void* q, const void* k_pages, const void* v_pages,
                                     const int32_t* block_tables, const int32_t* lengths, void* out, int B, int H,
                                     int Hkv, int D, int page_size, int pages_per_seq, int num_pages,
                                     int32_t* step_tile, int32_t* step_code, int32_t* step_count, int32_t* tile_first,
                                     tjx_stream_t stream) {
  using namespace tjx;
  if (int rc = check_device()) return rc;
  if (!q || !k_pages || !v_pages || !block_tables || !lengths || !out)
    return fail(TJX_E_ARG, "an input or output pointer is null");
  if (!step_tile || !step_code || !step_count || !tile_first)
    return fail(TJX_E_ARG, "a step table pointer is null");
  if (B <= 0 || H <= 0 || Hkv <= 0 || pages_per_seq <= 0 || num_pages <= 0)
    return fail(TJX_E_ARG, "sizes must be positive");
  if (D != DEC_D) return fail(TJX_E_ARG, "head dimension must be 128");
  if (page_size <= 0 || page_size % DEC_SUB != 0) return fail(TJX_E_ARG, "page size must be a multiple of 16");
  if (H % Hkv != 0) return fail(TJX_E_ARG, "H must be a multiple of Hkv");
  const int group = H / Hkv;
  if (group != 1 && group != 2 && group != 4 && group != 8)
    return fail(TJX_E_ARG, "H / Hkv must be 1, 2, 4 or 8");
  const size_t need = tjx_paged_gqa_decode_workspace_bytes(B, H, D, pages_per_seq);
  if (need > STATIC_SCRATCH_BYTES)
    return fail(TJX_E_LIMIT, "these sizes need " + std::to_string(need) + " bytes of scratch, more than the " +
                                 std::to_string(STATIC_SCRATCH_BYTES) +
                                 " bytes built into the library: use tjx_paged_gqa_decode_bf16 with a workspace");
  const uintptr_t ptrs[] = {reinterpret_cast<uintptr_t>(q), reinterpret_cast<uintptr_t>(k_pages),
                            reinterpret_cast<uintptr_t>(v_pages), reinterpret_cast<uintptr_t>(out)};
  for (uintptr_t a : ptrs)
    if (a & 15u) return fail(TJX_E_ARG, "q, k_pages, v_pages and out must be 16-byte aligned");
  void* scratch = nullptr;
  if (int rc = static_scratch_address(&scratch)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  if (int rc = launch_build_steps_lengths(lengths, B, nullptr, B, pages_per_seq, 0, page_size, step_tile, step_code,
                                          step_count, tile_first, s))
    return rc;

  DecodeParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_pages = static_cast<const __nv_bfloat16*>(k_pages);
  p.v_pages = static_cast<const __nv_bfloat16*>(v_pages);
  p.block_tables = block_tables, p.lengths = lengths;
  p.step_tile = step_tile, p.step_code = step_code, p.step_count = step_count, p.tile_first = tile_first;
  p.B = B, p.H = H, p.Hkv = Hkv, p.page_size = page_size, p.pages_per_seq = pages_per_seq, p.num_pages = num_pages;
  p.slots = decode_slots(pages_per_seq);
  // Nothing in the scratch has to start at zero: every partial the merge kernel reads was written earlier in
  // this same call, so whatever the previous call left behind is never looked at.
  const size_t rows = static_cast<size_t>(B) * p.slots * H;
  uint8_t* ws = static_cast<uint8_t*>(scratch);
  p.ws_m = reinterpret_cast<float*>(ws);
  p.ws_l = reinterpret_cast<float*>(ws + align256(rows * sizeof(float)));
  p.ws_acc = reinterpret_cast<float*>(ws + 2 * align256(rows * sizeof(float)));
  p.out = static_cast<__nv_bfloat16*>(out);

  const long long capacity = static_cast<long long>(B) * pages_per_seq;
  const int chunks = static_cast<int>((capacity + DEC_CHUNK - 1) / DEC_CHUNK);
  dim3 grid(chunks, (Hkv + DEC_WARPS - 1) / DEC_WARPS);
  switch (group) {
    case 1: decode_chunks_kernel<1><<<grid, DEC_WARPS * 32, 0, s>>>(p); break;
    case 2: decode_chunks_kernel<2><<<grid, DEC_WARPS * 32, 0, s>>>(p); break;
    case 4: decode_chunks_kernel<4><<<grid, DEC_WARPS * 32, 0, s>>>(p); break;
    default: decode_chunks_kernel<8><<<grid, DEC_WARPS * 32, 0, s>>>(p); break;
  }
  TJX_CUDA(cudaGetLastError());
  decode_combine_kernel<<<(B * H * 32 + 255) / 256, 256, 0, s>>>(p);
  TJX_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"

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
constexpr int DEC_SUB = 8;         // tokens a warp handles at a time (a page is a whole number of these)
constexpr int DEC_CHUNK = 8;       // steps (pages) per CTA
constexpr int DEC_WARPS = 4;       // KV heads per CTA
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

// Two f32 in one 64-bit register pair, for the packed FMA of sm_100 (one instruction, two lanes of math).
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// A register holding two bf16 -> the two values as packed f32 (element 0 in the low half).
__device__ __forceinline__ uint64_t bf16x2_to_f32x2(uint32_t u) {
  return pack2(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

constexpr float DEC_LOG2E = 1.4426950408889634f;

// One warp = one KV head and its G query heads over the chunk's steps. Lane = (half, dl): `half` picks one of
// the two tokens a warp-wide 16-byte load covers, dl (0..15) the 8 head dimensions 8 dl .. 8 dl + 7.
//
// Scores: each lane forms its 8-dimension partial dot product for the G heads with packed FMAs, then the 16
// lanes of a half-warp sum them with a transposing butterfly: at each of the first log2(G) exchange stages a
// lane keeps half of its values and hands the other half to its partner, so after the four stages every lane
// holds the complete score of ONE head (`hsel`, from dl's high bits) for its token. The softmax then runs once
// per (head, token) quartet of lanes instead of on every lane, and the probabilities travel back to all lanes
// by shuffle for the P V accumulation.
template <int G>
__global__ void __launch_bounds__(DEC_WARPS * 32, G <= 4 ? 4 : 1) decode_chunks_kernel(const DecodeParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.y * DEC_WARPS + warp;
  if (kvh >= p.Hkv) return;
  const int n_steps = p.step_count[0];
  const int chunk = blockIdx.x;
  const int s_begin = chunk * DEC_CHUNK;
  if (s_begin >= n_steps) return;
  const int n_here = min(DEC_CHUNK, n_steps - s_begin);

  const int half = lane >> 4;
  const int dl = lane & 15;
  const int d0 = dl * 8;
  const size_t row_elems = static_cast<size_t>(p.Hkv) * DEC_D;
  constexpr int LOG_G = G == 1 ? 0 : G == 2 ? 1 : G == 4 ? 2 : 3;
  // The head whose score this lane ends up with, and the lane (within this half-warp's 16) holding head h's.
  const int hsel = LOG_G == 0 ? 0 : (dl >> (4 - LOG_G));
  auto lane_of_head = [&](int h) { return (lane & ~(((1 << LOG_G) - 1) << (4 - LOG_G)) & 31) | (h << (4 - LOG_G)); };

  // The chunk's steps, one per lane (lanes 0..n_here-1), broadcast by shuffle when needed.
  int my_tile = -1, my_code = 4, my_page = 0, my_len = 0;
  if (lane < n_here) {
    my_tile = p.step_tile[s_begin + lane];
    my_code = p.step_code[s_begin + lane];
    my_len = p.lengths[my_tile];
    if (!(my_code & 4)) {
      const int pg = my_code >> 3;
      my_page = p.block_tables[static_cast<size_t>(my_tile) * p.pages_per_seq + pg];
      my_page = min(max(my_page, 0), p.num_pages - 1);
    }
  }

  uint64_t q2[G][4];    // this lane's 8 dimensions of each query head, packed in pairs
  uint64_t acc2[G][4];  // P V accumulator, same layout
  float m_run = DEC_MASK * DEC_LOG2E;  // running max of head `hsel`, log2 units
  float l_run = 0.f;                   // running sum of head `hsel` over this half's tokens
  int cur = -1;

  auto flush = [&]() {
    if (cur < 0) return;
    const int slot = chunk - p.tile_first[cur] / DEC_CHUNK;
    const size_t base = (static_cast<size_t>(cur) * p.slots + slot) * p.H + kvh * G;
    const float l_all = l_run + __shfl_xor_sync(0xFFFFFFFFu, l_run, 16);
#pragma unroll
    for (int h = 0; h < G; ++h) {
      float a[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float lo, hi;
        unpack2(acc2[h][j], lo, hi);
        a[2 * j] = lo + __shfl_xor_sync(0xFFFFFFFFu, lo, 16);
        a[2 * j + 1] = hi + __shfl_xor_sync(0xFFFFFFFFu, hi, 16);
      }
      if (half == 0) {
        float4* dst = reinterpret_cast<float4*>(p.ws_acc + (base + h) * DEC_D + d0);
        dst[0] = make_float4(a[0], a[1], a[2], a[3]);
        dst[1] = make_float4(a[4], a[5], a[6], a[7]);
      }
    }
    // The lane holding head hsel (the first of its quartet, token half 0) writes that head's statistics; the
    // partials keep the max in natural-log units, as the merge kernel expects.
    if (half == 0 && (dl & ((16 >> LOG_G) - 1)) == 0) {
      p.ws_m[base + hsel] = m_run * (1.0f / DEC_LOG2E);
      p.ws_l[base + hsel] = l_all;
    }
  };

  // Micro-steps: (step, 16-token sub-block of its page), visited in order; K of the next micro-step is
  // prefetched while the current one is being computed.
  uint4 kr[DEC_SUB / 2], vr[DEC_SUB / 2];
  auto addr_of = [&](int step, int sub) {
    const int page = __shfl_sync(0xFFFFFFFFu, my_page, step);
    return (static_cast<size_t>(page) * p.page_size + sub + half) * row_elems + kvh * DEC_D + d0;
  };
  auto load_k = [&](int step, int sub) {
    const __nv_bfloat16* kp = p.k_pages + addr_of(step, sub);
#pragma unroll
    for (int i = 0; i < DEC_SUB / 2; ++i) kr[i] = ld_nc_16(kp + static_cast<size_t>(2 * i) * row_elems);
  };
  auto load_v = [&](int step, int sub) {
    const __nv_bfloat16* vp = p.v_pages + addr_of(step, sub);
#pragma unroll
    for (int i = 0; i < DEC_SUB / 2; ++i) vr[i] = ld_nc_16(vp + static_cast<size_t>(2 * i) * row_elems);
  };
  // The next micro-step that has data after (step, sub), or step == n_here if none.
  auto next_data = [&](int step, int sub, int& nstep, int& nsub) {
    nstep = step, nsub = sub + DEC_SUB;
    for (;;) {
      if (nstep >= n_here) return;
      const int code = __shfl_sync(0xFFFFFFFFu, my_code, nstep);
      const int len = __shfl_sync(0xFFFFFFFFu, my_len, nstep);
      if (!(code & 4) && nsub < p.page_size && (code >> 3) * p.page_size + nsub < len) return;
      ++nstep, nsub = 0;
      if (nstep < n_here) {
        const int c2 = __shfl_sync(0xFFFFFFFFu, my_code, nstep);
        if (!(c2 & 4)) return;  // sub 0 of a non-empty step always holds a valid position
      }
    }
  };

  // Prefetch K of the first micro-step with data.
  int pf_step = 0, pf_sub = 0;
  {
    const int c0 = __shfl_sync(0xFFFFFFFFu, my_code, 0);
    if (c0 & 4) next_data(0, p.page_size, pf_step, pf_sub);  // skip an empty first step
    if (pf_step < n_here) load_k(pf_step, pf_sub);
  }

  for (int step = 0; step < n_here; ++step) {
    const int t = __shfl_sync(0xFFFFFFFFu, my_tile, step);
    const int code = __shfl_sync(0xFFFFFFFFu, my_code, step);
    const int len = __shfl_sync(0xFFFFFFFFu, my_len, step);
    if (t != cur) {
      flush();
      cur = t;
      const __nv_bfloat16* qp = p.q + (static_cast<size_t>(t) * p.H + kvh * G) * DEC_D + d0;
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const uint4 u = *reinterpret_cast<const uint4*>(qp + h * DEC_D);
        q2[h][0] = bf16x2_to_f32x2(u.x), q2[h][1] = bf16x2_to_f32x2(u.y);
        q2[h][2] = bf16x2_to_f32x2(u.z), q2[h][3] = bf16x2_to_f32x2(u.w);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc2[h][j] = 0ull;
      }
      m_run = DEC_MASK * DEC_LOG2E, l_run = 0.f;
    }
    if (code & 4) continue;  // an empty step: no position to read
    const int pg = code >> 3;
    for (int sub = 0; sub < p.page_size; sub += DEC_SUB) {
      const int base_pos = pg * p.page_size + sub;
      if (base_pos >= len) break;
      // K of this micro-step is in flight (prefetched); start V.
      load_v(step, sub);

      // Partial dot products over this lane's 8 dimensions, then the transposing butterfly.
      float sc[DEC_SUB / 2];
#pragma unroll
      for (int i = 0; i < DEC_SUB / 2; ++i) {
        const uint64_t k0 = bf16x2_to_f32x2(kr[i].x), k1 = bf16x2_to_f32x2(kr[i].y);
        const uint64_t k2 = bf16x2_to_f32x2(kr[i].z), k3 = bf16x2_to_f32x2(kr[i].w);
        float r[G];
#pragma unroll
        for (int h = 0; h < G; ++h) {
          uint64_t a = mul2(q2[h][0], k0);
          a = fma2(q2[h][1], k1, a), a = fma2(q2[h][2], k2, a), a = fma2(q2[h][3], k3, a);
          float lo, hi;
          unpack2(a, lo, hi);
          r[h] = lo + hi;
        }
        int n = G;
#pragma unroll
        for (int mask = 8; mask >= 1; mask >>= 1) {
          if (n > 1) {
            n >>= 1;
            const bool up = (dl & mask) != 0;
#pragma unroll
            for (int j = 0; j < n; ++j) {
              const float keep = up ? r[j + n] : r[j];
              const float send = up ? r[j] : r[j + n];
              r[j] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, mask);
            }
          } else {
            r[0] += __shfl_xor_sync(0xFFFFFFFFu, r[0], mask);
          }
        }
        const int pos = base_pos + 2 * i + half;
        sc[i] = pos < len ? r[0] * DEC_LOG2E : DEC_MASK * DEC_LOG2E;
      }

      // K registers are free: prefetch the next micro-step's K.
      next_data(step, sub, pf_step, pf_sub);
      if (pf_step < n_here) load_k(pf_step, pf_sub);

      // Online softmax of head hsel over this sub-block (both token halves).
      float mx = sc[0];
#pragma unroll
      for (int i = 1; i < DEC_SUB / 2; ++i) mx = fmaxf(mx, sc[i]);
      mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 16));
      const float m_new = fmaxf(m_run, mx);
      const float alpha = ex2(m_run - m_new);
      m_run = m_new;
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < DEC_SUB / 2; ++i) {
        const float pr = ex2(sc[i] - m_new);
        sum += pr;
        sc[i] = __bfloat162float(__float2bfloat16_rn(pr));  // P is rounded before it multiplies V
      }
      l_run = l_run * alpha + sum;
      // Every lane rescales its accumulators of all heads.
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const float a = __shfl_sync(0xFFFFFFFFu, alpha, lane_of_head(h));
        const uint64_t a2 = pack2(a, a);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc2[h][j] = mul2(acc2[h][j], a2);
      }
      // P V: each lane needs the probability of every head for its own token.
#pragma unroll
      for (int i = 0; i < DEC_SUB / 2; ++i) {
        const uint64_t v0 = bf16x2_to_f32x2(vr[i].x), v1 = bf16x2_to_f32x2(vr[i].y);
        const uint64_t v2 = bf16x2_to_f32x2(vr[i].z), v3 = bf16x2_to_f32x2(vr[i].w);
#pragma unroll
        for (int h = 0; h < G; ++h) {
          const float pr = __shfl_sync(0xFFFFFFFFu, sc[i], lane_of_head(h));
          const uint64_t p2 = pack2(pr, pr);
          acc2[h][0] = fma2(p2, v0, acc2[h][0]), acc2[h][1] = fma2(p2, v1, acc2[h][1]);
          acc2[h][2] = fma2(p2, v2, acc2[h][2]), acc2[h][3] = fma2(p2, v3, acc2[h][3]);
        }
      }
    }
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
  if (page_size <= 0 || page_size % 16 != 0) return fail(TJX_E_ARG, "page size must be a multiple of 16");
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
  if (page_size <= 0 || page_size % 16 != 0) return fail(TJX_E_ARG, "page size must be a multiple of 16");
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

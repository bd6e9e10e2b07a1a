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

#include <algorithm>
#include <mutex>
#include <string>

#include "../../include/tilejax_b200.h"

namespace tjx {

int launch_build_steps_lengths(const int32_t* lengths, int n_lengths, const int32_t* tile_values, int tiles,
                               int blocks, int value0, int value_step, int32_t* step_tile, int32_t* step_code,
                               int32_t* step_count, int32_t* tile_first, cudaStream_t stream);

constexpr int DEC_D = 128;         // head dimension
constexpr int DEC_SUB = 8;         // tokens per micro-step (a page is a whole number of these)
constexpr int DEC_STAGES = 2;      // ring slots per warp
constexpr int DEC_STAGE_BYTES = DEC_SUB * DEC_D * 2 * 2;  // K and V of one micro-step for one KV head
constexpr int DEC_CHUNK = 16;      // steps (pages) per CTA
constexpr int DEC_WARPS = 4;       // KV heads per CTA
constexpr float DEC_MASK = -1e30f;
// Shared memory per warp: the K/V ring, the partial-score scratch [4 pairs][G][32], P [8][G] and G rescale factors.
__host__ __device__ constexpr int dec_warp_bytes(int g) {
  return (DEC_STAGES * DEC_STAGE_BYTES + 4 * g * 32 * 4 + 8 * g * 4 + 8 * 4 + 127) / 128 * 128;  // TMA wants 128-byte slots
}

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
  int* status;
};


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
// the two tokens a 512-byte row pair holds, dl (0..15) the 8 head dimensions 8 dl .. 8 dl + 7.
//
// Data path: the warp owns a ring of DEC_STAGES shared-memory slots; lane 0 issues two TMA tile loads per
// micro-step (8 tokens of K and of V for this KV head: a [8 tokens x 1 head x 128 dims] box of the 3-D view
// [tokens, heads, dims] of the page pool, 2 KB each) one micro-step ahead, completing on the slot's mbarrier;
// the lanes then read their 16 bytes per token with conflict-free LDS.128.
//
// Scores: each lane forms its 8-dimension partial dot products for the G heads with packed FMAs and stores them
// to a per-warp scratch laid out [token pair][head][half][dl], one bank per lane. After the 4 token pairs, lane
// (h, tok) = (lane / 8, lane % 8) sums the 16 partials of ITS (head, token) — four LDS.128 and 15 adds replace a
// 16-step shuffle butterfly per token pair — so every lane owns one score (two for G = 8) and the softmax does no
// redundant work. Probabilities and rescale factors go back through shared memory ([token][head], one LDS.128
// per token) for the P V accumulation, again with packed FMAs.
template <int G>
__global__ void __launch_bounds__(DEC_WARPS * 32, G <= 4 ? 4 : 2)
    decode_chunks_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         const DecodeParams p) {
  extern __shared__ __align__(128) uint8_t dec_smem[];
  __shared__ __align__(8) uint64_t dec_bars[DEC_WARPS * DEC_STAGES];
  __shared__ int dec_abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.y * DEC_WARPS + warp;
  const int n_steps = p.step_count[0];
  if (threadIdx.x == 0) {
    for (int i = 0; i < DEC_WARPS * DEC_STAGES; ++i) mbar_init(smem_u32(&dec_bars[i]), 1);
    dec_abort = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (kvh >= p.Hkv) return;

  const int half = lane >> 4;
  const int dl = lane & 15;
  const int d0 = dl * 8;
  constexpr int IT = DEC_SUB / 2;           // token pairs per micro-step
  constexpr int NSC = G > 4 ? G / 4 : 1;    // scores a lane owns per micro-step
  // The (head, token) this lane owns: head lane / 8 (+ 4 j), token lane % 8; lanes beyond G heads own nothing.
  const int own_tok = lane & 7;
  const int own_h = lane >> 3;

  uint8_t* warp_smem = dec_smem + warp * dec_warp_bytes(G);
  const uint32_t ring = smem_u32(warp_smem);
  float* pb = reinterpret_cast<float*>(warp_smem + DEC_STAGES * DEC_STAGE_BYTES);  // [IT][G][32] partials
  float* pbuf = pb + IT * G * 32;                                                   // [8 tokens][G] P
  float* abuf = pbuf + 8 * G;                                                       // [G] rescale factors
  auto bar = [&](int stage) { return smem_u32(&dec_bars[warp * DEC_STAGES + stage]); };

  int n = 0;  // micro-steps consumed by this warp so far (ring position and barrier phase)
  bool ok = true;
  // A persistent CTA: chunks blockIdx.x, blockIdx.x + gridDim.x, ... of the steps that run.
  for (int chunk = blockIdx.x; chunk * DEC_CHUNK < n_steps && ok; chunk += gridDim.x) {
  const int s_begin = chunk * DEC_CHUNK;
  const int n_here = min(DEC_CHUNK, n_steps - s_begin);

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
  float m_run[NSC], l_run[NSC];  // running max (log2 units; same in the 8 lanes of a head) and this lane's sum
  int cur = -1;

  auto flush = [&]() {
    if (cur < 0) return;
    const int slot = chunk - p.tile_first[cur] / DEC_CHUNK;
    const size_t base = (static_cast<size_t>(cur) * p.slots + slot) * p.H + kvh * G;
#pragma unroll
    for (int j = 0; j < NSC; ++j) {
      float l_all = l_run[j];
      l_all += __shfl_xor_sync(0xFFFFFFFFu, l_all, 1);
      l_all += __shfl_xor_sync(0xFFFFFFFFu, l_all, 2);
      l_all += __shfl_xor_sync(0xFFFFFFFFu, l_all, 4);
      const int h = own_h + 4 * j;
      if (own_tok == 0 && h < G) {  // the partials keep the max in natural-log units
        p.ws_m[base + h] = m_run[j] * (1.0f / DEC_LOG2E);
        p.ws_l[base + h] = l_all;
      }
    }
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
  };

  // The next micro-step (step, 8-token sub-block) that has data after (step, sub); step == n_here if none.
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
  // Start the loads of micro-step number n (the n-th with data) into its ring slot.
  auto issue = [&](int n, int step, int sub) {
    const int page = __shfl_sync(0xFFFFFFFFu, my_page, step);
    if (lane == 0) {
      const int stage = n % DEC_STAGES;
      const uint32_t dst = ring + stage * DEC_STAGE_BYTES;
      const int token = page * p.page_size + sub;
      mbar_expect_tx(bar(stage), DEC_STAGE_BYTES);
      tma_load_3d(dst, &map_k, 0, kvh, token, bar(stage));
      tma_load_3d(dst + DEC_STAGE_BYTES / 2, &map_v, 0, kvh, token, bar(stage));
    }
  };

  // Prologue: the first DEC_STAGES - 1 micro-steps.
  int pf_step = 0, pf_sub = 0, pf_n = n;
  {
    const int c0 = __shfl_sync(0xFFFFFFFFu, my_code, 0);
    if (c0 & 4) next_data(0, p.page_size, pf_step, pf_sub);  // skip an empty first step
    for (int i = 0; i < DEC_STAGES - 1 && pf_step < n_here; ++i) {
      issue(pf_n++, pf_step, pf_sub);
      next_data(pf_step, pf_sub, pf_step, pf_sub);
    }
  }

  for (int step = 0; step < n_here && ok; ++step) {
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
#pragma unroll
      for (int j = 0; j < NSC; ++j) m_run[j] = DEC_MASK * DEC_LOG2E, l_run[j] = 0.f;
    }
    if (code & 4) continue;  // an empty step: no position to read
    const int pg = code >> 3;
    for (int sub = 0; sub < p.page_size; sub += DEC_SUB) {
      const int base_pos = pg * p.page_size + sub;
      if (base_pos >= len) break;
      // Keep the ring full: the slot freed by the previous micro-step takes the one DEC_STAGES - 1 ahead.
      if (pf_step < n_here) {
        issue(pf_n++, pf_step, pf_sub);
        next_data(pf_step, pf_sub, pf_step, pf_sub);
      }
      const int stage = n % DEC_STAGES;
      const bool got = mbar_wait(bar(stage), (n / DEC_STAGES) & 1, &dec_abort, p.status, TJX_ERR_WAIT_FULL);
      if (!__all_sync(0xFFFFFFFFu, got)) {
        ok = false;
        break;
      }
      ++n;
      const uint8_t* kbuf = warp_smem + stage * DEC_STAGE_BYTES + lane * 16;
      const uint8_t* vbuf = kbuf + DEC_STAGE_BYTES / 2;

      // Partial dot products over this lane's 8 dimensions -> scratch [pair][head][lane].
#pragma unroll
      for (int i = 0; i < IT; ++i) {
        const uint4 kk = *reinterpret_cast<const uint4*>(kbuf + i * 512);
        const uint64_t k0 = bf16x2_to_f32x2(kk.x), k1 = bf16x2_to_f32x2(kk.y);
        const uint64_t k2 = bf16x2_to_f32x2(kk.z), k3 = bf16x2_to_f32x2(kk.w);
#pragma unroll
        for (int h = 0; h < G; ++h) {
          uint64_t a = mul2(q2[h][0], k0);
          a = fma2(q2[h][1], k1, a), a = fma2(q2[h][2], k2, a), a = fma2(q2[h][3], k3, a);
          float lo, hi;
          unpack2(a, lo, hi);
          pb[(i * G + h) * 32 + lane] = lo + hi;
        }
      }
      __syncwarp();

      // This lane's score(s): the 16 partials of (head own_h + 4 j, token own_tok), then the online softmax of
      // that head over the sub-block's 8 tokens (the 8 lanes of a head).
      bool grew = false;
#pragma unroll
      for (int j = 0; j < NSC; ++j) {
        const int h = own_h + 4 * j;
        float score = DEC_MASK * DEC_LOG2E;
        if (h < G) {
          // The 32 lanes read 32 different 64-byte runs that all start on bank 0 or 16: each lane starts at a
          // different 16-byte unit of its run, so that one LDS.128 spreads over all banks.
          const float4* src = reinterpret_cast<const float4*>(pb + ((own_tok >> 1) * G + h) * 32 + (own_tok & 1) * 16);
          const int rot = (h + (own_tok >> 1)) & 3;
          const float4 a = src[rot], b = src[(rot + 1) & 3], c = src[(rot + 2) & 3], d = src[(rot + 3) & 3];
          const float sum = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w)) +
                            (((c.x + c.y) + (c.z + c.w)) + ((d.x + d.y) + (d.z + d.w)));
          if (base_pos + own_tok < len) score = sum * DEC_LOG2E;
        }
        float mx = score;
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 4));
        grew |= mx > m_run[j];
        const float m_new = fmaxf(m_run[j], mx);
        const float alpha = ex2(m_run[j] - m_new);
        m_run[j] = m_new;
        const float pr = ex2(score - m_new);
        l_run[j] = l_run[j] * alpha + pr;
        if (h < G) {
          pbuf[own_tok * G + h] = __bfloat162float(__float2bfloat16_rn(pr));  // P is rounded before P V
          if (own_tok == 0) abuf[h] = alpha;
        }
      }
      const bool rescale = __any_sync(0xFFFFFFFFu, grew);
      __syncwarp();

      if (rescale) {
#pragma unroll
        for (int h = 0; h < G; ++h) {
          const float a = abuf[h];
          const uint64_t a2 = pack2(a, a);
#pragma unroll
          for (int j = 0; j < 4; ++j) acc2[h][j] = mul2(acc2[h][j], a2);
        }
      }
      // P V: each lane reads the probabilities of every head for its own token.
#pragma unroll
      for (int i = 0; i < IT; ++i) {
        const uint4 vv = *reinterpret_cast<const uint4*>(vbuf + i * 512);
        const uint64_t v0 = bf16x2_to_f32x2(vv.x), v1 = bf16x2_to_f32x2(vv.y);
        const uint64_t v2 = bf16x2_to_f32x2(vv.z), v3 = bf16x2_to_f32x2(vv.w);
        float prs[G];
        if constexpr (G >= 4) {
#pragma unroll
          for (int h4 = 0; h4 < G / 4; ++h4) {
            const float4 t4 = reinterpret_cast<const float4*>(pbuf + (2 * i + half) * G)[h4];
            prs[4 * h4] = t4.x, prs[4 * h4 + 1] = t4.y, prs[4 * h4 + 2] = t4.z, prs[4 * h4 + 3] = t4.w;
          }
        } else {
#pragma unroll
          for (int h = 0; h < G; ++h) prs[h] = pbuf[(2 * i + half) * G + h];
        }
#pragma unroll
        for (int h = 0; h < G; ++h) {
          const float pr = prs[h];
          const uint64_t p2 = pack2(pr, pr);
          acc2[h][0] = fma2(p2, v0, acc2[h][0]), acc2[h][1] = fma2(p2, v1, acc2[h][1]);
          acc2[h][2] = fma2(p2, v2, acc2[h][2]), acc2[h][3] = fma2(p2, v3, acc2[h][3]);
        }
      }
      __syncwarp();  // every lane is done with the slot and the scratch before they are refilled
    }
  }
  if (ok) flush();
  }  // chunks
}

// Merge a sequence's partials: one warp per (sequence, query head), a lane per 4 head dimensions.
__global__ void __launch_bounds__(256) decode_combine_kernel(const DecodeParams p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= p.B * p.H) return;
  const int b = warp / p.H, h = warp - b * p.H;
  const int first = p.tile_first[b], next = p.tile_first[b + 1];
  const int n = (next - 1) / DEC_CHUNK - first / DEC_CHUNK + 1;  // a tile takes at least one step
  const size_t base = static_cast<size_t>(b) * p.slots * p.H + h;
  // Lane i holds partial i's statistics (32 at a time), so the maxima and weights come from a few parallel loads
  // and the accumulator rows stream in independent, unrolled loads.
  float mx = DEC_MASK;
  for (int i0 = 0; i0 < n; i0 += 32)
    if (i0 + lane < n) mx = fmaxf(mx, p.ws_m[base + static_cast<size_t>(i0 + lane) * p.H]);
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, d));
  float lsum = 0.f;
  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i0 = 0; i0 < n; i0 += 32) {
    float w_mine = 0.f;
    if (i0 + lane < n) {
      const size_t idx = base + static_cast<size_t>(i0 + lane) * p.H;
      w_mine = __expf(p.ws_m[idx] - mx);
      lsum += w_mine * p.ws_l[idx];
    }
    const int cnt = min(32, n - i0);
#pragma unroll 8
    for (int i = 0; i < cnt; ++i) {
      const float w = __shfl_sync(0xFFFFFFFFu, w_mine, i);
      const size_t idx = base + static_cast<size_t>(i0 + i) * p.H;
      const float4 a = *reinterpret_cast<const float4*>(p.ws_acc + idx * DEC_D + lane * 4);
      o.x = fmaf(w, a.x, o.x), o.y = fmaf(w, a.y, o.y), o.z = fmaf(w, a.z, o.z), o.w = fmaf(w, a.w, o.w);
    }
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) lsum += __shfl_xor_sync(0xFFFFFFFFu, lsum, d);
  const float inv = 1.0f / fmaxf(lsum, 1e-30f);
  uint2 r;
  r.x = pack_bf16(o.x * inv, o.y * inv);
  r.y = pack_bf16(o.z * inv, o.w * inv);
  *reinterpret_cast<uint2*>(p.out + (static_cast<size_t>(b) * p.H + h) * DEC_D + lane * 4) = r;
}

template <int G>
static int launch_chunks_for(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeParams& p, dim3 grid,
                             cudaStream_t s) {
  constexpr int SMEM = DEC_WARPS * dec_warp_bytes(G);
  auto kernel = decode_chunks_kernel<G>;
  static bool configured[64] = {};
  int dev = 0;
  TJX_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    TJX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured[dev & 63] = true;
  }
  kernel<<<grid, DEC_WARPS * 32, SMEM, s>>>(mk, mv, p);
  TJX_CUDA(cudaGetLastError());
  return 0;
}

// The page pools as 3-D tensors [token, KV head, dim] for TMA (box: 8 tokens x 1 head x 128 dims), then the
// chunk kernel for this group size. Allocates nothing.
static int launch_decode_chunks(DecodeParams& p, int group, cudaStream_t s) {
  p.status = device_status_word();
  if (p.status == nullptr) return fail(TJX_E_CUDA, "could not locate the device status word");
  const uint64_t dims[3] = {DEC_D, static_cast<uint64_t>(p.Hkv),
                            static_cast<uint64_t>(p.num_pages) * static_cast<uint64_t>(p.page_size)};
  const uint64_t strides[2] = {DEC_D * 2, static_cast<uint64_t>(p.Hkv) * DEC_D * 2};
  const uint32_t box[3] = {DEC_D, 1, DEC_SUB};
  CUtensorMap mk, mv;
  if (int rc = make_tensor_map(&mk, p.k_pages, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 3, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  if (int rc = make_tensor_map(&mv, p.v_pages, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 3, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_NONE))
    return rc;
  const long long capacity = static_cast<long long>(p.B) * p.pages_per_seq;
  const int chunks = static_cast<int>((capacity + DEC_CHUNK - 1) / DEC_CHUNK);
  const int groups = (p.Hkv + DEC_WARPS - 1) / DEC_WARPS;
  // One CTA per possible chunk: the hardware scheduler balances the ones that have work (a CTA past the end of
  // the steps that run exits at once). The kernel also accepts a smaller grid and then loops over chunks.
  dim3 grid(chunks, groups);
  switch (group) {
    case 1: return launch_chunks_for<1>(mk, mv, p, grid, s);
    case 2: return launch_chunks_for<2>(mk, mv, p, grid, s);
    case 4: return launch_chunks_for<4>(mk, mv, p, grid, s);
    default: return launch_chunks_for<8>(mk, mv, p, grid, s);
  }
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

  if (int rc = launch_decode_chunks(p, group, s)) return rc;
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

  if (int rc = launch_decode_chunks(p, group, s)) return rc;
  decode_combine_kernel<<<(B * H * 32 + 255) / 256, 256, 0, s>>>(p);
  TJX_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"

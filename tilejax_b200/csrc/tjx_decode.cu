// Ragged paged GQA decode attention on sm_100a, bound by HBM bandwidth: every valid K/V page is read once,
// by TMA straight into shared memory, and multiplied with warp-level MMAs (mma.sync m16n8k16, bf16 -> f32) whose
// 16 rows are the query heads of one KV head; the fifth-generation tensor core needs 64 or 128 rows and would
// compute mostly padding here.
//
// The work is the list of steps that run, one K/V page each, in tile (sequence) order — the same list the device
// step table (tjx_steps.cu) holds. For up to DEC_SELF_MAX_B (2048) sequences every CTA derives the list itself from
// `lengths` (a prefix sum in its prologue), so the kernel does not wait for the step-table kernel that runs
// beside it and only emits the tables for the caller; larger batches read the tables.
//
// The list is shared out evenly: as many CTAs as are resident at once (4 per SM) per pair of KV heads, each taking
// one contiguous share of the steps (at least DEC_CHUNK), so ragged lengths balance to within a step and a sequence
// is cut into as few pieces as possible. Inside a CTA warp w owns one KV head and its G query heads. A share may
// cover the end of one sequence and the start of the next; a (sequence, share) piece that is the sequence's only
// one is normalised and written at once; otherwise it writes an online-softmax partial (max, sum, accumulator) to
// scratch and counts itself on the sequence's arrival counter, and the warp that arrives last merges the
// sequence's partials, normalises and writes bf16 — no second kernel.
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

int check_step_table_sizes(int tiles, int blocks);
int launch_build_steps_lengths(const int32_t* lengths, int n_lengths, const int32_t* tile_values, int tiles,
                               int blocks, int value0, int value_step, int32_t* step_tile, int32_t* step_code,
                               int32_t* step_count, int32_t* tile_first, int32_t* zero_words, int n_zero,
                               cudaStream_t stream);

constexpr int DEC_D = 128;         // head dimension
constexpr int DEC_SUB = 16;        // tokens per micro-step (a page is a whole number of these)
#ifndef TJX_DEC_STAGES
#define TJX_DEC_STAGES 2
#endif
#ifndef TJX_DEC_WARPS
#define TJX_DEC_WARPS 2
#endif
#ifndef TJX_DEC_CTAS
#define TJX_DEC_CTAS 4  // resident CTAs per SM: 8 warps per SM measured fastest (12: +5 %, 6: +8 %, 4: +40 % time)
#endif
#ifndef TJX_DEC_CHUNK
#define TJX_DEC_CHUNK 12
#endif
constexpr int DEC_STAGES = TJX_DEC_STAGES;  // ring slots per warp
constexpr int DEC_HALF_BYTES = DEC_SUB * 64 * 2;           // one TMA box: 16 tokens x 64 dims, 128-byte rows
constexpr int DEC_STAGE_BYTES = 4 * DEC_HALF_BYTES;        // K (two dim halves) and V (two) of one micro-step
constexpr int DEC_CHUNK = TJX_DEC_CHUNK;  // steps (pages) per CTA (at most 32: a lane holds a step)
constexpr int DEC_WARPS = TJX_DEC_WARPS;  // KV heads per CTA
constexpr float DEC_MASK = -1e30f;
constexpr int DEC_SMEM = DEC_WARPS * DEC_STAGES * DEC_STAGE_BYTES + 1024;  // + slack to align the ring to 1024
// Up to this many sequences a CTA computes every sequence's first step itself (B + 1 ints of shared memory behind
// the ring); beyond it the kernel reads the tables the step-table kernel built.
constexpr int DEC_SELF_MAX_B = 2048;

struct DecodeParams {
  const __nv_bfloat16* q;        // [B, T, H, D]
  const __nv_bfloat16* k_pages;  // [num_pages, PAGE, Hkv * D]
  const __nv_bfloat16* v_pages;
  const int32_t* block_tables;   // [B, pages_per_seq]
  const int32_t* lengths;        // [B]
  const int32_t* step_tile;
  const int32_t* step_code;
  const int32_t* step_count;
  const int32_t* tile_first;     // [B + 1]
  float* ws_m;                   // [B, slots, rows]
  float* ws_l;                   // [B, slots, rows]
  float* ws_acc;                 // [B, slots, rows, D]
  int* arrivals;                 // [B, Hkv] pieces of a sequence's KV head that have written their partial
  __nv_bfloat16* out;            // [B, T, H, D]
  int B, H, Hkv, page_size, pages_per_seq, num_pages, slots;
  int T, rows;                   // new tokens per sequence; query rows per sequence = T * H (row t * H + h)
  int self_steps;                // != 0: derive the steps from `lengths` in the prologue instead of reading the tables
  float score_scale;             // scores are multiplied by this before the base-2 exponential: log2(e), times the
                                 // softmax scale when the queries do not arrive pre-scaled (ragged paged attention)
  long long kv_head_stride, kv_token_stride;  // elements between KV heads / tokens in the page pools (0: packed)
  int min_share;                 // steps a CTA takes at least (what bounds the partials a sequence can have)
  int* status;
  long long* profile;            // per-CTA counters (PROFILE_WORDS each) or null
};


constexpr float DEC_LOG2E = 1.4426950408889634f;

// Merge the partials of the G query heads h0 .. h0 + G - 1 of sequence b (n partials each, in slots 0..n-1),
// normalise and write bf16. One warp; a lane holds 4 head dimensions of every head, and the G heads go through
// the loop together so that G times as many loads are in flight. The partials were written by other CTAs: they
// are read past L1.
template <int G>
__device__ __forceinline__ void decode_merge_heads(const DecodeParams& p, int b, int h0, int n, int lane) {
  const size_t base = static_cast<size_t>(b) * p.slots * p.rows + h0;
  float mx[G], lsum[G];
  float4 o[G];
#pragma unroll
  for (int h = 0; h < G; ++h) mx[h] = DEC_MASK, lsum[h] = 0.f, o[h] = make_float4(0.f, 0.f, 0.f, 0.f);
  // Lane i holds partial i's statistics (32 at a time).
  for (int i0 = 0; i0 < n; i0 += 32)
    if (i0 + lane < n) {
#pragma unroll
      for (int h = 0; h < G; ++h)
        mx[h] = fmaxf(mx[h], __ldcg(p.ws_m + base + static_cast<size_t>(i0 + lane) * p.rows + h));
    }
#pragma unroll
  for (int h = 0; h < G; ++h)
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xFFFFFFFFu, mx[h], d));
  for (int i0 = 0; i0 < n; i0 += 32) {
    float w_mine[G];
#pragma unroll
    for (int h = 0; h < G; ++h) w_mine[h] = 0.f;
    if (i0 + lane < n) {
      const size_t idx = base + static_cast<size_t>(i0 + lane) * p.rows;
#pragma unroll
      for (int h = 0; h < G; ++h) {
        w_mine[h] = __expf(__ldcg(p.ws_m + idx + h) - mx[h]);
        lsum[h] += w_mine[h] * __ldcg(p.ws_l + idx + h);
      }
    }
    const int cnt = min(32, n - i0);
#pragma unroll 4
    for (int i = 0; i < cnt; ++i) {
      const size_t idx = base + static_cast<size_t>(i0 + i) * p.rows;
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const float w = __shfl_sync(0xFFFFFFFFu, w_mine[h], i);
        const float4 a = __ldcg(reinterpret_cast<const float4*>(p.ws_acc + (idx + h) * DEC_D + lane * 4));
        o[h].x = fmaf(w, a.x, o[h].x), o[h].y = fmaf(w, a.y, o[h].y);
        o[h].z = fmaf(w, a.z, o[h].z), o[h].w = fmaf(w, a.w, o[h].w);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < G; ++h) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) lsum[h] += __shfl_xor_sync(0xFFFFFFFFu, lsum[h], d);
    const float inv = 1.0f / fmaxf(lsum[h], 1e-30f);
    uint2 r;
    r.x = pack_bf16(o[h].x * inv, o[h].y * inv);
    r.y = pack_bf16(o[h].z * inv, o[h].w * inv);
    *reinterpret_cast<uint2*>(p.out + (static_cast<size_t>(b) * p.rows + h0 + h) * DEC_D + lane * 4) = r;
  }
}

// One warp = one KV head and its G query heads over the chunk's steps, 16 tokens (a micro-step) at a time.
//
// Data path: the warp owns a ring of DEC_STAGES shared-memory slots; lane 0 issues four TMA tile loads per
// micro-step — K and V of 16 tokens of this KV head, each as two boxes [16 tokens x 1 head x 64 dims] of the 3-D
// view [tokens, heads, dims] of the page pool, 128-byte swizzled — one micro-step ahead, completing on the slot's
// mbarrier. The page bytes never pass through registers on their way in.
//
// Arithmetic: warp-level mma.sync (m16n8k16, bf16 x bf16 -> f32). The 16 rows of the A operand are the query
// heads (G of them, the rest zero), so S = Q K^T for 16 tokens is 2 x 8 MMAs whose B fragments come straight from
// the K slot with ldmatrix, the probabilities — rounded to bf16, as the reference rounds them — are already in A
// fragment layout when they leave the softmax (no shared-memory round trip), and O += P V is 16 MMAs with B
// fragments from the V slot with ldmatrix.trans. Lane (g, t) = (lane / 4, lane % 4) holds of head g: scores of
// tokens 2t, 2t+1, 8+2t, 9+2t and output dims 8 n + 2t, + 1 for n = 0..15. A fifth-generation (tcgen05) MMA needs
// 64 or 128 rows; with at most 8 query heads per KV head this path stays bound by HBM with the warp-level MMA.
template <int G, bool WIDE>
__global__ void __launch_bounds__(DEC_WARPS * 32, WIDE ? (TJX_DEC_CTAS * 2 / 3) : TJX_DEC_CTAS)
    decode_chunks_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                         const DecodeParams p) {
  extern __shared__ uint8_t dec_smem_raw[];
  __shared__ __align__(8) uint64_t dec_bars[DEC_WARPS * DEC_STAGES];
  __shared__ int dec_abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.y * DEC_WARPS + warp;
  long long* prof = p.profile == nullptr ? nullptr
                        : p.profile + (static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * PROFILE_WORDS;
  long long in_wait = 0, fill_wait = -1, t_first = 0;
  if (prof != nullptr && threadIdx.x == 0) prof[0] = clock64();
  if (threadIdx.x == 0) {
    for (int i = 0; i < DEC_WARPS * DEC_STAGES; ++i) mbar_init(smem_u32(&dec_bars[i]), 1);
    dec_abort = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  // Launched with programmatic stream serialisation: this grid may run beside the step-table kernel before it in
  // the stream. Nothing that kernel writes (the tables, the cleared arrival counters) is touched before a
  // griddepcontrol.wait: at once when the steps come from its tables, else only before the first arrival is
  // counted — the pages, lengths and block tables were complete before that kernel started.
  int* s_first = reinterpret_cast<int*>(dec_smem_raw + DEC_SMEM);  // [B + 1] first step of every sequence (self_steps)
  int n_steps;
  if (p.self_steps) {
    __shared__ int s_part[DEC_WARPS * 32];
    // A sequence takes one step per page that holds a valid position, or one empty step if it has none
    // (src/autokernel/codegen.py:386-431). Thread i sums a contiguous range of sequences, then a scan over threads.
    const int per = (p.B + DEC_WARPS * 32 - 1) / (DEC_WARPS * 32);
    const int lo = min(p.B, static_cast<int>(threadIdx.x) * per), hi = min(p.B, lo + per);
    int sum = 0;
    for (int b = lo; b < hi; ++b) {
      const int len = p.lengths[b];
      const int runs = len > 0 ? min(p.pages_per_seq, (len + p.page_size - 1) / p.page_size) : 0;
      s_first[b] = sum;
      sum += max(runs, 1);
    }
    s_part[threadIdx.x] = sum;
    __syncthreads();
    int before = 0;
    for (int i = 0; i < static_cast<int>(threadIdx.x); ++i) before += s_part[i];
    for (int b = lo; b < hi; ++b) s_first[b] += before;
    if (threadIdx.x == DEC_WARPS * 32 - 1) s_first[p.B] = before + sum;
    __syncthreads();
    n_steps = s_first[p.B];
  } else {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    n_steps = p.step_count[0];
    __syncthreads();
  }
  if (kvh >= p.Hkv) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    return;
  }

  // Query rows of this KV head: row r = (new token r / G, query head r % G of the group), R = T * G of them. A
  // lane holds row g = lane / 4 and, when there are more than 8 rows (WIDE), row g + 8 as well.
  constexpr int NR = WIDE ? 2 : 1;
  const int g = lane >> 2;
  const int t = lane & 3;
  const int R = p.T * G;
  bool row_ok[NR];
  int row_tok[NR], row_head[NR];  // the row's new token, and its index t * H + h among the sequence's query rows
#pragma unroll
  for (int x = 0; x < NR; ++x) {
    const int r = g + 8 * x;
    row_ok[x] = r < R;
    row_tok[x] = r / G;
    row_head[x] = row_tok[x] * p.H + kvh * G + r % G;
  }
  const uint32_t ring = ((smem_u32(dec_smem_raw) + 1023u) & ~1023u) + warp * (DEC_STAGES * DEC_STAGE_BYTES);
  auto bar = [&](int stage) { return smem_u32(&dec_bars[warp * DEC_STAGES + stage]); };
  // ldmatrix addressing. A box is [16 tokens][128 bytes], its 16-byte units XOR-swizzled with token % 8.
  //   K (plain): matrix j of a load = dims 8 j .. 8 j + 7 of 8 tokens: lane i points at token i % 8, unit i / 8.
  //   V (trans): matrices = (tokens 0-7 | 8-15) x (dims n | n + 8): lane i points at token i % 8 + 8 (i / 8 % 2),
  //              unit i / 16.
  const int lrow = lane & 7;
  const uint32_t k_lane = lrow * 128;
  const int k_unit = lane >> 3;
  const uint32_t v_lane = (lrow + 8 * ((lane >> 3) & 1)) * 128;
  const int v_unit = lane >> 4;

  int n = 0;  // micro-steps consumed by this warp so far (ring position and barrier phase)
  bool ok = true;
  // A persistent CTA takes one contiguous share of the steps that run — the same number for every CTA, at least
  // DEC_CHUNK — so ragged lengths balance to within a step and a sequence is cut into as few pieces as possible.
  const int per = max(p.min_share, (n_steps + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x));
  const int r_begin = min(n_steps, static_cast<int>(blockIdx.x) * per), r_end = min(n_steps, r_begin + per);

  uint32_t qa[8][2 * NR];  // A fragments of Q: k-step j = dims 16 j .. + 15; row x: [2x] = dims + 2t, + 1, [2x + 1] = + 8
  float o[16][4];          // O fragments: [n][0..1] = row g, dims 8 n + 2t, + 1; [2..3] = row g + 8 (zero rows unless WIDE)
  float m_run[NR], l_run[NR];  // each row's running max (log2 units) and this lane's part of its sum
#pragma unroll
  for (int x = 0; x < NR; ++x) m_run[x] = DEC_MASK * DEC_LOG2E, l_run[x] = 0.f;
  int cur = -1;

  auto flush = [&]() {
    if (cur < 0) return;
    const int first = p.self_steps ? s_first[cur] : p.tile_first[cur];
    const int next = p.self_steps ? s_first[cur + 1] : p.tile_first[cur + 1];
    const int pieces = (next - 1) / per - first / per + 1;  // shares the sequence's steps fall in (it takes at least one)
    const int slot = static_cast<int>(blockIdx.x) - first / per;
    const size_t base = (static_cast<size_t>(cur) * p.slots + slot) * p.rows;
#pragma unroll
    for (int x = 0; x < NR; ++x) {
      float l_all = l_run[x];
      l_all += __shfl_xor_sync(0xFFFFFFFFu, l_all, 1);
      l_all += __shfl_xor_sync(0xFFFFFFFFu, l_all, 2);
      if (!row_ok[x]) continue;
      if (pieces == 1) {
        // The sequence's only piece: its partial is the result.
        const float inv = 1.0f / fmaxf(l_all, 1e-30f);
        uint32_t* dst = reinterpret_cast<uint32_t*>(p.out + (static_cast<size_t>(cur) * p.rows + row_head[x]) * DEC_D);
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) dst[nt * 4 + t] = pack_bf16(o[nt][2 * x] * inv, o[nt][2 * x + 1] * inv);
      } else {
        if (t == 0) {  // the partials keep the max in natural-log units
          p.ws_m[base + row_head[x]] = m_run[x] * (1.0f / DEC_LOG2E);
          p.ws_l[base + row_head[x]] = l_all;
        }
        float2* dst = reinterpret_cast<float2*>(p.ws_acc + (base + row_head[x]) * DEC_D);
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) dst[nt * 4 + t] = make_float2(o[nt][2 * x], o[nt][2 * x + 1]);
      }
    }
    if (pieces > 1) {
      // Count this piece; whoever counts last finds every partial of the sequence's KV head written and merges.
      // The counters were cleared by the step-table kernel: it must have finished.
      asm volatile("griddepcontrol.wait;" ::: "memory");
      __threadfence();
      __syncwarp();
      int last = 0;
      if (lane == 0) last = atomicAdd(p.arrivals + cur * p.Hkv + kvh, 1) == pieces - 1;
      last = __shfl_sync(0xFFFFFFFFu, last, 0);
      if (last) {
        __threadfence();
        for (int tok = 0; tok < p.T; ++tok) decode_merge_heads<G>(p, cur, tok * p.H + kvh * G, pieces, lane);
      }
    }
  };

  // The share is walked 32 steps at a time (a lane holds a step); the accumulators carry over.
  for (int s_begin = r_begin; s_begin < r_end && ok; s_begin += 32) {
  const int n_here = min(32, r_end - s_begin);

  // The chunk's steps, one per lane (lanes 0..n_here-1), broadcast by shuffle when needed.
  int my_tile = -1, my_code = 4, my_page = 0, my_len = 0;
  if (lane < n_here) {
    if (p.self_steps) {
      // The sequence holding step s: the last one whose first step is <= s (every sequence takes a step).
      const int st = s_begin + lane;
      int lo = 0, hi = p.B;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_first[mid] <= st) lo = mid; else hi = mid;
      }
      my_tile = lo;
      my_len = p.lengths[lo];
      my_code = ((st - s_first[lo]) << 3) | (my_len > 0 ? 0 : 4);
    } else {
      my_tile = p.step_tile[s_begin + lane];
      my_code = p.step_code[s_begin + lane];
      my_len = p.lengths[my_tile];
    }
    if (!(my_code & 4)) {
      const int pg = my_code >> 3;
      my_page = p.block_tables[static_cast<size_t>(my_tile) * p.pages_per_seq + pg];
      my_page = min(max(my_page, 0), p.num_pages - 1);
    }
  }

  // The next micro-step (step, 16-token sub-block) that has data after (step, sub); step == n_here if none.
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
      tma_load_3d(dst + DEC_HALF_BYTES, &map_k, 64, kvh, token, bar(stage));
      tma_load_3d(dst + 2 * DEC_HALF_BYTES, &map_v, 0, kvh, token, bar(stage));
      tma_load_3d(dst + 3 * DEC_HALF_BYTES, &map_v, 64, kvh, token, bar(stage));
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
    const int tile = __shfl_sync(0xFFFFFFFFu, my_tile, step);
    const int code = __shfl_sync(0xFFFFFFFFu, my_code, step);
    const int len = __shfl_sync(0xFFFFFFFFu, my_len, step);
    if (tile != cur) {
      flush();
      cur = tile;
#pragma unroll
      for (int x = 0; x < NR; ++x) {
        const uint32_t* qp = reinterpret_cast<const uint32_t*>(
            p.q + (static_cast<size_t>(tile) * p.rows + (row_ok[x] ? row_head[x] : 0)) * DEC_D);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          qa[j][2 * x] = row_ok[x] ? qp[8 * j + t] : 0u;
          qa[j][2 * x + 1] = row_ok[x] ? qp[8 * j + 4 + t] : 0u;
        }
        m_run[x] = DEC_MASK * DEC_LOG2E, l_run[x] = 0.f;
      }
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
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
      if (n == 0) t_first = clock64();
      const bool got = mbar_wait_timed(bar(stage), (n / DEC_STAGES) & 1, &dec_abort, p.status, TJX_ERR_WAIT_FULL, in_wait, prof != nullptr);
      if (fill_wait < 0) fill_wait = in_wait;
      if (!__all_sync(0xFFFFFFFFu, got)) {
        ok = false;
        break;
      }
      ++n;
      const uint32_t kbase = ring + stage * DEC_STAGE_BYTES;
      const uint32_t vbase = kbase + 2 * DEC_HALF_BYTES;

      // S = Q K^T: two tiles of 8 tokens; [tile][0..1] = row g, tokens 8 tile + 2t, + 1; [2..3] = row g + 8.
      float sc[2][4];
#pragma unroll
      for (int tl = 0; tl < 2; ++tl) {
        sc[tl][0] = sc[tl][1] = sc[tl][2] = sc[tl][3] = 0.f;
#pragma unroll
        for (int x = 0; x < 4; ++x) {  // a load covers dims 32 x .. 32 x + 31: k-steps 2x and 2x + 1
          const int unit = (4 * x + k_unit) & 7;          // the 16-byte unit within the 64-dim half
          const uint32_t addr = kbase + (x >> 1) * DEC_HALF_BYTES + tl * 1024 + k_lane + ((unit ^ lrow) << 4);
          uint32_t b[4];
          ldmatrix_x4(addr, b);
          if constexpr (WIDE) {
            mma_16x8x16(sc[tl], qa[2 * x][0], qa[2 * x][2], qa[2 * x][1], qa[2 * x][3], b[0], b[1]);
            mma_16x8x16(sc[tl], qa[2 * x + 1][0], qa[2 * x + 1][2], qa[2 * x + 1][1], qa[2 * x + 1][3], b[2], b[3]);
          } else {
            mma_16x8x16(sc[tl], qa[2 * x][0], 0u, qa[2 * x][1], 0u, b[0], b[1]);
            mma_16x8x16(sc[tl], qa[2 * x + 1][0], 0u, qa[2 * x + 1][1], 0u, b[2], b[3]);
          }
        }
      }
      // Online softmax of each row over the 16 tokens (4 per lane, the 4 lanes of a quad share a row). Row r's
      // new token sits at position len - T + token(r) and sees the positions up to its own.
      uint32_t pa[4] = {0u, 0u, 0u, 0u};  // P as the A fragment: [0] row g tokens 2t.., [1] row g + 8, [2], [3] tokens 8 + 2t..
      bool grew = false;
      float alpha[NR];
#pragma unroll
      for (int x = 0; x < NR; ++x) {
        float s4[4] = {sc[0][2 * x], sc[0][2 * x + 1], sc[1][2 * x], sc[1][2 * x + 1]};
        const int last_visible = len - p.T + row_tok[x];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int tok = (i >> 1) * 8 + 2 * t + (i & 1);
          s4[i] = base_pos + tok <= last_visible ? s4[i] * p.score_scale : DEC_MASK * DEC_LOG2E;
        }
        float mx = fmaxf(fmaxf(s4[0], s4[1]), fmaxf(s4[2], s4[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, 2));
        const float m_new = fmaxf(m_run[x], mx);
        alpha[x] = ex2(m_run[x] - m_new);
        grew |= m_new > m_run[x];
        m_run[x] = m_new;
        const float p0 = ex2(s4[0] - m_new), p1 = ex2(s4[1] - m_new), p2 = ex2(s4[2] - m_new), p3 = ex2(s4[3] - m_new);
        l_run[x] = l_run[x] * alpha[x] + ((p0 + p1) + (p2 + p3));
        pa[x] = pack_bf16(p0, p1), pa[2 + x] = pack_bf16(p2, p3);  // P is rounded before P V
      }
      if (__any_sync(0xFFFFFFFFu, grew)) {
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
          o[nt][0] *= alpha[0], o[nt][1] *= alpha[0];
          if constexpr (WIDE) o[nt][2] *= alpha[1], o[nt][3] *= alpha[1];
        }
      }
      // O += P V: a load covers dims 16 x .. 16 x + 15 (two output tiles) of all 16 tokens.
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        const int unit = (2 * x + v_unit) & 7;
        const uint32_t addr = vbase + (x >> 2) * DEC_HALF_BYTES + v_lane + ((unit ^ lrow) << 4);
        uint32_t b[4];
        ldmatrix_x4_trans(addr, b);
        mma_16x8x16(o[2 * x], pa[0], pa[1], pa[2], pa[3], b[0], b[1]);
        mma_16x8x16(o[2 * x + 1], pa[0], pa[1], pa[2], pa[3], b[2], b[3]);
      }
      __syncwarp();  // every lane is done with the slot before it is refilled
    }
  }
  }  // 32 steps of the share
  const long long t_last = clock64();
  if (ok) flush();
  if (prof != nullptr && threadIdx.x == 0) {
    prof[1] = t_first, prof[2] = t_last, prof[3] = in_wait, prof[4] = max(fill_wait, 0ll), prof[5] = 0, prof[6] = n;
    prof[7] = clock64();
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");  // never outlive the step-table kernel's writes unordered
}

template <int G, bool WIDE>
static int launch_chunks_for(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeParams& p, dim3 grid,
                             cudaStream_t s) {
  constexpr int SMEM = DEC_SMEM + (DEC_SELF_MAX_B + 1) * 4;
  auto kernel = decode_chunks_kernel<G, WIDE>;
  static bool configured[64] = {};
  int dev = 0;
  TJX_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    TJX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
    configured[dev & 63] = true;
  }
  // Programmatic stream serialisation: the grid may start while the step-table kernel before it in the stream
  // is still running; the kernel waits (griddepcontrol.wait) before it reads anything that kernel writes.
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid, cfg.blockDim = dim3(DEC_WARPS * 32), cfg.stream = s;
  cfg.dynamicSmemBytes = DEC_SMEM + (p.self_steps ? (p.B + 1) * 4 : 0);
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr, cfg.numAttrs = 1;
  TJX_CUDA(cudaLaunchKernelEx(&cfg, kernel, mk, mv, p));
  return 0;
}

// The page pools as 3-D tensors [token, KV head, dim] for TMA (box: 8 tokens x 1 head x 128 dims), then the
// chunk kernel for this group size. Allocates nothing.
static int launch_decode_chunks(DecodeParams& p, int group, cudaStream_t s) {
  p.status = device_status_word();
  if (p.status == nullptr) return fail(TJX_E_CUDA, "could not locate the device status word");
  const uint64_t dims[3] = {DEC_D, static_cast<uint64_t>(p.Hkv),
                            static_cast<uint64_t>(p.num_pages) * static_cast<uint64_t>(p.page_size)};
  const uint64_t head_stride = p.kv_head_stride > 0 ? static_cast<uint64_t>(p.kv_head_stride) : DEC_D;
  const uint64_t token_stride = p.kv_token_stride > 0 ? static_cast<uint64_t>(p.kv_token_stride)
                                                      : static_cast<uint64_t>(p.Hkv) * DEC_D;
  const uint64_t strides[2] = {head_stride * 2, token_stride * 2};
  const uint32_t box[3] = {64, 1, DEC_SUB};
  CUtensorMap mk, mv;
  if (int rc = make_tensor_map(&mk, p.k_pages, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 3, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (int rc = make_tensor_map(&mv, p.v_pages, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 3, dims, strides, box,
                               CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  const long long capacity = static_cast<long long>(p.B) * p.pages_per_seq;
  const int chunks = static_cast<int>((capacity + p.min_share - 1) / p.min_share);
  const int groups = (p.Hkv + DEC_WARPS - 1) / DEC_WARPS;
  const bool wide = p.T * group > 8;  // more than 8 query rows per KV head: both halves of the MMA's 16 rows
  // As many CTAs as are resident at once (never more than there are chunks of DEC_CHUNK steps): each takes an equal
  // contiguous share of the steps that run.
  const int resident = sm_count() * (wide ? TJX_DEC_CTAS * 2 / 3 : TJX_DEC_CTAS);
  dim3 grid(std::max(1, std::min(chunks, resident / groups)), groups);
  p.profile = profile_buffer(static_cast<int>(grid.x * grid.y));
  switch (group) {
    case 1: return wide ? launch_chunks_for<1, true>(mk, mv, p, grid, s) : launch_chunks_for<1, false>(mk, mv, p, grid, s);
    case 2: return wide ? launch_chunks_for<2, true>(mk, mv, p, grid, s) : launch_chunks_for<2, false>(mk, mv, p, grid, s);
    case 4: return wide ? launch_chunks_for<4, true>(mk, mv, p, grid, s) : launch_chunks_for<4, false>(mk, mv, p, grid, s);
    default: return wide ? launch_chunks_for<8, true>(mk, mv, p, grid, s) : launch_chunks_for<8, false>(mk, mv, p, grid, s);
  }
}

// Partials a sequence can have: the shares (of at least `min_share` steps) its pages_per_seq steps can fall in.
static int decode_slots(int pages_per_seq, int min_share = DEC_CHUNK) {
  return (pages_per_seq + min_share - 1) / min_share + 1;
}

// The least share for pages of `page_size` tokens: DEC_CHUNK pages of 16, as many tokens in larger pages. (With
// pages of 128 a share of DEC_CHUNK steps is 1536 tokens: 32 sequences of ~2000 tokens then keep a quarter of the
// resident warps busy and the kernel streams at 3 TB/s.)
static int min_share_for_pages_of(int page_size) {
  return std::max(1, (DEC_CHUNK * DEC_SUB + page_size - 1) / page_size);
}

static size_t align256(size_t n) { return (n + 255) & ~static_cast<size_t>(255); }

// Scratch layout, with rows = T * H query rows per sequence: max [B, slots, rows] | sum [B, slots, rows] |
// accumulators [B, slots, rows, D] | arrival counters [B, Hkv] (room for H per sequence). Nothing in it has to start at zero: the step-table kernel clears the
// counters at the start of every call, and every partial that is read was written earlier in the same call.
static size_t decode_scratch_bytes(int B, int T, int H, int D, int pages_per_seq, int min_share = DEC_CHUNK) {
  const size_t rows = static_cast<size_t>(B) * decode_slots(pages_per_seq, min_share) * T * H;
  return 2 * align256(rows * sizeof(float)) + align256(rows * D * sizeof(float)) +
         align256(static_cast<size_t>(B) * H * sizeof(int));
}

static int check_decode_args(const void* q, const void* k_pages, const void* v_pages, const int32_t* block_tables,
                             const int32_t* lengths, const void* out, int B, int T, int H, int Hkv, int D,
                             int page_size, int pages_per_seq, int num_pages, const int32_t* step_tile,
                             const int32_t* step_code, const int32_t* step_count, const int32_t* tile_first) {
  if (!q || !k_pages || !v_pages || !block_tables || !lengths || !out)
    return fail(TJX_E_ARG, "an input or output pointer is null");
  if (!step_tile || !step_code || !step_count || !tile_first)
    return fail(TJX_E_ARG, "a step table pointer is null");
  if (B <= 0 || T <= 0 || H <= 0 || Hkv <= 0 || pages_per_seq <= 0 || num_pages <= 0)
    return fail(TJX_E_ARG, "sizes must be positive");
  if (D != DEC_D) return fail(TJX_E_ARG, "head dimension must be 128");
  if (page_size <= 0 || page_size % 16 != 0) return fail(TJX_E_ARG, "page size must be a multiple of 16");
  if (H % Hkv != 0) return fail(TJX_E_ARG, "H must be a multiple of Hkv");
  const int group = H / Hkv;
  if (group != 1 && group != 2 && group != 4 && group != 8)
    return fail(TJX_E_ARG, "H / Hkv must be 1, 2, 4 or 8");
  if (T * group > 16)
    return fail(TJX_E_ARG, "new tokens x query heads per KV head must not exceed 16 (the rows of one warp-level MMA)");
  const uintptr_t ptrs[] = {reinterpret_cast<uintptr_t>(q), reinterpret_cast<uintptr_t>(k_pages),
                            reinterpret_cast<uintptr_t>(v_pages), reinterpret_cast<uintptr_t>(out)};
  for (uintptr_t a : ptrs)
    if (a & 15u) return fail(TJX_E_ARG, "q, k_pages, v_pages and out must be 16-byte aligned");
  return 0;
}

// The two launches of a decode call, with the partials and counters in `scratch` (decode_scratch_bytes of it,
// 256-byte aligned). Allocates nothing.
static int run_decode(const void* q, const void* k_pages, const void* v_pages, const int32_t* block_tables,
                      const int32_t* lengths, void* out, int B, int T, int H, int Hkv, int page_size,
                      int pages_per_seq, int num_pages, int32_t* step_tile, int32_t* step_code, int32_t* step_count,
                      int32_t* tile_first, void* scratch, cudaStream_t s, float softmax_scale = 1.0f,
                      long long kv_head_stride = 0, long long kv_token_stride = 0, int min_share = DEC_CHUNK) {
  DecodeParams p{};
  p.min_share = min_share;
  p.score_scale = DEC_LOG2E * softmax_scale;
  p.kv_head_stride = kv_head_stride, p.kv_token_stride = kv_token_stride;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k_pages = static_cast<const __nv_bfloat16*>(k_pages);
  p.v_pages = static_cast<const __nv_bfloat16*>(v_pages);
  p.block_tables = block_tables, p.lengths = lengths;
  p.step_tile = step_tile, p.step_code = step_code, p.step_count = step_count, p.tile_first = tile_first;
  p.B = B, p.H = H, p.Hkv = Hkv, p.page_size = page_size, p.pages_per_seq = pages_per_seq, p.num_pages = num_pages;
  p.T = T, p.rows = T * H;
  p.self_steps = B <= DEC_SELF_MAX_B ? 1 : 0;
  p.slots = decode_slots(pages_per_seq, min_share);
  const size_t rows = static_cast<size_t>(B) * p.slots * p.rows;
  uint8_t* ws = static_cast<uint8_t*>(scratch);
  p.ws_m = reinterpret_cast<float*>(ws);
  p.ws_l = reinterpret_cast<float*>(ws + align256(rows * sizeof(float)));
  p.ws_acc = reinterpret_cast<float*>(ws + 2 * align256(rows * sizeof(float)));
  p.arrivals = reinterpret_cast<int*>(ws + 2 * align256(rows * sizeof(float)) + align256(rows * DEC_D * sizeof(float)));
  p.out = static_cast<__nv_bfloat16*>(out);

  if (int rc = launch_build_steps_lengths(lengths, B, nullptr, B, pages_per_seq, 0, page_size, step_tile, step_code,
                                          step_count, tile_first, p.arrivals, B * Hkv, s))
    return rc;
  return launch_decode_chunks(p, H / Hkv, s);
}

}  // namespace tjx

extern "C" {

size_t tjx_paged_gqa_decode_workspace_bytes(int B, int T, int H, int D, int pages_per_seq) {
  if (B <= 0 || T <= 0 || H <= 0 || D <= 0 || pages_per_seq <= 0) return 0;
  return tjx::decode_scratch_bytes(B, T, H, D, pages_per_seq);
}

int tjx_paged_gqa_decode_bf16(const void* q, const void* k_pages, const void* v_pages, const int32_t* block_tables,
                              const int32_t* lengths, void* out, int B, int T, int H, int Hkv, int D, int page_size,
                              int pages_per_seq, int num_pages, int32_t* step_tile, int32_t* step_code,
                              int32_t* step_count, int32_t* tile_first, void* workspace, size_t workspace_bytes,
                              tjx_stream_t stream) {
  using namespace tjx;
  if (int rc = check_device()) return rc;
  if (int rc = check_decode_args(q, k_pages, v_pages, block_tables, lengths, out, B, T, H, Hkv, D, page_size,
                                 pages_per_seq, num_pages, step_tile, step_code, step_count, tile_first))
    return rc;
  const size_t need = tjx_paged_gqa_decode_workspace_bytes(B, T, H, D, pages_per_seq);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(TJX_E_ARG, "workspace is null or smaller than tjx_paged_gqa_decode_workspace_bytes");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(TJX_E_ARG, "workspace must be 256-byte aligned");
  return run_decode(q, k_pages, v_pages, block_tables, lengths, out, B, T, H, Hkv, page_size, pages_per_seq,
                    num_pages, step_tile, step_code, step_count, tile_first, workspace,
                    static_cast<cudaStream_t>(stream));
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------------------
// Ragged paged attention's cache write and decode case (examples/ragged_paged_attention.py:33-47, :121-149): q
// (T, H, D) with every sequence's new tokens concatenated, a cache (pages, page_size, Hkv, 2, D) holding each head's
// key and value side by side, kv_lens (S,) with the new tokens included, page_indices (S * pages_per_seq,),
// cu_q_lens (S + 1,), distribution (3,): sequences [0, d0) decode one token each (sequence s is token s).
// The decode case is the paged decode kernel above on the cache's own layout — K of (token, head) 2 D elements
// apart, V D elements after K: two tensor maps over one buffer — with the softmax scale folded into the score
// scale, the lengths of sequences outside [0, d0) set to zero, and only the decode tokens' rows written back.

namespace tjx {

// One CTA per new token: its sequence by bisection in cu_q_lens, its position kv_len - q_len + (t - first token),
// its page through page_indices; 128 threads copy the token's Hkv * D keys and values, 16 bytes at a time.
__global__ void __launch_bounds__(128)
    rpa_write_kernel(__nv_bfloat16* __restrict__ cache, const __nv_bfloat16* __restrict__ keys,
                     const __nv_bfloat16* __restrict__ values, const int32_t* __restrict__ kv_lens,
                     const int32_t* __restrict__ page_indices, const int32_t* __restrict__ cu_q_lens,
                     const int32_t* __restrict__ distribution, int S, int Hkv, int page_size, int pages_per_seq,
                     int num_pages) {
  chain_release();  // (a kernel chained behind this one may run beside it: see tjx_ragged_paged_attention_bf16)
  const int t = blockIdx.x;
  int lo = 0, hi = S;  // the sequence with cu_q_lens[s] <= t < cu_q_lens[s + 1]
  if (t >= cu_q_lens[S]) return;  // a padding token
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu_q_lens[mid] <= t) lo = mid; else hi = mid;
  }
  const int s = lo;
  if (s >= distribution[2]) return;
  const int first = cu_q_lens[s], q_len = cu_q_lens[s + 1] - first;
  const int pos = kv_lens[s] - q_len + (t - first);
  if (pos < 0 || pos >= pages_per_seq * page_size) return;
  const int page = min(max(page_indices[s * pages_per_seq + pos / page_size], 0), num_pages - 1);
  __nv_bfloat16* dst = cache + (static_cast<size_t>(page) * page_size + pos % page_size) * Hkv * 2 * DEC_D;
  const uint4* k = reinterpret_cast<const uint4*>(keys + static_cast<size_t>(t) * Hkv * DEC_D);
  const uint4* v = reinterpret_cast<const uint4*>(values + static_cast<size_t>(t) * Hkv * DEC_D);
  for (int u = threadIdx.x; u < Hkv * DEC_D / 8; u += blockDim.x) {
    const int h = u / (DEC_D / 8), d = (u % (DEC_D / 8)) * 8;
    *reinterpret_cast<uint4*>(dst + h * 2 * DEC_D + d) = k[u];
    *reinterpret_cast<uint4*>(dst + h * 2 * DEC_D + DEC_D + d) = v[u];
  }
}

// The same write from the run tables the reference's `rpa_write` kernel takes (examples/ragged_paged_attention.py:33-47):
// run w < n_writes[0] copies the tokens from write_rows[w] on to rows write_first[w] .. write_stop[w] - 1 of page
// page_indices[write_page[w]]. One CTA per (row of a page, run); rows past the run, runs past the count, tokens or
// rows out of range write nothing (the reference's out-of-bounds stores are dropped), indices into page_indices and
// page numbers are clamped as its gathers are.
__global__ void __launch_bounds__(128)
    rpa_write_runs_kernel(__nv_bfloat16* __restrict__ cache, const __nv_bfloat16* __restrict__ keys,
                          const __nv_bfloat16* __restrict__ values, const int32_t* __restrict__ page_indices,
                          const int32_t* __restrict__ write_page, const int32_t* __restrict__ write_rows,
                          const int32_t* __restrict__ write_first, const int32_t* __restrict__ write_stop,
                          const int32_t* __restrict__ n_writes, int T, int n_page_indices, int Hkv, int page_size,
                          int num_pages) {
  const int w = blockIdx.y, r = blockIdx.x;
  if (w >= n_writes[0]) return;
  const int first = write_first[w], stop = write_stop[w];
  const int row = first + r, t = write_rows[w] + r;
  if (row >= stop || row < 0 || row >= page_size || t < 0 || t >= T) return;
  const int entry = min(max(write_page[w], 0), n_page_indices - 1);
  const int page = min(max(page_indices[entry], 0), num_pages - 1);
  __nv_bfloat16* dst = cache + (static_cast<size_t>(page) * page_size + row) * Hkv * 2 * DEC_D;
  const uint4* k = reinterpret_cast<const uint4*>(keys + static_cast<size_t>(t) * Hkv * DEC_D);
  const uint4* v = reinterpret_cast<const uint4*>(values + static_cast<size_t>(t) * Hkv * DEC_D);
  for (int u = threadIdx.x; u < Hkv * DEC_D / 8; u += blockDim.x) {
    const int h = u / (DEC_D / 8), d = (u % (DEC_D / 8)) * 8;
    *reinterpret_cast<uint4*>(dst + h * 2 * DEC_D + d) = k[u];
    *reinterpret_cast<uint4*>(dst + h * 2 * DEC_D + DEC_D + d) = v[u];
  }
}

// lengths[s] = kv_lens[s] for the decode sequences, 0 for the others (which then take one empty step).
__global__ void rpa_decode_lengths_kernel(const int32_t* __restrict__ kv_lens, const int32_t* __restrict__ distribution,
                                          int32_t* __restrict__ lengths, int n, int max_len) {
  chain_release();  // (reads only the call's inputs: when chained it runs beside the kernel in front of it)
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s < n) lengths[s] = s < distribution[0] ? min(max(kv_lens[s], 0), max_len) : 0;
  chain_wait();  // ends after the kernel it was chained behind: what follows this one follows that one too
}

// out[s] = result[s] for the decode tokens (one CTA per token, 16 bytes per thread per pass); other rows keep q.
__global__ void __launch_bounds__(128)
    rpa_decode_scatter_kernel(const __nv_bfloat16* __restrict__ result, __nv_bfloat16* __restrict__ out,
                              const int32_t* __restrict__ distribution, int row_elements) {
  const int s = blockIdx.x;
  if (s >= distribution[0]) return;
  const uint4* src = reinterpret_cast<const uint4*>(result + static_cast<size_t>(s) * row_elements);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(s) * row_elements);
  for (int u = threadIdx.x; u < row_elements / 8; u += blockDim.x) dst[u] = src[u];
}

// The whole step's rows other than the prefill tiles': row r of out becomes the decode result of token r < decode
// sequences, or, where `keep` is set, stays the query unless a prefill tile covers it (those rows are the attention
// kernel's to write). One CTA per row; the tile list is short (a tile per 128 new tokens).
__global__ void __launch_bounds__(128)
    rpa_finish_rows_kernel(const __nv_bfloat16* __restrict__ result, const __nv_bfloat16* __restrict__ q,
                           __nv_bfloat16* __restrict__ out, const int32_t* __restrict__ distribution, int n,
                           int row_elements, const int32_t* __restrict__ tile_row0,
                           const int32_t* __restrict__ tile_rows, const int32_t* __restrict__ n_tiles, int max_tiles,
                           int keep) {
  __shared__ int covered;
  chain_release();
  const int r = blockIdx.x;
  const __nv_bfloat16* from;
  if (r < n && r < distribution[0]) {
    from = result;
  } else {
    if (!keep) return;
    if (threadIdx.x == 0) covered = 0;
    __syncthreads();
    const int count = min(max(n_tiles[0], 0), max_tiles);
    for (int k = threadIdx.x; k < count; k += blockDim.x) {
      const int first = tile_row0[k];
      if (r >= first && r < first + tile_rows[k]) covered = 1;
    }
    __syncthreads();
    if (covered) return;
    from = q;
  }
  const uint4* src = reinterpret_cast<const uint4*>(from + static_cast<size_t>(r) * row_elements);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * row_elements);
  for (int u = threadIdx.x; u < row_elements / 8; u += blockDim.x) dst[u] = src[u];
}

struct RpaScratch {
  int32_t *lengths, *step_tile, *step_code, *step_count, *tile_first;
  __nv_bfloat16* result;
  void* decode;
  size_t bytes;
};

static RpaScratch rpa_scratch(void* workspace, int n, int H, int page_size, int pages_per_seq) {
  uint8_t* w = static_cast<uint8_t*>(workspace);
  size_t at = 0;
  auto take = [&](size_t bytes) {
    uint8_t* ptr = w == nullptr ? nullptr : w + at;
    at += align256(bytes);
    return ptr;
  };
  RpaScratch r{};
  r.lengths = reinterpret_cast<int32_t*>(take(static_cast<size_t>(n) * 4));
  r.step_tile = reinterpret_cast<int32_t*>(take(static_cast<size_t>(n) * pages_per_seq * 4));
  r.step_code = reinterpret_cast<int32_t*>(take(static_cast<size_t>(n) * pages_per_seq * 4));
  r.step_count = reinterpret_cast<int32_t*>(take(4));
  r.tile_first = reinterpret_cast<int32_t*>(take(static_cast<size_t>(n + 1) * 4));
  r.result = reinterpret_cast<__nv_bfloat16*>(take(static_cast<size_t>(n) * H * DEC_D * 2));
  r.decode = take(decode_scratch_bytes(n, 1, H, DEC_D, pages_per_seq, min_share_for_pages_of(page_size)));
  r.bytes = at;
  return r;
}

}  // namespace tjx

extern "C" {

int tjx_rpa_write_bf16(void* kv_cache, const void* keys, const void* values, const int32_t* kv_lens,
                       const int32_t* page_indices, const int32_t* cu_q_lens, const int32_t* distribution, int T,
                       int S, int Hkv, int D, int page_size, int pages_per_seq, int num_pages, tjx_stream_t stream) {
  using namespace tjx;
  if (int rc = check_device()) return rc;
  if (!kv_cache || !keys || !values || !kv_lens || !page_indices || !cu_q_lens || !distribution)
    return fail(TJX_E_ARG, "an input pointer is null");
  if (T <= 0 || S <= 0 || Hkv <= 0 || page_size <= 0 || pages_per_seq <= 0 || num_pages <= 0)
    return fail(TJX_E_ARG, "sizes must be positive");
  if (D != DEC_D) return fail(TJX_E_ARG, "head dimension must be 128");
  const uintptr_t ptrs[] = {reinterpret_cast<uintptr_t>(kv_cache), reinterpret_cast<uintptr_t>(keys),
                            reinterpret_cast<uintptr_t>(values)};
  for (uintptr_t a : ptrs)
    if (a & 15u) return fail(TJX_E_ARG, "kv_cache, keys and values must be 16-byte aligned");
  rpa_write_kernel<<<T, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(kv_cache), static_cast<const __nv_bfloat16*>(keys),
      static_cast<const __nv_bfloat16*>(values), kv_lens, page_indices, cu_q_lens, distribution, S, Hkv, page_size,
      pages_per_seq, num_pages);
  TJX_CUDA(cudaGetLastError());
  return 0;
}

int tjx_rpa_write_runs_bf16(void* kv_cache, const void* keys, const void* values, const int32_t* page_indices,
                            const int32_t* write_page, const int32_t* write_rows, const int32_t* write_first,
                            const int32_t* write_stop, const int32_t* n_writes, int T, int n_page_indices, int max_runs,
                            int Hkv, int D, int page_size, int num_pages, tjx_stream_t stream) {
  using namespace tjx;
  if (int rc = check_device()) return rc;
  if (!kv_cache || !keys || !values || !page_indices || !write_page || !write_rows || !write_first || !write_stop ||
      !n_writes)
    return fail(TJX_E_ARG, "an input pointer is null");
  if (T <= 0 || n_page_indices <= 0 || max_runs <= 0 || Hkv <= 0 || page_size <= 0 || num_pages <= 0)
    return fail(TJX_E_ARG, "sizes must be positive");
  if (max_runs > 65535) return fail(TJX_E_LIMIT, "more than 65535 runs");
  if (D != DEC_D) return fail(TJX_E_ARG, "head dimension must be 128");
  const uintptr_t ptrs[] = {reinterpret_cast<uintptr_t>(kv_cache), reinterpret_cast<uintptr_t>(keys),
                            reinterpret_cast<uintptr_t>(values)};
  for (uintptr_t a : ptrs)
    if (a & 15u) return fail(TJX_E_ARG, "kv_cache, keys and values must be 16-byte aligned");
  rpa_write_runs_kernel<<<dim3(page_size, max_runs), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(kv_cache), static_cast<const __nv_bfloat16*>(keys),
      static_cast<const __nv_bfloat16*>(values), page_indices, write_page, write_rows, write_first, write_stop, n_writes,
      T, n_page_indices, Hkv, page_size, num_pages);
  TJX_CUDA(cudaGetLastError());
  return 0;
}

size_t tjx_rpa_decode_workspace_bytes(int T, int S, int H, int D, int page_size, int pages_per_seq) {
  if (T <= 0 || S <= 0 || H <= 0 || D <= 0 || page_size <= 0 || pages_per_seq <= 0) return 0;
  return tjx::rpa_scratch(nullptr, std::min(S, T), H, page_size, pages_per_seq).bytes;
}

int tjx_rpa_decode_bf16(const void* q, void* out, const void* kv_cache, const int32_t* kv_lens,
                        const int32_t* page_indices, const int32_t* distribution, int T, int S, int H, int Hkv, int D,
                        int page_size, int pages_per_seq, int num_pages, float sm_scale, void* workspace,
                        size_t workspace_bytes, tjx_stream_t stream) {
  using namespace tjx;
  if (int rc = check_device()) return rc;
  if (!kv_lens || !page_indices || !distribution) return fail(TJX_E_ARG, "an index array pointer is null");
  const int n = std::min(S, T);  // sequence s is token s
  const size_t need = tjx_rpa_decode_workspace_bytes(T, S, H, D, page_size, pages_per_seq);
  if (T <= 0 || S <= 0 || need == 0) return fail(TJX_E_ARG, "sizes must be positive");
  if (workspace == nullptr || workspace_bytes < need)
    return fail(TJX_E_ARG, "workspace is null or smaller than tjx_rpa_decode_workspace_bytes");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(TJX_E_ARG, "workspace must be 256-byte aligned");
  const RpaScratch w = rpa_scratch(workspace, n, H, page_size, pages_per_seq);
  const __nv_bfloat16* cache = static_cast<const __nv_bfloat16*>(kv_cache);
  if (int rc = check_decode_args(q, cache, cache == nullptr ? nullptr : cache + DEC_D, page_indices, w.lengths, out, n, 1,
                                 H, Hkv, D, page_size, pages_per_seq, num_pages, w.step_tile, w.step_code, w.step_count,
                                 w.tile_first))
    return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out != q)  // rows that are not decode tokens keep the query
    TJX_CUDA(cudaMemcpyAsync(out, q, static_cast<size_t>(T) * H * DEC_D * 2, cudaMemcpyDeviceToDevice, s));
  rpa_decode_lengths_kernel<<<(n + 127) / 128, 128, 0, s>>>(kv_lens, distribution, w.lengths, n,
                                                            pages_per_seq * page_size);
  TJX_CUDA(cudaGetLastError());
  if (int rc = run_decode(q, cache, cache + DEC_D, page_indices, w.lengths, w.result, n, 1, H, Hkv, page_size,
                          pages_per_seq, num_pages, w.step_tile, w.step_code, w.step_count, w.tile_first, w.decode, s,
                          sm_scale, 2 * DEC_D, static_cast<long long>(Hkv) * 2 * DEC_D, min_share_for_pages_of(page_size)))
    return rc;
  rpa_decode_scatter_kernel<<<n, 128, 0, s>>>(w.result, static_cast<__nv_bfloat16*>(out), distribution, H * DEC_D);
  TJX_CUDA(cudaGetLastError());
  return 0;
}

size_t tjx_ragged_paged_attention_workspace_bytes(int T, int S, int H, int D, int page_size, int pages_per_seq) {
  const size_t decode = tjx_rpa_decode_workspace_bytes(T, S, H, D, page_size, pages_per_seq);
  if (decode == 0) return 0;
  return tjx::align256(decode) + tjx::rpa_prefill_part_bytes(T, S);
}

int tjx_ragged_paged_attention_bf16(const void* q, const void* keys, const void* values, void* kv_cache,
                                    const int32_t* kv_lens, const int32_t* page_indices, const int32_t* cu_q_lens,
                                    const int32_t* distribution, void* out, int T, int S, int H, int Hkv, int D,
                                    int page_size, int pages_per_seq, int num_pages, float sm_scale, void* workspace,
                                    size_t workspace_bytes, tjx_stream_t stream) {
  using namespace tjx;
  if (int rc = check_device()) return rc;
  if (!q || !out || !keys || !values || !kv_cache || !kv_lens || !page_indices || !cu_q_lens || !distribution)
    return fail(TJX_E_ARG, "an input or output pointer is null");
  const size_t need = tjx_ragged_paged_attention_workspace_bytes(T, S, H, D, page_size, pages_per_seq);
  if (T <= 0 || S <= 0 || need == 0) return fail(TJX_E_ARG, "sizes must be positive");
  if (workspace == nullptr || workspace_bytes < need)
    return fail(TJX_E_ARG, "workspace is null or smaller than tjx_ragged_paged_attention_workspace_bytes");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(TJX_E_ARG, "workspace must be 256-byte aligned");
  // Every refusal of a size or a pointer comes before the first launch: the cache is not written by a call that fails.
  const int n = std::min(S, T);  // sequence s is token s
  if (int rc = check_step_table_sizes(n, pages_per_seq)) return rc;
  const RpaScratch w = rpa_scratch(workspace, n, H, page_size, pages_per_seq);
  void* prefill_ws = static_cast<uint8_t*>(workspace) + align256(w.bytes);
  const __nv_bfloat16* cache = static_cast<const __nv_bfloat16*>(kv_cache);
  if (int rc = check_decode_args(q, cache, cache + DEC_D, page_indices, w.lengths, out, n, 1, H, Hkv, D, page_size,
                                 pages_per_seq, num_pages, w.step_tile, w.step_code, w.step_count, w.tile_first))
    return rc;
  if (int rc = rpa_prefill_part_check(q, out, kv_cache, page_indices, T, S, H, Hkv, D, page_size, pages_per_seq, num_pages))
    return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // 1. The new tokens into the cache; beside it (chained, reading only index arrays) the decode lengths and the
  //    prefill tiles.
  if (int rc = tjx_rpa_write_bf16(kv_cache, keys, values, kv_lens, page_indices, cu_q_lens, distribution, T, S, Hkv, D,
                                  page_size, pages_per_seq, num_pages, stream))
    return rc;
  TJX_CUDA(launch_chained(rpa_decode_lengths_kernel, dim3((n + 127) / 128), dim3(128), 0, s, kv_lens, distribution,
                          w.lengths, n, pages_per_seq * page_size));
  RpaTiles tiles{};
  if (int rc = rpa_prefill_tiles_part(kv_lens, cu_q_lens, distribution, T, S, pages_per_seq, prefill_ws, s, &tiles))
    return rc;
  // 2. The decode sequences over the updated cache (ordinary launches: they follow everything above), into scratch.
  if (int rc = run_decode(q, cache, cache + DEC_D, page_indices, w.lengths, w.result, n, 1, H, Hkv, page_size,
                          pages_per_seq, num_pages, w.step_tile, w.step_code, w.step_count, w.tile_first, w.decode, s,
                          sm_scale, 2 * DEC_D, static_cast<long long>(Hkv) * 2 * DEC_D, min_share_for_pages_of(page_size)))
    return rc;
  // 3. Their rows of out, and q's rows that no case writes; 4. the prefill tiles' rows, queries straight from q, its
  //    set-up under kernel 3.
  rpa_finish_rows_kernel<<<T, 128, 0, s>>>(w.result, static_cast<const __nv_bfloat16*>(q),
                                           static_cast<__nv_bfloat16*>(out), distribution, n, H * DEC_D, tiles.row0,
                                           tiles.rows, tiles.count, tiles.max_tiles, out != q ? 1 : 0);
  TJX_CUDA(cudaGetLastError());
  LaunchChain chain(CHAIN_WAITS);
  return rpa_prefill_attention_part(q, out, kv_cache, page_indices, T, S, H, Hkv, pages_per_seq, num_pages, sm_scale,
                                    prefill_ws, s);
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
                                     const int32_t* block_tables, const int32_t* lengths, void* out, int B, int T,
                                     int H, int Hkv, int D, int page_size, int pages_per_seq, int num_pages,
                                     int32_t* step_tile, int32_t* step_code, int32_t* step_count, int32_t* tile_first,
                                     tjx_stream_t stream) {
  using namespace tjx;
  if (int rc = check_device()) return rc;
  if (int rc = check_decode_args(q, k_pages, v_pages, block_tables, lengths, out, B, T, H, Hkv, D, page_size,
                                 pages_per_seq, num_pages, step_tile, step_code, step_count, tile_first))
    return rc;
  const size_t need = tjx_paged_gqa_decode_workspace_bytes(B, T, H, D, pages_per_seq);
  if (need > STATIC_SCRATCH_BYTES)
    return fail(TJX_E_LIMIT, "these sizes need " + std::to_string(need) + " bytes of scratch, more than the " +
                                 std::to_string(STATIC_SCRATCH_BYTES) +
                                 " bytes built into the library: use tjx_paged_gqa_decode_bf16 with a workspace");
  void* scratch = nullptr;
  if (int rc = static_scratch_address(&scratch)) return rc;
  return run_decode(q, k_pages, v_pages, block_tables, lengths, out, B, T, H, Hkv, page_size, pages_per_seq,
                    num_pages, step_tile, step_code, step_count, tile_first, scratch,
                    static_cast<cudaStream_t>(stream));
}

}  // extern "C"

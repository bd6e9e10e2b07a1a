// Flash-style causal attention on sm_100a: the step loop of `causal_attention`
// (examples/causal_attention.py:37-63) with the scores and the output accumulator in TMEM.
//
// A work unit is one (b, h) and two consecutive query tiles of 128 rows ("slots" A and B); it walks the key/value
// blocks the step table lists for them in sub-blocks of 128 keys; a sub-block wholly in the future of a slot's
// rows is skipped for that slot (its probabilities would all be exp(-1e30 - max) = 0). Both slots share every
// K / V load. One persistent CTA per SM takes units heaviest first, dealt out in snake order (round k goes
// forwards over the CTAs for even k, backwards for odd k) so that every CTA gets the same amount of work;
// barriers, TMEM and the tensor maps are set up once, and the loads of the next unit start while the current
// one is still in its last blocks.
//
//   warp 0      producer: TMA loads Q (both slots, once per unit), then K and V sub-blocks into two 2-slot rings
//   warp 1      MMA issuer: S_t = Q_t K^T into TMEM, then O_t += P_t V with P_t read from TMEM. The whole warp
//               runs the loop (addresses and descriptors stay in uniform registers) and one elected lane issues
//               each accumulation's MMAs and its commit as one predicated block: issuing from inside a
//               one-lane branch cost ~60 cycles per MMA, as long as the 128 x 128 x 16 MMA itself takes
//   warps 2-5   softmax of slot A, warps 6-9 of slot B: a thread owns one query row — tcgen05.ld its 128
//               scores, running max / sum in f32 registers, exp2 (a quarter of them by a cubic on the FMA pipe,
//               the rest on the MUFU unit), P rounded to bf16 and stored back to TMEM over the scores, announced
//               in two halves so that P V starts on the first 64 keys while the rest are computed; rescales O in
//               TMEM when the running max grows; at the end normalises O and stores its row (256 contiguous
//               bytes) straight from registers
//
// TMEM (512 columns): S_A | S_B | O_A | O_B, 128 f32 columns each; P_t (bf16, two per column) overlays the
// first 64 columns of S_t. While one slot's softmax runs, the tensor core works on the other slot. Per slot the
// chain softmax -> P V -> next Q K^T is serial (S and P alias), which is what bounds the kernel: ~1800 cycles of
// softmax and ~1400 from its last store to the next scores, against 1024 cycles of MMAs per block and slot.
//
// Numerics follow the reference: q arrives pre-scaled; scores in f32 from bf16 operands; masked scores are
// -1e30; the row sum adds the unrounded probabilities while P is rounded to bf16 before P @ V; one division at
// the end. The running max is only raised when a block's max exceeds it by more than 8 (in log2 units), which
// changes no result beyond rounding: every term is scaled by the same power of two.
#include <algorithm>

#include "tjx_host.cuh"
#include "tjx_ptx.cuh"

#include "../../include/tilejax_b200.h"

namespace tjx {

constexpr int AT_D = 128;
constexpr int AT_BQ = 128;   // query rows per slot
constexpr int AT_BKV = 128;  // keys per sub-block
constexpr int AT_STAGES = 2;
constexpr int AT_THREADS = 320;
constexpr float AT_LOG2E = 1.4426950408889634f;
constexpr float AT_MASK = -1e30f;
constexpr float AT_RESCALE_THRESHOLD = 8.0f;

struct AttnParams {
  int B, H, S;
  int bq, bk;  // the user's blocks
  int pattern_steps, pattern_tiles;
  const int32_t* step_tile;
  const int32_t* step_code;
  int units_per_bh;  // pairs of 128-row query tiles per (b, h)
  int total_units;
  __nv_bfloat16* out;  // (B, H, S, D) in the input dtype, or null when `out_heads` is given
  float* out_heads;    // (B, S, H * D) f32: the heads side by side, unrounded (attention_block's `a`), or null
  int* status;
  long long* profile;  // per-CTA counters (PROFILE_WORDS each) or null
  // The paged variant (ragged paged attention's prefill case): tiles of up to 128 query tokens of one sequence.
  const int32_t* tile_row0;      // [tiles] first token (row of q (T, H, D)) of each tile
  const int32_t* tile_rows;      // [tiles] its tokens (1..128)
  const int32_t* tile_pos;       // [tiles] cache position of its first token
  const int32_t* tile_page;      // [tiles] index into page_indices of its sequence's first page
  const int32_t* n_tiles;        // [1]
  const int32_t* page_indices;
  int Hkv, group, num_pages;     // KV heads, query heads per KV head (even), pages in the pool
  int n_page_indices;            // entries of page_indices
  float scale_log2e;             // log2(e) times the softmax scale (the queries do not arrive pre-scaled)
  __nv_bfloat16* out_tokens;     // (T, H, D): row (token, head)
  int chain;                     // CHAIN_RELEASES: the kernel launched behind this one may be scheduled early;
                                 // CHAIN_WAITS: launched early itself, orders itself behind the kernel in front
};

constexpr int AT_MAX_TILES = 1024;  // user query tiles per (b, h) whose last key block is cached in shared memory

struct AttnSmem {
  static constexpr int TILE_BYTES = 128 * 128 * 2;  // a 128 x 128 bf16 tile: two 64-column boxes of 16 KB
  static constexpr int Q_OFF = 0;                    // 2 slots
  static constexpr int K_OFF = 2 * TILE_BYTES;       // AT_STAGES
  static constexpr int V_OFF = K_OFF + AT_STAGES * TILE_BYTES;
  static constexpr int BAR_OFF = V_OFF + AT_STAGES * TILE_BYTES;
  static constexpr int LAST_OFF = BAR_OFF + 256;               // last key block of each user query tile
  static constexpr int TOTAL = LAST_OFF + AT_MAX_TILES * 4 + 1024;
};

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x for a pair of elements. POLY: on the FMA pipe — x = n + f with n the nearest integer (the float trick of
// adding 1.5 * 2^23) and f in [-0.5, 0.5]; 2^f by a cubic fitted to a relative error of 7.5e-5 (P is rounded to
// bf16, 3.9e-3, right after); n goes into the exponent field by integer addition. x below -125 is held there
// (2^-125: nothing, after the rounding of P V and of the row sum).
#ifndef TJX_AT_POLY_PAIRS
#define TJX_AT_POLY_PAIRS 1
#endif
constexpr int AT_POLY_PAIRS = TJX_AT_POLY_PAIRS;  // of every four pairs, how many use the polynomial
__host__ __device__ constexpr bool poly_pair(int pair) {
  return AT_POLY_PAIRS == 4   ? true
         : AT_POLY_PAIRS == 3 ? (pair & 3) != 0
         : AT_POLY_PAIRS == 2 ? (pair & 1) != 0
         : AT_POLY_PAIRS == 1 ? (pair & 3) == 3
                              : false;
}
__device__ __forceinline__ float2 exp2_pair(float2 x, bool poly) {  // `poly` is a constant after unrolling
  if (!poly) {
    return make_float2(fast_exp2(x.x), fast_exp2(x.y));
  } else {
    constexpr float MAGIC = 12582912.f;  // 1.5 * 2^23
    x.x = fmaxf(x.x, -125.f), x.y = fmaxf(x.y, -125.f);
    const float2 t = __fadd2_rn(x, make_float2(MAGIC, MAGIC));
    const float2 n = __fadd2_rn(t, make_float2(-MAGIC, -MAGIC));
    const float2 f = __ffma2_rn(n, make_float2(-1.f, -1.f), x);
    float2 p = __ffma2_rn(f, make_float2(0.05517164617776871f, 0.05517164617776871f),
                          make_float2(0.2426111251115799f, 0.2426111251115799f));
    p = __ffma2_rn(p, f, make_float2(0.6932609677314758f, 0.6932609677314758f));
    p = __ffma2_rn(p, f, make_float2(0.9999280571937561f, 0.9999280571937561f));
    return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23)),
                       __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23)));
  }
}

// Keys a slot's rows [q0, q0 + 128) attend to, as a count of 128-key sub-blocks from key 0: what the step table
// lists for the user tile holding q0 (blocks 0 .. last, contiguous), cut at the slot's own diagonal.
__device__ __forceinline__ int slot_blocks(const AttnParams& p, const int* last_block, int q0) {
  if (q0 >= p.S) return 0;
  const int last = last_block[q0 / p.bq];
  const int keys = min(min((last + 1) * p.bk, q0 + AT_BQ), p.S);
  return keys / AT_BKV;
}

// PAGED: ragged paged attention's prefill case on the same pipeline. A unit is (tile of up to 128 query tokens of one
// sequence, KV head, pair of that KV head's query heads): the two slots are two query heads over the same tokens, so
// they share every K / V block as the two query tiles of the dense kernel do; a block is one 128-position page of the
// cache (pages, 128, Hkv, 2, D), found through page_indices; the tile's first token sits at cache position
// tile_pos and token r sees the positions up to tile_pos + r; the outputs replace the queries' rows.
// PROFILE: the instantiation a launch with a profile buffer runs; it alone reads the clock and keeps the counters
// (they cost the softmax warps registers they do not have to spare: 7 % of the kernel's time when always on).
template <bool PROFILE, bool PAGED>
__global__ void __launch_bounds__(AT_THREADS, 1)
    attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  using L = AttnSmem;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_base = base + L::BAR_OFF;
  // barriers: q_full[2], k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_ready[2], o_done[2], q_empty[2],
  // p_half[2]
  auto q_full = [&](int t) { return bar_base + 8u * t; };
  auto k_full = [&](int s) { return bar_base + 8u * (2 + s); };
  auto k_empty = [&](int s) { return bar_base + 8u * (4 + s); };
  auto v_full = [&](int s) { return bar_base + 8u * (6 + s); };
  auto v_empty = [&](int s) { return bar_base + 8u * (8 + s); };
  auto s_full = [&](int t) { return bar_base + 8u * (10 + t); };
  auto p_ready = [&](int t) { return bar_base + 8u * (12 + t); };
  auto o_done = [&](int t) { return bar_base + 8u * (14 + t); };
  auto q_empty = [&](int t) { return bar_base + 8u * (16 + t); };
  auto p_half = [&](int t) { return bar_base + 8u * (18 + t); };
  constexpr int N_BARS = 20;
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(base_ptr + L::BAR_OFF + 8 * N_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L::BAR_OFF + 8 * N_BARS + 8);
  int* last_block = reinterpret_cast<int*>(base_ptr + L::LAST_OFF);

  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
  const int bh_count = p.B * p.H;
  const int n_ctas = static_cast<int>(gridDim.x), cta = static_cast<int>(blockIdx.x);
  const int pairs_per_tile = PAGED ? p.Hkv * (p.group / 2) : 1;
  const int total_units = PAGED ? __shfl_sync(0xFFFFFFFFu, p.n_tiles[0], 0) * pairs_per_tile : p.total_units;
  // The k-th unit of this CTA in the heaviest-first list (later query tiles attend to more keys), or -1.
  auto unit_at = [&](int k) {
    const int i = k * n_ctas + ((k & 1) ? n_ctas - 1 - cta : cta);
    return i < total_units ? i : -1;
  };

  long long* prof = !PROFILE || p.profile == nullptr ? nullptr
                        : p.profile + static_cast<size_t>(blockIdx.x) * PROFILE_WORDS;
  if (PROFILE && prof != nullptr && threadIdx.x == 0) prof[0] = clock64();
  if (threadIdx.x == 0) {
    for (int i = 0; i < N_BARS; ++i) {
      const bool softmax_bar = i == 12 || i == 13 || i >= 18;  // p_ready, p_half: one arrival per softmax warp
      mbar_init(bar_base + 8u * i, softmax_bar ? 4 : 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  if (!PAGED) {
    // Last key block the step table lists for each user query tile (-1: none).
    for (int i = threadIdx.x; i < p.pattern_tiles; i += AT_THREADS) last_block[i] = -1;
    __syncthreads();
    for (int s = threadIdx.x; s < p.pattern_steps; s += AT_THREADS) {
      const int code = p.step_code[s], tile = p.step_tile[s];
      if (!(code & 4) && tile >= 0 && tile < p.pattern_tiles) atomicMax(&last_block[tile], code >> 3);
    }
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xFFFFFFFFu, *tmem_holder, 0);
  if (p.chain & CHAIN_WAITS) chain_wait();
  if (p.chain & CHAIN_RELEASES) chain_release();

  // What every role derives for a unit, identically.
  struct Unit {
    int row_base, q0[2], n_slot[2], n_blocks;
    int tok0, rows, head[2], kv_head, page0;  // paged: the tile's first token and tokens, the slots' query heads, ...
  };
  auto describe = [&](int i) {
    Unit u;
    if (PAGED) {
      const int tile = i / pairs_per_tile, rem = i % pairs_per_tile;
      u.kv_head = rem / (p.group / 2);
      u.head[0] = u.kv_head * p.group + 2 * (rem % (p.group / 2)), u.head[1] = u.head[0] + 1;
      u.tok0 = p.tile_row0[tile], u.rows = p.tile_rows[tile], u.page0 = p.tile_page[tile];
      u.q0[0] = u.q0[1] = p.tile_pos[tile];  // the cache position of the slots' first row
      u.row_base = 0;
      u.n_slot[0] = u.n_slot[1] = u.n_blocks = (u.q0[0] + u.rows + AT_BKV - 1) / AT_BKV;
      return u;
    }
    u.tok0 = u.rows = u.head[0] = u.head[1] = u.kv_head = u.page0 = 0;
    const int unit = p.units_per_bh - 1 - i / bh_count;
    const int bh = i % bh_count;
    u.row_base = bh * p.S;  // row of (b, h, 0) in the [B * H * S, D] view
    u.q0[0] = unit * 2 * AT_BQ, u.q0[1] = unit * 2 * AT_BQ + AT_BQ;
    u.n_slot[0] = slot_blocks(p, last_block, u.q0[0]);
    u.n_slot[1] = slot_blocks(p, last_block, u.q0[1]);
    u.n_blocks = max(u.n_slot[0], u.n_slot[1]);
    return u;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int g = 0;          // K/V blocks loaded so far (ring position)
      int used[2] = {0, 0};  // units that used slot t so far
      bool ok = true;
      for (int k = 0; ok; ++k) {
        const int i = unit_at(k);
        if (i < 0) break;
        const Unit u = describe(i);
        for (int t = 0; t < 2 && ok; ++t) {
          if (u.n_slot[t] == 0) continue;
          // The previous unit's last Q K^T of this slot has read the tile.
          if (!mbar_wait(q_empty(t), (used[t] & 1) ^ 1u, abort_flag, p.status, TJX_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          ++used[t];
          const uint32_t dst = base + L::Q_OFF + t * L::TILE_BYTES;
          mbar_expect_tx(q_full(t), L::TILE_BYTES);
          if (PAGED) {  // q as (D, H, T): 128 tokens of one head
            tma_load_3d(dst, &map_q, 0, u.head[t], u.tok0, q_full(t));
            tma_load_3d(dst + L::TILE_BYTES / 2, &map_q, 64, u.head[t], u.tok0, q_full(t));
          } else {
            tma_load_2d(dst, &map_q, 0, u.row_base + u.q0[t], q_full(t));
            tma_load_2d(dst + L::TILE_BYTES / 2, &map_q, 64, u.row_base + u.q0[t], q_full(t));
          }
        }
        for (int n = 0; n < u.n_blocks && ok; ++n, ++g) {
          const int stage = g % AT_STAGES;
          const uint32_t ph = (g / AT_STAGES) & 1;
          const int kv_row = u.row_base + n * AT_BKV;
          if (!mbar_wait(k_empty(stage), ph ^ 1u, abort_flag, p.status, TJX_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t kd = base + L::K_OFF + stage * L::TILE_BYTES;
          // Paged: block n is page page_indices[page0 + n] of the cache seen as (D, Hkv * 2, pages * 128), the key
          // of KV head g at index 2 g of the middle dimension, its value at 2 g + 1.
          const int page_row = PAGED ? min(max(p.page_indices[min(max(u.page0 + n, 0), p.n_page_indices - 1)], 0),
                                               p.num_pages - 1) * AT_BKV : 0;  // index and page clamped, as a gather's are
          mbar_expect_tx(k_full(stage), L::TILE_BYTES);
          if (PAGED) {
            tma_load_3d(kd, &map_k, 0, 2 * u.kv_head, page_row, k_full(stage));
            tma_load_3d(kd + L::TILE_BYTES / 2, &map_k, 64, 2 * u.kv_head, page_row, k_full(stage));
          } else {
            tma_load_2d(kd, &map_k, 0, kv_row, k_full(stage));
            tma_load_2d(kd + L::TILE_BYTES / 2, &map_k, 64, kv_row, k_full(stage));
          }
          if (!mbar_wait(v_empty(stage), ph ^ 1u, abort_flag, p.status, TJX_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t vd = base + L::V_OFF + stage * L::TILE_BYTES;
          mbar_expect_tx(v_full(stage), L::TILE_BYTES);
          if (PAGED) {
            tma_load_3d(vd, &map_v, 0, 2 * u.kv_head + 1, page_row, v_full(stage));
            tma_load_3d(vd + L::TILE_BYTES / 2, &map_v, 64, 2 * u.kv_head + 1, page_row, v_full(stage));
          } else {
            tma_load_2d(vd, &map_v, 0, kv_row, v_full(stage));
            tma_load_2d(vd + L::TILE_BYTES / 2, &map_v, 64, kv_row, v_full(stage));
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (whole warp; one lane issues)
    {
      const uint32_t idesc_qk = idesc_bf16_f32(128, 128, 0, 0);  // Q and K both K-major (K read "transposed")
      const uint32_t idesc_pv = idesc_bf16_f32(128, 128, 0, 1);  // P from TMEM, V MN-major
      int g0 = 0;            // ring position of the current unit's block 0
      int used[2] = {0, 0};  // units that used slot t so far
      int done[2] = {0, 0};  // blocks of slot t in earlier units (phase of s_full / p_ready / o_done)
      auto commit = [&](uint32_t bar) {
        if (elect_one()) mma_commit(bar);
      };
      long long issue_cyc = 0, issue_first = 0, issue_n = 0;
      auto issue_qk = [&](int t, int gn) {
        const long long c0 = PROFILE ? clock64() : 0;
        const int stage = gn % AT_STAGES;
        const uint32_t qa = base + L::Q_OFF + t * L::TILE_BYTES;
        const uint32_t ka = base + L::K_OFF + stage * L::TILE_BYTES;
        // The k-th 16-wide slice of a 128-byte-swizzled K-major tile: 32 bytes further along the row, the second
        // 64-column box after the first. (Descriptor addresses count 16 bytes; no carry out of their 14 bits.)
        const uint64_t q0 = smem_desc_sw128(qa, 16, 1024), k0 = smem_desc_sw128(ka, 16, 1024);
        uint64_t qd[8], kd[8];
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = ((kk >> 2) * (L::TILE_BYTES / 2) + (kk & 3) * 32) >> 4;
          qd[kk] = q0 + off, kd[kk] = k0 + off;
        }
        mma_ss_x8_commit(tmem_base + t * 128, qd, kd, idesc_qk, 0u, s_full(t));
        if (PROFILE) {
          const long long dt = clock64() - c0;
          if (issue_n++ == 0) issue_first = dt;
          issue_cyc += dt;
        }
      };
      // P V in two halves: keys 0..63 of the block as soon as their probabilities are in TMEM, the rest (and the
      // commit) when the block's are all there.
      auto issue_pv = [&](int t, int gn, bool first, int half) {
        const int stage = gn % AT_STAGES;
        const uint32_t va = base + L::V_OFF + stage * L::TILE_BYTES;
        const uint64_t v0 = smem_desc_sw128(va, L::TILE_BYTES / 2, 1024);
        uint64_t vd[4];
        uint32_t pa[4];
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          vd[kk] = v0 + (((half * 4 + kk) * 16 * 128) >> 4);
          pa[kk] = tmem_base + t * 128 + (half * 4 + kk) * 8;
        }
        if (half == 0)
          mma_ts_x4(tmem_base + 256 + t * 128, pa, vd, idesc_pv, first ? 0u : 1u);
        else
          mma_ts_x4_commit(tmem_base + 256 + t * 128, pa, vd, idesc_pv, 1u, o_done(t));
      };
      bool ok = true;
      long long t_first = 0, in_wait = 0, fill_wait = -1, p_wait = 0, units = 0;
      // Every lane waits; the vote makes the outcome one value for the warp, so the loops below stay uniform.
      auto wait = [&](uint32_t bar, uint32_t parity, int code, long long& waited) {
        return __all_sync(0xFFFFFFFFu, mbar_wait_timed(bar, parity, abort_flag, p.status, code, waited, PROFILE && prof != nullptr)) != 0;
      };
      for (int k = 0; ok; ++k) {
        const int i = unit_at(k);
        if (i < 0) break;
        Unit u = describe(i);
        // (Read from shared memory: the same in every lane, and said so to the compiler.)
        u.n_slot[0] = __shfl_sync(0xFFFFFFFFu, u.n_slot[0], 0), u.n_slot[1] = __shfl_sync(0xFFFFFFFFu, u.n_slot[1], 0);
        u.n_blocks = max(u.n_slot[0], u.n_slot[1]);
        if (PROFILE && units++ == 0) t_first = clock64();
        for (int t = 0; t < 2 && ok; ++t)
          if (u.n_slot[t] > 0) ok = wait(q_full(t), used[t] & 1, TJX_ERR_WAIT_FULL, in_wait);
        if (ok && u.n_blocks > 0) {
          ok = wait(k_full(g0 % AT_STAGES), (g0 / AT_STAGES) & 1, TJX_ERR_WAIT_FULL, in_wait);
          if (PROFILE && fill_wait < 0) fill_wait = in_wait;
          if (ok) {
            tc_fence_after_sync();
            for (int t = 0; t < 2; ++t)
              if (u.n_slot[t] > 0) {
                issue_qk(t, g0);
                if (u.n_slot[t] == 1) commit(q_empty(t));  // this slot's only Q K^T of the unit
              }
            commit(k_empty(g0 % AT_STAGES));
          }
        }
        for (int n = 0; n < u.n_blocks && ok; ++n) {
          const int gn = g0 + n;
          const int stage = gn % AT_STAGES;
          if (!wait(v_full(stage), (gn / AT_STAGES) & 1, TJX_ERR_WAIT_FULL, in_wait)) {
            ok = false;
            break;
          }
          bool next_k_waited = false, next_k_used = false;
          for (int t = 0; t < 2 && ok; ++t) {
            if (n >= u.n_slot[t]) continue;
            // Softmax warps reach block 0 of a unit only after their epilogue of the previous one, so this wait
            // also covers "O of the previous unit has been read".
            if (!wait(p_half(t), (done[t] + n) & 1, TJX_ERR_WAIT_OTHER, p_wait)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            issue_pv(t, gn, n == 0, 0);
            if (!wait(p_ready(t), (done[t] + n) & 1, TJX_ERR_WAIT_OTHER, p_wait)) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
            issue_pv(t, gn, n == 0, 1);
            if (n + 1 < u.n_slot[t]) {
              if (!next_k_waited) {
                const int ns = (gn + 1) % AT_STAGES;
                if (!wait(k_full(ns), ((gn + 1) / AT_STAGES) & 1, TJX_ERR_WAIT_FULL, in_wait)) {
                  ok = false;
                  break;
                }
                tc_fence_after_sync();
                next_k_waited = true;
              }
              issue_qk(t, gn + 1);
              if (n + 2 == u.n_slot[t]) commit(q_empty(t));  // that was this slot's last Q K^T of the unit
              next_k_used = true;
            }
          }
          if (!ok) break;
          commit(v_empty(stage));
          if (next_k_used) commit(k_empty((gn + 1) % AT_STAGES));
        }
        g0 += u.n_blocks;
        for (int t = 0; t < 2; ++t) {
          done[t] += u.n_slot[t];
          if (u.n_slot[t] > 0) ++used[t];
        }
      }
      if (PROFILE && prof != nullptr && lane == 0) {
        prof[1] = t_first, prof[2] = clock64(), prof[3] = in_wait, prof[4] = max(fill_wait, 0ll), prof[5] = 0;
        prof[6] = units, prof[8] = p_wait;
        prof[9] = issue_first, prof[10] = issue_cyc, prof[11] = issue_n;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int t = (warp - 2) >> 2;  // slot
    const int q = warp & 3;         // TMEM lane quarter
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_addr + t * 128;
    const uint32_t o_tmem = tmem_base + lane_addr + 256 + t * 128;
    int done = 0;  // blocks of this slot in earlier units
    bool ok = true;
    const float score_scale = PAGED ? p.scale_log2e : AT_LOG2E;  // scores to base-2 exponents
    long long sm_wait = 0, sm_busy = 0, sm_blocks = 0;
    int ph_ld = 0, ph_max = 0, ph_exp = 0;
    for (int k = 0; ok; ++k) {
    const int i = unit_at(k);
    if (i < 0) break;
    const Unit u = describe(i);
    const int n_mine = u.n_slot[t];
    const int q0 = u.q0[t];
    const int row = q0 + q * 32 + lane;  // query position of this thread's row
    float m_used = AT_MASK * AT_LOG2E;  // running max, in log2 units
    float l = 0.f;
    for (int n = 0; n < n_mine; ++n) {
      const long long w0 = PROFILE ? clock64() : 0;
      const bool got = mbar_wait(s_full(t), (done + n) & 1, abort_flag, p.status, TJX_ERR_WAIT_TMEM_FULL);
      const long long w1 = PROFILE ? clock64() : 0;
      if (PROFILE) sm_wait += w1 - w0, ++sm_blocks;
      if (!__all_sync(0xFFFFFFFFu, got)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int kv0 = n * AT_BKV;
      const bool diagonal = kv0 + AT_BKV - 1 > q0;  // some key of the block is in some row's future
      // The row's 128 scores come into registers once: four TMEM loads in flight, one wait.
      uint32_t v[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(s_tmem + c * 32, v[c]);
      tmem_wait_ld();
      const int c_ld = PROFILE ? clock() : 0;
      if (PROFILE) ph_ld += c_ld - static_cast<int>(w1);
      if (diagonal) {  // only the block on the diagonal holds keys in some row's future
        const int lim = row - kv0;  // columns j <= lim are visible
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c * 32 + j > lim) v[c][j] = __float_as_uint(AT_MASK);
      }
      // Row max over the block: three-input max, four independent chains.
      float mx;
      {
        float m0 = AT_MASK, m1 = AT_MASK, m2 = AT_MASK, m3 = AT_MASK;
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            m0 = fmax3(m0, __uint_as_float(v[c][j]), __uint_as_float(v[c][j + 1]));
            m1 = fmax3(m1, __uint_as_float(v[c][j + 2]), __uint_as_float(v[c][j + 3]));
            m2 = fmax3(m2, __uint_as_float(v[c][j + 4]), __uint_as_float(v[c][j + 5]));
            m3 = fmax3(m3, __uint_as_float(v[c][j + 6]), __uint_as_float(v[c][j + 7]));
          }
        mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      }
      const float m_blk = mx * score_scale;
      if (n == 0) {
        m_used = m_blk;
      } else if (__any_sync(0xFFFFFFFFu, m_blk > m_used + AT_RESCALE_THRESHOLD)) {
        // Raise the running max and rescale what has been accumulated. P V of the previous block finished
        // before this block's scores were produced (the tensor pipe runs one thread's MMAs in order).
        const float m_new = fmaxf(m_used, m_blk);
        const float alpha = fast_exp2(m_used - m_new);
        m_used = m_new;
        l *= alpha;
        const bool od = mbar_wait(o_done(t), (done + n - 1) & 1, abort_flag, p.status, TJX_ERR_WAIT_OTHER);
        if (!__all_sync(0xFFFFFFFFu, od)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld32(o_tmem + c * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
          tmem_st32(o_tmem + c * 32, v);
        }
        tmem_wait_st();
      }
      const int c_max = PROFILE ? clock() : 0;
      if (PROFILE) ph_max += c_max - c_ld;
      // Probabilities; P (bf16) overwrites the first half of the scores' columns (all already in registers). The
      // arithmetic is two elements per instruction, and AT_POLY_PAIRS of every four pairs take their exponential
      // from the FMA pipe instead of the MUFU unit, which two softmax warps per scheduler would otherwise saturate.
      {
        float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
        const float2 scale = make_float2(score_scale, score_scale), neg_m = make_float2(-m_used, -m_used);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const float2 x0 = __ffma2_rn(make_float2(__uint_as_float(v[c][j]), __uint_as_float(v[c][j + 1])), scale, neg_m);
            const float2 x1 = __ffma2_rn(make_float2(__uint_as_float(v[c][j + 2]), __uint_as_float(v[c][j + 3])), scale, neg_m);
            const float2 p0 = exp2_pair(x0, poly_pair(j / 2));
            const float2 p1 = exp2_pair(x1, poly_pair(j / 2 + 1));
            la = __fadd2_rn(la, p0), lb = __fadd2_rn(lb, p1);
            pk[j >> 1] = pack_bf16(p0.x, p0.y);
            pk[(j >> 1) + 1] = pack_bf16(p1.x, p1.y);
          }
          tmem_st16(s_tmem + c * 16, pk);
          if (c == 1) {  // the first 64 keys' probabilities are on their way: P V may begin with them
            tmem_wait_st();
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_half(t));
          }
        }
        l += (la.x + la.y) + (lb.x + lb.y);
      }
      if (PROFILE) ph_exp += clock() - c_max;
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready(t));
      if (PROFILE) sm_busy += clock64() - w1;
    }
    if (ok && n_mine > 0) {
      // Epilogue: O / l -> bf16 -> this thread's row of the output, 256 contiguous bytes.
      const bool od = mbar_wait(o_done(t), (done + n_mine - 1) & 1, abort_flag, p.status, TJX_ERR_WAIT_OTHER);
      if (!__all_sync(0xFFFFFFFFu, od)) {
        ok = false;
      } else {
        tc_fence_after_sync();
        const float inv = 1.0f / l;
        if (PAGED) {
          // Token tok0 + r, head head[t]: 256 contiguous bytes of (T, H, D); rows past the tile's tokens belong to
          // other sequences and are not written (every lane still takes part in the TMEM loads).
          const int r = q * 32 + lane;
          uint4* dst = reinterpret_cast<uint4*>(
              p.out_tokens + (static_cast<size_t>(u.tok0 + r) * p.H + u.head[t]) * AT_D);
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            tmem_ld32(o_tmem + c * 32, v);
            tmem_wait_ld();
            if (r < u.rows) {
#pragma unroll
              for (int x = 0; x < 4; ++x) {
                uint4 val;
                val.x = pack_bf16(__uint_as_float(v[8 * x + 0]) * inv, __uint_as_float(v[8 * x + 1]) * inv);
                val.y = pack_bf16(__uint_as_float(v[8 * x + 2]) * inv, __uint_as_float(v[8 * x + 3]) * inv);
                val.z = pack_bf16(__uint_as_float(v[8 * x + 4]) * inv, __uint_as_float(v[8 * x + 5]) * inv);
                val.w = pack_bf16(__uint_as_float(v[8 * x + 6]) * inv, __uint_as_float(v[8 * x + 7]) * inv);
                dst[c * 4 + x] = val;
              }
            }
          }
        } else if (p.out_heads != nullptr) {
          // Row (b, s) of the (B * S, H * D) f32 matrix, columns h * D .. h * D + 127: 512 contiguous bytes.
          const int bh = u.row_base / p.S, b = bh / p.H, h = bh % p.H;
          float4* dst = reinterpret_cast<float4*>(
              p.out_heads + (static_cast<size_t>(b) * p.S + row) * (static_cast<size_t>(p.H) * AT_D) + h * AT_D);
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            tmem_ld32(o_tmem + c * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 8; ++x)
              dst[c * 8 + x] = make_float4(__uint_as_float(v[4 * x]) * inv, __uint_as_float(v[4 * x + 1]) * inv,
                                           __uint_as_float(v[4 * x + 2]) * inv, __uint_as_float(v[4 * x + 3]) * inv);
          }
        } else {
          uint4* dst = reinterpret_cast<uint4*>(p.out + static_cast<size_t>(u.row_base + row) * AT_D);
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            tmem_ld32(o_tmem + c * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              uint4 val;
              val.x = pack_bf16(__uint_as_float(v[8 * x + 0]) * inv, __uint_as_float(v[8 * x + 1]) * inv);
              val.y = pack_bf16(__uint_as_float(v[8 * x + 2]) * inv, __uint_as_float(v[8 * x + 3]) * inv);
              val.z = pack_bf16(__uint_as_float(v[8 * x + 4]) * inv, __uint_as_float(v[8 * x + 5]) * inv);
              val.w = pack_bf16(__uint_as_float(v[8 * x + 6]) * inv, __uint_as_float(v[8 * x + 7]) * inv);
              dst[c * 4 + x] = val;
            }
          }
        }
        // The reads of O above are ordered before this warp's next arrival on p_ready, which is what the next
        // unit's first P V waits for before it overwrites O.
        tc_fence_before_sync();
      }
    }
    done += n_mine;
    }  // units
    if (PROFILE && prof != nullptr && warp == 2 && lane == 0) {
      prof[12] = sm_busy, prof[13] = sm_wait, prof[14] = sm_blocks;
      prof[15] = (static_cast<long long>(ph_ld) << 42) | (static_cast<long long>(ph_max) << 21) | ph_exp;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (PROFILE && prof != nullptr && threadIdx.x == 0) prof[7] = clock64();
  if (warp == 1) {
    if (*abort_flag) __nanosleep(100000);
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace tjx

namespace tjx {
// The launch behind tjx_causal_attention_bf16 (`out`: (B, H, S, D) bf16) and tjx_attention_block_bf16 (`out_heads`:
// (B, S, H * D) f32); exactly one of the two is given.
int attention_launch(const void* q, const void* k, const void* v, void* out, float* out_heads, int B, int H, int S,
                     int D, int block_q, int block_kv, const int32_t* step_tile, const int32_t* step_code,
                     int pattern_steps, int pattern_tiles, tjx_stream_t stream) {
  if (int rc = check_device()) return rc;
  if (!q || !k || !v || (!out && !out_heads)) return fail(TJX_E_ARG, "q, k, v or out is null");
  if (!step_tile || !step_code || pattern_steps <= 0 || pattern_tiles <= 0)
    return fail(TJX_E_ARG, "the step tables are missing");
  if (B <= 0 || H <= 0 || S <= 0) return fail(TJX_E_ARG, "sizes must be positive");
  if (D != AT_D) return fail(TJX_E_ARG, "head dimension must be 128");
  if (S % 128 != 0) return fail(TJX_E_ARG, "S must be a multiple of 128");
  if (block_q <= 0 || block_kv <= 0 || block_q % 128 != 0 || block_kv % 128 != 0 || S % block_q != 0 || S % block_kv != 0)
    return fail(TJX_E_ARG, "block_q and block_kv must be multiples of 128 that divide S");
  if (pattern_tiles != S / block_q) return fail(TJX_E_ARG, "pattern_tiles must be S / block_q");
  if (static_cast<long long>(B) * H * S >= (1ll << 31)) return fail(TJX_E_LIMIT, "B * H * S must fit in int32");

  AttnParams p{};
  p.B = B, p.H = H, p.S = S, p.bq = block_q, p.bk = block_kv;
  p.pattern_steps = pattern_steps, p.pattern_tiles = pattern_tiles;
  p.step_tile = step_tile, p.step_code = step_code;
  p.units_per_bh = (S / AT_BQ + 1) / 2;
  p.total_units = B * H * p.units_per_bh;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_heads = out_heads;
  if (pattern_tiles > AT_MAX_TILES) return fail(TJX_E_LIMIT, "more than 1024 query tiles per (batch, head)");
  p.status = device_status_word();
  if (p.status == nullptr) return fail(TJX_E_CUDA, "could not locate the device status word");
  p.chain = launch_chain();

  const uint64_t dims[2] = {static_cast<uint64_t>(D), static_cast<uint64_t>(B) * H * S};
  const uint64_t strides[1] = {static_cast<uint64_t>(D) * 2};
  const uint32_t box_in[2] = {64, 128};
  CUtensorMap mq, mk, mv;
  if (int rc = make_tensor_map(&mq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, dims, strides, box_in, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = make_tensor_map(&mk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, dims, strides, box_in, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;
  if (int rc = make_tensor_map(&mv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, dims, strides, box_in, CU_TENSOR_MAP_SWIZZLE_128B)) return rc;

  static bool configured[64] = {};
  int dev = 0;
  TJX_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    TJX_CUDA(cudaFuncSetAttribute(attention_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem::TOTAL));
    TJX_CUDA(cudaFuncSetAttribute(attention_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem::TOTAL));
    configured[dev & 63] = true;
  }
  const int grid = std::min(p.total_units, sm_count());
  p.profile = profile_buffer(grid);
  if (p.profile != nullptr)
    attention_kernel<true, false><<<grid, AT_THREADS, AttnSmem::TOTAL, static_cast<cudaStream_t>(stream)>>>(mq, mk, mv, p);
  else
    attention_kernel<false, false><<<grid, AT_THREADS, AttnSmem::TOTAL, static_cast<cudaStream_t>(stream)>>>(mq, mk, mv, p);
  TJX_CUDA(cudaGetLastError());
  return 0;
}
}  // namespace tjx

namespace tjx {

// Buckets of the tile kernels' counting sort: a tile's key is the number of 128-key blocks it attends to.
constexpr int RPA_SORT_KEYS = 1024;

// Exclusive scan of hist[RPA_SORT_KEYS] in place by a CTA of 256 threads (four buckets a thread).
__device__ __forceinline__ void rpa_scan_buckets(int* hist, int* scan_sh) {
  const int t = threadIdx.x;
  int v[4], sum = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = hist[4 * t + j], sum += v[j];
  scan_sh[t] = sum;
  __syncthreads();
  for (int d = 1; d < 256; d <<= 1) {  // inclusive scan of the threads' sums
    const int y = t >= d ? scan_sh[t - d] : 0;
    __syncthreads();
    scan_sh[t] += y;
    __syncthreads();
  }
  int at = scan_sh[t] - sum;
#pragma unroll
  for (int j = 0; j < 4; ++j) hist[4 * t + j] = at, at += v[j];
  __syncthreads();
}

// Bucket of a tile whose first row sits at cache position pos: longest first.
__device__ __forceinline__ int rpa_bucket(int pos, int rows) {
  const int blocks = (max(pos, 0) + rows + AT_BKV - 1) / AT_BKV;
  return RPA_SORT_KEYS - 1 - min(blocks, RPA_SORT_KEYS - 1);
}

// The prefill tiles of one step, on the device (what `prefill_tiles` computes in plain JAX,
// examples/ragged_paged_attention.py:252-275, for blocks of 128 queries): a tile per block of 128 new tokens of each
// sequence in [distribution[0], distribution[2]), listed longest first (by the key blocks a tile attends to: the
// attention kernel deals its units out in list order, and a short last round should hold the lightest). One CTA;
// thread s handles sequences s, s + 256, ...; a counting sort: one pass counts the tiles of every length, a scan
// gives each length its first slot, a second pass writes every tile to the next slot of its length.
__global__ void __launch_bounds__(256)
    rpa_prefill_tiles_kernel(const int32_t* __restrict__ kv_lens, const int32_t* __restrict__ cu_q_lens,
                             const int32_t* __restrict__ distribution, int S, int pages_per_seq, int max_tiles,
                             int32_t* __restrict__ tile_row0, int32_t* __restrict__ tile_rows,
                             int32_t* __restrict__ tile_pos, int32_t* __restrict__ tile_page,
                             int32_t* __restrict__ n_tiles) {
  __shared__ int hist[RPA_SORT_KEYS], scan_sh[256], total_sh;
  chain_release();  // (reads only the call's inputs: when chained it runs beside the kernel in front of it)
  for (int i = threadIdx.x; i < RPA_SORT_KEYS; i += 256) hist[i] = 0;
  if (threadIdx.x == 0) total_sh = 0;
  __syncthreads();
  const int d0 = distribution[0], d2 = min(distribution[2], S);
  for (int pass = 0; pass < 2; ++pass) {
    for (int s = threadIdx.x; s < S; s += 256) {
      const int q_len = cu_q_lens[s + 1] - cu_q_lens[s];
      const int mine = (s >= d0 && s < d2 && q_len > 0) ? (q_len + AT_BQ - 1) / AT_BQ : 0;
      for (int b = 0; b < mine; ++b) {
        const int pos = kv_lens[s] - q_len + b * AT_BQ, rows = min(AT_BQ, q_len - b * AT_BQ);
        if (pass == 0) {
          atomicAdd(&hist[rpa_bucket(pos, rows)], 1);
        } else {
          const int k = atomicAdd(&hist[rpa_bucket(pos, rows)], 1);
          if (k >= max_tiles) continue;
          tile_row0[k] = cu_q_lens[s] + b * AT_BQ;
          tile_rows[k] = rows;
          tile_pos[k] = pos;
          tile_page[k] = s * pages_per_seq;
        }
      }
      if (pass == 0 && mine > 0) atomicAdd(&total_sh, mine);
    }
    __syncthreads();
    if (pass == 0) rpa_scan_buckets(hist, scan_sh);
  }
  if (threadIdx.x == 0) n_tiles[0] = min(total_sh, max_tiles);
  chain_wait();  // ends after the kernel it was chained behind: what follows this one follows that one too
}

// The tiles of the reference's `rpa_prefill` kernel (examples/ragged_paged_attention.py:204-243: tile k is the query
// rows tile_rows[k] .. tile_rows[k + 1] - 1, up to 256 of them, the first at cache position tile_pos[k], of the
// sequence whose pages start at page_indices[tile_page[k]]) cut into this kernel's tiles of 128 queries. One CTA;
// thread t handles tiles t, t + 256, ...; an exclusive scan of their piece counts gives each its first piece.
__global__ void __launch_bounds__(256)
    rpa_split_tiles_kernel(const int32_t* __restrict__ in_page, const int32_t* __restrict__ in_rows,
                           const int32_t* __restrict__ in_pos, const int32_t* __restrict__ in_count, int max_in,
                           int max_tiles, int T, int32_t* __restrict__ tile_row0, int32_t* __restrict__ tile_rows,
                           int32_t* __restrict__ tile_pos, int32_t* __restrict__ tile_page,
                           int32_t* __restrict__ n_tiles) {
  __shared__ int carry_sh, scan_sh[256];
  if (threadIdx.x == 0) carry_sh = 0;
  __syncthreads();
  const int count = min(max(in_count[0], 0), max_in);
  for (int k0 = 0; k0 < count; k0 += 256) {
    const int k = k0 + threadIdx.x;
    int first_row = 0, rows = 0;
    if (k < count) {
      first_row = in_rows[k];
      rows = in_rows[k + 1] - first_row;
      if (first_row < 0 || rows < 0 || first_row + rows > T) rows = 0;  // not a range of q's rows: nothing to do
    }
    const int mine = (rows + AT_BQ - 1) / AT_BQ;
    scan_sh[threadIdx.x] = mine;
    __syncthreads();
    for (int d = 1; d < 256; d <<= 1) {  // inclusive scan
      const int y = threadIdx.x >= d ? scan_sh[threadIdx.x - d] : 0;
      __syncthreads();
      scan_sh[threadIdx.x] += y;
      __syncthreads();
    }
    const int first = carry_sh + scan_sh[threadIdx.x] - mine;
    for (int b = 0; b < mine; ++b) {
      const int out = first + b;
      if (out >= max_tiles) break;
      tile_row0[out] = first_row + b * AT_BQ;
      tile_rows[out] = min(AT_BQ, rows - b * AT_BQ);
      tile_pos[out] = max(in_pos[k], 0) + b * AT_BQ;  // (a position before the cache's start is not one)
      tile_page[out] = in_page[k];
    }
    __syncthreads();
    if (threadIdx.x == 255) carry_sh += scan_sh[255];
    __syncthreads();
  }
  if (threadIdx.x == 0) n_tiles[0] = min(carry_sh, max_tiles);
}

static size_t attn_align256(size_t n) { return (n + 255) & ~static_cast<size_t>(255); }

// The workspace's tile arrays (max_tiles entries each, then the count) as the kernel's parameters.
static void rpa_tile_arrays(AttnParams& p, void* workspace, int max_tiles) {
  uint8_t* w = static_cast<uint8_t*>(workspace);
  const size_t stride = attn_align256(static_cast<size_t>(max_tiles) * 4);
  p.tile_row0 = reinterpret_cast<int32_t*>(w), p.tile_rows = reinterpret_cast<int32_t*>(w + stride);
  p.tile_pos = reinterpret_cast<int32_t*>(w + 2 * stride), p.tile_page = reinterpret_cast<int32_t*>(w + 3 * stride);
  p.n_tiles = reinterpret_cast<int32_t*>(w + 4 * stride);
}

static int rpa_prefill_check(const void* q, const void* out, const void* kv_cache, const void* page_indices, int T,
                             int H, int Hkv, int D, int page_size, int num_pages) {
  if (!q || !out || !kv_cache || !page_indices) return fail(TJX_E_ARG, "an input or output pointer is null");
  if (T <= 0 || H <= 0 || Hkv <= 0 || num_pages <= 0) return fail(TJX_E_ARG, "sizes must be positive");
  if (D != AT_D) return fail(TJX_E_ARG, "head dimension must be 128");
  if (page_size != AT_BKV) return fail(TJX_E_ARG, "the prefill kernel takes pages of 128 positions");
  if (H % Hkv != 0 || (H / Hkv) % 2 != 0)
    return fail(TJX_E_ARG, "the prefill kernel takes an even number of query heads per KV head (two share each K / V block)");
  if (static_cast<long long>(num_pages) * page_size >= (1ll << 31) || static_cast<long long>(T) * H >= (1ll << 31))
    return fail(TJX_E_LIMIT, "num_pages * page_size and T * H must fit in int32");
  return 0;
}

// The paged attention launch over the tiles `p` lists (at most max_tiles of them, counted in p.n_tiles on the device).
static int rpa_prefill_launch(AttnParams& p, void* out, const void* kv_cache, const int32_t* page_indices,
                              int n_page_indices, int T, int H, int Hkv, int num_pages, float sm_scale, int max_tiles,
                              cudaStream_t s, const void* queries = nullptr) {
  if (queries == nullptr) queries = out;
  p.B = 1, p.H = H, p.S = 0, p.bq = p.bk = AT_BQ;
  p.page_indices = page_indices, p.Hkv = Hkv, p.group = H / Hkv, p.num_pages = num_pages;
  p.n_page_indices = n_page_indices;
  p.scale_log2e = AT_LOG2E * sm_scale;
  p.out_tokens = static_cast<__nv_bfloat16*>(out);
  p.status = device_status_word();
  if (p.status == nullptr) return fail(TJX_E_CUDA, "could not locate the device status word");
  // q (T, H, D) as (D, H, T); the cache (pages, 128, Hkv, 2, D) as (D, Hkv * 2, pages * 128). Unless the caller names
  // another buffer the queries are read from `out`: the rows the decode case has already replaced are not query
  // tiles of this case.
  CUtensorMap mq, mkv;
  {
    const uint64_t dims[3] = {AT_D, static_cast<uint64_t>(H), static_cast<uint64_t>(T)};
    const uint64_t strides[2] = {AT_D * 2, static_cast<uint64_t>(H) * AT_D * 2};
    const uint32_t box[3] = {64, 1, AT_BQ};
    if (int rc = make_tensor_map(&mq, queries, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const uint64_t dims[3] = {AT_D, static_cast<uint64_t>(Hkv) * 2, static_cast<uint64_t>(num_pages) * AT_BKV};
    const uint64_t strides[2] = {AT_D * 2, static_cast<uint64_t>(Hkv) * 2 * AT_D * 2};
    const uint32_t box[3] = {64, 1, AT_BKV};
    if (int rc = make_tensor_map(&mkv, kv_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  static bool configured[64] = {};
  int dev = 0;
  TJX_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    TJX_CUDA(cudaFuncSetAttribute(attention_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem::TOTAL));
    configured[dev & 63] = true;
  }
  const long long bound = static_cast<long long>(max_tiles) * Hkv * (p.group / 2);
  const int grid = static_cast<int>(std::min<long long>(bound, sm_count()));
  p.chain = launch_chain();
  if (p.chain & CHAIN_WAITS) {
    TJX_CUDA(launch_chained(attention_kernel<false, true>, dim3(grid), dim3(AT_THREADS), AttnSmem::TOTAL, s, mq, mkv, mkv, p));
  } else {
    attention_kernel<false, true><<<grid, AT_THREADS, AttnSmem::TOTAL, s>>>(mq, mkv, mkv, p);
    TJX_CUDA(cudaGetLastError());
  }
  return 0;
}

size_t rpa_prefill_part_bytes(int T, int S) {
  const size_t max_tiles = static_cast<size_t>((T + AT_BQ - 1) / AT_BQ) + S;
  return 4 * attn_align256(max_tiles * 4) + 256;
}

int rpa_prefill_part_check(const void* q, const void* out, const void* kv_cache, const void* page_indices, int T, int S,
                           int H, int Hkv, int D, int page_size, int pages_per_seq, int num_pages) {
  if (S <= 0 || pages_per_seq <= 0) return fail(TJX_E_ARG, "sizes must be positive");
  return rpa_prefill_check(q, out, kv_cache, page_indices, T, H, Hkv, D, page_size, num_pages);
}

int rpa_prefill_tiles_part(const int32_t* kv_lens, const int32_t* cu_q_lens, const int32_t* distribution, int T, int S,
                           int pages_per_seq, void* workspace, cudaStream_t stream, RpaTiles* tiles) {
  const int max_tiles = (T + AT_BQ - 1) / AT_BQ + S;
  AttnParams p{};
  rpa_tile_arrays(p, workspace, max_tiles);
  TJX_CUDA(launch_chained(rpa_prefill_tiles_kernel, dim3(1), dim3(256), 0, stream, kv_lens, cu_q_lens, distribution, S,
                          pages_per_seq, max_tiles, const_cast<int32_t*>(p.tile_row0), const_cast<int32_t*>(p.tile_rows),
                          const_cast<int32_t*>(p.tile_pos), const_cast<int32_t*>(p.tile_page),
                          const_cast<int32_t*>(p.n_tiles)));
  tiles->row0 = p.tile_row0, tiles->rows = p.tile_rows, tiles->count = p.n_tiles, tiles->max_tiles = max_tiles;
  return 0;
}

int rpa_prefill_attention_part(const void* q, void* out, const void* kv_cache, const int32_t* page_indices, int T, int S,
                               int H, int Hkv, int pages_per_seq, int num_pages, float sm_scale, void* workspace,
                               cudaStream_t stream) {
  const int max_tiles = (T + AT_BQ - 1) / AT_BQ + S;
  AttnParams p{};
  rpa_tile_arrays(p, workspace, max_tiles);
  return rpa_prefill_launch(p, out, kv_cache, page_indices, S * pages_per_seq, T, H, Hkv, num_pages, sm_scale, max_tiles,
                            stream, q);
}

}  // namespace tjx

extern "C" size_t tjx_rpa_prefill_workspace_bytes(int T, int S) {
  if (T <= 0 || S <= 0) return 0;
  const size_t max_tiles = static_cast<size_t>((T + tjx::AT_BQ - 1) / tjx::AT_BQ) + S;
  return 4 * tjx::attn_align256(max_tiles * 4) + 256;
}

extern "C" int tjx_rpa_prefill_bf16(const void* q, void* out, const void* kv_cache, const int32_t* kv_lens,
                                    const int32_t* page_indices, const int32_t* cu_q_lens,
                                    const int32_t* distribution, int T, int S, int H, int Hkv, int D, int page_size,
                                    int pages_per_seq, int num_pages, float sm_scale, void* workspace,
                                    size_t workspace_bytes, tjx_stream_t stream) {
  using namespace tjx;
  if (int rc = check_device()) return rc;
  if (!kv_lens || !cu_q_lens || !distribution) return fail(TJX_E_ARG, "an input or output pointer is null");
  if (S <= 0 || pages_per_seq <= 0) return fail(TJX_E_ARG, "sizes must be positive");
  if (int rc = rpa_prefill_check(q, out, kv_cache, page_indices, T, H, Hkv, D, page_size, num_pages)) return rc;
  const size_t need = tjx_rpa_prefill_workspace_bytes(T, S);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(TJX_E_ARG, "workspace is null or smaller than tjx_rpa_prefill_workspace_bytes");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(TJX_E_ARG, "workspace must be 256-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out != q)  // rows no tile covers keep what q holds (the decode case's outputs among them)
    TJX_CUDA(cudaMemcpyAsync(out, q, static_cast<size_t>(T) * H * AT_D * 2, cudaMemcpyDeviceToDevice, s));
  const int max_tiles = (T + AT_BQ - 1) / AT_BQ + S;
  AttnParams p{};
  rpa_tile_arrays(p, workspace, max_tiles);
  rpa_prefill_tiles_kernel<<<1, 256, 0, s>>>(kv_lens, cu_q_lens, distribution, S, pages_per_seq, max_tiles,
                                             const_cast<int32_t*>(p.tile_row0), const_cast<int32_t*>(p.tile_rows),
                                             const_cast<int32_t*>(p.tile_pos), const_cast<int32_t*>(p.tile_page),
                                             const_cast<int32_t*>(p.n_tiles));
  TJX_CUDA(cudaGetLastError());
  return rpa_prefill_launch(p, out, kv_cache, page_indices, S * pages_per_seq, T, H, Hkv, num_pages, sm_scale, max_tiles, s);
}

extern "C" size_t tjx_rpa_prefill_tiles_workspace_bytes(int T, int max_tiles) {
  if (T <= 0 || max_tiles <= 0) return 0;
  const size_t pieces = static_cast<size_t>((T + tjx::AT_BQ - 1) / tjx::AT_BQ) + max_tiles;
  return 4 * tjx::attn_align256(pieces * 4) + 256;
}

extern "C" int tjx_rpa_prefill_tiles_bf16(const void* q, void* out, const void* kv_cache, const int32_t* page_indices,
                                          const int32_t* tile_page, const int32_t* tile_rows, const int32_t* tile_pos,
                                          const int32_t* n_tiles, int T, int max_tiles, int n_page_indices, int H,
                                          int Hkv, int D, int page_size, int num_pages, float sm_scale, void* workspace,
                                          size_t workspace_bytes, tjx_stream_t stream) {
  using namespace tjx;
  if (int rc = check_device()) return rc;
  if (!tile_page || !tile_rows || !tile_pos || !n_tiles) return fail(TJX_E_ARG, "a tile table pointer is null");
  if (max_tiles <= 0 || n_page_indices <= 0) return fail(TJX_E_ARG, "sizes must be positive");
  if (int rc = rpa_prefill_check(q, out, kv_cache, page_indices, T, H, Hkv, D, page_size, num_pages)) return rc;
  const size_t need = tjx_rpa_prefill_tiles_workspace_bytes(T, max_tiles);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(TJX_E_ARG, "workspace is null or smaller than tjx_rpa_prefill_tiles_workspace_bytes");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(TJX_E_ARG, "workspace must be 256-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out != q) TJX_CUDA(cudaMemcpyAsync(out, q, static_cast<size_t>(T) * H * AT_D * 2, cudaMemcpyDeviceToDevice, s));
  const int pieces = (T + AT_BQ - 1) / AT_BQ + max_tiles;
  AttnParams p{};
  rpa_tile_arrays(p, workspace, pieces);
  rpa_split_tiles_kernel<<<1, 256, 0, s>>>(tile_page, tile_rows, tile_pos, n_tiles, max_tiles, pieces, T,
                                           const_cast<int32_t*>(p.tile_row0), const_cast<int32_t*>(p.tile_rows),
                                           const_cast<int32_t*>(p.tile_pos), const_cast<int32_t*>(p.tile_page),
                                           const_cast<int32_t*>(p.n_tiles));
  TJX_CUDA(cudaGetLastError());
  return rpa_prefill_launch(p, out, kv_cache, page_indices, n_page_indices, T, H, Hkv, num_pages, sm_scale, pieces, s);
}

extern "C" int tjx_causal_attention_bf16(const void* q, const void* k, const void* v, void* out, int B, int H, int S,
                                         int D, int block_q, int block_kv, const int32_t* step_tile,
                                         const int32_t* step_code, int pattern_steps, int pattern_tiles,
                                         tjx_stream_t stream) {
  if (!out) return tjx::fail(TJX_E_ARG, "q, k, v or out is null");
  return tjx::attention_launch(q, k, v, out, nullptr, B, H, S, D, block_q, block_kv, step_tile, step_code, pattern_steps,
                               pattern_tiles, stream);
}

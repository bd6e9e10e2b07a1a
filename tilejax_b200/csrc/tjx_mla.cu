// Absorbed MLA decode attention on sm_100a, `mla_decode` (examples/decode.py:226-250): the rows of a sequence are its
// (new token, head) pairs, token-major, and new token t of T sees the cache positions up to lengths[b] - T + t
// (`visible`, examples/decode.py:145-152). Every query head scores the same latent cache (512 latents + 128 RoPE columns per position) and the
// output of a head is its softmax-weighted latents, so a position's 1280 bytes are read once for all the heads of
// a head group.
//
// Two kernels: the tcgen05 one further down (the default) and the warp-level one described here (kept behind
// tjx_mla_set_mode(0), and used for more than 2048 sequences).
//
// Work = the device step table built from `lengths` (tjx_steps.cu): a step is one block of `block` cache
// positions of one sequence. A CTA takes one step and one group of 16 heads — the 16 rows of a warp-level MMA
// (mma.sync m16n8k16, bf16 -> f32). The block streams through a CTA-wide ring of shared-memory slots, 16
// positions (20 KB) at a time, loaded by TMA as ten 128-byte-swizzled boxes [16 positions x 64 columns]. The four
// warps split the work of a 16-position micro-step by columns:
//   scores  warp w multiplies the queries' latent columns 128 w .. 128 w + 127 and RoPE columns 32 w .. 32 w + 31
//           (B fragments by ldmatrix) -> a partial 16 x 16 score tile; the four partials meet in shared memory
//           and every warp adds them in the same order, so all warps hold the same scores
//   softmax in every warp (online, f32, exp2 with log2 e folded in), probabilities rounded to bf16 as the reference
//           rounds them, already in A-fragment layout
//   output  warp w accumulates latent columns 128 w .. 128 w + 127 of the 16 heads (B fragments by ldmatrix.trans
//           from the same slot)
// A step that is its sequence's only one is normalised and written at once; otherwise the CTA writes a partial
// (max, sum, accumulator), counts itself on the (sequence, head group) arrival counter, and the CTA that arrives
// last merges the partials — the scheme of the GQA decode kernel (tjx_decode.cu).
#include <algorithm>

#include "tjx_host.cuh"
#include "tjx_ptx.cuh"

#include "../../include/tilejax_b200.h"

namespace tjx {

int launch_build_steps_lengths(const int32_t* lengths, int n_lengths, const int32_t* tile_values, int tiles,
                               int blocks, int value0, int value_step, int32_t* step_tile, int32_t* step_code,
                               int32_t* step_count, int32_t* tile_first, int32_t* zero_words, int n_zero,
                               cudaStream_t stream);

constexpr int MLA_C = 512;       // latent columns
constexpr int MLA_R = 128;       // RoPE columns as stored (the upper 64 are zero padding in the reference's caches)
constexpr int MLA_HEADS = 16;    // heads per CTA: the rows of one MMA
constexpr int MLA_SUB = 16;      // positions per micro-step
constexpr int MLA_WARPS = 4;
constexpr int MLA_STAGES = 3;
constexpr int MLA_BOX_BYTES = MLA_SUB * 64 * 2;                 // one box: 16 positions x 64 columns
constexpr int MLA_BOXES = MLA_C / 64 + MLA_R / 64;              // 8 latent + 2 RoPE
constexpr int MLA_STAGE_BYTES = MLA_BOXES * MLA_BOX_BYTES;      // 20 KB
constexpr int MLA_XCH_BYTES = 2 * MLA_WARPS * 32 * 8 * 4;       // two buffers of per-warp partial score fragments
constexpr int MLA_SMEM = MLA_STAGES * MLA_STAGE_BYTES + MLA_XCH_BYTES + 1024;
constexpr float MLA_MASK = -1e30f;
constexpr float MLA_LOG2E = 1.4426950408889634f;

struct MlaParams {
  const __nv_bfloat16* q_c;      // [B, 1, H, 512]
  const __nv_bfloat16* q_r;      // [B, 1, H, 128]
  const int32_t* lengths;        // [B]
  const int32_t* step_tile;
  const int32_t* step_code;
  const int32_t* step_count;
  const int32_t* tile_first;     // [B + 1]
  float* ws_m;                   // [B, blocks, H]
  float* ws_l;                   // [B, blocks, H]
  float* ws_acc;                 // [B, blocks, H, 512]
  int* arrivals;                 // [B, H / 16]
  __nv_bfloat16* out;            // [B, 1, H, 512]
  int B, H, S, block, blocks;    // H: rows per sequence (new tokens x heads); cache positions per sequence,
                                 // positions per step, steps per sequence
  int heads, T;                  // heads per token, new tokens per sequence
  long long* profile;            // per-CTA counters (PROFILE_WORDS each) or null: the tcgen05 kernel fills them
  int* status;
};

// Merge `n` partials of rows h0 .. h0 + 3 of sequence b over this warp's 128 latent columns (from column c0; a
// lane holds 4 of them), normalise and write bf16. The partials were written by other CTAs: read past L1.
// `first_piece` is the index of the sequence's first partial in the workspace's [piece][row] arrays.
__device__ __forceinline__ void mla_merge_rows(const MlaParams& p, size_t first_piece, int b, int h0, int c0, int n,
                                               int lane) {
  const size_t base = first_piece * p.H + h0;
  float mx[4], lsum[4];
  float4 o[4];
#pragma unroll
  for (int h = 0; h < 4; ++h) mx[h] = MLA_MASK, lsum[h] = 0.f, o[h] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i0 = 0; i0 < n; i0 += 32)
    if (i0 + lane < n) {
#pragma unroll
      for (int h = 0; h < 4; ++h) mx[h] = fmaxf(mx[h], __ldcg(p.ws_m + base + static_cast<size_t>(i0 + lane) * p.H + h));
    }
#pragma unroll
  for (int h = 0; h < 4; ++h)
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xFFFFFFFFu, mx[h], d));
  for (int i0 = 0; i0 < n; i0 += 32) {
    float w_mine[4] = {0.f, 0.f, 0.f, 0.f};
    if (i0 + lane < n) {
      const size_t idx = base + static_cast<size_t>(i0 + lane) * p.H;
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        w_mine[h] = __expf(__ldcg(p.ws_m + idx + h) - mx[h]);
        lsum[h] += w_mine[h] * __ldcg(p.ws_l + idx + h);
      }
    }
    const int cnt = min(32, n - i0);
#pragma unroll 4
    for (int i = 0; i < cnt; ++i) {
      const size_t idx = base + static_cast<size_t>(i0 + i) * p.H;
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const float w = __shfl_sync(0xFFFFFFFFu, w_mine[h], i);
        const float4 a = __ldcg(reinterpret_cast<const float4*>(p.ws_acc + (idx + h) * MLA_C + c0 + lane * 4));
        o[h].x = fmaf(w, a.x, o[h].x), o[h].y = fmaf(w, a.y, o[h].y);
        o[h].z = fmaf(w, a.z, o[h].z), o[h].w = fmaf(w, a.w, o[h].w);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < 4; ++h) {
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) lsum[h] += __shfl_xor_sync(0xFFFFFFFFu, lsum[h], d);
    const float inv = 1.0f / fmaxf(lsum[h], 1e-30f);
    uint2 r;
    r.x = pack_bf16(o[h].x * inv, o[h].y * inv);
    r.y = pack_bf16(o[h].z * inv, o[h].w * inv);
    *reinterpret_cast<uint2*>(p.out + (static_cast<size_t>(b) * p.H + h0 + h) * MLA_C + c0 + lane * 4) = r;
  }
}

__global__ void __launch_bounds__(MLA_WARPS * 32, 3)
    mla_decode_kernel(const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_r,
                      const MlaParams p) {
  extern __shared__ uint8_t mla_smem_raw[];
  __shared__ __align__(8) uint64_t bars[2 * MLA_STAGES];  // full[stage], empty[stage]
  __shared__ int abort_sh, last_sh;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ring = (smem_u32(mla_smem_raw) + 1023u) & ~1023u;
  uint8_t* ring_ptr = mla_smem_raw + (ring - smem_u32(mla_smem_raw));
  float* xch = reinterpret_cast<float*>(ring_ptr + MLA_STAGES * MLA_STAGE_BYTES);
  auto full_bar = [&](int s) { return smem_u32(&bars[s]); };
  auto empty_bar = [&](int s) { return smem_u32(&bars[MLA_STAGES + s]); };
  if (threadIdx.x == 0) {
    for (int s = 0; s < MLA_STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), MLA_WARPS);
    }
    abort_sh = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_c);
    tma_prefetch_desc(&map_r);
  }
  // Launched with programmatic stream serialisation behind the step-table kernel: nothing it writes is read
  // before this returns.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __syncthreads();
  const int step = blockIdx.x;
  if (step >= p.step_count[0]) return;
  const int b = p.step_tile[step];
  const int code = p.step_code[step];
  const int h0 = blockIdx.y * MLA_HEADS;
  const int len = p.lengths[b];
  const int j0 = (code >> 3) * p.block;  // first cache position of the step
  const int n_micro = (code & 4) ? 0 : (min(p.block, len - j0) + MLA_SUB - 1) / MLA_SUB;
  // The 16 rows of a group belong to one new token (heads per token is a multiple of 16): it sees the positions
  // before lengths[b] - T + token + 1.
  const int visible_end = len - p.T + h0 / p.heads + 1;
  const int first = p.tile_first[b], pieces = p.tile_first[b + 1] - first;
  const int slot = step - first;

  const int g = lane >> 2, t = lane & 3;
  const int lrow = lane & 7;
  const uint32_t k_lane = lrow * 128;
  const int k_unit = lane >> 3;
  const uint32_t v_lane = (lrow + 8 * ((lane >> 3) & 1)) * 128;
  const int v_unit = lane >> 4;

  // A fragments of the queries: this warp's 8 latent k-steps and 2 RoPE k-steps; [0] = row g columns + 2t, [1] =
  // row g + 8, [2] = row g columns + 8 + 2t, [3] = row g + 8.
  uint32_t qa[10][4];
  {
    const uint32_t* qc0 = reinterpret_cast<const uint32_t*>(p.q_c + (static_cast<size_t>(b) * p.H + h0 + g) * MLA_C);
    const uint32_t* qc1 = qc0 + 8 * (MLA_C / 2);
    const uint32_t* qr0 = reinterpret_cast<const uint32_t*>(p.q_r + (static_cast<size_t>(b) * p.H + h0 + g) * MLA_R);
    const uint32_t* qr1 = qr0 + 8 * (MLA_R / 2);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int col = (128 * warp + 16 * j) / 2 + t;
      qa[j][0] = qc0[col], qa[j][1] = qc1[col], qa[j][2] = qc0[col + 4], qa[j][3] = qc1[col + 4];
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int col = (32 * warp + 16 * j) / 2 + t;
      qa[8 + j][0] = qr0[col], qa[8 + j][1] = qr1[col], qa[8 + j][2] = qr0[col + 4], qa[8 + j][3] = qr1[col + 4];
    }
  }
  float o[16][4];
#pragma unroll
  for (int nt = 0; nt < 16; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float m_run[2] = {MLA_MASK * MLA_LOG2E, MLA_MASK * MLA_LOG2E}, l_run[2] = {0.f, 0.f};

  const int token0 = b * p.S + j0;  // row of the step's first position in the [B * S, columns] views
  auto issue = [&](int i) {         // thread 0: loads of micro-step i into slot i % STAGES
    const int stage = i % MLA_STAGES;
    const uint32_t dst = ring + stage * MLA_STAGE_BYTES;
    const int row = token0 + i * MLA_SUB;
    mbar_expect_tx(full_bar(stage), MLA_STAGE_BYTES);
#pragma unroll
    for (int x = 0; x < MLA_C / 64; ++x) tma_load_2d(dst + x * MLA_BOX_BYTES, &map_c, 64 * x, row, full_bar(stage));
#pragma unroll
    for (int x = 0; x < MLA_R / 64; ++x)
      tma_load_2d(dst + (MLA_C / 64 + x) * MLA_BOX_BYTES, &map_r, 64 * x, row, full_bar(stage));
  };
  if (threadIdx.x == 0)
    for (int i = 0; i < MLA_STAGES - 1 && i < n_micro; ++i) issue(i);

  // Every warp runs every iteration and reaches its __syncthreads, whatever happens: a wait that gives up raises
  // the CTA's abort flag, which everyone reads right after the barrier, and from then on the iterations are empty.
  bool ok = true;
  for (int i = 0; i < n_micro; ++i) {
    const int stage = i % MLA_STAGES;
    const uint32_t sbase = ring + stage * MLA_STAGE_BYTES;
    float sc[2][4] = {};  // scores; the odd k-steps accumulate apart (sd) so that four MMA chains run side by side
    float sd[2][4] = {};
    if (ok) {
      if (threadIdx.x == 0 && i + MLA_STAGES - 1 < n_micro) {
        // The slot of micro-step i - 1 takes micro-step i + STAGES - 1 once every warp has left it.
        const int nxt = i + MLA_STAGES - 1;
        bool free_slot = true;
        if (nxt >= MLA_STAGES)
          free_slot = mbar_wait(empty_bar(nxt % MLA_STAGES), ((nxt / MLA_STAGES) - 1) & 1, &abort_sh, p.status,
                                TJX_ERR_WAIT_EMPTY);
        if (free_slot) issue(nxt);
      }
      const bool got = mbar_wait(full_bar(stage), (i / MLA_STAGES) & 1, &abort_sh, p.status, TJX_ERR_WAIT_FULL);
      if (__all_sync(0xFFFFFFFFu, got)) {
        // This warp's share of the scores: [tile][0..1] = row g, positions 8 tile + 2t, + 1; [2..3] = row g + 8.
#pragma unroll
        for (int tl = 0; tl < 2; ++tl) {
#pragma unroll
          for (int x = 0; x < 5; ++x) {  // four loads over 128 latent columns, one over 32 RoPE columns
            const int box = x < 4 ? 2 * warp + (x >> 1) : MLA_C / 64 + (warp >> 1);
            const int unit0 = x < 4 ? 4 * (x & 1) : 4 * (warp & 1);
            const int unit = unit0 + k_unit;
            const uint32_t addr = sbase + box * MLA_BOX_BYTES + tl * 1024 + k_lane + ((unit ^ lrow) << 4);
            uint32_t bf[4];
            ldmatrix_x4(addr, bf);
            mma_16x8x16(sc[tl], qa[2 * x][0], qa[2 * x][1], qa[2 * x][2], qa[2 * x][3], bf[0], bf[1]);
            mma_16x8x16(sd[tl], qa[2 * x + 1][0], qa[2 * x + 1][1], qa[2 * x + 1][2], qa[2 * x + 1][3], bf[2], bf[3]);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) sc[tl][e] += sd[tl][e];
        }
      }
    }
    // The four warps' partial scores meet in shared memory; everyone adds them in warp order.
    float* mine = xch + ((i & 1) * MLA_WARPS + warp) * 256 + lane * 8;
    reinterpret_cast<float4*>(mine)[0] = make_float4(sc[0][0], sc[0][1], sc[0][2], sc[0][3]);
    reinterpret_cast<float4*>(mine)[1] = make_float4(sc[1][0], sc[1][1], sc[1][2], sc[1][3]);
    __syncthreads();
    ok = ok && abort_sh == 0;
    if (!ok) continue;
    float s8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int w = 0; w < MLA_WARPS; ++w) {
      const float* src = xch + ((i & 1) * MLA_WARPS + w) * 256 + lane * 8;
      const float4 a = reinterpret_cast<const float4*>(src)[0], c = reinterpret_cast<const float4*>(src)[1];
      s8[0] += a.x, s8[1] += a.y, s8[2] += a.z, s8[3] += a.w, s8[4] += c.x, s8[5] += c.y, s8[6] += c.z, s8[7] += c.w;
    }
    // Online softmax of rows g and g + 8 over the 16 positions (4 per lane per row).
    const int pos0 = j0 + i * MLA_SUB;
    uint32_t pa[4];
    float alpha[2];
    bool grew = false;
#pragma unroll
    for (int x = 0; x < 2; ++x) {
      float s4[4] = {s8[2 * x], s8[2 * x + 1], s8[4 + 2 * x], s8[4 + 2 * x + 1]};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tok = (e >> 1) * 8 + 2 * t + (e & 1);
        s4[e] = pos0 + tok < visible_end ? s4[e] * MLA_LOG2E : MLA_MASK * MLA_LOG2E;
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
      for (int nt = 0; nt < 16; ++nt)
        o[nt][0] *= alpha[0], o[nt][1] *= alpha[0], o[nt][2] *= alpha[1], o[nt][3] *= alpha[1];
    }
    // O += P V over this warp's 128 latent columns (boxes 2 warp and 2 warp + 1).
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      const int unit = (2 * x + v_unit) & 7;
      const uint32_t addr = sbase + (2 * warp + (x >> 2)) * MLA_BOX_BYTES + v_lane + ((unit ^ lrow) << 4);
      uint32_t bf[4];
      ldmatrix_x4_trans(addr, bf);
      mma_16x8x16(o[2 * x], pa[0], pa[1], pa[2], pa[3], bf[0], bf[1]);
      mma_16x8x16(o[2 * x + 1], pa[0], pa[1], pa[2], pa[3], bf[2], bf[3]);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(stage));  // this warp has left the slot
  }
  if (!ok) return;  // the same in every thread of the CTA

  // Flush: rows g and g + 8 of this warp's 128 columns.
  const int c0 = 128 * warp;
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    float l_all = l_run[x];
    l_all += __shfl_xor_sync(0xFFFFFFFFu, l_all, 1);
    l_all += __shfl_xor_sync(0xFFFFFFFFu, l_all, 2);
    const int h = h0 + g + 8 * x;
    if (pieces == 1) {
      const float inv = 1.0f / fmaxf(l_all, 1e-30f);
      uint32_t* dst = reinterpret_cast<uint32_t*>(p.out + (static_cast<size_t>(b) * p.H + h) * MLA_C + c0);
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) dst[nt * 4 + t] = pack_bf16(o[nt][2 * x] * inv, o[nt][2 * x + 1] * inv);
    } else {
      const size_t row = (static_cast<size_t>(b) * p.blocks + slot) * p.H + h;
      if (warp == 0 && t == 0) {  // the partials keep the max in natural-log units
        p.ws_m[row] = m_run[x] * (1.0f / MLA_LOG2E);
        p.ws_l[row] = l_all;
      }
      float2* dst = reinterpret_cast<float2*>(p.ws_acc + row * MLA_C + c0);
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) dst[nt * 4 + t] = make_float2(o[nt][2 * x], o[nt][2 * x + 1]);
    }
  }
  if (pieces > 1) {
    // Count this step; the CTA that counts last finds every partial of (sequence, head group) written and merges.
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last_sh = atomicAdd(p.arrivals + b * (p.H / MLA_HEADS) + blockIdx.y, 1) == pieces - 1;
    __syncthreads();
    if (last_sh) {
      __threadfence();
      for (int r = 0; r < MLA_HEADS; r += 4)
        mla_merge_rows(p, static_cast<size_t>(b) * p.blocks, b, h0 + r, c0, pieces, lane);
    }
  }
}

// ------------------------------------------------------------------------------------------------ tcgen05 path
//
// The same attention on the tensor cores' own path: a CTA works on 64 rows ((new token, head) pairs) — the M of a
// 64-row tcgen05.mma — so a position's 1280 bytes are staged once for 64 heads instead of once per 16, and the
// scores and the output accumulate in TMEM. One persistent CTA per SM takes a contiguous range of the launch's
// 32-position units (see MtPiece below).
//
//   warp 0      producer: one ring of five 40 KB slots (ten 128-byte-swizzled boxes [32 rows x 64 columns]). A piece
//               sends its 64 rows of queries through two slots (rows 0-31, rows 32-63), then its units, 32 positions
//               a slot
//   warp 1      MMA issuer (whole warp, one elected lane): S = Q K^T over the 640 columns with Q read from TENSOR MEMORY
//               (40 MMAs of 64 x 32 x 16 into one of two score buffers), then O += P V as two halves of 256 latent
//               columns, P read from TMEM too
//   warps 2-5   queries, softmax, flush: a 64-row tile sits in TMEM lanes 0-15 of each 32-lane quarter (row 16 q + i in
//               lane 32 q + i); a second 64-row tile may use lanes 16-31 of the same columns. Lane i < 16 of warp q owns
//               row 16 q + i together with lane i + 16. At the start of a piece the pair copies the row's queries from the
//               ring into TMEM as the A operand: columns 0-319 (twenty K = 16 slices) into the lower lane, 320-639 into
//               the upper one. The scores of the two column halves accumulate in the lower and the upper lanes of one
//               score buffer, and the pair adds them (one shuffle). O's two halves of 256 latent columns are the two
//               tiles of columns 0-255; both lanes compute the same P and each stores it in its own lane, beside its
//               accumulator.
//
// TMEM: columns 0-255 O (both tiles), 256-287 and 288-319 the two score buffers (P, bf16, two per column, overlays
// the first 16 columns of its buffer), 320-479 the queries.
//
// Why the queries live in tensor memory: an MMA whose operands both come from shared memory is bound by the 128 bytes
// per cycle shared memory delivers (64 x 32 x 16 reads 2 KB of Q and 1 KB of K: 27.6 cycles measured back to back on
// an idle SM, 19.9 with Q in TMEM, against 16 of arithmetic at the half rate of a 64-row tile), and the queries' 80 KB
// were read again for every 32 positions. Out of shared memory they also leave room for a five-slot ring instead
// of three: a slot is wanted one unit after it is freed with three.
constexpr int MT_ROWS = 64;
constexpr int MT_POS = 32;                                   // positions per unit of work (one pass of the pipeline)
constexpr int MT_STAGES = 5;
constexpr int MT_KV_BOX = MT_POS * 128;                      // 32 positions x 64 columns
constexpr int MT_STAGE_BYTES = MLA_BOXES * MT_KV_BOX;        // 40 KB
constexpr int MT_Q_SLOTS = MT_ROWS / MT_POS;                 // ring slots a piece's queries take (32 rows each)
constexpr int MT_BAR_OFF = MT_STAGES * MT_STAGE_BYTES;
constexpr int MT_MAX_B = 2048;                               // sequences whose unit counts fit the shared-memory table
constexpr int MT_FIRST_OFF = MT_BAR_OFF + 256;               // int[B + 1]: units before each sequence
constexpr int MT_SMEM = MT_FIRST_OFF + (MT_MAX_B + 1) * 4 + 252 + 1024;
constexpr int MT_THREADS = 192;
constexpr int MT_S_COL = 256;                                // first column of the score buffers
constexpr int MT_Q_COL = 320;                                // first column of the queries (160 columns, both lane halves)
constexpr int MT_MAX_CTAS = 256;                             // CTAs per 64-row group (the SMs of one GPU)
constexpr int MT_MIN_SHARE = 2;                              // units a CTA takes at least
// What starting a piece costs (its queries into TMEM, the pipeline filling, its flush), in units: measured 5 200
// cycles against 1 340 a unit. The units are shared out with this much counted in front of every sequence, so that
// a CTA whose range crosses into another sequence gets fewer units. (tilejax_b200/schedule.py states the same
// arithmetic on the host, `mla_unit_ranges`, with these three constants; a test compares the two.)
constexpr int MT_PIECE_COST = 3;
constexpr float MT_RESCALE_THRESHOLD = 8.0f;

// The work of a launch is every sequence's cache in units of 32 positions, in sequence order; the CTAs of a 64-row
// group share the units out evenly, each taking one contiguous range, so ragged lengths balance to within a unit
// and a sequence is cut into as few pieces as there are CTAs crossing it. Every CTA derives the list itself from
// `lengths` (a warp scan in its prologue); the step-table kernel runs beside it and only emits the caller's tables.
// A piece = (sequence, range of its units) is one pass of the pipeline below; a piece that is its sequence's only
// one is normalised and written at once, else its partial goes to the workspace at index (CTA + sequence) — unique,
// and consecutive for the pieces of one sequence — and mla_tc_merge_kernel, launched behind this kernel, merges.
struct MtPiece {
  int b, unit0, n_units, len, pieces;
  int next;     // where the CTA's range continues (a position on the line of units with MT_PIECE_COST before each sequence)
  bool more;    // the range holds units of a later sequence
  size_t index;  // this piece's partial
};

__global__ void __launch_bounds__(MT_THREADS, 1)
    mla_tc_kernel(const __grid_constant__ CUtensorMap map_qc, const __grid_constant__ CUtensorMap map_qr,
                  const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_r,
                  const MlaParams p) {
  extern __shared__ uint8_t mt_smem_raw[];
  const uint32_t base = (smem_u32(mt_smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = mt_smem_raw + (base - smem_u32(mt_smem_raw));
  const uint32_t bar_base = base + MT_BAR_OFF;
  // barriers: kv_full[5], kv_empty[5], s_full[2], p_ready[2] (four warps arrive), o_done, q_ready (four warps)
  auto kv_full = [&](int s) { return bar_base + 8u * s; };
  auto kv_empty = [&](int s) { return bar_base + 8u * (MT_STAGES + s); };
  auto s_full = [&](int t) { return bar_base + 8u * (2 * MT_STAGES + t); };
  auto p_ready = [&](int t) { return bar_base + 8u * (2 * MT_STAGES + 2 + t); };
  const uint32_t o_done = bar_base + 8u * (2 * MT_STAGES + 4);
  const uint32_t q_ready = bar_base + 8u * (2 * MT_STAGES + 5);
  constexpr int N_BARS = 2 * MT_STAGES + 6;
  static_assert(8 * N_BARS + 32 <= 256, "barriers and flags fit before the unit table");
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(base_ptr + MT_BAR_OFF + 8 * N_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + MT_BAR_OFF + 8 * N_BARS + 8);
  int* q_release = reinterpret_cast<int*>(base_ptr + MT_BAR_OFF + 8 * N_BARS + 16);  // [2]: warps done with a query slot
  int* first_unit = reinterpret_cast<int*>(base_ptr + MT_FIRST_OFF);  // [B + 1]

  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
  long long* prof = p.profile == nullptr
                        ? nullptr
                        : p.profile + (static_cast<size_t>(blockIdx.y) * gridDim.x + blockIdx.x) * PROFILE_WORDS;
  if (prof != nullptr && threadIdx.x == 0) prof[0] = clock64(), prof[12] = static_cast<long long>(globaltimer_ns());
  if (threadIdx.x == 0) {
    for (int i = 0; i < N_BARS; ++i)
      mbar_init(bar_base + 8u * i, (i == 2 * MT_STAGES + 2 || i == 2 * MT_STAGES + 3 || i == 2 * MT_STAGES + 5) ? 4 : 1);
    *abort_flag = 0;
    q_release[0] = 0, q_release[1] = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_qc);
    tma_prefetch_desc(&map_qr);
    tma_prefetch_desc(&map_c);
    tma_prefetch_desc(&map_r);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), 512);
    tmem_relinquish();
  } else if (warp == 0) {
    // Units before each sequence: an inclusive warp scan over the sequences, 32 at a time.
    int carry = 0;
    for (int b0 = 0; b0 < p.B; b0 += 32) {
      const int b = b0 + lane;
      int x = b < p.B ? (min(max(p.lengths[b], 0), p.S) + MT_POS - 1) / MT_POS : 0;
      if (x > 0) x += MT_PIECE_COST;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int y = __shfl_up_sync(0xFFFFFFFFu, x, d);
        if (lane >= d) x += y;
      }
      if (b < p.B) first_unit[b + 1] = carry + x;
      carry += __shfl_sync(0xFFFFFFFFu, x, 31);
    }
    if (lane == 0) first_unit[0] = 0;
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xFFFFFFFFu, *tmem_holder, 0);
  // The merge kernel may be scheduled from here on: a CTA of it starts wherever an SM has room (in practice once
  // that SM's CTA of this kernel has left), works out its sequence's pieces, and then waits for this whole grid to
  // complete before it reads a partial.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int row0 = blockIdx.y * MT_ROWS;  // first of this CTA's rows among a sequence's p.H rows
  // (Read from shared memory: the same in every lane, and said so to the compiler, so that the MMA warp's loops over
  // this CTA's range stay warp-uniform and its descriptors in uniform registers.)
  const int total_units = __shfl_sync(0xFFFFFFFFu, first_unit[p.B], 0);
  const int share = max(MT_MIN_SHARE + MT_PIECE_COST,
                        (total_units + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x));
  const int cta = static_cast<int>(blockIdx.x);
  const int u_begin = min(cta * share, total_units), u_end = min(u_begin + share, total_units);
  // The piece at position `u` of this CTA's range (u < u_end): the same in every thread. Positions count units with
  // MT_PIECE_COST more in front of every sequence that has any; a range that ends inside that margin holds no unit of
  // the sequence (n_units == 0: every role skips it).
  auto piece_at = [&](int u) {
    int lo = 0, hi = p.B;  // the sequence with first_unit[b] <= u < first_unit[b + 1]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (first_unit[mid] <= u) lo = mid; else hi = mid;
    }
    MtPiece pc;
    pc.b = lo;
    const int l = first_unit[lo + 1];
    const int real0 = first_unit[lo] + MT_PIECE_COST;  // the sequence's first unit
    const int start = max(u, real0), end = min(u_end, l);
    pc.unit0 = start - real0;
    pc.n_units = max(end - start, 0);
    pc.next = end;
    pc.more = u_end > l + MT_PIECE_COST;
    pc.len = min(max(p.lengths[lo], 0), p.S);
    const int first_cta = real0 / share;
    pc.pieces = (l - 1) / share - first_cta + 1;
    pc.index = static_cast<size_t>(cta) + lo;
    return pc;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int slot = 0;  // ring slots filled so far: a piece's two query slots, then one per unit
      bool ok = true;
      auto fill = [&](const CUtensorMap* wide, const CUtensorMap* narrow, int row) {
        const int stage = slot % MT_STAGES;
        if (slot >= MT_STAGES &&
            !mbar_wait(kv_empty(stage), ((slot / MT_STAGES) - 1) & 1, abort_flag, p.status, TJX_ERR_WAIT_EMPTY))
          return false;
        const uint32_t dst = base + stage * MT_STAGE_BYTES;
        mbar_expect_tx(kv_full(stage), MT_STAGE_BYTES);
        for (int x = 0; x < MLA_C / 64; ++x) tma_load_2d(dst + x * MT_KV_BOX, wide, 64 * x, row, kv_full(stage));
        for (int x = 0; x < MLA_R / 64; ++x)
          tma_load_2d(dst + (MLA_C / 64 + x) * MT_KV_BOX, narrow, 64 * x, row, kv_full(stage));
        ++slot;
        return true;
      };
      for (int u = u_begin; u < u_end && ok;) {
        const MtPiece pc = piece_at(u);
        u = pc.next;
        if (pc.n_units == 0) continue;
        const int q_row = pc.b * p.H + row0;
        for (int h = 0; h < MT_Q_SLOTS && ok; ++h) ok = fill(&map_qc, &map_qr, q_row + h * MT_POS);
        const int token0 = pc.b * p.S + pc.unit0 * MT_POS;
        for (int i = 0; i < pc.n_units && ok; ++i) ok = fill(&map_c, &map_r, token0 + i * MT_POS);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (whole warp; one lane issues)
    const uint32_t idesc_qk = idesc_bf16_f32(MT_ROWS, MT_POS, 0, 0);  // Q from TMEM, K K-major
    const uint32_t idesc_pv = idesc_bf16_f32(MT_ROWS, 256, 0, 1);     // P from TMEM, the latents MN-major
    long long in_wait = 0, p_wait = 0, fill_wait = -1, units = 0, qk_cyc = 0, pv_cyc = 0;
    const long long t_first = prof != nullptr ? clock64() : 0;
    auto wait = [&](uint32_t bar, uint32_t parity, int err, long long& waited) {
      return __all_sync(0xFFFFFFFFu, mbar_wait_timed(bar, parity, abort_flag, p.status, err, waited, prof != nullptr)) != 0;
    };
    // The scores of unit g (counted over the CTA's whole range), whose positions are in ring slot `slot`: columns
    // 0-319 of Q and K into the lower lanes of the score buffer, 320-639 into the upper lanes.
    auto issue_qk = [&](int g, int slot) {
      const long long t0 = prof != nullptr ? clock64() : 0;
      const uint32_t kv = base + (slot % MT_STAGES) * MT_STAGE_BYTES;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint32_t tile = tmem_base + (static_cast<uint32_t>(16 * half) << 16);
        const uint32_t d = tile + MT_S_COL + (g & 1) * MT_POS;
#pragma unroll
        for (int bl = 0; bl < MLA_BOXES / 2; ++bl) {  // a 64-column box = four MMAs at a time
          uint32_t qa[4];
          uint64_t kd[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            qa[k] = tile + MT_Q_COL + (bl * 4 + k) * 8;
            kd[k] = smem_desc_sw128(kv + (half * (MLA_BOXES / 2) + bl) * MT_KV_BOX, 16, 1024) + ((k * 32) >> 4);
          }
          mma_ts_x4(d, qa, kd, idesc_qk, bl != 0 ? 1u : 0u);
        }
      }
      mma_commit_elected(s_full(g & 1));
      if (prof != nullptr) qk_cyc += clock64() - t0;
    };
    int g0 = 0, done = 0;  // units and pieces issued so far
    bool ok = true;
    for (int u = u_begin; u < u_end && ok;) {
      const MtPiece pc = piece_at(u);
      const int n = __shfl_sync(0xFFFFFFFFu, pc.n_units, 0);
      u = __shfl_sync(0xFFFFFFFFu, pc.next, 0);
      if (n == 0) continue;
      const int slot0 = g0 + MT_Q_SLOTS * (done + 1);  // the ring slot of the piece's first unit
      ok = wait(q_ready, done & 1, TJX_ERR_WAIT_FULL, in_wait) &&
           wait(kv_full(slot0 % MT_STAGES), (slot0 / MT_STAGES) & 1, TJX_ERR_WAIT_FULL, in_wait);
      if (fill_wait < 0) fill_wait = in_wait;
      if (!ok) break;
      tc_fence_after_sync();
      issue_qk(g0, slot0);
      for (int i = 0; i < n && ok; ++i) {
        const int g = g0 + i, slot = slot0 + i;
        if (i + 1 < n) {  // the next unit's scores run while this one's softmax does
          ok = wait(kv_full((slot + 1) % MT_STAGES), ((slot + 1) / MT_STAGES) & 1, TJX_ERR_WAIT_FULL, in_wait);
          if (!ok) break;
          tc_fence_after_sync();
          issue_qk(g + 1, slot + 1);
        }
        ok = wait(p_ready(g & 1), (g >> 1) & 1, TJX_ERR_WAIT_OTHER, p_wait);
        if (!ok) break;
        tc_fence_after_sync();
        const long long t_pv = prof != nullptr ? clock64() : 0;
        const int stage = slot % MT_STAGES;
        const uint32_t kv = base + stage * MT_STAGE_BYTES;
#pragma unroll
        for (int half = 0; half < 2; ++half) {  // latent columns 256 half .. 256 half + 255: the tile at lanes 16 half
          const uint32_t tile = static_cast<uint32_t>(16 * half) << 16;
#pragma unroll
          for (int kk = 0; kk < MT_POS / 16; ++kk) {
            const uint64_t vd = smem_desc_sw128(kv + half * 4 * MT_KV_BOX + kk * (16 * 128), MT_KV_BOX, 1024);
            const uint32_t pa = tmem_base + tile + MT_S_COL + (g & 1) * MT_POS + kk * 8;
            if (elect_one()) mma_ts(tmem_base + tile, pa, vd, idesc_pv, (i != 0 || kk != 0) ? 1u : 0u);
          }
        }
        mma_commit_elected(kv_empty(stage));
        mma_commit_elected(o_done);
        if (prof != nullptr) pv_cyc += clock64() - t_pv;
      }
      g0 += n, units += n;
      ++done;
    }
    if (prof != nullptr && lane == 0) {
      prof[1] = t_first, prof[2] = clock64(), prof[3] = in_wait, prof[4] = max(fill_wait, 0ll), prof[5] = 0, prof[6] = units;
      prof[8] = p_wait, prof[9] = qk_cyc, prof[10] = pv_cyc, prof[11] = done;
    }
  } else {
    // ------------------------------------------------------------------ softmax, correction, flush (warps 2..5)
    const int q = warp & 3;                      // the TMEM lane quarter this warp may touch
    const int r = 16 * q + (lane & 15);          // row within the CTA's 64
    const int half = lane >> 4;                  // which 256 latent columns of O this lane owns
    const int row = row0 + r;                    // row within the sequence
    const uint32_t quarter = static_cast<uint32_t>(32 * q) << 16;
    const uint32_t o_tmem = tmem_base + quarter;  // this lane: lane 32 q + lane, columns 0..255
    // Sequences without a position have no piece: their rows are zeros.
    if (row < p.H)
      for (int b = cta; b < p.B; b += static_cast<int>(gridDim.x))
        if (first_unit[b + 1] == first_unit[b]) {
          uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(b) * p.H + row) * MLA_C + 256 * half);
          for (int x = 0; x < 32; ++x) dst[x] = make_uint4(0u, 0u, 0u, 0u);
        }
    // This row's queries, from the ring into TMEM as the A operand of Q K^T. `first_slot` is the first of the piece's
    // two query slots: warps 0-1 find rows 0-31 there, warps 2-3 rows 32-63 in the next; a lane copies five 64-column
    // boxes, 128 bytes of its row each (the 16-byte chunk c of row r of a swizzled box sits at chunk c ^ (r & 7)).
    // Called when the previous piece's Q K^T have all completed: this warp has waited for each of their score buffers.
    auto stage_queries = [&](int first_slot) {
      const int q_slot = first_slot + (q >> 1);
      const int stage = q_slot % MT_STAGES;
      const bool got = mbar_wait(kv_full(stage), (q_slot / MT_STAGES) & 1, abort_flag, p.status, TJX_ERR_WAIT_FULL);
      if (!__all_sync(0xFFFFFFFFu, got)) return false;
      const int r_slot = 16 * (q & 1) + (lane & 15);
      const uint8_t* src = base_ptr + stage * MT_STAGE_BYTES + half * (MLA_BOXES / 2) * MT_KV_BOX + r_slot * 128;
#pragma unroll 1
      for (int bl = 0; bl < MLA_BOXES / 2; ++bl) {
        uint32_t w[32];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 x = *reinterpret_cast<const uint4*>(src + bl * MT_KV_BOX + ((c ^ (r_slot & 7)) << 4));
          w[4 * c] = x.x, w[4 * c + 1] = x.y, w[4 * c + 2] = x.z, w[4 * c + 3] = x.w;
        }
        tmem_st32(tmem_base + quarter + MT_Q_COL + bl * 32, w);
      }
      tmem_wait_st();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(q_ready);
        // The slot goes back to the producer when both of its warps have read it.
        __threadfence_block();
        if (atomicAdd(&q_release[q >> 1], 1) == 1) {
          q_release[q >> 1] = 0;
          mbar_arrive(kv_empty(stage));
        }
      }
      return true;
    };
    int g0 = 0, done = 0;  // units and pieces seen so far
    bool ok = true, staged = false;  // staged: the coming piece's queries are in TMEM already
    for (int u = u_begin; u < u_end && ok;) {
      const MtPiece pc = piece_at(u);
      const int n = pc.n_units;
      u = pc.next;
      if (n == 0) continue;
      if (!staged && !stage_queries(g0 + MT_Q_SLOTS * done)) break;
      const int j0 = pc.unit0 * MT_POS;
      // New token `row / heads` sees the positions before lengths[b] - T + token + 1.
      const int limit = min(pc.len - p.T + row / p.heads + 1, pc.len);
      float m_used = MLA_MASK * MLA_LOG2E, l = 0.f;
      for (int i = 0; i < n; ++i) {
        const int g = g0 + i;
        const bool got = mbar_wait(s_full(g & 1), (g >> 1) & 1, abort_flag, p.status, TJX_ERR_WAIT_TMEM_FULL);
        if (!__all_sync(0xFFFFFFFFu, got)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t s_tmem = tmem_base + quarter + MT_S_COL + (g & 1) * MT_POS;
        uint32_t v[32];
        tmem_ld32(s_tmem, v);
        tmem_wait_ld();
        const int pos0 = j0 + i * MT_POS;
        float mx = MLA_MASK * MLA_LOG2E;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          // The row's score is the sum over the two column halves, one in this lane, one in its partner.
          const float part = __uint_as_float(v[j]);
          const float sc = part + __shfl_xor_sync(0xFFFFFFFFu, part, 16);
          const float x = pos0 + j < limit ? sc * MLA_LOG2E : MLA_MASK * MLA_LOG2E;
          v[j] = __float_as_uint(x);
          mx = fmaxf(mx, x);
        }
        if (i == 0) {
          m_used = mx;
        } else if (__any_sync(0xFFFFFFFFu, mx > m_used + MT_RESCALE_THRESHOLD)) {
          // Raise the running max and rescale what has been accumulated, once O += P V of the previous unit is complete.
          const float m_new = fmaxf(m_used, mx);
          const float alpha = ex2(m_used - m_new);
          m_used = m_new;
          l *= alpha;
          const bool od = mbar_wait(o_done, (g - 1) & 1, abort_flag, p.status, TJX_ERR_WAIT_OTHER);
          if (!__all_sync(0xFFFFFFFFu, od)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            uint32_t o[32];
            tmem_ld32(o_tmem + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
            tmem_st32(o_tmem + c * 32, o);
          }
          tmem_wait_st();
        }
        uint32_t pk[16];
        float l0 = 0.f, l1 = 0.f;
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float p0 = ex2(__uint_as_float(v[j]) - m_used), p1 = ex2(__uint_as_float(v[j + 1]) - m_used);
          l0 += p0, l1 += p1;
          pk[j >> 1] = pack_bf16(p0, p1);  // P is rounded before P V
        }
        l += l0 + l1;
        tmem_st16(s_tmem, pk);
        tmem_wait_st();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready(g & 1));
        // Keep up with o_done: a parity wait is only right for a waiter at most one phase behind, and nothing else
        // makes this warp see P V of the previous unit complete (this unit's scores were issued before it). The
        // piece's last P V is waited for below, before O is read.
        if (i >= 1) {
          const bool od = mbar_wait(o_done, (g - 1) & 1, abort_flag, p.status, TJX_ERR_WAIT_OTHER);
          ok = __all_sync(0xFFFFFFFFu, od) != 0;
        }
        if (!ok) break;
        tc_fence_after_sync();
      }
      if (!ok) break;
      // The next piece's queries go in while the last P V runs: its first Q K^T then overlaps the flush below.
      staged = pc.more;
      if (staged && !stage_queries(g0 + n + MT_Q_SLOTS * (done + 1))) break;
      {
        const bool od = mbar_wait(o_done, (g0 + n - 1) & 1, abort_flag, p.status, TJX_ERR_WAIT_OTHER);
        if (!__all_sync(0xFFFFFFFFu, od)) break;
        tc_fence_after_sync();
      }
      // Flush this lane's 256 latent columns of its row: the output itself, or a partial for the merge. A partial is
      // laid out the way the warps hold it — [warp q][32-column step c][16-byte chunk x][lane] — so that every store
      // instruction of a warp writes 512 contiguous bytes; written by row, each lane's 16 bytes land in a line of
      // their own and a flush costs ~10 000 cycles between two pieces. (Rows past the sequence's last are written too:
      // the workspace holds whole 64-row groups, and the merge skips them.)
      const float inv = 1.0f / fmaxf(l, 1e-30f);
      const size_t block = pc.index * gridDim.y + blockIdx.y;  // this piece's 64 rows in the workspace
      if (pc.pieces > 1 && half == 0) {  // the partials keep the max in natural-log units
        p.ws_m[block * MT_ROWS + r] = m_used * (1.0f / MLA_LOG2E);
        p.ws_l[block * MT_ROWS + r] = l;
      }
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t o[32];
        tmem_ld32(o_tmem + c * 32, o);
        tmem_wait_ld();
        if (pc.pieces == 1) {
          if (row < p.H) {
            uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(pc.b) * p.H + row) * MLA_C + 256 * half + c * 32);
#pragma unroll
            for (int x = 0; x < 4; ++x) {
              uint4 val;
              val.x = pack_bf16(__uint_as_float(o[8 * x + 0]) * inv, __uint_as_float(o[8 * x + 1]) * inv);
              val.y = pack_bf16(__uint_as_float(o[8 * x + 2]) * inv, __uint_as_float(o[8 * x + 3]) * inv);
              val.z = pack_bf16(__uint_as_float(o[8 * x + 4]) * inv, __uint_as_float(o[8 * x + 5]) * inv);
              val.w = pack_bf16(__uint_as_float(o[8 * x + 6]) * inv, __uint_as_float(o[8 * x + 7]) * inv);
              dst[x] = val;
            }
          }
        } else {
          uint4* dst = reinterpret_cast<uint4*>(p.ws_acc + block * (MT_ROWS * MLA_C)) + ((q * 8 + c) * 8) * 32 + lane;
#pragma unroll
          for (int x = 0; x < 8; ++x) dst[x * 32] = make_uint4(o[4 * x], o[4 * x + 1], o[4 * x + 2], o[4 * x + 3]);
        }
      }
      // The reads of O above are ordered before this warp's next arrival on p_ready, which is what the next piece's
      // first P V waits for before it overwrites O. (Partials are merged by mla_tc_merge_kernel, launched behind this.)
      tc_fence_before_sync();
      g0 += n;
      ++done;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (prof != nullptr && threadIdx.x == 0) prof[7] = clock64(), prof[13] = static_cast<long long>(globaltimer_ns());
  if (warp == 1) {
    if (*abort_flag) __nanosleep(100000);
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// Merges the partials mla_tc_kernel left: a CTA per (sequence, 64-row group, 16 rows of it), a warp per step of 32
// latent columns, a lane per (row, half of the columns) exactly as the main kernel's warps held them, so that its
// reads are the 512-byte runs the main kernel wrote. It works out the sequence's pieces as the main kernel did
// (units before the sequence, the share of a CTA), returns at once for a sequence written directly, and otherwise
// reads the pieces' (max, sum, accumulator) past L1, weights them by exp(max_i - max), and writes the normalised
// rows in bf16. Launched with programmatic stream serialisation: the prologue runs beside the main kernel's tail.
constexpr int MG_WARPS = 8;

// (Its 188 registers a thread keep a CTA of it off an SM that still holds one of the main kernel's; capped at 168 it
// fits beside one, spills a little, and the call measured 2 us slower.)
__global__ void __launch_bounds__(MG_WARPS * 32)
    mla_tc_merge_kernel(const MlaParams p, int main_ctas, int groups) {
  __shared__ int seq_units[3];  // units before sequence b, before b + 1, in total
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x;
  if (warp == 0) {
    int carry = 0, before = 0, through = 0;
    for (int b0 = 0; b0 < p.B; b0 += 32) {
      const int i = b0 + lane;
      int x = i < p.B ? (min(max(p.lengths[i], 0), p.S) + MT_POS - 1) / MT_POS : 0;
      if (x > 0) x += MT_PIECE_COST;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int y = __shfl_up_sync(0xFFFFFFFFu, x, d);
        if (lane >= d) x += y;
      }
      const int incl = carry + x;
      if (i == b) through = incl;
      if (i == b - 1) before = incl;
      carry += __shfl_sync(0xFFFFFFFFu, x, 31);
    }
    // (Each of the two values was seen by one lane.)
    before = __reduce_max_sync(0xFFFFFFFFu, before), through = __reduce_max_sync(0xFFFFFFFFu, through);
    if (lane == 0) seq_units[0] = before, seq_units[1] = through, seq_units[2] = carry;
  }
  __syncthreads();
  const int f = seq_units[0], l = seq_units[1], total = seq_units[2];
  if (l == f) return;  // no position: the main kernel wrote zeros
  const int share = max(MT_MIN_SHARE + MT_PIECE_COST, (total + main_ctas - 1) / main_ctas);
  const int first_cta = (f + MT_PIECE_COST) / share;
  const int n = (l - 1) / share - first_cta + 1;
  if (n <= 1) return;  // written directly
  const int group = blockIdx.y >> 2, q = blockIdx.y & 3, c = warp;
  const int r = 16 * q + (lane & 15), half = lane >> 4;
  const int row = group * MT_ROWS + r;
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the partials are the main kernel's
  const size_t block0 = (static_cast<size_t>(first_cta) + b) * groups + group;  // piece i: block0 + i * groups
  // Four pieces at a time, all their loads issued before the first is used (the kernel is a handful of dependent
  // round trips to L2 long, nothing else), folded into a running (max, sum, accumulator) as the softmax itself is.
  constexpr int MG_CHUNK = 4;
  float mx = MLA_MASK, lsum = 0.f;
  float4 o[8];
#pragma unroll
  for (int x = 0; x < 8; ++x) o[x] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int i0 = 0; i0 < n; i0 += MG_CHUNK) {
    float m[MG_CHUNK], ls[MG_CHUNK];
    float4 a[MG_CHUNK][8];
#pragma unroll
    for (int k = 0; k < MG_CHUNK; ++k) {
      const bool live = i0 + k < n;
      const size_t block = block0 + static_cast<size_t>(live ? i0 + k : i0) * groups;
      m[k] = live ? __ldcg(p.ws_m + block * MT_ROWS + r) : MLA_MASK;
      ls[k] = live ? __ldcg(p.ws_l + block * MT_ROWS + r) : 0.f;
      const float4* src = reinterpret_cast<const float4*>(p.ws_acc + block * (MT_ROWS * MLA_C)) + ((q * 8 + c) * 8) * 32 + lane;
#pragma unroll
      for (int x = 0; x < 8; ++x) a[k][x] = live ? __ldcg(src + x * 32) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float m_new = mx;
#pragma unroll
    for (int k = 0; k < MG_CHUNK; ++k) m_new = fmaxf(m_new, m[k]);
    const float keep = __expf(mx - m_new);
    mx = m_new;
    lsum *= keep;
#pragma unroll
    for (int x = 0; x < 8; ++x) o[x].x *= keep, o[x].y *= keep, o[x].z *= keep, o[x].w *= keep;
#pragma unroll
    for (int k = 0; k < MG_CHUNK; ++k) {
      const float w = i0 + k < n ? __expf(m[k] - mx) : 0.f;
      lsum = fmaf(w, ls[k], lsum);
#pragma unroll
      for (int x = 0; x < 8; ++x) {
        o[x].x = fmaf(w, a[k][x].x, o[x].x), o[x].y = fmaf(w, a[k][x].y, o[x].y);
        o[x].z = fmaf(w, a[k][x].z, o[x].z), o[x].w = fmaf(w, a[k][x].w, o[x].w);
      }
    }
  }
  if (row >= p.H) return;
  const float inv = 1.0f / fmaxf(lsum, 1e-30f);
  uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<size_t>(b) * p.H + row) * MLA_C + 256 * half + 32 * c);
#pragma unroll
  for (int x = 0; x < 4; ++x) {
    uint4 val;
    val.x = pack_bf16(o[2 * x].x * inv, o[2 * x].y * inv), val.y = pack_bf16(o[2 * x].z * inv, o[2 * x].w * inv);
    val.z = pack_bf16(o[2 * x + 1].x * inv, o[2 * x + 1].y * inv), val.w = pack_bf16(o[2 * x + 1].z * inv, o[2 * x + 1].w * inv);
    dst[x] = val;
  }
}

int g_mla_mode = 1;  // 1: the tcgen05 kernel; 0: the warp-level MMA kernel (an A/B switch; values agree to rounding)

static size_t mla_align256(size_t n) { return (n + 255) & ~static_cast<size_t>(255); }

// Rows of partials the workspace holds, H rows a sequence: [sequence][block] for the warp-level kernel,
// [CTA + sequence] whole 64-row groups for the tcgen05 kernel; the larger of the two.
static size_t mla_partial_rows(int B, int H, int blocks) {
  const size_t groups = (static_cast<size_t>(H) + MT_ROWS - 1) / MT_ROWS;
  return std::max(static_cast<size_t>(B) * blocks * H, (static_cast<size_t>(MT_MAX_CTAS) + B) * groups * MT_ROWS);
}

}  // namespace tjx

extern "C" {

int tjx_mla_set_mode(int mode) {
  if (mode != 0 && mode != 1) return tjx::fail(TJX_E_ARG, "mode must be 0 (warp-level MMA) or 1 (tcgen05)");
  tjx::g_mla_mode = mode;
  return 0;
}

size_t tjx_mla_decode_workspace_bytes(int B, int T, int H, int S, int block) {
  if (B <= 0 || T <= 0 || H <= 0 || S <= 0 || block <= 0 || S % block != 0) return 0;
  H *= T;  // rows per sequence
  const size_t rows = tjx::mla_partial_rows(B, H, S / block);
  return 2 * tjx::mla_align256(rows * sizeof(float)) + tjx::mla_align256(rows * tjx::MLA_C * sizeof(float)) +
         tjx::mla_align256(static_cast<size_t>(B) * H * sizeof(int));
}

int tjx_mla_decode_bf16(const void* q_c, const void* q_r, const void* c_kv, const void* k_rope,
                        const int32_t* lengths, void* out, int B, int T, int H, int S, int C, int R, int block,
                        int32_t* step_tile, int32_t* step_code, int32_t* step_count, int32_t* tile_first,
                        void* workspace, size_t workspace_bytes, tjx_stream_t stream) {
  using namespace tjx;
  if (int rc = check_device()) return rc;
  if (!q_c || !q_r || !c_kv || !k_rope || !lengths || !out) return fail(TJX_E_ARG, "an input or output pointer is null");
  if (!step_tile || !step_code || !step_count || !tile_first) return fail(TJX_E_ARG, "a step table pointer is null");
  if (B <= 0 || T <= 0 || H <= 0 || S <= 0 || block <= 0) return fail(TJX_E_ARG, "sizes must be positive");
  if (C != MLA_C || R != MLA_R) return fail(TJX_E_ARG, "the latent cache is 512 columns wide and the RoPE cache 128");
  if (H % MLA_HEADS != 0) return fail(TJX_E_ARG, "the number of heads must be a multiple of 16");
  if (block % MLA_SUB != 0 || S % block != 0)
    return fail(TJX_E_ARG, "the block must be a multiple of 16 positions that divides the cache length");
  if (static_cast<long long>(B) * S >= (1ll << 31)) return fail(TJX_E_LIMIT, "B * S must fit in int32");
  const size_t need = tjx_mla_decode_workspace_bytes(B, T, H, S, block);
  const int heads = H;
  H *= T;  // rows per sequence from here on
  const bool tensor_path = g_mla_mode == 1 && B <= MT_MAX_B;
  if (workspace == nullptr || workspace_bytes < need)
    return fail(TJX_E_ARG, "workspace is null or smaller than tjx_mla_decode_workspace_bytes");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(TJX_E_ARG, "workspace must be 256-byte aligned");
  const uintptr_t ptrs[] = {reinterpret_cast<uintptr_t>(q_c), reinterpret_cast<uintptr_t>(q_r),
                            reinterpret_cast<uintptr_t>(c_kv), reinterpret_cast<uintptr_t>(k_rope),
                            reinterpret_cast<uintptr_t>(out)};
  for (uintptr_t a : ptrs)
    if (a & 15u) return fail(TJX_E_ARG, "q_c, q_r, c_kv, k_rope and out must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  MlaParams p{};
  p.q_c = static_cast<const __nv_bfloat16*>(q_c), p.q_r = static_cast<const __nv_bfloat16*>(q_r);
  p.lengths = lengths;
  p.step_tile = step_tile, p.step_code = step_code, p.step_count = step_count, p.tile_first = tile_first;
  p.B = B, p.H = H, p.S = S, p.block = block, p.blocks = S / block;
  p.heads = heads, p.T = T;
  const size_t rows = mla_partial_rows(B, H, p.blocks);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  p.ws_m = reinterpret_cast<float*>(ws);
  p.ws_l = reinterpret_cast<float*>(ws + mla_align256(rows * sizeof(float)));
  p.ws_acc = reinterpret_cast<float*>(ws + 2 * mla_align256(rows * sizeof(float)));
  p.arrivals = reinterpret_cast<int*>(ws + 2 * mla_align256(rows * sizeof(float)) +
                                      mla_align256(rows * MLA_C * sizeof(float)));
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = device_status_word();
  if (p.status == nullptr) return fail(TJX_E_CUDA, "could not locate the device status word");

  // Steps: block j of sequence b runs unless j * block >= lengths[b]; the kernel clears the arrival counters too.
  if (int rc = launch_build_steps_lengths(lengths, B, nullptr, B, p.blocks, 0, block, step_tile, step_code, step_count,
                                          tile_first, p.arrivals, B * (H / MLA_HEADS), s))
    return rc;

  if (tensor_path) {
    CUtensorMap mqc, mqr, mc, mr;
    const uint32_t kv_box[2] = {64, MT_POS};  // the queries travel in boxes of 32 rows too: two ring slots a piece
    const uint64_t q_rows = static_cast<uint64_t>(B) * H, kv_rows = static_cast<uint64_t>(B) * S;
    const struct { CUtensorMap* map; const void* ptr; uint64_t cols, rows; const uint32_t* box; } maps[4] = {
        {&mqc, q_c, MLA_C, q_rows, kv_box}, {&mqr, q_r, MLA_R, q_rows, kv_box},
        {&mc, c_kv, MLA_C, kv_rows, kv_box}, {&mr, k_rope, MLA_R, kv_rows, kv_box}};
    for (const auto& m : maps) {
      const uint64_t dims[2] = {m.cols, m.rows};
      const uint64_t strides[1] = {m.cols * 2};
      if (int rc = make_tensor_map(m.map, m.ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, dims, strides, m.box,
                                   CU_TENSOR_MAP_SWIZZLE_128B))
        return rc;
    }
    static bool tc_configured[64] = {};
    int dev = 0;
    TJX_CUDA(cudaGetDevice(&dev));
    if (!tc_configured[dev & 63]) {
      TJX_CUDA(cudaFuncSetAttribute(mla_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MT_SMEM));
      tc_configured[dev & 63] = true;
    }
    const int groups = (H + MT_ROWS - 1) / MT_ROWS;
    const int ctas = std::max(1, std::min(MT_MAX_CTAS, sm_count() / groups));
    p.profile = profile_buffer(ctas * groups);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ctas, groups), cfg.blockDim = dim3(MT_THREADS);
    cfg.dynamicSmemBytes = MT_SMEM, cfg.stream = s;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr, cfg.numAttrs = 1;
    TJX_CUDA(cudaLaunchKernelEx(&cfg, mla_tc_kernel, mqc, mqr, mc, mr, p));
    cudaLaunchConfig_t merge{};
    merge.gridDim = dim3(B, groups * 4), merge.blockDim = dim3(MG_WARPS * 32);
    merge.dynamicSmemBytes = 0, merge.stream = s;
    merge.attrs = &attr, merge.numAttrs = 1;
    TJX_CUDA(cudaLaunchKernelEx(&merge, mla_tc_merge_kernel, p, ctas, groups));
    return 0;
  }

  CUtensorMap mc, mr;
  const uint32_t box[2] = {64, MLA_SUB};
  {
    const uint64_t dims[2] = {MLA_C, static_cast<uint64_t>(B) * S};
    const uint64_t strides[1] = {MLA_C * 2};
    if (int rc = make_tensor_map(&mc, c_kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const uint64_t dims[2] = {MLA_R, static_cast<uint64_t>(B) * S};
    const uint64_t strides[1] = {MLA_R * 2};
    if (int rc = make_tensor_map(&mr, k_rope, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  static bool configured[64] = {};
  int dev = 0;
  TJX_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    TJX_CUDA(cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MLA_SMEM));
    configured[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(B * p.blocks, H / MLA_HEADS), cfg.blockDim = dim3(MLA_WARPS * 32);
  cfg.dynamicSmemBytes = MLA_SMEM, cfg.stream = s;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr, cfg.numAttrs = 1;
  TJX_CUDA(cudaLaunchKernelEx(&cfg, mla_decode_kernel, mc, mr, p));
  return 0;
}

}  // extern "C"

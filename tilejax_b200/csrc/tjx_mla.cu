// Absorbed MLA decode attention on sm_100a, `mla_decode` (examples/decode.py:226-250): the rows of a sequence are its
// (new token, head) pairs, token-major, and new token t of T sees the cache positions up to lengths[b] - T + t
// (`visible`, examples/decode.py:145-152). Every query head scores the same latent cache (512 latents + 128 RoPE columns per position) and the
// output of a head is its softmax-weighted latents, so a position's 1280 bytes are read once for all the heads of
// a head group.
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
  int* status;
};

// Merge `n` partials of rows h0 .. h0 + 3 of sequence b over this warp's 128 latent columns (from column c0; a
// lane holds 4 of them), normalise and write bf16. The partials were written by other CTAs: read past L1.
__device__ __forceinline__ void mla_merge_rows(const MlaParams& p, int b, int h0, int c0, int n, int lane) {
  const size_t base = static_cast<size_t>(b) * p.blocks * p.H + h0;
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
      for (int r = 0; r < MLA_HEADS; r += 4) mla_merge_rows(p, b, h0 + r, c0, pieces, lane);
    }
  }
}

static size_t mla_align256(size_t n) { return (n + 255) & ~static_cast<size_t>(255); }

}  // namespace tjx

extern "C" {

size_t tjx_mla_decode_workspace_bytes(int B, int T, int H, int S, int block) {
  if (B <= 0 || T <= 0 || H <= 0 || S <= 0 || block <= 0 || S % block != 0) return 0;
  H *= T;  // rows per sequence
  const size_t rows = static_cast<size_t>(B) * (S / block) * H;
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
  const size_t rows = static_cast<size_t>(B) * p.blocks * H;
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

// The matmul step loop on sm_100a: out = x @ y (bf16 operands, f32 accumulation in TMEM), optionally causal
// (tril) with skipped tiles written as zeros, walking a table of the output tiles that run.
//
// One persistent CTA per SM. A user tile (tm, tn) — the unit the tile tables and the skip sets are expressed
// in — is cut into CTA tiles of 128 x BN; work item w = (user tile, sub-tile) and CTA c takes items
// c, c + grid, c + 2 grid, ... All roles derive the same item sequence, so nothing is communicated.
//
//   warp 0   producer: TMA loads of the x tile [128 x 64] and the y tile [64 x BN] into a ring of STAGES
//            shared-memory slots (128-byte swizzle), one mbarrier pair (full / empty) per slot
//   warp 1   MMA issuer: one thread issues tcgen05.mma (M 128, N BN, K 16) four times per slot, accumulating
//            in one of two TMEM accumulators; tcgen05.commit frees the slot and, after the last K block,
//            hands the accumulator to the epilogue
//   warps 2-5 epilogue: tcgen05.ld the accumulator (each warp its 32 lanes), apply the causal mask, convert,
//            stage the tile in shared memory and TMA-store it; they also write the zero fills
//
// y [K, N] row-major is the MN-major B operand: a slot holds BN / 64 boxes of [64 n x 64 k], each row of a
// box one k with 64 consecutive n (128 bytes). y [N, K] (x @ y.T) is the K-major operand, one box [64 k x BN].
//
// Three kernels share this loop (and the epilogue code): gemm_kernel, described above; gemm_pair_kernel, the
// default whenever the user tile is a multiple of 256 x 256 — one MMA per pair of SMs (cta_group::2), each SM
// staging half of y's columns (see the section "CTA pairs" below); and its all-gather variant, which adds a
// copier warp per CTA that pulls the other ranks' rows of x out of peer memory while the tiles of the rows that
// are already here run (tjx_all_gather_gemm_bf16).
#include <algorithm>

#include "tjx_host.cuh"
#include "tjx_ptx.cuh"

#include "../../include/tilejax_b200.h"

namespace tjx {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  int M, N, K;
  int tm, tn;            // the user tile
  int tiles_m, tiles_n;  // user tiles along M and N (arithmetic order when there is no table)
  int band_tiles;        // width, in user tiles, of the column bands the arithmetic order walks
  int sub_m, sub_n;      // CTA tiles per user tile
  int n_tiles, n_fills;  // user tiles that run / that are filled
  const int32_t* tile_i;
  const int32_t* tile_j;
  const int32_t* fill_i;
  const int32_t* fill_j;
  int causal, out_f32, b_kmajor;
  int tail_split;        // the pair kernel may halve the pieces of a short last round (see its header)
  int chain;             // CHAIN_WAITS / CHAIN_RELEASES: how the pair kernel's launch is chained on the stream
  int num_kb;
  void* out;
  int* status;
  long long* profile;  // per-CTA counters (PROFILE_WORDS each) or null
  const float* row_scale;  // [M] or null: the epilogue multiplies row r of the accumulator by row_scale[r] (rmsnorm)
  int activation;          // 0: none; 1: tanh GELU of the f32 accumulator before the rounding (attention_block)
  // All-gather fused into the launch (gemm_pair_kernel<.., true> only): rows [own_lo, own_hi) of the gathered
  // operand are this GPU's shard and come from map_a_own; the other shards are pulled from peer memory into
  // `gather_dst` by one extra warp per CTA, 256-row block by block in arrival order, and counted in
  // `gather_arrivals` (one counter per 256-row block of the gathered operand; never reset: a launch waits for
  // gather_epoch * copier warps).
  int gather_ranks, gather_me, gather_rows;  // ranks, this rank, rows per shard
  int gather_epoch;
  const void* gather_src[8];                 // rank r's shard as mapped into this GPU's address space
  void* gather_dst;                          // [ranks * rows, K]
  int* gather_arrivals;
};

struct Item {
  int m0, n0;
  bool compute;  // runs the MMA pipeline; otherwise the epilogue writes zeros
  bool valid;    // false: a table entry out of range, nothing is written
};

template <int BMT, int BN>
__device__ __forceinline__ Item decode_item(const GemmParams& p, int w) {
  const int per = p.sub_m * p.sub_n;
  const int tw = w / per, r = w - tw * per;
  const int sm = r / p.sub_n, sn = r - sm * p.sub_n;
  // The fills come first: only the epilogue warps touch them, so their stores to HBM run while the TMA and MMA
  // warps are already deep into the first tiles that compute (whose order nobody can observe either).
  const int t = tw >= p.n_fills ? tw - p.n_fills : p.n_tiles + tw;
  int ti, tj;
  bool fill = false;
  if (t < p.n_tiles) {
    if (p.tile_i != nullptr) {
      ti = p.tile_i[t];
      tj = p.tile_j[t];
    } else {
      // No table: every tile runs, and their order is not observable, so walk them in column bands of
      // `band_tiles` tiles: the CTAs in flight then share a few thousand rows of x and columns of y that stay
      // in L2, instead of streaming all of y once per row of tiles.
      const int band_size = p.band_tiles * p.tiles_m;          // tiles in a full band
      const int band = t / band_size;
      const int first_col = band * p.band_tiles;
      const int width = min(p.band_tiles, p.tiles_n - first_col);
      const int in_band = t - band * band_size;
      ti = in_band / width;
      tj = first_col + in_band - ti * width;
    }
  } else {
    fill = true;
    ti = p.fill_i[t - p.n_tiles];
    tj = p.fill_j[t - p.n_tiles];
  }
  Item it;
  it.valid = ti >= 0 && tj >= 0 && static_cast<long long>(ti) * p.tm < p.M && static_cast<long long>(tj) * p.tn < p.N;
  it.m0 = ti * p.tm + sm * BMT;
  it.n0 = tj * p.tn + sn * BN;
  if (it.m0 >= p.M || it.n0 >= p.N) it.valid = false;  // a sub-tile wholly past the edge of a clipped tile
  // A sub-tile wholly above the diagonal of a causal tile is all zeros: no loads, no MMA.
  it.compute = it.valid && !fill && !(p.causal && it.n0 > it.m0 + BMT - 1);
  return it;
}

// jax.nn.gelu's default (approximate) form: 0.5 x (1 + tanh(sqrt(2 / pi) (x + 0.044715 x^3))), with the hardware's
// tanh.approx.f32 (relative error about 2^-11, far inside the rounding to bf16 that follows). The epilogue of the
// attention block's first matmul computes 32 768 of these per CTA and piece beside a main loop of only sixteen K
// blocks: with tanh as 1 - 2 / (exp(2 u) + 1) — two special-function operations an element — that matmul was bound by
// its epilogue (the block: 0.190 ms against 0.179).
#ifndef TJX_GELU_TANH_APPROX
#define TJX_GELU_TANH_APPROX 1  // 0: tanh from exp and a division (two special-function operations an element instead of one)
#endif
__device__ __forceinline__ float gelu_tanh(float x) {
  const float u = 0.7978845608028654f * fmaf(0.044715f * x * x, x, x);
#if TJX_GELU_TANH_APPROX
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
#else
  const float t = 1.0f - __fdividef(2.0f, __expf(2.0f * u) + 1.0f);
#endif
  return 0.5f * x * (1.0f + t);
}

// Zeros for 32 rows (row0 .. row0 + 31) of a CTA tile's BN columns from n0: 16 bytes per lane per pass.
template <int BN>
__device__ __forceinline__ void zero_rows(const GemmParams& p, int row0, int n0, int lane) {
  const int out_elt = p.out_f32 ? 4 : 2;
  const int row_bytes = BN * out_elt;
  for (int r = 0; r < 32; ++r) {
    const int row = row0 + r;
    if (row >= p.M) break;
    uint8_t* dst = static_cast<uint8_t*>(p.out) + (static_cast<size_t>(row) * p.N + n0) * out_elt;
    const int valid_bytes = min(row_bytes, (p.N - n0) * out_elt);
    for (int b = lane * 16; b < valid_bytes; b += 32 * 16)
      *reinterpret_cast<uint4*>(dst + b) = make_uint4(0u, 0u, 0u, 0u);
  }
}

// One epilogue warp's share of an accumulator: TMEM lanes of `t_row` (32 rows, output rows row0 .. row0 + 31),
// BN columns from n0. Chunks of 32 accumulator columns are masked (causal), converted, staged in one of the
// warp's two 32-row x 128-byte buffers (128-byte swizzled) and TMA-stored; the buffers alternate so a store can
// still be reading one while the warp fills the other. bf16: two chunks fill a buffer; f32: one chunk does.
template <int BN>
__device__ __forceinline__ void store_accumulator(const GemmParams& p, const CUtensorMap* map_c, uint32_t t_row,
                                                  int row0, int n0, uint8_t* c_ptr, uint32_t c_smem, int& c_buf,
                                                  int lane, int columns = BN) {
  const int row = row0 + lane;
  const int CHUNKS = columns / 32;
  const float scale = p.row_scale != nullptr && row < p.M ? p.row_scale[row] : 1.0f;
#pragma unroll 1
  for (int c = 0; c < CHUNKS; ++c) {
    uint32_t v[32];
    tmem_ld32(t_row + c * 32, v);
    tmem_wait_ld();
    if (p.row_scale != nullptr) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * scale);
    }
    if (p.activation == 1) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(gelu_tanh(__uint_as_float(v[j])));
    }
    if (p.causal) {
      const int col0 = n0 + c * 32;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j > row) v[j] = 0u;
    }
    const bool new_buf = p.out_f32 || (c & 1) == 0;
    if (new_buf) {
      // The TMA store issued two buffers ago has finished reading this buffer.
      if (lane == 0) tma_store_wait_read<1>();
      __syncwarp();
    }
    uint8_t* buf = c_ptr + c_buf * (32 * 128);
    // Row `lane` of the buffer is 128 bytes = eight 16-byte units; unit u is stored at u ^ (lane & 7).
    if (p.out_f32) {
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        uint4 val = make_uint4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
        *reinterpret_cast<uint4*>(buf + lane * 128 + ((u ^ (lane & 7)) << 4)) = val;
      }
    } else {
      const int half = c & 1;  // which 64 bytes of the 128-byte row
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint4 val;
        val.x = pack_bf16(__uint_as_float(v[8 * u + 0]), __uint_as_float(v[8 * u + 1]));
        val.y = pack_bf16(__uint_as_float(v[8 * u + 2]), __uint_as_float(v[8 * u + 3]));
        val.z = pack_bf16(__uint_as_float(v[8 * u + 4]), __uint_as_float(v[8 * u + 5]));
        val.w = pack_bf16(__uint_as_float(v[8 * u + 6]), __uint_as_float(v[8 * u + 7]));
        const int unit = half * 4 + u;
        *reinterpret_cast<uint4*>(buf + lane * 128 + ((unit ^ (lane & 7)) << 4)) = val;
      }
    }
    const bool flush = p.out_f32 || (c & 1) == 1;
    if (flush) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int col = p.out_f32 ? n0 + c * 32 : n0 + (c >> 1) * 64;
        tma_store_2d(map_c, c_smem + c_buf * (32 * 128), col, row0);
        tma_store_commit();
      }
      c_buf ^= 1;
    }
  }
}

template <int BN, int STAGES>
struct GemmSmem {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int C_BYTES = 4 * 32 * 64 * 2 * 2;  // per epilogue warp: two buffers of 32 rows x 128 bytes
  static constexpr int RING_OFF = 0;
  static constexpr int C_OFF = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = C_OFF + C_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;  // barriers + slack for 1024-byte alignment
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ CUtensorMap map_c, const GemmParams p) {
  using L = GemmSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_base = base + L::BAR_OFF;
  // barrier layout (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 + s); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(base_ptr + L::BAR_OFF + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L::BAR_OFF + 8 * (2 * STAGES + 4) + 8);

  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
  const int per = p.sub_m * p.sub_n;
  const int total_items = (p.n_tiles + p.n_fills) * per;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  long long* prof = p.profile == nullptr ? nullptr : p.profile + static_cast<size_t>(blockIdx.x) * PROFILE_WORDS;
  if (prof != nullptr && threadIdx.x == 0) prof[0] = clock64();

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    tma_prefetch_desc(&map_c);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xFFFFFFFFu, *tmem_holder, 0);

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_items && ok; w += gridDim.x) {
        const Item it = decode_item<BM, BN>(p, w);
        if (!it.compute) continue;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, TJX_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = base + L::RING_OFF + stage * L::STAGE_BYTES;
          const uint32_t b_dst = a_dst + L::A_BYTES;
          mbar_expect_tx(full_bar(stage), L::STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, kb * BK, it.m0, full_bar(stage));
          if (p.b_kmajor) {
            tma_load_2d(b_dst, &map_b, kb * BK, it.n0, full_bar(stage));
          } else {
#pragma unroll
            for (int nb = 0; nb < BN / 64; ++nb)
              tma_load_2d(b_dst + nb * (64 * BK * 2), &map_b, it.n0 + nb * 64, kb * BK, full_bar(stage));
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs the loop, so that addresses and descriptors stay in uniform registers; one elected lane
    // issues each ring slot's four MMAs and the commit as one predicated block.
    {
      const uint32_t idesc = idesc_bf16_f32(BM, BN, 0, p.b_kmajor ? 0 : 1);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      long long t_first = 0, in_wait = 0, fill_wait = -1, out_wait = 0, items = 0;
      auto wait = [&](uint32_t bar, uint32_t parity, int code, long long& waited) {
        return __all_sync(0xFFFFFFFFu, mbar_wait_timed(bar, parity, abort_flag, p.status, code, waited, prof != nullptr)) != 0;
      };
      for (int w = blockIdx.x; w < total_items && ok; w += gridDim.x) {
        const Item it = decode_item<BM, BN>(p, w);
        if (!__shfl_sync(0xFFFFFFFFu, static_cast<int>(it.compute), 0)) continue;
        if (items++ == 0) t_first = clock64();
        if (!wait(tempty_bar(acc), acc_phase ^ 1u, TJX_ERR_WAIT_TMEM_EMPTY, out_wait)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!wait(full_bar(stage), phase, TJX_ERR_WAIT_FULL, in_wait)) {
            ok = false;
            break;
          }
          if (fill_wait < 0) fill_wait = in_wait;
          tc_fence_after_sync();
          const uint32_t a_addr = base + L::RING_OFF + stage * L::STAGE_BYTES;
          const uint32_t b_addr = a_addr + L::A_BYTES;
          // (Descriptor addresses count 16 bytes; adding a slice's offset never carries out of the field.)
          const uint64_t a0 = smem_desc_sw128(a_addr, 16, 1024);
          const uint64_t b0 = p.b_kmajor ? smem_desc_sw128(b_addr, 16, 1024) : smem_desc_sw128(b_addr, 64 * BK * 2, 1024);
          const uint32_t b_step = p.b_kmajor ? 32 >> 4 : (16 * 128) >> 4;
          uint64_t ad[4], bd[4];
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) ad[kk] = a0 + kk * (32 >> 4), bd[kk] = b0 + kk * b_step;
          // The slot is free once these MMAs have read it.
          mma_ss_x4_commit(d_tmem, ad, bd, idesc, kb != 0 ? 1u : 0u, empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        mma_commit_elected(tfull_bar(acc));  // the accumulator is complete once every MMA above has finished
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      if (prof != nullptr && lane == 0) {
        prof[1] = t_first, prof[2] = clock64(), prof[3] = in_wait, prof[4] = max(fill_wait, 0ll), prof[5] = out_wait;
        prof[6] = items;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // the TMEM lane quarter this warp may read: lanes 32 q .. 32 q + 31
    const int ew = warp - 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    // Per warp: two staging buffers of 32 rows x 128 bytes (128-byte swizzled), alternated so a TMA store
    // can still be reading one while the warp fills the other.
    const uint32_t c_smem = base + L::C_OFF + ew * (2 * 32 * 128);
    uint8_t* c_ptr = base_ptr + L::C_OFF + ew * (2 * 32 * 128);
    int c_buf = 0;
    for (int w = blockIdx.x; w < total_items; w += gridDim.x) {
      const Item it = decode_item<BM, BN>(p, w);
      if (!it.valid) {
        if (lane == 0 && p.status != nullptr) atomicCAS(p.status, 0, TJX_ERR_BAD_TABLE);
        continue;
      }
      if (!it.compute) {
        zero_rows<BN>(p, it.m0 + q * 32, it.n0, lane);
        continue;
      }
      const bool got = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, TJX_ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xFFFFFFFFu, got)) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      store_accumulator<BN>(p, &map_c, t_row, it.m0 + q * 32, it.n0, c_ptr, c_smem, c_buf, lane);
      // The accumulator has been read: hand it back to the MMA warp.
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
    __syncwarp();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (prof != nullptr && threadIdx.x == 0) prof[7] = clock64();
  if (warp == 1) {
    if (*abort_flag) __nanosleep(100000);  // let whatever is still in flight land before TMEM goes away
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const GemmParams& p,
                       int grid, cudaStream_t stream) {
  using L = GemmSmem<BN, STAGES>;
  auto kernel = gemm_kernel<BN, STAGES>;
  static bool configured[64] = {};
  int dev = 0;
  TJX_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    TJX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    configured[dev & 63] = true;
  }
  kernel<<<grid, GEMM_THREADS, L::TOTAL, stream>>>(ma, mb, mc, p);
  TJX_CUDA(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------------ CTA pairs
//
// The same loop with one MMA per PAIR of SMs (a cluster of two CTAs, tcgen05 cta_group::2). A work item is a
// 256 x 256 piece of a user tile: each CTA of the pair stages its own 128 rows of x and its own 128 columns of y,
// the even CTA issues the M = 256 MMA, which reads both shared memories, and each CTA ends up with its 128 rows
// x 256 columns of the accumulator in its own TMEM. Per SM and per K = 16 step that is 4 KB of A + 4 KB of B
// read from shared memory instead of 4 + 8 KB, and a third fewer bytes from L2 into shared memory per flop: on a
// part that runs this loop at its power limit, fewer bytes moved per flop is a higher clock.
//
//   full[s]    lives in the even CTA: its producer posts the bytes of BOTH CTAs' loads, and the odd CTA's TMA
//              loads count their bytes on it too
//   empty[s]   one per CTA, for its own producer: the MMA thread commits to both
//   tfull[a]   one per CTA, for its own epilogue warps: the MMA thread commits to both
//   tempty[a]  lives in the even CTA: the eight epilogue warps of the pair arrive on it
constexpr int PAIR_BN = 256;
constexpr int PAIR_ROWS = 2 * BM;
// Three ring slots of two 64-k blocks each: the MMA thread commits (frees a slot) once per eight MMAs. Every
// commit drains the pair's MMA pipeline, and with one per four MMAs (six slots of one block) the tensor pipe
// measured 75 % busy against 94 % with this shape; two slots of three blocks prefetch too little.
constexpr int PAIR_STAGES = 3;
constexpr int PAIR_KSUB = 2;
constexpr int PAIR_STAGES_128 = 4;  // 128-wide pieces stage 8 KB less per K block: a fourth slot fits

// A causal launch's work items are of two kinds — pieces that compute and pieces that are only written with zeros —
// and item w, w + pairs, w + 2 pairs, ... can hold nine of the first kind for one pair of CTAs and seven for another.
// Such a launch numbers the two kinds separately in its prologue (a warp scan over all items) and pair r takes the
// r-th, (r + pairs)-th, ... of each: no pair computes more than one piece above the mean. The lists live in shared
// memory, this many entries each; a launch whose share would not fit walks the items the plain way.
//
// A short last round: with P computing pieces and n pairs, the last of ceil(P / n) rounds holds P mod n pieces and the
// other pairs wait for it (10 of 74 for the causal 8192^2, 34 of 74 for 4096^3). When at most half the pairs would
// be busy, each of those pieces is cut into its left and right 128 columns and two pairs take one each (an MMA with
// N = 128, half of the B tile staged, half of the accumulator stored): the round lasts half as long. K is summed in
// the same order, so the result is bit-identical. Pair r finds the piece of pair r / 2 in a third list.
constexpr int PAIR_LIST_CAP = 128;
#ifndef TJX_GEMM_TAIL_SPLIT
#define TJX_GEMM_TAIL_SPLIT 1  // 0: never halve the pieces of a short last round (an A/B switch)
#endif

constexpr int GATHER_THREADS = GEMM_THREADS + 32;  // the pair kernel with its copier warp
// 16-byte loads a copier lane keeps in flight: 148 warps x 32 lanes x 32 x 16 B = 2.4 MB on the wire, what a few
// microseconds of NVLink latency need at several hundred GB/s.
constexpr int GATHER_LOADS = 32;

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bounded wait until a 256-row block of the gathered operand has been written by every copier warp.
__device__ __forceinline__ bool gather_wait(const int* counter, int target, volatile int* abort_flag, int* status) {
  if (ld_acquire_gpu(counter) >= target) return true;
  unsigned long long start = 0, limit = 0;
  for (uint32_t it = 1;; ++it) {
    if (ld_acquire_gpu(counter) >= target) return true;
    if ((it & 63u) == 0) {
      if (*abort_flag) return false;
      const unsigned long long now = globaltimer_ns();
      if (start == 0) start = now, limit = wait_limit_ns(status);
      if (now - start > limit) {
        *abort_flag = 1;
        if (status != nullptr) atomicCAS(status, 0, TJX_ERR_WAIT_OTHER);
        return false;
      }
    }
  }
}

template <int PBN, int STAGES, int KSUB>
struct PairSmem {
  static constexpr int A_BYTES = BM * BK * 2;         // this CTA's 128 rows of x, one block of 64 k
  static constexpr int B_BYTES = (PBN / 2) * BK * 2;  // this CTA's half of the piece's columns of y, one block of 64 k
  static constexpr int SUB_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGE_BYTES = KSUB * SUB_BYTES;    // a ring slot holds KSUB blocks of 64 k
  static constexpr int C_BYTES = 4 * 32 * 64 * 2 * 2;
  static constexpr int RING_OFF = 0;
  static constexpr int C_OFF = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFF = C_OFF + C_BYTES;
  static constexpr int LIST_OFF = BAR_OFF + 256;        // two lists of work items (see PAIR_LIST_CAP)
  static constexpr int TOTAL = LIST_OFF + 3 * PAIR_LIST_CAP * 4 + 1024;
  static_assert(TOTAL <= 227 * 1024, "the pair kernel's shared memory fits one CTA per SM");
};

// PBN = columns of a piece (the N of the pair's MMA): 256, or 128 as an A/B switch (half-size pieces; slower: more
// operand bytes per flop through shared memory); both sum K in the same order, so their results are bit-identical.
template <int PBN, int STAGES, int KSUB, bool GATHER>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GATHER ? GATHER_THREADS : GEMM_THREADS, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_a_own,
                     const GemmParams p) {
  using L = PairSmem<PBN, STAGES, KSUB>;
  constexpr int BN = PBN;
  const int num_slots = (p.num_kb + KSUB - 1) / KSUB;  // ring slots per work item
  extern __shared__ uint8_t smem_raw[];
  // The dynamic shared-memory window starts at the same offset in both CTAs, so the aligned offsets agree.
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bar_base = base + L::BAR_OFF;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto tempty_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + 2 + s); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(base_ptr + L::BAR_OFF + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L::BAR_OFF + 8 * (2 * STAGES + 4) + 8);

  const int warp = uniform_warp_index(), lane = threadIdx.x & 31;
  const uint32_t rank = __shfl_sync(0xFFFFFFFFu, cluster_cta_rank(), 0);  // 0: issues the MMAs; 1: stages and stores its half
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int per = p.sub_m * p.sub_n;
  const int total_items = (p.n_tiles + p.n_fills) * per;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  long long* prof = p.profile == nullptr ? nullptr : p.profile + static_cast<size_t>(blockIdx.x) * PROFILE_WORDS;
  if (prof != nullptr && threadIdx.x == 0) prof[0] = clock64();

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tfull_bar(s), 1);
      mbar_init(tempty_bar(s), 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    tma_prefetch_desc(&map_c);
    if (GATHER) tma_prefetch_desc(&map_a_own);
  }
  int* list_compute = reinterpret_cast<int*>(base_ptr + L::LIST_OFF);
  int* list_zero = list_compute + PAIR_LIST_CAP;
  int* list_donor = list_zero + PAIR_LIST_CAP;  // the computing items of pair `pair / 2`: where a halved piece comes from
  volatile int* list_meta = abort_flag + 1;  // [0] lists in use, [1] computing items in all, [2] zero-only items of this pair
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_holder)), TMEM_COLS);
    tmem_relinquish_pair();
  } else if (warp == 2) {
    int use = 0, mine_c = 0, mine_z = 0;
    if (!GATHER && p.causal) {
      int seen_c = 0, seen_z = 0;
      constexpr int SCAN = 8;  // items a lane decodes per pass: their table reads are in flight together
      for (int w0 = 0; w0 < total_items; w0 += 32 * SCAN) {
        bool in[SCAN], computes[SCAN];
#pragma unroll
        for (int u = 0; u < SCAN; ++u) {
          const int w = w0 + u * 32 + lane;
          in[u] = w < total_items;
          computes[u] = in[u] && decode_item<PAIR_ROWS, BN>(p, w).compute;
        }
#pragma unroll
        for (int u = 0; u < SCAN; ++u) {
          const uint32_t mc = __ballot_sync(0xFFFFFFFFu, computes[u]), mz = __ballot_sync(0xFFFFFFFFu, in[u] && !computes[u]);
          if (in[u]) {
            const uint32_t below = (1u << lane) - 1u;
            const int index = computes[u] ? seen_c + __popc(mc & below) : seen_z + __popc(mz & below);
            if (index % n_pairs == pair && index / n_pairs < PAIR_LIST_CAP)
              (computes[u] ? list_compute : list_zero)[index / n_pairs] = w0 + u * 32 + lane;
            if (computes[u] && index % n_pairs == (pair >> 1) && index / n_pairs < PAIR_LIST_CAP)
              list_donor[index / n_pairs] = w0 + u * 32 + lane;
          }
          seen_c += __popc(mc), seen_z += __popc(mz);
        }
      }
      mine_c = seen_c;
      mine_z = seen_z > pair ? (seen_z - pair + n_pairs - 1) / n_pairs : 0;
      use = seen_c / n_pairs + 1 <= PAIR_LIST_CAP && mine_z <= PAIR_LIST_CAP;
    }
    if (lane == 0) list_meta[0] = use, list_meta[1] = mine_c, list_meta[2] = mine_z;
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything of ours can reach them
  tc_fence_after_sync();
  const uint32_t tmem_base = __shfl_sync(0xFFFFFFFFu, *tmem_holder, 0);
  // A chained launch: everything above ran beside the tail of the kernel in front; its results are needed from here.
  if (p.chain & CHAIN_WAITS) chain_wait();
  if (p.chain & CHAIN_RELEASES) chain_release();
  // This pair's walk: its list of computing items, or items pair, pair + pairs, ... of every kind; `rounds` whole
  // rounds and a last one of `tail` pieces, halved when that keeps twice as many pairs busy.
  const bool listed = __shfl_sync(0xFFFFFFFFu, list_meta[0], 0) != 0;
  const int n_pieces = __shfl_sync(0xFFFFFFFFu, listed ? list_meta[1] : total_items, 0);
  const int rounds = n_pieces / n_pairs, tail = n_pieces - rounds * n_pairs;
  const bool halved = PBN == 256 && !GATHER && p.tail_split != 0 && tail > 0 && 2 * tail <= n_pairs &&
                      (listed || (p.causal == 0 && p.n_fills == 0));
  const int n_walk = rounds + ((halved ? pair < 2 * tail : pair < tail) ? 1 : 0);
  // Item idx of the walk and which part of it: 0 the whole piece, 1 / 2 its left / right 128 columns.
  auto item_of = [&](int idx, int& part) {
    part = 0;
    if (idx < rounds || !halved) return listed ? list_compute[idx] : pair + idx * n_pairs;
    part = 1 + (pair & 1);
    return listed ? list_donor[rounds] : rounds * n_pairs + (pair >> 1);
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (one per CTA)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long gather_waited = 0;
      const int row_off = static_cast<int>(rank) * BM;
      for (int idx = 0; idx < n_walk && ok; ++idx) {
        int part;
        Item it = decode_item<PAIR_ROWS, BN>(p, item_of(idx, part));
        if (!it.compute) continue;
        const int my_cols = part != 0 ? BN / 4 : BN / 2;  // columns of y this CTA stages
        if (part != 0) it.n0 += (part - 1) * (BN / 2);
        const int col_off = static_cast<int>(rank) * my_cols;
        bool own = true;
        if (GATHER) {
          own = it.m0 / p.gather_rows == p.gather_me;
          if (!own) {
            const long long t0 = prof != nullptr ? clock64() : 0;
            // The rows of this piece come from another GPU: wait until the copier warps have all written them,
            // then order those (generic-proxy) writes before this thread's TMA reads.
            if (!gather_wait(p.gather_arrivals + it.m0 / PAIR_ROWS, p.gather_epoch * static_cast<int>(gridDim.x),
                             abort_flag, p.status)) {
              ok = false;
              break;
            }
            if (prof != nullptr) gather_waited += clock64() - t0;
            asm volatile("fence.proxy.async;" ::: "memory");
          }
        }
        for (int slot = 0; slot < num_slots; ++slot) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, TJX_ERR_WAIT_EMPTY)) {
            ok = false;
            break;
          }
          // Blocks past the end of K are loaded all the same: the TMA fills them with zeros, which add nothing.
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * KSUB * (L::A_BYTES + my_cols * BK * 2));
          const uint32_t bar = cluster_map(full_bar(stage), 0);
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            const int kb = slot * KSUB + sub;
            const uint32_t a_dst = base + L::RING_OFF + stage * L::STAGE_BYTES + sub * L::SUB_BYTES;
            const uint32_t b_dst = a_dst + L::A_BYTES;
            if (GATHER && own)
              tma_load_2d_pair(a_dst, &map_a_own, kb * BK, it.m0 - p.gather_me * p.gather_rows + row_off, bar);
            else
              tma_load_2d_pair(a_dst, &map_a, kb * BK, it.m0 + row_off, bar);
            if (p.b_kmajor) {
              tma_load_2d_pair(b_dst, &map_b, kb * BK, it.n0 + col_off, bar);
            } else {
#pragma unroll
              for (int nb = 0; nb < BN / 2 / 64; ++nb)
                if (nb * 64 < my_cols)
                  tma_load_2d_pair(b_dst + nb * (64 * BK * 2), &map_b, it.n0 + col_off + nb * 64, kb * BK, bar);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (GATHER && prof != nullptr) prof[10] = gather_waited;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (even CTA only)
    // The whole warp runs the loop (uniform registers for addresses and descriptors); one elected lane issues.
    if (rank == 0) {
      const uint32_t idesc_whole = idesc_bf16_f32(PAIR_ROWS, BN, 0, p.b_kmajor ? 0 : 1);
      const uint32_t idesc_half = idesc_bf16_f32(PAIR_ROWS, BN / 2, 0, p.b_kmajor ? 0 : 1);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      long long t_first = 0, in_wait = 0, fill_wait = -1, out_wait = 0, items = 0;
      auto wait = [&](uint32_t bar, uint32_t parity, int code, long long& waited) {
        return __all_sync(0xFFFFFFFFu, mbar_wait_timed(bar, parity, abort_flag, p.status, code, waited, prof != nullptr)) != 0;
      };
      for (int idx = 0; idx < n_walk && ok; ++idx) {
        int part;
        const Item it = decode_item<PAIR_ROWS, BN>(p, item_of(idx, part));
        if (!__shfl_sync(0xFFFFFFFFu, static_cast<int>(it.compute), 0)) continue;
        const uint32_t idesc = __shfl_sync(0xFFFFFFFFu, part, 0) != 0 ? idesc_half : idesc_whole;
        if (items++ == 0) t_first = clock64();
        if (!wait(tempty_bar(acc), acc_phase ^ 1u, TJX_ERR_WAIT_TMEM_EMPTY, out_wait)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int slot = 0; slot < num_slots; ++slot) {
          if (!wait(full_bar(stage), phase, TJX_ERR_WAIT_FULL, in_wait)) {
            ok = false;
            break;
          }
          if (fill_wait < 0) fill_wait = in_wait;
          tc_fence_after_sync();
          const uint32_t b_step = p.b_kmajor ? 32 >> 4 : (16 * 128) >> 4;
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            const uint32_t a_addr = base + L::RING_OFF + stage * L::STAGE_BYTES + sub * L::SUB_BYTES;
            const uint32_t b_addr = a_addr + L::A_BYTES;
            // (Descriptor addresses count 16 bytes; adding a slice's offset never carries out of the field.)
            const uint64_t a0 = smem_desc_sw128(a_addr, 16, 1024);
            const uint64_t b0 = p.b_kmajor ? smem_desc_sw128(b_addr, 16, 1024) : smem_desc_sw128(b_addr, 64 * BK * 2, 1024);
            uint64_t ad[4], bd[4];
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) ad[kk] = a0 + kk * (32 >> 4), bd[kk] = b0 + kk * b_step;
            mma_ss_pair_x4(d_tmem, ad, bd, idesc, (slot | sub) != 0 ? 1u : 0u);
          }
          // The slot is free in both CTAs once these MMAs have read it.
          mma_commit_pair_both(cluster_map(empty_bar(stage), 0), cluster_map(empty_bar(stage), 1));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        mma_commit_pair_both(cluster_map(tfull_bar(acc), 0), cluster_map(tfull_bar(acc), 1));
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      if (prof != nullptr && lane == 0) {
        prof[1] = t_first, prof[2] = clock64(), prof[3] = in_wait, prof[4] = max(fill_wait, 0ll), prof[5] = out_wait;
        prof[6] = items;
      }
    }
    __syncwarp();
  } else if (GATHER && warp == 6) {
    // ------------------------------------------------------------------ copier (one warp per CTA)
    // Pulls the other ranks' shards from peer memory into this GPU's copy, a 256-row block at a time in the order
    // the tiles will want them (round r brings the shard of rank (me - r) mod ranks), every CTA's warp a slice
    // of each block: 16 bytes per lane per load, GATHER_LOADS loads in flight. It waits for nothing — the peers' shards
    // were complete before the launch — so the warps that wait on its counters always see progress.
    const int per_shard = p.gather_rows / PAIR_ROWS;
    const size_t block_bytes = static_cast<size_t>(PAIR_ROWS) * p.K * 2;
    const size_t slice = ((block_bytes + gridDim.x - 1) / gridDim.x + 511) / 512 * 512;
    const size_t lo = min(block_bytes, slice * blockIdx.x), hi = min(block_bytes, lo + slice);
    for (int r = 1; r < p.gather_ranks; ++r) {
      const int src_rank = (p.gather_me - r + p.gather_ranks) % p.gather_ranks;
      for (int blk = 0; blk < per_shard; ++blk) {
        const uint8_t* src = static_cast<const uint8_t*>(p.gather_src[src_rank]) + blk * block_bytes;
        const int row_block = src_rank * per_shard + blk;
        uint8_t* dst = static_cast<uint8_t*>(p.gather_dst) + row_block * block_bytes;
        for (size_t off = lo + lane * 16; off < hi; off += GATHER_LOADS * 512) {
          uint4 v[GATHER_LOADS];
#pragma unroll
          for (int u = 0; u < GATHER_LOADS; ++u)
            if (off + u * 512 < hi) v[u] = __ldcg(reinterpret_cast<const uint4*>(src + off + u * 512));
#pragma unroll
          for (int u = 0; u < GATHER_LOADS; ++u)
            if (off + u * 512 < hi) *reinterpret_cast<uint4*>(dst + off + u * 512) = v[u];
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(p.gather_arrivals + row_block, 1);
      }
    }
    if (prof != nullptr && lane == 0) prof[11] = clock64();
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of each CTA)
    const int q = warp & 3;
    const int ew = warp - 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t c_smem = base + L::C_OFF + ew * (2 * 32 * 128);
    uint8_t* c_ptr = base_ptr + L::C_OFF + ew * (2 * 32 * 128);
    int c_buf = 0;
    // With lists: first the items that only write zeros (their stores run under the first pieces' loads).
    for (int idx = 0, n_zero = listed ? list_meta[2] : 0; idx < n_zero; ++idx) {
      const Item it = decode_item<PAIR_ROWS, BN>(p, list_zero[idx]);
      if (!it.valid) {
        if (lane == 0 && p.status != nullptr) atomicCAS(p.status, 0, TJX_ERR_BAD_TABLE);
        continue;
      }
      zero_rows<BN>(p, it.m0 + static_cast<int>(rank) * BM + q * 32, it.n0, lane);
    }
    for (int idx = 0; idx < n_walk; ++idx) {
      int part;
      Item it = decode_item<PAIR_ROWS, BN>(p, item_of(idx, part));
      if (part != 0) it.n0 += (part - 1) * (BN / 2);
      if (!it.valid) {
        if (lane == 0 && p.status != nullptr) atomicCAS(p.status, 0, TJX_ERR_BAD_TABLE);
        continue;
      }
      const int row0 = it.m0 + static_cast<int>(rank) * BM + q * 32;
      if (!it.compute) {
        zero_rows<BN>(p, row0, it.n0, lane);
        continue;
      }
      const bool got = mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, TJX_ERR_WAIT_TMEM_FULL);
      if (!__all_sync(0xFFFFFFFFu, got)) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
      if (row0 < p.M) store_accumulator<BN>(p, &map_c, t_row, row0, it.n0, c_ptr, c_smem, c_buf, lane, part != 0 ? BN / 2 : BN);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(cluster_map(tempty_bar(acc), 0));
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (lane == 0) tma_store_wait_all<0>();
    __syncwarp();
  }

  // Neither CTA may leave, or free the pair's TMEM, while the other can still read its shared memory or TMEM.
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (prof != nullptr && threadIdx.x == 0) prof[7] = clock64();
  if (warp == 1) {
    if (*abort_flag) __nanosleep(100000);
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <int PBN, int STAGES, int KSUB, bool GATHER>
static int launch_gemm_pair(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
                            const CUtensorMap& ma_own, const GemmParams& p, int grid, cudaStream_t stream) {
  using L = PairSmem<PBN, STAGES, KSUB>;
  auto kernel = gemm_pair_kernel<PBN, STAGES, KSUB, GATHER>;
  static bool configured[64] = {};
  int dev = 0;
  TJX_CUDA(cudaGetDevice(&dev));
  if (!configured[dev & 63]) {
    TJX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
    configured[dev & 63] = true;
  }
  if (p.chain & CHAIN_WAITS) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid), cfg.blockDim = dim3(GATHER ? GATHER_THREADS : GEMM_THREADS);
    cfg.dynamicSmemBytes = L::TOTAL, cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr, cfg.numAttrs = 1;
    TJX_CUDA(cudaLaunchKernelEx(&cfg, kernel, ma, mb, mc, ma_own, p));
    return 0;
  }
  kernel<<<grid, GATHER ? GATHER_THREADS : GEMM_THREADS, L::TOTAL, stream>>>(ma, mb, mc, ma_own, p);
  TJX_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace tjx

namespace tjx {
static thread_local int g_gemm_cta_limit = 0;  // 0 = one CTA per SM
static thread_local int g_gemm_pair_mode = 1;  // 0 never pairs; 1 (and 3) pairs with 256-wide pieces; 2 pairs with 128-wide
}

extern "C" int tjx_gemm_set_pair_mode(int mode) {
  if (mode < 0 || mode > 3)
    return tjx::fail(TJX_E_ARG, "mode must be 0 (single CTAs), 1 or 3 (pairs, 256-wide pieces) or 2 (pairs, 128-wide pieces)");
  tjx::g_gemm_pair_mode = mode;
  return 0;
}

extern "C" int tjx_gemm_set_cta_limit(int max_ctas) {
  if (max_ctas < 0) return tjx::fail(TJX_E_ARG, "max_ctas must be >= 0");
  tjx::g_gemm_cta_limit = max_ctas;
  return 0;
}

namespace tjx {
// The matmul launch behind tjx_gemm_bf16, tjx_rmsnorm_gemm_bf16 and tjx_attention_block_bf16 (`row_scale`,
// `activation`: see GemmParams).
int gemm_launch(const void* x, const void* y, void* out, int M, int N, int K, int y_transposed, int tm, int tn, int tk,
                int stages, int out_f32, int causal, const int32_t* tile_i, const int32_t* tile_j, int n_tiles,
                const int32_t* fill_i, const int32_t* fill_j, int n_fills, const float* row_scale, int activation,
                tjx_stream_t stream) {
  if (int rc = check_device()) return rc;
  if (x == nullptr || y == nullptr || out == nullptr) return fail(TJX_E_ARG, "x, y or out is null");
  if (M <= 0 || N <= 0 || K <= 0) return fail(TJX_E_ARG, "M, N, K must be positive");
  if (K % 8 != 0 || N % 8 != 0)
    return fail(TJX_E_ARG, "K and N must be multiples of 8 (16-byte rows for the TMA descriptors)");
  if (tm <= 0 || tn <= 0 || tk <= 0) return fail(TJX_E_ARG, "tile sizes must be positive");
  if (!(tm % 128 == 0 || tm == M)) return fail(TJX_E_ARG, "tm must be a multiple of 128, or all of M");
  if (!(tn % 128 == 0 || tn == N)) return fail(TJX_E_ARG, "tn must be a multiple of 128, or all of N");
  if (M % tm != 0 || N % tn != 0) return fail(TJX_E_ARG, "the tiles must cover M and N exactly");
  if ((tile_i == nullptr) != (tile_j == nullptr)) return fail(TJX_E_ARG, "tile_i and tile_j go together");
  if (n_fills < 0 || (n_fills > 0 && (fill_i == nullptr || fill_j == nullptr)))
    return fail(TJX_E_ARG, "fill tables are missing");
  if (causal && y_transposed == 0 && M != N) { /* tril of a rectangular product is still well defined */ }
  const int tiles_m = M / tm, tiles_n = N / tn;
  if (tile_i == nullptr) {
    if (n_tiles != 0 && n_tiles != tiles_m * tiles_n)
      return fail(TJX_E_ARG, "without a tile table every tile runs: n_tiles must be 0 or (M/tm)*(N/tn)");
    n_tiles = tiles_m * tiles_n;
  } else if (n_tiles <= 0) {
    return fail(TJX_E_ARG, "a tile table needs n_tiles > 0");
  }
  // CTA pairs need whole 256 x 256 pieces of every user tile; an explicit stage count asks for the single-CTA ring.
  const bool pair = g_gemm_pair_mode >= 1 && stages == 0 && tm % PAIR_ROWS == 0 && tn % PAIR_BN == 0;
  // Piece width of the pair kernel: 256 columns. 128-wide pieces (mode 2) would fill the last round of a launch
  // better (4096^3 would take 3.5 rounds' time instead of 4) but move 1.5x the operand bytes per flop through shared
  // memory and measured 1.3 - 1.4x slower (8192^3: 0.97 ms against 0.68 ms), so they are only kept as an A/B switch.
  const int pbn = (pair && g_gemm_pair_mode == 2) ? 128 : PAIR_BN;
  if (stages == 0) stages = 4;
  const int BN = (tn % 256 == 0) ? 256 : 128;
  if (!(stages == 4 || (BN == 128 && stages == 6) || (BN == 256 && stages == 3)))
    return fail(TJX_E_ARG, "stages must be 0 (default), 4, 3 (256-wide CTA tiles) or 6 (128-wide)");

  GemmParams p{};
  p.M = M, p.N = N, p.K = K, p.tm = tm, p.tn = tn, p.tiles_m = tiles_m, p.tiles_n = tiles_n;
  p.band_tiles = std::max(1, 2048 / tn);
  p.sub_m = pair ? tm / PAIR_ROWS : (tm + BM - 1) / BM;
  p.sub_n = pair ? tn / pbn : (tn + BN - 1) / BN;
  p.n_tiles = n_tiles, p.n_fills = n_fills;
  p.tile_i = tile_i, p.tile_j = tile_j, p.fill_i = fill_i, p.fill_j = fill_j;
  p.causal = causal ? 1 : 0, p.out_f32 = out_f32 ? 1 : 0, p.b_kmajor = y_transposed ? 1 : 0;
  p.tail_split = y_transposed ? 0 : TJX_GEMM_TAIL_SPLIT;  // (x @ y.T stages y through a box of fixed height)
  p.chain = launch_chain();  // (only the pair kernel looks at it: an ordinary launch is always right)
  p.num_kb = (K + BK - 1) / BK;
  p.out = out;
  p.row_scale = row_scale;
  p.activation = activation;
  p.status = device_status_word();
  if (p.status == nullptr) return fail(TJX_E_CUDA, "could not locate the device status word");

  CUtensorMap ma, mb, mc;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(K) * 2};
    const uint32_t box[2] = {BK, BM};
    if (int rc = make_tensor_map(&ma, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  if (y_transposed) {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(N)};
    const uint64_t strides[1] = {static_cast<uint64_t>(K) * 2};
    const uint32_t box[2] = {BK, static_cast<uint32_t>(pair ? pbn / 2 : BN)};
    if (int rc = make_tensor_map(&mb, y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  } else {
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(N) * 2};
    const uint32_t box[2] = {64, BK};
    if (int rc = make_tensor_map(&mb, y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    // Output staging: 32 rows x 128 bytes per store (64 bf16 or 32 f32 columns), 128-byte swizzled.
    const int elt = out_f32 ? 4 : 2;
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(N) * elt};
    const uint32_t box[2] = {static_cast<uint32_t>(128 / elt), 32};
    if (int rc = make_tensor_map(&mc, out, out_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                                 elt, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }

  const long long total_items = static_cast<long long>(n_tiles + n_fills) * p.sub_m * p.sub_n;
  if (total_items >= (1ll << 31)) return fail(TJX_E_LIMIT, "too many output tiles");
  int grid = static_cast<int>(total_items < sm_count() ? total_items : sm_count());
  if (g_gemm_cta_limit > 0 && grid > g_gemm_cta_limit) grid = g_gemm_cta_limit;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (pair) {
    int pairs = static_cast<int>(total_items < sm_count() / 2 ? total_items : sm_count() / 2);
    if (g_gemm_cta_limit > 0) pairs = std::max(1, std::min(pairs, g_gemm_cta_limit / 2));
    p.profile = profile_buffer(2 * pairs);
    if (pbn == 128) return launch_gemm_pair<128, PAIR_STAGES_128, PAIR_KSUB, false>(ma, mb, mc, ma, p, 2 * pairs, s);
    return launch_gemm_pair<PAIR_BN, PAIR_STAGES, PAIR_KSUB, false>(ma, mb, mc, ma, p, 2 * pairs, s);
  }
  p.profile = profile_buffer(grid);
  if (BN == 256) {
    if (stages == 3) return launch_gemm<256, 3>(ma, mb, mc, p, grid, s);
    return launch_gemm<256, 4>(ma, mb, mc, p, grid, s);
  }
  if (stages == 6) return launch_gemm<128, 6>(ma, mb, mc, p, grid, s);
  return launch_gemm<128, 4>(ma, mb, mc, p, grid, s);
}
}  // namespace tjx

extern "C" int tjx_gemm_bf16(const void* x, const void* y, void* out, int M, int N, int K, int y_transposed, int tm,
                             int tn, int tk, int stages, int out_f32, int causal, const int32_t* tile_i,
                             const int32_t* tile_j, int n_tiles, const int32_t* fill_i, const int32_t* fill_j,
                             int n_fills, tjx_stream_t stream) {
  return tjx::gemm_launch(x, y, out, M, N, K, y_transposed, tm, tn, tk, stages, out_f32, causal, tile_i, tile_j, n_tiles,
                          fill_i, fill_j, n_fills, nullptr, 0, stream);
}

// out = all_gather(x) @ y in ONE launch: the pair GEMM whose extra warp per CTA pulls the other ranks' shards from
// peer memory while the tensor cores work on the shards that are already here (the own one first).
extern "C" int tjx_all_gather_gemm_bf16(const void* x_own, const void* const* peer_shards, void* gathered,
                                        const void* y, void* out, int ranks, int me, int m, int N, int K, int tm,
                                        int tn, int tk, const int32_t* tile_i, const int32_t* tile_j, int n_tiles,
                                        int32_t* arrivals, int epoch, tjx_stream_t stream) {
  using namespace tjx;
  if (int rc = check_device()) return rc;
  if (!x_own || !peer_shards || !gathered || !y || !out || !arrivals || !tile_i || !tile_j)
    return fail(TJX_E_ARG, "a pointer is null");
  if (ranks < 2 || ranks > 8 || me < 0 || me >= ranks) return fail(TJX_E_ARG, "2 to 8 ranks, 0 <= me < ranks");
  if (m <= 0 || N <= 0 || K <= 0 || K % 8 != 0 || N % 8 != 0) return fail(TJX_E_ARG, "m, N, K must be positive, K and N multiples of 8");
  if (tm <= 0 || tn <= 0 || tk <= 0 || tm % PAIR_ROWS != 0 || tn % PAIR_BN != 0 || m % tm != 0 || N % tn != 0)
    return fail(TJX_E_ARG, "tm and tn must be multiples of 256 that divide a shard's rows and N");
  if (epoch <= 0 || epoch > (1 << 22)) return fail(TJX_E_ARG, "epoch counts this buffer's calls from 1 (at most 2^22)");
  const long long M = static_cast<long long>(ranks) * m;
  if (M >= (1ll << 31) || n_tiles != (M / tm) * (N / tn))
    return fail(TJX_E_ARG, "the tile table must list every tile of the [ranks * m, N] output once");
  for (int r = 0; r < ranks; ++r)
    if (r != me && (peer_shards[r] == nullptr || (reinterpret_cast<uintptr_t>(peer_shards[r]) & 15u)))
      return fail(TJX_E_ARG, "a peer shard pointer is null or not 16-byte aligned");

  GemmParams p{};
  p.M = static_cast<int>(M), p.N = N, p.K = K, p.tm = tm, p.tn = tn;
  p.tiles_m = static_cast<int>(M / tm), p.tiles_n = N / tn, p.band_tiles = 1;
  p.sub_m = tm / PAIR_ROWS, p.sub_n = tn / PAIR_BN;
  p.n_tiles = n_tiles, p.n_fills = 0, p.tile_i = tile_i, p.tile_j = tile_j;
  p.num_kb = (K + BK - 1) / BK;
  p.out = out;
  p.status = device_status_word();
  if (p.status == nullptr) return fail(TJX_E_CUDA, "could not locate the device status word");
  p.gather_ranks = ranks, p.gather_me = me, p.gather_rows = m, p.gather_epoch = epoch;
  for (int r = 0; r < ranks; ++r) p.gather_src[r] = r == me ? nullptr : peer_shards[r];
  p.gather_dst = gathered, p.gather_arrivals = arrivals;

  CUtensorMap ma, ma_own, mb, mc;
  const uint32_t box_a[2] = {BK, BM};
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(K) * 2};
    if (int rc = make_tensor_map(&ma, gathered, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, dims, strides, box_a,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(m)};
    const uint64_t strides[1] = {static_cast<uint64_t>(K) * 2};
    if (int rc = make_tensor_map(&ma_own, x_own, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, dims, strides, box_a,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
    const uint64_t strides[1] = {static_cast<uint64_t>(N) * 2};
    const uint32_t box[2] = {64, BK};
    if (int rc = make_tensor_map(&mb, y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(M)};
    const uint64_t strides[1] = {static_cast<uint64_t>(N) * 2};
    const uint32_t box[2] = {64, 32};
    if (int rc = make_tensor_map(&mc, out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 2, dims, strides, box,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  // Every CTA must be resident at once (the producers wait on counters the copier warps of all CTAs raise): one
  // CTA per SM, never more CTAs than SMs.
  const long long total_items = static_cast<long long>(n_tiles) * p.sub_m * p.sub_n;
  const int pairs = static_cast<int>(std::min<long long>(total_items, sm_count() / 2));
  p.profile = profile_buffer(2 * pairs);
  return launch_gemm_pair<PAIR_BN, PAIR_STAGES, PAIR_KSUB, true>(ma, mb, mc, ma_own, p, 2 * pairs,
                                                                static_cast<cudaStream_t>(stream));
}

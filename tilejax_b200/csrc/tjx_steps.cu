// Device step tables for runtime masks: which (tile, reduction block) steps run, compacted to the front in
// order, with the skipped ones behind them in their original order — exactly what the reference's generated
// `<kernel>_steps` returns (src/autokernel/codegen.py:386-431: keep = run | empty, first/last by argmax, packed
// codes, stable argsort of !keep). A stable partition needs no sort: one pass counts each tile's steps, a scan
// places the tiles, a second pass scatters every entry to its final position.
//
// One CTA of 32 warps, a warp per tile at a time; the whole table is a few thousand entries (decode: 64 x 256).
#include "tjx_host.cuh"
#include "tjx_ptx.cuh"

#include "../../include/tilejax_b200.h"

namespace tjx {

constexpr int STEPS_THREADS = 1024;
constexpr int STEPS_MAX_TILES = 8192;  // per-tile counters live in shared memory
constexpr int STEPS_LEN_CACHE = 2048;  // tables of up to this many tiles fetch every tile's length in one round

// run(t, k): does block k of tile t run? Masks `value0 + k * value_step >= lengths[tile_values[t]]` skip.
struct RunFromLengths {
  const int32_t* lengths;
  const int32_t* tile_values;
  int n_lengths;
  int value0, value_step;
  __device__ int length_of(int t) const {
    int idx = tile_values ? tile_values[t] : t;
    idx = min(max(idx, 0), n_lengths - 1);
    return lengths[idx];
  }
  __device__ bool run(int len, int, int k) const { return !(value0 + k * value_step >= len); }
};

struct RunFromBitmap {
  const uint8_t* bits;
  int blocks;
  __device__ int length_of(int) const { return 0; }
  __device__ bool run(int, int t, int k) const { return bits[static_cast<size_t>(t) * blocks + k] != 0; }
};

template <class Run>
__global__ void __launch_bounds__(STEPS_THREADS) build_steps_kernel(Run mask, int tiles, int blocks,
                                                                    int32_t* __restrict__ step_tile,
                                                                    int32_t* __restrict__ step_code,
                                                                    int32_t* __restrict__ step_count,
                                                                    int32_t* __restrict__ tile_first,
                                                                    int32_t* __restrict__ zero_words, int n_zero) {
  __shared__ int s_runs[STEPS_MAX_TILES];   // blocks that run per tile, then the tile's first step (scan)
  __shared__ int s_len[STEPS_LEN_CACHE];
  __shared__ int s_warp_sums[32];
  __shared__ int s_carry;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = STEPS_THREADS / 32;
  // A kernel launched behind this one with programmatic stream serialisation may start its prologue now; it
  // still waits for this whole grid before it reads the tables.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // Every tile's length in one round of (dependent) global loads, instead of one round per tile per pass.
  const bool cached = tiles <= STEPS_LEN_CACHE;
  if (cached) {
    for (int t = threadIdx.x; t < tiles; t += STEPS_THREADS) s_len[t] = mask.length_of(t);
  }
  // Words the caller wants cleared before its next kernel (arrival counters of the decode kernel).
  for (int i = threadIdx.x; i < n_zero; i += STEPS_THREADS) zero_words[i] = 0;
  if (cached) __syncthreads();

  // Pass 1: blocks that run in each tile.
  for (int t = warp; t < tiles; t += n_warps) {
    const int len = cached ? s_len[t] : mask.length_of(t);
    int n = 0;
    for (int k0 = 0; k0 < blocks; k0 += 32) {
      const int k = k0 + lane;
      const bool r = k < blocks && mask.run(len, t, k);
      n += __popc(__ballot_sync(0xFFFFFFFFu, r));
    }
    if (lane == 0) s_runs[t] = n;
  }
  if (threadIdx.x == 0) s_carry = 0;
  __syncthreads();

  // Scan: a tile takes max(runs, 1) steps (one empty step if nothing runs). s_runs[t] becomes
  // first_step(t) * 2 + (the tile is empty), so pass 2 needs no second array.
  for (int base = 0; base < tiles; base += STEPS_THREADS) {
    const int t = base + threadIdx.x;
    const int runs = t < tiles ? s_runs[t] : 0;
    const int steps = t < tiles ? max(runs, 1) : 0;
    int incl = steps;
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xFFFFFFFFu, incl, d);
      if (lane >= d) incl += o;
    }
    if (lane == 31) s_warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = lane < n_warps ? s_warp_sums[lane] : 0;
      for (int d = 1; d < 32; d <<= 1) {
        const int o = __shfl_up_sync(0xFFFFFFFFu, w, d);
        if (lane >= d) w += o;
      }
      s_warp_sums[lane] = w;
    }
    __syncthreads();
    const int before = s_carry + (warp ? s_warp_sums[warp - 1] : 0) + incl - steps;
    if (t < tiles) {
      s_runs[t] = before * 2 + (runs == 0 ? 1 : 0);
      if (tile_first) tile_first[t] = before;
    }
    __syncthreads();
    if (threadIdx.x == 0) s_carry += s_warp_sums[31];
    __syncthreads();
  }
  const int total = s_carry;
  if (threadIdx.x == 0) {
    step_count[0] = total;
    if (tile_first) tile_first[tiles] = total;
  }

  // Pass 2: scatter. Steps that run go to first_step(t) + rank; the others behind all of them, in tile-major
  // order: their position is total + (entries before them) - (kept entries before them).
  for (int t = warp; t < tiles; t += n_warps) {
    const int len = cached ? s_len[t] : mask.length_of(t);
    const int first_step = s_runs[t] >> 1;
    const bool empty_tile = s_runs[t] & 1;
    const int next_first = (t + 1 < tiles) ? (s_runs[t + 1] >> 1) : total;
    const int kept_in_tile = next_first - first_step;
    int rank0 = 0;  // kept entries of this tile before this chunk
    for (int k0 = 0; k0 < blocks; k0 += 32) {
      const int k = k0 + lane;
      const bool in = k < blocks;
      const bool r = in && mask.run(len, t, k);
      const bool empty = empty_tile && k == 0;
      const bool keep = r || empty;
      const unsigned ballot = __ballot_sync(0xFFFFFFFFu, keep);
      const int rank = rank0 + __popc(ballot & ((1u << lane) - 1u));
      if (in) {
        const bool first = keep && rank == 0;
        const bool last = keep && rank == kept_in_tile - 1;
        const int code = (k << 3) | (empty ? 4 : 0) | (first ? 2 : 0) | (last ? 1 : 0);
        const int pos = keep ? first_step + rank : total + (t * blocks + k) - (first_step + rank);
        step_tile[pos] = t;
        step_code[pos] = code;
      }
      rank0 += __popc(ballot);
    }
  }
}

static int check_common(int tiles, int blocks, const void* a, const void* b, const void* c) {
  if (a == nullptr || b == nullptr || c == nullptr) return fail(TJX_E_ARG, "step table output pointer is null");
  if (tiles <= 0 || blocks <= 0) return fail(TJX_E_ARG, "tiles and blocks must be positive");
  if (tiles > STEPS_MAX_TILES) return fail(TJX_E_LIMIT, "more than 8192 tiles in a device step table");
  if (blocks >= (1 << 28) || static_cast<long long>(tiles) * blocks >= (1ll << 31))
    return fail(TJX_E_LIMIT, "the step codes do not fit in int32");
  return 0;
}

// The size limits alone, for an entry point that must refuse before its first launch.
int check_step_table_sizes(int tiles, int blocks) {
  static const int placeholder = 0;
  return check_common(tiles, blocks, &placeholder, &placeholder, &placeholder);
}

int launch_build_steps_lengths(const int32_t* lengths, int n_lengths, const int32_t* tile_values, int tiles,
                               int blocks, int value0, int value_step, int32_t* step_tile, int32_t* step_code,
                               int32_t* step_count, int32_t* tile_first, int32_t* zero_words, int n_zero,
                               cudaStream_t stream) {
  // Every caller comes through here, the decode entry points included: the size limits of the kernel's shared
  // arrays are enforced before anything is launched.
  if (int rc = check_common(tiles, blocks, step_tile, step_code, step_count)) return rc;
  RunFromLengths mask{lengths, tile_values, n_lengths, value0, value_step};
  build_steps_kernel<<<1, STEPS_THREADS, 0, stream>>>(mask, tiles, blocks, step_tile, step_code, step_count,
                                                      tile_first, zero_words, n_zero);
  TJX_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace tjx

extern "C" {

int tjx_build_steps(const int32_t* lengths, int n_lengths, const int32_t* tile_values, int tiles, int blocks,
                    int value0, int value_step, int32_t* step_tile, int32_t* step_code, int32_t* step_count,
                    int32_t* tile_first, tjx_stream_t stream) {
  if (int rc = tjx::check_device()) return rc;
  if (lengths == nullptr || n_lengths <= 0) return tjx::fail(TJX_E_ARG, "lengths is null or empty");
  if (value_step <= 0) return tjx::fail(TJX_E_ARG, "value_step must be positive (loops count up)");
  return tjx::launch_build_steps_lengths(lengths, n_lengths, tile_values, tiles, blocks, value0, value_step,
                                         step_tile, step_code, step_count, tile_first, nullptr, 0,
                                         static_cast<cudaStream_t>(stream));
}

int tjx_build_steps_from_runs(const uint8_t* run, int tiles, int blocks, int32_t* step_tile, int32_t* step_code,
                              int32_t* step_count, int32_t* tile_first, tjx_stream_t stream) {
  if (int rc = tjx::check_device()) return rc;
  if (int rc = tjx::check_common(tiles, blocks, step_tile, step_code, step_count)) return rc;
  if (run == nullptr) return tjx::fail(TJX_E_ARG, "run is null");
  tjx::RunFromBitmap mask{run, blocks};
  tjx::build_steps_kernel<<<1, tjx::STEPS_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      mask, tiles, blocks, step_tile, step_code, step_count, tile_first, nullptr, 0);
  TJX_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"

/* tilejax_b200 — C ABI of the sm_100a step-loop kernels.
 *
 * Every entry point takes plain pointers and sizes, enqueues work on the CUDA stream it is given and returns
 * without synchronising: 0 on success, a negative TJX_E_* code otherwise (tjx_last_error() has the text).
 * Unless stated otherwise every data pointer is DEVICE memory that the callee borrows for the duration of
 * the enqueued work; nothing is allocated per call. The library never falls back to the CPU: on a device
 * that is not compute capability 10.x every compute entry point returns TJX_E_DEVICE.
 *
 * Each declaration cites the part of the reference (RKKatakam/tilejax, package `autokernel`) it stands in
 * for, by path within that project.
 */
#ifndef TILEJAX_B200_H_
#define TILEJAX_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* tjx_stream_t; /* a cudaStream_t */

#define TJX_E_ARG (-1)    /* bad argument: shape, alignment, null pointer */
#define TJX_E_CUDA (-2)   /* a CUDA call failed */
#define TJX_E_DEVICE (-3) /* not an sm_100 device */
#define TJX_E_LIMIT (-4)  /* a size exceeds what the entry point supports */
#define TJX_E_KERNEL (-5) /* a kernel reported an error through its status word */

/* Library version: major * 10000 + minor * 100 + patch. */
int tjx_version(void);

/* Text of the calling thread's last error ("" if none). */
const char* tjx_last_error(void);

/* Synchronises `stream`, then reads and clears the current device's kernel status word: *code is 0, or the
 * code of the first bounded wait that ran out inside a kernel (1xx). Returns 0, or TJX_E_KERNEL if *code != 0.
 * Replaces nothing in the reference: its kernels cannot report errors; here every device-side wait is bounded
 * and gives up through this word instead of hanging. */
int tjx_device_status(tjx_stream_t stream, int* code);

/* In-kernel profile, the counterpart of the trace regions the reference's generated kernels carry
 * (`<kernel>/wait`, `/out_wait`, `/compute`: src/autokernel/profiling.py:1-20, src/autokernel/codegen.py REGIONS).
 * While a buffer is set for the calling thread, every matmul, attention and paged-decode launch from it whose grid
 * fits writes one record of sixteen int64 per CTA (record i = CTA i; later launches overwrite earlier ones):
 *   [0] SM clock at CTA start, [1] when its issuing thread (MMA issuer; decode: warp 0) starts its first work item,
 *   [2] after its last, [3] cycles that thread waited for inputs, [4] of which its first wait (the pipeline
 *   filling), [5] cycles it waited for room for results (accumulator / output slot still draining), [6] work items,
 *   [7] SM clock at CTA end, [8..15] kernel-specific (attention: [8] cycles the MMA thread waited for the softmax
 *   warps' probabilities).
 * NULL unsets it. The buffer is device memory the caller owns: zero it before a launch to tell which CTAs wrote. */
int tjx_set_profile_buffer(void* device_buffer, size_t bytes);

/* Sets, for the current device, how long a device-side wait (on a ring slot, an accumulator, a peer's rows) may
 * last before the kernel gives up, records its code in the status word and returns: 1000 .. 10,000,000
 * microseconds, 2 s unless changed. Synchronises the device. Replaces nothing in the reference (see
 * tjx_device_status); a caller that prefers a failed step to a two-second stall lowers it, and the tests use a
 * short limit to take the give-up path on purpose. */
int tjx_set_wait_limit_us(int microseconds);

/* The device step-table builder for runtime masks of the form `value(k) >= lengths[tile_value[t]]: continue`
 * with value(k) = value0 + k * value_step — `paged_gqa_decode` (examples/decode.py:214, value = p * page_size)
 * and `gqa_decode` (examples/decode.py:188, value = j).
 * Stands in for the generated `<kernel>_steps` / `_phase_steps` (src/autokernel/codegen.py:376-451).
 *   lengths      int32[n_lengths]   index array the mask reads
 *   tile_values  int32[tiles] or NULL (NULL = 0..tiles-1): which length each tile reads (Schedule.tile_values,
 *                src/autokernel/schedule.py:267)
 *   step_tile    int32[tiles * blocks]  OUT  each step's tile
 *   step_code    int32[tiles * blocks]  OUT  block << 3 | empty << 2 | first << 1 | last
 *   step_count   int32[1]               OUT  steps that run (they come first, in order; the others follow in
 *                                            their original order, as the reference's stable argsort leaves them)
 *   tile_first   int32[tiles + 1] or NULL  OUT  extra: index of each tile's first step among those that run
 */
int tjx_build_steps(const int32_t* lengths, int n_lengths, const int32_t* tile_values, int tiles, int blocks,
                    int value0, int value_step, int32_t* step_tile, int32_t* step_code, int32_t* step_count,
                    int32_t* tile_first, tjx_stream_t stream);

/* The same compaction for an arbitrary mask already evaluated: run[t * blocks + k] != 0 where block k of tile t
 * runs (uint8). Follows src/autokernel/codegen.py:386-431 for any pattern of skipped blocks. */
int tjx_build_steps_from_runs(const uint8_t* run, int tiles, int blocks, int32_t* step_tile, int32_t* step_code,
                              int32_t* step_count, int32_t* tile_first, tjx_stream_t stream);

/* The step loop of `matmul` (examples/matmul.py:22-35), `causal_matmul` (examples/causal_matmul.py:23-40) and
 * the compute half of `all_gather_matmul` (examples/collective_matmul.py:44-59): out = x @ y with bf16
 * operands, f32 accumulation (src/autokernel/mxu.py:21-43) and a bf16 or f32 result, one output tile of
 * (tm, tn) after another, each summing K in blocks. Replaces the generated kernel's loop
 * (src/autokernel/codegen.py:1433-1538) with a persistent TMA + tcgen05 kernel.
 *   x [M, K] bf16 row-major; y [K, N] bf16 row-major, or [N, K] if y_transposed (x @ y.T, mxu.py:38-43)
 *   out [M, N] bf16, or f32 if out_f32
 *   tile_i, tile_j  int32[n_tiles] or NULL: block indices (i / tm, j / tn) of the tiles that run, in order
 *                   (Schedule.tables "tile_i"/"tile_j", src/autokernel/schedule.py:349-358); NULL = every tile,
 *                   row-major
 *   fill_i, fill_j  int32[n_fills] or NULL: tiles the mask skips, written with zeros (the output's fill)
 *   causal          != 0: entries above the diagonal of a computed tile are zero (`jnp.where(cols <= rows, ..)`)
 *   tk              the reduction block: reported only; the kernel sums K in its own blocks of 64
 *   stages          depth of the shared-memory ring (2..6; 0 = default)
 * Constraints: K % 8 == 0, N % 8 == 0; tm % 128 == 0 or tm == M; tn % 128 == 0 or tn == N. */
int tjx_gemm_bf16(const void* x, const void* y, void* out, int M, int N, int K, int y_transposed, int tm, int tn,
                  int tk, int stages, int out_f32, int causal, const int32_t* tile_i, const int32_t* tile_j,
                  int n_tiles, const int32_t* fill_i, const int32_t* fill_j, int n_fills, tjx_stream_t stream);

/* Bytes of scratch tjx_rmsnorm_gemm_bf16 needs for these sizes. */
size_t tjx_rmsnorm_gemm_workspace_bytes(int M, int D);

/* RMSNorm fused with the projection after it, the loop nest `rmsnorm_matmul` (examples/rmsnorm_matmul.py:31-47):
 * out = rsqrt(mean(x^2, axis 1) + eps) * ((x * gamma) @ w). One pass over x writes the gamma-scaled operand
 * bf16(f32(x) * f32(gamma)) — what the reference's `@` is fed (examples/rmsnorm_matmul.py:44) — and each row's scale
 * into `workspace`; the matmul step loop then multiplies row r of its f32 accumulator by scale[r] before the one
 * rounding to the output dtype (the nest's fused epilogue, examples/rmsnorm_matmul.py:45-46).
 *   x [M, D] bf16, gamma [1, D] bf16, w [D, N] bf16, out [M, N] bf16 (f32 if out_f32)
 *   workspace: at least tjx_rmsnorm_gemm_workspace_bytes(M, D) bytes, 256-byte aligned
 * Constraints: those of tjx_gemm_bf16 with K = D. */
int tjx_rmsnorm_gemm_bf16(const void* x, const void* gamma, const void* w, void* out, int M, int N, int D, float eps,
                          int tm, int tn, int tk, int out_f32, void* workspace, size_t workspace_bytes,
                          tjx_stream_t stream);

/* Bytes of scratch tjx_attention_block_bf16 needs for these sizes. */
size_t tjx_attention_block_workspace_bytes(int B, int H, int S, int Dh, int F);

/* A whole attention block, the two-phase loop nest `attention_block` (examples/attention_block.py:49-85): causal
 * multi-head attention (phase 1, the step tables' key blocks per query tile, as tjx_causal_attention_bf16), the heads
 * put side by side in f32, RMSNorm over the model dimension D = H * Dh, and the feed-forward layer
 * out = bf16(gelu(n @ w_up)) @ w_down (phase 2; tanh GELU, jax.nn.gelu's default) with f32 accumulation in both
 * products (src/autokernel/mxu.py:21-35). Where the reference keeps a query block's intermediates on chip, this runs
 * four launches on `stream` with them in `workspace`: attention, a row-wise norm, and two matmul step loops.
 *   q, k, v [B, H, S, Dh] bf16 (q pre-scaled); gamma [1, D] bf16; w_up [D, F] bf16; w_down [F, D] bf16
 *   out [B, S, D] bf16
 *   block_q, block_kv, step_tile, step_code, pattern_steps, pattern_tiles: as tjx_causal_attention_bf16
 *   workspace: at least tjx_attention_block_workspace_bytes(B, H, S, Dh, F) bytes, 256-byte aligned
 * Constraints: Dh == 128; S % 128 == 0; F % 128 == 0. */
int tjx_attention_block_bf16(const void* q, const void* k, const void* v, const void* gamma, const void* w_up,
                             const void* w_down, void* out, int B, int H, int S, int Dh, int F, int block_q,
                             int block_kv, float eps, const int32_t* step_tile, const int32_t* step_code,
                             int pattern_steps, int pattern_tiles, void* workspace, size_t workspace_bytes,
                             tjx_stream_t stream);

/* Caps the number of persistent CTAs tjx_gemm_bf16 launches from the calling thread (0 = one per SM, the
 * default). For callers that run communication kernels beside the GEMM — the collective matmul's exchange rounds
 * stand in for the ring DMAs of the reference's kernel (src/autokernel/codegen.py:1161-1229), which need no
 * compute units on a TPU but do on a GPU — so that those kernels find free SMs instead of delaying GEMM CTAs. */
int tjx_gemm_set_cta_limit(int max_ctas);

/* Chooses how tjx_gemm_bf16 maps CTA tiles to SMs for calls from this thread: 1 (default; 3 is the same) = one MMA
 * per pair of SMs, in pieces of 256 x 256, whenever tm % 256 == 0, tn % 256 == 0 and stages == 0; 2 = pairs with
 * 256 x 128 pieces (an A/B switch: measured slower); 0 = always one 128 x 256 (or 128 x 128) piece per SM. Results
 * are bit-identical: every mode sums K in the same order. The counterpart in the reference is the choice of tile
 * sizes left to its tuner (src/autokernel/tune.py:246-300): a launch-shape knob with no effect on values. */
int tjx_gemm_set_pair_mode(int mode);

/* `all_gather_matmul` in one launch (the ring kernel of src/autokernel/codegen.py:1149-1229, whose remote DMAs run
 * beside its matmul steps): out[ranks * m, N] = all_gather(x) @ y on this rank. The GEMM kernel carries one extra
 * warp per CTA that pulls the other ranks' shards out of peer memory (plain 16-byte loads over NVLink) into
 * `gathered`, 256 rows at a time in the order the ring would deliver them (round r: rank (me - r) mod ranks),
 * while the tensor cores work through the tile table — the own shard's tiles first, straight from x_own. A tile of
 * a remote shard starts once every CTA's slice of its 256-row block has landed (`arrivals`).
 *   peer_shards   ranks pointers: rank r's [m, K] shard as mapped into THIS process (entry `me` is ignored). Every
 *                 peer's shard must be complete and stay unchanged until this launch has finished on every rank:
 *                 the caller orders that with its own cross-rank barrier on the stream, before and after.
 *   gathered      [ranks * m, K] bf16 scratch on this GPU (rows of rank `me` are never written or read)
 *   tile_i/tile_j every (row tile, column tile) of the output once, in the order to walk them: own shard first, then
 *                 shards in arrival order (Schedule.tables of `all_gather_matmul`, src/autokernel/schedule.py:150-194)
 *   arrivals      int32[ranks * m / 256], zero before the first call; `epoch` = 1, 2, 3, ... counts the calls that
 *                 used this array (it is never reset)
 * Constraints: tm % 256 == 0, tn % 256 == 0, m % tm == 0, N % tn == 0, K % 8 == 0; 2 <= ranks <= 8. The launch
 * occupies every SM (its CTAs wait on one another's copier warps): run nothing else on the GPU beside it. */
int tjx_all_gather_gemm_bf16(const void* x_own, const void* const* peer_shards, void* gathered, const void* y,
                             void* out, int ranks, int me, int m, int N, int K, int tm, int tn, int tk,
                             const int32_t* tile_i, const int32_t* tile_j, int n_tiles, int32_t* arrivals, int epoch,
                             tjx_stream_t stream);

/* Flash-style causal attention, the step loop of `causal_attention` (examples/causal_attention.py:37-63):
 * q (pre-scaled), k, v, out [B, H, S, D] bf16, D == 128; online softmax in f32, P rounded to bf16 before P @ v.
 *   step_tile, step_code  int32[pattern_steps]: one (b, h)'s steps (Schedule.tables "step_tile"/"step_code",
 *                         src/autokernel/schedule.py:196-211): tile = query block, code = kv block << 3 | flags
 *   pattern_tiles         query blocks per (b, h) = S / block_q */
int tjx_causal_attention_bf16(const void* q, const void* k, const void* v, void* out, int B, int H, int S, int D,
                              int block_q, int block_kv, const int32_t* step_tile, const int32_t* step_code,
                              int pattern_steps, int pattern_tiles, tjx_stream_t stream);

/* Bytes of scratch tjx_paged_gqa_decode_bf16 needs for these sizes. */
size_t tjx_paged_gqa_decode_workspace_bytes(int B, int T, int H, int D, int pages_per_seq);

/* Ragged paged GQA decode attention, `paged_gqa_decode` (examples/decode.py:199-223) for T new tokens per
 * sequence: builds the step tables on the device from `lengths` (as the generated entry does before its kernel,
 * src/autokernel/codegen.py:465-467), then walks only the pages that hold valid positions.
 *   q [B, T, H, D] bf16 (pre-scaled); k_pages, v_pages [num_pages, page_size, Hkv * D] bf16
 *   block_tables int32[B, pages_per_seq] (entries clamped to [0, num_pages - 1], codegen.py:1045-1048)
 *   lengths int32[B], the new tokens included (0 = empty slot: its output is 0); out [B, T, H, D] bf16.
 *   New token t sits at position lengths[b] - T + t and attends to the positions up to its own (`visible`,
 *   examples/decode.py:145-152).
 *   step_tile, step_code int32[B * pages_per_seq], step_count int32[1], tile_first int32[B + 1]: OUT, the
 *   tables this call built and walked (bit-exact with the reference's)
 *   workspace: scratch of at least tjx_paged_gqa_decode_workspace_bytes(...) bytes, 256-byte aligned
 * Constraints: D == 128; H / Hkv in {1, 2, 4, 8}; T * (H / Hkv) <= 16; page_size a multiple of 16. */
int tjx_paged_gqa_decode_bf16(const void* q, const void* k_pages, const void* v_pages, const int32_t* block_tables,
                              const int32_t* lengths, void* out, int B, int T, int H, int Hkv, int D, int page_size,
                              int pages_per_seq, int num_pages, int32_t* step_tile, int32_t* step_code,
                              int32_t* step_count, int32_t* tile_first, void* workspace, size_t workspace_bytes,
                              tjx_stream_t stream);

/* Ragged paged attention, the in-place cache write (`rpa_write` with its runs, examples/ragged_paged_attention.py:33-79):
 * the step's new keys and values [T, Hkv, D] go to positions [kv_len - q_len, kv_len) of their sequences in the cache
 * [num_pages, page_size, Hkv, 2, D] (each head's key and value side by side), through page_indices
 * [S * pages_per_seq]; cu_q_lens [S + 1] gives each sequence's first token; sequences from distribution[2] on and
 * padding tokens (t >= cu_q_lens[S]) write nothing. One launch, a CTA per token. Constraint: D == 128. */
int tjx_rpa_write_bf16(void* kv_cache, const void* keys, const void* values, const int32_t* kv_lens,
                       const int32_t* page_indices, const int32_t* cu_q_lens, const int32_t* distribution, int T,
                       int S, int Hkv, int D, int page_size, int pages_per_seq, int num_pages, tjx_stream_t stream);

/* The same write from run tables, as the reference's `rpa_write` kernel takes them (examples/ragged_paged_attention.py:
 * 33-47; its `writes`, :49-71, makes them in plain JAX): run w < n_writes[0] copies the tokens from write_rows[w] on to
 * rows write_first[w] .. write_stop[w] - 1 of page page_indices[write_page[w]]. The table arrays are int32[max_runs],
 * n_writes int32[1], page_indices int32[n_page_indices]; rows, tokens or runs out of range write nothing. In place. */
int tjx_rpa_write_runs_bf16(void* kv_cache, const void* keys, const void* values, const int32_t* page_indices,
                            const int32_t* write_page, const int32_t* write_rows, const int32_t* write_first,
                            const int32_t* write_stop, const int32_t* n_writes, int T, int n_page_indices, int max_runs,
                            int Hkv, int D, int page_size, int num_pages, tjx_stream_t stream);

/* Bytes of scratch tjx_rpa_decode_bf16 needs for these sizes. */
size_t tjx_rpa_decode_workspace_bytes(int T, int S, int H, int D, int page_size, int pages_per_seq);

/* Ragged paged attention, the decode case (`rpa_decode`, examples/ragged_paged_attention.py:121-149): sequence
 * s < distribution[0] is token s; its query row q[s] [H, D] attends over the kv_lens[s] positions of its pages in the
 * cache (the new token already written), scores scaled by sm_scale; out[s] is the attention output and every other
 * row of out [T, H, D] is q's (out may be q: the update in place the reference's donated buffer gets). Runs the paged
 * decode kernel of tjx_paged_gqa_decode_bf16 on the cache's own layout (two tensor maps over the one buffer).
 *   workspace: at least tjx_rpa_decode_workspace_bytes(...) bytes, 256-byte aligned
 * Constraints: D == 128; H / Hkv in {1, 2, 4, 8}; page_size a multiple of 16. */
int tjx_rpa_decode_bf16(const void* q, void* out, const void* kv_cache, const int32_t* kv_lens,
                        const int32_t* page_indices, const int32_t* distribution, int T, int S, int H, int Hkv, int D,
                        int page_size, int pages_per_seq, int num_pages, float sm_scale, void* workspace,
                        size_t workspace_bytes, tjx_stream_t stream);

/* Bytes of scratch tjx_rpa_prefill_bf16 needs for these sizes (its tile arrays). */
size_t tjx_rpa_prefill_workspace_bytes(int T, int S);

/* Ragged paged attention, the prefill and mixed cases (`rpa_prefill` with its tiles,
 * examples/ragged_paged_attention.py:196-275): every sequence s in [distribution[0], distribution[2]) has
 * q_len = cu_q_lens[s + 1] - cu_q_lens[s] new tokens at cache positions [kv_lens[s] - q_len, kv_lens[s]); each attends
 * causally over its sequence's cache (the new tokens already written), scores scaled by sm_scale; the outputs replace
 * those tokens' rows of out [T, H, D], every other row of out is q's (out may be q). The tiles (here blocks of 128
 * queries; the reference's are 256) are built on the device; the kernel is the causal attention kernel's paged
 * instantiation: a unit is (tile, KV head, two of its query heads), a block one page.
 *   workspace: at least tjx_rpa_prefill_workspace_bytes(T, S) bytes, 256-byte aligned
 * Constraints: D == 128; page_size == 128; H / Hkv even. */
int tjx_rpa_prefill_bf16(const void* q, void* out, const void* kv_cache, const int32_t* kv_lens,
                         const int32_t* page_indices, const int32_t* cu_q_lens, const int32_t* distribution, int T,
                         int S, int H, int Hkv, int D, int page_size, int pages_per_seq, int num_pages, float sm_scale,
                         void* workspace, size_t workspace_bytes, tjx_stream_t stream);

/* Bytes of scratch tjx_rpa_prefill_tiles_bf16 needs for T token rows and tile tables of max_tiles entries. */
size_t tjx_rpa_prefill_tiles_workspace_bytes(int T, int max_tiles);

/* The same attention on the tile tables the reference's `rpa_prefill` kernel takes (examples/ragged_paged_attention.py:
 * 204-243; its `prefill_tiles`, :252-275, makes them in plain JAX): tile k < n_tiles[0] is the query rows tile_rows[k] ..
 * tile_rows[k + 1] - 1 of q (up to 256), the first at cache position tile_pos[k], of the sequence whose pages start at
 * page_indices[tile_page[k]]; a row at position p attends to the positions up to p. tile_page and tile_pos are
 * int32[max_tiles], tile_rows int32[max_tiles + 1], n_tiles int32[1]. A small kernel cuts the tiles into this kernel's
 * 128 queries; rows no tile covers keep q (out may be q). Constraints as tjx_rpa_prefill_bf16. */
int tjx_rpa_prefill_tiles_bf16(const void* q, void* out, const void* kv_cache, const int32_t* page_indices,
                               const int32_t* tile_page, const int32_t* tile_rows, const int32_t* tile_pos,
                               const int32_t* n_tiles, int T, int max_tiles, int n_page_indices, int H, int Hkv, int D,
                               int page_size, int num_pages, float sm_scale, void* workspace, size_t workspace_bytes,
                               tjx_stream_t stream);

/* Bytes of scratch tjx_ragged_paged_attention_bf16 needs for these sizes. */
size_t tjx_ragged_paged_attention_workspace_bytes(int T, int S, int H, int D, int page_size, int pages_per_seq);

/* One whole ragged paged attention step, the reference's `autokernel_rpa` (examples/ragged_paged_attention.py:279-290:
 * rpa_write, then rpa_decode, then rpa_prefill on its result) in one call: the new keys and values written into
 * kv_cache in place, then out [T, H, D] = the decode sequences' outputs in their rows, the prefill and mixed sequences'
 * outputs in theirs, and q's rows everywhere else (out may be q). Same results as tjx_rpa_write_bf16,
 * tjx_rpa_decode_bf16 and tjx_rpa_prefill_bf16 called in that order, for inputs whose decode tokens and prefill tokens
 * are different rows; it spares their copy of q into out (the prefill queries are read from q itself), and its small
 * kernels are chained to run beside their neighbours on the stream.
 *   workspace: at least tjx_ragged_paged_attention_workspace_bytes(...) bytes, 256-byte aligned
 * Constraints: those of the three entry points together (D == 128; page_size == 128; H / Hkv in {2, 4, 8}; at most
 * 8192 sequences, the device step table's limit). Sizes and pointers are checked before the first launch: a call
 * that returns an error for them has not touched the cache. */
int tjx_ragged_paged_attention_bf16(const void* q, const void* keys, const void* values, void* kv_cache,
                                    const int32_t* kv_lens, const int32_t* page_indices, const int32_t* cu_q_lens,
                                    const int32_t* distribution, void* out, int T, int S, int H, int Hkv, int D,
                                    int page_size, int pages_per_seq, int num_pages, float sm_scale, void* workspace,
                                    size_t workspace_bytes, tjx_stream_t stream);

/* Which kernel tjx_mla_decode_bf16 launches from now on: 1 (the default) the tcgen05 kernel, 64 rows per CTA with
 * scores and output in TMEM; 0 the warp-level MMA kernel, 16 rows per CTA. An A/B switch for measurements: the two
 * agree to rounding. No counterpart in the reference. */
int tjx_mla_set_mode(int mode);

/* Bytes of scratch tjx_mla_decode_bf16 needs for these sizes (0 if block does not divide S). */
size_t tjx_mla_decode_workspace_bytes(int B, int T, int H, int S, int block);

/* Absorbed MLA decode attention, `mla_decode` (examples/decode.py:226-250) for T new tokens per sequence: scores
 * q_c . c_kv + q_r . k_rope against a contiguous latent cache, softmax over the positions new token t sees (those up
 * to lengths[b] - T + t, `visible`, examples/decode.py:145-152), output = each head's softmax-weighted latents.
 * Builds the step tables on the device from `lengths` (a step = one block of `block` positions; blocks with
 * block_index * block >= lengths[b] are skipped) and walks only those.
 *   q_c [B, T, H, 512], q_r [B, T, H, 128] bf16 (pre-scaled); c_kv [B, S, 512], k_rope [B, S, 128] bf16
 *   lengths int32[B], the new tokens included (0 = empty: output 0); out [B, T, H, 512] bf16
 *   step_tile, step_code int32[B * S / block], step_count int32[1], tile_first int32[B + 1]: OUT, the tables built
 *   workspace: at least tjx_mla_decode_workspace_bytes(...) bytes, 256-byte aligned
 * Constraints: C == 512, R == 128, H % 16 == 0, block % 16 == 0, S % block == 0. */
int tjx_mla_decode_bf16(const void* q_c, const void* q_r, const void* c_kv, const void* k_rope,
                        const int32_t* lengths, void* out, int B, int T, int H, int S, int C, int R, int block,
                        int32_t* step_tile, int32_t* step_code, int32_t* step_count, int32_t* tile_first,
                        void* workspace, size_t workspace_bytes, tjx_stream_t stream);

/* Bytes of scratch built into the library for tjx_paged_gqa_decode_bf16_static (36 MiB). */
#define TJX_STATIC_SCRATCH_BYTES (36u * 1024u * 1024u)
size_t tjx_paged_gqa_decode_static_scratch_bytes(void);

/* tjx_paged_gqa_decode_bf16 for callers that must not allocate device memory and have no scratch buffer of their
 * own to lend: code running inside a memory pool that is already carved up, a plugin whose host forbids
 * cudaMalloc after start-up, a serving loop that may not touch the allocator on its hot path. This entry point
 * has no counterpart in the reference; it exists only for those callers. Same arguments and same results as
 * tjx_paged_gqa_decode_bf16 minus the workspace: the online-softmax partials go to a fixed 36 MiB array inside the
 * library instead (every GPU that loads the library holds that array until the process exits). The call itself
 * performs no cudaMalloc / cudaFree and calls no allocating routine.
 *   Limit: tjx_paged_gqa_decode_workspace_bytes(B, T, H, D, pages_per_seq) must not exceed TJX_STATIC_SCRATCH_BYTES
 *   (for example B 64, H 32, 256 pages per sequence fits); beyond it the call returns TJX_E_LIMIT and runs nothing.
 *   First call on a device: looks the array's device address up (once per device, with that device current).
 *   Make that first call outside any stream capture.
 *   Sharing: all calls on a device use the same array. Nothing in it needs clearing between calls (each call
 *   writes every partial before reading it), but two calls whose kernels overlap on the GPU — different streams,
 *   or different host threads on different streams — race on it: keep calls to this entry point on one stream,
 *   or order them with events. */
int tjx_paged_gqa_decode_bf16_static(const void* q, const void* k_pages, const void* v_pages,
                                     const int32_t* block_tables, const int32_t* lengths, void* out, int B, int T,
                                     int H, int Hkv, int D, int page_size, int pages_per_seq, int num_pages,
                                     int32_t* step_tile, int32_t* step_code, int32_t* step_count, int32_t* tile_first,
                                     tjx_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* TILEJAX_B200_H_ */

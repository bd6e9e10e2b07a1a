// XLA FFI handlers over the C ABI (include/tilejax_b200.h): the thin jax.ffi custom calls that let the reference's
// front end — `Kernel.lowered` -> `entry(*inputs)` (src/autokernel/api.py:258-266, :69-72) — launch these kernels
// from jitted JAX programs. One handler per entry point; each borrows XLA's buffers for the duration of the enqueue,
// runs on the stream XLA passes, allocates nothing (step tables and scratch are extra results, as the reference's
// hidden `xs` output is: src/autokernel/codegen.py:475-477) and turns a TJX_E_* code into an FFI error, never an
// abort.
//
// Built only where jaxlib ships the FFI headers (`jax.ffi.include_dir()`): `python -m tilejax_b200.csrc.build --ffi`.
// JAX is not installed where this library is developed and tested, so this file is written against the documented
// API (xla/ffi/api/ffi.h) and is exercised only by tests that skip without JAX; the kernels themselves are tested
// through the same C ABI from ctypes.
//
// Python side (tilejax_b200/xla_ffi.py):
//   jax.ffi.register_ffi_target("tjx_gemm", jax.ffi.pycapsule(lib.TjxGemm), platform="CUDA")
//   out = jax.ffi.ffi_call("tjx_gemm", jax.ShapeDtypeStruct((M, N), jnp.bfloat16))(x, y, tile_i, tile_j, fill_i,
//                          fill_j, tm=..., tn=..., tk=..., stages=0, causal=0, y_transposed=0)
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "../../include/tilejax_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error Failed(int code) {
  const char* text = tjx_last_error();
  std::string message = "tilejax_b200 (code " + std::to_string(code) + "): " + (text ? text : "unknown error");
  const ffi::ErrorCode kind = code == TJX_E_ARG || code == TJX_E_LIMIT ? ffi::ErrorCode::kInvalidArgument
                              : code == TJX_E_DEVICE                   ? ffi::ErrorCode::kFailedPrecondition
                                                                       : ffi::ErrorCode::kInternal;
  return ffi::Error(kind, message);
}

ffi::Error Bad(const std::string& message) { return ffi::Error(ffi::ErrorCode::kInvalidArgument, message); }

int Dim(const ffi::AnyBuffer& b, size_t i) { return static_cast<int>(b.dimensions()[i]); }

// A table argument may be absent: the caller then passes an int32 buffer of zero elements.
const int32_t* Table(const ffi::AnyBuffer& b) {
  return b.element_count() == 0 ? nullptr : static_cast<const int32_t*>(b.untyped_data());
}

// ------------------------------------------------------------------------------------------------ step tables

ffi::Error BuildStepsImpl(cudaStream_t stream, ffi::AnyBuffer lengths, ffi::Result<ffi::AnyBuffer> step_tile,
                          ffi::Result<ffi::AnyBuffer> step_code, ffi::Result<ffi::AnyBuffer> step_count,
                          ffi::Result<ffi::AnyBuffer> tile_first, int32_t tiles, int32_t blocks, int32_t value0,
                          int32_t value_step) {
  if (lengths.element_type() != ffi::S32) return Bad("lengths must be int32");
  if (step_tile->element_count() < static_cast<size_t>(tiles) * blocks || tile_first->element_count() < static_cast<size_t>(tiles) + 1)
    return Bad("step_tile / step_code hold tiles * blocks entries and tile_first tiles + 1");
  const int rc = tjx_build_steps(static_cast<const int32_t*>(lengths.untyped_data()),
                                 static_cast<int>(lengths.element_count()), nullptr, tiles, blocks, value0, value_step,
                                 static_cast<int32_t*>(step_tile->untyped_data()),
                                 static_cast<int32_t*>(step_code->untyped_data()),
                                 static_cast<int32_t*>(step_count->untyped_data()),
                                 static_cast<int32_t*>(tile_first->untyped_data()), stream);
  return rc == 0 ? ffi::Error::Success() : Failed(rc);
}

// ------------------------------------------------------------------------------------------------ matmul

ffi::Error GemmImpl(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer y, ffi::AnyBuffer tile_i,
                    ffi::AnyBuffer tile_j, ffi::AnyBuffer fill_i, ffi::AnyBuffer fill_j,
                    ffi::Result<ffi::AnyBuffer> out, int32_t tm, int32_t tn, int32_t tk, int32_t stages, int32_t causal,
                    int32_t y_transposed) {
  if (x.element_type() != ffi::BF16 || y.element_type() != ffi::BF16) return Bad("x and y must be bfloat16");
  if (x.dimensions().size() != 2 || y.dimensions().size() != 2 || out->dimensions().size() != 2)
    return Bad("x, y and out are matrices");
  const bool f32 = out->element_type() == ffi::F32;
  if (!f32 && out->element_type() != ffi::BF16) return Bad("out must be bfloat16 or float32");
  const int M = Dim(x, 0), K = Dim(x, 1), N = y_transposed ? Dim(y, 0) : Dim(y, 1);
  if ((y_transposed ? Dim(y, 1) : Dim(y, 0)) != K || Dim(*out, 0) != M || Dim(*out, 1) != N)
    return Bad("shapes do not agree: x [M, K], y [K, N] (or [N, K] transposed), out [M, N]");
  const int rc = tjx_gemm_bf16(x.untyped_data(), y.untyped_data(), out->untyped_data(), M, N, K, y_transposed, tm, tn, tk,
                               stages, f32 ? 1 : 0, causal, Table(tile_i), Table(tile_j),
                               static_cast<int>(tile_i.element_count()), Table(fill_i), Table(fill_j),
                               static_cast<int>(fill_i.element_count()), stream);
  return rc == 0 ? ffi::Error::Success() : Failed(rc);
}

// ------------------------------------------------------------------------------------------------ attention

ffi::Error CausalAttentionImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v,
                               ffi::AnyBuffer step_tile, ffi::AnyBuffer step_code, ffi::Result<ffi::AnyBuffer> out,
                               int32_t block_q, int32_t block_kv, int32_t pattern_tiles) {
  if (q.element_type() != ffi::BF16 || k.element_type() != ffi::BF16 || v.element_type() != ffi::BF16)
    return Bad("q, k and v must be bfloat16");
  if (q.dimensions().size() != 4) return Bad("q, k, v and out are [B, H, S, D]");
  const int rc = tjx_causal_attention_bf16(q.untyped_data(), k.untyped_data(), v.untyped_data(), out->untyped_data(),
                                           Dim(q, 0), Dim(q, 1), Dim(q, 2), Dim(q, 3), block_q, block_kv,
                                           Table(step_tile), Table(step_code),
                                           static_cast<int>(step_tile.element_count()), pattern_tiles, stream);
  return rc == 0 ? ffi::Error::Success() : Failed(rc);
}

// ------------------------------------------------------------------------------------------------ paged decode

ffi::Error PagedGqaDecodeImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k_pages, ffi::AnyBuffer v_pages,
                              ffi::AnyBuffer block_tables, ffi::AnyBuffer lengths, ffi::Result<ffi::AnyBuffer> out,
                              ffi::Result<ffi::AnyBuffer> step_tile, ffi::Result<ffi::AnyBuffer> step_code,
                              ffi::Result<ffi::AnyBuffer> step_count, ffi::Result<ffi::AnyBuffer> tile_first,
                              ffi::Result<ffi::AnyBuffer> workspace) {
  if (q.element_type() != ffi::BF16 || k_pages.element_type() != ffi::BF16 || v_pages.element_type() != ffi::BF16)
    return Bad("q, k_pages and v_pages must be bfloat16");
  if (block_tables.element_type() != ffi::S32 || lengths.element_type() != ffi::S32)
    return Bad("block_tables and lengths must be int32");
  if (q.dimensions().size() != 4 || k_pages.dimensions().size() != 3 || block_tables.dimensions().size() != 2)
    return Bad("q [B, T, H, D], pages [num_pages, page_size, Hkv * D], block_tables [B, pages_per_seq]");
  const int B = Dim(q, 0), T = Dim(q, 1), H = Dim(q, 2), D = Dim(q, 3);
  const int num_pages = Dim(k_pages, 0), page_size = Dim(k_pages, 1), width = Dim(k_pages, 2);
  const int pages_per_seq = Dim(block_tables, 1);
  if (D <= 0 || width % D != 0) return Bad("the pages' width must be Hkv * D");
  const size_t need = tjx_paged_gqa_decode_workspace_bytes(B, T, H, D, pages_per_seq);
  // The workspace result is a uint8 buffer of `need` + 256 bytes; XLA aligns buffers, but the offset is taken anyway.
  uintptr_t ws = reinterpret_cast<uintptr_t>(workspace->untyped_data());
  const uintptr_t aligned = (ws + 255) & ~static_cast<uintptr_t>(255);
  if (workspace->size_bytes() < need + (aligned - ws)) return Bad("the workspace result is too small");
  const int rc = tjx_paged_gqa_decode_bf16(
      q.untyped_data(), k_pages.untyped_data(), v_pages.untyped_data(),
      static_cast<const int32_t*>(block_tables.untyped_data()), static_cast<const int32_t*>(lengths.untyped_data()),
      out->untyped_data(), B, T, H, width / D, D, page_size, pages_per_seq, num_pages,
      static_cast<int32_t*>(step_tile->untyped_data()), static_cast<int32_t*>(step_code->untyped_data()),
      static_cast<int32_t*>(step_count->untyped_data()), static_cast<int32_t*>(tile_first->untyped_data()),
      reinterpret_cast<void*>(aligned), need, stream);
  return rc == 0 ? ffi::Error::Success() : Failed(rc);
}

// Scratch comes as a uint8 result of the entry point's `..._workspace_bytes` + 256 bytes; XLA aligns buffers, but the
// offset to a 256-byte boundary is taken anyway. Returns null if the result is too small.
void* Aligned(ffi::Result<ffi::AnyBuffer>& workspace, size_t need) {
  const uintptr_t ws = reinterpret_cast<uintptr_t>(workspace->untyped_data());
  const uintptr_t aligned = (ws + 255) & ~static_cast<uintptr_t>(255);
  return workspace->size_bytes() < need + (aligned - ws) ? nullptr : reinterpret_cast<void*>(aligned);
}

// ------------------------------------------------------------------------------------------------ fused epilogues

ffi::Error RmsnormGemmImpl(cudaStream_t stream, ffi::AnyBuffer x, ffi::AnyBuffer gamma, ffi::AnyBuffer w,
                           ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::AnyBuffer> workspace, int32_t tm,
                           int32_t tn, int32_t tk, float eps) {
  if (x.element_type() != ffi::BF16 || gamma.element_type() != ffi::BF16 || w.element_type() != ffi::BF16)
    return Bad("x, gamma and w must be bfloat16");
  if (x.dimensions().size() != 2 || w.dimensions().size() != 2 || Dim(w, 0) != Dim(x, 1))
    return Bad("x [M, D], gamma [1, D], w [D, N]");
  const int M = Dim(x, 0), D = Dim(x, 1), N = Dim(w, 1);
  const int out_f32 = out->element_type() == ffi::F32 ? 1 : 0;
  if (!out_f32 && out->element_type() != ffi::BF16) return Bad("out must be bfloat16 or float32");
  const size_t need = tjx_rmsnorm_gemm_workspace_bytes(M, D);
  void* ws = Aligned(workspace, need);
  if (ws == nullptr) return Bad("the workspace result is too small");
  const int rc = tjx_rmsnorm_gemm_bf16(x.untyped_data(), gamma.untyped_data(), w.untyped_data(), out->untyped_data(), M,
                                       N, D, eps, tm, tn, tk, out_f32, ws, need, stream);
  return rc == 0 ? ffi::Error::Success() : Failed(rc);
}

ffi::Error AttentionBlockImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v,
                              ffi::AnyBuffer gamma, ffi::AnyBuffer w_up, ffi::AnyBuffer w_down, ffi::AnyBuffer step_tile,
                              ffi::AnyBuffer step_code, ffi::Result<ffi::AnyBuffer> out,
                              ffi::Result<ffi::AnyBuffer> workspace, int32_t block_q, int32_t block_kv,
                              int32_t pattern_tiles, float eps) {
  for (const ffi::AnyBuffer* b : {&q, &k, &v, &gamma, &w_up, &w_down})
    if (b->element_type() != ffi::BF16) return Bad("q, k, v, gamma, w_up and w_down must be bfloat16");
  if (q.dimensions().size() != 4 || w_up.dimensions().size() != 2) return Bad("q [B, H, S, Dh], w_up [D, F]");
  const int B = Dim(q, 0), H = Dim(q, 1), S = Dim(q, 2), Dh = Dim(q, 3), F = Dim(w_up, 1);
  const size_t need = tjx_attention_block_workspace_bytes(B, H, S, Dh, F);
  void* ws = Aligned(workspace, need);
  if (ws == nullptr) return Bad("the workspace result is too small");
  const int rc = tjx_attention_block_bf16(q.untyped_data(), k.untyped_data(), v.untyped_data(), gamma.untyped_data(),
                                          w_up.untyped_data(), w_down.untyped_data(), out->untyped_data(), B, H, S, Dh,
                                          F, block_q, block_kv, eps, Table(step_tile), Table(step_code),
                                          static_cast<int>(step_tile.element_count()), pattern_tiles, ws, need, stream);
  return rc == 0 ? ffi::Error::Success() : Failed(rc);
}

// ------------------------------------------------------------------------------------------------ MLA decode

ffi::Error MlaDecodeImpl(cudaStream_t stream, ffi::AnyBuffer q_c, ffi::AnyBuffer q_r, ffi::AnyBuffer c_kv,
                         ffi::AnyBuffer k_rope, ffi::AnyBuffer lengths, ffi::Result<ffi::AnyBuffer> out,
                         ffi::Result<ffi::AnyBuffer> step_tile, ffi::Result<ffi::AnyBuffer> step_code,
                         ffi::Result<ffi::AnyBuffer> step_count, ffi::Result<ffi::AnyBuffer> tile_first,
                         ffi::Result<ffi::AnyBuffer> workspace, int32_t block) {
  for (const ffi::AnyBuffer* b : {&q_c, &q_r, &c_kv, &k_rope})
    if (b->element_type() != ffi::BF16) return Bad("q_c, q_r, c_kv and k_rope must be bfloat16");
  if (lengths.element_type() != ffi::S32) return Bad("lengths must be int32");
  if (q_c.dimensions().size() != 4 || c_kv.dimensions().size() != 3 || k_rope.dimensions().size() != 3)
    return Bad("q_c [B, T, H, C], c_kv [B, S, C], k_rope [B, S, R]");
  const int B = Dim(q_c, 0), T = Dim(q_c, 1), H = Dim(q_c, 2), C = Dim(q_c, 3), S = Dim(c_kv, 1), R = Dim(k_rope, 2);
  const size_t need = tjx_mla_decode_workspace_bytes(B, T, H, S, block);
  void* ws = need == 0 ? nullptr : Aligned(workspace, need);
  if (ws == nullptr) return Bad("the block must divide the cache length, and the workspace result hold the scratch");
  const int rc = tjx_mla_decode_bf16(q_c.untyped_data(), q_r.untyped_data(), c_kv.untyped_data(), k_rope.untyped_data(),
                                     static_cast<const int32_t*>(lengths.untyped_data()), out->untyped_data(), B, T, H,
                                     S, C, R, block, static_cast<int32_t*>(step_tile->untyped_data()),
                                     static_cast<int32_t*>(step_code->untyped_data()),
                                     static_cast<int32_t*>(step_count->untyped_data()),
                                     static_cast<int32_t*>(tile_first->untyped_data()), ws, need, stream);
  return rc == 0 ? ffi::Error::Success() : Failed(rc);
}

// ------------------------------------------------------------------------------------ ragged paged attention

// The whole step (`autokernel_rpa`, examples/ragged_paged_attention.py:279-290). The cache is updated in place: the
// caller aliases the cache operand to the cache result (input_output_aliases), as the reference donates it; where XLA
// hands over two different buffers the old cache is copied into the result first, on the same stream.
ffi::Error RaggedPagedAttentionImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer keys, ffi::AnyBuffer values,
                                    ffi::AnyBuffer kv_cache, ffi::AnyBuffer kv_lens, ffi::AnyBuffer page_indices,
                                    ffi::AnyBuffer cu_q_lens, ffi::AnyBuffer distribution,
                                    ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::AnyBuffer> cache_out,
                                    ffi::Result<ffi::AnyBuffer> workspace, float sm_scale) {
  for (const ffi::AnyBuffer* b : {&q, &keys, &values, &kv_cache})
    if (b->element_type() != ffi::BF16) return Bad("q, keys, values and kv_cache must be bfloat16");
  for (const ffi::AnyBuffer* b : {&kv_lens, &page_indices, &cu_q_lens, &distribution})
    if (b->element_type() != ffi::S32) return Bad("kv_lens, page_indices, cu_q_lens and distribution must be int32");
  if (q.dimensions().size() != 3 || keys.dimensions().size() != 3 || kv_cache.dimensions().size() != 5)
    return Bad("q [T, H, D], keys and values [T, Hkv, D], kv_cache [pages, page_size, Hkv, 2, D]");
  const int T = Dim(q, 0), H = Dim(q, 1), D = Dim(q, 2), Hkv = Dim(kv_cache, 2);
  const int num_pages = Dim(kv_cache, 0), page_size = Dim(kv_cache, 1);
  const int S = static_cast<int>(kv_lens.element_count());
  if (S <= 0 || page_indices.element_count() % static_cast<size_t>(S) != 0 ||
      cu_q_lens.element_count() != static_cast<size_t>(S) + 1 || distribution.element_count() != 3)
    return Bad("page_indices holds S * pages_per_seq entries, cu_q_lens S + 1, distribution 3");
  const int pages_per_seq = static_cast<int>(page_indices.element_count() / static_cast<size_t>(S));
  if (cache_out->size_bytes() != kv_cache.size_bytes()) return Bad("the cache result must have the cache's size");
  const size_t need = tjx_ragged_paged_attention_workspace_bytes(T, S, H, D, page_size, pages_per_seq);
  void* ws = need == 0 ? nullptr : Aligned(workspace, need);
  if (ws == nullptr) return Bad("the workspace result is too small");
  if (cache_out->untyped_data() != kv_cache.untyped_data()) {
    const cudaError_t e = cudaMemcpyAsync(cache_out->untyped_data(), kv_cache.untyped_data(), kv_cache.size_bytes(),
                                          cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return ffi::Error(ffi::ErrorCode::kInternal, cudaGetErrorString(e));
  }
  const int rc = tjx_ragged_paged_attention_bf16(
      q.untyped_data(), keys.untyped_data(), values.untyped_data(), cache_out->untyped_data(),
      static_cast<const int32_t*>(kv_lens.untyped_data()), static_cast<const int32_t*>(page_indices.untyped_data()),
      static_cast<const int32_t*>(cu_q_lens.untyped_data()), static_cast<const int32_t*>(distribution.untyped_data()),
      out->untyped_data(), T, S, H, Hkv, D, page_size, pages_per_seq, num_pages, sm_scale, ws, need, stream);
  return rc == 0 ? ffi::Error::Success() : Failed(rc);
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(TjxBuildSteps, BuildStepsImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // lengths
                                  .Ret<ffi::AnyBuffer>()   // step_tile
                                  .Ret<ffi::AnyBuffer>()   // step_code
                                  .Ret<ffi::AnyBuffer>()   // step_count
                                  .Ret<ffi::AnyBuffer>()   // tile_first
                                  .Attr<int32_t>("tiles")
                                  .Attr<int32_t>("blocks")
                                  .Attr<int32_t>("value0")
                                  .Attr<int32_t>("value_step"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(TjxGemm, GemmImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // x
                                  .Arg<ffi::AnyBuffer>()   // y
                                  .Arg<ffi::AnyBuffer>()   // tile_i (int32, may be empty)
                                  .Arg<ffi::AnyBuffer>()   // tile_j
                                  .Arg<ffi::AnyBuffer>()   // fill_i
                                  .Arg<ffi::AnyBuffer>()   // fill_j
                                  .Ret<ffi::AnyBuffer>()   // out
                                  .Attr<int32_t>("tm")
                                  .Attr<int32_t>("tn")
                                  .Attr<int32_t>("tk")
                                  .Attr<int32_t>("stages")
                                  .Attr<int32_t>("causal")
                                  .Attr<int32_t>("y_transposed"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(TjxCausalAttention, CausalAttentionImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // q
                                  .Arg<ffi::AnyBuffer>()   // k
                                  .Arg<ffi::AnyBuffer>()   // v
                                  .Arg<ffi::AnyBuffer>()   // step_tile
                                  .Arg<ffi::AnyBuffer>()   // step_code
                                  .Ret<ffi::AnyBuffer>()   // out
                                  .Attr<int32_t>("block_q")
                                  .Attr<int32_t>("block_kv")
                                  .Attr<int32_t>("pattern_tiles"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(TjxPagedGqaDecode, PagedGqaDecodeImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // q
                                  .Arg<ffi::AnyBuffer>()   // k_pages
                                  .Arg<ffi::AnyBuffer>()   // v_pages
                                  .Arg<ffi::AnyBuffer>()   // block_tables
                                  .Arg<ffi::AnyBuffer>()   // lengths
                                  .Ret<ffi::AnyBuffer>()   // out
                                  .Ret<ffi::AnyBuffer>()   // step_tile
                                  .Ret<ffi::AnyBuffer>()   // step_code
                                  .Ret<ffi::AnyBuffer>()   // step_count
                                  .Ret<ffi::AnyBuffer>()   // tile_first
                                  .Ret<ffi::AnyBuffer>());  // workspace (uint8)

XLA_FFI_DEFINE_HANDLER_SYMBOL(TjxRmsnormGemm, RmsnormGemmImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // x
                                  .Arg<ffi::AnyBuffer>()   // gamma
                                  .Arg<ffi::AnyBuffer>()   // w
                                  .Ret<ffi::AnyBuffer>()   // out
                                  .Ret<ffi::AnyBuffer>()   // workspace (uint8)
                                  .Attr<int32_t>("tm")
                                  .Attr<int32_t>("tn")
                                  .Attr<int32_t>("tk")
                                  .Attr<float>("eps"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(TjxAttentionBlock, AttentionBlockImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // q
                                  .Arg<ffi::AnyBuffer>()   // k
                                  .Arg<ffi::AnyBuffer>()   // v
                                  .Arg<ffi::AnyBuffer>()   // gamma
                                  .Arg<ffi::AnyBuffer>()   // w_up
                                  .Arg<ffi::AnyBuffer>()   // w_down
                                  .Arg<ffi::AnyBuffer>()   // step_tile
                                  .Arg<ffi::AnyBuffer>()   // step_code
                                  .Ret<ffi::AnyBuffer>()   // out
                                  .Ret<ffi::AnyBuffer>()   // workspace (uint8)
                                  .Attr<int32_t>("block_q")
                                  .Attr<int32_t>("block_kv")
                                  .Attr<int32_t>("pattern_tiles")
                                  .Attr<float>("eps"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(TjxMlaDecode, MlaDecodeImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // q_c
                                  .Arg<ffi::AnyBuffer>()   // q_r
                                  .Arg<ffi::AnyBuffer>()   // c_kv
                                  .Arg<ffi::AnyBuffer>()   // k_rope
                                  .Arg<ffi::AnyBuffer>()   // lengths
                                  .Ret<ffi::AnyBuffer>()   // out
                                  .Ret<ffi::AnyBuffer>()   // step_tile
                                  .Ret<ffi::AnyBuffer>()   // step_code
                                  .Ret<ffi::AnyBuffer>()   // step_count
                                  .Ret<ffi::AnyBuffer>()   // tile_first
                                  .Ret<ffi::AnyBuffer>()   // workspace (uint8)
                                  .Attr<int32_t>("block"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(TjxRaggedPagedAttention, RaggedPagedAttentionImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>()   // q
                                  .Arg<ffi::AnyBuffer>()   // keys
                                  .Arg<ffi::AnyBuffer>()   // values
                                  .Arg<ffi::AnyBuffer>()   // kv_cache (aliased to the cache result)
                                  .Arg<ffi::AnyBuffer>()   // kv_lens
                                  .Arg<ffi::AnyBuffer>()   // page_indices
                                  .Arg<ffi::AnyBuffer>()   // cu_q_lens
                                  .Arg<ffi::AnyBuffer>()   // distribution
                                  .Ret<ffi::AnyBuffer>()   // out
                                  .Ret<ffi::AnyBuffer>()   // kv_cache, updated
                                  .Ret<ffi::AnyBuffer>()   // workspace (uint8)
                                  .Attr<float>("sm_scale"));

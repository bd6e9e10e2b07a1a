// Host-side helpers shared by the C-ABI entry points: error reporting, device checks, TMA tensor maps.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace tjx {

// Error codes the C ABI returns (negative). Kernel-side codes (tjx_ptx.cuh) are positive.
enum : int {
  TJX_E_ARG = -1,      // bad argument (shape, alignment, null pointer)
  TJX_E_CUDA = -2,     // a CUDA runtime / driver call failed
  TJX_E_DEVICE = -3,   // not an sm_100 device
  TJX_E_LIMIT = -4,    // a size exceeds what the entry point supports
  TJX_E_KERNEL = -5,   // a kernel reported an error through its status word
};

void set_error(const std::string& msg);
int fail(int code, const std::string& msg);
int cuda_fail(cudaError_t e, const char* what);

// 0 if the current device is compute capability 10.x, else TJX_E_DEVICE (with the message set).
int check_device();
int sm_count();

// How the calling thread's next launches are chained to their neighbours on the stream (programmatic dependent
// launch): CHAIN_WAITS = launched so that it may start before the kernel in front of it has finished, and waits for
// that kernel's results itself (griddepcontrol.wait) before it reads or writes anything; CHAIN_RELEASES = lets the
// kernel behind it be scheduled as soon as its own CTAs have started. 0 = an ordinary launch. Set by an entry point
// that issues several dependent kernels (the attention block), around each of them.
enum : int { CHAIN_WAITS = 1, CHAIN_RELEASES = 2 };
int& launch_chain();
// Sets the calling thread's chain for the launches made while it lives.
struct LaunchChain {
  explicit LaunchChain(int how) { launch_chain() = how; }
  ~LaunchChain() { launch_chain() = 0; }
  LaunchChain(const LaunchChain&) = delete;
  LaunchChain& operator=(const LaunchChain&) = delete;
};

// A launch with programmatic stream serialization allowed: the kernel may be scheduled once the kernel in front of it
// on the stream has released (chain_release) or ended, and orders itself behind that kernel with chain_wait.
template <typename... Params, typename... Args>
cudaError_t launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                           Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr, cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<Params>(args)...);
}

// The prefill half of a ragged paged attention step, for the entry point that runs the whole step
// (tjx_ragged_paged_attention_bf16; defined beside the attention kernel). The tile arrays live in `workspace`
// (rpa_prefill_part_bytes, 256-byte aligned).
struct RpaTiles {
  const int32_t *row0, *rows, *count;  // tile k covers rows row0[k] .. row0[k] + rows[k] - 1 of q; count[0] tiles
  int max_tiles;
};
size_t rpa_prefill_part_bytes(int T, int S);
int rpa_prefill_part_check(const void* q, const void* out, const void* kv_cache, const void* page_indices, int T, int S,
                           int H, int Hkv, int D, int page_size, int pages_per_seq, int num_pages);
// Enqueues the kernel that lists the step's prefill tiles, chained behind the kernel in front of it.
int rpa_prefill_tiles_part(const int32_t* kv_lens, const int32_t* cu_q_lens, const int32_t* distribution, int T, int S,
                           int pages_per_seq, void* workspace, cudaStream_t stream, RpaTiles* tiles);
// Enqueues the paged attention over those tiles: queries from q, outputs to the tiles' rows of out; chained behind
// the kernel in front of it as launch_chain() says.
int rpa_prefill_attention_part(const void* q, void* out, const void* kv_cache, const int32_t* page_indices, int T, int S,
                               int H, int Hkv, int pages_per_seq, int num_pages, float sm_scale, void* workspace,
                               cudaStream_t stream);

// Per-device status word the kernels write error codes to: a fixed device variable inside the library (no
// allocation); the address is looked up once per device.
int* device_status_word();

// The calling thread's profile buffer (tjx_set_profile_buffer) if it has room for `ctas` records, else null.
long long* profile_buffer(int ctas);

// Encode a tiled tensor map over a row-major bf16/f32 matrix viewed as `rank` dims (innermost first).
// dims/box in elements, strides in bytes for dims 1..rank-1. Returns 0 or an error code.
int make_tensor_map(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, int rank,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    CUtensorMapSwizzle swizzle);

}  // namespace tjx

#define TJX_CUDA(call)                                         \
  do {                                                         \
    cudaError_t e__ = (call);                                  \
    if (e__ != cudaSuccess) return tjx::cuda_fail(e__, #call); \
  } while (0)

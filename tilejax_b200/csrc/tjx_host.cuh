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

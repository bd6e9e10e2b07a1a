// Host-side runtime shared by the entry points: thread-local error text, device checks, the per-device
// kernel status word, and TMA tensor-map encoding through the driver entry point (no link against libcuda,
// so the library also loads on a machine without a driver).
#include "tjx_host.cuh"

#include <mutex>

#include "../../include/tilejax_b200.h"

namespace tjx {

static thread_local std::string g_error;

void set_error(const std::string& msg) { g_error = msg; }

int fail(int code, const std::string& msg) {
  g_error = msg;
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  g_error = std::string(what) + ": " + cudaGetErrorString(e);
  return TJX_E_CUDA;
}

constexpr int MAX_DEVICES = 64;
static std::mutex g_mutex;
static int g_cc_major[MAX_DEVICES];  // 0 = unknown
static int g_sm_count[MAX_DEVICES];
static int* g_status[MAX_DEVICES];

// The kernels' error word: a fixed device variable (one per GPU that loads the library), so that no entry
// point ever has to allocate device memory. Host code only ever takes its address with cudaGetSymbolAddress.
// Word 0 is the status; word 1 is the longest a device-side wait may last, in microseconds (0 = the built-in 2 s).
static __device__ int g_status_word[64] = {0, 2000000};

static int current_device(int* dev) {
  cudaError_t e = cudaGetDevice(dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (*dev < 0 || *dev >= MAX_DEVICES) return fail(TJX_E_ARG, "device ordinal out of range");
  return 0;
}

int check_device() {
  int dev;
  if (int rc = current_device(&dev)) return rc;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_cc_major[dev] == 0) {
    int major = 0, sms = 0;
    cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
    g_cc_major[dev] = major;
    g_sm_count[dev] = sms;
  }
  if (g_cc_major[dev] != 10)
    return fail(TJX_E_DEVICE, "tilejax_b200 kernels are built for sm_100a only; this device is compute capability " +
                                  std::to_string(g_cc_major[dev]) + ".x (there is no fallback path)");
  return 0;
}

int& launch_chain() {
  static thread_local int chain = 0;
  return chain;
}

int sm_count() {
  int dev;
  if (current_device(&dev)) return 0;
  return g_sm_count[dev];
}

int* device_status_word() {
  int dev;
  if (current_device(&dev)) return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_status[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess || p == nullptr) return nullptr;
    g_status[dev] = static_cast<int*>(p);  // zero-initialised when the module loads
  }
  return g_status[dev];
}

static thread_local long long* g_profile = nullptr;
static thread_local size_t g_profile_bytes = 0;

long long* profile_buffer(int ctas) {
  if (g_profile == nullptr || static_cast<size_t>(ctas) * 16 * sizeof(long long) > g_profile_bytes) return nullptr;
  return g_profile;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tensor_map(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes, int rank,
                    const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                    CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return fail(TJX_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return fail(TJX_E_ARG, "tensor base is not 16-byte aligned");
  cuuint64_t gdims[5], gstrides[5];
  cuuint32_t gbox[5], gelem[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    gelem[i] = 1;
    if (box[i] == 0 || box[i] > 256) return fail(TJX_E_ARG, "TMA box dimension must be in 1..256");
  }
  for (int i = 0; i + 1 < rank; ++i) {
    gstrides[i] = strides_bytes[i];
    if (strides_bytes[i] % 16 != 0) return fail(TJX_E_ARG, "row pitch is not a multiple of 16 bytes");
  }
  if ((static_cast<uint64_t>(box[0]) * elem_bytes) % 16 != 0)
    return fail(TJX_E_ARG, "TMA box inner extent is not a multiple of 16 bytes");
  CUresult r = fn(out, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims, gstrides, gbox, gelem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TJX_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(r));
  return 0;
}

}  // namespace tjx

extern "C" {

int tjx_version(void) { return 100; }

const char* tjx_last_error(void) { return tjx::g_error.c_str(); }

int tjx_set_profile_buffer(void* device_buffer, size_t bytes) {
  if (device_buffer != nullptr && (reinterpret_cast<uintptr_t>(device_buffer) & 7u) != 0)
    return tjx::fail(TJX_E_ARG, "the profile buffer must be 8-byte aligned");
  tjx::g_profile = static_cast<long long*>(device_buffer);
  tjx::g_profile_bytes = device_buffer == nullptr ? 0 : bytes;
  return 0;
}

int tjx_set_wait_limit_us(int microseconds) {
  if (microseconds < 1000 || microseconds > 10000000)
    return tjx::fail(TJX_E_ARG, "the wait limit is between 1000 microseconds and 10 seconds");
  if (int rc = tjx::check_device()) return rc;
  int* word = tjx::device_status_word();
  if (word == nullptr) return tjx::fail(TJX_E_CUDA, "could not locate the device status word");
  TJX_CUDA(cudaDeviceSynchronize());  // no kernel is in the middle of a wait while the limit changes
  TJX_CUDA(cudaMemcpy(word + 1, &microseconds, sizeof(int), cudaMemcpyHostToDevice));
  return 0;
}

int tjx_device_status(tjx_stream_t stream, int* code) {
  if (code == nullptr) return tjx::fail(TJX_E_ARG, "code is null");
  *code = 0;
  if (int rc = tjx::check_device()) return rc;
  int* word = tjx::device_status_word();
  if (word == nullptr) return tjx::fail(TJX_E_CUDA, "could not locate the device status word");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TJX_CUDA(cudaStreamSynchronize(s));
  TJX_CUDA(cudaMemcpy(code, word, sizeof(int), cudaMemcpyDeviceToHost));
  if (*code != 0) {
    TJX_CUDA(cudaMemset(word, 0, sizeof(int)));
    return tjx::fail(TJX_E_KERNEL, "a kernel gave up on a bounded wait, code " + std::to_string(*code));
  }
  return 0;
}

}  // extern "C"

// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (MMA, TMEM
// allocation, TMEM loads/stores), proxy fences. Every wait is bounded: a wait that runs out records an
// error code and makes the whole CTA leave its loops, so a broken pipeline never hangs the GPU.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tjx {

// Error codes a kernel writes to its status word (0 = ok).
enum : int {
  TJX_OK = 0,
  TJX_ERR_WAIT_FULL = 101,    // consumer waited too long for a ring slot to fill
  TJX_ERR_WAIT_EMPTY = 102,   // producer waited too long for a ring slot to drain
  TJX_ERR_WAIT_TMEM_FULL = 103,
  TJX_ERR_WAIT_TMEM_EMPTY = 104,
  TJX_ERR_WAIT_OTHER = 105,
  TJX_ERR_BAD_TABLE = 110,    // a step/tile table entry out of range
};

// Longest a single wait may last before the kernel gives up (nanoseconds of %globaltimer) when the kernel has no
// status word to read the limit from. With a status word the limit is the word after it, in microseconds
// (tjx_set_wait_limit_us; 2 s unless changed).
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ unsigned long long wait_limit_ns(const int* status) {
  if (status == nullptr) return WAIT_LIMIT_NS;
  const unsigned us = static_cast<unsigned>(*reinterpret_cast<const volatile int*>(status + 1));
  return us == 0 ? WAIT_LIMIT_NS : static_cast<unsigned long long>(us) * 1000ull;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t lane_id() {
  uint32_t l;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(l));
  return l;
}

// ---------------------------------------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  // Makes barrier initialisation visible to the async proxy (TMA, tcgen05.commit).
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait on a barrier phase. `abort_flag` (shared memory) is raised by whichever thread of the CTA
// gives up first; every other waiter then leaves at its next poll. Returns false if the wait was abandoned.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int code) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long start = 0, limit = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0) {
      if (*abort_flag) return false;
      unsigned long long now = globaltimer_ns();
      if (start == 0) start = now, limit = wait_limit_ns(status);
      if (now - start > limit) {
        *abort_flag = 1;
        if (status != nullptr) atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

// The same wait with the cycles it lasted added to `waited` when `timed` (a launch with a profile buffer): what the
// in-kernel profile counts as time blocked on inputs, on the epilogue, on the softmax. The clock is read around the
// whole wait — mbarrier.try_wait may itself suspend the thread for a while before it answers.
__device__ __forceinline__ bool mbar_wait_timed(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                int code, long long& waited, bool timed) {
  if (!timed) return mbar_wait(bar, parity, abort_flag, status, code);
  const long long t0 = clock64();
  const bool ok = mbar_wait(bar, parity, abort_flag, status, code);
  waited += clock64() - t0;
  return ok;
}

// One CTA's record in the profile buffer (tjx_set_profile_buffer): sixteen 64-bit words.
//   [0] clock at CTA start   [1] clock when the issuing thread starts its first work item   [2] clock after its last
//   [3] cycles it waited for inputs (ring slots to fill)   [4] of which the first wait: the pipeline filling
//   [5] cycles it waited for room for its results (accumulator or output slot still being drained)
//   [6] work items it ran   [7] clock at CTA end
//   [8..15] kernel-specific. Attention: [8] cycles the MMA warp waited for the softmax warps' probabilities;
//           [9] cycles to issue the first Q K^T (idle pipe), [10] cycles in all Q K^T issues, [11] their count;
//           slot A's first softmax warp: [12] cycles busy, [13] cycles waiting for scores, [14] blocks,
//           [15] three 21-bit fields, high to low: cycles in the TMEM load, in the row max (and rescale), in the
//           exponentials. MLA decode (tcgen05 kernel): [8] as attention's, [9] cycles issuing score MMAs, [10] cycles
//           issuing output MMAs, [11] pieces, [12] and [13] %globaltimer (ns) at CTA start and end; work items are units of
//           32 positions.
//           All-gather matmul: [10] cycles this CTA's producer waited for gathered rows to arrive, [11] clock when
//           its copier warp had posted its last block
constexpr int PROFILE_WORDS = 16;

// ---------------------------------------------------------------------------------------------- fences

__device__ __forceinline__ void fence_proxy_async_smem() {
  // Orders generic-proxy writes to shared memory before async-proxy reads of it (TMA stores, tcgen05.mma).
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------- TMA

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// 2-D tile load global -> shared; completes `bytes of the box` on the mbarrier. x is the innermost
// coordinate (x * element size must be a multiple of 16 bytes).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, int x, int y, int z,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], "
      "[%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// 2-D tile store shared -> global (bulk async group).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(m)), "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  // At most N of this thread's bulk groups may still be reading their shared-memory source.
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------------------------- launch chains

// Programmatic dependent launch: wait until the kernels this one was chained behind have completed and their
// writes are visible (nothing happens in a kernel launched the ordinary way); let the kernel chained behind this
// one be scheduled.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- TMEM

// Allocate `cols` (power of two, 32..512) TMEM columns; the base address lands in shared memory at `dst`.
// One whole warp executes this.
__device__ __forceinline__ void tmem_alloc(uint32_t dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst), "r"(cols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// ---------------------------------------------------------------------------------------------- tcgen05.mma

// Shared-memory matrix descriptor (128-byte swizzle). Offsets in bytes, multiples of 16.
//   K-major operand  (rows of 128 B = 64 bf16 along K): sbo = bytes between 8-row groups (1024), lbo unused.
//   MN-major operand (rows of 128 B = 64 bf16 along M/N, one row per k): sbo = bytes between groups of 8 k
//   (1024), lbo = bytes between successive 64-element blocks along M/N.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version for sm_100
  d |= 2ull << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16 with bf16 operands and f32 accumulation.
__host__ __device__ constexpr uint32_t idesc_bf16_f32(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4)                                    // D format: f32
         | (1u << 7)                                  // A format: bf16
         | (1u << 10)                                 // B format: bf16
         | (static_cast<uint32_t>(a_mn_major) << 15)  // A major: 0 = K, 1 = MN
         | (static_cast<uint32_t>(b_mn_major) << 16)  // B major
         | (static_cast<uint32_t>(n >> 3) << 17)      // N / 8
         | (static_cast<uint32_t>(m >> 4) << 24);     // M / 16
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues it.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem]; A is bf16 packed two per 32-bit TMEM column.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same with the accumulate flag known at compile time (no predicate set-up in the issuing thread's path).
template <bool ACCUMULATE>
__device__ __forceinline__ void mma_ss_c(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
  if constexpr (ACCUMULATE) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc)
        : "memory");
  }
}

template <bool ACCUMULATE>
__device__ __forceinline__ void mma_ts_c(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc) {
  if constexpr (ACCUMULATE) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc)
        : "memory");
  }
}

// True in exactly one lane of a converged warp, the same lane every time. A role that issues tcgen05.mma runs its
// loop with the whole warp, so that the compiler keeps descriptors and addresses in uniform registers, and puts
// only the instruction itself under this predicate; a loop run by one lane of a diverged warp computes them in
// per-thread registers and pays a transfer to the uniform file for every operand of every MMA.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\telect.sync _|P, 0xFFFFFFFF;\n\tselp.u32 %0, 1, 0, P;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// Eight MMAs of one accumulation (K = 128 in steps of 16) and the commit that follows them, issued by the warp's
// elected lane without a branch in between: D[tmem] (+)= A_k * B_k for k = 0..7, `accumulate_first` deciding whether
// the first one adds to what D holds; then one arrival on `bar` when they have completed. Called by a whole warp.
__device__ __forceinline__ void mma_ss_x8_commit(uint32_t d_tmem, const uint64_t (&a)[8], const uint64_t (&b)[8],
                                                 uint32_t idesc, uint32_t accumulate_first, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred L, F, T;\n\t"
      "elect.sync _|L, 0xFFFFFFFF;\n\t"
      "setp.ne.b32 F, %2, 0;\n\t"
      "setp.eq.b32 T, 0, 0;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %4, %12, %1, F;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %5, %13, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %6, %14, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %7, %15, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %8, %16, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %9, %17, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %10, %18, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %11, %19, %1, T;\n\t"
      "@L tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%3];\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(idesc), "r"(accumulate_first), "r"(bar), "l"(a[0]), "l"(a[1]), "l"(a[2]), "l"(a[3]), "l"(a[4]),
        "l"(a[5]), "l"(a[6]), "l"(a[7]), "l"(b[0]), "l"(b[1]), "l"(b[2]), "l"(b[3]), "l"(b[4]), "l"(b[5]), "l"(b[6]),
        "l"(b[7])
      : "memory");
}

// Eight MMAs of one accumulation with both operands in shared memory, without a commit (a longer accumulation
// issues several of these and commits once).
__device__ __forceinline__ void mma_ss_x8(uint32_t d_tmem, const uint64_t (&a)[8], const uint64_t (&b)[8], uint32_t idesc,
                                          uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred L, F, T;\n\t"
      "elect.sync _|L, 0xFFFFFFFF;\n\t"
      "setp.ne.b32 F, %2, 0;\n\t"
      "setp.eq.b32 T, 0, 0;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %11, %1, F;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %4, %12, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %5, %13, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %6, %14, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %7, %15, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %8, %16, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %9, %17, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %10, %18, %1, T;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(idesc), "r"(accumulate_first), "l"(a[0]), "l"(a[1]), "l"(a[2]), "l"(a[3]), "l"(a[4]), "l"(a[5]),
        "l"(a[6]), "l"(a[7]), "l"(b[0]), "l"(b[1]), "l"(b[2]), "l"(b[3]), "l"(b[4]), "l"(b[5]), "l"(b[6]), "l"(b[7])
      : "memory");
}

// The same with A in TMEM (bf16, two per 32-bit column): a[k] is the TMEM address of the k-th 16-wide slice.
__device__ __forceinline__ void mma_ts_x8_commit(uint32_t d_tmem, const uint32_t (&a)[8], const uint64_t (&b)[8],
                                                 uint32_t idesc, uint32_t accumulate_first, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred L, F, T;\n\t"
      "elect.sync _|L, 0xFFFFFFFF;\n\t"
      "setp.ne.b32 F, %2, 0;\n\t"
      "setp.eq.b32 T, 0, 0;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%4], %12, %1, F;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%5], %13, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%6], %14, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%7], %15, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%8], %16, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%9], %17, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%10], %18, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%11], %19, %1, T;\n\t"
      "@L tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%3];\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(idesc), "r"(accumulate_first), "r"(bar), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]),
        "r"(a[5]), "r"(a[6]), "r"(a[7]), "l"(b[0]), "l"(b[1]), "l"(b[2]), "l"(b[3]), "l"(b[4]), "l"(b[5]), "l"(b[6]),
        "l"(b[7])
      : "memory");
}

// Half of such an accumulation with A in TMEM (four MMAs), without and with the commit: the two halves of a P V
// product whose P arrives in two parts.
__device__ __forceinline__ void mma_ts_x4(uint32_t d_tmem, const uint32_t* a, const uint64_t* b, uint32_t idesc,
                                          uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred L, F, T;\n\t"
      "elect.sync _|L, 0xFFFFFFFF;\n\t"
      "setp.ne.b32 F, %2, 0;\n\t"
      "setp.eq.b32 T, 0, 0;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%3], %7, %1, F;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%4], %8, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%5], %9, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%6], %10, %1, T;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(idesc), "r"(accumulate_first), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "l"(b[0]), "l"(b[1]),
        "l"(b[2]), "l"(b[3])
      : "memory");
}
__device__ __forceinline__ void mma_ts_x4_commit(uint32_t d_tmem, const uint32_t* a, const uint64_t* b, uint32_t idesc,
                                                 uint32_t accumulate_first, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred L, F, T;\n\t"
      "elect.sync _|L, 0xFFFFFFFF;\n\t"
      "setp.ne.b32 F, %2, 0;\n\t"
      "setp.eq.b32 T, 0, 0;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%4], %8, %1, F;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%5], %9, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%6], %10, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], [%7], %11, %1, T;\n\t"
      "@L tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%3];\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(idesc), "r"(accumulate_first), "r"(bar), "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "l"(b[0]),
        "l"(b[1]), "l"(b[2]), "l"(b[3])
      : "memory");
}

// The warp's index, known to the compiler as the same in every lane.
__device__ __forceinline__ int uniform_warp_index() {
  return __shfl_sync(0xFFFFFFFFu, static_cast<int>(threadIdx.x >> 5), 0);
}

// The barrier gets one arrival once every tcgen05.mma this thread issued before has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// ---------------------------------------------------------------------------------------------- CTA pairs
//
// The two-SM forms (cta_group::2): a cluster of two CTAs shares one MMA. Each CTA stages its own 128 rows of A
// and its own half of B's columns at the same shared-memory offsets; the even CTA of the pair issues the MMA,
// which reads both CTAs' shared memory and writes 128 accumulator rows into each CTA's TMEM.

__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// The shared::cluster address of this CTA's shared-memory location `addr` as it appears in CTA `rank`.
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
  return out;
}

// Every thread of every CTA of the cluster calls this (a full barrier with release/acquire ordering).
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// One arrival on a barrier anywhere in the cluster (address from cluster_map).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// 2-D tile load into THIS CTA's shared memory whose bytes are counted on a barrier that may live in the peer
// CTA of the pair (address from cluster_map). Each CTA fetches only what it stages itself.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, int x, int y,
                                                 uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}

// One warp of EACH CTA of the pair executes these, with the same `dst` offset.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst), "r"(cols)
               : "memory");
}

__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// D[tmem of both CTAs] (+)= A * B over the pair (M = 256: 128 rows per CTA); one thread of the even CTA issues.
__device__ __forceinline__ void mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// One arrival on `cluster_bar` (any CTA of the pair) once every pair MMA this thread issued before has completed.
__device__ __forceinline__ void mma_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
               : "memory");
}

// Four MMAs with both operands in shared memory (one 64-deep ring slot) and the commit that frees the slot.
__device__ __forceinline__ void mma_ss_x4_commit(uint32_t d_tmem, const uint64_t* a, const uint64_t* b, uint32_t idesc,
                                                 uint32_t accumulate_first, uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred L, F, T;\n\t"
      "elect.sync _|L, 0xFFFFFFFF;\n\t"
      "setp.ne.b32 F, %2, 0;\n\t"
      "setp.eq.b32 T, 0, 0;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %4, %8, %1, F;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %5, %9, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %6, %10, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::1.kind::f16 [%0], %7, %11, %1, T;\n\t"
      "@L tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%3];\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(idesc), "r"(accumulate_first), "r"(bar), "l"(a[0]), "l"(a[1]), "l"(a[2]), "l"(a[3]), "l"(b[0]),
        "l"(b[1]), "l"(b[2]), "l"(b[3])
      : "memory");
}

// The pair forms: four pair MMAs; one arrival on a barrier of each CTA of the pair.
__device__ __forceinline__ void mma_ss_pair_x4(uint32_t d_tmem, const uint64_t* a, const uint64_t* b, uint32_t idesc,
                                               uint32_t accumulate_first) {
  asm volatile(
      "{\n\t.reg .pred L, F, T;\n\t"
      "elect.sync _|L, 0xFFFFFFFF;\n\t"
      "setp.ne.b32 F, %2, 0;\n\t"
      "setp.eq.b32 T, 0, 0;\n\t"
      "@L tcgen05.mma.cta_group::2.kind::f16 [%0], %3, %7, %1, F;\n\t"
      "@L tcgen05.mma.cta_group::2.kind::f16 [%0], %4, %8, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::2.kind::f16 [%0], %5, %9, %1, T;\n\t"
      "@L tcgen05.mma.cta_group::2.kind::f16 [%0], %6, %10, %1, T;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(idesc), "r"(accumulate_first), "l"(a[0]), "l"(a[1]), "l"(a[2]), "l"(a[3]), "l"(b[0]), "l"(b[1]),
        "l"(b[2]), "l"(b[3])
      : "memory");
}
__device__ __forceinline__ void mma_commit_pair_both(uint32_t cluster_bar0, uint32_t cluster_bar1) {
  asm volatile(
      "{\n\t.reg .pred L;\n\t"
      "elect.sync _|L, 0xFFFFFFFF;\n\t"
      "@L tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "@L tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%1];\n\t"
      "}\n" ::"r"(cluster_bar0),
      "r"(cluster_bar1)
      : "memory");
}
__device__ __forceinline__ void mma_commit_elected(uint32_t bar) {
  asm volatile(
      "{\n\t.reg .pred L;\n\t"
      "elect.sync _|L, 0xFFFFFFFF;\n\t"
      "@L tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}\n" ::"r"(bar)
      : "memory");
}

// ---------------------------------------------------------------------------------------------- TMEM <-> regs

// 32 lanes x 32 columns of 32-bit: thread i of the warp gets lane (base lane + i), columns c..c+31.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
        "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------- warp-level MMA

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Four 8x8 b16 matrices from shared memory: lane i gives the address of row i % 8 of matrix i / 8; register j
// of every lane then holds, of matrix j, row lane / 4, columns 2 (lane % 4) and + 1 — or with .trans, column
// lane / 4, rows 2 (lane % 4) and + 1.
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// D (16 x 8, f32) += A (16 x 16, bf16, rows) * B (16 x 8, bf16, columns). The rows are the query rows of one KV
// head: (new token, query head) pairs, at most 16; a1 and a3 (rows 8..15) are zero when there are at most 8.
__device__ __forceinline__ void mma_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                            uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------------------------------------- misc

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);  // .x = lo (low 16 bits), .y = hi
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }

}  // namespace tjx

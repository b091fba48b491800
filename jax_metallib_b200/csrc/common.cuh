// Shared host/device helpers for the quantized-matmul kernel library (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "../../include/qmm.h"

// ---------------------------------------------------------------------------
// Host side: error reporting (errors are values, never exceptions or aborts)
// ---------------------------------------------------------------------------
namespace qmm {

int set_error(int status, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

#define QMM_CUDA_TRY(expr)                                                              \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess)                                                              \
      return ::qmm::set_error(QMM_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,             \
                              cudaGetErrorString(_e), __FILE__, __LINE__);              \
  } while (0)

#define QMM_REQUIRE(cond, status, ...)                               \
  do {                                                               \
    if (!(cond)) return ::qmm::set_error((status), __VA_ARGS__);     \
  } while (0)

// After a launch: surface launch-configuration errors without synchronising.
#define QMM_CHECK_LAUNCH(name)                                                           \
  do {                                                                                  \
    cudaError_t _e = cudaGetLastError();                                                \
    if (_e != cudaSuccess)                                                              \
      return ::qmm::set_error(QMM_ERR_CUDA, "launch of %s failed: %s", (name),          \
                              cudaGetErrorString(_e));                                  \
  } while (0)

// Launch with programmatic stream serialization: the kernel may start while the
// kernel before it on the stream is still running, and orders itself behind it
// with griddepcontrol.wait (dev::pdl_wait) before it touches anything that
// kernel, or one further back that may still be running, could write.
// Every kernel launched this way calls dev::pdl_wait.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}


// A host-mapped status word that device-side bounded waits write to when they
// give up (code in the low 16 bits, a site tag above).  Allocated once per
// process; readable by the host without synchronising.
int* device_status_word();   // device-visible pointer (may be null on failure)
int* device_status_word_if_ready();  // same, but never creates it (null until someone has)
int read_device_status();    // current value (0 = healthy)
int read_device_status_if_ready();  // same, but never creates the word (0 until someone has)
void clear_device_status();
int num_sms();               // of the current device (cached)

// Per-device "done once" bookkeeping.  Function attributes such as the dynamic
// shared-memory opt-in belong to a device's context, so a process that drives
// several GPUs has to set them once on each; `done` is a bit mask of device
// ordinals kept by the call site.  mark_device_once returns true for exactly
// one caller per (mask, ordinal) and is safe to call from any thread.
constexpr int kMaxDevices = 64;
inline bool device_marked(const std::atomic<uint64_t>& done, int ordinal) {
  return ordinal >= 0 && ordinal < kMaxDevices && ((done.load(std::memory_order_acquire) >> ordinal) & 1ull);
}
inline bool mark_device_once(std::atomic<uint64_t>& done, int ordinal) {
  if (ordinal < 0 || ordinal >= kMaxDevices) return true;  // untracked ordinals repeat the (idempotent) set-up
  const uint64_t bit = 1ull << ordinal;
  return (done.fetch_or(bit, std::memory_order_acq_rel) & bit) == 0;
}
// Opt a kernel in to `bytes` of dynamic shared memory on the current device,
// once per device.  `func` is the kernel's host symbol.
int ensure_dynamic_smem(const void* func, int bytes, std::atomic<uint64_t>& done);
// Environment switches are read once, when first asked for.
int env_int_once(const char* name, int dflt, std::atomic<int>& cache);
int gemm_ctas();             // CTAs a persistent GEMM may launch: num_sms() unless qmm_set_cta_limit lowered it

// 2-D tiled tensor map (TMA descriptor).  rows x cols elements of elem_bytes,
// row pitch in bytes, box = box_rows x box_cols, swizzle = CU_TENSOR_MAP_SWIZZLE_*.
int make_tensor_map_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt,
                       uint32_t elem_bytes, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                       uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swizzle);

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

}  // namespace qmm

// ---------------------------------------------------------------------------
// Device side
// ---------------------------------------------------------------------------
#ifdef __CUDACC__
namespace qmm {
namespace dev {

constexpr uint64_t kWaitLimitNs = 2000000000ull;  // bounded waits give up after ~2 s

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) {
  return __uint_as_float(static_cast<uint32_t>(b) << 16);
}
// round-to-nearest-even, NaN -> quiet NaN with the sign kept
__device__ __forceinline__ uint16_t float_to_bf16_bits(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
// Programmatic dependent launch: wait for the kernels before this one on the
// stream (complete and visible); allow the kernel after this one to start early.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier -------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// The same with a suspend-time hint: the thread may sleep in hardware for up to `ns` nanoseconds
// waiting for the phase instead of returning at once, so a waiting warp issues a few instructions
// per millisecond instead of a few per 30 cycles (polling warps otherwise take issue slots from
// the warps that share their scheduler).
__device__ __forceinline__ bool mbar_try_wait_sleep(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and records `tag` in the status word) when the
// phase did not complete within kWaitLimitNs; callers then stop issuing work
// and fall through to their teardown (free TMEM, return).  This form polls: the
// wake-up is immediate, at the price of issue slots; it is for waits on the
// critical path of a tensor-core pipeline.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int tag) {
  for (int i = 0; i < 128; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  const uint64_t t0 = globaltimer_ns();
  while (true) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (globaltimer_ns() - t0 > kWaitLimitNs) break;
  }
  if (status) atomicExch(status, (tag << 16) | QMM_ERR_TIMEOUT);
  return false;
}
// The same bound, sleeping in hardware between tries: for warps that wait long
// (an epilogue warp during a main loop) or whose wake-up latency does not matter
// (the bandwidth-bound decode kernels, where polling neighbours cost more).
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, int* status, int tag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    if (mbar_try_wait_sleep(bar, parity, 1000000u)) return true;  // sleeps up to 1 ms per try
    if (globaltimer_ns() - t0 > kWaitLimitNs) break;
  }
  if (status) atomicExch(status, (tag << 16) | QMM_ERR_TIMEOUT);
  return false;
}

// Warp-wide forms for waits that all 32 lanes make together: each lane waits
// (so each observes the phase itself), then the lanes agree on one outcome.
// Without the vote, right at the time limit one lane could see the phase
// complete while its neighbour gives up, and the lanes that went on would
// synchronise with lanes that have left.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, int* status, int tag) {
  return __all_sync(0xFFFFFFFFu, mbar_wait(bar, parity, status, tag));
}
__device__ __forceinline__ bool mbar_wait_relaxed_warp(uint64_t* bar, uint32_t parity, int* status, int tag) {
  return __all_sync(0xFFFFFFFFu, mbar_wait_relaxed(bar, parity, status, tag));
}

// ---- TMA --------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tile load, global -> this CTA's shared memory, completion on an mbarrier.
// c0 = innermost (column) coordinate in elements, c1 = row coordinate.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int32_t c0, int32_t c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
// Same with an L2 eviction-priority hint (createpolicy value).
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const CUtensorMap* m,
                                                 uint64_t* bar, int32_t c0, int32_t c1,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// 2-D tile store, this CTA's shared memory -> global, tracked by the issuing thread's bulk group.  Parts of the
// box outside the tensor are not written.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int32_t c0, int32_t c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
               : "memory");
}
// The same with an L2 eviction-priority hint (createpolicy value): results that nothing reads back soon should
// not push the operands of the next launch out of L2.
__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap* m, const void* smem_src, int32_t c0, int32_t c1,
                                                  uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "l"(policy)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until the issuing thread's bulk stores have read their shared-memory source (it may be overwritten).
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Make generic-proxy shared-memory writes visible to the async proxy (TMA / tcgen05).
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- system-scope ordering and multimem (NVSwitch multicast) ------------------
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
// One store to a multicast address lands at the same offset of every GPU bound to the
// multicast object (the switch replicates it), this GPU included.
__device__ __forceinline__ void multimem_st_b32(void* mc_addr, uint32_t v) {
  asm volatile("multimem.st.weak.global.b32 [%0], %1;" ::"l"(mc_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_st_v4_b32(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}
__device__ __forceinline__ void multimem_red_release_add_u32(uint32_t* mc_addr, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add_u32(uint32_t* addr, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u32(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// ---- tcgen05 / TMEM ---------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same MMAs with each descriptor given as its two 32-bit halves.  The start
// address (in 16-byte units) is the low 14 bits of the low half, so a descriptor
// is advanced with one 32-bit add.  The thread that issues the MMAs is the
// serial resource of a tcgen05 kernel: a tcgen05.mma costs it about 110 cycles
// and whatever it executes between two MMAs is added to that, so descriptors are
// never rebuilt inside the issue loop.
__device__ __forceinline__ void umma_f16_lh(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                            uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The same, issued only when `enable` is non-zero (a predicated instruction, no branch).
__device__ __forceinline__ void umma_f16_lh_if(uint32_t enable, uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                               uint32_t b_lo, uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tsetp.ne.b32 q, %7, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(enable)
      : "memory");
}
__device__ __forceinline__ void umma_i8_lh(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                           uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_i8_lh_if(uint32_t enable, uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi,
                                              uint32_t b_lo, uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tsetp.ne.b32 q, %7, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "@q tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n\t}" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate), "r"(enable)
      : "memory");
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading and
// stride byte offsets in 16-byte units, descriptor version 1, swizzle mode in
// bits 61..63 (0 none, 2 = 128B, 4 = 64B, 6 = 32B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, uint32_t layout_type) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version for sm_100
  d |= static_cast<uint64_t>(layout_type & 7) << 61;
  return d;
}

// Instruction descriptor for kind::f16 / kind::i8 (dense, no negate, no saturate).
//  c_format: 0 f16, 1 f32, 2 s32;  a/b_format: f16 kinds 0 f16, 1 bf16; i8 kinds 0 u8, 1 s8
//  a/b_major: 0 = K-major, 1 = MN-major
__host__ __device__ constexpr uint32_t make_idesc(uint32_t c_format, uint32_t a_format,
                                                  uint32_t b_format, uint32_t a_major,
                                                  uint32_t b_major, uint32_t M, uint32_t N) {
  return (c_format << 4) | (a_format << 7) | (b_format << 10) | (a_major << 15) |
         (b_major << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// 32 lanes x 32 consecutive 32-bit columns of TMEM into registers.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

}  // namespace dev
}  // namespace qmm
#endif  // __CUDACC__

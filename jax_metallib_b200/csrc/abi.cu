// Host-side plumbing shared by every entry point: error strings, the device
// status word, SM count cache and the TMA descriptor encoder.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include <atomic>

#include "common.cuh"

namespace qmm {

static thread_local char g_err[512] = {0};

int set_error(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return status;
}

static std::once_flag g_status_once;
static int* g_status_host = nullptr;
static int* g_status_dev = nullptr;

static void init_status_word() {
  void* h = nullptr;
  if (cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
    cudaGetLastError();
    return;
  }
  memset(h, 0, 64);
  void* d = nullptr;
  if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) {
    cudaGetLastError();
    cudaFreeHost(h);
    return;
  }
  g_status_host = static_cast<int*>(h);
  g_status_dev = static_cast<int*>(d);
}

int* device_status_word() {
  std::call_once(g_status_once, init_status_word);
  return g_status_dev;
}
// The status word if it has been created already, else null.  Never allocates.
int* device_status_word_if_ready() { return g_status_dev; }
// Current value if the word exists already, else 0.  Never allocates.
int read_device_status_if_ready() {
  return g_status_host ? *reinterpret_cast<volatile int*>(g_status_host) : 0;
}
int read_device_status() {
  std::call_once(g_status_once, init_status_word);
  return g_status_host ? *reinterpret_cast<volatile int*>(g_status_host) : 0;
}
void clear_device_status() {
  std::call_once(g_status_once, init_status_word);
  if (g_status_host) *reinterpret_cast<volatile int*>(g_status_host) = 0;
}

static std::atomic<int> g_cta_limit{0};

int gemm_ctas() {
  const int sms = num_sms();
  const int lim = g_cta_limit.load(std::memory_order_relaxed);
  return (lim > 0 && lim < sms) ? lim : sms;
}

int num_sms() {
  static thread_local int cached_dev = -1;
  static thread_local int cached = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev != cached_dev) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
      v = 148;
    cached = v;
    cached_dev = dev;
  }
  return cached;
}

int ensure_dynamic_smem(const void* func, int bytes, std::atomic<uint64_t>& done) {
  int dev = -1;
  QMM_CUDA_TRY(cudaGetDevice(&dev));
  if (device_marked(done, dev)) return QMM_OK;
  // Setting the attribute twice is harmless, so two threads racing here both set it; the mark is
  // made only after the attribute is in place, so nobody launches without it.
  QMM_CUDA_TRY(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  mark_device_once(done, dev);
  return QMM_OK;
}

int env_int_once(const char* name, int dflt, std::atomic<int>& cache) {
  // cache: INT_MIN = not read yet
  int v = cache.load(std::memory_order_relaxed);
  if (v != INT32_MIN) return v;
  const char* e = getenv(name);
  v = (e && *e) ? atoi(e) : dflt;
  if (v == INT32_MIN) v = dflt;
  cache.store(v, std::memory_order_relaxed);
  return v;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      cudaGetLastError();
  });
  return fn;
}

int make_tensor_map_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt,
                       uint32_t elem_bytes, uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                       uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  QMM_REQUIRE(fn != nullptr, QMM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  QMM_REQUIRE(aligned(base, 16), QMM_ERR_INVALID_ARGUMENT, "TMA base address must be 16-byte aligned");
  QMM_REQUIRE(pitch_bytes % 16 == 0, QMM_ERR_INVALID_ARGUMENT,
              "TMA row pitch (%llu bytes) must be a multiple of 16", (unsigned long long)pitch_bytes);
  QMM_REQUIRE((uint64_t)box_cols * elem_bytes % 16 == 0 && box_cols <= 256 && box_rows <= 256,
              QMM_ERR_INVALID_ARGUMENT, "bad TMA box %u x %u", box_rows, box_cols);
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  QMM_REQUIRE(r == CUDA_SUCCESS, QMM_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d",
              (int)r);
  (void)elem_bytes;
  return QMM_OK;
}

}  // namespace qmm

extern "C" {

int qmm_set_cta_limit(int max_ctas) {
  if (max_ctas < 0) return qmm::set_error(QMM_ERR_INVALID_ARGUMENT, "qmm_set_cta_limit: negative limit");
  qmm::g_cta_limit.store(max_ctas, std::memory_order_relaxed);
  return QMM_OK;
}


const char* qmm_version(void) { return "qmm-b200 0.1 (sm_100a)"; }

const char* qmm_status_name(int s) {
  switch (s) {
    case QMM_OK: return "QMM_OK";
    case QMM_ERR_INVALID_ARGUMENT: return "QMM_ERR_INVALID_ARGUMENT";
    case QMM_ERR_UNSUPPORTED: return "QMM_ERR_UNSUPPORTED";
    case QMM_ERR_CUDA: return "QMM_ERR_CUDA";
    case QMM_ERR_WORKSPACE: return "QMM_ERR_WORKSPACE";
    case QMM_ERR_TIMEOUT: return "QMM_ERR_TIMEOUT";
    case QMM_ERR_PARSE: return "QMM_ERR_PARSE";
    default: return "QMM_ERR_UNKNOWN";
  }
}

size_t qmm_last_error(char* buf, size_t cap) {
  size_t n = strlen(qmm::g_err);
  if (buf && cap) {
    size_t c = n < cap - 1 ? n : cap - 1;
    memcpy(buf, qmm::g_err, c);
    buf[c] = 0;
  }
  return n;
}

int qmm_selftest_host(void) {
  // per-device once bookkeeping: every ordinal fires exactly once, independently of the others
  std::atomic<uint64_t> mask{0};
  for (int round = 0; round < 2; ++round)
    for (int d = 0; d < qmm::kMaxDevices; ++d) {
      const bool first = qmm::mark_device_once(mask, d);
      if (first != (round == 0)) return 1;
      if (!qmm::device_marked(mask, d)) return 2;
    }
  std::atomic<uint64_t> other{0};
  if (qmm::device_marked(other, 3) || !qmm::mark_device_once(other, 3) || qmm::device_marked(other, 4)) return 3;
  if (!qmm::mark_device_once(other, -1) || !qmm::mark_device_once(other, qmm::kMaxDevices)) return 4;
  std::atomic<int> cache{INT32_MIN};
  if (qmm::env_int_once("QMM_SELFTEST_UNSET_VARIABLE", 7, cache) != 7 || cache.load() != 7) return 5;
  return 0;
}

int qmm_device_status(void) { return qmm::read_device_status(); }
void qmm_clear_device_status(void) { qmm::clear_device_status(); }

}  // extern "C"

// Runtime objects of libqmm.so: client, devices, memories, buffers, events and
// executables behind the C ABI of include/qmm_rt.h.
//
// The reference's counterparts are MpsClient / MpsDevice
// (src/pjrt_plugin/core/mps_client.mm), MpsBuffer (core/mps_buffer.mm),
// CompletionEventState (core/completion_event.h) and MpsExecutable's execute
// path (core/mps_executable.mm:9152-11725) with the PJRT glue in
// src/pjrt_plugin/api/*.cc.  The CUDA design differs where the hardware does:
//  * device memory comes from the device's stream-ordered pool (cudaMallocAsync)
//    and goes back with cudaFreeAsync behind the buffer's producer, so delete
//    keeps the reference's guarantee ("the GPU is done with it") without
//    blocking the host (the reference waits, core/mps_buffer.mm:656-669);
//  * every device has an execution stream (compute and uploads, in order) and a
//    download stream that waits on producer events;
//  * a host-visible event completes through a host function queued on the
//    stream, which only hands the event to the client's completion thread;
//    ready callbacks run there and may therefore call back into this library.
#include <cuda_runtime.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../../include/qmm_rt.h"
#include "../common.cuh"

using qmm::set_error;

namespace {

// ---------------------------------------------------------------------------
// completion state of a host-visible event
// ---------------------------------------------------------------------------
struct EventState {
  mutable std::mutex mu;
  mutable std::condition_variable cv;
  std::atomic<bool> ready{false};
  int status = QMM_OK;
  std::string message;
  std::vector<std::function<void()>> callbacks;

  void finish(int st, std::string msg) {
    std::vector<std::function<void()>> cbs;
    {
      std::lock_guard<std::mutex> lock(mu);
      if (ready.load(std::memory_order_relaxed)) return;  // the first completion wins
      status = st;
      message = std::move(msg);
      ready.store(true, std::memory_order_release);
      cbs.swap(callbacks);
    }
    cv.notify_all();
    for (auto& cb : cbs)
      if (cb) cb();
  }
  // true when ready within the timeout; the event stays pending otherwise
  bool await_ms(int timeout_ms) const {
    if (ready.load(std::memory_order_acquire)) return true;
    std::unique_lock<std::mutex> lock(mu);
    return cv.wait_for(lock, std::chrono::milliseconds(timeout_ms),
                       [&] { return ready.load(std::memory_order_relaxed); });
  }
  void add_callback(std::function<void()> cb) {
    bool now = false;
    {
      std::lock_guard<std::mutex> lock(mu);
      if (ready.load(std::memory_order_relaxed)) now = true;
      else callbacks.push_back(cb);
    }
    if (now) cb();
  }
};
using EventRef = std::shared_ptr<EventState>;

EventRef make_ready_event() {
  auto e = std::make_shared<EventState>();
  e->ready.store(true);
  return e;
}

int completion_timeout_ms() {
  // read per wait, like the reference's JAX_METALLIB_COMPLETION_TIMEOUT_MS
  const char* e = getenv("QMM_RT_COMPLETION_TIMEOUT_MS");
  const int v = e ? atoi(e) : 0;
  return v > 0 ? v : 30000;
}

struct CudaEvent {  // a device event shared by the outputs of one launch
  cudaEvent_t ev = nullptr;
  int ordinal = 0;
  ~CudaEvent() {
    if (ev) cudaEventDestroy(ev);
  }
};
using CudaEventRef = std::shared_ptr<CudaEvent>;

size_t dtype_bits(int dtype) {
  switch (dtype) {
    case QMM_F32: case QMM_S32: case QMM_U32: return 32;
    case QMM_F16: case QMM_BF16: return 16;
    case QMM_S8: case QMM_U8: return 8;
    case QMM_U4: return 4;
    default: return 0;
  }
}

}  // namespace

// ---------------------------------------------------------------------------
// handle structs
// ---------------------------------------------------------------------------
struct qmm_rt_event {
  EventRef st;
};

struct qmm_rt_memory {
  qmm_rt_device* device = nullptr;
  int id = 0;
  std::string debug, text;
  std::mutex mu;
  struct UserData { void* data; qmm_rt_user_data_deleter del; };
  std::map<uint64_t, UserData> user;
  ~qmm_rt_memory() {
    // each datum is destroyed exactly once, outside the lock
    std::map<uint64_t, UserData> tmp;
    {
      std::lock_guard<std::mutex> lock(mu);
      tmp.swap(user);
    }
    for (auto& kv : tmp)
      if (kv.second.del) kv.second.del(kv.second.data);
  }
};

struct qmm_rt_device {
  qmm_rt_client* client = nullptr;
  int id = 0;        // global id == local hardware id (one process)
  int ordinal = 0;   // CUDA device ordinal
  // Streams (and with them the device's CUDA context) are created when the device is first used,
  // so a client on a box with eight GPUs touches only the GPUs it is given work for.
  std::mutex stream_mu;
  bool streams_ready = false;
  cudaStream_t exec = nullptr, d2h = nullptr;
  std::string kind, debug, text;
  std::unique_ptr<qmm_rt_memory> memory;
  std::atomic<int64_t> bytes_in_use{0};
  int64_t bytes_limit = 0;
};

struct qmm_rt_client {
  std::vector<std::unique_ptr<qmm_rt_device>> devices;
  std::string platform_version;
  // completion thread: jobs are queued by host functions on the streams
  std::mutex qmu;
  std::condition_variable qcv;
  std::deque<std::function<void()>> jobs;
  bool stopping = false;
  std::thread worker;

  void post(std::function<void()> job) {
    {
      std::lock_guard<std::mutex> lock(qmu);
      jobs.push_back(std::move(job));
    }
    qcv.notify_one();
  }
  void run() {
    std::unique_lock<std::mutex> lock(qmu);
    while (true) {
      qcv.wait(lock, [&] { return stopping || !jobs.empty(); });
      if (jobs.empty() && stopping) return;
      auto job = std::move(jobs.front());
      jobs.pop_front();
      lock.unlock();
      job();
      lock.lock();
    }
  }
};

struct qmm_rt_buffer {
  qmm_rt_client* client = nullptr;
  qmm_rt_device* device = nullptr;
  int dtype = 0;
  std::vector<int64_t> dims;
  size_t bytes = 0;        // of the data
  size_t alloc_bytes = 0;  // of the allocation (placeholder for zero-element shapes)
  void* ptr = nullptr;
  bool owns = false;
  qmm_rt_on_delete on_delete = nullptr;
  void* on_delete_arg = nullptr;
  CudaEventRef produced;   // device-side: contents defined after this (null: defined already)
  EventRef ready;          // host-side view of the same (may carry an error)
  std::mutex mu;
  bool deleted = false;
  bool released = false;
  int external_refs = 0;
};

struct qmm_rt_executable {
  qmm_rt_client* client = nullptr;
  qmm_plan* plan = nullptr;
  std::string text, name, fingerprint;
  struct TensorInfo { int dtype; std::vector<int64_t> dims; size_t bytes; };
  std::vector<TensorInfo> args, outs;
  size_t workspace_bytes = 0;
  std::mutex mu;
  std::map<int, void*> workspace;  // per device ordinal, zeroed once
  std::atomic<bool> deleted{false};
};

namespace {

struct HostJob {
  qmm_rt_client* client;
  std::function<void()> fn;
};
void CUDART_CB host_trampoline(void* p) {
  // runs on a CUDA-internal thread: no CUDA calls here, only hand the job over
  std::unique_ptr<HostJob> job(static_cast<HostJob*>(p));
  job->client->post(std::move(job->fn));
}
// Run `fn` on the client's completion thread once everything queued on `stream` so far is done.
int after_stream(qmm_rt_client* c, cudaStream_t stream, std::function<void()> fn) {
  auto* job = new HostJob{c, std::move(fn)};
  cudaError_t e = cudaLaunchHostFunc(stream, host_trampoline, job);
  if (e != cudaSuccess) {
    delete job;
    return set_error(QMM_ERR_CUDA, "cudaLaunchHostFunc failed: %s", cudaGetErrorString(e));
  }
  return QMM_OK;
}

int device_ready(qmm_rt_device* d) {
  QMM_REQUIRE(d != nullptr, QMM_ERR_INVALID_ARGUMENT, "null device");
  std::lock_guard<std::mutex> lock(d->stream_mu);
  if (d->streams_ready) return QMM_OK;
  QMM_CUDA_TRY(cudaSetDevice(d->ordinal));
  QMM_CUDA_TRY(cudaStreamCreateWithFlags(&d->exec, cudaStreamNonBlocking));
  QMM_CUDA_TRY(cudaStreamCreateWithFlags(&d->d2h, cudaStreamNonBlocking));
  d->streams_ready = true;
  return QMM_OK;
}

int element_count(const int64_t* dims, int rank, int64_t* count) {
  int64_t n = 1;
  for (int i = 0; i < rank; ++i) {
    QMM_REQUIRE(dims[i] >= 0, QMM_ERR_INVALID_ARGUMENT, "negative dimension %lld", (long long)dims[i]);
    QMM_REQUIRE(dims[i] == 0 || n <= (int64_t(1) << 40) / (dims[i] ? dims[i] : 1), QMM_ERR_INVALID_ARGUMENT,
                "tensor too large");
    n *= dims[i];
  }
  *count = n;
  return QMM_OK;
}

int tensor_bytes(int dtype, const int64_t* dims, int rank, size_t* bytes) {
  const size_t bits = dtype_bits(dtype);
  QMM_REQUIRE(bits != 0, QMM_ERR_INVALID_ARGUMENT, "unknown element type %d", dtype);
  QMM_REQUIRE(rank >= 0 && rank <= 8 && (rank == 0 || dims != nullptr), QMM_ERR_INVALID_ARGUMENT, "bad rank %d", rank);
  int64_t n = 0;
  if (int rc = element_count(dims, rank, &n)) return rc;
  if (dtype == QMM_U4)
    QMM_REQUIRE(rank >= 1 && dims[rank - 1] % 2 == 0, QMM_ERR_INVALID_ARGUMENT,
                "4-bit tensors need an even innermost dimension (two elements per byte)");
  *bytes = static_cast<size_t>(n) * bits / 8;
  return QMM_OK;
}

qmm_rt_device* pick_device(qmm_rt_client* c, qmm_rt_device* d) {
  if (d) return d;
  return c->devices.empty() ? nullptr : c->devices[0].get();
}

// New owned buffer on `dev` (uninitialised), allocated in stream order on the execution stream.
int new_buffer(qmm_rt_client* c, qmm_rt_device* dev, int dtype, const int64_t* dims, int rank, qmm_rt_buffer** out) {
  size_t bytes = 0;
  if (int rc = tensor_bytes(dtype, dims, rank, &bytes)) return rc;
  QMM_REQUIRE(dev != nullptr && dev->client == c, QMM_ERR_INVALID_ARGUMENT, "the device does not belong to this client");
  if (int rc = device_ready(dev)) return rc;
  QMM_CUDA_TRY(cudaSetDevice(dev->ordinal));
  // a zero-element shape still gets an address of its own (a placeholder allocation)
  const size_t alloc = bytes ? bytes : 256;
  void* p = nullptr;
  QMM_CUDA_TRY(cudaMallocAsync(&p, alloc, dev->exec));
  auto* b = new qmm_rt_buffer();
  b->client = c;
  b->device = dev;
  b->dtype = dtype;
  b->dims.assign(dims, dims + rank);
  b->bytes = bytes;
  b->alloc_bytes = alloc;
  b->ptr = p;
  b->owns = true;
  b->ready = make_ready_event();
  dev->bytes_in_use.fetch_add(static_cast<int64_t>(alloc));
  *out = b;
  return QMM_OK;
}

// Hand the storage back (once).  Called with b->mu held.
void release_storage(qmm_rt_buffer* b) {
  if (b->released) return;
  b->released = true;
  if (!b->ptr) return;
  qmm_rt_device* dev = b->device;
  if (b->owns) {
    cudaSetDevice(dev->ordinal);
    // behind the producer and behind any download still reading it
    if (b->produced && b->produced->ev) cudaStreamWaitEvent(dev->exec, b->produced->ev, 0);
    cudaEvent_t tail = nullptr;
    if (cudaEventCreateWithFlags(&tail, cudaEventDisableTiming) == cudaSuccess) {
      cudaEventRecord(tail, dev->d2h);
      cudaStreamWaitEvent(dev->exec, tail, 0);
      cudaEventDestroy(tail);
    }
    cudaFreeAsync(b->ptr, dev->exec);
    dev->bytes_in_use.fetch_sub(static_cast<int64_t>(b->alloc_bytes));
  } else if (b->on_delete) {
    b->on_delete(b->ptr, b->on_delete_arg);
  }
  b->ptr = nullptr;
}

// Mark `b` as produced by whatever was queued on the execution stream so far.
int mark_produced(qmm_rt_buffer* b, CudaEventRef ev, EventRef ready) {
  b->produced = std::move(ev);
  b->ready = std::move(ready);
  return QMM_OK;
}

int record_event(qmm_rt_device* dev, cudaStream_t stream, CudaEventRef* out) {
  auto ev = std::make_shared<CudaEvent>();
  ev->ordinal = dev->ordinal;
  QMM_CUDA_TRY(cudaEventCreateWithFlags(&ev->ev, cudaEventDisableTiming));
  QMM_CUDA_TRY(cudaEventRecord(ev->ev, stream));
  *out = std::move(ev);
  return QMM_OK;
}

std::string fnv1a_hex(const std::string& s) {
  uint64_t h = 1469598103934665603ull;
  for (unsigned char c : s) {
    h ^= c;
    h *= 1099511628211ull;
  }
  char buf[17];
  snprintf(buf, sizeof(buf), "%016llx", (unsigned long long)h);
  return buf;
}

constexpr char kBlobMagic[4] = {'Q', 'M', 'M', 'X'};
constexpr uint32_t kBlobVersion = 1;

int make_executable(qmm_rt_client* c, const char* program, size_t size, qmm_rt_executable** out) {
  qmm_plan* plan = nullptr;
  if (int rc = qmm_plan_compile(program, size, &plan)) return rc;
  auto exe = std::unique_ptr<qmm_rt_executable>(new qmm_rt_executable());
  exe->client = c;
  exe->plan = plan;
  exe->text.assign(program, size);
  exe->name = qmm_plan_name(plan);
  exe->fingerprint = fnv1a_hex(exe->text);
  exe->workspace_bytes = qmm_plan_workspace_bytes(plan);
  auto fill = [&](bool results, int n, std::vector<qmm_rt_executable::TensorInfo>& v) -> int {
    for (int i = 0; i < n; ++i) {
      int dtype = -1, rank = 8;
      int64_t dims[8];
      int rc = results ? qmm_plan_result_info(plan, i, &dtype, dims, &rank) : qmm_plan_arg_info(plan, i, &dtype, dims, &rank);
      if (rc) return rc;
      size_t bytes = 0;
      QMM_REQUIRE(dtype >= 0, QMM_ERR_UNSUPPORTED, "%s %d has an element type this runtime has no buffers for",
                  results ? "result" : "argument", i);
      if (int rc2 = tensor_bytes(dtype, dims, rank, &bytes)) return rc2;
      v.push_back({dtype, std::vector<int64_t>(dims, dims + rank), bytes});
    }
    return QMM_OK;
  };
  int rc = fill(false, qmm_plan_num_args(plan), exe->args);
  if (!rc) rc = fill(true, qmm_plan_num_results(plan), exe->outs);
  if (rc) {
    qmm_plan_destroy(plan);
    return rc;
  }
  *out = exe.release();
  return QMM_OK;
}

}  // namespace

extern "C" {

int qmm_rt_status_to_pjrt_code(int status) {
  switch (status) {
    case QMM_OK: return 0;                        // OK
    case QMM_ERR_INVALID_ARGUMENT: return 3;      // INVALID_ARGUMENT
    case QMM_ERR_TIMEOUT: return 4;               // DEADLINE_EXCEEDED
    case QMM_ERR_WORKSPACE: return 8;             // RESOURCE_EXHAUSTED
    case QMM_ERR_UNSUPPORTED: return 12;          // UNIMPLEMENTED
    case QMM_ERR_PARSE: return 3;                 // INVALID_ARGUMENT
    case QMM_ERR_CUDA: default: return 13;        // INTERNAL
  }
}

// ------------------------------------------------------------------ client
int qmm_rt_client_create(qmm_rt_client** out) {
  QMM_REQUIRE(out != nullptr, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_client_create: null argument");
  *out = nullptr;
  int n = 0;
  QMM_CUDA_TRY(cudaGetDeviceCount(&n));
  QMM_REQUIRE(n > 0, QMM_ERR_CUDA, "no CUDA device is visible");
  auto c = std::unique_ptr<qmm_rt_client>(new qmm_rt_client());
  int rt = 0, drv = 0;
  cudaRuntimeGetVersion(&rt);
  cudaDriverGetVersion(&drv);
  c->platform_version = std::string(qmm_version()) + "; CUDA runtime " + std::to_string(rt) + ", driver " + std::to_string(drv);
  for (int i = 0; i < n; ++i) {
    auto d = std::unique_ptr<qmm_rt_device>(new qmm_rt_device());
    d->client = c.get();
    d->id = i;
    d->ordinal = i;
    cudaDeviceProp prop;
    QMM_CUDA_TRY(cudaGetDeviceProperties(&prop, i));
    d->kind = prop.name;
    d->bytes_limit = static_cast<int64_t>(prop.totalGlobalMem);
    d->debug = "QmmDevice(id=" + std::to_string(i) + ", kind=" + d->kind + ", sm_" + std::to_string(prop.major) +
               std::to_string(prop.minor) + ", " + std::to_string(prop.multiProcessorCount) + " SMs)";
    d->text = "qmm_b200:" + std::to_string(i);
    d->memory.reset(new qmm_rt_memory());
    d->memory->device = d.get();
    d->memory->id = i;
    d->memory->debug = "QmmMemory(id=" + std::to_string(i) + ", kind=device, device=" + std::to_string(i) + ")";
    d->memory->text = "device_memory:" + std::to_string(i);
    c->devices.push_back(std::move(d));
  }
  qmm_rt_client* raw = c.get();
  c->worker = std::thread([raw] { raw->run(); });
  *out = c.release();
  return QMM_OK;
}

int qmm_rt_client_destroy(qmm_rt_client* c) {
  if (!c) return QMM_OK;
  // everything queued on the client's streams completes first, so no host function is left
  // that could post to the completion thread after it has gone
  for (auto& d : c->devices) {
    if (!d->streams_ready) continue;
    cudaSetDevice(d->ordinal);
    cudaStreamSynchronize(d->exec);
    cudaStreamSynchronize(d->d2h);
  }
  {
    std::lock_guard<std::mutex> lock(c->qmu);
    c->stopping = true;
  }
  c->qcv.notify_all();
  if (c->worker.joinable()) c->worker.join();
  for (auto& d : c->devices) {
    if (!d->streams_ready) continue;
    cudaSetDevice(d->ordinal);
    cudaStreamDestroy(d->exec);
    cudaStreamDestroy(d->d2h);
  }
  delete c;
  return QMM_OK;
}

qmm_rt_client* qmm_rt_default_client(void) {
  static std::once_flag once;
  static qmm_rt_client* client = nullptr;  // lives until the process exits
  std::call_once(once, [] { qmm_rt_client_create(&client); });
  return client;
}

const char* qmm_rt_client_platform_name(const qmm_rt_client*) { return "qmm_b200"; }
const char* qmm_rt_client_platform_version(const qmm_rt_client* c) { return c ? c->platform_version.c_str() : ""; }
int qmm_rt_client_process_index(const qmm_rt_client*) { return 0; }
int qmm_rt_client_num_devices(const qmm_rt_client* c) { return c ? static_cast<int>(c->devices.size()) : 0; }
qmm_rt_device* qmm_rt_client_device(const qmm_rt_client* c, int i) {
  return (c && i >= 0 && i < static_cast<int>(c->devices.size())) ? c->devices[i].get() : nullptr;
}
int qmm_rt_client_lookup_device(const qmm_rt_client* c, int id, qmm_rt_device** out) {
  QMM_REQUIRE(c && out, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_client_lookup_device: null argument");
  *out = qmm_rt_client_device(c, id);
  QMM_REQUIRE(*out != nullptr, QMM_ERR_INVALID_ARGUMENT, "no device with id %d", id);
  return QMM_OK;
}
int qmm_rt_client_num_memories(const qmm_rt_client* c) { return qmm_rt_client_num_devices(c); }
qmm_rt_memory* qmm_rt_client_memory(const qmm_rt_client* c, int i) {
  qmm_rt_device* d = qmm_rt_client_device(c, i);
  return d ? d->memory.get() : nullptr;
}
int qmm_rt_client_default_device_assignment(const qmm_rt_client* c, int num_replicas, int num_partitions,
                                            int* assignment, size_t capacity) {
  QMM_REQUIRE(c && assignment && num_replicas >= 1 && num_partitions >= 1, QMM_ERR_INVALID_ARGUMENT,
              "qmm_rt_client_default_device_assignment: bad arguments");
  const size_t need = static_cast<size_t>(num_replicas) * num_partitions;
  QMM_REQUIRE(capacity >= need, QMM_ERR_INVALID_ARGUMENT, "assignment needs %zu entries, the caller has %zu", need, capacity);
  QMM_REQUIRE(need <= c->devices.size(), QMM_ERR_INVALID_ARGUMENT, "%zu devices requested, the client has %zu", need,
              c->devices.size());
  for (size_t i = 0; i < need; ++i) assignment[i] = static_cast<int>(i);
  return QMM_OK;
}

// ------------------------------------------------------------------ device
int qmm_rt_device_id(const qmm_rt_device* d) { return d ? d->id : -1; }
int qmm_rt_device_process_index(const qmm_rt_device*) { return 0; }
int qmm_rt_device_local_hardware_id(const qmm_rt_device* d) { return d ? d->ordinal : -1; }
int qmm_rt_device_is_addressable(const qmm_rt_device* d) { return d ? 1 : 0; }
const char* qmm_rt_device_kind(const qmm_rt_device* d) { return d ? d->kind.c_str() : ""; }
const char* qmm_rt_device_debug_string(const qmm_rt_device* d) { return d ? d->debug.c_str() : ""; }
const char* qmm_rt_device_to_string(const qmm_rt_device* d) { return d ? d->text.c_str() : ""; }
qmm_rt_memory* qmm_rt_device_default_memory(const qmm_rt_device* d) { return d ? d->memory.get() : nullptr; }
int qmm_rt_device_memory_stats(const qmm_rt_device* d, int64_t* in_use, int64_t* limit) {
  QMM_REQUIRE(d != nullptr, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_device_memory_stats: null device");
  if (in_use) *in_use = d->bytes_in_use.load();
  if (limit) *limit = d->bytes_limit;
  return QMM_OK;
}

// ------------------------------------------------------------------ memory
int qmm_rt_memory_id(const qmm_rt_memory* m) { return m ? m->id : -1; }
const char* qmm_rt_memory_kind(const qmm_rt_memory*) { return "device"; }
int qmm_rt_memory_kind_id(const qmm_rt_memory*) { return 0; }
const char* qmm_rt_memory_debug_string(const qmm_rt_memory* m) { return m ? m->debug.c_str() : ""; }
const char* qmm_rt_memory_to_string(const qmm_rt_memory* m) { return m ? m->text.c_str() : ""; }
qmm_rt_device* qmm_rt_memory_device(const qmm_rt_memory* m) { return m ? m->device : nullptr; }
int qmm_rt_memory_set_user_data(qmm_rt_memory* m, uint64_t key, void* data, qmm_rt_user_data_deleter del) {
  QMM_REQUIRE(m != nullptr, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_memory_set_user_data: null memory");
  qmm_rt_memory::UserData old{nullptr, nullptr};
  bool had = false;
  {
    std::lock_guard<std::mutex> lock(m->mu);
    auto it = m->user.find(key);
    if (it != m->user.end()) {
      old = it->second;
      had = true;
    }
    m->user[key] = {data, del};
  }
  if (had && old.del) old.del(old.data);  // the replaced datum, outside the lock
  return QMM_OK;
}
void* qmm_rt_memory_get_user_data(qmm_rt_memory* m, uint64_t key) {
  if (!m) return nullptr;
  std::lock_guard<std::mutex> lock(m->mu);
  auto it = m->user.find(key);
  return it == m->user.end() ? nullptr : it->second.data;
}

// ------------------------------------------------------------------- event
int qmm_rt_event_create(qmm_rt_event** out) {
  QMM_REQUIRE(out != nullptr, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_event_create: null argument");
  *out = new qmm_rt_event{std::make_shared<EventState>()};
  return QMM_OK;
}
int qmm_rt_event_set(qmm_rt_event* e, int status, const char* message) {
  QMM_REQUIRE(e && e->st, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_event_set: null event");
  e->st->finish(status, message ? message : "");
  return QMM_OK;
}
int qmm_rt_event_destroy(qmm_rt_event* e) {
  delete e;  // the completion state lives on while a stream job or a buffer still refers to it
  return QMM_OK;
}
int qmm_rt_event_is_ready(const qmm_rt_event* e) {
  return (!e || !e->st) ? 1 : (e->st->ready.load(std::memory_order_acquire) ? 1 : 0);
}
int qmm_rt_event_error(const qmm_rt_event* e) {
  if (!e || !e->st || !e->st->ready.load(std::memory_order_acquire)) return QMM_OK;
  std::lock_guard<std::mutex> lock(e->st->mu);
  if (e->st->status != QMM_OK) set_error(e->st->status, "%s", e->st->message.c_str());
  return e->st->status;
}
int qmm_rt_event_await(qmm_rt_event* e, int timeout_ms) {
  if (!e || !e->st) return QMM_OK;
  const int limit = timeout_ms > 0 ? timeout_ms : completion_timeout_ms();
  if (!e->st->await_ms(limit))
    return set_error(QMM_ERR_TIMEOUT,
                     "qmm_rt_event_await timed out after %d ms; the event stays pending and the device work goes on "
                     "(raise QMM_RT_COMPLETION_TIMEOUT_MS for longer programs)", limit);
  return qmm_rt_event_error(e);
}
int qmm_rt_event_on_ready(qmm_rt_event* e, qmm_rt_event_callback cb, void* arg) {
  if (!cb) return QMM_OK;
  if (!e || !e->st) {
    cb(QMM_OK, "", arg);
    return QMM_OK;
  }
  EventRef st = e->st;
  st->add_callback([st, cb, arg] {
    int status;
    std::string msg;
    {
      std::lock_guard<std::mutex> lock(st->mu);
      status = st->status;
      msg = st->message;
    }
    cb(status, msg.c_str(), arg);
  });
  return QMM_OK;
}

// ------------------------------------------------------------------ buffer
int qmm_rt_buffer_from_host(qmm_rt_client* c, const void* data, int dtype, const int64_t* dims, int rank,
                            const int64_t* byte_strides, qmm_rt_device* device, qmm_rt_buffer** out,
                            qmm_rt_event** done_with_host) {
  if (!c) c = qmm_rt_default_client();
  QMM_REQUIRE(c && out, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_buffer_from_host: null argument");
  *out = nullptr;
  if (done_with_host) *done_with_host = nullptr;
  qmm_rt_device* dev = pick_device(c, device);
  qmm_rt_buffer* b = nullptr;
  if (int rc = new_buffer(c, dev, dtype, dims, rank, &b)) return rc;
  EventRef done = make_ready_event();
  if (b->bytes > 0) {
    if (!data) {
      qmm_rt_buffer_destroy(b);
      return set_error(QMM_ERR_INVALID_ARGUMENT, "qmm_rt_buffer_from_host: null data for a non-empty tensor");
    }
    const size_t esz = dtype_bits(dtype) / 8;
    bool dense = true;
    if (byte_strides) {
      int64_t expect = static_cast<int64_t>(esz);
      for (int i = rank - 1; i >= 0; --i) {
        if (dims[i] != 1 && byte_strides[i] != expect) dense = false;
        expect *= dims[i];
      }
    }
    cudaError_t e = cudaSuccess;
    if (dense) {
      e = cudaMemcpyAsync(b->ptr, data, b->bytes, cudaMemcpyHostToDevice, dev->exec);
    } else {
      if (esz == 0) {
        qmm_rt_buffer_destroy(b);
        return set_error(QMM_ERR_UNSUPPORTED, "4-bit host tensors must be dense");
      }
      // gather the strided source into a dense staging copy: rows of the innermost dimension are
      // copied in one piece when that dimension is itself dense
      std::unique_ptr<char[]> staging(new char[b->bytes]);
      const char* src = static_cast<const char*>(data);
      const int64_t inner = dims[rank - 1];
      const bool inner_dense = byte_strides[rank - 1] == static_cast<int64_t>(esz) || inner == 1;
      std::vector<int64_t> idx(rank, 0);
      const int64_t rows = static_cast<int64_t>(b->bytes / esz) / (inner ? inner : 1);
      char* dst = staging.get();
      for (int64_t r = 0; r < rows; ++r) {
        int64_t off = 0;
        for (int d = 0; d < rank - 1; ++d) off += idx[d] * byte_strides[d];
        if (inner_dense) {
          memcpy(dst, src + off, static_cast<size_t>(inner) * esz);
        } else {
          for (int64_t i = 0; i < inner; ++i) memcpy(dst + i * esz, src + off + i * byte_strides[rank - 1], esz);
        }
        dst += static_cast<size_t>(inner) * esz;
        for (int d = rank - 2; d >= 0; --d) {
          if (++idx[d] < dims[d]) break;
          idx[d] = 0;
        }
      }
      e = cudaMemcpyAsync(b->ptr, staging.get(), b->bytes, cudaMemcpyHostToDevice, dev->exec);
      if (e == cudaSuccess) {
        // the staging copy must outlive the transfer: it is released on the completion thread
        char* keep = staging.release();
        if (after_stream(c, dev->exec, [keep] { delete[] keep; }) != QMM_OK) {
          cudaStreamSynchronize(dev->exec);
          delete[] keep;
        }
      }
    }
    if (e != cudaSuccess) {
      qmm_rt_buffer_destroy(b);
      return set_error(QMM_ERR_CUDA, "host to device copy failed: %s", cudaGetErrorString(e));
    }
    CudaEventRef ev;
    if (int rc = record_event(dev, dev->exec, &ev)) {
      qmm_rt_buffer_destroy(b);
      return rc;
    }
    done = std::make_shared<EventState>();
    EventRef d2 = done;
    if (int rc = after_stream(c, dev->exec, [d2] { d2->finish(QMM_OK, ""); })) {
      qmm_rt_buffer_destroy(b);
      return rc;
    }
    mark_produced(b, ev, done);
  }
  if (done_with_host) *done_with_host = new qmm_rt_event{done};
  *out = b;
  return QMM_OK;
}

int qmm_rt_buffer_create_uninitialized(qmm_rt_client* c, int dtype, const int64_t* dims, int rank,
                                       qmm_rt_device* device, qmm_rt_buffer** out) {
  if (!c) c = qmm_rt_default_client();
  QMM_REQUIRE(c && out, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_buffer_create_uninitialized: null argument");
  return new_buffer(c, pick_device(c, device), dtype, dims, rank, out);
}

int qmm_rt_buffer_view_of_device_memory(qmm_rt_client* c, void* device_ptr, int dtype, const int64_t* dims, int rank,
                                        qmm_rt_device* device, qmm_rt_on_delete on_delete, void* user_arg,
                                        qmm_rt_buffer** out) {
  if (!c) c = qmm_rt_default_client();
  QMM_REQUIRE(c && out, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_buffer_view_of_device_memory: null argument");
  size_t bytes = 0;
  if (int rc = tensor_bytes(dtype, dims, rank, &bytes)) return rc;
  QMM_REQUIRE(device_ptr != nullptr || bytes == 0, QMM_ERR_INVALID_ARGUMENT, "null device pointer");
  qmm_rt_device* dev = pick_device(c, device);
  QMM_REQUIRE(dev != nullptr && dev->client == c, QMM_ERR_INVALID_ARGUMENT, "the device does not belong to this client");
  if (int rc = device_ready(dev)) return rc;
  auto* b = new qmm_rt_buffer();
  b->client = c;
  b->device = dev;
  b->dtype = dtype;
  b->dims.assign(dims, dims + rank);
  b->bytes = b->alloc_bytes = bytes;
  b->ptr = device_ptr;
  b->owns = false;
  b->on_delete = on_delete;
  b->on_delete_arg = user_arg;
  b->ready = make_ready_event();
  *out = b;
  return QMM_OK;
}

int qmm_rt_buffer_create_error(qmm_rt_client* c, int status, const char* message, int dtype, const int64_t* dims,
                               int rank, qmm_rt_device* device, qmm_rt_buffer** out) {
  if (!c) c = qmm_rt_default_client();
  QMM_REQUIRE(c && out && status != QMM_OK, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_buffer_create_error: bad arguments");
  size_t bytes = 0;
  if (int rc = tensor_bytes(dtype, dims, rank, &bytes)) return rc;
  auto* b = new qmm_rt_buffer();
  b->client = c;
  b->device = pick_device(c, device);
  b->dtype = dtype;
  b->dims.assign(dims, dims + rank);
  b->bytes = bytes;
  b->ready = std::make_shared<EventState>();
  b->ready->finish(status, message ? message : "error buffer");
  *out = b;
  return QMM_OK;
}

int qmm_rt_buffer_dtype(const qmm_rt_buffer* b) { return b ? b->dtype : -1; }
int qmm_rt_buffer_rank(const qmm_rt_buffer* b) { return b ? static_cast<int>(b->dims.size()) : 0; }
const int64_t* qmm_rt_buffer_dims(const qmm_rt_buffer* b) { return b ? b->dims.data() : nullptr; }
size_t qmm_rt_buffer_size_bytes(const qmm_rt_buffer* b) { return b ? b->bytes : 0; }
qmm_rt_device* qmm_rt_buffer_device(const qmm_rt_buffer* b) { return b ? b->device : nullptr; }
qmm_rt_memory* qmm_rt_buffer_memory(const qmm_rt_buffer* b) { return (b && b->device) ? b->device->memory.get() : nullptr; }
int qmm_rt_buffer_is_on_cpu(const qmm_rt_buffer*) { return 0; }

int qmm_rt_buffer_delete(qmm_rt_buffer* b) {
  if (!b) return QMM_OK;
  std::lock_guard<std::mutex> lock(b->mu);
  b->deleted = true;
  if (b->external_refs == 0) release_storage(b);
  return QMM_OK;
}
int qmm_rt_buffer_is_deleted(const qmm_rt_buffer* b) {
  if (!b) return 1;
  std::lock_guard<std::mutex> lock(const_cast<qmm_rt_buffer*>(b)->mu);
  return b->deleted ? 1 : 0;
}
int qmm_rt_buffer_destroy(qmm_rt_buffer* b) {
  if (!b) return QMM_OK;
  {
    std::lock_guard<std::mutex> lock(b->mu);
    b->deleted = true;
    release_storage(b);  // the handle goes away: external references can no longer be dropped through it
  }
  delete b;
  return QMM_OK;
}

int qmm_rt_buffer_ready_event(qmm_rt_buffer* b, qmm_rt_event** out) {
  QMM_REQUIRE(b && out, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_buffer_ready_event: null argument");
  *out = new qmm_rt_event{b->ready ? b->ready : make_ready_event()};
  return QMM_OK;
}

static int read_to_host(qmm_rt_buffer* b, void* dst, int64_t offset, int64_t size, qmm_rt_event** out,
                        const char* what) {
  // failures are reported through the event, as the reference's ToHostBuffer does
  auto st = std::make_shared<EventState>();
  *out = new qmm_rt_event{st};
  auto fail = [&](int status, const std::string& msg) {
    st->finish(status, std::string(what) + ": " + msg);
    return QMM_OK;
  };
  std::lock_guard<std::mutex> lock(b->mu);
  if (b->deleted || b->released) return fail(QMM_ERR_INVALID_ARGUMENT, "the buffer is deleted");
  if (b->ready && b->ready->ready.load() && b->ready->status != QMM_OK)
    return fail(b->ready->status, b->ready->message);
  if (offset < 0 || size < 0 || static_cast<size_t>(offset) + static_cast<size_t>(size) > b->bytes)
    return fail(QMM_ERR_INVALID_ARGUMENT, "offset/size out of range");
  if (size == 0) {
    st->finish(QMM_OK, "");
    return QMM_OK;
  }
  if (!dst) return fail(QMM_ERR_INVALID_ARGUMENT, "null destination");
  qmm_rt_device* dev = b->device;
  cudaError_t e = cudaSetDevice(dev->ordinal);
  if (e == cudaSuccess && b->produced && b->produced->ev) e = cudaStreamWaitEvent(dev->d2h, b->produced->ev, 0);
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(dst, static_cast<const char*>(b->ptr) + offset, static_cast<size_t>(size), cudaMemcpyDeviceToHost,
                        dev->d2h);
  if (e != cudaSuccess) return fail(QMM_ERR_CUDA, cudaGetErrorString(e));
  EventRef producer = b->ready;
  if (after_stream(b->client, dev->d2h, [st, producer] {
        // a producer that failed (a kernel wait that gave up) taints what was read
        if (producer && producer->ready.load() && producer->status != QMM_OK) st->finish(producer->status, producer->message);
        else st->finish(QMM_OK, "");
      }) != QMM_OK) {
    cudaStreamSynchronize(dev->d2h);
    st->finish(QMM_OK, "");
  }
  return QMM_OK;
}

int qmm_rt_buffer_to_host(qmm_rt_buffer* b, void* dst, size_t dst_size, size_t* needed, qmm_rt_event** event) {
  QMM_REQUIRE(b != nullptr, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_buffer_to_host: null buffer");
  if (needed) *needed = b->bytes;
  if (!dst) {  // size query
    if (event) *event = new qmm_rt_event{make_ready_event()};
    return QMM_OK;
  }
  QMM_REQUIRE(event != nullptr, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_buffer_to_host: null event pointer");
  if (dst_size < b->bytes) {
    auto st = std::make_shared<EventState>();
    st->finish(QMM_ERR_INVALID_ARGUMENT, "ToHostBuffer: destination of " + std::to_string(dst_size) +
                                             " bytes is smaller than the buffer (" + std::to_string(b->bytes) + ")");
    *event = new qmm_rt_event{st};
    return QMM_OK;
  }
  return read_to_host(b, dst, 0, static_cast<int64_t>(b->bytes), event, "ToHostBuffer");
}

int qmm_rt_buffer_copy_raw_to_host(qmm_rt_buffer* b, void* dst, int64_t offset, int64_t size, qmm_rt_event** event) {
  QMM_REQUIRE(b && event, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_buffer_copy_raw_to_host: null argument");
  return read_to_host(b, dst, offset, size, event, "CopyRawToHost");
}

int qmm_rt_buffer_copy_to_device(qmm_rt_buffer* b, qmm_rt_device* device, qmm_rt_buffer** out) {
  QMM_REQUIRE(b && device && out, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_buffer_copy_to_device: null argument");
  QMM_REQUIRE(device->client == b->client, QMM_ERR_INVALID_ARGUMENT, "the target device belongs to another client");
  std::lock_guard<std::mutex> lock(b->mu);
  QMM_REQUIRE(!b->deleted && !b->released && (b->ptr || b->bytes == 0), QMM_ERR_INVALID_ARGUMENT, "the source buffer is deleted");
  qmm_rt_buffer* copy = nullptr;
  if (int rc = new_buffer(b->client, device, b->dtype, b->dims.data(), static_cast<int>(b->dims.size()), &copy)) return rc;
  if (b->bytes) {
    cudaError_t e = cudaSuccess;
    if (b->produced && b->produced->ev) e = cudaStreamWaitEvent(device->exec, b->produced->ev, 0);
    if (e == cudaSuccess)
      e = cudaMemcpyPeerAsync(copy->ptr, device->ordinal, b->ptr, b->device->ordinal, b->bytes, device->exec);
    if (e != cudaSuccess) {
      qmm_rt_buffer_destroy(copy);
      return set_error(QMM_ERR_CUDA, "device to device copy failed: %s", cudaGetErrorString(e));
    }
    CudaEventRef ev;
    if (int rc = record_event(device, device->exec, &ev)) {
      qmm_rt_buffer_destroy(copy);
      return rc;
    }
    auto done = std::make_shared<EventState>();
    EventRef d2 = done;
    if (after_stream(b->client, device->exec, [d2] { d2->finish(QMM_OK, ""); }) != QMM_OK) done = make_ready_event();
    mark_produced(copy, ev, done);
    // the source may be deleted right after this call: its free is queued on its own device's
    // stream, which must not run ahead of this copy
    if (b->device != device) {
      cudaSetDevice(b->device->ordinal);
      cudaStreamWaitEvent(b->device->exec, ev->ev, 0);
    }
  }
  *out = copy;
  return QMM_OK;
}

void* qmm_rt_buffer_device_pointer(const qmm_rt_buffer* b) { return b ? b->ptr : nullptr; }

int qmm_rt_buffer_increase_external_refs(qmm_rt_buffer* b) {
  QMM_REQUIRE(b != nullptr, QMM_ERR_INVALID_ARGUMENT, "null buffer");
  std::lock_guard<std::mutex> lock(b->mu);
  QMM_REQUIRE(!b->released, QMM_ERR_INVALID_ARGUMENT, "the buffer's storage is gone");
  ++b->external_refs;
  return QMM_OK;
}
int qmm_rt_buffer_decrease_external_refs(qmm_rt_buffer* b) {
  QMM_REQUIRE(b != nullptr, QMM_ERR_INVALID_ARGUMENT, "null buffer");
  std::lock_guard<std::mutex> lock(b->mu);
  QMM_REQUIRE(b->external_refs > 0, QMM_ERR_INVALID_ARGUMENT, "external reference count is already zero");
  if (--b->external_refs == 0 && b->deleted) release_storage(b);
  return QMM_OK;
}

// -------------------------------------------------------------- executable
int qmm_rt_client_compile(qmm_rt_client* c, const char* program, size_t size, const char* format,
                          qmm_rt_executable** out) {
  if (!c) c = qmm_rt_default_client();
  QMM_REQUIRE(c && program && out, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_client_compile: null argument");
  *out = nullptr;
  const std::string fmt = format ? format : "mlir";
  QMM_REQUIRE(fmt == "mlir", QMM_ERR_UNSUPPORTED,
              "program format '%s' is not supported: this backend compiles StableHLO (format \"mlir\")", fmt.c_str());
  if (size >= 4 && program[0] == 'M' && program[1] == 'L' && static_cast<unsigned char>(program[2]) == 0xEF &&
      program[3] == 'R')
    return set_error(QMM_ERR_UNSUPPORTED,
                     "the program is MLIR bytecode (a StableHLO portable artifact); this build has no MLIR reader, so "
                     "the plugin's Python side must deserialize the artifact and hand over its textual form");
  return make_executable(c, program, size, out);
}

int qmm_rt_executable_destroy(qmm_rt_executable* e) {
  if (!e) return QMM_OK;
  for (auto& kv : e->workspace) {
    cudaSetDevice(kv.first);
    qmm_rt_device* d = qmm_rt_client_device(e->client, kv.first);
    if (d && d->streams_ready) cudaStreamSynchronize(d->exec);  // a launch may still use it
    cudaFree(kv.second);
  }
  qmm_plan_destroy(e->plan);
  delete e;
  return QMM_OK;
}
int qmm_rt_executable_delete(qmm_rt_executable* e) {
  if (e) e->deleted.store(true);
  return QMM_OK;
}
int qmm_rt_executable_is_deleted(const qmm_rt_executable* e) { return (!e || e->deleted.load()) ? 1 : 0; }
const char* qmm_rt_executable_name(const qmm_rt_executable* e) { return e ? e->name.c_str() : ""; }
int qmm_rt_executable_num_replicas(const qmm_rt_executable* e) { return e ? qmm_plan_num_replicas(e->plan) : 0; }
int qmm_rt_executable_num_partitions(const qmm_rt_executable* e) { return e ? qmm_plan_num_partitions(e->plan) : 0; }
int qmm_rt_executable_num_outputs(const qmm_rt_executable* e) { return e ? static_cast<int>(e->outs.size()) : 0; }
int qmm_rt_executable_num_args(const qmm_rt_executable* e) { return e ? static_cast<int>(e->args.size()) : 0; }
int64_t qmm_rt_executable_code_size(const qmm_rt_executable* e) { return e ? static_cast<int64_t>(e->text.size()) : 0; }
const char* qmm_rt_executable_fingerprint(const qmm_rt_executable* e) { return e ? e->fingerprint.c_str() : ""; }
const char* qmm_rt_executable_program(const qmm_rt_executable* e, size_t* size) {
  if (size) *size = e ? e->text.size() : 0;
  return e ? e->text.c_str() : "";
}
static const qmm_rt_executable::TensorInfo* tinfo(const std::vector<qmm_rt_executable::TensorInfo>& v, int i) {
  return (i >= 0 && i < static_cast<int>(v.size())) ? &v[i] : nullptr;
}
int qmm_rt_executable_output_dtype(const qmm_rt_executable* e, int i) {
  auto* t = e ? tinfo(e->outs, i) : nullptr;
  return t ? t->dtype : -1;
}
int qmm_rt_executable_output_rank(const qmm_rt_executable* e, int i) {
  auto* t = e ? tinfo(e->outs, i) : nullptr;
  return t ? static_cast<int>(t->dims.size()) : -1;
}
const int64_t* qmm_rt_executable_output_dims(const qmm_rt_executable* e, int i) {
  auto* t = e ? tinfo(e->outs, i) : nullptr;
  return t ? t->dims.data() : nullptr;
}
const char* qmm_rt_executable_output_memory_kind(const qmm_rt_executable*, int) { return "device"; }
int qmm_rt_executable_arg_dtype(const qmm_rt_executable* e, int i) {
  auto* t = e ? tinfo(e->args, i) : nullptr;
  return t ? t->dtype : -1;
}
int qmm_rt_executable_arg_rank(const qmm_rt_executable* e, int i) {
  auto* t = e ? tinfo(e->args, i) : nullptr;
  return t ? static_cast<int>(t->dims.size()) : -1;
}
const int64_t* qmm_rt_executable_arg_dims(const qmm_rt_executable* e, int i) {
  auto* t = e ? tinfo(e->args, i) : nullptr;
  return t ? t->dims.data() : nullptr;
}
double qmm_rt_executable_flops(const qmm_rt_executable* e) { return e ? qmm_plan_flops(e->plan) : 0.0; }
size_t qmm_rt_executable_trace(const qmm_rt_executable* e, char* buf, size_t cap) {
  return e ? qmm_plan_trace(e->plan, buf, cap) : 0;
}
qmm_rt_client* qmm_rt_executable_client(const qmm_rt_executable* e) { return e ? e->client : nullptr; }

int qmm_rt_executable_serialize(const qmm_rt_executable* e, char** blob, size_t* size) {
  QMM_REQUIRE(e && blob && size, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_executable_serialize: null argument");
  const uint64_t n = e->text.size();
  const size_t total = 4 + 4 + 16 + 8 + e->text.size();
  char* p = static_cast<char*>(malloc(total));
  QMM_REQUIRE(p != nullptr, QMM_ERR_CUDA, "out of host memory");
  memcpy(p, kBlobMagic, 4);
  memcpy(p + 4, &kBlobVersion, 4);
  memcpy(p + 8, e->fingerprint.data(), 16);
  memcpy(p + 24, &n, 8);
  memcpy(p + 32, e->text.data(), e->text.size());
  *blob = p;
  *size = total;
  return QMM_OK;
}
void qmm_rt_serialized_free(char* blob) { free(blob); }
int qmm_rt_executable_deserialize_and_load(qmm_rt_client* c, const char* blob, size_t size, qmm_rt_executable** out) {
  if (!c) c = qmm_rt_default_client();
  QMM_REQUIRE(c && out, QMM_ERR_INVALID_ARGUMENT, "qmm_rt_executable_deserialize_and_load: null argument");
  *out = nullptr;
  QMM_REQUIRE(blob && size > 0, QMM_ERR_INVALID_ARGUMENT, "DeserializeAndLoad: empty serialized data");
  QMM_REQUIRE(size >= 32 && memcmp(blob, kBlobMagic, 4) == 0, QMM_ERR_INVALID_ARGUMENT,
              "DeserializeAndLoad: not a serialized executable of this library");
  uint32_t ver = 0;
  uint64_t n = 0;
  memcpy(&ver, blob + 4, 4);
  memcpy(&n, blob + 24, 8);
  QMM_REQUIRE(ver == kBlobVersion, QMM_ERR_UNSUPPORTED, "DeserializeAndLoad: blob version %u, this library reads %u", ver,
              kBlobVersion);
  QMM_REQUIRE(n == size - 32, QMM_ERR_INVALID_ARGUMENT, "DeserializeAndLoad: truncated blob");
  qmm_rt_executable* e = nullptr;
  if (int rc = make_executable(c, blob + 32, static_cast<size_t>(n), &e)) return rc;
  if (memcmp(e->fingerprint.data(), blob + 8, 16) != 0) {
    qmm_rt_executable_destroy(e);
    return set_error(QMM_ERR_INVALID_ARGUMENT, "DeserializeAndLoad: the program does not match its fingerprint");
  }
  *out = e;
  return QMM_OK;
}

int qmm_rt_executable_execute(qmm_rt_executable* e, qmm_rt_buffer* const* const* argument_lists, int num_devices,
                              int num_args, qmm_rt_buffer** const* output_lists, qmm_rt_event** device_complete_events) {
  QMM_REQUIRE(e != nullptr, QMM_ERR_INVALID_ARGUMENT, "No executable to execute");
  QMM_REQUIRE(!e->deleted.load(), QMM_ERR_INVALID_ARGUMENT, "the executable is deleted");
  QMM_REQUIRE(num_devices >= 1 && argument_lists && output_lists, QMM_ERR_INVALID_ARGUMENT,
              "qmm_rt_executable_execute: bad arguments");
  QMM_REQUIRE(num_args == static_cast<int>(e->args.size()), QMM_ERR_INVALID_ARGUMENT,
              "the program takes %zu arguments, %d were passed", e->args.size(), num_args);
  const int nout = static_cast<int>(e->outs.size());
  for (int d = 0; d < num_devices; ++d) {
    QMM_REQUIRE((num_args == 0 || argument_lists[d]) && output_lists[d], QMM_ERR_INVALID_ARGUMENT,
                "null argument or output list for device %d", d);
    qmm_rt_device* dev = num_args ? nullptr : qmm_rt_client_device(e->client, d);
    std::vector<const void*> args(num_args);
    for (int a = 0; a < num_args; ++a) {
      qmm_rt_buffer* b = argument_lists[d][a];
      QMM_REQUIRE(b != nullptr, QMM_ERR_INVALID_ARGUMENT, "argument %d of device list %d is null", a, d);
      QMM_REQUIRE(b->client == e->client, QMM_ERR_INVALID_ARGUMENT, "argument %d belongs to another client", a);
      if (!dev) dev = b->device;
      QMM_REQUIRE(b->device == dev, QMM_ERR_INVALID_ARGUMENT,
                  "argument %d of device list %d lives on device %d, the list's first argument on device %d", a, d,
                  b->device ? b->device->id : -1, dev ? dev->id : -1);
      const auto& want = e->args[a];
      QMM_REQUIRE(b->dtype == want.dtype && b->dims == want.dims, QMM_ERR_INVALID_ARGUMENT,
                  "argument %d does not have the element type and shape the program was compiled for", a);
    }
    QMM_REQUIRE(dev != nullptr, QMM_ERR_INVALID_ARGUMENT, "no device for list %d", d);
    if (int rc = device_ready(dev)) return rc;
    QMM_CUDA_TRY(cudaSetDevice(dev->ordinal));
    for (int a = 0; a < num_args; ++a) {
      qmm_rt_buffer* b = argument_lists[d][a];
      std::lock_guard<std::mutex> lock(b->mu);
      QMM_REQUIRE(!b->deleted && !b->released, QMM_ERR_INVALID_ARGUMENT, "argument %d is a deleted buffer", a);
      if (b->ready && b->ready->ready.load() && b->ready->status != QMM_OK)
        return set_error(b->ready->status, "argument %d is an error buffer: %s", a, b->ready->message.c_str());
      if (b->produced && b->produced->ev) QMM_CUDA_TRY(cudaStreamWaitEvent(dev->exec, b->produced->ev, 0));
      args[a] = b->ptr;
    }
    // scratch of the program on this device: allocated on first use, zeroed once (the kernels
    // leave it zeroed); launches of one executable on one device are ordered by the stream
    void* ws = nullptr;
    if (e->workspace_bytes) {
      std::lock_guard<std::mutex> lock(e->mu);
      auto it = e->workspace.find(dev->ordinal);
      if (it == e->workspace.end()) {
        QMM_CUDA_TRY(cudaMalloc(&ws, e->workspace_bytes));
        QMM_CUDA_TRY(cudaMemsetAsync(ws, 0, e->workspace_bytes, dev->exec));
        e->workspace[dev->ordinal] = ws;
      } else {
        ws = it->second;
      }
    }
    std::vector<qmm_rt_buffer*> outs(nout, nullptr);
    std::vector<void*> out_ptrs(nout, nullptr);
    int rc = QMM_OK;
    for (int o = 0; o < nout && rc == QMM_OK; ++o) {
      const auto& t = e->outs[o];
      rc = new_buffer(e->client, dev, t.dtype, t.dims.data(), static_cast<int>(t.dims.size()), &outs[o]);
      if (rc == QMM_OK) out_ptrs[o] = outs[o]->ptr;
    }
    if (rc == QMM_OK)
      rc = qmm_plan_execute(e->plan, args.data(), num_args, out_ptrs.data(), nout, ws, e->workspace_bytes, dev->exec);
    CudaEventRef ev;
    if (rc == QMM_OK) rc = record_event(dev, dev->exec, &ev);
    if (rc != QMM_OK) {
      for (auto* b : outs) qmm_rt_buffer_destroy(b);
      return rc;
    }
    auto done = std::make_shared<EventState>();
    EventRef d2 = done;
    if (after_stream(e->client, dev->exec, [d2] {
          // a device-side wait that gave up is recorded in the library's status word
          const int st = qmm_device_status();
          if (st != 0) d2->finish(QMM_ERR_TIMEOUT, "a kernel of this launch (or an earlier one) gave up waiting");
          else d2->finish(QMM_OK, "");
        }) != QMM_OK)
      done = make_ready_event();
    for (int o = 0; o < nout; ++o) {
      mark_produced(outs[o], ev, done);
      output_lists[d][o] = outs[o];
    }
    if (device_complete_events) device_complete_events[d] = new qmm_rt_event{done};
  }
  return QMM_OK;
}

}  // extern "C"

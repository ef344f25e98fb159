// Array runtime behind the DLArray C-ABI: pooled device / pinned-host memory,
// stream-ordered copies, opaque handles.  Replaces src/c_runtime_api.cc,
// src/cuda_device_api.cc and src/cpu_device_api.cc of the reference.
#include "common.h"
#include <stdarg.h>
#include <mutex>
#include <unordered_map>
#include <vector>
#include <chrono>
#include <string>

namespace tf {

static thread_local char t_err[512] = {0};
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof(t_err), fmt, ap);
  va_end(ap);
  static const bool verbose = getenv("TINYFLOW_VERBOSE") != nullptr;
  if (verbose) fprintf(stderr, "[tinyflow_b200] %s\n", t_err);
}

std::atomic<long long> g_launches{0};
bool g_sync_every_op = [] { const char* e = getenv("TINYFLOW_SYNC"); return e && e[0] == '1'; }();
int g_num_sms = 0;

int device_sm_count() {
  if (g_num_sms == 0) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0)
      g_num_sms = n;
    else
      g_num_sms = 148;
  }
  return g_num_sms;
}

int after_launch(cudaStream_t s, const char* what, int nkernels) {
  g_launches.fetch_add(nkernels, std::memory_order_relaxed);
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    cudaGetLastError();
    set_error("%s: launch failed: %s", what, cudaGetErrorString(e));
    return -1;
  }
  if (g_sync_every_op) {
    e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) { set_error("%s: %s", what, cudaGetErrorString(e)); return -1; }
  }
  return 0;
}

// ---- per-kernel timing registry ---------------------------------------------------------------
int g_timing_level = 0;
namespace {
struct Family { std::string name; double flops = 0, bytes = 0, ms = 0; long long launches = 0; };
struct PendingSpan { int family; cudaEvent_t a, b; };
std::mutex g_kt_mu;
std::vector<Family> g_families;
std::vector<PendingSpan> g_pending;
std::vector<cudaEvent_t> g_event_pool;
cudaEvent_t take_event() {
  if (!g_event_pool.empty()) { cudaEvent_t e = g_event_pool.back(); g_event_pool.pop_back(); return e; }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}
void resolve_pending_locked() {
  for (auto& p : g_pending) {
    float ms = 0.f;
    if (cudaEventSynchronize(p.b) == cudaSuccess && cudaEventElapsedTime(&ms, p.a, p.b) == cudaSuccess) g_families[p.family].ms += ms;
    g_event_pool.push_back(p.a);
    g_event_pool.push_back(p.b);
  }
  g_pending.clear();
}
}  // namespace
void KernelTimer::begin(const char* family, double flops, double bytes) {
  std::lock_guard<std::mutex> lk(g_kt_mu);
  int f = -1;
  for (size_t i = 0; i < g_families.size(); ++i) if (g_families[i].name == family) { f = (int)i; break; }
  if (f < 0) { g_families.push_back(Family{family}); f = (int)g_families.size() - 1; }
  g_families[f].flops += flops; g_families[f].bytes += bytes; g_families[f].launches += 1;
  PendingSpan p{f, take_event(), take_event()};
  cudaEventRecord(p.a, stream);
  g_pending.push_back(p);
  slot = (int)g_pending.size() - 1;
  if (g_pending.size() > 200000) { slot = -1; cudaEventRecord(p.b, stream); resolve_pending_locked(); }
}
void KernelTimer::end() {
  std::lock_guard<std::mutex> lk(g_kt_mu);
  if (slot >= 0 && slot < (int)g_pending.size()) cudaEventRecord(g_pending[slot].b, stream);
}

static std::atomic<cudaStream_t> g_compute_stream{(cudaStream_t)0};
void note_compute_stream(cudaStream_t s) { g_compute_stream.store(s, std::memory_order_relaxed); }
cudaStream_t last_compute_stream() { flush_deferred(); return g_compute_stream.load(std::memory_order_relaxed); }

// ---- the held-back elementwise call (see common.h) ----------------------------------------------
std::atomic<int> g_deferred_pending{0};
static std::mutex g_deferred_mu;
static DeferredOp g_deferred;
bool deferral_enabled() {
  static const bool on = [] {
    const char* e = getenv("TINYFLOW_DEFER");
    return (e ? atoi(e) != 0 : true) && getenv("TINYFLOW_SYNC") == nullptr;      // per-operator timing wants every operator launched in its own call
  }();
  return on;
}
void defer_op(const DeferredOp& op) {
  std::lock_guard<std::mutex> lk(g_deferred_mu);
  g_deferred = op;
  g_deferred_pending.store(1, std::memory_order_release);
}
// Both ways out of the slot keep the mutex until the kernel that replaces the held-back one is ENQUEUED, and the flag
// stays up until then: another thread (a swap worker about to copy the held-back call's output) that finds the flag up
// waits on the mutex and so cannot order its own work in front of that kernel.
bool take_deferred(int kind, const float* out, int64_t n, DeferredOp* op) {
  if (!g_deferred_pending.load(std::memory_order_acquire)) return false;
  g_deferred_mu.lock();
  if (!g_deferred_pending.load(std::memory_order_relaxed) || g_deferred.kind != kind || g_deferred.out != out || g_deferred.n != n) { g_deferred_mu.unlock(); return false; }
  *op = g_deferred;
  return true;        // still locked: the caller launches, then calls release_deferred()
}
void release_deferred() {
  g_deferred_pending.store(0, std::memory_order_release);
  g_deferred_mu.unlock();
}
// Freeing an array only concerns the held-back call if the array is one of its operands.
void flush_deferred_if_uses(const void* data) {
  if (!g_deferred_pending.load(std::memory_order_acquire)) return;
  std::lock_guard<std::mutex> lk(g_deferred_mu);
  if (!g_deferred_pending.load(std::memory_order_relaxed)) return;
  if (data != (const void*)g_deferred.a && data != (const void*)g_deferred.b && data != (const void*)g_deferred.out) return;
  launch_deferred_now(g_deferred);
  g_deferred_pending.store(0, std::memory_order_release);
}
void flush_deferred_slow() {
  std::lock_guard<std::mutex> lk(g_deferred_mu);
  if (!g_deferred_pending.load(std::memory_order_relaxed)) return;
  launch_deferred_now(g_deferred);      // a launch failure is recorded as the thread's last error and surfaces at the next synchronising call
  g_deferred_pending.store(0, std::memory_order_release);
}

// ---------------------------------------------------------------------------------
// Memory pools.  The executor allocates one array per graph node per step and drops
// them all at the start of the next step, so the same sizes recur every step: blocks
// are cached by exact (rounded) size and handed back without touching the driver.
// Reuse is safe without per-block events because (a) all compute is enqueued on one
// stream, and (b) copies on any other stream first wait for the compute stream's
// tail (see DLArrayCopyFromTo).  Once a process has shown that it swaps (a host-to-device
// copy on a side stream was seen), (b) is refined for those copies: every device block
// records an event on the compute stream when it is freed, and a side-stream copy INTO a
// recycled block waits for that event - the last possible reader of the block's previous
// contents - instead of for everything queued at the time of the call, so that a swap-in
// can run ahead of, and overlap with, the compute queued in front of its consumer.
// ---------------------------------------------------------------------------------
static std::atomic<bool> g_side_copies_seen{false};
struct Pool {
  std::mutex mu;
  std::unordered_map<size_t, std::vector<void*>> free_by_size;
  std::unordered_map<void*, size_t> size_of;   // every block we own, in use or cached
  struct Freed { cudaEvent_t ev = nullptr; int state = 0; };      // state 1: freed before events were kept, 2: ev marks the free
  std::unordered_map<void*, Freed> freed;      // device blocks that have been freed at least once
  long long in_use = 0, cached = 0;
  bool host;
  explicit Pool(bool h) : host(h) {}

  static size_t round(size_t b) {
    if (b < 512) return 512;
    if (b < (1u << 20)) return (b + 511) & ~size_t(511);
    return (b + (size_t(1) << 16) - 1) & ~((size_t(1) << 16) - 1);   // 64 KiB granules above 1 MiB
  }
  cudaError_t raw_alloc(void** p, size_t b) {
    return host ? cudaHostAlloc(p, b, cudaHostAllocDefault) : cudaMalloc(p, b);
  }
  void raw_free(void* p) { host ? cudaFreeHost(p) : cudaFree(p); }

  void release_cached_locked() {
    for (auto& kv : free_by_size) {
      for (void* p : kv.second) {
        auto f = freed.find(p);
        if (f != freed.end()) { if (f->second.ev) cudaEventDestroy(f->second.ev); freed.erase(f); }
        size_of.erase(p); raw_free(p);
      }
      kv.second.clear();
    }
    cached = 0;
  }
  // *hard (optional) is set when the allocation failed for a reason other than running out of memory (the context is
  // unusable, e.g. after a kernel fault): the caller reports an error instead of the out-of-memory protocol.  The
  // flag describes this call only.
  void* alloc(size_t bytes, bool* hard = nullptr) {
    if (hard) *hard = false;
    size_t b = round(bytes);
    std::lock_guard<std::mutex> lk(mu);
    auto it = free_by_size.find(b);
    if (it != free_by_size.end() && !it->second.empty()) {
      void* p = it->second.back();
      it->second.pop_back();
      cached -= (long long)b;
      in_use += (long long)b;
      return p;
    }
    void* p = nullptr;
    cudaError_t e = raw_alloc(&p, b);
    if (e != cudaSuccess && e != cudaErrorMemoryAllocation) {
      // not an out-of-memory condition: the context is unusable (an earlier kernel faulted)
      if (hard) *hard = true;
      set_error("device allocation failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    if (e != cudaSuccess) {
      cudaGetLastError();
      // Give cached blocks back to the driver and try once more before reporting OOM.
      if (!host) cudaDeviceSynchronize();
      release_cached_locked();
      e = raw_alloc(&p, b);
      if (e != cudaSuccess) { cudaGetLastError(); return nullptr; }
    }
    size_of[p] = b;
    in_use += (long long)b;
    return p;
  }
  bool free(void* p) {
    std::lock_guard<std::mutex> lk(mu);
    auto it = size_of.find(p);
    if (it == size_of.end()) return false;
    if (!host) {
      Freed& f = freed[p];
      f.state = 1;
      if (g_side_copies_seen.load(std::memory_order_relaxed)) {
        if (!f.ev && cudaEventCreateWithFlags(&f.ev, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); f.ev = nullptr; }
        if (f.ev && cudaEventRecord(f.ev, g_compute_stream.load(std::memory_order_relaxed)) == cudaSuccess) f.state = 2;
        else cudaGetLastError();
      }
    }
    free_by_size[it->second].push_back(p);
    in_use -= (long long)it->second;
    cached += (long long)it->second;
    return true;
  }
  // Orders stream s after the last use of block p's previous contents.  0: done (fresh block, or waited on the event of
  // its last free); 1: not known to this pool, or freed without an event - the caller falls back to the compute tail.
  int order_after_last_use(void* p, cudaStream_t s) {
    std::lock_guard<std::mutex> lk(mu);
    if (size_of.find(p) == size_of.end()) return 1;
    auto f = freed.find(p);
    if (f == freed.end()) return 0;                       // never freed: nothing was ever queued on it before this owner
    if (f->second.state != 2) return 1;
    if (cudaStreamWaitEvent(s, f->second.ev, 0) != cudaSuccess) { cudaGetLastError(); return 1; }
    return 0;
  }
};

// One device pool per GPU (a cached block is only ever handed out on the device it was allocated on); pinned host
// memory is not tied to a device.
constexpr int kMaxDevices = 64;
static Pool* g_device_pools[kMaxDevices] = {nullptr};
static std::mutex g_device_pools_mu;
static Pool& device_pool(int dev) {
  std::lock_guard<std::mutex> lk(g_device_pools_mu);
  if (dev < 0 || dev >= kMaxDevices) dev = 0;
  if (!g_device_pools[dev]) g_device_pools[dev] = new Pool(false);
  return *g_device_pools[dev];
}
static int current_device() { int dev = 0; if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); dev = 0; } return dev; }
static Pool& device_pool() { return device_pool(current_device()); }
static Pool& host_pool() { static Pool* p = new Pool(true); return *p; }

void* pool_alloc(size_t bytes) { return device_pool().alloc(bytes); }
void pool_free(void* p) {
  if (!p) return;
  if (device_pool().free(p)) return;
  for (int d = 0; d < kMaxDevices; ++d) {                                      // freed while another device is current
    Pool* other;
    { std::lock_guard<std::mutex> lk(g_device_pools_mu); other = g_device_pools[d]; }
    if (other && other->free(p)) return;
  }
}

void* persistent_scratch(int slot, size_t bytes) {
  static std::mutex mu;
  static void* ptr[16] = {nullptr};
  static size_t cap[16] = {0};
  std::lock_guard<std::mutex> lk(mu);
  if (slot < 0 || slot >= 16) return nullptr;
  if (cap[slot] >= bytes) return ptr[slot];
  // Growing while earlier kernels may still read the old block: hand the old block back
  // to the pool (stream order on the single compute stream keeps that safe).
  if (ptr[slot]) pool_free(ptr[slot]);
  size_t want = bytes + bytes / 4;
  ptr[slot] = pool_alloc(want);
  cap[slot] = ptr[slot] ? Pool::round(want) : 0;
  return ptr[slot];
}

static inline size_t data_bytes(const DLArray* a) { return (size_t)numel(a) * 4; }

}  // namespace tf

namespace tf { int tensor_path_error(); int dp_flush_if_pending(); }
using namespace tf;

extern "C" {

// src/c_runtime_api.cc:93 — element size is 4 bytes; a failed device allocation is
// reported through *memorytoSaving with return value 0 and *out left untouched.
int DLArrayAlloc(const index_t* shape, index_t ndim_in, DLContext ctx, DLArrayHandle* out,
                 int* memorytoSaving) {
  int ndim = (int)ndim_in;   // ctypes passes a 32-bit int; ignore the upper half of the register
  TF_REQUIRE(shape && out && ndim >= 0 && ndim <= 8, "DLArrayAlloc: bad arguments (ndim=%d)", ndim);
  size_t n = 1;
  for (int i = 0; i < ndim; ++i) {
    TF_REQUIRE(shape[i] >= 0, "DLArrayAlloc: negative extent");
    TF_REQUIRE(shape[i] == 0 || n <= (SIZE_MAX / 4) / (size_t)shape[i], "DLArrayAlloc: the array's byte size overflows");
    n *= (size_t)shape[i];
  }
  size_t bytes = n * 4;
  void* data = nullptr;
  bool hard = false;
  if (ctx.device_type == kGPU) {
    TF_REQUIRE(ctx.device_id >= 0 && ctx.device_id < kMaxDevices, "DLArrayAlloc: device id %d out of range", ctx.device_id);
    if (cudaSetDevice(ctx.device_id) != cudaSuccess) { cudaGetLastError(); TF_FAIL("DLArrayAlloc: cudaSetDevice(%d) failed", ctx.device_id); }
    data = device_pool(ctx.device_id).alloc(bytes, &hard);
  } else if (ctx.device_type == kCPU) {
    data = host_pool().alloc(bytes, &hard);     // pinned, as src/cpu_device_api.cc:18
  } else {
    TF_FAIL("DLArrayAlloc: unknown device type %d", (int)ctx.device_type);
  }
  if (!data && hard) return -1;          // not out of memory: this call hit an unusable context (message already set)
  if (!data) {
    if (memorytoSaving) *memorytoSaving = bytes > 0x7fffffffu ? 0x7fffffff : (int)bytes;
    return 0;
  }
  DLArray* arr = new DLArray;
  arr->data = data;
  arr->ctx = ctx;
  arr->ndim = ndim;
  arr->shape = new int64_t[ndim > 0 ? ndim : 1];
  for (int i = 0; i < ndim; ++i) arr->shape[i] = shape[i];
  *out = arr;
  return 0;
}

// src/c_runtime_api.cc:121
int DLArrayFree(DLArrayHandle handle) {
  if (!handle) return 0;
  flush_deferred_if_uses(handle->data);      // a held-back kernel may read or write this array
  if (handle->data) {
    if (handle->ctx.device_type == kGPU) note_write(handle->data);   // a recycled block is new data
    bool ok = (handle->ctx.device_type == kGPU) ? device_pool(handle->ctx.device_id).free(handle->data)
                                                : host_pool().free(handle->data);
    if (!ok) TF_FAIL("DLArrayFree: array was not allocated by DLArrayAlloc");
  }
  delete[] handle->shape;
  delete handle;
  return 0;
}

// src/c_runtime_api.cc:128 — `stream` is NULL (blocking copy) or the address of a cell
// holding a cudaStream_t (asynchronous copy, then synchronise that stream only).
int DLArrayCopyFromTo(DLArrayHandle from, DLArrayHandle to, DLStreamHandle stream) {
  flush_deferred();
  TF_REQUIRE(from && to && from->data && to->data, "DLArrayCopyFromTo: null array");
  size_t bytes = data_bytes(from);
  TF_REQUIRE(bytes == data_bytes(to), "DLArrayCopyFromTo: size mismatch (%zu vs %zu bytes)", bytes, data_bytes(to));
  const bool fg = from->ctx.device_type == kGPU, tg = to->ctx.device_type == kGPU;
  if (!fg && !tg) { memcpy(to->data, from->data, bytes); return 0; }
  TF_CUDA(cudaSetDevice(fg ? from->ctx.device_id : to->ctx.device_id));
  cudaMemcpyKind kind = fg && tg ? cudaMemcpyDeviceToDevice : (fg ? cudaMemcpyDeviceToHost : cudaMemcpyHostToDevice);
  if (bytes == 0) return 0;
  if (tg) note_write(to->data);
  if (stream == nullptr) {
    // A blocking copy between host and device is how a training loop uploads its next batch and reads its loss: in
    // data-parallel mode that is the step boundary, so pending gradient buckets are sent and waited for (on the device).
    if (fg != tg && dp_flush_if_pending() != 0) return -1;
    // Blocking copy on the legacy default stream: ordered after everything already
    // enqueued on the (blocking) compute streams, and complete on return.
    TF_CUDA(cudaMemcpy(to->data, from->data, bytes, kind));
    return 0;
  }
  cudaStream_t s = *(cudaStream_t*)stream;
  cudaStream_t cs = last_compute_stream();
  bool ordered = false;
  if (s != cs && tg && !fg) {
    // Swap-in: the destination is a pool block nobody reads yet; what has to be over is the last use of the block's
    // PREVIOUS contents, which the pool marked with an event when the block was freed.
    g_side_copies_seen.store(true, std::memory_order_relaxed);
    ordered = device_pool(to->ctx.device_id).order_after_last_use(to->data, s) == 0;
  }
  if (s != cs && !ordered) {
    // A side stream (swap traffic): order the copy after the compute enqueued so far, so a
    // tensor being swapped out is fully written and a recycled block is no longer read.
    static thread_local cudaEvent_t ev = nullptr;
    if (!ev) TF_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    TF_CUDA(cudaEventRecord(ev, cs));
    TF_CUDA(cudaStreamWaitEvent(s, ev, 0));
  }
  TF_CUDA(cudaMemcpyAsync(to->data, from->data, bytes, kind, s));
  if (kind == cudaMemcpyDeviceToDevice && s == cs) return 0;   // same-stream reshape copy: no host wait needed
  TF_CUDA(cudaStreamSynchronize(s));
  return 0;
}

int DLGpuCreatecudaStream(void** cudaStream) {
  TF_REQUIRE(cudaStream, "null cell");
  cudaStream_t s;
  TF_CUDA(cudaStreamCreate(&s));       // blocking stream: orders against legacy-default-stream copies
  *cudaStream = (void*)s;
  return 0;
}
int DLGpuDestroycudaStream(void** cudaStream) {
  TF_REQUIRE(cudaStream, "null cell");
  cudaStream_t s = (cudaStream_t)*cudaStream;
  if (last_compute_stream() == s) note_compute_stream(0);
  TF_CUDA(cudaStreamSynchronize(s));
  TF_CUDA(cudaStreamDestroy(s));
  *cudaStream = nullptr;
  return 0;
}

// The "cudnn" and "cublas" handles of the reference carry a stream binding only; here the
// handle is a small library-owned record of the stream cell's value.
struct LibHandle { int magic; cudaStream_t stream; };
static int make_handle(void** cell, void** cudaStream) {
  TF_REQUIRE(cell, "null cell");
  LibHandle* h = new LibHandle{0x7f5a, stream_of(cudaStream)};
  *cell = h;
  return 0;
}
static int drop_handle(void** cell) {
  TF_REQUIRE(cell, "null cell");
  LibHandle* h = (LibHandle*)*cell;
  if (h && h->magic == 0x7f5a) { h->magic = 0; delete h; }
  *cell = nullptr;
  return 0;
}
int DLGpuCreatecudnnHandle(void** cudnnHandle, void** cudaStream) { return make_handle(cudnnHandle, cudaStream); }
int DLGpuDestroycudnnHandle(void** cudnnHandle) { return drop_handle(cudnnHandle); }
int DLGpuCreatecublasHandle(void** cublasHandle, void** cudaStream) { return make_handle(cublasHandle, cudaStream); }
int DLGpuDestroycublasHandle(void** cublasHandle) { return drop_handle(cublasHandle); }

int getInt(int* intp) { return intp ? *intp : 0; }

// src/gpu_op.cu:4960 — host-link bandwidth probe, pageable vs pinned, both directions.
int testPcie(void) {
  const size_t bytes = size_t(256) << 20;
  void *dev = nullptr, *pinned = nullptr;
  void* pageable = malloc(bytes);
  if (!pageable) TF_FAIL("testPcie: malloc failed");
  memset(pageable, 1, bytes);
  if (cudaMalloc(&dev, bytes) != cudaSuccess || cudaHostAlloc(&pinned, bytes, cudaHostAllocDefault) != cudaSuccess) {
    cudaGetLastError(); free(pageable); if (dev) cudaFree(dev);
    TF_FAIL("testPcie: allocation failed");
  }
  memset(pinned, 1, bytes);
  auto run = [&](void* dst, const void* src, cudaMemcpyKind k) {
    cudaMemcpy(dst, src, bytes, k);   // warm-up
    auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < 4; ++i) cudaMemcpy(dst, src, bytes, k);
    cudaDeviceSynchronize();
    double s = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    return 4.0 * bytes / s / 1e9;
  };
  double a = run(dev, pageable, cudaMemcpyHostToDevice), b = run(pageable, dev, cudaMemcpyDeviceToHost);
  double c = run(dev, pinned, cudaMemcpyHostToDevice), d = run(pinned, dev, cudaMemcpyDeviceToHost);
  printf("host link GB/s: pageable H2D %.2f D2H %.2f | pinned H2D %.2f D2H %.2f\n", a, b, c, d);
  fflush(stdout);
  cudaFree(dev); cudaFreeHost(pinned); free(pageable);
  return 0;
}

// Per-kernel timing: enable (level 1 = contractions, 2 = all instrumented kernels; resets the table),
// then read a JSON array of {name, launches, ms, flops, bytes} rows.
int TfKernelTimingEnable(int level) {
  std::lock_guard<std::mutex> lk(g_kt_mu);
  resolve_pending_locked();
  if (level > 0) g_families.clear();
  g_timing_level = level;
  return 0;
}
int TfKernelTimingReport(char* buf, int buflen) {
  std::lock_guard<std::mutex> lk(g_kt_mu);
  resolve_pending_locked();
  std::string out = "[";
  char row[512];
  for (size_t i = 0; i < g_families.size(); ++i) {
    const Family& f = g_families[i];
    snprintf(row, sizeof(row), "%s{\"name\": \"%s\", \"launches\": %lld, \"ms\": %.6f, \"flops\": %.6e, \"bytes\": %.6e}", i ? ", " : "", f.name.c_str(), f.launches, f.ms, f.flops, f.bytes);
    out += row;
  }
  out += "]";
  if (!buf || buflen <= (int)out.size()) TF_FAIL("TfKernelTimingReport: buffer too small (%zu bytes needed)", out.size() + 1);
  memcpy(buf, out.c_str(), out.size() + 1);
  return 0;
}

int TfDeviceSynchronize(void) {
  flush_deferred();
  TF_CUDA(cudaDeviceSynchronize());
  TF_REQUIRE(tensor_path_error() == 0, "a tensor-core kernel timed out waiting on a barrier (results of that launch are invalid)");
  return 0;
}
int TfLaunchCount(long long* count) { if (count) *count = g_launches.load(); return 0; }
int TfLastError(char* buf, int buflen) {
  if (buf && buflen > 0) { strncpy(buf, t_err, buflen - 1); buf[buflen - 1] = 0; }
  return 0;
}
int TfAllocatorStats(long long* bytes_in_use, long long* bytes_cached) {
  Pool& p = device_pool();
  std::lock_guard<std::mutex> lk(p.mu);
  if (bytes_in_use) *bytes_in_use = p.in_use;
  if (bytes_cached) *bytes_cached = p.cached;
  return 0;
}
int TfReleaseCachedMemory(void) {
  cudaDeviceSynchronize();
  { Pool& p = device_pool(); std::lock_guard<std::mutex> lk(p.mu); p.release_cached_locked(); }
  { Pool& p = host_pool(); std::lock_guard<std::mutex> lk(p.mu); p.release_cached_locked(); }
  return 0;
}

}  // extern "C"

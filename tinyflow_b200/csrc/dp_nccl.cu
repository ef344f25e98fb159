// Data-parallel gradient exchange for one box: one process per GPU, NCCL over NVLink / NVSwitch.
//
// The reference has no distributed layer; the only places the library sees "this gradient is final" are the
// optimiser entry points, so that is where the exchange hooks in.  After TfDpInit:
//
//   DLGpuSgdUpdate(w, g, lr)        copies the gradient into the current bucket (compute stream) and records
//                                   {w, offset, count, lr}.
//   DLGpuAdam_mv(m, v, g, b1, b2)   same, recording the moment tensors; the DLGpuAdam(w, m, v, ...) call that
//   + DLGpuAdam(w, m, v, ...)       follows it (autodiff.py:2063-2070) completes the record with the parameter
//                                   and the step constants.  (The reference's executor is Adam-only.)
//
// A full bucket is handed to the communication stream: ONE all-reduce (sum) in place, then ONE kernel that applies
// every update of the bucket with the mean gradient (SGD: w -= lr/world * sum; Adam: moments, then the step).  The
// compute stream carries on with the rest of the backward pass meanwhile (optimiser nodes are interleaved with
// backward nodes by the executor, last layer first, so buckets fill while earlier layers still compute).
// From the second step on the library knows how many gradient bytes a step produces and closes the open bucket
// early once all but a small tail has arrived, so the all-reduce that cannot overlap anything (it follows the last
// backward kernel) moves a few megabytes at most.
//
//   TfDpFlush        sends the last, partly filled bucket and makes the compute stream wait (on the device, no host
//                    block) for every outstanding update, so the next forward pass reads updated weights.  A
//                    host-to-device or device-to-host DLArrayCopyFromTo flushes as well: a driver that knows
//                    nothing of this layer (the reference's executor) uploads its next batch through that call.
//
// Buckets form a small ring; a bucket is reused only after the event that marks its update as applied.
// A gradient larger than a bucket is reduced in place on its own.  NCCL is loaded with dlopen, so the
// library has no link-time dependency on it and single-GPU users never touch it.
//
// Failures.  Every host wait here is bounded: the rendezvous on the id file (TINYFLOW_DP_INIT_TIMEOUT_S, default
// 120 s), and, after each hand-off, a poll of ncclCommGetAsyncError; when a collective does not finish within
// TINYFLOW_DP_TIMEOUT_S (default 300 s, checked at TfDpFlush / TfDpShutdown) or NCCL reports an asynchronous error,
// the communicator is aborted (ncclCommAbort) and the call returns -1.
#include "common.h"
#include <dlfcn.h>
#include <unistd.h>
#include <chrono>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace tf {

// ---- minimal NCCL surface (types as in nccl.h) ---------------------------------------------------
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclFloat32 = 7, ncclSum = 0, ncclSuccess = 0, ncclInProgress = 7 };
struct NcclApi {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
};
static NcclApi g_nccl;

static int load_nccl() {
  if (g_nccl.lib) return 0;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  for (const char* n : names) { g_nccl.lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (g_nccl.lib) break; }
  TF_REQUIRE(g_nccl.lib, "TfDpInit: libnccl.so.2 not found (%s)", dlerror());
  g_nccl.GetUniqueId = (decltype(g_nccl.GetUniqueId))dlsym(g_nccl.lib, "ncclGetUniqueId");
  g_nccl.CommInitRank = (decltype(g_nccl.CommInitRank))dlsym(g_nccl.lib, "ncclCommInitRank");
  g_nccl.AllReduce = (decltype(g_nccl.AllReduce))dlsym(g_nccl.lib, "ncclAllReduce");
  g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy))dlsym(g_nccl.lib, "ncclCommDestroy");
  g_nccl.CommAbort = (decltype(g_nccl.CommAbort))dlsym(g_nccl.lib, "ncclCommAbort");
  g_nccl.CommGetAsyncError = (decltype(g_nccl.CommGetAsyncError))dlsym(g_nccl.lib, "ncclCommGetAsyncError");
  g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))dlsym(g_nccl.lib, "ncclGetErrorString");
  TF_REQUIRE(g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.AllReduce && g_nccl.CommDestroy, "TfDpInit: NCCL symbols missing");
  return 0;
}
#define TF_NCCL(expr) do { ncclResult_t _r = (expr); if (_r != 0) TF_FAIL("%s failed: %s", #expr, g_nccl.GetErrorString ? g_nccl.GetErrorString(_r) : "?"); } while (0)

static double env_seconds(const char* name, double dflt) {
  const char* e = getenv(name);
  if (!e) return dflt;
  double v = atof(e);
  return v > 0 ? v : dflt;
}

// ---- bucket planning (pure host logic, also exported for CPU tests) -------------------------------
// Walks tensors in arrival order; a tensor joins the open bucket if it fits, else closes it and opens a
// new one; a tensor larger than the capacity gets a bucket of its own (id marked negative: -(id+1)).
int plan_buckets(const long long* counts, int n, long long capacity, int* bucket_of) {
  int id = 0;
  long long fill = 0;
  for (int i = 0; i < n; ++i) {
    if (counts[i] > capacity) {
      if (fill > 0) { ++id; fill = 0; }
      bucket_of[i] = -(id + 1);
      ++id;
      continue;
    }
    if (fill + counts[i] > capacity) { ++id; fill = 0; }
    bucket_of[i] = id;
    fill += counts[i];
  }
  return fill > 0 ? id + 1 : id;
}
// The same walk with the early close: `step_total` floats arrive per step (0 = unknown yet); once all but `tail` of
// them have arrived the open bucket is closed, once per step, so the last bucket holds at most about `tail` floats.
int plan_buckets_tail(const long long* counts, int n, long long capacity, long long step_total, long long tail, int* bucket_of) {
  int id = 0;
  long long fill = 0, arrived = 0;
  bool closed_early = false;
  for (int i = 0; i < n; ++i) {
    if (counts[i] > capacity) {
      if (fill > 0) { ++id; fill = 0; }
      bucket_of[i] = -(id + 1);
      ++id;
      arrived += counts[i];
      continue;
    }
    if (fill + counts[i] > capacity) { ++id; fill = 0; }
    bucket_of[i] = id;
    fill += counts[i];
    arrived += counts[i];
    if (!closed_early && step_total > 0 && step_total - arrived <= tail && fill > 0 && arrived < step_total) { ++id; fill = 0; closed_early = true; }
  }
  return fill > 0 ? id + 1 : id;
}

// ---- state ----------------------------------------------------------------------------------------
enum { kSgd = 0, kAdam = 1 };
struct Entry {
  int kind;
  float* w; float* m; float* v;       // Adam: w stays null until DLGpuAdam names it
  long long offset, count;
  float lr, b1, b2, c1, c2, eps;
};
struct Bucket {
  float* buf = nullptr;
  long long fill = 0;
  std::vector<Entry> entries;
  cudaEvent_t applied = nullptr;      // recorded on the comm stream after the bucket's updates
  bool in_flight = false;
};
struct DpState {
  bool on = false;
  int rank = 0, world = 1;
  ncclComm_t comm = nullptr;
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ready = nullptr;        // compute stream -> comm stream hand-off
  long long capacity = 0;             // floats per bucket
  long long tail_floats = 0;          // early close: target size of the step's last bucket
  long long step_total = 0;           // floats of gradient per step, learned from the first step
  long long step_arrived = 0;
  bool closed_early = false;
  std::vector<Bucket> ring;
  int cur = 0;
  std::mutex mu;
  long long bytes_reduced = 0, allreduces = 0, apply_launches = 0, early_closes = 0;
  bool failed = false;
};
static DpState g_dp;

__global__ void __launch_bounds__(256) dp_copy_kernel(const float* __restrict__ g, float* __restrict__ dst, long long n) {
  grid_dep_sync();
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = g[i];
}

// Every update of one bucket in one launch.  Each entry owns a run of consecutive blocks (first_block .. first_block +
// blocks); the largest |w| written is recorded per entry for the tensor path's operand scaling (the next forward
// pass packs w).
constexpr int kApplyEntries = 24;
struct ApplyEntry {
  float* w; float* m; float* v;
  const float* sum;
  long long count;
  float lr, b1, b2, c1, c2, eps;
  int kind, first_block, blocks;
  AmaxOut am;
};
struct ApplyTable { int n; float inv_world; ApplyEntry e[kApplyEntries]; };
__global__ void __launch_bounds__(256) dp_apply_kernel(const __grid_constant__ ApplyTable t) {
  int idx = 0;
  while (idx + 1 < t.n && (int)blockIdx.x >= t.e[idx + 1].first_block) ++idx;
  const ApplyEntry& e = t.e[idx];
  const int local = blockIdx.x - e.first_block;
  const long long stride = (long long)e.blocks * blockDim.x;
  uint32_t mx = 0;
  if (e.kind == kSgd) {
    const float scale = e.lr * t.inv_world;
    for (long long i = (long long)local * blockDim.x + threadIdx.x; i < e.count; i += stride) {
      float v = e.w[i] - scale * e.sum[i];
      e.w[i] = v;
      mx = max(mx, amax_bits(v));
    }
  } else {
    for (long long i = (long long)local * blockDim.x + threadIdx.x; i < e.count; i += stride) {
      const float gi = e.sum[i] * t.inv_world;
      const float mi = e.m[i] * e.b1 + gi * (1.f - e.b1);
      const float vi = e.v[i] * e.b2 + gi * gi * (1.f - e.b2);
      e.m[i] = mi; e.v[i] = vi;
      if (e.w) {
        float w = e.w[i] - e.lr * mi / e.c1 / (sqrtf(vi / e.c2) + e.eps);
        e.w[i] = w;
        mx = max(mx, amax_bits(w));
      }
    }
  }
  if (!e.am.word) return;                                   // uniform over the entry's blocks
  __shared__ uint32_t red[8];
  const int lane = threadIdx.x & 31, wp = threadIdx.x >> 5;
  mx = __reduce_max_sync(0xffffffffu, mx);
  if (lane == 0) red[wp] = mx;
  __syncthreads();
  if (wp == 0) {
    uint32_t r = lane < 8 ? red[lane] : 0u;
    r = __reduce_max_sync(0xffffffffu, r);
    if (lane == 0 && r) atomicMax(e.am.word, r);
  }
  if (local == 0 && threadIdx.x == 0 && e.am.clear) *e.am.clear = 0u;
}

static int poll_async_error(const char* where) {
  if (!g_nccl.CommGetAsyncError || !g_dp.comm) return 0;
  ncclResult_t st = ncclSuccess;
  if (g_nccl.CommGetAsyncError(g_dp.comm, &st) != ncclSuccess) return 0;
  if (st == ncclSuccess || st == ncclInProgress) return 0;
  g_dp.failed = true;
  if (g_nccl.CommAbort) g_nccl.CommAbort(g_dp.comm);
  g_dp.comm = nullptr;
  TF_FAIL("%s: NCCL reported an asynchronous error (%s); the communicator was aborted", where, g_nccl.GetErrorString ? g_nccl.GetErrorString(st) : "?");
}
// Host wait with a limit for everything queued on the communication stream.
static int wait_comm_stream(const char* where) {
  const double limit = env_seconds("TINYFLOW_DP_TIMEOUT_S", 300.0);
  auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    cudaError_t q = cudaStreamQuery(g_dp.comm_stream);
    if (q == cudaSuccess) return 0;
    if (q != cudaErrorNotReady) { cudaGetLastError(); TF_FAIL("%s: the communication stream failed: %s", where, cudaGetErrorString(q)); }
    if (poll_async_error(where)) return -1;
    if (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > limit) {
      g_dp.failed = true;
      if (g_nccl.CommAbort && g_dp.comm) g_nccl.CommAbort(g_dp.comm);
      g_dp.comm = nullptr;
      TF_FAIL("%s: a collective did not finish within %.0f s (a peer is gone?); the communicator was aborted", where, limit);
    }
    std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
}

// Launches the updates of `entries` (which read their sums from `base`) on the comm stream.
static int launch_apply(const std::vector<Entry>& entries, const float* base) {
  for (size_t first = 0; first < entries.size(); first += kApplyEntries) {
    ApplyTable t;
    memset(&t, 0, sizeof(t));
    t.inv_world = 1.f / (float)g_dp.world;
    int blocks = 0;
    const size_t last = std::min(entries.size(), first + kApplyEntries);
    for (size_t i = first; i < last; ++i) {
      const Entry& e = entries[i];
      ApplyEntry& a = t.e[t.n++];
      a.w = e.w; a.m = e.m; a.v = e.v; a.sum = base + e.offset; a.count = e.count;
      a.lr = e.lr; a.b1 = e.b1; a.b2 = e.b2; a.c1 = e.c1; a.c2 = e.c2; a.eps = e.eps; a.kind = e.kind;
      long long nb = (e.count + 256 * 8 - 1) / (256 * 8);
      a.blocks = (int)(nb < 1 ? 1 : (nb > 128 ? 128 : nb));
      a.first_block = blocks;
      blocks += a.blocks;
      if (e.w) { note_write(e.w); a.am = amax_track_begin(e.w); }
      if (e.kind == kAdam) { note_write(e.m); note_write(e.v); }
    }
    dp_apply_kernel<<<blocks, 256, 0, g_dp.comm_stream>>>(t);
    g_dp.apply_launches += 1;
    if (after_launch(g_dp.comm_stream, "dp_apply", 1) != 0) return -1;
  }
  return 0;
}

// Hands bucket b to the comm stream: all-reduce, apply every entry, mark applied.
static int send_bucket(Bucket& b, cudaStream_t compute) {
  if (b.fill == 0) return 0;
  TF_REQUIRE(!g_dp.failed && g_dp.comm, "data-parallel exchange: the communicator has failed");
  TF_CUDA(cudaEventRecord(g_dp.ready, compute));
  TF_CUDA(cudaStreamWaitEvent(g_dp.comm_stream, g_dp.ready, 0));
  TF_NCCL(g_nccl.AllReduce(b.buf, b.buf, (size_t)b.fill, ncclFloat32, ncclSum, g_dp.comm, g_dp.comm_stream));
  g_dp.bytes_reduced += b.fill * 4; g_dp.allreduces += 1;
  if (launch_apply(b.entries, b.buf)) return -1;
  TF_CUDA(cudaEventRecord(b.applied, g_dp.comm_stream));
  b.in_flight = true;
  b.entries.clear();
  b.fill = 0;
  return poll_async_error("data-parallel exchange");
}

// Takes one gradient: into the open bucket, or (larger than a bucket) reduced in place with the compute stream waiting.
static int take_gradient(const Entry& proto, const float* g, int64_t n, cudaStream_t s) {
  g_dp.step_arrived += n;
  if (n > g_dp.capacity) {
    // larger than a bucket: close the open bucket, then reduce this gradient in place; the compute stream waits
    // for it, because the caller may recycle the gradient's memory right after this call returns
    if (send_bucket(g_dp.ring[g_dp.cur], s)) return -1;
    g_dp.cur = (g_dp.cur + 1) % (int)g_dp.ring.size();
    TF_REQUIRE(!g_dp.failed && g_dp.comm, "data-parallel exchange: the communicator has failed");
    TF_CUDA(cudaEventRecord(g_dp.ready, s));
    TF_CUDA(cudaStreamWaitEvent(g_dp.comm_stream, g_dp.ready, 0));
    TF_NCCL(g_nccl.AllReduce(g, (void*)g, (size_t)n, ncclFloat32, ncclSum, g_dp.comm, g_dp.comm_stream));
    g_dp.bytes_reduced += n * 4; g_dp.allreduces += 1;
    Entry e = proto;
    e.offset = 0; e.count = n;
    if (e.kind == kAdam) {
      // the step constants arrive with the DLGpuAdam call that follows: only the moments are updated here, the
      // parameter update then runs as usual on the compute stream (w = null)
      e.w = nullptr;
    }
    std::vector<Entry> one(1, e);
    if (launch_apply(one, g)) return -1;
    TF_CUDA(cudaEventRecord(g_dp.ready, g_dp.comm_stream));
    TF_CUDA(cudaStreamWaitEvent(s, g_dp.ready, 0));
    return 1;
  }
  Bucket* b = &g_dp.ring[g_dp.cur];
  if (b->fill + n > g_dp.capacity) {
    if (send_bucket(*b, s)) return -1;
    g_dp.cur = (g_dp.cur + 1) % (int)g_dp.ring.size();
    b = &g_dp.ring[g_dp.cur];
  }
  if (b->in_flight) {      // the ring wrapped: this bucket's previous contents must have been applied
    TF_CUDA(cudaStreamWaitEvent(s, b->applied, 0));
    b->in_flight = false;
  }
  launch_dep(dp_copy_kernel, dim3(grid_for(n, 256, 4)), dim3(256), 0, s, g, b->buf + b->fill, n);
  if (after_launch(s, "dp_copy", 1) != 0) return -1;
  Entry e = proto;
  e.offset = b->fill; e.count = n;
  b->entries.push_back(e);
  b->fill += (n + 3) & ~3ll;       // keep every tensor 16-byte aligned inside the bucket
  return 1;
}
// Early close: all but the tail of the step's gradients have arrived.  Never for an Adam record whose parameter has not
// been named yet (the caller checks).
static int maybe_close_early(cudaStream_t s) {
  if (g_dp.closed_early || g_dp.step_total <= 0 || g_dp.tail_floats <= 0) return 0;
  if (g_dp.step_arrived >= g_dp.step_total || g_dp.step_total - g_dp.step_arrived > g_dp.tail_floats) return 0;
  Bucket& b = g_dp.ring[g_dp.cur];
  if (b.fill == 0) return 0;
  g_dp.closed_early = true;
  g_dp.early_closes += 1;
  if (send_bucket(b, s)) return -1;
  g_dp.cur = (g_dp.cur + 1) % (int)g_dp.ring.size();
  return 0;
}

// Returns 1 when the update was taken over, 0 when data-parallel mode is off, -1 on error.
int dp_sgd_update(float* w, const float* g, int64_t n, float lr, cudaStream_t s) {
  if (!g_dp.on) return 0;
  std::lock_guard<std::mutex> lk(g_dp.mu);
  Entry e{};
  e.kind = kSgd; e.w = w; e.lr = lr;
  int rc = take_gradient(e, g, n, s);
  if (rc < 0) return -1;
  if (maybe_close_early(s)) return -1;
  return 1;
}
// Adam, first call of the pair: the gradient is final.  Returns like dp_sgd_update.
int dp_adam_moments(float* m, float* v, const float* g, int64_t n, float b1, float b2, cudaStream_t s) {
  if (!g_dp.on) return 0;
  std::lock_guard<std::mutex> lk(g_dp.mu);
  Entry e{};
  e.kind = kAdam; e.m = m; e.v = v; e.b1 = b1; e.b2 = b2;
  return take_gradient(e, g, n, s) < 0 ? -1 : 1;
}
// Adam, second call of the pair.  Returns 1 when the parameter update was attached to the pending record of (m, v)
// - it then runs after the all-reduce - and 0 when there is none (data-parallel mode off, or a gradient larger than a
// bucket, whose moments are already final on the compute stream): the caller then updates the parameter itself.
int dp_adam_step(float* w, const float* m, const float* v, float c1, float c2, float eps, float lr, cudaStream_t s) {
  if (!g_dp.on) return 0;
  std::lock_guard<std::mutex> lk(g_dp.mu);
  Bucket& b = g_dp.ring[g_dp.cur];
  for (auto it = b.entries.rbegin(); it != b.entries.rend(); ++it) {
    if (it->kind == kAdam && it->m == m && it->v == v && !it->w) {
      it->w = w; it->c1 = c1; it->c2 = c2; it->eps = eps; it->lr = lr;
      if (maybe_close_early(s)) return -1;
      return 1;
    }
  }
  return 0;
}
// End of a step as far as the exchange is concerned: sends what is pending and makes `s` wait for every update.
int dp_flush(cudaStream_t s) {
  if (!g_dp.on) return 0;
  std::lock_guard<std::mutex> lk(g_dp.mu);
  if (g_dp.step_arrived > 0) {                 // a step's worth of gradients went by: remember its size for the early close
    g_dp.step_total = g_dp.step_arrived;
    g_dp.step_arrived = 0;
    g_dp.closed_early = false;
  }
  if (send_bucket(g_dp.ring[g_dp.cur], s)) return -1;
  g_dp.cur = (g_dp.cur + 1) % (int)g_dp.ring.size();
  for (Bucket& b : g_dp.ring) {
    if (b.in_flight) { TF_CUDA(cudaStreamWaitEvent(s, b.applied, 0)); b.in_flight = false; }
  }
  return 0;
}
// Called by host<->device copies: a step boundary for drivers that do not call TfDpFlush.
int dp_flush_if_pending() {
  if (!g_dp.on) return 0;
  bool pending;
  {
    std::lock_guard<std::mutex> lk(g_dp.mu);
    pending = g_dp.step_arrived > 0;
    for (const Bucket& b : g_dp.ring) pending = pending || b.in_flight || b.fill > 0;
  }
  return pending ? dp_flush(last_compute_stream()) : 0;
}

}  // namespace tf

using namespace tf;

extern "C" {

// Pure host helper (no device needed): bucket id per tensor for the given sizes (in floats) and capacity.
int TfDpPlanBuckets(const long long* counts, int n, long long capacity_floats, int* bucket_of) {
  TF_REQUIRE(counts && bucket_of && n >= 0 && capacity_floats > 0, "TfDpPlanBuckets: bad arguments");
  return plan_buckets(counts, n, capacity_floats, bucket_of);
}
// The same with the early close of the last-but-one bucket (step_total_floats = 0: first step, size not known yet).
int TfDpPlanBucketsTail(const long long* counts, int n, long long capacity_floats, long long step_total_floats, long long tail_floats, int* bucket_of) {
  TF_REQUIRE(counts && bucket_of && n >= 0 && capacity_floats > 0 && tail_floats >= 0, "TfDpPlanBucketsTail: bad arguments");
  return plan_buckets_tail(counts, n, capacity_floats, step_total_floats, tail_floats, bucket_of);
}

// Rendezvous on a file: rank 0 writes {magic, nonce, NCCL id}; a stale file from a crashed run is removed first, and the
// other ranks accept a file only if it is complete and younger than the moment they started waiting minus a minute.
struct IdFile { unsigned long long magic, nonce; ncclUniqueId id; };
int TfDpInit(int rank, int world_size, const char* nccl_id_path) {
  TF_REQUIRE(world_size >= 1 && rank >= 0 && rank < world_size && nccl_id_path, "TfDpInit: bad arguments");
  TF_REQUIRE(!g_dp.on, "TfDpInit: already initialised");
  const unsigned long long kMagic = 0x74666470'6e63636cull;
  std::string path(nccl_id_path), tmp = path + ".tmp";
  IdFile idf;
  memset(&idf, 0, sizeof(idf));
  const double limit = env_seconds("TINYFLOW_DP_INIT_TIMEOUT_S", 120.0);
  if (rank == 0) {
    if (load_nccl()) return -1;
    unlink(path.c_str());                            // whatever a crashed run left behind
    TF_NCCL(g_nccl.GetUniqueId(&idf.id));
    idf.magic = kMagic;
    idf.nonce = (unsigned long long)std::chrono::duration_cast<std::chrono::seconds>(std::chrono::system_clock::now().time_since_epoch()).count();
    FILE* f = fopen(tmp.c_str(), "wb");
    TF_REQUIRE(f, "TfDpInit: cannot write %s", tmp.c_str());
    size_t put = fwrite(&idf, sizeof(idf), 1, f);
    fclose(f);
    TF_REQUIRE(put == 1 && rename(tmp.c_str(), path.c_str()) == 0, "TfDpInit: cannot publish %s", path.c_str());
  } else {
    const unsigned long long started = (unsigned long long)std::chrono::duration_cast<std::chrono::seconds>(std::chrono::system_clock::now().time_since_epoch()).count();
    auto t0 = std::chrono::steady_clock::now();
    for (;;) {      // bounded wait for rank 0's id file
      FILE* f = fopen(path.c_str(), "rb");
      if (f) {
        size_t got = fread(&idf, sizeof(idf), 1, f);
        fclose(f);
        if (got == 1 && idf.magic == kMagic && idf.nonce + 60 >= started) break;
      }
      TF_REQUIRE(std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() < limit, "TfDpInit: timed out after %.1f s waiting for %s", limit,
                 path.c_str());
      std::this_thread::sleep_for(std::chrono::milliseconds(20));
    }
    if (load_nccl()) return -1;
  }
  // NCCL's kernels share the SMs with the backward pass: keep their footprint small unless the user chose otherwise
  setenv("NCCL_MAX_CTAS", "8", 0);
  ncclResult_t r = g_nccl.CommInitRank(&g_dp.comm, world_size, idf.id, rank);
  if (rank == 0) unlink(path.c_str());               // every rank has the id once CommInitRank returned
  if (r != 0) { g_dp.comm = nullptr; TF_FAIL("ncclCommInitRank failed: %s", g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "?"); }
  auto fail = [&](const char* what) {
    for (Bucket& b : g_dp.ring) { if (b.buf) pool_free(b.buf); if (b.applied) cudaEventDestroy(b.applied); }
    g_dp.ring.clear();
    if (g_dp.ready) { cudaEventDestroy(g_dp.ready); g_dp.ready = nullptr; }
    if (g_dp.comm_stream) { cudaStreamDestroy(g_dp.comm_stream); g_dp.comm_stream = nullptr; }
    if (g_dp.comm) { g_nccl.CommDestroy(g_dp.comm); g_dp.comm = nullptr; }
    set_error("TfDpInit: %s", what);
    return -1;
  };
  int lo = 0, hi = 0;
  cudaDeviceGetStreamPriorityRange(&lo, &hi);        // hi is the numerically smallest = highest priority
  if (cudaStreamCreateWithPriority(&g_dp.comm_stream, cudaStreamNonBlocking, hi) != cudaSuccess) { cudaGetLastError(); return fail("cannot create the communication stream"); }
  if (cudaEventCreateWithFlags(&g_dp.ready, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); return fail("cannot create an event"); }
  const char* mb = getenv("TINYFLOW_BUCKET_MB");
  long long bucket_mb = mb ? atoll(mb) : 32;
  if (bucket_mb < 1) bucket_mb = 1;
  g_dp.capacity = bucket_mb * 1024 * 1024 / 4;
  const char* tail = getenv("TINYFLOW_DP_TAIL_MB");
  g_dp.tail_floats = (long long)((tail ? atof(tail) : 2.0) * 1024 * 1024 / 4);
  g_dp.ring.resize(4);
  for (Bucket& b : g_dp.ring) {
    b.buf = (float*)pool_alloc((size_t)g_dp.capacity * 4);
    if (!b.buf) return fail("bucket allocation failed");
    if (cudaEventCreateWithFlags(&b.applied, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); return fail("cannot create an event"); }
  }
  g_dp.rank = rank; g_dp.world = world_size; g_dp.cur = 0; g_dp.on = true; g_dp.failed = false;
  g_dp.step_total = g_dp.step_arrived = 0; g_dp.closed_early = false;
  return 0;
}

int TfDpFlush(void** cudaStream) {
  if (!g_dp.on) return 0;
  if (dp_flush(stream_of(cudaStream))) return -1;
  std::lock_guard<std::mutex> lk(g_dp.mu);
  return poll_async_error("TfDpFlush");
}

// bytes all-reduced and number of all-reduces since TfDpInit
int TfDpStats(long long* bytes_reduced, long long* allreduces) {
  if (bytes_reduced) *bytes_reduced = g_dp.bytes_reduced;
  if (allreduces) *allreduces = g_dp.allreduces;
  return 0;
}
// the same plus the update launches on the communication stream and how often a bucket was closed early
int TfDpStats2(long long* bytes_reduced, long long* allreduces, long long* apply_launches, long long* early_closes) {
  TfDpStats(bytes_reduced, allreduces);
  if (apply_launches) *apply_launches = g_dp.apply_launches;
  if (early_closes) *early_closes = g_dp.early_closes;
  return 0;
}

int TfDpShutdown(void) {
  if (!g_dp.on) return 0;
  int rc = 0;
  if (!g_dp.failed) rc = wait_comm_stream("TfDpShutdown");
  for (Bucket& b : g_dp.ring) { pool_free(b.buf); cudaEventDestroy(b.applied); }
  g_dp.ring.clear();
  if (g_dp.comm) g_nccl.CommDestroy(g_dp.comm);
  g_dp.comm = nullptr;
  cudaEventDestroy(g_dp.ready);
  cudaStreamDestroy(g_dp.comm_stream);
  g_dp.ready = nullptr; g_dp.comm_stream = nullptr;
  g_dp.on = false;
  return rc;
}

}  // extern "C"

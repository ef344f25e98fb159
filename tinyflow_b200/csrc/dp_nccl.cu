// Data-parallel gradient exchange for one box: one process per GPU, NCCL over NVLink / NVSwitch.
//
// The reference has no distributed layer; the only place the library sees "this gradient is final" is
// DLGpuSgdUpdate(param, grad, lr), so that is where the exchange hooks in.  After TfDpInit:
//
//   DLGpuSgdUpdate   copies the gradient into the current bucket (compute stream) and records
//                    {param, offset, count, lr}.  When the bucket is full it is handed to the
//                    communication stream: all-reduce (sum) in place, then  w -= (lr / world) * sum
//                    for every tensor of the bucket.  The compute stream carries on with the rest of
//                    the backward pass meanwhile (optimiser nodes are interleaved with backward nodes by
//                    the executor, last layer first, so buckets fill while earlier layers still compute).
//   TfDpFlush        sends the last, partly filled bucket and makes the compute stream wait (on the
//                    device, no host block) for every outstanding update, so the next forward pass reads
//                    updated weights.
//
// Buckets form a small ring; a bucket is reused only after the event that marks its update as applied.
// A gradient larger than a bucket is reduced in place on its own.  NCCL is loaded with dlopen, so the
// library has no link-time dependency on it and single-GPU users never touch it.
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
enum { ncclFloat32 = 7, ncclSum = 0 };
struct NcclApi {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
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
  g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))dlsym(g_nccl.lib, "ncclGetErrorString");
  TF_REQUIRE(g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.AllReduce && g_nccl.CommDestroy, "TfDpInit: NCCL symbols missing");
  return 0;
}
#define TF_NCCL(expr) do { ncclResult_t _r = (expr); if (_r != 0) TF_FAIL("%s failed: %s", #expr, g_nccl.GetErrorString ? g_nccl.GetErrorString(_r) : "?"); } while (0)

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

// ---- state ----------------------------------------------------------------------------------------
struct Entry { float* w; long long offset, count; float lr; };
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
  std::vector<Bucket> ring;
  int cur = 0;
  std::mutex mu;
  long long bytes_reduced = 0, allreduces = 0;
};
static DpState g_dp;

__global__ void __launch_bounds__(256) dp_copy_kernel(const float* __restrict__ g, float* __restrict__ dst, long long n) {
  grid_dep_sync();
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = g[i];
}
// w -= scale * sum, and max|w| of the result for the tensor path's operand scaling (the next forward pass packs w)
__global__ void __launch_bounds__(256) dp_apply_kernel(float* __restrict__ w, const float* __restrict__ sum, long long n, float scale, AmaxOut am) {
  long long stride = (long long)gridDim.x * blockDim.x;
  uint32_t m = 0;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float v = w[i] - scale * sum[i];
    w[i] = v;
    m = max(m, amax_bits(v));
  }
  amax_commit(am, m);
}

// Hands bucket b to the comm stream: all-reduce, apply every entry, mark applied.
static int send_bucket(Bucket& b, cudaStream_t compute) {
  if (b.fill == 0) return 0;
  TF_CUDA(cudaEventRecord(g_dp.ready, compute));
  TF_CUDA(cudaStreamWaitEvent(g_dp.comm_stream, g_dp.ready, 0));
  TF_NCCL(g_nccl.AllReduce(b.buf, b.buf, (size_t)b.fill, ncclFloat32, ncclSum, g_dp.comm, g_dp.comm_stream));
  g_dp.bytes_reduced += b.fill * 4; g_dp.allreduces += 1;
  for (const Entry& e : b.entries) {
    note_write(e.w);
    dp_apply_kernel<<<grid_for(e.count, 256, 4), 256, 0, g_dp.comm_stream>>>(e.w, b.buf + e.offset, e.count, e.lr / (float)g_dp.world, amax_track_begin(e.w));
  }
  if (after_launch(g_dp.comm_stream, "dp_apply", (int)b.entries.size()) != 0) return -1;
  TF_CUDA(cudaEventRecord(b.applied, g_dp.comm_stream));
  b.in_flight = true;
  b.entries.clear();
  b.fill = 0;
  return 0;
}

// Returns 1 when the update was taken over, 0 when data-parallel mode is off, -1 on error.
int dp_sgd_update(float* w, const float* g, int64_t n, float lr, cudaStream_t s) {
  if (!g_dp.on) return 0;
  std::lock_guard<std::mutex> lk(g_dp.mu);
  if (n > g_dp.capacity) {
    // larger than a bucket: close the open bucket, then reduce this gradient in place; the compute stream waits
    // for it, because the caller may recycle the gradient's memory right after this call returns
    if (send_bucket(g_dp.ring[g_dp.cur], s)) return -1;
    g_dp.cur = (g_dp.cur + 1) % (int)g_dp.ring.size();
    TF_CUDA(cudaEventRecord(g_dp.ready, s));
    TF_CUDA(cudaStreamWaitEvent(g_dp.comm_stream, g_dp.ready, 0));
    TF_NCCL(g_nccl.AllReduce(g, (void*)g, (size_t)n, ncclFloat32, ncclSum, g_dp.comm, g_dp.comm_stream));
    g_dp.bytes_reduced += n * 4; g_dp.allreduces += 1;
    note_write(w);
    dp_apply_kernel<<<grid_for(n, 256, 4), 256, 0, g_dp.comm_stream>>>(w, g, n, lr / (float)g_dp.world, amax_track_begin(w));
    if (after_launch(g_dp.comm_stream, "dp_apply", 1) != 0) return -1;
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
  b->entries.push_back(Entry{w, b->fill, (long long)n, lr});
  b->fill += (n + 3) & ~3ll;       // keep every tensor 16-byte aligned inside the bucket
  return 1;
}

}  // namespace tf

using namespace tf;

extern "C" {

// Pure host helper (no device needed): bucket id per tensor for the given sizes (in floats) and capacity.
int TfDpPlanBuckets(const long long* counts, int n, long long capacity_floats, int* bucket_of) {
  TF_REQUIRE(counts && bucket_of && n >= 0 && capacity_floats > 0, "TfDpPlanBuckets: bad arguments");
  return plan_buckets(counts, n, capacity_floats, bucket_of);
}

int TfDpInit(int rank, int world_size, const char* nccl_id_path) {
  TF_REQUIRE(world_size >= 1 && rank >= 0 && rank < world_size && nccl_id_path, "TfDpInit: bad arguments");
  TF_REQUIRE(!g_dp.on, "TfDpInit: already initialised");
  if (load_nccl()) return -1;
  ncclUniqueId id;
  std::string path(nccl_id_path), tmp = path + ".tmp";
  if (rank == 0) {
    TF_NCCL(g_nccl.GetUniqueId(&id));
    FILE* f = fopen(tmp.c_str(), "wb");
    TF_REQUIRE(f, "TfDpInit: cannot write %s", tmp.c_str());
    fwrite(&id, sizeof(id), 1, f);
    fclose(f);
    TF_REQUIRE(rename(tmp.c_str(), path.c_str()) == 0, "TfDpInit: rename to %s failed", path.c_str());
  } else {
    auto t0 = std::chrono::steady_clock::now();
    for (;;) {      // bounded wait for rank 0's id file
      FILE* f = fopen(path.c_str(), "rb");
      if (f) { size_t got = fread(&id, sizeof(id), 1, f); fclose(f); if (got == 1) break; }
      TF_REQUIRE(std::chrono::steady_clock::now() - t0 < std::chrono::seconds(120), "TfDpInit: timed out waiting for %s", path.c_str());
      std::this_thread::sleep_for(std::chrono::milliseconds(20));
    }
  }
  TF_NCCL(g_nccl.CommInitRank(&g_dp.comm, world_size, id, rank));
  if (rank == 0) { /* every rank has the id once CommInitRank returned */ unlink(path.c_str()); }
  TF_CUDA(cudaStreamCreateWithFlags(&g_dp.comm_stream, cudaStreamNonBlocking));
  TF_CUDA(cudaEventCreateWithFlags(&g_dp.ready, cudaEventDisableTiming));
  const char* mb = getenv("TINYFLOW_BUCKET_MB");
  long long bucket_mb = mb ? atoll(mb) : 32;
  if (bucket_mb < 1) bucket_mb = 1;
  g_dp.capacity = bucket_mb * 1024 * 1024 / 4;
  g_dp.ring.resize(4);
  for (Bucket& b : g_dp.ring) {
    b.buf = (float*)pool_alloc((size_t)g_dp.capacity * 4);
    TF_REQUIRE(b.buf, "TfDpInit: bucket allocation failed");
    TF_CUDA(cudaEventCreateWithFlags(&b.applied, cudaEventDisableTiming));
  }
  g_dp.rank = rank; g_dp.world = world_size; g_dp.cur = 0; g_dp.on = true;
  return 0;
}

int TfDpFlush(void** cudaStream) {
  if (!g_dp.on) return 0;
  std::lock_guard<std::mutex> lk(g_dp.mu);
  cudaStream_t s = stream_of(cudaStream);
  if (send_bucket(g_dp.ring[g_dp.cur], s)) return -1;
  g_dp.cur = (g_dp.cur + 1) % (int)g_dp.ring.size();
  for (Bucket& b : g_dp.ring) {
    if (b.in_flight) { TF_CUDA(cudaStreamWaitEvent(s, b.applied, 0)); b.in_flight = false; }
  }
  return 0;
}

int TfDpStats(long long* bytes_reduced, long long* allreduces) {
  if (bytes_reduced) *bytes_reduced = g_dp.bytes_reduced;
  if (allreduces) *allreduces = g_dp.allreduces;
  return 0;
}

int TfDpShutdown(void) {
  if (!g_dp.on) return 0;
  cudaStreamSynchronize(g_dp.comm_stream);
  for (Bucket& b : g_dp.ring) { pool_free(b.buf); cudaEventDestroy(b.applied); }
  g_dp.ring.clear();
  g_nccl.CommDestroy(g_dp.comm);
  cudaEventDestroy(g_dp.ready);
  cudaStreamDestroy(g_dp.comm_stream);
  g_dp.on = false;
  return 0;
}

}  // extern "C"

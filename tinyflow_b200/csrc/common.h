// Shared host/device helpers for the sm_100a operator library.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <atomic>
#include "../../include/c_runtime_api.h"

namespace tf {

// ---- error reporting (never abort; entry points return -1) -----------------
void set_error(const char* fmt, ...);
#define TF_FAIL(...) do { ::tf::set_error(__VA_ARGS__); return -1; } while (0)
#define TF_REQUIRE(cond, ...) do { if (!(cond)) TF_FAIL(__VA_ARGS__); } while (0)
#define TF_CUDA(expr) do { cudaError_t _e = (expr); if (_e != cudaSuccess) \
    TF_FAIL("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); } while (0)

// ---- launch accounting -------------------------------------------------------
extern std::atomic<long long> g_launches;
extern bool g_sync_every_op;          // TINYFLOW_SYNC=1
extern int g_num_sms;                 // streaming multiprocessors of the current device
int device_sm_count();

// Post-launch hook: counts the launch, surfaces launch errors, optional sync.
int after_launch(cudaStream_t s, const char* what, int nkernels = 1);
#define TF_AFTER(s, what) do { if (::tf::after_launch((s), (what)) != 0) return -1; } while (0)

// ---- optional per-kernel device timing (CUDA events on the launching stream) ------------
// Off by default.  Level 1 times the dense contractions only, level 2 every instrumented kernel.
// Construct before the launch; the destructor records the closing event.
extern int g_timing_level;
struct KernelTimer {
  int slot = -1;
  cudaStream_t stream;
  KernelTimer(const char* family, cudaStream_t s, double flops, double bytes, int level = 2) : stream(s) {
    if (g_timing_level >= level) begin(family, flops, bytes);
  }
  ~KernelTimer() { if (slot >= 0) end(); }
  void begin(const char* family, double flops, double bytes);
  void end();
};

// ---- streams ------------------------------------------------------------------
// The caller's cell holds a cudaStream_t.  A null cell means the legacy default stream.
// ---- an elementwise call held back for one call ----------------------------------------------
// Two operators do not launch at once; their arguments wait in a one-entry slot:
//  * DLGpuActivationBackward(relu): if the very next call into the library is the per-activation batch-norm backward that
//    consumes the ReLU's gradient, ONE kernel computes both (reads x and dy once, writes both gradients);
//  * DLGpuMatrixElementwiseAdd: if the very next call is the ReLU forward of the sum (the end of a residual block), ONE
//    kernel writes the sum and its ReLU.
// Every other way into the library - stream_of(), which every operator with a stream argument calls first,
// last_compute_stream(), which the stream-less operators and the copies call, the array free, the synchronising calls -
// launches the held-back kernel first (flush_deferred), so no caller can observe the difference.  One slot, guarded by
// a mutex; the fast path is one relaxed load.
enum { kDeferReluBwd = 1, kDeferAdd = 2 };
struct DeferredOp { int kind; const float* a; const float* b; float* out; int64_t n; cudaStream_t stream; };   // relu-bwd: a = the ReLU's input (mask), b = dy
extern std::atomic<int> g_deferred_pending;
void flush_deferred_slow();
inline void flush_deferred() { if (g_deferred_pending.load(std::memory_order_relaxed)) flush_deferred_slow(); }
void flush_deferred_if_uses(const void* data);                  // the array free: only if `data` is an operand of the held-back call
void defer_op(const DeferredOp& op);                            // the slot must be empty (flush first)
bool take_deferred(int kind, const float* out, int64_t n, DeferredOp* op);   // the held-back op if it is of this kind and writes `out`; on true the slot stays locked ...
void release_deferred();                                        // ... until the caller has enqueued the replacement and calls this
bool deferral_enabled();
int launch_deferred_now(const DeferredOp& op);                  // the plain elementwise kernel, now
long long fused_relu_bn_bwd_count();
long long fused_add_relu_count();

inline cudaStream_t stream_of(void** cell) { flush_deferred(); return cell ? (cudaStream_t)(*cell) : (cudaStream_t)0; }
inline cudaStream_t stream_of_keep_deferred(void** cell) { return cell ? (cudaStream_t)(*cell) : (cudaStream_t)0; }
void note_compute_stream(cudaStream_t s);   // remembered so side-stream copies can order after compute
cudaStream_t last_compute_stream();         // launches a held-back kernel first

// ---- write versions -------------------------------------------------------------
// Every entry point that writes a device array bumps the version of its data pointer; cached
// derived data (packed tensor-core operands) is valid only while the version is unchanged.
void note_write(const void* p);
uint64_t version_of(const void* p);
inline float* out_f32(DLArray* a) { note_write(a->data); return (float*)a->data; }

// ---- largest magnitude of a tensor, tracked by its producer ---------------------------
// The tensor path scales each operand by a power of two chosen from max|x|.  Kernels that write a whole tensor
// can fold that maximum into their pass: the launcher asks for a pair of device words after bumping the write
// version (amax_track_begin), the kernel ends with amax_commit(), and the consumer gets the word back through
// amax_tracked() for as long as nobody else wrote the tensor.  The two words of a tensor alternate between
// writes (the kernel of write k clears the word write k+1 will use), so no clearing launch is needed.
struct AmaxOut { uint32_t* word = nullptr; uint32_t* clear = nullptr; };
AmaxOut amax_track_begin(const void* data);
const uint32_t* amax_tracked(const void* data);
#ifdef __CUDACC__
__device__ __forceinline__ uint32_t amax_bits(float v) { return __float_as_uint(fabsf(v)); }
// Every thread of the block calls this once, after its last store, with the largest bit pattern it produced.
__device__ __forceinline__ void amax_commit(const AmaxOut& am, uint32_t m) {
  if (!am.word) return;                                  // uniform over the grid
  __shared__ uint32_t amax_red[32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  m = __reduce_max_sync(0xffffffffu, m);
  if (lane == 0) amax_red[w] = m;
  __syncthreads();
  if (w == 0) {
    uint32_t t = lane < nw ? amax_red[lane] : 0u;
    t = __reduce_max_sync(0xffffffffu, t);
    if (lane == 0 && t) atomicMax(am.word, t);
  }
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0 && am.clear) *am.clear = 0u;
}
#endif

// ---- producers that feed the tensor path ------------------------------------------------------------
// y = relu(x) fused with the packing of y for the convolution expected to read it (see gemm_tcgen05.cu); 1 = done,
// 0 = not applicable (run the plain kernel), -1 = error.
int tc_fused_relu_pack(const void* node, const float* x, float* y, int64_t n, cudaStream_t s);
void tc_note_relu_output(const void* node, const void* y);     // the plain ReLU of graph node `node` wrote y (after the version bump)
bool contraction_path_is_cuda_cores();

// ---- shapes -------------------------------------------------------------------
inline int64_t numel(const DLArray* a) {
  int64_t n = 1;
  for (int i = 0; i < a->ndim; ++i) n *= a->shape[i];
  return n;
}
inline bool same_shape(const DLArray* a, const DLArray* b) {
  if (a->ndim != b->ndim) return false;
  for (int i = 0; i < a->ndim; ++i) if (a->shape[i] != b->shape[i]) return false;
  return true;
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- device memory pool (thread-safe, size-class caching) --------------------
// Returns nullptr when the device is out of memory even after the cache was released.
void* pool_alloc(size_t bytes);
void pool_free(void* p);
// Scratch buffers that live as long as the library (grown on demand, never shrunk);
// slot ids are per purpose so concurrent purposes do not collide.
void* persistent_scratch(int slot, size_t bytes);

// ---- grid sizing: whole multiples of the SM count -----------------------------
inline int grid_for(int64_t work_items, int block, int per_thread = 1, int waves = 8) {
  int64_t need = (work_items + (int64_t)block * per_thread - 1) / ((int64_t)block * per_thread);
  if (need < 1) need = 1;
  int64_t cap = (int64_t)device_sm_count() * waves;
  if (need > cap) need = cap;                       // grid-stride loop covers the rest
  else if (need > device_sm_count()) {              // round up to a multiple of the SM count
    int sms = device_sm_count();
    need = (need + sms - 1) / sms * sms;
  }
  return (int)need;
}

// ---- programmatic dependent launch ---------------------------------------------------------
// A kernel launched through launch_dep() may be scheduled while the kernel in front of it on the stream is still
// draining; its first statement has to be grid_dep_sync(), which blocks until that kernel has completed and its
// writes are visible, and then lets the kernel behind start the same way.  Removes the launch gap between the
// ~700 short kernels of a step; a kernel launched with <<<>>> serialises as usual.
#ifdef __CUDACC__
__device__ __forceinline__ void grid_dep_sync() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
template <class... Params, class... Args>
inline cudaError_t launch_dep(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  static const bool off = getenv("TINYFLOW_NO_DEPENDENT_LAUNCH") != nullptr;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute attr;
  memset(&attr, 0, sizeof(attr));
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr; cfg.numAttrs = (off || s == (cudaStream_t)0) ? 0 : 1;      // the legacy default stream keeps plain stream order
  return cudaLaunchKernelEx(&cfg, kernel, Params(args)...);
}
#endif

// ---- plan structs stored in slot 0 of a descriptor list ----------------------
enum PlanKind : int { kPlanConv = 0x7f01, kPlanPool, kPlanAct, kPlanReduce, kPlanBN, kPlanTensor, kPlanDropout };

struct ConvPlan {
  int kind;
  int N, C, H, W;        // input
  int K, R, S;           // filter: K output channels, R x S window
  int P, Q;              // output spatial
  int pad_h, pad_w, stride_h, stride_w;
  int dataformat;
  void* tc_state;        // tensor-core path cache (packed operands, tensor maps)
};
struct PoolPlan {
  int kind;
  int N, C, H, W, P, Q;
  int mode;              // 0 max, 1 average (divisor includes padding)
  int pad_h, pad_w, stride_h, stride_w, win_h, win_w;
  int dataformat;
  // max pooling: first-maximum index per output, written by forward and reused by backward while the
  // input tensor (pointer + write version) is unchanged
  int32_t* argmax;
  const void* argmax_src;
  uint64_t argmax_version;
};
struct TensorPlan {      // activation / dropout input descriptor
  int kind;
  int ndim;
  int dims[5];
  int dataformat;
  int mode;
  int64_t batch, inner;  // batch = dims[0], inner = product of the rest
};
struct ReducePlan {
  int kind;
  int ndim;
  int in_dims[5];
  int out_dims[5];
};
struct BNPlan {
  int kind;
  int mode;              // 0 per-activation, 1 spatial
  int64_t N, C, HW;      // spatial: stats per C over N*HW; per-activation: stats per C*HW over N
  float* save_mean;      // library-owned, sized to the statistic count
  float* save_inv;
  int64_t nstat;
  const float* last_y;   // output of the last forward call and its write version: a ReLU gradient whose mask tensor is
  uint64_t last_y_version;   // still exactly that output can take its mask from x-hat instead of reading the tensor
};
struct DropoutState {
  int kind;
  float p;
  unsigned long long seed;
  int64_t count;
};

template <class T> T* plan_of(void*** cell, int kind) {
  if (!cell || !*cell) return nullptr;
  T* p = reinterpret_cast<T*>((*cell)[0]);
  if (!p || p->kind != kind) return nullptr;
  return p;
}
// Allocates the slot array the reference allocates (so a caller that frees it stays valid).
template <class T> T* new_plan(void*** cell, int kind, int slots) {
  void** arr = (void**)calloc(slots < 1 ? 1 : slots, sizeof(void*));
  T* p = (T*)calloc(1, sizeof(T));
  p->kind = kind;
  arr[0] = p;
  *cell = arr;
  return p;
}

}  // namespace tf

// HBM-bound operators: fill, broadcast, reductions, elementwise arithmetic, activations,
// softmax / losses, concat, dropout and the optimisers.  All fp32.  Every kernel moves
// 128-bit vectors when the pointers allow it, sizes its grid in multiples of the SM count
// and reduces with warp shuffles.
#include "common.h"
#include <math.h>

namespace tf {

constexpr int kBlock = 256;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Sum over a block of up to 1024 threads; result valid in every thread.
__device__ __forceinline__ float block_sum(float v, float* red /* >= 33 floats */) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// ---- generic vectorised map kernels ---------------------------------------------
// Functors whose outputs become operands of the tensor path (activations, their gradients, weights) carry a
// `kTrackAmax` member: only their launches reduce max|y| on the side.
template <class F, class = void> struct TracksAmax { static constexpr bool value = false; };
template <class F> struct TracksAmax<F, decltype((void)F::kTrackAmax)> { static constexpr bool value = F::kTrackAmax; };
__device__ __forceinline__ uint32_t amax4(uint32_t m, const float4& r) {
  return max(max(m, amax_bits(r.x)), max(amax_bits(r.y), max(amax_bits(r.z), amax_bits(r.w))));
}
template <class F> __global__ void __launch_bounds__(kBlock) map1_kernel(const float* __restrict__ a, float* __restrict__ o, int64_t n, F f, AmaxOut am) {
  grid_dep_sync();
  int64_t nv = n >> 2, stride = (int64_t)gridDim.x * blockDim.x;
  const float4* a4 = reinterpret_cast<const float4*>(a);
  float4* o4 = reinterpret_cast<float4*>(o);
  uint32_t m = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    float4 x = a4[i];
    x.x = f(x.x); x.y = f(x.y); x.z = f(x.z); x.w = f(x.w);
    o4[i] = x;
    if (TracksAmax<F>::value) m = amax4(m, x);
  }
  for (int64_t i = (nv << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) { float r = f(a[i]); o[i] = r; if (TracksAmax<F>::value) m = max(m, amax_bits(r)); }
  if (TracksAmax<F>::value) amax_commit(am, m);
}
template <class F> __global__ void __launch_bounds__(kBlock) map1_scalar_kernel(const float* a, float* o, int64_t n, F f) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) o[i] = f(a[i]);
}
template <class F> __global__ void __launch_bounds__(kBlock) map2_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ o, int64_t n, F f, AmaxOut am) {
  grid_dep_sync();
  int64_t nv = n >> 2, stride = (int64_t)gridDim.x * blockDim.x;
  const float4* a4 = reinterpret_cast<const float4*>(a);
  const float4* b4 = reinterpret_cast<const float4*>(b);
  float4* o4 = reinterpret_cast<float4*>(o);
  uint32_t m = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    float4 x = a4[i], y = b4[i], r;
    r.x = f(x.x, y.x); r.y = f(x.y, y.y); r.z = f(x.z, y.z); r.w = f(x.w, y.w);
    o4[i] = r;
    if (TracksAmax<F>::value) m = amax4(m, r);
  }
  for (int64_t i = (nv << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) { float r = f(a[i], b[i]); o[i] = r; if (TracksAmax<F>::value) m = max(m, amax_bits(r)); }
  if (TracksAmax<F>::value) amax_commit(am, m);
}
template <class F> __global__ void __launch_bounds__(kBlock) map2_scalar_kernel(const float* a, const float* b, float* o, int64_t n, F f) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) o[i] = f(a[i], b[i]);
}
template <class F> __global__ void __launch_bounds__(kBlock) map3_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ c, float* __restrict__ o, int64_t n, F f, AmaxOut am) {
  grid_dep_sync();
  int64_t nv = n >> 2, stride = (int64_t)gridDim.x * blockDim.x;
  const float4* a4 = reinterpret_cast<const float4*>(a);
  const float4* b4 = reinterpret_cast<const float4*>(b);
  const float4* c4 = reinterpret_cast<const float4*>(c);
  float4* o4 = reinterpret_cast<float4*>(o);
  uint32_t m = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    float4 x = a4[i], y = b4[i], z = c4[i], r;
    r.x = f(x.x, y.x, z.x); r.y = f(x.y, y.y, z.y); r.z = f(x.z, y.z, z.z); r.w = f(x.w, y.w, z.w);
    o4[i] = r;
    if (TracksAmax<F>::value) m = amax4(m, r);
  }
  for (int64_t i = (nv << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) { float r = f(a[i], b[i], c[i]); o[i] = r; if (TracksAmax<F>::value) m = max(m, amax_bits(r)); }
  if (TracksAmax<F>::value) amax_commit(am, m);
}
template <class F> __global__ void __launch_bounds__(kBlock) map3_scalar_kernel(const float* a, const float* b, const float* c, float* o, int64_t n, F f) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) o[i] = f(a[i], b[i], c[i]);
}

template <class F> static AmaxOut track_of(const float* out) { return TracksAmax<F>::value ? amax_track_begin(out) : AmaxOut{}; }

template <class F> static int run_map1(const float* a, float* o, int64_t n, cudaStream_t s, const char* what, F f) {
  if (n <= 0) return 0;
  note_compute_stream(s);
  KernelTimer kt(what, s, 0, 8.0 * n);
  if (aligned16(a) && aligned16(o)) launch_dep(map1_kernel<F>, dim3(grid_for(n, kBlock, 4)), dim3(kBlock), 0, s, a, o, n, f, track_of<F>(o));
  else map1_scalar_kernel<<<grid_for(n, kBlock, 1), kBlock, 0, s>>>(a, o, n, f);
  TF_AFTER(s, what);
  return 0;
}
template <class F> static int run_map2(const float* a, const float* b, float* o, int64_t n, cudaStream_t s, const char* what, F f) {
  if (n <= 0) return 0;
  note_compute_stream(s);
  KernelTimer kt(what, s, 0, 12.0 * n);
  if (aligned16(a) && aligned16(b) && aligned16(o)) launch_dep(map2_kernel<F>, dim3(grid_for(n, kBlock, 4)), dim3(kBlock), 0, s, a, b, o, n, f, track_of<F>(o));
  else map2_scalar_kernel<<<grid_for(n, kBlock, 1), kBlock, 0, s>>>(a, b, o, n, f);
  TF_AFTER(s, what);
  return 0;
}
template <class F> static int run_map3(const float* a, const float* b, const float* c, float* o, int64_t n, cudaStream_t s, const char* what, F f) {
  if (n <= 0) return 0;
  note_compute_stream(s);
  KernelTimer kt(what, s, 0, 16.0 * n);
  if (aligned16(a) && aligned16(b) && aligned16(c) && aligned16(o)) launch_dep(map3_kernel<F>, dim3(grid_for(n, kBlock, 4)), dim3(kBlock), 0, s, a, b, c, o, n, f, track_of<F>(o));
  else map3_scalar_kernel<<<grid_for(n, kBlock, 1), kBlock, 0, s>>>(a, b, c, o, n, f);
  TF_AFTER(s, what);
  return 0;
}

struct FSet { float v; __device__ float operator()(float) const { return v; } };
struct FAddC { float c; __device__ float operator()(float x) const { return x + c; } };
struct FMulC { float c; __device__ float operator()(float x) const { return x * c; } };
struct FRelu { static constexpr bool kTrackAmax = true; __device__ float operator()(float x) const { return x > 0.f ? x : (x != x ? x : 0.f); } };   // NaN propagates
struct FExp { __device__ float operator()(float x) const { return expf(x); } };
struct FLog { __device__ float operator()(float x) const { return logf(x); } };
struct FRecip { __device__ float operator()(float x) const { return 1.f / x; } };
struct FPow { float p; __device__ float operator()(float x) const { return powf(x, p); } };
struct FSigmoid { __device__ float operator()(float x) const { return 1.f / (1.f + expf(-x)); } };
struct FTanh { __device__ float operator()(float x) const { return tanhf(x); } };
struct FAdd { __device__ float operator()(float a, float b) const { return a + b; } };   // no max|y| on the side: the reduction costs the 36 sums of a ResNet-50 step what the 12 more fused ReLU packs it enables save
struct FMul { __device__ float operator()(float a, float b) const { return a * b; } };
struct FReluGrad { static constexpr bool kTrackAmax = true; __device__ float operator()(float x, float g) const { return x > 0.f ? g : 0.f; } };
struct FSgd { static constexpr bool kTrackAmax = true; float lr; __device__ float operator()(float w, float g) const { return w - lr * g; } };
struct FCross { float b; __device__ float operator()(float x, float y) const { return logf(x) * y * (-1.f) * b; } };
struct FCrossBwd { float b; __device__ float operator()(float x, float y, float d) const { return y * (-1.f) * b * (1.0f / x) * d; } };
struct FSigmoidBwd { __device__ float operator()(float y, float dy) const { return dy * y * (1.f - y); } };
struct FTanhBwd { __device__ float operator()(float y, float dy) const { return dy * (1.f - y * y); } };
struct FAdamStep { static constexpr bool kTrackAmax = true; float c1, c2, e, lr; __device__ float operator()(float w, float m, float v) const { return w - lr * m / c1 / (sqrtf(v / c2) + e); } };
struct FBce { __device__ float operator()(float a, float b) const { return b * logf(a) + (1.f - b) * logf(1.f - a); } };

// ---- broadcast --------------------------------------------------------------------
// out[i] = in[i % inner]  (trailing-dimension broadcast; src/gpu_op.cu:47-52)
__global__ void __launch_bounds__(kBlock) bcast_tail_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t inner, int64_t total) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) out[i] = __ldg(in + i % inner);
}
// out[n,c,:] = in[c]  (channel broadcast; src/gpu_op.cu:108-123)
__global__ void __launch_bounds__(kBlock) bcast_channel_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t C, int64_t low, int64_t total) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) out[i] = __ldg(in + (i / low) % C);
}

// ---- reductions --------------------------------------------------------------------
// Column sums of a row-major [rows x cols] matrix, out[c] = sum_r in[r, c].
// Block = 32 columns x 8 row lanes; grid.x tiles the columns, grid.y splits the rows; with several row
// splits each writes its partial sums to out[split * cols + c] (a scratch array) and colsum_final_kernel
// adds the splits in order, so the result does not depend on scheduling.
__global__ void __launch_bounds__(256) colsum_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t rows, int64_t cols, int64_t rows_per_split) {
  __shared__ float sm[8][33];
  int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  int64_t c = (int64_t)blockIdx.x * 32 + tx;
  int64_t r0 = (int64_t)blockIdx.y * rows_per_split, r1 = min(rows, r0 + rows_per_split);
  float acc = 0.f;
  if (c < cols) for (int64_t r = r0 + ty; r < r1; r += 8) acc += in[r * cols + c];
  sm[ty][tx] = acc;
  __syncthreads();
  if (ty == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) t += sm[j][tx];
    out[(int64_t)blockIdx.y * cols + c] = t;
  }
}
__global__ void __launch_bounds__(256) colsum_final_kernel(const float* __restrict__ part, float* __restrict__ out, int64_t cols, int splits) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float t = 0.f;
  for (int z = 0; z < splits; ++z) t += part[(int64_t)z * cols + c];
  out[c] = t;
}
// Sum of n contiguous floats into out[0]; two launches: per-block partials then one block.
__global__ void __launch_bounds__(kBlock) partial_sum_kernel(const float* __restrict__ in, float* __restrict__ part, int64_t n) {
  __shared__ float red[33];
  float acc = 0.f;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) acc += in[i];
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) part[blockIdx.x] = acc;
}
__global__ void __launch_bounds__(kBlock) final_sum_kernel(const float* __restrict__ part, float* __restrict__ out, int n, float scale) {
  __shared__ float red[33];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += part[i];
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) out[0] = acc * scale;
}
// out[o] = sum over the reduced coordinates, general strided form: one block per output
// element (used for the (N,C,H,W) -> (1,C,1,1) bias gradient and odd shapes).
struct ReduceGeom { int ndim; int64_t in_dims[5]; int64_t in_strides[5]; int reduced[5]; int64_t nred; };
__global__ void __launch_bounds__(kBlock) reduce_general_kernel(const float* __restrict__ in, float* __restrict__ out, ReduceGeom g) {
  __shared__ float red[33];
  // decode the kept coordinates of this output element
  int64_t o = blockIdx.x, base = 0;
  for (int d = g.ndim - 1; d >= 0; --d) {
    if (!g.reduced[d]) { int64_t c = o % g.in_dims[d]; o /= g.in_dims[d]; base += c * g.in_strides[d]; }
  }
  float acc = 0.f;
  for (int64_t r = threadIdx.x; r < g.nred; r += blockDim.x) {
    int64_t rr = r, off = base;
    for (int d = g.ndim - 1; d >= 0; --d) {
      if (g.reduced[d]) { int64_t c = rr % g.in_dims[d]; rr /= g.in_dims[d]; off += c * g.in_strides[d]; }
    }
    acc += in[off];
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) out[blockIdx.x] = acc;
}
// out[outer, inner] = sum_k in[outer, k, inner]  (axis reduction, src/gpu_op.cu:527)
__global__ void __launch_bounds__(kBlock) axis_sum_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t outer, int64_t red, int64_t inner) {
  int64_t total = outer * inner, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int64_t o = i / inner, j = i % inner;
    const float* p = in + o * red * inner + j;
    float acc = 0.f;
    for (int64_t k = 0; k < red; ++k) acc += p[k * inner];
    out[i] = acc;
  }
}
__global__ void __launch_bounds__(kBlock) axis_bcast_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t outer, int64_t red, int64_t inner) {
  int64_t total = outer * red * inner, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int64_t j = i % inner, o = i / (inner * red);
    out[i] = in[o * inner + j];
  }
}

// ---- softmax family ------------------------------------------------------------------
// One warp per row, max-subtracted (src/gpu_op.cu:237-258).
__global__ void __launch_bounds__(kBlock) row_softmax_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t rows, int64_t cols) {
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const float* x = in + r * cols;
    float m = -INFINITY;
    for (int64_t c = lane; c < cols; c += 32) m = fmaxf(m, x[c]);
    m = warp_max(m);
    float s = 0.f;
    for (int64_t c = lane; c < cols; c += 32) s += expf(x[c] - m);
    s = warp_sum(s);
    float inv = 1.f / s;
    for (int64_t c = lane; c < cols; c += 32) out[r * cols + c] = expf(x[c] - m) * inv;
  }
}
// dx = y * (dy - sum(dy*y)) per row (softmax backward over the non-batch elements).
__global__ void __launch_bounds__(kBlock) row_softmax_bwd_kernel(const float* __restrict__ y, const float* __restrict__ dy, float* __restrict__ dx, int64_t rows, int64_t cols) {
  int lane = threadIdx.x & 31;
  int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const float* yr = y + r * cols;
    const float* dr = dy + r * cols;
    float s = 0.f;
    for (int64_t c = lane; c < cols; c += 32) s += yr[c] * dr[c];
    s = warp_sum(s);
    for (int64_t c = lane; c < cols; c += 32) dx[r * cols + c] = yr[c] * (dr[c] - s);
  }
}
// mean over rows of -sum_c label*log(softmax(logits)); one block, one warp per row
// (src/gpu_op.cu:261-301, without its 4096-row limit).
__global__ void __launch_bounds__(1024) softmax_xent_kernel(const float* __restrict__ logits, const float* __restrict__ labels, float* __restrict__ out, int64_t rows, int64_t cols) {
  __shared__ float red[33];
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float acc = 0.f;
  for (int64_t r = w; r < rows; r += nw) {
    const float* x = logits + r * cols;
    const float* t = labels + r * cols;
    float m = -INFINITY;
    for (int64_t c = lane; c < cols; c += 32) m = fmaxf(m, x[c]);
    m = warp_max(m);
    float s = 0.f;
    for (int64_t c = lane; c < cols; c += 32) s += expf(x[c] - m);
    s = warp_sum(s);
    float ls = logf(s), l = 0.f;
    for (int64_t c = lane; c < cols; c += 32) l -= t[c] * (x[c] - m - ls);
    acc += l;   // every lane holds a partial of this row
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) out[0] = acc / (float)rows;
}
// Row-wise norms used by the L1 / L2 losses and regularisers: out[0] = scale * mean_rows(sum_c f(a,b)).
template <int MODE> __global__ void __launch_bounds__(1024) row_loss_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, int64_t rows, int64_t cols, float scale) {
  __shared__ float red[33];
  float acc = 0.f;
  int64_t n = rows * cols;
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    float d = b ? b[i] - a[i] : a[i];
    acc += MODE == 1 ? fabsf(d) : d * d;
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) out[0] = acc / (float)rows * scale;
}
template <int MODE> __global__ void __launch_bounds__(kBlock) loss_grad_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ g, float* __restrict__ o, int64_t n, float inv_rows) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  float gg = g[0] * inv_rows;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float d = b ? a[i] - b[i] : a[i];
    o[i] = MODE == 1 ? (d > 0.f ? gg : -gg) : d * gg;
  }
}

// ---- concat along axis 1 ---------------------------------------------------------------
// dst[n, off + j] = src[n, j] for j < src_inner; MODE 0 copies src -> dst slice, MODE 1 the
// slice of dst -> src (the backward split).  Rows are n, `inner` counts floats per sample.
// One grid row (blockIdx.y) per sample, so no per-element divide; V = float4 when both inner sizes and the offset
// are multiples of 4 floats, else float.
__device__ __forceinline__ uint32_t amax_of(const float4& v) { return amax4(0u, v); }
__device__ __forceinline__ uint32_t amax_of(float v) { return amax_bits(v); }
template <int MODE, typename V> __global__ void __launch_bounds__(kBlock) slice_copy_kernel(V* __restrict__ part, V* __restrict__ whole, int64_t nrows, int64_t part_inner, int64_t whole_inner, int64_t off, AmaxOut am) {
  grid_dep_sync();
  uint32_t m = 0;
  for (int64_t r = blockIdx.y; r < nrows; r += gridDim.y) {
    V* p = part + r * part_inner;
    V* w = whole + r * whole_inner + off;
    for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < part_inner; j += (int64_t)gridDim.x * blockDim.x) {
      V v = MODE == 0 ? p[j] : w[j];
      if (MODE == 0) w[j] = v; else p[j] = v;
      m = max(m, amax_of(v));
    }
  }
  amax_commit(am, m);
}
// `am` accumulates max|copied values| for the written tensor; a tensor written by two launches (concat forward)
// passes the clear word to the first launch only.
template <int MODE> static void launch_slice_copy(float* part, float* whole, int64_t rows, int64_t part_inner, int64_t whole_inner, int64_t off, cudaStream_t s, AmaxOut am) {
  if (rows <= 0 || part_inner <= 0) return;
  bool vec = part_inner % 4 == 0 && whole_inner % 4 == 0 && off % 4 == 0 && ((uintptr_t)part % 16 == 0) && ((uintptr_t)whole % 16 == 0);
  int64_t per_row = vec ? part_inner / 4 : part_inner;
  int gy = (int)(rows < 65535 ? rows : 65535);
  int64_t want = (per_row + kBlock - 1) / kBlock, cap = (int64_t)8 * 148 / gy + 1;
  int gx = (int)(want < cap ? want : cap);
  dim3 grid(gx < 1 ? 1 : gx, gy);
  if (vec) launch_dep(slice_copy_kernel<MODE, float4>, grid, dim3(kBlock), 0, s, (float4*)part, (float4*)whole, rows, part_inner / 4, whole_inner / 4, off / 4, am);
  else launch_dep(slice_copy_kernel<MODE, float>, grid, dim3(kBlock), 0, s, part, whole, rows, part_inner, whole_inner, off, am);
}

// ---- dropout: counter-based keep mask ---------------------------------------------------
// keep(i) is a pure function of (seed, i), so backward regenerates the forward mask and no
// mask tensor is stored.  The generator is a 64-bit mix (splitmix64 finaliser) of the
// element index keyed by the seed.
__device__ __forceinline__ float uniform01(unsigned long long seed, unsigned long long i) {
  unsigned long long z = (i + 1) * 0x9E3779B97F4A7C15ull + seed * 0xD1342543DE82EF95ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}
__global__ void __launch_bounds__(kBlock) dropout_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t n, float p, float scale, unsigned long long seed) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = uniform01(seed, (unsigned long long)i) >= p ? in[i] * scale : 0.f;
}

// ---- optimisers ----------------------------------------------------------------------------
__global__ void __launch_bounds__(kBlock) adam_moments_kernel(float* __restrict__ m, float* __restrict__ v, const float* __restrict__ g, int64_t n, float b1, float b2) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float gi = g[i];
    m[i] = m[i] * b1 + gi * (1.f - b1);
    v[i] = v[i] * b2 + gi * gi * (1.f - b2);
  }
}
// Multi-tensor variants: one launch walks a device table of tensor pointers.
struct TensorTable { int count; };
__global__ void __launch_bounds__(kBlock) sgd_table_kernel(float* const* __restrict__ w, float* const* __restrict__ g, const int* __restrict__ prefix, int ntensors, int64_t total, float lr) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int lo = 0, hi = ntensors;            // prefix[t] <= i < prefix[t+1]
    while (hi - lo > 1) { int mid = (lo + hi) >> 1; if (prefix[mid] <= i) lo = mid; else hi = mid; }
    int64_t j = i - prefix[lo];
    w[lo][j] -= lr * g[lo][j];
  }
}
__global__ void __launch_bounds__(kBlock) adam_table_kernel(float* const* __restrict__ w, float* const* __restrict__ m, float* const* __restrict__ v, float* const* __restrict__ g, const int* __restrict__ prefix, int ntensors, int64_t total, float b1, float b2, float c1, float c2, float e, float lr) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int lo = 0, hi = ntensors;
    while (hi - lo > 1) { int mid = (lo + hi) >> 1; if (prefix[mid] <= i) lo = mid; else hi = mid; }
    int64_t j = i - prefix[lo];
    float gi = g[lo][j];
    float mi = m[lo][j] * b1 + gi * (1.f - b1);
    float vi = v[lo][j] * b2 + gi * gi * (1.f - b2);
    m[lo][j] = mi; v[lo][j] = vi;
    w[lo][j] -= lr * mi / c1 / (sqrtf(vi / c2) + e);
  }
}

}  // namespace tf

using namespace tf;

// Data-parallel hook implemented in dp_nccl.cu: returns 1 when it took ownership of the update.
namespace tf {
int dp_sgd_update(float* w, const float* g, int64_t n, float lr, cudaStream_t s);
int dp_adam_moments(float* m, float* v, const float* g, int64_t n, float b1, float b2, cudaStream_t s);
int dp_adam_step(float* w, const float* m, const float* v, float c1, float c2, float eps, float lr, cudaStream_t s);
}

static inline const float* F(const DLArrayHandle a) { return (const float*)a->data; }
static inline float* FM(DLArrayHandle a) { return out_f32(a); }

namespace tf {
// The plain kernel of a held-back call (the output's write version was bumped when the call was recorded).
int launch_deferred_now(const DeferredOp& op) {
  if (op.kind == kDeferAdd) return run_map2(op.a, op.b, op.out, op.n, op.stream, "DLGpuMatrixElementwiseAdd", FAdd{});
  return run_map2(op.a, op.b, op.out, op.n, op.stream, "DLGpuActivationBackward(relu)", FReluGrad{});
}
// s = a + b and r = relu(s) in one pass (a residual block's sum and the ReLU behind it); max|r| tracked as FRelu does.
__global__ void __launch_bounds__(kBlock) add_relu_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ sum, float* __restrict__ r, int64_t n, AmaxOut am) {
  grid_dep_sync();
  const int64_t nv = n >> 2, stride = (int64_t)gridDim.x * blockDim.x;
  const float4* a4 = reinterpret_cast<const float4*>(a);
  const float4* b4 = reinterpret_cast<const float4*>(b);
  float4* s4 = reinterpret_cast<float4*>(sum);
  float4* r4 = reinterpret_cast<float4*>(r);
  const FRelu relu;
  uint32_t m = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
    const float4 x = a4[i], y = b4[i];
    float4 t, u;
    t.x = x.x + y.x; t.y = x.y + y.y; t.z = x.z + y.z; t.w = x.w + y.w;
    u.x = relu(t.x); u.y = relu(t.y); u.z = relu(t.z); u.w = relu(t.w);
    s4[i] = t;
    r4[i] = u;
    m = amax4(m, u);
  }
  for (int64_t i = (nv << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float t = a[i] + b[i], u = relu(t);
    sum[i] = t; r[i] = u;
    m = max(m, amax_bits(u));
  }
  amax_commit(am, m);
}
static std::atomic<long long> g_fused_add_relu{0};
long long fused_add_relu_count() { return g_fused_add_relu.load(); }
// The ReLU forward of a held-back sum: both in one kernel.  Called with the slot locked (take_deferred succeeded).
static bool launch_add_relu(const DeferredOp& add, float* r, cudaStream_t s) {
  if (!(aligned16(add.a) && aligned16(add.b) && aligned16(add.out) && aligned16(r))) return false;
  note_compute_stream(s);
  KernelTimer kt("Add+ReluForward", s, 0, 16.0 * add.n);
  launch_dep(add_relu_kernel, dim3(grid_for(add.n, kBlock, 4)), dim3(kBlock), 0, s, add.a, add.b, add.out, r, add.n, amax_track_begin(r));
  g_fused_add_relu.fetch_add(1);
  return true;
}
}  // namespace tf

extern "C" {

int DLGpuArraySet(DLArrayHandle arr, float value, void** cudaStream) {
  TF_REQUIRE(arr, "null array");
  return run_map1(F(arr), FM(arr), numel(arr), stream_of(cudaStream), "DLGpuArraySet", FSet{value});
}

int DLGpuBroadcastTo0(const DLArrayHandle input, DLArrayHandle output, void** cudaStream) {
  TF_REQUIRE(input && output, "null array");
  int64_t inner = numel(input), total = numel(output);
  TF_REQUIRE(inner > 0 && total % inner == 0, "DLGpuBroadcastTo0: output size %lld is not a multiple of input size %lld", (long long)total, (long long)inner);
  cudaStream_t s = stream_of(cudaStream);
  note_compute_stream(s);
  bcast_tail_kernel<<<grid_for(total, kBlock), kBlock, 0, s>>>(F(input), FM(output), inner, total);
  TF_AFTER(s, "DLGpuBroadcastTo0");
  return 0;
}

int DLGpuBroadcastTo1(const DLArrayHandle input, DLArrayHandle output, void** cudaStream) {
  TF_REQUIRE(input && output, "null array");
  TF_REQUIRE(input->ndim == 1 && output->ndim >= 2 && input->shape[0] == output->shape[1], "DLGpuBroadcastTo1: input must be (C,) matching output dim 1");
  int64_t low = 1;
  for (int i = 2; i < output->ndim; ++i) low *= output->shape[i];
  int64_t total = numel(output);
  cudaStream_t s = stream_of(cudaStream);
  note_compute_stream(s);
  bcast_channel_kernel<<<grid_for(total, kBlock), kBlock, 0, s>>>(F(input), FM(output), output->shape[1], low, total);
  TF_AFTER(s, "DLGpuBroadcastTo1");
  return 0;
}

static int reduce_to_scalar(const float* in, float* out, int64_t n, float scale, cudaStream_t s, const char* what) {
  int blocks = grid_for(n, kBlock, 8, 4);
  float* part = (float*)persistent_scratch(0, sizeof(float) * 4096);
  TF_REQUIRE(part, "%s: scratch allocation failed", what);
  if (blocks > 4096) blocks = 4096;
  note_compute_stream(s);
  partial_sum_kernel<<<blocks, kBlock, 0, s>>>(in, part, n);
  final_sum_kernel<<<1, kBlock, 0, s>>>(part, out, blocks, scale);
  if (after_launch(s, what, 2) != 0) return -1;
  return 0;
}

static int column_sums(const float* in, float* out, int64_t rows, int64_t cols, cudaStream_t s, const char* what) {
  int gx = (int)((cols + 31) / 32);
  int splits = 1;
  int sms = device_sm_count();
  if (gx < 2 * sms && rows >= 64) {                 // few column tiles: split the rows for occupancy
    splits = (int)((2 * sms + gx - 1) / gx);
    if (splits > rows / 16) splits = (int)(rows / 16);
    if (splits < 1) splits = 1;
  }
  int64_t rps = (rows + splits - 1) / splits;
  splits = (int)((rows + rps - 1) / rps);
  note_compute_stream(s);
  if (splits > 1) {
    float* part = (float*)persistent_scratch(2, sizeof(float) * (size_t)splits * (size_t)cols);
    if (part) {
      colsum_kernel<<<dim3(gx, splits), 256, 0, s>>>(in, part, rows, cols, rps);
      colsum_final_kernel<<<(unsigned)((cols + 255) / 256), 256, 0, s>>>(part, out, cols, splits);
      return after_launch(s, what, 2) != 0 ? -1 : 0;
    }
    rps = rows;                                  // no scratch: one split
  }
  colsum_kernel<<<dim3(gx, 1), 256, 0, s>>>(in, out, rows, cols, rps);
  if (after_launch(s, what, 1) != 0) return -1;
  return 0;
}

int DLGReduceSumGetCudnnlist(const int* input_shapes, const int* output_shapes, const int sizeofshape,
                             int dataformat, void*** cudnnlist, void** cudnnHandle) {
  (void)dataformat; (void)cudnnHandle;
  TF_REQUIRE(input_shapes && output_shapes && cudnnlist && sizeofshape >= 1 && sizeofshape <= 5, "DLGReduceSumGetCudnnlist: bad arguments");
  ReducePlan* p = new_plan<ReducePlan>(cudnnlist, kPlanReduce, 5);
  p->ndim = sizeofshape;
  for (int i = 0; i < sizeofshape; ++i) {
    p->in_dims[i] = input_shapes[i];
    p->out_dims[i] = output_shapes[i];
    if (!(output_shapes[i] == input_shapes[i] || output_shapes[i] == 1)) { set_error("DLGReduceSumGetCudnnlist: output extent must be 1 or match"); return -1; }
  }
  return 0;
}

// Sums over every axis whose output extent is 1 (the memory order is the order of the
// shape the plan was built with, for both data formats; src/gpu_op.cu:628-810).
int DLGpuReduceSum(const DLArrayHandle input, DLArrayHandle output, void*** cudnnlist, void** cudnnHandle,
                   int* memorytoSaving, void** cudaStream) {
  (void)cudnnHandle; (void)memorytoSaving;
  ReducePlan* p = plan_of<ReducePlan>(cudnnlist, kPlanReduce);
  TF_REQUIRE(p && input && output, "DLGpuReduceSum: missing plan or array");
  int64_t nin = 1, nout = 1;
  for (int i = 0; i < p->ndim; ++i) { nin *= p->in_dims[i]; nout *= p->out_dims[i]; }
  TF_REQUIRE(nin == numel(input) && nout == numel(output), "DLGpuReduceSum: arrays do not match the plan");
  cudaStream_t s = stream_of(cudaStream);
  if (nout == 1) return reduce_to_scalar(F(input), FM(output), nin, 1.f, s, "DLGpuReduceSum");
  // leading axes reduced, trailing kept  ->  column sums
  int first_kept = 0;
  while (first_kept < p->ndim && (p->out_dims[first_kept] == 1)) ++first_kept;
  bool tail_kept = true;
  for (int i = first_kept; i < p->ndim; ++i) if (p->out_dims[i] != p->in_dims[i]) tail_kept = false;
  if (tail_kept) return column_sums(F(input), FM(output), nin / nout, nout, s, "DLGpuReduceSum");
  ReduceGeom g;
  g.ndim = p->ndim; g.nred = 1;
  int64_t st = 1;
  for (int d = p->ndim - 1; d >= 0; --d) {
    g.in_dims[d] = p->in_dims[d]; g.in_strides[d] = st; st *= p->in_dims[d];
    g.reduced[d] = (p->out_dims[d] == 1 && p->in_dims[d] != 1) ? 1 : 0;
    if (g.reduced[d]) g.nred *= p->in_dims[d];
  }
  note_compute_stream(s);
  reduce_general_kernel<<<(unsigned)nout, kBlock, 0, s>>>(F(input), FM(output), g);
  TF_AFTER(s, "DLGpuReduceSum");
  return 0;
}

int DLGpuReduceSumAxisZero(const DLArrayHandle input, DLArrayHandle output) {
  TF_REQUIRE(input && output && input->ndim >= 1, "null array");
  int64_t rows = input->shape[0], cols = rows ? numel(input) / rows : 0;
  TF_REQUIRE(numel(output) == (cols ? cols : 1), "DLGpuReduceSumAxisZero: output size mismatch");
  if (input->ndim == 1) return reduce_to_scalar(F(input), FM(output), rows, 1.f, 0, "DLGpuReduceSumAxisZero");
  return column_sums(F(input), FM(output), rows, cols, 0, "DLGpuReduceSumAxisZero");
}
// The two legacy "broadcast backward" reductions: sum the leading axes down to the output's
// shape (trailing broadcast) or sum everything but the channel axis.
int DLGpuBroadcastToBackward0(const DLArrayHandle input, DLArrayHandle output) {
  TF_REQUIRE(input && output, "null array");
  int64_t nout = numel(output), nin = numel(input);
  TF_REQUIRE(nout > 0 && nin % nout == 0, "DLGpuBroadcastToBackward0: size mismatch");
  if (nout == 1) return reduce_to_scalar(F(input), FM(output), nin, 1.f, 0, "DLGpuBroadcastToBackward0");
  return column_sums(F(input), FM(output), nin / nout, nout, 0, "DLGpuBroadcastToBackward0");
}
int DLGpuBroadcastToBackward1(const DLArrayHandle input, DLArrayHandle output) {
  TF_REQUIRE(input && output && input->ndim >= 2 && output->ndim == 1 && output->shape[0] == input->shape[1], "DLGpuBroadcastToBackward1: output must be (C,)");
  ReduceGeom g;
  g.ndim = input->ndim; g.nred = 1;
  TF_REQUIRE(g.ndim <= 5, "DLGpuBroadcastToBackward1: rank > 5");
  int64_t st = 1;
  for (int d = g.ndim - 1; d >= 0; --d) {
    g.in_dims[d] = input->shape[d]; g.in_strides[d] = st; st *= input->shape[d];
    g.reduced[d] = d != 1;
    if (g.reduced[d]) g.nred *= input->shape[d];
  }
  note_compute_stream(0);
  reduce_general_kernel<<<(unsigned)output->shape[0], kBlock, 0, 0>>>(F(input), FM(output), g);
  TF_AFTER(0, "DLGpuBroadcastToBackward1");
  return 0;
}
int DLGpuReduceSumAxisN(const DLArrayHandle input, DLArrayHandle output, const int axis) {
  TF_REQUIRE(input && output && axis >= 0 && axis < input->ndim, "DLGpuReduceSumAxisN: bad axis");
  int64_t outer = 1, inner = 1, red = input->shape[axis];
  for (int i = 0; i < axis; ++i) outer *= input->shape[i];
  for (int i = axis + 1; i < input->ndim; ++i) inner *= input->shape[i];
  TF_REQUIRE(numel(output) == outer * inner, "DLGpuReduceSumAxisN: output size mismatch");
  note_compute_stream(0);
  axis_sum_kernel<<<grid_for(outer * inner, kBlock), kBlock>>>(F(input), FM(output), outer, red, inner);
  TF_AFTER(0, "DLGpuReduceSumAxisN");
  return 0;
}
int DLGpuReduceSumAxisNBackward(const DLArrayHandle input, DLArrayHandle output, const int axis) {
  TF_REQUIRE(input && output && axis >= 0 && axis < output->ndim, "DLGpuReduceSumAxisNBackward: bad axis");
  int64_t outer = 1, inner = 1, red = output->shape[axis];
  for (int i = 0; i < axis; ++i) outer *= output->shape[i];
  for (int i = axis + 1; i < output->ndim; ++i) inner *= output->shape[i];
  TF_REQUIRE(numel(input) == outer * inner, "DLGpuReduceSumAxisNBackward: input size mismatch");
  note_compute_stream(0);
  axis_bcast_kernel<<<grid_for(numel(output), kBlock), kBlock>>>(F(input), FM(output), outer, red, inner);
  TF_AFTER(0, "DLGpuReduceSumAxisNBackward");
  return 0;
}
int DLGpuReduceSumAll(const DLArrayHandle input, DLArrayHandle output) {
  TF_REQUIRE(input && output && numel(output) == 1, "DLGpuReduceSumAll: output must hold one element");
  return reduce_to_scalar(F(input), FM(output), numel(input), 1.f, 0, "DLGpuReduceSumAll");
}
}  // extern "C" (reopened below)

// ---- sum of all elements without any allocation ------------------------------------------------
// Some callers must not allocate while they run: code that replays a fixed sequence of launches and may
// not touch the allocator in between, code running inside a memory-planned region where every byte of the
// device is already assigned (the swap / recompute scheduler sizes its plan to the last byte), or a host
// thread that must not take the allocator's lock.  DLGpuReduceSumAll needs a scratch buffer for its
// per-block partial sums and gets it from the pool; this variant keeps that scratch in a fixed array that
// is part of the library image instead, so it calls no cudaMalloc / cudaFree / pool routine at all.
//
// The price is a size limit and shared state: the array holds kStaticPartials floats (16 KiB, resident on
// every GPU that loads the library until the process exits), one per block of kStaticElemsPerBlock inputs,
// so inputs above kStaticMaxElems elements are refused.  All calls use the same array: two calls that
// overlap on the GPU (different streams, or different host threads) race on it; calls on one stream are
// safe.  Nothing has to start at zero (each call overwrites exactly the partials it then reads).
constexpr int kStaticPartials = 4096;
constexpr int kStaticElemsPerBlock = kBlock * 32;                                   // 8192 inputs per block
constexpr long long kStaticMaxElems = (long long)kStaticPartials * kStaticElemsPerBlock;   // 33,554,432 floats (128 MiB)
static __device__ __align__(256) float g_static_partials[kStaticPartials];

// In host code `g_static_partials` is only a handle for the symbol, not a device address; the address a
// kernel can use comes from cudaGetSymbolAddress, once per device, with that device current.
// The per-device cache needs no lock: two threads that race on the first call both look the address up and store the
// same value (the write is idempotent), and the slots are atomics so neither can see a torn pointer.
static float* static_partials_ptr() {
  static std::atomic<float*> ptr[64];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); set_error("DLGpuReduceSumAllStatic: no current device"); return nullptr; }
  float* p = ptr[dev].load(std::memory_order_acquire);
  if (!p) {
    cudaError_t e = cudaGetSymbolAddress((void**)&p, g_static_partials);
    if (e != cudaSuccess) { cudaGetLastError(); set_error("DLGpuReduceSumAllStatic: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e)); return nullptr; }
    ptr[dev].store(p, std::memory_order_release);
  }
  return p;
}

extern "C" {

// output[0] = sum of every element of input, computed on *cudaStream (NULL: the legacy default stream).
// Allocation-free twin of DLGpuReduceSumAll; see the notes above.  The first call on a device looks up the
// scratch array's device address (a host-side runtime query, no allocation) and should therefore be made
// before any stream capture begins on that device; later calls only launch two kernels.
int DLGpuReduceSumAllStatic(const DLArrayHandle input, DLArrayHandle output, void** cudaStream) {
  TF_REQUIRE(input && output && numel(output) == 1, "DLGpuReduceSumAllStatic: output must hold one element");
  const int64_t n = numel(input);
  TF_REQUIRE(n <= kStaticMaxElems, "DLGpuReduceSumAllStatic: %lld elements exceed the fixed scratch capacity of %lld elements; use DLGpuReduceSumAll", (long long)n, kStaticMaxElems);
  float* part = static_partials_ptr();
  if (!part) return -1;
  cudaStream_t s = stream_of(cudaStream);
  int blocks = (int)((n + kStaticElemsPerBlock - 1) / kStaticElemsPerBlock);
  if (blocks < 1) blocks = 1;
  note_compute_stream(s);
  partial_sum_kernel<<<blocks, kBlock, 0, s>>>(F(input), part, n);
  final_sum_kernel<<<1, kBlock, 0, s>>>(part, FM(output), blocks, 1.f);
  if (after_launch(s, "DLGpuReduceSumAllStatic", 2) != 0) return -1;
  return 0;
}

int DLGpuReduceSumAllBackward(const DLArrayHandle input, DLArrayHandle output) {
  TF_REQUIRE(input && output && numel(input) >= 1, "null array");
  int64_t total = numel(output);
  note_compute_stream(0);
  bcast_tail_kernel<<<grid_for(total, kBlock), kBlock>>>(F(input), FM(output), 1, total);
  TF_AFTER(0, "DLGpuReduceSumAllBackward");
  return 0;
}

#define TF_SAME(a, b, name) TF_REQUIRE((a) && (b) && numel(a) == numel(b), name ": element counts differ")

int DLGpuMatrixElementwiseAdd(const DLArrayHandle matA, const DLArrayHandle matB, DLArrayHandle output, void** cudaStream) {
  TF_SAME(matA, matB, "DLGpuMatrixElementwiseAdd"); TF_SAME(matA, output, "DLGpuMatrixElementwiseAdd");
  cudaStream_t s = stream_of(cudaStream);
  // Held back for one call: if the ReLU forward of this sum comes next, one kernel writes both.
  if (deferral_enabled() && numel(output) >= (1 << 16)) {
    defer_op(DeferredOp{kDeferAdd, F(matA), F(matB), FM(output), numel(output), s});
    return 0;
  }
  return run_map2(F(matA), F(matB), FM(output), numel(output), s, "DLGpuMatrixElementwiseAdd", FAdd{});
}
int DLGpuMatrixElementwiseAddByConst(const DLArrayHandle input, float val, DLArrayHandle output, void** cudaStream) {
  TF_SAME(input, output, "DLGpuMatrixElementwiseAddByConst");
  return run_map1(F(input), FM(output), numel(output), stream_of(cudaStream), "DLGpuMatrixElementwiseAddByConst", FAddC{val});
}
int DLGpuMatrixElementwiseMultiply(const DLArrayHandle matA, const DLArrayHandle matB, DLArrayHandle output, void** cudaStream) {
  TF_SAME(matA, matB, "DLGpuMatrixElementwiseMultiply"); TF_SAME(matA, output, "DLGpuMatrixElementwiseMultiply");
  return run_map2(F(matA), F(matB), FM(output), numel(output), stream_of(cudaStream), "DLGpuMatrixElementwiseMultiply", FMul{});
}
int DLGpuMatrixMultiplyByConst(const DLArrayHandle input, float val, DLArrayHandle output, void** cudaStream) {
  TF_SAME(input, output, "DLGpuMatrixMultiplyByConst");
  return run_map1(F(input), FM(output), numel(output), stream_of(cudaStream), "DLGpuMatrixMultiplyByConst", FMulC{val});
}
int DLGpuRelu(const DLArrayHandle input, DLArrayHandle output) {
  TF_SAME(input, output, "DLGpuRelu");
  return run_map1(F(input), FM(output), numel(output), last_compute_stream(), "DLGpuRelu", FRelu{});
}
int DLGpuReluGradient(const DLArrayHandle input, const DLArrayHandle in_grad, DLArrayHandle output) {
  TF_SAME(input, in_grad, "DLGpuReluGradient"); TF_SAME(input, output, "DLGpuReluGradient");
  return run_map2(F(input), F(in_grad), FM(output), numel(output), last_compute_stream(), "DLGpuReluGradient", FReluGrad{});
}
int DLGpuMatrixExp(const DLArrayHandle input, DLArrayHandle output) {
  TF_SAME(input, output, "DLGpuMatrixExp");
  return run_map1(F(input), FM(output), numel(output), last_compute_stream(), "DLGpuMatrixExp", FExp{});
}
int DLGpuMatrixLog(const DLArrayHandle input, DLArrayHandle output, void** cudaStream) {
  TF_SAME(input, output, "DLGpuMatrixLog");
  return run_map1(F(input), FM(output), numel(output), stream_of(cudaStream), "DLGpuMatrixLog", FLog{});
}
int DLGpuMatrixReverse(const DLArrayHandle input, DLArrayHandle output) {
  TF_SAME(input, output, "DLGpuMatrixReverse");
  return run_map1(F(input), FM(output), numel(output), last_compute_stream(), "DLGpuMatrixReverse", FRecip{});
}
int DLGpuMatrixPow(const DLArrayHandle input, const float val, DLArrayHandle output) {
  TF_SAME(input, output, "DLGpuMatrixPow");
  return run_map1(F(input), FM(output), numel(output), last_compute_stream(), "DLGpuMatrixPow", FPow{val});
}

int DLGpuSoftmax(const DLArrayHandle input, DLArrayHandle output, void** cudaStream) {
  TF_REQUIRE(input && output && input->ndim == 2 && same_shape(input, output), "DLGpuSoftmax: expects matching 2-D arrays");
  int64_t rows = input->shape[0], cols = input->shape[1];
  cudaStream_t s = stream_of(cudaStream);
  note_compute_stream(s);
  row_softmax_kernel<<<grid_for(rows * 32, kBlock), kBlock, 0, s>>>(F(input), FM(output), rows, cols);
  TF_AFTER(s, "DLGpuSoftmax");
  return 0;
}
int DLGpuSoftmaxCrossEntropy(const DLArrayHandle input_a, const DLArrayHandle input_b, DLArrayHandle output, void** cudaStream) {
  TF_REQUIRE(input_a && input_b && output && input_a->ndim == 2 && same_shape(input_a, input_b) && numel(output) == 1, "DLGpuSoftmaxCrossEntropy: expects two matching 2-D arrays and a 1-element output");
  cudaStream_t s = stream_of(cudaStream);
  note_compute_stream(s);
  softmax_xent_kernel<<<1, 1024, 0, s>>>(F(input_a), F(input_b), FM(output), input_a->shape[0], input_a->shape[1]);
  TF_AFTER(s, "DLGpuSoftmaxCrossEntropy");
  return 0;
}
int DLGpuCrossEntropy(const DLArrayHandle input_a, const DLArrayHandle input_b, DLArrayHandle output) {
  TF_SAME(input_a, input_b, "DLGpuCrossEntropy"); TF_SAME(input_a, output, "DLGpuCrossEntropy");
  return run_map2(F(input_a), F(input_b), FM(output), numel(output), last_compute_stream(), "DLGpuCrossEntropy", FBce{});
}
static int row_loss(int mode, const DLArrayHandle a, const DLArrayHandle b, DLArrayHandle out, float scale, const char* what) {
  TF_REQUIRE(a && out && a->ndim >= 1 && numel(out) == 1, "%s: bad arguments", what);
  if (b) TF_REQUIRE(numel(a) == numel(b), "%s: element counts differ", what);
  int64_t rows = a->shape[0], cols = rows ? numel(a) / rows : 0;
  cudaStream_t s = last_compute_stream();
  if (mode == 1) row_loss_kernel<1><<<1, 1024, 0, s>>>(F(a), b ? F(b) : nullptr, FM(out), rows, cols, scale);
  else row_loss_kernel<2><<<1, 1024, 0, s>>>(F(a), b ? F(b) : nullptr, FM(out), rows, cols, scale);
  TF_AFTER(s, what);
  return 0;
}
static int loss_grad(int mode, const DLArrayHandle a, const DLArrayHandle b, const DLArrayHandle g, DLArrayHandle out, const char* what) {
  TF_REQUIRE(a && g && out && a->ndim >= 1 && numel(a) == numel(out) && numel(g) >= 1, "%s: bad arguments", what);
  int64_t n = numel(a);
  float inv = 1.f / (float)a->shape[0];
  cudaStream_t s = last_compute_stream();
  if (mode == 1) loss_grad_kernel<1><<<grid_for(n, kBlock), kBlock, 0, s>>>(F(a), b ? F(b) : nullptr, F(g), FM(out), n, inv);
  else loss_grad_kernel<2><<<grid_for(n, kBlock), kBlock, 0, s>>>(F(a), b ? F(b) : nullptr, F(g), FM(out), n, inv);
  TF_AFTER(s, what);
  return 0;
}
int DLGpuL1loss(const DLArrayHandle a, const DLArrayHandle b, DLArrayHandle o) { TF_REQUIRE(b, "null array"); return row_loss(1, a, b, o, 1.f, "DLGpuL1loss"); }
int DLGpuL2loss(const DLArrayHandle a, const DLArrayHandle b, DLArrayHandle o) { TF_REQUIRE(b, "null array"); return row_loss(2, a, b, o, .5f, "DLGpuL2loss"); }
int DLGpuL1regular(const DLArrayHandle a, DLArrayHandle o) { return row_loss(1, a, nullptr, o, 1.f, "DLGpuL1regular"); }
int DLGpuL2regular(const DLArrayHandle a, DLArrayHandle o) { return row_loss(2, a, nullptr, o, .5f, "DLGpuL2regular"); }
int DLGpuL1LossGradient(const DLArrayHandle a, const DLArrayHandle b, const DLArrayHandle g, DLArrayHandle o) { TF_REQUIRE(b, "null array"); return loss_grad(1, a, b, g, o, "DLGpuL1LossGradient"); }
int DLGpuL2LossGradient(const DLArrayHandle a, const DLArrayHandle b, const DLArrayHandle g, DLArrayHandle o) { TF_REQUIRE(b, "null array"); return loss_grad(2, a, b, g, o, "DLGpuL2LossGradient"); }
int DLGpuL1regularGradient(const DLArrayHandle a, const DLArrayHandle g, DLArrayHandle o) { return loss_grad(1, a, nullptr, g, o, "DLGpuL1regularGradient"); }
int DLGpuL2regularGradient(const DLArrayHandle a, const DLArrayHandle g, DLArrayHandle o) { return loss_grad(2, a, nullptr, g, o, "DLGpuL2regularGradient"); }

int DLGpuCross(const DLArrayHandle x, const DLArrayHandle y, DLArrayHandle output, float b, void** cudaStream) {
  TF_SAME(x, y, "DLGpuCross"); TF_SAME(x, output, "DLGpuCross");
  return run_map2(F(x), F(y), FM(output), numel(output), stream_of(cudaStream), "DLGpuCross", FCross{b});
}
int DLGpuCrossBackward(const DLArrayHandle x, const DLArrayHandle y, const DLArrayHandle doutput, DLArrayHandle output, float b, void** cudaStream) {
  TF_SAME(x, y, "DLGpuCrossBackward"); TF_SAME(x, output, "DLGpuCrossBackward"); TF_SAME(x, doutput, "DLGpuCrossBackward");
  return run_map3(F(x), F(y), F(doutput), FM(output), numel(output), stream_of(cudaStream), "DLGpuCrossBackward", FCrossBwd{b});
}

static int concat_geom(const DLArrayHandle a, const DLArrayHandle b, int64_t* rows, int64_t* ia, int64_t* ib) {
  TF_REQUIRE(a && b && a->ndim == b->ndim && a->ndim >= 2, "concat: ranks differ");
  for (int i = 0; i < a->ndim; ++i) if (i != 1) TF_REQUIRE(a->shape[i] == b->shape[i], "concat: extents differ off axis 1");
  *rows = a->shape[0];
  *ia = *rows ? numel(a) / *rows : 0;
  *ib = *rows ? numel(b) / *rows : 0;
  return 0;
}
int DLGpuConcatForward(const DLArrayHandle input1, const DLArrayHandle input2, DLArrayHandle output, void** cudaStream) {
  int64_t rows, ia, ib;
  if (concat_geom(input1, input2, &rows, &ia, &ib)) return -1;
  TF_REQUIRE(output && numel(output) == rows * (ia + ib), "DLGpuConcatForward: output size mismatch");
  cudaStream_t s = stream_of(cudaStream);
  note_compute_stream(s);
  KernelTimer kt("DLGpuConcatForward", s, 0, 8.0 * rows * (ia + ib), 2);
  float* whole = FM(output);
  AmaxOut am = (rows > 0 && ia > 0 && ib > 0) ? amax_track_begin(whole) : AmaxOut{};
  launch_slice_copy<0>((float*)input1->data, whole, rows, ia, ia + ib, 0, s, am);
  am.clear = nullptr;
  launch_slice_copy<0>((float*)input2->data, whole, rows, ib, ia + ib, ia, s, am);
  if (after_launch(s, "DLGpuConcatForward", 2) != 0) return -1;
  return 0;
}
int DLGpuConcataBackward(const DLArrayHandle input1, const DLArrayHandle input2, const DLArrayHandle doutput, DLArrayHandle dinput1, void** cudaStream) {
  int64_t rows, ia, ib;
  if (concat_geom(input1, input2, &rows, &ia, &ib)) return -1;
  TF_REQUIRE(doutput && dinput1 && numel(doutput) == rows * (ia + ib) && numel(dinput1) == rows * ia, "DLGpuConcataBackward: size mismatch");
  cudaStream_t s = stream_of(cudaStream);
  note_compute_stream(s);
  KernelTimer kt("DLGpuConcatBackward", s, 0, 8.0 * rows * ia);
  float* part = FM(dinput1);
  launch_slice_copy<1>(part, (float*)doutput->data, rows, ia, ia + ib, 0, s, (rows > 0 && ia > 0) ? amax_track_begin(part) : AmaxOut{});
  TF_AFTER(s, "DLGpuConcataBackward");
  return 0;
}
int DLGpuConcatbBackward(const DLArrayHandle input1, const DLArrayHandle input2, const DLArrayHandle doutput, DLArrayHandle dinput2, void** cudaStream) {
  int64_t rows, ia, ib;
  if (concat_geom(input1, input2, &rows, &ia, &ib)) return -1;
  TF_REQUIRE(doutput && dinput2 && numel(doutput) == rows * (ia + ib) && numel(dinput2) == rows * ib, "DLGpuConcatbBackward: size mismatch");
  cudaStream_t s = stream_of(cudaStream);
  note_compute_stream(s);
  KernelTimer kt("DLGpuConcatBackward", s, 0, 8.0 * rows * ib);
  float* part = FM(dinput2);
  launch_slice_copy<1>(part, (float*)doutput->data, rows, ib, ia + ib, ia, s, (rows > 0 && ib > 0) ? amax_track_begin(part) : AmaxOut{});
  TF_AFTER(s, "DLGpuConcatbBackward");
  return 0;
}

// ---- activation ----------------------------------------------------------------------------
static int fill_tensor_plan(TensorPlan* p, const int* shapes, int n, int dataformat, int mode) {
  p->ndim = n; p->dataformat = dataformat; p->mode = mode;
  p->batch = shapes[0]; p->inner = 1;
  for (int i = 0; i < n; ++i) { p->dims[i] = shapes[i]; if (i) p->inner *= shapes[i]; }
  return 0;
}
int DLGpuActivationGetCudnnlist(const int* input_shapes, const int sizeofshape, int dataformat, int activationMode, void*** cudnnlist) {
  TF_REQUIRE(input_shapes && cudnnlist && sizeofshape >= 1 && sizeofshape <= 5, "DLGpuActivationGetCudnnlist: bad arguments");
  TF_REQUIRE(activationMode >= 0 && activationMode <= 3, "DLGpuActivationGetCudnnlist: unknown mode %d", activationMode);
  return fill_tensor_plan(new_plan<TensorPlan>(cudnnlist, kPlanTensor, 2), input_shapes, sizeofshape, dataformat, activationMode);
}
int DLGpuActivationForward(const DLArrayHandle input, DLArrayHandle output, int activationMode, void*** cudnnlist, void** cudnnHandle, void** cudaStream) {
  (void)cudnnHandle;
  TF_SAME(input, output, "DLGpuActivationForward");
  int64_t n = numel(input);
  if (activationMode == 1) {
    // the sum this ReLU reads was held back: one kernel writes the sum and its ReLU
    DeferredOp add;
    const cudaStream_t s_here = stream_of_keep_deferred(cudaStream);
    if (take_deferred(kDeferAdd, F(input), n, &add)) {
      // the slot is locked until release_deferred(): nothing below may call stream_of() / last_compute_stream()
      float* r = (float*)output->data;
      bool fused = false;
      if (add.stream == s_here && r != add.out && r != add.a && r != add.b) {
        note_write(r);
        fused = launch_add_relu(add, r, s_here);
      }
      if (!fused) launch_deferred_now(add);
      release_deferred();
      if (fused) {
        tc_note_relu_output(plan_of<TensorPlan>(cudnnlist, kPlanTensor), output->data);
        TF_AFTER(s_here, "DLGpuActivationForward(relu)");
        return 0;
      }
    }
  }
  cudaStream_t s = stream_of(cudaStream);
  switch (activationMode) {
    case 0: return run_map1(F(input), FM(output), n, s, "DLGpuActivationForward(sigmoid)", FSigmoid{});
    case 1: {
      // when the tensor path is known to pack this output for a convolution next, one kernel writes y and the pack
      const void* node = plan_of<TensorPlan>(cudnnlist, kPlanTensor);
      int fused = tc_fused_relu_pack(node, F(input), (float*)output->data, n, s);
      if (fused < 0) return -1;
      if (fused) return 0;
      int rc = run_map1(F(input), FM(output), n, s, "DLGpuActivationForward(relu)", FRelu{});
      tc_note_relu_output(node, output->data);
      return rc;
    }
    case 2: return run_map1(F(input), FM(output), n, s, "DLGpuActivationForward(tanh)", FTanh{});
    case 3: {
      // softmax over all non-batch elements of each sample (src/gpu_op.cu:3238-3248)
      TensorPlan* p = plan_of<TensorPlan>(cudnnlist, kPlanTensor);
      int64_t rows = p ? p->batch : input->shape[0];
      TF_REQUIRE(rows > 0 && n % rows == 0, "DLGpuActivationForward(softmax): bad batch extent");
      note_compute_stream(s);
      row_softmax_kernel<<<grid_for(rows * 32, kBlock), kBlock, 0, s>>>(F(input), FM(output), rows, n / rows);
      TF_AFTER(s, "DLGpuActivationForward(softmax)");
      return 0;
    }
  }
  TF_FAIL("DLGpuActivationForward: unknown mode %d", activationMode);
}
int DLGpuActivationBackward(const DLArrayHandle input, DLArrayHandle dinput, const DLArrayHandle output, const DLArrayHandle doutput,
                            int activationMode, void*** cudnnlist, void** cudnnHandle, void** cudaStream) {
  (void)cudnnHandle;
  TF_SAME(input, dinput, "DLGpuActivationBackward"); TF_SAME(input, output, "DLGpuActivationBackward"); TF_SAME(input, doutput, "DLGpuActivationBackward");
  cudaStream_t s = stream_of(cudaStream);
  int64_t n = numel(input);
  switch (activationMode) {
    case 0: return run_map2(F(output), F(doutput), FM(dinput), n, s, "DLGpuActivationBackward(sigmoid)", FSigmoidBwd{});
    case 1:
      // Held back for one call: if the batch-norm backward that consumes this gradient comes next, one kernel does both.
      if (deferral_enabled() && n >= (1 << 16)) {
        defer_op(DeferredOp{kDeferReluBwd, F(input), F(doutput), FM(dinput), n, s});
        return 0;
      }
      return run_map2(F(input), F(doutput), FM(dinput), n, s, "DLGpuActivationBackward(relu)", FReluGrad{});
    case 2: return run_map2(F(output), F(doutput), FM(dinput), n, s, "DLGpuActivationBackward(tanh)", FTanhBwd{});
    case 3: {
      TensorPlan* p = plan_of<TensorPlan>(cudnnlist, kPlanTensor);
      int64_t rows = p ? p->batch : input->shape[0];
      TF_REQUIRE(rows > 0 && n % rows == 0, "DLGpuActivationBackward(softmax): bad batch extent");
      note_compute_stream(s);
      row_softmax_bwd_kernel<<<grid_for(rows * 32, kBlock), kBlock, 0, s>>>(F(output), F(doutput), FM(dinput), rows, n / rows);
      TF_AFTER(s, "DLGpuActivationBackward(softmax)");
      return 0;
    }
  }
  TF_FAIL("DLGpuActivationBackward: unknown mode %d", activationMode);
}

// ---- dropout ------------------------------------------------------------------------------------
int DLGpuGetInputDescriptor(const int* input_shapes, const int sizeofshape, int dataformat, void*** inputd) {
  TF_REQUIRE(input_shapes && inputd && sizeofshape >= 1 && sizeofshape <= 5, "DLGpuGetInputDescriptor: bad arguments");
  return fill_tensor_plan(new_plan<TensorPlan>(inputd, kPlanTensor, 1), input_shapes, sizeofshape, dataformat, -1);
}
int DLGpuDropoutForward(const DLArrayHandle input, DLArrayHandle output, int dataformat, const float dropout, const int seed,
                        void** reserveSpace_p, void*** inputd, void*** cudnnlist, void** cudnnHandle, int* memorytoSaving, void** cudaStream) {
  (void)dataformat; (void)inputd; (void)cudnnHandle; (void)memorytoSaving;
  TF_SAME(input, output, "DLGpuDropoutForward");
  TF_REQUIRE(dropout >= 0.f && dropout < 1.f, "DLGpuDropoutForward: rate must be in [0,1)");
  TF_REQUIRE(cudnnlist, "DLGpuDropoutForward: null descriptor cell");
  DropoutState* st = new_plan<DropoutState>(cudnnlist, kPlanDropout, 2);
  st->p = dropout; st->seed = (unsigned long long)(unsigned)seed; st->count = numel(input);
  if (reserveSpace_p) *reserveSpace_p = st;
  cudaStream_t s = stream_of(cudaStream);
  note_compute_stream(s);
  KernelTimer kt("DLGpuDropoutForward", s, 0, 8.0 * st->count);
  dropout_kernel<<<grid_for(st->count, kBlock), kBlock, 0, s>>>(F(input), FM(output), st->count, dropout, 1.f / (1.f - dropout), st->seed);
  TF_AFTER(s, "DLGpuDropoutForward");
  return 0;
}
// Applies the forward call's mask to the gradient and releases the forward state
// (the reference frees its reserve space and descriptor list here, src/gpu_op.cu:3686-3690).
int DLGpuDropoutBackward(const DLArrayHandle doutput, DLArrayHandle dinput, void** reserveSpace_p, void*** cudnnlist, void** cudnnHandle, void** cudaStream) {
  (void)cudnnHandle; (void)reserveSpace_p;
  TF_SAME(doutput, dinput, "DLGpuDropoutBackward");
  DropoutState* st = plan_of<DropoutState>(cudnnlist, kPlanDropout);
  TF_REQUIRE(st && st->count == numel(doutput), "DLGpuDropoutBackward: no matching forward state");
  cudaStream_t s = stream_of(cudaStream);
  note_compute_stream(s);
  KernelTimer kt("DLGpuDropoutBackward", s, 0, 8.0 * st->count);
  dropout_kernel<<<grid_for(st->count, kBlock), kBlock, 0, s>>>(F(doutput), FM(dinput), st->count, st->p, 1.f / (1.f - st->p), st->seed);
  st->kind = 0;
  free(st);
  free(*cudnnlist);
  *cudnnlist = nullptr;
  TF_AFTER(s, "DLGpuDropoutBackward");
  return 0;
}

// ---- optimisers ------------------------------------------------------------------------------------
int DLGpuSgdUpdate(DLArrayHandle output, const DLArrayHandle m, float b, void** cudaStream) {
  TF_SAME(output, m, "DLGpuSgdUpdate");
  cudaStream_t s = stream_of(cudaStream);
  int took = dp_sgd_update(FM(output), F(m), numel(output), b, s);
  if (took < 0) return -1;
  if (took) return 0;
  return run_map2(F(output), F(m), FM(output), numel(output), s, "DLGpuSgdUpdate", FSgd{b});
}
int DLGpuAdam_mv(DLArrayHandle m, DLArrayHandle v, const DLArrayHandle g, float b1, float b2, void** cudaStream) {
  TF_SAME(m, g, "DLGpuAdam_mv"); TF_SAME(v, g, "DLGpuAdam_mv");
  cudaStream_t s = stream_of(cudaStream);
  int64_t n = numel(g);
  note_compute_stream(s);
  // data-parallel mode: the moments are computed from the gradient averaged over the ranks, after its all-reduce
  int took = dp_adam_moments(FM(m), FM(v), F(g), n, b1, b2, s);
  if (took < 0) return -1;
  if (took) return 0;
  adam_moments_kernel<<<grid_for(n, kBlock), kBlock, 0, s>>>(FM(m), FM(v), F(g), n, b1, b2);
  TF_AFTER(s, "DLGpuAdam_mv");
  return 0;
}
int DLGpuAdam(DLArrayHandle output, const DLArrayHandle m, const DLArrayHandle v, float b1t, float b2t, float e, float learning_rate, void** cudaStream) {
  TF_SAME(output, m, "DLGpuAdam"); TF_SAME(output, v, "DLGpuAdam");
  // data-parallel mode: the step joins the pending record of (m, v) and runs behind the all-reduce
  int took = dp_adam_step(FM(output), F(m), F(v), 1.f - b1t, 1.f - b2t, e, learning_rate, stream_of(cudaStream));
  if (took < 0) return -1;
  if (took) return 0;
  return run_map3(F(output), F(m), F(v), FM(output), numel(output), stream_of(cudaStream), "DLGpuAdam", FAdamStep{1.f - b1t, 1.f - b2t, e, learning_rate});
}

// Pointer tables for the multi-tensor optimisers.  `result` receives a 1- or 2-slot host array:
// slot 0 = device table, slot 1 = host copy of the sizes.  indexlist slot 0 = device prefix sums.
// The host keeps its own copy of the table: the tensors a multi-tensor update writes (the parameters, and Adam's
// moments) have to get a new write version at every update, or packed copies of the old weights would be reused.
struct PtrTable { int n; int groups; void** dev; void** host; };
static int build_table(void** const* cols, int ncols, int number, void**** result) {
  TF_REQUIRE(result && number > 0, "pointer table: bad arguments");
  PtrTable* t = new PtrTable{number, ncols, nullptr, nullptr};
  void** host = (void**)malloc(sizeof(void*) * number * ncols);
  for (int c = 0; c < ncols; ++c) for (int i = 0; i < number; ++i) host[c * number + i] = cols[c][i];
  t->dev = (void**)pool_alloc(sizeof(void*) * number * ncols);
  if (!t->dev) { free(host); delete t; TF_FAIL("pointer table: allocation failed"); }
  cudaError_t e = cudaMemcpy(t->dev, host, sizeof(void*) * number * ncols, cudaMemcpyHostToDevice);
  t->host = host;
  if (e != cudaSuccess) { free(host); pool_free(t->dev); delete t; TF_FAIL("pointer table: copy failed"); }
  void*** arr = (void***)malloc(sizeof(void**));
  arr[0] = (void**)t;
  *result = arr;
  return 0;
}
int DLGpuGetN2CudaPointer(void** output, void** g, int number, void**** result) { void** cols[2] = {output, g}; return build_table(cols, 2, number, result); }
int DLGpuGetN4CudaPointer(void** output, void** m, void** v, void** g, int number, void**** result) { void** cols[4] = {output, m, v, g}; return build_table(cols, 4, number, result); }
// `prefix` holds count+1 exclusive prefix sums of the tensor sizes; index_to_number is unused here
// (the kernels binary-search the prefix array instead of reading a per-element map).
struct IndexInfo { int count; int64_t total; int* dev_prefix; };
int DLGpuGetIndextoVaribaleNumberCudaPointer(int* index_to_number, int* prefix, int count, void*** result) {
  (void)index_to_number;
  TF_REQUIRE(prefix && result && count > 0, "index table: bad arguments");
  IndexInfo* info = new IndexInfo{count, prefix[count], nullptr};
  info->dev_prefix = (int*)pool_alloc(sizeof(int) * (count + 1));
  if (!info->dev_prefix) { delete info; TF_FAIL("index table: allocation failed"); }
  if (cudaMemcpy(info->dev_prefix, prefix, sizeof(int) * (count + 1), cudaMemcpyHostToDevice) != cudaSuccess) { delete info; TF_FAIL("index table: copy failed"); }
  void** arr = (void**)malloc(sizeof(void*));
  arr[0] = info;
  *result = arr;
  return 0;
}
int DLGpuSgd_o(void**** n2list, const void*** indexlist, const int count, const float learning_rate) {
  TF_REQUIRE(n2list && *n2list && indexlist && *indexlist, "DLGpuSgd_o: null table");
  PtrTable* t = (PtrTable*)(**n2list);
  IndexInfo* info = (IndexInfo*)((*indexlist)[0]);
  TF_REQUIRE(t && info && t->groups == 2 && t->n == info->count && (count == t->n || count == (int)info->total), "DLGpuSgd_o: tables do not match");
  cudaStream_t s = last_compute_stream();
  for (int i = 0; i < t->n; ++i) note_write(t->host[i]);                      // column 0: the parameters
  sgd_table_kernel<<<grid_for(info->total, kBlock), kBlock, 0, s>>>((float* const*)t->dev, (float* const*)(t->dev + t->n), info->dev_prefix, t->n, info->total, learning_rate);
  TF_AFTER(s, "DLGpuSgd_o");
  return 0;
}
int DLGpuAdam_o(void**** n4list, const void*** indexlist, const int count, const float b1, const float b2, const float b1t, const float b2t, const float e, const float learning_rate) {
  TF_REQUIRE(n4list && *n4list && indexlist && *indexlist, "DLGpuAdam_o: null table");
  PtrTable* t = (PtrTable*)(**n4list);
  IndexInfo* info = (IndexInfo*)((*indexlist)[0]);
  TF_REQUIRE(t && info && t->groups == 4 && t->n == info->count && (count == t->n || count == (int)info->total), "DLGpuAdam_o: tables do not match");
  cudaStream_t s = last_compute_stream();
  for (int i = 0; i < 3 * t->n; ++i) note_write(t->host[i]);                  // columns 0-2: parameters and both moments
  adam_table_kernel<<<grid_for(info->total, kBlock), kBlock, 0, s>>>((float* const*)t->dev, (float* const*)(t->dev + t->n), (float* const*)(t->dev + 2 * t->n), (float* const*)(t->dev + 3 * t->n),
                                                                     info->dev_prefix, t->n, info->total, b1, b2, 1.f - b1t, 1.f - b2t, e, learning_rate);
  TF_AFTER(s, "DLGpuAdam_o");
  return 0;
}

}  // extern "C"

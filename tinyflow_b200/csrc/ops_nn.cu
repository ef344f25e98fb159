// Pooling and batch normalisation (NCHW fp32), forward and backward.  HBM-bound: each
// tensor is read once and written once; statistics are reduced in registers / warp shuffles.
#include "common.h"
#include <math.h>

namespace tf {

// =====================================================================================
// Pooling.  Window semantics follow cuDNN as used by the reference (src/gpu_op.cu:2880-2983):
// output extent = 1 + (in + 2*pad - window) / stride; max ignores padded taps; average divides
// by the full window area (padding included).  Two documented choices where cuDNN's behaviour
// cannot be observed: a max window that covers only padding yields 0, and on ties the first
// maximum in row-major window order receives the gradient.
// =====================================================================================
// Division of a 32-bit unsigned number by a divisor fixed at launch time (multiply-high, add, two shifts: the
// round-up method for invariant divisors): flat indices are split into (plane, row, column) per element, and
// a hardware-emulated 64-bit divide per split made these kernels instruction-bound.
struct FastDiv {
  uint32_t d, m, s1, s2;
  __host__ void init(uint32_t div) {
    d = div ? div : 1;
    uint32_t l = 0;
    while ((1ull << l) < d) ++l;                         // ceil(log2 d)
    m = (uint32_t)((((1ull << 32) * ((1ull << l) - d)) / d) + 1);
    s1 = l < 1 ? l : 1; s2 = l > 1 ? l - 1 : 0;
  }
  __device__ __forceinline__ uint32_t div(uint32_t n) const {
    uint32_t t = __umulhi(m, n);
    return (t + ((n - t) >> s1)) >> s2;
  }
};
struct PoolGeom { int C, H, W, P, Q, ph, pw, sh, sw, kh, kw; FastDiv dHW, dW, dPQ, dQ, dsh, dsw; };

// flat index -> (plane, a, b) with a * width + b the offset inside a plane of `area` elements
__device__ __forceinline__ void split_index(int64_t i, const FastDiv& area, const FastDiv& width, int64_t& plane, int& a, int& b) {
  if (i <= 0xffffffffll) {
    uint32_t n = (uint32_t)i, pl = area.div(n), rem = n - pl * area.d, r = width.div(rem);
    plane = pl; a = (int)r; b = (int)(rem - r * width.d);
  } else {
    plane = i / area.d;
    int rem = (int)(i - plane * area.d);
    a = rem / (int)width.d; b = rem - a * (int)width.d;
  }
}
// windows p with p*stride - pad <= h < p*stride - pad + win, clipped to [0, count)
__device__ __forceinline__ void covering(int h, int pad, int win, int stride, const FastDiv& ds, int count, int& lo, int& hi) {
  int t = h + pad - win + 1;                             // first window start that still covers h, times nothing yet
  lo = t <= 0 ? 0 : (int)ds.div((uint32_t)(t + stride - 1));
  hi = min(count - 1, (int)ds.div((uint32_t)(h + pad)));
}

// KH, KW > 0 fix the window at compile time (all loads of a window are issued before the first compare);
// KH = 0 takes the window from the geometry.
template <int KH, int KW>
__device__ __forceinline__ int window_argmax(const float* __restrict__ plane, const PoolGeom& g, int p, int q, float* best_out) {
  const int h0 = p * g.sh - g.ph, w0 = q * g.sw - g.pw;
  int best = -1;
  float bv = 0.f;
  if (KH > 0) {
    // row / column validity once per window (KH + KW range checks instead of 4 per tap), one base pointer, constant offsets
    bool rv[KH > 0 ? KH : 1], cv[KW > 0 ? KW : 1];
#pragma unroll
    for (int r = 0; r < KH; ++r) rv[r] = (unsigned)(h0 + r) < (unsigned)g.H;
#pragma unroll
    for (int s = 0; s < KW; ++s) cv[s] = (unsigned)(w0 + s) < (unsigned)g.W;
    const int o0 = h0 * g.W + w0;
    const float* p0 = plane + o0;
    float v[KH > 0 ? KH * KW : 1];
#pragma unroll
    for (int r = 0; r < KH; ++r)
#pragma unroll
      for (int s = 0; s < KW; ++s) v[r * KW + s] = (rv[r] && cv[s]) ? __ldg(p0 + r * g.W + s) : 0.f;
#pragma unroll
    for (int r = 0; r < KH; ++r)
#pragma unroll
      for (int s = 0; s < KW; ++s)
        if (rv[r] && cv[s] && (best < 0 || v[r * KW + s] > bv)) { best = o0 + r * g.W + s; bv = v[r * KW + s]; }
  } else {
    for (int r = 0; r < g.kh; ++r) {
      int h = h0 + r;
      if (h < 0 || h >= g.H) continue;
      for (int s = 0; s < g.kw; ++s) {
        int w = w0 + s;
        if (w < 0 || w >= g.W) continue;
        float v = __ldg(plane + h * g.W + w);
        if (best < 0 || v > bv) { best = h * g.W + w; bv = v; }
      }
    }
  }
  *best_out = bv;
  return best;
}

template <int KH, int KW>
__global__ void __launch_bounds__(256) maxpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int32_t* __restrict__ idx, int64_t total, PoolGeom g, AmaxOut am) {
  grid_dep_sync();
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  uint32_t amax = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int64_t plane; int p, q;
    split_index(i, g.dPQ, g.dQ, plane, p, q);
    float v;
    int a = window_argmax<KH, KW>(x + plane * g.dHW.d, g, p, q, &v);
    v = a < 0 ? 0.f : v;
    if (y) y[i] = v;
    if (idx) idx[i] = a;
    amax = max(amax, amax_bits(v));
  }
  amax_commit(am, amax);
}
// Gather form of the max-pool gradient: each input element sums dy over the windows whose
// first maximum it is.  No atomics, deterministic, dx fully written.
__global__ void __launch_bounds__(256) maxpool_bwd_kernel(const float* __restrict__ x, const float* __restrict__ dy, float* __restrict__ dx, int64_t total, PoolGeom g) {
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int64_t plane; int h, w;
    split_index(i, g.dHW, g.dW, plane, h, w);
    const int hw = h * g.W + w;
    const float* xp = x + plane * g.dHW.d;
    const float* dp = dy + plane * g.dPQ.d;
    int p_lo, p_hi, q_lo, q_hi;
    covering(h, g.ph, g.kh, g.sh, g.dsh, g.P, p_lo, p_hi);
    covering(w, g.pw, g.kw, g.sw, g.dsw, g.Q, q_lo, q_hi);
    float acc = 0.f;
    for (int p = p_lo; p <= p_hi; ++p)
      for (int q = q_lo; q <= q_hi; ++q) {
        float v;
        if (window_argmax<0, 0>(xp, g, p, q, &v) == hw) acc += dp[p * g.Q + q];
      }
    dx[i] = acc;
  }
}
// Same gather with the forward pass's saved first-maximum indices (MAXPOOL) or plain summation (average pooling).
// NP x NQ bounds the windows that can cover one input element (ceil(window / stride) per axis, 0 = take the bounds
// at run time); with compile-time bounds all index and dy loads are issued before the first use.
template <bool MAXPOOL, int NP, int NQ>
__global__ void __launch_bounds__(256) pool_bwd_gather_kernel(const int32_t* __restrict__ idx, const float* __restrict__ dy, float* __restrict__ dx, int64_t total, float scale, PoolGeom g) {
  grid_dep_sync();
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int64_t plane; int h, w;
    split_index(i, g.dHW, g.dW, plane, h, w);
    const int hw = h * g.W + w;
    const int32_t* ip = idx + plane * g.dPQ.d;
    const float* dp = dy + plane * g.dPQ.d;
    int p_lo, p_hi, q_lo, q_hi;
    covering(h, g.ph, g.kh, g.sh, g.dsh, g.P, p_lo, p_hi);
    covering(w, g.pw, g.kw, g.sw, g.dsw, g.Q, q_lo, q_hi);
    float acc = 0.f;
    if (NP > 0) {
      float v[NP > 0 ? NP * NQ : 1];
      int id[NP > 0 ? NP * NQ : 1];
      bool pv[NP > 0 ? NP : 1], qv[NQ > 0 ? NQ : 1];
#pragma unroll
      for (int a = 0; a < NP; ++a) pv[a] = p_lo + a <= p_hi;
#pragma unroll
      for (int b = 0; b < NQ; ++b) qv[b] = q_lo + b <= q_hi;
      const int o0 = p_lo * g.Q + q_lo;
#pragma unroll
      for (int a = 0; a < NP; ++a)
#pragma unroll
        for (int b = 0; b < NQ; ++b) {
          const bool ok = pv[a] && qv[b];
          v[a * NQ + b] = ok ? __ldg(dp + o0 + a * g.Q + b) : 0.f;
          id[a * NQ + b] = MAXPOOL ? (ok ? __ldg(ip + o0 + a * g.Q + b) : -1) : hw;
        }
#pragma unroll
      for (int k = 0; k < NP * NQ; ++k) acc += id[k] == hw ? v[k] : 0.f;
    } else {
      for (int p = p_lo; p <= p_hi; ++p)
        for (int q = q_lo; q <= q_hi; ++q) {
          float v = __ldg(dp + p * g.Q + q);
          int id = MAXPOOL ? __ldg(ip + p * g.Q + q) : hw;
          acc += id == hw ? v : 0.f;
        }
    }
    dx[i] = acc * scale;
  }
}
// Max-pool gradient for 3x3 windows, stride 2, no padding (the ResNet / Inception stem pools): one thread per 2x2
// block of dx.  The four elements share their candidate windows (p in {a-1, a}, q in {b-1, b}), so the four index / dy
// pairs are loaded once instead of 2.25 times per element; contributions are added in the same (p, q) order as the
// general gather, so the result is bit-identical to it.
__global__ void __launch_bounds__(256) maxpool_bwd_3x3s2_kernel(const int32_t* __restrict__ idx, const float* __restrict__ dy, float* __restrict__ dx,
                                                                int64_t blocks_total, int H, int W, int P, int Q, FastDiv dAB, FastDiv dB) {
  grid_dep_sync();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int PQ = P * Q, HW = H * W;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < blocks_total; i += stride) {
    int64_t plane; int a, b;
    split_index(i, dAB, dB, plane, a, b);
    const int32_t* ip = idx + plane * PQ;
    const float* dp = dy + plane * PQ;
    float* xp = dx + plane * HW;
    int id[4]; float v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int p = a - 1 + (k >> 1), q = b - 1 + (k & 1);
      const bool ok = (unsigned)p < (unsigned)P && (unsigned)q < (unsigned)Q;
      id[k] = ok ? __ldg(ip + p * Q + q) : -1;
      v[k] = ok ? __ldg(dp + p * Q + q) : 0.f;
    }
    const int h0 = 2 * a, w0 = 2 * b;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int h = h0 + r;
      if (h >= H) break;
      float o[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int hw = h * W + w0 + c;
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) acc += id[k] == hw ? v[k] : 0.f;
        o[c] = acc;
      }
      if (w0 + 1 < W) {
        if ((W & 1) == 0) *reinterpret_cast<float2*>(xp + h * W + w0) = make_float2(o[0], o[1]);
        else { xp[h * W + w0] = o[0]; xp[h * W + w0 + 1] = o[1]; }
      } else {
        xp[h * W + w0] = o[0];
      }
    }
  }
}

// Max-pool gradient for 2x2 windows, stride 2, no padding (VGG, LeNet): windows do not overlap, so one thread owns
// one window: it reads its index and dy and writes the window's four dx elements (dy at the maximum, 0 elsewhere).
// Rows / columns of dx past the last window (odd extents) are zero-filled by the threads of the last window row / column.
__global__ void __launch_bounds__(256) maxpool_bwd_2x2s2_kernel(const int32_t* __restrict__ idx, const float* __restrict__ dy, float* __restrict__ dx,
                                                                int64_t total, int H, int W, int P, int Q, FastDiv dPQ, FastDiv dQ) {
  grid_dep_sync();
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int PQ = P * Q, HW = H * W;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int64_t plane; int p, q;
    split_index(i, dPQ, dQ, plane, p, q);
    const int id = __ldg(idx + plane * PQ + p * Q + q);
    const float v = __ldg(dy + plane * PQ + p * Q + q);
    float* xp = dx + plane * HW;
    const int h0 = 2 * p, w0 = 2 * q;
    const int h_end = p == P - 1 ? H : h0 + 2, w_end = q == Q - 1 ? W : w0 + 2;     // the last windows also clear the leftover edge
    for (int h = h0; h < h_end; ++h) {
      if (w_end == w0 + 2 && (W & 1) == 0) {
        const int hw = h * W + w0;
        *reinterpret_cast<float2*>(xp + hw) = make_float2(id == hw ? v : 0.f, id == hw + 1 ? v : 0.f);
      } else {
        for (int w = w0; w < w_end; ++w) xp[h * W + w] = id == h * W + w ? v : 0.f;
      }
    }
  }
}

template <int KH, int KW>
__global__ void __launch_bounds__(256) avgpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t total, PoolGeom g, AmaxOut am) {
  grid_dep_sync();
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  uint32_t amax = 0;
  float inv = 1.f / (float)(g.kh * g.kw);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    int64_t plane; int p, q;
    split_index(i, g.dPQ, g.dQ, plane, p, q);
    const float* xp = x + plane * g.dHW.d;
    int h0 = p * g.sh - g.ph, w0 = q * g.sw - g.pw;
    float acc = 0.f;
    if (KH > 0) {
      bool rv[KH > 0 ? KH : 1], cv[KW > 0 ? KW : 1];
#pragma unroll
      for (int r = 0; r < KH; ++r) rv[r] = (unsigned)(h0 + r) < (unsigned)g.H;
#pragma unroll
      for (int s = 0; s < KW; ++s) cv[s] = (unsigned)(w0 + s) < (unsigned)g.W;
      const float* p0 = xp + h0 * g.W + w0;
      float v[KH > 0 ? KH * KW : 1];
#pragma unroll
      for (int r = 0; r < KH; ++r)
#pragma unroll
        for (int s = 0; s < KW; ++s) v[r * KW + s] = (rv[r] && cv[s]) ? __ldg(p0 + r * g.W + s) : 0.f;
#pragma unroll
      for (int k = 0; k < KH * KW; ++k) acc += v[k];
    } else {
      for (int r = 0; r < g.kh; ++r) {
        int h = h0 + r;
        if (h < 0 || h >= g.H) continue;
        for (int s = 0; s < g.kw; ++s) {
          int w = w0 + s;
          if (w >= 0 && w < g.W) acc += __ldg(xp + h * g.W + w);
        }
      }
    }
    y[i] = acc * inv;
    amax = max(amax, amax_bits(acc * inv));
  }
  amax_commit(am, amax);
}

static PoolGeom geom_of(const PoolPlan* p) {
  PoolGeom g;
  g.C = p->C; g.H = p->H; g.W = p->W; g.P = p->P; g.Q = p->Q;
  g.ph = p->pad_h; g.pw = p->pad_w; g.sh = p->stride_h; g.sw = p->stride_w; g.kh = p->win_h; g.kw = p->win_w;
  g.dHW.init((uint32_t)(p->H * p->W)); g.dW.init((uint32_t)p->W); g.dPQ.init((uint32_t)(p->P * p->Q)); g.dQ.init((uint32_t)p->Q);
  g.dsh.init((uint32_t)p->stride_h); g.dsw.init((uint32_t)p->stride_w);
  return g;
}

static void launch_maxpool_fwd(const PoolPlan* p, const float* x, float* y, int32_t* idx, int64_t total, cudaStream_t s) {
  PoolGeom g = geom_of(p);
  int grid = grid_for(total, 256);
  AmaxOut am = y ? amax_track_begin(y) : AmaxOut{};
  if (p->win_h == 3 && p->win_w == 3) launch_dep(maxpool_fwd_kernel<3, 3>, dim3(grid), dim3(256), 0, s, x, y, idx, total, g, am);
  else if (p->win_h == 2 && p->win_w == 2) launch_dep(maxpool_fwd_kernel<2, 2>, dim3(grid), dim3(256), 0, s, x, y, idx, total, g, am);
  else if (p->win_h == 1 && p->win_w == 1) launch_dep(maxpool_fwd_kernel<1, 1>, dim3(grid), dim3(256), 0, s, x, y, idx, total, g, am);
  else launch_dep(maxpool_fwd_kernel<0, 0>, dim3(grid), dim3(256), 0, s, x, y, idx, total, g, am);
}
template <bool MAXPOOL> static void launch_pool_gather(const PoolPlan* p, const int32_t* idx, const float* dy, float* dx, int64_t total, float scale, cudaStream_t s) {
  PoolGeom g = geom_of(p);
  if (MAXPOOL && p->win_h == 3 && p->win_w == 3 && p->stride_h == 2 && p->stride_w == 2 && p->pad_h == 0 && p->pad_w == 0 &&
      (reinterpret_cast<uintptr_t>(dx) & 7) == 0) {
    const int A = (p->H + 1) / 2, B = (p->W + 1) / 2;
    const int64_t blocks = (int64_t)p->N * p->C * A * B;
    FastDiv dAB, dB;
    dAB.init((uint32_t)(A * B)); dB.init((uint32_t)B);
    launch_dep(maxpool_bwd_3x3s2_kernel, dim3(grid_for(blocks, 256)), dim3(256), 0, s, idx, dy, dx, blocks, p->H, p->W, p->P, p->Q, dAB, dB);
    return;
  }
  if (MAXPOOL && p->win_h == 2 && p->win_w == 2 && p->stride_h == 2 && p->stride_w == 2 && p->pad_h == 0 && p->pad_w == 0 &&
      p->P > 0 && p->Q > 0 && (reinterpret_cast<uintptr_t>(dx) & 7) == 0) {
    const int64_t windows = (int64_t)p->N * p->C * p->P * p->Q;
    launch_dep(maxpool_bwd_2x2s2_kernel, dim3(grid_for(windows, 256)), dim3(256), 0, s, idx, dy, dx, windows, p->H, p->W, p->P, p->Q, g.dPQ, g.dQ);
    return;
  }
  int grid = grid_for(total, 256);
  auto bound = [](int win, int stride, int count) { int n = (win + stride - 1) / stride; return n < count ? n : count; };
  int np = bound(p->win_h, p->stride_h, p->P), nq = bound(p->win_w, p->stride_w, p->Q);
  if (np == 1 && nq == 1) launch_dep(pool_bwd_gather_kernel<MAXPOOL, 1, 1>, dim3(grid), dim3(256), 0, s, idx, dy, dx, total, scale, g);
  else if (np <= 2 && nq <= 2) launch_dep(pool_bwd_gather_kernel<MAXPOOL, 2, 2>, dim3(grid), dim3(256), 0, s, idx, dy, dx, total, scale, g);
  else if (np <= 3 && nq <= 3) launch_dep(pool_bwd_gather_kernel<MAXPOOL, 3, 3>, dim3(grid), dim3(256), 0, s, idx, dy, dx, total, scale, g);
  else launch_dep(pool_bwd_gather_kernel<MAXPOOL, 0, 0>, dim3(grid), dim3(256), 0, s, idx, dy, dx, total, scale, g);
}

// =====================================================================================
// Batch normalisation with unit scale and zero bias, batch statistics, eps = 1e-5
// (src/gpu_op.cu:4224-4460).  Forward saves the mean and 1/sqrt(var+eps) it used; backward
// computes  dx = inv * (dy - mean(dy) - xhat * mean(dy * xhat))  with xhat = (x - mean) * inv.
//
// Per-activation mode: one statistic per (c,h,w) feature, reduced over the batch only.  A warp
// owns 32 consecutive 128-bit feature vectors (coalesced for every sample), the batch is split over the
// eight warps of the block, and every value stays in registers between the reduction and the apply
// pass, so x (and dy) cross HBM exactly once.
// =====================================================================================
constexpr float kBnEps = 1e-5f;
constexpr int kBnMaxBatchInRegs = 64;     // = kBnGroups * kBnPerThread

template <int VEC> struct VecT;
template <> struct VecT<1> { using type = float; };
template <> struct VecT<2> { using type = float2; };
template <> struct VecT<4> { using type = float4; };

// Block = 32 feature vectors x kBnGroups sample groups.  Thread (tx, ty) owns feature vector fv0 + tx and the
// samples ty, ty + kBnGroups, ...: each warp reads 32 consecutive feature vectors of one sample (coalesced),
// every thread keeps only N / kBnGroups values per tensor in registers, and the per-feature sums are combined
// across the sample groups through shared memory.
constexpr int kBnGroups = 8;
constexpr int kBnPerThread = 8;          // covers batches up to 64

template <int VEC>
__device__ __forceinline__ void bn_group_sum(float (&part)[VEC], float (*red)[32][VEC], int tx, int ty) {
#pragma unroll
  for (int k = 0; k < VEC; ++k) red[ty][tx][k] = part[k];
  __syncthreads();
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    float t = 0.f;
#pragma unroll
    for (int g = 0; g < kBnGroups; ++g) t += red[g][tx][k];
    part[k] = t;
  }
  __syncthreads();
}

template <int VEC>
__global__ void __launch_bounds__(32 * kBnGroups) bn_pa_fwd_regs_kernel(const float* __restrict__ x, float* __restrict__ y, float* __restrict__ save_mean, float* __restrict__ save_inv, int N, int64_t F, AmaxOut am) {
  grid_dep_sync();
  using V = typename VecT<VEC>::type;
  __shared__ float red[kBnGroups][32][VEC];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t FV = F / VEC;
  const int64_t fv = (int64_t)blockIdx.x * 32 + tx;
  const bool live = fv < FV;
  const V* xv = reinterpret_cast<const V*>(x);
  V* yv = reinterpret_cast<V*>(y);
  float v[kBnPerThread][VEC];
#pragma unroll
  for (int i = 0; i < kBnPerThread; ++i) {
    int n = ty + i * kBnGroups;
    V t = {};
    if (live && n < N) t = xv[(int64_t)n * FV + fv];
    const float* tp = reinterpret_cast<const float*>(&t);
#pragma unroll
    for (int k = 0; k < VEC; ++k) v[i][k] = tp[k];
  }
  const float rn = 1.f / (float)N;
  float mean[VEC], inv[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kBnPerThread; ++i) s += v[i][k];       // missing samples were loaded as 0
    mean[k] = s;
  }
  bn_group_sum<VEC>(mean, red, tx, ty);
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    mean[k] *= rn;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < kBnPerThread; ++i) { float d = v[i][k] - mean[k]; if (ty + i * kBnGroups < N) q += d * d; }
    inv[k] = q;
  }
  bn_group_sum<VEC>(inv, red, tx, ty);
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    float a = inv[k] * rn + kBnEps;
    float r = rsqrtf(a);
    inv[k] = r * (1.5f - 0.5f * a * r * r);       // one Newton step: full fp32 accuracy
  }
  uint32_t amax = 0;
#pragma unroll
  for (int i = 0; i < kBnPerThread; ++i) {
    int n = ty + i * kBnGroups;
    if (live && n < N) {
      V t;
      float* tp = reinterpret_cast<float*>(&t);
#pragma unroll
      for (int k = 0; k < VEC; ++k) { tp[k] = (v[i][k] - mean[k]) * inv[k]; amax = max(amax, amax_bits(tp[k])); }
      yv[(int64_t)n * FV + fv] = t;
    }
  }
  if (live && ty == 0) {
#pragma unroll
    for (int k = 0; k < VEC; ++k) { save_mean[fv * VEC + k] = mean[k]; save_inv[fv * VEC + k] = inv[k]; }
  }
  amax_commit(am, amax);        // max|y|: the activation that follows can pack its output for the next convolution in its own pass
}

template <int VEC>
__global__ void __launch_bounds__(32 * kBnGroups) bn_pa_bwd_regs_kernel(const float* __restrict__ x, const float* __restrict__ dy, float* __restrict__ dx, const float* __restrict__ save_mean, const float* __restrict__ save_inv, int N, int64_t F, AmaxOut am) {
  grid_dep_sync();
  using V = typename VecT<VEC>::type;
  __shared__ float red[kBnGroups][32][VEC];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t FV = F / VEC;
  const int64_t fv = (int64_t)blockIdx.x * 32 + tx;
  const bool live = fv < FV;
  const V* xv = reinterpret_cast<const V*>(x);
  const V* gv = reinterpret_cast<const V*>(dy);
  V* ov = reinterpret_cast<V*>(dx);
  float m[VEC], inv[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) { m[k] = live ? save_mean[fv * VEC + k] : 0.f; inv[k] = live ? save_inv[fv * VEC + k] : 0.f; }
  float xh[kBnPerThread][VEC], g[kBnPerThread][VEC];
#pragma unroll
  for (int i = 0; i < kBnPerThread; ++i) {
    int n = ty + i * kBnGroups;
    V a = {}, b = {};
    if (live && n < N) { a = xv[(int64_t)n * FV + fv]; b = gv[(int64_t)n * FV + fv]; }
    const float* ap = reinterpret_cast<const float*>(&a);
    const float* bp = reinterpret_cast<const float*>(&b);
#pragma unroll
    for (int k = 0; k < VEC; ++k) { xh[i][k] = (live && n < N) ? (ap[k] - m[k]) * inv[k] : 0.f; g[i][k] = bp[k]; }
  }
  float s1[VEC], s2[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int i = 0; i < kBnPerThread; ++i) { a += g[i][k]; b += g[i][k] * xh[i][k]; }
    s1[k] = a; s2[k] = b;
  }
  bn_group_sum<VEC>(s1, red, tx, ty);
  bn_group_sum<VEC>(s2, red, tx, ty);
  const float rn = 1.f / (float)N;
  uint32_t amax = 0;
#pragma unroll
  for (int i = 0; i < kBnPerThread; ++i) {
    int n = ty + i * kBnGroups;
    if (live && n < N) {
      V t;
      float* tp = reinterpret_cast<float*>(&t);
#pragma unroll
      for (int k = 0; k < VEC; ++k) { tp[k] = inv[k] * (g[i][k] - s1[k] * rn - xh[i][k] * s2[k] * rn); amax = max(amax, amax_bits(tp[k])); }
      ov[(int64_t)n * FV + fv] = t;
    }
  }
  amax_commit(am, amax);
}

// ReLU backward and the batch-norm backward behind it in one pass: g = (mask > 0 ? dy : 0) is the ReLU's gradient (stored
// to dg: other consumers of that tensor may exist) and the batch-norm's incoming gradient.  XHAT_MASK: the ReLU's input
// is this layer's own forward output, which equals x-hat bit for bit (same subtraction and product of the same saved
// statistics), so the mask tensor is not read at all.
template <int VEC, bool XHAT_MASK>
__global__ void __launch_bounds__(32 * kBnGroups) bn_pa_bwd_relu_regs_kernel(const float* __restrict__ x, const float* __restrict__ dy, const float* __restrict__ mask, float* __restrict__ dg, float* __restrict__ dx, const float* __restrict__ save_mean, const float* __restrict__ save_inv, int N, int64_t F, AmaxOut am) {
  grid_dep_sync();
  using V = typename VecT<VEC>::type;
  __shared__ float red[kBnGroups][32][VEC];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t FV = F / VEC;
  const int64_t fv = (int64_t)blockIdx.x * 32 + tx;
  const bool live = fv < FV;
  const V* xv = reinterpret_cast<const V*>(x);
  const V* gv = reinterpret_cast<const V*>(dy);
  const V* mv = reinterpret_cast<const V*>(mask);
  V* dgv = reinterpret_cast<V*>(dg);
  V* ov = reinterpret_cast<V*>(dx);
  float m[VEC], inv[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) { m[k] = live ? save_mean[fv * VEC + k] : 0.f; inv[k] = live ? save_inv[fv * VEC + k] : 0.f; }
  float xh[kBnPerThread][VEC], g[kBnPerThread][VEC];
#pragma unroll
  for (int i = 0; i < kBnPerThread; ++i) {
    const int n = ty + i * kBnGroups;
    const bool on = live && n < N;
    V a = {}, b = {}, r = {};
    if (on) {
      a = xv[(int64_t)n * FV + fv]; b = gv[(int64_t)n * FV + fv];
      if (!XHAT_MASK) r = mv[(int64_t)n * FV + fv];
    }
    const float* ap = reinterpret_cast<const float*>(&a);
    const float* bp = reinterpret_cast<const float*>(&b);
    const float* rp = reinterpret_cast<const float*>(&r);
    V t;
    float* tp = reinterpret_cast<float*>(&t);
#pragma unroll
    for (int k = 0; k < VEC; ++k) {
      xh[i][k] = on ? (ap[k] - m[k]) * inv[k] : 0.f;
      const float sel = XHAT_MASK ? xh[i][k] : rp[k];
      g[i][k] = sel > 0.f ? bp[k] : 0.f;
      tp[k] = g[i][k];
    }
    if (on) dgv[(int64_t)n * FV + fv] = t;
  }
  float s1[VEC], s2[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) {
    float a = 0.f, b = 0.f;
#pragma unroll
    for (int i = 0; i < kBnPerThread; ++i) { a += g[i][k]; b += g[i][k] * xh[i][k]; }
    s1[k] = a; s2[k] = b;
  }
  bn_group_sum<VEC>(s1, red, tx, ty);
  bn_group_sum<VEC>(s2, red, tx, ty);
  const float rn = 1.f / (float)N;
  uint32_t amax = 0;
#pragma unroll
  for (int i = 0; i < kBnPerThread; ++i) {
    int n = ty + i * kBnGroups;
    if (live && n < N) {
      V t;
      float* tp = reinterpret_cast<float*>(&t);
#pragma unroll
      for (int k = 0; k < VEC; ++k) { tp[k] = inv[k] * (g[i][k] - s1[k] * rn - xh[i][k] * s2[k] * rn); amax = max(amax, amax_bits(tp[k])); }
      ov[(int64_t)n * FV + fv] = t;
    }
  }
  amax_commit(am, amax);
}

// Any batch size: three passes over the batch column (the re-reads are served by L2).
__global__ void __launch_bounds__(128) bn_pa_fwd_loop_kernel(const float* __restrict__ x, float* __restrict__ y, float* __restrict__ save_mean, float* __restrict__ save_inv, int N, int64_t F) {
  int64_t f = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (f >= F) return;
  float rn = 1.f / (float)N, s = 0.f, q = 0.f;
  for (int n = 0; n < N; ++n) s += x[(int64_t)n * F + f];
  float m = s * rn;
  for (int n = 0; n < N; ++n) { float d = x[(int64_t)n * F + f] - m; q += d * d; }
  float inv = 1.f / sqrtf(q * rn + kBnEps);
  for (int n = 0; n < N; ++n) y[(int64_t)n * F + f] = (x[(int64_t)n * F + f] - m) * inv;
  save_mean[f] = m; save_inv[f] = inv;
}
__global__ void __launch_bounds__(128) bn_pa_bwd_loop_kernel(const float* __restrict__ x, const float* __restrict__ dy, float* __restrict__ dx, const float* __restrict__ save_mean, const float* __restrict__ save_inv, int N, int64_t F) {
  int64_t f = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (f >= F) return;
  float m = save_mean[f], inv = save_inv[f], s1 = 0.f, s2 = 0.f, rn = 1.f / (float)N;
  for (int n = 0; n < N; ++n) { float g = dy[(int64_t)n * F + f]; s1 += g; s2 += g * (x[(int64_t)n * F + f] - m) * inv; }
  s1 *= rn; s2 *= rn;
  for (int n = 0; n < N; ++n) dx[(int64_t)n * F + f] = inv * (dy[(int64_t)n * F + f] - s1 - (x[(int64_t)n * F + f] - m) * inv * s2);
}

// Spatial mode: one statistic per channel over N*H*W.  One block per channel.
__device__ __forceinline__ float bsum(float v, float* red) {
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < nw ? red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__global__ void __launch_bounds__(512) bn_sp_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, float* __restrict__ save_mean, float* __restrict__ save_inv, int64_t N, int64_t C, int64_t HW) {
  __shared__ float red[33];
  int64_t c = blockIdx.x, cnt = N * HW;
  float s = 0.f;
  for (int64_t i = threadIdx.x; i < cnt; i += blockDim.x) s += x[((i / HW) * C + c) * HW + i % HW];
  float m = bsum(s, red) / (float)cnt, q = 0.f;
  for (int64_t i = threadIdx.x; i < cnt; i += blockDim.x) { float d = x[((i / HW) * C + c) * HW + i % HW] - m; q += d * d; }
  float inv = 1.f / sqrtf(bsum(q, red) / (float)cnt + kBnEps);
  for (int64_t i = threadIdx.x; i < cnt; i += blockDim.x) { int64_t o = ((i / HW) * C + c) * HW + i % HW; y[o] = (x[o] - m) * inv; }
  if (threadIdx.x == 0) { save_mean[c] = m; save_inv[c] = inv; }
}
__global__ void __launch_bounds__(512) bn_sp_bwd_kernel(const float* __restrict__ x, const float* __restrict__ dy, float* __restrict__ dx, const float* __restrict__ save_mean, const float* __restrict__ save_inv, int64_t N, int64_t C, int64_t HW) {
  __shared__ float red[33];
  int64_t c = blockIdx.x, cnt = N * HW;
  float m = save_mean[c], inv = save_inv[c], s1 = 0.f, s2 = 0.f;
  for (int64_t i = threadIdx.x; i < cnt; i += blockDim.x) { int64_t o = ((i / HW) * C + c) * HW + i % HW; float g = dy[o]; s1 += g; s2 += g * (x[o] - m) * inv; }
  s1 = bsum(s1, red) / (float)cnt;
  s2 = bsum(s2, red) / (float)cnt;
  for (int64_t i = threadIdx.x; i < cnt; i += blockDim.x) { int64_t o = ((i / HW) * C + c) * HW + i % HW; dx[o] = inv * (dy[o] - s1 - (x[o] - m) * inv * s2); }
}

static void launch_bn_fwd_regs(const float* x, float* y, float* sm, float* si, int N, int64_t F, cudaStream_t s) {
  AmaxOut am = amax_track_begin(y);
  if (F % 4 == 0 && aligned16(x) && aligned16(y)) launch_dep(bn_pa_fwd_regs_kernel<4>, dim3((unsigned)((F / 4 + 31) / 32)), dim3(32 * kBnGroups), 0, s, x, y, sm, si, N, F, am);
  else launch_dep(bn_pa_fwd_regs_kernel<1>, dim3((unsigned)((F + 31) / 32)), dim3(32 * kBnGroups), 0, s, x, y, sm, si, N, F, am);
}
static void launch_bn_bwd_regs(const float* x, const float* dy, float* dx, const float* sm, const float* si, int N, int64_t F, cudaStream_t s) {
  AmaxOut am = amax_track_begin(dx);          // dx is the output gradient of the convolution in front of this layer
  // 8-byte vectors: the 16-byte variant holds 2 x 8 x 4 values per thread (126 registers, two blocks per SM) and its
  // load / reduce / store phases overlap too little; with half the registers three blocks fit (1.89 -> 1.77 ms per
  // ResNet-50 step)
  if (F % 2 == 0 && aligned16(x) && aligned16(dy) && aligned16(dx)) launch_dep(bn_pa_bwd_regs_kernel<2>, dim3((unsigned)((F / 2 + 31) / 32)), dim3(32 * kBnGroups), 0, s, x, dy, dx, sm, si, N, F, am);
  else if (F % 4 == 0 && aligned16(x) && aligned16(dy) && aligned16(dx)) launch_dep(bn_pa_bwd_regs_kernel<4>, dim3((unsigned)((F / 4 + 31) / 32)), dim3(32 * kBnGroups), 0, s, x, dy, dx, sm, si, N, F, am);
  else launch_dep(bn_pa_bwd_regs_kernel<1>, dim3((unsigned)((F + 31) / 32)), dim3(32 * kBnGroups), 0, s, x, dy, dx, sm, si, N, F, am);
}
// The fused pair (a held-back ReLU backward and this batch-norm backward).  Returns false when the operands do not allow
// 8-byte vectors; the caller then runs the two kernels one after the other.
static bool launch_bn_bwd_relu_regs(const float* x, const float* dy, const float* mask, bool xhat_mask, float* dg, float* dx, const float* sm, const float* si, int N, int64_t F, cudaStream_t s) {
  if (!(F % 2 == 0 && aligned16(x) && aligned16(dy) && aligned16(mask) && aligned16(dg) && aligned16(dx))) return false;
  AmaxOut am = amax_track_begin(dx);
  const dim3 grid((unsigned)((F / 2 + 31) / 32)), block(32 * kBnGroups);
  if (xhat_mask) launch_dep(bn_pa_bwd_relu_regs_kernel<2, true>, grid, block, 0, s, x, dy, mask, dg, dx, sm, si, N, F, am);
  else launch_dep(bn_pa_bwd_relu_regs_kernel<2, false>, grid, block, 0, s, x, dy, mask, dg, dx, sm, si, N, F, am);
  return true;
}
static std::atomic<long long> g_fused_relu_bn_bwd{0};
long long fused_relu_bn_bwd_count() { return g_fused_relu_bn_bwd.load(); }

}  // namespace tf

using namespace tf;

extern "C" {

int DLGpuPooling2DForwardGetOutShape(const int* input_shapes, int* output_shapes, int dataformat, int poolingMode,
                                     const int padding_h, const int padding_w, const int u, const int v,
                                     const int filter_h, const int filter_w, void*** cudnnlist) {
  TF_REQUIRE(input_shapes && output_shapes && cudnnlist, "DLGpuPooling2DForwardGetOutShape: null argument");
  TF_REQUIRE(u > 0 && v > 0 && filter_h > 0 && filter_w > 0 && padding_h >= 0 && padding_w >= 0, "DLGpuPooling2DForwardGetOutShape: bad window");
  TF_REQUIRE(poolingMode == 0 || poolingMode == 1, "DLGpuPooling2DForwardGetOutShape: unknown mode %d", poolingMode);
  PoolPlan* p = new_plan<PoolPlan>(cudnnlist, kPlanPool, 3);
  p->dataformat = dataformat; p->mode = poolingMode;
  p->N = input_shapes[0];
  if (dataformat == 0) { p->C = input_shapes[1]; p->H = input_shapes[2]; p->W = input_shapes[3]; }
  else { p->C = input_shapes[3]; p->H = input_shapes[1]; p->W = input_shapes[2]; }
  p->pad_h = padding_h; p->pad_w = padding_w; p->stride_h = u; p->stride_w = v; p->win_h = filter_h; p->win_w = filter_w;
  p->P = 1 + (p->H + 2 * padding_h - filter_h) / u;
  p->Q = 1 + (p->W + 2 * padding_w - filter_w) / v;
  TF_REQUIRE(p->P > 0 && p->Q > 0, "DLGpuPooling2DForwardGetOutShape: window larger than padded input");
  output_shapes[0] = p->N;
  if (dataformat == 0) { output_shapes[1] = p->C; output_shapes[2] = p->P; output_shapes[3] = p->Q; }
  else { output_shapes[1] = p->P; output_shapes[2] = p->Q; output_shapes[3] = p->C; }
  return 0;
}

static int check_pool(const PoolPlan* p, const DLArrayHandle in, const DLArrayHandle out, const char* what) {
  TF_REQUIRE(p, "%s: descriptor was not built by DLGpuPooling2DForwardGetOutShape", what);
  TF_REQUIRE(p->dataformat == 0, "%s: only NCHW is implemented", what);
  TF_REQUIRE(in && numel(in) == (int64_t)p->N * p->C * p->H * p->W, "%s: input does not match the descriptor", what);
  TF_REQUIRE(out && numel(out) == (int64_t)p->N * p->C * p->P * p->Q, "%s: output does not match the descriptor", what);
  return 0;
}

int DLGpuPooling2DForward(const DLArrayHandle input, DLArrayHandle output, void*** cudnnlist, void** cudnnHandle, void** cudaStream) {
  (void)cudnnHandle;
  PoolPlan* p = plan_of<PoolPlan>(cudnnlist, kPlanPool);
  if (check_pool(p, input, output, "DLGpuPooling2DForward")) return -1;
  cudaStream_t s = stream_of(cudaStream);
  int64_t total = numel(output);
  note_compute_stream(s);
  if (p->mode == 0 && !p->argmax) p->argmax = (int32_t*)pool_alloc(sizeof(int32_t) * (size_t)total);   // optional: backward rescans if absent
  KernelTimer kt("DLGpuPooling2DForward", s, 0, 4.0 * (numel(input) + numel(output)));
  if (p->mode == 0) {
    launch_maxpool_fwd(p, (const float*)input->data, out_f32(output), p->argmax, total, s);
    p->argmax_src = input->data;
    p->argmax_version = version_of(input->data);
  }
  else {
    float* y = out_f32(output);
    AmaxOut am = amax_track_begin(y);
    if (p->win_h == 3 && p->win_w == 3) launch_dep(avgpool_fwd_kernel<3, 3>, dim3(grid_for(total, 256)), dim3(256), 0, s, (const float*)input->data, y, total, geom_of(p), am);
    else launch_dep(avgpool_fwd_kernel<0, 0>, dim3(grid_for(total, 256)), dim3(256), 0, s, (const float*)input->data, y, total, geom_of(p), am);
  }
  TF_AFTER(s, "DLGpuPooling2DForward");
  return 0;
}

int DLGpuPooling2DBackward(const DLArrayHandle input, const DLArrayHandle output, const DLArrayHandle doutput, DLArrayHandle dinput,
                           void*** cudnnlist, void** cudnnHandle, void** cudaStream) {
  (void)cudnnHandle;
  PoolPlan* p = plan_of<PoolPlan>(cudnnlist, kPlanPool);
  if (check_pool(p, input, output, "DLGpuPooling2DBackward")) return -1;
  TF_REQUIRE(doutput && dinput && numel(doutput) == numel(output) && numel(dinput) == numel(input), "DLGpuPooling2DBackward: gradient sizes do not match");
  cudaStream_t s = stream_of(cudaStream);
  int64_t total = numel(dinput);
  note_compute_stream(s);
  KernelTimer kt("DLGpuPooling2DBackward", s, 0, 4.0 * ((p->mode == 0 ? 2 : 1) * numel(input) + numel(output)));
  if (p->mode == 0) {
    if (p->argmax && p->argmax_src == input->data && p->argmax_version == version_of(input->data))
      launch_pool_gather<true>(p, p->argmax, (const float*)doutput->data, out_f32(dinput), total, 1.f, s);
    else
      maxpool_bwd_kernel<<<grid_for(total, 256), 256, 0, s>>>((const float*)input->data, (const float*)doutput->data, out_f32(dinput), total, geom_of(p));
  }
  else launch_pool_gather<false>(p, nullptr, (const float*)doutput->data, out_f32(dinput), total, 1.f / (float)(p->win_h * p->win_w), s);
  TF_AFTER(s, "DLGpuPooling2DBackward");
  return 0;
}

int TfPoolingArgmax(const DLArrayHandle input, int32_t* indices_dev, void*** cudnnlist, void** cudaStream) {
  PoolPlan* p = plan_of<PoolPlan>(cudnnlist, kPlanPool);
  TF_REQUIRE(p && p->dataformat == 0 && input && indices_dev && numel(input) == (int64_t)p->N * p->C * p->H * p->W, "TfPoolingArgmax: bad arguments");
  cudaStream_t s = stream_of(cudaStream);
  int64_t total = (int64_t)p->N * p->C * p->P * p->Q;
  note_compute_stream(s);
  launch_maxpool_fwd(p, (const float*)input->data, nullptr, indices_dev, total, s);
  TF_AFTER(s, "TfPoolingArgmax");
  return 0;
}

// ---- batch normalisation --------------------------------------------------------------------
int DLGpuBatchNormalizationGetCudnnlist(const int* input_shapes, int sizeofshape, int dataformat, int batchNormMode,
                                        void** mean_p, void** Variance_p, void*** cudnnlist) {
  (void)mean_p; (void)Variance_p;
  TF_REQUIRE(input_shapes && cudnnlist && sizeofshape >= 2 && sizeofshape <= 5, "DLGpuBatchNormalizationGetCudnnlist: bad arguments");
  TF_REQUIRE(batchNormMode == 0 || batchNormMode == 1, "DLGpuBatchNormalizationGetCudnnlist: unknown mode %d", batchNormMode);
  TF_REQUIRE(dataformat == 0 || batchNormMode == 0, "DLGpuBatchNormalizationGetCudnnlist: spatial mode is implemented for NCHW only");
  BNPlan* p = new_plan<BNPlan>(cudnnlist, kPlanBN, 3);
  p->mode = batchNormMode;
  p->N = input_shapes[0];
  // channel axis: dim 1 for NCHW, last dim for NHWC
  int64_t rest = 1;
  for (int i = 1; i < sizeofshape; ++i) rest *= input_shapes[i];
  p->C = dataformat == 0 ? input_shapes[1] : input_shapes[sizeofshape - 1];
  p->HW = p->C ? rest / p->C : 0;
  p->nstat = batchNormMode == 0 ? rest : p->C;
  return 0;
}

static int bn_buffers(BNPlan* p, int* memorytoSaving) {
  if (p->save_mean) return 0;
  size_t bytes = sizeof(float) * (size_t)p->nstat;
  p->save_mean = (float*)pool_alloc(bytes);
  p->save_inv = p->save_mean ? (float*)pool_alloc(bytes) : nullptr;
  if (!p->save_inv) {
    if (p->save_mean) { pool_free(p->save_mean); p->save_mean = nullptr; }
    if (memorytoSaving) *memorytoSaving = (int)bytes;
    return 1;
  }
  return 0;
}

int DLGpuBatchNormalizationForward(const DLArrayHandle input, DLArrayHandle output, int batchNormMode, int n, void** mean_p, void** Variance_p,
                                   void*** cudnnlist, void** cudnnHandle, int* memorytoSaving, void** cudaStream) {
  (void)n; (void)cudnnHandle;
  BNPlan* p = plan_of<BNPlan>(cudnnlist, kPlanBN);
  TF_REQUIRE(p && p->mode == batchNormMode, "DLGpuBatchNormalizationForward: descriptor / mode mismatch");
  TF_REQUIRE(input && output && numel(input) == numel(output) && numel(input) == p->N * p->C * p->HW, "DLGpuBatchNormalizationForward: arrays do not match the descriptor");
  if (bn_buffers(p, memorytoSaving)) return 0;    // soft out-of-memory
  if (mean_p) *mean_p = p->save_mean;
  if (Variance_p) *Variance_p = p->save_inv;
  cudaStream_t s = stream_of(cudaStream);
  const float* x = (const float*)input->data;
  float* y = out_f32(output);
  note_compute_stream(s);
  KernelTimer kt("DLGpuBatchNormalizationForward", s, 0, 8.0 * numel(input) + 8.0 * p->nstat);
  if (p->mode == 0) {
    int64_t F = p->nstat;
    int N = (int)p->N;
    p->last_y = y; p->last_y_version = version_of(y);
    if (N <= kBnMaxBatchInRegs) launch_bn_fwd_regs(x, y, p->save_mean, p->save_inv, N, F, s);
    else bn_pa_fwd_loop_kernel<<<(unsigned)((F + 127) / 128), 128, 0, s>>>(x, y, p->save_mean, p->save_inv, N, F);
  } else {
    bn_sp_fwd_kernel<<<(unsigned)p->C, 512, 0, s>>>(x, y, p->save_mean, p->save_inv, p->N, p->C, p->HW);
  }
  TF_AFTER(s, "DLGpuBatchNormalizationForward");
  return 0;
}

int DLGpuBatchNormalizationBackward(const DLArrayHandle input, const DLArrayHandle doutput, DLArrayHandle dinput, int batchNormMode,
                                    void** mean_p, void** Variance_p, void*** cudnnlist, void** cudnnHandle, int* memorytoSaving, void** cudaStream) {
  (void)mean_p; (void)Variance_p; (void)cudnnHandle; (void)memorytoSaving;
  BNPlan* p = plan_of<BNPlan>(cudnnlist, kPlanBN);
  TF_REQUIRE(p && p->mode == batchNormMode, "DLGpuBatchNormalizationBackward: descriptor / mode mismatch");
  TF_REQUIRE(p->save_mean && p->save_inv, "DLGpuBatchNormalizationBackward: forward has not run for this descriptor");
  TF_REQUIRE(input && doutput && dinput && numel(input) == p->N * p->C * p->HW && numel(doutput) == numel(input) && numel(dinput) == numel(input), "DLGpuBatchNormalizationBackward: arrays do not match the descriptor");
  const float* x = (const float*)input->data;
  const float* dy = (const float*)doutput->data;
  // A ReLU backward that was held back and whose output is this call's incoming gradient runs inside this kernel.
  DeferredOp relu;
  const cudaStream_t s_here = stream_of_keep_deferred(cudaStream);
  if (p->mode == 0 && p->N <= kBnMaxBatchInRegs && take_deferred(kDeferReluBwd, (const float*)dy, numel(input), &relu)) {
    // the slot is locked until release_deferred(): nothing below may call stream_of() / last_compute_stream()
    bool fused = false;
    float* dx_f = (float*)dinput->data;
    if (relu.stream == s_here && dx_f != relu.out && dx_f != relu.b && dx_f != relu.a && dx_f != x) {
      note_write(dx_f);
      note_compute_stream(s_here);
      // mask from x-hat when the ReLU's input is still exactly this layer's forward output
      const bool xhat_mask = relu.a == p->last_y && version_of(relu.a) == p->last_y_version;
      KernelTimer kt("ReluBackward+BatchNormalizationBackward", s_here, 0, (xhat_mask ? 16.0 : 20.0) * numel(input) + 8.0 * p->nstat);
      fused = launch_bn_bwd_relu_regs(x, relu.b, relu.a, xhat_mask, relu.out, dx_f, p->save_mean, p->save_inv, (int)p->N, p->nstat, s_here);
    }
    if (!fused) launch_deferred_now(relu);      // not a shape the fused kernel handles: the ReLU on its own, then as usual
    release_deferred();
    if (fused) {
      g_fused_relu_bn_bwd.fetch_add(1);
      TF_AFTER(s_here, "DLGpuBatchNormalizationBackward");
      return 0;
    }
  }
  cudaStream_t s = stream_of(cudaStream);
  float* dx = out_f32(dinput);
  note_compute_stream(s);
  KernelTimer kt("DLGpuBatchNormalizationBackward", s, 0, 12.0 * numel(input) + 8.0 * p->nstat);
  if (p->mode == 0) {
    int64_t F = p->nstat;
    int N = (int)p->N;
    unsigned grid = (unsigned)((F + 127) / 128);
    if (N <= kBnMaxBatchInRegs) launch_bn_bwd_regs(x, dy, dx, p->save_mean, p->save_inv, N, F, s);
    else bn_pa_bwd_loop_kernel<<<grid, 128, 0, s>>>(x, dy, dx, p->save_mean, p->save_inv, N, F);
  } else {
    bn_sp_bwd_kernel<<<(unsigned)p->C, 512, 0, s>>>(x, dy, dx, p->save_mean, p->save_inv, p->N, p->C, p->HW);
  }
  TF_AFTER(s, "DLGpuBatchNormalizationBackward");
  return 0;
}

}  // extern "C"

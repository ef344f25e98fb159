// CUDA-core (fp32 FMA) implicit-GEMM contraction kernels: matmul with either operand
// transposed, convolution forward, backward-data and backward-filter for any window, stride
// and padding.  This is the exact-fp32 general path; it serves the shapes the tensor-core
// path does not take (tiny channel counts, strided backward-data, very small problems) and is
// the cross-check for the tcgen05 kernels.
//
// One kernel template: C[M x N] += A[M x K] * B[K x N] on 64x64x16 tiles, 256 threads, a 4x4
// register micro-tile per thread.  Operand elements are fetched through small "view" structs
// that turn (row, k) / (k, col) into a tensor address or a padded zero, so convolution never
// materialises an im2col matrix.
#include "common.h"

namespace tf {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

// ---- operand views -----------------------------------------------------------------------
struct MatView {            // plain row-major matrix, optionally read transposed
  const float* p; int64_t ld; int trans;
  __device__ __forceinline__ float at(int64_t r, int64_t c) const { return trans ? p[c * ld + r] : p[r * ld + c]; }
};
struct ConvGeom {
  int N, C, H, W, K, R, S, P, Q, ph, pw, sh, sw;
};
// forward:  A = filter [K x CRS],  B = im2col(x) [CRS x NPQ]
struct FwdA { const float* w; int64_t CRS; __device__ __forceinline__ float at(int64_t m, int64_t k) const { return w[m * CRS + k]; } };
struct FwdB {
  const float* x; ConvGeom g;
  __device__ __forceinline__ float at(int64_t k, int64_t j) const {
    int RS = g.R * g.S, PQ = g.P * g.Q;
    int c = (int)(k / RS), rs = (int)(k % RS), r = rs / g.S, s = rs % g.S;
    int n = (int)(j / PQ), pq = (int)(j % PQ), p = pq / g.Q, q = pq % g.Q;
    int h = p * g.sh + r - g.ph, w = q * g.sw + s - g.pw;
    if (h < 0 || h >= g.H || w < 0 || w >= g.W) return 0.f;
    return x[(((int64_t)n * g.C + c) * g.H + h) * g.W + w];
  }
};
// backward-data:  A = filter^T [C x KRS],  B = scattered dy [KRS x NHW]
struct DgradA {
  const float* w; ConvGeom g;
  __device__ __forceinline__ float at(int64_t m, int64_t kk) const {
    int RS = g.R * g.S;
    int k = (int)(kk / RS), rs = (int)(kk % RS);
    return w[((int64_t)k * g.C + m) * RS + rs];
  }
};
struct DgradB {
  const float* dy; ConvGeom g;
  __device__ __forceinline__ float at(int64_t kk, int64_t j) const {
    int RS = g.R * g.S, HW = g.H * g.W;
    int k = (int)(kk / RS), rs = (int)(kk % RS), r = rs / g.S, s = rs % g.S;
    int n = (int)(j / HW), hw = (int)(j % HW), h = hw / g.W, w = hw % g.W;
    int ph = h + g.ph - r, pw = w + g.pw - s;
    if (ph < 0 || pw < 0 || ph % g.sh || pw % g.sw) return 0.f;
    int p = ph / g.sh, q = pw / g.sw;
    if (p >= g.P || q >= g.Q) return 0.f;
    return dy[(((int64_t)n * g.K + k) * g.P + p) * g.Q + q];
  }
};
// backward-filter:  A = dy [K x NPQ],  B = im2col(x)^T [NPQ x CRS]
struct WgradA {
  const float* dy; ConvGeom g;
  __device__ __forceinline__ float at(int64_t m, int64_t kk) const {
    int PQ = g.P * g.Q;
    int n = (int)(kk / PQ), pq = (int)(kk % PQ);
    return dy[((int64_t)n * g.K + m) * PQ + pq];
  }
};
struct WgradB {
  const float* x; ConvGeom g;
  __device__ __forceinline__ float at(int64_t kk, int64_t j) const {
    int RS = g.R * g.S, PQ = g.P * g.Q;
    int n = (int)(kk / PQ), pq = (int)(kk % PQ), p = pq / g.Q, q = pq % g.Q;
    int c = (int)(j / RS), rs = (int)(j % RS), r = rs / g.S, s = rs % g.S;
    int h = p * g.sh + r - g.ph, w = q * g.sw + s - g.pw;
    if (h < 0 || h >= g.H || w < 0 || w >= g.W) return 0.f;
    return x[(((int64_t)n * g.C + c) * g.H + h) * g.W + w];
  }
};

// ---- output views ----------------------------------------------------------------------------
struct MatOut { float* p; int64_t ld; __device__ __forceinline__ float* ptr(int64_t m, int64_t n) const { return p + m * ld + n; } };
struct NchwOut {            // rows = channel, cols = (image, pixel)
  float* p; int64_t chans, plane;
  __device__ __forceinline__ float* ptr(int64_t m, int64_t j) const { int64_t n = j / plane, px = j % plane; return p + (n * chans + m) * plane + px; }
};

// B_KFAST: consecutive loader threads walk K (for operands contiguous along K) instead of N.
// SPLIT: the reduction is cut over blockIdx.z; every cut writes its partial [M x N] result to `part` and
// contract_reduce_kernel adds the cuts in order (bit-reproducible, unlike atomic adds).
template <class AV, class BV, class OV, bool B_KFAST, bool SPLIT>
__global__ void __launch_bounds__(256) contract_kernel(AV A, BV B, OV O, int64_t M, int64_t N, int64_t K, int64_t k_per_split, float* __restrict__ part) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  int tid = threadIdx.x;
  int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
  int64_t kbeg = (int64_t)blockIdx.z * k_per_split, kend = min(K, kbeg + k_per_split);
  int tx = tid & 15, ty = tid >> 4;      // 16 x 16 threads, each a 4 x 4 micro-tile
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int64_t kt = kbeg; kt < kend; kt += BK) {
#pragma unroll
    for (int i = 0; i < (BM * BK) / 256; ++i) {
      int e = tid + i * 256, kk = e % BK, mm = e / BK;
      int64_t gm = m0 + mm, gk = kt + kk;
      As[kk][mm] = (gm < M && gk < kend) ? A.at(gm, gk) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < (BN * BK) / 256; ++i) {
      int e = tid + i * 256, kk, nn;
      if (B_KFAST) { kk = e % BK; nn = e / BK; } else { nn = e % BN; kk = e / BN; }
      int64_t gn = n0 + nn, gk = kt + kk;
      Bs[kk][nn] = (gn < N && gk < kend) ? B.at(gk, gn) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int64_t gm = m0 + ty * TM + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      int64_t gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      if (SPLIT) part[((int64_t)blockIdx.z * M + gm) * N + gn] = acc[i][j];
      else *O.ptr(gm, gn) = acc[i][j];
    }
  }
}

template <class OV>
__global__ void __launch_bounds__(256) contract_reduce_kernel(const float* __restrict__ part, OV O, int64_t M, int64_t N, int splits) {
  const int64_t total = M * N, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    float v = 0.f;
    for (int z = 0; z < splits; ++z) v += part[(int64_t)z * total + i];
    *O.ptr(i / N, i % N) = v;
  }
}

template <class AV, class BV, class OV, bool B_KFAST>
static int launch_contract(AV A, BV B, OV O, int64_t M, int64_t N, int64_t K, float* out_base, size_t out_bytes, bool allow_split, cudaStream_t s, const char* what) {
  if (M <= 0 || N <= 0) return 0;
  int64_t gx = (N + BN - 1) / BN, gy = (M + BM - 1) / BM;
  TF_REQUIRE(gy <= 65535, "%s: M too large for the CUDA-core path", what);
  int splits = 1;
  int sms = device_sm_count();
  if (allow_split && gx * gy < 2 * sms && K >= 4 * BK * 8) {
    splits = (int)((4 * sms) / (gx * gy));
    int64_t max_splits = K / (BK * 8);
    if (splits > max_splits) splits = (int)max_splits;
    if (splits > 65535) splits = 65535;
    if (splits < 1) splits = 1;
  }
  int64_t kps = ((K + splits - 1) / splits + BK - 1) / BK * BK;
  splits = (int)((K + kps - 1) / kps);
  if (K == 0) { splits = 1; kps = BK; }
  note_compute_stream(s);
  KernelTimer kt("contract_cudacore", s, 2.0 * (double)M * (double)N * (double)K, 0, 1);
  dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)splits);
  (void)out_base; (void)out_bytes;
  if (splits > 1) {
    float* part = (float*)persistent_scratch(3, sizeof(float) * (size_t)splits * (size_t)M * (size_t)N);
    if (!part) { splits = 1; kps = (K + BK - 1) / BK * BK; grid.z = 1; }       // no scratch: run unsplit
    else {
      contract_kernel<AV, BV, OV, B_KFAST, true><<<grid, 256, 0, s>>>(A, B, O, M, N, K, kps, part);
      contract_reduce_kernel<OV><<<grid_for(M * N, 256), 256, 0, s>>>(part, O, M, N, splits);
      if (after_launch(s, what, 2) != 0) return -1;
      return 0;
    }
  }
  contract_kernel<AV, BV, OV, B_KFAST, false><<<grid, 256, 0, s>>>(A, B, O, M, N, K, kps, nullptr);
  TF_AFTER(s, what);
  return 0;
}

// ---- 3-D convolution forward: A = filter [K x C*T*R*S], B = patches of x [C*T*R*S x N*Od*P*Q] ---------------------------
struct Conv3Geom { int N, C, D, H, W, K, T, R, S, Od, P, Q, pd, ph, pw, sd, sh, sw; };
struct Fwd3B {
  const float* x; Conv3Geom g;
  __device__ __forceinline__ float at(int64_t kk, int64_t j) const {
    const int RS = g.R * g.S, TRS = g.T * RS, PQ = g.P * g.Q, OPQ = g.Od * PQ;
    const int c = (int)(kk / TRS); int rem = (int)(kk % TRS);
    const int t = rem / RS; rem -= t * RS;
    const int r = rem / g.S, s = rem - r * g.S;
    const int n = (int)(j / OPQ); int o = (int)(j % OPQ);
    const int od = o / PQ; o -= od * PQ;
    const int p = o / g.Q, q = o - p * g.Q;
    const int z = od * g.sd + t - g.pd, h = p * g.sh + r - g.ph, w = q * g.sw + s - g.pw;
    if (z < 0 || z >= g.D || h < 0 || h >= g.H || w < 0 || w >= g.W) return 0.f;
    return x[((((int64_t)n * g.C + c) * g.D + z) * g.H + h) * g.W + w];
  }
};

static ConvGeom geom_of(const ConvPlan* p) {
  ConvGeom g;
  g.N = p->N; g.C = p->C; g.H = p->H; g.W = p->W; g.K = p->K; g.R = p->R; g.S = p->S; g.P = p->P; g.Q = p->Q;
  g.ph = p->pad_h; g.pw = p->pad_w; g.sh = p->stride_h; g.sw = p->stride_w;
  return g;
}

// Entry points used by the dispatchers in contract_api.cu
int cudacore_matmul(const float* A, bool tA, const float* B, bool tB, float* C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, cudaStream_t s) {
  MatView a{A, lda, tA ? 1 : 0};
  MatView bt{B, ldb, tB ? 1 : 0};
  MatOut o{C, N};
  // B is [K x N] logically; when stored transposed ([N x K]) it is contiguous along K.
  if (tB) return launch_contract<MatView, MatView, MatOut, true>(a, bt, o, M, N, K, C, sizeof(float) * M * N, true, s, "DLGpuMatrixMultiply");
  return launch_contract<MatView, MatView, MatOut, false>(a, bt, o, M, N, K, C, sizeof(float) * M * N, true, s, "DLGpuMatrixMultiply");
}
int cudacore_conv_fwd(const ConvPlan* p, const float* x, const float* w, float* y, cudaStream_t s) {
  ConvGeom g = geom_of(p);
  int64_t CRS = (int64_t)g.C * g.R * g.S, NPQ = (int64_t)g.N * g.P * g.Q;
  return launch_contract<FwdA, FwdB, NchwOut, false>(FwdA{w, CRS}, FwdB{x, g}, NchwOut{y, g.K, (int64_t)g.P * g.Q}, g.K, NPQ, CRS, y, sizeof(float) * g.K * NPQ, false, s, "DLGpuConvolution2DForward");
}
int cudacore_conv_dgrad(const ConvPlan* p, const float* dy, const float* w, float* dx, cudaStream_t s) {
  ConvGeom g = geom_of(p);
  int64_t KRS = (int64_t)g.K * g.R * g.S, NHW = (int64_t)g.N * g.H * g.W;
  return launch_contract<DgradA, DgradB, NchwOut, false>(DgradA{w, g}, DgradB{dy, g}, NchwOut{dx, g.C, (int64_t)g.H * g.W}, g.C, NHW, KRS, dx, sizeof(float) * g.C * NHW, false, s, "DLGpuConvolutionBackwardData");
}
int cudacore_conv_wgrad(const ConvPlan* p, const float* x, const float* dy, float* dw, cudaStream_t s) {
  ConvGeom g = geom_of(p);
  int64_t CRS = (int64_t)g.C * g.R * g.S, NPQ = (int64_t)g.N * g.P * g.Q;
  return launch_contract<WgradA, WgradB, MatOut, true>(WgradA{dy, g}, WgradB{x, g}, MatOut{dw, CRS}, g.K, CRS, NPQ, dw, sizeof(float) * g.K * CRS, true, s, "DLGpuConvolutionBackwardFilter");
}

// `d` points at the 18 ints N, C, D, H, W, K, T, R, S, Od, P, Q, pd, ph, pw, sd, sh, sw of the plan
int cudacore_conv3d_fwd(const int* d, const float* x, const float* w, float* y, cudaStream_t s) {
  Conv3Geom g;
  memcpy(&g, d, sizeof(g));
  const int64_t CTRS = (int64_t)g.C * g.T * g.R * g.S, vol = (int64_t)g.Od * g.P * g.Q, NV = (int64_t)g.N * vol;
  return launch_contract<FwdA, Fwd3B, NchwOut, false>(FwdA{w, CTRS}, Fwd3B{x, g}, NchwOut{y, g.K, vol}, g.K, NV, CTRS, y, sizeof(float) * g.K * NV, false, s,
                                                      "DLGpuConvolution3DForward");
}

}  // namespace tf

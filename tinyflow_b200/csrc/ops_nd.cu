// 1-D and 3-D convolution (forward) and pooling (forward / backward): src/gpu_op.cu:1435-1650, 2340-2530, 2647-3203.
// The reference reaches these through cuDNN as well; no benchmark graph uses them.
//
//   1-D   The reference itself describes a 1-D tensor (N, C, W) to cuDNN as the 4-D tensor (N, C, 1, W) with a window of
//         height 1 (src/gpu_op.cu:1535-1606, 2699-2748), so these entry points build 4-D views of their arguments and
//         call the 2-D entry points: a 1-D convolution of useful size runs on the tensor cores like any other.
//   3-D   Convolution forward is the CUDA-core contraction kernel over a 3-D patch view (exact fp32); pooling has
//         direct kernels: forward one thread per output, backward one thread per input element gathering from the
//         windows that cover it (no atomics; max pooling sends the gradient to the first maximum of a window in
//         (depth, row, column) order, an all-padding window yields 0, average pooling divides by the full window).
//   NCHW-style layouts only (dataformat 0), like the 2-D kernels.
#include "common.h"

namespace tf {

int cudacore_conv3d_fwd(const int* d, const float* x, const float* w, float* y, cudaStream_t s);   // contract_cudacore.cu

struct Conv3Plan { int kind; int N, C, D, H, W, K, T, R, S, Od, P, Q, pd, ph, pw, sd, sh, sw; };
struct Pool3Plan { int kind; int N, C, D, H, W, Od, P, Q, mode, pd, ph, pw, sd, sh, sw, kd, kh, kw; };
enum { kPlanConv3 = 0x7f21, kPlanPool3 };

struct Pool3Geom { int C, D, H, W, Od, P, Q, pd, ph, pw, sd, sh, sw, kd, kh, kw; };
static Pool3Geom geom3(const Pool3Plan* p) {
  return Pool3Geom{p->C, p->D, p->H, p->W, p->Od, p->P, p->Q, p->pd, p->ph, p->pw, p->sd, p->sh, p->sw, p->kd, p->kh, p->kw};
}

// first maximum of window (od, p, q) of one (image, channel) volume; returns the flat offset inside the volume or -1
__device__ __forceinline__ int pool3_argmax(const float* __restrict__ vol, const Pool3Geom& g, int od, int p, int q, float* best_out) {
  float best = 0.f;
  int arg = -1;
  for (int t = 0; t < g.kd; ++t) {
    const int z = od * g.sd + t - g.pd;
    if (z < 0 || z >= g.D) continue;
    for (int r = 0; r < g.kh; ++r) {
      const int i = p * g.sh + r - g.ph;
      if (i < 0 || i >= g.H) continue;
      for (int c = 0; c < g.kw; ++c) {
        const int j = q * g.sw + c - g.pw;
        if (j < 0 || j >= g.W) continue;
        const int off = (z * g.H + i) * g.W + j;
        const float v = vol[off];
        if (arg < 0 || v > best) { best = v; arg = off; }
      }
    }
  }
  if (best_out) *best_out = arg < 0 ? 0.f : best;
  return arg;
}

__global__ void __launch_bounds__(256) pool3_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t total, Pool3Geom g, int mode) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int out_vol = g.Od * g.P * g.Q, in_vol = g.D * g.H * g.W;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int64_t nc = idx / out_vol;
    int rem = (int)(idx - nc * out_vol);
    const int od = rem / (g.P * g.Q); rem -= od * g.P * g.Q;
    const int p = rem / g.Q, q = rem - p * g.Q;
    const float* vol = x + nc * in_vol;
    if (mode == 0) {
      float best;
      pool3_argmax(vol, g, od, p, q, &best);
      y[idx] = best;
    } else {
      float acc = 0.f;
      for (int t = 0; t < g.kd; ++t) {
        const int z = od * g.sd + t - g.pd;
        if (z < 0 || z >= g.D) continue;
        for (int r = 0; r < g.kh; ++r) {
          const int i = p * g.sh + r - g.ph;
          if (i < 0 || i >= g.H) continue;
          for (int c = 0; c < g.kw; ++c) {
            const int j = q * g.sw + c - g.pw;
            if (j >= 0 && j < g.W) acc += vol[(z * g.H + i) * g.W + j];
          }
        }
      }
      y[idx] = acc / (float)(g.kd * g.kh * g.kw);
    }
  }
}

// dx[n,c,z,i,j] = sum over the windows (od, p, q) that contain (z, i, j) of dy[od,p,q] * [window's first maximum sits
// here] (max) or dy[od,p,q] / window size (average)
__global__ void __launch_bounds__(256) pool3_bwd_kernel(const float* __restrict__ x, const float* __restrict__ dy, float* __restrict__ dx, int64_t total,
                                                        Pool3Geom g, int mode) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int out_vol = g.Od * g.P * g.Q, in_vol = g.D * g.H * g.W;
  const float inv = 1.f / (float)(g.kd * g.kh * g.kw);
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
    const int64_t nc = idx / in_vol;
    const int off = (int)(idx - nc * in_vol);
    int rem = off;
    const int z = rem / (g.H * g.W); rem -= z * g.H * g.W;
    const int i = rem / g.W, j = rem - i * g.W;
    const float* vol = x + nc * in_vol;
    const float* dvol = dy + nc * out_vol;
    // windows covering (z, i, j): od * sd - pd <= z < od * sd - pd + kd
    const int od_lo = max(0, (z + g.pd - g.kd + g.sd) / g.sd), od_hi = min(g.Od - 1, (z + g.pd) / g.sd);
    const int p_lo = max(0, (i + g.ph - g.kh + g.sh) / g.sh), p_hi = min(g.P - 1, (i + g.ph) / g.sh);
    const int q_lo = max(0, (j + g.pw - g.kw + g.sw) / g.sw), q_hi = min(g.Q - 1, (j + g.pw) / g.sw);
    float acc = 0.f;
    for (int od = od_lo; od <= od_hi; ++od)
      for (int p = p_lo; p <= p_hi; ++p)
        for (int q = q_lo; q <= q_hi; ++q) {
          const float d = dvol[(od * g.P + p) * g.Q + q];
          if (mode == 0) { if (pool3_argmax(vol, g, od, p, q, nullptr) == off) acc += d; }
          else acc += d * inv;
        }
    dx[idx] = acc;
  }
}

static int view4(const DLArrayHandle a, DLArray* v, int64_t* shape, const char* what) {
  TF_REQUIRE(a && a->ndim == 3, "%s: expects 3-D arrays (N, C, W)", what);
  shape[0] = a->shape[0]; shape[1] = a->shape[1]; shape[2] = 1; shape[3] = a->shape[2];
  v->data = a->data; v->ctx = a->ctx; v->ndim = 4; v->shape = shape;
  return 0;
}

}  // namespace tf

using namespace tf;

extern "C" {

// ---- 1-D: the 2-D entry points on (N, C, 1, W) views ------------------------------------------------------------------
int DLGpuConvolution1DForwardGetOutShape(const int* input_shapes, const int* filter_shapes, int* output_shapes, int dataformat, const int padding,
                                         const int v, void*** cudnnlist) {
  TF_REQUIRE(input_shapes && filter_shapes && output_shapes && cudnnlist, "DLGpuConvolution1DForwardGetOutShape: null argument");
  TF_REQUIRE(dataformat == 0, "DLGpuConvolution1DForwardGetOutShape: only the (N, C, W) layout is implemented");
  const int in4[4] = {input_shapes[0], input_shapes[1], 1, input_shapes[2]};
  const int f4[4] = {filter_shapes[0], filter_shapes[1], 1, filter_shapes[2]};
  int out4[4];
  if (DLGpuConvolution2DForwardGetOutShape(in4, f4, out4, 0, padding, 1, v, cudnnlist)) return -1;
  output_shapes[0] = out4[0]; output_shapes[1] = out4[1]; output_shapes[2] = out4[3];
  return 0;
}
int DLGpuConvolution1DForward(const DLArrayHandle input, const DLArrayHandle filter, DLArrayHandle output, void*** cudnnlist, void** cudnnHandle,
                              int* memorytoSaving) {
  DLArray x, w, y;
  int64_t sx[4], sw[4], sy[4];
  if (view4(input, &x, sx, "DLGpuConvolution1DForward") || view4(filter, &w, sw, "DLGpuConvolution1DForward") || view4(output, &y, sy, "DLGpuConvolution1DForward")) return -1;
  cudaStream_t s = last_compute_stream();          // the reference's wrapper passes no stream for the 1-D / 3-D calls
  void* cell = (void*)s;
  return DLGpuConvolution2DForward(&x, &w, &y, cudnnlist, cudnnHandle, memorytoSaving, &cell);
}
int DLGpuPooling1DForwardGetOutShape(const int* input_shapes, int* output_shapes, int dataformat, int poolingMode, const int padding_w, const int v,
                                     const int filter_w, void*** cudnnlist) {
  TF_REQUIRE(input_shapes && output_shapes && cudnnlist, "DLGpuPooling1DForwardGetOutShape: null argument");
  TF_REQUIRE(dataformat == 0, "DLGpuPooling1DForwardGetOutShape: only the (N, C, W) layout is implemented");
  const int in4[4] = {input_shapes[0], input_shapes[1], 1, input_shapes[2]};
  int out4[4];
  if (DLGpuPooling2DForwardGetOutShape(in4, out4, 0, poolingMode, 0, padding_w, 1, v, 1, filter_w, cudnnlist)) return -1;
  output_shapes[0] = out4[0]; output_shapes[1] = out4[1]; output_shapes[2] = out4[3];
  return 0;
}
int DLGpuPooling1DForward(const DLArrayHandle input, DLArrayHandle output, void*** cudnnlist, void** cudnnHandle) {
  DLArray x, y;
  int64_t sx[4], sy[4];
  if (view4(input, &x, sx, "DLGpuPooling1DForward") || view4(output, &y, sy, "DLGpuPooling1DForward")) return -1;
  void* cell = (void*)last_compute_stream();
  return DLGpuPooling2DForward(&x, &y, cudnnlist, cudnnHandle, &cell);
}
int DLGpuPooling1DBackward(const DLArrayHandle input, const DLArrayHandle output, const DLArrayHandle doutput, DLArrayHandle dinput, void*** cudnnlist,
                           void** cudnnHandle) {
  DLArray x, y, dy, dx;
  int64_t sx[4], sy[4], sdy[4], sdx[4];
  if (view4(input, &x, sx, "DLGpuPooling1DBackward") || view4(output, &y, sy, "DLGpuPooling1DBackward") || view4(doutput, &dy, sdy, "DLGpuPooling1DBackward") ||
      view4(dinput, &dx, sdx, "DLGpuPooling1DBackward"))
    return -1;
  void* cell = (void*)last_compute_stream();
  return DLGpuPooling2DBackward(&x, &y, &dy, &dx, cudnnlist, cudnnHandle, &cell);
}

// ---- 3-D --------------------------------------------------------------------------------------------------------------
// input (N, C, D, H, W), filter (K, C, T, R, S); pad = window / 2 per axis for SAME, 0 for VALID; strides s1, s2, s3
// along depth, height, width (src/gpu_op.cu:2431-2527).
int DLGpuConvolution3DForwardGetOutShape(const int* input_shapes, const int* filter_shapes, int* output_shapes, int dataformat, const int padding,
                                         const int s1, const int s2, const int s3, void*** cudnnlist) {
  TF_REQUIRE(input_shapes && filter_shapes && output_shapes && cudnnlist, "DLGpuConvolution3DForwardGetOutShape: null argument");
  TF_REQUIRE(dataformat == 0, "DLGpuConvolution3DForwardGetOutShape: only the (N, C, D, H, W) layout is implemented");
  TF_REQUIRE(s1 > 0 && s2 > 0 && s3 > 0, "DLGpuConvolution3DForwardGetOutShape: strides must be positive");
  TF_REQUIRE(filter_shapes[1] == input_shapes[1], "DLGpuConvolution3DForwardGetOutShape: filter channels %d != input channels %d", filter_shapes[1], input_shapes[1]);
  Conv3Plan* p = new_plan<Conv3Plan>(cudnnlist, kPlanConv3, 4);
  p->N = input_shapes[0]; p->C = input_shapes[1]; p->D = input_shapes[2]; p->H = input_shapes[3]; p->W = input_shapes[4];
  p->K = filter_shapes[0]; p->T = filter_shapes[2]; p->R = filter_shapes[3]; p->S = filter_shapes[4];
  p->pd = padding == 1 ? p->T / 2 : 0; p->ph = padding == 1 ? p->R / 2 : 0; p->pw = padding == 1 ? p->S / 2 : 0;
  p->sd = s1; p->sh = s2; p->sw = s3;
  TF_REQUIRE(p->D + 2 * p->pd >= p->T && p->H + 2 * p->ph >= p->R && p->W + 2 * p->pw >= p->S, "DLGpuConvolution3DForwardGetOutShape: filter larger than padded input");
  p->Od = 1 + (p->D + 2 * p->pd - p->T) / s1; p->P = 1 + (p->H + 2 * p->ph - p->R) / s2; p->Q = 1 + (p->W + 2 * p->pw - p->S) / s3;
  output_shapes[0] = p->N; output_shapes[1] = p->K; output_shapes[2] = p->Od; output_shapes[3] = p->P; output_shapes[4] = p->Q;
  return 0;
}
int DLGpuConvolution3DForward(const DLArrayHandle input, const DLArrayHandle filter, DLArrayHandle output, void*** cudnnlist, void** cudnnHandle,
                              int* memorytoSaving) {
  (void)cudnnHandle; (void)memorytoSaving;
  Conv3Plan* p = plan_of<Conv3Plan>(cudnnlist, kPlanConv3);
  TF_REQUIRE(p, "DLGpuConvolution3DForward: descriptor was not built by DLGpuConvolution3DForwardGetOutShape");
  TF_REQUIRE(input && numel(input) == (int64_t)p->N * p->C * p->D * p->H * p->W, "DLGpuConvolution3DForward: input does not match the descriptor");
  TF_REQUIRE(filter && numel(filter) == (int64_t)p->K * p->C * p->T * p->R * p->S, "DLGpuConvolution3DForward: filter does not match the descriptor");
  TF_REQUIRE(output && numel(output) == (int64_t)p->N * p->K * p->Od * p->P * p->Q, "DLGpuConvolution3DForward: output does not match the descriptor");
  return cudacore_conv3d_fwd(&p->N, (const float*)input->data, (const float*)filter->data, out_f32(output), last_compute_stream());
}

int DLGpuPooling3DForwardGetOutShape(const int* input_shapes, int* output_shapes, int dataformat, int poolingMode, const int padding1, const int padding2,
                                     const int padding3, const int s1, const int s2, const int s3, const int filter1, const int filter2, const int filter3,
                                     void*** cudnnlist) {
  TF_REQUIRE(input_shapes && output_shapes && cudnnlist, "DLGpuPooling3DForwardGetOutShape: null argument");
  TF_REQUIRE(dataformat == 0, "DLGpuPooling3DForwardGetOutShape: only the (N, C, D, H, W) layout is implemented");
  TF_REQUIRE(poolingMode == 0 || poolingMode == 1, "DLGpuPooling3DForwardGetOutShape: unknown mode %d", poolingMode);
  TF_REQUIRE(s1 > 0 && s2 > 0 && s3 > 0 && filter1 > 0 && filter2 > 0 && filter3 > 0 && padding1 >= 0 && padding2 >= 0 && padding3 >= 0,
             "DLGpuPooling3DForwardGetOutShape: bad window");
  Pool3Plan* p = new_plan<Pool3Plan>(cudnnlist, kPlanPool3, 3);
  p->N = input_shapes[0]; p->C = input_shapes[1]; p->D = input_shapes[2]; p->H = input_shapes[3]; p->W = input_shapes[4];
  p->mode = poolingMode;
  p->pd = padding1; p->ph = padding2; p->pw = padding3; p->sd = s1; p->sh = s2; p->sw = s3; p->kd = filter1; p->kh = filter2; p->kw = filter3;
  TF_REQUIRE(p->D + 2 * p->pd >= p->kd && p->H + 2 * p->ph >= p->kh && p->W + 2 * p->pw >= p->kw, "DLGpuPooling3DForwardGetOutShape: window larger than padded input");
  p->Od = 1 + (p->D + 2 * p->pd - p->kd) / s1; p->P = 1 + (p->H + 2 * p->ph - p->kh) / s2; p->Q = 1 + (p->W + 2 * p->pw - p->kw) / s3;
  output_shapes[0] = p->N; output_shapes[1] = p->C; output_shapes[2] = p->Od; output_shapes[3] = p->P; output_shapes[4] = p->Q;
  return 0;
}
static int check_pool3(const Pool3Plan* p, const DLArrayHandle in, const DLArrayHandle out, const char* what) {
  TF_REQUIRE(p, "%s: descriptor was not built by DLGpuPooling3DForwardGetOutShape", what);
  TF_REQUIRE(in && numel(in) == (int64_t)p->N * p->C * p->D * p->H * p->W, "%s: input does not match the descriptor", what);
  TF_REQUIRE(out && numel(out) == (int64_t)p->N * p->C * p->Od * p->P * p->Q, "%s: output does not match the descriptor", what);
  return 0;
}
int DLGpuPooling3DForward(const DLArrayHandle input, DLArrayHandle output, void*** cudnnlist, void** cudnnHandle) {
  (void)cudnnHandle;
  Pool3Plan* p = plan_of<Pool3Plan>(cudnnlist, kPlanPool3);
  if (check_pool3(p, input, output, "DLGpuPooling3DForward")) return -1;
  cudaStream_t s = last_compute_stream();
  const int64_t total = numel(output);
  note_compute_stream(s);
  pool3_fwd_kernel<<<grid_for(total, 256), 256, 0, s>>>((const float*)input->data, out_f32(output), total, geom3(p), p->mode);
  TF_AFTER(s, "DLGpuPooling3DForward");
  return 0;
}
int DLGpuPooling3DBackward(const DLArrayHandle input, const DLArrayHandle output, const DLArrayHandle doutput, DLArrayHandle dinput, void*** cudnnlist,
                           void** cudnnHandle) {
  (void)cudnnHandle;
  Pool3Plan* p = plan_of<Pool3Plan>(cudnnlist, kPlanPool3);
  if (check_pool3(p, input, output, "DLGpuPooling3DBackward")) return -1;
  TF_REQUIRE(doutput && dinput && numel(doutput) == numel(output) && numel(dinput) == numel(input), "DLGpuPooling3DBackward: gradient sizes do not match");
  cudaStream_t s = last_compute_stream();
  const int64_t total = numel(dinput);
  note_compute_stream(s);
  pool3_bwd_kernel<<<grid_for(total, 256), 256, 0, s>>>((const float*)input->data, (const float*)doutput->data, out_f32(dinput), total, geom3(p), p->mode);
  TF_AFTER(s, "DLGpuPooling3DBackward");
  return 0;
}

}  // extern "C"

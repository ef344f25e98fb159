// C-ABI entry points of the dense contractions (matmul, convolution forward / backward-data /
// backward-filter) and the dispatch between the tcgen05 tensor-core path and the CUDA-core path.
#include "common.h"

namespace tf {

int cudacore_matmul(const float* A, bool tA, const float* B, bool tB, float* C, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, cudaStream_t s);
int cudacore_conv_fwd(const ConvPlan* p, const float* x, const float* w, float* y, cudaStream_t s);
int cudacore_conv_dgrad(const ConvPlan* p, const float* dy, const float* w, float* dx, cudaStream_t s);
int cudacore_conv_wgrad(const ConvPlan* p, const float* x, const float* dy, float* dw, cudaStream_t s);

// Tensor-core path (gemm_tcgen05.cu).  Each returns 1 when it handled the call, 0 when the
// shape is outside what it takes (caller falls through to the CUDA-core path), -1 on error.
int tc_matmul(const float* A, bool tA, const float* B, bool tB, float* C, int64_t M, int64_t N, int64_t K, cudaStream_t s, int* oom_bytes);
int tc_conv_fwd(ConvPlan* p, const float* x, const float* w, float* y, cudaStream_t s, int* oom_bytes);
int tc_conv_dgrad(ConvPlan* p, const float* dy, const float* w, float* dx, cudaStream_t s, int* oom_bytes);
int tc_conv_wgrad(ConvPlan* p, const float* x, const float* dy, float* dw, cudaStream_t s, int* oom_bytes);

static int g_path = [] { const char* e = getenv("TINYFLOW_CONTRACTION"); return e ? atoi(e) : 0; }();   // 0 auto, 1 CUDA cores, 2 tensor cores
int contraction_path() { return g_path; }
bool contraction_path_is_cuda_cores() { return g_path == 1; }
int tensor_arithmetic();
void set_tensor_arithmetic(int a);
int tensor_path_error();
void tensor_path_error_clear();
int tensor_path_timeout_probe(long long limit_cycles, cudaStream_t s);
long long fused_relu_pack_count();
// which engine served this thread's most recent contraction: 1 = CUDA cores, 2 = tensor cores (0 = none yet)
static thread_local int t_last_path = 0;

}  // namespace tf

using namespace tf;

extern "C" {

int TfLastContractionPath(void) { return t_last_path; }

int TfSetArithmetic(int arithmetic) {
  TF_REQUIRE(arithmetic == 0 || arithmetic == 1, "TfSetArithmetic: 0 = 3xFP16, 1 = 3xTF32");
  set_tensor_arithmetic(arithmetic);
  return 0;
}
int TfGetArithmetic(void) { return tensor_arithmetic(); }

int TfTensorPathError(void) { return tensor_path_error(); }
int TfClearTensorPathError(void) { tensor_path_error_clear(); return 0; }
int TfFusedReluPackCount(long long* count) { if (count) *count = fused_relu_pack_count(); return 0; }
int TfFusedReluBnBackwardCount(long long* count) { if (count) *count = fused_relu_bn_bwd_count(); return 0; }
int TfFusedAddReluCount(long long* count) { if (count) *count = fused_add_relu_count(); return 0; }
int TfTensorPathTimeoutProbe(long long limit_cycles, void** cudaStream) { return tensor_path_timeout_probe(limit_cycles, stream_of(cudaStream)); }

int TfSetContractionPath(int path) {
  TF_REQUIRE(path >= 0 && path <= 2, "TfSetContractionPath: path must be 0, 1 or 2");
  g_path = path;
  return 0;
}

// C[M x N] = op(A) op(B), row-major, alpha 1, beta 0 (src/gpu_op.cu:1166-1199).
int DLGpuMatrixMultiply(const DLArrayHandle matA, bool transposeA, const DLArrayHandle matB, bool transposeB, DLArrayHandle matC,
                        void** cublasHandle, void** cudaStream) {
  (void)cublasHandle;
  TF_REQUIRE(matA && matB && matC && matA->ndim == 2 && matB->ndim == 2 && matC->ndim == 2, "DLGpuMatrixMultiply: expects 2-D arrays");
  int64_t M = matA->shape[transposeA ? 1 : 0], K = matA->shape[transposeA ? 0 : 1];
  int64_t Kb = matB->shape[transposeB ? 1 : 0], N = matB->shape[transposeB ? 0 : 1];
  TF_REQUIRE(K == Kb, "DLGpuMatrixMultiply: inner extents differ (%lld vs %lld)", (long long)K, (long long)Kb);
  TF_REQUIRE(matC->shape[0] == M && matC->shape[1] == N, "DLGpuMatrixMultiply: output shape mismatch");
  cudaStream_t s = stream_of(cudaStream);
  const float* A = (const float*)matA->data;
  const float* B = (const float*)matB->data;
  float* C = out_f32(matC);
  if (g_path != 1) {
    int oom = 0;
    int r = tc_matmul(A, transposeA, B, transposeB, C, M, N, K, s, &oom);
    if (r < 0) return -1;
    if (r == 1) { t_last_path = 2; return 0; }
    TF_REQUIRE(g_path != 2, "DLGpuMatrixMultiply: shape not taken by the tensor-core path (forced)");
  }
  t_last_path = 1;
  return cudacore_matmul(A, transposeA, B, transposeB, C, M, N, K, matA->shape[1], matB->shape[1], s);
}

// Output extent = 1 + (in + 2*pad - window) / stride with pad = window/2 for SAME, 0 for VALID
// (src/gpu_op.cu:2040-2175; cross-correlation, dilation 1).
int DLGpuConvolution2DForwardGetOutShape(const int* input_shapes, const int* filter_shapes, int* output_shapes, int dataformat,
                                         const int padding, const int u, const int v, void*** cudnnlist) {
  TF_REQUIRE(input_shapes && filter_shapes && output_shapes && cudnnlist, "DLGpuConvolution2DForwardGetOutShape: null argument");
  TF_REQUIRE(u > 0 && v > 0, "DLGpuConvolution2DForwardGetOutShape: strides must be positive");
  ConvPlan* p = new_plan<ConvPlan>(cudnnlist, kPlanConv, 4);
  p->dataformat = dataformat;
  p->N = input_shapes[0]; p->K = filter_shapes[0];
  if (dataformat == 0) {
    p->C = input_shapes[1]; p->H = input_shapes[2]; p->W = input_shapes[3];
    p->R = filter_shapes[2]; p->S = filter_shapes[3];
    TF_REQUIRE(filter_shapes[1] == p->C, "DLGpuConvolution2DForwardGetOutShape: filter channels %d != input channels %d", filter_shapes[1], p->C);
  } else {
    p->C = input_shapes[3]; p->H = input_shapes[1]; p->W = input_shapes[2];
    p->R = filter_shapes[1]; p->S = filter_shapes[2];
    TF_REQUIRE(filter_shapes[3] == p->C, "DLGpuConvolution2DForwardGetOutShape: filter channels %d != input channels %d", filter_shapes[3], p->C);
  }
  p->pad_h = padding == 1 ? p->R / 2 : 0;
  p->pad_w = padding == 1 ? p->S / 2 : 0;
  p->stride_h = u; p->stride_w = v;
  p->P = 1 + (p->H + 2 * p->pad_h - p->R) / u;
  p->Q = 1 + (p->W + 2 * p->pad_w - p->S) / v;
  TF_REQUIRE(p->P > 0 && p->Q > 0 && p->H + 2 * p->pad_h >= p->R && p->W + 2 * p->pad_w >= p->S, "DLGpuConvolution2DForwardGetOutShape: filter larger than padded input");
  output_shapes[0] = p->N;
  if (dataformat == 0) { output_shapes[1] = p->K; output_shapes[2] = p->P; output_shapes[3] = p->Q; }
  else { output_shapes[1] = p->P; output_shapes[2] = p->Q; output_shapes[3] = p->K; }
  return 0;
}

static int check_conv(const ConvPlan* p, const DLArrayHandle x, const DLArrayHandle w, const DLArrayHandle y, const char* what) {
  TF_REQUIRE(p, "%s: descriptor was not built by DLGpuConvolution2DForwardGetOutShape", what);
  TF_REQUIRE(p->dataformat == 0, "%s: only NCHW is implemented", what);
  TF_REQUIRE(x && numel(x) == (int64_t)p->N * p->C * p->H * p->W, "%s: input does not match the descriptor", what);
  TF_REQUIRE(w && numel(w) == (int64_t)p->K * p->C * p->R * p->S, "%s: filter does not match the descriptor", what);
  TF_REQUIRE(y && numel(y) == (int64_t)p->N * p->K * p->P * p->Q, "%s: output does not match the descriptor", what);
  return 0;
}

int DLGpuConvolution2DForward(const DLArrayHandle input, const DLArrayHandle filter, DLArrayHandle output, void*** cudnnlist,
                              void** cudnnHandle, int* memorytoSaving, void** cudaStream) {
  (void)cudnnHandle;
  ConvPlan* p = plan_of<ConvPlan>(cudnnlist, kPlanConv);
  if (check_conv(p, input, filter, output, "DLGpuConvolution2DForward")) return -1;
  cudaStream_t s = stream_of(cudaStream);
  if (g_path != 1) {
    int oom = 0;
    int r = tc_conv_fwd(p, (const float*)input->data, (const float*)filter->data, out_f32(output), s, &oom);
    if (r < 0) return -1;
    if (oom) { if (memorytoSaving) *memorytoSaving = oom; return 0; }
    if (r == 1) { t_last_path = 2; return 0; }
    TF_REQUIRE(g_path != 2, "DLGpuConvolution2DForward: shape not taken by the tensor-core path (forced)");
  }
  t_last_path = 1;
  return cudacore_conv_fwd(p, (const float*)input->data, (const float*)filter->data, out_f32(output), s);
}

int DLGpuConvolutionBackwardData(const DLArrayHandle input, const DLArrayHandle doutput, const DLArrayHandle filter, DLArrayHandle dinput,
                                 void*** cudnnlist, void** cudnnHandle, int* memorytoSaving, void** cudaStream) {
  (void)cudnnHandle;
  ConvPlan* p = plan_of<ConvPlan>(cudnnlist, kPlanConv);
  if (check_conv(p, input, filter, doutput, "DLGpuConvolutionBackwardData")) return -1;
  TF_REQUIRE(dinput && numel(dinput) == numel(input), "DLGpuConvolutionBackwardData: dinput does not match input");
  cudaStream_t s = stream_of(cudaStream);
  if (g_path != 1) {
    int oom = 0;
    int r = tc_conv_dgrad(p, (const float*)doutput->data, (const float*)filter->data, out_f32(dinput), s, &oom);
    if (r < 0) return -1;
    if (oom) { if (memorytoSaving) *memorytoSaving = oom; return 0; }
    if (r == 1) { t_last_path = 2; return 0; }
    TF_REQUIRE(g_path != 2, "DLGpuConvolutionBackwardData: shape not taken by the tensor-core path (forced)");
  }
  t_last_path = 1;
  return cudacore_conv_dgrad(p, (const float*)doutput->data, (const float*)filter->data, out_f32(dinput), s);
}

int DLGpuConvolutionBackwardFilter(const DLArrayHandle input, const DLArrayHandle doutput, const DLArrayHandle filter, DLArrayHandle dfilter,
                                   void*** cudnnlist, void** cudnnHandle, int* memorytoSaving, void** cudaStream) {
  (void)cudnnHandle;
  ConvPlan* p = plan_of<ConvPlan>(cudnnlist, kPlanConv);
  if (check_conv(p, input, filter, doutput, "DLGpuConvolutionBackwardFilter")) return -1;
  TF_REQUIRE(dfilter && numel(dfilter) == numel(filter), "DLGpuConvolutionBackwardFilter: dfilter does not match filter");
  cudaStream_t s = stream_of(cudaStream);
  if (g_path != 1) {
    int oom = 0;
    int r = tc_conv_wgrad(p, (const float*)input->data, (const float*)doutput->data, out_f32(dfilter), s, &oom);
    if (r < 0) return -1;
    if (oom) { if (memorytoSaving) *memorytoSaving = oom; return 0; }
    if (r == 1) { t_last_path = 2; return 0; }
    TF_REQUIRE(g_path != 2, "DLGpuConvolutionBackwardFilter: shape not taken by the tensor-core path (forced)");
  }
  t_last_path = 1;
  return cudacore_conv_wgrad(p, (const float*)input->data, (const float*)doutput->data, out_f32(dfilter), s);
}

}  // extern "C"

/*
 * C-ABI of libc_runtime_api.so, the B200 (sm_100a) operator library that sits
 * behind tinyflow's ctypes wrappers.
 *
 * Every entry point below replaces the reference function of the same name;
 * the citation after each declaration is the reference definition it stands in
 * for (path inside the tinyflow project : line).  Argument order, argument
 * meaning and the 0 / -1 return convention are the reference's.  Differences
 * that a caller can observe are listed once, here:
 *
 *   - No cuDNN / cuBLAS types.  The enum-typed arguments are plain `int`
 *     with the values the Python wrappers pass (pycode/tinyflow/gpu_op.py):
 *       dataformat      0 = NCHW, 1 = NHWC
 *       padding         1 = SAME (pad = k/2 on both sides), 0 = VALID
 *       poolingMode     0 = max, 1 = average (padding included in the divisor)
 *       activationMode  0 = sigmoid, 1 = relu, 2 = tanh, 3 = softmax
 *       batchNormMode   0 = per-activation, 1 = spatial
 *   - Handles (`void **cudaStream`, `void **cudnnHandle`, `void **cublasHandle`)
 *     are caller-owned cells; the library stores an opaque pointer in the cell.
 *   - Descriptor lists (`void ***cudnnlist`) are caller-owned cells; the library
 *     stores a malloc'ed slot array whose slot 0 is a library-owned plan struct.
 *   - Kernels are enqueued asynchronously on the stream in the cell.  Set the
 *     environment variable TINYFLOW_SYNC=1 to get the reference's
 *     synchronize-after-every-op behaviour (needed for per-op wall-clock timing).
 *   - Out-of-memory is not an error: the call returns 0 and writes the number of
 *     bytes it failed to get through `int *memorytoSaving` (written only then).
 *   - The library never calls exit()/abort(); bad arguments return -1.
 *   - Convolutions and matrix products of useful size run on the tensor cores in
 *     3xFP16: each fp32 operand tensor is scaled by a power of two taken from its
 *     largest magnitude and split into an fp16 hi/lo pair, products accumulate in
 *     fp32.  Results agree with fp32 arithmetic to better than 1e-4; precision is
 *     relative to each operand tensor's largest element (values more than 2^18
 *     below it lose low-order bits).  TfSetContractionPath(1) selects exact-fp32
 *     CUDA-core kernels instead.
 */
#ifndef TINYFLOW_B200_C_RUNTIME_API_H_
#define TINYFLOW_B200_C_RUNTIME_API_H_

#include <stddef.h>
#include <stdint.h>
#ifndef __cplusplus
#include <stdbool.h>
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- array types: src/dlarray.h:21-52 ---------------------------------- */
typedef enum { kCPU = 1, kGPU = 2 } DLDeviceType;
typedef struct { int device_id; DLDeviceType device_type; } DLContext;
typedef struct { void *data; DLContext ctx; int ndim; int64_t *shape; } DLArray;
typedef int64_t index_t;
typedef DLArray *DLArrayHandle;
typedef void *DLStreamHandle;

/* ---- runtime ----------------------------------------------------------- */
int DLArrayAlloc(const index_t *shape, index_t ndim, DLContext ctx,
                 DLArrayHandle *out, int *memorytoSaving);          /* src/c_runtime_api.cc:93 */
int DLArrayFree(DLArrayHandle handle);                              /* src/c_runtime_api.cc:121 */
int DLArrayCopyFromTo(DLArrayHandle from, DLArrayHandle to,
                      DLStreamHandle stream);                       /* src/c_runtime_api.cc:128 */
int DLGpuCreatecudaStream(void **cudaStream);                       /* src/gpu_op.cu:1352 */
int DLGpuDestroycudaStream(void **cudaStream);                      /* src/gpu_op.cu:1366 */
int DLGpuCreatecudnnHandle(void **cudnnHandle, void **cudaStream);  /* src/gpu_op.cu:1378 */
int DLGpuDestroycudnnHandle(void **cudnnHandle);                    /* src/gpu_op.cu:1392 */
int DLGpuCreatecublasHandle(void **cublasHandle, void **cudaStream);/* src/gpu_op.cu:1405 */
int DLGpuDestroycublasHandle(void **cublasHandle);                  /* src/gpu_op.cu:1420 */
int getInt(int *intp);                                              /* src/gpu_op.cu:4896 */
int testPcie(void);                                                 /* src/gpu_op.cu:4960 */

/* ---- fill / broadcast / reduce ------------------------------------------ */
int DLGpuArraySet(DLArrayHandle arr, float value, void **cudaStream);                 /* src/gpu_op.cu:331 */
int DLGpuBroadcastTo0(const DLArrayHandle input, DLArrayHandle output, void **cudaStream); /* src/gpu_op.cu:343 */
int DLGpuBroadcastToBackward0(const DLArrayHandle input, DLArrayHandle output);       /* src/gpu_op.cu:369 */
int DLGpuBroadcastTo1(const DLArrayHandle input, DLArrayHandle output, void **cudaStream); /* src/gpu_op.cu:450 */
int DLGpuBroadcastToBackward1(const DLArrayHandle input, DLArrayHandle output);       /* src/gpu_op.cu:473 */
int DLGpuReduceSumAxisZero(const DLArrayHandle input, DLArrayHandle output);          /* src/gpu_op.cu:950 */
int DLGpuReduceSumAxisN(const DLArrayHandle input, DLArrayHandle output, const int axis);          /* src/gpu_op.cu:555 */
int DLGpuReduceSumAxisNBackward(const DLArrayHandle input, DLArrayHandle output, const int axis);  /* src/gpu_op.cu:594 */
int DLGpuReduceSumAll(const DLArrayHandle input, DLArrayHandle output);               /* src/gpu_op.cu:885 */
int DLGpuReduceSumAllBackward(const DLArrayHandle input, DLArrayHandle output);       /* src/gpu_op.cu:933 */
int DLGReduceSumGetCudnnlist(const int *input_shapes, const int *output_shapes,
                             const int sizeofshape, int dataformat,
                             void ***cudnnlist, void **cudnnHandle);                  /* src/gpu_op.cu:628 */
int DLGpuReduceSum(const DLArrayHandle input, DLArrayHandle output, void ***cudnnlist,
                   void **cudnnHandle, int *memorytoSaving, void **cudaStream);       /* src/gpu_op.cu:812 */

/* ---- elementwise -------------------------------------------------------- */
int DLGpuMatrixElementwiseAdd(const DLArrayHandle matA, const DLArrayHandle matB,
                              DLArrayHandle output, void **cudaStream);               /* src/gpu_op.cu:1090 */
int DLGpuMatrixElementwiseAddByConst(const DLArrayHandle input, float val,
                                     DLArrayHandle output, void **cudaStream);        /* src/gpu_op.cu:1109 */
int DLGpuMatrixElementwiseMultiply(const DLArrayHandle matA, const DLArrayHandle matB,
                                   DLArrayHandle output, void **cudaStream);          /* src/gpu_op.cu:1127 */
int DLGpuMatrixMultiplyByConst(const DLArrayHandle input, float val,
                               DLArrayHandle output, void **cudaStream);              /* src/gpu_op.cu:1147 */
int DLGpuRelu(const DLArrayHandle input, DLArrayHandle output);                       /* src/gpu_op.cu:1201 */
int DLGpuReluGradient(const DLArrayHandle input, const DLArrayHandle in_grad,
                      DLArrayHandle output);                                          /* src/gpu_op.cu:1216 */
int DLGpuMatrixExp(const DLArrayHandle input, DLArrayHandle output);                  /* src/gpu_op.cu:1289 */
int DLGpuMatrixLog(const DLArrayHandle input, DLArrayHandle output, void **cudaStream); /* src/gpu_op.cu:1305 */
int DLGpuMatrixReverse(const DLArrayHandle input, DLArrayHandle output);              /* src/gpu_op.cu:1321 */
int DLGpuMatrixPow(const DLArrayHandle input, const float val, DLArrayHandle output); /* src/gpu_op.cu:1336 */

/* ---- dense contraction -------------------------------------------------- */
int DLGpuMatrixMultiply(const DLArrayHandle matA, bool transposeA,
                        const DLArrayHandle matB, bool transposeB, DLArrayHandle matC,
                        void **cublasHandle, void **cudaStream);                      /* src/gpu_op.cu:1166 */

/* ---- softmax and losses ------------------------------------------------- */
int DLGpuSoftmax(const DLArrayHandle input, DLArrayHandle output, void **cudaStream); /* src/gpu_op.cu:1235 */
int DLGpuSoftmaxCrossEntropy(const DLArrayHandle input_a, const DLArrayHandle input_b,
                             DLArrayHandle output, void **cudaStream);                /* src/gpu_op.cu:1256 */
int DLGpuCrossEntropy(const DLArrayHandle input_a, const DLArrayHandle input_b,
                      DLArrayHandle output);                                          /* src/gpu_op.cu:3880 */
int DLGpuL1loss(const DLArrayHandle input_a, const DLArrayHandle input_b, DLArrayHandle output);   /* src/gpu_op.cu:3909 */
int DLGpuL2loss(const DLArrayHandle input_a, const DLArrayHandle input_b, DLArrayHandle output);   /* src/gpu_op.cu:3938 */
int DLGpuL1LossGradient(const DLArrayHandle input, const DLArrayHandle input1,
                        const DLArrayHandle grad, DLArrayHandle output);              /* src/gpu_op.cu:3968 */
int DLGpuL2LossGradient(const DLArrayHandle input, const DLArrayHandle input1,
                        const DLArrayHandle grad, DLArrayHandle output);              /* src/gpu_op.cu:3992 */
int DLGpuL1regular(const DLArrayHandle input_a, DLArrayHandle output);                /* src/gpu_op.cu:4016 */
int DLGpuL2regular(const DLArrayHandle input_a, DLArrayHandle output);                /* src/gpu_op.cu:4040 */
int DLGpuL1regularGradient(const DLArrayHandle input, const DLArrayHandle grad,
                           DLArrayHandle output);                                     /* src/gpu_op.cu:4065 */
int DLGpuL2regularGradient(const DLArrayHandle input, const DLArrayHandle grad,
                           DLArrayHandle output);                                     /* src/gpu_op.cu:4086 */
int DLGpuCross(const DLArrayHandle x, const DLArrayHandle y, DLArrayHandle output,
               float b, void **cudaStream);                                           /* src/gpu_op.cu:4546 */
int DLGpuCrossBackward(const DLArrayHandle x, const DLArrayHandle y,
                       const DLArrayHandle doutput, DLArrayHandle output,
                       float b, void **cudaStream);                                   /* src/gpu_op.cu:4576 */

/* ---- concat -------------------------------------------------------------- */
int DLGpuConcatForward(const DLArrayHandle input1, const DLArrayHandle input2,
                       DLArrayHandle output, void **cudaStream);                      /* src/gpu_op.cu:981 */
int DLGpuConcataBackward(const DLArrayHandle input1, const DLArrayHandle input2,
                         const DLArrayHandle doutput, DLArrayHandle dinput1,
                         void **cudaStream);                                          /* src/gpu_op.cu:1019 */
int DLGpuConcatbBackward(const DLArrayHandle input1, const DLArrayHandle input2,
                         const DLArrayHandle doutput, DLArrayHandle dinput2,
                         void **cudaStream);                                          /* src/gpu_op.cu:1059 */

/* ---- convolution --------------------------------------------------------- */
int DLGpuConvolution2DForwardGetOutShape(const int *input_shapes, const int *filter_shapes,
                                         int *output_shapes, int dataformat, const int padding,
                                         const int u, const int v, void ***cudnnlist); /* src/gpu_op.cu:2040 */
int DLGpuConvolution2DForward(const DLArrayHandle input, const DLArrayHandle filter,
                              DLArrayHandle output, void ***cudnnlist, void **cudnnHandle,
                              int *memorytoSaving, void **cudaStream);                /* src/gpu_op.cu:1952 */
int DLGpuConvolutionBackwardFilter(const DLArrayHandle input, const DLArrayHandle doutput,
                                   const DLArrayHandle filter, DLArrayHandle dfilter,
                                   void ***cudnnlist, void **cudnnHandle,
                                   int *memorytoSaving, void **cudaStream);           /* src/gpu_op.cu:1653 */
int DLGpuConvolutionBackwardData(const DLArrayHandle input, const DLArrayHandle doutput,
                                 const DLArrayHandle filter, DLArrayHandle dinput,
                                 void ***cudnnlist, void **cudnnHandle,
                                 int *memorytoSaving, void **cudaStream);             /* src/gpu_op.cu:1739 */
/* 1-D / 3-D convolution and pooling: exported for symbol completeness, return -1
 * (not on the training path of any supported model). */
int DLGpuConvolution1DForwardGetOutShape(const int *input_shapes, const int *filter_shapes,
                                         int *output_shapes, int dataformat, const int padding,
                                         const int v, void ***cudnnlist);             /* src/gpu_op.cu:1523 */
int DLGpuConvolution3DForwardGetOutShape(const int *input_shapes, const int *filter_shapes,
                                         int *output_shapes, int dataformat, const int padding,
                                         const int s1, const int s2, const int s3,
                                         void ***cudnnlist);                          /* src/gpu_op.cu:2431 */
int DLGpuConvolution1DForward(const DLArrayHandle input, const DLArrayHandle filter,
                              DLArrayHandle output, void ***cudnnlist, void **cudnnHandle,
                              int *memorytoSaving);                                   /* src/gpu_op.cu:1435 */
int DLGpuConvolution3DForward(const DLArrayHandle input, const DLArrayHandle filter,
                              DLArrayHandle output, void ***cudnnlist, void **cudnnHandle,
                              int *memorytoSaving);                                   /* src/gpu_op.cu:2340 */

/* ---- pooling ------------------------------------------------------------- */
int DLGpuPooling2DForwardGetOutShape(const int *input_shapes, int *output_shapes,
                                     int dataformat, int poolingMode,
                                     const int padding_h, const int padding_w,
                                     const int u, const int v,
                                     const int filter_h, const int filter_w,
                                     void ***cudnnlist);                              /* src/gpu_op.cu:2880 */
int DLGpuPooling2DForward(const DLArrayHandle input, DLArrayHandle output,
                          void ***cudnnlist, void **cudnnHandle, void **cudaStream);  /* src/gpu_op.cu:2839 */
int DLGpuPooling2DBackward(const DLArrayHandle input, const DLArrayHandle output,
                           const DLArrayHandle doutput, DLArrayHandle dinput,
                           void ***cudnnlist, void **cudnnHandle, void **cudaStream); /* src/gpu_op.cu:2984 */
int DLGpuPooling1DForwardGetOutShape(const int *input_shapes, int *output_shapes,
                                     int dataformat, int poolingMode, const int padding_w,
                                     const int v, const int filter_w, void ***cudnnlist); /* src/gpu_op.cu:2688 */
int DLGpuPooling3DForwardGetOutShape(const int *input_shapes, int *output_shapes,
                                     int dataformat, int poolingMode,
                                     const int padding1, const int padding2, const int padding3,
                                     const int s1, const int s2, const int s3,
                                     const int filter1, const int filter2, const int filter3,
                                     void ***cudnnlist);                              /* src/gpu_op.cu:3071 */
int DLGpuPooling1DForward(const DLArrayHandle input, DLArrayHandle output,
                          void ***cudnnlist, void **cudnnHandle);                     /* src/gpu_op.cu:2647 */
int DLGpuPooling3DForward(const DLArrayHandle input, DLArrayHandle output,
                          void ***cudnnlist, void **cudnnHandle);                     /* src/gpu_op.cu:3029 */
int DLGpuPooling1DBackward(const DLArrayHandle input, const DLArrayHandle output,
                           const DLArrayHandle doutput, DLArrayHandle dinput,
                           void ***cudnnlist, void **cudnnHandle);                    /* src/gpu_op.cu:2791 */
int DLGpuPooling3DBackward(const DLArrayHandle input, const DLArrayHandle output,
                           const DLArrayHandle doutput, DLArrayHandle dinput,
                           void ***cudnnlist, void **cudnnHandle);                    /* src/gpu_op.cu:3155 */

/* ---- activation (relu / sigmoid / tanh / softmax over C*H*W) ------------ */
int DLGpuActivationGetCudnnlist(const int *input_shapes, const int sizeofshape,
                                int dataformat, int activationMode, void ***cudnnlist); /* src/gpu_op.cu:3364 */
int DLGpuActivationForward(const DLArrayHandle input, DLArrayHandle output,
                           int activationMode, void ***cudnnlist,
                           void **cudnnHandle, void **cudaStream);                    /* src/gpu_op.cu:3211 */
int DLGpuActivationBackward(const DLArrayHandle input, DLArrayHandle dinput,
                            const DLArrayHandle output, const DLArrayHandle doutput,
                            int activationMode, void ***cudnnlist,
                            void **cudnnHandle, void **cudaStream);                   /* src/gpu_op.cu:3475 */

/* ---- dropout -------------------------------------------------------------- */
int DLGpuGetInputDescriptor(const int *input_shapes, const int sizeofshape,
                            int dataformat, void ***inputd);                          /* src/gpu_op.cu:3276 */
int DLGpuDropoutForward(const DLArrayHandle input, DLArrayHandle output, int dataformat,
                        const float dropout, const int seed, void **reserveSpace_p,
                        void ***inputd, void ***cudnnlist, void **cudnnHandle,
                        int *memorytoSaving, void **cudaStream);                      /* src/gpu_op.cu:3547 */
int DLGpuDropoutBackward(const DLArrayHandle doutput, DLArrayHandle dinput,
                         void **reserveSpace_p, void ***cudnnlist,
                         void **cudnnHandle, void **cudaStream);                      /* src/gpu_op.cu:3642 */

/* ---- batch normalisation (scale 1, bias 0, eps 1e-5, batch statistics) --- */
int DLGpuBatchNormalizationGetCudnnlist(const int *input_shapes, int sizeofshape,
                                        int dataformat, int batchNormMode,
                                        void **mean_p, void **Variance_p,
                                        void ***cudnnlist);                           /* src/gpu_op.cu:4111 */
int DLGpuBatchNormalizationForward(const DLArrayHandle input, DLArrayHandle output,
                                   int batchNormMode, int n, void **mean_p,
                                   void **Variance_p, void ***cudnnlist, void **cudnnHandle,
                                   int *memorytoSaving, void **cudaStream);           /* src/gpu_op.cu:4224 */
int DLGpuBatchNormalizationBackward(const DLArrayHandle input, const DLArrayHandle doutput,
                                    DLArrayHandle dinput, int batchNormMode,
                                    void **mean_p, void **Variance_p, void ***cudnnlist,
                                    void **cudnnHandle, int *memorytoSaving,
                                    void **cudaStream);                               /* src/gpu_op.cu:4356 */

/* ---- optimisers ----------------------------------------------------------- */
int DLGpuSgdUpdate(DLArrayHandle output, const DLArrayHandle m, float b,
                   void **cudaStream);                                                /* src/gpu_op.cu:4609 */
int DLGpuAdam_mv(DLArrayHandle m, DLArrayHandle v, const DLArrayHandle g,
                 float b1, float b2, void **cudaStream);                              /* src/gpu_op.cu:4511 */
int DLGpuAdam(DLArrayHandle output, const DLArrayHandle m, const DLArrayHandle v,
              float b1t, float b2t, float e, float learning_rate, void **cudaStream); /* src/gpu_op.cu:4471 */
/* multi-tensor variants over a device-resident pointer table */
int DLGpuGetIndextoVaribaleNumberCudaPointer(int *index_to_number, int *prefix,
                                             int count, void ***result);              /* src/gpu_op.cu:4628 */
int DLGpuGetN2CudaPointer(void **output, void **g, int number, void ****result);      /* src/gpu_op.cu:4653 */
int DLGpuGetN4CudaPointer(void **output, void **m, void **v, void **g, int number,
                          void ****result);                                           /* src/gpu_op.cu:4674 */
int DLGpuSgd_o(void ****n2list, const void ***indexlist, const int count,
               const float learning_rate);                                            /* src/gpu_op.cu:4840 */
int DLGpuAdam_o(void ****n4list, const void ***indexlist, const int count,
                const float b1, const float b2, const float b1t, const float b2t,
                const float e, const float learning_rate);                            /* src/gpu_op.cu:4865 */

/* ==== additions with no counterpart in the reference ====================== */

/* Data-parallel training across the GPUs of one box (one process per GPU).
 * After TfDpInit the optimiser entry points exchange gradients: DLGpuSgdUpdate, and
 * the DLGpuAdam_mv + DLGpuAdam pair, sum the gradient over all ranks (bucketed NCCL
 * all-reduce on a side stream, overlapped with the rest of the backward pass) and
 * apply the update with the mean gradient (SGD: w -= (lr / world) * sum_r g_r).
 * `nccl_id_path` names a file rank 0 creates; the other ranks wait for it, at most
 * TINYFLOW_DP_INIT_TIMEOUT_S seconds (default 120).  Returns 0 on success. */
int TfDpInit(int rank, int world_size, const char *nccl_id_path);
/* Flush every pending bucket and make the stream wait for the updates (end of a
 * step).  A blocking host<->device DLArrayCopyFromTo does the same, so a training
 * loop that knows nothing of this layer stays correct.  Returns -1 if NCCL reported
 * an asynchronous error (the communicator is then aborted). */
int TfDpFlush(void **cudaStream);
/* Waits (at most TINYFLOW_DP_TIMEOUT_S seconds, default 300) for the communication
 * stream, then releases the communicator; -1 if the wait ran out (communicator aborted). */
int TfDpShutdown(void);
int TfDpStats(long long *bytes_reduced, long long *allreduces);   /* totals since TfDpInit */
int TfDpStats2(long long *bytes_reduced, long long *allreduces, long long *apply_launches,
               long long *early_closes);                          /* + update launches, early bucket closes */
/* Host-only: the bucket each gradient tensor lands in, given tensor sizes (floats) in arrival order and the
 * bucket capacity; a tensor larger than the capacity gets -(id+1).  Returns the number of buckets. */
int TfDpPlanBuckets(const long long *counts, int n, long long capacity_floats, int *bucket_of);
/* The same walk with the early close the exchange applies from its second step on: once all but `tail_floats`
 * of the step's `step_total_floats` have arrived, the open bucket is closed (once per step), so that the last,
 * un-overlapped all-reduce is small.  step_total_floats = 0 plans a first step. */
int TfDpPlanBucketsTail(const long long *counts, int n, long long capacity_floats, long long step_total_floats,
                        long long tail_floats, int *bucket_of);

/* Allocation-free twin of DLGpuReduceSumAll (no counterpart in the reference): output[0] = sum of all
 * elements of input, with the per-block partial sums kept in a fixed 16 KiB array inside the library
 * instead of pooled memory, for callers that must not allocate while they run.  At most 33,554,432 input
 * elements (-1 beyond that).  All calls share the array, so calls that overlap on the GPU race.  The first
 * call on a device resolves the array's address and should precede any stream capture. */
int DLGpuReduceSumAllStatic(const DLArrayHandle input, DLArrayHandle output, void **cudaStream);

/* Test / profiling hooks. */
int TfPoolingArgmax(const DLArrayHandle input, int32_t *indices_dev, void ***cudnnlist,
                    void **cudaStream);   /* first-maximum index (h*W+w in the input plane) per output */
int TfDeviceSynchronize(void);
int TfKernelTimingEnable(int level);      /* CUDA-event timing per kernel family: 0 off, 1 contractions, 2 all; resets the table */
int TfKernelTimingReport(char *buf, int buflen);  /* JSON rows {name, launches, ms, flops, bytes} */
int TfLaunchCount(long long *count);      /* kernels launched by this library so far */
int TfFusedReluPackCount(long long *count); /* ReLU forward calls that also wrote the next convolution's packed operand */
int TfFusedReluBnBackwardCount(long long *count); /* ReLU backward calls that ran inside the batch-norm backward kernel called next */
int TfFusedAddReluCount(long long *count);        /* elementwise sums that were computed by the ReLU forward kernel called next */
int TfSetContractionPath(int path);       /* 0 = auto, 1 = force CUDA-core path, 2 = force tcgen05 path */
int TfLastContractionPath(void);          /* engine that served this thread's last matmul / convolution: 1 = CUDA cores, 2 = tensor cores */
/* Arithmetic of the tensor-core path: 0 = 3xFP16 (default; fp16 hi/lo pairs of the operand scaled by a per-tensor
 * power of two), 1 = 3xTF32 (tf32 hi/lo pairs, no scaling, half the tensor rate and twice the operand bytes).
 * Also settable with the environment variable TINYFLOW_ARITH=3xfp16|3xtf32.  Takes effect at the next call. */
int TfSetArithmetic(int arithmetic);
int TfGetArithmetic(void);
/* A tensor-core kernel whose barrier wait ran out raises a sticky error word and later launches are refused;
 * TfTensorPathError reads it, TfClearTensorPathError resets it once the cause has been dealt with. */
int TfTensorPathError(void);
int TfClearTensorPathError(void);
/* Launches a one-thread kernel that waits, with the tensor path's bounded-wait helper and a limit of
 * `limit_cycles` GPU clock cycles, on a barrier nothing ever arms: the wait gives up and raises the error word.
 * Lets a test see the time-out path end to end without a stuck kernel. */
int TfTensorPathTimeoutProbe(long long limit_cycles, void **cudaStream);
int TfLastError(char *buf, int buflen);   /* message of the last -1 return on this thread */
int TfAllocatorStats(long long *bytes_in_use, long long *bytes_cached);
int TfReleaseCachedMemory(void);

#ifdef __cplusplus
}
#endif
#endif /* TINYFLOW_B200_C_RUNTIME_API_H_ */

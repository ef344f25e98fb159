"""ctypes wrappers over the DLGpu* C-ABI; host-side mirror of pycode/tinyflow/gpu_op.py.

Function names, argument order and return values are the reference's (citations give the
reference wrapper each one mirrors), so code written against the reference module runs
against this one.  Wrappers that can report a soft out-of-memory return the number of
bytes the library failed to allocate (0 on success), as the reference does.
"""
from __future__ import annotations

import ctypes

from . import ndarray as _nd
from ._base import _LIB, c_array, check_call, new_cell

_F = ctypes.c_float
_DATAFORMAT = {"NCHW": 0, "NHWC": 1}
_PADDING = {"SAME": 1, "VALID": 0}
_POOLING = {"max": 0, "mean": 1}
_ACTIVATION = {"sigmoid": 0, "relu": 1, "tanh": 2, "softmax": 3}
_BATCHNORM = {"pre_activation": 0, "spatial": 1}


def _h(arr):
    assert isinstance(arr, _nd.NDArray), "expected an NDArray, got %r" % type(arr)
    return arr.handle


def _code(table, key):
    if key not in table:
        raise AssertionError("unknown option %r (expected one of %s)" % (key, sorted(table)))
    return table[key]


def _short_cell():
    return ctypes.pointer(ctypes.c_int(0))


# ---- handles (gpu_op.py:8-35) --------------------------------------------------------------
def create_cudaStream():
    cell = new_cell(2)
    check_call(_LIB.DLGpuCreatecudaStream(cell))
    return cell


def destroy_cudaStream(cudaStream):
    check_call(_LIB.DLGpuDestroycudaStream(cudaStream))


def create_cudnnHandle(cudaStream):
    cell = new_cell(2)
    check_call(_LIB.DLGpuCreatecudnnHandle(cell, cudaStream))
    return cell


def destroy_cudnnHandle(cudnnHandle):
    check_call(_LIB.DLGpuDestroycudnnHandle(cudnnHandle))


def create_cublasHandle(cudaStream):
    cell = new_cell(2)
    check_call(_LIB.DLGpuCreatecublasHandle(cell, cudaStream))
    return cell


def destroy_cublasHandle(cublasHandle):
    check_call(_LIB.DLGpuDestroycublasHandle(cublasHandle))


# ---- fill / broadcast / reduce (gpu_op.py:41-176) ------------------------------------------
def array_set(arr, value, cudaStream):
    check_call(_LIB.DLGpuArraySet(_h(arr), _F(value), cudaStream))


def broadcast_to(in_arr, out_arr, type, cudaStream):
    fn = {"NHWC": _LIB.DLGpuBroadcastTo0, "NCHW": _LIB.DLGpuBroadcastTo1}[type]
    check_call(fn(_h(in_arr), _h(out_arr), cudaStream))


def broadcast_to_backward(in_arr, out_arr, type):
    fn = {"NHWC": _LIB.DLGpuBroadcastToBackward0, "NCHW": _LIB.DLGpuBroadcastToBackward1}[type]
    check_call(fn(_h(in_arr), _h(out_arr)))


def reduce_sum_get_real_shape(input_shapes, output_shapes, dataformat):
    """Shapes handed to the reduce descriptor: reduced axes become 1 (gpu_op.py:83-119)."""
    assert len(output_shapes) == 1
    n = len(input_shapes)
    if dataformat == "NCHW":
        assert 3 <= n <= 5 and input_shapes[1] == output_shapes[0]
        return input_shapes, (1, output_shapes[0]) + (1,) * (n - 2)
    if dataformat == "NHWC":
        if n == 1:
            assert output_shapes[0] == 1
            return (1, 1, input_shapes[0]), (1, 1, 1)
        if n == 2:
            assert output_shapes[0] in (1, input_shapes[1])
            return (1, input_shapes[0], input_shapes[1]), (1, 1, output_shapes[0])
        assert n <= 5 and input_shapes[-1] == output_shapes[0]
        return input_shapes, (1,) * (n - 1) + (output_shapes[0],)
    raise AssertionError("unknown data format %r" % (dataformat,))


def reduce_sum_get_cudnnlist(input_shapes, output_shapes, dataformat, cudnnHandle):
    cell = new_cell(3)
    check_call(_LIB.DLGReduceSumGetCudnnlist(c_array(ctypes.c_int, list(input_shapes)), c_array(ctypes.c_int, list(output_shapes)),
                                             len(input_shapes), _code(_DATAFORMAT, dataformat), cell, cudnnHandle))
    return cell


def reduce_sum_new(in_arr, out_arr, cudnnlist, cudnnHandle, cudaStream):
    short = _short_cell()
    check_call(_LIB.DLGpuReduceSum(_h(in_arr), _h(out_arr), cudnnlist, cudnnHandle, short, cudaStream))
    return _LIB.getInt(short)


def reduce_sum_axis_zero(in_arr, out_arr):
    check_call(_LIB.DLGpuReduceSumAxisZero(_h(in_arr), _h(out_arr)))


def reduce_sum(in_arr, out_arr, axis=-1):
    if axis == -1:
        check_call(_LIB.DLGpuReduceSumAll(_h(in_arr), _h(out_arr)))
    else:
        check_call(_LIB.DLGpuReduceSumAxisN(_h(in_arr), _h(out_arr), ctypes.c_int(axis)))


def reduce_sum_backward(dout_arr, din_arr, axis):
    if axis == -1:
        check_call(_LIB.DLGpuReduceSumAllBackward(_h(dout_arr), _h(din_arr)))
    else:
        check_call(_LIB.DLGpuReduceSumAxisNBackward(_h(dout_arr), _h(din_arr), ctypes.c_int(axis)))


def reduce_sum_get_outshape(in_shape, axis):
    if axis == -1 or len(in_shape) == 1:
        return (1,)
    return tuple(d for i, d in enumerate(in_shape) if i != axis)


def get_shape_size(shape):
    size = 1
    for d in shape:
        size *= d
    return size


# ---- elementwise (gpu_op.py:179-270) -------------------------------------------------------
def matrix_elementwise_add(matA, matB, matC, cudaStream):
    check_call(_LIB.DLGpuMatrixElementwiseAdd(_h(matA), _h(matB), _h(matC), cudaStream))


def matrix_elementwise_add_by_const(in_mat, val, out_mat, cudaStream):
    check_call(_LIB.DLGpuMatrixElementwiseAddByConst(_h(in_mat), _F(val), _h(out_mat), cudaStream))


def matrix_elementwise_multiply(matA, matB, matC, cudaStream):
    check_call(_LIB.DLGpuMatrixElementwiseMultiply(_h(matA), _h(matB), _h(matC), cudaStream))


def matrix_elementwise_multiply_by_const(in_mat, val, out_mat, cudaStream):
    check_call(_LIB.DLGpuMatrixMultiplyByConst(_h(in_mat), _F(val), _h(out_mat), cudaStream))


def matrix_multiply(matA, transA, matB, transB, matC, cublasHandle, cudaStream):
    check_call(_LIB.DLGpuMatrixMultiply(_h(matA), bool(transA), _h(matB), bool(transB), _h(matC), cublasHandle, cudaStream))


def relu(in_arr, out_arr):
    check_call(_LIB.DLGpuRelu(_h(in_arr), _h(out_arr)))


def relu_gradient(in_arr, in_grad_arr, out_arr):
    check_call(_LIB.DLGpuReluGradient(_h(in_arr), _h(in_grad_arr), _h(out_arr)))


def softmax(in_arr, out_arr, cudaStream):
    check_call(_LIB.DLGpuSoftmax(_h(in_arr), _h(out_arr), cudaStream))


def softmax_cross_entropy(in_arr_a, in_arr_b, out_arr, cudaStream):
    check_call(_LIB.DLGpuSoftmaxCrossEntropy(_h(in_arr_a), _h(in_arr_b), _h(out_arr), cudaStream))


def cross_entropy(in_arr_a, in_arr_b, out_arr):
    check_call(_LIB.DLGpuCrossEntropy(_h(in_arr_a), _h(in_arr_b), _h(out_arr)))


def matrix_exp(in_arr, out_arr):
    check_call(_LIB.DLGpuMatrixExp(_h(in_arr), _h(out_arr)))


def matrix_log(in_arr, out_arr, cudaStream):
    check_call(_LIB.DLGpuMatrixLog(_h(in_arr), _h(out_arr), cudaStream))


def matrix_reverse(in_arr, out_arr):
    check_call(_LIB.DLGpuMatrixReverse(_h(in_arr), _h(out_arr)))


def matrix_pow(in_arr, val, out_arr):
    check_call(_LIB.DLGpuMatrixPow(_h(in_arr), _F(val), _h(out_arr)))


# ---- convolution (gpu_op.py:291-339, 435-462) ----------------------------------------------
def convolution_2d_forward_get_out_shape(input_shapes, filter_shapes, dataformat, padding, u, v):
    assert len(input_shapes) == 4 and len(filter_shapes) == 4
    out = c_array(ctypes.c_int, [0, 0, 0, 0])
    cell = new_cell(3)
    check_call(_LIB.DLGpuConvolution2DForwardGetOutShape(c_array(ctypes.c_int, list(input_shapes)), c_array(ctypes.c_int, list(filter_shapes)), out,
                                                         _code(_DATAFORMAT, dataformat), _code(_PADDING, padding), int(u), int(v), cell))
    return tuple(out), cell


def _with_short(fn, *args):
    short = _short_cell()
    check_call(fn(*args[:-1], short, args[-1]))
    return _LIB.getInt(short)


def convolution_2d_forward(in_arr, in_filter, out_arr, cudnnlist, cudnnHandle, cudaStream):
    return _with_short(_LIB.DLGpuConvolution2DForward, _h(in_arr), _h(in_filter), _h(out_arr), cudnnlist, cudnnHandle, cudaStream)


def convolution_backward_filter(in_arr, dout_arr, in_filter, in_dfilter, cudnnlist, cudnnHandle, cudaStream):
    return _with_short(_LIB.DLGpuConvolutionBackwardFilter, _h(in_arr), _h(dout_arr), _h(in_filter), _h(in_dfilter), cudnnlist, cudnnHandle, cudaStream)


def convolution_backward_data(in_arr, dout_arr, in_filter, dinput_arr, cudnnlist, cudnnHandle, cudaStream):
    return _with_short(_LIB.DLGpuConvolutionBackwardData, _h(in_arr), _h(dout_arr), _h(in_filter), _h(dinput_arr), cudnnlist, cudnnHandle, cudaStream)


# ---- pooling (gpu_op.py:373-396, 602-626) --------------------------------------------------
def pooling_2d_forward_get_out_shape(input_shapes, dataformat, poolingMode, padding_h, padding_w, u, v, filter_h, filter_w):
    assert len(input_shapes) == 4
    out = c_array(ctypes.c_int, [0, 0, 0, 0])
    cell = new_cell(3)
    check_call(_LIB.DLGpuPooling2DForwardGetOutShape(c_array(ctypes.c_int, list(input_shapes)), out, _code(_DATAFORMAT, dataformat), _code(_POOLING, poolingMode),
                                                     int(padding_h), int(padding_w), int(u), int(v), int(filter_h), int(filter_w), cell))
    return tuple(out), cell


def pooling_2d_forward(in_arr, out_arr, cudnnlist, cudnnHandle, cudaStream):
    check_call(_LIB.DLGpuPooling2DForward(_h(in_arr), _h(out_arr), cudnnlist, cudnnHandle, cudaStream))


def pooling_2d_backward(in_arr, out_arr, dout_arr, din_arr, cudnnlist, cudnnHandle, cudaStream):
    check_call(_LIB.DLGpuPooling2DBackward(_h(in_arr), _h(out_arr), _h(dout_arr), _h(din_arr), cudnnlist, cudnnHandle, cudaStream))


# ---- activation (gpu_op.py:497-555) ---------------------------------------------------------
def activation_get_cudnnlist(input_shapes, dataformat, activationMode):
    cell = new_cell(3)
    check_call(_LIB.DLGpuActivationGetCudnnlist(c_array(ctypes.c_int, list(input_shapes)), len(input_shapes), _code(_DATAFORMAT, dataformat),
                                                _code(_ACTIVATION, activationMode), cell))
    return cell


def activation_forward(input, output, activationMode, cudnnlist, cudnnHandle, cudaStream):
    check_call(_LIB.DLGpuActivationForward(_h(input), _h(output), _code(_ACTIVATION, activationMode), cudnnlist, cudnnHandle, cudaStream))


def activation_backward(input, dinput, output, doutput, activationMode, cudnnlist, cudnnHandle, cudaStream):
    check_call(_LIB.DLGpuActivationBackward(_h(input), _h(dinput), _h(output), _h(doutput), _code(_ACTIVATION, activationMode), cudnnlist, cudnnHandle, cudaStream))


# ---- dropout (gpu_op.py:557-571, 657-692) ---------------------------------------------------
def get_input_descriptor(input_shapes, dataformat):
    cell = new_cell(3)
    check_call(_LIB.DLGpuGetInputDescriptor(c_array(ctypes.c_int, list(input_shapes)), len(input_shapes), _code(_DATAFORMAT, dataformat), cell))
    return cell


def dropout_forward(input, output, dataformat, dropout, seed, inputd, cudnnHandle, cudaStream):
    assert seed >= 0
    reserve = new_cell(2)
    cudnnlist = new_cell(3)
    short = _short_cell()
    check_call(_LIB.DLGpuDropoutForward(_h(input), _h(output), _code(_DATAFORMAT, dataformat), _F(dropout), ctypes.c_int(seed), reserve, inputd, cudnnlist,
                                        cudnnHandle, short, cudaStream))
    return reserve, cudnnlist, _LIB.getInt(short)


def dropout_backward(doutput, dinput, reserveSpace_p, cudnnlist, cudnnHandle, cudaStream):
    check_call(_LIB.DLGpuDropoutBackward(_h(doutput), _h(dinput), reserveSpace_p, cudnnlist, cudnnHandle, cudaStream))


# ---- losses (gpu_op.py:694-745, 866-879) ----------------------------------------------------
def L1loss(in_arr_a, in_arr_b, out_arr):
    check_call(_LIB.DLGpuL1loss(_h(in_arr_a), _h(in_arr_b), _h(out_arr)))


def L2loss(in_arr_a, in_arr_b, out_arr):
    check_call(_LIB.DLGpuL2loss(_h(in_arr_a), _h(in_arr_b), _h(out_arr)))


def l1loss_gradient(in_arr, in_arr1, in_grad_arr, out_arr):
    check_call(_LIB.DLGpuL1LossGradient(_h(in_arr), _h(in_arr1), _h(in_grad_arr), _h(out_arr)))


def l2loss_gradient(in_arr, in_arr1, in_grad_arr, out_arr):
    check_call(_LIB.DLGpuL2LossGradient(_h(in_arr), _h(in_arr1), _h(in_grad_arr), _h(out_arr)))


def L1regular(in_arr_a, out_arr):
    check_call(_LIB.DLGpuL1regular(_h(in_arr_a), _h(out_arr)))


def L2regular(in_arr_a, out_arr):
    check_call(_LIB.DLGpuL2regular(_h(in_arr_a), _h(out_arr)))


def l1regular_gradient(in_arr, in_grad_arr, out_arr):
    check_call(_LIB.DLGpuL1regularGradient(_h(in_arr), _h(in_grad_arr), _h(out_arr)))


def l2regular_gradient(in_arr, in_grad_arr, out_arr):
    check_call(_LIB.DLGpuL2regularGradient(_h(in_arr), _h(in_grad_arr), _h(out_arr)))


def cross(x, y, output, mean, cudaStream):
    check_call(_LIB.DLGpuCross(_h(x), _h(y), _h(output), _F(mean), cudaStream))


def cross_backward(x, y, doutput, output, mean, cudaStream):
    check_call(_LIB.DLGpuCrossBackward(_h(x), _h(y), _h(doutput), _h(output), _F(mean), cudaStream))


# ---- concat (gpu_op.py:746-766) --------------------------------------------------------------
def concat_forward(in_arr_a, in_arr_b, out_arr, cudaStream):
    check_call(_LIB.DLGpuConcatForward(_h(in_arr_a), _h(in_arr_b), _h(out_arr), cudaStream))


def concat_a_backward(in_arr_a, in_arr_b, out_arr, din_arr_a, cudaStream):
    check_call(_LIB.DLGpuConcataBackward(_h(in_arr_a), _h(in_arr_b), _h(out_arr), _h(din_arr_a), cudaStream))


def concat_b_backward(in_arr_a, in_arr_b, out_arr, din_arr_b, cudaStream):
    check_call(_LIB.DLGpuConcatbBackward(_h(in_arr_a), _h(in_arr_b), _h(out_arr), _h(din_arr_b), cudaStream))


# ---- batch normalisation (gpu_op.py:771-843) -------------------------------------------------
def bn_get_cudnnlist(input_shapes, dataformat, batchNormMode):
    mean_p, var_p, cell = new_cell(2), new_cell(2), new_cell(3)
    check_call(_LIB.DLGpuBatchNormalizationGetCudnnlist(c_array(ctypes.c_int, list(input_shapes)), len(input_shapes), _code(_DATAFORMAT, dataformat),
                                                        _code(_BATCHNORM, batchNormMode), mean_p, var_p, cell))
    return mean_p, var_p, cell


def bn_forward(input, output, batchNormMode, n, mean_p, var_p, cudnnlist, cudnnHandle, cudaStream):
    short = _short_cell()
    check_call(_LIB.DLGpuBatchNormalizationForward(_h(input), _h(output), _code(_BATCHNORM, batchNormMode), int(n), mean_p, var_p, cudnnlist, cudnnHandle, short, cudaStream))
    return _LIB.getInt(short)


def bn_backward(input, doutput, dinput, batchNormMode, mean_p, var_p, cudnnlist, cudnnHandle, cudaStream):
    short = _short_cell()
    check_call(_LIB.DLGpuBatchNormalizationBackward(_h(input), _h(doutput), _h(dinput), _code(_BATCHNORM, batchNormMode), mean_p, var_p, cudnnlist, cudnnHandle, short, cudaStream))
    return _LIB.getInt(short)


# ---- optimisers (gpu_op.py:846-958) -----------------------------------------------------------
def adam_compute(output, m, v, b1t, b2t, e, learning_rate, cudaStream):
    check_call(_LIB.DLGpuAdam(_h(output), _h(m), _h(v), _F(b1t), _F(b2t), _F(e), _F(learning_rate), cudaStream))


def adam_mv(m, v, g, b1, b2, cudaStream):
    check_call(_LIB.DLGpuAdam_mv(_h(m), _h(v), _h(g), _F(b1), _F(b2), cudaStream))


def sgd_update(output, g, learning_rate, cudaStream):
    check_call(_LIB.DLGpuSgdUpdate(_h(output), _h(g), _F(learning_rate), cudaStream))


def get_index_to_VaribaleNumber_cuda_pointer(index_to_Variable, prefix_list, index_count):
    cell = new_cell(3)
    check_call(_LIB.DLGpuGetIndextoVaribaleNumberCudaPointer(c_array(ctypes.c_int, list(index_to_Variable)), c_array(ctypes.c_int, list(prefix_list)),
                                                             ctypes.c_int(index_count), cell))
    return cell


def get_n2_cuda_pointer(output, g, number):
    cell = new_cell(4)
    check_call(_LIB.DLGpuGetN2CudaPointer(c_array(ctypes.c_void_p, list(output)), c_array(ctypes.c_void_p, list(g)), ctypes.c_int(number), cell))
    return cell


def get_n4_cuda_pointer(output, m, v, g, number):
    cell = new_cell(4)
    check_call(_LIB.DLGpuGetN4CudaPointer(c_array(ctypes.c_void_p, list(output)), c_array(ctypes.c_void_p, list(m)), c_array(ctypes.c_void_p, list(v)),
                                          c_array(ctypes.c_void_p, list(g)), ctypes.c_int(number), cell))
    return cell


def sgd_compute_o(n2list, indexinfolist, count, learning_rate):
    check_call(_LIB.DLGpuSgd_o(n2list, indexinfolist, ctypes.c_int(count), _F(learning_rate)))


def adam_compute_o(n4list, indexinfolist, count, b1, b2, b1t, b2t, e, learning_rate):
    check_call(_LIB.DLGpuAdam_o(n4list, indexinfolist, ctypes.c_int(count), _F(b1), _F(b2), _F(b1t), _F(b2t), _F(e), _F(learning_rate)))


def getInt(intp):
    return _LIB.getInt(intp)


def testPcie():
    check_call(_LIB.testPcie())


# ---- additions with no counterpart in the reference -------------------------------------------
def reduce_sum_all_static(in_arr, out_arr, cudaStream):
    """Sum of all elements into out_arr (one element) without any device allocation: the twin of
    ``reduce_sum(in_arr, out_arr, -1)`` for callers that must not allocate while they run.  Refuses inputs
    above 33,554,432 elements; calls share one fixed scratch array, so keep them on a single stream."""
    check_call(_LIB.DLGpuReduceSumAllStatic(_h(in_arr), _h(out_arr), cudaStream))


def device_synchronize():
    check_call(_LIB.TfDeviceSynchronize())


def launch_count() -> int:
    n = ctypes.c_longlong(0)
    _LIB.TfLaunchCount(ctypes.byref(n))
    return n.value


def set_contraction_path(path: int):
    """0 = automatic, 1 = CUDA-core kernels only, 2 = tcgen05 kernels only (error if a shape is not taken)."""
    check_call(_LIB.TfSetContractionPath(int(path)))


def last_contraction_path() -> int:
    """Engine that served this thread's most recent matmul / convolution: 1 = CUDA cores, 2 = tensor cores."""
    return int(_LIB.TfLastContractionPath())


def set_tensor_arithmetic(name: str):
    """"3xfp16" (default) or "3xtf32": how the tensor-core path represents fp32 operands."""
    check_call(_LIB.TfSetArithmetic({"3xfp16": 0, "3xtf32": 1}[name]))


def tensor_arithmetic() -> str:
    return {0: "3xfp16", 1: "3xtf32"}[int(_LIB.TfGetArithmetic())]


def allocator_stats():
    """(bytes handed out and not yet freed, bytes cached in the pools) of the device allocator."""
    used, cached = ctypes.c_longlong(0), ctypes.c_longlong(0)
    check_call(_LIB.TfAllocatorStats(ctypes.byref(used), ctypes.byref(cached)))
    return used.value, cached.value


def release_cached_memory():
    """Returns every cached (free) block of the device and pinned-host pools to the driver."""
    check_call(_LIB.TfReleaseCachedMemory())


def tensor_path_error() -> int:
    """Non-zero after a tensor-core kernel gave up on a barrier wait (sticky until cleared)."""
    return int(_LIB.TfTensorPathError())


def clear_tensor_path_error():
    check_call(_LIB.TfClearTensorPathError())


def fused_relu_bn_backward_count() -> int:
    """How many ReLU backward calls so far were computed inside the batch-norm backward kernel that was called next."""
    n = ctypes.c_longlong(0)
    check_call(_LIB.TfFusedReluBnBackwardCount(ctypes.byref(n)))
    return n.value


def fused_add_relu_count() -> int:
    """How many elementwise sums so far were computed inside the ReLU forward kernel that was called next."""
    n = ctypes.c_longlong(0)
    check_call(_LIB.TfFusedAddReluCount(ctypes.byref(n)))
    return n.value


def fused_relu_pack_count() -> int:
    """How many ReLU forward calls so far also wrote the packed operand of the convolution that reads their output."""
    n = ctypes.c_longlong(0)
    check_call(_LIB.TfFusedReluPackCount(ctypes.byref(n)))
    return n.value


# ---- 1-D / 3-D convolution (forward) and pooling (gpu_op.py:277-313, 368-404, 406-500, 577-660) ----------------------
def convolution_1d_forward_get_out_shape(input_shapes, filter_shapes, dataformat, padding, v):
    assert len(input_shapes) == 3 and len(filter_shapes) == 3
    out = c_array(ctypes.c_int, [0, 0, 0])
    cell = new_cell(3)
    check_call(_LIB.DLGpuConvolution1DForwardGetOutShape(c_array(ctypes.c_int, list(input_shapes)), c_array(ctypes.c_int, list(filter_shapes)), out,
                                                         _code(_DATAFORMAT, dataformat), _code(_PADDING, padding), int(v), cell))
    return tuple(out), cell


def convolution_1d_forward(in_arr, in_filter, out_arr, cudnnlist, cudnnHandle):
    short = _short_cell()
    check_call(_LIB.DLGpuConvolution1DForward(_h(in_arr), _h(in_filter), _h(out_arr), cudnnlist, cudnnHandle, short))
    return _LIB.getInt(short)


def convolution_3d_forward_get_out_shape(input_shapes, filter_shapes, dataformat, padding, s1, s2, s3):
    assert len(input_shapes) == 5 and len(filter_shapes) == 5
    out = c_array(ctypes.c_int, [0] * 5)
    cell = new_cell(3)
    check_call(_LIB.DLGpuConvolution3DForwardGetOutShape(c_array(ctypes.c_int, list(input_shapes)), c_array(ctypes.c_int, list(filter_shapes)), out,
                                                         _code(_DATAFORMAT, dataformat), _code(_PADDING, padding), int(s1), int(s2), int(s3), cell))
    return tuple(out), cell


def convolution_3d_forward(in_arr, in_filter, out_arr, cudnnlist, cudnnHandle):
    short = _short_cell()
    check_call(_LIB.DLGpuConvolution3DForward(_h(in_arr), _h(in_filter), _h(out_arr), cudnnlist, cudnnHandle, short))
    return _LIB.getInt(short)


def pooling_1d_forward_get_out_shape(input_shapes, dataformat, poolingMode, padding_w, v, filter_w):
    assert len(input_shapes) == 3
    out = c_array(ctypes.c_int, [0, 0, 0])
    cell = new_cell(3)
    check_call(_LIB.DLGpuPooling1DForwardGetOutShape(c_array(ctypes.c_int, list(input_shapes)), out, _code(_DATAFORMAT, dataformat), _code(_POOLING, poolingMode),
                                                     int(padding_w), int(v), int(filter_w), cell))
    return tuple(out), cell


def pooling_1d_forward(in_arr, out_arr, cudnnlist, cudnnHandle):
    check_call(_LIB.DLGpuPooling1DForward(_h(in_arr), _h(out_arr), cudnnlist, cudnnHandle))


def pooling_1d_backward(in_arr, out_arr, dout_arr, din_arr, cudnnlist, cudnnHandle):
    check_call(_LIB.DLGpuPooling1DBackward(_h(in_arr), _h(out_arr), _h(dout_arr), _h(din_arr), cudnnlist, cudnnHandle))


def pooling_3d_forward_get_out_shape(input_shapes, dataformat, poolingMode, padding1, padding2, padding3, s1, s2, s3, filter1, filter2, filter3):
    assert len(input_shapes) == 5
    out = c_array(ctypes.c_int, [0] * 5)
    cell = new_cell(3)
    check_call(_LIB.DLGpuPooling3DForwardGetOutShape(c_array(ctypes.c_int, list(input_shapes)), out, _code(_DATAFORMAT, dataformat), _code(_POOLING, poolingMode),
                                                     int(padding1), int(padding2), int(padding3), int(s1), int(s2), int(s3), int(filter1), int(filter2), int(filter3), cell))
    return tuple(out), cell


def pooling_3d_forward(in_arr, out_arr, cudnnlist, cudnnHandle):
    check_call(_LIB.DLGpuPooling3DForward(_h(in_arr), _h(out_arr), cudnnlist, cudnnHandle))


def pooling_3d_backward(in_arr, out_arr, dout_arr, din_arr, cudnnlist, cudnnHandle):
    check_call(_LIB.DLGpuPooling3DBackward(_h(in_arr), _h(out_arr), _h(dout_arr), _h(din_arr), cudnnlist, cudnnHandle))

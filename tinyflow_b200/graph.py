"""Computation graph, operators and reverse-mode autodiff.

Host-side mirror of the graph half of pycode/tinyflow/autodiff.py: the same node and operator
names (``ad.Variable``, ``ad.matmul_op``, ``ad.convolution_2d_forward_op`` ...), the same
attributes on nodes, the same gradient graph (so the quirks of the reference — softmax-CE
gradient not divided by the batch, ``cross_op`` dividing by batch*classes — come out the same)
and the same operator protocol::

    op.compute(node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False)
    op.gradient(node, output_grad) -> [grad nodes]
    op.infer_shape(node, input_shapes, cudnnHandle) -> shape

``compute`` launches CUDA kernels through :mod:`tinyflow_b200.gpu_op`.  There is no CPU path:
``use_numpy=True`` raises.  Citations name the reference class each operator mirrors.
"""
from __future__ import annotations

import random
from functools import reduce as _reduce

from . import gpu_op, ndarray


class Node(object):
    """A graph node (autodiff.py:153-215)."""

    def __init__(self):
        self.inputs = []
        self.op = None
        self.const_attr = None
        self.name = ""
        self.index = 0
        self.array_status = 0
        self.control_message_in = []
        self.control_message_in_time = 0
        self.control_message_out = []
        self.control_message_out_time = 0
        self.recompute_list = []
        self.release_list = []
        self.runtime = 0.00001
        self.issgd = 0      # 1: optimiser node, updates its first input in place, owns no output
        self.isw = 0        # 1: parameter, 2: data placeholder, 3: relocated optimiser node

    def __add__(self, other):
        return add_op(self, other) if isinstance(other, Node) else add_byconst_op(self, other)

    def __mul__(self, other):
        return mul_op(self, other) if isinstance(other, Node) else mul_byconst_op(self, other)

    __radd__ = __add__
    __rmul__ = __mul__

    def __str__(self):
        return self.name

    __repr__ = __str__


def Variable(name):
    """A trainable parameter (fed through feed_dict, updated in place by the optimiser node)."""
    node = placeholder_op()
    node.name = name
    node.isw = 1
    return node


def Placeholder(name):
    """A data input (fed through feed_dict each step)."""
    node = placeholder_op()
    node.name = name
    node.isw = 2
    return node


def _no_numpy(use_numpy):
    if use_numpy:
        raise NotImplementedError("tinyflow_b200 has no CPU execution path (use_numpy=True is not available)")


class Op(object):
    """Base operator.  Subclasses set ``name`` and implement make/compute/gradient/infer_shape."""
    name = "Op"

    def _node(self, inputs, **attrs):
        node = Node()
        node.op = self
        node.inputs = list(inputs)
        node.name = self.name
        for k, v in attrs.items():
            setattr(node, k, v)
        return node

    def __call__(self, *args, **kwargs):
        return self._node([])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        raise NotImplementedError

    def gradient(self, node, output_grad):
        raise NotImplementedError

    def infer_shape(self, node, input_shapes, cudnnHandle):
        raise NotImplementedError


def _scalar_of(arr):
    return float(arr.asnumpy().reshape(-1)[0])


# ---- arithmetic (AddOp, AddByConstOp, MulOp, MulByConstOp: autodiff.py:302-438) ----------
class AddOp(Op):
    name = "+"

    def __call__(self, node_A, node_B):
        return self._node([node_A, node_B])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        a, b = input_vals
        if a.shape == b.shape:
            gpu_op.matrix_elementwise_add(a, b, output_val, cudaStream)
        elif b.shape == (1,):
            gpu_op.matrix_elementwise_add_by_const(a, _scalar_of(b), output_val, cudaStream)
        elif a.shape == (1,):
            gpu_op.matrix_elementwise_add_by_const(b, _scalar_of(a), output_val, cudaStream)
        else:
            raise ValueError("add: shapes %s and %s do not match" % (a.shape, b.shape))
        return 0

    def gradient(self, node, output_grad):
        return [output_grad, output_grad]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        a, b = input_shapes
        if a == b:
            return a
        return b if a == (1,) else a


class AddByConstOp(Op):
    name = "+"

    def __call__(self, node_A, const_val):
        return self._node([node_A], const_attr=const_val)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.matrix_elementwise_add_by_const(input_vals[0], node.const_attr, output_val, cudaStream)
        return 0

    def gradient(self, node, output_grad):
        return [output_grad]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


class MulOp(Op):
    name = "*"

    def __call__(self, node_A, node_B):
        return self._node([node_A, node_B])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        a, b = input_vals
        if a.shape == b.shape:
            gpu_op.matrix_elementwise_multiply(a, b, output_val, cudaStream)
        elif b.shape == (1,):
            gpu_op.matrix_elementwise_multiply_by_const(a, _scalar_of(b), output_val, cudaStream)
        elif a.shape == (1,):
            gpu_op.matrix_elementwise_multiply_by_const(b, _scalar_of(a), output_val, cudaStream)
        else:
            raise ValueError("mul: shapes %s and %s do not match" % (a.shape, b.shape))
        return 0

    def gradient(self, node, output_grad):
        return [node.inputs[1] * output_grad, node.inputs[0] * output_grad]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        a, b = input_shapes
        if a == b:
            return a
        return b if a == (1,) else a


class MulByConstOp(Op):
    name = "*"

    def __call__(self, node_A, const_val):
        return self._node([node_A], const_attr=const_val)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.matrix_elementwise_multiply_by_const(input_vals[0], node.const_attr, output_val, cudaStream)
        return 0

    def gradient(self, node, output_grad):
        return [node.const_attr * output_grad]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


# ---- MatMulOp (autodiff.py:441-516) -------------------------------------------------------
class MatMulOp(Op):
    name = "MatMul"

    def __call__(self, node_A, node_B, trans_A=False, trans_B=False):
        return self._node([node_A, node_B], matmul_attr_trans_A=trans_A, matmul_attr_trans_B=trans_B)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.matrix_multiply(input_vals[0], node.matmul_attr_trans_A, input_vals[1], node.matmul_attr_trans_B,
                               output_val, cublasHandle, cudaStream)
        return 0

    def gradient(self, node, output_grad):
        A, B = node.inputs
        tA, tB = node.matmul_attr_trans_A, node.matmul_attr_trans_B
        if not tA and not tB:      # Y = A B
            return [matmul_op(output_grad, B, False, True), matmul_op(A, output_grad, True, False)]
        if tA and not tB:          # Y = A^T B
            return [matmul_op(B, output_grad, False, True), matmul_op(A, output_grad, False, False)]
        if not tA and tB:          # Y = A B^T
            return [matmul_op(output_grad, B, False, False), matmul_op(output_grad, A, True, False)]
        return [matmul_op(B, output_grad, True, True), matmul_op(output_grad, A, True, True)]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        a, b = input_shapes
        rows = a[1] if node.matmul_attr_trans_A else a[0]
        cols = b[0] if node.matmul_attr_trans_B else b[1]
        return (rows, cols)


class PlaceholderOp(Op):
    name = ""

    def __call__(self):
        return self._node([])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        raise AssertionError("placeholder %s values provided by feed_dict" % node.name)

    def gradient(self, node, output_grad):
        return None

    def infer_shape(self, node, input_shapes, cudnnHandle):
        raise AssertionError("placeholder %s shape provided by feed_shape" % node.name)


class _FillLikeOp(Op):
    value = 0.0

    def __call__(self, node_A):
        return self._node([node_A])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.array_set(output_val, self.value, cudaStream)
        return 0

    def gradient(self, node, output_grad):
        return [zeroslike_op(node.inputs[0])]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


class ZerosLikeOp(_FillLikeOp):   # autodiff.py:537
    name = "Zeroslike"
    value = 0.0


class OnesLikeOp(_FillLikeOp):    # autodiff.py:562
    name = "Oneslike"
    value = 1.0


class ReduceSumAxisZeroOp(Op):    # autodiff.py:587
    name = "ReduceSumAxisZero"

    def __call__(self, node_A):
        return self._node([node_A])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.reduce_sum_axis_zero(input_vals[0], output_val)
        return 0

    def gradient(self, node, output_grad):
        return [broadcastto_op(output_grad, node.inputs[0])]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        s = input_shapes[0]
        return (1,) if len(s) == 1 else tuple(s[1:])


class BroadcastToOp(Op):          # autodiff.py:621
    name = "BroadcastTo"

    def __call__(self, node_A, node_B, type="NHWC"):
        return self._node([node_A, node_B], type=type)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.broadcast_to(input_vals[0], output_val, node.type, cudaStream)
        return 0

    def gradient(self, node, output_grad):
        return [broadcastto_gradient_op(output_grad, node.inputs[0], node.type), zeroslike_op(node.inputs[1])]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[1]


class BroadcastToGradientOp(Op):  # autodiff.py:648
    name = "BroadcastToGradient"

    def __call__(self, node_A, node_B, type):
        return self._node([node_A, node_B], type=type, cudnnlist=[0])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        return gpu_op.reduce_sum_new(input_vals[0], output_val, node.cudnnlist[0], cudnnHandle, cudaStream)

    def infer_shape(self, node, input_shapes, cudnnHandle):
        ins, outs = gpu_op.reduce_sum_get_real_shape(input_shapes[0], input_shapes[1], node.type)
        node.cudnnlist[0] = gpu_op.reduce_sum_get_cudnnlist(ins, outs, node.type, cudnnHandle)
        return input_shapes[1]


class SoftmaxCrossEntropyOp(Op):  # autodiff.py:689
    name = "SoftmaxXEntropy"

    def __call__(self, node_A, node_B):
        return self._node([node_A, node_B])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.softmax_cross_entropy(input_vals[0], input_vals[1], output_val, cudaStream)
        return 0

    def gradient(self, node, output_grad):
        return [(softmax_op(node.inputs[0]) + -1 * node.inputs[1]) * output_grad, zeroslike_op(node.inputs[1])]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return (1,)


class _UnaryOp(Op):
    def __call__(self, node_A):
        return self._node([node_A])

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


class SoftmaxOp(_UnaryOp):        # autodiff.py:719
    name = "Softmax"

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.softmax(input_vals[0], output_val, cudaStream)
        return 0


class ReluOp(_UnaryOp):           # autodiff.py:744
    name = "Relu"

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.relu(input_vals[0], output_val)
        return 0

    def gradient(self, node, output_grad):
        return [relu_gradient_op(node.inputs[0], output_grad)]


class ReluGradientOp(Op):         # autodiff.py:767
    name = "ReluGradient"

    def __call__(self, node_A, node_B):
        return self._node([node_A, node_B])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.relu_gradient(input_vals[0], input_vals[1], output_val)
        return 0

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


class ExpOp(_UnaryOp):            # autodiff.py:792
    name = "Exp"

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.matrix_exp(input_vals[0], output_val)
        return 0

    def gradient(self, node, output_grad):
        return [output_grad * exp_op(node.inputs[0])]


class LogOp(_UnaryOp):            # autodiff.py:814
    name = "Log"

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.matrix_log(input_vals[0], output_val, cudaStream)
        return 0

    def gradient(self, node, output_grad):
        return [output_grad * reverse_op(node.inputs[0])]


class ReverseOp(_UnaryOp):        # autodiff.py:836
    name = "Reverse"

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.matrix_reverse(input_vals[0], output_val)
        return 0

    def gradient(self, node, output_grad):
        return [-1 * output_grad * reverse_op(node.inputs[0]) * reverse_op(node.inputs[0])]


class PowOp(Op):                  # autodiff.py:858
    name = "Pow"

    def __call__(self, node_A, val):
        return self._node([node_A], const_attr=val)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.matrix_pow(input_vals[0], node.const_attr, output_val)
        return 0

    def gradient(self, node, output_grad):
        return [node.const_attr * output_grad * pow_op(node.inputs[0], node.const_attr - 1)]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


# ---- convolution (Convolution2DForwardOp / Convolution2DBackwardOp: autodiff.py:944-1013) --
class Convolution2DForwardOp(Op):
    name = "Convolution2DForward"

    def __call__(self, node_A, node_B, dataformat, padding, u, v):
        return self._node([node_A, node_B], dataformat=dataformat, padding=padding, u=u, v=v, cudnnlist=[0])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        return gpu_op.convolution_2d_forward(input_vals[0], input_vals[1], output_val, node.cudnnlist[0], cudnnHandle, cudaStream)

    def gradient(self, node, output_grad):
        x, w = node.inputs
        return [convolution_2d_backward_op(x, w, output_grad, 0, node.padding, node.u, node.v, node.cudnnlist),
                convolution_2d_backward_op(x, w, output_grad, 1, node.padding, node.u, node.v, node.cudnnlist)]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        out, node.cudnnlist[0] = gpu_op.convolution_2d_forward_get_out_shape(input_shapes[0], input_shapes[1], node.dataformat,
                                                                             node.padding, node.u, node.v)
        return out


class Convolution2DBackwardOp(Op):
    name = "Convolution2DBackward"

    def __call__(self, node_A, node_B, node_C, type, padding, u, v, cudnnlist):
        # type 0: gradient w.r.t. the input, type 1: gradient w.r.t. the filter
        return self._node([node_A, node_B, node_C], type=type, padding=padding, u=u, v=v, cudnnlist=cudnnlist)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        x, w, dy = input_vals
        if node.type == 0:
            return gpu_op.convolution_backward_data(x, dy, w, output_val, node.cudnnlist[0], cudnnHandle, cudaStream)
        return gpu_op.convolution_backward_filter(x, dy, w, output_val, node.cudnnlist[0], cudnnHandle, cudaStream)

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0] if node.type == 0 else input_shapes[1]


# ---- reshapes (FlattenOp, SqueezeOp and their gradients: autodiff.py:1081-1122, 1987-2026) --
class _CopyReshapeOp(Op):
    def __call__(self, node_A):
        return self._node([node_A])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        input_vals[0].copyto(output_val, cudaStream)
        return 0


class FlattenOp(_CopyReshapeOp):
    name = "Flatten"

    def gradient(self, node, output_grad):
        return [flatten_gradient_op(node.inputs[0], output_grad)]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        s = input_shapes[0]
        return (s[0], gpu_op.get_shape_size(s[1:]))


class SqueezeOp(_CopyReshapeOp):
    name = "Squeeze"

    def gradient(self, node, output_grad):
        return [squeeze_gradient_op(node.inputs[0], output_grad)]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return (input_shapes[0][0], input_shapes[0][1])


class _CopyBackOp(Op):
    def __call__(self, node_A, node_B):
        return self._node([node_A, node_B])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        input_vals[1].copyto(output_val, cudaStream)
        return 0

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


class FlattenGradientOp(_CopyBackOp):
    name = "FlattenGradient"


class SqueezeGradientOp(_CopyBackOp):
    name = "SqueezeGradient"


# ---- activation (ActivationForwardOp .. FullyActivationBackwardOp: autodiff.py:1124-1169, 1448-1501)
class ActivationForwardOp(Op):
    name = "ActivationForward"
    _backward = "activation_backward_op"

    def __call__(self, node_A, dataformat, activationMode):
        return self._node([node_A], dataformat=dataformat, activationMode=activationMode, cudnnlist=[0])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.activation_forward(input_vals[0], output_val, node.activationMode, node.cudnnlist[0], cudnnHandle, cudaStream)
        return 0

    def gradient(self, node, output_grad):
        return [globals()[self._backward](node.inputs[0], output_grad, node, node.activationMode, node.cudnnlist)]

    def _descriptor_shape(self, shape):
        return shape

    def infer_shape(self, node, input_shapes, cudnnHandle):
        node.cudnnlist[0] = gpu_op.activation_get_cudnnlist(self._descriptor_shape(input_shapes[0]), node.dataformat, node.activationMode)
        return input_shapes[0]


class FullyActivationForwardOp(ActivationForwardOp):
    """Activation on a 2-D (batch, features) tensor, described to the library as (batch, 1, features)."""
    name = "FullyActivationForward"
    _backward = "fullyactivation_backward_op"

    def _descriptor_shape(self, shape):
        return (shape[0], 1, shape[1])


class ActivationBackwardOp(Op):
    name = "ActivationBackward"

    def __call__(self, node_A, node_B, node_C, activationMode, cudnnlist):
        # inputs: x, dy, y
        return self._node([node_A, node_B, node_C], activationMode=activationMode, cudnnlist=cudnnlist)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.activation_backward(input_vals[0], output_val, input_vals[2], input_vals[1], node.activationMode,
                                   node.cudnnlist[0], cudnnHandle, cudaStream)
        return 0

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


class FullyActivationBackwardOp(ActivationBackwardOp):
    name = "FullyActivationBackward"


# ---- pooling (Pooling2DForwardOp / Pooling2DBackwardOp: autodiff.py:1223-1276) -----------------
class Pooling2DForwardOp(Op):
    name = "Pooling2DForward"

    def __call__(self, node_A, dataformat, poolingMode, pad_h, pad_w, u, v, filter_h, filter_w):
        return self._node([node_A], dataformat=dataformat, poolingMode=poolingMode, pad_h=pad_h, pad_w=pad_w, u=u, v=v,
                          filter_h=filter_h, filter_w=filter_w, cudnnlist=[0])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.pooling_2d_forward(input_vals[0], output_val, node.cudnnlist[0], cudnnHandle, cudaStream)
        return 0

    def gradient(self, node, output_grad):
        return [pooling_2d_backward_op(node.inputs[0], output_grad, node, node.cudnnlist)]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        out, node.cudnnlist[0] = gpu_op.pooling_2d_forward_get_out_shape(input_shapes[0], node.dataformat, node.poolingMode, node.pad_h,
                                                                         node.pad_w, node.u, node.v, node.filter_h, node.filter_w)
        return out


class Pooling2DBackwardOp(Op):
    name = "Pooling2DBackward"

    def __call__(self, node_A, node_B, node_C, cudnnlist):
        # inputs: x, dy, y
        return self._node([node_A, node_B, node_C], cudnnlist=cudnnlist)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.pooling_2d_backward(input_vals[0], input_vals[2], input_vals[1], output_val, node.cudnnlist[0], cudnnHandle, cudaStream)
        return 0

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


# ---- dropout (DropoutForwardOp .. FullyDropoutBackwardOp: autodiff.py:1337-1446) ----------------
class DropoutForwardOp(Op):
    name = "DropoutForward"
    _backward = "dropout_backward_op"

    def __call__(self, node_A, dataformat, dropout):
        return self._node([node_A], dataformat=dataformat, dropout=dropout, seed=[0], reserveSpace_p=[0], cudnnlist=[0], inputd=[0])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        node.seed[0] = random.randint(0, 100)     # a fresh mask every step, as the reference draws it
        node.reserveSpace_p[0], node.cudnnlist[0], short = gpu_op.dropout_forward(
            input_vals[0], output_val, node.dataformat, node.dropout, node.seed[0], node.inputd[0], cudnnHandle, cudaStream)
        return short

    def gradient(self, node, output_grad):
        return [globals()[self._backward](output_grad, node.dropout, node.reserveSpace_p, node.cudnnlist)]

    def _descriptor_shape(self, shape):
        return shape

    def infer_shape(self, node, input_shapes, cudnnHandle):
        node.inputd[0] = gpu_op.get_input_descriptor(self._descriptor_shape(input_shapes[0]), node.dataformat)
        return input_shapes[0]


class FullyDropoutForwardOp(DropoutForwardOp):
    name = "FullyDropoutForward"
    _backward = "fullydropout_backward_op"

    def _descriptor_shape(self, shape):
        return (shape[0], 1, shape[1])


class DropoutBackwardOp(Op):
    name = "DropoutBackward"

    def __call__(self, node_A, dropout, reserveSpace_p, cudnnlist):
        return self._node([node_A], dropout=dropout, reserveSpace_p=reserveSpace_p, cudnnlist=cudnnlist)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.dropout_backward(input_vals[0], output_val, node.reserveSpace_p[0], node.cudnnlist[0], cudnnHandle, cudaStream)
        return 0

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


class FullyDropoutBackwardOp(DropoutBackwardOp):
    name = "FullyDropoutBackward"


# ---- reductions (ReduceSumOp, ReduceMeanOp, *BackwardOp: autodiff.py:1503-1616) -----------------
class ReduceSumOp(Op):
    name = "ReduceSumOp"
    scale_by_mean = False

    def __call__(self, node_A):
        return self._node([node_A], type="NHWC", cudnnlist=[0], meanfloat=[1.])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        short = gpu_op.reduce_sum_new(input_vals[0], output_val, node.cudnnlist[0], cudnnHandle, cudaStream)
        if self.scale_by_mean:
            gpu_op.matrix_elementwise_multiply_by_const(output_val, node.meanfloat[0], output_val, cudaStream)
        return short

    def gradient(self, node, output_grad):
        g = broadcastto_op(output_grad, node.inputs[0])
        return [g * node.meanfloat[0]] if self.scale_by_mean else [g]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        if self.scale_by_mean:
            node.meanfloat[0] = 1. / gpu_op.get_shape_size(input_shapes[0])
        ins, outs = gpu_op.reduce_sum_get_real_shape(input_shapes[0], (1,), node.type)
        node.cudnnlist[0] = gpu_op.reduce_sum_get_cudnnlist(ins, outs, node.type, cudnnHandle)
        return (1,)


class ReduceMeanOp(ReduceSumOp):
    scale_by_mean = True


class ReduceSumBackwardOp(Op):
    name = "ReduceSumBackward"

    def __call__(self, node_A, inputshape, axis):
        return self._node([node_A], axis=axis, inputshape=inputshape)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.reduce_sum_backward(input_vals[0], output_val, node.axis)
        return 0

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return node.inputshape[0]


class ReduceMeanBackwardOp(ReduceSumBackwardOp):
    name = "ReduceMeanBackward"

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.reduce_sum_backward(input_vals[0], output_val, node.axis)
        gpu_op.matrix_elementwise_multiply_by_const(output_val, 1. / node.inputshape[1], output_val, cudaStream)
        return 0


# ---- losses (CrossEntropyOp, L1/L2 loss and regularisers: autodiff.py:1618-1819) -----------------
class CrossEntropyOp(Op):
    """Element-wise binary cross-entropy terms  y*log(p) + (1-y)*log(1-p)  (no reduction)."""
    name = "CrossEntropy"

    def __call__(self, node_A, node_B):
        return self._node([node_A, node_B])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream=None, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.cross_entropy(input_vals[0], input_vals[1], output_val)
        return 0

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


def _loss_op(op_name, fwd, grad_op_name, binary):
    class _Loss(Op):
        name = op_name

        def __call__(self, *nodes):
            return self._node(list(nodes))

        def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
            _no_numpy(use_numpy)
            fwd(*input_vals, output_val)
            return 0

        def gradient(self, node, output_grad):
            g = globals()[grad_op_name](*node.inputs, output_grad)
            return [g, zeroslike_op(node.inputs[1])] if binary else [g]

        def infer_shape(self, node, input_shapes, cudnnHandle):
            return (1,)
    _Loss.__name__ = op_name + "Op"
    return _Loss


def _loss_grad_op(op_name, bwd):
    class _LossGrad(Op):
        name = op_name

        def __call__(self, *nodes):
            return self._node(list(nodes))

        def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
            _no_numpy(use_numpy)
            bwd(*input_vals, output_val)
            return 0

        def infer_shape(self, node, input_shapes, cudnnHandle):
            return input_shapes[0]
    _LossGrad.__name__ = op_name + "Op"
    return _LossGrad


L1lossOp = _loss_op("L1loss", gpu_op.L1loss, "l1loss_gradient_op", True)
L2lossOp = _loss_op("L2loss", gpu_op.L2loss, "l2loss_gradient_op", True)
L1regularOp = _loss_op("L1regular", gpu_op.L1regular, "l1regular_gradient_op", False)
L2regularOp = _loss_op("L2regular", gpu_op.L2regular, "l2regular_gradient_op", False)
L1lossgradientOp = _loss_grad_op("L1lossgradient", gpu_op.l1loss_gradient)
L2lossgradientOp = _loss_grad_op("L2lossgradient", gpu_op.l2loss_gradient)
L1regulargradientOp = _loss_grad_op("L1regulargradient", gpu_op.l1regular_gradient)
L2regulargradientOp = _loss_grad_op("L2regulargradient", gpu_op.l2regular_gradient)


# ---- batch normalisation (BNForwardOp .. FullyBNBackwardOp: autodiff.py:1821-1932) ---------------
class BNForwardOp(Op):
    name = "BNForward"
    _backward = "bn_backward_op"

    def __call__(self, node_A, dataformat, batchNormMode):
        return self._node([node_A], dataformat=dataformat, batchNormMode=batchNormMode, Save_p=[0, 0], n=0, cudnnlist=[0])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        short = gpu_op.bn_forward(input_vals[0], output_val, node.batchNormMode, node.n, node.Save_p[0], node.Save_p[1],
                                  node.cudnnlist[0], cudnnHandle, cudaStream)
        node.n += 1
        return short

    def gradient(self, node, output_grad):
        return [globals()[self._backward](node.inputs[0], output_grad, node.batchNormMode, node.Save_p, node.cudnnlist)]

    def _descriptor_shape(self, shape):
        return shape

    def infer_shape(self, node, input_shapes, cudnnHandle):
        node.Save_p[0], node.Save_p[1], node.cudnnlist[0] = gpu_op.bn_get_cudnnlist(self._descriptor_shape(input_shapes[0]),
                                                                                     node.dataformat, node.batchNormMode)
        return input_shapes[0]


class FullyBNForwardOp(BNForwardOp):
    name = "FullyBNForward"
    _backward = "fullybn_backward_op"

    def __call__(self, node_A, dataformat):
        return BNForwardOp.__call__(self, node_A, dataformat, "pre_activation")

    def _descriptor_shape(self, shape):
        return (shape[0], 1, shape[1])


class BNBackwardOp(Op):
    name = "BNBackward"

    def __call__(self, node_A, node_B, batchNormMode, Save_p, cudnnlist):
        return self._node([node_A, node_B], batchNormMode=batchNormMode, Save_p=Save_p, cudnnlist=cudnnlist)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        return gpu_op.bn_backward(input_vals[0], input_vals[1], output_val, node.batchNormMode, node.Save_p[0], node.Save_p[1],
                                  node.cudnnlist[0], cudnnHandle, cudaStream)

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


class FullyBNBackwardOp(BNBackwardOp):
    name = "FullyBNBackward"


# ---- concat (ConcatForwardOp / ConcatBackwardOp: autodiff.py:1935-1984) ---------------------------
class ConcatForwardOp(Op):
    name = "ConcatForward"

    def __call__(self, node_A, node_B):
        return self._node([node_A, node_B])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.concat_forward(input_vals[0], input_vals[1], output_val, cudaStream)
        return 0

    def gradient(self, node, output_grad):
        a, b = node.inputs
        return [concat_backward_op(a, b, output_grad, 0), concat_backward_op(a, b, output_grad, 1)]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        out = list(input_shapes[0])
        out[1] = input_shapes[0][1] + input_shapes[1][1]
        return tuple(out)


class ConcatBackwardOp(Op):
    name = "Concatbackward"

    def __call__(self, node_A, node_B, node_C, type):
        return self._node([node_A, node_B, node_C], type=type)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        fn = gpu_op.concat_a_backward if node.type == 0 else gpu_op.concat_b_backward
        fn(input_vals[0], input_vals[1], input_vals[2], output_val, cudaStream)
        return 0

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[node.type]


# ---- optimisers (SgdOp, AdamOp: autodiff.py:2028-2076) -----------------------------------------------
class SgdOp(Op):
    name = "SgdOp"

    def __call__(self, node_A, node_B, learning_rate):
        return self._node([node_A, node_B], learning_rate=learning_rate)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.sgd_update(input_vals[0], input_vals[1], node.learning_rate, cudaStream)
        return 0

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


class AdamOp(Op):
    name = "AdamOp"

    def __call__(self, node_A, node_B, node_C, node_D, b1, b2, b1t, b2t, e, learning_rate):
        # inputs: parameter, first moment, second moment, gradient; b1t / b2t are one-element lists
        return self._node([node_A, node_B, node_C, node_D], b1=b1, b2=b2, b1t=b1t, b2t=b2t, e=e, learning_rate=learning_rate)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        w, m, v, g = input_vals
        gpu_op.adam_mv(m, v, g, node.b1, node.b2, cudaStream)
        gpu_op.adam_compute(w, m, v, node.b1t[0], node.b2t[0], node.e, node.learning_rate, cudaStream)
        return 0

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


# ---- cross-entropy pieces of the CNN graphs (CrossOp / CrossBackwardOp: autodiff.py:2079-2123) --------
class CrossOp(Op):
    name = "CrossOp"

    def __call__(self, node_A, node_B, ismean):
        return self._node([node_A, node_B], ismean=ismean, meanfloat=[1.])

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.cross(input_vals[0], input_vals[1], output_val, node.meanfloat[0], cudaStream)
        return 0

    def gradient(self, node, output_grad):
        return [cross_backward_op(node.inputs[0], node.inputs[1], output_grad, node.meanfloat), zeroslike_op(node.inputs[1])]

    def infer_shape(self, node, input_shapes, cudnnHandle):
        if node.ismean:
            node.meanfloat[0] = 1. / gpu_op.get_shape_size(input_shapes[0])   # batch * classes, as the reference
        return input_shapes[0]


class CrossBackwardOp(Op):
    name = "CrossBackwardOp"

    def __call__(self, node_A, node_B, node_C, meanfloat):
        return self._node([node_A, node_B, node_C], meanfloat=meanfloat)

    def compute(self, node, input_vals, output_val, cudnnHandle, cublasHandle, cudaStream, use_numpy=False):
        _no_numpy(use_numpy)
        gpu_op.cross_backward(input_vals[0], input_vals[1], input_vals[2], output_val, node.meanfloat[0], cudaStream)
        return 0

    def infer_shape(self, node, input_shapes, cudnnHandle):
        return input_shapes[0]


# ---- composite builders (autodiff.py:2126-2157) ---------------------------------------------------------
def dense(X, W, b):
    xw = matmul_op(X, W)
    return xw + broadcastto_op(b, xw)


def conv2withbias(input, filter, bias, dataformat, padding, strideh, stridew):
    c = convolution_2d_forward_op(input, filter, dataformat, padding, strideh, stridew)
    return c + broadcastto_op(bias, c, dataformat)


def crossEntropy_loss(input, y_, ismean=True):
    return reduce_sum_op(cross_op(input, y_, ismean))


# ---- operator singletons (autodiff.py:2161-2226) ----------------------------------------------------------
adam_op = AdamOp()
sgd_op = SgdOp()
cross_op = CrossOp()
cross_backward_op = CrossBackwardOp()
add_op = AddOp()
mul_op = MulOp()
add_byconst_op = AddByConstOp()
mul_byconst_op = MulByConstOp()
matmul_op = MatMulOp()
placeholder_op = PlaceholderOp()
oneslike_op = OnesLikeOp()
zeroslike_op = ZerosLikeOp()
reducesumaxiszero_op = ReduceSumAxisZeroOp()
broadcastto_op = BroadcastToOp()
broadcastto_gradient_op = BroadcastToGradientOp()
softmaxcrossentropy_op = SoftmaxCrossEntropyOp()
softmax_op = SoftmaxOp()
relu_op = ReluOp()
relu_gradient_op = ReluGradientOp()
convolution_2d_forward_op = Convolution2DForwardOp()
convolution_2d_backward_op = Convolution2DBackwardOp()
flatten_op = FlattenOp()
flatten_gradient_op = FlattenGradientOp()
activation_forward_op = ActivationForwardOp()
activation_backward_op = ActivationBackwardOp()
pooling_2d_forward_op = Pooling2DForwardOp()
pooling_2d_backward_op = Pooling2DBackwardOp()
dropout_forward_op = DropoutForwardOp()
dropout_backward_op = DropoutBackwardOp()
fullydropout_forward_op = FullyDropoutForwardOp()
fullydropout_backward_op = FullyDropoutBackwardOp()
fullyactivation_forward_op = FullyActivationForwardOp()
fullyactivation_backward_op = FullyActivationBackwardOp()
exp_op = ExpOp()
log_op = LogOp()
reverse_op = ReverseOp()
pow_op = PowOp()
reduce_sum_op = ReduceSumOp()
reduce_sum_backward_op = ReduceSumBackwardOp()
reduce_mean_op = ReduceMeanOp()
reduce_mean_backward_op = ReduceMeanBackwardOp()
crossEntropy_op = CrossEntropyOp()
l1loss_op = L1lossOp()
l1loss_gradient_op = L1lossgradientOp()
l2loss_op = L2lossOp()
l2loss_gradient_op = L2lossgradientOp()
l1regular_op = L1regularOp()
l1regular_gradient_op = L1regulargradientOp()
l2regular_op = L2regularOp()
l2regular_gradient_op = L2regulargradientOp()
bn_forward_op = BNForwardOp()
bn_backward_op = BNBackwardOp()
fullybn_forward_op = FullyBNForwardOp()
fullybn_backward_op = FullyBNBackwardOp()
concat_forward_op = ConcatForwardOp()
concat_backward_op = ConcatBackwardOp()
squeeze_op = SqueezeOp()
squeeze_gradient_op = SqueezeGradientOp()


# ---- autodiff and graph utilities (autodiff.py:2894-3027) ------------------------------------------------
def find_topo_sort(node_list):
    """Post-order DFS over input edges; iterative so deep graphs do not hit the recursion limit."""
    visited, order = set(), []
    for root in node_list:
        if root in visited:
            continue
        visited.add(root)
        stack = [(root, iter(root.inputs))]
        while stack:
            node, it = stack[-1]
            advanced = False
            for child in it:
                if child not in visited:
                    visited.add(child)
                    stack.append((child, iter(child.inputs)))
                    advanced = True
                    break
            if not advanced:
                order.append(node)
                stack.pop()
    return order


def sum_node_list(node_list):
    return _reduce(lambda a, b: a + b, node_list)


def gradients(output_node, node_list):
    """Reverse-mode autodiff: gradient nodes of ``output_node`` w.r.t. each node in ``node_list``."""
    pending = {output_node: [oneslike_op(output_node)]}
    grad_of = {}
    for node in reversed(find_topo_sort([output_node])):
        grad = sum_node_list(pending[node])
        grad_of[node] = grad
        contributions = node.op.gradient(node, grad)
        for inp, g in zip(node.inputs, contributions or []):
            pending.setdefault(inp, []).append(g)
    return [grad_of[n] for n in node_list]


def get_Variable_node_list(node):
    """Parameters reachable from ``node`` in post-order (first use first)."""
    return [n for n in find_topo_sort([node]) if n.isw == 1]


def nodelist_to_name(nodelist):
    return [n.name for n in nodelist]

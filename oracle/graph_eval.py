"""Numpy evaluation of a tinyflow graph: the "numpy executor" the GPU path is checked against.

TEST INFRASTRUCTURE ONLY (see oracle/ops.py).  Walks a topological order of graph nodes (built
with ``tinyflow_b200.autodiff`` or, in the golden-vector generator, with the reference's own
``autodiff``) and evaluates each node with the restated operators of :mod:`oracle.ops`.  Dispatch
is by the operator's class name, which is the same in both graph libraries, so one evaluator
serves both.  The gradient formulas are NOT restated here: they come from the graph library's
``gradients()``, so the reference's quirks are reproduced automatically.
"""
from __future__ import annotations

import numpy as np

from . import ops


class OracleExecutor:
    def __init__(self, topo_order, dtype=np.float64, dropout_seeds=None):
        self.topo = list(topo_order)
        self.dtype = dtype
        self.values = {}
        self.dropout_seeds = dropout_seeds or {}    # DropoutForward node -> seed used by the GPU run
        self.adam_powers = None     # (b1^t, b2^t) of the step being checked; default: the node's current values

    def _conv_geom(self, node, x, w):
        return ops.conv_geometry(x.shape, w.shape, node.padding, node.u, node.v)

    def run(self, feed):
        v = self.values = {n: np.asarray(a, dtype=self.dtype) for n, a in feed.items()}
        for node in self.topo:
            if node in v:
                continue
            ins = [v[i] for i in node.inputs]
            out = self._eval(node, ins)
            if out is not None:
                v[node] = out
        return v

    # One branch per operator class (name shared by the reference and the mirror).
    def _eval(self, node, ins):
        kind = type(node.op).__name__
        dt = self.dtype
        if kind == "AddOp":
            return ins[0] + ins[1]
        if kind == "AddByConstOp":
            return ins[0] + dt(node.const_attr)
        if kind == "MulOp":
            return ins[0] * ins[1]
        if kind == "MulByConstOp":
            return ins[0] * dt(node.const_attr)
        if kind == "MatMulOp":
            a = ins[0].T if node.matmul_attr_trans_A else ins[0]
            b = ins[1].T if node.matmul_attr_trans_B else ins[1]
            return np.matmul(a, b)
        if kind == "ZerosLikeOp":
            return np.zeros_like(ins[0])
        if kind == "OnesLikeOp":
            return np.ones_like(ins[0])
        if kind == "ReduceSumAxisZeroOp":
            return ins[0].sum(axis=0) if ins[0].ndim > 1 else ins[0].sum(keepdims=True)
        if kind == "BroadcastToOp":
            if node.type == "NCHW":
                return ops.broadcast_channel(ins[0], ins[1].shape)
            return ops.broadcast_tail(ins[0], ins[1].shape)
        if kind == "BroadcastToGradientOp":
            target = ins[1].shape
            x = ins[0]
            if node.type == "NCHW":
                axes = (0,) + tuple(range(2, x.ndim))
                return x.sum(axis=axes).reshape(target)
            if int(np.prod(target)) == 1:
                return x.sum().reshape(target)
            return x.reshape(-1, int(np.prod(target))).sum(axis=0).reshape(target)
        if kind == "SoftmaxCrossEntropyOp":
            return ops.softmax_cross_entropy(ins[0], ins[1])
        if kind == "SoftmaxOp":
            return ops.softmax_rows(ins[0])
        if kind == "ReluOp":
            return ops.relu(ins[0])
        if kind == "ReluGradientOp":
            return ops.relu_grad(ins[0], ins[1])
        if kind == "Convolution2DForwardOp":
            return ops.conv2d_fwd(ins[0], ins[1], self._conv_geom(node, ins[0], ins[1]))
        if kind == "Convolution2DBackwardOp":
            g = self._conv_geom(node, ins[0], ins[1])
            return ops.conv2d_dgrad(ins[2], ins[1], g) if node.type == 0 else ops.conv2d_wgrad(ins[0], ins[2], g)
        if kind in ("FlattenOp", "SqueezeOp"):
            return ins[0].reshape(ins[0].shape[0], -1)
        if kind in ("FlattenGradientOp", "SqueezeGradientOp"):
            return ins[1].reshape(ins[0].shape)
        if kind in ("ActivationForwardOp", "FullyActivationForwardOp"):
            mode = node.activationMode
            if mode == "relu":
                return ops.relu(ins[0])
            if mode == "softmax":
                return ops.softmax_instance(ins[0])
            if mode == "sigmoid":
                return ops.sigmoid(ins[0])
            return np.tanh(ins[0])
        if kind in ("ActivationBackwardOp", "FullyActivationBackwardOp"):
            x, dy, y = ins
            mode = node.activationMode
            if mode == "relu":
                return ops.relu_grad(x, dy)
            if mode == "softmax":
                return ops.softmax_instance_bwd(y, dy)
            if mode == "sigmoid":
                return dy * y * (1 - y)
            return dy * (1 - y * y)
        if kind == "Pooling2DForwardOp":
            g = ops.pool_geometry(ins[0].shape, node.pad_h, node.pad_w, node.u, node.v, node.filter_h, node.filter_w)
            return ops.maxpool_fwd(ins[0], g)[0] if node.poolingMode == "max" else ops.avgpool_fwd(ins[0], g)
        if kind == "Pooling2DBackwardOp":
            fwd = node.inputs[2]
            g = ops.pool_geometry(ins[0].shape, fwd.pad_h, fwd.pad_w, fwd.u, fwd.v, fwd.filter_h, fwd.filter_w)
            return ops.maxpool_bwd(ins[0], ins[1], g) if fwd.poolingMode == "max" else ops.avgpool_bwd(ins[1], g)
        if kind in ("DropoutForwardOp", "FullyDropoutForwardOp"):
            if node.dropout == 0:
                return ins[0].copy()
            return ops.dropout(ins[0], node.dropout, self.dropout_seeds.get(node, node.seed[0]))
        if kind in ("DropoutBackwardOp", "FullyDropoutBackwardOp"):
            if node.dropout == 0:
                return ins[0].copy()
            fwd = next(n for n in self.topo if getattr(n, "reserveSpace_p", None) is node.reserveSpace_p
                       and type(n.op).__name__.endswith("DropoutForwardOp"))
            return ops.dropout(ins[0], node.dropout, self.dropout_seeds.get(fwd, fwd.seed[0]))
        if kind in ("ReduceSumOp", "ReduceMeanOp"):
            s = ins[0].sum().reshape(1)
            if kind == "ReduceMeanOp":
                node.meanfloat[0] = 1.0 / ins[0].size
                return s * dt(node.meanfloat[0])
            return s
        if kind in ("BNForwardOp", "FullyBNForwardOp"):
            return ops.bn_fwd(ins[0], node.batchNormMode)[0]
        if kind in ("BNBackwardOp", "FullyBNBackwardOp"):
            return ops.bn_bwd(ins[0], ins[1], node.batchNormMode)
        if kind == "ConcatForwardOp":
            return ops.concat(ins[0], ins[1])
        if kind == "ConcatBackwardOp":
            return ops.concat_split(ins[0].shape, ins[2], node.type)
        if kind == "CrossOp":
            if node.ismean:
                node.meanfloat[0] = 1.0 / ins[0].size      # what infer_shape stores (autodiff.py:2099-2102)
            return ops.cross(ins[0], ins[1], dt(node.meanfloat[0]))
        if kind == "CrossBackwardOp":
            return ops.cross_backward(ins[0], ins[1], ins[2], dt(node.meanfloat[0]))
        if kind == "SgdOp":
            self.values[node.inputs[0]] = ops.sgd(ins[0], ins[1], node.learning_rate)
            return None
        if kind == "AdamOp":
            b1t, b2t = self.adam_powers if self.adam_powers else (node.b1t[0], node.b2t[0])
            w, m, vv = ops.adam(ins[0], ins[1], ins[2], ins[3], dt(node.b1), dt(node.b2), dt(b1t), dt(b2t), dt(node.e), dt(node.learning_rate))
            self.values[node.inputs[0]], self.values[node.inputs[1]], self.values[node.inputs[2]] = w, m, vv
            return None
        if kind == "ExpOp":
            return np.exp(ins[0])
        if kind == "LogOp":
            return np.log(ins[0])
        if kind == "ReverseOp":
            return 1.0 / ins[0]
        if kind == "PowOp":
            return ins[0] ** dt(node.const_attr)
        raise NotImplementedError("oracle has no restatement for operator %s" % kind)

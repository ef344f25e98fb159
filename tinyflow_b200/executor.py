"""Training-step executor; host-side mirror of ``autodiff.Executor`` (autodiff.py:2237-2890).

The executor builds the gradient graph of ``targetloss`` w.r.t. every ``Variable`` it reaches,
appends one optimiser node per parameter, moves each optimiser node to just after the last
reader of its parameter (so updates interleave with the backward pass, autodiff.py:3002-3021)
and then runs the nodes in that order, one C-ABI call per node, allocating each node's output
through ``DLArrayAlloc`` every step exactly as the reference does.

``run(feed_dict)`` takes ``{node: NDArray}`` for the data placeholders, every parameter and (for
Adam) its two moment tensors, and returns ``[loss NDArray, {node: NDArray}]`` where the dict is
the feed dict for the next step (parameters and moments, updated in place).

Memory-plan messages from a scheduler keep the reference's layout
(autodiff.py:2561-2590): ``top_control_queue.put((swap_list, release_list, recompute_list))`` with
``swap_list`` entries ``(tensor_index, start_time_ms, start_node_index, move_to_gpu)`` and release /
recompute entries ``(start_node_index, tensor_index)``.  Swaps run on a worker thread over a side
stream through ``DLArrayCopyFromTo`` into pinned host arrays.
"""
from __future__ import annotations

import queue
import threading
import time

from . import gpu_op, ndarray
from .graph import (Variable, adam_op, find_topo_sort, get_Variable_node_list, gradients, sgd_op)


def getcomputelist(Variable_node_list, Variable_node_grad_list, b1, b2, b1t, b2t, e, learning_rate):
    """One Adam node per parameter plus its moment Variables (autodiff.py:2985-2999)."""
    computelist, mv, var_to_mv = [], [], {}
    for var, grad in zip(Variable_node_list, Variable_node_grad_list):
        m, v = Variable(var.name + "m"), Variable(var.name + "v")
        mv += [m, v]
        var_to_mv[var] = (m, v)
        node = adam_op(var, m, v, grad, b1, b2, b1t, b2t, e, learning_rate)
        node.issgd = 1
        computelist.append(node)
    return computelist, mv, var_to_mv


def getsgdcomputelist(Variable_node_list, Variable_node_grad_list, learning_rate):
    """One SGD node per parameter (the wiring of TrainExecute.py:315-324)."""
    computelist = []
    for var, grad in zip(Variable_node_list, Variable_node_grad_list):
        node = sgd_op(var, grad, learning_rate)
        node.issgd = 1
        computelist.append(node)
    return computelist


def swapadam(topoorder):
    """Move each optimiser node to just after the last non-optimiser reader of its parameter."""
    order = list(topoorder)
    i = 0
    n = len(order)
    for i in range(n):
        node = order[i]
        if node.issgd == 1 and node.isw == 0:
            node.isw = 3
            param = node.inputs[0]
            j = n - 1
            while j > i:
                if order[j].issgd != 1 and param in order[j].inputs:
                    break
                j -= 1
            order.pop(i)
            order.insert(j, node)
    return order


class _SwapWorker(threading.Thread):
    """Executes the swap requests of ONE direction for the executor on its own side stream, in the order they were
    submitted.  Two workers (device -> host and host -> device) let the two copy engines run at the same time; a
    swap-in first waits for the queued swap-out of the same tensor.  A reader of a tensor that still has requests
    queued waits for them (``wait_for``): it must not pick up the device array of a tensor whose swap-out is about to
    free it."""

    def __init__(self, executor, to_gpu, other=None):
        super().__init__(daemon=True)
        self.ex = executor
        self.to_gpu = to_gpu
        self.other = other             # the swap-out worker, for the swap-in worker
        self.q = queue.Queue()
        self.stream = None
        self.cond = threading.Condition()
        self.pending = 0
        self.pending_for = {}          # tensor index -> queued or running requests

    def submit(self, wait_ms, index):
        with self.cond:
            self.pending += 1
            self.pending_for[index] = self.pending_for.get(index, 0) + 1
        self.q.put((wait_ms, index))

    def run(self):
        self.stream = gpu_op.create_cudaStream()
        while True:
            item = self.q.get()
            if item is None:
                return
            wait_ms, index = item
            try:
                if wait_ms > 0:
                    time.sleep(wait_ms / 1000.0)
                if self.other is not None:
                    self.other.wait_for(index)        # the tensor's way out has to be complete before its way back
                self.ex._do_swap(index, self.to_gpu, self.stream)
            finally:
                with self.cond:
                    self.pending -= 1
                    self.pending_for[index] -= 1
                    self.cond.notify_all()

    def wait_for(self, index):
        with self.cond:
            while self.pending_for.get(index, 0) > 0:
                self.cond.wait()

    def drain(self):
        with self.cond:
            while self.pending > 0:
                self.cond.wait()


class _SwapWorkers(object):
    """The pair of workers behind the executor's swap requests."""

    def __init__(self, executor):
        self.out = _SwapWorker(executor, False)
        self.back = _SwapWorker(executor, True, other=self.out)
        self.out.start()
        self.back.start()

    def submit(self, wait_ms, index, to_gpu):
        (self.back if to_gpu else self.out).submit(wait_ms, index)

    def wait_for(self, index):
        self.out.wait_for(index)
        self.back.wait_for(index)

    def drain(self):
        self.out.drain()
        self.back.drain()


class Executor(object):
    def __init__(self, targetloss, y, learning_rate, top_control_queue=None, top_message_queue=None, log_path=None,
                 optimizer="adam"):
        self.b1, self.b2, self.e = 0.9, 0.999, 0.00000001
        self.b1t, self.b2t = [0.9], [0.999]
        self.targetloss, self.y, self.learning_rate = targetloss, y, learning_rate
        self.log_path = log_path
        self.optimizer = optimizer

        variables = get_Variable_node_list(targetloss)
        variables.reverse()                      # last layer first: its gradient is ready first
        self.Variable_node_grad_list = gradients(targetloss, variables)
        self.Variable_node_to_grad = dict(zip(variables, self.Variable_node_grad_list))
        if optimizer == "adam":
            compute, self.mv, self.Variable_node_to_mv = getcomputelist(
                variables, self.Variable_node_grad_list, self.b1, self.b2, self.b1t, self.b2t, self.e, learning_rate)
        elif optimizer == "sgd":
            compute, self.mv, self.Variable_node_to_mv = getsgdcomputelist(variables, self.Variable_node_grad_list, learning_rate), [], {}
        else:
            raise ValueError("optimizer must be 'adam' or 'sgd'")
        self.optimizer_nodes = compute
        self.topo_order = swapadam(find_topo_sort(compute))
        variables.reverse()                      # back to network order
        self.Variable_node_list = variables
        self.eval_node_list = [targetloss] + variables + [self.Variable_node_to_mv[v][0] for v in variables if v in self.Variable_node_to_mv] \
            + [self.Variable_node_to_mv[v][1] for v in variables if v in self.Variable_node_to_mv] + [y]
        for i, node in enumerate(self.topo_order):
            node.index = i
        self.total_node = len(self.topo_order)

        self.top_control_queue, self.top_message_queue = top_control_queue, top_message_queue
        # stream and handles are created on first use, so graph analysis works without a device
        self.cudaStream = self.cudnnHandle = self.cublasHandle = None
        self.ctx_cpu, self.ctx_gpu = ndarray.cpu(0), ndarray.gpu(0)
        self.node_to_shape_map = None
        self.feed_shapes = None
        self.values = {}           # node index -> NDArray on the GPU (None while swapped out)
        self.host_values = {}      # node index -> pinned host NDArray holding a swapped-out tensor
        self.have_plan = False
        self._swap_worker = None
        self._values_lock = threading.Lock()
        self.passive_swap_in = 0

    def _ensure_handles(self):
        if self.cudaStream is None:
            self.cudaStream = gpu_op.create_cudaStream()
            self.cudnnHandle = gpu_op.create_cudnnHandle(self.cudaStream)
            self.cublasHandle = gpu_op.create_cublasHandle(self.cudaStream)

    # ---- shape inference (autodiff.py:2318-2336): builds every descriptor exactly once ----------
    def infer_shape(self, feed_shapes):
        self.node_to_shape_map = dict(feed_shapes)
        for node in self.topo_order:
            if node in self.node_to_shape_map:
                continue
            input_shapes = [self.node_to_shape_map[i] for i in node.inputs]
            self.node_to_shape_map[node] = tuple(node.op.infer_shape(node, input_shapes, self.cudnnHandle))

    # ---- memory-plan messages ---------------------------------------------------------------------
    def _apply_plan(self, swap_list, release_list, recompute_list):
        for node in self.topo_order:
            node.control_message_out, node.control_message_out_time = [], 0
            node.release_list, node.recompute_list = [], []
        for tensor_index, start_time, start_node_index, move_to_gpu in swap_list:
            start = self.topo_order[start_node_index]
            wait = start_time if start.control_message_out_time == 0 else start_time - start.control_message_out_time
            start.control_message_out_time = start_time
            start.control_message_out.append((wait, tensor_index, move_to_gpu))
        for start_node_index, tensor_index in release_list:
            self.topo_order[start_node_index].release_list.append(tensor_index)
        for start_node_index, tensor_index in recompute_list:
            self.topo_order[start_node_index].recompute_list.append(tensor_index)
        self.have_plan = bool(swap_list or release_list or recompute_list)
        if swap_list and self._swap_worker is None:
            self._swap_worker = _SwapWorkers(self)

    def _do_swap(self, index, to_gpu, stream):
        shape = self.node_to_shape_map[self.topo_order[index]]
        if to_gpu:
            with self._values_lock:
                if self.values.get(index) is not None or index not in self.host_values:
                    return
            dev = ndarray.empty(shape, self.ctx_gpu)
            self.host_values[index].copyto(dev, stream)
            with self._values_lock:
                if self.values.get(index) is None:
                    self.values[index] = dev
        else:
            with self._values_lock:
                dev = self.values.get(index)
            if dev is None:
                return
            host = self.host_values.get(index)
            if host is None:
                host = ndarray.empty(shape, self.ctx_cpu)
            dev.copyto(host, stream)             # returns once the copy has completed
            with self._values_lock:
                self.host_values[index] = host
                self.values[index] = None
            dev.free_gpu()

    def _after_node(self, node):
        for wait, tensor_index, to_gpu in node.control_message_out:
            self._swap_worker.submit(wait, tensor_index, to_gpu)
        for tensor_index in node.release_list:
            with self._values_lock:
                arr = self.values.get(tensor_index)
                self.values[tensor_index] = None
            if arr is not None and self.topo_order[tensor_index].isw == 0:
                arr.free_gpu()

    def _resident(self, n):
        """The GPU array of node ``n``, swapping it in on demand (the reference's passive swap-in)."""
        if self._swap_worker is not None:
            self._swap_worker.wait_for(n.index)      # a queued swap-out would free the array under the reader
        arr = self.values.get(n.index)
        if arr is not None:
            return arr
        host = self.host_values.get(n.index)
        if host is None:
            raise RuntimeError("tensor of node %d (%s) is neither on the GPU nor swapped out" % (n.index, n.name))
        self.passive_swap_in += 1
        arr = ndarray.empty(self.node_to_shape_map[n], self.ctx_gpu)
        host.copyto(arr, self.cudaStream)
        self.values[n.index] = arr
        return arr

    def _compute(self, node):
        inputs = [self._resident(n) for n in node.inputs]
        if node.issgd:
            node.op.compute(node, inputs, None, self.cudnnHandle, self.cublasHandle, self.cudaStream, False)
            return
        out = ndarray.empty(self.node_to_shape_map[node], self.ctx_gpu)
        if isinstance(out, int):
            raise MemoryError("device out of memory allocating %d bytes for node %d (%s)" % (out, node.index, node.name))
        short = node.op.compute(node, inputs, out, self.cudnnHandle, self.cublasHandle, self.cudaStream, False)
        if short:
            raise MemoryError("device out of memory inside node %d (%s): %d bytes short" % (node.index, node.name, short))
        self.values[node.index] = out

    # ---- one training step ----------------------------------------------------------------------------
    def run(self, feed_dict, convert_to_numpy_ret_vals=False):
        self._ensure_handles()
        # The previous step's intermediates go back to the pool one at a time, each just before the node that produced it
        # runs again (its new output then takes the very block that was freed): dropping all ~600-1800 arrays here would
        # be a millisecond or two of DLArrayFree calls during which a GPU that has just been synchronised sits idle.
        stale, self.values = self.values, {}
        feed_shapes = {}
        for node, value in feed_dict.items():
            if not ndarray.is_gpu_ctx(value.ctx):
                value = value.copyto(self.ctx_gpu, None)
            self.values[node.index] = value
            feed_shapes[node] = value.shape
        if self.feed_shapes != feed_shapes:
            self.infer_shape(feed_shapes)
            self.feed_shapes = feed_shapes
        if self.top_control_queue is not None and not self.top_control_queue.empty():
            self._apply_plan(*self.top_control_queue.get())

        timed = self.top_message_queue is not None
        for node in self.topo_order:
            if node.index in self.values and not node.inputs:
                if self.have_plan:
                    self._after_node(node)
                continue
            stale.pop(node.index, None)
            if self.have_plan:
                for idx in node.recompute_list:
                    self._compute(self.topo_order[idx])
            if timed:
                t0 = time.perf_counter()
                self._compute(node)
                node.runtime = (time.perf_counter() - t0) * 1000.0
            else:
                self._compute(node)
            if self.have_plan:
                self._after_node(node)

        stale.clear()
        self.b1t[0] *= self.b1
        self.b2t[0] *= self.b2
        if self._swap_worker is not None:
            self._swap_worker.drain()
        loss = self._resident(self.targetloss)
        next_feed = {n: self.values[n.index] for n in feed_dict if n.isw == 1}
        if convert_to_numpy_ret_vals:
            return [loss.asnumpy(), {n: v.asnumpy() for n, v in next_feed.items()}]
        return [loss, next_feed]

    # ---- inspection helpers (no counterpart in the reference) ---------------------------------------------
    def value_of(self, node):
        """GPU array computed for ``node`` in the most recent ``run``."""
        return self._resident(node)

    def gradient_of(self, variable):
        return self._resident(self.Variable_node_to_grad[variable])

    def synchronize(self):
        gpu_op.device_synchronize()

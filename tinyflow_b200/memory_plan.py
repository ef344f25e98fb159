"""Memory plans for the executor: which tensors to swap out to pinned host memory, when to bring them
back, and which to release early.

The executor consumes plans in the reference's message format (autodiff.py:2561-2590, produced there by
Scheduler.py:304-331):

* ``swap_list``      entries ``(tensor_id, start_time_ms, start_node_id, move_to_gpu)``: once node ``start_node_id``
                     has been issued, wait ``start_time_ms`` and move tensor ``tensor_id`` (a node index of the
                     executor's topological order) to the host (0) or back to the GPU (1);
* ``release_list``   entries ``(start_node_id, tensor_id)``: free the tensor's device memory after that node;
* ``recompute_list`` entries ``(start_node_id, tensor_id)``: re-run the producer of the tensor before that node.

:func:`vdnn_plan` is a static policy in the style of vDNN (offload the inputs of convolution layers after their last
forward use, prefetch them ahead of their first backward use); the reference ships its vDNN baseline on another
branch, so the policy is restated here from the published description.  :func:`check_plan` verifies the
invariants a plan has to satisfy for the executor to run without passive swap-ins.
"""
from __future__ import annotations


def _consumers(order):
    users = {n.index: [] for n in order}
    for n in order:
        for i in n.inputs:
            users[i.index].append(n.index)
    return users


def vdnn_plan(executor, policy="conv", prefetch=48, release=True, min_bytes=1 << 20):
    """Build ``(swap_list, release_list, recompute_list)`` for ``executor`` (its shapes must have been inferred).

    policy    "conv": offload the input feature maps of convolution layers; "all": every activation that is read
              again by the backward pass.
    prefetch  how many nodes before the first backward reader the swap-in is issued (a 17 MB tensor takes 0.3 ms over the
              host link, the time of some tens of backward nodes: issued only a few nodes ahead, every swap-in stalls
              its reader for the whole copy).
    release   also free every intermediate tensor right after its last reader.
    min_bytes tensors smaller than this stay resident.
    """
    order = executor.topo_order
    shapes = executor.node_to_shape_map
    if shapes is None:
        raise ValueError("call executor.infer_shape (or run one step) before planning")
    loss_index = executor.targetloss.index
    users = _consumers(order)
    keep = {n.index for n in executor.eval_node_list}

    def nbytes(node):
        n = 4
        for d in shapes[node]:
            n *= int(d)
        return n

    swap_list, release_list = [], []
    for node in order:
        t = node.index
        if not node.inputs or node.issgd or t in keep or t >= loss_index:
            continue                                   # placeholders, parameters, optimiser nodes, backward tensors
        readers = users[t]
        fwd = [u for u in readers if u <= loss_index]
        bwd = [u for u in readers if u > loss_index]
        if not fwd or not bwd or nbytes(node) < min_bytes:
            continue
        if policy == "conv" and not any(type(order[u].op).__name__ == "Convolution2DForwardOp" for u in fwd):
            continue
        out_after = max(fwd)
        first_back = min(bwd)
        in_at = max(first_back - prefetch, out_after + 1, loss_index)
        if in_at >= first_back:
            continue                                   # nothing to gain: the tensor is needed again immediately
        swap_list.append((t, 0, out_after, 0))
        swap_list.append((t, 0, in_at, 1))
    if release:
        for node in order:
            t = node.index
            if not node.inputs or node.issgd or node.isw or t in keep or not users[t]:
                continue
            release_list.append((max(users[t]), t))
    # the executor walks a node's messages in list order: keep them sorted by trigger
    swap_list.sort(key=lambda e: (e[2], e[3]))
    release_list.sort()
    return swap_list, release_list, []


def check_plan(executor, plan):
    """Raise ``AssertionError`` unless: every tensor swapped out is swapped back in before its next reader, is not
    read while away, and nothing is released before its last reader.  Returns the bytes that are away from the GPU
    at the point of the plan where that figure peaks."""
    swap_list, release_list, recompute_list = plan
    order = executor.topo_order
    users = _consumers(order)
    shapes = executor.node_to_shape_map
    events = {}
    for t, _wait, start, to_gpu in swap_list:
        events.setdefault(t, []).append((start, to_gpu))
    away_delta = [0] * (len(order) + 1)
    for t, ev in events.items():
        ev.sort()
        assert [g for _, g in ev] == [0, 1] * (len(ev) // 2), "tensor %d: swap-out / swap-in must alternate" % t
        size = 4
        for d in shapes[order[t]]:
            size *= int(d)
        for (out_at, _), (in_at, _) in zip(ev[0::2], ev[1::2]):
            assert out_at >= t, "tensor %d swapped out before it exists" % t
            assert in_at > out_at
            for u in users[t]:
                assert not (out_at < u <= in_at), "tensor %d is read by node %d while swapped out" % (t, u)
            away_delta[out_at] += size
            away_delta[in_at] -= size
    for start, t in release_list:
        assert all(u <= start for u in users[t]), "tensor %d released before its last reader" % t
    for start, t in recompute_list:
        assert start > t
    peak = run = 0
    for d in away_delta:
        run += d
        peak = max(peak, run)
    return peak

"""Memory plans in the reference's message format (swap / release lists, autodiff.py:2561-2590) replayed by the
executor: the plan generator's invariants on CPU, and on the GPU a step under a plan against the same step
without one."""
import queue

import numpy as np
import pytest


def _executor(model, optimizer="adam", control=None):
    from tinyflow_b200 import autodiff as ad
    ex = ad.Executor(model.loss, model.y, 0.001, control, None, None, optimizer=optimizer)
    shapes = {model.X: model.input_shape, model.y_: model.label_shape}
    for var, shape in model.param_shapes.items():
        shapes[var] = tuple(shape)
        if var in ex.Variable_node_to_mv:
            m, v = ex.Variable_node_to_mv[var]
            shapes[m] = shapes[v] = tuple(shape)
    ex.infer_shape(shapes)
    return ex


@pytest.mark.parametrize("name,kwargs", [("resnet50", dict(batch=8, image=64)), ("inceptionv3", dict(batch=4, image=75)), ("vgg16", dict(batch=4, image=32))])
@pytest.mark.parametrize("policy", ["conv", "all"])
def test_vdnn_plan_invariants(lib_path, name, kwargs, policy):
    from tinyflow_b200 import models, memory_plan
    model = getattr(models, name)(**kwargs)
    ex = _executor(model)
    plan = memory_plan.vdnn_plan(ex, policy=policy, min_bytes=0)
    swap_list, release_list, recompute_list = plan
    assert swap_list and release_list and not recompute_list
    away = memory_plan.check_plan(ex, plan)
    assert away > 0
    order = ex.topo_order
    outs = [e for e in swap_list if e[3] == 0]
    assert len(outs) * 2 == len(swap_list)
    if policy == "conv":
        for t, _w, start, _g in outs:
            readers = [n for n in order if order[t] in n.inputs and n.index <= ex.targetloss.index]
            assert any(type(n.op).__name__ == "Convolution2DForwardOp" for n in readers)
            assert start == max(n.index for n in readers)          # after the LAST forward reader
    # parameters, optimiser state and the outputs the caller reads are never touched
    protected = {n.index for n in ex.eval_node_list}
    assert not protected & {e[0] for e in swap_list}
    assert not protected & {t for _s, t in release_list}


def test_check_plan_rejects_a_read_while_swapped_out(lib_path):
    from tinyflow_b200 import models, memory_plan
    model = models.vgg16(batch=4, image=32)
    ex = _executor(model)
    swap_list, release_list, _ = memory_plan.vdnn_plan(ex, min_bytes=0)
    t, w, start, _g = swap_list[0]
    bad = [(t, w, start - 1, 0)] + [e for e in swap_list[1:]]
    with pytest.raises(AssertionError):
        memory_plan.check_plan(ex, (bad, release_list, []))
    with pytest.raises(AssertionError):
        memory_plan.check_plan(ex, (swap_list, [(release_list[0][0] - 1, release_list[0][1])] + release_list[1:], []))


@pytest.mark.gpu
@pytest.mark.parametrize("optimizer", ["adam", "sgd"])
def test_step_under_a_swap_and_release_plan_matches_the_plain_step(lib_path, optimizer):
    """Inception-v3 (reduced) for one step, with and without a vDNN-style plan delivered through the control queue:
    same loss and same updated parameters (the plan only moves and frees tensors), no passive swap-in, and less
    device memory in use at the end of the step."""
    from tinyflow_b200 import models, memory_plan, ndarray, gpu_op
    from tests.test_gpu_models import _feed

    def one_step(with_plan):
        base_used, _ = gpu_op.allocator_stats()          # whatever earlier tests of this process still hold
        model = models.inceptionv3(batch=4, image=75, classes=100)
        model.set_dropout(0.0)
        control = queue.Queue()
        ex = _executor(model, optimizer, control)
        if with_plan:
            plan = memory_plan.vdnn_plan(ex, policy="conv", min_bytes=0)
            memory_plan.check_plan(ex, plan)
            control.put(plan)
        ctx = ndarray.gpu(0)
        feed_np = _feed(model)
        feed = {n: ndarray.array(v, ctx) for n, v in feed_np.items()}
        for var in model.param_shapes:
            if var in ex.Variable_node_to_mv:
                for mv in ex.Variable_node_to_mv[var]:
                    feed[mv] = ndarray.array(np.zeros(model.param_shapes[var], np.float32), ctx)
        loss, nxt = ex.run(feed)
        ex.synchronize()
        used, _cached = gpu_op.allocator_stats()
        out = {n.name: v.asnumpy() for n, v in nxt.items() if n in model.param_shapes}
        return float(loss.asnumpy().ravel()[0]), out, used - base_used, ex.passive_swap_in, len(ex.host_values)

    loss0, w0, used0, _p0, _h0 = one_step(False)
    loss1, w1, used1, passive, swapped = one_step(True)
    assert swapped > 20 and passive == 0
    assert loss1 == loss0
    for k in w0:
        scale = max(np.abs(w0[k]).max(), 1e-12)
        diff = np.abs(w1[k] - w0[k])
        assert diff.max() == 0.0, k                   # every kernel is bit-reproducible: the plan changes nothing
    assert used1 < 0.85 * used0          # parameters, optimiser state and the packed operands of the conv plans stay

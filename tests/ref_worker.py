"""Child process of tests/test_gpu_reference_python.py: drives this library through the reference's own,
unmodified Python (``baseline/_ref/pycode/tinyflow``) and writes what it computed to an .npz file.

    python tests/ref_worker.py <adam|plan> <out.npz> [steps]

The reference's ``Executor`` starts two non-daemon threads that never exit (autodiff.py:31-150,
2296-2299), so this process ends with ``os._exit`` as the reference's own drivers do (util.py:117-118).

mode adam  ``steps`` Adam steps of the ResNet-50 graph (batch 8, 64x64 images, 10 classes) through the reference's
           ``autodiff.Executor``, then the same steps through this repository's mirrored executor; both start from
           the same seeded parameters.
mode plan  the same through the reference executor with a swap / release plan (the reference's message format)
           put on its control queue after the first step, so that its ``MemoryManagerController`` /
           ``MemoryManager`` threads move tensors with DLArrayCopyFromTo / DLArrayFree while the main thread computes.
"""
import os
import queue
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
sys.path.insert(0, REPO)
sys.path.insert(0, HERE)


def build(models, ad):
    """The ResNet-50 graph built with graph library ``ad`` (the reference's or the mirror: same constructor names)."""
    saved = models.ad
    models.ad = ad
    try:
        model = models.resnet50(batch=8, image=64, classes=10)
    finally:
        models.ad = saved
    model.set_dropout(0.0)
    return model


def run_steps(ad, nd, model, params, X, Y, steps, plan_after=None, plan_fn=None):
    control, messages = queue.Queue(), queue.Queue()
    log_dir = tempfile.mkdtemp(prefix="tinyflow_vanilla_")          # any path without 'schedule' in it (autodiff.py:2611)
    ex = ad.Executor(model.loss, model.y, 0.001, control, messages, log_dir)
    ctx = nd.gpu(0)
    feed = {n: nd.array(v, ctx) for n, v in params.items()}
    for var in list(params):
        m, v = ex.Variable_node_to_mv[var]
        feed[m] = nd.array(np.zeros(params[var].shape, np.float32), ctx)
        feed[v] = nd.array(np.zeros(params[var].shape, np.float32), ctx)
    losses, snapshots = [], []
    for step in range(steps):
        if plan_after is not None and step == plan_after:
            control.put(plan_fn(ex))
        feed[model.X], feed[model.y_] = nd.array(X, ctx), nd.array(Y, ctx)
        res = ex.run(feed_dict=feed)
        losses.append(float(np.asarray(res[0].asnumpy()).ravel()[0]))
        feed = dict(res[1])
        if os.environ.get("TINYFLOW_REF_SNAPSHOTS"):
            snapshots.append({var.name: feed[var].asnumpy() for var in params})
    final = {var.name: feed[var].asnumpy() for var in params}
    if snapshots:
        for i, snap in enumerate(snapshots):
            final.update({"step%d_%s" % (i, k): v for k, v in snap.items()})
    return ex, losses, final


def main():
    mode, out = sys.argv[1], sys.argv[2]
    steps = int(sys.argv[3]) if len(sys.argv) > 3 else 2
    import reference_checkout
    ref_ad = reference_checkout.import_reference()
    from pycode.tinyflow import ndarray as ref_nd
    from tinyflow_b200 import autodiff as mirror_ad, memory_plan, models, ndarray as mirror_nd

    ref_model = build(models, ref_ad)
    X, Y = models.synthetic_batch(ref_model, seed=1234)
    ref_params = ref_model.init_params(seed=123)
    result = {}
    if mode == "adam":
        _, losses, final = run_steps(ref_ad, ref_nd, ref_model, ref_params, X, Y, steps)
        result["ref_losses"] = np.array(losses)
        result.update({"ref_" + k: v for k, v in final.items()})
        mir_model = build(models, mirror_ad)
        mir_params = mir_model.init_params(seed=123)
        _, losses, final = run_steps(mirror_ad, mirror_nd, mir_model, mir_params, X, Y, steps)
        result["mirror_losses"] = np.array(losses)
        result.update({"mirror_" + k: v for k, v in final.items()})
    elif mode == "plan":
        def plan_fn(ex):
            plan = memory_plan.vdnn_plan(ex, policy="conv", min_bytes=0)
            memory_plan.check_plan(ex, plan)
            result["swaps"] = np.array(len(plan[0]))
            result["releases"] = np.array(len(plan[1]))
            return plan
        _, losses, final = run_steps(ref_ad, ref_nd, ref_model, ref_params, X, Y, steps, plan_after=1, plan_fn=plan_fn)
        result["ref_losses"] = np.array(losses)
        result["control_messages_taken"] = np.array(int(ref_ad.have_got_control_message))
        result.update({"ref_" + k: v for k, v in final.items()})
    else:
        raise SystemExit("unknown mode " + mode)
    np.savez(out, **result)
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    try:
        main()
    except BaseException:
        import traceback
        traceback.print_exc()
        sys.stderr.flush()
        os._exit(1)

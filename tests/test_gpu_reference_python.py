"""The reference's own Python, unmodified, on top of this library (GPU).

``baseline/_ref/pycode`` (git-ignored; created by ``python tests/reference_checkout.py <reference checkout>``)
holds the reference's ``_base.py`` / ``ndarray.py`` / ``gpu_op.py`` / ``autodiff.py`` as they are.  The tests run
its ``autodiff.Executor`` (autodiff.py:2240-2890: ctypes calls without argtypes, pinned host mirror per node, the
``MemoryManagerController`` / ``MemoryManager`` threads) in a child process and compare with this repository's
mirrored executor and with the float64 oracle.  They are skipped, with a message, where the checkout is absent.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import reference_checkout  # noqa: E402

needs_reference = pytest.mark.skipif(not reference_checkout.available(),
                                     reason="baseline/_ref/pycode is absent: python tests/reference_checkout.py <reference checkout>")


def _worker(mode, out, steps):
    r = subprocess.run([sys.executable, os.path.join(HERE, "ref_worker.py"), mode, out, str(steps)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, "worker failed:\n" + r.stdout[-2000:] + r.stderr[-4000:]
    return np.load(out)


@needs_reference
def test_reference_executor_trains_resnet50_with_adam_like_the_mirror_and_the_oracle(lib_path, tmp_path):
    d = _worker("adam", str(tmp_path / "adam.npz"), 2)
    ref_losses, mir_losses = d["ref_losses"], d["mirror_losses"]
    assert np.all(np.isfinite(ref_losses))
    # the same library calls in the same order, and every kernel of the library is bit-reproducible (no floating-point
    # atomics): the two drivers must agree exactly
    np.testing.assert_array_equal(ref_losses, mir_losses)
    names = [k[4:] for k in d.files if k.startswith("ref_") and k != "ref_losses" and not k.startswith("ref_step")]
    assert len(names) >= 50
    for name in names:
        np.testing.assert_array_equal(d["ref_" + name], d["mirror_" + name], err_msg=name)
    # first step's loss against the float64 oracle on the same seeded inputs
    from oracle.graph_eval import OracleExecutor
    from tinyflow_b200 import autodiff as ad, models
    model = models.resnet50(batch=8, image=64, classes=10)
    model.set_dropout(0.0)
    ex = ad.Executor(model.loss, model.y, 0.001, None, None, None, optimizer="adam")
    X, Y = models.synthetic_batch(model, seed=1234)
    feed = {model.X: X, model.y_: Y}
    params = model.init_params(seed=123)
    feed.update(params)
    for var in params:
        m, v = ex.Variable_node_to_mv[var]
        feed[m], feed[v] = np.zeros_like(params[var]), np.zeros_like(params[var])
    # 53 per-activation batch-norms over a batch of 8 amplify fp32 rounding (see tests/test_gpu_models.py): the loss of an
    # fp32 execution is a 1e-3 quantity here, each kernel on its own inputs a 1e-4 one (checked there, node by node)
    want = float(OracleExecutor(ex.topo_order, np.float64).run(feed)[model.loss].ravel()[0])
    assert abs(ref_losses[0] - want) <= 1e-3 * abs(want)
    # Adam's first steps move every weight by about lr in the direction of -sign(g): the update is bounded
    for name in names:
        assert np.abs(d["ref_" + name] - params[[v for v in params if v.name == name][0]]).max() <= 2 * 0.001 * 1.01 + 1e-7, name


@needs_reference
def test_reference_memory_manager_threads_replay_a_swap_plan(lib_path, tmp_path):
    """A (swap, release, recompute) plan on the reference executor's control queue: its own swap threads call
    DLArrayCopyFromTo / DLArrayAlloc / DLArrayFree concurrently with the main thread.  The training result must not
    change."""
    plain = _worker("adam", str(tmp_path / "plain.npz"), 3)
    plan = _worker("plan", str(tmp_path / "plan.npz"), 3)
    assert int(plan["swaps"]) > 0 and int(plan["releases"]) > 0
    assert int(plan["control_messages_taken"]) >= 1
    np.testing.assert_array_equal(plan["ref_losses"], plain["ref_losses"])       # moving tensors must not change a bit
    for k in plan.files:
        if k.startswith("ref_") and k != "ref_losses":
            np.testing.assert_array_equal(plan[k], plain[k], err_msg=k)

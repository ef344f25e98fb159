"""Data-parallel path: bucket planning and the exchange arithmetic on CPU (gloo, world size 2), and the
NCCL path on real GPUs when the box has at least two."""
import ctypes
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_bucket_planner(lib_path):
    lib = ctypes.CDLL(lib_path)
    sizes = [10, 20, 30, 100, 5, 5, 41]
    counts = (ctypes.c_longlong * len(sizes))(*sizes)
    out = (ctypes.c_int * len(sizes))()
    n = lib.TfDpPlanBuckets(counts, len(sizes), ctypes.c_longlong(50), out)
    # 10+20 fit, 30 opens bucket 1, 100 is oversize (own bucket 2, marked negative), 5+5+... reopen at 3
    assert list(out) == [0, 0, 1, -3, 3, 3, 4] and n == 5
    # ResNet-50 gradient sizes in arrival order (last layer first) with 32 MiB buckets: a handful of buckets
    sys.path.insert(0, REPO)
    from tinyflow_b200 import models
    m = models.resnet50()
    sizes = [int(np.prod(s)) for s in reversed(list(m.param_shapes.values()))]
    counts = (ctypes.c_longlong * len(sizes))(*sizes)
    out = (ctypes.c_int * len(sizes))()
    n = lib.TfDpPlanBuckets(counts, len(sizes), ctypes.c_longlong(32 * 1024 * 1024 // 4), out)
    assert 4 <= n <= 8 and min(out) >= 0
    assert sum(sizes) == 29700264


def _gloo_rank(rank, world, port, q):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, REPO)
    from oracle.graph_eval import OracleExecutor
    from tinyflow_b200 import autodiff as ad, models
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    model = models.mlp(batch=16, sizes=(12, 10, 8, 4))
    params = list(model.param_shapes)
    grads = ad.gradients(model.loss, params)
    topo = ad.find_topo_sort([model.loss] + grads)
    X, Y = models.synthetic_batch(model, seed=77, rank=rank, input_dist="uniform")
    feed = {model.X: X, model.y_: Y}
    init = model.init_params(seed=5)
    feed.update(init)
    vals = OracleExecutor(topo, np.float64).run(feed)
    lr, out = 0.1, {}
    for p, g in zip(params, grads):
        t = torch.tensor(vals[g])
        dist.all_reduce(t)                       # the exchange step: sum over ranks
        out[p.name] = init[p].astype(np.float64) - lr / world * t.numpy()     # w -= (lr / world) * sum_r g_r
    if rank == 0:
        q.put(out)
    dist.destroy_process_group()


def test_two_rank_exchange_equals_large_batch_step():
    """The exchange rule  w -= (lr / world) * sum_r g_r  against one step on the concatenated batch.  The
    reference's softmax-cross-entropy gradient is a SUM over samples (it is not divided by the batch,
    autodiff.py:710-713), so sum_r g_r is exactly the gradient of the concatenated batch and the data-parallel
    step equals a large-batch step with learning rate lr / world.  World size 2 over gloo on CPU."""
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_gloo_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    sys.path.insert(0, REPO)
    from oracle.graph_eval import OracleExecutor
    from tinyflow_b200 import autodiff as ad, models
    model = models.mlp(batch=32, sizes=(12, 10, 8, 4))
    small = models.mlp(batch=16, sizes=(12, 10, 8, 4))
    shards = [models.synthetic_batch(small, seed=77, rank=r, input_dist="uniform") for r in range(2)]
    X, Y = np.concatenate([s[0] for s in shards]), np.concatenate([s[1] for s in shards])
    params = list(model.param_shapes)
    grads = ad.gradients(model.loss, params)
    feed = {model.X: X, model.y_: Y}
    init = model.init_params(seed=5)
    feed.update(init)
    vals = OracleExecutor(ad.find_topo_sort([model.loss] + grads), np.float64).run(feed)
    for p, g in zip(params, grads):
        np.testing.assert_allclose(got[p.name], init[p] - 0.1 / 2 * vals[g], rtol=1e-9, atol=1e-12)


@pytest.mark.gpu
def test_nccl_data_parallel_step_matches_oracle(lib_path):
    """Two ranks on two GPUs: weights after two data-parallel SGD steps equal the oracle's step with the
    rank-averaged gradient, and are identical on both ranks."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    with tempfile.TemporaryDirectory() as d:
        procs = []
        for r in range(world):
            env = dict(os.environ, RANK=str(r), WORLD=str(world), ID_FILE=os.path.join(d, "nccl_id"), OUT=os.path.join(d, "w%d.npz" % r),
                       CUDA_VISIBLE_DEVICES=str(r), STEPS="2", NCCL_NVLS_ENABLE="0")
            procs.append(subprocess.Popen([sys.executable, os.path.join(REPO, "tests", "dp_worker.py")], env=env))
        for p in procs:
            assert p.wait(timeout=300) == 0
        w = [dict(np.load(os.path.join(d, "w%d.npz" % r))) for r in range(world)]
    for k in w[0]:
        np.testing.assert_array_equal(w[0][k], w[1][k])
    # oracle: two steps with the averaged gradient
    sys.path.insert(0, REPO)
    from oracle.graph_eval import OracleExecutor
    from tinyflow_b200 import autodiff as ad, models
    sys.path.insert(0, os.path.join(REPO, "tests"))
    import dp_worker
    model = dp_worker.build()
    params = list(model.param_shapes)
    grads = ad.gradients(model.loss, params)
    topo = ad.find_topo_sort([model.loss] + grads)
    cur = {p: v.astype(np.float64) for p, v in model.init_params(seed=5).items()}
    for _ in range(2):
        acc = {p: 0.0 for p in params}
        for r in range(world):
            X, Y = dp_worker.shard(model, r)
            feed = {model.X: X, model.y_: Y}
            feed.update(cur)
            vals = OracleExecutor(topo, np.float64).run(feed)
            for p, g in zip(params, grads):
                acc[p] = acc[p] + vals[g]
        cur = {p: cur[p] - 0.05 / world * acc[p] for p in params}
    for p in params:
        want = cur[p]
        scale = np.maximum(np.abs(want), 0.05 * np.abs(want).max())
        assert (np.abs(w[0][p.name] - want) / scale).max() <= 1e-4, p.name

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
    # from the second step on the open bucket is closed once all but ~2 MiB of the step's gradients have arrived, so
    # that the step's last all-reduce (which nothing overlaps) is small
    total, tail = sum(sizes), 2 * 1024 * 1024 // 4
    out_tail = (ctypes.c_int * len(sizes))()
    n_tail = lib.TfDpPlanBucketsTail(counts, len(sizes), ctypes.c_longlong(32 * 1024 * 1024 // 4), ctypes.c_longlong(total), ctypes.c_longlong(tail), out_tail)
    assert n_tail == n + 1
    last = [sz for sz, b in zip(sizes, out_tail) if b == n_tail - 1]
    assert 0 < sum(last) <= tail
    first_step = (ctypes.c_int * len(sizes))()
    assert lib.TfDpPlanBucketsTail(counts, len(sizes), ctypes.c_longlong(32 * 1024 * 1024 // 4), ctypes.c_longlong(0), ctypes.c_longlong(tail), first_step) == n
    assert list(first_step) == list(out)


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
@pytest.mark.parametrize("opt,flush", [("sgd", "explicit"), ("adam", "explicit"), ("adam", "implicit")])
def test_nccl_data_parallel_step_matches_oracle(lib_path, opt, flush):
    """Two ranks on two GPUs: weights after two data-parallel steps equal the oracle's steps with the rank-averaged
    gradient, and are identical on both ranks - for SGD, for Adam (the reference executor's optimiser), and for a
    training loop that never calls TfDpFlush."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    with tempfile.TemporaryDirectory() as d:
        procs = []
        for r in range(world):
            env = dict(os.environ, RANK=str(r), WORLD=str(world), ID_FILE=os.path.join(d, "nccl_id"), OUT=os.path.join(d, "w%d.npz" % r),
                       CUDA_VISIBLE_DEVICES=str(r), STEPS="2", NCCL_NVLS_ENABLE="0", OPT=opt, FLUSH=flush)
            procs.append(subprocess.Popen([sys.executable, os.path.join(REPO, "tests", "dp_worker.py")], env=env))
        for p in procs:
            assert p.wait(timeout=300) == 0
        w = [dict(np.load(os.path.join(d, "w%d.npz" % r))) for r in range(world)]
    for k in w[0]:
        np.testing.assert_array_equal(w[0][k], w[1][k])
    # oracle: two steps with the averaged gradient
    sys.path.insert(0, REPO)
    import oracle.ops as ops
    from oracle.graph_eval import OracleExecutor
    from tinyflow_b200 import autodiff as ad, models
    sys.path.insert(0, os.path.join(REPO, "tests"))
    import dp_worker
    model = dp_worker.build()
    params = list(model.param_shapes)
    grads = ad.gradients(model.loss, params)
    topo = ad.find_topo_sort([model.loss] + grads)
    cur = {p: v.astype(np.float64) for p, v in model.init_params(seed=5).items()}
    mom = {p: (np.zeros_like(cur[p]), np.zeros_like(cur[p])) for p in params}
    lr = dp_worker.LR[opt]
    b1t, b2t = 0.9, 0.999
    for _ in range(2):
        acc = {p: 0.0 for p in params}
        for r in range(world):
            X, Y = dp_worker.shard(model, r)
            feed = {model.X: X, model.y_: Y}
            feed.update(cur)
            vals = OracleExecutor(topo, np.float64).run(feed)
            for p, g in zip(params, grads):
                acc[p] = acc[p] + vals[g]
        if opt == "sgd":
            cur = {p: cur[p] - lr / world * acc[p] for p in params}
        else:
            for p in params:
                w2, m2, v2 = ops.adam(cur[p], mom[p][0], mom[p][1], acc[p] / world, 0.9, 0.999, b1t, b2t, 1e-8, lr)
                cur[p], mom[p] = w2, (m2, v2)
            b1t, b2t = b1t * 0.9, b2t * 0.999
    for p in params:
        want = cur[p]
        if opt == "adam":
            # an Adam step is lr * m / sqrt(v): compare the two-step displacement, which is what the exchange affects
            start = model.init_params(seed=5)[p].astype(np.float64)
            got_step, want_step = w[0][p.name] - start, want - start
            clear = np.abs(want_step) > 0.5 * lr                      # entries whose gradient sign is not rounding noise
            assert np.abs(got_step[clear] - want_step[clear]).max() <= 2e-2 * lr * 2, p.name
            continue
        scale = np.maximum(np.abs(want), 1e-2 * np.abs(want).max())
        assert (np.abs(w[0][p.name] - want) / scale).max() <= 1e-4, p.name


# ---- failure handling on the host (no GPU is touched: the waits run out before NCCL is loaded) -----------------------
def _init_in_child(rank, world, path, timeout_s, q):
    os.environ["TINYFLOW_DP_INIT_TIMEOUT_S"] = str(timeout_s)
    import time
    lib = ctypes.CDLL(os.path.join(REPO, "build", "lib", "libc_runtime_api.so"))
    t0 = time.time()
    rc = lib.TfDpInit(rank, world, path.encode())
    buf = ctypes.create_string_buffer(512)
    lib.TfLastError(buf, 512)
    q.put((rc, time.time() - t0, buf.value.decode()))


def _run_init(path, timeout_s=0.6):
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_init_in_child, args=(1, 2, path, timeout_s, q))
    p.start()
    rc, took, msg = q.get(timeout=60)
    p.join(timeout=30)
    return rc, took, msg


def test_rendezvous_wait_is_bounded_when_rank_zero_never_arrives(lib_path, tmp_path):
    """Rank 1 of 2 waits for the id file of a rank 0 that never starts: TfDpInit returns -1 after the configured
    limit instead of blocking for good."""
    rc, took, msg = _run_init(str(tmp_path / "never_written"))
    assert rc == -1 and 0.5 <= took < 10 and "timed out" in msg


def test_rendezvous_rejects_a_stale_id_file(lib_path, tmp_path):
    """An id file left by a crashed run (right magic, an hour old) is not accepted: the other ranks keep waiting for
    rank 0 to publish a fresh one, within the limit."""
    import struct
    import time
    path = tmp_path / "stale"
    path.write_bytes(struct.pack("<QQ", 0x746664706E63636C, int(time.time()) - 3600) + bytes(128))
    rc, took, msg = _run_init(str(path))
    assert rc == -1 and "timed out" in msg
    path.write_bytes(b"short")                 # a truncated file is ignored as well
    rc, took, msg = _run_init(str(path))
    assert rc == -1 and "timed out" in msg

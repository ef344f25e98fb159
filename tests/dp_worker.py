"""One data-parallel rank: runs `steps` SGD steps of a small CNN on its own shard and saves the weights.
Launched by tests/test_dp.py with RANK / WORLD / ID_FILE / OUT in the environment and CUDA_VISIBLE_DEVICES
set to this rank's GPU (the executor addresses its GPU as gpu(0))."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def build():
    from tinyflow_b200 import models
    model = models.lenet5(batch=32)
    return model


def shard(model, rank):
    from tinyflow_b200 import models
    return models.synthetic_batch(model, seed=77, rank=rank, input_dist="uniform")


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD"])
    steps, lr = int(os.environ.get("STEPS", "2")), 0.05
    from tinyflow_b200 import autodiff as ad, ndarray
    from tinyflow_b200._base import _LIB, check_call
    check_call(_LIB.TfDpInit(rank, world, os.environ["ID_FILE"].encode()))
    model = build()
    X, Y = shard(model, rank)
    ex = ad.Executor(model.loss, model.y, lr, None, None, None, optimizer="sgd")
    ctx = ndarray.gpu(0)
    feed = {n: ndarray.array(v, ctx) for n, v in model.init_params(seed=5).items()}
    for _ in range(steps):
        feed[model.X], feed[model.y_] = ndarray.array(X, ctx), ndarray.array(Y, ctx)
        loss, feed = ex.run(feed)
        check_call(_LIB.TfDpFlush(ex.cudaStream))
    np.savez(os.environ["OUT"], **{n.name: v.asnumpy() for n, v in feed.items()})
    check_call(_LIB.TfDpShutdown())
    os._exit(0)


if __name__ == "__main__":
    main()

"""One data-parallel rank: runs `steps` optimiser steps of a small CNN on its own shard and saves the weights.
Launched by tests/test_dp.py with RANK / WORLD / ID_FILE / OUT in the environment and CUDA_VISIBLE_DEVICES
set to this rank's GPU (the executor addresses its GPU as gpu(0)).  OPT = sgd | adam; FLUSH = explicit (TfDpFlush after
every step) | implicit (nothing: the next step's blocking upload of the batch is the step boundary, as for a training
loop that does not know the exchange exists)."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

LR = {"sgd": 0.05, "adam": 0.001}


def build():
    from tinyflow_b200 import models
    model = models.lenet5(batch=32)
    return model


def shard(model, rank):
    from tinyflow_b200 import models
    return models.synthetic_batch(model, seed=77, rank=rank, input_dist="uniform")


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD"])
    steps, opt, flush = int(os.environ.get("STEPS", "2")), os.environ.get("OPT", "sgd"), os.environ.get("FLUSH", "explicit")
    from tinyflow_b200 import autodiff as ad, ndarray
    from tinyflow_b200._base import _LIB, check_call
    check_call(_LIB.TfDpInit(rank, world, os.environ["ID_FILE"].encode()))
    model = build()
    X, Y = shard(model, rank)
    ex = ad.Executor(model.loss, model.y, LR[opt], None, None, None, optimizer=opt)
    ctx = ndarray.gpu(0)
    init = model.init_params(seed=5)
    feed = {n: ndarray.array(v, ctx) for n, v in init.items()}
    if opt == "adam":
        for var, val in init.items():
            m, v = ex.Variable_node_to_mv[var]
            feed[m], feed[v] = ndarray.array(np.zeros_like(val), ctx), ndarray.array(np.zeros_like(val), ctx)
    for _ in range(steps):
        feed[model.X], feed[model.y_] = ndarray.array(X, ctx), ndarray.array(Y, ctx)
        loss, feed = ex.run(feed)
        if flush == "explicit":
            check_call(_LIB.TfDpFlush(ex.cudaStream))
    np.savez(os.environ["OUT"], **{n.name: v.asnumpy() for n, v in feed.items()})      # the read-back is a step boundary too
    check_call(_LIB.TfDpShutdown())
    return 0


if __name__ == "__main__":
    sys.exit(main())

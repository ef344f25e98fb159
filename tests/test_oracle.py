"""Pins the CPU oracle: against the reference's own numpy executor (golden fixtures) where the
reference has numpy branches, and against torch-CPU float64 autograd (an independent second
implementation) for the operators that are cuDNN calls in the reference."""
import json
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as Fn

from oracle import ops
from oracle.graph_eval import OracleExecutor

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
RNG = np.random.RandomState(0)


def _mirror_mlp(sizes, batch):
    from tinyflow_b200 import autodiff as ad, models
    m = models.mlp(batch=batch, sizes=sizes)
    params = list(m.param_shapes)
    grads = ad.gradients(m.loss, params)
    topo = ad.find_topo_sort([m.loss, m.y] + grads)
    return m, params, grads, topo


def test_mlp_small_matches_reference_numpy_executor(lib_path):
    g = np.load(os.path.join(GOLDEN, "mlp_small.npz"))
    m, params, grads, topo = _mirror_mlp((12, 20, 16, 5), 8)
    feed = {m.X: g["X"], m.y_: g["Y"]}
    feed.update({p: g[p.name] for p in params})
    vals = OracleExecutor(topo, np.float64).run(feed)
    np.testing.assert_allclose(vals[m.loss], g["loss"], rtol=1e-12)
    np.testing.assert_allclose(vals[m.y], g["logits"], rtol=1e-12)
    for p, gr in zip(params, grads):
        np.testing.assert_allclose(vals[gr], g["g" + p.name], rtol=1e-10, atol=1e-14)


def test_mlp_benchmark_config_matches_reference_digest(lib_path):
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    d = json.load(open(os.path.join(GOLDEN, "mlp_c1_digest.json")))
    X, Y, Ws, bs = mg.mlp_inputs(tuple(d["sizes"]), d["batch"], d["seed"])
    bs = [np.zeros_like(b) for b in bs]
    m, params, grads, topo = _mirror_mlp(tuple(d["sizes"]), d["batch"])
    feed = {m.X: X, m.y_: Y}
    feed.update(dict(zip(params, Ws + bs)))
    vals = OracleExecutor(topo, np.float64).run(feed)
    assert abs(vals[m.loss][0] - d["loss"]) <= 1e-12 * abs(d["loss"])
    for p, gr in zip(params, grads):
        gd = d["grads"][p.name]
        gv = vals[gr].reshape(-1)
        np.testing.assert_allclose(gv.sum(), gd["sum"], rtol=1e-9, atol=1e-12)
        np.testing.assert_allclose(np.abs(gv).sum(), gd["abs_sum"], rtol=1e-10)
        np.testing.assert_allclose(gv[gd["index"]], gd["value"], rtol=1e-10, atol=1e-15)


CONV_CASES = [
    # N, C, H, W, K, R, S, padding, sh, sw
    (2, 3, 9, 9, 4, 3, 3, "SAME", 1, 1),
    (2, 5, 11, 10, 6, 1, 1, "VALID", 2, 2),
    (1, 4, 12, 12, 3, 5, 5, "SAME", 1, 1),
    (2, 3, 13, 13, 4, 7, 7, "VALID", 2, 2),
    (2, 4, 9, 9, 5, 1, 7, "SAME", 1, 1),
    (2, 4, 9, 9, 5, 7, 1, "SAME", 1, 1),
    (2, 6, 11, 11, 4, 3, 3, "VALID", 2, 2),
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_matches_torch_autograd(case):
    N, C, H, W, K, R, S, padding, sh, sw = case
    x = RNG.randn(N, C, H, W)
    w = RNG.randn(K, C, R, S)
    g = ops.conv_geometry(x.shape, w.shape, padding, sh, sw)
    xt = torch.tensor(x, requires_grad=True)
    wt = torch.tensor(w, requires_grad=True)
    yt = Fn.conv2d(xt, wt, stride=(sh, sw), padding=(g["ph"], g["pw"]))
    y = ops.conv2d_fwd(x, w, g)
    np.testing.assert_allclose(y, yt.detach().numpy(), rtol=1e-10, atol=1e-12)
    dy = RNG.randn(*y.shape)
    yt.backward(torch.tensor(dy))
    np.testing.assert_allclose(ops.conv2d_dgrad(dy, w, g), xt.grad.numpy(), rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(ops.conv2d_wgrad(x, dy, g), wt.grad.numpy(), rtol=1e-10, atol=1e-12)


POOL_CASES = [(2, 3, 8, 8, 0, 0, 2, 2, 2, 2), (2, 3, 9, 9, 0, 0, 2, 2, 3, 3), (1, 2, 7, 7, 1, 1, 1, 1, 3, 3),
              (2, 2, 7, 7, 0, 0, 1, 1, 7, 7), (1, 2, 9, 9, 0, 0, 2, 2, 3, 3)]


@pytest.mark.parametrize("case", POOL_CASES)
def test_pooling_matches_torch_autograd(case):
    N, C, H, W, ph, pw, sh, sw, kh, kw = case
    x = RNG.randn(N, C, H, W)
    g = ops.pool_geometry(x.shape, ph, pw, sh, sw, kh, kw)
    for mode in ("max", "mean"):
        xt = torch.tensor(x, requires_grad=True)
        if mode == "max":
            yt = Fn.max_pool2d(xt, (kh, kw), (sh, sw), (ph, pw))
            y = ops.maxpool_fwd(x, g)[0]
        else:
            yt = Fn.avg_pool2d(xt, (kh, kw), (sh, sw), (ph, pw), count_include_pad=True)
            y = ops.avgpool_fwd(x, g)
        np.testing.assert_allclose(y, yt.detach().numpy(), rtol=1e-12)
        dy = RNG.randn(*y.shape)
        yt.backward(torch.tensor(dy))
        dx = ops.maxpool_bwd(x, dy, g) if mode == "max" else ops.avgpool_bwd(dy, g)
        np.testing.assert_allclose(dx, xt.grad.numpy(), rtol=1e-12, atol=1e-14)


def test_maxpool_ties_and_all_padding_windows():
    x = np.zeros((1, 1, 4, 4))
    g = ops.pool_geometry(x.shape, 0, 0, 2, 2, 2, 2)
    y, idx = ops.maxpool_fwd(x, g)
    assert idx.tolist() == [[[[0, 2], [8, 10]]]]            # first element of each window wins the tie
    # the reference's "zero padding" pool: 1x1 window, stride 1, padding 3
    x = RNG.randn(1, 1, 3, 3)
    g = ops.pool_geometry(x.shape, 3, 3, 1, 1, 1, 1)
    y, idx = ops.maxpool_fwd(x, g)
    assert y.shape == (1, 1, 9, 9)
    np.testing.assert_array_equal(y[0, 0, 3:6, 3:6], x[0, 0])
    assert np.all(y[0, 0, :3] == 0) and np.all(idx[0, 0, :3] == -1)


@pytest.mark.parametrize("mode,shape", [("pre_activation", (6, 3, 4, 5)), ("spatial", (6, 3, 4, 5)), ("pre_activation", (8, 1, 10))])
def test_batchnorm_matches_torch_autograd(mode, shape):
    x = RNG.randn(*shape) * 2 + 0.5
    dy = RNG.randn(*shape)
    xt = torch.tensor(x, requires_grad=True)
    if mode == "spatial":
        yt = Fn.batch_norm(xt, None, None, training=True, eps=ops.BN_EPS)
    else:
        flat = xt.reshape(shape[0], -1)
        yt = Fn.batch_norm(flat, None, None, training=True, eps=ops.BN_EPS).reshape(shape)
    np.testing.assert_allclose(ops.bn_fwd(x, mode)[0], yt.detach().numpy(), rtol=1e-9, atol=1e-12)
    yt.backward(torch.tensor(dy))
    np.testing.assert_allclose(ops.bn_bwd(x, dy, mode), xt.grad.numpy(), rtol=1e-8, atol=1e-11)


def test_softmax_and_cross_pieces_match_torch():
    x = RNG.randn(5, 1, 7)
    dy = RNG.randn(5, 1, 7)
    xt = torch.tensor(x, requires_grad=True)
    yt = torch.softmax(xt.reshape(5, -1), dim=1).reshape(x.shape)
    y = ops.softmax_instance(x)
    np.testing.assert_allclose(y, yt.detach().numpy(), rtol=1e-12)
    yt.backward(torch.tensor(dy))
    np.testing.assert_allclose(ops.softmax_instance_bwd(y, dy), xt.grad.numpy(), rtol=1e-10, atol=1e-14)
    p = np.abs(RNG.randn(4, 6)) + 0.1
    t = RNG.rand(4, 6)
    pt = torch.tensor(p, requires_grad=True)
    b = 1.0 / p.size
    lt = (-(torch.log(pt)) * torch.tensor(t) * b).sum()
    np.testing.assert_allclose(ops.cross(p, t, b).sum(), lt.item(), rtol=1e-12)
    lt.backward()
    np.testing.assert_allclose(ops.cross_backward(p, t, np.ones_like(p), b), pt.grad.numpy(), rtol=1e-12)


def test_dropout_mask_is_a_function_of_seed_and_index():
    x = np.ones(100000, np.float32)
    a, b = ops.dropout(x, 0.5, 3), ops.dropout(x, 0.5, 3)
    np.testing.assert_array_equal(a, b)
    keep = (a != 0).mean()
    assert abs(keep - 0.5) < 3 * np.sqrt(0.25 / x.size)
    assert set(np.unique(a)) == {0.0, 2.0}
    assert (ops.dropout(x, 0.5, 4) != a).any()


def test_reduce_and_broadcast_shapes():
    x = RNG.randn(4, 3, 2, 5)
    np.testing.assert_allclose(ops.reduce_sum(x, (4, 3, 2, 5), (1, 3, 1, 1)).reshape(-1), x.sum(axis=(0, 2, 3)))
    np.testing.assert_allclose(ops.reduce_sum(x.reshape(1, 4, 30), (1, 4, 30), (1, 1, 30)).reshape(-1), x.reshape(4, 30).sum(axis=0))
    b = RNG.randn(5)
    np.testing.assert_array_equal(ops.broadcast_tail(b, (3, 5)), np.broadcast_to(b, (3, 5)))
    c = RNG.randn(3)
    np.testing.assert_array_equal(ops.broadcast_channel(c, (2, 3, 4, 4))[1, :, 2, 3], c)


def test_small_resnet_style_graph_gradients_match_torch(lib_path):
    """conv -> per-activation BN -> relu -> pool -> flatten -> dense -> softmax -> cross: the mirror's
    gradient graph evaluated by the oracle equals torch autograd on the same network."""
    from tinyflow_b200 import autodiff as ad
    N, C, H, K, classes = 4, 3, 8, 5, 6
    X, y_ = ad.Placeholder("X"), ad.Placeholder("y_")
    W, Wd, bd = ad.Variable("W"), ad.Variable("Wd"), ad.Variable("bd")
    h = ad.convolution_2d_forward_op(X, W, "NCHW", "SAME", 1, 1)
    h = ad.activation_forward_op(ad.bn_forward_op(h, "NCHW", "pre_activation"), "NCHW", "relu")
    h = ad.pooling_2d_forward_op(h, "NCHW", "max", 0, 0, 2, 2, 2, 2)
    y = ad.fullyactivation_forward_op(ad.dense(ad.flatten_op(h), Wd, bd), "NCHW", "softmax")
    loss = ad.crossEntropy_loss(y, y_)
    params = [W, Wd, bd]
    grads = ad.gradients(loss, params)
    topo = ad.find_topo_sort([loss] + grads)
    xv, wv = RNG.randn(N, C, H, H), RNG.randn(K, C, 3, 3) * 0.3
    wdv, bdv = RNG.randn(K * 16, classes) * 0.2, RNG.randn(classes) * 0.1
    yv = np.eye(classes)[RNG.randint(0, classes, N)]
    vals = OracleExecutor(topo).run({X: xv, y_: yv, W: wv, Wd: wdv, bd: bdv})
    xt, wt = torch.tensor(xv), torch.tensor(wv, requires_grad=True)
    wdt, bdt = torch.tensor(wdv, requires_grad=True), torch.tensor(bdv, requires_grad=True)
    ht = Fn.conv2d(xt, wt, padding=1)
    ht = Fn.batch_norm(ht.reshape(N, -1), None, None, training=True, eps=ops.BN_EPS).reshape(ht.shape)
    ht = Fn.max_pool2d(torch.relu(ht), 2, 2)
    pt = torch.softmax(ht.reshape(N, -1) @ wdt + bdt, dim=1)
    lt = (-(torch.log(pt)) * torch.tensor(yv)).sum() / (N * classes)
    lt.backward()
    np.testing.assert_allclose(vals[loss][0], lt.item(), rtol=1e-10)
    for gnode, t in zip(grads, (wt, wdt, bdt)):
        np.testing.assert_allclose(vals[gnode], t.grad.numpy(), rtol=1e-7, atol=1e-11)


@pytest.mark.parametrize("case", [(2, 5, 9, 10, 4, 3, 3, "SAME", 1, 1), (2, 3, 11, 9, 6, 5, 3, "VALID", 2, 2),
                                  (3, 4, 8, 8, 5, 1, 7, "SAME", 1, 1), (2, 6, 10, 10, 4, 3, 3, "SAME", 2, 2)])
def test_sampled_convolution_oracle_equals_the_dense_one(case):
    """The coordinate-sampled convolution functions (used at benchmark sizes, where the dense oracle is too slow)
    give the dense oracle's values at those coordinates."""
    N, C, H, W, K, R, S, pad, sh, sw = case
    rng = np.random.RandomState(5)
    x, w = rng.randn(N, C, H, W), rng.randn(K, C, R, S)
    g = ops.conv_geometry(x.shape, w.shape, pad, sh, sw)
    dy = rng.randn(N, K, g["P"], g["Q"])
    T = 64
    n, k, c = rng.randint(0, N, T), rng.randint(0, K, T), rng.randint(0, C, T)
    p, q = rng.randint(0, g["P"], T), rng.randint(0, g["Q"], T)
    h, wi = rng.randint(0, H, T), rng.randint(0, W, T)
    r, s = rng.randint(0, R, T), rng.randint(0, S, T)
    np.testing.assert_allclose(ops.conv2d_fwd_at(x, w, g, n, k, p, q), ops.conv2d_fwd(x, w, g)[n, k, p, q], rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(ops.conv2d_dgrad_at(dy, w, g, n, c, h, wi), ops.conv2d_dgrad(dy, w, g)[n, c, h, wi], rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(ops.conv2d_wgrad_at(x, dy, g, k, c, r, s), ops.conv2d_wgrad(x, dy, g)[k, c, r, s], rtol=1e-12, atol=1e-12)


def test_3d_convolution_and_pooling_oracle_against_torch():
    """The 3-D restatements (cuDNN Nd descriptors in the reference, src/gpu_op.cu:2340-2530, 3029-3203) against torch-CPU
    float64, including the gradient of both pooling modes."""
    rng = np.random.RandomState(3)
    x, w = rng.randn(2, 3, 6, 7, 8), rng.randn(4, 3, 3, 3, 3)
    for pads, strides in [((1, 1, 1), (1, 1, 1)), ((0, 0, 0), (2, 1, 2)), ((1, 1, 1), (2, 2, 2))]:
        want = Fn.conv3d(torch.tensor(x), torch.tensor(w), stride=strides, padding=pads).numpy()
        np.testing.assert_allclose(ops.conv3d_fwd(x, w, pads, strides), want, rtol=1e-12, atol=1e-12)
    for mode in ("max", "mean"):
        for pads, strides, win in [((0, 0, 0), (2, 2, 2), (2, 2, 2)), ((1, 1, 1), (2, 2, 2), (3, 3, 3)), ((0, 1, 0), (1, 2, 1), (2, 3, 2))]:
            xt = torch.tensor(x, requires_grad=True)
            yt = Fn.max_pool3d(xt, win, strides, pads) if mode == "max" else Fn.avg_pool3d(xt, win, strides, pads, count_include_pad=True)
            y = ops.pool3d_fwd(x, mode, pads, strides, win)
            np.testing.assert_allclose(y, yt.detach().numpy(), rtol=1e-12, atol=1e-12)
            dy = rng.randn(*y.shape)
            yt.backward(torch.tensor(dy))
            np.testing.assert_allclose(ops.pool3d_bwd(x, dy, mode, pads, strides, win), xt.grad.numpy(), rtol=1e-12, atol=1e-12)

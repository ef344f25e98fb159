"""Per-layer parity at the real extents of the benchmark configurations, on real operands.

A training run of the benchmark graph (ResNet-50 and VGG-16 at batch 64, Inception-v3 at batch 32) is
advanced a few steps; then, for every distinct convolution shape of the graph, the three passes
(forward, backward-data, backward-filter) are recomputed on that layer's own activations, weights and
output gradient as the step left them:

* on the tensor-core path, in both arithmetic modes (3xFP16 and 3xTF32), asserting that the tensor
  path - not the CUDA-core kernel - took the call;
* on the exact-fp32 CUDA-core path.

Each result is judged against float64 dot products at a few thousand sampled output coordinates
(oracle.ops.conv2d_*_at) and, on every element, the tensor path against the CUDA-core path.
Errors are measured in units of fp32 roundoff (2^-24) of the dot product's own magnitude sum|a||b| - the
same pass evaluated on the operands' absolute values - which is the scale an fp32 accumulation (the
reference's cuDNN arithmetic) is accurate to, and has no floor tied to the tensor's largest value:

* samples:  |got - want| <= 1e-4 * |want| + 8 ulp for every path, and the tensor path's root-mean-square error in ulp
  may not exceed twice the fp32-FMA path's (plus a tenth of an ulp; the worst-of-2048 figures are recorded too, but the
  ratio of two maxima is too noisy to assert on);
* all elements:  |tensor - fp32| <= 2e-4 * |fp32| + 16 ulp.

Setting TINYFLOW_PARITY_TABLE=<file> dumps the per-layer figures as JSON.
"""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL, ULP = 1e-4, 2.0 ** -24


class _DeviceView:
    """Lets torch wrap an NDArray's device memory without a copy (element-wise comparisons stay on the GPU)."""

    def __init__(self, nd):
        self.__cuda_array_interface__ = {"shape": tuple(nd.shape), "typestr": "<f4", "data": (int(nd.data_ptr), False), "version": 2}


def _torch_view(nd):
    import torch
    return torch.as_tensor(_DeviceView(nd), device="cuda")


def _abs_copy(nd):
    """|nd| as a new device array."""
    from tinyflow_b200 import ndarray
    out = ndarray.empty(nd.shape, ndarray.gpu(0))
    _torch_view(out).copy_(_torch_view(nd).abs())
    return out


def _range_stats(t):
    """Fraction of the non-zero elements that lie more than 2^18 / 2^24 below the tensor's largest magnitude."""
    a = t.abs()
    amax = float(a.max())
    nz = a > 0
    n = max(int(nz.sum()), 1)
    return {"amax": amax, "zero_frac": 1.0 - n / a.numel(),
            "below_2^-18": float(((a < amax * 2.0 ** -18) & nz).sum()) / n,
            "below_2^-24": float(((a < amax * 2.0 ** -24) & nz).sum()) / n}


def _train(model_name, batch, image, steps):
    from tinyflow_b200 import autodiff as ad, models, ndarray
    model = models.BUILDERS[model_name](batch=batch, classes=1000, image=image)
    model.set_dropout(0.0)
    ex = ad.Executor(model.loss, model.y, 0.01, None, None, None, optimizer="sgd")
    ctx = ndarray.gpu(0)
    X, Y = models.synthetic_batch(model, seed=1234)
    feed = {n: ndarray.array(v, ctx) for n, v in model.init_params(seed=123).items()}
    Xd, Yd = ndarray.array(X, ctx), ndarray.array(Y, ctx)
    loss = None
    for _ in range(steps):
        feed[model.X], feed[model.y_] = Xd, Yd
        loss, feed = ex.run(feed)
    assert np.isfinite(loss.asnumpy()).all()
    return ex


def _conv_layers(ex):
    """One (forward node, backward-filter node) pair per distinct convolution geometry of the graph."""
    seen, out = set(), []
    bwd = {}
    for node in ex.topo_order:
        if type(node.op).__name__ == "Convolution2DBackwardOp" and node.type == 1:
            bwd[(node.inputs[0], node.inputs[1])] = node
    for node in ex.topo_order:
        if type(node.op).__name__ != "Convolution2DForwardOp":
            continue
        xs, ws = ex.node_to_shape_map[node.inputs[0]], ex.node_to_shape_map[node.inputs[1]]
        key = (xs, ws, node.padding, node.u, node.v)
        if key in seen:
            continue
        seen.add(key)
        out.append((node, bwd[(node.inputs[0], node.inputs[1])]))
    return out


def _check_layer(ex, fwd, bwd, rng, table, failures):
    from tinyflow_b200 import gpu_op, ndarray
    import oracle.ops as ops
    x, w, dy = ex.value_of(fwd.inputs[0]), ex.value_of(fwd.inputs[1]), ex.value_of(bwd.inputs[2])
    g = ops.conv_geometry(x.shape, w.shape, fwd.padding, fwd.u, fwd.v)
    out_shape, cell = gpu_op.convolution_2d_forward_get_out_shape(x.shape, w.shape, "NCHW", fwd.padding, fwd.u, fwd.v)
    assert tuple(out_shape) == tuple(dy.shape)
    ctx = ndarray.gpu(0)
    stream, cudnn = ex.cudaStream, ex.cudnnHandle
    has_dgrad = g["C"] >= 16          # the first layer's input gradient is never requested by the graphs
    name = "%dx%dx%dx%d k%d %dx%d %s s%d" % (g["N"], g["C"], g["H"], g["W"], g["K"], g["R"], g["S"], fwd.padding, fwd.u)

    def run(path, arith, operands):
        x, w, dy = operands
        y, dx, dw = ndarray.empty(out_shape, ctx), ndarray.empty(x.shape, ctx) if has_dgrad else None, ndarray.empty(w.shape, ctx)
        gpu_op.set_contraction_path(path)
        gpu_op.set_tensor_arithmetic(arith)
        try:
            assert gpu_op.convolution_2d_forward(x, w, y, cell, cudnn, stream) == 0
            assert gpu_op.last_contraction_path() == (2 if path == 2 else 1), name
            if has_dgrad:
                assert gpu_op.convolution_backward_data(x, dy, w, dx, cell, cudnn, stream) == 0
                assert gpu_op.last_contraction_path() == (2 if path == 2 else 1), name
            assert gpu_op.convolution_backward_filter(x, dy, w, dw, cell, cudnn, stream) == 0
            assert gpu_op.last_contraction_path() == (2 if path == 2 else 1), name
        finally:
            gpu_op.set_contraction_path(0)
            gpu_op.set_tensor_arithmetic("3xfp16")
        gpu_op.device_synchronize()
        return y, dx, dw

    import torch
    ref = run(1, "3xfp16", (x, w, dy))
    ax, aw, ady = _abs_copy(x), _abs_copy(w), _abs_copy(dy)
    torch.cuda.synchronize()
    mag = run(1, "3xfp16", (ax, aw, ady))           # sum |a||b| of every output element, per pass
    xh, wh, dyh = x.asnumpy(), w.asnumpy(), dy.asnumpy()
    axh, awh, adyh = np.abs(xh), np.abs(wh), np.abs(dyh)
    T = 2048
    n, k, c = rng.randint(0, g["N"], T), rng.randint(0, g["K"], T), rng.randint(0, g["C"], T)
    p, q = rng.randint(0, g["P"], T), rng.randint(0, g["Q"], T)
    h, wi = rng.randint(0, g["H"], T), rng.randint(0, g["W"], T)
    Tw = 96
    r, s = rng.randint(0, g["R"], Tw), rng.randint(0, g["S"], Tw)
    # per pass: (float64 values, their magnitudes, the coordinates)
    want = {"fwd": (ops.conv2d_fwd_at(xh, wh, g, n, k, p, q), ops.conv2d_fwd_at(axh, awh, g, n, k, p, q), (n, k, p, q)),
            "wgrad": (ops.conv2d_wgrad_at(xh, dyh, g, k[:Tw], c[:Tw], r, s), ops.conv2d_wgrad_at(axh, adyh, g, k[:Tw], c[:Tw], r, s), (k[:Tw], c[:Tw], r, s))}
    if has_dgrad:
        want["dgrad"] = (ops.conv2d_dgrad_at(dyh, wh, g, n, c, h, wi), ops.conv2d_dgrad_at(adyh, awh, g, n, c, h, wi), (n, c, h, wi))
    row = {"layer": name, "x": _range_stats(_torch_view(x)), "dy": _range_stats(_torch_view(dy)), "w": _range_stats(_torch_view(w))}
    order = {"fwd": 0, "dgrad": 1, "wgrad": 2}

    def sample_err(arr, ps):
        wv, mv, idx = want[ps]
        err = np.abs(arr.asnumpy()[idx].astype(np.float64) - wv)
        ok = bool(np.all(err <= REL * np.abs(wv) + 8 * ULP * mv))
        in_ulp = err / np.maximum(ULP * mv, 1e-300)
        return float(in_ulp.max()), ok, float(np.sqrt(np.mean(in_ulp ** 2)))

    for ps in want:
        row["fp32 " + ps], ok, row["fp32 %s rms" % ps] = sample_err(ref[order[ps]], ps)
        if not ok:
            failures.append("%s fp32 CUDA-core %s: %.2f ulp at the sampled coordinates" % (name, ps, row["fp32 " + ps]))
    for arith in ("3xfp16", "3xtf32"):
        got = run(2, arith, (x, w, dy))
        for ps in want:
            arr, ref_arr, mag_arr = got[order[ps]], ref[order[ps]], mag[order[ps]]
            e_ulp, ok, e_rms = sample_err(arr, ps)
            a, b, m = _torch_view(arr), _torch_view(ref_arr), _torch_view(mag_arr)
            diff = (a - b).abs()
            e_all = float((diff / (ULP * m).clamp_min(1e-300)).max())
            row["%s %s" % (arith, ps)] = e_ulp
            row["%s %s rms" % (arith, ps)] = e_rms
            row["%s %s vs fp32, all elements" % (arith, ps)] = e_all
            if not ok:
                failures.append("%s %s %s: %.2f ulp against float64 at the sampled coordinates" % (name, arith, ps, e_ulp))
            if e_rms > 2 * row["fp32 %s rms" % ps] + 0.1:
                failures.append("%s %s %s: rms error %.2f ulp vs %.2f ulp for fp32 FMA" % (name, arith, ps, e_rms, row["fp32 %s rms" % ps]))
            if not bool((diff <= 2 * REL * b.abs() + 16 * ULP * m).all()):
                failures.append("%s %s %s: %.2f ulp away from the fp32 CUDA-core result" % (name, arith, ps, e_all))
        del got
    table.append(row)
    torch.cuda.synchronize()


def _dump(table, tag):
    path = os.environ.get("TINYFLOW_PARITY_TABLE")
    if path:
        prev = json.load(open(path)) if os.path.exists(path) else {}
        prev[tag] = table
        json.dump(prev, open(path, "w"), indent=1)


@pytest.mark.parametrize("model_name,batch,image,steps", [("resnet50", 64, 224, 1), ("resnet50", 64, 224, 20), ("vgg16", 64, 224, 2),
                                                          ("inceptionv3", 32, 299, 2)])
def test_every_convolution_shape_at_benchmark_size_on_real_operands(lib_path, model_name, batch, image, steps):
    from tinyflow_b200 import gpu_op
    ex = _train(model_name, batch, image, steps)
    rng = np.random.RandomState(11)
    table, failures = [], []
    layers = _conv_layers(ex)
    assert len(layers) >= {"resnet50": 20, "vgg16": 9, "inceptionv3": 30}[model_name]
    try:
        for fwd, bwd in layers:
            _check_layer(ex, fwd, bwd, rng, table, failures)
    finally:
        _dump(table, "%s b%d after %d steps" % (model_name, batch, steps))
    gpu_op.device_synchronize()
    ex.values = {}
    gpu_op.release_cached_memory()
    assert not failures, "; ".join(failures[:20])

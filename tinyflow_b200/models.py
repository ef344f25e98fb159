"""Workload graphs for the five benchmark configurations, built with the mirrored ``ad`` API.

Each builder returns a :class:`Model` (placeholders, loss, prediction node, parameter shapes in
network order).  The graphs follow the reference's model scripts node for node:

* :func:`mlp`        tests/mnist_dlsys.py:177-194 (784-256-100-10, ReLU, softmax-cross-entropy)
* :func:`lenet5`     LeNet-5 with the layer sizes of the benchmark configuration, wired like the
                     reference's LeNet (tests/LeNet5/LeNet5_mnist_test.py:72-125: conv+bias, ReLU, max-pool)
* :func:`vgg16`      pycode/tinyflow/VGG16_test_leo.py:169-254
* :func:`resnet50`   pycode/tinyflow/ResNet50_test_leo.py:27-261
* :func:`inceptionv3` pycode/tinyflow/Inceptionv3_test_leo.py:558-1020
* :func:`densenet121` pycode/tinyflow/DenseNet_test_leo.py:13-127 (beyond the five configurations)

Initial values are synthetic: He-normal weights (std = sqrt(2 / fan_in)), zero biases, drawn from a
seeded ``numpy.random.RandomState``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from . import autodiff as ad


@dataclass
class Model:
    name: str
    X: object
    y_: object
    loss: object
    y: object
    param_shapes: dict = field(default_factory=dict)   # Variable node -> shape, network order
    input_shape: tuple = ()
    label_shape: tuple = ()
    dropout_nodes: list = field(default_factory=list)

    def init_params(self, seed=123, std=None):
        """He-normal weights / zero biases as float32 numpy arrays, keyed by Variable node."""
        rng = np.random.RandomState(seed)
        out = {}
        for node, shape in self.param_shapes.items():
            if len(shape) == 1:
                out[node] = np.zeros(shape, np.float32)
                continue
            fan_in = int(np.prod(shape[1:])) if len(shape) == 4 else shape[0]
            s = std if std is not None else np.sqrt(2.0 / fan_in)
            out[node] = rng.normal(0.0, s, size=shape).astype(np.float32)
        return out

    def set_dropout(self, rate):
        for n in self.dropout_nodes:
            n.dropout = rate


def mlp(batch=1000, sizes=(784, 256, 100, 10)):
    X, y_ = ad.Placeholder("X"), ad.Placeholder("y_")
    params, h = {}, X
    n_layers = len(sizes) - 1
    Ws = [ad.Variable("W%d" % (i + 1)) for i in range(n_layers)]
    bs = [ad.Variable("b%d" % (i + 1)) for i in range(n_layers)]
    for i in range(n_layers):
        z = ad.matmul_op(h, Ws[i])
        z = z + ad.broadcastto_op(bs[i], z)
        h = ad.relu_op(z) if i < n_layers - 1 else z
    loss = ad.softmaxcrossentropy_op(h, y_)
    for i in range(n_layers):
        params[Ws[i]] = (sizes[i], sizes[i + 1])
    for i in range(n_layers):
        params[bs[i]] = (sizes[i + 1],)
    return Model("mlp", X, y_, loss, h, params, (batch, sizes[0]), (batch, sizes[-1]))


def lenet5(batch=256, classes=10):
    X, y_ = ad.Placeholder("X"), ad.Placeholder("y_")
    W1, b1 = ad.Variable("W1"), ad.Variable("b1")
    W2, b2 = ad.Variable("W2"), ad.Variable("b2")
    W3, b3 = ad.Variable("W3"), ad.Variable("b3")
    W4, b4 = ad.Variable("W4"), ad.Variable("b4")
    W5, b5 = ad.Variable("W5"), ad.Variable("b5")
    c1 = ad.conv2withbias(X, W1, b1, "NCHW", "SAME", 1, 1)          # 1x28x28 -> 6x28x28
    a1 = ad.activation_forward_op(c1, "NCHW", "relu")
    p1 = ad.pooling_2d_forward_op(a1, "NCHW", "max", 0, 0, 2, 2, 2, 2)   # -> 6x14x14
    c2 = ad.conv2withbias(p1, W2, b2, "NCHW", "VALID", 1, 1)        # -> 16x10x10
    a2 = ad.activation_forward_op(c2, "NCHW", "relu")
    p2 = ad.pooling_2d_forward_op(a2, "NCHW", "max", 0, 0, 2, 2, 2, 2)   # -> 16x5x5
    f = ad.flatten_op(p2)
    d3 = ad.fullyactivation_forward_op(ad.dense(f, W3, b3), "NCHW", "relu")
    d4 = ad.fullyactivation_forward_op(ad.dense(d3, W4, b4), "NCHW", "relu")
    y = ad.dense(d4, W5, b5)
    loss = ad.softmaxcrossentropy_op(y, y_)
    params = {W1: (6, 1, 5, 5), b1: (6,), W2: (16, 6, 5, 5), b2: (16,), W3: (400, 120), b3: (120,),
              W4: (120, 84), b4: (84,), W5: (84, classes), b5: (classes,)}
    return Model("lenet5", X, y_, loss, y, params, (batch, 1, 28, 28), (batch, classes))


def _conv_relu(x, w, padding, sh, sw):
    return ad.activation_forward_op(ad.convolution_2d_forward_op(x, w, "NCHW", padding, sh, sw), "NCHW", "relu")


def vgg16(batch=64, classes=1000, image=224, dropout=0.5):
    X, y_ = ad.Placeholder("X"), ad.Placeholder("y_")
    cfg = [(64, 2), (128, 2), (256, 3), (512, 3), (512, 3)]
    params, h, cin = {}, X, 3
    conv_vars = []
    for bi, (cout, reps) in enumerate(cfg, start=1):
        for ri in range(1, reps + 1):
            conv_vars.append((ad.Variable("W%d_%d" % (bi, ri)), (cout, cin, 3, 3)))
            cin = cout
    W6, W7, W8 = ad.Variable("W6"), ad.Variable("W7"), ad.Variable("W8")
    b6, b7, b8 = ad.Variable("b6"), ad.Variable("b7"), ad.Variable("b8")
    it = iter(conv_vars)
    for cout, reps in cfg:
        for _ in range(reps):
            w, shape = next(it)
            params[w] = shape
            h = _conv_relu(h, w, "SAME", 1, 1)
        h = ad.pooling_2d_forward_op(h, "NCHW", "max", 0, 0, 2, 2, 2, 2)
    spatial = image // 32
    flat = ad.flatten_op(h)
    drops = []
    fc6 = ad.dense(flat, W6, b6)
    act6 = ad.fullyactivation_forward_op(fc6, "NCHW", "relu")
    drop6 = ad.fullydropout_forward_op(act6, "NCHW", dropout); drops.append(drop6)
    fc7 = ad.dense(drop6, W7, b7)
    act7 = ad.fullyactivation_forward_op(fc7, "NCHW", "relu")
    drop7 = ad.fullydropout_forward_op(act7, "NCHW", dropout); drops.append(drop7)
    fc8 = ad.dense(drop7, W8, b8)
    bn8 = ad.fullybn_forward_op(fc8, "NCHW")
    y = ad.fullyactivation_forward_op(bn8, "NCHW", "softmax")
    loss = ad.crossEntropy_loss(y, y_)
    params.update({W6: (512 * spatial * spatial, 4096), W7: (4096, 4096), W8: (4096, classes),
                   b6: (4096,), b7: (4096,), b8: (classes,)})
    return Model("vgg16", X, y_, loss, y, params, (batch, 3, image, image), (batch, classes), drops)


def _bottleneck(x, cin, filters, name, stride, projection, params):
    """Residual bottleneck (identity_block / convolutional_block, ResNet50_test_leo.py:27-111)."""
    f1, f2, f3 = filters
    W1, W2, W3 = ad.Variable(name + "W1"), ad.Variable(name + "W2"), ad.Variable(name + "W3")
    first_pad = "VALID" if projection else "SAME"
    h = ad.convolution_2d_forward_op(x, W1, "NCHW", first_pad, stride, stride)
    h = ad.activation_forward_op(ad.bn_forward_op(h, "NCHW", "pre_activation"), "NCHW", "relu")
    h = ad.convolution_2d_forward_op(h, W2, "NCHW", "SAME", 1, 1)
    h = ad.activation_forward_op(ad.bn_forward_op(h, "NCHW", "pre_activation"), "NCHW", "relu")
    h = ad.convolution_2d_forward_op(h, W3, "NCHW", "VALID", 1, 1)
    h = ad.bn_forward_op(h, "NCHW", "pre_activation")
    params[W1], params[W2], params[W3] = (f1, cin, 1, 1), (f2, f1, 3, 3), (f3, f2, 1, 1)
    if projection:
        Ws = ad.Variable(name + "W_shortcut")
        sc = ad.convolution_2d_forward_op(x, Ws, "NCHW", "VALID", stride, stride)
        sc = ad.bn_forward_op(sc, "NCHW", "pre_activation")
        params[Ws] = (f3, cin, 1, 1)
    else:
        sc = x
    return ad.activation_forward_op(ad.add_op(h, sc), "NCHW", "relu")


def resnet50(batch=64, classes=1000, image=224, dropout=0.5):
    X, y_ = ad.Placeholder("X"), ad.Placeholder("y_")
    W1, W6, b6, W7, b7 = ad.Variable("W1"), ad.Variable("W6"), ad.Variable("b6"), ad.Variable("W7"), ad.Variable("b7")
    params = {W1: (64, 3, 7, 7)}
    # the reference zero-pads with a 1x1 stride-1 max-pool that has padding 3 (ResNet50_test_leo.py:219)
    h = ad.pooling_2d_forward_op(X, "NCHW", "max", 3, 3, 1, 1, 1, 1)
    h = ad.convolution_2d_forward_op(h, W1, "NCHW", "VALID", 2, 2)
    h = ad.activation_forward_op(ad.bn_forward_op(h, "NCHW", "pre_activation"), "NCHW", "relu")
    h = ad.pooling_2d_forward_op(h, "NCHW", "max", 0, 0, 2, 2, 3, 3)
    cin = 64
    stages = [("2", [64, 64, 256], 3, 1), ("3", [128, 128, 512], 4, 2), ("4", [256, 256, 1024], 6, 2), ("5", [512, 512, 2048], 3, 2)]
    for sname, filters, blocks, stride in stages:
        for bi in range(blocks):
            name = "%s%s_" % (sname, "abcdef"[bi])
            h = _bottleneck(h, cin, filters, name, stride if bi == 0 else 1, bi == 0, params)
            cin = filters[2]
    final = image // 32
    h = ad.pooling_2d_forward_op(h, "NCHW", "mean", 0, 0, 1, 1, final, final)
    flat = ad.flatten_op(h)
    dense6 = ad.dense(flat, W6, b6)
    act6 = ad.fullyactivation_forward_op(dense6, "NCHW", "relu")
    drop6 = ad.fullydropout_forward_op(act6, "NCHW", dropout)
    dense7 = ad.dense(drop6, W7, b7)
    y = ad.fullyactivation_forward_op(dense7, "NCHW", "softmax")
    loss = ad.crossEntropy_loss(y, y_)
    params.update({W6: (2048, 2048), W7: (2048, classes), b6: (2048,), b7: (classes,)})
    return Model("resnet50", X, y_, loss, y, params, (batch, 3, image, image), (batch, classes), [drop6])


def inceptionv3(batch=32, classes=1000, image=299, dropout=0.8):
    """Inception-v3 without batch norm, wired like Inceptionv3_test_leo.py:558-1020 (conv+ReLU units, chained
    two-input channel concats, the 8x8 grid-reduction module reading the second 17x17 module's output)."""
    X, y_ = ad.Placeholder("X"), ad.Placeholder("y_")
    params = {}

    def unit(x, name, shape, padding="SAME", stride=1):
        w = ad.Variable(name)
        params[w] = shape
        return _conv_relu(x, w, padding, stride, stride)

    def cat(*xs):
        out = xs[0]
        for x in xs[1:]:
            out = ad.concat_forward_op(out, x)
        return out

    def avg3(x):
        return ad.pooling_2d_forward_op(x, "NCHW", "mean", 1, 1, 1, 1, 3, 3)

    # stem: 299 -> 35x35x192
    h = unit(X, "filterb_1", (32, 3, 3, 3), "VALID", 2)
    h = unit(h, "filterb_2", (32, 32, 3, 3), "VALID")
    h = unit(h, "filterb_3", (64, 32, 3, 3))
    h = ad.pooling_2d_forward_op(h, "NCHW", "max", 0, 0, 2, 2, 3, 3)
    h = unit(h, "filterb_4", (80, 64, 1, 1), "VALID")
    h = unit(h, "filterb_5", (192, 80, 3, 3), "VALID")
    h = ad.pooling_2d_forward_op(h, "NCHW", "max", 0, 0, 2, 2, 3, 3)

    # three 35x35 modules (1x1 | 1x1-5x5 | 1x1-3x3-3x3 | avgpool-1x1)
    cin = 192
    for i, proj in enumerate((32, 64, 64), start=1):
        f = "filter1_%d_" % i
        b0 = unit(h, f + "0", (64, cin, 1, 1))
        b1 = unit(unit(h, f + "1a", (48, cin, 1, 1)), f + "1b", (64, 48, 5, 5))
        b2 = unit(unit(unit(h, f + "2a", (64, cin, 1, 1)), f + "2b", (96, 64, 3, 3)), f + "2c", (96, 96, 3, 3))
        b3 = unit(avg3(h), f + ("3" if i == 3 else "3a"), (proj, cin, 1, 1))
        h = cat(b0, b1, b2, b3)
        cin = 64 + 64 + 96 + proj

    # grid reduction 35 -> 17
    b0 = unit(h, "filter2_1_0", (384, cin, 3, 3), "VALID", 2)
    b1 = unit(unit(unit(h, "filter2_1_1a", (64, cin, 1, 1)), "filter2_1_1b", (96, 64, 3, 3)), "filter2_1_1c", (96, 96, 3, 3), "VALID", 2)
    b2 = ad.pooling_2d_forward_op(h, "NCHW", "mean", 0, 0, 2, 2, 3, 3)
    h = cat(b0, b1, b2)
    cin = 384 + 96 + cin     # 768

    # four 17x17 modules with factorised 7x7 convolutions
    outs17 = []
    for i, mid in zip(range(2, 6), (128, 160, 160, 160)):
        f = "filter2_%d_" % i
        b0 = unit(h, f + "0", (192, cin, 1, 1))
        b1 = unit(h, f + "1a", (mid, cin, 1, 1))
        b1 = unit(b1, f + "1b", (mid, mid, 1, 7))
        b1 = unit(b1, f + "1c", (192, mid, 7, 1))
        b2 = unit(h, f + "2a", (mid, cin, 1, 1))
        b2 = unit(b2, f + "2b", (mid, mid, 7, 1))
        b2 = unit(b2, f + "2c", (mid, mid, 1, 7))
        b2 = unit(b2, f + "2d", (mid, mid, 7, 1))
        b2 = unit(b2, f + "2e", (192, mid, 1, 7))
        b3 = unit(avg3(h), f + "3a", (192, cin, 1, 1))
        h = cat(b0, b1, b2, b3)
        outs17.append(h)

    # grid reduction 17 -> 8; its second branch and its pooling branch read the output of the FIRST 17x17 module
    # (Inceptionv3_test_leo.py:893-898), which is kept here so that the node sequence matches.
    early = outs17[0]
    b0 = unit(unit(h, "filter3_1_0a", (192, cin, 1, 1)), "filter3_1_0b", (320, 192, 3, 3), "VALID", 2)
    b1 = unit(early, "filter3_1_1a", (192, cin, 1, 1))
    b1 = unit(b1, "filter3_1_1b", (192, 192, 1, 7))
    b1 = unit(b1, "filter3_1_1c", (192, 192, 7, 1))
    b1 = unit(b1, "filter3_1_1d", (192, 192, 3, 3), "VALID", 2)
    b2 = ad.pooling_2d_forward_op(early, "NCHW", "mean", 0, 0, 2, 2, 3, 3)
    h = cat(b0, b1, b2)
    cin = 320 + 192 + cin    # 1280

    # two 8x8 modules with split 1x3 / 3x1 branches
    for i in (2, 3):
        f = "filter3_%d_" % i
        b0 = unit(h, f + "0", (320, cin, 1, 1))
        b1a = unit(h, f + "1a", (384, cin, 1, 1))
        b1 = ad.concat_forward_op(unit(b1a, f + "1b", (384, 384, 1, 3)), unit(b1a, f + "1c", (384, 384, 3, 1)))
        b2b = unit(unit(h, f + "2a", (448, cin, 1, 1)), f + "2b", (384, 448, 3, 3))
        b2 = ad.concat_forward_op(unit(b2b, f + "2c", (384, 384, 1, 3)), unit(b2b, f + "2d", (384, 384, 3, 1)))
        b3 = unit(avg3(h), f + "3a", (192, cin, 1, 1))
        h = cat(b0, b1, b2, b3)
        cin = 320 + 768 + 768 + 192    # 2048

    final = (((image - 3) // 2 + 1 - 2 - 3) // 2 + 1 - 2 - 3) // 2 + 1     # 35 for 299
    final = ((final - 3) // 2 + 1 - 3) // 2 + 1                              # 8
    h = ad.pooling_2d_forward_op(h, "NCHW", "mean", 0, 0, 1, 1, final, final)
    drop = ad.dropout_forward_op(h, "NCHW", dropout)
    h = unit(drop, "filtera1", (classes, cin, 1, 1))
    W, b = ad.Variable("filtersmul"), ad.Variable("biases")
    dense = ad.dense(ad.squeeze_op(h), W, b)
    y = ad.fullyactivation_forward_op(dense, "NCHW", "softmax")
    loss = ad.crossEntropy_loss(y, y_)
    params[W], params[b] = (classes, classes), (classes,)
    return Model("inceptionv3", X, y_, loss, y, params, (batch, 3, image, image), (batch, classes), [drop])


def densenet121(batch=32, classes=1000, image=224, dropout=0.2, growth=32):
    """DenseNet-121 wired like DenseNet_test_leo.py:28-127: BN -> ReLU -> 1x1 conv -> dropout -> BN -> ReLU -> 3x3 conv ->
    dropout bottlenecks whose outputs are concatenated onto their inputs (6 / 12 / 24 / 16 per block), transition layers
    that halve channels (1x1 conv) and resolution (2x2 average pool), global average pool, one dense layer."""
    X, y_ = ad.Placeholder("X"), ad.Placeholder("y_")
    W0, W1, b1 = ad.Variable("W0"), ad.Variable("W1"), ad.Variable("b1")
    params = {W0: (2 * growth, 3, 7, 7)}
    tail = {}
    drops = []

    def bn_relu(x):
        return ad.activation_forward_op(ad.bn_forward_op(x, "NCHW", "pre_activation"), "NCHW", "relu")

    def drop(x):
        d = ad.dropout_forward_op(x, "NCHW", dropout)
        drops.append(d)
        return d

    def bottleneck(x, cin, name):
        Wa, Wb = ad.Variable(name + "_W1"), ad.Variable(name + "_W2")
        params[Wa], params[Wb] = (4 * growth, cin, 1, 1), (growth, 4 * growth, 3, 3)
        h = drop(ad.convolution_2d_forward_op(bn_relu(x), Wa, "NCHW", "SAME", 1, 1))
        return drop(ad.convolution_2d_forward_op(bn_relu(h), Wb, "NCHW", "SAME", 1, 1))

    def dense_block(x, cin, layers, name):
        for i in range(layers):
            x = ad.concat_forward_op(x, bottleneck(x, cin, "%s_bottleneck%d" % (name, i)))
            cin += growth
        return x, cin

    def transition(x, cin, name):
        Wt = ad.Variable(name + "_W1")
        params[Wt] = (cin // 2, cin, 1, 1)
        h = drop(ad.convolution_2d_forward_op(bn_relu(x), Wt, "NCHW", "SAME", 1, 1))
        return ad.pooling_2d_forward_op(h, "NCHW", "mean", 0, 0, 2, 2, 2, 2), cin // 2

    h = ad.convolution_2d_forward_op(X, W0, "NCHW", "SAME", 2, 2)
    h = ad.pooling_2d_forward_op(h, "NCHW", "max", 1, 1, 2, 2, 3, 3)
    cin = 2 * growth
    for bi, layers in enumerate((6, 12, 24, 16)):
        h, cin = dense_block(h, cin, layers, "dense%d" % (bi + 1))
        if bi < 3:
            h, cin = transition(h, cin, "trans%d" % (bi + 1))
    final = image // 32
    h = ad.pooling_2d_forward_op(bn_relu(h), "NCHW", "mean", 0, 0, 1, 1, final, final)
    y = ad.fullyactivation_forward_op(ad.dense(ad.flatten_op(h), W1, b1), "NCHW", "softmax")
    loss = ad.crossEntropy_loss(y, y_)
    # the reference feeds W0, W1, b1 first and the blocks' filters after them (DenseNet_test_leo.py:107-114)
    ordered = {W0: params.pop(W0), W1: (cin, classes), b1: (classes,)}
    ordered.update(params)
    return Model("densenet121", X, y_, loss, y, ordered, (batch, 3, image, image), (batch, classes), drops)


def inceptionv4(batch=32, classes=1000, image=299, dropout=0.8):
    """Inception-v4 without batch norm, wired like Inceptionv4_test_leo.py:28-340: conv+ReLU units, chained two-input
    channel concats; stem with two pooled/strided forks and a 7x1 / 1x7 fork, 4 A modules at 35x35x384, reduction to
    17x17x1024, 7 B modules, reduction to 8x8x1536, 3 C modules with split 1x3 / 3x1 ends, global average pool,
    squeeze, dropout, one dense layer."""
    X, y_ = ad.Placeholder("X"), ad.Placeholder("y_")
    params = {}

    def unit(x, name, shape, padding="SAME", stride=1):
        w = ad.Variable(name)
        params[w] = shape
        return _conv_relu(x, w, padding, stride, stride)

    def chain(x, prefix, specs):
        for suffix, shape in specs:
            x = unit(x, prefix + suffix, shape)
        return x

    def cat(*xs):
        out = xs[0]
        for x in xs[1:]:
            out = ad.concat_forward_op(out, x)
        return out

    def avg3(x):
        return ad.pooling_2d_forward_op(x, "NCHW", "mean", 1, 1, 1, 1, 3, 3)

    def pool_s2(x, mode):
        return ad.pooling_2d_forward_op(x, "NCHW", mode, 0, 0, 2, 2, 3, 3)

    # stem: 299 -> 35x35x384
    h = unit(X, "f1", (32, 3, 3, 3), "VALID", 2)
    h = unit(h, "f2", (32, 32, 3, 3), "VALID")
    h = unit(h, "f3", (64, 32, 3, 3))
    h = cat(pool_s2(h, "max"), unit(h, "f4", (96, 64, 3, 3), "VALID", 2))                     # 160 channels
    left = unit(unit(h, "f5_1", (64, 160, 1, 1)), "f5_2", (96, 64, 3, 3), "VALID")
    right = chain(h, "f6_", [("1", (64, 160, 1, 1)), ("2", (64, 64, 7, 1)), ("3", (64, 64, 1, 7))])
    right = unit(right, "f6_4", (96, 64, 3, 3), "VALID")
    h = cat(left, right)                                                                      # 192 channels
    strided = unit(h, "f7", (192, 192, 3, 3), "VALID", 2)
    h = cat(pool_s2(h, "max"), strided)                                                       # 384 channels
    W, b = ad.Variable("W"), ad.Variable("b")
    params[W], params[b] = (1536, classes), (classes,)

    def module_a(x, name):
        f = name + "filter1_1_"
        b0 = unit(x, f + "0", (96, 384, 1, 1))
        b1 = chain(x, f, [("1a", (64, 384, 1, 1)), ("1b", (96, 64, 3, 3))])
        b2 = chain(x, f, [("2a", (64, 384, 1, 1)), ("2b", (96, 64, 3, 3)), ("2c", (96, 96, 3, 3))])
        return cat(b0, b1, b2, unit(avg3(x), f + "3a", (96, 384, 1, 1)))

    def reduce_a(x, cin, name):
        f = name + "filter2_1_"
        b0 = unit(x, f + "0", (384, cin, 3, 3), "VALID", 2)
        b1 = chain(x, f, [("1a", (192, cin, 1, 1)), ("1b", (224, 192, 3, 3))])
        b1 = unit(b1, f + "1c", (256, 224, 3, 3), "VALID", 2)
        return cat(b0, b1, pool_s2(x, "mean"))

    def module_b(x, cin, name):
        f = name + "filter2_2_"
        b0 = unit(x, f + "0", (384, cin, 1, 1))
        b1 = chain(x, f, [("1a", (192, cin, 1, 1)), ("1b", (224, 192, 1, 7)), ("1c", (256, 224, 7, 1))])
        b2 = chain(x, f, [("2a", (192, cin, 1, 1)), ("2b", (192, 192, 7, 1)), ("2c", (224, 192, 1, 7)),
                          ("2d", (224, 224, 7, 1)), ("2e", (256, 224, 1, 7))])
        return cat(b0, b1, b2, unit(avg3(x), f + "3a", (128, cin, 1, 1)))

    def reduce_b(x, cin, name):
        f = name + "filter3_1_"
        b0 = unit(unit(x, f + "0a", (192, cin, 1, 1)), f + "0b", (192, 192, 3, 3), "VALID", 2)
        b1 = chain(x, f, [("1a", (256, cin, 1, 1)), ("1b", (256, 256, 1, 7)), ("1c", (320, 256, 7, 1))])
        b1 = unit(b1, f + "1d", (320, 320, 3, 3), "VALID", 2)
        return cat(b0, b1, pool_s2(x, "mean"))

    def module_c(x, cin, name):
        f = name + "filter3_2_"
        b0 = unit(x, f + "0", (256, cin, 1, 1))
        b1a = unit(x, f + "1a", (384, cin, 1, 1))
        b1 = ad.concat_forward_op(unit(b1a, f + "1b", (256, 384, 1, 3)), unit(b1a, f + "1c", (256, 384, 3, 1)))
        b2c = chain(x, f, [("2a", (384, cin, 1, 1)), ("2b", (448, 384, 1, 3)), ("2c", (512, 448, 3, 1))])
        b2 = ad.concat_forward_op(unit(b2c, f + "2d", (256, 512, 3, 1)), unit(b2c, f + "2e", (256, 512, 1, 3)))
        return cat(b0, b1, b2, unit(avg3(x), f + "3a", (256, cin, 1, 1)))

    for i in range(1, 5):
        h = module_a(h, "a%d" % i)
    h = reduce_a(h, 384, "ra")
    for i in range(1, 8):
        h = module_b(h, 1024, "b%d" % i)
    h = reduce_b(h, 1024, "rb")
    for i in range(1, 4):
        h = module_c(h, 1536, "c%d" % i)

    side = (image - 3) // 2 + 1 - 2          # 147 for 299
    side = (side - 3) // 2 + 1 - 2           # 71
    for _ in range(3):
        side = (side - 3) // 2 + 1           # 35, 17, 8
    h = ad.pooling_2d_forward_op(h, "NCHW", "mean", 0, 0, 1, 1, side, side)
    drop = ad.fullydropout_forward_op(ad.squeeze_op(h), "NCHW", dropout)
    y = ad.fullyactivation_forward_op(ad.dense(drop, W, b), "NCHW", "softmax")
    loss = ad.crossEntropy_loss(y, y_)
    return Model("inceptionv4", X, y_, loss, y, params, (batch, 3, image, image), (batch, classes), [drop])


BUILDERS = {"mlp": mlp, "lenet5": lenet5, "vgg16": vgg16, "resnet50": resnet50, "inceptionv3": inceptionv3, "densenet121": densenet121,
            "inceptionv4": inceptionv4}


def synthetic_batch(model: Model, seed=1234, rank=0, input_dist="normal"):
    """Seeded synthetic inputs of the model's shapes: X ~ N(0,1) or U[0,1), uniformly drawn one-hot labels."""
    rng = np.random.RandomState(seed + rank)
    if input_dist == "uniform":
        X = rng.uniform(0.0, 1.0, size=model.input_shape).astype(np.float32)
    else:
        X = rng.normal(0.0, 1.0, size=model.input_shape).astype(np.float32)
    labels = rng.randint(0, model.label_shape[1], size=model.label_shape[0])
    y = np.zeros(model.label_shape, np.float32)
    y[np.arange(model.label_shape[0]), labels] = 1.0
    return X, y

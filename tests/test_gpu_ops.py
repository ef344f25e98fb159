"""Per-operator parity: every CUDA entry point, called through the C-ABI wrappers, against the
CPU oracle (float64) on the same seeded inputs.  Tolerances for floating point:

* dense contractions (matmul, the three convolution passes): per element
  |got - want| <= 1e-4 * |want| + 8 * 2^-24 * sum_i |a_i| |b_i|, i.e. relative 1e-4, or eight units of
  fp32 roundoff of the dot product's own magnitude where the terms cancel (an fp32 accumulation - the
  reference's cuBLAS / cuDNN arithmetic - lands 2.5 to 4 such units from the exact value on the worst of a
  few million elements, see the exact-fp32 CUDA-core path in these tests; there is no floor tied to the
  tensor's largest value), plus ||got - want||_2 <= 5e-5 * ||want||_2;
* everything else: |got - want| <= 1e-4 * max(|want|, 1e-2 * max|want|) (the floor is 16 units of fp32
  roundoff of the tensor's largest element: outputs that are differences of O(max) quantities);
* indices and masks bit-exact."""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RNG = np.random.RandomState(42)


ULP = 2.0 ** -24          # unit roundoff of fp32


def close_dot(got, want, mag, rel=1e-4, ulps=8.0, what=""):
    """Parity of a dense contraction: `mag` is the same contraction evaluated on the absolute values of the operands."""
    want, got, mag = np.asarray(want, np.float64), np.asarray(got, np.float64), np.asarray(mag, np.float64)
    assert got.shape == want.shape == mag.shape, (what, got.shape, want.shape)
    assert np.all(np.isfinite(got)), what
    excess = np.abs(got - want) - (rel * np.abs(want) + ulps * ULP * mag)
    assert excess.max() <= 0, "%s: |err| %.3e at %s (want %.3e, magnitude %.3e, %.2f ulp of it)" % (
        what, np.abs(got - want).flat[excess.argmax()], np.unravel_index(excess.argmax(), excess.shape), want.flat[excess.argmax()],
        mag.flat[excess.argmax()], np.abs(got - want).flat[excess.argmax()] / max(ULP * mag.flat[excess.argmax()], 1e-300))
    l2 = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
    assert l2 <= 5e-5, "%s: relative L2 error %.3e" % (what, l2)


def close(got, want, rel=1e-4, floor=1e-2, what=""):
    want = np.asarray(want, dtype=np.float64)
    got = np.asarray(got, dtype=np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    scale = np.maximum(np.abs(want), floor * (np.abs(want).max() if want.size else 1.0))
    err = np.abs(got - want) / np.maximum(scale, 1e-30)
    assert np.all(np.isfinite(got)), what
    assert err.max() <= rel if err.size else True, "%s: max rel err %.3e at %s" % (what, err.max(), np.unravel_index(err.argmax(), err.shape))
    if want.size > 1:
        l2 = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
        assert l2 <= 5e-5 or rel > 1e-4, "%s: relative L2 error %.3e" % (what, l2)


@pytest.fixture(scope="module")
def env(lib_path):
    from tinyflow_b200 import gpu_op, ndarray
    import oracle.ops as ops

    class Env:
        pass
    e = Env()
    e.gpu_op, e.nd, e.ops = gpu_op, ndarray, ops
    e.ctx = ndarray.gpu(0)
    e.stream = gpu_op.create_cudaStream()
    e.cudnn = gpu_op.create_cudnnHandle(e.stream)
    e.cublas = gpu_op.create_cublasHandle(e.stream)
    e.dev = lambda a: ndarray.array(np.asarray(a, dtype=np.float32), e.ctx)
    e.empty = lambda s: ndarray.empty(s, e.ctx)
    return e


def f32(*shape, scale=1.0):
    return (RNG.randn(*shape) * scale).astype(np.float32)


# ---- runtime -----------------------------------------------------------------------------------
def test_alloc_copy_roundtrip_and_block_reuse(env):
    a = f32(37, 5)
    d = env.dev(a)
    np.testing.assert_array_equal(d.asnumpy(), a)
    ptr = d.data_ptr
    del d
    d2 = env.empty((37, 5))
    assert d2.data_ptr == ptr          # same size comes back from the pool
    h = env.nd.array(a, env.nd.cpu(0))  # pinned host array
    d3 = h.copyto(env.ctx, env.stream)
    np.testing.assert_array_equal(d3.asnumpy(), a)
    back = d3.copyto(env.nd.cpu(0), env.stream)
    np.testing.assert_array_equal(back.asnumpy(), a)


def test_soft_out_of_memory_protocol(env):
    """A failed device allocation returns the missing byte count instead of an array (c_runtime_api.cc:109-114)."""
    res = env.nd.empty((1 << 20, 1 << 20), env.ctx)       # 4 TiB
    assert isinstance(res, int) and res > 0
    ok = env.empty((4, 4))
    assert isinstance(ok, env.nd.NDArray)


def test_array_set_and_scalars(env):
    d = env.empty((13, 7))
    env.gpu_op.array_set(d, 2.5, env.stream)
    np.testing.assert_array_equal(d.asnumpy(), np.full((13, 7), 2.5, np.float32))
    a = f32(1001)
    o = env.empty((1001,))
    env.gpu_op.matrix_elementwise_add_by_const(env.dev(a), 1.25, o, env.stream)
    np.testing.assert_array_equal(o.asnumpy(), a + np.float32(1.25))
    env.gpu_op.matrix_elementwise_multiply_by_const(env.dev(a), -3.0, o, env.stream)
    np.testing.assert_array_equal(o.asnumpy(), a * np.float32(-3.0))


@pytest.mark.parametrize("n", [1, 3, 4, 1023, 4096, 100003])
def test_elementwise_binary(env, n):
    a, b = f32(n), f32(n)
    o = env.empty((n,))
    env.gpu_op.matrix_elementwise_add(env.dev(a), env.dev(b), o, env.stream)
    np.testing.assert_array_equal(o.asnumpy(), a + b)
    env.gpu_op.matrix_elementwise_multiply(env.dev(a), env.dev(b), o, env.stream)
    np.testing.assert_array_equal(o.asnumpy(), a * b)
    env.gpu_op.relu(env.dev(a), o)
    np.testing.assert_array_equal(o.asnumpy(), np.maximum(a, 0))
    env.gpu_op.relu_gradient(env.dev(a), env.dev(b), o)
    np.testing.assert_array_equal(o.asnumpy(), np.where(a > 0, b, 0))


def test_add_in_place_aliasing(env):
    a, b = f32(777), f32(777)
    da = env.dev(a)
    env.gpu_op.matrix_elementwise_add(da, env.dev(b), da, env.stream)
    np.testing.assert_array_equal(da.asnumpy(), a + b)


def test_broadcast(env):
    b = f32(100)
    o = env.empty((64, 100))
    env.gpu_op.broadcast_to(env.dev(b), o, "NHWC", env.stream)
    np.testing.assert_array_equal(o.asnumpy(), np.broadcast_to(b, (64, 100)))
    one = f32(1)
    env.gpu_op.broadcast_to(env.dev(one), o, "NHWC", env.stream)
    np.testing.assert_array_equal(o.asnumpy(), np.full((64, 100), one[0]))
    c = f32(6)
    o4 = env.empty((5, 6, 7, 3))
    env.gpu_op.broadcast_to(env.dev(c), o4, "NCHW", env.stream)
    np.testing.assert_array_equal(o4.asnumpy(), env.ops.broadcast_channel(c, (5, 6, 7, 3)))


@pytest.mark.parametrize("shape,out", [((64, 4096), (4096,)), ((1000, 10), (10,)), ((64, 1000), (1,)), ((7, 33), (33,)), ((4096, 3), (3,))])
def test_reduce_sum_bias_and_scalar(env, shape, out):
    x = f32(*shape)
    ins, outs = env.gpu_op.reduce_sum_get_real_shape(shape, out, "NHWC")
    cell = env.gpu_op.reduce_sum_get_cudnnlist(ins, outs, "NHWC", env.cudnn)
    o = env.empty(out)
    assert env.gpu_op.reduce_sum_new(env.dev(x), o, cell, env.cudnn, env.stream) == 0
    want = env.ops.reduce_sum(x.astype(np.float64), ins, outs).reshape(out)
    close(o.asnumpy(), want, what="reduce_sum %s" % (shape,))


def test_reduce_sum_channel(env):
    x = f32(6, 5, 7, 9)
    ins, outs = env.gpu_op.reduce_sum_get_real_shape(x.shape, (5,), "NCHW")
    cell = env.gpu_op.reduce_sum_get_cudnnlist(ins, outs, "NCHW", env.cudnn)
    o = env.empty((5,))
    env.gpu_op.reduce_sum_new(env.dev(x), o, cell, env.cudnn, env.stream)
    close(o.asnumpy(), x.astype(np.float64).sum(axis=(0, 2, 3)), what="channel reduce")


def test_legacy_reductions(env):
    x = f32(50, 70)
    o = env.empty((70,))
    env.gpu_op.reduce_sum_axis_zero(env.dev(x), o)
    close(o.asnumpy(), x.astype(np.float64).sum(axis=0))
    x3 = f32(4, 6, 5)
    o2 = env.empty((4, 5))
    env.gpu_op.reduce_sum(env.dev(x3), o2, axis=1)
    close(o2.asnumpy(), x3.astype(np.float64).sum(axis=1))
    o3 = env.empty((1,))
    env.gpu_op.reduce_sum(env.dev(x3), o3, axis=-1)
    close(o3.asnumpy(), [x3.astype(np.float64).sum()])
    back = env.empty((4, 6, 5))
    env.gpu_op.reduce_sum_backward(o2, back, 1)
    np.testing.assert_array_equal(back.asnumpy(), np.repeat(o2.asnumpy()[:, None, :], 6, axis=1))


# ---- matmul: the three shapes the reference asserts (tests/test_gpu_op.py:103-131) plus odd ones ------------
MATMUL = [(500, 700, 1000, False, False), (1000, 500, 2000, False, True), (1000, 500, 2000, True, True),
          (1000, 784, 256, False, False), (784, 1000, 256, True, False), (1000, 10, 100, False, True),
          (64, 2048, 2048, False, False), (64, 2048, 1000, True, False), (3, 5, 7, False, False), (129, 65, 33, True, True),
          (300, 512, 192, False, True), (257, 320, 160, True, True), (512, 256, 288, False, True)]


@pytest.mark.parametrize("M,K,N,tA,tB", MATMUL)
@pytest.mark.parametrize("path", [0, 1])
def test_matmul(env, M, K, N, tA, tB, path):
    A = f32(*((K, M) if tA else (M, K)))
    B = f32(*((N, K) if tB else (K, N)))
    C = env.empty((M, N))
    env.gpu_op.set_contraction_path(path)
    try:
        env.gpu_op.matrix_multiply(env.dev(A), tA, env.dev(B), tB, C, env.cublas, env.stream)
    finally:
        env.gpu_op.set_contraction_path(0)
    a64, b64 = A.astype(np.float64), B.astype(np.float64)
    a64, b64 = (a64.T if tA else a64), (b64.T if tB else b64)
    close_dot(C.asnumpy(), a64 @ b64, np.abs(a64) @ np.abs(b64), what="matmul %s" % ((M, K, N, tA, tB),))


# ---- scaling of the fp16 hi/lo split ------------------------------------------------------------------------------
@pytest.mark.parametrize("sa,sb", [(1.0, 1.0), (1e-20, 1e15), (3e18, 2e-30), (7e-12, 5e-9)])
def test_matmul_tensor_path_is_scale_invariant(env, sa, sb):
    """The tensor path rescales each operand by a power of two taken from its largest magnitude, so operands far
    outside the fp16 range must give the same relative accuracy as O(1) ones."""
    M, K, N = 256, 512, 192
    A, B = (f32(M, K) * sa).astype(np.float32), (f32(K, N) * sb).astype(np.float32)
    C = env.empty((M, N))
    env.gpu_op.set_contraction_path(2)
    try:
        env.gpu_op.matrix_multiply(env.dev(A), False, env.dev(B), False, C, env.cublas, env.stream)
    finally:
        env.gpu_op.set_contraction_path(0)
    a64, b64 = A.astype(np.float64), B.astype(np.float64)
    close_dot(C.asnumpy(), a64 @ b64, np.abs(a64) @ np.abs(b64), what="matmul scaled %g %g" % (sa, sb))


def test_matmul_tensor_path_wide_dynamic_range(env):
    """Magnitudes spread over 2^-10 .. 2^10 inside one operand: every element still carries 22 bits."""
    M, K, N = 192, 1024, 256
    A = (f32(M, K) * np.exp2(RNG.uniform(-10, 10, (M, K)))).astype(np.float32)
    B = (f32(K, N) * np.exp2(RNG.uniform(-10, 10, (K, N)))).astype(np.float32)
    C = env.empty((M, N))
    env.gpu_op.set_contraction_path(2)
    try:
        env.gpu_op.matrix_multiply(env.dev(A), False, env.dev(B), False, C, env.cublas, env.stream)
    finally:
        env.gpu_op.set_contraction_path(0)
    a64, b64 = A.astype(np.float64), B.astype(np.float64)
    close_dot(C.asnumpy(), a64 @ b64, np.abs(a64) @ np.abs(b64), what="matmul dynamic range")


def test_all_zero_operand_gives_zero(env):
    A, B = np.zeros((128, 256), np.float32), f32(256, 128)
    C = env.empty((128, 128))
    env.gpu_op.set_contraction_path(2)
    try:
        env.gpu_op.matrix_multiply(env.dev(A), False, env.dev(B), False, C, env.cublas, env.stream)
    finally:
        env.gpu_op.set_contraction_path(0)
    assert not C.asnumpy().any()


def test_tracked_maximum_is_dropped_when_the_tensor_is_overwritten(env):
    """ReLU records max|y| for its output while it writes it.  Overwriting that array by a host upload with values
    10^6 times larger must invalidate the recorded maximum: a stale one would overflow the fp16 split."""
    N, C, H, W, K = 4, 32, 20, 20, 32
    x_small = np.abs(f32(N, C, H, W)) * 1e-3
    w = f32(K, C, 3, 3, scale=0.2)
    g = env.ops.conv_geometry(x_small.shape, w.shape, "SAME", 1, 1)
    out_shape, cell = env.gpu_op.convolution_2d_forward_get_out_shape(x_small.shape, w.shape, "NCHW", "SAME", 1, 1)
    act = env.empty(x_small.shape)
    y = env.empty(out_shape)
    env.gpu_op.relu(env.dev(x_small), act)                      # tracked producer
    wd = env.dev(w)
    env.gpu_op.set_contraction_path(2)
    try:
        assert env.gpu_op.convolution_2d_forward(act, wd, y, cell, env.cudnn, env.stream) == 0
        xs64, w64 = x_small.astype(np.float64), w.astype(np.float64)
        close_dot(y.asnumpy(), env.ops.conv2d_fwd(xs64, w64, g), env.ops.conv2d_fwd(np.abs(xs64), np.abs(w64), g), what="conv on relu output")
        x_big = f32(N, C, H, W) * 1e3
        act._sync_copyfrom(x_big)
        assert env.gpu_op.convolution_2d_forward(act, wd, y, cell, env.cudnn, env.stream) == 0
        xb64 = x_big.astype(np.float64)
        close_dot(y.asnumpy(), env.ops.conv2d_fwd(xb64, w64, g), env.ops.conv2d_fwd(np.abs(xb64), np.abs(w64), g), what="conv after overwrite")
    finally:
        env.gpu_op.set_contraction_path(0)


# ---- softmax family ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("rows,cols", [(1000, 10), (64, 1000), (3, 1), (257, 33)])
def test_softmax_and_cross_entropy(env, rows, cols):
    x = f32(rows, cols, scale=3.0)
    t = np.eye(cols, dtype=np.float32)[RNG.randint(0, cols, rows)]
    o = env.empty((rows, cols))
    env.gpu_op.softmax(env.dev(x), o, env.stream)
    close(o.asnumpy(), env.ops.softmax_rows(x.astype(np.float64)), what="softmax")
    l = env.empty((1,))
    env.gpu_op.softmax_cross_entropy(env.dev(x), env.dev(t), l, env.stream)
    close(l.asnumpy(), env.ops.softmax_cross_entropy(x.astype(np.float64), t.astype(np.float64)), what="softmax-CE")


def test_activation_modes(env):
    for shape in [(8, 1, 1000), (4, 3, 5, 7)]:
        x, dy = f32(*shape), f32(*shape)
        x64, dy64 = x.astype(np.float64), dy.astype(np.float64)
        for mode, fwd, bwd in [("relu", env.ops.relu, lambda y: env.ops.relu_grad(x64, dy64)),
                               ("sigmoid", env.ops.sigmoid, lambda y: dy64 * y * (1 - y)),
                               ("tanh", np.tanh, lambda y: dy64 * (1 - y * y)),
                               ("softmax", env.ops.softmax_instance, lambda y: env.ops.softmax_instance_bwd(y, dy64))]:
            cell = env.gpu_op.activation_get_cudnnlist(shape, "NCHW", mode)
            y, dx = env.empty(shape), env.empty(shape)
            dxd = env.dev(x)
            env.gpu_op.activation_forward(dxd, y, mode, cell, env.cudnn, env.stream)
            want_y = fwd(x64)
            close(y.asnumpy(), want_y, what="act fwd " + mode)
            env.gpu_op.activation_backward(dxd, dx, y, env.dev(dy), mode, cell, env.cudnn, env.stream)
            close(dx.asnumpy(), bwd(want_y), what="act bwd " + mode)


def test_relu_propagates_nan(env):
    x = np.array([np.nan, -1.0, 2.0, 0.0] * 3, np.float32)
    cell = env.gpu_op.activation_get_cudnnlist(x.shape, "NCHW", "relu") if False else None
    o = env.empty(x.shape)
    env.gpu_op.relu(env.dev(x), o)
    got = o.asnumpy()
    assert np.isnan(got[0]) and got[1] == 0 and got[2] == 2 and got[3] == 0


def test_cross_and_cross_backward(env):
    p = (np.abs(RNG.randn(64, 1000)) + 0.05).astype(np.float32)
    t = np.eye(1000, dtype=np.float32)[RNG.randint(0, 1000, 64)]
    d = f32(64, 1000)
    b = 1.0 / p.size
    o = env.empty(p.shape)
    env.gpu_op.cross(env.dev(p), env.dev(t), o, b, env.stream)
    close(o.asnumpy(), env.ops.cross(p.astype(np.float64), t, b), floor=1e-6, what="cross")
    env.gpu_op.cross_backward(env.dev(p), env.dev(t), env.dev(d), o, b, env.stream)
    close(o.asnumpy(), env.ops.cross_backward(p.astype(np.float64), t, d.astype(np.float64), b), floor=1e-6, what="cross bwd")


def test_concat_forward_and_split(env):
    a, b = f32(4, 5, 6, 7), f32(4, 9, 6, 7)
    o = env.empty((4, 14, 6, 7))
    env.gpu_op.concat_forward(env.dev(a), env.dev(b), o, env.stream)
    np.testing.assert_array_equal(o.asnumpy(), np.concatenate([a, b], axis=1))
    da, db = env.empty(a.shape), env.empty(b.shape)
    env.gpu_op.concat_a_backward(env.dev(a), env.dev(b), o, da, env.stream)
    env.gpu_op.concat_b_backward(env.dev(a), env.dev(b), o, db, env.stream)
    np.testing.assert_array_equal(da.asnumpy(), a)
    np.testing.assert_array_equal(db.asnumpy(), b)


# ---- convolution ---------------------------------------------------------------------------------------------
CONV = [
    # N, C, H, W, K, R, S, padding, sh, sw
    (2, 3, 9, 9, 4, 3, 3, "SAME", 1, 1),
    (3, 8, 15, 15, 16, 1, 1, "VALID", 1, 1),
    (2, 16, 14, 14, 32, 1, 1, "VALID", 2, 2),
    (2, 3, 29, 29, 8, 7, 7, "VALID", 2, 2),
    (4, 1, 28, 28, 6, 5, 5, "SAME", 1, 1),
    (4, 6, 14, 14, 16, 5, 5, "VALID", 1, 1),
    (2, 12, 17, 17, 20, 1, 7, "SAME", 1, 1),
    (2, 12, 17, 17, 20, 7, 1, "SAME", 1, 1),
    (2, 10, 13, 13, 12, 3, 3, "VALID", 2, 2),
    (2, 64, 55, 55, 64, 3, 3, "SAME", 1, 1),
    (2, 64, 55, 55, 256, 1, 1, "VALID", 1, 1),
    (2, 256, 55, 55, 128, 1, 1, "VALID", 2, 2),
    (2, 128, 28, 28, 128, 3, 3, "SAME", 1, 1),
    (4, 512, 7, 7, 512, 3, 3, "SAME", 1, 1),
    (4, 512, 7, 7, 2048, 1, 1, "VALID", 1, 1),
    (3, 96, 14, 14, 160, 3, 3, "SAME", 1, 1),
    (2, 40, 9, 9, 72, 1, 1, "SAME", 1, 1),
    # stride-1 windows without padding (frame wider than the input on both sides of dy)
    (2, 32, 37, 37, 32, 3, 3, "VALID", 1, 1),
    (2, 80, 21, 21, 192, 3, 3, "VALID", 1, 1),
    # few input channels: several taps share one tile of the filter-gradient GEMM
    (2, 16, 28, 28, 64, 3, 3, "SAME", 1, 1),
    (2, 48, 35, 35, 64, 5, 5, "SAME", 1, 1),
    # output widths that take the 96-column tile
    (2, 128, 17, 17, 160, 1, 7, "SAME", 1, 1),
    (2, 64, 17, 17, 192, 1, 1, "VALID", 1, 1),
    (2, 192, 9, 9, 288, 3, 3, "SAME", 1, 1),
    # strided windows: one frame per stride phase
    (2, 32, 35, 35, 64, 3, 3, "VALID", 2, 2),
    (2, 96, 17, 17, 96, 3, 3, "VALID", 2, 2),
    (2, 64, 16, 16, 32, 3, 3, "SAME", 2, 2),
    (2, 288, 15, 15, 128, 3, 3, "VALID", 2, 2),
    (2, 32, 23, 23, 32, 5, 5, "SAME", 3, 3),
    (2, 64, 20, 18, 64, 1, 3, "SAME", 2, 2),
    # three input channels: patch-matrix path
    (4, 3, 64, 64, 64, 7, 7, "VALID", 2, 2),
    (16, 3, 75, 75, 32, 3, 3, "VALID", 2, 2),
]


@pytest.mark.parametrize("case", CONV)
@pytest.mark.parametrize("path", [0, 1])
def test_conv_forward_backward(env, case, path):
    N, C, H, W, K, R, S, padding, sh, sw = case
    x, w = f32(N, C, H, W), f32(K, C, R, S, scale=0.2)
    g = env.ops.conv_geometry(x.shape, w.shape, padding, sh, sw)
    out_shape, cell = env.gpu_op.convolution_2d_forward_get_out_shape(x.shape, w.shape, "NCHW", padding, sh, sw)
    assert out_shape == (N, K, g["P"], g["Q"])
    dy = f32(*out_shape)
    dx_, dw_, dy_ = env.dev(x), env.dev(w), env.dev(dy)
    y, dx, dw = env.empty(out_shape), env.empty(x.shape), env.empty(w.shape)
    env.gpu_op.set_contraction_path(path)
    try:
        assert env.gpu_op.convolution_2d_forward(dx_, dw_, y, cell, env.cudnn, env.stream) == 0
        assert env.gpu_op.convolution_backward_data(dx_, dy_, dw_, dx, cell, env.cudnn, env.stream) == 0
        assert env.gpu_op.convolution_backward_filter(dx_, dy_, dw_, dw, cell, env.cudnn, env.stream) == 0
    finally:
        env.gpu_op.set_contraction_path(0)
    x64, w64, dy64 = x.astype(np.float64), w.astype(np.float64), dy.astype(np.float64)
    ax, aw, ady = np.abs(x64), np.abs(w64), np.abs(dy64)
    close_dot(y.asnumpy(), env.ops.conv2d_fwd(x64, w64, g), env.ops.conv2d_fwd(ax, aw, g), what="conv fwd %s" % (case,))
    close_dot(dx.asnumpy(), env.ops.conv2d_dgrad(dy64, w64, g), env.ops.conv2d_dgrad(ady, aw, g), what="conv dgrad %s" % (case,))
    close_dot(dw.asnumpy(), env.ops.conv2d_wgrad(x64, dy64, g), env.ops.conv2d_wgrad(ax, ady, g), what="conv wgrad %s" % (case,))


# ---- pooling ---------------------------------------------------------------------------------------------------
POOL = [(2, 3, 8, 8, 0, 0, 2, 2, 2, 2), (2, 4, 112, 112, 0, 0, 2, 2, 3, 3), (2, 3, 24, 24, 3, 3, 1, 1, 1, 1),
        (3, 5, 7, 7, 0, 0, 1, 1, 7, 7), (2, 6, 17, 17, 1, 1, 1, 1, 3, 3), (2, 6, 17, 17, 0, 0, 2, 2, 3, 3), (1, 2, 8, 8, 0, 0, 1, 1, 8, 8),
        (2, 5, 147, 147, 0, 0, 2, 2, 3, 3), (2, 3, 9, 11, 0, 0, 2, 2, 2, 2), (2, 2, 14, 14, 0, 0, 2, 2, 2, 2), (1, 3, 7, 8, 0, 0, 2, 2, 2, 2), (3, 2, 20, 13, 0, 0, 2, 2, 3, 3), (2, 3, 9, 10, 0, 0, 2, 2, 3, 3)]


@pytest.mark.parametrize("case", POOL)
@pytest.mark.parametrize("mode", ["max", "mean"])
def test_pooling(env, case, mode):
    N, C, H, W, ph, pw, sh, sw, kh, kw = case
    x = f32(N, C, H, W)
    if mode == "max":
        x[0, 0, :4, :4] = 0.0        # a block of ties
    g = env.ops.pool_geometry(x.shape, ph, pw, sh, sw, kh, kw)
    out_shape, cell = env.gpu_op.pooling_2d_forward_get_out_shape(x.shape, "NCHW", mode, ph, pw, sh, sw, kh, kw)
    assert out_shape == (N, C, g["P"], g["Q"])
    dy = f32(*out_shape)
    xd, y, dx = env.dev(x), env.empty(out_shape), env.empty(x.shape)
    env.gpu_op.pooling_2d_forward(xd, y, cell, env.cudnn, env.stream)
    env.gpu_op.pooling_2d_backward(xd, y, env.dev(dy), dx, cell, env.cudnn, env.stream)
    if mode == "max":
        want_y, want_idx = env.ops.maxpool_fwd(x, g)
        np.testing.assert_array_equal(y.asnumpy(), want_y)        # a selection: exact
        from tinyflow_b200._base import _LIB
        idx_buf = env.empty(out_shape)                           # 4-byte elements: reuse as an int32 buffer
        _LIB.TfPoolingArgmax(xd.handle, ctypes.c_void_p(idx_buf.data_ptr), cell, env.stream)
        got_idx = idx_buf.asnumpy().view(np.int32)
        np.testing.assert_array_equal(got_idx, want_idx)         # indices bit-exact
        close(dx.asnumpy(), env.ops.maxpool_bwd(x.astype(np.float64), dy.astype(np.float64), g), what="maxpool bwd")
    else:
        close(y.asnumpy(), env.ops.avgpool_fwd(x.astype(np.float64), g), what="avgpool fwd")
        close(dx.asnumpy(), env.ops.avgpool_bwd(dy.astype(np.float64), g), what="avgpool bwd")


# ---- batch normalisation ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape,mode", [((64, 8, 7, 9), "pre_activation"), ((5, 3, 4, 4), "pre_activation"), ((32, 6, 5, 5), "pre_activation"),
                                         ((100, 2, 3, 3), "pre_activation"), ((64, 1, 1000), "pre_activation"), ((8, 5, 6, 7), "spatial"),
                                         ((64, 3, 55, 55), "pre_activation")])
def test_batchnorm(env, shape, mode):
    x, dy = f32(*shape, scale=2.0) + np.float32(0.7), f32(*shape)
    mean_p, var_p, cell = env.gpu_op.bn_get_cudnnlist(shape, "NCHW", mode)
    xd, y, dx = env.dev(x), env.empty(shape), env.empty(shape)
    assert env.gpu_op.bn_forward(xd, y, mode, 0, mean_p, var_p, cell, env.cudnn, env.stream) == 0
    assert env.gpu_op.bn_backward(xd, env.dev(dy), dx, mode, mean_p, var_p, cell, env.cudnn, env.stream) == 0
    x64 = x.astype(np.float64)
    close(y.asnumpy(), env.ops.bn_fwd(x64, mode)[0], what="bn fwd")
    close(dx.asnumpy(), env.ops.bn_bwd(x64, dy.astype(np.float64), mode), what="bn bwd")


@pytest.mark.parametrize("shape", [(64, 16, 28, 28), (32, 24, 17, 17), (8, 64, 56, 56)])
@pytest.mark.parametrize("mask_is_bn_output", [True, False])
def test_relu_backward_runs_inside_the_batchnorm_backward_that_follows(env, shape, mask_is_bn_output):
    """DLGpuActivationBackward(relu) is held back for one call; when DLGpuBatchNormalizationBackward on its output comes
    next, one kernel writes both gradients.  Both must be bit-identical to the two kernels run one after the other
    (a synchronising call in between launches the held-back kernel on its own), and within tolerance of the oracle.  The
    ReLU's mask comes from x-hat when its input is this layer's own forward output, else from the tensor itself."""
    from tinyflow_b200._base import _LIB
    x, dy = f32(*shape, scale=2.0) + np.float32(0.3), f32(*shape)
    mean_p, var_p, cell = env.gpu_op.bn_get_cudnnlist(shape, "NCHW", "pre_activation")
    xd, dyd = env.dev(x), env.dev(dy)
    y = env.empty(shape)
    assert env.gpu_op.bn_forward(xd, y, "pre_activation", 0, mean_p, var_p, cell, env.cudnn, env.stream) == 0
    if mask_is_bn_output:
        relu_in = y
    else:                                   # a residual sum in between: the ReLU reads another tensor
        relu_in = env.empty(shape)
        env.gpu_op.matrix_elementwise_add(y, env.dev(f32(*shape)), relu_in, env.stream)
    relu_out = env.empty(shape)
    act = env.gpu_op.activation_get_cudnnlist(shape, "NCHW", "relu") if hasattr(env.gpu_op, "activation_get_cudnnlist") else None
    env.gpu_op.activation_forward(relu_in, relu_out, "relu", act, env.cudnn, env.stream)
    results = []
    for fused in (True, False):
        d_relu, d_bn = env.empty(shape), env.empty(shape)
        before = env.gpu_op.fused_relu_bn_backward_count()
        env.gpu_op.activation_backward(relu_in, d_relu, relu_out, dyd, "relu", act, env.cudnn, env.stream)
        if not fused:
            assert _LIB.TfDeviceSynchronize() == 0          # any other call launches the held-back kernel
        assert env.gpu_op.bn_backward(xd, d_relu, d_bn, "pre_activation", mean_p, var_p, cell, env.cudnn, env.stream) == 0
        assert env.gpu_op.fused_relu_bn_backward_count() - before == (1 if fused else 0)
        results.append((d_relu.asnumpy(), d_bn.asnumpy()))
    np.testing.assert_array_equal(results[0][0], results[1][0])
    np.testing.assert_array_equal(results[0][1], results[1][1])
    mask_src = relu_in.asnumpy()
    want_relu = np.where(mask_src > 0, dy, 0).astype(np.float32)
    np.testing.assert_array_equal(results[0][0], want_relu)
    close(results[0][1], env.ops.bn_bwd(x.astype(np.float64), want_relu.astype(np.float64), "pre_activation"), what="fused bn bwd")


@pytest.mark.parametrize("shape", [(64, 32, 28, 28), (7, 33, 19, 17)])
def test_a_sum_is_computed_by_the_relu_forward_that_follows(env, shape):
    """DLGpuMatrixElementwiseAdd is held back for one call; when the ReLU forward of the sum comes next (the end of a
    residual block) one kernel writes the sum and its ReLU.  Both outputs are exact, the fusion is counted, and a
    synchronising call in between (or an in-place ReLU) gives the same bits through the two plain kernels."""
    from tinyflow_b200._base import _LIB
    a, b = f32(*shape), f32(*shape)
    act = env.gpu_op.activation_get_cudnnlist(shape, "NCHW", "relu")
    ad, bd = env.dev(a), env.dev(b)
    for fused in (True, False):
        ssum, r = env.empty(shape), env.empty(shape)
        before = env.gpu_op.fused_add_relu_count()
        env.gpu_op.matrix_elementwise_add(ad, bd, ssum, env.stream)
        if not fused:
            assert _LIB.TfDeviceSynchronize() == 0
        env.gpu_op.activation_forward(ssum, r, "relu", act, env.cudnn, env.stream)
        assert env.gpu_op.fused_add_relu_count() - before == (1 if fused else 0)
        np.testing.assert_array_equal(ssum.asnumpy(), a + b)
        np.testing.assert_array_equal(r.asnumpy(), np.maximum(a + b, 0))
    # the ReLU overwrites the sum in place: not fused, still right
    ssum = env.empty(shape)
    env.gpu_op.matrix_elementwise_add(ad, bd, ssum, env.stream)
    env.gpu_op.activation_forward(ssum, ssum, "relu", act, env.cudnn, env.stream)
    np.testing.assert_array_equal(ssum.asnumpy(), np.maximum(a + b, 0))
    # a held-back sum is visible to a reader that is not a ReLU
    ssum, twice = env.empty(shape), env.empty(shape)
    env.gpu_op.matrix_elementwise_add(ad, bd, ssum, env.stream)
    env.gpu_op.matrix_elementwise_multiply(ssum, ssum, twice, env.stream)
    np.testing.assert_array_equal(twice.asnumpy(), (a + b) * (a + b))


def test_a_held_back_relu_backward_is_visible_to_every_other_reader(env):
    """The held-back kernel must have run before anything else can look: a copy to the host right after the call, a free
    of its operand, an unrelated operator on another tensor."""
    shape = (16, 32, 28, 28)
    x, dy = f32(*shape), f32(*shape)
    want = np.where(x > 0, dy, 0).astype(np.float32)
    act = env.gpu_op.activation_get_cudnnlist(shape, "NCHW", "relu") if hasattr(env.gpu_op, "activation_get_cudnnlist") else None
    xd, out = env.dev(x), env.empty(shape)
    # (a) read straight back
    dx, dyd = env.empty(shape), env.dev(dy)
    env.gpu_op.activation_backward(xd, dx, out, dyd, "relu", act, env.cudnn, env.stream)
    np.testing.assert_array_equal(dx.asnumpy(), want)
    # (b) the gradient operand is freed before anything else happens
    dx, dyd = env.empty(shape), env.dev(dy)
    env.gpu_op.activation_backward(xd, dx, out, dyd, "relu", act, env.cudnn, env.stream)
    del dyd
    other = env.dev(f32(*shape))
    np.testing.assert_array_equal(dx.asnumpy(), want)
    # (c) an unrelated operator overwrites the gradient operand in place right after
    dx, dyd = env.empty(shape), env.dev(dy)
    env.gpu_op.activation_backward(xd, dx, out, dyd, "relu", act, env.cudnn, env.stream)
    env.gpu_op.matrix_elementwise_add(other, other, dyd, env.stream)
    np.testing.assert_array_equal(dx.asnumpy(), want)


# ---- dropout: the mask is bit-exact against the oracle's counter-based generator ------------------------------------
@pytest.mark.parametrize("p", [0.0, 0.5, 0.3])
def test_dropout_mask_consistency(env, p):
    shape = (64, 1, 4096)
    x, dy = f32(*shape), f32(*shape)
    inputd = env.gpu_op.get_input_descriptor(shape, "NCHW")
    y, dx = env.empty(shape), env.empty(shape)
    reserve, cell, short = env.gpu_op.dropout_forward(env.dev(x), y, "NCHW", p, 17, inputd, env.cudnn, env.stream)
    assert short == 0
    env.gpu_op.dropout_backward(env.dev(dy), dx, reserve, cell, env.cudnn, env.stream)
    want = env.ops.dropout(x, p, 17)
    np.testing.assert_array_equal(y.asnumpy() != 0, want != 0)      # same mask
    close(y.asnumpy(), want, rel=1e-5)
    close(dx.asnumpy(), env.ops.dropout(dy, p, 17), rel=1e-5)          # backward reuses the forward mask
    if p > 0:
        keep = (y.asnumpy() != 0).mean()
        assert abs(keep - (1 - p)) < 4 * np.sqrt(p * (1 - p) / x.size)


# ---- optimisers -------------------------------------------------------------------------------------------------------
def test_sgd_and_adam(env):
    w, g = f32(1000, 33), f32(1000, 33)
    wd = env.dev(w)
    env.gpu_op.sgd_update(wd, env.dev(g), 0.1, env.stream)
    close(wd.asnumpy(), env.ops.sgd(w.astype(np.float64), g.astype(np.float64), np.float32(0.1)), rel=1e-5)
    m, v = np.abs(f32(1000, 33)) * 0.1, np.abs(f32(1000, 33)) * 0.01
    wd, md, vd = env.dev(w), env.dev(m), env.dev(v)
    env.gpu_op.adam_mv(md, vd, env.dev(g), 0.9, 0.999, env.stream)
    env.gpu_op.adam_compute(wd, md, vd, 0.9, 0.999, 1e-8, 0.001, env.stream)
    w2, m2, v2 = env.ops.adam(w.astype(np.float64), m.astype(np.float64), v.astype(np.float64), g.astype(np.float64),
                              np.float32(0.9), np.float32(0.999), np.float32(0.9), np.float32(0.999), np.float32(1e-8), np.float32(0.001))
    close(md.asnumpy(), m2, rel=1e-5)
    close(vd.asnumpy(), v2, rel=1e-5)
    close(wd.asnumpy(), w2, rel=1e-5)


def test_multi_tensor_sgd_matches_per_tensor_updates(env):
    shapes = [(17,), (33, 5), (1000,), (3, 3, 3, 3)]
    ws, gs = [f32(*s) for s in shapes], [f32(*s) for s in shapes]
    wd, gd = [env.dev(a) for a in ws], [env.dev(a) for a in gs]
    sizes = [a.size for a in ws]
    prefix = np.concatenate([[0], np.cumsum(sizes)]).astype(int).tolist()
    n2 = env.gpu_op.get_n2_cuda_pointer([a.data_ptr for a in wd], [a.data_ptr for a in gd], len(ws))
    info = env.gpu_op.get_index_to_VaribaleNumber_cuda_pointer([0] * len(ws), prefix, len(ws))
    env.gpu_op.sgd_compute_o(n2, info, len(ws), 0.05)
    for a, w, g in zip(wd, ws, gs):
        close(a.asnumpy(), w - np.float32(0.05) * g, rel=1e-5)


def test_multi_tensor_adam_matches_the_oracle(env):
    """DLGpuAdam_o over a four-column pointer table (src/gpu_op.cu:4674, 4865): moments and parameters of every tensor."""
    shapes = [(17,), (33, 5), (1000,), (3, 3, 3, 3)]
    ws, gs = [f32(*s) for s in shapes], [f32(*s) for s in shapes]
    ms, vs = [np.abs(f32(*s)) * 0.1 for s in shapes], [np.abs(f32(*s)) * 0.01 for s in shapes]
    wd, gd, md, vd = ([env.dev(a) for a in arrs] for arrs in (ws, gs, ms, vs))
    prefix = np.concatenate([[0], np.cumsum([a.size for a in ws])]).astype(int).tolist()
    n4 = env.gpu_op.get_n4_cuda_pointer([a.data_ptr for a in wd], [a.data_ptr for a in md], [a.data_ptr for a in vd], [a.data_ptr for a in gd], len(ws))
    info = env.gpu_op.get_index_to_VaribaleNumber_cuda_pointer([0] * len(ws), prefix, len(ws))
    b1, b2, b1t, b2t, e, lr = 0.9, 0.999, 0.9 ** 3, 0.999 ** 3, 1e-8, 0.001
    env.gpu_op.adam_compute_o(n4, info, len(ws), b1, b2, b1t, b2t, e, lr)
    for k in range(len(ws)):
        w2, m2, v2 = env.ops.adam(ws[k].astype(np.float64), ms[k].astype(np.float64), vs[k].astype(np.float64), gs[k].astype(np.float64),
                                  np.float32(b1), np.float32(b2), np.float32(b1t), np.float32(b2t), np.float32(e), np.float32(lr))
        close(md[k].asnumpy(), m2, rel=1e-5)
        close(vd[k].asnumpy(), v2, rel=1e-5)
        close(wd[k].asnumpy(), w2, rel=1e-5)


def test_multi_tensor_update_invalidates_packed_filters(env):
    """A convolution after DLGpuSgd_o must see the new weights: the tensor path keeps packed copies of its filters keyed
    by (pointer, write version), and the multi-tensor update writes the parameters through a pointer table."""
    N, C, H, W, K = 4, 32, 20, 20, 32
    x, w, gw = f32(N, C, H, W), f32(K, C, 3, 3, scale=0.2), f32(K, C, 3, 3)
    g = env.ops.conv_geometry(x.shape, w.shape, "SAME", 1, 1)
    out_shape, cell = env.gpu_op.convolution_2d_forward_get_out_shape(x.shape, w.shape, "NCHW", "SAME", 1, 1)
    xd, wd, gd, y = env.dev(x), env.dev(w), env.dev(gw), env.empty(out_shape)
    n2 = env.gpu_op.get_n2_cuda_pointer([wd.data_ptr], [gd.data_ptr], 1)
    info = env.gpu_op.get_index_to_VaribaleNumber_cuda_pointer([0], [0, w.size], 1)
    env.gpu_op.set_contraction_path(2)
    try:
        assert env.gpu_op.convolution_2d_forward(xd, wd, y, cell, env.cudnn, env.stream) == 0
        env.gpu_op.sgd_compute_o(n2, info, 1, 0.5)
        assert env.gpu_op.convolution_2d_forward(xd, wd, y, cell, env.cudnn, env.stream) == 0
        got_tensor = y.asnumpy()
        env.gpu_op.set_contraction_path(1)
        assert env.gpu_op.convolution_2d_forward(xd, wd, y, cell, env.cudnn, env.stream) == 0
        got_cuda_core = y.asnumpy()
    finally:
        env.gpu_op.set_contraction_path(0)
    x64, w2 = x.astype(np.float64), (w - np.float32(0.5) * gw).astype(np.float64)
    want, mag = env.ops.conv2d_fwd(x64, w2, g), env.ops.conv2d_fwd(np.abs(x64), np.abs(w2), g)
    close_dot(got_tensor, want, mag, what="conv after multi-tensor SGD (tensor path)")
    close_dot(got_cuda_core, want, mag, what="conv after multi-tensor SGD (CUDA-core path)")


# ---- losses, regularisers and the remaining elementwise entry points ----------------------------------------------
def test_losses_regularisers_and_their_gradients(env):
    a, b = f32(37, 21), f32(37, 21)
    g = np.array([0.7], np.float32)
    a64, b64, g64 = a.astype(np.float64), b.astype(np.float64), g.astype(np.float64)
    ad, bd, gd = env.dev(a), env.dev(b), env.dev(g)
    o1, oa = env.empty((1,)), env.empty(a.shape)
    for fn, want in [(lambda: env.gpu_op.L1loss(ad, bd, o1), env.ops.l1_loss(a64, b64)), (lambda: env.gpu_op.L2loss(ad, bd, o1), env.ops.l2_loss(a64, b64)),
                     (lambda: env.gpu_op.L1regular(ad, o1), env.ops.l1_regular(a64)), (lambda: env.gpu_op.L2regular(ad, o1), env.ops.l2_regular(a64))]:
        fn()
        close(o1.asnumpy(), want, rel=1e-5)
    for fn, want in [(lambda: env.gpu_op.l1loss_gradient(ad, bd, gd, oa), env.ops.l1_loss_grad(a64, b64, g64)),
                     (lambda: env.gpu_op.l2loss_gradient(ad, bd, gd, oa), env.ops.l2_loss_grad(a64, b64, g64)),
                     (lambda: env.gpu_op.l1regular_gradient(ad, gd, oa), env.ops.l1_regular_grad(a64, g64)),
                     (lambda: env.gpu_op.l2regular_gradient(ad, gd, oa), env.ops.l2_regular_grad(a64, g64))]:
        fn()
        close(oa.asnumpy(), want, rel=1e-5)


def test_cross_entropy_terms_and_unary_maps(env):
    p = RNG.uniform(0.05, 0.95, (64, 10)).astype(np.float32)
    t = np.eye(10, dtype=np.float32)[RNG.randint(0, 10, 64)]
    o = env.empty(p.shape)
    env.gpu_op.cross_entropy(env.dev(p), env.dev(t), o)
    close(o.asnumpy(), env.ops.binary_cross_entropy_terms(p.astype(np.float64), t.astype(np.float64)), rel=1e-5)
    x = (np.abs(f32(1000, 7)) + 0.1).astype(np.float32)
    o = env.empty(x.shape)
    x64, xd = x.astype(np.float64), env.dev(x)
    env.gpu_op.matrix_exp(xd, o)
    close(o.asnumpy(), np.exp(x64), rel=1e-5)
    env.gpu_op.matrix_log(xd, o, env.stream)
    close(o.asnumpy(), np.log(x64), rel=1e-5)
    env.gpu_op.matrix_reverse(xd, o)
    close(o.asnumpy(), 1.0 / x64, rel=1e-6)
    env.gpu_op.matrix_pow(xd, 2.5, o)
    close(o.asnumpy(), x64 ** 2.5, rel=1e-5)


def test_broadcast_backward(env):
    d = f32(64, 100)
    o = env.empty((100,))
    env.gpu_op.broadcast_to_backward(env.dev(d), o, "NHWC")
    close(o.asnumpy(), d.astype(np.float64).sum(axis=0))
    o1 = env.empty((1,))
    env.gpu_op.broadcast_to_backward(env.dev(d), o1, "NHWC")
    close(o1.asnumpy(), [d.astype(np.float64).sum()])
    d4 = f32(5, 6, 7, 3)
    oc = env.empty((6,))
    env.gpu_op.broadcast_to_backward(env.dev(d4), oc, "NCHW")
    close(oc.asnumpy(), d4.astype(np.float64).sum(axis=(0, 2, 3)))


def test_host_link_probe_runs(env, capfd):
    """testPcie (src/gpu_op.cu:4960): the host-link bandwidth probe prints four positive figures."""
    assert env.gpu_op.testPcie() in (0, None)
    out = capfd.readouterr().out
    import re
    nums = [float(v) for v in re.findall(r"(\d+\.\d+)", out)]
    assert len(nums) >= 4 and all(v > 0.1 for v in nums[:4]), out


# ---- 1-D and 3-D convolution (forward) and pooling --------------------------------------------------------------------
@pytest.mark.parametrize("case", [(4, 8, 50, 16, 5, "SAME", 1), (3, 64, 400, 96, 7, "VALID", 2), (64, 128, 512, 128, 3, "SAME", 1)])
def test_conv1d_forward(env, case):
    """A 1-D convolution is the 2-D one on (N, C, 1, W) (the reference hands cuDNN exactly that, src/gpu_op.cu:1535-1606);
    the last case is large enough for the tensor cores."""
    N, C, W, K, S, padding, v = case
    x, w = f32(N, C, W), f32(K, C, S, scale=0.2)
    out_shape, cell = env.gpu_op.convolution_1d_forward_get_out_shape(x.shape, w.shape, "NCHW", padding, v)
    g = env.ops.conv_geometry((N, C, 1, W), (K, C, 1, S), padding, 1, v)
    assert out_shape == (N, K, g["Q"])
    y = env.empty(out_shape)
    assert env.gpu_op.convolution_1d_forward(env.dev(x), env.dev(w), y, cell, env.cudnn) == 0
    x4, w4 = x.astype(np.float64).reshape(N, C, 1, W), w.astype(np.float64).reshape(K, C, 1, S)
    close_dot(y.asnumpy().reshape(N, K, 1, g["Q"]), env.ops.conv2d_fwd(x4, w4, g), env.ops.conv2d_fwd(np.abs(x4), np.abs(w4), g), what="conv1d %s" % (case,))


@pytest.mark.parametrize("mode", ["max", "mean"])
def test_pool1d_forward_backward(env, mode):
    N, C, W, pad, v, k = 3, 5, 37, 1, 2, 3
    x = f32(N, C, W)
    out_shape, cell = env.gpu_op.pooling_1d_forward_get_out_shape(x.shape, "NCHW", mode, pad, v, k)
    g = env.ops.pool_geometry((N, C, 1, W), 0, pad, 1, v, 1, k)
    assert out_shape == (N, C, g["Q"])
    dy = f32(*out_shape)
    xd, y, dx = env.dev(x), env.empty(out_shape), env.empty(x.shape)
    env.gpu_op.pooling_1d_forward(xd, y, cell, env.cudnn)
    env.gpu_op.pooling_1d_backward(xd, y, env.dev(dy), dx, cell, env.cudnn)
    x4, dy4 = x.astype(np.float64).reshape(N, C, 1, W), dy.astype(np.float64).reshape(N, C, 1, -1)
    if mode == "max":
        np.testing.assert_array_equal(y.asnumpy().reshape(N, C, 1, -1), env.ops.maxpool_fwd(x.reshape(N, C, 1, W), g)[0])
        close(dx.asnumpy().reshape(N, C, 1, W), env.ops.maxpool_bwd(x4, dy4, g), what="maxpool1d bwd")
    else:
        close(y.asnumpy().reshape(N, C, 1, -1), env.ops.avgpool_fwd(x4, g), what="avgpool1d fwd")
        close(dx.asnumpy().reshape(N, C, 1, W), env.ops.avgpool_bwd(dy4, g), what="avgpool1d bwd")


@pytest.mark.parametrize("case", [(2, 3, 6, 7, 8, 4, 3, 3, 3, "SAME", (1, 1, 1)), (2, 8, 9, 10, 11, 12, 3, 2, 3, "VALID", (2, 1, 2)), (1, 16, 8, 12, 12, 24, 3, 3, 3, "SAME", (1, 2, 2))])
def test_conv3d_forward(env, case):
    N, C, D, H, W, K, T, R, S, padding, strides = case
    x, w = f32(N, C, D, H, W), f32(K, C, T, R, S, scale=0.2)
    pads = (T // 2, R // 2, S // 2) if padding == "SAME" else (0, 0, 0)
    out_shape, cell = env.gpu_op.convolution_3d_forward_get_out_shape(x.shape, w.shape, "NCHW", padding, *strides)
    x64, w64 = x.astype(np.float64), w.astype(np.float64)
    want = env.ops.conv3d_fwd(x64, w64, pads, strides)
    assert out_shape == want.shape
    y = env.empty(out_shape)
    assert env.gpu_op.convolution_3d_forward(env.dev(x), env.dev(w), y, cell, env.cudnn) == 0
    close_dot(y.asnumpy(), want, env.ops.conv3d_fwd(np.abs(x64), np.abs(w64), pads, strides), what="conv3d %s" % (case,))


@pytest.mark.parametrize("mode", ["max", "mean"])
@pytest.mark.parametrize("geom", [((0, 0, 0), (2, 2, 2), (2, 2, 2)), ((1, 1, 1), (2, 2, 2), (3, 3, 3)), ((0, 1, 0), (1, 2, 1), (2, 3, 2))])
def test_pool3d_forward_backward(env, mode, geom):
    pads, strides, win = geom
    x = f32(2, 3, 6, 7, 8)
    if mode == "max":
        x[0, 0, :3, :3, :3] = 0.0            # a block of ties: the first maximum of a window takes the gradient
    out_shape, cell = env.gpu_op.pooling_3d_forward_get_out_shape(x.shape, "NCHW", mode, *pads, *strides, *win)
    want_y = env.ops.pool3d_fwd(x.astype(np.float64), mode, pads, strides, win)
    assert out_shape == want_y.shape
    dy = f32(*out_shape)
    xd, y, dx = env.dev(x), env.empty(out_shape), env.empty(x.shape)
    env.gpu_op.pooling_3d_forward(xd, y, cell, env.cudnn)
    env.gpu_op.pooling_3d_backward(xd, y, env.dev(dy), dx, cell, env.cudnn)
    if mode == "max":
        np.testing.assert_array_equal(y.asnumpy(), want_y.astype(np.float32))        # a selection: exact
    else:
        close(y.asnumpy(), want_y, what="avgpool3d fwd")
    close(dx.asnumpy(), env.ops.pool3d_bwd(x.astype(np.float64), dy.astype(np.float64), mode, pads, strides, win), what="pool3d bwd %s" % mode)


# ---- cross-operator fusion: the ReLU in front of a convolution packs the convolution's operand ---------------------------
@pytest.mark.parametrize("case", [(8, 64, 28, 28, 96, 3, 3, "SAME"), (8, 128, 14, 14, 256, 1, 1, "VALID"), (4, 40, 19, 17, 64, 5, 5, "SAME")])
@pytest.mark.parametrize("arith", ["3xfp16", "3xtf32"])
def test_relu_packs_the_next_convolutions_operand(env, case, arith):
    """BN -> ReLU -> convolution as three separate calls, twice on the same arrays (as an executor does step after step).
    The second time the ReLU writes y and the convolution's packed operand in one kernel; y must be the plain ReLU's,
    bit for bit, and the convolution's result must not change."""
    N, C, H, W, K, R, S, padding = case
    x, w = f32(N, C, H, W, scale=2.0), f32(K, C, R, S, scale=0.2)
    mean_p, var_p, bn_cell = env.gpu_op.bn_get_cudnnlist(x.shape, "NCHW", "pre_activation")
    act_cell = env.gpu_op.activation_get_cudnnlist(x.shape, "NCHW", "relu")
    g = env.ops.conv_geometry(x.shape, w.shape, padding, 1, 1)
    out_shape, cell = env.gpu_op.convolution_2d_forward_get_out_shape(x.shape, w.shape, "NCHW", padding, 1, 1)
    xd, wd = env.dev(x), env.dev(w)
    bn_out, y, conv_out = env.empty(x.shape), env.empty(x.shape), env.empty(out_shape)
    env.gpu_op.set_contraction_path(2)
    env.gpu_op.set_tensor_arithmetic(arith)
    try:
        results = []
        for step in range(3):
            if step == 2:
                xd._sync_copyfrom(x * np.float32(1.7) - np.float32(0.3))       # new data, same arrays: nothing stale may be reused
            before = env.gpu_op.fused_relu_pack_count()
            assert env.gpu_op.bn_forward(xd, bn_out, "pre_activation", 0, mean_p, var_p, bn_cell, env.cudnn, env.stream) == 0
            env.gpu_op.activation_forward(bn_out, y, "relu", act_cell, env.cudnn, env.stream)
            assert env.gpu_op.convolution_2d_forward(y, wd, conv_out, cell, env.cudnn, env.stream) == 0
            assert env.gpu_op.last_contraction_path() == 2
            results.append((env.gpu_op.fused_relu_pack_count() - before, bn_out.asnumpy(), y.asnumpy(), conv_out.asnumpy()))
    finally:
        env.gpu_op.set_contraction_path(0)
        env.gpu_op.set_tensor_arithmetic("3xfp16")
    assert results[0][0] == 0 and results[1][0] == 1 and results[2][0] == 1      # learned at the first pass, fused afterwards
    for fused, b, yy, cc in results:
        np.testing.assert_array_equal(yy, np.maximum(b, 0))
        y64, w64 = yy.astype(np.float64), w.astype(np.float64)
        close_dot(cc, env.ops.conv2d_fwd(y64, w64, g), env.ops.conv2d_fwd(np.abs(y64), np.abs(w64), g), what="conv behind the fused ReLU %s" % (case,))
    if arith == "3xtf32":
        # tf32 packs carry no scale, so the fused pass is the same arithmetic bit for bit; the fp16 pack's power-of-two
        # scale comes from max|BN output| (an upper bound known before the pass) instead of max|y|, which may round
        # the low halves differently
        np.testing.assert_array_equal(results[0][3], results[1][3])


# ---- failure reporting of the tensor path -----------------------------------------------------------------------------
def test_bounded_barrier_wait_reports_refuses_and_recovers(env):
    """Every barrier wait of the tensor-core kernels has a cycle limit.  The probe kernel waits, with a 20,000-cycle
    limit, on a barrier nothing arms: it returns by itself, the library's error word is raised, tensor-core launches are
    refused (return -1) until the word is cleared, and after that the path works again."""
    from tinyflow_b200._base import _LIB, TinyflowError
    assert env.gpu_op.tensor_path_error() == 0
    A, B = f32(256, 512), f32(512, 128)
    C = env.empty((256, 128))
    try:
        assert _LIB.TfTensorPathTimeoutProbe(ctypes.c_longlong(20000), env.stream) == 0
        assert _LIB.TfDeviceSynchronize() == -1               # the synchronising call reports the time-out
        assert env.gpu_op.tensor_path_error() == 1
        env.gpu_op.set_contraction_path(2)
        with pytest.raises(TinyflowError):
            env.gpu_op.matrix_multiply(env.dev(A), False, env.dev(B), False, C, env.cublas, env.stream)
    finally:
        env.gpu_op.clear_tensor_path_error()
        env.gpu_op.set_contraction_path(0)
    assert env.gpu_op.tensor_path_error() == 0
    env.gpu_op.set_contraction_path(2)
    try:
        env.gpu_op.matrix_multiply(env.dev(A), False, env.dev(B), False, C, env.cublas, env.stream)
    finally:
        env.gpu_op.set_contraction_path(0)
    a64, b64 = A.astype(np.float64), B.astype(np.float64)
    close_dot(C.asnumpy(), a64 @ b64, np.abs(a64) @ np.abs(b64), what="matmul after the error word was cleared")


# ---- size-independent properties at benchmark sizes ---------------------------------------------------------------------
def test_conv_linearity_and_adjointness_at_full_size(env):
    """At ResNet-50 batch-64 size the oracle is too slow; check <conv(x,w), dy> == <x, dgrad(dy,w)> == <w, wgrad(x,dy)>."""
    N, C, H, W, K = 64, 64, 55, 55, 64
    x, w = f32(N, C, H, W), f32(K, C, 3, 3, scale=0.05)
    out_shape, cell = env.gpu_op.convolution_2d_forward_get_out_shape(x.shape, w.shape, "NCHW", "SAME", 1, 1)
    dy = f32(*out_shape)
    xd, wd, dyd = env.dev(x), env.dev(w), env.dev(dy)
    y, dx, dw = env.empty(out_shape), env.empty(x.shape), env.empty(w.shape)
    env.gpu_op.convolution_2d_forward(xd, wd, y, cell, env.cudnn, env.stream)
    env.gpu_op.convolution_backward_data(xd, dyd, wd, dx, cell, env.cudnn, env.stream)
    env.gpu_op.convolution_backward_filter(xd, dyd, wd, dw, cell, env.cudnn, env.stream)
    a = np.vdot(y.asnumpy().astype(np.float64), dy.astype(np.float64))
    b = np.vdot(x.astype(np.float64), dx.asnumpy().astype(np.float64))
    c = np.vdot(w.astype(np.float64), dw.asnumpy().astype(np.float64))
    assert abs(a - b) <= 1e-5 * abs(a) and abs(a - c) <= 1e-5 * abs(a)


def test_batchnorm_output_statistics_at_full_size(env):
    shape = (64, 256, 55, 55)
    x = f32(*shape, scale=3.0) + np.float32(1.5)
    mean_p, var_p, cell = env.gpu_op.bn_get_cudnnlist(shape, "NCHW", "pre_activation")
    y = env.empty(shape)
    env.gpu_op.bn_forward(env.dev(x), y, "pre_activation", 0, mean_p, var_p, cell, env.cudnn, env.stream)
    yn = y.asnumpy().astype(np.float64)
    assert np.abs(yn.mean(axis=0)).max() < 1e-5
    assert np.abs(yn.var(axis=0) - 1.0).max() < 1e-3     # var/(var+eps) with eps 1e-5 and var ~ 9


_SPLIT_WORKER = r"""
import sys, numpy as np
from tinyflow_b200 import gpu_op, ndarray
ctx = ndarray.gpu(0)
stream = gpu_op.create_cudaStream(); cudnn = gpu_op.create_cudnnHandle(stream)
rng = np.random.RandomState(5)
out = {}
for i, (N, C, H, W, K, R, S, pad) in enumerate([(64, 256, 14, 14, 256, 3, 3, "SAME"), (64, 64, 28, 28, 96, 3, 3, "SAME"), (32, 512, 7, 7, 2048, 1, 1, "VALID"), (16, 192, 17, 17, 224, 1, 7, "SAME")]):
    x = rng.randn(N, C, H, W).astype(np.float32); w = (0.1 * rng.randn(K, C, R, S)).astype(np.float32)
    shape, cell = gpu_op.convolution_2d_forward_get_out_shape(x.shape, w.shape, "NCHW", pad, 1, 1)
    dy = rng.randn(*shape).astype(np.float32)
    xd, wd, dyd = ndarray.array(x, ctx), ndarray.array(w, ctx), ndarray.array(dy, ctx)
    y, dx, dw = ndarray.empty(shape, ctx), ndarray.empty(x.shape, ctx), ndarray.empty(w.shape, ctx)
    gpu_op.set_contraction_path(2)
    for rep in range(2):
        gpu_op.convolution_2d_forward(xd, wd, y, cell, cudnn, stream)
        gpu_op.convolution_backward_data(xd, dyd, wd, dx, cell, cudnn, stream)
        gpu_op.convolution_backward_filter(xd, dyd, wd, dw, cell, cudnn, stream)
        got = (y.asnumpy(), dx.asnumpy(), dw.asnumpy())
        if rep:
            for a, b in zip(got, first):
                assert np.array_equal(a, b), "two launches on the same operands disagree"
        first = got
    out["y%d" % i], out["dx%d" % i], out["dw%d" % i] = got
np.savez(sys.argv[1], **out)
"""


def test_split_reductions_give_the_same_bits_every_time(env, tmp_path):
    """The last, partial wave of tiles is cut into per-CTA pieces whose partial sums go through a workspace and are added
    by a second kernel in a fixed order (no floating-point atomics): two launches in one process and two processes must
    produce the same bits."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    files = []
    for tag in ("a", "b"):
        path = str(tmp_path / ("%s.npz" % tag))
        envv = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        r = subprocess.run([sys.executable, "-c", _SPLIT_WORKER, path], env=envv, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
        files.append(np.load(path))
    a, b = files
    for k in a.files:
        np.testing.assert_array_equal(a[k], b[k], err_msg="%s differs between two processes" % k)


_PAIR_WORKER = r"""
import sys, json, ctypes, numpy as np
from tinyflow_b200 import gpu_op, ndarray
from tinyflow_b200._base import _LIB
ctx = ndarray.gpu(0)
stream = gpu_op.create_cudaStream(); cudnn = gpu_op.create_cudnnHandle(stream)
cases = json.loads(sys.argv[2])
rng = np.random.RandomState(9)
out = {}
_LIB.TfKernelTimingEnable(2)
gpu_op.set_contraction_path(2)
for i, (N, C, H, W, K, R, S, pad) in enumerate(cases):
    x = rng.randn(N, C, H, W).astype(np.float32); w = (0.2 * rng.randn(K, C, R, S)).astype(np.float32)
    shape, cell = gpu_op.convolution_2d_forward_get_out_shape(x.shape, w.shape, "NCHW", pad, 1, 1)
    dy = rng.randn(*shape).astype(np.float32)
    xd, wd, dyd = ndarray.array(x, ctx), ndarray.array(w, ctx), ndarray.array(dy, ctx)
    y, dx = ndarray.empty(shape, ctx), ndarray.empty(x.shape, ctx)
    gpu_op.convolution_2d_forward(xd, wd, y, cell, cudnn, stream)
    gpu_op.convolution_backward_data(xd, dyd, wd, dx, cell, cudnn, stream)
    out["x%d" % i], out["w%d" % i], out["dy%d" % i], out["y%d" % i], out["dx%d" % i] = x, w, dy, y.asnumpy(), dx.asnumpy()
buf = ctypes.create_string_buffer(1 << 16)
_LIB.TfKernelTimingReport(buf, len(buf))
out["kernels"] = np.array([r["name"] for r in json.loads(buf.value.decode() or "[]")])
np.savez(sys.argv[1], **out)
"""


def test_cta_pair_kernel_matches_the_oracle(env, tmp_path):
    """TINYFLOW_PAIRS=2 sends every 128-column convolution (forward and backward-data) through the cta_group::2 kernel:
    clusters of two CTAs, each loading half of the B tile, one MMA stream for both SMs.  Same bound as the one-CTA
    kernel, including an odd number of 128-row tiles (the second CTA of the last pair has nothing to store) and output
    widths that are not multiples of 128."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cases = [(4, 128, 14, 14, 256, 3, 3, "SAME"), (8, 256, 9, 9, 128, 1, 1, "VALID"), (3, 64, 20, 20, 384, 3, 3, "SAME"), (4, 192, 8, 8, 320, 1, 3, "SAME")]
    path = str(tmp_path / "pairs.npz")
    envv = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""), TINYFLOW_PAIRS="2", TINYFLOW_TIMING_DETAIL="1")
    r = subprocess.run([sys.executable, "-c", _PAIR_WORKER, path, json.dumps(cases)], env=envv, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    got = np.load(path)
    assert any("pairs" in str(k) for k in got["kernels"]), "the pair kernel did not run: %s" % list(got["kernels"])
    for i, (N, C, H, W, K, R, S, pad) in enumerate(cases):
        x64, w64, dy64 = got["x%d" % i].astype(np.float64), got["w%d" % i].astype(np.float64), got["dy%d" % i].astype(np.float64)
        g = env.ops.conv_geometry(x64.shape, w64.shape, pad, 1, 1)
        close_dot(got["y%d" % i], env.ops.conv2d_fwd(x64, w64, g), env.ops.conv2d_fwd(np.abs(x64), np.abs(w64), g), what="pairs fwd %s" % (cases[i],))
        close_dot(got["dx%d" % i], env.ops.conv2d_dgrad(dy64, w64, g), env.ops.conv2d_dgrad(np.abs(dy64), np.abs(w64), g), what="pairs dgrad %s" % (cases[i],))

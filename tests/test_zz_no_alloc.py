"""The allocation-free sum entry point (DLGpuReduceSumAllStatic) against the pooled one.

Who needs it: callers that cannot allocate while they run, for instance a step replayed from a fixed
launch sequence, or an executor inside a memory plan that has given away every byte of the device, so
that even the pool's occasional cudaMalloc could fail or stall.  The variant keeps its per-block partial
sums in a fixed array inside the library; this test checks, through the C-ABI, that it returns what
DLGpuReduceSumAll returns, on two calls in a row (the second smaller, so stale partials from the first
would show), that the device allocator's books (bytes handed out, bytes cached) do not move across a call -
the property the entry point exists for - and that it refuses inputs beyond its stated capacity.
Collected last on purpose."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

MAX_ELEMS = 4096 * 8192


def _stats(lib):
    used, cached = ctypes.c_longlong(0), ctypes.c_longlong(0)
    assert lib.TfAllocatorStats(ctypes.byref(used), ctypes.byref(cached)) == 0
    return used.value, cached.value


def _sum_both(lib, nd, ctx, stream, x):
    dx = nd.array(x, ctx)
    a, b, c = nd.empty((1,), ctx), nd.empty((1,), ctx), nd.empty((1,), ctx)
    assert lib.DLGpuReduceSumAll(dx.handle, a.handle) == 0
    before = _stats(lib)
    assert lib.DLGpuReduceSumAllStatic(dx.handle, b.handle, stream) == 0
    assert lib.DLGpuReduceSumAllStatic(dx.handle, c.handle, stream) == 0
    assert _stats(lib) == before, "the allocation-free entry point touched the device allocator"
    assert float(b.asnumpy()[0]) == float(c.asnumpy()[0])           # same stream, same input: same bits
    return float(a.asnumpy()[0]), float(b.asnumpy()[0])


def test_static_scratch_sum_matches_pooled_sum(lib_path):
    from tinyflow_b200 import gpu_op, ndarray as nd
    from tinyflow_b200._base import _LIB, last_error
    ctx = nd.gpu(0)
    stream = gpu_op.create_cudaStream()
    rng = np.random.RandomState(5)
    for shape in [(3000, 1111), (64, 1000), (7,)]:          # 3.3 M elements (407 blocks), then far fewer
        x = rng.randn(*shape).astype(np.float32)
        pooled, static = _sum_both(_LIB, nd, ctx, stream, x)
        want = float(x.astype(np.float64).sum())
        scale = float(np.abs(x).astype(np.float64).sum())
        assert abs(static - want) <= 1e-6 * scale, (shape, static, want)
        assert abs(static - pooled) <= 1e-6 * scale, (shape, static, pooled)
    # capacity: one element too many is refused with a message, and nothing is launched
    big = nd.empty((MAX_ELEMS + 1,), ctx)
    out = nd.empty((1,), ctx)
    assert _LIB.DLGpuReduceSumAllStatic(big.handle, out.handle, stream) == -1
    assert "capacity" in last_error()
    gpu_op.device_synchronize()

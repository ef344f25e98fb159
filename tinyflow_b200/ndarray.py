"""Array container over the DLArray C-ABI; host-side mirror of pycode/tinyflow/ndarray.py.

Same public names and meaning as the reference module: ``DLContext``, ``DLArray``,
``cpu()``, ``gpu()``, ``is_gpu_ctx()``, ``NDArray`` (``shape``, ``ctx``, ``asnumpy()``,
``copyto()``, ``free_gpu()``, ``arr[:] = value``), ``array()``, ``empty()`` and the random
initialisers.  As in the reference, ``empty()`` / ``array()`` return an ``int`` (the number of
bytes that could not be allocated) instead of an NDArray when the device is out of memory.
"""
from __future__ import annotations

import ctypes

import numpy as np

from ._base import _LIB, c_array, check_call


class DLContext(ctypes.Structure):
    _fields_ = [("device_id", ctypes.c_int), ("device_type", ctypes.c_int)]
    MASK2STR = {1: "cpu", 2: "gpu"}

    def __init__(self, device_id=0, device_type=1):
        super().__init__()
        self.device_id = device_id
        self.device_type = device_type

    def __repr__(self):
        return "%s(%d)" % (DLContext.MASK2STR[self.device_type], self.device_id)


class DLArray(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("ctx", DLContext), ("ndim", ctypes.c_int),
                ("shape", ctypes.POINTER(ctypes.c_int64))]


DLArrayHandle = ctypes.POINTER(DLArray)

# No argtypes are declared, as in the reference (ndarray.py:96-259): integers travel as C ints, the
# context by value, everything else as the ctypes pointer object the caller built.


def cpu(dev_id=0):
    return DLContext(dev_id, 1)


def gpu(dev_id=0):
    return DLContext(dev_id, 2)


def is_gpu_ctx(ctx):
    return bool(ctx) and ctx.device_type == 2


def _borrow_numpy(np_data):
    """A stack DLArray aliasing a C-contiguous float32 numpy array (never freed by the library)."""
    assert np_data.flags["C_CONTIGUOUS"] and np_data.dtype == np.float32
    arr = DLArray()
    shape = c_array(ctypes.c_int64, np_data.shape)
    arr.data = np_data.ctypes.data_as(ctypes.c_void_p)
    arr.shape = shape
    arr.ndim = np_data.ndim
    arr.ctx = cpu(0)
    return arr, shape


class NDArray(object):
    """A buffer with a shape on the CPU (pinned) or GPU; no arithmetic."""
    __slots__ = ["handle", "is_freed", "_shape"]

    def __init__(self, handle):
        self.handle = handle
        self.is_freed = False
        c = handle.contents
        self._shape = tuple(c.shape[i] for i in range(c.ndim))

    def __del__(self):
        if self.is_freed or _LIB is None:
            return
        self.is_freed = True
        _LIB.DLArrayFree(self.handle)

    def free_gpu(self):
        if self.is_freed:
            return
        self.is_freed = True
        check_call(_LIB.DLArrayFree(self.handle))

    @property
    def shape(self):
        return self._shape

    @property
    def ctx(self):
        return self.handle.contents.ctx

    @property
    def data_ptr(self):
        return self.handle.contents.data

    def __setitem__(self, in_slice, value):
        if not isinstance(in_slice, slice) or in_slice.start is not None or in_slice.stop is not None:
            raise ValueError("Array only support set from numpy array")
        if isinstance(value, NDArray):
            if value.handle is not self.handle:
                value.copyto(self, None)
        elif isinstance(value, (np.ndarray, np.generic)):
            self._sync_copyfrom(value)
        else:
            raise TypeError("type %s not supported" % str(type(value)))

    def _sync_copyfrom(self, source_array):
        source_array = np.ascontiguousarray(source_array, dtype=np.float32)
        if source_array.shape != self.shape:
            raise ValueError("array shape do not match the shape of NDArray")
        src, keep = _borrow_numpy(source_array)
        check_call(_LIB.DLArrayCopyFromTo(ctypes.byref(src), self.handle, None))
        del keep

    def asnumpy(self):
        out = np.empty(self.shape, dtype=np.float32)
        dst, keep = _borrow_numpy(out)
        check_call(_LIB.DLArrayCopyFromTo(self.handle, ctypes.byref(dst), None))
        del keep
        return out

    def copyto(self, target, cudaStream=None):
        """Copy into ``target`` (an NDArray of the same size, or a context to allocate in)."""
        if isinstance(target, DLContext):
            target = empty(self.shape, target)
            if isinstance(target, int):
                return target
        if not isinstance(target, NDArray):
            raise ValueError("Unsupported target type %s" % str(type(target)))
        check_call(_LIB.DLArrayCopyFromTo(self.handle, target.handle, cudaStream))
        return target


def empty(shape, ctx=cpu(0)):
    shape = tuple(int(s) for s in shape)
    cshape = c_array(ctypes.c_int64, shape)
    handle = DLArrayHandle()
    short = ctypes.c_int(0)
    check_call(_LIB.DLArrayAlloc(cshape, len(shape), ctx, ctypes.byref(handle), ctypes.byref(short)))
    if short.value != 0:
        return short.value
    return NDArray(handle)


def array(arr, ctx=cpu(0)):
    if not isinstance(arr, np.ndarray):
        arr = np.array(arr)
    ret = empty(arr.shape, ctx)
    if isinstance(ret, int):
        return ret
    ret._sync_copyfrom(arr)
    return ret


def _filled(sample, ctx):
    return array(np.asarray(sample), ctx)


def Normal(loc=0, scale=1, size=None, ctx=cpu(0)):
    return _filled(np.random.normal(loc, scale, size), ctx)


def Uniform(low=0, high=1, size=None, ctx=cpu(0)):
    return _filled(np.random.uniform(low, high, size), ctx)


def xavier_Normal(loc=0, size=None, ctx=cpu(0)):
    return _filled(np.random.normal(loc, np.sqrt(2.0 / (size[0] + size[1])), size), ctx)


def xavier_Uniform(size=None, ctx=cpu(0)):
    a = np.sqrt(6.0 / (size[0] + size[1]))
    return _filled(np.random.uniform(-a, a, size), ctx)


def _pair(w, b0, ctx):
    wa = _filled(w, ctx)
    if isinstance(wa, int):
        return wa
    ba = empty(np.asarray(w).shape, ctx)
    if isinstance(ba, int):
        return ba
    ba._sync_copyfrom(np.broadcast_to(np.asarray(b0, dtype=np.float32).reshape((-1,) + (1,) * (np.asarray(w).ndim - 1)), np.asarray(w).shape))
    return wa, ba


def Normalex(loc=0, scale=1, size=None, ctx=cpu(0)):
    return _pair(np.random.normal(loc, scale, size), np.random.normal(loc, scale, size[0]), ctx)


def Uniformex(low=0, high=1, size=None, ctx=cpu(0)):
    return _pair(np.random.uniform(low, high, size), np.random.uniform(low, high, size[0]), ctx)


def xavier_Normalex(loc=0, size=None, ctx=cpu(0)):
    s = np.sqrt(2.0 / (size[0] + size[1]))
    return _pair(np.random.normal(loc, s, size), np.random.normal(loc, s, size[0]), ctx)


def xavier_Uniformex(size=None, ctx=cpu(0)):
    a = np.sqrt(6.0 / (size[0] + size[1]))
    return _pair(np.random.uniform(-a, a, size), np.random.uniform(-a, a, size[0]), ctx)

"""Loads the operator library and holds the ctypes helpers every wrapper uses.

Mirrors pycode/tinyflow/_base.py of the reference: one process-wide ``_LIB`` opened with
RTLD_GLOBAL from ``<repo>/build/lib/libc_runtime_api.so``.  There is no CPU fallback: a
missing library is an ImportError that says how to build it.

The library is mapped on the first call into it, not at import: building and analysing a graph
(``graph``, ``models``, ``Executor.__init__``) needs no device code, so a process that only walks
graphs (the CPU baseline arm of the benchmark) never maps the CUDA library.
"""
from __future__ import annotations

import ctypes
import os

_REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.environ.get("TINYFLOW_B200_LIB", os.path.join(_REPO, "build", "lib", "libc_runtime_api.so"))


def _load_lib():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: the CUDA operator library is not built. "
            "Run `python -m tinyflow_b200.build` (needs nvcc); there is no CPU fallback.")
    return ctypes.CDLL(LIB_PATH, ctypes.RTLD_GLOBAL)


class _LazyLib(object):
    """Stands for the ``ctypes.CDLL``; opens it when the first symbol is looked up."""

    def __init__(self):
        object.__setattr__(self, "_cdll", None)

    def _load(self):
        cdll = object.__getattribute__(self, "_cdll")
        if cdll is None:
            cdll = _load_lib()
            object.__setattr__(self, "_cdll", cdll)
        return cdll

    @property
    def loaded(self):
        return object.__getattribute__(self, "_cdll") is not None

    def __getattr__(self, name):
        return getattr(self._load(), name)


_LIB = _LazyLib()


class TinyflowError(RuntimeError):
    """A library call returned -1; carries the library's message."""


def last_error() -> str:
    buf = ctypes.create_string_buffer(512)
    _LIB.TfLastError(buf, 512)
    return buf.value.decode(errors="replace")


def check_call(ret):
    """Every C entry point returns 0 on success and -1 on failure."""
    if ret != 0:
        raise TinyflowError(last_error() or f"library call failed with {ret}")


def c_array(ctype, values):
    return (ctype * len(values))(*values)


def new_cell(depth: int):
    """A caller-owned cell the library writes an opaque pointer into.

    depth=2 gives the ``void **`` cells used for streams / handles / saved statistics,
    depth=3 the ``void ***`` descriptor-list cells, depth=4 the pointer-table cells.
    """
    cell = ctypes.c_void_p(0)
    cell = ctypes.pointer(cell)
    for _ in range(depth - 1):
        cell = ctypes.pointer(cell)
    return cell

"""Brings the reference's own Python layer under ``baseline/_ref/`` so that tests can drive this
library through the UNMODIFIED reference code (``pycode/tinyflow/{_base,ndarray,gpu_op,autodiff}.py``).

    python tests/reference_checkout.py /path/to/reference-checkout     (or set TINYFLOW_REFERENCE)

``baseline/_ref/`` is git-ignored: nothing of the reference enters this repository's history.  The
reference loads its operator library from ``<its root>/build/lib/libc_runtime_api.so``
(pycode/tinyflow/_base.py:10-20); :func:`import_reference` points that path at this repository's
build and stubs the modules the reference imports but the training step never calls
(``line_profiler``, the keras latency predictor).
"""
from __future__ import annotations

import os
import shutil
import sys
import types

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_ROOT = os.path.join(REPO, "baseline", "_ref")


def available() -> bool:
    return os.path.isfile(os.path.join(REF_ROOT, "pycode", "tinyflow", "autodiff.py"))


def populate(ref_checkout: str) -> str:
    """Copies ``<ref_checkout>/pycode`` to ``baseline/_ref/pycode`` (unchanged)."""
    src = os.path.join(ref_checkout, "pycode")
    if not os.path.isdir(src):
        raise SystemExit("%s has no pycode/ directory" % ref_checkout)
    dst = os.path.join(REF_ROOT, "pycode")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return dst


def _link_library():
    lib = os.path.join(REPO, "build", "lib", "libc_runtime_api.so")
    if not os.path.exists(lib):
        raise ImportError("build the library first: python -m tinyflow_b200.build")
    lib_dir = os.path.join(REF_ROOT, "build", "lib")
    os.makedirs(lib_dir, exist_ok=True)
    link = os.path.join(lib_dir, "libc_runtime_api.so")
    if os.path.islink(link) or os.path.exists(link):
        if os.path.exists(link) and os.path.samefile(link, lib):
            return
        os.remove(link)
    os.symlink(lib, link)


def import_reference():
    """Returns the reference's ``autodiff`` module, loaded from ``baseline/_ref`` over this repository's library."""
    if not available():
        raise ImportError("baseline/_ref/pycode is absent: run python tests/reference_checkout.py <reference checkout>")
    _link_library()
    if "line_profiler" not in sys.modules:
        try:
            import line_profiler  # noqa: F401
        except Exception:
            lp = types.ModuleType("line_profiler")
            lp.LineProfiler = object
            sys.modules["line_profiler"] = lp
    pred = types.ModuleType("pycode.tinyflow.agetinputsofmodel")      # keras latency predictor: not on the step's path
    pred.gettime = lambda *a, **k: 0.0
    sys.modules["pycode.tinyflow.agetinputsofmodel"] = pred
    if REF_ROOT not in sys.path:
        sys.path.insert(0, REF_ROOT)
    from pycode.tinyflow import autodiff as ref_ad
    return ref_ad


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TINYFLOW_REFERENCE")
    if not root:
        raise SystemExit("usage: reference_checkout.py /path/to/reference-checkout")
    print(populate(root))

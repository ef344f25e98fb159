"""The shared library must load without a GPU and export every symbol the boundary names."""
import ctypes
import json
import os
import re

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(REPO, "include", "c_runtime_api.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\bint\s+(\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib_path):
    lib = ctypes.CDLL(lib_path)
    names = _declared_symbols()
    assert len(names) > 90
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_library_exports_every_symbol_the_reference_wrappers_call(lib_path):
    """abi_symbols.json lists every _LIB.<name> in the reference's gpu_op.py / ndarray.py."""
    lib = ctypes.CDLL(lib_path)
    names = json.load(open(os.path.join(REPO, "tests", "golden", "abi_symbols.json")))
    # the 1-D/3-D/2-D fused "Backward" convolutions are declared by the reference header but their
    # definitions are commented out there (src/gpu_op.cu:1827-1946, 2220-2337, 2527-2643)
    undefined_in_reference = {"DLGpuConvolution1DBackward", "DLGpuConvolution2DBackward", "DLGpuConvolution3DBackward"}
    missing = [n for n in names if n not in undefined_in_reference and not hasattr(lib, n)]
    assert not missing, missing


def test_shape_functions_run_without_a_device(lib_path):
    from tinyflow_b200 import gpu_op
    out, _ = gpu_op.convolution_2d_forward_get_out_shape((64, 3, 230, 230), (64, 3, 7, 7), "NCHW", "VALID", 2, 2)
    assert out == (64, 64, 112, 112)
    out, _ = gpu_op.convolution_2d_forward_get_out_shape((2, 128, 17, 17), (128, 128, 1, 7), "NCHW", "SAME", 1, 1)
    assert out == (2, 128, 17, 17)
    out, _ = gpu_op.pooling_2d_forward_get_out_shape((64, 3, 224, 224), "NCHW", "max", 3, 3, 1, 1, 1, 1)
    assert out == (64, 3, 230, 230)
    out, _ = gpu_op.pooling_2d_forward_get_out_shape((64, 64, 112, 112), "NCHW", "max", 0, 0, 2, 2, 3, 3)
    assert out == (64, 64, 55, 55)


def test_bad_arguments_return_minus_one_not_abort(lib_path):
    import pytest
    from tinyflow_b200 import gpu_op
    from tinyflow_b200._base import TinyflowError
    with pytest.raises(TinyflowError):
        gpu_op.convolution_2d_forward_get_out_shape((1, 3, 8, 8), (4, 5, 3, 3), "NCHW", "SAME", 1, 1)   # channel mismatch
    with pytest.raises(TinyflowError):
        gpu_op.pooling_2d_forward_get_out_shape((1, 3, 2, 2), "NCHW", "max", 0, 0, 1, 1, 5, 5)          # window > input


def test_no_cpu_fallback(lib_path):
    """use_numpy=True is refused: the product has no CPU execution path."""
    import pytest
    from tinyflow_b200 import autodiff as ad
    a, b = ad.Variable("a"), ad.Variable("b")
    node = ad.add_op(a, b)
    with pytest.raises(NotImplementedError):
        node.op.compute(node, [None, None], None, None, None, None, use_numpy=True)

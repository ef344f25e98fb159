"""tinyflow_b200: B200 (sm_100a) operator library and host-side mirror of tinyflow's
ndarray / gpu_op / autodiff interface for the training-step hot path.

Importing the package does not load the CUDA library; ``tinyflow_b200.ndarray`` (and
everything built on it) does, and raises if ``build/lib/libc_runtime_api.so`` is missing.
"""
__all__ = ["ndarray", "gpu_op", "autodiff", "models", "build"]

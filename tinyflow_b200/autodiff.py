"""Namespace mirror of pycode/tinyflow/autodiff.py: ``from tinyflow_b200 import autodiff as ad``.

Graph construction and autodiff live in :mod:`tinyflow_b200.graph`, the training-step executor
in :mod:`tinyflow_b200.executor`; this module re-exports both under the reference's names.
"""
from .graph import *          # noqa: F401,F403
from .graph import (Node, Op, Variable, Placeholder, gradients, find_topo_sort, sum_node_list,  # noqa: F401
                    get_Variable_node_list, nodelist_to_name, dense, conv2withbias, crossEntropy_loss)
from .executor import Executor, getcomputelist, getsgdcomputelist, swapadam  # noqa: F401
from . import gpu_op, ndarray  # noqa: F401

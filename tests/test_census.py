"""The mirrored graph library must build the reference's graphs node for node.

tests/golden/census_*.json hold the reference executor's node order (operator name and inferred
output shape, optimiser nodes included) for the benchmark shapes, produced by running the
reference's own graph construction / gradients / topological sort / optimiser relocation
(tests/golden/make_golden.py).  The same pipeline on the mirror must give the same sequence.
"""
import json
import os

import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _mirror_census(name, batch):
    from tinyflow_b200 import autodiff as ad, models
    model = getattr(models, name)(batch=batch)
    ex = ad.Executor(model.loss, model.y, 0.001, None, None, None, optimizer="adam")
    shapes = {model.X: model.input_shape, model.y_: model.label_shape}
    for var, shape in model.param_shapes.items():
        shapes[var] = tuple(shape)
        m, v = ex.Variable_node_to_mv[var]
        shapes[m] = shapes[v] = tuple(shape)
    ex.infer_shape(shapes)
    return [[n.name, list(ex.node_to_shape_map[n])] for n in ex.topo_order]


@pytest.mark.parametrize("name,batch", [("resnet50", 64), ("vgg16", 64), ("inceptionv3", 32), ("densenet121", 32),
                                        ("inceptionv4", 32)])
def test_node_order_matches_reference(lib_path, name, batch):
    from tinyflow_b200 import models
    if not hasattr(models, name):
        pytest.skip("%s builder not present" % name)
    want = json.load(open(os.path.join(GOLDEN, "census_%s.json" % name)))["nodes"]
    got = _mirror_census(name, batch)
    assert len(got) == len(want)
    for i, (g, w) in enumerate(zip(got, want)):
        assert g == w, "node %d differs: mirror %s, reference %s" % (i, g, w)

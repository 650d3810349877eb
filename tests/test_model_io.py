"""The model file reader (the reference's YAML format) and, where the reference checkout is present, the reference's
own example model and frames as one more pin of the CPU oracle."""
import math
import os

import numpy as np
import pytest

import golden_io as G
import oracle as O
import refharness as R
from visualmesh_b200 import model_io
from visualmesh_b200 import workloads as W

EXAMPLE = os.path.join(os.environ.get("VM_REFERENCE", "/root/reference"), "example")


def test_round_trip_and_shape_checks(tmp_path):
    net = W.make_network(5, 6, [8, 3])
    net[0].append(W.Layer(np.eye(8, dtype=np.float32), np.zeros(8, np.float32), W.TANH))
    net[1][0] = W.Layer(net[1][0].weights, net[1][0].biases, W.SOFTMAX)
    path = str(tmp_path / "model.yaml")
    model_io.save_model(path, net, "RING6", {"shape": "SPHERE", "radius": 0.0949996})
    got, mesh, geometry = model_io.load_model(path)
    assert mesh == "RING6" and geometry["shape"] == "SPHERE"
    assert model_io.n_neighbours_of(got) == 6
    assert [len(g) for g in got] == [2, 1]
    for ga, gb in zip(got, net):
        for la, lb in zip(ga, gb):
            assert np.array_equal(la.weights, lb.weights) and np.array_equal(la.biases, lb.biases)
            assert la.activation == lb.activation
    with pytest.raises(ValueError, match="Unknown activation"):
        model_io.parse_model({"network": [[{"activation": "gelu", "weights": [[1.0]], "biases": [0.0]}]]})
    with pytest.raises(ValueError):
        model_io.parse_model({"network": [[{"activation": "selu", "weights": [[1.0, 2.0]] * 27, "biases": [0.0, 0.0]}]]})
    with pytest.raises(ValueError):
        model_io.parse_model({"mesh": "RING6"})


@pytest.mark.skipif(not (os.path.exists(EXAMPLE) and R.available()), reason="reference checkout not present")
def test_reference_example_model_and_frame_pin_the_oracle():
    """example/model.yaml (13 groups, first layer 28 x 16) on example/images/image0000000.jpg with its lens file:
    the plain-C oracle against the compiled reference, bit for bit."""
    import yaml
    from PIL import Image
    net, mesh_name, geometry = model_io.load_model(os.path.join(EXAMPLE, "model.yaml"))
    assert mesh_name == "RING6" and len(net) == 13 and net[0][0].weights.shape == (28, 16)
    lens_doc = yaml.safe_load(open(os.path.join(EXAMPLE, "images", "lens0000000.yaml")))
    img = np.asarray(Image.open(os.path.join(EXAMPLE, "images", "image0000000.jpg")).convert("RGBA"))
    H, Wd = img.shape[:2]
    proj = {"RECTILINEAR": W.RECTILINEAR, "EQUISOLID": W.EQUISOLID, "EQUIDISTANT": W.EQUIDISTANT}[lens_doc["projection"]]
    fov = float(lens_doc.get("fov", 2.0 * math.atan(math.hypot(Wd, H) * 0.5 / float(lens_doc["focal_length"]))))
    lens = W.Lens((Wd, H), proj, float(lens_doc["focal_length"]), tuple(lens_doc.get("centre", (0.0, 0.0))),
                  tuple(lens_doc.get("k", (0.0, 0.0))), fov)
    Hoc = np.asarray(lens_doc["Hoc"], dtype=np.float32).reshape(4, 4)
    spec = W.MeshSpec("RING6", "SPHERE", float(geometry["radius"]), 0.0, float(Hoc[2, 3]), 4.0, 10.0)
    mesh = R.RefMesh(spec)
    rays, nbrs = mesh.nodes()
    ranges = mesh.lookup(Hoc, lens)
    image = np.ascontiguousarray(img).reshape(-1)
    ref = mesh.classify(net, Hoc, lens, image, W.fourcc("RGBA"))
    out = O.classify(rays, nbrs, ranges, net, Hoc, lens, image, W.fourcc("RGBA"))
    assert len(ref["global_indices"]) > 100
    for key in ref:
        assert np.array_equal(G.bits(out[key]), G.bits(ref[key])), key


def test_example_model_fixture_pins_the_oracle_and_the_host_mesh_builder():
    """The stored outputs of the reference CPU engine for its own trained network on three of its example frames:
    the engine's host mesh builder reproduces the mesh, its host lookup the ranges, and the plain-C oracle every output
    array, bit for bit - on any machine, without the reference checkout."""
    from visualmesh_b200.engine import Mesh
    case = G.ExampleModelCase()
    assert len(case.network) == 13 and case.network[0][0].weights.shape == (28, 16)
    assert case.network[-1][0].weights.shape == (56, 5) and case.network[-1][0].activation == W.SOFTMAX
    mesh = Mesh.from_spec(case.mesh_spec)
    case.check_mesh(mesh.rays, mesh.neighbours)
    for fr in case.frames:
        ranges = mesh.lookup(fr["Hoc"], fr["lens"])
        assert np.array_equal(ranges, fr["ranges"])
        out = O.classify(mesh.rays, mesh.neighbours, ranges, case.network, fr["Hoc"], fr["lens"], fr["image"], case.format)
        assert len(out["global_indices"]) > 1000
        for key in ("global_indices", "neighbourhood", "pixel_coordinates", "classifications"):
            assert np.array_equal(G.bits(out[key]), G.bits(fr[key])), key

"""Loads the fixtures of tests/golden/ (written by tests/golden/make_golden.py from the reference itself)."""
import os

import numpy as np

from visualmesh_b200 import workloads as W

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = ["ring6_equisolid_rgba", "ring8_equidistant_bgra", "xygrid6_cylinder_rectilinear_rggb",
         "ring4_rectilinear_grey"]


class Case:
    def __init__(self, name):
        z = np.load(os.path.join(GOLDEN, name + ".npz"))
        self.name = name
        self.rays, self.nbrs = z["rays"], z["nbrs"]
        self.bsp = (z["bsp_ranges"], z["bsp_children"], z["bsp_cones"])
        self.lens = W.Lens(tuple(int(v) for v in z["lens_dimensions"]), int(z["lens_projection"]),
                           float(z["lens_focal_length"]), tuple(float(v) for v in z["lens_centre"]),
                           tuple(float(v) for v in z["lens_k"]), float(z["lens_fov"]))
        self.format = int(z["format"])
        s = [str(v) for v in z["mesh_spec"]]
        self.mesh_spec = W.MeshSpec(s[0], s[1], float(s[2]), float(s[3]), float(s[4]), float(s[5]), float(s[6]))
        lpg = z["net_layers_per_group"]
        self.network, i = [], 0
        for n in lpg:
            group = []
            for _ in range(int(n)):
                group.append(W.Layer(z[f"net_w{i}"], z[f"net_b{i}"], int(z[f"net_a{i}"])))
                i += 1
            self.network.append(group)
        self.frames = []
        for f in range(int(z["n_frames"])):
            self.frames.append(dict(Hoc=z[f"f{f}_Hoc"], image=z[f"f{f}_image"], ranges=z[f"f{f}_ranges"],
                                    pixel_coordinates=z[f"f{f}_px"], global_indices=z[f"f{f}_gi"],
                                    neighbourhood=z[f"f{f}_nb"], classifications=z[f"f{f}_cls"]))


def units():
    z = np.load(os.path.join(GOLDEN, "units.npz"))
    lenses = []
    for i in range(3):
        v = z[f"lens{i}"]
        lenses.append(W.Lens((int(v[0]), int(v[1])), int(v[2]), float(v[3]), (float(v[4]), float(v[5])),
                             (float(v[6]), float(v[7])), float(v[8])))
    return z, lenses


def bits(a):
    """Bit pattern view for exact float comparison (NaN == NaN, -0 != +0)."""
    a = np.ascontiguousarray(a)
    return a.view(np.uint32) if a.dtype == np.float32 else a


class ExampleModelCase:
    """The reference's trained example network (example/model.yaml) on three of its example frames, outputs of the
    reference CPU engine (written by make_golden.py's make_example_model_case). The mesh is rebuilt by the caller from
    mesh_spec; mesh_digest is the sha256 of the reference's rays and neighbour table."""

    NAME = "example_model_ring6_rectilinear_rgba"

    def __init__(self):
        z = np.load(os.path.join(GOLDEN, self.NAME + ".npz"))
        self.format = int(z["format"])
        s = [str(v) for v in z["mesh_spec"]]
        self.mesh_spec = W.MeshSpec(s[0], s[1], float(s[2]), float(s[3]), float(s[4]), float(s[5]), float(s[6]))
        self.mesh_digest = str(z["mesh_digest"])
        self.network, i = [], 0
        for n in z["net_layers_per_group"]:
            group = []
            for _ in range(int(n)):
                group.append(W.Layer(z[f"net_w{i}"], z[f"net_b{i}"], int(z[f"net_a{i}"])))
                i += 1
            self.network.append(group)
        self.frames = []
        for f in range(int(z["n_frames"])):
            v = z[f"f{f}_lens"]
            lens = W.Lens((int(v[0]), int(v[1])), int(v[2]), float(v[3]), (float(v[4]), float(v[5])),
                          (float(v[6]), float(v[7])), float(v[8]))
            rgb = z[f"f{f}_rgb"]
            rgba = np.concatenate([rgb, np.full(rgb.shape[:2] + (1,), 255, np.uint8)], axis=2).reshape(-1)
            self.frames.append(dict(lens=lens, Hoc=z[f"f{f}_Hoc"], image=np.ascontiguousarray(rgba),
                                    ranges=z[f"f{f}_ranges"], pixel_coordinates=z[f"f{f}_px"],
                                    global_indices=z[f"f{f}_gi"], neighbourhood=z[f"f{f}_nb"],
                                    classifications=z[f"f{f}_cls"]))

    def check_mesh(self, rays, neighbours):
        import hashlib
        got = hashlib.sha256(np.ascontiguousarray(rays, np.float32).tobytes()
                             + np.ascontiguousarray(neighbours, np.int32).tobytes()).hexdigest()
        assert got == self.mesh_digest, "the host mesh builder did not reproduce the reference's mesh tables"

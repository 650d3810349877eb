"""Generates the golden fixtures in this folder FROM THE REFERENCE ITSELF.

Run where the reference checkout exists and oracle/_ref/libvmref.so has been built (make -C oracle):

    python tests/golden/make_golden.py

Every array below is an output of the unmodified reference (cpu::Engine, Mesh::lookup, visualmesh::project,
cpu::interpolate) on seeded inputs; the inputs that cannot be regenerated without the reference (mesh nodes and BSP)
are stored with them. The fixtures pin the plain-C oracle and the CUDA engine on machines without the reference.
"""
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, ".."))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

import refharness as R  # noqa: E402
from visualmesh_b200 import workloads as W  # noqa: E402

deg = math.pi / 180.0

ALL_FORMATS = ["RGGB", "GRBG", "GBRG", "BGGR", "BGR3", "BGR8", "BGRA", "RGB3", "RGB8", "RGBA", "GRAY", "GREY", "Y8  "]


def bpp(code):
    if code in ("RGBA", "BGRA"):
        return 4
    if code in ("RGB3", "RGB8", "BGR3", "BGR8"):
        return 3
    return 1


def multi_layer_network(seed, n_neighbours):
    """Two groups, the first with two dense layers after one gather, exercising every activation."""
    slots = n_neighbours + 1
    u = lambda s, shape, lim: W.uniform(W._mix_seed(seed, s), int(np.prod(shape)), -lim, lim).reshape(shape).astype(np.float32)
    g0 = [W.Layer(u(1, (slots * 4, 6), 0.4), u(2, (6,), 0.1), W.RELU),
          W.Layer(u(3, (6, 5), 0.5), u(4, (5,), 0.1), W.TANH)]
    g1 = [W.Layer(u(5, (slots * 5, 8), 0.4), u(6, (8,), 0.1), W.SELU),
          W.Layer(u(7, (8, 3), 0.5), u(8, (3,), 0.1), W.SOFTMAX)]
    return [g0, g1]


def net_arrays(net):
    out = {}
    out["net_layers_per_group"] = np.array([len(g) for g in net], dtype=np.int32)
    i = 0
    for g in net:
        for l in g:
            out[f"net_w{i}"] = l.weights
            out[f"net_b{i}"] = l.biases
            out[f"net_a{i}"] = np.int32(l.activation)
            i += 1
    return out


CASES = [
    # name, mesh spec, lens, (pitch, roll) list, format, network kind
    ("ring6_equisolid_rgba", W.MeshSpec("RING6", "SPHERE", 0.0949, 0.0, 1.2, 2.0, 6.0),
     W.Lens((160, 128), W.EQUISOLID, 0.35 * 160, (0.0, 0.0), (0.0, 0.0), math.pi),
     [(-45, 0), (-80, 15), (10, -5)], "RGBA", [8, 8, 3]),
    ("ring8_equidistant_bgra", W.MeshSpec("RING8", "SPHERE", 0.0949, 0.0, 0.8, 2.0, 5.0),
     W.Lens((192, 144), W.EQUIDISTANT, 0.3 * 192, (3.0, -2.0), (-0.1 / 192**2, 0.02 / 192**4), math.pi),
     [(-60, 5), (-25, -10)], "BGRA", "multi"),
    ("xygrid6_cylinder_rectilinear_rggb", W.MeshSpec("XYGRID6", "CYLINDER", 0.2, 1.8, 1.0, 1.0, 6.0),
     W.Lens((256, 192), W.RECTILINEAR, 0.6 * 256, (0.0, 0.0), (-0.05 / 256**2, 0.01 / 256**4),
            2.0 * math.atan(math.hypot(256, 192) * 0.5 / (0.6 * 256))),
     [(-35, 0), (-10, 0), (-89, 0)], "RGGB", [16, 12, 2]),
    ("ring4_rectilinear_grey", W.MeshSpec("RING4", "CIRCLE", 0.1, 0.0, 1.0, 2.0, 5.0),
     W.Lens((128, 96), W.RECTILINEAR, 0.8 * 128, (-1.5, 2.5), (0.0, 0.0),
            2.0 * math.atan(math.hypot(128, 96) * 0.5 / (0.8 * 128))),
     [(-50, 3), (60, 0)], "GREY", [4, 2]),
]


def make_case(name, spec, lens, poses, code, netkind, seed=1234):
    mesh = R.RefMesh(spec)
    rays, nbrs = mesh.nodes()
    b_ranges, b_children, b_cones = mesh.bsp()
    net = multi_layer_network(seed, mesh.n_neighbours) if netkind == "multi" else W.make_network(
        seed, mesh.n_neighbours, netkind)
    fmt = W.fourcc(code)
    out = dict(rays=rays, nbrs=nbrs, bsp_ranges=b_ranges, bsp_children=b_children, bsp_cones=b_cones,
               lens_dimensions=np.array(lens.dimensions, np.int32), lens_projection=np.int32(lens.projection),
               lens_focal_length=np.float32(lens.focal_length), lens_centre=np.array(lens.centre, np.float32),
               lens_k=np.array(lens.k, np.float32), lens_fov=np.float32(lens.fov), format=np.uint32(fmt),
               n_frames=np.int32(len(poses)),
               mesh_spec=np.array([spec.model, spec.shape, repr(spec.shape_a), repr(spec.shape_b), repr(spec.h),
                                   repr(spec.k), repr(spec.max_distance)]))
    out.update(net_arrays(net))
    for f, (pitch, roll) in enumerate(poses):
        Hoc = W.make_Hoc(pitch * deg, roll * deg, spec.h)
        image = W.random_bytes(W._mix_seed(seed, 77, f), lens.dimensions[0] * lens.dimensions[1] * bpp(code))
        ranges = mesh.lookup(Hoc, lens)
        c = mesh.classify(net, Hoc, lens, image, fmt)
        out[f"f{f}_Hoc"] = Hoc
        out[f"f{f}_image"] = image
        out[f"f{f}_ranges"] = ranges
        out[f"f{f}_px"] = c["pixel_coordinates"]
        out[f"f{f}_gi"] = c["global_indices"]
        out[f"f{f}_nb"] = c["neighbourhood"]
        out[f"f{f}_cls"] = c["classifications"]
        print(name, f, "nodes", mesh.n_nodes, "ranges", len(ranges), "on screen", len(c["global_indices"]))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)


def make_units(seed=99):
    out = {}
    # visualmesh::project on random unit vectors around the optical axis, incl. the axis itself and |x| > 1
    n = 4096
    v = W.uniform(W._mix_seed(seed, 1), 3 * n, -1, 1).reshape(n, 3)
    v[:, 0] = np.abs(v[:, 0]) * 1.5 + 0.05
    v /= np.linalg.norm(v, axis=1, keepdims=True)
    rays = v.astype(np.float32)
    rays[0] = (1.0, 0.0, 0.0)
    rays[1] = (np.float32(1.0000001), 0.0, 0.0)
    rays[2] = (0.0, 1.0, 0.0)
    rays[3] = (-0.5, 0.5, math.sqrt(0.5))
    out["rays"] = rays
    lenses = [
        W.Lens((1280, 1024), W.EQUISOLID, 448.0, (0.0, 0.0), (0.0, 0.0), math.pi),
        W.Lens((1280, 1024), W.EQUIDISTANT, 384.0, (4.0, -7.0), (-0.1 / 1280**2, 0.02 / 1280**4), math.pi),
        W.Lens((2048, 1536), W.RECTILINEAR, 1228.8, (0.0, 0.0), (-0.05 / 2048**2, 0.01 / 2048**4), 1.612),
    ]
    for i, lens in enumerate(lenses):
        out[f"lens{i}"] = np.array([lens.dimensions[0], lens.dimensions[1], lens.projection, lens.focal_length,
                                    lens.centre[0], lens.centre[1], lens.k[0], lens.k[1], lens.fov], np.float64)
        out[f"px{i}"] = R.project_rays(rays, lens)
    # cpu::interpolate for every fourcc on a small image, incl. borders
    Wd, Ht = 37, 23
    m = 600
    px = np.stack([W.uniform(W._mix_seed(seed, 2), m, 0, Wd - 1), W.uniform(W._mix_seed(seed, 3), m, 0, Ht - 1)], 1)
    px = px.astype(np.float32)
    px[0] = (0.0, 0.0)
    px[1] = (Wd - 1.001, Ht - 1.001)
    px[2] = (0.25, Ht - 1.5)
    px[3] = (Wd - 1.5, 0.75)
    px[4] = (5.0, 7.0)
    out["sample_px"] = px
    out["sample_dims"] = np.array([Wd, Ht], np.int32)
    for code in ALL_FORMATS:
        image = W.random_bytes(W._mix_seed(seed, 4, W.fourcc(code)), Wd * Ht * bpp(code))
        out[f"sample_image_{code.strip()}"] = image
        out[f"sample_out_{code.strip()}"] = R.interpolate(px, image, Wd, Ht, W.fourcc(code))
    np.savez_compressed(os.path.join(HERE, "units.npz"), **out)


def make_example_model_case(reference, name="example_model_ring6_rectilinear_rgba", indices=(0, 10, 20), scale=2):
    """The reference's own trained network (example/model.yaml: 13 groups, 28x16 ... 56x5, read as
    example/load_model.hpp:25-52 reads it) on three of its example frames (example/images/imageNNNNNNN.jpg with the
    lens and Hoc of lensNNNNNNN.yaml), through the reference CPU engine. The frames are stored decoded (JPEG decoders
    differ in their last bits) at 1/scale of their resolution, with the focal length scaled to match, to keep the
    fixture small; the mesh is the benchmark's Ring6 over the model's sphere (example/benchmark.cpp:121-122) at the
    first frame's camera height with fewer intersections and a shorter range. Mesh tables are not stored: the engine's own
    host mesh builder reproduces them (their digest is stored and checked)."""
    import hashlib

    import yaml
    from PIL import Image

    from visualmesh_b200 import model_io
    example = os.path.join(reference, "example")
    net, mesh_name, geometry = model_io.load_model(os.path.join(example, "model.yaml"))
    assert mesh_name == "RING6"
    docs = [yaml.safe_load(open(os.path.join(example, "images", f"lens{i:07d}.yaml"))) for i in indices]
    # the frames' camera heights differ slightly (1.07 .. 1.2 m); like a table entry of the benchmark's VisualMesh, one
    # Mesh (at the first frame's height) serves them all - the Mesh overload of the engines takes the mesh it is given
    spec = W.MeshSpec("RING6", "SPHERE", float(geometry["radius"]), 0.0, float(docs[0]["Hoc"][2][3]), 4.0, 10.0)
    mesh = R.RefMesh(spec)
    rays, nbrs = mesh.nodes()
    digest = hashlib.sha256(rays.tobytes() + nbrs.tobytes()).hexdigest()
    first = Image.open(os.path.join(example, "images", f"image{indices[0]:07d}.jpg"))
    Wd, Ht = first.size[0] // scale, first.size[1] // scale
    proj = {"RECTILINEAR": W.RECTILINEAR, "EQUISOLID": W.EQUISOLID, "EQUIDISTANT": W.EQUIDISTANT}
    fmt = W.fourcc("RGBA")
    out = dict(format=np.uint32(fmt), n_frames=np.int32(len(indices)), mesh_digest=np.array(digest),
               mesh_spec=np.array([spec.model, spec.shape, repr(spec.shape_a), repr(spec.shape_b), repr(spec.h),
                                   repr(spec.k), repr(spec.max_distance)]),
               source=np.array([f"example/images/image{i:07d}.jpg" for i in indices]))
    out.update(net_arrays(net))
    for f, (i, doc) in enumerate(zip(indices, docs)):
        img = Image.open(os.path.join(example, "images", f"image{i:07d}.jpg")).convert("RGB")
        rgb = np.asarray(img.resize((Wd, Ht), Image.BILINEAR), dtype=np.uint8)
        rgba = np.concatenate([rgb, np.full((Ht, Wd, 1), 255, np.uint8)], axis=2).reshape(-1)
        focal = float(doc["focal_length"]) / scale
        fov = float(doc.get("fov", 2.0 * math.atan(math.hypot(Wd, Ht) * 0.5 / focal)))
        k = [float(v) for v in doc.get("k", (0.0, 0.0))]
        # k applies to radii in pixels (cpp/visualmesh/utility/projection.hpp:163-176): r' = r / scale
        lens = W.Lens((Wd, Ht), proj[doc["projection"]], focal, tuple(float(v) / scale for v in doc.get("centre", (0, 0))),
                      (k[0] * scale**2, k[1] * scale**4), fov)
        Hoc = np.asarray(doc["Hoc"], dtype=np.float32).reshape(4, 4)
        c = mesh.classify(net, Hoc, lens, rgba, fmt)
        out[f"f{f}_lens"] = np.array([Wd, Ht, lens.projection, lens.focal_length, lens.centre[0], lens.centre[1],
                                      lens.k[0], lens.k[1], lens.fov], np.float64)
        out[f"f{f}_Hoc"] = Hoc
        out[f"f{f}_rgb"] = rgb
        out[f"f{f}_ranges"] = mesh.lookup(Hoc, lens)
        out[f"f{f}_px"] = c["pixel_coordinates"]
        out[f"f{f}_gi"] = c["global_indices"]
        out[f"f{f}_nb"] = c["neighbourhood"]
        out[f"f{f}_cls"] = c["classifications"]
        print(name, f, "nodes", mesh.n_nodes, "on screen", len(c["global_indices"]),
              "classes argmax histogram", np.bincount(c["classifications"][:-1].argmax(1), minlength=5))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)


if __name__ == "__main__":
    reference = os.environ.get("VM_REFERENCE", "/root/reference")
    if "--example-model-only" not in sys.argv:
        for case in CASES:
            make_case(*case)
        make_units()
    make_example_model_case(reference)
    total = sum(os.path.getsize(os.path.join(HERE, f)) for f in os.listdir(HERE) if f.endswith(".npz"))
    print("total fixture bytes", total)

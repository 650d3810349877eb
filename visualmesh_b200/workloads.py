"""Seeded synthetic workloads: the five benchmark configurations as concrete inputs.

Everything here is a pure function of (seed, config, frame): images, camera poses, lenses and network weights come
from a splitmix64 stream written out below, never from a library distribution whose algorithm may change.
The frames stand in for camera frames; only sizes, formats and value distributions are taken from the configurations.

Resolutions of what the configuration text leaves open or names differently from the reference:
  * distortion k is given width-normalised; the lens wants pixels: k_px = (k1 / W^2, k2 / W^4)
    (the reference applies k to radii in pixels, cpp/visualmesh/utility/projection.hpp:163-176);
  * "3 RGB input channels": first-layer weights are drawn for (N+1)*3 rows and a zero row is inserted for alpha, as
    the reference's exporter does (training/export.py:83-89) - the engine's input is always 4 channels
    (cpp/visualmesh/engine/cpu/engine.hpp:208-209);
  * Radial8 -> Ring8, Grid6 -> XYGrid6 (cpp/visualmesh/model/); Cylinder is a new host shape (see hostmesh);
  * unspecified fov -> pi for fisheye lenses, the diagonal field of view for the rectilinear one
    (cpp/visualmesh/lens.hpp:46-50); unspecified roll -> 0; unspecified pitch (config 3) -> -45 degrees.
"""
import math
from dataclasses import dataclass, field
from typing import List, Tuple

import numpy as np

RECTILINEAR, EQUISOLID, EQUIDISTANT = 0, 1, 2
SELU, RELU, SOFTMAX, TANH = 0, 1, 2, 3

_M64 = (1 << 64) - 1


def fourcc(code: str) -> int:
    """cpp/visualmesh/utility/fourcc.hpp:34-36"""
    assert len(code) == 4
    return ord(code[0]) | (ord(code[1]) << 8) | (ord(code[2]) << 16) | (ord(code[3]) << 24)


def _mix_seed(*parts: int) -> int:
    z = 0x9E3779B97F4A7C15
    for p in parts:
        z = (z ^ (p & _M64)) & _M64
        z = (z * 0xBF58476D1CE4E5B9) & _M64
        z ^= z >> 29
        z = (z * 0x94D049BB133111EB) & _M64
        z ^= z >> 32
    return z & _M64


def splitmix64(seed: int, n: int) -> np.ndarray:
    """n outputs of the splitmix64 generator started at `seed`, as uint64."""
    with np.errstate(over="ignore"):
        z = np.uint64(seed) + np.arange(1, n + 1, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def uniform(seed: int, n: int, lo: float = 0.0, hi: float = 1.0) -> np.ndarray:
    u = (splitmix64(seed, n) >> np.uint64(11)).astype(np.float64) * (1.0 / (1 << 53))
    return lo + (hi - lo) * u


def random_bytes(seed: int, n: int) -> np.ndarray:
    words = splitmix64(seed, (n + 7) // 8)
    return words.view(np.uint8)[:n].copy()


@dataclass
class Lens:
    """visualmesh::Lens<float>, cpp/visualmesh/lens.hpp:35-52"""
    dimensions: Tuple[int, int]
    projection: int
    focal_length: float
    centre: Tuple[float, float] = (0.0, 0.0)
    k: Tuple[float, float] = (0.0, 0.0)
    fov: float = math.pi


@dataclass
class Layer:
    """visualmesh::Layer<float>; weights [n_in][n_out], cpp/visualmesh/network_structure.hpp:25-45"""
    weights: np.ndarray
    biases: np.ndarray
    activation: int


# A network is a list of groups, a group a list of layers (cpp/visualmesh/network_structure.hpp:47-52)
Network = List[List[Layer]]


def make_Hoc(pitch: float, roll: float, height: float) -> np.ndarray:
    """Camera-to-observation-plane transform. Camera x is the optical axis, y left, z up
    (readme/flavour/orientation.md:4-16); the columns of the rotation block are the camera axes in world space."""
    cp, sp = math.cos(pitch), math.sin(pitch)
    cr, sr = math.cos(roll), math.sin(roll)
    x_c = np.array([cp, 0.0, sp])
    y0 = np.array([0.0, 1.0, 0.0])
    z0 = np.array([-sp, 0.0, cp])
    y_c = cr * y0 + sr * z0
    z_c = -sr * y0 + cr * z0
    H = np.eye(4, dtype=np.float64)
    H[:3, 0], H[:3, 1], H[:3, 2] = x_c, y_c, z_c
    H[2, 3] = height
    return H.astype(np.float32)


def make_network(seed: int, n_neighbours: int, widths: List[int], rgb_first_layer: bool = True) -> Network:
    """Glorot-uniform weights, U(-0.1, 0.1) biases, SELU everywhere and softmax on the last layer;
    one dense layer per group."""
    net: Network = []
    c_in = 4
    for li, c_out in enumerate(widths):
        slots = n_neighbours + 1
        s = _mix_seed(seed, 0x6E6574, li)
        if li == 0 and rgb_first_layer:
            fan_in = slots * 3
            lim = math.sqrt(6.0 / (fan_in + c_out))
            w3 = uniform(s, fan_in * c_out, -lim, lim).reshape(slots, 3, c_out)
            w = np.zeros((slots, 4, c_out), dtype=np.float64)
            w[:, :3, :] = w3
            w = w.reshape(slots * 4, c_out)
        else:
            fan_in = slots * c_in
            lim = math.sqrt(6.0 / (fan_in + c_out))
            w = uniform(s, fan_in * c_out, -lim, lim).reshape(fan_in, c_out)
        b = uniform(_mix_seed(s, 1), c_out, -0.1, 0.1)
        act = SOFTMAX if li == len(widths) - 1 else SELU
        net.append([Layer(np.ascontiguousarray(w, dtype=np.float32), b.astype(np.float32), act)])
        c_in = c_out
    return net


@dataclass
class MeshSpec:
    model: str
    shape: str
    shape_a: float
    shape_b: float
    h: float
    k: float
    max_distance: float

    def key(self):
        return (self.model, self.shape, self.shape_a, self.shape_b, self.h, self.k, self.max_distance)


@dataclass
class Frame:
    mesh: MeshSpec
    Hoc: np.ndarray
    lens: Lens
    format: int
    image_seed: int
    image_bytes: int

    def image(self) -> np.ndarray:
        return random_bytes(self.image_seed, self.image_bytes)


@dataclass
class Workload:
    name: str
    description: str
    n_neighbours: int
    network: Network
    frames: List[Frame] = field(default_factory=list)


def _bpp(fmt: int) -> int:
    return 4 if fmt in (fourcc("RGBA"), fourcc("BGRA")) else 1


def config(index: int, seed: int = 0, n_frames: int = None) -> Workload:
    """The five benchmark configurations. n_frames overrides the frame count (a prefix or a longer stream of the same
    generator)."""
    deg = math.pi / 180.0
    ring6 = MeshSpec("RING6", "SPHERE", 0.0949, 0.0, 1.2, 6.0, 20.0)
    if index == 0:
        W, H, fmt = 1280, 1024, fourcc("RGBA")
        n = 1 if n_frames is None else n_frames
        net = make_network(_mix_seed(seed, 0), 6, [16, 16, 8, 2])
        lens = Lens((W, H), EQUISOLID, 0.35 * W, (0.0, 0.0), (0.0, 0.0), math.pi)
        wl = Workload("cfg0", "Ring6/Sphere h=1.2, 1280x1024 RGBA, equisolid, 4 layers 16,16,8,2", 6, net)
        for f in range(n):
            wl.frames.append(Frame(ring6, make_Hoc(-45 * deg, 0.0, 1.2), lens, fmt, _mix_seed(seed, 0, 1, f), W * H * 4))
        return wl
    if index == 1:
        W, H, fmt = 1280, 1024, fourcc("RGBA")
        n = 64 if n_frames is None else n_frames
        net = make_network(_mix_seed(seed, 1), 6, [16, 16, 16, 16, 8, 8, 8, 3])
        lens = Lens((W, H), EQUIDISTANT, 0.3 * W, (0.0, 0.0), (-0.1 / W**2, 0.02 / W**4), math.pi)
        wl = Workload("cfg1", "Ring6/Sphere h=1.2, 64x 1280x1024 RGBA, equidistant k=[-0.1,0.02]/W^n, 8 layers", 6, net)
        pose = uniform(_mix_seed(seed, 1, 2), 2 * n)
        for f in range(n):
            pitch = (-70 + 50 * pose[2 * f]) * deg
            roll = (-10 + 20 * pose[2 * f + 1]) * deg
            wl.frames.append(Frame(ring6, make_Hoc(pitch, roll, 1.2), lens, fmt, _mix_seed(seed, 1, 1, f), W * H * 4))
        return wl
    if index == 2:
        W, H, fmt = 2048, 1536, fourcc("RGGB")
        n = 32 if n_frames is None else n_frames
        mesh = MeshSpec("XYGRID6", "CYLINDER", 0.2, 1.8, 1.0, 4.0, 15.0)
        net = make_network(_mix_seed(seed, 2), 6, [16, 16, 12, 8, 8, 2])
        f_px = 0.6 * W
        fov = 2.0 * math.atan(math.hypot(W, H) * 0.5 / f_px)
        lens = Lens((W, H), RECTILINEAR, f_px, (0.0, 0.0), (-0.05 / W**2, 0.01 / W**4), fov)
        wl = Workload("cfg2", "XYGrid6/Cylinder(0.2,1.8) h=1.0, 32x 2048x1536 BayerRG8, rectilinear, 6 layers", 6, net)
        pose = uniform(_mix_seed(seed, 2, 2), n)
        for f in range(n):
            pitch = (-60 + 50 * pose[f]) * deg
            wl.frames.append(Frame(mesh, make_Hoc(pitch, 0.0, 1.0), lens, fmt, _mix_seed(seed, 2, 1, f), W * H))
        return wl
    if index == 3:
        W, H, fmt = 2592, 2048, fourcc("RGBA")
        n = 32 if n_frames is None else n_frames
        mesh = MeshSpec("RING8", "SPHERE", 0.0949, 0.0, 1.6, 12.0, 50.0)
        net = make_network(_mix_seed(seed, 3), 8, [32] * 9 + [4])
        lens = Lens((W, H), EQUISOLID, 0.35 * W, (0.0, 0.0), (0.0, 0.0), math.pi)
        wl = Workload("cfg3", "Ring8/Sphere k=12 d=50 h=1.6, 32x 2592x2048 RGBA, equisolid, 10 layers of 32", 8, net)
        for f in range(n):
            wl.frames.append(Frame(mesh, make_Hoc(-45 * deg, 0.0, 1.6), lens, fmt, _mix_seed(seed, 3, 1, f), W * H * 4))
        return wl
    if index == 4:
        W, H, fmt = 1280, 1024, fourcc("RGBA")
        n = 4096 if n_frames is None else n_frames
        net = make_network(_mix_seed(seed, 0), 6, [16, 16, 8, 2])
        lens = Lens((W, H), EQUISOLID, 0.35 * W, (0.0, 0.0), (0.0, 0.0), math.pi)
        wl = Workload("cfg4", "cfg0 mesh at h in {0.4,0.8,1.2,1.6}, stream of 1280x1024 RGBA frames", 6, net)
        pose = uniform(_mix_seed(seed, 4, 2), 3 * n)
        heights = [0.4, 0.8, 1.2, 1.6]
        for f in range(n):
            h = heights[min(int(pose[3 * f] * 4), 3)]
            pitch = (-70 + 50 * pose[3 * f + 1]) * deg
            roll = (-10 + 20 * pose[3 * f + 2]) * deg
            mesh = MeshSpec("RING6", "SPHERE", 0.0949, 0.0, h, 6.0, 20.0)
            wl.frames.append(Frame(mesh, make_Hoc(pitch, roll, h), lens, fmt, _mix_seed(seed, 4, 1, f), W * H * 4))
        return wl
    raise ValueError("config index must be 0..4")

"""ctypes front end of oracle/_ref/libvmref.so - the unmodified reference compiled behind a C ABI.

Test infrastructure only. The library is built by oracle/Makefile from the reference's headers; where it has not
been built (no reference checkout on this machine and no prebuilt file) `available()` is False and tests that need
it skip. libvmref.so holds reference code only. A second build of the same harness, libvmref_cuda.so, also carries
the C++ drop-in engine (include/visualmesh/engine/cuda/engine.hpp) and therefore links the CUDA library; it is loaded
only by the tests that call the drop-in (`classify(cuda=True)`), never by the timed CPU baseline.
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "..", "oracle", "_ref", "libvmref.so")
_CUDA_LIB_PATH = os.path.join(_HERE, "..", "oracle", "_ref", "libvmref_cuda.so")


class CLens(C.Structure):
    _fields_ = [
        ("dimensions", C.c_int32 * 2),
        ("projection", C.c_int32),
        ("focal_length", C.c_float),
        ("centre", C.c_float * 2),
        ("k", C.c_float * 2),
        ("fov", C.c_float),
    ]


class CLayer(C.Structure):
    _fields_ = [
        ("weights", C.c_void_p),
        ("biases", C.c_void_p),
        ("n_in", C.c_int32),
        ("n_out", C.c_int32),
        ("activation", C.c_int32),
    ]


def c_lens(lens) -> CLens:
    out = CLens()
    out.dimensions[0], out.dimensions[1] = int(lens.dimensions[0]), int(lens.dimensions[1])
    out.projection = int(lens.projection)
    out.focal_length = float(lens.focal_length)
    out.centre[0], out.centre[1] = float(lens.centre[0]), float(lens.centre[1])
    out.k[0], out.k[1] = float(lens.k[0]), float(lens.k[1])
    out.fov = float(lens.fov)
    return out


def c_network(network):
    """Returns (layers array, layers_per_group array, n_groups, keepalive list)."""
    flat = [layer for group in network for layer in group]
    arr = (CLayer * max(len(flat), 1))()
    keep = []
    for i, layer in enumerate(flat):
        w = np.ascontiguousarray(layer.weights, dtype=np.float32)
        b = np.ascontiguousarray(layer.biases, dtype=np.float32)
        keep += [w, b]
        arr[i].weights = w.ctypes.data
        arr[i].biases = b.ctypes.data
        arr[i].n_in, arr[i].n_out = w.shape
        arr[i].activation = int(layer.activation)
    lpg = (C.c_int32 * max(len(network), 1))(*[len(g) for g in network])
    return arr, lpg, len(network), keep


_lib = None
_cuda_lib = None


def available() -> bool:
    return os.path.exists(_LIB_PATH)


def drop_in_available() -> bool:
    return os.path.exists(_CUDA_LIB_PATH)


def cuda_lib():
    """The harness build that also carries the C++ drop-in CUDA engine. Meshes are created by the library that uses
    them: a RefMesh made with cuda=True lives in this one."""
    global _cuda_lib
    if _cuda_lib is None:
        _cuda_lib = _declare(C.CDLL(_CUDA_LIB_PATH))
    return _cuda_lib


def lib():
    global _lib
    if _lib is None:
        _lib = _declare(C.CDLL(_LIB_PATH))
    return _lib


def _declare(l):
    l.vmref_last_error.restype = C.c_char_p
    l.vmref_mesh_create.restype = C.c_void_p
    l.vmref_mesh_create.argtypes = [C.c_char_p, C.c_char_p] + [C.c_float] * 5
    l.vmref_mesh_destroy.argtypes = [C.c_void_p]
    for name in ("vmref_mesh_n_nodes", "vmref_mesh_n_neighbours", "vmref_mesh_n_bsp"):
        getattr(l, name).argtypes = [C.c_void_p]
        getattr(l, name).restype = C.c_int
    l.vmref_mesh_nodes.argtypes = [C.c_void_p] * 3
    l.vmref_mesh_bsp.argtypes = [C.c_void_p] * 4
    l.vmref_mesh_lookup.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(CLens), C.c_void_p, C.c_int]
    l.vmref_project.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(CLens), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
    l.vmref_classify.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(CLens), C.c_void_p, C.c_uint32,
                                 C.POINTER(CLayer), C.POINTER(C.c_int32), C.c_int,
                                 C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                 C.POINTER(C.c_int)]
    if hasattr(l, "vmref_cuda_classify"):
        l.vmref_cuda_classify.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(CLens), C.c_void_p, C.c_uint32,
                                          C.POINTER(CLayer), C.POINTER(C.c_int32), C.c_int, C.c_int,
                                          C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                          C.POINTER(C.c_int)]
    l.vmref_project_rays.argtypes = [C.c_void_p, C.c_int, C.POINTER(CLens), C.c_void_p]
    l.vmref_interpolate.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_uint32, C.c_void_p]
    l.vmref_run_stream.restype = C.c_double
    l.vmref_run_stream.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                   C.POINTER(CLayer), C.POINTER(C.c_int32), C.c_int, C.c_int,
                                   C.POINTER(C.c_longlong)]
    return l


class RefMesh:
    """visualmesh::Mesh<float, Model> of the reference. with_drop_in=True builds it inside the harness that also
    carries the C++ drop-in CUDA engine, so that both engines can be called on this one object."""

    def __init__(self, spec, with_drop_in=False):
        self.spec = spec
        self._l = cuda_lib() if with_drop_in else lib()
        self.ptr = self._l.vmref_mesh_create(spec.model.encode(), spec.shape.encode(), spec.shape_a, spec.shape_b,
                                           spec.h, spec.k, spec.max_distance)
        if not self.ptr:
            raise RuntimeError(self._l.vmref_last_error().decode())
        self.n_nodes = self._l.vmref_mesh_n_nodes(self.ptr)
        self.n_neighbours = self._l.vmref_mesh_n_neighbours(self.ptr)
        self._nodes = None

    def __del__(self):
        if getattr(self, "ptr", None):
            self._l.vmref_mesh_destroy(self.ptr)
            self.ptr = None

    def nodes(self):
        if self._nodes is None:
            rays = np.empty((self.n_nodes, 3), dtype=np.float32)
            nbrs = np.empty((self.n_nodes, self.n_neighbours), dtype=np.int32)
            self._l.vmref_mesh_nodes(self.ptr, rays.ctypes.data, nbrs.ctypes.data)
            self._nodes = (rays, nbrs)
        return self._nodes

    def bsp(self):
        n = self._l.vmref_mesh_n_bsp(self.ptr)
        ranges = np.empty((n, 2), dtype=np.int32)
        children = np.empty((n, 2), dtype=np.int32)
        cones = np.empty((n, 5), dtype=np.float32)
        self._l.vmref_mesh_bsp(self.ptr, ranges.ctypes.data, children.ctypes.data, cones.ctypes.data)
        return ranges, children, cones

    def lookup(self, Hoc, lens):
        Hoc = np.ascontiguousarray(Hoc, dtype=np.float32)
        cap = 1 << 16
        ranges = np.empty((cap, 2), dtype=np.int32)
        n = self._l.vmref_mesh_lookup(self.ptr, Hoc.ctypes.data, C.byref(c_lens(lens)), ranges.ctypes.data, cap)
        if n < 0:
            raise RuntimeError(self._l.vmref_last_error().decode())
        assert n <= cap
        return ranges[:n].copy()

    def _outputs(self, n_classes_max):
        cap = self.n_nodes
        px = np.empty((cap, 2), dtype=np.float32)
        nb = np.empty((cap + 1, self.n_neighbours), dtype=np.int32)
        gi = np.empty((cap,), dtype=np.int32)
        cl = np.empty(((cap + 1) * max(n_classes_max, 1),), dtype=np.float32)
        return cap, px, nb, gi, cl

    def project(self, Hoc, lens):
        Hoc = np.ascontiguousarray(Hoc, dtype=np.float32)
        cap, px, nb, gi, _ = self._outputs(0)
        n = self._l.vmref_project(self.ptr, Hoc.ctypes.data, C.byref(c_lens(lens)), px.ctypes.data, nb.ctypes.data,
                                gi.ctypes.data, cap)
        if n < 0:
            raise RuntimeError(self._l.vmref_last_error().decode())
        return dict(pixel_coordinates=px[:n].copy(), neighbourhood=nb[:n + 1].copy(), global_indices=gi[:n].copy())

    def classify(self, network, Hoc, lens, image, fmt, cuda=False, project_only=False):
        """cpu::Engine (or, with cuda=True, the drop-in cuda::Engine) on this reference Mesh object."""
        Hoc = np.ascontiguousarray(Hoc, dtype=np.float32)
        image = np.ascontiguousarray(image, dtype=np.uint8)
        layers, lpg, n_groups, keep = c_network(network)
        n_out = network[-1][-1].biases.shape[0] if network else 0
        cap, px, nb, gi, cl = self._outputs(n_out)
        ncls = C.c_int(0)
        if cuda:
            n = self._l.vmref_cuda_classify(self.ptr, Hoc.ctypes.data, C.byref(c_lens(lens)), image.ctypes.data, fmt,
                                          layers, lpg, n_groups, int(project_only), px.ctypes.data, nb.ctypes.data,
                                          gi.ctypes.data, cl.ctypes.data, cap, cl.size, C.byref(ncls))
        else:
            n = self._l.vmref_classify(self.ptr, Hoc.ctypes.data, C.byref(c_lens(lens)), image.ctypes.data, fmt,
                                     layers, lpg, n_groups, px.ctypes.data, nb.ctypes.data, gi.ctypes.data,
                                     cl.ctypes.data, cap, cl.size, C.byref(ncls))
        if n < 0:
            raise RuntimeError(self._l.vmref_last_error().decode())
        k = ncls.value
        if n == 0:
            return dict(pixel_coordinates=px[:0], neighbourhood=nb[:0], global_indices=gi[:0],
                        classifications=np.empty((0, n_out), np.float32))
        return dict(pixel_coordinates=px[:n].copy(), neighbourhood=nb[:n + 1].copy(), global_indices=gi[:n].copy(),
                    classifications=cl[:(n + 1) * k].reshape(n + 1, k).copy())


def project_rays(rays, lens):
    rays = np.ascontiguousarray(rays, dtype=np.float32)
    px = np.empty((rays.shape[0], 2), dtype=np.float32)
    if lib().vmref_project_rays(rays.ctypes.data, rays.shape[0], C.byref(c_lens(lens)), px.ctypes.data) != 0:
        raise RuntimeError(lib().vmref_last_error().decode())
    return px


def interpolate(px, image, width, height, fmt):
    px = np.ascontiguousarray(px, dtype=np.float32)
    image = np.ascontiguousarray(image, dtype=np.uint8)
    out = np.empty((px.shape[0], 4), dtype=np.float32)
    if lib().vmref_interpolate(px.ctypes.data, px.shape[0], image.ctypes.data, width, height, fmt,
                               out.ctypes.data) != 0:
        raise RuntimeError(lib().vmref_last_error().decode())
    return out


def run_stream(meshes, Hocs, lenses, images, formats, network, n_threads):
    """Timed CPU baseline. Returns (seconds, total on-screen points)."""
    n = len(meshes)
    mesh_ptrs = (C.c_void_p * n)(*[m.ptr for m in meshes])
    H = np.ascontiguousarray(np.stack(Hocs), dtype=np.float32)
    L = (CLens * n)(*[c_lens(l) for l in lenses])
    imgs = [np.ascontiguousarray(i, dtype=np.uint8) for i in images]
    img_ptrs = (C.c_void_p * n)(*[i.ctypes.data for i in imgs])
    fmts = (C.c_uint32 * n)(*formats)
    layers, lpg, n_groups, keep = c_network(network)
    total = C.c_longlong(0)
    secs = lib().vmref_run_stream(mesh_ptrs, H.ctypes.data, L, img_ptrs, fmts, n, layers, lpg, n_groups, n_threads,
                                  C.byref(total))
    if secs < 0:
        raise RuntimeError("reference engine threw")
    return secs, total.value

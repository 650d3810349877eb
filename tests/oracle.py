"""ctypes front end of oracle/libvmoracle.so - the plain-C restatement of the reference CPU path.

Test infrastructure only: imported by tests/, the smoke check and the CPU-baseline leg of bench.py.
"""
import ctypes as C
import os

import numpy as np

from refharness import CLayer, CLens, c_lens, c_network

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "..", "oracle", "libvmoracle.so")
_lib = None


def available() -> bool:
    return os.path.exists(_LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        l = C.CDLL(_LIB_PATH)
        l.vmo_project_rays.argtypes = [C.c_void_p, C.c_int, C.POINTER(CLens), C.c_void_p]
        l.vmo_unproject.argtypes = [C.c_void_p, C.c_int, C.POINTER(CLens), C.c_void_p]
        l.vmo_lookup.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p,
                                 C.POINTER(CLens), C.c_void_p, C.c_int]
        l.vmo_project_mesh.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                                       C.POINTER(CLens), C.c_void_p, C.c_void_p, C.c_void_p]
        l.vmo_interpolate.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_uint32, C.c_void_p]
        l.vmo_network.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.POINTER(CLayer), C.POINTER(C.c_int32),
                                  C.c_int, C.c_void_p]
        l.vmo_classify.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                                   C.POINTER(CLens), C.c_void_p, C.c_uint32, C.POINTER(CLayer), C.POINTER(C.c_int32),
                                   C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_int)]
        _lib = l
    return _lib


def project_rays(rays, lens):
    rays = np.ascontiguousarray(rays, dtype=np.float32)
    px = np.empty((rays.shape[0], 2), dtype=np.float32)
    if lib().vmo_project_rays(rays.ctypes.data, rays.shape[0], C.byref(c_lens(lens)), px.ctypes.data) != 0:
        raise RuntimeError("Cannot project: Unknown lens type")
    return px


def lookup(rays, bsp, Hoc, lens):
    rays = np.ascontiguousarray(rays, dtype=np.float32)
    b_ranges, b_children, b_cones = [np.ascontiguousarray(a) for a in bsp]
    Hoc = np.ascontiguousarray(Hoc, dtype=np.float32)
    cap = 1 << 16
    out = np.empty((cap, 2), dtype=np.int32)
    n = lib().vmo_lookup(rays.ctypes.data, b_ranges.ctypes.data, b_children.ctypes.data, b_cones.ctypes.data,
                         b_ranges.shape[0], Hoc.ctypes.data, C.byref(c_lens(lens)), out.ctypes.data, cap)
    if n < 0:
        raise RuntimeError("Unknown lens type")
    assert n <= cap
    return out[:n].copy()


def project_mesh(rays, nbrs, ranges, Hoc, lens):
    rays = np.ascontiguousarray(rays, dtype=np.float32)
    nbrs = np.ascontiguousarray(nbrs, dtype=np.int32)
    ranges = np.ascontiguousarray(ranges, dtype=np.int32).reshape(-1, 2)
    Hoc = np.ascontiguousarray(Hoc, dtype=np.float32)
    m = int((ranges[:, 1] - ranges[:, 0]).sum()) if len(ranges) else 0
    N = nbrs.shape[1]
    px = np.empty((m, 2), dtype=np.float32)
    gi = np.empty((m,), dtype=np.int32)
    nb = np.empty((m + 1, N), dtype=np.int32)
    n = lib().vmo_project_mesh(rays.ctypes.data, nbrs.ctypes.data, rays.shape[0], N, ranges.ctypes.data,
                               ranges.shape[0], Hoc.ctypes.data, C.byref(c_lens(lens)), px.ctypes.data,
                               gi.ctypes.data, nb.ctypes.data)
    if n < 0:
        raise RuntimeError("Cannot project: Unknown lens type")
    return dict(pixel_coordinates=px[:n].copy(), neighbourhood=nb[:n + 1].copy(), global_indices=gi[:n].copy())


def interpolate(px, image, width, height, fmt):
    px = np.ascontiguousarray(px, dtype=np.float32)
    image = np.ascontiguousarray(image, dtype=np.uint8)
    out = np.empty((px.shape[0], 4), dtype=np.float32)
    if lib().vmo_interpolate(px.ctypes.data, px.shape[0], image.ctypes.data, width, height, fmt,
                             out.ctypes.data) != 0:
        raise RuntimeError("Unsupported image format")
    return out


def network(inputs, neighbourhood, net):
    inputs = np.ascontiguousarray(inputs, dtype=np.float32)
    neighbourhood = np.ascontiguousarray(neighbourhood, dtype=np.int32)
    layers, lpg, n_groups, keep = c_network(net)
    n_rows = inputs.shape[0]
    max_w = max([4] + [l.biases.shape[0] for g in net for l in g])
    out = np.empty((n_rows * max_w,), dtype=np.float32)
    w = lib().vmo_network(inputs.ctypes.data, neighbourhood.ctypes.data, n_rows, neighbourhood.shape[1], layers, lpg,
                          n_groups, out.ctypes.data)
    if w < 0:
        raise RuntimeError("network shapes do not chain")
    return out[:n_rows * w].reshape(n_rows, w).copy()


def classify(rays, nbrs, ranges, net, Hoc, lens, image, fmt):
    rays = np.ascontiguousarray(rays, dtype=np.float32)
    nbrs = np.ascontiguousarray(nbrs, dtype=np.int32)
    ranges = np.ascontiguousarray(ranges, dtype=np.int32).reshape(-1, 2)
    Hoc = np.ascontiguousarray(Hoc, dtype=np.float32)
    image = np.ascontiguousarray(image, dtype=np.uint8)
    m = int((ranges[:, 1] - ranges[:, 0]).sum()) if len(ranges) else 0
    N = nbrs.shape[1]
    layers, lpg, n_groups, keep = c_network(net)
    n_out = max([4] + [l.biases.shape[0] for g in net for l in g])
    px = np.empty((m, 2), dtype=np.float32)
    gi = np.empty((m,), dtype=np.int32)
    nb = np.empty((m + 1, N), dtype=np.int32)
    cl = np.empty(((m + 1) * n_out,), dtype=np.float32)
    ncls = C.c_int(0)
    n = lib().vmo_classify(rays.ctypes.data, nbrs.ctypes.data, rays.shape[0], N, ranges.ctypes.data, ranges.shape[0],
                           Hoc.ctypes.data, C.byref(c_lens(lens)), image.ctypes.data, fmt, layers, lpg, n_groups,
                           px.ctypes.data, gi.ctypes.data, nb.ctypes.data, cl.ctypes.data, C.byref(ncls))
    if n < 0:
        raise RuntimeError("oracle failed: unknown lens, format or network shape")
    k = ncls.value
    if n == 0:
        return dict(pixel_coordinates=px[:0], neighbourhood=nb[:0], global_indices=gi[:0],
                    classifications=np.empty((0, k), np.float32))
    return dict(pixel_coordinates=px[:n].copy(), neighbourhood=nb[:n + 1].copy(), global_indices=gi[:n].copy(),
                classifications=cl[:(n + 1) * k].reshape(n + 1, k).copy())

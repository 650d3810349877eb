"""Host-side mirror of the reference's engine interface on top of the C ABI.

Same names and argument meaning as the reference (cpp/visualmesh/engine/cpu/engine.hpp):

    engine = Engine(structure)                              # Engine(const NetworkStructure<float>&)   :57
    projected = engine(mesh, Hoc, lens)                     # operator()(mesh, Hoc, lens)               :85-87
    classified = engine(mesh, Hoc, lens, image, format)     # operator()(mesh, Hoc, lens, image, fmt)   :181-185

`mesh` is a Mesh (one camera height) or a VisualMesh (a table of heights; the engine picks height(Hoc[2][3]) as
:160-165 and :289-296 do). Results carry the reference's four arrays with the reference's lengths: n pixel
coordinates and global indices, n + 1 neighbourhood and classification rows (the last is the off-screen row).
Errors the reference throws as exceptions are raised as VisualMeshError. Nothing here computes: every call goes to
libvmcuda.so, and a missing library or GPU is an error, not a fallback.
"""
import ctypes as C
import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from . import abi
from .abi import VisualMeshError  # noqa: F401  (re-export)
from .workloads import Lens


def _c_lens(lens) -> abi.vm_lens:
    out = abi.vm_lens()
    out.dimensions[0], out.dimensions[1] = int(lens.dimensions[0]), int(lens.dimensions[1])
    out.projection = int(lens.projection)
    out.focal_length = float(lens.focal_length)
    out.centre[0], out.centre[1] = float(lens.centre[0]), float(lens.centre[1])
    out.k[0], out.k[1] = float(lens.k[0]), float(lens.k[1])
    out.fov = float(lens.fov)
    return out


class Mesh:
    """visualmesh::Mesh<float, Model> (cpp/visualmesh/mesh.hpp:56): nodes in BSP order, the BSP, lookup()."""

    def __init__(self, model: str, shape: str, shape_a: float, shape_b: float, h: float, k: float,
                 max_distance: float):
        lib = abi.load()
        ptr = C.c_void_p()
        abi.check(lib.vm_hostmesh_create(model.encode(), shape.encode(), shape_a, shape_b, h, k, max_distance,
                                         C.byref(ptr)))
        self._ptr = ptr
        self.h = float(h)
        self.max_distance = float(max_distance)
        self.n_nodes = lib.vm_hostmesh_n_nodes(ptr)
        self.n_neighbours = lib.vm_hostmesh_n_neighbours(ptr)
        self.rays = np.empty((self.n_nodes, 3), dtype=np.float32)
        self.neighbours = np.empty((self.n_nodes, self.n_neighbours), dtype=np.int32)
        abi.check(lib.vm_hostmesh_nodes(ptr, self.rays.ctypes.data, self.neighbours.ctypes.data))
        n_bsp = lib.vm_hostmesh_n_bsp(ptr)
        self.bsp_ranges = np.empty((n_bsp, 2), dtype=np.int32)
        self.bsp_children = np.empty((n_bsp, 2), dtype=np.int32)
        self.bsp_cones = np.empty((n_bsp, 5), dtype=np.float32)
        abi.check(lib.vm_hostmesh_bsp(ptr, self.bsp_ranges.ctypes.data, self.bsp_children.ctypes.data,
                                      self.bsp_cones.ctypes.data))

    @classmethod
    def from_spec(cls, spec):
        return cls(spec.model, spec.shape, spec.shape_a, spec.shape_b, spec.h, spec.k, spec.max_distance)

    @classmethod
    def from_arrays(cls, rays, neighbours, bsp=None, h=0.0, max_distance=0.0):
        """A mesh whose tables were built elsewhere (for example dumped from the reference's Mesh object)."""
        self = cls.__new__(cls)
        self._ptr = None
        self.h, self.max_distance = float(h), float(max_distance)
        self.rays = np.ascontiguousarray(rays, dtype=np.float32)
        self.neighbours = np.ascontiguousarray(neighbours, dtype=np.int32)
        self.n_nodes, self.n_neighbours = self.neighbours.shape
        if bsp is not None:
            self.bsp_ranges = np.ascontiguousarray(bsp[0], dtype=np.int32)
            self.bsp_children = np.ascontiguousarray(bsp[1], dtype=np.int32)
            self.bsp_cones = np.ascontiguousarray(bsp[2], dtype=np.float32)
        else:
            self.bsp_ranges = self.bsp_children = self.bsp_cones = None
        return self

    def __del__(self):
        if getattr(self, "_ptr", None):
            try:
                abi.load().vm_hostmesh_destroy(self._ptr)
            except Exception:
                pass
            self._ptr = None

    def lookup(self, Hoc, lens) -> np.ndarray:
        """Mesh::lookup on the host (cpp/visualmesh/mesh.hpp:499-595): [start, end) index ranges on screen."""
        if self._ptr is None:
            raise VisualMeshError(abi.VM_ERR_NO_BSP, "this mesh was made from arrays: it has no host lookup")
        Hoc = np.ascontiguousarray(Hoc, dtype=np.float32)
        cap = 4096
        while True:
            out = np.empty((cap, 2), dtype=np.int32)
            n = C.c_int32(0)
            abi.check(abi.load().vm_hostmesh_lookup(self._ptr, Hoc.ctypes.data, C.byref(_c_lens(lens)),
                                                    out.ctypes.data, cap, C.byref(n)))
            if n.value <= cap:
                return out[:n.value].copy()
            cap = n.value


class VisualMesh:
    """visualmesh::VisualMesh<float, Model> (cpp/visualmesh/visualmesh.hpp:65-135): meshes for a range of camera
    heights, bisected until neighbouring heights differ by less than max_error intersections; height() returns the
    nearest."""

    def __init__(self, model, shape, shape_a, shape_b, min_height, max_height, k, max_error, max_distance):
        f = np.float32
        self._args = (model, shape, shape_a, shape_b)
        self.luts = {}
        make = lambda h: Mesh(model, shape, shape_a, shape_b, float(h), k, max_distance)
        self.luts[f(min_height)] = make(min_height)
        self.luts[f(max_height)] = make(max_height)
        stack = [(f(min_height), f(max_height))]
        while stack:
            lo, hi = stack.pop()
            h = f((lo + hi) / f(2))
            lower_err = abs(f(k) - f(k) * self._shape_k(lo, h))
            upper_err = abs(f(k) - f(k) * self._shape_k(hi, h))
            if lower_err > max_error or upper_err > max_error:
                self.luts[h] = make(h)
                stack.append((lo, h))
                stack.append((h, hi))
        self._heights = sorted(self.luts)

    def _shape_k(self, h0, h1):
        f = np.float32
        _, shape, a, b = self._args
        a, b = f(a), f(b)
        if shape == "SPHERE":  # cpp/visualmesh/geometry/Sphere.hpp:106-108
            return (np.log(f(h1 - 2 * a)) - np.log(f(h1))) / (np.log(f(h0 - 2 * a)) - np.log(f(h0)))
        if shape == "CIRCLE":  # cpp/visualmesh/geometry/Circle.hpp:106-108
            return f(h0) / f(h1)
        half = f(b * f(0.5))
        return (f(h0) - half) / (f(h1) - half)

    def height(self, h) -> Mesh:
        hs = self._heights
        h = np.float32(h)
        i = int(np.searchsorted(np.array(hs, dtype=np.float32), h, side="left"))  # lower_bound
        if i == 0:
            return self.luts[hs[0]]
        if i == len(hs):
            return self.luts[hs[-1]]
        return self.luts[hs[i]] if abs(hs[i] - h) < abs(hs[i - 1] - h) else self.luts[hs[i - 1]]


@dataclass
class ProjectedMesh:
    """visualmesh::ProjectedMesh (cpp/visualmesh/projected_mesh.hpp:33-42)"""
    pixel_coordinates: np.ndarray
    neighbourhood: np.ndarray
    global_indices: np.ndarray


@dataclass
class ClassifiedMesh(ProjectedMesh):
    """visualmesh::ClassifiedMesh (cpp/visualmesh/classified_mesh.hpp:38-49)"""
    classifications: np.ndarray = None


@dataclass
class FrameInput:
    mesh: Mesh
    Hoc: np.ndarray
    lens: Lens
    image: object = None           # numpy uint8 array (host), or an int device pointer with image_on_device
    format: int = 0
    ranges: Optional[np.ndarray] = None  # None: lookup on the device
    image_on_device: bool = False


class BatchResult:
    """Results of Engine.run_batch: per-frame views into the engine's pinned buffers (valid until its next call),
    or device pointers when the batch was run with results_on_device."""

    def __init__(self, raw: abi.vm_batch_result):
        self.raw = raw
        self.n_frames = raw.n_frames
        self.n_neighbours = raw.n_neighbours
        self.n_classes = raw.n_classes
        self.on_device = bool(raw.on_device)
        self.offsets = np.ctypeslib.as_array(raw.offsets, shape=(raw.n_frames + 1,)).copy()
        self.total_points = int(self.offsets[-1])
        if not self.on_device:
            total, rows = self.total_points, self.total_points + self.n_frames
            N, Cn = self.n_neighbours, self.n_classes
            self._px = np.ctypeslib.as_array(raw.pixel_coordinates, shape=(max(total, 1), 2))[:total]
            self._gi = np.ctypeslib.as_array(raw.global_indices, shape=(max(total, 1),))[:total]
            self._nb = np.ctypeslib.as_array(raw.neighbourhood, shape=(rows, N))
            self._cls = np.ctypeslib.as_array(raw.classifications, shape=(rows, Cn)) if Cn > 0 else None

    def frame(self, f: int, copy: bool = True):
        if self.on_device:
            raise VisualMeshError(abi.VM_ERR_INVALID_ARGUMENT, "results were left on the device")
        p0, p1 = int(self.offsets[f]), int(self.offsets[f + 1])
        r0, r1 = p0 + f, p1 + f + 1
        cp = (lambda a: a.copy()) if copy else (lambda a: a)
        if p1 == p0:
            # the reference returns a default-constructed (empty) result, cpp/visualmesh/engine/cpu/engine.hpp:193
            empty = ProjectedMesh(np.empty((0, 2), np.float32), np.empty((0, self.n_neighbours), np.int32),
                                  np.empty((0,), np.int32))
            if self._cls is None:
                return empty
            return ClassifiedMesh(empty.pixel_coordinates, empty.neighbourhood, empty.global_indices,
                                  np.empty((0, self.n_classes), np.float32))
        if self._cls is None:
            return ProjectedMesh(cp(self._px[p0:p1]), cp(self._nb[r0:r1]), cp(self._gi[p0:p1]))
        return ClassifiedMesh(cp(self._px[p0:p1]), cp(self._nb[r0:r1]), cp(self._gi[p0:p1]), cp(self._cls[r0:r1]))


class Engine:
    """visualmesh::engine::cuda::Engine<float>: the reference engine interface backed by the sm_100a kernels."""

    def __init__(self, structure=None, device: int = -1, max_cached_meshes: Optional[int] = None):
        """max_cached_meshes: keep at most this many meshes on the device, releasing the least recently used one
        (None = unbounded, like the OpenCL engine's grow-only cache). A prepared batch refers to device meshes by
        handle: with a bound, prepare it again after other meshes have gone through the engine."""
        self._lib = abi.load()
        self._max_cached_meshes = max_cached_meshes
        self._ptr = None
        structure = structure or []
        flat = [layer for group in structure for layer in group]
        layers = (abi.vm_layer * max(len(flat), 1))()
        keep = []
        for i, layer in enumerate(flat):
            w = np.ascontiguousarray(layer.weights, dtype=np.float32)
            b = np.ascontiguousarray(layer.biases, dtype=np.float32)
            if w.ndim != 2 or b.ndim != 1 or w.shape[1] != b.shape[0]:
                raise VisualMeshError(abi.VM_ERR_NETWORK_SHAPE, "weights must be [n_in][n_out] and biases [n_out]")
            keep += [w, b]
            layers[i].weights, layers[i].biases = w.ctypes.data, b.ctypes.data
            layers[i].n_in, layers[i].n_out = w.shape
            layers[i].activation = int(layer.activation)
        lpg = (C.c_int32 * max(len(structure), 1))(*[len(g) for g in structure])
        ptr = C.c_void_p()
        abi.check(self._lib.vm_engine_create(device, layers, lpg, len(structure), C.byref(ptr)))
        self._ptr = ptr
        self._meshes = {}  # id(mesh) -> (mesh, device handle): the cache the OpenCL engine keeps per &mesh
        self.n_classes = flat[-1].biases.shape[0] if flat else 0

    def close(self):
        if self._ptr:
            self._lib.vm_engine_destroy(self._ptr)
            self._ptr = None
            self._meshes = {}

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def clear_cache(self):
        """cpp/visualmesh/engine/opencl/engine.hpp:559-572"""
        for _, handle in self._meshes.values():
            self._lib.vm_mesh_release(self._ptr, handle)
        self._meshes = {}

    def _device_mesh(self, mesh: Mesh):
        hit = self._meshes.get(id(mesh))
        if hit is not None:
            self._meshes[id(mesh)] = self._meshes.pop(id(mesh))  # most recently used goes last
            return hit[1]
        handle = C.c_void_p()
        abi.check(self._lib.vm_mesh_upload(self._ptr, mesh.rays.ctypes.data, mesh.neighbours.ctypes.data,
                                           mesh.n_nodes, mesh.n_neighbours, C.byref(handle)))
        if mesh.bsp_ranges is not None:
            abi.check(self._lib.vm_mesh_set_bsp(self._ptr, handle, mesh.bsp_ranges.shape[0],
                                                mesh.bsp_ranges.ctypes.data, mesh.bsp_children.ctypes.data,
                                                mesh.bsp_cones.ctypes.data))
        self._meshes[id(mesh)] = (mesh, handle)
        while self._max_cached_meshes and len(self._meshes) > self._max_cached_meshes:
            oldest = next(iter(self._meshes))
            self._lib.vm_mesh_release(self._ptr, self._meshes.pop(oldest)[1])
        return handle

    def prepare_batch(self, frames: Sequence[FrameInput]):
        """Marshals frames into the C ABI's vm_frame array once; the result can be run many times with run_prepared
        (a stream of batches re-uses its frame descriptors instead of rebuilding them per call)."""
        n = len(frames)
        arr = (abi.vm_frame * max(n, 1))()
        keep = []
        for i, fr in enumerate(frames):
            mesh = fr.mesh.height(fr.Hoc[2][3]) if isinstance(fr.mesh, VisualMesh) else fr.mesh
            arr[i].mesh = self._device_mesh(mesh)
            if fr.ranges is not None:
                r = np.ascontiguousarray(fr.ranges, dtype=np.int32).reshape(-1, 2)
                keep.append(r)
                # a non-null pointer even for zero ranges: NULL means "look up on the device"
                arr[i].ranges = r.ctypes.data if r.shape[0] > 0 else C.addressof(arr)
                arr[i].n_ranges = r.shape[0]
            H = np.ascontiguousarray(fr.Hoc, dtype=np.float32).reshape(16)
            for j in range(16):
                arr[i].Hoc[j] = float(H[j])
            arr[i].lens = _c_lens(fr.lens)
            if fr.image is not None:
                if fr.image_on_device:
                    arr[i].image = int(fr.image)
                    arr[i].image_on_device = 1
                else:
                    img = fr.image if isinstance(fr.image, np.ndarray) and fr.image.flags["C_CONTIGUOUS"] \
                        and fr.image.dtype == np.uint8 else np.ascontiguousarray(fr.image, dtype=np.uint8)
                    keep.append(img)
                    arr[i].image = img.ctypes.data
                arr[i].format = int(fr.format)
        return (arr, n, keep)

    def run_prepared(self, prepared, results_on_device=False, time_stages=False, raw=False):
        arr, n, _ = prepared
        flags = (abi.VM_RESULTS_ON_DEVICE if results_on_device else 0) | (abi.VM_TIME_STAGES if time_stages else 0)
        res = abi.vm_batch_result()
        abi.check(self._lib.vm_run_batch(self._ptr, arr, n, flags, C.byref(res)))
        return res if raw else BatchResult(res)

    def run_batch(self, frames: Sequence[FrameInput], results_on_device=False, time_stages=False) -> BatchResult:
        return self.run_prepared(self.prepare_batch(frames), results_on_device, time_stages)

    def __call__(self, mesh, Hoc, lens, image=None, format=None, ranges="host"):
        """The two reference calls. ranges="host" runs Mesh::lookup on the host as the reference engines do
        (cpp/visualmesh/engine/opencl/engine.hpp:581), ranges="device" walks the BSP on the GPU, or pass the ranges."""
        Hoc = np.asarray(Hoc, dtype=np.float32).reshape(4, 4)
        m = mesh.height(Hoc[2][3]) if isinstance(mesh, VisualMesh) else mesh
        if isinstance(ranges, str):
            r = m.lookup(Hoc, lens) if ranges == "host" else None
        else:
            r = ranges
        if image is not None and self.n_classes == 0:
            raise VisualMeshError(abi.VM_ERR_NETWORK_SHAPE, "this engine was created without a network")
        fr = FrameInput(m, Hoc, lens, image, int(format or 0), r)
        return self.run_batch([fr]).frame(0)

    def stage_times(self):
        """(name, milliseconds) of every kernel of the last run_batch(time_stages=True), in launch order."""
        n = C.c_int32(0)
        abi.check(self._lib.vm_stage_times(self._ptr, None, None, 0, C.byref(n)))
        names = (C.c_char_p * max(n.value, 1))()
        ms = (C.c_float * max(n.value, 1))()
        abi.check(self._lib.vm_stage_times(self._ptr, names, ms, n.value, C.byref(n)))
        return [(names[i].decode(), float(ms[i])) for i in range(n.value)]

    def timer_start(self):
        """Starts the engine's device-side stopwatch (a CUDA event on its own stream)."""
        abi.check(self._lib.vm_timer_start(self._ptr))

    def timer_stop(self) -> float:
        """Milliseconds of device time since timer_start, measured after all of the engine's streams."""
        ms = C.c_float(0)
        abi.check(self._lib.vm_timer_stop(self._ptr, C.byref(ms)))
        return float(ms.value)

    def set_wait_limit(self, polls: int) -> None:
        """Polls one bounded wait of the tensor-core kernels makes before the kernel gives up and the call fails with
        VM_ERR_DEVICE_ABORT (vm_set_wait_limit); 0 makes every such wait give up at once."""
        abi.check(self._lib.vm_set_wait_limit(self._ptr, int(polls)))

    def launch_count(self) -> int:
        return int(self._lib.vm_launch_count(self._ptr))

    # stand-alone stages, for parity tests against the reference function each replaces
    def sample(self, pixel_coordinates, image, width, height, fmt) -> np.ndarray:
        px = np.ascontiguousarray(pixel_coordinates, dtype=np.float32).reshape(-1, 2)
        img = np.ascontiguousarray(image, dtype=np.uint8)
        out = np.empty((px.shape[0], 4), dtype=np.float32)
        abi.check(self._lib.vm_sample(self._ptr, px.ctypes.data, px.shape[0], img.ctypes.data, width, height, fmt,
                                      out.ctypes.data))
        return out

    def network(self, inputs, neighbourhood) -> np.ndarray:
        x = np.ascontiguousarray(inputs, dtype=np.float32).reshape(-1, 4)
        nb = np.ascontiguousarray(neighbourhood, dtype=np.int32)
        out = np.empty((x.shape[0], self.n_classes), dtype=np.float32)
        abi.check(self._lib.vm_network(self._ptr, x.ctypes.data, nb.ctypes.data, x.shape[0], nb.shape[1],
                                       out.ctypes.data))
        return out


def pinned_empty(nbytes: int) -> np.ndarray:
    """A uint8 array in pinned host memory (vm_host_alloc); frames placed here are copied without staging."""
    ptr = C.c_void_p()
    abi.check(abi.load().vm_host_alloc(C.byref(ptr), nbytes))
    buf = (C.c_uint8 * nbytes).from_address(ptr.value)
    return np.ctypeslib.as_array(buf)


def pinned_free(arr) -> None:
    abi.load().vm_host_free(arr.ctypes.data)

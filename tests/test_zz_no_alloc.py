"""vm_project_static: the projection entry point that allocates nothing.

It exists for callers that cannot allocate device memory while running - a camera thread in a fixed-period control
loop (cudaMalloc takes a driver lock and may synchronise the device, which shows up as a missed deadline), or a process
whose GPU memory is already owned by another framework's caching allocator. Its scratch is one ~4.3 MB array inside the
library image, shared by every call, so this test runs two calls in a row (the second on different inputs, finding the
first call's leftovers in the array) and checks each against the ordinary entry point, which uses allocated scratch.
The same kernels run on both paths, so the outputs must be identical bit for bit.

The file name sorts last on purpose: if the shared array broke anything, every other test has already run.
"""
import ctypes as C

import numpy as np
import pytest

import golden_io as G
from visualmesh_b200 import abi
from visualmesh_b200.engine import Engine, FrameInput, Mesh, _c_lens

pytestmark = pytest.mark.gpu


def _static_call(engine, mesh, Hoc, lens, n_nodes, N):
    import torch
    # the caller's own output buffers, sized for the whole mesh (allocated here, not by the entry point)
    px = torch.full((n_nodes, 2), float("nan"), dtype=torch.float32, device="cuda")
    gi = torch.full((n_nodes,), -7, dtype=torch.int32, device="cuda")
    nb = torch.full((n_nodes + 1, N), -7, dtype=torch.int32, device="cuda")
    cnt = torch.full((1,), -7, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    H = np.ascontiguousarray(Hoc, dtype=np.float32)
    n = C.c_int32(-1)
    handle = engine._device_mesh(mesh)
    abi.check(abi.load().vm_project_static(engine._ptr, handle, H.ctypes.data, C.byref(_c_lens(lens)), px.data_ptr(),
                                           gi.data_ptr(), nb.data_ptr(), cnt.data_ptr(), C.byref(n)))
    assert int(cnt.item()) == n.value
    k = n.value
    return px[:k].cpu().numpy(), gi[:k].cpu().numpy(), nb[:k + 1].cpu().numpy(), gi[k:].cpu().numpy()


def _free_device_bytes():
    import torch
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


def test_static_projection_matches_the_allocating_entry_point_twice_in_a_row():
    case = G.Case("ring6_equisolid_rgba")
    engine = Engine()  # projection only
    mesh = Mesh.from_arrays(case.rays, case.nbrs, case.bsp)
    n_nodes, N = case.nbrs.shape
    for fr in (case.frames[1], case.frames[0], case.frames[2]):  # the larger frame first: leftovers beyond n remain
        want = engine.run_batch([FrameInput(mesh, fr["Hoc"], case.lens, None, 0, None)]).frame(0)
        px, gi, nb, untouched = _static_call(engine, mesh, fr["Hoc"], case.lens, n_nodes, N)
        assert gi.shape[0] == want.global_indices.shape[0] == fr["global_indices"].shape[0]
        assert np.array_equal(gi, want.global_indices)
        assert np.array_equal(nb, want.neighbourhood)
        assert np.array_equal(G.bits(px), G.bits(want.pixel_coordinates))
        assert np.all(untouched == -7), "entries past n must be left alone"
        # and both agree with the reference fixture on the on-screen set and the neighbourhood
        assert np.array_equal(gi, fr["global_indices"]) and np.array_equal(nb, fr["neighbourhood"])
    engine.close()


def test_static_projection_allocates_no_device_memory():
    """The property the entry point exists for: with the caller's output buffers in place, the free device memory is
    the same before and after the second and the third call (the first call of a process may load the library's
    kernels, which is why set-up should make it)."""
    import torch
    case = G.Case("ring6_equisolid_rgba")
    engine = Engine()
    mesh = Mesh.from_arrays(case.rays, case.nbrs, case.bsp)
    n_nodes, N = case.nbrs.shape
    handle = engine._device_mesh(mesh)
    px = torch.empty((n_nodes, 2), dtype=torch.float32, device="cuda")
    gi = torch.empty((n_nodes,), dtype=torch.int32, device="cuda")
    nb = torch.empty((n_nodes + 1, N), dtype=torch.int32, device="cuda")
    lens = _c_lens(case.lens)
    lib = abi.load()

    def call(fr):
        H = np.ascontiguousarray(fr["Hoc"], dtype=np.float32)
        n = C.c_int32(-1)
        abi.check(lib.vm_project_static(engine._ptr, handle, H.ctypes.data, C.byref(lens), px.data_ptr(), gi.data_ptr(),
                                        nb.data_ptr(), None, C.byref(n)))
        return n.value

    assert call(case.frames[0]) == len(case.frames[0]["global_indices"])
    free = _free_device_bytes()
    for fr in (case.frames[1], case.frames[2]):
        assert call(fr) == len(fr["global_indices"])
        assert _free_device_bytes() == free, "vm_project_static changed the amount of free device memory"
    engine.close()


def test_static_projection_rejects_what_does_not_fit():
    lib = abi.load()
    engine = Engine()
    n = abi.load().vm_launch_count(engine._ptr)
    big = np.zeros((300000, 3), np.float32)
    big[:, 2] = -1.0
    nbrs = np.full((300000, 6), 300000, np.int32)
    bsp = (np.array([[0, 300000]], np.int32), np.array([[-1, -1]], np.int32), np.array([[0, 0, -1, -1, 0]], np.float32))
    mesh = Mesh.from_arrays(big, nbrs, bsp)
    handle = engine._device_mesh(mesh)
    case = G.Case("ring4_rectilinear_grey")
    H = np.ascontiguousarray(case.frames[0]["Hoc"], dtype=np.float32)
    dummy = C.c_void_p(256)  # never dereferenced: the size check comes first
    status = lib.vm_project_static(engine._ptr, handle, H.ctypes.data, C.byref(_c_lens(case.lens)), dummy, dummy, dummy,
                                   None, None)
    assert status == abi.VM_ERR_INVALID_ARGUMENT
    assert b"VM_STATIC_MAX_NODES" in lib.vm_last_error()
    assert lib.vm_launch_count(engine._ptr) == n, "a rejected call must not launch anything"
    # a mesh without a BSP cannot be looked up on the device
    small = Mesh.from_arrays(case.rays, case.nbrs, None)
    status = lib.vm_project_static(engine._ptr, engine._device_mesh(small), H.ctypes.data, C.byref(_c_lens(case.lens)),
                                   dummy, dummy, dummy, None, None)
    assert status == abi.VM_ERR_NO_BSP
    # a mesh that was uploaded through another engine is refused
    other = Engine()
    foreign = other._device_mesh(Mesh.from_arrays(case.rays, case.nbrs, case.bsp))
    status = lib.vm_project_static(engine._ptr, foreign, H.ctypes.data, C.byref(_c_lens(case.lens)), dummy, dummy, dummy,
                                   None, None)
    assert status == abi.VM_ERR_INVALID_ARGUMENT and b"another engine" in lib.vm_last_error()
    # and so are lens dimensions that are not positive
    bad = _c_lens(case.lens)
    bad.dimensions[0] = 0
    status = lib.vm_project_static(engine._ptr, engine._device_mesh(Mesh.from_arrays(case.rays, case.nbrs, case.bsp)),
                                   H.ctypes.data, C.byref(bad), dummy, dummy, dummy, None, None)
    assert status == abi.VM_ERR_INVALID_ARGUMENT
    assert lib.vm_launch_count(engine._ptr) == n
    other.close()
    engine.close()

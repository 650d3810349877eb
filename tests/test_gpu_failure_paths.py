"""Error paths of the CUDA engine that a host can provoke without faulting, trapping or hanging a GPU. Needs a GPU.

Every device-side loop or wait that depends on data or on another agent is bounded; when the bound runs out the kernel
raises a flag, leaves through its normal tear-down, and the call returns VM_ERR_DEVICE_ABORT. The tests make the bound
run out with well-formed but useless inputs (a BSP with a cycle, a poll limit of zero) and then
use the same engine again.
"""
import os

import numpy as np
import pytest

import golden_io as G
import oracle as O
import parity as P
from visualmesh_b200 import abi
from visualmesh_b200 import workloads as W
from visualmesh_b200.engine import Engine, FrameInput, Mesh, VisualMeshError

pytestmark = pytest.mark.gpu


def _engine_with_env(network, **env):
    old = {k: os.environ.get(k) for k in env}
    os.environ.update({k: str(v) for k, v in env.items()})
    try:
        return Engine(network)
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k)
            else:
                os.environ[k] = v


def _random_rows(n, n_neighbours, seed):
    x = W.uniform(seed, n * 4, -1.0, 1.0).reshape(n, 4).astype(np.float32)
    x[-1] = -1.0
    nb = (W.splitmix64(seed + 1, n * n_neighbours) % np.uint64(n)).astype(np.int32).reshape(n, n_neighbours)
    nb[-1] = n - 1
    return x, nb


def test_bsp_with_a_cycle_stops_after_128_levels():
    """The device lookup follows the BSP between the root and the leaves (cpp/visualmesh/mesh.hpp:559-583). An inner
    element whose children are the root passes the upload's range checks but closes a cycle: the walk stops at its
    depth limit, the call reports VM_ERR_DEVICE_ABORT, and the engine then runs the intact mesh as if nothing had
    happened."""
    case = G.Case("ring6_equisolid_rgba")
    fr = case.frames[0]
    engine = Engine(case.network)
    good = Mesh.from_arrays(case.rays, case.nbrs, case.bsp)
    children = case.bsp[1].copy()
    inner = [i for i in range(1, len(children)) if children[i][0] >= 0]
    children[inner[0]] = (0, 0)
    looped = Mesh.from_arrays(case.rays, case.nbrs, (case.bsp[0], children, case.bsp[2]))
    with pytest.raises(VisualMeshError) as e:
        engine.run_batch([FrameInput(looped, fr["Hoc"], case.lens, fr["image"], case.format, None)])
    assert e.value.status == abi.VM_ERR_DEVICE_ABORT, str(e.value)
    # host ranges do not walk the BSP: the same mesh works with them
    out = engine.run_batch([FrameInput(looped, fr["Hoc"], case.lens, fr["image"], case.format, fr["ranges"])]).frame(0)
    assert P.compare(out, fr, case.lens.dimensions).ok
    out = engine.run_batch([FrameInput(good, fr["Hoc"], case.lens, fr["image"], case.format, None)]).frame(0)
    assert P.compare(out, fr, case.lens.dimensions).ok
    engine.close()


@pytest.mark.parametrize("n_neighbours,widths", [(6, [16, 16, 16, 3]), (8, [32, 32, 32, 4])])
def test_poll_limit_zero_makes_the_tensor_core_kernels_give_up_cleanly(n_neighbours, widths):
    """With a poll limit of zero the MMA issuer gives up before issuing anything and every other role leaves through
    the tear-down (tensor memory freed): VM_ERR_DEVICE_ABORT, no hang. With the limit restored the same engine computes
    the layer correctly."""
    net = W.make_network(31, n_neighbours, widths)
    x, nb = _random_rows(20_000, n_neighbours, 37)
    want = O.network(x, nb, net)
    engine = _engine_with_env(net, VMCUDA_TC=2)
    engine.set_wait_limit(0)
    with pytest.raises(VisualMeshError) as e:
        engine.network(x, nb)
    assert e.value.status == abi.VM_ERR_DEVICE_ABORT, str(e.value)
    engine.set_wait_limit(4_000_000)
    for _ in range(2):
        got = engine.network(x, nb)
        assert np.abs(got.astype(np.float64) - want.astype(np.float64)).max() <= P.TOL_CLS / 4
    engine.close()


def test_fp16_range_overflow_in_an_early_chunk_of_a_batch_is_not_missed():
    """Six one-frame chunks rotate over the engine's three streams. Only the first frame drives a feature beyond the
    range of the fp16 split (its image is bright, the others are black), so the flag is raised by an early chunk while
    later chunks run on other streams. The batch must come back bit for bit as an engine without tensor-core kernels
    computes it."""
    case = G.Case("ring6_equisolid_rgba")
    fr = case.frames[0]
    net = W.make_network(9, 6, [16, 16, 2])
    net[0][0].weights[:] = np.abs(net[0][0].weights) * 3.0e5   # bright pixels -> ~1e5, the off-screen row (-1) -> SELU floor
    net[1][0].weights[:] *= 1.0e-6
    mesh_spec = dict(rays=case.rays, neighbours=case.nbrs, bsp=case.bsp)
    bright = np.full_like(fr["image"], 255)
    black = np.zeros_like(fr["image"])

    def frames(mesh):
        return [FrameInput(mesh, fr["Hoc"], case.lens, bright if f == 0 else black, case.format, None) for f in range(6)]

    plain = _engine_with_env(net, VMCUDA_TC=0, VMCUDA_CHUNK_FRAMES=1)
    want = plain.run_batch(frames(Mesh.from_arrays(**mesh_spec)))
    want = [want.frame(f) for f in range(6)]
    plain.close()
    assert all(np.all(np.isfinite(w.classifications)) for w in want)
    engine = _engine_with_env(net, VMCUDA_TC=2, VMCUDA_CHUNK_FRAMES=1)
    mesh = Mesh.from_arrays(**mesh_spec)
    for _ in range(2):  # the second batch runs on the engine that has already fallen back
        got = engine.run_batch(frames(mesh))
        for f in range(6):
            assert np.array_equal(G.bits(got.frame(f).classifications), G.bits(want[f].classifications)), f"frame {f}"
    engine.close()


def test_layer_without_a_tensor_core_kernel_between_two_that_have_one():
    """8 -> 32 has a tensor-core weight layout but no kernel instantiation: it must run on the FFMA kernels and the
    32 -> 32 layer behind it must still be fed the layout its kernel expects (tensor cores forced on wherever a kernel
    exists)."""
    net = W.make_network(41, 6, [8, 32, 32, 2])
    x, nb = _random_rows(5_000, 6, 43)
    want = O.network(x, nb, net)
    for mode in (0, 1, 2):
        engine = _engine_with_env(net, VMCUDA_TC=mode)
        got = engine.network(x, nb)
        d = np.abs(got.astype(np.float64) - want.astype(np.float64)).max()
        print(f"8->32->32 tensor-core mode {mode}: max |d| = {d:.3g}")
        assert d <= P.TOL_CLS / 4
        engine.close()


def test_sampler_rejects_coordinates_outside_the_image():
    """vm_sample takes its coordinates from the caller; one outside the image (or not finite) would be read outside the
    image buffer on the GPU, so the call is refused on the host and launches nothing."""
    engine = Engine()
    image = W.random_bytes(3, 64 * 48 * 4)
    ok = np.array([[0.0, 0.0], [62.5, 46.5], [63.0, 47.0]], np.float32)
    out = engine.sample(ok[:2], image, 64, 48, W.fourcc("RGBA"))
    assert out.shape == (2, 4) and np.all(np.isfinite(out))
    before = engine.launch_count()
    for bad in ([64.0, 1.0], [1.0, 48.0], [-0.5, 1.0], [np.nan, 1.0], [np.inf, 1.0], [1.0, 1.0e30]):
        px = np.array([[1.0, 1.0], bad], np.float32)
        with pytest.raises(VisualMeshError) as e:
            engine.sample(px, image, 64, 48, W.fourcc("RGBA"))
        assert e.value.status == abi.VM_ERR_INVALID_ARGUMENT
    assert engine.launch_count() == before
    engine.close()


def test_mesh_of_another_engine_is_refused():
    case = G.Case("ring4_rectilinear_grey")
    fr = case.frames[0]
    a, b = Engine(case.network), Engine(case.network)
    mesh = Mesh.from_arrays(case.rays, case.nbrs, case.bsp)
    prepared = a.prepare_batch([FrameInput(mesh, fr["Hoc"], case.lens, fr["image"], case.format, None)])
    with pytest.raises(VisualMeshError) as e:
        b.run_prepared(prepared)
    assert e.value.status == abi.VM_ERR_INVALID_ARGUMENT
    assert P.compare(a.run_prepared(prepared).frame(0), fr, case.lens.dimensions).ok
    a.close()
    b.close()


def test_nvtx_ranges_do_not_change_results():
    """VMCUDA_NVTX=1 wraps every launch and every batch in an NVTX range; with no profiler attached the ranges are
    no-ops and the results are those of an engine without them."""
    case = G.Case("ring6_equisolid_rgba")
    fr = case.frames[0]
    engine = _engine_with_env(case.network, VMCUDA_NVTX=1)
    mesh = Mesh.from_arrays(case.rays, case.nbrs, case.bsp)
    for _ in range(2):
        out = engine.run_batch([FrameInput(mesh, fr["Hoc"], case.lens, fr["image"], case.format, None)]).frame(0)
        assert P.compare(out, fr, case.lens.dimensions).ok
    engine.close()

"""The host mesh tables (vm_hostmesh_*) against the reference's Mesh: nodes, neighbours, BSP and per-frame lookup,
bit for bit - from the golden fixtures everywhere, and from the compiled reference where it is present."""
import math

import numpy as np
import pytest

import golden_io as G
import oracle as O
import refharness as R
from visualmesh_b200 import workloads as W
from visualmesh_b200.engine import Mesh, VisualMesh


@pytest.mark.parametrize("name", G.CASES)
def test_tables_and_lookup_match_the_reference_fixture(name):
    case = G.Case(name)
    mesh = Mesh.from_spec(case.mesh_spec)
    assert mesh.n_nodes == case.rays.shape[0]
    assert np.array_equal(G.bits(mesh.rays), G.bits(case.rays))
    assert np.array_equal(mesh.neighbours, case.nbrs)
    assert np.array_equal(mesh.bsp_ranges, case.bsp[0])
    assert np.array_equal(mesh.bsp_children, case.bsp[1])
    assert np.array_equal(G.bits(mesh.bsp_cones), G.bits(case.bsp[2]))
    for fr in case.frames:
        assert np.array_equal(mesh.lookup(fr["Hoc"], case.lens), fr["ranges"])


def test_bsp_is_a_partition_of_the_nodes():
    mesh = Mesh("RING6", "SPHERE", 0.0949, 0.0, 1.0, 3.0, 10.0)
    r, c = mesh.bsp_ranges, mesh.bsp_children
    assert tuple(r[0]) == (0, mesh.n_nodes)
    leaves = c[:, 0] < 0
    assert np.all((c[:, 0] < 0) == (c[:, 1] < 0))
    # leaves tile [0, n) in order and hold at most 8 nodes (cpp/visualmesh/mesh.hpp:143)
    lr = r[leaves]
    lr = lr[np.argsort(lr[:, 0])]
    assert lr[0, 0] == 0 and lr[-1, 1] == mesh.n_nodes and np.array_equal(lr[1:, 0], lr[:-1, 1])
    assert np.all(lr[:, 1] - lr[:, 0] <= 8)
    inner = np.where(~leaves)[0]
    assert np.array_equal(r[c[inner, 0], 0], r[inner, 0]) and np.array_equal(r[c[inner, 1], 1], r[inner, 1])
    assert np.array_equal(r[c[inner, 0], 1], r[c[inner, 1], 0])
    # every node lies inside the cone of the leaf that holds it
    for e in np.where(leaves)[0][:200]:
        axis, cos_t = mesh.bsp_cones[e, :3], mesh.bsp_cones[e, 3]
        assert np.all(mesh.rays[r[e, 0]:r[e, 1]] @ axis >= cos_t - 1e-5)


def test_neighbour_table_is_in_range_and_mostly_symmetric():
    mesh = Mesh("RING6", "SPHERE", 0.0949, 0.0, 1.0, 3.0, 10.0)
    nb = mesh.neighbours
    assert nb.min() >= 0 and nb.max() <= mesh.n_nodes  # n_nodes = no such node
    # left/right links (columns 0 and 3 of a ring mesh) are mutual everywhere except at the origin node
    valid = nb[:, 0] < mesh.n_nodes
    mutual = nb[nb[valid, 0], 3] == np.where(valid)[0]
    assert mutual.sum() >= mutual.size - 2


def test_oracle_lookup_agrees_with_host_lookup_over_many_poses():
    mesh = Mesh("RING8", "SPHERE", 0.0949, 0.0, 0.9, 3.0, 8.0)
    bsp = (mesh.bsp_ranges, mesh.bsp_children, mesh.bsp_cones)
    lenses = [W.Lens((320, 240), W.EQUISOLID, 100.0, (0, 0), (0, 0), math.pi),
              W.Lens((320, 240), W.EQUIDISTANT, 90.0, (2, -3), (-0.1 / 320**2, 0.02 / 320**4), 2.5),
              W.Lens((320, 240), W.RECTILINEAR, 200.0, (0, 0), (0, 0), 1.6)]
    poses = W.uniform(5, 60).reshape(30, 2)
    for i, (a, b) in enumerate(poses):
        Hoc = W.make_Hoc(math.radians(-90 + 120 * a), math.radians(-20 + 40 * b), 0.9)
        lens = lenses[i % 3]
        assert np.array_equal(mesh.lookup(Hoc, lens), O.lookup(mesh.rays, bsp, Hoc, lens))


def test_visualmesh_height_picks_the_nearest_table():
    vm = VisualMesh("RING6", "SPHERE", 0.0949, 0.0, 0.5, 1.5, 2.0, 0.5, 4.0)
    hs = sorted(vm.luts)
    assert hs[0] == np.float32(0.5) and hs[-1] == np.float32(1.5) and len(hs) >= 3
    assert vm.height(0.1) is vm.luts[hs[0]]
    assert vm.height(9.0) is vm.luts[hs[-1]]
    mid = float(hs[1])
    assert vm.height(mid + 1e-4) is vm.luts[hs[1]]


@pytest.mark.skipif(not R.available(), reason="compiled reference (oracle/_ref/libvmref.so) not present")
@pytest.mark.parametrize("spec", [
    W.MeshSpec("RING6", "SPHERE", 0.0949, 0.0, 1.2, 6.0, 20.0),
    W.MeshSpec("RING8", "SPHERE", 0.0949, 0.0, 1.6, 4.0, 12.0),
    W.MeshSpec("RING4", "CIRCLE", 0.1, 0.0, 1.0, 2.0, 5.0),
    W.MeshSpec("XYGRID6", "CYLINDER", 0.2, 1.8, 1.0, 4.0, 15.0),
    W.MeshSpec("XYGRID8", "CIRCLE", 0.1, 0.0, 1.0, 2.0, 8.0),
    W.MeshSpec("XMGRID6", "SPHERE", 0.1, 0.0, 1.0, 2.0, 8.0),
    W.MeshSpec("XMGRID4", "CIRCLE", 0.1, 0.0, 0.7, 2.0, 6.0),
    W.MeshSpec("NMGRID6", "SPHERE", 0.1, 0.0, 1.0, 2.0, 8.0),
    W.MeshSpec("NMGRID4", "CIRCLE", 0.1, 0.0, 0.7, 2.0, 6.0),
    W.MeshSpec("NMGRID8", "CYLINDER", 0.2, 1.8, 1.0, 2.0, 8.0),
], ids=lambda s: f"{s.model}-{s.shape}")
def test_tables_and_lookup_match_the_compiled_reference(spec):
    ref, own = R.RefMesh(spec), Mesh.from_spec(spec)
    rays, nbrs = ref.nodes()
    b = ref.bsp()
    assert np.array_equal(G.bits(rays), G.bits(own.rays)) and np.array_equal(nbrs, own.neighbours)
    assert np.array_equal(b[0], own.bsp_ranges) and np.array_equal(b[1], own.bsp_children)
    assert np.array_equal(G.bits(b[2]), G.bits(own.bsp_cones))
    for cfg in range(4):
        for fr in W.config(cfg, n_frames=3).frames:
            H = fr.Hoc.copy()
            H[2, 3] = spec.h
            assert np.array_equal(ref.lookup(H, fr.lens), own.lookup(H, fr.lens))

"""Parity of the CUDA engine with the reference CPU engine, through the C ABI. Needs a GPU (-m gpu).

Layers of the check, so that a last-bit difference of a transcendental cannot hide a real defect:
  1. projection alone: on-screen set, neighbourhood, pixel coordinates;
  2. sampler and network alone, fed with the REFERENCE's pixel coordinates and neighbourhood: must match to 1e-4
     (in practice ~1e-6; the only difference is fused multiply-add and the device's expf);
  3. the whole call, host ranges and device lookup, Python front end and the C++ drop-in header.
On uniform-noise images one ulp of a pixel coordinate already moves a classification by more than 1e-4 through an
8-layer network, and the host libm's acosf/sinf/tanf are not correctly rounded. The engine therefore reproduces the
host libm's last bit from tabulated low bits (csrc/libm_tables.hpp); with that the pixel coordinates are expected to be
bit-identical and every check below demands the stated tolerances on every entry.
"""
import numpy as np
import pytest

import golden_io as G
import oracle as O
import parity as P
import refharness as R
from visualmesh_b200 import workloads as W
from visualmesh_b200.engine import Engine, FrameInput, Mesh, VisualMeshError

pytestmark = pytest.mark.gpu


def _mesh_from_case(case):
    return Mesh.from_arrays(case.rays, case.nbrs, case.bsp)


@pytest.fixture(scope="module")
def cases():
    return {name: G.Case(name) for name in G.CASES}


# ---- 1 + 3: golden fixtures, whole call -----------------------------------------------------------------------------

@pytest.mark.parametrize("name", G.CASES)
@pytest.mark.parametrize("lookup", ["host_ranges", "device_lookup"])
def test_golden_whole_call(cases, name, lookup):
    case = cases[name]
    engine = Engine(case.network)
    mesh = _mesh_from_case(case)
    for f, fr in enumerate(case.frames):
        ranges = fr["ranges"] if lookup == "host_ranges" else None
        out = engine.run_batch([FrameInput(mesh, fr["Hoc"], case.lens, fr["image"], case.format, ranges)]).frame(0)
        rep = P.compare(out, fr, case.lens.dimensions)
        print(f"{name}[{f}] {lookup}: {rep}")
        assert rep.projection_ok, str(rep)
        assert rep.n_out == rep.n_ref or rep.border_nodes
        assert rep.ok, str(rep)
    engine.close()


@pytest.mark.parametrize("name", G.CASES)
def test_golden_projection_only(cases, name):
    case = cases[name]
    engine = Engine()
    mesh = _mesh_from_case(case)
    for f, fr in enumerate(case.frames):
        out = engine(mesh, fr["Hoc"], case.lens, ranges=fr["ranges"])
        assert not hasattr(out, "classifications") or out.classifications is None
        rep = P.compare(out, {k: fr[k] for k in ("pixel_coordinates", "neighbourhood", "global_indices")},
                        case.lens.dimensions)
        assert rep.projection_ok, str(rep)
        if len(fr["global_indices"]) == 0:
            assert out.global_indices.size == 0
    engine.close()


# ---- 2: stages alone, identical inputs ------------------------------------------------------------------------------

def test_sampler_bit_exact_for_every_fourcc():
    z, _ = G.units()
    Wd, Ht = [int(v) for v in z["sample_dims"]]
    engine = Engine()
    for code in ["RGGB", "GRBG", "GBRG", "BGGR", "BGR3", "BGR8", "BGRA", "RGB3", "RGB8", "RGBA", "GRAY", "GREY",
                 "Y8  "]:
        out = engine.sample(z["sample_px"], z[f"sample_image_{code.strip()}"], Wd, Ht, W.fourcc(code))
        assert np.array_equal(G.bits(out), G.bits(z[f"sample_out_{code.strip()}"])), code
    engine.close()


@pytest.mark.parametrize("name", G.CASES)
def test_network_on_reference_inputs(cases, name):
    case = cases[name]
    engine = Engine(case.network)
    for f, fr in enumerate(case.frames):
        n = len(fr["global_indices"])
        if n == 0:
            continue
        sampled = engine.sample(fr["pixel_coordinates"], fr["image"], *case.lens.dimensions, case.format)
        want = O.interpolate(fr["pixel_coordinates"], fr["image"], *case.lens.dimensions, case.format)
        assert np.array_equal(G.bits(sampled), G.bits(want)), f"{name}[{f}] sampler"
        inputs = np.concatenate([sampled, -np.ones((1, 4), np.float32)])
        out = engine.network(inputs, fr["neighbourhood"])
        d = np.abs(out.astype(np.float64) - fr["classifications"].astype(np.float64)).max()
        print(f"{name}[{f}] network on reference inputs: max |d| = {d:.3g}")
        assert d <= P.TOL_CLS
    engine.close()


# ---- batches ---------------------------------------------------------------------------------------------------------

def test_batch_equals_single_frames_bit_for_bit(cases):
    case = cases["ring6_equisolid_rgba"]
    engine = Engine(case.network)
    mesh = _mesh_from_case(case)
    frames = []
    for rep in range(3):  # 9 frames, mixing host ranges and device lookup
        for f, fr in enumerate(case.frames):
            frames.append(FrameInput(mesh, fr["Hoc"], case.lens, fr["image"], case.format,
                                     fr["ranges"] if (rep + f) % 2 == 0 else None))
    singles = [engine.run_batch([fr]).frame(0) for fr in frames]
    import os
    os.environ["VMCUDA_CHUNK_FRAMES"] = "2"  # several chunks rotating over the lanes
    engine2 = Engine(case.network)
    os.environ.pop("VMCUDA_CHUNK_FRAMES")
    mesh2 = _mesh_from_case(case)
    frames2 = [FrameInput(mesh2, fr.Hoc, fr.lens, fr.image, fr.format, fr.ranges) for fr in frames]
    for eng, frs in ((engine, frames), (engine2, frames2)):
        batch = eng.run_batch(frs)
        assert batch.n_frames == len(frames)
        for f, single in enumerate(singles):
            got = batch.frame(f)
            for key in ("pixel_coordinates", "global_indices", "neighbourhood", "classifications"):
                assert np.array_equal(G.bits(getattr(got, key)), G.bits(getattr(single, key))), f"frame {f} {key}"
    engine.close()
    engine2.close()


def test_empty_frames_and_empty_ranges(cases):
    case = cases["ring4_rectilinear_grey"]
    engine = Engine(case.network)
    mesh = _mesh_from_case(case)
    fr = case.frames[1]  # camera looks up: nothing on screen
    assert len(fr["global_indices"]) == 0
    for ranges in (fr["ranges"], None):
        out = engine.run_batch([FrameInput(mesh, fr["Hoc"], case.lens, fr["image"], case.format, ranges)]).frame(0)
        assert out.global_indices.size == 0 and out.classifications.size == 0
    # an empty frame between two full ones does not disturb them
    full = case.frames[0]
    batch = engine.run_batch([FrameInput(mesh, full["Hoc"], case.lens, full["image"], case.format, full["ranges"]),
                              FrameInput(mesh, fr["Hoc"], case.lens, fr["image"], case.format, fr["ranges"]),
                              FrameInput(mesh, full["Hoc"], case.lens, full["image"], case.format, None)])
    a, b = batch.frame(0), batch.frame(2)
    assert batch.frame(1).global_indices.size == 0
    assert np.array_equal(a.global_indices, full["global_indices"])
    assert np.array_equal(G.bits(a.classifications), G.bits(b.classifications))
    engine.close()


def test_errors_match_the_reference_conditions(cases):
    case = cases["ring6_equisolid_rgba"]
    engine = Engine(case.network)
    mesh = _mesh_from_case(case)
    fr = case.frames[0]
    with pytest.raises(VisualMeshError) as e:
        engine(mesh, fr["Hoc"], case.lens, fr["image"], W.fourcc("NV12"), ranges=fr["ranges"])
    assert e.value.status == 2 and "Unsupported image format" in str(e.value)
    bad = W.Lens(case.lens.dimensions, 9, case.lens.focal_length)
    with pytest.raises(VisualMeshError) as e:
        engine(mesh, fr["Hoc"], bad, fr["image"], case.format, ranges=fr["ranges"])
    assert e.value.status == 3
    no_bsp = Mesh.from_arrays(case.rays, case.nbrs, None)
    with pytest.raises(VisualMeshError) as e:
        engine.run_batch([FrameInput(no_bsp, fr["Hoc"], case.lens, fr["image"], case.format, None)])
    assert e.value.status == 8
    # the engine is still usable after a failed call
    out = engine(mesh, fr["Hoc"], case.lens, fr["image"], case.format, ranges=fr["ranges"])
    assert np.array_equal(out.global_indices, fr["global_indices"])
    engine.close()


# ---- benchmark configurations against the compiled reference -------------------------------------------------------

needs_ref = pytest.mark.skipif(not R.available(), reason="compiled reference (oracle/_ref/libvmref.so) not present")


def _check_config(cfg, n_frames, via_cpp):
    wl = W.config(cfg, n_frames=n_frames)
    ref_meshes, own_meshes = {}, {}
    engine = Engine(wl.network)
    frames_ok = 0
    for f, fr in enumerate(wl.frames):
        if fr.mesh.key() not in ref_meshes:
            ref_meshes[fr.mesh.key()] = R.RefMesh(fr.mesh, with_drop_in=via_cpp)
        ref_mesh = ref_meshes[fr.mesh.key()]
        image = fr.image()
        ref = ref_mesh.classify(wl.network, fr.Hoc, fr.lens, image, fr.format)
        if via_cpp:
            out = ref_mesh.classify(wl.network, fr.Hoc, fr.lens, image, fr.format, cuda=True)
        else:
            if fr.mesh.key() not in own_meshes:
                own_meshes[fr.mesh.key()] = Mesh.from_spec(fr.mesh)
            out = engine.run_batch([FrameInput(own_meshes[fr.mesh.key()], fr.Hoc, fr.lens, image, fr.format,
                                               None)]).frame(0)
        rep = P.compare(out, ref, fr.lens.dimensions)
        print(f"cfg{cfg}[{f}] {'c++ drop-in' if via_cpp else 'python/C-ABI'}: {rep}")
        assert rep.projection_ok, str(rep)
        assert rep.n_ref > 0
        assert rep.ok, str(rep)
        assert rep.px_bit_identical > 0.999, str(rep)
        frames_ok += rep.ok
    engine.close()
    return frames_ok


@needs_ref
@pytest.mark.parametrize("cfg,n_frames", [(0, 1), (1, 3), (2, 3), (4, 4)])
def test_benchmark_config_vs_compiled_reference(cfg, n_frames):
    _check_config(cfg, n_frames, via_cpp=False)


@needs_ref
@pytest.mark.skipif(not R.drop_in_available(), reason="harness with the CUDA drop-in (oracle/_ref/libvmref_cuda.so) not present")
@pytest.mark.parametrize("cfg,n_frames", [(0, 1), (2, 2)])
def test_cpp_drop_in_engine_vs_cpu_engine_on_the_same_mesh_object(cfg, n_frames):
    _check_config(cfg, n_frames, via_cpp=True)


@needs_ref
def test_config3_dense_mesh_projection_and_two_layers():
    """Config 3's mesh (1.7M nodes, 0.93M on screen) with a cut-down network so the CPU reference finishes quickly."""
    wl = W.config(3, n_frames=1)
    fr = wl.frames[0]
    net = wl.network[:1] + [[W.Layer(wl.network[-1][0].weights, wl.network[-1][0].biases, W.SOFTMAX)]]
    ref_mesh = R.RefMesh(fr.mesh)
    image = fr.image()
    ref = ref_mesh.classify(net, fr.Hoc, fr.lens, image, fr.format)
    engine = Engine(net)
    out = engine.run_batch([FrameInput(Mesh.from_spec(fr.mesh), fr.Hoc, fr.lens, image, fr.format, None)]).frame(0)
    rep = P.compare(out, ref, fr.lens.dimensions)
    print(f"cfg3 (2 layers): {rep}")
    assert rep.ok and rep.n_ref > 900000, str(rep)
    engine.close()


@needs_ref
def test_config3_dense_mesh_through_the_tensor_core_layers():
    """Config 3's frame (0.93M rows = 7280 tiles) through first layer, two 32 -> 32 layers on the tensor cores (default
    policy) and the softmax layer, against the reference CPU engine on the same mesh: the whole call at full size."""
    wl = W.config(3, n_frames=1)
    fr = wl.frames[0]
    net = wl.network[:3] + [[W.Layer(wl.network[-1][0].weights, wl.network[-1][0].biases, W.SOFTMAX)]]
    ref_mesh = R.RefMesh(fr.mesh)
    image = fr.image()
    ref = ref_mesh.classify(net, fr.Hoc, fr.lens, image, fr.format)
    engine = Engine(net)
    out = engine.run_batch([FrameInput(Mesh.from_spec(fr.mesh), fr.Hoc, fr.lens, image, fr.format, None)]).frame(0)
    rep = P.compare(out, ref, fr.lens.dimensions)
    print(f"cfg3 (4 layers, tcgen05): {rep}")
    assert rep.ok and rep.n_ref > 900000, str(rep)
    engine.close()


# ---- the reference's own trained model on its own example frames ----------------------------------------------------

@pytest.mark.parametrize("lookup", ["host_ranges", "device_lookup"])
def test_example_model_on_example_frames(lookup):
    """example/model.yaml (13 groups, 28x16 ... 56x5 softmax, trained weights) on three frames of example/images,
    against the stored outputs of the reference CPU engine - the whole call through the C ABI."""
    case = G.ExampleModelCase()
    mesh = Mesh.from_spec(case.mesh_spec)
    case.check_mesh(mesh.rays, mesh.neighbours)
    engine = Engine(case.network)
    frames = [FrameInput(mesh, fr["Hoc"], fr["lens"], fr["image"], case.format,
                         fr["ranges"] if lookup == "host_ranges" else None) for fr in case.frames]
    singles = [engine.run_batch([f]).frame(0) for f in frames]
    batch = engine.run_batch(frames)
    for f, fr in enumerate(case.frames):
        rep = P.compare(singles[f], fr, fr["lens"].dimensions)
        print(f"example model frame {f} {lookup}: {rep}")
        assert rep.ok and rep.indices_exact and rep.n_ref > 1000, str(rep)
        assert rep.px_bit_identical > 0.999, str(rep)
        assert np.array_equal(G.bits(batch.frame(f).classifications), G.bits(singles[f].classifications))
    engine.close()


@pytest.mark.skipif(not R.drop_in_available(), reason="harness with the CUDA drop-in (oracle/_ref/libvmref_cuda.so) not present")
def test_example_model_through_the_cpp_drop_in_engine():
    """The same case through visualmesh::engine::cuda::Engine<float> on a reference Mesh object."""
    case = G.ExampleModelCase()
    ref_mesh = R.RefMesh(case.mesh_spec, with_drop_in=True)
    case.check_mesh(*ref_mesh.nodes())
    for f, fr in enumerate(case.frames):
        out = ref_mesh.classify(case.network, fr["Hoc"], fr["lens"], fr["image"], case.format, cuda=True)
        rep = P.compare(out, fr, fr["lens"].dimensions)
        print(f"example model frame {f} c++ drop-in: {rep}")
        assert rep.ok and rep.indices_exact, str(rep)


# ---- staged layers (tile plan, shared-memory windows, warp-level MMAs) -----------------------------------------------

@needs_ref
def test_staged_layers_on_the_dense_mesh_with_halo_overflow():
    """A 16-wide network on configuration 3's dense Ring8 mesh (0.93 M rows, 9 slots): a few percent of its 256-row
    super-tiles have more outside rows than halo slots, so staged neighbours and neighbours fetched from global memory
    mix inside one launch. The whole call against the reference CPU engine, and staged against not staged."""
    import os
    wl = W.config(3, n_frames=1)
    fr = wl.frames[0]
    net = W.make_network(29, 8, [16, 16, 8, 2])
    ref_mesh = R.RefMesh(fr.mesh)
    image = fr.image()
    ref = ref_mesh.classify(net, fr.Hoc, fr.lens, image, fr.format)
    mesh = Mesh.from_spec(fr.mesh)
    outs = {}
    for staged in ("1", "0"):
        os.environ["VMCUDA_STAGED"] = staged
        try:
            engine = Engine(net)
        finally:
            os.environ.pop("VMCUDA_STAGED")
        outs[staged] = engine.run_batch([FrameInput(mesh, fr.Hoc, fr.lens, image, fr.format, None)]).frame(0)
        rep = P.compare(outs[staged], ref, fr.lens.dimensions)
        print(f"cfg3 mesh, 16-wide network, staged={staged}: {rep}")
        assert rep.ok and rep.n_ref > 900000, str(rep)
        engine.close()
    d = np.abs(outs["1"].classifications.astype(np.float64) - outs["0"].classifications.astype(np.float64)).max()
    assert d <= P.TOL_CLS / 4


def test_staged_and_unstaged_layers_agree_on_a_batch_of_unequal_frames(cases):
    """Frames of different sizes in one launch (super-tiles never straddle frames; the last super-tile of a frame is
    partial)."""
    import os
    case = cases["ring6_equisolid_rgba"]
    net = W.make_network(33, 6, [16, 16, 16, 8, 3])
    mesh_args = (case.rays, case.nbrs, case.bsp)
    order = [0, 2, 1, 0, 1, 2, 2]
    results = {}
    for staged in ("1", "0"):
        os.environ["VMCUDA_STAGED"] = staged
        try:
            engine = Engine(net)
        finally:
            os.environ.pop("VMCUDA_STAGED")
        mesh = Mesh.from_arrays(*mesh_args)
        frames = [FrameInput(mesh, case.frames[i]["Hoc"], case.lens, case.frames[i]["image"], case.format, None) for i in order]
        batch = engine.run_batch(frames)
        results[staged] = [batch.frame(f) for f in range(len(order))]
        for f, i in enumerate(order):
            fr = case.frames[i]
            want = O.classify(case.rays, case.nbrs, fr["ranges"], net, fr["Hoc"], case.lens, fr["image"], case.format)
            assert P.compare(results[staged][f], want, case.lens.dimensions).ok
        engine.close()
    for a, b in zip(results["1"], results["0"]):
        assert np.array_equal(a.global_indices, b.global_indices)
        assert np.abs(a.classifications.astype(np.float64) - b.classifications.astype(np.float64)).max() <= P.TOL_CLS / 4


# ---- tensor-core graph convolution (tcgen05) ---------------------------------------------------------------------------

def _engine_with_tc(network, mode):
    import os
    old = os.environ.get("VMCUDA_TC")
    os.environ["VMCUDA_TC"] = str(mode)
    try:
        return Engine(network)
    finally:
        if old is None:
            os.environ.pop("VMCUDA_TC")
        else:
            os.environ["VMCUDA_TC"] = old


def _random_rows(n, n_neighbours, seed):
    x = W.uniform(seed, n * 4, -1.0, 1.0).reshape(n, 4).astype(np.float32)
    x[-1] = -1.0
    nb = (W.splitmix64(seed + 1, n * n_neighbours) % np.uint64(n)).astype(np.int32).reshape(n, n_neighbours)
    nb[-1] = n - 1
    return x, nb


@pytest.mark.parametrize("n_neighbours,widths", [(6, [16, 16, 16, 8, 8, 3]), (8, [32, 32, 32, 4]), (4, [16, 32, 16, 2])])
def test_tensor_core_layers_match_the_oracle(n_neighbours, widths):
    """Every layer shape that has a tcgen05 kernel (mode 2 forces them on), several tiles and a ragged last tile."""
    net = W.make_network(7, n_neighbours, widths)
    x, nb = _random_rows(1000, n_neighbours, 11)
    want = O.network(x, nb, net)
    for mode in (0, 2):
        engine = _engine_with_tc(net, mode)
        got = engine.network(x, nb)
        d = np.abs(got.astype(np.float64) - want.astype(np.float64)).max()
        print(f"N={n_neighbours} widths={widths} tensor-core mode {mode}: max |d| = {d:.3g}")
        assert d <= P.TOL_CLS / 4
        engine.close()


@pytest.mark.parametrize("n_neighbours,widths", [(6, [16, 16, 16, 3]), (8, [32, 32, 4])])
def test_tensor_core_layers_over_many_tiles_per_cta(n_neighbours, widths):
    """More 128-row tiles than resident CTAs: every CTA walks several tiles, so the loads that run ahead across tile
    boundaries, the double-buffered accumulators and every phase of the register-buffer rotation are exercised."""
    net = W.make_network(21, n_neighbours, widths)
    x, nb = _random_rows(150_001, n_neighbours, 23)
    want = O.network(x, nb, net)
    engine = _engine_with_tc(net, 2)
    for _ in range(2):
        got = engine.network(x, nb)
        d = np.abs(got.astype(np.float64) - want.astype(np.float64)).max()
        print(f"N={n_neighbours} widths={widths}, 1172 tiles: max |d| = {d:.3g}")
        assert d <= P.TOL_CLS / 4
    engine.close()


def test_tensor_core_range_fallback():
    """Features beyond the range of the fp16 split make the engine recompute with the FFMA kernels, transparently:
    the result is bit for bit what an engine without tensor-core kernels returns."""
    net = W.make_network(9, 6, [16, 16, 2])
    net[0][0].weights[:] *= 3.0e5  # first layer output ~1e5: too large for fp16
    net[1][0].weights[:] *= 1.0e-5
    x, nb = _random_rows(700, 6, 13)
    plain = _engine_with_tc(net, 0)
    want = plain.network(x, nb)
    plain.close()
    assert np.all(np.isfinite(want))
    engine = _engine_with_tc(net, 2)
    for _ in range(2):  # the second call runs on the engine that has already fallen back
        got = engine.network(x, nb)
        assert np.array_equal(G.bits(got), G.bits(want))
    engine.close()


def test_network_shaped_like_the_reference_example_model(cases):
    """13 groups with the layer shapes of the reference's example/model.yaml (28x16, 5 x 112x16, 112x8, 5 x 56x8,
    56x5 softmax), seeded weights, on the reference's sampled inputs and neighbourhood."""
    case = cases["ring6_equisolid_rgba"]
    net = W.make_network(21, 6, [16] * 6 + [8] * 6 + [5])
    engine = Engine(net)
    for fr in case.frames[:2]:
        sampled = O.interpolate(fr["pixel_coordinates"], fr["image"], *case.lens.dimensions, case.format)
        inputs = np.concatenate([sampled, -np.ones((1, 4), np.float32)])
        want = O.network(inputs, fr["neighbourhood"], net)
        got = engine.network(inputs, fr["neighbourhood"])
        assert got.shape == want.shape and got.shape[1] == 5
        assert np.abs(got.astype(np.float64) - want.astype(np.float64)).max() <= P.TOL_CLS
    engine.close()


def test_mesh_cache_bound_releases_the_least_recently_used_mesh():
    """cfg4's four heights through an engine that may keep two meshes on the device: results are those of an unbounded
    engine, and the cache never holds more than two."""
    wl = W.config(4, n_frames=8)
    meshes = {}
    frames = []
    for fr in wl.frames:
        mesh = meshes.setdefault(id(fr.mesh), Mesh.from_spec(fr.mesh))
        frames.append(FrameInput(mesh, fr.Hoc, fr.lens, fr.image(), fr.format, None))
    assert len(meshes) >= 3
    plain, bounded = Engine(wl.network), Engine(wl.network, max_cached_meshes=2)
    for fr in frames:  # one frame per call, heights alternating: every eviction path is taken
        want = plain(fr.mesh, fr.Hoc, fr.lens, fr.image, fr.format)
        got = bounded(fr.mesh, fr.Hoc, fr.lens, fr.image, fr.format)
        assert len(bounded._meshes) <= 2
        assert np.array_equal(got.global_indices, want.global_indices)
        assert np.array_equal(G.bits(got.classifications), G.bits(want.classifications))
    assert len(plain._meshes) == len(meshes)
    plain.close()
    bounded.close()


def test_visualmesh_height_table_through_the_engine():
    """The VisualMesh overloads (cpp/visualmesh/engine/cpu/engine.hpp:160-165, :289-296): the engine picks the table
    nearest to Hoc[2][3] and gives what a call on that Mesh gives."""
    from visualmesh_b200.engine import VisualMesh
    import math
    vm = VisualMesh("RING6", "SPHERE", 0.0949, 0.0, 0.6, 1.4, 2.0, 0.5, 5.0)
    net = W.make_network(3, 6, [8, 2])
    engine = Engine(net)
    lens = W.Lens((160, 128), W.EQUISOLID, 56.0, (0.0, 0.0), (0.0, 0.0), math.pi)
    image = W.random_bytes(5, 160 * 128 * 4)
    for h in (0.55, 0.93, 1.7):
        Hoc = W.make_Hoc(math.radians(-50), math.radians(4), h)
        a = engine(vm, Hoc, lens, image, W.fourcc("RGBA"))
        mesh = vm.height(h)
        b = engine(mesh, Hoc, lens, image, W.fourcc("RGBA"), ranges="device")
        ranges = mesh.lookup(Hoc, lens)
        want = O.classify(mesh.rays, mesh.neighbours, ranges, net, Hoc, lens, image, W.fourcc("RGBA"))
        assert len(a.global_indices) > 50
        for key in ("global_indices", "neighbourhood", "pixel_coordinates", "classifications"):
            assert np.array_equal(G.bits(getattr(a, key)), G.bits(getattr(b, key))), key
        rep = P.compare(a, want, lens.dimensions)
        assert rep.ok, str(rep)
    engine.close()

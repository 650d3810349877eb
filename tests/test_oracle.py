"""Pins the plain-C oracle: bit for bit against the golden fixtures (outputs of the reference itself) and, where the
compiled reference is present, against the reference on the benchmark configurations."""
import numpy as np
import pytest

import golden_io as G
import oracle as O
import refharness as R
from visualmesh_b200 import workloads as W

pytestmark = pytest.mark.skipif(not O.available(), reason="oracle/libvmoracle.so not built")


def test_project_rays_matches_reference_fixture():
    z, lenses = G.units()
    for i, lens in enumerate(lenses):
        px = O.project_rays(z["rays"], lens)
        assert np.array_equal(G.bits(px), G.bits(z[f"px{i}"])), f"lens {i}"


def test_interpolate_every_fourcc_matches_reference_fixture():
    z, _ = G.units()
    Wd, Ht = [int(v) for v in z["sample_dims"]]
    for code in ["RGGB", "GRBG", "GBRG", "BGGR", "BGR3", "BGR8", "BGRA", "RGB3", "RGB8", "RGBA", "GRAY", "GREY",
                 "Y8  "]:
        out = O.interpolate(z["sample_px"], z[f"sample_image_{code.strip()}"], Wd, Ht, W.fourcc(code))
        assert np.array_equal(G.bits(out), G.bits(z[f"sample_out_{code.strip()}"])), code


def test_unknown_format_and_lens_are_errors():
    z, lenses = G.units()
    with pytest.raises(RuntimeError):
        O.interpolate(z["sample_px"], z["sample_image_RGBA"], 37, 23, W.fourcc("NV12"))
    bad = W.Lens((64, 64), 7, 30.0)
    with pytest.raises(RuntimeError):
        O.project_rays(z["rays"], bad)


@pytest.mark.parametrize("name", G.CASES)
def test_whole_path_matches_reference_fixture(name):
    case = G.Case(name)
    for f, fr in enumerate(case.frames):
        ranges = O.lookup(case.rays, case.bsp, fr["Hoc"], case.lens)
        assert np.array_equal(ranges, fr["ranges"]), f"{name} frame {f}: lookup"
        out = O.classify(case.rays, case.nbrs, ranges, case.network, fr["Hoc"], case.lens, fr["image"], case.format)
        for key in ("pixel_coordinates", "global_indices", "neighbourhood", "classifications"):
            want = fr[key]
            if want.size == 0:
                assert out[key].size == 0, f"{name} frame {f}: {key} should be empty"
            else:
                assert np.array_equal(G.bits(out[key]), G.bits(want)), f"{name} frame {f}: {key}"


def test_network_stage_alone_matches_fixture():
    case = G.Case("ring8_equidistant_bgra")
    fr = case.frames[0]
    n = fr["global_indices"].shape[0]
    inputs = np.concatenate([O.interpolate(fr["pixel_coordinates"], fr["image"], *case.lens.dimensions, case.format),
                             -np.ones((1, 4), np.float32)])
    out = O.network(inputs, fr["neighbourhood"], case.network)
    assert out.shape == (n + 1, 3)
    assert np.array_equal(G.bits(out), G.bits(fr["classifications"]))


@pytest.mark.skipif(not R.available(), reason="compiled reference (oracle/_ref/libvmref.so) not present")
@pytest.mark.parametrize("cfg", [0, 1, 2])
def test_matches_compiled_reference_on_benchmark_configs(cfg):
    wl = W.config(cfg, n_frames=2)
    meshes = {}
    for fr in wl.frames:
        mesh = meshes.setdefault(fr.mesh.key(), R.RefMesh(fr.mesh))
        rays, nbrs = mesh.nodes()
        ranges = mesh.lookup(fr.Hoc, fr.lens)
        assert np.array_equal(O.lookup(rays, mesh.bsp(), fr.Hoc, fr.lens), ranges)
        image = fr.image()
        ref = mesh.classify(wl.network, fr.Hoc, fr.lens, image, fr.format)
        out = O.classify(rays, nbrs, ranges, wl.network, fr.Hoc, fr.lens, image, fr.format)
        assert ref["global_indices"].shape[0] > 100
        for key in ref:
            assert np.array_equal(G.bits(out[key]), G.bits(ref[key])), f"cfg{cfg}: {key}"

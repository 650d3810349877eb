"""Every frame of every benchmark configuration, CUDA engine against the compiled reference CPU engine. Needs a GPU.

The target: at least 90 % of the frames of each configuration within the tolerances (on-screen set and neighbourhood
bit-exact up to reported border nodes, pixel coordinates within 1e-3 px, classifications within 1e-4). Configuration 3
runs its full ten layers - a 4 -> 32 layer, eight chained 32 -> 32 layers on the tensor cores, each fed by the previous
one's split-layout output, and the softmax layer. The reference needs about a minute of all host cores for that one.
"""
import pytest

import parity as P
import refharness as R

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not R.available(), reason="compiled reference (oracle/_ref/libvmref.so) not present")]


@pytest.mark.parametrize("cfg", [0, 1, 2, 3, 4])
def test_every_frame_of_the_configuration(cfg):
    rep = P.config_parity(cfg, P.FULL_PARITY_FRAMES[cfg])
    print(f"cfg{cfg}: {rep}")
    assert rep["frames"] == P.FULL_PARITY_FRAMES[cfg]
    assert rep["nodes"] > 0
    assert rep["stray_nodes"] == 0, rep
    assert rep["max_px"] <= P.TOL_PX, rep
    assert rep["frames_ok"] >= 0.9 * rep["frames"], rep

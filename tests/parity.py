"""Comparison of an engine result with the reference's, under the tolerances of the task:

  * global_indices and neighbourhood bit-exact, except nodes whose projection lies within 1e-3 px of the image
    border (these are reported, and the rest is compared on the common nodes);
  * pixel_coordinates within 1e-3 px;
  * classifications within 1e-4 absolute.
"""
from dataclasses import dataclass, field

import numpy as np

TOL_PX = 1e-3
TOL_CLS = 1e-4


@dataclass
class Report:
    n_ref: int = 0
    n_out: int = 0
    indices_exact: bool = True
    border_nodes: list = field(default_factory=list)   # global ids present on one side only, all within TOL_PX of the border
    stray_nodes: list = field(default_factory=list)    # ... and those that are not: a failure
    neighbourhood_exact: bool = True
    max_px: float = 0.0
    px_bit_identical: float = 1.0    # fraction of pixel coordinates (x and y) with identical bit patterns
    max_cls: float = 0.0
    cls_over_tol: int = 0
    cls_entries: int = 0

    @property
    def projection_ok(self):
        return not self.stray_nodes and self.neighbourhood_exact and self.max_px <= TOL_PX

    @property
    def ok(self):
        return self.projection_ok and self.cls_over_tol == 0

    def __str__(self):
        return (f"n={self.n_out}/{self.n_ref} idx_exact={self.indices_exact} border={len(self.border_nodes)} "
                f"stray={len(self.stray_nodes)} nb_exact={self.neighbourhood_exact} max_px={self.max_px:.3g} "
                f"px_bits={self.px_bit_identical:.4f} max_cls={self.max_cls:.3g} "
                f"cls_over={self.cls_over_tol}/{self.cls_entries}")


def _near_border(px, dims):
    W, H = dims
    x, y = px[:, 0], px[:, 1]
    return (np.abs(x) <= TOL_PX) | (np.abs(x + 1 - W) <= TOL_PX) | (np.abs(y) <= TOL_PX) | (np.abs(y + 1 - H) <= TOL_PX)


def compare(out, ref, dims) -> Report:
    """out / ref: objects or dicts with pixel_coordinates, neighbourhood, global_indices[, classifications]."""
    get = (lambda o, k: o[k]) if isinstance(ref, dict) else getattr
    geto = (lambda o, k: o[k]) if isinstance(out, dict) else getattr
    r_gi, o_gi = get(ref, "global_indices"), geto(out, "global_indices")
    r_px, o_px = get(ref, "pixel_coordinates"), geto(out, "pixel_coordinates")
    r_nb, o_nb = get(ref, "neighbourhood"), geto(out, "neighbourhood")
    r_cls = get(ref, "classifications") if (isinstance(ref, dict) and "classifications" in ref) or hasattr(ref, "classifications") else None
    o_cls = geto(out, "classifications") if r_cls is not None else None
    rep = Report(n_ref=len(r_gi), n_out=len(o_gi))
    if len(r_gi) == 0 and len(o_gi) == 0:
        return rep
    rep.indices_exact = len(r_gi) == len(o_gi) and np.array_equal(r_gi, o_gi)
    if rep.indices_exact:
        ri = oi = np.arange(len(r_gi))
    else:
        common, ri, oi = np.intersect1d(r_gi, o_gi, return_indices=True)
        only_r = np.setdiff1d(np.arange(len(r_gi)), ri)
        only_o = np.setdiff1d(np.arange(len(o_gi)), oi)
        for idx, gi, px in ((only_r, r_gi, r_px), (only_o, o_gi, o_px)):
            if len(idx):
                near = _near_border(px[idx], dims)
                rep.border_nodes += [int(g) for g in gi[idx][near]]
                rep.stray_nodes += [int(g) for g in gi[idx][~near]]
    # neighbourhood: compare in global ids so that a border node missing on one side does not shift everything
    def to_global(nb, gi):
        table = np.concatenate([gi, [-1]]).astype(np.int64)
        return table[nb[:-1]]
    if len(r_gi) and len(o_gi):
        g_r, g_o = to_global(r_nb, r_gi)[ri], to_global(o_nb, o_gi)[oi]
        if rep.indices_exact:
            rep.neighbourhood_exact = np.array_equal(r_nb, o_nb)
        else:
            lost = set(rep.border_nodes)
            diff = g_r != g_o
            # a neighbour that is a border node on one side is the off-screen row on the other
            excus = np.isin(g_r, list(lost)) | np.isin(g_o, list(lost))
            rep.neighbourhood_exact = not np.any(diff & ~excus)
        d = np.abs(r_px[ri].astype(np.float64) - o_px[oi].astype(np.float64))
        rep.max_px = float(d.max()) if d.size else 0.0
        rep.px_bit_identical = float(np.mean(r_px[ri].view(np.uint32) == o_px[oi].view(np.uint32))) if d.size else 1.0
        if r_cls is not None:
            rows_r = np.concatenate([ri, [len(r_gi)]])
            rows_o = np.concatenate([oi, [len(o_gi)]])
            dc = np.abs(r_cls[rows_r].astype(np.float64) - o_cls[rows_o].astype(np.float64))
            rep.max_cls = float(dc.max())
            rep.cls_over_tol = int((dc > TOL_CLS).sum())
            rep.cls_entries = int(dc.size)
    return rep


# ---------------------------------------------------------------------------------------------------------------------
# Whole configurations: every frame through the compiled reference CPU engine and through the CUDA engine
# ---------------------------------------------------------------------------------------------------------------------

def config_parity(cfg, n_frames=None, seed=0, threads=None, batch_frames=16, engine=None):
    """Runs the first n_frames of benchmark configuration `cfg` (all of them when None) through the reference CPU
    engine (oracle/_ref/libvmref.so: a fresh cpu::Engine per frame, `threads` frames at a time) and through the CUDA
    engine (device-side lookup, host images, batches of `batch_frames`), and compares frame by frame under the
    tolerances at the top of this file. Returns a dict:

        frames, frames_ok          frames compared / frames with every entry within tolerance
        nodes                      on-screen nodes over all frames (reference)
        indices_exact_frames       frames whose global_indices and neighbourhood are bit-exact
        border_nodes, stray_nodes  nodes on one side only: within 1e-3 px of the border (allowed, reported) / not (failure)
        max_px, px_bit_identical   largest pixel difference; fraction of coordinates with identical bits
        max_cls, cls_over_tol, cls_entries
        reference_seconds          wall time of the reference runs
    """
    import os
    import time
    from concurrent.futures import ThreadPoolExecutor

    import refharness as R
    from visualmesh_b200 import workloads as W
    from visualmesh_b200.engine import Engine, FrameInput, Mesh

    wl = W.config(cfg, seed=seed, n_frames=n_frames)
    threads = threads or os.cpu_count() or 1
    own_engine = engine is None
    if own_engine:
        engine = Engine(wl.network)
    ref_meshes, meshes = {}, {}
    for fr in wl.frames:
        if fr.mesh.key() not in ref_meshes:
            ref_meshes[fr.mesh.key()] = R.RefMesh(fr.mesh)
            meshes[fr.mesh.key()] = Mesh.from_spec(fr.mesh)

    total = dict(frames=0, frames_ok=0, nodes=0, indices_exact_frames=0, border_nodes=0, stray_nodes=0, max_px=0.0,
                 max_cls=0.0, cls_over_tol=0, cls_entries=0, reference_seconds=0.0)
    px_same, px_count = 0.0, 0
    # a window of frames at a time bounds the memory held (a config-3 frame and its results are ~150 MB)
    window = max(batch_frames, threads)
    with ThreadPoolExecutor(max_workers=threads) as pool:
        for w0 in range(0, len(wl.frames), window):
            frames = wl.frames[w0:w0 + window]
            images = [fr.image() for fr in frames]
            t0 = time.perf_counter()
            refs = list(pool.map(lambda a: ref_meshes[a[0].mesh.key()].classify(wl.network, a[0].Hoc, a[0].lens, a[1],
                                                                                a[0].format), zip(frames, images)))
            total["reference_seconds"] += time.perf_counter() - t0
            for b0 in range(0, len(frames), batch_frames):
                part = range(b0, min(b0 + batch_frames, len(frames)))
                batch = engine.run_batch([FrameInput(meshes[frames[i].mesh.key()], frames[i].Hoc, frames[i].lens,
                                                     images[i], frames[i].format, None) for i in part])
                for j, i in enumerate(part):
                    rep = compare(batch.frame(j, copy=False), refs[i], frames[i].lens.dimensions)
                    total["frames"] += 1
                    total["frames_ok"] += int(rep.ok and (rep.n_ref == rep.n_out or bool(rep.border_nodes)))
                    total["nodes"] += rep.n_ref
                    total["indices_exact_frames"] += int(rep.indices_exact and rep.neighbourhood_exact)
                    total["border_nodes"] += len(rep.border_nodes)
                    total["stray_nodes"] += len(rep.stray_nodes)
                    total["max_px"] = max(total["max_px"], rep.max_px)
                    total["max_cls"] = max(total["max_cls"], rep.max_cls)
                    total["cls_over_tol"] += rep.cls_over_tol
                    total["cls_entries"] += rep.cls_entries
                    px_same += rep.px_bit_identical * 2 * rep.n_ref
                    px_count += 2 * rep.n_ref
    total["px_bit_identical"] = px_same / px_count if px_count else 1.0
    total["pass"] = f"{total['frames_ok']}/{total['frames']}"
    if own_engine:
        engine.close()
    return total


# frames per configuration that "every frame" means: the configurations' own counts, and a 256-frame prefix of the
# 4096-frame stream of configuration 4 (all four camera heights occur in it)
FULL_PARITY_FRAMES = {0: 1, 1: 64, 2: 32, 3: 32, 4: 256}

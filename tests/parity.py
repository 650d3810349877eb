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

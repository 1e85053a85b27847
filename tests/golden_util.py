"""Loader of tests/golden/ref_cases.npz (outputs of the reference's own CPU code,
produced by tests/golden/make_golden.py)."""
import os

import numpy as np

from oracle.common import HostFsaVec

PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_cases.npz")


def load():
    z = np.load(PATH)
    cases = []
    for name in z["names"].tolist():
        g = lambda k: z[f"{name}.{k}"]  # noqa: E731
        amap = g("amap")
        cases.append(dict(
            name=name, a=HostFsaVec(g("a_rs1"), g("a_rs2"), g("a_arcs")), scores=g("scores"),
            brs=g("brs"), beam=float(g("beam")), amap=None if amap.size == 0 else amap,
            lattice=HostFsaVec(g("l_rs1"), g("l_rs2"), g("l_arcs"), arc_map_a=g("map_a"),
                               arc_map_b=g("map_b")),
            fwd_log=g("fwd_log"), bwd_log=g("bwd_log"), tot_log=g("tot_log"),
            post_log=g("post_log"), fwd_trop=g("fwd_trop"), bwd_trop=g("bwd_trop"),
            tot_trop=g("tot_trop"), post_trop=g("post_trop"), entering=g("entering"),
            path_splits=g("path_splits"), best=g("best"), props=g("props"),
            symbols=z[f"{name}.symbols"] if f"{name}.symbols" in z else None,
            aux=z[f"{name}.aux"] if f"{name}.aux" in z else None))
    return cases

"""Generates tests/golden/ref_cases.npz by running the k2 reference's own CPU code
(oracle/_ref/libk2ref.so, built by `make -C oracle ref REF=<k2 checkout>`) on
seeded inputs.  Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import ref  # noqa: E402
from oracle.common import HostFsaVec  # noqa: E402
from util import random_dense, random_fsa_vec  # noqa: E402


def pack(prefix, out, a: HostFsaVec, scores, brs, beam, amap):
    lat = ref.intersect_dense(a, scores, brs, beam, amap)
    out[f"{prefix}.a_rs1"], out[f"{prefix}.a_rs2"], out[f"{prefix}.a_arcs"] = \
        a.row_splits1, a.row_splits2, a.arcs
    out[f"{prefix}.scores"], out[f"{prefix}.brs"] = scores, brs
    out[f"{prefix}.beam"] = np.float32(beam)
    out[f"{prefix}.amap"] = np.zeros(0, np.int32) if amap is None else amap
    out[f"{prefix}.l_rs1"], out[f"{prefix}.l_rs2"], out[f"{prefix}.l_arcs"] = \
        lat.row_splits1, lat.row_splits2, lat.arcs
    out[f"{prefix}.map_a"], out[f"{prefix}.map_b"] = lat.arc_map_a, lat.arc_map_b
    for log in (True, False):
        tag = "log" if log else "trop"
        f = ref.forward_scores(lat, log, True)
        b = ref.backward_scores(lat, log, True)
        tot, post = ref.tot_scores_and_arc_post(lat, f, b, True)
        out[f"{prefix}.fwd_{tag}"], out[f"{prefix}.bwd_{tag}"] = f, b
        out[f"{prefix}.tot_{tag}"], out[f"{prefix}.post_{tag}"] = tot, post
    _, ea = ref.forward_scores(lat, False, True, want_entering_arcs=True)
    ps, best = ref.shortest_path(lat, ea)
    out[f"{prefix}.entering"], out[f"{prefix}.path_splits"], out[f"{prefix}.best"] = ea, ps, best
    out[f"{prefix}.props"] = ref.properties(lat)[0]


def main():
    out = {}
    rng = np.random.default_rng(2024)
    names = []
    for k in range(6):
        n = int(rng.integers(2, 6))
        a = random_fsa_vec(rng, n, max_states=10, max_arcs=30, acyclic=bool(k % 2))
        scores, brs = random_dense(rng, n, 8, 5)
        amap = np.sort(rng.integers(0, n, size=n)).astype(np.int32) if k == 3 else None
        pack(f"rand{k}", out, a, scores, brs, [0.5, 2.0, 10.0, 100.0, 4.0, 1.0][k], amap)
        names.append(f"rand{k}")
    # CTC graphs from the reference's own builder, standard and modified
    for k, modified in enumerate((False, True)):
        syms = [[int(x) for x in rng.integers(1, 5, size=int(rng.integers(1, 5)))]
                for _ in range(3)]
        g = ref.ctc_graphs(syms, modified)
        out[f"ctc{k}.symbols"] = np.asarray([len(s) for s in syms] + [x for s in syms for x in s],
                                            np.int32)
        out[f"ctc{k}.aux"] = g.aux_labels
        scores, brs = random_dense(rng, 3, 12, 5, low_rows=False)
        pack(f"ctc{k}", out, g, scores, brs, 6.0, None)
        names.append(f"ctc{k}")
    out["names"] = np.asarray(names)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ref_cases.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()

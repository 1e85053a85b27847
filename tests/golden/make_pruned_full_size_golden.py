"""Generates tests/golden/pruned_full_size.json: sha256 checksums of the lattice that the
k2 reference's own CPU IntersectDensePruned (oracle/_ref/libk2ref.so, built by
`make -C oracle ref REF=<k2 checkout>`) produces for the full decoding configuration
(hlg_decode: a 200 000-state graph shared by 32 sequences of 500 frames; search beam 20,
output beam 8, 30..10 000 active states).  The lattice itself is 4 M arcs, so only its
sizes and the digests of its arrays are kept.  About a minute on one core.  Run from the
repository root:
    python tests/golden/make_pruned_full_size_golden.py
"""
import hashlib
import importlib.util
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import ref  # noqa: E402
from oracle.common import HostFsaVec  # noqa: E402

PARAMS = dict(search_beam=20.0, output_beam=8.0, min_active_states=30, max_active_states=10000)


def load_synthetic():
    spec = importlib.util.spec_from_file_location(
        "_k2b200_synthetic", os.path.join(ROOT, "k2_b200", "synthetic.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod
    spec.loader.exec_module(mod)
    return mod


def digest(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def host_scores(w):
    seg = w.supervision_segments.numpy()
    N, T, C = w.log_probs.shape
    rows = int(seg[:, 2].sum() + len(seg))
    scores = np.full((rows, C + 1), -np.inf, np.float32)
    row_splits = np.zeros(len(seg) + 1, np.int32)
    lp = w.log_probs.numpy()
    r = 0
    for i, (n, s, d) in enumerate(seg.tolist()):
        scores[r:r + d, 1:] = lp[n, s:s + d]
        scores[r + d, 0] = 0.0
        r += d + 1
        row_splits[i + 1] = r
    return scores, row_splits


def main():
    w = load_synthetic().hlg_decode(seed=0)
    S = len(w.graph_row_splits2) - 1
    a = HostFsaVec(np.array([0, S], np.int32), w.graph_row_splits2.astype(np.int32), w.graph_arcs)
    scores, row_splits = host_scores(w)
    lat = ref.intersect_dense_pruned(a, scores, row_splits, *PARAMS.values(), False)
    out = {"workload": "hlg_decode seed 0", **PARAMS, "num_states": int(lat.num_states),
           "num_arcs": int(lat.num_arcs),
           "sha256": {"row_splits1": digest(lat.row_splits1.astype(np.int32)),
                      "row_splits2": digest(lat.row_splits2.astype(np.int32)),
                      "arcs": digest(lat.arcs.astype(np.int32)),
                      "arc_map_a": digest(lat.arc_map_a.astype(np.int32)),
                      "arc_map_b": digest(lat.arc_map_b.astype(np.int32))}}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "pruned_full_size.json")
    with open(path, "w") as f:
        json.dump(out, f, indent=1)
        f.write("\n")
    print(json.dumps(out, indent=1))


if __name__ == "__main__":
    main()

"""Generates tests/golden/pruned_cases.npz by running the k2 reference's own CPU
IntersectDensePruned (oracle/_ref/libk2ref.so, built by `make -C oracle ref
REF=<k2 checkout>`) on seeded inputs.  Run from the repository root:
    python tests/golden/make_pruned_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle import ref  # noqa: E402
from pruned_util import pruned_cases  # noqa: E402


def main():
    out, names = {}, []
    for c in pruned_cases(small=True):
        lat = ref.intersect_dense_pruned(c["a"], c["scores"], c["brs"], *c["params"])
        name = c["name"]
        out[f"{name}.l_rs1"], out[f"{name}.l_rs2"], out[f"{name}.l_arcs"] = \
            lat.row_splits1, lat.row_splits2, lat.arcs
        out[f"{name}.map_a"], out[f"{name}.map_b"] = lat.arc_map_a, lat.arc_map_b
        names.append(name)
        print(name, lat.num_states, "states", lat.num_arcs, "arcs")
    out["names"] = np.asarray(names)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "pruned_cases.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()

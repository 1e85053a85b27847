"""Seeded input generators and comparison helpers shared by the tests."""
import numpy as np

from oracle.common import HostFsaVec, make_arcs

NEG_INF = -np.inf


def random_fsa_vec(rng: np.random.Generator, num_fsas: int, max_states: int = 12,
                   max_arcs: int = 40, max_label: int = 4, acyclic: bool = False,
                   allow_empty: bool = True) -> HostFsaVec:
    """Random valid FsaVec in the spirit of k2's RandomFsaVec
    (k2/csrc/fsa_utils.cu:1936-2043): arbitrary (possibly cyclic) graphs whose
    arcs into the final state carry -1 and only those."""
    rs1, rs2, rows = [0], [0], []
    for _ in range(num_fsas):
        if allow_empty and rng.random() < 0.05:
            rs1.append(rs1[-1])
            continue
        ns = int(rng.integers(2, max_states + 1))
        na = int(rng.integers(1, max_arcs + 1))
        src = np.sort(rng.integers(0, ns - 1, size=na))
        for s in range(ns):
            mine = np.nonzero(src == s)[0]
            for _k in mine:
                lo = s + 1 if acyclic else 0
                dest = int(rng.integers(lo, ns))
                label = -1 if dest == ns - 1 else int(rng.integers(0, max_label + 1))
                score = float(np.float32(rng.normal()))
                rows.append((s, dest, label, score))
            rs2.append(len(rows))
        rs1.append(rs1[-1] + ns)
    if rows:
        r = np.array(rows, dtype=np.float64)
        arcs = make_arcs(r[:, 0].astype(np.int32), r[:, 1].astype(np.int32),
                         r[:, 2].astype(np.int32), r[:, 3].astype(np.float32))
    else:
        arcs = np.zeros((0, 4), np.int32)
    return HostFsaVec(np.asarray(rs1, np.int32), np.asarray(rs2, np.int32), arcs)


def random_dense(rng: np.random.Generator, num_seqs: int, max_frames: int, num_classes: int,
                 scale: float = 1.0, low_rows: bool = True):
    """scores [sum(T_i+1), C+1] and row_splits, durations sorted decreasingly
    (k2/csrc/intersect_test.cu:285-299 also plants some very low rows)."""
    durs = np.sort(rng.integers(1, max_frames + 1, size=num_seqs))[::-1]
    rows = int(durs.sum() + num_seqs)
    scores = np.full((rows, num_classes + 1), NEG_INF, np.float32)
    row_splits = np.zeros(num_seqs + 1, np.int32)
    r = 0
    for i, d in enumerate(durs):
        x = (rng.normal(size=(d, num_classes)) * scale).astype(np.float32)
        x = x - np.log(np.exp(x).sum(-1, keepdims=True)).astype(np.float32)
        if low_rows and rng.random() < 0.3:
            x[int(rng.integers(0, d))] -= 100.0
        scores[r:r + d, 1:] = x
        scores[r + d, 0] = 0.0
        r += d + 1
        row_splits[i + 1] = r
    return scores, row_splits


def same_fsa(a: HostFsaVec, b: HostFsaVec, what=""):
    assert np.array_equal(a.row_splits1, b.row_splits1), f"{what}: row_splits1 differ"
    assert np.array_equal(a.row_splits2, b.row_splits2), f"{what}: row_splits2 differ"
    assert np.array_equal(a.arcs, b.arcs), f"{what}: arcs differ"
    for name in ("arc_map_a", "arc_map_b"):
        x, y = getattr(a, name), getattr(b, name)
        if x is not None and y is not None:
            assert np.array_equal(x, y), f"{what}: {name} differ"


def close(a, b, rtol=1e-6, atol=1e-6):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    both_inf = np.isinf(a) & np.isinf(b) & (np.sign(a) == np.sign(b))
    with np.errstate(invalid="ignore"):
        ok = both_inf | (np.abs(a - b) <= atol + rtol * np.abs(b))
    return bool(np.all(ok))


def host_levels(arcs):
    """Longest-distance layering of a RaggedArc computed with numpy from a host copy:
    the checker of k2b200_fsa_levels.  Returns (offsets, splits) as numpy arrays."""
    rs1 = arcs.h_row_splits1
    rs2 = arcs._row_splits2.cpu().numpy()
    vals = arcs._values.cpu().numpy()
    ns = arcs.num_states
    level = np.zeros(ns, dtype=np.int64)
    order_ok = True
    for i in range(len(rs1) - 1):
        b, e = int(rs1[i]), int(rs1[i + 1])
        for s in range(b, e):
            a0, a1 = int(rs2[s]), int(rs2[s + 1])
            if a1 > a0:
                d = vals[a0:a1, 1].astype(np.int64) + b
                if np.any(d <= s):
                    order_ok = False
                np.maximum.at(level, d, level[s] + 1)
    if not order_ok:
        raise RuntimeError("forward/backward scores need a top-sorted, acyclic FsaVec")
    # states must be grouped by level within each FSA for contiguous layers; when
    # they are not, fall back to one state per layer (always valid when top-sorted)
    offsets = [0]
    splits = []
    for i in range(len(rs1) - 1):
        b, e = int(rs1[i]), int(rs1[i + 1])
        lv = level[b:e]
        if e > b and np.all(np.diff(lv) >= 0):
            change = np.nonzero(np.diff(lv))[0] + 1
            starts = np.concatenate([[0], change]) + b
        else:
            starts = np.arange(b, e)
        splits.extend(starts.tolist())
        offsets.append(len(splits))
    splits.append(int(rs1[-1]))
    return np.asarray(offsets, np.int32), np.asarray(splits, np.int32)

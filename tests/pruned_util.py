"""Seeded inputs of the pruned-intersection tests.  The small set is what
tests/golden/pruned_cases.npz holds the reference's answers for."""
import numpy as np

from oracle import oracle
from oracle.common import HostFsaVec, make_arcs
from util import random_dense, random_fsa_vec


def decoding_graph(rng, num_states, num_classes, mean_degree=3.0, eps=0.05):
    """A random arc-sorted graph shaped like a decoding graph: every state is reachable
    from state 0, out-degree Poisson + 1, weights -Exponential(1), one final state."""
    S = num_states
    rows = []
    for s in range(S - 1):
        deg = int(rng.poisson(mean_degree)) + 1
        dests = rng.integers(0, S - 1, size=deg)
        if s + 1 < S - 1:
            dests[0] = s + 1  # a chain through all states keeps them connected
        labels = np.where(rng.random(deg) < eps, 0, rng.integers(1, num_classes, size=deg))
        arcs = sorted(zip(labels.tolist(), dests.tolist()))
        for lab, d in arcs:
            rows.append((s, d, lab, -float(rng.exponential())))
        if rng.random() < 0.2 or s == S - 2:
            rows.append((s, S - 1, -1, -float(rng.exponential())))
    r = np.array(rows, dtype=np.float64)
    arcs = make_arcs(r[:, 0].astype(np.int32), r[:, 1].astype(np.int32), r[:, 2].astype(np.int32),
                     r[:, 3].astype(np.float32))
    rs2 = np.zeros(S + 1, np.int32)
    np.add.at(rs2, r[:, 0].astype(np.int64) + 1, 1)
    return HostFsaVec(np.asarray([0, S], np.int32), np.cumsum(rs2).astype(np.int32), arcs)


def pruned_cases(small: bool):
    """dicts with name, a (HostFsaVec), scores, brs, params = (search_beam, output_beam,
    min_active, max_active, allow_partial)."""
    rng = np.random.default_rng(77 if small else 78)
    cases = []
    scale = 1 if small else 4
    # one CTC graph per sequence, several pruning windows, generous beams
    n = 3
    syms = [[int(x) for x in rng.integers(1, 6, size=int(rng.integers(3, 9)))] for _ in range(n)]
    scores, brs = random_dense(rng, n, 45 * scale, 6, low_rows=False)
    cases.append(dict(name="ctc_wide", a=oracle.ctc_graphs(syms, False), scores=scores, brs=brs,
                      params=(20.0, 8.0, 0, 10000, False)))
    # the same with tight limits: the search beam shrinks and grows
    cases.append(dict(name="ctc_tight", a=oracle.ctc_graphs(syms, True), scores=scores, brs=brs,
                      params=(4.0, 2.0, 3, 6, False)))
    # random cyclic graphs, one per sequence
    a = random_fsa_vec(rng, 4, max_states=12, max_arcs=40, max_label=4, allow_empty=False)
    scores, brs = random_dense(rng, 4, 25 * scale, 5)
    cases.append(dict(name="rand_graphs", a=a, scores=scores, brs=brs,
                      params=(10.0, 4.0, 2, 8, False)))
    # a shared decoding graph
    g = decoding_graph(rng, 60 * scale, 7)
    scores, brs = random_dense(rng, 5, 50 * scale, 7, scale=2.0, low_rows=False)
    cases.append(dict(name="shared_wide", a=g, scores=scores, brs=brs,
                      params=(15.0, 6.0, 5, 40 * scale, False)))
    cases.append(dict(name="shared_tight", a=g, scores=scores, brs=brs,
                      params=(6.0, 3.0, 2, 10, False)))
    # allow_partial: a graph whose final state is hard to reach in time
    cases.append(dict(name="shared_partial", a=g, scores=scores, brs=brs,
                      params=(3.0, 2.0, 0, 4, True)))
    cases.append(dict(name="rand_partial", a=a, scores=cases[2]["scores"], brs=cases[2]["brs"],
                      params=(2.0, 1.0, 0, 3, True)))
    return cases

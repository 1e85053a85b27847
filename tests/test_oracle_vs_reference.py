"""Pins the C restatement (oracle/k2_oracle.c) against the reference's own CPU code
(oracle/_ref/libk2ref.so) on seeded random inputs: everything must be identical,
bit for bit - lattices, arc maps, float and double scores, best paths, graphs."""
import numpy as np
import pytest

from oracle import oracle, ref
from util import random_dense, random_fsa_vec, same_fsa

pytestmark = pytest.mark.skipif(
    not ref.available(), reason="oracle/_ref/libk2ref.so not built (needs the k2 checkout)")


def test_intersect_and_scores_identical():
    rng = np.random.default_rng(0)
    for trial in range(120):
        n = int(rng.integers(1, 6))
        a = random_fsa_vec(rng, n, acyclic=bool(trial % 2))
        scores, brs = random_dense(rng, n, 10, 5)
        beam = float(rng.choice([0.5, 2.0, 10.0, 100.0]))
        amap = np.sort(rng.integers(0, n, size=n)).astype(np.int32) if trial % 5 == 0 else None
        r = ref.intersect_dense(a, scores, brs, beam, amap)
        o = oracle.intersect_dense(a, scores, brs, beam, amap)
        same_fsa(r, o, f"trial {trial}")
        for log in (True, False):
            for dbl in (True, False):
                rf, of = ref.forward_scores(r, log, dbl), oracle.forward_scores(o, log, dbl)
                rb, ob = ref.backward_scores(r, log, dbl), oracle.backward_scores(o, log, dbl)
                assert np.array_equal(rf, of) and np.array_equal(rb, ob), (trial, log, dbl)
                rt, rp = ref.tot_scores_and_arc_post(r, rf, rb, dbl)
                ot, op = oracle.tot_scores_and_arc_post(o, of, ob, dbl)
                assert np.array_equal(rt, ot) and np.array_equal(rp, op, equal_nan=True)
        _, rea = ref.forward_scores(r, False, True, True)
        _, oea = oracle.forward_scores(o, False, True, True)
        assert np.array_equal(rea, oea)
        rs, rbest = ref.shortest_path(r, rea)
        os_, obest = oracle.shortest_path(o, oea)
        assert np.array_equal(rs, os_) and np.array_equal(rbest, obest)
        rp_, ro = ref.properties(r), oracle.properties(o)
        assert np.array_equal(rp_[0], ro[0]) and rp_[1] == ro[1]


def test_beam_reduction_identical():
    # limits are set to 70% of what beam 50 keeps, and only where that is far above
    # the best paths alone: the reference's retry loop (intersect_dense.cu:240-320)
    # never ends when even a vanishing beam exceeds the limit
    rng = np.random.default_rng(5)
    done = 0
    for trial in range(60):
        n = int(rng.integers(2, 6))
        a = random_fsa_vec(rng, n, max_states=20, max_arcs=80, allow_empty=False)
        scores, brs = random_dense(rng, n, 12, 5, low_rows=False)
        full = oracle.intersect_dense(a, scores, brs, 50.0)
        path_states = int(np.diff(brs).sum() + n)
        if full.num_states < 3 * path_states or full.num_arcs < 6 * path_states:
            continue
        kw = dict(max_states=int(0.7 * full.num_states)) if trial % 2 else dict(
            max_arcs=int(0.7 * full.num_arcs) + 4 * path_states)
        r = ref.intersect_dense(a, scores, brs, 50.0, None, **kw)
        o = oracle.intersect_dense(a, scores, brs, 50.0, None, **kw)
        same_fsa(r, o, f"trial {trial} {kw}")
        done += 1
    assert done >= 5


def test_ctc_graphs_identical():
    rng = np.random.default_rng(1)
    for modified in (False, True):
        for _ in range(40):
            syms = [[int(x) for x in rng.integers(1, 5, size=int(rng.integers(0, 7)))]
                    for _ in range(int(rng.integers(1, 6)))]
            r, o = ref.ctc_graphs(syms, modified), oracle.ctc_graphs(syms, modified)
            same_fsa(r, o)
            assert np.array_equal(r.aux_labels, o.aux_labels)


def test_reference_rejects_what_the_oracle_rejects():
    rng = np.random.default_rng(3)
    a = random_fsa_vec(rng, 2, allow_empty=False)
    scores, brs = random_dense(rng, 2, 6, 5)
    with pytest.raises(RuntimeError):
        ref.intersect_dense(a, scores, brs, 10.0, np.array([1, 0], np.int32))
    with pytest.raises(RuntimeError):
        oracle.intersect_dense(a, scores, brs, 10.0, np.array([1, 0], np.int32))


def test_pruned_intersection_fixtures_are_the_reference_answers():
    """tests/golden/pruned_cases.npz (what the GPU path is compared with) against the
    reference library run now on the same seeded inputs."""
    import os
    from oracle.common import HostFsaVec
    from pruned_util import pruned_cases
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden",
                             "pruned_cases.npz"))
    for c in pruned_cases(small=True):
        name = c["name"]
        r = ref.intersect_dense_pruned(c["a"], c["scores"], c["brs"], *c["params"])
        want = HostFsaVec(z[f"{name}.l_rs1"], z[f"{name}.l_rs2"], z[f"{name}.l_arcs"],
                          arc_map_a=z[f"{name}.map_a"], arc_map_b=z[f"{name}.map_b"])
        same_fsa(r, want, name)


def test_pruned_intersection_with_wide_beams_is_the_exact_lattice_best_path():
    """With beams that prune nothing the pruned search keeps a superset of the exact
    lattice and the best path score is the same (tropical total of intersect_dense)."""
    rng = np.random.default_rng(11)
    for trial in range(10):
        n = int(rng.integers(1, 4))
        syms = [[int(x) for x in rng.integers(1, 5, size=int(rng.integers(1, 6)))]
                for _ in range(n)]
        g = oracle.ctc_graphs(syms, False)
        scores, brs = random_dense(rng, n, 40, 5, low_rows=False)
        exact = ref.intersect_dense(g, scores, brs, 1000.0, None)
        pruned = ref.intersect_dense_pruned(g, scores, brs, 1000.0, 1000.0, 0, 100000)
        te = ref.tot_scores_and_arc_post(exact, ref.forward_scores(exact, False, True),
                                         ref.backward_scores(exact, False, True), True)[0]
        tp = ref.tot_scores_and_arc_post(pruned, ref.forward_scores(pruned, False, True),
                                         ref.backward_scores(pruned, False, True), True)[0]
        np.testing.assert_allclose(te, tp, rtol=1e-6)


def test_ctc_topo_is_the_reference_topology():
    """k2_b200.ctc_topo (host-built graph) against k2::CtcTopo, arc for arc."""
    import k2_b200 as k2
    for max_token in (1, 2, 7, 30):
        for modified in (False, True):
            want = ref.ctc_topo(max_token, modified)
            got = k2.ctc_topo(max_token, modified)
            assert np.array_equal(got.arcs._row_splits2.numpy(), want.row_splits2)
            assert np.array_equal(got.arcs.values().numpy(), want.arcs)
            assert np.array_equal(got.aux_labels.numpy(), want.aux_labels)


def test_pruned_intersection_restatement_is_identical():
    """oracle.intersect_dense_pruned (plain C) against the reference's
    IntersectDensePruned: lattices and arc maps bit for bit, over per-sequence and
    shared graphs, beams that bind and beams that do not, allow_partial."""
    from pruned_util import decoding_graph, pruned_cases
    cases = pruned_cases(small=True) + pruned_cases(small=False)
    rng = np.random.default_rng(33)
    for trial in range(40):
        n = int(rng.integers(1, 6))
        if trial % 3 == 0:
            a = decoding_graph(rng, int(rng.integers(5, 80)), 5)
        else:
            a = random_fsa_vec(rng, n, max_states=14, max_arcs=60, max_label=4, allow_empty=True)
        scores, brs = random_dense(rng, n, int(rng.integers(1, 75)), 5, low_rows=trial % 2 == 0)
        params = (float(rng.choice([2.0, 6.0, 20.0])), float(rng.choice([1.0, 4.0, 8.0])),
                  int(rng.integers(0, 4)), int(rng.integers(4, 40)), bool(trial % 4 == 1))
        cases.append(dict(name=f"trial{trial}", a=a, scores=scores, brs=brs, params=params))
    for c in cases:
        r = ref.intersect_dense_pruned(c["a"], c["scores"], c["brs"], *c["params"])
        o = oracle.intersect_dense_pruned(c["a"], c["scores"], c["brs"], *c["params"])
        same_fsa(r, o, c["name"])

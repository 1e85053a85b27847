"""The CPU oracle against (1) fixtures produced by the reference's own CPU code
(tests/golden/ref_cases.npz) and (2) the literal known answers written in the
reference's Python tests."""
import numpy as np
import pytest

from golden_util import load
from oracle import oracle
from oracle.common import HostFsaVec, make_arcs
from util import close, same_fsa


@pytest.mark.parametrize("case", load(), ids=lambda c: c["name"])
def test_oracle_reproduces_reference_fixtures(case):
    lat = oracle.intersect_dense(case["a"], case["scores"], case["brs"], case["beam"],
                                 case["amap"])
    same_fsa(lat, case["lattice"], case["name"])
    for tag, log in (("log", True), ("trop", False)):
        f = oracle.forward_scores(lat, log, True)
        b = oracle.backward_scores(lat, log, True)
        tot, post = oracle.tot_scores_and_arc_post(lat, f, b, True)
        assert np.array_equal(f, case[f"fwd_{tag}"]) and np.array_equal(b, case[f"bwd_{tag}"])
        assert np.array_equal(tot, case[f"tot_{tag}"])
        assert np.array_equal(post, case[f"post_{tag}"], equal_nan=True)
    _, ea = oracle.forward_scores(lat, False, True, want_entering_arcs=True)
    assert np.array_equal(ea, case["entering"])
    ps, best = oracle.shortest_path(lat, ea)
    assert np.array_equal(ps, case["path_splits"]) and np.array_equal(best, case["best"])
    assert np.array_equal(oracle.properties(lat)[0], case["props"])
    if case["symbols"] is not None:
        n = 3
        lens = case["symbols"][:n]
        flat = case["symbols"][n:].tolist()
        syms, k = [], 0
        for ln in lens.tolist():
            syms.append(flat[k:k + ln])
            k += ln
        g = oracle.ctc_graphs(syms, modified=case["name"] == "ctc1")
        same_fsa(g, case["a"])
        assert np.array_equal(g.aux_labels, case["aux"])


def _dense(log_probs_list):
    """DenseFsaVec layout for a list of [T_i, C] arrays (already sorted)."""
    C = log_probs_list[0].shape[1]
    rows = sum(x.shape[0] + 1 for x in log_probs_list)
    scores = np.full((rows, C + 1), -np.inf, np.float32)
    brs = [0]
    r = 0
    for x in log_probs_list:
        scores[r:r + x.shape[0], 1:] = x
        scores[r + x.shape[0], 0] = 0
        r += x.shape[0] + 1
        brs.append(r)
    return scores, np.asarray(brs, np.int32)


def _fsa(rows, num_states):
    r = np.asarray(rows, np.float64)
    arcs = make_arcs(r[:, 0].astype(np.int32), r[:, 1].astype(np.int32), r[:, 2].astype(np.int32),
                     r[:, 3].astype(np.float32))
    rs2 = np.zeros(num_states + 1, np.int32)
    np.add.at(rs2, r[:, 0].astype(np.int64) + 1, 1)
    return HostFsaVec(np.array([0, num_states], np.int32), np.cumsum(rs2).astype(np.int32), arcs)


def test_intersect_dense_simple_known_answer():
    # k2/python/tests/intersect_dense_test.py:40-88 (expected values computed with gtn)
    a = _fsa([(0, 1, 1, 1.0), (1, 1, 1, 50.0), (1, 2, 2, 2.0), (2, 3, -1, 3.0)], 4)
    scores, brs = _dense([np.array([[0.1, 0.2, 0.3], [0.04, 0.05, 0.06]], np.float32)])
    out = oracle.loss_path(a, scores, brs, 100000.0, use_double=False, log_semiring=False)
    assert np.allclose(out["lattice"].scores, [1.2, 2.06, 3.0])
    # tropical gradient: 1 on the best path
    _, ea = oracle.forward_scores(out["lattice"], False, False, want_entering_arcs=True)
    _, best = oracle.shortest_path(out["lattice"], ea)
    grad_a = np.zeros(4)
    np.add.at(grad_a, out["lattice"].arc_map_a[best], 1.0)
    assert grad_a.tolist() == [1.0, 0.0, 1.0, 1.0]
    grad_b = np.zeros(scores.size)
    np.add.at(grad_b, out["lattice"].arc_map_b[best], 1.0)
    grad_lp = grad_b.reshape(scores.shape)[:2, 1:]
    assert grad_lp.reshape(-1).tolist() == [0.0, 1.0, 0.0, 0.0, 0.0, 1.0]


def test_get_tot_scores_known_answers():
    # k2/python/tests/get_tot_scores_test.py:197-326 (gtn values)
    f1 = _fsa([(0, 1, 1, 0.1), (0, 2, 2, 0.2), (1, 2, 3, 0.3), (1, 3, 4, 0.4), (2, 3, 5, 0.5),
               (3, 4, -1, 0)], 5)
    f2 = _fsa([(0, 3, 3, 0.1), (0, 1, 1, 0.2), (0, 2, 2, 0.3), (1, 2, 2, 0.4), (1, 3, 3, 0.5),
               (2, 3, 3, 0.6), (2, 4, 4, 0.7), (3, 4, 4, 0.8), (3, 5, -1, 0.9), (4, 5, -1, 1.0)], 6)
    want_tot = [1.8119014501571655, 4.533502578735352]
    want_grad = [[0.6710670590400696, 0.32893291115760803, 0.4017595648765564,
                  0.2693074941635132, 0.7306925058364868, 1.0],
                 [0.10102888941764832, 0.5947467088699341, 0.3042244613170624, 0.410660058259964,
                  0.1840866357088089, 0.5283515453338623, 0.18653297424316406,
                  0.5783339142799377, 0.2351330667734146, 0.764866828918457]]
    for f, t, g in zip((f1, f2), want_tot, want_grad):
        for dbl in (False, True):
            fwd = oracle.forward_scores(f, True, dbl)
            bwd = oracle.backward_scores(f, True, dbl)
            tot, post = oracle.tot_scores_and_arc_post(f, fwd, bwd, dbl)
            assert abs(tot[0] - t) < 1e-5
            assert np.allclose(np.exp(post), g, atol=1e-5)


def _log_softmax(x):
    x = np.asarray(x, np.float64)
    return (x - np.log(np.exp(x - x.max(-1, keepdims=True)).sum(-1, keepdims=True))
            - x.max(-1, keepdims=True)).astype(np.float32)


def test_ctc_loss_known_answers():
    # k2/python/tests/ctc_loss_test.py:69-309: literal losses, also equal to
    # torch.nn.functional.ctc_loss there
    act3 = [[-5, -4, -3, -2, -1], [-10, -9, -8, -7, -6], [-15, -14, -13, -12, -11.]]
    act2 = np.arange(1, 16).reshape(3, 5)
    act1 = [[0.2] * 5]
    cases = [(act1, [1], 1.6094379425049), (act2, [3, 3], 7.355742931366),
             (act3, [2, 3], 4.938850402832)]
    for act, target, want in cases:
        g = oracle.ctc_graphs([target])
        scores, brs = _dense([_log_softmax(act)])
        out = oracle.loss_path(g, scores, brs, 10.0)
        assert abs(-out["tot_scores"][0] - want) < 1e-5
    # the batch of three, sorted by length (ctc_loss_test.py:232-309)
    g = oracle.ctc_graphs([[2, 3], [3, 3], [1]])
    scores, brs = _dense([_log_softmax(act3), _log_softmax(act2), _log_softmax(act1)])
    out = oracle.loss_path(g, scores, brs, 10.0)
    assert abs(-out["tot_scores"].sum() - (4.938850402832 + 7.355742931366 + 1.6094379425049)) < 1e-4

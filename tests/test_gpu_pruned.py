"""Pruned intersection (k2.intersect_dense_pruned) on the GPU: bit-identical lattices
and arc maps.  The small cases are checked against the reference's own answers
(tests/golden/pruned_cases.npz, made by tests/golden/make_pruned_golden.py); the
larger ones against the C restatement in oracle/ (itself pinned against the
reference on CPU, tests/test_oracle_vs_reference.py) and, when it has been built,
against the reference library too (oracle/_ref)."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle, ref
from oracle.common import HostFsaVec
from pruned_util import decoding_graph, pruned_cases
from util import random_dense, same_fsa

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "pruned_cases.npz")


@pytest.fixture(scope="module")
def k2():
    import k2_b200
    return k2_b200


def run_gpu(k2, c, team_ctas=0):
    from gpu_util import dense_from_scores, fsa_to_host, host_to_fsa
    from k2_b200.autograd import _intersect_dense_pruned_arcs
    a = host_to_fsa(c["a"])
    dense = dense_from_scores(c["scores"], c["brs"])
    sb, ob, mn, mx, partial = c["params"]
    ragged, ma, mb = _intersect_dense_pruned_arcs(a.arcs, dense, sb, ob, mn, mx, partial,
                                                  team_ctas)
    lat = k2.Fsa(ragged, _check=False)
    return lat, fsa_to_host(lat, ma, mb)


def test_small_cases_match_the_committed_reference_answers(k2):
    z = np.load(GOLDEN)
    cases = {c["name"]: c for c in pruned_cases(small=True)}
    assert sorted(cases) == sorted(z["names"].tolist())
    for name, c in cases.items():
        want = HostFsaVec(z[f"{name}.l_rs1"], z[f"{name}.l_rs2"], z[f"{name}.l_arcs"],
                          arc_map_a=z[f"{name}.map_a"], arc_map_b=z[f"{name}.map_b"])
        for team in (0, 1, 2, 8):
            _, got = run_gpu(k2, c, team)
            same_fsa(got, want, f"{name}, {team} CTAs per sequence")


def test_larger_cases_match_the_oracle_and_the_reference_library(k2):
    for c in pruned_cases(small=False):
        want = oracle.intersect_dense_pruned(c["a"], c["scores"], c["brs"], *c["params"])
        _, got = run_gpu(k2, c)
        same_fsa(got, want, c["name"])
        if ref.available():
            same_fsa(got, ref.intersect_dense_pruned(c["a"], c["scores"], c["brs"],
                                                     *c["params"]), c["name"] + " (reference)")


def test_decoding_graph_many_windows(k2):
    rng = np.random.default_rng(5)
    g = decoding_graph(rng, 3000, 40, mean_degree=4.0)
    scores, brs = random_dense(rng, 6, 300, 40, scale=2.0, low_rows=False)
    for params in ((12.0, 5.0, 30, 400, False), (8.0, 4.0, 10, 60, True)):
        c = dict(a=g, scores=scores, brs=brs, params=params)
        want = oracle.intersect_dense_pruned(g, scores, brs, *params)
        for team in (1, 4):
            lat, got = run_gpu(k2, c, team)
            same_fsa(got, want, f"{params}, {team} CTAs per sequence")
        assert want.num_arcs > 1000


def test_public_api_scores_attributes_and_gradients(k2):
    from gpu_util import DEV, host_to_fsa
    c = pruned_cases(small=True)[0]
    a = host_to_fsa(c["a"])
    a.aux_labels = torch.arange(a.arcs.num_elements(), dtype=torch.int32, device=DEV)
    a.scores.requires_grad_(True)
    scores = torch.from_numpy(c["scores"]).to(DEV).requires_grad_(True)
    dense = k2.DenseFsaVec._from_dense_fsa_vec(scores, c["brs"])
    lat = k2.intersect_dense_pruned(a, dense, 20.0, 8.0, 0, 10000, seqframe_idx_name="seqframe",
                                    frame_idx_name="frame")
    z = np.load(GOLDEN)
    map_a, map_b = z["ctc_wide.map_a"], z["ctc_wide.map_b"]
    np.testing.assert_array_equal(lat.aux_labels.cpu().numpy(), map_a)
    np.testing.assert_array_equal(lat.seqframe.cpu().numpy(), map_b // c["scores"].shape[1])
    row_of = np.repeat(np.arange(len(c["brs"]) - 1), np.diff(c["brs"]))
    np.testing.assert_array_equal(lat.frame.cpu().numpy(),
                                  map_b // c["scores"].shape[1] - c["brs"][row_of[
                                      map_b // c["scores"].shape[1]]])
    w = torch.linspace(0.5, 1.5, lat.scores.numel(), device=DEV)
    (lat.scores * w).sum().backward()
    ga = np.zeros(a.arcs.num_elements(), np.float32)
    np.add.at(ga, map_a, w.cpu().numpy())
    gb = np.zeros(c["scores"].size, np.float32)
    np.add.at(gb, map_b, w.cpu().numpy())
    np.testing.assert_allclose(a.scores.grad.cpu().numpy(), ga, rtol=1e-6)
    np.testing.assert_allclose(scores.grad.cpu().numpy().reshape(-1), gb, rtol=1e-6)
    # the lattice is a valid, top-sorted FsaVec whose best path has the tropical total
    tot = lat.get_tot_scores(use_double_scores=True, log_semiring=False)
    best = k2.shortest_path(lat, use_double_scores=True)
    assert torch.allclose(best.get_tot_scores(use_double_scores=True, log_semiring=False), tot)


def test_argument_checks(k2):
    from gpu_util import dense_from_scores, host_to_fsa
    cs = pruned_cases(small=True)
    a = host_to_fsa(cs[0]["a"])
    dense = dense_from_scores(cs[0]["scores"], cs[0]["brs"])
    with pytest.raises(RuntimeError, match="positive"):
        k2.intersect_dense_pruned(a, dense, 0.0, 8.0, 0, 100)
    with pytest.raises(RuntimeError, match="min_active"):
        k2.intersect_dense_pruned(a, dense, 20.0, 8.0, 10, 10)
    two = host_to_fsa(HostFsaVec(cs[0]["a"].row_splits1[:3], cs[0]["a"].row_splits2[
        :cs[0]["a"].row_splits1[2] + 1], cs[0]["a"].arcs[:cs[0]["a"].row_splits2[
            cs[0]["a"].row_splits1[2]]]))
    with pytest.raises(RuntimeError, match="one graph per sequence"):
        k2.intersect_dense_pruned(two, dense, 20.0, 8.0, 0, 100)


def test_small_arena_is_grown(k2, monkeypatch):
    from k2_b200 import autograd
    monkeypatch.setattr(autograd, "PRUNED_ARCS_TOTAL", 1 << 8)
    monkeypatch.setattr(autograd, "PRUNED_ARCS_MIN", 1 << 6)
    monkeypatch.setattr(autograd, "_pruned_capacity", {})
    c = pruned_cases(small=True)[3]
    z = np.load(GOLDEN)
    want = HostFsaVec(z["shared_wide.l_rs1"], z["shared_wide.l_rs2"], z["shared_wide.l_arcs"],
                      arc_map_a=z["shared_wide.map_a"], arc_map_b=z["shared_wide.map_b"])
    _, got = run_gpu(k2, c)
    same_fsa(got, want, "after growing the arena")
    assert list(autograd._pruned_capacity.values())[0] > 1 << 6


def test_best_path_agrees_with_the_exact_intersection_on_a_decoding_graph(k2):
    """Scaled-down decoding configuration (20 000-state graph shared by 8 sequences of
    100 frames): with a wide search beam the pruned lattice holds the same best path,
    with the same score, as the exact intersect_dense lattice."""
    from gpu_util import DEV
    from k2_b200 import synthetic as syn
    from k2_b200.fsa_algo import _fsa_vec_from_numpy
    w = syn.hlg_decode(seed=3, scale=0.25, num_states=20000)
    S = len(w.graph_row_splits2) - 1
    shared = _fsa_vec_from_numpy(np.array([0, S]), w.graph_row_splits2, w.graph_arcs, DEV)
    stacked = syn.build_graphs(w, DEV)
    dense = k2.DenseFsaVec(w.log_probs.to(DEV), w.supervision_segments)
    exact = k2.intersect_dense(stacked, dense, output_beam=8.0)
    pruned = k2.intersect_dense_pruned(shared, dense, 40.0, 8.0, 30, 100000)
    te = exact.get_tot_scores(use_double_scores=True, log_semiring=False)
    tp = pruned.get_tot_scores(use_double_scores=True, log_semiring=False)
    assert torch.isfinite(te).all()
    assert torch.allclose(te, tp, rtol=1e-6, atol=1e-4)
    be = k2.shortest_path(exact, use_double_scores=True)
    bp = k2.shortest_path(pruned, use_double_scores=True)
    assert torch.equal(be.arcs.values()[:, 2], bp.arcs.values()[:, 2])
    # the search with everyday limits never scores above the exact best path
    narrow = k2.intersect_dense_pruned(shared, dense, 20.0, 8.0, 30, 10000)
    tn = narrow.get_tot_scores(use_double_scores=True, log_semiring=False)
    assert (tn <= te + 1e-4).all()


def test_many_sequences_with_their_own_graphs(k2):
    """More sequences than SMs (one CTA per sequence), one CTC graph each, lengths from
    1 frame to several pruning windows."""
    rng = np.random.default_rng(9)
    n = 200
    syms = [[int(x) for x in rng.integers(1, 9, size=int(rng.integers(1, 12)))] for _ in range(n)]
    scores, brs = random_dense(rng, n, 70, 9, low_rows=False)
    assert np.diff(brs).min() == 2  # a sequence of a single frame
    g = oracle.ctc_graphs(syms, False)
    for params in ((20.0, 8.0, 0, 1000, False), (5.0, 3.0, 4, 12, True)):
        want = oracle.intersect_dense_pruned(g, scores, brs, *params)
        _, got = run_gpu(k2, dict(a=g, scores=scores, brs=brs, params=params))
        same_fsa(got, want, str(params))


def test_decode_helpers_recover_the_transcripts(k2):
    """get_lattice / one_best_decoding / get_aux_labels (k2/python/k2/decode.py) on
    log-probs peaked along a valid CTC alignment, with tensor and ragged aux_labels."""
    from gpu_util import DEV
    rng = np.random.default_rng(2)
    texts = [[int(x) for x in rng.integers(1, 9, size=int(rng.integers(2, 7)))] for _ in range(4)]
    T, C = 40, 9
    logits = torch.full((len(texts), T, C), -4.0)
    lens = []
    for i, text in enumerate(texts):
        t = 0
        for sym in text:
            logits[i, t, 0] = 4.0          # a blank, then the symbol twice
            logits[i, t + 1, sym] = 4.0
            logits[i, t + 2, sym] = 4.0
            t += 3
        logits[i, t:, 0] = 4.0
        lens.append(min(T, t + 2 + i))
    log_prob = torch.log_softmax(logits, -1).to(DEV)
    graphs = k2.ctc_graph(texts, device=DEV)
    lattice = k2.get_lattice(log_prob, torch.tensor(lens), graphs, search_beam=20, output_beam=8,
                             min_active_states=0, max_active_states=1000)
    best = k2.one_best_decoding(lattice)
    assert k2.get_aux_labels(best) == texts
    # the same with a list per arc instead of one symbol per arc
    aux = graphs.aux_labels.cpu().tolist()
    del graphs.aux_labels
    graphs.aux_labels = k2.RaggedTensor([[x] if x != 0 else [] for x in aux], device=DEV)
    lattice = k2.get_lattice(log_prob, torch.tensor(lens), graphs, min_active_states=0)
    assert k2.get_aux_labels(k2.one_best_decoding(lattice)) == texts


def test_ctc_decoding_with_the_shared_topology(k2):
    """get_lattice with H = ctc_topo shared by the batch: greedy-like CTC decoding of
    peaked log-probs gives back the symbol sequences."""
    from gpu_util import DEV
    rng = np.random.default_rng(6)
    C = 12
    texts = [[int(x) for x in rng.integers(1, C, size=int(rng.integers(1, 8)))] for _ in range(5)]
    T = 30
    logits = torch.full((len(texts), T, C), -5.0)
    for i, text in enumerate(texts):
        t = 0
        for sym in text:
            logits[i, t, 0] = 5.0
            logits[i, t + 1, sym] = 5.0
            t += 2
        logits[i, t:, 0] = 5.0
    log_prob = torch.log_softmax(logits, -1).to(DEV)
    lens = torch.full((len(texts),), T)
    for modified in (False, True):
        H = k2.ctc_topo(C - 1, modified=modified, device=DEV)
        lattice = k2.get_lattice(log_prob, lens, H, min_active_states=0)
        assert k2.get_aux_labels(k2.one_best_decoding(lattice)) == texts

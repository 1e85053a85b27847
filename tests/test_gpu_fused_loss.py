"""The lattice-free loss path (`intersect_dense_tot_scores`, used by `ctc_loss`)
against the CPU oracle's intersect_dense -> forward/backward -> posteriors chain
and against this package's own lattice path on the same inputs.

Total scores agree to 1e-6 relative (1e-4 is the tolerance of the path): the lattice
rounds every arc score (graph score + dense score) to float32 before the float64
sums, the lattice-free recursion multiplies the two exact factors instead.
Gradients w.r.t. graph scores and dense scores: 1e-4 absolute."""
import numpy as np
import pytest
import torch

from oracle import oracle
from util import close, random_dense, random_fsa_vec

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _fused(a_host, scores, brs, beam, amap=None, tot_grad=None, use_double=True,
           want_grad_a=True, **limits):
    import k2_b200 as k2
    from gpu_util import dense_from_scores, host_to_fsa
    fsa = host_to_fsa(a_host)
    fsa.scores.requires_grad_(want_grad_a)
    dense = dense_from_scores(scores, brs, requires_grad=True)
    m = None if amap is None else torch.as_tensor(amap, dtype=torch.int32)
    assert k2.dense_loss_supported(fsa, dense, m)
    tot = k2.intersect_dense_tot_scores(fsa, dense, beam, a_to_b_map=m,
                                        use_double_scores=use_double, **limits)
    g = torch.ones_like(tot) if tot_grad is None else torch.as_tensor(
        tot_grad, dtype=tot.dtype, device=tot.device)
    finite = torch.isfinite(tot)
    if bool(finite.any()):
        (tot[finite] * g[finite]).sum().backward()
        gb = dense.scores.grad.cpu().numpy()
        ga = fsa.scores.grad.cpu().numpy() if want_grad_a else None
    else:
        ga = np.zeros(a_host.num_arcs, np.float32)
        gb = np.zeros(scores.shape, np.float32)
    return tot.detach().cpu().numpy(), ga, gb


def _compare(a, scores, brs, beam, amap=None, tot_grad=None, tag=""):
    want = oracle.loss_path(a, scores, brs, beam, amap, tot_grad=tot_grad)
    tot, ga, gb = _fused(a, scores, brs, beam, amap, tot_grad)
    assert close(tot, want["tot_scores"], rtol=1e-6, atol=1e-6), (tag, tot, want["tot_scores"])
    assert np.abs(ga - want["grad_a"]).max(initial=0) <= 1e-4, tag
    assert np.abs(gb - want["grad_b"]).max(initial=0) <= 1e-4, tag


def test_random_fsa_vecs():
    rng = np.random.default_rng(11)
    for trial in range(60):
        n = int(rng.integers(1, 7))
        a = random_fsa_vec(rng, n, acyclic=bool(trial % 2))
        scores, brs = random_dense(rng, n, 10, 5)
        beam = float(rng.choice([0.5, 2.0, 10.0, 100.0]))
        amap = None
        if trial % 4 == 0:
            amap = np.sort(rng.integers(0, n, size=n)).astype(np.int32)
        tot_grad = rng.normal(size=n) if trial % 3 == 0 else None
        _compare(a, scores, brs, beam, amap, tot_grad, f"trial {trial}")


def test_extreme_scores_take_the_per_state_exponent_kernels():
    # arc scores of +-100 and dense rows near -300 are outside what the
    # shared-exponent recursion accepts: those graphs are recomputed by the
    # mantissa/exponent kernels; the results must not show the seam
    rng = np.random.default_rng(23)
    for trial in range(12):
        n = int(rng.integers(1, 5))
        a = random_fsa_vec(rng, n, acyclic=bool(trial % 2))
        scores, brs = random_dense(rng, n, 10, 5, low_rows=False)
        if trial % 3 == 0:
            a.arcs[:, 3] = (a.scores * 40.0).astype(np.float32).view(np.int32)
        elif trial % 3 == 1:
            finite = np.isfinite(scores)
            scores = np.where(finite, scores * 150.0, scores).astype(np.float32)
        else:
            a.arcs[::3, 3] = np.float32(-np.inf).view(np.int32)
        _compare(a, scores, brs, 1.0e4 if trial % 3 else 50.0, tag=f"extreme {trial}")


def test_dense_gradient_alone():
    # without a gradient for the graph scores: graphs in which every state has one label
    # (CTC graphs, the LF-MMI denominator graph) take it from state posteriors, all others
    # from the arc posteriors as before; same numbers either way
    from gpu_util import fsa_to_host
    from k2_b200 import synthetic as syn
    import k2_b200 as k2
    rng = np.random.default_rng(31)
    for trial in range(12):
        n = int(rng.integers(1, 6))
        a = random_fsa_vec(rng, n, acyclic=bool(trial % 2))
        scores, brs = random_dense(rng, n, 10, 5)
        amap = np.sort(rng.integers(0, n, size=n)).astype(np.int32) if trial % 4 == 0 else None
        tot_grad = rng.normal(size=n)
        want = oracle.loss_path(a, scores, brs, 5.0, amap, tot_grad=tot_grad)
        tot, ga, gb = _fused(a, scores, brs, 5.0, amap, tot_grad, want_grad_a=False)
        assert close(tot, want["tot_scores"], rtol=1e-6, atol=1e-6)
        assert np.abs(gb - want["grad_b"]).max(initial=0) <= 1e-4, trial
    for name in ("ctc_small", "lfmmi_den"):
        w = syn.WORKLOADS[name](scale=0.25)
        graphs = syn.build_graphs(w, DEV)
        dense = k2.DenseFsaVec(w.log_probs.to(DEV), w.supervision_segments)
        a, scores, brs = fsa_to_host(graphs), dense.scores.cpu().numpy(), dense.h_row_splits
        want = oracle.loss_path(a, scores, brs, w.output_beam)
        tot, _, gb = _fused(a, scores, brs, w.output_beam, want_grad_a=False)
        assert close(tot, want["tot_scores"], rtol=1e-6, atol=1e-6)
        assert np.abs(gb - want["grad_b"]).max(initial=0) <= 1e-4, name


def test_micro_example():
    from test_gpu_parity import _micro
    a, scores, brs = _micro()
    _compare(a, scores, brs, 100.0)
    _compare(a, scores, brs, 0.4)


@pytest.mark.parametrize("name", ["ctc_small", "ctc_modified", "lfmmi_den"])
def test_workloads_against_oracle(name):
    from gpu_util import fsa_to_host
    from k2_b200 import synthetic as syn
    w = syn.WORKLOADS[name](scale=0.25)
    graphs = syn.build_graphs(w, DEV)
    import k2_b200 as k2
    dense = k2.DenseFsaVec(w.log_probs.to(DEV), w.supervision_segments)
    _compare(fsa_to_host(graphs), dense.scores.cpu().numpy(), dense.h_row_splits, w.output_beam,
             tag=name)


def test_float32_output_and_beam_reduction():
    rng = np.random.default_rng(5)
    a = random_fsa_vec(rng, 4, acyclic=False)
    scores, brs = random_dense(rng, 4, 12, 5, low_rows=False)
    want = oracle.loss_path(a, scores, brs, 50.0)
    tot, _, _ = _fused(a, scores, brs, 50.0, use_double=False)
    assert tot.dtype == np.float32
    assert close(tot, want["tot_scores"], rtol=1e-4, atol=1e-4)
    # a state limit below the beam-50 lattice forces the reference's beam shrinking
    lat = want["lattice"]
    if lat.num_states > 20:
        limit = int(lat.num_states * 0.7)
        shrunk = oracle.intersect_dense(a, scores, brs, 50.0, max_states=limit)
        if 0 < shrunk.num_states <= limit:
            import k2_b200 as k2  # noqa: F401
            from gpu_util import dense_from_scores, host_to_fsa, intersect_raw
            lat2, _, _ = intersect_raw(host_to_fsa(a), dense_from_scores(scores, brs), 50.0,
                                       max_states=limit)
            ref_tot = lat2.get_tot_scores(True, True).cpu().numpy()
            tot2, _, _ = _fused(a, scores, brs, 50.0, max_states=limit)
            assert close(tot2, ref_tot, rtol=1e-6, atol=1e-6)


def test_ctc_loss_uses_the_same_numbers_either_way():
    import k2_b200 as k2
    from k2_b200 import ctc_loss as ctc_mod
    from k2_b200 import synthetic as syn
    w = syn.ctc_small(scale=0.5)
    graphs = syn.build_graphs(w, DEV)
    out = {}
    for fused in (True, False):
        lp = w.log_probs.to(DEV).requires_grad_(True)
        dense = k2.DenseFsaVec(lp, w.supervision_segments)
        ctc_mod.FUSED_LOSS = fused
        try:
            loss = k2.ctc_loss(graphs, dense, output_beam=w.output_beam, reduction="sum")
        finally:
            ctc_mod.FUSED_LOSS = True
        loss.backward()
        out[fused] = (float(loss.detach()), lp.grad.cpu().numpy())
    assert abs(out[True][0] - out[False][0]) <= 1e-6 * abs(out[False][0])
    assert np.abs(out[True][1] - out[False][1]).max() <= 1e-4


def _star_graph(rng, fan, tail_states, num_labels):
    """A graph whose start state has `fan` leaving arcs (more than a lane plan can
    place when fan > 256), followed by a few random states, all reaching the final
    state."""
    rows = []
    mid = list(range(1, 1 + tail_states))
    final = 1 + tail_states
    for k in range(fan):
        rows.append((0, mid[k % tail_states], int(rng.integers(0, num_labels)), float(rng.normal())))
    for s in mid:
        for _ in range(3):
            d = int(rng.integers(1, final))
            rows.append((s, d, int(rng.integers(0, num_labels)), float(rng.normal())))
        rows.append((s, final, -1, float(rng.normal())))
    rows.sort(key=lambda r: r[0])
    return rows, final + 1


def _stars(rng, fans):
    """An FsaVec of star graphs, one per entry of `fans`."""
    from oracle.common import HostFsaVec, make_arcs
    rs1, rs2, arcs = [0], [0], []
    for fan in fans:
        rows, ns = _star_graph(rng, fan, 6, 5)
        base = len(arcs)
        src = np.array([r[0] for r in rows])
        for s in range(ns):
            rs2.append(base + int(np.sum(src <= s)))
        arcs.extend(rows)
        rs1.append(rs1[-1] + ns)
    r = np.array(arcs, dtype=np.float64)
    return HostFsaVec(np.asarray(rs1, np.int32), np.asarray(rs2, np.int32),
                      make_arcs(r[:, 0].astype(np.int32), r[:, 1].astype(np.int32),
                                r[:, 2].astype(np.int32), r[:, 3].astype(np.float32)))


def test_graphs_a_plan_cannot_place_take_the_fallback_kernels():
    # one graph with a 300-arc state (no lane plan possible: > 32 lanes of 8 arcs)
    # next to ordinary ones: plan-less graphs go through PersistentViterbi, GridChain
    # and GridGradWarp while the others keep the planned kernels, in the same call
    from oracle.common import HostFsaVec, make_arcs
    rng = np.random.default_rng(17)
    rs1, rs2, arcs = [0], [0], []
    for fan in (300, 12, 40):
        rows, ns = _star_graph(rng, fan, 6, 5)
        base = len(arcs)
        src = np.array([r[0] for r in rows])
        for s in range(ns):
            rs2.append(base + int(np.sum(src <= s)))
        arcs.extend(rows)
        rs1.append(rs1[-1] + ns)
    r = np.array(arcs, dtype=np.float64)
    a = HostFsaVec(np.asarray(rs1, np.int32), np.asarray(rs2, np.int32),
                   make_arcs(r[:, 0].astype(np.int32), r[:, 1].astype(np.int32),
                             r[:, 2].astype(np.int32), r[:, 3].astype(np.float32)))
    scores, brs = random_dense(rng, 3, 14, 5, low_rows=False)
    for beam in (4.0, 30.0):
        _compare(a, scores, brs, beam, tag=f"star beam {beam}")
    # the lattice path on the same batch: planned Viterbi for two graphs, the
    # shared-memory kernel for the third, bit-exact lattice
    from gpu_util import dense_from_scores, fsa_to_host, host_to_fsa, intersect_raw
    from util import same_fsa
    lat, ma, mb = intersect_raw(host_to_fsa(a), dense_from_scores(scores, brs), 30.0, mode=0)
    same_fsa(fsa_to_host(lat, ma, mb), oracle.intersect_dense(a, scores, brs, 30.0), "star lattice")


def test_ctc_graphs_with_more_than_512_states():
    # the 1024-thread instantiations of the register kernels
    import k2_b200 as k2
    from gpu_util import fsa_to_host
    rng = np.random.default_rng(19)
    syms = [[int(x) for x in rng.integers(1, 20, size=n)] for n in (300, 280)]
    graphs = k2.ctc_graph(syms, device=DEV)
    assert graphs.arcs.num_states > 1024 and max(np.diff(graphs.arcs.h_row_splits1)) > 512
    T = 330
    lp = torch.log_softmax(torch.randn(2, T, 20, generator=torch.Generator().manual_seed(1)) * 2, -1)
    segs = torch.tensor([[0, 0, T], [1, 0, T - 10]], dtype=torch.int32)
    dense = k2.DenseFsaVec(lp.to(DEV), segs)
    _compare(fsa_to_host(graphs), dense.scores.cpu().numpy(), dense.h_row_splits, 12.0,
             tag="long ctc")


def test_gradient_goes_straight_to_the_log_probs():
    """A DenseFsaVec made from a log-prob tensor hands the loss that tensor: the
    gradient written in its layout is bit-identical to the one that travels through
    the score matrix and the adjoint of the layout, with offsets, truncation, a
    permuted and duplicated a_to_b_map."""
    import k2_b200 as k2
    rng = np.random.default_rng(8)
    N, T, C = 5, 23, 7
    lp0 = torch.log_softmax(torch.from_numpy(rng.normal(size=(N, T, C)).astype(np.float32)), -1)
    seg = torch.tensor([[3, 0, 23], [0, 2, 20], [4, 1, 15], [1, 5, 9]], dtype=torch.int32)
    texts = [[1, 2, 3], [4, 4], [5], [2, 6, 1]]
    for a_to_b in (None, torch.tensor([0, 1, 1, 3, 3], dtype=torch.int32)):
        n_graphs = 4 if a_to_b is None else 5
        graphs = k2.ctc_graph((texts + [[3, 3, 1]])[:n_graphs], device=DEV)
        grads = []
        for direct in (True, False):
            lp = lp0.clone().to(DEV).requires_grad_(True)
            dense = k2.DenseFsaVec(lp, seg, allow_truncate=0)
            assert dense._source is not None
            if not direct:
                dense._source = None
            tot = k2.intersect_dense_tot_scores(graphs, dense, 10.0, a_to_b_map=a_to_b)
            w = torch.linspace(0.5, 2.0, tot.numel(), device=DEV, dtype=tot.dtype)
            (tot * w).sum().backward()
            grads.append(lp.grad.clone())
        assert torch.isfinite(grads[0]).all() and grads[0].abs().sum() > 0
        if a_to_b is None:
            assert torch.equal(grads[0], grads[1])
        else:  # rows shared by two graphs are summed with atomics: order may differ
            assert torch.allclose(grads[0], grads[1], rtol=1e-6, atol=1e-7)
    # overlapping segments keep the route through the score matrix
    lp = lp0.clone().to(DEV).requires_grad_(True)
    over = k2.DenseFsaVec(lp, torch.tensor([[0, 0, 20], [0, 10, 13]], dtype=torch.int32))
    assert over._source is None


def test_bounded_waits_of_the_lane_kernels_expire_and_the_fallback_takes_over():
    """With a poll limit of 0 the waits of GridChainLanes / GridChainMasked for their row
    copies run out: they flag the graph and return (nothing traps or hangs), the
    shared-memory fallback launched behind them recomputes it, and totals and gradients
    are the oracle's - for graphs on identity lanes and for graphs on a lane plan."""
    from k2_b200 import _lib
    rng = np.random.default_rng(77)
    cases = []
    for trial in range(4):  # degree <= 4: identity lanes (GridChainLanes)
        n = int(rng.integers(1, 4))
        cases.append((random_fsa_vec(rng, n, acyclic=bool(trial % 2)),) + random_dense(rng, n, 12, 5))
    # states of 12 and 40 arcs: a lane plan (GridChainMasked)
    cases.append((_stars(rng, (12, 40)),) + random_dense(rng, 2, 14, 5, low_rows=False))
    try:
        _lib.lib.k2b200_debug_set_copy_wait_limit(0)
        for k, (a, scores, brs) in enumerate(cases):
            _compare(a, scores, brs, 10.0, tag=f"wait limit 0, case {k}")
    finally:
        _lib.lib.k2b200_debug_set_copy_wait_limit(-1)
    for k, (a, scores, brs) in enumerate(cases):
        _compare(a, scores, brs, 10.0, tag=f"default limit, case {k}")

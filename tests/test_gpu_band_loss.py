"""The band-graph kernels of the lattice-free loss (`k2b200_band_loss_*`, taken by
`intersect_dense_tot_scores` and `ctc_loss` for CTC-shaped graphs on a DenseFsaVec made
from a log-prob tensor) against the CPU oracle's intersect_dense -> forward/backward
-> posteriors chain, against the general lattice-free kernels and against the lattice
path of this package on the same inputs.

Tolerances: total scores 1e-6 relative (the path's own is 1e-4: the lattice rounds
arc score + dense score to float32 before its float64 sums, these kernels multiply the
two exact factors); gradients 1e-4 absolute."""
import numpy as np
import pytest
import torch

from oracle import oracle
from oracle.common import HostFsaVec, make_arcs
from util import close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def random_band_graphs(rng, n, max_states, num_classes, zero_scores=False):
    """Random graphs of the band shape: arcs s -> s, s+1, s+2 only, one label per
    destination state, -1 on (all and only) the arcs into the last state."""
    rs1, rs2, rows = [0], [0], []
    for _ in range(n):
        ns = int(rng.integers(2, max_states + 1))
        lab = rng.integers(0, num_classes + (1 if rng.random() < 0.2 else 0), size=ns)
        lab[ns - 1] = -1
        for s in range(ns - 1):
            for d in (0, 1, 2):
                if s + d > ns - 1 or rng.random() < 0.25:
                    continue
                w = 0.0 if zero_scores else float(np.float32(rng.normal()))
                if not zero_scores and rng.random() < 0.03:
                    w = -np.inf
                rows.append((s, s + d, int(lab[s + d]), w))
            rs2.append(len(rows))
        rs2.append(len(rows))  # the final state has no arcs
        rs1.append(rs1[-1] + ns)
    r = np.array(rows, dtype=np.float64).reshape(-1, 4)
    arcs = make_arcs(r[:, 0].astype(np.int32), r[:, 1].astype(np.int32),
                     r[:, 2].astype(np.int32), r[:, 3].astype(np.float32))
    return HostFsaVec(np.asarray(rs1, np.int32), np.asarray(rs2, np.int32), arcs)


def random_log_probs(rng, n, max_frames, num_classes, scale=1.0, low=False):
    """log_probs [n, T, C] and supervision segments sorted by decreasing duration."""
    durs = np.sort(rng.integers(1, max_frames + 1, size=n))[::-1]
    T = int(durs.max())
    x = (rng.normal(size=(n, T, num_classes)) * scale).astype(np.float32)
    x = x - np.log(np.exp(x.astype(np.float64)).sum(-1, keepdims=True)).astype(np.float32)
    if low:
        x[rng.random(size=x.shape[:2]) < 0.1] -= 120.0
    seg = np.stack([np.arange(n), np.zeros(n, np.int64), durs], axis=1).astype(np.int32)
    return torch.from_numpy(x), torch.from_numpy(seg)


def host_scores(lp, seg):
    lp = lp.numpy()
    N, T, C = lp.shape
    seg = seg.numpy()
    rows = int(seg[:, 2].sum() + len(seg))
    scores = np.full((rows, C + 1), -np.inf, np.float32)
    brs = np.zeros(len(seg) + 1, np.int32)
    r = 0
    for i, (n, s, d) in enumerate(seg.tolist()):
        scores[r:r + d, 1:] = lp[n, s:s + d]
        scores[r + d, 0] = 0.0
        r += d + 1
        brs[i + 1] = r
    return scores, brs


def to_lp_layout(grad_scores, lp_shape, seg):
    out = np.zeros(lp_shape, np.float32)
    r = 0
    for (n, s, d) in seg.numpy().tolist():
        out[n, s:s + d] += grad_scores[r:r + d, 1:]
        r += d + 1
    return out


def run(a_host, lp, seg, beam, amap=None, tot_grad=None, band=True, scores_layout=False,
        **limits):
    import k2_b200 as k2
    from gpu_util import host_to_fsa
    fsa = host_to_fsa(a_host)
    fsa.scores.requires_grad_(True)
    lpd = lp.to(DEV)
    if not scores_layout:
        lpd.requires_grad_(True)
    dense = k2.DenseFsaVec(lpd, seg)
    leaf = lpd
    if scores_layout:
        leaf = dense.scores.requires_grad_(True)
    m = None if amap is None else torch.as_tensor(amap, dtype=torch.int32)
    if band:
        assert k2.autograd.band_loss_supported(fsa, dense, m)
    tot = k2.intersect_dense_tot_scores(fsa, dense, beam, a_to_b_map=m, band=band, **limits)
    if band:
        assert type(tot.grad_fn).__name__.startswith("_BandTotScores"), tot.grad_fn
    g = torch.ones_like(tot) if tot_grad is None else torch.as_tensor(
        tot_grad, dtype=tot.dtype, device=tot.device)
    finite = torch.isfinite(tot)
    if bool(finite.any()):
        (tot[finite] * g[finite]).sum().backward()
        ga, gb = fsa.scores.grad.cpu().numpy(), leaf.grad.cpu().numpy()
    else:
        ga = np.zeros(a_host.num_arcs, np.float32)
        gb = np.zeros(tuple(leaf.shape), np.float32)
    return tot.detach().cpu().numpy(), ga, gb


def compare(a, lp, seg, beam, amap=None, tot_grad=None, tag=""):
    scores, brs = host_scores(lp, seg)
    want = oracle.loss_path(a, scores, brs, beam, amap, tot_grad=tot_grad)
    tot, ga, gb = run(a, lp, seg, beam, amap, tot_grad)
    assert close(tot, want["tot_scores"], rtol=1e-6, atol=1e-6), (tag, tot, want["tot_scores"])
    assert np.abs(ga - want["grad_a"]).max(initial=0) <= 1e-4, tag
    want_lp = to_lp_layout(want["grad_b"], tuple(lp.shape), seg)
    assert np.abs(gb - want_lp).max(initial=0) <= 1e-4, tag
    return want, tot, ga, gb


def test_random_band_graphs():
    rng = np.random.default_rng(101)
    for trial in range(40):
        n = int(rng.integers(1, 6))
        C = int(rng.choice([4, 8, 12]))
        a = random_band_graphs(rng, n, int(rng.choice([4, 9, 40])), C)
        lp, seg = random_log_probs(rng, n, 12, C, low=trial % 5 == 0)
        beam = float(rng.choice([0.5, 2.0, 10.0, 100.0]))
        tot_grad = rng.normal(size=n) if trial % 3 == 0 else None
        compare(a, lp, seg, beam, None, tot_grad, f"trial {trial}")


def test_shared_sequences_and_score_matrix_layout():
    # two graphs on every sequence (numerator and denominator style): a_to_b_map
    # [0, 0, 1, 1, ...] makes both write the same rows of the gradient
    rng = np.random.default_rng(7)
    for trial in range(6):
        nseq = int(rng.integers(1, 4))
        a = random_band_graphs(rng, 2 * nseq, 12, 8)
        lp, seg = random_log_probs(rng, nseq, 10, 8)
        amap = np.repeat(np.arange(nseq), 2).astype(np.int32)
        compare(a, lp, seg, 20.0, amap, rng.normal(size=2 * nseq), f"map {trial}")
        # gradient taken in the layout of the DenseFsaVec's score matrix
        scores, brs = host_scores(lp, seg)
        want = oracle.loss_path(a, scores, brs, 20.0, amap)
        tot, ga, gb = run(a, lp, seg, 20.0, amap, scores_layout=True)
        assert close(tot, want["tot_scores"], rtol=1e-6, atol=1e-6)
        assert gb.shape == want["grad_b"].shape
        assert np.abs(gb - want["grad_b"]).max(initial=0) <= 1e-4
        assert np.abs(ga - want["grad_a"]).max(initial=0) <= 1e-4


def test_extreme_scores():
    # arc scores of +-100 and log-probs near -300: the mantissa/exponent sums have no
    # range limit, so nothing has to fall back
    rng = np.random.default_rng(29)
    for trial in range(9):
        n = int(rng.integers(1, 4))
        a = random_band_graphs(rng, n, 10, 8)
        lp, seg = random_log_probs(rng, n, 10, 8)
        if trial % 3 == 0:
            a.arcs[:, 3] = (a.scores * 40.0).astype(np.float32).view(np.int32)
        elif trial % 3 == 1:
            lp = lp * 150.0
        else:
            a.arcs[::3, 3] = np.float32(-np.inf).view(np.int32)
        compare(a, lp, seg, 1.0e4 if trial % 3 else 50.0, tag=f"extreme {trial}")


@pytest.mark.parametrize("name,scale", [("ctc_small", 1.0), ("ctc_large", 0.25),
                                        ("ctc_modified", 0.25)])
def test_workloads_against_oracle(name, scale):
    import k2_b200 as k2
    from gpu_util import fsa_to_host
    from k2_b200 import synthetic as syn
    w = syn.WORKLOADS[name](scale=scale)
    graphs = syn.build_graphs(w, DEV)
    a = fsa_to_host(graphs)
    want, tot, _, gb = compare(a, w.log_probs, w.supervision_segments, w.output_beam, tag=name)
    # and through ctc_loss, on the graphs that ctc_graph wrote on the device
    lp = w.log_probs.to(DEV).requires_grad_(True)
    dense = k2.DenseFsaVec(lp, w.supervision_segments)
    loss = k2.ctc_loss(graphs, dense, output_beam=w.output_beam, reduction="sum")
    loss.backward()
    assert dense._scores is None, "the band kernels do not need the score matrix"
    assert close(loss.item(), -want["tot_scores"].sum(), rtol=1e-5, atol=1e-3)
    assert np.abs(lp.grad.cpu().numpy() + gb).max() <= 1e-5


def test_long_transcripts_sixteen_states_per_lane():
    # graphs of 300..500 states: the instantiation with 16 states per lane
    rng = np.random.default_rng(3)
    from k2_b200.fsa_algo import ctc_graph
    from gpu_util import fsa_to_host
    C, T, n = 40, 260, 3
    symbols = [rng.integers(1, C, size=int(L)).tolist() for L in (249, 200, 150)]
    graphs = ctc_graph(symbols, device=DEV)
    x = (rng.normal(size=(n, T, C)) * 1.5).astype(np.float32)
    x = x - np.log(np.exp(x.astype(np.float64)).sum(-1, keepdims=True)).astype(np.float32)
    seg = torch.tensor([[0, 0, 260], [1, 0, 255], [2, 0, 251]], dtype=torch.int32)
    compare(fsa_to_host(graphs), torch.from_numpy(x), seg, 10.0, tag="long")


def test_summed_ctc_loss_as_one_node_equals_the_composition():
    # ctc_loss(reduction="sum") on the band path is one autograd node; the same numbers
    # and gradients as -tot_scores.sum() composed from its parts, for a loss that is scaled
    # before the backward pass and for float32 total scores
    import k2_b200 as k2
    from k2_b200.fsa_algo import ctc_graph
    rng = np.random.default_rng(21)
    C, T, n = 12, 30, 4
    graphs = ctc_graph([rng.integers(1, C, size=int(L)).tolist() for L in (9, 7, 4, 1)],
                       device=DEV)
    x = rng.normal(size=(n, T, C)).astype(np.float32)
    x = x - np.log(np.exp(x.astype(np.float64)).sum(-1, keepdims=True)).astype(np.float32)
    seg = torch.tensor([[0, 0, 30], [1, 0, 28], [2, 0, 20], [3, 0, 11]], dtype=torch.int32)
    for use_double in (True, False):
        grads = []
        for fused in (True, False):
            lp = torch.from_numpy(x).to(DEV).requires_grad_(True)
            dense = k2.DenseFsaVec(lp, seg)
            if fused:
                loss = k2.ctc_loss(graphs, dense, output_beam=8.0, reduction="sum",
                                   use_double_scores=use_double)
                assert type(loss.grad_fn).__name__.startswith("_BandNegSum"), loss.grad_fn
            else:
                tot = k2.intersect_dense_tot_scores(graphs, dense, 8.0,
                                                    use_double_scores=use_double)
                loss = (-1 * tot).to(torch.float32).sum()
            (loss * 3.0).backward()
            grads.append((loss.detach().item(), lp.grad.cpu().numpy()))
        assert grads[0][0] == grads[1][0]
        assert np.array_equal(grads[0][1], grads[1][1])


def _most_states_kept(a, lp, seg, beam):
    """Per sequence, the largest number of distinct graph states on one frame of the
    oracle's pruned lattice."""
    scores, brs = host_scores(lp, seg)
    lat = oracle.intersect_dense(a, scores, brs, beam)
    row = lat.arc_map_b // scores.shape[1]
    src = a.arcs[lat.arc_map_a, 0]
    out = []
    for i in range(len(brs) - 1):
        m = (row >= brs[i]) & (row < brs[i + 1])
        key = np.unique((row[m] - brs[i]).astype(np.int64) * 100000 + src[m])
        out.append(int(np.bincount((key // 100000).astype(np.int64)).max()))
    return out


def test_levels_with_about_a_hundred_surviving_states():
    # flat log-probs and wide beams: levels with 96..127 surviving states take four
    # registers per lane of the list recursion, levels with more send the graph to the
    # (mantissa, exponent) recursion; both next to graphs that need neither
    rng = np.random.default_rng(11)
    from k2_b200.fsa_algo import ctc_graph
    from gpu_util import fsa_to_host
    C, T, n = 40, 200, 3
    symbols = [rng.integers(1, C, size=int(L)).tolist() for L in (95, 90, 60)]
    a = fsa_to_host(ctc_graph(symbols, device=DEV))
    x = (rng.normal(size=(n, T, C)) * 0.5).astype(np.float32)
    x = x - np.log(np.exp(x.astype(np.float64)).sum(-1, keepdims=True)).astype(np.float32)
    lp = torch.from_numpy(x)
    seg = torch.tensor([[0, 0, 200], [1, 0, 196], [2, 0, 190]], dtype=torch.int32)
    widest = {beam: _most_states_kept(a, lp, seg, beam) for beam in (14.0, 20.0, 40.0)}
    assert 96 <= widest[14.0][0] <= 127 and widest[14.0][2] <= 95, widest
    assert all(96 <= w <= 127 for w in widest[20.0]), widest
    assert widest[40.0][0] > 127 and 96 <= widest[40.0][2] <= 127, widest
    for beam in widest:
        compare(a, lp, seg, beam, tot_grad=rng.normal(size=n), tag=f"beam {beam}")


def test_same_numbers_as_the_general_kernels_and_the_lattice():
    import k2_b200 as k2
    from gpu_util import host_to_fsa
    rng = np.random.default_rng(17)
    for trial in range(5):
        n = int(rng.integers(2, 6))
        a = random_band_graphs(rng, n, 30, 16, zero_scores=trial % 2 == 0)
        lp, seg = random_log_probs(rng, n, 25, 16)
        tot1, ga1, gb1 = run(a, lp, seg, 6.0, band=True)
        tot0, ga0, gb0 = run(a, lp, seg, 6.0, band=False)
        # the band kernels take exp(dense score) to float precision
        assert close(tot1, tot0, rtol=1e-7, atol=1e-6)
        assert np.abs(ga1 - ga0).max(initial=0) <= 1e-5
        assert np.abs(gb1 - gb0).max(initial=0) <= 1e-5
        dense = k2.DenseFsaVec(lp.to(DEV), seg)
        lat = k2.intersect_dense(host_to_fsa(a), dense, 6.0)
        tot2 = lat.get_tot_scores(log_semiring=True, use_double_scores=True).cpu().numpy()
        assert close(tot1, tot2, rtol=1e-6, atol=1e-6)


def test_beam_reduction_under_a_state_limit():
    import k2_b200 as k2
    from gpu_util import host_to_fsa, intersect_raw
    rng = np.random.default_rng(5)
    a = random_band_graphs(rng, 4, 30, 8, zero_scores=True)
    lp, seg = random_log_probs(rng, 4, 20, 8)
    scores, brs = host_scores(lp, seg)
    full = oracle.intersect_dense(a, scores, brs, 50.0)
    assert full.num_states > 40
    limit = int(full.num_states * 0.7)
    shrunk = oracle.intersect_dense(a, scores, brs, 50.0, max_states=limit)
    assert 0 < shrunk.num_states <= limit
    dense = k2.DenseFsaVec(lp.to(DEV), seg)
    lat, _, _ = intersect_raw(host_to_fsa(a), dense, 50.0, max_states=limit)
    assert lat.arcs.num_states == shrunk.num_states
    ref_tot = lat.get_tot_scores(True, True).cpu().numpy()
    tot, _, _ = run(a, lp, seg, 50.0, max_states=limit)
    assert close(tot, ref_tot, rtol=1e-6, atol=1e-6)
    # limits around the number of survivors, around the part of the grid that the start
    # state reaches and that reaches the last state (below that the host reads the counts,
    # from there on it does not) and up to the whole grid
    S = np.diff(a.row_splits1).astype(np.int64)
    T = seg[:, 2].numpy().astype(np.int64)
    grid = int(((T + 2) * S).sum())
    for limit in sorted({full.num_states - 1, full.num_states, full.num_states + 1,
                         (full.num_states + grid) // 2, grid - 1, grid}):
        lat, _, _ = intersect_raw(host_to_fsa(a), dense, 50.0, max_states=limit)
        want = oracle.intersect_dense(a, scores, brs, 50.0, max_states=limit)
        assert lat.arcs.num_states == want.num_states, limit
        ref_tot = lat.get_tot_scores(True, True).cpu().numpy()
        tot, _, _ = run(a, lp, seg, 50.0, max_states=limit)
        assert close(tot, ref_tot, rtol=1e-6, atol=1e-6), limit


def test_state_limit_at_the_number_of_reachable_grid_states():
    # complete band graphs, zero scores, a beam that keeps everything: the survivors are
    # all but a few of the grid states that the start state reaches and that reach the
    # last state, which is the bound from which on the host does not read the counts.
    # Limits on both sides of the survivors and of that bound.
    import k2_b200 as k2
    from gpu_util import host_to_fsa, intersect_raw
    rng = np.random.default_rng(8)
    C = 8
    rs1, rs2, rows = [0], [0], []
    for ns in (9, 14, 6, 2):
        lab = rng.integers(0, C, size=ns)
        lab[ns - 1] = -1
        for s in range(ns - 1):
            for d in (0, 1, 2):
                if s + d <= ns - 1:
                    rows.append((s, s + d, int(lab[s + d]), 0.0))
            rs2.append(len(rows))
        rs2.append(len(rows))
        rs1.append(rs1[-1] + ns)
    r = np.array(rows, dtype=np.float64).reshape(-1, 4)
    a = HostFsaVec(np.asarray(rs1, np.int32), np.asarray(rs2, np.int32),
                   make_arcs(r[:, 0].astype(np.int32), r[:, 1].astype(np.int32),
                             r[:, 2].astype(np.int32), r[:, 3].astype(np.float32)))
    x = rng.normal(size=(4, 12, C)).astype(np.float32)
    lp = torch.from_numpy(
        x - np.log(np.exp(x.astype(np.float64)).sum(-1, keepdims=True)).astype(np.float32))
    # (every graph can reach its last state within its frames)
    seg = torch.tensor([[0, 0, 12], [1, 0, 9], [2, 0, 9], [3, 0, 3]], dtype=torch.int32)
    scores, brs = host_scores(lp, seg)
    reachable = 0
    for S, T in zip((9, 14, 6, 2), seg[:, 2].tolist()):
        m, R = S - 1, T + 1
        reachable += sum(min(m, 2 * l) - max(0, m - 2 * (R - l)) + 1 for l in range(R + 1))
    beam = 1.0e4
    kept = oracle.intersect_dense(a, scores, brs, beam).num_states
    assert kept <= reachable
    dense = k2.DenseFsaVec(lp.to(DEV), seg)
    for limit in sorted({kept - 1, kept, (kept + reachable) // 2, reachable - 1, reachable,
                         reachable + 1}):
        want = oracle.intersect_dense(a, scores, brs, beam, max_states=limit)
        lat, _, _ = intersect_raw(host_to_fsa(a), dense, beam, max_states=limit)
        assert lat.arcs.num_states == want.num_states, limit
        ref_tot = lat.get_tot_scores(True, True).cpu().numpy()
        tot, _, _ = run(a, lp, seg, beam, max_states=limit)
        assert close(tot, ref_tot, rtol=1e-6, atol=1e-6), limit
    assert oracle.intersect_dense(a, scores, brs, beam, max_states=kept - 1).num_states < kept


def test_graphs_that_are_not_band_graphs_take_the_general_kernels():
    import k2_b200 as k2
    from gpu_util import host_to_fsa
    rng = np.random.default_rng(9)
    # (src, dest, label): an arc that skips three states; two labels into one state
    cases = [[(0, 1, 1), (0, 3, 2), (1, 2, 3), (2, 3, 2), (3, 4, -1)],
             [(0, 0, 0), (0, 1, 1), (1, 1, 2), (1, 2, -1)]]
    for rows in cases:
        ns = max(r[1] for r in rows) + 1
        src = np.array([r[0] for r in rows], np.int32)
        arcs = make_arcs(src, np.array([r[1] for r in rows], np.int32),
                         np.array([r[2] for r in rows], np.int32),
                         rng.normal(size=len(rows)).astype(np.float32))
        rs2 = np.searchsorted(src, np.arange(ns + 1)).astype(np.int32)
        g = HostFsaVec(np.array([0, ns], np.int32), rs2, arcs)
        lp, seg = random_log_probs(rng, 1, 8, 4)
        fsa = host_to_fsa(g)
        dense = k2.DenseFsaVec(lp.to(DEV), seg)
        assert not k2.autograd.band_loss_supported(fsa, dense)
        tot = k2.intersect_dense_tot_scores(fsa, dense, 10.0)
        scores, brs = host_scores(lp, seg)
        want = oracle.loss_path(g, scores, brs, 10.0)
        assert close(tot.cpu().numpy(), want["tot_scores"], rtol=1e-6, atol=1e-6)


def test_a_wait_that_gives_up_is_reported_and_the_general_kernels_take_over():
    # With a poll limit of 0 every bounded wait for a row copy gives up at once: the
    # kernel flags it and returns (nothing hangs or traps), the status word says so,
    # the totals are NaN; with BAND_VERIFY the call is then served by the general
    # kernels and the numbers are the oracle's.
    import ctypes
    import k2_b200 as k2
    from k2_b200 import _lib
    from k2_b200 import autograd as ag
    from gpu_util import host_to_fsa
    rng = np.random.default_rng(41)
    a = random_band_graphs(rng, 3, 20, 8, zero_scores=True)
    lp, seg = random_log_probs(rng, 3, 15, 8)
    scores, brs = host_scores(lp, seg)
    want = oracle.loss_path(a, scores, brs, 10.0)
    fsa = host_to_fsa(a)
    try:
        _lib.lib.k2b200_debug_set_copy_wait_limit(0)
        dense = k2.DenseFsaVec(lp.to(DEV), seg)
        band = ag._band_loss_args(fsa, dense, None, 10.0, 15000000, 1 << 30)
        assert band is not None
        args = band[0]
        nbytes = ctypes.c_size_t()
        _lib.check(_lib.lib.k2b200_band_loss_workspace_bytes(ctypes.byref(args),
                                                              ctypes.byref(nbytes)))
        ws = torch.empty(nbytes.value, dtype=torch.uint8, device=DEV)
        tot = torch.empty(3, dtype=torch.float64, device=DEV)
        beam = ctypes.c_float()
        stream = _lib.stream_of(torch.device(DEV))
        _lib.check(_lib.lib.k2b200_band_loss_forward(ctypes.byref(args), _lib.ptr(ws),
                                                      nbytes.value, stream, _lib.ptr(tot),
                                                      ctypes.byref(beam)))
        status = ctypes.c_int32()
        _lib.check(_lib.lib.k2b200_band_loss_status(ctypes.byref(args), _lib.ptr(ws),
                                                     nbytes.value, stream, ctypes.byref(status)))
        assert status.value & 2
        assert bool(torch.isnan(tot).all())
        ag.BAND_VERIFY = True
        lpd = lp.to(DEV).requires_grad_(True)
        dense = k2.DenseFsaVec(lpd, seg)
        tot2 = k2.intersect_dense_tot_scores(fsa, dense, 10.0)
        tot2.sum().backward()
        assert close(tot2.detach().cpu().numpy(), want["tot_scores"], rtol=1e-6, atol=1e-6)
        want_lp = to_lp_layout(want["grad_b"], tuple(lp.shape), seg)
        assert np.abs(lpd.grad.cpu().numpy() - want_lp).max() <= 1e-4
    finally:
        ag.BAND_VERIFY = False
        _lib.lib.k2b200_debug_set_copy_wait_limit(-1)
    # and with the limit restored the band kernels serve the same call
    tot3, _, _ = run(a, lp, seg, 10.0)
    assert close(tot3, want["tot_scores"], rtol=1e-6, atol=1e-6)

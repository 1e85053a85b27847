"""GPU parity: the CUDA path (through the C-ABI) against the CPU oracle on the
same seeded inputs.  Lattices, arc maps, best paths and property bits must be
bit-exact; float64 scores agree to 1e-9, float32 scores to 1e-4 relative, and
gradients w.r.t. the dense scores to 1e-4 absolute (the tolerances of this path)."""
import numpy as np
import pytest
import torch

from oracle import oracle
from util import close, random_dense, random_fsa_vec, same_fsa

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def k2():
    import k2_b200
    return k2_b200


def _micro():
    from oracle.common import HostFsaVec, make_arcs
    arcs1 = make_arcs([0, 0, 1, 1, 2], [1, 1, 1, 2, 3], [1, 2, 1, 2, -1],
                      [1.0, 0.5, 50.0, 2.0, 3.0])
    rs2_one = np.array([0, 2, 4, 5, 5])
    a = HostFsaVec(np.array([0, 4, 8], np.int32),
                   np.concatenate([rs2_one, rs2_one[1:] + 5]).astype(np.int32),
                   np.concatenate([arcs1, arcs1]))
    ninf = -np.inf
    scores = np.array([[ninf, .1, .2, .3], [ninf, .04, .05, .06], [ninf, 0, 0, 0],
                       [0, ninf, ninf, ninf], [ninf, .1, .2, .3], [ninf, .4, .5, .6],
                       [0, ninf, ninf, ninf]], np.float32)
    return a, scores, np.array([0, 4, 7], np.int32)


@pytest.mark.parametrize("mode", [1, 2, 3])
def test_micro_example_known_answer(k2, mode):
    # worked example computed with the reference: two copies of a 4-state graph
    from gpu_util import dense_from_scores, fsa_to_host, host_to_fsa, intersect_raw
    a, scores, brs = _micro()
    lat, ma, mb = intersect_raw(host_to_fsa(a), dense_from_scores(scores, brs), 100.0, mode=mode)
    h = fsa_to_host(lat, ma, mb)
    assert h.row_splits1.tolist() == [0, 5, 9]
    assert h.row_splits2.tolist() == [0, 2, 3, 4, 5, 5, 7, 8, 9, 9]
    assert h.arc_map_a.tolist() == [0, 1, 2, 3, 4, 5, 6, 8, 9]
    assert h.arc_map_b.tolist() == [2, 3, 6, 11, 12, 18, 19, 23, 24]
    assert h.arcs[:, :3].tolist() == [[0, 1, 1], [0, 1, 2], [1, 2, 1], [2, 3, 2], [3, 4, -1],
                                      [0, 1, 1], [0, 1, 2], [1, 2, 2], [2, 3, -1]]
    np.testing.assert_array_equal(
        h.scores, np.array([1.2, 0.8, 50.05, 2.0, 3.0, 1.2, 0.8, 2.6, 3.0], np.float32))
    # strict '>' at the beam: the 0.4-worse arc of the first FSA is dropped
    lat2, _, _ = intersect_raw(host_to_fsa(a), dense_from_scores(scores, brs), 0.4, mode=mode)
    assert fsa_to_host(lat2).arcs[:, :3].tolist() == [[0, 1, 1], [1, 2, 1], [2, 3, 2], [3, 4, -1],
                                                      [0, 1, 1], [0, 1, 2], [1, 2, 2], [2, 3, -1]]


@pytest.mark.parametrize("mode", [1, 2])
def test_random_fsa_vecs_bit_exact(k2, mode):
    # in the spirit of Intersect.RandomFsaVec (k2/csrc/intersect_test.cu:262-380)
    from gpu_util import dense_from_scores, fsa_to_host, host_to_fsa, intersect_raw
    rng = np.random.default_rng(1)
    for trial in range(60):
        n = int(rng.integers(1, 7))
        a = random_fsa_vec(rng, n, acyclic=bool(trial % 2))
        scores, brs = random_dense(rng, n, 10, 5)
        beam = float(rng.choice([0.5, 2.0, 10.0, 100.0]))
        amap = None
        if trial % 5 == 0:
            amap = np.sort(rng.integers(0, n, size=n)).astype(np.int32)
        want = oracle.intersect_dense(a, scores, brs, beam, amap)
        lat, ma, mb = intersect_raw(host_to_fsa(a), dense_from_scores(scores, brs), beam, amap,
                                    mode=mode)
        same_fsa(fsa_to_host(lat, ma, mb), want, f"trial {trial}")
        assert lat.properties == oracle.properties(want)[1]


def _check_scores(k2, lat, want):
    from gpu_util import fsa_to_host
    for log_semiring in (True, False):
        for use_double in (True, False):
            tol = dict(rtol=1e-9, atol=1e-9) if use_double else dict(rtol=1e-4, atol=1e-4)
            of = oracle.forward_scores(want, log_semiring, use_double)
            ob = oracle.backward_scores(want, log_semiring, use_double)
            ot, op = oracle.tot_scores_and_arc_post(want, of, ob, use_double)
            f = lat.get_forward_scores(use_double, log_semiring).detach().cpu().numpy()
            b = lat.get_backward_scores(use_double, log_semiring).detach().cpu().numpy()
            t = lat.get_tot_scores(use_double, log_semiring).detach().cpu().numpy()
            p = lat.get_arc_post(use_double, log_semiring).detach().cpu().numpy()
            assert close(f, of, **tol) and close(b, ob, **tol), (log_semiring, use_double)
            assert close(t, ot, **tol), (log_semiring, use_double)
            finite = np.isfinite(op)
            # float32 posteriors are differences of scores of magnitude max|fwd|:
            # allow a few ulps of that magnitude (the reference's float path
            # carries the same cancellation error)
            mag = float(np.abs(of[np.isfinite(of)]).max()) if np.isfinite(of).any() else 1.0
            ptol = tol if use_double else dict(rtol=1e-4, atol=max(1e-4, 8 * 1.2e-7 * mag))
            assert close(p[finite], op[finite], **ptol)
    _, oea = oracle.forward_scores(want, False, True, want_entering_arcs=True)
    ea = lat._get_entering_arcs(True).cpu().numpy()
    np.testing.assert_array_equal(ea, oea)
    osplits, obest = oracle.shortest_path(want, oea)
    best = k2.shortest_path(lat, True)
    np.testing.assert_array_equal(best._best_arc_map.cpu().numpy(), obest)
    np.testing.assert_array_equal(np.diff(best.arcs.h_row_splits1),
                                  np.where(np.diff(osplits) > 0, np.diff(osplits) + 1, 0))


def test_scores_on_random_lattices(k2):
    from gpu_util import dense_from_scores, host_to_fsa, intersect_raw
    rng = np.random.default_rng(2)
    for trial in range(25):
        n = int(rng.integers(1, 6))
        a = random_fsa_vec(rng, n, acyclic=bool(trial % 2))
        scores, brs = random_dense(rng, n, 12, 5, low_rows=False)
        want = oracle.intersect_dense(a, scores, brs, 20.0)
        lat, _, _ = intersect_raw(host_to_fsa(a), dense_from_scores(scores, brs), 20.0)
        _check_scores(k2, lat, want)


def _workload_case(k2, w, mode=0, check_scores=False):
    """intersect -> log tot_scores -> backward through the public API, against
    the oracle's loss path."""
    from gpu_util import DEV, fsa_to_host
    from k2_b200 import synthetic as syn
    from k2_b200 import autograd
    graphs = syn.build_graphs(w, DEV)
    log_probs = w.log_probs.to(DEV).requires_grad_(True)
    dense = k2.DenseFsaVec(log_probs, w.supervision_segments)
    autograd.VITERBI_MODE = mode
    try:
        lat = k2.intersect_dense(graphs, dense, w.output_beam)
    finally:
        autograd.VITERBI_MODE = 0
    tot = lat.get_tot_scores(log_semiring=True, use_double_scores=True)
    (-tot.sum()).backward()
    a_host = fsa_to_host(graphs)
    scores_host = dense.scores.detach().cpu().numpy()
    want = oracle.loss_path(a_host, scores_host, dense.h_row_splits, w.output_beam)
    same_fsa(fsa_to_host(lat), want["lattice"], w.name)
    assert close(tot.detach().cpu().numpy(), want["tot_scores"], rtol=1e-4, atol=0)
    # gradient w.r.t. log_probs = -(grad_b without column 0, un-gathered)
    C = log_probs.shape[-1]
    seg = w.supervision_segments.numpy()
    expect = np.zeros(tuple(log_probs.shape), np.float32)
    gb = want["grad_b"]
    r = 0
    for (n, s, d) in seg.tolist():
        expect[n, s:s + d] -= gb[r:r + d, 1:]
        r += d + 1
    got = log_probs.grad.cpu().numpy()
    assert np.abs(got - expect).max() <= 1e-4, np.abs(got - expect).max()
    if check_scores:
        _check_scores(k2, lat, want["lattice"])
    return lat, want


def test_ctc_small_full_size(k2):
    from k2_b200 import synthetic as syn
    lat, want = _workload_case(k2, syn.ctc_small(), check_scores=True)
    assert want["lattice"].num_arcs > 50000  # beam 10 keeps ~72k arcs on this workload


@pytest.mark.parametrize("mode", [1, 2, 3])
def test_ctc_large_quarter(k2, mode):
    from k2_b200 import synthetic as syn
    _workload_case(k2, syn.ctc_large(scale=0.25), mode=mode)


def test_ctc_modified_scaled(k2):
    from k2_b200 import synthetic as syn
    _workload_case(k2, syn.ctc_modified(scale=0.2))


@pytest.mark.parametrize("mode", [1, 2])
def test_lfmmi_den_scaled(k2, mode):
    from k2_b200 import synthetic as syn
    _workload_case(k2, syn.lfmmi_den(scale=0.05), mode=mode)


def test_hlg_decode_scaled_viterbi_and_log(k2):
    # 70k states: beyond what the reference's uint16 state ids can represent
    from k2_b200 import synthetic as syn
    w = syn.hlg_decode(scale=0.04, num_states=70001)
    lat, want = _workload_case(k2, w, check_scores=False)
    _, oea = oracle.forward_scores(want["lattice"], False, True, want_entering_arcs=True)
    _, obest = oracle.shortest_path(want["lattice"], oea)
    best = k2.shortest_path(lat, True)
    np.testing.assert_array_equal(best._best_arc_map.cpu().numpy(), obest)


def test_ctc_loss_matches_torch(k2):
    # second, independent check as in k2/python/tests/ctc_loss_test.py:311-441
    from gpu_util import DEV
    gen = torch.Generator().manual_seed(7)
    N, T, C = 4, 30, 10
    logits = torch.randn(N, T, C, generator=gen)
    lens = torch.tensor([30, 27, 25, 20], dtype=torch.int32)
    targets = [torch.randint(1, C, (int(k),), generator=gen).tolist() for k in (5, 7, 3, 6)]
    ours_in = logits.clone().to(DEV).requires_grad_(True)
    lp = torch.log_softmax(ours_in, -1)
    seg = torch.stack([torch.arange(N, dtype=torch.int32), torch.zeros(N, dtype=torch.int32),
                       lens], 1)
    dense = k2.DenseFsaVec(lp, seg)
    graph = k2.ctc_graph(targets, device=DEV)
    loss = k2.ctc_loss(graph, dense, output_beam=1000.0, reduction="sum")
    loss.backward()
    t_in = logits.clone().requires_grad_(True)
    t_lp = torch.log_softmax(t_in, -1).permute(1, 0, 2)
    t_loss = torch.nn.functional.ctc_loss(
        t_lp, torch.tensor([x for t in targets for x in t]), lens.long(),
        torch.tensor([len(t) for t in targets]), reduction="sum")
    t_loss.backward()
    assert abs(loss.item() - t_loss.item()) < 1e-3
    assert (ours_in.grad.cpu() - t_in.grad).abs().max() < 1e-4


def test_edge_cases(k2):
    from gpu_util import DEV, dense_from_scores, fsa_to_host, host_to_fsa, intersect_raw
    from oracle.common import HostFsaVec, make_arcs
    a, scores, brs = _micro()
    # both graphs against sequence 0 (a_to_b_map = [0, 0],
    # k2/python/tests/intersect_dense_test.py:111-114)
    want = oracle.intersect_dense(a, scores, brs, 100.0, np.array([0, 0], np.int32))
    lat, ma, mb = intersect_raw(host_to_fsa(a), dense_from_scores(scores, brs), 100.0, [0, 0])
    same_fsa(fsa_to_host(lat, ma, mb), want)
    # no path of the right length: FSA 1 needs >= 3 arcs but its sequence has 2 rows
    brs2 = np.array([0, 4, 6], np.int32)
    sc2 = scores[:6].copy()
    sc2[5] = scores[6]
    want = oracle.intersect_dense(a, sc2, brs2, 100.0)
    lat, ma, mb = intersect_raw(host_to_fsa(a), dense_from_scores(sc2, brs2), 100.0)
    same_fsa(fsa_to_host(lat, ma, mb), want)
    assert want.row_splits1[2] == want.row_splits1[1]  # empty second FSA
    tot = lat.get_tot_scores(True, True).detach().cpu().numpy()
    assert np.isneginf(tot[1]) and np.isfinite(tot[0])
    # a label beyond the classes scores -inf: nothing survives, no error
    bad = HostFsaVec(a.row_splits1.copy(), a.row_splits2.copy(), a.arcs.copy())
    bad.arcs[:, 2] = np.where(bad.arcs[:, 2] > 0, 7, bad.arcs[:, 2])
    lat, _, _ = intersect_raw(host_to_fsa(bad), dense_from_scores(scores, brs), 100.0)
    assert lat.num_arcs == 0 and lat.arcs.num_states == 0
    # unsorted sequence lengths are rejected like the reference's K2_CHECK
    with pytest.raises(RuntimeError, match="sorted"):
        intersect_raw(host_to_fsa(a), dense_from_scores(scores[[4, 5, 6, 0, 1, 2, 3]],
                                                        np.array([0, 3, 7], np.int32)), 10.0)
    with pytest.raises(RuntimeError, match="monotonic"):
        intersect_raw(host_to_fsa(a), dense_from_scores(scores, brs), 10.0, [1, 0])
    with pytest.raises(RuntimeError, match="output_beam"):
        intersect_raw(host_to_fsa(a), dense_from_scores(scores, brs), 0.0)
    # an FSA with no states in a_fsas
    e = HostFsaVec(np.array([0, 4, 4, 8], np.int32), a.row_splits2, a.arcs)
    sc3 = np.concatenate([scores[:4], scores[:4], scores[4:]])
    brs3 = np.array([0, 4, 8, 11], np.int32)
    want = oracle.intersect_dense(e, sc3, brs3, 100.0)
    lat, ma, mb = intersect_raw(host_to_fsa(e), dense_from_scores(sc3, brs3), 100.0)
    same_fsa(fsa_to_host(lat, ma, mb), want)


def test_beam_shrinks_when_limits_hit(k2):
    # intersect_dense.cu:240-320: retry with a smaller beam until within limits
    from gpu_util import DEV, fsa_to_host, intersect_raw
    from k2_b200 import synthetic as syn
    w = syn.ctc_small(scale=0.5)
    graphs = syn.build_graphs(w, DEV)
    dense = k2.DenseFsaVec(w.log_probs.to(DEV), w.supervision_segments)
    a_host = fsa_to_host(graphs)
    sc = dense.scores.cpu().numpy()
    for kw in (dict(max_states=2000), dict(max_arcs=3000)):
        want = oracle.intersect_dense(a_host, sc, dense.h_row_splits, 10.0, **kw)
        lat, ma, mb = intersect_raw(graphs, dense, 10.0, **kw)
        same_fsa(fsa_to_host(lat, ma, mb), want)
        assert want.extra["final_beam"] < 10.0
        assert abs(lat.arcs.output_beam_used - want.extra["final_beam"]) < 1e-6


def test_generic_ragged_ops(k2):
    import ctypes
    from gpu_util import DEV
    from k2_b200 import _lib
    rng = np.random.default_rng(3)
    for n in (0, 1, 5, 2047, 2048, 2049, 100000, 1 << 20):
        x = rng.integers(0, 7, size=n).astype(np.int32)
        t = torch.from_numpy(x).to(DEV)
        out = torch.empty(n + 1, dtype=torch.int32, device=DEV)
        tmp = torch.empty(_lib.lib.k2b200_exclusive_sum_tmp_bytes(n) + 16, dtype=torch.uint8,
                          device=DEV)
        _lib.check(_lib.lib.k2b200_exclusive_sum(_lib.ptr(t), _lib.ptr(out), n, _lib.ptr(tmp),
                                                 _lib.stream_of(torch.device(DEV))))
        want = np.concatenate([[0], np.cumsum(x)]).astype(np.int32)
        np.testing.assert_array_equal(out.cpu().numpy(), want)
    # host integers -> device through kernel parameters, across the 960-value launches
    for n in (0, 1, 959, 960, 961, 5000):
        x = rng.integers(-2**31, 2**31, size=n).astype(np.int32)
        np.testing.assert_array_equal(_lib.upload_i32(x, DEV).cpu().numpy(), x)
    # incoming index against a stable host sort
    a = random_fsa_vec(rng, 9, max_states=30, max_arcs=300)
    from gpu_util import host_to_fsa
    f = host_to_fsa(a)
    in_splits, in_arcs, in_src, in_score = f.arcs.incoming()
    state_of = np.repeat(np.arange(a.num_states), np.diff(a.row_splits2))
    fsa_of = np.repeat(np.arange(a.num_fsas), np.diff(a.row_splits1))[state_of]
    dest01 = a.row_splits1[fsa_of] + a.arcs[:, 1]
    order = np.argsort(dest01, kind="stable")
    np.testing.assert_array_equal(in_arcs.cpu().numpy(), order)
    cnt = np.bincount(dest01, minlength=a.num_states)
    np.testing.assert_array_equal(in_splits.cpu().numpy(), np.concatenate([[0], np.cumsum(cnt)]))
    np.testing.assert_array_equal(f.arcs.row_ids(2).cpu().numpy(), state_of)
    np.testing.assert_array_equal(in_src.cpu().numpy(), state_of[order])
    np.testing.assert_array_equal(in_score.cpu().numpy(), a.scores[order])


def test_ctc_graph_on_gpu_matches_oracle(k2):
    from gpu_util import DEV
    rng = np.random.default_rng(4)
    for modified in (False, True):
        for trial in range(25):
            n = int(rng.integers(1, 7))
            syms = [[int(x) for x in rng.integers(1, 5, size=int(rng.integers(0, 9)))]
                    for _ in range(n)]
            if trial == 0:
                syms = [[] for _ in range(n)]  # only empty transcripts
            g = k2.ctc_graph(syms, modified=modified, device=DEV)
            o = oracle.ctc_graphs(syms, modified)
            np.testing.assert_array_equal(g.arcs.values().cpu().numpy(), o.arcs)
            np.testing.assert_array_equal(g.arcs.row_splits(1).cpu().numpy(), o.row_splits1)
            np.testing.assert_array_equal(g.arcs.row_splits(2).cpu().numpy(), o.row_splits2)
            np.testing.assert_array_equal(g.aux_labels.cpu().numpy(), o.aux_labels)
            np.testing.assert_array_equal(g.arcs.h_row_splits1, o.row_splits1)
            np.testing.assert_array_equal(g.arcs.h_arc_splits, o.row_splits2[o.row_splits1])
            assert g.properties == oracle.properties(o)[1]


def test_replicated_graph_is_read_through_its_first_copy(k2):
    # one graph copied once per sequence (how decoding graphs are stacked): with the
    # sharing threshold lowered the kernels read copy 0 only; lattice, arc maps and
    # gradients must not change
    from gpu_util import dense_from_scores, fsa_to_host, host_to_fsa
    from k2_b200 import autograd
    from oracle.common import HostFsaVec
    rng = np.random.default_rng(31)
    one = random_fsa_vec(rng, 1, max_states=40, max_arcs=200, acyclic=False, allow_empty=False)
    n, S, A = 5, one.num_states, one.num_arcs
    rs1 = (np.arange(n + 1) * S).astype(np.int32)
    rs2 = np.concatenate([one.row_splits2[:-1] + i * A for i in range(n)] + [[n * A]]).astype(np.int32)
    a = HostFsaVec(rs1, rs2, np.tile(one.arcs, (n, 1)))
    scores, brs = random_dense(rng, n, 12, 5, low_rows=False)
    out = {}
    for shared in (False, True):
        autograd.SHARED_GRAPH_MIN_BYTES = 0 if shared else 1 << 40
        try:
            fsa = host_to_fsa(a)
            assert fsa.arcs.replicated(autograd.SHARED_GRAPH_MIN_BYTES) == shared
            fsa.scores.requires_grad_(True)
            dense = dense_from_scores(scores, brs, requires_grad=True)
            lat, ma, mb = autograd._intersect_dense_arcs(fsa.arcs, dense, None, 8.0, 15000000, 1 << 30)
            tot = k2.intersect_dense_tot_scores(fsa, dense, 8.0)
            tot[torch.isfinite(tot)].sum().backward()
            out[shared] = (fsa_to_host(k2.Fsa(lat, _check=False), ma, mb),
                           tot.detach().cpu().numpy(), fsa.scores.grad.cpu().numpy(),
                           dense.scores.grad.cpu().numpy())
        finally:
            autograd.SHARED_GRAPH_MIN_BYTES = 32 << 20
    same_fsa(out[True][0], out[False][0], "shared")
    np.testing.assert_array_equal(out[True][1], out[False][1])
    np.testing.assert_allclose(out[True][2], out[False][2], atol=1e-6)
    np.testing.assert_array_equal(out[True][3], out[False][3])
    want = oracle.intersect_dense(a, scores, brs, 8.0)
    same_fsa(out[True][0], want, "shared vs oracle")


def test_layering_of_arbitrary_fsa_vecs(k2):
    # k2b200_fsa_levels against the numpy longest-distance layering
    from gpu_util import host_to_fsa
    from util import host_levels
    rng = np.random.default_rng(41)
    for trial in range(30):
        a = random_fsa_vec(rng, int(rng.integers(1, 7)), max_states=30, max_arcs=80, acyclic=True)
        arcs = host_to_fsa(a).arcs
        arcs._levels = None
        off, spl = arcs.levels()
        want_off, want_spl = host_levels(arcs)
        np.testing.assert_array_equal(off.cpu().numpy(), want_off, f"trial {trial}")
        np.testing.assert_array_equal(spl.cpu().numpy(), want_spl, f"trial {trial}")
    # a linear chain (one state per layer) and a graph with a cycle
    lin = k2.linear_fsa([3, 1, 4, 1, 5], device="cuda:0").arcs
    lin._levels = None
    off, spl = lin.levels()
    assert off.tolist() == [0, 7] and spl.tolist() == list(range(8))
    cyc = random_fsa_vec(rng, 2, max_states=8, max_arcs=30, acyclic=False, allow_empty=False)
    cyc_arcs = host_to_fsa(cyc).arcs
    cyc_arcs._levels = None
    if np.any(cyc.arcs[:, 1] <= cyc.arcs[:, 0]):
        with pytest.raises(RuntimeError):
            cyc_arcs.levels()


def test_dense_fsa_vec_from_logits_matches_log_softmax(k2):
    torch.manual_seed(3)
    dev = "cuda:0"
    logits = (torch.randn(5, 37, 91, device=dev) * 3.0)
    segs = torch.tensor([[0, 0, 37], [3, 2, 30], [1, 5, 25], [4, 0, 12], [2, 10, 7]], dtype=torch.int32)
    a = logits.clone().requires_grad_(True)
    b = logits.clone().requires_grad_(True)
    d1 = k2.DenseFsaVec(torch.log_softmax(a, dim=-1), segs)
    d2 = k2.DenseFsaVec.from_logits(b, segs)
    assert torch.equal(torch.isinf(d1.scores), torch.isinf(d2.scores))
    fin = torch.isfinite(d1.scores)
    assert (d1.scores[fin] - d2.scores[fin]).abs().max().item() <= 2e-6
    g = torch.randn_like(d1.scores)
    g[~fin] = 0.0
    (d1.scores.masked_fill(~fin, 0.0) * g).sum().backward()
    (d2.scores.masked_fill(~fin, 0.0) * g).sum().backward()
    assert (a.grad - b.grad).abs().max().item() <= 2e-5
    # frames outside every segment get no gradient
    assert float(b.grad[2, :10].abs().max()) == 0.0


def test_ragged_attributes_follow_the_arc_maps(k2):
    """A ragged attribute (a list per arc, like ragged aux_labels) is carried through
    intersect_dense, intersect_dense_pruned, arc_sort and shortest_path by rows."""
    from gpu_util import DEV, dense_from_scores, host_to_fsa, intersect_raw
    rng = np.random.default_rng(12)
    a = random_fsa_vec(rng, 3, max_states=8, max_arcs=24, max_label=3, allow_empty=False)
    scores, brs = random_dense(rng, 3, 9, 4)
    rows = [[int(x) for x in rng.integers(1, 50, size=int(rng.integers(0, 4)))]
            for _ in range(a.num_arcs)]
    fsa = host_to_fsa(a)
    fsa.tokens = k2.RaggedTensor(rows, device=DEV)
    dense = dense_from_scores(scores, brs)
    _, map_a, _ = intersect_raw(fsa, dense, 100.0)
    lat = k2.intersect_dense(fsa, dense, output_beam=100.0)
    assert lat.tokens.tolist() == [rows[i] for i in map_a.cpu().tolist()]
    best = k2.shortest_path(lat, use_double_scores=True)
    picked = lat.tokens.tolist()
    assert best.tokens.tolist() == [picked[i] for i in best._best_arc_map.cpu().tolist()]
    pruned = k2.intersect_dense_pruned(fsa, dense, 50.0, 50.0, 0, 1000)
    assert sorted(map(tuple, pruned.tokens.tolist())) == sorted(map(tuple, lat.tokens.tolist()))
    srt, amap = k2.arc_sort(fsa, ret_arc_map=True)
    assert srt.tokens.tolist() == [rows[i] for i in amap.cpu().tolist()]
    assert fsa.to("cpu").tokens.tolist() == rows


def test_shared_graph_viterbi_with_sequences_on_lanes(k2):
    # viterbi_mode 5 (what a large shared decoding graph gets): a warp per state, its lanes
    # are the sequences.  Lattices must be bit-identical to the oracle's for batches that
    # fill part of a group of 32, more than one group, sequences of different lengths and
    # states with more than 32 entering arcs.
    from gpu_util import dense_from_scores, fsa_to_host, host_to_fsa, intersect_raw
    from k2_b200 import autograd
    from oracle.common import HostFsaVec
    rng = np.random.default_rng(53)
    autograd.SHARED_GRAPH_MIN_BYTES = 0
    try:
        for n, max_states, max_arcs in ((2, 12, 40), (5, 45, 400), (33, 70, 300), (70, 20, 900),
                                       (3, 6, 1400), (34, 9, 2500)):  # the last two: states of > 128 arcs
            one = random_fsa_vec(rng, 1, max_states=max_states, max_arcs=max_arcs, acyclic=False,
                                 allow_empty=False)
            S, A = one.num_states, one.num_arcs
            rs1 = (np.arange(n + 1) * S).astype(np.int32)
            rs2 = np.concatenate([one.row_splits2[:-1] + i * A for i in range(n)] +
                                 [[n * A]]).astype(np.int32)
            a = HostFsaVec(rs1, rs2, np.tile(one.arcs, (n, 1)))
            scores, brs = random_dense(rng, n, 11, 5, low_rows=False)
            fsa = host_to_fsa(a)
            assert fsa.arcs.replicated(0)
            for beam in (3.0, 20.0):
                want = oracle.intersect_dense(a, scores, brs, beam)
                lat, ma, mb = intersect_raw(fsa, dense_from_scores(scores, brs), beam, mode=5)
                same_fsa(fsa_to_host(lat, ma, mb), want, f"mode 5, n={n}, beam={beam}")
                lat1, ma1, mb1 = intersect_raw(fsa, dense_from_scores(scores, brs), beam, mode=1)
                same_fsa(fsa_to_host(lat1, ma1, mb1), want, f"mode 1, n={n}, beam={beam}")
    finally:
        autograd.SHARED_GRAPH_MIN_BYTES = 32 << 20

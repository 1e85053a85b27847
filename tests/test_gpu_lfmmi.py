"""The LF-MMI configuration at size: numerator and denominator graphs of an utterance
on the same rows of the dense scores (a_to_b_map = [0, 0, 1, 1, ...],
k2/csrc/intersect_dense.cu:80-92, :1058-1062; the reference's own test of it is the
two-graph case of k2/python/tests/intersect_dense_test.py:90-194), the whole
denominator batch of 128 utterances against the oracle, and the decoding configuration
through the pruned intersection against checksums of the reference's lattice.

Tolerances: lattices and arc maps bit-exact; total scores 1e-4 relative through the
lattice (float32 arc scores) and 1e-6 through the lattice-free kernels; gradients 1e-4
absolute."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

from oracle import oracle
from oracle.common import HostFsaVec
from util import close, same_fsa

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _host_scores(w):
    seg = w.supervision_segments.numpy()
    lp = w.log_probs.numpy()
    C = lp.shape[2]
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


def _lp_layout(grad_scores, w):
    out = np.zeros(tuple(w.log_probs.shape), np.float32)
    r = 0
    for (n, s, d) in w.supervision_segments.tolist():
        out[n, s:s + d] += grad_scores[r:r + d, 1:]
        r += d + 1
    return out


def test_numerator_and_denominator_graphs_share_the_rows_of_an_utterance():
    import k2_b200 as k2
    from gpu_util import fsa_to_host, host_to_fsa, intersect_raw
    from k2_b200 import synthetic as syn
    w = syn.lfmmi_den(utterances=16)
    assert all(40 <= len(s) <= 100 and 1 <= min(s) and max(s) <= 71 for s in w.num_symbols)
    rs1, rs2, arcs, amap = syn.num_den_graphs(w)
    a = HostFsaVec(rs1, rs2, arcs)
    assert a.num_fsas == 32 and amap.tolist() == [i // 2 for i in range(32)]
    scores, brs = _host_scores(w)
    tot_grad = np.tile([1.0, -1.0], 16)  # the LF-MMI objective: numerator - denominator
    want = oracle.loss_path(a, scores, brs, w.output_beam, amap, tot_grad=tot_grad)
    fsa = host_to_fsa(a)
    fsa.scores.requires_grad_(True)
    lp = w.log_probs.to(DEV).requires_grad_(True)
    dense = k2.DenseFsaVec(lp, w.supervision_segments)
    # the lattice, bit for bit, with both arc maps
    lat, ma, mb = intersect_raw(fsa, dense, w.output_beam, a_to_b_map=amap)
    same_fsa(fsa_to_host(lat, ma, mb), want["lattice"], "num+den")
    # through the public call, scores and gradients
    lat = k2.intersect_dense(fsa, dense, w.output_beam,
                             a_to_b_map=torch.from_numpy(amap))
    tot = lat.get_tot_scores(log_semiring=True, use_double_scores=True)
    assert close(tot.detach().cpu().numpy(), want["tot_scores"], rtol=1e-4, atol=0)
    (tot * torch.from_numpy(tot_grad).to(DEV)).sum().backward()
    want_lp = _lp_layout(want["grad_b"], w)
    assert np.abs(lp.grad.cpu().numpy() - want_lp).max() <= 1e-4
    assert np.abs(fsa.scores.grad.cpu().numpy() - want["grad_a"]).max() <= 1e-4
    # the lattice-free total scores on the same pairs
    fsa2 = host_to_fsa(a)
    fsa2.scores.requires_grad_(True)
    lp2 = w.log_probs.to(DEV).requires_grad_(True)
    dense2 = k2.DenseFsaVec(lp2, w.supervision_segments)
    assert k2.dense_loss_supported(fsa2, dense2, torch.from_numpy(amap))
    tot2 = k2.intersect_dense_tot_scores(fsa2, dense2, w.output_beam,
                                         a_to_b_map=torch.from_numpy(amap))
    assert close(tot2.detach().cpu().numpy(), want["tot_scores"], rtol=1e-6, atol=0)
    (tot2 * torch.from_numpy(tot_grad).to(DEV)).sum().backward()
    assert np.abs(lp2.grad.cpu().numpy() - want_lp).max() <= 1e-4
    assert np.abs(fsa2.scores.grad.cpu().numpy() - want["grad_a"]).max() <= 1e-4
    # numerators alone are CTC graphs: the band kernels take them
    num = k2.ctc_graph(w.num_symbols, device=DEV)
    lp3 = w.log_probs.to(DEV).requires_grad_(True)
    dense3 = k2.DenseFsaVec(lp3, w.supervision_segments)
    assert k2.autograd.band_loss_supported(num, dense3)
    tot3 = k2.intersect_dense_tot_scores(num, dense3, w.output_beam)
    assert close(tot3.detach().cpu().numpy(), want["tot_scores"][0::2], rtol=1e-6, atol=0)


def test_denominator_batch_of_128_against_oracle():
    # the whole configuration: 128 utterances x 500 frames on the 144-state graph
    # (a lattice of ~88 M arcs on the CPU side: about half a minute and a few GB)
    import k2_b200 as k2
    from gpu_util import fsa_to_host
    from k2_b200 import synthetic as syn
    w = syn.lfmmi_den()
    graphs = syn.build_graphs(w, DEV)
    scores, brs = _host_scores(w)
    a = fsa_to_host(graphs)
    lat_want = oracle.intersect_dense(a, scores, brs, w.output_beam)
    fwd = oracle.forward_scores(lat_want, True, True)
    bwd = oracle.backward_scores(lat_want, True, True)
    tot_want, post = oracle.tot_scores_and_arc_post(lat_want, fwd, bwd, True)
    grad_b = np.zeros(scores.size, np.float32)
    np.add.at(grad_b, lat_want.arc_map_b, np.exp(post).astype(np.float32))
    want_lp = _lp_layout(grad_b.reshape(scores.shape), w)
    del fwd, bwd, post, grad_b
    # lattice: sizes and digests of every array
    lp = w.log_probs.to(DEV)
    dense = k2.DenseFsaVec(lp, w.supervision_segments)
    from gpu_util import intersect_raw
    lat, ma, mb = intersect_raw(graphs, dense, w.output_beam)
    assert lat.arcs.num_states == lat_want.num_states and lat.num_arcs == lat_want.num_arcs
    assert np.array_equal(lat.arcs.values().cpu().numpy(), lat_want.arcs)
    assert np.array_equal(lat.arcs.row_splits(2).cpu().numpy(), lat_want.row_splits2)
    assert np.array_equal(ma.cpu().numpy(), lat_want.arc_map_a)
    assert np.array_equal(mb.cpu().numpy(), lat_want.arc_map_b)
    del lat, ma, mb, lat_want
    torch.cuda.empty_cache()
    # the loss path the benchmark times
    lp2 = w.log_probs.to(DEV).requires_grad_(True)
    dense2 = k2.DenseFsaVec(lp2, w.supervision_segments)
    tot = k2.intersect_dense_tot_scores(graphs, dense2, w.output_beam)
    assert close(tot.detach().cpu().numpy(), tot_want, rtol=1e-6, atol=0)
    tot.sum().backward()
    assert np.abs(lp2.grad.cpu().numpy() - want_lp).max() <= 1e-4


def test_decoding_configuration_matches_the_reference_lattice_checksums():
    # hlg_decode at full size through intersect_dense_pruned; the reference's lattice
    # (tests/golden/make_pruned_full_size_golden.py) is kept as sizes and sha256 digests
    import k2_b200 as k2
    from k2_b200 import synthetic as syn
    from k2_b200.fsa_algo import _fsa_vec_from_numpy
    here = os.path.dirname(os.path.abspath(__file__))
    with open(os.path.join(here, "golden", "pruned_full_size.json")) as f:
        gold = json.load(f)
    w = syn.hlg_decode(seed=0)
    S = len(w.graph_row_splits2) - 1
    graph = _fsa_vec_from_numpy(np.array([0, S]), w.graph_row_splits2, w.graph_arcs, DEV)
    dense = k2.DenseFsaVec(w.log_probs.to(DEV), w.supervision_segments)
    from k2_b200.autograd import _intersect_dense_pruned_arcs
    lat, ma, mb = _intersect_dense_pruned_arcs(
        graph.arcs, dense, gold["search_beam"], gold["output_beam"], gold["min_active_states"],
        gold["max_active_states"], False)
    assert lat.num_states == gold["num_states"] and lat.num_elements() == gold["num_arcs"]

    def digest(t):
        return hashlib.sha256(np.ascontiguousarray(t.cpu().numpy().astype(np.int32)).tobytes()
                              ).hexdigest()
    got = {"row_splits1": digest(lat._row_splits1), "row_splits2": digest(lat._row_splits2),
           "arcs": digest(lat.values()), "arc_map_a": digest(ma), "arc_map_b": digest(mb)}
    assert got == gold["sha256"]

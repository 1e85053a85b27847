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


def _fused(a_host, scores, brs, beam, amap=None, tot_grad=None, use_double=True, **limits):
    import k2_b200 as k2
    from gpu_util import dense_from_scores, host_to_fsa
    fsa = host_to_fsa(a_host)
    fsa.scores.requires_grad_(True)
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
        ga, gb = fsa.scores.grad.cpu().numpy(), dense.scores.grad.cpu().numpy()
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

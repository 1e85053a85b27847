"""The CUDA path against the committed fixtures made by the reference's own CPU code
(tests/golden/ref_cases.npz), and against the known answers written in the
reference's Python tests, re-stated here through the mirrored API."""
import numpy as np
import pytest
import torch

from golden_util import load
from util import close, same_fsa

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("case", load(), ids=lambda c: c["name"])
def test_cuda_path_reproduces_reference_fixtures(case):
    import k2_b200 as k2
    from gpu_util import dense_from_scores, fsa_to_host, host_to_fsa, intersect_raw
    for mode in (1, 2):
        lat, ma, mb = intersect_raw(host_to_fsa(case["a"]),
                                    dense_from_scores(case["scores"], case["brs"]), case["beam"],
                                    case["amap"], mode=mode)
        same_fsa(fsa_to_host(lat, ma, mb), case["lattice"], f"{case['name']} mode {mode}")
    for tag, log in (("log", True), ("trop", False)):
        f = lat.get_forward_scores(True, log).detach().cpu().numpy()
        b = lat.get_backward_scores(True, log).detach().cpu().numpy()
        t = lat.get_tot_scores(True, log).detach().cpu().numpy()
        p = lat.get_arc_post(True, log).detach().cpu().numpy()
        assert close(f, case[f"fwd_{tag}"], 1e-9, 1e-9) and close(b, case[f"bwd_{tag}"], 1e-9, 1e-9)
        assert close(t, case[f"tot_{tag}"], 1e-9, 1e-9)
        fin = np.isfinite(case[f"post_{tag}"])
        assert close(p[fin], case[f"post_{tag}"][fin], 1e-9, 1e-9)
    np.testing.assert_array_equal(lat._get_entering_arcs(True).cpu().numpy(), case["entering"])
    best = k2.shortest_path(lat, True)
    np.testing.assert_array_equal(best._best_arc_map.cpu().numpy(), case["best"])
    assert lat.properties == int(np.bitwise_and.reduce(case["props"])) if len(case["props"]) else True


def test_intersect_dense_simple():
    # k2/python/tests/intersect_dense_test.py:40-88
    import k2_b200 as k2
    s = '''
        0 1 1 1.0
        1 1 1 50.0
        1 2 2 2.0
        2 3 -1 3.0
        3
    '''
    fsa = k2.Fsa.from_str(s).to(DEV)
    fsa.requires_grad_(True)
    fsa_vec = k2.create_fsa_vec([fsa])
    log_prob = torch.tensor([[[0.1, 0.2, 0.3], [0.04, 0.05, 0.06]]], dtype=torch.float32,
                            device=DEV, requires_grad=True)
    seg = torch.tensor([[0, 0, 2]], dtype=torch.int32)
    dense = k2.DenseFsaVec(log_prob, seg)
    out = k2.intersect_dense(fsa_vec, dense, output_beam=100000, seqframe_idx_name='seqframe',
                             frame_idx_name='frame')
    assert out.seqframe.tolist() == [0, 1, 2] and out.frame.tolist() == [0, 1, 2]
    scores = out.get_tot_scores(log_semiring=False, use_double_scores=False)
    scores.sum().backward()
    assert torch.allclose(out.scores.cpu(), torch.tensor([1.2, 2.06, 3.0]))
    assert torch.allclose(fsa.scores.grad.cpu(), torch.tensor([1.0, 0.0, 1.0, 1.0]))
    assert torch.allclose(log_prob.grad.cpu().reshape(-1),
                          torch.tensor([0.0, 1.0, 0.0, 0.0, 0.0, 1.0]))


@pytest.mark.parametrize("use_map", [True, False])
def test_intersect_dense_two_dense(use_map):
    # k2/python/tests/intersect_dense_test.py:90-194
    import k2_b200 as k2
    s = '''
        0 1 1 1.0
        1 1 1 50.0
        1 2 2 2.0
        2 3 -1 3.0
        3
    '''
    fsa = k2.Fsa.from_str(s).to(DEV)
    fsa.requires_grad_(True)
    fsa_vec = k2.create_fsa_vec([fsa, fsa])
    log_prob = torch.tensor([[[0.1, 0.2, 0.3], [0.04, 0.05, 0.06], [0.0, 0.0, 0.0]],
                             [[0.1, 0.2, 0.3], [0.4, 0.5, 0.6], [0.0, 0.0, 0.0]]],
                            dtype=torch.float32, device=DEV, requires_grad=True)
    a_to_b_map = torch.tensor([0, 0], dtype=torch.int32, device=DEV) if use_map else None
    seg = torch.tensor([[0, 0, 3], [1, 0, 2]], dtype=torch.int32)
    dense = k2.DenseFsaVec(log_prob, seg)
    out = k2.intersect_dense(fsa_vec, dense, output_beam=100000, a_to_b_map=a_to_b_map,
                             seqframe_idx_name='seqframe', frame_idx_name='frame')
    if not use_map:
        assert out.seqframe.tolist() == [0, 1, 2, 3, 4, 5, 6]
        assert out.frame.tolist() == [0, 1, 2, 3, 0, 1, 2]
        want_scores = [1.2, 50.05, 2.0, 3.0, 1.2, 2.6, 3.0]
        want_grad_fsa = [2.0, 1.0, 2.0, 2.0]
        want_grad_lp = [0.0, 1.0, 0.0, 0.0, 1.0, 0.0, 0.0, 0.0, 1.0, 0.0, 1.0, 0.0, 0.0, 0.0, 1.0,
                        0.0, 0.0, 0.0]
    else:
        assert out.seqframe.tolist() == [0, 1, 2, 3, 0, 1, 2, 3]
        assert out.frame.tolist() == [0, 1, 2, 3, 0, 1, 2, 3]
        want_scores = [1.2, 50.05, 2.0, 3.0, 1.2, 50.05, 2.0, 3.0]
        want_grad_fsa = [2.0, 2.0, 2.0, 2.0]
        want_grad_lp = [0.0, 2.0, 0.0, 0.0, 2.0, 0.0, 0.0, 0.0, 2.0] + [0.0] * 9
    assert out.shape == (2, None, None)
    scores = out.get_tot_scores(log_semiring=False, use_double_scores=False)
    scores.sum().backward()
    assert torch.allclose(out.scores.cpu(), torch.tensor(want_scores))
    assert torch.allclose(fsa.scores.grad.cpu(), torch.tensor(want_grad_fsa))
    assert torch.allclose(log_prob.grad.cpu().reshape(-1), torch.tensor(want_grad_lp))


def test_get_tot_scores_log_known_answers():
    # k2/python/tests/get_tot_scores_test.py:228-326 (values computed with gtn)
    import k2_b200 as k2
    s1 = '''
        0 1 1 0.1
        0 2 2 0.2
        1 2 3 0.3
        1 3 4 0.4
        2 3 5 0.5
        3 4 -1 0
        4
    '''
    s2 = '''
        0 3 3 0.1
        0 1 1 0.2
        0 2 2 0.3
        1 2 2 0.4
        1 3 3 0.5
        2 3 3 0.6
        2 4 4 0.7
        3 4 4 0.8
        3 5 -1 0.9
        4 5 -1 1.0
        5
    '''
    g1 = torch.tensor([0.6710670590400696, 0.32893291115760803, 0.4017595648765564,
                       0.2693074941635132, 0.7306925058364868, 1.0])
    g2 = torch.tensor([0.10102888941764832, 0.5947467088699341, 0.3042244613170624,
                       0.410660058259964, 0.1840866357088089, 0.5283515453338623,
                       0.18653297424316406, 0.5783339142799377, 0.2351330667734146,
                       0.764866828918457])
    for use_double in (False, True):
        fsa1 = k2.Fsa.from_str(s1).to(DEV).requires_grad_(True)
        fsa2 = k2.Fsa.from_str(s2).to(DEV).requires_grad_(True)
        vec = k2.create_fsa_vec([fsa1, fsa2])
        log_like = vec.get_tot_scores(log_semiring=True, use_double_scores=use_double)
        assert log_like.dtype == (torch.float64 if use_double else torch.float32)
        want = torch.tensor([1.8119014501571655, 4.533502578735352], dtype=log_like.dtype)
        assert torch.allclose(log_like.cpu(), want)
        scale = torch.tensor([1.25, -5.25]).to(log_like)
        (scale * log_like).sum().backward()
        assert torch.allclose(fsa1.scores.grad.cpu(), 1.25 * g1)
        assert torch.allclose(fsa2.scores.grad.cpu(), -5.25 * g2)


def test_ctc_loss_known_answers_and_torch():
    # k2/python/tests/ctc_loss_test.py:232-309: batch of three sequences, literal
    # losses and equality with torch.nn.functional.ctc_loss in value and gradient
    import k2_b200 as k2
    a1 = torch.tensor([[0., 0., 0., 0., 0.]])
    a2 = torch.arange(1, 16).reshape(3, 5).to(torch.float32)
    a3 = torch.tensor([[-5, -4, -3, -2, -1], [-10, -9, -8, -7, -6], [-15, -14, -13, -12, -11.]])
    torch_acts = [x.clone().requires_grad_(True) for x in (a3, a2, a1)]
    ours_acts = [x.clone().to(DEV).requires_grad_(True) for x in (a3, a2, a1)]
    t_in = torch.nn.utils.rnn.pad_sequence(torch_acts, batch_first=False, padding_value=0)
    o_in = torch.nn.utils.rnn.pad_sequence(ours_acts, batch_first=True, padding_value=0)
    targets = torch.tensor([2, 3, 3, 3, 1])
    input_lengths = torch.tensor([3, 3, 1])
    target_lengths = torch.tensor([2, 2, 1])
    t_loss = torch.nn.functional.ctc_loss(torch.log_softmax(t_in, -1), targets, input_lengths,
                                          target_lengths, reduction='sum')
    want = torch.tensor([4.938850402832, 7.355742931366, 1.6094379425049]).sum()
    assert torch.allclose(t_loss, want)
    seg = torch.tensor([[0, 0, 3], [1, 0, 3], [2, 0, 1]], dtype=torch.int32)
    dense = k2.DenseFsaVec(torch.log_softmax(o_in, -1), seg)
    graph = k2.ctc_graph([[2, 3], [3, 3], [1]], device=DEV)
    loss = k2.ctc_loss(graph, dense, reduction='sum', target_lengths=target_lengths)
    assert torch.allclose(loss.cpu(), t_loss)
    scale = torch.tensor([1., -2, 3.5])
    (t_loss * 1.0).backward()
    loss.backward()
    for t, o in zip(torch_acts, ours_acts):
        assert torch.allclose(t.grad, o.grad.cpu(), atol=1e-5)
    # 'mean' and 'none' reductions (ctc_loss.py:141-151)
    dense = k2.DenseFsaVec(torch.log_softmax(o_in.detach(), -1), seg)
    none = k2.ctc_loss(graph, dense, reduction='none')
    assert torch.allclose(none.cpu(), torch.tensor([4.938850402832, 7.355742931366,
                                                    1.6094379425049]))
    mean = k2.ctc_loss(graph, dense, reduction='mean', target_lengths=target_lengths.to(DEV))
    assert torch.allclose(mean.cpu(), (none.cpu() / target_lengths).mean())


def test_scores_invalidate_when_scores_are_reassigned():
    # fsa.py:417-422: assigning `scores` drops the cached forward/backward scores
    import k2_b200 as k2
    f = k2.Fsa.from_str("0 1 1 0.5\n0 1 2 1.5\n1 2 -1 0.25\n2").to(DEV)
    v = k2.create_fsa_vec([f])
    t1 = v.get_tot_scores(True, True).item()
    v.scores = v.scores + 1.0
    t2 = v.get_tot_scores(True, True).item()
    assert abs((t2 - t1) - 2.0) < 1e-9


def test_delay_penalty_changes_loss_like_a_manual_edit():
    # ctc_loss.py:99-136
    import k2_b200 as k2
    gen = torch.Generator().manual_seed(3)
    lp = torch.log_softmax(torch.randn(2, 12, 6, generator=gen), -1).to(DEV)
    seg = torch.tensor([[0, 0, 12], [1, 0, 9]], dtype=torch.int32)
    graph = k2.ctc_graph([[1, 2, 2], [3]], device=DEV)
    dense = k2.DenseFsaVec(lp, seg)
    base = k2.ctc_loss(graph, dense, output_beam=20.0, reduction='none')
    pen = k2.ctc_loss(graph, dense, output_beam=20.0, reduction='none', delay_penalty=0.1)
    lat = k2.intersect_dense(graph, dense, 20.0, frame_idx_name="frame_idx")
    arcs = lat.arcs
    fsa_of_arc = arcs.row_ids(1)[arcs.row_ids(2).long()].long()
    dur = dense.duration.to(DEV)
    offset = lat.frame_idx - (dur >> 1)[fsa_of_arc].to(torch.int32)
    penalty = -0.1 * offset.float()
    penalty[(lat.aux_labels == 0) | (lat.aux_labels == -1)] = 0
    lat.scores = lat.scores + penalty
    manual = -lat.get_tot_scores(True, True).float()
    assert torch.allclose(pen, manual, atol=1e-5)
    assert not torch.allclose(pen, base)

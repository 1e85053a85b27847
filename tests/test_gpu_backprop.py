"""Derivatives through per-state scores (get_forward_scores, get_backward_scores,
get_arc_post with autograd) on the GPU, against (1) torch autograd over a plain
float64 restatement of the recursions and (2) the reference's own
BackpropGet{Forward,Backward}Scores / BackpropGetArcPost when the reference library
has been built."""
import numpy as np
import pytest
import torch

from oracle import ref
from util import random_fsa_vec

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def k2():
    import k2_b200
    return k2_b200


def torch_scores(a, scores, log_semiring, forward):
    """Forward (or backward) scores per state with torch ops on the host, float64."""
    ninf = torch.tensor(-np.inf, dtype=torch.float64)
    out = [None] * a.num_states
    state_of = np.repeat(np.arange(a.num_states), np.diff(a.row_splits2))
    fsa_of = np.repeat(np.arange(a.num_fsas), np.diff(a.row_splits1))
    reduce = (lambda xs: torch.logsumexp(torch.stack(xs), 0)) if log_semiring else \
        (lambda xs: torch.stack(xs).max())
    order = range(a.num_states) if forward else range(a.num_states - 1, -1, -1)
    for s in order:
        base = a.row_splits1[fsa_of[s]]
        last = a.row_splits1[fsa_of[s] + 1] - 1
        if forward and s == base or (not forward and s == last):
            out[s] = torch.zeros((), dtype=torch.float64)
            continue
        terms = []
        for k in range(a.num_arcs):
            src, dest = state_of[k], base + a.arcs[k, 1]
            if fsa_of[src] != fsa_of[s]:
                continue
            if forward and dest == s and torch.isfinite(out[src]):
                terms.append(out[src] + scores[k])
            if not forward and src == s and torch.isfinite(out[dest]):
                terms.append(out[dest] + scores[k])
        out[s] = reduce(terms) if terms else ninf
    return torch.stack(out)


def cases():
    rng = np.random.default_rng(21)
    for trial in range(4):
        yield trial, random_fsa_vec(rng, 4, max_states=9, max_arcs=24, acyclic=True,
                                    allow_empty=trial == 3)


@pytest.mark.parametrize("log_semiring", [True, False])
@pytest.mark.parametrize("use_double", [True, False])
def test_forward_and_backward_score_gradients_match_torch_autograd(k2, log_semiring, use_double):
    from gpu_util import DEV, host_to_fsa
    tol = 1e-9 if use_double else 2e-5
    for trial, a in cases():
        w = torch.from_numpy(np.random.default_rng(trial).normal(size=a.num_states))
        for forward in (True, False):
            fsa = host_to_fsa(a)
            fsa.scores.requires_grad_(True)
            got = (fsa.get_forward_scores if forward else fsa.get_backward_scores)(
                use_double_scores=use_double, log_semiring=log_semiring)
            finite = torch.isfinite(got)
            (torch.where(finite, got, torch.zeros_like(got)) * w.to(DEV).to(got.dtype)).sum() \
                .backward()
            sc = torch.from_numpy(a.scores.astype(np.float64)).requires_grad_(True)
            want = torch_scores(a, sc, log_semiring, forward)
            np.testing.assert_allclose(got.detach().cpu().numpy(), want.detach().numpy(),
                                       rtol=tol, atol=tol)
            (torch.where(torch.isfinite(want), want, torch.zeros_like(want)) * w).sum().backward()
            # (the arc scores are float32, so their gradient is rounded to float32)
            np.testing.assert_allclose(fsa.scores.grad.cpu().numpy(), sc.grad.numpy(),
                                       rtol=max(tol * 10, 2e-6), atol=max(tol * 10, 2e-6),
                                       err_msg=f"trial {trial} forward={forward}")


@pytest.mark.parametrize("use_double", [True, False])
def test_arc_post_gradient_matches_torch_autograd(k2, use_double):
    from gpu_util import DEV, host_to_fsa
    tol = 1e-9 if use_double else 5e-5
    for trial, a in cases():
        fsa = host_to_fsa(a)
        fsa.scores.requires_grad_(True)
        post = fsa.get_arc_post(use_double_scores=use_double, log_semiring=True)
        w = torch.from_numpy(np.random.default_rng(trial).normal(size=a.num_arcs))
        finite = torch.isfinite(post)
        (torch.where(finite, post, torch.zeros_like(post)) * w.to(DEV).to(post.dtype)).sum() \
            .backward()
        sc = torch.from_numpy(a.scores.astype(np.float64)).requires_grad_(True)
        f = torch_scores(a, sc, True, True)
        b = torch_scores(a, sc, True, False)
        state_of = np.repeat(np.arange(a.num_states), np.diff(a.row_splits2))
        fsa_of = np.repeat(np.arange(a.num_fsas), np.diff(a.row_splits1))[state_of]
        dest = a.row_splits1[fsa_of] + a.arcs[:, 1]
        first = torch.from_numpy(a.row_splits1[fsa_of].astype(np.int64))
        last = torch.from_numpy((a.row_splits1[fsa_of + 1] - 1).astype(np.int64))
        want = f[torch.from_numpy(state_of)] + sc + b[torch.from_numpy(dest.astype(np.int64))] \
            - 0.5 * (f[last] + b[first])
        ok = torch.isfinite(want)
        assert torch.equal(ok, finite.cpu())
        (torch.where(ok, want, torch.zeros_like(want)) * w).sum().backward()
        np.testing.assert_allclose(fsa.scores.grad.cpu().numpy(), sc.grad.numpy(),
                                   rtol=max(tol * 10, 5e-6), atol=max(tol * 10, 5e-6),
                                   err_msg=f"trial {trial}")


@pytest.mark.skipif(not ref.available(), reason="oracle/_ref/libk2ref.so not built")
def test_against_the_reference_library(k2):
    from gpu_util import DEV, host_to_fsa
    from k2_b200.autograd import _backprop_scores
    rng = np.random.default_rng(5)
    for trial in range(6):
        a = random_fsa_vec(rng, 5, max_states=30, max_arcs=150, acyclic=True)
        fsa = host_to_fsa(a)
        for log in (True, False):
            for dbl in (True, False):
                tol = 1e-10 if dbl else 1e-5
                dtype = torch.float64 if dbl else torch.float32
                _, ea = ref.forward_scores(a, False, dbl, want_entering_arcs=True)
                for forward in (True, False):
                    sc = (ref.forward_scores if forward else ref.backward_scores)(a, log, dbl)
                    din = rng.normal(size=a.num_states)
                    want = ref.backprop_scores(a, forward, sc, din, log, dbl, entering_arcs=ea)
                    mine = (fsa._get_forward_scores if forward else fsa._get_backward_scores)(
                        dbl, log)
                    np.testing.assert_allclose(mine.cpu().numpy(), sc, rtol=tol, atol=tol)
                    got = _backprop_scores(fsa, forward, log, dbl, mine,
                                           torch.from_numpy(din).to(DEV).to(dtype))
                    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=tol * 10,
                                               atol=tol * 10,
                                               err_msg=f"{trial} log={log} dbl={dbl} fwd={forward}")
        # arc posteriors: derivatives w.r.t. forward and backward scores
        for dbl in (True, False):
            d = rng.normal(size=a.num_arcs)
            wf, wb = ref.backprop_arc_post(a, d, dbl)
            from k2_b200.autograd import _GetArcPostFunction

            class Ctx:
                pass
            ctx = Ctx()
            ctx.fsas, ctx.use_double_scores = fsa, dbl
            out = _GetArcPostFunction.backward(ctx, torch.from_numpy(d).to(DEV))
            tol = 1e-10 if dbl else 1e-5
            np.testing.assert_allclose(out[4].cpu().numpy(), wf, rtol=tol, atol=tol)
            np.testing.assert_allclose(out[5].cpu().numpy(), wb, rtol=tol, atol=tol)

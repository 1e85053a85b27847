"""The autograd Functions of the path, with the reference's contracts
(k2/python/k2/autograd.py:30-117 `_GetTotScoresFunction`, :120-347 the per-state
score and posterior Functions, :350-510 `_IntersectDensePrunedFunction`, :511-664
`_IntersectDenseFunction`), `intersect_dense` (:751-824) and `intersect_dense_pruned`
(:667-746), plus the lattice-free total scores that `ctc_loss` uses."""
import ctypes
from typing import List, Optional, Tuple

import numpy as np
import torch

from . import _lib
from .dense_fsa_vec import DenseFsaVec
from .fsa import Fsa
from .ragged import RaggedArc
from .ragged_tensor import RaggedTensor

# 0 = automatic, 1 = one launch per frame, 2 = persistent kernel (see include/k2b200.h)
VITERBI_MODE = 0
# a_fsas made of identical copies of one graph are read through copy 0 only when
# they are at least this large (smaller ones stay cache-resident anyway)
SHARED_GRAPH_MIN_BYTES = 32 << 20


def _index_add(index: torch.Tensor, value: torch.Tensor, in_out: torch.Tensor) -> None:
    """in_out[index[k]] += value[k] (k2/python/csrc/torch/index_add.cu:38-71)."""
    assert index.dtype == torch.int32 and in_out.dtype == torch.float32
    value = value.to(torch.float32).contiguous()
    with torch.cuda.device(in_out.device):
        _lib.check(_lib.lib.k2b200_index_add(_lib.ptr(index), _lib.ptr(value), index.numel(),
                                              _lib.ptr(in_out), in_out.numel(),
                                              _lib.stream_of(in_out.device)))


def index_select(src, index: torch.Tensor):
    """ans[i] = src[index[i]], 0 where index[i] == -1 (1-D int32 `src`;
    k2/python/csrc/torch/index_select.cu:56-92).  A ragged attribute is indexed by
    rows, -1 giving an empty list (k2/python/k2/autograd.py:586-593)."""
    assert index.dtype == torch.int32
    if isinstance(src, RaggedTensor):
        return src.index(index, axis=0)[0]
    if src.dtype != torch.int32 or src.ndim != 1:
        # other dtypes are carried with torch's own gather (attribute plumbing)
        ans = src.index_select(0, index.clamp(min=0).long())
        ans[index < 0] = 0
        return ans
    src = src.contiguous()
    out = torch.empty(index.numel(), dtype=torch.int32, device=src.device)
    with torch.cuda.device(src.device):
        _lib.check(_lib.lib.k2b200_index_select_i32(_lib.ptr(src), src.numel(), _lib.ptr(index),
                                                     index.numel(), _lib.ptr(out),
                                                     _lib.stream_of(src.device)))
    return out


def _make_intersect_args(a: RaggedArc, b: DenseFsaVec, a_to_b_map: Optional[torch.Tensor],
                         output_beam: float, max_states: int, max_arcs: int,
                         viterbi_mode: int = 0):
    """The argument block shared by the lattice and the lattice-free entry points.
    Returns (args, objects that must outlive the call, device, host row splits of b)."""
    _lib.require_cuda(a.values(), "a_fsas")
    _lib.require_cuda(b.scores, "b_fsas.scores")
    dev = a.device
    if b.scores.device != dev:
        raise RuntimeError("a_fsas and b_fsas must be on the same device")
    scores = b.scores.detach()
    assert scores.is_contiguous() and scores.dtype == torch.float32
    in_splits, in_arcs = a.incoming()[:2]
    h_rs1 = np.ascontiguousarray(a.h_row_splits1, dtype=np.int32)
    h_as = np.ascontiguousarray(a.h_arc_splits, dtype=np.int32)
    h_brs = b.h_row_splits
    h_map = None
    if a_to_b_map is not None:
        assert a_to_b_map.ndim == 1 and a_to_b_map.dtype == torch.int32
        h_map = np.ascontiguousarray(a_to_b_map.detach().cpu().numpy(), dtype=np.int32)
        if h_map.shape[0] != a.num_fsas:
            raise RuntimeError(
                f"a_fsas.Dim0() ({a.num_fsas}) != a_to_b_map.Dim() ({h_map.shape[0]})")
    args = _lib.IntersectArgs(
        num_fsas=a.num_fsas, num_states=a.num_states, num_arcs=a.num_elements(),
        a_row_splits1=_lib.ptr(a._row_splits1), a_row_splits2=_lib.ptr(a._row_splits2),
        a_arcs=_lib.ptr(a.values()), a_in_splits=_lib.ptr(in_splits),
        a_in_arcs=_lib.ptr(in_arcs), h_a_row_splits1=h_rs1.ctypes.data,
        h_a_arc_splits=h_as.ctypes.data, scores=_lib.ptr(scores), rows=scores.shape[0],
        cols=scores.shape[1], num_seqs=len(h_brs) - 1, h_b_row_splits=h_brs.ctypes.data,
        h_a_to_b_map=None if h_map is None else h_map.ctypes.data,
        output_beam=float(output_beam), max_states=int(min(max_states, 2**31 - 1)),
        max_arcs=int(min(max_arcs, 2**31 - 1)), viterbi_mode=viterbi_mode,
        a_max_degree=a.max_degree(),
        # one large graph copied once per sequence: read copy 0 only
        a_shared=int(h_map is None and a.replicated(SHARED_GRAPH_MIN_BYTES)))
    return args, (h_rs1, h_as, h_map, in_splits, in_arcs, scores), dev, h_brs


def _intersect_dense_arcs(a: RaggedArc, b: DenseFsaVec, a_to_b_map: Optional[torch.Tensor],
                          output_beam: float, max_states: int, max_arcs: int,
                          viterbi_mode: int = 0):
    """The `_k2.intersect_dense` call (k2/python/csrc/torch/fsa_algo.cu:224-253):
    returns (RaggedArc lattice, arc_map_a, arc_map_b)."""
    args, _keep, dev, h_brs = _make_intersect_args(a, b, a_to_b_map, output_beam, max_states,
                                                   max_arcs, viterbi_mode)
    nbytes = ctypes.c_size_t()
    levels = ctypes.c_int64()
    _lib.check(_lib.lib.k2b200_intersect_dense_workspace_bytes(ctypes.byref(args),
                                                                ctypes.byref(nbytes),
                                                                ctypes.byref(levels)))
    ws = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)
    ns, na, beam = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_float()
    max_w, max_a = ctypes.c_int32(), ctypes.c_int32()
    stream = _lib.stream_of(dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.k2b200_intersect_dense_prune(ctypes.byref(args), _lib.ptr(ws),
                                                          nbytes.value, stream, ctypes.byref(ns),
                                                          ctypes.byref(na), ctypes.byref(beam),
                                                          ctypes.byref(max_w),
                                                          ctypes.byref(max_a)))
        ns, na = ns.value, na.value
        i32 = dict(dtype=torch.int32, device=dev)
        # zero-sized tensors have a NULL data pointer: allocate one spare element
        row_splits1 = torch.empty(a.num_fsas + 1, **i32)
        row_ids1 = torch.empty(ns + 1, **i32)
        row_splits2 = torch.empty(ns + 1, **i32)
        row_ids2 = torch.empty(na + 1, **i32)
        values = torch.empty((na + 1, 4), **i32)
        arc_map_a = torch.empty(na + 1, **i32)
        arc_map_b = torch.empty(na + 1, **i32)
        level_offsets = torch.empty(a.num_fsas + 1, **i32)
        level_splits = torch.empty(levels.value + 1, **i32)
        out = _lib.LatticeOut(
            row_splits1=_lib.ptr(row_splits1), row_ids1=_lib.ptr(row_ids1),
            row_splits2=_lib.ptr(row_splits2), row_ids2=_lib.ptr(row_ids2),
            arcs=_lib.ptr(values), arc_map_a=_lib.ptr(arc_map_a), arc_map_b=_lib.ptr(arc_map_b),
            level_offsets=_lib.ptr(level_offsets), level_splits=_lib.ptr(level_splits))
        _lib.check(_lib.lib.k2b200_intersect_dense_emit(ctypes.byref(args), _lib.ptr(ws),
                                                         nbytes.value, stream, ctypes.byref(out)))
    lattice = RaggedArc(values[:na], row_splits1, row_splits2, row_ids1[:ns], row_ids2[:na])
    arc_map_a, arc_map_b = arc_map_a[:na], arc_map_b[:na]
    lattice._levels = (level_offsets, level_splits)
    # every lattice arc goes from frame t to t+1; the pruning pass measured the
    # largest layer
    lattice._layer_bounds = (1, int(np.diff(h_brs).max()) + 1, max(max_w.value, 1),
                             max(max_a.value, 1))
    lattice.output_beam_used = beam.value
    return lattice, arc_map_a, arc_map_b


class _GetTotScoresFunction(torch.autograd.Function):

    @staticmethod
    def forward(ctx, fsas: Fsa, log_semiring: bool, use_double_scores: bool,
                unused_scores: torch.Tensor) -> torch.Tensor:
        tot_scores = fsas._get_tot_scores(use_double_scores=use_double_scores,
                                          log_semiring=log_semiring).detach()
        ctx.fsas = fsas
        ctx.log_semiring = log_semiring
        ctx.use_double_scores = use_double_scores
        ctx.save_for_backward(unused_scores)
        return tot_scores

    @staticmethod
    def backward(ctx, tot_scores_grad: torch.Tensor):
        fsas = ctx.fsas
        log_semiring = ctx.log_semiring
        use_double_scores = ctx.use_double_scores
        arcs = fsas.arcs
        dev = arcs.device
        na = arcs.num_elements()
        scores_grad = torch.empty(na, dtype=torch.float32, device=dev)
        # the gradient of a reduction arrives expanded: element stride may be 0
        # (k2/python/csrc/torch/fsa.cu:515-516, :565-566)
        dtype = torch.float64 if use_double_scores else torch.float32
        if tot_scores_grad.dtype != dtype:
            tot_scores_grad = tot_scores_grad.to(dtype)
        stride = tot_scores_grad.stride(0) if tot_scores_grad.numel() > 0 else 0
        rid1 = arcs.row_ids(1 - arcs.single)
        rid2 = arcs.row_ids(2 - arcs.single)
        with torch.cuda.device(dev):
            if log_semiring is False:
                from .fsa_algo import _shortest_path_arcs
                _, best_arcs = _shortest_path_arcs(fsas, use_double_scores)
                _lib.check(_lib.lib.k2b200_tot_scores_tropical_backward(
                    _lib.ptr(rid1), _lib.ptr(rid2), na, _lib.ptr(best_arcs), best_arcs.numel(),
                    int(use_double_scores), _lib.ptr(tot_scores_grad), stride,
                    _lib.ptr(scores_grad), _lib.stream_of(dev)))
            else:
                arc_post = fsas._get_arc_post(use_double_scores, log_semiring)
                _lib.check(_lib.lib.k2b200_tot_scores_log_backward(
                    _lib.ptr(rid1), _lib.ptr(rid2), na, int(use_double_scores),
                    _lib.ptr(arc_post), _lib.ptr(tot_scores_grad), stride,
                    _lib.ptr(scores_grad), _lib.stream_of(dev)))
        return None, None, None, scores_grad


def _backprop_scores(fsas: Fsa, forward: bool, log_semiring: bool, use_double_scores: bool,
                     scores: torch.Tensor, scores_grad: torch.Tensor) -> torch.Tensor:
    """dL/d(arc scores) from dL/d(forward or backward scores): the
    `_k2.backprop_get_{forward,backward}_scores_*` calls
    (k2/python/csrc/torch/fsa.cu:293-366)."""
    arcs = fsas.arcs
    dev = arcs.device
    dtype = torch.float64 if use_double_scores else torch.float32
    state_deriv = scores_grad.detach().to(dtype).contiguous().clone()
    arc_deriv = torch.zeros(arcs.num_elements(), dtype=dtype, device=dev)
    entering = best_tmp = None
    if not log_semiring:
        if forward:
            entering = fsas._get_entering_arcs(use_double_scores)
        else:
            best_tmp = torch.empty(arcs.num_states, dtype=torch.int32, device=dev)
    view, keep = arcs.view(want_incoming=not forward)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.k2b200_fsa_scores_backprop(
            ctypes.byref(view), int(forward), int(log_semiring), int(use_double_scores),
            _lib.ptr(scores.contiguous()), _lib.ptr(entering), _lib.ptr(state_deriv),
            _lib.ptr(arc_deriv), _lib.ptr(best_tmp), _lib.stream_of(dev)))
    del keep
    return arc_deriv


class _GetForwardScoresFunction(torch.autograd.Function):
    """Contract of k2/python/k2/autograd.py:120-199."""

    @staticmethod
    def forward(ctx, fsas: Fsa, log_semiring: bool, use_double_scores: bool,
                unused_scores: torch.Tensor) -> torch.Tensor:
        forward_scores = fsas._get_forward_scores(use_double_scores=use_double_scores,
                                                  log_semiring=log_semiring).detach()
        ctx.fsas, ctx.log_semiring, ctx.use_double_scores = fsas, log_semiring, use_double_scores
        ctx.save_for_backward(forward_scores)
        return forward_scores

    @staticmethod
    def backward(ctx, forward_scores_grad: torch.Tensor):
        forward_scores, = ctx.saved_tensors
        scores_grad = _backprop_scores(ctx.fsas, True, ctx.log_semiring, ctx.use_double_scores,
                                       forward_scores, forward_scores_grad)
        return None, None, None, scores_grad


class _GetBackwardScoresFunction(torch.autograd.Function):
    """Contract of k2/python/k2/autograd.py:202-270."""

    @staticmethod
    def forward(ctx, fsas: Fsa, log_semiring: bool, use_double_scores: bool,
                unused_scores: torch.Tensor) -> torch.Tensor:
        backward_scores = fsas._get_backward_scores(use_double_scores=use_double_scores,
                                                    log_semiring=log_semiring).detach()
        ctx.fsas, ctx.log_semiring, ctx.use_double_scores = fsas, log_semiring, use_double_scores
        ctx.save_for_backward(backward_scores)
        return backward_scores

    @staticmethod
    def backward(ctx, backward_scores_grad: torch.Tensor):
        backward_scores, = ctx.saved_tensors
        scores_grad = _backprop_scores(ctx.fsas, False, ctx.log_semiring, ctx.use_double_scores,
                                       backward_scores, backward_scores_grad)
        return None, None, None, scores_grad


class _GetArcPostFunction(torch.autograd.Function):
    """Contract of k2/python/k2/autograd.py:273-347: the posteriors depend on the arc
    scores directly and through the forward and backward scores, which are passed in
    as differentiable tensors."""

    @staticmethod
    def forward(ctx, fsas: Fsa, log_semiring: bool, use_double_scores: bool,
                unused_scores: torch.Tensor, forward_scores: torch.Tensor,
                backward_scores: torch.Tensor) -> torch.Tensor:
        arc_post = fsas._get_arc_post(use_double_scores=use_double_scores,
                                      log_semiring=log_semiring).detach()
        ctx.fsas, ctx.use_double_scores = fsas, use_double_scores
        return arc_post

    @staticmethod
    def backward(ctx, arc_post_grad: torch.Tensor):
        arcs = ctx.fsas.arcs
        dev = arcs.device
        dtype = torch.float64 if ctx.use_double_scores else torch.float32
        arc_scores_grad = arc_post_grad.detach().to(dtype).contiguous().clone()
        forward_grad = torch.zeros(arcs.num_states, dtype=dtype, device=dev)
        backward_grad = torch.zeros(arcs.num_states, dtype=dtype, device=dev)
        view, keep = arcs.view(want_incoming=True)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.k2b200_fsa_arc_post_backprop(
                ctypes.byref(view), int(ctx.use_double_scores), _lib.ptr(arc_scores_grad),
                _lib.ptr(forward_grad), _lib.ptr(backward_grad), _lib.stream_of(dev)))
        del keep
        return None, None, None, arc_scores_grad, forward_grad, backward_grad


class _IntersectDenseFunction(torch.autograd.Function):

    @staticmethod
    def forward(ctx, a_fsas: Fsa, b_fsas: DenseFsaVec, out_fsa: List[Fsa], output_beam: float,
                max_states: int, max_arcs: int, unused_scores_a: torch.Tensor,
                unused_scores_b: torch.Tensor, a_to_b_map: Optional[torch.Tensor] = None,
                seqframe_idx_name: Optional[str] = None,
                frame_idx_name: Optional[str] = None) -> torch.Tensor:
        assert len(out_fsa) == 1
        ragged_arc, arc_map_a, arc_map_b = _intersect_dense_arcs(
            a_fsas.arcs, b_fsas, a_to_b_map, output_beam, max_states, max_arcs, VITERBI_MODE)
        # the lattice is valid by construction; its property bits are computed on
        # first use rather than with a host round trip on every call
        out_fsa[0] = Fsa(ragged_arc, _check=False)

        for name, a_value in a_fsas.named_tensor_attr(include_scores=False):
            if name == 'labels':
                continue
            setattr(out_fsa[0], name, index_select(a_value, arc_map_a))
        for name, a_value in a_fsas.named_non_tensor_attr():
            setattr(out_fsa[0], name, a_value)

        ctx.arc_map_a = arc_map_a
        ctx.arc_map_b = arc_map_b
        ctx.save_for_backward(unused_scores_a, unused_scores_b)

        seqframe_idx = None
        if frame_idx_name is not None:
            num_cols = b_fsas.scores.shape[1]
            seqframe_idx = torch.div(arc_map_b, num_cols, rounding_mode="floor")
            row_ids = torch.repeat_interleave(
                torch.arange(b_fsas.dim0(), dtype=torch.int32, device=arc_map_b.device),
                torch.from_numpy(np.diff(b_fsas.h_row_splits)).to(arc_map_b.device))
            fsa_idx0 = row_ids[seqframe_idx.long()]
            frame_idx = seqframe_idx - b_fsas.row_splits[fsa_idx0.long()]
            assert not hasattr(out_fsa[0], frame_idx_name)
            setattr(out_fsa[0], frame_idx_name, frame_idx.to(torch.int32))
        if seqframe_idx_name is not None:
            if seqframe_idx is None:
                num_cols = b_fsas.scores.shape[1]
                seqframe_idx = torch.div(arc_map_b, num_cols, rounding_mode="floor")
            assert not hasattr(out_fsa[0], seqframe_idx_name)
            setattr(out_fsa[0], seqframe_idx_name, seqframe_idx)

        return out_fsa[0].scores

    @staticmethod
    def backward(ctx, out_fsa_grad: torch.Tensor):
        a_scores, b_scores = ctx.saved_tensors
        arc_map_a = ctx.arc_map_a
        arc_map_b = ctx.arc_map_b
        grad_a = torch.zeros(a_scores.size(0), dtype=torch.float32, device=a_scores.device,
                             requires_grad=False)
        grad_b = torch.zeros(*b_scores.shape, dtype=torch.float32, device=b_scores.device,
                             requires_grad=False).contiguous()
        _index_add(arc_map_a, out_fsa_grad, grad_a)
        _index_add(arc_map_b, out_fsa_grad, grad_b.view(-1))
        return (None, None, None, None, None, None, grad_a, grad_b, None, None, None)


def intersect_dense(a_fsas: Fsa, b_fsas: DenseFsaVec, output_beam: float,
                    max_states: int = 15000000, max_arcs: int = 1073741824,
                    a_to_b_map: Optional[torch.Tensor] = None,
                    seqframe_idx_name: Optional[str] = None,
                    frame_idx_name: Optional[str] = None) -> Fsa:
    """Intersect graphs with a DenseFsaVec; exact forward-backward pruning to
    `output_beam` (k2/python/k2/autograd.py:751-824).  `a_fsas` has one graph
    per entry of `a_to_b_map` (default: one per sequence of `b_fsas`), whose
    sequences must be sorted by decreasing length."""
    out_fsa = [0]
    _IntersectDenseFunction.apply(a_fsas, b_fsas, out_fsa, output_beam, max_states, max_arcs,
                                  a_fsas.scores, b_fsas.scores, a_to_b_map, seqframe_idx_name,
                                  frame_idx_name)
    return out_fsa[0]


# Arena capacity that `intersect_dense_pruned` starts from: arcs alive at one time over
# all sequences, and the most one sequence gets of it (the call is repeated with four
# times as much per sequence while some sequence overflows its share).
PRUNED_ARCS_TOTAL = 1 << 26
PRUNED_ARCS_PER_SEQ = 1 << 21
PRUNED_ARCS_MIN = 1 << 16
_pruned_capacity = {}  # (device, num_seqs) -> capacity that the last call needed


def _intersect_dense_pruned_arcs(a: RaggedArc, b: DenseFsaVec, search_beam: float,
                                 output_beam: float, min_active_states: int,
                                 max_active_states: int, allow_partial: bool,
                                 team_ctas: int = 0):
    """The `_k2.intersect_dense_pruned` call (k2/python/csrc/torch/fsa_algo.cu:200-222):
    returns (RaggedArc lattice, arc_map_a, arc_map_b).  `team_ctas` (0 = automatic) is
    the number of CTAs that share a sequence; it changes the speed only."""
    dev = b.scores.device
    _lib.require_cuda(a.values(), "a_fsas")
    _lib.require_cuda(b.scores, "b_fsas.scores")
    if a.device != dev:
        raise RuntimeError("a_fsas and b_fsas must be on the same device")
    scores = b.scores.detach()
    assert scores.is_contiguous() and scores.dtype == torch.float32
    h_brs = np.ascontiguousarray(b.h_row_splits, dtype=np.int32)
    num_seqs = h_brs.shape[0] - 1
    cap_a = max(PRUNED_ARCS_MIN, min(PRUNED_ARCS_PER_SEQ, PRUNED_ARCS_TOTAL // max(num_seqs, 1)))
    cap_a = max(cap_a, _pruned_capacity.get((str(dev), num_seqs), 0))
    stream = _lib.stream_of(dev)
    i32 = dict(dtype=torch.int32, device=dev)
    while True:
        args = _lib.PrunedArgs(
            num_fsas=a.num_fsas, num_states=a.num_states, num_arcs=a.num_elements(),
            a_row_splits1=_lib.ptr(a._row_splits1), a_row_splits2=_lib.ptr(a._row_splits2),
            a_arcs=_lib.ptr(a.values()), scores=_lib.ptr(scores), rows=scores.shape[0],
            cols=scores.shape[1], num_seqs=num_seqs, b_row_splits=_lib.ptr(b.row_splits),
            h_b_row_splits=h_brs.ctypes.data, search_beam=search_beam, output_beam=output_beam,
            min_active_states=min_active_states, max_active_states=max_active_states,
            allow_partial=int(bool(allow_partial)), max_states_per_seq=max(cap_a // 2, 2),
            max_arcs_per_seq=cap_a, team_ctas=team_ctas)
        nbytes, levels = ctypes.c_size_t(), ctypes.c_int64()
        _lib.check(_lib.lib.k2b200_intersect_dense_pruned_workspace_bytes(
            ctypes.byref(args), ctypes.byref(nbytes), ctypes.byref(levels)))
        ws = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)
        ns, na, full = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.k2b200_intersect_dense_pruned_search(
                ctypes.byref(args), _lib.ptr(ws), nbytes.value, stream, ctypes.byref(ns),
                ctypes.byref(na), ctypes.byref(full)))
        if not full.value:
            _pruned_capacity[(str(dev), num_seqs)] = cap_a
            break
        del ws
        cap_a *= 4
        if cap_a >= 1 << 30:
            raise RuntimeError("intersect_dense_pruned: more than 2^30 arcs alive in one sequence")
    ns, na = ns.value, na.value
    with torch.cuda.device(dev):
        row_splits1 = torch.empty(num_seqs + 1, **i32)
        row_ids1 = torch.empty(ns + 1, **i32)
        row_splits2 = torch.empty(ns + 1, **i32)
        row_ids2 = torch.empty(na + 1, **i32)
        values = torch.empty((na + 1, 4), **i32)
        arc_map_a = torch.empty(na + 1, **i32)
        arc_map_b = torch.empty(na + 1, **i32)
        level_offsets = torch.empty(num_seqs + 1, **i32)
        level_splits = torch.empty(levels.value + 1, **i32)
        out = _lib.LatticeOut(
            row_splits1=_lib.ptr(row_splits1), row_ids1=_lib.ptr(row_ids1),
            row_splits2=_lib.ptr(row_splits2), row_ids2=_lib.ptr(row_ids2),
            arcs=_lib.ptr(values), arc_map_a=_lib.ptr(arc_map_a), arc_map_b=_lib.ptr(arc_map_b),
            level_offsets=_lib.ptr(level_offsets), level_splits=_lib.ptr(level_splits))
        _lib.check(_lib.lib.k2b200_intersect_dense_pruned_emit(
            ctypes.byref(args), _lib.ptr(ws), nbytes.value, stream, ctypes.byref(out)))
    lattice = RaggedArc(values[:na], row_splits1, row_splits2, row_ids1[:ns], row_ids2[:na])
    lattice._levels = (level_offsets, level_splits)
    return lattice, arc_map_a[:na], arc_map_b[:na]


class _IntersectDensePrunedFunction(torch.autograd.Function):
    """Autograd contract of k2/python/k2/autograd.py:350-510."""

    @staticmethod
    def forward(ctx, a_fsas: Fsa, b_fsas: DenseFsaVec, out_fsa: List[Fsa], search_beam: float,
                output_beam: float, min_active_states: int, max_active_states: int,
                allow_partial: bool, unused_scores_a: torch.Tensor,
                unused_scores_b: torch.Tensor, seqframe_idx_name: Optional[str] = None,
                frame_idx_name: Optional[str] = None) -> torch.Tensor:
        assert len(out_fsa) == 1
        ragged_arc, arc_map_a, arc_map_b = _intersect_dense_pruned_arcs(
            a_fsas.arcs, b_fsas, search_beam, output_beam, min_active_states,
            max_active_states, allow_partial)
        out_fsa[0] = Fsa(ragged_arc, _check=False)
        for name, a_value in a_fsas.named_tensor_attr(include_scores=False):
            if name == 'labels':
                continue
            setattr(out_fsa[0], name, index_select(a_value, arc_map_a))
        for name, a_value in a_fsas.named_non_tensor_attr():
            setattr(out_fsa[0], name, a_value)
        ctx.arc_map_a = arc_map_a
        ctx.arc_map_b = arc_map_b
        ctx.save_for_backward(unused_scores_a, unused_scores_b)
        seqframe_idx = None
        if frame_idx_name is not None or seqframe_idx_name is not None:
            seqframe_idx = torch.div(arc_map_b, b_fsas.scores.shape[1], rounding_mode="floor")
        if frame_idx_name is not None:
            row_ids = torch.repeat_interleave(
                torch.arange(b_fsas.dim0(), dtype=torch.int32, device=arc_map_b.device),
                torch.from_numpy(np.diff(b_fsas.h_row_splits)).to(arc_map_b.device))
            fsa_idx0 = row_ids[seqframe_idx.long()]
            frame_idx = seqframe_idx - b_fsas.row_splits[fsa_idx0.long()]
            assert not hasattr(out_fsa[0], frame_idx_name)
            setattr(out_fsa[0], frame_idx_name, frame_idx.to(torch.int32))
        if seqframe_idx_name is not None:
            assert not hasattr(out_fsa[0], seqframe_idx_name)
            setattr(out_fsa[0], seqframe_idx_name, seqframe_idx)
        return out_fsa[0].scores

    @staticmethod
    def backward(ctx, out_fsa_grad: torch.Tensor):
        a_scores, b_scores = ctx.saved_tensors
        grad_a = torch.zeros(a_scores.size(0), dtype=torch.float32, device=a_scores.device)
        grad_b = torch.zeros(*b_scores.shape, dtype=torch.float32,
                             device=b_scores.device).contiguous()
        _index_add(ctx.arc_map_a, out_fsa_grad, grad_a)  # -1 (allow_partial arcs) is skipped
        _index_add(ctx.arc_map_b, out_fsa_grad, grad_b.view(-1))
        return (None, None, None, None, None, None, None, None, grad_a, grad_b, None, None)


def intersect_dense_pruned(a_fsas: Fsa, b_fsas: DenseFsaVec, search_beam: float,
                           output_beam: float, min_active_states: int, max_active_states: int,
                           seqframe_idx_name: Optional[str] = None,
                           frame_idx_name: Optional[str] = None,
                           allow_partial: bool = False) -> Fsa:
    """Pruned intersection for decoding (k2/python/k2/autograd.py:667-746): `a_fsas` holds
    one arc-sorted graph per sequence of `b_fsas`, or a single graph shared by all."""
    out_fsa = [0]
    _IntersectDensePrunedFunction.apply(a_fsas, b_fsas, out_fsa, search_beam, output_beam,
                                        min_active_states, max_active_states, allow_partial,
                                        a_fsas.scores, b_fsas.scores, seqframe_idx_name,
                                        frame_idx_name)
    return out_fsa[0]


class _DenseTotScoresFunction(torch.autograd.Function):
    """tot_scores = log-semiring total score of intersect_dense(a_fsas, b_fsas) per
    graph, with gradients to the graph scores and the dense scores, computed on the
    (frame, state) grid without building the lattice.  Same pruning as
    `intersect_dense` followed by `get_tot_scores(log_semiring=True)`."""

    @staticmethod
    def forward(ctx, a_fsas: Fsa, b_fsas: DenseFsaVec, output_beam: float, max_states: int,
                max_arcs: int, use_double_scores: bool, a_to_b_map: Optional[torch.Tensor],
                unused_scores_a: torch.Tensor, unused_scores_b: torch.Tensor) -> torch.Tensor:
        args, keep, dev, _ = _make_intersect_args(a_fsas.arcs, b_fsas, a_to_b_map, output_beam,
                                                  max_states, max_arcs, VITERBI_MODE)
        nbytes = ctypes.c_size_t()
        _lib.check(_lib.lib.k2b200_dense_loss_workspace_bytes(ctypes.byref(args),
                                                               ctypes.byref(nbytes)))
        lease = _lib.workspace(nbytes.value, dev)
        ws = lease.tensor
        tot = torch.empty(a_fsas.arcs.num_fsas, dtype=torch.float64, device=dev)
        beam = ctypes.c_float()
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.k2b200_dense_loss_forward(
                ctypes.byref(args), _lib.ptr(ws), nbytes.value, _lib.stream_of(dev),
                _lib.ptr(tot), ctypes.byref(beam)))
        ctx.args, ctx.keep, ctx.ws, ctx.ws_bytes = args, (keep, a_fsas.arcs), ws, nbytes.value
        ctx.lease = lease
        ctx.dev = dev
        ctx.shape_a = unused_scores_a.shape
        ctx.shape_b = unused_scores_b.shape
        # when the last argument is the log-prob tensor the DenseFsaVec was made from
        # (not its score matrix), the backward writes the gradient in that layout
        ctx.lp_row = None
        src = b_fsas._source
        if src is not None and unused_scores_b is src[0]:
            key = None if a_to_b_map is None else tuple(keep[2].tolist())
            if key not in b_fsas._source_rows:
                rows = src[1] if key is None else src[1][keep[2]]
                b_fsas._source_rows[key] = _lib.upload_i32(rows, dev)
            ctx.lp_row = b_fsas._source_rows[key]
        ctx.output_beam_used = beam.value
        return tot if use_double_scores else tot.to(torch.float32)

    @staticmethod
    def backward(ctx, tot_grad: torch.Tensor):
        dev = ctx.dev
        if tot_grad.dtype != torch.float64:
            tot_grad = tot_grad.to(torch.float64)
        stride = tot_grad.stride(0) if tot_grad.numel() > 0 else 0
        # without a gradient for the graph scores the library may take the dense gradient
        # from state posteriors (graphs in which a state has one label)
        grad_a = None
        if ctx.needs_input_grad[7]:
            grad_a = torch.zeros(ctx.shape_a, dtype=torch.float32, device=dev)
        grad_b = torch.zeros(ctx.shape_b, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            if ctx.lp_row is None:
                _lib.check(_lib.lib.k2b200_dense_loss_backward(
                    ctypes.byref(ctx.args), _lib.ptr(ctx.ws), ctx.ws_bytes, _lib.ptr(tot_grad),
                    stride, _lib.ptr(grad_a), _lib.ptr(grad_b), _lib.stream_of(dev)))
            else:
                _lib.check(_lib.lib.k2b200_dense_loss_backward_log_probs(
                    ctypes.byref(ctx.args), _lib.ptr(ctx.ws), ctx.ws_bytes, _lib.ptr(tot_grad),
                    stride, _lib.ptr(grad_a), _lib.ptr(grad_b), _lib.ptr(ctx.lp_row),
                    ctx.shape_b[-1], _lib.stream_of(dev)))
        return None, None, None, None, None, None, None, grad_a, grad_b


# ---------------------------------------------------------------------------
# Band graphs (CTC): the lattice-free loss reads the log-probs in place
# ---------------------------------------------------------------------------
# When True, every band-path forward is followed by a host wait and a look at the
# status word of the kernels; a bounded wait that gave up then sends the call to the
# general lattice-free path instead of returning NaN totals.
BAND_VERIFY = False
_band_state = {"status": 0}  # status word of the last verified band-path forward


def _band_loss_args(a_fsas: Fsa, b_fsas: DenseFsaVec, a_to_b_map: Optional[torch.Tensor],
                    output_beam: float, max_states: int, max_arcs: int):
    """(args, keep-alive objects, host map) of the k2b200_band_loss_* entry points, or
    None when they do not apply: `b_fsas` must come from a float32 CUDA log-prob tensor
    with 16-byte aligned rows and the graphs must be band graphs of at most 512 states."""
    src = b_fsas._source
    a = a_fsas.arcs
    cached = b_fsas._band_args
    version = (a.values()._version, None if a_to_b_map is None else a_to_b_map._version)
    if (cached is not None and cached[0] is a and cached[1] is a_to_b_map
            and cached[3] == version):
        # same graphs, same sequences: only the limits can differ
        if cached[2] is None:
            return None
        args0, keep, h_map = cached[2]
        args = _lib.BandLossArgs.from_buffer_copy(args0)
        args.ws_bytes = args0.ws_bytes
        args.zero_fill, args.zero_fill_bytes = None, 0
        args.output_beam = float(output_beam)
        args.max_states = int(min(max_states, 2**31 - 1))
        args.max_arcs = int(min(max_arcs, 2**31 - 1))
        return args, keep, h_map
    ans = _band_loss_args_uncached(a_fsas, b_fsas, a_to_b_map, output_beam, max_states, max_arcs)
    b_fsas._band_args = (a, a_to_b_map, ans, version)
    return ans


def _band_loss_args_uncached(a_fsas: Fsa, b_fsas: DenseFsaVec,
                             a_to_b_map: Optional[torch.Tensor], output_beam: float,
                             max_states: int, max_arcs: int):
    src = b_fsas._source
    a = a_fsas.arcs
    if src is None or not a.values().is_cuda:
        return None
    lp = src[0]
    if not (lp.is_cuda and lp.dtype == torch.float32 and lp.is_contiguous()
            and lp.device == a.device and lp.shape[-1] % 4 == 0 and lp.data_ptr() % 16 == 0):
        return None
    h_map = None
    if a_to_b_map is not None:
        assert a_to_b_map.ndim == 1 and a_to_b_map.dtype == torch.int32
        h_map = np.ascontiguousarray(a_to_b_map.detach().cpu().numpy(), dtype=np.int32)
        if h_map.shape[0] != a.num_fsas:
            raise RuntimeError(
                f"a_fsas.Dim0() ({a.num_fsas}) != a_to_b_map.Dim() ({h_map.shape[0]})")
        if h_map.size and (h_map.min() < 0 or h_map.max() >= b_fsas.dim0()
                           or np.any(np.diff(h_map) < 0)):
            return None  # the general path reports the error
    elif a.num_fsas != b_fsas.dim0():
        return None
    states, arcs, ok = a.band_tables()
    if not ok:
        return None
    # host arrays of the graphs, kept with the tables (which follow the arc tensor's version)
    host = getattr(a, "_band_host", None)
    if host is None or host[0] is not states:
        h_rs1 = np.ascontiguousarray(a.h_row_splits1, dtype=np.int32)
        host = a._band_host = (states, h_rs1, np.ascontiguousarray(a.h_arc_splits, dtype=np.int32),
                               int(np.diff(h_rs1).max(initial=0)))
    _, h_rs1, h_as, most_states = host
    if most_states > 512:
        return None
    frames = np.diff(b_fsas.h_row_splits) - 1
    first = src[1]
    if h_map is not None:
        frames, first = frames[h_map], first[h_map]
    frames = np.ascontiguousarray(frames, dtype=np.int32)
    first = np.ascontiguousarray(first, dtype=np.int32)
    args = _lib.BandLossArgs(
        num_fsas=a.num_fsas, num_states=a.num_states, a_row_splits2=_lib.ptr(a._row_splits2),
        h_a_row_splits1=h_rs1.ctypes.data, h_a_arc_splits=h_as.ctypes.data,
        band_states=_lib.ptr(states), band_arcs=_lib.ptr(arcs), log_probs=_lib.ptr(lp),
        log_prob_rows=lp.numel() // lp.shape[-1], num_classes=lp.shape[-1],
        h_first_row=first.ctypes.data, h_frames=frames.ctypes.data,
        output_beam=float(output_beam), max_states=int(min(max_states, 2**31 - 1)),
        max_arcs=int(min(max_arcs, 2**31 - 1)))
    ok = ctypes.c_int32()
    _lib.check(_lib.lib.k2b200_band_loss_supported(ctypes.byref(args), ctypes.byref(ok)))
    if not ok.value:
        return None
    nbytes = ctypes.c_size_t()
    _lib.check(_lib.lib.k2b200_band_loss_workspace_bytes(ctypes.byref(args), ctypes.byref(nbytes)))
    args.ws_bytes = nbytes.value  # a Python attribute beside the C fields: depends on the sizes only
    return args, (h_rs1, h_as, frames, first, states, arcs, lp, a), h_map


class _BandTotScoresFunction(torch.autograd.Function):
    """`_DenseTotScoresFunction` for band graphs (`k2b200_band_loss_*`): same values,
    the dense scores read straight from the log-prob tensor."""

    @staticmethod
    def forward(ctx, a_fsas: Fsa, b_fsas: DenseFsaVec, band, use_double_scores: bool,
                unused_scores_a: torch.Tensor, unused_scores_b: torch.Tensor) -> torch.Tensor:
        args, keep, h_map = band
        dev = a_fsas.arcs.device
        nbytes = ctypes.c_size_t(args.ws_bytes)
        lease = _lib.workspace(nbytes.value, dev)
        ws = lease.tensor
        tot = torch.empty(a_fsas.arcs.num_fsas, dtype=torch.float64, device=dev)
        beam = ctypes.c_float()
        # the gradient of the log-probs, when the backward will want it: the forward call
        # clears it beside its recursions, so the backward has no zero-fill of its own
        ctx.grad_b = None
        args.zero_fill, args.zero_fill_bytes = None, 0
        if ctx.needs_input_grad[5] and unused_scores_b is b_fsas._source[0]:
            ctx.grad_b = torch.empty(unused_scores_b.shape, dtype=torch.float32, device=dev)
            args.zero_fill = ctx.grad_b.data_ptr()
            args.zero_fill_bytes = ctx.grad_b.numel() * 4
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.k2b200_band_loss_forward(
                ctypes.byref(args), _lib.ptr(ws), nbytes.value, _lib.stream_of(dev),
                _lib.ptr(tot), ctypes.byref(beam)))
            _band_state["status"] = 0
            if BAND_VERIFY:
                status = ctypes.c_int32()
                _lib.check(_lib.lib.k2b200_band_loss_status(
                    ctypes.byref(args), _lib.ptr(ws), nbytes.value, _lib.stream_of(dev),
                    ctypes.byref(status)))
                _band_state["status"] = status.value
        ctx.args, ctx.keep, ctx.ws, ctx.ws_bytes, ctx.dev = args, keep, ws, nbytes.value, dev
        ctx.lease = lease
        ctx.shape_a, ctx.shape_b = unused_scores_a.shape, unused_scores_b.shape
        src = b_fsas._source
        if unused_scores_b is src[0]:  # gradient in the layout of the log-probs
            ctx.grad_rows = None       # the rows the forward read
            ctx.grad_pitch, ctx.grad_col_off = int(args.num_classes), 0
        else:                          # in the layout of the score matrix
            rows = b_fsas.h_row_splits[:-1] if h_map is None else b_fsas.h_row_splits[h_map]
            ctx.grad_rows = _lib.upload_i32(rows, dev)
            ctx.grad_pitch, ctx.grad_col_off = int(args.num_classes) + 1, 1
        ctx.output_beam_used = beam.value
        return tot if use_double_scores else tot.to(torch.float32)

    @staticmethod
    def backward(ctx, tot_grad: torch.Tensor):
        dev = ctx.dev
        if tot_grad.dtype != torch.float64:
            tot_grad = tot_grad.to(torch.float64)
        stride = tot_grad.stride(0) if tot_grad.numel() > 0 else 0
        grad_a = None
        if ctx.needs_input_grad[4]:
            grad_a = torch.zeros(ctx.shape_a, dtype=torch.float32, device=dev)
        grad_b, ctx.grad_b = ctx.grad_b, None  # cleared by the forward call; used once
        if grad_b is None:
            grad_b = torch.zeros(ctx.shape_b, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.k2b200_band_loss_backward(
                ctypes.byref(ctx.args), _lib.ptr(ctx.ws), ctx.ws_bytes, _lib.ptr(tot_grad),
                stride, _lib.ptr(grad_a), _lib.ptr(grad_b), _lib.ptr(ctx.grad_rows),
                ctx.grad_pitch, ctx.grad_col_off, _lib.stream_of(dev)))
        return None, None, None, None, grad_a, grad_b


class _BandNegSumFunction(torch.autograd.Function):
    """`-tot_scores.sum(dtype=torch.float32)` over `_BandTotScoresFunction` as ONE node of
    the autograd graph (the `reduction="sum"` of k2/python/k2/ctc_loss.py:72-84 on the band
    path): the same kernels, two nodes less to build in the forward and to run in the
    backward, on the thread that feeds the GPU."""

    @staticmethod
    def forward(ctx, a_fsas: Fsa, b_fsas: DenseFsaVec, band, use_double_scores: bool,
                unused_scores_a: torch.Tensor, unused_scores_b: torch.Tensor) -> torch.Tensor:
        tot = _BandTotScoresFunction.forward(ctx, a_fsas, b_fsas, band, use_double_scores,
                                             unused_scores_a, unused_scores_b)
        ctx.tot_shape = tot.shape
        # (-1 * tot_scores).to(float32).sum() of the reference: the reduction casts every
        # element before adding, and negation commutes with rounding, so the bits are the same
        return -tot.sum(dtype=torch.float32)

    @staticmethod
    def backward(ctx, loss_grad: torch.Tensor):
        tot_grad = (-loss_grad).to(torch.float64).expand(ctx.tot_shape)  # stride 0
        return _BandTotScoresFunction.backward(ctx, tot_grad)


def band_ctc_loss_sum(a_fsas: Fsa, b_fsas: DenseFsaVec, output_beam: float,
                      use_double_scores: bool = True) -> Optional[torch.Tensor]:
    """`-intersect_dense_tot_scores(...).sum(dtype=torch.float32)` on the band kernels, or
    None when they do not take these inputs."""
    args = _band_loss_args(a_fsas, b_fsas, None, output_beam, 15000000, 1073741824)
    if args is None or BAND_VERIFY:
        return None
    src = b_fsas._source
    from_log_probs = src[0].requires_grad and src[0].dtype == torch.float32
    scores_b = src[0] if (from_log_probs or b_fsas._scores is None) else b_fsas.scores
    return _BandNegSumFunction.apply(a_fsas, b_fsas, args, use_double_scores, a_fsas.scores,
                                     scores_b)


def band_loss_supported(a_fsas: Fsa, b_fsas: DenseFsaVec,
                        a_to_b_map: Optional[torch.Tensor] = None) -> bool:
    """Can `intersect_dense_tot_scores` take the band-graph kernels for these inputs?"""
    return _band_loss_args(a_fsas, b_fsas, a_to_b_map, 1.0, 1, 1) is not None


def dense_loss_supported(a_fsas: Fsa, b_fsas: DenseFsaVec,
                         a_to_b_map: Optional[torch.Tensor] = None) -> bool:
    """Can `intersect_dense_tot_scores` handle these inputs (CUDA tensors, graphs
    small enough for the shared-memory recursion)?"""
    if not (a_fsas.arcs.values().is_cuda and b_fsas.device.type == "cuda"):
        return False
    if band_loss_supported(a_fsas, b_fsas, a_to_b_map):
        return True
    args, _keep, _, _ = _make_intersect_args(a_fsas.arcs, b_fsas, a_to_b_map, 1.0, 1, 1)
    ok = ctypes.c_int32()
    _lib.check(_lib.lib.k2b200_dense_loss_supported(ctypes.byref(args), ctypes.byref(ok)))
    return bool(ok.value)


def intersect_dense_tot_scores(a_fsas: Fsa, b_fsas: DenseFsaVec, output_beam: float,
                               max_states: int = 15000000, max_arcs: int = 1073741824,
                               a_to_b_map: Optional[torch.Tensor] = None,
                               use_double_scores: bool = True,
                               band: bool = True) -> torch.Tensor:
    """`intersect_dense(a_fsas, b_fsas, output_beam, ...).get_tot_scores(
    log_semiring=True, use_double_scores=...)` in one step (the composition
    k2/python/k2/ctc_loss.py:86-140 makes), differentiable w.r.t. `a_fsas.scores`
    and `b_fsas.scores`.  The lattice is not built.  When `b_fsas` was made from a
    log-prob tensor that takes part in autograd, the gradient goes to that tensor
    directly rather than through the score matrix and the adjoint of its layout.
    Band graphs (CTC) take kernels of their own that read the log-probs in place
    (`band=False` keeps them on the general kernels)."""
    src = b_fsas._source
    from_log_probs = src is not None and src[0].requires_grad and src[0].dtype == torch.float32
    args = _band_loss_args(a_fsas, b_fsas, a_to_b_map, output_beam, max_states,
                           max_arcs) if band else None
    if args is not None:
        # without autograd on the log-probs the gradient (if any) is that of the score
        # matrix, which then exists anyway
        scores_b = src[0] if (from_log_probs or b_fsas._scores is None) else b_fsas.scores
        tot = _BandTotScoresFunction.apply(a_fsas, b_fsas, args, use_double_scores,
                                           a_fsas.scores, scores_b)
        if not (BAND_VERIFY and _band_state["status"] & 2):
            return tot
        # a bounded wait of the band kernels gave up: the general kernels take the call
    scores_b = src[0] if from_log_probs else b_fsas.scores
    return _DenseTotScoresFunction.apply(a_fsas, b_fsas, output_beam, max_states, max_arcs,
                                         use_double_scores, a_to_b_map, a_fsas.scores,
                                         scores_b)

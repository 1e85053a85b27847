"""`Fsa`: the host-side mirror of `k2.Fsa` (k2/python/k2/fsa.py) for the dense
intersection / total-score path, backed by CUDA kernels through the C-ABI.

Kept from the reference: the constructor signature, the `arcs` / `scores` /
`labels` / `aux_labels` attributes and arbitrary per-arc tensor attributes, the
score cache and its invalidation when `scores` is re-assigned (fsa.py:242-273,
:417-422), `get_tot_scores` / `get_forward_scores` / `get_backward_scores` /
`get_arc_post` / `_get_entering_arcs`, `properties`, `from_str`, `to`,
`requires_grad_`, `shape`, `num_arcs`.  Not mirrored (outside this path):
ragged attributes, symbol tables, drawing, (de)serialisation, indexing helpers.
"""
import ctypes
import re
from typing import Any, Dict, Iterator, List, Optional, Tuple, Union

import numpy as np
import torch

from . import _lib
from .ragged import RaggedArc
from .ragged_tensor import RaggedTensor
from .ragged_tensor import cat as _ragged_cat

# k2/csrc/fsa.h:75-101
VALID = 0x01
NONEMPTY = 0x02
TOPSORTED = 0x04
TOPSORTED_AND_ACYCLIC = 0x08
ARC_SORTED = 0x10
ARC_SORTED_AND_DETERMINISTIC = 0x20
EPSILON_FREE = 0x40
ACCESSIBLE = 0x80
COACCESSIBLE = 0x0100
ALL = 0x01FF


def _fsa_from_tensor(arcs: torch.Tensor) -> RaggedArc:
    """A single FSA from an [A,4] int32 tensor whose rows are sorted by source
    state (k2::FsaFromTensor, k2/csrc/fsa.cu:340-400): the number of states is
    the largest state mentioned plus one."""
    assert arcs.dtype == torch.int32 and arcs.ndim == 2 and arcs.shape[1] == 4
    host = arcs.detach().cpu().numpy()
    if host.shape[0] == 0:
        num_states = 0
    else:
        num_states = int(max(host[:, 0].max(), host[:, 1].max())) + 1
    src = host[:, 0]
    if np.any(np.diff(src) < 0):
        raise ValueError("arcs must be sorted by source state")
    rs2 = np.zeros(num_states + 1, dtype=np.int32)
    np.add.at(rs2, src + 1, 1)
    rs2 = np.cumsum(rs2).astype(np.int32)
    rs1 = np.array([0, num_states], dtype=np.int32)
    dev = arcs.device
    return RaggedArc(arcs.contiguous(), torch.from_numpy(rs1).to(dev),
                     torch.from_numpy(rs2).to(dev), single=True, h_row_splits1=rs1,
                     h_arc_splits=np.array([0, host.shape[0]], dtype=np.int32))


class Fsa(object):

    def __init__(self, arcs: Union[torch.Tensor, RaggedArc],
                 aux_labels: Optional[torch.Tensor] = None, properties=None,
                 _check: bool = True) -> None:
        if isinstance(arcs, torch.Tensor):
            arcs = _fsa_from_tensor(arcs)
        assert isinstance(arcs, RaggedArc)
        self.__dict__['arcs'] = arcs
        self.__dict__['_properties'] = properties
        for name in ['_tensor_attr', '_non_tensor_attr', '_cache']:
            self.__dict__[name] = dict()
        values = arcs.values()
        self._tensor_attr['scores'] = values[:, 3].view(torch.float32)
        self._tensor_attr['labels'] = values[:, 2]
        if aux_labels is not None:
            self.aux_labels = aux_labels.to(torch.int32)
        if _check and properties is None:
            _ = self.properties  # validity check, as the reference does eagerly

    # ------------------------------------------------------------------ attributes
    def __setattr__(self, name: str, value: Any) -> None:
        assert name not in ('_tensor_attr', '_non_tensor_attr', 'arcs', '_cache', '_properties',
                            'properties')
        if isinstance(value, RaggedTensor):
            # one list per arc, e.g. ragged aux_labels (k2/python/k2/fsa.py:389-396)
            assert value.dim0 == self.arcs.values().shape[0]
            assert value.device == self.device
            assert name not in ('labels', 'scores')
            self._tensor_attr[name] = value
        elif isinstance(value, torch.Tensor):
            assert value.shape[0] == self.arcs.values().shape[0]
            assert value.device == self.device
            if name == 'labels':
                assert value.dtype == torch.int32
                self.arcs.values()[:, 2] = value
                self.__dict__['_properties'] = None
                self.arcs._incoming = None
                return
            self._tensor_attr[name] = value
            if name == 'scores':
                assert value.dtype == torch.float32
                # the float bit patterns are stored in the int32 arc tensor
                self.arcs.values()[:, 3] = value.detach().view(torch.int32)
                self.arcs._incoming = None  # it carries a copy of the scores
                self._invalidate_cache_()
        else:
            self._non_tensor_attr[name] = value

    def __getattr__(self, name: str) -> Any:
        if name in self._tensor_attr:
            return self._tensor_attr[name]
        if name in self._non_tensor_attr:
            return self._non_tensor_attr[name]
        if name in self._cache:
            return self._cache[name]
        if name == 'grad':
            return self.scores.grad
        raise AttributeError(f'Unknown attribute {name}')

    def __delattr__(self, name: str) -> None:
        assert name not in ('arcs', 'scores', 'labels', 'properties', '_cache', '_properties',
                            '_tensor_attr', '_non_tensor_attr')
        if name in self._tensor_attr:
            del self._tensor_attr[name]
        elif name in self._non_tensor_attr:
            del self._non_tensor_attr[name]
        elif name in self._cache:
            del self._cache[name]
        else:
            raise AttributeError(f'No such attribute in Fsa: {name}')

    def _invalidate_cache_(self, scores_only: bool = True) -> None:
        if scores_only is False:
            self.__dict__['_cache'] = dict()
            return
        pattern = re.compile(r'score|arc_cdf|arc_post')
        to_remove = [k for k in self._cache if pattern.search(k)]
        if 'entering_arcs' in self._cache:
            to_remove.append('entering_arcs')
        for k in to_remove:
            del self._cache[k]

    def named_tensor_attr(self, include_scores: bool = True) -> Iterator[Tuple[str, Any]]:
        if include_scores:
            for name, value in self._tensor_attr.items():
                yield name, value
        else:
            for name, value in self._tensor_attr.items():
                if name != 'scores':
                    yield name, value

    def named_non_tensor_attr(self) -> Iterator[Tuple[str, Any]]:
        for name, value in self._non_tensor_attr.items():
            yield name, value

    # ------------------------------------------------------------------ basics
    @property
    def device(self) -> torch.device:
        return self.arcs.device

    @property
    def num_arcs(self) -> int:
        return self.arcs.num_elements()

    @property
    def shape(self) -> Tuple[int, ...]:
        if self.arcs.num_axes() == 2:
            return (self.arcs.dim0(), None)
        return (self.arcs.dim0(), None, None)

    @property
    def requires_grad(self) -> bool:
        return self.scores.requires_grad

    def requires_grad_(self, requires_grad: bool) -> 'Fsa':
        self.scores.requires_grad_(requires_grad)
        return self

    def to(self, device: Union[str, torch.device]) -> 'Fsa':
        device = torch.device(device)
        if device == self.device:
            return self
        ans = Fsa(self.arcs.to(device), properties=self.__dict__['_properties'], _check=False)
        for name, value in self.named_tensor_attr(include_scores=False):
            if name != 'labels':
                setattr(ans, name, value.to(device))
        for name, value in self.named_non_tensor_attr():
            setattr(ans, name, value)
        return ans

    def clone(self) -> 'Fsa':
        ans = Fsa(self.arcs.clone(), properties=self.__dict__['_properties'], _check=False)
        for name, value in self.named_tensor_attr(include_scores=False):
            if name != 'labels':
                setattr(ans, name, value.clone())
        for name, value in self.named_non_tensor_attr():
            setattr(ans, name, value)
        return ans

    @property
    def properties(self) -> int:
        properties = self.__dict__.get('_properties', None)
        if properties is not None:
            return properties
        properties = _basic_properties(self.arcs)
        self.__dict__['_properties'] = properties
        if properties & VALID != 1:
            raise ValueError(f'Fsa is not valid, properties are: {properties}')
        return properties

    def _arcs_for_algo(self) -> RaggedArc:
        """The 3-axis view every FsaVec algorithm works on."""
        return self.arcs

    # ------------------------------------------------------------------ scores
    def _score_key(self, what: str, use_double_scores: bool, log_semiring: bool) -> str:
        return (f"{what}_{'double' if use_double_scores else 'float'}_"
                f"{'log' if log_semiring else 'tropical'}")

    def _compute_scores(self, use_double_scores: bool, log_semiring: bool, want_forward: bool,
                        want_backward: bool) -> None:
        """One launch computes the requested directions (two independent CTAs per
        FSA), results go to the cache under the reference's key names."""
        arcs = self.arcs
        _lib.require_cuda(arcs.values(), "Fsa")
        dev = arcs.device
        dtype = torch.float64 if use_double_scores else torch.float32
        ns, na, nf = arcs.num_states, arcs.num_elements(), arcs.num_fsas
        fkey = self._score_key('forward_scores', use_double_scores, log_semiring)
        bkey = self._score_key('backward_scores', use_double_scores, log_semiring)
        fwd = torch.empty(ns, dtype=dtype, device=dev) if want_forward else None
        bwd = torch.empty(ns, dtype=dtype, device=dev) if want_backward else None
        entering = None
        if want_forward and not log_semiring:
            entering = torch.empty(ns, dtype=torch.int32, device=dev)
        view, keep = arcs.view(want_incoming=want_forward)
        scratch, nscratch = None, 0
        if log_semiring and arcs._layer_bounds[0]:
            nscratch = _lib.lib.k2b200_fsa_scores_scratch_bytes(ctypes.byref(view))
            scratch = torch.empty(nscratch, dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.k2b200_fsa_scores(
                ctypes.byref(view), int(log_semiring), int(use_double_scores), _lib.ptr(fwd),
                _lib.ptr(bwd), _lib.ptr(entering), _lib.ptr(scratch), nscratch,
                _lib.stream_of(dev)))
        del keep, scratch
        if want_forward:
            self._cache[fkey] = fwd
            if entering is not None:
                self._cache['entering_arcs'] = entering
        if want_backward:
            self._cache[bkey] = bwd

    def _get_forward_scores(self, use_double_scores: bool, log_semiring: bool) -> torch.Tensor:
        key = self._score_key('forward_scores', use_double_scores, log_semiring)
        if key not in self._cache:
            # When the scores take part in autograd the backward scores will be
            # needed for the posteriors: compute both directions in one launch.
            bkey = self._score_key('backward_scores', use_double_scores, log_semiring)
            both = self.scores.requires_grad and bkey not in self._cache
            self._compute_scores(use_double_scores, log_semiring, True, both)
        return self._cache[key]

    def _get_backward_scores(self, use_double_scores: bool, log_semiring: bool) -> torch.Tensor:
        key = self._score_key('backward_scores', use_double_scores, log_semiring)
        if key not in self._cache:
            self._compute_scores(use_double_scores, log_semiring, False, True)
        return self._cache[key]

    def _get_entering_arcs(self, use_double_scores: bool) -> torch.Tensor:
        if 'entering_arcs' not in self._cache:
            key = self._score_key('forward_scores', use_double_scores, False)
            self._cache.pop(key, None)
            self._compute_scores(use_double_scores, False, True, False)
        return self._cache['entering_arcs']

    def _get_tot_scores(self, use_double_scores: bool, log_semiring: bool) -> torch.Tensor:
        key = self._score_key('tot_scores', use_double_scores, log_semiring)
        if key not in self._cache:
            fwd = self._get_forward_scores(use_double_scores, log_semiring)
            arcs = self.arcs
            tot = torch.empty(arcs.num_fsas, dtype=fwd.dtype, device=fwd.device)
            with torch.cuda.device(fwd.device):
                _lib.check(_lib.lib.k2b200_fsa_tot_scores(
                    _lib.ptr(arcs._row_splits1), arcs.num_fsas, int(use_double_scores),
                    _lib.ptr(fwd), _lib.ptr(tot), _lib.stream_of(fwd.device)))
            self._cache[key] = tot
        return self._cache[key]

    def _get_arc_post(self, use_double_scores: bool, log_semiring: bool) -> torch.Tensor:
        key = self._score_key('arc_post', use_double_scores, log_semiring)
        if key not in self._cache:
            fwd = self._get_forward_scores(use_double_scores, log_semiring)
            bwd = self._get_backward_scores(use_double_scores, log_semiring)
            arcs = self.arcs
            post = torch.empty(arcs.num_elements(), dtype=fwd.dtype, device=fwd.device)
            with torch.cuda.device(fwd.device):
                _lib.check(_lib.lib.k2b200_fsa_arc_post(
                    _lib.ptr(arcs._row_splits1), _lib.ptr(arcs.row_ids(1 - arcs.single)),
                    _lib.ptr(arcs.row_ids(2 - arcs.single)), _lib.ptr(arcs.values()),
                    arcs.num_fsas, arcs.num_elements(), int(use_double_scores), _lib.ptr(fwd),
                    _lib.ptr(bwd), _lib.ptr(post), _lib.stream_of(fwd.device)))
            self._cache[key] = post
        return self._cache[key]

    def get_tot_scores(self, use_double_scores: bool, log_semiring: bool) -> torch.Tensor:
        """Total score per FSA (k2/python/k2/fsa.py:676-693); differentiable w.r.t.
        `self.scores`."""
        from .autograd import _GetTotScoresFunction
        return _GetTotScoresFunction.apply(self, log_semiring, use_double_scores, self.scores)

    def get_forward_scores(self, use_double_scores: bool, log_semiring: bool) -> torch.Tensor:
        """Forward score per state (k2/python/k2/fsa.py:626-644); differentiable w.r.t.
        `self.scores`."""
        from .autograd import _GetForwardScoresFunction
        return _GetForwardScoresFunction.apply(self, log_semiring, use_double_scores,
                                               self.scores)

    def get_backward_scores(self, use_double_scores: bool, log_semiring: bool) -> torch.Tensor:
        """Backward score per state (k2/python/k2/fsa.py:734-752); differentiable w.r.t.
        `self.scores`."""
        from .autograd import _GetBackwardScoresFunction
        return _GetBackwardScoresFunction.apply(self, log_semiring, use_double_scores,
                                                self.scores)

    def get_arc_post(self, use_double_scores: bool, log_semiring: bool) -> torch.Tensor:
        """Log posterior per arc (k2/python/k2/fsa.py:790-817); differentiable w.r.t.
        `self.scores`, directly and through the forward and backward scores."""
        from .autograd import _GetArcPostFunction
        forward_scores = self.get_forward_scores(use_double_scores, log_semiring)
        backward_scores = self.get_backward_scores(use_double_scores, log_semiring)
        return _GetArcPostFunction.apply(self, log_semiring, use_double_scores, self.scores,
                                         forward_scores, backward_scores)

    # ------------------------------------------------------------------ text form
    @classmethod
    def from_str(cls, s: str, acceptor: Optional[bool] = None,
                 num_aux_labels: Optional[int] = None,
                 aux_label_names: Optional[List[str]] = None) -> 'Fsa':
        """k2's text format (fsa.py:1226-1330): lines `src dest label [aux...] score`
        and a last line holding the final state."""
        if acceptor is True:
            num_aux_labels = 0
        lines = [ln.split() for ln in s.strip().split('\n') if ln.strip()]
        arc_lines = [ln for ln in lines if len(ln) > 2]
        if num_aux_labels is None:
            num_aux_labels = (len(arc_lines[0]) - 4) if arc_lines else 0
        if aux_label_names is None:
            aux_label_names = ['aux_labels'] if num_aux_labels == 1 else [
                f'aux_labels{i + 1}' if i else 'aux_labels' for i in range(num_aux_labels)]
        rows, aux = [], [[] for _ in range(num_aux_labels)]
        for ln in arc_lines:
            assert len(ln) == 4 + num_aux_labels, f'bad arc line: {ln}'
            src, dest, label = int(ln[0]), int(ln[1]), int(ln[2])
            score = np.float32(float(ln[-1]))
            rows.append((src, dest, label, int(np.array(score).view(np.int32))))
            for k in range(num_aux_labels):
                aux[k].append(int(ln[3 + k]))
        arcs = torch.tensor(rows, dtype=torch.int32).reshape(-1, 4)
        ans = cls(arcs)
        for k, name in enumerate(aux_label_names):
            setattr(ans, name, torch.tensor(aux[k], dtype=torch.int32))
        return ans

    def __str__(self) -> str:
        return (f"k2_b200.Fsa(shape={self.shape}, num_arcs={self.num_arcs}, "
                f"device={self.device})")

    __repr__ = __str__


def _basic_properties(arcs: RaggedArc) -> int:
    """AND of the per-FSA property bits (k2/csrc/fsa.cu:54-217)."""
    if not arcs.values().is_cuda:
        return _host_properties(arcs)
    dev = arcs.device
    nf, ns, na = arcs.num_fsas, arcs.num_states, arcs.num_elements()
    props = torch.empty(nf + 1, dtype=torch.int32, device=dev)
    tmp = torch.empty(_lib.lib.k2b200_fsa_properties_tmp_bytes(nf, ns), dtype=torch.uint8,
                      device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.k2b200_fsa_properties(
            _lib.ptr(arcs._row_splits1), _lib.ptr(arcs.row_ids(1 - arcs.single)),
            _lib.ptr(arcs._row_splits2), _lib.ptr(arcs.row_ids(2 - arcs.single)),
            _lib.ptr(arcs.values()), nf, ns, na, _lib.ptr(props), _lib.ptr(tmp),
            _lib.stream_of(dev)))
    return int(props[nf].item())


def _host_properties(arcs: RaggedArc) -> int:
    """Property bits of a host-resident graph (input preparation only: graphs are
    built on the host before they are moved to the GPU)."""
    rs1 = arcs.h_row_splits1
    rs2 = arcs._row_splits2.numpy()
    v = arcs.values().numpy()
    tot = ALL
    ns = arcs.num_states
    reach = np.zeros(2 * ns + 2, dtype=bool)
    for i in range(len(rs1) - 1):
        b, e = int(rs1[i]), int(rs1[i + 1])
        n = e - b
        neg = 0
        a0, a1 = int(rs2[b]), int(rs2[e])
        if a1 > a0:
            src, dest, label = v[a0:a1, 0], v[a0:a1, 1], v[a0:a1, 2]
            state_of = np.repeat(np.arange(b, e), np.diff(rs2[b:e + 1]))
            if np.any(src != state_of - b):
                neg |= VALID
            if np.any(dest <= src):
                neg |= TOPSORTED_AND_ACYCLIC
            if np.any(dest < src):
                neg |= TOPSORTED
            if np.any(label == 0):
                neg |= EPSILON_FREE
            if np.any(label < -1) or np.any((label == -1) & (dest != n - 1)):
                neg |= VALID
            if np.any((label != -1) & (dest == n - 1)):
                neg |= VALID
            bad = (dest < 0) | (dest >= n)
            if np.any(bad):
                neg |= VALID
            ok = ~bad & (dest != src)
            reach[b + dest[ok]] = True
            reach[b] = True
            reach[ns + e - 1] = True
            reach[ns + state_of[dest != src]] = True
            first = np.ones(a1 - a0, dtype=bool)
            first[1:] = state_of[1:] != state_of[:-1]
            ul = label.astype(np.uint32)
            nf_ = ~first
            if np.any(nf_[1:] & (ul[1:] <= ul[:-1])):
                neg |= ARC_SORTED_AND_DETERMINISTIC
            if np.any(nf_[1:] & (ul[1:] < ul[:-1])):
                neg |= ARC_SORTED
            if np.any(nf_[1:] & (label[1:] == label[:-1]) & (dest[1:] < dest[:-1])):
                neg |= ARC_SORTED
        else:
            neg |= NONEMPTY
        if n > 0 and not reach[b:e].all():
            neg |= ACCESSIBLE
        if n > 0 and not reach[ns + b:ns + e].all():
            neg |= COACCESSIBLE
        tot &= (~neg) & ALL
    return int(tot)


def create_fsa_vec(fsas: List[Fsa]) -> Fsa:
    """Stack single FSAs (or FsaVecs) into one FsaVec (k2/python/k2/utils.py
    create_fsa_vec): per-arc tensor attributes present on every input are carried."""
    rs1, rs2, vals = [0], [0], []
    for f in fsas:
        a = f.arcs
        h1 = a.h_row_splits1
        r2 = a._row_splits2.cpu().numpy()
        for i in range(len(h1) - 1):
            rs1.append(rs1[-1] + int(h1[i + 1] - h1[i]))
        rs2.extend((r2[1:] - r2[0] + rs2[-1]).tolist())
        vals.append(a.values().cpu())
    dev = fsas[0].device
    values = torch.cat(vals, dim=0).contiguous().to(dev) if vals else torch.zeros(
        (0, 4), dtype=torch.int32, device=dev)
    h1 = np.asarray(rs1, dtype=np.int32)
    r2 = np.asarray(rs2, dtype=np.int32)
    arcs = RaggedArc(values, torch.from_numpy(h1).to(dev), torch.from_numpy(r2).to(dev),
                     h_row_splits1=h1, h_arc_splits=r2[h1].astype(np.int32))
    ans = Fsa(arcs)
    if any(f.scores.requires_grad for f in fsas):
        # keep the autograd link from the stacked scores to the inputs' scores
        ans.scores = torch.cat([f.scores for f in fsas], dim=0)
    names = None
    for f in fsas:
        these = {n for n, _ in f.named_tensor_attr(include_scores=False) if n != 'labels'}
        names = these if names is None else names & these
    for name in sorted(names or []):
        parts = [getattr(f, name) for f in fsas]
        if isinstance(parts[0], RaggedTensor):
            setattr(ans, name, _ragged_cat(parts).to(dev))
        else:
            setattr(ans, name, torch.cat(parts, dim=0).to(dev))
    return ans

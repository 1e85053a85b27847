"""CUDA-resident counterpart of `_k2.RaggedArc` (k2/python/csrc/torch/ragged.cu:40-160).

A RaggedArc is k2's `Ragged<Arc>` with 3 axes [fsa][state][arc]:
  values       int32 [num_arcs, 4]: src_state, dest_state, label, score bits
  row_splits1  int32 [num_fsas + 1]   fsa   -> first state (idx01)
  row_splits2  int32 [num_states + 1] state -> first arc (idx012)
  row_ids1/2   the inverse maps, built on demand by a CUDA kernel
A 2-axis Fsa (single FSA) is stored as a 3-axis one with one entry and
`single=True`, which is how the reference lifts it before every FsaVec
algorithm (k2/python/csrc/torch/fsa_algo.cu:236-238).
"""
from typing import Optional

import numpy as np
import torch

from . import _lib


class RaggedArc:

    def __init__(self, values: torch.Tensor, row_splits1: torch.Tensor,
                 row_splits2: torch.Tensor, row_ids1: Optional[torch.Tensor] = None,
                 row_ids2: Optional[torch.Tensor] = None, single: bool = False,
                 h_row_splits1: Optional[np.ndarray] = None,
                 h_arc_splits: Optional[np.ndarray] = None):
        assert values.dtype == torch.int32 and values.ndim == 2 and values.shape[1] == 4
        assert values.is_contiguous()
        assert row_splits1.dtype == torch.int32 and row_splits2.dtype == torch.int32
        self._values = values
        self._row_splits1 = row_splits1.contiguous()
        self._row_splits2 = row_splits2.contiguous()
        self._row_ids1 = row_ids1
        self._row_ids2 = row_ids2
        self.single = single
        self._h_row_splits1 = h_row_splits1
        self._h_arc_splits = h_arc_splits
        # lazily built device-side helpers
        self._incoming = None  # (in_splits, in_arcs, in_src, in_score)
        self._incoming_key = None
        self._levels = None    # (level_offsets, level_splits) of a layered FsaVec
        # (strict, max_layers, max_layer_states, max_layer_arcs): set for lattices
        # whose arcs all go from one layer to the next, with bounds on layer sizes
        self._layer_bounds = (0, 0, 0, 0)

    # ---- _k2.RaggedArc interface ----------------------------------------
    def values(self) -> torch.Tensor:
        return self._values

    def num_axes(self) -> int:
        return 2 if self.single else 3

    def dim0(self) -> int:
        if self.single:
            return self.num_states
        return self._row_splits1.shape[0] - 1

    @property
    def num_fsas(self) -> int:
        return self._row_splits1.shape[0] - 1

    @property
    def num_states(self) -> int:
        return self._row_splits2.shape[0] - 1

    def num_elements(self) -> int:
        return self._values.shape[0]

    def tot_size(self, axis: int) -> int:
        if self.single:
            axis += 1
        return [self.num_fsas, self.num_states, self.num_elements()][axis]

    @property
    def device(self) -> torch.device:
        return self._values.device

    def row_splits(self, axis: int) -> torch.Tensor:
        if self.single:
            axis += 1
        assert axis in (1, 2)
        return self._row_splits1 if axis == 1 else self._row_splits2

    def row_ids(self, axis: int) -> torch.Tensor:
        if self.single:
            axis += 1
        assert axis in (1, 2)
        if axis == 1:
            if self._row_ids1 is None:
                self._row_ids1 = _row_ids(self._row_splits1, self.num_states)
            return self._row_ids1
        if self._row_ids2 is None:
            self._row_ids2 = _row_ids(self._row_splits2, self.num_elements())
        return self._row_ids2

    def to(self, device) -> "RaggedArc":
        device = torch.device(device)
        if device == self.device:
            return self
        mv = lambda t: None if t is None else t.to(device)  # noqa: E731
        out = RaggedArc(self._values.to(device), self._row_splits1.to(device),
                        self._row_splits2.to(device), mv(self._row_ids1), mv(self._row_ids2),
                        self.single, self.h_row_splits1, self.h_arc_splits)
        return out

    def clone(self) -> "RaggedArc":
        out = RaggedArc(self._values.clone(), self._row_splits1, self._row_splits2,
                        self._row_ids1, self._row_ids2, self.single, self._h_row_splits1,
                        self._h_arc_splits)
        out._levels = self._levels
        out._layer_bounds = self._layer_bounds
        return out

    # ---- host copies of the small per-FSA splits ---------------------------
    @property
    def h_row_splits1(self) -> np.ndarray:
        if self._h_row_splits1 is None:
            self._h_row_splits1 = self._row_splits1.cpu().numpy().astype(np.int32)
        return self._h_row_splits1

    @property
    def h_arc_splits(self) -> np.ndarray:
        """row_splits2[row_splits1[i]]: first arc of every FSA, on the host."""
        if self._h_arc_splits is None:
            idx = self._row_splits1.long()
            self._h_arc_splits = self._row_splits2[idx].cpu().numpy().astype(np.int32)
        return self._h_arc_splits

    # ---- device-side helpers -------------------------------------------------
    def incoming(self):
        """(in_splits, in_arcs, in_src, in_score): the arcs entering every state by
        arc index, with their source state (idx01) and score in the same order.
        Cached; the reference recomputes the index on every intersect_dense call
        (k2/csrc/intersect_dense.cu:139-142).  The cache is dropped when the
        scores or labels of the owning Fsa are re-assigned."""
        key = (self._values.data_ptr(), self._values._version)
        if self._incoming is None or self._incoming_key != key:
            _lib.require_cuda(self._values, "arcs")
            ns, na = self.num_states, self.num_elements()
            dev = self.device
            in_splits = torch.empty(ns + 1, dtype=torch.int32, device=dev)
            buf = torch.empty((3, max(na, 1)), dtype=torch.int32, device=dev)
            tmp = torch.empty(_lib.lib.k2b200_fsa_incoming_tmp_bytes(ns, na), dtype=torch.uint8,
                              device=dev)
            with torch.cuda.device(dev):
                _lib.check(_lib.lib.k2b200_fsa_incoming(
                    _lib.ptr(self._row_splits1), _lib.ptr(self.row_ids(1 - self.single)),
                    _lib.ptr(self.row_ids(2 - self.single)), _lib.ptr(self._values),
                    self.num_fsas, ns, na, _lib.ptr(in_splits), buf[0].data_ptr(),
                    buf[1].data_ptr(), buf[2].data_ptr(), _lib.ptr(tmp), _lib.stream_of(dev)))
            self._incoming = (in_splits, buf[0, :na], buf[1, :na],
                              buf[2, :na].view(torch.float32))
            self._incoming_key = key
        return self._incoming

    def band_tables(self):
        """(band_states, band_arcs, ok): the per-state tables of k2b200_band_tables
        for this FsaVec, and whether every graph is a band graph (arcs from a state s
        to s, s+1 or s+2 only, one arc per (source, destination), one label per
        destination) - the shape of CTC graphs.  Cached per version of the arc
        tensor.  Graphs that `ctc_graph` wrote are band graphs by construction; for
        any other FsaVec the answer costs one host read, once."""
        vals = self._values
        key = (vals.data_ptr(), vals._version)
        cached = getattr(self, "_band", None)
        if cached is not None and cached[0] == key:
            return cached[1]
        _lib.require_cuda(vals, "arcs")
        dev = self.device
        ns = self.num_states
        sb, ab = _lib.c_sz(), _lib.c_sz()
        import ctypes
        _lib.check(_lib.lib.k2b200_band_tables_bytes(ns, ctypes.byref(sb), ctypes.byref(ab)))
        states = torch.empty(sb.value, dtype=torch.uint8, device=dev)
        arcs = torch.empty(ab.value, dtype=torch.uint8, device=dev)
        status = torch.empty(1, dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.k2b200_band_tables(
                _lib.ptr(self._row_splits1), self.num_fsas, _lib.ptr(self._row_splits2),
                _lib.ptr(vals), ns, _lib.ptr(states), _lib.ptr(arcs), _lib.ptr(status),
                _lib.stream_of(dev)))
        if getattr(self, "_band_by_construction", None) == key:
            ok = True
        else:
            ok = (int(status.item()) & 1) == 0
        ans = (states, arcs, ok)
        self._band = (key, ans)
        return ans

    def replicated(self, min_bytes: int = 32 << 20) -> bool:
        """Is every FSA of this FsaVec an exact copy of FSA 0 (states, arcs and
        scores), and is the whole large enough (`min_bytes`) for that to matter?
        Decoding graphs are stacked like this, one copy per sequence.  One device
        comparison and host read per version of the arc tensor, then cached."""
        n = self.num_fsas
        vals = self._values
        if n < 2 or vals.numel() * 4 < min_bytes or not vals.is_cuda:
            return False
        key = (vals.data_ptr(), vals._version, self._row_splits2.data_ptr())
        cached = getattr(self, "_replicated", None)
        if cached is not None and cached[0] == key:
            return cached[1]
        h1 = np.asarray(self.h_row_splits1, dtype=np.int64)
        ha = np.asarray(self.h_arc_splits, dtype=np.int64)
        S, A = int(h1[1] - h1[0]), int(ha[1] - ha[0])
        same = bool(np.all(np.diff(h1) == S) and np.all(np.diff(ha) == A)) and S > 0 and A > 0
        if same:
            v = vals.view(n, A, 4)
            rs2 = self._row_splits2[:-1].view(n, S)
            same = bool(((v == v[0]).all() & ((rs2 - rs2[:, :1]) == (rs2[0] - rs2[0, 0])).all())
                        .item())
        self._replicated = (key, same)
        return same

    def max_degree(self) -> int:
        """Largest in- or out-degree of any state (one host read, cached)."""
        if getattr(self, "_max_degree", None) is None:
            if self.num_elements() == 0:
                self._max_degree = 0
            else:
                in_splits = self.incoming()[0]
                m = torch.maximum(torch.diff(in_splits).max(), torch.diff(self._row_splits2).max())
                self._max_degree = int(m.item())
        return self._max_degree

    def view(self, want_incoming: bool):
        """The k2b200_fsa_view of this FsaVec (keeps the tensors it points to alive
        through the returned tuple)."""
        lvl_off, lvl_splits = self.levels()
        inc = self.incoming() if want_incoming else (None, None, None, None)
        strict, max_layers, max_w, max_a = self._layer_bounds
        rid1, rid2 = self.row_ids(1 - self.single), self.row_ids(2 - self.single)
        v = _lib.FsaView(
            num_fsas=self.num_fsas, num_states=self.num_states, num_arcs=self.num_elements(),
            row_splits1=_lib.ptr(self._row_splits1), row_ids1=_lib.ptr(rid1),
            row_splits2=_lib.ptr(self._row_splits2), row_ids2=_lib.ptr(rid2),
            arcs=_lib.ptr(self._values), in_splits=_lib.ptr(inc[0]), in_arcs=_lib.ptr(inc[1]),
            in_src=_lib.ptr(inc[2]), in_score=_lib.ptr(inc[3]),
            level_offsets=_lib.ptr(lvl_off), level_splits=_lib.ptr(lvl_splits),
            strict_layers=strict, max_layers=max_layers, max_layer_states=max_w,
            max_layer_arcs=max_a)
        return v, (inc, lvl_off, lvl_splits, rid1, rid2)

    def levels(self):
        """(level_offsets, level_splits): a layering of the states such that every
        arc goes from a lower to a higher layer.  Lattices made by intersect_dense
        carry their frame layering; for any other top-sorted acyclic FsaVec the
        layering (longest distance from a state without entering arcs) is computed
        on the GPU once and cached (k2b200_fsa_levels; one host read of its status
        and of the number of layers)."""
        if self._levels is None:
            self._levels = _gpu_levels(self)
        return self._levels

    def __repr__(self):
        return (f"RaggedArc(num_fsas={self.num_fsas}, num_states={self.num_states}, "
                f"num_arcs={self.num_elements()}, device={self.device})")


def _row_ids(row_splits: torch.Tensor, num_elems: int) -> torch.Tensor:
    out = torch.empty(num_elems, dtype=torch.int32, device=row_splits.device)
    if num_elems == 0:
        return out
    if row_splits.is_cuda:
        with torch.cuda.device(row_splits.device):
            _lib.check(_lib.lib.k2b200_row_splits_to_row_ids(
                _lib.ptr(row_splits), row_splits.shape[0] - 1, _lib.ptr(out), num_elems,
                _lib.stream_of(row_splits.device)))
        return out
    # host-resident graphs (e.g. straight out of ctc_graph before .to(device))
    rs = row_splits.numpy()
    return torch.from_numpy(
        np.repeat(np.arange(len(rs) - 1, dtype=np.int32), np.diff(rs)).astype(np.int32))


def _gpu_levels(arcs: RaggedArc):
    _lib.require_cuda(arcs._values, "fsas")
    dev = arcs.device
    ns, na, nf = arcs.num_states, arcs.num_elements(), arcs.num_fsas
    i32 = dict(dtype=torch.int32, device=dev)
    offsets = torch.empty(nf + 2, **i32)   # [nf + 1] offsets, then the status word
    splits = torch.empty(ns + 2, **i32)
    tmp = torch.empty(_lib.lib.k2b200_fsa_levels_tmp_bytes(ns), dtype=torch.uint8, device=dev)
    rid2 = arcs.row_ids(2 - arcs.single)
    status = offsets[nf + 1:]
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.k2b200_fsa_levels(
            _lib.ptr(arcs._row_splits1), _lib.ptr(arcs._row_splits2), _lib.ptr(rid2),
            _lib.ptr(arcs._values), nf, ns, na, _lib.ptr(offsets), _lib.ptr(splits),
            _lib.ptr(status), _lib.ptr(tmp), _lib.stream_of(dev)))
    total, bad = (int(v) for v in offsets[nf:].tolist())
    if bad:
        raise RuntimeError("forward/backward scores need a top-sorted, acyclic FsaVec")
    return offsets[:nf + 1], splits[:total + 1]

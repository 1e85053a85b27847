"""Chunk-by-chunk decoding with the reference's names
(k2/python/k2/online_dense_intersecter.py:16-147 over k2::OnlineDenseIntersecter,
k2/csrc/intersect_dense_pruned.cu:1739-1853): `decode` takes the DenseFsaVec of one
chunk and the states of the streams in it, and returns the lattice of everything those
streams have decoded so far together with their new states."""
import ctypes
from typing import List, Optional, Tuple

import numpy as np
import torch

from . import _lib
from .dense_fsa_vec import DenseFsaVec
from .fsa import Fsa
from .ragged import RaggedArc


class DecodeStateInfo:
    """What one stream has decoded so far (k2::DecodeStateInfo,
    k2/csrc/intersect_dense_pruned.h:113-137): the pruned frames as device arrays, the
    number of frames and the current search beam.  `DecodeStateInfo()` (or `None`) in the
    list given to `decode` starts a new stream."""

    def __init__(self, tensors=None, frames: int = 0, beam: Optional[float] = None):
        self.is_new = tensors is None
        if tensors is not None:
            (self.astate, self.forward, self.arc0, self.arc_graph, self.arc_score,
             self.arc_dest, self.frame_state0, self.frame_arc0) = tensors
        self.frames = frames
        self.beam = beam

    def _c(self) -> '_lib.OnlineStream':
        return _lib.OnlineStream(
            num_states=self.astate.numel(), num_arcs=self.arc_graph.numel(),
            astate=_lib.ptr(self.astate), forward=_lib.ptr(self.forward), arc0=_lib.ptr(self.arc0),
            arc_graph=_lib.ptr(self.arc_graph), arc_score=_lib.ptr(self.arc_score),
            arc_dest=_lib.ptr(self.arc_dest), frame_state0=_lib.ptr(self.frame_state0),
            frame_arc0=_lib.ptr(self.frame_arc0))


def _alloc_state(num_states: int, num_arcs: int, frames: int, beam: float, dev) -> DecodeStateInfo:
    i32 = dict(dtype=torch.int32, device=dev)
    return DecodeStateInfo(
        (torch.empty(max(num_states, 1), **i32)[:num_states],
         torch.empty(max(num_states, 1), **i32)[:num_states],
         torch.empty(num_states + 1, **i32),
         torch.empty(max(num_arcs, 1), **i32)[:num_arcs],
         torch.empty(max(num_arcs, 1), dtype=torch.float32, device=dev)[:num_arcs],
         torch.empty(max(num_arcs, 1), **i32)[:num_arcs],
         torch.empty(frames + 2, **i32), torch.empty(frames + 2, **i32)), frames, beam)


class OnlineDenseIntersecter:

    def __init__(self, decoding_graph: Fsa, num_streams: int, search_beam: float,
                 output_beam: float, min_active_states: int, max_active_states: int,
                 allow_partial: bool = True) -> None:
        arcs = decoding_graph.arcs
        _lib.require_cuda(arcs.values(), "decoding_graph")
        if arcs.num_fsas != 1:
            raise RuntimeError("the decoding graph must be a single Fsa shared by the streams")
        self.decoding_graph = decoding_graph
        self.device = arcs.device
        self.num_streams_ = num_streams
        self.search_beam, self.output_beam = float(search_beam), float(output_beam)
        self.min_active_states, self.max_active_states = min_active_states, max_active_states
        self.allow_partial = bool(allow_partial)
        self._arcs_per_seq = 1 << 16

    @property
    def num_streams(self) -> int:
        return self.num_streams_

    def _new_stream(self) -> DecodeStateInfo:
        dev = self.device
        st = _alloc_state(1, 0, 0, self.search_beam, dev)
        st.astate.zero_()          # the start state of the graph
        st.forward.zero_()         # a forward score of 0.0 in order-preserving int form
        st.arc0.zero_()
        st.frame_state0.copy_(torch.tensor([0, 1], dtype=torch.int32))
        st.frame_arc0.zero_()
        return st

    def decode(self, dense_fsas: DenseFsaVec, decode_states: List[Optional[DecodeStateInfo]]
               ) -> Tuple[Fsa, List[DecodeStateInfo]]:
        dev = self.device
        arcs = self.decoding_graph.arcs
        n = dense_fsas.dim0()
        if len(decode_states) != n:
            raise RuntimeError(f"{len(decode_states)} decode states for {n} sequences")
        states = [self._new_stream() if s is None or s.is_new else s for s in decode_states]
        h_brs = np.ascontiguousarray(dense_fsas.h_row_splits, dtype=np.int32)
        h_hist = np.asarray([s.frames for s in states], dtype=np.int32)
        beams_in = np.asarray([s.beam for s in states], dtype=np.float32)
        scores = dense_fsas.scores.detach()
        chunk = int(h_brs[1] - h_brs[0]) - 1
        need_a = max(s.arc_graph.numel() for s in states)
        need_s = max(s.astate.numel() for s in states)
        cap_a = max(self._arcs_per_seq, 2 * need_a, 4 * need_s)
        stream = _lib.stream_of(dev)
        i32 = dict(dtype=torch.int32, device=dev)
        while True:
            args = _lib.OnlineArgs(
                num_states=arcs.num_states, num_arcs=arcs.num_elements(),
                a_row_splits1=_lib.ptr(arcs._row_splits1), a_row_splits2=_lib.ptr(arcs._row_splits2),
                a_arcs=_lib.ptr(arcs.values()), scores=_lib.ptr(scores), rows=scores.shape[0],
                cols=scores.shape[1], num_seqs=n, b_row_splits=_lib.ptr(dense_fsas.row_splits),
                h_b_row_splits=h_brs.ctypes.data, search_beam=self.search_beam,
                output_beam=self.output_beam, min_active_states=self.min_active_states,
                max_active_states=self.max_active_states, allow_partial=int(self.allow_partial),
                h_hist=h_hist.ctypes.data, max_states_per_seq=max(cap_a // 2, need_s + 2),
                max_arcs_per_seq=cap_a, team_ctas=0)
            nbytes = ctypes.c_size_t()
            _lib.check(_lib.lib.k2b200_online_decode_workspace_bytes(ctypes.byref(args),
                                                                     ctypes.byref(nbytes)))
            ws = torch.empty(nbytes.value, dtype=torch.uint8, device=dev)
            beams_out = np.zeros(n, np.float32)
            counts = np.zeros(2 * n, np.int32)
            ns, na, full = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
            with torch.cuda.device(dev):
                loads = (_lib.OnlineStream * n)(*[s._c() for s in states])
                _lib.check(_lib.lib.k2b200_online_decode_load_all(
                    ctypes.byref(args), _lib.ptr(ws), loads, stream))
                _lib.check(_lib.lib.k2b200_online_decode_run(
                    ctypes.byref(args), _lib.ptr(ws), nbytes.value, stream,
                    beams_in.ctypes.data, beams_out.ctypes.data, counts.ctypes.data,
                    ctypes.byref(ns), ctypes.byref(na), ctypes.byref(full)))
            if not full.value:
                self._arcs_per_seq = max(self._arcs_per_seq, cap_a)
                break
            del ws
            cap_a *= 4
            if cap_a >= 1 << 30:
                raise RuntimeError("OnlineDenseIntersecter: more than 2^30 arcs alive in a stream")
        ns, na = ns.value, na.value
        new_states = []
        with torch.cuda.device(dev):
            row_splits1 = torch.empty(n + 1, **i32)
            row_ids1 = torch.empty(ns + 1, **i32)
            row_splits2 = torch.empty(ns + 1, **i32)
            row_ids2 = torch.empty(na + 1, **i32)
            values = torch.empty((na + 1, 4), **i32)
            arc_map_a = torch.empty(na + 1, **i32)
            level_offsets = torch.empty(n + 1, **i32)
            level_splits = torch.empty(int(h_hist.sum()) + n * (chunk + 2) + 1, **i32)
            out = _lib.LatticeOut(
                row_splits1=_lib.ptr(row_splits1), row_ids1=_lib.ptr(row_ids1),
                row_splits2=_lib.ptr(row_splits2), row_ids2=_lib.ptr(row_ids2),
                arcs=_lib.ptr(values), arc_map_a=_lib.ptr(arc_map_a), arc_map_b=None,
                level_offsets=_lib.ptr(level_offsets), level_splits=_lib.ptr(level_splits))
            _lib.check(_lib.lib.k2b200_online_decode_emit(
                ctypes.byref(args), _lib.ptr(ws), nbytes.value, stream, ctypes.byref(out)))
            # one allocation for the arrays of all streams of the batch
            sizes = [(int(counts[2 * i]), int(counts[2 * i + 1]), s.frames + chunk)
                     for i, s in enumerate(states)]
            pool = torch.empty(sum(3 * a + 1 + 3 * b + 2 * (f + 2) for a, b, f in sizes) + 1, **i32)
            at = 0
            for i, (a, b, f) in enumerate(sizes):
                parts = []
                for count in (a, a, a + 1, b, b, b, f + 2, f + 2):
                    parts.append(pool[at:at + count])
                    at += count
                parts[4] = parts[4].view(torch.float32)
                new_states.append(DecodeStateInfo(tuple(parts), f, float(beams_out[i])))
            stores = (_lib.OnlineStream * n)(*[s._c() for s in new_states])
            _lib.check(_lib.lib.k2b200_online_decode_store_all(
                ctypes.byref(args), _lib.ptr(ws), stores, stream))
        lattice = RaggedArc(values[:na], row_splits1, row_splits2, row_ids1[:ns], row_ids2[:na])
        lattice._levels = (level_offsets, level_splits)  # frames are layers
        arc_map_a = arc_map_a[:na]
        # attributes of the graph follow the arc map, as
        # k2.utils.fsa_from_unary_function_tensor does (k2/python/k2/utils.py)
        from .autograd import index_select
        out_fsa = Fsa(lattice, _check=False)
        for name, value in self.decoding_graph.named_tensor_attr(include_scores=False):
            if name != 'labels':
                setattr(out_fsa, name, index_select(value, arc_map_a))
        for name, value in self.decoding_graph.named_non_tensor_attr():
            setattr(out_fsa, name, value)
        out_fsa._arc_map_a = arc_map_a
        return out_fsa, new_states

"""Graph construction and best-path helpers around the hot path: `ctc_graph`
(k2/python/k2/fsa_algo.py:1160-1249 over k2::CtcGraphs, k2/csrc/fsa_algo.cu:577-730),
`linear_fsa`, `arc_sort` and `shortest_path` (fsa_algo.py:598-620 over
k2::ShortestPath, fsa_algo.cu:869-1144)."""
from typing import List, Optional, Tuple, Union

import itertools

import numpy as np
import torch

from . import _lib
from .autograd import index_select
from .fsa import Fsa
from .ragged import RaggedArc


def _fsa_vec_from_numpy(rs1: np.ndarray, rs2: np.ndarray, values: np.ndarray, device,
                        aux_labels: Optional[np.ndarray] = None) -> Fsa:
    rs1 = np.ascontiguousarray(rs1, dtype=np.int32)
    rs2 = np.ascontiguousarray(rs2, dtype=np.int32)
    values = np.ascontiguousarray(values, dtype=np.int32).reshape(-1, 4)
    device = torch.device(device)
    arcs = RaggedArc(torch.from_numpy(values).to(device), torch.from_numpy(rs1).to(device),
                     torch.from_numpy(rs2).to(device), h_row_splits1=rs1,
                     h_arc_splits=rs2[rs1].astype(np.int32))
    aux = None if aux_labels is None else torch.from_numpy(
        np.ascontiguousarray(aux_labels, dtype=np.int32)).to(device)
    return Fsa(arcs, aux_labels=aux)


def ctc_graph(symbols: List[List[int]], modified: bool = False,
              device: Optional[Union[torch.device, str]] = "cpu") -> Fsa:
    """CTC graphs of a batch of transcripts, all arc scores 0.

    For a transcript of L symbols the graph has 2L+2 states: state 2k is the
    blank state in front of symbol k (2L: the trailing blank state), 2k+1 the
    state of symbol k, 2L+1 the final state.  Blank states carry a blank
    self-loop and an arc to the next symbol (or the final arc); symbol states an
    arc to the next blank state, a self-loop and - unless the next symbol is the
    same and `modified` is False - an arc that skips the blank.  `aux_labels`
    holds the symbol on the arcs that enter a symbol state (fsa_algo.cu:672-727).
    """
    n = len(symbols)
    lens = np.fromiter(map(len, symbols), dtype=np.int64, count=n)
    tot = int(lens.sum())
    # (labels are int32 everywhere below; converting Python ints is what this call costs)
    sym = np.fromiter(itertools.chain.from_iterable(symbols), dtype=np.int32, count=tot)
    assert not np.any(sym == -1), "symbols must not contain -1"
    if torch.device(device).type == "cuda":
        return _ctc_graph_cuda(lens, sym, modified, torch.device(device))
    sym_off = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(lens, out=sym_off[1:])
    fsa_of_sym = np.repeat(np.arange(n), lens)
    k = np.arange(tot) - sym_off[fsa_of_sym]          # position within its transcript
    is_last = k == lens[fsa_of_sym] - 1
    nxt = np.where(is_last, -1, np.append(sym[1:], -1) if tot else sym)
    has3 = np.ones(tot, dtype=bool) if modified else (sym != nxt)

    # per-symbol arc block: blank state 2k (2 arcs) then symbol state 2k+1 (2 or 3)
    per_sym = 4 + has3.astype(np.int64)
    state_off = 2 * sym_off + 2 * np.arange(n + 1)     # first state of each FSA
    arc_fsa_off = np.zeros(n + 1, dtype=np.int64)      # first arc of each FSA
    arcs_per_fsa = np.zeros(n, dtype=np.int64)
    np.add.at(arcs_per_fsa, fsa_of_sym, per_sym)
    arcs_per_fsa += 2                                  # trailing blank state
    np.cumsum(arcs_per_fsa, out=arc_fsa_off[1:])
    num_arcs = int(arc_fsa_off[-1])
    num_states = int(state_off[-1])

    # offset of each symbol's block inside its FSA
    blk = np.zeros(tot, dtype=np.int64)
    if tot:
        c = np.cumsum(per_sym) - per_sym
        blk = c - c[sym_off[fsa_of_sym]] + arc_fsa_off[fsa_of_sym]

    values = np.zeros((num_arcs, 4), dtype=np.int32)   # score bits 0 == 0.0f
    aux = np.zeros(num_arcs, dtype=np.int32)
    rs2 = np.zeros(num_states + 1, dtype=np.int64)
    s_blank = 2 * k
    s_sym = 2 * k + 1

    def put(pos, src, dest, label, auxv):
        values[pos, 0] = src
        values[pos, 1] = dest
        values[pos, 2] = label
        aux[pos] = auxv

    if tot:
        put(blk + 0, s_blank, s_blank, 0, 0)
        put(blk + 1, s_blank, s_sym, sym, sym)
        put(blk + 2, s_sym, s_sym + 1, 0, 0)
        put(blk + 3, s_sym, s_sym, sym, 0)
        p3 = blk[has3] + 4
        put(p3, s_sym[has3], s_sym[has3] + 2, nxt[has3], nxt[has3])  # -1 when last
        gs = state_off[fsa_of_sym]
        rs2[gs + s_blank] = blk
        rs2[gs + s_sym] = blk + 2
    # trailing blank state 2L and final state 2L+1 of every FSA
    tail = arc_fsa_off[1:] - 2
    L2 = 2 * lens
    put(tail, L2, L2, 0, 0)
    put(tail + 1, L2, L2 + 1, -1, -1)
    rs2[state_off[:-1] + L2] = tail
    rs2[state_off[:-1] + L2 + 1] = tail + 2
    rs2[num_states] = num_arcs
    return _fsa_vec_from_numpy(state_off, rs2, values, device, aux)


def _ctc_graph_splits(lens: np.ndarray, sym: np.ndarray, modified: bool):
    """(first symbol, first state, first arc) of every graph, int64 [n + 1] each.  A
    transcript of L symbols gives 2L + 2 states; its symbol states have 3 arcs - 2 when
    the next symbol of the transcript is the same and `modified` is False -, its blank
    states 2.  (A few numpy calls over the flat symbols: this runs on the thread that
    feeds the GPU whenever a batch brings new transcripts.)"""
    n, tot = len(lens), len(sym)
    sym_off = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(lens, out=sym_off[1:])
    per_fsa = 5 * lens + 2
    if tot > 1 and not modified:
        same = sym[1:] == sym[:-1]
        # the last symbol of a transcript always has its third arc (into the final state)
        ends = sym_off[1:][lens > 0] - 1
        same[ends[ends < tot - 1]] = False
        at = np.searchsorted(np.flatnonzero(same), sym_off)  # symbols without one, before each
        per_fsa -= at[1:] - at[:-1]
    h_arc_splits = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(per_fsa, out=h_arc_splits[1:])
    h_rs1 = 2 * sym_off + 2 * np.arange(n + 1)
    return sym_off, h_rs1, h_arc_splits


def _ctc_graph_cuda(lens: np.ndarray, sym: np.ndarray, modified: bool, device) -> Fsa:
    """The graphs are written by CUDA kernels; the host only counts the arcs (to
    size the outputs) and derives the per-FSA splits it needs later anyway."""
    n, tot = len(lens), int(lens.sum())
    sym_off, h_rs1, h_arc_splits = _ctc_graph_splits(lens, sym, modified)
    num_arcs, num_states = int(h_arc_splits[-1]), int(h_rs1[-1])
    h_meta = np.empty(n + 1 + tot, dtype=np.int32)
    h_meta[:n + 1] = sym_off
    h_meta[n + 1:] = sym
    meta = _lib.upload_i32(h_meta, device)
    i32 = dict(dtype=torch.int32, device=device)
    rs1 = torch.empty(n + 1, **i32)
    rs2 = torch.empty(num_states + 1, **i32)
    values = torch.empty((num_arcs, 4), **i32)
    aux = torch.empty(num_arcs, **i32)
    tmp = torch.empty(_lib.lib.k2b200_ctc_graph_tmp_bytes(tot), dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        _lib.check(_lib.lib.k2b200_ctc_graph(
            _lib.ptr(meta[:n + 1]), _lib.ptr(meta[n + 1:]), n, tot, int(modified), _lib.ptr(rs1),
            _lib.ptr(rs2), _lib.ptr(values), _lib.ptr(aux), _lib.ptr(tmp),
            _lib.stream_of(device)))
    arcs = RaggedArc(values, rs1, rs2, h_row_splits1=h_rs1.astype(np.int32),
                     h_arc_splits=h_arc_splits.astype(np.int32))
    # CTC graphs are band graphs (RaggedArc.band_tables) for as long as nobody edits them
    arcs._band_by_construction = (values.data_ptr(), values._version)
    # valid, non-empty, not top-sorted (self-loops), epsilon arcs present (blank = 0),
    # accessible and co-accessible by construction: the bits the host path computes
    return Fsa(arcs, aux_labels=aux, _check=False)


def linear_fsa(labels: Union[List[int], List[List[int]]],
               device: Optional[Union[torch.device, str]] = "cpu") -> Fsa:
    """Linear acceptor(s) for symbol sequence(s), each with a final arc -1
    (k2/python/k2/fsa_algo.py linear_fsa over k2::LinearFsas)."""
    single = len(labels) == 0 or not isinstance(labels[0], (list, tuple))
    seqs = [labels] if single else labels
    rs1, rs2, rows = [0], [], []
    for seq in seqs:
        full = list(seq) + [-1]
        for s, lab in enumerate(full):
            rs2.append(len(rows))
            rows.append((s, s + 1, lab, 0))
        rs2.append(len(rows))  # final state
        rs1.append(rs1[-1] + len(full) + 1)
    rs2.append(len(rows))
    ans = _fsa_vec_from_numpy(np.asarray(rs1), np.asarray(rs2), np.asarray(rows), device)
    if single:
        ans.arcs.single = True
    return ans


def ctc_topo(max_token: int, modified: bool = False,
             device: Optional[Union[torch.device, str]] = None) -> Fsa:
    """The CTC topology over tokens 1..max_token with blank 0, as a single Fsa with
    `aux_labels` (k2/python/k2/fsa_algo.py ctc_topo over k2::CtcTopo,
    k2/csrc/fsa_algo.cu:732-817): all scores 0, the output symbol is emitted when a
    token is entered.

    Standard: states 0..max_token (state i = "last symbol was i", 0 for blank) plus the
    final state; from every state an arc to every state j with label j (-1 into the
    final state) and aux label 0 on self-loops, else j.
    Modified: state 0 has a self-loop for every symbol and an arc to every token
    state; a token state has its self-loop and an arc back to state 0, both with
    aux label 0."""
    states = max_token + 2
    if modified:
        n0 = states - 1
        src = np.concatenate([np.zeros(2 * n0, np.int64), np.repeat(np.arange(1, states - 1), 2)])
        dest0 = np.arange(1, states)
        dest = np.concatenate([np.zeros(n0, np.int64), dest0,
                               np.stack([np.arange(1, states - 1),
                                         np.zeros(states - 2, np.int64)], 1).reshape(-1)])
        lab0 = np.where(dest0 == states - 1, -1, dest0)
        label = np.concatenate([np.arange(n0), lab0, np.repeat(np.arange(1, states - 1), 2)])
        aux = np.concatenate([np.arange(n0), lab0, np.zeros(2 * (states - 2), np.int64)])
    else:
        i, j = np.meshgrid(np.arange(states - 1), np.arange(states), indexing="ij")
        src, dest = i.reshape(-1), j.reshape(-1)
        label = np.where(dest == states - 1, -1, dest)
        aux = np.where(src == dest, 0, label)
    rows = np.stack([src, dest, label, np.zeros_like(src)], 1)
    rs2 = np.zeros(states + 1, np.int64)
    np.add.at(rs2, src + 1, 1)
    ans = _fsa_vec_from_numpy(np.asarray([0, states]), np.cumsum(rs2), rows, device or "cpu",
                              aux_labels=aux)
    ans.arcs.single = True
    return ans


def arc_sort(fsa: Fsa, ret_arc_map: bool = False):
    """Sort the arcs leaving each state by (label as uint32, dest_state)
    (k2/csrc/fsa.h:54-62, k2/csrc/fsa_algo.cu:852-867).  Graph preparation: runs
    on a host copy."""
    a = fsa.arcs
    v = a.values().cpu().numpy()
    rs2 = a._row_splits2.cpu().numpy()
    state = np.repeat(np.arange(a.num_states), np.diff(rs2))
    order = np.lexsort((v[:, 1], v[:, 2].astype(np.uint32), state)).astype(np.int32)
    dev = fsa.device
    arcs = RaggedArc(torch.from_numpy(np.ascontiguousarray(v[order])).to(dev), a._row_splits1,
                     a._row_splits2, single=a.single, h_row_splits1=a._h_row_splits1,
                     h_arc_splits=a._h_arc_splits)
    ans = Fsa(arcs)
    amap = torch.from_numpy(order).to(dev)
    for name, value in fsa.named_tensor_attr(include_scores=False):
        if name != 'labels':
            setattr(ans, name, index_select(value, amap))
    for name, value in fsa.named_non_tensor_attr():
        setattr(ans, name, value)
    return (ans, amap) if ret_arc_map else ans


def _shortest_path_arcs(fsa: Fsa, use_double_scores: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """(path_splits [num_fsas+1], best arc indexes in path order)."""
    arcs = fsa.arcs
    dev = arcs.device
    entering = fsa._get_entering_arcs(use_double_scores)
    nf = arcs.num_fsas
    path_splits = torch.empty(nf + 1, dtype=torch.int32, device=dev)
    best = torch.empty(max(arcs.num_states, 1), dtype=torch.int32, device=dev)
    tmp = torch.empty(_lib.lib.k2b200_shortest_path_tmp_bytes(nf), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib.k2b200_shortest_path(
            _lib.ptr(arcs._row_splits1), _lib.ptr(arcs.values()), _lib.ptr(entering), nf,
            _lib.ptr(path_splits), _lib.ptr(best), _lib.ptr(tmp), _lib.stream_of(dev)))
    total = int(path_splits[nf].item())
    return path_splits, best[:total]


def shortest_path(fsa: Fsa, use_double_scores: bool) -> Fsa:
    """Best path of each FSA in the tropical semiring (max), as linear FSAs; ties
    between equally good entering arcs go to the one with the higher arc index.
    Per-arc tensor attributes are carried along; `arc_map` of the result is kept
    in the attribute `_best_arc_map`."""
    path_splits, best = _shortest_path_arcs(fsa, use_double_scores)
    dev = fsa.device
    src_vals = fsa.arcs.values()
    n = best.numel()
    h_splits = path_splits.cpu().numpy().astype(np.int64)
    lens = np.diff(h_splits)
    # k2::FsaVecFromArcIndexes (k2/csrc/fsa_utils.cu:2079-2153): n arcs -> n+1 states
    nstates = np.where(lens > 0, lens + 1, 0)
    rs1 = np.zeros(len(lens) + 1, dtype=np.int64)
    np.cumsum(nstates, out=rs1[1:])
    pos_in_path = np.arange(n) - np.repeat(h_splits[:-1], lens)
    state_of_arc = np.repeat(rs1[:-1], lens) + pos_in_path
    rs2 = np.zeros(int(rs1[-1]) + 1, dtype=np.int64)
    np.add.at(rs2, state_of_arc + 1, 1)
    rs2 = np.cumsum(rs2)
    picked = src_vals[best.long()].clone()
    pos = torch.from_numpy(pos_in_path.astype(np.int32)).to(dev)
    picked[:, 0] = pos
    picked[:, 1] = pos + 1
    arcs = RaggedArc(picked.contiguous(), torch.from_numpy(rs1.astype(np.int32)).to(dev),
                     torch.from_numpy(rs2.astype(np.int32)).to(dev),
                     h_row_splits1=rs1.astype(np.int32),
                     h_arc_splits=rs2[rs1].astype(np.int32))
    ans = Fsa(arcs, _check=False)
    for name, value in fsa.named_tensor_attr(include_scores=False):
        if name != 'labels':
            setattr(ans, name, index_select(value, best))
    for name, value in fsa.named_non_tensor_attr():
        setattr(ans, name, value)
    ans._best_arc_map = best
    return ans

"""Seeded synthetic workloads with the shapes, sizes and value distributions of the
five benchmark configurations of this path.  No dataset is involved: logits are
Gaussian, transcripts and graphs are random.  Everything is generated on the host
from one `torch.Generator` / `numpy` seed so that every consumer (GPU path, CPU
checker, benchmark) sees identical bytes.

  ctc_small      N=8   T=200  C=500   targets 20..50,   standard CTC, beam 10
  ctc_large      N=64  T=1000 C=500   frames 600..1000, targets 100..250, beam 10
  ctc_modified   N=32  T=500  C=5000  targets 50..150,  modified CTC, beam 10
  lfmmi_den      N=128 T=500  C=72    one shared denominator graph (CTC topology
                 composed with a random phone bigram, 30 successors per phone), beam 8
  hlg_decode     N=32  T=500  C=500   random 200k-state / ~1.2M-arc decoding graph, beam 8
"""
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np
import torch


@dataclass
class Workload:
    name: str
    log_probs: torch.Tensor             # [N, T, C] float32, host
    supervision_segments: torch.Tensor  # [N, 3] int32 host, durations decreasing
    output_beam: float
    symbols: Optional[List[List[int]]] = None   # CTC transcripts (per utterance)
    modified: bool = False
    # explicit graph (one FSA, shared by every utterance): row_splits2, arcs [A,4]
    graph_row_splits2: Optional[np.ndarray] = None
    graph_arcs: Optional[np.ndarray] = None
    # LF-MMI: per-utterance transcripts of the numerator graphs (CTC graphs over phones)
    num_symbols: Optional[List[List[int]]] = None
    meta: Dict = field(default_factory=dict)

    @property
    def num_frames(self) -> int:
        return int(self.supervision_segments[:, 2].sum())


def _log_probs(gen: torch.Generator, n: int, t: int, c: int, sigma: float) -> torch.Tensor:
    logits = torch.randn(n, t, c, generator=gen, dtype=torch.float32) * sigma
    return torch.log_softmax(logits, dim=-1)


def _segments(durations: np.ndarray) -> torch.Tensor:
    order = np.argsort(-durations, kind="stable")
    seg = np.stack([order, np.zeros_like(order), durations[order]], axis=1).astype(np.int32)
    return torch.from_numpy(seg)


def _ctc_workload(name, seed, n, t, c, sigma, dur_lo, dur_hi, len_lo, len_hi, modified, beam):
    gen = torch.Generator().manual_seed(seed)
    log_probs = _log_probs(gen, n, t, c, sigma)
    lens = torch.randint(len_lo, len_hi + 1, (n,), generator=gen)
    symbols = [torch.randint(1, c, (int(l),), generator=gen).tolist() for l in lens]
    if dur_lo == dur_hi:
        durs = np.full(n, dur_hi, dtype=np.int64)
    else:
        durs = torch.randint(dur_lo, dur_hi + 1, (n,), generator=gen).numpy().astype(np.int64)
    seg = _segments(durs)
    # graph i pairs with supervision segment i: order transcripts like the segments
    symbols = [symbols[int(k)] for k in seg[:, 0].tolist()]
    return Workload(name, log_probs, seg, beam, symbols=symbols, modified=modified,
                    meta=dict(N=n, T=t, C=c))


def ctc_small(seed: int = 0, scale: float = 1.0) -> Workload:
    n, t = max(1, int(8 * scale)), max(8, int(200 * scale))
    return _ctc_workload("ctc_small", seed, n, t, 500, 1.0, t, t, max(1, int(20 * scale)),
                         max(2, int(50 * scale)), False, 10.0)


def ctc_large(seed: int = 0, scale: float = 1.0) -> Workload:
    n, t = max(1, int(64 * scale)), max(10, int(1000 * scale))
    return _ctc_workload("ctc_large", seed, n, t, 500, 1.5, max(6, int(600 * scale)), t,
                         max(1, int(100 * scale)), max(2, int(250 * scale)), False, 10.0)


def ctc_modified(seed: int = 0, scale: float = 1.0) -> Workload:
    n, t = max(1, int(32 * scale)), max(8, int(500 * scale))
    return _ctc_workload("ctc_modified", seed, n, t, 5000, 1.0, t, t, max(1, int(50 * scale)),
                         max(2, int(150 * scale)), True, 10.0)


def _arc_sort_rows(rows: np.ndarray) -> np.ndarray:
    """Sort [A,5] rows (src,dest,label,score,_) by (src, label as uint32, dest)."""
    order = np.lexsort((rows[:, 1], rows[:, 2].astype(np.int64) & 0xFFFFFFFF, rows[:, 0]))
    return rows[order]


def _pack_graph(rows_src, rows_dest, rows_label, rows_score, num_states):
    src = np.asarray(rows_src, dtype=np.int64)
    dest = np.asarray(rows_dest, dtype=np.int64)
    label = np.asarray(rows_label, dtype=np.int64)
    score = np.asarray(rows_score, dtype=np.float32)
    order = np.lexsort((dest, label & 0xFFFFFFFF, src))
    arcs = np.zeros((len(src), 4), dtype=np.int32)
    arcs[:, 0] = src[order]
    arcs[:, 1] = dest[order]
    arcs[:, 2] = label[order]
    arcs[:, 3] = score[order].view(np.int32)
    rs2 = np.zeros(num_states + 1, dtype=np.int64)
    np.add.at(rs2, src + 1, 1)
    return np.cumsum(rs2).astype(np.int32), arcs


def den_graph(seed: int = 0, num_phones: int = 71, successors: int = 30):
    """CTC topology over blank + `num_phones` phones composed with a random phone
    bigram, built directly in composed form.  States: (history h, in blank) for
    h = 0..P (h = 0: nothing emitted yet), (h, in phone) for h = 1..P, and one
    final state: 2P + 2 states.  From (h, blank): blank self-loop, every successor
    q of h with the bigram weight, and the final arc.  From (h, phone): self-loop on
    h, blank to (h, blank), every successor q != h directly, and the final arc.
    Each history has `successors` successors drawn without replacement and
    log-softmax weights over them and the final arc.  The result is arc-sorted."""
    rng = np.random.default_rng(seed)
    P = num_phones
    blank_state = lambda h: h                  # 0..P          # noqa: E731
    phone_state = lambda h: P + h              # P+1..2P (h>=1) # noqa: E731
    final = 2 * P + 1
    src, dest, label, score = [], [], [], []
    for h in range(P + 1):
        succ = rng.permutation(P)[:successors] + 1
        w = rng.normal(size=successors + 1)
        w = (w - np.log(np.exp(w).sum())).astype(np.float32)
        froms = [(blank_state(h), True)] + ([(phone_state(h), False)] if h >= 1 else [])
        for s, in_blank in froms:
            if in_blank:
                src.append(s); dest.append(s); label.append(0); score.append(0.0)
            else:
                src.append(s); dest.append(s); label.append(h); score.append(0.0)
                src.append(s); dest.append(blank_state(h)); label.append(0); score.append(0.0)
            for q, wq in zip(succ.tolist(), w[:-1].tolist()):
                if not in_blank and q == h:
                    continue  # a repeated phone needs the blank in between
                src.append(s); dest.append(phone_state(q)); label.append(q); score.append(wq)
            src.append(s); dest.append(final); label.append(-1); score.append(float(w[-1]))
    return _pack_graph(src, dest, label, score, final + 1)


def lfmmi_den(seed: int = 0, scale: float = 1.0, utterances: Optional[int] = None) -> Workload:
    """`utterances` overrides the batch size alone (e.g. 16: one GPU's share of the
    batch of 128 split eight ways)."""
    n, t = max(1, int(128 * scale)), max(8, int(500 * scale))
    if utterances is not None:
        n = utterances
    gen = torch.Generator().manual_seed(seed)
    log_probs = _log_probs(gen, n, t, 72, 1.0)
    seg = _segments(np.full(n, t, dtype=np.int64))
    rs2, arcs = den_graph(seed)
    # numerator graphs: CTC graphs of random phone strings of 40..100 phones (tokens 1..71),
    # drawn after the log-probs so that those keep their bytes
    lens = torch.randint(max(1, int(40 * scale)), max(2, int(100 * scale)) + 1, (n,), generator=gen)
    num_symbols = [torch.randint(1, 72, (int(l),), generator=gen).tolist() for l in lens]
    return Workload("lfmmi_den", log_probs, seg, 8.0, graph_row_splits2=rs2, graph_arcs=arcs,
                    num_symbols=num_symbols,
                    meta=dict(N=n, T=t, C=72, graph_states=len(rs2) - 1, graph_arcs=len(arcs)))


def decoding_graph(seed: int = 0, num_states: int = 200000, num_classes: int = 500,
                   eps_frac: float = 0.05, final_frac: float = 0.002):
    """Random HLG-like graph: out-degree Poisson(5)+1, labels uniform in
    0..C-1 with a share forced to epsilon, weights -Exp(1).  State s has an arc
    to s+1 (so every state is reachable from state 0 and can reach the single
    final state), the other arcs go to random non-final states, and a few states
    carry a final arc.  Arc-sorted."""
    rng = np.random.default_rng(seed)
    S = num_states
    final = S - 1
    deg = rng.poisson(5.0, size=S - 1) + 1
    src = np.repeat(np.arange(S - 1, dtype=np.int64), deg)
    A = len(src)
    first = np.zeros(A, dtype=bool)
    starts = np.cumsum(deg) - deg
    first[starts] = True
    dest = rng.integers(0, S - 1, size=A)
    dest[first] = src[first] + 1
    label = rng.integers(1, num_classes, size=A)
    label[rng.random(A) < eps_frac] = 0
    is_final_arc = dest == final
    extra = (rng.random(A) < final_frac) & ~first
    dest[extra] = final
    is_final_arc |= extra
    label[is_final_arc] = -1
    score = (-rng.exponential(1.0, size=A)).astype(np.float32)
    return _pack_graph(src, dest, label, score, S)


def hlg_decode(seed: int = 0, scale: float = 1.0, num_states: Optional[int] = None) -> Workload:
    n, t = max(1, int(32 * scale)), max(8, int(500 * scale))
    if num_states is None:
        num_states = max(50, int(200000 * scale))
    gen = torch.Generator().manual_seed(seed)
    log_probs = _log_probs(gen, n, t, 500, 2.0)
    seg = _segments(np.full(n, t, dtype=np.int64))
    rs2, arcs = decoding_graph(seed, num_states, 500)
    return Workload("hlg_decode", log_probs, seg, 8.0, graph_row_splits2=rs2, graph_arcs=arcs,
                    meta=dict(N=n, T=t, C=500, graph_states=len(rs2) - 1, graph_arcs=len(arcs)))


def num_den_graphs(w: Workload):
    """Host arrays of the LF-MMI graph pair set of a workload: for every utterance its
    numerator graph (the CTC graph of its phone string) followed by the shared
    denominator graph - 2N graphs [num_0, den_0, num_1, den_1, ...] that go with
    a_to_b_map = [0, 0, 1, 1, ...], both graphs of an utterance reading the same rows of
    the dense scores (k2/csrc/intersect_dense.cu:80-92).  Returns (row_splits1,
    row_splits2, arcs [A, 4], a_to_b_map)."""
    assert w.num_symbols is not None and w.graph_arcs is not None
    n = w.supervision_segments.shape[0]
    den_rs2 = np.asarray(w.graph_row_splits2, dtype=np.int64)
    den_arcs = np.asarray(w.graph_arcs, dtype=np.int32)
    rs1, rs2, arcs = [0], [0], []

    def append(g_rs2, g_arcs):
        rs2.extend((g_rs2[1:] + rs2[-1]).tolist())
        arcs.append(g_arcs)
        rs1.append(rs1[-1] + len(g_rs2) - 1)

    from .fsa_algo import ctc_graph
    num = ctc_graph(w.num_symbols, modified=False, device="cpu").arcs
    n_rs1 = np.asarray(num.h_row_splits1, dtype=np.int64)
    n_rs2 = num.row_splits(2).numpy().astype(np.int64)
    n_arcs = num.values().numpy()
    for i in range(n):
        s0, s1 = int(n_rs1[i]), int(n_rs1[i + 1])
        a0, a1 = int(n_rs2[s0]), int(n_rs2[s1])
        append(n_rs2[s0:s1 + 1] - a0, n_arcs[a0:a1])
        append(den_rs2, den_arcs)
    a_to_b_map = np.repeat(np.arange(n, dtype=np.int32), 2)
    return (np.asarray(rs1, dtype=np.int32), np.asarray(rs2, dtype=np.int32),
            np.concatenate(arcs), a_to_b_map)


WORKLOADS = {
    "ctc_small": ctc_small,
    "ctc_large": ctc_large,
    "ctc_modified": ctc_modified,
    "lfmmi_den": lfmmi_den,
    "hlg_decode": hlg_decode,
}


def build_graphs(w: Workload, device="cpu"):
    """The a_fsas FsaVec of a workload: per-utterance CTC graphs, or the shared
    graph replicated once per utterance (the reference cannot share a graph
    across sequences in intersect_dense, k2/csrc/intersect_dense.cu:75-93)."""
    from .fsa_algo import _fsa_vec_from_numpy, ctc_graph
    if w.symbols is not None:
        return ctc_graph(w.symbols, modified=w.modified, device=device)
    n = w.supervision_segments.shape[0]
    S = len(w.graph_row_splits2) - 1
    A = len(w.graph_arcs)
    rs1 = np.arange(n + 1, dtype=np.int64) * S
    rs2 = (np.arange(n, dtype=np.int64)[:, None] * A + w.graph_row_splits2[None, :-1]).reshape(-1)
    rs2 = np.append(rs2, n * A)
    arcs = np.tile(w.graph_arcs, (n, 1))
    return _fsa_vec_from_numpy(rs1, rs2, arcs, device)

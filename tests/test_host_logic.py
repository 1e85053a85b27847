"""Host-side logic without a GPU: graph construction, DenseFsaVec layout, text
format, sharding, and the C-ABI library's exported symbols."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import k2_b200 as k2
from k2_b200 import parallel
from k2_b200 import synthetic as syn
from oracle import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "k2b200.h")).read()
    declared = sorted(set(re.findall(r"\b(k2b200_[a-z0-9_]+)\s*\(", header)))
    assert len(declared) >= 25
    lib = ctypes.CDLL(os.path.join(ROOT, "k2_b200", "libk2b200.so"))
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/k2b200.h but not exported"
    from k2_b200 import _lib
    assert sorted(_lib.EXPORTED) == [d for d in declared if d in _lib.EXPORTED]
    assert set(declared) == set(_lib.EXPORTED)
    assert lib.k2b200_abi_version() == 5


def test_no_cpu_path():
    g = k2.ctc_graph([[1, 2]])
    lp = torch.log_softmax(torch.randn(1, 4, 5), -1)
    dense = k2.DenseFsaVec(lp, torch.tensor([[0, 0, 4]], dtype=torch.int32))
    with pytest.raises(RuntimeError, match="CUDA"):
        k2.intersect_dense(g, dense, 10.0)


def test_ctc_graph_matches_oracle():
    rng = np.random.default_rng(0)
    for modified in (False, True):
        for _ in range(30):
            syms = [[int(x) for x in rng.integers(1, 5, size=int(rng.integers(0, 7)))]
                    for _ in range(int(rng.integers(1, 6)))]
            g = k2.ctc_graph(syms, modified=modified)
            o = oracle.ctc_graphs(syms, modified)
            assert np.array_equal(g.arcs.values().numpy(), o.arcs)
            assert np.array_equal(g.arcs.row_splits(1).numpy(), o.row_splits1)
            assert np.array_equal(g.arcs.row_splits(2).numpy(), o.row_splits2)
            assert np.array_equal(g.aux_labels.numpy(), o.aux_labels)
            assert g.properties == oracle.properties(o)[1]


def test_dense_fsa_vec_layout():
    # k2/python/tests/dense_fsa_vec_test.py:41-127
    lp = torch.arange(2 * 4 * 3, dtype=torch.float32).reshape(2, 4, 3)
    seg = torch.tensor([[1, 0, 4], [0, 1, 2]], dtype=torch.int32)
    d = k2.DenseFsaVec(lp, seg)
    assert d.scores.shape == (4 + 1 + 2 + 1, 4)
    assert d.h_row_splits.tolist() == [0, 5, 8]
    assert d.duration.tolist() == [4, 2]
    assert torch.equal(d.scores[0:4, 1:], lp[1])
    assert torch.equal(d.scores[5:7, 1:], lp[0, 1:3])
    inf = float("inf")
    assert d.scores[4].tolist() == [0, -inf, -inf, -inf]
    assert d.scores[7].tolist() == [0, -inf, -inf, -inf]
    assert torch.all(d.scores[[0, 1, 2, 3, 5, 6], 0] == -inf)
    # allow_truncate
    d2 = k2.DenseFsaVec(lp, torch.tensor([[0, 2, 4]], dtype=torch.int32), allow_truncate=2)
    assert d2.duration.tolist() == [2]


def test_from_str_and_properties():
    f = k2.Fsa.from_str("0 1 1 0.5\n0 1 2 1.5\n1 2 -1 0.25\n2")
    assert f.shape == (3, None) and f.num_arcs == 3
    assert f.scores.tolist() == [0.5, 1.5, 0.25] and f.labels.tolist() == [1, 2, -1]
    assert f.properties & k2.fsa.VALID and f.properties & k2.fsa.ARC_SORTED
    t = k2.Fsa.from_str("0 1 1 10 0.5\n1 2 -1 -1 0.25\n2", num_aux_labels=1)
    assert t.aux_labels.tolist() == [10, -1]
    with pytest.raises(ValueError):
        k2.Fsa.from_str("0 1 -1 0.5\n1 2 -1 0.25\n2")  # -1 on an arc not entering the final state
    v = k2.create_fsa_vec([f, f])
    assert v.shape == (2, None, None) and v.arcs.row_splits(1).tolist() == [0, 3, 6]
    s = k2.arc_sort(k2.Fsa.from_str("0 1 2 0.5\n0 1 1 1.5\n1 2 -1 0.25\n2"))
    assert s.labels.tolist() == [1, 2, -1]


def test_synthetic_workloads_are_deterministic_and_valid():
    w1, w2 = syn.ctc_small(), syn.ctc_small()
    assert torch.equal(w1.log_probs, w2.log_probs) and w1.symbols == w2.symbols
    assert w1.supervision_segments[:, 2].tolist() == sorted(
        w1.supervision_segments[:, 2].tolist(), reverse=True)
    g = syn.build_graphs(w1)
    assert g.num_arcs == 1325 and g.arcs.num_states == 540
    big = syn.ctc_large(scale=0.1)
    d = big.supervision_segments[:, 2].tolist()
    assert d == sorted(d, reverse=True)
    rs2, arcs = syn.den_graph(0)
    assert len(rs2) - 1 == 144 and 4500 < len(arcs) < 4700
    den = syn.build_graphs(syn.lfmmi_den(scale=0.02))
    assert den.properties & k2.fsa.ARC_SORTED_AND_DETERMINISTIC
    hlg = syn.build_graphs(syn.hlg_decode(scale=0.02, num_states=500))
    assert hlg.properties & k2.fsa.VALID and hlg.properties & k2.fsa.ACCESSIBLE


def test_shard_utterances_balances_and_keeps_order():
    durs = [1000, 990, 800, 750, 700, 650, 600, 600]
    seen = []
    for rank in range(4):
        idx = parallel.shard_utterances(durs, 4, rank)
        d = [durs[i] for i in idx]
        assert d == sorted(d, reverse=True)
        seen.extend(idx.tolist())
    assert sorted(seen) == list(range(8))
    seg = torch.tensor([[i, 0, d] for i, d in enumerate(durs)], dtype=torch.int32)
    mine, idx = parallel.shard_segments(seg, 2, 1)
    assert mine[:, 2].tolist() == [990, 750, 650, 600]


def _host_args(num_states_per, num_arcs_per, n, rows_per, cols, max_degree, sorted_ok=True,
               shared=0):
    """A k2b200_intersect_args block whose device pointers are never dereferenced:
    the sizing / validation entry points only read the host arrays."""
    import ctypes
    from k2_b200 import _lib
    rs1 = (np.arange(n + 1) * num_states_per).astype(np.int32)
    asp = (np.arange(n + 1) * num_arcs_per).astype(np.int32)
    lens = np.full(n, rows_per, np.int32)
    if not sorted_ok:
        lens[-1] += 3
    brs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    fake = 256  # any non-NULL address
    args = _lib.IntersectArgs(
        num_fsas=n, num_states=int(rs1[-1]), num_arcs=int(asp[-1]), a_row_splits1=fake,
        a_row_splits2=fake, a_arcs=fake, a_in_splits=fake, a_in_arcs=fake,
        h_a_row_splits1=rs1.ctypes.data, h_a_arc_splits=asp.ctypes.data, scores=fake,
        rows=int(brs[-1]), cols=cols, num_seqs=n, h_b_row_splits=brs.ctypes.data,
        h_a_to_b_map=None, output_beam=10.0, max_states=15000000, max_arcs=1 << 30,
        viterbi_mode=0, a_max_degree=max_degree, a_shared=shared)
    return args, (rs1, asp, brs)


def test_workspace_sizing_and_validation_need_no_gpu():
    import ctypes
    from k2_b200 import _lib
    lib = _lib.lib
    # a CTC-sized problem: the loss workspace holds the intersect workspace plus the
    # packed matrix and the alpha / beta grids
    args, keep = _host_args(101, 250, 8, 201, 501, 3)
    b1, b2, lv = ctypes.c_size_t(), ctypes.c_size_t(), ctypes.c_int64()
    assert lib.k2b200_intersect_dense_workspace_bytes(ctypes.byref(args), ctypes.byref(b1),
                                                      ctypes.byref(lv)) == 0
    assert lv.value == 8 * 202
    assert lib.k2b200_dense_loss_workspace_bytes(ctypes.byref(args), ctypes.byref(b2)) == 0
    grid = 8 * 202 * 101
    pack = 8 * 201 * (4 * 504 + 8 * 502)
    assert b2.value >= b1.value + pack + 2 * 16 * grid
    ok = ctypes.c_int32()
    assert lib.k2b200_dense_loss_supported(ctypes.byref(args), ctypes.byref(ok)) == 0 and ok.value == 1
    # a 200 000-state graph is not for the lattice-free path
    big, keep2 = _host_args(200000, 600000, 2, 101, 501, 12)
    assert lib.k2b200_dense_loss_supported(ctypes.byref(big), ctypes.byref(ok)) == 0 and ok.value == 0
    # sequences must be sorted by decreasing length (intersect_dense.cu:168-177)
    bad, keep3 = _host_args(101, 250, 4, 201, 501, 3, sorted_ok=False)
    assert lib.k2b200_dense_loss_workspace_bytes(ctypes.byref(bad), ctypes.byref(b2)) != 0
    assert b"sorted order" in lib.k2b200_last_error()
    # a_shared with graphs of different sizes is refused
    sh, keep4 = _host_args(50, 120, 3, 51, 73, 9, shared=1)
    keep4[0][3] += 1  # last graph has one more state
    sh.num_states += 1
    assert lib.k2b200_intersect_dense_workspace_bytes(ctypes.byref(sh), ctypes.byref(b1),
                                                      ctypes.byref(lv)) != 0
    assert b"a_shared" in lib.k2b200_last_error()


def test_pruned_intersection_sizing_and_validation_need_no_gpu():
    import ctypes
    from k2_b200 import _lib
    lib = _lib.lib
    brs = np.array([0, 101, 181, 232], np.int32)

    def args(**kw):
        base = dict(num_fsas=1, num_states=5000, num_arcs=30000, rows=232, cols=41, num_seqs=3,
                    h_b_row_splits=brs.ctypes.data, search_beam=20.0, output_beam=8.0,
                    min_active_states=30, max_active_states=10000, allow_partial=0,
                    max_states_per_seq=1 << 15, max_arcs_per_seq=1 << 16)
        base.update(kw)
        return _lib.PrunedArgs(**base)

    nbytes, levels = ctypes.c_size_t(), ctypes.c_int64()
    a = args()
    assert lib.k2b200_intersect_dense_pruned_workspace_bytes(
        ctypes.byref(a), ctypes.byref(nbytes), ctypes.byref(levels)) == 0
    # layers: (longest sequence's rows + 2) per sequence
    assert levels.value == 3 * (101 + 2)
    # 17 bytes per arc, 24 per state, one 8-byte table entry per (sequence, graph state)
    arenas = 3 * (17 * (1 << 16) + 24 * ((1 << 15) + 1))
    assert arenas + 3 * 5000 * 8 <= nbytes.value <= arenas + 3 * 5000 * 8 + (1 << 16)
    for bad, msg in ((dict(search_beam=0.0), b"positive"),
                     (dict(min_active_states=10, max_active_states=10), b"min_active_states"),
                     (dict(num_fsas=2), b"one graph per sequence"),
                     (dict(rows=233), b"do not cover"),
                     (dict(max_arcs_per_seq=0), b"capacities")):
        a = args(**bad)
        assert lib.k2b200_intersect_dense_pruned_workspace_bytes(
            ctypes.byref(a), ctypes.byref(nbytes), ctypes.byref(levels)) != 0
        assert msg in lib.k2b200_last_error(), (bad, lib.k2b200_last_error())


def test_ragged_attribute_tensor_on_cpu():
    """RaggedTensor.index / remove_values_leq / cat against plain Python lists
    (k2.RaggedTensor semantics: an index of -1 gives an empty list)."""
    import torch
    from k2_b200.ragged_tensor import RaggedTensor, cat
    rng = np.random.default_rng(4)
    rows = [[int(x) for x in rng.integers(-1, 9, size=int(rng.integers(0, 5)))] for _ in range(40)]
    r = RaggedTensor(rows)
    assert r.tolist() == rows and r.dim0 == 40 and r.numel() == sum(map(len, rows))
    idx = rng.integers(-1, 40, size=100).astype(np.int32)
    out, pos = r.index(torch.from_numpy(idx), need_value_indexes=True)
    assert out.tolist() == [rows[i] if i >= 0 else [] for i in idx]
    assert torch.equal(r.values[pos.long()], out.values)
    assert r.remove_values_leq(0).tolist() == [[x for x in row if x > 0] for row in rows]
    assert cat([r, out]).tolist() == rows + out.tolist()
    assert r.clone() == r and RaggedTensor([[1], []]) != RaggedTensor([[1]])


def test_numa_binding_is_a_no_op_without_a_gpu_topology():
    import os
    from k2_b200.parallel import bind_to_gpu_numa_node
    before = os.sched_getaffinity(0)
    info = bind_to_gpu_numa_node("cuda:0")
    assert info["bound"] is False or os.sched_getaffinity(0) <= before
    if not info["bound"]:
        assert os.sched_getaffinity(0) == before


def test_online_decoding_sizing_and_validation_need_no_gpu():
    import ctypes
    from k2_b200 import _lib
    lib = _lib.lib
    brs = (np.arange(4) * 9).astype(np.int32)       # three streams, 8 frames + final row
    hist = np.array([0, 24, 8], np.int32)

    def args(**kw):
        base = dict(num_states=500, num_arcs=3000, rows=27, cols=41, num_seqs=3,
                    h_b_row_splits=brs.ctypes.data, search_beam=20.0, output_beam=8.0,
                    min_active_states=30, max_active_states=10000, allow_partial=1,
                    h_hist=hist.ctypes.data, max_states_per_seq=1 << 12,
                    max_arcs_per_seq=1 << 13, team_ctas=0)
        base.update(kw)
        return _lib.OnlineArgs(**base)

    nbytes = ctypes.c_size_t()
    a = args()
    assert lib.k2b200_online_decode_workspace_bytes(ctypes.byref(a), ctypes.byref(nbytes)) == 0
    arenas = 3 * (17 * (1 << 13) + 24 * ((1 << 12) + 1))
    assert nbytes.value >= arenas + 3 * 500 * 8 + 2 * 3 * (24 + 8 + 2) * 4
    uneven = np.array([0, 9, 17, 26], np.int32)
    for bad, msg in ((dict(h_b_row_splits=uneven.ctypes.data, rows=26), b"same number of frames"),
                     (dict(search_beam=-1.0), b"positive")):
        a = args(**bad)
        assert lib.k2b200_online_decode_workspace_bytes(ctypes.byref(a),
                                                        ctypes.byref(nbytes)) != 0
        assert msg in lib.k2b200_last_error(), (bad, lib.k2b200_last_error())


def test_splits_of_the_device_ctc_graphs_match_the_host_builder():
    # the CUDA ctc_graph sizes its outputs from host prefix sums over the flat symbols; the
    # host builder writes the same graphs arc by arc
    import itertools
    from k2_b200 import fsa_algo
    rng = np.random.default_rng(0)
    for trial in range(200):
        n = int(rng.integers(1, 8))
        symbols = [rng.integers(1, 4, size=int(rng.integers(0, 7))).tolist() for _ in range(n)]
        if trial % 10 == 0:
            symbols = [[] for _ in range(n)]
        lens = np.fromiter(map(len, symbols), dtype=np.int64, count=n)
        sym = np.fromiter(itertools.chain.from_iterable(symbols), dtype=np.int64,
                          count=int(lens.sum()))
        for modified in (False, True):
            arcs = fsa_algo.ctc_graph(symbols, modified=modified, device="cpu").arcs
            sym_off, rs1, arc_splits = fsa_algo._ctc_graph_splits(lens, sym, modified)
            want_rs1 = np.asarray(arcs.h_row_splits1)
            assert np.array_equal(sym_off[1:], np.cumsum(lens))
            assert np.array_equal(rs1, want_rs1), symbols
            assert np.array_equal(arc_splits, arcs._row_splits2.numpy()[want_rs1]), symbols

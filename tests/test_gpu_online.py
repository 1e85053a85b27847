"""Chunk-by-chunk decoding (k2.OnlineDenseIntersecter) on the GPU against the
reference's own OnlineDenseIntersecter run on the CPU, chunk after chunk: lattices and
arc maps bit-identical, search beams equal."""
import numpy as np
import pytest
import torch

from oracle import ref
from oracle.common import HostFsaVec
from pruned_util import decoding_graph

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref.available(), reason="oracle/_ref/libk2ref.so not built")]


@pytest.fixture(scope="module")
def k2():
    import k2_b200
    return k2_b200


def chunk_scores(rng, n, frames, classes, scale=1.0):
    sc = np.full((n * (frames + 1), classes + 1), -np.inf, np.float32)
    for i in range(n):
        x = (rng.normal(size=(frames, classes)) * scale).astype(np.float32)
        x -= np.log(np.exp(x).sum(-1, keepdims=True))
        sc[i * (frames + 1):i * (frames + 1) + frames, 1:] = x
        sc[i * (frames + 1) + frames, 0] = 0
    return sc, (np.arange(n + 1) * (frames + 1)).astype(np.int32)


def run_both(k2, graph: HostFsaVec, params, schedule, frames, classes, seed, scale=1.0,
             small_arena=False):
    """schedule: per chunk, the list of stream ids in the batch (new ids start streams)."""
    from gpu_util import DEV, dense_from_scores, fsa_to_host, host_to_fsa
    rng = np.random.default_rng(seed)
    n = len(schedule[0])
    theirs = ref.OnlineIntersecter(graph, n, *params)
    g = host_to_fsa(graph)
    ours = k2.OnlineDenseIntersecter(g, n, *params)
    if small_arena:
        ours._arcs_per_seq = 8  # every chunk overflows first and is retried
    their_streams, our_streams = {}, {}
    for k, ids in enumerate(schedule):
        sc, brs = chunk_scores(rng, n, frames, classes, scale)
        want, new_theirs = theirs.decode(sc, brs, [their_streams.get(i) for i in ids])
        lat, new_ours = ours.decode(dense_from_scores(sc, brs), [our_streams.get(i) for i in ids])
        got = fsa_to_host(lat, lat._arc_map_a)
        assert np.array_equal(got.row_splits1, want.row_splits1), f"chunk {k}: row_splits1"
        assert np.array_equal(got.row_splits2, want.row_splits2), f"chunk {k}: row_splits2"
        assert np.array_equal(got.arcs, want.arcs), f"chunk {k}: arcs"
        assert np.array_equal(got.arc_map_a, want.arc_map_a), f"chunk {k}: arc_map_a"
        for i, a, b in zip(ids, new_theirs, new_ours):
            their_streams[i], our_streams[i] = a, b
            assert ref.OnlineIntersecter.beam(a) == np.float32(b.beam), f"chunk {k}: beam"
    return lat


def test_streams_that_start_together(k2):
    topo = ref.ctc_topo(5, False)
    for params in ((10.0, 2.0, 1, 10, True), (20.0, 8.0, 0, 1000, True), (4.0, 3.0, 2, 6, False)):
        run_both(k2, topo, params, [[0, 1]] * 4, frames=5, classes=6, seed=1)
    rng = np.random.default_rng(3)
    g = decoding_graph(rng, 300, 9, mean_degree=3.0)
    run_both(k2, g, (8.0, 4.0, 5, 60, True), [[0, 1, 2]] * 5, frames=16, classes=9, seed=2,
             scale=2.0)
    lat = run_both(k2, g, (8.0, 4.0, 5, 60, True), [[0, 1, 2]] * 3, frames=16, classes=9, seed=2,
                   scale=2.0, small_arena=True)
    assert lat.arcs.num_elements() > 100
    # more streams than SMs / 2: one CTA per stream
    run_both(k2, g, (6.0, 3.0, 2, 30, True), [list(range(90))] * 2, frames=5, classes=9, seed=7)


def test_streams_that_join_and_leave(k2):
    """Streams of different ages in one batch: the reference aligns them at their ends,
    so the pruning window of a young stream starts inside it."""
    topo = ref.ctc_topo(5, False)
    schedule = [[0, 1], [0, 2], [3, 2], [3, 0], [1, 0], [4, 1]]
    for params in ((10.0, 2.0, 1, 10, True), (6.0, 4.0, 0, 50, True)):
        run_both(k2, topo, params, schedule, frames=4, classes=6, seed=5)
    rng = np.random.default_rng(4)
    g = decoding_graph(rng, 200, 8, mean_degree=3.0)
    run_both(k2, g, (8.0, 4.0, 5, 40, True), [[0, 1, 2], [3, 1, 2], [3, 4, 2], [0, 4, 1]],
             frames=7, classes=8, seed=6, scale=2.0)


def test_text_of_the_best_path_grows_with_the_chunks(k2):
    """Decoding peaked log-probs chunk by chunk gives the symbols seen so far."""
    from gpu_util import DEV
    C = 8
    H = k2.ctc_topo(C - 1, device=DEV)
    H = k2.create_fsa_vec([H])
    text = [3, 5, 5, 1, 7, 2]
    frames = []
    for sym in text:
        frames += [0, sym, sym]
    T = len(frames)
    logits = torch.full((1, T, C), -6.0)
    for t, sym in enumerate(frames):
        logits[0, t, sym] = 6.0
    log_prob = torch.log_softmax(logits, -1)
    dec = k2.OnlineDenseIntersecter(H, 1, 20.0, 8.0, 0, 1000)
    states = [k2.DecodeStateInfo()]  # as the reference's own test starts its streams
    chunk = 6
    for k in range(T // chunk):
        lp = log_prob[:, k * chunk:(k + 1) * chunk].contiguous().to(DEV)
        dense = k2.DenseFsaVec(lp, torch.tensor([[0, 0, chunk]], dtype=torch.int32))
        lat, states = dec.decode(dense, states)
        got = k2.get_aux_labels(k2.one_best_decoding(lat))
        assert got == [text[:2 * (k + 1)]], (k, got)

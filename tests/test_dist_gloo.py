"""World-size-2 checks of the multi-GPU plumbing on CPU (gloo): every rank takes its
shard of the utterances, and the single all-reduce of [loss, frames] gives every
rank the totals of the whole batch - with a stand-in loss, with the CPU checker's CTC
loss of each shard, and with a rank that fails before the collective."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, durations, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from k2_b200 import parallel
    idx = parallel.shard_utterances(durations, world, rank)
    frames = int(sum(durations[i] for i in idx))
    # stand-in for the per-rank loss: a deterministic function of the shard
    loss = torch.tensor(float(sum((i + 1) * durations[i] for i in idx)), dtype=torch.float64)
    tot_loss, tot_frames = parallel.all_reduce_loss(loss, frames)
    np.save(os.path.join(out_dir, f"r{rank}.npy"),
            np.array([float(tot_loss), tot_frames] + idx.tolist(), dtype=np.float64))
    dist.destroy_process_group()


def test_two_rank_shard_and_all_reduce(tmp_path):
    durations = [900, 850, 700, 640, 600]
    port = _free_port()
    mp.spawn(_worker, args=(2, port, durations, str(tmp_path)), nprocs=2, join=True)
    r0 = np.load(tmp_path / "r0.npy")
    r1 = np.load(tmp_path / "r1.npy")
    want_loss = float(sum((i + 1) * d for i, d in enumerate(durations)))
    assert r0[0] == r1[0] == want_loss
    assert r0[1] == r1[1] == sum(durations)
    assert sorted(r0[2:].tolist() + r1[2:].tolist()) == [0, 1, 2, 3, 4]


def _loss_worker(rank, world, port, out_dir):
    """Each rank runs the path (here: the CPU checker) on its shard of one batch."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from k2_b200 import parallel
    from k2_b200 import synthetic as syn
    from oracle import oracle
    w = syn.ctc_small(scale=0.25)
    seg, idx = parallel.shard_segments(w.supervision_segments, world, rank)
    assert seg[:, 2].tolist() == sorted(seg[:, 2].tolist(), reverse=True)
    loss, frames = _oracle_loss(w, oracle, idx)
    tot_loss, tot_frames = parallel.all_reduce_loss(torch.tensor(loss, dtype=torch.float64),
                                                    frames)
    np.save(os.path.join(out_dir, f"l{rank}.npy"), np.array([float(tot_loss), tot_frames]))
    dist.destroy_process_group()


def _oracle_loss(w, oracle, idx):
    """CTC loss (negated log-semiring total scores) of utterances `idx` of a workload."""
    seg = w.supervision_segments.numpy()[idx]
    lp = w.log_probs.numpy()
    C = lp.shape[2]
    rows = int(seg[:, 2].sum() + len(seg))
    scores = np.full((rows, C + 1), -np.inf, np.float32)
    brs = np.zeros(len(seg) + 1, np.int32)
    r = 0
    for i, (n, s, d) in enumerate(seg.tolist()):
        scores[r:r + d, 1:] = lp[n, s:s + d]
        scores[r + d, 0] = 0.0
        r += d + 1
        brs[i + 1] = r
    graphs = oracle.ctc_graphs([w.symbols[int(k)] for k in idx], w.modified)
    out = oracle.loss_path(graphs, scores, brs, w.output_beam)
    return float(-out["tot_scores"].sum()), int(seg[:, 2].sum())


def test_sharded_loss_equals_the_loss_of_the_whole_batch(tmp_path):
    from k2_b200 import synthetic as syn
    from oracle import oracle
    port = _free_port()
    mp.spawn(_loss_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    w = syn.ctc_small(scale=0.25)
    want, frames = _oracle_loss(w, oracle, np.arange(w.supervision_segments.shape[0]))
    for r in range(2):
        got = np.load(tmp_path / f"l{r}.npy")
        assert abs(got[0] - want) <= 1e-9 * abs(want), (got, want)
        assert got[1] == frames


def _failing_worker(rank, world, port, out_dir):
    """Rank 1 fails on the host before the collective; rank 0 must get an error from
    its all-reduce within the group's timeout instead of waiting for ever."""
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=5))
    from k2_b200 import parallel
    if rank == 1:
        os._exit(3)  # a rank that dies between steps, no collective in flight
    t0 = time.time()
    try:
        parallel.all_reduce_loss(torch.tensor(1.0, dtype=torch.float64), 10)
        outcome = "returned"
    except Exception as e:  # noqa: BLE001 - any error from the collective is the point
        outcome = "error:" + type(e).__name__
    with open(os.path.join(out_dir, "outcome.txt"), "w") as f:
        f.write(f"{outcome} {time.time() - t0:.1f}")


def test_a_rank_that_dies_before_the_all_reduce_gives_an_error_not_a_hang(tmp_path):
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, str(tmp_path)))
             for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
    assert not any(p.is_alive() for p in procs), "a rank is still waiting"
    assert procs[1].exitcode == 3
    outcome, seconds = open(tmp_path / "outcome.txt").read().split()
    assert outcome.startswith("error:"), outcome
    assert float(seconds) < 60


def _reducer_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from k2_b200 import parallel
    reducer = parallel.LossReducer("cpu")
    got = []
    for step in range(3):
        loss = torch.tensor(float(10 * step + rank + 1))
        reducer.submit(loss, 100 * (rank + 1) + step)
        tot_loss, tot_frames = reducer.result()
        got += [float(tot_loss), float(tot_frames)]
    reducer.close()
    np.save(os.path.join(out_dir, f"q{rank}.npy"), np.array(got))
    dist.destroy_process_group()


def test_loss_reducer_thread(tmp_path):
    """The helper-thread all-reduce gives every rank the totals of every step."""
    port = _free_port()
    mp.spawn(_reducer_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "q0.npy"), np.load(tmp_path / "q1.npy")
    want = []
    for step in range(3):
        want += [float(20 * step + 3), float(300 + 2 * step)]
    assert r0.tolist() == r1.tolist() == want

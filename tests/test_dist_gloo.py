"""World-size-2 check of the multi-GPU plumbing on CPU (gloo): every rank takes its
shard of the utterances, and the single all-reduce of [loss, frames] gives every
rank the totals of the whole batch."""
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

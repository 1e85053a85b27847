"""Sharding of the path across GPUs: utterances are independent, so a batch is
split by utterance with no data-path collective; the only exchange is one small
all-reduce of the summed loss and the frame count."""
from typing import List, Sequence, Tuple

import numpy as np
import torch


def shard_utterances(durations: Sequence[int], world_size: int, rank: int) -> np.ndarray:
    """Indexes (into the duration-sorted batch) of the utterances of `rank`:
    utterance k of the list sorted by decreasing duration goes to rank k mod
    world_size, which balances frames and keeps every shard sorted as
    intersect_dense requires (k2/csrc/intersect_dense.cu:168-177)."""
    order = np.argsort(-np.asarray(durations, dtype=np.int64), kind="stable")
    return order[rank::world_size]


def shard_segments(supervision_segments: torch.Tensor, world_size: int,
                   rank: int) -> Tuple[torch.Tensor, np.ndarray]:
    """Rows of `supervision_segments` owned by `rank` (still sorted by decreasing
    duration) and their indexes in the full batch."""
    idx = shard_utterances(supervision_segments[:, 2].tolist(), world_size, rank)
    return supervision_segments[torch.from_numpy(idx.astype(np.int64))], idx


def all_reduce_loss(loss_sum: torch.Tensor, num_frames: int, group=None) -> Tuple[torch.Tensor, int]:
    """Sum of the per-rank loss sums and frame counts over the process group (a
    16-byte all-reduce); identity without an initialised group."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return loss_sum, num_frames
    buf = torch.stack([loss_sum.detach().double().reshape(()),
                       torch.tensor(float(num_frames), dtype=torch.float64,
                                    device=loss_sum.device)])
    dist.all_reduce(buf, group=group)
    return buf[0], int(round(buf[1].item()))

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


class HostPrefetcher:
    """Double-buffered host -> device input pipeline for a training loop: the copy
    of batch k+1 (from pinned host memory, on its own stream) runs while batch k is
    being processed.  Usage::

        pf = HostPrefetcher("cuda:0")
        pf.submit(first_batch)
        for k in range(steps):
            x = pf.get()                    # batch k on the device
            if k + 1 < steps:
                pf.submit(next_batch)       # overlaps the work on batch k
            ...                             # forward / backward on x

    A buffer is reused `depth` batches later; `submit` first makes the copy stream
    wait for everything already enqueued on the current stream, so work that still
    reads the buffer is never overtaken."""

    def __init__(self, device, depth: int = 2):
        self.device = torch.device(device)
        self.depth = depth
        self.stream = torch.cuda.Stream(self.device)
        self.bufs: List[torch.Tensor] = [None] * depth
        self.ready = [torch.cuda.Event() for _ in range(depth)]
        self.submitted = 0
        self.taken = 0

    def submit(self, host_tensor: torch.Tensor) -> None:
        assert self.submitted - self.taken < self.depth, "all buffers are in flight"
        slot = self.submitted % self.depth
        buf = self.bufs[slot]
        if buf is None or buf.shape != host_tensor.shape or buf.dtype != host_tensor.dtype:
            buf = torch.empty(host_tensor.shape, dtype=host_tensor.dtype, device=self.device)
            self.bufs[slot] = buf
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            buf.copy_(host_tensor, non_blocking=True)
            self.ready[slot].record(self.stream)
        self.submitted += 1

    def get(self) -> torch.Tensor:
        assert self.taken < self.submitted, "nothing submitted"
        slot = self.taken % self.depth
        torch.cuda.current_stream(self.device).wait_event(self.ready[slot])
        self.taken += 1
        return self.bufs[slot]


def bind_to_gpu_numa_node(device) -> dict:
    """Restricts this process to the CPUs of the NUMA node its GPU hangs off, so that
    pinned host buffers allocated afterwards (first touch) and the threads that feed
    the GPU sit next to its PCIe root: with one process per GPU on a multi-socket host,
    copies that cross the socket interconnect share its bandwidth with every other
    rank.  Reads the node from sysfs; does nothing when the topology cannot be read or
    the node's CPUs are not among those the process may use.  Returns what it did."""
    import os
    info = {"bound": False}
    try:
        props = torch.cuda.get_device_properties(torch.device(device))
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        info.update(pci=bus, node=node)
        if node < 0:
            return info
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        mine = cpus & allowed
        info["cpus_on_node"] = len(mine)
        if mine and mine != allowed:
            os.sched_setaffinity(0, mine)
            info["bound"] = True
    except (OSError, ValueError, AttributeError, RuntimeError, AssertionError) as e:
        info["error"] = str(e)
    return info

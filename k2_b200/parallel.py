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


class LossReducer:
    """The per-step all-reduce of [sum of losses, frames], enqueued by a helper thread.

    Launching a collective costs the host about as much as launching all gradient
    kernels of a step; when the host is what paces the loop that shows in full.  So
    `submit` (called as soon as the loss exists) only records an event and hands the
    job over; the helper thread enqueues the all-reduce on a side stream behind that
    event while the caller goes on to launch the backward pass, and `result` makes the
    caller's stream wait for the collective::

        reducer = LossReducer(device)
        loss = k2.ctc_loss(...)
        reducer.submit(loss, num_frames)
        loss.backward()                      # gradient kernels and collective overlap
        total_loss, total_frames = reducer.result()   # device tensors, no host wait

    The gradient of a summed loss does not depend on the other ranks, so nothing
    waits for the collective but the consumer of the totals.  On CPU tensors (gloo)
    the helper thread runs the collective itself."""

    def __init__(self, device, group=None):
        import queue
        import threading
        self.device = torch.device(device)
        self.group = group
        self.cuda = self.device.type == "cuda"
        self.bufs = [torch.zeros(2, dtype=torch.float64, device=self.device) for _ in range(2)]
        self.unit = torch.tensor([1.0, 0.0], dtype=torch.float64, device=self.device)
        self.step = 0
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.ready = torch.cuda.Event() if self.cuda else None
        self.jobs = queue.SimpleQueue()
        self.done = threading.Event()
        self.error = None
        self.pending = False
        self.thread = threading.Thread(target=self._run, name="k2b200-loss-reducer", daemon=True)
        self.thread.start()

    def _run(self):
        import torch.distributed as dist
        if self.cuda:
            torch.cuda.set_device(self.device)
        while True:
            buf = self.jobs.get()
            if buf is None:
                return
            try:
                if self.cuda:
                    self.stream.wait_event(self.ready)
                    with torch.cuda.stream(self.stream):
                        dist.all_reduce(buf, group=self.group)
                else:
                    dist.all_reduce(buf, group=self.group)
            except Exception as e:  # handed to the caller by result()
                self.error = e
            self.done.set()

    def submit(self, loss_sum: torch.Tensor, num_frames: int) -> None:
        assert not self.pending, "result() of the previous step has not been taken"
        buf = self.bufs[self.step & 1]
        with torch.no_grad():
            # [loss, 0] then + [0, frames]: two small kernels, no allocation
            torch.mul(self.unit, loss_sum.detach().reshape(()), out=buf)
            buf[1] += float(num_frames)
        if self.cuda:
            self.ready.record(torch.cuda.current_stream(self.device))
        self.pending = True
        self.jobs.put(buf)

    def result(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(total loss, total frames) as 0-dim float64 tensors on the device; the current
        stream waits for the collective, the host only for its launch."""
        assert self.pending, "nothing submitted"
        self.done.wait()
        self.done.clear()
        self.pending = False
        if self.error is not None:
            e, self.error = self.error, None
            raise e
        buf = self.bufs[self.step & 1]
        self.step += 1
        if self.cuda:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
        return buf[0], buf[1]

    def close(self) -> None:
        self.jobs.put(None)
        self.thread.join(timeout=5)


class PeerLossReducer:
    """`LossReducer` over peer memory: one kernel of this library
    (`k2b200_loss_sum_all_reduce`) sums the rank's losses and exchanges (loss, frames)
    with the other GPUs of the node by stores into their memory - no collective library
    on the step, a single launch from the thread that feeds the GPU::

        reducer = PeerLossReducer(device)          # once; the process group is used to
        ...                                        # exchange the buffers' handles
        loss = k2.ctc_loss(..., reduction="sum")   # or the per-utterance losses
        reducer.submit(loss, num_frames)           # side stream, behind the loss
        loss.backward()
        total_loss, total_frames = reducer.result()

    All ranks of `group` must be processes of one node, one GPU each."""

    def __init__(self, device, group=None, poll_limit: int = -1):
        import ctypes
        import torch.distributed as dist
        from . import _lib
        self._lib, self._ct = _lib, ctypes
        self.device = torch.device(device)
        self.poll_limit = poll_limit
        on = dist.is_available() and dist.is_initialized()
        self.rank = dist.get_rank(group) if on else 0
        self.world = dist.get_world_size(group) if on else 1
        with torch.cuda.device(self.device):
            local = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(64)
            _lib.check(_lib.lib.k2b200_peer_reduce_create(ctypes.byref(local), handle))
            self.local = local.value
            handles = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, bytes(handle.raw), group=group)
            self.bufs = (ctypes.c_void_p * self.world)()
            self.opened = []
            error = None
            try:
                for r in range(self.world):
                    if r == self.rank:
                        self.bufs[r] = self.local
                    else:
                        p = ctypes.c_void_p()
                        _lib.check(_lib.lib.k2b200_peer_reduce_open(handles[r], ctypes.byref(p)))
                        self.bufs[r] = p.value
                        self.opened.append(p.value)
            except RuntimeError as e:  # e.g. no peer access between two of the GPUs
                error = e
            if self.world > 1:
                # every rank has mapped every buffer - or none goes on: a rank that failed must
                # not leave the others waiting for it in the first exchange
                ok = torch.tensor([0 if error is not None else 1], dtype=torch.int32,
                                  device=self.device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
                if int(ok.item()) == 0:
                    self.close()
                    raise RuntimeError("PeerLossReducer: a rank could not map a peer's buffer"
                                       + (f" ({error})" if error is not None else ""))
            elif error is not None:
                raise error
        self.stream = torch.cuda.Stream(self.device)
        self.out = [torch.zeros(2, dtype=torch.float64, device=self.device) for _ in range(2)]
        # what a step needs, looked up once: the host side of a step is a single call
        self._stream = self.stream.cuda_stream
        self._out_ptr = [t.data_ptr() for t in self.out]
        self._out = [(t[0], t[1]) for t in self.out]
        self._call = _lib.lib.k2b200_loss_sum_all_reduce
        self._index = self.device.index if self.device.index is not None \
            else torch.cuda.current_device()
        self.seq = 0
        self.pending = False

    def submit(self, losses: torch.Tensor, num_frames: int, sign: float = 1.0) -> None:
        """losses: a 0-dim or 1-dim float32 / float64 device tensor; its sum times `sign`
        is this rank's loss.  The exchange is queued on the reducer's stream behind what the
        current stream holds."""
        assert not self.pending, "result() of the previous step has not been taken"
        assert losses.is_cuda and losses.dtype in (torch.float32, torch.float64)
        if not losses.is_contiguous():
            losses = losses.contiguous()
        self.seq += 1
        losses.record_stream(self.stream)
        args = (losses.data_ptr(), losses.numel(), losses.dtype == torch.float32, sign,
                num_frames, self.bufs, self.rank, self.world, self.seq, self.poll_limit,
                self._out_ptr[self.seq & 1], self._stream)
        if torch.cuda.current_device() == self._index:
            rc = self._call(*args, self._lib.stream_of(self.device))
        else:
            with torch.cuda.device(self.device):
                rc = self._call(*args, self._lib.stream_of(self.device))
        if rc != 0:
            self._lib.check(rc)
        self.pending = True

    def result(self, join: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
        """(total loss, total frames), 0-dim float64 device tensors.  With `join` the current
        stream waits for the exchange (the host does not), so whatever is queued next may
        read them; without it they are only valid after `self.stream` has been waited for
        (a trainer that logs the totals every so many steps joins then, and the ranks do not
        run in lockstep in between).  The buffers are reused two steps later."""
        assert self.pending, "nothing submitted"
        self.pending = False
        if join:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
        return self._out[self.seq & 1]

    def status(self) -> int:
        """Waits for the exchange stream; bit 0 = a bounded wait for a peer gave up (the
        totals of that step are invalid)."""
        st = self._ct.c_int32()
        with torch.cuda.device(self.device):
            self._lib.check(self._lib.lib.k2b200_peer_reduce_status(
                self.local, self.stream.cuda_stream, self._ct.byref(st)))
        return st.value

    def close(self) -> None:
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for p in self.opened:
                self._lib.check(self._lib.lib.k2b200_peer_reduce_close(p))
            self.opened = []
            if self.local:
                self._lib.check(self._lib.lib.k2b200_peer_reduce_destroy(self.local))
                self.local = None


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


def bind_to_gpu_numa_node(device, cpus_per_gpu: int = 4) -> dict:
    """Restricts this process to the CPUs of the NUMA node its GPU hangs off, so that
    pinned host buffers allocated afterwards (first touch) and the threads that feed
    the GPU sit next to its PCIe root: with one process per GPU on a multi-socket host,
    copies that cross the socket interconnect share its bandwidth with every other
    rank.  Reads the node from sysfs; does nothing when the topology cannot be read or
    the node's CPUs are not among those the process may use, and does not bind either
    when that would leave fewer than `cpus_per_gpu` CPUs for each visible GPU of the
    node (a container whose CPU set lies mostly on the other socket: ranks that crowd
    onto two or three CPUs run several times slower than ranks that cross the
    interconnect).  Returns what it did."""
    import os
    info = {"bound": False}

    def node_of(index):
        props = torch.cuda.get_device_properties(index)
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            return bus, int(f.read().strip())

    try:
        device = torch.device(device)
        index = device.index if device.index is not None else torch.cuda.current_device()
        bus, node = node_of(index)
        info.update(pci=bus, node=node)
        if node < 0:
            return info
        gpus_on_node = sum(1 for k in range(torch.cuda.device_count()) if node_of(k)[1] == node)
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = os.sched_getaffinity(0)
        mine = cpus & allowed
        info.update(cpus_on_node=len(mine), cpus_allowed=len(allowed), gpus_on_node=gpus_on_node)
        if mine and mine != allowed and len(mine) >= cpus_per_gpu * gpus_on_node:
            os.sched_setaffinity(0, mine)
            info["bound"] = True
    except (OSError, ValueError, AttributeError, RuntimeError, AssertionError) as e:
        info["error"] = str(e)
    return info

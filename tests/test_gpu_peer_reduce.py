"""The loss sum + (loss, frames) all-reduce kernel over peer memory
(k2b200_loss_sum_all_reduce): one rank, the bounded wait for a peer that never
writes, and - where two GPUs are present - two ranks as two processes."""
import ctypes
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_single_rank_sum():
    from k2_b200 import parallel
    dev = torch.device("cuda", 0)
    reducer = parallel.PeerLossReducer(dev)
    g = torch.Generator().manual_seed(3)
    for step, n in enumerate([1, 7, 300, 5000]):
        tot = torch.randn(n, generator=g, dtype=torch.float64).to(dev)
        reducer.submit(tot, 1000 + step, sign=-1.0)
        loss, frames = reducer.result()
        np.testing.assert_allclose(float(loss), -float(tot.sum()), rtol=1e-12)
        assert float(frames) == 1000 + step
    lf = torch.randn(64, generator=g).to(dev)  # float32 input
    reducer.submit(lf, 5)
    loss, frames = reducer.result()
    np.testing.assert_allclose(float(loss), float(lf.double().sum()), rtol=1e-12)
    assert reducer.status() == 0
    reducer.close()


def test_bounded_wait_for_absent_peer():
    """A world of two in which nothing ever writes the second rank's slot: the wait runs
    out, the status bit is set, the call returns."""
    from k2_b200 import _lib
    dev = torch.device("cuda", 0)
    with torch.cuda.device(dev):
        a, b = ctypes.c_void_p(), ctypes.c_void_p()
        h = ctypes.create_string_buffer(64)
        _lib.check(_lib.lib.k2b200_peer_reduce_create(ctypes.byref(a), h))
        _lib.check(_lib.lib.k2b200_peer_reduce_create(ctypes.byref(b), h))
        bufs = (ctypes.c_void_p * 2)(a.value, b.value)
        vals = torch.ones(4, dtype=torch.float64, device=dev)
        out = torch.zeros(2, dtype=torch.float64, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream
        _lib.check(_lib.lib.k2b200_loss_sum_all_reduce(
            vals.data_ptr(), 4, 0, 1.0, 10.0, bufs, 0, 2, 1, 1000, out.data_ptr(), stream, None))
        st = ctypes.c_int32()
        _lib.check(_lib.lib.k2b200_peer_reduce_status(a.value, stream, ctypes.byref(st)))
        assert st.value & 1
        torch.cuda.synchronize(dev)  # the context is still usable
        assert float(vals.sum()) == 4.0
        _lib.check(_lib.lib.k2b200_peer_reduce_destroy(a.value))
        _lib.check(_lib.lib.k2b200_peer_reduce_destroy(b.value))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from k2_b200 import parallel
    reducer = parallel.PeerLossReducer(dev)
    got = []
    for step in range(50):
        vals = torch.full((8,), float(step + rank + 1), dtype=torch.float64, device=dev)
        reducer.submit(vals, 100 * (rank + 1) + step)
        loss, frames = reducer.result()
        got += [float(loss), float(frames)]
    assert reducer.status() == 0
    np.save(os.path.join(out_dir, f"p{rank}.npy"), np.array(got))
    dist.barrier()
    reducer.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks(tmp_path):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_rank, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = np.load(tmp_path / "p0.npy"), np.load(tmp_path / "p1.npy")
    want = []
    for step in range(50):
        want += [8.0 * (2 * step + 3), 300.0 + 2 * step]
    assert r0.tolist() == r1.tolist() == want

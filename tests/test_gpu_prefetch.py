"""HostPrefetcher: batches arrive intact and in order while work on the previous
batch is still queued."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_batches_arrive_in_order():
    from k2_b200.parallel import HostPrefetcher
    dev = "cuda:0"
    batches = [torch.full((1 << 20,), float(k)).pin_memory() for k in range(6)]
    pf = HostPrefetcher(dev)
    pf.submit(batches[0])
    sums = []
    for k in range(len(batches)):
        x = pf.get()
        if k + 1 < len(batches):
            pf.submit(batches[k + 1])
        y = x
        for _ in range(20):  # keep the compute stream busy with work that reads x
            y = y * 1.0 + 0.0
        sums.append(y.sum())
    got = [float(s.item()) for s in sums]
    assert got == [float(k) * (1 << 20) for k in range(len(batches))]

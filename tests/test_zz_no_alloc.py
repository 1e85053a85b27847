"""The scratch-free exclusive sum (k2b200_exclusive_sum_static) against the regular
entry point, through the C-ABI.

That entry point serves hosts that cannot give the library a scratch buffer - a
C/C++ service without a tensor allocator, or one whose device memory is fixed at
start-up - by keeping the scan's tile sums in an array inside the library.  The
array is shared by all calls and keeps what the last call left there, so the test
runs two different inputs back to back and expects both to match the regular
entry point exactly (integer sums: bit-exact).  This file sorts last on purpose:
a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _regular(lib, _lib, t, n, dev):
    out = torch.empty(n + 1, dtype=torch.int32, device=dev)
    tmp = torch.empty(lib.k2b200_exclusive_sum_tmp_bytes(n) + 16, dtype=torch.uint8, device=dev)
    _lib.check(lib.k2b200_exclusive_sum(_lib.ptr(t), _lib.ptr(out), n, _lib.ptr(tmp),
                                        _lib.stream_of(dev)))
    return out


def test_static_scratch_matches_regular_entry_point_twice_in_a_row():
    from k2_b200 import _lib
    lib = _lib.lib
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(11)
    max_len = lib.k2b200_exclusive_sum_static_max_len()
    assert max_len == 16384 * 2048 - 1
    # two calls in a row with different lengths: the second must not see the
    # first one's tile sums (a long input first, then a shorter one, then longer)
    for n in (3_000_001, 70_000, 5_000_000, 0, 1, 2048, 2049):
        x = torch.from_numpy(rng.integers(0, 50, size=n).astype(np.int32)).to(dev)
        want = _regular(lib, _lib, x, n, dev)
        got = torch.empty(n + 1, dtype=torch.int32, device=dev)
        _lib.check(lib.k2b200_exclusive_sum_static(_lib.ptr(x), _lib.ptr(got), n,
                                                   _lib.stream_of(dev)))
        assert torch.equal(got, want), f"n={n}"
        host = np.concatenate([[0], np.cumsum(x.cpu().numpy(), dtype=np.int64)])
        assert np.array_equal(got.cpu().numpy(), host.astype(np.int32)), f"n={n}"
    # in place
    x = torch.from_numpy(rng.integers(0, 9, size=100_001).astype(np.int32)).to(dev)
    want = _regular(lib, _lib, x[:100_000], 100_000, dev)
    _lib.check(lib.k2b200_exclusive_sum_static(_lib.ptr(x), _lib.ptr(x), 100_000,
                                               _lib.stream_of(dev)))
    assert torch.equal(x, want)


def test_static_scratch_rejects_inputs_beyond_its_limit():
    from k2_b200 import _lib
    lib = _lib.lib
    dev = torch.device("cuda:0")
    small = torch.zeros(8, dtype=torch.int32, device=dev)
    too_long = lib.k2b200_exclusive_sum_static_max_len() + 1
    status = lib.k2b200_exclusive_sum_static(_lib.ptr(small), _lib.ptr(small), too_long,
                                             _lib.stream_of(dev))
    assert status == 4  # K2B200_TOO_LARGE, nothing was launched
    msg = lib.k2b200_last_error().decode()
    assert "k2b200_exclusive_sum_static" in msg and str(too_long) in msg
    torch.cuda.synchronize()

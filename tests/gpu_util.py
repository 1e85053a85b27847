"""Helpers for the GPU parity tests: move data between the product's CUDA objects
and the host containers the oracle works on."""
import numpy as np
import torch

import k2_b200 as k2
from k2_b200.fsa_algo import _fsa_vec_from_numpy
from oracle.common import HostFsaVec

DEV = "cuda:0"


def fsa_to_host(fsa: "k2.Fsa", arc_map_a=None, arc_map_b=None) -> HostFsaVec:
    a = fsa.arcs
    cp = lambda t: None if t is None else t.detach().cpu().numpy()  # noqa: E731
    return HostFsaVec(cp(a._row_splits1), cp(a._row_splits2), cp(a.values()),
                      arc_map_a=cp(arc_map_a), arc_map_b=cp(arc_map_b))


def host_to_fsa(h: HostFsaVec, device=DEV) -> "k2.Fsa":
    return _fsa_vec_from_numpy(h.row_splits1, h.row_splits2, h.arcs, device)


def dense_from_scores(scores: np.ndarray, row_splits: np.ndarray, device=DEV,
                      requires_grad=False) -> "k2.DenseFsaVec":
    t = torch.from_numpy(np.ascontiguousarray(scores)).to(device)
    if requires_grad:
        t.requires_grad_(True)
    return k2.DenseFsaVec._from_dense_fsa_vec(t, row_splits)


def intersect_raw(a_fsa, dense, beam, a_to_b_map=None, mode=0, max_states=15000000,
                  max_arcs=1 << 30):
    """Lattice + arc maps through the C-ABI with an explicit Viterbi mode."""
    from k2_b200.autograd import _intersect_dense_arcs
    m = None if a_to_b_map is None else torch.as_tensor(a_to_b_map, dtype=torch.int32)
    ragged, ma, mb = _intersect_dense_arcs(a_fsa.arcs, dense, m, beam, max_states, max_arcs, mode)
    lat = k2.Fsa(ragged, _check=False)
    return lat, ma, mb

"""CTC decoding helpers with the reference's names and signatures
(k2/python/k2/decode.py:17-150): `get_lattice` wraps DenseFsaVec + pruned
intersection, `one_best_decoding` the best path, `get_aux_labels` reads the output
symbols of the best paths."""
from typing import List

import torch

from .autograd import intersect_dense_pruned
from .dense_fsa_vec import DenseFsaVec
from .fsa import Fsa
from .fsa_algo import shortest_path
from .ragged_tensor import RaggedTensor


def get_lattice(log_prob: torch.Tensor, log_prob_len: torch.Tensor, decoding_graph: Fsa,
                search_beam: float = 20, output_beam: float = 8, min_active_states: int = 30,
                max_active_states: int = 10000, subsampling_factor: int = 1) -> Fsa:
    """Decoding lattice of `log_prob` (N, T, C; `log_prob_len` valid frames each) against
    `decoding_graph` (one graph shared by the batch, or one per sequence)."""
    assert log_prob.ndim == 3, log_prob.shape
    assert log_prob_len.ndim == 1, log_prob_len.shape
    assert log_prob.size(0) == log_prob_len.size(0), (log_prob.shape, log_prob_len.shape)
    batch_size = log_prob.size(0)
    supervision_segment = torch.stack([
        torch.arange(batch_size), torch.zeros(batch_size), log_prob_len.cpu()]).t().to(torch.int32)
    dense_fsa_vec = DenseFsaVec(log_prob, supervision_segment,
                                allow_truncate=subsampling_factor - 1)
    return intersect_dense_pruned(decoding_graph, dense_fsa_vec, search_beam=search_beam,
                                  output_beam=output_beam, min_active_states=min_active_states,
                                  max_active_states=max_active_states)


def one_best_decoding(lattice: Fsa, use_double_scores: bool = True) -> Fsa:
    return shortest_path(lattice, use_double_scores=use_double_scores)


def get_aux_labels(best_paths: Fsa) -> List[List[int]]:
    """Output symbols per best path, without 0 (epsilon) and -1 (final)."""
    arcs = best_paths.arcs
    # arc -> FSA: compose the two row_splits of the FsaVec
    fsa_arc_splits = arcs._row_splits2[arcs._row_splits1.long()]
    aux = best_paths.aux_labels
    if isinstance(aux, RaggedTensor):
        aux = aux.remove_values_leq(0)
        splits = aux.row_splits()[fsa_arc_splits.long()]
        return RaggedTensor(aux.values, splits.to(torch.int32)).tolist()
    return RaggedTensor(aux.to(torch.int32), fsa_arc_splits.to(torch.int32)) \
        .remove_values_leq(0).tolist()

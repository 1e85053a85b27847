"""`CtcLoss` / `ctc_loss`: mirror of k2/python/k2/ctc_loss.py:28-208."""
from typing import Optional

import torch
import torch.nn as nn

from .autograd import (band_ctc_loss_sum, band_loss_supported, dense_loss_supported, intersect_dense,
                       intersect_dense_tot_scores)
from .dense_fsa_vec import DenseFsaVec
from .fsa import Fsa


# With no delay penalty nothing but the total scores of the lattice is used, so they
# are computed without building it when the graphs allow; set to False to force
# the reference's intersect_dense + get_tot_scores sequence.
FUSED_LOSS = True
# Outside the band-graph kernels (CTC graphs), the lattice-free path exponentiates
# every element of the dense matrix and streams whole rows through shared memory; with
# very many classes, of which a graph uses few, building the (small) lattice is cheaper.
FUSED_MAX_CLASSES = 2048


class CtcLoss(nn.Module):
    """CTC loss as the negated log-semiring total score of the graph intersected
    with the network output.  Blank is label 0."""

    def __init__(self, output_beam: float, reduction: str = "sum",
                 use_double_scores: bool = True):
        super().__init__()
        assert reduction in ("none", "mean", "sum")
        self.output_beam = output_beam
        self.reduction = reduction
        self.use_double_scores = use_double_scores

    def forward(self, decoding_graph: Fsa, dense_fsa_vec: DenseFsaVec,
                delay_penalty: float = 0.0,
                target_lengths: Optional[torch.Tensor] = None) -> torch.Tensor:
        if FUSED_LOSS and delay_penalty <= 0.0 and self.reduction == "sum":
            loss = band_ctc_loss_sum(decoding_graph, dense_fsa_vec, self.output_beam,
                                     self.use_double_scores)
            if loss is not None:
                return loss
        if FUSED_LOSS and delay_penalty <= 0.0 and (
                band_loss_supported(decoding_graph, dense_fsa_vec)
                or (dense_fsa_vec.num_cols <= FUSED_MAX_CLASSES
                    and dense_loss_supported(decoding_graph, dense_fsa_vec))):
            tot_scores = intersect_dense_tot_scores(
                decoding_graph, dense_fsa_vec, self.output_beam,
                use_double_scores=self.use_double_scores)
            return self._reduce(tot_scores, target_lengths)

        lattice = intersect_dense(
            a_fsas=decoding_graph, b_fsas=dense_fsa_vec, output_beam=self.output_beam,
            frame_idx_name="frame_idx" if delay_penalty > 0.0 else None)

        if delay_penalty > 0.0:
            # ctc_loss.py:99-136: penalise late non-blank symbols relative to the
            # middle frame of their sequence
            arcs = lattice.arcs
            fsa_of_arc = arcs.row_ids(1)[arcs.row_ids(2).long()].long()
            duration = dense_fsa_vec.duration.to(lattice.device)
            offset = lattice.frame_idx - (duration >> 1)[fsa_of_arc].to(torch.int32)
            penalty = -delay_penalty * offset.to(torch.float32)
            if hasattr(lattice, "_is_repeat_token_"):
                mask = ((lattice.labels == 0) | (lattice.labels == -1)
                        | lattice._is_repeat_token_)
            else:
                assert hasattr(lattice, "aux_labels")
                mask = (lattice.aux_labels == 0) | (lattice.aux_labels == -1)
            penalty.masked_fill_(mask, 0.0)
            lattice.scores = lattice.scores + penalty

        tot_scores = lattice.get_tot_scores(log_semiring=True,
                                            use_double_scores=self.use_double_scores)
        return self._reduce(tot_scores, target_lengths)

    def _reduce(self, tot_scores: torch.Tensor,
                target_lengths: Optional[torch.Tensor]) -> torch.Tensor:
        if self.reduction == "sum":
            # (-1 * tot_scores).to(float32).sum() of the reference in two kernels: the
            # reduction casts every element before adding, and negation commutes with
            # rounding, so the bits are the same
            return -tot_scores.sum(dtype=torch.float32)
        loss = -1 * tot_scores
        loss = loss.to(torch.float32)
        if self.reduction == "none":
            return loss
        elif self.reduction == "sum":
            return loss.sum()
        else:
            assert self.reduction == "mean"
            loss /= target_lengths
            return loss.mean()


_modules = {}


def ctc_loss(decoding_graph: Fsa, dense_fsa_vec: DenseFsaVec, output_beam: float = 10,
             delay_penalty: float = 0.0, reduction: str = "sum",
             use_double_scores: bool = True,
             target_lengths: Optional[torch.Tensor] = None) -> torch.Tensor:
    key = (output_beam, reduction, use_double_scores)
    m = _modules.get(key)
    if m is None:  # the module has no state beyond its three settings
        if len(_modules) >= 64:
            _modules.clear()
        m = _modules[key] = CtcLoss(output_beam=output_beam, reduction=reduction,
                                    use_double_scores=use_double_scores)
    return m(decoding_graph=decoding_graph, dense_fsa_vec=dense_fsa_vec,
             delay_penalty=delay_penalty, target_lengths=target_lengths)

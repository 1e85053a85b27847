"""`DenseFsaVec`: mirror of `k2.DenseFsaVec` (k2/python/k2/dense_fsa_vec.py:43-145).

scores is [sum_i (T_i + 1), C + 1] float32: column 0 is the final symbol (-1),
column c+1 holds class c; every sequence is followed by one extra row
[0, -inf, -inf, ...].  The gather from `log_probs` is a plain differentiable
torch index_select, so gradients w.r.t. `scores` flow back to `log_probs`.
"""
import numpy as np
import torch


class DenseFsaVec(object):

    def __init__(self, log_probs: torch.Tensor, supervision_segments: torch.Tensor,
                 allow_truncate: int = 0) -> None:
        assert log_probs.ndim == 3
        assert log_probs.dtype == torch.float32
        assert supervision_segments.ndim == 2
        assert supervision_segments.dtype == torch.int32
        assert supervision_segments.device.type == 'cpu'
        assert allow_truncate >= 0

        N, T, C = log_probs.shape
        seg = supervision_segments.numpy().astype(np.int64)
        indexes = []
        last_frame_indexes = []
        cur = 0
        for segment_index, start_frame, duration in seg.tolist():
            assert 0 <= segment_index < N
            assert 0 <= start_frame < T
            assert duration >= 0
            assert start_frame + duration <= T + allow_truncate
            end_frame = min(start_frame + duration, T)
            duration = end_frame - start_frame
            indexes.append(np.arange(start_frame, end_frame, dtype=np.int64) + segment_index * T)
            indexes.append(np.zeros(1, dtype=np.int64))  # placeholder for the extra row
            cur += duration
            last_frame_indexes.append(cur)
            cur += 1

        device = log_probs.device
        index = torch.from_numpy(np.concatenate(indexes)).to(device, non_blocking=True)
        scores = torch.empty(cur, C + 1, dtype=log_probs.dtype, device=device)
        scores[:, 1:] = log_probs.reshape(-1, C).index_select(0, index)
        scores[:, 0] = float('-inf')
        last = torch.tensor(last_frame_indexes, dtype=torch.int64).to(device, non_blocking=True)
        scores[last] = torch.tensor([0] + [float('-inf')] * C, dtype=log_probs.dtype,
                                    device=device)

        row_splits = np.zeros(seg.shape[0] + 1, dtype=np.int32)
        row_splits[1:] = np.asarray(last_frame_indexes, dtype=np.int32) + 1
        self._init(scores, row_splits)

    def _init(self, scores: torch.Tensor, h_row_splits: np.ndarray) -> None:
        assert scores.is_contiguous()
        self.scores = scores  # for back propagation
        self.h_row_splits = np.ascontiguousarray(h_row_splits, dtype=np.int32)
        self.row_splits = torch.from_numpy(self.h_row_splits).to(scores.device)
        self._duration = torch.from_numpy(np.diff(self.h_row_splits) - 1)

    @classmethod
    def _from_dense_fsa_vec(cls, scores: torch.Tensor, h_row_splits) -> 'DenseFsaVec':
        """From an already laid-out score matrix (fsa.h:138-185) and its row
        splits, as `_k2.DenseFsaVec(scores, row_splits)` does
        (k2/python/csrc/torch/fsa.cu:387-402)."""
        ans = cls.__new__(cls)
        ans._init(scores, np.asarray(h_row_splits, dtype=np.int32))
        return ans

    @property
    def duration(self) -> torch.Tensor:
        """Number of frames of each sequence (on CPU), without the extra row."""
        return self._duration

    def dim0(self) -> int:
        return len(self.h_row_splits) - 1

    @property
    def device(self) -> torch.device:
        return self.scores.device

    def to(self, device) -> 'DenseFsaVec':
        device = torch.device(device)
        if device == self.scores.device:
            return self
        return DenseFsaVec._from_dense_fsa_vec(self.scores.to(device), self.h_row_splits)

    def __str__(self) -> str:
        return (f"k2_b200.DenseFsaVec(num_seqs={self.dim0()}, "
                f"scores={tuple(self.scores.shape)}, device={self.device})")

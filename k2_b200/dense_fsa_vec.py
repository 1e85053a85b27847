"""`DenseFsaVec`: mirror of `k2.DenseFsaVec` (k2/python/k2/dense_fsa_vec.py:43-145).

scores is [sum_i (T_i + 1), C + 1] float32: column 0 is the final symbol (-1),
column c+1 holds class c; every sequence is followed by one extra row
[0, -inf, -inf, ...].  The gather from `log_probs` is a plain differentiable
torch index_select, so gradients w.r.t. `scores` flow back to `log_probs`.
"""
import numpy as np
import torch

from . import _lib


class _DenseFsaVecFunction(torch.autograd.Function):
    """scores = layout(log_probs) on the GPU: one kernel forward, one backward
    (the CPU branch below keeps the reference's torch formulation)."""

    @staticmethod
    def forward(ctx, log_probs: torch.Tensor, segments: torch.Tensor,
                row_splits: torch.Tensor, rows: int, overlapping: bool) -> torch.Tensor:
        log_probs = log_probs.contiguous()
        N, T, C = log_probs.shape
        dev = log_probs.device
        scores = torch.empty(rows, C + 1, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.k2b200_dense_fsa_vec_fill(
                _lib.ptr(log_probs), N, T, C, _lib.ptr(segments), _lib.ptr(row_splits),
                segments.shape[0], _lib.ptr(scores), rows, _lib.stream_of(dev)))
        ctx.save_for_backward(segments, row_splits)
        ctx.shape = (N, T, C)
        ctx.rows = rows
        ctx.overlapping = overlapping
        return scores

    @staticmethod
    def backward(ctx, grad_scores: torch.Tensor):
        segments, row_splits = ctx.saved_tensors
        N, T, C = ctx.shape
        grad_scores = grad_scores.contiguous()
        dev = grad_scores.device
        grad = torch.empty(N, T, C, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.k2b200_dense_fsa_vec_backward(
                _lib.ptr(grad_scores), N, T, C, _lib.ptr(segments), _lib.ptr(row_splits),
                segments.shape[0], ctx.rows, int(ctx.overlapping), _lib.ptr(grad),
                _lib.stream_of(dev)))
        return grad, None, None, None, None


class _LogSoftmaxDenseFunction(torch.autograd.Function):
    """scores = layout(log_softmax(logits, dim=-1)): normalisation and layout in one
    kernel, and one kernel for the gradient w.r.t. the logits."""

    @staticmethod
    def forward(ctx, logits: torch.Tensor, segments: torch.Tensor,
                row_splits: torch.Tensor, rows: int, overlapping: bool) -> torch.Tensor:
        logits = logits.contiguous()
        N, T, C = logits.shape
        dev = logits.device
        scores = torch.empty(rows, C + 1, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.k2b200_dense_fsa_vec_from_logits(
                _lib.ptr(logits), N, T, C, _lib.ptr(segments), _lib.ptr(row_splits),
                segments.shape[0], _lib.ptr(scores), rows, _lib.stream_of(dev)))
        ctx.save_for_backward(segments, row_splits, scores)
        ctx.shape = (N, T, C)
        ctx.rows = rows
        ctx.overlapping = overlapping
        return scores

    @staticmethod
    def backward(ctx, grad_scores: torch.Tensor):
        segments, row_splits, scores = ctx.saved_tensors
        N, T, C = ctx.shape
        grad_scores = grad_scores.contiguous()
        dev = grad_scores.device
        grad = torch.empty(N, T, C, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            _lib.check(_lib.lib.k2b200_dense_fsa_vec_from_logits_backward(
                _lib.ptr(grad_scores), _lib.ptr(scores), N, T, C, _lib.ptr(segments),
                _lib.ptr(row_splits), segments.shape[0], ctx.rows, int(ctx.overlapping),
                _lib.ptr(grad), _lib.stream_of(dev)))
        return grad, None, None, None, None


class DenseFsaVec(object):

    def __init__(self, log_probs: torch.Tensor, supervision_segments: torch.Tensor,
                 allow_truncate: int = 0, _logits: bool = False) -> None:
        assert log_probs.ndim == 3
        assert log_probs.dtype == torch.float32
        assert supervision_segments.ndim == 2
        assert supervision_segments.dtype == torch.int32
        assert supervision_segments.device.type == 'cpu'
        assert allow_truncate >= 0

        N, T, C = log_probs.shape
        seg = supervision_segments.numpy()  # int32 [num_segs, 3]: sequence, start, duration
        num_segs = seg.shape[0]
        seq, start = seg[:, 0], seg[:, 1]
        dur = seg[:, 2]
        truncated = False
        if num_segs:
            # (few numpy calls: this runs on the thread that feeds the GPU, every step)
            top = seg.max(axis=0)
            assert seg.min() >= 0 and top[0] < N and top[1] < T
            if int(top[1]) + int(top[2]) > T:  # only then can a segment pass the end
                end = start.astype(np.int64) + dur
                assert end.max() <= T + allow_truncate
                # durations after truncation
                dur = (np.minimum(end, T) - start).astype(np.int32)
                truncated = True
        # every segment gets one extra (final) row
        row_splits = np.zeros(num_segs + 1, dtype=np.int32)
        np.cumsum(dur + 1, out=row_splits[1:])
        rows = int(row_splits[-1])
        device = log_probs.device

        if log_probs.is_cuda:
            # one kernel writes the whole matrix; two segments that touch the same
            # frame make the backward use atomic adds
            first = seq * np.int32(T) + start if N * T < 2**31 else seq.astype(np.int64) * T + start
            if num_segs == 0 or np.bincount(seq, minlength=N).max() <= 1:
                overlapping = False  # at most one segment per sequence
            else:
                order = np.argsort(first, kind="stable")
                overlapping = bool(np.any((first + dur)[order][:-1] > first[order][1:]))
            # (a copy: the caller's tensor may change before the scores are made)
            eff = seg.copy() if not truncated else \
                np.stack([seq, start, dur], axis=1).astype(np.int32)
            fn = _LogSoftmaxDenseFunction if _logits else _DenseFsaVecFunction
            # The score matrix, and the device copy of the row splits, are made on first
            # use: a loss that reads the log-probs directly (k2b200_band_loss_*) needs
            # neither.
            self._init(None, row_splits, device=device, num_cols=C + 1)
            # (no closure over self: a reference cycle would keep the log-probs and
            # their gradient alive until the cycle collector runs)
            self._make_scores = (fn, log_probs, eff, rows, overlapping)
            if not _logits and not overlapping:
                # what a loss needs to read `log_probs` in place and to send its
                # gradient straight to it (k2b200_band_loss_*,
                # k2b200_dense_loss_backward_log_probs): the tensor and, per
                # sequence, the row of its first frame
                self._source = (log_probs, first.astype(np.int32, copy=False))
            return
        else:
            if _logits:
                log_probs = torch.log_softmax(log_probs, dim=-1)
            # host tensors (layout checks, graph preparation): the reference's own
            # formulation with torch ops
            last_frame_indexes = (row_splits[1:] - 1).astype(np.int64)
            index = np.zeros(rows, dtype=np.int64)
            for k in range(seg.shape[0]):
                r0 = int(row_splits[k])
                index[r0:r0 + int(dur[k])] = np.arange(int(seg[k, 1]), int(seg[k, 1]) + int(dur[k])) + \
                    int(seg[k, 0]) * T
            scores = torch.empty(rows, C + 1, dtype=log_probs.dtype, device=device)
            scores[:, 1:] = log_probs.reshape(-1, C).index_select(0, torch.from_numpy(index))
            scores[:, 0] = float('-inf')
            scores[torch.from_numpy(last_frame_indexes)] = torch.tensor(
                [0] + [float('-inf')] * C, dtype=log_probs.dtype)
        self._init(scores, row_splits)

    @classmethod
    def from_logits(cls, logits: torch.Tensor, supervision_segments: torch.Tensor,
                    allow_truncate: int = 0) -> 'DenseFsaVec':
        """`DenseFsaVec(torch.log_softmax(logits, dim=-1), supervision_segments,
        allow_truncate)` without materialising the log-probs: on CUDA the
        normalisation runs inside the layout kernel (and its adjoint inside the
        scatter of the gradient)."""
        return cls(logits, supervision_segments, allow_truncate, _logits=True)

    def _init(self, scores: torch.Tensor, h_row_splits: np.ndarray,
              d_row_splits: torch.Tensor = None, device=None, num_cols: int = 0) -> None:
        assert scores is None or scores.is_contiguous()
        self._source = None
        self._source_rows = {}
        self._make_scores = None
        self._scores = scores  # for back propagation
        self._device = scores.device if scores is not None else torch.device(device)
        self._num_cols = scores.shape[1] if scores is not None else num_cols
        self.h_row_splits = np.ascontiguousarray(h_row_splits, dtype=np.int32)
        self._row_splits = d_row_splits
        self._duration = None
        self._band_args = None  # the last k2b200_band_loss_* arguments made from this object

    @property
    def row_splits(self) -> torch.Tensor:
        """Row splits of the score matrix on `device` (made on first use)."""
        if self._row_splits is None:
            if self._device.type == "cuda":
                self._row_splits = _lib.upload_i32(self.h_row_splits, self._device)
            else:
                self._row_splits = torch.from_numpy(self.h_row_splits)
        return self._row_splits

    @property
    def scores(self) -> torch.Tensor:
        """The [sum_i (T_i + 1), C + 1] score matrix (k2/csrc/fsa.h:138-185)."""
        if self._scores is None:
            fn, log_probs, eff, rows, overlapping = self._make_scores
            segments = _lib.upload_i32(eff.reshape(-1), self._device).view(-1, 3)
            self._scores = fn.apply(log_probs, segments, self.row_splits, rows, overlapping)
            self._make_scores = None
        return self._scores

    @scores.setter
    def scores(self, value: torch.Tensor) -> None:
        assert value.is_contiguous()
        self._scores = value
        self._make_scores = None
        self._source = None  # no longer the layout of the tensor it was made from
        self._source_rows = {}
        self._band_args = None

    @property
    def num_cols(self) -> int:
        """Columns of the score matrix: classes + 1."""
        return self._num_cols

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
        if self._duration is None:
            self._duration = torch.from_numpy(np.diff(self.h_row_splits) - 1)
        return self._duration

    def dim0(self) -> int:
        return len(self.h_row_splits) - 1

    @property
    def device(self) -> torch.device:
        return self._device

    def to(self, device) -> 'DenseFsaVec':
        device = torch.device(device)
        if device == self._device:
            return self
        return DenseFsaVec._from_dense_fsa_vec(self.scores.to(device), self.h_row_splits)

    def __str__(self) -> str:
        return (f"k2_b200.DenseFsaVec(num_seqs={self.dim0()}, "
                f"scores=({int(self.h_row_splits[-1])}, {self._num_cols}), device={self.device})")

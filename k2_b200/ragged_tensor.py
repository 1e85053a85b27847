"""A two-axis ragged tensor of int32, as much of k2.RaggedTensor as FSA attributes
need on this path: an attribute such as `aux_labels` may hold a list of symbols per
arc, and every algorithm that maps arcs (intersection, best path, arc sorting) has
to carry it along with `index` (k2/python/csrc/torch/v2/ragged_any.cu `index`,
k2/csrc/ragged_ops.cu `Index`; used by k2/python/k2/autograd.py:430-439,586-593).

This is attribute plumbing, not part of the hot path: rows are gathered with torch
index arithmetic plus the library's row_ids kernel."""
from typing import List, Optional, Tuple, Union

import numpy as np
import torch

from . import _lib


class RaggedTensor:

    def __init__(self, data: Union[List[List[int]], torch.Tensor],
                 row_splits: Optional[torch.Tensor] = None, device=None):
        if isinstance(data, torch.Tensor):
            assert row_splits is not None and data.dtype == torch.int32
            assert row_splits.dtype == torch.int32 and row_splits.device == data.device
            self._values, self._row_splits = data.contiguous(), row_splits.contiguous()
        else:
            lens = np.fromiter((len(r) for r in data), dtype=np.int64, count=len(data))
            rs = np.zeros(len(data) + 1, np.int32)
            np.cumsum(lens, out=rs[1:])
            flat = np.fromiter((x for r in data for x in r), dtype=np.int32, count=int(rs[-1]))
            self._values = torch.from_numpy(flat)
            self._row_splits = torch.from_numpy(rs)
            if device is not None:
                self._values = self._values.to(device)
                self._row_splits = self._row_splits.to(device)

    # ------------------------------------------------------------------ shape
    @property
    def values(self) -> torch.Tensor:
        return self._values

    @property
    def dtype(self):
        return torch.int32

    @property
    def device(self) -> torch.device:
        return self._values.device

    @property
    def dim0(self) -> int:
        return self._row_splits.shape[0] - 1

    @property
    def num_axes(self) -> int:
        return 2

    def numel(self) -> int:
        return self._values.shape[0]

    def row_splits(self, axis: int = 1) -> torch.Tensor:
        assert axis == 1
        return self._row_splits

    def row_ids(self, axis: int = 1) -> torch.Tensor:
        assert axis == 1
        return _row_ids(self._row_splits, self.numel())

    @property
    def shape(self) -> Tuple[int, None]:
        return (self.dim0, None)

    def to(self, device) -> 'RaggedTensor':
        return RaggedTensor(self._values.to(device), self._row_splits.to(device))

    def clone(self) -> 'RaggedTensor':
        return RaggedTensor(self._values.clone(), self._row_splits.clone())

    def tolist(self) -> List[List[int]]:
        v = self._values.cpu().tolist()
        rs = self._row_splits.cpu().tolist()
        return [v[rs[i]:rs[i + 1]] for i in range(len(rs) - 1)]

    def __eq__(self, other) -> bool:
        return (isinstance(other, RaggedTensor) and
                torch.equal(self._row_splits.cpu(), other._row_splits.cpu()) and
                torch.equal(self._values.cpu(), other._values.cpu()))

    def __repr__(self) -> str:
        return f"RaggedTensor({self.tolist()}, device='{self.device}')"

    # ------------------------------------------------------------------ ops
    def index(self, indexes: torch.Tensor, axis: int = 0,
              need_value_indexes: bool = False) -> Tuple['RaggedTensor', Optional[torch.Tensor]]:
        """ans[i] = self[indexes[i]]; an index of -1 gives an empty list.  With
        need_value_indexes the second result maps every value of `ans` to its position
        in `self.values`."""
        assert axis == 0 and indexes.dtype == torch.int32 and indexes.ndim == 1
        idx = indexes.to(self.device).long()
        ok = idx >= 0
        safe = idx.clamp(min=0)
        begin = self._row_splits[safe].long()
        lens = torch.where(ok, self._row_splits[safe + 1].long() - begin, torch.zeros_like(begin))
        new_rs = torch.zeros(idx.shape[0] + 1, dtype=torch.int32, device=self.device)
        new_rs[1:] = torch.cumsum(lens, 0).to(torch.int32)
        total = int(new_rs[-1].item())
        row = _row_ids(new_rs, total).long()
        pos = begin[row] + (torch.arange(total, device=self.device) - new_rs[row].long())
        ans = RaggedTensor(self._values[pos], new_rs)
        return ans, (pos.to(torch.int32) if need_value_indexes else None)

    def remove_values_leq(self, cutoff: int) -> 'RaggedTensor':
        """Drops the values <= cutoff (k2 uses it to strip epsilons and -1 from aux
        labels, k2/python/k2/utils.py get_texts)."""
        keep = self._values > cutoff
        counts = torch.zeros(self.dim0 + 1, dtype=torch.int64, device=self.device)
        counts[1:] = torch.cumsum(
            torch.zeros(self.dim0, dtype=torch.int64, device=self.device).index_add_(
                0, self.row_ids().long(), keep.long()), 0)
        return RaggedTensor(self._values[keep], counts.to(torch.int32))


def _row_ids(row_splits: torch.Tensor, num_elems: int) -> torch.Tensor:
    out = torch.empty(num_elems, dtype=torch.int32, device=row_splits.device)
    if num_elems == 0:
        return out
    if row_splits.is_cuda:
        with torch.cuda.device(row_splits.device):
            _lib.check(_lib.lib.k2b200_row_splits_to_row_ids(
                _lib.ptr(row_splits), row_splits.shape[0] - 1, _lib.ptr(out), num_elems,
                _lib.stream_of(row_splits.device)))
        return out
    lens = (row_splits[1:] - row_splits[:-1]).long()
    return torch.repeat_interleave(torch.arange(lens.shape[0], dtype=torch.int32), lens)


def cat(srcs: List[RaggedTensor]) -> RaggedTensor:
    """Concatenation along axis 0."""
    values = torch.cat([s.values for s in srcs])
    offs, pieces = 0, [torch.zeros(1, dtype=torch.int32, device=values.device)]
    for s in srcs:
        pieces.append(s.row_splits()[1:] + offs)
        offs += s.numel()
    return RaggedTensor(values, torch.cat(pieces).to(torch.int32))

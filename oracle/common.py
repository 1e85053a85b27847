"""TEST INFRASTRUCTURE ONLY: host-side FsaVec container shared by the oracle bindings."""
from dataclasses import dataclass, field
from typing import Optional

import numpy as np


@dataclass
class HostFsaVec:
    row_splits1: np.ndarray
    row_splits2: np.ndarray
    arcs: np.ndarray  # [A, 4] int32: src, dest, label, score bits
    aux_labels: Optional[np.ndarray] = None
    arc_map_a: Optional[np.ndarray] = None
    arc_map_b: Optional[np.ndarray] = None
    extra: dict = field(default_factory=dict)

    @property
    def scores(self) -> np.ndarray:
        return np.ascontiguousarray(self.arcs[:, 3]).view(np.float32)

    @property
    def num_fsas(self):
        return len(self.row_splits1) - 1

    @property
    def num_states(self):
        return len(self.row_splits2) - 1

    @property
    def num_arcs(self):
        return self.arcs.shape[0]


def make_arcs(src, dest, label, score) -> np.ndarray:
    a = np.empty((len(src), 4), dtype=np.int32)
    a[:, 0] = src
    a[:, 1] = dest
    a[:, 2] = label
    a[:, 3] = np.asarray(score, dtype=np.float32).view(np.int32)
    return a

"""k2_b200: a B200 (sm_100a) backend for k2's dense-intersection / CTC - LF-MMI
loss path, behind k2's own Python API names for that path."""
from . import _lib  # noqa: F401  (fails loudly when the CUDA library is missing)
from .autograd import (dense_loss_supported, index_select, intersect_dense,  # noqa: F401
                       intersect_dense_pruned, intersect_dense_tot_scores)
from .ctc_loss import CtcLoss, ctc_loss  # noqa: F401
from .decode import get_aux_labels, get_lattice, one_best_decoding  # noqa: F401
from .dense_fsa_vec import DenseFsaVec  # noqa: F401
from .fsa import Fsa, create_fsa_vec  # noqa: F401
from .fsa_algo import arc_sort, ctc_graph, ctc_topo, linear_fsa, shortest_path  # noqa: F401
from .online_dense_intersecter import DecodeStateInfo, OnlineDenseIntersecter  # noqa: F401
from .ragged import RaggedArc  # noqa: F401
from .ragged_tensor import RaggedTensor  # noqa: F401

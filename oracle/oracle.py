"""TEST INFRASTRUCTURE ONLY: ctypes binding of oracle/libk2oracle.so.

libk2oracle.so is built from oracle/k2_oracle.c, the plain-C CPU restatement of
the k2 reference algorithms on the dense-intersection hot path.  It has the same
Python interface as oracle/ref.py (the real reference), so the same checks run
against either.  Only tests, the smoke test and the CPU-baseline leg of the
benchmark may import it; the product package never does.
"""
import ctypes
import os
import subprocess

import numpy as np

from .common import HostFsaVec, make_arcs  # noqa: F401

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libk2oracle.so")
SRC_PATH = os.path.join(_HERE, "k2_oracle.c")

_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_vp = ctypes.c_void_p
_i32 = ctypes.c_int32


def build(force: bool = False) -> str:
    """Compile k2_oracle.c with gcc if the library is missing or stale."""
    if (force or not os.path.exists(LIB_PATH)
            or os.path.getmtime(LIB_PATH) < os.path.getmtime(SRC_PATH)):
        subprocess.check_call(["make", "-C", _HERE, "oracle"], stdout=subprocess.DEVNULL)
    return LIB_PATH


def _p(a, t):
    return a.ctypes.data_as(t) if a is not None else None


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(LIB_PATH)
        L.k2o_last_error.restype = ctypes.c_char_p
        L.k2o_free.argtypes = [_vp]
        L.k2o_dims.argtypes = [_vp, _i32p, _i32p, _i32p]
        L.k2o_final_beam.restype = ctypes.c_float
        L.k2o_final_beam.argtypes = [_vp]
        L.k2o_copy.argtypes = [_vp, _i32p, _i32p, _vp, _i32p, _i32p, _i32p]
        L.k2o_ctc_graphs.restype = _vp
        L.k2o_ctc_graphs.argtypes = [_i32p, _i32, _i32p, _i32]
        L.k2o_intersect_dense.restype = _vp
        L.k2o_intersect_dense.argtypes = [_i32p, _i32, _i32p, _vp, _f32p, _i32, _i32, _i32p,
                                          _i32, _i32p, ctypes.c_float, _i32, _i32]
        L.k2o_intersect_dense_pruned.restype = _vp
        L.k2o_intersect_dense_pruned.argtypes = [
            _i32p, _i32, _i32p, _vp, _f32p, _i32, _i32, _i32p, _i32, ctypes.c_float,
            ctypes.c_float, _i32, _i32, _i32]
        L.k2o_forward_scores.argtypes = [_i32p, _i32, _i32p, _vp, _i32, _i32, _f64p, _i32p]
        L.k2o_backward_scores.argtypes = [_i32p, _i32, _i32p, _vp, _i32, _i32, _f64p]
        L.k2o_tot_scores_and_arc_post.argtypes = [_i32p, _i32, _i32p, _vp, _i32, _f64p, _f64p,
                                                  _f64p, _f64p]
        L.k2o_shortest_path.argtypes = [_i32p, _i32, _vp, _i32p, _i32p, _i32p]
        L.k2o_properties.argtypes = [_i32p, _i32, _i32p, _vp, _i32p]
        _lib = L
    return _lib


def _take(ptr, aux=False, maps=False) -> HostFsaVec:
    if not ptr:
        raise RuntimeError("oracle: " + lib().k2o_last_error().decode())
    ptr = _vp(ptr)
    try:
        a, b, c = _i32(), _i32(), _i32()
        lib().k2o_dims(ptr, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
        nf, ns, na = a.value, b.value, c.value
        rs1 = np.zeros(nf + 1, np.int32)
        rs2 = np.zeros(ns + 1, np.int32)
        arcs = np.zeros((na, 4), np.int32)
        auxa = np.zeros(na, np.int32) if aux else None
        ma = np.zeros(na, np.int32) if maps else None
        mb = np.zeros(na, np.int32) if maps else None
        lib().k2o_copy(ptr, _p(rs1, _i32p), _p(rs2, _i32p), arcs.ctypes.data_as(_vp),
                       _p(auxa, _i32p), _p(ma, _i32p), _p(mb, _i32p))
        out = HostFsaVec(rs1, rs2, arcs, auxa, ma, mb)
        out.extra["final_beam"] = float(lib().k2o_final_beam(ptr))
        return out
    finally:
        lib().k2o_free(ptr)


def _fsa_args(f: HostFsaVec):
    rs1 = np.ascontiguousarray(f.row_splits1, np.int32)
    rs2 = np.ascontiguousarray(f.row_splits2, np.int32)
    arcs = np.ascontiguousarray(f.arcs, np.int32)
    return rs1, rs2, arcs


def ctc_graphs(symbols, modified=False) -> HostFsaVec:
    rs = np.zeros(len(symbols) + 1, np.int32)
    rs[1:] = np.cumsum([len(s) for s in symbols])
    vals = np.asarray([x for s in symbols for x in s], np.int32)
    if vals.size == 0:
        vals = np.zeros(1, np.int32)
    return _take(lib().k2o_ctc_graphs(_p(rs, _i32p), len(symbols), _p(vals, _i32p),
                                      int(modified)), aux=True)


def intersect_dense(a: HostFsaVec, scores: np.ndarray, b_row_splits: np.ndarray,
                    output_beam: float, a_to_b_map=None, max_states=15000000,
                    max_arcs=1 << 30) -> HostFsaVec:
    rs1, rs2, arcs = _fsa_args(a)
    scores = np.ascontiguousarray(scores, np.float32)
    brs = np.ascontiguousarray(b_row_splits, np.int32)
    m = None if a_to_b_map is None else np.ascontiguousarray(a_to_b_map, np.int32)
    return _take(lib().k2o_intersect_dense(
        _p(rs1, _i32p), len(rs1) - 1, _p(rs2, _i32p), arcs.ctypes.data_as(_vp),
        _p(scores, _f32p), scores.shape[0], scores.shape[1], _p(brs, _i32p), len(brs) - 1,
        _p(m, _i32p), float(output_beam), int(max_states), int(max_arcs)), maps=True)


def intersect_dense_pruned(a: HostFsaVec, scores: np.ndarray, b_row_splits: np.ndarray,
                           search_beam: float, output_beam: float, min_active: int,
                           max_active: int, allow_partial: bool = False) -> HostFsaVec:
    """`a` holds one graph per sequence or a single graph shared by all."""
    rs1, rs2, arcs = _fsa_args(a)
    scores = np.ascontiguousarray(scores, np.float32)
    brs = np.ascontiguousarray(b_row_splits, np.int32)
    return _take(lib().k2o_intersect_dense_pruned(
        _p(rs1, _i32p), len(rs1) - 1, _p(rs2, _i32p), arcs.ctypes.data_as(_vp),
        _p(scores, _f32p), scores.shape[0], scores.shape[1], _p(brs, _i32p), len(brs) - 1,
        float(search_beam), float(output_beam), int(min_active), int(max_active),
        int(bool(allow_partial))), maps=True)


def forward_scores(f: HostFsaVec, log_semiring=True, use_double=True,
                   want_entering_arcs=False):
    rs1, rs2, arcs = _fsa_args(f)
    out = np.zeros(f.num_states, np.float64)
    ea = np.full(f.num_states, -1, np.int32) if want_entering_arcs else None
    lib().k2o_forward_scores(_p(rs1, _i32p), len(rs1) - 1, _p(rs2, _i32p),
                             arcs.ctypes.data_as(_vp), int(log_semiring), int(use_double),
                             _p(out, _f64p), _p(ea, _i32p))
    return (out, ea) if want_entering_arcs else out


def backward_scores(f: HostFsaVec, log_semiring=True, use_double=True):
    rs1, rs2, arcs = _fsa_args(f)
    out = np.zeros(f.num_states, np.float64)
    lib().k2o_backward_scores(_p(rs1, _i32p), len(rs1) - 1, _p(rs2, _i32p),
                              arcs.ctypes.data_as(_vp), int(log_semiring), int(use_double),
                              _p(out, _f64p))
    return out


def tot_scores_and_arc_post(f: HostFsaVec, fwd, bwd, use_double=True):
    rs1, rs2, arcs = _fsa_args(f)
    fwd = np.ascontiguousarray(fwd, np.float64)
    bwd = np.ascontiguousarray(bwd, np.float64)
    tot = np.zeros(f.num_fsas, np.float64)
    post = np.zeros(max(f.num_arcs, 1), np.float64)
    lib().k2o_tot_scores_and_arc_post(_p(rs1, _i32p), len(rs1) - 1, _p(rs2, _i32p),
                                      arcs.ctypes.data_as(_vp), int(use_double),
                                      _p(fwd, _f64p), _p(bwd, _f64p), _p(tot, _f64p),
                                      _p(post, _f64p))
    return tot, post[:f.num_arcs]


def shortest_path(f: HostFsaVec, entering_arcs):
    rs1, rs2, arcs = _fsa_args(f)
    ea = np.ascontiguousarray(entering_arcs, np.int32)
    prs = np.zeros(f.num_fsas + 1, np.int32)
    best = np.zeros(max(f.num_arcs, 1), np.int32)
    n = lib().k2o_shortest_path(_p(rs1, _i32p), len(rs1) - 1, arcs.ctypes.data_as(_vp),
                                _p(ea, _i32p), _p(prs, _i32p), _p(best, _i32p))
    return prs, best[:n].copy()


def properties(f: HostFsaVec):
    rs1, rs2, arcs = _fsa_args(f)
    props = np.zeros(max(f.num_fsas, 1), np.int32)
    tot = lib().k2o_properties(_p(rs1, _i32p), len(rs1) - 1, _p(rs2, _i32p),
                               arcs.ctypes.data_as(_vp), _p(props, _i32p))
    return props[:f.num_fsas], tot


# ---------------------------------------------------------------------------
# The whole loss path on the host, as the reference's Python layer strings it
# together (k2/python/k2/ctc_loss.py:92-151, autograd.py:74-117, :631-664):
# intersect -> log-semiring forward/backward -> tot_scores, and the gradient
# d(sum_i w_i * tot_i)/d(scores) scattered through arc_map_b.
# ---------------------------------------------------------------------------
def loss_path(a: HostFsaVec, scores: np.ndarray, b_row_splits, output_beam, a_to_b_map=None,
              use_double=True, tot_grad=None, log_semiring=True):
    lat = intersect_dense(a, scores, b_row_splits, output_beam, a_to_b_map)
    fwd = forward_scores(lat, log_semiring, use_double)
    bwd = backward_scores(lat, log_semiring, use_double)
    tot, post = tot_scores_and_arc_post(lat, fwd, bwd, use_double)
    if tot_grad is None:
        tot_grad = np.ones(lat.num_fsas)
    # arc -> fsa
    state_fsa = np.repeat(np.arange(lat.num_fsas), np.diff(lat.row_splits1))
    arc_state = np.repeat(np.arange(lat.num_states), np.diff(lat.row_splits2))
    arc_fsa = state_fsa[arc_state] if lat.num_arcs else np.zeros(0, np.int64)
    if use_double:
        arc_grad = (np.exp(post) * np.asarray(tot_grad, np.float64)[arc_fsa]).astype(np.float32)
    else:
        arc_grad = (np.exp(post.astype(np.float32)) *
                    np.asarray(tot_grad, np.float32)[arc_fsa]).astype(np.float32)
    grad_b = np.zeros(scores.size, np.float32)
    np.add.at(grad_b, lat.arc_map_b, arc_grad)
    grad_a = np.zeros(a.num_arcs, np.float32)
    np.add.at(grad_a, lat.arc_map_a, arc_grad)
    return dict(lattice=lat, forward=fwd, backward=bwd, tot_scores=tot, arc_post=post,
                arc_grad=arc_grad, grad_b=grad_b.reshape(scores.shape), grad_a=grad_a)

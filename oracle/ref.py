"""TEST INFRASTRUCTURE ONLY: ctypes binding of oracle/_ref/libk2ref.so.

libk2ref.so is the k2 reference's own CPU code (compiled by oracle/Makefile from
the reference checkout) behind the small C shim in oracle/ref_shim.cc.  It is
used to pin the C restatement in oracle/k2_oracle.c, to generate the golden
fixtures under tests/golden/, and as the "reference" CPU baseline of bench.py.
Nothing in the product package may import this module.

All arrays are host numpy arrays.  An FsaVec is the `HostFsaVec` tuple of
row_splits1 [N+1], row_splits2 [S+1] and arcs [A,4] int32 whose 4th column holds
the float32 score bits (the layout of k2's 16-byte Arc, k2/csrc/fsa.h:31-63).
"""
import ctypes
import os
import numpy as np

from .common import HostFsaVec, make_arcs  # noqa: F401

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libk2ref.so")

_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)


def available() -> bool:
    return os.path.exists(LIB_PATH)


def _p(a, t):
    return a.ctypes.data_as(t) if a is not None else None


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not available():
            raise RuntimeError(
                f"{LIB_PATH} is missing: run `make -C oracle ref REF=<k2 checkout>`")
        L = ctypes.CDLL(LIB_PATH)
        L.kref_last_error.restype = ctypes.c_char_p
        L.kref_fsavec_create.restype = ctypes.c_void_p
        L.kref_fsavec_create.argtypes = [_i32p, ctypes.c_int32, _i32p, ctypes.c_int32,
                                         ctypes.c_void_p, ctypes.c_int32]
        L.kref_fsavec_free.argtypes = [ctypes.c_void_p]
        L.kref_fsavec_dims.argtypes = [ctypes.c_void_p, _i32p, _i32p, _i32p]
        L.kref_fsavec_copy.argtypes = [ctypes.c_void_p, _i32p, _i32p, ctypes.c_void_p,
                                       _i32p, _i32p, _i32p]
        L.kref_ctc_graphs.restype = ctypes.c_void_p
        L.kref_ctc_graphs.argtypes = [_i32p, ctypes.c_int32, _i32p, ctypes.c_int32]
        L.kref_ctc_topo.restype = ctypes.c_void_p
        L.kref_ctc_topo.argtypes = [ctypes.c_int32, ctypes.c_int32]
        L.kref_arc_sort.restype = ctypes.c_void_p
        L.kref_arc_sort.argtypes = [ctypes.c_void_p, _i32p]
        L.kref_intersect_dense.restype = ctypes.c_void_p
        L.kref_intersect_dense.argtypes = [ctypes.c_void_p, _f32p, ctypes.c_int32,
                                           ctypes.c_int32, _i32p, ctypes.c_int32, _i32p,
                                           ctypes.c_float, ctypes.c_int32, ctypes.c_int32]
        L.kref_intersect_dense_pruned.restype = ctypes.c_void_p
        L.kref_intersect_dense_pruned.argtypes = [
            ctypes.c_void_p, _f32p, ctypes.c_int32, ctypes.c_int32, _i32p, ctypes.c_int32,
            ctypes.c_float, ctypes.c_float, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
        L.kref_online_create.restype = ctypes.c_void_p
        L.kref_online_create.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_float,
                                         ctypes.c_float, ctypes.c_int32, ctypes.c_int32,
                                         ctypes.c_int32]
        L.kref_online_free.argtypes = [ctypes.c_void_p]
        L.kref_online_stream_free.argtypes = [ctypes.c_void_p]
        L.kref_online_stream_beam.restype = ctypes.c_float
        L.kref_online_stream_beam.argtypes = [ctypes.c_void_p]
        L.kref_online_decode.restype = ctypes.c_void_p
        L.kref_online_decode.argtypes = [ctypes.c_void_p, _f32p, ctypes.c_int32, ctypes.c_int32,
                                         _i32p, ctypes.c_int32,
                                         ctypes.POINTER(ctypes.c_void_p)]
        L.kref_forward_scores.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                                          _f64p, _i32p]
        L.kref_backward_scores.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                                           _f64p]
        L.kref_tot_scores_and_arc_post.argtypes = [ctypes.c_void_p, ctypes.c_int32, _f64p,
                                                   _f64p, _f64p, _f64p]
        L.kref_backprop_scores.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                                           ctypes.c_int32, _f64p, _i32p, _f64p, _f64p]
        L.kref_backprop_arc_post.argtypes = [ctypes.c_void_p, ctypes.c_int32, _f64p, _f64p,
                                             _f64p]
        L.kref_shortest_path.argtypes = [ctypes.c_void_p, _i32p, _i32p, _i32p]
        L.kref_properties.argtypes = [ctypes.c_void_p, _i32p]
        _lib = L
    return _lib


def _err():
    return lib().kref_last_error().decode(errors="replace")


class _Handle:
    """Owns a reference-side FsaVec."""

    def __init__(self, ptr):
        if not ptr:
            raise RuntimeError("k2 reference raised: " + _err())
        self.ptr = ctypes.c_void_p(ptr)

    def __del__(self):
        try:
            lib().kref_fsavec_free(self.ptr)
        except Exception:
            pass

    def dims(self):
        a, b, c = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
        lib().kref_fsavec_dims(self.ptr, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
        return a.value, b.value, c.value

    def to_host(self, aux=False, maps=False) -> HostFsaVec:
        nf, ns, na = self.dims()
        rs1 = np.zeros(nf + 1, np.int32)
        rs2 = np.zeros(ns + 1, np.int32)
        arcs = np.zeros((na, 4), np.int32)
        auxa = np.zeros(na, np.int32) if aux else None
        ma = np.zeros(na, np.int32) if maps else None
        mb = np.zeros(na, np.int32) if maps and maps != "a" else None
        lib().kref_fsavec_copy(self.ptr, _p(rs1, _i32p), _p(rs2, _i32p),
                               arcs.ctypes.data_as(ctypes.c_void_p), _p(auxa, _i32p),
                               _p(ma, _i32p), _p(mb, _i32p))
        return HostFsaVec(rs1, rs2, arcs, auxa, ma, mb)


def to_handle(f: HostFsaVec) -> _Handle:
    rs1 = np.ascontiguousarray(f.row_splits1, np.int32)
    rs2 = np.ascontiguousarray(f.row_splits2, np.int32)
    arcs = np.ascontiguousarray(f.arcs, np.int32)
    return _Handle(lib().kref_fsavec_create(_p(rs1, _i32p), len(rs1) - 1, _p(rs2, _i32p),
                                            len(rs2) - 1,
                                            arcs.ctypes.data_as(ctypes.c_void_p),
                                            arcs.shape[0]))


def ctc_graphs(symbols, modified=False) -> HostFsaVec:
    rs = np.zeros(len(symbols) + 1, np.int32)
    rs[1:] = np.cumsum([len(s) for s in symbols])
    vals = np.asarray([x for s in symbols for x in s], np.int32)
    if vals.size == 0:
        vals = np.zeros(1, np.int32)
    h = _Handle(lib().kref_ctc_graphs(_p(rs, _i32p), len(symbols), _p(vals, _i32p),
                                      int(modified)))
    return h.to_host(aux=True)


def ctc_topo(max_token: int, modified=False) -> HostFsaVec:
    return _Handle(lib().kref_ctc_topo(int(max_token), int(modified))).to_host(aux=True)


def arc_sort(f: HostFsaVec):
    h = to_handle(f)
    amap = np.zeros(f.num_arcs, np.int32)
    out = _Handle(lib().kref_arc_sort(h.ptr, _p(amap, _i32p))).to_host()
    return out, amap


def intersect_dense(a: HostFsaVec, scores: np.ndarray, b_row_splits: np.ndarray,
                    output_beam: float, a_to_b_map=None, max_states=15000000,
                    max_arcs=1 << 30) -> HostFsaVec:
    ha = to_handle(a)
    scores = np.ascontiguousarray(scores, np.float32)
    brs = np.ascontiguousarray(b_row_splits, np.int32)
    m = None if a_to_b_map is None else np.ascontiguousarray(a_to_b_map, np.int32)
    out = _Handle(lib().kref_intersect_dense(ha.ptr, _p(scores, _f32p), scores.shape[0],
                                             scores.shape[1], _p(brs, _i32p), len(brs) - 1,
                                             _p(m, _i32p), float(output_beam),
                                             int(max_states), int(max_arcs)))
    return out.to_host(maps=True)


def intersect_dense_pruned(a: HostFsaVec, scores, b_row_splits, search_beam, output_beam,
                           min_active, max_active, allow_partial=False):
    """The reference's IntersectDensePruned on CPU; `a` holds one graph per sequence or a
    single shared graph.  Returns a HostFsaVec with arc_map_a / arc_map_b."""
    ha = to_handle(a)
    scores = np.ascontiguousarray(scores, np.float32)
    brs = np.ascontiguousarray(b_row_splits, np.int32)
    out = _Handle(lib().kref_intersect_dense_pruned(
        ha.ptr, _p(scores, _f32p), scores.shape[0], scores.shape[1], _p(brs, _i32p),
        len(brs) - 1, float(search_beam), float(output_beam), int(min_active),
        int(max_active), int(bool(allow_partial))))
    return out.to_host(maps=True)


class OnlineIntersecter:
    """The reference's OnlineDenseIntersecter on CPU.  Streams are opaque handles
    (None starts a new one); `decode` returns the lattice so far (arc_map_a only) and
    the updated handles."""

    def __init__(self, graph: HostFsaVec, num_seqs, search_beam, output_beam, min_active,
                 max_active, allow_partial=True):
        self._graph = to_handle(graph)
        self._ptr = lib().kref_online_create(self._graph.ptr, int(num_seqs), float(search_beam),
                                             float(output_beam), int(min_active),
                                             int(max_active), int(bool(allow_partial)))
        if not self._ptr:
            raise RuntimeError("k2 reference raised: " + _err())

    def decode(self, scores, b_row_splits, streams):
        scores = np.ascontiguousarray(scores, np.float32)
        brs = np.ascontiguousarray(b_row_splits, np.int32)
        n = len(brs) - 1
        arr = (ctypes.c_void_p * n)(*[s for s in streams])
        out = _Handle(lib().kref_online_decode(self._ptr, _p(scores, _f32p), scores.shape[0],
                                               scores.shape[1], _p(brs, _i32p), n, arr))
        return out.to_host(maps="a"), [arr[i] for i in range(n)]

    @staticmethod
    def beam(stream) -> float:
        return float(lib().kref_online_stream_beam(stream))


def forward_scores(f: HostFsaVec, log_semiring=True, use_double=True,
                   want_entering_arcs=False):
    h = to_handle(f)
    out = np.zeros(f.num_states, np.float64)
    ea = np.full(f.num_states, -1, np.int32) if want_entering_arcs else None
    if lib().kref_forward_scores(h.ptr, int(log_semiring), int(use_double), _p(out, _f64p),
                                 _p(ea, _i32p)) != 0:
        raise RuntimeError("k2 reference raised: " + _err())
    return (out, ea) if want_entering_arcs else out


def backprop_scores(f: HostFsaVec, forward: bool, scores, deriv_in, log_semiring=True,
                    use_double=True, entering_arcs=None):
    """d(sum(deriv_in * scores)) / d(arc scores) for forward (or backward) scores."""
    h = to_handle(f)
    scores = np.ascontiguousarray(scores, np.float64)
    deriv_in = np.ascontiguousarray(deriv_in, np.float64)
    ea = None if entering_arcs is None else np.ascontiguousarray(entering_arcs, np.int32)
    out = np.zeros(f.num_arcs, np.float64)
    if lib().kref_backprop_scores(h.ptr, int(forward), int(log_semiring), int(use_double),
                                  _p(scores, _f64p), _p(ea, _i32p), _p(deriv_in, _f64p),
                                  _p(out, _f64p)) != 0:
        raise RuntimeError("k2 reference raised: " + _err())
    return out


def backprop_arc_post(f: HostFsaVec, arc_post_deriv, use_double=True):
    h = to_handle(f)
    d = np.ascontiguousarray(arc_post_deriv, np.float64)
    fd, bd = np.zeros(f.num_states, np.float64), np.zeros(f.num_states, np.float64)
    if lib().kref_backprop_arc_post(h.ptr, int(use_double), _p(d, _f64p), _p(fd, _f64p),
                                    _p(bd, _f64p)) != 0:
        raise RuntimeError("k2 reference raised: " + _err())
    return fd, bd


def backward_scores(f: HostFsaVec, log_semiring=True, use_double=True):
    h = to_handle(f)
    out = np.zeros(f.num_states, np.float64)
    if lib().kref_backward_scores(h.ptr, int(log_semiring), int(use_double),
                                  _p(out, _f64p)) != 0:
        raise RuntimeError("k2 reference raised: " + _err())
    return out


def tot_scores_and_arc_post(f: HostFsaVec, fwd, bwd, use_double=True):
    h = to_handle(f)
    fwd = np.ascontiguousarray(fwd, np.float64)
    bwd = np.ascontiguousarray(bwd, np.float64)
    tot = np.zeros(f.num_fsas, np.float64)
    post = np.zeros(max(f.num_arcs, 1), np.float64)
    if lib().kref_tot_scores_and_arc_post(h.ptr, int(use_double), _p(fwd, _f64p),
                                          _p(bwd, _f64p), _p(tot, _f64p),
                                          _p(post, _f64p)) != 0:
        raise RuntimeError("k2 reference raised: " + _err())
    return tot, post[:f.num_arcs]


def shortest_path(f: HostFsaVec, entering_arcs):
    h = to_handle(f)
    ea = np.ascontiguousarray(entering_arcs, np.int32)
    rs = np.zeros(f.num_fsas + 1, np.int32)
    best = np.zeros(max(f.num_arcs, 1), np.int32)
    n = lib().kref_shortest_path(h.ptr, _p(ea, _i32p), _p(rs, _i32p), _p(best, _i32p))
    if n < 0:
        raise RuntimeError("k2 reference raised: " + _err())
    return rs, best[:n].copy()


def properties(f: HostFsaVec):
    h = to_handle(f)
    props = np.zeros(max(f.num_fsas, 1), np.int32)
    tot = lib().kref_properties(h.ptr, _p(props, _i32p))
    return props[:f.num_fsas], tot

"""ctypes binding of libk2b200.so (the C-ABI declared in include/k2b200.h).

There is no CPU path and no fallback: importing this module fails loudly when the
CUDA library has not been built.
"""
import ctypes
import threading
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libk2b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} not found: build it with `python k2_b200/build.py` "
        "(nvcc, sm_100a). k2_b200 has no CPU or PyTorch fallback.")

lib = ctypes.CDLL(LIB_PATH)

c_i32 = ctypes.c_int32
c_i64 = ctypes.c_int64
c_vp = ctypes.c_void_p
c_sz = ctypes.c_size_t
c_f32 = ctypes.c_float


class IntersectArgs(ctypes.Structure):
    _fields_ = [
        ("num_fsas", c_i32), ("num_states", c_i32), ("num_arcs", c_i32),
        ("a_row_splits1", c_vp), ("a_row_splits2", c_vp), ("a_arcs", c_vp),
        ("a_in_splits", c_vp), ("a_in_arcs", c_vp),
        ("h_a_row_splits1", c_vp), ("h_a_arc_splits", c_vp),
        ("scores", c_vp), ("rows", c_i32), ("cols", c_i32), ("num_seqs", c_i32),
        ("h_b_row_splits", c_vp), ("h_a_to_b_map", c_vp),
        ("output_beam", c_f32), ("max_states", c_i32), ("max_arcs", c_i32),
        ("viterbi_mode", c_i32), ("a_max_degree", c_i32), ("a_shared", c_i32),
    ]


class BandLossArgs(ctypes.Structure):
    _fields_ = [
        ("num_fsas", c_i32), ("num_states", c_i32),
        ("a_row_splits2", c_vp), ("h_a_row_splits1", c_vp), ("h_a_arc_splits", c_vp),
        ("band_states", c_vp), ("band_arcs", c_vp),
        ("log_probs", c_vp), ("log_prob_rows", c_i64), ("num_classes", c_i32),
        ("h_first_row", c_vp), ("h_frames", c_vp),
        ("output_beam", c_f32), ("max_states", c_i32), ("max_arcs", c_i32),
        ("zero_fill", c_vp), ("zero_fill_bytes", c_sz),
    ]


class LatticeOut(ctypes.Structure):
    _fields_ = [
        ("row_splits1", c_vp), ("row_ids1", c_vp), ("row_splits2", c_vp), ("row_ids2", c_vp),
        ("arcs", c_vp), ("arc_map_a", c_vp), ("arc_map_b", c_vp),
        ("level_offsets", c_vp), ("level_splits", c_vp),
    ]


class PrunedArgs(ctypes.Structure):
    _fields_ = [
        ("num_fsas", c_i32), ("num_states", c_i32), ("num_arcs", c_i32),
        ("a_row_splits1", c_vp), ("a_row_splits2", c_vp), ("a_arcs", c_vp),
        ("scores", c_vp), ("rows", c_i32), ("cols", c_i32), ("num_seqs", c_i32),
        ("b_row_splits", c_vp), ("h_b_row_splits", c_vp),
        ("search_beam", c_f32), ("output_beam", c_f32),
        ("min_active_states", c_i32), ("max_active_states", c_i32), ("allow_partial", c_i32),
        ("max_states_per_seq", c_i64), ("max_arcs_per_seq", c_i64), ("team_ctas", c_i32),
    ]


class OnlineStream(ctypes.Structure):
    _fields_ = [
        ("num_states", c_i32), ("num_arcs", c_i32),
        ("astate", c_vp), ("forward", c_vp), ("arc0", c_vp), ("arc_graph", c_vp),
        ("arc_score", c_vp), ("arc_dest", c_vp), ("frame_state0", c_vp), ("frame_arc0", c_vp),
    ]


class OnlineArgs(ctypes.Structure):
    _fields_ = [
        ("num_states", c_i32), ("num_arcs", c_i32),
        ("a_row_splits1", c_vp), ("a_row_splits2", c_vp), ("a_arcs", c_vp),
        ("scores", c_vp), ("rows", c_i32), ("cols", c_i32), ("num_seqs", c_i32),
        ("b_row_splits", c_vp), ("h_b_row_splits", c_vp),
        ("search_beam", c_f32), ("output_beam", c_f32),
        ("min_active_states", c_i32), ("max_active_states", c_i32), ("allow_partial", c_i32),
        ("h_hist", c_vp), ("max_states_per_seq", c_i64), ("max_arcs_per_seq", c_i64),
        ("team_ctas", c_i32),
    ]


class FsaView(ctypes.Structure):
    _fields_ = [
        ("num_fsas", c_i32), ("num_states", c_i32), ("num_arcs", c_i32),
        ("row_splits1", c_vp), ("row_ids1", c_vp), ("row_splits2", c_vp), ("row_ids2", c_vp),
        ("arcs", c_vp),
        ("in_splits", c_vp), ("in_arcs", c_vp), ("in_src", c_vp), ("in_score", c_vp),
        ("level_offsets", c_vp), ("level_splits", c_vp),
        ("strict_layers", c_i32), ("max_layers", c_i32), ("max_layer_states", c_i32),
        ("max_layer_arcs", c_i32),
    ]


def _sig(name, restype, argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


_sig("k2b200_last_error", ctypes.c_char_p, [])
_sig("k2b200_abi_version", c_i32, [])
_sig("k2b200_kernel_launch_count", c_i64, [])
_sig("k2b200_profile_enable", None, [c_i32])
_sig("k2b200_profile_kernel", ctypes.c_char_p, [c_i32])
_sig("k2b200_profile_read_ms", ctypes.c_double, [c_i32, ctypes.POINTER(c_i64)])
_sig("k2b200_row_splits_to_row_ids", c_i32, [c_vp, c_i32, c_vp, c_i32, c_vp])
_sig("k2b200_upload_i32", c_i32, [c_vp, c_i64, c_vp, c_vp])
_sig("k2b200_dense_loss_backward_log_probs", c_i32,
     [ctypes.POINTER(IntersectArgs), c_vp, c_sz, c_vp, c_i32, c_vp, c_vp, c_vp, c_i32, c_vp])
_sig("k2b200_online_decode_workspace_bytes", c_i32,
     [ctypes.POINTER(OnlineArgs), ctypes.POINTER(c_sz)])
_sig("k2b200_online_decode_load", c_i32,
     [ctypes.POINTER(OnlineArgs), c_vp, c_i32, ctypes.POINTER(OnlineStream), c_vp])
_sig("k2b200_online_decode_load_all", c_i32,
     [ctypes.POINTER(OnlineArgs), c_vp, ctypes.POINTER(OnlineStream), c_vp])
_sig("k2b200_online_decode_store_all", c_i32,
     [ctypes.POINTER(OnlineArgs), c_vp, ctypes.POINTER(OnlineStream), c_vp])
_sig("k2b200_online_decode_run", c_i32,
     [ctypes.POINTER(OnlineArgs), c_vp, c_sz, c_vp, c_vp, c_vp, c_vp, ctypes.POINTER(c_i32),
      ctypes.POINTER(c_i32), ctypes.POINTER(c_i32)])
_sig("k2b200_online_decode_emit", c_i32,
     [ctypes.POINTER(OnlineArgs), c_vp, c_sz, c_vp, ctypes.POINTER(LatticeOut)])
_sig("k2b200_online_decode_store", c_i32,
     [ctypes.POINTER(OnlineArgs), c_vp, c_i32, ctypes.POINTER(OnlineStream), c_vp])
_sig("k2b200_fsa_scores_backprop", c_i32,
     [ctypes.POINTER(FsaView), c_i32, c_i32, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp])
_sig("k2b200_fsa_arc_post_backprop", c_i32,
     [ctypes.POINTER(FsaView), c_i32, c_vp, c_vp, c_vp, c_vp])
_sig("k2b200_intersect_dense_pruned_workspace_bytes", c_i32,
     [ctypes.POINTER(PrunedArgs), ctypes.POINTER(c_sz), ctypes.POINTER(c_i64)])
_sig("k2b200_intersect_dense_pruned_search", c_i32,
     [ctypes.POINTER(PrunedArgs), c_vp, c_sz, c_vp, ctypes.POINTER(c_i32),
      ctypes.POINTER(c_i32), ctypes.POINTER(c_i32)])
_sig("k2b200_intersect_dense_pruned_emit", c_i32,
     [ctypes.POINTER(PrunedArgs), c_vp, c_sz, c_vp, ctypes.POINTER(LatticeOut)])
_sig("k2b200_exclusive_sum_tmp_bytes", c_sz, [c_i64])
_sig("k2b200_exclusive_sum", c_i32, [c_vp, c_vp, c_i64, c_vp, c_vp])
_sig("k2b200_exclusive_sum_static_max_len", c_i64, [])
_sig("k2b200_exclusive_sum_static", c_i32, [c_vp, c_vp, c_i64, c_vp])
_sig("k2b200_fsa_incoming_tmp_bytes", c_sz, [c_i32, c_i32])
_sig("k2b200_fsa_incoming", c_i32,
     [c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp])
_sig("k2b200_intersect_dense_workspace_bytes", c_i32,
     [ctypes.POINTER(IntersectArgs), ctypes.POINTER(c_sz), ctypes.POINTER(c_i64)])
_sig("k2b200_intersect_dense_prune", c_i32,
     [ctypes.POINTER(IntersectArgs), c_vp, c_sz, c_vp, ctypes.POINTER(c_i32),
      ctypes.POINTER(c_i32), ctypes.POINTER(c_f32), ctypes.POINTER(c_i32),
      ctypes.POINTER(c_i32)])
_sig("k2b200_intersect_dense_emit", c_i32,
     [ctypes.POINTER(IntersectArgs), c_vp, c_sz, c_vp, ctypes.POINTER(LatticeOut)])
_sig("k2b200_dense_loss_supported", c_i32,
     [ctypes.POINTER(IntersectArgs), ctypes.POINTER(c_i32)])
_sig("k2b200_dense_loss_workspace_bytes", c_i32,
     [ctypes.POINTER(IntersectArgs), ctypes.POINTER(c_sz)])
_sig("k2b200_dense_loss_forward", c_i32,
     [ctypes.POINTER(IntersectArgs), c_vp, c_sz, c_vp, c_vp, ctypes.POINTER(c_f32)])
_sig("k2b200_dense_loss_backward", c_i32,
     [ctypes.POINTER(IntersectArgs), c_vp, c_sz, c_vp, c_i32, c_vp, c_vp, c_vp])
_sig("k2b200_band_tables_bytes", c_i32, [c_i32, ctypes.POINTER(c_sz), ctypes.POINTER(c_sz)])
_sig("k2b200_band_tables", c_i32, [c_vp, c_i32, c_vp, c_vp, c_i32, c_vp, c_vp, c_vp, c_vp])
_sig("k2b200_band_loss_supported", c_i32,
     [ctypes.POINTER(BandLossArgs), ctypes.POINTER(c_i32)])
_sig("k2b200_band_loss_workspace_bytes", c_i32,
     [ctypes.POINTER(BandLossArgs), ctypes.POINTER(c_sz)])
_sig("k2b200_band_loss_forward", c_i32,
     [ctypes.POINTER(BandLossArgs), c_vp, c_sz, c_vp, c_vp, ctypes.POINTER(c_f32)])
_sig("k2b200_band_loss_backward", c_i32,
     [ctypes.POINTER(BandLossArgs), c_vp, c_sz, c_vp, c_i32, c_vp, c_vp, c_vp, c_i32, c_i32,
      c_vp])
_sig("k2b200_band_loss_status", c_i32,
     [ctypes.POINTER(BandLossArgs), c_vp, c_sz, c_vp, ctypes.POINTER(c_i32)])
_sig("k2b200_debug_set_copy_wait_limit", None, [c_i32])
_sig("k2b200_fsa_levels_tmp_bytes", c_sz, [c_i32])
_sig("k2b200_fsa_levels", c_i32,
     [c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp])
_sig("k2b200_fsa_scores_scratch_bytes", c_sz, [ctypes.POINTER(FsaView)])
_sig("k2b200_fsa_scores", c_i32,
     [ctypes.POINTER(FsaView), c_i32, c_i32, c_vp, c_vp, c_vp, c_vp, c_sz, c_vp])
_sig("k2b200_fsa_tot_scores", c_i32, [c_vp, c_i32, c_i32, c_vp, c_vp, c_vp])
_sig("k2b200_fsa_arc_post", c_i32,
     [c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp, c_vp])
_sig("k2b200_tot_scores_log_backward", c_i32,
     [c_vp, c_vp, c_i32, c_i32, c_vp, c_vp, c_i64, c_vp, c_vp])
_sig("k2b200_tot_scores_tropical_backward", c_i32,
     [c_vp, c_vp, c_i32, c_vp, c_i32, c_i32, c_vp, c_i64, c_vp, c_vp])
_sig("k2b200_index_add", c_i32, [c_vp, c_vp, c_i32, c_vp, c_i64, c_vp])
_sig("k2b200_index_select_i32", c_i32, [c_vp, c_i64, c_vp, c_i32, c_vp, c_vp])
_sig("k2b200_ctc_graph_tmp_bytes", c_sz, [c_i32])
_sig("k2b200_ctc_graph", c_i32,
     [c_vp, c_vp, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp, c_vp, c_vp, c_vp])
_sig("k2b200_dense_fsa_vec_fill", c_i32,
     [c_vp, c_i64, c_i64, c_i32, c_vp, c_vp, c_i32, c_vp, c_i32, c_vp])
_sig("k2b200_dense_fsa_vec_backward", c_i32,
     [c_vp, c_i64, c_i64, c_i32, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp, c_vp])
_sig("k2b200_dense_fsa_vec_from_logits", c_i32,
     [c_vp, c_i64, c_i64, c_i32, c_vp, c_vp, c_i32, c_vp, c_i32, c_vp])
_sig("k2b200_dense_fsa_vec_from_logits_backward", c_i32,
     [c_vp, c_vp, c_i64, c_i64, c_i32, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp, c_vp])
_sig("k2b200_shortest_path_tmp_bytes", c_sz, [c_i32])
_sig("k2b200_shortest_path", c_i32, [c_vp, c_vp, c_vp, c_i32, c_vp, c_vp, c_vp, c_vp])
_sig("k2b200_fsa_properties_tmp_bytes", c_sz, [c_i32, c_i32])
_sig("k2b200_fsa_properties", c_i32,
     [c_vp, c_vp, c_vp, c_vp, c_vp, c_i32, c_i32, c_i32, c_vp, c_vp, c_vp])

_sig("k2b200_peer_reduce_create", c_i32, [ctypes.POINTER(c_vp), c_vp])
_sig("k2b200_peer_reduce_open", c_i32, [c_vp, ctypes.POINTER(c_vp)])
_sig("k2b200_peer_reduce_close", c_i32, [c_vp])
_sig("k2b200_peer_reduce_destroy", c_i32, [c_vp])
_sig("k2b200_loss_sum_all_reduce", c_i32,
     [c_vp, c_i32, c_i32, ctypes.c_double, ctypes.c_double, ctypes.POINTER(c_vp), c_i32, c_i32,
      ctypes.c_uint64, c_i32, c_vp, c_vp, c_vp])
_sig("k2b200_peer_reduce_status", c_i32, [c_vp, c_vp, ctypes.POINTER(c_i32)])

EXPORTED = [
    "k2b200_last_error", "k2b200_abi_version", "k2b200_kernel_launch_count",
    "k2b200_profile_enable", "k2b200_profile_kernel", "k2b200_profile_read_ms", "k2b200_row_splits_to_row_ids",
    "k2b200_upload_i32",
    "k2b200_exclusive_sum_tmp_bytes", "k2b200_exclusive_sum",
    "k2b200_exclusive_sum_static_max_len", "k2b200_exclusive_sum_static", "k2b200_fsa_incoming_tmp_bytes",
    "k2b200_fsa_incoming", "k2b200_intersect_dense_workspace_bytes",
    "k2b200_intersect_dense_prune", "k2b200_intersect_dense_emit", "k2b200_fsa_scores",
    "k2b200_fsa_scores_scratch_bytes",
    "k2b200_fsa_tot_scores", "k2b200_fsa_arc_post", "k2b200_tot_scores_log_backward",
    "k2b200_tot_scores_tropical_backward", "k2b200_index_add", "k2b200_index_select_i32",
    "k2b200_shortest_path_tmp_bytes", "k2b200_shortest_path",
    "k2b200_dense_fsa_vec_fill", "k2b200_dense_fsa_vec_backward",
    "k2b200_dense_fsa_vec_from_logits", "k2b200_dense_fsa_vec_from_logits_backward",
    "k2b200_ctc_graph_tmp_bytes", "k2b200_ctc_graph",
    "k2b200_fsa_properties_tmp_bytes", "k2b200_fsa_properties",
    "k2b200_fsa_levels_tmp_bytes", "k2b200_fsa_levels",
    "k2b200_dense_loss_supported", "k2b200_dense_loss_workspace_bytes",
    "k2b200_dense_loss_forward", "k2b200_dense_loss_backward",
    "k2b200_intersect_dense_pruned_workspace_bytes", "k2b200_intersect_dense_pruned_search",
    "k2b200_intersect_dense_pruned_emit",
    "k2b200_fsa_scores_backprop", "k2b200_fsa_arc_post_backprop",
    "k2b200_dense_loss_backward_log_probs",
    "k2b200_peer_reduce_create", "k2b200_peer_reduce_open", "k2b200_peer_reduce_close",
    "k2b200_peer_reduce_destroy", "k2b200_loss_sum_all_reduce", "k2b200_peer_reduce_status",
    "k2b200_online_decode_workspace_bytes", "k2b200_online_decode_load",
    "k2b200_online_decode_run", "k2b200_online_decode_emit", "k2b200_online_decode_store",
    "k2b200_online_decode_load_all", "k2b200_online_decode_store_all",
    "k2b200_band_tables_bytes", "k2b200_band_tables", "k2b200_band_loss_supported",
    "k2b200_band_loss_workspace_bytes", "k2b200_band_loss_forward",
    "k2b200_band_loss_backward", "k2b200_band_loss_status",
    "k2b200_debug_set_copy_wait_limit",
]


def check(status: int) -> None:
    """The reference raises a C++ exception that Python sees as RuntimeError
    (k2/csrc/log.h:196-203); a non-zero status is surfaced the same way."""
    if status != 0:
        raise RuntimeError(lib.k2b200_last_error().decode(errors="replace"))


_dummy = {}


def ptr(t) -> int:
    """Device address of a tensor; None -> NULL.  Empty tensors have no storage
    address in torch, so they get the address of a small per-device scratch
    buffer (never dereferenced: their size is 0)."""
    if t is None:
        return None
    if t.numel() == 0:
        key = str(t.device)
        if key not in _dummy:
            _dummy[key] = torch.zeros(64, dtype=torch.int32, device=t.device)
        return _dummy[key].data_ptr()
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_of(device) -> int:
    """The current CUDA stream of `device` as a raw handle."""
    if _raw_stream is not None:
        idx = device.index if isinstance(device, torch.device) else torch.device(device).index
        return _raw_stream(torch.cuda.current_device() if idx is None else idx)
    return torch.cuda.current_stream(device).cuda_stream


# Workspaces of the loss calls are a gigabyte or more and live from a forward to its
# backward.  Handed back to torch's caching allocator they get split for smaller tensors,
# after which the next step needs a fresh cudaMalloc, which waits for the whole device.
# So the last few are kept here, per device and stream (a workspace that comes back
# may still be read by kernels queued on that stream; the next user queues behind them).
_WS_POOL_MIN = 32 << 20   # smaller ones go through torch's allocator
_WS_POOL_KEEP = 3         # idle workspaces kept per (device, stream)
_ws_idle = {}
_ws_lock = threading.Lock()


class Workspace(object):
    """A device byte buffer that returns to the pool when the last reference goes."""
    __slots__ = ("tensor", "_key")

    def __init__(self, tensor: torch.Tensor, key) -> None:
        self.tensor = tensor
        self._key = key

    def __del__(self):
        try:
            if self._key is None:
                return
            with _ws_lock:
                idle = _ws_idle.setdefault(self._key, [])
                idle.append(self.tensor)
                if len(idle) > _WS_POOL_KEEP:
                    idle.sort(key=lambda t: t.numel())
                    idle.pop(0)
        except Exception:  # interpreter shutdown
            pass


def workspace(nbytes: int, device) -> Workspace:
    """A buffer of at least `nbytes` bytes on `device` for the current stream."""
    device = torch.device(device)
    if nbytes < _WS_POOL_MIN:
        return Workspace(torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device), None)
    key = (device.index, stream_of(device))
    with _ws_lock:
        idle = _ws_idle.get(key, [])
        best = None
        for k, t in enumerate(idle):
            if nbytes <= t.numel() <= 2 * nbytes and (best is None or
                                                      t.numel() < idle[best].numel()):
                best = k
        if best is not None:
            return Workspace(idle.pop(best), key)
    # some headroom, so that a slightly larger batch still fits
    return Workspace(torch.empty(nbytes + nbytes // 8, dtype=torch.uint8, device=device), key)


def release_workspaces() -> None:
    """Gives the idle workspaces back to torch's allocator."""
    with _ws_lock:
        _ws_idle.clear()


def upload_i32(arr, device) -> torch.Tensor:
    """Host int32 array -> new device tensor.  The values travel as kernel parameters
    (k2b200_upload_i32): no stream synchronisation, unlike a torch copy from pageable
    memory, and no queueing behind a large host-to-device transfer in flight."""
    import numpy as np
    arr = np.ascontiguousarray(arr, dtype=np.int32).reshape(-1)
    out = torch.empty(arr.shape[0], dtype=torch.int32, device=device)
    if arr.shape[0]:
        with torch.cuda.device(out.device):
            check(lib.k2b200_upload_i32(arr.ctypes.data, arr.shape[0], out.data_ptr(),
                                        stream_of(out.device)))
    return out


def require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"{what} must be a CUDA tensor: k2_b200 runs on sm_100a only and has no CPU path")


def launch_count() -> int:
    """Kernels launched by libk2b200.so so far (counted inside the library)."""
    return int(lib.k2b200_kernel_launch_count())


PHASES = ["viterbi", "prune", "emit", "scores", "post", "incoming", "dense", "chain", "grad"]


def profile_enable(on: bool) -> None:
    lib.k2b200_profile_enable(int(on))


def profile_kernels():
    """{phase: name of the kernel(s) that last ran under it}."""
    return {name: lib.k2b200_profile_kernel(k).decode() for k, name in enumerate(PHASES)}


def profile_read():
    """{phase: (milliseconds, intervals)} since the last read."""
    out = {}
    for k, name in enumerate(PHASES):
        n = c_i64()
        ms = lib.k2b200_profile_read_ms(k, ctypes.byref(n))
        out[name] = (float(ms), int(n.value))
    return out

"""Benchmark of the dense-intersection loss path: CTC loss forward + backward.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                  [--workload ctc_large] [--scale 1.0]

Workload (default): "ctc_large" - 64 utterances, T=1000, C=500, 600..1000 frames
each, transcripts of 100..250 tokens, standard CTC graphs, output_beam 10;
synthetic (seeded Gaussian logits, random transcripts).

One step = DenseFsaVec construction from device-resident log-probs, ctc_loss
(intersect_dense + log-semiring total scores in float64) and the backward pass to
the gradient w.r.t. the log-probs.  `value` is supervised frames per second with
the inputs resident in HBM; `e2e` times the same step from pinned host log-probs
(host->device copy inside the timed region) to the loss on the host.  With N > 1
every rank runs its own batch (weak scaling, utterances are independent) and the
only collective is one all-reduce of [loss, frames].

--impl reference times the reference's own CPU code for the same path
(oracle/_ref/libk2ref.so when present, else the C restatement in oracle/) on the
host cores, single-threaded as the reference is by construction.

Diagnostics of the N > 1 arm (environment): K2B_NCCL_REDUCE=1 exchanges [loss, frames]
with torch.distributed on a helper thread instead of the peer-memory kernel,
K2B_NO_REDUCE=1 runs the ranks side by side with no exchange at all, K2B_PEER_POLL=n
bounds the kernel's wait for a peer to n polls, K2B_NO_NUMA_BIND=1 leaves the ranks
unbound.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default="ctc_large")
    p.add_argument("--scale", type=float, default=1.0)
    p.add_argument("--utterances", type=int, default=None,
                   help="lfmmi_den only: batch size, e.g. 16 = one GPU's share of 128 split 8 ways")
    p.add_argument("--max-frames", type=int, default=None,
                   help="cut every sequence of the workload to its first frames (profiling)")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-lfmmi-den", action="store_true",
                   help="skip the LF-MMI denominator block of the default line")
    p.add_argument("--decode", action="store_true",
                   help="time the decoding path instead: hlg_decode through intersect_dense_pruned")
    p.add_argument("--chunk", type=int, default=0,
                   help="with --decode: decode chunk by chunk (OnlineDenseIntersecter), this many "
                        "frames per chunk")
    return p.parse_args()


def load_synthetic():
    """k2_b200/synthetic.py loaded by path: the CPU arms make their inputs from it without
    importing the package (and with it the CUDA library)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "_k2b200_synthetic", os.path.join(ROOT, "k2_b200", "synthetic.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = mod  # dataclasses look their module up by name
    spec.loader.exec_module(mod)
    return mod


def make_workload(args, seed, syn=None, name=None):
    syn = syn or load_synthetic()
    name = name or args.workload
    if name == "lfmmi_den" and args.utterances is not None:
        return syn.lfmmi_den(seed=seed, scale=args.scale, utterances=args.utterances)
    w = syn.WORKLOADS[name](seed=seed, scale=args.scale)
    if getattr(args, "max_frames", None):
        # the same batch cut to its first frames: a case small enough for an ncu capture of
        # a workload whose grids would otherwise hold tens of GB
        import dataclasses
        t = int(args.max_frames)
        seg = w.supervision_segments.clone()
        seg[:, 2] = seg[:, 2].clamp(max=t)
        w = dataclasses.replace(w, log_probs=w.log_probs[:, :t].contiguous(),
                                supervision_segments=seg)
    return w


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed
    region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU arm
def cpu_reference_step(w, graphs_host, scores, row_splits, impl_mod):
    """The reference's path on the host: intersect_dense, log-semiring forward and
    backward scores in double, total scores, arc posteriors and the gradient
    scatter.  Returns (seconds, loss)."""
    import numpy as np
    t0 = time.perf_counter()
    lat = impl_mod.intersect_dense(graphs_host, scores, row_splits, w.output_beam)
    fwd = impl_mod.forward_scores(lat, True, True)
    bwd = impl_mod.backward_scores(lat, True, True)
    tot, post = impl_mod.tot_scores_and_arc_post(lat, fwd, bwd, True)
    grad = np.zeros(scores.size, np.float32)
    np.add.at(grad, lat.arc_map_b, np.exp(post).astype(np.float32))
    dt = time.perf_counter() - t0
    return dt, float(-tot.sum())


def host_inputs(w, impl_mod):
    """Graphs and the DenseFsaVec score matrix of a workload as host arrays, made with
    numpy and the CPU implementation itself (no part of the CUDA package)."""
    import numpy as np
    from oracle.common import HostFsaVec
    if w.symbols is not None:
        graphs = impl_mod.ctc_graphs(w.symbols, w.modified)
    else:  # one graph, stacked once per utterance (the reference cannot share it)
        n = w.supervision_segments.shape[0]
        S, A = len(w.graph_row_splits2) - 1, len(w.graph_arcs)
        rs1 = (np.arange(n + 1, dtype=np.int64) * S).astype(np.int32)
        rs2 = (np.arange(n, dtype=np.int64)[:, None] * A +
               w.graph_row_splits2[None, :-1]).reshape(-1)
        rs2 = np.append(rs2, n * A).astype(np.int32)
        graphs = HostFsaVec(rs1, rs2, np.tile(w.graph_arcs, (n, 1)))
    scores, row_splits = host_scores(w)
    return graphs, scores, row_splits


def host_scores(w):
    """The DenseFsaVec score matrix and row_splits of a workload as host arrays."""
    import numpy as np
    seg = w.supervision_segments.numpy()
    N, T, C = w.log_probs.shape
    rows = int(seg[:, 2].sum() + len(seg))
    scores = np.full((rows, C + 1), -np.inf, np.float32)
    row_splits = np.zeros(len(seg) + 1, np.int32)
    lp = w.log_probs.numpy()
    r = 0
    for i, (n, s, d) in enumerate(seg.tolist()):
        scores[r:r + d, 1:] = lp[n, s:s + d]
        scores[r + d, 0] = 0.0
        r += d + 1
        row_splits[i + 1] = r
    return scores, row_splits


def pick_cpu_impl():
    from oracle import ref
    if ref.available():
        return ref, "reference"
    from oracle import oracle
    return oracle, "port"


_SHARDS = None  # per-process inputs of the sharded CPU run (inherited through fork)


def _shard_inputs(w, graphs, scores, row_splits, num_shards):
    """Split a batch by utterance (round-robin over the duration-sorted list, as
    the multi-GPU path does) into host inputs for independent reference runs."""
    import numpy as np
    from oracle.common import HostFsaVec
    n = len(row_splits) - 1
    shards = []
    for r in range(num_shards):
        idx = list(range(r, n, num_shards))
        if not idx:
            continue
        rs1, rs2, arcs, rows, brs = [0], [0], [], [], [0]
        for i in idx:
            s0, s1 = int(graphs.row_splits1[i]), int(graphs.row_splits1[i + 1])
            a0, a1 = int(graphs.row_splits2[s0]), int(graphs.row_splits2[s1])
            rs1.append(rs1[-1] + s1 - s0)
            rs2.extend((graphs.row_splits2[s0 + 1:s1 + 1] - a0 + rs2[-1]).tolist())
            arcs.append(graphs.arcs[a0:a1])
            rows.append(scores[row_splits[i]:row_splits[i + 1]])
            brs.append(brs[-1] + int(row_splits[i + 1] - row_splits[i]))
        shards.append((HostFsaVec(np.asarray(rs1, np.int32), np.asarray(rs2, np.int32),
                                  np.concatenate(arcs)),
                       np.ascontiguousarray(np.concatenate(rows)), np.asarray(brs, np.int32)))
    return shards


def _run_shard(k):
    w, impl_name, shards = _SHARDS
    impl_mod = __import__("oracle." + impl_name, fromlist=[impl_name])
    g, sc, brs = shards[k]
    return cpu_reference_step(w, g, sc, brs, impl_mod)


def cpu_reference_sharded(w, graphs, scores, row_splits, impl_mod, cores, repeats):
    """Wall time of the reference path with the batch sharded by utterance over
    `cores` worker processes (the reference itself is single-threaded; sharding
    independent utterances is what a caller with more cores can do)."""
    global _SHARDS
    import multiprocessing as mp
    shards = _shard_inputs(w, graphs, scores, row_splits, cores)
    _SHARDS = (w, impl_mod.__name__.split(".")[-1], shards)
    ctx = mp.get_context("fork")
    best = None
    with ctx.Pool(len(shards)) as pool:
        pool.map(_run_shard, range(len(shards)))  # warm-up
        for _ in range(repeats):
            t0 = time.perf_counter()
            pool.map(_run_shard, range(len(shards)))
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
    return best, len(shards)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = make_workload(args, 0)
    impl_mod, kind = pick_cpu_impl()
    graphs, scores, row_splits = host_inputs(w, impl_mod)
    frames = w.num_frames
    # single thread, as the reference runs this path
    cpu_reference_step(w, graphs, scores, row_splits, impl_mod)
    single = min(cpu_reference_step(w, graphs, scores, row_splits, impl_mod)[0]
                 for _ in range(2))
    # all host cores: one reference run per utterance shard
    cores = max(1, min(os.cpu_count() or 1, len(row_splits) - 1))
    import multiprocessing as mp
    global _SHARDS
    shards = _shard_inputs(w, graphs, scores, row_splits, cores)
    _SHARDS = (w, impl_mod.__name__.split(".")[-1], shards)
    used = len(shards)
    with mp.get_context("fork").Pool(used) as pool:
        pool.map(_run_shard, range(used))  # warm-up
        t0 = time.perf_counter()
        for _ in range(args.steps):
            pool.map(_run_shard, range(used))
        total = time.perf_counter() - t0
    value = frames * args.steps / total
    line = {
        "impl": "reference", "metric": "ctc_loss_fwd_bwd_frames_per_sec", "value": value,
        "unit": "frames/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32+f64", "data": "synthetic",
        "config": workload_config(w, args),
        "cpu_baseline": {"value": value, "unit": "frames/s", "cores": used, "kind": kind,
                         "single_thread_value": frames / single,
                         "sample": f"{args.steps} full batches of {args.workload} "
                                   f"({frames} frames each): intersect + log scores + posteriors "
                                   f"+ gradient scatter, sharded by utterance over {used} worker "
                                   "processes (the reference's path itself is single-threaded)"},
        "e2e": {"value": value, "unit": "frames/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(w, args):
    return {"workload": w.name, "utterances": int(w.log_probs.shape[0]),
            "max_frames": int(w.log_probs.shape[1]), "classes": int(w.log_probs.shape[2]),
            "frames": w.num_frames, "output_beam": w.output_beam, "scale": args.scale,
            "l2": "inputs larger than L2: a step touches the log-probs and their gradient "
                  "(128 MB each at ctc_large), the two Viterbi grids and the lists of surviving "
                  "states, several times the 126 MB L2; no explicit flush"}


# --------------------------------------------------------------------------- GPU arm
def algorithmic_bytes(frames, N, T, C, A, A_out, S_out, lattice_written):
    """Bytes that must cross HBM at least once per step: every supervised log-prob row
    read once, the dense gradient written once (zeros included), the graph arcs once,
    and - only when the timed path writes the lattice - its arcs, arc maps and rows."""
    b = 4 * frames * C + 4 * N * T * C + 16 * A
    if lattice_written:
        b += 24 * A_out + 8 * S_out
    return b


def implementation_bytes(phase, kernel, frames, N, T, C, A, A_out, S_out, grid_states):
    """What the kernels of a phase actually move per step by their design (reads and
    writes they cannot avoid as written) - the figure ncu's DRAM traffic is checked
    against, not a roofline denominator."""
    R = frames
    table = {
        # every row by both directions, both grids written
        "BandViterbi": 2 * 4 * R * C + 8 * grid_states,
        # BandKeep reads both grids and writes 64 bytes of keep bits per level; BandPrep reads
        # them back, per surviving state two table entries and five grid values, and writes a
        # list entry (8 bytes) and a factor record (32 bytes) per entry of the padded lists
        # (at least 32 entries per level)
        "BandKeep+BandPrep": 8 * grid_states + 128 * (R + 2 * N) + 84 * S_out +
                             40 * max(S_out, 32 * (R + 2 * N)),
        # both directions read the factor records and write a value per padded entry
        "BandChainLists": 2 * 40 * max(S_out, 32 * (R + 2 * N)),
        # list entry, alpha and beta per surviving state, a gradient element per (frame, label)
        "BandGrad": 24 * S_out + 4 * S_out,
        "RegisterViterbi": 2 * 4 * R * C + 8 * grid_states,
        "LanesViterbi": 2 * 4 * R * C + 8 * grid_states,
        "GridChainLanes": 2 * 12 * R * C + 16 * grid_states + 32 * S_out,
        "ArcMasks+GridChainMasked": 24 * R * C + 16 * grid_states + 32 * S_out,
        "GridGradItems": 8 * grid_states + 32 * S_out + 12 * R * C + 4 * A_out,
        "GridGradLanes": 8 * grid_states + 32 * S_out + 12 * R * C + 4 * A_out,
        "GridGradWarp": 8 * grid_states + 32 * S_out + 12 * R * C + 4 * A_out,
        "CountStates": 8 * grid_states,
        "ProbScoresStaged": 16 * A_out + 16 * S_out,
        "EmitLattice": 8 * grid_states + 24 * A_out + 8 * S_out,
    }
    return table.get(kernel)


def run_ours(args):
    import numpy as np
    import torch

    import k2_b200 as k2
    from k2_b200 import _lib
    from k2_b200 import synthetic as syn
    from k2_b200.parallel import HostPrefetcher, shard_segments

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    numa = {"bound": False}
    if world > 1 and os.environ.get("K2B_NO_NUMA_BIND") is None:
        from k2_b200.parallel import bind_to_gpu_numa_node
        numa = bind_to_gpu_numa_node(dev)  # before the pinned host buffers are allocated
    if world > 1:
        every = [None] * world
        dist.all_gather_object(every, numa)
        numa = {"by_rank": [[n.get("node"), n.get("cpus_on_node"), n.get("cpus_allowed"),
                             int(n.get("bound", False))] for n in every],
                "columns": ["node", "cpus_on_node", "cpus_allowed", "bound"]}
    # every rank owns a whole batch (weak scaling); seeds differ per rank
    w = make_workload(args, rank, syn)
    frames = w.num_frames
    graphs = syn.build_graphs(w, dev)
    host_lp = w.log_probs.pin_memory()
    dev_lp = w.log_probs.to(dev)
    seg = w.supervision_segments
    # per step the ranks all-reduce [loss, frames] on a side stream, right after the
    # total scores exist and beside the gradient kernels (the gradient of a summed loss
    # does not depend on the other ranks)
    from k2_b200.parallel import LossReducer, PeerLossReducer
    reducer = None
    if dist is not None and os.environ.get("K2B_NO_REDUCE"):
        pass  # no exchange at all: what running the ranks side by side costs by itself
    elif dist is not None:  # K2B_NCCL_REDUCE=1: the collective library instead of peer stores
        if os.environ.get("K2B_NCCL_REDUCE"):
            reducer = LossReducer(dev)
        else:
            try:
                reducer = PeerLossReducer(dev, poll_limit=int(os.environ.get("K2B_PEER_POLL", -1)))
            except RuntimeError as e:  # raised on every rank alike
                if rank == 0:
                    print(f"bench: {e}; using the NCCL all-reduce", file=sys.stderr)
                reducer = LossReducer(dev)
    frames_of = {}

    def loss_step(lp, g, segments, beam, read_totals=False):
        lp = lp.detach().requires_grad_(True)
        dense = k2.DenseFsaVec(lp, segments)
        loss = k2.ctc_loss(g, dense, output_beam=beam, reduction="sum")
        if reducer is not None:
            nf = frames_of.get(id(segments))
            if nf is None:
                nf = frames_of[id(segments)] = int(segments[:, 2].sum())
            reducer.submit(loss, nf)
        loss.backward()
        if reducer is not None:
            # the totals are consumed on the host (logging): a step that does not read them
            # does not make its stream wait for the other ranks either
            if isinstance(reducer, PeerLossReducer):
                return reducer.result(join=read_totals)[0], lp.grad
            return reducer.result()[0], lp.grad
        return loss.detach(), lp.grad

    def step(lp, read_totals=False):
        return loss_step(lp, graphs, seg, w.output_beam, read_totals)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(nsteps, fn, profile=False):
        """K steps of fn() between barriers; device time, max over ranks."""
        barrier()
        if profile:
            _lib.profile_enable(True)
        launches0 = _lib.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(nsteps):
            fn()
        e1.record()
        barrier()
        wall = time.perf_counter() - t0
        ms = e0.elapsed_time(e1)
        launches = _lib.launch_count() - launches0
        phases = None
        if profile:
            phases = _lib.profile_read()
            _lib.profile_enable(False)
        timed.own_ms = ms
        return max_over_ranks(ms), wall, launches, phases

    def timed_from_host(nsteps, pipelined):
        """End to end: every step's log-probs are copied from pinned host memory inside
        the timed region and every step's loss is read on the host.  pipelined: the copy
        of step k+1 runs on a copy stream while step k computes (HostPrefetcher), as a
        training loop feeds the GPU; otherwise copy, compute and read-back follow one
        another."""
        pf = HostPrefetcher(dev)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if pipelined:
            pf.submit(host_lp)
        for k in range(nsteps):
            if pipelined:
                lp = pf.get()
                if k + 1 < nsteps:
                    pf.submit(host_lp)
            else:
                lp = host_lp.to(dev, non_blocking=True)
            out, _ = step(lp, read_totals=True)
            float(out.item())
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # before the warm-up so that it is sampling by the timed region
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step(dev_lp)
    ms, wall, launches, _ = timed(args.steps, lambda: step(dev_lp))
    own_ms = timed.own_ms / args.steps
    # the same steps again with per-phase events, for the roofline of the top kernel
    _, _, _, phases = timed(args.steps, lambda: step(dev_lp), profile=True)
    kernels = _lib.profile_kernels()
    # time inside this library's kernels per step on every rank
    busy = sum(v[0] for k, v in phases.items()) / args.steps
    busy_by_rank, ms_by_rank = [busy], [own_ms]
    if dist is not None:
        t = torch.zeros(2, world, dtype=torch.float64, device=dev)
        t[0, rank] = busy
        t[1, rank] = own_ms
        dist.all_reduce(t)
        busy_by_rank = [float(x) for x in t[0].tolist()]
        ms_by_rank = [float(x) for x in t[1].tolist()]
    timed_from_host(2, False)
    serial_ms = timed_from_host(args.steps, False)
    timed_from_host(2, True)
    e2e_ms = timed_from_host(args.steps, True)

    # cold graphs: a training loop sees new transcripts every batch, so the graphs are
    # built (ctc_graph on the device) and prepared inside the step
    cold_ms = None
    if w.symbols is not None:
        rng = np.random.default_rng(1234 + rank)
        C = int(w.log_probs.shape[2])
        fresh = [[rng.integers(1, C, size=len(s)).tolist() for s in w.symbols]
                 for _ in range(args.steps + 2)]
        it = iter(fresh)

        def cold_step():
            g = k2.ctc_graph(next(it), modified=w.modified, device=dev)
            return loss_step(dev_lp, g, seg, w.output_beam)
        cold_step()
        cold_step()
        cold_ms, _, _, _ = timed(args.steps, cold_step)

    # ---- the LF-MMI denominator, ONE batch of 128 split by utterance over the ranks
    # (strong split): each rank takes every world-th utterance of the duration-sorted
    # batch, the shared graph is replicated, the only exchange is the 16-byte all-reduce
    den = None
    if args.workload == "ctc_large" and args.scale == 1.0 and not args.no_lfmmi_den:
        wd = syn.lfmmi_den(seed=0)
        d_seg, d_idx = shard_segments(wd.supervision_segments, world, rank)
        # this rank's utterances, renumbered 0..n-1 in its own log-prob tensor
        d_lp = wd.log_probs[torch.from_numpy(wd.supervision_segments[:, 0].numpy()[d_idx]
                                             .astype(np.int64))].contiguous().to(dev)
        d_seg = d_seg.clone()
        d_seg[:, 0] = torch.arange(d_seg.shape[0], dtype=torch.int32)
        sub = syn.Workload("lfmmi_den", wd.log_probs[:d_seg.shape[0]], d_seg, wd.output_beam,
                           graph_row_splits2=wd.graph_row_splits2, graph_arcs=wd.graph_arcs)
        d_graphs = syn.build_graphs(sub, dev)
        d_frames_all = wd.num_frames
        d_arc_frames = int(len(wd.graph_arcs)) * d_frames_all

        def den_step():
            return loss_step(d_lp, d_graphs, d_seg, wd.output_beam)
        for _ in range(warm):
            den_step()
        d_ms, _, _, _ = timed(args.steps, den_step)
        _, _, _, d_phases = timed(args.steps, den_step, profile=True)
        d_kernels = _lib.profile_kernels()
        Nd, Td, Cd = wd.log_probs.shape
        d_alg = algorithmic_bytes(d_frames_all, Nd, Td, Cd, Nd * len(wd.graph_arcs), 0, 0, False)
        den = {"workload": "lfmmi_den", "utterances": int(Nd), "utterances_per_gpu": int(d_seg.shape[0]),
               "split": "strong: one batch of 128 split by utterance over the ranks",
               "ms_per_step": d_ms / args.steps,
               "frames_per_sec": d_frames_all * args.steps / (d_ms * 1e-3),
               "arc_frames_per_sec": d_arc_frames * args.steps / (d_ms * 1e-3),
               "algorithmic_bytes_per_step": d_alg,
               "phases_ms_per_step": {k: v[0] / args.steps for k, v in d_phases.items() if v[0] > 0},
               "kernels": {k: d_kernels[k] for k, v in d_phases.items() if v[0] > 0}}

    clocks = sampler.stop() if rank == 0 else None

    # lattice size for the byte figures (what the lattice path would write)
    with torch.no_grad():
        dense = k2.DenseFsaVec(dev_lp, seg)
        lat = k2.intersect_dense(graphs, dense, w.output_beam)
    N, T, C = w.log_probs.shape
    A = graphs.num_arcs
    A_out, S_out = lat.num_arcs, lat.arcs.num_states
    arc_frames = int(sum(int(graphs.arcs.h_arc_splits[i + 1] - graphs.arcs.h_arc_splits[i]) *
                         int(seg[i, 2]) for i in range(seg.shape[0])))
    grid_states = sum(int(graphs.arcs.h_row_splits1[i + 1] - graphs.arcs.h_row_splits1[i]) *
                      (int(seg[i, 2]) + 2) for i in range(seg.shape[0]))
    lattice_written = phases["emit"][0] > 0
    b_alg = algorithmic_bytes(frames, N, T, C, A, A_out, S_out, lattice_written)
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_src = "measured" if "hbm_gbs" in peaks else "fallback"
    # the dominant phase of the timed region carries the roofline figure: the path's
    # algorithmic bytes per launch (one launch of it per step) over its duration
    top = max(phases, key=lambda k: phases[k][0])
    top_ms, top_n = phases[top]
    top_avg_ms = top_ms / args.steps
    achieved = b_alg / (top_avg_ms * 1e-3) / 1e9 if top_avg_ms > 0 else 0.0
    impl_b = implementation_bytes(top, kernels[top], frames, N, T, C, A, A_out, S_out, grid_states)
    # dram read + write of one launch from the ncu capture of this workload (profiles/)
    traffic = None
    if w.name == "ctc_large" and args.scale == 1.0:
        traffic = NCU_TRAFFIC.get(kernels[top])
    if den is not None:
        den["path_gbs"] = den["algorithmic_bytes_per_step"] * args.steps / (d_ms * 1e-3) / 1e9
        den["path_frac_of_hbm"] = den["path_gbs"] / (hbm_peak * world)

    # a bounded wait of the loss exchange that gave up would have made the totals invalid
    reduce_status = reducer.status() if isinstance(reducer, PeerLossReducer) else 0
    if reduce_status != 0:
        print(f"bench: rank {rank}: an exchange of (loss, frames) between the ranks timed out",
              file=sys.stderr)
    if dist is not None:
        dist.barrier()
        if reducer is not None:
            reducer.close()
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    sec = ms * 1e-3
    value = world * frames * args.steps / sec
    line = {
        "metric": "ctc_loss_fwd_bwd_frames_per_sec", "value": value, "unit": "frames/s",
        "n_gpus": world, "steps": args.steps, "warmup": warm,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32+f64", "data": "synthetic",
        "config": workload_config(w, args),
        "arc_frames_per_sec": world * arc_frames * args.steps / sec,
        # whole path: algorithmic bytes of a step over the step
        "path_gbs": b_alg * args.steps / sec / 1e9,
        "path_frac_of_hbm": b_alg * args.steps / sec / 1e9 / hbm_peak,
        "algorithmic_bytes_per_step": b_alg,
        "lattice_written": lattice_written,
        "wall_ms_per_step": 1e3 * wall / args.steps,
        "cold_graphs_ms_per_step": None if cold_ms is None else cold_ms / args.steps,
        "phases_ms_per_step": {k: v[0] / args.steps for k, v in phases.items()},
        "phase_kernels": {k: kernels[k] for k, v in phases.items() if v[0] > 0},
        "kernel_ms_per_step_by_rank": busy_by_rank,
        "ms_per_step_by_rank": ms_by_rank,
        "numa": numa,
        "lattice": {"arcs": A_out, "states": S_out, "graph_arcs": A, "arc_frames": arc_frames,
                    "grid_states": grid_states},
        "roofline": {"kernel": kernels[top], "bound": "hbm", "achieved": achieved,
                     "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                     "peak_source": peak_src, "algorithmic_bytes_per_launch": b_alg,
                     "avg_launch_ms": top_avg_ms, "traffic": traffic,
                     # what the kernel moves by its design over its time: DRAM utilisation,
                     # not a roofline fraction
                     "dram_utilisation": None if not impl_b or top_avg_ms <= 0 else
                     impl_b / (top_avg_ms * 1e-3) / 1e9 / hbm_peak,
                     "implementation_bytes_per_launch": impl_b,
                     "note": "latency-bound: a chain of T dependent frames per utterance; "
                             "achieved = the path's algorithmic bytes per step over the "
                             "dominant kernel's launch; traffic = ncu dram read+write of one "
                             "launch on this workload (profiles/)"},
        # value: the copy of step k+1 overlaps step k (k2_b200.parallel.HostPrefetcher), as
        # a training loop feeds the GPU; serial_value: copy, compute and read-back of one
        # step strictly after one another.  The loss (8 bytes) is read back every step;
        # the gradient stays on the device, where the optimiser uses it.
        "e2e": {"value": world * frames * args.steps / (e2e_ms * 1e-3), "unit": "frames/s",
                "h2d_bytes_per_step": int(w.log_probs.numel() * 4), "d2h_bytes_per_step": 8,
                "ms_per_step": e2e_ms / args.steps,
                "serial_value": world * frames * args.steps / (serial_ms * 1e-3),
                "serial_ms_per_step": serial_ms / args.steps},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    if dist is not None:
        line["loss_exchange"] = {"kind": type(reducer).__name__ if reducer is not None else "none",
                                 "status": int(reduce_status)}
    if den is not None:
        line["lfmmi_den"] = den
    if world == 1 and not args.no_cpu_baseline:
        impl_mod, kind = pick_cpu_impl()
        graphs_h, scores_h, rs_h = host_inputs(w, impl_mod)
        cpu_reference_step(w, graphs_h, scores_h, rs_h, impl_mod)
        single = min(cpu_reference_step(w, graphs_h, scores_h, rs_h, impl_mod)[0]
                     for _ in range(2))
        cores = max(1, min(os.cpu_count() or 1, seg.shape[0]))
        best, used = cpu_reference_sharded(w, graphs_h, scores_h, rs_h, impl_mod, cores, 3)
        line["cpu_baseline"] = {
            "value": frames / best, "unit": "frames/s", "cores": used, "kind": kind,
            "single_thread_value": frames / single, "host_cores": os.cpu_count(),
            "sample": f"best of 3 full batches of {w.name} ({frames} frames): intersect + log "
                      f"scores + posteriors + gradient scatter, sharded by utterance over {used} "
                      "worker processes; single_thread_value is the unsharded run (the "
                      "reference's path is single-threaded by construction)"}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


# ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch on ctc_large (profiles/)
NCU_TRAFFIC = {"BandViterbi": 289.5e6, "BandKeep+BandPrep": 296.5e6, "BandChainLists": 101.4e6,
               "BandGrad": 77.8e6}


# --------------------------------------------------------------------------- decoding
DECODE_PARAMS = dict(search_beam=20.0, output_beam=8.0, min_active_states=30,
                     max_active_states=10000)


def run_decode(args):
    """The decoding configuration (a 200 000-state graph shared by 32 sequences of 500
    frames): one step = intersect_dense_pruned + Viterbi best path + log-semiring total
    scores.  An extra line beside the headline benchmark; single GPU.  With --impl
    reference the reference's own CPU IntersectDensePruned runs on the first sequences
    of the same batch (it is single-threaded)."""
    import numpy as np

    w = load_synthetic().hlg_decode(seed=0, scale=args.scale)
    S = len(w.graph_row_splits2) - 1
    n, t = int(w.log_probs.shape[0]), int(w.log_probs.shape[1])
    config = {"workload": "hlg_decode (pruned)", "sequences": n, "frames_per_sequence": t,
              "classes": int(w.log_probs.shape[2]), "graph_states": S,
              "graph_arcs": int(len(w.graph_arcs)), **DECODE_PARAMS}
    if args.impl == "reference":
        from oracle import oracle, ref
        from oracle.common import HostFsaVec
        # the reference's own code when it has been compiled, else its C restatement
        impl, kind = (ref, "reference") if ref.available() else (oracle, "port")
        m = min(n, 2)
        scores, row_splits = host_scores(w)
        rows = int(row_splits[m])
        a = HostFsaVec(np.array([0, S], np.int32), w.graph_row_splits2.astype(np.int32),
                       w.graph_arcs)
        t0 = time.perf_counter()
        lat = impl.intersect_dense_pruned(a, scores[:rows], row_splits[:m + 1],
                                          *DECODE_PARAMS.values())
        dt = time.perf_counter() - t0
        print(json.dumps({"metric": "decode_frames_per_sec", "impl": "reference",
                          "value": m * t / dt, "unit": "frames/s", "n_gpus": 0,
                          "ms_per_step": dt * 1e3 * n / m, "higher_is_better": True,
                          "config": config,
                          "cpu_baseline": {"value": m * t / dt, "unit": "frames/s", "cores": 1,
                                           "kind": kind,
                                           "sample": f"{m} of {n} sequences, lattice only "
                                                     f"({lat.num_arcs} arcs)"}}))
        return
    import torch

    import k2_b200 as k2
    from k2_b200 import _lib
    from k2_b200.fsa_algo import _fsa_vec_from_numpy
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback)"
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    graph = _fsa_vec_from_numpy(np.array([0, S]), w.graph_row_splits2, w.graph_arcs, dev)
    dense = k2.DenseFsaVec(w.log_probs.to(dev), w.supervision_segments)

    if args.chunk > 0:
        # streaming: one OnlineDenseIntersecter.decode per chunk, every call returning the
        # lattice of everything decoded so far; a "step" is the whole batch, all chunks
        lp = w.log_probs.to(dev)
        seg = torch.tensor([[i, 0, args.chunk] for i in range(n)], dtype=torch.int32)
        decoder = k2.OnlineDenseIntersecter(graph, n, *DECODE_PARAMS.values())
        config["chunk_frames"] = args.chunk
        chunk_ms = []

        def step():
            states = [None] * n
            lat = None
            for k in range(t // args.chunk):
                x = lp[:, k * args.chunk:(k + 1) * args.chunk].contiguous()
                c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                c0.record()
                lat, states = decoder.decode(k2.DenseFsaVec(x, seg), states)
                c1.record()
                chunk_ms.append((c0, c1))
            best = k2.shortest_path(lat, use_double_scores=True)
            tot = lat.get_tot_scores(use_double_scores=True, log_semiring=True)
            return lat, best, tot
    else:
        def step():
            lat = k2.intersect_dense_pruned(graph, dense, **DECODE_PARAMS)
            best = k2.shortest_path(lat, use_double_scores=True)
            tot = lat.get_tot_scores(use_double_scores=True, log_semiring=True)
            return lat, best, tot

    for _ in range(max(args.warmup, 3)):
        lat, best, tot = step()
    torch.cuda.synchronize()
    if args.chunk > 0:
        chunk_ms.clear()
    clocks = ClockSampler(0)
    clocks.start()
    n0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        lat, best, tot = step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    launches = (_lib.launch_count() - n0) // args.steps
    extra = {}
    if args.chunk > 0:
        per = sorted(a.elapsed_time(b) for a, b in chunk_ms)
        extra = {"ms_per_chunk_median": per[len(per) // 2], "ms_per_chunk_max": per[-1]}
    print(json.dumps({
        **extra,
        "metric": "decode_frames_per_sec", "value": n * t / (ms * 1e-3), "unit": "frames/s",
        "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "dtype": "f32", "data": "synthetic", "config": config,
        "lattice": {"states": lat.arcs.num_states, "arcs": lat.arcs.num_elements()},
        "best_path_arcs": best.arcs.num_elements(), "tot_scores_mean": float(tot.mean().item()),
        "gpu_launches": int(launches), "clocks": clocks.stop()}))


def main():
    args = parse_args()
    if args.decode:
        run_decode(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

/* k2b200.h - C-ABI of libk2b200.so, the B200 (sm_100a) backend for k2's
 * dense-intersection / total-score path.
 *
 * Every entry point takes plain pointers and sizes.  Pointers are DEVICE
 * pointers unless the name starts with h_ (HOST).  All device memory - inputs,
 * outputs and workspaces - is owned by the caller; the library never allocates
 * device memory.  `stream` is a cudaStream_t passed as void*.  Functions
 * return 0 on success or a non-zero k2b200_status; k2b200_last_error() then
 * describes the failure (the reference raises a C++ exception, which its Python
 * layer surfaces as RuntimeError - the Python host layer of this library does
 * the same with the status).
 *
 * Data layouts are k2's:
 *   Arc      16 bytes {int32 src_state, int32 dest_state, int32 label, float
 *            score}; states are relative to the first state of their FSA
 *            (k2/csrc/fsa.h:31-63).
 *   FsaVec   row_splits1[num_fsas+1] (fsa -> state), row_ids1[num_states],
 *            row_splits2[num_states+1] (state -> arc), row_ids2[num_arcs],
 *            arcs[num_arcs] (k2/csrc/ragged.h:330, fsa.h:113-120).
 *   DenseFsaVec  scores[rows, cols] contiguous float32 with cols = C+1 and
 *            column = label+1, plus row_splits[num_seqs+1]; each sequence has
 *            its T frames followed by one final row [0,-inf,...]
 *            (k2/csrc/fsa.h:138-185, k2/python/k2/dense_fsa_vec.py:43-145).
 */
#ifndef K2B200_H_
#define K2B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  K2B200_OK = 0,
  K2B200_INVALID_ARGUMENT = 1,
  K2B200_CUDA_ERROR = 2,
  K2B200_WORKSPACE_TOO_SMALL = 3,
  K2B200_TOO_LARGE = 4
} k2b200_status;

/* Text of the last error on the calling thread. */
const char *k2b200_last_error(void);
/* ABI version of the library (bumped on any signature change or new entry point;
 * 3: pruned intersection, score derivatives, k2b200_upload_i32;
 * 4: k2b200_band_*;
 * 5: k2b200_peer_reduce_*, k2b200_loss_sum_all_reduce, zero_fill in k2b200_band_loss_args). */
int32_t k2b200_abi_version(void);

/* Benchmark bookkeeping (no counterpart in the reference's bindings; its
 * benchmark harness, k2/csrc/benchmark/benchmark.h:49-66, times from outside).
 * k2b200_kernel_launch_count: kernels launched by this library so far.
 * k2b200_profile_enable(1) makes the entry points bracket their phases with
 * cudaEvents on the launching stream; k2b200_profile_read_ms(phase, &n) waits
 * for them, returns the summed milliseconds of the n recorded intervals and
 * resets the phase.  Phases: 0 Viterbi recursion, 1 pruning (count + numbering),
 * 2 lattice emission, 3 forward/backward scores, 4 posteriors + gradient
 * scatter, 5 incoming-arc index, 6 DenseFsaVec construction and its backward,
 * 7 lattice-free alpha/beta recursion, 8 lattice-free gradients. */
int64_t k2b200_kernel_launch_count(void);
/* name of the kernel(s) that last ran under a phase ("" if none yet) */
const char *k2b200_profile_kernel(int32_t phase);
void k2b200_profile_enable(int32_t on);
double k2b200_profile_read_ms(int32_t phase, int64_t *intervals);

/* ---------------------------------------------------------------------------
 * Ragged helpers.
 * ------------------------------------------------------------------------- */

/* row_ids[k] = row r with row_splits[r] <= k < row_splits[r+1].
 * Replaces k2::RowSplitsToRowIds, k2/csrc/utils.cu:75-130. */
int32_t k2b200_row_splits_to_row_ids(const int32_t *row_splits, int32_t num_rows,
                                     int32_t *row_ids, int32_t num_elems,
                                     void *stream);

/* n int32 values from (pageable or pinned) host memory to device memory, passed as
 * kernel parameters in launches of up to 960 values: asynchronous on `stream`, the
 * host array is free for reuse on return, and the copy engine is not involved.  For
 * the few hundred integers of a batch description (segments, row_splits, symbol
 * lists), where k2 copies through Array1::To (k2/csrc/array.h:234-250). */
int32_t k2b200_upload_i32(const int32_t *host_values, int64_t n, int32_t *device_out,
                          void *stream);

/* Exclusive sum of n int32: out[0..n], out[n] = total; in and out may alias.
 * tmp must hold k2b200_exclusive_sum_tmp_bytes(n) bytes.
 * Replaces k2::ExclusiveSum, k2/csrc/utils_inl.h:40-60 (cub::DeviceScan). */
size_t k2b200_exclusive_sum_tmp_bytes(int64_t n);
int32_t k2b200_exclusive_sum(const int32_t *in, int32_t *out, int64_t n, void *tmp,
                             void *stream);

/* The same exclusive sum for callers that cannot provide scratch memory.  It has
 * no counterpart in the reference, whose ExclusiveSum always allocates its
 * temporary storage from the tensor library's allocator.  It is meant for hosts
 * that drive this library without such an allocator (a plain C/C++ service) or
 * whose device memory is partitioned once at start-up, where allocating in the
 * request path is not possible or would stall the device.
 *
 * The scratch (the per-tile sums) is a 64 KB array that lives inside the library
 * on every GPU that loads it, for the lifetime of the process, so:
 *   - n may be at most k2b200_exclusive_sum_static_max_len() (33 554 431);
 *     a longer input is refused with K2B200_TOO_LARGE and an explanatory message,
 *     and k2b200_exclusive_sum is the call to use instead;
 *   - the first call on each device looks up the array's device address (with
 *     that device current); make that first call during set-up, before any
 *     stream capture is begun;
 *   - all calls on a device share the array: two calls that may run at the same
 *     time on that device (different streams or threads) race and must be
 *     ordered by the caller.  Nothing has to be cleared between calls - each
 *     call overwrites every entry it later reads.
 * No device memory is allocated or freed; in, out and the result layout are
 * those of k2b200_exclusive_sum (out[0..n], out[n] = total, in == out allowed). */
int64_t k2b200_exclusive_sum_static_max_len(void);
int32_t k2b200_exclusive_sum_static(const int32_t *in, int32_t *out, int64_t n,
                                    void *stream);

/* Incoming-arc index of an FsaVec: in_splits[num_states+1], in_arcs[num_arcs];
 * the arcs entering each state, in increasing arc index.  in_src and in_score
 * (each [num_arcs], either may be NULL) receive the source state (idx01) and the
 * score of those arcs in the same order; k2b200_fsa_scores reads them.
 * Replaces k2::GetDestStates + k2::GetIncomingArcs,
 * k2/csrc/fsa_utils.cu:650-677, :901-928 (called from
 * k2/csrc/intersect_dense.cu:139-142 and k2/python/k2/fsa.py:529-562). */
size_t k2b200_fsa_incoming_tmp_bytes(int32_t num_states, int32_t num_arcs);
int32_t k2b200_fsa_incoming(const int32_t *row_splits1, const int32_t *row_ids1,
                            const int32_t *row_ids2, const void *arcs,
                            int32_t num_fsas, int32_t num_states, int32_t num_arcs,
                            int32_t *in_splits, int32_t *in_arcs, int32_t *in_src,
                            float *in_score, void *tmp, void *stream);

/* ---------------------------------------------------------------------------
 * CTC graphs.
 * Builds the CTC graphs of num_seqs transcripts (sym_row_splits[num_seqs+1] into
 * symbols[num_symbols], both on the device; symbols != -1) with all scores 0:
 * row_splits1[num_seqs+1], row_splits2[num_states+1] with num_states =
 * 2*num_symbols + 2*num_seqs, arcs and aux_labels[num_arcs].  num_arcs =
 * 4*num_symbols + 2*num_seqs + (number of symbol positions with a third arc:
 * every position when modified != 0, otherwise those whose next symbol differs
 * or that are last) - the caller counts it to size the outputs.
 * Replaces k2::CtcGraphs, k2/csrc/fsa_algo.cu:577-730 (bound as _k2.ctc_graph).
 * ------------------------------------------------------------------------- */
size_t k2b200_ctc_graph_tmp_bytes(int32_t num_symbols);
int32_t k2b200_ctc_graph(const int32_t *sym_row_splits, const int32_t *symbols,
                         int32_t num_seqs, int32_t num_symbols, int32_t modified,
                         int32_t *row_splits1, int32_t *row_splits2, void *arcs,
                         int32_t *aux_labels, void *tmp, void *stream);

/* ---------------------------------------------------------------------------
 * DenseFsaVec.
 * k2b200_dense_fsa_vec_fill writes the whole score matrix of a DenseFsaVec
 * (scores[rows, C+1], rows = sum_i (dur_i + 1)) from log_probs[N, T, C]: column
 * 0 is -inf, columns 1..C hold the frames of each supervision segment, and the
 * extra last row of each segment is [0, -inf, ...].  segments is the DEVICE copy
 * of the [num_segs, 3] int32 (sequence, start_frame, duration) rows, durations
 * already truncated to the frames that exist; row_splits[num_segs+1] (device)
 * gives the first score row of each segment.  Replaces the gather and fills of
 * k2.DenseFsaVec.__init__, k2/python/k2/dense_fsa_vec.py:101-133.
 * k2b200_dense_fsa_vec_backward is its adjoint: grad_log_probs[N, T, C] is
 * zero-filled and receives grad_scores[:, 1:] of the frame rows; pass
 * overlapping != 0 when two segments may cover the same frame (atomic adds).
 * ------------------------------------------------------------------------- */
int32_t k2b200_dense_fsa_vec_fill(const float *log_probs, int64_t num_seqs,
                                  int64_t num_frames, int32_t num_classes,
                                  const int32_t *segments, const int32_t *row_splits,
                                  int32_t num_segs, float *scores, int32_t rows,
                                  void *stream);
int32_t k2b200_dense_fsa_vec_backward(const float *grad_scores, int64_t num_seqs,
                                      int64_t num_frames, int32_t num_classes,
                                      const int32_t *segments, const int32_t *row_splits,
                                      int32_t num_segs, int32_t rows, int32_t overlapping,
                                      float *grad_log_probs, void *stream);

/* The same with log_softmax(logits, dim=-1) fused in: scores =
 * layout(log_softmax(logits)), and the adjoint w.r.t. the logits (needs the scores
 * the forward call wrote).  Replaces torch.log_softmax followed by the
 * DenseFsaVec constructor, k2/python/k2/dense_fsa_vec.py:101-133, in one pass each
 * way. */
int32_t k2b200_dense_fsa_vec_from_logits(const float *logits, int64_t num_seqs,
                                         int64_t num_frames, int32_t num_classes,
                                         const int32_t *segments, const int32_t *row_splits,
                                         int32_t num_segs, float *scores, int32_t rows,
                                         void *stream);
int32_t k2b200_dense_fsa_vec_from_logits_backward(const float *grad_scores, const float *scores,
                                                  int64_t num_seqs, int64_t num_frames,
                                                  int32_t num_classes, const int32_t *segments,
                                                  const int32_t *row_splits, int32_t num_segs,
                                                  int32_t rows, int32_t overlapping,
                                                  float *grad_logits, void *stream);

/* ---------------------------------------------------------------------------
 * intersect_dense.
 * Replaces k2::IntersectDense / MultiGraphDenseIntersect,
 * k2/csrc/intersect_dense.cu:100-1073, as bound by _k2.intersect_dense,
 * k2/python/csrc/torch/fsa_algo.cu:224-253.
 *
 * Protocol (one host synchronisation, to size the outputs):
 *   1. k2b200_intersect_dense_workspace_bytes(&args, &bytes)
 *   2. k2b200_intersect_dense_prune(&args, ws, bytes, stream, &ns, &na, &beam)
 *      runs the Viterbi forward/backward recursion over all frames, applies the
 *      output beam (shrinking it like the reference when max_states / max_arcs
 *      would be exceeded), numbers the surviving states and arcs and returns
 *      their counts, plus (optional, may be NULL) the largest number of states in
 *      one (fsa, frame) layer and of arcs between two layers - the bounds a
 *      k2b200_fsa_view of the lattice wants;
 *   3. k2b200_intersect_dense_emit(&args, ws, bytes, stream, &out) with output
 *      buffers of those sizes writes the lattice and both arc maps.
 * ------------------------------------------------------------------------- */
typedef struct {
  /* a_fsas: the graphs, one per entry of a_to_b_map */
  int32_t num_fsas, num_states, num_arcs;
  const int32_t *a_row_splits1;   /* [num_fsas+1] */
  const int32_t *a_row_splits2;   /* [num_states+1] */
  const void *a_arcs;             /* [num_arcs] Arc */
  const int32_t *a_in_splits;     /* [num_states+1] from k2b200_fsa_incoming */
  const int32_t *a_in_arcs;       /* [num_arcs] */
  const int32_t *h_a_row_splits1; /* HOST copy of a_row_splits1 */
  const int32_t *h_a_arc_splits;  /* HOST [num_fsas+1]: a_row_splits2[a_row_splits1[i]] */
  /* b_fsas: the DenseFsaVec */
  const float *scores;            /* [rows, cols] contiguous */
  int32_t rows, cols, num_seqs;
  const int32_t *h_b_row_splits;  /* HOST [num_seqs+1] */
  /* HOST [num_fsas], non-decreasing, or NULL for the identity map */
  const int32_t *h_a_to_b_map;
  float output_beam;
  int32_t max_states, max_arcs;
  /* 0 = choose automatically, 1 = one launch per frame (any graph size),
   * 2 = persistent frame-synchronous kernel (graphs that fit in shared memory),
   * 3 = persistent kernel with the arcs in registers (needs a_max_degree <= 4
   *     and at most 1024 states per graph), 4 = persistent kernel with a lane plan
   *     (graphs of at most 768 states with states of more than four arcs),
   * 5 = one launch per frame with the sequences on the lanes of a warp (needs a_shared
   *     and at least two sequences; what 0 chooses for a shared graph too large for 2-4) */
  int32_t viterbi_mode;
  /* largest number of arcs entering or leaving any state of a_fsas; 0 = unknown
   * (then mode 3 is never chosen) */
  int32_t a_max_degree;
  /* non-zero: every graph of a_fsas is a copy of graph 0 (same states, arcs and
   * scores), as k2 users build them for decoding (one HLG per sequence) because
   * k2::IntersectDense cannot share a graph (k2/csrc/intersect_dense.cu:75-93).
   * Only graph 0 is then read, so that it stays cache-resident; results are the
   * same as with 0.  The caller vouches for the equality. */
  int32_t a_shared;
} k2b200_intersect_args;

typedef struct {
  int32_t *row_splits1; /* [num_fsas+1] */
  int32_t *row_ids1;    /* [num_states_out] */
  int32_t *row_splits2; /* [num_states_out+1] */
  int32_t *row_ids2;    /* [num_arcs_out] */
  void *arcs;           /* [num_arcs_out] Arc */
  int32_t *arc_map_a;   /* [num_arcs_out] arc idx012 in a_fsas, may be NULL */
  int32_t *arc_map_b;   /* [num_arcs_out] offset into scores, may be NULL */
  /* Optional (may be NULL): the time layering of the lattice, used by
   * k2b200_fsa_scores.  level_offsets[num_fsas+1] gives, per FSA, its range in
   * level_splits; level_splits[total_levels+1] gives the first state (idx01)
   * of every (fsa, frame) layer, total_levels = sum_i (T_i + 2). */
  int32_t *level_offsets;
  int32_t *level_splits;
} k2b200_lattice_out;

int32_t k2b200_intersect_dense_workspace_bytes(const k2b200_intersect_args *args,
                                               size_t *bytes,
                                               int64_t *total_levels);
int32_t k2b200_intersect_dense_prune(const k2b200_intersect_args *args, void *workspace,
                                     size_t workspace_bytes, void *stream,
                                     int32_t *num_states_out, int32_t *num_arcs_out,
                                     float *beam_used, int32_t *max_layer_states,
                                     int32_t *max_layer_arcs);
int32_t k2b200_intersect_dense_emit(const k2b200_intersect_args *args, void *workspace,
                                    size_t workspace_bytes, void *stream,
                                    const k2b200_lattice_out *out);

/* ---------------------------------------------------------------------------
 * Pruned intersection (decoding): a beam search over the frames with a dynamic
 * beam per sequence between min_active_states and max_active_states, and
 * backward pruning to output_beam in windows of 30 frames every 20.
 * Replaces k2::IntersectDensePruned (k2/csrc/intersect_dense_pruned.cu:1678-1694;
 * declaration k2/csrc/fsa_algo.h:150-206), bound as _k2.intersect_dense_pruned
 * (k2/python/csrc/torch/fsa_algo.cu:200-222).  a_fsas holds one graph per
 * sequence or a single graph shared by all sequences (num_fsas == 1).  States of
 * a frame are numbered as the reference's CPU build numbers them (by the first
 * arc that reaches them above the cutoff), so lattices and arc maps are
 * identical to it.  Chunk-by-chunk decoding: k2b200_online_decode_* below.
 *
 * Protocol (one host synchronisation):
 *   1. k2b200_intersect_dense_pruned_workspace_bytes(&args, &bytes, &levels)
 *   2. k2b200_intersect_dense_pruned_search(&args, ws, bytes, stream, &ns, &na,
 *      &arena_full): one CTA per sequence walks all frames.  arena_full = 1 means
 *      max_states_per_seq / max_arcs_per_seq were too small for some sequence:
 *      call again with larger values (and a workspace sized for them).
 *   3. k2b200_intersect_dense_pruned_emit(&args, ws, bytes, stream, &out) writes
 *      the lattice (ns states, na arcs), both arc maps (arc_map_a is -1 on the
 *      arcs that allow_partial turned into final arcs) and, optionally, the
 *      layering: levels = num_seqs * (T + 2) with T the longest sequence's rows.
 * ------------------------------------------------------------------------- */
typedef struct {
  int32_t num_fsas, num_states, num_arcs; /* a_fsas; num_fsas is 1 or num_seqs */
  const int32_t *a_row_splits1;           /* [num_fsas+1] */
  const int32_t *a_row_splits2;           /* [num_states+1] */
  const void *a_arcs;                     /* [num_arcs] Arc, arc-sorted */
  const float *scores;                    /* [rows, cols] contiguous */
  int32_t rows, cols, num_seqs;
  const int32_t *b_row_splits;            /* device [num_seqs+1] */
  const int32_t *h_b_row_splits;          /* HOST copy */
  float search_beam, output_beam;
  int32_t min_active_states, max_active_states, allow_partial;
  /* capacity, per sequence, for the states and arcs alive at any one time: the
   * pruned frames so far plus the unpruned last 30 */
  int64_t max_states_per_seq, max_arcs_per_seq;
  /* CTAs (a thread-block cluster) that share one sequence: 0 = as many as keep
   * the GPU filled, else 1, 2, 4 or 8.  The result does not depend on it. */
  int32_t team_ctas;
} k2b200_pruned_args;

int32_t k2b200_intersect_dense_pruned_workspace_bytes(const k2b200_pruned_args *args,
                                                      size_t *bytes, int64_t *total_levels);
int32_t k2b200_intersect_dense_pruned_search(const k2b200_pruned_args *args, void *workspace,
                                             size_t workspace_bytes, void *stream,
                                             int32_t *num_states_out, int32_t *num_arcs_out,
                                             int32_t *arena_full);
int32_t k2b200_intersect_dense_pruned_emit(const k2b200_pruned_args *args, void *workspace,
                                           size_t workspace_bytes, void *stream,
                                           const k2b200_lattice_out *out);

/* ---------------------------------------------------------------------------
 * Chunk-by-chunk decoding: the pruned intersection over a stream of chunks, each call
 * returning the lattice of everything decoded so far.
 * Replaces k2::OnlineDenseIntersecter::Decode (k2/csrc/intersect_dense_pruned.cu:
 * 1739-1853; class k2/csrc/intersect_dense_pruned.h:168-204), bound as
 * _k2.OnlineDenseIntersecter.decode (k2/python/csrc/torch/fsa_algo.cu:755-800).
 * One graph is shared by all streams.  What a stream has decoded so far lives in
 * caller-owned arrays (k2b200_online_stream, the counterpart of k2::DecodeStateInfo);
 * a call loads them into the workspace, searches the chunk, prunes the last two
 * frames of the history together with the chunk, closes the lattice with the final
 * arcs that the chunk's extra row [0, -inf, ...] allows, and stores the streams back:
 *   1. k2b200_online_decode_workspace_bytes(&args, &bytes)
 *   2. k2b200_online_decode_load(&args, ws, i, &stream_i, cuda_stream) for every i
 *   3. k2b200_online_decode_run(...): lattice sizes, per-stream (states, arcs)
 *      counts for the new stream arrays, updated beams; arena_full = 1 asks for a
 *      retry with larger max_*_per_seq (reload the streams)
 *   4. k2b200_online_decode_emit(&args, ws, bytes, cuda_stream, &out)  (no arc_map_b;
 *      the optional layering has sum_i (history_i + chunk + 2) layers)
 *   5. k2b200_online_decode_store(&args, ws, i, &new_stream_i, cuda_stream)
 * A new stream is: one state (the graph's start state, forward score 0), no arcs,
 * history 0, frame tables {0, 1} and {0, 0}, beam = search_beam.
 * ------------------------------------------------------------------------- */
typedef struct {
  int32_t num_states, num_arcs;
  int32_t *astate;        /* [num_states] graph state */
  int32_t *forward;       /* [num_states] forward score, order-preserving int form */
  int32_t *arc0;          /* [num_states+1] first arc of every state */
  int32_t *arc_graph;     /* [num_arcs] arc of the graph */
  float *arc_score;       /* [num_arcs] */
  int32_t *arc_dest;      /* [num_arcs] state of the next frame */
  int32_t *frame_state0;  /* [history+2] first state of every frame */
  int32_t *frame_arc0;    /* [history+2] first arc of every frame */
} k2b200_online_stream;

typedef struct {
  int32_t num_states, num_arcs;   /* the one shared graph */
  const int32_t *a_row_splits1;   /* [2] */
  const int32_t *a_row_splits2;   /* [num_states+1] */
  const void *a_arcs;
  const float *scores;            /* the chunk: [rows, cols] */
  int32_t rows, cols, num_seqs;
  const int32_t *b_row_splits;    /* device [num_seqs+1], equal lengths */
  const int32_t *h_b_row_splits;  /* HOST copy */
  float search_beam, output_beam;
  int32_t min_active_states, max_active_states, allow_partial;
  const int32_t *h_hist;          /* HOST [num_seqs]: frames decoded so far per stream */
  int64_t max_states_per_seq, max_arcs_per_seq;
  int32_t team_ctas;              /* as in k2b200_pruned_args */
} k2b200_online_args;

int32_t k2b200_online_decode_workspace_bytes(const k2b200_online_args *args, size_t *bytes);
int32_t k2b200_online_decode_load(const k2b200_online_args *args, void *workspace, int32_t seq,
                                  const k2b200_online_stream *st, void *stream);
int32_t k2b200_online_decode_run(const k2b200_online_args *args, void *workspace,
                                 size_t workspace_bytes, void *stream, const float *h_beams_in,
                                 float *h_beams_out, int32_t *h_counts, int32_t *num_states_out,
                                 int32_t *num_arcs_out, int32_t *arena_full);
int32_t k2b200_online_decode_emit(const k2b200_online_args *args, void *workspace,
                                  size_t workspace_bytes, void *stream,
                                  const k2b200_lattice_out *out);
int32_t k2b200_online_decode_store(const k2b200_online_args *args, void *workspace, int32_t seq,
                                   const k2b200_online_stream *st, void *stream);
/* The same for all streams of the batch in one launch; `streams` is a HOST array of
 * num_seqs descriptors (the store must come before the next load: the list of copies
 * lives in the workspace). */
int32_t k2b200_online_decode_load_all(const k2b200_online_args *args, void *workspace,
                                      const k2b200_online_stream *streams, void *stream);
int32_t k2b200_online_decode_store_all(const k2b200_online_args *args, void *workspace,
                                       const k2b200_online_stream *streams, void *stream);

/* ---------------------------------------------------------------------------
 * Lattice-free total scores: the log-semiring total score of
 * intersect_dense(a_fsas, b_fsas, output_beam) for every graph, and its
 * gradients, without materialising the lattice.
 * Replaces, for callers that only want the loss, the chain
 *   k2::IntersectDense (k2/csrc/intersect_dense.cu:100-1073) ->
 *   k2::GetForwardScores / GetTotScores (k2/csrc/fsa_utils.cu:1124-1278, :1456-1490) ->
 *   k2::GetArcPost (:1492-1560) -> index_add through both arc maps
 *   (k2/python/k2/autograd.py:30-117, :560-664),
 * as k2.ctc_loss drives it (k2/python/k2/ctc_loss.py:86-150).  The same states and
 * arcs survive pruning as in the lattice (same fp32 tests, same beam reduction
 * against max_states / max_arcs); sums run in float64.
 *
 *   k2b200_dense_loss_supported: *supported = 1 when every graph fits the
 *     shared-memory recursion; otherwise use the lattice entry points.
 *   k2b200_dense_loss_forward: tot_scores[num_fsas] (device, float64; -inf for a
 *     graph with no surviving path).  The workspace keeps what the backward needs.
 *   k2b200_dense_loss_backward: with tot_grad[i * tot_grad_stride] = dL/dtot[i]
 *     (device, float64), ADDS dL/d(arc score) to grad_a[num_arcs] and
 *     dL/d(scores) to grad_b[rows * cols]; both must be zero-filled (or hold
 *     gradients to accumulate onto) and the workspace must be the one the forward
 *     call filled, with the same args.  grad_a may be NULL when the gradient of the
 *     arc scores is not wanted; for graphs in which all arcs entering a state carry
 *     the same label the dense gradient then comes from state posteriors
 *     (alpha * beta / Z per surviving state) and no arc is visited.
 * ------------------------------------------------------------------------- */
int32_t k2b200_dense_loss_supported(const k2b200_intersect_args *args, int32_t *supported);
int32_t k2b200_dense_loss_workspace_bytes(const k2b200_intersect_args *args, size_t *bytes);
int32_t k2b200_dense_loss_forward(const k2b200_intersect_args *args, void *workspace,
                                  size_t workspace_bytes, void *stream, double *tot_scores,
                                  float *beam_used);
int32_t k2b200_dense_loss_backward(const k2b200_intersect_args *args, void *workspace,
                                   size_t workspace_bytes, const double *tot_grad,
                                   int32_t tot_grad_stride, float *grad_a, float *grad_b,
                                   void *stream);
/* The same, with dL/d(scores) written straight into the layout of the log-probs the
 * DenseFsaVec was made from (k2/python/k2/dense_fsa_vec.py:43-145), which saves the
 * pass that the adjoint of that layout would otherwise make over both matrices:
 * grad_log_probs is [.., num_classes] (zero-filled, num_classes = cols - 1) and
 * log_prob_row[i] (device, one per graph) is the row of it that holds frame 0 of
 * graph i's sequence, i.e. segment_index * frames_per_sequence + segment_start. */
int32_t k2b200_dense_loss_backward_log_probs(const k2b200_intersect_args *args, void *workspace,
                                             size_t workspace_bytes, const double *tot_grad,
                                             int32_t tot_grad_stride, float *grad_a,
                                             float *grad_log_probs, const int32_t *log_prob_row,
                                             int32_t num_classes, void *stream);

/* ---------------------------------------------------------------------------
 * Lattice-free total scores for BAND graphs: the same chain as above,
 *   k2::IntersectDense (k2/csrc/intersect_dense.cu:100-1073) ->
 *   k2::GetForwardScores / GetBackwardScores / GetTotScores
 *   (k2/csrc/fsa_utils.cu:1124-1454, :1809-1837) -> k2::GetArcPost (:1839-1901) ->
 *   index_add through both arc maps (k2/python/k2/autograd.py:30-117, :511-664),
 * specialised for graphs of the shape k2::CtcGraphs builds (k2/csrc/fsa_algo.cu:577-730):
 * every arc goes from a state s to s, s+1 or s+2, there is at most one arc per (source,
 * destination), and all arcs entering a state carry the same label.  The same states and
 * arcs survive pruning as in the lattice (same fp32 tests, same beam reduction against
 * max_states / max_arcs); sums run in float64 mantissa/exponent arithmetic, so any score
 * range is handled.  The dense scores are read from the log-prob matrix the DenseFsaVec was
 * made from (k2/python/k2/dense_fsa_vec.py:43-145), not from its [rows, C+1] score matrix:
 * log_probs is [log_prob_rows, num_classes] contiguous float32, 16-byte aligned, with
 * num_classes a multiple of 4, and graph i reads rows h_first_row[i] .. + h_frames[i] - 1;
 * the extra final row of a sequence is implied.
 *
 *   k2b200_band_tables: per-state tables of a_fsas (band_states: tables_bytes' first size,
 *     band_arcs: its second) and *status (device int32) bit 0 = some graph is not a band
 *     graph, in which case the tables must not be used.  They depend on the graphs only and
 *     can be kept for as long as the arcs do not change.
 *   k2b200_band_loss_supported: *supported = 0 when the sizes do not fit (more than 512
 *     states in a graph, unaligned rows, frames beyond shared memory);
 *     k2b200_last_error() says which.  Host-side only.
 *   k2b200_band_loss_forward: tot_scores[num_fsas] (device, float64; -inf for a graph
 *     with no surviving path; NaN if a copy into shared memory timed out, see
 *     k2b200_band_loss_status).  The workspace keeps what the backward needs.  The call
 *     waits on the host (for the numbers of surviving states and arcs, behind the kernels it
 *     has already launched) only when max_states is below the number of grid states that
 *     the start state can reach and that can reach the last state, or max_arcs below
 *     (frames + 1) x arcs summed over the graphs; otherwise no reduction of the beam is
 *     possible and the call is asynchronous.
 *   k2b200_band_loss_backward: with tot_grad[i * tot_grad_stride] = dL/dtot[i] (device,
 *     float64), ADDS dL/d(dense score) to grad_b[(grad_row0[i] + frame) * grad_pitch +
 *     label + grad_col_off] (grad_row0: device, one per graph; NULL = h_first_row as the
 *     forward call was given it).  grad_col_off = 0,
 *     grad_pitch = num_classes, grad_row0 = h_first_row gives the log-prob layout;
 *     grad_col_off = 1, grad_pitch = num_classes + 1 and grad_row0 = first row of the
 *     sequence the layout of the DenseFsaVec score matrix (including column 0 of the final
 *     rows).  grad_a (may be NULL: not wanted) receives dL/d(arc score), added.
 *   k2b200_band_loss_status: waits for `stream` and returns the status word of the last
 *     forward call on this workspace: bit 1 = a bounded wait for a row copy gave up (the
 *     results are invalid; nothing hangs or traps).
 *   k2b200_debug_set_copy_wait_limit: polls of an mbarrier before such a wait gives up
 *     (default 4 000 000; 0 makes every wait give up at once - for tests of that path;
 *     negative restores the default).
 * ------------------------------------------------------------------------- */
typedef struct {
  int32_t num_fsas, num_states;
  const int32_t *a_row_splits2;   /* [num_states+1] */
  const int32_t *h_a_row_splits1; /* HOST [num_fsas+1] */
  const int32_t *h_a_arc_splits;  /* HOST [num_fsas+1] */
  const void *band_states;        /* from k2b200_band_tables */
  const void *band_arcs;
  const float *log_probs;         /* [log_prob_rows, num_classes] */
  int64_t log_prob_rows;
  int32_t num_classes;
  const int32_t *h_first_row;     /* HOST [num_fsas] */
  const int32_t *h_frames;        /* HOST [num_fsas], non-increasing */
  float output_beam;
  int32_t max_states, max_arcs;
  /* Optional (forward only): zero_fill_bytes bytes at zero_fill (device) are cleared beside
   * the recursions, which leave most SMs idle - meant for the gradient buffer that the
   * backward call adds into, so that its zero-fill costs no time of its own.  The clear is
   * complete, in stream order, when the forward call's work on `stream` is.  NULL: none. */
  void *zero_fill;
  size_t zero_fill_bytes;
} k2b200_band_loss_args;

int32_t k2b200_band_tables_bytes(int32_t num_states, size_t *states_bytes, size_t *arcs_bytes);
int32_t k2b200_band_tables(const int32_t *row_splits1, int32_t num_fsas,
                           const int32_t *row_splits2, const void *arcs, int32_t num_states,
                           void *band_states, void *band_arcs, int32_t *status, void *stream);
int32_t k2b200_band_loss_supported(const k2b200_band_loss_args *args, int32_t *supported);
int32_t k2b200_band_loss_workspace_bytes(const k2b200_band_loss_args *args, size_t *bytes);
int32_t k2b200_band_loss_forward(const k2b200_band_loss_args *args, void *workspace,
                                 size_t workspace_bytes, void *stream, double *tot_scores,
                                 float *beam_used);
int32_t k2b200_band_loss_backward(const k2b200_band_loss_args *args, void *workspace,
                                  size_t workspace_bytes, const double *tot_grad,
                                  int32_t tot_grad_stride, float *grad_a, float *grad_b,
                                  const int32_t *grad_row0, int32_t grad_pitch,
                                  int32_t grad_col_off, void *stream);
int32_t k2b200_band_loss_status(const k2b200_band_loss_args *args, void *workspace,
                                size_t workspace_bytes, void *stream, int32_t *status);
void k2b200_debug_set_copy_wait_limit(int32_t polls);

/* ---------------------------------------------------------------------------
 * Forward / backward scores of a layered (top-sorted, acyclic) FsaVec.
 * Replaces k2::GetForwardScores / GetBackwardScores,
 * k2/csrc/fsa_utils.cu:1124-1278, :1345-1454 (bound at
 * k2/python/csrc/torch/fsa.cu:262-341), with the layering taken from
 * level_offsets/level_splits instead of GetStateBatches (:679-899).
 *
 * use_double selects float64 or float32 state scores (`forward` / `backward`
 * point to num_states elements of that type; either may be NULL to skip that
 * direction).  log_semiring != 0: log-sum-exp; == 0: max, and entering_arcs
 * (may be NULL) receives for every state the best entering arc (ties go to the
 * highest arc index; -1 when no arc enters), as
 * k2/csrc/ragged_ops_inl.h:627-657.
 *
 * When the view says the layering is strict (every arc goes from one layer to
 * the next - true for the lattices of k2b200_intersect_dense_emit) and gives
 * bounds on the layer sizes, a shared-memory staged kernel is used; otherwise a
 * general one.  Both give the same values.
 * ------------------------------------------------------------------------- */
typedef struct {
  int32_t num_fsas, num_states, num_arcs;
  const int32_t *row_splits1; /* [num_fsas+1] */
  const int32_t *row_ids1;    /* [num_states], may be NULL where not needed */
  const int32_t *row_splits2; /* [num_states+1] */
  const int32_t *row_ids2;    /* [num_arcs] */
  const void *arcs;           /* [num_arcs] Arc */
  /* incoming-arc index from k2b200_fsa_incoming (forward direction only) */
  const int32_t *in_splits, *in_arcs, *in_src;
  const float *in_score;
  /* layering: level_offsets[num_fsas+1] into level_splits[total_levels+1] */
  const int32_t *level_offsets, *level_splits;
  int32_t strict_layers;    /* 1: every arc goes from layer l to layer l+1 */
  int32_t max_layers;       /* upper bound on layers per FSA, 0 = unknown */
  int32_t max_layer_states; /* upper bound on states per layer, 0 = unknown */
  int32_t max_layer_arcs;   /* upper bound on arcs between two layers */
} k2b200_fsa_view;

/* scratch (k2b200_fsa_scores_scratch_bytes(fsas) bytes; may be NULL) enables the
 * fastest log-semiring kernel for strictly layered views: it keeps every score
 * as mantissa * 2^exponent so that no exp/log sits on the layer-to-layer
 * dependency chain (the arcs' exp() and the states' log() run in separate fully
 * parallel kernels).  Without scratch a slower kernel gives the same values. */
size_t k2b200_fsa_scores_scratch_bytes(const k2b200_fsa_view *fsas);
int32_t k2b200_fsa_scores(const k2b200_fsa_view *fsas, int32_t log_semiring,
                          int32_t use_double, void *forward, void *backward,
                          int32_t *entering_arcs, void *scratch, size_t scratch_bytes,
                          void *stream);

/* tot_scores[i] = forward score of the last state of FSA i, -inf if empty.
 * Replaces k2::GetTotScores, k2/csrc/fsa_utils.cu:1809-1837. */
int32_t k2b200_fsa_tot_scores(const int32_t *row_splits1, int32_t num_fsas,
                              int32_t use_double, const void *forward,
                              void *tot_scores, void *stream);

/* arc_post[a] = score + forward[src] + backward[dest] - 0.5*(forward[final] +
 * backward[start]).  Replaces k2::GetArcPost, k2/csrc/fsa_utils.cu:1839-1901. */
int32_t k2b200_fsa_arc_post(const int32_t *row_splits1, const int32_t *row_ids1,
                            const int32_t *row_ids2, const void *arcs,
                            int32_t num_fsas, int32_t num_arcs, int32_t use_double,
                            const void *forward, const void *backward,
                            void *arc_post, void *stream);

/* grad[a] = exp(arc_post[a]) * tot_scores_grad[fsa(a) * grad_stride]; float32
 * output.  Replaces GetTotScoresLogBackward,
 * k2/python/csrc/torch/fsa.cu:544-592 (grad_stride is 0 when autograd expanded
 * the gradient of a sum, :565-566). */
int32_t k2b200_tot_scores_log_backward(const int32_t *row_ids1, const int32_t *row_ids2,
                                       int32_t num_arcs, int32_t use_double,
                                       const void *arc_post,
                                       const void *tot_scores_grad,
                                       int64_t grad_stride, float *arc_grad,
                                       void *stream);

/* grad (zero-filled here) gets tot_scores_grad[fsa] on the arcs of the best
 * paths.  Replaces GetTotScoresTropicalBackward,
 * k2/python/csrc/torch/fsa.cu:493-534. */
int32_t k2b200_tot_scores_tropical_backward(const int32_t *row_ids1,
                                            const int32_t *row_ids2, int32_t num_arcs,
                                            const int32_t *best_arcs,
                                            int32_t num_best_arcs, int32_t use_double,
                                            const void *tot_scores_grad,
                                            int64_t grad_stride, float *arc_grad,
                                            void *stream);

/* in_out[index[k]] += value[k] for index[k] >= 0 (atomic float adds).
 * Replaces k2::IndexAdd, k2/csrc/tensor_ops.cu:304-334, as bound by
 * _k2.index_add, k2/python/csrc/torch/index_add.cu:38-71, and used by
 * _IntersectDenseFunction.backward, k2/python/k2/autograd.py:649-650. */
int32_t k2b200_index_add(const int32_t *index, const float *value, int32_t n,
                         float *in_out, int64_t in_out_size, void *stream);

/* out[k] = index[k] >= 0 ? src[index[k]] : 0 (int32).  Replaces the 1-D
 * _k2.index_select used to carry arc attributes through arc_map_a,
 * k2/python/csrc/torch/index_select.cu:56-92 (autograd.py:580-590). */
int32_t k2b200_index_select_i32(const int32_t *src, int64_t src_size,
                                const int32_t *index, int32_t n, int32_t *out,
                                void *stream);

/* Best path per FSA from entering_arcs (see k2b200_fsa_scores): path_splits
 * [num_fsas+1] and best_arcs (arc idx012 in path order; capacity: the number
 * of states) are written on the device; the total number of best-path arcs is
 * path_splits[num_fsas].  An FSA whose trace does not reach its start state
 * gets an empty path.  tmp: k2b200_shortest_path_tmp_bytes(num_fsas) bytes.
 * Replaces k2::ShortestPath, k2/csrc/fsa_algo.cu:869-1144. */
size_t k2b200_shortest_path_tmp_bytes(int32_t num_fsas);
int32_t k2b200_shortest_path(const int32_t *row_splits1, const void *arcs,
                             const int32_t *entering_arcs, int32_t num_fsas,
                             int32_t *path_splits, int32_t *best_arcs, void *tmp,
                             void *stream);

/* Layering of a top-sorted, acyclic FsaVec for k2b200_fsa_scores (what the
 * reference calls state batches, k2::GetStateBatches, k2/csrc/fsa_utils.cu:679-899):
 * level_offsets[num_fsas+1] and level_splits[<= num_states+1] (allocate
 * num_states + 1 entries; level_offsets[num_fsas] is the number of layers).  Every
 * arc leads from a lower to a higher layer.  *status (device) receives 0, or 1 when
 * some arc does not lead to a higher-numbered state (not top-sorted, cyclic or a
 * self-loop): the outputs are then meaningless.  row_ids2[num_arcs]: state (idx01)
 * of every arc.  tmp: k2b200_fsa_levels_tmp_bytes(num_states) bytes. */
size_t k2b200_fsa_levels_tmp_bytes(int32_t num_states);
int32_t k2b200_fsa_levels(const int32_t *row_splits1, const int32_t *row_splits2,
                          const int32_t *row_ids2, const void *arcs, int32_t num_fsas,
                          int32_t num_states, int32_t num_arcs, int32_t *level_offsets,
                          int32_t *level_splits, int32_t *status, void *tmp, void *stream);

/* Per-FSA property bits (k2/csrc/fsa.h:75-101) and their AND.
 * Replaces k2::GetFsaVecBasicProperties, k2/csrc/fsa.cu:54-217.  tmp must hold
 * k2b200_fsa_properties_tmp_bytes(...) bytes; properties[num_fsas+1] is written
 * on the device with the AND over FSAs in the last entry. */
size_t k2b200_fsa_properties_tmp_bytes(int32_t num_fsas, int32_t num_states);
int32_t k2b200_fsa_properties(const int32_t *row_splits1, const int32_t *row_ids1,
                              const int32_t *row_splits2, const int32_t *row_ids2,
                              const void *arcs, int32_t num_fsas, int32_t num_states,
                              int32_t num_arcs, int32_t *properties, void *tmp,
                              void *stream);

/* ---------------------------------------------------------------------------
 * Derivatives through per-state scores, for callers that differentiate
 * get_forward_scores / get_backward_scores / get_arc_post.
 * Replace k2::BackpropGetForwardScores (k2/csrc/fsa_utils.cu:1638-1795),
 * k2::BackpropGetBackwardScores (:1457-1624) and k2::BackpropGetArcPost
 * (:1281-1334), bound as _k2.backprop_get_{forward,backward}_scores_{float,double}
 * and _k2.backprop_get_arc_post_* (k2/python/csrc/torch/fsa.cu:293-366, :461-490).
 *
 * k2b200_fsa_scores_backprop: `scores` are the forward (forward != 0) or backward
 * scores of `fsas` in the given semiring and type; state_deriv[num_states] holds
 * dL/d(score) on entry and is overwritten with the accumulated per-state
 * derivatives; arc_deriv[num_arcs] receives dL/d(arc score).  The view needs the
 * layering; the backward direction also the incoming-arc index.  Tropical forward
 * scores need entering_arcs[num_states] (from k2b200_fsa_scores); tropical backward
 * scores need best_leaving_tmp[num_states] as scratch and row_ids1 in the view.
 * One launch, one CTA per FSA walking its layers.
 *
 * k2b200_fsa_arc_post_backprop: forward_deriv[s] / backward_deriv[s] = sum of
 * arc_post_deriv over the arcs leaving / entering s, except the final state's
 * forward and the start state's backward derivative, which are -0.5 times the sum
 * over all arcs of the FSA.
 * ------------------------------------------------------------------------- */
int32_t k2b200_fsa_scores_backprop(const k2b200_fsa_view *fsas, int32_t forward,
                                   int32_t log_semiring, int32_t use_double,
                                   const void *scores, const int32_t *entering_arcs,
                                   void *state_deriv, void *arc_deriv,
                                   int32_t *best_leaving_tmp, void *stream);
int32_t k2b200_fsa_arc_post_backprop(const k2b200_fsa_view *fsas, int32_t use_double,
                                     const void *arc_post_deriv, void *forward_deriv,
                                     void *backward_deriv, void *stream);

/* ---------------------------------------------------------------------------
 * Sum of a rank's losses and the all-reduce of (loss, frames) over the GPUs of a node,
 * in one kernel over peer memory.  Replaces the `-1 * tot_scores` ... `.sum()` of
 * k2/python/k2/ctc_loss.py:72-84 together with the trainer's all-reduce of the summed
 * loss and the frame count (the reference leaves that collective to the training
 * script); utterances are independent, so it is the only exchange of the path.
 *
 *   k2b200_peer_reduce_create: allocates this rank's exchange buffer on the current device,
 *     zeroed, and returns its address and a K2B200_IPC_HANDLE_BYTES-byte handle that the
 *     other processes of the node pass to k2b200_peer_reduce_open (exchange the handles over
 *     any host channel, e.g. the process group's store) to map it; _close unmaps, _destroy
 *     frees.  With one rank no handle needs to travel.
 *   k2b200_loss_sum_all_reduce: out[0] = sum over ranks of sign * sum(values[0..n)),
 *     out[1] = sum over ranks of num_frames (device, float64), the same bits on every rank.
 *     values: device, float32 (values_are_f32 != 0) or float64.  bufs[world]: host array,
 *     bufs[r] = rank r's buffer as mapped in this process (bufs[rank] = the own one).
 *     seq: 1, 2, 3, ... - the same on every rank for the same step.  Every rank of the world
 *     must make the call; a rank's launch waits (occupying one CTA) for the others'.  That
 *     wait is bounded: after poll_limit polls (negative: the default, a few seconds) bit 0
 *     of the status word is set and out is invalid; nothing hangs or traps.  With
 *     after_stream not NULL (and not `stream`) the launch on `stream` is ordered behind
 *     everything after_stream holds at the time of the call: the stream that computes
 *     `values` never waits for another rank, the exchange runs beside it.
 *   k2b200_peer_reduce_status: waits for `stream`, returns the status word.
 * ------------------------------------------------------------------------- */
#define K2B200_IPC_HANDLE_BYTES 64
int32_t k2b200_peer_reduce_create(void **local_buf, void *ipc_handle_out);
int32_t k2b200_peer_reduce_open(const void *ipc_handle, void **peer_buf);
int32_t k2b200_peer_reduce_close(void *peer_buf);
int32_t k2b200_peer_reduce_destroy(void *local_buf);
int32_t k2b200_loss_sum_all_reduce(const void *values, int32_t n, int32_t values_are_f32,
                                   double sign, double num_frames, void *const *bufs,
                                   int32_t rank, int32_t world, uint64_t seq,
                                   int32_t poll_limit, double *out, void *stream,
                                   void *after_stream);
int32_t k2b200_peer_reduce_status(void *local_buf, void *stream, int32_t *status);

#ifdef __cplusplus
}
#endif
#endif /* K2B200_H_ */

// Internal declarations shared by intersect.cu and viterbi_persistent.cu.
#pragma once
#include <vector>

#include "../../include/k2b200.h"
#include "common.cuh"

namespace k2b {

// Per (graph, sequence) pair; built on the host, uploaded once per call.
struct FsaInfo {
  int32_t state_off;   // first state (idx01) of the graph in a_fsas
  int32_t num_states;  // S
  int32_t arc_off;     // first arc (idx012)
  int32_t num_arcs;
  int32_t row0;        // first row of the sequence in `scores`
  int32_t tk;          // rows of the sequence = frames + 1 (k2's FsaInfo.T)
  int32_t level_off;   // sum over earlier pairs of (tk + 1)
  int32_t words;       // ceil(S / 32)
  int32_t arc_out_off; // added to a graph arc index when it names the arc to the caller
                       // (arc_map_a, grad_a): non-zero only when graphs share storage
  int64_t grid_off;    // sum over earlier pairs of (tk + 1) * S
  int64_t word_off;    // sum over earlier pairs of (tk + 1) * words
};

struct Layout {
  std::vector<FsaInfo> infos;
  int64_t grid_elems = 0, total_words = 0, total_levels = 0;
  int32_t max_states = 0, max_tk = 0, max_arcs = 0;
  // byte offsets into the workspace
  size_t off_infos, off_cutoffs, off_fwd, off_bwd, off_mask, off_counts, off_scan_tmp,
      off_block_cand, off_totals, off_plan, off_unfit, off_shared_vit, total_bytes;
  // one large graph shared by all sequences: the sequence-per-lane Viterbi kernels and their
  // transposed buffers (viterbi_shared.cu)
  bool shared_vit = false;
  // graphs with states of more than four arcs, small enough for one CTA: lanes are
  // assigned to states by a plan (viterbi_persistent.cu)
  bool lane_plan = false;
  int32_t count_blocks, tiles_per_pair, emit_tiles_per_pair;
};

// intersect.cu
int32_t MakeLayout(const k2b200_intersect_args *a, Layout *L);
int32_t RunViterbi(const Layout &L, const k2b200_intersect_args *a, char *ws,
                   cudaStream_t stream, bool plan_ready = false);
// sizes_only: just the totals the beam reduction needs (states and candidate arcs),
// no keep masks or numbering.
int32_t LaunchSizeCount(const Layout &L, const k2b200_intersect_args *args, char *ws,
                        cudaStream_t stream);
bool ReduceBeam(const k2b200_intersect_args *args, const long long *h_totals, float *beam);
int32_t PruneLoop(const Layout &L, const k2b200_intersect_args *args, char *ws,
                  cudaStream_t stream, float *beam_io, long long *h_totals,
                  bool sizes_only = false);
// cutoffs[i] = min(best forward, best backward total) - beam, from the Viterbi grids
int32_t LaunchCutoffs(const Layout &L, const k2b200_intersect_args *a, char *ws, float beam,
                      cudaStream_t stream);

// viterbi_shared.cu
bool SharedViterbiApplies(const Layout &L, const k2b200_intersect_args *a);
size_t SharedViterbiBytes(const Layout &L, const k2b200_intersect_args *a);
int32_t LaunchSharedViterbi(const Layout &L, const k2b200_intersect_args *a, char *region,
                            const FsaInfo *d_infos, float *fwd, float *bwd, cudaStream_t stream);

// viterbi_persistent.cu
bool PersistentViterbiFits(const Layout &L, const k2b200_intersect_args *a);
int32_t LaunchPersistentViterbi(const Layout &L, const k2b200_intersect_args *a,
                                const FsaInfo *d_infos, float *fwd, float *bwd,
                                cudaStream_t stream, const int32_t *only_unfit = nullptr);

// Lane plans: CTA size and arcs per lane of the kernels that use them.
constexpr int kLaneThreads = 768;
constexpr int kLaneDeg = 8;
bool LanePlanApplies(const Layout &L, const k2b200_intersect_args *a);
// Clears unfit[] and, when L.lane_plan, writes the plans of both directions.
int32_t LaunchPlanLanes(const Layout &L, const k2b200_intersect_args *a, char *ws,
                        cudaStream_t stream);
int32_t LaunchLanesViterbi(const Layout &L, const k2b200_intersect_args *a,
                           const FsaInfo *d_infos, float *fwd, float *bwd, const int32_t *plan,
                           const int32_t *unfit, cudaStream_t stream);

bool RegisterViterbiFits(const Layout &L, const k2b200_intersect_args *a);
int32_t LaunchRegisterViterbi(const Layout &L, const k2b200_intersect_args *a,
                              const FsaInfo *d_infos, float *fwd, float *bwd,
                              cudaStream_t stream);

}  // namespace k2b

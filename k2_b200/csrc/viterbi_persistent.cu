// Persistent frame-synchronous Viterbi kernel for graphs that fit in shared memory.
//
// One CTA per (graph/sequence pair, direction) walks all frames in-kernel: the
// graph's arcs (in incoming order for the forward direction, leaving order for
// the backward one) and the two ping-pong score vectors live in shared memory,
// the dense rows are prefetched into a shared-memory ring with cp.async several
// frames ahead of the recursion, and one __syncthreads per frame is the only
// synchronisation.  Each frame's state scores are also written to the global
// (t, state) grids that the pruning pass reads.
//
// Same arithmetic as the per-frame launch path (and as the reference's DoStep,
// k2/csrc/intersect_dense.cu:778-847): (prev + arc.score) + dense, then max.
#include <algorithm>
#include <vector>

#include <type_traits>

#include "cp_async.cuh"
#include "intersect_internal.cuh"

namespace k2b {

constexpr size_t kSmemBudget = 200 * 1024;  // of the 227 KB a CTA may use
constexpr int kMaxStages = 8;

struct SmemPlan {
  int32_t s_pad, a_pad, row_pad, stages;
  size_t bytes;
};

static SmemPlan PlanSmem(int32_t max_states, int32_t max_arcs, int32_t cols) {
  SmemPlan p;
  p.s_pad = (max_states + 1 + 3) & ~3;
  p.a_pad = (max_arcs + 3) & ~3;
  p.row_pad = (cols + 1 + 3) & ~3;  // +1: a -inf slot for out-of-range labels
  size_t fixed = sizeof(float) * 2 * p.s_pad      // score ping-pong
                 + sizeof(int32_t) * p.s_pad      // splits
                 + (size_t)12 * p.a_pad;          // other-end state, column slot, score
  size_t row = sizeof(float) * p.row_pad;
  int32_t stages = 0;
  if (fixed < kSmemBudget) stages = (int32_t)std::min<size_t>(kMaxStages, (kSmemBudget - fixed) / row);
  p.stages = stages;
  p.bytes = fixed + row * std::max(stages, 0);
  return p;
}

bool PersistentViterbiFits(const Layout &L, const k2b200_intersect_args *a) {
  SmemPlan p = PlanSmem(L.max_states, L.max_arcs, a->cols);
  return p.stages >= 2 && a->num_fsas <= 65535;
}

// grid = (2 directions, pairs); dynamic shared memory per PlanSmem.
__global__ void __launch_bounds__(1024)
PersistentViterbi(const FsaInfo *__restrict__ infos, const Arc *__restrict__ arcs,
                  const int32_t *__restrict__ a_row_splits2,
                  const int32_t *__restrict__ in_splits, const int32_t *__restrict__ in_arcs,
                  const float *__restrict__ scores, int32_t cols, float *__restrict__ fwd,
                  float *__restrict__ bwd, int32_t s_pad, int32_t a_pad, int32_t row_pad,
                  int32_t stages, int32_t lanes_log2, const int32_t *__restrict__ only_unfit) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  if (only_unfit != nullptr && !only_unfit[blockIdx.y]) return;
  const FsaInfo f = infos[blockIdx.y];
  const int dir = blockIdx.x;  // 0 forward, 1 backward
  const int32_t S = f.num_states, A = f.num_arcs, Tk = f.tk;
  if (S == 0) return;
  float *score_buf = reinterpret_cast<float *>(smem_raw);           // [2][s_pad]
  int32_t *splits = reinterpret_cast<int32_t *>(score_buf + 2 * s_pad);  // [s_pad]
  int32_t *arc_state = splits + s_pad;                              // [a_pad]
  int32_t *arc_col = arc_state + a_pad;                             // [a_pad]
  float *arc_score = reinterpret_cast<float *>(arc_col + a_pad);   // [a_pad]
  float *ring = arc_score + a_pad;                                  // [stages][row_pad]

  const int tid = threadIdx.x, nt = blockDim.x;
  // ---- stage the graph --------------------------------------------------
  const int32_t *gsplits = (dir == 0 ? in_splits : a_row_splits2) + f.state_off;
  for (int32_t s = tid; s <= S; s += nt) splits[s] = gsplits[s] - f.arc_off;
  for (int32_t k = tid; k < A; k += nt) {
    Arc arc = arcs[dir == 0 ? in_arcs[f.arc_off + k] : f.arc_off + k];
    arc_state[k] = dir == 0 ? arc.src : arc.dest;
    int32_t c = arc.label + 1;
    arc_col[k] = (c >= 0 && c < cols) ? c : cols;  // slot `cols` holds -inf
    arc_score[k] = arc.score;
  }
  for (int32_t st = tid; st < stages; st += nt) ring[(size_t)st * row_pad + cols] = -INFINITY;
  // ---- initial scores -----------------------------------------------------
  float *grid = (dir == 0 ? fwd : bwd) + f.grid_off;
  for (int32_t s = tid; s < S; s += nt) {
    float v = (dir == 0 ? (s == 0) : (s == S - 1)) ? 0.0f : -INFINITY;
    score_buf[s] = v;
    grid[(int64_t)(dir == 0 ? 0 : Tk) * S + s] = v;
  }
  // ---- prefetch the first stages-1 rows -----------------------------------
  // step t (1..Tk) consumes dense row t-1 (forward) or Tk-t (backward)
  auto issue_row = [&](int32_t step) {
    if (step <= Tk) {
      const int64_t row = (int64_t)f.row0 + (dir == 0 ? step - 1 : Tk - step);
      const float *src = scores + row * cols;
      float *dst = ring + (size_t)((step - 1) % stages) * row_pad;
      for (int32_t c = tid; c < cols; c += nt) CpAsync4(dst + c, src + c);
    }
    CpAsyncCommit();  // always commit so the group count stays uniform
  };
  for (int32_t step = 1; step < stages; ++step) issue_row(step);

  const int32_t G = 1 << lanes_log2, g = tid & (G - 1);
  const int32_t states_per_pass = nt >> lanes_log2;
  for (int32_t t = 1; t <= Tk; ++t) {
    CpAsyncWaitDyn(stages - 2);  // this thread's copies of row for step t have landed
    __syncthreads();             // ... everyone's have; previous frame's scores are complete
    issue_row(t + stages - 1);   // refills the slot consumed by step t-1
    const float *cur = score_buf + ((t - 1) & 1) * s_pad;
    float *nxt = score_buf + (t & 1) * s_pad;
    const float *row = ring + (size_t)((t - 1) % stages) * row_pad;
    float *gout = grid + (int64_t)(dir == 0 ? t : Tk - t) * S;
    for (int32_t s0 = 0; s0 < S; s0 += states_per_pass) {
      const int32_t s = s0 + (tid >> lanes_log2);
      float best = -INFINITY;
      if (s < S) {
        for (int32_t k = splits[s] + g; k < splits[s + 1]; k += G) {
          float v = __fadd_rn(__fadd_rn(cur[arc_state[k]], arc_score[k]), row[arc_col[k]]);
          best = v > best ? v : best;
        }
      }
      for (int32_t d = G >> 1; d > 0; d >>= 1) {
        float o = __shfl_xor_sync(0xffffffffu, best, d);
        best = o > best ? o : best;
      }
      if (s < S && g == 0) {
        nxt[s] = best;
        gout[s] = best;
      }
    }
  }
  CpAsyncWait<0>();
}

// ---------------------------------------------------------------------------
// Register variant for graphs whose states have at most kMaxDeg arcs in each
// direction (CTC graphs have 3) and at most 1024 states: one thread per state keeps
// its arcs in registers and fetches the dense scores of its own arcs straight from
// global memory kPrefetch frames ahead, so a frame costs one __syncthreads, kMaxDeg
// shared-memory reads of the previous frame's scores and a few adds.  Unused arc
// slots carry a score of -inf and never win the max.
// ---------------------------------------------------------------------------
constexpr int kRegMaxDeg = 4;  // largest degree any instantiation handles

bool RegisterViterbiFits(const Layout &L, const k2b200_intersect_args *a) {
  return a->a_max_degree > 0 && a->a_max_degree <= kRegMaxDeg && L.max_states <= 1024 &&
         a->num_fsas <= 65535;
}

template <int kMaxThreads, int kDeg, int kRegPrefetch>
__global__ void __launch_bounds__(kMaxThreads)
RegisterViterbi(const FsaInfo *__restrict__ infos, const Arc *__restrict__ arcs,
                const int32_t *__restrict__ a_row_splits2, const int32_t *__restrict__ in_splits,
                const int32_t *__restrict__ in_arcs, const float *__restrict__ scores,
                int32_t cols, float *__restrict__ fwd, float *__restrict__ bwd) {
  __shared__ float buf[2][1024];
  const FsaInfo f = infos[blockIdx.y];
  const int dir = blockIdx.x;
  const int32_t S = f.num_states, Tk = f.tk;
  if (S == 0) return;
  const int32_t s = threadIdx.x;
  const bool active = s < S;

  int32_t other[kDeg], col[kDeg];
  float w[kDeg];
#pragma unroll
  for (int j = 0; j < kDeg; ++j) {
    other[j] = 0;
    col[j] = 0;
    w[j] = -INFINITY;
  }
  if (active) {
    const int32_t *splits = dir == 0 ? in_splits : a_row_splits2;
    const int32_t a0 = splits[f.state_off + s], n = splits[f.state_off + s + 1] - a0;
#pragma unroll
    for (int j = 0; j < kDeg; ++j) {
      if (j < n) {
        const Arc arc = arcs[dir == 0 ? in_arcs[a0 + j] : a0 + j];
        other[j] = dir == 0 ? arc.src : arc.dest;
        const int32_t c = arc.label + 1;
        if (c >= 0 && c < cols) {
          col[j] = c;
          w[j] = arc.score;
        }
      }
    }
  }
  // step t (1..Tk) consumes dense row t-1 (forward) or Tk-t (backward)
  const float *base = scores + (int64_t)f.row0 * cols;
  auto row_of = [&](int32_t step) {
    step = step > Tk ? Tk : step;
    return dir == 0 ? step - 1 : Tk - step;
  };
  float x[kDeg][kRegPrefetch];
#pragma unroll
  for (int d = 0; d < kRegPrefetch; ++d) {
    const int32_t r = row_of(1 + d) * cols;
#pragma unroll
    for (int j = 0; j < kDeg; ++j) x[j][d] = __ldg(base + r + col[j]);
  }
  float *grid = (dir == 0 ? fwd : bwd) + f.grid_off;
  {
    const float v = (dir == 0 ? (s == 0) : (s == S - 1)) ? 0.0f : -INFINITY;
    buf[0][s] = v;
    if (active) grid[(int64_t)(dir == 0 ? 0 : Tk) * S + s] = v;
  }
  for (int32_t t0 = 1; t0 <= Tk; t0 += kRegPrefetch) {
#pragma unroll
    for (int u = 0; u < kRegPrefetch; ++u) {
      const int32_t t = t0 + u;
      if (t > Tk) break;
      __syncthreads();
      const float *cur = buf[(t - 1) & 1];
      float best = -INFINITY;
#pragma unroll
      for (int j = 0; j < kDeg; ++j) {
        const float v = __fadd_rn(__fadd_rn(cur[other[j]], w[j]), x[j][u]);
        best = v > best ? v : best;
      }
      const int32_t r = row_of(t + kRegPrefetch) * cols;
#pragma unroll
      for (int j = 0; j < kDeg; ++j) x[j][u] = __ldg(base + r + col[j]);
      buf[t & 1][s] = best;
      if (active) grid[(int64_t)(dir == 0 ? t : Tk - t) * S + s] = best;
    }
  }
}

// ---------------------------------------------------------------------------
// Lane plans.  The recursion kernel keeps the arcs of state s in the registers of
// G(s) = ceil(degree(s) / kDeg) lanes of one warp, so that a frame costs every lane
// the same few arcs whatever the degree distribution of the graph is.  PlanLanes
// lays the lane groups of one graph and direction out over a CTA of kLaneThreads
// threads: groups sorted by size, largest first (states in increasing order within
// a size), packed next-fit into warps - a group never straddles two warps.
//   plan[(dir * n + i) * kLaneThreads + thread] = state | lane << 16 | G << 24, or -1
// bit 0 of unfit[i] is set when graph i needs more lanes than a CTA has (or has more than
// 32 * kDeg arcs on a state); the shared-memory kernels below take those graphs.
// Graphs whose largest degree is at most kDeg need no plan: thread s owns state s.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
PlanLanes(const FsaInfo *__restrict__ infos, int32_t n,
          const int32_t *__restrict__ a_row_splits2, const int32_t *__restrict__ in_splits,
          int32_t k_deg, int32_t *__restrict__ plan, int32_t *__restrict__ unfit) {
  // per group size G = 1..32: number of states, lanes left in the warp where the
  // size class starts, first lane of that start, first lane of the following warps
  __shared__ int32_t count[33], head_room[33], head_pos[33], body_pos[33];
  __shared__ int32_t bad;
  const int32_t i = blockIdx.y, dir = blockIdx.x;
  const FsaInfo f = infos[i];
  const int32_t S = f.num_states;
  const int tid = threadIdx.x, nt = blockDim.x;
  int32_t *out = plan + ((int64_t)dir * n + i) * kLaneThreads;
  for (int32_t t = tid; t < kLaneThreads; t += nt) out[t] = -1;
  if (tid < 33) count[tid] = 0;
  if (tid == 0) bad = S > kLaneThreads;
  __syncthreads();
  const int32_t *splits = (dir == 0 ? in_splits : a_row_splits2) + f.state_off;
  auto lanes_of = [&](int32_t s) {
    const int32_t deg = splits[s + 1] - splits[s];
    return deg <= k_deg ? 1 : (deg + k_deg - 1) / k_deg;
  };
  if (S <= kLaneThreads)
    for (int32_t s = tid; s < S; s += nt) {
      const int32_t G = lanes_of(s);
      if (G > 32) bad = 1; else atomicAdd(&count[G], 1);
    }
  __syncthreads();
  if (tid == 0 && !bad) {
    int32_t pos = 0;
    for (int G = 32; G >= 1; --G) {
      const int32_t c = count[G];
      if (c == 0) continue;
      const int32_t room = (32 - (pos & 31)) / G;  // groups that still fit in this warp
      const int32_t per_warp = 32 / G;
      head_room[G] = room;
      head_pos[G] = pos;
      if (c <= room) {
        pos += c * G;
      } else {
        const int32_t rest = c - room;
        const int32_t body = (pos + room * G + 31) & ~31;
        body_pos[G] = body;
        pos = body + (rest / per_warp) * 32 + (rest % per_warp) * G;
      }
      if (pos > kLaneThreads) bad = 1;
    }
  }
  __syncthreads();
  if (bad) {
    if (tid == 0) atomicOr(&unfit[i], 1);
    return;
  }
  // warp w places the size classes w, w + 8, ...: ordered compaction by ballot
  const int warp = tid >> 5, lane = tid & 31;
  for (int G = 1 + warp; G <= 32; G += nt >> 5) {
    if (count[G] == 0) continue;
    const int32_t per_warp = 32 / G, room = head_room[G];
    int32_t seen = 0;
    for (int32_t s0 = 0; s0 < S; s0 += 32) {
      const int32_t s = s0 + lane;
      const bool in = s < S && lanes_of(s) == G;
      const uint32_t m = __ballot_sync(0xffffffffu, in);
      if (in) {
        const int32_t j = seen + __popc(m & ((1u << lane) - 1u));
        int32_t p0;
        if (j < room) {
          p0 = head_pos[G] + j * G;
        } else {
          const int32_t r = j - room;
          p0 = body_pos[G] + (r / per_warp) * 32 + (r % per_warp) * G;
        }
        for (int32_t g = 0; g < G; ++g) out[p0 + g] = s | (g << 16) | (G << 24);
      }
      seen += __popc(m);
    }
  }
}


bool LanePlanApplies(const Layout &L, const k2b200_intersect_args *a) {
  const bool register_fit = a->a_max_degree > 0 && a->a_max_degree <= 4 && L.max_states <= 1024;
  return !register_fit && L.max_states <= kLaneThreads && a->num_fsas <= 65535 &&
         PersistentViterbiFits(L, a);
}

int32_t LaunchPlanLanes(const Layout &L, const k2b200_intersect_args *a, char *ws,
                        cudaStream_t stream) {
  int32_t *unfit = reinterpret_cast<int32_t *>(ws + L.off_unfit);
  K2B_CUDA_OK(cudaMemsetAsync(unfit, 0, sizeof(int32_t) * a->num_fsas, stream));
  if (!L.lane_plan) return kOk;
  { PlanLanes<<<dim3(2, a->num_fsas), 256, 0, stream>>>(
      reinterpret_cast<const FsaInfo *>(ws + L.off_infos), a->num_fsas, a->a_row_splits2,
      a->a_in_splits, kLaneDeg, reinterpret_cast<int32_t *>(ws + L.off_plan), unfit);
    NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

// ---------------------------------------------------------------------------
// Viterbi recursion with planned lanes: as RegisterViterbi, but the arcs of a state
// are spread over the G(s) lanes its plan gives it, which take the max by shuffles.
// The rows of dense scores arrive in a ring in shared memory by 4-byte cp.async, kVitAhead
// frames ahead (rows of C + 1 floats are not 16-byte aligned).  The frame loop is unrolled
// over the ring, so a frame costs a lane, per arc, a load of the neighbour's score and of
// the dense score at constant offsets, two additions and a max.  When all arcs of a warp's
// lanes carry the label of their state (walking forward in a graph where every state has
// one entering label) the dense score is added once per state, after the max: rounding is
// monotonic, so max_j fl(y_j + x) = fl(max_j y_j + x), bit for bit.
// Graphs marked unfit are skipped (PersistentViterbi handles them).
// ---------------------------------------------------------------------------
constexpr int kVitRing = 4;   // slots of the row ring = frames per unrolled group
constexpr int kVitAhead = 3;  // rows requested ahead of the frame that uses them

// kV: plan lanes per thread.  Thread t of a CTA of kLaneThreads / kV threads works for the
// plan's lanes t, t + blockDim, ...: a multiple of 32 apart, so the lanes of a plan warp stay
// the lanes of one warp and the shuffles of a group work as before.  Fewer, fatter warps:
// the per-frame cost of a warp that does not depend on its arcs (barrier, row ring, loop) is
// paid fewer times, and the gathers of a thread's lanes are in flight together.
template <int kDeg, int kV>
__global__ void __launch_bounds__(kLaneThreads / kV)
LanesViterbi(const FsaInfo *__restrict__ infos, int32_t n, const Arc *__restrict__ arcs,
             const int32_t *__restrict__ a_row_splits2, const int32_t *__restrict__ in_splits,
             const int32_t *__restrict__ in_arcs, const float *__restrict__ scores,
             int32_t cols, int32_t cols_pad, float *__restrict__ fwd, float *__restrict__ bwd,
             const int32_t *__restrict__ plan, const int32_t *__restrict__ unfit) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float buf[2][kLaneThreads];
  const int32_t i = blockIdx.y;
  if (unfit[i] & 1) return;
  const FsaInfo f = infos[i];
  const int dir = blockIdx.x;
  const int32_t S = f.num_states, Tk = f.tk;
  if (S == 0) return;
  const int tid = threadIdx.x, nt = blockDim.x;  // nt == kLaneThreads / kV
  float *ring = reinterpret_cast<float *>(smem_raw);  // [kVitRing][cols_pad]
  int32_t s[kV], g[kV], G[kV], g_max[kV], col0[kV];
  int32_t other[kV][kDeg], col[kV][kDeg];
  float w[kV][kDeg];
  bool same = true;
#pragma unroll
  for (int v = 0; v < kV; ++v) {
    s[v] = -1;
    g[v] = 0;
    G[v] = 1;
    col0[v] = -1;
    const int32_t code = plan[((int64_t)dir * n + i) * kLaneThreads + tid + v * nt];
    if (code >= 0) {
      s[v] = code & 0xffff;
      g[v] = (code >> 16) & 0xff;
      G[v] = code >> 24;
    }
#pragma unroll
    for (int j = 0; j < kDeg; ++j) {
      other[v][j] = 0;
      col[v][j] = 0;
      w[v][j] = -INFINITY;
    }
    if (s[v] >= 0) {
      const int32_t *splits = dir == 0 ? in_splits : a_row_splits2;
      const int32_t a0 = splits[f.state_off + s[v]], a1 = splits[f.state_off + s[v] + 1];
#pragma unroll
      for (int j = 0; j < kDeg; ++j) {
        const int32_t k = a0 + g[v] + j * G[v];
        if (k < a1) {
          const Arc arc = arcs[dir == 0 ? in_arcs[k] : k];
          other[v][j] = dir == 0 ? arc.src : arc.dest;
          const int32_t c = arc.label + 1;
          if (c >= 0 && c < cols) {
            col[v][j] = c;
            w[v][j] = arc.score;
            if (col0[v] < 0) col0[v] = c;
            else if (c != col0[v]) same = false;
          }
        }
      }
    }
    if (col0[v] < 0) col0[v] = 0;
    g_max[v] = __reduce_max_sync(0xffffffffu, G[v]);  // widest lane group of this plan warp
  }
  const bool hoist = __syncthreads_and(same);  // uniform over the CTA
  // step t (1..Tk) consumes dense row t-1 (forward) or Tk-t (backward)
  const float *base = scores + (int64_t)f.row0 * cols;
  auto issue_row = [&](int32_t step, int32_t slot) {
    if (step <= Tk) {
      const float *src = base + (int64_t)(dir == 0 ? step - 1 : Tk - step) * cols;
      float *dst = ring + slot * cols_pad;
      for (int32_t c = tid; c < cols; c += nt) CpAsync4(dst + c, src + c);
    }
    CpAsyncCommit();
  };
  for (int32_t step = 1; step <= kVitAhead; ++step) issue_row(step, (step - 1) % kVitRing);
  float *grid = (dir == 0 ? fwd : bwd) + f.grid_off;
  for (int32_t q = tid; q < S; q += nt) {
    const float v0 = (dir == 0 ? (q == 0) : (q == S - 1)) ? 0.0f : -INFINITY;
    buf[0][q] = v0;
    grid[(int64_t)(dir == 0 ? 0 : Tk) * S + q] = v0;
  }
  const int64_t stride = dir == 0 ? (int64_t)S : -(int64_t)S;
  float *gout = grid + (dir == 0 ? 1 : Tk - 1) * (int64_t)S;
  // the frame loop once per kind of CTA, so that the unrolled code of only one is fetched
  auto frames = [&](auto hoist_tag) {
    constexpr bool kHoist = decltype(hoist_tag)::value;
  for (int32_t t0 = 1; t0 <= Tk; t0 += kVitRing) {
#pragma unroll
      for (int u = 0; u < kVitRing; ++u) {
        const int32_t t = t0 + u;
        if (t > Tk) break;
        CpAsyncWait<kVitAhead - 1>();  // this thread's part of row t has landed
        __syncthreads();               // ... everyone's has; the scores of step t - 1 are complete
        issue_row(t + kVitAhead, (u + kVitAhead) % kVitRing);
        const float *cur = buf[u & 1];  // t0 is odd: (t - 1) & 1 == u & 1
        const float *row = ring + u * cols_pad;
        float best[kV];
#pragma unroll
        for (int v = 0; v < kV; ++v) {
          best[v] = -INFINITY;
          if (kHoist) {
#pragma unroll
            for (int j = 0; j < kDeg; ++j) {
              const float x = __fadd_rn(cur[other[v][j]], w[v][j]);
              best[v] = x > best[v] ? x : best[v];
            }
          } else {
#pragma unroll
            for (int j = 0; j < kDeg; ++j) {
              const float x = __fadd_rn(__fadd_rn(cur[other[v][j]], w[v][j]), row[col[v][j]]);
              best[v] = x > best[v] ? x : best[v];
            }
          }
        }
#pragma unroll
        for (int v = 0; v < kV; ++v) {
#pragma unroll
          for (int32_t d = 16; d > 0; d >>= 1) {
            if (d < g_max[v]) {  // warp-uniform
              const float o = __shfl_down_sync(0xffffffffu, best[v], d);
              if (g[v] + d < G[v]) best[v] = o > best[v] ? o : best[v];
            }
          }
          if (s[v] >= 0 && g[v] == 0) {
            if (kHoist) best[v] = __fadd_rn(best[v], row[col0[v]]);
            buf[(u + 1) & 1][s[v]] = best[v];
            gout[s[v]] = best[v];
          }
        }
        gout += stride;
      }
    }
  };
  if (hoist) frames(std::true_type{}); else frames(std::false_type{});
  CpAsyncWait<0>();
}

int32_t LaunchLanesViterbi(const Layout &L, const k2b200_intersect_args *a,
                           const FsaInfo *d_infos, float *fwd, float *bwd, const int32_t *plan,
                           const int32_t *unfit, cudaStream_t stream) {
  (void)L;
  dim3 grid(2, a->num_fsas);
  const int32_t cols_pad = (a->cols + 3) & ~3;
  const size_t smem = sizeof(float) * kVitRing * (size_t)cols_pad;
  K2B_REQUIRE(smem <= 200 * 1024, "too many columns for the lane Viterbi kernel");
  constexpr int kV = 1;  // plan lanes per thread (2 was slower: 0.39 against 0.30 ms at 500 frames)
  K2B_CUDA_OK(cudaFuncSetAttribute(LanesViterbi<kLaneDeg, kV>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  { LanesViterbi<kLaneDeg, kV><<<grid, kLaneThreads / kV, smem, stream>>>(
      d_infos, a->num_fsas, reinterpret_cast<const Arc *>(a->a_arcs), a->a_row_splits2,
      a->a_in_splits, a->a_in_arcs, a->scores, a->cols, cols_pad, fwd, bwd, plan, unfit);
    NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t LaunchRegisterViterbi(const Layout &L, const k2b200_intersect_args *a,
                              const FsaInfo *d_infos, float *fwd, float *bwd,
                              cudaStream_t stream) {
  int32_t threads = std::max(32, (L.max_states + 31) / 32 * 32);
  dim3 grid(2, a->num_fsas);
  const Arc *arcs = reinterpret_cast<const Arc *>(a->a_arcs);
#define K2B_LAUNCH_REG(MAXT, DEG, PF)                                                      \
  { RegisterViterbi<MAXT, DEG, PF><<<grid, threads, 0, stream>>>(                         \
        d_infos, arcs, a->a_row_splits2, a->a_in_splits, a->a_in_arcs, a->scores, a->cols, \
        fwd, bwd); NoteLaunch(); }
  if (threads <= 512) {
    if (a->a_max_degree <= 3) K2B_LAUNCH_REG(512, 3, 12) else K2B_LAUNCH_REG(512, 4, 8)
  } else {
    if (a->a_max_degree <= 3) K2B_LAUNCH_REG(1024, 3, 8) else K2B_LAUNCH_REG(1024, 4, 6)
  }
#undef K2B_LAUNCH_REG
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t LaunchPersistentViterbi(const Layout &L, const k2b200_intersect_args *a,
                                const FsaInfo *d_infos, float *fwd, float *bwd,
                                cudaStream_t stream, const int32_t *only_unfit) {
  SmemPlan p = PlanSmem(L.max_states, L.max_arcs, a->cols);
  K2B_CUDA_OK(cudaFuncSetAttribute(PersistentViterbi, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)p.bytes));
  // lanes per state: about half the mean degree, so every lane loops ~2 arcs
  int32_t mean_deg = a->num_states > 0 ? (a->num_arcs + a->num_states - 1) / a->num_states : 1;
  int32_t lanes_log2 = 0;
  while ((2 << lanes_log2) <= mean_deg / 2 && lanes_log2 < 5) ++lanes_log2;
  int64_t lanes = (int64_t)L.max_states << lanes_log2;
  int32_t threads = (int32_t)std::min<int64_t>(1024, std::max<int64_t>(128, (lanes + 31) / 32 * 32));
  dim3 grid(2, a->num_fsas);
  { PersistentViterbi<<<grid, threads, p.bytes, stream>>>(
      d_infos, reinterpret_cast<const Arc *>(a->a_arcs), a->a_row_splits2, a->a_in_splits,
      a->a_in_arcs, a->scores, a->cols, fwd, bwd, p.s_pad, p.a_pad, p.row_pad, p.stages,
      lanes_log2, only_unfit); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

}  // namespace k2b

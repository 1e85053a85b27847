// Lattice-free total scores and gradients for band graphs (CTC and alike): the path
//   lattice = intersect_dense(graphs, dense, beam)        k2/csrc/intersect_dense.cu:100-1073
//   tot     = lattice.get_tot_scores(log_semiring=True)   k2/csrc/fsa_utils.cu:1124-1454,1809-1837
//   backward through arc posteriors and both arc maps     k2/csrc/fsa_utils.cu:1839-1901,
//                                                         k2/python/k2/autograd.py:30-117,511-664
// for graphs in which
//   * every arc goes from state s to s, s+1 or s+2, at most one arc per (source, destination), and
//   * all arcs entering a state carry the same label
// (what k2.ctc_graph builds, standard and modified: k2/csrc/fsa_algo.cu:577-730).  Then a state
// needs ONE dense score per frame (that of its label), the recursion over the states of a graph
// has neighbours only, and the states that survive pruning on a frame are few (a few tens out of
// hundreds).  The kernels are built on that:
//
//   BandViterbi   one WARP per (graph, direction) walks all frames: a lane owns K consecutive
//                 states in registers, neighbours come by two shuffles, the log-prob row of the
//                 frame arrives in a shared-memory ring by one bulk copy (TMA, mbarrier) issued
//                 many frames ahead.  No block barrier, no shared-memory traffic for scores.
//                 Same fp32 expressions as the reference: (prev + arc.score) + dense, then max.
//   BandPrep      all (graph, frame) levels in parallel: the reference's keep tests
//                 (intersect_dense.cu:289-296, 430-471) on the two Viterbi grids, then per level
//                 the COMPACT list of surviving states with, per state, exp(dense score) as
//                 mantissa/exponent and one bit per entering / leaving arc that survives.
//   BandChain     one warp per (graph, direction) walks the levels over the compact lists only:
//                 a lane takes one surviving state, reads its neighbours' alpha (beta) of the
//                 previous level from shared memory by state number, and adds the surviving arcs
//                 in mantissa/exponent arithmetic (no exp/log on the chain, any score range).
//                 The lists arrive through a ring of per-lane asynchronous copies.
//   BandGrad      all levels in parallel: posterior of (level, state) = alpha * beta / Z is the
//                 gradient of that state's dense score; optionally arc posteriors for the
//                 gradient of the graph's arc scores.
//
// The dense scores are read straight from the log-prob tensor the DenseFsaVec was made from
// ([rows, C], 16-byte aligned rows): the [rows + N, C + 1] score matrix is not needed.  The extra
// final row of a sequence ([0, -inf, ...], k2/csrc/fsa.h:138-185) is implied: on the level after
// the last frame a state scores 0 if its label is -1 and -inf otherwise.
#include <algorithm>
#include <cmath>
#include <vector>

#include "../../include/k2b200.h"
#include "common.cuh"
#include "cp_async.cuh"
#include "prob_math.cuh"

namespace k2b {

constexpr int32_t kNoLabel = INT32_MIN;
constexpr int kBandMaxStates = 512;   // K = 16 states per lane
constexpr int kBandMaxDepth = 16;     // dense rows in flight per Viterbi warp
constexpr int kRingItems = 64;        // list entries per level staged ahead of the chain
constexpr int kChainAhead = 12;       // levels in flight in the chain kernel
constexpr int kPrepLevels = 16;       // levels per warp of BandPrep
constexpr int kGradLevels = 8;        // levels per warp of BandGrad
constexpr int kDrainPolls = 4000000;  // bounded wait for copies in flight when a kernel gives up

static int32_t g_wait_limit = 4000000;  // polls of an mbarrier before a kernel gives up

// Per (graph, sequence) pair; built on the host, uploaded once per call.
struct BandInfo {
  int32_t state_off;   // first state (idx01) of the graph in a_fsas
  int32_t num_states;  // S
  int32_t pitch;       // S rounded up to a multiple of 4: row pitch of this pair's grids
  int32_t frames;      // T
  int32_t lp_row;      // row of the log-prob matrix that holds frame 0
  int32_t level_off;   // sum over earlier pairs of (T + 2)
  int64_t grid_off;    // sum over earlier pairs of (T + 2) * pitch
};

// Per state (idx01): the arcs entering it.  w[d] = score of the arc from state s - d
// (-inf: no such arc); label = their common label (kNoLabel: no entering arc).
struct __align__(16) BandState {
  float w[3];
  int32_t label;
};
// Per (state, d): exp(w[d]) = f * 2^k and the arc's index (idx012), -1 if absent.
struct __align__(16) BandArc {
  double f;
  int32_t k;
  int32_t arc;
};
// Entry of a level's list of surviving states.
struct __align__(16) BandItem {
  double pm;        // exp(dense score of the state on the frame before) = pm * 2^pe
  int32_t pe;
  uint8_t inb;      // bit d: the arc from state s - d of the level before survives
  uint8_t outb;     // bit d: the arc to state s + d of the next level survives
  uint16_t s;       // state
};
static_assert(sizeof(BandItem) == 16, "BandItem must be 16 bytes");

// ---------------------------------------------------------------------------
// Tables of a band graph, and the check that it is one.  One thread per state.
// status bit 0 is set when some graph is not a band graph.
// ---------------------------------------------------------------------------
__global__ void BandTables(const int32_t *__restrict__ row_splits1, int32_t num_fsas,
                           const int32_t *__restrict__ row_splits2, const Arc *__restrict__ arcs,
                           int32_t num_states, BandState *__restrict__ tab,
                           BandArc *__restrict__ tabf, int32_t *__restrict__ status) {
  const int32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= num_states) return;
  int32_t lo = 0, hi = num_fsas;  // row_splits1[lo] <= idx < row_splits1[hi]
  while (lo + 1 < hi) {
    const int32_t mid = (lo + hi) >> 1;
    if (row_splits1[mid] <= idx) lo = mid; else hi = mid;
  }
  const int32_t s = idx - row_splits1[lo];
  bool bad = false;
  {  // the arcs leaving this state: at most three, to s, s + 1, s + 2, no destination twice
    const int32_t a0 = row_splits2[idx], a1 = row_splits2[idx + 1];
    bad = a1 - a0 > 3;
    uint32_t seen = 0;
    for (int32_t k = a0; k < a1 && k < a0 + 3; ++k) {
      const Arc arc = arcs[k];
      const int32_t d = arc.dest - arc.src;
      if (arc.src != s || d < 0 || d > 2 || (seen >> d) & 1u) bad = true;
      else seen |= 1u << d;
    }
  }
  BandState st;
  st.label = kNoLabel;
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    st.w[d] = -INFINITY;
    BandArc fa;
    fa.f = 0.0;
    fa.k = kZeroExp;
    fa.arc = -1;
    if (s - d >= 0) {
      const int32_t a0 = row_splits2[idx - d], a1 = min(row_splits2[idx - d + 1], a0 + 3);
      for (int32_t k = a0; k < a1; ++k) {
        const Arc arc = arcs[k];
        if (arc.dest != s || fa.arc >= 0) continue;
        st.w[d] = arc.score;
        fa.arc = k;
        ExpToMantExp(arc.score, &fa.f, &fa.k);
        if (st.label == kNoLabel) st.label = arc.label;
        else if (st.label != arc.label) bad = true;
      }
    }
    tabf[(int64_t)idx * 3 + d] = fa;
  }
  tab[idx] = st;
  if (bad) atomicOr(status, 1);
}

// ---------------------------------------------------------------------------
// Viterbi forward / backward.  grid = (2 directions, pairs), one warp per CTA.
// Level l (0 .. T + 1) of the forward grid: best score of any path from the start state
// at level 0 to the state at level l; of the backward grid: from the state at level l to
// the final state at level T + 1.  The step between levels l and l + 1 consumes dense row l
// (row T being the implied final row).
// ---------------------------------------------------------------------------
template <int K>
__device__ __forceinline__ void StoreRow(float *__restrict__ row, int32_t s0, int32_t pitch,
                                         const float (&v)[K]) {
#pragma unroll
  for (int c = 0; c < K / 4; ++c)
    if (s0 + 4 * c < pitch)
      *reinterpret_cast<float4 *>(row + s0 + 4 * c) =
          make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
}

template <int K>
__device__ __forceinline__ void LoadRow(const float *__restrict__ row, int32_t s0, int32_t pitch,
                                        float (&v)[K]) {
#pragma unroll
  for (int c = 0; c < K / 4; ++c) {
    float4 x = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    if (s0 + 4 * c < pitch) x = *reinterpret_cast<const float4 *>(row + s0 + 4 * c);
    v[4 * c] = x.x;
    v[4 * c + 1] = x.y;
    v[4 * c + 2] = x.z;
    v[4 * c + 3] = x.w;
  }
}

__device__ __forceinline__ float Max3(float a, float b, float c) { return fmaxf(fmaxf(a, b), c); }

// Polls an mbarrier at most `limit` times.
__device__ __forceinline__ bool WaitSlot(uint64_t *bar, unsigned parity, int32_t limit) {
  for (int32_t k = 0; k < limit; ++k)
    if (MbarTryWait(bar, parity)) return true;
  return false;
}

template <int K>
__global__ void __launch_bounds__(32)
BandViterbi(const BandInfo *__restrict__ infos, const BandState *__restrict__ tab,
            const float *__restrict__ lp, int32_t C, float *__restrict__ vf,
            float *__restrict__ vb, int32_t depth, int32_t slot_floats, int32_t wait_limit,
            int32_t *__restrict__ status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full[kBandMaxDepth];
  constexpr unsigned kAll = 0xffffffffu;
  const int dir = blockIdx.x;
  const BandInfo f = infos[blockIdx.y];
  const int lane = threadIdx.x;
  const int32_t S = f.num_states, T = f.frames, pitch = f.pitch;
  if (S == 0) return;
  float *ring = reinterpret_cast<float *>(smem_raw);  // [depth][slot_floats]
  // a slot: four floats of -inf (what a state without a usable label reads), then the row
  for (int32_t k = lane; k < depth * 4; k += 32) ring[(k >> 2) * slot_floats + (k & 3)] = -INFINITY;
  if (lane == 0) {
    for (int st = 0; st < depth; ++st) MbarInit(&full[st], 1);
    MbarInitFence();
  }
  __syncwarp();
  const unsigned row_bytes = 4u * (unsigned)C;
  const float *lp0 = lp + (int64_t)f.lp_row * C;
  // rows in the order this direction consumes them: i = 0 .. T - 1
  int32_t issued = 0;
  auto issue = [&](int32_t i) {  // lane 0 only
    if (i >= T) return;
    const int32_t row = dir == 0 ? i : T - 1 - i;
    const int32_t slot = i % depth;
    MbarArriveExpectTx(&full[slot], row_bytes);
    BulkCopyG2S(ring + (size_t)slot * slot_floats + 4, lp0 + (int64_t)row * C, row_bytes,
                &full[slot]);
    issued = i + 1;
  };
  if (lane == 0)
    for (int32_t i = 0; i < depth; ++i) issue(i);

  const int32_t s0 = lane * K;
  float *grid = (dir == 0 ? vf : vb) + f.grid_off;
  bool late = false;
  float v[K];
  if (dir == 0) {
    // ---- forward: state s from s, s - 1, s - 2 ----------------------------------
    float w0[K], w1[K], w2[K];
    int32_t col[K];
    uint32_t fin = 0;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int32_t s = s0 + k;
      w0[k] = w1[k] = w2[k] = -INFINITY;
      col[k] = 0;
      if (s < S) {
        const BandState t = tab[f.state_off + s];
        w0[k] = t.w[0];
        w1[k] = t.w[1];
        w2[k] = t.w[2];
        if (t.label >= 0 && t.label < C) col[k] = 4 + t.label;
        if (t.label == -1) fin |= 1u << k;
      }
      v[k] = s == 0 ? 0.0f : -INFINITY;
    }
    StoreRow<K>(grid, s0, pitch, v);
    for (int32_t l = 1; l <= T + 1; ++l) {
      const int32_t i = l - 1;  // dense row
      float x[K];
      if (l <= T) {
        const int32_t slot = i % depth;
        if (!late) late = !WaitSlot(&full[slot], (unsigned)(i / depth) & 1u, wait_limit);
        const float *rowbuf = ring + (size_t)slot * slot_floats;
#pragma unroll
        for (int k = 0; k < K; ++k) x[k] = rowbuf[col[k]];
      } else {
#pragma unroll
        for (int k = 0; k < K; ++k) x[k] = (fin >> k) & 1u ? 0.0f : -INFINITY;
      }
      float h1 = __shfl_up_sync(kAll, v[K - 1], 1), h2 = __shfl_up_sync(kAll, v[K - 2], 1);
      if (lane == 0) h1 = h2 = -INFINITY;
      float nv[K];
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const float a = v[k];
        const float b = k >= 1 ? v[k - 1] : h1;
        const float c = k >= 2 ? v[k - 2] : (k == 1 ? h1 : h2);
        const float m = Max3(__fadd_rn(a, w0[k]), __fadd_rn(b, w1[k]), __fadd_rn(c, w2[k]));
        nv[k] = __fadd_rn(m, x[k]);
      }
      __syncwarp();  // every lane has read its scores of this row
      if (lane == 0 && !late) issue(i + depth);
#pragma unroll
      for (int k = 0; k < K; ++k) v[k] = nv[k];
      StoreRow<K>(grid + (int64_t)l * pitch, s0, pitch, v);
    }
  } else {
    // ---- backward: state s to s, s + 1, s + 2 -----------------------------------
    float wo[K][3];       // score of the arc s -> s + d
    int32_t col[K + 2];   // of states s0 .. s0 + K + 1
    uint32_t fin = 0;
#pragma unroll
    for (int k = 0; k < K + 2; ++k) {
      const int32_t s = s0 + k;
      col[k] = 0;
      BandState t;
      t.w[0] = t.w[1] = t.w[2] = -INFINITY;
      t.label = kNoLabel;
      if (s < S) t = tab[f.state_off + s];
      if (t.label >= 0 && t.label < C) col[k] = 4 + t.label;
      if (t.label == -1) fin |= 1u << k;
#pragma unroll
      for (int d = 0; d < 3; ++d)
        if (k - d >= 0 && k - d < K) wo[k - d][d] = t.w[d];
    }
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = (s0 + k == S - 1) ? 0.0f : -INFINITY;
    StoreRow<K>(grid + (int64_t)(T + 1) * pitch, s0, pitch, v);
    for (int32_t l = T; l >= 0; --l) {  // level l from level l + 1 through dense row l
      const int32_t i = T - 1 - l;      // order of consumption (-1: the implied final row)
      float x[K + 2];
      if (l < T) {
        const int32_t slot = i % depth;
        if (!late) late = !WaitSlot(&full[slot], (unsigned)(i / depth) & 1u, wait_limit);
        const float *rowbuf = ring + (size_t)slot * slot_floats;
#pragma unroll
        for (int k = 0; k < K + 2; ++k) x[k] = rowbuf[col[k]];
      } else {
#pragma unroll
        for (int k = 0; k < K + 2; ++k) x[k] = (fin >> k) & 1u ? 0.0f : -INFINITY;
      }
      float g1 = __shfl_down_sync(kAll, v[0], 1), g2 = __shfl_down_sync(kAll, v[1], 1);
      if (lane == 31) g1 = g2 = -INFINITY;
      float nv[K];
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const float a = v[k];
        const float b = k + 1 < K ? v[k + 1] : g1;
        const float c = k + 2 < K ? v[k + 2] : (k + 2 == K ? g1 : g2);
        nv[k] = Max3(__fadd_rn(__fadd_rn(a, wo[k][0]), x[k]),
                     __fadd_rn(__fadd_rn(b, wo[k][1]), x[k + 1]),
                     __fadd_rn(__fadd_rn(c, wo[k][2]), x[k + 2]));
      }
      __syncwarp();
      if (lane == 0 && !late && l < T) issue(i + depth);
#pragma unroll
      for (int k = 0; k < K; ++k) v[k] = nv[k];
      StoreRow<K>(grid + (int64_t)l * pitch, s0, pitch, v);
    }
  }
  if (__any_sync(kAll, late)) {
    // A copy did not arrive in time: the grids hold garbage.  Say so, and let the copies
    // that are still in flight towards this CTA's shared memory land before it retires.
    if (lane == 0) {
      atomicOr(status, 2);
      for (int32_t i = max(0, issued - depth); i < issued; ++i)
        WaitSlot(&full[i % depth], (unsigned)(i / depth) & 1u, kDrainPolls);
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------
// Keep tests and the per-level lists.  grid = (level chunks, pairs), a warp per chunk of
// kPrepLevels levels; lane owns K consecutive states as in BandViterbi.  A warp writes the
// complete entries of the levels it owns, for which it also needs the surviving arcs into
// the level after its last (recomputed from one more row of each grid).
// totals[0] += surviving states, totals[2] += the arcs leaving them (the sizes the beam
// reduction looks at, intersect_dense.cu:289-320).
// ---------------------------------------------------------------------------
template <int K>
__global__ void __launch_bounds__(128)
BandPrep(const BandInfo *__restrict__ infos, const BandState *__restrict__ tab,
         const int32_t *__restrict__ a_row_splits2, const float *__restrict__ lp, int32_t C,
         const float *__restrict__ vf, const float *__restrict__ vb, float beam,
         BandItem *__restrict__ items, int32_t *__restrict__ counts,
         float *__restrict__ cutoffs, unsigned long long *__restrict__ totals) {
  constexpr unsigned kAll = 0xffffffffu;
  const int32_t i = blockIdx.y;
  const BandInfo f = infos[i];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int32_t S = f.num_states, T = f.frames, pitch = f.pitch;
  if (S == 0) return;
  const int32_t a = (blockIdx.x * 4 + warp) * kPrepLevels;  // owns levels a .. b - 1
  if (a > T + 1) return;
  const int32_t b = min(a + kPrepLevels, T + 2);
  const float *fg = vf + f.grid_off, *bg = vb + f.grid_off;
  float cutoff;
  {
    const float start = bg[0], end = fg[(int64_t)(T + 1) * pitch + (S - 1)];
    cutoff = __fsub_rn(start < end ? start : end, beam);
  }
  if (a == 0 && lane == 0) cutoffs[i] = cutoff;
  const int32_t s0 = lane * K;
  float w[K][3];
  int32_t label[K];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    BandState t;
    t.w[0] = t.w[1] = t.w[2] = -INFINITY;
    t.label = kNoLabel;
    if (s0 + k < S) t = tab[f.state_off + s0 + k];
    w[k][0] = t.w[0];
    w[k][1] = t.w[1];
    w[k][2] = t.w[2];
    label[k] = t.label;
  }
  const float *lp0 = lp + (int64_t)f.lp_row * C;
  float Fp[K], Bp[K];
  uint32_t keep_p = 0;
#pragma unroll
  for (int k = 0; k < K; ++k) Fp[k] = Bp[k] = -INFINITY;
  if (a >= 1) {
    LoadRow<K>(fg + (int64_t)(a - 1) * pitch, s0, pitch, Fp);
    LoadRow<K>(bg + (int64_t)(a - 1) * pitch, s0, pitch, Bp);
#pragma unroll
    for (int k = 0; k < K; ++k)
      if (__fadd_rn(Fp[k], Bp[k]) > cutoff) keep_p |= 1u << k;
  }
  int32_t base_p = 0;  // list position of this lane's first surviving state, level before
  uint32_t n_states = 0, n_cand = 0;
  for (int32_t l = a; l <= b && l <= T + 1; ++l) {
    const bool own = l < b;
    float Fc[K], Bc[K];
    LoadRow<K>(fg + (int64_t)l * pitch, s0, pitch, Fc);
    LoadRow<K>(bg + (int64_t)l * pitch, s0, pitch, Bc);
    uint32_t keep_c = 0;
#pragma unroll
    for (int k = 0; k < K; ++k)
      if (__fadd_rn(Fc[k], Bc[k]) > cutoff) keep_c |= 1u << k;
    const uint32_t lanes_c = __ballot_sync(kAll, keep_c != 0);
    // position of this lane's survivors in the level's list
    int32_t cnt = __popc(keep_c), incl = cnt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t o = __shfl_up_sync(kAll, incl, d);
      if (lane >= d) incl += o;
    }
    const int32_t base_c = incl - cnt;
    const int32_t n_c = __shfl_sync(kAll, incl, 31);
    // the two states before this lane's first, from the previous lane
    float hF1 = __shfl_up_sync(kAll, Fp[K - 1], 1), hF2 = __shfl_up_sync(kAll, Fp[K - 2], 1);
    uint32_t hk = __shfl_up_sync(kAll, keep_p, 1);
    if (lane == 0) {
      hF1 = hF2 = -INFINITY;
      hk = 0;
    }
    uint32_t inb[K];
    BandItem *out = items + f.grid_off + (int64_t)l * pitch;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      inb[k] = 0;
      if (!((keep_c >> k) & 1u)) continue;
      float x = -INFINITY;
      if (l >= 1) {
        const int32_t row = l - 1;
        if (row < T) {
          if (label[k] >= 0 && label[k] < C) x = __ldg(lp0 + (int64_t)row * C + label[k]);
        } else if (label[k] == -1) {
          x = 0.0f;
        }
#pragma unroll
        for (int d = 0; d < 3; ++d) {
          const float srcF = k - d >= 0 ? Fp[k - d > 0 ? k - d : 0] : (k - d == -1 ? hF1 : hF2);
          const bool kept = k - d >= 0 ? (keep_p >> (k - d > 0 ? k - d : 0)) & 1u
                                       : (hk >> (K + k - d)) & 1u;
          const float sc = __fadd_rn(w[k][d], x);
          const float through = __fadd_rn(__fadd_rn(srcF, sc), Bc[k]);
          if (kept && through > cutoff) inb[k] |= 1u << d;
        }
      }
      if (own) {
        BandItem it;
        ExpToMantExp(x, &it.pm, &it.pe);
        it.inb = (uint8_t)inb[k];
        it.outb = 0;
        it.s = (uint16_t)(s0 + k);
        out[base_c + __popc(keep_c & ((1u << k) - 1u))] = it;
        ++n_states;
        const int32_t idx = f.state_off + s0 + k;
        n_cand += a_row_splits2[idx + 1] - a_row_splits2[idx];
      }
    }
    if (own && lane == 0) counts[f.level_off + l] = n_c;
    // arcs leaving the states of level l - 1 (owned when l - 1 >= a): bit d of state s is
    // bit d of the entering arcs of state s + d on this level
    if (l - 1 >= a && __any_sync(kAll, keep_p != 0) && lanes_c != 0) {
      uint32_t n1 = __shfl_down_sync(kAll, inb[0], 1), n2 = __shfl_down_sync(kAll, inb[1], 1);
      if (lane == 31) n1 = n2 = 0;
      unsigned char *prev_bytes =
          reinterpret_cast<unsigned char *>(items + f.grid_off + (int64_t)(l - 1) * pitch);
#pragma unroll
      for (int k = 0; k < K; ++k) {
        if (!((keep_p >> k) & 1u)) continue;
        const uint32_t i1 = k + 1 < K ? inb[k + 1 < K ? k + 1 : 0] : n1;
        const uint32_t i2 = k + 2 < K ? inb[k + 2 < K ? k + 2 : 0] : (k + 2 == K ? n1 : n2);
        const uint32_t ob = (inb[k] & 1u) | (i1 & 2u) | (i2 & 4u);
        if (ob)
          prev_bytes[(size_t)(base_p + __popc(keep_p & ((1u << k) - 1u))) * sizeof(BandItem) + 13] =
              (unsigned char)ob;
      }
    }
#pragma unroll
    for (int k = 0; k < K; ++k) {
      Fp[k] = Fc[k];
      Bp[k] = Bc[k];
    }
    keep_p = keep_c;
    base_p = base_c;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    n_states += __shfl_xor_sync(kAll, n_states, d);
    n_cand += __shfl_xor_sync(kAll, n_cand, d);
  }
  if (lane == 0 && (n_states | n_cand)) {
    atomicAdd(&totals[0], (unsigned long long)n_states);
    atomicAdd(&totals[2], (unsigned long long)n_cand);
  }
}

// ---------------------------------------------------------------------------
// alpha (dir 0) and beta (dir 1) over the lists.  grid = (2, pairs), one warp per CTA.
//   alpha_0[start] = 1;  alpha_l[s] = p_l[s] * sum_d [arc s-d -> s survives] e^w alpha_{l-1}[s-d]
//   beta_{T+1}[final] = 1;  beta_l[s] = sum_d [arc s -> s+d survives] e^w p_{l+1}[s+d] beta_{l+1}[s+d]
// Values are m * 2^e with m in [1, 2) or 0.  Shared memory holds, by state number, the
// values of the previous level (for beta: already multiplied by p) in two buffers used in
// turn; an entry of the buffer read is current whenever the arc bit that selects it is set.
// Outputs: alpha / beta (mantissas and exponents) at the list positions, tot[i].
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(32)
BandChain(const BandInfo *__restrict__ infos, const BandArc *__restrict__ tabf,
          const BandItem *__restrict__ items, const int32_t *__restrict__ counts,
          double *__restrict__ am, int32_t *__restrict__ ae, double *__restrict__ bm,
          int32_t *__restrict__ be, double *__restrict__ tot, const int32_t *__restrict__ status,
          int32_t st_pad, int32_t lv_pad) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int dir = blockIdx.x;
  const int32_t i = blockIdx.y;
  const BandInfo f = infos[i];
  const int lane = threadIdx.x;
  const int32_t S = f.num_states, T = f.frames, pitch = f.pitch, L = T + 2;
  if (dir == 0 && lane == 0) tot[i] = -INFINITY;
  if (S == 0) return;
  ProbState *st = reinterpret_cast<ProbState *>(smem_raw);            // [2][st_pad], state s at s + 2
  BandArc *af = reinterpret_cast<BandArc *>(st + 2 * st_pad);         // [st_pad][3]
  BandItem *ring = reinterpret_cast<BandItem *>(af + 3 * st_pad);     // [kChainAhead][kRingItems]
  int32_t *cnt = reinterpret_cast<int32_t *>(ring + kChainAhead * kRingItems);  // [lv_pad]
  for (int32_t l = lane; l < L; l += 32) cnt[l] = counts[f.level_off + l];
  for (int32_t k = lane; k < 3 * st_pad; k += 32) {
    BandArc z;
    z.f = 0.0;
    z.k = kZeroExp;
    z.arc = -1;
    af[k] = k < 3 * S ? tabf[(int64_t)f.state_off * 3 + k] : z;
  }
  for (int32_t k = lane; k < 2 * st_pad; k += 32) {
    ProbState z;
    z.m = 0.0;
    z.e = kZeroExp;
    z.pad = 0;
    st[k] = z;
  }
  __syncwarp();
  const BandItem *items0 = items + f.grid_off;
  auto level_of = [&](int32_t step) { return dir == 0 ? step : L - 1 - step; };
  auto prefetch = [&](int32_t step) {
    if (step < L) {
      const int32_t l = level_of(step);
      const int32_t n = min(cnt[l], kRingItems);
      const BandItem *src = items0 + (int64_t)l * pitch;
      BandItem *dst = ring + (step % kChainAhead) * kRingItems;
      for (int32_t j = lane; j < n; j += 32) CpAsync16(dst + j, src + j);
    }
    CpAsyncCommit();
  };
  for (int32_t step = 0; step < kChainAhead - 1; ++step) prefetch(step);
  double *om = (dir == 0 ? am : bm) + f.grid_off;
  int32_t *oe = (dir == 0 ? ae : be) + f.grid_off;
  for (int32_t step = 0; step < L; ++step) {
    prefetch(step + kChainAhead - 1);
    CpAsyncWait<kChainAhead - 1>();
    const int32_t l = level_of(step);
    const int32_t n = cnt[l];
    ProbState *cur = st + (step & 1) * st_pad + 2;
    const ProbState *prv = st + ((step & 1) ^ 1) * st_pad + 2;
    const BandItem *slot = ring + (step % kChainAhead) * kRingItems;
    const int64_t row = (int64_t)l * pitch;
    for (int32_t j0 = 0; j0 < n; j0 += 32) {
      const int32_t j = j0 + lane;
      if (j < n) {
        const BandItem it = j < kRingItems ? slot[j] : items0[row + j];
        const int32_t s = it.s;
        double m;
        int32_t e;
        if (step == 0) {
          const bool one = s == (dir == 0 ? 0 : S - 1);
          m = one ? 1.0 : 0.0;
          e = one ? 0 : kZeroExp;
        } else {
          const uint32_t bits = dir == 0 ? it.inb : it.outb;
          double t[3];
          int32_t x[3];
#pragma unroll
          for (int d = 0; d < 3; ++d) {
            const ProbState q = dir == 0 ? prv[s - d] : prv[s + d];
            const BandArc arc = dir == 0 ? af[3 * s + d] : af[3 * (s + d) + d];
            double td = q.m * arc.f;
            td = (bits >> d) & 1u ? td : 0.0;
            t[d] = td;
            x[d] = td != 0.0 ? q.e + arc.k : kZeroExp;
          }
          const int32_t E = max(x[0], max(x[1], x[2]));
          const double sum =
              ScaleDown(t[0], x[0] - E) + ScaleDown(t[1], x[1] - E) + ScaleDown(t[2], x[2] - E);
          e = E;
          if (dir == 0) {
            e += it.pe;
            m = Renorm(sum * it.pm, &e);
          } else {
            m = Renorm(sum, &e);
          }
        }
        om[row + j] = m;
        oe[row + j] = e;
        ProbState r;
        r.pad = 0;
        if (dir == 0) {
          r.m = m;
          r.e = e;
          if (l == T + 1 && s == S - 1)
            tot[i] = m == 0.0 ? -INFINITY : log(m) + (double)e * 0.69314718055994530942;
        } else {  // what the level below adds: beta * p
          r.e = e + it.pe;
          r.m = Renorm(m * it.pm, &r.e);
        }
        cur[s] = r;
      }
    }
    __syncwarp();
  }
  CpAsyncWait<0>();
  if (dir == 0 && lane == 0 && *status != 0) tot[i] = nan("");
}

// ---------------------------------------------------------------------------
// Gradients.  grid = (level chunks, pairs), a warp per chunk of kGradLevels levels.
// posterior(l, s) = alpha_l[s] * beta_l[s] / Z is dL/d(dense score of state s's label on
// frame l - 1) up to dL/dtot; it is ADDED to grad_b[(grad_row0[i] + l - 1) * grad_pitch +
// label + grad_col_off] (skipped when label + grad_col_off < 0: the final symbol has no
// column in the log-prob layout).  With kArcs the posterior of every surviving arc,
// alpha_{l-1}[src] e^w p_l[dest] beta_l[dest] / Z, is added to grad_a[arc]; the warp keeps
// alpha of the level before by state number in shared memory for that.
// ---------------------------------------------------------------------------
__device__ __forceinline__ double Pow2Clamp(int32_t e) {
  if (e < -1000) return 0.0;
  e = e > 1000 ? 1000 : e;
  return __longlong_as_double((long long)(1023 + e) << 52);
}

template <bool kArcs>
__global__ void __launch_bounds__(128)
BandGrad(const BandInfo *__restrict__ infos, const BandState *__restrict__ tab,
         const BandArc *__restrict__ tabf, const BandItem *__restrict__ items,
         const int32_t *__restrict__ counts, const double *__restrict__ am,
         const int32_t *__restrict__ ae, const double *__restrict__ bm,
         const int32_t *__restrict__ be, const double *__restrict__ tot_grad,
         int32_t tot_grad_stride, float *__restrict__ grad_a, float *__restrict__ grad_b,
         const int32_t *__restrict__ grad_row0, int32_t grad_pitch, int32_t grad_col_off,
         int32_t C, int32_t st_pad, int32_t exclusive_rows) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr unsigned kAll = 0xffffffffu;
  const int32_t i = blockIdx.y;
  const BandInfo f = infos[i];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int32_t S = f.num_states, T = f.frames, pitch = f.pitch;
  if (S == 0) return;
  const int32_t a = 1 + (blockIdx.x * 4 + warp) * kGradLevels;  // levels a .. b - 1
  if (a > T + 1) return;
  const int32_t b = min(a + kGradLevels, T + 2);
  const int32_t *cnt = counts + f.level_off;
  const BandItem *items0 = items + f.grid_off;
  const double *am0 = am + f.grid_off, *bm0 = bm + f.grid_off;
  const int32_t *ae0 = ae + f.grid_off, *be0 = be + f.grid_off;
  // Z = alpha of the final state on the last level: the last entry of that level's list
  const int32_t n_last = cnt[T + 1];
  if (n_last == 0) return;
  const int64_t zpos = (int64_t)(T + 1) * pitch + n_last - 1;
  if (items0[zpos].s != S - 1) return;
  const double zm = am0[zpos];
  if (zm == 0.0) return;
  const double zinv = 1.0 / zm;
  const int32_t ze = ae0[zpos];
  const double tg = tot_grad[(int64_t)i * tot_grad_stride];
  const int64_t row0 = grad_row0[i];
  ProbState *prev = nullptr;  // alpha of the level before, state s at s + 2
  if (kArcs) {
    prev = reinterpret_cast<ProbState *>(smem_raw) + (size_t)warp * st_pad + 2;
    const int32_t l = a - 1, n = cnt[l];
    for (int32_t j = lane; j < n; j += 32) {
      ProbState q;
      q.m = am0[(int64_t)l * pitch + j];
      q.e = ae0[(int64_t)l * pitch + j];
      q.pad = 0;
      prev[items0[(int64_t)l * pitch + j].s] = q;
    }
    __syncwarp();
  }
  for (int32_t l = a; l < b; ++l) {
    const int32_t n = cnt[l];
    const int64_t row = (int64_t)l * pitch;
    for (int32_t j0 = 0; j0 < n; j0 += 32) {
      const int32_t j = j0 + lane;
      float g = 0.0f;
      int32_t key = -1 - lane;  // lanes with nothing to add are groups of their own
      if (j < n) {
        const BandItem it = items0[row + j];
        const double alm = am0[row + j], bem = bm0[row + j];
        if (alm != 0.0 && bem != 0.0) {
          const int32_t ale = ae0[row + j], bee = be0[row + j];
          const int32_t s = it.s;
          const int32_t label = tab[f.state_off + s].label;
          const int32_t col = label + grad_col_off;
          if (label != kNoLabel && label < C && col >= 0) {
            const double post = alm * bem * zinv * Pow2Clamp(ale + bee - ze);
            g = (float)(tg * post);
            key = col;
          }
          if (kArcs) {
#pragma unroll
            for (int d = 0; d < 3; ++d) {
              if (!((it.inb >> d) & 1u)) continue;
              const ProbState q = prev[s - d];
              const BandArc arc = tabf[(int64_t)(f.state_off + s) * 3 + d];
              // two steps, so that no intermediate product leaves the range of a double
              const double post = (q.m * arc.f * it.pm) * (bem * zinv) *
                                  Pow2Clamp(q.e + arc.k + it.pe + bee - ze);
              if (post != 0.0) atomicAdd(grad_a + arc.arc, (float)(tg * post));
            }
          }
        }
      }
      // States with the same label (the blank states of a CTC graph) add to the same
      // element: their lanes are summed in lane order and one of them writes, so the
      // dense gradient does not depend on the order in which atomics would land.
      const uint32_t grp = __match_any_sync(kAll, key);
      const int32_t members = __popc(grp);
      const int32_t rounds = __reduce_max_sync(kAll, key >= 0 ? members : 0);
      float sum = 0.0f;
      for (int32_t r = 0; r < rounds; ++r) {
        const uint32_t src = __fns(grp, 0, r + 1);
        const float v = __shfl_sync(kAll, g, (int)(src & 31u));
        if (r < members) sum += v;
      }
      if (key >= 0 && lane == __ffs(grp) - 1) {
        float *p = grad_b + (row0 + l - 1) * grad_pitch + key;
        if (exclusive_rows) *p += sum; else atomicAdd(p, sum);
      }
      __syncwarp();  // a later part of the level may add to the same elements
    }
    if (kArcs) {
      __syncwarp();  // the level before has been read
      for (int32_t j = lane; j < n; j += 32) {
        ProbState q;
        q.m = am0[row + j];
        q.e = ae0[row + j];
        q.pad = 0;
        prev[items0[row + j].s] = q;
      }
      __syncwarp();
    }
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
struct BandLayout {
  std::vector<BandInfo> infos;
  int64_t grid_elems = 0, levels = 0;
  long long arc_frames = 0;
  int32_t max_states = 0, max_frames = 0;
  int K = 4;
  int32_t depth = 0, slot_floats = 0, st_pad = 0, lv_pad = 0;
  size_t chain_smem = 0, viterbi_smem = 0;
  size_t off_infos, off_vf, off_vb, off_items, off_counts, off_cutoffs, off_am, off_ae, off_bm,
      off_be, off_totals, off_status, total_bytes;  // off_status = off_totals + 40
  bool ok = true;
  const char *why = "";
  bool exclusive_rows = true;  // no two graphs on one sequence (they would share gradient rows)
};

constexpr size_t kBandSmemBudget = 200 * 1024;

static int32_t MakeBandLayout(const k2b200_band_loss_args *a, BandLayout *L) {
  K2B_REQUIRE(a != nullptr, "args is NULL");
  K2B_REQUIRE(a->num_fsas > 0, "a_fsas must contain at least one FSA (got %d)", a->num_fsas);
  K2B_REQUIRE(a->output_beam > 0, "output_beam must be > 0 (got %f)", a->output_beam);
  K2B_REQUIRE(a->h_a_row_splits1 && a->h_a_arc_splits && a->h_first_row && a->h_frames,
              "host arrays of the batch description are required");
  K2B_REQUIRE(a->num_classes > 0, "empty log-prob matrix");
  L->infos.resize(a->num_fsas);
  int64_t grid = 0, levels = 0;
  for (int32_t i = 0; i < a->num_fsas; ++i) {
    BandInfo &f = L->infos[i];
    f.state_off = a->h_a_row_splits1[i];
    f.num_states = a->h_a_row_splits1[i + 1] - f.state_off;
    f.pitch = (f.num_states + 3) & ~3;
    f.frames = a->h_frames[i];
    K2B_REQUIRE(f.frames >= 0, "sequence of graph %d has a negative number of frames", i);
    if (i > 0)
      K2B_REQUIRE(f.frames <= a->h_frames[i - 1],
                  "Sequences (DenseFsaVec) must be in sorted order from greatest to least "
                  "length; graph %d has %d frames after %d",
                  i, f.frames, a->h_frames[i - 1]);
    f.lp_row = a->h_first_row[i];
    K2B_REQUIRE(f.lp_row >= 0 && (int64_t)f.lp_row + f.frames <= a->log_prob_rows,
                "frames of graph %d lie outside the log-prob matrix", i);
    if (i > 0 && f.lp_row == a->h_first_row[i - 1]) L->exclusive_rows = false;
    f.level_off = (int32_t)levels;
    f.grid_off = grid;
    grid += (int64_t)(f.frames + 2) * f.pitch;
    levels += f.frames + 2;
    L->max_states = std::max(L->max_states, f.num_states);
    L->max_frames = std::max(L->max_frames, f.frames);
    L->arc_frames += (long long)(f.frames + 1) *
                     (a->h_a_arc_splits[i + 1] - a->h_a_arc_splits[i]);
  }
  if (levels >= ((int64_t)1 << 31)) {
    SetError("problem too large: %lld (fsa, frame) levels", (long long)levels);
    return kTooLarge;
  }
  L->grid_elems = grid;
  L->levels = levels;
  L->K = L->max_states <= 128 ? 4 : (L->max_states <= 256 ? 8 : 16);
  // shared memory of the kernels
  L->slot_floats = 4 + ((a->num_classes + 3) & ~3);
  const size_t slot_bytes = sizeof(float) * (size_t)L->slot_floats;
  L->depth = (int32_t)std::min<size_t>(kBandMaxDepth, kBandSmemBudget / slot_bytes);
  L->viterbi_smem = slot_bytes * (size_t)std::max(L->depth, 1);
  L->st_pad = ((L->max_states + 4) + 3) & ~3;
  L->lv_pad = (L->max_frames + 2 + 3) & ~3;
  L->chain_smem = sizeof(ProbState) * 2 * (size_t)L->st_pad + sizeof(BandArc) * 3 * (size_t)L->st_pad +
                  sizeof(BandItem) * kChainAhead * kRingItems + sizeof(int32_t) * (size_t)L->lv_pad;
  if (L->max_states > kBandMaxStates) {
    L->ok = false;
    L->why = "a graph has more than 512 states";
  } else if (a->num_classes % 4 != 0 || (reinterpret_cast<uintptr_t>(a->log_probs) & 15) != 0) {
    L->ok = false;
    L->why = "rows of the log-prob matrix are not 16-byte aligned";
  } else if (L->depth < 2) {
    L->ok = false;
    L->why = "too many classes for the row ring";
  } else if (L->chain_smem > kBandSmemBudget) {
    L->ok = false;
    L->why = "too many frames for the level table in shared memory";
  } else if (a->num_fsas > 65535) {
    L->ok = false;
    L->why = "more than 65535 graphs";
  }
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off += AlignUp(bytes ? bytes : 1);
    return o;
  };
  L->off_infos = take(sizeof(BandInfo) * a->num_fsas);
  L->off_vf = take(sizeof(float) * (size_t)grid);
  L->off_vb = take(sizeof(float) * (size_t)grid);
  L->off_items = take(sizeof(BandItem) * (size_t)grid);
  L->off_counts = take(sizeof(int32_t) * (size_t)levels);
  L->off_cutoffs = take(sizeof(float) * a->num_fsas);
  L->off_am = take(sizeof(double) * (size_t)grid);
  L->off_ae = take(sizeof(int32_t) * (size_t)grid);
  L->off_bm = take(sizeof(double) * (size_t)grid);
  L->off_be = take(sizeof(int32_t) * (size_t)grid);
  L->off_totals = take(64);  // five 64-bit totals, then the status word
  L->off_status = L->off_totals + 5 * sizeof(long long);
  L->total_bytes = off;
  return kOk;
}

template <int K>
static int32_t LaunchBandViterbi(const BandLayout &L, const k2b200_band_loss_args *a, char *ws,
                                 cudaStream_t stream) {
  K2B_CUDA_OK(cudaFuncSetAttribute(BandViterbi<K>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)L.viterbi_smem));
  dim3 grid(2, a->num_fsas);
  { BandViterbi<K><<<grid, 32, L.viterbi_smem, stream>>>(
      reinterpret_cast<const BandInfo *>(ws + L.off_infos),
      reinterpret_cast<const BandState *>(a->band_states), a->log_probs, a->num_classes,
      reinterpret_cast<float *>(ws + L.off_vf), reinterpret_cast<float *>(ws + L.off_vb), L.depth,
      L.slot_floats, g_wait_limit, reinterpret_cast<int32_t *>(ws + L.off_status)); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

template <int K>
static int32_t LaunchBandPrep(const BandLayout &L, const k2b200_band_loss_args *a, char *ws,
                              float beam, cudaStream_t stream) {
  dim3 grid(CeilDiv(L.max_frames + 2, 4 * kPrepLevels), a->num_fsas);
  { BandPrep<K><<<grid, 128, 0, stream>>>(
      reinterpret_cast<const BandInfo *>(ws + L.off_infos),
      reinterpret_cast<const BandState *>(a->band_states), a->a_row_splits2, a->log_probs,
      a->num_classes, reinterpret_cast<const float *>(ws + L.off_vf),
      reinterpret_cast<const float *>(ws + L.off_vb), beam,
      reinterpret_cast<BandItem *>(ws + L.off_items),
      reinterpret_cast<int32_t *>(ws + L.off_counts),
      reinterpret_cast<float *>(ws + L.off_cutoffs),
      reinterpret_cast<unsigned long long *>(ws + L.off_totals)); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

static bool BandReduceBeam(const k2b200_band_loss_args *a, const long long *h_totals,
                           float *beam) {
  long long limit = 0, total = 0;
  if (h_totals[0] > a->max_states) {
    limit = a->max_states;
    total = h_totals[0];
  } else if (h_totals[2] > a->max_arcs) {
    limit = a->max_arcs;
    total = h_totals[2];
  } else {
    return false;
  }
  // the reference's rule, intersect_dense.cu:854-862
  float cur = *beam, next = cur * sqrt(limit * 1.0 / total);
  if (next < cur * 0.25) next = cur * 0.25;
  if (next > cur * 0.75) next = cur * 0.75;
  *beam = next;
  return true;
}

}  // namespace k2b

using namespace k2b;

extern "C" {

void k2b200_debug_set_copy_wait_limit(int32_t polls) { g_wait_limit = polls < 0 ? 4000000 : polls; }

int32_t k2b200_band_tables_bytes(int32_t num_states, size_t *states_bytes, size_t *arcs_bytes) {
  K2B_REQUIRE(states_bytes && arcs_bytes, "NULL output pointer");
  const size_t n = (size_t)std::max(num_states, 1);
  *states_bytes = sizeof(BandState) * n;
  *arcs_bytes = sizeof(BandArc) * 3 * n;
  return kOk;
}

int32_t k2b200_band_tables(const int32_t *row_splits1, int32_t num_fsas,
                           const int32_t *row_splits2, const void *arcs, int32_t num_states,
                           void *band_states, void *band_arcs, int32_t *status, void *stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  K2B_REQUIRE(row_splits1 && row_splits2 && band_states && band_arcs && status,
              "NULL device pointer");
  K2B_REQUIRE(num_fsas > 0, "a_fsas must contain at least one FSA (got %d)", num_fsas);
  K2B_CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
  if (num_states > 0)
    { BandTables<<<CeilDiv(num_states, 128), 128, 0, stream>>>(
        row_splits1, num_fsas, row_splits2, reinterpret_cast<const Arc *>(arcs), num_states,
        reinterpret_cast<BandState *>(band_states), reinterpret_cast<BandArc *>(band_arcs),
        status); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t k2b200_band_loss_supported(const k2b200_band_loss_args *args, int32_t *supported) {
  K2B_REQUIRE(supported != nullptr, "NULL output pointer");
  BandLayout L;
  K2B_FORWARD(MakeBandLayout(args, &L));
  *supported = L.ok ? 1 : 0;
  if (!L.ok) SetError("band loss path not applicable: %s", L.why);
  return kOk;
}

int32_t k2b200_band_loss_workspace_bytes(const k2b200_band_loss_args *args, size_t *bytes) {
  K2B_REQUIRE(bytes != nullptr, "NULL output pointer");
  BandLayout L;
  K2B_FORWARD(MakeBandLayout(args, &L));
  *bytes = L.total_bytes;
  return kOk;
}

int32_t k2b200_band_loss_forward(const k2b200_band_loss_args *args, void *workspace,
                                 size_t workspace_bytes, void *stream_v, double *tot_scores,
                                 float *beam_used) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  BandLayout L;
  K2B_FORWARD(MakeBandLayout(args, &L));
  K2B_REQUIRE(L.ok, "band loss path not applicable: %s", L.why);
  if (workspace == nullptr || workspace_bytes < L.total_bytes) {
    SetError("workspace of %zu bytes is smaller than the %zu required", workspace_bytes,
             L.total_bytes);
    return kWorkspaceTooSmall;
  }
  K2B_REQUIRE(args->a_row_splits2 && args->band_states && args->band_arcs && args->log_probs &&
                  tot_scores,
              "NULL device pointer");
  char *ws = reinterpret_cast<char *>(workspace);
  static_assert(sizeof(BandInfo) % sizeof(int32_t) == 0, "BandInfo is uploaded as int32 words");
  K2B_FORWARD(UploadInts(reinterpret_cast<const int32_t *>(L.infos.data()),
                         (int64_t)L.infos.size() * (sizeof(BandInfo) / sizeof(int32_t)),
                         reinterpret_cast<int32_t *>(ws + L.off_infos), stream));
  K2B_CUDA_OK(cudaMemsetAsync(ws + L.off_status, 0, 8, stream));
  {
    PhaseTimer timer(kPhaseViterbi, stream);
    NotePhaseKernel(kPhaseViterbi, "BandViterbi");
    if (L.K == 4) K2B_FORWARD(LaunchBandViterbi<4>(L, args, ws, stream));
    else if (L.K == 8) K2B_FORWARD(LaunchBandViterbi<8>(L, args, ws, stream));
    else K2B_FORWARD(LaunchBandViterbi<16>(L, args, ws, stream));
  }
  // The lattice is never built, but its size still decides the beam
  // (intersect_dense.cu:300-320).  The grid bounds it: the host reads the counts only
  // when that bound does not already satisfy the limits, and after it has launched the
  // recursions, which in the rare case of a reduction run again.
  const bool need_count = L.grid_elems > args->max_states || L.arc_frames > args->max_arcs;
  float beam = args->output_beam;
  K2B_CUDA_OK(cudaFuncSetAttribute(BandChain, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)L.chain_smem));
  for (int iter = 0;; ++iter) {
    K2B_CUDA_OK(cudaMemsetAsync(ws + L.off_totals, 0, 5 * sizeof(long long), stream));
    {
      PhaseTimer timer(kPhasePrune, stream);
      NotePhaseKernel(kPhasePrune, "BandPrep");
      if (L.K == 4) K2B_FORWARD(LaunchBandPrep<4>(L, args, ws, beam, stream));
      else if (L.K == 8) K2B_FORWARD(LaunchBandPrep<8>(L, args, ws, beam, stream));
      else K2B_FORWARD(LaunchBandPrep<16>(L, args, ws, beam, stream));
    }
    cudaStream_t side = nullptr;
    if (need_count) K2B_FORWARD(SideFork(stream, &side));  // behind the counts, before the chain
    {
      PhaseTimer timer(kPhaseChain, stream);
      NotePhaseKernel(kPhaseChain, "BandChain");
      dim3 grid(2, args->num_fsas);
      { BandChain<<<grid, 32, L.chain_smem, stream>>>(
          reinterpret_cast<const BandInfo *>(ws + L.off_infos),
          reinterpret_cast<const BandArc *>(args->band_arcs),
          reinterpret_cast<const BandItem *>(ws + L.off_items),
          reinterpret_cast<const int32_t *>(ws + L.off_counts),
          reinterpret_cast<double *>(ws + L.off_am), reinterpret_cast<int32_t *>(ws + L.off_ae),
          reinterpret_cast<double *>(ws + L.off_bm), reinterpret_cast<int32_t *>(ws + L.off_be),
          tot_scores, reinterpret_cast<const int32_t *>(ws + L.off_status), L.st_pad, L.lv_pad);
        NoteLaunch(); }
      K2B_CUDA_OK(cudaGetLastError());
    }
    if (!need_count) break;
    long long h_totals[6];
    K2B_FORWARD(SideReadBack(ws + L.off_totals, sizeof(h_totals), h_totals));
    K2B_REQUIRE((h_totals[5] & 2) == 0,
                "a copy of log-prob rows into shared memory did not complete in time");
    if (!BandReduceBeam(args, h_totals, &beam)) break;
    K2B_REQUIRE(iter < 200, "output beam reduction did not converge");
  }
  if (beam_used) *beam_used = beam;
  return kOk;
}

int32_t k2b200_band_loss_backward(const k2b200_band_loss_args *args, void *workspace,
                                  size_t workspace_bytes, const double *tot_grad,
                                  int32_t tot_grad_stride, float *grad_a, float *grad_b,
                                  const int32_t *grad_row0, int32_t grad_pitch,
                                  int32_t grad_col_off, void *stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  BandLayout L;
  K2B_FORWARD(MakeBandLayout(args, &L));
  K2B_REQUIRE(L.ok, "band loss path not applicable: %s", L.why);
  if (workspace == nullptr || workspace_bytes < L.total_bytes) {
    SetError("workspace of %zu bytes is smaller than the %zu required", workspace_bytes,
             L.total_bytes);
    return kWorkspaceTooSmall;
  }
  K2B_REQUIRE(tot_grad && grad_b && grad_row0, "NULL device pointer");
  K2B_REQUIRE(grad_col_off == 0 || grad_col_off == 1, "grad_col_off must be 0 or 1");
  char *ws = reinterpret_cast<char *>(workspace);
  PhaseTimer timer(kPhaseGrad, stream);
  NotePhaseKernel(kPhaseGrad, "BandGrad");
  dim3 grid(CeilDiv(L.max_frames + 1, 4 * kGradLevels), args->num_fsas);
#define K2B_BAND_GRAD(ARCS, SMEM)                                                             \
  { BandGrad<ARCS><<<grid, 128, SMEM, stream>>>(                                              \
      reinterpret_cast<const BandInfo *>(ws + L.off_infos),                                   \
      reinterpret_cast<const BandState *>(args->band_states),                                 \
      reinterpret_cast<const BandArc *>(args->band_arcs),                                     \
      reinterpret_cast<const BandItem *>(ws + L.off_items),                                   \
      reinterpret_cast<const int32_t *>(ws + L.off_counts),                                   \
      reinterpret_cast<const double *>(ws + L.off_am),                                        \
      reinterpret_cast<const int32_t *>(ws + L.off_ae),                                       \
      reinterpret_cast<const double *>(ws + L.off_bm),                                        \
      reinterpret_cast<const int32_t *>(ws + L.off_be), tot_grad, tot_grad_stride, grad_a,    \
      grad_b, grad_row0, grad_pitch, grad_col_off, args->num_classes, L.st_pad,              \
      L.exclusive_rows ? 1 : 0); NoteLaunch(); }
  if (grad_a != nullptr) {
    const size_t smem = sizeof(ProbState) * 4 * (size_t)L.st_pad;
    K2B_BAND_GRAD(true, smem)
  } else {
    K2B_BAND_GRAD(false, 0)
  }
#undef K2B_BAND_GRAD
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t k2b200_band_loss_status(const k2b200_band_loss_args *args, void *workspace,
                                size_t workspace_bytes, void *stream_v, int32_t *status) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  K2B_REQUIRE(status != nullptr, "NULL output pointer");
  BandLayout L;
  K2B_FORWARD(MakeBandLayout(args, &L));
  K2B_REQUIRE(workspace != nullptr && workspace_bytes >= L.total_bytes, "workspace too small");
  K2B_CUDA_OK(cudaMemcpyAsync(status, reinterpret_cast<char *>(workspace) + L.off_status,
                              sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  K2B_CUDA_OK(cudaStreamSynchronize(stream));
  return kOk;
}

}  // extern "C"

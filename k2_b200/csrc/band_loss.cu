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
//   BandViterbi   one small CTA per (graph, direction) walks all frames: a thread owns four
//                 consecutive states in registers, neighbours come by two shuffles (and a
//                 two-float hand-over between warps), the log-prob row of the frame arrives in a
//                 shared-memory ring by one bulk copy (TMA, mbarrier) issued many frames ahead.
//                 Same fp32 expressions as the reference: (prev + arc.score) + dense, then max.
//   BandPrep      all (graph, frame) levels in parallel: the reference's keep tests
//                 (intersect_dense.cu:289-296, 430-471) on the two Viterbi grids, then per level
//                 the COMPACT list of surviving states with, per state and entering arc, the
//                 factor exp(arc score) * exp(dense score) if the arc survives and 0 otherwise,
//                 and the list positions of the states the arcs come from and go to.
//   BandChainLists  one warp per (graph, direction) walks the levels over the lists only: a lane
//                 holds the value of one surviving state, an entry names the list positions of
//                 its neighbours on the previous level, whose values come by shuffles: three
//                 multiply-adds per state and level, no exp or log, no test, no shared-memory
//                 traffic for values.  The lists arrive by bulk copies.  Values of a level
//                 share a power-of-two scale that follows the data.
//   BandChainExact  the same recursion with a (mantissa, exponent) pair per state, by state
//                 number in shared memory, for the graphs whose scores leave what a double
//                 with a per-level scale can hold or whose levels are wider than the registers
//                 of a warp; it runs after BandChainLists and returns at once for every other
//                 graph.
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
constexpr int kBandMaxStates = 512;
constexpr int kVitK = 4;              // states per thread of BandViterbi
constexpr int kPrepK = 16;            // states per lane of BandPrep's row scan
constexpr int kPrepLevels = 16;       // levels per chunk: their lists share one padded size
constexpr int kPrepSub = 8;           // levels per warp of BandPrep
constexpr int kGradLevels = 4;        // levels per warp of BandGrad
constexpr int kDrainPolls = 4000000;  // bounded wait for copies in flight when a kernel gives up

// bits of the status word
constexpr int32_t kStatusNotBand = 1, kStatusLate = 2;
// bits of unfit[i]: the lean recursion cannot represent this graph's numbers
constexpr int32_t kUnfitFactors = 1, kUnfitRange = 2;


// Per (graph, sequence) pair; built on the host, uploaded once per call.
struct BandInfo {
  int32_t state_off;   // first state (idx01) of the graph in a_fsas
  int32_t num_states;  // S
  int32_t pitch;       // 32 * (S / 32 + 1): row pitch of this pair's grids; a padded list fits
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
struct __align__(8) BandItem {
  int32_t label;  // of the arcs entering the state
  uint16_t s;     // the state
  uint8_t inb;    // bit d: the arc from state s - d of the level before survives
  uint8_t outb;   // bit d: the arc to state s + d of the next level survives
};
static_assert(sizeof(BandItem) == 8, "BandItem must be 8 bytes");
constexpr int kOutbByte = 7;
// What the recursions read per list entry (level l, state s):
//   pw[d]  = exp(score of the arc from state s - d) * exp(dense score of s's label on
//            frame l - 1) if that arc survives between levels l - 1 and l, else 0;
//   src[d] = position, in the list of level l - 1, of state s - d (0 when pw[d] is 0);
//   dst[d] = position, in the list of level l + 1, of state s + d if the arc to it
//            survives (whose factor is pw[d] of THAT entry), else kNoDst.
// The lists of the kPrepLevels levels of a chunk are padded to the same multiple of 32 entries,
// larger than the longest of them: a padding entry has pw = 0, src = 0 and dst = kNoDst, and
// kNoDst (lane 31 of the last register) always names a padding entry of the next level.
struct __align__(16) BandFactor {
  double pw[3];
  uint8_t src[4];  // [3] unused
  uint8_t dst[4];  // [3] unused
};
static_assert(sizeof(BandFactor) == 32, "BandFactor must be 32 bytes");
constexpr int kDstByte = 28;
constexpr uint32_t kNoDst = 255;
constexpr int kMaxRegs = 4;     // values of a level that a lane of the register recursion holds
constexpr int kMaxListed = 32 * kMaxRegs - 1;  // entries of a level that it handles (one lane is padding)
// words of BandPrep's per-state scratch: bit 15 = the state survives, bits 0-8 = its
// position in the level's list, bits 9-11 = entering-arc bits
constexpr uint32_t kMetaKept = 0x8000u, kMetaPos = 0x1ffu;
constexpr int kMetaInShift = 9;

// alpha of the final state on the last level (= Z) of a graph, as m * 2^e
struct __align__(16) BandTotal {
  double m;
  int32_t e;
  int32_t pad;
};

__device__ __forceinline__ double Pow2Clamp(int32_t e) {
  if (e < -1000) return 0.0;
  e = e > 1000 ? 1000 : e;
  return __longlong_as_double((long long)(1023 + e) << 52);
}

// Polls an mbarrier at most `limit` times.
__device__ __forceinline__ bool WaitSlot(uint64_t *bar, unsigned parity, int32_t limit) {
  for (int32_t k = 0; k < limit; ++k)
    if (MbarTryWait(bar, parity)) return true;
  return false;
}

// Dense score of a state with `label` on dense row `row` of a sequence of T frames whose
// frame 0 is at lp0 (the row T is the implied final row).
__device__ __forceinline__ float BandDense(const float *__restrict__ lp0, int32_t C, int32_t T,
                                           int32_t row, int32_t label) {
  if (row < T) return (label >= 0 && label < C) ? __ldg(lp0 + (int64_t)row * C + label) : -INFINITY;
  return label == -1 ? 0.0f : -INFINITY;
}

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
  if (bad) atomicOr(status, kStatusNotBand);
}

// ---------------------------------------------------------------------------
// Viterbi forward / backward.  grid = (2 directions, pairs).
// Level l (0 .. T + 1) of the forward grid: best score of any path from the start state
// at level 0 to the state at level l; of the backward grid: from the state at level l to
// the final state at level T + 1.  The step between levels l and l + 1 consumes dense row l
// (row T being the implied final row).
//
// A thread holds four consecutive states in registers.  A warp OWNS the states of its
// last 32 - H lanes and recomputes, in its first H lanes, the 4H states before them (the
// mirror image walking backward): a state depends on itself and its two predecessors, so
// what the warp computes for its own states stays exact for 2H frames without hearing
// from its neighbour.  Frames are therefore taken in batches of F = 2H: the log-prob rows
// of a batch are contiguous and arrive by ONE bulk copy (TMA, completion on an mbarrier)
// requested batches ahead, the warps exchange their boundary states through shared memory
// once per batch, and the frames of a batch run without any wait, barrier or
// shared-memory store: per frame four shared-memory reads, two shuffles, the adds and
// maxima, one 16-byte store.  Same fp32 expressions as the reference:
// (prev + arc.score) + dense, then max.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float Max3(float a, float b, float c) { return fmaxf(fmaxf(a, b), c); }

constexpr int kVitMaxBatches = 4;  // batches of rows in flight
constexpr int kVitMaxWarps = 8;

__global__ void __launch_bounds__(32 * kVitMaxWarps)
BandViterbi(const BandInfo *__restrict__ infos, const BandState *__restrict__ tab,
            const float *__restrict__ lp, int32_t C, float *__restrict__ vf,
            float *__restrict__ vb, int32_t F, int32_t nbatch, int32_t xch_pad,
            int32_t wait_limit, int32_t *__restrict__ status) {
  constexpr int K = kVitK;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full[kVitMaxBatches];
  __shared__ int32_t any_late;
  constexpr unsigned kAll = 0xffffffffu;
  const int dir = blockIdx.x;
  const BandInfo f = infos[blockIdx.y];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int32_t S = f.num_states, T = f.frames, pitch = f.pitch;
  if (S == 0) return;
  const int32_t H = F >> 1;         // lanes that recompute the neighbour's states
  const int32_t own = 32 - H;       // lanes whose states this warp owns
  float *ring = reinterpret_cast<float *>(smem_raw);                    // [nbatch][F][C]
  float *xch = ring + (size_t)nbatch * F * C;                           // [2][xch_pad], state s at s + 4H
  if (tid == 0) {
    for (int st = 0; st < nbatch; ++st) MbarInit(&full[st], 1);
    MbarInitFence();
    any_late = 0;
  }
  for (int32_t k = tid; k < 2 * xch_pad; k += blockDim.x) xch[k] = -INFINITY;
  __syncthreads();
  const int32_t num_batches = (T + F - 1) / F;
  const float *lp0 = lp + (int64_t)f.lp_row * C;
  int32_t issued = 0;
  auto issue = [&]() {  // thread 0 only: the rows of the next batch into the next slot
    if (issued >= num_batches) return;
    const int32_t q = issued;
    // batch q: forward rows [qF, min((q+1)F, T)); backward rows [max(T-(q+1)F, 0), T-qF)
    const int32_t r0 = dir == 0 ? q * F : max(T - (q + 1) * F, 0);
    const int32_t r1 = dir == 0 ? min((q + 1) * F, T) : T - q * F;
    const unsigned bytes = (unsigned)(r1 - r0) * 4u * (unsigned)C;
    const int32_t slot = q % nbatch;
    MbarArriveExpectTx(&full[slot], bytes);
    BulkCopyG2S(ring + (size_t)slot * F * C, lp0 + (int64_t)r0 * C, bytes, &full[slot]);
    ++issued;
  };
  if (tid == 0)
    for (int32_t q = 0; q < nbatch; ++q) issue();

  // first state of this lane: forward, the recomputed states come first; backward, last
  const int32_t s0 = warp * own * K + (dir == 0 ? (lane - H) * K : lane * K);
  const bool mine = dir == 0 ? lane >= H : lane < own;   // a lane that owns its states
  const bool stores = mine && s0 < pitch;
  float *grid = (dir == 0 ? vf : vb) + f.grid_off + s0;
  bool late = false;
  float v[K] = {0.0f, 0.0f, 0.0f, 0.0f};
  // exchange of boundary states: owners publish, recomputing lanes pick up
  auto exchange = [&](int32_t which) {
    float *x = xch + (size_t)which * xch_pad + 4 * H;
    if (mine && s0 < xch_pad - 4 * H - 3)
      *reinterpret_cast<float4 *>(x + s0) = make_float4(v[0], v[1], v[2], v[3]);
    __syncthreads();
    if (!mine && s0 + 4 * H >= 0 && s0 < xch_pad - 4 * H - 3) {
      const float4 t = *reinterpret_cast<const float4 *>(x + s0);
      v[0] = t.x;
      v[1] = t.y;
      v[2] = t.z;
      v[3] = t.w;
    }
  };
  if (dir == 0) {
    // ---- forward: state s from s, s - 1, s - 2 ----------------------------------
    float w0[K], w1[K], w2[K];     // on the frames; -inf for a state whose label has no column
    float f0[K], f1[K], f2[K];     // on the implied final row: only arcs labelled -1 score
    int32_t col[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int32_t s = s0 + k;
      w0[k] = w1[k] = w2[k] = f0[k] = f1[k] = f2[k] = -INFINITY;
      col[k] = 0;
      if (s >= 0 && s < S) {
        const BandState t = tab[f.state_off + s];
        if (t.label >= 0 && t.label < C) {
          col[k] = t.label;
          w0[k] = t.w[0];
          w1[k] = t.w[1];
          w2[k] = t.w[2];
        } else if (t.label == -1) {
          f0[k] = t.w[0];
          f1[k] = t.w[1];
          f2[k] = t.w[2];
        }
      }
      v[k] = s == 0 ? 0.0f : -INFINITY;
    }
    if (stores) *reinterpret_cast<float4 *>(grid) = make_float4(v[0], v[1], v[2], v[3]);
    int32_t xpar = 0;
    for (int32_t q = 0; q < num_batches; ++q) {
      const int32_t slot = q % nbatch;
      if (!late) late = !WaitSlot(&full[slot], (unsigned)(q / nbatch) & 1u, wait_limit);
      if (q > 0) {
        exchange(xpar);  // its barrier also says: every warp has finished batch q - 1
        xpar ^= 1;
        if (tid == 0 && !late) issue();  // into the slot batch q - 1 used
      }
      const int32_t nf = min(F, T - q * F);
      const float *rowbuf = ring + (size_t)slot * F * C;
#pragma unroll 4
      for (int32_t r = 0; r < nf; ++r, rowbuf += C) {
        float x[K];
#pragma unroll
        for (int k = 0; k < K; ++k) x[k] = rowbuf[col[k]];
        float h1 = __shfl_up_sync(kAll, v[K - 1], 1), h2 = __shfl_up_sync(kAll, v[K - 2], 1);
        if (lane == 0) h1 = h2 = -INFINITY;
        float nv[K];
#pragma unroll
        for (int k = 0; k < K; ++k) {
          const float a = v[k];
          const float b = k >= 1 ? v[k >= 1 ? k - 1 : 0] : h1;
          const float c = k >= 2 ? v[k >= 2 ? k - 2 : 0] : (k == 1 ? h1 : h2);
          const float m = Max3(__fadd_rn(a, w0[k]), __fadd_rn(b, w1[k]), __fadd_rn(c, w2[k]));
          nv[k] = __fadd_rn(m, x[k]);
        }
#pragma unroll
        for (int k = 0; k < K; ++k) v[k] = nv[k];
        grid += pitch;
        if (stores) *reinterpret_cast<float4 *>(grid) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
    // the implied final row: level T + 1
    exchange(xpar);
    {
      float h1 = __shfl_up_sync(kAll, v[K - 1], 1), h2 = __shfl_up_sync(kAll, v[K - 2], 1);
      if (lane == 0) h1 = h2 = -INFINITY;
      float nv[K];
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const float a = v[k];
        const float b = k >= 1 ? v[k >= 1 ? k - 1 : 0] : h1;
        const float c = k >= 2 ? v[k >= 2 ? k - 2 : 0] : (k == 1 ? h1 : h2);
        const float m = Max3(__fadd_rn(a, f0[k]), __fadd_rn(b, f1[k]), __fadd_rn(c, f2[k]));
        nv[k] = __fadd_rn(m, 0.0f);
      }
      grid += pitch;
      if (stores) *reinterpret_cast<float4 *>(grid) = make_float4(nv[0], nv[1], nv[2], nv[3]);
    }
  } else {
    // ---- backward: state s to s, s + 1, s + 2 -----------------------------------
    float wo[K][3];   // score of the arc s -> s + d on the frames (-inf: its label has no column)
    float fo[K][3];   // on the implied final row
    int32_t col[K + 2];   // of states s0 .. s0 + K + 1
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
      for (int d = 0; d < 3; ++d) wo[k][d] = fo[k][d] = -INFINITY;
#pragma unroll
    for (int k = 0; k < K + 2; ++k) {
      const int32_t s = s0 + k;
      col[k] = 0;
      BandState t;
      t.w[0] = t.w[1] = t.w[2] = -INFINITY;
      t.label = kNoLabel;
      if (s < S) t = tab[f.state_off + s];
      const bool frame_label = t.label >= 0 && t.label < C;
      if (frame_label) col[k] = t.label;
#pragma unroll
      for (int d = 0; d < 3; ++d)
        if (k - d >= 0 && k - d < K) {
          if (frame_label) wo[k - d >= 0 ? k - d : 0][d] = t.w[d];
          else if (t.label == -1) fo[k - d >= 0 ? k - d : 0][d] = t.w[d];
        }
    }
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] = (s0 + k == S - 1) ? 0.0f : -INFINITY;
    grid += (int64_t)(T + 1) * pitch;
    if (stores) *reinterpret_cast<float4 *>(grid) = make_float4(v[0], v[1], v[2], v[3]);
    {  // level T from level T + 1 through the implied final row (nothing to exchange yet:
       // only the final state is not -inf, and every lane knows it)
      float g1 = __shfl_down_sync(kAll, v[0], 1), g2 = __shfl_down_sync(kAll, v[1], 1);
      if (lane == 31) g1 = g2 = -INFINITY;
      float nv[K];
#pragma unroll
      for (int k = 0; k < K; ++k) {
        const float a = v[k];
        const float b = k + 1 < K ? v[k + 1 < K ? k + 1 : 0] : g1;
        const float c = k + 2 < K ? v[k + 2 < K ? k + 2 : 0] : (k + 2 == K ? g1 : g2);
        nv[k] = Max3(__fadd_rn(__fadd_rn(a, fo[k][0]), 0.0f), __fadd_rn(__fadd_rn(b, fo[k][1]), 0.0f),
                     __fadd_rn(__fadd_rn(c, fo[k][2]), 0.0f));
      }
#pragma unroll
      for (int k = 0; k < K; ++k) v[k] = nv[k];
      grid -= pitch;
      if (stores) *reinterpret_cast<float4 *>(grid) = make_float4(v[0], v[1], v[2], v[3]);
    }
    int32_t xpar = 0;
    for (int32_t q = 0; q < num_batches; ++q) {
      const int32_t slot = q % nbatch;
      if (!late) late = !WaitSlot(&full[slot], (unsigned)(q / nbatch) & 1u, wait_limit);
      exchange(xpar);  // also: every warp has finished batch q - 1
      xpar ^= 1;
      if (q > 0 && tid == 0 && !late) issue();
      const int32_t r1 = T - q * F, r0 = max(T - (q + 1) * F, 0);
      const float *rowbuf = ring + (size_t)slot * F * C + (size_t)(r1 - 1 - r0) * C;
#pragma unroll 4
      for (int32_t r = r1 - 1; r >= r0; --r, rowbuf -= C) {  // level r from level r + 1
        float x[K + 2];
#pragma unroll
        for (int k = 0; k < K + 2; ++k) x[k] = rowbuf[col[k]];
        float g1 = __shfl_down_sync(kAll, v[0], 1), g2 = __shfl_down_sync(kAll, v[1], 1);
        if (lane == 31) g1 = g2 = -INFINITY;
        float nv[K];
#pragma unroll
        for (int k = 0; k < K; ++k) {
          const float a = v[k];
          const float b = k + 1 < K ? v[k + 1 < K ? k + 1 : 0] : g1;
          const float c = k + 2 < K ? v[k + 2 < K ? k + 2 : 0] : (k + 2 == K ? g1 : g2);
          nv[k] = Max3(__fadd_rn(__fadd_rn(a, wo[k][0]), x[k]),
                       __fadd_rn(__fadd_rn(b, wo[k][1]), x[k + 1]),
                       __fadd_rn(__fadd_rn(c, wo[k][2]), x[k + 2]));
        }
#pragma unroll
        for (int k = 0; k < K; ++k) v[k] = nv[k];
        grid -= pitch;
        if (stores) *reinterpret_cast<float4 *>(grid) = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
  }
  if (late) any_late = 1;
  __syncthreads();
  if (any_late) {
    // A copy did not arrive in time: the grids hold garbage.  Say so, and let the copies
    // that are still in flight towards this CTA's shared memory land before it retires.
    if (tid == 0) {
      atomicOr(status, kStatusLate);
      for (int32_t q = max(0, issued - nbatch); q < issued; ++q)
        WaitSlot(&full[q % nbatch], (unsigned)(q / nbatch) & 1u, kDrainPolls);
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// Which states survive (intersect_dense.cu:289-296): state s of level l is kept iff
// vf[l][s] + vb[l][s] > cutoff.  grid = (level chunks, pairs), a warp per kKeepLevels levels;
// lane j looks at states K j .. K j + K - 1 (K = 16, or 8 when no graph has more than 256
// states, which keeps more lanes busy) and writes their keep bits: bit (s & 15) of the 16-bit
// word keep[(level_off + l) * 32 + s / 16] is the bit of state s.  totals[0] += surviving states, totals[2] += the arcs
// leaving them: the sizes the beam reduction looks at (intersect_dense.cu:289-320), which
// the host can read while the kernels behind this one run.
// ---------------------------------------------------------------------------
constexpr int kKeepLevels = 8;

template <int K>
__global__ void __launch_bounds__(128)
BandKeep(const BandInfo *__restrict__ infos, const int32_t *__restrict__ a_row_splits2,
         const float *__restrict__ vf, const float *__restrict__ vb, float beam,
         uint16_t *__restrict__ keep_bits, float *__restrict__ cutoffs,
         unsigned long long *__restrict__ totals, int32_t count_arcs) {
  static_assert(K == 8 || K == 16, "keep bits are stored as bytes or 16-bit words");
  constexpr unsigned kAll = 0xffffffffu;
  const int32_t i = blockIdx.y;
  const BandInfo f = infos[i];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int32_t S = f.num_states, T = f.frames, pitch = f.pitch;
  if (S == 0) return;
  const int32_t a = (blockIdx.x * 4 + warp) * kKeepLevels;
  if (a > T + 1) return;
  const int32_t b = min(a + kKeepLevels, T + 2);
  const float *fg = vf + f.grid_off, *bg = vb + f.grid_off;
  float cutoff;
  {
    const float start = bg[0], end = fg[(int64_t)(T + 1) * pitch + (S - 1)];
    cutoff = __fsub_rn(start < end ? start : end, beam);
  }
  if (a == 0 && lane == 0) cutoffs[i] = cutoff;
  const int32_t s0 = lane * K;
  uint32_t n_states = 0, n_cand = 0;
#pragma unroll 4
  for (int32_t l = a; l < b; ++l) {
    uint32_t keep = 0;
#pragma unroll
    for (int c = 0; c < K / 4; ++c) {
      if (s0 + 4 * c >= S) continue;
      const float4 F = *reinterpret_cast<const float4 *>(fg + (int64_t)l * pitch + s0 + 4 * c);
      const float4 B = *reinterpret_cast<const float4 *>(bg + (int64_t)l * pitch + s0 + 4 * c);
      if (__fadd_rn(F.x, B.x) > cutoff) keep |= 1u << (4 * c);
      if (__fadd_rn(F.y, B.y) > cutoff) keep |= 2u << (4 * c);
      if (__fadd_rn(F.z, B.z) > cutoff) keep |= 4u << (4 * c);
      if (__fadd_rn(F.w, B.w) > cutoff) keep |= 8u << (4 * c);
    }
    if (K == 16) {
      keep_bits[(int64_t)(f.level_off + l) * 32 + lane] = (uint16_t)keep;
    } else {  // the same layout byte by byte; states 256 .. 511 do not exist
      unsigned char *row = reinterpret_cast<unsigned char *>(keep_bits + (int64_t)(f.level_off + l) * 32);
      row[lane] = (unsigned char)keep;
      row[32 + lane] = 0;
    }
    n_states += __popc(keep);
    if (count_arcs) {  // uniform; the host leaves it out when no count could reach max_arcs
      for (uint32_t m = keep; m; m &= m - 1) {
        const int32_t idx = f.state_off + s0 + __ffs(m) - 1;
        n_cand += __ldg(a_row_splits2 + idx + 1) - __ldg(a_row_splits2 + idx);
      }
    }
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
// Keep tests.  grid = (level chunks, pairs), 4 warps per CTA, a warp per chunk of
// kPrepLevels levels.  Per level the warp
//   1. scans the two Viterbi rows (a lane reads 16 consecutive states of each; the rows of
//      the next level are requested before this level is worked on), marks the surviving
//      states and writes them, in state order, to a list in shared memory;
//   2. takes the list one state per lane: the reference's arc tests
//      (intersect_dense.cu:430-471) against the rows of the level before and the dense
//      score of the state's label give the entering-arc bits, the factors and where in the
//      previous list the sources are;
//   3. gives the entries of the level before their leaving-arc bits and destinations, which
//      are the entering arcs of this level seen from the source.
// Per level the result is the compact list of surviving states: a BandItem (label, state,
// bits) and a BandFactor per entry.  A warp writes the complete entries of the levels it
// owns, so it also runs step 1 for the level before its first and steps 1-2 for the level
// after its last.  totals[0] += surviving states, totals[2] += the arcs leaving them (the
// sizes the beam reduction looks at, intersect_dense.cu:289-320).  unfit[i] is set when the
// register recursion cannot take graph i: a score outside its arithmetic, or a level with
// more than kMaxListed surviving states.
// ---------------------------------------------------------------------------
constexpr float kMinLeanDense = -60.0f;   // dense score of a surviving arc
constexpr int32_t kMaxLeanArcExp = 60, kMinLeanArcExp = -90;  // binary exponent of exp(arc score)

__global__ void __launch_bounds__(128)
BandPrep(const BandInfo *__restrict__ infos, const BandState *__restrict__ tab,
         const BandArc *__restrict__ tabf, const uint16_t *__restrict__ keep_bits,
         const float *__restrict__ lp, int32_t C, const float *__restrict__ vf,
         const float *__restrict__ vb, const float *__restrict__ cutoffs,
         BandItem *__restrict__ items, BandFactor *__restrict__ factors,
         int2 *__restrict__ lists, int32_t *__restrict__ chunk_r, int32_t *__restrict__ unfit,
         int32_t s_pad) {
  constexpr int K = kPrepK;
  constexpr unsigned kAll = 0xffffffffu;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int32_t i = blockIdx.y;
  const BandInfo f = infos[i];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int32_t S = f.num_states, T = f.frames, pitch = f.pitch;
  if (S == 0) return;
  // a warp owns kPrepSub levels a .. b - 1, part of the chunk of kPrepLevels levels ca .. cb - 1
  const int32_t a = (blockIdx.x * 4 + warp) * kPrepSub;
  if (a > T + 1) return;
  const int32_t b = min(a + kPrepSub, T + 2);
  const int32_t ca = a / kPrepLevels * kPrepLevels, cb = min(ca + kPrepLevels, T + 2);
  // per warp: a word per state for the current and the previous level (zero outside the
  // lists), and the two lists
  uint16_t *meta_sm = reinterpret_cast<uint16_t *>(smem_raw) +
                      (size_t)warp * (4 * s_pad + 32 * (kPrepLevels + 2));  // [2][s_pad]
  uint16_t *list_sm = meta_sm + 2 * s_pad;                                  // [2][s_pad]
  uint16_t *keep_sm = list_sm + 2 * s_pad;  // [kPrepLevels + 2][32]: the lanes' keep bits
  for (int32_t k = lane; k < 2 * s_pad; k += 32) meta_sm[k] = 0;
  const float *fg = vf + f.grid_off, *bg = vb + f.grid_off;
  const float cutoff = cutoffs[i];
  const float *lp0 = lp + (int64_t)f.lp_row * C;
  const int32_t s0 = lane * K;
  const int32_t first = max(a - 1, 0);  // first level looked at (its list only)
  const int32_t last = min(b, T + 1);   // last level looked at
  // ---- 0. the keep bits of every level this warp looks at; the longest list of the
  // CHUNK's levels decides how many entries every level of the chunk gets (every warp of a
  // chunk finds the same number) ----------------------------------------------------------
  int32_t longest = 0;
  const int32_t lo = min(first, ca), hi = max(last, cb - 1);
#pragma unroll 6
  for (int32_t l = lo; l <= hi; ++l) {
    const uint32_t keep = keep_bits[(int64_t)(f.level_off + l) * 32 + lane];
    if (l >= first && l <= last) keep_sm[(l - first) * 32 + lane] = (uint16_t)keep;
    const int32_t n = __reduce_add_sync(kAll, __popc(keep));
    if (l >= ca && l < cb) longest = max(longest, n);
  }
  const int32_t padded = 32 * (longest / 32 + 1);  // entries per level of this chunk
  if (lane == 0 && a == ca) chunk_r[f.level_off + ca] = padded / 32;
  int32_t n_prev = 0;
  // the lists of a warp's levels lie `padded` entries apart from the start of its chunk
  // (pitch >= padded); lists[level] = (start, size)
  int32_t run = ca * pitch + (a - ca) * padded, prev_start = 0;
  bool risky = false;
  __syncwarp();
  for (int32_t l = first; l <= last; ++l) {
    const bool own = l >= a && l < b;
    uint16_t *cur_list = list_sm + (l & 1) * s_pad, *prev_list = list_sm + ((l & 1) ^ 1) * s_pad;
    uint16_t *cur_meta = meta_sm + (l & 1) * s_pad, *prev_meta = meta_sm + ((l & 1) ^ 1) * s_pad;
    // ---- 1. surviving states ------------------------------------------------------
    const uint32_t keep = keep_sm[(l - first) * 32 + lane];
    const int32_t mine = __popc(keep);
    int32_t incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int32_t o = __shfl_up_sync(kAll, incl, d);
      if (lane >= d) incl += o;
    }
    const int32_t n = __shfl_sync(kAll, incl, 31);
    {
      int32_t pos = incl - mine;
      for (uint32_t m = keep; m; m &= m - 1) {
        const int32_t s = s0 + __ffs(m) - 1;
        cur_list[pos] = (uint16_t)s;
        cur_meta[s] = (uint16_t)(kMetaKept | (uint32_t)pos);
        ++pos;
      }
    }
    if (n > kMaxListed) risky = true;
    __syncwarp();
    if (l >= a) {
      // ---- 2. one surviving state per lane ------------------------------------------
      BandItem *out = items + f.grid_off + run;
      BandFactor *fout = factors + f.grid_off + run;
      const float *fprev = fg + (int64_t)(l - 1) * pitch, *bprev = bg + (int64_t)(l - 1) * pitch;
      const float *bcur = bg + (int64_t)l * pitch;
      for (int32_t j = lane; j < n; j += 32) {
        const int32_t s = cur_list[j];
        const BandState t = tab[f.state_off + s];
        uint32_t inb = 0;
        BandFactor fa;
        fa.pw[0] = fa.pw[1] = fa.pw[2] = 0.0;
        fa.src[0] = fa.src[1] = fa.src[2] = fa.src[3] = 0;
        fa.dst[0] = fa.dst[1] = fa.dst[2] = fa.dst[3] = (uint8_t)kNoDst;
        if (l >= 1) {
          const float x = BandDense(lp0, C, T, l - 1, t.label);
          const float bc = bcur[s];
          const double p = exp((double)x);
#pragma unroll
          for (int d = 0; d < 3; ++d) {
            if (s - d < 0) continue;
            const float sf = fprev[s - d];
            const bool kept = __fadd_rn(sf, bprev[s - d]) > cutoff;
            const float sc = __fadd_rn(t.w[d], x);
            if (kept && __fadd_rn(__fadd_rn(sf, sc), bc) > cutoff) {
              inb |= 1u << d;
              if (own) {
                const BandArc arc = tabf[(int64_t)(f.state_off + s) * 3 + d];
                fa.pw[d] = arc.f * Pow2Clamp(arc.k) * p;
                fa.src[d] = (uint8_t)(prev_meta[s - d] & kMetaPos);
                // outside what doubles with a scale that follows the data every few
                // levels hold: such graphs go to the (mantissa, exponent) recursion
                if (!(x >= kMinLeanDense) || arc.k > kMaxLeanArcExp || arc.k < kMinLeanArcExp)
                  risky = true;
              }
            }
          }
        }
        cur_meta[s] = (uint16_t)(cur_meta[s] | (inb << kMetaInShift));
        if (own) {
          BandItem it;
          it.label = t.label;
          it.s = (uint16_t)s;
          it.inb = (uint8_t)inb;
          it.outb = 0;
          out[j] = it;
          fout[j] = fa;
        }
      }
      if (own) {
        BandFactor none;
        none.pw[0] = none.pw[1] = none.pw[2] = 0.0;
        none.src[0] = none.src[1] = none.src[2] = none.src[3] = 0;
        none.dst[0] = none.dst[1] = none.dst[2] = none.dst[3] = (uint8_t)kNoDst;
        for (int32_t j = n + lane; j < padded; j += 32) fout[j] = none;
        if (lane == 0) lists[f.level_off + l] = make_int2(run, n);
      }
      __syncwarp();
      // ---- 3. leaving arcs of the level before --------------------------------------------
      if (l - 1 >= a) {
        unsigned char *ibytes = reinterpret_cast<unsigned char *>(items + f.grid_off + prev_start);
        unsigned char *fbytes = reinterpret_cast<unsigned char *>(factors + f.grid_off + prev_start);
        for (int32_t j = lane; j < n_prev; j += 32) {
          const int32_t s = prev_list[j];
          uint32_t ob = 0;
#pragma unroll
          for (int d = 0; d < 3; ++d) {
            const uint32_t m = cur_meta[s + d];
            if ((m >> (kMetaInShift + d)) & 1u) {
              ob |= 1u << d;
              fbytes[(size_t)j * sizeof(BandFactor) + kDstByte + d] = (unsigned char)(m & kMetaPos);
            }
          }
          if (ob) ibytes[(size_t)j * sizeof(BandItem) + kOutbByte] = (unsigned char)ob;
        }
      }
    }
    __syncwarp();
    // the previous level's words go back to zero for the level after this one
    for (int32_t j = lane; j < n_prev; j += 32) prev_meta[prev_list[j]] = 0;
    __syncwarp();
    n_prev = n;
    if (l >= a) {
      prev_start = run;
      run += padded;
    }
  }
  if (__any_sync(kAll, risky) && lane == 0) atomicOr(&unfit[i], kUnfitFactors);
}

// ---------------------------------------------------------------------------
// alpha (dir 0) and beta (dir 1) over the lists, in registers.  grid = (2, pairs), one warp
// per CTA.  Lane j holds the value of entry j (and j + 32, j + 64, j + 96) of the current level's
// list; an entry says at which POSITIONS of the previous list its neighbours are, so the
// values it needs come by shuffles from the lanes that hold them:
//   alpha_l[j] = sum_d pw_l[j][d] * alpha_{l-1}[src_l[j][d]]
//   beta_l[j]  = sum_d (pw_{l+1}[.][d] * beta_{l+1}[.]) at position dst_l[j][d]
// Every level of a chunk of kPrepLevels levels has the same padded number of entries, 32 per
// register, so inside a chunk every address is a constant: the fifteen levels after a
// chunk's first are straight-line code, per level two 16-byte loads from shared memory, six
// shuffles, three multiply-adds and a store per register: no test (an absent neighbour is
// a padding entry, whose value is 0), no address arithmetic, no synchronisation.  The chunks
// arrive in a ring in shared memory by one bulk copy each, requested chunks ahead.
// The values of a level are stored divided by 2^K; K changes every kRescale levels by the
// exponent of the largest value since the last change.  A value that is not zero and
// below 2^-900 (or a value above 2^900) marks the graph in `unfit` for BandChainExact,
// like the graphs BandPrep marked, which return at once here.
// Outputs: alpha / beta at the list positions, K per level, tot[i], total[i].
// ---------------------------------------------------------------------------
constexpr int kRescale = 8;                     // levels between changes of the shared scale
constexpr int kChainSlots = 3;                  // chunks in flight
constexpr int kFacSlot = kPrepLevels * 32 * kMaxRegs;  // BandFactor entries of a chunk's levels
constexpr int kChainMaxChunks = 4096;           // of a graph: 65534 frames
constexpr int kSlotItems = kPrepLevels * 128;   // BandItem entries likewise (BandChainExact)

// The ring of chunks: lane 0 requests, every lane waits.
template <typename Item, int kCap>
struct ChunkRing {
  uint64_t *full;          // [kChainSlots]
  Item *slots;             // [kChainSlots][kCap]
  const Item *items0;      // the pair's lists
  const int2 *lst;         // (start, size) of every level, in shared memory
  int32_t pitch, L, num_chunks, dir, issued;
  __device__ __forceinline__ int32_t ChunkOf(int32_t q) const {
    return dir == 0 ? q : num_chunks - 1 - q;
  }
  // entries of a chunk's lists (they are contiguous from the chunk's start)
  __device__ __forceinline__ int32_t ChunkItems(int32_t c) const {
    const int32_t l1 = min((c + 1) * kPrepLevels, L) - 1;
    return lst[l1].x + lst[l1].y - c * kPrepLevels * pitch;
  }
  __device__ __forceinline__ void Issue() {  // lane 0: the next chunk into the next slot
    if (issued >= num_chunks) return;
    const int32_t c = ChunkOf(issued), slot = issued % kChainSlots;
    // a multiple of 16 bytes, at least 16, so that the copy is legal and the slot's barrier
    // completes once per use (a chunk starts on a multiple of four entries and has room for
    // at least four)
    constexpr int32_t kPer16 = sizeof(Item) >= 16 ? 1 : 16 / sizeof(Item);
    const int32_t n = max((min(ChunkItems(c), kCap) + kPer16 - 1) / kPer16 * kPer16, kPer16);
    const unsigned bytes = (unsigned)n * (unsigned)sizeof(Item);
    MbarArriveExpectTx(&full[slot], bytes);
    BulkCopyG2S(slots + (size_t)slot * kCap, items0 + (int64_t)c * kPrepLevels * pitch, bytes,
                &full[slot]);
    ++issued;
  }
  __device__ __forceinline__ void Drain() {  // lane 0, after giving up
    for (int32_t k = max(0, issued - kChainSlots); k < issued; ++k)
      WaitSlot(&full[k % kChainSlots], (unsigned)(k / kChainSlots) & 1u, kDrainPolls);
  }
};

// One level of the walk.  `rec` = this lane's entry of the level's first 32 (in shared
// memory), `out` = where its value goes; RC registers per lane on this level, RP on the one
// walked before.  v = values of the level before (forward), pc[d] = the products
// pw[d] * value of the level before (backward); both are replaced by this level's.
template <int DIR, int RC, int RP, bool kScaled>
__device__ __forceinline__ void ChainLevel(const BandFactor *rec, double *__restrict__ out,
                                           double scale, double (&v)[kMaxRegs],
                                           double (&pc)[3][kMaxRegs], int32_t &hi_max,
                                           uint32_t &min_hi) {
  constexpr unsigned kAll = 0xffffffffu;
  double nv[RC], pw[RC][3];
#pragma unroll
  for (int r = 0; r < RC; ++r) {
    const double2 p01 = *reinterpret_cast<const double2 *>(rec + 32 * r);
    const int4 q = *(reinterpret_cast<const int4 *>(rec + 32 * r) + 1);
    pw[r][0] = p01.x;
    pw[r][1] = p01.y;
    pw[r][2] = __hiloint2double(q.y, q.x);
    const uint32_t word = DIR == 0 ? (uint32_t)q.z : (uint32_t)q.w;
    double x[3];
#pragma unroll
    for (int d = 0; d < 3; ++d) {
      // a shuffle looks at the low five bits of the lane only
      const uint32_t pos = RP == 1 ? word >> (8 * d) : (word >> (8 * d)) & 0xffu;
      x[d] = __shfl_sync(kAll, DIR == 0 ? v[0] : pc[d][0], (int)pos);
      if (RP > 1) {
        const double x1 = __shfl_sync(kAll, DIR == 0 ? v[1] : pc[d][1], (int)pos);
        x[d] = pos >= 32u ? x1 : x[d];
      }
      if (RP > 2) {
        const double x2 = __shfl_sync(kAll, DIR == 0 ? v[2] : pc[d][2], (int)pos);
        x[d] = pos >= 64u ? x2 : x[d];
      }
      if (RP > 3) {
        const double x3 = __shfl_sync(kAll, DIR == 0 ? v[3] : pc[d][3], (int)pos);
        x[d] = pos >= 96u ? x3 : x[d];
      }
    }
    double acc;
    if (DIR == 0) acc = fma(pw[r][0], x[0], fma(pw[r][1], x[1], pw[r][2] * x[2]));
    else acc = (x[0] + x[1]) + x[2];
    nv[r] = kScaled ? acc * scale : acc;
  }
#pragma unroll
  for (int r = 0; r < RC; ++r) {
    out[32 * r] = nv[r];
    const int32_t hi = __double2hiint(nv[r]);  // values are not negative
    hi_max = max(hi_max, hi);
    min_hi = min(min_hi, (uint32_t)hi - 1u);  // a zero does not count
    v[r] = nv[r];
    if (DIR == 1) {
      pc[0][r] = pw[r][0] * nv[r];
      pc[1][r] = pw[r][1] * nv[r];
      pc[2][r] = pw[r][2] * nv[r];
    }
  }
}

// The same with the register counts known at run time only.
template <int DIR>
__device__ __forceinline__ void ChainLevelAny(int32_t rc, int32_t rp, const BandFactor *rec,
                                              double *__restrict__ out, double scale,
                                              double (&v)[kMaxRegs],
                                              double (&pc)[3][kMaxRegs], int32_t &hi_max,
                                              uint32_t &min_hi) {
#define K2B_LEVEL(RC, RP) \
  case RC * 8 + RP: ChainLevel<DIR, RC, RP, true>(rec, out, scale, v, pc, hi_max, min_hi); break;
  switch (rc * 8 + rp) {
    K2B_LEVEL(1, 1) K2B_LEVEL(1, 2) K2B_LEVEL(1, 3) K2B_LEVEL(1, 4)
    K2B_LEVEL(2, 1) K2B_LEVEL(2, 2) K2B_LEVEL(2, 3) K2B_LEVEL(2, 4)
    K2B_LEVEL(3, 1) K2B_LEVEL(3, 2) K2B_LEVEL(3, 3) K2B_LEVEL(3, 4)
    K2B_LEVEL(4, 1) K2B_LEVEL(4, 2) K2B_LEVEL(4, 3)
    default: ChainLevel<DIR, 4, 4, true>(rec, out, scale, v, pc, hi_max, min_hi); break;
  }
#undef K2B_LEVEL
}

// The new scale after kRescale levels: the exponent of the largest value since the last one.
__device__ __forceinline__ double ChainRescale(int32_t &hi_max, int32_t &Ksh) {
  const int32_t hm = __reduce_max_sync(0xffffffffu, hi_max);
  const int32_t e = hm > 0 ? (hm >> 20) - 1023 : 0;
  Ksh += e;
  hi_max = 0;
  return __longlong_as_double((long long)(1023 - e) << 52);
}

// Levels 1 .. 15 (in walking order) of a full chunk with RC registers per lane: seven levels,
// the level that changes the scale, seven levels.  kChainUnroll levels of straight-line code per
// loop iteration: a single warp has nobody to hide an instruction-cache miss behind, so the
// code of a chunk should stay small.
constexpr int kChainUnroll = 1;  // (fully unrolled: 178 us for ctc_large; 1: 147 us)

template <int DIR, int RC>
__device__ __forceinline__ void ChainRest(const BandFactor *base, double *__restrict__ ob,
                                          int32_t *__restrict__ osc, int lane, double (&v)[kMaxRegs],
                                          double (&pc)[3][kMaxRegs], int32_t &hi_max, uint32_t &min_hi,
                                          int32_t &Ksh) {
  static_assert(kPrepLevels == 2 * kRescale, "a chunk is two groups of kRescale levels");
  constexpr int kStep = DIR == 0 ? 1 : -1;
  auto plain = [&](int kk_first) {  // kRescale - 1 levels without a change of scale
    const int m0 = DIR == 0 ? kk_first : kPrepLevels - 1 - kk_first;
    const BandFactor *r = base + m0 * 32 * RC;
    double *o = ob + m0 * 32 * RC;
    int32_t *sc = osc + m0;
#pragma unroll kChainUnroll
    for (int k = 0; k < kRescale - 1; ++k) {
      ChainLevel<DIR, RC, RC, false>(r, o, 1.0, v, pc, hi_max, min_hi);
      if (lane == 0) *sc = Ksh;
      r += kStep * 32 * RC;
      o += kStep * 32 * RC;
      sc += kStep;
    }
  };
  plain(1);
  {
    const int m = DIR == 0 ? kRescale : kPrepLevels - 1 - kRescale;
    const double scale = ChainRescale(hi_max, Ksh);
    ChainLevel<DIR, RC, RC, true>(base + m * 32 * RC, ob + m * 32 * RC, scale, v, pc, hi_max,
                                  min_hi);
    if (lane == 0) osc[m] = Ksh;
  }
  plain(kRescale + 1);
}

template <int DIR>
__device__ __forceinline__ void ChainWalk(const BandInfo &f, int32_t i, BandFactor *ring,
                                          unsigned char *crc, uint64_t *full,
                                          const BandFactor *__restrict__ factors,
                                          const int32_t *__restrict__ chunk_r,
                                          double *__restrict__ om, int32_t *__restrict__ oscale,
                                          double *__restrict__ tot, BandTotal *__restrict__ total,
                                          int32_t *__restrict__ unfit,
                                          int32_t *__restrict__ status, int32_t wait_limit) {
  constexpr unsigned kAll = 0xffffffffu;
  const int lane = threadIdx.x;
  const int32_t T = f.frames, pitch = f.pitch, L = T + 2;
  const int32_t num_chunks = (L + kPrepLevels - 1) / kPrepLevels;
  for (int32_t c = lane; c < num_chunks; c += 32)
    crc[c] = (unsigned char)chunk_r[f.level_off + c * kPrepLevels];
  if (lane == 0) {
    for (int st = 0; st < kChainSlots; ++st) MbarInit(&full[st], 1);
    MbarInitFence();
  }
  __syncwarp();
  const BandFactor *fac0 = factors + f.grid_off;
  om += f.grid_off;
  oscale += f.level_off;
  int32_t issued = 0;
  // lane 0: the next chunk (in walking order) into the next slot; a chunk is
  // levels * 32 * registers entries, a multiple of 1 KB
  auto issue = [&]() {
    if (issued >= num_chunks) return;
    const int32_t c = DIR == 0 ? issued : num_chunks - 1 - issued, slot = issued % kChainSlots;
    const int32_t nl = min((c + 1) * kPrepLevels, L) - c * kPrepLevels;
    const unsigned bytes = (unsigned)(nl * 32 * (int32_t)crc[c]) * (unsigned)sizeof(BandFactor);
    MbarArriveExpectTx(&full[slot], bytes);
    BulkCopyG2S(ring + (size_t)slot * kFacSlot, fac0 + (int64_t)c * kPrepLevels * pitch, bytes,
                &full[slot]);
    ++issued;
  };
  if (lane == 0)
    for (int32_t k = 0; k < kChainSlots; ++k) issue();
  double v[kMaxRegs], pc[3][kMaxRegs];
#pragma unroll
  for (int r = 0; r < kMaxRegs; ++r) v[r] = pc[0][r] = pc[1][r] = pc[2][r] = 0.0;
  int32_t Ksh = 0;
  int32_t hi_max = 0;              // largest high word since the last change of scale
  uint32_t min_hi = 0xffffffffu;   // smallest (high word - 1), zeros apart
  bool late = false;
  int32_t rp = 1;
  for (int32_t q = 0; q < num_chunks; ++q) {
    const int32_t c = DIR == 0 ? q : num_chunks - 1 - q, slot = q % kChainSlots;
    late = !WaitSlot(&full[slot], (unsigned)(q / kChainSlots) & 1u, wait_limit);
    late = __any_sync(kAll, late);
    if (late) break;
    const int32_t l_lo = c * kPrepLevels, nl = min(l_lo + kPrepLevels, L) - l_lo;
    const int32_t rc = crc[c];
    const BandFactor *base = ring + (size_t)slot * kFacSlot + lane;
    double *ob = om + (int64_t)l_lo * pitch + lane;
    int32_t *osc = oscale + l_lo;
    // the chunk's first level meets the registers of the chunk before; the levels of a
    // short chunk (the last of a graph) are taken the same way
    int32_t kk = 0;
    do {
      const int32_t m = DIR == 0 ? kk : nl - 1 - kk, l = l_lo + m;
      const BandFactor *rec = base + m * 32 * rc;
      double *out = ob + m * 32 * rc;
      if (q == 0 && kk == 0) {
        // the first level holds one state, with the value 1: the start state walking
        // forward, the final state walking backward
        v[0] = lane == 0 ? 1.0 : 0.0;
#pragma unroll
        for (int r = 1; r < kMaxRegs; ++r) v[r] = 0.0;
#pragma unroll
        for (int r = 0; r < kMaxRegs; ++r) {
          if (r >= rc) break;  // uniform
          out[32 * r] = v[r];
          if (DIR == 1) {
            const BandFactor e = rec[32 * r];
            pc[0][r] = e.pw[0] * v[r];
            pc[1][r] = e.pw[1] * v[r];
            pc[2][r] = e.pw[2] * v[r];
          }
        }
      } else {
        double scale = 1.0;
        if ((l & (kRescale - 1)) == (DIR == 0 ? 0 : kRescale - 1)) scale = ChainRescale(hi_max, Ksh);
        ChainLevelAny<DIR>(rc, kk == 0 ? rp : rc, rec, out, scale, v, pc, hi_max, min_hi);
      }
      if (lane == 0) osc[m] = Ksh;
      ++kk;
    } while (kk < nl && nl != kPrepLevels);
    if (nl == kPrepLevels) {
      if (rc == 1) ChainRest<DIR, 1>(base, ob, osc, lane, v, pc, hi_max, min_hi, Ksh);
      else if (rc == 2) ChainRest<DIR, 2>(base, ob, osc, lane, v, pc, hi_max, min_hi, Ksh);
      else if (rc == 3) ChainRest<DIR, 3>(base, ob, osc, lane, v, pc, hi_max, min_hi, Ksh);
      else ChainRest<DIR, 4>(base, ob, osc, lane, v, pc, hi_max, min_hi, Ksh);
    }
    rp = rc;
    __syncwarp();  // every lane has read the slot
    if (lane == 0) issue();  // the chunk is done with: its slot takes the next one
  }
  if (late) {
    if (lane == 0) {
      atomicOr(status, kStatusLate);
      for (int32_t k = max(0, issued - kChainSlots); k < issued; ++k)
        WaitSlot(&full[k % kChainSlots], (unsigned)(k / kChainSlots) & 1u, kDrainPolls);
    }
    __syncwarp();
  }
  {
    // values that are not zero must have kept clear of the ends of a double's range
    const int32_t hm = __reduce_max_sync(kAll, hi_max);
    const uint32_t hn = __reduce_min_sync(kAll, min_hi);
    if ((hm >= ((1023 + 900) << 20) || hn < (uint32_t)(((1023 - 900) << 20) - 1)) && lane == 0)
      atomicOr(&unfit[i], kUnfitRange);
  }
  if (DIR == 0 && lane == 0) {
    const double last = v[0];  // entry 0 of the last level is the final state
    if (*status & kStatusLate) {
      tot[i] = nan("");
    } else if (!late && last > 0.0) {
      tot[i] = log(last) + (double)Ksh * 0.69314718055994530942;
      BandTotal z;
      z.m = last;
      z.e = Ksh;
      z.pad = 0;
      total[i] = z;
    }
  }
}

__global__ void __launch_bounds__(32)
BandChainLists(const BandInfo *__restrict__ infos, const BandFactor *__restrict__ factors,
               const int32_t *__restrict__ chunk_r, double *__restrict__ am,
               double *__restrict__ bm, int32_t *__restrict__ a_scale,
               int32_t *__restrict__ b_scale, double *__restrict__ tot,
               BandTotal *__restrict__ total, int32_t *__restrict__ unfit,
               int32_t *__restrict__ status, int32_t wait_limit) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full[kChainSlots];
  __shared__ unsigned char crc[kChainMaxChunks];
  const int dir = blockIdx.x;
  const int32_t i = blockIdx.y;
  const BandInfo f = infos[i];
  if (dir == 0 && threadIdx.x == 0) {
    tot[i] = -INFINITY;
    BandTotal z;
    z.m = 0.0;
    z.e = 0;
    z.pad = 0;
    total[i] = z;
  }
  if (f.num_states == 0 || unfit[i] != 0) return;  // BandChainExact takes the graphs BandPrep marked
  BandFactor *ring = reinterpret_cast<BandFactor *>(smem_raw);  // [slots][kFacSlot]
  if (dir == 0)
    ChainWalk<0>(f, i, ring, crc, full, factors, chunk_r, am, a_scale, tot, total, unfit, status,
                 wait_limit);
  else
    ChainWalk<1>(f, i, ring, crc, full, factors, chunk_r, bm, b_scale, tot, total, unfit, status,
                 wait_limit);
}

// The same recursion with a (mantissa, exponent) pair per state, for the graphs marked in
// `unfit`; every other graph returns at once.  exp(dense score) is recomputed from the
// log-probs, the arc factors come from the graph's tables: no range limit.
__global__ void __launch_bounds__(32)
BandChainExact(const BandInfo *__restrict__ infos, const BandArc *__restrict__ tabf,
               const float *__restrict__ lp, int32_t C, const BandItem *__restrict__ items,
               const int2 *__restrict__ lists, double *__restrict__ am,
               int32_t *__restrict__ ae, double *__restrict__ bm, int32_t *__restrict__ be,
               double *__restrict__ tot, BandTotal *__restrict__ total,
               const int32_t *__restrict__ unfit, int32_t *__restrict__ status, int32_t st_pad,
               int32_t lv_pad, int32_t wait_limit) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full[kChainSlots];
  constexpr unsigned kAll = 0xffffffffu;
  const int dir = blockIdx.x;
  const int32_t i = blockIdx.y;
  if (unfit[i] == 0) return;  // the lean recursion served this graph
  const BandInfo f = infos[i];
  const int lane = threadIdx.x;
  const int32_t S = f.num_states, T = f.frames, pitch = f.pitch, L = T + 2;
  if (S == 0) return;
  BandItem *ring = reinterpret_cast<BandItem *>(smem_raw);
  int2 *lst = reinterpret_cast<int2 *>(ring + kChainSlots * kSlotItems);
  ProbState *vals = reinterpret_cast<ProbState *>(lst + lv_pad);  // [2][st_pad], state s at s + 2
  for (int32_t l = lane; l < L; l += 32) lst[l] = lists[f.level_off + l];
  for (int32_t k = lane; k < 2 * st_pad; k += 32) {
    ProbState z;
    z.m = 0.0;
    z.e = kZeroExp;
    z.pad = 0;
    vals[k] = z;
  }
  if (lane == 0) {
    for (int st = 0; st < kChainSlots; ++st) MbarInit(&full[st], 1);
    MbarInitFence();
  }
  __syncwarp();
  ChunkRing<BandItem, kSlotItems> rg;
  rg.full = full;
  rg.slots = ring;
  rg.items0 = items + f.grid_off;
  rg.lst = lst;
  rg.pitch = pitch;
  rg.L = L;
  rg.num_chunks = (L + kPrepLevels - 1) / kPrepLevels;
  rg.dir = dir;
  rg.issued = 0;
  if (lane == 0)
    for (int32_t k = 0; k < kChainSlots; ++k) rg.Issue();
  const float *lp0 = lp + (int64_t)f.lp_row * C;
  const BandArc *my_arcs = tabf + (int64_t)f.state_off * 3;
  double *om = (dir == 0 ? am : bm) + f.grid_off;
  int32_t *oe = (dir == 0 ? ae : be) + f.grid_off;
  bool late = false;
  int32_t step = 0;
  for (int32_t q = 0; q < rg.num_chunks; ++q) {
    const int32_t c = rg.ChunkOf(q), slot = q % kChainSlots;
    if (!late) late = !WaitSlot(&full[slot], (unsigned)(q / kChainSlots) & 1u, wait_limit);
    late = __any_sync(kAll, late);
    if (late) break;
    const int32_t chunk_start = c * kPrepLevels * pitch;
    const int32_t l_lo = c * kPrepLevels, nl = min(l_lo + kPrepLevels, L) - l_lo;
    const bool fits = rg.ChunkItems(c) <= kSlotItems;
    const BandItem *src = fits ? ring + (size_t)slot * kSlotItems - chunk_start : rg.items0;
    for (int32_t k = 0; k < nl; ++k, ++step) {
      const int32_t l = dir == 0 ? l_lo + k : l_lo + nl - 1 - k;
      const int2 ls = lst[l];
      ProbState *cur = vals + (step & 1) * st_pad + 2;
      const ProbState *prv = vals + ((step & 1) ^ 1) * st_pad + 2;
      for (int32_t j = lane; j < ls.y; j += 32) {
        const BandItem it = src[ls.x + j];
        const int32_t s = it.s;
        // exp(dense score) of this state's label on frame l - 1
        double pm = 0.0;
        int32_t pe = kZeroExp;
        if (l >= 1) ExpToMantExp(BandDense(lp0, C, T, l - 1, it.label), &pm, &pe);
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
            // forward: alpha of the source; backward: beta * p of the destination
            t[d] = 0.0;
            x[d] = kZeroExp;
            if ((bits >> d) & 1u) {  // the bit names an arc of this graph
              const ProbState qs = dir == 0 ? prv[s - d] : prv[s + d];
              const BandArc arc = dir == 0 ? my_arcs[3 * s + d] : my_arcs[3 * (s + d) + d];
              t[d] = qs.m * arc.f;
              if (t[d] != 0.0) x[d] = qs.e + arc.k;
            }
          }
          const int32_t E = max(x[0], max(x[1], x[2]));
          const double sum =
              ScaleDown(t[0], x[0] - E) + ScaleDown(t[1], x[1] - E) + ScaleDown(t[2], x[2] - E);
          e = E;
          if (dir == 0) {
            e += pe;
            m = Renorm(sum * pm, &e);
          } else {
            m = Renorm(sum, &e);
          }
        }
        om[ls.x + j] = m;
        oe[ls.x + j] = e;
        ProbState r;
        r.pad = 0;
        if (dir == 0) {
          r.m = m;
          r.e = e;
          if (l == T + 1 && s == S - 1) {
            tot[i] = m == 0.0 ? -INFINITY : log(m) + (double)e * 0.69314718055994530942;
            BandTotal z;
            z.m = m;
            z.e = e;
            z.pad = 0;
            total[i] = z;
          }
        } else {  // what the level below adds: beta * p
          r.e = e + pe;
          r.m = Renorm(m * pm, &r.e);
        }
        cur[s] = r;
      }
      __syncwarp();  // the level is complete
    }
    if (lane == 0) rg.Issue();
  }
  if (late) {
    if (lane == 0) {
      atomicOr(status, kStatusLate);
      rg.Drain();
    }
    __syncwarp();
  }
  if (dir == 0 && lane == 0 && (*status & kStatusLate)) tot[i] = nan("");
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
template <bool kArcs>
__global__ void __launch_bounds__(128)
BandGrad(const BandInfo *__restrict__ infos, const BandArc *__restrict__ tabf,
         const float *__restrict__ lp, const BandItem *__restrict__ items,
         const int2 *__restrict__ lists, const double *__restrict__ am,
         const int32_t *__restrict__ ae, const double *__restrict__ bm,
         const int32_t *__restrict__ be, const int32_t *__restrict__ a_scale,
         const int32_t *__restrict__ b_scale, const BandTotal *__restrict__ total,
         const int32_t *__restrict__ unfit, const double *__restrict__ tot_grad,
         int32_t tot_grad_stride, float *__restrict__ grad_a, float *__restrict__ grad_b,
         const int32_t *__restrict__ grad_row0, int32_t grad_pitch, int32_t grad_col_off,
         int32_t C, int32_t st_pad) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int32_t i = blockIdx.y;
  const BandInfo f = infos[i];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int32_t S = f.num_states, T = f.frames;
  if (S == 0) return;
  const int32_t a = 1 + (blockIdx.x * 4 + warp) * kGradLevels;  // levels a .. b - 1
  if (a > T + 1) return;
  const int32_t b = min(a + kGradLevels, T + 2);
  const BandTotal z = total[i];
  if (z.m == 0.0) return;  // no path survives: all gradients are zero
  const double zinv = 1.0 / z.m;
  const bool exact = unfit[i] != 0;  // per-state exponents instead of per-level scales
  const int2 *lst = lists + f.level_off;
  const BandItem *items0 = items + f.grid_off;
  const double *am0 = am + f.grid_off, *bm0 = bm + f.grid_off;
  const int32_t *ae0 = ae + f.grid_off, *be0 = be + f.grid_off;
  const int32_t *as0 = a_scale + f.level_off, *bs0 = b_scale + f.level_off;
  const double tg = tot_grad[(int64_t)i * tot_grad_stride];
  const int64_t row0 = grad_row0 != nullptr ? grad_row0[i] : f.lp_row;
  const float *lp0 = lp + (int64_t)f.lp_row * C;
  // this warp's row of sums, one per column of the gradient (all zero between levels)
  const int32_t cols = C + grad_col_off;
  uint32_t *sums = reinterpret_cast<uint32_t *>(smem_raw) + (size_t)warp * cols;
  for (int32_t k = lane; k < cols; k += 32) sums[k] = 0u;
  __syncwarp();
  ProbState *prev = nullptr;  // alpha of the level before, state s at s + 2
  auto stage_alpha = [&](int32_t l) {
    const int32_t n = lst[l].y;
    const int64_t row = lst[l].x;
    for (int32_t j = lane; j < n; j += 32) {
      ProbState q;
      q.m = am0[row + j];
      q.e = exact ? ae0[row + j] : as0[l];
      q.pad = 0;
      prev[items0[row + j].s] = q;
    }
  };
  if (kArcs) {
    prev = reinterpret_cast<ProbState *>(smem_raw + (((size_t)4 * cols * sizeof(uint32_t) + 15) & ~(size_t)15)) +
           (size_t)warp * st_pad + 2;
    stage_alpha(a - 1);
    __syncwarp();
  }
  // the first 32 entries of the chunk's levels are requested together, before any is used
  int2 ls4[kGradLevels];
  BandItem it4[kGradLevels];
  double al4[kGradLevels], be4[kGradLevels];
#pragma unroll
  for (int u = 0; u < kGradLevels; ++u) {
    ls4[u] = a + u < b ? lst[a + u] : make_int2(0, 0);
    al4[u] = be4[u] = 0.0;
    it4[u].s = 0;
  }
#pragma unroll
  for (int u = 0; u < kGradLevels; ++u)
    if (lane < ls4[u].y) {
      it4[u] = items0[ls4[u].x + lane];
      al4[u] = am0[ls4[u].x + lane];
      be4[u] = bm0[ls4[u].x + lane];
    }
#pragma unroll
  for (int u = 0; u < kGradLevels; ++u) {
    const int32_t l = a + u;
    if (l >= b) break;
    const int32_t n = ls4[u].y;
    const int64_t row = ls4[u].x;
    const int32_t ea_l = as0[l], eb_l = bs0[l];
    for (int32_t j0 = 0; j0 < n; j0 += 32) {
      const int32_t j = j0 + lane;
      float g = 0.0f;
      int32_t key = -1 - lane;  // lanes with nothing to add are groups of their own
      if (j < n) {
        const BandItem it = j0 == 0 ? it4[u] : items0[row + j];
        const double alm = j0 == 0 ? al4[u] : am0[row + j], bem = j0 == 0 ? be4[u] : bm0[row + j];
        if (alm != 0.0 && bem != 0.0) {
          const int32_t ale = exact ? ae0[row + j] : ea_l, bee = exact ? be0[row + j] : eb_l;
          const int32_t col = it.label + grad_col_off;
          if (it.label != kNoLabel && it.label < C && col >= 0) {
            g = (float)(alm * bem * zinv * Pow2Clamp(ale + bee - z.e));
            key = col;
          }
          if (kArcs) {
            const int32_t s = it.s;
            double pm;
            int32_t pe;
            ExpToMantExp(BandDense(lp0, C, T, l - 1, it.label), &pm, &pe);
#pragma unroll
            for (int d = 0; d < 3; ++d) {
              if (!((it.inb >> d) & 1u)) continue;
              const ProbState q = prev[s - d];
              const BandArc arc = tabf[(int64_t)(f.state_off + s) * 3 + d];
              // two steps, so that no intermediate product leaves the range of a double
              const double post = (q.m * arc.f * pm) * (bem * zinv) *
                                  Pow2Clamp(q.e + arc.k + pe + bee - z.e);
              if (post != 0.0) atomicAdd(grad_a + arc.arc, (float)(tg * post));
            }
          }
        }
      }
      // States with the same label (the blank states of a CTC graph) add to the same
      // element.  Their posteriors are summed in this warp's row of shared memory, in fixed
      // point (2^-31 units: a sum of posteriors of one frame is at most 1) with integer
      // atomics - native in shared memory, and independent of the order of the additions -
      // then every lane takes the sum of its column out of the row, which leaves the row
      // zero again, and whoever got it adds it to the gradient.
      if (key >= 0) atomicAdd(&sums[key], __float2uint_rn(g * 2147483648.0f));
      __syncwarp();
      if (key >= 0) {
        const uint32_t fixed = atomicExch(&sums[key], 0u);
        if (fixed != 0u)
          atomicAdd(grad_b + (row0 + l - 1) * grad_pitch + key,
                    (float)tg * ((float)fixed * (1.0f / 2147483648.0f)));
      }
      __syncwarp();
    }
    if (kArcs) {
      __syncwarp();  // the level before has been read
      stage_alpha(l);
      __syncwarp();
    }
  }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
struct BandLayout {
  std::vector<BandInfo> infos;
  int64_t grid_elems = 0, reachable_states = 0, levels = 0;
  long long arc_frames = 0;
  int32_t max_states = 0, max_frames = 0;
  int32_t vit_threads = 32, vit_frames = 0, vit_batches = 0, xch_pad = 0;
  int32_t st_pad = 0, lv_pad = 0;
  size_t chain_smem = 0, exact_smem = 0, viterbi_smem = 0, prep_smem = 0;
  size_t off_infos, off_vf, off_vb, off_items, off_factors, off_lists, off_chunk_r, off_keep, off_cutoffs, off_am, off_ae, off_bm,
      off_be, off_a_scale, off_b_scale, off_total, off_unfit, off_totals, off_status,
      total_bytes;  // off_status = off_totals + 40
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
    f.pitch = 32 * (f.num_states / 32 + 1);
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
    {
      // States that can survive: level l (0 .. R = T + 1) holds state s only if the start
      // state reaches it (arcs advance by at most two states: s <= 2 l) and it reaches
      // the last state m = S - 1 at level R (m - s <= 2 (R - l)).  Summed over the
      // levels, with k = m / 2: the grid without two triangles of k (k + 1) states.
      const int64_t S = f.num_states, m = S - 1, R = (int64_t)f.frames + 1, k = m / 2;
      L->reachable_states += (S > 0 && 2 * R >= m) ? 2 * k * (k + 1) + (R - 2 * k - 1) * m + R + 1
                                              : (R + 1) * S;
    }
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
  // BandViterbi: frames per batch (even, at most 16) so that at least two batches of rows
  // fit in shared memory, up to three batches within ~100 KB so that two CTAs share an SM
  {
    const size_t row_bytes = sizeof(float) * (size_t)a->num_classes;
    int32_t F = 16;
    while (F > 2 && 2 * F * row_bytes > kBandSmemBudget - 8192) F >>= 1;
    L->vit_frames = F;
    L->vit_batches = (int32_t)std::max<size_t>(
        2, std::min<size_t>(3, (100 * 1024) / std::max<size_t>(F * row_bytes, 1)));
    const int32_t own_states = (32 - F / 2) * kVitK;
    const int32_t warps = std::max(1, CeilDiv(std::max(L->max_states, 1), own_states));
    L->vit_threads = 32 * warps;
    L->xch_pad = (warps * own_states + 4 * kVitK * (F / 2) + 3) & ~3;
    L->viterbi_smem = (size_t)L->vit_batches * F * row_bytes + sizeof(float) * 2 * (size_t)L->xch_pad;
    if (warps > kVitMaxWarps || 2 * F * row_bytes > kBandSmemBudget - 8192) {
      L->ok = false;
      L->why = "too many states or classes for the Viterbi kernel";
    }
  }
  L->st_pad = ((L->max_states + 4) + 15) & ~15;
  L->lv_pad = (L->max_frames + 2 + 3) & ~3;
  L->prep_smem = (size_t)4 * (8 * L->st_pad + 64 * (kPrepLevels + 2));
  L->exact_smem = sizeof(BandItem) * kChainSlots * kSlotItems + sizeof(int2) * (size_t)L->lv_pad +
                  sizeof(ProbState) * 2 * (size_t)L->st_pad;
  L->chain_smem = sizeof(BandFactor) * kChainSlots * kFacSlot;
  if (L->max_states > kBandMaxStates) {
    L->ok = false;
    L->why = "a graph has more than 512 states";
  } else if (a->num_classes % 4 != 0 || (reinterpret_cast<uintptr_t>(a->log_probs) & 15) != 0) {
    L->ok = false;
    L->why = "rows of the log-prob matrix are not 16-byte aligned";
  } else if (L->chain_smem > kBandSmemBudget || L->exact_smem > kBandSmemBudget) {
    L->ok = false;
    L->why = "too many frames, states or classes for the shared memory of the recursions";
  } else if (L->max_frames + 2 > kChainMaxChunks * kPrepLevels) {
    L->ok = false;
    L->why = "a sequence has more than 65534 frames";
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
  L->off_lists = take(sizeof(int2) * (size_t)levels);
  L->off_chunk_r = take(sizeof(int32_t) * (size_t)levels);
  L->off_keep = take(sizeof(uint16_t) * 32 * (size_t)levels);
  L->off_factors = take(sizeof(BandFactor) * (size_t)grid);
  L->off_cutoffs = take(sizeof(float) * a->num_fsas);
  L->off_am = take(sizeof(double) * (size_t)grid);
  L->off_ae = take(sizeof(int32_t) * (size_t)grid);
  L->off_bm = take(sizeof(double) * (size_t)grid);
  L->off_be = take(sizeof(int32_t) * (size_t)grid);
  L->off_a_scale = take(sizeof(int32_t) * (size_t)levels);
  L->off_b_scale = take(sizeof(int32_t) * (size_t)levels);
  L->off_total = take(sizeof(BandTotal) * a->num_fsas);
  L->off_unfit = take(sizeof(int32_t) * a->num_fsas);
  L->off_totals = take(64);  // five 64-bit totals, then the status word
  L->off_status = L->off_totals + 5 * sizeof(long long);
  L->total_bytes = off;
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

static int32_t LaunchBandChains(const BandLayout &L, const k2b200_band_loss_args *args, char *ws,
                                double *tot_scores, cudaStream_t stream) {
  K2B_CUDA_OK(cudaFuncSetAttribute(BandChainLists, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)L.chain_smem));
  K2B_CUDA_OK(cudaFuncSetAttribute(BandChainExact, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)L.exact_smem));
  dim3 grid(2, args->num_fsas);
  const BandInfo *infos = reinterpret_cast<const BandInfo *>(ws + L.off_infos);
  const BandItem *items = reinterpret_cast<const BandItem *>(ws + L.off_items);
  const int2 *lists = reinterpret_cast<const int2 *>(ws + L.off_lists);
  double *am = reinterpret_cast<double *>(ws + L.off_am), *bm = reinterpret_cast<double *>(ws + L.off_bm);
  BandTotal *total = reinterpret_cast<BandTotal *>(ws + L.off_total);
  int32_t *unfit = reinterpret_cast<int32_t *>(ws + L.off_unfit);
  int32_t *status = reinterpret_cast<int32_t *>(ws + L.off_status);
  { BandChainLists<<<grid, 32, L.chain_smem, stream>>>(
      infos, reinterpret_cast<const BandFactor *>(ws + L.off_factors),
      reinterpret_cast<const int32_t *>(ws + L.off_chunk_r), am, bm,
      reinterpret_cast<int32_t *>(ws + L.off_a_scale),
      reinterpret_cast<int32_t *>(ws + L.off_b_scale), tot_scores, total, unfit, status,
      CopyWaitLimit()); NoteLaunch(); }
  { BandChainExact<<<grid, 32, L.exact_smem, stream>>>(
      infos, reinterpret_cast<const BandArc *>(args->band_arcs), args->log_probs,
      args->num_classes, items, lists, am, reinterpret_cast<int32_t *>(ws + L.off_ae), bm,
      reinterpret_cast<int32_t *>(ws + L.off_be), tot_scores, total, unfit, status, L.st_pad,
      L.lv_pad, CopyWaitLimit()); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

}  // namespace k2b

using namespace k2b;

extern "C" {

void k2b200_debug_set_copy_wait_limit(int32_t polls) { SetCopyWaitLimit(polls); }

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
  // unfit words, totals and the status word lie one after the other: one clear for the first
  // pass (a repeated pass clears the first two again, not the status of the Viterbi kernels)
  K2B_CUDA_OK(cudaMemsetAsync(ws + L.off_unfit, 0, L.off_totals + 64 - L.off_unfit, stream));
  {
    PhaseTimer timer(kPhaseViterbi, stream);
    NotePhaseKernel(kPhaseViterbi, "BandViterbi");
    K2B_CUDA_OK(cudaFuncSetAttribute(BandViterbi, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)L.viterbi_smem));
    dim3 grid(2, args->num_fsas);
    { BandViterbi<<<grid, L.vit_threads, L.viterbi_smem, stream>>>(
        reinterpret_cast<const BandInfo *>(ws + L.off_infos),
        reinterpret_cast<const BandState *>(args->band_states), args->log_probs,
        args->num_classes, reinterpret_cast<float *>(ws + L.off_vf),
        reinterpret_cast<float *>(ws + L.off_vb), L.vit_frames, L.vit_batches, L.xch_pad,
        CopyWaitLimit(), reinterpret_cast<int32_t *>(ws + L.off_status)); NoteLaunch(); }
    K2B_CUDA_OK(cudaGetLastError());
  }
  // The lattice is never built, but its size still decides the beam
  // (intersect_dense.cu:300-320).  The grid bounds it (for the states: the part of the grid
  // that lies both behind the start state and before the last one): the host reads the
  // counts only when that bound does not already satisfy the limits, and after it has
  // launched the recursions, which in the rare case of a reduction run again.
  const bool need_count = L.reachable_states > args->max_states || L.arc_frames > args->max_arcs;
  float beam = args->output_beam;
  bool join_side = false;
  struct JoinOnExit {  // also on error returns: the caller may free the buffer being cleared
    cudaStream_t main;
    bool *armed;
    ~JoinOnExit() { if (*armed) SideJoin(main); }
  } join_guard{stream, &join_side};
  for (int iter = 0;; ++iter) {
    SideReadBackScope readback;
    if (iter > 0) {
      K2B_CUDA_OK(cudaMemsetAsync(ws + L.off_totals, 0, 5 * sizeof(long long), stream));
      K2B_CUDA_OK(cudaMemsetAsync(ws + L.off_unfit, 0, sizeof(int32_t) * args->num_fsas, stream));
    }
    cudaStream_t side = nullptr;
    {
      PhaseTimer timer(kPhasePrune, stream);
      NotePhaseKernel(kPhasePrune, "BandKeep+BandPrep");
      dim3 kgrid(CeilDiv(L.max_frames + 2, 4 * kKeepLevels), args->num_fsas);
#define K2B_BAND_KEEP(KK)                                                                   \
      { BandKeep<KK><<<kgrid, 128, 0, stream>>>(                                                \
          reinterpret_cast<const BandInfo *>(ws + L.off_infos), args->a_row_splits2,            \
          reinterpret_cast<const float *>(ws + L.off_vf),                                       \
          reinterpret_cast<const float *>(ws + L.off_vb), beam,                                 \
          reinterpret_cast<uint16_t *>(ws + L.off_keep),                                        \
          reinterpret_cast<float *>(ws + L.off_cutoffs),                                        \
          reinterpret_cast<unsigned long long *>(ws + L.off_totals),                            \
          L.arc_frames > args->max_arcs ? 1 : 0); NoteLaunch(); }
      if (L.max_states <= 256) K2B_BAND_KEEP(8) else K2B_BAND_KEEP(kPrepK)
#undef K2B_BAND_KEEP
      // the host reads the counts behind BandKeep, while what follows runs
      if (need_count) {
        K2B_FORWARD(SideFork(stream, &side));
        K2B_FORWARD(readback.Begin(ws + L.off_totals, sizeof(long long) * 6));
      }
      dim3 grid(CeilDiv(L.max_frames + 2, 4 * kPrepSub), args->num_fsas);
      { BandPrep<<<grid, 128, L.prep_smem, stream>>>(
          reinterpret_cast<const BandInfo *>(ws + L.off_infos),
          reinterpret_cast<const BandState *>(args->band_states),
          reinterpret_cast<const BandArc *>(args->band_arcs),
          reinterpret_cast<const uint16_t *>(ws + L.off_keep), args->log_probs,
          args->num_classes, reinterpret_cast<const float *>(ws + L.off_vf),
          reinterpret_cast<const float *>(ws + L.off_vb),
          reinterpret_cast<const float *>(ws + L.off_cutoffs),
          reinterpret_cast<BandItem *>(ws + L.off_items),
          reinterpret_cast<BandFactor *>(ws + L.off_factors),
          reinterpret_cast<int2 *>(ws + L.off_lists),
          reinterpret_cast<int32_t *>(ws + L.off_chunk_r),
          reinterpret_cast<int32_t *>(ws + L.off_unfit), L.st_pad); NoteLaunch(); }
      K2B_CUDA_OK(cudaGetLastError());
    }
    if (iter == 0 && args->zero_fill != nullptr && args->zero_fill_bytes > 0) {
      // behind BandPrep, beside the recursions (one warp per graph and direction: the SMs
      // are all but idle); joined below
      K2B_FORWARD(SideFork(stream, &side));
      K2B_CUDA_OK(cudaMemsetAsync(args->zero_fill, 0, args->zero_fill_bytes, side));
      join_side = true;
    }
    {
      PhaseTimer timer(kPhaseChain, stream);
      NotePhaseKernel(kPhaseChain, "BandChainLists");
      K2B_FORWARD(LaunchBandChains(L, args, ws, tot_scores, stream));
    }
    if (!need_count) break;
    long long h_totals[6];
    K2B_FORWARD(readback.End(h_totals));
    K2B_REQUIRE((h_totals[5] & kStatusLate) == 0,
                "a copy of log-prob rows into shared memory did not complete in time");
    const float beam_before = beam;
    if (!BandReduceBeam(args, h_totals, &beam)) break;
    K2B_LOG(kLogInfo, "band loss: %lld states / %lld arcs exceed max_states %d / max_arcs %d, "
            "output beam %g -> %g", h_totals[0], h_totals[2], args->max_states, args->max_arcs,
            (double)beam_before, (double)beam);
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
  K2B_REQUIRE(tot_grad && grad_b, "NULL device pointer");
  K2B_REQUIRE(grad_col_off == 0 || grad_col_off == 1, "grad_col_off must be 0 or 1");
  char *ws = reinterpret_cast<char *>(workspace);
  PhaseTimer timer(kPhaseGrad, stream);
  NotePhaseKernel(kPhaseGrad, "BandGrad");
  dim3 grid(CeilDiv(L.max_frames + 1, 4 * kGradLevels), args->num_fsas);
#define K2B_BAND_GRAD(ARCS, SMEM)                                                             \
  { BandGrad<ARCS><<<grid, 128, SMEM, stream>>>(                                              \
      reinterpret_cast<const BandInfo *>(ws + L.off_infos),                                   \
      reinterpret_cast<const BandArc *>(args->band_arcs), args->log_probs,                    \
      reinterpret_cast<const BandItem *>(ws + L.off_items),                                   \
      reinterpret_cast<const int2 *>(ws + L.off_lists),                                       \
      reinterpret_cast<const double *>(ws + L.off_am),                                        \
      reinterpret_cast<const int32_t *>(ws + L.off_ae),                                       \
      reinterpret_cast<const double *>(ws + L.off_bm),                                        \
      reinterpret_cast<const int32_t *>(ws + L.off_be),                                       \
      reinterpret_cast<const int32_t *>(ws + L.off_a_scale),                                  \
      reinterpret_cast<const int32_t *>(ws + L.off_b_scale),                                  \
      reinterpret_cast<const BandTotal *>(ws + L.off_total),                                  \
      reinterpret_cast<const int32_t *>(ws + L.off_unfit), tot_grad, tot_grad_stride, grad_a, \
      grad_b, grad_row0, grad_pitch, grad_col_off, args->num_classes, L.st_pad); NoteLaunch(); }
  const size_t sums_bytes =
      (sizeof(uint32_t) * 4 * (size_t)(args->num_classes + grad_col_off) + 15) & ~(size_t)15;
  K2B_REQUIRE(sums_bytes + sizeof(ProbState) * 4 * (size_t)L.st_pad <= kBandSmemBudget,
              "too many classes for the gradient kernel");
  if (grad_a != nullptr) {
    const size_t smem = sums_bytes + sizeof(ProbState) * 4 * (size_t)L.st_pad;
    K2B_CUDA_OK(cudaFuncSetAttribute(BandGrad<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)smem));
    K2B_BAND_GRAD(true, smem)
  } else {
    K2B_CUDA_OK(cudaFuncSetAttribute(BandGrad<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)sums_bytes));
    K2B_BAND_GRAD(false, sums_bytes)
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
  if (*status & kStatusLate)
    K2B_LOG(kLogWarning, "band loss: a bounded wait for a copy into shared memory gave up; the "
            "results of that call are invalid");
  return kOk;
}

}  // extern "C"

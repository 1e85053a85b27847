// Pruned intersection of decoding graphs with a DenseFsaVec: a frame-synchronous
// beam search with a dynamic beam per sequence, followed window by window by a
// backward pass that applies the output beam.  Behaviour follows
// k2/csrc/intersect_dense_pruned.cu:41-1694 (MultiGraphDenseIntersectPruned with
// online_decoding == false) as its CPU build executes it:
//   - the states of frame t+1 are numbered in the order of the first arc of frame t
//     (in [state][arc] order) that reaches them above the cutoff; the reference
//     inserts into a hash sequentially on CPU, so the first arc wins (:1005-1028);
//   - the search beam per sequence moves towards `search_beam`, shrinks while more
//     than max_active states are alive and grows while fewer than min_active are,
//     in the reference's mixed float/double arithmetic (:687-767);
//   - every 20 frames the last 30 are pruned backwards (:164-199, :1373-1634); the
//     backward thread of the reference never changes what the forward pass reads,
//     so the windows are simply run in order.
//
// Sequences are independent, so one team of CTAs (a thread-block cluster of 1 to 8)
// owns one sequence from the first frame to the last: no host round trip per frame,
// no hash (a direct table per sequence, indexed by graph state, plays its role) and
// no kernel waits on another.  States and arcs of all frames of a sequence live in
// one arena, frame after frame, so the pruned result is already in lattice order and
// the output pass is a copy.
#include <algorithm>
#include <climits>
#include <cmath>
#include <cstring>
#include <vector>

#include <cooperative_groups.h>

#include "common.cuh"
#include "../../include/k2b200.h"

namespace cg = cooperative_groups;

namespace k2b {
namespace {

constexpr int kSearchThreads = 1024;
constexpr int kWindow = 30;       // frames pruned per backward phase (:171)
constexpr int kWindowShift = 20;  // frames between two phases (:172)

// order-preserving float <-> int (as k2/csrc/utils.h:406-414)
__device__ __forceinline__ int32_t OrderedInt(float f) {
  int32_t i = __float_as_int(f);
  return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float OrderedFloat(int32_t i) {
  return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff);
}

struct SearchArgs {
  // graphs
  const int32_t *a_rs1, *a_rs2;
  const Arc *a_arcs;
  int32_t a_stride;  // 1: one graph per sequence, 0: one graph shared by all
  int32_t a_states;  // states of all graphs together
  // dense scores
  const float *scores;
  int32_t rows, cols;
  const int32_t *b_rs;
  int32_t num_seqs, T;  // T = rows of the longest sequence
  float search_beam, output_beam, min_active, max_active;
  int32_t allow_partial;
  // arenas, [num_seqs] slices of cap_s (+1) and cap_a elements
  int64_t cap_s, cap_a;
  int32_t *st_astate, *st_fwd, *st_arc0, *st_new, *st_cnt;
  float *st_bwd;
  int32_t *arc_aidx, *arc_dest;
  float *arc_ll, *arc_end;
  uint8_t *arc_keep;
  unsigned long long *winner;  // [num_seqs * a_states] (shared) or [a_states]
  int32_t *frame_s0, *frame_a0;  // [num_seqs][T + 2]
  int32_t *seq_out;           // [num_seqs][4]: states, arcs, extra final state, status
};

enum : int32_t { kSeqOk = 0, kSeqOverflow = 1, kSeqManyFinal = 2 };

// The CTAs that work on one sequence: a thread-block cluster (of one CTA when there are
// enough sequences to fill the GPU).  Arena data is exchanged through global memory,
// ordered by the cluster barrier; scan totals and maxima through distributed shared
// memory.  Item k of a pass is handled by team thread k mod team size, and the CTAs
// of a cluster are always co-resident, so the barrier cannot wait for an unscheduled
// CTA.
struct Shared {
  int32_t scan[65];
  float fmax[33];
  unsigned long long scan2[65];
  unsigned long long team_l[2];
  int32_t team_i[2];  // this CTA's contribution to the team-wide scan / or
  float team_f[2];    // ... and to the team-wide max; two slots used alternately
  int32_t phase_i, phase_f, phase_l;
  int32_t new_s0[kWindow], new_a0[kWindow];  // used by the first thread of the team only
  int32_t wbest[kSearchThreads / 32][32], wcnt[kSearchThreads / 32][32];  // per warp
  float cutoff;
  float beam;
};

struct Team {
  cg::cluster_group cluster;
  Shared *sh;
  int32_t rank, size;     // this CTA within the cluster
  int32_t tid, threads;   // this thread within the team

  __device__ Team(Shared *shared) : cluster(cg::this_cluster()), sh(shared) {
    rank = (int32_t)cluster.block_rank();
    size = (int32_t)cluster.num_blocks();
    tid = rank * kSearchThreads + (int32_t)threadIdx.x;
    threads = size * kSearchThreads;
  }
  __device__ __forceinline__ void Sync() const {
    if (size == 1) __syncthreads(); else cluster.sync();
  }

  // exclusive scan of one int per team thread; every thread gets the total
  __device__ int32_t Scan(int32_t v, int32_t *total) const {
    int32_t *s = sh->scan;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int32_t inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int32_t o = __shfl_up_sync(0xffffffffu, inc, d);
      if (lane >= d) inc += o;
    }
    if (lane == 31) s[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      int32_t w = s[lane];
      int32_t winc = w;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        int32_t o = __shfl_up_sync(0xffffffffu, winc, d);
        if (lane >= d) winc += o;
      }
      s[32 + lane] = winc - w;
      if (lane == 31) s[64] = winc;
    }
    __syncthreads();
    int32_t ex = s[32 + warp] + inc - v;
    int32_t all = s[64];
    if (size == 1) {
      __syncthreads();  // s is reused by the next call
      *total = all;
      return ex;
    }
    // a slot is rewritten two calls later, after a cluster barrier that every CTA
    // reaches only when it has read the slot
    const int32_t slot = sh->phase_i & 1;
    if (threadIdx.x == 0) sh->team_i[slot] = all;
    cluster.sync();
    int32_t before = 0, sum = 0;
    for (int32_t r = 0; r < size; ++r) {
      const int32_t x = *cluster.map_shared_rank(&sh->team_i[slot], r);
      sum += x;
      if (r < rank) before += x;
    }
    __syncthreads();
    if (threadIdx.x == 0) sh->phase_i += 1;
    __syncthreads();
    *total = sum;
    return before + ex;
  }

  // the same for a pair of counts, both below 2^31 in total, packed into 64 bits
  __device__ int32_t Scan2(int32_t a, int32_t b, int32_t *ex_b, int32_t *total_a,
                           int32_t *total_b) const {
    unsigned long long *s = sh->scan2;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned long long v = (unsigned long long)(uint32_t)a | ((unsigned long long)(uint32_t)b << 32);
    unsigned long long inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      unsigned long long o = __shfl_up_sync(0xffffffffu, inc, d);
      if (lane >= d) inc += o;
    }
    if (lane == 31) s[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      unsigned long long w = s[lane];
      unsigned long long winc = w;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        unsigned long long o = __shfl_up_sync(0xffffffffu, winc, d);
        if (lane >= d) winc += o;
      }
      s[32 + lane] = winc - w;
      if (lane == 31) s[64] = winc;
    }
    __syncthreads();
    unsigned long long ex = s[32 + warp] + inc - v;
    unsigned long long all = s[64];
    if (size == 1) {
      __syncthreads();
    } else {
      const int32_t slot = sh->phase_l & 1;
      if (threadIdx.x == 0) sh->team_l[slot] = all;
      cluster.sync();
      unsigned long long before = 0, sum = 0;
      for (int32_t r = 0; r < size; ++r) {
        const unsigned long long x = *cluster.map_shared_rank(&sh->team_l[slot], r);
        sum += x;
        if (r < rank) before += x;
      }
      __syncthreads();
      if (threadIdx.x == 0) sh->phase_l += 1;
      __syncthreads();
      ex += before;
      all = sum;
    }
    *ex_b = (int32_t)(ex >> 32);
    *total_a = (int32_t)(all & 0xffffffffu);
    *total_b = (int32_t)(all >> 32);
    return (int32_t)(ex & 0xffffffffu);
  }

  __device__ float Max(float v) const {
    float *s = sh->fmax;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
    if (lane == 0) s[warp] = v;
    __syncthreads();
    if (warp == 0) {
      float w = s[lane];
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) w = fmaxf(w, __shfl_xor_sync(0xffffffffu, w, d));
      if (lane == 0) s[32] = w;
    }
    __syncthreads();
    float r = s[32];
    const int32_t slot = sh->phase_f & 1;
    if (threadIdx.x == 0) sh->team_f[slot] = r;
    Sync();  // also orders the global writes made before the call
    if (size > 1) {
      for (int32_t k = 0; k < size; ++k)
        r = fmaxf(r, *cluster.map_shared_rank(&sh->team_f[slot], k));
    }
    __syncthreads();
    if (threadIdx.x == 0) sh->phase_f += 1;
    __syncthreads();
    return r;
  }

  // true when `v` is non-zero on any thread of the team
  __device__ bool Any(int32_t v) const {
    int32_t total;
    Scan(v != 0, &total);
    return total != 0;
  }
};

// Views of one sequence's slices of the arenas.
struct SeqView {
  int32_t *st_astate, *st_fwd, *st_arc0, *st_new, *st_cnt;
  float *st_bwd;
  int32_t *arc_aidx, *arc_dest;
  float *arc_ll, *arc_end;
  uint8_t *arc_keep;
  unsigned long long *winner;
  int32_t *frame_s0, *frame_a0;
};

__device__ __forceinline__ SeqView ViewOf(const SearchArgs &g, int32_t seq) {
  SeqView v;
  const int64_t so = (int64_t)seq * (g.cap_s + 1), ao = (int64_t)seq * g.cap_a;
  v.st_astate = g.st_astate + so;
  v.st_fwd = g.st_fwd + so;
  v.st_arc0 = g.st_arc0 + so;
  v.st_new = g.st_new + so;
  v.st_cnt = g.st_cnt + so;
  v.st_bwd = g.st_bwd + so;
  v.arc_aidx = g.arc_aidx + ao;
  v.arc_dest = g.arc_dest + ao;
  v.arc_ll = g.arc_ll + ao;
  v.arc_end = g.arc_end + ao;
  v.arc_keep = g.arc_keep + ao;
  // the reference's hash key is dest_state_idx01 + seq * stride with the stride 0
  // for per-sequence graphs (:118-127): the same index works for a direct table
  v.winner = g.winner + (g.a_stride ? 0 : (int64_t)seq * g.a_states);
  v.frame_s0 = g.frame_s0 + (int64_t)seq * (g.T + 2);
  v.frame_a0 = g.frame_a0 + (int64_t)seq * (g.T + 2);
  return v;
}

// The search beam and the cutoff of frame t (:718-766).  `dyn` is the beam carried
// from the previous frame; products with the literals 0.8, 0.2 and 1.25 are double
// products in the reference and are rounded to float on assignment.
__device__ float NextBeam(float dyn, float best, int32_t active, int32_t t, int32_t final_t,
                          const SearchArgs &g, float *cutoff) {
  const float default_beam = g.search_beam, max_active = g.max_active,
              min_active = g.min_active;
  float cur_min = min_active;
  if (t + 5 >= final_t) cur_min = fmaxf(min_active, max_active / 2);
  if ((float)active <= max_active) {
    if ((float)active >= cur_min || active == 0) {
      dyn = (float)(0.8 * (double)dyn + 0.2 * (double)default_beam);
    } else {
      if (dyn < default_beam) dyn = default_beam;
      dyn = (float)((double)dyn * 1.25);
    }
  } else if (t + 5 < final_t) {
    if (dyn > default_beam) dyn = default_beam;
    dyn = (float)((double)dyn * 0.8);
  }
  if (t == final_t - 1) dyn = 1.0e+10f;
  *cutoff = best - dyn;
  return dyn;
}

constexpr int kPer = 8;      // consecutive arcs per thread in the compaction pass
constexpr int kPerScan = 8;  // ... and where the new states are numbered
constexpr int kBatch = 4;    // arcs whose loads a thread issues together
constexpr int kExpand = 2;   // ... in the arc expansion

// Entries of the direct table that replaces the reference's hash: the frame in the
// high word, so that entries of earlier frames lose against any entry of this frame
// and the table never needs clearing; in the low word either an arc (a smaller arc
// index gives a larger value, so atomicMax keeps the first arc) or, with the top bit
// set, the number of the state that arc created.
__device__ __forceinline__ unsigned long long ArcEntry(int32_t t, int32_t q) {
  return ((unsigned long long)(uint32_t)(t + 1) << 32) | (uint32_t)(0x7fffffff - q);
}
__device__ __forceinline__ unsigned long long StateEntry(int32_t t, int32_t j) {
  return ((unsigned long long)(uint32_t)(t + 1) << 32) | 0x80000000u | (uint32_t)j;
}

// One step of the search (GetArcs + PropagateForward, :778-1153): expands the na arcs
// leaving the ns states of frame t at [s0, s0 + ns) - their arc ranges (st_arc0,
// starting at a0) were laid out when the states were created - and creates the states
// of frame t + 1 behind them, with their arc ranges.  Returns false when an arena is
// full.  *ns_next / *na_next: states of frame t + 1 and the arcs leaving them.
__device__ bool SearchStep(const SearchArgs &g, const SeqView &v, const Team &tm, int32_t seq,
                           int32_t t, int32_t final_t, int32_t row0, int32_t s0, int32_t ns,
                           int32_t a0, int32_t na, int32_t *ns_next, int32_t *na_next) {
  Shared *sh = tm.sh;
  const float kNegInf = -INFINITY;
  if ((int64_t)a0 + na > g.cap_a) return false;

  // graph of this sequence: its final state, for allow_partial (:861-871)
  const int32_t gi = seq * g.a_stride;
  const int32_t g_final = g.a_rs1[gi + 1] - 1;
  bool redirect = false;
  if (g.allow_partial && t == final_t - 1) {
    // is there any arc with label -1 among the arcs expanded on this frame (:839-857)
    int32_t has = 0;
    for (int32_t k = tm.tid; k < ns; k += tm.threads) {
      const int32_t as = v.st_astate[s0 + k];
      for (int32_t a = g.a_rs2[as]; a < g.a_rs2[as + 1]; ++a) has |= (g.a_arcs[a].label == -1);
    }
    redirect = !tm.Any(has);
  }

  // arcs: scores, destination (as a graph state) and the best end score (:858-905).
  // A warp takes 32 consecutive states; its lanes walk the arcs of those states as
  // one flat range and find the state of an arc by a search over the 32 range
  // starts held in registers, so the work per lane is even whatever the out-degrees.
  // (a row past the end is only asked for by a malformed graph whose arcs with
  // label -1 do not end in a state without arcs)
  const bool row_ok = row0 + t < g.rows;
  const float *row = g.scores + (int64_t)(row_ok ? row0 + t : 0) * g.cols;
  float best = kNegInf;
  {
    const int lane = threadIdx.x & 31;
    const int32_t team_warp = tm.tid >> 5, team_warps = tm.threads >> 5;
    for (int32_t kb = team_warp * 32; kb < ns; kb += team_warps * 32) {
      const int32_t k = kb + lane;
      int32_t as = 0, fwd = 0, p0 = 0x7fffffff, ga0 = 0;
      if (k < ns) {
        as = v.st_astate[s0 + k];
        fwd = v.st_fwd[s0 + k];
        p0 = v.st_arc0[s0 + k];
        ga0 = g.a_rs2[as];
      }
      const int32_t first = __shfl_sync(0xffffffffu, p0, 0);
      const int32_t last = v.st_arc0[s0 + min(kb + 32, ns)];
      for (int32_t pb = first; pb < last; pb += 32 * kExpand) {
        int32_t p[kExpand], j[kExpand], aidx[kExpand];
        Arc arc[kExpand];
#pragma unroll
        for (int i = 0; i < kExpand; ++i) {
          p[i] = pb + i * 32 + lane;
          // largest j with p0[j] <= p (p0 is non-decreasing; absent states hold +inf)
          int32_t lo = 0;
#pragma unroll
          for (int step = 16; step > 0; step >>= 1) {
            const int32_t cand = __shfl_sync(0xffffffffu, p0, lo + step);
            if (cand <= p[i]) lo += step;
          }
          j[i] = lo;
          const int32_t jp0 = __shfl_sync(0xffffffffu, p0, lo);
          const int32_t jga0 = __shfl_sync(0xffffffffu, ga0, lo);
          aidx[i] = p[i] < last ? jga0 + (p[i] - jp0) : -1;
        }
#pragma unroll
        for (int i = 0; i < kExpand; ++i) {
          if (aidx[i] >= 0) arc[i] = g.a_arcs[aidx[i]];
        }
#pragma unroll
        for (int i = 0; i < kExpand; ++i) {
          const int32_t jas = __shfl_sync(0xffffffffu, as, j[i]);
          const int32_t jfwd = __shfl_sync(0xffffffffu, fwd, j[i]);
          if (aidx[i] >= 0) {
            const uint32_t col = (uint32_t)(arc[i].label + 1);
            float acoustic = (row_ok && col < (uint32_t)g.cols) ? row[col] : kNegInf;
            int32_t dest = jas + arc[i].dest - arc[i].src;
            if (redirect) {
              dest = g_final;
              acoustic = 0.0f;
            }
            const float ll = acoustic + arc[i].score;
            const float end = OrderedFloat(jfwd) + ll;
            v.arc_aidx[p[i]] = aidx[i];
            v.arc_ll[p[i]] = ll;
            v.arc_dest[p[i]] = dest;
            v.arc_end[p[i]] = end;
            best = fmaxf(best, end);
          }
        }
      }
    }
  }
  best = tm.Max(best);  // also makes the arc records visible to the team
  if (threadIdx.x == 0) sh->beam = NextBeam(sh->beam, best, ns, t, final_t, g, &sh->cutoff);
  __syncthreads();
  const float cutoff = sh->cutoff;

  // first arc above the cutoff into every destination state (:1005-1028)
  for (int32_t q0 = tm.tid; q0 < na; q0 += kBatch * tm.threads) {
    float end[kBatch];
    int32_t dest[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int32_t q = q0 + i * tm.threads;
      end[i] = q < na ? v.arc_end[a0 + q] : kNegInf;
      dest[i] = q < na ? v.arc_dest[a0 + q] : 0;
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      if (end[i] > cutoff) atomicMax(&v.winner[dest[i]], ArcEntry(t, q0 + i * tm.threads));
    }
  }
  tm.Sync();
  // which arcs created their destination state, and how many arcs leave it: one
  // byte per arc (0: none; else out-degree + 1, 255 standing for "254 or more")
  for (int32_t q0 = tm.tid; q0 < na; q0 += kBatch * tm.threads) {
    float end[kBatch];
    int32_t dest[kBatch];
    unsigned long long w[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int32_t q = q0 + i * tm.threads;
      end[i] = q < na ? v.arc_end[a0 + q] : kNegInf;
      dest[i] = q < na ? v.arc_dest[a0 + q] : 0;
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) w[i] = end[i] > cutoff ? v.winner[dest[i]] : 0ull;
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int32_t q = q0 + i * tm.threads;
      if (q < na) {
        uint8_t flag = 0;
        if (end[i] > cutoff && w[i] == ArcEntry(t, q)) {
          const int32_t deg = g.a_rs2[dest[i] + 1] - g.a_rs2[dest[i]];
          flag = (uint8_t)(min(deg, 254) + 1);
        }
        v.arc_keep[a0 + q] = flag;
      }
    }
  }
  tm.Sync();
  // number the new states in the order of their winning arcs (:1031-1100) and lay
  // out the arcs that will leave them
  const int32_t s1 = s0 + ns, a1 = a0 + na;
  int32_t nn = 0, na1 = 0;
  for (int32_t base = 0; base < na; base += tm.threads * kPerScan) {
    const int32_t q0 = base + tm.tid * kPerScan;
    int32_t deg[kPerScan];
    int32_t won = 0, degs = 0;  // bit i: arc q0 + i created its destination state
#pragma unroll
    for (int i = 0; i < kPerScan; ++i) {
      deg[i] = 0;
      const int32_t flag = q0 + i < na ? v.arc_keep[a0 + q0 + i] : 0;
      if (flag) {
        won |= 1 << i;
        deg[i] = flag - 1;
      }
    }
    if (won) {
#pragma unroll
      for (int i = 0; i < kPerScan; ++i) {
        if (deg[i] == 254) {
          const int32_t d = v.arc_dest[a0 + q0 + i];
          deg[i] = g.a_rs2[d + 1] - g.a_rs2[d];
        }
        degs += deg[i];
      }
    }
    int32_t tot, dtot, arcs_before;
    int32_t j = nn + tm.Scan2(__popc(won), degs, &arcs_before, &tot, &dtot);
    arcs_before += na1;
    if (won) {
#pragma unroll
      for (int i = 0; i < kPerScan; ++i) {
        if (won >> i & 1) {
          const int32_t d = v.arc_dest[a0 + q0 + i];
          const int32_t first = a1 + arcs_before;
          if ((int64_t)s1 + j < g.cap_s && (int64_t)first + deg[i] <= g.cap_a) {
            v.st_astate[s1 + j] = d;
            v.st_fwd[s1 + j] = OrderedInt(kNegInf);
            v.st_arc0[s1 + j] = first;
            v.winner[d] = StateEntry(t, j);
          }
          arcs_before += deg[i];
          ++j;
        }
      }
    }
    nn += tot;
    na1 += dtot;
  }
  if ((int64_t)s1 + nn > g.cap_s || (int64_t)a1 + na1 > g.cap_a) return false;
  if (tm.tid == 0) v.st_arc0[s1 + nn] = a1 + na1;
  tm.Sync();
  // destination index of every arc and the best score into every new state; an
  // arc below the cutoff still enters a state that another arc created (:1103-1138)
  for (int32_t q0 = tm.tid; q0 < na; q0 += kBatch * tm.threads) {
    float end[kBatch];
    int32_t dest[kBatch];
    unsigned long long w[kBatch];
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int32_t q = q0 + i * tm.threads;
      end[i] = q < na ? v.arc_end[a0 + q] : kNegInf;
      dest[i] = q < na ? v.arc_dest[a0 + q] : -1;
    }
#pragma unroll
    for (int i = 0; i < kBatch; ++i) w[i] = dest[i] >= 0 ? v.winner[dest[i]] : 0ull;
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
      const int32_t q = q0 + i * tm.threads;
      if (q < na) {
        int32_t idx1 = -1;
        if ((uint32_t)(w[i] >> 32) == (uint32_t)(t + 1) && (w[i] & 0x80000000u)) {
          idx1 = (int32_t)(w[i] & 0x7fffffffu);
          atomicMax(&v.st_fwd[s1 + idx1], OrderedInt(end[i]));
        }
        v.arc_dest[a0 + q] = idx1;
      }
    }
  }
  tm.Sync();
  *ns_next = nn;
  *na_next = na1;
  return true;
}

// Backward pass over frames [begin, end) with the output beam (PruneTimeRange,
// :1373-1634, with SetBackwardProbsFinal :1170-1193 and PropagateBackward
// :1239-1346), then compaction of those frames in place.  On entry the frames up to
// `end` are complete and frame `end` has its states and the layout of the na_end arcs
// that will leave them, but not the arcs; on return *s_top / *a_top are the ends of
// the arenas and the frame tables are updated.
__device__ void PruneWindow(const SearchArgs &g, const SeqView &v, const Team &tm, int32_t seq,
                            int32_t begin, int32_t end, int32_t na_end, int32_t *s_top,
                            int32_t *a_top, bool keep_all_at_begin = true) {
  Shared *sh = tm.sh;
  const float kNegInf = -INFINITY;
  const int32_t gi = seq * g.a_stride;
  const int32_t g_final = g.a_rs1[gi + 1] - 1;  // last state of this sequence's graph
  const float beam = g.output_beam;

  {  // frame `end`: backward score = -forward score, whatever the state
    const int32_t s0 = v.frame_s0[end], ns = *s_top - s0;
    for (int32_t k = tm.tid; k < ns; k += tm.threads) {
      const float fwd = OrderedFloat(v.st_fwd[s0 + k]);
      v.st_bwd[s0 + k] = (fwd - fwd == 0.0f) ? -fwd : kNegInf;
    }
  }
  tm.Sync();

  // backwards: arc and state survival, backward scores, new state numbers
  for (int32_t t = end - 1; t >= begin; --t) {
    const int32_t s0 = v.frame_s0[t], ns = v.frame_s0[t + 1] - s0, s_next = v.frame_s0[t + 1];
    int32_t kept = 0;
    for (int32_t base = 0; base < ns; base += tm.threads) {
      // a warp takes 32 consecutive states and walks their arcs as one flat range
      // (as in the search step); per-state maxima and counts gather in shared memory
      const int32_t k = base + tm.tid;
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
      int32_t keep_state = 0, p0 = 0x7fffffff;
      float fwd = 0.0f;
      if (k < ns) {
        fwd = OrderedFloat(v.st_fwd[s0 + k]);
        p0 = v.st_arc0[s0 + k];
      }
      sh->wbest[warp][lane] = OrderedInt(kNegInf);
      sh->wcnt[warp][lane] = 0;
      __syncwarp();
      const int32_t first = __shfl_sync(0xffffffffu, p0, 0);
      const int32_t last = v.st_arc0[s0 + min(k - lane + 32, ns)];
      for (int32_t pb = first; pb < last; pb += 32 * kExpand) {
        int32_t p[kExpand], j[kExpand], d[kExpand];
        float ll[kExpand], nb[kExpand];
#pragma unroll
        for (int i = 0; i < kExpand; ++i) {
          p[i] = pb + i * 32 + lane;
          int32_t lo = 0;
#pragma unroll
          for (int step = 16; step > 0; step >>= 1) {
            const int32_t cand = __shfl_sync(0xffffffffu, p0, lo + step);
            if (cand <= p[i]) lo += step;
          }
          j[i] = lo;
          d[i] = p[i] < last ? v.arc_dest[p[i]] : -1;
          ll[i] = p[i] < last ? v.arc_ll[p[i]] : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < kExpand; ++i) nb[i] = d[i] >= 0 ? v.st_bwd[s_next + d[i]] : kNegInf;
#pragma unroll
        for (int i = 0; i < kExpand; ++i) {
          const float jfwd = __shfl_sync(0xffffffffu, fwd, j[i]);
          if (p[i] < last) {
            uint8_t keep = 0;
            if (d[i] >= 0) {
              const float bl = ll[i] + nb[i];
              if (bl + jfwd >= -beam) {
                keep = 1;
                atomicMax(&sh->wbest[warp][j[i]], OrderedInt(bl));
                atomicAdd(&sh->wcnt[warp][j[i]], 1);
              }
            }
            v.arc_keep[p[i]] = keep;
          }
        }
      }
      __syncwarp();
      if (k < ns) {
        const float best = OrderedFloat(sh->wbest[warp][lane]);
        v.st_cnt[s0 + k] = sh->wcnt[warp][lane];
        const float bwd = (v.st_astate[s0 + k] == g_final) ? -fwd : best;
        v.st_bwd[s0 + k] = bwd;
        keep_state = (bwd != kNegInf) || (t == begin && keep_all_at_begin);
      }
      int32_t tot;
      const int32_t j = kept + tm.Scan(keep_state, &tot);
      if (k < ns) v.st_new[s0 + k] = keep_state ? j : -1;
      kept += tot;
    }
    // (the barrier inside the last scan has published this frame's backward scores)
  }

  // forwards: move the surviving states and arcs down.  Reads of a chunk complete
  // before its writes (the scans synchronise), and writes never reach past the
  // chunk being read, so the compaction is done in place.
  int32_t ws = v.frame_s0[begin], wa = v.frame_a0[begin];
  int32_t old_s0 = ws, old_a0 = wa;
  for (int32_t t = begin; t < end; ++t) {
    const int32_t old_s1 = v.frame_s0[t + 1], old_a1 = v.frame_a0[t + 1];
    const int32_t ns = old_s1 - old_s0, na = old_a1 - old_a0;
    int32_t s_run = 0, a_run = 0;
    for (int32_t base = 0; base < ns; base += tm.threads) {
      const int32_t k = base + tm.tid;
      int32_t keep_state = 0, cnt = 0, as = 0, fwd = 0;
      float bwd = 0.0f;
      if (k < ns) {
        keep_state = v.st_new[old_s0 + k] >= 0;
        as = v.st_astate[old_s0 + k];
        fwd = v.st_fwd[old_s0 + k];
        bwd = v.st_bwd[old_s0 + k];
        cnt = v.st_cnt[old_s0 + k];
      }
      int32_t stot, atot, aj;
      const int32_t sj = s_run + tm.Scan2(keep_state, cnt, &aj, &stot, &atot);
      aj += a_run;
      if (keep_state) {
        v.st_astate[ws + sj] = as;
        v.st_fwd[ws + sj] = fwd;
        v.st_bwd[ws + sj] = bwd;
        v.st_arc0[ws + sj] = wa + aj;
      }
      s_run += stot;
      a_run += atot;
    }
    int32_t moved = 0;
    const bool renumber = t + 1 < end;  // the states of frame `end` keep their numbers
    for (int32_t base = 0; base < na; base += tm.threads * kPer) {
      const int32_t q0 = base + tm.tid * kPer;
      int32_t aidx[kPer], dest[kPer];
      float ll[kPer];
      int32_t keep = 0;
#pragma unroll
      for (int i = 0; i < kPer; ++i) {
        if (q0 + i < na && v.arc_keep[old_a0 + q0 + i]) {
          keep |= 1 << i;
          aidx[i] = v.arc_aidx[old_a0 + q0 + i];
          ll[i] = v.arc_ll[old_a0 + q0 + i];
          dest[i] = v.arc_dest[old_a0 + q0 + i];
          if (renumber) dest[i] = v.st_new[old_s1 + dest[i]];
        }
      }
      int32_t tot;
      int32_t j = moved + tm.Scan(__popc(keep), &tot);
#pragma unroll
      for (int i = 0; i < kPer; ++i) {
        if (keep >> i & 1) {
          v.arc_aidx[wa + j] = aidx[i];
          v.arc_ll[wa + j] = ll[i];
          v.arc_dest[wa + j] = dest[i];
          ++j;
        }
      }
      moved += tot;
    }
    // the new offsets go to the frame tables after the loop: a thread that runs
    // ahead through empty frames must still find the old ones
    if (tm.tid == 0) {
      sh->new_s0[t - begin] = ws;
      sh->new_a0[t - begin] = wa;
    }
    ws += s_run;
    wa += a_run;
    old_s0 = old_s1;
    old_a0 = old_a1;
  }
  // frame `end`: its states, and the layout of their arcs, follow the compacted frames
  const int32_t ns_end = *s_top - old_s0;
  for (int32_t base = 0; base < ns_end; base += tm.threads) {
    const int32_t k = base + tm.tid;
    int32_t as = 0, fwd = 0, arc0 = 0;
    float bwd = 0.0f;
    if (k < ns_end) {
      as = v.st_astate[old_s0 + k];
      fwd = v.st_fwd[old_s0 + k];
      bwd = v.st_bwd[old_s0 + k];
      arc0 = v.st_arc0[old_s0 + k];
    }
    tm.Sync();
    if (k < ns_end) {
      v.st_astate[ws + k] = as;
      v.st_fwd[ws + k] = fwd;
      v.st_bwd[ws + k] = bwd;
      v.st_arc0[ws + k] = arc0 - old_a0 + wa;
    }
  }
  tm.Sync();  // every thread is past the old frame tables
  if (tm.tid == 0) {
    for (int32_t t = begin; t < end; ++t) {
      v.frame_s0[t] = sh->new_s0[t - begin];
      v.frame_a0[t] = sh->new_a0[t - begin];
    }
    v.frame_s0[end] = ws;
    v.frame_a0[end] = wa;
    v.st_arc0[ws + ns_end] = wa + na_end;  // closes the last arc range
  }
  tm.Sync();
  *s_top = ws + ns_end;
  *a_top = wa;
}

// One team per sequence: all frames of the search with the pruning windows in the
// reference's schedule (:164-199, :213-229).
__global__ void __launch_bounds__(kSearchThreads, 1) PrunedSearch(const SearchArgs g) {
  __shared__ Shared sh;
  if (threadIdx.x == 0) {
    sh.phase_i = sh.phase_f = sh.phase_l = 0;
    sh.beam = g.search_beam;
  }
  __syncthreads();
  const Team tm(&sh);
  const int32_t seq = blockIdx.x / tm.size;
  const SeqView v = ViewOf(g, seq);
  const int32_t row0 = g.b_rs[seq], final_t = g.b_rs[seq + 1] - row0;
  const int32_t T = g.T;
  const int32_t gi = seq * g.a_stride;
  const int32_t g_start = g.a_rs1[gi], g_states = g.a_rs1[gi + 1] - g_start;

  // frame 0: the start state, if the graph has states (:435-472)
  int32_t s0 = 0, ns = g_states > 0 ? 1 : 0, a0 = 0;
  int32_t na = ns ? g.a_rs2[g_start + 1] - g.a_rs2[g_start] : 0;
  if (tm.tid == 0) {
    v.frame_s0[0] = 0;
    v.frame_a0[0] = 0;
    v.st_arc0[0] = 0;
    if (ns) {
      v.st_astate[0] = g_start;
      v.st_fwd[0] = OrderedInt(0.0f);
      v.st_arc0[1] = na;
    }
  }
  tm.Sync();
  int32_t s_top = ns, a_top = 0;
  int32_t status = kSeqOk;
  int32_t next_end = kWindowShift;  // end of the next pruning window
  for (int32_t t = 0; t < T; ++t) {
    if (tm.tid == 0) {  // published by the barriers inside the step
      v.frame_s0[t + 1] = s0 + ns;
      v.frame_a0[t + 1] = a0 + na;
    }
    int32_t nn, na1;
    if (!SearchStep(g, v, tm, seq, t, final_t, row0, s0, ns, a0, na, &nn, &na1)) {
      status = kSeqOverflow;
      break;
    }
    s0 += ns;
    a0 += na;
    ns = nn;
    na = na1;
    s_top = s0 + ns;
    a_top = a0;
    const int32_t this_end = next_end >= T ? T : next_end;
    if (t == this_end - 1) {
      const int32_t begin = max(0, next_end - kWindow);
      PruneWindow(g, v, tm, seq, begin, this_end, na, &s_top, &a_top);
      s0 = s_top - ns;
      a0 = a_top;
      next_end += kWindowShift;
    }
  }
  if (status == kSeqOk) {  // the states of the last frame have no arcs in the lattice
    for (int32_t k = tm.tid; k < ns; k += tm.threads) v.st_arc0[s0 + k] = a_top;
  }
  if (tm.tid == 0) {
    int32_t extra = 0;
    if (status == kSeqOk) {
      v.frame_s0[T + 1] = s_top;  // frame T has no arcs
      v.frame_a0[T + 1] = a_top;
      v.st_arc0[s_top] = a_top;
      // a sequence whose final state did not survive still gets a final state, so
      // that the result is a valid FSA (:519-547)
      const int32_t at_final = v.frame_s0[final_t + 1] - v.frame_s0[final_t];
      if (at_final > 1) status = kSeqManyFinal;
      extra = (g_states > 0) * (1 - min(at_final, 1));
    }
    int32_t *o = g.seq_out + 4 * seq;
    o[0] = s_top + extra;
    o[1] = a_top;
    o[2] = extra;
    o[3] = status;
  }
  tm.Sync();  // no CTA leaves while another may still read its shared memory
}

struct FormatArgs {
  SearchArgs g;
  const int32_t *out_rs1;   // [num_seqs + 1] first lattice state of every sequence
  const int32_t *arc_base;  // [num_seqs + 1] first lattice arc of every sequence
  int32_t *row_ids1, *row_splits2, *row_ids2;
  Arc *arcs;
  int32_t *arc_map_a, *arc_map_b;
  int32_t *level_offsets, *level_splits;
};

// Lattice of one (sequence, frame) per CTA (FormatOutput, :474-657): the arenas are
// already in [sequence][frame][state][arc] order.
__global__ void FormatPruned(const FormatArgs f) {
  const SearchArgs &g = f.g;
  const int32_t seq = blockIdx.y, t = blockIdx.x;  // t in [0, T + 1]
  const SeqView v = ViewOf(g, seq);
  const int32_t row0 = g.b_rs[seq], final_t = g.b_rs[seq + 1] - row0;
  const int32_t sb = f.out_rs1[seq], ab = f.arc_base[seq];
  const int32_t s0 = v.frame_s0[t], s1 = v.frame_s0[t + 1];
  if (f.level_splits != nullptr && threadIdx.x == 0) {
    f.level_splits[(int64_t)seq * (g.T + 2) + t] = sb + s0;
    if (t == 0) f.level_offsets[seq] = seq * (g.T + 2);
    if (seq == g.num_seqs - 1 && t == g.T + 1) {
      f.level_offsets[g.num_seqs] = g.num_seqs * (g.T + 2);
      f.level_splits[(int64_t)g.num_seqs * (g.T + 2)] = f.out_rs1[g.num_seqs];
    }
  }
  if (t == g.T + 1) {
    // the extra final state, if any, and the end of the row_splits
    if (threadIdx.x == 0) {
      const int32_t extra = g.seq_out[4 * seq + 2];
      if (extra) {
        f.row_ids1[sb + s0] = seq;
        f.row_splits2[sb + s0] = ab + g.seq_out[4 * seq + 1];
      }
      if (seq == g.num_seqs - 1) f.row_splits2[f.out_rs1[g.num_seqs]] = f.arc_base[g.num_seqs];
    }
    return;
  }
  const int32_t next_s0 = s1;  // the states of frame t + 1 start where frame t ends
  for (int32_t k = s0 + threadIdx.x; k < s1; k += blockDim.x) {
    const int32_t p0 = v.st_arc0[k], p1 = v.st_arc0[k + 1];
    f.row_ids1[sb + k] = seq;
    f.row_splits2[sb + k] = ab + p0;
    for (int32_t p = p0; p < p1; ++p) {
      int32_t aidx = v.arc_aidx[p];
      const int32_t graph_label = g.a_arcs[aidx].label;
      Arc out;
      out.src = k;
      out.dest = next_s0 + v.arc_dest[p];
      out.label = graph_label;
      out.score = v.arc_ll[p];
      if (t == final_t - 1 && graph_label != -1) {  // allow_partial (:625-634)
        out.label = -1;
        aidx = -1;
      }
      f.arcs[ab + p] = out;
      f.row_ids2[ab + p] = sb + k;
      f.arc_map_a[ab + p] = aidx;
      f.arc_map_b[ab + p] = (row0 + t) * g.cols + graph_label + 1;
    }
  }
}


// ---------------------------------------------------------------------------
// Chunk-by-chunk decoding (OnlineDenseIntersecter, k2/csrc/intersect_dense_pruned.cu:
// 247-312 OnlineIntersect, :336-405 GetFinalFrame, :1739-1853 Decode).  Every stream
// brings the frames it has decoded so far (loaded into its arena slice before the
// launch); the kernel searches the frames of the chunk, prunes the last two frames of
// the history together with the chunk (:274-277), and closes the lattice with the final
// arcs that the extra row [0, -inf, ...] of the chunk allows.
// ---------------------------------------------------------------------------
struct OnlineArgs {
  SearchArgs g;            // g.T + 2 = capacity of the frame tables
  const int32_t *hist;     // [num_seqs] frames searched so far (index of the frontier)
  const float *beam_in;    // [num_seqs]
  float *beam_out;         // [num_seqs]
  int32_t chunk;           // frames in this chunk
  int32_t hist_max;        // longest history in the batch (the reference aligns streams
                           // at their ends, so the pruning window is counted from there)
};

// Arc ranges of the states of a frame whose arcs are about to be expanded.
__device__ int32_t LayoutFrame(const SearchArgs &g, const SeqView &v, const Team &tm, int32_t s0,
                               int32_t ns, int32_t a0) {
  int32_t na = 0;
  for (int32_t base = 0; base < ns; base += tm.threads) {
    const int32_t k = base + tm.tid;
    int32_t deg = 0;
    if (k < ns) {
      const int32_t as = v.st_astate[s0 + k];
      deg = g.a_rs2[as + 1] - g.a_rs2[as];
    }
    int32_t tot;
    const int32_t ex = tm.Scan(deg, &tot);
    if (k < ns) v.st_arc0[s0 + k] = a0 + na + ex;
    na += tot;
  }
  if (tm.tid == 0) v.st_arc0[s0 + ns] = a0 + na;
  tm.Sync();
  return na;
}

// GetFinalFrame (:336-405): the arcs that leave the frontier on the extra row of the
// chunk; only those with a finite score stay (label -1, or every arc when
// allow_partial finds no final arc), all of them entering one final state.  Returns
// their number, or -1 when the arena is full.
__device__ int32_t FinalArcs(const SearchArgs &g, const SeqView &v, const Team &tm, int32_t seq,
                             int32_t row, int32_t s0, int32_t ns, int32_t a0) {
  const int32_t gi = seq * g.a_stride;
  (void)gi;
  const bool row_ok = row < g.rows;
  const float *r = g.scores + (int64_t)(row_ok ? row : 0) * g.cols;
  bool redirect = false;
  if (g.allow_partial) {
    int32_t has = 0;
    for (int32_t k = tm.tid; k < ns; k += tm.threads) {
      const int32_t as = v.st_astate[s0 + k];
      for (int32_t a = g.a_rs2[as]; a < g.a_rs2[as + 1]; ++a) has |= (g.a_arcs[a].label == -1);
    }
    redirect = !tm.Any(has);
  }
  int32_t na = 0;
  for (int32_t base = 0; base < ns; base += tm.threads) {
    const int32_t k = base + tm.tid;
    int32_t cnt = 0, as = 0;
    if (k < ns) {
      as = v.st_astate[s0 + k];
      for (int32_t a = g.a_rs2[as]; a < g.a_rs2[as + 1]; ++a) {
        const Arc arc = g.a_arcs[a];
        const uint32_t col = (uint32_t)(arc.label + 1);
        float acoustic = (row_ok && col < (uint32_t)g.cols) ? r[col] : -INFINITY;
        if (redirect) acoustic = 0.0f;
        const float ll = acoustic + arc.score;
        cnt += (ll - ll == 0.0f);
      }
    }
    int32_t tot;
    const int32_t ex = tm.Scan(cnt, &tot);
    const bool fits = (int64_t)a0 + na + tot <= g.cap_a;
    if (k < ns && fits) {
      int32_t p = a0 + na + ex;
      v.st_arc0[s0 + k] = p;
      for (int32_t a = g.a_rs2[as]; a < g.a_rs2[as + 1]; ++a) {
        const Arc arc = g.a_arcs[a];
        const uint32_t col = (uint32_t)(arc.label + 1);
        float acoustic = (row_ok && col < (uint32_t)g.cols) ? r[col] : -INFINITY;
        if (redirect) acoustic = 0.0f;
        const float ll = acoustic + arc.score;
        if (ll - ll == 0.0f) {
          v.arc_aidx[p] = a;
          v.arc_ll[p] = ll;
          v.arc_dest[p] = 0;
          ++p;
        }
      }
    }
    na += tot;
    if (!fits) return -1;
  }
  if (tm.tid == 0) v.st_arc0[s0 + ns] = a0 + na;
  tm.Sync();
  return na;
}

__global__ void __launch_bounds__(kSearchThreads, 1) OnlineChunk(const OnlineArgs o) {
  __shared__ Shared sh;
  const SearchArgs &g = o.g;
  const Team tm0(&sh);
  const int32_t seq = blockIdx.x / tm0.size;
  if (threadIdx.x == 0) {
    sh.phase_i = sh.phase_f = sh.phase_l = 0;
    sh.beam = o.beam_in[seq];
  }
  __syncthreads();
  const Team tm(&sh);
  const SeqView v = ViewOf(g, seq);
  const int32_t row0 = g.b_rs[seq];
  const int32_t h = o.hist[seq];
  const int32_t kNoFinalFrame = 0x3fffffff;  // online: no end-of-sequence rules (:725-760)
  // the frontier: the states of frame h; what was kept of its arcs (the final arcs of
  // the previous chunk) is dropped and they are expanded again (:354-361)
  int32_t s0 = v.frame_s0[h], ns = v.frame_s0[h + 1] - s0, a0 = v.frame_a0[h];
  int32_t na = LayoutFrame(g, v, tm, s0, ns, a0);
  int32_t s_top = s0 + ns, a_top = a0;
  int32_t status = kSeqOk;
  for (int32_t t = 0; t < o.chunk; ++t) {
    if (tm.tid == 0) {
      v.frame_s0[h + t + 1] = s0 + ns;
      v.frame_a0[h + t + 1] = a0 + na;
    }
    int32_t nn, na1;
    if (!SearchStep(g, v, tm, seq, t, kNoFinalFrame, row0, s0, ns, a0, na, &nn, &na1)) {
      status = kSeqOverflow;
      break;
    }
    s0 += ns;
    a0 += na;
    ns = nn;
    na = na1;
    s_top = s0 + ns;
    a_top = a0;
  }
  const int32_t end = h + o.chunk;
  if (status == kSeqOk) {
    // PruneTimeRange(max(0, T_ - 2), T_ + chunk) in frames counted from the end of the
    // longest history: a stream with a shorter one starts inside the window, and then
    // its first frame is not the one whose states are all kept
    const int32_t begin_aligned = max(0, o.hist_max - 2) - (o.hist_max - h);
    PruneWindow(g, v, tm, seq, max(begin_aligned, 0), end, na, &s_top, &a_top,
                begin_aligned >= 0);
    s0 = s_top - ns;
    a0 = a_top;
    const int32_t nf = FinalArcs(g, v, tm, seq, row0 + o.chunk, s0, ns, a0);
    if (nf < 0) {
      status = kSeqOverflow;
    } else {
      a_top = a0 + nf;
      if (tm.tid == 0) {
        v.frame_s0[end + 1] = s_top;
        v.frame_a0[end + 1] = a_top;
        v.st_arc0[s_top] = a_top;
      }
    }
  }
  if (tm.tid == 0) {
    int32_t *out = g.seq_out + 4 * seq;
    out[0] = s_top;      // states without the final one
    out[1] = a_top;
    out[2] = end;        // frames: the frontier is frame `end`
    out[3] = status;
    o.beam_out[seq] = sh.beam;
  }
  tm.Sync();
}

// Lattice of one (stream, frame) per CTA, all frames so far plus one final state that
// the final arcs enter (FormatOutput with online_decoding, :474-657; a stream without
// final arcs gets the state all the same, :519-547).  No arc_map_b.
__global__ void FormatOnline(const FormatArgs f, const int32_t *__restrict__ hist, int32_t chunk) {
  const SearchArgs &g = f.g;
  const int32_t seq = blockIdx.y, t = blockIdx.x;
  const SeqView v = ViewOf(g, seq);
  const int32_t end = hist[seq] + chunk;  // the frontier
  if (t > end + 1) return;
  const int32_t sb = f.out_rs1[seq], ab = f.arc_base[seq];
  if (f.level_splits != nullptr && threadIdx.x == 0) {
    // frames are layers; the final state is a layer of its own
    const int32_t lo = f.level_offsets[seq];
    f.level_splits[lo + t] = sb + v.frame_s0[t];
    if (seq == g.num_seqs - 1 && t == end + 1) f.level_splits[lo + t + 1] = f.out_rs1[g.num_seqs];
  }
  if (t == end + 1) {
    if (threadIdx.x == 0) {
      const int32_t s_top = v.frame_s0[end + 1];
      f.row_ids1[sb + s_top] = seq;
      f.row_splits2[sb + s_top] = ab + v.frame_a0[end + 1];
      if (seq == g.num_seqs - 1) f.row_splits2[f.out_rs1[g.num_seqs]] = f.arc_base[g.num_seqs];
    }
    return;
  }
  const int32_t s0 = v.frame_s0[t], s1 = v.frame_s0[t + 1];
  for (int32_t k = s0 + threadIdx.x; k < s1; k += blockDim.x) {
    const int32_t p0 = v.st_arc0[k], p1 = v.st_arc0[k + 1];
    f.row_ids1[sb + k] = seq;
    f.row_splits2[sb + k] = ab + p0;
    for (int32_t p = p0; p < p1; ++p) {
      int32_t aidx = v.arc_aidx[p];
      const int32_t graph_label = g.a_arcs[aidx].label;
      Arc out;
      out.src = k;
      out.dest = s1 + v.arc_dest[p];
      out.label = graph_label;
      out.score = v.arc_ll[p];
      if (t == end && graph_label != -1) {  // allow_partial (:625-634)
        out.label = -1;
        aidx = -1;
      }
      f.arcs[ab + p] = out;
      f.row_ids2[ab + p] = sb + k;
      f.arc_map_a[ab + p] = aidx;
    }
  }
}

// Carves the workspace.  Everything is sized from the arguments alone, so the
// search and the output call agree on it.
struct PrunedLayout {
  SearchArgs g;
  int32_t *out_rs1, *arc_base;  // [num_seqs + 1] each
  size_t winner_bytes, bytes;
};

size_t Take(size_t *off, size_t n) {
  const size_t at = *off;
  *off += AlignUp(n);
  return at;
}

int32_t MakePrunedLayout(const k2b200_pruned_args *a, char *ws, PrunedLayout *L) {
  K2B_REQUIRE(a != nullptr, "NULL arguments");
  K2B_REQUIRE(a->search_beam > 0 && a->output_beam > 0, "search_beam and output_beam must be positive");
  K2B_REQUIRE(a->min_active_states >= 0 && a->max_active_states > a->min_active_states,
              "need 0 <= min_active_states < max_active_states");
  K2B_REQUIRE(a->num_seqs >= 1 && a->num_seqs <= 65535, "num_seqs must be in [1, 65535]");
  K2B_REQUIRE(a->num_fsas == a->num_seqs || a->num_fsas == 1,
              "a_fsas must hold one graph per sequence or a single shared graph (got %d graphs "
              "for %d sequences)", a->num_fsas, a->num_seqs);
  K2B_REQUIRE(a->h_b_row_splits != nullptr, "NULL h_b_row_splits");
  K2B_REQUIRE(a->max_states_per_seq >= 2 && a->max_arcs_per_seq >= 1 &&
                  a->max_states_per_seq < 0x7f000000 && a->max_arcs_per_seq < 0x7f000000,
              "arena capacities out of range");
  int32_t T = 0;
  for (int32_t i = 0; i < a->num_seqs; ++i) {
    const int32_t rows = a->h_b_row_splits[i + 1] - a->h_b_row_splits[i];
    K2B_REQUIRE(rows >= 1, "sequence %d has no rows", i);
    T = std::max(T, rows);
  }
  K2B_REQUIRE(a->h_b_row_splits[a->num_seqs] == a->rows, "b row_splits do not cover the scores");
  SearchArgs &g = L->g;
  g.a_rs1 = a->a_row_splits1;
  g.a_rs2 = a->a_row_splits2;
  g.a_arcs = reinterpret_cast<const Arc *>(a->a_arcs);
  g.a_stride = a->num_fsas == 1 && a->num_seqs > 1 ? 0 : 1;
  g.a_states = a->num_states;
  g.scores = a->scores;
  g.rows = a->rows;
  g.cols = a->cols;
  g.b_rs = a->b_row_splits;
  g.num_seqs = a->num_seqs;
  g.T = T;
  g.search_beam = a->search_beam;
  g.output_beam = a->output_beam;
  g.min_active = (float)a->min_active_states;
  g.max_active = (float)a->max_active_states;
  g.allow_partial = a->allow_partial;
  g.cap_s = a->max_states_per_seq;
  g.cap_a = a->max_arcs_per_seq;
  const size_t n = (size_t)a->num_seqs, ns = n * ((size_t)g.cap_s + 1), na = n * (size_t)g.cap_a;
  size_t off = 0;
  auto i32 = [&](size_t count) { return reinterpret_cast<int32_t *>(ws + Take(&off, 4 * count)); };
  auto f32 = [&](size_t count) { return reinterpret_cast<float *>(ws + Take(&off, 4 * count)); };
  g.st_astate = i32(ns);
  g.st_fwd = i32(ns);
  g.st_arc0 = i32(ns);
  g.st_new = i32(ns);
  g.st_cnt = i32(ns);
  g.st_bwd = f32(ns);
  g.arc_aidx = i32(na);
  g.arc_dest = i32(na);
  g.arc_ll = f32(na);
  g.arc_end = f32(na);
  g.arc_keep = reinterpret_cast<uint8_t *>(ws + Take(&off, na));
  L->winner_bytes = 8 * (g.a_stride ? (size_t)std::max(a->num_states, 1)
                                    : n * (size_t)std::max(a->num_states, 1));
  g.winner = reinterpret_cast<unsigned long long *>(ws + Take(&off, L->winner_bytes));
  g.frame_s0 = i32(n * ((size_t)T + 2));
  g.frame_a0 = i32(n * ((size_t)T + 2));
  g.seq_out = i32(4 * n);
  L->out_rs1 = i32(n + 1);
  L->arc_base = i32(n + 1);
  L->bytes = off;
  return kOk;
}


// Many small device-to-device copies in one launch (the eight arrays of every stream):
// one CTA per copy, 4-byte elements.
struct CopyJob {
  const int32_t *src;
  int32_t *dst;
  int64_t count;
};
__global__ void CopyMany(const CopyJob *__restrict__ jobs) {
  const CopyJob j = jobs[blockIdx.x];
  for (int64_t k = threadIdx.x; k < j.count; k += blockDim.x) j.dst[k] = j.src[k];
}

// The online entry points share the arena layout of the batch search: the frame
// tables are sized for the longest history plus the chunk.
struct OnlineLayout {
  PrunedLayout base;
  int32_t *hist;
  float *beam_in, *beam_out;
  CopyJob *jobs;  // [8 * num_seqs]
  int32_t chunk, hist_max;
  size_t bytes;
};

int32_t MakeOnlineLayout(const k2b200_online_args *a, char *ws, OnlineLayout *L) {
  K2B_REQUIRE(a != nullptr && a->h_hist != nullptr && a->h_b_row_splits != nullptr,
              "NULL arguments");
  K2B_REQUIRE(a->num_seqs >= 1, "num_seqs must be positive");
  const int32_t rows0 = a->h_b_row_splits[1] - a->h_b_row_splits[0];
  int32_t hist_max = 0;
  for (int32_t i = 0; i < a->num_seqs; ++i) {
    K2B_REQUIRE(a->h_b_row_splits[i + 1] - a->h_b_row_splits[i] == rows0,
                "the streams of a chunk must all have the same number of frames");
    K2B_REQUIRE(a->h_hist[i] >= 0, "negative history length");
    hist_max = std::max(hist_max, a->h_hist[i]);
  }
  K2B_REQUIRE(rows0 >= 2, "a chunk needs at least one frame besides its final row");
  // a batch-mode argument block whose longest sequence has hist_max + chunk rows gives
  // frame tables of hist_max + chunk + 2 entries
  k2b200_pruned_args p = {};
  p.num_fsas = 1;
  p.num_states = a->num_states;
  p.num_arcs = a->num_arcs;
  p.a_row_splits1 = a->a_row_splits1;
  p.a_row_splits2 = a->a_row_splits2;
  p.a_arcs = a->a_arcs;
  p.scores = a->scores;
  p.rows = a->rows;
  p.cols = a->cols;
  p.num_seqs = a->num_seqs;
  p.b_row_splits = a->b_row_splits;
  p.search_beam = a->search_beam;
  p.output_beam = a->output_beam;
  p.min_active_states = a->min_active_states;
  p.max_active_states = a->max_active_states;
  p.allow_partial = a->allow_partial;
  p.max_states_per_seq = a->max_states_per_seq;
  p.max_arcs_per_seq = a->max_arcs_per_seq;
  std::vector<int32_t> fake(a->num_seqs + 1);
  for (int32_t i = 0; i <= a->num_seqs; ++i) fake[i] = i * (hist_max + rows0 - 1);
  p.h_b_row_splits = fake.data();
  p.rows = fake[a->num_seqs];
  K2B_FORWARD(MakePrunedLayout(&p, ws, &L->base));
  SearchArgs &g = L->base.g;
  g.rows = a->rows;
  g.a_stride = 0;  // one graph, a table per stream
  g.T = hist_max + rows0 - 1;
  // the winner table of the batch layout was sized for a shared graph only when there is
  // more than one sequence; make room for one table per stream in every case
  size_t off = L->base.bytes;
  L->base.winner_bytes = 8 * (size_t)a->num_seqs * (size_t)std::max(a->num_states, 1);
  g.winner = reinterpret_cast<unsigned long long *>(ws + Take(&off, L->base.winner_bytes));
  L->hist = reinterpret_cast<int32_t *>(ws + Take(&off, 4 * (size_t)a->num_seqs));
  L->beam_in = reinterpret_cast<float *>(ws + Take(&off, 4 * (size_t)a->num_seqs));
  L->beam_out = reinterpret_cast<float *>(ws + Take(&off, 4 * (size_t)a->num_seqs));
  L->jobs = reinterpret_cast<CopyJob *>(ws + Take(&off, sizeof(CopyJob) * 8 * (size_t)a->num_seqs));
  L->chunk = rows0 - 1;
  L->hist_max = hist_max;
  L->bytes = off;
  return kOk;
}

}  // namespace
}  // namespace k2b

using namespace k2b;  // NOLINT

extern "C" {

int32_t k2b200_intersect_dense_pruned_workspace_bytes(const k2b200_pruned_args *args,
                                                      size_t *bytes, int64_t *total_levels) {
  PrunedLayout L;
  K2B_FORWARD(MakePrunedLayout(args, nullptr, &L));
  K2B_REQUIRE(bytes != nullptr, "NULL bytes");
  *bytes = L.bytes;
  if (total_levels) *total_levels = (int64_t)args->num_seqs * (L.g.T + 2);
  return kOk;
}

int32_t k2b200_intersect_dense_pruned_search(const k2b200_pruned_args *args, void *workspace,
                                             size_t workspace_bytes, void *stream_v,
                                             int32_t *num_states_out, int32_t *num_arcs_out,
                                             int32_t *arena_full) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  PrunedLayout L;
  K2B_FORWARD(MakePrunedLayout(args, reinterpret_cast<char *>(workspace), &L));
  K2B_REQUIRE(workspace != nullptr && workspace_bytes >= L.bytes, "workspace too small");
  K2B_REQUIRE(num_states_out && num_arcs_out && arena_full, "NULL output pointer");
  K2B_REQUIRE(args->a_row_splits1 && args->a_row_splits2 && args->b_row_splits &&
                  (args->a_arcs || args->num_arcs == 0) && args->scores,
              "NULL input pointer");
  const int32_t n = args->num_seqs;
  K2B_CUDA_OK(cudaMemsetAsync(L.g.winner, 0, L.winner_bytes, stream));
  {
    // CTAs per sequence: as many as keep the GPU filled, within the portable
    // cluster size
    int dev = 0, sms = 0;
    K2B_CUDA_OK(cudaGetDevice(&dev));
    K2B_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    int32_t team = 1;
    while (team < 8 && n * team * 2 <= sms) team *= 2;
    if (args->team_ctas > 0) team = args->team_ctas;
    K2B_REQUIRE(team == 1 || team == 2 || team == 4 || team == 8, "team_ctas must be 1, 2, 4 or 8");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n * team);
    cfg.blockDim = dim3(kSearchThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = team;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    K2B_CUDA_OK(cudaLaunchKernelEx(&cfg, PrunedSearch, L.g));
    NoteLaunch();
  }
  K2B_CUDA_OK(cudaGetLastError());
  std::vector<int32_t> h(4 * (size_t)n);
  K2B_CUDA_OK(cudaMemcpyAsync(h.data(), L.g.seq_out, sizeof(int32_t) * h.size(),
                              cudaMemcpyDeviceToHost, stream));
  K2B_CUDA_OK(cudaStreamSynchronize(stream));
  std::vector<int32_t> bases(2 * ((size_t)n + 1));
  int32_t *srs = bases.data(), *ars = bases.data() + n + 1;
  int64_t ts = 0, ta = 0;
  *arena_full = 0;
  for (int32_t i = 0; i < n; ++i) {
    if (h[4 * i + 3] == kSeqOverflow) *arena_full = 1;
    K2B_REQUIRE(h[4 * i + 3] != kSeqManyFinal,
                "sequence %d reaches more than one state on its last frame: arcs with label -1 "
                "must enter the final state of their graph", i);
    srs[i] = (int32_t)ts;
    ars[i] = (int32_t)ta;
    ts += h[4 * i + 0];
    ta += h[4 * i + 1];
  }
  srs[n] = (int32_t)ts;
  ars[n] = (int32_t)ta;
  *num_states_out = *num_arcs_out = 0;
  if (*arena_full) return kOk;
  K2B_REQUIRE(ts < INT_MAX && ta < INT_MAX, "the lattice has too many states or arcs for int32");
  // out_rs1 and arc_base are adjacent in the workspace only up to alignment: two uploads
  K2B_FORWARD(UploadInts(srs, n + 1, L.out_rs1, stream));
  K2B_FORWARD(UploadInts(ars, n + 1, L.arc_base, stream));
  *num_states_out = (int32_t)ts;
  *num_arcs_out = (int32_t)ta;
  return kOk;
}

int32_t k2b200_intersect_dense_pruned_emit(const k2b200_pruned_args *args, void *workspace,
                                           size_t workspace_bytes, void *stream_v,
                                           const k2b200_lattice_out *out) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  PrunedLayout L;
  K2B_FORWARD(MakePrunedLayout(args, reinterpret_cast<char *>(workspace), &L));
  K2B_REQUIRE(workspace != nullptr && workspace_bytes >= L.bytes, "workspace too small");
  K2B_REQUIRE(out && out->row_splits1 && out->row_ids1 && out->row_splits2 && out->row_ids2 &&
                  out->arcs && out->arc_map_a && out->arc_map_b,
              "NULL output pointer");
  K2B_REQUIRE((out->level_offsets == nullptr) == (out->level_splits == nullptr),
              "level_offsets and level_splits go together");
  FormatArgs f;
  f.g = L.g;
  f.out_rs1 = L.out_rs1;
  f.arc_base = L.arc_base;
  f.row_ids1 = out->row_ids1;
  f.row_splits2 = out->row_splits2;
  f.row_ids2 = out->row_ids2;
  f.arcs = reinterpret_cast<Arc *>(out->arcs);
  f.arc_map_a = out->arc_map_a;
  f.arc_map_b = out->arc_map_b;
  f.level_offsets = out->level_offsets;
  f.level_splits = out->level_splits;
  K2B_CUDA_OK(cudaMemcpyAsync(out->row_splits1, L.out_rs1, sizeof(int32_t) * (args->num_seqs + 1),
                              cudaMemcpyDeviceToDevice, stream));
  dim3 grid(L.g.T + 2, args->num_seqs);
  { FormatPruned<<<grid, 128, 0, stream>>>(f); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}


int32_t k2b200_online_decode_workspace_bytes(const k2b200_online_args *args, size_t *bytes) {
  OnlineLayout L;
  K2B_FORWARD(MakeOnlineLayout(args, nullptr, &L));
  K2B_REQUIRE(bytes != nullptr, "NULL bytes");
  *bytes = L.bytes;
  return kOk;
}

// Copies what stream `seq` has decoded so far into its slice of the arenas.
int32_t k2b200_online_decode_load(const k2b200_online_args *args, void *workspace, int32_t seq,
                                  const k2b200_online_stream *st, void *stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  OnlineLayout L;
  K2B_FORWARD(MakeOnlineLayout(args, reinterpret_cast<char *>(workspace), &L));
  K2B_REQUIRE(st != nullptr && seq >= 0 && seq < args->num_seqs, "bad stream");
  const SearchArgs &g = L.base.g;
  const int32_t h = args->h_hist[seq];
  K2B_REQUIRE(st->num_states <= g.cap_s && st->num_arcs <= g.cap_a,
              "the arena is smaller than what stream %d already holds", seq);
  const int64_t so = (int64_t)seq * (g.cap_s + 1), ao = (int64_t)seq * g.cap_a,
                fo = (int64_t)seq * (g.T + 2);
  auto copy = [&](void *dst, const void *src, size_t n) {
    return n == 0 ? cudaSuccess
                  : cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToDevice, stream);
  };
  K2B_CUDA_OK(copy(g.st_astate + so, st->astate, 4 * (size_t)st->num_states));
  K2B_CUDA_OK(copy(g.st_fwd + so, st->forward, 4 * (size_t)st->num_states));
  K2B_CUDA_OK(copy(g.st_arc0 + so, st->arc0, 4 * ((size_t)st->num_states + 1)));
  K2B_CUDA_OK(copy(g.arc_aidx + ao, st->arc_graph, 4 * (size_t)st->num_arcs));
  K2B_CUDA_OK(copy(g.arc_ll + ao, st->arc_score, 4 * (size_t)st->num_arcs));
  K2B_CUDA_OK(copy(g.arc_dest + ao, st->arc_dest, 4 * (size_t)st->num_arcs));
  K2B_CUDA_OK(copy(g.frame_s0 + fo, st->frame_state0, 4 * ((size_t)h + 2)));
  K2B_CUDA_OK(copy(g.frame_a0 + fo, st->frame_arc0, 4 * ((size_t)h + 2)));
  return kOk;
}

int32_t k2b200_online_decode_run(const k2b200_online_args *args, void *workspace,
                                 size_t workspace_bytes, void *stream_v, const float *h_beams_in,
                                 float *h_beams_out, int32_t *h_counts, int32_t *num_states_out,
                                 int32_t *num_arcs_out, int32_t *arena_full) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  OnlineLayout L;
  K2B_FORWARD(MakeOnlineLayout(args, reinterpret_cast<char *>(workspace), &L));
  K2B_REQUIRE(workspace != nullptr && workspace_bytes >= L.bytes, "workspace too small");
  K2B_REQUIRE(h_beams_in && h_beams_out && h_counts && num_states_out && num_arcs_out &&
                  arena_full, "NULL pointer");
  const int32_t n = args->num_seqs;
  K2B_CUDA_OK(cudaMemsetAsync(L.base.g.winner, 0, L.base.winner_bytes, stream));
  K2B_FORWARD(UploadInts(args->h_hist, n, L.hist, stream));
  K2B_FORWARD(UploadInts(reinterpret_cast<const int32_t *>(h_beams_in), n,
                         reinterpret_cast<int32_t *>(L.beam_in), stream));
  OnlineArgs o;
  o.g = L.base.g;
  o.hist = L.hist;
  o.beam_in = L.beam_in;
  o.beam_out = L.beam_out;
  o.chunk = L.chunk;
  o.hist_max = L.hist_max;
  {
    int dev = 0, sms = 0;
    K2B_CUDA_OK(cudaGetDevice(&dev));
    K2B_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    int32_t team = 1;
    while (team < 8 && n * team * 2 <= sms) team *= 2;
    if (args->team_ctas > 0) team = args->team_ctas;
    K2B_REQUIRE(team == 1 || team == 2 || team == 4 || team == 8, "team_ctas must be 1, 2, 4 or 8");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n * team);
    cfg.blockDim = dim3(kSearchThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = team;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    K2B_CUDA_OK(cudaLaunchKernelEx(&cfg, OnlineChunk, o));
    NoteLaunch();
  }
  std::vector<int32_t> h(4 * (size_t)n);
  K2B_CUDA_OK(cudaMemcpyAsync(h.data(), L.base.g.seq_out, sizeof(int32_t) * h.size(),
                              cudaMemcpyDeviceToHost, stream));
  K2B_CUDA_OK(cudaMemcpyAsync(h_beams_out, L.beam_out, sizeof(float) * n, cudaMemcpyDeviceToHost,
                              stream));
  K2B_CUDA_OK(cudaStreamSynchronize(stream));
  std::vector<int32_t> bases(2 * ((size_t)n + 1));
  int32_t *srs = bases.data(), *ars = bases.data() + n + 1;
  int64_t ts = 0, ta = 0;
  *arena_full = 0;
  for (int32_t i = 0; i < n; ++i) {
    if (h[4 * i + 3] == kSeqOverflow) *arena_full = 1;
    h_counts[2 * i] = h[4 * i];
    h_counts[2 * i + 1] = h[4 * i + 1];
    srs[i] = (int32_t)ts;
    ars[i] = (int32_t)ta;
    ts += h[4 * i] + 1;  // one final state per stream
    ta += h[4 * i + 1];
  }
  srs[n] = (int32_t)ts;
  ars[n] = (int32_t)ta;
  *num_states_out = *num_arcs_out = 0;
  if (*arena_full) return kOk;
  K2B_REQUIRE(ts < INT_MAX && ta < INT_MAX, "the lattice has too many states or arcs for int32");
  K2B_FORWARD(UploadInts(srs, n + 1, L.base.out_rs1, stream));
  K2B_FORWARD(UploadInts(ars, n + 1, L.base.arc_base, stream));
  *num_states_out = (int32_t)ts;
  *num_arcs_out = (int32_t)ta;
  return kOk;
}

int32_t k2b200_online_decode_emit(const k2b200_online_args *args, void *workspace,
                                  size_t workspace_bytes, void *stream_v,
                                  const k2b200_lattice_out *out) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  OnlineLayout L;
  K2B_FORWARD(MakeOnlineLayout(args, reinterpret_cast<char *>(workspace), &L));
  K2B_REQUIRE(workspace != nullptr && workspace_bytes >= L.bytes, "workspace too small");
  K2B_REQUIRE(out && out->row_splits1 && out->row_ids1 && out->row_splits2 && out->row_ids2 &&
                  out->arcs && out->arc_map_a, "NULL output pointer");
  FormatArgs f;
  f.g = L.base.g;
  f.out_rs1 = L.base.out_rs1;
  f.arc_base = L.base.arc_base;
  f.row_ids1 = out->row_ids1;
  f.row_splits2 = out->row_splits2;
  f.row_ids2 = out->row_ids2;
  f.arcs = reinterpret_cast<Arc *>(out->arcs);
  f.arc_map_a = out->arc_map_a;
  f.arc_map_b = nullptr;
  K2B_REQUIRE((out->level_offsets == nullptr) == (out->level_splits == nullptr),
              "level_offsets and level_splits go together");
  f.level_offsets = out->level_offsets;
  f.level_splits = out->level_splits;
  if (out->level_offsets != nullptr) {
    // stream i has (history + chunk + 2) layers: its frames and the final state
    std::vector<int32_t> lo(args->num_seqs + 1, 0);
    for (int32_t i = 0; i < args->num_seqs; ++i)
      lo[i + 1] = lo[i] + args->h_hist[i] + L.chunk + 2;
    K2B_FORWARD(UploadInts(lo.data(), args->num_seqs + 1, out->level_offsets, stream));
  }
  K2B_CUDA_OK(cudaMemcpyAsync(out->row_splits1, L.base.out_rs1,
                              sizeof(int32_t) * (args->num_seqs + 1), cudaMemcpyDeviceToDevice,
                              stream));
  dim3 grid(L.base.g.T + 2, args->num_seqs);
  { FormatOnline<<<grid, 128, 0, stream>>>(f, L.hist, L.chunk); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

// Copies stream `seq` out of its arena slice: num_states / num_arcs as reported by
// k2b200_online_decode_run, frame tables of (history + chunk + 2) entries.
int32_t k2b200_online_decode_store(const k2b200_online_args *args, void *workspace, int32_t seq,
                                   const k2b200_online_stream *st, void *stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  OnlineLayout L;
  K2B_FORWARD(MakeOnlineLayout(args, reinterpret_cast<char *>(workspace), &L));
  K2B_REQUIRE(st != nullptr && seq >= 0 && seq < args->num_seqs, "bad stream");
  const SearchArgs &g = L.base.g;
  const int32_t h = args->h_hist[seq] + L.chunk;
  const int64_t so = (int64_t)seq * (g.cap_s + 1), ao = (int64_t)seq * g.cap_a,
                fo = (int64_t)seq * (g.T + 2);
  auto copy = [&](const void *dst, const void *src, size_t n) {
    return n == 0 ? cudaSuccess
                  : cudaMemcpyAsync(const_cast<void *>(dst), src, n, cudaMemcpyDeviceToDevice,
                                    stream);
  };
  K2B_CUDA_OK(copy(st->astate, g.st_astate + so, 4 * (size_t)st->num_states));
  K2B_CUDA_OK(copy(st->forward, g.st_fwd + so, 4 * (size_t)st->num_states));
  K2B_CUDA_OK(copy(st->arc0, g.st_arc0 + so, 4 * ((size_t)st->num_states + 1)));
  K2B_CUDA_OK(copy(st->arc_graph, g.arc_aidx + ao, 4 * (size_t)st->num_arcs));
  K2B_CUDA_OK(copy(st->arc_score, g.arc_ll + ao, 4 * (size_t)st->num_arcs));
  K2B_CUDA_OK(copy(st->arc_dest, g.arc_dest + ao, 4 * (size_t)st->num_arcs));
  K2B_CUDA_OK(copy(st->frame_state0, g.frame_s0 + fo, 4 * ((size_t)h + 2)));
  K2B_CUDA_OK(copy(st->frame_arc0, g.frame_a0 + fo, 4 * ((size_t)h + 2)));
  return kOk;
}


// All streams in one launch: `streams` is a HOST array of num_seqs descriptors.
static int32_t CopyStreams(const k2b200_online_args *args, void *workspace,
                           const k2b200_online_stream *streams, bool load, cudaStream_t stream) {
  OnlineLayout L;
  K2B_FORWARD(MakeOnlineLayout(args, reinterpret_cast<char *>(workspace), &L));
  K2B_REQUIRE(streams != nullptr, "NULL streams");
  const SearchArgs &g = L.base.g;
  const int32_t n = args->num_seqs;
  std::vector<CopyJob> jobs;
  jobs.reserve(8 * (size_t)n);
  for (int32_t i = 0; i < n; ++i) {
    const k2b200_online_stream &st = streams[i];
    K2B_REQUIRE(st.num_states <= g.cap_s && st.num_arcs <= g.cap_a,
                "the arena is smaller than what stream %d holds", i);
    const int64_t h = args->h_hist[i] + (load ? 0 : L.chunk);
    const int64_t so = (int64_t)i * (g.cap_s + 1), ao = (int64_t)i * g.cap_a,
                  fo = (int64_t)i * (g.T + 2);
    struct { int32_t *arena; void *mine; int64_t count; } parts[8] = {
        {g.st_astate + so, st.astate, st.num_states},
        {g.st_fwd + so, st.forward, st.num_states},
        {g.st_arc0 + so, st.arc0, (int64_t)st.num_states + 1},
        {g.arc_aidx + ao, st.arc_graph, st.num_arcs},
        {reinterpret_cast<int32_t *>(g.arc_ll + ao), st.arc_score, st.num_arcs},
        {g.arc_dest + ao, st.arc_dest, st.num_arcs},
        {g.frame_s0 + fo, st.frame_state0, h + 2},
        {g.frame_a0 + fo, st.frame_arc0, h + 2}};
    for (const auto &p : parts) {
      CopyJob j;
      j.src = load ? reinterpret_cast<const int32_t *>(p.mine) : p.arena;
      j.dst = load ? p.arena : reinterpret_cast<int32_t *>(p.mine);
      j.count = p.count;
      jobs.push_back(j);
    }
  }
  static_assert(sizeof(CopyJob) % 4 == 0, "jobs travel as 32-bit words");
  K2B_FORWARD(UploadInts(reinterpret_cast<const int32_t *>(jobs.data()),
                         (int64_t)(jobs.size() * sizeof(CopyJob) / 4),
                         reinterpret_cast<int32_t *>(L.jobs), stream));
  { CopyMany<<<(unsigned)jobs.size(), 256, 0, stream>>>(L.jobs); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t k2b200_online_decode_load_all(const k2b200_online_args *args, void *workspace,
                                      const k2b200_online_stream *streams, void *stream_v) {
  return CopyStreams(args, workspace, streams, true, reinterpret_cast<cudaStream_t>(stream_v));
}

int32_t k2b200_online_decode_store_all(const k2b200_online_args *args, void *workspace,
                                       const k2b200_online_stream *streams, void *stream_v) {
  return CopyStreams(args, workspace, streams, false, reinterpret_cast<cudaStream_t>(stream_v));
}

}  // extern "C"

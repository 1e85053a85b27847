// Total scores of intersect_dense(a_fsas, b_fsas) in the log semiring, and their
// gradients, without ever writing the lattice.
//
// The reference computes a CTC / LF-MMI loss as
//   lattice = intersect_dense(graphs, dense, beam)      (k2/csrc/intersect_dense.cu)
//   tot     = lattice.get_tot_scores(log_semiring=True) (k2/csrc/fsa_utils.cu:708-1271)
// and back-propagates through the arc posteriors and the two arc maps
// (k2/python/k2/autograd.py:30-117, :511-664).  Every lattice state is a (frame,
// graph state) pair and every lattice arc a (frame, graph arc) pair, so the same
// numbers can be had from recursions over the dense (frame, state) grid that the
// pruning pass already uses:
//
//   1. the Viterbi grids and the cutoffs decide, exactly as for the lattice, which
//      (frame, state) and (frame, arc) pairs survive pruning;
//   2. alpha[t][s] and beta[t][s] are the log-semiring forward / backward scores
//      of the surviving pairs, carried as mantissa * 2^exponent so that the
//      frame-to-frame chain has no exp or log on it;
//   3. the posterior of (t, arc) is alpha[t][src] * w(arc) * p(t, label) *
//      beta[t+1][dest] / Z; summed over t it is the gradient of the graph arc,
//      summed over the arcs with one label it is the gradient of one element of
//      the dense matrix.  No arc map, no scatter through lattice-sized arrays.
//
// exp() of the dense scores is taken once per element in a parallel pass
// (ExpDense) shared by both recursions and the gradient pass.
#include <algorithm>
#include <type_traits>

#include "cp_async.cuh"
#include "intersect_internal.cuh"
#include "prob_math.cuh"

namespace k2b {

// The dense scores are repacked once per call, one 16-byte aligned record per row:
//   float  lp[cols4]   the scores themselves (for the pruning tests), then
//   double p[cols2]    exp(lp) (0 where that would be subnormal);
// element `cols` of both parts is the "no such column" entry (-inf / 0).  A whole
// record moves to shared memory with one bulk copy.
struct DensePack {
  int32_t cols, cols4, cols2, pitch;  // pitch in bytes, a multiple of 16
};
static DensePack MakeDensePack(int32_t cols) {
  DensePack d;
  d.cols = cols;
  d.cols4 = (cols + 1 + 3) & ~3;
  d.cols2 = (cols + 1 + 1) & ~1;
  d.pitch = 4 * d.cols4 + 8 * d.cols2;
  return d;
}
__device__ __forceinline__ const float *PackLp(const unsigned char *rec) {
  return reinterpret_cast<const float *>(rec);
}
__device__ __forceinline__ const double *PackP(const unsigned char *rec, const DensePack &d) {
  return reinterpret_cast<const double *>(rec + 4 * d.cols4);
}

// exp(arc.score) = f * 2^k of a graph arc.
struct __align__(16) ArcFactor {
  double f;
  int32_t k;
  int32_t pad;
};

// *low_flag is set when some finite score is below `low` (the shared-exponent
// recursion then leaves the whole batch to the per-state-exponent kernel).
__global__ void ExpDense(const float *__restrict__ scores, int64_t rows, DensePack d,
                         unsigned char *__restrict__ out, float low,
                         int32_t *__restrict__ low_flag) {
  const int64_t n = rows * d.cols4;
  bool found = false;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / d.cols4;
    const int32_t c = (int32_t)(idx - r * d.cols4);
    unsigned char *rec = out + r * d.pitch;
    const float lp = c < d.cols ? scores[r * d.cols + c] : -INFINITY;
    found |= lp < low && lp != -INFINITY;
    reinterpret_cast<float *>(rec)[c] = lp;
    if (c < d.cols2) {
      double p = exp((double)lp);
      if (p < 1e-300) p = 0.0;
      reinterpret_cast<double *>(rec + 4 * d.cols4)[c] = p;
    }
  }
  if (__any_sync(0xffffffffu, found) && (threadIdx.x & 31) == 0) atomicOr(low_flag, 1);
}

// t = m * 2^e with m in [1,2) from a positive normal double; (0, kZeroExp) for 0.
__device__ __forceinline__ double SplitExp(double t, int32_t *e) {
  if (t == 0.0) {
    *e = kZeroExp;
    return 0.0;
  }
  const int32_t hi = __double2hiint(t);
  const int32_t ex = (hi >> 20) - 1023;
  *e = ex;
  return __hiloint2double(hi - (ex << 20), __double2loint(t));
}

// 2^e, 0 below 2^-1000 and 2^1000 above that.
__device__ __forceinline__ double Pow2Clamped(int32_t e) {
  if (e < -1000) return 0.0;
  e = e > 1000 ? 1000 : e;
  return __longlong_as_double((long long)(1023 + e) << 52);
}

__global__ void ExpArcs(const Arc *__restrict__ arcs, int32_t n, ArcFactor *__restrict__ out) {
  int32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  ArcFactor a;
  ExpToMantExp(arcs[i].score, &a.f, &a.k);
  a.pad = 0;
  out[i] = a;
}

struct LaneSmem {
  int32_t s_pad, stages;
  int32_t vrow;  // bytes reserved per Viterbi row in a ring slot (a multiple of 16)
  size_t bytes;
};
constexpr size_t kChainSmemBudget = 220 * 1024;

// frames per unrolled group = ring slots = prefetch depth of the lane kernel (even)
constexpr int kChainGroup = 6, kChainGroupSmall = 2;

static LaneSmem PlanLaneSmem(const Layout &L, const DensePack &d, int group) {
  LaneSmem p;
  p.s_pad = (L.max_states + 3) & ~3;
  const size_t fixed = (sizeof(double) + sizeof(float)) * 2 * p.s_pad;
  // a row of S floats starting anywhere, widened to 16-byte boundaries on both sides
  p.vrow = ((L.max_states * 4 + 15) & ~15) + 16;
  p.bytes = fixed + ((size_t)d.pitch + 2 * p.vrow) * group;
  p.stages = p.bytes <= kChainSmemBudget ? group : 0;
  return p;
}

// Limits of the shared-exponent arithmetic below; outside them a graph is handed
// to the per-state-exponent kernel.
constexpr float kMaxAbsArcScore = 80.0f;   // |arc score| of every arc with a finite score
constexpr float kMinDenseScore = -200.0f;  // every finite dense score
constexpr int32_t kMinExponent = -480;     // binary exponent of every non-zero stored value

// ---------------------------------------------------------------------------
// The alpha / beta recursion for graphs whose states have at most four arcs each
// way (CTC): one thread per state, its arcs in registers.  grid = (2 directions,
// pairs), one CTA walks all frames of its pair.  Per frame three bulk copies (issued kU - 1 frames ahead by
// thread 0, completion on one mbarrier) bring the packed dense row and the two
// Viterbi rows of the level into a shared-memory ring of kU slots; every lane runs
// the reference's pruning test (intersect_dense.cu:430-470) on its arcs with the
// same fp32 expressions and adds the survivors' alpha[src] * exp(w) * exp(lp).
// The frame loop is unrolled by kU, so ring
// slots and buffers are compile-time constants.  Nothing is prefetched through
// registers: with the Viterbi scores fetched that way the frames still waited on
// global loads; the ring removed that wait.
//
// Arithmetic: all states of a level share one binary exponent K, so a value is a
// plain double v with alpha = v * 2^K and an arc costs two multiplies and an add.
// K follows the data in steps: every kChainGroup levels the values are scaled by
// 2^-e, e the exponent of the largest value of the level before (a shared-memory
// max), and every stored value's exponent is checked against the limits.  The
// grid receives (v, K) per state, the same (mantissa, exponent) format the
// per-state-exponent kernel writes.  A double spans 2^+-1022, far more than the
// survivors of one level normally differ by; when a surviving value does get
// within reach of the limits above, the graph is marked in `unfit` and the
// per-state-exponent kernel, which runs next, recomputes it.  The same happens
// when a wait on a copy gives up.
//
// `oth` holds, for the states of the previous frame, the Viterbi score the arc
// test needs (forward score walking forward, backward score walking backward), or
// -inf when that state was pruned - which fails the arc test by itself.
// ---------------------------------------------------------------------------
template <int kDeg, int kMaxThreads, int kU>
__global__ void __launch_bounds__(kMaxThreads)
GridChainLanes(const FsaInfo *__restrict__ infos, int32_t n, const Arc *__restrict__ arcs,
               const int32_t *__restrict__ a_row_splits2, const int32_t *__restrict__ in_splits,
               const int32_t *__restrict__ in_arcs, const unsigned char *__restrict__ dense,
               DensePack dp, const float *__restrict__ vfwd, const float *__restrict__ vbwd,
               const float *__restrict__ cutoffs, ProbState *__restrict__ alpha,
               ProbState *__restrict__ beta, double *__restrict__ tot,
               int32_t *__restrict__ unfit, const int32_t *__restrict__ low_flag,
               LaneSmem sm, int32_t wait_limit) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full[kU];
  __shared__ int32_t emax;
  __shared__ int32_t t_fail_sm;  // step whose wait gave up  // largest exponent among the values of a group's last level
  constexpr int32_t kNone = INT32_MIN;
  const int32_t i = blockIdx.y;
  const int dir = blockIdx.x;
  const FsaInfo f = infos[i];
  const int32_t S = f.num_states, Tk = f.tk, cols = dp.cols;
  const int tid = threadIdx.x, nt = blockDim.x;
  if (S == 0) {
    if (dir == 0 && tid == 0) tot[i] = -INFINITY;
    return;
  }
  const int32_t s_pad = sm.s_pad;
  // ring slot: the packed dense row, then the forward and the backward Viterbi row
  const uint32_t slot_bytes = (uint32_t)dp.pitch + 2u * (uint32_t)sm.vrow;
  unsigned char *ring = smem_raw;                                     // [kU][slot_bytes]
  double *pv = reinterpret_cast<double *>(ring + (size_t)kU * slot_bytes);  // [2][s_pad]
  float *oth = reinterpret_cast<float *>(pv + 2 * s_pad);             // [2][s_pad]

  const bool producer = tid == 0;  // issues the bulk copies
  const int32_t s = tid < S ? tid : -1;  // one thread per state
  // ---- this lane's arcs: dir 0 arcs entering s (other end = source), dir 1 leaving
  int32_t other_col[kDeg];  // other-end state | column << 16
  float w[kDeg];            // arc score, -inf for an unused slot
  double ew[kDeg];          // exp(w)
  // something is outside the limits of this arithmetic (kMinDenseScore is checked
  // on the whole matrix when it is repacked)
  bool risky = *low_flag != 0;
#pragma unroll
  for (int j = 0; j < kDeg; ++j) {
    other_col[j] = cols << 16;
    w[j] = -INFINITY;
    ew[j] = 0.0;
  }
  if (s >= 0) {
    const int32_t *gsplits = dir == 0 ? in_splits : a_row_splits2;
    const int32_t a0 = gsplits[f.state_off + s], a1 = gsplits[f.state_off + s + 1];
#pragma unroll
    for (int j = 0; j < kDeg; ++j) {
      const int32_t k = a0 + j;
      if (k < a1) {
        const Arc arc = arcs[dir == 0 ? in_arcs[k] : k];
        const int32_t c = arc.label + 1;
        if (c >= 0 && c < cols && arc.score != -INFINITY) {
          other_col[j] = (dir == 0 ? arc.src : arc.dest) | (c << 16);
          w[j] = arc.score;
          ew[j] = exp((double)arc.score);
          if (!(fabsf(arc.score) <= kMaxAbsArcScore)) risky = true;
        }
      }
    }
  }
  if (tid == 0) {
    for (int st = 0; st < kU; ++st) MbarInit(&full[st], 1);
    emax = kNone;
    MbarInitFence();
  }
  if (__syncthreads_or(risky)) {  // also orders the initialisation above
    if (tid == 0) atomicOr(&unfit[i], 2);
    return;
  }
  const float cutoff = cutoffs[i];
  const float *fgrid = vfwd + f.grid_off, *bgrid = vbwd + f.grid_off;
  ProbState *out = (dir == 0 ? alpha : beta) + f.grid_off;
  // ---- first level: the start (final) state holds 1 = 1.0 * 2^0 -------------------
  {
    const int64_t lv = dir == 0 ? 0 : Tk;
    for (int32_t q = tid; q < S; q += nt) {
      const float fu = fgrid[lv * S + q], bu = bgrid[lv * S + q];
      const bool keep = __fadd_rn(fu, bu) > cutoff;
      const bool one = keep && q == (dir == 0 ? 0 : S - 1);
      ProbState v;
      v.m = one ? 1.0 : 0.0;
      v.e = 0;
      v.pad = 0;
      pv[q] = v.m;
      oth[q] = keep ? (dir == 0 ? fu : bu) : -INFINITY;
      out[lv * S + q] = v;
      if (one) emax = 0;
    }
  }
  __syncthreads();
  // Step t (1..Tk) handles level t (forward) / Tk - t (backward) and reads dense
  // row t - 1 / Tk - t.  Steps come in groups of kU: step t0 + u (t0 = 1, 1 + kU, ...)
  // always finds its row in ring slot u and its operands in buffer u & 1.
  const int64_t step_stride = dir == 0 ? (int64_t)S : -(int64_t)S;
  const unsigned char *dense0 = dense + (int64_t)f.row0 * dp.pitch;
  // A row of a Viterbi grid starts at any multiple of 4 bytes; the bulk copy takes
  // the 16-byte aligned range around it (the grids sit inside the workspace with
  // other arrays before and after them), and the reader skips the leading floats.
  const unsigned vbytes = (((unsigned)S * 4u + 15u) & ~15u) + 16u;
  auto issue_row = [&](int32_t step, int32_t slot) {  // producer only
    if (step > Tk) return;
    const int64_t row = dir == 0 ? step - 1 : Tk - step;
    const int64_t lv = dir == 0 ? step : Tk - step;
    unsigned char *dst = ring + (size_t)slot * slot_bytes;
    const uintptr_t fa = reinterpret_cast<uintptr_t>(fgrid + lv * S) & ~(uintptr_t)15;
    const uintptr_t ba = reinterpret_cast<uintptr_t>(bgrid + lv * S) & ~(uintptr_t)15;
    MbarArriveExpectTx(&full[slot], (unsigned)dp.pitch + 2u * vbytes);
    BulkCopyG2S(dst, dense0 + row * dp.pitch, (unsigned)dp.pitch, &full[slot]);
    BulkCopyG2S(dst + dp.pitch, reinterpret_cast<const void *>(fa), vbytes, &full[slot]);
    BulkCopyG2S(dst + dp.pitch + sm.vrow, reinterpret_cast<const void *>(ba), vbytes,
                &full[slot]);
  };
  if (producer)
    for (int32_t step = 1; step < kU; ++step) issue_row(step, step - 1);

  const int32_t s_ld = s >= 0 ? s : 0;
  const int64_t first = dir == 0 ? 1 : Tk - 1;  // level of step 1
  int64_t pos = first * S + s_ld;  // grid index of this lane's state at step t
  double last = 0.0;
  int32_t K = 0;  // exponent shared by the stored values
  unsigned parity = 0;
  uint32_t rec_off = 0;  // ring offset of the frame's slot
  // A staged Viterbi row starts `skip` floats into its 16-byte aligned range; the
  // two grids have the same layout, so one value serves both.  It advances by S
  // (mod 4) per step.
  int32_t skip = (int32_t)(((reinterpret_cast<uintptr_t>(fgrid) >> 2) + (uintptr_t)(first * S)) & 3);
  const int32_t skip_step = (int32_t)(step_stride & 3);
  bool gave_up = false;
  for (int32_t t0 = 1; t0 <= Tk && !gave_up; t0 += kU) {
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int32_t t = t0 + u;
      if (t > Tk) break;
      // (the usual limit as a constant: the polling loop the compiler makes of it is the cheaper one)
      const bool late = !MbarTryWait(&full[u], parity) &&
                        !(wait_limit == 4000000 ? MbarWaitBounded(&full[u], parity)
                                                : MbarWaitBounded(&full[u], parity, wait_limit));
      // the previous frame is complete; nobody reads its ring slot any more
      if (__syncthreads_or(late)) {  // uniform
        gave_up = true;
        if (tid == 0) t_fail_sm = t;  // shared memory: nothing of it stays live in the loop
        break;
      }
      if (producer) {
        // the slot the previous frame used takes the rows of step t + kU - 1
        issue_row(t + kU - 1, (u + kU - 1) % kU);
        if (u == 1) emax = kNone;  // read by everyone during the frame before
      }
      double scale = 1.0;
      if (u == 0) {  // once per group: renormalise by the exponent of the largest value
        const int32_t e_prev = emax;
        const int32_t shift = e_prev == kNone ? 0 : e_prev;
        K += shift;
        scale = __longlong_as_double((long long)(1023 - shift) << 52);
      }
      const double *prev = pv + (u & 1) * s_pad;
      double *cur = pv + ((u + 1) & 1) * s_pad;
      const float *po = oth + (u & 1) * s_pad;
      float *co = oth + ((u + 1) & 1) * s_pad;
      // ring slot u, as a running offset (kept opaque so that the unrolled frames
      // do not each pin their own pointers in registers)
      rec_off = u == 0 ? 0u : rec_off + slot_bytes;
      asm volatile("" : "+r"(rec_off));
      const unsigned char *rec = ring + rec_off;
      const float *lprow = PackLp(rec);
      const double *prow = PackP(rec, dp);
      const float fu = reinterpret_cast<const float *>(rec + dp.pitch)[skip + s_ld];
      const float bu = reinterpret_cast<const float *>(rec + dp.pitch + sm.vrow)[skip + s_ld];
      skip = (skip + skip_step) & 3;
      const bool keep = s >= 0 && __fadd_rn(fu, bu) > cutoff;
      double sum = 0.0;
      if (__any_sync(0xffffffffu, keep)) {  // most warps of a sparse lattice skip this
#pragma unroll
        for (int j = 0; j < kDeg; ++j) {
          const int32_t o_idx = other_col[j] & 0xffff, c = other_col[j] >> 16;
          const float sc = __fadd_rn(w[j], lprow[c]);
          const float o = po[o_idx];
          const float through = dir == 0 ? __fadd_rn(__fadd_rn(o, sc), bu)
                                         : __fadd_rn(__fadd_rn(fu, sc), o);
          // computed for every arc of the warp and selected: cheaper than a divergent
          // branch per arc
          const double term = prev[o_idx] * ew[j] * prow[c];
          sum += (keep && through > cutoff) ? term : 0.0;
        }
      }
      const double v = u == 0 ? sum * scale : sum;
      const int32_t vhi = __double2hiint(v);  // v >= 0: the exponent is vhi >> 20
      if (s >= 0) {
        cur[s] = v;
        co[s] = keep ? (dir == 0 ? fu : bu) : -INFINITY;
        if (keep || t == Tk) {  // pruned states of the grid are read on the last level only
          ProbState r;
          r.m = v;
          r.e = K;
          r.pad = 0;
          out[pos] = r;
          last = v;
          risky |= v != 0.0 && vhi < ((1023 + kMinExponent) << 20);
        }
      }
      pos += step_stride;
      if (u == kU - 1) {  // the next group renormalises by this level's largest value
        int32_t ex = (s >= 0 && v != 0.0) ? (vhi >> 20) - 1023 : kNone;
        ex = __reduce_max_sync(0xffffffffu, ex);
        if ((tid & 31) == 0 && ex != kNone) atomicMax(&emax, ex);
      }
    }
    parity ^= 1u;
  }
  const int32_t any_risky = __syncthreads_or(risky);
  if (gave_up) {
    if (tid == 0) {
      atomicOr(&unfit[i], 2);
      // copies may still be in flight towards this CTA's shared memory (the rows of steps
      // t_fail .. t_fail + kU - 2): wait for each, with a limit, before the CTA retires
      const int32_t t_fail = t_fail_sm;
      for (int32_t k = t_fail; k <= min(t_fail + kU - 2, Tk); ++k)
        MbarWaitBounded(&full[(k - 1) % kU], (unsigned)((k - 1) / kU) & 1u);
    }
    __syncthreads();
    return;
  }
  if (any_risky) {
    if (tid == 0) atomicOr(&unfit[i], 2);
    return;
  }
  if (dir == 0 && s == S - 1)
    tot[i] = last == 0.0 ? -INFINITY : log(last) + (double)K * 0.69314718055994530942;
}

// ---------------------------------------------------------------------------
// Arc survival masks for planned graphs.  The pruning test of a (frame, arc) pair
// is needed three times - by the forward recursion (arcs grouped by destination),
// by the backward recursion and by the gradients (arcs grouped by source).  The
// recursions are chains of dependent frames, where every instruction counts; the
// tests have no such dependency.  So they run here, for all frames at once:
//   masks[(dir * total_levels + level_off(i) + r) * kLaneThreads + lane], bit j =
//   slot j of that lane survives at row r
// with r the step t = 1..T of the forward recursion (dir 0) or the level u = 0..T-1
// the arc leaves from (dir 1).  grid = (row chunks, pairs, 2 directions); the CTA
// stages the Viterbi scores of its levels (-inf for pruned states) and the dense
// scores of its rows in shared memory.  Also enforces kMinDenseScore (on every finite
// element of the rows, a little stricter than on surviving arcs only).
// ---------------------------------------------------------------------------
// The state pitch of the staged scores and the rows per CTA are compile-time, and the row loop
// is unrolled, so the score of an arc's other end is one load at (byte offset of that state,
// fixed for the call) + constant.  Walking forward in a graph where every state has one
// entering label the dense score of a lane's arcs is one load per row.
template <int kDeg, int kSPad, int kMaskRows>
__global__ void __launch_bounds__(kLaneThreads)
ArcMasks(const FsaInfo *__restrict__ infos, int32_t n, int64_t total_levels,
         const Arc *__restrict__ arcs, const int32_t *__restrict__ a_row_splits2,
         const int32_t *__restrict__ in_splits, const int32_t *__restrict__ in_arcs,
         const unsigned char *__restrict__ dense, DensePack dp,
         const float *__restrict__ vfwd, const float *__restrict__ vbwd,
         const float *__restrict__ cutoffs, const int32_t *__restrict__ plan,
         int32_t *__restrict__ unfit, unsigned char *__restrict__ masks) {
  static_assert(kDeg <= 8, "one byte per lane");
  constexpr int32_t s_pad = kSPad;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int32_t i = blockIdx.y, dir = blockIdx.z;
  if (unfit[i] & 1) return;
  const FsaInfo f = infos[i];
  const int32_t S = f.num_states, Tk = f.tk, cols = dp.cols;
  const int32_t r0 = blockIdx.x * kMaskRows + (dir == 0 ? 1 : 0);
  const int32_t r_end = dir == 0 ? Tk + 1 : Tk;
  if (S == 0 || r0 >= r_end) return;
  const int32_t nf = min(kMaskRows, r_end - r0);
  const int32_t lb = dir == 0 ? r0 - 1 : r0;  // first staged level and first dense row
  const int tid = threadIdx.x, nt = blockDim.x;
  float *fo = reinterpret_cast<float *>(smem_raw);  // [kMaskRows + 1][s_pad]
  float *bo = fo + (kMaskRows + 1) * s_pad;         // [kMaskRows + 1][s_pad]
  float *lp = bo + (kMaskRows + 1) * s_pad;         // [kMaskRows][cols4]
  const float cutoff = cutoffs[i];
  const float *fgrid = vfwd + f.grid_off, *bgrid = vbwd + f.grid_off;
  for (int32_t idx = tid; idx < (nf + 1) * S; idx += nt) {
    const int32_t l = idx / S, q = idx - l * S;
    const int64_t gi = (int64_t)(lb + l) * S + q;
    const float fu = fgrid[gi], bu = bgrid[gi];
    const bool keep = __fadd_rn(fu, bu) > cutoff;
    fo[l * s_pad + q] = keep ? fu : -INFINITY;
    bo[l * s_pad + q] = keep ? bu : -INFINITY;
  }
  bool risky = false;
  for (int32_t idx = tid; idx < nf * dp.cols4; idx += nt) {
    const int32_t l = idx / dp.cols4, c = idx - l * dp.cols4;
    const float v = PackLp(dense + ((int64_t)f.row0 + lb + l) * dp.pitch)[c];
    lp[idx] = v;
    // checked per row element rather than per surviving arc: stricter, and off the
    // inner loop
    risky |= v < kMinDenseScore && v != -INFINITY;
  }
  int32_t s = -1, g = 0, G = 1;
  {
    const int32_t code = plan[((int64_t)dir * n + i) * kLaneThreads + tid];
    if (code >= 0) {
      s = code & 0xffff;
      g = (code >> 16) & 0xff;
      G = code >> 24;
    }
  }
  // byte offsets of an arc's other end in a level of staged scores and of its column in a row
  uint32_t other_off[kDeg], col_off[kDeg];
  float w[kDeg];
  int32_t col0 = -1;
  bool same = true;
#pragma unroll
  for (int j = 0; j < kDeg; ++j) {
    other_off[j] = 0;
    col_off[j] = 0;
    w[j] = -INFINITY;
  }
  if (s >= 0) {
    const int32_t *gsplits = dir == 0 ? in_splits : a_row_splits2;
    const int32_t a0 = gsplits[f.state_off + s], a1 = gsplits[f.state_off + s + 1];
#pragma unroll
    for (int j = 0; j < kDeg; ++j) {
      const int32_t k = a0 + g + j * G;
      if (k < a1) {
        const Arc arc = arcs[dir == 0 ? in_arcs[k] : k];
        const int32_t c = arc.label + 1;
        if (c >= 0 && c < cols && arc.score != -INFINITY) {
          other_off[j] = 4u * (uint32_t)(dir == 0 ? arc.src : arc.dest);
          col_off[j] = 4u * (uint32_t)c;
          w[j] = arc.score;
          if (col0 < 0) col0 = c;
          else if (c != col0) same = false;
        }
      }
    }
  }
  const bool hoist = __all_sync(0xffffffffu, same);
  const uint32_t col0_off = 4u * (uint32_t)(col0 < 0 ? 0 : col0);
  __syncthreads();
  // (a slot without an arc has w = -inf: it fails the test like any pruned arc)
  unsigned char *out = masks + ((int64_t)dir * total_levels + f.level_off + r0) * kLaneThreads + tid;
  const int32_t s_ld = s >= 0 ? s : 0;
  // dir 0: arcs from level k into level k + 1 (own); dir 1: from level k (own) to k + 1
  const float *own_p = (dir == 0 ? bo + s_pad : fo) + s_ld;
  const unsigned char *oth_p = reinterpret_cast<const unsigned char *>(dir == 0 ? fo : bo + s_pad);
  const unsigned char *lp_p = reinterpret_cast<const unsigned char *>(lp);
  const uint32_t lp_stride = 4u * (uint32_t)dp.cols4;
  auto at = [](const unsigned char *base, uint32_t off) {
    return *reinterpret_cast<const float *>(base + off);
  };
  constexpr int kUnroll = 4;
  static_assert(kMaskRows % kUnroll == 0, "rows per CTA");
  for (int32_t k0 = 0; k0 < nf; k0 += kUnroll) {
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (k0 + u >= nf) break;
      uint32_t bits = 0;
      const float own = s >= 0 ? own_p[u * s_pad] : -INFINITY;
      if (own != -INFINITY) {
        const unsigned char *oth = oth_p + u * (4 * s_pad);
        const unsigned char *lprow = lp_p + u * lp_stride;
        if (hoist) {
          const float x = at(lprow, col0_off);
#pragma unroll
          for (int j = 0; j < kDeg; ++j) {
            const float sc = __fadd_rn(w[j], x);
            const float o = at(oth, other_off[j]);
            const float through = dir == 0 ? __fadd_rn(__fadd_rn(o, sc), own)
                                           : __fadd_rn(__fadd_rn(own, sc), o);
            if (through > cutoff) bits |= 1u << j;
          }
        } else {
#pragma unroll
          for (int j = 0; j < kDeg; ++j) {
            const float sc = __fadd_rn(w[j], at(lprow, col_off[j]));
            const float o = at(oth, other_off[j]);
            const float through = dir == 0 ? __fadd_rn(__fadd_rn(o, sc), own)
                                           : __fadd_rn(__fadd_rn(own, sc), o);
            if (through > cutoff) bits |= 1u << j;
          }
        }
      }
      out[(int64_t)u * kLaneThreads] = (unsigned char)bits;
    }
    own_p += kUnroll * s_pad;
    oth_p += kUnroll * 4 * s_pad;
    lp_p += kUnroll * lp_stride;
    out += (int64_t)kUnroll * kLaneThreads;
  }
  if (__syncthreads_or(risky) && tid == 0) atomicOr(&unfit[i], 2);
}

// ---------------------------------------------------------------------------
// The alpha / beta recursion for planned graphs, driven by the masks of ArcMasks:
// same arithmetic as GridChainLanes, but a frame needs no Viterbi score and no test - one
// mask byte per lane says which of its arcs to add.  The packed dense rows and the rows of
// mask bytes of kU consecutive frames are one block of memory each (ascending walking
// forward, descending walking backward): a batch of kU frames arrives by TWO bulk copies,
// three batches in a ring (a pair of copies per frame kept thread 0, and with it every
// barrier, busy).  The frames of a batch are unrolled; there is one frame loop per kind
// of CTA (see kHoist) so that the code a CTA runs stays small.  When all arcs of a CTA's
// lanes carry the label of their state (walking forward in a graph where every state has
// one entering label), exp(dense score) multiplies the sum once per state instead of every
// term.  Every state is written to the grid (0 for pruned ones).
// ---------------------------------------------------------------------------
constexpr int kMaskedBatches = 3;  // batches of kU frames in the ring

template <int kDeg, int kU>
__global__ void __launch_bounds__(kLaneThreads)
GridChainMasked(const FsaInfo *__restrict__ infos, int32_t n, int64_t total_levels,
                const Arc *__restrict__ arcs, const int32_t *__restrict__ a_row_splits2,
                const int32_t *__restrict__ in_splits, const int32_t *__restrict__ in_arcs,
                const unsigned char *__restrict__ dense, DensePack dp,
                const unsigned char *__restrict__ masks, const float *__restrict__ vfwd,
                const float *__restrict__ vbwd, const float *__restrict__ cutoffs,
                ProbState *__restrict__ alpha, ProbState *__restrict__ beta,
                double *__restrict__ tot, const int32_t *__restrict__ plan,
                int32_t *__restrict__ unfit, int32_t s_pad, int32_t wait_limit) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t full[kMaskedBatches];
  __shared__ int32_t emax;
  __shared__ int32_t t_fail_sm;  // batch whose wait gave up
  constexpr int32_t kNone = INT32_MIN;
  const int32_t i = blockIdx.y;
  const int dir = blockIdx.x;
  if (unfit[i]) return;  // no plan, or outside the limits: the fallback kernel takes it
  const FsaInfo f = infos[i];
  const int32_t S = f.num_states, Tk = f.tk, cols = dp.cols;
  const int tid = threadIdx.x, nt = blockDim.x;
  if (S == 0) {
    if (dir == 0 && tid == 0) tot[i] = -INFINITY;
    return;
  }
  (void)s_pad;
  constexpr int kSPad = kLaneThreads;  // a planned graph has at most that many states
  // a batch: kU packed dense rows, then kU rows of mask bytes
  const uint32_t batch_bytes = (uint32_t)kU * ((uint32_t)dp.pitch + (uint32_t)kLaneThreads);
  unsigned char *ring = smem_raw;                                  // [kMaskedBatches][batch_bytes]
  double *pv = reinterpret_cast<double *>(ring + (size_t)kMaskedBatches * batch_bytes);  // [2][kSPad]
  int32_t s = -1, g = 0, G = 1;
  {
    const int32_t code = plan[((int64_t)dir * n + i) * kLaneThreads + tid];
    if (code >= 0) {
      s = code & 0xffff;
      g = (code >> 16) & 0xff;
      G = code >> 24;
    }
  }
  // byte offsets of an arc's neighbour in a state buffer and of its column in a dense row
  uint32_t other_off[kDeg], col_off[kDeg];
  double ew[kDeg];
  bool risky = false;
  int32_t col0 = -1;
  bool same = true;
#pragma unroll
  for (int j = 0; j < kDeg; ++j) {
    other_off[j] = 0;
    col_off[j] = 8u * (uint32_t)cols;  // the padding column: 0
    ew[j] = 0.0;
  }
  if (s >= 0) {
    const int32_t *gsplits = dir == 0 ? in_splits : a_row_splits2;
    const int32_t a0 = gsplits[f.state_off + s], a1 = gsplits[f.state_off + s + 1];
#pragma unroll
    for (int j = 0; j < kDeg; ++j) {
      const int32_t k = a0 + g + j * G;
      if (k < a1) {
        const Arc arc = arcs[dir == 0 ? in_arcs[k] : k];
        const int32_t c = arc.label + 1;
        if (c >= 0 && c < cols && arc.score != -INFINITY) {
          other_off[j] = 8u * (uint32_t)(dir == 0 ? arc.src : arc.dest);
          col_off[j] = 8u * (uint32_t)c;
          ew[j] = exp((double)arc.score);
          if (!(fabsf(arc.score) <= kMaxAbsArcScore)) risky = true;
          if (col0 < 0) col0 = c;
          else if (c != col0) same = false;
        }
      }
    }
  }
  const bool hoist = __syncthreads_and(same);  // uniform over the CTA
  const uint32_t col0_off = 8u * (uint32_t)(col0 < 0 ? 0 : col0);  // no arc: the sum is 0
  if (tid == 0) {
    for (int st = 0; st < kMaskedBatches; ++st) MbarInit(&full[st], 1);
    emax = kNone;
    MbarInitFence();
  }
  if (__syncthreads_or(risky)) {
    if (tid == 0) atomicOr(&unfit[i], 2);
    return;
  }
  ProbState *out = (dir == 0 ? alpha : beta) + f.grid_off;
  {  // first level: 1 for the start (final) state if it survives, 0 elsewhere
    const int64_t lv = dir == 0 ? 0 : Tk;
    const int32_t q1 = dir == 0 ? 0 : S - 1;
    const bool one_ok = __fadd_rn(vfwd[f.grid_off + lv * S + q1], vbwd[f.grid_off + lv * S + q1]) >
                        cutoffs[i];
    for (int32_t q = tid; q < S; q += nt) {
      ProbState v;
      v.m = (q == q1 && one_ok) ? 1.0 : 0.0;
      v.e = 0;
      v.pad = 0;
      pv[q] = v.m;
      out[lv * S + q] = v;
    }
    if (tid == 0 && one_ok) emax = 0;
  }
  __syncthreads();
  const int64_t step_stride = dir == 0 ? (int64_t)S : -(int64_t)S;
  const unsigned char *dense_rows = dense + (int64_t)f.row0 * dp.pitch;
  const uint32_t row_bytes = (uint32_t)dp.pitch, lp_bytes = 4u * (uint32_t)dp.cols4;
  const unsigned char *mask0 = masks + ((int64_t)dir * total_levels + f.level_off) * kLaneThreads;
  const int32_t num_batches = (Tk + kU - 1) / kU;
  // thread 0: the rows of steps b * kU + 1 .. of batch b, as two copies.  Walking forward the
  // dense rows and the mask rows of consecutive steps ascend, walking backward they descend:
  // either way they are one block of memory; frame u of the batch is row u of the block
  // (forward) or row nf - 1 - u (backward).
  auto issue_batch = [&](int32_t b) {
    if (b >= num_batches) return;
    const int32_t t_first = b * kU + 1, nf = min(kU, Tk - b * kU);
    const int64_t row_lo = dir == 0 ? t_first - 1 : Tk - t_first - nf + 1;  // dense rows
    const int64_t r_lo = dir == 0 ? t_first : Tk - t_first - nf + 1;        // mask rows
    const int32_t slot = b % kMaskedBatches;
    unsigned char *dst = ring + (size_t)slot * batch_bytes;
    MbarArriveExpectTx(&full[slot], (unsigned)nf * (row_bytes + (unsigned)kLaneThreads));
    BulkCopyG2S(dst, dense_rows + row_lo * row_bytes, (unsigned)nf * row_bytes, &full[slot]);
    BulkCopyG2S(dst + kU * row_bytes, mask0 + r_lo * kLaneThreads, (unsigned)nf * kLaneThreads,
                &full[slot]);
  };
  if (tid == 0)
    for (int32_t b = 0; b < kMaskedBatches - 1; ++b) issue_batch(b);
  const int32_t g_max = __reduce_max_sync(0xffffffffu, G);  // widest lane group of this warp
  const int32_t s_ld = s >= 0 ? s : 0;
  int64_t pos = (dir == 0 ? 1 : Tk - 1) * (int64_t)S + s_ld;
  double last = 0.0;
  int32_t K = 0;
  bool gave_up = false;
  // the frame loop once per kind of CTA, so that the unrolled code of only one is fetched
  auto frames = [&](auto hoist_tag) {
    constexpr bool kHoist = decltype(hoist_tag)::value;
    for (int32_t b = 0; b < num_batches; ++b) {
      const int32_t slot = b % kMaskedBatches;
      const unsigned parity = (unsigned)(b / kMaskedBatches) & 1u;
      // (the usual limit as a constant: the polling loop the compiler makes of it is the cheaper one)
      const bool late = !MbarTryWait(&full[slot], parity) &&
                        !(wait_limit == 4000000 ? MbarWaitBounded(&full[slot], parity)
                                                : MbarWaitBounded(&full[slot], parity, wait_limit));
      // also: the last frame of the batch before is complete; nobody reads its slot any more
      if (__syncthreads_or(late)) {  // uniform
        gave_up = true;
        if (tid == 0) t_fail_sm = b;  // shared memory: nothing of it stays live in the loop
        break;
      }
      if (tid == 0) issue_batch(b + kMaskedBatches - 1);
      const unsigned char *base = ring + (size_t)slot * batch_bytes;
      const int32_t nf = min(kU, Tk - b * kU);
      const int pb = (kU % 2 == 0) ? 0 : (b & 1);  // parity of the state buffers at the batch's start
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        if (u >= nf) break;
        if (u > 0) __syncthreads();  // the values of the frame before are complete
        if (tid == 0 && u == (kU > 1 ? 1 : 0) && kU > 1) emax = kNone;  // read during frame 0
        double scale = 1.0;
        if (u == 0) {
          const int32_t e_prev = emax;
          const int32_t shift = e_prev == kNone ? 0 : e_prev;
          K += shift;
          scale = __longlong_as_double((long long)(1023 - shift) << 52);
        }
        const unsigned char *prev = reinterpret_cast<const unsigned char *>(pv + ((pb + u) & 1) * kSPad);
        double *cur = pv + ((pb + u + 1) & 1) * kSPad;
        const int32_t idx = dir == 0 ? u : nf - 1 - u;
        const unsigned char *prow = base + (uint32_t)idx * row_bytes + lp_bytes;
        const uint32_t m = (base + kU * row_bytes + (uint32_t)idx * kLaneThreads)[tid];
        auto at = [](const unsigned char *p0, uint32_t off) {
          return *reinterpret_cast<const double *>(p0 + off);
        };
        double sum = 0.0;
        if (__any_sync(0xffffffffu, m != 0)) {
          double sum1 = 0.0;  // two partial sums: half the chain of dependent additions
          if (kHoist) {
#pragma unroll
            for (int j = 0; j < kDeg; j += 2) {
              if (m & (1u << j)) sum = fma(at(prev, other_off[j]), ew[j], sum);
              if (j + 1 < kDeg && (m & (2u << j)))
                sum1 = fma(at(prev, other_off[j + 1]), ew[j + 1], sum1);
            }
          } else {
#pragma unroll
            for (int j = 0; j < kDeg; j += 2) {
              if (m & (1u << j))
                sum = fma(at(prev, other_off[j]) * ew[j], at(prow, col_off[j]), sum);
              if (j + 1 < kDeg && (m & (2u << j)))
                sum1 = fma(at(prev, other_off[j + 1]) * ew[j + 1], at(prow, col_off[j + 1]), sum1);
            }
          }
          sum += sum1;
#pragma unroll
          for (int32_t d = 16; d > 0; d >>= 1) {
            if (d < g_max) {  // warp-uniform: no group of this warp is that wide
              const double so = __shfl_down_sync(0xffffffffu, sum, d);
              if (g + d < G) sum += so;
            }
          }
          if (kHoist) sum *= at(prow, col0_off);
        }
        const double v = u == 0 ? sum * scale : sum;
        const int32_t vhi = __double2hiint(v);
        if (s >= 0 && g == 0) {
          cur[s] = v;
          ProbState r;
          r.m = v;
          r.e = K;
          r.pad = 0;
          out[pos] = r;
          last = v;
          risky |= v != 0.0 && vhi < ((1023 + kMinExponent) << 20);
        }
        pos += step_stride;
        if (u == kU - 1) {  // the next batch renormalises by this level's largest value
          if (kU == 1) {    // no frame in between in which to reset the maximum
            __syncthreads();
            if (tid == 0) emax = kNone;
            __syncthreads();
          }
          int32_t ex = (s >= 0 && g == 0 && v != 0.0) ? (vhi >> 20) - 1023 : kNone;
          ex = __reduce_max_sync(0xffffffffu, ex);
          if ((tid & 31) == 0 && ex != kNone) atomicMax(&emax, ex);
        }
      }
    }
  };
  if (hoist) frames(std::true_type{}); else frames(std::false_type{});
  const int32_t any_risky = __syncthreads_or(risky);
  if (gave_up) {
    if (tid == 0) {
      atomicOr(&unfit[i], 2);
      // the copies still in flight (batches b_fail .. b_fail + kMaskedBatches - 2) land before
      // the CTA retires
      const int32_t b_fail = t_fail_sm;
      for (int32_t b = b_fail; b <= min(b_fail + kMaskedBatches - 2, num_batches - 1); ++b)
        MbarWaitBounded(&full[b % kMaskedBatches], (unsigned)(b / kMaskedBatches) & 1u);
    }
    __syncthreads();
    return;
  }
  if (any_risky) {
    if (tid == 0) atomicOr(&unfit[i], 2);
    return;
  }
  if (dir == 0 && s == S - 1 && g == 0)
    tot[i] = last == 0.0 ? -INFINITY : log(last) + (double)K * 0.69314718055994530942;
}

// Writes the fixed-point sums gb[frame][col] of a CTA's frames (2^-31 units, times tg)
// as dL/d(dense score): into the score matrix layout grad[(row0 + u0 + frame) * cols +
// col], or - when lp_row0 >= 0 - straight into the layout of the log-probs the
// DenseFsaVec was made from, grad[(lp_row0 + u0 + frame) * lp_cols + col - 1]: column 0
// (the final-arc column) has no log-prob behind it and is dropped, as the adjoint of
// the DenseFsaVec layout drops it.
__device__ __forceinline__ void StoreDenseGrad(float *__restrict__ grad, int32_t row0, int32_t u0,
                                               int32_t cols, const uint32_t *gb, int32_t elems,
                                               float tg, int32_t exclusive_rows,
                                               int32_t lp_row0, int32_t lp_cols, int32_t tid,
                                               int32_t nt) {
  if (lp_row0 < 0) {
    float *grow = grad + ((int64_t)row0 + u0) * cols;
    for (int32_t k = tid; k < elems; k += nt) {
      const uint32_t fixed = gb[k];
      if (fixed != 0u) {
        const float v = tg * ((float)fixed * (1.0f / 2147483648.0f));
        if (exclusive_rows) grow[k] = v; else atomicAdd(&grow[k], v);
      }
    }
    return;
  }
  float *base = grad + ((int64_t)lp_row0 + u0) * lp_cols;
  for (int32_t k = tid; k < elems; k += nt) {
    const uint32_t fixed = gb[k];
    if (fixed != 0u) {
      const int32_t fl = k / cols, c = k - fl * cols;
      if (c > 0) {
        const float v = tg * ((float)fixed * (1.0f / 2147483648.0f));
        float *p = base + (int64_t)fl * lp_cols + (c - 1);
        if (exclusive_rows) *p = v; else atomicAdd(p, v);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Gradients.  grid = (frame chunks, pairs): frames do not depend on one another,
// so the GPU is filled with (pair, chunk) CTAs and every warp of a CTA takes whole
// frames.  For its frame u the warp scans the states 32 at a time, keeps the
// surviving ones as a bit mask, and hands them to groups of 2^lanes_log2 lanes;
// the lanes of a group walk the arcs leaving the state, run the pruning test and
// add posterior = alpha[u][src] * w * p(u, label) * beta[u+1][dest] / Z to
//   * gb[u - u0][label + 1] in shared memory, written to grad_b once per CTA;
//   * ga[arc] in shared memory (global memory for very large graphs), added to
//     grad_a once per CTA.
// With kStage the warp first copies what the arcs of the frame can touch - beta
// and the backward Viterbi score of level u + 1 - into its own shared-memory
// scratch, so that the arc loop has no dependent global loads (small, dense
// graphs); without it those are gathered from global memory (large sparse ones).
// ---------------------------------------------------------------------------
struct __align__(16) NextState {
  double m;
  int32_t e;
  float bo;  // backward Viterbi score, -inf when the state was pruned
};

constexpr int kGradWarps = 8;

template <bool kStage>
__global__ void __launch_bounds__(kGradWarps * 32)
GridGradWarp(const FsaInfo *__restrict__ infos, const Arc *__restrict__ arcs,
             const ArcFactor *__restrict__ arc_factors,
             const int32_t *__restrict__ a_row_splits2, const unsigned char *__restrict__ dense,
             DensePack dp, const float *__restrict__ vfwd, const float *__restrict__ vbwd,
             const float *__restrict__ cutoffs, const ProbState *__restrict__ alpha,
             const ProbState *__restrict__ beta, const double *__restrict__ tot_grad,
             int32_t tot_grad_stride, float *__restrict__ grad_a, float *__restrict__ grad_b,
             int32_t frames_per_cta, int32_t lanes_log2, int32_t s_pad, int32_t ga_in_smem,
             int32_t exclusive_rows, const int32_t *__restrict__ only_noplan,
             const int32_t *__restrict__ lp_row, int32_t lp_cols,
             const int32_t *__restrict__ served) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int32_t i = blockIdx.y;
  if (served != nullptr && *served) return;  // GridGradStates wrote the gradients
  if (only_noplan != nullptr && !(only_noplan[i] & 1)) return;  // the lane kernel took it
  const FsaInfo f = infos[i];
  const int32_t S = f.num_states, A = f.num_arcs, Tk = f.tk, cols = dp.cols;
  const int32_t u0 = blockIdx.x * frames_per_cta;
  if (S == 0 || u0 >= Tk) return;
  const int32_t u1 = min(u0 + frames_per_cta, Tk);
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5;
  NextState *nb_all = reinterpret_cast<NextState *>(smem_raw);  // [warps][s_pad] if kStage
  // sums of posteriors in fixed point (integer atomics are native in shared memory,
  // float ones are compare-and-swap loops; the sums also become order independent):
  // gb per (frame, column) in 2^-31 units (a sum of at most 1), ga per arc in 2^-26
  // units (at most one per frame of the chunk, frames_per_cta <= 32)
  uint32_t *gb = reinterpret_cast<uint32_t *>(nb_all + (kStage ? kGradWarps * s_pad : 0));
  uint32_t *ga = gb + (((size_t)frames_per_cta * cols + 3) & ~(size_t)3);  // [A] when ga_in_smem
  const ProbState *al = alpha + f.grid_off, *be = beta + f.grid_off;
  const ProbState z = al[(int64_t)Tk * S + (S - 1)];
  if (z.m == 0.0) return;  // no path survives: all gradients are zero
  const double zinv = 1.0 / z.m;
  const float tg = (float)tot_grad[(int64_t)i * tot_grad_stride];
  const int32_t zk = -z.e;
  const int32_t gb_elems = (u1 - u0) * cols;
  for (int32_t k = tid; k < gb_elems; k += nt) gb[k] = 0u;
  if (ga_in_smem)
    for (int32_t k = tid; k < A; k += nt) ga[k] = 0u;
  __syncthreads();
  const float cutoff = cutoffs[i];
  const float *fgrid = vfwd + f.grid_off, *bgrid = vbwd + f.grid_off;
  const Arc *my_arcs = arcs + f.arc_off;
  const ArcFactor *my_factors = arc_factors + f.arc_off;
  const int32_t *splits = a_row_splits2 + f.state_off;
  const int32_t lg = lanes_log2, G = 1 << lg, sub = lane & (G - 1), grp = lane >> lg,
                groups = 32 >> lg;
  NextState *nb = nb_all + warp * s_pad;
  for (int32_t u = u0 + warp; u < u1; u += kGradWarps) {
    const int64_t cur = (int64_t)u * S, nxt = (int64_t)(u + 1) * S;
    if (kStage) {
      __syncwarp();  // the previous frame's readers are done with nb
      for (int32_t q = lane; q < S; q += 32) {
        const float fn = fgrid[nxt + q], bn = bgrid[nxt + q];
        const ProbState b = be[nxt + q];
        NextState nx;
        nx.m = b.m;
        nx.e = b.e;
        nx.bo = __fadd_rn(fn, bn) > cutoff ? bn : -INFINITY;
        nb[q] = nx;
      }
      __syncwarp();
    }
    const unsigned char *rec = dense + ((int64_t)f.row0 + u) * dp.pitch;
    const float *lprow = PackLp(rec);
    const double *prow = PackP(rec, dp);
    uint32_t *gbrow = gb + (size_t)(u - u0) * cols;
    // four words of 32 states at a time, so that their loads overlap (most words
    // of a sparse lattice hold no survivor)
    for (int32_t cc = 0; cc < S; cc += 128) {
      float fu4[4], bu4[4];
#pragma unroll
      for (int w4 = 0; w4 < 4; ++w4) {
        const int32_t q = cc + 32 * w4 + lane;
        fu4[w4] = q < S ? fgrid[cur + q] : -INFINITY;
        bu4[w4] = q < S ? bgrid[cur + q] : -INFINITY;
      }
#pragma unroll
    for (int w4 = 0; w4 < 4; ++w4) {
      const int32_t c0 = cc + 32 * w4;
      if (c0 >= S) break;
      const int32_t q = c0 + lane;
      const float fu = fu4[w4], bu = bu4[w4];
      ProbState a;
      a.m = 0.0;
      a.e = kZeroExp;
      if (__fadd_rn(fu, bu) > cutoff) a = al[cur + q];
      const uint32_t m = __ballot_sync(0xffffffffu, a.m != 0.0);
      const int32_t kept = __popc(m);
      for (int32_t r0 = 0; r0 < kept; r0 += groups) {  // warp-uniform
        const int32_t nth = r0 + grp;
        const int32_t owner = nth < kept ? (int32_t)__fns(m, 0, nth + 1) : 0;
        const float fs = __shfl_sync(0xffffffffu, fu, owner);
        const double am = __shfl_sync(0xffffffffu, a.m, owner);
        const int32_t ae = __shfl_sync(0xffffffffu, a.e, owner);
        if (nth >= kept) continue;
        const int32_t sq = c0 + owner;
        const int32_t k1 = splits[sq + 1] - f.arc_off;
        for (int32_t k = splits[sq] - f.arc_off + sub; k < k1; k += G) {
          const Arc arc = my_arcs[k];
          const int32_t c = arc.label + 1;
          if (c < 0 || c >= cols) continue;
          const float sc = __fadd_rn(arc.score, lprow[c]);
          double bm;
          int32_t bexp;
          if (kStage) {
            const NextState nx = nb[arc.dest];
            if (!(__fadd_rn(__fadd_rn(fs, sc), nx.bo) > cutoff)) continue;
            bm = nx.m;
            bexp = nx.e;
          } else {
            const float fn = fgrid[nxt + arc.dest], bn = bgrid[nxt + arc.dest];
            if (!(__fadd_rn(fn, bn) > cutoff)) continue;
            if (!(__fadd_rn(__fadd_rn(fs, sc), bn) > cutoff)) continue;
            const ProbState b = be[nxt + arc.dest];
            bm = b.m;
            bexp = b.e;
          }
          const ArcFactor af = my_factors[k];
          // two steps, so that no intermediate product leaves the range of a double
          int32_t e1;
          const double m1 = SplitExp(am * af.f * prow[c], &e1);
          const double prod = m1 * bm * zinv;
          if (prod == 0.0) continue;
          const float post = (float)(prod * Pow2Clamped(e1 + ae + af.k + bexp + zk));
          atomicAdd(&gbrow[c], __float2uint_rn(post * 2147483648.0f));
          if (grad_a == nullptr) continue;
          if (ga_in_smem) atomicAdd(&ga[k], __float2uint_rn(post * 67108864.0f));
          else atomicAdd(&grad_a[f.arc_off + f.arc_out_off + k], tg * post);
        }
      }
    }
    }
  }
  __syncthreads();
  StoreDenseGrad(grad_b, f.row0, u0, cols, gb, gb_elems, tg, exclusive_rows,
                 lp_row ? lp_row[i] : -1, lp_cols, tid, nt);
  if (ga_in_smem && grad_a != nullptr)
    for (int32_t k = tid; k < A; k += nt) {
      const uint32_t fixed = ga[k];
      if (fixed != 0u)
        atomicAdd(&grad_a[f.arc_off + f.arc_out_off + k],
                  tg * ((float)fixed * (1.0f / 67108864.0f)));
    }
}

// ---------------------------------------------------------------------------
// Gradients of sparse lattices (CTC: a few tens of surviving states per frame out
// of hundreds).  grid = (frame chunks, pairs).  The CTA first compacts the surviving
// (frame, state) pairs of its frames into a list in shared memory - a coalesced scan
// of the Viterbi grids by warps, positions from ballots and one shared counter (the
// order of the list does not matter: the sums are integers) - and then spreads (survivor, arc) items over all its threads, so that the dependent
// gathers of an arc (destination scores, beta, factors) of many arcs are in flight
// at once instead of one warp walking one frame.  Same fixed-point sums as
// GridGradWarp.
// ---------------------------------------------------------------------------
constexpr int kItemThreads = 256;
constexpr int kItemCap = 1024;  // list entries; at least the states of one frame

__global__ void __launch_bounds__(kItemThreads)
GridGradItems(const FsaInfo *__restrict__ infos, const Arc *__restrict__ arcs,
              const ArcFactor *__restrict__ arc_factors,
              const int32_t *__restrict__ a_row_splits2, const unsigned char *__restrict__ dense,
              DensePack dp, const float *__restrict__ vfwd, const float *__restrict__ vbwd,
              const float *__restrict__ cutoffs, const ProbState *__restrict__ alpha,
              const ProbState *__restrict__ beta, const double *__restrict__ tot_grad,
              int32_t tot_grad_stride, float *__restrict__ grad_a, float *__restrict__ grad_b,
              int32_t frames_per_cta, int32_t lanes_log2, int32_t ga_in_smem,
              int32_t exclusive_rows, const int32_t *__restrict__ lp_row, int32_t lp_cols,
              const int32_t *__restrict__ served) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int32_t list_count;
  const int32_t i = blockIdx.y;
  if (served != nullptr && *served) return;  // GridGradStates wrote the gradients
  const FsaInfo f = infos[i];
  const int32_t S = f.num_states, A = f.num_arcs, Tk = f.tk, cols = dp.cols;
  const int32_t u0 = blockIdx.x * frames_per_cta;
  if (S == 0 || u0 >= Tk) return;
  const int32_t nf = min(u0 + frames_per_cta, Tk) - u0;
  const int tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5,
            nw = nt >> 5;
  double *it_am = reinterpret_cast<double *>(smem_raw);              // [kItemCap]
  float *it_fu = reinterpret_cast<float *>(it_am + kItemCap);        // [kItemCap]
  int32_t *it_ae = reinterpret_cast<int32_t *>(it_fu + kItemCap);    // [kItemCap]
  int32_t *it_su = it_ae + kItemCap;                                 // state | frame << 16
  uint32_t *gb = reinterpret_cast<uint32_t *>(it_su + kItemCap);     // [frames_per_cta][cols]
  uint32_t *ga = gb + (((size_t)frames_per_cta * cols + 3) & ~(size_t)3);  // [A] if ga_in_smem
  const ProbState *al = alpha + f.grid_off, *be = beta + f.grid_off;
  const ProbState z = al[(int64_t)Tk * S + (S - 1)];
  if (z.m == 0.0) return;  // no path survives: all gradients are zero
  const double zinv = 1.0 / z.m;
  const int32_t zk = -z.e;
  const float tg = (float)tot_grad[(int64_t)i * tot_grad_stride];
  for (int32_t k = tid; k < nf * cols; k += nt) gb[k] = 0u;
  if (ga_in_smem)
    for (int32_t k = tid; k < A; k += nt) ga[k] = 0u;
  const float cutoff = cutoffs[i];
  const float *fgrid = vfwd + f.grid_off, *bgrid = vbwd + f.grid_off;
  const Arc *my_arcs = arcs + f.arc_off;
  const ArcFactor *my_factors = arc_factors + f.arc_off;
  const int32_t *splits = a_row_splits2 + f.state_off;
  const int32_t lg = lanes_log2, G = 1 << lg;
  // frames per round: all of them if their survivors fit the list (the usual case),
  // else as many as fit whatever survives
  const int32_t words = (S + 31) >> 5, safe_step = max(1, kItemCap / S);
  int32_t step = nf;
  for (int32_t f0 = 0; f0 < nf;) {
    const int32_t f1 = min(nf, f0 + step);
    if (tid == 0) list_count = 0;
    __syncthreads();
    // ---- compact the survivors of frames f0 .. f1 - 1: one 32-state word per warp and
    // trip, four trips' loads issued together ---------------------------------------
    const int32_t nwords = (f1 - f0) * words;
    for (int32_t w0 = warp; w0 < nwords; w0 += 4 * nw) {
      float fu4[4], bu4[4];
      int32_t fr4[4], q4[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int32_t w = w0 + r * nw;
        const int32_t fr = f0 + w / words, q = (w % words) * 32 + lane;
        fr4[r] = fr;
        q4[r] = q;
        const bool in = w < nwords && q < S;
        const int64_t gi = (int64_t)(u0 + fr) * S + q;
        fu4[r] = in ? fgrid[gi] : -INFINITY;
        bu4[r] = in ? bgrid[gi] : -INFINITY;
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const bool keep = __fadd_rn(fu4[r], bu4[r]) > cutoff;
        const uint32_t m = __ballot_sync(0xffffffffu, keep);
        if (m == 0) continue;  // warp-uniform
        int32_t base = 0;
        if (lane == 0) base = atomicAdd(&list_count, __popc(m));
        base = __shfl_sync(0xffffffffu, base, 0);
        if (keep) {
          const int32_t p = base + __popc(m & ((1u << lane) - 1u));
          if (p < kItemCap) {
            const ProbState a = al[(int64_t)(u0 + fr4[r]) * S + q4[r]];
            it_am[p] = a.m * zinv;
            it_ae[p] = a.e + zk;
            it_fu[p] = fu4[r];
            it_su[p] = q4[r] | (fr4[r] << 16);
          }
        }
      }
    }
    __syncthreads();
    const int32_t survivors = list_count;
    if (survivors > kItemCap) {  // uniform: does not fit, take fewer frames (always fits)
      step = safe_step;
      __syncthreads();  // everyone has read list_count before it is reset
      continue;
    }
    // ---- (survivor, lane) items over all threads -------------------------------------
    const int32_t items = survivors << lg;
    for (int32_t idx = tid; idx < items; idx += nt) {
      const int32_t it = idx >> lg, sub = idx & (G - 1);
      const double am = it_am[it];
      if (am == 0.0) continue;
      const int32_t sq = it_su[it] & 0xffff, fr = it_su[it] >> 16, ae = it_ae[it];
      const float fs = it_fu[it];
      const int64_t nxt = (int64_t)(u0 + fr + 1) * S;
      const unsigned char *rec = dense + ((int64_t)f.row0 + u0 + fr) * dp.pitch;
      const float *lprow = PackLp(rec);
      const double *prow = PackP(rec, dp);
      uint32_t *gbrow = gb + (size_t)fr * cols;
      const int32_t k1 = splits[sq + 1] - f.arc_off;
      for (int32_t k = splits[sq] - f.arc_off + sub; k < k1; k += G) {
        const Arc arc = my_arcs[k];
        const int32_t c = arc.label + 1;
        if (c < 0 || c >= cols) continue;
        const float fn = fgrid[nxt + arc.dest], bn = bgrid[nxt + arc.dest];
        if (!(__fadd_rn(fn, bn) > cutoff)) continue;
        const float sc = __fadd_rn(arc.score, lprow[c]);
        if (!(__fadd_rn(__fadd_rn(fs, sc), bn) > cutoff)) continue;
        const ProbState b = be[nxt + arc.dest];
        const ArcFactor af = my_factors[k];
        int32_t e1;
        const double m1 = SplitExp(am * af.f * prow[c], &e1);
        const double prod = m1 * b.m;
        if (prod == 0.0) continue;
        const float post = (float)(prod * Pow2Clamped(e1 + ae + af.k + b.e));
        atomicAdd(&gbrow[c], __float2uint_rn(post * 2147483648.0f));
        if (grad_a == nullptr) continue;
        if (ga_in_smem) atomicAdd(&ga[k], __float2uint_rn(post * 67108864.0f));
        else atomicAdd(&grad_a[f.arc_off + f.arc_out_off + k], tg * post);
      }
    }
    __syncthreads();
    f0 = f1;
  }
  StoreDenseGrad(grad_b, f.row0, u0, cols, gb, nf * cols, tg, exclusive_rows,
                 lp_row ? lp_row[i] : -1, lp_cols, tid, nt);
  if (ga_in_smem && grad_a != nullptr)
    for (int32_t k = tid; k < A; k += nt) {
      const uint32_t fixed = ga[k];
      if (fixed != 0u)
        atomicAdd(&grad_a[f.arc_off + f.arc_out_off + k],
                  tg * ((float)fixed * (1.0f / 67108864.0f)));
    }
}

// ---------------------------------------------------------------------------
// Gradients with planned lanes, for the graphs PlanLanes placed (dense lattices:
// most states and a good part of the arcs survive on every frame).  grid = (frame
// chunks, pairs).  The CTA first copies everything its frames can touch into shared
// memory - per (level, state) the surviving alpha and beta, normalised, and the
// Viterbi scores the arc test needs; per frame the packed dense row - then every
// lane walks the chunk's frames over the arcs it holds in registers (leaving
// order, the plan of the backward recursion) with no further barrier.
// ---------------------------------------------------------------------------
template <int kDeg>
__global__ void __launch_bounds__(kLaneThreads)
GridGradLanes(const FsaInfo *__restrict__ infos, int32_t n, const Arc *__restrict__ arcs,
              const int32_t *__restrict__ a_row_splits2, const unsigned char *__restrict__ dense,
              DensePack dp, const unsigned char *__restrict__ masks, int64_t total_levels,
              const ProbState *__restrict__ alpha,
              const ProbState *__restrict__ beta, const double *__restrict__ tot_grad,
              int32_t tot_grad_stride, float *__restrict__ grad_a, float *__restrict__ grad_b,
              const int32_t *__restrict__ plan, const int32_t *__restrict__ unfit,
              int32_t frames_per_cta, int32_t sub_frames, int32_t s_pad,
              int32_t exclusive_rows, const int32_t *__restrict__ lp_row, int32_t lp_cols,
              const int32_t *__restrict__ served) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int32_t i = blockIdx.y;
  if (served != nullptr && *served) return;  // GridGradStates wrote the gradients
  if (unfit[i] & 1) return;  // no plan: the warp-per-frame kernel takes this graph
  const FsaInfo f = infos[i];
  const int32_t S = f.num_states, Tk = f.tk, cols = dp.cols;
  const int32_t cta_u0 = blockIdx.x * frames_per_cta;
  if (S == 0 || cta_u0 >= Tk) return;
  const int32_t cta_u1 = min(cta_u0 + frames_per_cta, Tk);
  const int tid = threadIdx.x, nt = blockDim.x;
  // per (level, state), as separate arrays so that gathers by state spread over the
  // banks: alpha / Z and beta mantissas (0 when pruned or unreachable), their
  // exponents, and the Viterbi scores (-inf when pruned)
  const int32_t lv_elems = (sub_frames + 1) * s_pad;
  double *st_am = reinterpret_cast<double *>(smem_raw);
  double *st_bm = st_am + lv_elems;
  int32_t *st_ae = reinterpret_cast<int32_t *>(st_bm + lv_elems);
  int32_t *st_be = st_ae + lv_elems;
  unsigned char *rows = reinterpret_cast<unsigned char *>(st_be + lv_elems);
  // posteriors per (frame, column) in fixed point, 2^-31 units: integer atomics are
  // native in shared memory (float ones are compare-and-swap loops) and make the sum
  // independent of the order of the additions
  unsigned char *mk = rows + (size_t)sub_frames * dp.pitch;  // [sub_frames][kLaneThreads]
  uint32_t *gb = reinterpret_cast<uint32_t *>(mk + (size_t)sub_frames * kLaneThreads);
  const ProbState *al = alpha + f.grid_off, *be = beta + f.grid_off;
  const ProbState z = al[(int64_t)Tk * S + (S - 1)];
  if (z.m == 0.0) return;  // no path survives: all gradients are zero
  int32_t zex;
  const double zm = SplitExp(z.m, &zex);
  const double zinv = 1.0 / zm;
  const float tg = (float)tot_grad[(int64_t)i * tot_grad_stride];
  const int32_t zk = -(z.e + zex);
  // survival bits of the lanes' arcs, one row of bytes per level (ArcMasks, direction 1)
  const unsigned char *mask0 = masks + (total_levels + f.level_off) * (int64_t)kLaneThreads;
  // ---- this lane's arcs --------------------------------------------------------
  int32_t s = -1, g = 0, G = 1;
  {
    const int32_t code = plan[((int64_t)n + i) * kLaneThreads + tid];  // direction 1
    if (code >= 0) {
      s = code & 0xffff;
      g = (code >> 16) & 0xff;
      G = code >> 24;
    }
  }
  int32_t dest_col[kDeg];
  float w[kDeg];
  double ewf[kDeg];
  int32_t ewk[kDeg];
  float ga[kDeg];
  int32_t first_arc = 0;
#pragma unroll
  for (int j = 0; j < kDeg; ++j) {
    dest_col[j] = cols << 16;
    w[j] = -INFINITY;
    ewf[j] = 0.0;
    ewk[j] = 0;
    ga[j] = 0.0f;
  }
  if (s >= 0) {
    const int32_t a0 = a_row_splits2[f.state_off + s], a1 = a_row_splits2[f.state_off + s + 1];
    first_arc = a0 + g;
#pragma unroll
    for (int j = 0; j < kDeg; ++j) {
      const int32_t k = a0 + g + j * G;
      if (k < a1) {
        const Arc arc = arcs[k];
        const int32_t c = arc.label + 1;
        if (c >= 0 && c < cols && arc.score != -INFINITY) {
          dest_col[j] = arc.dest | (c << 16);
          w[j] = arc.score;
          ExpToMantExp(arc.score, &ewf[j], &ewk[j]);
        }
      }
    }
  }
  // the CTA's frames in sub-chunks that fit in shared memory; arcs and their
  // gradients stay in registers throughout
  for (int32_t u0 = cta_u0; u0 < cta_u1; u0 += sub_frames) {
    const int32_t u1 = min(u0 + sub_frames, cta_u1), nf = u1 - u0;
    __syncthreads();  // the previous sub-chunk is flushed
    // ---- stage levels u0 .. u1 ---------------------------------------------------
    for (int32_t idx = tid; idx < (nf + 1) * S; idx += nt) {
      const int32_t l = idx / S, q = idx - l * S;
      const int64_t gi = (int64_t)(u0 + l) * S + q;
      // the recursions wrote every state (0 for pruned or unreachable ones)
      const ProbState a = al[gi], b = be[gi];
      int32_t ex;
      const double am = SplitExp(a.m, &ex) * zinv;
      const int32_t ae = a.m == 0.0 ? 0 : a.e + ex + zk;
      const double bm = SplitExp(b.m, &ex);
      const int32_t bexp = b.m == 0.0 ? 0 : b.e + ex;
      const int32_t k = l * s_pad + q;
      st_am[k] = am;
      st_bm[k] = bm;
      st_ae[k] = ae;
      st_be[k] = bexp;
    }
    {
      const int32_t chunks = dp.pitch / 16;
      const uint4 *src = reinterpret_cast<const uint4 *>(dense + ((int64_t)f.row0 + u0) * dp.pitch);
      uint4 *dst = reinterpret_cast<uint4 *>(rows);
      for (int32_t k = tid; k < nf * chunks; k += nt) dst[k] = src[k];
    }
    for (int32_t k = tid; k < nf * cols; k += nt) gb[k] = 0u;
    {
      const uint4 *src = reinterpret_cast<const uint4 *>(mask0 + (int64_t)u0 * kLaneThreads);
      uint4 *dst = reinterpret_cast<uint4 *>(mk);
      for (int32_t k = tid; k < nf * (kLaneThreads / 16); k += nt) dst[k] = src[k];
    }
    __syncthreads();
    if (s >= 0) {
      for (int32_t l = 0; l < nf; ++l) {
        const double own_am = st_am[l * s_pad + s];
        if (own_am == 0.0) continue;  // pruned or unreachable
        const uint32_t m = mk[l * kLaneThreads + tid];
        if (m == 0) continue;
        const int32_t own_ae = st_ae[l * s_pad + s];
        const int32_t nx = (l + 1) * s_pad;
        const unsigned char *rec = rows + (size_t)l * dp.pitch;
        const double *prow = PackP(rec, dp);
        uint32_t *gbrow = gb + l * cols;
        // all posteriors first, then the additions: a shared-memory atomic between
        // two arcs would order the loads of the second behind it
        float post[kDeg];
#pragma unroll
        for (int j = 0; j < kDeg; ++j) {
          const int32_t d = dest_col[j] & 0xffff, c = dest_col[j] >> 16;
          post[j] = 0.0f;
          if (m & (1u << j)) {
            const double bm = st_bm[nx + d];
            const int32_t e = own_ae + ewk[j] + st_be[nx + d];
            // alpha/Z, exp(w) and beta have mantissas in [0.5, 2); exp(lp) >= 1e-300
            const double prod = own_am * ewf[j] * prow[c] * bm;
            post[j] = (float)(prod * Pow2Clamped(e));
          }
        }
#pragma unroll
        for (int j = 0; j < kDeg; ++j) {
          if (post[j] != 0.0f) {
            ga[j] += post[j];
            atomicAdd(&gbrow[dest_col[j] >> 16], __float2uint_rn(post[j] * 2147483648.0f));
          }
        }
      }
    }
    __syncthreads();
    StoreDenseGrad(grad_b, f.row0, u0, cols, gb, nf * cols, tg, exclusive_rows,
                   lp_row ? lp_row[i] : -1, lp_cols, tid, nt);
  }
  if (s >= 0 && grad_a != nullptr) {
#pragma unroll
    for (int j = 0; j < kDeg; ++j)
      if (ga[j] != 0.0f) atomicAdd(&grad_a[first_arc + f.arc_out_off + j * G], tg * ga[j]);
  }
}

// ---------------------------------------------------------------------------
// Shared-memory variants for the graphs PlanLanes could not place (very high or
// very uneven degrees): the arcs sit in shared memory (incoming order walking
// forward, leaving order walking backward) and G = 2^lanes_log2 lanes per state
// loop over them; dense rows are staged with 16-byte cp.async.  Slower, any degree.
// With only_unfit set they skip every graph the lane kernels handled.
// ---------------------------------------------------------------------------
struct ChainPlan {
  int32_t s_pad, a_pad, stages, lanes_log2, threads;
  size_t bytes;
};

static ChainPlan PlanChain(const Layout &L, const k2b200_intersect_args *a, const DensePack &d) {
  ChainPlan p;
  p.s_pad = (L.max_states + 1 + 3) & ~3;
  p.a_pad = (L.max_arcs + 3) & ~3;
  size_t fixed = sizeof(ProbState) * 2 * p.s_pad + (size_t)24 * p.a_pad +
                 sizeof(float) * 2 * p.s_pad + sizeof(int32_t) * p.s_pad;
  p.stages = 0;
  if (fixed < kChainSmemBudget)
    p.stages = (int32_t)std::min<size_t>(8, (kChainSmemBudget - fixed) / d.pitch);
  p.bytes = fixed + (size_t)d.pitch * std::max(p.stages, 0);
  int32_t mean_deg = a->num_states > 0 ? (a->num_arcs + a->num_states - 1) / a->num_states : 1;
  int32_t lg = 0;
  while ((2 << lg) <= mean_deg / 2 && lg < 5) ++lg;
  while (lg > 0 && ((int64_t)L.max_states << lg) > 1024) --lg;
  p.lanes_log2 = lg;
  int64_t lanes = (int64_t)L.max_states << lg;
  p.threads = (int32_t)std::min<int64_t>(1024, std::max<int64_t>(128, (lanes + 31) / 32 * 32));
  return p;
}

__global__ void __launch_bounds__(1024)
GridChain(const FsaInfo *__restrict__ infos, const Arc *__restrict__ arcs,
          const int32_t *__restrict__ a_row_splits2, const int32_t *__restrict__ in_splits,
          const int32_t *__restrict__ in_arcs, const unsigned char *__restrict__ dense,
          DensePack dp, const float *__restrict__ vfwd, const float *__restrict__ vbwd,
          const float *__restrict__ cutoffs, ProbState *__restrict__ alpha,
          ProbState *__restrict__ beta, double *__restrict__ tot,
          const int32_t *__restrict__ only_unfit, ChainPlan p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int32_t i = blockIdx.y;
  if (only_unfit != nullptr && !only_unfit[i]) return;
  const FsaInfo f = infos[i];
  const int dir = blockIdx.x;  // 0 forward, 1 backward
  const int32_t S = f.num_states, A = f.num_arcs, Tk = f.tk, cols = dp.cols;
  const int tid = threadIdx.x, nt = blockDim.x;
  if (S == 0) {
    if (dir == 0 && tid == 0) tot[i] = -INFINITY;
    return;
  }
  const int32_t s_pad = p.s_pad, stages = p.stages;
  unsigned char *ring = smem_raw;                                              // [stages][pitch]
  ProbState *ps = reinterpret_cast<ProbState *>(ring + (size_t)stages * dp.pitch);  // [2][s_pad]
  int4 *meta = reinterpret_cast<int4 *>(ps + 2 * s_pad);                       // [a_pad]
  double *ewf = reinterpret_cast<double *>(meta + p.a_pad);                    // [a_pad]
  float *oth = reinterpret_cast<float *>(ewf + p.a_pad);                       // [2][s_pad]
  int32_t *splits = reinterpret_cast<int32_t *>(oth + 2 * s_pad);              // [s_pad]

  // ---- stage the graph ------------------------------------------------------
  const int32_t *gsplits = (dir == 0 ? in_splits : a_row_splits2) + f.state_off;
  for (int32_t s = tid; s <= S; s += nt) splits[s] = gsplits[s] - f.arc_off;
  for (int32_t k = tid; k < A; k += nt) {
    const Arc arc = arcs[dir == 0 ? in_arcs[f.arc_off + k] : f.arc_off + k];
    double ef;
    int32_t ek;
    ExpToMantExp(arc.score, &ef, &ek);
    const int32_t c = arc.label + 1;
    meta[k] = make_int4(dir == 0 ? arc.src : arc.dest, (c >= 0 && c < cols) ? c : cols,
                        __float_as_int(arc.score), ek);
    ewf[k] = ef;
  }
  const float cutoff = cutoffs[i];
  const float *fgrid = vfwd + f.grid_off, *bgrid = vbwd + f.grid_off;
  ProbState *out = (dir == 0 ? alpha : beta) + f.grid_off;
  {
    const int64_t lv = dir == 0 ? 0 : Tk;
    for (int32_t s = tid; s < S; s += nt) {
      const float fu = fgrid[lv * S + s], bu = bgrid[lv * S + s];
      const bool keep = __fadd_rn(fu, bu) > cutoff;
      ProbState v;
      v.pad = 0;
      if (keep && s == (dir == 0 ? 0 : S - 1)) {
        v.m = 1.0;
        v.e = 0;
      } else {
        v.m = 0.0;
        v.e = kZeroExp;
      }
      ps[s] = v;
      oth[s] = keep ? (dir == 0 ? fu : bu) : -INFINITY;
      out[lv * S + s] = v;
    }
  }
  const unsigned char *dense0 = dense + (int64_t)f.row0 * dp.pitch;
  const int32_t chunks = dp.pitch / 16;
  auto issue_row = [&](int32_t step) {
    if (step <= Tk) {
      const int64_t row = dir == 0 ? step - 1 : Tk - step;
      const unsigned char *src = dense0 + row * dp.pitch;
      unsigned char *dst = ring + (size_t)((step - 1) % stages) * dp.pitch;
      for (int32_t c = tid; c < chunks; c += nt) CpAsync16(dst + 16 * c, src + 16 * c);
    }
    CpAsyncCommit();
  };
  for (int32_t step = 1; step < stages; ++step) issue_row(step);

  const int32_t lg = p.lanes_log2, G = 1 << lg, g = tid & (G - 1);
  const int32_t per_pass = nt >> lg;
  const int32_t s_own = tid >> lg;
  ProbState last;
  last.m = 0.0;
  last.e = kZeroExp;
  for (int32_t t = 1; t <= Tk; ++t) {
    CpAsyncWaitDyn(stages - 2);
    __syncthreads();
    issue_row(t + stages - 1);
    const ProbState *prev = ps + ((t - 1) & 1) * s_pad;
    ProbState *cur = ps + (t & 1) * s_pad;
    const float *po = oth + ((t - 1) & 1) * s_pad;
    float *co = oth + (t & 1) * s_pad;
    const unsigned char *rec = ring + (size_t)((t - 1) % stages) * dp.pitch;
    const float *lprow = PackLp(rec);
    const double *prow = PackP(rec, dp);
    const int64_t lv = dir == 0 ? t : Tk - t;
    for (int32_t s0 = 0; s0 < S; s0 += per_pass) {
      const int32_t s = s0 + s_own;
      float fu = -INFINITY, bu = -INFINITY;
      if (s < S) {
        fu = fgrid[lv * S + s];
        bu = bgrid[lv * S + s];
      }
      const bool keep = s < S && __fadd_rn(fu, bu) > cutoff;
      double sum = 0.0;
      int32_t E = kZeroExp;
      if (keep) {
        const int32_t k1 = splits[s + 1];
        for (int32_t k = splits[s] + g; k < k1; k += G) {
          const int4 m = meta[k];
          const float sc = __fadd_rn(__int_as_float(m.z), lprow[m.y]);
          const float o = po[m.x];
          const float through = dir == 0 ? __fadd_rn(__fadd_rn(o, sc), bu)
                                         : __fadd_rn(__fadd_rn(fu, sc), o);
          if (through > cutoff) {
            const ProbState q = prev[m.x];
            int32_t ex;
            const double t0 = SplitExp(q.m * ewf[k] * prow[m.y], &ex);
            const int32_t e0 = t0 != 0.0 ? q.e + m.w + ex : kZeroExp;
            const int32_t En = E > e0 ? E : e0;
            sum = ScaleDown(sum, E - En) + ScaleDown(t0, e0 - En);
            E = En;
          }
        }
      }
      for (int32_t d = G >> 1; d > 0; d >>= 1) {
        const int32_t Eo = __shfl_xor_sync(0xffffffffu, E, d);
        const double so = __shfl_xor_sync(0xffffffffu, sum, d);
        const int32_t En = Eo > E ? Eo : E;
        sum = ScaleDown(sum, E - En) + ScaleDown(so, Eo - En);
        E = En;
      }
      if (s < S && g == 0) {
        ProbState r;
        r.e = E;
        r.m = Renorm(sum, &r.e);
        r.pad = 0;
        cur[s] = r;
        co[s] = keep ? (dir == 0 ? fu : bu) : -INFINITY;
        out[lv * S + s] = r;
        if (s == S - 1) last = r;
      }
    }
  }
  CpAsyncWait<0>();
  // the thread that owns the final state holds alpha[Tk][final]
  if (dir == 0 && g == 0 && ((S - 1) % per_pass) == s_own)
    tot[i] = last.m == 0.0 ? -INFINITY
                           : log(last.m) + (double)last.e * 0.69314718055994530942;
}

// ---------------------------------------------------------------------------
// Gradient of the dense scores from STATE posteriors.  When all arcs that enter a state
// carry the same label (CTC graphs, the LF-MMI denominator graph: a state "is" a symbol),
// the posteriors of the arcs entering (level l, state s) add up to alpha_l[s] * beta_l[s] / Z,
// and all of them belong to one element of the dense matrix: no arc has to be visited.
// StateInLabels finds the label of every state and whether the property holds for the
// whole batch (*one_label, initialised to 1 by the caller); GridGradStates then serves a
// backward call that does not want the gradient of the arc scores, and returns at once
// otherwise.  grid = (frame chunks, pairs); sums per (frame, column) in shared memory in
// fixed point, as in the arc-posterior kernels.
// ---------------------------------------------------------------------------
constexpr int32_t kNoInLabel = INT32_MIN;

__global__ void StateInLabels(const Arc *__restrict__ arcs, const int32_t *__restrict__ in_splits,
                              const int32_t *__restrict__ in_arcs, int32_t num_states,
                              int32_t *__restrict__ state_label, int32_t *__restrict__ one_label) {
  const int32_t s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= num_states) return;
  int32_t label = kNoInLabel;
  bool same = true;
  for (int32_t k = in_splits[s]; k < in_splits[s + 1]; ++k) {
    const int32_t lab = arcs[in_arcs[k]].label;
    if (label == kNoInLabel) label = lab;
    else if (lab != label) same = false;
  }
  state_label[s] = label;
  if (!same) atomicAnd(one_label, 0);
}

__global__ void __launch_bounds__(256)
GridGradStates(const FsaInfo *__restrict__ infos, const int32_t *__restrict__ state_label,
               const int32_t *__restrict__ one_label, int32_t cols,
               const float *__restrict__ vfwd, const float *__restrict__ vbwd,
               const float *__restrict__ cutoffs,
               const ProbState *__restrict__ alpha, const ProbState *__restrict__ beta,
               const double *__restrict__ tot_grad, int32_t tot_grad_stride,
               float *__restrict__ grad_b, int32_t frames_per_cta, int32_t exclusive_rows,
               const int32_t *__restrict__ lp_row, int32_t lp_cols) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  if (!*one_label) return;  // the arc-posterior kernels take the call
  const int32_t i = blockIdx.y;
  const FsaInfo f = infos[i];
  const int32_t S = f.num_states, Tk = f.tk;
  const int32_t u0 = blockIdx.x * frames_per_cta;  // frames u0 .. u1 - 1 = levels u0 + 1 .. u1
  if (S == 0 || u0 >= Tk) return;
  const int32_t u1 = min(u0 + frames_per_cta, Tk);
  const int tid = threadIdx.x, nt = blockDim.x;
  uint32_t *gb = reinterpret_cast<uint32_t *>(smem_raw);  // [frames_per_cta][cols], 2^-31 units
  const ProbState *al = alpha + f.grid_off, *be = beta + f.grid_off;
  const ProbState z = al[(int64_t)Tk * S + (S - 1)];
  if (z.m == 0.0) return;  // no path survives: all gradients are zero
  int32_t zex;
  const double zm = SplitExp(z.m, &zex);
  const double zinv = 1.0 / zm;
  const int32_t zk = -(z.e + zex);
  const float tg = (float)tot_grad[(int64_t)i * tot_grad_stride];
  const int32_t elems = (u1 - u0) * cols;
  for (int32_t k = tid; k < elems; k += nt) gb[k] = 0u;
  __syncthreads();
  const int32_t *labels = state_label + f.state_off;
  const float cutoff = cutoffs[i];
  const float *fgrid = vfwd + f.grid_off, *bgrid = vbwd + f.grid_off;
  for (int32_t k = tid; k < (u1 - u0) * S; k += nt) {
    const int32_t fr = k / S, s = k - fr * S;
    const int32_t c = labels[s] + 1;
    if (c < 0 || c >= cols) continue;
    const int64_t gi = (int64_t)(u0 + fr + 1) * S + s;
    // the recursions of some graphs leave the grids of pruned states unwritten
    if (!(__fadd_rn(fgrid[gi], bgrid[gi]) > cutoff)) continue;
    const ProbState a = al[gi];
    if (a.m == 0.0) continue;
    const ProbState b = be[gi];
    if (b.m == 0.0) continue;
    const float post = (float)(a.m * b.m * zinv * Pow2Clamped(a.e + b.e + zk));
    if (post != 0.0f) atomicAdd(&gb[fr * cols + c], __float2uint_rn(post * 2147483648.0f));
  }
  __syncthreads();
  StoreDenseGrad(grad_b, f.row0, u0, cols, gb, elems, tg, exclusive_rows,
                 lp_row ? lp_row[i] : -1, lp_cols, tid, nt);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
struct LossLayout {
  Layout base;
  DensePack pack;
  size_t off_dense, off_arc_factors, off_alpha, off_beta, off_masks, off_flags, off_state_label,
      off_one_label, total_bytes;
  // set by the backward entry point when the state-posterior kernel may serve the call:
  // the flag the arc-posterior kernels look at before doing anything
  const int32_t *served = nullptr;
  bool exclusive_rows;
  // set by the backward entry point: gradients go straight to the log-prob layout
  const int32_t *lp_row = nullptr;  // per pair, log-prob row of its first frame
  int32_t lp_cols = 0;
  int32_t k_deg;      // arcs per lane of the lane kernel
  bool identity;      // every degree <= k_deg: thread s owns state s, no plan
  int32_t threads;    // CTA size of the lane kernel
};

static int32_t MakeLossLayout(const k2b200_intersect_args *a, LossLayout *LL) {
  K2B_FORWARD(MakeLayout(a, &LL->base));
  LL->pack = MakeDensePack(a->cols);
  LL->identity = !LL->base.lane_plan;
  LL->k_deg = LL->identity ? (a->a_max_degree <= 3 ? 3 : 4) : kLaneDeg;
  LL->threads = LL->identity ? std::max(32, (LL->base.max_states + 31) / 32 * 32) : kLaneThreads;
  size_t off = AlignUp(LL->base.total_bytes);
  auto take = [&](size_t bytes) {
    size_t o = off;
    off += AlignUp(bytes ? bytes : 1);
    return o;
  };
  LL->off_dense = take((size_t)LL->pack.pitch * (size_t)a->rows);
  LL->off_arc_factors = take(sizeof(ArcFactor) * (size_t)std::max(a->num_arcs, 1));
  LL->off_alpha = take(sizeof(ProbState) * (size_t)LL->base.grid_elems);
  LL->off_beta = take(sizeof(ProbState) * (size_t)LL->base.grid_elems);
  // arc survival bytes, planned graphs only: [2 directions][levels][lanes]
  LL->off_masks = take(LL->identity ? 0 : (size_t)2 * LL->base.total_levels * kLaneThreads + 16);
  LL->off_flags = take(sizeof(int32_t));
  LL->off_state_label = take(sizeof(int32_t) * (size_t)std::max(a->num_states, 1));
  LL->off_one_label = take(sizeof(int32_t));
  LL->total_bytes = off;
  // two graphs on one sequence write the same rows of the dense gradient
  LL->exclusive_rows = true;
  if (a->h_a_to_b_map)
    for (int32_t i = 1; i < a->num_fsas; ++i)
      if (a->h_a_to_b_map[i] == a->h_a_to_b_map[i - 1]) LL->exclusive_rows = false;
  return kOk;
}

static bool LossFits(const LossLayout &LL, const k2b200_intersect_args *a, ChainPlan *p,
                     LaneSmem *ls) {
  *p = PlanChain(LL.base, a, LL.pack);
  // the deep ring when it fits (identity lanes only), else two slots
  *ls = PlanLaneSmem(LL.base, LL.pack, kChainGroup);
  if (!LL.identity || ls->stages == 0) *ls = PlanLaneSmem(LL.base, LL.pack, kChainGroupSmall);
  const bool lanes_ok = LL.base.lane_plan ||
                        (a->a_max_degree > 0 && a->a_max_degree <= 4 && LL.base.max_states <= 1024);
  return lanes_ok && p->stages >= 2 && ls->stages >= 2 && a->num_fsas <= 65535 &&
         a->cols < 32768 && LL.base.max_states < 65536;
}

template <int kDeg, int kMaxThreads, int kU>
static int32_t LaunchChainLanes(const LossLayout &LL, const k2b200_intersect_args *args, char *ws,
                                const LaneSmem &ls, double *tot, cudaStream_t stream) {
  const Layout &L = LL.base;
  K2B_CUDA_OK(cudaFuncSetAttribute(GridChainLanes<kDeg, kMaxThreads, kU>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ls.bytes));
  dim3 grid(2, args->num_fsas);
  { GridChainLanes<kDeg, kMaxThreads, kU><<<grid, LL.threads, ls.bytes, stream>>>(
      reinterpret_cast<const FsaInfo *>(ws + L.off_infos), args->num_fsas,
      reinterpret_cast<const Arc *>(args->a_arcs), args->a_row_splits2, args->a_in_splits,
      args->a_in_arcs, reinterpret_cast<const unsigned char *>(ws + LL.off_dense), LL.pack,
      reinterpret_cast<const float *>(ws + L.off_fwd),
      reinterpret_cast<const float *>(ws + L.off_bwd),
      reinterpret_cast<const float *>(ws + L.off_cutoffs),
      reinterpret_cast<ProbState *>(ws + LL.off_alpha),
      reinterpret_cast<ProbState *>(ws + LL.off_beta), tot,
      reinterpret_cast<int32_t *>(ws + L.off_unfit),
      reinterpret_cast<const int32_t *>(ws + LL.off_flags), ls, CopyWaitLimit()); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

// Planned graphs: survival masks for all frames, then the mask-driven recursion.
static int32_t LaunchChainMasked(const LossLayout &LL, const k2b200_intersect_args *args,
                                 char *ws, double *tot, cudaStream_t stream) {
  const Layout &L = LL.base;
  const int32_t s_pad = (L.max_states + 3) & ~3;
  const FsaInfo *d_infos = reinterpret_cast<const FsaInfo *>(ws + L.off_infos);
  const Arc *arcs = reinterpret_cast<const Arc *>(args->a_arcs);
  const unsigned char *dense = reinterpret_cast<const unsigned char *>(ws + LL.off_dense);
  const float *fwd = reinterpret_cast<const float *>(ws + L.off_fwd),
              *bwd = reinterpret_cast<const float *>(ws + L.off_bwd),
              *cutoffs = reinterpret_cast<const float *>(ws + L.off_cutoffs);
  const int32_t *plan = reinterpret_cast<const int32_t *>(ws + L.off_plan);
  int32_t *unfit = reinterpret_cast<int32_t *>(ws + L.off_unfit);
  unsigned char *masks = reinterpret_cast<unsigned char *>(ws + LL.off_masks);
  {
#define K2B_ARC_MASKS(SPAD, ROWS)                                                              \
    {                                                                                          \
      const size_t smem = sizeof(float) * ((size_t)2 * ((ROWS) + 1) * (SPAD) +                 \
                                           (size_t)(ROWS) * LL.pack.cols4);                    \
      K2B_REQUIRE(smem <= kChainSmemBudget, "too many columns for the fused loss path");       \
      K2B_CUDA_OK(cudaFuncSetAttribute(ArcMasks<kLaneDeg, SPAD, ROWS>,                         \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                                       (int)smem));                                            \
      dim3 grid(CeilDiv(L.max_tk + 1, (ROWS)), args->num_fsas, 2);                             \
      { ArcMasks<kLaneDeg, SPAD, ROWS><<<grid, kLaneThreads, smem, stream>>>(                  \
          d_infos, args->num_fsas, L.total_levels, arcs, args->a_row_splits2,                  \
          args->a_in_splits, args->a_in_arcs, dense, LL.pack, fwd, bwd, cutoffs, plan, unfit,  \
          masks); NoteLaunch(); }                                                              \
    }
    // state pitch of the staged Viterbi scores, in three sizes
    if (L.max_states <= 192) K2B_ARC_MASKS(192, 32)
    else if (L.max_states <= 384) K2B_ARC_MASKS(384, 32)
    else K2B_ARC_MASKS(768, 16)
#undef K2B_ARC_MASKS
  }
  {
    dim3 grid(2, args->num_fsas);
#define K2B_CHAIN_MASKED(KU)                                                                  \
    {                                                                                         \
      const size_t smem = (size_t)kMaskedBatches * (KU) * ((size_t)LL.pack.pitch + kLaneThreads) + \
                          sizeof(double) * 2 * kLaneThreads;                                  \
      K2B_CUDA_OK(cudaFuncSetAttribute(GridChainMasked<kLaneDeg, KU>,                         \
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                                       (int)smem));                                           \
      { GridChainMasked<kLaneDeg, KU><<<grid, kLaneThreads, smem, stream>>>(                  \
          d_infos, args->num_fsas, L.total_levels, arcs, args->a_row_splits2,                 \
          args->a_in_splits, args->a_in_arcs, dense, LL.pack, masks, fwd, bwd, cutoffs,       \
          reinterpret_cast<ProbState *>(ws + LL.off_alpha),                                   \
          reinterpret_cast<ProbState *>(ws + LL.off_beta), tot, plan, unfit, s_pad,           \
          CopyWaitLimit());                                                                   \
        NoteLaunch(); }                                                                       \
    }
    // frames per batch (one bulk copy of dense rows and one of mask rows each): as many as
    // three batches of them leave room for in shared memory
    const size_t per_frame = (size_t)kMaskedBatches * ((size_t)LL.pack.pitch + kLaneThreads);
    const size_t room = kChainSmemBudget - sizeof(double) * 2 * kLaneThreads;
    K2B_REQUIRE(per_frame <= room, "too many columns for the fused loss path");
    if (4 * per_frame <= room) K2B_CHAIN_MASKED(4)
    else if (2 * per_frame <= room) K2B_CHAIN_MASKED(2)
    else K2B_CHAIN_MASKED(1)
#undef K2B_CHAIN_MASKED
  }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

template <bool kStage>
static int32_t LaunchGrad(const LossLayout &LL, const k2b200_intersect_args *args, char *ws,
                          const double *tot_grad, int32_t stride, float *grad_a, float *grad_b,
                          const int32_t *only_noplan, cudaStream_t stream) {
  const Layout &L = LL.base;
  const int32_t s_pad = (L.max_states + 3) & ~3;
  const size_t nb_bytes = kStage ? sizeof(NextState) * kGradWarps * (size_t)s_pad : 0;
  // frames per CTA: the chunk's rows of the dense gradient live in shared memory
  int32_t frames = 32;
  while (frames > kGradWarps && sizeof(float) * (size_t)frames * args->cols > 48 * 1024)
    frames >>= 1;
  const size_t gb_bytes = sizeof(float) * (((size_t)frames * args->cols + 3) & ~(size_t)3);
  const size_t ga_bytes = sizeof(float) * (size_t)L.max_arcs;
  size_t smem = nb_bytes + gb_bytes;
  const int32_t ga_in_smem = smem + ga_bytes <= 100 * 1024;
  if (ga_in_smem) smem += ga_bytes;
  K2B_REQUIRE(smem <= kChainSmemBudget, "too many columns for the fused loss path");
  K2B_CUDA_OK(cudaFuncSetAttribute(GridGradWarp<kStage>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  // lanes per surviving state: about the mean out-degree
  int32_t mean_deg =
      args->num_states > 0 ? (args->num_arcs + args->num_states - 1) / args->num_states : 1;
  int32_t lg = 0;
  while ((1 << lg) < mean_deg && lg < 5) ++lg;
  dim3 grid(CeilDiv(L.max_tk, frames), args->num_fsas);
  { GridGradWarp<kStage><<<grid, kGradWarps * 32, smem, stream>>>(
      reinterpret_cast<const FsaInfo *>(ws + L.off_infos),
      reinterpret_cast<const Arc *>(args->a_arcs),
      reinterpret_cast<const ArcFactor *>(ws + LL.off_arc_factors), args->a_row_splits2,
      reinterpret_cast<const unsigned char *>(ws + LL.off_dense), LL.pack,
      reinterpret_cast<const float *>(ws + L.off_fwd),
      reinterpret_cast<const float *>(ws + L.off_bwd),
      reinterpret_cast<const float *>(ws + L.off_cutoffs),
      reinterpret_cast<const ProbState *>(ws + LL.off_alpha),
      reinterpret_cast<const ProbState *>(ws + LL.off_beta), tot_grad, stride, grad_a, grad_b,
      frames, lg, s_pad, ga_in_smem, LL.exclusive_rows ? 1 : 0, only_noplan, LL.lp_row,
      LL.lp_cols, LL.served); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

static int32_t LaunchGradItems(const LossLayout &LL, const k2b200_intersect_args *args, char *ws,
                               const double *tot_grad, int32_t stride, float *grad_a,
                               float *grad_b, cudaStream_t stream) {
  const Layout &L = LL.base;
  // few frames per CTA: the shared memory of a CTA decides how many CTAs an SM holds,
  // and the gathers want many warps in flight
  int32_t frames = 16;
  while (frames > 4 && sizeof(float) * (size_t)frames * args->cols > 16 * 1024) frames >>= 1;
  const size_t list_bytes = (size_t)kItemCap * (8 + 4 + 4 + 4);
  const size_t gb_bytes = sizeof(float) * (((size_t)frames * args->cols + 3) & ~(size_t)3);
  const size_t ga_bytes = sizeof(float) * (size_t)L.max_arcs;
  size_t smem = list_bytes + gb_bytes;
  const int32_t ga_in_smem = smem + ga_bytes <= 100 * 1024;
  if (ga_in_smem) smem += ga_bytes;
  K2B_REQUIRE(smem <= kChainSmemBudget, "too many columns for the fused loss path");
  K2B_CUDA_OK(cudaFuncSetAttribute(GridGradItems, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)smem));
  int32_t mean_deg =
      args->num_states > 0 ? (args->num_arcs + args->num_states - 1) / args->num_states : 1;
  int32_t lg = 0;
  while ((1 << lg) < mean_deg && lg < 5) ++lg;
  dim3 grid(CeilDiv(L.max_tk, frames), args->num_fsas);
  { GridGradItems<<<grid, kItemThreads, smem, stream>>>(
      reinterpret_cast<const FsaInfo *>(ws + L.off_infos),
      reinterpret_cast<const Arc *>(args->a_arcs),
      reinterpret_cast<const ArcFactor *>(ws + LL.off_arc_factors), args->a_row_splits2,
      reinterpret_cast<const unsigned char *>(ws + LL.off_dense), LL.pack,
      reinterpret_cast<const float *>(ws + L.off_fwd),
      reinterpret_cast<const float *>(ws + L.off_bwd),
      reinterpret_cast<const float *>(ws + L.off_cutoffs),
      reinterpret_cast<const ProbState *>(ws + LL.off_alpha),
      reinterpret_cast<const ProbState *>(ws + LL.off_beta), tot_grad, stride, grad_a, grad_b,
      frames, lg, ga_in_smem, LL.exclusive_rows ? 1 : 0, LL.lp_row, LL.lp_cols, LL.served);
    NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

static int32_t LaunchGradLanes(const LossLayout &LL, const k2b200_intersect_args *args, char *ws,
                               const double *tot_grad, int32_t stride, float *grad_a,
                               float *grad_b, cudaStream_t stream) {
  const Layout &L = LL.base;
  const int32_t s_pad = (L.max_states + 3) & ~3;
  auto bytes_for = [&](int32_t frames) {
    return (size_t)24 * (frames + 1) * s_pad + (size_t)frames * LL.pack.pitch +
           (size_t)frames * kLaneThreads + sizeof(float) * (size_t)frames * args->cols;
  };
  int32_t sub = 16;
  while (sub > 1 && bytes_for(sub) > 100 * 1024) sub >>= 1;
  const size_t smem = bytes_for(sub);
  const int32_t frames = 4 * sub;  // per CTA: amortises loading the arcs and adding grad_a
  K2B_REQUIRE(smem <= kChainSmemBudget, "graphs too large for the fused loss path");
  K2B_CUDA_OK(cudaFuncSetAttribute(GridGradLanes<kLaneDeg>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(CeilDiv(L.max_tk, frames), args->num_fsas);
  { GridGradLanes<kLaneDeg><<<grid, kLaneThreads, smem, stream>>>(
      reinterpret_cast<const FsaInfo *>(ws + L.off_infos), args->num_fsas,
      reinterpret_cast<const Arc *>(args->a_arcs), args->a_row_splits2,
      reinterpret_cast<const unsigned char *>(ws + LL.off_dense), LL.pack,
      reinterpret_cast<const unsigned char *>(ws + LL.off_masks), L.total_levels,
      reinterpret_cast<const ProbState *>(ws + LL.off_alpha),
      reinterpret_cast<const ProbState *>(ws + LL.off_beta), tot_grad, stride, grad_a, grad_b,
      reinterpret_cast<const int32_t *>(ws + L.off_plan),
      reinterpret_cast<const int32_t *>(ws + L.off_unfit), frames, sub, s_pad,
      LL.exclusive_rows ? 1 : 0, LL.lp_row, LL.lp_cols, LL.served); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

}  // namespace k2b

using namespace k2b;

extern "C" {

int32_t k2b200_dense_loss_supported(const k2b200_intersect_args *args, int32_t *supported) {
  K2B_REQUIRE(supported != nullptr, "NULL output pointer");
  LossLayout LL;
  K2B_FORWARD(MakeLossLayout(args, &LL));
  ChainPlan p;
  LaneSmem ls;
  *supported = LossFits(LL, args, &p, &ls) ? 1 : 0;
  return kOk;
}

int32_t k2b200_dense_loss_workspace_bytes(const k2b200_intersect_args *args, size_t *bytes) {
  K2B_REQUIRE(bytes != nullptr, "NULL output pointer");
  LossLayout LL;
  K2B_FORWARD(MakeLossLayout(args, &LL));
  *bytes = LL.total_bytes;
  return kOk;
}

int32_t k2b200_dense_loss_forward(const k2b200_intersect_args *args, void *workspace,
                                  size_t workspace_bytes, void *stream_v, double *tot_scores,
                                  float *beam_used) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  LossLayout LL;
  K2B_FORWARD(MakeLossLayout(args, &LL));
  const Layout &L = LL.base;
  if (workspace == nullptr || workspace_bytes < LL.total_bytes) {
    SetError("workspace of %zu bytes is smaller than the %zu required", workspace_bytes,
             LL.total_bytes);
    return kWorkspaceTooSmall;
  }
  K2B_REQUIRE(args->a_row_splits1 && args->a_row_splits2 && args->a_arcs && args->a_in_splits &&
                  args->a_in_arcs && args->scores && tot_scores,
              "NULL device pointer");
  ChainPlan p;
  LaneSmem ls;
  K2B_REQUIRE(LossFits(LL, args, &p, &ls),
              "graphs too large for the fused loss path (%d states, %d arcs, %d columns): "
              "use intersect_dense + get_tot_scores",
              L.max_states, L.max_arcs, args->cols);
  char *ws = reinterpret_cast<char *>(workspace);
  K2B_CUDA_OK(cudaMemcpyAsync(ws + L.off_infos, L.infos.data(), sizeof(FsaInfo) * args->num_fsas,
                              cudaMemcpyHostToDevice, stream));
  const FsaInfo *d_infos = reinterpret_cast<const FsaInfo *>(ws + L.off_infos);
  unsigned char *dense = reinterpret_cast<unsigned char *>(ws + LL.off_dense);
  int32_t *unfit = reinterpret_cast<int32_t *>(ws + L.off_unfit);
  // The repacking does not depend on the Viterbi pass.  It is enqueued on the side
  // stream AFTER the Viterbi kernels have been launched, so that their CTAs own the
  // SMs first and the repacking fills in beside them; joined before the recursions
  // read the packed rows.
  struct JoinOnExit {  // also on error returns: the caller may free the workspace
    cudaStream_t main;
    bool armed;
    ~JoinOnExit() { if (armed) SideJoin(main); }
  } join_guard{stream, false};
  K2B_CUDA_OK(cudaMemsetAsync(ws + LL.off_flags, 0, sizeof(int32_t), stream));
  cudaStream_t side;
  K2B_FORWARD(SideFork(stream, &side));
  join_guard.armed = true;
  K2B_FORWARD(LaunchPlanLanes(L, args, ws, stream));
  {
    PhaseTimer timer(kPhaseViterbi, stream);
    K2B_FORWARD(RunViterbi(L, args, ws, stream, /*plan_ready=*/true));
  }
  // the label of every state and whether a state has one (for the backward pass): beside
  // the Viterbi kernels, like the repacking
  K2B_CUDA_OK(cudaMemsetAsync(ws + LL.off_one_label, 0xff, sizeof(int32_t), side));
  if (args->num_states > 0)
    { StateInLabels<<<CeilDiv(args->num_states, 256), 256, 0, side>>>(
        reinterpret_cast<const Arc *>(args->a_arcs), args->a_in_splits, args->a_in_arcs,
        args->num_states, reinterpret_cast<int32_t *>(ws + LL.off_state_label),
        reinterpret_cast<int32_t *>(ws + LL.off_one_label)); NoteLaunch(); }
  {
    PhaseTimer timer(kPhaseDense, side);  // repacking belongs with the dense matrix
    const int64_t n_dense = (int64_t)args->rows * LL.pack.cols4;
    { ExpDense<<<(int)std::min<int64_t>(CeilDiv(n_dense, 256), 148 * 8), 256, 0, side>>>(
        args->scores, args->rows, LL.pack, dense, kMinDenseScore,
        reinterpret_cast<int32_t *>(ws + LL.off_flags)); NoteLaunch(); }
  }
  // The lattice is never built, but its size still decides the beam
  // (intersect_dense.cu:300-320).  The grid itself bounds it: count only when the
  // bound does not already satisfy the limits.  The count runs on the side stream
  // beside the recursions, which start from the current beam at once; in the rare
  // case that the sizes exceed the limits the beam shrinks and they run again.
  float beam = args->output_beam;
  long long arc_frames = 0;
  for (const FsaInfo &f : L.infos) arc_frames += (long long)f.tk * f.num_arcs;
  const bool need_count = L.grid_elems > args->max_states || arc_frames > args->max_arcs;
  K2B_FORWARD(SideJoin(stream));  // the packed rows are ready before the recursions
  for (int iter = 0;; ++iter) {
    K2B_FORWARD(LaunchCutoffs(L, args, ws, beam, stream));
    if (need_count) {
      K2B_FORWARD(SideFork(stream, &side));  // behind the cutoffs
      PhaseTimer timer(kPhasePrune, side);
      NotePhaseKernel(kPhasePrune, "CountStates");
      K2B_FORWARD(LaunchSizeCount(L, args, ws, side));
    }
    {
      PhaseTimer timer(kPhaseChain, stream);
#define K2B_CHAIN(DEG, MAXT)                                                              \
  (ls.stages == kChainGroup                                                               \
       ? LaunchChainLanes<DEG, MAXT, kChainGroup>(LL, args, ws, ls, tot_scores, stream)   \
       : LaunchChainLanes<DEG, MAXT, kChainGroupSmall>(LL, args, ws, ls, tot_scores, stream))
      NotePhaseKernel(kPhaseChain, LL.identity ? "GridChainLanes" : "ArcMasks+GridChainMasked");
      if (LL.k_deg == 3 && LL.threads <= 512) K2B_FORWARD(K2B_CHAIN(3, 512));
      else if (LL.k_deg == 3) K2B_FORWARD(K2B_CHAIN(3, 1024));
      else if (LL.k_deg == 4 && LL.threads <= 512) K2B_FORWARD(K2B_CHAIN(4, 512));
      else if (LL.k_deg == 4) K2B_FORWARD(K2B_CHAIN(4, 1024));
      else
        K2B_FORWARD(LaunchChainMasked(LL, args, ws, tot_scores, stream));
#undef K2B_CHAIN
    // graphs the lane kernel skipped or gave up on
    K2B_CUDA_OK(cudaFuncSetAttribute(GridChain, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)p.bytes));
    dim3 grid(2, args->num_fsas);
    { GridChain<<<grid, p.threads, p.bytes, stream>>>(
        d_infos, reinterpret_cast<const Arc *>(args->a_arcs), args->a_row_splits2,
        args->a_in_splits, args->a_in_arcs, dense, LL.pack,
        reinterpret_cast<const float *>(ws + L.off_fwd),
        reinterpret_cast<const float *>(ws + L.off_bwd),
        reinterpret_cast<const float *>(ws + L.off_cutoffs),
        reinterpret_cast<ProbState *>(ws + LL.off_alpha),
        reinterpret_cast<ProbState *>(ws + LL.off_beta), tot_scores, unfit, p); NoteLaunch(); }
    }
    K2B_CUDA_OK(cudaGetLastError());
    if (!need_count) break;
    long long h_totals[5];
    K2B_FORWARD(SideReadBack(ws + L.off_totals, sizeof(h_totals), h_totals));
    const float beam_before = beam;
    if (!ReduceBeam(args, h_totals, &beam)) break;
    K2B_LOG(kLogInfo, "dense loss: %lld states / %lld arcs exceed max_states %d / max_arcs %d, "
            "output beam %g -> %g", h_totals[0], h_totals[2], args->max_states, args->max_arcs,
            (double)beam_before, (double)beam);
    K2B_REQUIRE(iter < 200, "output beam reduction did not converge");
  }
  if (beam_used) *beam_used = beam;
  join_guard.armed = false;
  K2B_FORWARD(SideJoin(stream));
  return kOk;
}

static int32_t DenseLossBackward(const k2b200_intersect_args *args, void *workspace,
                                 size_t workspace_bytes, const double *tot_grad,
                                 int32_t tot_grad_stride, float *grad_a, float *grad_b,
                                 const int32_t *lp_row, int32_t lp_cols, cudaStream_t stream) {
  LossLayout LL;
  K2B_FORWARD(MakeLossLayout(args, &LL));
  LL.lp_row = lp_row;
  LL.lp_cols = lp_cols;
  const Layout &L = LL.base;
  if (workspace == nullptr || workspace_bytes < LL.total_bytes) {
    SetError("workspace of %zu bytes is smaller than the %zu required", workspace_bytes,
             LL.total_bytes);
    return kWorkspaceTooSmall;
  }
  K2B_REQUIRE(tot_grad && grad_b, "NULL device pointer");
  if (L.max_states == 0 || L.max_tk == 0) return kOk;
  char *ws = reinterpret_cast<char *>(workspace);
  PhaseTimer timer(kPhaseGrad, stream);
  if (grad_a == nullptr) {
    // only the dense gradient is wanted: state posteriors give it when every state has
    // one label; the kernels below look at the same flag and return if it did
    LL.served = reinterpret_cast<const int32_t *>(ws + LL.off_one_label);
    int32_t frames = 32;
    while (frames > 1 && sizeof(uint32_t) * (size_t)frames * args->cols > 64 * 1024) frames >>= 1;
    const size_t smem = sizeof(uint32_t) * (size_t)frames * args->cols;
    K2B_REQUIRE(smem <= kChainSmemBudget, "too many columns for the fused loss path");
    K2B_CUDA_OK(cudaFuncSetAttribute(GridGradStates, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)smem));
    dim3 grid(CeilDiv(L.max_tk, frames), args->num_fsas);
    { GridGradStates<<<grid, 256, smem, stream>>>(
        reinterpret_cast<const FsaInfo *>(ws + L.off_infos),
        reinterpret_cast<const int32_t *>(ws + LL.off_state_label), LL.served, args->cols,
        reinterpret_cast<const float *>(ws + L.off_fwd),
        reinterpret_cast<const float *>(ws + L.off_bwd),
        reinterpret_cast<const float *>(ws + L.off_cutoffs),
        reinterpret_cast<const ProbState *>(ws + LL.off_alpha),
        reinterpret_cast<const ProbState *>(ws + LL.off_beta), tot_grad, tot_grad_stride, grad_b,
        frames, LL.exclusive_rows ? 1 : 0, LL.lp_row, LL.lp_cols); NoteLaunch(); }
    K2B_CUDA_OK(cudaGetLastError());
  }
  if (args->num_arcs > 0)
    { ExpArcs<<<CeilDiv(args->num_arcs, 256), 256, 0, stream>>>(
        reinterpret_cast<const Arc *>(args->a_arcs), args->num_arcs,
        reinterpret_cast<ArcFactor *>(ws + LL.off_arc_factors)); NoteLaunch(); }
  const int32_t *only_noplan = nullptr;
  NotePhaseKernel(kPhaseGrad, grad_a == nullptr ? "GridGradStates (arc posteriors when a state has several labels)"
                              : !LL.identity ? "GridGradLanes"
                              : (L.max_states > 256 && L.max_states <= 1024) ? "GridGradItems"
                                                                             : "GridGradWarp");
  if (!LL.identity) {
    K2B_FORWARD(LaunchGradLanes(LL, args, ws, tot_grad, tot_grad_stride, grad_a, grad_b, stream));
    only_noplan = reinterpret_cast<const int32_t *>(ws + L.off_unfit);
  }
  // register-lane graphs of some size (CTC): compacted survivor list
  if (LL.identity && L.max_states > 256 && L.max_states <= 1024)
    return LaunchGradItems(LL, args, ws, tot_grad, tot_grad_stride, grad_a, grad_b, stream);
  // small graphs: stage level u + 1 per warp; large ones: gather
  if (L.max_states <= 256)
    return LaunchGrad<true>(LL, args, ws, tot_grad, tot_grad_stride, grad_a, grad_b, only_noplan,
                            stream);
  return LaunchGrad<false>(LL, args, ws, tot_grad, tot_grad_stride, grad_a, grad_b, only_noplan,
                           stream);
}

int32_t k2b200_dense_loss_backward(const k2b200_intersect_args *args, void *workspace,
                                   size_t workspace_bytes, const double *tot_grad,
                                   int32_t tot_grad_stride, float *grad_a, float *grad_b,
                                   void *stream_v) {
  return DenseLossBackward(args, workspace, workspace_bytes, tot_grad, tot_grad_stride, grad_a,
                           grad_b, nullptr, 0, reinterpret_cast<cudaStream_t>(stream_v));
}

int32_t k2b200_dense_loss_backward_log_probs(const k2b200_intersect_args *args, void *workspace,
                                             size_t workspace_bytes, const double *tot_grad,
                                             int32_t tot_grad_stride, float *grad_a,
                                             float *grad_log_probs, const int32_t *log_prob_row,
                                             int32_t num_classes, void *stream_v) {
  K2B_REQUIRE(log_prob_row != nullptr, "NULL log_prob_row");
  K2B_REQUIRE(args != nullptr && num_classes == args->cols - 1,
              "num_classes must be the score matrix's columns minus one");
  return DenseLossBackward(args, workspace, workspace_bytes, tot_grad, tot_grad_stride, grad_a,
                           grad_log_probs, log_prob_row, num_classes,
                           reinterpret_cast<cudaStream_t>(stream_v));
}

}  // extern "C"

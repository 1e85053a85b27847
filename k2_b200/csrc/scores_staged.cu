// Forward/backward scores of a strictly layered FsaVec (every arc goes from one
// layer to the next, as in the lattices intersect_dense emits), one persistent CTA
// per (FSA, direction).
//
// The recursion is a chain of T dependent layers, so what matters is the latency
// of one layer.  Nothing on that chain touches global memory:
//   * the layer boundaries of the FSA and the arc offsets at those boundaries sit
//     in shared memory from the start;
//   * per layer, the per-state splits and the arcs' (other-end state, score) are
//     contiguous in global memory (incoming order for forward - in_src/in_score -
//     and leaving order for backward) and are copied into a shared-memory ring by
//     cp.async several layers ahead;
//   * the scores of the previous layer are kept in a shared ping-pong buffer.
// Each layer costs one __syncthreads.  Same arithmetic as LayeredScores in
// scores.cu (reference: k2/csrc/fsa_utils.cu:1124-1278, :1345-1454).
#include <algorithm>

#include "../../include/k2b200.h"
#include "common.cuh"
#include "cp_async.cuh"
#include "prob_math.cuh"
#include "scores_internal.cuh"

namespace k2b {

constexpr size_t kStagedSmemBudget = 200 * 1024;

struct StagedPlan {
  int32_t maxw, maxa, nl_cap, stages, stage_ints, lanes_log2, threads;
  size_t bytes;
  bool ok;
};

static StagedPlan PlanStaged(const k2b200_fsa_view *v, size_t real_bytes, bool tropical) {
  StagedPlan p = {};
  p.ok = false;
  if (!v->strict_layers || v->max_layer_states <= 0 || v->max_layer_arcs < 0 ||
      v->max_layers <= 0)
    return p;
  p.maxw = (v->max_layer_states + 3) & ~3;
  p.maxa = (std::max(v->max_layer_arcs, 1) + 3) & ~3;
  p.nl_cap = v->max_layers;
  // one ring stage, in 4-byte units: splits, then either (src, score[, arc id]) or
  // 16-byte arcs; both directions share the stride
  int32_t splits_ints = (p.maxw + 1 + 3) & ~3;
  int32_t fwd_ints = p.maxa * (tropical ? 3 : 2);
  int32_t bwd_ints = p.maxa * 4;
  p.stage_ints = splits_ints + std::max(fwd_ints, bwd_ints);
  size_t fixed = sizeof(int32_t) * 2 * (size_t)((p.nl_cap + 1 + 3) & ~3) +
                 real_bytes * 2 * (size_t)p.maxw;
  size_t stage_bytes = sizeof(int32_t) * (size_t)p.stage_ints;
  if (fixed + 2 * stage_bytes > kStagedSmemBudget) return p;
  p.stages = (int32_t)std::min<size_t>(8, (kStagedSmemBudget - fixed) / stage_bytes);
  p.bytes = fixed + stage_bytes * p.stages;
  int32_t mean_deg = v->num_states > 0 ? (v->num_arcs + v->num_states - 1) / v->num_states : 1;
  p.lanes_log2 = 0;
  while ((2 << p.lanes_log2) <= mean_deg / 2 && p.lanes_log2 < 5) ++p.lanes_log2;
  p.threads = ((int64_t)p.maxw << p.lanes_log2) > 64 ? 128 : 64;
  if (p.lanes_log2 >= 3) p.threads = 256;
  p.ok = true;
  return p;
}

template <typename Real, bool kLog>
__global__ void __launch_bounds__(256)
LayeredScoresStaged(k2b200_fsa_view v, Real *forward, Real *backward,
                    int32_t *__restrict__ entering_arcs, int32_t dir_base, int32_t fsa_base,
                    StagedPlan p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int32_t i = fsa_base + blockIdx.y, dir = blockIdx.x + dir_base;
  const int32_t s_begin = v.row_splits1[i], s_end = v.row_splits1[i + 1];
  if (s_end == s_begin) return;
  const int32_t lv0 = v.level_offsets[i], nl = v.level_offsets[i + 1] - lv0;
  const int tid = threadIdx.x, nt = blockDim.x;
  const Arc *arcs = reinterpret_cast<const Arc *>(v.arcs);
  Real *out = dir == 0 ? forward : backward;
  const Real kNegInf = -INFINITY;

  const int32_t lvl_ints = (p.nl_cap + 1 + 3) & ~3;
  int32_t *lvl = reinterpret_cast<int32_t *>(smem_raw);  // first state of each layer
  int32_t *alvl = lvl + lvl_ints;                        // first arc of each layer
  Real *score_buf = reinterpret_cast<Real *>(alvl + lvl_ints);  // [2][maxw]
  int32_t *ring = reinterpret_cast<int32_t *>(score_buf + 2 * p.maxw);
  const int32_t splits_ints = (p.maxw + 1 + 3) & ~3;
  const int32_t *gsplits = dir == 0 ? v.in_splits : v.row_splits2;

  // Layer boundaries; a layer wider than the plan allows (the caller's bounds were
  // wrong) makes this CTA take the plain global-memory route below.
  __shared__ int32_t too_wide;
  if (tid == 0) too_wide = (nl > p.nl_cap);
  __syncthreads();
  if (!too_wide) {
    for (int32_t k = tid; k <= nl; k += nt) {
      int32_t s = v.level_splits[lv0 + k];
      lvl[k] = s;
      alvl[k] = gsplits[s];
    }
  }
  __syncthreads();
  if (!too_wide) {
    int32_t bad = 0;
    for (int32_t k = tid; k < nl; k += nt)
      bad |= (lvl[k + 1] - lvl[k] > p.maxw) | (alvl[k + 1] - alvl[k] > p.maxa);
    if (bad) too_wide = 1;
  }
  __syncthreads();
  if (too_wide) {
    LayeredScoresDevice<Real, kLog>(v, i, dir, forward, backward, entering_arcs);
    return;
  }

  const int32_t stages = p.stages;
  auto layer_of = [&](int32_t step) { return dir == 0 ? step : nl - 1 - step; };
  auto issue = [&](int32_t step) {
    if (step < nl) {
      const int32_t li = layer_of(step);
      const int32_t b = lvl[li], w = lvl[li + 1] - b, ab = alvl[li], na = alvl[li + 1] - ab;
      int32_t *st = ring + (size_t)(step % stages) * p.stage_ints;
      for (int32_t k = tid; k <= w; k += nt) CpAsync4(st + k, gsplits + b + k);
      int32_t *body = st + splits_ints;
      if (dir == 0) {
        for (int32_t k = tid; k < na; k += nt) {
          CpAsync4(body + k, v.in_src + ab + k);
          CpAsync4(body + p.maxa + k, v.in_score + ab + k);
          if (!kLog) CpAsync4(body + 2 * p.maxa + k, v.in_arcs + ab + k);
        }
      } else {
        for (int32_t k = tid; k < na; k += nt) CpAsync16(body + 4 * k, arcs + ab + k);
      }
    }
    CpAsyncCommit();
  };
  for (int32_t step = 0; step < stages - 1; ++step) issue(step);

  const int32_t lg = p.lanes_log2, G = 1 << lg, g = tid & (G - 1), per_pass = nt >> lg;
  for (int32_t step = 0; step < nl; ++step) {
    CpAsyncWaitDyn(stages - 2);
    __syncthreads();
    issue(step + stages - 1);
    const int32_t li = layer_of(step);
    const int32_t b = lvl[li], w = lvl[li + 1] - b, ab = alvl[li];
    // first state of the layer the arcs come from (forward) or lead to (backward)
    const int32_t other_base = step == 0 ? 0 : lvl[dir == 0 ? li - 1 : li + 1];
    const int32_t *st = ring + (size_t)(step % stages) * p.stage_ints;
    const int32_t *body = st + splits_ints;
    const Real *prev = score_buf + ((step + 1) & 1) * p.maxw;
    Real *cur = score_buf + (step & 1) * p.maxw;
    for (int32_t j0 = 0; j0 < w; j0 += per_pass) {
      const int32_t j = j0 + (tid >> lg);
      Real val = kNegInf;
      int32_t best = -1;
      int32_t k0 = 0, k1 = 0;
      if (j < w) {
        k0 = st[j] - ab;
        k1 = st[j + 1] - ab;
      }
      auto term = [&](int32_t k) -> Real {
        if (dir == 0) {
          return prev[body[k] - other_base] + (Real)__int_as_float(body[p.maxa + k]);
        } else {
          return prev[s_begin + body[4 * k + 1] - other_base] +
                 (Real)__int_as_float(body[4 * k + 3]);
        }
      };
      if (kLog) {
        Real m = kNegInf;
        for (int32_t k = k0 + g; k < k1; k += G) {
          Real x = term(k);
          m = x > m ? x : m;
        }
        for (int32_t d = G >> 1; d > 0; d >>= 1) {
          Real o = __shfl_xor_sync(0xffffffffu, m, d);
          m = o > m ? o : m;
        }
        Real sum = 0;
        if (m != kNegInf)
          for (int32_t k = k0 + g; k < k1; k += G) sum += ExpReal<Real>(term(k) - m);
        for (int32_t d = G >> 1; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
        if (m != kNegInf) val = m + LogReal<Real>(sum);
      } else {
        for (int32_t k = k0 + g; k < k1; k += G) {
          Real x = term(k);
          if (dir == 0) {
            int32_t a = body[2 * p.maxa + k];
            if (x > val || (x == val && a > best)) {
              val = x;
              best = a;
            }
          } else {
            val = x > val ? x : val;
          }
        }
        for (int32_t d = G >> 1; d > 0; d >>= 1) {
          Real o = __shfl_xor_sync(0xffffffffu, val, d);
          int32_t ob = __shfl_xor_sync(0xffffffffu, best, d);
          if (o > val || (o == val && ob > best)) {
            val = o;
            best = ob;
          }
        }
      }
      if (j < w && g == 0) {
        const int32_t s = b + j;
        if (val == kNegInf && s == (dir == 0 ? s_begin : s_end - 1)) val = 0;
        cur[j] = val;
        out[s] = val;
        if (!kLog && dir == 0 && entering_arcs) entering_arcs[s] = best;
      }
    }
  }
  CpAsyncWait<0>();
}

template <typename Real>
int32_t LaunchStagedScores(const k2b200_fsa_view *v, int32_t log_semiring, Real *fwd, Real *bwd,
                           int32_t *entering, cudaStream_t stream, bool *launched) {
  *launched = false;
  if (fwd != nullptr && (v->in_src == nullptr || v->in_score == nullptr)) return kOk;
  StagedPlan p = PlanStaged(v, sizeof(Real), !log_semiring);
  if (!p.ok) return kOk;
  int32_t ndir = (fwd != nullptr) + (bwd != nullptr);
  int32_t dir_base = fwd ? 0 : 1;
  auto kernel = log_semiring ? LayeredScoresStaged<Real, true> : LayeredScoresStaged<Real, false>;
  K2B_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)p.bytes));
  for (int32_t first = 0; first < v->num_fsas; first += 65535) {
    int32_t n = std::min(v->num_fsas - first, 65535);
    dim3 grid(ndir, n);
    { kernel<<<grid, p.threads, p.bytes, stream>>>(*v, fwd, bwd, entering, dir_base, first, p);
      NoteLaunch(); }
  }
  K2B_CUDA_OK(cudaGetLastError());
  *launched = true;
  return kOk;
}

// ---------------------------------------------------------------------------
// Log-semiring scores without transcendental functions on the dependency chain.
//
// A log-sum-exp recursion spends most of a layer's latency in one exp per arc and
// one log per state (hundreds of cycles each in double precision).  Here every
// score is carried as a number with a separate integer exponent,
//     value = m * 2^e   (m a double in [1,2), or m == 0),
// so a layer is: multiply by the arc weight (also stored as f * 2^k with f in
// [1,2)), bring the terms of a state to their largest exponent with exact powers
// of two, add, renormalise.  All of that is a handful of multiply/add and integer
// instructions; the exponent is a 32-bit integer, so nothing under- or overflows
// however far apart the scores of a layer are.  exp() of the arc scores and log()
// of the state values are taken off the chain, in fully parallel kernels before
// and after.  Rounding differs from the reference's sequential LogAdd by ~1e-15
// relative per operation.
// ---------------------------------------------------------------------------
struct __align__(16) ProbArc {
  double f;       // mantissa of exp(score) in [1,2), 0 when score == -inf
  int32_t other;  // source (forward) / destination (backward) state, relative to the first
                  // state of its layer
  int32_t k;      // binary exponent of exp(score)
};
static_assert(sizeof(ProbArc) == 16, "ProbArc must be 16 bytes");

// fwd_arcs[k] (incoming order) and bwd_arcs[a] (leaving order) from the arc scores.
__global__ void PrepareProbArcs(k2b200_fsa_view v, ProbArc *__restrict__ fwd_arcs,
                                ProbArc *__restrict__ bwd_arcs) {
  int32_t k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= v.num_arcs) return;
  const Arc *arcs = reinterpret_cast<const Arc *>(v.arcs);
  // index of state s (idx01, in FSA i) within its layer
  auto local_index = [&](int32_t i, int32_t s) {
    int32_t lo = v.level_offsets[i], hi = v.level_offsets[i + 1];
    while (hi - lo > 1) {
      const int32_t mid = (lo + hi) >> 1;
      if (v.level_splits[mid] <= s) lo = mid; else hi = mid;
    }
    return s - v.level_splits[lo];
  };
  if (bwd_arcs) {
    Arc arc = arcs[k];
    ProbArc p;
    ExpToMantExp(arc.score, &p.f, &p.k);
    const int32_t i = v.row_ids1[v.row_ids2[k]];
    p.other = local_index(i, v.row_splits1[i] + arc.dest);
    bwd_arcs[k] = p;
  }
  if (fwd_arcs) {
    ProbArc p;
    ExpToMantExp(v.in_score[k], &p.f, &p.k);
    const int32_t src = v.in_src[k];
    p.other = local_index(v.row_ids1[src], src);
    fwd_arcs[k] = p;
  }
}

// out[s] = log(m[s]) + e[s] * ln 2
template <typename Real>
__global__ void FinishLogScores(const double *__restrict__ m, const int32_t *__restrict__ e,
                                int32_t n, Real *__restrict__ out) {
  int32_t s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= n) return;
  double mm = m[s];
  out[s] = mm == 0.0 ? (Real)-INFINITY
                     : (Real)(log(mm) + (double)e[s] * 0.69314718055994530942);
}

constexpr int kMaxSlots = 64;

struct ProbPlan {
  int32_t maxw, maxa, nl_cap, stages, stage_bytes, splits_bytes, lanes_log2, threads;
  size_t bytes;
  bool ok;
};

static ProbPlan PlanProb(const k2b200_fsa_view *v) {
  ProbPlan p = {};
  if (!v->strict_layers || v->max_layer_states <= 0 || v->max_layer_arcs < 0 ||
      v->max_layers <= 0)
    return p;
  p.maxw = (v->max_layer_states + 3) & ~3;
  p.maxa = std::max(v->max_layer_arcs, 1);
  p.nl_cap = v->max_layers;
  // splits chunk: up to 3 leading and 3 trailing ints (the copy starts and ends on
  // 16-byte boundaries) + w + 1
  p.splits_bytes = (((p.maxw + 8) * 4) + 15) & ~15;
  p.stage_bytes = p.splits_bytes + p.maxa * 16;
  size_t fixed = 1024                                     // 64 full + 64 empty mbarriers
                 + 8 * (size_t)((p.nl_cap + 1 + 3) & ~3)  // layer / arc boundaries
                 + 2 * (size_t)p.maxw * 16 + 16;          // (mantissa, exponent) ping-pong
  // with more CTAs (2 per FSA) than SMs, leave room for two CTAs per SM
  size_t budget = 2 * (size_t)v->num_fsas > 148 ? kStagedSmemBudget / 2 : kStagedSmemBudget;
  if (fixed + 2 * (size_t)p.stage_bytes > budget) budget = kStagedSmemBudget;
  if (fixed + 2 * (size_t)p.stage_bytes > budget) return p;
  p.stages = (int32_t)std::min<size_t>(8, (budget - fixed) / p.stage_bytes);
  p.bytes = fixed + (size_t)p.stage_bytes * p.stages;
  int32_t mean_deg = v->num_states > 0 ? (v->num_arcs + v->num_states - 1) / v->num_states : 1;
  p.lanes_log2 = 0;
  while ((2 << p.lanes_log2) <= mean_deg / 2 && p.lanes_log2 < 5) ++p.lanes_log2;
  // compute threads plus one producer warp
  p.threads = (p.lanes_log2 >= 3 ? 224 : (p.lanes_log2 >= 1 ? 128 : 64)) + 32;
  p.ok = true;
  return p;
}

// grid = (directions, fsas).  m_out / e_out: [2][num_states] (forward then backward).
// Per layer one thread starts two bulk (TMA) copies into the ring - the per-state
// splits (from the 16-byte boundary below the first one) and the layer's ProbArcs -
// and every thread waits on the stage's mbarrier; the waits are bounded and raise
// *status when they give up.
__global__ void __launch_bounds__(256)
ProbScoresStaged(k2b200_fsa_view v, const ProbArc *__restrict__ fwd_arcs,
                 const ProbArc *__restrict__ bwd_arcs, double *__restrict__ m_out,
                 int32_t *__restrict__ e_out, int32_t dir_base, int32_t fsa_base, ProbPlan p,
                 int32_t *__restrict__ status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int32_t i = fsa_base + blockIdx.y, dir = blockIdx.x + dir_base;
  const int32_t s_begin = v.row_splits1[i], s_end = v.row_splits1[i + 1];
  if (s_end == s_begin) return;
  const int32_t lv0 = v.level_offsets[i], nl = v.level_offsets[i + 1] - lv0;
  const int tid = threadIdx.x, nt = blockDim.x;
  double *mo = m_out + (size_t)dir * v.num_states;
  int32_t *eo = e_out + (size_t)dir * v.num_states;

  uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw);  // [stages], 128 bytes reserved
  const int32_t lvl_ints = (p.nl_cap + 1 + 3) & ~3;
  int32_t *lvl = reinterpret_cast<int32_t *>(smem_raw + 1024);
  int32_t *alvl = lvl + lvl_ints;
  ProbState *pstate = reinterpret_cast<ProbState *>(alvl + lvl_ints);  // [2][maxw]
  unsigned char *ring = reinterpret_cast<unsigned char *>(pstate + 2 * p.maxw);
  const int32_t *gsplits = dir == 0 ? v.in_splits : v.row_splits2;
  const ProbArc *garcs = dir == 0 ? fwd_arcs : bwd_arcs;
  // last 4-int boundary inside the splits array (num_states + 1 entries)
  const int32_t splits_aligned_end = (v.num_states + 1) & ~3;

  __shared__ int32_t bad_shared;
  if (tid == 0) {
    bad_shared = (nl > p.nl_cap);
    for (int32_t s = 0; s < kMaxSlots; ++s) {
      MbarInit(&bars[s], 1);              // full: the producer's arrive + the copies' bytes
      MbarInit(&bars[kMaxSlots + s], 1);  // empty: one elected compute thread
    }
    MbarInitFence();
  }
  __syncthreads();
  if (!bad_shared)
    for (int32_t k = tid; k <= nl; k += nt) {
      int32_t s = v.level_splits[lv0 + k];
      lvl[k] = s;
      alvl[k] = gsplits[s];
    }
  __syncthreads();
  if (!bad_shared) {
    int32_t bad = 0;
    for (int32_t k = tid; k < nl; k += nt)
      bad |= (lvl[k + 1] - lvl[k] > p.maxw) | (alvl[k + 1] - alvl[k] > p.maxa);
    if (bad) bad_shared = 1;
  }
  __syncthreads();
  if (bad_shared) {  // the caller's bounds do not hold: report, the host falls back
    if (tid == 0) atomicExch(status, 1);
    return;
  }

  // The plan's stage size comes from loose bounds (a layer could hold every state
  // and arc of the graph); the layers of this lattice are usually smaller.  The ring
  // is re-cut into slots of the largest layer actually present so that more layers
  // are in flight.
  __shared__ int32_t max_splits_ints, max_arcs_shared;
  if (tid == 0) {
    max_splits_ints = 0;
    max_arcs_shared = 0;
  }
  __syncthreads();
  {
    int32_t ms = 0, ma = 0;
    for (int32_t k = tid; k < nl; k += nt) {
      ms = max(ms, lvl[k + 1] - lvl[k] + 8);
      ma = max(ma, alvl[k + 1] - alvl[k]);
    }
    atomicMax(&max_splits_ints, ms);
    atomicMax(&max_arcs_shared, ma);
  }
  __syncthreads();
  const int32_t splits_bytes = ((max_splits_ints * 4) + 15) & ~15;
  const int32_t slot_bytes = splits_bytes + (max_arcs_shared > 0 ? max_arcs_shared : 1) * 16;
  const int32_t ring_bytes = p.stage_bytes * p.stages;
  int32_t stages = ring_bytes / slot_bytes;
  stages = stages > kMaxSlots ? kMaxSlots : stages;
  // The last warp only feeds the ring (one thread of it); the others own the
  // states.  full[slot] completes when a layer's copies have landed, empty[slot]
  // when the compute warps are done reading it, so the producer runs up to
  // `stages` layers ahead and is never on the layer-to-layer critical path.
  const int32_t nc = nt - 32;
  uint64_t *full = bars, *empty = bars + kMaxSlots;
  auto layer_of = [&](int32_t step) { return dir == 0 ? step : nl - 1 - step; };
  if (tid >= nc) {
    if (tid != nc) return;
    int32_t slot = 0;
    unsigned empty_parity = 1;  // a fresh barrier counts as "previous phase complete"
    for (int32_t step = 0; step < nl; ++step) {
      if (!MbarTryWait(&empty[slot], empty_parity) &&
          !MbarWaitBounded(&empty[slot], empty_parity)) {
        atomicExch(status, 3);
        return;
      }
      const int32_t li = layer_of(step);
      const int32_t b = lvl[li], e = lvl[li + 1], ab = alvl[li], na = alvl[li + 1] - ab;
      unsigned char *st = ring + (size_t)slot * slot_bytes;
      int32_t *sp = reinterpret_cast<int32_t *>(st);
      const int32_t lo = b & ~3;
      int32_t hi = (e + 1 + 3) & ~3;
      hi = hi < splits_aligned_end ? hi : splits_aligned_end;
      hi = hi > lo ? hi : lo;
      const unsigned bytes_splits = (unsigned)(hi - lo) * 4u, bytes_arcs = (unsigned)na * 16u;
      for (int32_t k = hi; k <= e; ++k) sp[k - lo] = gsplits[k];  // at most 3 trailing ints
      MbarArriveExpectTx(&full[slot], bytes_splits + bytes_arcs);
      if (bytes_splits) BulkCopyG2S(sp, gsplits + lo, bytes_splits, &full[slot]);
      if (bytes_arcs) BulkCopyG2S(st + splits_bytes, garcs + ab, bytes_arcs, &full[slot]);
      slot = slot + 1 == stages ? 0 : slot + 1;
      empty_parity ^= (slot == 0);
    }
    return;
  }

  const int32_t lg = p.lanes_log2, G = 1 << lg, g = tid & (G - 1), per_pass = nc >> lg;
  int32_t slot = 0, prev_slot = -1;
  unsigned parity = 0;
  // first state of the layer handled in the previous step (the layer the arcs of
  // this step come from / lead to) and, walking forward, of the current layer
  int32_t edge = dir == 0 ? lvl[0] : lvl[nl];
  for (int32_t step = 0; step < nl; ++step) {
    if (!MbarTryWait(&full[slot], parity) && !MbarWaitBounded(&full[slot], parity)) {
      atomicExch(status, 2);
      *reinterpret_cast<volatile int32_t *>(&bad_shared) = 2;
    }
    // compute warps only: the previous layer's scores are complete and nobody reads
    // the previous slot any more
    asm volatile("bar.sync 1, %0;" ::"r"(nc) : "memory");
    if (*reinterpret_cast<volatile int32_t *>(&bad_shared)) break;  // uniform: a wait gave up
    if (tid == 0 && prev_slot >= 0)
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SmemAddr(&empty[prev_slot]))
                   : "memory");
    prev_slot = slot;
    int32_t b, w, ab;
    if (dir == 0) {
      b = edge;
      edge = lvl[step + 1];
      w = edge - b;
      ab = alvl[step];
    } else {
      const int32_t li = nl - 1 - step;
      b = lvl[li];
      w = edge - b;
      edge = b;
      ab = alvl[li];
    }
    const unsigned char *st = ring + (size_t)slot * slot_bytes;
    const int32_t *sp = reinterpret_cast<const int32_t *>(st) + (b & 3);
    const ProbArc *body = reinterpret_cast<const ProbArc *>(st + splits_bytes);
    slot = slot + 1 == stages ? 0 : slot + 1;
    parity ^= (slot == 0);
    const ProbState *prev = pstate + ((step + 1) & 1) * p.maxw;
    ProbState *cur = pstate + (step & 1) * p.maxw;
    for (int32_t j0 = 0; j0 < w; j0 += per_pass) {
      const int32_t j = j0 + (tid >> lg);
      int32_t k0 = 0, k1 = 0;
      if (j < w) {
        k0 = sp[j] - ab;
        k1 = sp[j + 1] - ab;
      }
      // Running sum of the terms m_prev * f * 2^(e_prev + k), kept as sum * 2^E with E
      // the largest exponent met so far; two arcs per trip so that their loads and
      // multiplies overlap.
      double sum = 0.0;
      int32_t E = kZeroExp;
      for (int32_t k = k0 + 2 * g; k < k1; k += 2 * G) {
        const bool two = k + 1 < k1;
        const ProbArc a0 = body[k], a1 = body[two ? k + 1 : k];
        const ProbState s0 = prev[a0.other], s1 = prev[a1.other];
        const double t0 = s0.m * a0.f, t1 = two ? s1.m * a1.f : 0.0;
        const int32_t e0 = t0 != 0.0 ? s0.e + a0.k : kZeroExp;
        const int32_t e1 = t1 != 0.0 ? s1.e + a1.k : kZeroExp;
        int32_t En = e0 > e1 ? e0 : e1;
        En = E > En ? E : En;
        sum = ScaleDown(sum, E - En) + ScaleDown(t0, e0 - En) + ScaleDown(t1, e1 - En);
        E = En;
      }
      for (int32_t d = G >> 1; d > 0; d >>= 1) {
        const int32_t Eo = __shfl_xor_sync(0xffffffffu, E, d);
        const double so = __shfl_xor_sync(0xffffffffu, sum, d);
        const int32_t En = Eo > E ? Eo : E;
        sum = ScaleDown(sum, E - En) + ScaleDown(so, Eo - En);
        E = En;
      }
      if (j < w && g == 0) {
        const int32_t s = b + j;
        ProbState r;
        r.e = E;
        r.m = Renorm(sum, &r.e);
        r.pad = 0;
        if (r.m == 0.0 && s == (dir == 0 ? s_begin : s_end - 1)) {  // start / final state: 1
          r.m = 1.0;
          r.e = 0;
        }
        cur[j] = r;
        mo[s] = r.m;
        eo[s] = r.e;
      }
    }
  }
}

size_t ProbScratchBytes(const k2b200_fsa_view *v) {
  // ProbArc arrays for both directions, (mantissa, exponent) per state and
  // direction, one status word
  return AlignUp(2 * sizeof(ProbArc) * (size_t)std::max(v->num_arcs, 1)) +
         AlignUp(2 * sizeof(double) * (size_t)std::max(v->num_states, 1)) +
         AlignUp(2 * sizeof(int32_t) * (size_t)std::max(v->num_states, 1)) + 256;
}

int32_t *ProbStatusWord(const k2b200_fsa_view *v, void *scratch) {
  char *q = reinterpret_cast<char *>(scratch);
  q += AlignUp(2 * sizeof(ProbArc) * (size_t)std::max(v->num_arcs, 1));
  q += AlignUp(2 * sizeof(double) * (size_t)std::max(v->num_states, 1));
  q += AlignUp(2 * sizeof(int32_t) * (size_t)std::max(v->num_states, 1));
  return reinterpret_cast<int32_t *>(q);
}

// Log-semiring scores through the mantissa/exponent recursion.  *launched stays
// false when the view does not qualify (the caller then uses another kernel).
// Kernels that find the view's bounds violated raise *status_word (device); the
// host reads it only via CheckProbStatus.
template <typename Real>
int32_t LaunchProbScores(const k2b200_fsa_view *v, Real *fwd, Real *bwd, void *scratch,
                         size_t scratch_bytes, cudaStream_t stream, bool *launched) {
  *launched = false;
  if (scratch == nullptr || scratch_bytes < ProbScratchBytes(v)) return kOk;
  if (fwd != nullptr && (v->in_src == nullptr || v->in_score == nullptr)) return kOk;
  if (v->row_ids1 == nullptr || v->row_ids2 == nullptr) return kOk;
  ProbPlan p = PlanProb(v);
  if (!p.ok || v->num_arcs == 0) return kOk;
  // bulk copies need 16-byte aligned sources
  auto aligned16 = [](const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
  if (!aligned16(scratch) || !aligned16(v->row_splits2) || (fwd && !aligned16(v->in_splits)))
    return kOk;
  char *q = reinterpret_cast<char *>(scratch);
  ProbArc *fwd_arcs = reinterpret_cast<ProbArc *>(q);
  ProbArc *bwd_arcs = fwd_arcs + std::max(v->num_arcs, 1);
  q += AlignUp(2 * sizeof(ProbArc) * (size_t)std::max(v->num_arcs, 1));
  double *m_out = reinterpret_cast<double *>(q);
  q += AlignUp(2 * sizeof(double) * (size_t)std::max(v->num_states, 1));
  int32_t *e_out = reinterpret_cast<int32_t *>(q);
  q += AlignUp(2 * sizeof(int32_t) * (size_t)std::max(v->num_states, 1));
  int32_t *status = reinterpret_cast<int32_t *>(q);
  K2B_CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
  { PrepareProbArcs<<<CeilDiv(v->num_arcs, 256), 256, 0, stream>>>(*v, fwd ? fwd_arcs : nullptr,
                                                                   bwd ? bwd_arcs : nullptr);
    NoteLaunch(); }
  int32_t ndir = (fwd != nullptr) + (bwd != nullptr), dir_base = fwd ? 0 : 1;
  K2B_CUDA_OK(cudaFuncSetAttribute(ProbScoresStaged, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)p.bytes));
  for (int32_t first = 0; first < v->num_fsas; first += 65535) {
    int32_t n = std::min(v->num_fsas - first, 65535);
    dim3 grid(ndir, n);
    { ProbScoresStaged<<<grid, p.threads, p.bytes, stream>>>(*v, fwd_arcs, bwd_arcs, m_out, e_out,
                                                            dir_base, first, p, status);
      NoteLaunch(); }
  }
  int32_t ns = v->num_states;
  if (fwd) { FinishLogScores<Real><<<CeilDiv(ns, 256), 256, 0, stream>>>(m_out, e_out, ns, fwd);
             NoteLaunch(); }
  if (bwd) { FinishLogScores<Real><<<CeilDiv(ns, 256), 256, 0, stream>>>(m_out + ns, e_out + ns,
                                                                        ns, bwd);
             NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  *launched = true;
  return kOk;
}

template int32_t LaunchProbScores<float>(const k2b200_fsa_view *, float *, float *, void *,
                                         size_t, cudaStream_t, bool *);
template int32_t LaunchProbScores<double>(const k2b200_fsa_view *, double *, double *, void *,
                                          size_t, cudaStream_t, bool *);

template int32_t LaunchStagedScores<float>(const k2b200_fsa_view *, int32_t, float *, float *,
                                           int32_t *, cudaStream_t, bool *);
template int32_t LaunchStagedScores<double>(const k2b200_fsa_view *, int32_t, double *, double *,
                                            int32_t *, cudaStream_t, bool *);

}  // namespace k2b

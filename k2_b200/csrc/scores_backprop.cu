// Derivatives of forward scores, backward scores and arc posteriors with respect to
// the arc scores of a top-sorted FsaVec, for callers that differentiate through
// per-state scores (k2's get_forward_scores / get_backward_scores / get_arc_post).
// Replaces k2::BackpropGetForwardScores (k2/csrc/fsa_utils.cu:1638-1795),
// k2::BackpropGetBackwardScores (:1457-1624) and k2::BackpropGetArcPost (:1281-1334).
//
// The reference walks its state batches with three launches and a segmented sum per
// batch.  Here one CTA owns one FSA and walks its layers (runs of states that no arc
// connects, see levels.cu) in a single launch: a thread takes a state, sums the
// derivatives of its leaving (forward scores) or entering (backward scores) arcs in arc
// order - the order of the reference's sequential sum - and adds the sum to the state's
// own derivative, which the next layer then reads.
#include <algorithm>
#include <cmath>

#include "../../include/k2b200.h"
#include "common.cuh"

namespace k2b {
namespace {

constexpr int kBackpropThreads = 512;

template <typename Real>
__device__ __forceinline__ Real NegInf() { return -(Real)INFINITY; }

// state_deriv: on entry dL/d(score) per state, on exit the accumulated derivatives;
// arc_deriv: dL/d(arc score) per arc.
// kForward: scores are forward scores; layers are walked from the last to the first
//   and a state gathers from its leaving arcs; `pick` = entering_arcs (tropical).
// !kForward: scores are backward scores; layers first to last, a state gathers from
//   its entering arcs; `pick` = best leaving arc per state (tropical).
template <typename Real, bool kForward>
__global__ void __launch_bounds__(kBackpropThreads)
BackpropScores(const int32_t *__restrict__ row_splits1, const int32_t *__restrict__ row_splits2,
               const Arc *__restrict__ arcs, const int32_t *__restrict__ in_splits,
               const int32_t *__restrict__ in_arcs, const int32_t *__restrict__ in_src,
               const int32_t *__restrict__ level_offsets,
               const int32_t *__restrict__ level_splits, const Real *__restrict__ scores,
               const int32_t *__restrict__ pick, int32_t log_semiring, Real *state_deriv,
               Real *__restrict__ arc_deriv, int32_t first_fsa) {
  const int32_t i = first_fsa + blockIdx.x;
  const int32_t base = row_splits1[i];
  const int32_t l0 = level_offsets[i], l1 = level_offsets[i + 1];
  for (int32_t step = 0; step < l1 - l0; ++step) {
    const int32_t layer = kForward ? l1 - 1 - step : l0 + step;
    const int32_t s_begin = level_splits[layer], s_end = level_splits[layer + 1];
    for (int32_t s = s_begin + threadIdx.x; s < s_end; s += blockDim.x) {
      Real sum = 0;
      if (kForward) {
        const Real src_score = scores[s];
        for (int32_t a = row_splits2[s]; a < row_splits2[s + 1]; ++a) {
          const Arc arc = arcs[a];
          const int32_t d = base + arc.dest;
          Real deriv;
          if (log_semiring) {
            Real dest_score = scores[d];
            if (dest_score == NegInf<Real>()) dest_score = -NegInf<Real>();
            deriv = exp(src_score + (Real)arc.score - dest_score) * state_deriv[d];
          } else {
            deriv = pick[d] == a ? state_deriv[d] : (Real)0;
          }
          arc_deriv[a] = deriv;
          sum += deriv;
        }
      } else {
        const Real dest_score = scores[s];
        for (int32_t k = in_splits[s]; k < in_splits[s + 1]; ++k) {
          const int32_t a = in_arcs[k], src = in_src[k];
          Real deriv;
          if (log_semiring) {
            Real src_score = scores[src];
            if (src_score == NegInf<Real>()) src_score = -NegInf<Real>();
            deriv = exp(dest_score + (Real)arcs[a].score - src_score) * state_deriv[src];
          } else {
            deriv = pick[src] == a ? state_deriv[src] : (Real)0;
          }
          arc_deriv[a] = deriv;
          sum += deriv;
        }
      }
      state_deriv[s] += sum;
    }
    __syncthreads();
  }
}

// best leaving arc of every state for the tropical backward scores: the last arc
// among those with the largest backward[dest] + score, -1 for a state without arcs
// (ArgMaxPerSublist with `>=`, k2/csrc/ragged_ops_inl.h:643-656)
template <typename Real>
__global__ void BestLeavingArc(const int32_t *__restrict__ row_splits2,
                               const int32_t *__restrict__ row_ids1,
                               const int32_t *__restrict__ row_splits1,
                               const Arc *__restrict__ arcs, const Real *__restrict__ backward,
                               int32_t num_states, int32_t *__restrict__ best) {
  const int32_t s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= num_states) return;
  const int32_t base = row_splits1[row_ids1[s]];
  Real val = NegInf<Real>();
  int32_t idx = -1;
  for (int32_t a = row_splits2[s]; a < row_splits2[s + 1]; ++a) {
    const Real x = backward[base + arcs[a].dest] + (Real)arcs[a].score;
    if (x >= val) {
      val = x;
      idx = a;
    }
  }
  best[s] = idx;
}

// forward_deriv[s] = sum of arc_post_deriv over the arcs leaving s, backward_deriv[s]
// the same over the arcs entering s; the final state's forward derivative and the
// start state's backward derivative are -0.5 * (sum over all arcs of the FSA), because
// the posterior subtracts half of each of the two total scores.
template <typename Real>
__global__ void __launch_bounds__(kBackpropThreads)
BackpropArcPost(const int32_t *__restrict__ row_splits1, const int32_t *__restrict__ row_splits2,
                const int32_t *__restrict__ in_splits, const int32_t *__restrict__ in_arcs,
                const Real *__restrict__ arc_post_deriv, Real *__restrict__ forward_deriv,
                Real *__restrict__ backward_deriv, int32_t first_fsa) {
  __shared__ Real partial[kBackpropThreads / 32];
  const int32_t i = first_fsa + blockIdx.x;
  const int32_t s_begin = row_splits1[i], s_end = row_splits1[i + 1];
  Real total = 0;
  for (int32_t s = s_begin + threadIdx.x; s < s_end; s += blockDim.x) {
    Real f = 0, b = 0;
    for (int32_t a = row_splits2[s]; a < row_splits2[s + 1]; ++a) f += arc_post_deriv[a];
    for (int32_t k = in_splits[s]; k < in_splits[s + 1]; ++k) b += arc_post_deriv[in_arcs[k]];
    forward_deriv[s] = f;
    backward_deriv[s] = b;
    total += f;
  }
  for (int d = 16; d > 0; d >>= 1) total += __shfl_xor_sync(0xffffffffu, total, d);
  if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = total;
  __syncthreads();
  if (threadIdx.x == 0 && s_end > s_begin) {
    Real t = 0;
    for (int w = 0; w < kBackpropThreads / 32; ++w) t += partial[w];
    forward_deriv[s_end - 1] = (Real)-0.5 * t;
    backward_deriv[s_begin] = (Real)-0.5 * t;
  }
}

template <typename Real>
int32_t LaunchBackprop(const k2b200_fsa_view *v, bool forward, int32_t log_semiring,
                       const void *scores, const int32_t *pick, void *state_deriv,
                       void *arc_deriv, int32_t *best_tmp, cudaStream_t stream) {
  const Arc *arcs = reinterpret_cast<const Arc *>(v->arcs);
  const Real *sc = reinterpret_cast<const Real *>(scores);
  if (!forward && !log_semiring && v->num_states > 0) {
    { BestLeavingArc<Real><<<CeilDiv(v->num_states, 256), 256, 0, stream>>>(
        v->row_splits2, v->row_ids1, v->row_splits1, arcs, sc, v->num_states, best_tmp);
      NoteLaunch(); }
    pick = best_tmp;
  }
  for (int32_t first = 0; first < v->num_fsas; first += 65535) {
    const int32_t n = std::min(v->num_fsas - first, 65535);
    if (forward) {
      { BackpropScores<Real, true><<<n, kBackpropThreads, 0, stream>>>(
          v->row_splits1, v->row_splits2, arcs, v->in_splits, v->in_arcs, v->in_src,
          v->level_offsets, v->level_splits, sc, pick, log_semiring,
          reinterpret_cast<Real *>(state_deriv), reinterpret_cast<Real *>(arc_deriv), first);
        NoteLaunch(); }
    } else {
      { BackpropScores<Real, false><<<n, kBackpropThreads, 0, stream>>>(
          v->row_splits1, v->row_splits2, arcs, v->in_splits, v->in_arcs, v->in_src,
          v->level_offsets, v->level_splits, sc, pick, log_semiring,
          reinterpret_cast<Real *>(state_deriv), reinterpret_cast<Real *>(arc_deriv), first);
        NoteLaunch(); }
    }
  }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

}  // namespace
}  // namespace k2b

using namespace k2b;  // NOLINT

extern "C" {

int32_t k2b200_fsa_scores_backprop(const k2b200_fsa_view *fsas, int32_t forward,
                                   int32_t log_semiring, int32_t use_double, const void *scores,
                                   const int32_t *entering_arcs, void *state_deriv,
                                   void *arc_deriv, int32_t *best_leaving_tmp, void *stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  K2B_REQUIRE(fsas != nullptr, "NULL view");
  if (fsas->num_fsas == 0 || fsas->num_states == 0) return kOk;
  K2B_REQUIRE(fsas->row_splits1 && fsas->row_splits2 && fsas->level_offsets && fsas->level_splits,
              "the view needs row_splits and the layering");
  K2B_REQUIRE(scores && state_deriv && (arc_deriv || fsas->num_arcs == 0), "NULL pointer");
  if (forward) {
    K2B_REQUIRE(log_semiring || entering_arcs,
                "tropical forward scores need entering_arcs to backpropagate");
  } else {
    K2B_REQUIRE(fsas->in_splits && fsas->in_arcs && fsas->in_src,
                "backward scores need the incoming-arc index to backpropagate");
    K2B_REQUIRE(log_semiring || (best_leaving_tmp && fsas->row_ids1),
                "tropical backward scores need best_leaving_tmp[num_states] and row_ids1");
  }
  return use_double ? LaunchBackprop<double>(fsas, forward != 0, log_semiring, scores,
                                             entering_arcs, state_deriv, arc_deriv,
                                             best_leaving_tmp, stream)
                    : LaunchBackprop<float>(fsas, forward != 0, log_semiring, scores,
                                            entering_arcs, state_deriv, arc_deriv,
                                            best_leaving_tmp, stream);
}

int32_t k2b200_fsa_arc_post_backprop(const k2b200_fsa_view *fsas, int32_t use_double,
                                     const void *arc_post_deriv, void *forward_deriv,
                                     void *backward_deriv, void *stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  K2B_REQUIRE(fsas != nullptr, "NULL view");
  if (fsas->num_fsas == 0 || fsas->num_states == 0) return kOk;
  K2B_REQUIRE(fsas->row_splits1 && fsas->row_splits2 && fsas->in_splits && fsas->in_arcs,
              "the view needs row_splits and the incoming-arc index");
  K2B_REQUIRE((arc_post_deriv || fsas->num_arcs == 0) && forward_deriv && backward_deriv,
              "NULL pointer");
  for (int32_t first = 0; first < fsas->num_fsas; first += 65535) {
    const int32_t n = std::min(fsas->num_fsas - first, 65535);
    if (use_double) {
      { BackpropArcPost<double><<<n, kBackpropThreads, 0, stream>>>(
          fsas->row_splits1, fsas->row_splits2, fsas->in_splits, fsas->in_arcs,
          reinterpret_cast<const double *>(arc_post_deriv),
          reinterpret_cast<double *>(forward_deriv), reinterpret_cast<double *>(backward_deriv),
          first); NoteLaunch(); }
    } else {
      { BackpropArcPost<float><<<n, kBackpropThreads, 0, stream>>>(
          fsas->row_splits1, fsas->row_splits2, fsas->in_splits, fsas->in_arcs,
          reinterpret_cast<const float *>(arc_post_deriv),
          reinterpret_cast<float *>(forward_deriv), reinterpret_cast<float *>(backward_deriv),
          first); NoteLaunch(); }
    }
  }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

}  // extern "C"

// Internal declarations shared by scores.cu and scores_staged.cu.
#pragma once
#include <cmath>

#include "../../include/k2b200.h"
#include "common.cuh"

namespace k2b {

template <typename Real> __device__ __forceinline__ Real ExpReal(Real x);
template <> __device__ __forceinline__ float ExpReal<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ double ExpReal<double>(double x) { return exp(x); }
template <typename Real> __device__ __forceinline__ Real LogReal(Real x);
template <> __device__ __forceinline__ float LogReal<float>(float x) { return logf(x); }
template <> __device__ __forceinline__ double LogReal<double>(double x) { return log(x); }

// Scores of FSA i in direction dir (0 forward, 1 backward), all threads of the CTA
// cooperating: one __syncthreads per layer; every load goes to global memory, so
// this works for any layering and any size.  forward/backward are read with
// ordinary (coherent) loads because the same CTA wrote them a layer earlier.
template <typename Real, bool kLog>
__device__ void LayeredScoresDevice(const k2b200_fsa_view &v, int32_t i, int32_t dir,
                                    Real *forward, Real *backward, int32_t *entering_arcs) {
  const int32_t *row_splits1 = v.row_splits1, *row_splits2 = v.row_splits2,
                *row_ids2 = v.row_ids2, *in_splits = v.in_splits, *in_arcs = v.in_arcs,
                *level_offsets = v.level_offsets, *level_splits = v.level_splits;
  const Arc *arcs = reinterpret_cast<const Arc *>(v.arcs);
  const int32_t s_begin = row_splits1[i], s_end = row_splits1[i + 1];
  if (s_end == s_begin) return;
  const int32_t lv0 = level_offsets[i], lv1 = level_offsets[i + 1];
  const Real kNegInf = -INFINITY;
  if (dir == 0) {
    for (int32_t lv = lv0; lv < lv1; ++lv) {
      const int32_t b = level_splits[lv], e = level_splits[lv + 1];
      for (int32_t s = b + threadIdx.x; s < e; s += blockDim.x) {
        const int32_t k0 = in_splits[s], k1 = in_splits[s + 1];
        Real val = kNegInf;
        int32_t best = -1;
        if (kLog) {
          Real m = kNegInf;
          for (int32_t k = k0; k < k1; ++k) {
            int32_t a = in_arcs[k];
            Real x = forward[row_ids2[a]] + (Real)arcs[a].score;
            m = x > m ? x : m;
          }
          if (m != kNegInf) {
            Real sum = 0;
            for (int32_t k = k0; k < k1; ++k) {
              int32_t a = in_arcs[k];
              Real x = forward[row_ids2[a]] + (Real)arcs[a].score;
              sum += ExpReal<Real>(x - m);
            }
            val = m + LogReal<Real>(sum);
          }
        } else {
          for (int32_t k = k0; k < k1; ++k) {
            int32_t a = in_arcs[k];
            Real x = forward[row_ids2[a]] + (Real)arcs[a].score;
            if (x >= val) {  // ties: the later arc wins (ragged_ops_inl.h:649-655)
              val = x;
              best = a;
            }
          }
        }
        if (s == s_begin && val == kNegInf) val = 0;  // start state
        forward[s] = val;
        if (entering_arcs) entering_arcs[s] = best;
      }
      __syncthreads();
    }
  } else {
    for (int32_t lv = lv1 - 1; lv >= lv0; --lv) {
      const int32_t b = level_splits[lv], e = level_splits[lv + 1];
      for (int32_t s = b + threadIdx.x; s < e; s += blockDim.x) {
        const int32_t k0 = row_splits2[s], k1 = row_splits2[s + 1];
        Real val = kNegInf;
        if (kLog) {
          Real m = kNegInf;
          for (int32_t k = k0; k < k1; ++k) {
            Real x = backward[s_begin + arcs[k].dest] + (Real)arcs[k].score;
            m = x > m ? x : m;
          }
          if (m != kNegInf) {
            Real sum = 0;
            for (int32_t k = k0; k < k1; ++k) {
              Real x = backward[s_begin + arcs[k].dest] + (Real)arcs[k].score;
              sum += ExpReal<Real>(x - m);
            }
            val = m + LogReal<Real>(sum);
          }
        } else {
          for (int32_t k = k0; k < k1; ++k) {
            Real x = backward[s_begin + arcs[k].dest] + (Real)arcs[k].score;
            val = x > val ? x : val;
          }
        }
        if (s == s_end - 1 && val == kNegInf) val = 0;  // final state
        backward[s] = val;
      }
      __syncthreads();
    }
  }
}


// Mantissa/exponent log-semiring recursion (scores_staged.cu).
size_t ProbScratchBytes(const k2b200_fsa_view *v);
template <typename Real>
int32_t LaunchProbScores(const k2b200_fsa_view *v, Real *fwd, Real *bwd, void *scratch,
                         size_t scratch_bytes, cudaStream_t stream, bool *launched);
// Address of the status word inside the scratch: non-zero after LaunchProbScores
// means the view's layer bounds did not hold and the results must be recomputed.
int32_t *ProbStatusWord(const k2b200_fsa_view *v, void *scratch);

template <typename Real>
int32_t LaunchStagedScores(const k2b200_fsa_view *v, int32_t log_semiring, Real *fwd, Real *bwd,
                           int32_t *entering, cudaStream_t stream, bool *launched);

}  // namespace k2b

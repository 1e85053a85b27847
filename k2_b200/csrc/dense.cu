// DenseFsaVec construction and its backward as single kernels.
//
// The reference builds the [sum(T_i + 1), C + 1] score matrix with a Python loop, a
// torch index_select over whole rows and three fill operations
// (k2/python/k2/dense_fsa_vec.py:101-133); autograd later replays that backwards
// with an index_add over the full matrix.  Here one kernel writes every element of
// the matrix exactly once (column 0, the gathered log-probs, and the extra final
// row of each sequence), and one kernel scatters the gradient back.
#include "../../include/k2b200.h"
#include "common.cuh"

namespace k2b {

// Segment owning score row r (row_splits has num_segs + 1 entries).
__device__ __forceinline__ int32_t SegmentOfRow(const int32_t *__restrict__ row_splits,
                                                int32_t num_segs, int32_t r) {
  int32_t lo = 0, hi = num_segs;
  while (hi - lo > 1) {
    int32_t mid = (lo + hi) >> 1;
    if (row_splits[mid] <= r) lo = mid; else hi = mid;
  }
  return lo;
}

// One warp per score row (no block-level synchronisation: the rows are short and
// there are tens of thousands of them).  segments: [num_segs, 3] = (sequence,
// start_frame, duration after truncation).
constexpr int kRowsPerCta = 8;

// Row of log_probs viewed as [N*T, C] that score row r copies, -1 for a final row.
__device__ __forceinline__ int64_t SourceRow(const int32_t *__restrict__ segments,
                                             const int32_t *__restrict__ row_splits,
                                             int32_t num_segs, int64_t T, int32_t r) {
  const int32_t k = SegmentOfRow(row_splits, num_segs, r);
  const int32_t t = r - row_splits[k], dur = row_splits[k + 1] - row_splits[k] - 1;
  return t < dur ? (int64_t)segments[3 * k] * T + segments[3 * k + 1] + t : -1;
}

__global__ void __launch_bounds__(32 * kRowsPerCta)
DenseFill(const float *__restrict__ log_probs, int64_t T, int32_t C,
          const int32_t *__restrict__ segments, const int32_t *__restrict__ row_splits,
          int32_t num_segs, int32_t rows, float *__restrict__ scores) {
  const int32_t r = blockIdx.x * kRowsPerCta + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const int64_t src = SourceRow(segments, row_splits, num_segs, T, r);
  float *out = scores + (int64_t)r * (C + 1);
  if (src >= 0) {
    const float *in = log_probs + src * C;
    if (lane == 0) out[0] = -INFINITY;
    for (int32_t c = lane; c < C; c += 32) out[1 + c] = __ldg(in + c);
  } else {
    if (lane == 0) out[0] = 0.0f;
    for (int32_t c = lane; c < C; c += 32) out[1 + c] = -INFINITY;
  }
}

// grad_log_probs[seq, start + t, c] (+)= grad_scores[row, 1 + c].
__global__ void __launch_bounds__(32 * kRowsPerCta)
DenseBackward(const float *__restrict__ grad_scores, int64_t T, int32_t C,
              const int32_t *__restrict__ segments, const int32_t *__restrict__ row_splits,
              int32_t num_segs, int32_t rows, int32_t use_atomics,
              float *__restrict__ grad_log_probs) {
  const int32_t r = blockIdx.x * kRowsPerCta + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const int64_t dst = SourceRow(segments, row_splits, num_segs, T, r);
  if (dst < 0) return;
  const float *in = grad_scores + (int64_t)r * (C + 1) + 1;
  float *out = grad_log_probs + dst * C;
  if (use_atomics) {
    for (int32_t c = lane; c < C; c += 32) atomicAdd(out + c, in[c]);
  } else {
    for (int32_t c = lane; c < C; c += 32) out[c] = in[c];
  }
}

// ---------------------------------------------------------------------------
// log_softmax fused with the layout: scores = layout(log_softmax(logits, dim=-1)).
// The reference's callers run torch.log_softmax over [N, T, C] and then build the
// DenseFsaVec from the result (k2/python/k2/dense_fsa_vec.py:101-133): two full
// passes over the matrix forward and two more backward.  Here one warp per score row
// normalises its row while it lays it out, and the backward applies
//   dL/dlogit[c] = g[c] - softmax[c] * sum_c' g[c'],   softmax = exp(scores)
// while it scatters.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float WarpMax(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
  return v;
}
__device__ __forceinline__ float WarpSum(float v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

// One warp per score row, as DenseFill.
__global__ void __launch_bounds__(32 * kRowsPerCta)
LogSoftmaxFill(const float *__restrict__ logits, int64_t T, int32_t C,
               const int32_t *__restrict__ segments, const int32_t *__restrict__ row_splits,
               int32_t num_segs, int32_t rows, float *__restrict__ scores) {
  const int32_t r = blockIdx.x * kRowsPerCta + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const int64_t src = SourceRow(segments, row_splits, num_segs, T, r);
  float *out = scores + (int64_t)r * (C + 1);
  if (src < 0) {
    if (lane == 0) out[0] = 0.0f;
    for (int32_t c = lane; c < C; c += 32) out[1 + c] = -INFINITY;
    return;
  }
  const float *in = logits + src * C;
  float mx = -INFINITY;
  for (int32_t c = lane; c < C; c += 32) mx = fmaxf(mx, __ldg(in + c));
  mx = WarpMax(mx);
  float sum = 0.0f;
  for (int32_t c = lane; c < C; c += 32) sum += expf(__ldg(in + c) - mx);
  const float lse = logf(WarpSum(sum));
  if (lane == 0) out[0] = -INFINITY;
  for (int32_t c = lane; c < C; c += 32) out[1 + c] = (__ldg(in + c) - mx) - lse;
}

__global__ void __launch_bounds__(32 * kRowsPerCta)
LogSoftmaxBackward(const float *__restrict__ grad_scores, const float *__restrict__ scores,
                   int64_t T, int32_t C, const int32_t *__restrict__ segments,
                   const int32_t *__restrict__ row_splits, int32_t num_segs, int32_t rows,
                   int32_t use_atomics, float *__restrict__ grad_logits) {
  const int32_t r = blockIdx.x * kRowsPerCta + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const int64_t dst = SourceRow(segments, row_splits, num_segs, T, r);
  if (dst < 0) return;
  const float *g = grad_scores + (int64_t)r * (C + 1) + 1;
  const float *lp = scores + (int64_t)r * (C + 1) + 1;
  float gsum = 0.0f;
  for (int32_t c = lane; c < C; c += 32) gsum += g[c];
  gsum = WarpSum(gsum);
  float *out = grad_logits + dst * C;
  for (int32_t c = lane; c < C; c += 32) {
    const float v = g[c] - expf(lp[c]) * gsum;
    if (use_atomics) atomicAdd(out + c, v); else out[c] = v;
  }
}

}  // namespace k2b

using namespace k2b;

extern "C" {

int32_t k2b200_dense_fsa_vec_fill(const float *log_probs, int64_t num_seqs, int64_t num_frames,
                                  int32_t num_classes, const int32_t *segments,
                                  const int32_t *row_splits, int32_t num_segs, float *scores,
                                  int32_t rows, void *stream) {
  (void)num_seqs;
  K2B_REQUIRE(log_probs && segments && row_splits && scores, "NULL pointer");
  K2B_REQUIRE(num_segs > 0 && num_classes > 0 && rows > 0, "empty DenseFsaVec");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  PhaseTimer timer(kPhaseDense, s);
  { DenseFill<<<CeilDiv(rows, kRowsPerCta), 32 * kRowsPerCta, 0, s>>>(
      log_probs, num_frames, num_classes, segments, row_splits, num_segs, rows, scores);
    NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t k2b200_dense_fsa_vec_backward(const float *grad_scores, int64_t num_seqs,
                                      int64_t num_frames, int32_t num_classes,
                                      const int32_t *segments, const int32_t *row_splits,
                                      int32_t num_segs, int32_t rows, int32_t overlapping,
                                      float *grad_log_probs, void *stream) {
  K2B_REQUIRE(grad_scores && segments && row_splits && grad_log_probs, "NULL pointer");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  PhaseTimer timer(kPhaseDense, s);
  K2B_CUDA_OK(cudaMemsetAsync(grad_log_probs, 0,
                              sizeof(float) * (size_t)num_seqs * num_frames * num_classes, s));
  if (rows > 0)
    { DenseBackward<<<CeilDiv(rows, kRowsPerCta), 32 * kRowsPerCta, 0, s>>>(
        grad_scores, num_frames, num_classes, segments, row_splits, num_segs, rows, overlapping,
        grad_log_probs); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t k2b200_dense_fsa_vec_from_logits(const float *logits, int64_t num_seqs,
                                         int64_t num_frames, int32_t num_classes,
                                         const int32_t *segments, const int32_t *row_splits,
                                         int32_t num_segs, float *scores, int32_t rows,
                                         void *stream) {
  (void)num_seqs;
  K2B_REQUIRE(logits && segments && row_splits && scores, "NULL pointer");
  K2B_REQUIRE(num_segs > 0 && num_classes > 0 && rows > 0, "empty DenseFsaVec");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  PhaseTimer timer(kPhaseDense, s);
  { LogSoftmaxFill<<<CeilDiv(rows, kRowsPerCta), 32 * kRowsPerCta, 0, s>>>(
      logits, num_frames, num_classes, segments, row_splits, num_segs, rows, scores);
    NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t k2b200_dense_fsa_vec_from_logits_backward(const float *grad_scores, const float *scores,
                                                  int64_t num_seqs, int64_t num_frames,
                                                  int32_t num_classes, const int32_t *segments,
                                                  const int32_t *row_splits, int32_t num_segs,
                                                  int32_t rows, int32_t overlapping,
                                                  float *grad_logits, void *stream) {
  K2B_REQUIRE(grad_scores && scores && segments && row_splits && grad_logits, "NULL pointer");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  PhaseTimer timer(kPhaseDense, s);
  K2B_CUDA_OK(cudaMemsetAsync(grad_logits, 0,
                              sizeof(float) * (size_t)num_seqs * num_frames * num_classes, s));
  if (rows > 0)
    { LogSoftmaxBackward<<<CeilDiv(rows, kRowsPerCta), 32 * kRowsPerCta, 0, s>>>(
        grad_scores, scores, num_frames, num_classes, segments, row_splits, num_segs, rows,
        overlapping, grad_logits); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

}  // extern "C"

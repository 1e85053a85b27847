// Layering of a top-sorted, acyclic FsaVec for the score kernels: level(s) = length
// of the longest path from any state without entering arcs to s, so every arc goes
// from a lower to a higher level.  The reference gets its "state batches" from a
// repeated frontier expansion (k2/csrc/fsa_utils.cu:679-899, GetStateBatches); here
// one CTA per FSA relaxes level[dest] = max(level[dest], level[src] + 1) over the
// FSA's arcs until nothing changes (at most depth + 1 sweeps), then the levels are
// turned into contiguous layers: where the states of an FSA are already ordered by
// level a layer is a run of equal levels, otherwise every state is its own layer
// (always valid for a top-sorted FSA).
#include <algorithm>

#include "../../include/k2b200.h"
#include "common.cuh"

namespace k2b {

// status bits
constexpr int32_t kNotTopSorted = 1;

__global__ void __launch_bounds__(1024)
LevelsRelax(const int32_t *__restrict__ row_splits1, const int32_t *__restrict__ row_splits2,
            const int32_t *__restrict__ row_ids2, const Arc *__restrict__ arcs,
            int32_t *__restrict__ level, int32_t *__restrict__ flags,
            int32_t *__restrict__ status) {
  const int32_t i = blockIdx.x;
  const int32_t b = row_splits1[i], e = row_splits1[i + 1];
  if (e == b) return;
  const int32_t a0 = row_splits2[b], a1 = row_splits2[e];
  const int tid = threadIdx.x, nt = blockDim.x;
  for (int32_t s = b + tid; s < e; s += nt) level[s] = 0;
  bool bad = false;
  for (int32_t a = a0 + tid; a < a1; a += nt)
    if (b + arcs[a].dest <= row_ids2[a]) bad = true;  // not top-sorted (or a self-loop)
  if (__syncthreads_or(bad)) {
    if (tid == 0) atomicOr(status, kNotTopSorted);
    return;
  }
  // at most (number of states) sweeps can change anything in an acyclic graph
  for (int32_t sweep = 0; sweep <= e - b; ++sweep) {
    bool changed = false;
    for (int32_t a = a0 + tid; a < a1; a += nt) {
      const int32_t want = level[row_ids2[a]] + 1, d = b + arcs[a].dest;
      if (level[d] < want) {
        atomicMax(&level[d], want);
        changed = true;
      }
    }
    if (!__syncthreads_or(changed)) break;
  }
  // layers: runs of equal level when the states are ordered by level
  bool ordered = true;
  for (int32_t s = b + 1 + tid; s < e; s += nt)
    if (level[s] < level[s - 1]) ordered = false;
  ordered = !__syncthreads_or(!ordered);
  for (int32_t s = b + tid; s < e; s += nt)
    flags[s] = (s == b || !ordered || level[s] != level[s - 1]) ? 1 : 0;
}

__global__ void LevelsWrite(const int32_t *__restrict__ row_splits1, int32_t num_fsas,
                            int32_t num_states, const int32_t *__restrict__ flags,
                            const int32_t *__restrict__ pos, int32_t *__restrict__ level_offsets,
                            int32_t *__restrict__ level_splits) {
  const int32_t k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k < num_states && flags[k]) level_splits[pos[k]] = k;
  if (k <= num_fsas) level_offsets[k] = pos[row_splits1[k]];  // pos[num_states] = total
  if (k == 0) level_splits[pos[num_states]] = num_states;
}

}  // namespace k2b

using namespace k2b;

extern "C" {

size_t k2b200_fsa_levels_tmp_bytes(int32_t num_states) {
  // levels, flags (+1), positions (+1), scan scratch
  return AlignUp(sizeof(int32_t) * (size_t)std::max(num_states, 1)) +
         2 * AlignUp(sizeof(int32_t) * ((size_t)num_states + 1)) +
         AlignUp(sizeof(int32_t) * ScanTmpInts(num_states + 1));
}

int32_t k2b200_fsa_levels(const int32_t *row_splits1, const int32_t *row_splits2,
                          const int32_t *row_ids2, const void *arcs, int32_t num_fsas,
                          int32_t num_states, int32_t num_arcs, int32_t *level_offsets,
                          int32_t *level_splits, int32_t *status, void *tmp, void *stream_v) {
  (void)num_arcs;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  K2B_REQUIRE(row_splits1 && row_splits2 && level_offsets && level_splits && status && tmp,
              "NULL pointer");
  K2B_REQUIRE(num_fsas >= 0 && num_states >= 0, "negative size");
  char *p = reinterpret_cast<char *>(tmp);
  int32_t *level = reinterpret_cast<int32_t *>(p);
  p += AlignUp(sizeof(int32_t) * (size_t)std::max(num_states, 1));
  int32_t *flags = reinterpret_cast<int32_t *>(p);
  p += AlignUp(sizeof(int32_t) * ((size_t)num_states + 1));
  int32_t *pos = reinterpret_cast<int32_t *>(p);
  p += AlignUp(sizeof(int32_t) * ((size_t)num_states + 1));
  int32_t *scan_tmp = reinterpret_cast<int32_t *>(p);
  K2B_CUDA_OK(cudaMemsetAsync(status, 0, sizeof(int32_t), stream));
  K2B_CUDA_OK(cudaMemsetAsync(flags, 0, sizeof(int32_t) * ((size_t)num_states + 1), stream));
  if (num_fsas > 0 && num_states > 0)
    { LevelsRelax<<<num_fsas, 1024, 0, stream>>>(row_splits1, row_splits2, row_ids2,
                                                 reinterpret_cast<const Arc *>(arcs), level, flags,
                                                 status); NoteLaunch(); }
  K2B_FORWARD(ExclusiveSum(flags, pos, num_states, scan_tmp, stream));
  { LevelsWrite<<<CeilDiv(std::max(num_states, num_fsas) + 1, 256), 256, 0, stream>>>(
      row_splits1, num_fsas, num_states, flags, pos, level_offsets, level_splits); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

}  // extern "C"

// intersect_dense for sm_100a: Viterbi forward/backward recursion over the frames
// of every (graph, sequence) pair, exact output-beam pruning, and compaction of
// the surviving states and arcs into a k2 FsaVec with both arc maps.
//
// Behaviour follows k2::MultiGraphDenseIntersect (k2/csrc/intersect_dense.cu):
//   DoStep0/DoStep   :745-847   max-recursion, (prev + arc.score) + dense score
//   GetScoreCutoffs  :870-924   cutoff = min(bwd[start], fwd[final]) - beam
//   FormatOutput     :226-603   keep tests, numbering (fsa, t, state), arc maps
//   DecreaseBeam     :854-862   beam shrink when max_states / max_arcs is hit
// but not its structure: there is no per-arc score buffer, no segmented reduce
// library call and no per-frame host work in the persistent mode.
//
// Compiled with -fmad=false: every sum that decides whether a state or an arc is
// kept is a chain of plain IEEE fp32 additions in the reference's order.
#include <algorithm>
#include <cmath>
#include <vector>

#include "intersect_internal.cuh"

namespace k2b {

constexpr int kCountThreads = 256;
constexpr int kWordsPerCtaHost = 4 * 4 * (kCountThreads / 32);  // == kWordsPerCta below

int32_t MakeLayout(const k2b200_intersect_args *a, Layout *L) {
  K2B_REQUIRE(a != nullptr, "args is NULL");
  K2B_REQUIRE(a->num_fsas > 0, "a_fsas must contain at least one FSA (got %d)", a->num_fsas);
  K2B_REQUIRE(a->output_beam > 0, "output_beam must be > 0 (got %f)", a->output_beam);
  K2B_REQUIRE(a->h_a_row_splits1 && a->h_a_arc_splits && a->h_b_row_splits,
              "host copies of the row splits are required");
  K2B_REQUIRE(a->num_seqs > 0 && a->cols > 0, "empty DenseFsaVec");
  if (a->h_a_to_b_map == nullptr)
    K2B_REQUIRE(a->num_fsas == a->num_seqs,
                "a_fsas.Dim0() (%d) != b_fsas.Dim0() (%d) and no a_to_b_map given",
                a->num_fsas, a->num_seqs);
  for (int32_t j = 1; j < a->num_seqs; ++j) {
    int32_t prev = a->h_b_row_splits[j] - a->h_b_row_splits[j - 1],
            cur = a->h_b_row_splits[j + 1] - a->h_b_row_splits[j];
    K2B_REQUIRE(cur <= prev,
                "Sequences (DenseFsaVec) must be in sorted order from greatest to least "
                "length; sequence %d has %d rows after %d",
                j, cur, prev);
  }
  K2B_REQUIRE((int64_t)a->rows * a->cols < ((int64_t)1 << 31),
              "scores has too many elements for int32 arc_map_b");
  L->infos.resize(a->num_fsas);
  int64_t grid = 0, words = 0, levels = 0;
  for (int32_t i = 0; i < a->num_fsas; ++i) {
    int32_t j = a->h_a_to_b_map ? a->h_a_to_b_map[i] : i;
    K2B_REQUIRE(j >= 0 && j < a->num_seqs, "a_to_b_map[%d] = %d out of range [0, %d)", i, j,
                a->num_seqs);
    if (i > 0 && a->h_a_to_b_map)
      K2B_REQUIRE(a->h_a_to_b_map[i] >= a->h_a_to_b_map[i - 1],
                  "a_to_b_map should be monotonically increasing");
    FsaInfo &f = L->infos[i];
    f.state_off = a->h_a_row_splits1[i];
    f.num_states = a->h_a_row_splits1[i + 1] - f.state_off;
    f.arc_off = a->h_a_arc_splits[i];
    f.num_arcs = a->h_a_arc_splits[i + 1] - f.arc_off;
    f.arc_out_off = 0;
    if (a->a_shared) {  // read graph 0 in place of its copy i
      K2B_REQUIRE(f.num_states == a->h_a_row_splits1[1] - a->h_a_row_splits1[0] &&
                      f.num_arcs == a->h_a_arc_splits[1] - a->h_a_arc_splits[0],
                  "a_shared is set but graph %d differs in size from graph 0", i);
      f.arc_out_off = f.arc_off - a->h_a_arc_splits[0];
      f.state_off = a->h_a_row_splits1[0];
      f.arc_off = a->h_a_arc_splits[0];
    }
    f.row0 = a->h_b_row_splits[j];
    f.tk = a->h_b_row_splits[j + 1] - f.row0;
    K2B_REQUIRE(f.tk >= 1, "sequence %d has no rows", j);
    f.level_off = (int32_t)levels;
    f.words = (f.num_states + 31) / 32;
    f.grid_off = grid;
    f.word_off = words;
    grid += (int64_t)(f.tk + 1) * f.num_states;
    words += (int64_t)(f.tk + 1) * f.words;
    levels += f.tk + 1;
    L->max_states = std::max(L->max_states, f.num_states);
    L->max_arcs = std::max(L->max_arcs, f.num_arcs);
    L->max_tk = std::max(L->max_tk, f.tk);
  }
  if (levels >= ((int64_t)1 << 31) || words >= ((int64_t)1 << 31)) {
    SetError("problem too large: %lld (fsa, frame) levels, %lld state words",
             (long long)levels, (long long)words);
    return kTooLarge;
  }
  L->grid_elems = grid;
  L->total_words = words;
  L->total_levels = levels;
  // CountKept / EmitLattice run on a (word tiles of the largest pair, pairs) grid
  int64_t max_pair_words = 0;
  for (const FsaInfo &f : L->infos)
    max_pair_words = std::max<int64_t>(max_pair_words, (int64_t)(f.tk + 1) * f.words);
  L->tiles_per_pair = CeilDiv(max_pair_words, kWordsPerCtaHost);
  L->emit_tiles_per_pair = CeilDiv(max_pair_words, 16 * 8);  // kEmitWordsPerCta
  L->count_blocks = (int32_t)std::min<int64_t>((int64_t)L->tiles_per_pair * a->num_fsas,
                                               0x7fffffff);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off += AlignUp(bytes ? bytes : 1);
    return o;
  };
  L->off_infos = take(sizeof(FsaInfo) * a->num_fsas);
  L->off_cutoffs = take(sizeof(float) * a->num_fsas);
  L->off_fwd = take(sizeof(float) * (size_t)grid);
  L->off_bwd = take(sizeof(float) * (size_t)grid);
  L->off_mask = take(sizeof(uint32_t) * (size_t)words);
  L->off_counts = take(sizeof(int2) * ((size_t)words + 1));
  L->off_scan_tmp = take(sizeof(int2) * ScanTmpInts(words));
  L->off_block_cand = take(sizeof(unsigned long long) * (size_t)L->count_blocks);
  L->off_totals = take(64);
  L->lane_plan = LanePlanApplies(*L, a);
  L->off_plan = take(L->lane_plan ? sizeof(int32_t) * 2 * (size_t)a->num_fsas * kLaneThreads : 0);
  L->off_unfit = take(sizeof(int32_t) * (size_t)a->num_fsas);
  // a shared graph too large for the one-CTA kernels: sequences on the lanes of a warp
  L->shared_vit = (a->viterbi_mode == 5 ||
                   (a->viterbi_mode == 0 && !RegisterViterbiFits(*L, a) && !L->lane_plan &&
                    !PersistentViterbiFits(*L, a))) &&
                  SharedViterbiApplies(*L, a);
  L->off_shared_vit = take(L->shared_vit ? SharedViterbiBytes(*L, a) : 0);
  L->total_bytes = off;
  return kOk;
}

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ float DenseScore(const float *__restrict__ scores, int64_t row,
                                            int32_t cols, int32_t label) {
  int32_t c = label + 1;
  return (c >= 0 && c < cols) ? __ldg(scores + row * cols + c) : -INFINITY;
}

// ---------------------------------------------------------------------------
// Viterbi recursion, one launch per frame (any graph size).
// grid = (state tiles, pairs, 2 directions); G = 2^lanes_log2 lanes per state.
// ---------------------------------------------------------------------------
__global__ void ViterbiInit(const FsaInfo *__restrict__ infos, float *__restrict__ fwd,
                            float *__restrict__ bwd) {
  FsaInfo f = infos[blockIdx.y];
  int32_t s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= f.num_states) return;
  fwd[f.grid_off + s] = (s == 0) ? 0.0f : -INFINITY;
  bwd[f.grid_off + (int64_t)f.tk * f.num_states + s] =
      (s == f.num_states - 1) ? 0.0f : -INFINITY;
}

__global__ void __launch_bounds__(256)
ViterbiStep(const FsaInfo *__restrict__ infos, int32_t t, const Arc *__restrict__ arcs,
            const int32_t *__restrict__ a_row_splits2, const int32_t *__restrict__ in_splits,
            const int32_t *__restrict__ in_arcs, const float *__restrict__ scores,
            int32_t cols, float *__restrict__ fwd, float *__restrict__ bwd,
            int32_t lanes_log2) {
  const FsaInfo f = infos[blockIdx.y];
  if (t > f.tk) return;
  const int32_t gtid = blockIdx.x * blockDim.x + threadIdx.x;
  const int32_t s = gtid >> lanes_log2, g = gtid & ((1 << lanes_log2) - 1), G = 1 << lanes_log2;
  const bool active = s < f.num_states;
  const int32_t S = f.num_states;
  float best = -INFINITY;
  if (blockIdx.z == 0) {
    // forward: state copies of time t from time t-1, dense row t-1
    if (active) {
      const float *prev = fwd + f.grid_off + (int64_t)(t - 1) * S;
      const int64_t row = (int64_t)f.row0 + (t - 1);
      const int32_t idx01 = f.state_off + s;
      for (int32_t k = in_splits[idx01] + g; k < in_splits[idx01 + 1]; k += G) {
        Arc arc = arcs[in_arcs[k]];
        float v = __fadd_rn(__fadd_rn(prev[arc.src], arc.score),
                            DenseScore(scores, row, cols, arc.label));
        best = v > best ? v : best;
      }
    }
  } else {
    // backward: time position tk - t from position tk - t + 1, dense row tk - t
    if (active) {
      const float *next = bwd + f.grid_off + (int64_t)(f.tk - t + 1) * S;
      const int64_t row = (int64_t)f.row0 + (f.tk - t);
      const int32_t idx01 = f.state_off + s;
      for (int32_t k = a_row_splits2[idx01] + g; k < a_row_splits2[idx01 + 1]; k += G) {
        Arc arc = arcs[k];
        float v = __fadd_rn(__fadd_rn(next[arc.dest], arc.score),
                            DenseScore(scores, row, cols, arc.label));
        best = v > best ? v : best;
      }
    }
  }
  for (int32_t d = G >> 1; d > 0; d >>= 1) {
    float o = __shfl_xor_sync(0xffffffffu, best, d);
    best = o > best ? o : best;
  }
  if (active && g == 0) {
    if (blockIdx.z == 0) fwd[f.grid_off + (int64_t)t * S + s] = best;
    else bwd[f.grid_off + (int64_t)(f.tk - t) * S + s] = best;
  }
}

// ---------------------------------------------------------------------------
// pruning: cutoffs, keep masks + counts, numbering, emission
// ---------------------------------------------------------------------------
__global__ void Cutoffs(const FsaInfo *__restrict__ infos, int32_t n,
                        const float *__restrict__ fwd, const float *__restrict__ bwd,
                        float beam, float *__restrict__ cutoffs) {
  int32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  FsaInfo f = infos[i];
  float start = -INFINITY, end = -INFINITY;
  if (f.num_states > 0) {
    start = bwd[f.grid_off];  // backward score of state 0 at time 0
    end = fwd[f.grid_off + (int64_t)f.tk * f.num_states + (f.num_states - 1)];
  }
  float mn = start < end ? start : end;
  cutoffs[i] = __fsub_rn(mn, beam);
}

// Does arc (leaving a kept state at time t) survive?  fs = forward score of its
// source at t; fwd1/bwd1 = forward/backward rows of time t + 1.
__device__ __forceinline__ bool KeepArc(const Arc &arc, float fs, const float *fwd1,
                                        const float *bwd1, const float *scores, int64_t row,
                                        int32_t cols, float cutoff, float *arc_score) {
  float bd = bwd1[arc.dest];
  if (!(__fadd_rn(fwd1[arc.dest], bd) > cutoff)) return false;  // dest state pruned
  float sc = __fadd_rn(arc.score, DenseScore(scores, row, cols, arc.label));
  *arc_score = sc;
  return __fadd_rn(__fadd_rn(fs, sc), bd) > cutoff;
}

// Each warp handles kWordsPerWarp consecutive 32-state words of the (pair, t, state)
// grid; the loads of all its words are issued before any is used.  Most words hold
// no surviving state and cost two loads, a ballot and one 12-byte store.
constexpr int kWordsPerWarp = 4;
constexpr int kCountRounds = 4;
constexpr int kWordsPerCta = kCountRounds * kWordsPerWarp * (kCountThreads / 32);

__global__ void __launch_bounds__(kCountThreads)
CountKept(const FsaInfo *__restrict__ infos, int32_t n, int64_t total_words,
          const Arc *__restrict__ arcs, const int32_t *__restrict__ a_row_splits2,
          const float *__restrict__ scores, int32_t cols, const float *__restrict__ fwd,
          const float *__restrict__ bwd, const float *__restrict__ cutoffs,
          uint32_t *__restrict__ mask, int2 *__restrict__ counts,
          unsigned long long *__restrict__ block_cand, int32_t fsa_base) {
  __shared__ unsigned long long cand_smem;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int32_t i = blockIdx.y + fsa_base;
  const FsaInfo f = infos[i];
  const int64_t pair_words = (int64_t)(f.tk + 1) * f.words;
  if (threadIdx.x == 0) cand_smem = 0;
  __syncthreads();
  const int32_t S = f.num_states;
  const float cutoff = cutoffs[i];
  const float *fgrid = fwd + f.grid_off, *bgrid = bwd + f.grid_off;
  int32_t cand = 0;
  bool any = false;
  for (int round = 0; round < kCountRounds; ++round) {
  const int64_t rel0 = (int64_t)blockIdx.x * kWordsPerCta +
                       ((int64_t)round * (kCountThreads / 32) + warp) * kWordsPerWarp;
  if (rel0 >= pair_words) break;  // warp-uniform
  float fs[kWordsPerWarp], bs[kWordsPerWarp];
  int32_t ts[kWordsPerWarp], ss[kWordsPerWarp];
  // (level, word) of the warp's first word by one 32-bit division (a pair has fewer than
  // 2^31 words), of the following ones by stepping
  int32_t t_run = (int32_t)((uint32_t)rel0 / (uint32_t)f.words);
  int32_t w_run = (int32_t)((uint32_t)rel0 - (uint32_t)t_run * (uint32_t)f.words);
#pragma unroll
  for (int u = 0; u < kWordsPerWarp; ++u) {
    const int64_t rel = rel0 + u;
    const int32_t t = t_run, s = w_run * 32 + lane;
    if (++w_run == f.words) {
      w_run = 0;
      ++t_run;
    }
    ts[u] = t;
    ss[u] = s;
    const bool in = rel < pair_words && s < S;
    fs[u] = in ? fgrid[(int64_t)t * S + s] : -INFINITY;
    bs[u] = in ? bgrid[(int64_t)t * S + s] : -INFINITY;
  }
#pragma unroll
  for (int u = 0; u < kWordsPerWarp; ++u) {
    const int64_t rel = rel0 + u;
    if (rel >= pair_words) break;  // warp-uniform
    const bool keep = __fadd_rn(fs[u], bs[u]) > cutoff;
    const uint32_t m = __ballot_sync(0xffffffffu, keep);
    const int64_t w = f.word_off + rel;
    if (m == 0) {
      if (lane == 0) {
        mask[w] = 0;
        counts[w] = make_int2(0, 0);
      }
      continue;
    }
    any = true;
    int32_t narcs = 0;
    if (keep) {
      const int32_t t = ts[u];
      const int32_t idx01 = f.state_off + ss[u], a0 = a_row_splits2[idx01],
                    a1 = a_row_splits2[idx01 + 1];
      cand += a1 - a0;
      if (t < f.tk) {
        const float *fwd1 = fgrid + (int64_t)(t + 1) * S, *bwd1 = bgrid + (int64_t)(t + 1) * S;
        const int64_t row = (int64_t)f.row0 + t;
        for (int32_t a = a0; a < a1; ++a) {
          float sc;
          narcs += KeepArc(arcs[a], fs[u], fwd1, bwd1, scores, row, cols, cutoff, &sc);
        }
      }
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) narcs += __shfl_xor_sync(0xffffffffu, narcs, d);
    if (lane == 0) {
      mask[w] = m;
      counts[w] = make_int2(__popc(m), narcs);
    }
  }
  }  // rounds
  if (any) {  // warp-uniform
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) cand += __shfl_xor_sync(0xffffffffu, cand, d);
    if (lane == 0 && cand) atomicAdd(&cand_smem, (unsigned long long)cand);
  }
  __syncthreads();
  if (threadIdx.x == 0)
    block_cand[(size_t)(blockIdx.y + fsa_base) * gridDim.x + blockIdx.x] = cand_smem;
}

// totals[0] = kept states, [1] = kept arcs, [2] = sum over kept states of their
// out-degree (the reference's `tot_arcs`, intersect_dense.cu:298,310).
__global__ void Totals(const int2 *__restrict__ bases, int64_t total_words,
                       const unsigned long long *__restrict__ block_cand, int32_t nblocks,
                       long long *__restrict__ totals) {
  __shared__ unsigned long long red[1024];
  unsigned long long c0 = 0, c1 = 0, c2 = 0, c3 = 0;
  int32_t k = threadIdx.x;
  for (; k + 3 * (int32_t)blockDim.x < nblocks; k += 4 * blockDim.x) {
    c0 += block_cand[k];
    c1 += block_cand[k + blockDim.x];
    c2 += block_cand[k + 2 * blockDim.x];
    c3 += block_cand[k + 3 * blockDim.x];
  }
  for (; k < nblocks; k += blockDim.x) c0 += block_cand[k];
  red[threadIdx.x] = c0 + c1 + c2 + c3;
  __syncthreads();
  for (int d = blockDim.x >> 1; d > 0; d >>= 1) {
    if (threadIdx.x < d) red[threadIdx.x] += red[threadIdx.x + d];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    int2 tot = bases[total_words];
    totals[0] = tot.x;
    totals[1] = tot.y;
    totals[2] = (long long)red[0];
    totals[3] = 0;
    totals[4] = 0;
  }
}

// Largest number of kept states in any (pair, t) layer and of kept arcs between two
// layers: totals[3], totals[4].  One thread per layer.
__global__ void LayerMaxima(const FsaInfo *__restrict__ infos, int32_t n, int32_t total_levels,
                            const int2 *__restrict__ bases, long long *__restrict__ totals) {
  const int32_t lv = blockIdx.x * blockDim.x + threadIdx.x;
  int32_t ns = 0, na = 0;
  if (lv < total_levels) {
    int32_t lo = 0, hi = n;
    while (hi - lo > 1) {
      const int32_t mid = (lo + hi) >> 1;
      if (infos[mid].level_off <= lv) lo = mid; else hi = mid;
    }
    const FsaInfo f = infos[lo];
    if (f.words > 0) {
      const int64_t w0 = f.word_off + (int64_t)(lv - f.level_off) * f.words;
      const int2 a = bases[w0], b = bases[w0 + f.words];
      ns = b.x - a.x;
      na = b.y - a.y;
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    ns = max(ns, __shfl_xor_sync(0xffffffffu, ns, d));
    na = max(na, __shfl_xor_sync(0xffffffffu, na, d));
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMax(reinterpret_cast<long long *>(totals + 3), (long long)ns);
    atomicMax(reinterpret_cast<long long *>(totals + 4), (long long)na);
  }
}

// One warp writes the states of word `rel` of pair i and the arcs leaving them.
__device__ __forceinline__ void
EmitWord(const FsaInfo &f, int32_t i, int32_t n, int64_t rel, float cutoff, int lane,
         const Arc *__restrict__ arcs, const int32_t *__restrict__ a_row_splits2,
         const float *__restrict__ scores, int32_t cols, const float *__restrict__ fwd,
         const float *__restrict__ bwd, const uint32_t *__restrict__ mask,
         const int2 *__restrict__ bases, const k2b200_lattice_out &out) {
  const int64_t w = f.word_off + rel;
  const int32_t t = (int32_t)((uint32_t)rel / (uint32_t)f.words),
                wi = (int32_t)((uint32_t)rel - (uint32_t)t * (uint32_t)f.words), s = wi * 32 + lane;
  const uint32_t m = mask[w];
  if (m == 0 && wi != 0) return;  // nothing kept in this word and no layer boundary to record
  const int32_t S = f.num_states;
  const int2 base = bases[w];
  const int32_t fsa_first_state = bases[f.word_off].x;

  if (lane == 0) {
    if (wi == 0) {
      if (out.level_splits) out.level_splits[f.level_off + t] = base.x;
      if (t == 0) {
        out.row_splits1[i] = base.x;
        if (out.level_offsets) out.level_offsets[i] = f.level_off;
      }
    }
  }
  const bool keep = (m >> lane) & 1u;
  const float *fwd0 = fwd + f.grid_off + (int64_t)t * S, *bwd0 = bwd + f.grid_off + (int64_t)t * S;
  const float *fwd1 = fwd0 + S, *bwd1 = bwd0 + S;
  const int64_t row = (int64_t)f.row0 + t;
  int32_t a0 = 0, a1 = 0, narcs = 0;
  float fs = 0;
  if (keep) {
    const int32_t idx01 = f.state_off + s;
    a0 = a_row_splits2[idx01];
    a1 = a_row_splits2[idx01 + 1];
    fs = fwd0[s];
    if (t < f.tk) {
      for (int32_t a = a0; a < a1; ++a) {
        float sc;
        narcs += KeepArc(arcs[a], fs, fwd1, bwd1, scores, row, cols, cutoff, &sc);
      }
    }
  }
  // exclusive prefix of narcs across the warp
  int32_t inc = narcs;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int32_t o = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += o;
  }
  if (!keep) return;
  const int32_t state_id = base.x + __popc(m & ((1u << lane) - 1u));
  int32_t pos = base.y + inc - narcs;
  out.row_splits2[state_id] = pos;
  out.row_ids1[state_id] = i;
  if (t >= f.tk || narcs == 0) return;
  const int64_t next_word0 = f.word_off + (int64_t)(t + 1) * f.words;
  Arc *out_arcs = reinterpret_cast<Arc *>(out.arcs);
  for (int32_t a = a0; a < a1; ++a) {
    Arc arc = arcs[a];
    float sc;
    if (!KeepArc(arc, fs, fwd1, bwd1, scores, row, cols, cutoff, &sc)) continue;
    const int64_t wd = next_word0 + (arc.dest >> 5);
    const int32_t dest_id = bases[wd].x + __popc(mask[wd] & ((1u << (arc.dest & 31)) - 1u));
    Arc o;
    o.src = state_id - fsa_first_state;
    o.dest = dest_id - fsa_first_state;
    o.label = arc.label;
    o.score = sc;
    out_arcs[pos] = o;
    out.row_ids2[pos] = state_id;
    if (out.arc_map_a) out.arc_map_a[pos] = a + f.arc_out_off;
    if (out.arc_map_b) out.arc_map_b[pos] = (int32_t)(row * cols + (arc.label + 1));
    ++pos;
  }
}


constexpr int kEmitWordsPerWarp = 16;
constexpr int kEmitWordsPerCta = kEmitWordsPerWarp * 8;

// Each warp walks kEmitWordsPerWarp consecutive words (few, fat CTAs: most words
// hold nothing and are skipped after one load).
__global__ void __launch_bounds__(256)
EmitLattice(const FsaInfo *__restrict__ infos, int32_t n, int64_t total_words,
            const Arc *__restrict__ arcs, const int32_t *__restrict__ a_row_splits2,
            const float *__restrict__ scores, int32_t cols, const float *__restrict__ fwd,
            const float *__restrict__ bwd, const float *__restrict__ cutoffs,
            const uint32_t *__restrict__ mask, const int2 *__restrict__ bases,
            k2b200_lattice_out out, int32_t fsa_base) {
  const int lane = threadIdx.x & 31;
  const int32_t i = blockIdx.y + fsa_base;
  const FsaInfo f = infos[i];
  const float cutoff = cutoffs[i];
  const int64_t pair_words = (int64_t)(f.tk + 1) * f.words;
  const int64_t rel0 =
      ((int64_t)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5)) * kEmitWordsPerWarp;
  for (int u = 0; u < kEmitWordsPerWarp; ++u) {
    const int64_t rel = rel0 + u;
    if (rel >= pair_words) return;
    EmitWord(f, i, n, rel, cutoff, lane, arcs, a_row_splits2, scores, cols, fwd, bwd, mask, bases,
             out);
  }
}

// Entries EmitLattice cannot reach: the closing element of every splits array, and
// pairs whose graph is empty (they own no word).
__global__ void EmitTails(const FsaInfo *__restrict__ infos, int32_t n, int64_t total_words,
                          int32_t total_levels, const int2 *__restrict__ bases,
                          k2b200_lattice_out out) {
  int32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > n) return;
  if (i == n) {
    int2 tot = bases[total_words];
    out.row_splits1[n] = tot.x;
    out.row_splits2[tot.x] = tot.y;
    if (out.level_offsets) out.level_offsets[n] = total_levels;
    if (out.level_splits) out.level_splits[total_levels] = tot.x;
    return;
  }
  FsaInfo f = infos[i];
  if (f.num_states != 0) return;
  int32_t first = bases[f.word_off].x;  // == first state of the next non-empty pair
  out.row_splits1[i] = first;
  if (out.level_offsets) out.level_offsets[i] = f.level_off;
  if (out.level_splits)
    for (int32_t t = 0; t <= f.tk; ++t) out.level_splits[f.level_off + t] = first;
}

int32_t RunViterbi(const Layout &L, const k2b200_intersect_args *a, char *ws, cudaStream_t stream,
                   bool plan_ready) {
  const FsaInfo *d_infos = reinterpret_cast<const FsaInfo *>(ws + L.off_infos);
  float *fwd = reinterpret_cast<float *>(ws + L.off_fwd),
        *bwd = reinterpret_cast<float *>(ws + L.off_bwd);
  if (L.max_states == 0) return kOk;
  int32_t mode = a->viterbi_mode;
  if (mode == 0)
    mode = RegisterViterbiFits(L, a) ? 3 : L.lane_plan ? 4 : (PersistentViterbiFits(L, a) ? 2 : 1);
  if (mode == 3) {
    K2B_REQUIRE(RegisterViterbiFits(L, a),
                "viterbi_mode=3 needs a_max_degree <= 4 and at most 1024 states per graph");
    NotePhaseKernel(kPhaseViterbi, "RegisterViterbi");
    return LaunchRegisterViterbi(L, a, d_infos, fwd, bwd, stream);
  }
  if (mode == 4) {
    K2B_REQUIRE(L.lane_plan, "viterbi_mode=4 needs graphs of at most %d states that fit in "
                "shared memory, with some state of more than four arcs", kLaneThreads);
    if (!plan_ready) K2B_FORWARD(LaunchPlanLanes(L, a, ws, stream));
    NotePhaseKernel(kPhaseViterbi, "LanesViterbi");
    const int32_t *unfit = reinterpret_cast<const int32_t *>(ws + L.off_unfit);
    K2B_FORWARD(LaunchLanesViterbi(L, a, d_infos, fwd, bwd,
                                   reinterpret_cast<const int32_t *>(ws + L.off_plan), unfit,
                                   stream));
    return LaunchPersistentViterbi(L, a, d_infos, fwd, bwd, stream, unfit);
  }
  if (mode == 2) {
    K2B_REQUIRE(PersistentViterbiFits(L, a),
                "viterbi_mode=2 requested but a graph does not fit in shared memory");
    NotePhaseKernel(kPhaseViterbi, "PersistentViterbi");
    return LaunchPersistentViterbi(L, a, d_infos, fwd, bwd, stream);
  }
  if (mode == 5) K2B_REQUIRE(L.shared_vit, "viterbi_mode=5 needs one graph shared by all sequences "
                             "(a_shared) and at least two of them");
  if (L.shared_vit) {
    NotePhaseKernel(kPhaseViterbi, "SharedViterbiStep");
    return LaunchSharedViterbi(L, a, ws + L.off_shared_vit, d_infos, fwd, bwd, stream);
  }
  const Arc *arcs = reinterpret_cast<const Arc *>(a->a_arcs);
  NotePhaseKernel(kPhaseViterbi, "ViterbiStep");
  dim3 init_grid(CeilDiv(L.max_states, 256), a->num_fsas);
  { ViterbiInit<<<init_grid, 256, 0, stream>>>(d_infos, fwd, bwd); NoteLaunch(); }
  // lanes per state from the mean degree of the batch
  int32_t mean_deg = a->num_states > 0 ? (a->num_arcs + a->num_states - 1) / a->num_states : 1;
  int32_t lanes_log2 = 0;
  while ((1 << lanes_log2) < mean_deg && lanes_log2 < 5) ++lanes_log2;
  dim3 grid(CeilDiv((int64_t)L.max_states << lanes_log2, 256), a->num_fsas, 2);
  for (int32_t t = 1; t <= L.max_tk; ++t) {
    { ViterbiStep<<<grid, 256, 0, stream>>>(d_infos, t, arcs, a->a_row_splits2, a->a_in_splits,
                                          a->a_in_arcs, a->scores, a->cols, fwd, bwd,
                                          lanes_log2); NoteLaunch(); }
  }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}


// Sizes only, for callers that never build the lattice: the number of surviving
// (frame, state) pairs and of arcs leaving them (the two totals the beam reduction
// looks at), added into totals[0] and totals[2].  grid = (tiles, pairs).
__global__ void __launch_bounds__(256)
CountStates(const FsaInfo *__restrict__ infos, const int32_t *__restrict__ a_row_splits2,
            const float *__restrict__ fwd, const float *__restrict__ bwd,
            const float *__restrict__ cutoffs, unsigned long long *__restrict__ totals,
            int32_t fsa_base) {
  const int32_t i = blockIdx.y + fsa_base;
  const FsaInfo f = infos[i];
  const int64_t elems = (int64_t)(f.tk + 1) * f.num_states;
  const float cutoff = cutoffs[i];
  const float *fg = fwd + f.grid_off, *bg = bwd + f.grid_off;
  const int32_t *splits = a_row_splits2 + f.state_off;
  uint32_t states = 0, cand = 0;
  // state of element k, kept up to date without a division per element
  const int32_t S = f.num_states;
  const int64_t k0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x,
                stride = (int64_t)gridDim.x * blockDim.x;
  int32_t s = S > 0 ? (int32_t)(k0 % S) : 0;
  const int32_t s_step = S > 0 ? (int32_t)(stride % S) : 0;
  for (int64_t k = k0; k < elems; k += stride) {
    if (__fadd_rn(fg[k], bg[k]) > cutoff) {
      ++states;
      cand += splits[s + 1] - splits[s];
    }
    s += s_step;
    if (s >= S) s -= S;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    states += __shfl_xor_sync(0xffffffffu, states, d);
    cand += __shfl_xor_sync(0xffffffffu, cand, d);
  }
  // one pair of atomics per CTA: all of them hit the same two words
  __shared__ uint32_t cta_states, cta_cand;
  if (threadIdx.x == 0) cta_states = cta_cand = 0;
  __syncthreads();
  if ((threadIdx.x & 31) == 0 && (states | cand)) {
    atomicAdd(&cta_states, states);
    atomicAdd(&cta_cand, cand);
  }
  __syncthreads();
  if (threadIdx.x == 0 && (cta_states | cta_cand)) {
    atomicAdd(&totals[0], (unsigned long long)cta_states);
    atomicAdd(&totals[2], (unsigned long long)cta_cand);
  }
}

int32_t LaunchCutoffs(const Layout &L, const k2b200_intersect_args *a, char *ws, float beam,
                      cudaStream_t stream) {
  { Cutoffs<<<CeilDiv(a->num_fsas, 128), 128, 0, stream>>>(
      reinterpret_cast<const FsaInfo *>(ws + L.off_infos), a->num_fsas,
      reinterpret_cast<const float *>(ws + L.off_fwd),
      reinterpret_cast<const float *>(ws + L.off_bwd), beam,
      reinterpret_cast<float *>(ws + L.off_cutoffs)); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

// Keep masks, counts and numbering for the current beam, shrinking the beam as the
// reference does (intersect_dense.cu:300-320 and :854-862) until the lattice fits
// max_states / max_arcs.  One host synchronisation per iteration.  h_totals:
// states, arcs, candidate arcs, largest layer in states and in arcs.
// Counts the states and arcs that the current cutoffs keep into totals[0] / totals[2]
// (the sizes the lattice would have), without numbering anything.
int32_t LaunchSizeCount(const Layout &L, const k2b200_intersect_args *args, char *ws,
                        cudaStream_t stream) {
  const FsaInfo *d_infos = reinterpret_cast<const FsaInfo *>(ws + L.off_infos);
  const float *cutoffs = reinterpret_cast<const float *>(ws + L.off_cutoffs);
  const float *fwd = reinterpret_cast<const float *>(ws + L.off_fwd),
              *bwd = reinterpret_cast<const float *>(ws + L.off_bwd);
  long long *totals = reinterpret_cast<long long *>(ws + L.off_totals);
  K2B_CUDA_OK(cudaMemsetAsync(totals, 0, 5 * sizeof(long long), stream));
  if (L.grid_elems > 0)
    for (int32_t first = 0; first < args->num_fsas; first += 65535) {
      int64_t max_elems = (int64_t)(L.max_tk + 1) * L.max_states;
      dim3 grid((unsigned)std::min<int64_t>(CeilDiv(max_elems, 256 * 16), 64),
                std::min(args->num_fsas - first, 65535));
      { CountStates<<<grid, 256, 0, stream>>>(
          d_infos, args->a_row_splits2, fwd, bwd, cutoffs,
          reinterpret_cast<unsigned long long *>(totals), first); NoteLaunch(); }
    }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

// The reference's retry rule (intersect_dense.cu:300-320 and :854-862): when the
// lattice would exceed max_states or max_arcs the beam shrinks by
// sqrt(limit / total), clamped to [0.25, 0.75] of itself.  Returns false when the
// sizes are within the limits.
bool ReduceBeam(const k2b200_intersect_args *args, const long long *h_totals, float *beam) {
  long long limit = 0, total = 0;
  if (h_totals[0] > args->max_states) {
    limit = args->max_states;
    total = h_totals[0];
  } else if (h_totals[2] > args->max_arcs) {
    limit = args->max_arcs;
    total = h_totals[2];
  } else {
    return false;
  }
  float cur = *beam, next = cur * sqrt(limit * 1.0 / total);
  if (next < cur * 0.25) next = cur * 0.25;
  if (next > cur * 0.75) next = cur * 0.75;
  *beam = next;
  return true;
}

int32_t PruneLoop(const Layout &L, const k2b200_intersect_args *args, char *ws,
                  cudaStream_t stream, float *beam_io, long long *h_totals, bool sizes_only) {
  const FsaInfo *d_infos = reinterpret_cast<const FsaInfo *>(ws + L.off_infos);
  float *cutoffs = reinterpret_cast<float *>(ws + L.off_cutoffs);
  float *fwd = reinterpret_cast<float *>(ws + L.off_fwd),
        *bwd = reinterpret_cast<float *>(ws + L.off_bwd);
  uint32_t *mask = reinterpret_cast<uint32_t *>(ws + L.off_mask);
  int2 *counts = reinterpret_cast<int2 *>(ws + L.off_counts);
  int2 *scan_tmp = reinterpret_cast<int2 *>(ws + L.off_scan_tmp);
  unsigned long long *block_cand = reinterpret_cast<unsigned long long *>(ws + L.off_block_cand);
  long long *totals = reinterpret_cast<long long *>(ws + L.off_totals);
  const Arc *arcs = reinterpret_cast<const Arc *>(args->a_arcs);
  float beam = *beam_io;
  PhaseTimer prune_timer(kPhasePrune, stream);

  for (int iter = 0;; ++iter) {
    { Cutoffs<<<CeilDiv(args->num_fsas, 128), 128, 0, stream>>>(d_infos, args->num_fsas, fwd, bwd,
                                                              beam, cutoffs); NoteLaunch(); }
    if (sizes_only) {
      K2B_FORWARD(LaunchSizeCount(L, args, ws, stream));
    } else {
      if (L.total_words > 0)
        for (int32_t first = 0; first < args->num_fsas; first += 65535) {
          dim3 grid(L.tiles_per_pair, std::min(args->num_fsas - first, 65535));
          { CountKept<<<grid, kCountThreads, 0, stream>>>(
              d_infos, args->num_fsas, L.total_words, arcs, args->a_row_splits2, args->scores,
              args->cols, fwd, bwd, cutoffs, mask, counts, block_cand, first); NoteLaunch(); }
        }
      K2B_FORWARD(ExclusiveSum2(counts, counts, L.total_words, scan_tmp, stream));
      { Totals<<<1, 1024, 0, stream>>>(counts, L.total_words, block_cand,
                                    L.total_words > 0 ? L.count_blocks : 0, totals); NoteLaunch(); }
      if (L.total_words > 0)
        { LayerMaxima<<<CeilDiv(L.total_levels, 256), 256, 0, stream>>>(
            d_infos, args->num_fsas, (int32_t)L.total_levels, counts, totals); NoteLaunch(); }
    }
    K2B_CUDA_OK(cudaGetLastError());
    K2B_CUDA_OK(cudaMemcpyAsync(h_totals, totals, 5 * sizeof(long long), cudaMemcpyDeviceToHost,
                                stream));
    K2B_CUDA_OK(cudaStreamSynchronize(stream));
    if (!ReduceBeam(args, h_totals, &beam)) break;
    if (iter > 200) {
      SetError("output beam reduction did not converge");
      return kInvalidArgument;
    }
  }
  *beam_io = beam;
  return kOk;
}

}  // namespace k2b

using namespace k2b;

extern "C" {

int32_t k2b200_intersect_dense_workspace_bytes(const k2b200_intersect_args *args,
                                               size_t *bytes, int64_t *total_levels) {
  Layout L;
  K2B_FORWARD(MakeLayout(args, &L));
  if (bytes) *bytes = L.total_bytes;
  if (total_levels) *total_levels = L.total_levels;
  return kOk;
}

int32_t k2b200_intersect_dense_prune(const k2b200_intersect_args *args, void *workspace,
                                     size_t workspace_bytes, void *stream_v,
                                     int32_t *num_states_out, int32_t *num_arcs_out,
                                     float *beam_used, int32_t *max_layer_states,
                                     int32_t *max_layer_arcs) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  Layout L;
  K2B_FORWARD(MakeLayout(args, &L));
  if (workspace == nullptr || workspace_bytes < L.total_bytes) {
    SetError("workspace of %zu bytes is smaller than the %zu required", workspace_bytes,
             L.total_bytes);
    return kWorkspaceTooSmall;
  }
  K2B_REQUIRE(args->a_row_splits1 && args->a_row_splits2 && args->a_arcs && args->a_in_splits &&
                  args->a_in_arcs && args->scores,
              "NULL device pointer in args");
  K2B_REQUIRE(num_states_out && num_arcs_out, "NULL output pointer");
  char *ws = reinterpret_cast<char *>(workspace);
  K2B_CUDA_OK(cudaMemcpyAsync(ws + L.off_infos, L.infos.data(), sizeof(FsaInfo) * args->num_fsas,
                              cudaMemcpyHostToDevice, stream));
  {
    PhaseTimer timer(kPhaseViterbi, stream);
    K2B_FORWARD(RunViterbi(L, args, ws, stream));
  }
  float beam = args->output_beam;
  long long h_totals[5] = {0, 0, 0, 0, 0};
  K2B_FORWARD(PruneLoop(L, args, ws, stream, &beam, h_totals));
  *num_states_out = (int32_t)h_totals[0];
  *num_arcs_out = (int32_t)h_totals[1];
  if (beam_used) *beam_used = beam;
  if (max_layer_states) *max_layer_states = (int32_t)h_totals[3];
  if (max_layer_arcs) *max_layer_arcs = (int32_t)h_totals[4];
  return kOk;
}

int32_t k2b200_intersect_dense_emit(const k2b200_intersect_args *args, void *workspace,
                                    size_t workspace_bytes, void *stream_v,
                                    const k2b200_lattice_out *out) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  Layout L;
  K2B_FORWARD(MakeLayout(args, &L));
  if (workspace == nullptr || workspace_bytes < L.total_bytes) {
    SetError("workspace of %zu bytes is smaller than the %zu required", workspace_bytes,
             L.total_bytes);
    return kWorkspaceTooSmall;
  }
  K2B_REQUIRE(out && out->row_splits1 && out->row_ids1 && out->row_splits2 && out->row_ids2 &&
                  out->arcs,
              "NULL lattice output pointer");
  char *ws = reinterpret_cast<char *>(workspace);
  const FsaInfo *d_infos = reinterpret_cast<const FsaInfo *>(ws + L.off_infos);
  PhaseTimer timer(kPhaseEmit, stream);
  { EmitTails<<<CeilDiv(args->num_fsas + 1, 128), 128, 0, stream>>>(
      d_infos, args->num_fsas, L.total_words, (int32_t)L.total_levels,
      reinterpret_cast<const int2 *>(ws + L.off_counts), *out); NoteLaunch(); }
  if (L.total_words > 0)
    for (int32_t first = 0; first < args->num_fsas; first += 65535) {
      dim3 grid(L.emit_tiles_per_pair, std::min(args->num_fsas - first, 65535));
      { EmitLattice<<<grid, 256, 0, stream>>>(
          d_infos, args->num_fsas, L.total_words, reinterpret_cast<const Arc *>(args->a_arcs),
          args->a_row_splits2, args->scores, args->cols,
          reinterpret_cast<const float *>(ws + L.off_fwd),
          reinterpret_cast<const float *>(ws + L.off_bwd),
          reinterpret_cast<const float *>(ws + L.off_cutoffs),
          reinterpret_cast<const uint32_t *>(ws + L.off_mask),
          reinterpret_cast<const int2 *>(ws + L.off_counts), *out, first); NoteLaunch(); }
    }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

}  // extern "C"

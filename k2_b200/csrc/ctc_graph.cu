// CTC graphs of a batch of transcripts, built on the GPU.
//
// Same graphs, arc for arc, as k2::CtcGraphs (k2/csrc/fsa_algo.cu:577-730): a
// transcript of L symbols gives 2L+2 states - state 2k the blank state in front of
// symbol k (2L the trailing one), 2k+1 the state of symbol k, 2L+1 the final state.
// The reference launches one lambda per state and per arc around two ExclusiveSums;
// here one kernel sizes the per-symbol arc blocks, one exclusive sum places them and
// one kernel writes arcs, aux_labels and both row_splits.
#include "../../include/k2b200.h"
#include "common.cuh"

namespace k2b {

// Arcs contributed by symbol position k: blank state (2) + symbol state (2 or 3).
__global__ void CtcCountArcs(const int32_t *__restrict__ sym_row_splits,
                             const int32_t *__restrict__ sym_row_ids,
                             const int32_t *__restrict__ symbols, int32_t tot,
                             int32_t modified, int32_t *__restrict__ per_sym) {
  int32_t k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= tot) return;
  const int32_t i = sym_row_ids[k];
  const bool last = k + 1 == sym_row_splits[i + 1];
  const int32_t next = last ? -1 : symbols[k + 1];
  per_sym[k] = 4 + ((modified || symbols[k] != next) ? 1 : 0);
}

__global__ void CtcWriteArcs(const int32_t *__restrict__ sym_row_splits,
                             const int32_t *__restrict__ sym_row_ids,
                             const int32_t *__restrict__ symbols, int32_t num_seqs, int32_t tot,
                             int32_t modified, const int32_t *__restrict__ sym_arc_off,
                             int32_t *__restrict__ row_splits1, int32_t *__restrict__ row_splits2,
                             Arc *__restrict__ arcs, int32_t *__restrict__ aux) {
  int32_t k = blockIdx.x * blockDim.x + threadIdx.x;
  auto put = [&](int32_t pos, int32_t src, int32_t dest, int32_t label, int32_t a) {
    Arc arc;
    arc.src = src;
    arc.dest = dest;
    arc.label = label;
    arc.score = 0.0f;
    arcs[pos] = arc;
    aux[pos] = a;
  };
  if (k < tot) {
    const int32_t i = sym_row_ids[k], s0 = sym_row_splits[i];
    const int32_t pos_in = k - s0;                  // position in its transcript
    const int32_t state0 = 2 * s0 + 2 * i;          // first state (idx01) of FSA i
    const int32_t blk = sym_arc_off[k] + 2 * i;     // 2 tail arcs per earlier FSA
    const bool last = k + 1 == sym_row_splits[i + 1];
    const int32_t sym = symbols[k], next = last ? -1 : symbols[k + 1];
    const int32_t sb = 2 * pos_in, ss = sb + 1;
    put(blk + 0, sb, sb, 0, 0);
    put(blk + 1, sb, ss, sym, sym);
    put(blk + 2, ss, ss + 1, 0, 0);
    put(blk + 3, ss, ss, sym, 0);
    if (modified || sym != next) put(blk + 4, ss, ss + 2, next, next);
    row_splits2[state0 + sb] = blk;
    row_splits2[state0 + ss] = blk + 2;
  }
  if (k < num_seqs) {  // the trailing blank state and the final state of FSA k
    const int32_t s0 = sym_row_splits[k], s1 = sym_row_splits[k + 1], L = s1 - s0;
    const int32_t state0 = 2 * s0 + 2 * k;
    const int32_t tail = sym_arc_off[s1] + 2 * k;   // sym_arc_off has tot + 1 entries
    put(tail, 2 * L, 2 * L, 0, 0);
    put(tail + 1, 2 * L, 2 * L + 1, -1, -1);
    row_splits1[k] = state0;
    row_splits2[state0 + 2 * L] = tail;
    row_splits2[state0 + 2 * L + 1] = tail + 2;
    if (k == num_seqs - 1) {
      row_splits1[num_seqs] = state0 + 2 * L + 2;
      row_splits2[state0 + 2 * L + 2] = tail + 2;
    }
  }
}

}  // namespace k2b

using namespace k2b;

extern "C" {

size_t k2b200_ctc_graph_tmp_bytes(int32_t num_symbols) {
  return AlignUp(sizeof(int32_t) * ((size_t)num_symbols + 1)) +
         AlignUp(sizeof(int32_t) * ((size_t)num_symbols + 1)) +
         AlignUp(sizeof(int32_t) * ScanTmpInts(num_symbols));
}

int32_t k2b200_ctc_graph(const int32_t *sym_row_splits, const int32_t *symbols, int32_t num_seqs,
                         int32_t num_symbols, int32_t modified, int32_t *row_splits1,
                         int32_t *row_splits2, void *arcs, int32_t *aux_labels, void *tmp,
                         void *stream_v) {
  K2B_REQUIRE(num_seqs > 0 && num_symbols >= 0, "need at least one transcript");
  K2B_REQUIRE(sym_row_splits && row_splits1 && row_splits2 && arcs && aux_labels && tmp,
              "NULL pointer");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  char *p = reinterpret_cast<char *>(tmp);
  int32_t *sym_row_ids = reinterpret_cast<int32_t *>(p);
  p += AlignUp(sizeof(int32_t) * ((size_t)num_symbols + 1));
  int32_t *per_sym = reinterpret_cast<int32_t *>(p);
  p += AlignUp(sizeof(int32_t) * ((size_t)num_symbols + 1));
  int32_t *scan_tmp = reinterpret_cast<int32_t *>(p);
  K2B_FORWARD(RowSplitsToRowIds(sym_row_splits, num_seqs, sym_row_ids, num_symbols, stream));
  if (num_symbols > 0)
    { CtcCountArcs<<<CeilDiv(num_symbols, 256), 256, 0, stream>>>(
        sym_row_splits, sym_row_ids, symbols, num_symbols, modified, per_sym); NoteLaunch(); }
  K2B_FORWARD(ExclusiveSum(per_sym, per_sym, num_symbols, scan_tmp, stream));
  int32_t n = num_symbols > num_seqs ? num_symbols : num_seqs;
  { CtcWriteArcs<<<CeilDiv(n, 256), 256, 0, stream>>>(
      sym_row_splits, sym_row_ids, symbols, num_seqs, num_symbols, modified, per_sym, row_splits1,
      row_splits2, reinterpret_cast<Arc *>(arcs), aux_labels); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

}  // extern "C"

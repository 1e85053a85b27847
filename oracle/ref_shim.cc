// TEST INFRASTRUCTURE ONLY - never linked into or loaded by the product path.
//
// C-ABI shim over the *unmodified* k2 reference C++ sources, which are compiled
// for CPU where they lie in the reference checkout by oracle/Makefile (no
// reference source is copied into this repository).  The shim lets the tests
// and the CPU-baseline leg of bench.py call the reference's own
//   IntersectDense              k2/csrc/intersect_dense.cu:1045-1073
//   GetForwardScores            k2/csrc/fsa_utils.cu:1124-1278
//   GetBackwardScores           k2/csrc/fsa_utils.cu:1345-1454
//   GetTotScores / GetArcPost   k2/csrc/fsa_utils.cu:1809-1901
//   ShortestPath                k2/csrc/fsa_algo.cu:869-1144
//   CtcGraphs                   k2/csrc/fsa_algo.cu:577-730
//   GetFsaVecBasicProperties    k2/csrc/fsa.cu:54-217
// through plain pointers (ctypes).  The only reference symbol the sources leave
// undefined in a torch-free CPU build is k2::GetCpuContext(); a malloc-backed
// Context is supplied here for it.
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "k2/csrc/array.h"
#include "k2/csrc/array_ops.h"
#include "k2/csrc/context.h"
#include "k2/csrc/fsa.h"
#include "k2/csrc/fsa_algo.h"
#include "k2/csrc/fsa_utils.h"
#include "k2/csrc/intersect_dense_pruned.h"
#include "k2/csrc/ragged.h"
#include "k2/csrc/ragged_ops.h"

namespace k2 {

class ShimCpuContext : public Context {
 public:
  DeviceType GetDeviceType() const override { return kCpu; }
  void *Allocate(size_t bytes, void **deleter_context) override {
    if (deleter_context != nullptr) *deleter_context = nullptr;
    if (bytes == 0) return nullptr;
    void *p = nullptr;
    if (posix_memalign(&p, 64, bytes) != 0) throw std::bad_alloc();
    return p;
  }
  void Deallocate(void *data, void * /*deleter_context*/) override {
    free(data);
  }
  bool IsCompatible(const Context &other) const override {
    return other.GetDeviceType() == kCpu;
  }
  void CopyDataTo(size_t num_bytes, const void *src, ContextPtr dst_context,
                  void *dst) override {
    (void)dst_context;
    if (num_bytes) memcpy(dst, src, num_bytes);
  }
};

ContextPtr GetCpuContext() {
  static ContextPtr ctx = std::make_shared<ShimCpuContext>();
  return ctx;
}

}  // namespace k2

namespace {

thread_local std::string g_last_error;

template <typename T>
k2::Array1<T> FromHost(const T *data, int32_t n) {
  k2::Array1<T> a(k2::GetCpuContext(), n);
  if (n > 0) memcpy(a.Data(), data, sizeof(T) * (size_t)n);
  return a;
}

struct FsaVecHandle {
  k2::FsaVec fsas;
  k2::Array1<int32_t> aux;  // optional side output (ctc_graphs aux_labels)
  k2::Array1<int32_t> arc_map_a, arc_map_b;
};

}  // namespace

#define KREF_TRY try {
#define KREF_CATCH(ret)                 \
  }                                     \
  catch (const std::exception &e) {     \
    g_last_error = e.what();            \
    return ret;                         \
  }                                     \
  catch (...) {                         \
    g_last_error = "unknown exception"; \
    return ret;                         \
  }

template <typename T>
static k2::Array1<T> Narrow(const double *src, int32_t n) {
  k2::Array1<T> a(k2::GetCpuContext(), n);
  for (int32_t i = 0; i < n; ++i) a.Data()[i] = (T)src[i];
  return a;
}

template <typename T>
static void BackpropScoresT(k2::FsaVec &fsas, bool forward, bool log_semiring,
                            const double *scores, const int32_t *entering_arcs,
                            const double *deriv_in, double *arc_deriv) {
  int32_t ns = fsas.TotSize(1), na = fsas.NumElements();
  k2::Ragged<int32_t> state_batches = k2::GetStateBatches(fsas, true);
  k2::Array1<T> sc = Narrow<T>(scores, ns), din = Narrow<T>(deriv_in, ns);
  k2::Array1<T> out;
  if (forward) {
    k2::Ragged<int32_t> leaving = k2::GetLeavingArcIndexBatches(fsas, state_batches);
    k2::Array1<int32_t> ea;
    if (!log_semiring) ea = FromHost(entering_arcs, ns);
    out = k2::BackpropGetForwardScores<T>(fsas, state_batches, leaving, log_semiring,
                                          log_semiring ? nullptr : &ea, sc, din);
  } else {
    k2::Array1<int32_t> dest_states = k2::GetDestStates(fsas, true);
    k2::Ragged<int32_t> incoming = k2::GetIncomingArcs(fsas, dest_states);
    k2::Ragged<int32_t> entering =
        k2::GetEnteringArcIndexBatches(fsas, incoming, state_batches);
    out = k2::BackpropGetBackwardScores<T>(fsas, state_batches, entering, log_semiring, sc,
                                           din);
  }
  for (int32_t i = 0; i < na; ++i) arc_deriv[i] = out.Data()[i];
}

extern "C" {

const char *kref_last_error() { return g_last_error.c_str(); }

void *kref_fsavec_create(const int32_t *row_splits1, int32_t num_fsas,
                         const int32_t *row_splits2, int32_t num_states,
                         const void *arcs, int32_t num_arcs) {
  KREF_TRY
  k2::Array1<int32_t> rs1 = FromHost(row_splits1, num_fsas + 1),
                      rs2 = FromHost(row_splits2, num_states + 1);
  k2::Array1<k2::Arc> values =
      FromHost(reinterpret_cast<const k2::Arc *>(arcs), num_arcs);
  k2::RaggedShape shape =
      k2::RaggedShape3(&rs1, nullptr, num_states, &rs2, nullptr, num_arcs);
  auto *h = new FsaVecHandle;
  h->fsas = k2::FsaVec(shape, values);
  return h;
  KREF_CATCH(nullptr)
}

void kref_fsavec_free(void *handle) {
  delete reinterpret_cast<FsaVecHandle *>(handle);
}

void kref_fsavec_dims(void *handle, int32_t *num_fsas, int32_t *num_states,
                      int32_t *num_arcs) {
  auto *h = reinterpret_cast<FsaVecHandle *>(handle);
  *num_fsas = h->fsas.Dim0();
  *num_states = h->fsas.TotSize(1);
  *num_arcs = h->fsas.TotSize(2);
}

// Copies row_splits1 [num_fsas+1], row_splits2 [num_states+1], arcs
// [num_arcs*16 bytes] and the optional per-arc int32 side arrays (each may be
// NULL) out of the handle.
void kref_fsavec_copy(void *handle, int32_t *row_splits1, int32_t *row_splits2,
                      void *arcs, int32_t *aux, int32_t *arc_map_a,
                      int32_t *arc_map_b) {
  auto *h = reinterpret_cast<FsaVecHandle *>(handle);
  k2::FsaVec &f = h->fsas;
  memcpy(row_splits1, f.RowSplits(1).Data(), sizeof(int32_t) * (f.Dim0() + 1));
  memcpy(row_splits2, f.RowSplits(2).Data(),
         sizeof(int32_t) * (f.TotSize(1) + 1));
  if (f.NumElements() > 0) {
    memcpy(arcs, f.values.Data(), sizeof(k2::Arc) * (size_t)f.NumElements());
    size_t nb = sizeof(int32_t) * (size_t)f.NumElements();
    if (aux && h->aux.Dim() == f.NumElements()) memcpy(aux, h->aux.Data(), nb);
    if (arc_map_a && h->arc_map_a.Dim() == f.NumElements())
      memcpy(arc_map_a, h->arc_map_a.Data(), nb);
    if (arc_map_b && h->arc_map_b.Dim() == f.NumElements())
      memcpy(arc_map_b, h->arc_map_b.Data(), nb);
  }
}

void *kref_ctc_graphs(const int32_t *sym_row_splits, int32_t num_seqs,
                      const int32_t *symbols, int32_t modified) {
  KREF_TRY
  k2::Array1<int32_t> rs = FromHost(sym_row_splits, num_seqs + 1);
  int32_t n = sym_row_splits[num_seqs];
  k2::Array1<int32_t> vals = FromHost(symbols, n);
  k2::Ragged<int32_t> syms(k2::RaggedShape2(&rs, nullptr, n), vals);
  auto *h = new FsaVecHandle;
  h->fsas = k2::CtcGraphs(syms, modified != 0, &h->aux);
  return h;
  KREF_CATCH(nullptr)
}

// k2::CtcTopo (k2/csrc/fsa_algo.cu:732-817) as an FsaVec of one FSA, with aux labels.
void *kref_ctc_topo(int32_t max_token, int32_t modified) {
  KREF_TRY
  auto *h = new FsaVecHandle;
  k2::Fsa topo = k2::CtcTopo(k2::GetCpuContext(), max_token, modified != 0, &h->aux);
  h->fsas = k2::FsaToFsaVec(topo);
  return h;
  KREF_CATCH(nullptr)
}

void *kref_arc_sort(void *handle, int32_t *arc_map /* [num_arcs] or NULL */) {
  KREF_TRY
  auto *h = reinterpret_cast<FsaVecHandle *>(handle);
  auto *out = new FsaVecHandle;
  k2::Array1<int32_t> map;
  k2::ArcSort(h->fsas, &out->fsas, &map);
  if (arc_map && map.Dim() > 0)
    memcpy(arc_map, map.Data(), sizeof(int32_t) * (size_t)map.Dim());
  return out;
  KREF_CATCH(nullptr)
}

// scores: [rows, cols] contiguous; b_row_splits: [num_seqs + 1].
// a_to_b_map may be NULL.  Returns a new handle carrying arc_map_a/b.
void *kref_intersect_dense(void *a_handle, const float *scores, int32_t rows,
                           int32_t cols, const int32_t *b_row_splits,
                           int32_t num_seqs, const int32_t *a_to_b_map,
                           float output_beam, int32_t max_states,
                           int32_t max_arcs) {
  KREF_TRY
  auto *a = reinterpret_cast<FsaVecHandle *>(a_handle);
  k2::ContextPtr c = k2::GetCpuContext();
  k2::Array2<float> sc(c, rows, cols);
  if (rows * cols > 0)
    memcpy(sc.Data(), scores, sizeof(float) * (size_t)rows * (size_t)cols);
  k2::Array1<int32_t> brs = FromHost(b_row_splits, num_seqs + 1);
  k2::RaggedShape bshape = k2::RaggedShape2(&brs, nullptr, rows);
  k2::DenseFsaVec b(bshape, sc);
  k2::Array1<int32_t> map;
  if (a_to_b_map) map = FromHost(a_to_b_map, a->fsas.Dim0());
  auto *out = new FsaVecHandle;
  try {
    k2::IntersectDense(a->fsas, b, a_to_b_map ? &map : nullptr, output_beam,
                       max_states, max_arcs, &out->fsas, &out->arc_map_a,
                       &out->arc_map_b);
  } catch (...) {
    delete out;
    throw;
  }
  return out;
  KREF_CATCH(nullptr)
}

// Pruned intersection (k2/csrc/intersect_dense_pruned.cu:1678-1694).  a_handle holds
// one graph per sequence, or a single graph shared by all of them.
void *kref_intersect_dense_pruned(void *a_handle, const float *scores, int32_t rows,
                                  int32_t cols, const int32_t *b_row_splits,
                                  int32_t num_seqs, float search_beam,
                                  float output_beam, int32_t min_active,
                                  int32_t max_active, int32_t allow_partial) {
  KREF_TRY
  auto *a = reinterpret_cast<FsaVecHandle *>(a_handle);
  k2::ContextPtr c = k2::GetCpuContext();
  k2::Array2<float> sc(c, rows, cols);
  if (rows * cols > 0)
    memcpy(sc.Data(), scores, sizeof(float) * (size_t)rows * (size_t)cols);
  k2::Array1<int32_t> brs = FromHost(b_row_splits, num_seqs + 1);
  k2::RaggedShape bshape = k2::RaggedShape2(&brs, nullptr, rows);
  k2::DenseFsaVec b(bshape, sc);
  auto *out = new FsaVecHandle;
  try {
    k2::IntersectDensePruned(a->fsas, b, search_beam, output_beam, min_active,
                             max_active, allow_partial != 0, &out->fsas,
                             &out->arc_map_a, &out->arc_map_b);
  } catch (...) {
    delete out;
    throw;
  }
  return out;
  KREF_CATCH(nullptr)
}

// Online (chunk by chunk) pruned intersection, k2/csrc/intersect_dense_pruned.cu:1739-1853.
// An intersecter handle owns the shared graph; a stream handle owns one
// k2::DecodeStateInfo.  kref_online_decode takes the chunk's score matrix and one
// stream handle per sequence (NULL starts a new stream and the new handle is written
// back), and returns the lattice of everything decoded so far (arc_map_a only).
struct OnlineHandle {
  k2::FsaVec graph;
  k2::OnlineDenseIntersecter *impl;
};

void *kref_online_create(void *a_handle, int32_t num_seqs, float search_beam,
                         float output_beam, int32_t min_active, int32_t max_active,
                         int32_t allow_partial) {
  KREF_TRY
  auto *h = new OnlineHandle;
  h->graph = reinterpret_cast<FsaVecHandle *>(a_handle)->fsas;
  h->impl = new k2::OnlineDenseIntersecter(h->graph, num_seqs, search_beam, output_beam,
                                           min_active, max_active, allow_partial != 0);
  return h;
  KREF_CATCH(nullptr)
}

void kref_online_free(void *handle) {
  auto *h = reinterpret_cast<OnlineHandle *>(handle);
  delete h->impl;
  delete h;
}

void kref_online_stream_free(void *stream) {
  delete reinterpret_cast<k2::DecodeStateInfo *>(stream);
}

float kref_online_stream_beam(void *stream) {
  return reinterpret_cast<k2::DecodeStateInfo *>(stream)->beam;
}

void *kref_online_decode(void *handle, const float *scores, int32_t rows, int32_t cols,
                         const int32_t *b_row_splits, int32_t num_seqs, void **streams) {
  KREF_TRY
  auto *h = reinterpret_cast<OnlineHandle *>(handle);
  k2::ContextPtr c = k2::GetCpuContext();
  k2::Array2<float> sc(c, rows, cols);
  if (rows * cols > 0)
    memcpy(sc.Data(), scores, sizeof(float) * (size_t)rows * (size_t)cols);
  k2::Array1<int32_t> brs = FromHost(b_row_splits, num_seqs + 1);
  k2::RaggedShape bshape = k2::RaggedShape2(&brs, nullptr, rows);
  k2::DenseFsaVec b(bshape, sc);
  std::vector<k2::DecodeStateInfo *> states(num_seqs);
  for (int32_t i = 0; i < num_seqs; ++i) {
    if (streams[i] == nullptr) streams[i] = new k2::DecodeStateInfo();
    states[i] = reinterpret_cast<k2::DecodeStateInfo *>(streams[i]);
  }
  auto *out = new FsaVecHandle;
  try {
    h->impl->Decode(b, &states, &out->fsas, &out->arc_map_a);
  } catch (...) {
    delete out;
    throw;
  }
  return out;
  KREF_CATCH(nullptr)
}

// Forward scores of a top-sorted acyclic FsaVec.  `out` is [num_states] double
// (float results are widened exactly).  entering_arcs may be NULL; it is only
// filled when log_semiring == 0.
int32_t kref_forward_scores(void *handle, int32_t log_semiring,
                            int32_t use_double, double *out,
                            int32_t *entering_arcs) {
  KREF_TRY
  k2::FsaVec &fsas = reinterpret_cast<FsaVecHandle *>(handle)->fsas;
  k2::Ragged<int32_t> state_batches = k2::GetStateBatches(fsas, true);
  k2::Array1<int32_t> dest_states = k2::GetDestStates(fsas, true);
  k2::Ragged<int32_t> incoming = k2::GetIncomingArcs(fsas, dest_states);
  k2::Ragged<int32_t> entering_batches =
      k2::GetEnteringArcIndexBatches(fsas, incoming, state_batches);
  k2::Array1<int32_t> ea;
  k2::Array1<int32_t> *ea_ptr =
      (entering_arcs != nullptr && !log_semiring) ? &ea : nullptr;
  int32_t n = fsas.TotSize(1);
  if (use_double) {
    k2::Array1<double> s = k2::GetForwardScores<double>(
        fsas, state_batches, entering_batches, log_semiring != 0, ea_ptr);
    for (int32_t i = 0; i < n; ++i) out[i] = s.Data()[i];
  } else {
    k2::Array1<float> s = k2::GetForwardScores<float>(
        fsas, state_batches, entering_batches, log_semiring != 0, ea_ptr);
    for (int32_t i = 0; i < n; ++i) out[i] = s.Data()[i];
  }
  if (ea_ptr && n > 0) memcpy(entering_arcs, ea.Data(), sizeof(int32_t) * n);
  return 0;
  KREF_CATCH(-1)
}

int32_t kref_backward_scores(void *handle, int32_t log_semiring,
                             int32_t use_double, double *out) {
  KREF_TRY
  k2::FsaVec &fsas = reinterpret_cast<FsaVecHandle *>(handle)->fsas;
  k2::Ragged<int32_t> state_batches = k2::GetStateBatches(fsas, true);
  k2::Ragged<int32_t> leaving_batches =
      k2::GetLeavingArcIndexBatches(fsas, state_batches);
  int32_t n = fsas.TotSize(1);
  if (use_double) {
    k2::Array1<double> s = k2::GetBackwardScores<double>(
        fsas, state_batches, leaving_batches, log_semiring != 0);
    for (int32_t i = 0; i < n; ++i) out[i] = s.Data()[i];
  } else {
    k2::Array1<float> s = k2::GetBackwardScores<float>(
        fsas, state_batches, leaving_batches, log_semiring != 0);
    for (int32_t i = 0; i < n; ++i) out[i] = s.Data()[i];
  }
  return 0;
  KREF_CATCH(-1)
}

// tot_scores: [num_fsas] double; arc_post: [num_arcs] double (may be NULL).
int32_t kref_tot_scores_and_arc_post(void *handle, int32_t use_double,
                                     const double *forward,
                                     const double *backward,
                                     double *tot_scores, double *arc_post) {
  KREF_TRY
  k2::FsaVec &fsas = reinterpret_cast<FsaVecHandle *>(handle)->fsas;
  k2::ContextPtr c = k2::GetCpuContext();
  int32_t ns = fsas.TotSize(1), nf = fsas.Dim0(), na = fsas.NumElements();
  if (use_double) {
    k2::Array1<double> f = FromHost(forward, ns), b = FromHost(backward, ns);
    k2::Array1<double> tot = k2::GetTotScores<double>(fsas, f);
    for (int32_t i = 0; i < nf; ++i) tot_scores[i] = tot.Data()[i];
    if (arc_post) {
      k2::Array1<double> p = k2::GetArcPost<double>(fsas, f, b);
      for (int32_t i = 0; i < na; ++i) arc_post[i] = p.Data()[i];
    }
  } else {
    k2::Array1<float> f(c, ns), b(c, ns);
    for (int32_t i = 0; i < ns; ++i) {
      f.Data()[i] = (float)forward[i];
      b.Data()[i] = (float)backward[i];
    }
    k2::Array1<float> tot = k2::GetTotScores<float>(fsas, f);
    for (int32_t i = 0; i < nf; ++i) tot_scores[i] = tot.Data()[i];
    if (arc_post) {
      k2::Array1<float> p = k2::GetArcPost<float>(fsas, f, b);
      for (int32_t i = 0; i < na; ++i) arc_post[i] = p.Data()[i];
    }
  }
  return 0;
  KREF_CATCH(-1)
}

// Derivatives of forward / backward scores w.r.t. the arc scores
// (k2/csrc/fsa_utils.cu:1638-1795 and :1457-1624).  scores / deriv_in: [num_states]
// double (narrowed when use_double == 0); arc_deriv: [num_arcs] double.
int32_t kref_backprop_scores(void *handle, int32_t forward, int32_t log_semiring,
                             int32_t use_double, const double *scores,
                             const int32_t *entering_arcs, const double *deriv_in,
                             double *arc_deriv) {
  KREF_TRY
  k2::FsaVec &fsas = reinterpret_cast<FsaVecHandle *>(handle)->fsas;
  if (use_double)
    BackpropScoresT<double>(fsas, forward != 0, log_semiring != 0, scores, entering_arcs,
                            deriv_in, arc_deriv);
  else
    BackpropScoresT<float>(fsas, forward != 0, log_semiring != 0, scores, entering_arcs,
                           deriv_in, arc_deriv);
  return 0;
  KREF_CATCH(-1)
}

// Derivatives of the arc posteriors w.r.t. forward and backward scores
// (k2/csrc/fsa_utils.cu:1281-1334).
int32_t kref_backprop_arc_post(void *handle, int32_t use_double, const double *arc_post_deriv,
                               double *forward_deriv, double *backward_deriv) {
  KREF_TRY
  k2::FsaVec &fsas = reinterpret_cast<FsaVecHandle *>(handle)->fsas;
  int32_t ns = fsas.TotSize(1), na = fsas.NumElements();
  k2::Array1<int32_t> dest_states = k2::GetDestStates(fsas, true);
  k2::Ragged<int32_t> incoming = k2::GetIncomingArcs(fsas, dest_states);
  if (use_double) {
    k2::Array1<double> d = Narrow<double>(arc_post_deriv, na), f, b;
    k2::BackpropGetArcPost<double>(fsas, incoming, d, &f, &b);
    for (int32_t i = 0; i < ns; ++i) forward_deriv[i] = f.Data()[i], backward_deriv[i] = b.Data()[i];
  } else {
    k2::Array1<float> d = Narrow<float>(arc_post_deriv, na), f, b;
    k2::BackpropGetArcPost<float>(fsas, incoming, d, &f, &b);
    for (int32_t i = 0; i < ns; ++i) forward_deriv[i] = f.Data()[i], backward_deriv[i] = b.Data()[i];
  }
  return 0;
  KREF_CATCH(-1)
}

// best_arcs must have room for num_arcs entries; path_row_splits for
// num_fsas + 1.  Returns the total number of best-path arcs or -1.
int32_t kref_shortest_path(void *handle, const int32_t *entering_arcs,
                           int32_t *path_row_splits, int32_t *best_arcs) {
  KREF_TRY
  k2::FsaVec &fsas = reinterpret_cast<FsaVecHandle *>(handle)->fsas;
  k2::Array1<int32_t> ea = FromHost(entering_arcs, fsas.TotSize(1));
  k2::Ragged<int32_t> best = k2::ShortestPath(fsas, ea);
  memcpy(path_row_splits, best.RowSplits(1).Data(),
         sizeof(int32_t) * (fsas.Dim0() + 1));
  int32_t n = best.NumElements();
  if (n > 0) memcpy(best_arcs, best.values.Data(), sizeof(int32_t) * n);
  return n;
  KREF_CATCH(-1)
}

// properties: [num_fsas]; returns the AND over FSAs (tot_properties) or -1.
int32_t kref_properties(void *handle, int32_t *properties) {
  KREF_TRY
  k2::FsaVec &fsas = reinterpret_cast<FsaVecHandle *>(handle)->fsas;
  k2::Array1<int32_t> props;
  int32_t tot = 0;
  k2::GetFsaVecBasicProperties(fsas, &props, &tot);
  if (properties && props.Dim() > 0)
    memcpy(properties, props.Data(), sizeof(int32_t) * props.Dim());
  return tot;
  KREF_CATCH(-1)
}

}  // extern "C"

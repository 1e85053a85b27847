// Forward/backward scores, total scores, arc posteriors and their gradients over a
// layered (top-sorted, acyclic) FsaVec, plus the small gather/scatter, best-path and
// property kernels that sit on the same path.
//
// Follows the arithmetic of the reference (k2/csrc/fsa_utils.cu:1124-1278
// GetForwardScores, :1345-1454 GetBackwardScores, :1809-1837 GetTotScores,
// :1839-1901 GetArcPost; k2/python/csrc/torch/fsa.cu:493-592 the backward of
// tot_scores; k2/csrc/tensor_ops.cu:304-334 IndexAdd; k2/csrc/fsa_algo.cu:869-1144
// ShortestPath; k2/csrc/fsa.cu:54-217 properties) but walks the layers inside one
// persistent kernel per (FSA, direction) instead of launching per state batch.
#include <cmath>

#include "scores_internal.cuh"

namespace k2b {

// grid = (directions, fsas).  dir = blockIdx.x + dir_base: 0 forward, 1 backward.
template <typename Real, bool kLog>
__global__ void __launch_bounds__(256)
LayeredScores(k2b200_fsa_view v, Real *forward, Real *backward, int32_t *entering_arcs,
              int32_t dir_base, int32_t fsa_base, const int32_t *run_if) {
  // run_if (optional): only do the work when the word it points to is non-zero
  if (run_if != nullptr && *run_if == 0) return;
  LayeredScoresDevice<Real, kLog>(v, fsa_base + blockIdx.y, blockIdx.x + dir_base, forward,
                                  backward, entering_arcs);
}

template <typename Real>
__global__ void TotScores(const int32_t *__restrict__ row_splits1, int32_t num_fsas,
                          const Real *__restrict__ forward, Real *__restrict__ tot) {
  int32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= num_fsas) return;
  int32_t b = row_splits1[i], e = row_splits1[i + 1];
  tot[i] = e > b ? forward[e - 1] : (Real)-INFINITY;
}

template <typename Real>
__global__ void ArcPost(const int32_t *__restrict__ row_splits1,
                        const int32_t *__restrict__ row_ids1,
                        const int32_t *__restrict__ row_ids2, const Arc *__restrict__ arcs,
                        int32_t num_arcs, const Real *__restrict__ forward,
                        const Real *__restrict__ backward, Real *__restrict__ post) {
  int32_t a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= num_arcs) return;
  const int32_t src01 = row_ids2[a], fsa = row_ids1[src01];
  const int32_t b = row_splits1[fsa], e = row_splits1[fsa + 1];
  const Real kNegInf = -INFINITY;
  Real tot = (Real)0.5 * (forward[e - 1] + backward[b]);
  Real neg = tot != kNegInf ? -tot : kNegInf;
  Arc arc = arcs[a];
  post[a] = (Real)arc.score + forward[src01] + backward[b + arc.dest] + neg;
}

template <typename Real>
__global__ void LogBackward(const int32_t *__restrict__ row_ids1,
                            const int32_t *__restrict__ row_ids2, int32_t num_arcs,
                            const Real *__restrict__ post, const Real *__restrict__ tot_grad,
                            int64_t stride, float *__restrict__ grad) {
  int32_t a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= num_arcs) return;
  int32_t fsa = row_ids1[row_ids2[a]];
  grad[a] = (float)(ExpReal<Real>(post[a]) * tot_grad[fsa * stride]);
}

template <typename Real>
__global__ void TropicalBackward(const int32_t *__restrict__ row_ids1,
                                 const int32_t *__restrict__ row_ids2,
                                 const int32_t *__restrict__ best_arcs, int32_t num_best,
                                 const Real *__restrict__ tot_grad, int64_t stride,
                                 float *__restrict__ grad) {
  int32_t k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= num_best) return;
  int32_t a = best_arcs[k];
  grad[a] = (float)tot_grad[row_ids1[row_ids2[a]] * stride];
}

__global__ void IndexAdd(const int32_t *__restrict__ index, const float *__restrict__ value,
                         int32_t n, float *__restrict__ in_out, int64_t size) {
  int32_t k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  int32_t j = index[k];
  if (j >= 0 && j < size) atomicAdd(in_out + j, value[k]);
}

__global__ void IndexSelectI32(const int32_t *__restrict__ src, int64_t size,
                               const int32_t *__restrict__ index, int32_t n,
                               int32_t *__restrict__ out) {
  int32_t k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= n) return;
  int32_t j = index[k];
  out[k] = (j >= 0 && j < size) ? src[j] : 0;
}

// Length of the best path of every FSA (0 when the trace does not reach the
// start state).  One thread per FSA; the walk is bounded by the FSA's state count.
__global__ void PathLengths(const int32_t *__restrict__ row_splits1, const Arc *__restrict__ arcs,
                            const int32_t *__restrict__ entering, int32_t num_fsas,
                            int32_t *__restrict__ lengths) {
  int32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= num_fsas) return;
  int32_t b = row_splits1[i], e = row_splits1[i + 1], len = 0;
  if (e > b) {
    int32_t cur = e - 1, idx = entering[cur];
    while (idx != -1 && len <= e - b) {
      ++len;
      cur = b + arcs[idx].src;
      idx = entering[cur];
    }
    if (cur != b || len > e - b) len = 0;
  }
  lengths[i] = len;
}

__global__ void PathFill(const int32_t *__restrict__ row_splits1, const Arc *__restrict__ arcs,
                         const int32_t *__restrict__ entering, int32_t num_fsas,
                         const int32_t *__restrict__ path_splits, int32_t *__restrict__ best) {
  int32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= num_fsas) return;
  int32_t p0 = path_splits[i], len = path_splits[i + 1] - p0;
  if (len == 0) return;
  int32_t b = row_splits1[i], cur = row_splits1[i + 1] - 1;
  for (int32_t k = len - 1; k >= 0; --k) {
    int32_t idx = entering[cur];
    best[p0 + k] = idx;
    cur = b + arcs[idx].src;
  }
}

constexpr int32_t kAllProps = 0x1FF;

__global__ void PropsInit(int32_t *props, int32_t n_plus_one, char *reach, int64_t nreach) {
  int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (k < n_plus_one) props[k] = kAllProps;
  if (k < nreach) reach[k] = 0;
}

__global__ void PropsArcs(const int32_t *__restrict__ row_splits1,
                          const int32_t *__restrict__ row_ids1,
                          const int32_t *__restrict__ row_splits2,
                          const int32_t *__restrict__ row_ids2, const Arc *__restrict__ arcs,
                          int32_t num_states, int32_t num_arcs, int32_t *props, char *reach) {
  int32_t a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= num_arcs) return;
  Arc arc = arcs[a];
  const int32_t idx01 = row_ids2[a], idx2 = a - row_splits2[idx01], idx0 = row_ids1[idx01],
                idx0x = row_splits1[idx0], idx0x_next = row_splits1[idx0 + 1],
                idx1 = idx01 - idx0x, idx0xx = row_splits2[idx0x], n = idx0x_next - idx0x;
  int32_t neg = 0;
  if (arc.src != idx1) neg |= 0x01;
  if (arc.dest <= arc.src) {
    neg |= 0x08;
    if (arc.dest < arc.src) neg |= 0x04;
  }
  if (arc.label == 0) neg |= 0x40;
  if (arc.label < 0) {
    if (arc.label != -1) neg |= 0x01;
    else if (arc.dest != n - 1) neg |= 0x01;
  }
  if (arc.label != -1 && arc.dest == n - 1) neg |= 0x01;
  if (arc.dest < 0 || arc.dest >= n) neg |= 0x01;
  else if (arc.dest != arc.src) reach[idx0x + arc.dest] = 1;
  if (idx0xx == a) {
    reach[idx0x] = 1;
    reach[num_states + idx0x_next - 1] = 1;
  }
  if (arc.dest != arc.src) reach[num_states + idx01] = 1;
  if (idx2 != 0) {
    Arc p = arcs[a - 1];
    if ((uint32_t)arc.label <= (uint32_t)p.label) neg |= 0x20;
    if ((uint32_t)arc.label < (uint32_t)p.label) neg |= 0x10;
    if (arc.label == p.label && arc.dest < p.dest) neg |= 0x10;
  }
  if (neg) atomicAnd(&props[idx0], ~neg);
}

__global__ void PropsStates(const int32_t *__restrict__ row_ids1, int32_t num_states,
                            const char *__restrict__ reach, int32_t *props) {
  int32_t s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= num_states) return;
  int32_t neg = (reach[s] ? 0 : 0x80) | (reach[num_states + s] ? 0 : 0x100);
  if (neg) atomicAnd(&props[row_ids1[s]], ~neg);
}

__global__ void PropsFinish(const int32_t *__restrict__ row_splits1,
                            const int32_t *__restrict__ row_splits2, int32_t num_fsas,
                            int32_t *props) {
  int32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= num_fsas) return;
  if (row_splits2[row_splits1[i]] == row_splits2[row_splits1[i + 1]]) atomicAnd(&props[i], ~0x02);
  __threadfence();
  atomicAnd(&props[num_fsas], props[i] & kAllProps);
}

}  // namespace k2b

using namespace k2b;

#define STREAM(s) reinterpret_cast<cudaStream_t>(s)

template <typename Real>
static int32_t LaunchGeneric(const k2b200_fsa_view *v, int32_t log_semiring, Real *fwd, Real *bwd,
                             int32_t *entering, const int32_t *run_if, cudaStream_t stream) {
  int32_t ndir = (fwd != nullptr) + (bwd != nullptr), dir_base = fwd ? 0 : 1;
  for (int32_t first = 0; first < v->num_fsas; first += 65535) {
    int32_t n = v->num_fsas - first < 65535 ? v->num_fsas - first : 65535;
    dim3 grid(ndir, n);
    if (log_semiring)
      { LayeredScores<Real, true><<<grid, 256, 0, stream>>>(*v, fwd, bwd, nullptr, dir_base,
                                                            first, run_if); NoteLaunch(); }
    else
      { LayeredScores<Real, false><<<grid, 256, 0, stream>>>(*v, fwd, bwd, entering, dir_base,
                                                             first, run_if); NoteLaunch(); }
  }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

template <typename Real>
static int32_t LaunchScores(const k2b200_fsa_view *v, int32_t log_semiring, Real *fwd, Real *bwd,
                            int32_t *entering, void *scratch, size_t scratch_bytes,
                            cudaStream_t stream) {
  int32_t ndir = (fwd != nullptr) + (bwd != nullptr);
  if (ndir == 0 || v->num_fsas == 0) return kOk;
  PhaseTimer timer(kPhaseScores, stream);
  bool launched = false;
  if (log_semiring) {
    K2B_FORWARD(LaunchProbScores<Real>(v, fwd, bwd, scratch, scratch_bytes, stream, &launched));
    // if a CTA found the layer bounds violated, redo everything the general way
    if (launched)
      return LaunchGeneric<Real>(v, 1, fwd, bwd, nullptr, ProbStatusWord(v, scratch), stream);
  }
  K2B_FORWARD(LaunchStagedScores<Real>(v, log_semiring, fwd, bwd, entering, stream, &launched));
  if (launched) return kOk;
  return LaunchGeneric<Real>(v, log_semiring, fwd, bwd, entering, nullptr, stream);
}

extern "C" {

const char *k2b200_last_error(void) { return LastError(); }
int32_t k2b200_abi_version(void) { return 5; }
int64_t k2b200_kernel_launch_count(void) { return LaunchCount(); }
void k2b200_profile_enable(int32_t on) { SetProfiling(on != 0); }
const char *k2b200_profile_kernel(int32_t phase) { return PhaseKernel(phase); }
double k2b200_profile_read_ms(int32_t phase, int64_t *intervals) {
  long long n = 0;
  double ms = (phase >= 0 && phase < kNumPhases) ? ReadPhase(phase, &n) : 0.0;
  if (intervals) *intervals = n;
  return ms;
}

int32_t k2b200_row_splits_to_row_ids(const int32_t *row_splits, int32_t num_rows,
                                     int32_t *row_ids, int32_t num_elems, void *stream) {
  return RowSplitsToRowIds(row_splits, num_rows, row_ids, num_elems, STREAM(stream));
}

int32_t k2b200_upload_i32(const int32_t *host_values, int64_t n, int32_t *device_out,
                          void *stream) {
  K2B_REQUIRE(n >= 0, "negative length");
  K2B_REQUIRE(n == 0 || (host_values != nullptr && device_out != nullptr), "NULL pointer");
  return UploadInts(host_values, n, device_out, STREAM(stream));
}

size_t k2b200_exclusive_sum_tmp_bytes(int64_t n) { return sizeof(int32_t) * ScanTmpInts(n); }
int32_t k2b200_exclusive_sum(const int32_t *in, int32_t *out, int64_t n, void *tmp,
                             void *stream) {
  return ExclusiveSum(in, out, n, reinterpret_cast<int32_t *>(tmp), STREAM(stream));
}

int64_t k2b200_exclusive_sum_static_max_len(void) { return ExclusiveSumStaticMaxLen(); }
int32_t k2b200_exclusive_sum_static(const int32_t *in, int32_t *out, int64_t n, void *stream) {
  K2B_REQUIRE(n == 0 || (in != nullptr && out != nullptr), "NULL pointer");
  K2B_REQUIRE(out != nullptr, "NULL output pointer");
  return ExclusiveSumStatic(in, out, n, STREAM(stream));
}

size_t k2b200_fsa_incoming_tmp_bytes(int32_t num_states, int32_t num_arcs) {
  return IncomingTmpBytes(num_states, num_arcs);
}
int32_t k2b200_fsa_incoming(const int32_t *row_splits1, const int32_t *row_ids1,
                            const int32_t *row_ids2, const void *arcs, int32_t num_fsas,
                            int32_t num_states, int32_t num_arcs, int32_t *in_splits,
                            int32_t *in_arcs, int32_t *in_src, float *in_score, void *tmp,
                            void *stream) {
  K2B_REQUIRE(num_fsas >= 0 && num_states >= 0 && num_arcs >= 0, "negative size");
  K2B_REQUIRE(in_splits && tmp, "NULL pointer");
  PhaseTimer timer(kPhaseIncoming, STREAM(stream));
  return BuildIncoming(row_splits1, row_ids1, row_ids2, reinterpret_cast<const Arc *>(arcs),
                       num_fsas, num_states, num_arcs, in_splits, in_arcs, in_src, in_score, tmp,
                       STREAM(stream));
}

size_t k2b200_fsa_scores_scratch_bytes(const k2b200_fsa_view *v) {
  return v ? ProbScratchBytes(v) : 0;
}

int32_t k2b200_fsa_scores(const k2b200_fsa_view *v, int32_t log_semiring, int32_t use_double,
                          void *forward, void *backward, int32_t *entering_arcs, void *scratch,
                          size_t scratch_bytes, void *stream) {
  K2B_REQUIRE(v != nullptr, "NULL view");
  K2B_REQUIRE(v->row_splits1 && v->row_splits2 && v->level_offsets && v->level_splits,
              "NULL pointer in the FsaVec view");
  K2B_REQUIRE(forward == nullptr || v->num_arcs == 0 ||
                  (v->in_splits && v->in_arcs && v->row_ids2),
              "forward scores need the incoming-arc index and row_ids2");
  if (use_double)
    return LaunchScores<double>(v, log_semiring, reinterpret_cast<double *>(forward),
                                reinterpret_cast<double *>(backward), entering_arcs, scratch,
                                scratch_bytes, STREAM(stream));
  return LaunchScores<float>(v, log_semiring, reinterpret_cast<float *>(forward),
                             reinterpret_cast<float *>(backward), entering_arcs, scratch,
                             scratch_bytes, STREAM(stream));
}

int32_t k2b200_fsa_tot_scores(const int32_t *row_splits1, int32_t num_fsas, int32_t use_double,
                              const void *forward, void *tot_scores, void *stream) {
  if (num_fsas <= 0) return kOk;
  if (use_double)
    { TotScores<double><<<CeilDiv(num_fsas, 128), 128, 0, STREAM(stream)>>>(
        row_splits1, num_fsas, reinterpret_cast<const double *>(forward),
        reinterpret_cast<double *>(tot_scores)); NoteLaunch(); }
  else
    { TotScores<float><<<CeilDiv(num_fsas, 128), 128, 0, STREAM(stream)>>>(
        row_splits1, num_fsas, reinterpret_cast<const float *>(forward),
        reinterpret_cast<float *>(tot_scores)); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t k2b200_fsa_arc_post(const int32_t *row_splits1, const int32_t *row_ids1,
                            const int32_t *row_ids2, const void *arcs, int32_t num_fsas,
                            int32_t num_arcs, int32_t use_double, const void *forward,
                            const void *backward, void *arc_post, void *stream) {
  PhaseTimer timer(kPhasePost, STREAM(stream));
  (void)num_fsas;
  if (num_arcs <= 0) return kOk;
  const Arc *a = reinterpret_cast<const Arc *>(arcs);
  if (use_double)
    { ArcPost<double><<<CeilDiv(num_arcs, 256), 256, 0, STREAM(stream)>>>(
        row_splits1, row_ids1, row_ids2, a, num_arcs, reinterpret_cast<const double *>(forward),
        reinterpret_cast<const double *>(backward), reinterpret_cast<double *>(arc_post)); NoteLaunch(); }
  else
    { ArcPost<float><<<CeilDiv(num_arcs, 256), 256, 0, STREAM(stream)>>>(
        row_splits1, row_ids1, row_ids2, a, num_arcs, reinterpret_cast<const float *>(forward),
        reinterpret_cast<const float *>(backward), reinterpret_cast<float *>(arc_post)); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t k2b200_tot_scores_log_backward(const int32_t *row_ids1, const int32_t *row_ids2,
                                       int32_t num_arcs, int32_t use_double,
                                       const void *arc_post, const void *tot_scores_grad,
                                       int64_t grad_stride, float *arc_grad, void *stream) {
  PhaseTimer timer(kPhasePost, STREAM(stream));
  if (num_arcs <= 0) return kOk;
  if (use_double)
    { LogBackward<double><<<CeilDiv(num_arcs, 256), 256, 0, STREAM(stream)>>>(
        row_ids1, row_ids2, num_arcs, reinterpret_cast<const double *>(arc_post),
        reinterpret_cast<const double *>(tot_scores_grad), grad_stride, arc_grad); NoteLaunch(); }
  else
    { LogBackward<float><<<CeilDiv(num_arcs, 256), 256, 0, STREAM(stream)>>>(
        row_ids1, row_ids2, num_arcs, reinterpret_cast<const float *>(arc_post),
        reinterpret_cast<const float *>(tot_scores_grad), grad_stride, arc_grad); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t k2b200_tot_scores_tropical_backward(const int32_t *row_ids1, const int32_t *row_ids2,
                                            int32_t num_arcs, const int32_t *best_arcs,
                                            int32_t num_best_arcs, int32_t use_double,
                                            const void *tot_scores_grad, int64_t grad_stride,
                                            float *arc_grad, void *stream) {
  if (num_arcs <= 0) return kOk;
  K2B_CUDA_OK(cudaMemsetAsync(arc_grad, 0, sizeof(float) * (size_t)num_arcs, STREAM(stream)));
  if (num_best_arcs <= 0) return kOk;
  if (use_double)
    { TropicalBackward<double><<<CeilDiv(num_best_arcs, 256), 256, 0, STREAM(stream)>>>(
        row_ids1, row_ids2, best_arcs, num_best_arcs,
        reinterpret_cast<const double *>(tot_scores_grad), grad_stride, arc_grad); NoteLaunch(); }
  else
    { TropicalBackward<float><<<CeilDiv(num_best_arcs, 256), 256, 0, STREAM(stream)>>>(
        row_ids1, row_ids2, best_arcs, num_best_arcs,
        reinterpret_cast<const float *>(tot_scores_grad), grad_stride, arc_grad); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t k2b200_index_add(const int32_t *index, const float *value, int32_t n, float *in_out,
                         int64_t in_out_size, void *stream) {
  PhaseTimer timer(kPhasePost, STREAM(stream));
  if (n <= 0) return kOk;
  { IndexAdd<<<CeilDiv(n, 256), 256, 0, STREAM(stream)>>>(index, value, n, in_out, in_out_size); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t k2b200_index_select_i32(const int32_t *src, int64_t src_size, const int32_t *index,
                                int32_t n, int32_t *out, void *stream) {
  if (n <= 0) return kOk;
  { IndexSelectI32<<<CeilDiv(n, 256), 256, 0, STREAM(stream)>>>(src, src_size, index, n, out); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

size_t k2b200_shortest_path_tmp_bytes(int32_t num_fsas) {
  return AlignUp(sizeof(int32_t) * ((size_t)num_fsas + 1)) +
         AlignUp(sizeof(int32_t) * ScanTmpInts(num_fsas));
}

int32_t k2b200_shortest_path(const int32_t *row_splits1, const void *arcs,
                             const int32_t *entering_arcs, int32_t num_fsas,
                             int32_t *path_splits, int32_t *best_arcs, void *tmp, void *stream) {
  if (num_fsas <= 0) return kOk;
  K2B_REQUIRE(row_splits1 && entering_arcs && path_splits && best_arcs && tmp, "NULL pointer");
  char *p = reinterpret_cast<char *>(tmp);
  int32_t *lengths = reinterpret_cast<int32_t *>(p);
  int32_t *scan_tmp =
      reinterpret_cast<int32_t *>(p + AlignUp(sizeof(int32_t) * ((size_t)num_fsas + 1)));
  const Arc *a = reinterpret_cast<const Arc *>(arcs);
  { PathLengths<<<CeilDiv(num_fsas, 64), 64, 0, STREAM(stream)>>>(row_splits1, a, entering_arcs,
                                                               num_fsas, lengths); NoteLaunch(); }
  K2B_FORWARD(ExclusiveSum(lengths, path_splits, num_fsas, scan_tmp, STREAM(stream)));
  { PathFill<<<CeilDiv(num_fsas, 64), 64, 0, STREAM(stream)>>>(row_splits1, a, entering_arcs,
                                                            num_fsas, path_splits, best_arcs); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

size_t k2b200_fsa_properties_tmp_bytes(int32_t num_fsas, int32_t num_states) {
  (void)num_fsas;
  return AlignUp(2 * (size_t)num_states + 2);
}

int32_t k2b200_fsa_properties(const int32_t *row_splits1, const int32_t *row_ids1,
                              const int32_t *row_splits2, const int32_t *row_ids2,
                              const void *arcs, int32_t num_fsas, int32_t num_states,
                              int32_t num_arcs, int32_t *properties, void *tmp, void *stream) {
  K2B_REQUIRE(properties && tmp, "NULL pointer");
  char *reach = reinterpret_cast<char *>(tmp);
  int64_t nreach = 2 * (int64_t)num_states;
  int64_t n0 = nreach > num_fsas + 1 ? nreach : num_fsas + 1;
  { PropsInit<<<CeilDiv(n0, 256), 256, 0, STREAM(stream)>>>(properties, num_fsas + 1, reach, nreach); NoteLaunch(); }
  if (num_arcs > 0)
    { PropsArcs<<<CeilDiv(num_arcs, 256), 256, 0, STREAM(stream)>>>(
        row_splits1, row_ids1, row_splits2, row_ids2, reinterpret_cast<const Arc *>(arcs),
        num_states, num_arcs, properties, reach); NoteLaunch(); }
  if (num_states > 0)
    { PropsStates<<<CeilDiv(num_states, 256), 256, 0, STREAM(stream)>>>(row_ids1, num_states, reach,
                                                                     properties); NoteLaunch(); }
  if (num_fsas > 0)
    { PropsFinish<<<CeilDiv(num_fsas, 128), 128, 0, STREAM(stream)>>>(row_splits1, row_splits2,
                                                                   num_fsas, properties); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

}  // extern "C"

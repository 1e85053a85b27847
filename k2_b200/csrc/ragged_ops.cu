// Generic ragged-array primitives, hand-written for sm_100a: multi-block exclusive
// sums, row_splits -> row_ids, and the incoming-arc index of an FsaVec.  They take
// the place of the cub / moderngpu wrappers the reference leans on
// (k2/csrc/utils_inl.h:40-90 ExclusiveSum, k2/csrc/utils.cu:75-200
// RowSplitsToRowIds, k2/csrc/fsa_utils.cu:901-928 GetIncomingArcs).
#include <nvtx3/nvToolsExt.h>
#include <atomic>
#include <cstring>
#include <cstdlib>
#include <strings.h>
#include <cstdio>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace k2b {

// ----------------------------------------------------------------------------
// error text (thread local so concurrent callers do not clobber each other)
// ----------------------------------------------------------------------------
static thread_local char g_error[1024] = "";

void SetError(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
const char *LastError() { return g_error; }

// ----------------------------------------------------------------------------
// logger
// ----------------------------------------------------------------------------
static int ReadLogLevel() {
  const char *v = getenv("K2_LOG_LEVEL");
  if (v == nullptr) return kLogInfo;
  static const char *const names[] = {"TRACE", "DEBUG", "INFO", "WARNING", "ERROR", "FATAL"};
  for (int k = 0; k < 6; ++k)
    if (strcasecmp(v, names[k]) == 0) return k;
  return kLogInfo;
}
bool LogEnabled(LogLevel level) {
  static const int threshold = ReadLogLevel();
  return (int)level >= threshold;
}
void LogLine(LogLevel level, const char *fmt, ...) {
  static const char kTag[] = "TDIWEF";
  char line[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(line, sizeof(line), fmt, ap);
  va_end(ap);
  fprintf(stderr, "[%c] k2b200: %s\n", kTag[level], line);
}

// ----------------------------------------------------------------------------
// launch counter and phase timers
// ----------------------------------------------------------------------------
static std::atomic<long long> g_launches{0};
void NoteLaunch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
long long LaunchCount() { return g_launches.load(std::memory_order_relaxed); }

static std::atomic<int32_t> g_copy_wait_limit{4000000};
int32_t CopyWaitLimit() { return g_copy_wait_limit.load(std::memory_order_relaxed); }
void SetCopyWaitLimit(int32_t polls) {
  g_copy_wait_limit.store(polls < 0 ? 4000000 : polls, std::memory_order_relaxed);
}

static const char *g_phase_kernel[kNumPhases] = {};
void NotePhaseKernel(int phase, const char *name) {
  if (phase >= 0 && phase < kNumPhases) g_phase_kernel[phase] = name;
}
const char *PhaseKernel(int phase) {
  return (phase >= 0 && phase < kNumPhases && g_phase_kernel[phase]) ? g_phase_kernel[phase] : "";
}

namespace {
struct EventPair { cudaEvent_t start, stop; };
struct PhaseLog {
  std::vector<EventPair> pool;  // reused across reads
  size_t used = 0;
};
std::mutex g_prof_mutex;
bool g_profiling = false;
PhaseLog g_phase[kNumPhases];
}  // namespace

void SetProfiling(bool on) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  g_profiling = on;
  for (auto &p : g_phase) p.used = 0;
}

// NVTX ranges (as the reference's NVTX_RANGE, k2/csrc/nvtx.h:31-61) around the same phases:
// no-ops unless a tool that injects an NVTX library is attached.
static const char *const kPhaseNames[kNumPhases] = {
    "k2b200:viterbi", "k2b200:prune", "k2b200:emit", "k2b200:scores", "k2b200:posteriors",
    "k2b200:incoming", "k2b200:dense", "k2b200:chain", "k2b200:grad"};

PhaseTimer::PhaseTimer(int phase, cudaStream_t stream) : phase_(phase), stream_(stream), slot_(-1) {
  nvtxRangePushA(kPhaseNames[phase]);
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  if (!g_profiling) return;
  PhaseLog &log = g_phase[phase];
  if (log.used == log.pool.size()) {
    EventPair e;
    if (cudaEventCreate(&e.start) != cudaSuccess || cudaEventCreate(&e.stop) != cudaSuccess) return;
    log.pool.push_back(e);
  }
  slot_ = (int)log.used++;
  cudaEventRecord(log.pool[slot_].start, stream);
}
PhaseTimer::~PhaseTimer() {
  nvtxRangePop();
  if (slot_ < 0) return;
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  cudaEventRecord(g_phase[phase_].pool[slot_].stop, stream_);
}

// Sum of the recorded durations of `phase` in ms (waits for the events); resets
// the phase's log.  count receives the number of recorded intervals.
double ReadPhase(int phase, long long *count) {
  std::lock_guard<std::mutex> lock(g_prof_mutex);
  PhaseLog &log = g_phase[phase];
  double total = 0;
  for (size_t k = 0; k < log.used; ++k) {
    float ms = 0;
    cudaEventSynchronize(log.pool[k].stop);
    if (cudaEventElapsedTime(&ms, log.pool[k].start, log.pool[k].stop) == cudaSuccess) total += ms;
  }
  if (count) *count = (long long)log.used;
  log.used = 0;
  return total;
}

// ----------------------------------------------------------------------------
// side stream (one per device, created on first use)
// ----------------------------------------------------------------------------
namespace {
struct SideState {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork_ev = nullptr, join_ev = nullptr, host_ev = nullptr, scope_ev = nullptr;
  void *pinned = nullptr;  // kSidePinnedBytes of page-locked host memory
};
constexpr size_t kSidePinnedBytes = 256;
std::mutex g_side_mutex;
std::vector<SideState> g_side;

int32_t SideOfCurrentDevice(SideState **out) {
  int dev = 0;
  K2B_CUDA_OK(cudaGetDevice(&dev));
  if ((size_t)dev >= g_side.size()) g_side.resize(dev + 1);
  SideState &st = g_side[dev];
  if (st.stream == nullptr) {
    K2B_CUDA_OK(cudaStreamCreateWithFlags(&st.stream, cudaStreamNonBlocking));
    K2B_CUDA_OK(cudaEventCreateWithFlags(&st.fork_ev, cudaEventDisableTiming));
    K2B_CUDA_OK(cudaEventCreateWithFlags(&st.join_ev, cudaEventDisableTiming));
    K2B_CUDA_OK(cudaEventCreateWithFlags(&st.host_ev, cudaEventDisableTiming));
    K2B_CUDA_OK(cudaEventCreateWithFlags(&st.scope_ev, cudaEventDisableTiming));
    K2B_CUDA_OK(cudaHostAlloc(&st.pinned, kSidePinnedBytes, cudaHostAllocDefault));
  }
  *out = &st;
  return kOk;
}
}  // namespace

int32_t SideFork(cudaStream_t main, cudaStream_t *side) {
  std::lock_guard<std::mutex> lock(g_side_mutex);
  SideState *st;
  K2B_FORWARD(SideOfCurrentDevice(&st));
  K2B_CUDA_OK(cudaEventRecord(st->fork_ev, main));
  K2B_CUDA_OK(cudaStreamWaitEvent(st->stream, st->fork_ev, 0));
  *side = st->stream;
  return kOk;
}

int32_t SideJoin(cudaStream_t main) {
  std::lock_guard<std::mutex> lock(g_side_mutex);
  SideState *st;
  K2B_FORWARD(SideOfCurrentDevice(&st));
  K2B_CUDA_OK(cudaEventRecord(st->join_ev, st->stream));
  K2B_CUDA_OK(cudaStreamWaitEvent(main, st->join_ev, 0));
  return kOk;
}

// Copies `bytes` (at most 256) of device memory to `host_out` behind the work queued
// on the side stream, and blocks the host until that copy - not the main stream - is
// done.
int32_t SideReadBack(const void *device_src, size_t bytes, void *host_out) {
  std::lock_guard<std::mutex> lock(g_side_mutex);
  SideState *st;
  K2B_FORWARD(SideOfCurrentDevice(&st));
  K2B_REQUIRE(bytes <= kSidePinnedBytes / 2, "SideReadBack: too many bytes");
  K2B_CUDA_OK(cudaMemcpyAsync(st->pinned, device_src, bytes, cudaMemcpyDeviceToHost, st->stream));
  K2B_CUDA_OK(cudaEventRecord(st->host_ev, st->stream));
  K2B_CUDA_OK(cudaEventSynchronize(st->host_ev));
  memcpy(host_out, st->pinned, bytes);
  return kOk;
}

static std::mutex g_readback_mutex;  // held from Begin to End (or to the scope's end)

int32_t SideReadBackScope::Begin(const void *device_src, size_t bytes) {
  K2B_REQUIRE(!held_, "SideReadBackScope::Begin called twice");
  K2B_REQUIRE(bytes <= kSidePinnedBytes / 2, "SideReadBackScope: too many bytes");
  g_readback_mutex.lock();
  held_ = true;
  bytes_ = bytes;
  std::lock_guard<std::mutex> lock(g_side_mutex);
  SideState *st;
  K2B_FORWARD(SideOfCurrentDevice(&st));
  // the second half of the pinned buffer: SideReadBack uses the first
  K2B_CUDA_OK(cudaMemcpyAsync(static_cast<char *>(st->pinned) + kSidePinnedBytes / 2, device_src,
                              bytes, cudaMemcpyDeviceToHost, st->stream));
  K2B_CUDA_OK(cudaEventRecord(st->scope_ev, st->stream));
  return kOk;
}

int32_t SideReadBackScope::End(void *host_out) {
  K2B_REQUIRE(held_, "SideReadBackScope::End without Begin");
  SideState *st;
  {
    std::lock_guard<std::mutex> lock(g_side_mutex);
    K2B_FORWARD(SideOfCurrentDevice(&st));
  }
  K2B_CUDA_OK(cudaEventSynchronize(st->scope_ev));
  memcpy(host_out, static_cast<char *>(st->pinned) + kSidePinnedBytes / 2, bytes_);
  held_ = false;
  g_readback_mutex.unlock();
  return kOk;
}

SideReadBackScope::~SideReadBackScope() {
  if (held_) g_readback_mutex.unlock();
}

// ----------------------------------------------------------------------------
// A few hundred host integers to device memory without the copy engine: the values
// travel as kernel parameters.  A copy from pageable memory synchronises the stream
// in torch, and one from pinned memory queues behind whatever large transfer the
// application has in flight; a launch does neither.
// ----------------------------------------------------------------------------
struct IntChunk {
  int32_t v[960];  // kernel parameters are limited to 4 KB
};
__global__ void StoreInts(IntChunk c, int32_t n, int32_t *__restrict__ out) {
  const int32_t k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k < n) out[k] = c.v[k];
}

int32_t UploadInts(const int32_t *host, int64_t n, int32_t *device_out, cudaStream_t stream) {
  IntChunk c;
  for (int64_t done = 0; done < n; done += 960) {
    const int32_t m = (int32_t)std::min<int64_t>(960, n - done);
    memcpy(c.v, host + done, sizeof(int32_t) * m);
    { StoreInts<<<CeilDiv(m, 256), 256, 0, stream>>>(c, m, device_out + done); NoteLaunch(); }
  }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

// ----------------------------------------------------------------------------
// exclusive sum: reduce tiles -> scan the tile sums in one block -> rescan tiles
// ----------------------------------------------------------------------------
constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;
constexpr int kScanTile = kScanThreads * kScanItems;

__device__ __forceinline__ int32_t Add(int32_t a, int32_t b) { return a + b; }
__device__ __forceinline__ int2 Add(int2 a, int2 b) { return make_int2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ int32_t Sub(int32_t a, int32_t b) { return a - b; }
__device__ __forceinline__ int2 Sub(int2 a, int2 b) { return make_int2(a.x - b.x, a.y - b.y); }
__device__ __forceinline__ int32_t Zero(int32_t) { return 0; }
__device__ __forceinline__ int2 Zero(int2) { return make_int2(0, 0); }
__device__ __forceinline__ int32_t ShflUp(int32_t v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
__device__ __forceinline__ int2 ShflUp(int2 v, int d) {
  return make_int2(__shfl_up_sync(0xffffffffu, v.x, d), __shfl_up_sync(0xffffffffu, v.y, d));
}

// Inclusive scan of one value per thread across the block; returns the inclusive
// prefix, *total receives the block sum.  smem must hold kScanThreads/32 values.
template <typename T>
__device__ __forceinline__ T BlockInclusiveScan(T v, T *smem, T *total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    T o = ShflUp(v, d);
    if (lane >= d) v = Add(v, o);
  }
  if (lane == 31) smem[warp] = v;
  __syncthreads();
  if (warp == 0) {
    T w = lane < (kScanThreads / 32) ? smem[lane] : Zero(v);
#pragma unroll
    for (int d = 1; d < kScanThreads / 32; d <<= 1) {
      T o = ShflUp(w, d);
      if (lane >= d) w = Add(w, o);
    }
    if (lane < kScanThreads / 32) smem[lane] = w;
  }
  __syncthreads();
  if (warp > 0) v = Add(v, smem[warp - 1]);
  *total = smem[kScanThreads / 32 - 1];
  __syncthreads();
  return v;
}

template <typename T>
__global__ void __launch_bounds__(kScanThreads)
ScanTileSums(const T *__restrict__ in, int64_t n, T *__restrict__ tile_sums) {
  __shared__ T smem[kScanThreads / 32];
  int64_t base = (int64_t)blockIdx.x * kScanTile + (int64_t)threadIdx.x * kScanItems;
  T acc = Zero(T());
#pragma unroll
  for (int k = 0; k < kScanItems; ++k)
    if (base + k < n) acc = Add(acc, in[base + k]);
  T total;
  BlockInclusiveScan(acc, smem, &total);
  if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
}

// One block turns tile_sums[0..nb) into exclusive offsets (in place).
template <typename T>
__global__ void __launch_bounds__(kScanThreads)
ScanTileOffsets(T *tile_sums, int32_t nb) {
  __shared__ T smem[kScanThreads / 32];
  T running = Zero(T());
  for (int32_t base = 0; base < nb; base += kScanThreads) {
    int32_t i = base + threadIdx.x;
    T v = i < nb ? tile_sums[i] : Zero(T());
    T total;
    T inc = BlockInclusiveScan(v, smem, &total);
    if (i < nb) {
      T ex = Sub(Add(running, inc), v);  // exclusive = inclusive - own value
      tile_sums[i] = ex;
    }
    running = Add(running, total);
  }
}

// out[0..n] (n + 1 entries): exclusive sums, out[n] = grand total.
template <typename T>
__global__ void __launch_bounds__(kScanThreads)
ScanApply(const T *in, T *out, int64_t n, const T *__restrict__ tile_offsets) {
  __shared__ T smem[kScanThreads / 32];
  int64_t base = (int64_t)blockIdx.x * kScanTile + (int64_t)threadIdx.x * kScanItems;
  T vals[kScanItems];
  T acc = Zero(T());
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    vals[k] = (base + k < n) ? in[base + k] : Zero(T());
    acc = Add(acc, vals[k]);
  }
  T total;
  T inc = BlockInclusiveScan(acc, smem, &total);
  // exclusive prefix of this thread = tile offset + inclusive - own sum
  T run = Sub(Add(tile_offsets[blockIdx.x], inc), acc);
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    if (base + k <= n) out[base + k] = run;
    run = Add(run, vals[k]);
  }
}

size_t ScanTmpInts(int64_t n) { return (size_t)((n + 1 + kScanTile - 1) / kScanTile) + 1; }

template <typename T>
static int32_t ExclusiveSumImpl(const T *in, T *out, int64_t n, T *tmp, cudaStream_t stream) {
  if (n < 0) {
    SetError("ExclusiveSum: negative length");
    return kInvalidArgument;
  }
  int64_t nb64 = (n + 1 + kScanTile - 1) / kScanTile;
  if (nb64 > 0x7fffffff) {
    SetError("ExclusiveSum: too many elements");
    return kTooLarge;
  }
  int32_t nb = (int32_t)nb64;
  { ScanTileSums<T><<<nb, kScanThreads, 0, stream>>>(in, n, tmp); NoteLaunch(); }
  { ScanTileOffsets<T><<<1, kScanThreads, 0, stream>>>(tmp, nb); NoteLaunch(); }
  { ScanApply<T><<<nb, kScanThreads, 0, stream>>>(in, out, n, tmp); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t ExclusiveSum(const int32_t *in, int32_t *out, int64_t n, int32_t *tmp,
                     cudaStream_t stream) {
  return ExclusiveSumImpl<int32_t>(in, out, n, tmp, stream);
}
int32_t ExclusiveSum2(const int2 *in, int2 *out, int64_t n, int2 *tmp, cudaStream_t stream) {
  return ExclusiveSumImpl<int2>(in, out, n, tmp, stream);
}

// ----------------------------------------------------------------------------
// Exclusive sum that needs no memory from the caller beyond input and output.
//
// Some users of this library cannot hand it a scratch buffer: a C or C++ host
// that drives the kernels itself (no tensor library with a caching allocator
// behind it), or a service whose device memory was carved up once at start-up and
// must not grow - there a cudaMalloc in the request path is either unavailable
// or an unwanted device-wide synchronisation.  For them the tile sums of the
// scan live in the fixed array below, which every GPU that loads the library
// keeps for the lifetime of the process (kStaticScanTiles * 4 bytes = 64 KB).
//
// kStaticScanTiles tiles of kScanTile elements bound the input length.
// ----------------------------------------------------------------------------
constexpr int kStaticScanTiles = 16384;
static __device__ __align__(256) int32_t g_static_scan_tiles[kStaticScanTiles + 1];

constexpr int kMaxDevices = 64;
static std::mutex g_static_scan_mutex;
static int32_t *g_static_scan_ptr[kMaxDevices] = {nullptr};

int64_t ExclusiveSumStaticMaxLen() { return (int64_t)kStaticScanTiles * kScanTile - 1; }

// Device address of the array on the current device.  `g_static_scan_tiles` named
// in host code is only a handle for the runtime, not an address a kernel could
// use, so it is translated once per device with cudaGetSymbolAddress.
static int32_t StaticScanScratch(int32_t **ptr) {
  int dev = -1;
  K2B_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    SetError("device ordinal %d out of range", dev);
    return kInvalidArgument;
  }
  std::lock_guard<std::mutex> lock(g_static_scan_mutex);
  if (g_static_scan_ptr[dev] == nullptr) {
    void *p = nullptr;
    K2B_CUDA_OK(cudaGetSymbolAddress(&p, g_static_scan_tiles));
    g_static_scan_ptr[dev] = reinterpret_cast<int32_t *>(p);
  }
  *ptr = g_static_scan_ptr[dev];
  return kOk;
}

int32_t ExclusiveSumStatic(const int32_t *in, int32_t *out, int64_t n, cudaStream_t stream) {
  if (n < 0 || n > ExclusiveSumStaticMaxLen()) {
    SetError("k2b200_exclusive_sum_static: n = %lld is outside [0, %lld]; use "
             "k2b200_exclusive_sum with a caller-provided scratch buffer for longer inputs",
             (long long)n, (long long)ExclusiveSumStaticMaxLen());
    return kTooLarge;
  }
  int32_t *scratch = nullptr;
  K2B_FORWARD(StaticScanScratch(&scratch));
  // every tile sum that is read is written first by ScanTileSums of this call,
  // so nothing left over from an earlier call needs clearing
  return ExclusiveSumImpl<int32_t>(in, out, n, scratch, stream);
}

// ----------------------------------------------------------------------------
// row_splits -> row_ids by binary search per element
// ----------------------------------------------------------------------------
__global__ void RowIdsKernel(const int32_t *__restrict__ row_splits, int32_t num_rows,
                             int32_t *__restrict__ row_ids, int32_t num_elems) {
  int32_t k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= num_elems) return;
  int32_t lo = 0, hi = num_rows;  // find largest r with row_splits[r] <= k
  while (hi - lo > 1) {
    int32_t mid = (lo + hi) >> 1;
    if (row_splits[mid] <= k) lo = mid; else hi = mid;
  }
  row_ids[k] = lo;
}

int32_t RowSplitsToRowIds(const int32_t *row_splits, int32_t num_rows, int32_t *row_ids,
                          int32_t num_elems, cudaStream_t stream) {
  if (num_elems <= 0) return kOk;
  { RowIdsKernel<<<CeilDiv(num_elems, 256), 256, 0, stream>>>(row_splits, num_rows, row_ids,
                                                            num_elems); NoteLaunch(); }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

// ----------------------------------------------------------------------------
// incoming-arc index: count -> exclusive sum -> scatter (atomic cursor) -> sort
// every bucket by arc index so the result does not depend on scheduling.
// ----------------------------------------------------------------------------
__global__ void IncomingCount(const int32_t *__restrict__ row_splits1,
                              const int32_t *__restrict__ row_ids1,
                              const int32_t *__restrict__ row_ids2, const Arc *__restrict__ arcs,
                              int32_t num_arcs, int32_t *__restrict__ counts) {
  int32_t a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= num_arcs) return;
  int32_t fsa = row_ids1[row_ids2[a]];
  atomicAdd(&counts[row_splits1[fsa] + arcs[a].dest], 1);
}

__global__ void IncomingFill(const int32_t *__restrict__ row_splits1,
                             const int32_t *__restrict__ row_ids1,
                             const int32_t *__restrict__ row_ids2, const Arc *__restrict__ arcs,
                             int32_t num_arcs, const int32_t *__restrict__ in_splits,
                             int32_t *__restrict__ cursor, int32_t *__restrict__ unsorted) {
  int32_t a = blockIdx.x * blockDim.x + threadIdx.x;
  if (a >= num_arcs) return;
  int32_t fsa = row_ids1[row_ids2[a]];
  int32_t d = row_splits1[fsa] + arcs[a].dest;
  int32_t pos = atomicAdd(&cursor[d], 1);
  unsorted[in_splits[d] + pos] = a;
}

constexpr int kSmallBucket = 8;    // sorted by one thread
constexpr int kMediumBucket = 64;  // sorted by one warp with shuffles, two keys per lane

// One thread per state: rank sort of buckets of at most kSmallBucket arcs; larger
// buckets are queued in `large` (count in large[num_states]) for the warp kernel.
// in_src / in_score (optional) receive the source state (idx01) and the score of
// every arc in incoming order, so that forward recursions read them contiguously.
__global__ void IncomingSortSmall(const int32_t *__restrict__ in_splits, int32_t num_states,
                                  const int32_t *__restrict__ unsorted,
                                  const int32_t *__restrict__ row_ids2,
                                  const Arc *__restrict__ arcs, int32_t *__restrict__ in_arcs,
                                  int32_t *__restrict__ in_src, float *__restrict__ in_score,
                                  int32_t *__restrict__ large) {
  int32_t s = blockIdx.x * blockDim.x + threadIdx.x;
  int32_t b = 0, n = 0;
  if (s < num_states) {
    b = in_splits[s];
    n = in_splits[s + 1] - b;
  }
  // queue the larger buckets, one atomic per warp
  const bool queue = n > kSmallBucket;
  const unsigned qmask = __ballot_sync(0xffffffffu, queue);
  if (qmask) {
    const int lane = threadIdx.x & 31, leader = __ffs(qmask) - 1;
    int32_t base = 0;
    if (lane == leader) base = atomicAdd(&large[num_states], __popc(qmask));
    base = __shfl_sync(0xffffffffu, base, leader);
    if (queue) large[base + __popc(qmask & ((1u << lane) - 1u))] = s;
  }
  if (queue || s >= num_states) return;
  for (int32_t i = 0; i < n; ++i) {
    int32_t x = unsorted[b + i], rank = 0;
    for (int32_t j = 0; j < n; ++j) rank += (unsorted[b + j] < x);
    in_arcs[b + rank] = x;
    if (in_src) in_src[b + rank] = row_ids2[x];
    if (in_score) in_score[b + rank] = arcs[x].score;
  }
}

// One warp per queued state.  Buckets of up to kMediumBucket arcs are ranked with
// shuffles (each lane holds two keys and compares them with every other key);
// larger ones by reading the bucket from memory once per key.
__global__ void IncomingSortLarge(const int32_t *__restrict__ in_splits, int32_t num_states,
                                  const int32_t *__restrict__ unsorted,
                                  const int32_t *__restrict__ row_ids2,
                                  const Arc *__restrict__ arcs, int32_t *__restrict__ in_arcs,
                                  int32_t *__restrict__ in_src, float *__restrict__ in_score,
                                  const int32_t *__restrict__ large) {
  const int32_t nwarps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int32_t nlarge = large[num_states];
  for (int32_t e = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; e < nlarge; e += nwarps) {
    const int32_t s = large[e];
    const int32_t b = in_splits[s], n = in_splits[s + 1] - b;
    if (n <= kMediumBucket) {
      const int32_t big = 0x7fffffff;
      const int32_t x0 = lane < n ? unsorted[b + lane] : big;
      const int32_t x1 = lane + 32 < n ? unsorted[b + lane + 32] : big;
      int32_t r0 = 0, r1 = 0;
#pragma unroll 8
      for (int j = 0; j < 32; ++j) {
        const int32_t y0 = __shfl_sync(0xffffffffu, x0, j), y1 = __shfl_sync(0xffffffffu, x1, j);
        r0 += (y0 < x0) + (y1 < x0);
        r1 += (y0 < x1) + (y1 < x1);
      }
      if (lane < n) {
        in_arcs[b + r0] = x0;
        if (in_src) in_src[b + r0] = row_ids2[x0];
        if (in_score) in_score[b + r0] = arcs[x0].score;
      }
      if (lane + 32 < n) {
        in_arcs[b + r1] = x1;
        if (in_src) in_src[b + r1] = row_ids2[x1];
        if (in_score) in_score[b + r1] = arcs[x1].score;
      }
      continue;
    }
    for (int32_t i = lane; i < n; i += 32) {
      int32_t x = unsorted[b + i], rank = 0;
      for (int32_t j = 0; j < n; ++j) rank += (unsorted[b + j] < x);
      in_arcs[b + rank] = x;
      if (in_src) in_src[b + rank] = row_ids2[x];
      if (in_score) in_score[b + rank] = arcs[x].score;
    }
  }
}

size_t IncomingTmpBytes(int32_t num_states, int32_t num_arcs) {
  // counts/cursor [S+1], unsorted [A], scan tmp
  return AlignUp(sizeof(int32_t) * ((size_t)num_states + 1)) +
         AlignUp(sizeof(int32_t) * ((size_t)num_arcs + 1)) +
         AlignUp(sizeof(int32_t) * ScanTmpInts(num_states));
}

int32_t BuildIncoming(const int32_t *row_splits1, const int32_t *row_ids1,
                      const int32_t *row_ids2, const Arc *arcs, int32_t num_fsas,
                      int32_t num_states, int32_t num_arcs, int32_t *in_splits,
                      int32_t *in_arcs, int32_t *in_src, float *in_score, void *tmp,
                      cudaStream_t stream) {
  (void)num_fsas;
  char *p = reinterpret_cast<char *>(tmp);
  int32_t *counts = reinterpret_cast<int32_t *>(p);
  p += AlignUp(sizeof(int32_t) * ((size_t)num_states + 1));
  int32_t *unsorted = reinterpret_cast<int32_t *>(p);
  p += AlignUp(sizeof(int32_t) * ((size_t)num_arcs + 1));
  int32_t *scan_tmp = reinterpret_cast<int32_t *>(p);

  K2B_CUDA_OK(cudaMemsetAsync(counts, 0, sizeof(int32_t) * ((size_t)num_states + 1), stream));
  if (num_arcs > 0)
    { IncomingCount<<<CeilDiv(num_arcs, 256), 256, 0, stream>>>(row_splits1, row_ids1, row_ids2,
                                                              arcs, num_arcs, counts); NoteLaunch(); }
  K2B_FORWARD(ExclusiveSum(counts, in_splits, num_states, scan_tmp, stream));
  if (num_arcs > 0) {
    K2B_CUDA_OK(cudaMemsetAsync(counts, 0, sizeof(int32_t) * ((size_t)num_states + 1), stream));
    { IncomingFill<<<CeilDiv(num_arcs, 256), 256, 0, stream>>>(row_splits1, row_ids1, row_ids2,
                                                             arcs, num_arcs, in_splits, counts,
                                                             unsorted); NoteLaunch(); }
    // the cursor array is free again: it becomes the queue of large buckets
    K2B_CUDA_OK(cudaMemsetAsync(counts + num_states, 0, sizeof(int32_t), stream));
    { IncomingSortSmall<<<CeilDiv(num_states, 256), 256, 0, stream>>>(
        in_splits, num_states, unsorted, row_ids2, arcs, in_arcs, in_src, in_score, counts);
      NoteLaunch(); }
    { IncomingSortLarge<<<148 * 8, 256, 0, stream>>>(in_splits, num_states, unsorted, row_ids2, arcs,
                                                in_arcs, in_src, in_score, counts);
      NoteLaunch(); }
  }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

}  // namespace k2b

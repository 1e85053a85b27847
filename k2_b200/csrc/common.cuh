// Shared declarations of the k2-b200 CUDA library: error reporting, the 16-byte
// Arc (same layout as k2's, k2/csrc/fsa.h:31-63) and small device helpers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

namespace k2b {

struct __align__(16) Arc {
  int32_t src;    // source state, relative to the first state of its FSA
  int32_t dest;   // destination state, likewise
  int32_t label;  // -1 = final symbol, 0 = blank/epsilon
  float score;
};
static_assert(sizeof(Arc) == 16, "Arc must be 16 bytes");

// Status codes returned by every entry point of the C-ABI.
enum Status : int32_t {
  kOk = 0,
  kInvalidArgument = 1,
  kCudaError = 2,
  kWorkspaceTooSmall = 3,
  kTooLarge = 4,
};

void SetError(const char *fmt, ...);
const char *LastError();

// Log lines on stderr, filtered by the environment variable K2_LOG_LEVEL (TRACE, DEBUG, INFO,
// WARNING, ERROR or FATAL; default INFO), as the reference's logger (k2/csrc/log.h:297-352).
// The library logs rare events only - a beam reduction, a graph sent to a fallback kernel,
// a bounded wait that gave up - never anything per call on the usual path.
enum LogLevel : int { kLogTrace = 0, kLogDebug, kLogInfo, kLogWarning, kLogError, kLogFatal };
bool LogEnabled(LogLevel level);
void LogLine(LogLevel level, const char *fmt, ...);
#define K2B_LOG(level, ...)                                             \
  do {                                                                  \
    if (::k2b::LogEnabled(level)) ::k2b::LogLine(level, __VA_ARGS__);   \
  } while (0)

#define K2B_CUDA_OK(expr)                                                      \
  do {                                                                         \
    cudaError_t e__ = (expr);                                                  \
    if (e__ != cudaSuccess) {                                                  \
      ::k2b::SetError("%s:%d: %s failed: %s", __FILE__, __LINE__, #expr,       \
                      cudaGetErrorString(e__));                                \
      return ::k2b::kCudaError;                                                \
    }                                                                          \
  } while (0)

#define K2B_REQUIRE(cond, ...)            \
  do {                                    \
    if (!(cond)) {                        \
      ::k2b::SetError(__VA_ARGS__);       \
      return ::k2b::kInvalidArgument;     \
    }                                     \
  } while (0)

#define K2B_FORWARD(expr)                 \
  do {                                    \
    int32_t s__ = (expr);                 \
    if (s__ != ::k2b::kOk) return s__;    \
  } while (0)

// Bookkeeping for benchmarks: number of kernels this library has launched, and
// optional cudaEvent timing of named phases on the launching stream.
void NoteLaunch(int n = 1);
enum Phase : int { kPhaseViterbi = 0, kPhasePrune, kPhaseEmit, kPhaseScores, kPhasePost,
                   kPhaseIncoming, kPhaseDense, kPhaseChain, kPhaseGrad, kNumPhases };
long long LaunchCount();
// Name of the kernel(s) that last ran under a phase, for whoever reads the phase times.
void NotePhaseKernel(int phase, const char *name);
const char *PhaseKernel(int phase);
// Polls of an mbarrier before a kernel's wait for a copy gives up (a test hook lowers it:
// k2b200_debug_set_copy_wait_limit).
int32_t CopyWaitLimit();
void SetCopyWaitLimit(int32_t polls);
void SetProfiling(bool on);
double ReadPhase(int phase, long long *count);
struct PhaseTimer {  // records start/stop events when profiling is enabled
  PhaseTimer(int phase, cudaStream_t stream);
  ~PhaseTimer();
  int phase_;
  cudaStream_t stream_;
  int slot_;
};

// A second stream per device for kernels that do not depend on what the caller's
// stream is running (they fill the SMs that a latency-bound recursion leaves mostly
// idle).  SideFork makes the side stream wait for everything enqueued on `main` so
// far and returns it; SideJoin makes `main` wait for the side stream.  Both are
// plain event record/wait pairs, so they are also legal under stream capture.
int32_t SideFork(cudaStream_t main, cudaStream_t *side);
int32_t SideJoin(cudaStream_t main);
// device -> host copy of a few bytes behind the side stream's work; blocks the host
// until it (and not the main stream) is done
int32_t SideReadBack(const void *device_src, size_t bytes, void *host_out);
// The same in two steps: Begin queues the copy behind what the side stream has been given
// so far, End waits for it on the host - so that work queued on the side stream in between
// does not delay the answer.  One read-back at a time per process (the scope holds a lock).
struct SideReadBackScope {
  SideReadBackScope() = default;
  ~SideReadBackScope();
  int32_t Begin(const void *device_src, size_t bytes);
  int32_t End(void *host_out);
  size_t bytes_ = 0;
  bool held_ = false;
};

static inline size_t AlignUp(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

static inline int CeilDiv(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

// ---- generic ragged primitives (ragged_ops.cu) --------------------------------
// Exclusive prefix sum of n int32 values into out[0..n] (out[n] = total).  `tmp`
// must hold ScanTmpInts(n) int32.  in and out may alias.
size_t ScanTmpInts(int64_t n);
int32_t ExclusiveSum(const int32_t *in, int32_t *out, int64_t n, int32_t *tmp,
                     cudaStream_t stream);
// Variant whose scratch is a fixed array inside the library (no caller memory).
int64_t ExclusiveSumStaticMaxLen();
int32_t ExclusiveSumStatic(const int32_t *in, int32_t *out, int64_t n, cudaStream_t stream);
// Same for two interleaved counters (x, y) at once.
int32_t ExclusiveSum2(const int2 *in, int2 *out, int64_t n, int2 *tmp,
                      cudaStream_t stream);
// row_ids[k] = the row r with row_splits[r] <= k < row_splits[r+1].
int32_t RowSplitsToRowIds(const int32_t *row_splits, int32_t num_rows,
                          int32_t *row_ids, int32_t num_elems,
                          cudaStream_t stream);

// n host integers -> device memory as kernel parameters (no copy engine, no sync).
int32_t UploadInts(const int32_t *host, int64_t n, int32_t *device_out, cudaStream_t stream);

// Incoming-arc index of an FsaVec: for every state (idx01) the arcs (idx012) that
// enter it, in increasing arc order.
//   in_splits [num_states + 1], in_arcs [num_arcs]; optional in_src [num_arcs]
//   (source state idx01) and in_score [num_arcs] in the same order
// workspace: IncomingTmpBytes(num_states, num_arcs).
size_t IncomingTmpBytes(int32_t num_states, int32_t num_arcs);
int32_t BuildIncoming(const int32_t *row_splits1, const int32_t *row_ids1,
                      const int32_t *row_ids2, const Arc *arcs, int32_t num_fsas,
                      int32_t num_states, int32_t num_arcs, int32_t *in_splits,
                      int32_t *in_arcs, int32_t *in_src, float *in_score, void *tmp,
                      cudaStream_t stream);

}  // namespace k2b

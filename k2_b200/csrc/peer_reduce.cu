// Sum of a rank's per-utterance losses and the all-reduce of (loss, frames) over the GPUs of
// one node, in ONE kernel over peer memory: the sum
//   loss = -sum(tot_scores)                      k2/python/k2/ctc_loss.py:72-84
// followed by what a data-parallel trainer does with it, the all-reduce of (loss, frames)
// that normalises the step's loss over all ranks.  Utterances are independent, so this
// 16-byte exchange is the only collective of the path.
//
// Every rank owns a small buffer in its own memory that all ranks of the node map
// (cudaIpc*): slots[parity][sender].  A launch sums its values, writes (loss, frames, seq)
// into ITS slot of EVERY rank's buffer - plain stores over NVLink, data first, then the
// sequence number with release semantics - and then waits, reading only its own memory,
// until every sender's slot of this parity carries this call's sequence number; the totals
// are added in rank order, so every rank gets the same bits.  Two parities suffice: a rank
// cannot start call k + 2 before every rank has finished reading call k, because call
// k + 1 waits for every rank's k + 1.
//
// The wait is bounded: after poll_limit polls the kernel sets bit 0 of the status word,
// returns what it has (the result is then invalid), and nothing hangs or traps.
#include <cstdint>
#include <cstring>

#include "../../include/k2b200.h"
#include "common.cuh"

namespace k2b {

constexpr int kMaxPeers = 16;
constexpr int kPeerThreads = 256;

struct __align__(32) PeerSlot {
  double loss, frames;
  unsigned long long seq;
  unsigned long long pad;
};
// per rank: the slots, then the status word
constexpr size_t kPeerBufBytes = sizeof(PeerSlot) * 2 * kMaxPeers + 256;

struct PeerBufs {
  PeerSlot *buf[kMaxPeers];  // buf[r] = rank r's buffer as mapped in this process
};

__device__ __forceinline__ unsigned long long LoadAcquireSys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void StoreReleaseSys(unsigned long long *p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kPeerThreads)
LossSumAllReduce(const T *__restrict__ values, int32_t n, double sign, double frames,
                 PeerBufs peers, int32_t rank, int32_t world, unsigned long long seq,
                 int32_t poll_limit, double *__restrict__ out, int32_t *__restrict__ status) {
  __shared__ double part[kPeerThreads / 32];
  __shared__ double got[kMaxPeers][2];
  __shared__ double mine;
  const int tid = threadIdx.x;
  // ---- this rank's sum, in a fixed order -----------------------------------------------
  double s = 0.0;
  for (int32_t k = tid; k < n; k += kPeerThreads) s += (double)values[k];
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) s += __shfl_down_sync(0xffffffffu, s, d);
  if ((tid & 31) == 0) part[tid >> 5] = s;
  __syncthreads();
  if (tid == 0) {
    double t = 0.0;
    for (int k = 0; k < kPeerThreads / 32; ++k) t += part[k];
    mine = sign * t;
  }
  __syncthreads();
  const int parity = (int)(seq & 1ull);
  // ---- to every rank's buffer (its own included) ------------------------------------------
  if (tid < world) {
    PeerSlot *dst = peers.buf[tid] + parity * kMaxPeers + rank;
    dst->loss = mine;
    dst->frames = frames;
    StoreReleaseSys(&dst->seq, seq);
  }
  // ---- from every rank, out of this rank's own memory -------------------------------------
  if (tid < world) {
    const PeerSlot *src = peers.buf[rank] + parity * kMaxPeers + tid;
    bool ok = false;
    for (int32_t k = 0; k < poll_limit; ++k) {
      if (LoadAcquireSys(&src->seq) == seq) {
        ok = true;
        break;
      }
      __nanosleep(100);
    }
    if (!ok) atomicOr(status, 1);
    got[tid][0] = ok ? src->loss : 0.0;
    got[tid][1] = ok ? src->frames : 0.0;
  }
  __syncthreads();
  if (tid == 0) {
    double l = 0.0, f = 0.0;
    for (int r = 0; r < world; ++r) {
      l += got[r][0];
      f += got[r][1];
    }
    out[0] = l;
    out[1] = f;
  }
}

// One event per device and host thread for ordering a launch behind another stream (a wait
// takes the event's state at the time of the call, so the event is reused right away).
int32_t ForkEvent(cudaEvent_t *ev) {
  constexpr int kMaxDevices = 64;
  thread_local cudaEvent_t events[kMaxDevices] = {nullptr};
  int dev = 0;
  K2B_CUDA_OK(cudaGetDevice(&dev));
  K2B_REQUIRE(dev >= 0 && dev < kMaxDevices, "device ordinal %d", dev);
  if (events[dev] == nullptr)
    K2B_CUDA_OK(cudaEventCreateWithFlags(&events[dev], cudaEventDisableTiming));
  *ev = events[dev];
  return kOk;
}

}  // namespace k2b

using namespace k2b;

extern "C" {

int32_t k2b200_peer_reduce_create(void **local_buf, void *ipc_handle_out) {
  K2B_REQUIRE(local_buf && ipc_handle_out, "NULL output pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == K2B200_IPC_HANDLE_BYTES, "handle size");
  void *p = nullptr;
  K2B_CUDA_OK(cudaMalloc(&p, kPeerBufBytes));
  K2B_CUDA_OK(cudaMemset(p, 0, kPeerBufBytes));
  K2B_CUDA_OK(cudaDeviceSynchronize());  // zero before any peer can see the handle
  cudaIpcMemHandle_t h;
  K2B_CUDA_OK(cudaIpcGetMemHandle(&h, p));
  memcpy(ipc_handle_out, &h, sizeof(h));
  *local_buf = p;
  return kOk;
}

int32_t k2b200_peer_reduce_open(const void *ipc_handle, void **peer_buf) {
  K2B_REQUIRE(ipc_handle && peer_buf, "NULL pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle, sizeof(h));
  K2B_CUDA_OK(cudaIpcOpenMemHandle(peer_buf, h, cudaIpcMemLazyEnablePeerAccess));
  return kOk;
}

int32_t k2b200_peer_reduce_close(void *peer_buf) {
  if (peer_buf) K2B_CUDA_OK(cudaIpcCloseMemHandle(peer_buf));
  return kOk;
}

int32_t k2b200_peer_reduce_destroy(void *local_buf) {
  if (local_buf) K2B_CUDA_OK(cudaFree(local_buf));
  return kOk;
}

int32_t k2b200_loss_sum_all_reduce(const void *values, int32_t n, int32_t values_are_f32,
                                   double sign, double num_frames, void *const *bufs,
                                   int32_t rank, int32_t world, uint64_t seq,
                                   int32_t poll_limit, double *out, void *stream_v,
                                   void *after_stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  cudaStream_t after = reinterpret_cast<cudaStream_t>(after_stream_v);
  K2B_REQUIRE(values && bufs && out, "NULL pointer");
  K2B_REQUIRE(world >= 1 && world <= kMaxPeers, "world size %d outside 1..%d", world, kMaxPeers);
  K2B_REQUIRE(rank >= 0 && rank < world, "rank %d outside the world of %d", rank, world);
  K2B_REQUIRE(n >= 0 && seq >= 1, "n must be >= 0 and seq >= 1");
  PeerBufs peers;
  for (int r = 0; r < kMaxPeers; ++r) peers.buf[r] = nullptr;
  for (int r = 0; r < world; ++r) {
    K2B_REQUIRE(bufs[r] != nullptr, "buffer of rank %d is NULL", r);
    peers.buf[r] = reinterpret_cast<PeerSlot *>(bufs[r]);
  }
  int32_t *status = reinterpret_cast<int32_t *>(reinterpret_cast<char *>(bufs[rank]) +
                                                sizeof(PeerSlot) * 2 * kMaxPeers);
  if (poll_limit < 0) poll_limit = 20000000;  // a few seconds
  if (after != nullptr && after != stream) {
    // behind what `after` holds now (the kernels that produce `values`)
    cudaEvent_t ev = nullptr;
    K2B_FORWARD(ForkEvent(&ev));
    K2B_CUDA_OK(cudaEventRecord(ev, after));
    K2B_CUDA_OK(cudaStreamWaitEvent(stream, ev, 0));
  }
  if (values_are_f32) {
    LossSumAllReduce<float><<<1, kPeerThreads, 0, stream>>>(
        reinterpret_cast<const float *>(values), n, sign, num_frames, peers, rank, world,
        (unsigned long long)seq, poll_limit, out, status);
  } else {
    LossSumAllReduce<double><<<1, kPeerThreads, 0, stream>>>(
        reinterpret_cast<const double *>(values), n, sign, num_frames, peers, rank, world,
        (unsigned long long)seq, poll_limit, out, status);
  }
  NoteLaunch();
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

int32_t k2b200_peer_reduce_status(void *local_buf, void *stream_v, int32_t *status) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  K2B_REQUIRE(local_buf && status, "NULL pointer");
  K2B_CUDA_OK(cudaMemcpyAsync(status,
                              reinterpret_cast<char *>(local_buf) + sizeof(PeerSlot) * 2 * kMaxPeers,
                              sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  K2B_CUDA_OK(cudaStreamSynchronize(stream));
  return kOk;
}

}  // extern "C"

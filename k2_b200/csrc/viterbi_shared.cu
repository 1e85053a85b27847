// Viterbi recursion for ONE large graph shared by all sequences of the batch (a decoding
// graph stacked once per sequence and read through its first copy): the reference's
// forward / backward passes, k2/csrc/intersect_dense.cu:778-847, one launch per frame.
//
// With one thread per (sequence, state) every arc costs a 4-byte gather of the other
// end's score and a 4-byte gather of the dense score, each its own 32-byte sector; for a
// 200 000-state graph and 32 sequences that is L2-sector bound.  The graph is the same
// for every sequence, so here a warp takes one state and its 32 LANES are 32 SEQUENCES:
// the arcs are read once per warp, and the scores of the other end of an arc for the 32
// sequences are one 128-byte line of a [state][sequence] copy of the previous level; the
// dense scores of a label for the 32 sequences are one line of a [row][label][sequence]
// copy of the dense matrix, made once per call.  A CTA handles 32 states: the results
// go to the [state][sequence] buffer for the next step directly and, through a 32 x 32 tile
// in shared memory, to the caller's [sequence][level][state] grids with 128-byte lines as
// well.  Same fp32 expression as everywhere, (other + arc.score) + dense, and max is order
// independent: the grids are bit-identical to those of the other Viterbi kernels.
#include <algorithm>

#include "../../include/k2b200.h"
#include "common.cuh"
#include "intersect_internal.cuh"

namespace k2b {

constexpr int kSharedStates = 32;   // states per CTA
constexpr int kSharedThreads = 256;

constexpr int kHeavyDeg = 128;    // a state with more arcs than this (entering arcs walking forward,
                                  // leaving arcs walking backward) is split over many CTAs
constexpr int kHeavyChunk = 256;  // arcs of such a state per CTA

struct SharedPlan {
  int32_t groups, upad, tk_max, cap_states, cap_chunks;
  // relative to the region's start; the heavy lists are per direction:
  // counts[2] (states, chunks), states[cap_states], chunk_state[cap_chunks], chunk_begin[cap_chunks]
  size_t off_xt, off_dtf, off_dtb, off_heavy, heavy_stride, bytes;
};

static SharedPlan PlanShared(const Layout &L, const k2b200_intersect_args *a) {
  SharedPlan p;
  p.groups = (a->num_fsas + 31) / 32;
  p.upad = 32 * p.groups;
  p.tk_max = L.max_tk;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t o = off;
    off += AlignUp(bytes ? bytes : 1);
    return o;
  };
  // [direction][parity][group][state][32]
  p.off_xt = take(sizeof(float) * 2 * 2 * (size_t)p.upad * (size_t)L.max_states);
  // [step][column][sequence]: forward step t reads row t - 1 of every sequence, backward
  // step t reads row tk - t of every sequence
  p.off_dtf = take(sizeof(float) * (size_t)p.tk_max * (size_t)a->cols * (size_t)p.upad);
  p.off_dtb = take(sizeof(float) * (size_t)p.tk_max * (size_t)a->cols * (size_t)p.upad);
  p.cap_states = L.max_arcs / kHeavyDeg + 2;
  p.cap_chunks = L.max_arcs / kHeavyChunk + L.max_arcs / kHeavyDeg + 2;
  p.heavy_stride = AlignUp(sizeof(int32_t) * (4 + (size_t)p.cap_states + 2 * (size_t)p.cap_chunks));
  p.off_heavy = take(2 * p.heavy_stride);
  p.bytes = off;
  return p;
}

bool SharedViterbiApplies(const Layout &L, const k2b200_intersect_args *a) {
  if (!a->a_shared || a->num_fsas < 2 || L.max_states < 1) return false;
  const SharedPlan p = PlanShared(L, a);
  return p.bytes < ((size_t)8 << 30);
}

size_t SharedViterbiBytes(const Layout &L, const k2b200_intersect_args *a) {
  return SharedViterbiApplies(L, a) ? PlanShared(L, a).bytes : 0;
}

// dtf[(t * cols + c) * upad + u] = scores[(row0_u + t) * cols + c]            (t < tk_u)
// dtb[(t * cols + c) * upad + u] = scores[(row0_u + tk_u - 1 - t) * cols + c]  (t < tk_u)
// and -inf where the sequence has no such row.
__global__ void SharedDenseTranspose(const FsaInfo *__restrict__ infos, int32_t n, int32_t upad,
                                     int32_t tk_max, const float *__restrict__ scores,
                                     int32_t cols, float *__restrict__ dtf,
                                     float *__restrict__ dtb) {
  const int64_t total = (int64_t)tk_max * cols * upad;
  for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < total;
       k += (int64_t)gridDim.x * blockDim.x) {
    const int32_t u = (int32_t)(k % upad);
    const int64_t tc = k / upad;
    const int32_t c = (int32_t)(tc % cols), t = (int32_t)(tc / cols);
    float vf = -INFINITY, vb = -INFINITY;
    if (u < n) {
      const FsaInfo f = infos[u];
      if (t < f.tk) {
        vf = __ldg(scores + ((int64_t)f.row0 + t) * cols + c);
        vb = __ldg(scores + ((int64_t)f.row0 + f.tk - 1 - t) * cols + c);
      }
    }
    dtf[k] = vf;
    dtb[k] = vb;
  }
}

// level 0 of the forward pass (state 0 scores 0) and the last level of the backward pass
// (the final state scores 0), in both layouts
__global__ void SharedViterbiInit(const FsaInfo *__restrict__ infos, int32_t n, int32_t upad,
                                  int32_t S, float *__restrict__ xt, float *__restrict__ fwd,
                                  float *__restrict__ bwd) {
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= (int64_t)S * upad) return;
  const int32_t u = (int32_t)(k % upad), s = (int32_t)(k / upad);
  const int32_t g = u >> 5, lane = u & 31;
  const float vf = s == 0 ? 0.0f : -INFINITY, vb = s == S - 1 ? 0.0f : -INFINITY;
  // xt[((dir * 2 + parity) * groups + g) * S * 32 + s * 32 + lane], parity 0
  const int64_t groups = upad >> 5;
  xt[((int64_t)(0 * 2 + 0) * groups + g) * S * 32 + (int64_t)s * 32 + lane] = vf;
  xt[((int64_t)(1 * 2 + 0) * groups + g) * S * 32 + (int64_t)s * 32 + lane] = vb;
  if (u < n) {
    const FsaInfo f = infos[u];
    fwd[f.grid_off + s] = vf;
    bwd[f.grid_off + (int64_t)f.tk * S + s] = vb;
  }
}

// The states with more than kHeavyDeg arcs in a direction, and their arcs in chunks of
// kHeavyChunk (the order of the lists does not matter: a max is order independent).
__global__ void SharedHeavyList(const int32_t *__restrict__ splits, int32_t S, int32_t *__restrict__ counts,
                                int32_t *__restrict__ states, int32_t *__restrict__ chunk_state,
                                int32_t *__restrict__ chunk_begin) {
  const int32_t s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= S) return;
  const int32_t a0 = splits[s], deg = splits[s + 1] - a0;
  if (deg <= kHeavyDeg) return;
  states[atomicAdd(&counts[0], 1)] = s;
  const int32_t nch = (deg + kHeavyChunk - 1) / kHeavyChunk;
  const int32_t c0 = atomicAdd(&counts[1], nch);
  for (int32_t j = 0; j < nch; ++j) {
    chunk_state[c0 + j] = s;
    chunk_begin[c0 + j] = a0 + j * kHeavyChunk;
  }
}

__device__ __forceinline__ void AtomicMaxFloat(float *addr, float v) {
  // the integer order of the bit patterns is the float order for v >= 0 and its reverse below
  if (v >= 0.0f) atomicMax(reinterpret_cast<int *>(addr), __float_as_int(v));
  else atomicMin(reinterpret_cast<unsigned int *>(addr), __float_as_uint(v));
}

// One chunk of a heavy state's arcs per CTA, 32 arcs per warp; the partial maxima meet in the
// [state][sequence] buffer of the step (which the step kernel left at -inf for such states).
// grid = (chunk capacity, groups); CTAs beyond the list return at once.
__global__ void __launch_bounds__(kHeavyChunk)
SharedViterbiHeavy(const FsaInfo *__restrict__ infos, int32_t groups, int32_t t, int32_t dir,
                   const Arc *__restrict__ arcs, const int32_t *__restrict__ a_row_splits2,
                   const int32_t *__restrict__ in_splits, const int32_t *__restrict__ in_arcs,
                   int32_t cols, const float *__restrict__ dtf, const float *__restrict__ dtb,
                   float *__restrict__ xt, const int32_t *__restrict__ counts,
                   const int32_t *__restrict__ chunk_state, const int32_t *__restrict__ chunk_begin) {
  constexpr unsigned kAll = 0xffffffffu;
  if ((int32_t)blockIdx.x >= counts[1]) return;
  const int g = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const FsaInfo f0 = infos[0];
  const int32_t S = f0.num_states, upad = groups * 32, u = g * 32 + lane;
  const int32_t s = chunk_state[blockIdx.x];
  const int32_t *splits = (dir == 0 ? in_splits : a_row_splits2) + f0.state_off;
  const int32_t kb = chunk_begin[blockIdx.x] + 32 * warp;
  const int32_t ke = min(kb + 32, min(chunk_begin[blockIdx.x] + kHeavyChunk, splits[s + 1]));
  if (kb >= ke) return;  // uniform per warp
  const int parity = (t - 1) & 1;
  const float *prev = xt + ((int64_t)(dir * 2 + parity) * groups + g) * S * 32 + lane;
  float *cur = xt + ((int64_t)(dir * 2 + (parity ^ 1)) * groups + g) * S * 32 + lane;
  const float *dt = (dir == 0 ? dtf : dtb) + (int64_t)(t - 1) * cols * upad + u;
  const int32_t n_here = ke - kb;
  int4 mine = make_int4(0, 0, 0, 0);
  if (lane < n_here) {
    const int32_t idx = dir == 0 ? in_arcs[kb + lane] : kb + lane;
    mine = *reinterpret_cast<const int4 *>(arcs + idx);
  }
  float best = -INFINITY;
  constexpr int kRound = 8;
  for (int32_t j0 = 0; j0 < n_here; j0 += kRound) {
    float pv[kRound], xv[kRound], wv[kRound];
#pragma unroll
    for (int r = 0; r < kRound; ++r) {
      const int32_t j = min(j0 + r, n_here - 1);
      const int32_t other = __shfl_sync(kAll, dir == 0 ? mine.x : mine.y, j);
      const int32_t c = __shfl_sync(kAll, mine.z, j) + 1;
      wv[r] = __int_as_float(__shfl_sync(kAll, mine.w, j));
      xv[r] = (c >= 0 && c < cols) ? dt[(uint32_t)c * (uint32_t)upad] : -INFINITY;
      pv[r] = prev[(uint32_t)other * 32u];
    }
#pragma unroll
    for (int r = 0; r < kRound; ++r) {
      const float v = __fadd_rn(__fadd_rn(pv[r], wv[r]), xv[r]);
      best = v > best ? v : best;
    }
  }
  if (best != -INFINITY) AtomicMaxFloat(cur + (int64_t)s * 32, best);
}

// The heavy states' results into the caller's grids.  grid = (state capacity, groups), 32 threads.
__global__ void SharedHeavyStore(const FsaInfo *__restrict__ infos, int32_t n, int32_t groups,
                                 int32_t t, int32_t dir, const float *__restrict__ xt,
                                 const int32_t *__restrict__ counts,
                                 const int32_t *__restrict__ states, float *__restrict__ fwd,
                                 float *__restrict__ bwd) {
  if ((int32_t)blockIdx.x >= counts[0]) return;
  const int g = blockIdx.y, lane = threadIdx.x, u = g * 32 + lane;
  if (u >= n) return;
  const FsaInfo f = infos[u];
  if (t > f.tk) return;
  const int32_t S = f.num_states, s = states[blockIdx.x];
  const int parity = (t - 1) & 1;
  const float v = xt[((int64_t)(dir * 2 + (parity ^ 1)) * groups + g) * S * 32 + (int64_t)s * 32 + lane];
  (dir == 0 ? fwd : bwd)[f.grid_off + (int64_t)(dir == 0 ? t : f.tk - t) * S + s] = v;
}

// Step t (1 .. tk_max) of direction dir0 + blockIdx.z.  grid = (state tiles, groups of 32
// sequences, directions in this launch).
__global__ void __launch_bounds__(kSharedThreads, 4)
SharedViterbiStep(const FsaInfo *__restrict__ infos, int32_t n, int32_t groups, int32_t t,
                  int32_t dir0,
                  const Arc *__restrict__ arcs, const int32_t *__restrict__ a_row_splits2,
                  const int32_t *__restrict__ in_splits, const int32_t *__restrict__ in_arcs,
                  int32_t cols, const float *__restrict__ dtf, const float *__restrict__ dtb,
                  float *__restrict__ xt, float *__restrict__ fwd, float *__restrict__ bwd) {
  __shared__ float tile[kSharedStates][33];
  __shared__ long long out_off[32];  // per sequence: where this step's level starts, or -1
  constexpr unsigned kAll = 0xffffffffu;
  const int dir = dir0 + blockIdx.z, g = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int32_t u = g * 32 + lane;
  const FsaInfo f0 = infos[0];
  const int32_t S = f0.num_states, upad = groups * 32;
  const int32_t sb = blockIdx.x * kSharedStates;
  if (threadIdx.x < 32) {
    long long off = -1;
    if (u < n) {
      const FsaInfo f = infos[u];
      if (t <= f.tk) off = f.grid_off + (long long)(dir == 0 ? t : f.tk - t) * S;
    }
    out_off[lane] = off;
  }
  const int parity = (t - 1) & 1;
  const float *prev = xt + ((int64_t)(dir * 2 + parity) * groups + g) * S * 32 + lane;
  float *cur = xt + ((int64_t)(dir * 2 + (parity ^ 1)) * groups + g) * S * 32 + lane;
  const float *dt = (dir == 0 ? dtf : dtb) + (int64_t)(t - 1) * cols * upad + u;
  const int32_t *splits = (dir == 0 ? in_splits : a_row_splits2) + f0.state_off;
  // A warp takes kPerWarp consecutive states.  Their arcs (entering arcs walking forward,
  // leaving arcs walking backward) are ONE contiguous range of the graph's arc list or
  // incoming-arc index, which the lanes fetch 32 at a time with one coalesced load; then
  // every lane walks the arcs in order, kRound at a time with all gathers of a round issued
  // before any is used, and closes a state when the walk crosses into the next one.
  constexpr int kPerWarp = kSharedStates / (kSharedThreads / 32);  // 4
  constexpr int kRound = 8;
  const int32_t s4 = sb + warp * kPerWarp;
  int32_t sp = 0;
  if (lane <= kPerWarp) sp = splits[min(s4 + lane, S)];
  int32_t bound[kPerWarp + 1];  // bound[q] = first arc of state s4 + q
#pragma unroll
  for (int q = 0; q <= kPerWarp; ++q) bound[q] = __shfl_sync(kAll, sp, q);
  const int32_t A0 = bound[0], A1 = bound[kPerWarp];
  int32_t q_cur = 0;
  int32_t next = bound[1];
  float best = -INFINITY;
  auto close_state = [&]() {  // uniform
    if (s4 + q_cur < S) cur[(int64_t)(s4 + q_cur) * 32] = best;
    tile[warp * kPerWarp + q_cur][lane] = best;
    best = -INFINITY;
    ++q_cur;
    next = q_cur == 1 ? bound[2] : q_cur == 2 ? bound[3] : bound[4];
  };
  auto walk = [&](int32_t kb, int32_t ke) {  // the arcs kb .. ke - 1, in order
    for (int32_t k0 = kb; k0 < ke; k0 += 32) {
      const int32_t n_here = min(32, ke - k0);
      int4 mine = make_int4(0, 0, 0, 0);
      if (lane < n_here) {
        const int32_t idx = dir == 0 ? in_arcs[k0 + lane] : k0 + lane;
        mine = *reinterpret_cast<const int4 *>(arcs + idx);
      }
      for (int32_t j0 = 0; j0 < n_here; j0 += kRound) {
        float pv[kRound], xv[kRound], wv[kRound];
#pragma unroll
        for (int r = 0; r < kRound; ++r) {
          const int32_t j = min(j0 + r, n_here - 1);  // an arc taken twice does not change a max
          const int32_t other = __shfl_sync(kAll, dir == 0 ? mine.x : mine.y, j);
          const int32_t c = __shfl_sync(kAll, mine.z, j) + 1;
          wv[r] = __int_as_float(__shfl_sync(kAll, mine.w, j));
          xv[r] = (c >= 0 && c < cols) ? dt[(uint32_t)c * (uint32_t)upad] : -INFINITY;
          pv[r] = prev[(uint32_t)other * 32u];
        }
#pragma unroll
        for (int r = 0; r < kRound; ++r) {
          const int32_t k = k0 + min(j0 + r, n_here - 1);
          while (k >= next && q_cur < kPerWarp - 1) close_state();  // also states without arcs
          const float v = __fadd_rn(__fadd_rn(pv[r], wv[r]), xv[r]);
          best = v > best ? v : best;
        }
      }
    }
  };
  // A state with very many arcs would keep this warp busy long after the rest of the grid
  // has finished: its arcs are left out here (it comes out as -inf) and SharedViterbiHeavy,
  // launched behind this kernel, takes them with many CTAs.
  int32_t kb = A0;
#pragma unroll
  for (int q = 0; q < kPerWarp; ++q) {
    if (bound[q + 1] - bound[q] > kHeavyDeg) {  // uniform
      walk(kb, bound[q]);
      kb = bound[q + 1];
    }
  }
  walk(kb, A1);
  // the state the walk ended in, and any states without arcs behind it
  while (q_cur < kPerWarp - 1) close_state();
  if (s4 + q_cur < S) cur[(int64_t)(s4 + q_cur) * 32] = best;
  tile[warp * kPerWarp + q_cur][lane] = best;
  __syncthreads();
  // the caller's grids: one 128-byte line of 32 states per sequence
  for (int32_t ul = warp; ul < 32; ul += kSharedThreads / 32) {
    const long long off = out_off[ul];
    // written once, read much later by other kernels: streaming stores keep them from
    // evicting the [state][sequence] buffers from L2
    if (off >= 0 && sb + lane < S) __stcs((dir == 0 ? fwd : bwd) + off + sb + lane, tile[lane][ul]);
  }
}

int32_t LaunchSharedViterbi(const Layout &L, const k2b200_intersect_args *a, char *region,
                            const FsaInfo *d_infos, float *fwd, float *bwd,
                            cudaStream_t stream) {
  const SharedPlan p = PlanShared(L, a);
  const int32_t S = L.max_states;
  float *xt = reinterpret_cast<float *>(region + p.off_xt);
  float *dtf = reinterpret_cast<float *>(region + p.off_dtf);
  float *dtb = reinterpret_cast<float *>(region + p.off_dtb);
  { SharedDenseTranspose<<<148 * 8, 256, 0, stream>>>(d_infos, a->num_fsas, p.upad, p.tk_max,
                                                       a->scores, a->cols, dtf, dtb);
    NoteLaunch(); }
  { SharedViterbiInit<<<CeilDiv((int64_t)S * p.upad, 256), 256, 0, stream>>>(
        d_infos, a->num_fsas, p.upad, S, xt, fwd, bwd); NoteLaunch(); }
  K2B_CUDA_OK(cudaMemsetAsync(region + p.off_heavy, 0, 2 * p.heavy_stride, stream));
  const int32_t state_off = L.infos.empty() ? 0 : L.infos[0].state_off;
  int32_t *heavy[2], *h_states[2], *h_chunk_state[2], *h_chunk_begin[2];
  for (int dir = 0; dir < 2; ++dir) {
    heavy[dir] = reinterpret_cast<int32_t *>(region + p.off_heavy + dir * p.heavy_stride);
    h_states[dir] = heavy[dir] + 4;
    h_chunk_state[dir] = h_states[dir] + p.cap_states;
    h_chunk_begin[dir] = h_chunk_state[dir] + p.cap_chunks;
    { SharedHeavyList<<<CeilDiv(S, 256), 256, 0, stream>>>(
          (dir == 0 ? a->a_in_splits : a->a_row_splits2) + state_off, S, heavy[dir],
          h_states[dir], h_chunk_state[dir], h_chunk_begin[dir]); NoteLaunch(); }
  }
  // how many there are decides the grids of a thousand launches: worth one small read-back
  int32_t h_counts[2][4] = {};
  for (int dir = 0; dir < 2; ++dir)
    K2B_CUDA_OK(cudaMemcpyAsync(h_counts[dir], heavy[dir], sizeof(int32_t) * 4,
                                cudaMemcpyDeviceToHost, stream));
  K2B_CUDA_OK(cudaStreamSynchronize(stream));
  // one direction after the other: the working set of a direction (its two [state][sequence]
  // buffers and the graph) then fits in L2, which both together do not for large graphs
  dim3 grid(CeilDiv(S, kSharedStates), p.groups, 1);
  const Arc *arcs = reinterpret_cast<const Arc *>(a->a_arcs);
  for (int32_t dir = 0; dir < 2; ++dir)
    for (int32_t t = 1; t <= p.tk_max; ++t) {
      { SharedViterbiStep<<<grid, kSharedThreads, 0, stream>>>(
            d_infos, a->num_fsas, p.groups, t, dir, arcs, a->a_row_splits2, a->a_in_splits,
            a->a_in_arcs, a->cols, dtf, dtb, xt, fwd, bwd); NoteLaunch(); }
      if (h_counts[dir][0] == 0) continue;
      // the heavy states of this direction
      { SharedViterbiHeavy<<<dim3(h_counts[dir][1], p.groups), kHeavyChunk, 0, stream>>>(
            d_infos, p.groups, t, dir, arcs, a->a_row_splits2, a->a_in_splits, a->a_in_arcs,
            a->cols, dtf, dtb, xt, heavy[dir], h_chunk_state[dir], h_chunk_begin[dir]);
        NoteLaunch(); }
      { SharedHeavyStore<<<dim3(h_counts[dir][0], p.groups), 32, 0, stream>>>(
            d_infos, a->num_fsas, p.groups, t, dir, xt, heavy[dir], h_states[dir], fwd, bwd);
        NoteLaunch(); }
    }
  K2B_CUDA_OK(cudaGetLastError());
  return kOk;
}

}  // namespace k2b

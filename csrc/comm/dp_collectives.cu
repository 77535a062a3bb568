// Data-parallel collectives of the distributed optimizer over peer memory (NVLink / NVSwitch P2P loads):
//
//   mcb_dp_reduce_scatter_f32   every rank sums its shard of a gradient bucket over all ranks' fp32 gradient buffers
//                               (fixed rank order, so all runs and all ranks agree bit for bit), scales it and writes
//                               it in place into its own buffer
//   mcb_dp_all_gather           every rank copies the other ranks' shards of a parameter bucket into its own buffer
//
// Both take the same symmetric layout: one buffer per rank, a bucket at the same byte offset in each, shard `r` of the
// bucket owned by rank `r`.  A call is bracketed by two flag rounds in the ranks' signal pads: READY (my part of the
// bucket is final: stream order on the launching stream puts the producers before this kernel) before the first peer
// load, DONE (I have read everything I need from every peer) before the kernel returns, so that a peer may overwrite
// its buffer as soon as its own call has returned.  Every wait is bounded: on a time-out the kernel records
// ST_TIMEOUT_PEER_FLAG in the status word, skips the remaining work and returns.
//
// Flags carry the call's epoch (monotonically increasing per workspace), so they never need clearing.
#include <cuda_runtime.h>

#include "../common/ptx.cuh"

namespace mcb {
namespace {

constexpr int DP_MAX_WORLD = 8;
constexpr int DP_READY = 0;    // [world] flag words: rank s is ready for call `epoch`
constexpr int DP_DONE = 16;    // [world] rank s has finished reading for call `epoch`
constexpr int DP_TICKET = 32;  // local: CTAs that have finished their loads in this call
constexpr int AG_U = 8;         // 16-byte vectors a thread of the all-gather keeps in flight
constexpr int DP_THREADS = 256;  // small CTAs: they have to find room next to the compute kernels of the main stream

struct DpArgs {
  void* bufs[DP_MAX_WORLD];
  uint32_t* flags[DP_MAX_WORLD];
  long long offset_bytes;  // bucket start inside every rank's buffer (multiple of 16)
  long long shard_bytes;   // bytes per rank (multiple of 16)
  int world, rank;
  uint32_t epoch;
  float scale;
  int* status;
};

// publish `word + rank = epoch` in every peer's pad (one thread per peer)
__device__ __forceinline__ void dp_signal(const DpArgs& a, int word) {
  if (threadIdx.x < a.world && threadIdx.x != a.rank) st_release_sys(a.flags[threadIdx.x] + word + a.rank, a.epoch);
}

// thread s < world waits for peer s; returns false for the whole CTA when any wait ran out
__device__ __forceinline__ bool dp_wait(const DpArgs& a, int word, volatile int* abort_flag) {
  if (threadIdx.x < a.world && threadIdx.x != a.rank)
    wait_flag<SCOPE_SYS>(a.flags[a.rank] + word + threadIdx.x, a.epoch, false, abort_flag, a.status);
  __syncthreads();
  return *abort_flag == 0;
}

// The last CTA of the grid to finish its loads tells the peers that this rank is done with their buffers and then
// waits for theirs; the other CTAs just leave.  (Stores of this kernel only touch this rank's own shard, which no peer
// reads in this call.)
__device__ __forceinline__ void dp_finish(const DpArgs& a, volatile int* abort_flag) {
  __shared__ int last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t* ticket = a.flags[a.rank] + DP_TICKET;
    const uint32_t t = atomicAdd(ticket, 1u);
    last = (t == gridDim.x - 1);
    if (last) *ticket = 0;
  }
  __syncthreads();
  if (!last) return;
  fence_acq_rel_sys();
  dp_signal(a, DP_DONE);
  dp_wait(a, DP_DONE, abort_flag);
}

// W = world size known at compile time (0: read it from the arguments), U = 16-byte vectors per thread and iteration.
// A thread keeps U x (world - 1) peer loads in flight, which is what hides the NVLink round trip.
template <int W, int U>
__global__ void __launch_bounds__(DP_THREADS) dp_reduce_scatter_f32_kernel(const DpArgs a) {
  __shared__ int abort_flag;
  if (threadIdx.x == 0) abort_flag = (a.status && *reinterpret_cast<volatile int*>(a.status) != 0) ? 1 : 0;
  __syncthreads();
  if (abort_flag) return;
  if (blockIdx.x == 0) dp_signal(a, DP_READY);
  if (!dp_wait(a, DP_READY, &abort_flag)) return;
  constexpr int WM = W ? W : DP_MAX_WORLD;
  const int world = W ? W : a.world;
  const long long n4 = a.shard_bytes / 16;
  const long long base = (a.offset_bytes + (long long)a.rank * a.shard_bytes) / 16;
  const float4* src[WM];
#pragma unroll
  for (int s = 0; s < WM; ++s) src[s] = reinterpret_cast<const float4*>(a.bufs[s < world ? s : 0]) + base;
  float4* dst = reinterpret_cast<float4*>(a.bufs[a.rank]) + base;
  const long long stride = (long long)gridDim.x * DP_THREADS;
  for (long long i0 = (long long)blockIdx.x * DP_THREADS + threadIdx.x; i0 < n4; i0 += stride * U) {
    float4 v[U][WM];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
#pragma unroll
      for (int s = 0; s < WM; ++s)
        if (s < world && i < n4) v[u][s] = src[s][i];   // every load is issued before the first add
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + u * stride;
      if (i >= n4) break;
      float4 acc = v[u][0];                             // fixed rank order: identical bits on every run and rank
#pragma unroll
      for (int s = 1; s < WM; ++s)
        if (s < world) {
          acc.x += v[u][s].x; acc.y += v[u][s].y; acc.z += v[u][s].z; acc.w += v[u][s].w;
        }
      acc.x *= a.scale; acc.y *= a.scale; acc.z *= a.scale; acc.w *= a.scale;
      dst[i] = acc;
    }
  }
  dp_finish(a, &abort_flag);
}

__global__ void __launch_bounds__(DP_THREADS) dp_all_gather_kernel(const DpArgs a) {
  __shared__ int abort_flag;
  if (threadIdx.x == 0) abort_flag = (a.status && *reinterpret_cast<volatile int*>(a.status) != 0) ? 1 : 0;
  __syncthreads();
  if (abort_flag) return;
  if (blockIdx.x == 0) dp_signal(a, DP_READY);
  if (!dp_wait(a, DP_READY, &abort_flag)) return;
  const long long n4 = a.shard_bytes / 16;
  const long long total = n4 * (a.world - 1);
  // peers are visited starting with rank + 1 so that at any time the ranks read from different sources
  for (long long j = (long long)blockIdx.x * DP_THREADS + threadIdx.x; j < total;
       j += (long long)gridDim.x * DP_THREADS * AG_U) {
    uint4 v[AG_U];
    long long at[AG_U];
#pragma unroll
    for (int u = 0; u < AG_U; ++u) {
      const long long jj = j + (long long)u * gridDim.x * DP_THREADS;
      at[u] = -1;
      if (jj < total) {
        const int step = (int)(jj / n4);
        const int s = (a.rank + 1 + step) % a.world;
        at[u] = (a.offset_bytes + (long long)s * a.shard_bytes) / 16 + (jj - (long long)step * n4);
        v[u] = reinterpret_cast<const uint4*>(a.bufs[s])[at[u]];
      }
    }
#pragma unroll
    for (int u = 0; u < AG_U; ++u)
      if (at[u] >= 0) reinterpret_cast<uint4*>(a.bufs[a.rank])[at[u]] = v[u];
  }
  dp_finish(a, &abort_flag);
}

int fill(DpArgs& a, void* const* buf_ptrs, void* const* flag_ptrs, long long offset_bytes, long long shard_bytes,
         int world, int rank, int epoch, float scale, int* status) {
  if (world < 2 || world > DP_MAX_WORLD || rank < 0 || rank >= world) return -2;
  if (offset_bytes % 16 || shard_bytes % 16 || shard_bytes <= 0) return -2;
  for (int i = 0; i < world; ++i) {
    a.bufs[i] = buf_ptrs[i];
    a.flags[i] = reinterpret_cast<uint32_t*>(flag_ptrs[i]);
  }
  for (int i = world; i < DP_MAX_WORLD; ++i) {
    a.bufs[i] = buf_ptrs[0];
    a.flags[i] = reinterpret_cast<uint32_t*>(flag_ptrs[0]);
  }
  a.offset_bytes = offset_bytes;
  a.shard_bytes = shard_bytes;
  a.world = world;
  a.rank = rank;
  a.epoch = (uint32_t)epoch;
  a.scale = scale;
  a.status = status;
  return 0;
}

int grid_for(long long vectors, int max_ctas) {
  long long g = (vectors + DP_THREADS - 1) / DP_THREADS;
  if (g < 1) g = 1;
  return (int)(g < max_ctas ? g : max_ctas);
}

}  // namespace
}  // namespace mcb

extern "C" {

// buf_ptrs / flag_ptrs: host arrays of `world` device pointers (index = group rank).  `ctas` <= 0 picks the default.
int mcb_dp_reduce_scatter_f32(void* const* buf_ptrs, void* const* flag_ptrs, long long offset_bytes,
                              long long shard_bytes, int world, int rank, int epoch, float scale, int ctas, int* status,
                              void* stream) {
  mcb::DpArgs a;
  int rc = mcb::fill(a, buf_ptrs, flag_ptrs, offset_bytes, shard_bytes, world, rank, epoch, scale, status);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int cap = ctas > 0 ? ctas : 128;
  using namespace mcb;
  if (world == 2) {
    dp_reduce_scatter_f32_kernel<2, 4><<<grid_for(shard_bytes / 16 / 4, cap), DP_THREADS, 0, st>>>(a);
  } else if (world == 4) {
    dp_reduce_scatter_f32_kernel<4, 2><<<grid_for(shard_bytes / 16 / 2, cap), DP_THREADS, 0, st>>>(a);
  } else if (world == 8) {
    dp_reduce_scatter_f32_kernel<8, 1><<<grid_for(shard_bytes / 16, cap), DP_THREADS, 0, st>>>(a);
  } else {
    dp_reduce_scatter_f32_kernel<0, 1><<<grid_for(shard_bytes / 16, cap), DP_THREADS, 0, st>>>(a);
  }
  return (int)cudaGetLastError();
}

int mcb_dp_all_gather(void* const* buf_ptrs, void* const* flag_ptrs, long long offset_bytes, long long shard_bytes,
                      int world, int rank, int epoch, int ctas, int* status, void* stream) {
  mcb::DpArgs a;
  int rc = mcb::fill(a, buf_ptrs, flag_ptrs, offset_bytes, shard_bytes, world, rank, epoch, 1.f, status);
  if (rc) return rc;
  const int grid = mcb::grid_for(shard_bytes / 16 * (world - 1) / mcb::AG_U, ctas > 0 ? ctas : 128);
  mcb::dp_all_gather_kernel<<<grid, mcb::DP_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
  return (int)cudaGetLastError();
}

}  // extern "C"

// Mixture-of-experts routing and token exchange for sm_100a.
//
//   router_fwd / router_bwd   softmax | sigmoid scores, expert bias, group-limited selection, top-k, probability
//                             normalisation and scaling, per-expert counts and score sums (aux loss) — one warp per
//                             token, one pass over the logits.
//   moe_layout                from the [world][E] count table: padded segment offsets of the local experts and the
//                             offset of every source rank inside each segment.
//   moe_pull_dispatch         the rank that owns an expert PULLS the routed token rows out of the sources' published
//                             activations (peer loads over NVLink) straight into its expert-sorted, 128-row padded
//                             GEMM input, and tells each source where its copy went.  The all-to-all and the permute
//                             are one kernel and the result lands in ordinary local memory.
//   moe_pull_rows             same, driven by a saved row map (backward: gradient rows).
//   moe_combine               each source pulls its k result rows from the owners' output buffers and sums them —
//                             the return all-to-all fused with the un-permute.
//   flag_signal / flag_wait   epoch flags in peer memory; every wait is bounded.
//
// With one rank all "peer" pointers are local and the same kernels run (single-GPU tests, EP = 1 training).
#include "../common/host_utils.cuh"
#include "../common/ptx.cuh"

using namespace mcb;

namespace {

constexpr int MAX_WORLD = 8;
constexpr int PADM = 128;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// warp-wide argmax over (value, index); ties -> lowest index
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) {
      v = ov;
      i = oi;
    }
  }
}

struct RouterArgs {
  int T, E, k;
  int sigmoid;        // 0 softmax, 1 sigmoid
  int renorm;         // probabilities = selected scores / their sum
  int groups, group_topk;
  float scaling;
};

// lane l owns experts [l*EPL, (l+1)*EPL)
template <int EPL>
__global__ void router_fwd_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                  const uint8_t* __restrict__ valid, float* __restrict__ probs, int* __restrict__ idx,
                                  float* __restrict__ scores_out, int* __restrict__ counts,
                                  float* __restrict__ score_sum, RouterArgs a) {
  extern __shared__ float sh[];  // [E] score sums then [E] counts (as float) per block
  float* sh_sum = sh;
  int* sh_cnt = reinterpret_cast<int*>(sh + a.E);
  for (int i = threadIdx.x; i < 2 * a.E; i += blockDim.x) sh[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < a.T; t += gridDim.x * wpb) {
    float s[EPL], sel[EPL];
    const float* lr = logits + (long long)t * a.E + lane * EPL;
#pragma unroll
    for (int j = 0; j < EPL; ++j) s[j] = lr[j];
    if (a.sigmoid) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) s[j] = 1.f / (1.f + __expf(-s[j]));
    } else {
      float m = s[0];
#pragma unroll
      for (int j = 1; j < EPL; ++j) m = fmaxf(m, s[j]);
      m = warp_max(m);
      float z = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) {
        s[j] = __expf(s[j] - m);
        z += s[j];
      }
      z = warp_sum(z);
      const float inv = 1.f / z;
#pragma unroll
      for (int j = 0; j < EPL; ++j) s[j] *= inv;
    }
    float* so = scores_out + (long long)t * a.E + lane * EPL;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      so[j] = s[j];
      sel[j] = s[j] + (bias ? bias[lane * EPL + j] : 0.f);
    }
    const bool ok = valid ? valid[t] != 0 : true;
    // group-limited routing: keep the `group_topk` groups with the largest sum of their top (k / group_topk) entries
    if (a.groups > 1 && a.group_topk > 0 && a.group_topk < a.groups) {
      const int per_group = a.E / a.groups;
      const int lanes_per_group = per_group / EPL;   // launcher guarantees >= 1 and a divisor of 32
      const int my_group = lane / lanes_per_group;
      const int take = max(1, a.k / a.group_topk);
      float gscore = 0.f;
      {
        float tmp[EPL];
#pragma unroll
        for (int j = 0; j < EPL; ++j) tmp[j] = sel[j];
        for (int r = 0; r < take; ++r) {
          float bv = -INFINITY;
          int bi = 0x7fffffff;
#pragma unroll
          for (int j = 0; j < EPL; ++j)
            if (tmp[j] > bv) { bv = tmp[j]; bi = lane * EPL + j; }
          // argmax inside the group's lanes only
          for (int o = lanes_per_group >> 1; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
          }
          gscore += bv;
#pragma unroll
          for (int j = 0; j < EPL; ++j)
            if (lane * EPL + j == bi) tmp[j] = -INFINITY;
        }
      }
      // rank of my group among all groups (ties -> lower group index wins)
      int better = 0;
      for (int g = 0; g < a.groups; ++g) {
        const float og = __shfl_sync(0xffffffffu, gscore, g * lanes_per_group);
        if (og > gscore || (og == gscore && g < my_group)) ++better;
      }
      if (better >= a.group_topk) {
#pragma unroll
        for (int j = 0; j < EPL; ++j) sel[j] = -INFINITY;
      }
    }
    // top-k by repeated warp argmax
    float chosen_score[16];
    int chosen[16];
    float denom = 0.f;
    for (int r = 0; r < a.k; ++r) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < EPL; ++j)
        if (sel[j] > bv) { bv = sel[j]; bi = lane * EPL + j; }
      warp_argmax(bv, bi);
      float sc = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j)
        if (lane * EPL + j == bi) { sel[j] = -INFINITY; sc = s[j]; }
      sc = __shfl_sync(0xffffffffu, sc, bi / EPL);
      chosen[r] = bi;
      chosen_score[r] = sc;
      denom += sc;
    }
    const float norm = a.renorm ? 1.f / (denom + (a.sigmoid ? 1e-20f : 0.f)) : 1.f;
    if (lane < a.k) {
      // every lane holds all k results; lane r writes entry r
      float pv = 0.f;
      int iv = 0;
      for (int r = 0; r < a.k; ++r)
        if (r == lane) { pv = chosen_score[r]; iv = chosen[r]; }
      probs[(long long)t * a.k + lane] = pv * norm * a.scaling;
      idx[(long long)t * a.k + lane] = iv;
      if (ok && counts) atomicAdd(&sh_cnt[iv], 1);
    }
    if (ok && score_sum) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) atomicAdd(&sh_sum[lane * EPL + j], s[j]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < a.E; i += blockDim.x) {
    if (score_sum && sh_sum[i] != 0.f) atomicAdd(score_sum + i, sh_sum[i]);
    if (counts && sh_cnt[i] != 0) atomicAdd(counts + i, sh_cnt[i]);
  }
}

// dlogits from dprobs (+ a per-expert gradient on the scores coming from the load-balancing loss)
template <int EPL>
__global__ void router_bwd_kernel(const float* __restrict__ dprobs, const int* __restrict__ idx,
                                  const float* __restrict__ scores, const float* __restrict__ dscore_vec,
                                  const uint8_t* __restrict__ valid, float* __restrict__ dlogits, RouterArgs a) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < a.T; t += gridDim.x * wpb) {
    float s[EPL], ds[EPL];
    const float* sr = scores + (long long)t * a.E + lane * EPL;
    const bool ok = valid ? valid[t] != 0 : true;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      s[j] = sr[j];
      ds[j] = (dscore_vec && ok) ? dscore_vec[lane * EPL + j] : 0.f;
    }
    // selected scores, their sum and sum_i dprob_i * score_i
    float denom = 0.f, dot = 0.f;
    int my_idx = 0;
    float my_dp = 0.f, my_sc = 0.f;
    if (lane < a.k) {
      my_idx = idx[(long long)t * a.k + lane];
      my_dp = dprobs[(long long)t * a.k + lane] * a.scaling;
    }
    for (int r = 0; r < a.k; ++r) {
      const int e = __shfl_sync(0xffffffffu, my_idx, r);
      float sc = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j)
        if (lane * EPL + j == e) sc = s[j];
      sc = __shfl_sync(0xffffffffu, sc, e / EPL);
      if (lane == r) my_sc = sc;
      denom += sc;
    }
    dot = warp_sum(lane < a.k ? my_dp * my_sc : 0.f);
    const float inv = a.renorm ? 1.f / (denom + (a.sigmoid ? 1e-20f : 0.f)) : 1.f;
    for (int r = 0; r < a.k; ++r) {
      const int e = __shfl_sync(0xffffffffu, my_idx, r);
      const float dp = __shfl_sync(0xffffffffu, my_dp, r);
      const float g = a.renorm ? (dp * inv - dot * inv * inv) : dp;
#pragma unroll
      for (int j = 0; j < EPL; ++j)
        if (lane * EPL + j == e) ds[j] += g;
    }
    float* dl = dlogits + (long long)t * a.E + lane * EPL;
    if (a.sigmoid) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) dl[j] = ds[j] * s[j] * (1.f - s[j]);
    } else {
      float inner = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) inner += ds[j] * s[j];
      inner = warp_sum(inner);
#pragma unroll
      for (int j = 0; j < EPL; ++j) dl[j] = s[j] * (ds[j] - inner);
    }
  }
}

// ------------------------------------------------------------------------------------------- exchange layout
// table[s][e]: copies rank s routes to global expert e.  For the local experts [rank*El, (rank+1)*El):
//   seg_off[el] (El+1, padded to 128), src_off[s][el] = start of rank s inside segment el.
struct CountPtrs {
  const int* p[MAX_WORLD];   // each rank's published counts [E]
};

__global__ void moe_layout_kernel(CountPtrs table, int world, int rank, int E, int El,
                                  int* __restrict__ seg_off, int* __restrict__ src_off, int capacity,
                                  int* __restrict__ status) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int acc = 0;
  for (int el = 0; el < El; ++el) {
    seg_off[el] = acc;
    int within = 0;
    for (int s = 0; s < world; ++s) {
      src_off[s * El + el] = within;
      within += table.p[s][rank * El + el];
    }
    acc += (within + PADM - 1) / PADM * PADM;
  }
  seg_off[El] = acc;
  if (acc > capacity && status) atomicMax(status, ST_MOE_OVERFLOW);  // receive buffer too small for this routing
}

struct PullArgs {
  int world, rank, T, k, E, El, H;
  int capacity;
  const void* x_ptrs[MAX_WORLD];       // published activations [T, H] bf16
  const int* idx_ptrs[MAX_WORLD];      // published routing [T, k]
  const float* prob_ptrs[MAX_WORLD];   // published probabilities [T, k] (may be null)
  int* sent_row_ptrs[MAX_WORLD];       // per source: [T, k] row of each copy on its owner (written here)
};

__device__ __forceinline__ void copy_row(const __nv_bfloat16* src, __nv_bfloat16* dst, int H, int lane) {
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
  uint4* d4 = reinterpret_cast<uint4*>(dst);
  const int n = H / 8;
  for (int i = lane; i < n; i += 32 * 4) {
    uint4 v0 = s4[i];
    uint4 v1 = (i + 32 < n) ? s4[i + 32] : make_uint4(0, 0, 0, 0);
    uint4 v2 = (i + 64 < n) ? s4[i + 64] : make_uint4(0, 0, 0, 0);
    uint4 v3 = (i + 96 < n) ? s4[i + 96] : make_uint4(0, 0, 0, 0);
    d4[i] = v0;
    if (i + 32 < n) d4[i + 32] = v1;
    if (i + 64 < n) d4[i + 64] = v2;
    if (i + 96 < n) d4[i + 96] = v3;
  }
}

// one warp per published (source, token, choice) entry
__global__ void moe_pull_dispatch_kernel(PullArgs a, const int* __restrict__ seg_off, const int* __restrict__ src_off,
                                         int* __restrict__ cursor /* [world][El] zeroed */,
                                         __nv_bfloat16* __restrict__ xp, float* __restrict__ row_probs,
                                         int* __restrict__ row_src /* [capacity] entry id or -1 */) {
  const int lane = threadIdx.x & 31;
  const long long per_src = (long long)a.T * a.k;
  const long long total = per_src * a.world;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long w = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < total; w += nwarps) {
    // start with the next rank so the eight owners do not all read the same source at once
    const int step = (int)(w / per_src);
    const int s = (a.rank + 1 + step) % a.world;
    const long long ent = w - (long long)step * per_src;
    const int e = a.idx_ptrs[s][ent];
    const int el = e - a.rank * a.El;
    if (el < 0 || el >= a.El) continue;
    int row = 0;
    if (lane == 0) {
      const int slot = atomicAdd(&cursor[s * a.El + el], 1);
      row = seg_off[el] + src_off[s * a.El + el] + slot;
    }
    row = __shfl_sync(0xffffffffu, row, 0);
    if (row >= a.capacity) continue;   // flagged by the layout kernel
    const int t = (int)(ent / a.k);
    copy_row(reinterpret_cast<const __nv_bfloat16*>(a.x_ptrs[s]) + (long long)t * a.H, xp + (long long)row * a.H, a.H, lane);
    if (lane == 0) {
      if (row_probs) row_probs[row] = a.prob_ptrs[s] ? a.prob_ptrs[s][ent] : 1.f;
      row_src[row] = s * (int)per_src + (int)ent;
      a.sent_row_ptrs[s][ent] = row;
    }
  }
}

// backward / replay: row r takes token (s, t) recorded in row_src
__global__ void moe_pull_rows_kernel(PullArgs a, const int* __restrict__ row_src, int rows,
                                     __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long long per_src = (long long)a.T * a.k;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += nwarps) {
    const int id = row_src[r];
    __nv_bfloat16* dst = out + r * a.H;
    if (id < 0) {
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      for (int i = lane; i < a.H / 8; i += 32) d4[i] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const int s = id / (int)per_src;
    const int t = (id - s * (int)per_src) / a.k;
    copy_row(reinterpret_cast<const __nv_bfloat16*>(a.x_ptrs[s]) + (long long)t * a.H, dst, a.H, lane);
  }
}

struct CombineArgs {
  int world, T, k, El, H;
  const void* y_ptrs[MAX_WORLD];       // owners' output rows [capacity, H] bf16
  const float* scalar_ptrs[MAX_WORLD]; // optional per-row scalar on the owner (e.g. d(prob))
};

// out[t] = sum_k y_owner[row(t,k)]; optionally scalar_out[t,k] = scalar_owner[row(t,k)]
__global__ void moe_combine_kernel(CombineArgs a, const int* __restrict__ idx, const int* __restrict__ sent_row,
                                   __nv_bfloat16* __restrict__ out, float* __restrict__ scalar_out) {
  const int lane = threadIdx.x & 31;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = a.H / 8;
  for (long long t = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < a.T; t += nwarps) {
    for (int v0 = lane; v0 < nvec; v0 += 32) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int kk = 0; kk < a.k; ++kk) {
        const int e = idx[t * a.k + kk];
        const int row = sent_row[t * a.k + kk];
        if (row < 0) continue;
        const uint4 raw = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.y_ptrs[e / a.El]) +
                                                         (long long)row * a.H)[v0];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(h[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out + t * a.H)[v0] = o;
    }
    if (scalar_out && lane < a.k) {
      const int e = idx[t * a.k + lane];
      const int row = sent_row[t * a.k + lane];
      scalar_out[t * a.k + lane] = (row >= 0 && a.scalar_ptrs[e / a.El]) ? a.scalar_ptrs[e / a.El][row] : 0.f;
    }
  }
}

struct FlagArgs {
  int world, rank;
  uint32_t* flag_ptrs[MAX_WORLD];
};

// writes `value` into slot [base + rank] of every rank's flag region (after making prior writes visible)
__global__ void flag_signal_kernel(FlagArgs a, int base, uint32_t value) {
  if ((int)threadIdx.x < a.world) {
    fence_acq_rel_sys();
    st_release_sys(a.flag_ptrs[threadIdx.x] + base + a.rank, value);
  }
}

// waits until slots [base, base + world) of the local flag region have all reached `value`
__global__ void flag_wait_kernel(FlagArgs a, int base, uint32_t value, int* status) {
  __shared__ int abort_flag;
  if (threadIdx.x == 0) abort_flag = 0;
  __syncthreads();
  if ((int)threadIdx.x < a.world)
    wait_flag<SCOPE_SYS>(a.flag_ptrs[a.rank] + base + threadIdx.x, value, false, &abort_flag, status);
}

int grid_for(long long warps, int threads) {
  long long blocks = (warps * 32 + threads - 1) / threads;
  long long cap = (long long)device_sm_count() * 16;
  if (blocks < 1) blocks = 1;
  return (int)(blocks < cap ? blocks : cap);
}

}  // namespace

extern "C" {

int mcb_router_fwd(const float* logits, const float* bias, const uint8_t* valid, float* probs, int* idx, float* scores,
                   int* counts, float* score_sum, int T, int E, int k, int sigmoid, int renorm, int groups,
                   int group_topk, float scaling, void* stream_) {
  if (T == 0) return 0;
  if (E % 32 || k > 16 || k > E) return -1;
  const int epl = E / 32;
  if (groups > 1) {
    if (E % groups) return -2;
    const int per_group = E / groups;
    if (per_group % epl) return -2;
    const int lpg = per_group / epl;
    if (lpg < 1 || (lpg & (lpg - 1))) return -2;
  }
  RouterArgs a{T, E, k, sigmoid, renorm, groups, group_topk, scaling};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const int threads = 256;
  const int grid = grid_for(T, threads);
  const size_t sh = 2 * E * sizeof(float);
#define RF(N) router_fwd_kernel<N><<<grid, threads, sh, s>>>(logits, bias, valid, probs, idx, scores, counts, score_sum, a)
  switch (epl) {
    case 1: RF(1); break;
    case 2: RF(2); break;
    case 4: RF(4); break;
    case 8: RF(8); break;
    case 16: RF(16); break;
    default: return -3;
  }
#undef RF
  return (int)cudaGetLastError();
}

int mcb_router_bwd(const float* dprobs, const int* idx, const float* scores, const float* dscore_vec,
                   const uint8_t* valid, float* dlogits, int T, int E, int k, int sigmoid, int renorm, float scaling,
                   void* stream_) {
  if (T == 0) return 0;
  if (E % 32 || k > 16) return -1;
  const int epl = E / 32;
  RouterArgs a{T, E, k, sigmoid, renorm, 0, 0, scaling};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const int threads = 256;
  const int grid = grid_for(T, threads);
#define RB(N) router_bwd_kernel<N><<<grid, threads, 0, s>>>(dprobs, idx, scores, dscore_vec, valid, dlogits, a)
  switch (epl) {
    case 1: RB(1); break;
    case 2: RB(2); break;
    case 4: RB(4); break;
    case 8: RB(8); break;
    case 16: RB(16); break;
    default: return -3;
  }
#undef RB
  return (int)cudaGetLastError();
}

int mcb_moe_layout(const int* const* count_ptrs, int world, int rank, int E, int El, int* seg_off, int* src_off,
                   int capacity, int* status, void* stream_) {
  if (world < 1 || world > MAX_WORLD) return -1;
  CountPtrs table{};
  for (int i = 0; i < world; ++i) table.p[i] = count_ptrs[i];
  moe_layout_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(table, world, rank, E, El, seg_off, src_off,
                                                                          capacity, status);
  return (int)cudaGetLastError();
}

int mcb_moe_pull_dispatch(const void* const* x_ptrs, const int* const* idx_ptrs, const float* const* prob_ptrs,
                          int* const* sent_row_ptrs, int world, int rank, int T, int k, int E, int El, int H,
                          int capacity, const int* seg_off, const int* src_off, int* cursor, void* xp, float* row_probs,
                          int* row_src, void* stream_) {
  if (world < 1 || world > MAX_WORLD || H % 8) return -1;
  PullArgs a{};
  a.world = world; a.rank = rank; a.T = T; a.k = k; a.E = E; a.El = El; a.H = H; a.capacity = capacity;
  for (int i = 0; i < world; ++i) {
    a.x_ptrs[i] = x_ptrs[i];
    a.idx_ptrs[i] = idx_ptrs[i];
    a.prob_ptrs[i] = prob_ptrs ? prob_ptrs[i] : nullptr;
    a.sent_row_ptrs[i] = sent_row_ptrs[i];
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const long long warps = (long long)world * T * k;
  moe_pull_dispatch_kernel<<<grid_for(warps, 256), 256, 0, s>>>(a, seg_off, src_off, cursor, (__nv_bfloat16*)xp,
                                                                 row_probs, row_src);
  return (int)cudaGetLastError();
}

int mcb_moe_pull_rows(const void* const* x_ptrs, int world, int T, int k, int H, const int* row_src, int rows, void* out,
                      void* stream_) {
  if (world < 1 || world > MAX_WORLD || H % 8) return -1;
  if (rows == 0) return 0;
  PullArgs a{};
  a.world = world; a.T = T; a.k = k; a.H = H;
  for (int i = 0; i < world; ++i) a.x_ptrs[i] = x_ptrs[i];
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  moe_pull_rows_kernel<<<grid_for(rows, 256), 256, 0, s>>>(a, row_src, rows, (__nv_bfloat16*)out);
  return (int)cudaGetLastError();
}

int mcb_moe_combine(const void* const* y_ptrs, const float* const* scalar_ptrs, int world, int T, int k, int El, int H,
                    const int* idx, const int* sent_row, void* out, float* scalar_out, void* stream_) {
  if (world < 1 || world > MAX_WORLD || H % 8 || k > 32) return -1;
  if (T == 0) return 0;
  CombineArgs a{};
  a.world = world; a.T = T; a.k = k; a.El = El; a.H = H;
  for (int i = 0; i < world; ++i) {
    a.y_ptrs[i] = y_ptrs[i];
    a.scalar_ptrs[i] = scalar_ptrs ? scalar_ptrs[i] : nullptr;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  moe_combine_kernel<<<grid_for(T, 256), 256, 0, s>>>(a, idx, sent_row, (__nv_bfloat16*)out, scalar_out);
  return (int)cudaGetLastError();
}

int mcb_flag_signal(void* const* flag_ptrs, int world, int rank, int base, unsigned value, void* stream_) {
  if (world < 1 || world > MAX_WORLD) return -1;
  FlagArgs a{};
  a.world = world; a.rank = rank;
  for (int i = 0; i < world; ++i) a.flag_ptrs[i] = reinterpret_cast<uint32_t*>(flag_ptrs[i]);
  flag_signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(a, base, value);
  return (int)cudaGetLastError();
}

int mcb_flag_wait(void* const* flag_ptrs, int world, int rank, int base, unsigned value, int* status, void* stream_) {
  if (world < 1 || world > MAX_WORLD) return -1;
  FlagArgs a{};
  a.world = world; a.rank = rank;
  for (int i = 0; i < world; ++i) a.flag_ptrs[i] = reinterpret_cast<uint32_t*>(flag_ptrs[i]);
  flag_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(a, base, value, status);
  return (int)cudaGetLastError();
}

}  // extern "C"

// MoE token dispatch fused with the grouped expert GEMM (one launch):
//
//   source side   mcb_moe_sort: the routing of a rank's tokens, sorted by expert (stable), so that the entries that go
//                 to one expert are one contiguous, deterministically ordered run of the published `order` table
//   owner side    mcb_moe_pull_gemm: every CTA of a persistent grid carries the GEMM roles plus four communication
//                 warps.  The communication warps of all CTAs gather the routed rows from the sources' published
//                 activations over NVLink (vector loads, eight in flight per lane: one SM alone keeps too few bytes
//                 in flight to feed the GEMM) into the expert-sorted, 128-row padded GEMM input and publish a flag
//                 per 128-row block; the GEMM roles run the grouped expert GEMM C[rows of expert e] = X[rows of e] .
//                 W_e^T on tcgen05 and consume the blocks in arrival order, so the exchange hides behind the math.
//
// Rows are assigned without atomics: expert segment -> source rank -> position in that source's sorted run, which
// makes the row order (and therefore every fp32 weight-gradient sum over rows) reproducible.  The same kernel replays
// a recorded assignment (`row_src`) for the backward pass, where the rows are output gradients and the GEMM is the
// data gradient of the second expert layer.
//
// No TMA multicast; remote memory is read by plain vector loads and written by 4-byte stores.  Every
// wait is bounded and reports through the status word.
#include "../common/host_utils.cuh"
#include "../gemm/gemm_pipe.cuh"

using namespace mcb;

namespace {

constexpr int MAX_WORLD = 8;
constexpr int PADM = 128;
constexpr int MAX_EL = 64;            // local experts per rank the fused kernel supports
constexpr int PULL_WARPS = 4;         // communication warps per CTA (warps 6..9)
constexpr int PULL_LOADS = 8;         // 16-byte loads a lane keeps in flight
constexpr int MOE_THREADS = GEMM_THREADS + PULL_WARPS * 32;

// ---------------------------------------------------------------------------------------------------------------
// source side: stable counting sort of the routing entries by expert
// ---------------------------------------------------------------------------------------------------------------
// One CTA of 32 warps per expert.  Warp w owns a contiguous slice of the entries; pass 1 counts its matches, pass 2
// writes them behind the matches of the warps before it, so entries keep their order inside an expert's run.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ idx, const int* __restrict__ counts,
                                                        int n_entries, int E, int* __restrict__ eoff,
                                                        int* __restrict__ order) {
  const int e = blockIdx.x;
  __shared__ int s_base;
  __shared__ int s_warp[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    int b = 0;
    for (int i = 0; i < e; ++i) b += counts[i];
    s_base = b;
    eoff[e] = b;
    if (e == E - 1) eoff[E] = b + counts[e];
  }
  const int per_warp = ((n_entries + 31) / 32 + 31) / 32 * 32;   // a multiple of 32 so that slices stay aligned
  const int lo = warp * per_warp, hi = min(n_entries, lo + per_warp);
  int cnt = 0;
  for (int base = lo; base < hi; base += 32) {
    const int i = base + lane;
    const bool m = i < hi && idx[i] == e;
    cnt += __popc(__ballot_sync(0xffffffffu, m));
  }
  if (lane == 0) s_warp[warp] = cnt;
  __syncthreads();
  int running = s_base;
  for (int w = 0; w < warp; ++w) running += s_warp[w];
  for (int base = lo; base < hi; base += 32) {
    const int i = base + lane;
    const bool m = i < hi && idx[i] == e;
    const unsigned b = __ballot_sync(0xffffffffu, m);
    if (m) order[running + __popc(b & ((1u << lane) - 1u))] = i;
    running += __popc(b);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// owner side: pull + grouped GEMM
// ---------------------------------------------------------------------------------------------------------------
struct MoeFusedParams {
  int world, rank, T, k, E, El;
  int H;                  // width of the pulled rows = contraction size of the GEMM
  int N;                  // output width of the GEMM (per expert)
  int capacity;           // rows of xp / C (a multiple of 128)
  int mode;               // 0: assign rows from the sources' sorted tables; 1: replay the assignment in row_src
  const void* x_ptrs[MAX_WORLD];      // published rows [T, H] bf16
  const int* order_ptrs[MAX_WORLD];   // mode 0: entries sorted by expert [T * k]
  const int* eoff_ptrs[MAX_WORLD];    // mode 0: start of every expert's run [E + 1]
  const float* prob_ptrs[MAX_WORLD];  // mode 0: routing probabilities [T, k] (may be null)
  int* sent_row_ptrs[MAX_WORLD];      // mode 0: [T, k] row of each entry on its owner (written here)
  int* seg_off;                       // [El + 1] first row of every local expert (written in mode 0, read in mode 1)
  int* row_src;                       // [capacity] source entry of every row or -1 (written in mode 0)
  float* row_probs;                   // [capacity] routing probability of every row (mode 0, may be null)
  __nv_bfloat16* xp;                  // [capacity, H] gathered rows
  uint32_t* blk_flags;                // [2 * capacity / 128]: "block landed" flags (epoch stamped), then the quarter
                                      // counters of every block (zero between calls)
  uint32_t epoch;
  void* C;                            // [capacity, N] bf16
  long long ldc;
  int b_group_rows;                   // rows between consecutive experts in the 2-D view of B
  int* status;
};

struct Layout {
  int seg_off[MAX_EL + 1];
  int src_off[(MAX_WORLD + 1) * MAX_EL];   // [s][el]: rows of expert el that come from sources < s
  int eoff_base[MAX_WORLD * MAX_EL];       // [s][el]: start of expert (rank * El + el) in source s's sorted table
};

template <int BN, bool B_MN>
__global__ void __launch_bounds__(MOE_THREADS, 1)
moe_pull_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const MoeFusedParams p) {
  constexpr uint32_t TMEM_COLS = 2 * BN;
  extern __shared__ uint8_t smem_raw[];
  __shared__ Layout L;
  if (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) {
    // an earlier kernel gave up (or a receive buffer overflowed): do not pile up, and leave offsets behind that keep
    // the kernels that follow in this step inside their buffers (the step's update is skipped anyway)
    if (p.mode == 0 && blockIdx.x == 0)
      for (int el = threadIdx.x; el <= p.El; el += blockDim.x) p.seg_off[el] = 0;
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int El = p.El;

  // ------------------------------------------------------------------ row layout (every CTA computes it itself)
  if (p.mode == 0) {
    for (int el = threadIdx.x; el < El; el += blockDim.x) {
      int run = 0;
      for (int s = 0; s < p.world; ++s) {
        const int* eo = p.eoff_ptrs[s] + p.rank * El + el;
        const int b = eo[0], c = eo[1] - b;
        L.src_off[s * MAX_EL + el] = run;
        L.eoff_base[s * MAX_EL + el] = b;
        run += c;
      }
      L.src_off[p.world * MAX_EL + el] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int acc = 0;
      for (int el = 0; el < El; ++el) {
        L.seg_off[el] = acc;
        acc += (L.src_off[p.world * MAX_EL + el] + PADM - 1) / PADM * PADM;
      }
      L.seg_off[El] = acc;
      if (blockIdx.x == 0) {
        // published offsets never point past the buffer, also when the routing does not fit it
        for (int el = 0; el <= El; ++el) p.seg_off[el] = min(L.seg_off[el], p.capacity);
        if (acc > p.capacity && p.status) atomicMax(p.status, ST_MOE_OVERFLOW);
      }
    }
  } else {
    for (int el = threadIdx.x; el <= El; el += blockDim.x) L.seg_off[el] = p.seg_off[el];
  }
  __syncthreads();
  const int valid_rows = min(L.seg_off[El], p.capacity);
  const int nblocks = valid_rows / PADM;
  const int tiles_n = (p.N + BN - 1) / BN;

  // ===================================================================== GEMM CTA
  Pipe<BN> P(smem_raw);
  if (threadIdx.x == 0) {
    P.init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(P.tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *P.tmem_slot;
  const int g0 = blockIdx.x, gs = gridDim.x;
  const int total = nblocks * tiles_n;      // row-block major: the tiles of a block wait for the same flag
  auto expert_of = [&](int mb) {
    int el = 0;
    while (el + 1 < El && L.seg_off[el + 1] <= mb * PADM) ++el;
    return el;
  };

  if (warp >= GEMM_THREADS / 32) {
    // =================================================================== communication warps: gather the rows.
    // A unit is a quarter (32 rows) of a 128-row block; lane l works out where row l of the unit comes from, then the
    // warp copies the rows one after the other with every lane keeping up to eight 16-byte loads in flight.  The
    // warp that completes a block's fourth quarter publishes the block.
    const uint32_t row_bytes = (uint32_t)p.H * 2u;
    const int n16 = (int)(row_bytes / 16);
    const long long per_src = (long long)p.T * p.k;
    uint32_t* blk_cnt = p.blk_flags + p.capacity / PADM;
    const int cw = (int)blockIdx.x * PULL_WARPS + (warp - GEMM_THREADS / 32);
    const int ncw = (int)gridDim.x * PULL_WARPS;
    for (int u = cw; u < nblocks * 4; u += ncw) {
      const int b = u >> 2;
      const int R = u * 32 + lane;
      const uint8_t* src = nullptr;
      if (p.mode == 0) {
        int el = 0;
        while (el + 1 < El && L.seg_off[el + 1] <= R) ++el;
        const int i = R - L.seg_off[el];
        int sr = -1;
        if (i < L.src_off[p.world * MAX_EL + el]) {
          sr = 0;
          while (sr + 1 < p.world && L.src_off[(sr + 1) * MAX_EL + el] <= i) ++sr;
        }
        int id = -1;
        float prob = 0.f;
        if (sr >= 0) {
          const int j = i - L.src_off[sr * MAX_EL + el];
          const int ent = p.order_ptrs[sr][L.eoff_base[sr * MAX_EL + el] + j];
          if (ent >= 0 && ent < per_src) {          // a torn table would otherwise turn into a wild address
            src = reinterpret_cast<const uint8_t*>(p.x_ptrs[sr]) + (long long)(ent / p.k) * row_bytes;
            id = sr * (int)per_src + ent;
            prob = p.prob_ptrs[sr] ? p.prob_ptrs[sr][ent] : 1.f;
            p.sent_row_ptrs[sr][ent] = R;
          }
        }
        p.row_src[R] = id;
        if (p.row_probs) p.row_probs[R] = prob;
      } else {
        const int id = p.row_src[R];
        if (id >= 0) {
          const int sr = id / (int)per_src;
          const int ent = id - sr * (int)per_src;
          if (sr < p.world) src = reinterpret_cast<const uint8_t*>(p.x_ptrs[sr]) + (long long)(ent / p.k) * row_bytes;
        }
      }
      uint4* dst_row = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.xp) + (long long)(u * 32) * row_bytes);
      auto copy_row = [&](const uint4* s16, uint4* d16) {
        if (s16 == nullptr) {
          for (int c = lane; c < n16; c += 32) d16[c] = make_uint4(0, 0, 0, 0);   // padding row
          return;
        }
        for (int base = 0; base < n16; base += 32 * PULL_LOADS) {
          uint4 v[PULL_LOADS];
#pragma unroll
          for (int j = 0; j < PULL_LOADS; ++j) {
            const int c = base + j * 32 + lane;
            if (c < n16) v[j] = s16[c];                 // every load is issued before the first store
          }
#pragma unroll
          for (int j = 0; j < PULL_LOADS; ++j) {
            const int c = base + j * 32 + lane;
            if (c < n16) d16[c] = v[j];
          }
        }
      };
#pragma unroll 1
      for (int r = 0; r < 32; r += 2, dst_row += 2 * n16) {
        const uint4* sa = reinterpret_cast<const uint4*>(__shfl_sync(0xffffffffu, reinterpret_cast<uintptr_t>(src), r));
        const uint4* sb =
            reinterpret_cast<const uint4*>(__shfl_sync(0xffffffffu, reinterpret_cast<uintptr_t>(src), r + 1));
        if (sa != nullptr && sb != nullptr && n16 <= 32 * PULL_LOADS) {
          // two rows of at most 4 KiB at once: 2 x PULL_LOADS loads in flight per lane
          uint4 va[PULL_LOADS], vb[PULL_LOADS];
#pragma unroll
          for (int j = 0; j < PULL_LOADS; ++j) {
            const int c = j * 32 + lane;
            if (c < n16) {
              va[j] = sa[c];
              vb[j] = sb[c];
            }
          }
#pragma unroll
          for (int j = 0; j < PULL_LOADS; ++j) {
            const int c = j * 32 + lane;
            if (c < n16) {
              dst_row[c] = va[j];
              dst_row[n16 + c] = vb[j];
            }
          }
        } else {
          copy_row(sa, dst_row);
          copy_row(sb, dst_row + n16);
        }
      }
      __syncwarp();
      if (lane == 0) {
        // the fence orders this warp's stores before its count; the fence after the fourth count orders the other
        // warps' (counted, hence fenced) stores before the flag
        __threadfence();
        const uint32_t done = atomicAdd(blk_cnt + b, 1u) + 1u;
        if (done == 4u) {
          __threadfence();
          blk_cnt[b] = 0;
          st_release_gpu(p.blk_flags + b, p.epoch);
        }
      }
    }
  } else if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      int seen = -1;
      for (int t = g0; t < total; t += gs) {
        const int mb = t / tiles_n, tn = t - mb * tiles_n;
        const int el = expert_of(mb);
        if (mb != seen) {
          if (!wait_flag<SCOPE_GPU>(p.blk_flags + mb, p.epoch, false, P.abort_flag, p.status)) break;
          fence_proxy_async_all();
          seen = mb;
        }
        const int n0 = B_MN ? tn * BN : el * p.b_group_rows + tn * BN;
        if (!load_tile<BN, B_MN>(P, &tmap_a, &tmap_b, mb * PADM, n0, p.H, it, p.status, B_MN ? el * p.b_group_rows : 0))
          break;
      }
      drain_loads<BN>(P, it);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int t = g0; t < total && ok; t += gs, ++lt) {
        const uint32_t acc = lt & 1, aph = (lt >> 1) & 1;
        if (!mbar_wait(smem_u32(&P.tempty_bar[acc]), aph ^ 1, P.abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        issue_mma_tile<BN, B_MN>(P, tmem_base + acc * BN, p.H, it, p.status, ok);
        if (ok) umma_commit(smem_u32(&P.tfull_bar[acc]));
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t lt = 0;
    for (int t = g0; t < total; t += gs, ++lt) {
      const int mb = t / tiles_n, tn = t - mb * tiles_n;
      const int n0 = tn * BN;
      const uint32_t acc = lt & 1, aph = (lt >> 1) & 1;
      if (!mbar_wait(smem_u32(&P.tfull_bar[acc]), aph, P.abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const long long row = (long long)mb * PADM + q * 32 + lane;
      __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc;
#pragma unroll 1
      for (int cc = 0; cc < BN; cc += 32) {
        if (n0 + cc >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (uint32_t(q * 32) << 16) + acc * BN + cc, r);
        tmem_ld_wait();
        const int col0 = n0 + cc;
        if (col0 + 32 <= p.N) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            o.y = pack_bf16x2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            o.z = pack_bf16x2(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
            o.w = pack_bf16x2(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
            *reinterpret_cast<uint4*>(crow + col0 + j) = o;
          }
        } else {
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) crow[col0 + j] = __float2bfloat16(__uint_as_float(r[j]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&P.tempty_bar[acc]));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// owner side: grouped GEMM whose epilogue scatters every output row to the rank and slot it came from
// ---------------------------------------------------------------------------------------------------------------
// Second expert layer (forward) and data gradient of the first (backward).  Row R of the expert-sorted operand
// belongs to routing entry `ent` of source rank `s` (row_src[R] = s * T * k + ent, recorded by the dispatch); its
// result goes straight from the accumulator to slot `ent` of that rank's [T * k, N] buffer, over NVLink for remote
// sources, while later tiles are still being multiplied.  The source then adds the k slots of each token in a fixed
// order (moe_sum_slots_kernel): the combine needs no second pass over the owners' memory and no atomics.
struct MoeScatterParams {
  int world, T, k, El;
  int K;                  // contraction size
  int N;                  // output width = slot width (a multiple of 64)
  int capacity;
  const int* seg_off;     // [El + 1]
  const int* row_src;     // [capacity]
  void* slot_ptrs[MAX_WORLD];         // [T * k, N] bf16 on every source
  float* sslot_ptrs[MAX_WORLD];       // optional [T * k] fp32: per-entry scalar (gradient of the routing probability)
  const float* scalar;                // optional [capacity]: the scalar of every row
  int b_group_rows;
  int* status;
};

constexpr int SC_STAGE_BYTES = 32 * 128;   // per epilogue warp: 32 rows x 64 bf16 columns

template <int BN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
moe_gemm_scatter_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                        const MoeScatterParams p) {
  constexpr uint32_t TMEM_COLS = 2 * BN;
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_seg[MAX_EL + 1];
  if (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int El = p.El;
  for (int el = threadIdx.x; el <= El; el += blockDim.x) s_seg[el] = p.seg_off[el];
  Pipe<BN> P(smem_raw);
  if (threadIdx.x == 0) {
    P.init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(P.tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *P.tmem_slot;
  const int valid_rows = min(s_seg[El], p.capacity);
  const int nblocks = valid_rows / PADM;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int total = nblocks * tiles_n;
  const int g0 = blockIdx.x, gs = gridDim.x;
  const long long per_src = (long long)p.T * p.k;
  auto expert_of = [&](int mb) {
    int el = 0;
    while (el + 1 < El && s_seg[el + 1] <= mb * PADM) ++el;
    return el;
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      for (int t = g0; t < total; t += gs) {
        const int mb = t / tiles_n, tn = t - mb * tiles_n;
        const int el = expert_of(mb);
        const int n0 = B_MN ? tn * BN : el * p.b_group_rows + tn * BN;
        if (!load_tile<BN, B_MN>(P, &tmap_a, &tmap_b, mb * PADM, n0, p.K, it, p.status, B_MN ? el * p.b_group_rows : 0))
          break;
      }
      drain_loads<BN>(P, it);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int t = g0; t < total && ok; t += gs, ++lt) {
        const uint32_t acc = lt & 1, aph = (lt >> 1) & 1;
        if (!mbar_wait(smem_u32(&P.tempty_bar[acc]), aph ^ 1, P.abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        issue_mma_tile<BN, B_MN>(P, tmem_base + acc * BN, p.K, it, p.status, ok);
        if (ok) umma_commit(smem_u32(&P.tfull_bar[acc]));
      }
    }
  } else {
    const int q = warp & 3;
    // this warp's transposition buffer: rows go in one per lane, come out 128 contiguous bytes per quarter-warp
    uint8_t* stage = P.smem + GemmSmem<BN>::STAGES * GemmSmem<BN>::STAGE_BYTES + GemmSmem<BN>::BAR_BYTES + q * SC_STAGE_BYTES;
    uint32_t lt = 0;
    for (int t = g0; t < total; t += gs, ++lt) {
      const int mb = t / tiles_n, tn = t - mb * tiles_n;
      const int n0 = tn * BN;
      const uint32_t acc = lt & 1, aph = (lt >> 1) & 1;
      // destination of this lane's row (null: padding row, nothing to send)
      const int R = mb * PADM + q * 32 + lane;
      uint8_t* dst_row = nullptr;
      const int id = p.row_src[R];
      if (id >= 0) {
        const int sr = id / (int)per_src;
        const int ent = id - sr * (int)per_src;
        if (sr < p.world) dst_row = reinterpret_cast<uint8_t*>(p.slot_ptrs[sr]) + ((long long)ent * p.N + n0) * 2;
        else if (p.status) atomicCAS(p.status, 0, ST_BAD_ARGUMENT);      // a torn table: report, send nothing
      }
      if (!mbar_wait(smem_u32(&P.tfull_bar[acc]), aph, P.abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
#pragma unroll 1
      for (int cc = 0; cc < BN; cc += 64) {
        if (n0 + cc >= p.N) break;
        uint32_t r[64];
        tmem_ld_32x32_x64(tmem_base + (uint32_t(q * 32) << 16) + acc * BN + cc, r);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(r[8 * u]), __uint_as_float(r[8 * u + 1]));
          o.y = pack_bf16x2(__uint_as_float(r[8 * u + 2]), __uint_as_float(r[8 * u + 3]));
          o.z = pack_bf16x2(__uint_as_float(r[8 * u + 4]), __uint_as_float(r[8 * u + 5]));
          o.w = pack_bf16x2(__uint_as_float(r[8 * u + 6]), __uint_as_float(r[8 * u + 7]));
          *reinterpret_cast<uint4*>(stage + lane * 128 + ((u ^ (lane & 7)) << 4)) = o;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int row = i * 4 + (lane >> 3), u = lane & 7;
          const uint4 v = *reinterpret_cast<const uint4*>(stage + row * 128 + ((u ^ (row & 7)) << 4));
          uint8_t* base = reinterpret_cast<uint8_t*>(__shfl_sync(0xffffffffu, reinterpret_cast<uintptr_t>(dst_row), row));
          if (base) *reinterpret_cast<uint4*>(base + cc * 2 + u * 16) = v;
        }
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&P.tempty_bar[acc]));
    }
    // per-entry scalars (backward: gradient of each routing probability) ride along
    if (p.scalar) {
      const int tid = (int)blockIdx.x * 128 + (int)threadIdx.x - 64, nthr = (int)gridDim.x * 128;
      for (int R = tid; R < valid_rows; R += nthr) {
        const int id = p.row_src[R];
        if (id < 0) continue;
        const int sr = id / (int)per_src;
        const int ent = id - sr * (int)per_src;
        if (sr < p.world && p.sslot_ptrs[sr]) p.sslot_ptrs[sr][ent] = p.scalar[R];
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// out[t] = sum over the k slots of token t whose entry was delivered (sent_row >= 0), in slot order
__global__ void __launch_bounds__(256) moe_sum_slots_kernel(const __nv_bfloat16* __restrict__ slots,
                                                            const int* __restrict__ sent_row, int T, int k, int N,
                                                            __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nvec = N / 8;
  for (long long t = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += nwarps) {
    const int mine = lane < k ? sent_row[t * k + lane] : -1;
    const unsigned have = __ballot_sync(0xffffffffu, mine >= 0);
    for (int v0 = lane; v0 < nvec; v0 += 32) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int kk = 0; kk < k; ++kk) {
        if (!((have >> kk) & 1u)) continue;
        const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(slots + ((long long)t * k + kk) * N) + v0);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out + t * N)[v0] = o;
    }
  }
}

}  // namespace

extern "C" {

// idx [n_entries] expert of every routing entry (entry = token * k + choice), counts [E] entries per expert ->
// eoff [E + 1] start of every expert's run, order [n_entries] entries sorted by expert, ties in entry order.
int mcb_moe_sort(const int* idx, const int* counts, int n_entries, int E, int* eoff, int* order, void* stream_) {
  if (E < 1 || n_entries < 0) return -1;
  moe_sort_kernel<<<E, 1024, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(idx, counts, n_entries, E, eoff, order);
  return (int)cudaGetLastError();
}

// Pointer arrays hold `world` device pointers (index = rank in the expert-parallel group).  B is the stacked expert
// weight: K-major `[El * N, H]` (b_mn = 0, forward of the first expert layer) or MN-major `[El * H, N]` (b_mn = 1,
// data gradient of the second expert layer: rows are contraction indices).  `blk_flags` holds 2 * capacity / 128
// words: first the epoch of the call that last filled each block (monotonically increasing, never cleared), then the
// per-block counters of landed quarters (zero when allocated, zero again after every call).
int mcb_moe_pull_gemm(const void* const* x_ptrs, const int* const* order_ptrs, const int* const* eoff_ptrs,
                      const float* const* prob_ptrs, int* const* sent_row_ptrs, int world, int rank, int T, int k, int E,
                      int El, int H, int N, int capacity, int mode, int* seg_off, int* row_src, float* row_probs, void* xp,
                      unsigned* blk_flags, unsigned epoch, const void* B, long long b_inner, long long b_outer,
                      long long ldb, int b_mn, int b_group_rows, void* C, long long ldc, int* status,
                      void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (world < 1 || world > MAX_WORLD || El < 1 || El > MAX_EL || H % 8 || N % 8 || capacity % PADM || ldc % 8) return -2;
  if ((long long)world * T * k >= (1ll << 31)) return -3;
  constexpr int BN = 256;
  const int sms = device_sm_count();
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, xp, H, capacity, H, GEMM_BK, GEMM_BM);
  if (rc) return rc;
  rc = b_mn ? make_tmap_2d_bf16(&tb, B, b_inner, b_outer, ldb, 64, GEMM_BK)
            : make_tmap_2d_bf16(&tb, B, b_inner, b_outer, ldb, GEMM_BK, BN);
  if (rc) return rc;
  MoeFusedParams p{};
  p.world = world; p.rank = rank; p.T = T; p.k = k; p.E = E; p.El = El; p.H = H; p.N = N; p.capacity = capacity;
  p.mode = mode;
  for (int i = 0; i < world; ++i) {
    p.x_ptrs[i] = x_ptrs[i];
    p.order_ptrs[i] = order_ptrs ? order_ptrs[i] : nullptr;
    p.eoff_ptrs[i] = eoff_ptrs ? eoff_ptrs[i] : nullptr;
    p.prob_ptrs[i] = prob_ptrs ? prob_ptrs[i] : nullptr;
    p.sent_row_ptrs[i] = sent_row_ptrs ? sent_row_ptrs[i] : nullptr;
  }
  if (mode == 0 && (!order_ptrs || !eoff_ptrs || !sent_row_ptrs || !row_src || !seg_off)) return -2;
  if (mode == 1 && (!row_src || !seg_off)) return -2;
  p.seg_off = seg_off; p.row_src = row_src; p.row_probs = row_probs; p.xp = reinterpret_cast<__nv_bfloat16*>(xp);
  p.blk_flags = blk_flags; p.epoch = epoch; p.C = C; p.ldc = ldc; p.b_group_rows = b_group_rows; p.status = status;
  const int smem = GemmSmem<BN>::TOTAL;
  static bool cfg[2] = {false, false};
  cudaError_t e;
  if (b_mn) {
    auto kern = moe_pull_gemm_kernel<BN, true>;
    if (!cfg[1]) {
      if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess) return (int)e;
      cfg[1] = true;
    }
    kern<<<sms, MOE_THREADS, smem, stream>>>(ta, tb, p);
  } else {
    auto kern = moe_pull_gemm_kernel<BN, false>;
    if (!cfg[0]) {
      if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess) return (int)e;
      cfg[0] = true;
    }
    kern<<<sms, MOE_THREADS, smem, stream>>>(ta, tb, p);
  }
  return (int)cudaGetLastError();
}

// Grouped GEMM C[rows of expert e] = A[rows of e] . B_e with the result rows scattered to their sources:
// A [capacity, K] bf16 (expert-sorted rows, segments `seg_off`), B stacked expert weights K-major `[El * N, K]`
// (b_mn = 0) or MN-major `[El * K, N]` (b_mn = 1), row_src [capacity] from the dispatch, slot_ptrs[s] = rank s's
// [T * k, N] bf16 slot buffer, sslot_ptrs / scalar optional (per-entry fp32 values pushed the same way).
int mcb_moe_gemm_scatter(const void* A, const void* B, long long b_inner, long long b_outer, long long ldb, int b_mn,
                         int b_group_rows, void* const* slot_ptrs, void* const* sslot_ptrs, const float* scalar,
                         const int* seg_off, const int* row_src, int world, int T, int k, int El, int K, int N,
                         int capacity, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (world < 1 || world > MAX_WORLD || El < 1 || El > MAX_EL || K % 8 || N % 64 || capacity % PADM) return -2;
  if ((long long)world * T * k >= (1ll << 31)) return -3;
  constexpr int BN = 256;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, A, K, capacity, K, GEMM_BK, GEMM_BM);
  if (rc) return rc;
  rc = b_mn ? make_tmap_2d_bf16(&tb, B, b_inner, b_outer, ldb, 64, GEMM_BK)
            : make_tmap_2d_bf16(&tb, B, b_inner, b_outer, ldb, GEMM_BK, BN);
  if (rc) return rc;
  MoeScatterParams p{};
  p.world = world; p.T = T; p.k = k; p.El = El; p.K = K; p.N = N; p.capacity = capacity;
  p.seg_off = seg_off; p.row_src = row_src; p.scalar = scalar; p.b_group_rows = b_group_rows; p.status = status;
  for (int i = 0; i < world; ++i) {
    p.slot_ptrs[i] = slot_ptrs[i];
    p.sslot_ptrs[i] = sslot_ptrs ? reinterpret_cast<float*>(sslot_ptrs[i]) : nullptr;
  }
  const int smem = GemmSmem<BN>::TOTAL + 4 * SC_STAGE_BYTES;
  const int sms = device_sm_count();
  static bool cfg[2] = {false, false};
  cudaError_t e;
  if (b_mn) {
    auto kern = moe_gemm_scatter_kernel<BN, true>;
    if (!cfg[1]) {
      if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess) return (int)e;
      cfg[1] = true;
    }
    kern<<<sms, GEMM_THREADS, smem, stream>>>(ta, tb, p);
  } else {
    auto kern = moe_gemm_scatter_kernel<BN, false>;
    if (!cfg[0]) {
      if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)) != cudaSuccess) return (int)e;
      cfg[0] = true;
    }
    kern<<<sms, GEMM_THREADS, smem, stream>>>(ta, tb, p);
  }
  return (int)cudaGetLastError();
}

// out [T, N] = per token, the sum of its delivered slots (slots [T * k, N] bf16, sent_row [T, k]: < 0 = not delivered)
int mcb_moe_sum_slots(const void* slots, const int* sent_row, int T, int k, int N, void* out, void* stream_) {
  if (N % 8 || k < 1 || k > 32) return -1;
  if (T == 0) return 0;
  long long blocks = ((long long)T * 32 + 255) / 256;
  const long long cap = (long long)device_sm_count() * 16;
  if (blocks > cap) blocks = cap;
  moe_sum_slots_kernel<<<(int)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      reinterpret_cast<const __nv_bfloat16*>(slots), sent_row, T, k, N, reinterpret_cast<__nv_bfloat16*>(out));
  return (int)cudaGetLastError();
}

}  // extern "C"

// Variable-length causal GQA attention backward for sm_100a.  Three kernels:
//
//   delta   : delta[h, i] = sum_d O[i, h, d] * dO[i, h, d]                                  (memory bound)
//   dq      : one CTA per (128-query tile, query head), loops over 64-key blocks:
//               S = Q K^T, dP = dO V^T on tcgen05 -> P = exp2(S*c - lse), dS = P*(dP - delta)*scale in registers
//               -> dS (bf16) to shared memory -> dQ += dS K accumulated in TMEM
//   dk/dv   : one CTA per (128-key tile, kv head), loops over the query heads of the group and 64-query blocks:
//               S^T = K Q^T, dP^T = V dO^T -> P^T, dS^T -> dV += P^T dO, dK += dS^T Q accumulated in TMEM
//
// All operand layouts are the ones the forward kernel uses (row-major [tokens, heads*d] tiles fetched by TMA with
// the 128-byte swizzle, consumed K-major or MN-major), P is recomputed from the forward's log-sum-exp so nothing
// but O and lse is kept from the forward.  The mask is the forward's: a per-query inclusive key range
// [k_lo[i], k_hi[i]] (k_hi null = the query's own index, i.e. packed causal self-attention); queries and keys may be
// different token sets.  The dK/dV kernel additionally takes, per key, bounds [q_lo[n], q_hi[n]] on the queries that
// can see it (null = derived from the causal structure), which only limit its loop: visibility itself is always
// decided by the per-query ranges.
//
// Warp roles in dq and dk/dv (320 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..9
// element-wise in two groups of four (thread = TMEM lane = query row in dq, key row in dk/dv); group g takes the
// blocks j = g, g+2, ... and owns TMEM / shared-memory buffer g, so every scheduler has two element-wise warps to
// interleave and the exponentials of one block overlap the TMEM reads of the next.  Every wait is bounded and
// reports through the status buffer.
#include <climits>

#include "../common/host_utils.cuh"
#include "../common/ptx.cuh"
#include "attn_common.cuh"

using namespace mcb;

namespace {

constexpr int TM = 128;   // rows of the CTA's resident tile (TMEM lanes)
constexpr int BLK = 64;   // rows of the streamed blocks (MMA N for the score GEMMs, K for the gradient GEMMs)
constexpr int BWD_THREADS = 320;
constexpr float LOG2E = 1.4426950408889634f;

struct BwdParams {
  int T, Tk, nq, nkv, d;    // T queries, Tk keys
  float scale, scale_log2;
  const int* k_lo;          // [T] first visible key of each query
  const int* k_hi;          // [T] last visible key, or null: the query's own index
  const int* q_lo;          // [Tk] bounds on the queries that see each key, or null (causal self-attention)
  const int* q_hi;
  const float* lse;         // [nq, T]
  const float* delta;       // [nq, T]
  __nv_bfloat16* dq;        // [T, nq, d]
  __nv_bfloat16* dk;        // [Tk, nkv, d]
  __nv_bfloat16* dv;        // [Tk, nkv, d]
  int* status;
  float* partial;           // head-split mode: [2 (dv, dk), splits, Tk, nkv, d] fp32 partial sums, else null
  int splits;               // CTAs per (key tile, kv head); each takes qpg / splits query heads
};

// K-major operand: tile of `rows` x D stored as D/64 boxes of [rows x 64]; kk-th 16-wide slice of the reduction dim
__device__ __forceinline__ uint64_t kdesc(uint32_t base, int kk, int rows) {
  return make_smem_desc_sw128(base + (kk >> 2) * (rows * 128) + (kk & 3) * 32, 16, 1024);
}
// MN-major B operand: tile of `rows` (reduction dim) x D (N dim) in the same box layout; kk-th 16-row slice
__device__ __forceinline__ uint64_t mndesc(uint32_t base, int kk, int rows) {
  return make_smem_desc_sw128(base + kk * 2048, rows * 128, 1024);
}

__host__ __device__ constexpr uint32_t idesc(int m, int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(b_mn ? 1 : 0) << 16) | (uint32_t(n >> 3) << 17) |
         (uint32_t(m >> 4) << 24);
}

// writes 32 consecutive bf16 of row r (columns c..c+31 of a [128 x 64] K-major swizzled tile)
__device__ __forceinline__ void store_row_chunk(uint8_t* tile, int r, int c, const float* x) {
  uint8_t* row = tile + r * 128;
#pragma unroll
  for (int e = 0; e < 32; e += 8) {
    uint4 o;
    o.x = pack_bf16x2(x[e], x[e + 1]);
    o.y = pack_bf16x2(x[e + 2], x[e + 3]);
    o.z = pack_bf16x2(x[e + 4], x[e + 5]);
    o.w = pack_bf16x2(x[e + 6], x[e + 7]);
    const int chunk = (c + e) >> 3;
    *reinterpret_cast<uint4*>(row + ((chunk ^ (r & 7)) << 4)) = o;
  }
}

// one TMEM lane's D accumulator columns -> a bf16 row in global memory
template <int COLS>
__device__ __forceinline__ void store_acc_row(uint32_t taddr, __nv_bfloat16* dst, bool ok) {
#pragma unroll 1
  for (int c = 0; c < COLS; c += 32) {
    uint32_t v[32];
    tmem_ld_32x32(taddr + c, v);
    tmem_ld_wait();
    if (ok) {
#pragma unroll
      for (int e = 0; e < 32; e += 8) {
        uint4 o;
        o.x = pack_bf16x2(__uint_as_float(v[e]), __uint_as_float(v[e + 1]));
        o.y = pack_bf16x2(__uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
        o.z = pack_bf16x2(__uint_as_float(v[e + 4]), __uint_as_float(v[e + 5]));
        o.w = pack_bf16x2(__uint_as_float(v[e + 6]), __uint_as_float(v[e + 7]));
        *reinterpret_cast<uint4*>(dst + c + e) = o;
      }
    }
  }
}

// one TMEM lane's accumulator columns -> an fp32 row in global memory
template <int COLS>
__device__ __forceinline__ void store_acc_row_f32(uint32_t taddr, float* dst, bool ok) {
#pragma unroll 1
  for (int c = 0; c < COLS; c += 32) {
    uint32_t v[32];
    tmem_ld_32x32(taddr + c, v);
    tmem_ld_wait();
    if (ok) {
#pragma unroll
      for (int e = 0; e < 32; e += 4)
        *reinterpret_cast<uint4*>(dst + c + e) = make_uint4(v[e], v[e + 1], v[e + 2], v[e + 3]);
    }
  }
}

__device__ __forceinline__ void drain(uint64_t* bar, uint32_t it) {
  uint64_t t0 = globaltimer_ns();
  while (!mbar_try_wait(smem_u32(bar), (it >> 1) & 1))
    if (globaltimer_ns() - t0 > 200000000ull) break;
}

// ---------------------------------------------------------------------------------------------------- delta
template <int D>
__global__ void attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                      float* __restrict__ delta, int T, int nq) {
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= (long long)T * nq) return;
  const int i = int(w / nq), h = int(w % nq);
  const __nv_bfloat16* po = o + w * D;
  const __nv_bfloat16* pd = dout + w * D;
  float acc = 0.f;
  for (int c = lane * 2; c < D; c += 64) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(po + c);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(pd + c);
    acc += __bfloat162float(a.x) * __bfloat162float(b.x) + __bfloat162float(a.y) * __bfloat162float(b.y);
  }
#pragma unroll
  for (int s = 16; s; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[(long long)h * T + i] = acc;
}

// ---------------------------------------------------------------------------------------------------- dQ
template <int D>
struct DqSmem {
  static constexpr int TILE = TM * D * 2;
  static constexpr int BLOCK = BLK * D * 2;
  static constexpr int DS = TM * BLK * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = TILE;
  static constexpr int OFF_K = 2 * TILE;               // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * BLOCK;      // 2 stages
  static constexpr int OFF_DS = OFF_V + 2 * BLOCK;     // 2 buffers
  static constexpr int OFF_BAR = OFF_DS + 2 * DS;
  static constexpr int TOTAL = OFF_BAR + 1024 + 1024;
};

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                   const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                   const BwdParams p) {
  using L = DqSmem<D>;
  constexpr int NBOX = D / 64;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DQ = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars;             // 1
  uint64_t* kv_full = bars + 1;        // 2
  uint64_t* kv_empty = bars + 3;       // 2
  uint64_t* s_full = bars + 5;         // 2
  uint64_t* s_empty = bars + 7;        // 2
  uint64_t* ds_full = bars + 9;        // 2
  uint64_t* ds_empty = bars + 11;      // 2
  uint64_t* dq_full = bars + 13;       // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tile = gridDim.x - 1 - blockIdx.x;
  const int head = blockIdx.y;
  const int kvh = head / (p.nq / p.nkv);
  const int m0 = m_tile * TM;
  __shared__ int s_rng[8];
  tile_range_partial(p.k_lo, p.k_hi, m0, p.T, s_rng);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(q_full), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&kv_full[i]), 1);
      mbar_init(smem_u32(&kv_empty[i]), 1);
      mbar_init(smem_u32(&s_full[i]), 1);
      mbar_init(smem_u32(&s_empty[i]), 4);
      mbar_init(smem_u32(&ds_full[i]), 128);
      mbar_init(smem_u32(&ds_empty[i]), 1);
    }
    mbar_init(smem_u32(dq_full), 1);
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_do);
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int kmin = tile_range_min(s_rng), kmax = tile_range_max(s_rng);
  const int kb0 = kmin / BLK;
  const int nblk = kmax >= kmin ? kmax / BLK - kb0 + 1 : 0;

  if (nblk <= 0) {
    // no row of this tile sees any key: its queries get a zero gradient
    if (warp >= 2) {
      const int grp = (warp - 2) >> 2;
      const int i = m0 + (warp & 3) * 32 + lane;
      if (i < p.T) {
        uint4* row = reinterpret_cast<uint4*>(p.dq + ((long long)i * p.nq + head) * D + grp * (D / 2));
#pragma unroll
        for (int c = 0; c < D / 16; ++c) row[c] = make_uint4(0, 0, 0, 0);
      }
    }
  } else if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(smem_u32(q_full), 2 * L::TILE);
#pragma unroll
      for (int b = 0; b < NBOX; ++b) {
        tma_load_2d(smem_u32(smem + L::OFF_Q + b * TM * 128), &tm_q, head * D + b * 64, m0, smem_u32(q_full));
        tma_load_2d(smem_u32(smem + L::OFF_DO + b * TM * 128), &tm_do, head * D + b * 64, m0, smem_u32(q_full));
      }
      int j = 0;
      for (; j < nblk; ++j) {
        const uint32_t st = j & 1, ph = (j >> 1) & 1;
        const int n0 = (kb0 + j) * BLK;
        if (!mbar_wait(smem_u32(&kv_empty[st]), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(smem_u32(&kv_full[st]), 2 * L::BLOCK);
#pragma unroll
        for (int b = 0; b < NBOX; ++b) {
          tma_load_2d(smem_u32(smem + L::OFF_K + st * L::BLOCK + b * BLK * 128), &tm_k, kvh * D + b * 64, n0,
                      smem_u32(&kv_full[st]));
          tma_load_2d(smem_u32(smem + L::OFF_V + st * L::BLOCK + b * BLK * 128), &tm_v, kvh * D + b * 64, n0,
                      smem_u32(&kv_full[st]));
        }
      }
      for (int i = (j > 2 ? j - 2 : 0); i < j; ++i) drain(&kv_full[i & 1], i);   // loads land before the CTA exits
      drain(q_full, 0);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc(TM, BLK, false);
      constexpr uint32_t idesc_dq = idesc(TM, D, true);
      const uint32_t sq = smem_u32(smem + L::OFF_Q), sdo = smem_u32(smem + L::OFF_DO);
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, p.status, ST_TIMEOUT_FULL);
      auto issue_sdp = [&](int j) -> bool {
        const uint32_t st = j & 1, ph = (j >> 1) & 1;
        if (!mbar_wait(smem_u32(&kv_full[st]), ph, abort_flag, p.status, ST_TIMEOUT_FULL)) return false;
        if (!mbar_wait(smem_u32(&s_empty[st]), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + L::OFF_K + st * L::BLOCK);
        const uint32_t sv = smem_u32(smem + L::OFF_V + st * L::BLOCK);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16(tmem + COL_S + st * BLK, kdesc(sq, kk, TM), kdesc(sk, kk, BLK), idesc_s, kk ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16(tmem + COL_DP + st * BLK, kdesc(sdo, kk, TM), kdesc(sv, kk, BLK), idesc_s, kk ? 1u : 0u);
        umma_commit(smem_u32(&s_full[st]));
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) {
          ok = issue_sdp(j + 1);
          if (!ok) break;
        }
        const uint32_t st = j & 1, ph = (j >> 1) & 1;
        if (!mbar_wait(smem_u32(&ds_full[st]), ph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sds = smem_u32(smem + L::OFF_DS + st * L::DS);
        const uint32_t sk = smem_u32(smem + L::OFF_K + st * L::BLOCK);
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk)
          umma_f16(tmem + COL_DQ, kdesc(sds, kk, TM), mndesc(sk, kk, BLK), idesc_dq, (j | kk) ? 1u : 0u);
        umma_commit(smem_u32(&ds_empty[st]));
        umma_commit(smem_u32(&kv_empty[st]));
      }
      if (ok) umma_commit(smem_u32(dq_full));
    }
  } else {
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;
    const int r = q * 32 + lane;
    const int i = m0 + r;
    const bool row_ok = i < p.T;
    int lo, hi;
    attn_row_range(p.k_lo, p.k_hi, i, p.T, lo, hi);
    // a query that sees nothing has lse = -inf; its masked probabilities are zeroed below, keep the arithmetic finite
    const float lse_i = row_ok ? p.lse[(long long)head * p.T + i] : 0.f;
    const float lse2 = (lse_i == -INFINITY) ? 0.f : lse_i * LOG2E;
    const float dl = row_ok ? p.delta[(long long)head * p.T + i] : 0.f;
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    const uint32_t st = grp;
    bool ok = true;
    for (int j = grp; j < nblk && ok; j += 2) {
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(smem_u32(&s_full[st]), ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      if (!mbar_wait(smem_u32(&ds_empty[st]), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
      tc_fence_after();
      const int n0 = (kb0 + j) * BLK;
      const bool full = (lo <= n0) && (n0 + BLK - 1 <= hi);
      uint8_t* tile = smem + L::OFF_DS + st * L::DS;
#pragma unroll 1
      for (int c = 0; c < BLK; c += 32) {
        uint32_t s[32], dp[32];
        tmem_ld_32x32(tmem + lane_addr + COL_S + st * BLK + c, s);
        tmem_ld_32x32(tmem + lane_addr + COL_DP + st * BLK + c, dp);
        tmem_ld_wait();
        float ds[32];
        if (full) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const float pr = exp2f(__uint_as_float(s[e]) * p.scale_log2 - lse2);
            ds[e] = pr * (__uint_as_float(dp[e]) - dl) * p.scale;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int key = n0 + c + e;
            const float pr = exp2f(__uint_as_float(s[e]) * p.scale_log2 - lse2);
            ds[e] = (key >= lo && key <= hi) ? pr * (__uint_as_float(dp[e]) - dl) * p.scale : 0.f;
          }
        }
        store_row_chunk(tile, r, c, ds);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_empty[st]));
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&ds_full[st]));
    }
    if (ok && mbar_wait(smem_u32(dq_full), 0, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      // each group writes half of the row
      store_acc_row<D / 2>(tmem + lane_addr + COL_DQ + grp * (D / 2),
                           p.dq + ((long long)i * p.nq + head) * D + grp * (D / 2), row_ok);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------------- dK / dV
template <int D>
struct DkvSmem {
  static constexpr int TILE = TM * D * 2;
  static constexpr int BLOCK = BLK * D * 2;
  static constexpr int PT = TM * BLK * 2;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE;
  static constexpr int OFF_Q = 2 * TILE;                // 2 stages
  static constexpr int OFF_DO = OFF_Q + 2 * BLOCK;      // 2 stages
  static constexpr int OFF_P = OFF_DO + 2 * BLOCK;      // 2 buffers
  static constexpr int OFF_DS = OFF_P + 2 * PT;         // 2 buffers
  static constexpr int OFF_COL = OFF_DS + 2 * PT;       // per-column lse / delta / k_lo / k_hi + 4 ints of block
                                                        // bounds, 2 buffers per group
  static constexpr int COL_BYTES = 4 * BLK * 4 + 16;
  static constexpr int OFF_BAR = OFF_COL + 4 * COL_BYTES;
  static constexpr int TOTAL = OFF_BAR + 1024 + 1024;
};

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                    const BwdParams p) {
  using L = DkvSmem<D>;
  constexpr int NBOX = D / 64;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DV = 256, COL_DK = 256 + D;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* kv_full = bars;            // 1
  uint64_t* qdo_full = bars + 1;       // 2
  uint64_t* qdo_empty = bars + 3;      // 2
  uint64_t* s_full = bars + 5;         // 2
  uint64_t* s_empty = bars + 7;        // 2
  uint64_t* pds_full = bars + 9;       // 2
  uint64_t* pds_empty = bars + 11;     // 2
  uint64_t* out_full = bars + 13;      // 1
  uint64_t* col_full = bars + 14;      // 4
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* i_end_slot = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.y;
  const int qpg = p.nq / p.nkv;
  const int n0 = blockIdx.x * TM;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(kv_full), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&qdo_full[i]), 1);
      mbar_init(smem_u32(&qdo_empty[i]), 1);
      mbar_init(smem_u32(&s_full[i]), 1);
      mbar_init(smem_u32(&s_empty[i]), 4);
      mbar_init(smem_u32(&pds_full[i]), 128);
      mbar_init(smem_u32(&pds_empty[i]), 1);
      mbar_init(smem_u32(&col_full[i]), 128);
      mbar_init(smem_u32(&col_full[2 + i]), 128);
    }
    mbar_init(smem_u32(out_full), 1);
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tensormap(&tm_k);
    prefetch_tensormap(&tm_v);
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_do);
    if (p.q_lo == nullptr) {
      // causal self-attention: the last query that can see a key of this tile is the largest i with
      // k_lo[i] <= last key (k_lo = sequence starts, sorted); the first one is the tile's first key itself
      const int n_last = min(n0 + TM - 1, p.Tk - 1);
      int lo = n_last, hi = p.T - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (p.k_lo[mid] <= n_last) lo = mid; else hi = mid - 1;
      }
      i_end_slot[0] = n0;
      i_end_slot[1] = lo;
    }
  }
  __shared__ int s_rng[8];
  if (p.q_lo != nullptr) tile_range_partial(p.q_lo, p.q_hi, n0, p.Tk, s_rng);
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int i_first = p.q_lo ? tile_range_min(s_rng) : i_end_slot[0];
  const int i_last = p.q_lo ? min(tile_range_max(s_rng), p.T - 1) : i_end_slot[1];
  const int qb0 = i_first / BLK;
  const int nqb = i_last >= i_first ? i_last / BLK - qb0 + 1 : 0;   // 0: no query sees a key of this tile
  const int hps = qpg / p.splits;                 // query heads handled by this CTA
  const int h_first = kvh * qpg + blockIdx.z * hps;
  const int iters = hps * nqb;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(smem_u32(kv_full), 2 * L::TILE);
#pragma unroll
      for (int b = 0; b < NBOX; ++b) {
        tma_load_2d(smem_u32(smem + L::OFF_K + b * TM * 128), &tm_k, kvh * D + b * 64, n0, smem_u32(kv_full));
        tma_load_2d(smem_u32(smem + L::OFF_V + b * TM * 128), &tm_v, kvh * D + b * 64, n0, smem_u32(kv_full));
      }
      int it = 0;
      for (; it < iters; ++it) {
        const uint32_t st = it & 1, ph = (it >> 1) & 1;
        const int h = h_first + it / nqb;
        const int i0 = (qb0 + it % nqb) * BLK;
        if (!mbar_wait(smem_u32(&qdo_empty[st]), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(smem_u32(&qdo_full[st]), 2 * L::BLOCK);
#pragma unroll
        for (int b = 0; b < NBOX; ++b) {
          tma_load_2d(smem_u32(smem + L::OFF_Q + st * L::BLOCK + b * BLK * 128), &tm_q, h * D + b * 64, i0,
                      smem_u32(&qdo_full[st]));
          tma_load_2d(smem_u32(smem + L::OFF_DO + st * L::BLOCK + b * BLK * 128), &tm_do, h * D + b * 64, i0,
                      smem_u32(&qdo_full[st]));
        }
      }
      for (int i = (it > 2 ? it - 2 : 0); i < it; ++i) drain(&qdo_full[i & 1], i);
      drain(kv_full, 0);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc(TM, BLK, false);
      constexpr uint32_t idesc_o = idesc(TM, D, true);
      const uint32_t sk = smem_u32(smem + L::OFF_K), sv = smem_u32(smem + L::OFF_V);
      bool ok = mbar_wait(smem_u32(kv_full), 0, abort_flag, p.status, ST_TIMEOUT_FULL);
      auto issue_sdp = [&](int it) -> bool {
        const uint32_t st = it & 1, ph = (it >> 1) & 1;
        if (!mbar_wait(smem_u32(&qdo_full[st]), ph, abort_flag, p.status, ST_TIMEOUT_FULL)) return false;
        if (!mbar_wait(smem_u32(&s_empty[st]), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t sq = smem_u32(smem + L::OFF_Q + st * L::BLOCK);
        const uint32_t sdo = smem_u32(smem + L::OFF_DO + st * L::BLOCK);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16(tmem + COL_S + st * BLK, kdesc(sk, kk, TM), kdesc(sq, kk, BLK), idesc_s, kk ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16(tmem + COL_DP + st * BLK, kdesc(sv, kk, TM), kdesc(sdo, kk, BLK), idesc_s, kk ? 1u : 0u);
        umma_commit(smem_u32(&s_full[st]));
        return true;
      };
      if (ok && iters > 0) ok = issue_sdp(0);
      for (int it = 0; it < iters && ok; ++it) {
        if (it + 1 < iters) {
          ok = issue_sdp(it + 1);
          if (!ok) break;
        }
        const uint32_t st = it & 1, ph = (it >> 1) & 1;
        if (!mbar_wait(smem_u32(&pds_full[st]), ph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sp = smem_u32(smem + L::OFF_P + st * L::PT);
        const uint32_t sds = smem_u32(smem + L::OFF_DS + st * L::PT);
        const uint32_t sq = smem_u32(smem + L::OFF_Q + st * L::BLOCK);
        const uint32_t sdo = smem_u32(smem + L::OFF_DO + st * L::BLOCK);
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk)
          umma_f16(tmem + COL_DV, kdesc(sp, kk, TM), mndesc(sdo, kk, BLK), idesc_o, (it | kk) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < BLK / 16; ++kk)
          umma_f16(tmem + COL_DK, kdesc(sds, kk, TM), mndesc(sq, kk, BLK), idesc_o, (it | kk) ? 1u : 0u);
        umma_commit(smem_u32(&pds_empty[st]));
        umma_commit(smem_u32(&qdo_empty[st]));
      }
      if (ok) umma_commit(smem_u32(out_full));
    }
  } else {
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;
    const int r = q * 32 + lane;            // key row of this thread
    const int n = n0 + r;
    const bool row_ok = n < p.Tk;
    const int t = (threadIdx.x - 64) & 127; // 0..127 inside the group
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    const uint32_t st = grp;
    bool ok = true;
    for (int it = grp; it < iters && ok; it += 2) {
      const uint32_t ph = (it >> 1) & 1;
      const int h = h_first + it / nqb;
      const int i0 = (qb0 + it % nqb) * BLK;
      // per-column values of this query block; two buffers per group: a thread can run at most one of the group's
      // iterations ahead of the slowest reader, because passing col_full needs every thread's arrival
      const uint32_t cb = st * 2 + ph;
      float* col_lse = reinterpret_cast<float*>(smem + L::OFF_COL + cb * L::COL_BYTES);
      float* col_delta = col_lse + BLK;
      int* col_lo = reinterpret_cast<int*>(col_delta + BLK);
      int* col_hi = col_lo + BLK;
      int* col_meta = col_hi + BLK;            // [0..1] largest k_lo, [2..3] smallest k_hi of each half of the block
      {
        const int c = t & (BLK - 1);
        const int i = i0 + c;
        if (t < BLK) {
          int klo, khi;
          attn_row_range(p.k_lo, p.k_hi, i, p.T, klo, khi);
          col_lo[c] = klo;
          col_hi[c] = khi;
          int mxlo = klo, mnhi = khi;
#pragma unroll
          for (int sft = 16; sft; sft >>= 1) {
            mxlo = max(mxlo, __shfl_xor_sync(0xffffffffu, mxlo, sft));
            mnhi = min(mnhi, __shfl_xor_sync(0xffffffffu, mnhi, sft));
          }
          if ((t & 31) == 0) {
            col_meta[t >> 5] = mxlo;
            col_meta[2 + (t >> 5)] = mnhi;
          }
        } else {
          const float l = i < p.T ? p.lse[(long long)h * p.T + i] : 0.f;
          col_lse[c] = (l == -INFINITY) ? 0.f : l * LOG2E;    // such a query sees nothing: masked below
          col_delta[c] = i < p.T ? p.delta[(long long)h * p.T + i] : 0.f;
        }
      }
      mbar_arrive(smem_u32(&col_full[cb]));
      if (!mbar_wait(smem_u32(&col_full[cb]), (it >> 2) & 1, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
      if (!mbar_wait(smem_u32(&s_full[st]), ph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      if (!mbar_wait(smem_u32(&pds_empty[st]), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
      tc_fence_after();
      // every query of the block sees this key: largest lower bound <= n <= smallest upper bound
      const bool full = row_ok && max(col_meta[0], col_meta[1]) <= n && n <= min(col_meta[2], col_meta[3]);
      uint8_t* tile_p = smem + L::OFF_P + st * L::PT;
      uint8_t* tile_ds = smem + L::OFF_DS + st * L::PT;
#pragma unroll 1
      for (int c = 0; c < BLK; c += 32) {
        uint32_t s[32], dp[32];
        tmem_ld_32x32(tmem + lane_addr + COL_S + st * BLK + c, s);
        tmem_ld_32x32(tmem + lane_addr + COL_DP + st * BLK + c, dp);
        tmem_ld_wait();
        float pr[32], ds[32];
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(col_lse + c + e);
          const float4 d4 = *reinterpret_cast<const float4*>(col_delta + c + e);
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, dd[4] = {d4.x, d4.y, d4.z, d4.w};
          if (full) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const float x = exp2f(__uint_as_float(s[e + u]) * p.scale_log2 - ls[u]);
              pr[e + u] = x;
              ds[e + u] = x * (__uint_as_float(dp[e + u]) - dd[u]) * p.scale;
            }
          } else {
            const int4 s4 = *reinterpret_cast<const int4*>(col_lo + c + e);
            const int4 h4 = *reinterpret_cast<const int4*>(col_hi + c + e);
            const int ss[4] = {s4.x, s4.y, s4.z, s4.w}, hh[4] = {h4.x, h4.y, h4.z, h4.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const bool vis = row_ok && ss[u] <= n && n <= hh[u];
              const float x = exp2f(__uint_as_float(s[e + u]) * p.scale_log2 - ls[u]);
              pr[e + u] = vis ? x : 0.f;
              ds[e + u] = vis ? x * (__uint_as_float(dp[e + u]) - dd[u]) * p.scale : 0.f;
            }
          }
        }
        store_row_chunk(tile_p, r, c, pr);
        store_row_chunk(tile_ds, r, c, ds);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_empty[st]));
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(&pds_full[st]));
    }
    if (iters == 0) {
      // no query sees this tile's keys: zero gradients (the accumulators were never written)
      const long long row_off = ((long long)n * p.nkv + kvh) * D;
      if (row_ok) {
        if (p.partial == nullptr) {
          uint4* dst = reinterpret_cast<uint4*>((grp == 0 ? p.dv : p.dk) + row_off);
#pragma unroll 1
          for (int c = 0; c < D / 8; ++c) dst[c] = make_uint4(0, 0, 0, 0);
        } else {
          const long long plane = (long long)p.Tk * p.nkv * D;
          uint4* dst = reinterpret_cast<uint4*>(p.partial + ((long long)grp * p.splits + blockIdx.z) * plane + row_off);
#pragma unroll 1
          for (int c = 0; c < D / 4; ++c) dst[c] = make_uint4(0, 0, 0, 0);
        }
      }
    } else if (ok && mbar_wait(smem_u32(out_full), 0, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) {
      tc_fence_after();
      // group 0 writes dV, group 1 writes dK
      const long long row_off = ((long long)n * p.nkv + kvh) * D;
      if (p.partial == nullptr) {
        if (grp == 0) store_acc_row<D>(tmem + lane_addr + COL_DV, p.dv + row_off, row_ok);
        else store_acc_row<D>(tmem + lane_addr + COL_DK, p.dk + row_off, row_ok);
      } else {
        const long long plane = (long long)p.Tk * p.nkv * D;
        float* dst = p.partial + ((long long)grp * p.splits + blockIdx.z) * plane + row_off;
        store_acc_row_f32<D>(tmem + lane_addr + (grp == 0 ? COL_DV : COL_DK), dst, row_ok);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// sums the head-split partials: out[i] = sum_s partial[s][i] (fp32 -> bf16), 8 elements per thread
__global__ void attn_bwd_reduce_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ dv,
                                       __nv_bfloat16* __restrict__ dk, long long plane, int splits) {
  const long long i8 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i8 >= plane) return;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s2 = 0; s2 < splits; ++s2) {
      const float* src = partial + ((long long)which * splits + s2) * plane + i8;
      const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    *reinterpret_cast<uint4*>((which == 0 ? dv : dk) + i8) = o;
  }
}

template <int D>
int launch_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, float* delta,
               bool delta_given, const BwdParams& p, cudaStream_t stream) {
  const long long rows = (long long)p.T * p.nq;
  cudaError_t e = cudaSuccess;
  if (!delta_given) {
    attn_bwd_delta_kernel<D><<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(
        (const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta, p.T, p.nq);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  CUtensorMap tq128, tdo128, tk64, tv64, tk128, tv128, tq64, tdo64;
  const long long wq = (long long)p.nq * D, wk = (long long)p.nkv * D;
  int rc = 0;
  if ((rc = make_tmap_2d_bf16(&tq128, q, wq, p.T, wq, 64, TM))) return rc;
  if ((rc = make_tmap_2d_bf16(&tdo128, dout, wq, p.T, wq, 64, TM))) return rc;
  if ((rc = make_tmap_2d_bf16(&tk64, k, wk, p.Tk, wk, 64, BLK))) return rc;
  if ((rc = make_tmap_2d_bf16(&tv64, v, wk, p.Tk, wk, 64, BLK))) return rc;
  if ((rc = make_tmap_2d_bf16(&tk128, k, wk, p.Tk, wk, 64, TM))) return rc;
  if ((rc = make_tmap_2d_bf16(&tv128, v, wk, p.Tk, wk, 64, TM))) return rc;
  if ((rc = make_tmap_2d_bf16(&tq64, q, wq, p.T, wq, 64, BLK))) return rc;
  if ((rc = make_tmap_2d_bf16(&tdo64, dout, wq, p.T, wq, 64, BLK))) return rc;
  static bool cfg = false;
  if (!cfg) {
    e = cudaFuncSetAttribute(attn_bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, DqSmem<D>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(attn_bwd_dkv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvSmem<D>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    cfg = true;
  }
  const int tiles = (p.T + TM - 1) / TM, ktiles = (p.Tk + TM - 1) / TM;
  attn_bwd_dq_kernel<D><<<dim3(tiles, p.nq), BWD_THREADS, DqSmem<D>::TOTAL, stream>>>(tq128, tdo128, tk64, tv64, p);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  attn_bwd_dkv_kernel<D><<<dim3(ktiles, p.nkv, p.splits), BWD_THREADS, DkvSmem<D>::TOTAL, stream>>>(tk128, tv128, tq64,
                                                                                                     tdo64, p);
  e = cudaGetLastError();
  if (e != cudaSuccess || p.partial == nullptr) return (int)e;
  const long long plane = (long long)p.Tk * p.nkv * D;
  attn_bwd_reduce_kernel<<<(unsigned)((plane / 8 + 255) / 256), 256, 0, stream>>>(p.partial, p.dv, p.dk, plane,
                                                                                  p.splits);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

// General form.  q/o/dout/dq [T, nq, d], k/v/dk/dv [Tk, nkv, d] bf16 contiguous; lse, delta [nq, T] fp32 (delta is
// scratch filled here, or, with `delta_given`, read as passed: ring attention computes it once from the merged
// output).  k_lo / k_hi [T]: the forward's per-query key ranges (k_hi null = the query's index).  q_lo / q_hi [Tk]:
// per key, bounds on the queries that can see it (both null for causal self-attention).  `scale` is the softmax
// scale the forward used.
//
// Head split: with few kv heads and few key tiles the dK/dV grid (tiles x nkv CTAs) cannot fill the GPU.  Passing
// `splits` > 1 (a divisor of nq / nkv) and `partial` (fp32, 2 * splits * Tk * nkv * d elements) lets `splits` CTAs
// share a (tile, kv head) pair, each over nq / nkv / splits query heads; a reduction kernel sums their partial results.
int mcb_attn_bwd_ranges(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                        float* delta, int delta_given, const int* k_lo, const int* k_hi, const int* q_lo,
                        const int* q_hi, void* dq, void* dk, void* dv, int T, int Tk, int nq, int nkv, int d,
                        float scale, float* partial, int splits, int* status, void* stream_) {
  if (T == 0 || Tk == 0) return 0;
  if (nq % nkv || (k_hi == nullptr && Tk < T) || ((q_lo == nullptr) != (q_hi == nullptr))) return -2;
  if (q_lo == nullptr && k_hi != nullptr) return -2;   // general masks need the per-key query bounds
  if (splits < 1 || (nq / nkv) % splits) return -4;
  if (splits == 1) partial = nullptr;
  else if (partial == nullptr) return -5;
  BwdParams p{T, Tk, nq, nkv, d, scale, scale * LOG2E, k_lo, k_hi, q_lo, q_hi, lse, delta,
              (__nv_bfloat16*)dq, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, status, partial, splits};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  if (d == 128) return launch_bwd<128>(q, k, v, o, dout, delta, delta_given != 0, p, s);
  if (d == 64) return launch_bwd<64>(q, k, v, o, dout, delta, delta_given != 0, p, s);
  return -3;
}

// Packed causal self-attention: seq_start [T] int32 = first token of each token's sequence.
int mcb_attn_bwd_split(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                       float* delta, const int* seq_start, void* dq, void* dk, void* dv, int T, int nq, int nkv, int d,
                       float scale, float* partial, int splits, int* status, void* stream_) {
  return mcb_attn_bwd_ranges(q, k, v, o, dout, lse, delta, 0, seq_start, nullptr, nullptr, nullptr, dq, dk, dv, T, T, nq,
                             nkv, d, scale, partial, splits, status, stream_);
}

int mcb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                 float* delta, const int* seq_start, void* dq, void* dk, void* dv, int T, int nq, int nkv, int d,
                 float scale, int* status, void* stream_) {
  return mcb_attn_bwd_split(q, k, v, o, dout, lse, delta, seq_start, dq, dk, dv, T, nq, nkv, d, scale, nullptr, 1,
                            status, stream_);
}

}  // extern "C"

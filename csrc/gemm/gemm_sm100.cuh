// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared memory ->
// tcgen05.mma (accumulators in TMEM, double buffered) -> tcgen05.ld epilogue.
//
//   C[M,N] (+)= alpha * A[M,K] . B[N,K]^T (+ bias)
//
// Both operands may be K-major (row index slow, contraction index contiguous) or MN-major
// (contraction index slow), which covers forward (NT), dgrad (NN) and wgrad (TN) of a linear
// layer without any transposed copy.  Three scheduling modes share the kernel:
//   dense      one problem
//   grouped-M  rows of A/C are ragged per group (MoE experts, forward + dgrad); B is [G,N,K]
//   grouped-K  the contraction is ragged per group (MoE wgrad); C is [G,M,N]
// Group offsets are read on the device, so routing results never sync with the host.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2..5 = epilogue (each owns the 32 TMEM lanes its warp id % 4 selects).
#pragma once
#include "../common/ptx.cuh"

namespace mcb {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_MAX_GROUPS = 512;

enum GemmMode : int { GEMM_DENSE = 0, GEMM_GROUPED_M = 1, GEMM_GROUPED_K = 2 };
// Epilogues.  The cross-entropy ones belong to the fused language-model head (logits = h . W^T are never stored):
//   EPI_CE_STATS  per row and column tile, the running maximum and sum of exp(logit - max) over the tile's columns go
//                 to `ce_part`, and the logit of the row's label (when its column lies in the tile) to `ce_tgt`
//   EPI_CE_GRAD   C = (exp(logit - lse[row]) - [column == label]) * g[row] in bf16: the gradient w.r.t. the logits
enum GemmEpilogue : int { EPI_NONE = 0, EPI_CE_STATS = 2, EPI_CE_GRAD = 3 };

struct GemmParams {
  int M, N, K;          // dense: the problem.  grouped-M: M = upper bound on padded rows.
                        // grouped-K: M,N = per-group output, K unused (taken from offsets)
  void* C;
  long long ldc;        // elements
  long long c_group_stride;  // grouped-K: elements between consecutive group outputs
  const void* bias;     // optional, bf16 [N] (grouped-M: [G,N])
  int c_fp32;           // 0: bf16 output, 1: fp32 output
  int accumulate;       // C += ...  (1: as reductions at the L2; 2: read-add-write with prefetched old values)
  float alpha;
  int mode;
  int num_groups;
  const int* offsets;   // [G+1] device ints; multiples of 128
  int b_group_rows;     // grouped-M: rows between consecutive groups in the 2-D view of B
  int epilogue;         // EPI_*
  const long long* ce_labels;  // [M] global label of each row (cross-entropy epilogues)
  int ce_col0;                 // global index of this shard's column 0 (vocab-parallel head)
  float* ce_part;              // EPI_CE_STATS: [M, tiles_n, 2] (max, sum exp) per row and column tile
  float* ce_tgt;               // EPI_CE_STATS: [M] label logit, written by the tile that holds the label's column
  const float* ce_lse;         // EPI_CE_GRAD: [M] log-sum-exp over the whole vocabulary
  const float* ce_g;           // EPI_CE_GRAD: [M] upstream gradient of each row's loss
  int* status;          // device status word, 0 = ok
};

template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN >= 256) ? 4 : (BN >= 128 ? 6 : 8);
  static constexpr int BAR_BYTES = 1024;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // +1024 alignment slack
};

// C[row, n0 .. n0 + BN) += alpha * accumulator row, fp32, for tiles whose valid columns are a multiple of 32.  The old
// values of two 32-column chunks ahead are already on their way while the current chunk is added and stored, which
// keeps about 32 KiB of reads in flight per SM: short-K problems (expert weight gradients) have many output tiles per
// unit of math, and an epilogue that waits for each chunk's read, or 16-byte reductions that queue at the L2's
// atomic units, would bound them.
template <int BN>
__device__ __forceinline__ void epilogue_accumulate_fp32(uint32_t tmem_row, float* crow, int chunks, bool row_ok,
                                                         float alpha) {
  float4 nxt[2][8];
#pragma unroll
  for (int a = 0; a < 2; ++a)
    if (row_ok && a < chunks) {
#pragma unroll
      for (int j = 0; j < 8; ++j) nxt[a][j] = *reinterpret_cast<const float4*>(crow + a * 32 + j * 4);
    }
#pragma unroll 1
  for (int ch = 0; ch < chunks; ch += 2) {
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      if (ch + a >= chunks) break;
      float4 cur[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) cur[j] = nxt[a][j];
      if (row_ok && ch + a + 2 < chunks) {
#pragma unroll
        for (int j = 0; j < 8; ++j) nxt[a][j] = *reinterpret_cast<const float4*>(crow + (ch + a + 2) * 32 + j * 4);
      }
      uint32_t r[32];
      tmem_ld_32x32(tmem_row + (ch + a) * 32, r);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          cur[j].x += __uint_as_float(r[4 * j]) * alpha;
          cur[j].y += __uint_as_float(r[4 * j + 1]) * alpha;
          cur[j].z += __uint_as_float(r[4 * j + 2]) * alpha;
          cur[j].w += __uint_as_float(r[4 * j + 3]) * alpha;
          *reinterpret_cast<float4*>(crow + (ch + a) * 32 + j * 4) = cur[j];
        }
      }
    }
  }
}

struct TileCoord {
  int m0, n0;        // output tile origin (row within C / group output)
  int k_begin, k_end;  // contraction range in elements
  int group;
  int m_limit;       // rows valid: row < m_limit are stored
  int a_row0;        // row coordinate for A loads (K-major A) / mn coordinate (MN-major A)
  int b_row0;        // row coordinate for B loads
  bool valid;
};

// Maps a linear tile id to coordinates.  Identical in all three roles.
struct TileScheduler {
  const GemmParams& p;
  const int* s_off;  // offsets staged in shared memory (grouped modes)
  int tiles_m, tiles_n, total;
  int BN;
  __device__ TileScheduler(const GemmParams& p_, const int* s_off_, int bn) : p(p_), s_off(s_off_), BN(bn) {
    tiles_m = (p.M + GEMM_BM - 1) / GEMM_BM;
    tiles_n = (p.N + BN - 1) / BN;
    total = tiles_m * tiles_n * (p.mode == GEMM_GROUPED_K ? p.num_groups : 1);
  }
  __device__ TileCoord get(int t) const {
    TileCoord c;
    c.valid = true;
    int per_group = tiles_m * tiles_n;
    int g = 0;
    if (p.mode == GEMM_GROUPED_K) {
      g = t / per_group;
      t -= g * per_group;
    }
    // supergroups of 8 m-tiles walk n fastest inside -> the B panel stays in L2 for 8 row blocks
    constexpr int G = 8;
    int per_sg = G * tiles_n;
    int sg = t / per_sg;
    int first_m = sg * G;
    int gsize = min(tiles_m - first_m, G);
    int r = t - sg * per_sg;
    int tm = first_m + r % gsize;
    int tn = r / gsize;
    c.m0 = tm * GEMM_BM;
    c.n0 = tn * BN;
    c.group = g;
    c.k_begin = 0;
    c.k_end = p.K;
    c.m_limit = p.M;
    c.a_row0 = c.m0;
    c.b_row0 = c.n0;
    if (p.mode == GEMM_GROUPED_M) {
      int total_rows = s_off[p.num_groups];
      if (c.m0 >= total_rows) {
        c.valid = false;
        return c;
      }
      int lo = 0, hi = p.num_groups - 1;  // last group with offset <= m0
      while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if (s_off[mid] <= c.m0) lo = mid; else hi = mid - 1;
      }
      c.group = lo;
      c.m_limit = s_off[lo + 1];
      c.b_row0 = lo * p.b_group_rows + c.n0;
    } else if (p.mode == GEMM_GROUPED_K) {
      c.k_begin = s_off[g];
      c.k_end = s_off[g + 1];
    }
    return c;
  }
};

template <int BN, bool A_MN, bool B_MN, int EPI = EPI_NONE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const GemmParams p) {
  using L = GemmSmem<BN>;
  constexpr int STAGES = L::STAGES;
  constexpr uint32_t TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;  // two accumulators
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * L::STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  __shared__ int s_off[GEMM_MAX_GROUPS + 1];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (p.mode != GEMM_DENSE) {
    for (int i = threadIdx.x; i <= p.num_groups; i += blockDim.x) s_off[i] = p.offsets[i];
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tfull_bar[a]), 1);
      mbar_init(smem_u32(&tempty_bar[a]), 4);  // one arrive per epilogue warp
    }
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  TileScheduler sched(p, s_off, BN);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;  // global k-block counter -> stage / phase
      bool ok = true;
      for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
        TileCoord c = sched.get(t);
        if (!c.valid) continue;
        for (int k = c.k_begin; k < c.k_end; k += GEMM_BK, ++it) {
          const uint32_t s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          const uint32_t fb = smem_u32(&full_bar[s]);
          mbar_expect_tx(fb, L::STAGE_BYTES);
          const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
          if (!A_MN) {
            tma_load_2d(sa, &tmap_a, k, c.a_row0, fb);
          } else {
#pragma unroll
            for (int j = 0; j < GEMM_BM / 64; ++j) tma_load_2d(sa + j * 8192, &tmap_a, c.a_row0 + j * 64, k, fb);
          }
          if (!B_MN) {
            if (BN <= 256) tma_load_2d(sb, &tmap_b, k, c.b_row0, fb);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) {
              int krow = (p.mode == GEMM_GROUPED_M) ? (c.group * p.b_group_rows + k) : k;
              tma_load_2d(sb + j * 8192, &tmap_b, c.n0 + j * 64, krow, fb);
            }
          }
        }
      }
      // drain: every load this thread issued must have landed before the CTA may exit
      uint32_t first = it > STAGES ? it - STAGES : 0;
      for (uint32_t j = first; j < it; ++j) {
        const uint32_t s = j % STAGES, ph = (j / STAGES) & 1;
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(smem_u32(&full_bar[s]), ph)) {
          if (globaltimer_ns() - t0 > 200000000ull) break;  // 0.2 s per stage, then give up
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(GEMM_BM, BN, A_MN, B_MN);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
        TileCoord c = sched.get(t);
        if (!c.valid || c.k_end <= c.k_begin) continue;
        const uint32_t acc = lt & 1, aph = (lt >> 1) & 1;
        if (!mbar_wait(smem_u32(&tempty_bar[acc]), aph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool first = true;
        for (int k = c.k_begin; k < c.k_end; k += GEMM_BK, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, abort_flag, p.status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
            // K-major: 16 bf16 = 32 B inside the swizzle row.  MN-major: 16 k-rows = 2048 B.
            uint64_t ad = A_MN ? make_smem_desc_sw128(sa + kk * 2048, 8192, 1024)
                               : make_smem_desc_sw128(sa + kk * 32, 16, 1024);
            uint64_t bd = B_MN ? make_smem_desc_sw128(sb + kk * 2048, 8192, 1024)
                               : make_smem_desc_sw128(sb + kk * 32, 16, 1024);
            umma_f16(d_tmem, ad, bd, idesc, first ? 0u : 1u);
            first = false;
          }
          umma_commit(smem_u32(&empty_bar[s]));  // frees the smem stage when these MMAs retire
        }
        if (ok) umma_commit(smem_u32(&tfull_bar[acc]));
        ++lt;
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t lt = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < sched.total && ok; t += gridDim.x) {
      TileCoord c = sched.get(t);
      if (!c.valid) continue;
      const bool has_acc = c.k_end > c.k_begin;
      const uint32_t acc = lt & 1, aph = (lt >> 1) & 1;
      if (has_acc) {
        if (!mbar_wait(smem_u32(&tfull_bar[acc]), aph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) break;
        tc_fence_after();
      }
      const int row = c.m0 + q * 32 + lane;
      const bool row_ok = row < c.m_limit;
      const long long cbase = (p.mode == GEMM_GROUPED_K ? (long long)c.group * p.c_group_stride : 0ll) +
                              (long long)row * p.ldc;
      const __nv_bfloat16* bias =
          p.bias ? reinterpret_cast<const __nv_bfloat16*>(p.bias) + (p.mode == GEMM_GROUPED_M ? (long long)c.group * p.N : 0)
                 : nullptr;
      const bool vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
      if constexpr (EPI == EPI_CE_STATS || EPI == EPI_CE_GRAD) {
        // fused language-model head: one thread owns one row of the tile
        constexpr float LOG2E = 1.4426950408889634f;
        const int label_col = row_ok ? (int)(p.ce_labels[row] - p.ce_col0) - c.n0 : -1;   // column inside this tile
        float run_m = -INFINITY, run_s = 0.f, tgt = 0.f;
        const float lse2 = (EPI == EPI_CE_GRAD && row_ok) ? p.ce_lse[row] * LOG2E : 0.f;
        const float g = (EPI == EPI_CE_GRAD && row_ok) ? p.ce_g[row] : 0.f;
#pragma unroll 1
        for (int cc = 0; cc < BN; cc += 32) {
          if (c.n0 + cc >= p.N) break;
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + (uint32_t(q * 32) << 16) + acc * BN + cc, r);
          tmem_ld_wait();
          if (!row_ok) continue;
          const int valid = min(32, p.N - (c.n0 + cc));
          if constexpr (EPI == EPI_CE_STATS) {
            float cm = -INFINITY;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) cm = fmaxf(cm, __uint_as_float(r[j]) * p.alpha);
            const float nm = fmaxf(run_m, cm);
            float add = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < valid) add += exp2f((__uint_as_float(r[j]) * p.alpha - nm) * LOG2E);
            run_s = run_s * exp2f((run_m - nm) * LOG2E) + add;
            run_m = nm;
            const int lj = label_col - cc;
            if (lj >= 0 && lj < valid) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (j == lj) tgt = __uint_as_float(r[j]) * p.alpha;
            }
          } else {
            const int lj = label_col - cc;
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = (exp2f(__uint_as_float(r[j]) * p.alpha * LOG2E - lse2) - (j == lj ? 1.f : 0.f)) * g;
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + c.n0 + cc;
            if (vec_ok && valid == 32) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 o;
                o.x = pack_bf16x2(v[j], v[j + 1]);
                o.y = pack_bf16x2(v[j + 2], v[j + 3]);
                o.z = pack_bf16x2(v[j + 4], v[j + 5]);
                o.w = pack_bf16x2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(dst + j) = o;
              }
            } else {
              for (int j = 0; j < valid; ++j) dst[j] = __float2bfloat16(v[j]);
            }
          }
        }
        if constexpr (EPI == EPI_CE_STATS) {
          if (row_ok) {
            float* part = p.ce_part + ((long long)row * sched.tiles_n + c.n0 / BN) * 2;
            part[0] = run_m;
            part[1] = run_s;
            if (label_col >= 0 && label_col < BN && c.n0 + label_col < p.N) p.ce_tgt[row] = tgt;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
        ++lt;
        continue;
      }
      const int cols_valid = min(BN, p.N - c.n0);
      if (p.accumulate == 2 && p.c_fp32 && vec_ok && has_acc && !bias && cols_valid % 32 == 0) {
        epilogue_accumulate_fp32<BN>(tmem_base + (uint32_t(q * 32) << 16) + acc * BN,
                                     reinterpret_cast<float*>(p.C) + cbase + c.n0, cols_valid / 32, row_ok, p.alpha);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
        ++lt;
        continue;
      }
#pragma unroll 1
      for (int cc = 0; cc < BN; cc += 32) {
        if (c.n0 + cc >= p.N) break;  // whole chunk out of range (uniform across the warp)
        uint32_t r[32];
        if (has_acc) {
          tmem_ld_32x32(tmem_base + (uint32_t(q * 32) << 16) + acc * BN + cc, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0;
        }
        if (row_ok) {
          const int col0 = c.n0 + cc;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
          if (bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) v[j] += __bfloat162float(bias[col0 + j]);
          }
          if (p.c_fp32) {
            float* dst = reinterpret_cast<float*>(p.C) + cbase + col0;
            if (vec_ok && col0 + 32 <= p.N) {
              if (p.accumulate) {
                // C += tile as vector reductions performed at the L2: nothing is read back, so the epilogue does not
                // wait on memory latency (every output element belongs to exactly one tile: no ordering to respect)
#pragma unroll
                for (int j = 0; j < 32; j += 4) red_add_v4_f32(dst + j, v[j], v[j + 1], v[j + 2], v[j + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) dst[j] = p.accumulate ? dst[j] + v[j] : v[j];
            }
          } else {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + cbase + col0;
            if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (p.accumulate) {
                  uint4 old = *reinterpret_cast<uint4*>(dst + j);
                  const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    float2 f = __bfloat1622float2(ob[e]);
                    v[j + 2 * e] += f.x;
                    v[j + 2 * e + 1] += f.y;
                  }
                }
                uint4 o;
                o.x = pack_bf16x2(v[j], v[j + 1]);
                o.y = pack_bf16x2(v[j + 2], v[j + 3]);
                o.z = pack_bf16x2(v[j + 4], v[j + 5]);
                o.w = pack_bf16x2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(dst + j) = o;
              }
            } else {
              for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N)
                  dst[j] = __float2bfloat16(p.accumulate ? __bfloat162float(dst[j]) + v[j] : v[j]);
            }
          }
        }
      }
      if (has_acc) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
        ++lt;
      }
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace mcb

// Dense bf16 GEMM on CTA pairs: a cluster of two CTAs computes one 256 x 256 output tile with
// tcgen05.mma.cta_group::2.  Each CTA stages 128 rows of A and 128 of the tile's 256 B rows per k-block, so a
// k-block costs each SM 32 KiB of shared-memory traffic instead of the 48 KiB of the single-CTA 128 x 256 tile;
// the tensor cores of both SMs read both halves of B.  Each CTA keeps the 128 x 256 accumulator of its own rows
// in its TMEM (double buffered) and runs its own epilogue.
//
//   C[M,N] (+)= alpha * A[M,K] . B[N,K]^T (+ bias)        operands K-major or MN-major, as in gemm_sm100.cuh
//
// Roles per CTA (192 threads): warp 0 TMA producer, warp 1 TMEM owner (and, in the leader CTA only, MMA issuer),
// warps 2..5 epilogue.  Synchronisation across the pair:
//   full[s]    leader's barrier; both CTAs' TMA loads count their bytes on it (loads carry .cta_group::2, no multicast)
//   empty[s]   one per CTA; the leader commits to its own and to the peer's after the MMAs of the stage
//   tfull[a]   one per CTA; committed to both after the last MMA of a tile
//   tempty[a]  leader's barrier; the epilogue warps of both CTAs arrive on it (the peer's through the cluster)
// Every wait is bounded; a CTA that gives up raises its abort flag and falls through to the cluster barrier at the
// end, which its peer reaches after its own bounded waits.
#pragma once
#include "gemm_sm100.cuh"

namespace mcb {

constexpr int PAIR_BM = 256;        // rows of C per cluster (128 per CTA)
constexpr int PAIR_BN = 256;        // columns of C per cluster
constexpr int PAIR_HALF_N = 128;    // B rows staged per CTA
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_A_BYTES = GEMM_BM * GEMM_BK * 2;       // 16 KiB
constexpr int PAIR_B_BYTES = PAIR_HALF_N * GEMM_BK * 2;   // 16 KiB
constexpr int PAIR_STAGE_BYTES = PAIR_A_BYTES + PAIR_B_BYTES;
constexpr int PAIR_SMEM = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 1024;

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const GemmParams p) {
  constexpr int STAGES = PAIR_STAGES;
  constexpr uint32_t TMEM_COLS = 2 * PAIR_BN;  // two accumulators of 256 columns
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * PAIR_STAGE_BYTES);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + STAGES;
  uint64_t* tfull_bar = bars + 2 * STAGES;
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();       // 0 = leader
  const uint32_t peer = cta ^ 1u;
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);    // the leader's arrive.expect_tx
      mbar_init(smem_u32(&empty_bar[s]), 1);   // one commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tfull_bar[a]), 1);
      mbar_init(smem_u32(&tempty_bar[a]), 8);  // four epilogue warps in each CTA of the pair
    }
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // the peer's barriers exist before anything of this CTA can signal them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (p.M + PAIR_BM - 1) / PAIR_BM;
  const int tiles_n = (p.N + PAIR_BN - 1) / PAIR_BN;
  const int total = tiles_m * tiles_n;
  // supergroups of 4 row tiles walk the columns fastest inside, so a B panel is reused from L2 by 4 x 256 rows
  auto tile_of = [&](int t, int& tm, int& tn) {
    constexpr int G = 4;
    const int per_sg = G * tiles_n;
    const int sg = t / per_sg;
    const int first_m = sg * G;
    const int gsize = min(tiles_m - first_m, G);
    const int r = t - sg * per_sg;
    tm = first_m + r % gsize;
    tn = r / gsize;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = cluster_id; t < total && ok; t += num_clusters) {
        int tm, tn;
        tile_of(t, tm, tn);
        const int a_row0 = tm * PAIR_BM + (int)cta * GEMM_BM;          // this CTA's 128 rows of A / C
        const int b_row0 = tn * PAIR_BN + (int)cta * PAIR_HALF_N;      // this CTA's half of the tile's B rows
        for (int k = 0; k < p.K; k += GEMM_BK, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          // bytes of both CTAs are counted on the leader's barrier
          const uint32_t fb = mapa_shared(smem_u32(&full_bar[s]), 0);
          if (cta == 0) mbar_expect_tx(smem_u32(&full_bar[s]), 2 * PAIR_STAGE_BYTES);
          const uint32_t sa = smem_u32(smem + s * PAIR_STAGE_BYTES);
          const uint32_t sb = sa + PAIR_A_BYTES;
          if (!A_MN) {
            tma_load_2d_pair(sa, &tmap_a, k, a_row0, fb);
          } else {
#pragma unroll
            for (int j = 0; j < GEMM_BM / 64; ++j) tma_load_2d_pair(sa + j * 8192, &tmap_a, a_row0 + j * 64, k, fb);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tmap_b, k, b_row0, fb);
          } else {
#pragma unroll
            for (int j = 0; j < PAIR_HALF_N / 64; ++j) tma_load_2d_pair(sb + j * 8192, &tmap_b, b_row0 + j * 64, k, fb);
          }
        }
      }
      // drain: the loads of this CTA's last stages must have landed (their MMAs retired) before it may exit
      const uint32_t first = it > STAGES ? it - STAGES : 0;
      for (uint32_t j = first; j < it; ++j) {
        const uint32_t s = j % STAGES, ph = (j / STAGES) & 1;
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(smem_u32(&empty_bar[s]), ph)) {
          if (*abort_flag || globaltimer_ns() - t0 > 200000000ull) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(PAIR_BM, PAIR_BN, A_MN, B_MN);
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int t = cluster_id; t < total && ok; t += num_clusters, ++lt) {
        const uint32_t acc = lt & 1, aph = (lt >> 1) & 1;
        if (!mbar_wait(smem_u32(&tempty_bar[acc]), aph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * PAIR_BN;
        bool first = true;
        for (int k = 0; k < p.K; k += GEMM_BK, ++it) {
          const uint32_t s = it % STAGES, ph = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(&full_bar[s]), ph, abort_flag, p.status, ST_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * PAIR_STAGE_BYTES);
          const uint32_t sb = sa + PAIR_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
            const uint64_t ad = A_MN ? make_smem_desc_sw128(sa + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sa + kk * 32, 16, 1024);
            const uint64_t bd = B_MN ? make_smem_desc_sw128(sb + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(sb + kk * 32, 16, 1024);
            umma_f16_pair(d_tmem, ad, bd, idesc, first ? 0u : 1u);
            first = false;
          }
          // the stage is free in both CTAs once these MMAs retire
          umma_commit_pair(smem_u32(&empty_bar[s]));
          umma_commit_pair(mapa_shared(smem_u32(&empty_bar[s]), peer));
        }
        if (ok) {
          umma_commit_pair(smem_u32(&tfull_bar[acc]));
          umma_commit_pair(mapa_shared(smem_u32(&tfull_bar[acc]), peer));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int q = warp & 3;
    const uint32_t tempty_leader0 = mapa_shared(smem_u32(&tempty_bar[0]), 0);
    const uint32_t tempty_leader1 = mapa_shared(smem_u32(&tempty_bar[1]), 0);
    uint32_t lt = 0;
    for (int t = cluster_id; t < total; t += num_clusters, ++lt) {
      int tm, tn;
      tile_of(t, tm, tn);
      const uint32_t acc = lt & 1, aph = (lt >> 1) & 1;
      if (!mbar_wait(smem_u32(&tfull_bar[acc]), aph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int row = tm * PAIR_BM + (int)cta * GEMM_BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const int n0 = tn * PAIR_BN;
      const long long cbase = (long long)row * p.ldc;
      const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(p.bias);
      const bool vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
#pragma unroll 1
      for (int cc = 0; cc < PAIR_BN; cc += 32) {
        if (n0 + cc >= p.N) break;  // whole chunk out of range (uniform across the warp)
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (uint32_t(q * 32) << 16) + acc * PAIR_BN + cc, r);
        tmem_ld_wait();
        if (row_ok) {
          const int col0 = n0 + cc;
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
              if (p.accumulate) {   // vector reductions at the L2: no read-back latency in the epilogue
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
                  const uint4 old = *reinterpret_cast<uint4*>(dst + j);
                  const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(ob[e]);
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc ? tempty_leader1 : tempty_leader0);
    }
  }

  // ------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // neither CTA leaves while the other may still read its shared memory or signal its barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace mcb

// Block-scaled fp8 (e4m3) GEMM for sm_100a and its quantisation kernels.
//
//   C[M, N] (bf16) = sum_kb  sa[kb, m] * sb[n / 128, kb] * ( A8[m, kb*128 : kb*128+128] . B8[n, kb*128 : ...] )
//
// A8 [M, K] carries one fp32 scale per row per 128 columns (1 x 128 blocks, activations), B8 [N, K] one per
// 128 x 128 block (weights): the scaling of DeepSeek-V3 style fp8 training and of `weight_scale_inv` checkpoints.
// Because the scales are arbitrary fp32 numbers that change every 128 elements of K, each 128-deep partial product
// is formed on the tensor cores (tcgen05.mma kind::f8f6f4, fp32 accumulate in TMEM) and promoted into fp32
// registers with its scale by the epilogue warps; TMEM holds four partial products in flight so the tensor pipe
// does not wait for the promotion.
//
// Persistent kernel, 320 threads: warp 0 TMA producer (6-stage ring of 128 x 128-byte A and B tiles), warp 1 MMA
// issuer + TMEM owner, warps 2..9 promotion/epilogue (thread = row; warps 2..5 own columns 0..63 of the 128-wide tile,
// warps 6..9 columns 64..127).
#include <cuda_fp8.h>

#include "../common/host_utils.cuh"
#include "../common/ptx.cuh"

using namespace mcb;

namespace {

constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128;
constexpr int F8_STAGES = 6;
constexpr int F8_PARTS = 4;
constexpr int F8_THREADS = 320;
constexpr int F8_TILE_BYTES = F8_BM * F8_BK;   // one operand tile: 128 rows x 128 bytes
constexpr int F8_GROUP_M = 16;

struct Fp8Params {
  int M, N, K;
  const float* sa;       // [K/128, M]
  const float* sb;       // [ceil(N/128), K/128]
  __nv_bfloat16* c;      // [M, N]
  int* status;
};

struct Fp8Smem {
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = F8_STAGES * F8_TILE_BYTES;
  static constexpr int OFF_BAR = 2 * F8_STAGES * F8_TILE_BYTES;
  static constexpr int TOTAL = OFF_BAR + 1024 + 1024;
};

__host__ __device__ constexpr uint32_t idesc_e4m3(int m, int n) {
  // c_format f32 (bit 4), a/b format e4m3 (0), K-major operands, n >> 3 at bit 17, m >> 4 at bit 24
  return (1u << 4) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int& mt, int& nt) {
  const int per_group = F8_GROUP_M * n_tiles;
  const int g = tile / per_group;
  const int first_m = g * F8_GROUP_M;
  const int rows = min(F8_GROUP_M, m_tiles - first_m);
  const int in_g = tile - g * per_group;
  mt = first_m + in_g % rows;
  nt = in_g / rows;
}

__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const Fp8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Fp8Smem::OFF_BAR);
  uint64_t* full = bars;                              // STAGES
  uint64_t* empty = bars + F8_STAGES;                 // STAGES
  uint64_t* part_full = bars + 2 * F8_STAGES;         // PARTS
  uint64_t* part_empty = part_full + F8_PARTS;        // PARTS
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(part_empty + F8_PARTS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + F8_BM - 1) / F8_BM, n_tiles = (p.N + F8_BN - 1) / F8_BN;
  const int tiles = m_tiles * n_tiles;
  const int KB = p.K / F8_BK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < F8_STAGES; ++i) {
      mbar_init(smem_u32(&full[i]), 1);
      mbar_init(smem_u32(&empty[i]), 1);
    }
    for (int i = 0; i < F8_PARTS; ++i) {
      mbar_init(smem_u32(&part_full[i]), 1);
      mbar_init(smem_u32(&part_empty[i]), 8);
    }
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tensormap(&tm_a);
    prefetch_tensormap(&tm_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (p.status[0] != 0) goto done;   // an earlier kernel reported a failure: do not start new waits

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        int mt, nt;
        tile_coords(tile, m_tiles, n_tiles, mt, nt);
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const uint32_t s = it % F8_STAGES, ph = (it / F8_STAGES) & 1;
          if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(smem_u32(&full[s]), 2 * F8_TILE_BYTES);
          tma_load_2d(smem_u32(smem + Fp8Smem::OFF_A + s * F8_TILE_BYTES), &tm_a, kb * F8_BK, mt * F8_BM,
                      smem_u32(&full[s]));
          tma_load_2d(smem_u32(smem + Fp8Smem::OFF_B + s * F8_TILE_BYTES), &tm_b, kb * F8_BK, nt * F8_BN,
                      smem_u32(&full[s]));
        }
      }
      // the last loads must land before the CTA exits
      const uint32_t first = it > F8_STAGES ? it - F8_STAGES : 0;
      for (uint32_t i = first; i < it; ++i) {
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(smem_u32(&full[i % F8_STAGES]), (i / F8_STAGES) & 1))
          if (globaltimer_ns() - t0 > 200000000ull) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_e4m3(F8_BM, F8_BN);
      uint32_t it = 0, pc = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < KB; ++kb, ++it, ++pc) {
          const uint32_t s = it % F8_STAGES, ph = (it / F8_STAGES) & 1;
          const uint32_t pb = pc % F8_PARTS, pph = (pc / F8_PARTS) & 1;
          if (!mbar_wait(smem_u32(&part_empty[pb]), pph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&full[s]), ph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + Fp8Smem::OFF_A + s * F8_TILE_BYTES);
          const uint32_t sb = smem_u32(smem + Fp8Smem::OFF_B + s * F8_TILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < F8_BK / 32; ++kk)
            umma_f8f6f4(tmem + pb * F8_BN, make_smem_desc_sw128(sa + kk * 32, 16, 1024),
                        make_smem_desc_sw128(sb + kk * 32, 16, 1024), idesc, kk ? 1u : 0u);
          umma_commit(smem_u32(&empty[s]));
          umma_commit(smem_u32(&part_full[pb]));
        }
      }
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = q * 32 + lane;
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    uint32_t pc = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
      int mt, nt;
      tile_coords(tile, m_tiles, n_tiles, mt, nt);
      const int row = mt * F8_BM + r;
      const int row_c = min(row, p.M - 1);
      const float* sb_row = p.sb + (long long)nt * KB;
      float acc[64];
#pragma unroll
      for (int e = 0; e < 64; ++e) acc[e] = 0.f;
      // scales are fetched four k-blocks ahead into a register ring and multiplied only when used, so the global
      // load latency (longer than one k-block of tensor work) never stalls the in-order issue of this warp
      float ra[4], rb[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int kk = min(u, KB - 1);
        ra[u] = p.sa[(long long)kk * p.M + row_c];
        rb[u] = sb_row[kk];
      }
      for (int kb0 = 0; kb0 < KB && ok; kb0 += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int kb = kb0 + u;
          if (kb >= KB) break;
          const float sc = ra[u] * rb[u];
          const int kn = min(kb + 4, KB - 1);
          ra[u] = p.sa[(long long)kn * p.M + row_c];
          rb[u] = sb_row[kn];
          const uint32_t pb = pc % F8_PARTS, pph = (pc / F8_PARTS) & 1;
          ++pc;
          if (!mbar_wait(smem_u32(&part_full[pb]), pph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
          tc_fence_after();
          uint32_t v0[32], v1[32];
          tmem_ld_32x32(tmem + lane_addr + pb * F8_BN + half * 64, v0);
          tmem_ld_32x32(tmem + lane_addr + pb * F8_BN + half * 64 + 32, v1);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&part_empty[pb]));
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            acc[e] = fmaf(__uint_as_float(v0[e]), sc, acc[e]);
            acc[32 + e] = fmaf(__uint_as_float(v1[e]), sc, acc[32 + e]);
          }
        }
      }
      if (ok && row < p.M) {
        __nv_bfloat16* crow = p.c + (long long)row * p.N + nt * F8_BN + half * 64;
        const int col0 = nt * F8_BN + half * 64;
#pragma unroll
        for (int e = 0; e < 64; e += 8) {
          if (col0 + e + 8 <= p.N) {
            uint4 o;
            o.x = pack_bf16x2(acc[e], acc[e + 1]);
            o.y = pack_bf16x2(acc[e + 2], acc[e + 3]);
            o.z = pack_bf16x2(acc[e + 4], acc[e + 5]);
            o.w = pack_bf16x2(acc[e + 6], acc[e + 7]);
            *reinterpret_cast<uint4*>(crow + e) = o;
          }
        }
      }
    }
  }
done:
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---------------------------------------------------------------------------------------------- quantisation
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int s = 16; s; s >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, s));
  return v;
}

// x [M, K] bf16 -> x8 [M, K] e4m3, scales [K/128, M] (scale = amax / 448, value = x / scale); one warp per block
__global__ void quant_1x128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ x8,
                                   float* __restrict__ scales, int M, int K) {
  const int KB = K / 128;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (w >= (long long)M * KB) return;
  const int row = int(w / KB), kb = int(w % KB);
  const __nv_bfloat16* src = x + (long long)row * K + kb * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  float f[4] = {__bfloat162float(a.x), __bfloat162float(a.y), __bfloat162float(b.x), __bfloat162float(b.y)};
  float amax = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
  amax = warp_max(amax);
  const float scale = amax > 0.f ? amax * (1.f / 448.f) : 1.f;
  uint32_t out = 0;
#pragma unroll
  for (int e = 0; e < 4; ++e)   // IEEE division, so the result is the same as the torch restatement bit for bit
    out |= uint32_t(__nv_cvt_float_to_fp8(__fdiv_rn(f[e], scale), __NV_SATFINITE, __NV_E4M3)) << (8 * e);
  *reinterpret_cast<uint32_t*>(x8 + (long long)row * K + kb * 128 + lane * 4) = out;
  if (lane == 0) scales[(long long)kb * M + row] = scale;
}

// w [N, K] bf16 -> w8 [N, K] e4m3 with one scale per 128 x 128 block, scales [ceil(N/128), K/128].  Optionally also
// the transposed copy w8t [K, N_pad] (row length `ldt`) with scales_t [K/128, ceil(N/128)], for the data-gradient
// GEMM.  One 256-thread CTA per block.
__global__ void quant_128x128_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ w8,
                                     float* __restrict__ scales, uint8_t* __restrict__ w8t,
                                     float* __restrict__ scales_t, int N, int K, int ldt) {
  __shared__ float red[8];
  __shared__ uint8_t tile[128][128 + 4];
  const int KB = K / 128, NB = (N + 127) / 128;
  const int nb = blockIdx.x / KB, kb = blockIdx.x % KB;
  const int t = threadIdx.x;
  // thread t covers 4 consecutive columns (t % 32) * 4 of rows (t / 32) + 8 * i
  const int c4 = (t & 31) * 4, r0 = t >> 5;
  float f[16][4];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int row = nb * 128 + r0 + 8 * i;
    if (row < N) {
      const uint2 raw = *reinterpret_cast<const uint2*>(w + (long long)row * K + kb * 128 + c4);
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
      const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
      f[i][0] = __bfloat162float(a.x); f[i][1] = __bfloat162float(a.y);
      f[i][2] = __bfloat162float(b.x); f[i][3] = __bfloat162float(b.y);
    } else {
      f[i][0] = f[i][1] = f[i][2] = f[i][3] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) amax = fmaxf(amax, fabsf(f[i][e]));
  }
  amax = warp_max(amax);
  if ((t & 31) == 0) red[t >> 5] = amax;
  __syncthreads();
  amax = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
  const float scale = amax > 0.f ? amax * (1.f / 448.f) : 1.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int lr = r0 + 8 * i, row = nb * 128 + lr;
    uint32_t out = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e)
      out |= uint32_t(__nv_cvt_float_to_fp8(__fdiv_rn(f[i][e], scale), __NV_SATFINITE, __NV_E4M3)) << (8 * e);
    if (row < N) *reinterpret_cast<uint32_t*>(w8 + (long long)row * K + kb * 128 + c4) = out;
    if (w8t) *reinterpret_cast<uint32_t*>(&tile[lr][c4]) = out;
  }
  if (t == 0) {
    scales[(long long)nb * KB + kb] = scale;
    if (scales_t) scales_t[(long long)kb * NB + nb] = scale;
  }
  if (w8t) {
    __syncthreads();
    // transposed write: thread t covers 4 consecutive n of k-rows (t / 32) + 8 * i
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int lk = r0 + 8 * i;
      uint32_t out = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) out |= uint32_t(tile[c4 + e][lk]) << (8 * e);
      const int ncol = nb * 128 + c4;
      if (ncol + 4 <= ldt) *reinterpret_cast<uint32_t*>(w8t + (long long)(kb * 128 + lk) * ldt + ncol) = out;
    }
  }
}

}  // namespace

extern "C" {

// a8 [M, K], b8 [N, K] e4m3 bytes; sa [K/128, M], sb [ceil(N/128), K/128] fp32; c [M, N] bf16.  K % 128 == 0, N % 8 == 0.
int mcb_gemm_fp8_blockscaled(const void* a8, const float* sa, const void* b8, const float* sb, void* c, int M, int N,
                             int K, int* status, void* stream_) {
  if (M == 0 || N == 0) return 0;
  if (K % 128 != 0 || K == 0 || N % 8 != 0) return -2;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, a8, K, M, K, F8_BK, F8_BM, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  rc = make_tmap_2d(&tb, b8, K, N, K, F8_BK, F8_BN, 1, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Fp8Smem::TOTAL);
    if (e != cudaSuccess) return (int)e;
    cfg = true;
  }
  Fp8Params p{M, N, K, sa, sb, (__nv_bfloat16*)c, status};
  const int tiles = ((M + F8_BM - 1) / F8_BM) * ((N + F8_BN - 1) / F8_BN);
  const int grid = tiles < device_sm_count() ? tiles : device_sm_count();
  gemm_fp8_kernel<<<grid, F8_THREADS, Fp8Smem::TOTAL, reinterpret_cast<cudaStream_t>(stream_)>>>(ta, tb, p);
  return (int)cudaGetLastError();
}

int mcb_quant_fp8_1x128(const void* x, void* x8, float* scales, int M, int K, void* stream_) {
  if (M == 0) return 0;
  if (K % 128 != 0) return -2;
  const long long warps = (long long)M * (K / 128);
  quant_1x128_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      (const __nv_bfloat16*)x, (uint8_t*)x8, scales, M, K);
  return (int)cudaGetLastError();
}

// w8t / scales_t may be null.  `ldt` is the row length of w8t (>= N, multiple of 16 for the TMA descriptor).
int mcb_quant_fp8_128x128(const void* w, void* w8, float* scales, void* w8t, float* scales_t, int N, int K, int ldt,
                          void* stream_) {
  if (N == 0) return 0;
  if (K % 128 != 0) return -2;
  const int blocks = ((N + 127) / 128) * (K / 128);
  quant_128x128_kernel<<<blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      (const __nv_bfloat16*)w, (uint8_t*)w8, scales, (uint8_t*)w8t, scales_t, N, K, ldt);
  return (int)cudaGetLastError();
}

}  // extern "C"

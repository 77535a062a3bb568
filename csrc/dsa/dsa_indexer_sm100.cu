// DSA lightning indexer for sm_100a.
//
//   score[i, j] = sum_h  w[i, h] * relu( q[i, h, :] . k[j, :] )      for keys j visible to query i, else -inf
//
// followed by a per-row top-k selection.  q [T, H, 128] and k [T, 128] are bf16, w [T, H] fp32 (head weights with the
// softmax scale folded in), visibility is causal inside a packed sequence: seq_start[i] <= j <= i.
//
// Score kernel: persistent over the lower-triangular 128 x 128 (query x key) tiles.  The key tile stays in shared
// memory for the whole tile; the H query-head tiles stream through a 4-stage TMA ring; every head is one 128 x 128 x 128
// tcgen05 product into one of four TMEM buffers, which the eight epilogue warps (thread = query row, two column
// halves) turn into  acc += w * relu(.)  in registers.  After the last head the tile is written with the mask
// applied.  Tiles that lie entirely before the first visible key of their queries are not computed (the output is
// pre-filled with -inf by the caller).
//
// Top-k kernel: one CTA per row; a 4-pass radix select on the order-preserving integer image of the fp32 scores finds
// the k-th largest value, then the indices above it and as many equal to it as needed are written (unordered).
#include "../common/host_utils.cuh"
#include "../common/ptx.cuh"

using namespace mcb;

namespace {

constexpr int IX_TILE = 128, IX_D = 128;
constexpr int IX_STAGES = 4, IX_PARTS = 4, IX_THREADS = 320;
constexpr int IX_TILE_BYTES = IX_TILE * IX_D * 2;    // 32 KB

struct IxParams {
  int T, H;
  const float* w;          // [T, H]
  const int* seq_start;    // [T]
  float* out;              // [T, T]
  int* status;
};

struct IxSmem {
  static constexpr int OFF_K = 0;
  static constexpr int OFF_Q = IX_TILE_BYTES;
  static constexpr int OFF_BAR = IX_TILE_BYTES * (1 + IX_STAGES);
  static constexpr int TOTAL = OFF_BAR + 1024 + 1024;
};

__device__ __forceinline__ uint64_t ix_kdesc(uint32_t base, int kk) {
  return make_smem_desc_sw128(base + (kk >> 2) * (IX_TILE * 128) + (kk & 3) * 32, 16, 1024);
}

// tile id -> (query tile m, key tile n) with n <= m
__device__ __forceinline__ void tri_coords(int t, int& m, int& n) {
  m = int((sqrtf(8.f * float(t) + 1.f) - 1.f) * 0.5f);
  while ((m + 1) * (m + 2) / 2 <= t) ++m;
  while (m * (m + 1) / 2 > t) --m;
  n = t - m * (m + 1) / 2;
}

__global__ void __launch_bounds__(IX_THREADS, 1)
dsa_index_scores_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const IxParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + IxSmem::OFF_BAR);
  uint64_t* q_full = bars;                         // STAGES
  uint64_t* q_empty = bars + IX_STAGES;            // STAGES
  uint64_t* k_full = bars + 2 * IX_STAGES;         // 1
  uint64_t* k_empty = k_full + 1;                  // 1
  uint64_t* part_full = k_empty + 1;               // PARTS
  uint64_t* part_empty = part_full + IX_PARTS;     // PARTS
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(part_empty + IX_PARTS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mt_count = (p.T + IX_TILE - 1) / IX_TILE;
  const int tiles = mt_count * (mt_count + 1) / 2;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < IX_STAGES; ++i) {
      mbar_init(smem_u32(&q_full[i]), 1);
      mbar_init(smem_u32(&q_empty[i]), 1);
    }
    mbar_init(smem_u32(k_full), 1);
    mbar_init(smem_u32(k_empty), 1);
    for (int i = 0; i < IX_PARTS; ++i) {
      mbar_init(smem_u32(&part_full[i]), 1);
      mbar_init(smem_u32(&part_empty[i]), 8);
    }
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tensormap(&tm_q);
    prefetch_tensormap(&tm_k);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // every role walks the same tile list and skips the same tiles
  auto tile_active = [&](int tile, int& mt, int& nt) -> bool {
    tri_coords(tile, mt, nt);
    const int first_visible = p.seq_start[mt * IX_TILE];      // seq_start is non-decreasing
    return nt * IX_TILE + IX_TILE - 1 >= first_visible;
  };

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0, kt = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        int mt, nt;
        if (!tile_active(tile, mt, nt)) continue;
        if (!mbar_wait(smem_u32(k_empty), (kt & 1) ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) break;
        mbar_expect_tx(smem_u32(k_full), IX_TILE_BYTES);
        tma_load_2d(smem_u32(smem + IxSmem::OFF_K), &tm_k, 0, nt * IX_TILE, smem_u32(k_full));
        tma_load_2d(smem_u32(smem + IxSmem::OFF_K + IX_TILE * 128), &tm_k, 64, nt * IX_TILE, smem_u32(k_full));
        ++kt;
        for (int h = 0; h < p.H; ++h, ++it) {
          const uint32_t s = it % IX_STAGES, ph = (it / IX_STAGES) & 1;
          if (!mbar_wait(smem_u32(&q_empty[s]), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(smem_u32(&q_full[s]), IX_TILE_BYTES);
          uint8_t* dst = smem + IxSmem::OFF_Q + s * IX_TILE_BYTES;
          tma_load_2d(smem_u32(dst), &tm_q, h * IX_D, mt * IX_TILE, smem_u32(&q_full[s]));
          tma_load_2d(smem_u32(dst + IX_TILE * 128), &tm_q, h * IX_D + 64, mt * IX_TILE, smem_u32(&q_full[s]));
        }
      }
      const uint32_t first = it > IX_STAGES ? it - IX_STAGES : 0;
      for (uint32_t i = first; i < it; ++i) {
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(smem_u32(&q_full[i % IX_STAGES]), (i / IX_STAGES) & 1))
          if (globaltimer_ns() - t0 > 200000000ull) break;
      }
      if (kt) {
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(smem_u32(k_full), (kt - 1) & 1))
          if (globaltimer_ns() - t0 > 200000000ull) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(IX_TILE >> 3) << 17) |
                                 (uint32_t(IX_TILE >> 4) << 24);
      uint32_t it = 0, pc = 0, kt = 0;
      bool ok = true;
      const uint32_t sk = smem_u32(smem + IxSmem::OFF_K);
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        int mt, nt;
        if (!tile_active(tile, mt, nt)) continue;
        if (!mbar_wait(smem_u32(k_full), kt & 1, abort_flag, p.status, ST_TIMEOUT_FULL)) break;
        for (int h = 0; h < p.H; ++h, ++it, ++pc) {
          const uint32_t s = it % IX_STAGES, ph = (it / IX_STAGES) & 1;
          const uint32_t pb = pc % IX_PARTS, pph = (pc / IX_PARTS) & 1;
          if (!mbar_wait(smem_u32(&part_empty[pb]), pph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
          if (!mbar_wait(smem_u32(&q_full[s]), ph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sq = smem_u32(smem + IxSmem::OFF_Q + s * IX_TILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < IX_D / 16; ++kk)
            umma_f16(tmem + pb * IX_TILE, ix_kdesc(sq, kk), ix_kdesc(sk, kk), idesc, kk ? 1u : 0u);
          umma_commit(smem_u32(&q_empty[s]));
          umma_commit(smem_u32(&part_full[pb]));
        }
        umma_commit(smem_u32(k_empty));     // the key tile may be replaced once this tile's products are done
        ++kt;
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
      if (!tile_active(tile, mt, nt)) continue;
      const int row = mt * IX_TILE + r;
      const int row_c = min(row, p.T - 1);
      const float* wrow = p.w + (long long)row_c * p.H;
      float acc[64];
#pragma unroll
      for (int e = 0; e < 64; ++e) acc[e] = 0.f;
      float ring[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) ring[u] = wrow[min(u, p.H - 1)];
      for (int h0 = 0; h0 < p.H && ok; h0 += 4) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int h = h0 + u;
          if (h >= p.H) break;
          const float wv = ring[u];
          ring[u] = wrow[min(h + 4, p.H - 1)];
          const uint32_t pb = pc % IX_PARTS, pph = (pc / IX_PARTS) & 1;
          ++pc;
          if (!mbar_wait(smem_u32(&part_full[pb]), pph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
          tc_fence_after();
          uint32_t v0[32], v1[32];
          tmem_ld_32x32(tmem + lane_addr + pb * IX_TILE + half * 64, v0);
          tmem_ld_32x32(tmem + lane_addr + pb * IX_TILE + half * 64 + 32, v1);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&part_empty[pb]));
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            acc[e] = fmaf(fmaxf(__uint_as_float(v0[e]), 0.f), wv, acc[e]);
            acc[32 + e] = fmaf(fmaxf(__uint_as_float(v1[e]), 0.f), wv, acc[32 + e]);
          }
        }
      }
      if (ok && row < p.T) {
        const int lo = p.seq_start[row], hi = row;
        const int col0 = nt * IX_TILE + half * 64;
        float* orow = p.out + (long long)row * p.T + col0;
#pragma unroll
        for (int e = 0; e < 64; e += 4) {
          float4 o;
          float* of = reinterpret_cast<float*>(&o);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int key = col0 + e + u;
            of[u] = (key >= lo && key <= hi) ? acc[e + u] : -INFINITY;
          }
          if (col0 + e + 4 <= p.T) {
            *reinterpret_cast<float4*>(orow + e) = o;
          } else {
            for (int u = 0; u < 4; ++u)
              if (col0 + e + u < p.T) orow[e + u] = of[u];
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------------------------------------ top-k select
__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);      // larger float -> larger unsigned
}

// scores [rows, n] fp32 (row stride ld); idx [rows, k] int64: the positions of the k largest entries of each row
// (any order; ties at the threshold resolved towards smaller positions).  Entries equal to -inf are selected only
// when fewer than k finite entries exist, as with a sort-based top-k.
__global__ void __launch_bounds__(256)
topk_select_kernel(const float* __restrict__ scores, long long ld, int n, int k, long long* __restrict__ idx) {
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix, s_mask;
  __shared__ int s_remaining, s_above, s_equal;
  const float* row = scores + (long long)blockIdx.x * ld;
  long long* out = idx + (long long)blockIdx.x * k;
  if (threadIdx.x == 0) {
    s_prefix = 0;
    s_mask = 0;
    s_remaining = k;
  }
  __syncthreads();
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix, mask = s_mask;
    for (int j = threadIdx.x; j < n; j += blockDim.x) {
      const uint32_t key = order_key(row[j]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int remaining = s_remaining, b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= remaining) break;
        remaining -= hist[b];
      }
      s_prefix = prefix | (uint32_t(b) << shift);
      s_mask = mask | (0xffu << shift);
      s_remaining = remaining;       // how many entries with exactly this prefix are still needed
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix;     // key of the k-th largest entry
  const int need_equal = s_remaining;
  if (threadIdx.x == 0) {
    s_above = 0;
    s_equal = 0;
  }
  __syncthreads();
  // entries strictly above the threshold: any order
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    if (order_key(row[j]) > thr) {
      const int pos = atomicAdd(&s_above, 1);
      if (pos < k) out[pos] = j;
    }
  }
  __syncthreads();
  const int above = s_above;
  // entries equal to the threshold: lowest positions first; warp 0 compacts them in order with ballots
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int taken = 0;
    const int want = min(need_equal, k - above);
    for (int j0 = 0; j0 < n && taken < want; j0 += 32) {
      const int j = j0 + lane;
      const bool eq = j < n && order_key(row[j]) == thr;
      const uint32_t bal = __ballot_sync(0xffffffffu, eq);
      const int pos = taken + __popc(bal & ((1u << lane) - 1u));
      if (eq && pos < want) out[above + pos] = j;
      taken += __popc(bal);
    }
    taken = min(taken, want);
    for (int t = above + taken + lane; t < k; t += 32) out[t] = t < n ? t : 0;   // cannot happen for k <= n
  }
}

}  // namespace

extern "C" {

// q [T, H, 128] bf16, k [T, 128] bf16, w [T, H] fp32, seq_start [T] int32 -> out [T, T] fp32.  The caller fills `out`
// with -inf beforehand; only tiles that contain visible keys are written.
int mcb_dsa_index_scores(const void* q, const void* k, const float* w, const int* seq_start, float* out, int T, int H,
                         int D, int* status, void* stream_) {
  if (T == 0) return 0;
  if (D != IX_D || H < 1 || T % 4 != 0) return -2;
  CUtensorMap tq, tk;
  int rc = make_tmap_2d_bf16(&tq, q, (long long)H * D, T, (long long)H * D, 64, IX_TILE);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tk, k, D, T, D, 64, IX_TILE);
  if (rc) return rc;
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(dsa_index_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         IxSmem::TOTAL);
    if (e != cudaSuccess) return (int)e;
    cfg = true;
  }
  IxParams p{T, H, w, seq_start, out, status};
  const int mt = (T + IX_TILE - 1) / IX_TILE;
  const int tiles = mt * (mt + 1) / 2;
  const int grid = tiles < device_sm_count() ? tiles : device_sm_count();
  dsa_index_scores_kernel<<<grid, IX_THREADS, IxSmem::TOTAL, reinterpret_cast<cudaStream_t>(stream_)>>>(tq, tk, p);
  return (int)cudaGetLastError();
}

int mcb_topk_select(const float* scores, long long ld, int rows, int n, int k, long long* idx, void* stream_) {
  if (rows == 0 || k == 0) return 0;
  if (k > n) return -2;
  topk_select_kernel<<<rows, 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(scores, ld, n, k, idx);
  return (int)cudaGetLastError();
}

}  // extern "C"

// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (one kernel each):
//
// Every CTA runs the GEMM roles (TMA producer, MMA issuer, four epilogue warps) plus four communication warps, so no
// SM is taken away from the tensor cores and all 148 SMs contribute loads in flight to the exchange (a single SM
// sustains only a few tens of GB/s of peer or staged reads; the link needs several hundred).
//
//   all-gather -> GEMM   C[M,N] = gather(A_shards)[M,K] . B^T       (column-parallel fwd, row-parallel dgrad)
//       The communication warps pull the peers' shards with vector loads over NVLink into a local gathered buffer,
//       16 KiB units in ring order, and publish a flag per 128-row block once its units are all in; the GEMM roles
//       start on the local shard and consume remote blocks in arrival order, so the transfer hides behind the math.
//
//   GEMM -> reduce-scatter   out[M/w, N] = sum_ranks (A . B^T)[rows of this rank]   (row-parallel fwd, column dgrad)
//       Each epilogue warp pushes its part of a bf16 partial tile straight into the staging buffer of the rank
//       that owns the rows (contiguous 4 KiB bulk copies over NVLink) and bumps a counter there; the communication
//       warps sum the rows this rank owns, row block by row block, as their counters fill.
//
// No TMA multicast anywhere; remote data is only touched by plain bulk copies, ld/st and red.
// Every cross-rank wait is bounded and reports through the status word.
#include <cstdlib>

#include "../common/host_utils.cuh"
#include "../gemm/gemm_pipe.cuh"
#include "../gemm/gemm_sm100.cuh"

using namespace mcb;

namespace {

constexpr int MAX_WORLD = 8;
// flag-region layout (uint32 indices)
constexpr int F_READY = 0;        // [world]   AG: shard of rank i is ready (epoch)
constexpr int F_BLOCK = 64;       // [<=4096]  AG: gathered 128-row block landed (epoch)
constexpr int F_DONE = 0;         // [world]   RS: rank i finished reducing (epoch)
constexpr int F_TICKET = 32;      // RS: CTA completion ticket
constexpr int F_CNT = 64;         // [2][2048] RS: tiles pushed per row block, per epoch parity
constexpr int F_CNT_STRIDE = 2048;

constexpr int F_BLKCNT = 4160;    // [<=4096]  AG: copy units finished per gathered block (the finisher resets it)

constexpr int COMM_WARPS = 4;                                  // communication warps per CTA (warps 6..9)
constexpr int COMM_THREADS = GEMM_THREADS + COMM_WARPS * 32;   // 320
constexpr int RS_THREADS = COMM_THREADS + 32;                  // + the warp that publishes finished tiles (warp 10)
constexpr int AG_UNIT_BYTES = 16384;                           // what one warp copies between two flag updates
constexpr int AG_LOADS = 16;                                   // 16-byte loads a lane keeps in flight

struct CommGemmParams {
  int M, N, K;
  int world, rank, epoch;
  int rows_per_rank;
  const void* peer_shard[MAX_WORLD];
  void* gathered;
  uint32_t* peer_flags[MAX_WORLD];
  void* C;
  long long ldc;
  const void* bias;
  void* peer_stage[MAX_WORLD];
  void* out;
  long long ld_out;
  int* status;
};

constexpr int RS_SLAB_COLS = 64;
constexpr int RS_SLAB_BYTES = GEMM_BM * RS_SLAB_COLS * 2;  // 16 KiB: 128 rows x 64 bf16 columns
constexpr int RS_TILE_BYTES = 4 * RS_SLAB_BYTES;           // 64 KiB: one 128 x 256 partial tile

struct CommSched {
  int tiles_m, tiles_n, total, bps, BN, world, rank, first_step;
  __device__ CommSched(const CommGemmParams& p, int bn, int first) : BN(bn), world(p.world), rank(p.rank), first_step(first) {
    tiles_m = p.M / GEMM_BM;
    tiles_n = (p.N + bn - 1) / bn;
    total = tiles_m * tiles_n;
    bps = p.rows_per_rank / GEMM_BM;
  }
  // logical m index j -> (owning shard, block inside the shard); step 0 is `first_step` ranks after our own
  __device__ void get(int t, int& shard, int& blk, int& n0, int& step) const {
    const int G = bps < 8 ? bps : 8;
    const int per_sg = G * tiles_n;
    const int sg = t / per_sg;
    const int first_m = sg * G;
    const int gsize = min(tiles_m - first_m, G);
    const int r = t - sg * per_sg;
    const int j = first_m + r % gsize;
    n0 = (r / gsize) * BN;
    step = j / bps;
    blk = j - step * bps;
    shard = (rank + first_step + step) % world;
  }
};

// ----------------------------------------------------------------------------------------------------------
// all-gather -> GEMM
// ----------------------------------------------------------------------------------------------------------
template <int BN, bool B_MN>
__global__ void __launch_bounds__(COMM_THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a_local, const __grid_constant__ CUtensorMap tmap_a_gath,
               const __grid_constant__ CUtensorMap tmap_b, const CommGemmParams p) {
  using L = GemmSmem<BN>;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  extern __shared__ uint8_t smem_raw[];
  if (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) return;  // an earlier wait gave up: do not pile up
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t* lflags = p.peer_flags[p.rank];
  const uint32_t epoch = (uint32_t)p.epoch;
  const int bps = p.rows_per_rank / GEMM_BM;

  Pipe<BN> P(smem_raw);
  if (threadIdx.x == 0) {
    P.init();
    prefetch_tensormap(&tmap_a_local);
    prefetch_tensormap(&tmap_a_gath);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(P.tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  // announce that this rank's shard (written by the preceding kernel in stream order) may be read
  if (blockIdx.x == 0 && warp == 2 && lane < p.world && lane != p.rank) {
    fence_acq_rel_sys();
    st_release_sys(p.peer_flags[lane] + F_READY + p.rank, epoch);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *P.tmem_slot;
  CommSched sched(p, BN, 0);
  const int g0 = blockIdx.x, gs = gridDim.x;

  if (warp >= GEMM_THREADS / 32) {
    // =================================================================== communication warps: gather the shards
    const long long block_bytes = (long long)GEMM_BM * p.K * 2;
    const int upb = (int)((block_bytes + AG_UNIT_BYTES - 1) / AG_UNIT_BYTES);   // units per 128-row block
    const long long units = (long long)p.world * bps * upb;     // remote shards in ring order, then the local one
    const long long cw = (long long)blockIdx.x * COMM_WARPS + (warp - GEMM_THREADS / 32);
    const long long ncw = (long long)gridDim.x * COMM_WARPS;
    int ready_src = -1;
    for (long long u = cw; u < units; u += ncw) {
      const int i = (int)(u / upb), c = (int)(u - (long long)i * upb);
      const int step = i / bps, blk = i - step * bps;
      const int s = step < p.world - 1 ? (p.rank + 1 + step) % p.world : p.rank;
      if (s != p.rank && s != ready_src) {
        int good = 1;
        if (lane == 0) good = wait_flag<SCOPE_SYS>(lflags + F_READY + s, epoch, false, P.abort_flag, p.status);
        good = __shfl_sync(0xffffffffu, good, 0);
        if (!good) break;
        ready_src = s;
      }
      const int gblock = s * bps + blk;
      const long long off = (long long)c * AG_UNIT_BYTES;
      const int n16 = (int)(min((long long)AG_UNIT_BYTES, block_bytes - off) / 16);
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.peer_shard[s]) +
                                                        (long long)blk * block_bytes + off);
      uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.gathered) + (long long)gblock * block_bytes + off);
      for (int base = 0; base < n16; base += 32 * AG_LOADS) {
        uint4 v[AG_LOADS];
#pragma unroll
        for (int j = 0; j < AG_LOADS; ++j) {
          const int idx = base + j * 32 + lane;
          if (idx < n16) v[j] = src[idx];               // every load is issued before the first store
        }
#pragma unroll
        for (int j = 0; j < AG_LOADS; ++j) {
          const int idx = base + j * 32 + lane;
          if (idx < n16) dst[idx] = v[j];
        }
      }
      __syncwarp();
      if (lane == 0 && s != p.rank) {
        // the warp that completes a block publishes it: its own fence orders its stores before the count, the
        // fence after the count orders the other warps' (already counted, hence fenced) stores before the flag
        __threadfence();
        const uint32_t done = atomicAdd(lflags + F_BLKCNT + gblock, 1u) + 1u;
        if (done == (uint32_t)upb) {
          __threadfence();
          lflags[F_BLKCNT + gblock] = 0;
          st_release_gpu(lflags + F_BLOCK + gblock, epoch);
        }
      }
    }
  } else

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      int seen_block = -1;
      for (int t = g0; t < sched.total; t += gs) {
        int shard, blk, n0, step;
        sched.get(t, shard, blk, n0, step);
        const int gblock = shard * bps + blk;
        const CUtensorMap* ta = &tmap_a_local;
        int a_row = blk * GEMM_BM;
        if (shard != p.rank) {
          if (gblock != seen_block) {
            if (!wait_flag<SCOPE_GPU>(lflags + F_BLOCK + gblock, epoch, false, P.abort_flag, p.status)) break;
            fence_proxy_async_all();
            seen_block = gblock;
          }
          ta = &tmap_a_gath;
          a_row = gblock * GEMM_BM;
        }
        if (!load_tile<BN, B_MN>(P, ta, &tmap_b, a_row, n0, p.K, it, p.status)) break;
      }
      drain_loads<BN>(P, it);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, lt = 0;
      bool ok = true;
      for (int t = g0; t < sched.total && ok; t += gs, ++lt) {
        const uint32_t acc = lt & 1, aph = (lt >> 1) & 1;
        if (!mbar_wait(smem_u32(&P.tempty_bar[acc]), aph ^ 1, P.abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        issue_mma_tile<BN, B_MN>(P, tmem_base + acc * BN, p.K, it, p.status, ok);
        if (ok) umma_commit(smem_u32(&P.tfull_bar[acc]));
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t lt = 0;
    for (int t = g0; t < sched.total; t += gs, ++lt) {
      int shard, blk, n0, step;
      sched.get(t, shard, blk, n0, step);
      const uint32_t acc = lt & 1, aph = (lt >> 1) & 1;
      if (!mbar_wait(smem_u32(&P.tfull_bar[acc]), aph, P.abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const long long row = (long long)(shard * bps + blk) * GEMM_BM + q * 32 + lane;
      __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + row * p.ldc;
      const __nv_bfloat16* bias = reinterpret_cast<const __nv_bfloat16*>(p.bias);
#pragma unroll 1
      for (int cc = 0; cc < BN; cc += 32) {
        if (n0 + cc >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (uint32_t(q * 32) << 16) + acc * BN + cc, r);
        tmem_ld_wait();
        const int col0 = n0 + cc;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (bias) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) v[j] += __bfloat162float(bias[col0 + j]);
        }
        if (col0 + 32 <= p.N) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 o;
            o.x = pack_bf16x2(v[j], v[j + 1]);
            o.y = pack_bf16x2(v[j + 2], v[j + 3]);
            o.z = pack_bf16x2(v[j + 4], v[j + 5]);
            o.w = pack_bf16x2(v[j + 6], v[j + 7]);
            *reinterpret_cast<uint4*>(crow + col0 + j) = o;
          }
        } else {
          for (int j = 0; j < 32; ++j)
            if (col0 + j < p.N) crow[col0 + j] = __float2bfloat16(v[j]);
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

// ----------------------------------------------------------------------------------------------------------
// GEMM -> reduce-scatter
// ----------------------------------------------------------------------------------------------------------
// Staging layout (the owner's buffer, one half per epoch parity): tile-major, each 128x256 partial tile stored as
// four 16 KiB slabs of 64 columns, a slab as [8 column chunks of 16 bytes][128 rows],
//     offset = ((source_rank * bps + row_block) * tiles_n + tile_n) * 64 KiB + slab * 16 KiB + (chunk * 128 + row) * 16.
// An epilogue thread owns one row of the accumulator, so the 32 lanes of a warp hold 32 consecutive rows and each of
// their store instructions covers 512 contiguous bytes of a chunk.  Because the sum over sources is element-wise, the
// reducer adds the staged tiles in that order and only the output address undoes the layout.
//
// Tile order is row-block-major: for each row block, every destination rank in turn (own rows last), every column
// tile.  A row block of the owner is therefore complete once every source is 1/bps of the way through its tiles,
// and the communication warps of all CTAs sum finished row blocks while the GEMM roles are still pushing.
struct RsSched {
  int tiles_n, total, bps, world, rank, BN;
  __device__ RsSched(const CommGemmParams& p, int bn) : world(p.world), rank(p.rank), BN(bn) {
    tiles_n = (p.N + bn - 1) / bn;
    bps = p.rows_per_rank / GEMM_BM;
    total = bps * world * tiles_n;
  }
  __device__ void get(int t, int& shard, int& blk, int& tn) const {
    const int per_blk = world * tiles_n;
    blk = t / per_blk;
    const int r = t - blk * per_blk;
    const int step = r / tiles_n;
    tn = r - step * tiles_n;
    shard = (rank + 1 + step) % world;
  }
};

// One warp sums RS_UNIT_POS consecutive 16-byte positions of one row block over SRC (>= world) staged sources and
// writes bf16 output rows.  A lane keeps 16 loads in flight (16 / SRC positions x SRC sources).
constexpr int RS_UNIT_POS = 1024;     // 16 KiB per source between two counter checks

template <int SRC>
__device__ __forceinline__ void rs_reduce_unit(const CommGemmParams& p, const uint8_t* stage, int blk, int bps, int tiles_n,
                                               long long pos0, int lane) {
  constexpr int POS = 16 / SRC;
  const long long src_stride = (long long)bps * tiles_n * RS_TILE_BYTES;
  const uint8_t* base = stage + (long long)blk * tiles_n * RS_TILE_BYTES;
#pragma unroll 1
  for (int r0 = 0; r0 < RS_UNIT_POS; r0 += 32 * POS) {
    uint4 raw[POS][SRC];
#pragma unroll
    for (int u = 0; u < POS; ++u) {
      const long long pos = pos0 + r0 + u * 32 + lane;
#pragma unroll
      for (int s = 0; s < SRC; ++s) {
        if (s < p.world) raw[u][s] = __ldcs(reinterpret_cast<const uint4*>(base + s * src_stride + pos * 16));
        else raw[u][s] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < POS; ++u) {
      const long long pos = pos0 + r0 + u * 32 + lane;
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
      for (int s = 0; s < SRC; ++s) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u][s]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h[e]);
          acc[2 * e] += f.x;
          acc[2 * e + 1] += f.y;
        }
      }
      const int tn = (int)(pos >> 12);            // 4096 positions per tile
      const int i = (int)(pos & 4095);
      const int slab = i >> 10, w = i & 1023;     // 1024 positions per slab: [8 column chunks][128 rows]
      const int r = w & (GEMM_BM - 1);
      const int col = tn * 256 + slab * RS_SLAB_COLS + (w >> 7) * 8;
      if (col < p.N) {
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.out) + ((long long)blk * GEMM_BM + r) * p.ld_out;
        *reinterpret_cast<uint4*>(orow + col) = o;
      }
    }
  }
}

template <int BN, bool B_MN>
__global__ void __launch_bounds__(RS_THREADS, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const CommGemmParams p) {
  static_assert(BN == 256, "the staging layout assumes 256-column tiles");
  constexpr uint32_t TMEM_COLS = 2 * BN;
  extern __shared__ uint8_t smem_raw[];
  if (p.status && *reinterpret_cast<volatile int*>(p.status) != 0) return;  // an earlier wait gave up: do not pile up
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t* lflags = p.peer_flags[p.rank];
  const uint32_t epoch = (uint32_t)p.epoch;
  const int parity = p.epoch & 1;
  RsSched sched(p, BN);
  const int bps = sched.bps;
  const int gemm_ctas = (int)gridDim.x;
  Pipe<BN> P(smem_raw);
  uint32_t* pushed = P.tmem_slot + 2;     // [4]: tiles whose stores each epilogue warp has issued

  {
    // ================================================================= GEMM CTA
    if (threadIdx.x == 0) {
      P.init();
      for (int i = 0; i < 4; ++i) pushed[i] = 0;
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

    if (warp == COMM_THREADS / 32) {
      // ================================================================= publisher: a system-scope fence costs a
      // round trip to the peers, so it is kept off the epilogue warps.  This thread watches how many tiles all four
      // epilogue warps have stored, fences once for everything new (the stores reach it through the warps'
      // release / acquire on `pushed`), then bumps the owners' row-block counters.
      if (lane == 0) {
        const uint32_t my_tiles =
            (int)blockIdx.x < sched.total ? (uint32_t)((sched.total - 1 - (int)blockIdx.x) / gemm_ctas + 1) : 0u;
        uint32_t done = 0;
        while (done < my_tiles) {
          uint32_t n = done;
          uint64_t t0 = 0;
          bool good = false;
          for (uint32_t it = 0; it < 0x7fffffffu; ++it) {
            uint32_t lo = 0xffffffffu;
#pragma unroll
            for (int i = 0; i < 4; ++i) lo = min(lo, ld_acquire_cta_shared(smem_u32(pushed + i)));
            if (lo > done) {
              n = lo;
              good = true;
              break;
            }
            if ((it & 0x3fu) == 0x3fu) {
              if (*P.abort_flag) break;
              const uint64_t now = globaltimer_ns();
              if (t0 == 0) t0 = now;
              if (now - t0 > wait_limit_ns(p.status)) {
                *P.abort_flag = 1;
                if (p.status) atomicCAS(p.status, 0, ST_TIMEOUT_TMEM_FULL);
                break;
              }
            }
            __nanosleep(32);
          }
          if (!good) break;
          fence_acq_rel_sys();
          for (uint32_t i = done; i < n; ++i) {
            int shard, blk, tn;
            sched.get((int)blockIdx.x + (int)i * gemm_ctas, shard, blk, tn);
            red_relaxed_sys_add(p.peer_flags[shard] + F_CNT + parity * F_CNT_STRIDE + blk, 4u);
          }
          done = n;
        }
      }
    } else if (warp >= GEMM_THREADS / 32) {
      // ================================================================= communication warps: sum the rows this
      // rank owns, row block by row block, as the counters say that every source has pushed its tiles
      const uint32_t want = (uint32_t)(p.world * sched.tiles_n * 4);  // the publisher adds 4 per tile
      const long long npos_blk = (long long)sched.tiles_n * (RS_TILE_BYTES / 16);
      const int upb = (int)(npos_blk / RS_UNIT_POS);
      const long long units = (long long)bps * upb;
      const uint8_t* stage = reinterpret_cast<const uint8_t*>(p.peer_stage[p.rank]);
      const long long cw = (long long)blockIdx.x * COMM_WARPS + (warp - GEMM_THREADS / 32);
      const long long ncw = (long long)gridDim.x * COMM_WARPS;
      int ready_blk = -1;
      for (long long u = cw; u < units; u += ncw) {
        const int blk = (int)(u / upb);
        const long long pos0 = (u - (long long)blk * upb) * RS_UNIT_POS;
        if (blk != ready_blk) {
          int good = 1;
          if (lane == 0)
            good = wait_flag<SCOPE_SYS>(lflags + F_CNT + parity * F_CNT_STRIDE + blk, want, false, P.abort_flag, p.status);
          good = __shfl_sync(0xffffffffu, good, 0);
          if (!good) break;
          ready_blk = blk;
        }
        if (p.world <= 2) rs_reduce_unit<2>(p, stage, blk, bps, sched.tiles_n, pos0, lane);
        else if (p.world <= 4) rs_reduce_unit<4>(p, stage, blk, bps, sched.tiles_n, pos0, lane);
        else rs_reduce_unit<8>(p, stage, blk, bps, sched.tiles_n, pos0, lane);
      }
    } else if (warp == 0) {
      if (lane == 0) {
        uint32_t it = 0;
        for (int t = blockIdx.x; t < sched.total; t += gemm_ctas) {
          int shard, blk, tn;
          sched.get(t, shard, blk, tn);
          if (!load_tile<BN, B_MN>(P, &tmap_a, &tmap_b, (shard * bps + blk) * GEMM_BM, tn * BN, p.K, it, p.status)) break;
        }
        drain_loads<BN>(P, it);
      }
    } else if (warp == 1) {
      if (lane == 0) {
        uint32_t it = 0, lt = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < sched.total && ok; t += gemm_ctas, ++lt) {
          const uint32_t acc = lt & 1, aph = (lt >> 1) & 1;
          if (!mbar_wait(smem_u32(&P.tempty_bar[acc]), aph ^ 1, P.abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) break;
          tc_fence_after();
          issue_mma_tile<BN, B_MN>(P, tmem_base + acc * BN, p.K, it, p.status, ok);
          if (ok) umma_commit(smem_u32(&P.tfull_bar[acc]));
        }
      }
    } else {
      // Epilogue: TMEM -> registers -> bf16 -> vector stores straight into the owner's staging tile (peer memory for
      // the other ranks' rows).  The staging layout puts the 32 rows of a warp next to each other for every 16-byte
      // column chunk, so each store instruction of a warp writes 512 contiguous bytes: full NVLink write packets
      // without a shared-memory detour.  The warp then only notes the tile in shared memory; the publisher warp
      // makes it visible to the owner.
      const int q = warp & 3;
      const int r_local = q * 32 + lane;
      uint32_t lt = 0;
      uint32_t verified = 0;       // bit s: rank s has released the staging half we are about to write
      for (int t = blockIdx.x; t < sched.total; t += gemm_ctas, ++lt) {
        int shard, blk, tn;
        sched.get(t, shard, blk, tn);
        const int n0 = tn * BN;
        const uint32_t acc = lt & 1, aph = (lt >> 1) & 1;
        if (!mbar_wait(smem_u32(&P.tfull_bar[acc]), aph, P.abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) break;
        tc_fence_after();
        if (!(verified & (1u << shard))) {
          // the owner must have finished reducing the call that last used this staging half (two calls ago)
          if (p.epoch > 2 && shard != p.rank) {
            int good = 1;
            if (lane == 0) good = wait_flag<SCOPE_SYS>(lflags + F_DONE + shard, epoch - 2, false, P.abort_flag, p.status);
            good = __shfl_sync(0xffffffffu, good, 0);
            if (!good) break;
          }
          verified |= 1u << shard;
        }
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.peer_stage[shard]) +
                                              ((long long)(p.rank * bps + blk) * sched.tiles_n + tn) * RS_TILE_BYTES) +
                     r_local;
#pragma unroll 1
        for (int cc = 0; cc < BN; cc += RS_SLAB_COLS) {
          if (n0 + cc >= p.N) break;
          uint32_t r[64];
          tmem_ld_32x32_x64(tmem_base + (uint32_t(q * 32) << 16) + acc * BN + cc, r);
          tmem_ld_wait();
          uint4* slab = dst + (cc / RS_SLAB_COLS) * (RS_SLAB_BYTES / 16);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[8 * j]), __uint_as_float(r[8 * j + 1]));
            o.y = pack_bf16x2(__uint_as_float(r[8 * j + 2]), __uint_as_float(r[8 * j + 3]));
            o.z = pack_bf16x2(__uint_as_float(r[8 * j + 4]), __uint_as_float(r[8 * j + 5]));
            o.w = pack_bf16x2(__uint_as_float(r[8 * j + 6]), __uint_as_float(r[8 * j + 7]));
            slab[j * GEMM_BM] = o;     // chunk j of row r_local: unit (j * 128 + r_local) of the slab
          }
        }
        tc_fence_before();
        __syncwarp();                  // orders every lane's stores before lane 0's release below
        if (lane == 0) {
          mbar_arrive(smem_u32(&P.tempty_bar[acc]));
          st_release_cta_shared(smem_u32(pushed + q), lt + 1);
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

  __syncthreads();
  // the last CTA to get here resets the counters of this parity and tells every peer that this rank is done reading
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t ticket = atomicAdd(lflags + F_TICKET, 1u);
    if (ticket == gridDim.x - 1) {
      for (int b = 0; b < bps; ++b) lflags[F_CNT + parity * F_CNT_STRIDE + b] = 0;
      lflags[F_TICKET] = 0;
      fence_acq_rel_sys();
      for (int s = 0; s < p.world; ++s)
        if (s != p.rank) st_release_sys(p.peer_flags[s] + F_DONE + p.rank, epoch);
    }
  }
}

template <typename Kern>
cudaError_t set_smem(Kern k, int bytes) {
  return cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

}  // namespace

extern "C" {

// flags_ptrs / shard_ptrs / stage_ptrs: host arrays of `world` device pointers (index = group rank)
int mcb_ag_gemm_bf16(const void* const* shard_ptrs, void* const* flag_ptrs, void* gathered, const void* B, long long b_inner,
                     long long b_outer, long long ldb, int b_mn, void* C, long long ldc, const void* bias, int M, int N,
                     int K, int world, int rank, int epoch, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (world < 2 || world > MAX_WORLD || M % (world * GEMM_BM) || K % 8 || N % 8) return -2;
  const int rows = M / world;
  if (M / GEMM_BM > 4096) return -3;
  constexpr int BN = 256;
  const int sms = device_sm_count();
  CUtensorMap ta_l, ta_g, tb;
  int rc = make_tmap_2d_bf16(&ta_l, shard_ptrs[rank], K, rows, K, GEMM_BK, GEMM_BM);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&ta_g, gathered, K, M, K, GEMM_BK, GEMM_BM);
  if (rc) return rc;
  rc = b_mn ? make_tmap_2d_bf16(&tb, B, b_inner, b_outer, ldb, 64, GEMM_BK)
            : make_tmap_2d_bf16(&tb, B, b_inner, b_outer, ldb, GEMM_BK, BN);
  if (rc) return rc;
  CommGemmParams p{};
  p.M = M; p.N = N; p.K = K; p.world = world; p.rank = rank; p.epoch = epoch; p.rows_per_rank = rows;
  for (int i = 0; i < world; ++i) {
    p.peer_shard[i] = shard_ptrs[i];
    p.peer_flags[i] = reinterpret_cast<uint32_t*>(flag_ptrs[i]);
  }
  p.gathered = gathered; p.C = C; p.ldc = ldc; p.bias = bias; p.status = status;
  const int smem = GemmSmem<BN>::TOTAL;
  // every CTA also carries communication warps, so the whole GPU takes part even when there are few tiles
  const int grid = sms;
  static bool cfg[2] = {false, false};
  cudaError_t e;
  if (b_mn) {
    if (!cfg[1]) { if ((e = set_smem(ag_gemm_kernel<BN, true>, smem)) != cudaSuccess) return (int)e; cfg[1] = true; }
    ag_gemm_kernel<BN, true><<<grid, COMM_THREADS, smem, stream>>>(ta_l, ta_g, tb, p);
  } else {
    if (!cfg[0]) { if ((e = set_smem(ag_gemm_kernel<BN, false>, smem)) != cudaSuccess) return (int)e; cfg[0] = true; }
    ag_gemm_kernel<BN, false><<<grid, COMM_THREADS, smem, stream>>>(ta_l, ta_g, tb, p);
  }
  return (int)cudaGetLastError();
}

// Bytes of one staging half that a call with these sizes writes on every rank (tile-major, 64 KiB per tile).
long long mcb_gemm_rs_stage_bytes(int M, int N) {
  return (long long)(M / GEMM_BM) * ((N + 255) / 256) * RS_TILE_BYTES;
}

int mcb_gemm_rs_bf16(const void* A, long long lda, const void* B, long long b_inner, long long b_outer, long long ldb,
                     int b_mn, void* const* stage_ptrs, void* const* flag_ptrs, void* out, long long ld_out, int M, int N,
                     int K, int world, int rank, int epoch, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (world < 2 || world > MAX_WORLD || M % (world * GEMM_BM) || K % 8 || N % 8 || lda % 8 || ld_out % 8) return -2;
  if ((reinterpret_cast<uintptr_t>(out) & 15) != 0) return -2;
  const int rows = M / world;
  if (rows / GEMM_BM > F_CNT_STRIDE) return -3;
  constexpr int BN = 256;
  const int sms = device_sm_count();
  const long long tiles = (long long)(M / GEMM_BM) * ((N + BN - 1) / BN);
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, A, K, M, lda, GEMM_BK, GEMM_BM);
  if (rc) return rc;
  rc = b_mn ? make_tmap_2d_bf16(&tb, B, b_inner, b_outer, ldb, 64, GEMM_BK)
            : make_tmap_2d_bf16(&tb, B, b_inner, b_outer, ldb, GEMM_BK, BN);
  if (rc) return rc;
  CommGemmParams p{};
  p.M = M; p.N = N; p.K = K; p.world = world; p.rank = rank; p.epoch = epoch; p.rows_per_rank = rows;
  for (int i = 0; i < world; ++i) {
    p.peer_stage[i] = stage_ptrs[i];
    p.peer_flags[i] = reinterpret_cast<uint32_t*>(flag_ptrs[i]);
  }
  p.out = out; p.ld_out = ld_out; p.status = status;
  const int smem = GemmSmem<BN>::TOTAL;
  (void)tiles;
  const int grid = sms;      // every CTA also carries reducer warps
  static bool cfg[2] = {false, false};
  cudaError_t e;
  if (b_mn) {
    if (!cfg[1]) { if ((e = set_smem(gemm_rs_kernel<BN, true>, smem)) != cudaSuccess) return (int)e; cfg[1] = true; }
    gemm_rs_kernel<BN, true><<<grid, RS_THREADS, smem, stream>>>(ta, tb, p);
  } else {
    if (!cfg[0]) { if ((e = set_smem(gemm_rs_kernel<BN, false>, smem)) != cudaSuccess) return (int)e; cfg[0] = true; }
    gemm_rs_kernel<BN, false><<<grid, RS_THREADS, smem, stream>>>(ta, tb, p);
  }
  return (int)cudaGetLastError();
}

}  // extern "C"

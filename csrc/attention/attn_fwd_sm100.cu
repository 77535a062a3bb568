// Variable-length causal GQA attention forward for sm_100a: S = Q K^T and O += P V on tcgen05 with accumulators in
// TMEM, operands staged by TMA, softmax in registers.
//
// One CTA per (128-query tile, query head).  The mask is a per-query inclusive key range [k_lo[i], k_hi[i]] (see
// attn_common.cuh): packed causal self-attention is k_lo = first token of the query's sequence, k_hi = the query
// itself, so tiles may straddle sequence boundaries and nothing is synchronised with the host; queries and keys may
// also be different token sets (the steps of context-parallel ring attention, non-causal attention).
//
// Two passes over the key blocks instead of online rescaling: pass 1 computes only the row maxima (Q K^T + max),
// pass 2 recomputes S, forms P = exp2(S - max) and accumulates O += P V directly in TMEM with no correction step.
// The extra Q K^T is cheap next to the exponentials, which bound attention on this architecture, and the kernel
// needs no accumulator rescaling traffic.
//
// Warp roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2..9 softmax in two groups of
// four (thread = query row).  Group g owns score buffer g in TMEM, i.e. every other key block of both passes, so each
// scheduler has two softmax warps to interleave (exponentials of one block overlap the TMEM reads of the next); the
// groups exchange their partial row maxima after pass 1 and their partial row sums after pass 2 through shared memory.
#include <type_traits>
#include "../common/host_utils.cuh"
#include "../common/ptx.cuh"
#include "attn_common.cuh"

using namespace mcb;

namespace {

constexpr int BM = 128;  // queries per CTA
constexpr int BNK = 128; // keys per block
constexpr int ATT_THREADS = 320;

struct AttnParams {
  int T, Tk, nq, nkv, d;  // T queries, Tk keys
  float scale_log2;       // softmax scale * log2(e)
  const int* k_lo;        // [T] first visible key of each query
  const int* k_hi;        // [T] last visible key, or null: the query's own index
  const float* sinks;     // [nq] or null: a per-head logit that joins every row's softmax with a zero value vector
  __nv_bfloat16* o;       // [T, nq, d]
  float* lse;             // [nq, T] natural log of sum exp(scaled scores); -inf for a query that sees no key
  int* status;
};

template <int D>
struct AttnSmem {
  static constexpr int TILE = BM * D * 2;            // one 128-row operand tile
  static constexpr int P_BYTES = BM * BNK * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = TILE;                  // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * TILE;      // 2 stages
  static constexpr int OFF_P = OFF_V + 2 * TILE;      // 2 buffers
  static constexpr int OFF_BAR = OFF_P + 2 * P_BYTES;
  static constexpr int TOTAL = OFF_BAR + 1024 + 1024;
};

// K-major operand tile [128 rows x D] stored as D/64 boxes of [128 x 64]; descriptor for the kk-th 16-wide k slice
template <int D>
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t base, int kk) {
  return make_smem_desc_sw128(base + (kk >> 2) * (BM * 128) + (kk & 3) * 32, 16, 1024);
}

__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(b_mn ? 1 : 0) << 16) | (uint32_t(n >> 3) << 17) |
         (uint32_t(m >> 4) << 24);
}

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  using L = AttnSmem<D>;
  constexpr int NBOX = D / 64;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0, COL_O = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2
  uint64_t* k_empty = bars + 3;       // 2
  uint64_t* v_full = bars + 5;        // 2
  uint64_t* v_empty = bars + 7;       // 2
  uint64_t* s_full = bars + 9;        // 2
  uint64_t* s_empty = bars + 11;      // 2
  uint64_t* p_full = bars + 13;       // 2
  uint64_t* p_empty = bars + 15;      // 2
  uint64_t* o_full = bars + 17;       // 1
  uint64_t* xchg = bars + 18;         // 2: row maxima / row sums exchanged between the softmax groups
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tile = gridDim.x - 1 - blockIdx.x;  // long tiles first
  const int head = blockIdx.y;
  const int kvh = head / (p.nq / p.nkv);
  const int m0 = m_tile * BM;
  __shared__ int s_rng[8];
  tile_range_partial(p.k_lo, p.k_hi, m0, p.T, s_rng);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(smem_u32(q_full), 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&k_full[i]), 1);
      mbar_init(smem_u32(&k_empty[i]), 1);
      mbar_init(smem_u32(&v_full[i]), 1);
      mbar_init(smem_u32(&v_empty[i]), 1);
      mbar_init(smem_u32(&s_full[i]), 1);
      mbar_init(smem_u32(&s_empty[i]), 4);
      mbar_init(smem_u32(&p_full[i]), 128);
      mbar_init(smem_u32(&p_empty[i]), 1);
    }
    mbar_init(smem_u32(o_full), 1);
    mbar_init(smem_u32(&xchg[0]), 256);
    mbar_init(smem_u32(&xchg[1]), 256);
    fence_barrier_init();
    fence_proxy_async_smem();
    prefetch_tensormap(&tm_q);
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
  const int kb0 = kmin / BNK;                      // first key block any row of this tile can see
  const int nblk = kmax >= kmin ? kmax / BNK - kb0 + 1 : 0;

  if (nblk <= 0) {
    // no row of this tile sees any key: the output is zero and the log-sum-exp -inf
    if (warp >= 2) {
      const int grp = (warp - 2) >> 2;
      const int i = m0 + (warp & 3) * 32 + lane;
      if (i < p.T) {
        uint4* orow = reinterpret_cast<uint4*>(p.o + ((long long)i * p.nq + head) * D + grp * (D / 2));
#pragma unroll
        for (int c = 0; c < D / 16; ++c) orow[c] = make_uint4(0, 0, 0, 0);
        if (grp == 0) p.lse[(long long)head * p.T + i] = p.sinks ? p.sinks[head] : -INFINITY;
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(smem_u32(q_full), L::TILE);
#pragma unroll
      for (int b = 0; b < NBOX; ++b)
        tma_load_2d(smem_u32(smem + L::OFF_Q + b * BM * 128), &tm_q, head * D + b * 64, m0, smem_u32(q_full));
      uint32_t kit = 0;
      bool ok = true;
      for (int pass = 0; pass < 2 && ok; ++pass) {
        for (int j = 0; j < nblk && ok; ++j, ++kit) {
          const int n0 = (kb0 + j) * BNK;
          const uint32_t st = kit & 1, ph = (kit >> 1) & 1;
          if (!mbar_wait(smem_u32(&k_empty[st]), ph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
          mbar_expect_tx(smem_u32(&k_full[st]), L::TILE);
#pragma unroll
          for (int b = 0; b < NBOX; ++b)
            tma_load_2d(smem_u32(smem + L::OFF_K + st * L::TILE + b * BM * 128), &tm_k, kvh * D + b * 64, n0,
                        smem_u32(&k_full[st]));
          if (pass == 1) {
            const uint32_t vst = j & 1, vph = (j >> 1) & 1;
            if (!mbar_wait(smem_u32(&v_empty[vst]), vph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
            mbar_expect_tx(smem_u32(&v_full[vst]), L::TILE);
#pragma unroll
            for (int b = 0; b < NBOX; ++b)
              tma_load_2d(smem_u32(smem + L::OFF_V + vst * L::TILE + b * BM * 128), &tm_v, kvh * D + b * 64, n0,
                          smem_u32(&v_full[vst]));
          }
        }
      }
      // drain: the last loads must land before the CTA exits
      for (uint32_t i = (kit > 2 ? kit - 2 : 0); i < kit; ++i) {
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(smem_u32(&k_full[i & 1]), (i >> 1) & 1))
          if (globaltimer_ns() - t0 > 200000000ull) break;
      }
      for (int j = (nblk > 2 ? nblk - 2 : 0); j < nblk; ++j) {
        uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(smem_u32(&v_full[j & 1]), (j >> 1) & 1))
          if (globaltimer_ns() - t0 > 200000000ull) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = idesc_bf16(BM, BNK, false);
      constexpr uint32_t idesc_o = idesc_bf16(BM, D, true);
      const uint32_t sq = smem_u32(smem + L::OFF_Q);
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag, p.status, ST_TIMEOUT_FULL);
      uint32_t kit = 0, sit = 0;
      auto issue_s = [&](uint32_t kit_, uint32_t sit_) -> bool {
        const uint32_t st = kit_ & 1, ph = (kit_ >> 1) & 1, sb = sit_ & 1, sph = (sit_ >> 1) & 1;
        if (!mbar_wait(smem_u32(&k_full[st]), ph, abort_flag, p.status, ST_TIMEOUT_FULL)) return false;
        if (!mbar_wait(smem_u32(&s_empty[sb]), sph ^ 1, abort_flag, p.status, ST_TIMEOUT_TMEM_EMPTY)) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + L::OFF_K + st * L::TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_f16(tmem + COL_S + sb * BNK, kmajor_desc<D>(sq, kk), kmajor_desc<D>(sk, kk), idesc_s, kk ? 1u : 0u);
        umma_commit(smem_u32(&k_empty[st]));
        umma_commit(smem_u32(&s_full[sb]));
        return true;
      };
      // pass 1: row maxima
      for (int j = 0; j < nblk && ok; ++j, ++kit, ++sit) ok = issue_s(kit, sit);
      // pass 2: S again, then O += P V one block behind
      if (ok) ok = issue_s(kit, sit);
      ++kit; ++sit;
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) {
          ok = issue_s(kit, sit);
          ++kit; ++sit;
          if (!ok) break;
        }
        const uint32_t pb = j & 1, pph = (j >> 1) & 1;
        if (!mbar_wait(smem_u32(&p_full[pb]), pph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
        if (!mbar_wait(smem_u32(&v_full[pb]), pph, abort_flag, p.status, ST_TIMEOUT_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sp = smem_u32(smem + L::OFF_P + pb * L::P_BYTES);
        const uint32_t sv = smem_u32(smem + L::OFF_V + pb * L::TILE);
#pragma unroll
        for (int kk = 0; kk < BNK / 16; ++kk) {
          const uint64_t ad = make_smem_desc_sw128(sp + (kk >> 2) * (BM * 128) + (kk & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc_sw128(sv + kk * 2048, BM * 128, 1024);
          umma_f16(tmem + COL_O, ad, bd, idesc_o, (j | kk) ? 1u : 0u);
        }
        umma_commit(smem_u32(&p_empty[pb]));
        umma_commit(smem_u32(&v_empty[pb]));
      }
      if (ok) umma_commit(smem_u32(o_full));
    }
  } else {
    // ------------------------------------------------------------------ softmax warps: thread = query row
    const int q = warp & 3;
    const int grp = (warp - 2) >> 2;
    const int r = q * 32 + lane;
    const int i = m0 + r;
    const bool row_ok = i < p.T;
    int lo, hi;
    attn_row_range(p.k_lo, p.k_hi, i, p.T, lo, hi);
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    const uint32_t sb = grp;                         // this group's score buffer
    float mx = -INFINITY;
    bool ok = true;
    // pass 1: score iterations sit = j (this group takes sit & 1 == grp)
    for (int j = grp; j < nblk && ok; j += 2) {
      const uint32_t sph = (uint32_t(j) >> 1) & 1;
      if (!mbar_wait(smem_u32(&s_full[sb]), sph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int n0 = (kb0 + j) * BNK;
      const bool full = (lo <= n0) && (n0 + BNK - 1 <= hi);
      // the whole 128-column row in one TMEM round trip; the score buffer is released as soon as the values are in
      // registers, so the next QK^T of this group overlaps the arithmetic below
      uint32_t v0[64], v1[64];
      tmem_ld_32x32_x64(tmem + lane_addr + COL_S + sb * BNK, v0);
      tmem_ld_32x32_x64(tmem + lane_addr + COL_S + sb * BNK + 64, v1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_empty[sb]));
      if (full) {
#pragma unroll
        for (int e = 0; e < 64; ++e) mx = fmaxf(mx, fmaxf(__uint_as_float(v0[e]), __uint_as_float(v1[e])));
      } else {
#pragma unroll
        for (int e = 0; e < 64; ++e) {
          const int key = n0 + e;
          if (key >= lo && key <= hi) mx = fmaxf(mx, __uint_as_float(v0[e]));
          if (key + 64 >= lo && key + 64 <= hi) mx = fmaxf(mx, __uint_as_float(v1[e]));
        }
      }
    }
    // The row maximum is over both groups' blocks.  The partial maxima travel through the P buffers, which nothing
    // has written yet: a group leaves its value in the buffer the *other* group owns in pass 2, so the value is
    // overwritten only by its reader, after it has been read.
    {
      const int pb_mine = (grp + nblk) & 1;
      reinterpret_cast<float*>(smem + L::OFF_P + (pb_mine ^ 1) * L::P_BYTES)[r] = mx;
      mbar_arrive(smem_u32(&xchg[0]));
      if (ok && !mbar_wait(smem_u32(&xchg[0]), 0, abort_flag, p.status, ST_TIMEOUT_FULL)) ok = false;
      if (ok) mx = fmaxf(mx, reinterpret_cast<const float*>(smem + L::OFF_P + pb_mine * L::P_BYTES)[r]);
    }
    // learnable softmax sink: an extra logit (already in softmax units, no scale) in the row's maximum and sum
    const float sink2 = p.sinks ? p.sinks[head] * 1.4426950408889634f : -INFINITY;
    const float m_tot = fmaxf((mx == -INFINITY) ? -INFINITY : mx * p.scale_log2, sink2);
    const float m2 = (m_tot == -INFINITY) ? 0.f : m_tot;
    float sum = (p.sinks && grp == 0) ? exp2f(sink2 - m2) : 0.f;
    // pass 2: score iterations sit = nblk + j; this group takes the j with (nblk + j) & 1 == grp, which all share
    // one P buffer
    const int j0 = (grp + nblk) & 1;
    for (int j = j0; j < nblk && ok; j += 2) {
      const uint32_t sit = uint32_t(nblk + j);
      const uint32_t sph = (sit >> 1) & 1, pb = j & 1, pph = (uint32_t(j) >> 1) & 1;
      if (!mbar_wait(smem_u32(&s_full[sb]), sph, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      uint32_t v0[64], v1[64];
      tmem_ld_32x32_x64(tmem + lane_addr + COL_S + sb * BNK, v0);
      tmem_ld_32x32_x64(tmem + lane_addr + COL_S + sb * BNK + 64, v1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&s_empty[sb]));   // scores are in registers: the next QK^T may start
      if (!mbar_wait(smem_u32(&p_empty[pb]), pph ^ 1, abort_flag, p.status, ST_TIMEOUT_EMPTY)) { ok = false; break; }
      const int n0 = (kb0 + j) * BNK;
      const bool full = (lo <= n0) && (n0 + BNK - 1 <= hi);
      uint8_t* prow = smem + L::OFF_P + pb * L::P_BYTES + r * 128;
      auto half = [&](const uint32_t (&v)[64], int c0, auto fullc) {
        constexpr bool FULL = decltype(fullc)::value;
        uint8_t* box = prow + (c0 >> 6) * (BM * 128);
#pragma unroll
        for (int e = 0; e < 64; e += 8) {
          float pv[8];
#pragma unroll
          for (int t = 0; t < 8; ++t) {
            const float x = exp2f(__uint_as_float(v[e + t]) * p.scale_log2 - m2);
            const int key = n0 + c0 + e + t;
            pv[t] = (FULL || (key >= lo && key <= hi)) ? x : 0.f;
            sum += pv[t];
          }
          uint4 o;
          o.x = pack_bf16x2(pv[0], pv[1]);
          o.y = pack_bf16x2(pv[2], pv[3]);
          o.z = pack_bf16x2(pv[4], pv[5]);
          o.w = pack_bf16x2(pv[6], pv[7]);
          *reinterpret_cast<uint4*>(box + (((e >> 3) ^ (r & 7)) << 4)) = o;
        }
      };
      if (full) {
        half(v0, 0, std::true_type{});
        half(v1, 64, std::true_type{});
      } else {
        half(v0, 0, std::false_type{});
        half(v1, 64, std::false_type{});
      }
      fence_proxy_async_smem();   // P stores -> visible to the tensor core's shared-memory reads
      mbar_arrive(smem_u32(&p_full[pb]));
    }
    // once every MMA has completed the Q tile is free: the partial row sums are exchanged through it
    const bool done = ok && mbar_wait(smem_u32(o_full), 0, abort_flag, p.status, ST_TIMEOUT_TMEM_FULL);
    float* sbuf = reinterpret_cast<float*>(smem + L::OFF_Q);
    if (done) sbuf[grp * BM + r] = sum;
    mbar_arrive(smem_u32(&xchg[1]));
    if (done && mbar_wait(smem_u32(&xchg[1]), 0, abort_flag, p.status, ST_TIMEOUT_FULL)) {
      sum += sbuf[(grp ^ 1) * BM + r];
      tc_fence_after();
      const float inv = sum > 0.f ? 1.f / sum : 0.f;
      // each group writes half of the head dimension
      __nv_bfloat16* orow = p.o + ((long long)i * p.nq + head) * D + grp * (D / 2);
      constexpr int OW = (D / 2 >= 64) ? 64 : 32;   // columns per TMEM load
#pragma unroll 1
      for (int c = 0; c < D / 2; c += OW) {
        uint32_t v[OW];
        if constexpr (OW == 64) tmem_ld_32x32_x64(tmem + lane_addr + COL_O + grp * (D / 2) + c, v);
        else tmem_ld_32x32(tmem + lane_addr + COL_O + grp * (D / 2) + c, v);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int e = 0; e < OW; e += 8) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(v[e]) * inv, __uint_as_float(v[e + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(v[e + 2]) * inv, __uint_as_float(v[e + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(v[e + 4]) * inv, __uint_as_float(v[e + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(v[e + 6]) * inv, __uint_as_float(v[e + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c + e) = o;
          }
        }
      }
      if (row_ok && grp == 0)
        p.lse[(long long)head * p.T + i] = (sum > 0.f) ? (m2 + log2f(sum)) * 0.6931471805599453f : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

template <int D>
int launch_fwd(const void* q, const void* k, const void* v, const AttnParams& p, cudaStream_t stream) {
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_2d_bf16(&tq, q, (long long)p.nq * D, p.T, (long long)p.nq * D, 64, BM);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tk, k, (long long)p.nkv * D, p.Tk, (long long)p.nkv * D, 64, BNK);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tv, v, (long long)p.nkv * D, p.Tk, (long long)p.nkv * D, 64, BNK);
  if (rc) return rc;
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<D>::TOTAL);
    if (e != cudaSuccess) return (int)e;
    cfg = true;
  }
  dim3 grid((p.T + BM - 1) / BM, p.nq);
  attn_fwd_kernel<D><<<grid, ATT_THREADS, AttnSmem<D>::TOTAL, stream>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}

}  // namespace

extern "C" {

// General form.  q [T, nq, d], k/v [Tk, nkv, d] bf16 contiguous; k_lo / k_hi [T] int32: query i attends to the keys
// k_lo[i] .. k_hi[i] (inclusive; k_hi may be null = i, which needs Tk >= T); sinks [nq] fp32 or null; o [T, nq, d];
// lse [nq, T] fp32 (it includes the sink, which is what the backward kernels need to recompute the probabilities).
int mcb_attn_fwd_ranges(const void* q, const void* k, const void* v, const int* k_lo, const int* k_hi,
                        const float* sinks, void* o, float* lse, int T, int Tk, int nq, int nkv, int d, float scale,
                        int* status, void* stream_) {
  if (T == 0) return 0;
  if (nq % nkv || Tk <= 0 || (k_hi == nullptr && Tk < T)) return -2;
  AttnParams p{T, Tk, nq, nkv, d, scale * 1.4426950408889634f, k_lo, k_hi, sinks, (__nv_bfloat16*)o, lse, status};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  if (d == 128) return launch_fwd<128>(q, k, v, p, s);
  if (d == 64) return launch_fwd<64>(q, k, v, p, s);
  return -3;
}

// Packed causal self-attention: seq_start [T] int32 = first token of each token's sequence.
int mcb_attn_fwd(const void* q, const void* k, const void* v, const int* seq_start, void* o, float* lse, int T, int nq,
                 int nkv, int d, float scale, int* status, void* stream_) {
  return mcb_attn_fwd_ranges(q, k, v, seq_start, nullptr, nullptr, o, lse, T, T, nq, nkv, d, scale, status, stream_);
}

}  // extern "C"

// Mainloop pieces shared by the kernels that embed the tcgen05 GEMM next to another role in the same launch (the
// tensor-parallel GEMMs fused with their collective, the MoE expert GEMM fused with the token dispatch): the
// shared-memory pipeline with its barriers, the TMA loads of one output tile and the MMA issue loop of one tile.
// Same tile shape and barrier protocol as gemm_sm100.cuh (128 x BN x 64, two TMEM accumulators).
#pragma once
#include "gemm_sm100.cuh"

namespace mcb {

template <int BN>
struct Pipe {
  using L = GemmSmem<BN>;
  uint8_t* smem;
  uint64_t *full_bar, *empty_bar, *tfull_bar, *tempty_bar;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
  __device__ Pipe(uint8_t* raw) {
    smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::STAGES * L::STAGE_BYTES);
    full_bar = bars;
    empty_bar = bars + L::STAGES;
    tfull_bar = bars + 2 * L::STAGES;
    tempty_bar = bars + 2 * L::STAGES + 2;
    tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * L::STAGES + 4);
    abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  }
  __device__ void init() {
    *abort_flag = 0;
    for (int s = 0; s < L::STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&tfull_bar[a]), 1);
      mbar_init(smem_u32(&tempty_bar[a]), 4);
    }
    fence_barrier_init();
    fence_proxy_async_smem();
  }
};

template <int BN, bool B_MN>
__device__ __forceinline__ void issue_mma_tile(Pipe<BN>& P, uint32_t d_tmem, int K, uint32_t& it, int* status, bool& ok) {
  using L = GemmSmem<BN>;
  constexpr uint32_t idesc = make_idesc_bf16(GEMM_BM, BN, false, B_MN);
  bool first = true;
  for (int k = 0; k < K; k += GEMM_BK, ++it) {
    const uint32_t s = it % L::STAGES, ph = (it / L::STAGES) & 1;
    if (!mbar_wait(smem_u32(&P.full_bar[s]), ph, P.abort_flag, status, ST_TIMEOUT_FULL)) {
      ok = false;
      return;
    }
    tc_fence_after();
    const uint32_t sa = smem_u32(P.smem + s * L::STAGE_BYTES);
    const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
    for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
      uint64_t ad = make_smem_desc_sw128(sa + kk * 32, 16, 1024);
      uint64_t bd = B_MN ? make_smem_desc_sw128(sb + kk * 2048, 8192, 1024) : make_smem_desc_sw128(sb + kk * 32, 16, 1024);
      umma_f16(d_tmem, ad, bd, idesc, first ? 0u : 1u);
      first = false;
    }
    umma_commit(smem_u32(&P.empty_bar[s]));
  }
}

template <int BN, bool B_MN>
__device__ __forceinline__ bool load_tile(Pipe<BN>& P, const CUtensorMap* ta, const CUtensorMap* tb, int a_row, int n0,
                                          int K, uint32_t& it, int* status, int b_k_base = 0) {
  using L = GemmSmem<BN>;
  for (int k = 0; k < K; k += GEMM_BK, ++it) {
    const uint32_t s = it % L::STAGES, ph = (it / L::STAGES) & 1;
    if (!mbar_wait(smem_u32(&P.empty_bar[s]), ph ^ 1, P.abort_flag, status, ST_TIMEOUT_EMPTY)) return false;
    const uint32_t fb = smem_u32(&P.full_bar[s]);
    mbar_expect_tx(fb, L::STAGE_BYTES);
    const uint32_t sa = smem_u32(P.smem + s * L::STAGE_BYTES);
    const uint32_t sb = sa + L::A_BYTES;
    tma_load_2d(sa, ta, k, a_row, fb);
    if (!B_MN) {
      tma_load_2d(sb, tb, k, n0, fb);
    } else {
#pragma unroll
      for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, tb, n0 + j * 64, b_k_base + k, fb);
    }
  }
  return true;
}

template <int BN>
__device__ __forceinline__ void drain_loads(Pipe<BN>& P, uint32_t it) {
  using L = GemmSmem<BN>;
  uint32_t first = it > L::STAGES ? it - L::STAGES : 0;
  for (uint32_t j = first; j < it; ++j) {
    const uint32_t s = j % L::STAGES, ph = (j / L::STAGES) & 1;
    uint64_t t0 = globaltimer_ns();
    while (!mbar_try_wait(smem_u32(&P.full_bar[s]), ph)) {
      if (globaltimer_ns() - t0 > 200000000ull) break;
    }
  }
}


}  // namespace mcb

// Host launcher for the tcgen05 GEMM: builds TMA descriptors, picks the tile width and launches
// the persistent kernel.  C ABI so Python reaches it through ctypes without a torch build step.
#include <mutex>

#include "../common/host_utils.cuh"
#include "gemm_sm100.cuh"
#include "gemm_sm100_2cta.cuh"

using namespace mcb;

namespace {

template <int BN, bool A_MN, bool B_MN>
cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t stream) {
  auto kern = gemm_bf16_sm100_kernel<BN, A_MN, B_MN>;
  static bool configured = false;  // per template instantiation
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN>::TOTAL);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  kern<<<grid, GEMM_THREADS, GemmSmem<BN>::TOTAL, stream>>>(ta, tb, p);
  return cudaGetLastError();
}

template <int BN>
cudaError_t launch_major(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                         int grid, cudaStream_t s) {
  if (!a_mn && !b_mn) return launch<BN, false, false>(ta, tb, p, grid, s);
  if (!a_mn && b_mn) return launch<BN, false, true>(ta, tb, p, grid, s);
  if (a_mn && b_mn) return launch<BN, true, true>(ta, tb, p, grid, s);
  return launch<BN, true, false>(ta, tb, p, grid, s);
}

template <bool A_MN, bool B_MN>
cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid, cudaStream_t stream) {
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  kern<<<grid, GEMM_THREADS, PAIR_SMEM, stream>>>(ta, tb, p);   // cluster of two CTAs (kernel attribute)
  return cudaGetLastError();
}

cudaError_t launch_pair_major(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                              int grid, cudaStream_t s) {
  if (!a_mn && !b_mn) return launch_pair<false, false>(ta, tb, p, grid, s);
  if (!a_mn && b_mn) return launch_pair<false, true>(ta, tb, p, grid, s);
  if (a_mn && b_mn) return launch_pair<true, true>(ta, tb, p, grid, s);
  return launch_pair<true, false>(ta, tb, p, grid, s);
}

// CTA pairs (256 x 256 tiles) pay off once there are enough tiles to fill the 74 clusters a few times over; small or
// skinny problems keep the single-CTA tiles, whose narrower variants quantise better.
bool use_pair(int M, int N, int K, int mode, int sms) {
  if (mode != GEMM_DENSE || M < 512 || N < 256 || K < 128) return false;
  const long long tiles = (long long)((M + PAIR_BM - 1) / PAIR_BM) * ((N + PAIR_BN - 1) / PAIR_BN);
  return tiles >= (sms / 2);
}

int pick_bn(int M, int N, int groups, int sms) {
  const int cand[3] = {256, 128, 64};
  const float penalty[3] = {1.0f, 1.8f, 3.0f};  // measured: 128-wide tiles reach ~55% of the 256-wide rate
  int best = 256;
  float best_cost = 1e30f;
  for (int i = 0; i < 3; ++i) {
    long long tiles = (long long)((M + GEMM_BM - 1) / GEMM_BM) * ((N + cand[i] - 1) / cand[i]) * groups;
    long long waves = (tiles + sms - 1) / sms;
    float cost = waves * cand[i] * penalty[i];
    if (cost < best_cost) {
      best_cost = cost;
      best = cand[i];
    }
  }
  return best;
}

}  // namespace

extern "C" {

// Returns 0 on success, a negative code for bad arguments, or a positive cudaError_t.
//   A: K-major  -> [a_outer rows, a_inner = contraction] with leading dimension lda
//      MN-major -> [a_outer = contraction rows, a_inner = M] with leading dimension lda
//   B likewise (rows of a K-major B are the N index).
int mcb_gemm_bf16(const void* A, long long a_inner, long long a_outer, long long lda, int a_mn,  //
                  const void* B, long long b_inner, long long b_outer, long long ldb, int b_mn,  //
                  void* C, long long ldc, long long c_group_stride, int c_fp32, int accumulate,  //
                  int M, int N, int K, float alpha, const void* bias,                            //
                  int mode, int num_groups, const int* offsets, int b_group_rows,               //
                  int* status, int max_sms, int force_bn, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (mode != GEMM_DENSE && (num_groups <= 0 || num_groups > GEMM_MAX_GROUPS || offsets == nullptr)) return -2;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -3;  // TMA needs 16-byte aligned bases and strides
  int sms = device_sm_count();
  if (max_sms > 0 && max_sms < sms) sms = max_sms;
  int groups = (mode == GEMM_GROUPED_K) ? num_groups : 1;
  // force_bn: 0 = choose; 64 / 128 / 256 = single-CTA tile width; 512 = CTA pairs (256 x 256 per cluster)
  const bool pair = force_bn == 512 || (force_bn == 0 && use_pair(M, N, K, mode, sms));
  if (pair && mode != GEMM_DENSE) return -4;
  int bn = pair ? PAIR_HALF_N : (force_bn > 0 ? force_bn : pick_bn(M, N, groups, sms));
  if (bn != 256 && bn != 128 && bn != 64) return -4;

  CUtensorMap ta, tb;
  int rc;
  if (!a_mn)
    rc = make_tmap_2d_bf16(&ta, A, a_inner, a_outer, lda, GEMM_BK, GEMM_BM);
  else
    rc = make_tmap_2d_bf16(&ta, A, a_inner, a_outer, lda, 64, GEMM_BK);
  if (rc) return rc;
  if (!b_mn)
    rc = make_tmap_2d_bf16(&tb, B, b_inner, b_outer, ldb, GEMM_BK, bn);
  else
    rc = make_tmap_2d_bf16(&tb, B, b_inner, b_outer, ldb, 64, GEMM_BK);
  if (rc) return rc;

  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.C = C; p.ldc = ldc; p.c_group_stride = c_group_stride;
  p.bias = bias; p.c_fp32 = c_fp32; p.alpha = alpha;
  // grouped-K (expert weight gradients): many output tiles per unit of math, where reductions would queue at the L2
  p.accumulate = accumulate ? (mode == GEMM_GROUPED_K && c_fp32 ? 2 : 1) : 0;
  p.mode = mode; p.num_groups = num_groups; p.offsets = offsets; p.b_group_rows = b_group_rows;
  p.epilogue = EPI_NONE;
  p.status = status;

  if (pair) {
    const long long ptiles = (long long)((M + PAIR_BM - 1) / PAIR_BM) * ((N + PAIR_BN - 1) / PAIR_BN);
    const int clusters = (int)(ptiles < sms / 2 ? ptiles : sms / 2);
    return (int)launch_pair_major(a_mn, b_mn, ta, tb, p, 2 * clusters, stream);
  }
  long long tiles = (long long)((M + GEMM_BM - 1) / GEMM_BM) * ((N + bn - 1) / bn) * groups;
  int grid = (int)(tiles < sms ? tiles : sms);
  cudaError_t e;
  if (bn == 256) e = launch_major<256>(a_mn, b_mn, ta, tb, p, grid, stream);
  else if (bn == 128) e = launch_major<128>(a_mn, b_mn, ta, tb, p, grid, stream);
  else e = launch_major<64>(a_mn, b_mn, ta, tb, p, grid, stream);
  return (int)e;
}

// Fused language-model head on the GEMM engine: logits = A[M,K] . B[N,K]^T (both K-major) are consumed by the
// epilogue and never stored.
//   grad == 0: `part` [M, ceil(N/256), 2] receives per row and 256-column tile (max, sum exp(logit - max)); `tgt` [M]
//              the logit of the row's label when its column is in [col0, col0 + N) (untouched otherwise: zero it first)
//   grad != 0: C [M, N] bf16 = (exp(logit - lse[row]) - [col0 + column == label]) * g[row]
int mcb_gemm_ce_bf16(const void* A, long long lda, const void* B, long long ldb, int M, int N, int K,
                     const long long* labels, int col0, float* part, float* tgt, const float* lse, const float* g,
                     void* C, long long ldc, int grad, int* status, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  if (labels == nullptr || (grad ? (C == nullptr || lse == nullptr || g == nullptr) : (part == nullptr || tgt == nullptr)))
    return -2;
  constexpr int BN = 256;
  const int sms = device_sm_count();
  CUtensorMap ta, tb;
  int rc = make_tmap_2d_bf16(&ta, A, K, M, lda, GEMM_BK, GEMM_BM);
  if (rc) return rc;
  rc = make_tmap_2d_bf16(&tb, B, K, N, ldb, GEMM_BK, BN);
  if (rc) return rc;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = C; p.ldc = ldc; p.alpha = 1.f; p.mode = GEMM_DENSE;
  p.epilogue = grad ? EPI_CE_GRAD : EPI_CE_STATS;
  p.ce_labels = labels; p.ce_col0 = col0; p.ce_part = part; p.ce_tgt = tgt; p.ce_lse = lse; p.ce_g = g;
  p.status = status;
  const long long tiles = (long long)((M + GEMM_BM - 1) / GEMM_BM) * ((N + BN - 1) / BN);
  const int grid = (int)(tiles < sms ? tiles : sms);
  static bool cfg[2] = {false, false};
  cudaError_t e;
  if (grad) {
    auto kern = gemm_bf16_sm100_kernel<BN, false, false, EPI_CE_GRAD>;
    if (!cfg[1]) {
      if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN>::TOTAL)) != cudaSuccess)
        return (int)e;
      cfg[1] = true;
    }
    kern<<<grid, GEMM_THREADS, GemmSmem<BN>::TOTAL, stream>>>(ta, tb, p);
  } else {
    auto kern = gemm_bf16_sm100_kernel<BN, false, false, EPI_CE_STATS>;
    if (!cfg[0]) {
      if ((e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN>::TOTAL)) != cudaSuccess)
        return (int)e;
      cfg[0] = true;
    }
    kern<<<grid, GEMM_THREADS, GemmSmem<BN>::TOTAL, stream>>>(ta, tb, p);
  }
  return (int)cudaGetLastError();
}

}  // extern "C"

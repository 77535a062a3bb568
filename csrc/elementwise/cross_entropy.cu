// Softmax statistics and gradient for (vocab-parallel) cross entropy over one chunk of logits.
//   mcb_ce_stats   : per row max, sum exp(l - max) and the target logit (0 when the label is in another shard)
//   mcb_ce_dlogits : (exp(l - lse) - onehot(label)) * g  written as bf16 or fp32
// One block per row, 16-byte loads, a single pass (online max/sum).
#include "../common/host_utils.cuh"
#include "../common/ptx.cuh"

using namespace mcb;

namespace {

constexpr int CE_THREADS = 512;

__device__ __forceinline__ void online_merge(float& m, float& s, float m2, float s2) {
  float nm = fmaxf(m, m2);
  if (nm == -INFINITY) {
    s = 0.f;
  } else {
    s = s * __expf(m - nm) + s2 * __expf(m2 - nm);
  }
  m = nm;
}

template <bool FP32>
__device__ __forceinline__ void load8(const void* base, long long idx, float (&f)[8]) {
  if (FP32) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
    float4 a = p[0], b = p[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + idx);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __bfloat1622float2(p[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
}
template <bool FP32>
__device__ __forceinline__ float load1(const void* base, long long idx) {
  return FP32 ? reinterpret_cast<const float*>(base)[idx]
              : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
}

template <bool FP32>
__global__ void __launch_bounds__(CE_THREADS)
ce_stats_kernel(const void* __restrict__ logits, long long ld, const long long* __restrict__ labels, long long rows,
                int V, int vocab_start, float* __restrict__ omax, float* __restrict__ osum, float* __restrict__ otgt) {
  __shared__ float sm[CE_THREADS / 32], ss[CE_THREADS / 32];
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long base = row * ld;
    float m = -INFINITY, s = 0.f;
    const int nvec = V / 8;
    for (int vi = threadIdx.x; vi < nvec; vi += CE_THREADS) {
      float f[8];
      load8<FP32>(logits, base + (long long)vi * 8, f);
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
      float nm = fmaxf(m, lm);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
      s = s * __expf(m - nm) + acc;
      m = nm;
    }
    for (int i = nvec * 8 + threadIdx.x; i < V; i += CE_THREADS) online_merge(m, s, load1<FP32>(logits, base + i), 1.f);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
      online_merge(m, s, m2, s2);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) {
      sm[warp] = m;
      ss[warp] = s;
    }
    __syncthreads();
    if (warp == 0) {
      m = lane < CE_THREADS / 32 ? sm[lane] : -INFINITY;
      s = lane < CE_THREADS / 32 ? ss[lane] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
        online_merge(m, s, m2, s2);
      }
      if (lane == 0) {
        omax[row] = m;
        osum[row] = s;
        long long lab = labels[row] - vocab_start;
        otgt[row] = (lab >= 0 && lab < V) ? load1<FP32>(logits, base + lab) : 0.f;
      }
    }
  }
}

template <bool FP32_IN, bool FP32_OUT>
__global__ void __launch_bounds__(CE_THREADS)
ce_dlogits_kernel(const void* __restrict__ logits, long long ld, const long long* __restrict__ labels,
                  const float* __restrict__ lse, const float* __restrict__ g, long long rows, int V, int vocab_start,
                  void* __restrict__ out) {
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const long long base = row * ld, obase = row * (long long)V;
    const float l = lse[row], gr = g[row];
    const long long lab = labels[row] - vocab_start;
    const int nvec = V / 8;
    for (int vi = threadIdx.x; vi < nvec; vi += CE_THREADS) {
      float f[8];
      load8<FP32_IN>(logits, base + (long long)vi * 8, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float p = __expf(f[j] - l);
        if ((long long)vi * 8 + j == lab) p -= 1.f;
        f[j] = p * gr;
      }
      if (FP32_OUT) {
        float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + obase + (long long)vi * 8);
        o[0] = make_float4(f[0], f[1], f[2], f[3]);
        o[1] = make_float4(f[4], f[5], f[6], f[7]);
      } else {
        uint4 o;
        o.x = pack_bf16x2(f[0], f[1]);
        o.y = pack_bf16x2(f[2], f[3]);
        o.z = pack_bf16x2(f[4], f[5]);
        o.w = pack_bf16x2(f[6], f[7]);
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + obase + (long long)vi * 8) = o;
      }
    }
    for (int i = nvec * 8 + threadIdx.x; i < V; i += CE_THREADS) {
      float p = __expf(load1<FP32_IN>(logits, base + i) - l);
      if (i == lab) p -= 1.f;
      p *= gr;
      if (FP32_OUT) reinterpret_cast<float*>(out)[obase + i] = p;
      else reinterpret_cast<__nv_bfloat16*>(out)[obase + i] = __float2bfloat16(p);
    }
  }
}

}  // namespace

extern "C" {

int mcb_ce_stats(const void* logits, int fp32, long long ld, const long long* labels, long long rows, int V,
                 int vocab_start, float* omax, float* osum, float* otgt, void* stream_) {
  if (rows == 0) return 0;
  const int align = fp32 ? 4 : 8;
  if (ld % align || (reinterpret_cast<uintptr_t>(logits) & 15)) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  long long cap = (long long)device_sm_count() * 4;
  int grid = (int)(rows < cap ? rows : cap);
  if (fp32) ce_stats_kernel<true><<<grid, CE_THREADS, 0, s>>>(logits, ld, labels, rows, V, vocab_start, omax, osum, otgt);
  else ce_stats_kernel<false><<<grid, CE_THREADS, 0, s>>>(logits, ld, labels, rows, V, vocab_start, omax, osum, otgt);
  return (int)cudaGetLastError();
}

int mcb_ce_dlogits(const void* logits, int fp32_in, long long ld, const long long* labels, const float* lse,
                   const float* g, long long rows, int V, int vocab_start, void* out, int fp32_out, void* stream_) {
  if (rows == 0) return 0;
  const int align = fp32_in ? 4 : 8;
  if (ld % align || V % 8 || (reinterpret_cast<uintptr_t>(logits) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  long long cap = (long long)device_sm_count() * 4;
  int grid = (int)(rows < cap ? rows : cap);
#define L(A, B) ce_dlogits_kernel<A, B><<<grid, CE_THREADS, 0, s>>>(logits, ld, labels, lse, g, rows, V, vocab_start, out)
  if (fp32_in && fp32_out) L(true, true);
  else if (fp32_in) L(true, false);
  else if (fp32_out) L(false, true);
  else L(false, false);
#undef L
  return (int)cudaGetLastError();
}

}  // extern "C"

// Fused AdamW step over one contiguous shard of the distributed optimizer, plus the squared-norm reduction
// used for global gradient clipping.  One pass: reads fp32 grad / main param / exp_avg / exp_avg_sq, writes
// them back and writes the bf16 model parameter.  The clip coefficient and the step-dependent bias
// corrections are read from device memory so the step never synchronises with the host.
#include "../common/host_utils.cuh"
#include "../common/ptx.cuh"

using namespace mcb;

namespace {

struct AdamScalars {  // device-resident, 8 floats
  float lr, beta1, beta2, eps, weight_decay, bias_c1, bias_c2, grad_scale;
};

__device__ __forceinline__ void adam_update(float g, float& p, float& m, float& v, const AdamScalars& s) {
  m = s.beta1 * m + (1.f - s.beta1) * g;
  v = s.beta2 * v + (1.f - s.beta2) * g * g;
  const float denom = sqrtf(v / s.bias_c2) + s.eps;
  p = p * (1.f - s.lr * s.weight_decay) - s.lr * (m / s.bias_c1) / denom;
}

// grad_scale = 1/loss_scale ; clip_coef (device) multiplies it ; found_inf != 0 skips the update
template <bool BF16>
__global__ void adam_kernel(const float* __restrict__ grad, float* __restrict__ main, float* __restrict__ m,
                            float* __restrict__ v, void* __restrict__ param, long long n,
                            const AdamScalars* __restrict__ sc, const float* __restrict__ clip_coef,
                            const int* __restrict__ found_inf) {
  if (found_inf && *found_inf) return;
  const AdamScalars s = *sc;
  const float gs = s.grad_scale * (clip_coef ? *clip_coef : 1.f);
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
    if (i + 4 <= n) {
      float4 g = *reinterpret_cast<const float4*>(grad + i);
      float4 p = *reinterpret_cast<float4*>(main + i);
      float4 mm = *reinterpret_cast<float4*>(m + i);
      float4 vv = *reinterpret_cast<float4*>(v + i);
      adam_update(g.x * gs, p.x, mm.x, vv.x, s);
      adam_update(g.y * gs, p.y, mm.y, vv.y, s);
      adam_update(g.z * gs, p.z, mm.z, vv.z, s);
      adam_update(g.w * gs, p.w, mm.w, vv.w, s);
      *reinterpret_cast<float4*>(main + i) = p;
      *reinterpret_cast<float4*>(m + i) = mm;
      *reinterpret_cast<float4*>(v + i) = vv;
      if (param) {
        if (BF16) {
          uint2 o;
          o.x = pack_bf16x2(p.x, p.y);
          o.y = pack_bf16x2(p.z, p.w);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(param) + i) = o;
        } else {
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(param) + i) = p;
        }
      }
    } else {
      for (long long k = i; k < n; ++k) {
        float pk = main[k], mk = m[k], vk = v[k];
        adam_update(grad[k] * gs, pk, mk, vk, s);
        main[k] = pk;
        m[k] = mk;
        v[k] = vk;
        if (param) {
          if (BF16) reinterpret_cast<__nv_bfloat16*>(param)[k] = __float2bfloat16(pk);
          else reinterpret_cast<float*>(param)[k] = pk;
        }
      }
    }
  }
}

// Sum of squares.  With `scratch` every CTA writes its partial sum there and the last CTA to finish (a ticket counter
// at scratch[SQ_MAX_CTAS]) adds the partials in CTA order, so the result repeats bit for bit; without, CTAs add to
// `out` with atomics.
constexpr int SQ_MAX_CTAS = 1024;

__global__ void sqnorm_kernel(const float* __restrict__ x, long long n, float* __restrict__ out,
                              float* __restrict__ scratch) {
  float acc = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x * 4;
  long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  // four independent 16-byte loads in flight per thread while whole strides remain
  for (; i + 3 * stride + 4 <= n; i += 4 * stride) {
    float4 g[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) g[u] = __ldcs(reinterpret_cast<const float4*>(x + i + u * stride));
#pragma unroll
    for (int u = 0; u < 4; ++u) acc += g[u].x * g[u].x + g[u].y * g[u].y + g[u].z * g[u].z + g[u].w * g[u].w;
  }
  for (; i < n; i += stride) {
    if (i + 4 <= n) {
      float4 g = *reinterpret_cast<const float4*>(x + i);
      acc += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
    } else {
      for (long long k = i; k < n; ++k) acc += x[k] * x[k];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float red[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    acc = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
      if (!scratch) {
        atomicAdd(out, acc);
      } else {
        scratch[blockIdx.x] = acc;
        __threadfence();
        unsigned* ticket = reinterpret_cast<unsigned*>(scratch + SQ_MAX_CTAS);
        if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
          __threadfence();
          float total = 0.f;
          for (unsigned b = 0; b < gridDim.x; ++b) total += *reinterpret_cast<volatile float*>(scratch + b);
          *out += total;
          *ticket = 0;
        }
      }
    }
  }
}

// coef = min(1, max_norm / (sqrt(total_sq) + 1e-6)); also stores the norm itself
__global__ void clip_coef_kernel(const float* total_sq, float max_norm, float* coef, float* norm_out) {
  float nrm = sqrtf(*total_sq);
  *norm_out = nrm;
  *coef = max_norm > 0.f ? fminf(1.f, max_norm / (nrm + 1e-6f)) : 1.f;
}

}  // namespace

extern "C" {

int mcb_adam_step(const float* grad, float* main, float* m, float* v, void* param, int param_is_bf16, long long n,
                  const float* scalars, const float* clip_coef, const int* found_inf, void* stream_) {
  if (n == 0) return 0;
  if ((reinterpret_cast<uintptr_t>(grad) | reinterpret_cast<uintptr_t>(main) | reinterpret_cast<uintptr_t>(m) |
       reinterpret_cast<uintptr_t>(v)) & 15)
    return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  long long blocks = (n / 4 + 255) / 256;
  long long cap = (long long)device_sm_count() * 8;
  int grid = (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
  const AdamScalars* sc = reinterpret_cast<const AdamScalars*>(scalars);
  if (param_is_bf16) adam_kernel<true><<<grid, 256, 0, s>>>(grad, main, m, v, param, n, sc, clip_coef, found_inf);
  else adam_kernel<false><<<grid, 256, 0, s>>>(grad, main, m, v, param, n, sc, clip_coef, found_inf);
  return (int)cudaGetLastError();
}

// out (1 float) is accumulated into: zero it before the first call of a step.  `scratch` (optional, 1025 floats, zero
// when allocated, owned by one stream of calls) makes the sum order fixed.
int mcb_sqnorm_accum(const float* x, long long n, float* out, float* scratch, void* stream_) {
  if (n == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  long long blocks = (n / 4 + 255) / 256;
  long long cap = (long long)device_sm_count() * 4;
  if (cap > SQ_MAX_CTAS) cap = SQ_MAX_CTAS;
  int grid = (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
  sqnorm_kernel<<<grid, 256, 0, s>>>(x, n, out, scratch);
  return (int)cudaGetLastError();
}

int mcb_clip_coef(const float* total_sq, float max_norm, float* coef, float* norm_out, void* stream_) {
  clip_coef_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(total_sq, max_norm, coef, norm_out);
  return (int)cudaGetLastError();
}

}  // extern "C"

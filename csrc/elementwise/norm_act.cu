// RMSNorm (plain / zero-centred gamma) forward + backward and SwiGLU-family forward + backward.
// Memory-bound kernels: 16-byte vector accesses, fp32 math, persistent grids sized to the SM count.
#include "../common/partials.cuh"
#include "../common/host_utils.cuh"
#include "../common/ptx.cuh"

using namespace mcb;

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over the block; every thread gets the result.  `red` has 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

struct bf16x8 {
  uint4 raw;
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __bfloat1622float2(p[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ __forceinline__ void pack(const float (&f)[8]) {
    raw.x = pack_bf16x2(f[0], f[1]);
    raw.y = pack_bf16x2(f[2], f[3]);
    raw.z = pack_bf16x2(f[4], f[5]);
    raw.w = pack_bf16x2(f[6], f[7]);
  }
};

// ------------------------------------------------------------------ RMSNorm forward
// One block per row (grid-stride over rows).  H % 8 == 0.  Optional residual add fused in:
// if `res_in` is given, x' = x + res_in is normalised and also written to `res_out`.
template <int VPT>  // vectors (8 bf16) per thread
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res_in,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out, long long rows,
                                   int H, long long ldx, float eps, int zero_centered) {
  __shared__ float red[33];
  const int nvec = H / 8;
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
    const uint4* rr = res_in ? reinterpret_cast<const uint4*>(res_in + row * (long long)H) : nullptr;
    float v[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        bf16x8 t;
        t.raw = xr[vi];
        t.unpack(v[i]);
        if (rr) {
          bf16x8 r;
          r.raw = rr[vi];
          float rf[8];
          r.unpack(rf);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i][j] += rf[j];
          bf16x8 o;
          o.pack(v[i]);
          reinterpret_cast<uint4*>(res_out + row * (long long)H)[vi] = o.raw;
          o.unpack(v[i]);  // normalise exactly what was stored
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
      }
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / H + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        bf16x8 wv;
        wv.raw = reinterpret_cast<const uint4*>(w)[vi];
        float wf[8], o[8];
        wv.unpack(wf);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * (zero_centered ? 1.f + wf[j] : wf[j]);
        bf16x8 ov;
        ov.pack(o);
        reinterpret_cast<uint4*>(y + row * (long long)H)[vi] = ov.raw;
      }
    }
  }
}

// ------------------------------------------------------------------ RMSNorm backward
// dx = rstd * (g - xh * mean(g * xh)),  g = dy * w_eff, xh = x * rstd;  dw += sum_rows dy * xh.
// Persistent blocks: each thread owns fixed columns, accumulates dw over its rows, one atomic per column at the end.
// Two rows are processed per iteration: their loads are in flight together and their row reductions share one
// round of barriers, which is what bounds a one-row-at-a-time block.
__device__ __forceinline__ void block_sum2(float& a, float& b, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  a = warp_sum(a);
  b = warp_sum(b);
  __syncthreads();
  if (lane == 0) {
    red[warp] = a;
    red[33 + warp] = b;
  }
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f, u = lane < nw ? red[33 + lane] : 0.f;
    t = warp_sum(t);
    u = warp_sum(u);
    if (lane == 0) {
      red[32] = t;
      red[65] = u;
    }
  }
  __syncthreads();
  a = red[32];
  b = red[65];
}

template <int VPT>
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                                   float* __restrict__ dw, float* __restrict__ partials, long long rows, int H,
                                   long long ldx, float eps, int zero_centered) {
  __shared__ float red[66];
  const int nvec = H / 8;
  float dwacc[VPT][8];
  float wf[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int vi = threadIdx.x + i * blockDim.x;
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
    if (vi < nvec) {
      bf16x8 wv;
      wv.raw = reinterpret_cast<const uint4*>(w)[vi];
      wv.unpack(wf[i]);
      if (zero_centered) {
#pragma unroll
        for (int j = 0; j < 8; ++j) wf[i][j] += 1.f;
      }
    }
  }
  for (long long row0 = 2LL * blockIdx.x; row0 < rows; row0 += 2LL * gridDim.x) {
    const bool two = row0 + 1 < rows;
    uint4 xr[2][VPT], gr[2][VPT];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const long long row = row0 + ((r == 1 && two) ? 1 : 0);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = threadIdx.x + i * blockDim.x;
        if (vi < nvec) {
          xr[r][i] = reinterpret_cast<const uint4*>(x + row * ldx)[vi];
          gr[r][i] = reinterpret_cast<const uint4*>(dy + row * (long long)H)[vi];
        }
      }
    }
    float ss[2] = {0.f, 0.f}, dot[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; ++r)
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = threadIdx.x + i * blockDim.x;
        if (vi < nvec) {
          float xv[8], gv[8];
          bf16x8 a, b;
          a.raw = xr[r][i];
          b.raw = gr[r][i];
          a.unpack(xv);
          b.unpack(gv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            ss[r] += xv[j] * xv[j];
            dot[r] += gv[j] * wf[i][j] * xv[j];
          }
        }
      }
    float rstd[2];
    if (rstd_in) {
      rstd[0] = rstd_in[row0];
      rstd[1] = two ? rstd_in[row0 + 1] : 0.f;
    } else {
      block_sum2(ss[0], ss[1], red);
      rstd[0] = rsqrtf(ss[0] / H + eps);
      rstd[1] = rsqrtf(ss[1] / H + eps);
    }
    block_sum2(dot[0], dot[1], red);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (r == 1 && !two) break;
      const long long row = row0 + r;
      const float c = dot[r] * rstd[r] * rstd[r] * rstd[r] / H;  // mean(g*xh) * rstd, with xh = x*rstd folded in
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int vi = threadIdx.x + i * blockDim.x;
        if (vi < nvec) {
          float xv[8], gv[8], o[8];
          bf16x8 a, b;
          a.raw = xr[r][i];
          b.raw = gr[r][i];
          a.unpack(xv);
          b.unpack(gv);
          if (dres) {
            bf16x8 rr;
            rr.raw = reinterpret_cast<const uint4*>(dres + row * (long long)H)[vi];
            rr.unpack(o);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = 0.f;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            o[j] += gv[j] * wf[i][j] * rstd[r] - xv[j] * c;
            dwacc[i][j] += gv[j] * xv[j] * rstd[r];
          }
          bf16x8 ov;
          ov.pack(o);
          reinterpret_cast<uint4*>(dx + row * (long long)H)[vi] = ov.raw;
        }
      }
    }
  }
  if (partials) {
    // one row of partial sums per CTA; reduce_partials_kernel adds the rows in a fixed order
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
        float4* o = reinterpret_cast<float4*>(partials + (long long)blockIdx.x * H + vi * 8);
        o[0] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
        o[1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
      }
    }
  } else if (dw) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int vi = threadIdx.x + i * blockDim.x;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(dw + vi * 8 + j, dwacc[i][j]);
      }
    }
  }
}

// ------------------------------------------------------------------ gated activations
// in: [rows, 2F] = [gate | up] ; out: [rows, F].  kind 0: silu(g)*u ; kind 1: quick-geglu with clamp+offset ;
// kind 2: gelu_tanh(g)*u.  Optional per-row scale `probs` (MoE: weight the expert output by the router prob).
__device__ __forceinline__ float act_fwd(float g, int kind) {
  if (kind == 0) return g / (1.f + __expf(-g));
  if (kind == 1) return g / (1.f + __expf(-1.702f * g));
  const float k0 = 0.7978845608f, k1 = 0.044715f;
  float t = tanhf(k0 * (g + k1 * g * g * g));
  return 0.5f * g * (1.f + t);
}
__device__ __forceinline__ float act_grad(float g, int kind) {
  if (kind == 0) {
    float s = 1.f / (1.f + __expf(-g));
    return s * (1.f + g * (1.f - s));
  }
  if (kind == 1) {
    float s = 1.f / (1.f + __expf(-1.702f * g));
    return s * (1.f + 1.702f * g * (1.f - s));
  }
  const float k0 = 0.7978845608f, k1 = 0.044715f;
  float u = k0 * (g + k1 * g * g * g);
  float t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * k0 * (1.f + 3.f * k1 * g * g);
}

__global__ void glu_fwd_kernel(const __nv_bfloat16* __restrict__ in, const float* __restrict__ probs,
                               __nv_bfloat16* __restrict__ out, long long rows, int F, long long ld_in, int kind,
                               float clamp, float offset) {
  const int nvec = F / 8;
  const long long total = rows * nvec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / nvec;
    const int vi = (int)(i - row * nvec);
    bf16x8 g, u;
    g.raw = reinterpret_cast<const uint4*>(in + row * ld_in)[vi];
    u.raw = reinterpret_cast<const uint4*>(in + row * ld_in + F)[vi];
    float gf[8], uf[8], o[8];
    g.unpack(gf);
    u.unpack(uf);
    const float pr = probs ? probs[row] : 1.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float gg = gf[j], uu = uf[j];
      if (clamp > 0.f) {
        gg = fminf(gg, clamp);
        uu = fminf(fmaxf(uu, -clamp), clamp);
      }
      o[j] = act_fwd(gg, kind) * (uu + offset) * pr;
    }
    bf16x8 ov;
    ov.pack(o);
    reinterpret_cast<uint4*>(out + row * (long long)F)[vi] = ov.raw;
  }
}

// din[rows, 2F] from dout[rows, F]; optional dprobs[row] = sum_j dout * act(g) * (u+offset)
__global__ void glu_bwd_kernel(const __nv_bfloat16* __restrict__ in, const float* __restrict__ probs,
                               const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ din,
                               float* __restrict__ dprobs, long long rows, int F, long long ld_in, int kind,
                               float clamp, float offset) {
  // one warp per row chunk so the dprobs reduction stays inside a warp
  const int nvec = F / 8;
  const int lane = threadIdx.x & 31;
  const long long warp_global = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp_global; row < rows; row += nwarps) {
    const float pr = probs ? probs[row] : 1.f;
    float dp = 0.f;
    for (int vi = lane; vi < nvec; vi += 32) {
      bf16x8 g, u, d;
      g.raw = reinterpret_cast<const uint4*>(in + row * ld_in)[vi];
      u.raw = reinterpret_cast<const uint4*>(in + row * ld_in + F)[vi];
      d.raw = reinterpret_cast<const uint4*>(dout + row * (long long)F)[vi];
      float gf[8], uf[8], df[8], dg[8], du[8];
      g.unpack(gf);
      u.unpack(uf);
      d.unpack(df);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float gg = gf[j], uu = uf[j];
        bool g_pass = true, u_pass = true;
        if (clamp > 0.f) {
          g_pass = gg <= clamp;
          u_pass = (uu >= -clamp) && (uu <= clamp);
          gg = fminf(gg, clamp);
          uu = fminf(fmaxf(uu, -clamp), clamp);
        }
        const float a = act_fwd(gg, kind);
        dp += df[j] * a * (uu + offset);
        dg[j] = g_pass ? df[j] * pr * (uu + offset) * act_grad(gg, kind) : 0.f;
        du[j] = u_pass ? df[j] * pr * a : 0.f;
      }
      bf16x8 og, ou;
      og.pack(dg);
      ou.pack(du);
      reinterpret_cast<uint4*>(din + row * (long long)(2 * F))[vi] = og.raw;
      reinterpret_cast<uint4*>(din + row * (long long)(2 * F) + F)[vi] = ou.raw;
    }
    if (dprobs) {
      dp = warp_sum(dp);
      if (lane == 0) dprobs[row] = dp;
    }
  }
}

int pick_threads(int H, int* vpt) {
  const int nvec = H / 8;
  int threads = 128;
  while (threads < 1024 && nvec > threads * 2) threads *= 2;
  *vpt = (nvec + threads - 1) / threads;
  return threads;
}

}  // namespace

extern "C" {

int mcb_rmsnorm_fwd(const void* x, const void* res_in, const void* w, void* y, void* res_out, float* rstd,
                    long long rows, int H, long long ldx, float eps, int zero_centered, void* stream_) {
  if (rows == 0) return 0;
  if (H % 8 || ldx % 8) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  int vpt, threads = pick_threads(H, &vpt);
  long long grid = rows < (long long)device_sm_count() * 16 ? rows : (long long)device_sm_count() * 16;
#define LAUNCH(V)                                                                                                    \
  rmsnorm_fwd_kernel<V><<<(int)grid, threads, 0, s>>>(                                                                \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)res_in, (const __nv_bfloat16*)w, (__nv_bfloat16*)y,              \
      (__nv_bfloat16*)res_out, rstd, rows, H, ldx, eps, zero_centered)
  if (vpt <= 1) LAUNCH(1);
  else if (vpt <= 2) LAUNCH(2);
  else if (vpt <= 4) LAUNCH(4);
  else if (vpt <= 8) LAUNCH(8);
  else return -2;
#undef LAUNCH
  return (int)cudaGetLastError();
}

static int rmsnorm_bwd_launch(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                              float* dw, float* partials, long long rows, int H, long long ldx, float eps,
                              int zero_centered, cudaStream_t s) {
  if (rows == 0) return 0;
  if (H % 8 || ldx % 8) return -1;
  // the two-rows-per-iteration kernel needs up to ~160 registers: blocks stay at <= 256 threads
  const int nvec = H / 8;
  int threads = nvec <= 128 ? 128 : 256;
  int vpt = (nvec + threads - 1) / threads;
  if (vpt > 8) return -2;                      // H > 16384
  long long cap = (long long)device_sm_count() * (vpt <= 2 ? 2 : 1);
  long long pairs = (rows + 1) / 2;
  long long grid = pairs < cap ? pairs : cap;
  if (!dw) partials = nullptr;
#define LAUNCH(V)                                                                                                    \
  rmsnorm_bwd_kernel<V><<<(int)grid, threads, 0, s>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x,              \
                                                      (const __nv_bfloat16*)w, rstd, (const __nv_bfloat16*)dres,      \
                                                      (__nv_bfloat16*)dx, dw, partials, rows, H, ldx, eps,            \
                                                      zero_centered)
  if (vpt <= 1) LAUNCH(1);
  else if (vpt <= 2) LAUNCH(2);
  else if (vpt <= 4) LAUNCH(4);
  else if (vpt <= 8) LAUNCH(8);
  else return -2;
#undef LAUNCH
  if (partials) launch_reduce_partials(partials, (int)grid, H, dw, nullptr, H, s);
  return (int)cudaGetLastError();
}

// dw (fp32, [H]) is accumulated into (with atomics: the sum order varies from run to run); pass nullptr to skip.
// dres (optional) is added to dx (residual branch).
int mcb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                    float* dw, long long rows, int H, long long ldx, float eps, int zero_centered, void* stream_) {
  return rmsnorm_bwd_launch(dy, x, w, rstd, dres, dx, dw, nullptr, rows, H, ldx, eps, zero_centered,
                            reinterpret_cast<cudaStream_t>(stream_));
}

// Rows of fp32 scratch the deterministic variant needs for `rows` rows of width H (each H floats wide).
int mcb_rmsnorm_bwd_partial_rows(long long rows, int H) {
  const int nvec = H / 8;
  const int threads = nvec <= 128 ? 128 : 256;
  const int vpt = (nvec + threads - 1) / threads;
  const long long cap = (long long)device_sm_count() * (vpt <= 2 ? 2 : 1);
  const long long pairs = (rows + 1) / 2;
  return (int)(pairs < cap ? pairs : cap);
}

// Same as mcb_rmsnorm_bwd, but the weight gradient is summed in a fixed order through `partials`
// ([mcb_rmsnorm_bwd_partial_rows(rows, H), H] fp32 scratch), so it repeats bit for bit.
int mcb_rmsnorm_bwd_det(const void* dy, const void* x, const void* w, const float* rstd, const void* dres, void* dx,
                        float* dw, float* partials, long long rows, int H, long long ldx, float eps, int zero_centered,
                        void* stream_) {
  return rmsnorm_bwd_launch(dy, x, w, rstd, dres, dx, dw, partials, rows, H, ldx, eps, zero_centered,
                            reinterpret_cast<cudaStream_t>(stream_));
}

int mcb_glu_fwd(const void* in, const float* probs, void* out, long long rows, int F, long long ld_in, int kind,
                float clamp, float offset, void* stream_) {
  if (rows == 0) return 0;
  if (F % 8 || ld_in % 8) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  long long total = rows * (F / 8);
  long long blocks = (total + 255) / 256;
  long long cap = (long long)device_sm_count() * 8;
  glu_fwd_kernel<<<(int)(blocks < cap ? blocks : cap), 256, 0, s>>>((const __nv_bfloat16*)in, probs,
                                                                     (__nv_bfloat16*)out, rows, F, ld_in, kind, clamp,
                                                                     offset);
  return (int)cudaGetLastError();
}

int mcb_glu_bwd(const void* in, const float* probs, const void* dout, void* din, float* dprobs, long long rows, int F,
                long long ld_in, int kind, float clamp, float offset, void* stream_) {
  if (rows == 0) return 0;
  if (F % 8 || ld_in % 8) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  long long blocks = (rows + 7) / 8;  // 8 warps per block, one row per warp
  long long cap = (long long)device_sm_count() * 8;
  glu_bwd_kernel<<<(int)(blocks < cap ? blocks : cap), 256, 0, s>>>((const __nv_bfloat16*)in, probs,
                                                                     (const __nv_bfloat16*)dout, (__nv_bfloat16*)din,
                                                                     dprobs, rows, F, ld_in, kind, clamp, offset);
  return (int)cudaGetLastError();
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// RMSNorm backward for callers that must not allocate (declaration and contract: norm_noalloc.h).
// The weight-gradient accumulator that mcb_rmsnorm_bwd receives from its caller lives here in a fixed device array.
// ---------------------------------------------------------------------------------------------------------------
#define MCB_NOALLOC_MAX_H 16384

static __device__ __align__(256) float g_rmsnorm_dw_scratch[MCB_NOALLOC_MAX_H];

namespace {

__global__ void dw_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int H) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < H) dst[i] = __float2bfloat16(src[i]);
}

// Device address of the scratch array on the current device; resolved once per device.
// In host code `g_rmsnorm_dw_scratch` itself is only a handle for the runtime, never a pointer a kernel may use.
// The cache is filled without a lock: two host threads that race on a device's first call both resolve the same
// address and store the same value (an aligned pointer store), so the race is benign.
int noalloc_scratch_ptr(float** out) {
  static float* per_device[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return -5;
  if (per_device[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rmsnorm_dw_scratch);
    if (e != cudaSuccess) return (int)e;
    per_device[dev] = p;
  }
  *out = per_device[dev];
  return 0;
}

}  // namespace

extern "C" int mcb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, void* dx, void* dw_bf16,
                                       long long rows, int H, long long ldx, float eps, int zero_centered,
                                       void* stream_) {
  if (H <= 0 || H > MCB_NOALLOC_MAX_H) return -20;  // beyond the fixed scratch: use mcb_rmsnorm_bwd instead
  if (H % 8 || ldx % 8) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  float* scratch = nullptr;
  int rc = noalloc_scratch_ptr(&scratch);
  if (rc) return rc;
  // the array keeps the previous call's sums: clear the part this call uses
  cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(float) * H, s);
  if (e != cudaSuccess) return (int)e;
  if (rows > 0) {
    rc = mcb_rmsnorm_bwd(dy, x, w, nullptr, nullptr, dx, dw_bf16 ? scratch : nullptr, rows, H, ldx, eps,
                         zero_centered, stream_);
    if (rc) return rc;
  }
  if (dw_bf16) {
    dw_to_bf16_kernel<<<(H + 255) / 256, 256, 0, s>>>(scratch, reinterpret_cast<__nv_bfloat16*>(dw_bf16), H);
    e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}

// Element-wise and recurrent kernels of the linear-attention blocks (gated DeltaNet, lightning attention).
//
//   causal depthwise conv1d (+SiLU) forward / backward over packed sequences          (memory bound)
//   gated RMSNorm  y = rmsnorm(x) * w * silu(z)  forward / backward                  (memory bound)
//   simple gated linear attention with a constant per-head decay, forward / backward (recurrent, fp32 state in
//   registers):   S_t = exp(g_h) S_{t-1} + k_t v_t^T,   o_t = scale * S_t^T q_t
//
// Packed sequences are described by `seq_start[t]` (index of the first token of t's sequence), as in the attention
// kernels: no host synchronisation, histories never cross a sequence boundary.
#include "../common/host_utils.cuh"
#include "../common/ptx.cuh"

using namespace mcb;

namespace {

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]);
  o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]);
  o.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = o;
}

// the KW taps of 8 consecutive channels are 8 * KW contiguous bf16 (w is [C, KW]): fetched with 16-byte loads when the
// span is a multiple of 16 bytes, which it is for KW = 2 and 4
template <int KW>
__device__ __forceinline__ void load_taps(const __nv_bfloat16* __restrict__ w, int c0, float (&wt)[8][KW]) {
  if constexpr ((8 * KW * 2) % 16 == 0) {
    const uint4* src = reinterpret_cast<const uint4*>(w + (long long)c0 * KW);
    float flat[8 * KW];
#pragma unroll
    for (int v = 0; v < 8 * KW / 8; ++v) {
      const uint4 raw = src[v];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(h[i]);
        flat[v * 8 + 2 * i] = t.x;
        flat[v * 8 + 2 * i + 1] = t.y;
      }
    }
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
      for (int j = 0; j < KW; ++j) wt[c][j] = flat[c * KW + j];
  } else {
#pragma unroll
    for (int c = 0; c < 8; ++c)
#pragma unroll
      for (int j = 0; j < KW; ++j) wt[c][j] = __bfloat162float(w[(c0 + c) * KW + j]);
  }
}

// ------------------------------------------------------------------------------------------ causal conv1d + SiLU
// x, y [T, C] bf16; w [C, KW] bf16 (KW <= 4); thread = (token, 8 channels)
template <int KW>
__global__ void conv1d_silu_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                       const int* __restrict__ seq_start, __nv_bfloat16* __restrict__ y, int T, int C,
                                       int act) {
  const int cv = C / 8;
  const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (id >= (long long)T * cv) return;
  const int t = int(id / cv), c0 = int(id % cv) * 8;
  const int s0 = seq_start[t];
  float wt[8][KW];
  load_taps<KW>(w, c0, wt);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < KW; ++j) {
    const int tt = t - (KW - 1) + j;
    if (tt >= s0) {
      float f[8];
      load8(x + (long long)tt * C + c0, f);
#pragma unroll
      for (int c = 0; c < 8; ++c) acc[c] = fmaf(wt[c][j], f[c], acc[c]);
    }
  }
  if (act) {
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = acc[c] * sigmoidf_(acc[c]);
  }
  store8(y + (long long)t * C + c0, acc);
}

// dx [T, C] bf16, dw [C, KW] fp32 (accumulated with atomics; zeroed by the caller).  Block = 32 tokens x 8-channel
// groups: each thread walks 32 consecutive tokens of its channels so the dw partial sums stay in registers.
template <int KW>
__global__ void conv1d_silu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                       const __nv_bfloat16* __restrict__ dy, const int* __restrict__ seq_start,
                                       __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, int T, int C, int act) {
  constexpr int TOK = 32;
  const int cv = C / 8;
  const long long id = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int nchunk = (T + TOK - 1) / TOK;
  if (id >= (long long)nchunk * cv) return;
  const int chunk = int(id / cv), c0 = int(id % cv) * 8;
  const int t_lo = chunk * TOK, t_hi = min(T, t_lo + TOK);
  float wt[8][KW], dwa[8][KW];
  load_taps<KW>(w, c0, wt);
#pragma unroll
  for (int c = 0; c < 8; ++c)
#pragma unroll
    for (int j = 0; j < KW; ++j) dwa[c][j] = 0.f;
  // dpre of tokens t .. t+KW-1 is needed for dx[t]; walk tokens and keep a window of dpre values
  // dpre[u] = dy[u] * d silu(pre[u]),  pre[u] = sum_j w[j] x[u-(KW-1)+j]
  auto dpre_at = [&](int u, bool own, float (&out)[8]) {
    const int s0 = seq_start[u];
    float pre[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float xs[KW][8];
#pragma unroll
    for (int j = 0; j < KW; ++j) {
      const int tt = u - (KW - 1) + j;
      if (tt >= s0) {
        load8(x + (long long)tt * C + c0, xs[j]);
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c) xs[j][c] = 0.f;
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) pre[c] = fmaf(wt[c][j], xs[j][c], pre[c]);
    }
    float g[8];
    load8(dy + (long long)u * C + c0, g);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float d = g[c];
      if (act) {
        const float s = sigmoidf_(pre[c]);
        d *= s * (1.f + pre[c] * (1.f - s));
      }
      out[c] = d;
      if (own) {   // every token's weight-gradient term is added exactly once, by the thread that owns the token
#pragma unroll
        for (int j = 0; j < KW; ++j) dwa[c][j] = fmaf(d, xs[j][c], dwa[c][j]);
      }
    }
  };
  for (int t = t_lo; t < t_hi; ++t) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const int s0 = seq_start[t];
    // dx[t] = sum_j w[j] * dpre[t + (KW-1) - j]  for targets in the same sequence
#pragma unroll
    for (int j = 0; j < KW; ++j) {
      const int u = t + (KW - 1) - j;
      if (u < T && seq_start[u] == s0) {
        float d[8];
        dpre_at(u, u == t, d);
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = fmaf(wt[c][j], d[c], acc[c]);
      }
    }
    store8(dx + (long long)t * C + c0, acc);
  }
#pragma unroll
  for (int c = 0; c < 8; ++c)
#pragma unroll
    for (int j = 0; j < KW; ++j) atomicAdd(&dw[(c0 + c) * KW + j], dwa[c][j]);
}

// ------------------------------------------------------------------------------------------ gated RMSNorm
// rows x D (D = 64, 128 or 256): one warp per row.  y = x * rstd * w * silu(z)
template <int D>
__global__ void gated_rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ z,
                                         const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                         float* __restrict__ rstd, long long rows, float eps) {
  constexpr int PER = D / 32;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  float xv[PER], zv[PER];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    xv[i] = __bfloat162float(x[row * D + lane + 32 * i]);
    zv[i] = __bfloat162float(z[row * D + lane + 32 * i]);
    ss += xv[i] * xv[i];
  }
  ss = wsum(ss);
  const float r = rsqrtf(ss / D + eps);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    // the normalised value is rounded to bf16 before the weight multiply, as the module it replaces does
    const float n = __bfloat162float(__float2bfloat16(xv[i] * r));
    const float wv = __bfloat162float(w[lane + 32 * i]);
    y[row * D + lane + 32 * i] = __float2bfloat16(wv * n * zv[i] * sigmoidf_(zv[i]));
  }
  if (lane == 0) rstd[row] = r;
}

template <int D>
__global__ void gated_rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ z,
                                         const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ dy,
                                         const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx,
                                         __nv_bfloat16* __restrict__ dz, float* __restrict__ dw, long long rows) {
  constexpr int PER = D / 32;
  __shared__ float dws[D];
  for (int i = threadIdx.x; i < D; i += blockDim.x) dws[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float dwl[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) dwl[i] = 0.f;
  for (long long row = (long long)blockIdx.x * nw + wib; row < rows; row += (long long)gridDim.x * nw) {
    const float r = rstd[row];
    float xv[PER], gz[PER], dn[PER];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int c = lane + 32 * i;
      xv[i] = __bfloat162float(x[row * D + c]);
      const float zv = __bfloat162float(z[row * D + c]);
      const float g = __bfloat162float(dy[row * D + c]);
      const float wv = __bfloat162float(w[c]);
      const float s = sigmoidf_(zv);
      const float n = xv[i] * r;
      gz[i] = g * wv * n * s * (1.f + zv * (1.f - s));     // d/dz of silu(z)
      dn[i] = g * wv * zv * s;                             // gradient w.r.t. the normalised value
      dwl[i] += g * n * zv * s;
      dot += dn[i] * xv[i];
    }
    dot = wsum(dot);
    const float k = dot * r * r * r / D;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int c = lane + 32 * i;
      dx[row * D + c] = __float2bfloat16(dn[i] * r - xv[i] * k);
      dz[row * D + c] = __float2bfloat16(gz[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < PER; ++i) atomicAdd(&dws[lane + 32 * i], dwl[i]);
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(&dw[i], dws[i]);
}

// ------------------------------------------------------------------------------------------ simple GLA (recurrent)
// q, k [T, H, DK], v, o [T, H, DV] bf16; decay[h] = g_h <= 0 (log-decay per step); one CTA of DV threads per
// (sequence, head): thread j keeps column j of the state S [DK x DV] in registers.  q and k of the current token are
// staged in shared memory (double buffered) so every thread reads them as broadcasts.
template <int DK, int DV>
__global__ void __launch_bounds__(DV)
simple_gla_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                      const __nv_bfloat16* __restrict__ v, const float* __restrict__ decay,
                      const int* __restrict__ cu_seqlens, __nv_bfloat16* __restrict__ o, int H, float scale) {
  __shared__ float qs[2][DK], ks[2][DK];
  const int seq = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
  const int t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
  const float a = __expf(decay[h]);
  float S[DK];
#pragma unroll
  for (int i = 0; i < DK; ++i) S[i] = 0.f;
  auto stage = [&](int t, int b) {
    for (int i = j; i < DK; i += DV) {
      qs[b][i] = __bfloat162float(q[((long long)t * H + h) * DK + i]) * scale;
      ks[b][i] = __bfloat162float(k[((long long)t * H + h) * DK + i]);
    }
  };
  if (t0 < t1) stage(t0, 0);
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    const int b = (t - t0) & 1;
    if (t + 1 < t1) stage(t + 1, b ^ 1);
    const float vj = __bfloat162float(v[((long long)t * H + h) * DV + j]);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < DK; ++i) {
      S[i] = fmaf(S[i], a, ks[b][i] * vj);
      acc = fmaf(S[i], qs[b][i], acc);
    }
    o[((long long)t * H + h) * DV + j] = __float2bfloat16(acc);
    __syncthreads();
  }
}

// Backward in three sweeps with no stored states (DK == DV == number of threads).
//   forward sweep, thread = row i of S_t :      dq_t[i] = scale * sum_c S_t[i, c] do_t[c]
//   reverse sweep, thread = row i of R_t :      R_t = a R_{t+1} + scale * q_t do_t^T,   dk_t[i] = sum_c R_t[i, c] v_t[c]
//   reverse sweep, thread = column c of R_t :   dv_t[c] = sum_i R_t[i, c] k_t[i]
// Owning rows for dq / dk and columns for dv keeps every reduction inside a thread.
template <int DK, int DV>
__global__ void __launch_bounds__(DK)
simple_gla_bwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                      const __nv_bfloat16* __restrict__ v, const __nv_bfloat16* __restrict__ dout,
                      const float* __restrict__ decay, const int* __restrict__ cu_seqlens,
                      __nv_bfloat16* __restrict__ dq, __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv,
                      int H, float scale) {
  static_assert(DK == DV, "square state only");
  __shared__ float sa[DV], sb[DV];
  const int seq = blockIdx.x, h = blockIdx.y, i = threadIdx.x;
  const int t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
  const float a = __expf(decay[h]);
  float M[DV];
  // ---- forward sweep: dq (row i of S)
#pragma unroll
  for (int c = 0; c < DV; ++c) M[c] = 0.f;
  for (int t = t0; t < t1; ++t) {
    const long long base = (long long)t * H + h;
    sa[i] = __bfloat162float(v[base * DV + i]);
    sb[i] = __bfloat162float(dout[base * DV + i]);
    __syncthreads();
    const float ki = __bfloat162float(k[base * DK + i]);
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < DV; ++c) {
      M[c] = fmaf(M[c], a, ki * sa[c]);
      acc = fmaf(M[c], sb[c], acc);
    }
    dq[base * DK + i] = __float2bfloat16(acc * scale);
    __syncthreads();
  }
  // ---- reverse sweep: dk (row i of R)
#pragma unroll
  for (int c = 0; c < DV; ++c) M[c] = 0.f;
  for (int t = t1 - 1; t >= t0; --t) {
    const long long base = (long long)t * H + h;
    sa[i] = __bfloat162float(v[base * DV + i]);
    sb[i] = __bfloat162float(dout[base * DV + i]);
    __syncthreads();
    const float qi = __bfloat162float(q[base * DK + i]) * scale;
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < DV; ++c) {
      M[c] = fmaf(M[c], a, qi * sb[c]);
      acc = fmaf(M[c], sa[c], acc);
    }
    dk[base * DK + i] = __float2bfloat16(acc);
    __syncthreads();
  }
  // ---- reverse sweep: dv (column i of R)
#pragma unroll
  for (int c = 0; c < DK; ++c) M[c] = 0.f;
  for (int t = t1 - 1; t >= t0; --t) {
    const long long base = (long long)t * H + h;
    sa[i] = __bfloat162float(q[base * DK + i]) * scale;
    sb[i] = __bfloat162float(k[base * DK + i]);
    __syncthreads();
    const float gi = __bfloat162float(dout[base * DV + i]);
    float acc = 0.f;
#pragma unroll
    for (int r = 0; r < DK; ++r) {
      M[r] = fmaf(M[r], a, sa[r] * gi);
      acc = fmaf(M[r], sb[r], acc);
    }
    dv[base * DV + i] = __float2bfloat16(acc);
    __syncthreads();
  }
}

}  // namespace

extern "C" {

int mcb_conv1d_silu_fwd(const void* x, const void* w, const int* seq_start, void* y, int T, int C, int KW, int act,
                        void* stream_) {
  if (T == 0) return 0;
  if (C % 8) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const long long n = (long long)T * (C / 8);
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (KW == 4)
    conv1d_silu_fwd_kernel<4><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, seq_start,
                                                   (__nv_bfloat16*)y, T, C, act);
  else if (KW == 2)
    conv1d_silu_fwd_kernel<2><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, seq_start,
                                                   (__nv_bfloat16*)y, T, C, act);
  else if (KW == 3)
    conv1d_silu_fwd_kernel<3><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, seq_start,
                                                   (__nv_bfloat16*)y, T, C, act);
  else
    return -3;
  return (int)cudaGetLastError();
}

// dw [C, KW] fp32 must be zero on entry
int mcb_conv1d_silu_bwd(const void* x, const void* w, const void* dy, const int* seq_start, void* dx, float* dw, int T,
                        int C, int KW, int act, void* stream_) {
  if (T == 0) return 0;
  if (C % 8) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const long long n = (long long)((T + 31) / 32) * (C / 8);
  const unsigned grid = (unsigned)((n + 127) / 128);
#define MCB_CONV_BWD(K_)                                                                                              \
  conv1d_silu_bwd_kernel<K_><<<grid, 128, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,                    \
                                                  (const __nv_bfloat16*)dy, seq_start, (__nv_bfloat16*)dx, dw, T, C, act)
  if (KW == 4) MCB_CONV_BWD(4);
  else if (KW == 3) MCB_CONV_BWD(3);
  else if (KW == 2) MCB_CONV_BWD(2);
  else return -3;
#undef MCB_CONV_BWD
  return (int)cudaGetLastError();
}

int mcb_gated_rmsnorm_fwd(const void* x, const void* z, const void* w, void* y, float* rstd, long long rows, int D,
                          float eps, void* stream_) {
  if (rows == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const unsigned grid = (unsigned)((rows + 7) / 8);
#define MCB_GN_FWD(D_)                                                                                               \
  gated_rmsnorm_fwd_kernel<D_><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)z,                 \
                                                    (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rstd, rows, eps)
  if (D == 128) MCB_GN_FWD(128);
  else if (D == 64) MCB_GN_FWD(64);
  else if (D == 256) MCB_GN_FWD(256);
  else return -3;
#undef MCB_GN_FWD
  return (int)cudaGetLastError();
}

// dw [D] fp32 must be zero on entry
int mcb_gated_rmsnorm_bwd(const void* x, const void* z, const void* w, const void* dy, const float* rstd, void* dx,
                          void* dz, float* dw, long long rows, int D, void* stream_) {
  if (rows == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const long long want = (rows + 7) / 8;
  const unsigned grid = (unsigned)(want < 4LL * device_sm_count() ? want : 4LL * device_sm_count());
#define MCB_GN_BWD(D_)                                                                                               \
  gated_rmsnorm_bwd_kernel<D_><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)z,                 \
                                                    (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy, rstd,          \
                                                    (__nv_bfloat16*)dx, (__nv_bfloat16*)dz, dw, rows)
  if (D == 128) MCB_GN_BWD(128);
  else if (D == 64) MCB_GN_BWD(64);
  else if (D == 256) MCB_GN_BWD(256);
  else return -3;
#undef MCB_GN_BWD
  return (int)cudaGetLastError();
}

// q, k [T, H, DK]; v, o [T, H, DV]; decay [H] fp32 (log-decay per step, <= 0); cu_seqlens [n_seq + 1] int32
int mcb_simple_gla_fwd(const void* q, const void* k, const void* v, const float* decay, const int* cu_seqlens, void* o,
                       int n_seq, int H, int DK, int DV, float scale, void* stream_) {
  if (n_seq == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  dim3 grid(n_seq, H);
  if (DK == 128 && DV == 128)
    simple_gla_fwd_kernel<128, 128><<<grid, 128, 0, s>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
                                                         (const __nv_bfloat16*)v, decay, cu_seqlens, (__nv_bfloat16*)o,
                                                         H, scale);
  else if (DK == 64 && DV == 64)
    simple_gla_fwd_kernel<64, 64><<<grid, 64, 0, s>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k,
                                                      (const __nv_bfloat16*)v, decay, cu_seqlens, (__nv_bfloat16*)o, H,
                                                      scale);
  else
    return -3;
  return (int)cudaGetLastError();
}

int mcb_simple_gla_bwd(const void* q, const void* k, const void* v, const void* dout, const float* decay,
                       const int* cu_seqlens, void* dq, void* dk, void* dv, int n_seq, int H, int DK, int DV,
                       float scale, void* stream_) {
  if (n_seq == 0) return 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  dim3 grid(n_seq, H);
  if (DK == 128 && DV == 128)
    simple_gla_bwd_kernel<128, 128><<<grid, 128, 0, s>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const __nv_bfloat16*)dout, decay,
        cu_seqlens, (__nv_bfloat16*)dq, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, H, scale);
  else if (DK == 64 && DV == 64)
    simple_gla_bwd_kernel<64, 64><<<grid, 64, 0, s>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (const __nv_bfloat16*)dout, decay,
        cu_seqlens, (__nv_bfloat16*)dq, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, H, scale);
  else
    return -3;
  return (int)cudaGetLastError();
}

}  // extern "C"

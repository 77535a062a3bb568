// Fused post-processing of a packed QKV projection: split per query group, per-head RMSNorm on q/k
// (optional), rotary embedding on the first `rot` dims (rotate-half or interleaved pairs), and the
// transposition-free scatter into separate q / k / v (/ gate) tensors the attention kernel reads.
// One pass over the data instead of split + 2 norms + 2 ropes + copies.  Backward is the exact
// transpose (inverse rotation, norm backward, per-head weight gradients).
//
// Packed layout per token (the layout the bridge produces for `linear_qkv`):
//   for each of `ng` groups: [ qpg query heads (each optionally followed by its gate head) | k | v ], head size d.
// cos/sin are per-token tables [T, rot/2] fp32, so positions, packing, context-parallel chunking,
// MRoPE sections and attention scaling are all decided by whoever builds the table.
#include "../common/host_utils.cuh"
#include "../common/ptx.cuh"

using namespace mcb;

namespace {

constexpr int MAX_D = 256;
constexpr int WARPS = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct QkvLayout {
  int ng, qpg, d, gate;  // gate: 1 -> q heads are interleaved with gate heads
  int rot;               // rotary dims (0 = none)
  int interleaved;       // 1 -> pairs (2i, 2i+1); 0 -> pairs (i, i + rot/2)
  int norm;              // 1 -> per-head RMSNorm on q and k
  int zero_centered;
  float eps;
  long long ld;          // row stride of the packed tensor
};

// slot -> kind: 0 q, 1 gate, 2 k, 3 v ; head index within its output tensor
__device__ __forceinline__ void decode_slot(const QkvLayout& L, int slot, int& kind, int& head) {
  const int per_group = L.qpg * (1 + L.gate) + 2;
  const int g = slot / per_group, r = slot - g * per_group;
  const int nqslots = L.qpg * (1 + L.gate);
  if (r < nqslots) {
    if (L.gate) {
      kind = (r & 1) ? 1 : 0;
      head = g * L.qpg + (r >> 1);
    } else {
      kind = 0;
      head = g * L.qpg + r;
    }
  } else if (r == nqslots) {
    kind = 2;
    head = g;
  } else {
    kind = 3;
    head = g;
  }
}

__global__ void __launch_bounds__(WARPS * 32)
qkv_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ wq,
               const __nv_bfloat16* __restrict__ wk, const float* __restrict__ cosb, const float* __restrict__ sinb,
               __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ v,
               __nv_bfloat16* __restrict__ gate, long long T, QkvLayout L) {
  __shared__ float sm[WARPS][MAX_D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slots = L.ng * (L.qpg * (1 + L.gate) + 2);
  const int nq = L.ng * L.qpg, d = L.d, half = L.rot / 2;
  // a block walks tokens, its warps walk the heads of the token: no 64-bit division on the hot path
  for (long long t = blockIdx.x; t < T; t += gridDim.x)
  for (int slot = warp; slot < slots; slot += WARPS) {
    int kind, head;
    decode_slot(L, slot, kind, head);
    const __nv_bfloat16* src = qkv + t * L.ld + (long long)slot * d;
    __nv_bfloat16* dst = kind == 0 ? q + (t * nq + head) * d
                         : kind == 1 ? gate + (t * nq + head) * d
                         : kind == 2 ? k + (t * L.ng + head) * d
                                     : v + (t * L.ng + head) * d;
    if (kind == 1 || kind == 3 || (!L.norm && L.rot == 0)) {
      for (int i = lane * 8; i < d; i += 256) *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
      continue;
    }
    float ss = 0.f;
    for (int i = lane * 2; i < d; i += 64) {
      float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + i));
      sm[warp][i] = f.x;
      sm[warp][i + 1] = f.y;
      ss += f.x * f.x + f.y * f.y;
    }
    float rstd = 1.f;
    const __nv_bfloat16* wn = kind == 0 ? wq : wk;
    if (L.norm) {
      ss = warp_sum(ss);
      rstd = rsqrtf(ss / d + L.eps);
    }
    __syncwarp();
    for (int i = lane * 2; i < d; i += 64) {
      float o[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int idx = i + e;
        float val = sm[warp][idx] * rstd;
        if (L.norm) val *= (L.zero_centered ? 1.f : 0.f) + __bfloat162float(wn[idx]);
        if (idx < L.rot) {
          int partner, fi;
          float sign;
          if (L.interleaved) {
            partner = idx ^ 1;
            fi = idx >> 1;
            sign = (idx & 1) ? 1.f : -1.f;
          } else {
            partner = idx < half ? idx + half : idx - half;
            fi = idx < half ? idx : idx - half;
            sign = idx < half ? -1.f : 1.f;
          }
          float pv = sm[warp][partner] * rstd;
          if (L.norm) pv *= (L.zero_centered ? 1.f : 0.f) + __bfloat162float(wn[partner]);
          const float c = cosb[t * half + fi], s = sinb[t * half + fi];
          val = val * c + sign * pv * s;
        }
        o[e] = val;
      }
      *reinterpret_cast<uint32_t*>(dst + i) = pack_bf16x2(o[0], o[1]);
    }
    __syncwarp();
  }
}

__global__ void __launch_bounds__(WARPS * 32)
qkv_bwd_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ wq,
               const __nv_bfloat16* __restrict__ wk, const float* __restrict__ cosb, const float* __restrict__ sinb,
               const __nv_bfloat16* __restrict__ dq, const __nv_bfloat16* __restrict__ dk,
               const __nv_bfloat16* __restrict__ dv, const __nv_bfloat16* __restrict__ dgate,
               __nv_bfloat16* __restrict__ dqkv, float* __restrict__ dwq, float* __restrict__ dwk, long long T,
               QkvLayout L) {
  __shared__ float sx[WARPS][MAX_D];   // raw input head
  __shared__ float sg[WARPS][MAX_D];   // gradient after inverse rotation
  __shared__ float sdw[2][MAX_D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slots = L.ng * (L.qpg * (1 + L.gate) + 2);
  const int nq = L.ng * L.qpg, d = L.d, half = L.rot / 2;
  for (int i = threadIdx.x; i < 2 * MAX_D; i += blockDim.x) (&sdw[0][0])[i] = 0.f;
  __syncthreads();
  // every lane always touches the same head positions, so the norm-weight gradients are summed in registers over all
  // the heads a warp visits and meet in shared memory once, after the loop
  float dw_acc[2][MAX_D / 32];
#pragma unroll
  for (int a = 0; a < 2; ++a)
#pragma unroll
    for (int b = 0; b < MAX_D / 32; ++b) dw_acc[a][b] = 0.f;
  // a block walks tokens, its warps walk the heads of the token: no 64-bit division on the hot path
  for (long long t = blockIdx.x; t < T; t += gridDim.x)
  for (int slot = warp; slot < slots; slot += WARPS) {
    int kind, head;
    decode_slot(L, slot, kind, head);
    const __nv_bfloat16* src = qkv + t * L.ld + (long long)slot * d;
    __nv_bfloat16* dst = dqkv + t * L.ld + (long long)slot * d;
    const __nv_bfloat16* gsrc = kind == 0 ? dq + (t * nq + head) * d
                                : kind == 1 ? (dgate ? dgate + (t * nq + head) * d : nullptr)
                                : kind == 2 ? dk + (t * L.ng + head) * d
                                            : dv + (t * L.ng + head) * d;
    if (kind == 1 || kind == 3 || (!L.norm && L.rot == 0)) {
      for (int i = lane * 8; i < d; i += 256)
        *reinterpret_cast<uint4*>(dst + i) = gsrc ? *reinterpret_cast<const uint4*>(gsrc + i) : make_uint4(0, 0, 0, 0);
      continue;
    }
    float ss = 0.f;
    for (int i = lane * 2; i < d; i += 64) {
      float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + i));
      float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gsrc + i));
      sx[warp][i] = f.x;
      sx[warp][i + 1] = f.y;
      sg[warp][i] = g.x;
      sg[warp][i + 1] = g.y;
      ss += f.x * f.x + f.y * f.y;
    }
    float rstd = 1.f;
    if (L.norm) {
      ss = warp_sum(ss);
      rstd = rsqrtf(ss / d + L.eps);
    }
    __syncwarp();
    const __nv_bfloat16* wn = kind == 0 ? wq : wk;
    // pass 1: gradient w.r.t. the normalised (pre-rotation) head, dot product for the norm backward
    float gn[MAX_D / 32];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_D / 64; ++j) {
      const int i = lane * 2 + j * 64;
      if (i < d) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int idx = i + e;
          float g = sg[warp][idx];
          if (idx < L.rot) {
            int partner, fi;
            float sign;  // transpose of the forward rotation
            if (L.interleaved) {
              partner = idx ^ 1;
              fi = idx >> 1;
              sign = (idx & 1) ? -1.f : 1.f;
            } else {
              partner = idx < half ? idx + half : idx - half;
              fi = idx < half ? idx : idx - half;
              sign = idx < half ? 1.f : -1.f;
            }
            const float c = cosb[t * half + fi], s = sinb[t * half + fi];
            g = g * c + sign * sg[warp][partner] * s;
          }
          gn[2 * j + e] = g;
          if (L.norm) {
            const float wv = (L.zero_centered ? 1.f : 0.f) + __bfloat162float(wn[idx]);
            dot += g * wv * sx[warp][idx];
          }
        }
      }
    }
    float c3 = 0.f;
    if (L.norm) {
      dot = warp_sum(dot);
      c3 = dot * rstd * rstd * rstd / d;
    }
#pragma unroll
    for (int j = 0; j < MAX_D / 64; ++j) {
      const int i = lane * 2 + j * 64;
      if (i < d) {
        float o[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int idx = i + e;
          const float g = gn[2 * j + e];
          if (L.norm) {
            const float wv = (L.zero_centered ? 1.f : 0.f) + __bfloat162float(wn[idx]);
            o[e] = g * wv * rstd - sx[warp][idx] * c3;
            const float contrib = g * sx[warp][idx] * rstd;
            if (kind == 0) dw_acc[0][2 * j + e] += contrib; else dw_acc[1][2 * j + e] += contrib;
          } else {
            o[e] = g;
          }
        }
        *reinterpret_cast<uint32_t*>(dst + i) = pack_bf16x2(o[0], o[1]);
      }
    }
    __syncwarp();
  }
  if (L.norm) {
#pragma unroll
    for (int j = 0; j < MAX_D / 64; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int idx = lane * 2 + j * 64 + e;
        if (idx < d) {
          atomicAdd(&sdw[0][idx], dw_acc[0][2 * j + e]);
          atomicAdd(&sdw[1][idx], dw_acc[1][2 * j + e]);
        }
      }
  }
  __syncthreads();
  if (L.norm) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      if (dwq) atomicAdd(dwq + i, sdw[0][i]);
      if (dwk) atomicAdd(dwk + i, sdw[1][i]);
    }
  }
}

}  // namespace

extern "C" {

int mcb_qkv_split_norm_rope_fwd(const void* qkv, const void* wq, const void* wk, const float* cosb, const float* sinb,
                                void* q, void* k, void* v, void* gate, long long T, int ng, int qpg, int d,
                                int has_gate, int rot, int interleaved, int norm, int zero_centered, float eps,
                                long long ld, void* stream_) {
  if (T == 0) return 0;
  if (d > MAX_D || d % 8 || rot > d || (rot & 1) || ld % 8) return -1;
  QkvLayout L{ng, qpg, d, has_gate, rot, interleaved, norm, zero_centered, eps, ld};
  long long blocks = T;
  long long cap = (long long)device_sm_count() * 16;
  qkv_fwd_kernel<<<(int)(blocks < cap ? blocks : cap), WARPS * 32, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk, cosb, sinb, (__nv_bfloat16*)q,
      (__nv_bfloat16*)k, (__nv_bfloat16*)v, (__nv_bfloat16*)gate, T, L);
  return (int)cudaGetLastError();
}

// dwq / dwk: fp32 [d], accumulated into (caller zeroes or carries them across micro-batches)
int mcb_qkv_split_norm_rope_bwd(const void* qkv, const void* wq, const void* wk, const float* cosb, const float* sinb,
                                const void* dq, const void* dk, const void* dv, const void* dgate, void* dqkv,
                                float* dwq, float* dwk, long long T, int ng, int qpg, int d, int has_gate, int rot,
                                int interleaved, int norm, int zero_centered, float eps, long long ld, void* stream_) {
  if (T == 0) return 0;
  if (d > MAX_D || d % 8 || rot > d || (rot & 1) || ld % 8) return -1;
  QkvLayout L{ng, qpg, d, has_gate, rot, interleaved, norm, zero_centered, eps, ld};
  long long blocks = T;
  long long cap = (long long)device_sm_count() * 8;
  qkv_bwd_kernel<<<(int)(blocks < cap ? blocks : cap), WARPS * 32, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk, cosb, sinb,
      (const __nv_bfloat16*)dq, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)dv, (const __nv_bfloat16*)dgate,
      (__nv_bfloat16*)dqkv, dwq, dwk, T, L);
  return (int)cudaGetLastError();
}

}  // extern "C"

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
#include "../common/partials.cuh"
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
               __nv_bfloat16* __restrict__ dqkv, float* __restrict__ dwq, float* __restrict__ dwk,
               float* __restrict__ partials, long long T,
               QkvLayout L) {
  __shared__ float sx[WARPS][MAX_D];   // raw input head
  __shared__ float sg[WARPS][MAX_D];   // gradient after inverse rotation
  __shared__ float sdw[WARPS][2][MAX_D];   // one slot per warp: summed in warp order below, no atomics
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slots = L.ng * (L.qpg * (1 + L.gate) + 2);
  const int nq = L.ng * L.qpg, d = L.d, half = L.rot / 2;
  for (int i = threadIdx.x; i < WARPS * 2 * MAX_D; i += blockDim.x) (&sdw[0][0][0])[i] = 0.f;
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
          sdw[warp][0][idx] = dw_acc[0][2 * j + e];
          sdw[warp][1][idx] = dw_acc[1][2 * j + e];
        }
      }
  }
  __syncthreads();
  if (L.norm) {
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      float a = 0.f, b = 0.f;
      for (int w = 0; w < WARPS; ++w) {
        a += sdw[w][0][i];
        b += sdw[w][1][i];
      }
      if (partials) {                       // fixed-order sum over CTAs in qkv_dw_reduce_kernel
        partials[((long long)blockIdx.x * 2) * d + i] = a;
        partials[((long long)blockIdx.x * 2 + 1) * d + i] = b;
      } else {
        if (dwq) atomicAdd(dwq + i, a);
        if (dwk) atomicAdd(dwk + i, b);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// Fast path for head size 128 with rotate-half RoPE over the whole head (the Qwen3 / Llama layout): a lane holds
// elements {2l, 2l+1} and their rotation partners {64+2l, 65+2l}, so the head never leaves registers.
__device__ __forceinline__ float2 ld_bf2(const __nv_bfloat16* p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

__global__ void __launch_bounds__(WARPS * 32)
qkv_fwd_fast_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ wq,
                    const __nv_bfloat16* __restrict__ wk, const float* __restrict__ cosb,
                    const float* __restrict__ sinb, __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                    __nv_bfloat16* __restrict__ v, __nv_bfloat16* __restrict__ gate, long long T, QkvLayout L) {
  constexpr int D = 128;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slots = L.ng * (L.qpg * (1 + L.gate) + 2);
  const int nq = L.ng * L.qpg;
  const float wbase = L.zero_centered ? 1.f : 0.f;
  float2 wqa = make_float2(1.f, 1.f), wqb = wqa, wka = wqa, wkb = wqa;
  if (L.norm) {
    wqa = ld_bf2(wq + 2 * lane); wqb = ld_bf2(wq + 64 + 2 * lane);
    wka = ld_bf2(wk + 2 * lane); wkb = ld_bf2(wk + 64 + 2 * lane);
    wqa.x += wbase; wqa.y += wbase; wqb.x += wbase; wqb.y += wbase;
    wka.x += wbase; wka.y += wbase; wkb.x += wbase; wkb.y += wbase;
  }
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    const float2 c = *reinterpret_cast<const float2*>(cosb + t * 64 + 2 * lane);
    const float2 sn = *reinterpret_cast<const float2*>(sinb + t * 64 + 2 * lane);
    for (int slot = warp; slot < slots; slot += WARPS) {
      int kind, head;
      decode_slot(L, slot, kind, head);
      const __nv_bfloat16* src = qkv + t * L.ld + (long long)slot * D;
      __nv_bfloat16* dst = kind == 0 ? q + (t * nq + head) * D
                           : kind == 1 ? gate + (t * nq + head) * D
                           : kind == 2 ? k + (t * L.ng + head) * D
                                       : v + (t * L.ng + head) * D;
      if (kind == 1 || kind == 3) {
        *reinterpret_cast<uint2*>(dst + 4 * lane) = *reinterpret_cast<const uint2*>(src + 4 * lane);
        continue;
      }
      float2 a = ld_bf2(src + 2 * lane), b = ld_bf2(src + 64 + 2 * lane);
      if (L.norm) {
        const float ss = warp_sum(a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y);
        const float rstd = rsqrtf(ss * (1.f / D) + L.eps);
        const float2 wa = kind == 0 ? wqa : wka, wb = kind == 0 ? wqb : wkb;
        a.x *= rstd * wa.x; a.y *= rstd * wa.y; b.x *= rstd * wb.x; b.y *= rstd * wb.y;
      }
      *reinterpret_cast<uint32_t*>(dst + 2 * lane) = pack_bf16x2(a.x * c.x - b.x * sn.x, a.y * c.y - b.y * sn.y);
      *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = pack_bf16x2(b.x * c.x + a.x * sn.x, b.y * c.y + a.y * sn.y);
    }
  }
}

__global__ void __launch_bounds__(WARPS * 32)
qkv_bwd_fast_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ wq,
                    const __nv_bfloat16* __restrict__ wk, const float* __restrict__ cosb,
                    const float* __restrict__ sinb, const __nv_bfloat16* __restrict__ dq,
                    const __nv_bfloat16* __restrict__ dk, const __nv_bfloat16* __restrict__ dv,
                    const __nv_bfloat16* __restrict__ dgate, __nv_bfloat16* __restrict__ dqkv,
                    float* __restrict__ dwq, float* __restrict__ dwk, float* __restrict__ partials, long long T,
                    QkvLayout L) {
  constexpr int D = 128;
  __shared__ float sdw[WARPS][2][D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slots = L.ng * (L.qpg * (1 + L.gate) + 2);
  const int nq = L.ng * L.qpg;
  for (int i = threadIdx.x; i < WARPS * 2 * D; i += blockDim.x) (&sdw[0][0][0])[i] = 0.f;
  __syncthreads();
  const float wbase = L.zero_centered ? 1.f : 0.f;
  float2 wqa = make_float2(1.f, 1.f), wqb = wqa, wka = wqa, wkb = wqa;
  if (L.norm) {
    wqa = ld_bf2(wq + 2 * lane); wqb = ld_bf2(wq + 64 + 2 * lane);
    wka = ld_bf2(wk + 2 * lane); wkb = ld_bf2(wk + 64 + 2 * lane);
    wqa.x += wbase; wqa.y += wbase; wqb.x += wbase; wqb.y += wbase;
    wka.x += wbase; wka.y += wbase; wkb.x += wbase; wkb.y += wbase;
  }
  float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    const float2 c = *reinterpret_cast<const float2*>(cosb + t * 64 + 2 * lane);
    const float2 sn = *reinterpret_cast<const float2*>(sinb + t * 64 + 2 * lane);
    for (int slot = warp; slot < slots; slot += WARPS) {
      int kind, head;
      decode_slot(L, slot, kind, head);
      const __nv_bfloat16* src = qkv + t * L.ld + (long long)slot * D;
      __nv_bfloat16* dst = dqkv + t * L.ld + (long long)slot * D;
      const __nv_bfloat16* gsrc = kind == 0 ? dq + (t * nq + head) * D
                                  : kind == 1 ? (dgate ? dgate + (t * nq + head) * D : nullptr)
                                  : kind == 2 ? dk + (t * L.ng + head) * D
                                              : dv + (t * L.ng + head) * D;
      if (kind == 1 || kind == 3) {
        *reinterpret_cast<uint2*>(dst + 4 * lane) =
            gsrc ? *reinterpret_cast<const uint2*>(gsrc + 4 * lane) : make_uint2(0, 0);
        continue;
      }
      const float2 ga = ld_bf2(gsrc + 2 * lane), gb = ld_bf2(gsrc + 64 + 2 * lane);
      // transpose of the rotation
      float2 na = make_float2(ga.x * c.x + gb.x * sn.x, ga.y * c.y + gb.y * sn.y);
      float2 nb = make_float2(gb.x * c.x - ga.x * sn.x, gb.y * c.y - ga.y * sn.y);
      if (L.norm) {
        const float2 xa = ld_bf2(src + 2 * lane), xb = ld_bf2(src + 64 + 2 * lane);
        const float2 wa = kind == 0 ? wqa : wka, wb = kind == 0 ? wqb : wkb;
        float ss = xa.x * xa.x + xa.y * xa.y + xb.x * xb.x + xb.y * xb.y;
        float dot = na.x * wa.x * xa.x + na.y * wa.y * xa.y + nb.x * wb.x * xb.x + nb.y * wb.y * xb.y;
        ss = warp_sum(ss);
        dot = warp_sum(dot);
        const float rstd = rsqrtf(ss * (1.f / D) + L.eps);
        const float c3 = dot * rstd * rstd * rstd * (1.f / D);
        const float d0 = na.x * xa.x * rstd, d1 = na.y * xa.y * rstd, d2 = nb.x * xb.x * rstd, d3 = nb.y * xb.y * rstd;
        if (kind == 0) { acc[0][0] += d0; acc[0][1] += d1; acc[0][2] += d2; acc[0][3] += d3; }
        else { acc[1][0] += d0; acc[1][1] += d1; acc[1][2] += d2; acc[1][3] += d3; }
        na.x = na.x * wa.x * rstd - xa.x * c3; na.y = na.y * wa.y * rstd - xa.y * c3;
        nb.x = nb.x * wb.x * rstd - xb.x * c3; nb.y = nb.y * wb.y * rstd - xb.y * c3;
      }
      *reinterpret_cast<uint32_t*>(dst + 2 * lane) = pack_bf16x2(na.x, na.y);
      *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = pack_bf16x2(nb.x, nb.y);
    }
  }
  if (L.norm) {
#pragma unroll
    for (int a = 0; a < 2; ++a) {
      sdw[warp][a][2 * lane] = acc[a][0];
      sdw[warp][a][2 * lane + 1] = acc[a][1];
      sdw[warp][a][64 + 2 * lane] = acc[a][2];
      sdw[warp][a][65 + 2 * lane] = acc[a][3];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      float a = 0.f, b = 0.f;
      for (int w = 0; w < WARPS; ++w) {
        a += sdw[w][0][i];
        b += sdw[w][1][i];
      }
      if (partials) {
        partials[((long long)blockIdx.x * 2) * D + i] = a;
        partials[((long long)blockIdx.x * 2 + 1) * D + i] = b;
      } else {
        if (dwq) atomicAdd(dwq + i, a);
        if (dwk) atomicAdd(dwk + i, b);
      }
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
  if (d == 128 && rot == 128 && !interleaved) {
    qkv_fwd_fast_kernel<<<(int)(blocks < cap ? blocks : cap), WARPS * 32, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
        (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk, cosb, sinb, (__nv_bfloat16*)q,
        (__nv_bfloat16*)k, (__nv_bfloat16*)v, (__nv_bfloat16*)gate, T, L);
    return (int)cudaGetLastError();
  }
  qkv_fwd_kernel<<<(int)(blocks < cap ? blocks : cap), WARPS * 32, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk, cosb, sinb, (__nv_bfloat16*)q,
      (__nv_bfloat16*)k, (__nv_bfloat16*)v, (__nv_bfloat16*)gate, T, L);
  return (int)cudaGetLastError();
}

// CTAs the backward kernels launch for T tokens = rows of `partials` ([rows, 2, d] fp32) the caller provides
int mcb_qkv_bwd_partial_rows(long long T) {
  const long long cap = (long long)device_sm_count() * 8;
  return (int)(T < cap ? T : cap);
}

// dwq / dwk: fp32 [d], accumulated into (caller zeroes or carries them across micro-batches).  With `partials` the
// norm-weight gradients are summed in a fixed order (bit-reproducible); without, with atomics.
int mcb_qkv_split_norm_rope_bwd(const void* qkv, const void* wq, const void* wk, const float* cosb, const float* sinb,
                                const void* dq, const void* dk, const void* dv, const void* dgate, void* dqkv,
                                float* dwq, float* dwk, float* partials, long long T, int ng, int qpg, int d, int has_gate,
                                int rot, int interleaved, int norm, int zero_centered, float eps, long long ld,
                                void* stream_) {
  if (T == 0) return 0;
  if (d > MAX_D || d % 8 || rot > d || (rot & 1) || ld % 8) return -1;
  QkvLayout L{ng, qpg, d, has_gate, rot, interleaved, norm, zero_centered, eps, ld};
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const int grid = mcb_qkv_bwd_partial_rows(T);
  if (!norm) partials = nullptr;
  if (d == 128 && rot == 128 && !interleaved) {
    qkv_bwd_fast_kernel<<<grid, WARPS * 32, 0, s>>>(
        (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk, cosb, sinb,
        (const __nv_bfloat16*)dq, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)dv, (const __nv_bfloat16*)dgate,
        (__nv_bfloat16*)dqkv, dwq, dwk, partials, T, L);
  } else {
    qkv_bwd_kernel<<<grid, WARPS * 32, 0, s>>>(
        (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wk, cosb, sinb,
        (const __nv_bfloat16*)dq, (const __nv_bfloat16*)dk, (const __nv_bfloat16*)dv, (const __nv_bfloat16*)dgate,
        (__nv_bfloat16*)dqkv, dwq, dwk, partials, T, L);
  }
  if (partials) launch_reduce_partials(partials, grid, 2 * d, dwq, dwk, d, s);   // rows are [dwq | dwk]
  return (int)cudaGetLastError();
}

}  // extern "C"

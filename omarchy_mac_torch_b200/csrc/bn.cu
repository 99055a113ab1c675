// BatchNorm2d kernels: batch statistics, normalise(+ReLU), eval, backward(+ReLU mask). All are HBM-bound: every
// kernel reads its activations once with 128-bit accesses where the layout allows and reduces with warp shuffles.
//
// Behaviour follows the reference's BN shaders: shifted one-pass statistics (bn_stats_part.wgsl:22-31,
// bn_stats_fin.wgsl:15-21), running-stat update with the unbiased correction count/(count-1) (csrc/nn.cpp:44),
// apply/ReLU (bn_apply.wgsl, bn_relu.wgsl, bn_relu_rv.wgsl), backward (bnb_reduce.wgsl, bnb_apply.wgsl) and the
// ReLU-masked backward (bn_bwd_part.wgsl:25-38, bn_bwd_apply.wgsl:19-23). Two layouts: NCHW-contiguous (the
// reference's) and channels-last.
#include <algorithm>

#include "common.cuh"

namespace omt {

// ---------------------------------------------------------------------------------------------------------------
// ReLU bit mask. The forward pass can leave, behind y, one bit per element in memory order: word k, bit b = (y[32k + b] > 0).
// The backward passes then read 1/8 byte per element for the mask instead of 4 (they use nothing else of y).
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t mask_nibble(const uint32_t* __restrict__ bits, int64_t e) {  // elements e..e+3, e % 4 == 0
  return (__ldg(bits + (e >> 5)) >> (uint32_t)(e & 31)) & 0xFu;
}
__device__ __forceinline__ bool mask_bit(const uint32_t* __restrict__ bits, int64_t e) { return (__ldg(bits + (e >> 5)) >> (uint32_t)(e & 31)) & 1u; }

// ---------------------------------------------------------------------------------------------------------------
// partial sums. part layout: [c][S][2]
// ---------------------------------------------------------------------------------------------------------------

// NCHW: block (channel, slice); slice sl takes images sl, sl+S, ...
// MODE 0: stats of x (shifted by x[0,ch,0,0]); MODE 1: backward sums (sum g, sum g*xhat), g masked by y>0 if RELU.
template <int MODE, bool RELU>
__global__ void __launch_bounds__(256) bn_part_nchw(const float* __restrict__ x, const float* __restrict__ g,
                                                    const float* __restrict__ y, const uint32_t* __restrict__ bits,
                                                    const float* __restrict__ mean, const float* __restrict__ invstd, int n, int c, int hw, int S,
                                                    float* __restrict__ part) {
  __shared__ float red[32];
  const int ch = blockIdx.x, sl = blockIdx.y;
  float a0, a1;
  if (MODE == 0) { a0 = __ldg(x + (int64_t)ch * hw); a1 = 0.f; }
  else { a0 = __ldg(mean + ch); a1 = __ldg(invstd + ch); }
  float s1 = 0.f, s2 = 0.f;
  const bool vec = (hw & 3) == 0;
  for (int img = sl; img < n; img += S) {
    const int64_t base = ((int64_t)img * c + ch) * hw;
    if (vec) {
      const float4* x4 = reinterpret_cast<const float4*>(x + base);
      const float4* g4 = reinterpret_cast<const float4*>(g + base);
      const float4* y4 = reinterpret_cast<const float4*>(y + base);
      for (int e = threadIdx.x; e < hw / 4; e += blockDim.x) {
        float4 xv = __ldg(x4 + e);
        if (MODE == 0) {
          float d0 = xv.x - a0, d1 = xv.y - a0, d2 = xv.z - a0, d3 = xv.w - a0;
          s1 += (d0 + d1) + (d2 + d3);
          s2 += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
        } else {
          float4 gv = __ldg(g4 + e);
          if (RELU) {
            if (bits) {
              const uint32_t m = mask_nibble(bits, base + 4 * (int64_t)e);
              gv.x = (m & 1u) ? gv.x : 0.f; gv.y = (m & 2u) ? gv.y : 0.f; gv.z = (m & 4u) ? gv.z : 0.f; gv.w = (m & 8u) ? gv.w : 0.f;
            } else {
              float4 yv = __ldg(y4 + e);
              gv.x = yv.x > 0.f ? gv.x : 0.f; gv.y = yv.y > 0.f ? gv.y : 0.f;
              gv.z = yv.z > 0.f ? gv.z : 0.f; gv.w = yv.w > 0.f ? gv.w : 0.f;
            }
          }
          s1 += (gv.x + gv.y) + (gv.z + gv.w);
          s2 += (gv.x * (xv.x - a0) + gv.y * (xv.y - a0) + gv.z * (xv.z - a0) + gv.w * (xv.w - a0)) * a1;
        }
      }
    } else {
      for (int e = threadIdx.x; e < hw; e += blockDim.x) {
        float xv = __ldg(x + base + e);
        if (MODE == 0) {
          float d = xv - a0;
          s1 += d; s2 += d * d;
        } else {
          float gv = __ldg(g + base + e);
          if (RELU) gv = (bits ? mask_bit(bits, base + e) : __ldg(y + base + e) > 0.f) ? gv : 0.f;
          s1 += gv; s2 += gv * (xv - a0) * a1;
        }
      }
    }
  }
  s1 = block_sum(s1, red);
  s2 = block_sum(s2, red);
  if (threadIdx.x == 0) {
    part[((int64_t)ch * S + sl) * 2] = s1;
    part[((int64_t)ch * S + sl) * 2 + 1] = s2;
  }
}

// NHWC: x is [P pixels][c]. Block = CX channel groups of 4 x PY pixel lanes; slice sl takes pixels sl*PY+py, +S*PY ...
template <int MODE, bool RELU>
__global__ void __launch_bounds__(256) bn_part_nhwc(const float* __restrict__ x, const float* __restrict__ g,
                                                    const float* __restrict__ y, const uint32_t* __restrict__ bits,
                                                    const float* __restrict__ mean, const float* __restrict__ invstd, int64_t P, int c, int S, int CX,
                                                    float* __restrict__ part) {
  __shared__ float4 sh1[256], sh2[256];
  const int cx = threadIdx.x % CX, py = threadIdx.x / CX, PY = blockDim.x / CX;
  const int c4 = (blockIdx.x * CX + cx) * 4, sl = blockIdx.y;
  float4 s1 = make_float4(0, 0, 0, 0), s2 = s1;
  if (c4 < c) {
    float4 a0, a1 = make_float4(0, 0, 0, 0);
    if (MODE == 0) a0 = __ldg(reinterpret_cast<const float4*>(x + c4));
    else { a0 = __ldg(reinterpret_cast<const float4*>(mean + c4)); a1 = __ldg(reinterpret_cast<const float4*>(invstd + c4)); }
    int64_t p = (int64_t)sl * PY + py;
    if (MODE == 0) {
      // four independent loads per trip keep enough bytes in flight at 50 % occupancy; same summation order every run
      const int64_t step = (int64_t)S * PY;
      for (; p + 3 * step < P; p += 4 * step) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) v[u] = __ldg(reinterpret_cast<const float4*>(x + (p + u * step) * c + c4));
#pragma unroll
        for (int u = 0; u < 4; u++) {
          float d0 = v[u].x - a0.x, d1 = v[u].y - a0.y, d2 = v[u].z - a0.z, d3 = v[u].w - a0.w;
          s1.x += d0; s1.y += d1; s1.z += d2; s1.w += d3;
          s2.x += d0 * d0; s2.y += d1 * d1; s2.z += d2 * d2; s2.w += d3 * d3;
        }
      }
    }
    for (; p < P; p += (int64_t)S * PY) {
      float4 xv = __ldg(reinterpret_cast<const float4*>(x + p * c + c4));
      if (MODE == 0) {
        float d0 = xv.x - a0.x, d1 = xv.y - a0.y, d2 = xv.z - a0.z, d3 = xv.w - a0.w;
        s1.x += d0; s1.y += d1; s1.z += d2; s1.w += d3;
        s2.x += d0 * d0; s2.y += d1 * d1; s2.z += d2 * d2; s2.w += d3 * d3;
      } else {
        float4 gv = __ldg(reinterpret_cast<const float4*>(g + p * c + c4));
        if (RELU) {
          if (bits) {
            const uint32_t m = mask_nibble(bits, p * c + c4);
            gv.x = (m & 1u) ? gv.x : 0.f; gv.y = (m & 2u) ? gv.y : 0.f; gv.z = (m & 4u) ? gv.z : 0.f; gv.w = (m & 8u) ? gv.w : 0.f;
          } else {
            float4 yv = __ldg(reinterpret_cast<const float4*>(y + p * c + c4));
            gv.x = yv.x > 0.f ? gv.x : 0.f; gv.y = yv.y > 0.f ? gv.y : 0.f;
            gv.z = yv.z > 0.f ? gv.z : 0.f; gv.w = yv.w > 0.f ? gv.w : 0.f;
          }
        }
        s1.x += gv.x; s1.y += gv.y; s1.z += gv.z; s1.w += gv.w;
        s2.x += gv.x * (xv.x - a0.x) * a1.x; s2.y += gv.y * (xv.y - a0.y) * a1.y;
        s2.z += gv.z * (xv.z - a0.z) * a1.z; s2.w += gv.w * (xv.w - a0.w) * a1.w;
      }
    }
  }
  sh1[threadIdx.x] = s1; sh2[threadIdx.x] = s2;
  __syncthreads();
  if (py == 0 && c4 < c) {
    for (int q = 1; q < PY; q++) {
      float4 u = sh1[q * CX + cx], v = sh2[q * CX + cx];
      s1.x += u.x; s1.y += u.y; s1.z += u.z; s1.w += u.w;
      s2.x += v.x; s2.y += v.y; s2.z += v.z; s2.w += v.w;
    }
    const float a[4] = {s1.x, s1.y, s1.z, s1.w}, b[4] = {s2.x, s2.y, s2.z, s2.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      part[((int64_t)(c4 + j) * S + sl) * 2] = a[j];
      part[((int64_t)(c4 + j) * S + sl) * 2 + 1] = b[j];
    }
  }
}

// finalise statistics: one warp per channel sums the S partial pairs (contiguous in memory), lane 0 writes.
// shift_stride = distance between channels' first elements.
__global__ void __launch_bounds__(256) bn_stats_fin(const float* __restrict__ x, int64_t shift_stride, const float* __restrict__ part, int c, int S,
                                                    float count, float corr, float momentum, float eps, float* mean, float* var, float* invstd,
                                                    const float* rm_in, const float* rv_in, float* rm_out, float* rv_out) {
  const int ch = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (ch >= c) return;
  float s1 = 0.f, s2 = 0.f;
  const float2* p = reinterpret_cast<const float2*>(part) + (int64_t)ch * S;
  for (int k = lane; k < S; k += 32) {
    float2 v = __ldg(p + k);
    s1 += v.x; s2 += v.y;
  }
  s1 = warp_sum(s1); s2 = warp_sum(s2);
  if (lane) return;
  float a = s1 / count, shift = x ? x[ch * shift_stride] : 0.f;
  float m = shift + a, v = fmaxf(s2 / count - a * a, 0.f);
  if (mean) mean[ch] = m;
  if (var) var[ch] = v;
  if (invstd) invstd[ch] = rsqrtf(v + eps);
  if (rm_out) {
    float r0 = rm_in[ch], r1 = rv_in[ch];
    rm_out[ch] = r0 + momentum * (m - r0);
    rv_out[ch] = r1 + momentum * (v * corr - r1);
  }
}
// finalise backward sums: dgb[0][c] = dgamma (s2), dgb[1][c] = dbeta (s1)   (bn_bwd_fin.wgsl)
__global__ void __launch_bounds__(256) bn_bwd_fin(const float* __restrict__ part, int c, int S, float scale, float* dgb, float* raw) {
  const int ch = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (ch >= c) return;
  float s1 = 0.f, s2 = 0.f;
  const float2* p = reinterpret_cast<const float2*>(part) + (int64_t)ch * S;
  for (int k = lane; k < S; k += 32) {
    float2 v = __ldg(p + k);
    s1 += v.x; s2 += v.y;
  }
  s1 = warp_sum(s1); s2 = warp_sum(s2);
  if (lane) return;
  raw[ch] = s2; raw[c + ch] = s1;  // unscaled, for the dx formula
  dgb[ch] = s2 * scale; dgb[c + ch] = s1 * scale;
}

// ---------------------------------------------------------------------------------------------------------------
// elementwise passes. KIND 0: y = (x-mean)*inv*gamma+beta (train; inv given) ; 1: eval (inv = rsqrt(rv+eps))
//                     KIND 2: dx = gamma*inv/m*(m*g - dbeta - xhat*dgamma)
// ---------------------------------------------------------------------------------------------------------------
struct BnEw {
  const float* x; const float* g; const float* y; float* out;
  const float* res;  // KIND 0/1: optional residual added before the ReLU (same layout as x)
  float* gz;         // KIND 2 with RELU: optional second output, the ReLU-masked incoming gradient
  uint32_t* bits_out;       // KIND 0 with RELU: optional ReLU bit mask of the output (one bit per element, memory order)
  const uint32_t* bits_in;  // KIND 2 with RELU: the mask comes from these bits instead of from y's values
  const float* mean; const float* inv; const float* gamma; const float* beta; const float* dgb;
  float eps, m;
  int c, hw;
  int64_t total;
};

// gv: KIND 2 the (already masked) incoming gradient; KIND 0/1 the residual value (0 without one)
template <int KIND, bool RELU>
__device__ __forceinline__ float bn_ew_one(const BnEw& a, float xv, float gv, float mean, float inv, float ga, float be, float dg, float db) {
  if (KIND <= 1) {
    float r = (xv - mean) * inv * ga + be + gv;
    return RELU ? fmaxf(r, 0.f) : r;
  } else {
    float xhat = (xv - mean) * inv;
    return ga * inv / a.m * (a.m * gv - db - xhat * dg);
  }
}

template <int KIND, bool RELU, bool NHWC>
__global__ void __launch_bounds__(256) bn_ew_vec4(BnEw a) {
  int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= a.total) return;  // (exited lanes of the last warp: the mask words below then carry unspecified bits past the end, which nobody reads)
  float4 xv = __ldg(reinterpret_cast<const float4*>(a.x + i)), gv = make_float4(0.f, 0.f, 0.f, 0.f), o;
  if (KIND == 2) {
    gv = __ldg(reinterpret_cast<const float4*>(a.g + i));
    if (RELU) {
      if (a.bits_in) {
        const uint32_t m = mask_nibble(a.bits_in, i);
        gv.x = (m & 1u) ? gv.x : 0.f; gv.y = (m & 2u) ? gv.y : 0.f; gv.z = (m & 4u) ? gv.z : 0.f; gv.w = (m & 8u) ? gv.w : 0.f;
      } else {
        const float4 yv = __ldg(reinterpret_cast<const float4*>(a.y + i));
        gv.x = yv.x > 0.f ? gv.x : 0.f; gv.y = yv.y > 0.f ? gv.y : 0.f; gv.z = yv.z > 0.f ? gv.z : 0.f; gv.w = yv.w > 0.f ? gv.w : 0.f;
      }
      if (a.gz) *reinterpret_cast<float4*>(a.gz + i) = gv;
    }
  } else if (a.res) {
    gv = __ldg(reinterpret_cast<const float4*>(a.res + i));
  }
  if (NHWC) {
    int ch = a.total < 0x7fffffffll ? (int)((uint32_t)i % (uint32_t)a.c) : (int)(i % a.c);
    float4 mean = __ldg(reinterpret_cast<const float4*>(a.mean + ch)), inv = __ldg(reinterpret_cast<const float4*>(a.inv + ch));
    float4 ga = __ldg(reinterpret_cast<const float4*>(a.gamma + ch));
    float4 be = ga, dg = ga, db = ga;
    if (KIND <= 1) be = __ldg(reinterpret_cast<const float4*>(a.beta + ch));
    if (KIND == 1) { inv.x = rsqrtf(inv.x + a.eps); inv.y = rsqrtf(inv.y + a.eps); inv.z = rsqrtf(inv.z + a.eps); inv.w = rsqrtf(inv.w + a.eps); }
    if (KIND == 2) { dg = __ldg(reinterpret_cast<const float4*>(a.dgb + ch)); db = __ldg(reinterpret_cast<const float4*>(a.dgb + a.c + ch)); }
    o.x = bn_ew_one<KIND, RELU>(a, xv.x, gv.x, mean.x, inv.x, ga.x, be.x, dg.x, db.x);
    o.y = bn_ew_one<KIND, RELU>(a, xv.y, gv.y, mean.y, inv.y, ga.y, be.y, dg.y, db.y);
    o.z = bn_ew_one<KIND, RELU>(a, xv.z, gv.z, mean.z, inv.z, ga.z, be.z, dg.z, db.z);
    o.w = bn_ew_one<KIND, RELU>(a, xv.w, gv.w, mean.w, inv.w, ga.w, be.w, dg.w, db.w);
  } else {
    int ch = a.total < 0x7fffffffll ? (int)(((uint32_t)i / (uint32_t)a.hw) % (uint32_t)a.c) : (int)((i / a.hw) % a.c);
    float mean = __ldg(a.mean + ch), inv = __ldg(a.inv + ch), ga = __ldg(a.gamma + ch), be = 0.f, dg = 0.f, db = 0.f;
    if (KIND <= 1) be = __ldg(a.beta + ch);
    if (KIND == 1) inv = rsqrtf(inv + a.eps);
    if (KIND == 2) { dg = __ldg(a.dgb + ch); db = __ldg(a.dgb + a.c + ch); }
    o.x = bn_ew_one<KIND, RELU>(a, xv.x, gv.x, mean, inv, ga, be, dg, db);
    o.y = bn_ew_one<KIND, RELU>(a, xv.y, gv.y, mean, inv, ga, be, dg, db);
    o.z = bn_ew_one<KIND, RELU>(a, xv.z, gv.z, mean, inv, ga, be, dg, db);
    o.w = bn_ew_one<KIND, RELU>(a, xv.w, gv.w, mean, inv, ga, be, dg, db);
  }
  *reinterpret_cast<float4*>(a.out + i) = o;
  if (KIND == 0 && RELU && a.bits_out) {  // 8 lanes x 4 elements make one word; lane 0 of each group of 8 stores it
    const int lane = threadIdx.x & 31;
    uint32_t v = ((o.x > 0.f ? 1u : 0u) | (o.y > 0.f ? 2u : 0u) | (o.z > 0.f ? 4u : 0u) | (o.w > 0.f ? 8u : 0u)) << (4 * (lane & 7));
    v |= __shfl_xor_sync(0xffffffffu, v, 1); v |= __shfl_xor_sync(0xffffffffu, v, 2); v |= __shfl_xor_sync(0xffffffffu, v, 4);
    if ((lane & 7) == 0) a.bits_out[i >> 5] = v;
  }
}

// Channels-last with c % 32 == 0 and a pixel count divisible by 4: a thread takes its 4 channels of FOUR consecutive pixels,
// so the per-channel parameters (four to six 128-bit loads) are fetched once per 64 bytes of activation instead of once
// per 16, and four independent activation loads are in flight per thread. Same arithmetic as bn_ew_vec4.
template <int KIND, bool RELU>
__global__ void __launch_bounds__(256) bn_ew_nhwc_px4(BnEw a) {
  const int c4 = a.c >> 2;
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // t = pixel group * c4 + channel quad
  const int64_t pg = t < 0x7fffffffll ? (int64_t)((uint32_t)t / (uint32_t)c4) : t / c4;
  const int ch = (int)(t - pg * c4) * 4;
  const int64_t i0 = pg * 4 * a.c + ch;
  if (i0 >= a.total) return;  // (c4 % 8 == 0: the 8 lanes that share a mask word leave together)
  const float4 mean = __ldg(reinterpret_cast<const float4*>(a.mean + ch));
  float4 inv = __ldg(reinterpret_cast<const float4*>(a.inv + ch));
  const float4 ga = __ldg(reinterpret_cast<const float4*>(a.gamma + ch));
  float4 be = ga, dg = ga, db = ga;
  if (KIND <= 1) be = __ldg(reinterpret_cast<const float4*>(a.beta + ch));
  if (KIND == 1) { inv.x = rsqrtf(inv.x + a.eps); inv.y = rsqrtf(inv.y + a.eps); inv.z = rsqrtf(inv.z + a.eps); inv.w = rsqrtf(inv.w + a.eps); }
  if (KIND == 2) { dg = __ldg(reinterpret_cast<const float4*>(a.dgb + ch)); db = __ldg(reinterpret_cast<const float4*>(a.dgb + a.c + ch)); }
  float4 xv[4], gv[4];
  uint32_t mk[4] = {0xFu, 0xFu, 0xFu, 0xFu};
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const int64_t i = i0 + (int64_t)k * a.c;
    xv[k] = __ldg(reinterpret_cast<const float4*>(a.x + i));
    gv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (KIND == 2) {
      gv[k] = __ldg(reinterpret_cast<const float4*>(a.g + i));
      if (RELU) {
        if (a.bits_in) {
          mk[k] = mask_nibble(a.bits_in, i);
        } else {
          const float4 yv = __ldg(reinterpret_cast<const float4*>(a.y + i));
          mk[k] = (yv.x > 0.f ? 1u : 0u) | (yv.y > 0.f ? 2u : 0u) | (yv.z > 0.f ? 4u : 0u) | (yv.w > 0.f ? 8u : 0u);
        }
      }
    } else if (a.res) {
      gv[k] = __ldg(reinterpret_cast<const float4*>(a.res + i));
    }
  }
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const int64_t i = i0 + (int64_t)k * a.c;
    float4 g = gv[k], o;
    if (KIND == 2 && RELU) {
      g.x = (mk[k] & 1u) ? g.x : 0.f; g.y = (mk[k] & 2u) ? g.y : 0.f; g.z = (mk[k] & 4u) ? g.z : 0.f; g.w = (mk[k] & 8u) ? g.w : 0.f;
      if (a.gz) *reinterpret_cast<float4*>(a.gz + i) = g;
    }
    o.x = bn_ew_one<KIND, RELU>(a, xv[k].x, g.x, mean.x, inv.x, ga.x, be.x, dg.x, db.x);
    o.y = bn_ew_one<KIND, RELU>(a, xv[k].y, g.y, mean.y, inv.y, ga.y, be.y, dg.y, db.y);
    o.z = bn_ew_one<KIND, RELU>(a, xv[k].z, g.z, mean.z, inv.z, ga.z, be.z, dg.z, db.z);
    o.w = bn_ew_one<KIND, RELU>(a, xv[k].w, g.w, mean.w, inv.w, ga.w, be.w, dg.w, db.w);
    *reinterpret_cast<float4*>(a.out + i) = o;
    if (KIND == 0 && RELU && a.bits_out) {  // 8 lanes x 4 elements make one word; lane 0 of each group of 8 stores it
      uint32_t v = ((o.x > 0.f ? 1u : 0u) | (o.y > 0.f ? 2u : 0u) | (o.z > 0.f ? 4u : 0u) | (o.w > 0.f ? 8u : 0u)) << (4 * (lane & 7));
      v |= __shfl_xor_sync(0xffffffffu, v, 1); v |= __shfl_xor_sync(0xffffffffu, v, 2); v |= __shfl_xor_sync(0xffffffffu, v, 4);
      if ((lane & 7) == 0) a.bits_out[i >> 5] = v;
    }
  }
}

template <int KIND, bool RELU>
__global__ void __launch_bounds__(256) bn_ew_scalar(BnEw a, bool nhwc) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= a.total) return;
  int ch = nhwc ? (int)(i % a.c) : (int)((i / a.hw) % a.c);
  float xv = __ldg(a.x + i), gv = KIND == 2 ? __ldg(a.g + i) : (a.res ? __ldg(a.res + i) : 0.f);
  if (KIND == 2 && RELU) {
    if (!(a.bits_in ? mask_bit(a.bits_in, i) : __ldg(a.y + i) > 0.f)) gv = 0.f;
    if (a.gz) a.gz[i] = gv;
  }
  float inv = __ldg(a.inv + ch);
  if (KIND == 1) inv = rsqrtf(inv + a.eps);
  const float o = bn_ew_one<KIND, RELU>(a, xv, gv, __ldg(a.mean + ch), inv, __ldg(a.gamma + ch), KIND <= 1 ? __ldg(a.beta + ch) : 0.f,
                                        KIND == 2 ? __ldg(a.dgb + ch) : 0.f, KIND == 2 ? __ldg(a.dgb + a.c + ch) : 0.f);
  a.out[i] = o;
  if (KIND == 0 && RELU && a.bits_out) {  // a warp covers 32 consecutive elements starting at a multiple of 32: one word
    const uint32_t v = __ballot_sync(0xffffffffu, o > 0.f);
    if ((threadIdx.x & 31) == 0) a.bits_out[i >> 5] = v;
  }
}

template <int KIND>
static int launch_ew(const BnEw& a, bool relu, bool nhwc, cudaStream_t s, const char* name) {
  bool vec = nhwc ? (a.c % 4 == 0) : (a.hw % 4 == 0);
  vec = vec && ((reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.out) | reinterpret_cast<uintptr_t>(a.g) |
                 reinterpret_cast<uintptr_t>(a.y) | reinterpret_cast<uintptr_t>(a.res) | reinterpret_cast<uintptr_t>(a.gz)) & 15) == 0;
  if (nhwc)  // per-channel tables are read as float4 too
    vec = vec && ((reinterpret_cast<uintptr_t>(a.mean) | reinterpret_cast<uintptr_t>(a.inv) | reinterpret_cast<uintptr_t>(a.gamma) |
                   reinterpret_cast<uintptr_t>(a.beta) | reinterpret_cast<uintptr_t>(a.dgb)) & 15) == 0;
  if (vec && nhwc && a.c % 32 == 0 && (a.total / a.c) % 4 == 0) {
    const unsigned blocks = (unsigned)cdiv(a.total / 16, 256);
    if (relu) bn_ew_nhwc_px4<KIND, true><<<blocks, 256, 0, s>>>(a);
    else bn_ew_nhwc_px4<KIND, false><<<blocks, 256, 0, s>>>(a);
  } else if (vec) {
    unsigned blocks = (unsigned)cdiv(a.total / 4, 256);
    if (nhwc) {
      if (relu) bn_ew_vec4<KIND, true, true><<<blocks, 256, 0, s>>>(a);
      else bn_ew_vec4<KIND, false, true><<<blocks, 256, 0, s>>>(a);
    } else {
      if (relu) bn_ew_vec4<KIND, true, false><<<blocks, 256, 0, s>>>(a);
      else bn_ew_vec4<KIND, false, false><<<blocks, 256, 0, s>>>(a);
    }
  } else {
    unsigned blocks = (unsigned)cdiv(a.total, 256);
    if (relu) bn_ew_scalar<KIND, true><<<blocks, 256, 0, s>>>(a, nhwc);
    else bn_ew_scalar<KIND, false><<<blocks, 256, 0, s>>>(a, nhwc);
  }
  return check_launch(name);
}

// ---------------------------------------------------------------------------------------------------------------
// normalise (+ReLU) and 2x2 stride-2 max pool in one pass: x is read once; y (full resolution, what the backward masks
// with) is optional; z is the pooled output and idx in {0..3} = dy*2+dx of the first maximum (pool_fwd.wgsl:15-21).
// ---------------------------------------------------------------------------------------------------------------
struct BnPool {
  ActView x, y, z;
  uint8_t* idx;
  const float* mean; const float* inv; const float* gamma; const float* beta;
  int n, c, oh, ow;
  bool relu;
};
__device__ __forceinline__ void pool4(const float v[4], float& best, int& bi) {
  best = v[0]; bi = 0;
  if (v[1] > best) { best = v[1]; bi = 1; }
  if (v[2] > best) { best = v[2]; bi = 2; }
  if (v[3] > best) { best = v[3]; bi = 3; }
}
// channels-last, c % 4 == 0: one thread per output pixel and 4 channels
__global__ void __launch_bounds__(256) bn_pool2_nhwc4(BnPool a) {
  const int c4 = a.c >> 2;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.oh * a.ow * c4) return;
  const int ch = (int)(i % c4) * 4;
  int64_t r = i / c4;
  const int ox = (int)(r % a.ow); r /= a.ow;
  const int oy = (int)(r % a.oh), img = (int)(r / a.oh);
  const float4 mean = __ldg(reinterpret_cast<const float4*>(a.mean + ch)), inv = __ldg(reinterpret_cast<const float4*>(a.inv + ch));
  const float4 ga = __ldg(reinterpret_cast<const float4*>(a.gamma + ch)), be = __ldg(reinterpret_cast<const float4*>(a.beta + ch));
  const float iv[4] = {inv.x, inv.y, inv.z, inv.w}, gm[4] = {ga.x, ga.y, ga.z, ga.w}, mu[4] = {mean.x, mean.y, mean.z, mean.w}, bt[4] = {be.x, be.y, be.z, be.w};
  float v[4][4];  // [channel][window position]
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const int64_t off = a.x.off(img, ch, 2 * oy + (k >> 1), 2 * ox + (k & 1));
    const float4 xv = __ldg(reinterpret_cast<const float4*>(a.x.p + off));
    const float in[4] = {xv.x, xv.y, xv.z, xv.w};
    float o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      // same operation order as bn_ew_one: ((x - mean) * inv) * gamma + beta
      o[j] = (in[j] - mu[j]) * iv[j] * gm[j] + bt[j];
      if (a.relu) o[j] = fmaxf(o[j], 0.f);
      v[j][k] = o[j];
    }
    if (a.y.p) *reinterpret_cast<float4*>(a.y.p + a.y.off(img, ch, 2 * oy + (k >> 1), 2 * ox + (k & 1))) = make_float4(o[0], o[1], o[2], o[3]);
  }
  float best[4];
  int bi[4];
#pragma unroll
  for (int j = 0; j < 4; j++) pool4(v[j], best[j], bi[j]);
  const int64_t zo = a.z.off(img, ch, oy, ox);
  *reinterpret_cast<float4*>(a.z.p + zo) = make_float4(best[0], best[1], best[2], best[3]);
  if (a.idx) *reinterpret_cast<uchar4*>(a.idx + zo) = make_uchar4((uint8_t)bi[0], (uint8_t)bi[1], (uint8_t)bi[2], (uint8_t)bi[3]);
}
// any layout: one thread per output element, in the memory order of z
template <bool NHWC>
__global__ void __launch_bounds__(256) bn_pool2_scalar(BnPool a) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.c * a.oh * a.ow) return;
  int img, ch, oy, ox;
  if (NHWC) { ch = (int)(i % a.c); i /= a.c; ox = (int)(i % a.ow); i /= a.ow; oy = (int)(i % a.oh); img = (int)(i / a.oh); }
  else { ox = (int)(i % a.ow); i /= a.ow; oy = (int)(i % a.oh); i /= a.oh; ch = (int)(i % a.c); img = (int)(i / a.c); }
  const float mean = __ldg(a.mean + ch), inv = __ldg(a.inv + ch), ga = __ldg(a.gamma + ch), be = __ldg(a.beta + ch);
  float v[4];
#pragma unroll
  for (int k = 0; k < 4; k++) {
    float o = (__ldg(a.x.p + a.x.off(img, ch, 2 * oy + (k >> 1), 2 * ox + (k & 1))) - mean) * inv * ga + be;
    if (a.relu) o = fmaxf(o, 0.f);
    v[k] = o;
    if (a.y.p) a.y.p[a.y.off(img, ch, 2 * oy + (k >> 1), 2 * ox + (k & 1))] = o;
  }
  float best;
  int bi;
  pool4(v, best, bi);
  const int64_t zo = a.z.off(img, ch, oy, ox);
  a.z.p[zo] = best;
  if (a.idx) a.idx[zo] = (uint8_t)bi;
}

// layout of an activation: 0 NCHW contiguous, 1 NHWC contiguous, -1 neither
static int layout_of(const OmtAct* a, int c, int h, int w) {
  if (is_nchw(a, c, h, w)) return 0;
  if (is_nhwc(a, c, h, w)) return 1;
  return -1;
}

// partial-sum launch shared by forward statistics (MODE 0) and backward (MODE 1)
template <int MODE>
static int launch_part(int lay, const float* x, const float* g, const float* y, const uint32_t* bits, const float* mean, const float* invstd,
                       bool relu, int n, int c, int h, int w, int* S_out, float* part, cudaStream_t s) {
  const int hw = h * w;
  if (lay == 1 && c % 4 == 0) {
    int64_t P = (int64_t)n * hw;
    int CX = std::min(c / 4, 64);
    while (256 % CX) CX--;  // CX must divide the block
    int PY = 256 / CX, gx = (int)cdiv(c / 4, CX);
    int S = (int)std::max<int64_t>(1, std::min<int64_t>(cdiv(P, PY * 4), cdiv(4 * sm_count(), gx)));
    *S_out = S;
    dim3 grid(gx, S);
    if (relu) bn_part_nhwc<MODE, true><<<grid, 256, 0, s>>>(x, g, y, bits, mean, invstd, P, c, S, CX, part);
    else bn_part_nhwc<MODE, false><<<grid, 256, 0, s>>>(x, g, y, bits, mean, invstd, P, c, S, CX, part);
    return check_launch(MODE == 0 ? "bn_stats_part_nhwc" : "bn_bwd_part_nhwc");
  }
  // NCHW (also used for channels-last with c % 4 != 0 through the caller's layout check)
  int S = (int)std::max<int64_t>(1, std::min<int64_t>(n, cdiv(4 * sm_count(), c)));
  *S_out = S;
  dim3 grid(c, S);
  if (relu) bn_part_nchw<MODE, true><<<grid, 256, 0, s>>>(x, g, y, bits, mean, invstd, n, c, hw, S, part);
  else bn_part_nchw<MODE, false><<<grid, 256, 0, s>>>(x, g, y, bits, mean, invstd, n, c, hw, S, part);
  return check_launch(MODE == 0 ? "bn_stats_part_nchw" : "bn_bwd_part_nchw");
}

// Statistics from the per-group partials a conv epilogue wrote (OMT_EPI_BNSTATS): for each 32-row group g and channel the
// group's sum and the sum of squared deviations from the group's own mean, part[(2g + {0,1}) * c + ch], and the group's row
// count cnt[g]. Two sets (n_a, mean_a, M2_a), (n_b, mean_b, M2_b) merge exactly (Chan et al.):
//   n = n_a + n_b,  d = mean_b - mean_a,  mean = mean_a + d * n_b / n,  M2 = M2_a + M2_b + d^2 * n_a * n_b / n
// so no sum ever holds more than the spread of the data, whatever the mean, and the order of the merges is fixed.
struct Moments { float n, mean, m2; };
__device__ __forceinline__ void merge(Moments& a, float nb, float mb, float m2b) {
  if (nb <= 0.f) return;
  const float n = a.n + nb, d = mb - a.mean, f = __fdividef(nb, n);
  a.mean = fmaf(d, f, a.mean);
  a.m2 += m2b + d * d * a.n * f;
  a.n = n;
}
// One launch: block = 32 channels x 16 group lanes; slice sl of S takes groups sl*16 + lane, + S*16, ... (two independent
// chains per lane, merged at the end) and leaves its merged moments in out[sl][3][c]; the block that finishes last for a
// channel block (a ticket counter in `tickets`, which must be zero on entry and is reset on exit) merges the S slices,
// 16 lanes per channel again, and writes what bn_stats_fin writes. Every order of merging is fixed: deterministic.
struct BnFromPartials {
  const float* part; const float* cnt; unsigned* tickets; float* out;
  int groups, c, S;
  float momentum, eps;
  float* mean; float* var; float* invstd; const float* rm_in; const float* rv_in; float* rm_out; float* rv_out;
};
constexpr int MERGE_LANES = 16;
__device__ __forceinline__ void merge_lanes(Moments& m, float (*sh)[MERGE_LANES][32], int gl, int cx) {  // result in lane 0
  sh[0][gl][cx] = m.n; sh[1][gl][cx] = m.mean; sh[2][gl][cx] = m.m2;
  __syncthreads();
  if (gl == 0)
    for (int k = 1; k < MERGE_LANES; k++) merge(m, sh[0][k][cx], sh[1][k][cx], sh[2][k][cx]);
}
__global__ void __launch_bounds__(32 * MERGE_LANES) bn_partials_kernel(BnFromPartials a) {
  __shared__ float sh[3][MERGE_LANES][32];
  __shared__ bool last;
  const int cx = threadIdx.x & 31, gl = threadIdx.x >> 5, ch = blockIdx.x * 32 + cx, sl = blockIdx.y, c = a.c;
  Moments m{0.f, 0.f, 0.f}, m1{0.f, 0.f, 0.f};
  if (ch < c) {
    const int step = a.S * MERGE_LANES;
    int g = sl * MERGE_LANES + gl;
    for (; g + step < a.groups; g += 2 * step) {
      const float n0 = __ldg(a.cnt + g), n1 = __ldg(a.cnt + g + step);
      const float s0 = __ldg(a.part + (int64_t)2 * g * c + ch), q0 = __ldg(a.part + ((int64_t)2 * g + 1) * c + ch);
      const float s1 = __ldg(a.part + (int64_t)2 * (g + step) * c + ch), q1 = __ldg(a.part + ((int64_t)2 * (g + step) + 1) * c + ch);
      if (n0 > 0.f) merge(m, n0, __fdividef(s0, n0), q0);
      if (n1 > 0.f) merge(m1, n1, __fdividef(s1, n1), q1);
    }
    if (g < a.groups) {
      const float n0 = __ldg(a.cnt + g);
      if (n0 > 0.f) merge(m, n0, __fdividef(__ldg(a.part + (int64_t)2 * g * c + ch), n0), __ldg(a.part + ((int64_t)2 * g + 1) * c + ch));
    }
    merge(m, m1.n, m1.mean, m1.m2);
  }
  merge_lanes(m, sh, gl, cx);
  if (gl == 0 && ch < c) {
    a.out[((int64_t)sl * 3) * c + ch] = m.n; a.out[((int64_t)sl * 3 + 1) * c + ch] = m.mean; a.out[((int64_t)sl * 3 + 2) * c + ch] = m.m2;
  }
  if (a.S > 1) {
    __threadfence();  // this block's slice is visible before its ticket is
    __syncthreads();
    if (threadIdx.x == 0) last = atomicAdd(a.tickets + blockIdx.x, 1u) == (unsigned)a.S - 1;
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (threadIdx.x == 0) a.tickets[blockIdx.x] = 0;  // ready for the next call
    m = Moments{0.f, 0.f, 0.f};
    if (ch < c)
      for (int k = gl; k < a.S; k += MERGE_LANES)
        merge(m, __ldcg(a.out + ((int64_t)k * 3) * c + ch), __ldcg(a.out + ((int64_t)k * 3 + 1) * c + ch), __ldcg(a.out + ((int64_t)k * 3 + 2) * c + ch));
    __syncthreads();  // (every thread of the block is here: `last` is uniform)
    merge_lanes(m, sh, gl, cx);
  }
  if (gl != 0 || ch >= c) return;
  const float v = m.n > 0.f ? m.m2 / m.n : 0.f, corr = m.n / fmaxf(m.n - 1.f, 1.f);
  if (a.mean) a.mean[ch] = m.mean;
  if (a.var) a.var[ch] = v;
  if (a.invstd) a.invstd[ch] = rsqrtf(v + a.eps);
  if (a.rm_out) {
    const float r0 = a.rm_in[ch], r1 = a.rv_in[ch];
    a.rm_out[ch] = r0 + a.momentum * (m.mean - r0);
    a.rv_out[ch] = r1 + a.momentum * (v * corr - r1);
  }
}

static size_t part_floats(int c) { return (size_t)c * (size_t)std::max(8, 4 * sm_count()) * 2 + 64; }

}  // namespace omt

using namespace omt;

extern "C" {

int omt_bn_stats(const OmtAct* x, int32_t n, int32_t c, int32_t h, int32_t w, float* mean, float* var, float* invstd,
                 float* rm, float* rv, float* new_rm, float* new_rv, float momentum, float eps, uint32_t flags,
                 omt_stream_t stream) {
  OMT_REQUIRE(x && x->p && n > 0 && c > 0 && h > 0 && w > 0, "omt_bn_stats: bad arguments");
  int lay = layout_of(x, c, h, w);
  OMT_REQUIRE(lay == 0 || (lay == 1 && c % 4 == 0), "omt_bn_stats: activation must be NCHW- or NHWC-contiguous (c %% 4 == 0)");
  OMT_REQUIRE(!(flags & OMT_BN_FUNCTIONAL) || (rm && rv && new_rm && new_rv), "omt_bn_stats: functional mode needs rm, rv, new_rm, new_rv");
  cudaStream_t s = st(stream);
  Scratch sc;
  int r = sc.get(nullptr, 0, part_floats(c) * sizeof(float), stream);
  if (r) return r;
  float* part = (float*)sc.p;
  int S = 1;
  r = launch_part<0>(lay, x->p, nullptr, nullptr, nullptr, nullptr, nullptr, false, n, c, h, w, &S, part, s);
  if (r) return r;
  float count = (float)((int64_t)n * h * w);
  float corr = count / std::max(count - 1.f, 1.f);
  bool fn = flags & OMT_BN_FUNCTIONAL;
  bn_stats_fin<<<(unsigned)cdiv((int64_t)c * 32, 256), 256, 0, s>>>(x->p, lay == 0 ? (int64_t)h * w : 1, part, c, S, count, corr, momentum, eps,
                                                      mean, var, invstd, rm, rv, rm ? (fn ? new_rm : rm) : nullptr,
                                                      rm ? (fn ? new_rv : rv) : nullptr);
  return check_launch("bn_stats_fin");
}

int omt_bn_stats_from_partials(const float* partials, int32_t groups, int32_t c, float* mean, float* var, float* invstd, float* rm, float* rv,
                               float* new_rm, float* new_rv, float momentum, float eps, uint32_t flags, omt_stream_t stream) {
  OMT_REQUIRE(partials && c > 0 && groups > 0, "omt_bn_stats_from_partials: bad arguments");
  OMT_REQUIRE(!(flags & OMT_BN_FUNCTIONAL) || (rm && rv && new_rm && new_rv), "omt_bn_stats_from_partials: functional mode needs rm, rv, new_rm, new_rv");
  cudaStream_t s = st(stream);
  const int gx = (int)cdiv(c, 32);
  // slices: enough blocks to fill the device twice, at least 32 groups per lane, at most 64 (the last block merges them)
  const int S = (int)std::max<int64_t>(1, std::min<int64_t>({cdiv(groups, 16 * MERGE_LANES), cdiv(2 * sm_count(), gx), 64}));
  // per-slice moments from the caching allocator; the ticket counters sit behind the group counts in the caller's buffer,
  // zeroed by the convolution that wrote the partials
  Scratch sc;
  int r = sc.get(nullptr, 0, (size_t)S * 3 * c * sizeof(float), stream);
  if (r) return r;
  const bool fn = flags & OMT_BN_FUNCTIONAL;
  const float* cnt = partials + (size_t)2 * groups * c;
  BnFromPartials a{partials, cnt, reinterpret_cast<unsigned*>(const_cast<float*>(cnt + groups)), (float*)sc.p, groups, c, S, momentum, eps,
                   mean, var, invstd, rm, rv, rm ? (fn ? new_rm : rm) : nullptr, rm ? (fn ? new_rv : rv) : nullptr};
  bn_partials_kernel<<<dim3(gx, S), 32 * MERGE_LANES, 0, s>>>(a);
  return check_launch("bn_stats_from_partials");
}

int omt_bn_apply_add(const OmtAct* x, const OmtAct* res, const OmtAct* y, int32_t n, int32_t c, int32_t h, int32_t w, const float* mean,
                     const float* invstd, const float* gamma, const float* beta, uint32_t flags, omt_stream_t stream) {
  OMT_REQUIRE(x && y && x->p && y->p && mean && invstd && gamma && beta, "omt_bn_apply: bad arguments");
  int lay = layout_of(x, c, h, w);
  OMT_REQUIRE(lay >= 0 && layout_of(y, c, h, w) == lay, "omt_bn_apply: x and y must share an NCHW or NHWC contiguous layout");
  const bool has_res = res && res->p;
  OMT_REQUIRE(!has_res || layout_of(res, c, h, w) == lay, "omt_bn_apply_add: the residual must have the layout of x");
  BnEw a{};
  a.x = x->p; a.g = x->p; a.y = x->p; a.out = y->p; a.mean = mean; a.inv = invstd; a.gamma = gamma; a.beta = beta;
  a.res = has_res ? res->p : nullptr;
  a.c = c; a.hw = h * w; a.total = (int64_t)n * c * h * w;
  OMT_REQUIRE(!(flags & OMT_BN_MASKBITS) || (flags & OMT_BN_RELU), "omt_bn_apply: OMT_BN_MASKBITS is the mask of the ReLU: it needs OMT_BN_RELU");
  if (flags & OMT_BN_MASKBITS) a.bits_out = reinterpret_cast<uint32_t*>(y->p + a.total);
  return launch_ew<0>(a, flags & OMT_BN_RELU, lay == 1, st(stream), has_res ? "bn_apply_add" : "bn_apply");
}
int omt_bn_apply(const OmtAct* x, const OmtAct* y, int32_t n, int32_t c, int32_t h, int32_t w, const float* mean,
                 const float* invstd, const float* gamma, const float* beta, uint32_t flags, omt_stream_t stream) {
  return omt_bn_apply_add(x, nullptr, y, n, c, h, w, mean, invstd, gamma, beta, flags, stream);
}

int omt_bn_apply_pool2(const OmtAct* x, const OmtAct* y, const OmtAct* z, uint8_t* idx, int32_t n, int32_t c, int32_t h, int32_t w,
                       const float* mean, const float* invstd, const float* gamma, const float* beta, uint32_t flags, omt_stream_t stream) {
  OMT_REQUIRE(x && z && x->p && z->p && mean && invstd && gamma && beta && n > 0 && c > 0, "omt_bn_apply_pool2: bad arguments");
  OMT_REQUIRE(h >= 2 && w >= 2 && h % 2 == 0 && w % 2 == 0, "omt_bn_apply_pool2: needs even height and width (got %d x %d)", h, w);
  const int lay = layout_of(x, c, h, w);
  OMT_REQUIRE(lay >= 0 && layout_of(z, c, h / 2, w / 2) == lay && (!y || !y->p || layout_of(y, c, h, w) == lay),
              "omt_bn_apply_pool2: x, y and z must share an NCHW or NHWC contiguous layout");
  BnPool a{view(x), y && y->p ? view(y) : ActView{nullptr, 0, 0, 0, 0}, view(z), idx, mean, invstd, gamma, beta, n, c, h / 2, w / 2,
           (flags & OMT_BN_RELU) != 0};
  const int64_t outs = (int64_t)n * c * (h / 2) * (w / 2);
  const bool vec = lay == 1 && c % 4 == 0 &&
                   ((reinterpret_cast<uintptr_t>(x->p) | reinterpret_cast<uintptr_t>(a.y.p) | reinterpret_cast<uintptr_t>(z->p) |
                     reinterpret_cast<uintptr_t>(mean) | reinterpret_cast<uintptr_t>(invstd) | reinterpret_cast<uintptr_t>(gamma) |
                     reinterpret_cast<uintptr_t>(beta)) & 15) == 0 && (reinterpret_cast<uintptr_t>(idx) & 3) == 0;
  if (vec) bn_pool2_nhwc4<<<(unsigned)cdiv(outs / 4, 256), 256, 0, st(stream)>>>(a);
  else if (lay == 1) bn_pool2_scalar<true><<<(unsigned)cdiv(outs, 256), 256, 0, st(stream)>>>(a);
  else bn_pool2_scalar<false><<<(unsigned)cdiv(outs, 256), 256, 0, st(stream)>>>(a);
  return check_launch("bn_apply_pool2");
}

int omt_bn_eval(const OmtAct* x, const OmtAct* y, int32_t n, int32_t c, int32_t h, int32_t w, const float* rm,
                const float* rv, const float* gamma, const float* beta, float eps, uint32_t flags, omt_stream_t stream) {
  OMT_REQUIRE(x && y && x->p && y->p && rm && rv && gamma && beta, "omt_bn_eval: bad arguments");
  int lay = layout_of(x, c, h, w);
  OMT_REQUIRE(lay >= 0 && layout_of(y, c, h, w) == lay, "omt_bn_eval: x and y must share an NCHW or NHWC contiguous layout");
  BnEw a{};
  a.x = x->p; a.g = x->p; a.y = x->p; a.out = y->p; a.mean = rm; a.inv = rv; a.gamma = gamma; a.beta = beta; a.eps = eps;
  a.c = c; a.hw = h * w; a.total = (int64_t)n * c * h * w;
  return launch_ew<1>(a, flags & OMT_BN_RELU, lay == 1, st(stream), "bn_eval");
}

int omt_bn_backward(const OmtAct* gy, const OmtAct* x, const OmtAct* y, const OmtAct* dx, int32_t n, int32_t c, int32_t h,
                    int32_t w, const float* mean, const float* invstd, const float* gamma, float* dgb, float scale,
                    uint32_t flags, omt_stream_t stream) {
  return omt_bn_backward_add(gy, x, y, dx, nullptr, n, c, h, w, mean, invstd, gamma, dgb, scale, flags, stream);
}
int omt_bn_backward_add(const OmtAct* gy, const OmtAct* x, const OmtAct* y, const OmtAct* dx, const OmtAct* dres, int32_t n, int32_t c,
                        int32_t h, int32_t w, const float* mean, const float* invstd, const float* gamma, float* dgb, float scale,
                        uint32_t flags, omt_stream_t stream) {
  bool relu = flags & OMT_BN_RELU;
  const bool has_dres = dres && dres->p;
  OMT_REQUIRE(!has_dres || (relu && dx && dx->p), "omt_bn_backward_add: the masked gradient is written by the ReLU-masked dx pass");
  OMT_REQUIRE(gy && x && gy->p && x->p && mean && invstd && gamma && dgb, "omt_bn_backward: bad arguments");
  OMT_REQUIRE(!relu || (y && y->p), "omt_bn_backward: the ReLU mask needs y");
  int lay = layout_of(x, c, h, w);
  OMT_REQUIRE(lay == 0 || (lay == 1 && c % 4 == 0), "omt_bn_backward: activation must be NCHW- or NHWC-contiguous (c %% 4 == 0)");
  OMT_REQUIRE(layout_of(gy, c, h, w) == lay && (!relu || layout_of(y, c, h, w) == lay) &&
                  (!dx || !dx->p || layout_of(dx, c, h, w) == lay),
              "omt_bn_backward: gy, x, y, dx must share one layout");
  cudaStream_t s = st(stream);
  Scratch sc;
  int r = sc.get(nullptr, 0, (part_floats(c) + 2 * (size_t)c) * sizeof(float), stream);
  if (r) return r;
  float* part = (float*)sc.p;
  float* raw = part + part_floats(c);
  int S = 1;
  // OMT_BN_MASKBITS: the ReLU mask is the bit words the forward pass left behind y; y's values are not read
  const uint32_t* bits = (relu && (flags & OMT_BN_MASKBITS)) ? reinterpret_cast<const uint32_t*>(y->p + (int64_t)n * c * h * w) : nullptr;
  r = launch_part<1>(lay, x->p, gy->p, relu ? y->p : x->p, bits, mean, invstd, relu, n, c, h, w, &S, part, s);
  if (r) return r;
  bn_bwd_fin<<<(unsigned)cdiv((int64_t)c * 32, 256), 256, 0, s>>>(part, c, S, scale, dgb, raw);
  r = check_launch("bn_bwd_fin");
  if (r || !dx || !dx->p) return r;
  BnEw a{};
  OMT_REQUIRE(!has_dres || layout_of(dres, c, h, w) == lay, "omt_bn_backward_add: dres must have the layout of x");
  a.x = x->p; a.g = gy->p; a.y = relu ? y->p : x->p; a.out = dx->p; a.mean = mean; a.inv = invstd; a.gamma = gamma; a.dgb = raw;
  a.gz = has_dres ? dres->p : nullptr;
  a.bits_in = bits;
  a.m = (float)((int64_t)n * h * w); a.c = c; a.hw = h * w; a.total = (int64_t)n * c * h * w;
  return launch_ew<2>(a, relu, lay == 1, st(stream), has_dres ? "bn_bwd_apply_add" : "bn_bwd_apply");
}

}  // extern "C"

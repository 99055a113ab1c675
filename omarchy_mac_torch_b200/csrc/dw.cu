// Depthwise convolution (groups == channels): forward, input gradient, weight gradient, for any ks <= 11,
// stride 1..4, pad <= ks. HBM-bound kernels: each activation element is fetched from DRAM once (neighbouring taps
// hit L1/L2), outputs are written with coalesced (NCHW: along x; channels-last: 128-bit along c) stores, and the
// weight gradient keeps all ks*ks tap sums of a channel in registers so x and gy are read once, not ks*ks times.
//
// Semantics: reference dw_fwd/dw_gin/dw_gwt (stride 1, "same" padding) and dwg_fwd/dwg_gin/dwg_gwt (general) in
// csrc/kernels/, dispatched from csrc/conv.cpp:194-229. One code path covers both families here.
#include <algorithm>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace omt {

struct DwArgs {
  ActView x, y;  // fwd: x in, y out. dgrad: x = gy (in), y = dx (out). wgrad: x = x, y = gy.
  const float* w;
  const float* bias;
  int n, c, ih, iw, oh, ow, ks, stride, pad;
  uint32_t flags;
};

// index order follows the memory layout so that consecutive threads touch consecutive addresses
// index -> (img, ch, y, x) in memory order of the layout; 32-bit arithmetic whenever the index fits (64-bit division is
// emulated and would dominate these bandwidth-bound kernels)
template <bool NHWC, class I>
__device__ __forceinline__ void decode_t(I i, int c, int h, int w, int& img, int& ch, int& y, int& x) {
  if (NHWC) {
    ch = (int)(i % (I)c); i /= (I)c;
    x = (int)(i % (I)w); i /= (I)w;
    y = (int)(i % (I)h); img = (int)(i / (I)h);
  } else {
    x = (int)(i % (I)w); i /= (I)w;
    y = (int)(i % (I)h); i /= (I)h;
    ch = (int)(i % (I)c); img = (int)(i / (I)c);
  }
}
template <bool NHWC>
__device__ __forceinline__ void decode(int64_t i, int c, int h, int w, int& img, int& ch, int& y, int& x) {
  if (i < 0x7fffffffll) decode_t<NHWC, uint32_t>((uint32_t)i, c, h, w, img, ch, y, x);
  else decode_t<NHWC, int64_t>(i, c, h, w, img, ch, y, x);
}

template <bool NHWC>
__global__ void __launch_bounds__(256) dw_fwd_kernel(DwArgs a) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.c * a.oh * a.ow) return;
  int img, ch, oy, ox;
  decode<NHWC>(i, a.c, a.oh, a.ow, img, ch, oy, ox);
  const int y0 = oy * a.stride - a.pad, x0 = ox * a.stride - a.pad;
  const float* xp = a.x.p + img * a.x.sn + ch * a.x.sc;
  const float* wp = a.w + (int64_t)ch * a.ks * a.ks;
  float s = 0.f;
  for (int ky = 0; ky < a.ks; ky++) {
    int sy = y0 + ky;
    if (sy < 0 || sy >= a.ih) continue;
    for (int kx = 0; kx < a.ks; kx++) {
      int sx = x0 + kx;
      if (sx < 0 || sx >= a.iw) continue;
      s = fmaf(__ldg(xp + sy * a.x.sh + sx * a.x.sw), __ldg(wp + ky * a.ks + kx), s);
    }
  }
  if (a.flags & OMT_EPI_BIAS) s += __ldg(a.bias + ch);
  if (a.flags & OMT_EPI_RELU) s = fmaxf(s, 0.f);
  a.y.p[a.y.off(img, ch, oy, ox)] = s;
}

// channels-last, 4 channels per thread: 128-bit loads of x, weights re-laid as float4 per tap on the fly
__global__ void __launch_bounds__(256) dw_fwd_nhwc4_kernel(DwArgs a) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int c4n = a.c / 4;
  if (i >= (int64_t)a.n * c4n * a.oh * a.ow) return;
  int img, cg, oy, ox;
  decode<true>(i, c4n, a.oh, a.ow, img, cg, oy, ox);
  const int ch = cg * 4, kk = a.ks * a.ks;
  const int y0 = oy * a.stride - a.pad, x0 = ox * a.stride - a.pad;
  const float* xp = a.x.p + img * a.x.sn + ch;
  const float* wp = a.w + (int64_t)ch * kk;
  float4 s = make_float4(0, 0, 0, 0);
  for (int ky = 0; ky < a.ks; ky++) {
    int sy = y0 + ky;
    if (sy < 0 || sy >= a.ih) continue;
    for (int kx = 0; kx < a.ks; kx++) {
      int sx = x0 + kx;
      if (sx < 0 || sx >= a.iw) continue;
      float4 xv = __ldg(reinterpret_cast<const float4*>(xp + sy * a.x.sh + sx * a.x.sw));
      int t = ky * a.ks + kx;
      s.x = fmaf(xv.x, __ldg(wp + t), s.x);
      s.y = fmaf(xv.y, __ldg(wp + kk + t), s.y);
      s.z = fmaf(xv.z, __ldg(wp + 2 * kk + t), s.z);
      s.w = fmaf(xv.w, __ldg(wp + 3 * kk + t), s.w);
    }
  }
  if (a.flags & OMT_EPI_BIAS) {
    float4 b = __ldg(reinterpret_cast<const float4*>(a.bias + ch));
    s.x += b.x; s.y += b.y; s.z += b.z; s.w += b.w;
  }
  if (a.flags & OMT_EPI_RELU) { s.x = fmaxf(s.x, 0.f); s.y = fmaxf(s.y, 0.f); s.z = fmaxf(s.z, 0.f); s.w = fmaxf(s.w, 0.f); }
  *reinterpret_cast<float4*>(a.y.p + a.y.off(img, ch, oy, ox)) = s;
}

// input gradient as a gather: dx[y,x] = sum over taps with (y+p-ky) % s == 0 of gy[(y+p-ky)/s, (x+p-kx)/s] * w[ky,kx]
template <bool NHWC>
__global__ void __launch_bounds__(256) dw_dgrad_kernel(DwArgs a) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.c * a.ih * a.iw) return;
  int img, ch, yy, xx;
  decode<NHWC>(i, a.c, a.ih, a.iw, img, ch, yy, xx);
  const float* gp = a.x.p + img * a.x.sn + ch * a.x.sc;
  const float* wp = a.w + (int64_t)ch * a.ks * a.ks;
  const int s_ = a.stride;
  float s = 0.f;
  // first tap on the stride grid, then step by the stride: no per-tap modulo
  for (int ky = (yy + a.pad) % s_; ky < a.ks; ky += s_) {
    int oy = (yy + a.pad - ky) / s_;
    if (yy + a.pad - ky < 0 || oy >= a.oh) continue;
    for (int kx = (xx + a.pad) % s_; kx < a.ks; kx += s_) {
      int ox = (xx + a.pad - kx) / s_;
      if (xx + a.pad - kx < 0 || ox >= a.ow) continue;
      s = fmaf(__ldg(gp + oy * a.x.sh + ox * a.x.sw), __ldg(wp + ky * a.ks + kx), s);
    }
  }
  a.y.p[a.y.off(img, ch, yy, xx)] = s;
}

// weight gradient, NCHW: block (channel, slice) walks output pixels; thread keeps KS*KS partial sums in registers
template <int KS>
__global__ void __launch_bounds__(256) dw_wgrad_nchw_kernel(DwArgs a, int S, float* __restrict__ part) {
  __shared__ float red[32];
  const int ch = blockIdx.x, sl = blockIdx.y, ohw = a.oh * a.ow;
  float acc[KS * KS];
#pragma unroll
  for (int t = 0; t < KS * KS; t++) acc[t] = 0.f;
  for (int img = sl; img < a.n; img += S) {
    const float* gp = a.y.p + img * a.y.sn + ch * a.y.sc;
    const float* xp = a.x.p + img * a.x.sn + ch * a.x.sc;
    for (int e = threadIdx.x; e < ohw; e += blockDim.x) {
      int oy = e / a.ow, ox = e - oy * a.ow;
      float gv = __ldg(gp + oy * a.y.sh + ox * a.y.sw);
      int y0 = oy * a.stride - a.pad, x0 = ox * a.stride - a.pad;
#pragma unroll
      for (int ky = 0; ky < KS; ky++) {
        int sy = y0 + ky;
        bool oky = sy >= 0 && sy < a.ih;
#pragma unroll
        for (int kx = 0; kx < KS; kx++) {
          int sx = x0 + kx;
          if (oky && sx >= 0 && sx < a.iw) acc[ky * KS + kx] = fmaf(gv, __ldg(xp + sy * a.x.sh + sx * a.x.sw), acc[ky * KS + kx]);
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < KS * KS; t++) {
    float v = block_sum(acc[t], red);
    if (threadIdx.x == 0) part[((int64_t)ch * S + sl) * (KS * KS) + t] = v;
  }
}
// any kernel size: one tap per blockIdx.z (re-reads the activations ks*ks times; only used for ks not in {3,5,7})
__global__ void __launch_bounds__(256) dw_wgrad_tap_kernel(DwArgs a, int S, float* __restrict__ part) {
  __shared__ float red[32];
  const int ch = blockIdx.x, sl = blockIdx.y, t = blockIdx.z, ky = t / a.ks, kx = t - ky * a.ks, ohw = a.oh * a.ow;
  float acc = 0.f;
  for (int img = sl; img < a.n; img += S) {
    const float* gp = a.y.p + img * a.y.sn + ch * a.y.sc;
    const float* xp = a.x.p + img * a.x.sn + ch * a.x.sc;
    for (int e = threadIdx.x; e < ohw; e += blockDim.x) {
      int oy = e / a.ow, ox = e - oy * a.ow;
      int sy = oy * a.stride - a.pad + ky, sx = ox * a.stride - a.pad + kx;
      if (sy >= 0 && sy < a.ih && sx >= 0 && sx < a.iw)
        acc = fmaf(__ldg(gp + oy * a.y.sh + ox * a.y.sw), __ldg(xp + sy * a.x.sh + sx * a.x.sw), acc);
    }
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) part[((int64_t)ch * S + sl) * (a.ks * a.ks) + t] = acc;
}
// channels-last: one thread per channel (coalesced across c), slices over pixels; no block reduction needed
template <int KS>
__global__ void __launch_bounds__(128) dw_wgrad_nhwc_kernel(DwArgs a, int S, float* __restrict__ part) {
  const int ch = blockIdx.x * blockDim.x + threadIdx.x, sl = blockIdx.y;
  if (ch >= a.c) return;
  float acc[KS * KS];
#pragma unroll
  for (int t = 0; t < KS * KS; t++) acc[t] = 0.f;
  const int64_t P = (int64_t)a.n * a.oh * a.ow;
  for (int64_t p = sl; p < P; p += S) {
    int ox = (int)(p % a.ow);
    int64_t q = p / a.ow;
    int oy = (int)(q % a.oh), img = (int)(q / a.oh);
    float gv = __ldg(a.y.p + a.y.off(img, ch, oy, ox));
    const float* xp = a.x.p + img * a.x.sn + ch;
    int y0 = oy * a.stride - a.pad, x0 = ox * a.stride - a.pad;
#pragma unroll
    for (int ky = 0; ky < KS; ky++) {
      int sy = y0 + ky;
      bool oky = sy >= 0 && sy < a.ih;
#pragma unroll
      for (int kx = 0; kx < KS; kx++) {
        int sx = x0 + kx;
        if (oky && sx >= 0 && sx < a.iw) acc[ky * KS + kx] = fmaf(gv, __ldg(xp + sy * a.x.sh + sx * a.x.sw), acc[ky * KS + kx]);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < KS * KS; t++) part[((int64_t)ch * S + sl) * (KS * KS) + t] = acc[t];
}
// ---------------------------------------------------------------------------------------------------------------------
// Channels-last fast paths (c % 4 == 0, dense tensors, 16-byte aligned): 4 channels per thread with 128-bit accesses, and
// the filter re-laid once per call as wt[tap][c] so a thread's four weights of a tap are one 128-bit load.
// ---------------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) dw_weight_tc_kernel(const float* __restrict__ w, float* __restrict__ wt, int c, int kk) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;  // i = t * c + ch
  if (i >= c * kk) return;
  int t = i / c, ch = i - t * c;
  wt[i] = __ldg(w + (int64_t)ch * kk + t);
}

// Forward (FLIP = false) and stride-1 input gradient (FLIP = true: taps mirrored, pad = ks-1-pad, the caller swaps the
// tensors). A thread produces TX consecutive output pixels of one row for its 4 channels: per filter row it loads the
// (TX-1)*stride + KS input pixels once and slides the taps over them in registers.
template <int KS, int STRIDE, bool FLIP, int TX>
__global__ void __launch_bounds__(256) dw_rows_nhwc4_kernel(DwArgs a, const float* __restrict__ wt) {
  constexpr int SPAN = (TX - 1) * STRIDE + KS;
  const int c4n = a.c >> 2, gx = (a.ow + TX - 1) / TX;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.oh * gx * c4n) return;
  int img, cq, oy, xg;
  decode<true>(i, c4n, a.oh, gx, img, cq, oy, xg);
  const int ch = cq * 4, ox0 = xg * TX;
  const int y0 = oy * STRIDE - a.pad, x0 = ox0 * STRIDE - a.pad;
  // pointer to input pixel (y0, x0) of this thread's channels; only dereferenced where that pixel exists
  const float* xbase = a.x.p + (((int64_t)img * a.ih + y0) * a.iw + x0) * a.c + ch;
  const int rs = a.iw * a.c;  // floats per input row
  const bool interior = x0 >= 0 && x0 + SPAN <= a.iw;
  const float* wq = wt + ch;
  float4 acc[TX];
#pragma unroll
  for (int j = 0; j < TX; j++) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int ky = 0; ky < KS; ky++) {
    const int sy = y0 + ky;
    if (sy < 0 || sy >= a.ih) continue;
    const float* xr = xbase + (int64_t)ky * rs;
    float4 in[SPAN];
    if (interior) {
#pragma unroll
      for (int k = 0; k < SPAN; k++) in[k] = __ldg(reinterpret_cast<const float4*>(xr + k * a.c));
    } else {
#pragma unroll
      for (int k = 0; k < SPAN; k++) {
        const int sx = x0 + k;
        in[k] = (sx >= 0 && sx < a.iw) ? __ldg(reinterpret_cast<const float4*>(xr + k * a.c)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int kx = 0; kx < KS; kx++) {
      const int t = FLIP ? (KS - 1 - ky) * KS + (KS - 1 - kx) : ky * KS + kx;
      const float4 wv = __ldg(reinterpret_cast<const float4*>(wq + t * a.c));
#pragma unroll
      for (int j = 0; j < TX; j++) {
        const float4 v = in[j * STRIDE + kx];
        acc[j].x = fmaf(v.x, wv.x, acc[j].x); acc[j].y = fmaf(v.y, wv.y, acc[j].y);
        acc[j].z = fmaf(v.z, wv.z, acc[j].z); acc[j].w = fmaf(v.w, wv.w, acc[j].w);
      }
    }
  }
  float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
  if (a.flags & OMT_EPI_BIAS) b = __ldg(reinterpret_cast<const float4*>(a.bias + ch));
  float* yp = a.y.p + (((int64_t)img * a.oh + oy) * a.ow + ox0) * a.c + ch;
#pragma unroll
  for (int j = 0; j < TX; j++) {
    if (ox0 + j >= a.ow) break;
    float4 o = make_float4(acc[j].x + b.x, acc[j].y + b.y, acc[j].z + b.z, acc[j].w + b.w);
    if (a.flags & OMT_EPI_RELU) { o.x = fmaxf(o.x, 0.f); o.y = fmaxf(o.y, 0.f); o.z = fmaxf(o.z, 0.f); o.w = fmaxf(o.w, 0.f); }
    *reinterpret_cast<float4*>(yp + (int64_t)j * a.c) = o;
  }
}

// strided input gradient, channels-last: the gather of dw_dgrad_kernel on 4 channels at a time
__global__ void __launch_bounds__(256) dw_dgrad_nhwc4_kernel(DwArgs a, const float* __restrict__ wt) {
  const int c4n = a.c >> 2;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.ih * a.iw * c4n) return;
  int img, cq, yy, xx;
  decode<true>(i, c4n, a.ih, a.iw, img, cq, yy, xx);
  const int ch = cq * 4, s_ = a.stride;
  const float* gp = a.x.p + (int64_t)img * a.oh * a.ow * a.c + ch;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int ky = (yy + a.pad) % s_; ky < a.ks; ky += s_) {
    const int oy = (yy + a.pad - ky) / s_;
    if (yy + a.pad - ky < 0 || oy >= a.oh) continue;
    for (int kx = (xx + a.pad) % s_; kx < a.ks; kx += s_) {
      const int ox = (xx + a.pad - kx) / s_;
      if (xx + a.pad - kx < 0 || ox >= a.ow) continue;
      const float4 g = __ldg(reinterpret_cast<const float4*>(gp + ((int64_t)oy * a.ow + ox) * a.c));
      const float4 wv = __ldg(reinterpret_cast<const float4*>(wt + (int64_t)(ky * a.ks + kx) * a.c + ch));
      acc.x = fmaf(g.x, wv.x, acc.x); acc.y = fmaf(g.y, wv.y, acc.y); acc.z = fmaf(g.z, wv.z, acc.z); acc.w = fmaf(g.w, wv.w, acc.w);
    }
  }
  *reinterpret_cast<float4*>(a.y.p + (((int64_t)img * a.ih + yy) * a.iw + xx) * a.c + ch) = acc;
}

// weight gradient, channels-last: a thread keeps the KS*KS tap sums of 4 channels; a block is CL channel quads x PL pixel
// lanes, slices over pixels across blockIdx.y; the pixel lanes are summed through shared memory in a fixed order.
// A work item is a group of TX = 4 consecutive pixels of one output row: per filter row its (TX-1)*stride + KS input pixels
// and the 4 gy pixels are loaded together (enough loads in flight to cover DRAM latency at one block per SM), then
// every tap takes its 4 products from registers.
template <int KS, int STRIDE>
__global__ void __launch_bounds__(256) dw_wgrad_nhwc4_kernel(DwArgs a, int S, int CL, float* __restrict__ part) {
  constexpr int TX = 4, SPAN = (TX - 1) * STRIDE + KS;
  extern __shared__ float4 red4[];  // [PL][CL]
  const int PL = blockDim.x / CL;
  const int cl = threadIdx.x % CL, pl = threadIdx.x / CL;
  const int cq = blockIdx.x * CL + cl, sl = blockIdx.y;
  const bool live = pl < PL && cq < (a.c >> 2);
  const int ch = cq * 4;
  float4 acc[KS * KS];
#pragma unroll
  for (int t = 0; t < KS * KS; t++) acc[t] = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
    const uint32_t gx = (uint32_t)(a.ow + TX - 1) / TX;
    const uint32_t items = (uint32_t)a.n * a.oh * gx;
    const int rs = a.iw * a.c;
    for (uint32_t it = (uint32_t)sl * PL + pl; it < items; it += (uint32_t)S * PL) {
      const uint32_t xg = it % gx, r = it / gx;
      const int oy = (int)(r % (uint32_t)a.oh), img = (int)(r / (uint32_t)a.oh);
      const int ox0 = (int)xg * TX;
      const int y0 = oy * STRIDE - a.pad, x0 = ox0 * STRIDE - a.pad;
      const float* gp = a.y.p + (((int64_t)img * a.oh + oy) * a.ow + ox0) * a.c + ch;
      float4 g[TX];
#pragma unroll
      for (int j = 0; j < TX; j++) g[j] = ox0 + j < a.ow ? __ldg(reinterpret_cast<const float4*>(gp + j * a.c)) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float* xbase = a.x.p + (((int64_t)img * a.ih + y0) * a.iw + x0) * a.c + ch;
      const bool interior = x0 >= 0 && x0 + SPAN <= a.iw;
#pragma unroll
      for (int ky = 0; ky < KS; ky++) {
        const int sy = y0 + ky;
        if (sy < 0 || sy >= a.ih) continue;
        const float* xr = xbase + (int64_t)ky * rs;
        float4 in[SPAN];
        if (interior) {
#pragma unroll
          for (int k = 0; k < SPAN; k++) in[k] = __ldg(reinterpret_cast<const float4*>(xr + k * a.c));
        } else {
#pragma unroll
          for (int k = 0; k < SPAN; k++) {
            const int sx = x0 + k;
            in[k] = (sx >= 0 && sx < a.iw) ? __ldg(reinterpret_cast<const float4*>(xr + k * a.c)) : make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
#pragma unroll
        for (int kx = 0; kx < KS; kx++) {
          float4& q = acc[ky * KS + kx];
#pragma unroll
          for (int j = 0; j < TX; j++) {
            const float4 v = in[j * STRIDE + kx];
            q.x = fmaf(g[j].x, v.x, q.x); q.y = fmaf(g[j].y, v.y, q.y); q.z = fmaf(g[j].z, v.z, q.z); q.w = fmaf(g[j].w, v.w, q.w);
          }
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < KS * KS; t++) {
    __syncthreads();
    if (pl < PL) red4[pl * CL + cl] = acc[t];
    __syncthreads();
    if (pl == 0 && live) {
      float4 s4 = red4[cl];
      for (int k = 1; k < PL; k++) {
        const float4 v = red4[k * CL + cl];
        s4.x += v.x; s4.y += v.y; s4.z += v.z; s4.w += v.w;
      }
      const int kk = KS * KS;
      part[((int64_t)(ch + 0) * S + sl) * kk + t] = s4.x;
      part[((int64_t)(ch + 1) * S + sl) * kk + t] = s4.y;
      part[((int64_t)(ch + 2) * S + sl) * kk + t] = s4.z;
      part[((int64_t)(ch + 3) * S + sl) * kk + t] = s4.w;
    }
  }
}
// one warp per output (ch, tap): lanes stride over the S slices, then a shuffle tree (fixed order: deterministic)
__global__ void __launch_bounds__(256) dw_wgrad_fin_kernel(const float* __restrict__ part, int64_t total, int kk, int S, float scale, float* out) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;  // i = ch*kk + t
  const int lane = threadIdx.x & 31;
  if (i >= total) return;
  const int64_t ch = i / kk;
  const int t = (int)(i - ch * kk);
  float s = 0.f;
  for (int k = lane; k < S; k += 32) s += __ldg(part + (ch * S + k) * kk + t);
  s = warp_sum(s);
  if (lane == 0) out[i] = s * scale;
}

// ---------------------------------------------------------------------------------------------------------------------
// Rolling kernels (channels-last, dense, 16-byte aligned, ks in {3, 5, 7}, stride 1 or 2). A thread owns a strip of TX
// output columns and `seg_rows` output rows for CH channels and walks DOWN the strip's input rows once: each input row is
// loaded once and feeds the R = ceil(ks / stride) output rows it overlaps, whose partial sums wait in registers. Against
// one output row per thread (dw_rows_nhwc4_kernel) that cuts the loads per output pixel from ks * span / TX to span / TX:
// the 5x5 kernels were bound by L1 traffic (65 bytes per output element), not by HBM.
//   CH = 4 (128-bit accesses) for 3x3, whose nine weights also stay in registers; CH = 2 (64-bit) for 5x5 and 7x7, where the
//   R x TX partial sums of four channels would not fit.
// ---------------------------------------------------------------------------------------------------------------------
template <int CH>
struct Vec {
  float v[CH];
};
template <int CH>
__device__ __forceinline__ Vec<CH> ldv(const float* p) {
  Vec<CH> r;
  if constexpr (CH == 4) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(p));
    r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
  } else {
    const float2 t = __ldg(reinterpret_cast<const float2*>(p));
    r.v[0] = t.x; r.v[1] = t.y;
  }
  return r;
}
template <int CH>
__device__ __forceinline__ void stv(float* p, const Vec<CH>& r) {
  if constexpr (CH == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
  else *reinterpret_cast<float2*>(p) = make_float2(r.v[0], r.v[1]);
}
template <int CH>
__device__ __forceinline__ Vec<CH> zerov() {
  Vec<CH> r;
#pragma unroll
  for (int k = 0; k < CH; k++) r.v[k] = 0.f;
  return r;
}
template <int CH>
__device__ __forceinline__ void fmav(Vec<CH>& acc, const Vec<CH>& a, const Vec<CH>& b) {
#pragma unroll
  for (int k = 0; k < CH; k++) acc.v[k] = fmaf(a.v[k], b.v[k], acc.v[k]);
}
// two channels: one packed multiply-add (fma.rn.f32x2, the two-lane FP32 instruction of sm_100): same rounding per lane
template <>
__device__ __forceinline__ void fmav<2>(Vec<2>& acc, const Vec<2>& a, const Vec<2>& b) {
  asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%0, %1};\n\t"
      "fma.rn.f32x2 rc, ra, rb, rc;\n\tmov.b64 {%0, %1}, rc;\n\t}"
      : "+f"(acc.v[0]), "+f"(acc.v[1])
      : "f"(a.v[0]), "f"(a.v[1]), "f"(b.v[0]), "f"(b.v[1]));
}
__host__ __device__ constexpr int floor_div(int a, int b) { return a >= 0 ? a / b : -((-a + b - 1) / b); }
__host__ __device__ constexpr int pos_mod(int a, int b) { return ((a % b) + b) % b; }

// one row of SPAN input pixels starting at column x0 (zero outside the image)
template <int CH, int SPAN>
__device__ __forceinline__ void load_span(Vec<CH> (&in)[SPAN], const float* __restrict__ row, int x0, int iw, int c, bool interior) {
  if (interior) {
#pragma unroll
    for (int k = 0; k < SPAN; k++) in[k] = ldv<CH>(row + (int64_t)k * c);
  } else {
#pragma unroll
    for (int k = 0; k < SPAN; k++) in[k] = (x0 + k >= 0 && x0 + k < iw) ? ldv<CH>(row + (int64_t)k * c) : zerov<CH>();
  }
}

// Input rows reach the rolling kernels through a private ring in shared memory, filled by cp.async DEPTH rows ahead of their
// use: the copies hold no registers while in flight, so a thread keeps (DEPTH - 1) * SPAN vectors travelling at 8-12 warps per
// SM (with plain loads and one row in flight these kernels sat at 42 % of the DRAM bandwidth, stalled on the scoreboard).
// Layout [slot][k][thread]: consecutive threads, consecutive vectors; nobody else touches a thread's slots, so no block barrier.
constexpr int ROLL_THREADS = 128, ROLL_DEPTH = 4;
template <int CH>
__device__ __forceinline__ void cp_async_vec(uint32_t dst, const float* src, bool valid) {  // !valid: zeros are written
  const uint32_t n = valid ? CH * 4 : 0;
  if constexpr (CH == 4) asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
  else asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
template <int CH, int SPAN>
struct RowRing {
  uint32_t base;  // shared-memory address of this thread's vector in slot 0, k = 0
  __device__ __forceinline__ uint32_t at(int slot, int k) const { return base + (uint32_t)((slot * SPAN + k) * ROLL_THREADS * CH * 4); }
  // request row `r` (pointer to its pixel x0; pixels outside [0, iw) become zeros; `safe` always points inside the tensor)
  __device__ __forceinline__ void request(int r, bool row_valid, const float* row, const float* safe, int x0, int iw, int c) const {
    if (row_valid) {
      const int slot = r % ROLL_DEPTH;
#pragma unroll
      for (int k = 0; k < SPAN; k++) {
        const bool in = x0 + k >= 0 && x0 + k < iw;
        cp_async_vec<CH>(at(slot, k), in ? row + (int64_t)k * c : safe, in);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");  // (an empty group when the row lies outside the image: the count stays uniform)
  }
  __device__ __forceinline__ void wait_oldest() const { asm volatile("cp.async.wait_group %0;" ::"n"(ROLL_DEPTH - 1) : "memory"); }
  __device__ __forceinline__ void read(int r, Vec<CH> (&in)[SPAN]) const {
    const int slot = r % ROLL_DEPTH;
#pragma unroll
    for (int k = 0; k < SPAN; k++) {
      if constexpr (CH == 4) {
        float4 t;
        asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(t.x), "=f"(t.y), "=f"(t.z), "=f"(t.w) : "r"(at(slot, k)) : "memory");
        in[k].v[0] = t.x; in[k].v[1] = t.y; in[k].v[2] = t.z; in[k].v[3] = t.w;
      } else {
        float2 t;
        asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(t.x), "=f"(t.y) : "r"(at(slot, k)) : "memory");
        in[k].v[0] = t.x; in[k].v[1] = t.y;
      }
    }
  }
};
template <int CH, int SPAN>
constexpr size_t ring_bytes() { return (size_t)ROLL_DEPTH * SPAN * ROLL_THREADS * CH * 4; }

// Forward (FLIP = false) and stride-1 input gradient (FLIP = true: taps mirrored, pad = ks-1-pad, the caller swaps the tensors).
template <int KS, int S, bool FLIP, int TX, int CH, bool WREG>
__global__ void __launch_bounds__(ROLL_THREADS) dw_roll_kernel(DwArgs a, const float* __restrict__ wt, int seg_rows, int segs) {
  constexpr int SPAN = (TX - 1) * S + KS, R = (KS + S - 1) / S, U = R * S;
  extern __shared__ __align__(16) uint8_t ring_raw[];
  const int cqn = a.c / CH, gx = (a.ow + TX - 1) / TX;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * segs * gx * cqn) return;
  int img, cq, seg, xg;
  decode<true>(i, cqn, segs, gx, img, cq, seg, xg);
  const int ch = cq * CH, ox0 = xg * TX;
  const int oy_begin = seg * seg_rows, nrows = min(seg_rows, a.oh - oy_begin);
  const int sy0 = oy_begin * S - a.pad, x0 = ox0 * S - a.pad;
  const int n_in = (nrows - 1) * S + KS;  // input rows the strip touches
  // pointer to input pixel (sy0, x0) of this thread's channels; only dereferenced where that pixel exists
  const float* xbase = a.x.p + (((int64_t)img * a.ih + sy0) * a.iw + x0) * a.c + ch;
  const int64_t rs = (int64_t)a.iw * a.c;
  const float* wq = wt + ch;
  Vec<CH> wreg[WREG ? KS * KS : 1];
  if constexpr (WREG) {
#pragma unroll
    for (int t = 0; t < KS * KS; t++) wreg[t] = ldv<CH>(wq + (FLIP ? KS * KS - 1 - t : t) * a.c);
  }
  Vec<CH> acc[R][TX];
#pragma unroll
  for (int q = 0; q < R; q++)
#pragma unroll
    for (int j = 0; j < TX; j++) acc[q][j] = zerov<CH>();
  Vec<CH> b = zerov<CH>();
  if (a.flags & OMT_EPI_BIAS) b = ldv<CH>(a.bias + ch);
  const bool relu = a.flags & OMT_EPI_RELU;
  float* ybase = a.y.p + (((int64_t)img * a.oh + oy_begin) * a.ow + ox0) * a.c + ch;
  const RowRing<CH, SPAN> ring{(uint32_t)__cvta_generic_to_shared(ring_raw) + threadIdx.x * CH * 4};
  auto row_valid = [&](int r) { return r < n_in && sy0 + r >= 0 && sy0 + r < a.ih; };
  const float* safe = a.x.p + ch;
#pragma unroll
  for (int d = 0; d < ROLL_DEPTH; d++) ring.request(d, row_valid(d), xbase + d * rs, safe, x0, a.iw, a.c);
  if constexpr (S == 1 && KS >= 5) {
    // Large filters: the walk unrolled over its R-row period is tens of KB of code, and the kernel then waits for instructions
    // (measured: 1.1 "no instruction" stalls per issue at 5x5). Here the loop body is ONE input row: acc[ky] holds the sums of
    // the output row that this input row is filter row ky of, and the sums move up one place per row (R * TX moves against
    // KS * KS * TX multiply-adds).
#pragma unroll 1
    for (int r = 0; r < n_in; r++) {
      ring.wait_oldest();
      const bool have = row_valid(r);
      Vec<CH> in[SPAN];
      if (have) ring.read(r, in);
      ring.request(r + ROLL_DEPTH, row_valid(r + ROLL_DEPTH), xbase + (r + ROLL_DEPTH) * rs, safe, x0, a.iw, a.c);
      if (have) {
#pragma unroll
        for (int ky = 0; ky < KS; ky++) {
          const int q = r - ky;
          if (q < 0 || q >= nrows) continue;
#pragma unroll
          for (int kx = 0; kx < KS; kx++) {
            const int t = FLIP ? (KS - 1 - ky) * KS + (KS - 1 - kx) : ky * KS + kx;
            const Vec<CH> wv = WREG ? wreg[ky * KS + kx] : ldv<CH>(wq + t * a.c);
#pragma unroll
            for (int j = 0; j < TX; j++) fmav<CH>(acc[ky][j], in[j + kx], wv);
          }
        }
      }
      const int q = r - (KS - 1);  // complete after this row
      if (q >= 0 && q < nrows) {
        float* yp = ybase + (int64_t)q * a.ow * a.c;
#pragma unroll
        for (int j = 0; j < TX; j++) {
          if (ox0 + j < a.ow) {
            Vec<CH> o;
#pragma unroll
            for (int k = 0; k < CH; k++) {
              o.v[k] = acc[KS - 1][j].v[k] + b.v[k];
              if (relu) o.v[k] = fmaxf(o.v[k], 0.f);
            }
            stv<CH>(yp + (int64_t)j * a.c, o);
          }
        }
      }
#pragma unroll
      for (int ky = KS - 1; ky > 0; ky--)
#pragma unroll
        for (int j = 0; j < TX; j++) acc[ky][j] = acc[ky - 1][j];
#pragma unroll
      for (int j = 0; j < TX; j++) acc[0][j] = zerov<CH>();
    }
    return;
  }
  for (int base = 0; base < n_in; base += U) {
    const int qb = base / S;  // output row (within the strip) whose first input row is `base`
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int r = base + u;
      if (r >= n_in) break;
      ring.wait_oldest();
      const bool have = row_valid(r);
      Vec<CH> in[SPAN];
      if (have) ring.read(r, in);
      ring.request(r + ROLL_DEPTH, row_valid(r + ROLL_DEPTH), xbase + (r + ROLL_DEPTH) * rs, safe, x0, a.iw, a.c);  // into the slot just read
      if (have) {
#pragma unroll
        for (int ky = 0; ky < KS; ky++) {
          if (pos_mod(u - ky, S) != 0) continue;  // (known at compile time once u and ky are unrolled)
          const int dq = floor_div(u - ky, S), slot = pos_mod(dq, R);
          const int q = qb + dq;  // input row r is filter row ky of output row q
          if (q < 0 || q >= nrows) continue;
#pragma unroll
          for (int kx = 0; kx < KS; kx++) {
            const int t = FLIP ? (KS - 1 - ky) * KS + (KS - 1 - kx) : ky * KS + kx;
            const Vec<CH> wv = WREG ? wreg[ky * KS + kx] : ldv<CH>(wq + t * a.c);
#pragma unroll
            for (int j = 0; j < TX; j++) fmav<CH>(acc[slot][j], in[j * S + kx], wv);
          }
        }
      }
      if (pos_mod(u - (KS - 1), S) == 0) {  // this was the last input row of an output row: store it, free its sums
        const int dq = floor_div(u - (KS - 1), S), slot = pos_mod(dq, R);
        const int q = qb + dq;
        if (q >= 0 && q < nrows) {
          float* yp = ybase + (int64_t)q * a.ow * a.c;
#pragma unroll
          for (int j = 0; j < TX; j++) {
            if (ox0 + j < a.ow) {
              Vec<CH> o;
#pragma unroll
              for (int k = 0; k < CH; k++) {
                o.v[k] = acc[slot][j].v[k] + b.v[k];
                if (relu) o.v[k] = fmaxf(o.v[k], 0.f);
              }
              stv<CH>(yp + (int64_t)j * a.c, o);
            }
            acc[slot][j] = zerov<CH>();
          }
        }
      }
    }
  }
}

// Input gradient of a stride-2 convolution: dx(yy, xx) sums the taps with ky = (yy + pad) mod 2, kx = (xx + pad) mod 2 (mod 2),
// gy pixel ((yy + pad - ky) / 2, (xx + pad - kx) / 2). A thread produces TX (even) consecutive pixels of one dx row: per
// tap row it loads the G gy pixels they share once; which of them pixel j pairs with tap kx is known at compile time up to
// the parity of the strip's first column, so no division or modulo is left per tap.
template <int KS, int TX, int CH>
__global__ void __launch_bounds__(256) dw_dgrad_s2_kernel(DwArgs a, const float* __restrict__ wt) {  // a.x = gy, a.y = dx
  constexpr int HALF = (KS - 1) / 2, G = HALF + TX / 2 + 1;
  const int cqn = a.c / CH, gx = (a.iw + TX - 1) / TX;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.ih * gx * cqn) return;
  int img, cq, yy, xg;
  decode<true>(i, cqn, a.ih, gx, img, cq, yy, xg);
  const int ch = cq * CH, x0 = xg * TX;
  const int e = x0 + a.pad, pe = e & 1, h = e >> 1, ey = yy + a.pad;
  const int ox_base = h - HALF;
  const float* gimg = a.x.p + (int64_t)img * a.oh * a.ow * a.c + ch;
  const float* wq = wt + ch;
  Vec<CH> acc[TX];
#pragma unroll
  for (int j = 0; j < TX; j++) acc[j] = zerov<CH>();
  const bool interior = ox_base >= 0 && ox_base + G <= a.ow;
  for (int ky = ey & 1; ky < KS; ky += 2) {
    if (ey < ky) break;
    const int oy = (ey - ky) >> 1;
    if (oy >= a.oh) continue;
    Vec<CH> g[G];
    load_span<CH, G>(g, gimg + ((int64_t)oy * a.ow + ox_base) * a.c, ox_base, a.ow, a.c, interior);
    const float* wr = wq + (int64_t)ky * KS * a.c;
    auto taps = [&](auto parity) {
      constexpr int PE = decltype(parity)::value;
#pragma unroll
      for (int j = 0; j < TX; j++) {
#pragma unroll
        for (int m = 0; m <= HALF; m++) {
          const int kx = ((PE + j) & 1) + 2 * m;
          if (kx >= KS) continue;
          fmav<CH>(acc[j], g[HALF + ((PE + j) >> 1) - m], ldv<CH>(wr + kx * a.c));
        }
      }
    };
    if (pe) taps(std::integral_constant<int, 1>{});
    else taps(std::integral_constant<int, 0>{});
  }
  float* yp = a.y.p + (((int64_t)img * a.ih + yy) * a.iw + x0) * a.c + ch;
#pragma unroll
  for (int j = 0; j < TX; j++)
    if (x0 + j < a.iw) stv<CH>(yp + (int64_t)j * a.c, acc[j]);
}

// Weight gradient, rolling: a (channel group, pixel lane) thread walks strips of TX columns x seg_rows output rows; an input row
// is loaded once and meets the R gy rows it overlaps (kept in registers), every tap's sum stays in registers for the
// whole walk. Pixel lanes are summed through shared memory in a fixed order, slices (blockIdx.y) by dw_wgrad_fin_kernel.
template <int KS, int S, int TX, int CH>
__global__ void __launch_bounds__(ROLL_THREADS) dw_wgrad_roll_kernel(DwArgs a, int SL, int CL, int seg_rows, int segs, float* __restrict__ part) {
  constexpr int SPAN = (TX - 1) * S + KS, R = (KS + S - 1) / S, U = R * S;
  extern __shared__ __align__(16) uint8_t ring_raw[];  // the row ring; after the walk its start is reused as [PL][CL] vectors of CH floats
  const int PL = blockDim.x / CL;
  const int cl = threadIdx.x % CL, pl = threadIdx.x / CL;
  const int cq = blockIdx.x * CL + cl, sl = blockIdx.y;
  const bool live = pl < PL && cq < a.c / CH;
  const int ch = cq * CH;
  Vec<CH> acc[KS * KS];
#pragma unroll
  for (int t = 0; t < KS * KS; t++) acc[t] = zerov<CH>();
  if (live) {
    const uint32_t gx = (uint32_t)(a.ow + TX - 1) / TX;
    const uint32_t items = (uint32_t)a.n * segs * gx;
    const int64_t rs = (int64_t)a.iw * a.c;
    const RowRing<CH, SPAN> ring{(uint32_t)__cvta_generic_to_shared(ring_raw) + threadIdx.x * CH * 4};
    const float* safe = a.x.p + ch;
    for (uint32_t it = (uint32_t)sl * PL + pl; it < items; it += (uint32_t)SL * PL) {
      const uint32_t xg = it % gx, r_ = it / gx;
      const int seg = (int)(r_ % (uint32_t)segs), img = (int)(r_ / (uint32_t)segs);
      const int ox0 = (int)xg * TX, oy_begin = seg * seg_rows, nrows = min(seg_rows, a.oh - oy_begin);
      const int sy0 = oy_begin * S - a.pad, x0 = ox0 * S - a.pad;
      const int n_in = (nrows - 1) * S + KS;
      const float* xbase = a.x.p + (((int64_t)img * a.ih + sy0) * a.iw + x0) * a.c + ch;
      const float* gbase = a.y.p + (((int64_t)img * a.oh + oy_begin) * a.ow + ox0) * a.c + ch;
      const bool gfull = ox0 + TX <= a.ow;
      Vec<CH> g[R][TX];
      auto row_valid = [&](int r) { return r < n_in && sy0 + r >= 0 && sy0 + r < a.ih; };
#pragma unroll
      for (int d = 0; d < ROLL_DEPTH; d++) ring.request(d, row_valid(d), xbase + d * rs, safe, x0, a.iw, a.c);
      if constexpr (S == 1 && KS >= 5) {  // one input row per trip, g[ky] = the gy row this input row is filter row ky of (see dw_roll_kernel)
#pragma unroll 1
        for (int r = 0; r < n_in; r++) {
#pragma unroll
          for (int ky = KS - 1; ky > 0; ky--)
#pragma unroll
            for (int j = 0; j < TX; j++) g[ky][j] = g[ky - 1][j];
          if (r < nrows) load_span<CH, TX>(g[0], gbase + (int64_t)r * a.ow * a.c, ox0, a.ow, a.c, gfull);
          ring.wait_oldest();
          const bool have = row_valid(r);
          Vec<CH> in[SPAN];
          if (have) ring.read(r, in);
          ring.request(r + ROLL_DEPTH, row_valid(r + ROLL_DEPTH), xbase + (r + ROLL_DEPTH) * rs, safe, x0, a.iw, a.c);
          if (!have) continue;
#pragma unroll
          for (int ky = 0; ky < KS; ky++) {
            const int q = r - ky;
            if (q < 0 || q >= nrows) continue;
#pragma unroll
            for (int kx = 0; kx < KS; kx++)
#pragma unroll
              for (int j = 0; j < TX; j++) fmav<CH>(acc[ky * KS + kx], g[ky][j], in[j + kx]);
          }
        }
        continue;
      }
      for (int base = 0; base < n_in; base += U) {
        const int qb = base / S;
#pragma unroll
        for (int u = 0; u < U; u++) {
          const int r = base + u;
          if (r >= n_in) break;
          if (u % S == 0) {  // the first input row of output row q: its gy pixels enter the ring
            const int dq = u / S, slot = dq % R, q = qb + dq;
            if (q < nrows) load_span<CH, TX>(g[slot], gbase + (int64_t)q * a.ow * a.c, ox0, a.ow, a.c, gfull);
          }
          ring.wait_oldest();
          const bool have = row_valid(r);
          Vec<CH> in[SPAN];
          if (have) ring.read(r, in);
          ring.request(r + ROLL_DEPTH, row_valid(r + ROLL_DEPTH), xbase + (r + ROLL_DEPTH) * rs, safe, x0, a.iw, a.c);
          if (!have) continue;
#pragma unroll
          for (int ky = 0; ky < KS; ky++) {
            if (pos_mod(u - ky, S) != 0) continue;
            const int dq = floor_div(u - ky, S), slot = pos_mod(dq, R);
            const int q = qb + dq;
            if (q < 0 || q >= nrows) continue;
#pragma unroll
            for (int kx = 0; kx < KS; kx++)
#pragma unroll
              for (int j = 0; j < TX; j++) fmav<CH>(acc[ky * KS + kx], g[slot][j], in[j * S + kx]);
          }
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");  // (only empty groups can be pending here)
  Vec<CH>* red = reinterpret_cast<Vec<CH>*>(ring_raw);
#pragma unroll
  for (int t = 0; t < KS * KS; t++) {
    __syncthreads();
    if (pl < PL) red[pl * CL + cl] = acc[t];
    __syncthreads();
    if (pl == 0 && live) {
      Vec<CH> s4 = red[cl];
      for (int k = 1; k < PL; k++) {
        const Vec<CH> v = red[k * CL + cl];
#pragma unroll
        for (int e = 0; e < CH; e++) s4.v[e] += v.v[e];
      }
      const int kk = KS * KS;
#pragma unroll
      for (int e = 0; e < CH; e++) part[((int64_t)(ch + e) * SL + sl) * kk + t] = s4.v[e];
    }
  }
}

static int check_geo(const OmtConvGeo* g, const char* who) {
  OMT_REQUIRE(g && g->groups == g->ci && g->ci == g->co && g->ci >= 1, "%s: depthwise needs groups == ci == co", who);
  OMT_REQUIRE(g->ks >= 1 && g->ks <= 11 && g->stride >= 1 && g->stride <= 4 && g->pad >= 0 && g->pad <= g->ks,
              "%s: ks<=11, stride 1..4, pad<=ks", who);
  OMT_REQUIRE(g->oh == (g->ih + 2 * g->pad - g->ks) / g->stride + 1 && g->ow == (g->iw + 2 * g->pad - g->ks) / g->stride + 1 &&
                  g->oh > 0 && g->ow > 0 && g->n > 0,
              "%s: inconsistent output size", who);
  return OMT_OK;
}
static DwArgs mk(const OmtConvGeo* g, const OmtAct* x, const OmtAct* y, const float* w, const float* bias, uint32_t flags) {
  DwArgs a{};
  a.x = view(x); a.y = view(y); a.w = w; a.bias = bias;
  a.n = g->n; a.c = g->ci; a.ih = g->ih; a.iw = g->iw; a.oh = g->oh; a.ow = g->ow; a.ks = g->ks; a.stride = g->stride; a.pad = g->pad;
  a.flags = flags;
  return a;
}
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static bool rows_ok(const OmtConvGeo* g) { return (g->ks == 3 || g->ks == 5 || g->ks == 7) && (g->stride == 1 || g->stride == 2); }
// strips of the rolling kernels: as tall as possible (a strip re-reads ks - stride input rows of its upper neighbour) while
// the launch still has `want` work items; returns rows per strip, sets the strips per column
static int strip_rows(int oh, int ks, int64_t items_per_seg, int64_t want, int& segs) {
  const int64_t by_work = std::max<int64_t>(1, cdiv(want, std::max<int64_t>(1, items_per_seg)));
  const int most = std::max(1, oh / std::min(oh, ks + 1));  // no strip shorter than ks + 1 rows (unless the image is)
  const int rows = (int)cdiv(oh, std::min<int64_t>(by_work, most));
  segs = (int)cdiv(oh, rows);
  return rows;
}
// the rolling kernels' rings can exceed the 48 KB a kernel gets without asking; once per kernel
template <auto Kernel>
static void allow_shared_memory(size_t bytes) {
  static std::once_flag once;
  std::call_once(once, [bytes] {
    if (cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess) cudaGetLastError();  // (the launch reports it)
  });
}
template <int KS, int S, bool FLIP>
static void launch_roll(const DwArgs& a, const float* wt, cudaStream_t s) {
  constexpr int CH = KS == 3 ? 4 : 2, TX = 4, SPAN = (TX - 1) * S + KS;
  constexpr bool WREG = KS <= 5;  // the filter in registers: no loads but the input rows inside the walk
  const int64_t per_seg = (int64_t)a.n * cdiv(a.ow, TX) * (a.c / CH);
  int segs;
  const int rows = strip_rows(a.oh, KS, per_seg, (int64_t)sm_count() * 1536, segs);
  constexpr size_t smem = ring_bytes<CH, SPAN>();
  allow_shared_memory<dw_roll_kernel<KS, S, FLIP, TX, CH, WREG>>(smem);
  dw_roll_kernel<KS, S, FLIP, TX, CH, WREG><<<(unsigned)cdiv(per_seg * segs, ROLL_THREADS), ROLL_THREADS, smem, s>>>(a, wt, rows, segs);
}
template <int KS, int S, int TX, int CH>
static void launch_wgrad_roll(const DwArgs& a, dim3 grid, int SL, int CL, int rows, int segs, float* part, cudaStream_t s) {
  constexpr size_t smem = ring_bytes<CH, (TX - 1) * S + KS>();
  allow_shared_memory<dw_wgrad_roll_kernel<KS, S, TX, CH>>(smem);
  dw_wgrad_roll_kernel<KS, S, TX, CH><<<grid, ROLL_THREADS, smem, s>>>(a, SL, CL, rows, segs, part);
}
// Which kernel serves which case (measured on 128 x 96 x 56 x 56 and 64 x 96 x 112 x 112 -> 56 x 56, fraction of the copy
// bandwidth): stride 1, 3x3 and 5x5: the rolling kernel (3x3: 0.75 against 0.66); stride 2 and 7x7: one output row per thread
// (3x3 stride 2: 0.82 against 0.62 -- half of a strip's input rows serve one output row only, the ring buys nothing).
template <int KS, bool FLIP>
static void launch_rows_ks(const DwArgs& a, int stride, const float* wt, cudaStream_t s) {
  if (stride == 1 && KS <= 5) return launch_roll<KS == 7 ? 5 : KS, 1, FLIP>(a, wt, s);
  const int64_t total = (int64_t)a.n * a.oh * cdiv(a.ow, 4) * (a.c / 4);
  const unsigned blocks = (unsigned)cdiv(total, 256);
  if (stride == 1) dw_rows_nhwc4_kernel<KS, 1, FLIP, 4><<<blocks, 256, 0, s>>>(a, wt);
  else dw_rows_nhwc4_kernel<KS, 2, FLIP, 4><<<blocks, 256, 0, s>>>(a, wt);
}
// `a` describes the convolution the kernel performs (for the flipped input gradient: gy -> dx with stride 1)
static int launch_rows(const DwArgs& a, const OmtConvGeo* g, float* wt, bool flip, cudaStream_t s, const char* name) {
  const int kk = g->ks * g->ks;
  dw_weight_tc_kernel<<<(unsigned)cdiv((int64_t)a.c * kk, 256), 256, 0, s>>>(a.w, wt, a.c, kk);
  const int stride = flip ? 1 : g->stride;
  if (flip) {
    if (g->ks == 3) launch_rows_ks<3, true>(a, stride, wt, s);
    else if (g->ks == 5) launch_rows_ks<5, true>(a, stride, wt, s);
    else launch_rows_ks<7, true>(a, stride, wt, s);
  } else {
    if (g->ks == 3) launch_rows_ks<3, false>(a, stride, wt, s);
    else if (g->ks == 5) launch_rows_ks<5, false>(a, stride, wt, s);
    else launch_rows_ks<7, false>(a, stride, wt, s);
  }
  return check_launch(name);
}

}  // namespace omt

using namespace omt;

extern "C" {

int omt_dw_fwd(const OmtConvGeo* g, const OmtAct* x, const float* w, const float* bias, const OmtAct* y, uint32_t flags,
               omt_stream_t stream) {
  int r = check_geo(g, "omt_dw_fwd");
  if (r) return r;
  OMT_REQUIRE(x && y && x->p && y->p && w && (!(flags & OMT_EPI_BIAS) || bias), "omt_dw_fwd: null pointer");
  DwArgs a = mk(g, x, y, w, bias, flags);
  bool xn = is_nhwc(x, g->ci, g->ih, g->iw), yn = is_nhwc(y, g->co, g->oh, g->ow);
  int64_t total = (int64_t)g->n * g->co * g->oh * g->ow;
  if (xn && yn && g->ci % 4 == 0 && aligned16(x->p) && aligned16(y->p) && (!bias || aligned16(bias))) {
    if (rows_ok(g)) {
      Scratch sc;
      r = sc.get(nullptr, 0, (size_t)g->ci * g->ks * g->ks * sizeof(float), stream);
      if (r) return r;
      return launch_rows(a, g, (float*)sc.p, false, st(stream), "dw_fwd_rows_nhwc4");
    }
    dw_fwd_nhwc4_kernel<<<(unsigned)cdiv(total / 4, 256), 256, 0, st(stream)>>>(a);
    return check_launch("dw_fwd_nhwc4");
  }
  if (yn) dw_fwd_kernel<true><<<(unsigned)cdiv(total, 256), 256, 0, st(stream)>>>(a);
  else dw_fwd_kernel<false><<<(unsigned)cdiv(total, 256), 256, 0, st(stream)>>>(a);
  return check_launch("dw_fwd");
}

int omt_dw_dgrad(const OmtConvGeo* g, const OmtAct* gy, const float* w, const OmtAct* dx, omt_stream_t stream) {
  int r = check_geo(g, "omt_dw_dgrad");
  if (r) return r;
  OMT_REQUIRE(gy && dx && gy->p && dx->p && w, "omt_dw_dgrad: null pointer");
  DwArgs a = mk(g, gy, dx, w, nullptr, 0);
  int64_t total = (int64_t)g->n * g->ci * g->ih * g->iw;
  if (g->ci % 4 == 0 && is_nhwc(dx, g->ci, g->ih, g->iw) && is_nhwc(gy, g->ci, g->oh, g->ow) && aligned16(gy->p) && aligned16(dx->p)) {
    Scratch sc;
    r = sc.get(nullptr, 0, (size_t)g->ci * g->ks * g->ks * sizeof(float), stream);
    if (r) return r;
    if (g->stride == 1 && rows_ok(g) && g->pad <= g->ks - 1) {
      // stride 1: the forward kernel over gy with mirrored taps and padding ks-1-pad, producing the ih x iw grid
      DwArgs f = a;
      f.ih = g->oh; f.iw = g->ow; f.oh = g->ih; f.ow = g->iw; f.pad = g->ks - 1 - g->pad;
      return launch_rows(f, g, (float*)sc.p, true, st(stream), "dw_dgrad_rows_nhwc4");
    }
    const int kk = g->ks * g->ks;
    dw_weight_tc_kernel<<<(unsigned)cdiv((int64_t)g->ci * kk, 256), 256, 0, st(stream)>>>(w, (float*)sc.p, g->ci, kk);
    if (g->stride == 2 && rows_ok(g)) {
      const int64_t threads = (int64_t)g->n * g->ih * cdiv(g->iw, 4) * (g->ci / 4);
      const unsigned blocks = (unsigned)cdiv(threads, 256);
      if (g->ks == 3) dw_dgrad_s2_kernel<3, 4, 4><<<blocks, 256, 0, st(stream)>>>(a, (const float*)sc.p);
      else if (g->ks == 5) dw_dgrad_s2_kernel<5, 4, 4><<<blocks, 256, 0, st(stream)>>>(a, (const float*)sc.p);
      else dw_dgrad_s2_kernel<7, 4, 4><<<blocks, 256, 0, st(stream)>>>(a, (const float*)sc.p);
      return check_launch("dw_dgrad_s2_nhwc4");
    }
    dw_dgrad_nhwc4_kernel<<<(unsigned)cdiv(total / 4, 256), 256, 0, st(stream)>>>(a, (const float*)sc.p);
    return check_launch("dw_dgrad_nhwc4");
  }
  if (is_nhwc(dx, g->ci, g->ih, g->iw)) dw_dgrad_kernel<true><<<(unsigned)cdiv(total, 256), 256, 0, st(stream)>>>(a);
  else dw_dgrad_kernel<false><<<(unsigned)cdiv(total, 256), 256, 0, st(stream)>>>(a);
  return check_launch("dw_dgrad");
}

int omt_dw_wgrad(const OmtConvGeo* g, const OmtAct* x, const OmtAct* gy, float* dw, float scale, omt_stream_t stream) {
  int r = check_geo(g, "omt_dw_wgrad");
  if (r) return r;
  OMT_REQUIRE(x && gy && x->p && gy->p && dw, "omt_dw_wgrad: null pointer");
  DwArgs a = mk(g, x, gy, nullptr, nullptr, 0);
  cudaStream_t s = st(stream);
  const int c = g->ci, kk = g->ks * g->ks;
  const bool nhwc = is_nhwc(x, c, g->ih, g->iw) && is_nhwc(gy, c, g->oh, g->ow) && c >= 32;
  const bool reg = g->ks == 3 || g->ks == 5 || g->ks == 7;
  if (is_nhwc(x, c, g->ih, g->iw) && is_nhwc(gy, c, g->oh, g->ow) && c % 4 == 0 && (g->ks == 3 || g->ks == 5) && g->stride <= 2 &&
      aligned16(x->p) && aligned16(gy->p)) {
    float* part = nullptr;
    int S = 1;
    Scratch sc;
    if (g->stride == 1) {
      // rolling strips; 4 channels per thread for 3x3, 2 for 5x5 (25 tap sums per channel)
      const int CH = g->ks == 3 ? 4 : 2, TX = 4;
      const int cqn = c / CH;
      const int CL = std::min(cqn, 32), PL = ROLL_THREADS / CL;
      const int gx = (int)cdiv(cqn, CL);
      const int64_t per_seg = (int64_t)g->n * cdiv(g->ow, TX);
      // three resident blocks per SM; strips short enough that every pixel lane walks at least four of them
      S = (int)std::max<int64_t>(1, cdiv(3 * sm_count(), gx));
      int segs;
      const int rows = strip_rows(g->oh, g->ks, per_seg, (int64_t)4 * S * PL, segs);
      S = (int)std::max<int64_t>(1, std::min<int64_t>(S, cdiv(per_seg * segs, PL)));
      r = sc.get(nullptr, 0, (size_t)c * S * kk * sizeof(float), stream);
      if (r) return r;
      part = (float*)sc.p;
      dim3 grid(gx, S);
      if (g->ks == 3) launch_wgrad_roll<3, 1, 4, 4>(a, grid, S, CL, rows, segs, part, s);
      else launch_wgrad_roll<5, 1, 4, 2>(a, grid, S, CL, rows, segs, part, s);
    } else {  // stride 2: a group of four output pixels per trip (measured 0.77 of the copy bandwidth against 0.61 for strips)
      const int c4 = c / 4;
      const int CL = std::min(c4, 32), PL = 256 / CL;
      const int gx = (int)cdiv(c4, CL);
      const int64_t items = (int64_t)g->n * g->oh * cdiv(g->ow, 4);
      S = (int)std::max<int64_t>(1, std::min<int64_t>(cdiv(items, (int64_t)PL * 4), cdiv(4 * sm_count(), gx)));
      r = sc.get(nullptr, 0, (size_t)c * S * kk * sizeof(float), stream);
      if (r) return r;
      part = (float*)sc.p;
      dim3 grid(gx, S);
      const size_t smem = (size_t)PL * CL * sizeof(float4);
      if (g->ks == 3) dw_wgrad_nhwc4_kernel<3, 2><<<grid, 256, smem, s>>>(a, S, CL, part);
      else dw_wgrad_nhwc4_kernel<5, 2><<<grid, 256, smem, s>>>(a, S, CL, part);
    }
    r = check_launch(g->stride == 1 ? "dw_wgrad_strips_nhwc" : "dw_wgrad_nhwc4");
    if (r) return r;
    const int64_t total = (int64_t)c * kk;
    dw_wgrad_fin_kernel<<<(unsigned)cdiv(total * 32, 256), 256, 0, s>>>(part, total, kk, S, scale, dw);
    return check_launch("dw_wgrad_fin");
  }
  int S;
  if (nhwc && reg) {
    int64_t P = (int64_t)g->n * g->oh * g->ow;
    S = (int)std::max<int64_t>(1, std::min<int64_t>(P / 16 + 1, cdiv(8 * sm_count(), cdiv(c, 128))));
  } else {
    S = (int)std::max<int64_t>(1, std::min<int64_t>(g->n, cdiv(4 * sm_count(), c)));
  }
  Scratch sc;
  r = sc.get(nullptr, 0, (size_t)c * S * kk * sizeof(float), stream);
  if (r) return r;
  float* part = (float*)sc.p;
  if (nhwc && reg) {
    dim3 grid((unsigned)cdiv(c, 128), S);
    if (g->ks == 3) dw_wgrad_nhwc_kernel<3><<<grid, 128, 0, s>>>(a, S, part);
    else if (g->ks == 5) dw_wgrad_nhwc_kernel<5><<<grid, 128, 0, s>>>(a, S, part);
    else dw_wgrad_nhwc_kernel<7><<<grid, 128, 0, s>>>(a, S, part);
    r = check_launch("dw_wgrad_nhwc");
  } else if (reg) {
    dim3 grid(c, S);
    if (g->ks == 3) dw_wgrad_nchw_kernel<3><<<grid, 256, 0, s>>>(a, S, part);
    else if (g->ks == 5) dw_wgrad_nchw_kernel<5><<<grid, 256, 0, s>>>(a, S, part);
    else dw_wgrad_nchw_kernel<7><<<grid, 256, 0, s>>>(a, S, part);
    r = check_launch("dw_wgrad_nchw");
  } else {
    dim3 grid(c, S, kk);
    dw_wgrad_tap_kernel<<<grid, 256, 0, s>>>(a, S, part);
    r = check_launch("dw_wgrad_tap");
  }
  if (r) return r;
  int64_t total = (int64_t)c * kk;
  dw_wgrad_fin_kernel<<<(unsigned)cdiv(total * 32, 256), 256, 0, s>>>(part, total, kk, S, scale, dw);
  return check_launch("dw_wgrad_fin");
}

}  // extern "C"

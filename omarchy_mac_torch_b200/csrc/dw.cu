// Depthwise convolution (groups == channels): forward, input gradient, weight gradient, for any ks <= 11,
// stride 1..4, pad <= ks. HBM-bound kernels: each activation element is fetched from DRAM once (neighbouring taps
// hit L1/L2), outputs are written with coalesced (NCHW: along x; channels-last: 128-bit along c) stores, and the
// weight gradient keeps all ks*ks tap sums of a channel in registers so x and gy are read once, not ks*ks times.
//
// Semantics: reference dw_fwd/dw_gin/dw_gwt (stride 1, "same" padding) and dwg_fwd/dwg_gin/dwg_gwt (general) in
// csrc/kernels/, dispatched from csrc/conv.cpp:194-229. One code path covers both families here.
#include <algorithm>

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
template <int KS, bool FLIP>
static void launch_rows_ks(const DwArgs& a, int stride, const float* wt, cudaStream_t s) {
  // 8 output pixels per thread for 3x3 stride 1 on wide rows (fewer redundant input and weight loads), else 4
  const bool wide = KS == 3 && stride == 1 && a.ow >= 16;
  const int tx = wide ? 8 : 4;
  const int64_t total = (int64_t)a.n * a.oh * cdiv(a.ow, tx) * (a.c / 4);
  const unsigned blocks = (unsigned)cdiv(total, 256);
  if (wide) dw_rows_nhwc4_kernel<KS == 3 ? 3 : KS, 1, FLIP, KS == 3 ? 8 : 4><<<blocks, 256, 0, s>>>(a, wt);
  else if (stride == 1) dw_rows_nhwc4_kernel<KS, 1, FLIP, 4><<<blocks, 256, 0, s>>>(a, wt);
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
    const int c4 = c / 4;
    const int CL = std::min(c4, 32), PL = 256 / CL;
    const int gx = (int)cdiv(c4, CL);
    const int64_t items = (int64_t)g->n * g->oh * cdiv(g->ow, 4);
    const int S = (int)std::max<int64_t>(1, std::min<int64_t>(cdiv(items, (int64_t)PL * 4), cdiv(4 * sm_count(), gx)));
    Scratch sc;
    r = sc.get(nullptr, 0, (size_t)c * S * kk * sizeof(float), stream);
    if (r) return r;
    float* part = (float*)sc.p;
    dim3 grid(gx, S);
    const size_t smem = (size_t)PL * CL * sizeof(float4);
    if (g->ks == 3 && g->stride == 1) dw_wgrad_nhwc4_kernel<3, 1><<<grid, 256, smem, s>>>(a, S, CL, part);
    else if (g->ks == 3) dw_wgrad_nhwc4_kernel<3, 2><<<grid, 256, smem, s>>>(a, S, CL, part);
    else if (g->stride == 1) dw_wgrad_nhwc4_kernel<5, 1><<<grid, 256, smem, s>>>(a, S, CL, part);
    else dw_wgrad_nhwc4_kernel<5, 2><<<grid, 256, smem, s>>>(a, S, CL, part);
    r = check_launch("dw_wgrad_nhwc4");
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

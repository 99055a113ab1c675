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
__global__ void dw_wgrad_fin_kernel(const float* __restrict__ part, int64_t total, int kk, int S, float scale, float* out) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // i = ch*kk + t
  if (i >= total) return;
  int64_t ch = i / kk;
  int t = (int)(i - ch * kk);
  float s = 0.f;
  for (int k = 0; k < S; k++) s += part[(ch * S + k) * kk + t];
  out[i] = s * scale;
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
  dw_wgrad_fin_kernel<<<(unsigned)cdiv(total, 256), 256, 0, s>>>(part, total, kk, S, scale, dw);
  return check_launch("dw_wgrad_fin");
}

}  // extern "C"

// Pooling kernels: the plan's 2x2 max / average pools and global average pool, and the general aten pools.
// All HBM-bound, one thread per output (forward) or per input (backward gather), indexed in memory order of the
// written tensor so stores coalesce for both NCHW and channels-last.
//
// Semantics: pool_fwd.wgsl:15-21 / pool_bwd.wgsl:14-21 (index 0..3, first maximum wins), avgpool_fwd/bwd.wgsl,
// gap_fwd/bwd.wgsl, maxpool_gen_fwd.wgsl:16-28 (int64 flat index, NaN propagates) / maxpool_gen_bwd.wgsl,
// avgpool_gen_fwd/bwd.wgsl (aten divisor rules), adapool_fwd/bwd.wgsl; host side csrc/nn.cpp:137-222 and
// csrc/plans.cpp:188-213.
#include "common.cuh"

namespace omt {

// index -> (img, ch, y, x) in memory order of the layout; 32-bit arithmetic whenever the index fits (64-bit division is
// emulated and would dominate these bandwidth-bound kernels)
template <bool NHWC, class I>
__device__ __forceinline__ void decode4_t(I i, int c, int h, int w, int& img, int& ch, int& y, int& x) {
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
__device__ __forceinline__ void decode4(int64_t i, int c, int h, int w, int& img, int& ch, int& y, int& x) {
  if (i < 0x7fffffffll) decode4_t<NHWC, uint32_t>((uint32_t)i, c, h, w, img, ch, y, x);
  else decode4_t<NHWC, int64_t>(i, c, h, w, img, ch, y, x);
}

// ---- 2x2 stride-2 max pool with 2-bit argmax ----
template <bool NHWC>
__global__ void __launch_bounds__(256) pool2_fwd_kernel(ActView x, ActView y, uint8_t* idx, int n, int c, int oh, int ow) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)n * c * oh * ow) return;
  int img, ch, oy, ox;
  decode4<NHWC>(i, c, oh, ow, img, ch, oy, ox);
  const float* p = x.p + x.off(img, ch, 2 * oy, 2 * ox);
  float best = __ldg(p);
  int bi = 0;
  float v1 = __ldg(p + x.sw); if (v1 > best) { best = v1; bi = 1; }
  float v2 = __ldg(p + x.sh); if (v2 > best) { best = v2; bi = 2; }
  float v3 = __ldg(p + x.sh + x.sw); if (v3 > best) { best = v3; bi = 3; }
  int64_t o = y.off(img, ch, oy, ox);
  y.p[o] = best;
  idx[o] = (uint8_t)bi;
}
template <bool NHWC>
__global__ void __launch_bounds__(256) pool2_bwd_kernel(ActView g, const uint8_t* idx, ActView gx, int n, int c, int h, int w,
                                                        int oh, int ow) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)n * c * h * w) return;
  int img, ch, yy, xx;
  decode4<NHWC>(i, c, h, w, img, ch, yy, xx);
  int oy = yy >> 1, ox = xx >> 1;
  float v = 0.f;
  if (oy < oh && ox < ow) {
    int64_t o = g.off(img, ch, oy, ox);
    if (idx[o] == (uint8_t)((yy & 1) * 2 + (xx & 1))) v = __ldg(g.p + o);
  }
  gx.p[gx.off(img, ch, yy, xx)] = v;
}
template <bool NHWC>
__global__ void __launch_bounds__(256) avgpool2_fwd_kernel(ActView x, ActView y, int n, int c, int oh, int ow) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)n * c * oh * ow) return;
  int img, ch, oy, ox;
  decode4<NHWC>(i, c, oh, ow, img, ch, oy, ox);
  const float* p = x.p + x.off(img, ch, 2 * oy, 2 * ox);
  y.p[y.off(img, ch, oy, ox)] = (__ldg(p) + __ldg(p + x.sw) + __ldg(p + x.sh) + __ldg(p + x.sh + x.sw)) * 0.25f;
}
template <bool NHWC>
__global__ void __launch_bounds__(256) avgpool2_bwd_kernel(ActView g, ActView gx, int n, int c, int h, int w, int oh, int ow) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)n * c * h * w) return;
  int img, ch, yy, xx;
  decode4<NHWC>(i, c, h, w, img, ch, yy, xx);
  int oy = yy >> 1, ox = xx >> 1;
  gx.p[gx.off(img, ch, yy, xx)] = (oy < oh && ox < ow) ? __ldg(g.p + g.off(img, ch, oy, ox)) * 0.25f : 0.f;
}

// ---- general max pool ----
struct PoolArgs {
  ActView x, y;
  int n, c, ih, iw, oh, ow;
  OmtPool p;
  int include_pad, divisor;
};
__device__ __forceinline__ bool isnan_bits(float v) { return (__float_as_uint(v) & 0x7fffffffu) > 0x7f800000u; }

template <bool NHWC>
__global__ void __launch_bounds__(256) maxpool_fwd_kernel(PoolArgs a, int64_t* idx) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.c * a.oh * a.ow) return;
  int img, ch, oy, ox;
  decode4<NHWC>(i, a.c, a.oh, a.ow, img, ch, oy, ox);
  const float* xp = a.x.p + img * a.x.sn + ch * a.x.sc;
  float best = -INFINITY;
  int bi = -1;
  bool done = false;
  for (int ky = 0; ky < a.p.kh && !done; ky++) {
    int y = oy * a.p.sh + ky * a.p.dh - a.p.ph;
    if (y < 0 || y >= a.ih) continue;
    for (int kx = 0; kx < a.p.kw; kx++) {
      int xx = ox * a.p.sw + kx * a.p.dw - a.p.pw;
      if (xx < 0 || xx >= a.iw) continue;
      float v = __ldg(xp + y * a.x.sh + xx * a.x.sw);
      bool nan = isnan_bits(v);
      if (bi < 0 || nan || v > best) {
        best = v; bi = y * a.iw + xx;
        if (nan) { done = true; break; }
      }
    }
  }
  int64_t o = a.y.off(img, ch, oy, ox);
  a.y.p[o] = best;
  idx[o] = bi;
}
template <bool NHWC>
__global__ void __launch_bounds__(256) maxpool_bwd_kernel(PoolArgs a, const int64_t* idx) {
  // a.x = gy (strides of the forward output), a.y = gx
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.c * a.ih * a.iw) return;
  int img, ch, y, xx;
  decode4<NHWC>(i, a.c, a.ih, a.iw, img, ch, y, xx);
  // outputs whose window can contain (y, xx)
  int ylo = max(0, (y + a.p.ph - (a.p.kh - 1) * a.p.dh + a.p.sh - 1) / a.p.sh), yhi = min(a.oh - 1, (y + a.p.ph) / a.p.sh);
  int xlo = max(0, (xx + a.p.pw - (a.p.kw - 1) * a.p.dw + a.p.sw - 1) / a.p.sw), xhi = min(a.ow - 1, (xx + a.p.pw) / a.p.sw);
  int64_t me = (int64_t)y * a.iw + xx;
  float acc = 0.f;
  for (int oy = ylo; oy <= yhi; oy++)
    for (int ox = xlo; ox <= xhi; ox++) {
      int64_t o = a.x.off(img, ch, oy, ox);
      if (idx[o] == me) acc += __ldg(a.x.p + o);
    }
  a.y.p[a.y.off(img, ch, y, xx)] = acc;
}

// Channels-last, 4 channels per thread (c % 4 == 0, dense tensors): 128-bit loads and stores, two 128-bit index accesses.
// x / gx are [n, ih, iw, c], y / gy / idx are [n, oh, ow, c].
__global__ void __launch_bounds__(256) maxpool_fwd_nhwc4_kernel(PoolArgs a, int64_t* __restrict__ idx) {
  const int c4 = a.c >> 2;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.oh * a.ow * c4) return;
  int img, cq, oy, ox;
  decode4<true>(i, c4, a.oh, a.ow, img, cq, oy, ox);
  const float* xp = a.x.p + ((int64_t)img * a.ih * a.iw) * a.c + cq * 4;
  float best[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
  int bi[4] = {-1, -1, -1, -1};
  bool done[4] = {false, false, false, false};
  for (int ky = 0; ky < a.p.kh; ky++) {
    const int y = oy * a.p.sh + ky * a.p.dh - a.p.ph;
    if (y < 0 || y >= a.ih) continue;
    for (int kx = 0; kx < a.p.kw; kx++) {
      const int xx = ox * a.p.sw + kx * a.p.dw - a.p.pw;
      if (xx < 0 || xx >= a.iw) continue;
      const float4 v4 = __ldg(reinterpret_cast<const float4*>(xp + ((int64_t)y * a.iw + xx) * a.c));
      const float v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const bool nan = isnan_bits(v[k]);
        if (!done[k] && (bi[k] < 0 || nan || v[k] > best[k])) {
          best[k] = v[k]; bi[k] = y * a.iw + xx;
          done[k] = nan;  // the first NaN of the window wins
        }
      }
    }
  }
  const int64_t o = (((int64_t)img * a.oh + oy) * a.ow + ox) * a.c + cq * 4;
  *reinterpret_cast<float4*>(a.y.p + o) = make_float4(best[0], best[1], best[2], best[3]);
  longlong2* ip = reinterpret_cast<longlong2*>(idx + o);
  ip[0] = make_longlong2(bi[0], bi[1]);
  ip[1] = make_longlong2(bi[2], bi[3]);
}
__global__ void __launch_bounds__(256) maxpool_bwd_nhwc4_kernel(PoolArgs a, const int64_t* __restrict__ idx) {
  // a.x = gy, a.y = gx
  const int c4 = a.c >> 2;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.ih * a.iw * c4) return;
  int img, cq, y, xx;
  decode4<true>(i, c4, a.ih, a.iw, img, cq, y, xx);
  const int ylo = max(0, (y + a.p.ph - (a.p.kh - 1) * a.p.dh + a.p.sh - 1) / a.p.sh), yhi = min(a.oh - 1, (y + a.p.ph) / a.p.sh);
  const int xlo = max(0, (xx + a.p.pw - (a.p.kw - 1) * a.p.dw + a.p.sw - 1) / a.p.sw), xhi = min(a.ow - 1, (xx + a.p.pw) / a.p.sw);
  const long long me = (long long)y * a.iw + xx;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int oy = ylo; oy <= yhi; oy++)
    for (int ox = xlo; ox <= xhi; ox++) {
      const int64_t o = (((int64_t)img * a.oh + oy) * a.ow + ox) * a.c + cq * 4;
      const longlong2* ip = reinterpret_cast<const longlong2*>(idx + o);
      const longlong2 i0 = __ldg(ip), i1 = __ldg(ip + 1);
      const float4 g = __ldg(reinterpret_cast<const float4*>(a.x.p + o));
      if (i0.x == me) acc[0] += g.x;
      if (i0.y == me) acc[1] += g.y;
      if (i1.x == me) acc[2] += g.z;
      if (i1.y == me) acc[3] += g.w;
    }
  *reinterpret_cast<float4*>(a.y.p + (((int64_t)img * a.ih + y) * a.iw + xx) * a.c + cq * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
}

// The same for a compile-time window (KS x KS, stride ST, no dilation): ResNet's 3x3 stride-2 stem pool and the like. A
// thread produces TX consecutive outputs of a row for its 4 channels, so that the (TX-1)*ST + KS input pixels of a window
// row are loaded once and shared by the windows; window bounds and strides are constants, so the index arithmetic is
// shifts and the loops unroll. Same update rule as above (first maximum wins, the first NaN wins outright).
template <int KS, int ST, int TX>
__global__ void __launch_bounds__(256) maxpool_fwd_nhwc4_fixed_kernel(PoolArgs a, int64_t* __restrict__ idx) {
  constexpr int SPAN = (TX - 1) * ST + KS;
  const int c4 = a.c >> 2, gx = (a.ow + TX - 1) / TX;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.oh * gx * c4) return;
  int img, cq, oy, xg;
  decode4<true>(i, c4, a.oh, gx, img, cq, oy, xg);
  const int ox0 = xg * TX, y0 = oy * ST - a.p.ph, x0 = ox0 * ST - a.p.pw;
  const float* xp = a.x.p + ((int64_t)img * a.ih * a.iw) * a.c + cq * 4;
  // "first maximum wins, the first NaN wins outright" without per-element flags: the running best starts at -inf with the
  // index of the window's first element (what an all -inf window reports), a value replaces it when it is larger, or when it
  // is a NaN and the best is not one yet; after that no comparison with the NaN best succeeds.
  float best[TX][4];
  int bi[TX][4];
  const int yf = max(y0, 0);
#pragma unroll
  for (int j = 0; j < TX; j++) {
    const int first = yf * a.iw + max(x0 + j * ST, 0);
#pragma unroll
    for (int k = 0; k < 4; k++) { best[j][k] = -INFINITY; bi[j][k] = first; }
  }
  const bool interior = x0 >= 0 && x0 + SPAN <= a.iw;
#pragma unroll
  for (int ky = 0; ky < KS; ky++) {
    const int y = y0 + ky;
    if (y < 0 || y >= a.ih) continue;
    float4 in[SPAN];
    const float* row = xp + ((int64_t)y * a.iw + x0) * a.c;
    if (interior) {
#pragma unroll
      for (int k = 0; k < SPAN; k++) in[k] = __ldg(reinterpret_cast<const float4*>(row + (int64_t)k * a.c));
    } else {
#pragma unroll
      for (int k = 0; k < SPAN; k++) {
        const int xx = x0 + k;
        in[k] = (xx >= 0 && xx < a.iw) ? __ldg(reinterpret_cast<const float4*>(row + (int64_t)k * a.c)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    const int rowi = y * a.iw + x0;
#pragma unroll
    for (int j = 0; j < TX; j++)
#pragma unroll
      for (int kx = 0; kx < KS; kx++) {
        if (!interior) {
          const int xx = x0 + j * ST + kx;
          if (xx < 0 || xx >= a.iw) continue;
        }
        const float4 v4 = in[j * ST + kx];
        const float v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
          const float b = best[j][k];
          if ((v[k] > b) | ((v[k] != v[k]) & (b == b))) { best[j][k] = v[k]; bi[j][k] = rowi + j * ST + kx; }
        }
      }
  }
#pragma unroll
  for (int j = 0; j < TX; j++) {
    if (ox0 + j >= a.ow) break;
    const int64_t o = (((int64_t)img * a.oh + oy) * a.ow + ox0 + j) * a.c + cq * 4;
    *reinterpret_cast<float4*>(a.y.p + o) = make_float4(best[j][0], best[j][1], best[j][2], best[j][3]);
    longlong2* ip = reinterpret_cast<longlong2*>(idx + o);
    ip[0] = make_longlong2(bi[j][0], bi[j][1]);
    ip[1] = make_longlong2(bi[j][2], bi[j][3]);
  }
}
template <int KS, int ST>
__global__ void __launch_bounds__(256) maxpool_bwd_nhwc4_fixed_kernel(PoolArgs a, const int64_t* __restrict__ idx) {
  // a.x = gy, a.y = gx; the windows that can hold input (y, xx): output rows ceil((y + p - KS + 1) / ST) .. floor((y + p) / ST)
  constexpr int NW = (KS + ST - 1) / ST;  // at most this many windows per axis
  const int c4 = a.c >> 2;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.ih * a.iw * c4) return;
  int img, cq, y, xx;
  decode4<true>(i, c4, a.ih, a.iw, img, cq, y, xx);
  const int yhi = (y + a.p.ph) / ST, xhi = (xx + a.p.pw) / ST;
  const long long me = (long long)y * a.iw + xx;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int dy = 0; dy < NW; dy++) {
    const int oy = yhi - dy;
    if (oy < 0 || oy >= a.oh || oy * ST - a.p.ph + KS <= y) continue;
#pragma unroll
    for (int dx = 0; dx < NW; dx++) {
      const int ox = xhi - dx;
      if (ox < 0 || ox >= a.ow || ox * ST - a.p.pw + KS <= xx) continue;
      const int64_t o = (((int64_t)img * a.oh + oy) * a.ow + ox) * a.c + cq * 4;
      const longlong2* ip = reinterpret_cast<const longlong2*>(idx + o);
      const longlong2 i0 = __ldg(ip), i1 = __ldg(ip + 1);
      const float4 g = __ldg(reinterpret_cast<const float4*>(a.x.p + o));
      if (i0.x == me) acc[0] += g.x;
      if (i0.y == me) acc[1] += g.y;
      if (i1.x == me) acc[2] += g.z;
      if (i1.y == me) acc[3] += g.w;
    }
  }
  *reinterpret_cast<float4*>(a.y.p + (((int64_t)img * a.ih + y) * a.iw + xx) * a.c + cq * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
}

// Stride 2: one thread takes an even-aligned 2 x 2 block of input pixels. The block meets at most two windows per axis, whose
// indices and gradients are loaded once and serve all four pixels: 4 window loads per block instead of 9 per-pixel ones
// (this kernel is bound by the bytes that cross L1, not by HBM). Indices are compared in 32 bits (h * w < 2^31).
template <int KS>
__global__ void __launch_bounds__(256) maxpool_bwd_nhwc4_s2_block_kernel(PoolArgs a, const int64_t* __restrict__ idx) {
  const int c4 = a.c >> 2, hb = (a.ih + 1) >> 1, wb = (a.iw + 1) >> 1;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * hb * wb * c4) return;
  int img, cq, yb, xb;
  decode4<true>(i, c4, hb, wb, img, cq, yb, xb);
  const int y0 = 2 * yb, x0 = 2 * xb;
  // windows whose rows [2 oy - p, 2 oy - p + KS) meet {y0, y0 + 1}
  const int oy_lo = max(0, (y0 + a.p.ph - KS + 2) >> 1), oy_hi = min(a.oh - 1, (y0 + 1 + a.p.ph) >> 1);
  const int ox_lo = max(0, (x0 + a.p.pw - KS + 2) >> 1), ox_hi = min(a.ow - 1, (x0 + 1 + a.p.pw) >> 1);
  const int me = y0 * a.iw + x0;  // pixel (py, px) of the block has index me + py * iw + px
  float acc[2][2][4];
#pragma unroll
  for (int py = 0; py < 2; py++)
#pragma unroll
    for (int px = 0; px < 2; px++)
#pragma unroll
      for (int k = 0; k < 4; k++) acc[py][px][k] = 0.f;
#pragma unroll
  for (int wy = 0; wy < 2; wy++) {
    const int oy = oy_lo + wy;
    if (oy > oy_hi) break;
#pragma unroll
    for (int wx = 0; wx < 2; wx++) {
      const int ox = ox_lo + wx;
      if (ox > ox_hi) break;
      const int64_t o = (((int64_t)img * a.oh + oy) * a.ow + ox) * a.c + cq * 4;
      const longlong2* ip = reinterpret_cast<const longlong2*>(idx + o);
      const longlong2 i0 = __ldg(ip), i1 = __ldg(ip + 1);
      const float4 g4 = __ldg(reinterpret_cast<const float4*>(a.x.p + o));
      const int id[4] = {(int)i0.x - me, (int)i0.y - me, (int)i1.x - me, (int)i1.y - me};
      const float g[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
      for (int k = 0; k < 4; k++) {
        if (id[k] == 0) acc[0][0][k] += g[k];
        else if (id[k] == 1) acc[0][1][k] += g[k];
        else if (id[k] == a.iw) acc[1][0][k] += g[k];
        else if (id[k] == a.iw + 1) acc[1][1][k] += g[k];
      }
    }
  }
#pragma unroll
  for (int py = 0; py < 2; py++) {
    if (y0 + py >= a.ih) break;
#pragma unroll
    for (int px = 0; px < 2; px++) {
      if (x0 + px >= a.iw) break;
      *reinterpret_cast<float4*>(a.y.p + (((int64_t)img * a.ih + y0 + py) * a.iw + x0 + px) * a.c + cq * 4) =
          make_float4(acc[py][px][0], acc[py][px][1], acc[py][px][2], acc[py][px][3]);
    }
  }
}

// ---- general average pool (aten divisor rules) ----
__device__ __forceinline__ float avg_div(const PoolArgs& a, int oy, int ox) {
  if (a.divisor) return (float)a.divisor;
  int hs = oy * a.p.sh - a.p.ph, ws = ox * a.p.sw - a.p.pw;
  int he = min(hs + a.p.kh, a.ih + a.p.ph), we = min(ws + a.p.kw, a.iw + a.p.pw);
  int pool = (he - hs) * (we - ws);
  if (a.include_pad) return (float)pool;
  hs = max(hs, 0); ws = max(ws, 0);
  he = min(he, a.ih); we = min(we, a.iw);
  return (float)((he - hs) * (we - ws));
}
template <bool NHWC>
__global__ void __launch_bounds__(256) avgpool_fwd_kernel(PoolArgs a) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.c * a.oh * a.ow) return;
  int img, ch, oy, ox;
  decode4<NHWC>(i, a.c, a.oh, a.ow, img, ch, oy, ox);
  const float* xp = a.x.p + img * a.x.sn + ch * a.x.sc;
  float s = 0.f;
  for (int ky = 0; ky < a.p.kh; ky++) {
    int y = oy * a.p.sh + ky - a.p.ph;
    if (y < 0 || y >= a.ih) continue;
    for (int kx = 0; kx < a.p.kw; kx++) {
      int xx = ox * a.p.sw + kx - a.p.pw;
      if (xx < 0 || xx >= a.iw) continue;
      s += __ldg(xp + y * a.x.sh + xx * a.x.sw);
    }
  }
  a.y.p[a.y.off(img, ch, oy, ox)] = s / avg_div(a, oy, ox);
}
template <bool NHWC>
__global__ void __launch_bounds__(256) avgpool_bwd_kernel(PoolArgs a) {  // a.x = gy, a.y = gx
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.c * a.ih * a.iw) return;
  int img, ch, y, xx;
  decode4<NHWC>(i, a.c, a.ih, a.iw, img, ch, y, xx);
  int ylo = max(0, (y + a.p.ph - (a.p.kh - 1) + a.p.sh - 1) / a.p.sh), yhi = min(a.oh - 1, (y + a.p.ph) / a.p.sh);
  int xlo = max(0, (xx + a.p.pw - (a.p.kw - 1) + a.p.sw - 1) / a.p.sw), xhi = min(a.ow - 1, (xx + a.p.pw) / a.p.sw);
  float acc = 0.f;
  for (int oy = ylo; oy <= yhi; oy++)
    for (int ox = xlo; ox <= xhi; ox++) acc += __ldg(a.x.p + a.x.off(img, ch, oy, ox)) / avg_div(a, oy, ox);
  a.y.p[a.y.off(img, ch, y, xx)] = acc;
}

// ---- adaptive average pool: window [floor(o*I/O), ceil((o+1)*I/O)) ----
__device__ __forceinline__ int ad_start(int o, int I, int O) { return (int)(((int64_t)o * I) / O); }
__device__ __forceinline__ int ad_end(int o, int I, int O) { return (int)((((int64_t)o + 1) * I + O - 1) / O); }
template <bool NHWC>
__global__ void __launch_bounds__(256) adapool_fwd_kernel(PoolArgs a) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.c * a.oh * a.ow) return;
  int img, ch, oy, ox;
  decode4<NHWC>(i, a.c, a.oh, a.ow, img, ch, oy, ox);
  int y0 = ad_start(oy, a.ih, a.oh), y1 = ad_end(oy, a.ih, a.oh), x0 = ad_start(ox, a.iw, a.ow), x1 = ad_end(ox, a.iw, a.ow);
  const float* xp = a.x.p + img * a.x.sn + ch * a.x.sc;
  float s = 0.f;
  for (int y = y0; y < y1; y++)
    for (int xx = x0; xx < x1; xx++) s += __ldg(xp + y * a.x.sh + xx * a.x.sw);
  a.y.p[a.y.off(img, ch, oy, ox)] = s / (float)((y1 - y0) * (x1 - x0));
}
// global average pool over an NCHW plane: one warp per (n, c) plane, coalesced, shuffle-reduced
__global__ void __launch_bounds__(256) gap_nchw_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t planes, int hw) {
  int64_t pl = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  if (pl >= planes) return;
  const float* p = x + pl * hw;
  float s = 0.f;
  for (int e = lane; e < hw; e += 32) s += __ldg(p + e);
  s = warp_sum(s);
  if (lane == 0) y[pl] = s / (float)hw;
}
template <bool NHWC>
__global__ void __launch_bounds__(256) adapool_bwd_kernel(PoolArgs a) {  // a.x = gy, a.y = gx
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.c * a.ih * a.iw) return;
  int img, ch, y, xx;
  decode4<NHWC>(i, a.c, a.ih, a.iw, img, ch, y, xx);
  // outputs o with start(o) <= y < end(o)
  int oy0 = (int)(((int64_t)y * a.oh) / a.ih), ox0 = (int)(((int64_t)xx * a.ow) / a.iw);
  float acc = 0.f;
  for (int oy = max(0, oy0 - 1); oy < a.oh && ad_start(oy, a.ih, a.oh) <= y; oy++) {
    if (ad_end(oy, a.ih, a.oh) <= y) continue;
    int hy = ad_end(oy, a.ih, a.oh) - ad_start(oy, a.ih, a.oh);
    for (int ox = max(0, ox0 - 1); ox < a.ow && ad_start(ox, a.iw, a.ow) <= xx; ox++) {
      if (ad_end(ox, a.iw, a.ow) <= xx) continue;
      int wx = ad_end(ox, a.iw, a.ow) - ad_start(ox, a.iw, a.ow);
      acc += __ldg(a.x.p + a.x.off(img, ch, oy, ox)) / (float)(hy * wx);
    }
  }
  a.y.p[a.y.off(img, ch, y, xx)] = acc;
}

static bool chan_last(const OmtAct* a) { return a->sc == 1 && a->sw != 1; }
static int pool_check(const OmtPool* p, const char* who) {
  OMT_REQUIRE(p && p->kh > 0 && p->kw > 0 && p->sh > 0 && p->sw > 0 && p->ph >= 0 && p->pw >= 0 && p->ph <= p->kh / 2 &&
                  p->pw <= p->kw / 2 && p->dh >= 1 && p->dw >= 1,
              "%s: window/stride must be positive and padding <= kernel/2", who);
  return OMT_OK;
}

static inline bool aligned16(const void* a, const void* b, const void* c) {
  return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15) == 0;
}
#define LAUNCH_BY_LAYOUT(kern, nhwc, total, s, ...)                                      \
  do {                                                                                   \
    unsigned blocks_ = (unsigned)cdiv((total), 256);                                     \
    if (nhwc) kern<true><<<blocks_, 256, 0, (s)>>>(__VA_ARGS__);                          \
    else kern<false><<<blocks_, 256, 0, (s)>>>(__VA_ARGS__);                              \
  } while (0)

}  // namespace omt

using namespace omt;

extern "C" {

int omt_pool2_fwd(const OmtAct* x, const OmtAct* y, uint8_t* idx, int32_t n, int32_t c, int32_t h, int32_t w, omt_stream_t stream) {
  OMT_REQUIRE(x && y && x->p && y->p && idx && n > 0 && c > 0 && h >= 2 && w >= 2, "omt_pool2_fwd: bad arguments");
  int oh = h / 2, ow = w / 2;
  LAUNCH_BY_LAYOUT(pool2_fwd_kernel, chan_last(y), (int64_t)n * c * oh * ow, st(stream), view(x), view(y), idx, n, c, oh, ow);
  return check_launch("pool2_fwd");
}
int omt_pool2_bwd(const OmtAct* gy, const uint8_t* idx, const OmtAct* gx, int32_t n, int32_t c, int32_t h, int32_t w,
                  omt_stream_t stream) {
  OMT_REQUIRE(gy && gx && gy->p && gx->p && idx && n > 0 && c > 0 && h >= 2 && w >= 2, "omt_pool2_bwd: bad arguments");
  LAUNCH_BY_LAYOUT(pool2_bwd_kernel, chan_last(gx), (int64_t)n * c * h * w, st(stream), view(gy), idx, view(gx), n, c, h, w, h / 2,
                   w / 2);
  return check_launch("pool2_bwd");
}
int omt_avgpool2_fwd(const OmtAct* x, const OmtAct* y, int32_t n, int32_t c, int32_t h, int32_t w, omt_stream_t stream) {
  OMT_REQUIRE(x && y && x->p && y->p && n > 0 && c > 0 && h >= 2 && w >= 2, "omt_avgpool2_fwd: bad arguments");
  LAUNCH_BY_LAYOUT(avgpool2_fwd_kernel, chan_last(y), (int64_t)n * c * (h / 2) * (w / 2), st(stream), view(x), view(y), n, c, h / 2,
                   w / 2);
  return check_launch("avgpool2_fwd");
}
int omt_avgpool2_bwd(const OmtAct* gy, const OmtAct* gx, int32_t n, int32_t c, int32_t h, int32_t w, omt_stream_t stream) {
  OMT_REQUIRE(gy && gx && gy->p && gx->p && n > 0 && c > 0 && h >= 2 && w >= 2, "omt_avgpool2_bwd: bad arguments");
  LAUNCH_BY_LAYOUT(avgpool2_bwd_kernel, chan_last(gx), (int64_t)n * c * h * w, st(stream), view(gy), view(gx), n, c, h, w, h / 2,
                   w / 2);
  return check_launch("avgpool2_bwd");
}

static PoolArgs pa(const OmtAct* x, const OmtAct* y, int n, int c, int ih, int iw, int oh, int ow, const OmtPool* p, int inc, int div) {
  PoolArgs a{};
  a.x = view(x); a.y = view(y); a.n = n; a.c = c; a.ih = ih; a.iw = iw; a.oh = oh; a.ow = ow;
  if (p) a.p = *p;
  a.include_pad = inc; a.divisor = div;
  return a;
}

int omt_maxpool_fwd(const OmtAct* x, const OmtAct* y, int64_t* idx, int32_t n, int32_t c, int32_t ih, int32_t iw, int32_t oh,
                    int32_t ow, const OmtPool* p, omt_stream_t stream) {
  int r = pool_check(p, "omt_maxpool_fwd");
  if (r) return r;
  OMT_REQUIRE(x && y && x->p && y->p && idx && n > 0 && c > 0 && oh > 0 && ow > 0, "omt_maxpool_fwd: bad arguments");
  if (c % 4 == 0 && is_nhwc(x, c, ih, iw) && is_nhwc(y, c, oh, ow) && aligned16(x->p, y->p, idx)) {
    const int64_t total = (int64_t)n * oh * ow * (c / 4);
    const bool square = p->kh == p->kw && p->sh == p->sw && p->dh == 1 && p->dw == 1;
    if (square && p->kh == 3 && p->sh == 2) {
      maxpool_fwd_nhwc4_fixed_kernel<3, 2, 4><<<(unsigned)cdiv((int64_t)n * oh * cdiv(ow, 4) * (c / 4), 256), 256, 0, st(stream)>>>(
          pa(x, y, n, c, ih, iw, oh, ow, p, 0, 0), idx);
      return check_launch("maxpool_fwd_nhwc4_k3s2");
    }
    if (square && p->kh == 2 && p->sh == 2) {
      maxpool_fwd_nhwc4_fixed_kernel<2, 2, 4><<<(unsigned)cdiv((int64_t)n * oh * cdiv(ow, 4) * (c / 4), 256), 256, 0, st(stream)>>>(
          pa(x, y, n, c, ih, iw, oh, ow, p, 0, 0), idx);
      return check_launch("maxpool_fwd_nhwc4_k2s2");
    }
    maxpool_fwd_nhwc4_kernel<<<(unsigned)cdiv(total, 256), 256, 0, st(stream)>>>(pa(x, y, n, c, ih, iw, oh, ow, p, 0, 0), idx);
    return check_launch("maxpool_fwd_nhwc4");
  }
  LAUNCH_BY_LAYOUT(maxpool_fwd_kernel, chan_last(y), (int64_t)n * c * oh * ow, st(stream), pa(x, y, n, c, ih, iw, oh, ow, p, 0, 0), idx);
  return check_launch("maxpool_fwd");
}
int omt_maxpool_bwd(const OmtAct* gy, const int64_t* idx, const OmtAct* gx, int32_t n, int32_t c, int32_t ih, int32_t iw,
                    int32_t oh, int32_t ow, const OmtPool* p, omt_stream_t stream) {
  int r = pool_check(p, "omt_maxpool_bwd");
  if (r) return r;
  OMT_REQUIRE(gy && gx && gy->p && gx->p && idx && n > 0 && c > 0 && oh > 0 && ow > 0, "omt_maxpool_bwd: bad arguments");
  if (c % 4 == 0 && is_nhwc(gy, c, oh, ow) && is_nhwc(gx, c, ih, iw) && aligned16(gy->p, gx->p, idx)) {
    const int64_t total = (int64_t)n * ih * iw * (c / 4);
    const bool square = p->kh == p->kw && p->sh == p->sw && p->dh == 1 && p->dw == 1;
    const int64_t blocks2 = (int64_t)n * ((ih + 1) / 2) * ((iw + 1) / 2) * (c / 4);  // 2 x 2 pixel blocks x channel quads
    if (square && p->kh == 3 && p->sh == 2 && iw > 1) {
      maxpool_bwd_nhwc4_s2_block_kernel<3><<<(unsigned)cdiv(blocks2, 256), 256, 0, st(stream)>>>(pa(gy, gx, n, c, ih, iw, oh, ow, p, 0, 0), idx);
      return check_launch("maxpool_bwd_nhwc4_k3s2");
    }
    if (square && p->kh == 2 && p->sh == 2 && iw > 1) {
      maxpool_bwd_nhwc4_s2_block_kernel<2><<<(unsigned)cdiv(blocks2, 256), 256, 0, st(stream)>>>(pa(gy, gx, n, c, ih, iw, oh, ow, p, 0, 0), idx);
      return check_launch("maxpool_bwd_nhwc4_k2s2");
    }
    maxpool_bwd_nhwc4_kernel<<<(unsigned)cdiv(total, 256), 256, 0, st(stream)>>>(pa(gy, gx, n, c, ih, iw, oh, ow, p, 0, 0), idx);
    return check_launch("maxpool_bwd_nhwc4");
  }
  LAUNCH_BY_LAYOUT(maxpool_bwd_kernel, chan_last(gx), (int64_t)n * c * ih * iw, st(stream), pa(gy, gx, n, c, ih, iw, oh, ow, p, 0, 0),
                   idx);
  return check_launch("maxpool_bwd");
}
int omt_avgpool_fwd(const OmtAct* x, const OmtAct* y, int32_t n, int32_t c, int32_t ih, int32_t iw, int32_t oh, int32_t ow,
                    const OmtPool* p, int32_t count_include_pad, int32_t divisor, omt_stream_t stream) {
  int r = pool_check(p, "omt_avgpool_fwd");
  if (r) return r;
  OMT_REQUIRE(x && y && x->p && y->p && n > 0 && c > 0 && oh > 0 && ow > 0 && divisor >= 0, "omt_avgpool_fwd: bad arguments");
  LAUNCH_BY_LAYOUT(avgpool_fwd_kernel, chan_last(y), (int64_t)n * c * oh * ow, st(stream),
                   pa(x, y, n, c, ih, iw, oh, ow, p, count_include_pad, divisor));
  return check_launch("avgpool_fwd");
}
int omt_avgpool_bwd(const OmtAct* gy, const OmtAct* gx, int32_t n, int32_t c, int32_t ih, int32_t iw, int32_t oh, int32_t ow,
                    const OmtPool* p, int32_t count_include_pad, int32_t divisor, omt_stream_t stream) {
  int r = pool_check(p, "omt_avgpool_bwd");
  if (r) return r;
  OMT_REQUIRE(gy && gx && gy->p && gx->p && n > 0 && c > 0 && oh > 0 && ow > 0 && divisor >= 0, "omt_avgpool_bwd: bad arguments");
  LAUNCH_BY_LAYOUT(avgpool_bwd_kernel, chan_last(gx), (int64_t)n * c * ih * iw, st(stream),
                   pa(gy, gx, n, c, ih, iw, oh, ow, p, count_include_pad, divisor));
  return check_launch("avgpool_bwd");
}
int omt_adaptive_avgpool_fwd(const OmtAct* x, const OmtAct* y, int32_t n, int32_t c, int32_t ih, int32_t iw, int32_t oh,
                             int32_t ow, omt_stream_t stream) {
  OMT_REQUIRE(x && y && x->p && y->p && n > 0 && c > 0 && ih > 0 && iw > 0 && oh > 0 && ow > 0, "omt_adaptive_avgpool_fwd: bad arguments");
  if (oh == 1 && ow == 1 && is_nchw(x, c, ih, iw) && y->sc == 1 && y->sn == c) {
    int64_t planes = (int64_t)n * c;
    gap_nchw_kernel<<<(unsigned)cdiv(planes * 32, 256), 256, 0, st(stream)>>>(x->p, y->p, planes, ih * iw);
    return check_launch("gap_fwd_nchw");
  }
  LAUNCH_BY_LAYOUT(adapool_fwd_kernel, chan_last(y) || (oh == 1 && ow == 1 && chan_last(x)), (int64_t)n * c * oh * ow, st(stream),
                   pa(x, y, n, c, ih, iw, oh, ow, nullptr, 0, 0));
  return check_launch("adaptive_avgpool_fwd");
}
int omt_adaptive_avgpool_bwd(const OmtAct* gy, const OmtAct* gx, int32_t n, int32_t c, int32_t ih, int32_t iw, int32_t oh,
                             int32_t ow, omt_stream_t stream) {
  OMT_REQUIRE(gy && gx && gy->p && gx->p && n > 0 && c > 0 && ih > 0 && iw > 0 && oh > 0 && ow > 0, "omt_adaptive_avgpool_bwd: bad arguments");
  LAUNCH_BY_LAYOUT(adapool_bwd_kernel, chan_last(gx), (int64_t)n * c * ih * iw, st(stream), pa(gy, gx, n, c, ih, iw, oh, ow, nullptr, 0, 0));
  return check_launch("adaptive_avgpool_bwd");
}

}  // extern "C"

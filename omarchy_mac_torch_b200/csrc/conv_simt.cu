// fp32 implicit-GEMM convolution on the CUDA cores: forward, input gradient (all stride phases in one launch) and
// weight gradient (split-K + deterministic slab sum). This is the exact-fp32 path: it serves every geometry the op
// layer accepts (ks <= 11, stride 1..4, pad <= ks, any activation strides) and cross-checks the tensor-core path.
//
// Behaviour follows the reference's generated kernels (omarchy_mac_torch/gemm.py: kinds 0, 1, 5, 2) and their host
// side (csrc/conv.cpp:70-114); the structure does not: one templated kernel, im2col index decomposition hoisted out
// of the K loop (rows/columns are decomposed once per thread, the K index once per thread per step), register
// prefetch with double-buffered shared tiles, 128-bit shared loads and stores.
#include <algorithm>

#include "common.cuh"

namespace omt {

struct ConvArgs {
  ActView a;  // GEMM A-side activation: x (fwd), gy (dgrad), gy (wgrad)
  ActView b;  // second activation: y (fwd, output), dx (dgrad, output), x (wgrad, B operand)
  const float* w;
  const float* bias;
  float* out;  // wgrad: partial slabs [slices][M][N] (or dw when slices == 1)
  int n, ci, co, ih, iw, oh, ow, ks, stride, pad;
  int M, N, K, kslice, slices;
  uint32_t flags;
  float scale;
};

constexpr int BK = 8;

// ---- forward: m=(img,oy,ox) k=(ci,ky,kx) n=co ---------------------------------------------------------------------
struct Fwd {
  static constexpr bool A_MFAST = true, B_NFAST = false;
  const ConvArgs& g;
  int M, N, kbeg, kend;
  __device__ Fwd(const ConvArgs& g_, int) : g(g_), M(g_.M), N(g_.N), kbeg(0), kend(g_.K) {}
  struct Row { int64_t base; int iy0, ix0; };  // iy0 = INT_MIN/2 marks an out-of-range row
  struct KIdx { int64_t off; int ky, kx; bool ok; };
  struct Col { const float* p; };
  __device__ Row row(int m) const {
    if (m >= M) return {0, -(1 << 28), 0};
    int ohw = g.oh * g.ow, img = m / ohw, r = m - img * ohw, oy = r / g.ow, ox = r - oy * g.ow;
    int iy0 = oy * g.stride - g.pad, ix0 = ox * g.stride - g.pad;
    return {img * g.a.sn + iy0 * g.a.sh + ix0 * g.a.sw, iy0, ix0};
  }
  __device__ KIdx kidx(int k) const {
    if (k >= kend) return {0, 0, 0, false};
    int kk = g.ks * g.ks, c = k / kk, r = k - c * kk, ky = r / g.ks, kx = r - ky * g.ks;
    return {c * g.a.sc + ky * g.a.sh + kx * g.a.sw, ky, kx, true};
  }
  __device__ float loadA(const Row& r, const KIdx& k) const {
    int y = r.iy0 + k.ky, x = r.ix0 + k.kx;
    if (!k.ok || y < 0 || y >= g.ih || x < 0 || x >= g.iw) return 0.f;
    return __ldg(g.a.p + r.base + k.off);
  }
  __device__ Col col(int nn) const { return {nn < N ? g.w + (int64_t)nn * g.K : nullptr}; }
  __device__ float loadB(const Col& c, const KIdx& k, int kabs) const { return (c.p && k.ok) ? __ldg(c.p + kabs) : 0.f; }
  // 4 consecutive rows (m..m+3) x 4 consecutive columns (nn..nn+3)
  __device__ void store(int m, int nn, const float (&v)[4][4]) const {
    int ohw = g.oh * g.ow;
    if (g.b.sc == 1 && nn + 3 < N) {  // channels-last output: the 4 columns of a row are contiguous
      float bv[4];
#pragma unroll
      for (int j = 0; j < 4; j++) bv[j] = (g.flags & OMT_EPI_BIAS) ? __ldg(g.bias + nn + j) : 0.f;
      bool done = true;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        int mm = m + i;
        if (mm >= M) break;
        int im2 = mm / ohw, r2 = mm - im2 * ohw, oy = r2 / g.ow, ox = r2 - oy * g.ow;
        float* p = g.b.p + g.b.off(im2, nn, oy, ox);
        if (reinterpret_cast<uintptr_t>(p) & 15) { done = false; break; }
        float4 o = make_float4(v[i][0] + bv[0], v[i][1] + bv[1], v[i][2] + bv[2], v[i][3] + bv[3]);
        if (g.flags & OMT_EPI_RELU) o = make_float4(fmaxf(o.x, 0.f), fmaxf(o.y, 0.f), fmaxf(o.z, 0.f), fmaxf(o.w, 0.f));
        *reinterpret_cast<float4*>(p) = o;
      }
      if (done) return;
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int c = nn + j;
      if (c >= N) break;
      float bv = (g.flags & OMT_EPI_BIAS) ? __ldg(g.bias + c) : 0.f;
      float o[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        o[i] = v[i][j] + bv;
        if (g.flags & OMT_EPI_RELU) o[i] = fmaxf(o[i], 0.f);
      }
      int img = m / ohw, r = m - img * ohw;
      if (g.b.sw == 1 && g.b.sh == g.ow && m + 3 < M && r + 3 < ohw) {
        float* p = g.b.p + img * g.b.sn + c * g.b.sc + r;
        if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
          *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
          continue;
        }
      }
#pragma unroll
      for (int i = 0; i < 4; i++) {
        int mm = m + i;
        if (mm >= M) break;
        int im2 = mm / ohw, r2 = mm - im2 * ohw, oy = r2 / g.ow, ox = r2 - oy * g.ow;
        g.b.p[g.b.off(im2, c, oy, ox)] = o[i];
      }
    }
  }
};

// ---- input gradient, one stride phase per blockIdx.z: m=(img,i,j) k=(co,ty,tx) n=ci -----------------------------------
// Phase (py,px) covers input pixels y=py+s*i, x=px+s*j. Only taps ky=ky0+s*ty, kx=kx0+s*tx reach them, from output
// pixel (i+qy-ty, j+qx-tx). Same index algebra as the reference host loop (csrc/conv.cpp:78-95).
struct Dgrad {
  static constexpr bool A_MFAST = true, B_NFAST = true;
  const ConvArgs& g;
  int M, N, kbeg, kend;
  int py, px, ky0, kx0, qy, qx, hi, wi, jy, jx;
  __device__ Dgrad(const ConvArgs& g_, int z) : g(g_) {
    int s = g.stride;
    py = z / s; px = z - py * s;
    hi = (g.ih - py + s - 1) / s; wi = (g.iw - px + s - 1) / s;
    if (hi < 0) hi = 0;
    if (wi < 0) wi = 0;
    ky0 = (py + g.pad) % s; kx0 = (px + g.pad) % s;
    jy = ky0 < g.ks ? (g.ks - ky0 + s - 1) / s : 0;
    jx = kx0 < g.ks ? (g.ks - kx0 + s - 1) / s : 0;
    qy = (py + g.pad - ky0) / s; qx = (px + g.pad - kx0) / s;
    M = g.n * hi * wi; N = g.ci; kbeg = 0; kend = g.co * jy * jx;
  }
  struct Row { int64_t base; int oy0, ox0; };
  struct KIdx { int64_t off; int ty, tx, wofs; bool ok; };
  struct Col { int64_t wofs; bool ok; };
  __device__ Row row(int m) const {
    if (m >= M) return {0, -(1 << 28), 0};
    int hw = hi * wi, img = m / hw, r = m - img * hw, i = r / wi, j = r - i * wi;
    int oy0 = i + qy, ox0 = j + qx;
    return {img * g.a.sn + oy0 * g.a.sh + ox0 * g.a.sw, oy0, ox0};
  }
  __device__ KIdx kidx(int k) const {
    if (k >= kend) return {0, 0, 0, 0, false};
    int jj = jy * jx, co = k / jj, r = k - co * jj, ty = r / jx, tx = r - ty * jx;
    int ky = ky0 + g.stride * ty, kx = kx0 + g.stride * tx;
    return {co * g.a.sc - ty * g.a.sh - tx * g.a.sw, ty, tx, (co * g.ci * g.ks + ky) * g.ks + kx, true};
  }
  __device__ float loadA(const Row& r, const KIdx& k) const {
    int oy = r.oy0 - k.ty, ox = r.ox0 - k.tx;
    if (!k.ok || oy < 0 || oy >= g.oh || ox < 0 || ox >= g.ow) return 0.f;
    return __ldg(g.a.p + r.base + k.off);
  }
  __device__ Col col(int nn) const { return {(int64_t)nn * g.ks * g.ks, nn < N}; }
  __device__ float loadB(const Col& c, const KIdx& k, int) const {
    return (c.ok && k.ok) ? __ldg(g.w + k.wofs + c.wofs) : 0.f;
  }
  __device__ void store(int m, int nn, const float (&v)[4][4]) const {
    int hw = hi * wi;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      int c = nn + j;
      if (c >= N) break;
      int img = m / hw, r = m - img * hw, i0 = r / wi, j0 = r - i0 * wi;
      if (g.stride == 1 && g.b.sw == 1 && m + 3 < M && j0 + 3 < wi) {
        float* p = g.b.p + g.b.off(img, c, i0, j0);
        if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
          *reinterpret_cast<float4*>(p) = make_float4(v[0][j], v[1][j], v[2][j], v[3][j]);
          continue;
        }
      }
#pragma unroll
      for (int i = 0; i < 4; i++) {
        int mm = m + i;
        if (mm >= M) break;
        int im2 = mm / hw, r2 = mm - im2 * hw, ii = r2 / wi, jj2 = r2 - ii * wi;
        g.b.p[g.b.off(im2, c, py + g.stride * ii, px + g.stride * jj2)] = v[i][j];
      }
    }
  }
};

// ---- weight gradient, one K slice per blockIdx.z: m=co k=(img,oy,ox) n=(ci,ky,kx) -------------------------------------
struct Wgrad {
  static constexpr bool A_MFAST = false, B_NFAST = false;
  const ConvArgs& g;
  int M, N, kbeg, kend, z;
  __device__ Wgrad(const ConvArgs& g_, int z_) : g(g_), M(g_.M), N(g_.N), z(z_) {
    kbeg = z_ * g.kslice;
    kend = min(g.K, kbeg + g.kslice);
  }
  struct Row { int64_t off; bool ok; };
  struct KIdx { int64_t aoff, boff; int iy0, ix0; bool ok; };
  struct Col { int64_t off; int ky, kx; bool ok; };
  __device__ Row row(int m) const { return {m * g.a.sc, m < M}; }
  __device__ KIdx kidx(int k) const {
    if (k >= kend) return {0, 0, 0, 0, false};
    int ohw = g.oh * g.ow, img = k / ohw, r = k - img * ohw, oy = r / g.ow, ox = r - oy * g.ow;
    int iy0 = oy * g.stride - g.pad, ix0 = ox * g.stride - g.pad;
    return {img * g.a.sn + oy * g.a.sh + ox * g.a.sw, img * g.b.sn + iy0 * g.b.sh + ix0 * g.b.sw, iy0, ix0, true};
  }
  __device__ float loadA(const Row& r, const KIdx& k) const { return (r.ok && k.ok) ? __ldg(g.a.p + r.off + k.aoff) : 0.f; }
  __device__ Col col(int nn) const {
    if (nn >= N) return {0, 0, 0, false};
    int kk = g.ks * g.ks, c = nn / kk, r = nn - c * kk, ky = r / g.ks, kx = r - ky * g.ks;
    return {c * g.b.sc + ky * g.b.sh + kx * g.b.sw, ky, kx, true};
  }
  __device__ float loadB(const Col& c, const KIdx& k, int) const {
    int y = k.iy0 + c.ky, x = k.ix0 + c.kx;
    if (!c.ok || !k.ok || y < 0 || y >= g.ih || x < 0 || x >= g.iw) return 0.f;
    return __ldg(g.b.p + k.boff + c.off);
  }
  __device__ void store(int m, int nn, const float (&v)[4][4]) const {
    float* base = g.out + (int64_t)z * M * N;
    float sc = g.slices == 1 ? g.scale : 1.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      if (m + i >= M) break;
#pragma unroll
      for (int j = 0; j < 4; j++)
        if (nn + j < N) base[(int64_t)(m + i) * N + nn + j] = v[i][j] * sc;
    }
  }
};

// C tile BM x BN per block of 256 threads; each thread owns TM x TN as (TM/4) x (TN/4) groups of 4x4, groups BM/2 or
// BN/2 apart, threads m-fastest so stores along m coalesce for NCHW outputs.
template <class L, int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__(256) conv_gemm_simt(ConvArgs g) {
  constexpr int TY = BM / TM, GM = TM / 4, GN = TN / 4;
  constexpr int RA = BM / 32, RB = (BN + 31) / 32;
  static_assert((BM / TM) * (BN / TN) == 256, "256 threads");
  __shared__ __align__(16) float As[2][BK][BM + 4];
  __shared__ __align__(16) float Bs[2][BK][BN + 4];
  L ld(g, blockIdx.z);
  const int M = ld.M, N = ld.N;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;  // M tiles on x: its limit is 2^31-1, y's is 65535
  if (m0 >= M) return;
  const int tid = threadIdx.x;
  const int a_k = L::A_MFAST ? (tid >> 5) : (tid & 7), a_r = L::A_MFAST ? (tid & 31) : (tid >> 3);
  const int b_k = L::B_NFAST ? (tid >> 5) : (tid & 7), b_r = L::B_NFAST ? (tid & 31) : (tid >> 3);
  typename L::Row ra[RA];
  typename L::Col cb[RB];
#pragma unroll
  for (int i = 0; i < RA; i++) ra[i] = ld.row(m0 + a_r + 32 * i);
#pragma unroll
  for (int i = 0; i < RB; i++) cb[i] = ld.col((b_r + 32 * i < BN) ? n0 + b_r + 32 * i : N);
  float acc[GM][GN][4][4];
#pragma unroll
  for (int a = 0; a < GM; a++)
#pragma unroll
    for (int b = 0; b < GN; b++)
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[a][b][i][j] = 0.f;
  float pa[RA], pb[RB];
  auto fetch = [&](int k0) {
    typename L::KIdx ka = ld.kidx(k0 + a_k);
#pragma unroll
    for (int i = 0; i < RA; i++) pa[i] = ld.loadA(ra[i], ka);
    if constexpr (L::A_MFAST == L::B_NFAST) {
#pragma unroll
      for (int i = 0; i < RB; i++) pb[i] = ld.loadB(cb[i], ka, k0 + b_k);
    } else {
      typename L::KIdx kb = ld.kidx(k0 + b_k);
#pragma unroll
      for (int i = 0; i < RB; i++) pb[i] = ld.loadB(cb[i], kb, k0 + b_k);
    }
  };
  auto commit = [&](int buf) {
#pragma unroll
    for (int i = 0; i < RA; i++) As[buf][a_k][a_r + 32 * i] = pa[i];
#pragma unroll
    for (int i = 0; i < RB; i++)
      if (b_r + 32 * i < BN) Bs[buf][b_k][b_r + 32 * i] = pb[i];
  };
  const int tm = tid % TY, tn = tid / TY;
  int buf = 0;
  if (ld.kbeg < ld.kend) {
    fetch(ld.kbeg);
    commit(0);
  }
  __syncthreads();
  for (int k0 = ld.kbeg; k0 < ld.kend; k0 += BK) {
    const bool more = k0 + BK < ld.kend;
    if (more) fetch(k0 + BK);
#pragma unroll
    for (int kk = 0; kk < BK; kk++) {
      float4 av[GM], bv[GN];
#pragma unroll
      for (int a = 0; a < GM; a++) av[a] = *reinterpret_cast<const float4*>(&As[buf][kk][tm * 4 + a * (BM / 2)]);
#pragma unroll
      for (int b = 0; b < GN; b++) bv[b] = *reinterpret_cast<const float4*>(&Bs[buf][kk][tn * 4 + b * (BN / 2)]);
#pragma unroll
      for (int a = 0; a < GM; a++) {
        const float ar[4] = {av[a].x, av[a].y, av[a].z, av[a].w};
#pragma unroll
        for (int b = 0; b < GN; b++) {
          const float br[4] = {bv[b].x, bv[b].y, bv[b].z, bv[b].w};
#pragma unroll
          for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[a][b][i][j] = fmaf(ar[i], br[j], acc[a][b][i][j]);
        }
      }
    }
    if (more) commit(buf ^ 1);
    __syncthreads();
    buf ^= 1;
  }
#pragma unroll
  for (int a = 0; a < GM; a++)
#pragma unroll
    for (int b = 0; b < GN; b++) {
      int m = m0 + tm * 4 + a * (BM / 2), nn = n0 + tn * 4 + b * (BN / 2);
      if (m < M && nn < N) ld.store(m, nn, acc[a][b]);
    }
}

// dw[i] = scale * sum_z part[z][i]   (reference csrc/kernels/gemm_reduce.wgsl:7-13, vectorised)
__global__ void __launch_bounds__(256) slab_sum_kernel(const float* __restrict__ part, float* __restrict__ out, int64_t total,
                                                       int slices, float scale) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  float s = 0.f;
  for (int z = 0; z < slices; z++) s += __ldg(part + (int64_t)z * total + i);
  out[i] = s * scale;
}

template <class L>
static int launch_gemm(const ConvArgs& a, int64_t Mmax, int64_t N, int gz, cudaStream_t s, const char* name) {
  // tile choice: narrow-N tiles for tiny channel counts, smaller tiles when the grid would not fill the SMs
  int sms = sm_count();
  auto blocks = [&](int bm, int bn) { return cdiv(Mmax, bm) * cdiv(N, bn) * gz; };
  // M tiles on grid.x (limit 2^31-1), N tiles on grid.y (limit 65535: N is a channel count, or ci*ks*ks for the weight gradient)
  OMT_REQUIRE(cdiv(N, N <= 16 ? 16 : 64) <= 65535 && gz <= 65535, "%s: %lld GEMM columns exceed the launch grid", name, (long long)N);
  if (N <= 16) {
    dim3 grid((unsigned)cdiv(Mmax, 256), (unsigned)cdiv(N, 16), gz);
    conv_gemm_simt<L, 256, 16, 4, 4><<<grid, 256, 0, s>>>(a);
  } else if (N <= 64 || blocks(128, 128) < sms) {
    if (blocks(128, 64) < sms) {
      dim3 grid((unsigned)cdiv(Mmax, 64), (unsigned)cdiv(N, 64), gz);
      conv_gemm_simt<L, 64, 64, 4, 4><<<grid, 256, 0, s>>>(a);
    } else {
      dim3 grid((unsigned)cdiv(Mmax, 128), (unsigned)cdiv(N, 64), gz);
      conv_gemm_simt<L, 128, 64, 8, 4><<<grid, 256, 0, s>>>(a);
    }
  } else {
    dim3 grid((unsigned)cdiv(Mmax, 128), (unsigned)cdiv(N, 128), gz);
    conv_gemm_simt<L, 128, 128, 8, 8><<<grid, 256, 0, s>>>(a);
  }
  return check_launch(name);
}

static ConvArgs base_args(const OmtConvGeo* g) {
  ConvArgs a{};
  a.n = g->n; a.ci = g->ci; a.co = g->co; a.ih = g->ih; a.iw = g->iw; a.oh = g->oh; a.ow = g->ow;
  a.ks = g->ks; a.stride = g->stride; a.pad = g->pad;
  a.slices = 1; a.scale = 1.f;
  return a;
}

int simt_conv_fwd(const OmtConvGeo* g, const OmtAct* x, const float* w, const float* bias, const OmtAct* y,
                  uint32_t flags, cudaStream_t s) {
  ConvArgs a = base_args(g);
  a.a = view(x); a.b = view(y); a.w = w; a.bias = bias; a.flags = flags;
  a.M = g->n * g->oh * g->ow; a.N = g->co; a.K = g->ci * g->ks * g->ks;
  return launch_gemm<Fwd>(a, a.M, a.N, 1, s, "conv_fwd_simt");
}

// ---------------------------------------------------------------------------------------------------------------------
// Input gradient for <= 4 input channels (a network's first layer): the GEMM would have N = ci <= 4 columns, so instead
// one thread owns one input pixel and all its channels. A block works on one stride phase (py, px) of one image: every
// thread then needs the same filter taps (ky = ky0 + s*ty, kx = kx0 + s*tx; the phase algebra of csrc/conv.cpp:78-95),
// whose weights sit in shared memory as float4 per (tap, co) and are read as warp-wide broadcasts, while consecutive
// lanes read consecutive output pixels of gy.
// ---------------------------------------------------------------------------------------------------------------------
struct DgSmallArgs {
  ActView gy, dx;
  const float* w;
  int n, ci, co, ih, iw, oh, ow, ks, stride, pad;
};

__global__ void __launch_bounds__(128) dgrad_small_ci_kernel(DgSmallArgs a) {
  extern __shared__ float4 wsm[];  // [jy * jx][co]
  const int s = a.stride;
  const int py = blockIdx.y / s, px = blockIdx.y - py * s, img = blockIdx.z;
  const int hi = (a.ih - py + s - 1) / s, wi = (a.iw - px + s - 1) / s;  // pixels of this phase
  const int ky0 = (py + a.pad) % s, kx0 = (px + a.pad) % s;
  const int jy = ky0 < a.ks ? (a.ks - ky0 + s - 1) / s : 0, jx = kx0 < a.ks ? (a.ks - kx0 + s - 1) / s : 0;
  const int taps = jy * jx;
  for (int i = threadIdx.x; i < taps * a.co; i += blockDim.x) {
    const int t = i / a.co, o = i - t * a.co;
    const int ky = ky0 + s * (t / jx), kx = kx0 + s * (t % jx);
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (int c = 0; c < a.ci; c++) v[c] = __ldg(a.w + (((int64_t)o * a.ci + c) * a.ks + ky) * a.ks + kx);
    wsm[i] = make_float4(v[0], v[1], v[2], v[3]);
  }
  __syncthreads();
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= hi * wi) return;
  const int yi = p / wi, xi = p - yi * wi;
  const int y = py + s * yi, x = px + s * xi;
  // output pixel reached through tap (ty, tx): oy = (y + pad - ky) / s = qy - ty with qy = (y + pad - ky0) / s
  const int qy = (y + a.pad - ky0) / s, qx = (x + a.pad - kx0) / s;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  const bool vec = a.gy.sc == 1 && (a.co & 3) == 0 && ((reinterpret_cast<uintptr_t>(a.gy.p) & 15) == 0) && (a.gy.sw & 3) == 0 &&
                   (a.gy.sh & 3) == 0 && (a.gy.sn & 3) == 0;
  for (int ty = 0; ty < jy; ty++) {
    const int oy = qy - ty;
    if (oy < 0 || oy >= a.oh) continue;
    for (int tx = 0; tx < jx; tx++) {
      const int ox = qx - tx;
      if (ox < 0 || ox >= a.ow) continue;
      const float4* wt = wsm + (ty * jx + tx) * a.co;
      const float* gp = a.gy.p + a.gy.off(img, 0, oy, ox);
      if (vec) {
        for (int o = 0; o < a.co; o += 4) {
          const float4 g4 = __ldg(reinterpret_cast<const float4*>(gp + o));
          const float gv[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
          for (int k = 0; k < 4; k++) {
            const float4 wv = wt[o + k];
            acc[0] = fmaf(gv[k], wv.x, acc[0]); acc[1] = fmaf(gv[k], wv.y, acc[1]);
            acc[2] = fmaf(gv[k], wv.z, acc[2]); acc[3] = fmaf(gv[k], wv.w, acc[3]);
          }
        }
      } else {
#pragma unroll 4
        for (int o = 0; o < a.co; o++) {
          const float gv = __ldg(gp + (int64_t)o * a.gy.sc);
          const float4 wv = wt[o];
          acc[0] = fmaf(gv, wv.x, acc[0]); acc[1] = fmaf(gv, wv.y, acc[1]);
          acc[2] = fmaf(gv, wv.z, acc[2]); acc[3] = fmaf(gv, wv.w, acc[3]);
        }
      }
    }
  }
  float* out = a.dx.p + a.dx.off(img, 0, y, x);
  for (int c = 0; c < a.ci; c++) out[(int64_t)c * a.dx.sc] = acc[c];
}

bool dgrad_small_ci_ok(const OmtConvGeo* g) {
  if (g->ci > 4 || g->groups != 1 || g->n > 65535 || g->stride * g->stride > 65535) return false;
  const int jmax = (int)cdiv(g->ks, g->stride);
  return (size_t)jmax * jmax * g->co * sizeof(float4) <= 200 * 1024;
}
int dgrad_small_ci(const OmtConvGeo* g, const OmtAct* gy, const float* w, const OmtAct* dx, cudaStream_t s) {
  DgSmallArgs a{view(gy), view(dx), w, g->n, g->ci, g->co, g->ih, g->iw, g->oh, g->ow, g->ks, g->stride, g->pad};
  const int jmax = (int)cdiv(g->ks, g->stride);
  const size_t smem = (size_t)jmax * jmax * g->co * sizeof(float4);
  static size_t attr = 0;
  if (smem > 48 * 1024 && smem > attr) {
    OMT_CUDA(cudaFuncSetAttribute(dgrad_small_ci_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    attr = smem;
  }
  const int64_t per_phase = cdiv(g->ih, g->stride) * cdiv(g->iw, g->stride);
  dim3 grid((unsigned)cdiv(per_phase, 128), (unsigned)(g->stride * g->stride), (unsigned)g->n);
  dgrad_small_ci_kernel<<<grid, 128, smem, s>>>(a);
  return check_launch("conv_dgrad_small_ci");
}

int simt_conv_dgrad(const OmtConvGeo* g, const OmtAct* gy, const float* w, const OmtAct* dx, cudaStream_t s) {
  if (dgrad_small_ci_ok(g)) return dgrad_small_ci(g, gy, w, dx, s);
  ConvArgs a = base_args(g);
  a.a = view(gy); a.b = view(dx); a.w = w;
  int st_ = g->stride;
  int64_t hi = cdiv(g->ih, st_), wi = cdiv(g->iw, st_);  // phase (0,0) is the largest
  a.N = g->ci;
  return launch_gemm<Dgrad>(a, (int64_t)g->n * hi * wi, a.N, st_ * st_, s, "conv_dgrad_simt");
}

// Split-K slicing: enough slices to fill the machine about twice over, each at least 64 deep (the reference's
// bound, csrc/conv.cpp:106-109, with the M1's "512 workgroups" target replaced by 2 x SM count).
void wgrad_slices(const OmtConvGeo* g, int* slices, int* kslice) {
  int64_t M = g->co, N = (int64_t)g->ci * g->ks * g->ks, K = (int64_t)g->n * g->oh * g->ow;
  int bm = 128, bn = N <= 16 ? 16 : (N <= 64 ? 64 : 128);
  if (N <= 16) bm = 256;
  int64_t tiles = cdiv(M, bm) * cdiv(N, bn);
  int64_t want = std::max<int64_t>(1, (2 * sm_count()) / tiles);
  int64_t sl = std::max<int64_t>(1, std::min<int64_t>(want, K / 64));
  int64_t ks = cdiv(cdiv(K, sl), BK) * BK;
  *kslice = (int)ks;
  *slices = (int)cdiv(K, ks);
}

int simt_conv_wgrad(const OmtConvGeo* g, const OmtAct* x, const OmtAct* gy, float* dw, float scale, float* part,
                    cudaStream_t s) {
  ConvArgs a = base_args(g);
  a.a = view(gy); a.b = view(x); a.scale = scale;
  a.M = g->co; a.N = g->ci * g->ks * g->ks; a.K = g->n * g->oh * g->ow;
  wgrad_slices(g, &a.slices, &a.kslice);
  a.out = a.slices == 1 ? dw : part;
  int r = launch_gemm<Wgrad>(a, a.M, a.N, a.slices, s, "conv_wgrad_simt");
  if (r != OMT_OK || a.slices == 1) return r;
  int64_t total = (int64_t)a.M * a.N;
  slab_sum_kernel<<<(unsigned)cdiv(total, 256), 256, 0, s>>>(part, dw, total, a.slices, scale);
  return check_launch("conv_wgrad_slab_sum");
}

size_t simt_wgrad_workspace(const OmtConvGeo* g) {
  int slices, kslice;
  wgrad_slices(g, &slices, &kslice);
  if (slices == 1) return 0;
  return (size_t)slices * g->co * g->ci * g->ks * g->ks * sizeof(float);
}

// ---------------------------------------------------------------------------------------------------------------------
// weight gradient without any allocation
// ---------------------------------------------------------------------------------------------------------------------
// Scratch for the split-K slabs of omt_conv_wgrad_noalloc. It lives in the library image: every GPU that loads the
// library holds these 16 MiB until the process exits. All calls on a device share it.
constexpr size_t NOALLOC_SCRATCH_FLOATS = (size_t)4 << 20;
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_SCRATCH_FLOATS];

constexpr int NOALLOC_MAX_DEVICES = 64;
static float* g_noalloc_ptr[NOALLOC_MAX_DEVICES];  // device address of g_noalloc_scratch, per device ordinal

}  // namespace omt

using namespace omt;

extern "C" size_t omt_conv_wgrad_noalloc_capacity(void) { return NOALLOC_SCRATCH_FLOATS * sizeof(float); }

extern "C" int omt_conv_wgrad_noalloc(const OmtConvGeo* g, const OmtAct* x, const OmtAct* gy, float* dw, float scale,
                                      omt_stream_t stream) {
  int r = check_dense(g, "omt_conv_wgrad_noalloc");  // the same checks as omt_conv_wgrad (extents below 2^31 included)
  if (r) return r;
  OMT_REQUIRE(x && gy && x->p && gy->p && dw, "omt_conv_wgrad_noalloc: null pointer");
  const size_t need = simt_wgrad_workspace(g);
  if (need > NOALLOC_SCRATCH_FLOATS * sizeof(float)) {
    set_error("omt_conv_wgrad_noalloc: this geometry needs %zu bytes of split-K scratch, the built-in scratch holds %zu", need,
              NOALLOC_SCRATCH_FLOATS * sizeof(float));
    return OMT_ETOOBIG;
  }
  int dev = -1;
  OMT_CUDA(cudaGetDevice(&dev));
  OMT_REQUIRE(dev >= 0 && dev < NOALLOC_MAX_DEVICES, "omt_conv_wgrad_noalloc: device ordinal %d out of range", dev);
  if (!g_noalloc_ptr[dev]) {
    // The array's name is only a host-side handle; the kernels need its address on the current device. Looked up once per
    // device (this first call should therefore come before any stream capture).
    float* p = nullptr;
    OMT_CUDA(cudaGetSymbolAddress((void**)&p, g_noalloc_scratch));
    g_noalloc_ptr[dev] = p;
  }
  return simt_conv_wgrad(g, x, gy, dw, scale, g_noalloc_ptr[dev], st(stream));
}

namespace omt {

// ---- bias gradient: db[c] = sum gy[:, c, :, :] ---------------------------------------------------------------------
// One block per (channel, slice) with 128-bit loads when the plane is contiguous, then a second tiny kernel; the
// reference used one workgroup per channel (csrc/kernels/csum_nchw.wgsl), i.e. 64 blocks for 64 channels.
__global__ void __launch_bounds__(256) csum_part_kernel(ActView gy, int n, int c, int h, int w, int S, float* part) {
  __shared__ float red[32];
  int ch = blockIdx.x, sl = blockIdx.y;
  int hw = h * w;
  float s = 0.f;
  bool plane = gy.sw == 1 && gy.sh == w;
  for (int img = sl; img < n; img += S) {
    if (plane) {
      const float* p = gy.p + img * gy.sn + ch * gy.sc;
      if (((reinterpret_cast<uintptr_t>(p) & 15) == 0) && (hw & 3) == 0) {
        const float4* p4 = reinterpret_cast<const float4*>(p);
        for (int e = threadIdx.x; e < hw / 4; e += blockDim.x) {
          float4 v = __ldg(p4 + e);
          s += (v.x + v.y) + (v.z + v.w);
        }
      } else {
        for (int e = threadIdx.x; e < hw; e += blockDim.x) s += __ldg(p + e);
      }
    } else {
      for (int e = threadIdx.x; e < hw; e += blockDim.x) s += __ldg(gy.p + gy.off(img, ch, e / w, e % w));
    }
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) part[ch * S + sl] = s;
}
__global__ void csum_fin_kernel(const float* part, int c, int S, float scale, float* out) {
  int ch = blockIdx.x * blockDim.x + threadIdx.x;
  if (ch >= c) return;
  float s = 0.f;
  for (int k = 0; k < S; k++) s += part[ch * S + k];
  out[ch] = s * scale;
}
// channels-last: threads across channels, blocks across pixel ranges, atomics avoided by a two-level sum
__global__ void __launch_bounds__(256) csum_nhwc_part_kernel(const float* __restrict__ gy, int64_t pixels, int c, int S,
                                                             float* part) {
  int ch = blockIdx.x * blockDim.x + threadIdx.x, sl = blockIdx.y;
  if (ch >= c) return;
  float s = 0.f;
  for (int64_t p = sl; p < pixels; p += S) s += __ldg(gy + p * c + ch);
  part[(int64_t)ch * S + sl] = s;
}

}  // namespace omt

using namespace omt;

extern "C" int omt_conv_bias_grad(const OmtAct* gy, int32_t n, int32_t c, int32_t h, int32_t w, float* db, float scale,
                                  omt_stream_t stream) {
  OMT_REQUIRE(gy && gy->p && db && n > 0 && c > 0 && h > 0 && w > 0, "omt_conv_bias_grad: bad arguments");
  cudaStream_t s = st(stream);
  bool nhwc = is_nhwc(gy, c, h, w) && c > 1;
  int S = nhwc ? (int)std::min<int64_t>(512, std::max<int64_t>(1, (int64_t)n * h * w / 64))
               : (int)std::min<int64_t>(n, std::max<int64_t>(1, (4 * sm_count()) / c));
  Scratch sc;
  int r = sc.get(nullptr, 0, (size_t)c * S * sizeof(float), stream);
  if (r) return r;
  float* part = (float*)sc.p;
  if (nhwc) {
    dim3 grid((unsigned)cdiv(c, 256), S);
    csum_nhwc_part_kernel<<<grid, 256, 0, s>>>(gy->p, (int64_t)n * h * w, c, S, part);
    r = check_launch("bias_grad_nhwc_part");
  } else {
    dim3 grid(c, S);
    csum_part_kernel<<<grid, 256, 0, s>>>(view(gy), n, c, h, w, S, part);
    r = check_launch("bias_grad_part");
  }
  if (r) return r;
  csum_fin_kernel<<<(unsigned)cdiv(c, 128), 128, 0, s>>>(part, c, S, scale, db);
  return check_launch("bias_grad_fin");
}

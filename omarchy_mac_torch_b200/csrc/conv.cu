// Dense convolution entry points: argument checks (the reference's conv_kind / NEED rules, csrc/conv.cpp:167-183),
// path selection (tcgen05 tensor-core kernels when the geometry and layout allow, exact-fp32 CUDA-core kernels
// otherwise), workspace handling, and two small copy helpers.
#include <algorithm>
#include <array>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

namespace omt {

// conv_simt.cu
int simt_conv_fwd(const OmtConvGeo* g, const OmtAct* x, const float* w, const float* bias, const OmtAct* y, uint32_t flags,
                  cudaStream_t s);
int simt_conv_dgrad(const OmtConvGeo* g, const OmtAct* gy, const float* w, const OmtAct* dx, cudaStream_t s);
int simt_conv_wgrad(const OmtConvGeo* g, const OmtAct* x, const OmtAct* gy, float* dw, float scale, float* part, cudaStream_t s);
size_t simt_wgrad_workspace(const OmtConvGeo* g);
// conv_tc.cu
bool tc_supported(int kind, const OmtConvGeo* g, const OmtAct* a, const OmtAct* b);
size_t tc_workspace(int kind, const OmtConvGeo* g);
int tc_conv_fwd(const OmtConvGeo* g, const OmtAct* x, const float* w, const float* bias, const OmtAct* y, float* stats,
                uint32_t flags, void* ws, cudaStream_t s);
int tc_conv_dgrad(const OmtConvGeo* g, const OmtAct* gy, const float* w, const OmtAct* dx, uint32_t flags, void* ws, cudaStream_t s);
int tc_conv_wgrad(const OmtConvGeo* g, const OmtAct* x, const OmtAct* gy, float* dw, float scale, void* ws, cudaStream_t s);
int tc_bnstats_groups(const OmtConvGeo* g, const OmtAct* x, const OmtAct* y);

// ---- per-geometry plan overrides (the reference's tuning cache g_conv_cache, csrc/conv.cpp:29-60, 116-155) ----
// key: pass (0 forward, 1 input gradient, 2 weight gradient), n, ci, co, ih, iw, oh, ow, ks, stride, pad
using PlanKey = std::array<int, 11>;
static std::map<PlanKey, PlanOverride> g_plans;
static std::mutex g_plans_mu;
static std::atomic<int> g_plans_count{0};
static PlanKey plan_key(int kind, const OmtConvGeo* g) {
  return {kind, g->n, g->ci, g->co, g->ih, g->iw, g->oh, g->ow, g->ks, g->stride, g->pad};
}
// installs the override stored for (kind, g) for the lifetime of the object (none stored: the planner's rules)
struct PlanScope {
  PlanOverride saved;
  PlanScope(int kind, const OmtConvGeo* g) : saved(tl_plan) {
    tl_plan = PlanOverride{0, 0.0};
    if (!g || g_plans_count.load(std::memory_order_relaxed) == 0) return;
    std::lock_guard<std::mutex> l(g_plans_mu);
    auto it = g_plans.find(plan_key(kind, g));
    if (it != g_plans.end()) tl_plan = it->second;
  }
  ~PlanScope() { tl_plan = saved; }
};

// ---- optional per-call timing of the three passes ----
static bool g_timing = false;
struct TimedCall {
  cudaEvent_t a, b;
  int kind;
  double flops, bytes;
};
static std::vector<TimedCall> g_timed;
static std::mutex g_timed_mu;
struct CallTimer {
  bool on;
  TimedCall c{};
  cudaStream_t s;
  CallTimer(int kind, const OmtConvGeo* g, cudaStream_t s_) : on(g_timing), s(s_) {
    if (!on) return;
    c.kind = kind;
    c.flops = 2.0 * g->n * g->co * g->oh * g->ow * (double)g->ci * g->ks * g->ks;
    c.bytes = 4.0 * ((double)g->n * g->ci * g->ih * g->iw + (double)g->n * g->co * g->oh * g->ow + (double)g->co * g->ci * g->ks * g->ks);
    if (cudaEventCreate(&c.a) != cudaSuccess || cudaEventCreate(&c.b) != cudaSuccess) { on = false; return; }
    cudaEventRecord(c.a, s);
  }
  ~CallTimer() {
    if (!on) return;
    cudaEventRecord(c.b, s);
    std::lock_guard<std::mutex> l(g_timed_mu);
    g_timed.push_back(c);
  }
};

__global__ void __launch_bounds__(256) scale_copy_kernel(float* __restrict__ dst, const float* __restrict__ src, int64_t n, float scale) {
  int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n) {
    float4 v = __ldg(reinterpret_cast<const float4*>(src + i));
    *reinterpret_cast<float4*>(dst + i) = make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale);
  } else {
    for (; i < n; i++) dst[i] = src[i] * scale;
  }
}
__global__ void __launch_bounds__(256) scale_copy_scalar_kernel(float* __restrict__ dst, const float* __restrict__ src, int64_t n, float scale) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = src[i] * scale;
}

// Layout change through a 32x32 shared tile: reads coalesced along the source's fast axis, writes along the
// destination's. View both tensors as [n][c][hw]; one of (c, hw) is contiguous in each.
__global__ void __launch_bounds__(256) transpose_kernel(const float* __restrict__ src, float* __restrict__ dst, int c, int hw,
                                                        bool src_c_fast) {
  __shared__ float tile[32][33];
  const int img = blockIdx.z;
  const int c0 = blockIdx.y * 32, p0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  const int64_t base = (int64_t)img * c * hw;
  if (src_c_fast) {  // src [hw][c] -> dst [c][hw]
    for (int j = ty; j < 32; j += 8) {
      int p = p0 + j, ch = c0 + tx;
      if (p < hw && ch < c) tile[j][tx] = __ldg(src + base + (int64_t)p * c + ch);
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
      int ch = c0 + j, p = p0 + tx;
      if (p < hw && ch < c) dst[base + (int64_t)ch * hw + p] = tile[tx][j];
    }
  } else {  // src [c][hw] -> dst [hw][c]
    for (int j = ty; j < 32; j += 8) {
      int ch = c0 + j, p = p0 + tx;
      if (p < hw && ch < c) tile[j][tx] = __ldg(src + base + (int64_t)ch * hw + p);
    }
    __syncthreads();
    for (int j = ty; j < 32; j += 8) {
      int p = p0 + j, ch = c0 + tx;
      if (p < hw && ch < c) dst[base + (int64_t)p * c + ch] = tile[tx][j];
    }
  }
}
__global__ void __launch_bounds__(256) strided_copy_kernel(ActView src, ActView dst, int n, int c, int h, int w) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)n * c * h * w) return;
  int x = (int)(i % w); i /= w;
  int y = (int)(i % h); i /= h;
  int ch = (int)(i % c), img = (int)(i / c);
  dst.p[dst.off(img, ch, y, x)] = __ldg(src.p + src.off(img, ch, y, x));
}

}  // namespace omt

using namespace omt;

// An NCHW-contiguous operand that the tensor-core path would take if it were channels-last: copy it into scratch from the
// library's allocator (one transpose pass) when that is what stands between the call and the tensor cores. Only without a
// caller workspace: omt_conv_workspace_bytes does not see layouts.
struct ClCopy {
  Scratch sc;
  OmtAct act{};
  bool made = false;
  int make(const OmtAct* a, int n, int c, int h, int w, omt_stream_t stream) {
    int r = sc.get(nullptr, 0, (size_t)n * c * h * w * sizeof(float), stream);
    if (r) return r;
    act.p = (float*)sc.p; act.sc = 1; act.sw = c; act.sh = (int64_t)w * c; act.sn = (int64_t)h * w * c;
    made = true;
    return omt_act_copy(a, &act, n, c, h, w, stream);
  }
};
static bool could_be_cl(const OmtAct* a, int c, int h, int w) { return a && a->p && c % 4 == 0 && is_nchw(a, c, h, w) && !is_nhwc(a, c, h, w); }
static OmtAct as_cl(const OmtAct* a, int c, int h, int w) {  // what the copy would look like (for the eligibility test)
  OmtAct r = *a;
  r.p = reinterpret_cast<float*>(256);  // aligned placeholder: only strides and alignment are inspected
  r.sc = 1; r.sw = c; r.sh = (int64_t)w * c; r.sn = (int64_t)h * w * c;
  return r;
}

// ---------------------------------------------------------------------------------------------------------------------
// Input gradient for <= 4 input channels (a network's first layer) on the tensor cores. As an implicit GEMM per stride phase
// its tiles would have ci <= 4 useful columns, and the work of loading and splitting the gy tiles does not shrink with the
// columns. So the sum is taken the other way round: T[p][(ky, kx, c)] = sum_co gy[p][co] * w[co][c][ky][kx] for every output
// pixel p is ONE dense product with ci * ks * ks columns (the input gradient of a 1x1 convolution: tcgen05 kernels, no waste),
// and dx(y, x, c) then gathers its taps from T (col2im): oy = (y + pad - ky) / s for the ky on y's stride phase
// (csrc/conv.cpp:78-95), likewise ox. T costs one write and one read of P * ci * ks^2 floats; for AlexNet's first layer
// (n = 16) that is 70 MB against a GEMM of 2.3 GFLOP. Used only with scratch from the library's allocator (T can be large).
// ---------------------------------------------------------------------------------------------------------------------
namespace omt {
constexpr size_t TAPS_MAX_BYTES = (size_t)1 << 30;  // beyond this T the CUDA-core kernel runs instead

__global__ void __launch_bounds__(256) taps_weight_kernel(const float* __restrict__ w, float* __restrict__ wm, int co, int ci, int kk, int colsp) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;  // wm[o][t * ci + c] = w[o][c][t]; columns past ci * kk are zero
  if (i >= co * colsp) return;
  const int o = i / colsp, col = i - o * colsp;
  const int t = col / ci, c = col - t * ci;
  wm[i] = t < kk ? __ldg(w + ((int64_t)o * ci + c) * kk + t) : 0.f;
}

struct Col2imArgs {
  const float* T;
  ActView dx;
  int n, ci, ih, iw, oh, ow, ks, stride, pad, colsp;
};
// one thread per input pixel (consecutive threads, consecutive x): the s threads of one stride period read s * ci consecutive
// floats of one row of T per tap
__global__ void __launch_bounds__(256) col2im_kernel(Col2imArgs a) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)a.n * a.ih * a.iw) return;
  const int x = (int)(i % a.iw);
  const int64_t r = i / a.iw;
  const int y = (int)(r % a.ih), img = (int)(r / a.ih);
  const int s = a.stride;
  const int ky0 = (y + a.pad) % s, kx0 = (x + a.pad) % s;
  const int qy = (y + a.pad - ky0) / s, qx = (x + a.pad - kx0) / s;  // output pixel reached through tap (ky0 + s*ty, kx0 + s*tx) is (qy - ty, qx - tx)
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int ky = ky0, oy = qy; ky < a.ks; ky += s, oy--) {
    if (oy < 0) break;
    if (oy >= a.oh) continue;
    for (int kx = kx0, ox = qx; kx < a.ks; kx += s, ox--) {
      if (ox < 0) break;
      if (ox >= a.ow) continue;
      const float* t = a.T + (((int64_t)img * a.oh + oy) * a.ow + ox) * a.colsp + (ky * a.ks + kx) * a.ci;
      for (int c = 0; c < a.ci; c++) acc[c] += __ldg(t + c);
    }
  }
  float* out = a.dx.p + a.dx.off(img, 0, y, x);
  for (int c = 0; c < a.ci; c++) out[(int64_t)c * a.dx.sc] = acc[c];
}

static int taps_cols(const OmtConvGeo* g) { return (int)cdiv((int64_t)g->ci * g->ks * g->ks, 8) * 8; }  // (a multiple of 32 bytes per row of T)
static OmtConvGeo taps_geo(const OmtConvGeo* g) { return OmtConvGeo{g->n, taps_cols(g), g->co, g->oh, g->ow, g->oh, g->ow, 1, 1, 0, 1}; }
// gy: the channels-last gradient (or what its channels-last copy would look like)
static bool dgrad_by_taps_ok(const OmtConvGeo* g, const OmtAct* gy_cl) {
  if (g->ci > 4 || g->groups != 1 || taps_cols(g) < 8) return false;
  const OmtConvGeo g1 = taps_geo(g);
  if ((size_t)g->n * g->oh * g->ow * g1.ci * sizeof(float) > TAPS_MAX_BYTES) return false;
  OmtAct t{reinterpret_cast<float*>(256), (int64_t)g1.ci * g->oh * g->ow, 1, (int64_t)g1.ci * g->ow, g1.ci};
  return tc_supported(1, &g1, gy_cl, &t);
}
static int dgrad_by_taps(const OmtConvGeo* g, const OmtAct* gy, const float* w, const OmtAct* dx, omt_stream_t stream) {
  const OmtConvGeo g1 = taps_geo(g);
  PlanScope plan(1, nullptr);  // the inner 1x1 product is another geometry: the planner's rules
  const int colsp = g1.ci, kk = g->ks * g->ks;
  const size_t P = (size_t)g->n * g->oh * g->ow;
  const size_t wm_floats = ((size_t)g->co * colsp + 63) / 64 * 64;
  Scratch sc, ws;
  int r = sc.get(nullptr, 0, (wm_floats + P * colsp) * sizeof(float), stream);
  if (r) return r;
  r = ws.get(nullptr, 0, tc_workspace(1, &g1), stream);
  if (r) return r;
  float* wm = (float*)sc.p;
  float* T = wm + wm_floats;
  cudaStream_t s = st(stream);
  taps_weight_kernel<<<(unsigned)cdiv((int64_t)g->co * colsp, 256), 256, 0, s>>>(w, wm, g->co, g->ci, kk, colsp);
  r = check_launch("conv_dgrad_taps_weights");
  if (r) return r;
  OmtAct t{T, (int64_t)colsp * g->oh * g->ow, 1, (int64_t)colsp * g->ow, colsp};
  r = tc_conv_dgrad(&g1, gy, wm, &t, 0, ws.p, s);
  if (r) return r;
  Col2imArgs a{T, view(dx), g->n, g->ci, g->ih, g->iw, g->oh, g->ow, g->ks, g->stride, g->pad, colsp};
  col2im_kernel<<<(unsigned)cdiv((int64_t)g->n * g->ih * g->iw, 256), 256, 0, s>>>(a);
  return check_launch("conv_dgrad_col2im");
}
}  // namespace omt

extern "C" {

size_t omt_conv_workspace_bytes(int kind, const OmtConvGeo* g, uint32_t flags) {
  if (!g || g->groups != 1) return 0;
  size_t simt = kind == 2 ? simt_wgrad_workspace(g) : 0;
  if (flags & OMT_FORCE_SIMT) return simt;
  PlanScope plan(kind, g);
  return std::max(simt, tc_workspace(kind, g));
}

int32_t omt_conv_bnstats_groups(const OmtConvGeo* g, const OmtAct* x, const OmtAct* y) {
  if (check_dense(g, "omt_conv_bnstats_groups") || !x || !y || !x->p || !y->p) return 0;
  PlanScope plan(0, g);
  return tc_bnstats_groups(g, x, y);
}

size_t omt_conv_bnstats_floats(int32_t groups, int32_t co) {
  if (groups <= 0 || co <= 0) return 0;
  return (size_t)groups * (2 * (size_t)co + 1) + (size_t)cdiv(co, 32);
}

int omt_conv_fwd(const OmtConvGeo* g, const OmtAct* x, const float* w, const float* bias, const OmtAct* y, float* stats,
                 uint32_t flags, void* workspace, size_t workspace_bytes, omt_stream_t stream) {
  int r = check_dense(g, "omt_conv_fwd");
  if (r) return r;
  PlanScope plan(0, g);
  OMT_REQUIRE(x && y && x->p && y->p && w, "omt_conv_fwd: null pointer");
  OMT_REQUIRE(!(flags & OMT_EPI_BIAS) || bias, "omt_conv_fwd: OMT_EPI_BIAS without a bias pointer");
  OMT_REQUIRE(!(flags & OMT_EPI_BNSTATS) || stats, "omt_conv_fwd: OMT_EPI_BNSTATS without a stats pointer");
  bool tc = !(flags & OMT_FORCE_SIMT) && tc_supported(0, g, x, y);
  CallTimer timer(0, g, st(stream));
  ClCopy xc;
  if (!tc && !(flags & (OMT_FORCE_SIMT | OMT_FORCE_TC)) && !workspace && could_be_cl(x, g->ci, g->ih, g->iw)) {
    OmtAct probe = as_cl(x, g->ci, g->ih, g->iw);
    if (tc_supported(0, g, &probe, y)) {
      r = xc.make(x, g->n, g->ci, g->ih, g->iw, stream);
      if (r) return r;
      x = &xc.act;
      tc = true;
    }
  }
  OMT_REQUIRE(tc || !(flags & OMT_FORCE_TC), "omt_conv_fwd: geometry/layout not covered by the tensor-core path");
  OMT_REQUIRE(tc || !(flags & OMT_EPI_BNSTATS), "omt_conv_fwd: OMT_EPI_BNSTATS needs the tensor-core path");
  if (!tc) return simt_conv_fwd(g, x, w, bias, y, flags, st(stream));
  Scratch sc;
  r = sc.get(workspace, workspace_bytes, tc_workspace(0, g), stream);
  if (r) return r;
  return tc_conv_fwd(g, x, w, bias, y, stats, flags, sc.p, st(stream));
}

int omt_conv_dgrad(const OmtConvGeo* g, const OmtAct* gy, const float* w, const OmtAct* dx, uint32_t flags, void* workspace,
                   size_t workspace_bytes, omt_stream_t stream) {
  int r = check_dense(g, "omt_conv_dgrad");
  if (r) return r;
  PlanScope plan(1, g);
  OMT_REQUIRE(gy && dx && gy->p && dx->p && w, "omt_conv_dgrad: null pointer");
  bool tc = !(flags & OMT_FORCE_SIMT) && tc_supported(1, g, gy, dx);
  CallTimer timer(1, g, st(stream));
  ClCopy gc;
  if (!tc && !(flags & (OMT_FORCE_SIMT | OMT_FORCE_TC)) && !workspace && could_be_cl(gy, g->co, g->oh, g->ow)) {
    OmtAct probe = as_cl(gy, g->co, g->oh, g->ow);
    if (tc_supported(1, g, &probe, dx)) {
      r = gc.make(gy, g->n, g->co, g->oh, g->ow, stream);
      if (r) return r;
      gy = &gc.act;
      tc = true;
    }
  }
  // few input channels: the product over all taps on the tensor cores, then a gather (library scratch only)
  if (!tc && g->ci <= 4 && !(flags & (OMT_FORCE_SIMT | OMT_EPI_ACCUM)) && !workspace) {
    const bool cg = could_be_cl(gy, g->co, g->oh, g->ow);
    OmtAct probe = cg ? as_cl(gy, g->co, g->oh, g->ow) : *gy;
    if (dgrad_by_taps_ok(g, &probe)) {
      if (cg) {
        r = gc.make(gy, g->n, g->co, g->oh, g->ow, stream);
        if (r) return r;
        gy = &gc.act;
      }
      return dgrad_by_taps(g, gy, w, dx, stream);
    }
  }
  OMT_REQUIRE(tc || !(flags & OMT_FORCE_TC), "omt_conv_dgrad: geometry/layout not covered by the tensor-core path");
  OMT_REQUIRE(tc || !(flags & OMT_EPI_ACCUM), "omt_conv_dgrad: OMT_EPI_ACCUM needs the tensor-core path");
  if (!tc) return simt_conv_dgrad(g, gy, w, dx, st(stream));
  Scratch sc;
  r = sc.get(workspace, workspace_bytes, tc_workspace(1, g), stream);
  if (r) return r;
  return tc_conv_dgrad(g, gy, w, dx, flags, sc.p, st(stream));
}

int omt_conv_wgrad(const OmtConvGeo* g, const OmtAct* x, const OmtAct* gy, float* dw, float scale, uint32_t flags, void* workspace,
                   size_t workspace_bytes, omt_stream_t stream) {
  int r = check_dense(g, "omt_conv_wgrad");
  if (r) return r;
  PlanScope plan(2, g);
  OMT_REQUIRE(x && gy && x->p && gy->p && dw, "omt_conv_wgrad: null pointer");
  bool tc = !(flags & OMT_FORCE_SIMT) && tc_supported(2, g, x, gy);
  CallTimer timer(2, g, st(stream));
  ClCopy xc, gc;
  if (!tc && !(flags & (OMT_FORCE_SIMT | OMT_FORCE_TC)) && !workspace) {
    const bool cx = could_be_cl(x, g->ci, g->ih, g->iw), cg = could_be_cl(gy, g->co, g->oh, g->ow);
    OmtAct px = cx ? as_cl(x, g->ci, g->ih, g->iw) : *x, pg = cg ? as_cl(gy, g->co, g->oh, g->ow) : *gy;
    if ((cx || cg) && tc_supported(2, g, &px, &pg)) {
      // a window-mode x (<= 4 channels) is staged by the kernel itself; everything else has to be channels-last
      OmtAct only_g = *x;
      const bool x_needed = cx && !tc_supported(2, g, &only_g, &pg);
      if (x_needed) {
        r = xc.make(x, g->n, g->ci, g->ih, g->iw, stream);
        if (r) return r;
        x = &xc.act;
      }
      if (cg) {
        r = gc.make(gy, g->n, g->co, g->oh, g->ow, stream);
        if (r) return r;
        gy = &gc.act;
      }
      tc = true;
    }
  }
  OMT_REQUIRE(tc || !(flags & OMT_FORCE_TC), "omt_conv_wgrad: geometry/layout not covered by the tensor-core path");
  Scratch sc;
  r = sc.get(workspace, workspace_bytes, tc ? tc_workspace(2, g) : simt_wgrad_workspace(g), stream);
  if (r) return r;
  if (tc) return tc_conv_wgrad(g, x, gy, dw, scale, sc.p, st(stream));
  return simt_conv_wgrad(g, x, gy, dw, scale, (float*)sc.p, st(stream));
}

int omt_gemm(const float* a, int64_t a_rs, int64_t a_cs, const float* b, int64_t b_rs, int64_t b_cs, const float* bias, float* out, int32_t M,
             int32_t N, int32_t K, omt_stream_t stream) {
  OMT_REQUIRE(a && b && out && M > 0 && N > 0 && K > 0, "omt_gemm: bad arguments");
  // a [rows, ch] row-major matrix as a channels-last activation of 1x1 images
  auto rows_act = [](const float* p, int64_t ch) { return OmtAct{const_cast<float*>(p), ch, 1, ch, ch}; };
  const bool a_rm = a_cs == 1 && a_rs == K, a_cm = a_rs == 1 && a_cs == M, b_rm = b_cs == 1 && b_rs == N, b_cm = b_rs == 1 && b_cs == K;
  OmtAct o = rows_act(out, N);
  if (a_rm && b_cm) {  // out[m, n] = sum_k A[m, k] W[n, k]: forward of a 1x1 convolution with weights W
    OmtConvGeo g{M, K, N, 1, 1, 1, 1, 1, 1, 0, 1};
    OmtAct x = rows_act(a, K);
    return omt_conv_fwd(&g, &x, b, bias, &o, nullptr, bias ? OMT_EPI_BIAS : 0u, nullptr, 0, stream);
  }
  OMT_REQUIRE(!bias, "omt_gemm: a bias is added only when B is column-major (the nn.Linear forward case)");
  if (a_rm && b_rm) {  // out[m, n] = sum_k A[m, k] B[k, n]: input gradient of a 1x1 convolution with weights B [co = K, ci = N]
    OmtConvGeo g{M, N, K, 1, 1, 1, 1, 1, 1, 0, 1};
    OmtAct gy = rows_act(a, K);
    return omt_conv_dgrad(&g, &gy, b, &o, 0, nullptr, 0, stream);
  }
  if (a_cm && b_rm) {  // out[m, n] = sum_k G[k, m] B[k, n]: weight gradient over K "pixels", gy = G [K, co = M], x = B [K, ci = N]
    OmtConvGeo g{K, N, M, 1, 1, 1, 1, 1, 1, 0, 1};
    OmtAct gy = rows_act(a, M), x = rows_act(b, N);
    return omt_conv_wgrad(&g, &x, &gy, out, 1.f, 0, nullptr, 0, stream);
  }
  set_error("omt_gemm: operand strides (%lld,%lld) x (%lld,%lld) match none of the three supported layouts", (long long)a_rs, (long long)a_cs,
            (long long)b_rs, (long long)b_cs);
  return OMT_EINVAL;
}

int omt_conv_timing(int enable) {
  g_timing = enable != 0;
  return OMT_OK;
}
int omt_conv_timing_read(double flops[3], double ms[3], int64_t calls[3], int reset) {
  std::lock_guard<std::mutex> l(g_timed_mu);
  for (int k = 0; k < 3; k++) { flops[k] = 0; ms[k] = 0; calls[k] = 0; }
  for (auto& c : g_timed) {
    OMT_CUDA(cudaEventSynchronize(c.b));
    float t = 0.f;
    OMT_CUDA(cudaEventElapsedTime(&t, c.a, c.b));
    flops[c.kind] += c.flops; ms[c.kind] += t; calls[c.kind]++;
  }
  if (reset) {
    for (auto& c : g_timed) { cudaEventDestroy(c.a); cudaEventDestroy(c.b); }
    g_timed.clear();
  }
  return OMT_OK;
}

int omt_conv_timing_bytes(double bytes[3]) {
  std::lock_guard<std::mutex> l(g_timed_mu);
  for (int k = 0; k < 3; k++) bytes[k] = 0;
  for (auto& c : g_timed) bytes[c.kind] += c.bytes;
  return OMT_OK;
}

int omt_scale_copy(float* dst, const float* src, int64_t n, float scale, omt_stream_t stream) {
  OMT_REQUIRE(dst && src && n >= 0, "omt_scale_copy: bad arguments");
  if (n == 0) return OMT_OK;
  if (((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0)
    scale_copy_kernel<<<(unsigned)cdiv(cdiv(n, 4), 256), 256, 0, st(stream)>>>(dst, src, n, scale);
  else
    scale_copy_scalar_kernel<<<(unsigned)cdiv(n, 256), 256, 0, st(stream)>>>(dst, src, n, scale);
  return check_launch("scale_copy");
}

int omt_act_copy(const OmtAct* src, const OmtAct* dst, int32_t n, int32_t c, int32_t h, int32_t w, omt_stream_t stream) {
  OMT_REQUIRE(src && dst && src->p && dst->p && n > 0 && c > 0 && h > 0 && w > 0, "omt_act_copy: bad arguments");
  bool s_nchw = is_nchw(src, c, h, w), s_nhwc = is_nhwc(src, c, h, w), d_nchw = is_nchw(dst, c, h, w), d_nhwc = is_nhwc(dst, c, h, w);
  int64_t total = (int64_t)n * c * h * w;
  if ((s_nchw && d_nchw) || (s_nhwc && d_nhwc)) return omt_memcpy_d2d(dst->p, src->p, total * sizeof(float), stream);
  if (((s_nchw && d_nhwc) || (s_nhwc && d_nchw)) && n <= 65535) {
    dim3 grid((unsigned)cdiv(h * w, 32), (unsigned)cdiv(c, 32), n);
    transpose_kernel<<<grid, 256, 0, st(stream)>>>(src->p, dst->p, c, h * w, s_nhwc);
    return check_launch("act_transpose");
  }
  strided_copy_kernel<<<(unsigned)cdiv(total, 256), 256, 0, st(stream)>>>(view(src), view(dst), n, c, h, w);
  return check_launch("act_strided_copy");
}

// ---- plan overrides and the timing pass that finds them (reference autotune / tune_dump / tune_load, csrc/conv.cpp:116-155, 243-272) ----

int omt_conv_plan_set(int kind, const OmtConvGeo* g, int32_t tile, double mult) {
  OMT_REQUIRE(g && kind >= 0 && kind <= 2, "omt_conv_plan_set: bad arguments");
  OMT_REQUIRE(tile == 0 || tile == 64 || tile == 128 || tile == 256 || (kind == 2 && tile == 192), "omt_conv_plan_set: tile width %d", (int)tile);
  OMT_REQUIRE(mult >= 0 && mult <= 16 && (kind == 2 || mult == 0 || mult == 1), "omt_conv_plan_set: slice factor %g", mult);
  std::lock_guard<std::mutex> l(g_plans_mu);
  if (tile == 0 && (mult == 0 || mult == 1)) g_plans.erase(plan_key(kind, g));
  else g_plans[plan_key(kind, g)] = PlanOverride{(int)tile, mult == 1 ? 0.0 : mult};
  g_plans_count.store((int)g_plans.size(), std::memory_order_relaxed);
  return OMT_OK;
}

int omt_conv_plan_get(int kind, const OmtConvGeo* g, int32_t* tile, double* mult) {
  OMT_REQUIRE(g && tile && mult, "omt_conv_plan_get: bad arguments");
  std::lock_guard<std::mutex> l(g_plans_mu);
  auto it = g_plans.find(plan_key(kind, g));
  *tile = it == g_plans.end() ? 0 : it->second.bn;
  *mult = it == g_plans.end() || it->second.mult == 0 ? 1.0 : it->second.mult;
  return it == g_plans.end() ? 0 : 1;
}

size_t omt_conv_plans_dump(char* buf, size_t n) {
  std::string out;
  {
    std::lock_guard<std::mutex> l(g_plans_mu);
    char line[160];
    for (auto& kv : g_plans) {
      int len = 0;
      for (int i = 0; i < 11; i++) len += snprintf(line + len, sizeof(line) - len, i ? ",%d" : "%d", kv.first[i]);
      snprintf(line + len, sizeof(line) - len, "=%d,%g\n", kv.second.bn, kv.second.mult == 0 ? 1.0 : kv.second.mult);
      out += line;
    }
  }
  if (buf && n) {
    const size_t m = std::min(n - 1, out.size());
    memcpy(buf, out.data(), m);
    buf[m] = 0;
  }
  return out.size();
}

int omt_conv_plans_load(const char* text) {
  OMT_REQUIRE(text, "omt_conv_plans_load: null text");
  int loaded = 0;
  const char* p = text;
  while (*p) {
    int k[11], tile = 0, used = 0;
    double mult = 1.0;
    const int got = sscanf(p, "%d,%d,%d,%d,%d,%d,%d,%d,%d,%d,%d=%d,%lf%n", &k[0], &k[1], &k[2], &k[3], &k[4], &k[5], &k[6], &k[7], &k[8], &k[9], &k[10],
                           &tile, &mult, &used);
    if (got == 13) {
      OmtConvGeo g{k[1], k[2], k[3], k[4], k[5], k[6], k[7], k[8], k[9], k[10], 1};
      if (k[0] >= 0 && k[0] <= 2 && omt_conv_plan_set(k[0], &g, tile, mult) == OMT_OK) loaded++;
    }
    while (*p && *p != '\n') p++;  // entries that do not parse or name a tile this build does not have are skipped
    if (*p) p++;
  }
  return loaded;
}

int omt_conv_autotune(int kind, const OmtConvGeo* g, int32_t* tile, double* mult, float* best_ms, float* rule_ms, omt_stream_t stream) {
  int r = check_dense(g, "omt_conv_autotune");
  if (r) return r;
  OMT_REQUIRE(kind >= 0 && kind <= 2, "omt_conv_autotune: pass %d", kind);
  if (tile) *tile = 0;
  if (mult) *mult = 1.0;
  if (best_ms) *best_ms = 0.f;
  if (rule_ms) *rule_ms = 0.f;
  cudaStream_t s = st(stream);
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  OMT_CUDA(cudaStreamIsCapturing(s, &cap));
  OMT_REQUIRE(cap == cudaStreamCaptureStatusNone, "omt_conv_autotune: the stream is being captured (the timing pass synchronises)");
  // channels-last operands filled with zeros (the kernels' time does not depend on the values)
  const size_t xn = (size_t)g->n * g->ci * g->ih * g->iw, yn = (size_t)g->n * g->co * g->oh * g->ow, wn = (size_t)g->co * g->ci * g->ks * g->ks;
  struct Buf {
    void* p = nullptr;
    ~Buf() { if (p) omt_free(p); }
  } bx, by, bw;
  bx.p = omt_malloc(xn * 4, stream); by.p = omt_malloc(yn * 4, stream); bw.p = omt_malloc(wn * 4, stream);
  OMT_REQUIRE(bx.p && by.p && bw.p, "omt_conv_autotune: out of device memory for the trial operands");
  OMT_CUDA(cudaMemsetAsync(bx.p, 0, xn * 4, s)); OMT_CUDA(cudaMemsetAsync(by.p, 0, yn * 4, s)); OMT_CUDA(cudaMemsetAsync(bw.p, 0, wn * 4, s));
  OmtAct ax{(float*)bx.p, (int64_t)g->ih * g->iw * g->ci, 1, (int64_t)g->iw * g->ci, g->ci};
  OmtAct ay{(float*)by.p, (int64_t)g->oh * g->ow * g->co, 1, (int64_t)g->ow * g->co, g->co};
  if (!(kind == 0 ? tc_supported(0, g, &ax, &ay) : kind == 1 ? tc_supported(1, g, &ay, &ax) : tc_supported(2, g, &ax, &ay))) return OMT_OK;
  // candidates: tile widths the geometry can fill; forward / input gradient only where no width splits the reduction over
  // CTAs (the statistics epilogue and the callers' workspace sizes then do not depend on the choice)
  std::vector<PlanOverride> cands;
  if (kind == 2) {
    const int chunks = g->ks * g->ks * (int)cdiv(g->ci, 32);
    for (int bn : {64, 128, 192, 256})
      if (bn / 32 <= 2 * chunks)
        for (double m : {0.5, 1.0, 2.0}) cands.push_back(PlanOverride{bn, m == 1.0 ? 0.0 : m});
  } else {
    const int cols = kind == 0 ? g->co : g->ci;
    const int64_t rows = kind == 0 ? (int64_t)g->n * g->oh * g->ow : (int64_t)g->n * cdiv(g->ih, g->stride) * cdiv(g->iw, g->stride);
    if (g->ci <= 4 || cols <= 128 || cdiv(rows, 128) * cdiv(cols, 256) * 2 <= sm_count()) return OMT_OK;  // (<= 128 columns: one width)
    cands.push_back(PlanOverride{128, 0.0});
    cands.push_back(PlanOverride{256, 0.0});
  }
  cudaEvent_t e0, e1;
  OMT_CUDA(cudaEventCreate(&e0));
  if (cudaEventCreate(&e1) != cudaSuccess) { cudaEventDestroy(e0); set_error("omt_conv_autotune: cudaEventCreate failed"); return OMT_ECUDA; }
  auto run = [&]() -> int {
    if (kind == 0) return omt_conv_fwd(g, &ax, (const float*)bw.p, nullptr, &ay, nullptr, 0, nullptr, 0, stream);
    if (kind == 1) return omt_conv_dgrad(g, &ay, (const float*)bw.p, &ax, 0, nullptr, 0, stream);
    return omt_conv_wgrad(g, &ax, &ay, (float*)bw.p, 1.f, 0, nullptr, 0, stream);
  };
  // one warm-up call, one timed call, then up to six more (about 15 ms of timing per candidate, as the reference's pass)
  auto time_it = [&](float* ms) -> int {
    int rr = run();
    if (rr) return rr;
    float first = 0.f, rest = 0.f;
    cudaEventRecord(e0, s);
    rr = run();
    cudaEventRecord(e1, s);
    if (rr || cudaEventSynchronize(e1) != cudaSuccess || cudaEventElapsedTime(&first, e0, e1) != cudaSuccess) return rr ? rr : OMT_ECUDA;
    const int reps = (int)std::max(1.0, std::min(6.0, 15.0 / std::max((double)first, 0.05)));
    *ms = first;
    if (reps > 1) {
      cudaEventRecord(e0, s);
      for (int i = 0; i < reps && !rr; i++) rr = run();
      cudaEventRecord(e1, s);
      if (rr || cudaEventSynchronize(e1) != cudaSuccess || cudaEventElapsedTime(&rest, e0, e1) != cudaSuccess) return rr ? rr : OMT_ECUDA;
      *ms = std::min(first, rest / reps);
    }
    return OMT_OK;
  };
  float base = 0.f, best = 0.f;
  PlanOverride best_plan{0, 0.0};
  omt_conv_plan_set(kind, g, 0, 0);  // the planner's rules first
  r = time_it(&base);
  best = base;
  for (size_t i = 0; i < cands.size() && !r; i++) {
    float ms = 0.f;
    if (omt_conv_plan_set(kind, g, cands[i].bn, cands[i].mult == 0 ? 1.0 : cands[i].mult) != OMT_OK) continue;
    r = time_it(&ms);
    if (!r && ms < best) { best = ms; best_plan = cands[i]; }
  }
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  // an override has to pay for itself: within 3 % of the rules' time the rules stay
  if (r || best > 0.97f * base) best_plan = PlanOverride{0, 0.0};
  omt_conv_plan_set(kind, g, best_plan.bn, best_plan.mult == 0 ? 1.0 : best_plan.mult);
  if (r) return r;
  if (tile) *tile = best_plan.bn;
  if (mult) *mult = best_plan.mult == 0 ? 1.0 : best_plan.mult;
  if (best_ms) *best_ms = best_plan.bn || best_plan.mult ? best : base;
  if (rule_ms) *rule_ms = base;
  return OMT_OK;
}

}  // extern "C"

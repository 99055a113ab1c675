// Shared internals of libomt_b200.so: error reporting, launch accounting, small device helpers.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/omt_b200.h"

namespace omt {

// ---- errors (thread-local message, sticky async flag) ----
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);  // records the message, returns OMT_ECUDA
void note_launch(const char* kernel);             // bumps the launch counter and the per-kernel count
int check_launch(const char* kernel);             // note_launch + cudaGetLastError

#define OMT_CUDA(call)                                          \
  do {                                                          \
    cudaError_t e_ = (call);                                    \
    if (e_ != cudaSuccess) return ::omt::cuda_fail(e_, #call);  \
  } while (0)

#define OMT_REQUIRE(cond, ...)       \
  do {                               \
    if (!(cond)) {                   \
      ::omt::set_error(__VA_ARGS__); \
      return OMT_EINVAL;             \
    }                                \
  } while (0)

// Per-kernel timing (omt_kernel_timing): every entry point turns its stream handle into a cudaStream_t with st(), which,
// while timing is on, records a "begin" event there; check_launch() then records an event after each launch, and a
// kernel's time is the distance to the event before it on the same thread.
extern bool g_kernel_timing;
void timing_begin(cudaStream_t s);
inline cudaStream_t st(omt_stream_t s) {
  if (g_kernel_timing) timing_begin((cudaStream_t)s);
  return (cudaStream_t)s;
}
inline int64_t cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

int sm_count();  // SMs of the current device (148 on B200)
int tc_error_word();  // conv_tc.cu: non-zero once a tensor-core kernel gave up on a bounded wait (-1: cannot read)

// Scratch from the library's own caching allocator, returned to the pool when the guard dies. The pool is
// stream-ordered: a block freed right after the launch is only handed to later work on the same stream.
struct Scratch {
  void* p = nullptr;
  bool owned = false;
  int get(void* user, size_t user_bytes, size_t need, omt_stream_t s) {
    if (need == 0) return OMT_OK;
    if (user) {
      if (user_bytes < need) {
        set_error("workspace too small: %zu < %zu bytes", user_bytes, need);
        return OMT_EWORKSPACE;
      }
      p = user;
      return OMT_OK;
    }
    p = omt_malloc(need, s);
    if (!p) return OMT_ENOMEM;
    owned = true;
    return OMT_OK;
  }
  ~Scratch() {
    if (owned) omt_free(p);
  }
};

// ---- device helpers ----
struct ActView {  // OmtAct by value for kernels
  float* p;
  int64_t sn, sc, sh, sw;
  __host__ __device__ int64_t off(int n, int c, int h, int w) const { return n * sn + c * sc + h * sh + w * sw; }
};
inline ActView view(const OmtAct* a) { return ActView{a->p, a->sn, a->sc, a->sh, a->sw}; }
// (the stride of a dimension of size 1 never enters an address: a [n, c, 1, 1] tensor is both layouts at once)
inline bool is_nchw(const OmtAct* a, int c, int h, int w) {
  return (w == 1 || a->sw == 1) && (h == 1 || a->sh == w) && (c == 1 || a->sc == (int64_t)h * w) && a->sn == (int64_t)c * h * w;
}
inline bool is_nhwc(const OmtAct* a, int c, int h, int w) {
  return (c == 1 || a->sc == 1) && (w == 1 || a->sw == c) && (h == 1 || a->sh == (int64_t)w * c) && a->sn == (int64_t)h * w * c;
}

// A per-geometry plan override for the tensor-core convolution kernels: `bn` = tile width in columns (0: the planner's
// rule), `mult` = factor on the weight gradient's split-K slice count (0: the rule). The public entry points install the
// override stored for their (pass, geometry), if any, in this thread-local for the duration of the call, so that every
// planning function the call reaches (tile choice, split-K, workspace size) sees the same one.
struct PlanOverride { int bn; double mult; };
extern thread_local PlanOverride tl_plan;

// Argument checks every dense-convolution entry point starts with (the reference's conv_kind / NEED rules,
// csrc/conv.cpp:167-183): a square kernel up to 11, stride 1..4, pad <= ks, consistent output size, GEMM extents below 2^31.
inline int check_dense(const OmtConvGeo* g, const char* who) {
  OMT_REQUIRE(g != nullptr, "%s: null geometry", who);
  OMT_REQUIRE(g->groups == 1, "%s: groups must be 1 (use omt_dw_* for depthwise)", who);
  OMT_REQUIRE(g->n > 0 && g->ci > 0 && g->co > 0 && g->ih > 0 && g->iw > 0, "%s: empty tensor", who);
  OMT_REQUIRE(g->ks >= 1 && g->ks <= 11 && g->stride >= 1 && g->stride <= 4 && g->pad >= 0 && g->pad <= g->ks,
              "%s: needs ks<=11, stride 1..4, pad<=ks (got ks=%d stride=%d pad=%d)", who, g->ks, g->stride, g->pad);
  OMT_REQUIRE(g->oh == (g->ih + 2 * g->pad - g->ks) / g->stride + 1 && g->ow == (g->iw + 2 * g->pad - g->ks) / g->stride + 1 &&
                  g->oh > 0 && g->ow > 0,
              "%s: output size does not match the geometry", who);
  OMT_REQUIRE((int64_t)g->n * g->oh * g->ow < (1ll << 31) && (int64_t)g->n * g->ih * g->iw < (1ll << 31) &&
                  (int64_t)g->co * g->ci * g->ks * g->ks < (1ll << 31),
              "%s: GEMM extent exceeds 2^31", who);
  return OMT_OK;
}

#ifdef __CUDACC__
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// Sum over a block of up to 1024 threads; result valid in every thread. `red` holds 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[wid] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : 0.f;
  r = warp_sum(r);
  return r;
}
#endif

}  // namespace omt

// Classification loss on [rows, cols] float32 logits: log-softmax over the last dimension, negative log-likelihood with
// int64 targets (optional class weights, ignore_index, reductions none / mean / sum), their gradients, and the fused pair
// F.cross_entropy decomposes into. Replaces softmax.wgsl (mode 1), softmax_bwd.wgsl, nll_fwd.wgsl + the two row reductions
// and the division behind them, and nll_bwd.wgsl as driven by csrc/reduce.cpp:128-201.
//
// One warp owns a row (three passes over it: max, sum of exponentials, write; the second and third hit L1). The fused
// forward writes log-probabilities, per-row losses and weights, and the block that takes the last ticket sums the rows in
// a fixed order, so loss and total weight come out of the same launch, deterministically. These matrices are small
// ([batch, classes]); what the fusion saves is launches, not bandwidth.
#include "common.cuh"

namespace omt {

constexpr int LOSS_WARPS = 8;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// logsumexp pieces of one row for the calling warp: returns max and log(sum(exp(x - max)))
__device__ __forceinline__ void row_lse(const float* __restrict__ xr, int cols, int lane, float& mx, float& lse) {
  mx = -INFINITY;
  for (int j = lane; j < cols; j += 32) mx = fmaxf(mx, __ldg(xr + j));
  mx = warp_max(mx);
  float s = 0.f;
  for (int j = lane; j < cols; j += 32) s += expf(__ldg(xr + j) - mx);
  lse = logf(warp_sum(s));
}

// per-row loss term: -w[t] * logp[t]; rows whose target is ignore_index count nothing, a target outside [0, cols) gives NaN
__device__ __forceinline__ void row_nll(float lp_t_or_nan, int64_t t, int64_t ignore, const float* __restrict__ weight, int cols, float& loss, float& w) {
  if (t == ignore) { loss = 0.f; w = 0.f; return; }
  if (t < 0 || t >= cols) { loss = NAN; w = 0.f; return; }
  w = weight ? __ldg(weight + t) : 1.f;
  loss = -w * lp_t_or_nan;
}

struct LossArgs {
  const float* x;       // logits (fused, log_softmax) or log-probabilities (nll)
  const int64_t* target;
  const float* weight;  // [cols] or null
  float* logp;          // [rows, cols] out (fused, log_softmax) or null
  float* loss;          // reduction none: [rows]; else [1]
  float* total_weight;  // [1]
  float* row_loss;      // scratch [rows] (mean / sum)
  float* row_w;         // scratch [rows]
  unsigned int* ticket; // scratch word, zero before the launch
  int64_t rows, ignore;
  int32_t cols, reduction;  // 0 none, 1 mean, 2 sum
};

// SOFTMAX: x holds logits and logp is written; else x holds log-probabilities. NLL: the loss part runs.
template <bool SOFTMAX, bool NLL>
__global__ void __launch_bounds__(LOSS_WARPS * 32) loss_fwd_kernel(LossArgs a) {
  __shared__ float red[32];
  __shared__ bool last;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  for (int64_t r = (int64_t)blockIdx.x * LOSS_WARPS + wid; r < a.rows; r += (int64_t)gridDim.x * LOSS_WARPS) {
    const float* xr = a.x + r * a.cols;
    float mx = 0.f, lse = 0.f;
    if (SOFTMAX) {
      row_lse(xr, a.cols, lane, mx, lse);
      float* lr = a.logp + r * a.cols;
      for (int j = lane; j < a.cols; j += 32) lr[j] = __ldg(xr + j) - mx - lse;
    }
    if (NLL && lane == 0) {
      const int64_t t = a.target[r];
      const bool ok = t != a.ignore && t >= 0 && t < a.cols;
      const float lp = ok ? __ldg(xr + t) - mx - lse : 0.f;
      float l, w;
      row_nll(lp, t, a.ignore, a.weight, a.cols, l, w);
      if (a.reduction == 0) a.loss[r] = l;
      else { a.row_loss[r] = l; a.row_w[r] = w; }
    }
  }
  if (!NLL) return;
  if (a.reduction == 0) {
    if (blockIdx.x == 0 && threadIdx.x == 0) *a.total_weight = 0.f;
    return;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(a.ticket, 1u) == gridDim.x - 1;
  __syncthreads();
  if (!last) return;
  __threadfence();
  float sl = 0.f, sw = 0.f;
  for (int64_t r = threadIdx.x; r < a.rows; r += blockDim.x) { sl += __ldcg(a.row_loss + r); sw += __ldcg(a.row_w + r); }
  sl = block_sum(sl, red);
  sw = block_sum(sw, red);
  if (threadIdx.x == 0) {
    *a.loss = a.reduction == 1 ? sl / sw : sl;
    *a.total_weight = sw;
  }
}

struct LossBwdArgs {
  const float* g;       // log_softmax backward: [rows, cols]; nll / fused: [rows] (reduction none) or [1]
  const float* logp;
  const int64_t* target;
  const float* weight;
  const float* total_weight;
  float* dx;
  int64_t rows, ignore;
  int32_t cols, reduction;
};

// dx = g - exp(logp) * rowsum(g)
__global__ void __launch_bounds__(LOSS_WARPS * 32) log_softmax_bwd_kernel(LossBwdArgs a) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  for (int64_t r = (int64_t)blockIdx.x * LOSS_WARPS + wid; r < a.rows; r += (int64_t)gridDim.x * LOSS_WARPS) {
    const float* gr = a.g + r * a.cols;
    const float* lr = a.logp + r * a.cols;
    float s = 0.f;
    for (int j = lane; j < a.cols; j += 32) s += __ldg(gr + j);
    s = warp_sum(s);
    float* dr = a.dx + r * a.cols;
    for (int j = lane; j < a.cols; j += 32) dr[j] = __ldg(gr + j) - expf(__ldg(lr + j)) * s;
  }
}

// the scale a row's gradient carries: w[t] * g / (total weight for mean); 0 for ignored (and out-of-range) targets
__device__ __forceinline__ float row_scale(const LossBwdArgs& a, int64_t r, int64_t t) {
  if (t == a.ignore || t < 0 || t >= a.cols) return 0.f;
  const float w = a.weight ? __ldg(a.weight + t) : 1.f;
  const float g = __ldg(a.g + (a.reduction == 0 ? r : 0));
  return a.reduction == 1 ? w * g / __ldg(a.total_weight) : w * g;
}

// FUSED: dx = (exp(logp) - onehot(t)) * scale (gradient with respect to the logits); else dlogp = -onehot(t) * scale
template <bool FUSED>
__global__ void __launch_bounds__(LOSS_WARPS * 32) nll_bwd_kernel(LossBwdArgs a) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  for (int64_t r = (int64_t)blockIdx.x * LOSS_WARPS + wid; r < a.rows; r += (int64_t)gridDim.x * LOSS_WARPS) {
    const int64_t t = a.target[r];
    const float s = row_scale(a, r, t);
    float* dr = a.dx + r * a.cols;
    const float* lr = FUSED ? a.logp + r * a.cols : nullptr;
    for (int j = lane; j < a.cols; j += 32) {
      const float hot = j == t ? 1.f : 0.f;
      dr[j] = FUSED ? (expf(__ldg(lr + j)) - hot) * s : -hot * s;
    }
  }
}

static unsigned loss_grid(int64_t rows) { return (unsigned)std::min<int64_t>(cdiv(rows, LOSS_WARPS), 148 * 8); }

static int check_rows(int64_t rows, int32_t cols, const char* who) {
  OMT_REQUIRE(rows > 0 && cols > 0, "%s: empty matrix", who);
  return OMT_OK;
}

template <bool SOFTMAX>
static int nll_forward(const float* x, const int64_t* target, const float* weight, float* logp, float* loss, float* total_weight, int64_t rows,
                       int32_t cols, int64_t ignore, int32_t reduction, omt_stream_t stream, const char* name) {
  OMT_REQUIRE(x && target && loss && total_weight && (!SOFTMAX || logp), "%s: null pointer", name);
  OMT_REQUIRE(reduction >= 0 && reduction <= 2, "%s: reduction must be 0 (none), 1 (mean) or 2 (sum)", name);
  if (int e = check_rows(rows, cols, name)) return e;
  LossArgs a{};
  a.x = x; a.target = target; a.weight = weight; a.logp = logp; a.loss = loss; a.total_weight = total_weight;
  a.rows = rows; a.cols = cols; a.ignore = ignore; a.reduction = reduction;
  Scratch sc;
  if (reduction != 0) {
    const size_t need = (size_t)(2 * rows + 1) * sizeof(float);
    if (int e = sc.get(nullptr, 0, need, stream)) return e;
    a.row_loss = (float*)sc.p;
    a.row_w = a.row_loss + rows;
    a.ticket = (unsigned int*)(a.row_w + rows);
    OMT_CUDA(cudaMemsetAsync(a.ticket, 0, sizeof(unsigned int), st(stream)));
  }
  loss_fwd_kernel<SOFTMAX, true><<<loss_grid(rows), LOSS_WARPS * 32, 0, st(stream)>>>(a);
  return check_launch(name);
}

}  // namespace omt

using namespace omt;

extern "C" {

int omt_log_softmax(const float* x, float* logp, int64_t rows, int32_t cols, omt_stream_t stream) {
  OMT_REQUIRE(x && logp, "omt_log_softmax: null pointer");
  if (int e = check_rows(rows, cols, "omt_log_softmax")) return e;
  LossArgs a{};
  a.x = x; a.logp = logp; a.rows = rows; a.cols = cols;
  loss_fwd_kernel<true, false><<<loss_grid(rows), LOSS_WARPS * 32, 0, st(stream)>>>(a);
  return check_launch("log_softmax");
}

int omt_log_softmax_backward(const float* g, const float* logp, float* dx, int64_t rows, int32_t cols, omt_stream_t stream) {
  OMT_REQUIRE(g && logp && dx, "omt_log_softmax_backward: null pointer");
  if (int e = check_rows(rows, cols, "omt_log_softmax_backward")) return e;
  LossBwdArgs a{};
  a.g = g; a.logp = logp; a.dx = dx; a.rows = rows; a.cols = cols;
  log_softmax_bwd_kernel<<<loss_grid(rows), LOSS_WARPS * 32, 0, st(stream)>>>(a);
  return check_launch("log_softmax_bwd");
}

int omt_nll_loss(const float* logp, const int64_t* target, const float* weight, float* loss, float* total_weight, int64_t rows, int32_t cols,
                 int64_t ignore_index, int32_t reduction, omt_stream_t stream) {
  return nll_forward<false>(logp, target, weight, nullptr, loss, total_weight, rows, cols, ignore_index, reduction, stream, "nll_fwd");
}

int omt_softmax_nll(const float* x, const int64_t* target, const float* weight, float* logp, float* loss, float* total_weight, int64_t rows,
                    int32_t cols, int64_t ignore_index, int32_t reduction, omt_stream_t stream) {
  return nll_forward<true>(x, target, weight, logp, loss, total_weight, rows, cols, ignore_index, reduction, stream, "softmax_nll_fwd");
}

static int nll_backward(bool fused, const float* g, const float* logp, const int64_t* target, const float* weight, const float* total_weight,
                        float* dx, int64_t rows, int32_t cols, int64_t ignore, int32_t reduction, omt_stream_t stream) {
  const char* name = fused ? "softmax_nll_bwd" : "nll_bwd";
  OMT_REQUIRE(g && target && dx && (!fused || logp) && (reduction != 1 || total_weight), "%s: null pointer", name);
  OMT_REQUIRE(reduction >= 0 && reduction <= 2, "%s: reduction must be 0 (none), 1 (mean) or 2 (sum)", name);
  if (int e = check_rows(rows, cols, name)) return e;
  LossBwdArgs a{};
  a.g = g; a.logp = logp; a.target = target; a.weight = weight; a.total_weight = total_weight; a.dx = dx;
  a.rows = rows; a.cols = cols; a.ignore = ignore; a.reduction = reduction;
  if (fused) nll_bwd_kernel<true><<<loss_grid(rows), LOSS_WARPS * 32, 0, st(stream)>>>(a);
  else nll_bwd_kernel<false><<<loss_grid(rows), LOSS_WARPS * 32, 0, st(stream)>>>(a);
  return check_launch(name);
}

int omt_nll_loss_backward(const float* g, const int64_t* target, const float* weight, const float* total_weight, float* dlogp, int64_t rows,
                          int32_t cols, int64_t ignore_index, int32_t reduction, omt_stream_t stream) {
  return nll_backward(false, g, nullptr, target, weight, total_weight, dlogp, rows, cols, ignore_index, reduction, stream);
}

int omt_softmax_nll_backward(const float* g, const float* logp, const int64_t* target, const float* weight, const float* total_weight, float* dx,
                             int64_t rows, int32_t cols, int64_t ignore_index, int32_t reduction, omt_stream_t stream) {
  return nll_backward(true, g, logp, target, weight, total_weight, dx, rows, cols, ignore_index, reduction, stream);
}

}  // extern "C"

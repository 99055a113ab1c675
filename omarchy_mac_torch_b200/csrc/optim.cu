// Fused SGD and Adam/AdamW: one launch updates every parameter tensor of the step (multi-tensor), 128-bit accesses,
// each element read and written exactly once (SGD+momentum 20 B/param, Adam 28 B/param).
//
// Arithmetic follows the reference shaders line by line in meaning: sgd.wgsl:9-24 (maximize, weight decay, momentum
// with dampening, first-step rule, nesterov) and adam.wgsl:13-27 (step count read from the parameter's device step
// tensor, bias corrections computed on the device, decoupled decay for AdamW). The reference dispatches once per
// parameter (csrc/optim.cpp:20-25, 41-46); here a chunk table maps blocks to (tensor, offset).
#include <vector>

#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace omt {

constexpr int CHUNK = 4096;  // elements per block: 256 threads x 4 float4

struct DevParam {
  float* p;
  const float* g;
  float* m;
  float* v;
  const float* step;
  int64_t numel;
  int64_t first_chunk;  // index of this tensor's first chunk in the grid
};

struct SgdH { float lr, mom, damp, wd; int nesterov, first, maximize; };
struct AdamH { float lr, b1, b2, eps, wd; int decoupled, maximize; };

__device__ __forceinline__ int find_tensor(const DevParam* t, int count, int64_t chunk) {
  int lo = 0, hi = count - 1;
  while (lo < hi) {  // last tensor with first_chunk <= chunk
    int mid = (lo + hi + 1) >> 1;
    if (t[mid].first_chunk <= chunk) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ void sgd_one(const SgdH& h, float& pv, float gr, float& mv, bool has_m) {
  if (h.maximize) gr = -gr;
  gr = gr + h.wd * pv;
  float d = gr;
  if (has_m) {
    float v = gr;
    if (!h.first) v = h.mom * mv + (1.f - h.damp) * gr;
    mv = v;
    d = h.nesterov ? gr + h.mom * v : v;
  }
  pv = pv - h.lr * d;
}

__global__ void __launch_bounds__(256) sgd_kernel(const DevParam* __restrict__ table, int count, SgdH h) {
  const int ti = find_tensor(table, count, blockIdx.x);
  const DevParam t = table[ti];
  const int64_t base = ((int64_t)blockIdx.x - t.first_chunk) * CHUNK;
  const bool has_m = h.mom != 0.f && t.m != nullptr;
  const bool vec = ((reinterpret_cast<uintptr_t>(t.p) | reinterpret_cast<uintptr_t>(t.g) | reinterpret_cast<uintptr_t>(t.m)) & 15) == 0;
  if (vec) {
#pragma unroll
    for (int r = 0; r < 4; r++) {
      int64_t i = base + ((int64_t)r * 256 + threadIdx.x) * 4;
      if (i + 3 < t.numel) {
        float4 pv = *reinterpret_cast<float4*>(t.p + i), gv = __ldg(reinterpret_cast<const float4*>(t.g + i));
        float4 mv = has_m ? *reinterpret_cast<float4*>(t.m + i) : make_float4(0, 0, 0, 0);
        sgd_one(h, pv.x, gv.x, mv.x, has_m); sgd_one(h, pv.y, gv.y, mv.y, has_m);
        sgd_one(h, pv.z, gv.z, mv.z, has_m); sgd_one(h, pv.w, gv.w, mv.w, has_m);
        *reinterpret_cast<float4*>(t.p + i) = pv;
        if (has_m) *reinterpret_cast<float4*>(t.m + i) = mv;
      } else {
        for (int64_t j = i; j < t.numel && j < i + 4; j++) {
          float pv = t.p[j], mv = has_m ? t.m[j] : 0.f;
          sgd_one(h, pv, t.g[j], mv, has_m);
          t.p[j] = pv;
          if (has_m) t.m[j] = mv;
        }
      }
    }
  } else {
    for (int64_t j = base + threadIdx.x; j < t.numel && j < base + CHUNK; j += 256) {
      float pv = t.p[j], mv = has_m ? t.m[j] : 0.f;
      sgd_one(h, pv, t.g[j], mv, has_m);
      t.p[j] = pv;
      if (has_m) t.m[j] = mv;
    }
  }
}

__device__ __forceinline__ void adam_one(const AdamH& h, float bc1, float sbc2, float& pv, float gr, float& mi, float& vi) {
  if (h.maximize) gr = -gr;
  if (h.decoupled) pv = pv * (1.f - h.lr * h.wd); else gr = gr + h.wd * pv;
  mi = mi + (1.f - h.b1) * (gr - mi);
  vi = h.b2 * vi + (1.f - h.b2) * gr * gr;
  pv = pv - (h.lr / bc1) * mi / (sqrtf(vi) / sbc2 + h.eps);
}

__global__ void __launch_bounds__(256) adam_kernel(const DevParam* __restrict__ table, int count, AdamH h) {
  const int ti = find_tensor(table, count, blockIdx.x);
  const DevParam t = table[ti];
  const int64_t base = ((int64_t)blockIdx.x - t.first_chunk) * CHUNK;
  const float step = __ldg(t.step);
  const float bc1 = 1.f - powf(h.b1, step), sbc2 = sqrtf(1.f - powf(h.b2, step));
  const bool vec = ((reinterpret_cast<uintptr_t>(t.p) | reinterpret_cast<uintptr_t>(t.g) | reinterpret_cast<uintptr_t>(t.m) |
                     reinterpret_cast<uintptr_t>(t.v)) & 15) == 0;
  if (vec) {
#pragma unroll
    for (int r = 0; r < 4; r++) {
      int64_t i = base + ((int64_t)r * 256 + threadIdx.x) * 4;
      if (i + 3 < t.numel) {
        float4 pv = *reinterpret_cast<float4*>(t.p + i), gv = __ldg(reinterpret_cast<const float4*>(t.g + i));
        float4 mv = *reinterpret_cast<float4*>(t.m + i), vv = *reinterpret_cast<float4*>(t.v + i);
        adam_one(h, bc1, sbc2, pv.x, gv.x, mv.x, vv.x); adam_one(h, bc1, sbc2, pv.y, gv.y, mv.y, vv.y);
        adam_one(h, bc1, sbc2, pv.z, gv.z, mv.z, vv.z); adam_one(h, bc1, sbc2, pv.w, gv.w, mv.w, vv.w);
        *reinterpret_cast<float4*>(t.p + i) = pv;
        *reinterpret_cast<float4*>(t.m + i) = mv;
        *reinterpret_cast<float4*>(t.v + i) = vv;
      } else {
        for (int64_t j = i; j < t.numel && j < i + 4; j++) {
          float pv = t.p[j], mv = t.m[j], vv = t.v[j];
          adam_one(h, bc1, sbc2, pv, t.g[j], mv, vv);
          t.p[j] = pv; t.m[j] = mv; t.v[j] = vv;
        }
      }
    }
  } else {
    for (int64_t j = base + threadIdx.x; j < t.numel && j < base + CHUNK; j += 256) {
      float pv = t.p[j], mv = t.m[j], vv = t.v[j];
      adam_one(h, bc1, sbc2, pv, t.g[j], mv, vv);
      t.p[j] = pv; t.m[j] = mv; t.v[j] = vv;
    }
  }
}

// builds the device table; returns total chunks (0 if nothing to do) or a negative error
static int64_t stage_table(const OmtParam* table, int32_t count, bool adam, omt_stream_t stream, Scratch& sc) {
  std::vector<DevParam> host;
  host.reserve(count);
  int64_t chunks = 0;
  for (int i = 0; i < count; i++) {
    const OmtParam& t = table[i];
    if (t.numel <= 0) continue;
    if (!t.p || !t.g || (adam && (!t.m || !t.v || !t.step))) {
      set_error("optimizer table entry %d has a null pointer", i);
      return OMT_EINVAL;
    }
    host.push_back({t.p, t.g, t.m, t.v, t.step, t.numel, chunks});
    chunks += cdiv(t.numel, CHUNK);
  }
  if (host.empty()) return 0;
  size_t bytes = host.size() * sizeof(DevParam);
  // The table of a training loop is the same every step (same parameter, gradient and state addresses), so device copies
  // are kept and reused: no host-to-device copy on the steady-state path, which also keeps a step capturable in a CUDA
  // graph (a copy from a temporary host buffer would be replayed from freed memory).
  // The upload is ordered on the stream of the call that made it; a later call on another stream waits for the entry's
  // `ready` event first and registers itself as a user of the block, so that an evicted table is not recycled under it.
  struct Cached { std::vector<DevParam> host; void* dev = nullptr; uint64_t used = 0; cudaStream_t stream = nullptr; cudaEvent_t ready = nullptr; };
  static std::mutex mu;
  static Cached cache[8];
  static uint64_t tick = 0;
  std::lock_guard<std::mutex> lock(mu);
  Cached* slot = &cache[0];
  for (Cached& c : cache) {
    if (c.dev && c.host.size() == host.size() && std::memcmp(c.host.data(), host.data(), bytes) == 0) {
      c.used = ++tick;
      if (c.stream != st(stream)) {
        if (c.ready && cudaStreamWaitEvent(st(stream), c.ready, 0) != cudaSuccess) return cuda_fail(cudaGetLastError(), "cudaStreamWaitEvent(optimizer table)");
        omt_record_stream(c.dev, stream);
      }
      sc.p = c.dev;  // not owned by the Scratch
      return ((int64_t)host.size() << 40) | chunks;
    }
    if (c.used < slot->used) slot = &c;
  }
  if (slot->dev) omt_free(slot->dev);  // stream-ordered: kernels already queued with the old table are unaffected
  slot->dev = omt_malloc(bytes, stream);
  if (!slot->dev) return OMT_ENOMEM;
  slot->host = std::move(host);
  slot->used = ++tick;
  // pageable source that stays alive in the cache entry
  cudaError_t e = cudaMemcpyAsync(slot->dev, slot->host.data(), bytes, cudaMemcpyHostToDevice, st(stream));
  if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpyAsync(optimizer table)");
  slot->stream = st(stream);
  if (!slot->ready && cudaEventCreateWithFlags(&slot->ready, cudaEventDisableTiming) != cudaSuccess) slot->ready = nullptr;
  if (slot->ready) cudaEventRecord(slot->ready, st(stream));
  sc.p = slot->dev;
  return ((int64_t)slot->host.size() << 40) | chunks;
}

}  // namespace omt

using namespace omt;

extern "C" {

int omt_sgd(const OmtParam* table, int32_t count, float lr, float momentum, float dampening, float weight_decay, int32_t nesterov,
            int32_t first_step, int32_t maximize, omt_stream_t stream) {
  OMT_REQUIRE(count >= 0 && (count == 0 || table), "omt_sgd: bad table");
  Scratch sc;
  int64_t r = stage_table(table, count, false, stream, sc);
  if (r <= 0) return (int)r;
  int tensors = (int)(r >> 40);
  int64_t chunks = r & (((int64_t)1 << 40) - 1);
  SgdH h{lr, momentum, dampening, weight_decay, nesterov, first_step, maximize};
  sgd_kernel<<<(unsigned)chunks, 256, 0, st(stream)>>>((const DevParam*)sc.p, tensors, h);
  return check_launch("sgd_multi");
}

int omt_adam(const OmtParam* table, int32_t count, float lr, float beta1, float beta2, float eps, float weight_decay,
             int32_t decoupled, int32_t maximize, omt_stream_t stream) {
  OMT_REQUIRE(count >= 0 && (count == 0 || table), "omt_adam: bad table");
  Scratch sc;
  int64_t r = stage_table(table, count, true, stream, sc);
  if (r <= 0) return (int)r;
  int tensors = (int)(r >> 40);
  int64_t chunks = r & (((int64_t)1 << 40) - 1);
  AdamH h{lr, beta1, beta2, eps, weight_decay, decoupled, maximize};
  adam_kernel<<<(unsigned)chunks, 256, 0, st(stream)>>>((const DevParam*)sc.p, tensors, h);
  return check_launch("adam_multi");
}

}  // extern "C"

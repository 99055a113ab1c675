// Runtime half of libomt_b200.so: device selection, error state, caching allocator, streams/events, transfers,
// launch accounting. Replaces the reference's wgpu runtime (csrc/runtime.cpp) and the allocator / guard parts of
// csrc/device.cpp with CUDA equivalents behind a C ABI.
#include <algorithm>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"

namespace omt {

static thread_local char t_err[512];
static int g_sticky = 0;  // first asynchronous failure seen (cudaError_t), reported by omt_check_errors
static std::mutex g_mu;
static int g_device = -1;
static int g_sms = 0;
static uint64_t g_launches = 0;
static std::map<std::string, uint64_t> g_kcount;

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_err, sizeof(t_err), fmt, ap);
  va_end(ap);
}
int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
  // Sticky only for errors that leave the device in doubt. A launch the runtime refused up front (bad grid, too much
  // shared memory, a bad argument) or an allocation that failed has run nothing: the caller gets its code and carries on.
  const bool recoverable = e == cudaErrorMemoryAllocation || e == cudaErrorNotReady || e == cudaErrorInvalidConfiguration ||
                           e == cudaErrorInvalidValue || e == cudaErrorLaunchOutOfResources;
  if (!recoverable && !g_sticky) g_sticky = (int)e;
  return OMT_ECUDA;
}
// ---- per-kernel device timing (reference debug_time_kernels / kernel_times, csrc/runtime.cpp:598-610) ----
bool g_kernel_timing = false;
struct TimedLaunch { std::string name; cudaEvent_t a, b; };
static std::vector<TimedLaunch> g_timed_launches;  // guarded by g_mu
static thread_local cudaStream_t t_stream = nullptr;
static thread_local cudaEvent_t t_prev = nullptr;    // the event the next launch on this thread starts from
void timing_begin(cudaStream_t s) {
  cudaEvent_t e;
  if (cudaEventCreate(&e) != cudaSuccess) return;
  cudaEventRecord(e, s);
  t_stream = s; t_prev = e;
}
static void timing_after_launch(const char* kernel) {
  if (!t_prev) return;
  cudaEvent_t e;
  if (cudaEventCreate(&e) != cudaSuccess) return;
  cudaEventRecord(e, t_stream);
  std::lock_guard<std::mutex> l(g_mu);
  g_timed_launches.push_back({kernel, t_prev, e});  // (events are shared between neighbours: destroyed once, at read-out)
  t_prev = e;
}
void note_launch(const char* kernel) {
  {
    std::lock_guard<std::mutex> l(g_mu);
    g_launches++;
    g_kcount[kernel]++;
  }
  if (g_kernel_timing) timing_after_launch(kernel);
}
int check_launch(const char* kernel) {
  note_launch(kernel);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, kernel);
  return OMT_OK;
}
int sm_count() {
  if (g_sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_sms <= 0) g_sms = 148;
  }
  return g_sms;
}

// ---------------------------------------------------------------------------------------------------------------
// caching allocator
// ---------------------------------------------------------------------------------------------------------------
//
// Size classes: multiples of 512 B below 1 MiB; above, the next of {1, 1.25, 1.5, 1.75} x 2^k (at most 25 % slack,
// few distinct classes, so a training loop that asks for the same shapes every step hits the cache after the first).
// Free blocks are kept per (class, stream): reuse on the same stream needs no synchronisation because the stream
// orders the old and the new user. A block that other streams touched (omt_record_stream) is parked with one event
// per such stream and only returns to its free list when they have completed.

struct Block {
  void* p;
  size_t bytes;
  cudaStream_t stream;
  std::vector<cudaStream_t> extra;
};
struct Parked {
  Block* b;
  std::vector<cudaEvent_t> ev;
};
static std::unordered_map<void*, Block*> g_live;
static std::map<std::pair<size_t, cudaStream_t>, std::vector<Block*>> g_free;
static std::vector<Parked> g_parked;
static size_t g_allocated = 0, g_reserved = 0;

static size_t size_class(size_t n) {
  if (n < 512) n = 512;
  if (n <= (1u << 20)) return (n + 511) / 512 * 512;
  size_t p = (size_t)1 << 20;
  while (p * 2 <= n) p *= 2;  // p <= n < 2p
  for (int q = 4; q <= 8; q++) {
    size_t c = p / 4 * q;
    if (c >= n) return c;
  }
  return p * 2;
}

static void reap_parked_locked() {
  for (size_t i = 0; i < g_parked.size();) {
    bool done = true;
    for (cudaEvent_t e : g_parked[i].ev)
      if (cudaEventQuery(e) != cudaSuccess) { done = false; break; }
    if (!done) { i++; continue; }
    for (cudaEvent_t e : g_parked[i].ev) cudaEventDestroy(e);
    Block* b = g_parked[i].b;
    b->extra.clear();
    g_free[{b->bytes, b->stream}].push_back(b);
    g_parked[i] = g_parked.back();
    g_parked.pop_back();
  }
  (void)cudaGetLastError();  // cudaErrorNotReady from the queries is not an error
}

static void release_cache_locked() {
  reap_parked_locked();
  for (auto& kv : g_free)
    for (Block* b : kv.second) {
      cudaFree(b->p);
      g_reserved -= b->bytes;
      delete b;
    }
  g_free.clear();
}

}  // namespace omt

using namespace omt;

extern "C" {

int omt_init(int device_ordinal) {
  std::lock_guard<std::mutex> l(g_mu);
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDeviceCount");
  if (device_ordinal < 0 || device_ordinal >= count) {
    set_error("omt_init: device %d of %d", device_ordinal, count);
    return OMT_EINVAL;
  }
  OMT_CUDA(cudaSetDevice(device_ordinal));
  OMT_CUDA(cudaFree(0));
  cudaDeviceProp prop;
  OMT_CUDA(cudaGetDeviceProperties(&prop, device_ordinal));
  if (prop.major != 10) {
    set_error("omt_init: device %d is sm_%d%d; this library only carries sm_100a code", device_ordinal, prop.major,
              prop.minor);
    return OMT_EINVAL;
  }
  g_device = device_ordinal;
  g_sms = prop.multiProcessorCount;
  return OMT_OK;
}
int omt_device(void) { return g_device; }

int omt_last_error(char* buf, size_t n) {
  size_t len = strlen(t_err);
  if (buf && n) {
    size_t c = len < n - 1 ? len : n - 1;
    memcpy(buf, t_err, c);
    buf[c] = 0;
  }
  return (int)len;
}
int omt_check_errors(void) {
  if (g_sticky) {
    set_error("asynchronous CUDA error %d (%s) reported earlier", g_sticky, cudaGetErrorString((cudaError_t)g_sticky));
    return OMT_ECUDA;
  }
  return OMT_OK;
}
int omt_sync(void) {
  OMT_CUDA(cudaDeviceSynchronize());
  int e = tc_error_word();
  if (e > 0) {
    set_error("a tensor-core convolution kernel gave up waiting on a barrier (code %d); its output is invalid", e);
    if (!g_sticky) g_sticky = (int)cudaErrorLaunchFailure;
    return OMT_ECUDA;
  }
  return OMT_OK;
}

void* omt_malloc(size_t bytes, omt_stream_t stream) {
  size_t cls = size_class(bytes);
  cudaStream_t s = st(stream);
  std::lock_guard<std::mutex> l(g_mu);
  if (!g_parked.empty()) reap_parked_locked();
  auto it = g_free.find({cls, s});
  Block* b = nullptr;
  if (it != g_free.end() && !it->second.empty()) {
    b = it->second.back();
    it->second.pop_back();
  } else {
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, cls);
    if (e == cudaErrorMemoryAllocation) {  // release the cache and retry once
      (void)cudaGetLastError();
      cudaDeviceSynchronize();
      release_cache_locked();
      e = cudaMalloc(&p, cls);
    }
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      set_error("out of device memory allocating %zu bytes (%zu allocated, %zu reserved)", cls, g_allocated, g_reserved);
      return nullptr;
    }
    b = new Block{p, cls, s, {}};
    g_reserved += cls;
  }
  g_allocated += b->bytes;
  g_live[b->p] = b;
  return b->p;
}

void omt_free(void* p) {
  if (!p) return;
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_live.find(p);
  if (it == g_live.end()) return;
  Block* b = it->second;
  g_live.erase(it);
  g_allocated -= b->bytes;
  if (b->extra.empty()) {
    g_free[{b->bytes, b->stream}].push_back(b);
    return;
  }
  Parked pk{b, {}};
  for (cudaStream_t s : b->extra) {
    cudaEvent_t e;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) == cudaSuccess) {
      cudaEventRecord(e, s);
      pk.ev.push_back(e);
    }
  }
  g_parked.push_back(pk);
}

int omt_record_stream(void* p, omt_stream_t stream) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_live.find(p);
  if (it == g_live.end()) return OMT_OK;  // not ours (or interior pointer): nothing to track
  Block* b = it->second;
  cudaStream_t s = st(stream);
  if (s == b->stream) return OMT_OK;
  for (cudaStream_t e : b->extra)
    if (e == s) return OMT_OK;
  b->extra.push_back(s);
  return OMT_OK;
}

void omt_empty_cache(void) {
  std::lock_guard<std::mutex> l(g_mu);
  cudaDeviceSynchronize();
  release_cache_locked();
}
size_t omt_memory_allocated(void) { return g_allocated; }
size_t omt_memory_reserved(void) { return g_reserved; }

omt_stream_t omt_stream_create(int high_priority) {
  cudaStream_t s = nullptr;
  int lo = 0, hi = 0;
  cudaDeviceGetStreamPriorityRange(&lo, &hi);
  cudaError_t e = cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, high_priority ? hi : lo);
  if (e != cudaSuccess) {
    cuda_fail(e, "cudaStreamCreateWithPriority");
    return nullptr;
  }
  return (omt_stream_t)s;
}
int omt_stream_destroy(omt_stream_t s) {
  OMT_CUDA(cudaStreamDestroy(st(s)));
  return OMT_OK;
}
int omt_stream_sync(omt_stream_t s) {
  OMT_CUDA(cudaStreamSynchronize(st(s)));
  return OMT_OK;
}
int omt_stream_query(omt_stream_t s) {
  cudaError_t e = cudaStreamQuery(st(s));
  if (e == cudaSuccess) return 1;
  if (e == cudaErrorNotReady) {
    (void)cudaGetLastError();
    return 0;
  }
  return cuda_fail(e, "cudaStreamQuery");
}
omt_event_t omt_event_create(int timing) {
  cudaEvent_t e = nullptr;
  cudaError_t r = cudaEventCreateWithFlags(&e, timing ? cudaEventDefault : cudaEventDisableTiming);
  if (r != cudaSuccess) {
    cuda_fail(r, "cudaEventCreateWithFlags");
    return nullptr;
  }
  return (omt_event_t)e;
}
int omt_event_destroy(omt_event_t e) {
  OMT_CUDA(cudaEventDestroy((cudaEvent_t)e));
  return OMT_OK;
}
int omt_event_record(omt_event_t e, omt_stream_t s) {
  OMT_CUDA(cudaEventRecord((cudaEvent_t)e, st(s)));
  return OMT_OK;
}
int omt_event_query(omt_event_t e) {
  cudaError_t r = cudaEventQuery((cudaEvent_t)e);
  if (r == cudaSuccess) return 1;
  if (r == cudaErrorNotReady) {
    (void)cudaGetLastError();
    return 0;
  }
  return cuda_fail(r, "cudaEventQuery");
}
int omt_event_sync(omt_event_t e) {
  OMT_CUDA(cudaEventSynchronize((cudaEvent_t)e));
  return OMT_OK;
}
int omt_stream_wait_event(omt_stream_t s, omt_event_t e) {
  OMT_CUDA(cudaStreamWaitEvent(st(s), (cudaEvent_t)e, 0));
  return OMT_OK;
}
int omt_event_elapsed_ms(omt_event_t a, omt_event_t b, float* ms) {
  OMT_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)a, (cudaEvent_t)b));
  return OMT_OK;
}

int omt_memcpy_h2d(void* dst, const void* src, size_t bytes, omt_stream_t s) {
  if (!bytes) return OMT_OK;
  OMT_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, st(s)));
  return OMT_OK;
}
int omt_memcpy_d2h(void* dst, const void* src, size_t bytes, omt_stream_t s) {
  if (!bytes) return OMT_OK;
  OMT_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, st(s)));
  OMT_CUDA(cudaStreamSynchronize(st(s)));
  return OMT_OK;
}
int omt_memcpy_d2d(void* dst, const void* src, size_t bytes, omt_stream_t s) {
  if (!bytes) return OMT_OK;
  OMT_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, st(s)));
  return OMT_OK;
}
int omt_memset(void* dst, int byte, size_t bytes, omt_stream_t s) {
  if (!bytes) return OMT_OK;
  OMT_CUDA(cudaMemsetAsync(dst, byte, bytes, st(s)));
  return OMT_OK;
}

int omt_kernel_timing(int enable) {
  g_kernel_timing = enable != 0;
  return OMT_OK;
}
size_t omt_kernel_times(char* buf, size_t n, int reset) {
  std::vector<TimedLaunch> launches;
  {
    std::lock_guard<std::mutex> l(g_mu);
    launches = g_timed_launches;
    if (reset) g_timed_launches.clear();
  }
  std::map<std::string, double> ms;
  std::vector<cudaEvent_t> events;
  for (auto& t : launches) {
    float v = 0.f;
    if (cudaEventSynchronize(t.b) == cudaSuccess && cudaEventElapsedTime(&v, t.a, t.b) == cudaSuccess) ms[t.name] += v;
    events.push_back(t.a); events.push_back(t.b);
  }
  (void)cudaGetLastError();
  if (reset) {
    std::sort(events.begin(), events.end());
    events.erase(std::unique(events.begin(), events.end()), events.end());
    for (cudaEvent_t e : events) cudaEventDestroy(e);
  }
  std::string s;
  char line[160];
  for (auto& kv : ms) {
    snprintf(line, sizeof(line), "%s=%.6f\n", kv.first.c_str(), kv.second);
    s += line;
  }
  if (buf && n) {
    size_t c = s.size() < n - 1 ? s.size() : n - 1;
    memcpy(buf, s.data(), c);
    buf[c] = 0;
  }
  return s.size() + 1;
}

uint64_t omt_launch_count(void) { return g_launches; }
size_t omt_kernel_counts(char* buf, size_t n, int reset) {
  std::lock_guard<std::mutex> l(g_mu);
  std::string s;
  for (auto& kv : g_kcount) s += kv.first + "=" + std::to_string(kv.second) + "\n";
  if (buf && n) {
    size_t c = s.size() < n - 1 ? s.size() : n - 1;
    memcpy(buf, s.data(), c);
    buf[c] = 0;
  }
  if (reset) g_kcount.clear();
  return s.size() + 1;
}

}  // extern "C"

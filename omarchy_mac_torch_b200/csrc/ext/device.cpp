// Allocator, device guard (with events), hooks and generator, memory/copy/view ops, and the bridge that serves ops
// outside the hot path with ATen's CUDA kernels on the same memory.
//
// Registration surface = the reference's csrc/device.cpp:238-256 (empty.memory_format, empty_strided, _copy_from,
// _copy_from_and_resize, _local_scalar_dense, set_ variants, view ops, the boxed fallback); what sits underneath is
// different: storages are CUDA memory from the caching allocator of libomt_b200.so, and the fallback does not leave
// the GPU.
#include "omt.h"

#include <atomic>
#include <unordered_map>
#include <c10/cuda/CUDAGuard.h>

#include <ATen/CPUGeneratorImpl.h>
#include <ATen/EmptyTensor.h>
#include <ATen/detail/CUDAHooksInterface.h>
#include <ATen/detail/PrivateUse1HooksInterface.h>
#include <ATen/native/Resize.h>
#include <c10/core/impl/DeviceGuardImplInterface.h>
#include <c10/cuda/CUDAFunctions.h>
#include <cuda_runtime.h>

#include <cstdlib>

namespace omt {

std::recursive_mutex& big_lock() {
  static std::recursive_mutex m;
  return m;
}
Stats& stats() {
  static Stats s;
  return s;
}

// ------------------------------------------------------------------------------------------------
// runtime glue
// ------------------------------------------------------------------------------------------------

static int g_index = -1;

static int pick_device() {
  for (const char* name : {"OMARCHY_MAC_TORCH_CUDA_DEVICE", "LOCAL_RANK"}) {
    const char* e = std::getenv(name);
    if (e && *e) {
      int v = std::atoi(e);
      if (v >= 0 && v < c10::cuda::device_count()) return v;
    }
  }
  return 0;
}

void ensure_init() {
  if (g_index >= 0) {
    if (c10::cuda::current_device() != g_index) c10::cuda::set_device((c10::DeviceIndex)g_index);
    return;
  }
  OMT_LOCK;
  if (g_index >= 0) return;
  TORCH_CHECK(c10::cuda::device_count() > 0,
              "omarchy-mac-torch: no CUDA device is visible; this backend has no CPU path and needs a B200");
  int idx = pick_device();
  c10::cuda::set_device((c10::DeviceIndex)idx);
  int r = omt_init(idx);
  if (r != OMT_OK) {
    char buf[512];
    omt_last_error(buf, sizeof(buf));
    TORCH_CHECK(false, "omarchy-mac-torch: cannot initialise CUDA device ", idx, ": ", buf);
  }
  g_index = idx;
}
int device_index() {
  ensure_init();
  return g_index;
}
// Autograd runs backward nodes on worker threads whose current CUDA stream is their own default stream: it only carries
// the forward's stream over for tensors of the process's accelerator type (CUDA), not for this PrivateUse1 device. A
// process-wide override lets a scope (CUDA-graph capture and its warm-up, omarchy_mac_torch_b200.graphs) put every
// thread's work of this device on one stream.
static std::atomic<cudaStream_t> g_stream_override{nullptr};
static std::atomic<bool> g_has_override{false};
void set_stream_override(uint64_t cuda_stream, bool on) {
  g_stream_override.store((cudaStream_t)cuda_stream);
  g_has_override.store(on);
}
bool stream_override(cudaStream_t* s) {
  if (!g_has_override.load(std::memory_order_relaxed)) return false;
  *s = g_stream_override.load();
  return true;
}
omt_stream_t cur_stream() {
  cudaStream_t s;
  if (stream_override(&s)) return (omt_stream_t)s;
  return (omt_stream_t)c10::cuda::getCurrentCUDAStream((c10::DeviceIndex)device_index()).stream();
}

void check(int status, const char* what) {
  if (status == OMT_OK) return;
  char buf[512];
  omt_last_error(buf, sizeof(buf));
  if (status == OMT_ENOMEM) TORCH_CHECK_WITH(OutOfMemoryError, false, "omarchy-mac-torch: ", what, ": ", buf);
  TORCH_CHECK(false, "omarchy-mac-torch: ", what, " failed (", status, "): ", buf);
}
void check_errors() {
  if (g_index < 0) return;
  if (omt_check_errors() != OMT_OK) {
    char buf[512];
    omt_last_error(buf, sizeof(buf));
    TORCH_CHECK(false, "omarchy-mac-torch: ", buf);
  }
}
void debug_end(const char* op) {  // OMARCHY_MAC_TORCH_DEBUG=1: surface asynchronous failures at the op that caused them
  cudaError_t e = cudaStreamSynchronize((cudaStream_t)cur_stream());
  if (e == cudaSuccess) e = cudaGetLastError();
  TORCH_CHECK(e == cudaSuccess, "omarchy-mac-torch: CUDA error after ", op, ": ", cudaGetErrorString(e));
}

// ------------------------------------------------------------------------------------------------
// allocator
// ------------------------------------------------------------------------------------------------

static std::mutex g_mask_mu;
static std::unordered_map<const void*, int64_t> g_relu_masks;  // allocation start -> elements whose ReLU mask sits behind them
void relu_mask_note(const void* p, int64_t numel) {
  std::lock_guard<std::mutex> l(g_mask_mu);
  g_relu_masks[p] = numel;
}
bool relu_mask_known(const void* p, int64_t numel) {
  std::lock_guard<std::mutex> l(g_mask_mu);
  auto it = g_relu_masks.find(p);
  return it != g_relu_masks.end() && it->second == numel;
}
static void free_block(void* p) {
  {
    std::lock_guard<std::mutex> l(g_mask_mu);
    if (!g_relu_masks.empty()) g_relu_masks.erase(p);
  }
  omt_free(p);
}

struct Allocator final : c10::Allocator {
  c10::DataPtr allocate(size_t n) override {
    ensure_init();
    void* p = omt_malloc(std::max<size_t>(n, 4), cur_stream());
    if (!p) {
      char buf[512];
      omt_last_error(buf, sizeof(buf));
      TORCH_CHECK_WITH(OutOfMemoryError, false, "omarchy-mac-torch: ", buf);
    }
    return {p, p, &free_block, c10::Device(kDev, 0)};
  }
  void copy_data(void* dst, const void* src, std::size_t count) const override {
    ensure_init();
    check(omt_memcpy_d2d(dst, src, count, cur_stream()), "storage copy");
  }
  c10::DeleterFnPtr raw_deleter() const override { return &free_block; }
};
static Allocator g_alloc;
REGISTER_ALLOCATOR(c10::DeviceType::PrivateUse1, &g_alloc);

Tensor empty_dev(IntArrayRef size, c10::ScalarType dt, bool channels_last) {
  c10::DispatchKeySet ks(c10::DispatchKey::PrivateUse1);
  return at::detail::empty_generic(size, &g_alloc, ks, dt,
                                   channels_last && size.size() == 4 ? std::optional<at::MemoryFormat>(at::MemoryFormat::ChannelsLast)
                                                                     : std::nullopt);
}

Tensor empty_dev_tail(IntArrayRef size, bool channels_last, int64_t tail_floats) {
  TORCH_INTERNAL_ASSERT(size.size() == 4);
  const int64_t n = size[0], c = size[1], h = size[2], w = size[3], numel = n * c * h * w;
  Tensor flat = empty_dev({numel + tail_floats}, at::kFloat);
  std::vector<int64_t> st = channels_last ? std::vector<int64_t>{h * w * c, 1, w * c, c} : std::vector<int64_t>{c * h * w, h * w, w, 1};
  return flat.as_strided(size, st, 0);
}

// ------------------------------------------------------------------------------------------------
// CUDA aliases of device tensors and back
// ------------------------------------------------------------------------------------------------

Tensor cuda_alias(const Tensor& t) {
  auto opts = t.options().device(at::Device(at::kCUDA, (c10::DeviceIndex)device_index()));
  if (t.numel() == 0) return at::empty_strided(t.sizes(), t.strides(), opts);
  Tensor keep = t;  // the alias keeps the device storage alive
  return at::from_blob(t.data_ptr(), t.sizes(), t.strides(), [keep](void*) {}, opts);
}

Tensor wrap_cuda(const Tensor& c) {
  auto* keep = new Tensor(c);
  c10::DataPtr dp(c.storage().mutable_data(), keep, [](void* p) { delete static_cast<Tensor*>(p); }, c10::Device(kDev, 0));
  c10::Storage st(c10::Storage::use_byte_size_t(), c.storage().nbytes(), std::move(dp), &g_alloc, /*resizable=*/true);
  Tensor out = at::detail::make_tensor<c10::TensorImpl>(std::move(st), c10::DispatchKeySet(c10::DispatchKey::PrivateUse1), c.dtype());
  out.unsafeGetTensorImpl()->set_sizes_and_strides(c.sizes(), c.strides(), c.storage_offset());
  return out;
}

int layout4(const Tensor& t) {
  if (t.dim() != 4) return -1;
  if (t.is_contiguous()) return 0;
  if (t.is_contiguous(at::MemoryFormat::ChannelsLast)) return 1;
  return -1;
}
Tensor contig(const Tensor& t) {
  if (t.is_contiguous()) return t;
  Tensor out = empty_dev(t.sizes(), t.scalar_type());
  cuda_alias(out).copy_(cuda_alias(t));
  return out;
}
// strides as the kernels expect them for a given layout (size-1 dimensions make PyTorch's strides ambiguous)
static Tensor canon(const Tensor& t, int layout) {
  int64_t c = t.size(1), h = t.size(2), w = t.size(3);
  std::vector<int64_t> st = layout == 0 ? std::vector<int64_t>{c * h * w, h * w, w, 1} : std::vector<int64_t>{h * w * c, 1, w * c, c};
  if (t.strides() == IntArrayRef(st)) return t;
  return t.as_strided(t.sizes(), st);
}
Tensor dense4(const Tensor& t) {
  int l = layout4(t);
  if (l >= 0) return canon(t, l);
  return canon(contig(t), 0);
}
Tensor to_layout(const Tensor& t_, int layout) {
  Tensor t = dense4(t_);
  int have = layout4(t);
  if (have == layout || (t.is_contiguous() && t.is_contiguous(at::MemoryFormat::ChannelsLast))) return canon(t, layout);
  Tensor out = canon(empty_dev(t.sizes(), at::kFloat, layout == 1), layout);
  OmtAct a = act(t), b = act(out);
  check(omt_act_copy(&a, &b, (int)t.size(0), (int)t.size(1), (int)t.size(2), (int)t.size(3), cur_stream()), "layout change");
  return out;
}

// ------------------------------------------------------------------------------------------------
// memory / copy ops
// ------------------------------------------------------------------------------------------------

static Tensor empty_memory_format_impl(IntArrayRef size, std::optional<at::ScalarType> dtype, std::optional<at::Layout>,
                                       std::optional<at::Device>, std::optional<bool>, std::optional<at::MemoryFormat> mf) {
  c10::DispatchKeySet ks(c10::DispatchKey::PrivateUse1);
  return at::detail::empty_generic(size, &g_alloc, ks, dtype.value_or(at::kFloat), mf);
}
static Tensor empty_strided_impl(IntArrayRef size, IntArrayRef stride, std::optional<at::ScalarType> dtype, std::optional<at::Layout>,
                                 std::optional<at::Device>, std::optional<bool>) {
  c10::DispatchKeySet ks(c10::DispatchKey::PrivateUse1);
  return at::detail::empty_strided_generic(size, stride, &g_alloc, ks, dtype.value_or(at::kFloat));
}

// copy self -> dst in any direction; ATen's CUDA copy does dtype conversion, strides and broadcasting
static Tensor copy_from_impl(const Tensor& self, const Tensor& dst, bool non_blocking) {
  ensure_init();
  Tensor a = is_dev(self) ? cuda_alias(self) : self;
  Tensor b = is_dev(dst) ? cuda_alias(dst) : dst;
  b.copy_(a, non_blocking);
  return dst;
}
static void grow_storage(const c10::Storage& storage, size_t newsize);  // below, with the hooks

// resize_ for device tensors. ATen's generic implementation grows the storage with a host memcpy, which cannot touch
// device memory, so the growth goes through the allocator and a device copy here.
static const Tensor& resize_impl(const Tensor& self, IntArrayRef size, std::optional<at::MemoryFormat> mf) {
  auto* impl = self.unsafeGetTensorImpl();
  int64_t numel = 1;
  for (int64_t d : size) numel *= d;
  size_t need = (size_t)(impl->storage_offset() + numel) * impl->dtype().itemsize();
  if (numel > 0 && need > impl->unsafe_storage().nbytes()) grow_storage(impl->unsafe_storage(), need);
  impl->set_sizes_contiguous(size);
  if (mf && *mf != at::MemoryFormat::Preserve && *mf != at::MemoryFormat::Contiguous) impl->empty_tensor_restride(*mf);
  return self;
}
static Tensor copy_from_and_resize_impl(const Tensor& self, const Tensor& dst) {
  resize_impl(dst, self.sizes(), std::nullopt);
  return copy_from_impl(self, dst, false);
}
static c10::Scalar local_scalar(const Tensor& self) {
  ensure_init();
  return cuda_alias(self).item();
}
static Tensor& set_storage(Tensor& self, c10::Storage src, int64_t off, IntArrayRef size, IntArrayRef stride) {
  return at::native::set_storage_cpu_(self, src, off, size, stride);  // metadata only
}

// ------------------------------------------------------------------------------------------------
// device guard with events. One logical stream per device: PyTorch's current CUDA stream.
// ------------------------------------------------------------------------------------------------

struct Guard final : c10::impl::DeviceGuardImplInterface {
  c10::DeviceType type() const override { return kDev; }
  c10::Device exchangeDevice(c10::Device) const override {
    if (g_index >= 0) ensure_init();
    return {kDev, 0};
  }
  c10::Device getDevice() const override { return {kDev, 0}; }
  void setDevice(c10::Device) const override {
    if (g_index >= 0) ensure_init();  // worker threads (autograd) start on CUDA device 0: move them to ours
  }
  void uncheckedSetDevice(c10::Device) const noexcept override {
    if (g_index >= 0) cudaSetDevice(g_index);
  }
  // Streams of this device are PyTorch's CUDA streams of the GPU underneath, under the same stream ids. Autograd records
  // the stream an op ran on and makes its worker thread run the backward node there (exchangeStream): without the
  // mapping the backward of work issued on a side stream, or inside a CUDA-graph capture, would land on the worker
  // thread's default stream.
  static c10::DeviceIndex cuda_index() { return (c10::DeviceIndex)(g_index >= 0 ? g_index : 0); }
  static c10::Stream as_mine(const c10::cuda::CUDAStream& cs) { return c10::Stream(c10::Stream::UNSAFE, c10::Device(kDev, 0), cs.id()); }
  static c10::cuda::CUDAStream as_cuda(const c10::Stream& s) {
    return c10::cuda::CUDAStream(c10::cuda::CUDAStream::UNCHECKED, c10::Stream(c10::Stream::UNSAFE, c10::Device(c10::kCUDA, cuda_index()), s.id()));
  }
  // (autograd's engine asks every registered backend for streams, also in processes that never touch a GPU)
  static bool has_gpu() {
    static const bool yes = c10::cuda::device_count() > 0;
    return yes;
  }
  c10::Stream getStream(c10::Device d) const noexcept override {
    if (!has_gpu()) return c10::Stream(c10::Stream::DEFAULT, d);
    return as_mine(c10::cuda::getCurrentCUDAStream(cuda_index()));
  }
  c10::Stream getDefaultStream(c10::Device d) const override {
    if (!has_gpu()) return c10::Stream(c10::Stream::DEFAULT, d);
    return as_mine(c10::cuda::getDefaultCUDAStream(cuda_index()));
  }
  c10::Stream getNewStream(c10::Device d, int priority) const override {
    if (!has_gpu()) return c10::Stream(c10::Stream::DEFAULT, d);
    return as_mine(c10::cuda::getStreamFromPool(priority, cuda_index()));
  }
  c10::Stream exchangeStream(c10::Stream s) const noexcept override {
    if (!has_gpu()) return s;
    c10::Stream old = as_mine(c10::cuda::getCurrentCUDAStream(cuda_index()));
    c10::cuda::setCurrentCUDAStream(as_cuda(s));
    return old;
  }
  c10::DeviceIndex deviceCount() const noexcept override { return 1; }
  // The CUDA stream behind a stream of this device: the one PyTorch names (autograd records events on the producer's stream
  // and makes the consumer's stream wait, from threads whose current stream is a third one), unless a process-wide
  // override is in force (a CUDA-graph capture keeps all of the device's work on its capture stream).
  static omt_stream_t handle(const c10::Stream& s) {
    cudaStream_t o;
    if (stream_override(&o)) return (omt_stream_t)o;
    if (!has_gpu()) return cur_stream();
    return (omt_stream_t)as_cuda(s).stream();
  }
  void record(void** event, const c10::Stream& s, const c10::DeviceIndex, const c10::EventFlag) const override {
    ensure_init();
    if (!*event) *event = omt_event_create(0);
    check(omt_event_record((omt_event_t)*event, handle(s)), "event record");
  }
  void block(void* event, const c10::Stream& s) const override {
    if (event) check(omt_stream_wait_event(handle(s), (omt_event_t)event), "stream wait event");
  }
  bool queryEvent(void* event) const override { return !event || omt_event_query((omt_event_t)event) == 1; }
  void destroyEvent(void* event, const c10::DeviceIndex) const noexcept override {
    if (event) omt_event_destroy((omt_event_t)event);
  }
  void synchronizeEvent(void* event) const override {
    if (event) check(omt_event_sync((omt_event_t)event), "event synchronize");
  }
  bool queryStream(const c10::Stream& s) const override { return omt_stream_query(handle(s)) == 1; }
  void synchronizeStream(const c10::Stream& s) const override { check(omt_stream_sync(handle(s)), "stream synchronize"); }
  void synchronizeDevice(const c10::DeviceIndex) const override {
    ensure_init();
    check(omt_sync(), "device synchronize");
  }
  void recordDataPtrOnStream(const c10::DataPtr& p, const c10::Stream& s) const override { omt_record_stream(p.get(), handle(s)); }
};
C10_REGISTER_GUARD_IMPL(PrivateUse1, Guard);

// Tensor.record_stream(stream): the allocator must not hand the block out again before that stream's pending work is done
static void record_stream_impl(Tensor& self, c10::Stream s) {
  if (!self.defined() || !self.has_storage() || !self.storage().data()) return;
  check(omt_record_stream(self.storage().mutable_data(), Guard::handle(s)), "record_stream");
}

// ------------------------------------------------------------------------------------------------
// hooks and generator (random fills are drawn on the host with this device's own generator, then uploaded)
// ------------------------------------------------------------------------------------------------

struct Generator : at::CPUGeneratorImpl {
  explicit Generator(c10::DeviceIndex i) {
    device_ = c10::Device(kDev, i);
    key_set_ = c10::DispatchKeySet(c10::DispatchKey::PrivateUse1);
  }
};
static const at::Generator& default_generator() {
  static at::Generator g = at::make_generator<Generator>(0);
  return g;
}

struct Hooks final : at::PrivateUse1HooksInterface {
  bool isBuilt() const override { return true; }
  bool isAvailable() const override { return true; }
  bool hasPrimaryContext(c10::DeviceIndex) const override { return true; }
  c10::DeviceIndex deviceCount() const override { return 1; }
  c10::DeviceIndex getCurrentDevice() const override { return 0; }
  void setCurrentDevice(c10::DeviceIndex) const override {}
  c10::DeviceIndex exchangeDevice(c10::DeviceIndex) const override { return 0; }
  c10::DeviceIndex maybeExchangeDevice(c10::DeviceIndex) const override { return 0; }
  const at::Generator& getDefaultGenerator(c10::DeviceIndex) const override { return default_generator(); }
  at::Generator getNewGenerator(c10::DeviceIndex i) const override { return at::make_generator<Generator>(i < 0 ? 0 : i); }
  at::Device getDeviceFromPtr(void*) const override { return {kDev, 0}; }
  // pinned host memory is CUDA's: tensor.pin_memory() keeps working with this device registered
  bool isPinnedPtr(const void* data) const override { return at::detail::getCUDAHooks().isPinnedPtr(data); }
  c10::Allocator* getPinnedMemoryAllocator() const override { return at::detail::getCUDAHooks().getPinnedMemoryAllocator(); }
  void resizePrivateUse1Bytes(const c10::Storage& storage, size_t newsize) const override { grow_storage(storage, newsize); }
};
static void grow_storage(const c10::Storage& storage, size_t newsize) {
  ensure_init();
  c10::DataPtr fresh = newsize ? g_alloc.allocate(newsize) : c10::DataPtr(nullptr, c10::Device(kDev, 0));
  size_t keep = std::min(newsize, storage.nbytes());
  if (keep && storage.data()) check(omt_memcpy_d2d(fresh.get(), storage.data(), keep, cur_stream()), "storage resize");
  storage.unsafeGetStorageImpl()->set_data_ptr_noswap(std::move(fresh));
  storage.unsafeGetStorageImpl()->set_nbytes(newsize);
}
static struct HooksRegistrar {
  HooksRegistrar() {
    static Hooks hooks;
    at::RegisterPrivateUse1HooksInterface(&hooks);
  }
} g_hooks_registrar;

at::CPUGeneratorImpl* generator(const std::optional<at::Generator>& gen) {
  const at::Generator& g = (gen && gen->defined()) ? *gen : default_generator();
  TORCH_CHECK(g.device().type() == kDev, "omarchy-mac-torch: expected a generator for this device, got one for ", g.device());
  return static_cast<at::CPUGeneratorImpl*>(g.unsafeGetGeneratorImpl());
}

// ------------------------------------------------------------------------------------------------
// the bridge: ops without a kernel in this library run ATen's CUDA kernel on aliases of the same memory
// ------------------------------------------------------------------------------------------------

std::map<std::string, int64_t>& fallback_counts() {
  static std::map<std::string, int64_t> m;
  return m;
}
void note_fallback(const std::string& op, const std::string& why) { fallback_counts()[op + " (" + why + ")"]++; }
bool strict_mode() {
  static bool s = [] {
    const char* e = std::getenv("OMARCHY_MAC_TORCH_STRICT");
    return e && e[0] == '1';
  }();
  return s;
}

namespace {
struct AliasMap {
  std::vector<Tensor> dev, cuda;
  Tensor to_cuda(const Tensor& t) {
    if (!is_dev(t)) return t;
    for (size_t i = 0; i < dev.size(); i++)
      if (dev[i].unsafeGetTensorImpl() == t.unsafeGetTensorImpl()) return cuda[i];
    dev.push_back(t);
    cuda.push_back(cuda_alias(t));
    return cuda.back();
  }
  // out= arguments that arrive empty are resized by the ATen kernel: give the device tensor the new storage and shape
  void adopt_resized() {
    for (size_t i = 0; i < dev.size(); i++) {
      if (dev[i].numel() != 0 || cuda[i].numel() == 0) continue;
      Tensor w = wrap_cuda(cuda[i]);
      auto* impl = dev[i].unsafeGetTensorImpl();
      impl->set_storage_keep_dtype(w.storage());
      impl->set_sizes_and_strides(cuda[i].sizes(), cuda[i].strides(), cuda[i].storage_offset());
    }
  }
  Tensor to_dev(const Tensor& c) {
    if (!c.defined() || !c.is_cuda()) return c;
    for (size_t i = 0; i < cuda.size(); i++)
      if (cuda[i].unsafeGetTensorImpl() == c.unsafeGetTensorImpl()) return dev[i];  // in-place / out= result
    for (size_t i = 0; i < cuda.size(); i++)
      if (c.is_alias_of(cuda[i])) {  // a view of an input: rebuild it over the input's device storage
        Tensor v = at::detail::make_tensor<c10::TensorImpl>(c10::Storage(dev[i].storage()), dev[i].key_set(), c.dtype());
        v.unsafeGetTensorImpl()->set_sizes_and_strides(c.sizes(), c.strides(),
                                                       dev[i].storage_offset() * (int64_t)dev[i].element_size() / (int64_t)c.element_size() +
                                                           c.storage_offset());
        return v;
      }
    return wrap_cuda(c);
  }
};
}  // namespace

static void bridge_impl(const c10::OperatorHandle& op, torch::jit::Stack* stack, bool count) {
  ensure_init();
  const auto& schema = op.schema();
  const std::string key = schema.name().substr(6) + (schema.overload_name().empty() ? "" : "." + schema.overload_name());
  if (!op.hasKernelForDispatchKey(c10::DispatchKey::CUDA)) {  // nothing on the GPU for it anywhere: host fallback, recorded
    TORCH_CHECK(!strict_mode(), "omarchy-mac-torch (strict): ", key, " has no GPU kernel");
    {
      OMT_LOCK;
      if (count) fallback_counts()[key]++;
    }
    at::native::cpu_fallback(op, stack);
    return;
  }
  OMT_LOCK;
  if (count) stats().bridge[key]++;
  const size_t nargs = schema.arguments().size(), begin = stack->size() - nargs;
  const c10::Device cuda_dev(at::kCUDA, (c10::DeviceIndex)device_index());
  AliasMap map;
  for (size_t i = 0; i < nargs; i++) {
    c10::IValue& v = (*stack)[begin + i];
    if (v.isTensor()) {
      v = map.to_cuda(v.toTensor());
    } else if (v.isTensorList()) {
      c10::List<Tensor> out;
      for (const Tensor& t : v.toTensorVector()) out.push_back(map.to_cuda(t));
      v = out;
    } else if (v.isOptionalTensorList()) {
      c10::List<std::optional<Tensor>> out;
      for (const std::optional<Tensor>& t : v.toOptionalTensorVector())
        out.push_back(t && t->defined() ? std::optional<Tensor>(map.to_cuda(*t)) : t);
      v = out;
    } else if (v.isDevice() && v.toDevice().type() == kDev) {
      v = cuda_dev;
    }
  }
  {
    // the ATen CUDA kernel launches on this thread's current CUDA stream: follow the override if one is set
    std::optional<c10::cuda::CUDAStreamGuard> follow;
    cudaStream_t forced;
    if (stream_override(&forced)) follow.emplace(c10::cuda::getStreamFromExternal(forced, (c10::DeviceIndex)device_index()));
    op.redispatchBoxed(c10::DispatchKeySet(c10::DispatchKey::CUDA), stack);
  }
  map.adopt_resized();
  const size_t nret = schema.returns().size(), rbegin = stack->size() - nret;
  for (size_t i = 0; i < nret; i++) {
    c10::IValue& v = (*stack)[rbegin + i];
    if (v.isTensor()) {
      v = map.to_dev(v.toTensor());
    } else if (v.isTensorList()) {
      c10::List<Tensor> out;
      for (const Tensor& t : v.toTensorVector()) out.push_back(map.to_dev(t));
      v = out;
    }
  }
}
void bridge_boxed(const c10::OperatorHandle& op, torch::jit::Stack* stack) { bridge_impl(op, stack, true); }
void bridge_quiet(const c10::OperatorHandle& op, torch::jit::Stack* stack) { bridge_impl(op, stack, false); }

TORCH_LIBRARY_IMPL(_, PrivateUse1, m) { m.fallback(torch::CppFunction::makeFromBoxedFunction<&bridge_boxed>()); }

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  OMT_IMPL(m, empty_memory_format, empty_memory_format_impl);
  OMT_IMPL(m, empty_strided, empty_strided_impl);
  OMT_IMPL(m, _copy_from, copy_from_impl);
  OMT_IMPL(m, _copy_from_and_resize, copy_from_and_resize_impl);
  OMT_IMPL(m, _local_scalar_dense, local_scalar);
  OMT_IMPL(m, set__source_Storage_storage_offset, set_storage);
  m.impl("view", &at::native::view);
  m.impl("_unsafe_view", &at::native::_unsafe_view);
  m.impl("as_strided", &at::native::as_strided_tensorimpl);
  m.impl("_reshape_alias", &at::native::_reshape_alias);
  m.impl("resize_", &resize_impl);
  m.impl("unfold", &at::native::unfold);  // views cannot go through the bridge's alias rebuild safely: explicit impls
  m.impl("view_as_real", &at::native::view_as_real);
  m.impl("view_as_complex", &at::native::view_as_complex);
  m.impl("set_.source_Storage", &at::native::set_);
  m.impl("record_stream", &record_stream_impl);
}

}  // namespace omt

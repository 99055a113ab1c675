// Python bindings (omarchy_mac_torch_b200._native). Keeps the names the reference's Python package uses
// (csrc/module.cpp:16-59); the ones that only made sense for generated WGSL kernels or the wgpu queue are inert.
#include "omt.h"

#include <ATen/CPUGeneratorImpl.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>

namespace omt {

void bind_conv(py::module_& m);
void bind_plans(py::module_& m);
void set_stream_override(uint64_t cuda_stream, bool on);
at::CPUGeneratorImpl* generator(const std::optional<at::Generator>& gen);

static std::map<std::string, int64_t> kernel_counts(bool reset) {
  size_t n = omt_kernel_counts(nullptr, 0, 0);
  std::string buf(n + 1, '\0');
  omt_kernel_counts(buf.data(), buf.size(), reset ? 1 : 0);
  std::map<std::string, int64_t> out;
  size_t pos = 0;
  while (pos < buf.size()) {
    size_t nl = buf.find('\n', pos);
    if (nl == std::string::npos) break;
    std::string line = buf.substr(pos, nl - pos);
    size_t eq = line.find('=');
    if (eq != std::string::npos) out[line.substr(0, eq)] = std::stoll(line.substr(eq + 1));
    pos = nl + 1;
  }
  return out;
}

PYBIND11_MODULE(_native, m) {
  m.def("init", []() { ensure_init(); });
  m.def("sync", []() { ensure_init(); check(omt_sync(), "synchronize"); check_errors(); });
  m.def("check_errors", []() { OMT_LOCK; check_errors(); });
  m.def("empty_cache", []() { omt_empty_cache(); });
  m.def("memory_allocated", []() { return (int64_t)omt_memory_allocated(); });
  m.def("memory_reserved", []() { return (int64_t)omt_memory_reserved(); });
  m.def("adapter_name", []() {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_index()) != cudaSuccess) return std::string("unknown CUDA device");
    return std::string(prop.name) + " (sm_" + std::to_string(prop.major) + std::to_string(prop.minor) + ")";
  });
  m.def("cuda_device_index", []() { return device_index(); });
  m.def("set_debug", [](bool on) { OMT_LOCK; stats().debug = on; });
  m.def("kernel_counts", [](bool reset) { return kernel_counts(reset); });
  m.def("launch_count", []() { return (int64_t)omt_launch_count(); });
  m.def("bridge_counts", [](bool reset) {
    OMT_LOCK;
    auto r = stats().bridge;
    if (reset) stats().bridge.clear();
    return r;
  });
  m.def("fallback_counts", []() { OMT_LOCK; return fallback_counts(); });
  m.def("reset_fallbacks", []() { OMT_LOCK; fallback_counts().clear(); });
  m.def("set_stream_override", &set_stream_override,
        "route the work of every thread (autograd workers included) to this cudaStream_t while `on`; graphs.capture uses it");
  m.def("as_cuda", [](const Tensor& t) { return cuda_alias(t); }, "a CUDA tensor aliasing a device tensor's memory (collectives, interop)");
  m.def("from_cuda", [](const Tensor& t) { return wrap_cuda(t); }, "a device tensor aliasing a CUDA tensor's memory");
  // RNG of the device = one CPU generator (values are drawn on the host and copied, csrc/nn.cpp of this extension)
  auto locked = [](auto&& fn) {
    auto* g = generator(std::nullopt);
    std::lock_guard<std::mutex> lock(g->mutex_);
    return fn(*g);
  };
  m.def("manual_seed", [locked](uint64_t s) { locked([&](at::CPUGeneratorImpl& g) { g.set_current_seed(s); return 0; }); });
  m.def("seed", [locked]() {
    const uint64_t s = c10::detail::getNonDeterministicRandom();
    locked([&](at::CPUGeneratorImpl& g) { g.set_current_seed(s); return 0; });
    return s;
  });
  m.def("initial_seed", []() { return generator(std::nullopt)->current_seed(); });
  m.def("get_rng_state", [locked]() { return locked([](at::CPUGeneratorImpl& g) { return Tensor(g.get_state()); }); });
  m.def("set_rng_state", [locked](const Tensor& state) {
    locked([&](at::CPUGeneratorImpl& g) { g.set_state(*state.unsafeGetTensorImpl()); return 0; });
  });
  // Names that only meant something for run-time generated WGSL and the wgpu submission queue: accepted, no effect.
  m.def("register_source", [](const std::string&, const std::string&) {});
  m.def("validate_kernels", []() { return std::vector<std::string>(); });
  m.def("kernel_times", [](bool reset) {  // {kernel: summed milliseconds} since debug_time_kernels(True)
    size_t n = omt_kernel_times(nullptr, 0, 0);
    std::string buf(n + 1, '\0');
    omt_kernel_times(buf.data(), buf.size(), reset ? 1 : 0);
    std::map<std::string, double> out;
    size_t pos = 0;
    while (pos < buf.size()) {
      size_t eol = buf.find('\n', pos);
      if (eol == std::string::npos) break;
      std::string line = buf.substr(pos, eol - pos);
      size_t eq = line.rfind('=');
      if (eq != std::string::npos) out[line.substr(0, eq)] = std::stod(line.substr(eq + 1));
      pos = eol + 1;
    }
    return out;
  }, py::arg("reset") = true);
  m.def("debug_time_kernels", [](bool on) { omt_kernel_timing(on ? 1 : 0); });
  m.def("set_mm_planner", [](py::object) {});  // the reference's generated-GEMM planner hook (csrc/linalg.cpp:94-96): nothing to plan here
  m.def("queue_state", []() { return std::make_tuple(0, 0, 0, 0.0); });
  m.def("set_queue", [](int, int) {});
  m.def("set_target_backlog_ms", [](double) {});
  m.def("debug_skip_submit", [](bool) {});
  m.def("flush", []() {});
  m.attr("built_with_torch") = TORCH_VERSION;
  bind_conv(m);
  bind_plans(m);
}

}  // namespace omt

// Shared declarations of the PyTorch device extension (_native): the "omarchy_mac_torch" PrivateUse1 backend whose
// hot ops call the C ABI of libomt_b200.so (include/omt_b200.h).
//
// Layout of the extension sources (same split as the reference's csrc/, minus its wgpu runtime):
//   device.cpp  allocator, device guard, hooks, generator, empty/copy/view ops, the ATen-CUDA bridge for long-tail ops
//   conv.cpp    aten::convolution / convolution_backward (dense + depthwise)
//   nn.cpp      batch norm, pooling, random fills
//   fused.cpp   omt:: custom ops (bn_relu_train, bn_relu_backward, conv_act, conv_bn_act_eval)
//   plans.cpp   fused conv/BN/ReLU/pool stacks (make_plan / Plan)
//   optim.cpp   _fused_sgd_ / _fused_adam_ / _fused_adamw_
//   module.cpp  Python bindings
//
// Memory model: a device tensor's storage is plain CUDA device memory from the library's caching allocator, holding
// exactly the bytes PyTorch would hold on any device, so storage-level operations (torch.save, deepcopy, views) behave
// as usual. Kernels run on PyTorch's current CUDA stream of the device, which also orders them with the ATen CUDA
// kernels the bridge calls for ops outside the hot path.
#pragma once

#include <ATen/ATen.h>
#include <ATen/Operators.h>
#include <ATen/native/CPUFallback.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>
#include <torch/library.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "omt_b200.h"

namespace omt {

using at::Tensor;
using c10::IntArrayRef;
constexpr auto kDev = c10::DeviceType::PrivateUse1;

// One lock around op entry points (autograd runs backward on another thread). Recursive because ops call ops.
std::recursive_mutex& big_lock();
#define OMT_LOCK std::lock_guard<std::recursive_mutex> omt_lock_(::omt::big_lock())

// ---- runtime glue -------------------------------------------------------------------------------------------------
void ensure_init();                 // omt_init on the process's device (LOCAL_RANK aware), once
int device_index();                 // CUDA ordinal behind omarchy_mac_torch:0
omt_stream_t cur_stream();          // PyTorch's current CUDA stream on that device
void check(int status, const char* what);  // non-zero C-ABI status -> c10::Error with omt_last_error()
void check_errors();                // sticky asynchronous error -> exception at the next op (reference check_errors)

struct Stats {
  bool debug = false;
  std::map<std::string, int64_t> bridge;  // long-tail ops served by ATen CUDA kernels through the bridge
};
Stats& stats();

// ---- tensors --------------------------------------------------------------------------------------------------------
inline bool is_dev(const Tensor& t) { return t.defined() && t.device().type() == kDev; }
inline bool f32(const Tensor& t) { return is_dev(t) && t.scalar_type() == at::kFloat; }
inline bool defined(const std::optional<Tensor>& t) { return t && t->defined(); }
Tensor empty_dev(IntArrayRef size, c10::ScalarType dt, bool channels_last = false);
// A dense float32 4-D tensor (NCHW or channels-last) whose allocation extends `tail_floats` floats beyond its elements.
Tensor empty_dev_tail(IntArrayRef size, bool channels_last, int64_t tail_floats);
// ReLU bit masks kept behind activations (OMT_BN_MASKBITS): the forward op notes that the allocation starting at `p` carries
// the mask of its `numel` elements; the backward op asks; the entry goes when the allocation is freed.
void relu_mask_note(const void* p, int64_t numel);
bool relu_mask_known(const void* p, int64_t numel);
inline float* fptr(const Tensor& t) { return t.defined() ? t.data_ptr<float>() : nullptr; }
inline float* fptr(const std::optional<Tensor>& t) { return defined(t) ? t->data_ptr<float>() : nullptr; }

// layout of a 4-D tensor: 0 NCHW-contiguous, 1 channels-last contiguous, -1 other
int layout4(const Tensor& t);
// returns t itself when it is NCHW- or channels-last-contiguous, else an NCHW-contiguous copy
Tensor dense4(const Tensor& t);
// t in the requested layout (copy through omt_act_copy when it differs)
Tensor to_layout(const Tensor& t, int layout);
inline OmtAct act(const Tensor& t) {
  return OmtAct{t.data_ptr<float>(), t.stride(0), t.stride(1), t.stride(2), t.stride(3)};
}
inline OmtAct null_act() { return OmtAct{nullptr, 0, 0, 0, 0}; }
Tensor contig(const Tensor& t);  // contiguous (any dtype), on the device

// A CUDA tensor aliasing the memory of a device tensor (same sizes/strides/dtype); used by the bridge and by copies.
Tensor cuda_alias(const Tensor& t);
// Wraps a CUDA tensor produced by an ATen kernel as a device tensor sharing its memory.
Tensor wrap_cuda(const Tensor& cuda);

// ---- "supported or fall back" -----------------------------------------------------------------------------------------
// An op implementation checks what it covers with NEED(cond, why) before launching anything. A failed NEED throws
// Unsupported; Safe<> then records "op (why)" in the fallback counts and serves the call through the bridge (ATen's
// CUDA kernel on the same memory) or, if ATen has no CUDA kernel either, PyTorch's CPU fallback.
// OMARCHY_MAC_TORCH_STRICT=1 turns that into an error.
struct Unsupported : std::exception {
  std::string why;
  explicit Unsupported(std::string w) : why(std::move(w)) {}
  const char* what() const noexcept override { return why.c_str(); }
};
#define NEED(cond, why)                            \
  do {                                             \
    if (!(cond)) throw ::omt::Unsupported(why);    \
  } while (0)

void bridge_boxed(const c10::OperatorHandle& op, torch::jit::Stack* stack);        // counts in stats().bridge
void bridge_quiet(const c10::OperatorHandle& op, torch::jit::Stack* stack);        // after Safe<> recorded the reason
void note_fallback(const std::string& op, const std::string& why);
std::map<std::string, int64_t>& fallback_counts();
bool strict_mode();
void debug_end(const char* op);

template <class Op, auto Fn, class Sig = typename Op::schema>
struct Safe;
template <class Op, auto Fn, class R, class... A>
struct Safe<Op, Fn, R(A...)> {
  static R call(typename c10::maybe_keep_symint<false, A>::type... a) {
    OMT_LOCK;
    check_errors();
    try {
      if (!stats().debug) return Fn(a...);
      if constexpr (std::is_void_v<R>) {
        Fn(a...);
        debug_end(Op::name);
      } else {
        R r = Fn(a...);
        debug_end(Op::name);
        return r;
      }
    } catch (const Unsupported& e) {
      std::string name = std::string(Op::name).substr(6);
      if (Op::overload_name[0]) name += std::string(".") + Op::overload_name;
      TORCH_CHECK(!strict_mode(), "omarchy-mac-torch (strict): ", name, " not supported by the device kernels: ", e.why);
      note_fallback(name, e.why);
      return at::native::call_fallback_fn<&bridge_quiet, Op>::call(a...);
    }
  }
};
#define OMT_IMPL(m, op, fn) ::omt::impl_name<at::_ops::op>(m, &::omt::Safe<at::_ops::op, fn>::call)
template <class Op, class F>
void impl_name(torch::Library& m, F f) {
  std::string name = std::string(Op::name).substr(6);
  if (Op::overload_name[0]) name += std::string(".") + Op::overload_name;
  m.impl(name.c_str(), f);
}

// omt:: ops: device implementation first; when it declines (Unsupported) the composite runs instead and the reason is recorded.
template <auto Dev, auto Ref, class... A>
auto dev_or_composite(const char* name, const A&... a) {
  OMT_LOCK;
  try {
    return Dev(a...);
  } catch (const Unsupported& e) {
    note_fallback(name, e.why);
    return Ref(a...);
  }
}

// ---- conv (conv.cpp), used by fused.cpp and plans.cpp ---------------------------------------------------------------
OmtConvGeo conv_geo(int64_t n, int64_t ci, int64_t co, int64_t ih, int64_t iw, int64_t ks, int64_t stride, int64_t pad,
                    int64_t groups = 1);
// y = conv(x, w) (+bias)(ReLU) into a fresh tensor; x must be dense4. Output is channels-last when prefer_cl() says so.
Tensor conv_forward(const Tensor& x, const Tensor& w, const Tensor* bias, const OmtConvGeo& g, bool relu);
bool prefer_cl(const Tensor& x, int64_t co);
// The same (no ReLU) with the batch-norm partial statistics of y taken in the GEMM epilogue when the call allows it: `groups`
// is the number of 32-row groups in `partials` (0 and an undefined tensor otherwise; see omt_conv_bnstats_groups).
Tensor conv_forward_stats(const Tensor& x, const Tensor& w, const Tensor* bias, const OmtConvGeo& g, Tensor& partials, int& groups);
extern int g_fold;  // eval-plan BN folding (set_fold): 0 off, anything else folds BatchNorm into the conv that feeds it

}  // namespace omt

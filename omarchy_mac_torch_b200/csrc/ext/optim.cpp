// Fused SGD and Adam / AdamW (torch.optim's fused=True path): the whole parameter list in one multi-tensor launch.
// Same registrations and support rules as the reference (csrc/optim.cpp:12-67); only the `double lr` overloads exist.
#include "omt.h"

namespace omt {

static void fused_sgd_(at::TensorList params, at::TensorList grads, at::TensorList momentum_bufs, double weight_decay, double momentum,
                       double lr, double dampening, bool nesterov, bool maximize, bool is_first_step,
                       const std::optional<Tensor>& grad_scale, const std::optional<Tensor>& found_inf) {
  NEED(!grad_scale && !found_inf, "fused SGD with grad scaling");
  for (size_t i = 0; i < params.size(); i++)
    NEED(f32(params[i]) && f32(grads[i]) && params[i].is_contiguous() && grads[i].is_contiguous(), "contiguous float32 params");
  std::vector<OmtParam> table(params.size());
  for (size_t i = 0; i < params.size(); i++) {
    bool has_m = momentum != 0 && momentum_bufs.size() > i && momentum_bufs[i].defined();
    NEED(!has_m || (f32(momentum_bufs[i]) && momentum_bufs[i].is_contiguous()), "contiguous float32 momentum buffers");
    table[i] = OmtParam{params[i].data_ptr<float>(), grads[i].data_ptr<float>(), has_m ? momentum_bufs[i].data_ptr<float>() : nullptr,
                        nullptr, nullptr, params[i].numel()};
  }
  check(omt_sgd(table.data(), (int)table.size(), (float)lr, (float)momentum, (float)dampening, (float)weight_decay, nesterov,
                is_first_step, maximize, cur_stream()),
        "fused SGD");
}

static void adam_impl(at::TensorList params, at::TensorList grads, at::TensorList exp_avgs, at::TensorList exp_avg_sqs,
                      at::TensorList state_steps, double lr, double beta1, double beta2, double weight_decay, double eps, bool amsgrad,
                      bool maximize, bool decoupled, const std::optional<Tensor>& grad_scale, const std::optional<Tensor>& found_inf) {
  NEED(!amsgrad && !grad_scale && !found_inf, "fused Adam with amsgrad or grad scaling");
  std::vector<OmtParam> table(params.size());
  for (size_t i = 0; i < params.size(); i++) {
    NEED(f32(params[i]) && f32(grads[i]) && f32(exp_avgs[i]) && f32(exp_avg_sqs[i]) && f32(state_steps[i]),
         "float32 params and device step tensors");
    NEED(params[i].is_contiguous() && grads[i].is_contiguous() && exp_avgs[i].is_contiguous() && exp_avg_sqs[i].is_contiguous(),
         "contiguous params");
    table[i] = OmtParam{params[i].data_ptr<float>(), grads[i].data_ptr<float>(), exp_avgs[i].data_ptr<float>(),
                        exp_avg_sqs[i].data_ptr<float>(), state_steps[i].data_ptr<float>(), params[i].numel()};
  }
  check(omt_adam(table.data(), (int)table.size(), (float)lr, (float)beta1, (float)beta2, (float)eps, (float)weight_decay, decoupled,
                 maximize, cur_stream()),
        "fused Adam");
}
static void fused_adam_(at::TensorList params, at::TensorList grads, at::TensorList exp_avgs, at::TensorList exp_avg_sqs, at::TensorList,
                        at::TensorList state_steps, double lr, double beta1, double beta2, double weight_decay, double eps, bool amsgrad,
                        bool maximize, const std::optional<Tensor>& grad_scale, const std::optional<Tensor>& found_inf) {
  adam_impl(params, grads, exp_avgs, exp_avg_sqs, state_steps, lr, beta1, beta2, weight_decay, eps, amsgrad, maximize, false, grad_scale,
            found_inf);
}
static void fused_adamw_(at::TensorList params, at::TensorList grads, at::TensorList exp_avgs, at::TensorList exp_avg_sqs, at::TensorList,
                         at::TensorList state_steps, double lr, double beta1, double beta2, double weight_decay, double eps, bool amsgrad,
                         bool maximize, const std::optional<Tensor>& grad_scale, const std::optional<Tensor>& found_inf) {
  adam_impl(params, grads, exp_avgs, exp_avg_sqs, state_steps, lr, beta1, beta2, weight_decay, eps, amsgrad, maximize, true, grad_scale,
            found_inf);
}

// torch.optim advances the device-resident step counters of a fused optimizer with _foreach_add_(steps, 1). Without a
// kernel for this device that op decomposes into one add per tensor (one launch per parameter); here the whole list goes
// through ATen's multi-tensor CUDA kernel on aliases of the same memory: one or two launches.
static void foreach_add_scalar_(at::TensorList self, const at::Scalar& scalar) {
  std::vector<Tensor> alias;
  alias.reserve(self.size());
  for (const Tensor& t : self) {
    NEED(is_dev(t), "device tensors");
    alias.push_back(cuda_alias(t));
  }
  at::_foreach_add_(alias, scalar);
}

// The functional form: the compile backend gathers the step counters of all BatchNorm layers of a graph (num_batches_tracked
// + 1, one tiny launch each otherwise) into one call.
static std::vector<Tensor> foreach_add_scalar(at::TensorList self, const at::Scalar& scalar) {
  std::vector<Tensor> alias;
  alias.reserve(self.size());
  for (const Tensor& t : self) {
    NEED(is_dev(t), "device tensors");
    alias.push_back(cuda_alias(t));
  }
  std::vector<Tensor> out;
  out.reserve(self.size());
  for (const Tensor& t : at::_foreach_add(alias, scalar)) out.push_back(wrap_cuda(t));
  return out;
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  OMT_IMPL(m, _foreach_add_Scalar, foreach_add_scalar);
  OMT_IMPL(m, _foreach_add__Scalar, foreach_add_scalar_);
  OMT_IMPL(m, _fused_sgd_, fused_sgd_);
  OMT_IMPL(m, _fused_adam_, fused_adam_);
  OMT_IMPL(m, _fused_adamw_, fused_adamw_);
}

}  // namespace omt

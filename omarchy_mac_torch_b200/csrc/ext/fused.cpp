// Fused ops that the torch.compile backend rewrites graphs to use (same op library, schemas and composite reference
// implementations as the reference's csrc/fused.cpp:213-233), plus the traced-graph BatchNorm variants.
//
//   omt::bn_relu_train      training BatchNorm2d + ReLU: statistics, then normalise + ReLU in one pass
//   omt::bn_relu_backward   its backward: ReLU mask folded into the BN backward reductions and apply
//   omt::bn_add_relu_train / omt::bn_add_relu_backward   the same pair across a residual add (BatchNorm, + identity, ReLU):
//                           the forward reads the identity branch in the apply pass, the backward also returns the masked
//                           gradient that flows into the identity branch
//   omt::conv_bn_train      conv2d feeding a training BatchNorm2d (+ identity branch)(+ ReLU): the conv epilogue reduces the
//                           batch statistics while it stores its output, so the BatchNorm reads that output once, not twice
//   omt::conv_act           conv2d + bias + optional ReLU in the GEMM epilogue
//   omt::conv_bn_act_eval   eval conv2d + BatchNorm (folded into the conv's weights and bias) + optional ReLU
//   omt::fused_pointwise    declared for schema parity; generated pointwise kernels are not built in this library
#include "omt.h"

namespace omt {

// ---- composite (reference) implementations: csrc/fused.cpp:19-49 -------------------------------------------------------

static std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> bn_relu_train_ref(const Tensor& x, const Tensor& w, const Tensor& b, const Tensor& rm,
                                                                          const Tensor& rv, double mom, double eps) {
  auto r = at::_native_batch_norm_legit_functional(x, w, b, rm, rv, true, mom, eps);
  return {at::relu(std::get<0>(r)), std::get<1>(r), std::get<2>(r), std::get<3>(r), std::get<4>(r)};
}
static std::tuple<Tensor, Tensor, Tensor> bn_relu_backward_ref(const Tensor& g, const Tensor& x, const Tensor& y, const Tensor& w,
                                                               const Tensor& mean, const Tensor& invstd, std::array<bool, 3> mask) {
  Tensor gz = at::threshold_backward(g, y, 0);
  return at::native_batch_norm_backward(gz, x, w, std::nullopt, std::nullopt, mean, invstd, true, 0.0, mask);
}
static std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> bn_add_relu_train_ref(const Tensor& x, const Tensor& res, const Tensor& w, const Tensor& b,
                                                                              const Tensor& rm, const Tensor& rv, double mom, double eps) {
  auto r = at::_native_batch_norm_legit_functional(x, w, b, rm, rv, true, mom, eps);
  return {at::relu(std::get<0>(r) + res), std::get<1>(r), std::get<2>(r), std::get<3>(r), std::get<4>(r)};
}
static std::tuple<Tensor, Tensor, Tensor, Tensor> bn_add_relu_backward_ref(const Tensor& g, const Tensor& x, const Tensor& y, const Tensor& w,
                                                                           const Tensor& mean, const Tensor& invstd, std::array<bool, 3> mask) {
  Tensor gz = at::threshold_backward(g, y, 0);
  auto r = at::native_batch_norm_backward(gz, x, w, std::nullopt, std::nullopt, mean, invstd, true, 0.0, mask);
  return {std::get<0>(r), std::get<1>(r), std::get<2>(r), gz};
}
// (yconv, z, mean, invstd, new_rm, new_rv): yconv is the conv output the backward graph keeps, z the block's output
static std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, Tensor> conv_bn_train_ref(const Tensor& x, const Tensor& cw, const std::optional<Tensor>& cb,
                                                                                   IntArrayRef stride, IntArrayRef padding,
                                                                                   const std::optional<Tensor>& res, const Tensor& w, const Tensor& b,
                                                                                   const Tensor& rm, const Tensor& rv, double mom, double eps,
                                                                                   int64_t act_) {
  Tensor y = at::convolution(x, cw, cb, stride, padding, {1, 1}, false, {0, 0}, 1);
  auto r = at::_native_batch_norm_legit_functional(y, w, b, rm, rv, true, mom, eps);
  Tensor z = std::get<0>(r);
  if (defined(res)) z = z + *res;
  if (act_ == 1) z = at::relu(z);
  return {y, z, std::get<1>(r), std::get<2>(r), std::get<3>(r), std::get<4>(r)};
}
static Tensor conv_act_ref(const Tensor& x, const Tensor& w, const std::optional<Tensor>& b, IntArrayRef stride, IntArrayRef padding, int64_t act_) {
  Tensor y = at::convolution(x, w, b, stride, padding, {1, 1}, false, {0, 0}, 1);
  return act_ == 1 ? at::relu(y) : y;
}
static std::pair<Tensor, Tensor> fold_bn(const Tensor& cw, const std::optional<Tensor>& cb, const Tensor& w, const Tensor& b, const Tensor& rm,
                                         const Tensor& rv, double eps) {
  Tensor scale = w * at::rsqrt(rv + eps);  // per output channel
  Tensor fw = cw * scale.view({-1, 1, 1, 1});
  Tensor fb = (defined(cb) ? (*cb - rm) : -rm) * scale + b;
  return {fw, fb};
}
static Tensor conv_bn_act_eval_ref(const Tensor& x, const Tensor& cw, const std::optional<Tensor>& cb, const Tensor& w, const Tensor& b,
                                   const Tensor& rm, const Tensor& rv, double eps, IntArrayRef stride, IntArrayRef padding, int64_t act_) {
  auto f = fold_bn(cw, cb, w, b, rm, rv, eps);
  return conv_act_ref(x, f.first, f.second, stride, padding, act_);
}
static Tensor fused_pointwise_ref(c10::string_view, at::TensorList) {
  TORCH_CHECK(false, "omt::fused_pointwise: generated pointwise kernels are not built in this library");
}

// ---- device implementations ------------------------------------------------------------------------------------------------

static bool whole(const Tensor& t) { return f32(t) && t.is_contiguous(); }

// Statistics then normalise(+ identity)(+ReLU). When `partials` comes from the conv that produced x_ (groups > 0) the
// statistics are merged from them instead of being reduced from x_. mean and invstd are separate tensors: the reference
// returns them as two halves of one buffer (csrc/fused.cpp:65-67), which an op schema without alias annotations may not do.
static std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> bn_res_relu_train(const Tensor& x_, const Tensor* res_, const Tensor& w, const Tensor& b,
                                                                          const Tensor& rm, const Tensor& rv, double mom, double eps,
                                                                          bool relu = true, const Tensor* partials = nullptr, int groups = 0) {
  NEED(f32(x_) && x_.dim() == 4 && x_.numel() > 0 && whole(w) && whole(b) && whole(rm) && whole(rv), "4-D float32 with contiguous parameters");
  NEED(!res_ || (f32(*res_) && res_->sizes() == x_.sizes()), "residual of the activation's shape");
  Tensor x = dense4(x_);
  if (layout4(x) == 1 && x.size(1) % 4 != 0) x = to_layout(x, 0);
  Tensor res = res_ ? to_layout(*res_, layout4(x)) : Tensor();
  const int n = (int)x.size(0), c = (int)x.size(1), h = (int)x.size(2), wd = (int)x.size(3);
  Tensor nrm = empty_dev({c}, at::kFloat), nrv = empty_dev({c}, at::kFloat);
  Tensor mean = empty_dev({c}, at::kFloat), inv = empty_dev({c}, at::kFloat);
  // With a ReLU the output's allocation extends by one bit per element: the apply pass leaves the ReLU mask there, and the
  // backward op (which receives this same tensor as its `y`) reads those bits instead of y's values.
  const int64_t numel = x.numel();
  Tensor y = relu ? empty_dev_tail(x.sizes(), layout4(x) == 1, (numel + 31) / 32) : dense4(empty_dev(x.sizes(), at::kFloat, layout4(x) == 1));
  OmtAct ax = act(x), ay = act(y);
  if (partials && groups > 0 && x.is_same(x_)) {
    check(omt_bn_stats_from_partials(partials->data_ptr<float>(), groups, c, fptr(mean), nullptr, fptr(inv), fptr(rm), fptr(rv), fptr(nrm), fptr(nrv),
                                     (float)mom, (float)eps, OMT_BN_FUNCTIONAL, cur_stream()),
          "batch statistics from the conv epilogue");
  } else {
    check(omt_bn_stats(&ax, n, c, h, wd, fptr(mean), nullptr, fptr(inv), fptr(rm), fptr(rv), fptr(nrm), fptr(nrv), (float)mom, (float)eps,
                       OMT_BN_FUNCTIONAL, cur_stream()),
          "bn_relu_train statistics");
  }
  OmtAct ar = res_ ? act(res) : null_act();
  check(omt_bn_apply_add(&ax, &ar, &ay, n, c, h, wd, fptr(mean), fptr(inv), fptr(w), fptr(b), relu ? (OMT_BN_RELU | OMT_BN_MASKBITS) : 0u,
                         cur_stream()),
        "bn_relu_train apply");
  if (relu) relu_mask_note(y.data_ptr(), numel);
  return {y, mean, inv, nrm, nrv};
}
static std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> bn_relu_train_dev(const Tensor& x, const Tensor& w, const Tensor& b, const Tensor& rm,
                                                                          const Tensor& rv, double mom, double eps) {
  return bn_res_relu_train(x, nullptr, w, b, rm, rv, mom, eps);
}
static std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> bn_add_relu_train_dev(const Tensor& x, const Tensor& res, const Tensor& w, const Tensor& b,
                                                                              const Tensor& rm, const Tensor& rv, double mom, double eps) {
  return bn_res_relu_train(x, &res, w, b, rm, rv, mom, eps);
}

static std::tuple<Tensor, Tensor, Tensor, Tensor> bn_res_relu_backward(const Tensor& g_, const Tensor& x_, const Tensor& y_, const Tensor& w,
                                                                       const Tensor& mean_, const Tensor& invstd_, std::array<bool, 3> mask,
                                                                       bool want_dres) {
  NEED(f32(g_) && f32(x_) && f32(y_) && x_.dim() == 4 && x_.numel() > 0 && whole(w) && f32(mean_) && f32(invstd_), "4-D float32");
  Tensor x = dense4(x_);
  if (layout4(x) == 1 && x.size(1) % 4 != 0) x = to_layout(x, 0);
  const int lay = layout4(x);
  Tensor g = to_layout(g_, lay), y = to_layout(y_, lay), mean = contig(mean_), inv = contig(invstd_);
  // y as the forward op made it (same allocation, same layout, not a copy) carries its ReLU mask as bits behind its values
  const bool bits = y.data_ptr() == y_.data_ptr() && y.storage_offset() == 0 && relu_mask_known(y.data_ptr(), y.numel());
  const int n = (int)x.size(0), c = (int)x.size(1), h = (int)x.size(2), wd = (int)x.size(3);
  Tensor dgb = empty_dev({2, c}, at::kFloat), gx, gres;
  OmtAct ag = act(g), ax = act(x), ay = act(y), adx = null_act(), adr = null_act();
  if (mask[0] || want_dres) {  // the masked gradient is a by-product of the dx pass
    gx = dense4(empty_dev(x.sizes(), at::kFloat, lay == 1));
    adx = act(gx);
  }
  if (want_dres) {
    gres = dense4(empty_dev(x.sizes(), at::kFloat, lay == 1));
    adr = act(gres);
  }
  check(omt_bn_backward_add(&ag, &ax, &ay, &adx, &adr, n, c, h, wd, fptr(mean), fptr(inv), fptr(w), dgb.data_ptr<float>(), 1.f,
                            OMT_BN_RELU | (bits ? OMT_BN_MASKBITS : 0u), cur_stream()),
        "bn_relu_backward");
  return {mask[0] ? gx : Tensor(), mask[1] ? dgb.select(0, 0) : Tensor(), mask[2] ? dgb.select(0, 1) : Tensor(), gres};
}
static std::tuple<Tensor, Tensor, Tensor> bn_relu_backward_dev(const Tensor& g, const Tensor& x, const Tensor& y, const Tensor& w, const Tensor& mean,
                                                               const Tensor& invstd, std::array<bool, 3> mask) {
  auto r = bn_res_relu_backward(g, x, y, w, mean, invstd, mask, false);
  return {std::get<0>(r), std::get<1>(r), std::get<2>(r)};
}
static std::tuple<Tensor, Tensor, Tensor, Tensor> bn_add_relu_backward_dev(const Tensor& g, const Tensor& x, const Tensor& y, const Tensor& w,
                                                                           const Tensor& mean, const Tensor& invstd, std::array<bool, 3> mask) {
  return bn_res_relu_backward(g, x, y, w, mean, invstd, mask, true);
}

static Tensor conv_act_dev(const Tensor& x_, const Tensor& w_, const std::optional<Tensor>& b, IntArrayRef stride, IntArrayRef padding, int64_t act_) {
  NEED(f32(x_) && f32(w_) && x_.dim() == 4 && w_.dim() == 4 && x_.numel() > 0 && w_.size(2) == w_.size(3) && stride[0] == stride[1] &&
           padding[0] == padding[1] && stride[0] >= 1 && stride[0] <= 4 && w_.size(2) <= 11 && padding[0] <= w_.size(2) &&
           x_.size(1) == w_.size(1) && (!defined(b) || f32(*b)),
       "dense square conv");
  Tensor x = dense4(x_), w = contig(w_);
  OmtConvGeo g = conv_geo(x.size(0), x.size(1), w.size(0), x.size(2), x.size(3), w.size(2), stride[0], padding[0]);
  NEED(g.oh > 0 && g.ow > 0, "empty output");
  Tensor bb = defined(b) ? contig(*b) : Tensor();
  return conv_forward(x, w, bb.defined() ? &bb : nullptr, g, act_ == 1);
}

static std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, Tensor> conv_bn_train_dev(const Tensor& x_, const Tensor& cw_, const std::optional<Tensor>& cb,
                                                                                   IntArrayRef stride, IntArrayRef padding,
                                                                                   const std::optional<Tensor>& res, const Tensor& w, const Tensor& b,
                                                                                   const Tensor& rm, const Tensor& rv, double mom, double eps,
                                                                                   int64_t act_) {
  NEED(f32(x_) && f32(cw_) && x_.dim() == 4 && cw_.dim() == 4 && x_.numel() > 0 && cw_.size(2) == cw_.size(3) && stride[0] == stride[1] &&
           padding[0] == padding[1] && stride[0] >= 1 && stride[0] <= 4 && cw_.size(2) <= 11 && padding[0] <= cw_.size(2) &&
           x_.size(1) == cw_.size(1) && (!defined(cb) || f32(*cb)),
       "dense square conv");
  NEED(whole(w) && whole(b) && whole(rm) && whole(rv) && w.numel() == cw_.size(0), "contiguous float32 BatchNorm parameters");
  NEED(!defined(res) || f32(*res), "float32 residual");
  Tensor x = dense4(x_), cw = contig(cw_);
  OmtConvGeo g = conv_geo(x.size(0), x.size(1), cw.size(0), x.size(2), x.size(3), cw.size(2), stride[0], padding[0]);
  NEED(g.oh > 0 && g.ow > 0, "empty output");
  Tensor bb = defined(cb) ? contig(*cb) : Tensor(), partials;
  int groups = 0;
  Tensor y = conv_forward_stats(x, cw, bb.defined() ? &bb : nullptr, g, partials, groups);
  auto r = bn_res_relu_train(y, defined(res) ? &*res : nullptr, w, b, rm, rv, mom, eps, act_ == 1, &partials, groups);
  return {y, std::get<0>(r), std::get<1>(r), std::get<2>(r), std::get<3>(r), std::get<4>(r)};
}

static Tensor conv_bn_act_eval_dev(const Tensor& x, const Tensor& cw, const std::optional<Tensor>& cb, const Tensor& w, const Tensor& b,
                                   const Tensor& rm, const Tensor& rv, double eps, IntArrayRef stride, IntArrayRef padding, int64_t act_) {
  NEED(f32(cw) && f32(w) && f32(b) && f32(rm) && f32(rv), "float32");
  auto f = fold_bn(cw, cb, w, b, rm, rv, eps);  // a few tiny elementwise ops on the weights, then one GEMM with the epilogue
  return conv_act_dev(x, f.first, f.second, stride, padding, act_);
}

static Tensor fused_pointwise_dev(c10::string_view kernel, at::TensorList ins) { return fused_pointwise_ref(kernel, ins); }

// eager entry points for the non-functional BatchNorm variants that traced / compiled graphs call (csrc/fused.cpp:173-181)
static std::tuple<Tensor, Tensor, Tensor> bn_legit(const Tensor& x, const std::optional<Tensor>& w, const std::optional<Tensor>& b, Tensor& rm,
                                                   Tensor& rv, bool training, double mom, double eps) {
  return at::native_batch_norm(x, w, b, rm, rv, training, mom, eps);
}
static std::tuple<Tensor, Tensor, Tensor> bn_legit_no_training(const Tensor& x, const std::optional<Tensor>& w, const std::optional<Tensor>& b,
                                                               const Tensor& rm, const Tensor& rv, double mom, double eps) {
  return at::native_batch_norm(x, w, b, rm, rv, false, mom, eps);
}

// Device implementation first; when it declines (Unsupported) the composite runs instead and the reason is recorded.
template <auto Dev, auto Ref, class... A>
static auto dev_or_composite(const char* name, const A&... a) {
  OMT_LOCK;
  try {
    return Dev(a...);
  } catch (const Unsupported& e) {
    note_fallback(name, e.why);
    return Ref(a...);
  }
}

TORCH_LIBRARY(omt, m) {
  m.def("bn_relu_train(Tensor x, Tensor w, Tensor b, Tensor rm, Tensor rv, float momentum, float eps) -> (Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("bn_relu_backward(Tensor g, Tensor x, Tensor y, Tensor w, Tensor mean, Tensor invstd, bool[3] mask) -> (Tensor, Tensor, Tensor)");
  m.def("bn_add_relu_train(Tensor x, Tensor res, Tensor w, Tensor b, Tensor rm, Tensor rv, float momentum, float eps) -> (Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("bn_add_relu_backward(Tensor g, Tensor x, Tensor y, Tensor w, Tensor mean, Tensor invstd, bool[3] mask) -> (Tensor, Tensor, Tensor, Tensor)");
  m.def("conv_bn_train(Tensor x, Tensor cw, Tensor? cb, int[] stride, int[] padding, Tensor? res, Tensor w, Tensor b, Tensor rm, Tensor rv, "
        "float momentum, float eps, int act) -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("conv_act(Tensor x, Tensor w, Tensor? b, int[] stride, int[] padding, int act) -> Tensor");
  m.def("conv_bn_act_eval(Tensor x, Tensor cw, Tensor? cb, Tensor w, Tensor b, Tensor rm, Tensor rv, float eps, int[] stride, int[] padding, int act) -> Tensor");
  m.def("fused_pointwise(str kernel, Tensor[] inputs) -> Tensor");
}
TORCH_LIBRARY_IMPL(omt, CompositeExplicitAutograd, m) {
  m.impl("bn_relu_train", &bn_relu_train_ref);
  m.impl("bn_relu_backward", &bn_relu_backward_ref);
  m.impl("bn_add_relu_train", &bn_add_relu_train_ref);
  m.impl("bn_add_relu_backward", &bn_add_relu_backward_ref);
  m.impl("conv_bn_train", &conv_bn_train_ref);
  m.impl("conv_act", &conv_act_ref);
  m.impl("conv_bn_act_eval", &conv_bn_act_eval_ref);
  m.impl("fused_pointwise", &fused_pointwise_ref);
}
TORCH_LIBRARY_IMPL(omt, PrivateUse1, m) {
  m.impl("bn_relu_train", [](const Tensor& x, const Tensor& w, const Tensor& b, const Tensor& rm, const Tensor& rv, double mom, double eps) {
    return dev_or_composite<&bn_relu_train_dev, &bn_relu_train_ref>("bn_relu_train", x, w, b, rm, rv, mom, eps);
  });
  m.impl("bn_relu_backward", [](const Tensor& g, const Tensor& x, const Tensor& y, const Tensor& w, const Tensor& mean, const Tensor& invstd,
                                std::array<bool, 3> mask) {
    return dev_or_composite<&bn_relu_backward_dev, &bn_relu_backward_ref>("bn_relu_backward", g, x, y, w, mean, invstd, mask);
  });
  m.impl("bn_add_relu_train", [](const Tensor& x, const Tensor& res, const Tensor& w, const Tensor& b, const Tensor& rm, const Tensor& rv, double mom,
                                 double eps) {
    return dev_or_composite<&bn_add_relu_train_dev, &bn_add_relu_train_ref>("bn_add_relu_train", x, res, w, b, rm, rv, mom, eps);
  });
  m.impl("bn_add_relu_backward", [](const Tensor& g, const Tensor& x, const Tensor& y, const Tensor& w, const Tensor& mean, const Tensor& invstd,
                                    std::array<bool, 3> mask) {
    return dev_or_composite<&bn_add_relu_backward_dev, &bn_add_relu_backward_ref>("bn_add_relu_backward", g, x, y, w, mean, invstd, mask);
  });
  m.impl("conv_bn_train", [](const Tensor& x, const Tensor& cw, const std::optional<Tensor>& cb, IntArrayRef s, IntArrayRef p,
                             const std::optional<Tensor>& res, const Tensor& w, const Tensor& b, const Tensor& rm, const Tensor& rv, double mom, double eps,
                             int64_t a) {
    return dev_or_composite<&conv_bn_train_dev, &conv_bn_train_ref>("conv_bn_train", x, cw, cb, s, p, res, w, b, rm, rv, mom, eps, a);
  });
  m.impl("conv_act", [](const Tensor& x, const Tensor& w, const std::optional<Tensor>& b, IntArrayRef s, IntArrayRef p, int64_t a) {
    return dev_or_composite<&conv_act_dev, &conv_act_ref>("conv_act", x, w, b, s, p, a);
  });
  m.impl("conv_bn_act_eval", [](const Tensor& x, const Tensor& cw, const std::optional<Tensor>& cb, const Tensor& w, const Tensor& b,
                                const Tensor& rm, const Tensor& rv, double eps, IntArrayRef s, IntArrayRef p, int64_t a) {
    return dev_or_composite<&conv_bn_act_eval_dev, &conv_bn_act_eval_ref>("conv_bn_act_eval", x, cw, cb, w, b, rm, rv, eps, s, p, a);
  });
  m.impl("fused_pointwise", &fused_pointwise_dev);
}
TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  OMT_IMPL(m, _native_batch_norm_legit, bn_legit);
  OMT_IMPL(m, _native_batch_norm_legit_no_training, bn_legit_no_training);
}

}  // namespace omt

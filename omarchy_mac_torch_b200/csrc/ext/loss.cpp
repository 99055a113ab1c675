// Classification loss on the device: aten::_log_softmax / _log_softmax_backward_data over the last dimension of a 2-D
// float32 matrix, aten::nll_loss_forward / nll_loss_backward on (N, C) with int64 targets -- the four ops F.cross_entropy
// decomposes into, covered like the reference's csrc/reduce.cpp:141-201 -- and the fused pair the compile backend
// rewrites them to: omt::softmax_nll (logits -> loss, log-probabilities, total weight in one launch) and
// omt::softmax_nll_backward (gradient of the logits in one launch).
#include "omt.h"

namespace omt {

static bool last_dim_2d(const Tensor& x, int64_t dim) { return x.dim() == 2 && (dim == 1 || dim == -1); }
static const float* wptr(const std::optional<Tensor>& w, Tensor& keep) {
  if (!defined(w)) return nullptr;
  keep = contig(*w);
  return keep.data_ptr<float>();
}

static Tensor log_softmax_(const Tensor& x_, int64_t dim, bool half_to_float) {
  NEED(f32(x_) && !half_to_float && last_dim_2d(x_, dim) && x_.numel() > 0 && x_.size(1) < (1ll << 31), "log_softmax over the last dimension of a float32 matrix");
  Tensor x = contig(x_), out = empty_dev(x.sizes(), at::kFloat);
  check(omt_log_softmax(x.data_ptr<float>(), out.data_ptr<float>(), x.size(0), (int32_t)x.size(1), cur_stream()), "log_softmax");
  return out;
}

static Tensor log_softmax_bwd_(const Tensor& g_, const Tensor& y_, int64_t dim, at::ScalarType dt) {
  NEED(f32(g_) && f32(y_) && dt == at::kFloat && last_dim_2d(y_, dim) && y_.numel() > 0 && g_.sizes() == y_.sizes() && y_.size(1) < (1ll << 31),
       "log_softmax backward over the last dimension of a float32 matrix");
  Tensor g = contig(g_), y = contig(y_), out = empty_dev(y.sizes(), at::kFloat);
  check(omt_log_softmax_backward(g.data_ptr<float>(), y.data_ptr<float>(), out.data_ptr<float>(), y.size(0), (int32_t)y.size(1), cur_stream()),
        "log_softmax backward");
  return out;
}

static void need_nll(const Tensor& x, const Tensor& t, const std::optional<Tensor>& w, int64_t reduction) {
  NEED(f32(x) && x.dim() == 2 && x.numel() > 0 && x.size(1) < (1ll << 31) && is_dev(t) && t.scalar_type() == at::kLong && t.dim() == 1 &&
           t.size(0) == x.size(0),
       "nll_loss on (N, C) float32 with int64 targets");
  NEED(!defined(w) || (f32(*w) && w->dim() == 1 && w->size(0) == x.size(1)), "float32 class weights");
  NEED(reduction >= 0 && reduction <= 2, "reduction");
}

static std::tuple<Tensor, Tensor> nll_fwd(const Tensor& x_, const Tensor& t_, const std::optional<Tensor>& w_, int64_t reduction, int64_t ignore) {
  need_nll(x_, t_, w_, reduction);
  Tensor x = contig(x_), t = contig(t_), wk;
  const float* w = wptr(w_, wk);
  Tensor loss = reduction == 0 ? empty_dev({x.size(0)}, at::kFloat) : empty_dev({}, at::kFloat), tw = empty_dev({}, at::kFloat);
  check(omt_nll_loss(x.data_ptr<float>(), t.data_ptr<int64_t>(), w, loss.data_ptr<float>(), tw.data_ptr<float>(), x.size(0), (int32_t)x.size(1), ignore,
                     (int32_t)reduction, cur_stream()),
        "nll_loss");
  return {loss, tw};
}

// g for reduction none is [N], else a scalar
static void need_grad(const Tensor& g, const Tensor& x, int64_t reduction) {
  NEED(f32(g) && (reduction == 0 ? (g.dim() == 1 && g.size(0) == x.size(0)) : g.numel() == 1), "gradient of the loss");
}

static Tensor nll_bwd(const Tensor& g_, const Tensor& x, const Tensor& t_, const std::optional<Tensor>& w_, int64_t reduction, int64_t ignore,
                      const Tensor& total_weight) {
  need_nll(x, t_, w_, reduction);
  need_grad(g_, x, reduction);
  NEED(reduction != 1 || f32(total_weight), "total weight on the device");
  Tensor g = contig(g_), t = contig(t_), wk;
  const float* w = wptr(w_, wk);
  Tensor gx = empty_dev(x.sizes(), at::kFloat);
  check(omt_nll_loss_backward(g.data_ptr<float>(), t.data_ptr<int64_t>(), w, reduction == 1 ? total_weight.data_ptr<float>() : nullptr,
                              gx.data_ptr<float>(), x.size(0), (int32_t)x.size(1), ignore, (int32_t)reduction, cur_stream()),
        "nll_loss backward");
  return gx;
}

// ---- the fused pair ---------------------------------------------------------------------------------------------------

static std::tuple<Tensor, Tensor, Tensor> softmax_nll_ref(const Tensor& x, const Tensor& t, const std::optional<Tensor>& w, int64_t reduction,
                                                          int64_t ignore) {
  Tensor lp = at::_log_softmax(x, 1, false);
  auto [loss, tw] = at::nll_loss_forward(lp, t, w, reduction, ignore);
  return {loss, lp, tw};
}
static Tensor softmax_nll_backward_ref(const Tensor& g, const Tensor& lp, const Tensor& t, const std::optional<Tensor>& w, int64_t reduction,
                                       int64_t ignore, const Tensor& tw) {
  return at::_log_softmax_backward_data(at::nll_loss_backward(g, lp, t, w, reduction, ignore, tw), lp, 1, lp.scalar_type());
}

static std::tuple<Tensor, Tensor, Tensor> softmax_nll_dev(const Tensor& x_, const Tensor& t_, const std::optional<Tensor>& w_, int64_t reduction,
                                                          int64_t ignore) {
  need_nll(x_, t_, w_, reduction);
  Tensor x = contig(x_), t = contig(t_), wk;
  const float* w = wptr(w_, wk);
  Tensor lp = empty_dev(x.sizes(), at::kFloat);
  Tensor loss = reduction == 0 ? empty_dev({x.size(0)}, at::kFloat) : empty_dev({}, at::kFloat), tw = empty_dev({}, at::kFloat);
  check(omt_softmax_nll(x.data_ptr<float>(), t.data_ptr<int64_t>(), w, lp.data_ptr<float>(), loss.data_ptr<float>(), tw.data_ptr<float>(), x.size(0),
                        (int32_t)x.size(1), ignore, (int32_t)reduction, cur_stream()),
        "softmax_nll");
  return {loss, lp, tw};
}
static Tensor softmax_nll_backward_dev(const Tensor& g_, const Tensor& lp_, const Tensor& t_, const std::optional<Tensor>& w_, int64_t reduction,
                                       int64_t ignore, const Tensor& tw) {
  need_nll(lp_, t_, w_, reduction);
  need_grad(g_, lp_, reduction);
  NEED(reduction != 1 || f32(tw), "total weight on the device");
  Tensor g = contig(g_), lp = contig(lp_), t = contig(t_), wk;
  const float* w = wptr(w_, wk);
  Tensor dx = empty_dev(lp.sizes(), at::kFloat);
  check(omt_softmax_nll_backward(g.data_ptr<float>(), lp.data_ptr<float>(), t.data_ptr<int64_t>(), w, reduction == 1 ? tw.data_ptr<float>() : nullptr,
                                 dx.data_ptr<float>(), lp.size(0), (int32_t)lp.size(1), ignore, (int32_t)reduction, cur_stream()),
        "softmax_nll backward");
  return dx;
}

TORCH_LIBRARY_FRAGMENT(omt, m) {
  m.def("softmax_nll(Tensor x, Tensor target, Tensor? weight, int reduction, int ignore_index) -> (Tensor, Tensor, Tensor)");
  m.def("softmax_nll_backward(Tensor g, Tensor logp, Tensor target, Tensor? weight, int reduction, int ignore_index, Tensor total_weight) -> Tensor");
}
TORCH_LIBRARY_IMPL(omt, CompositeExplicitAutograd, m) {
  m.impl("softmax_nll", &softmax_nll_ref);
  m.impl("softmax_nll_backward", &softmax_nll_backward_ref);
}
TORCH_LIBRARY_IMPL(omt, PrivateUse1, m) {
  m.impl("softmax_nll", [](const Tensor& x, const Tensor& t, const std::optional<Tensor>& w, int64_t reduction, int64_t ignore) {
    return dev_or_composite<&softmax_nll_dev, &softmax_nll_ref>("softmax_nll", x, t, w, reduction, ignore);
  });
  m.impl("softmax_nll_backward", [](const Tensor& g, const Tensor& lp, const Tensor& t, const std::optional<Tensor>& w, int64_t reduction, int64_t ignore,
                                    const Tensor& tw) {
    return dev_or_composite<&softmax_nll_backward_dev, &softmax_nll_backward_ref>("softmax_nll_backward", g, lp, t, w, reduction, ignore, tw);
  });
}
TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  OMT_IMPL(m, _log_softmax, log_softmax_);
  OMT_IMPL(m, _log_softmax_backward_data, log_softmax_bwd_);
  OMT_IMPL(m, nll_loss_forward, nll_fwd);
  OMT_IMPL(m, nll_loss_backward, nll_bwd);
}

}  // namespace omt

// aten::convolution / aten::convolution_backward for the device: dense (implicit GEMM: tensor-core or exact-fp32 path,
// chosen inside libomt_b200.so) and depthwise. Same coverage rules as the reference's conv_kind (csrc/conv.cpp:167-177)
// and the same op signatures (csrc/conv.cpp:179-237, 285-288); tile planning / autotuning callbacks of the reference
// (csrc/conv.cpp:29-60, 116-155) have no counterpart because the kernels are compiled ahead of time and pick their
// tile from the geometry, so the planner/tuning bindings are kept as inert shims.
#include "omt.h"

#include <cstdlib>

#include <pybind11/functional.h>
#include <pybind11/stl.h>

namespace omt {

int g_fold = 1;
static int g_cl_mode = 0;  // 0: conv outputs follow the input layout; 1: channels-last whenever co % 4 == 0
static bool g_tune = true;
static int g_num_tiles = 0;

OmtConvGeo conv_geo(int64_t n, int64_t ci, int64_t co, int64_t ih, int64_t iw, int64_t ks, int64_t stride, int64_t pad, int64_t groups) {
  OmtConvGeo g;
  g.n = (int)n; g.ci = (int)ci; g.co = (int)co; g.ih = (int)ih; g.iw = (int)iw;
  g.oh = (int)((ih + 2 * pad - ks) / stride + 1); g.ow = (int)((iw + 2 * pad - ks) / stride + 1);
  g.ks = (int)ks; g.stride = (int)stride; g.pad = (int)pad; g.groups = (int)groups;
  return g;
}

bool prefer_cl(const Tensor& x, int64_t co) {
  if (layout4(x) == 1 && !(x.is_contiguous())) return true;
  return g_cl_mode == 1 && co % 4 == 0;
}

// which device path covers a convolution ("" = none): csrc/conv.cpp:167-177
static std::string conv_kind(const Tensor& x, const Tensor& w, IntArrayRef stride, IntArrayRef padding, IntArrayRef dilation,
                             bool transposed, int64_t groups) {
  if (transposed || !f32(x) || !f32(w) || x.dim() != 4 || w.dim() != 4) return "";
  if (dilation[0] != 1 || dilation[1] != 1 || w.size(2) != w.size(3)) return "";
  if (stride[0] != stride[1] || padding[0] != padding[1]) return "";
  int64_t ks = w.size(2), s = stride[0], p = padding[0];
  if (x.numel() == 0 || (x.size(2) + 2 * p - ks) / s + 1 <= 0 || (x.size(3) + 2 * p - ks) / s + 1 <= 0) return "";
  if (groups == 1 && ks <= 11 && s >= 1 && s <= 4 && p <= ks) return "dense";
  if (groups == x.size(1) && groups == w.size(0) && groups > 1 && ks <= 11 && s >= 1 && s <= 4 && p <= ks) return "dw";
  return "";
}

Tensor conv_forward(const Tensor& x, const Tensor& w, const Tensor* bias, const OmtConvGeo& g, bool relu) {
  Tensor out = empty_dev({g.n, g.co, g.oh, g.ow}, at::kFloat, prefer_cl(x, g.co));
  out = dense4(out);
  OmtAct ax = act(x), ay = act(out);
  uint32_t flags = (bias ? OMT_EPI_BIAS : 0u) | (relu ? OMT_EPI_RELU : 0u);
  check(omt_conv_fwd(&g, &ax, w.data_ptr<float>(), bias ? bias->data_ptr<float>() : nullptr, &ay, nullptr, flags, nullptr, 0,
                     cur_stream()),
        "conv forward");
  return out;
}

Tensor conv_forward_stats(const Tensor& x, const Tensor& w, const Tensor* bias, const OmtConvGeo& g, Tensor& partials, int& groups) {
  Tensor out = dense4(empty_dev({g.n, g.co, g.oh, g.ow}, at::kFloat, prefer_cl(x, g.co)));
  OmtAct ax = act(x), ay = act(out);
  // OMARCHY_MAC_TORCH_EPILOGUE_STATS=0 leaves the statistics to a separate pass over y (for A/B measurements)
  static const bool enabled = [] { const char* e = std::getenv("OMARCHY_MAC_TORCH_EPILOGUE_STATS"); return !(e && e[0] == '0'); }();
  groups = enabled ? omt_conv_bnstats_groups(&g, &ax, &ay) : 0;
  uint32_t flags = bias ? OMT_EPI_BIAS : 0u;
  if (groups > 0) {
    partials = empty_dev({(int64_t)omt_conv_bnstats_floats(groups, g.co)}, at::kFloat);
    flags |= OMT_EPI_BNSTATS;
  }
  check(omt_conv_fwd(&g, &ax, w.data_ptr<float>(), bias ? bias->data_ptr<float>() : nullptr, &ay, groups > 0 ? partials.data_ptr<float>() : nullptr,
                     flags, nullptr, 0, cur_stream()),
        "conv forward");
  return out;
}

static Tensor convolution_(const Tensor& x_, const Tensor& w_, const std::optional<Tensor>& bias, IntArrayRef stride,
                           IntArrayRef padding, IntArrayRef dilation, bool transposed, IntArrayRef, int64_t groups) {
  std::string kind = conv_kind(x_, w_, stride, padding, dilation, transposed, groups);
  NEED(!kind.empty(), "dilated, transposed, grouped or non-square convolution");
  bool has_bias = defined(bias);
  NEED(!has_bias || f32(*bias), "float32 bias");
  Tensor x = dense4(x_), w = contig(w_);
  Tensor b = has_bias ? contig(*bias) : Tensor();
  OmtConvGeo g = conv_geo(x.size(0), x.size(1), w.size(0), x.size(2), x.size(3), w.size(2), stride[0], padding[0], groups);
  if (kind == "dense") return conv_forward(x, w, has_bias ? &b : nullptr, g, false);
  Tensor out = dense4(empty_dev({g.n, g.co, g.oh, g.ow}, at::kFloat, layout4(x) == 1 && !x.is_contiguous()));
  OmtAct ax = act(x), ay = act(out);
  check(omt_dw_fwd(&g, &ax, w.data_ptr<float>(), fptr(b), &ay, has_bias ? OMT_EPI_BIAS : 0u, cur_stream()), "depthwise forward");
  return out;
}

static std::tuple<Tensor, Tensor, Tensor> convolution_backward_(const Tensor& gy_, const Tensor& x_, const Tensor& w_,
                                                                at::OptionalIntArrayRef, IntArrayRef stride, IntArrayRef padding,
                                                                IntArrayRef dilation, bool transposed, IntArrayRef, int64_t groups,
                                                                std::array<bool, 3> mask) {
  std::string kind = conv_kind(x_, w_, stride, padding, dilation, transposed, groups);
  NEED(!kind.empty() && f32(gy_), "dilated, transposed, grouped or non-square convolution");
  Tensor gy = dense4(gy_), x = dense4(x_), w = contig(w_);
  OmtConvGeo g = conv_geo(x.size(0), x.size(1), w.size(0), x.size(2), x.size(3), w.size(2), stride[0], padding[0], groups);
  NEED(gy.size(2) == g.oh && gy.size(3) == g.ow, "grad_output size does not match the geometry");
  const bool cl = layout4(x) == 1 && !x.is_contiguous();
  OmtAct ag = act(gy), ax = act(x);
  Tensor gx, gw, gb;
  if (mask[0]) {
    gx = dense4(empty_dev(x.sizes(), at::kFloat, cl));
    OmtAct adx = act(gx);
    if (kind == "dense") check(omt_conv_dgrad(&g, &ag, w.data_ptr<float>(), &adx, 0, nullptr, 0, cur_stream()), "conv input gradient");
    else check(omt_dw_dgrad(&g, &ag, w.data_ptr<float>(), &adx, cur_stream()), "depthwise input gradient");
  }
  if (mask[1]) {
    gw = empty_dev(w.sizes(), at::kFloat);
    if (kind == "dense") check(omt_conv_wgrad(&g, &ax, &ag, gw.data_ptr<float>(), 1.f, 0, nullptr, 0, cur_stream()), "conv weight gradient");
    else check(omt_dw_wgrad(&g, &ax, &ag, gw.data_ptr<float>(), 1.f, cur_stream()), "depthwise weight gradient");
  }
  if (mask[2]) {
    gb = empty_dev({g.co}, at::kFloat);
    check(omt_conv_bias_grad(&ag, g.n, g.co, g.oh, g.ow, gb.data_ptr<float>(), 1.f, cur_stream()), "conv bias gradient");
  }
  return {gx, gw, gb};
}

// omt::conv_backward_acc: convolution_backward whose input gradient is ADDED to `acc` (a gradient that another consumer
// of the same tensor already produced) instead of being written to a new tensor and summed by a separate add. The
// compile backend rewrites  add(convolution_backward(...)[0], other)  to it when `other` is used nowhere else. The
// tensor-core epilogue does the accumulation (TMA reduce-add); geometries outside that path add separately.
static std::tuple<Tensor, Tensor> conv_backward_acc_ref(const Tensor& gy, const Tensor& x, const Tensor& w, Tensor& acc, IntArrayRef stride,
                                                        IntArrayRef padding, bool need_w) {
  auto r = at::convolution_backward(gy, x, w, std::nullopt, stride, padding, {1, 1}, false, {0, 0}, 1, {true, need_w, false});
  acc.add_(std::get<0>(r));
  return {acc, std::get<1>(r)};
}
static std::tuple<Tensor, Tensor> conv_backward_acc_dev(const Tensor& gy_, const Tensor& x_, const Tensor& w_, Tensor& acc, IntArrayRef stride,
                                                        IntArrayRef padding, bool need_w) {
  std::string kind = conv_kind(x_, w_, stride, padding, {1, 1}, false, 1);
  NEED(kind == "dense" && f32(gy_) && f32(acc) && acc.sizes() == x_.sizes(), "dense float32 convolution");
  NEED(layout4(acc) >= 0 && (acc.is_contiguous() || acc.is_contiguous(at::MemoryFormat::ChannelsLast)), "accumulator must be dense");
  Tensor gy = dense4(gy_), x = dense4(x_), w = contig(w_);
  OmtConvGeo g = conv_geo(x.size(0), x.size(1), w.size(0), x.size(2), x.size(3), w.size(2), stride[0], padding[0], 1);
  NEED(gy.size(2) == g.oh && gy.size(3) == g.ow, "grad_output size does not match the geometry");
  OmtAct ag = act(gy), ax = act(x), aacc = act(acc);
  int st = omt_conv_dgrad(&g, &ag, w.data_ptr<float>(), &aacc, OMT_EPI_ACCUM, nullptr, 0, cur_stream());
  if (st == OMT_EINVAL) {  // not a tensor-core geometry: plain input gradient, then the add
    Tensor gx = dense4(empty_dev(x.sizes(), at::kFloat, layout4(acc) == 1));
    OmtAct adx = act(gx);
    check(omt_conv_dgrad(&g, &ag, w.data_ptr<float>(), &adx, 0, nullptr, 0, cur_stream()), "conv input gradient");
    acc.add_(gx);
  } else {
    check(st, "conv input gradient (accumulating)");
  }
  Tensor gw;
  if (need_w) {
    gw = empty_dev(w.sizes(), at::kFloat);
    check(omt_conv_wgrad(&g, &ax, &ag, gw.data_ptr<float>(), 1.f, 0, nullptr, 0, cur_stream()), "conv weight gradient");
  }
  return {acc, gw};
}

void bind_conv(py::module_& m) {
  // Inert shims for the reference's generated-kernel planner (csrc/conv.cpp:239-283): kept so code written against the
  // reference's _native module keeps importing; the CUDA kernels need no runtime source generation or per-shape tuning.
  m.def("set_conv_planner", [](py::object) {});
  m.def("set_fold", [](int f) { g_fold = f; });
  m.def("set_tuning", [](bool on, int num_tiles) { g_tune = on; g_num_tiles = num_tiles; });
  m.def("tune_dump", []() { return std::map<std::string, std::pair<int, double>>(); });
  m.def("tune_load", [](std::map<std::string, std::pair<int, double>>) {});
  m.def("tuned_plans", []() { return std::map<std::string, std::string>(); });
  m.def("set_channels_last", [](int mode) { g_cl_mode = mode; }, "0: conv outputs follow the input layout; 1: channels-last when co % 4 == 0");
  m.def("channels_last_mode", []() { return g_cl_mode; });
}

TORCH_LIBRARY_FRAGMENT(omt, m) {
  m.def("conv_backward_acc(Tensor gy, Tensor x, Tensor w, Tensor(a!) acc, int[] stride, int[] padding, bool need_w) -> (Tensor(a!), Tensor)");
}
TORCH_LIBRARY_IMPL(omt, CompositeExplicitAutograd, m) { m.impl("conv_backward_acc", &conv_backward_acc_ref); }
TORCH_LIBRARY_IMPL(omt, PrivateUse1, m) {
  m.impl("conv_backward_acc", [](const Tensor& gy, const Tensor& x, const Tensor& w, Tensor& acc, IntArrayRef stride, IntArrayRef padding, bool need_w) {
    OMT_LOCK;
    try {
      return conv_backward_acc_dev(gy, x, w, acc, stride, padding, need_w);
    } catch (const Unsupported& e) {
      note_fallback("conv_backward_acc", e.why);
      return conv_backward_acc_ref(gy, x, w, acc, stride, padding, need_w);
    }
  });
}
TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  OMT_IMPL(m, convolution, convolution_);
  OMT_IMPL(m, convolution_backward, convolution_backward_);
}

}  // namespace omt

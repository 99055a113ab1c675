// aten::convolution / aten::convolution_backward for the device: dense (implicit GEMM: tensor-core or exact-fp32 path,
// chosen inside libomt_b200.so) and depthwise. Same coverage rules as the reference's conv_kind (csrc/conv.cpp:167-177)
// and the same op signatures (csrc/conv.cpp:179-237, 285-288). The reference's planner callback (csrc/conv.cpp:29-60) has
// no counterpart: the kernels are compiled ahead of time and pick their tile from the geometry. Its tuning pass has
// (csrc/conv.cpp:116-155): with set_tuning(true, ...) the first use of a (pass, geometry) times the library's candidate
// plans (omt_conv_autotune) and later calls use the winner; tune_dump / tune_load / tuned_plans move the choices in and out.
#include "omt.h"

#include <array>
#include <cstdlib>
#include <map>
#include <mutex>
#include <set>
#include <string>

#include <cuda_runtime.h>

#include <pybind11/functional.h>
#include <pybind11/stl.h>

namespace omt {

int g_fold = 1;
static int g_cl_mode = 0;  // 0: conv outputs follow the input layout; 1: channels-last whenever co % 4 == 0
static bool g_tune = false;
static int g_num_tiles = 0;

// set_tuning(true): the first dense conv call of a (pass, geometry) runs the library's timing pass (csrc/conv.cpp:29-60
// conv_plan -> autotune on a cache miss). Not while the stream is being captured (the pass synchronises).
static std::mutex g_tuned_mu;
static std::set<std::array<int, 11>> g_tuned;
void maybe_tune(int kind, const OmtConvGeo& g) {
  if (!g_tune || g.groups != 1) return;
  const std::array<int, 11> key{kind, g.n, g.ci, g.co, g.ih, g.iw, g.oh, g.ow, g.ks, g.stride, g.pad};
  {
    std::lock_guard<std::mutex> l(g_tuned_mu);
    if (g_tuned.count(key)) return;
  }
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing((cudaStream_t)cur_stream(), &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return;
  int32_t tile = 0;
  double mult = 1.0;
  if (omt_conv_plan_get(kind, &g, &tile, &mult) == 0)  // nothing loaded for it
    check(omt_conv_autotune(kind, &g, nullptr, nullptr, nullptr, nullptr, cur_stream()), "conv tuning pass");
  std::lock_guard<std::mutex> l(g_tuned_mu);
  g_tuned.insert(key);
}

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
  maybe_tune(0, g);
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
  maybe_tune(0, g);  // (before the statistics query below: both follow the stored plan)
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
    if (kind == "dense") maybe_tune(1, g);
    if (kind == "dense") check(omt_conv_dgrad(&g, &ag, w.data_ptr<float>(), &adx, 0, nullptr, 0, cur_stream()), "conv input gradient");
    else check(omt_dw_dgrad(&g, &ag, w.data_ptr<float>(), &adx, cur_stream()), "depthwise input gradient");
  }
  if (mask[1]) {
    gw = empty_dev(w.sizes(), at::kFloat);
    if (kind == "dense") maybe_tune(2, g);
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
  maybe_tune(1, g);
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
    maybe_tune(2, g);
    check(omt_conv_wgrad(&g, &ax, &ag, gw.data_ptr<float>(), 1.f, 0, nullptr, 0, cur_stream()), "conv weight gradient");
  }
  return {acc, gw};
}

void bind_conv(py::module_& m) {
  // set_conv_planner is an inert shim for the reference's generated-kernel planner (csrc/conv.cpp:239-241): kept so code
  // written against the reference's _native module keeps importing; the CUDA kernels need no runtime source generation.
  m.def("set_conv_planner", [](py::object) {});
  m.def("set_fold", [](int f) { g_fold = f; });
  m.def("set_tuning", [](bool on, int num_tiles) { g_tune = on; g_num_tiles = num_tiles; });
  // geometry key "pass,n,ci,co,ih,iw,oh,ow,ks,stride,pad" -> (tile width in columns, split-K slice factor): csrc/conv.cpp:243-272
  m.def("tune_dump", []() {
    std::map<std::string, std::pair<int, double>> r;
    std::string text(omt_conv_plans_dump(nullptr, 0) + 1, '\0');
    omt_conv_plans_dump(text.data(), text.size());
    size_t pos = 0;
    while (pos < text.size() && text[pos]) {
      size_t nl = text.find('\n', pos);
      if (nl == std::string::npos) break;
      const std::string line = text.substr(pos, nl - pos);
      const size_t eq = line.find('='), comma = line.find(',', eq == std::string::npos ? 0 : eq);
      if (eq != std::string::npos && comma != std::string::npos)
        r[line.substr(0, eq)] = {std::stoi(line.substr(eq + 1, comma - eq - 1)), std::stod(line.substr(comma + 1))};
      pos = nl + 1;
    }
    return r;
  });
  m.def("tune_load", [](std::map<std::string, std::pair<int, double>> entries) {
    std::string text;
    for (auto& e : entries) text += e.first + "=" + std::to_string(e.second.first) + "," + std::to_string(e.second.second) + "\n";
    return omt_conv_plans_load(text.c_str());
  });
  m.def("tuned_plans", []() {
    std::map<std::string, std::string> r;
    std::string text(omt_conv_plans_dump(nullptr, 0) + 1, '\0');
    omt_conv_plans_dump(text.data(), text.size());
    size_t pos = 0;
    while (pos < text.size() && text[pos]) {
      size_t nl = text.find('\n', pos);
      if (nl == std::string::npos) break;
      const std::string line = text.substr(pos, nl - pos);
      const size_t eq = line.find('=');
      if (eq != std::string::npos) r[line.substr(0, eq)] = line.substr(eq + 1);
      pos = nl + 1;
    }
    return r;
  });
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

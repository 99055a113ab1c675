// Fused conv / BatchNorm+ReLU / pool stacks: an nn.Sequential compiled once per input shape into a fixed list of
// kernel calls, driven from Python by a small autograd Function (stacks.py). Same Python-visible contract as the
// reference's csrc/plans.cpp:338-360: make_plan(layers, shape, train, input_grad, params, rms, rvs) -> Plan with
// forward(x), backward(g) -> (gx | None, [grads]) and a `busy` flag; gradients are views into one slab (csrc/plans.cpp:54-60,
// 319-328) so a data-parallel bucket can be reduced in place.
//
// What differs from the reference: the step list calls C-ABI kernels; a training conv -> BatchNorm+ReLU -> max pool block is
// three launches (the conv, whose epilogue also reduces the batch statistics; the merge of those partial statistics; one
// pass that normalises, applies the ReLU and pools with a 1-byte argmax) where the reference runs five (csrc/plans.cpp:
// 135-138, 180-199); the BN backward is ReLU-masked; conv layers may carry a bias, eval plans fold BatchNorm into the weights of the
// conv that produces its input (one GEMM with bias+ReLU epilogue per conv-BN-ReLU block), and activations come from the
// caching allocator per call instead of plan-owned buffers, so outputs need no copy out of the plan.
#include "omt.h"

#include <pybind11/stl.h>

namespace omt {

namespace {

struct Layer {
  std::string kind;  // conv convb dw dwb bn pool apool gap   ("b" = carries a bias)
  int64_t ci = 0, co = 0, ks = 0;
  double momentum = 0.1;
  int param = -1;  // index of the first parameter of this layer in Plan::params
  int bn = -1;     // index into rms / rvs
  bool is_conv() const { return kind == "conv" || kind == "convb"; }
  bool is_dw() const { return kind == "dw" || kind == "dwb"; }
  bool has_bias() const { return kind == "convb" || kind == "dwb"; }
};
struct Saved {  // what backward needs from forward, per layer
  Tensor x, y, stats, idx;
  Tensor partials;  // a bn layer: partial batch statistics the conv in front of it reduced in its epilogue
  int groups = 0;
};
struct GradSlot {
  int param;
  int64_t off, numel;
};

constexpr float kEps = 1e-5f;  // fusable() only admits BatchNorm2d with eps == 1e-5 (stacks.py)

}  // namespace

struct Plan {
  bool train = false, input_grad = false, busy = false;
  std::vector<int64_t> shape;
  std::vector<Layer> layers;
  std::vector<Tensor> params, rms, rvs;
  std::vector<Saved> saved;
  std::vector<GradSlot> slots;
  int64_t gwords = 0;
  Tensor gstore;
};

static int64_t add_slot(Plan& p, int param, int64_t numel) {
  int64_t off = p.gwords;
  p.slots.push_back({param, off, numel});
  p.gwords += (std::max<int64_t>(numel, 1) + 63) / 64 * 64;  // 256-byte aligned slots
  return off;
}

static std::shared_ptr<Plan> build_plan(const std::vector<Layer>& layers_, std::vector<int64_t> shape, bool train, bool input_grad,
                                        std::vector<Tensor> params, std::vector<Tensor> rms, std::vector<Tensor> rvs) {
  OMT_LOCK;
  ensure_init();
  NEED(shape.size() == 4, "plan input must be 4-D");
  for (auto& t : params) NEED(f32(t) && t.is_contiguous(), "plan parameters must be contiguous float32 tensors");
  auto P = std::make_shared<Plan>();
  Plan& p = *P;
  p.train = train; p.input_grad = input_grad; p.shape = shape;
  p.params = params; p.rms = rms; p.rvs = rvs;
  p.layers = layers_;
  int pi = 0, bi = 0;
  int64_t c = shape[1], h = shape[2], w = shape[3];
  for (Layer& L : p.layers) {
    if (L.is_conv() || L.is_dw()) {
      NEED(L.ci == c, "layer channel count does not match its input");
      NEED(pi + (L.has_bias() ? 2 : 1) <= (int)params.size(), "too few parameters for the layer list");
      L.param = pi;
      pi += L.has_bias() ? 2 : 1;
      c = L.co;
    } else if (L.kind == "bn") {
      NEED(pi + 2 <= (int)params.size() && bi < (int)rms.size() && bi < (int)rvs.size(), "too few BatchNorm parameters");
      NEED(params[pi].numel() == c, "BatchNorm width does not match its input");
      L.param = pi; L.bn = bi;
      pi += 2; bi++;
    } else if (L.kind == "pool" || L.kind == "apool") {
      NEED(h >= 2 && w >= 2, "2x2 pool on an input smaller than 2x2");
      h /= 2; w /= 2;
    } else if (L.kind == "gap") {
      h = 1; w = 1;
    } else {
      NEED(false, "unknown plan layer kind");
    }
  }
  if (train) {  // gradient slab: one slot per parameter, in backward order like the reference
    for (int li = (int)p.layers.size() - 1; li >= 0; li--) {
      const Layer& L = p.layers[li];
      if (L.kind == "bn") {
        add_slot(p, L.param, params[L.param].numel() * 2);  // [dgamma | dbeta]
      } else if (L.is_conv() || L.is_dw()) {
        add_slot(p, L.param, params[L.param].numel());
        if (L.has_bias()) add_slot(p, L.param + 1, params[L.param + 1].numel());
      }
    }
  }
  p.saved.resize(p.layers.size());
  return P;
}

static Tensor run_conv(const Tensor& x, const Tensor& w, const Tensor* bias, const Layer& L, bool relu) {
  OmtConvGeo g = conv_geo(x.size(0), x.size(1), L.co, x.size(2), x.size(3), L.ks, 1, L.ks / 2, L.is_dw() ? L.ci : 1);
  if (L.is_conv()) return conv_forward(x, w, bias, g, relu);
  Tensor out = dense4(empty_dev({g.n, g.co, g.oh, g.ow}, at::kFloat, layout4(x) == 1));
  OmtAct ax = act(x), ay = act(out);
  check(omt_dw_fwd(&g, &ax, w.data_ptr<float>(), bias ? bias->data_ptr<float>() : nullptr, &ay,
                   (bias ? OMT_EPI_BIAS : 0u) | (relu ? OMT_EPI_RELU : 0u), cur_stream()),
        "plan depthwise forward");
  return out;
}

static Tensor plan_forward(Plan& p, const Tensor& x_) {
  OMT_LOCK;
  check_errors();
  TORCH_CHECK(f32(x_) && x_.dim() == 4 && x_.sizes() == IntArrayRef(p.shape), "omarchy-mac-torch plan: bad input");
  Tensor cur = dense4(x_);
  for (size_t li = 0; li < p.layers.size(); li++) {
    const Layer& L = p.layers[li];
    Saved& sv = p.saved[li];
    const int n = (int)cur.size(0), c = (int)cur.size(1), h = (int)cur.size(2), w = (int)cur.size(3);
    if (p.train) sv.x = cur;
    if (L.is_conv() || L.is_dw()) {
      const Tensor& wt = p.params[L.param];
      const Tensor* bias = L.has_bias() ? &p.params[L.param + 1] : nullptr;
      // eval: BatchNorm(+ReLU) right after the conv is folded into its weights and bias (fold_bn, csrc/fused.cpp:34-40)
      bool fold = !p.train && g_fold > 0 && li + 1 < p.layers.size() && p.layers[li + 1].kind == "bn";
      if (fold) {
        const Layer& B = p.layers[li + 1];
        Tensor scale = p.params[B.param] * at::rsqrt(p.rvs[B.bn] + (double)kEps);
        Tensor fw = (wt * scale.view({-1, 1, 1, 1})).contiguous();
        Tensor fb = ((bias ? (*bias - p.rms[B.bn]) : -p.rms[B.bn]) * scale + p.params[B.param + 1]).contiguous();
        cur = run_conv(cur, fw, &fb, L, true);
        li++;  // the bn layer is done
      } else if (p.train && L.is_conv() && li + 1 < p.layers.size() && p.layers[li + 1].kind == "bn") {
        // the conv epilogue reduces the BatchNorm's batch statistics while it stores its output
        OmtConvGeo g = conv_geo(cur.size(0), cur.size(1), L.co, cur.size(2), cur.size(3), L.ks, 1, L.ks / 2, 1);
        Saved& nx = p.saved[li + 1];
        cur = conv_forward_stats(cur, wt, bias, g, nx.partials, nx.groups);
      } else {
        cur = run_conv(cur, wt, bias, L, false);
      }
    } else if (L.kind == "bn") {
      if (layout4(cur) == 1 && c % 4 != 0) {
        cur = to_layout(cur, 0);
        sv.groups = 0;  // the partial statistics belong to the tensor the conv wrote; this copy is reduced the usual way
        if (p.train) sv.x = cur;
      }
      Tensor y = dense4(empty_dev(cur.sizes(), at::kFloat, layout4(cur) == 1));
      OmtAct ax = act(cur), ay = act(y);
      if (p.train) {
        sv.stats = empty_dev({3 * (int64_t)c}, at::kFloat);  // mean | invstd | var
        float* s = sv.stats.data_ptr<float>();
        if (sv.groups > 0) {
          check(omt_bn_stats_from_partials(sv.partials.data_ptr<float>(), sv.groups, c, s, s + 2 * c, s + c, fptr(p.rms[L.bn]), fptr(p.rvs[L.bn]),
                                           nullptr, nullptr, (float)L.momentum, kEps, 0, cur_stream()),
                "plan BN statistics from the conv epilogue");
        } else {
          check(omt_bn_stats(&ax, n, c, h, w, s, s + 2 * c, s + c, fptr(p.rms[L.bn]), fptr(p.rvs[L.bn]), nullptr, nullptr, (float)L.momentum,
                             kEps, 0, cur_stream()),
                "plan BN statistics");
        }
        sv.partials = Tensor(); sv.groups = 0;
        sv.y = y;
        if (li + 1 < p.layers.size() && p.layers[li + 1].kind == "pool" && h % 2 == 0 && w % 2 == 0) {
          // normalise + ReLU + 2x2 max pool in one pass; y is still written (the backward masks with it)
          const bool cl = layout4(cur) == 1;
          Tensor z = dense4(empty_dev({n, c, h / 2, w / 2}, at::kFloat, cl));
          Tensor idx = empty_dev({n, c, h / 2, w / 2}, at::kByte, cl).as_strided(z.sizes(), z.strides());
          OmtAct az = act(z);
          check(omt_bn_apply_pool2(&ax, &ay, &az, idx.data_ptr<uint8_t>(), n, c, h, w, s, s + c, fptr(p.params[L.param]),
                                   fptr(p.params[L.param + 1]), OMT_BN_RELU, cur_stream()),
                "plan BN apply + max pool");
          Saved& pv = p.saved[li + 1];
          pv.x = y; pv.idx = idx;
          cur = z;
          li++;  // the pool layer is done
          continue;
        }
        check(omt_bn_apply(&ax, &ay, n, c, h, w, s, s + c, fptr(p.params[L.param]), fptr(p.params[L.param + 1]), OMT_BN_RELU, cur_stream()),
              "plan BN apply");
      } else {
        check(omt_bn_eval(&ax, &ay, n, c, h, w, fptr(p.rms[L.bn]), fptr(p.rvs[L.bn]), fptr(p.params[L.param]), fptr(p.params[L.param + 1]), kEps,
                          OMT_BN_RELU, cur_stream()),
              "plan BN eval");
      }
      cur = y;
    } else if (L.kind == "pool") {
      Tensor y = dense4(empty_dev({n, c, h / 2, w / 2}, at::kFloat, layout4(cur) == 1));
      Tensor idx = empty_dev({n, c, h / 2, w / 2}, at::kByte, layout4(cur) == 1).as_strided(y.sizes(), y.strides());
      OmtAct ax = act(cur), ay = act(y);
      check(omt_pool2_fwd(&ax, &ay, idx.data_ptr<uint8_t>(), n, c, h, w, cur_stream()), "plan max pool");
      if (p.train) sv.idx = idx;
      cur = y;
    } else if (L.kind == "apool") {
      Tensor y = dense4(empty_dev({n, c, h / 2, w / 2}, at::kFloat, layout4(cur) == 1));
      OmtAct ax = act(cur), ay = act(y);
      check(omt_avgpool2_fwd(&ax, &ay, n, c, h, w, cur_stream()), "plan avg pool");
      cur = y;
    } else {  // gap
      Tensor y = empty_dev({n, c, 1, 1}, at::kFloat);
      OmtAct ax = act(cur), ay = act(y);
      check(omt_adaptive_avgpool_fwd(&ax, &ay, n, c, h, w, 1, 1, cur_stream()), "plan global avg pool");
      cur = y;
    }
  }
  return cur;
}

static std::pair<std::optional<Tensor>, std::vector<Tensor>> plan_backward(Plan& p, const Tensor& g_) {
  OMT_LOCK;
  check_errors();
  TORCH_CHECK(p.train, "omarchy-mac-torch plan: backward on an eval plan");
  // previous gradients may still be alive (gradient accumulation): never overwrite a slab that is referenced elsewhere
  if (!p.gstore.defined() || p.gstore.storage().use_count() > 1) p.gstore = empty_dev({std::max<int64_t>(p.gwords, 64)}, at::kFloat);
  float* gbase = p.gstore.data_ptr<float>();
  auto slot_of = [&](int param) -> float* {
    for (auto& s : p.slots)
      if (s.param == param) return gbase + s.off;
    TORCH_INTERNAL_ASSERT(false, "no gradient slot");
  };
  Tensor g = dense4(g_);
  for (int li = (int)p.layers.size() - 1; li >= 0; li--) {
    const Layer& L = p.layers[li];
    Saved& sv = p.saved[li];
    const Tensor& x = sv.x;
    const int n = (int)x.size(0), c = (int)x.size(1), h = (int)x.size(2), w = (int)x.size(3);
    const bool cl = layout4(x) == 1;
    const bool first = li == 0;
    if (L.kind == "pool") {
      Tensor gx = dense4(empty_dev(x.sizes(), at::kFloat, cl));
      g = to_layout(g, cl ? 1 : 0);
      OmtAct ag = act(g), agx = act(gx);
      check(omt_pool2_bwd(&ag, sv.idx.data_ptr<uint8_t>(), &agx, n, c, h, w, cur_stream()), "plan max pool backward");
      g = gx;
    } else if (L.kind == "apool") {
      Tensor gx = dense4(empty_dev(x.sizes(), at::kFloat, cl));
      OmtAct ag = act(g), agx = act(gx);
      check(omt_avgpool2_bwd(&ag, &agx, n, c, h, w, cur_stream()), "plan avg pool backward");
      g = gx;
    } else if (L.kind == "gap") {
      Tensor gx = dense4(empty_dev(x.sizes(), at::kFloat, cl));
      OmtAct ag = act(g), agx = act(gx);
      check(omt_adaptive_avgpool_bwd(&ag, &agx, n, c, h, w, 1, 1, cur_stream()), "plan global avg pool backward");
      g = gx;
    } else if (L.kind == "bn") {
      Tensor gx = dense4(empty_dev(x.sizes(), at::kFloat, cl));
      g = to_layout(g, cl ? 1 : 0);
      const float* s = sv.stats.data_ptr<float>();
      OmtAct ag = act(g), ax = act(x), ay = act(sv.y), agx = act(gx);
      check(omt_bn_backward(&ag, &ax, &ay, &agx, n, c, h, w, s, s + c, fptr(p.params[L.param]), slot_of(L.param), 1.f, OMT_BN_RELU, cur_stream()),
            "plan BN backward");
      g = gx;
    } else {  // conv / dw
      OmtConvGeo geo = conv_geo(n, c, L.co, h, w, L.ks, 1, L.ks / 2, L.is_dw() ? L.ci : 1);
      OmtAct ag = act(g), ax = act(x);
      if (L.is_conv()) check(omt_conv_wgrad(&geo, &ax, &ag, slot_of(L.param), 1.f, 0, nullptr, 0, cur_stream()), "plan conv weight gradient");
      else check(omt_dw_wgrad(&geo, &ax, &ag, slot_of(L.param), 1.f, cur_stream()), "plan depthwise weight gradient");
      if (L.has_bias()) check(omt_conv_bias_grad(&ag, n, (int)L.co, geo.oh, geo.ow, slot_of(L.param + 1), 1.f, cur_stream()), "plan bias gradient");
      if (!first || p.input_grad) {
        Tensor gx = dense4(empty_dev(x.sizes(), at::kFloat, cl));
        OmtAct agx = act(gx);
        const float* wt = p.params[L.param].data_ptr<float>();
        if (L.is_conv()) check(omt_conv_dgrad(&geo, &ag, wt, &agx, 0, nullptr, 0, cur_stream()), "plan conv input gradient");
        else check(omt_dw_dgrad(&geo, &ag, wt, &agx, cur_stream()), "plan depthwise input gradient");
        g = gx;
      }
    }
    sv = Saved();  // release the saved activations of this layer
  }
  std::vector<Tensor> grads(p.params.size());
  for (auto& s : p.slots) {
    const Tensor& prm = p.params[s.param];
    bool bn_pair = s.numel == 2 * prm.numel() && prm.dim() == 1;
    if (bn_pair) {
      grads[s.param] = p.gstore.as_strided({prm.numel()}, {1}, s.off);
      grads[s.param + 1] = p.gstore.as_strided({prm.numel()}, {1}, s.off + prm.numel());
    } else {
      grads[s.param] = p.gstore.as_strided(prm.sizes(), prm.strides(), s.off);
    }
  }
  std::optional<Tensor> gx;
  if (p.input_grad) gx = g;
  return {gx, grads};
}

void bind_plans(py::module_& m) {
  py::class_<Plan, std::shared_ptr<Plan>>(m, "Plan")
      .def_readwrite("busy", &Plan::busy)
      .def("forward", [](Plan& p, const Tensor& x) { return plan_forward(p, x); })
      .def("backward",
           [](Plan& p, const Tensor& g) {
             auto r = plan_backward(p, g);
             return py::make_tuple(r.first ? py::cast(*r.first) : py::none(), r.second);
           })
      .def("grad_slab", [](Plan& p) { return p.gstore; }, "the flat tensor the parameter gradients of the last backward are views of");
  m.def("make_plan", [](std::vector<std::tuple<std::string, int64_t, int64_t, int64_t, double>> layers, std::vector<int64_t> shape, bool train,
                        bool input_grad, std::vector<Tensor> params, std::vector<Tensor> rms, std::vector<Tensor> rvs) {
    std::vector<Layer> L;
    for (auto& t : layers) {
      Layer l;
      l.kind = std::get<0>(t); l.ci = std::get<1>(t); l.co = std::get<2>(t); l.ks = std::get<3>(t); l.momentum = std::get<4>(t);
      L.push_back(l);
    }
    try {
      return build_plan(L, shape, train, input_grad, params, rms, rvs);
    } catch (const Unsupported& e) {
      throw std::runtime_error(std::string("omarchy-mac-torch: cannot build a fused stack: ") + e.why);
    }
  });
}

}  // namespace omt

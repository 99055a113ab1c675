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
//   omt::fused_pointwise    a chain of elementwise ops in one kernel (compile pass 4). The reference passes the name of a
//                           shader it generated for the chain; here the `kernel` string is the chain itself, a small
//                           straight-line program that one ahead-of-time interpreter kernel runs (omt_pointwise)
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
// ---- pointwise programs ------------------------------------------------------------------------------------------------
// Text form, written by compile.py's pass 4:  "pw1|<n inputs>|<op>,<a>,<b>,<c>;...|<literal>,<literal>,..."  with operands
// vK (input K), tJ (result of instruction J) and #L (literal L; numbers in C hex-float notation, or inf / -inf / nan).
static const char* const kPwNames[OMT_PW_OP_COUNT] = {
    "add", "sub", "rsub", "mul", "div", "neg", "relu", "exp", "log", "sqrt", "rsqrt", "recip", "abs", "tanh", "sigmoid", "silu", "max", "min", "pow",
    "threshold_bwd", "sigmoid_bwd", "tanh_bwd", "silu_bwd", "gelu", "gelu_tanh", "gelu_bwd", "gelu_tanh_bwd", "clamp", "hardswish", "hardswish_bwd",
    "hardsigmoid", "hardsigmoid_bwd"};
struct PwParsed {
  OmtPwProgram prog{};
  int n_inputs = 0, n_literals = 0;
};
static std::vector<std::string> split(const std::string& s, char sep) {
  std::vector<std::string> out;
  size_t pos = 0;
  while (true) {
    size_t e = s.find(sep, pos);
    out.push_back(s.substr(pos, e == std::string::npos ? std::string::npos : e - pos));
    if (e == std::string::npos) break;
    pos = e + 1;
  }
  return out;
}
static const PwParsed& parse_program(const std::string& text) {
  static std::mutex mu;
  static std::map<std::string, PwParsed> cache;
  std::lock_guard<std::mutex> l(mu);
  auto it = cache.find(text);
  if (it != cache.end()) return it->second;
  PwParsed p;
  auto parts = split(text, '|');
  TORCH_CHECK(parts.size() == 4 && parts[0] == "pw1", "omt::fused_pointwise: not a pointwise program: ", text);
  p.n_inputs = std::stoi(parts[1]);
  TORCH_CHECK(p.n_inputs >= 1 && p.n_inputs <= OMT_PW_MAX_INPUTS, "omt::fused_pointwise: 1 to ", OMT_PW_MAX_INPUTS, " inputs");
  if (!parts[3].empty())
    for (auto& lit : split(parts[3], ',')) {
      TORCH_CHECK(p.n_literals < OMT_PW_MAX_LITERALS, "omt::fused_pointwise: too many literals");
      p.prog.literal[p.n_literals++] = std::strtof(lit.c_str(), nullptr);
    }
  for (auto& ins : split(parts[2], ';')) {
    auto f = split(ins, ',');
    TORCH_CHECK(f.size() == 4 && p.prog.n_instr < OMT_PW_MAX_INSTR, "omt::fused_pointwise: malformed or too long program: ", text);
    OmtPwInstr& o = p.prog.instr[p.prog.n_instr];
    o.op = -1;
    for (int k = 0; k < OMT_PW_OP_COUNT; k++)
      if (f[0] == kPwNames[k]) o.op = k;
    TORCH_CHECK(o.op >= 0, "omt::fused_pointwise: unknown op '", f[0], "'");
    int32_t* dst[3] = {&o.a, &o.b, &o.c};
    for (int q = 0; q < 3; q++) {
      const std::string& t = f[q + 1];
      TORCH_CHECK(t.size() >= 2, "omt::fused_pointwise: malformed operand '", t, "'");
      const int v = std::stoi(t.substr(1));
      if (t[0] == 'v') { TORCH_CHECK(v >= 0 && v < p.n_inputs, "omt::fused_pointwise: input out of range"); *dst[q] = v; }
      else if (t[0] == 't') { TORCH_CHECK(v >= 0 && v < p.prog.n_instr, "omt::fused_pointwise: use before definition"); *dst[q] = OMT_PW_MAX_INPUTS + v; }
      else if (t[0] == '#') { TORCH_CHECK(v >= 0 && v < p.n_literals, "omt::fused_pointwise: literal out of range"); *dst[q] = -1 - v; }
      else TORCH_CHECK(false, "omt::fused_pointwise: malformed operand '", t, "'");
    }
    p.prog.n_instr++;
  }
  TORCH_CHECK(p.prog.n_instr >= 1, "omt::fused_pointwise: empty program");
  return cache.emplace(text, p).first->second;
}

// composite definition: the program evaluated op by op with aten (any device)
static Tensor fused_pointwise_ref(c10::string_view kernel, at::TensorList ins) {
  const PwParsed& p = parse_program(std::string(kernel));
  TORCH_CHECK((int)ins.size() == p.n_inputs, "omt::fused_pointwise: the program takes ", p.n_inputs, " inputs, got ", ins.size());
  std::vector<Tensor> val(OMT_PW_MAX_INPUTS + p.prog.n_instr);
  for (int k = 0; k < p.n_inputs; k++) val[k] = ins[k];
  auto lit = [&](int32_t o) -> double { TORCH_CHECK(o < 0, "omt::fused_pointwise: this operand must be a number"); return p.prog.literal[-1 - o]; };
  auto ten = [&](int32_t o) -> Tensor { return o >= 0 ? val[o] : at::scalar_tensor(p.prog.literal[-1 - o], ins[0].options()); };
  Tensor r;
  for (int j = 0; j < p.prog.n_instr; j++) {
    const OmtPwInstr& i = p.prog.instr[j];
    switch (i.op) {
      case OMT_PW_ADD: r = at::add(ten(i.a), ten(i.b), lit(i.c)); break;
      case OMT_PW_SUB: r = at::sub(ten(i.a), ten(i.b), lit(i.c)); break;
      case OMT_PW_RSUB: r = at::sub(ten(i.b), ten(i.a), lit(i.c)); break;
      case OMT_PW_MUL: r = at::mul(ten(i.a), ten(i.b)); break;
      case OMT_PW_DIV: r = at::div(ten(i.a), ten(i.b)); break;
      case OMT_PW_NEG: r = at::neg(ten(i.a)); break;
      case OMT_PW_RELU: r = at::relu(ten(i.a)); break;
      case OMT_PW_EXP: r = at::exp(ten(i.a)); break;
      case OMT_PW_LOG: r = at::log(ten(i.a)); break;
      case OMT_PW_SQRT: r = at::sqrt(ten(i.a)); break;
      case OMT_PW_RSQRT: r = at::rsqrt(ten(i.a)); break;
      case OMT_PW_RECIP: r = at::reciprocal(ten(i.a)); break;
      case OMT_PW_ABS: r = at::abs(ten(i.a)); break;
      case OMT_PW_TANH: r = at::tanh(ten(i.a)); break;
      case OMT_PW_SIGMOID: r = at::sigmoid(ten(i.a)); break;
      case OMT_PW_SILU: r = at::silu(ten(i.a)); break;
      case OMT_PW_MAX: r = at::maximum(ten(i.a), ten(i.b)); break;
      case OMT_PW_MIN: r = at::minimum(ten(i.a), ten(i.b)); break;
      case OMT_PW_POW: r = at::pow(ten(i.a), lit(i.b)); break;
      case OMT_PW_THRESHOLD_BWD: r = at::threshold_backward(ten(i.a), ten(i.b), lit(i.c)); break;
      case OMT_PW_SIGMOID_BWD: r = at::sigmoid_backward(ten(i.a), ten(i.b)); break;
      case OMT_PW_TANH_BWD: r = at::tanh_backward(ten(i.a), ten(i.b)); break;
      case OMT_PW_SILU_BWD: r = at::silu_backward(ten(i.a), ten(i.b)); break;
      case OMT_PW_GELU: r = at::gelu(ten(i.a), "none"); break;
      case OMT_PW_GELU_TANH: r = at::gelu(ten(i.a), "tanh"); break;
      case OMT_PW_GELU_BWD: r = at::gelu_backward(ten(i.a), ten(i.b), "none"); break;
      case OMT_PW_GELU_TANH_BWD: r = at::gelu_backward(ten(i.a), ten(i.b), "tanh"); break;
      case OMT_PW_CLAMP: r = at::clamp(ten(i.a), lit(i.b), lit(i.c)); break;
      case OMT_PW_HARDSWISH: r = at::hardswish(ten(i.a)); break;
      case OMT_PW_HARDSWISH_BWD: r = at::hardswish_backward(ten(i.a), ten(i.b)); break;
      case OMT_PW_HARDSIGMOID: r = at::hardsigmoid(ten(i.a)); break;
      case OMT_PW_HARDSIGMOID_BWD: r = at::hardsigmoid_backward(ten(i.a), ten(i.b)); break;
      default: TORCH_CHECK(false, "omt::fused_pointwise: bad op");
    }
    val[OMT_PW_MAX_INPUTS + j] = r;
  }
  std::vector<int64_t> shape = ins[0].sizes().vec();  // (a chain whose last value is narrower than its inputs broadcasts like them)
  for (auto& t : ins) shape = at::infer_size(shape, t.sizes());
  return r.sizes() == IntArrayRef(shape) ? r : r.expand(shape).contiguous();
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

// device: one launch of the interpreter kernel. The output takes the layout of the first full-shape dense input (so a
// channels-last chain stays channels-last), else it is contiguous.
static Tensor fused_pointwise_dev(c10::string_view kernel, at::TensorList ins) {
  const PwParsed& p = parse_program(std::string(kernel));
  NEED((int)ins.size() == p.n_inputs, "input count");
  std::vector<int64_t> shape = ins[0].sizes().vec();
  for (auto& t : ins) {
    NEED(f32(t), "float32 device inputs");
    shape = at::infer_size(shape, t.sizes());
  }
  const int R = (int)shape.size();
  NEED(R <= 8, "rank <= 8");
  int64_t numel = 1;
  for (int64_t d : shape) numel *= d;
  NEED(numel > 0 && numel < (1ll << 40), "empty or oversized output");
  Tensor out;
  for (auto& t : ins)
    if (!out.defined() && t.sizes() == IntArrayRef(shape) && t.is_non_overlapping_and_dense() && !t.is_contiguous())
      out = empty_dev({numel}, at::kFloat).as_strided(shape, t.strides());
  if (!out.defined()) out = empty_dev(shape, at::kFloat);
  const float* ptrs[OMT_PW_MAX_INPUTS] = {};
  int64_t strides[OMT_PW_MAX_INPUTS * 8] = {}, ostr[8] = {};
  int32_t shp[8] = {};
  for (int d = 0; d < R; d++) { shp[d] = (int32_t)shape[d]; ostr[d] = out.stride(d); NEED(shape[d] < (1ll << 31), "dimension below 2^31"); }
  for (size_t k = 0; k < ins.size(); k++) {
    ptrs[k] = ins[k].data_ptr<float>();
    for (int d = 0; d < R; d++) {
      const int di = d - (R - (int)ins[k].dim());
      strides[k * 8 + d] = (di >= 0 && ins[k].size(di) != 1) ? ins[k].stride(di) : 0;
    }
  }
  check(omt_pointwise(&p.prog, p.n_inputs, ptrs, strides, ostr, shp, R, out.data_ptr<float>(), cur_stream()), "fused pointwise chain");
  return out;
}

// eager entry points for the non-functional BatchNorm variants that traced / compiled graphs call (csrc/fused.cpp:173-181)
static std::tuple<Tensor, Tensor, Tensor> bn_legit(const Tensor& x, const std::optional<Tensor>& w, const std::optional<Tensor>& b, Tensor& rm,
                                                   Tensor& rv, bool training, double mom, double eps) {
  return at::native_batch_norm(x, w, b, rm, rv, training, mom, eps);
}
static std::tuple<Tensor, Tensor, Tensor> bn_legit_no_training(const Tensor& x, const std::optional<Tensor>& w, const std::optional<Tensor>& b,
                                                               const Tensor& rm, const Tensor& rv, double mom, double eps) {
  return at::native_batch_norm(x, w, b, rm, rv, false, mom, eps);
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
  m.impl("fused_pointwise", [](c10::string_view kernel, at::TensorList ins) {
    return dev_or_composite<&fused_pointwise_dev, &fused_pointwise_ref>("fused_pointwise", kernel, ins);
  });
}
TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  OMT_IMPL(m, _native_batch_norm_legit, bn_legit);
  OMT_IMPL(m, _native_batch_norm_legit_no_training, bn_legit_no_training);
}

}  // namespace omt

// Batch norm, pooling and random fills for the device. Signatures and support rules follow the reference's
// csrc/nn.cpp (batch_norm_ :25-58, batch_norm_backward_ :60-78, pools :137-222, uniform_/normal_ :262-273); layer norm
// and dropout are not part of the hot path here and are served by the bridge.
#include "omt.h"

#include <ATen/CPUGeneratorImpl.h>
#include <ATen/native/Pool.h>

namespace omt {

at::CPUGeneratorImpl* generator(const std::optional<at::Generator>& gen);  // device.cpp

static bool whole(const Tensor& t) { return f32(t) && t.is_contiguous(); }
// activations the BN kernels take: NCHW-contiguous, or channels-last with c % 4 == 0
static Tensor bn_input(const Tensor& x_) {
  Tensor x = dense4(x_);
  if (layout4(x) == 1 && x.size(1) % 4 != 0) x = to_layout(x, 0);
  return x;
}

// ------------------------------------------------------------------------------------------------
// batch norm (affine, with running statistics)
// ------------------------------------------------------------------------------------------------

static std::tuple<Tensor, Tensor, Tensor> batch_norm_(const Tensor& x_, const std::optional<Tensor>& weight, const std::optional<Tensor>& bias,
                                                      const std::optional<Tensor>& rm, const std::optional<Tensor>& rv, bool training,
                                                      double momentum, double eps) {
  NEED(defined(weight) && defined(bias) && defined(rm) && defined(rv) && f32(x_) && x_.dim() == 4 && x_.numel() > 0,
       "batch norm without affine parameters or running stats, or not 4-D");
  NEED(whole(*weight) && whole(*bias) && whole(*rm) && whole(*rv), "batch norm parameters must be contiguous float32 tensors");
  Tensor x = bn_input(x_);
  const int n = (int)x.size(0), c = (int)x.size(1), h = (int)x.size(2), w = (int)x.size(3);
  Tensor y = dense4(empty_dev(x.sizes(), at::kFloat, layout4(x) == 1));
  OmtAct ax = act(x), ay = act(y);
  if (!training) {
    check(omt_bn_eval(&ax, &ay, n, c, h, w, fptr(rm), fptr(rv), fptr(weight), fptr(bias), (float)eps, 0, cur_stream()), "batch norm (eval)");
    return {y, empty_dev({0}, at::kFloat), empty_dev({0}, at::kFloat)};
  }
  Tensor stats = empty_dev({3 * (int64_t)c}, at::kFloat);  // mean | invstd | var
  float* s = stats.data_ptr<float>();
  check(omt_bn_stats(&ax, n, c, h, w, s, s + 2 * c, s + c, fptr(rm), fptr(rv), nullptr, nullptr, (float)momentum, (float)eps, 0, cur_stream()),
        "batch norm statistics");
  check(omt_bn_apply(&ax, &ay, n, c, h, w, s, s + c, fptr(weight), fptr(bias), 0, cur_stream()), "batch norm apply");
  return {y, stats.narrow(0, 0, c), stats.narrow(0, c, c)};
}

static std::tuple<Tensor, Tensor, Tensor> batch_norm_backward_(const Tensor& gy_, const Tensor& x_, const std::optional<Tensor>& weight,
                                                               const std::optional<Tensor>&, const std::optional<Tensor>&,
                                                               const std::optional<Tensor>& sm, const std::optional<Tensor>& si, bool train,
                                                               double, std::array<bool, 3> mask) {
  NEED(train && defined(weight) && defined(sm) && defined(si) && f32(x_) && f32(gy_) && x_.dim() == 4 && x_.numel() > 0,
       "eval-mode or non-affine batch norm backward");
  NEED(whole(*weight), "contiguous weight");
  Tensor x = bn_input(x_);
  Tensor gy = to_layout(gy_, layout4(x));
  Tensor mean = contig(*sm), inv = contig(*si);
  const int n = (int)x.size(0), c = (int)x.size(1), h = (int)x.size(2), w = (int)x.size(3);
  Tensor dgb = empty_dev({2, c}, at::kFloat);
  Tensor gx;
  OmtAct ag = act(gy), ax = act(x), adx = null_act(), none = null_act();
  if (mask[0]) {
    gx = dense4(empty_dev(x.sizes(), at::kFloat, layout4(x) == 1));
    adx = act(gx);
  }
  check(omt_bn_backward(&ag, &ax, &none, &adx, n, c, h, w, fptr(mean), fptr(inv), fptr(weight), dgb.data_ptr<float>(), 1.f, 0, cur_stream()),
        "batch norm backward");
  return {gx, mask[1] ? dgb.select(0, 0) : Tensor(), mask[2] ? dgb.select(0, 1) : Tensor()};
}

// ------------------------------------------------------------------------------------------------
// pooling
// ------------------------------------------------------------------------------------------------

static OmtPool pool_args(IntArrayRef k, IntArrayRef s, IntArrayRef p, IntArrayRef d) {
  auto at2 = [](IntArrayRef a, size_t i, int64_t dflt) { return a.empty() ? dflt : a[a.size() == 1 ? 0 : i]; };
  OmtPool r;
  r.kh = (int)at2(k, 0, 1); r.kw = (int)at2(k, 1, 1);
  r.sh = (int)at2(s, 0, r.kh); r.sw = (int)at2(s, 1, r.kw);
  r.ph = (int)at2(p, 0, 0); r.pw = (int)at2(p, 1, 0);
  r.dh = (int)at2(d, 0, 1); r.dw = (int)at2(d, 1, 1);
  return r;
}
static bool pool_ok(const Tensor& x, const OmtPool& a) {
  return f32(x) && x.dim() == 4 && x.numel() > 0 && a.kh > 0 && a.kw > 0 && a.sh > 0 && a.sw > 0 && a.ph <= a.kh / 2 && a.pw <= a.kw / 2;
}
static bool is_cl(const Tensor& x) { return layout4(x) == 1; }

static std::tuple<Tensor, Tensor> max_pool2d_(const Tensor& x_, IntArrayRef k, IntArrayRef s, IntArrayRef p, IntArrayRef d, bool ceil) {
  OmtPool a = pool_args(k, s, p, d);
  NEED(pool_ok(x_, a), "max pool: 4-D float32 with padding <= kernel / 2");
  Tensor x = dense4(x_);
  int64_t n = x.size(0), c = x.size(1), h = x.size(2), w = x.size(3);
  int64_t oh = at::native::pooling_output_shape<int64_t>(h, a.kh, a.ph, a.sh, a.dh, ceil);
  int64_t ow = at::native::pooling_output_shape<int64_t>(w, a.kw, a.pw, a.sw, a.dw, ceil);
  NEED(oh > 0 && ow > 0, "empty pooling output");
  Tensor out = dense4(empty_dev({n, c, oh, ow}, at::kFloat, is_cl(x)));
  Tensor idx = empty_dev({n, c, oh, ow}, at::kLong, is_cl(x)).as_strided({n, c, oh, ow}, out.strides());
  OmtAct ax = act(x), ay = act(out);
  check(omt_maxpool_fwd(&ax, &ay, idx.data_ptr<int64_t>(), (int)n, (int)c, (int)h, (int)w, (int)oh, (int)ow, &a, cur_stream()), "max pool");
  return {out, idx};
}
static Tensor max_pool2d_backward_(const Tensor& gy_, const Tensor& x, IntArrayRef k, IntArrayRef s, IntArrayRef p, IntArrayRef d, bool,
                                   const Tensor& idx_) {
  OmtPool a = pool_args(k, s, p, d);
  NEED(pool_ok(x, a) && f32(gy_) && is_dev(idx_) && idx_.scalar_type() == at::kLong, "max pool backward");
  Tensor idx = idx_;
  if (layout4(idx) < 0) idx = contig(idx);
  const int lay = layout4(idx) == 1 ? 1 : 0;
  Tensor gy = to_layout(gy_, lay);
  int64_t n = x.size(0), c = x.size(1), h = x.size(2), w = x.size(3);
  idx = idx.as_strided(idx.sizes(), gy.strides());  // same layout as gy after canonicalisation
  Tensor gx = dense4(empty_dev(x.sizes(), at::kFloat, lay == 1));
  OmtAct ag = act(gy), agx = act(gx);
  check(omt_maxpool_bwd(&ag, idx.data_ptr<int64_t>(), &agx, (int)n, (int)c, (int)h, (int)w, (int)gy.size(2), (int)gy.size(3), &a, cur_stream()),
        "max pool backward");
  return gx;
}

static Tensor avg_pool2d_(const Tensor& x_, IntArrayRef k, IntArrayRef s, IntArrayRef p, bool ceil, bool include_pad,
                          std::optional<int64_t> divisor) {
  OmtPool a = pool_args(k, s, p, {});
  NEED(pool_ok(x_, a) && (!divisor || *divisor > 0), "avg pool: 4-D float32 with padding <= kernel / 2");
  Tensor x = dense4(x_);
  int64_t n = x.size(0), c = x.size(1), h = x.size(2), w = x.size(3);
  int64_t oh = at::native::pooling_output_shape<int64_t>(h, a.kh, a.ph, a.sh, 1, ceil);
  int64_t ow = at::native::pooling_output_shape<int64_t>(w, a.kw, a.pw, a.sw, 1, ceil);
  NEED(oh > 0 && ow > 0, "empty pooling output");
  Tensor out = dense4(empty_dev({n, c, oh, ow}, at::kFloat, is_cl(x)));
  OmtAct ax = act(x), ay = act(out);
  check(omt_avgpool_fwd(&ax, &ay, (int)n, (int)c, (int)h, (int)w, (int)oh, (int)ow, &a, include_pad, (int)divisor.value_or(0), cur_stream()),
        "avg pool");
  return out;
}
static Tensor avg_pool2d_backward_(const Tensor& gy_, const Tensor& x, IntArrayRef k, IntArrayRef s, IntArrayRef p, bool, bool include_pad,
                                   std::optional<int64_t> divisor) {
  OmtPool a = pool_args(k, s, p, {});
  NEED(pool_ok(x, a) && f32(gy_) && (!divisor || *divisor > 0), "avg pool backward");
  Tensor gy = dense4(gy_);
  int64_t n = x.size(0), c = x.size(1), h = x.size(2), w = x.size(3);
  Tensor gx = dense4(empty_dev(x.sizes(), at::kFloat, is_cl(gy)));
  OmtAct ag = act(gy), agx = act(gx);
  check(omt_avgpool_bwd(&ag, &agx, (int)n, (int)c, (int)h, (int)w, (int)gy.size(2), (int)gy.size(3), &a, include_pad,
                        (int)divisor.value_or(0), cur_stream()),
        "avg pool backward");
  return gx;
}

static Tensor adaptive_avg_pool2d_(const Tensor& x_, IntArrayRef os) {
  NEED(f32(x_) && x_.dim() == 4 && x_.numel() > 0 && os[0] > 0 && os[1] > 0, "adaptive avg pool: 4-D float32");
  Tensor x = dense4(x_);
  Tensor out = dense4(empty_dev({x.size(0), x.size(1), os[0], os[1]}, at::kFloat, is_cl(x) && os[0] * os[1] > 1));
  OmtAct ax = act(x), ay = act(out);
  check(omt_adaptive_avgpool_fwd(&ax, &ay, (int)x.size(0), (int)x.size(1), (int)x.size(2), (int)x.size(3), (int)os[0], (int)os[1], cur_stream()),
        "adaptive avg pool");
  return out;
}
static Tensor adaptive_avg_pool2d_backward_(const Tensor& gy_, const Tensor& x) {
  NEED(f32(x) && f32(gy_) && x.dim() == 4 && x.numel() > 0, "adaptive avg pool backward");
  Tensor gy = dense4(gy_);
  Tensor gx = dense4(empty_dev(x.sizes(), at::kFloat, layout4(x) == 1));
  OmtAct ag = act(gy), agx = act(gx);
  check(omt_adaptive_avgpool_bwd(&ag, &agx, (int)x.size(0), (int)x.size(1), (int)x.size(2), (int)x.size(3), (int)gy.size(2), (int)gy.size(3),
                                 cur_stream()),
        "adaptive avg pool backward");
  return gx;
}

// ------------------------------------------------------------------------------------------------
// random fills: drawn on the host with this device's generator, then uploaded (csrc/nn.cpp:262-273)
// ------------------------------------------------------------------------------------------------

static uint64_t next_seed(const std::optional<at::Generator>& gen) {
  auto* g = generator(gen);
  std::lock_guard<std::mutex> lock(g->mutex_);
  return g->random64();
}
static Tensor& uniform_(Tensor& self, double from, double to, std::optional<at::Generator> gen) {
  at::Generator cpu = at::make_generator<at::CPUGeneratorImpl>(next_seed(gen));
  Tensor h = at::empty(self.sizes(), self.options().device(c10::kCPU)).uniform_(from, to, cpu);
  return self.copy_(h);
}
static Tensor& normal_(Tensor& self, double mean, double std, std::optional<at::Generator> gen) {
  at::Generator cpu = at::make_generator<at::CPUGeneratorImpl>(next_seed(gen));
  Tensor h = at::empty(self.sizes(), self.options().device(c10::kCPU)).normal_(mean, std, cpu);
  return self.copy_(h);
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  OMT_IMPL(m, native_batch_norm, batch_norm_);
  OMT_IMPL(m, native_batch_norm_backward, batch_norm_backward_);
  OMT_IMPL(m, max_pool2d_with_indices, max_pool2d_);
  OMT_IMPL(m, max_pool2d_with_indices_backward, max_pool2d_backward_);
  OMT_IMPL(m, avg_pool2d, avg_pool2d_);
  OMT_IMPL(m, avg_pool2d_backward, avg_pool2d_backward_);
  OMT_IMPL(m, _adaptive_avg_pool2d, adaptive_avg_pool2d_);
  OMT_IMPL(m, _adaptive_avg_pool2d_backward, adaptive_avg_pool2d_backward_);
  OMT_IMPL(m, uniform_, uniform_);
  OMT_IMPL(m, normal_, normal_);
}

}  // namespace omt

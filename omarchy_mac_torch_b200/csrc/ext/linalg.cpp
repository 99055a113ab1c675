// aten::mm and aten::addmm for 2-D float32 tensors on the device: the classifier heads and their gradients run on the same
// tcgen05 3xTF32 kernels as the convolutions (a matrix product is the 1x1 case of the implicit GEMM), through omt_gemm.
// Same op coverage as the reference's csrc/linalg.cpp:62-92 (mm, addmm, bmm); the
// reference's planner callback for generated GEMM kernels (csrc/linalg.cpp:94-96) has no counterpart, set_mm_planner is
// an inert shim in module.cpp.
#include "omt.h"

namespace omt {

// a as omt_gemm takes it: row-major or column-major without a copy, otherwise a row-major copy
static Tensor gemm_operand(const Tensor& t) {
  const int64_t r = t.size(0), c = t.size(1);
  const bool rm = (t.stride(1) == 1 || c == 1) && (t.stride(0) == c || r == 1), cm = (t.stride(0) == 1 || r == 1) && (t.stride(1) == r || c == 1);
  return rm || cm ? t : contig(t);
}
static bool row_major(const Tensor& t) { return (t.stride(1) == 1 || t.size(1) == 1) && (t.stride(0) == t.size(1) || t.size(0) == 1); }

// out = a @ b (+ bias[n]); false when omt_gemm does not take this combination of layouts
static bool gemm_into(const Tensor& a_, const Tensor& b_, const Tensor* bias, Tensor& out) {
  const int64_t M = a_.size(0), K = a_.size(1), N = b_.size(1);
  Tensor a = gemm_operand(a_), b = gemm_operand(b_);
  // strides as the library expects them for each layout (size-1 dimensions leave PyTorch's strides arbitrary)
  const bool arm = row_major(a), brm = row_major(b);
  if (!arm && !brm) a = contig(a);  // A^T * B^T: copy A
  const bool arm2 = row_major(a);
  int st = omt_gemm(a.data_ptr<float>(), arm2 ? K : 1, arm2 ? 1 : M, b.data_ptr<float>(), brm ? N : 1, brm ? 1 : K,
                    bias && !brm ? bias->data_ptr<float>() : nullptr, out.data_ptr<float>(), (int)M, (int)N, (int)K, cur_stream());
  if (st == OMT_EINVAL) return false;
  check(st, "matrix product");
  if (bias && brm) cuda_alias(out).add_(cuda_alias(*bias));  // (bias outside the nn.Linear layout: added separately)
  return true;
}

static Tensor mm_(const Tensor& a, const Tensor& b) {
  NEED(f32(a) && f32(b) && a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(0), "float32 2-D mm");
  NEED(a.numel() > 0 && b.numel() > 0 && a.size(0) < (1ll << 31) && b.size(1) < (1ll << 31) && a.size(1) < (1ll << 31), "empty or oversized operand");
  Tensor out = empty_dev({a.size(0), b.size(1)}, at::kFloat);
  if (!gemm_into(a, b, nullptr, out)) {  // column-major A with column-major B and the like: one operand copied row-major
    Tensor ac = contig(a);
    NEED(gemm_into(ac, b, nullptr, out), "operand layout");
  }
  return out;
}

static Tensor addmm_(const Tensor& bias, const Tensor& a, const Tensor& b, const at::Scalar& beta, const at::Scalar& alpha) {
  NEED(f32(a) && f32(b) && f32(bias) && a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(0), "float32 addmm");
  NEED(a.numel() > 0 && b.numel() > 0 && a.size(0) < (1ll << 31) && b.size(1) < (1ll << 31) && a.size(1) < (1ll << 31), "empty or oversized operand");
  // nn.Linear: bias [N] added in the GEMM epilogue; every other form of addmm goes to the bridge
  NEED(beta.to<double>() == 1 && alpha.to<double>() == 1 && bias.dim() == 1 && bias.size(0) == b.size(1) && bias.is_contiguous(),
       "addmm other than out = bias[N] + a @ b");
  Tensor out = empty_dev({a.size(0), b.size(1)}, at::kFloat);
  if (!gemm_into(a, b, &bias, out)) {
    Tensor ac = contig(a);
    NEED(gemm_into(ac, b, &bias, out), "operand layout");
  }
  return out;
}

// batched product (reference csrc/linalg.cpp:81-92, which puts the batch on the dispatch's z dimension): here one GEMM
// launch per matrix of the batch; batches of many small matrices are better served by ATen's batched kernel and stay
// with the bridge
static Tensor bmm_(const Tensor& a, const Tensor& b) {
  NEED(f32(a) && f32(b) && a.dim() == 3 && b.dim() == 3 && a.size(0) == b.size(0) && a.size(2) == b.size(1), "float32 3-D bmm");
  NEED(a.numel() > 0 && b.numel() > 0 && a.size(0) <= 64 && a.size(1) * b.size(2) >= 128 * 128, "empty operands, or a batch of many small matrices");
  Tensor out = empty_dev({a.size(0), a.size(1), b.size(2)}, at::kFloat);
  for (int64_t i = 0; i < a.size(0); i++) {
    Tensor ai = a.select(0, i), bi = b.select(0, i), oi = out.select(0, i);
    if (!gemm_into(ai, bi, nullptr, oi)) {
      Tensor ac = contig(ai);
      NEED(gemm_into(ac, bi, nullptr, oi), "operand layout");
    }
  }
  return out;
}

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  OMT_IMPL(m, bmm, bmm_);
  OMT_IMPL(m, mm, mm_);
  OMT_IMPL(m, addmm, addmm_);
}

}  // namespace omt

// Fused pointwise chains: one kernel evaluates a short straight-line program (up to 32 instructions over up to 6 input
// tensors, scalars as literals) per output element, so a chain of elementwise ops reads each input once and writes one
// output instead of one round trip through HBM per op.
//
// This is the device half of compile pass 4. The reference generates WGSL source per chain at run time and registers it
// with its runtime (omarchy_mac_torch/compile.py:256-336, csrc/fused.cpp:139-170); kernels here are compiled ahead of
// time, so the chain arrives as a program for a fixed interpreter kernel instead. The interpreter keeps its values in
// shared memory, one column per thread (dynamic register indices would go to local memory), and every thread runs the
// same instruction stream, so decoding is uniform across the block.
#include "common.cuh"

namespace omt {

constexpr int PW_THREADS = 256;
constexpr int PW_VALUES = OMT_PW_MAX_INPUTS + OMT_PW_MAX_INSTR;  // value slots: inputs first, then one per instruction

struct PwArgs {
  OmtPwProgram prog;
  const float* in[OMT_PW_MAX_INPUTS];
  int64_t stride[OMT_PW_MAX_INPUTS][8];  // element strides per output dimension (0 where the input broadcasts)
  int64_t ostride[8];
  int32_t shape[8];
  int32_t rank, n_in;
  uint32_t same;  // bit k: input k has exactly the output's strides (offset = the output's)
  int32_t out_dense;  // the output's strides are those of a dense tensor enumerated in memory order: offset = linear index
  int64_t numel;
  float* out;
};

__device__ __forceinline__ float pw_powf(float x, float p) {  // aten.pow.Tensor_Scalar for the exponents a chain carries
  if (p == 2.f) return x * x;
  if (p == 1.f) return x;
  if (p == 0.5f) return sqrtf(x);
  if (p == 0.f) return 1.f;
  return powf(x, p);
}

__device__ __forceinline__ float pw_eval(int op, float a, float b, float c) {
  switch (op) {
    case OMT_PW_ADD: return a + c * b;            // a + alpha * b
    case OMT_PW_SUB: return a - c * b;
    case OMT_PW_RSUB: return b - c * a;           // rsub(a, b, alpha) = b - alpha * a
    case OMT_PW_MUL: return a * b;
    case OMT_PW_DIV: return a / b;
    case OMT_PW_NEG: return -a;
    case OMT_PW_RELU: return fmaxf(a, 0.f);
    case OMT_PW_EXP: return expf(a);
    case OMT_PW_LOG: return logf(a);
    case OMT_PW_SQRT: return sqrtf(a);
    case OMT_PW_RSQRT: return rsqrtf(a);
    case OMT_PW_RECIP: return 1.f / a;
    case OMT_PW_ABS: return fabsf(a);
    case OMT_PW_TANH: return tanhf(a);
    case OMT_PW_SIGMOID: return 1.f / (1.f + expf(-a));
    case OMT_PW_SILU: return a / (1.f + expf(-a));
    case OMT_PW_MAX: return (a != a || b != b) ? a + b : fmaxf(a, b);  // NaN propagates like aten.maximum
    case OMT_PW_MIN: return (a != a || b != b) ? a + b : fminf(a, b);
    case OMT_PW_POW: return pw_powf(a, b);
    case OMT_PW_THRESHOLD_BWD: return b > c ? a : 0.f;                 // threshold_backward(grad, self, threshold)
    case OMT_PW_SIGMOID_BWD: return a * b * (1.f - b);                 // (grad, output)
    case OMT_PW_TANH_BWD: return a * (1.f - b * b);
    case OMT_PW_SILU_BWD: { const float s = 1.f / (1.f + expf(-b)); return a * s * (1.f + b * (1.f - s)); }
    case OMT_PW_GELU: return 0.5f * a * (1.f + erff(a * 0.70710678118654752f));
    case OMT_PW_GELU_TANH: { const float k = 0.7978845608028654f * (a + 0.044715f * a * a * a); return 0.5f * a * (1.f + tanhf(k)); }
    case OMT_PW_GELU_BWD: return a * (0.5f * (1.f + erff(b * 0.70710678118654752f)) + b * 0.3989422804014327f * expf(-0.5f * b * b));
    case OMT_PW_GELU_TANH_BWD: {
      const float k = 0.7978845608028654f * (b + 0.044715f * b * b * b), t = tanhf(k);
      return a * (0.5f * (1.f + t) + 0.5f * b * (1.f - t * t) * 0.7978845608028654f * (1.f + 0.134145f * b * b));
    }
    case OMT_PW_CLAMP: return fminf(fmaxf(a, b), c);                   // (x, lo, hi); NaN x stays NaN: fmaxf/fminf return the other operand
    case OMT_PW_HARDSWISH: return a * fminf(fmaxf(a + 3.f, 0.f), 6.f) * (1.f / 6.f);
    case OMT_PW_HARDSWISH_BWD: return b < -3.f ? 0.f : (b <= 3.f ? a * (b * (1.f / 3.f) + 0.5f) : a);  // (grad, self)
    case OMT_PW_HARDSIGMOID: return fminf(fmaxf(a + 3.f, 0.f), 6.f) * (1.f / 6.f);
    case OMT_PW_HARDSIGMOID_BWD: return (b > -3.f && b < 3.f) ? a * (1.f / 6.f) : 0.f;
    default: return a;
  }
}

__global__ void __launch_bounds__(PW_THREADS) pointwise_kernel(const __grid_constant__ PwArgs a) {
  __shared__ float val[PW_VALUES][PW_THREADS];
  const int tid = threadIdx.x;
  const int64_t i = (int64_t)blockIdx.x * PW_THREADS + tid;
  if (i >= a.numel) return;
  // offset of output element i (linear over the logical shape) and of each input
  int64_t oo = 0, off[OMT_PW_MAX_INPUTS];
#pragma unroll
  for (int k = 0; k < OMT_PW_MAX_INPUTS; k++) off[k] = 0;
  const bool all_same = a.out_dense && a.same == (1u << a.n_in) - 1u;
  if (all_same) {
    oo = i;  // every tensor has the output's dense layout: walk memory linearly
#pragma unroll
    for (int k = 0; k < OMT_PW_MAX_INPUTS; k++) off[k] = i;
  } else {
    int64_t rem = i;
    for (int d = a.rank - 1; d >= 0; d--) {
      const int64_t c = rem % a.shape[d];
      rem /= a.shape[d];
      oo += c * a.ostride[d];
#pragma unroll
      for (int k = 0; k < OMT_PW_MAX_INPUTS; k++)
        if (k < a.n_in) off[k] += c * a.stride[k][d];
    }
  }
#pragma unroll
  for (int k = 0; k < OMT_PW_MAX_INPUTS; k++)
    if (k < a.n_in) val[k][tid] = __ldg(a.in[k] + off[k]);
  float r = 0.f;
  for (int j = 0; j < a.prog.n_instr; j++) {
    const OmtPwInstr ins = a.prog.instr[j];
    float v[3];
#pragma unroll
    for (int q = 0; q < 3; q++) {
      const int32_t o = q == 0 ? ins.a : (q == 1 ? ins.b : ins.c);
      v[q] = o >= 0 ? val[o][tid] : a.prog.literal[-1 - o];  // >= 0: a value slot; < 0: literal number -1 - o
    }
    r = pw_eval(ins.op, v[0], v[1], v[2]);
    val[OMT_PW_MAX_INPUTS + j][tid] = r;
  }
  a.out[oo] = r;
}

}  // namespace omt

using namespace omt;

extern "C" int omt_pointwise(const OmtPwProgram* prog, int32_t n_inputs, const float* const* inputs, const int64_t* in_strides,
                             const int64_t* out_strides, const int32_t* shape, int32_t rank, float* out, omt_stream_t stream) {
  OMT_REQUIRE(prog && inputs && in_strides && out_strides && shape && out, "omt_pointwise: null pointer");
  OMT_REQUIRE(n_inputs >= 1 && n_inputs <= OMT_PW_MAX_INPUTS && rank >= 0 && rank <= 8, "omt_pointwise: 1..%d inputs, rank <= 8", OMT_PW_MAX_INPUTS);
  OMT_REQUIRE(prog->n_instr >= 1 && prog->n_instr <= OMT_PW_MAX_INSTR, "omt_pointwise: 1..%d instructions", OMT_PW_MAX_INSTR);
  for (int j = 0; j < prog->n_instr; j++) {
    const OmtPwInstr& ins = prog->instr[j];
    OMT_REQUIRE(ins.op >= 0 && ins.op < OMT_PW_OP_COUNT, "omt_pointwise: unknown op %d in instruction %d", ins.op, j);
    for (int32_t o : {ins.a, ins.b, ins.c}) {
      const bool slot = o >= 0 && (o < n_inputs || (o >= OMT_PW_MAX_INPUTS && o < OMT_PW_MAX_INPUTS + j));
      OMT_REQUIRE(slot || (o < 0 && -1 - o < OMT_PW_MAX_LITERALS), "omt_pointwise: instruction %d reads operand %d, which is not defined before it", j, o);
    }
  }
  PwArgs a{};
  a.prog = *prog; a.rank = rank; a.n_in = n_inputs; a.out = out; a.numel = 1;
  for (int d = 0; d < rank; d++) {
    OMT_REQUIRE(shape[d] > 0, "omt_pointwise: empty dimension");
    a.shape[d] = shape[d]; a.ostride[d] = out_strides[d]; a.numel *= shape[d];
  }
  // dense output enumerated in memory order when its strides are the contiguous ones; a permuted dense layout (channels-last)
  // is walked linearly too when every input shares it: then the logical index does not matter, each offset equals i
  bool contiguous = true;
  int64_t expect = 1;
  for (int d = rank - 1; d >= 0; d--) {
    if (shape[d] != 1 && out_strides[d] != expect) contiguous = false;
    expect *= shape[d];
  }
  // a permuted dense layout: the sorted strides multiply up without gaps
  bool dense = contiguous;
  if (!dense) {
    int order[8];
    for (int d = 0; d < rank; d++) order[d] = d;
    for (int x = 0; x < rank; x++)
      for (int y = x + 1; y < rank; y++)
        if (out_strides[order[y]] < out_strides[order[x]]) { int t = order[x]; order[x] = order[y]; order[y] = t; }
    dense = true;
    int64_t e = 1;
    for (int x = 0; x < rank; x++) {
      const int d = order[x];
      if (shape[d] == 1) continue;
      if (out_strides[d] != e) { dense = false; break; }
      e *= shape[d];
    }
  }
  a.out_dense = dense ? 1 : 0;
  for (int k = 0; k < n_inputs; k++) {
    OMT_REQUIRE(inputs[k], "omt_pointwise: null input %d", k);
    a.in[k] = inputs[k];
    bool same = true;
    for (int d = 0; d < rank; d++) {
      a.stride[k][d] = in_strides[k * 8 + d];
      if (shape[d] != 1 && a.stride[k][d] != a.ostride[d]) same = false;
    }
    if (same) a.same |= 1u << k;
  }
  pointwise_kernel<<<(unsigned)cdiv(a.numel, PW_THREADS), PW_THREADS, 0, st(stream)>>>(a);
  return check_launch("pointwise_program");
}

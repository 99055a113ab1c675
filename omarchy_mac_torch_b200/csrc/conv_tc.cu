// Tensor-core (tcgen05 / TMEM / TMA) implicit-GEMM convolution. Placeholder until the kernels land: reports every
// geometry as unsupported so the exact-fp32 CUDA-core path serves it.
#include "common.cuh"

namespace omt {
bool tc_supported(int, const OmtConvGeo*, const OmtAct*, const OmtAct*) { return false; }
size_t tc_workspace(int, const OmtConvGeo*) { return 0; }
int tc_conv_fwd(const OmtConvGeo*, const OmtAct*, const float*, const float*, const OmtAct*, float*, uint32_t, void*, cudaStream_t) {
  set_error("tensor-core path not built");
  return OMT_EINVAL;
}
int tc_conv_dgrad(const OmtConvGeo*, const OmtAct*, const float*, const OmtAct*, void*, cudaStream_t) {
  set_error("tensor-core path not built");
  return OMT_EINVAL;
}
int tc_conv_wgrad(const OmtConvGeo*, const OmtAct*, const OmtAct*, float*, float, void*, cudaStream_t) {
  set_error("tensor-core path not built");
  return OMT_EINVAL;
}
}  // namespace omt

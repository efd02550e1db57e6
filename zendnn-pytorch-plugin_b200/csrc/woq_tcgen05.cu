#include "woq.cuh"
namespace zt {
bool woq_tcgen05_supported(const zt_woq_linear_args_t &) { return false; }
int woq_tcgen05_launch(const zt_woq_linear_args_t &, cudaStream_t) {
  set_error("woq tcgen05 kernel not built");
  return ZT_UNSUPPORTED;
}
}  // namespace zt

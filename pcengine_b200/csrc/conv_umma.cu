// tcgen05 / tensor-memory fused gather-matmul-scatter (placeholder until the
// kernel lands: reports "unsupported" so the dispatcher keeps to CUDA cores).
#include "common.cuh"

namespace pce {
bool conv_umma_supported(int, int, int) { return false; }
int conv_umma(const void*, const void*, const uint32_t*, const int*, const int*, int, int, int, int, void*,
              const pce_epilogue*, cudaStream_t) {
  return PCE_ERR_UNSUPPORTED;
}
}  // namespace pce

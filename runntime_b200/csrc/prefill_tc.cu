// Tensor-core prefill (placeholder until the tcgen05 kernel lands): no shape is
// routed here yet, so every prefill takes the FP32-pipe kernel.
#include "common.cuh"

namespace rt {

bool prefill_tc_supported(const AttnParams&, int) { return false; }

cudaError_t launch_prefill_tc(const AttnParams&, int, int*, cudaStream_t, std::string* err) {
  *err = "tensor-core prefill is not built";
  return cudaErrorNotSupported;
}

}  // namespace rt

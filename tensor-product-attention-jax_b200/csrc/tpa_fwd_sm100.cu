// Placeholder until the tcgen05 kernel lands: nothing is routed here.
#include "tpa_common.cuh"

namespace tpa {
bool sm100_supported(const Params&) { return false; }
size_t sm100_workspace_bytes(const Params&) { return 0; }
cudaError_t launch_sm100(const Params&, void*, TpaKernelInfo*, bool, cudaStream_t) {
  return cudaErrorNotSupported;
}
}  // namespace tpa

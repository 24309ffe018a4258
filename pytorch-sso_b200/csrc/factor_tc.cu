// Kronecker-factor construction on the 5th-generation tensor cores (tcgen05, TMEM accumulators).
// Placeholder until the tcgen05 kernel is validated on hardware: reports "unsupported", so the
// dispatcher in api.cu uses the fp32 SIMT kernel.
#include "common.cuh"
#include "factor_params.cuh"

namespace sso {

size_t factor_tc_workspace_bytes(int64_t, int64_t) { return 0; }
bool factor_tc_supported(const FactorParams&, int) { return false; }
int factor_tc_launch(FactorParams, int, void*, size_t, cudaStream_t) {
  return fail(-4, "tcgen05 factor path not built");
}

}  // namespace sso

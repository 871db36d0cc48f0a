// Tensor-core (tcgen05 + TMEM + TMA) fused neighborhood attention for sm_100a.
#include "fna_sm100.cuh"

namespace nb {

bool sm100_forward_supported(const Geo&, int) { return false; }
bool sm100_backward_supported(const Geo&, int) { return false; }
const char* sm100_unsupported_reason(const Geo&, int) { return "tensor-core kernels are not built yet"; }
int run_fused_forward_sm100(const Geo&, int, const FusedArgs&, cudaStream_t) {
  return set_error(NATTEN_B200_EINVAL, "tensor-core forward is not available");
}
int run_fused_backward_sm100(const Geo&, int, const FusedArgs&, cudaStream_t) {
  return set_error(NATTEN_B200_EINVAL, "tensor-core backward is not available");
}
size_t fused_backward_scratch_sm100(const Geo&, int) { return 0; }

}  // namespace nb

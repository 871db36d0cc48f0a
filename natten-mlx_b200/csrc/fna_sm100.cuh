// Tensor-core (tcgen05 + TMEM + TMA) fused neighborhood attention for sm_100a.
#pragma once

#include "launch.cuh"

namespace nb {

// Whether the tensor-core kernels cover this geometry and dtype.
bool sm100_forward_supported(const Geo& g, int dtype);
bool sm100_backward_supported(const Geo& g, int dtype);
// Human-readable reason when they do not.
const char* sm100_unsupported_reason(const Geo& g, int dtype);

int run_fused_forward_sm100(const Geo& g, int dtype, const FusedArgs& a, cudaStream_t s);
int run_fused_backward_sm100(const Geo& g, int dtype, const FusedArgs& a, cudaStream_t s);
size_t fused_backward_scratch_sm100(const Geo& g, int dtype);

}  // namespace nb

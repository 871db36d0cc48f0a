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

// 1 when a tensor-core kernel on the current device gave up on a wait since
// the last call (synchronises with the device and clears the flag).
int sm100_read_status();
// Device address of the status word of the current device (nullptr without a device).
int* sm100_status_word();
// Diagnostic builds (-DNB_SM100_PROFILE): buffer that receives the kernels' cycle counters.
void sm100_set_profile_buffer(float* ptr);
// Text description of the tiling chosen for a geometry (no GPU needed).
// mode: 0 forward, 1 dQ kernel, 2 dK/dV kernel.
int sm100_describe_plan(const Geo& g, int dtype, int mode, char* buf, size_t cap);
int sm100_plan_hint(const Geo& g, int dtype, int mode, const int tile[3], int max_cols);

}  // namespace nb

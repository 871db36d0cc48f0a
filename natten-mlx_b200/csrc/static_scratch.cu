// Fused backward for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at the point where the
// backward runs: code inside a region where the allocator is frozen (a
// captured or replayed execution plan, a real-time serving loop with a fixed
// memory budget, a plugin sandbox that only hands out pre-registered buffers).
// For them this entry point keeps the backward's scratch (the per-row delta
// vector, and the extra-token accumulators when there are extra tokens) in a
// fixed array that is part of the library image: every GPU that loads the
// library holds kStaticScratchBytes of it until the process exits.
#include <mutex>

#include "launch.cuh"

namespace nb {
namespace {

constexpr size_t kStaticScratchBytes = 4u << 20;   // 4 MiB: up to 1,048,576 (query, head) rows

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of the array on the current device.  In host code the array's
// name is only a handle; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
int static_scratch_ptr(void** out) {
  static void* ptrs[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    (void)cudaGetLastError();
    return set_error(NATTEN_B200_ENODEVICE, "static scratch: no current CUDA device");
  }
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      return set_error(NATTEN_B200_ELAUNCH, "static scratch: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    }
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return NATTEN_B200_OK;
}

}  // namespace
}  // namespace nb

extern "C" {

size_t natten_b200_static_scratch_capacity(void) { return nb::kStaticScratchBytes; }

int natten_b200_fused_backward_static_scratch(const natten_b200_geom* g, const void* q, const void* k, const void* v,
                                              const void* k_extra, const void* v_extra, const void* out,
                                              const float* lse, const void* dout, const float* dlse, void* dq,
                                              void* dk, void* dv, void* dk_extra, void* dv_extra, void* stream) {
  const size_t need = natten_b200_fused_backward_scratch_bytes(g);
  if (need > nb::kStaticScratchBytes)
    return nb::set_error(NATTEN_B200_ERESOURCE,
                         "fused_backward_static_scratch: this geometry needs %zu bytes of scratch, the built-in "
                         "array holds %zu; use natten_b200_fused_backward with a caller-provided buffer",
                         need, nb::kStaticScratchBytes);
  void* scratch = nullptr;
  if (int rc = nb::static_scratch_ptr(&scratch)) return rc;
  return natten_b200_fused_backward(g, q, k, v, k_extra, v_extra, out, lse, dout, dlse, dq, dk, dv, dk_extra,
                                    dv_extra, scratch, nb::kStaticScratchBytes, stream);
}

}  // extern "C"

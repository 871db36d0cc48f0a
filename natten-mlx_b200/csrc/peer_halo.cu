// Halo transport over peer memory for volumes sharded along their leading axis: one process per GPU, buffers mapped
// into each other's address space by the caller (CUDA IPC or symmetric memory).  Two kernels: a pitched copy with
// plain 16-byte loads and stores (the destination or the source may be another GPU's memory; the traffic crosses
// NVLink as ordinary memory transactions) and a barrier over per-rank flag words with a bounded wait.
#include <cuda_runtime.h>

#include <cstdint>

#include "fna_sm100.cuh"
#include "launch.cuh"
#include "../../include/natten_b200.h"

namespace nb {
namespace {

constexpr int kMaxPeers = 16;

struct PeerFlags {
  unsigned int* base[kMaxPeers];   // base[p]: rank p's flag block (one word per rank) as mapped in this process
};

// Rows of `w16` 16-byte words; blockIdx.y walks the rows, four transfers in flight per thread.
__global__ void __launch_bounds__(256) k_peer_copy2d(uint4* __restrict__ dst, size_t dpitch16, const uint4* __restrict__ src,
                                                     size_t spitch16, size_t w16, size_t rows) {
  const size_t step = (size_t)gridDim.x * blockDim.x;
  for (size_t r = blockIdx.y; r < rows; r += gridDim.y) {
    uint4* d = dst + r * dpitch16;
    const uint4* s = src + r * spitch16;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * step < w16; i += 4 * step) {
      uint4 v0 = s[i], v1 = s[i + step], v2 = s[i + 2 * step], v3 = s[i + 3 * step];
      d[i] = v0; d[i + step] = v1; d[i + 2 * step] = v2; d[i + 3 * step] = v3;
    }
    for (; i < w16; i += step) d[i] = s[i];
  }
}

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Thread p announces this rank's arrival at `epoch` in rank p's block and waits for rank p's arrival in its own.
// Everything this GPU wrote before the launch (earlier kernels of the stream) is visible to a peer that has seen
// the flag.  A wait that outlasts `timeout_ns` records status 2 and returns: nothing spins without a limit.
__global__ void k_peer_barrier(PeerFlags f, int world, int rank, unsigned int epoch, unsigned long long timeout_ns, int* status) {
  const int p = threadIdx.x;
  if (p >= world || p == rank) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f.base[p] + rank), "r"(epoch) : "memory");
  const unsigned int* mine = f.base[rank] + p;
  const unsigned long long t0 = now_ns();
  unsigned int spins = 0;
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int)(v - epoch) >= 0) break;
    if ((++spins & 63u) == 0) {
      if (now_ns() - t0 > timeout_ns) {
        if (status != nullptr) atomicExch(status, 2);
        break;
      }
      __nanosleep(200);
    }
  }
  __threadfence_system();
}

}  // namespace
}  // namespace nb

extern "C" {

int natten_b200_peer_copy2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes, size_t rows,
                            void* stream) {
  using namespace nb;
  if (width_bytes == 0 || rows == 0) return NATTEN_B200_OK;
  if (dst == nullptr || src == nullptr) return set_error(NATTEN_B200_EINVAL, "peer copy: null pointer");
  if (((uintptr_t)dst | (uintptr_t)src | dst_pitch | src_pitch | width_bytes) & 15)
    return set_error(NATTEN_B200_EINVAL, "peer copy: addresses, pitches and width must be multiples of 16 bytes");
  if (rows > 1 && (dst_pitch < width_bytes || src_pitch < width_bytes))
    return set_error(NATTEN_B200_EINVAL, "peer copy: a pitch is smaller than the width");
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) != cudaSuccess) return set_error(NATTEN_B200_ENODEVICE, "no CUDA device");
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const size_t w16 = width_bytes / 16;
  const unsigned gy = (unsigned)(rows < 8 ? rows : 8);
  size_t gx = (w16 + 256 * 4 - 1) / (256 * 4);
  const size_t cap = (size_t)sms * 8 / gy > 0 ? (size_t)sms * 8 / gy : 1;
  if (gx > cap) gx = cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  NB_LAUNCH("peer_copy2d", s,
            k_peer_copy2d<<<dim3((unsigned)gx, gy), 256, 0, s>>>(static_cast<uint4*>(dst), dst_pitch / 16,
                                                                 static_cast<const uint4*>(src), src_pitch / 16, w16, rows));
  return check_launch("peer_copy2d");
}

int natten_b200_peer_copy2d_dma(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                                size_t rows, void* stream) {
  using namespace nb;
  if (width_bytes == 0 || rows == 0) return NATTEN_B200_OK;
  if (dst == nullptr || src == nullptr) return set_error(NATTEN_B200_EINVAL, "peer copy: null pointer");
  if (rows > 1 && (dst_pitch < width_bytes || src_pitch < width_bytes))
    return set_error(NATTEN_B200_EINVAL, "peer copy: a pitch is smaller than the width");
  const cudaError_t e = cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDefault,
                                          static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return set_error(NATTEN_B200_ELAUNCH, "peer copy (copy engine): %s", cudaGetErrorString(e));
  return NATTEN_B200_OK;
}

int natten_b200_peer_barrier(const uint64_t* flag_blocks, int32_t world, int32_t rank, uint32_t epoch, uint32_t timeout_ms,
                             void* stream) {
  using namespace nb;
  if (flag_blocks == nullptr || world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    return set_error(NATTEN_B200_EINVAL, "peer barrier: world must be 1..%d and rank inside it", kMaxPeers);
  if (world == 1) return NATTEN_B200_OK;
  PeerFlags f{};
  for (int p = 0; p < world; ++p) {
    if (flag_blocks[p] == 0 || (flag_blocks[p] & 3)) return set_error(NATTEN_B200_EINVAL, "peer barrier: bad flag block of rank %d", p);
    f.base[p] = reinterpret_cast<unsigned int*>(static_cast<uintptr_t>(flag_blocks[p]));
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned long long ns = (unsigned long long)(timeout_ms == 0 ? 10000u : timeout_ms) * 1000000ull;
  NB_LAUNCH("peer_barrier", s, k_peer_barrier<<<1, 32, 0, s>>>(f, world, rank, epoch, ns, sm100_status_word()));
  return check_launch("peer_barrier");
}

}  // extern "C"

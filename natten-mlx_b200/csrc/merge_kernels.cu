// Pairwise merge of two attention results that share queries, and its
// gradient (src/natten_mlx/merge.py:56-68).  With s = sigmoid(l1 - l0):
//   out = o0 - s * (o0 - o1),   lse = l0 - logsigmoid(l0 - l1) = logaddexp(l0, l1)
//   do0 = (1 - s) dout,  do1 = s dout,  t = s (1 - s) * sum_d dout (o1 - o0)
//   dl0 = (1 - s) dlse - t,  dl1 = s dlse + t
// All arithmetic is float32 whatever the storage type.
#include <math.h>

#include "launch.cuh"

namespace nb {
namespace {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float logaddexpf_(float a, float b) {
  const float m = fmaxf(a, b);
  if (m == -INFINITY) return -INFINITY;
  return m + log1pf(expf(-fabsf(a - b)));
}

template <typename T>
__global__ void __launch_bounds__(256)
k_merge_fwd(long long rows, int D, const T* __restrict__ o0, const float* __restrict__ l0,
            const T* __restrict__ o1, const float* __restrict__ l1, T* __restrict__ out,
            float* __restrict__ lse) {
  const long long total = rows * D;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / D;
    const float a = l0[r], b = l1[r];
    const float s = sigmoidf_(b - a);
    const float x0 = to_f<T>(o0[i]), x1 = to_f<T>(o1[i]);
    out[i] = from_f<T>(x0 - s * (x0 - x1));
    if (i % D == 0) lse[r] = logaddexpf_(a, b);
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
k_merge_bwd(long long rows, int D, const T* __restrict__ o0, const float* __restrict__ l0,
            const T* __restrict__ o1, const float* __restrict__ l1, const T* __restrict__ dout,
            const float* __restrict__ dlse, T* __restrict__ do0, float* __restrict__ dl0,
            T* __restrict__ do1, float* __restrict__ dl1) {
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x >> 5;
  for (long long r = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); r < rows;
       r += (long long)gridDim.x * wpb) {
    const float s = sigmoidf_(l1[r] - l0[r]);
    float part = 0.f;
    for (int d = lane; d < D; d += 32) {
      const long long i = r * D + d;
      const float g = to_f<T>(dout[i]);
      part = fmaf(g, to_f<T>(o1[i]) - to_f<T>(o0[i]), part);
      do0[i] = from_f<T>((1.f - s) * g);
      do1[i] = from_f<T>(s * g);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (lane == 0) {
      const float t = s * (1.f - s) * part;
      const float gl = dlse != nullptr ? dlse[r] : 0.f;
      dl0[r] = (1.f - s) * gl - t;
      dl1[r] = s * gl + t;
    }
  }
}

template <typename T>
int fwd(long long rows, int D, const void* o0, const float* l0, const void* o1, const float* l1,
        void* out, float* lse, cudaStream_t s) {
  long long blocks = (rows * D + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (blocks < 1) blocks = 1;
  NB_LAUNCH("merge_fwd", s, k_merge_fwd<T><<<(int)blocks, 256, 0, s>>>(rows, D, (const T*)o0, l0, (const T*)o1, l1, (T*)out, lse));
  return check_launch("merge forward");
}

template <typename T>
int bwd(long long rows, int D, const void* o0, const float* l0, const void* o1, const float* l1,
        const void* dout, const float* dlse, void* do0, float* dl0, void* do1, float* dl1,
        cudaStream_t s) {
  long long blocks = (rows + 3) / 4;
  if (blocks > 148 * 64) blocks = 148 * 64;
  if (blocks < 1) blocks = 1;
  NB_LAUNCH("merge_bwd", s, k_merge_bwd<T><<<(int)blocks, 128, 0, s>>>(rows, D, (const T*)o0, l0, (const T*)o1, l1,
                                              (const T*)dout, dlse, (T*)do0, dl0, (T*)do1, dl1));
  return check_launch("merge backward");
}

}  // namespace

int run_merge_forward(int dtype, long long rows, int D, const void* o0, const float* l0,
                      const void* o1, const float* l1, void* out, float* lse, cudaStream_t s) {
  switch (dtype) {
    case NATTEN_B200_F32: return fwd<float>(rows, D, o0, l0, o1, l1, out, lse, s);
    case NATTEN_B200_F16: return fwd<__half>(rows, D, o0, l0, o1, l1, out, lse, s);
    case NATTEN_B200_BF16: return fwd<__nv_bfloat16>(rows, D, o0, l0, o1, l1, out, lse, s);
  }
  return set_error(NATTEN_B200_EINVAL, "unsupported dtype %d", dtype);
}

int run_merge_backward(int dtype, long long rows, int D, const void* o0, const float* l0,
                       const void* o1, const float* l1, const void* dout, const float* dlse,
                       void* do0, float* dl0, void* do1, float* dl1, cudaStream_t s) {
  switch (dtype) {
    case NATTEN_B200_F32: return bwd<float>(rows, D, o0, l0, o1, l1, dout, dlse, do0, dl0, do1, dl1, s);
    case NATTEN_B200_F16: return bwd<__half>(rows, D, o0, l0, o1, l1, dout, dlse, do0, dl0, do1, dl1, s);
    case NATTEN_B200_BF16: return bwd<__nv_bfloat16>(rows, D, o0, l0, o1, l1, dout, dlse, do0, dl0, do1, dl1, s);
  }
  return set_error(NATTEN_B200_EINVAL, "unsupported dtype %d", dtype);
}

}  // namespace nb

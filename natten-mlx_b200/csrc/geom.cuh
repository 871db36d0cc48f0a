// Geometry shared by every kernel: window arithmetic, the normalised
// three-axis problem description and small dtype helpers.
//
// The window arithmetic restates src/natten_mlx/utils/window.py:8-62 and the
// per-axis validity rule of src/natten_mlx/_core/pure.py:52-73; it is compiled
// for host and device so that the integer tables can be checked without a GPU.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/natten_b200.h"

namespace nb {

#define NB_HD __host__ __device__ __forceinline__

NB_HD int imin(int a, int b) { return a < b ? a : b; }
NB_HD int imax(int a, int b) { return a > b ? a : b; }

// First key coordinate of a non-causal window (src/natten_mlx/utils/window.py:8-34).
NB_HD int window_start(int p, int len, int ksize, int dil) {
  const int nh = ksize >> 1;
  if (dil <= 1) {
    int s = imax(p - nh, 0);
    if (p + nh >= len) s += len - p - nh - 1;
    return s;
  }
  if (p - nh * dil < 0) return p % dil;
  if (p + nh * dil >= len) {
    const int r = p % dil;
    const int a = (len / dil) * dil;
    const int b = len - a;
    return (r < b) ? (len - b + r - 2 * nh * dil) : (a + r - ksize * dil);
  }
  return p - nh * dil;
}

// First relative-position-bias slot (src/natten_mlx/utils/window.py:42-62).
NB_HD int pb_start(int p, int len, int ksize, int dil) {
  const int nh = ksize >> 1;
  if (dil <= 1) {
    int v = nh;
    if (p < nh) v += nh - p;
    if (p + nh >= len) v += len - p - 1 - nh;
    return v;
  }
  if (p - nh * dil < 0) return ksize - 1 - (p / dil);
  if (p + nh * dil >= len) return (len - p - 1) / dil;
  return nh;
}

// Window of query coordinate p on one axis: slot s addresses start + s*dil and
// is valid iff 0 <= start + s*dil < hi  (src/natten_mlx/_core/pure.py:62-72).
// causal: 0 = centred (clamped) window, 1 = causal window, 2 = the whole axis
// (ksize == len; what the reference's dense route computes when the kernel
// covers the extent, src/natten_mlx/functional.py:141-187).
NB_HD void axis_window(int p, int len, int ksize, int dil, int causal, int& start, int& hi) {
  if (causal == 2) {
    start = 0;
    hi = len;
  } else if (causal) {
    start = p - (ksize - 1) * dil;
    hi = imin(p + 1, len);
  } else {
    start = window_start(p, len, ksize, dil);
    hi = imin(len, start + ksize * dil);
  }
}

// Problem description normalised to three axes (missing leading axes have
// extent 1, kernel 1).  Passed to kernels by value.
struct Geo {
  int B, Hq, Hkv, rep, D;
  int rank;            // original rank, used to index `extents`
  int qe[3], ke[3], ge[3], qo[3], ko[3];
  int me[3];           // extents that give the memory strides (== ge unless the tensors are corners of larger arrays)
  bool pitched;
  int K[3], st[3], dl[3], ca[3], out[3];
  int kvol, n_extra;
  float scale;
  const int* extents;  // [B, rank] or nullptr
  const int* host_extents;  // host copy of extents (lets the tensor-core kernels take a variable-size batch) or nullptr
  long long n_out;     // out[0]*out[1]*out[2]
  long long n_q;       // qe[0]*qe[1]*qe[2]
  long long n_kv;      // ke[0]*ke[1]*ke[2]
};

// Per-sample global extents (variable-size batches override the global ones).
__device__ __forceinline__ void sample_extent(const Geo& g, int b, int ext[3]) {
  ext[0] = g.ge[0]; ext[1] = g.ge[1]; ext[2] = g.ge[2];
  if (g.extents != nullptr) {
    const int lead = 3 - g.rank;
    for (int a = 0; a < g.rank; ++a) ext[lead + a] = g.extents[b * g.rank + a];
  }
}

// ---------------------------------------------------------------------------
// dtype helpers
// ---------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Number of elements of T in a 16-byte vector.
template <typename T> struct Vec16 { static constexpr int n = 16 / sizeof(T); };

// Load / store `n` (= Vec16<T>::n) consecutive elements through one 16-byte access.
template <typename T>
__device__ __forceinline__ void load16(const T* p, float* out) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec16<T>::n; ++i) out[i] = to_f<T>(e[i]);
}
template <typename T>
__device__ __forceinline__ void store16(T* p, const float* in) {
  uint4 raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int i = 0; i < Vec16<T>::n; ++i) e[i] = from_f<T>(in[i]);
  *reinterpret_cast<uint4*>(p) = raw;
}

// Dot product of two rows of D elements; `vec` says whether rows are 16-byte
// aligned multiples of 16 bytes.
template <typename T>
__device__ __forceinline__ float dot_rows(const T* a, const T* b, int D, bool vec) {
  float acc = 0.f;
  if (vec) {
    constexpr int n = Vec16<T>::n;
    for (int i = 0; i < D; i += n) {
      float x[n], y[n];
      load16<T>(a + i, x);
      load16<T>(b + i, y);
#pragma unroll
      for (int j = 0; j < n; ++j) acc = fmaf(x[j], y[j], acc);
    }
  } else {
    for (int i = 0; i < D; ++i) acc = fmaf(to_f<T>(a[i]), to_f<T>(b[i]), acc);
  }
  return acc;
}

}  // namespace nb

// CUDA-core kernels of the split operators (QK, AV and their gradients).
//
// Three kernel shapes cover all eight operators:
//   pair_dot      one thread per (query, head, slot): dot of a query-side row
//                 with the neighbour row      -> QK forward, AV backward (dattn)
//   weighted_sum  one thread per (query, head, 16-byte chunk): sum over slots
//                 of weight * neighbour row   -> AV forward, QK backward (dq)
//   inverse_sum   one thread per (key, kv head, chunk): sum over every
//                 (query, slot) that addresses the key -> dk, dv
// The arithmetic follows src/natten_mlx/_core/pure.py:258-494 (forward) and the
// autodiff-defined gradients of src/natten_mlx/_core/pure.py:735-808.
#include "launch.cuh"

namespace nb {

struct RowIdx {
  int b, o[3], h;
};

__device__ __forceinline__ RowIdx decode_row(const Geo& g, long long row) {
  RowIdx r;
  r.h = (int)(row % g.Hq); row /= g.Hq;
  r.o[2] = (int)(row % g.out[2]); row /= g.out[2];
  r.o[1] = (int)(row % g.out[1]); row /= g.out[1];
  r.o[0] = (int)(row % g.out[0]); row /= g.out[0];
  r.b = (int)row;
  return r;
}

// Resolves the window of one query row: per-axis start/hi in global
// coordinates; returns false when the query lies outside the sample's extent.
__device__ __forceinline__ bool row_window(const Geo& g, const RowIdx& r, int ext[3], int p[3],
                                           int start[3], int hi[3]) {
  sample_extent(g, r.b, ext);
  bool inside = true;
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    p[a] = g.qo[a] + r.o[a] * g.st[a];
    inside = inside && (p[a] < ext[a]);
    axis_window(p[a], ext[a], g.K[a], g.dl[a], g.ca[a], start[a], hi[a]);
  }
  return inside;
}

// Local linear key index of slot (s0,s1,s2), or -1 when the slot is invalid.
__device__ __forceinline__ long long slot_key(const Geo& g, const int start[3], const int hi[3],
                                              int s0, int s1, int s2) {
  const int x0 = start[0] + s0 * g.dl[0];
  const int x1 = start[1] + s1 * g.dl[1];
  const int x2 = start[2] + s2 * g.dl[2];
  if (x0 < 0 || x0 >= hi[0] || x1 < 0 || x1 >= hi[1] || x2 < 0 || x2 >= hi[2]) return -1;
  return ((long long)(x0 - g.ko[0]) * g.ke[1] + (x1 - g.ko[1])) * g.ke[2] + (x2 - g.ko[2]);
}

// ---------------------------------------------------------------------------
// pair_dot
// ---------------------------------------------------------------------------
// x_out_indexed: the query-side tensor is laid out over output positions
// (a cotangent of `out`) instead of over query positions.
template <typename T>
__global__ void __launch_bounds__(256)
k_pair_dot(Geo g, const T* __restrict__ x, const T* __restrict__ y, const float* __restrict__ bias,
           T* __restrict__ dst, float alpha, float masked_value, int x_out_indexed, int vec) {
  const long long total = (long long)g.B * g.n_out * g.Hq * g.kvol;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int slot = (int)(idx % g.kvol);
    const long long row = idx / g.kvol;
    const RowIdx r = decode_row(g, row);
    int ext[3], p[3], start[3], hi[3];
    const bool inside = row_window(g, r, ext, p, start, hi);
    const int s2 = slot % g.K[2];
    const int s1 = (slot / g.K[2]) % g.K[1];
    const int s0 = slot / (g.K[2] * g.K[1]);
    const long long key = inside ? slot_key(g, start, hi, s0, s1, s2) : -1;
    float val = masked_value;
    if (key >= 0) {
      long long xrow;
      if (x_out_indexed) {
        xrow = row;
      } else {
        const long long ql = ((long long)(r.o[0] * g.st[0]) * g.qe[1] + r.o[1] * g.st[1]) * g.qe[2] + r.o[2] * g.st[2];
        xrow = ((long long)r.b * g.n_q + ql) * g.Hq + r.h;
      }
      const long long yrow = ((long long)r.b * g.n_kv + key) * g.Hkv + r.h / g.rep;
      val = alpha * dot_rows<T>(x + xrow * g.D, y + yrow * g.D, g.D, vec != 0);
      if (bias != nullptr) {
        const int w0 = 2 * g.K[0] - 1, w1 = 2 * g.K[1] - 1, w2 = 2 * g.K[2] - 1;
        const int b0 = pb_start(p[0], ext[0], g.K[0], g.dl[0]) + s0;
        const int b1 = pb_start(p[1], ext[1], g.K[1], g.dl[1]) + s1;
        const int b2 = pb_start(p[2], ext[2], g.K[2], g.dl[2]) + s2;
        val += bias[(long long)r.h * w0 * w1 * w2 + ((long long)b0 * w1 + b1) * w2 + b2];
      }
    } else if (!inside) {
      val = 0.f;  // padded query of a variable-size batch
    }
    dst[idx] = from_f<T>(val);
  }
}

// Accumulates the gradient of the relative position bias.
template <typename T>
__global__ void __launch_bounds__(256)
k_bias_grad(Geo g, const T* __restrict__ dlogits, float* __restrict__ dbias) {
  const long long total = (long long)g.B * g.n_out * g.Hq * g.kvol;
  const int w0 = 2 * g.K[0] - 1, w1 = 2 * g.K[1] - 1, w2 = 2 * g.K[2] - 1;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int slot = (int)(idx % g.kvol);
    const RowIdx r = decode_row(g, idx / g.kvol);
    int ext[3], p[3], start[3], hi[3];
    if (!row_window(g, r, ext, p, start, hi)) continue;
    const int s2 = slot % g.K[2];
    const int s1 = (slot / g.K[2]) % g.K[1];
    const int s0 = slot / (g.K[2] * g.K[1]);
    if (slot_key(g, start, hi, s0, s1, s2) < 0) continue;
    const int b0 = pb_start(p[0], ext[0], g.K[0], g.dl[0]) + s0;
    const int b1 = pb_start(p[1], ext[1], g.K[1], g.dl[1]) + s1;
    const int b2 = pb_start(p[2], ext[2], g.K[2], g.dl[2]) + s2;
    atomicAdd(dbias + (long long)r.h * w0 * w1 * w2 + ((long long)b0 * w1 + b1) * w2 + b2,
              to_f<T>(dlogits[idx]));
  }
}

// ---------------------------------------------------------------------------
// weighted_sum
// ---------------------------------------------------------------------------
// dst_q_indexed: write at the query position inside a q-shaped tensor (dq)
// instead of at the output position.
template <typename T, int CH>
__global__ void __launch_bounds__(256)
k_weighted_sum(Geo g, const T* __restrict__ w, const T* __restrict__ y, T* __restrict__ dst,
               float alpha, int dst_q_indexed) {
  const int chunks = g.D / CH;
  const long long total = (long long)g.B * g.n_out * g.Hq * chunks;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % chunks);
    const long long row = idx / chunks;
    const RowIdx r = decode_row(g, row);
    int ext[3], p[3], start[3], hi[3];
    const bool inside = row_window(g, r, ext, p, start, hi);
    float acc[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) acc[i] = 0.f;
    if (inside) {
      const T* wrow = w + row * g.kvol;
      const long long ybase = (long long)r.b * g.n_kv;
      const int hk = r.h / g.rep;
      int slot = 0;
      for (int s0 = 0; s0 < g.K[0]; ++s0)
        for (int s1 = 0; s1 < g.K[1]; ++s1)
          for (int s2 = 0; s2 < g.K[2]; ++s2, ++slot) {
            const long long key = slot_key(g, start, hi, s0, s1, s2);
            if (key < 0) continue;
            const float wt = to_f<T>(wrow[slot]);
            const T* yp = y + ((ybase + key) * g.Hkv + hk) * g.D + c * CH;
            if (CH == 1) {
              acc[0] = fmaf(wt, to_f<T>(yp[0]), acc[0]);
            } else {
              float v[CH];
              load16<T>(yp, v);
#pragma unroll
              for (int i = 0; i < CH; ++i) acc[i] = fmaf(wt, v[i], acc[i]);
            }
          }
    }
#pragma unroll
    for (int i = 0; i < CH; ++i) acc[i] *= alpha;
    long long drow = row;
    if (dst_q_indexed) {
      const long long ql = ((long long)(r.o[0] * g.st[0]) * g.qe[1] + r.o[1] * g.st[1]) * g.qe[2] + r.o[2] * g.st[2];
      drow = ((long long)r.b * g.n_q + ql) * g.Hq + r.h;
    }
    T* dp = dst + drow * g.D + c * CH;
    if (CH == 1) dp[0] = from_f<T>(acc[0]);
    else store16<T>(dp, acc);
  }
}

// ---------------------------------------------------------------------------
// inverse_sum
// ---------------------------------------------------------------------------
// For key coordinate x on one axis, candidate queries are x + m*dil for
// |m| <= K; a candidate counts when it lies on the stride lattice inside the
// local query slab and its window holds x.  Returns the slot or -1.
__device__ __forceinline__ int inverse_slot(const Geo& g, int a, int ext, int x, int m, int& o) {
  const int p = x + m * g.dl[a];
  if (p < 0 || p >= ext) return -1;
  const int pl = p - g.qo[a];
  if (pl < 0 || pl >= g.qe[a] || (pl % g.st[a]) != 0) return -1;
  o = pl / g.st[a];
  int start, hi;
  axis_window(p, ext, g.K[a], g.dl[a], g.ca[a], start, hi);
  if (x >= hi || x < start) return -1;
  const int s = (x - start) / g.dl[a];
  return (s < g.K[a]) ? s : -1;
}

// src_out_indexed: the query-side rows are laid out over output positions.
template <typename T, int CH>
__global__ void __launch_bounds__(256)
k_inverse_sum(Geo g, const T* __restrict__ w, const T* __restrict__ src, T* __restrict__ dst,
              float alpha, int src_out_indexed) {
  const int chunks = g.D / CH;
  const long long total = (long long)g.B * g.n_kv * g.Hkv * chunks;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % chunks);
    long long t = idx / chunks;
    const int hk = (int)(t % g.Hkv); t /= g.Hkv;
    const int j2 = (int)(t % g.ke[2]); t /= g.ke[2];
    const int j1 = (int)(t % g.ke[1]); t /= g.ke[1];
    const int j0 = (int)(t % g.ke[0]); t /= g.ke[0];
    const int b = (int)t;
    int ext[3];
    sample_extent(g, b, ext);
    const int x0 = g.ko[0] + j0, x1 = g.ko[1] + j1, x2 = g.ko[2] + j2;
    float acc[CH];
#pragma unroll
    for (int i = 0; i < CH; ++i) acc[i] = 0.f;
    if (x0 < ext[0] && x1 < ext[1] && x2 < ext[2]) {
      for (int m0 = -g.K[0]; m0 <= g.K[0]; ++m0) {
        int o0;
        const int s0 = inverse_slot(g, 0, ext[0], x0, m0, o0);
        if (s0 < 0) continue;
        for (int m1 = -g.K[1]; m1 <= g.K[1]; ++m1) {
          int o1;
          const int s1 = inverse_slot(g, 1, ext[1], x1, m1, o1);
          if (s1 < 0) continue;
          for (int m2 = -g.K[2]; m2 <= g.K[2]; ++m2) {
            int o2;
            const int s2 = inverse_slot(g, 2, ext[2], x2, m2, o2);
            if (s2 < 0) continue;
            const int slot = (s0 * g.K[1] + s1) * g.K[2] + s2;
            const long long ol = ((long long)o0 * g.out[1] + o1) * g.out[2] + o2;
            const long long ql = ((long long)(o0 * g.st[0]) * g.qe[1] + o1 * g.st[1]) * g.qe[2] + o2 * g.st[2];
            for (int hh = 0; hh < g.rep; ++hh) {
              const int h = hk * g.rep + hh;
              const long long wrow = ((long long)b * g.n_out + ol) * g.Hq + h;
              const float wt = to_f<T>(w[wrow * g.kvol + slot]);
              const long long srow = src_out_indexed ? wrow : ((long long)b * g.n_q + ql) * g.Hq + h;
              const T* sp = src + srow * g.D + c * CH;
              if (CH == 1) {
                acc[0] = fmaf(wt, to_f<T>(sp[0]), acc[0]);
              } else {
                float v[CH];
                load16<T>(sp, v);
#pragma unroll
                for (int i = 0; i < CH; ++i) acc[i] = fmaf(wt, v[i], acc[i]);
              }
            }
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < CH; ++i) acc[i] *= alpha;
    T* dp = dst + (idx / chunks) * g.D + c * CH;
    if (CH == 1) dp[0] = from_f<T>(acc[0]);
    else store16<T>(dp, acc);
  }
}

// ---------------------------------------------------------------------------
// host launchers
// ---------------------------------------------------------------------------
static int grid_for(long long total, int block) {
  long long blocks = (total + block - 1) / block;
  const long long cap = 148LL * 32;  // grid-stride beyond 32 resident waves of 148 SMs
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

template <typename T>
static int launch_split(SplitOp op, const Geo& g, const void* a, const void* b, const void* c,
                        const float* bias, void* o0, void* o1, float* dbias, cudaStream_t s) {
  const bool vec = (g.D * (int)sizeof(T)) % 16 == 0;
  constexpr int CH = Vec16<T>::n;
  const long long n_logits = (long long)g.B * g.n_out * g.Hq * g.kvol;
  const T* A = static_cast<const T*>(a);
  const T* Bp = static_cast<const T*>(b);
  const T* C = static_cast<const T*>(c);
  const float ninf = -__builtin_huge_valf();
  auto wsum = [&](const T* w, const T* y, T* dst, float alpha, int dst_q) {
    if (vec) {
      const long long total = (long long)g.B * g.n_out * g.Hq * (g.D / CH);
      NB_LAUNCH("weighted_sum", s, k_weighted_sum<T, CH><<<grid_for(total, 256), 256, 0, s>>>(g, w, y, dst, alpha, dst_q));
    } else {
      const long long total = (long long)g.B * g.n_out * g.Hq * g.D;
      NB_LAUNCH("weighted_sum", s, k_weighted_sum<T, 1><<<grid_for(total, 256), 256, 0, s>>>(g, w, y, dst, alpha, dst_q));
    }
  };
  auto isum = [&](const T* w, const T* src, T* dst, float alpha, int src_out) {
    if (vec) {
      const long long total = (long long)g.B * g.n_kv * g.Hkv * (g.D / CH);
      NB_LAUNCH("inverse_sum", s, k_inverse_sum<T, CH><<<grid_for(total, 256), 256, 0, s>>>(g, w, src, dst, alpha, src_out));
    } else {
      const long long total = (long long)g.B * g.n_kv * g.Hkv * g.D;
      NB_LAUNCH("inverse_sum", s, k_inverse_sum<T, 1><<<grid_for(total, 256), 256, 0, s>>>(g, w, src, dst, alpha, src_out));
    }
  };
  switch (op) {
    case SplitOp::QkForward:
      NB_LAUNCH("pair_dot", s, k_pair_dot<T><<<grid_for(n_logits, 256), 256, 0, s>>>(g, A, Bp, bias, static_cast<T*>(o0), g.scale, ninf, 0, vec));
      break;
    case SplitOp::QkBackward: {  // a=q, b=k, c=dlogits -> o0=dq, o1=dk
      const bool strided = g.st[0] * g.st[1] * g.st[2] != 1 || g.n_out != g.n_q;
      if (strided) cudaMemsetAsync(o0, 0, (size_t)g.B * g.n_q * g.Hq * g.D * sizeof(T), s);
      wsum(C, Bp, static_cast<T*>(o0), g.scale, 1);
      isum(C, A, static_cast<T*>(o1), g.scale, 0);
      break;
    }
    case SplitOp::AvForward:  // a=attn, b=v -> o0=out
      wsum(A, Bp, static_cast<T*>(o0), 1.f, 0);
      break;
    case SplitOp::AvBackward:  // a=attn, b=v, c=dout -> o0=dattn, o1=dv
      NB_LAUNCH("pair_dot", s, k_pair_dot<T><<<grid_for(n_logits, 256), 256, 0, s>>>(g, C, Bp, nullptr, static_cast<T*>(o0), 1.f, 0.f, 1, vec));
      isum(A, C, static_cast<T*>(o1), 1.f, 1);
      break;
  }
  return check_launch("split operator");
}

template <typename T>
static void launch_bias_grad(const Geo& g, const void* dlogits, float* dbias, cudaStream_t s) {
  const long long n_logits = (long long)g.B * g.n_out * g.Hq * g.kvol;
  NB_LAUNCH("bias_grad", s, k_bias_grad<T><<<grid_for(n_logits, 256), 256, 0, s>>>(g, static_cast<const T*>(dlogits), dbias));
}

int run_split(SplitOp op, const Geo& g, int dtype, const void* a, const void* b, const void* c,
              const float* bias, void* o0, void* o1, float* dbias, cudaStream_t s) {
  if (op == SplitOp::QkBackward && dbias != nullptr && !run_bias_grad_rows(g, dtype, c, dbias, s)) {
    // a bias table too large for shared memory: one global atomic per logit
    switch (dtype) {
      case NATTEN_B200_F32: launch_bias_grad<float>(g, c, dbias, s); break;
      case NATTEN_B200_F16: launch_bias_grad<__half>(g, c, dbias, s); break;
      case NATTEN_B200_BF16: launch_bias_grad<__nv_bfloat16>(g, c, dbias, s); break;
    }
  }
  if (run_split_rows(op, g, dtype, a, b, c, bias, o0, o1, s)) return check_launch("split operator");
  switch (dtype) {
    case NATTEN_B200_F32: return launch_split<float>(op, g, a, b, c, bias, o0, o1, dbias, s);
    case NATTEN_B200_F16: return launch_split<__half>(op, g, a, b, c, bias, o0, o1, dbias, s);
    case NATTEN_B200_BF16: return launch_split<__nv_bfloat16>(op, g, a, b, c, bias, o0, o1, dbias, s);
  }
  return set_error(NATTEN_B200_EINVAL, "unsupported dtype %d", dtype);
}

}  // namespace nb

// Row-per-thread kernels of the split operators for small head dims.
//
// The generic kernels of split_kernels.cu give one thread to every (query, head, slot) or
// (query, head, 16-byte chunk): at head dims like 12 or 16 most of their instructions decode
// indices, and a query row is fetched once per slot.  Here one thread owns a whole row: it
// decodes its position and window once (32-bit arithmetic), keeps the D values of its row in
// registers (16-byte loads: three float4 per fp32 row of 12), walks the kernel slots and reads
// or writes its K_vol logits as one contiguous run.  The same three shapes cover all eight
// operators:
//   row_dot      QK forward (+ relative position bias), AV backward (dattn)
//   row_wsum     AV forward, QK backward (dq)
//   row_inverse  dk, dv
// and the gradient of the bias is reduced in shared memory before it touches global memory.
// This is the small-head-dim path of the reference's DiNAT-style ops
// (src/natten_mlx/extras/allin1/functional_metal.py:1934-1963, kernels.py:190-234, 273-317:
// rows of float4 x 3, indices worked out once per query); arithmetic as in
// src/natten_mlx/_core/pure.py:258-494 and src/natten_mlx/extras/allin1/__init__.py:40-180.
#include "launch.cuh"

namespace nb {
namespace {

struct Row32 {
  int b, o[3], h;
};

__device__ __forceinline__ Row32 decode_row32(const Geo& g, int row) {
  Row32 r;
  r.h = row % g.Hq; row /= g.Hq;
  r.o[2] = row % g.out[2]; row /= g.out[2];
  r.o[1] = row % g.out[1]; row /= g.out[1];
  r.o[0] = row % g.out[0]; row /= g.out[0];
  r.b = row;
  return r;
}

template <typename T, int D>
__device__ __forceinline__ void load_row(const T* p, float (&out)[D]) {
  constexpr int n = Vec16<T>::n;
#pragma unroll
  for (int i = 0; i < D; i += n) load16<T>(p + i, out + i);
}

template <typename T, int D>
__device__ __forceinline__ void store_row(T* p, const float (&in)[D]) {
  constexpr int n = Vec16<T>::n;
#pragma unroll
  for (int i = 0; i < D; i += n) store16<T>(p + i, in + i);
}

// Window of one row: per-axis start / end, the sample's extents and the query coordinates.
struct RowWin {
  int ext[3], p[3], start[3], hi[3];
  bool inside;
};

__device__ __forceinline__ RowWin row_win(const Geo& g, const Row32& r) {
  RowWin w;
  sample_extent(g, r.b, w.ext);
  w.inside = true;
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    w.p[a] = g.qo[a] + r.o[a] * g.st[a];
    w.inside = w.inside && (w.p[a] < w.ext[a]);
    axis_window(w.p[a], w.ext[a], g.K[a], g.dl[a], g.ca[a], w.start[a], w.hi[a]);
  }
  return w;
}

__device__ __forceinline__ long long q_row_of(const Geo& g, const Row32& r) {
  const long long ql = ((long long)(r.o[0] * g.st[0]) * g.qe[1] + r.o[1] * g.st[1]) * g.qe[2] + r.o[2] * g.st[2];
  return ((long long)r.b * g.n_q + ql) * g.Hq + r.h;
}

// ---------------------------------------------------------------------------
// row_dot: dst[row, slot] = alpha * <x[row], y[key(row, slot)]> (+ bias)
// ---------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(256)
k_row_dot(Geo g, const T* __restrict__ x, const T* __restrict__ y, const float* __restrict__ bias,
          T* __restrict__ dst, float alpha, float masked_value, int x_out_indexed, int n_rows) {
  for (long long row64 = (long long)blockIdx.x * blockDim.x + threadIdx.x; row64 < n_rows; row64 += (long long)gridDim.x * blockDim.x) {
    const int row = (int)row64;
    const Row32 r = decode_row32(g, row);
    const RowWin w = row_win(g, r);
    T* drow = dst + (long long)row * g.kvol;
    if (!w.inside) {   // padded query of a variable-size batch
      for (int s = 0; s < g.kvol; ++s) drow[s] = from_f<T>(0.f);
      continue;
    }
    float xr[D];
    load_row<T, D>(x + (x_out_indexed ? (long long)row : q_row_of(g, r)) * D, xr);
    const long long ybase = (long long)r.b * g.n_kv;
    const int hk = r.h / g.rep;
    int pb[3] = {0, 0, 0};
    long long bias_h = 0;
    const int w1 = 2 * g.K[1] - 1, w2 = 2 * g.K[2] - 1;
    if (bias != nullptr) {
#pragma unroll
      for (int a = 0; a < 3; ++a) pb[a] = pb_start(w.p[a], w.ext[a], g.K[a], g.dl[a]);
      bias_h = (long long)r.h * (2 * g.K[0] - 1) * w1 * w2;
    }
    int slot = 0;
    for (int s0 = 0; s0 < g.K[0]; ++s0) {
      const int x0 = w.start[0] + s0 * g.dl[0];
      const bool v0 = x0 >= 0 && x0 < w.hi[0];
      for (int s1 = 0; s1 < g.K[1]; ++s1) {
        const int x1 = w.start[1] + s1 * g.dl[1];
        const bool v1 = v0 && x1 >= 0 && x1 < w.hi[1];
        const long long k01 = ((long long)(x0 - g.ko[0]) * g.ke[1] + (x1 - g.ko[1])) * g.ke[2] - g.ko[2];
        for (int s2 = 0; s2 < g.K[2]; ++s2, ++slot) {
          const int x2 = w.start[2] + s2 * g.dl[2];
          float val = masked_value;
          if (v1 && x2 >= 0 && x2 < w.hi[2]) {
            float yr[D];
            load_row<T, D>(y + ((ybase + k01 + x2) * g.Hkv + hk) * D, yr);
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < D; ++i) acc = fmaf(xr[i], yr[i], acc);
            val = alpha * acc;
            if (bias != nullptr) val += bias[bias_h + ((long long)(pb[0] + s0) * w1 + (pb[1] + s1)) * w2 + (pb[2] + s2)];
          }
          drow[slot] = from_f<T>(val);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------
// row_wsum: dst[row] = alpha * sum_slot w[row, slot] * y[key(row, slot)]
// ---------------------------------------------------------------------------
template <typename T, int D>
__global__ void __launch_bounds__(256)
k_row_wsum(Geo g, const T* __restrict__ wt, const T* __restrict__ y, T* __restrict__ dst, float alpha,
           int dst_q_indexed, int n_rows) {
  for (long long row64 = (long long)blockIdx.x * blockDim.x + threadIdx.x; row64 < n_rows; row64 += (long long)gridDim.x * blockDim.x) {
    const int row = (int)row64;
    const Row32 r = decode_row32(g, row);
    const RowWin w = row_win(g, r);
    float acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) acc[i] = 0.f;
    if (w.inside) {
      const T* wrow = wt + (long long)row * g.kvol;
      const long long ybase = (long long)r.b * g.n_kv;
      const int hk = r.h / g.rep;
      int slot = 0;
      for (int s0 = 0; s0 < g.K[0]; ++s0) {
        const int x0 = w.start[0] + s0 * g.dl[0];
        const bool v0 = x0 >= 0 && x0 < w.hi[0];
        for (int s1 = 0; s1 < g.K[1]; ++s1) {
          const int x1 = w.start[1] + s1 * g.dl[1];
          const bool v1 = v0 && x1 >= 0 && x1 < w.hi[1];
          const long long k01 = ((long long)(x0 - g.ko[0]) * g.ke[1] + (x1 - g.ko[1])) * g.ke[2] - g.ko[2];
          for (int s2 = 0; s2 < g.K[2]; ++s2, ++slot) {
            const int x2 = w.start[2] + s2 * g.dl[2];
            if (!(v1 && x2 >= 0 && x2 < w.hi[2])) continue;
            const float ws = to_f<T>(wrow[slot]);
            float yr[D];
            load_row<T, D>(y + ((ybase + k01 + x2) * g.Hkv + hk) * D, yr);
#pragma unroll
            for (int i = 0; i < D; ++i) acc[i] = fmaf(ws, yr[i], acc[i]);
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < D; ++i) acc[i] *= alpha;
    store_row<T, D>(dst + (dst_q_indexed ? q_row_of(g, r) : (long long)row) * D, acc);
  }
}

// Walks the kernel slots of one row in row-major order (slot = (s0 * K1 + s1) * K2 + s2) and hands out, slot by
// slot, whether the slot is valid and the row of the key it addresses.
struct SlotWalk {
  int s0, s1, s2, slot;
  __device__ __forceinline__ SlotWalk() : s0(0), s1(0), s2(0), slot(0) {}
  __device__ __forceinline__ bool next(const Geo& g, const RowWin& w, long long ybase, long long& key_row) {
    const int x0 = w.start[0] + s0 * g.dl[0], x1 = w.start[1] + s1 * g.dl[1], x2 = w.start[2] + s2 * g.dl[2];
    const bool ok = x0 >= 0 && x0 < w.hi[0] && x1 >= 0 && x1 < w.hi[1] && x2 >= 0 && x2 < w.hi[2];
    key_row = ybase + ((long long)(x0 - g.ko[0]) * g.ke[1] + (x1 - g.ko[1])) * g.ke[2] + (x2 - g.ko[2]);
    ++slot;
    if (++s2 == g.K[2]) {
      s2 = 0;
      if (++s1 == g.K[1]) { s1 = 0; ++s0; }
    }
    return ok;
  }
};

// ---------------------------------------------------------------------------
// row_fused: out[row] = softmax_slot(alpha * <q[row], k[key]> + bias) . v[key]   (forward only)
// ---------------------------------------------------------------------------
// QK + relative position bias, softmax and AV of one (query, head) row in one thread: the logits never reach
// memory.  The softmax runs online over the slots (running maximum m, sum l, output acc), so any kernel volume
// works with the same registers.  The fused path of the reference's DiNAT-style ops
// (src/natten_mlx/extras/allin1/functional_metal.py:2130-2170).
template <typename T, int D>
__global__ void __launch_bounds__(256)
k_row_fused(Geo g, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
            const float* __restrict__ bias, T* __restrict__ out, float* __restrict__ lse, int n_rows) {
  constexpr int NB = D <= 16 ? 2 : 1;
  const int w1 = 2 * g.K[1] - 1, w2 = 2 * g.K[2] - 1;
  for (long long row64 = (long long)blockIdx.x * blockDim.x + threadIdx.x; row64 < n_rows; row64 += (long long)gridDim.x * blockDim.x) {
    const int row = (int)row64;
    const Row32 r = decode_row32(g, row);
    const RowWin w = row_win(g, r);
    float acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    if (w.inside) {
      float qr[D];
      load_row<T, D>(q + q_row_of(g, r) * D, qr);
      const long long ybase = (long long)r.b * g.n_kv;
      const int hk = r.h / g.rep;
      int pb[3] = {0, 0, 0};
      long long bias_h = 0;
      if (bias != nullptr) {
#pragma unroll
        for (int a = 0; a < 3; ++a) pb[a] = pb_start(w.p[a], w.ext[a], g.K[a], g.dl[a]);
        bias_h = (long long)r.h * (2 * g.K[0] - 1) * w1 * w2;
      }
      SlotWalk walk;
      for (int s = 0; s < g.kvol; s += NB) {
        float kr[NB][D], vr[NB][D], bv[NB];
        bool ok[NB];
#pragma unroll
        for (int u = 0; u < NB; ++u) {
          ok[u] = false;
          bv[u] = 0.f;
          if (s + u < g.kvol) {
            const int b0 = pb[0] + walk.s0, b1 = pb[1] + walk.s1, b2 = pb[2] + walk.s2;
            long long key_row;
            ok[u] = walk.next(g, w, ybase, key_row);
            if (ok[u]) {
              load_row<T, D>(k + (key_row * g.Hkv + hk) * D, kr[u]);
              load_row<T, D>(v + (key_row * g.Hkv + hk) * D, vr[u]);
              if (bias != nullptr) bv[u] = bias[bias_h + ((long long)b0 * w1 + b1) * w2 + b2];
            }
          }
        }
#pragma unroll
        for (int u = 0; u < NB; ++u) {
          if (ok[u]) {
            float d = 0.f;
#pragma unroll
            for (int i = 0; i < D; ++i) d = fmaf(qr[i], kr[u][i], d);
            const float sc = g.scale * d + bv[u];
            const float m_new = fmaxf(m, sc);
            const float c = __expf(m - m_new);            // 0 on the first valid slot (m = -inf)
            const float pr = __expf(sc - m_new);
            l = l * c + pr;
#pragma unroll
            for (int i = 0; i < D; ++i) acc[i] = fmaf(acc[i], c, pr * vr[u][i]);
            m = m_new;
          }
        }
      }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < D; ++i) acc[i] *= inv;
    store_row<T, D>(out + (long long)row * D, acc);
    if (lse != nullptr) lse[row] = l > 0.f ? m + __logf(l) : (w.inside ? -INFINITY : 0.f);
  }
}

// ---------------------------------------------------------------------------
// row_inverse: dst[key row] = alpha * sum over every (query, slot) that addresses the key of
//              w[query, slot] * src[query]
// ---------------------------------------------------------------------------
// For key coordinate x on one axis the candidate queries are x + m * dilation, |m| <= K; a
// candidate counts when it lies on the stride lattice inside the local query slab and its
// window holds x.  Returns the slot or -1.
__device__ __forceinline__ int inverse_slot32(const Geo& g, int a, int ext, int x, int m, int& o) {
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

template <typename T, int D>
__global__ void __launch_bounds__(256)
k_row_inverse(Geo g, const T* __restrict__ wt, const T* __restrict__ src, T* __restrict__ dst, float alpha,
              int src_out_indexed, int n_rows) {
  for (long long row64 = (long long)blockIdx.x * blockDim.x + threadIdx.x; row64 < n_rows; row64 += (long long)gridDim.x * blockDim.x) {
    const int row = (int)row64;
    int t = row;
    const int hk = t % g.Hkv; t /= g.Hkv;
    const int j2 = t % g.ke[2]; t /= g.ke[2];
    const int j1 = t % g.ke[1]; t /= g.ke[1];
    const int j0 = t % g.ke[0]; t /= g.ke[0];
    const int b = t;
    int ext[3];
    sample_extent(g, b, ext);
    const int x0 = g.ko[0] + j0, x1 = g.ko[1] + j1, x2 = g.ko[2] + j2;
    float acc[D];
#pragma unroll
    for (int i = 0; i < D; ++i) acc[i] = 0.f;
    if (x0 < ext[0] && x1 < ext[1] && x2 < ext[2]) {
      for (int m0 = -g.K[0]; m0 <= g.K[0]; ++m0) {
        int o0;
        const int s0 = inverse_slot32(g, 0, ext[0], x0, m0, o0);
        if (s0 < 0) continue;
        for (int m1 = -g.K[1]; m1 <= g.K[1]; ++m1) {
          int o1;
          const int s1 = inverse_slot32(g, 1, ext[1], x1, m1, o1);
          if (s1 < 0) continue;
          for (int m2 = -g.K[2]; m2 <= g.K[2]; ++m2) {
            int o2;
            const int s2 = inverse_slot32(g, 2, ext[2], x2, m2, o2);
            if (s2 < 0) continue;
            const int slot = (s0 * g.K[1] + s1) * g.K[2] + s2;
            const long long ol = ((long long)o0 * g.out[1] + o1) * g.out[2] + o2;
            const long long ql = ((long long)(o0 * g.st[0]) * g.qe[1] + o1 * g.st[1]) * g.qe[2] + o2 * g.st[2];
            for (int hh = 0; hh < g.rep; ++hh) {
              const int h = hk * g.rep + hh;
              const long long wrow = ((long long)b * g.n_out + ol) * g.Hq + h;
              const float ws = to_f<T>(wt[wrow * g.kvol + slot]);
              const long long srow = src_out_indexed ? wrow : ((long long)b * g.n_q + ql) * g.Hq + h;
              float sr[D];
              load_row<T, D>(src + srow * D, sr);
#pragma unroll
              for (int i = 0; i < D; ++i) acc[i] = fmaf(ws, sr[i], acc[i]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < D; ++i) acc[i] *= alpha;
    store_row<T, D>(dst + (long long)row * D, acc);
  }
}

// ---------------------------------------------------------------------------
// gradient of the relative position bias
// ---------------------------------------------------------------------------
// One thread per (query, head) row.  Each warp adds into its own copy of the bias table in
// shared memory (the rows of a warp mostly share a handful of bins), the copies are summed
// and every block issues one global atomic per bin it touched.
template <typename T>
__global__ void __launch_bounds__(256)
k_row_bias_grad(Geo g, const T* __restrict__ dlogits, float* __restrict__ dbias, int n_rows, int bins, int copies) {
  extern __shared__ float hist[];
  for (int i = threadIdx.x; i < bins * copies; i += blockDim.x) hist[i] = 0.f;
  __syncthreads();
  float* mine = hist + ((threadIdx.x >> 5) % copies) * bins;
  const int w1 = 2 * g.K[1] - 1, w2 = 2 * g.K[2] - 1;
  for (long long row64 = (long long)blockIdx.x * blockDim.x + threadIdx.x; row64 < n_rows; row64 += (long long)gridDim.x * blockDim.x) {
    const int row = (int)row64;
    const Row32 r = decode_row32(g, row);
    const RowWin w = row_win(g, r);
    if (!w.inside) continue;
    int pb[3];
#pragma unroll
    for (int a = 0; a < 3; ++a) pb[a] = pb_start(w.p[a], w.ext[a], g.K[a], g.dl[a]);
    const int bias_h = r.h * (2 * g.K[0] - 1) * w1 * w2;
    const T* drow = dlogits + (long long)row * g.kvol;
    int slot = 0;
    for (int s0 = 0; s0 < g.K[0]; ++s0) {
      const int x0 = w.start[0] + s0 * g.dl[0];
      const bool v0 = x0 >= 0 && x0 < w.hi[0];
      for (int s1 = 0; s1 < g.K[1]; ++s1) {
        const int x1 = w.start[1] + s1 * g.dl[1];
        const bool v1 = v0 && x1 >= 0 && x1 < w.hi[1];
        for (int s2 = 0; s2 < g.K[2]; ++s2, ++slot) {
          const int x2 = w.start[2] + s2 * g.dl[2];
          if (!(v1 && x2 >= 0 && x2 < w.hi[2])) continue;
          atomicAdd(mine + bias_h + ((pb[0] + s0) * w1 + (pb[1] + s1)) * w2 + (pb[2] + s2), to_f<T>(drow[slot]));
        }
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < bins; i += blockDim.x) {
    float s = 0.f;
    for (int c = 0; c < copies; ++c) s += hist[c * bins + i];
    if (s != 0.f) atomicAdd(dbias + i, s);
  }
}

int grid_rows(long long rows) {
  long long blocks = (rows + 255) / 256;
  const long long cap = 148LL * 16;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

template <typename T, int D>
void launch_rows(SplitOp op, const Geo& g, const T* A, const T* Bp, const T* C, const float* bias, T* o0, T* o1,
                 cudaStream_t s) {
  const int n_out_rows = (int)((long long)g.B * g.n_out * g.Hq);
  const int n_kv_rows = (int)((long long)g.B * g.n_kv * g.Hkv);
  const float ninf = -__builtin_huge_valf();
  switch (op) {
    case SplitOp::QkForward:
      NB_LAUNCH("row_dot", s, k_row_dot<T, D><<<grid_rows(n_out_rows), 256, 0, s>>>(g, A, Bp, bias, o0, g.scale, ninf, 0, n_out_rows));
      break;
    case SplitOp::QkBackward: {   // A = q, Bp = k, C = dlogits -> o0 = dq, o1 = dk
      const bool strided = g.st[0] * g.st[1] * g.st[2] != 1 || g.n_out != g.n_q;
      if (strided) cudaMemsetAsync(o0, 0, (size_t)g.B * g.n_q * g.Hq * g.D * sizeof(T), s);
      NB_LAUNCH("row_wsum", s, k_row_wsum<T, D><<<grid_rows(n_out_rows), 256, 0, s>>>(g, C, Bp, o0, g.scale, 1, n_out_rows));
      NB_LAUNCH("row_inverse", s, k_row_inverse<T, D><<<grid_rows(n_kv_rows), 256, 0, s>>>(g, C, A, o1, g.scale, 0, n_kv_rows));
      break;
    }
    case SplitOp::AvForward:      // A = attn, Bp = v -> o0 = out
      NB_LAUNCH("row_wsum", s, k_row_wsum<T, D><<<grid_rows(n_out_rows), 256, 0, s>>>(g, A, Bp, o0, 1.f, 0, n_out_rows));
      break;
    case SplitOp::AvBackward:     // A = attn, Bp = v, C = dout -> o0 = dattn, o1 = dv
      NB_LAUNCH("row_dot", s, k_row_dot<T, D><<<grid_rows(n_out_rows), 256, 0, s>>>(g, C, Bp, nullptr, o0, 1.f, 0.f, 1, n_out_rows));
      NB_LAUNCH("row_inverse", s, k_row_inverse<T, D><<<grid_rows(n_kv_rows), 256, 0, s>>>(g, A, C, o1, 1.f, 1, n_kv_rows));
      break;
  }
}

template <typename T>
bool dispatch_rows(SplitOp op, const Geo& g, const void* a, const void* b, const void* c, const float* bias, void* o0,
                   void* o1, cudaStream_t s) {
  const T* A = static_cast<const T*>(a);
  const T* Bp = static_cast<const T*>(b);
  const T* C = static_cast<const T*>(c);
  T* O0 = static_cast<T*>(o0);
  T* O1 = static_cast<T*>(o1);
  switch (g.D) {
    case 8: launch_rows<T, 8>(op, g, A, Bp, C, bias, O0, O1, s); return true;
    case 12:
      if constexpr (sizeof(T) == 4) {   // 48-byte rows; 24-byte rows of the 16-bit types are no multiple of 16
        launch_rows<T, 12>(op, g, A, Bp, C, bias, O0, O1, s);
        return true;
      }
      return false;
    case 16: launch_rows<T, 16>(op, g, A, Bp, C, bias, O0, O1, s); return true;
    case 24: launch_rows<T, 24>(op, g, A, Bp, C, bias, O0, O1, s); return true;
    case 32: launch_rows<T, 32>(op, g, A, Bp, C, bias, O0, O1, s); return true;
  }
  return false;
}

template <typename T>
bool dispatch_fused(const Geo& g, const void* q, const void* k, const void* v, const float* bias, void* out, float* lse,
                    cudaStream_t s) {
  const int n_rows = (int)((long long)g.B * g.n_out * g.Hq);
#define NB_ROW_FUSED(DD)                                                                                              \
  NB_LAUNCH("row_fused", s, k_row_fused<T, DD><<<grid_rows(n_rows), 256, 0, s>>>(                                      \
      g, static_cast<const T*>(q), static_cast<const T*>(k), static_cast<const T*>(v), bias, static_cast<T*>(out), lse, n_rows)); \
  return true
  switch (g.D) {
    case 8: NB_ROW_FUSED(8);
    case 12:
      if constexpr (sizeof(T) == 4) { NB_ROW_FUSED(12); }
      return false;
    case 16: NB_ROW_FUSED(16);
    case 24: NB_ROW_FUSED(24);
    case 32: NB_ROW_FUSED(32);
  }
#undef NB_ROW_FUSED
  return false;
}

}  // namespace

// QK + bias -> softmax -> AV of every (query, head) row in one launch (forward only); false when the head dim is
// not one the row kernels are built for.
bool run_fused_rows(const Geo& g, int dtype, const void* q, const void* k, const void* v, const float* bias, void* out,
                    float* lse, cudaStream_t s) {
  switch (dtype) {
    case NATTEN_B200_F32: return dispatch_fused<float>(g, q, k, v, bias, out, lse, s);
    case NATTEN_B200_F16: return dispatch_fused<__half>(g, q, k, v, bias, out, lse, s);
    case NATTEN_B200_BF16: return dispatch_fused<__nv_bfloat16>(g, q, k, v, bias, out, lse, s);
  }
  return false;
}

// Serves a split operator with the row-per-thread kernels when the head dim is one of the small
// sizes they are built for (rows are then multiples of 16 bytes); returns false otherwise.
bool run_split_rows(SplitOp op, const Geo& g, int dtype, const void* a, const void* b, const void* c,
                    const float* bias, void* o0, void* o1, cudaStream_t s) {
  switch (dtype) {
    case NATTEN_B200_F32: return dispatch_rows<float>(op, g, a, b, c, bias, o0, o1, s);
    case NATTEN_B200_F16: return dispatch_rows<__half>(op, g, a, b, c, bias, o0, o1, s);
    case NATTEN_B200_BF16: return dispatch_rows<__nv_bfloat16>(op, g, a, b, c, bias, o0, o1, s);
  }
  return false;
}

// Gradient of the relative position bias with the per-block reduction; false when the bias table
// does not fit into shared memory (the caller then uses one global atomic per logit).
bool run_bias_grad_rows(const Geo& g, int dtype, const void* dlogits, float* dbias, cudaStream_t s) {
  const long long bins64 = (long long)g.Hq * (2 * g.K[0] - 1) * (2 * g.K[1] - 1) * (2 * g.K[2] - 1);
  if (bins64 > 10240) return false;
  const int bins = (int)bins64;
  int copies = 8;
  while (copies > 1 && (size_t)bins * copies * sizeof(float) > 40960) copies >>= 1;
  const int n_rows = (int)((long long)g.B * g.n_out * g.Hq);
  // few blocks: every block ends with one global atomic per bin
  long long blocks = (n_rows + 255) / 256;
  if (blocks > 148 * 2) blocks = 148 * 2;
  const size_t smem = (size_t)bins * copies * sizeof(float);
  switch (dtype) {
    case NATTEN_B200_F32:
      NB_LAUNCH("row_bias_grad", s, k_row_bias_grad<float><<<(int)blocks, 256, smem, s>>>(g, (const float*)dlogits, dbias, n_rows, bins, copies));
      return true;
    case NATTEN_B200_F16:
      NB_LAUNCH("row_bias_grad", s, k_row_bias_grad<__half><<<(int)blocks, 256, smem, s>>>(g, (const __half*)dlogits, dbias, n_rows, bins, copies));
      return true;
    case NATTEN_B200_BF16:
      NB_LAUNCH("row_bias_grad", s, k_row_bias_grad<__nv_bfloat16><<<(int)blocks, 256, smem, s>>>(g, (const __nv_bfloat16*)dlogits, dbias, n_rows, bins, copies));
      return true;
  }
  return false;
}

}  // namespace nb

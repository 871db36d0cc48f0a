// CUDA-core fused neighborhood attention (forward and backward) for every
// shape and dtype: float32 inputs, head dims that do not fit the tensor-core
// tiles, very small problems.  One warp owns one (query, head) row in the
// forward and in the dQ kernel, and one (key, kv head) row in the dK/dV kernel,
// so no kernel needs atomics except the extra-token gradient.
//
// Math: src/natten_mlx/_core/pure.py:155-255 (forward), its autodiff-defined
// backward (src/natten_mlx/_core/pure.py:691-733) written out from the saved
// log-sum-exp, and the extra-token / LSE composition of
// src/natten_mlx/functional.py:71-104, 368-381 folded into the same softmax.
#include <math.h>

#include "launch.cuh"

namespace nb {

namespace {

constexpr int kWarps = 4;

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

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Dot of a float row in shared memory with a row of T in global memory.
template <typename T>
__device__ __forceinline__ float dot_smem(const float* a, const T* b, int D, bool vec) {
  float acc = 0.f;
  if (vec) {
    constexpr int n = Vec16<T>::n;
    for (int i = 0; i < D; i += n) {
      float y[n];
      load16<T>(b + i, y);
#pragma unroll
      for (int j = 0; j < n; ++j) acc = fmaf(a[i + j], y[j], acc);
    }
  } else {
    for (int i = 0; i < D; ++i) acc = fmaf(a[i], to_f<T>(b[i]), acc);
  }
  return acc;
}

// Key row (in elements of T) addressed by slot `slot` of a query window, the
// extra-token row for slots past the window, or nullptr when invalid.
template <typename T>
__device__ __forceinline__ const T* slot_row(const Geo& g, const RowIdx& r, const int start[3],
                                             const int hi[3], int slot, const T* kv, const T* extra) {
  const int hk = r.h / g.rep;
  if (slot >= g.kvol) {
    return extra + (((long long)r.b * g.n_extra + (slot - g.kvol)) * g.Hkv + hk) * g.D;
  }
  const int s2 = slot % g.K[2];
  const int s1 = (slot / g.K[2]) % g.K[1];
  const int s0 = slot / (g.K[2] * g.K[1]);
  const int x0 = start[0] + s0 * g.dl[0];
  const int x1 = start[1] + s1 * g.dl[1];
  const int x2 = start[2] + s2 * g.dl[2];
  if (x0 < 0 || x0 >= hi[0] || x1 < 0 || x1 >= hi[1] || x2 < 0 || x2 >= hi[2]) return nullptr;
  const long long key = ((long long)(x0 - g.ko[0]) * g.ke[1] + (x1 - g.ko[1])) * g.ke[2] + (x2 - g.ko[2]);
  return kv + (((long long)r.b * g.n_kv + key) * g.Hkv + hk) * g.D;
}

__device__ __forceinline__ bool row_window(const Geo& g, const RowIdx& r, int start[3], int hi[3]) {
  int ext[3];
  sample_extent(g, r.b, ext);
  bool inside = true;
#pragma unroll
  for (int a = 0; a < 3; ++a) {
    const int p = g.qo[a] + r.o[a] * g.st[a];
    inside = inside && (p < ext[a]);
    axis_window(p, ext[a], g.K[a], g.dl[a], g.ca[a], start[a], hi[a]);
  }
  return inside;
}

__device__ __forceinline__ long long q_row_of(const Geo& g, const RowIdx& r) {
  const long long ql = ((long long)(r.o[0] * g.st[0]) * g.qe[1] + r.o[1] * g.st[1]) * g.qe[2] + r.o[2] * g.st[2];
  return ((long long)r.b * g.n_q + ql) * g.Hq + r.h;
}

// Lane layout for "sum over slots of weight * row": lanes form G groups of cp
// lanes; group sg takes slots sg, sg+G, ...; lane c of a group owns chunk c.
struct ChunkMap {
  int cp, G, sg, c;
  bool active;
};
__device__ __forceinline__ ChunkMap chunk_map(int chunks, int lane) {
  ChunkMap m;
  int cp = 1;
  while (cp < chunks && cp < 32) cp <<= 1;
  m.cp = cp;
  m.G = 32 / cp;
  m.sg = lane / cp;
  m.c = lane % cp;
  m.active = m.c < chunks;
  return m;
}
template <int CH>
__device__ __forceinline__ void reduce_groups(float (&acc)[CH], int cp) {
  for (int o = cp; o < 32; o <<= 1) {
#pragma unroll
    for (int i = 0; i < CH; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
  }
}

template <typename T, int CH>
__device__ __forceinline__ void axpy_row(float w, const T* row, float (&acc)[CH]) {
  if (CH == 1) {
    acc[0] = fmaf(w, to_f<T>(row[0]), acc[0]);
  } else {
    float v[CH];
    load16<T>(row, v);
#pragma unroll
    for (int i = 0; i < CH; ++i) acc[i] = fmaf(w, v[i], acc[i]);
  }
}

template <typename T, int CH>
__device__ __forceinline__ void store_chunk(T* dst, const float (&acc)[CH]) {
  if (CH == 1) dst[0] = from_f<T>(acc[0]);
  else store16<T>(dst, acc);
}

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
// Shared memory per warp: q row [D] float, weights [NS] float, row pointers as
// element offsets [NS] (long long), NS = K_vol + n_extra.
template <typename T, int CH>
__global__ void __launch_bounds__(kWarps * 32)
k_fused_fwd(Geo g, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
            const T* __restrict__ ke, const T* __restrict__ ve, T* __restrict__ out,
            float* __restrict__ lse, long long n_rows) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int NS = g.kvol + g.n_extra;
  const int Dp = (g.D + 3) & ~3;
  const size_t per_warp = (size_t)Dp * 4 + (size_t)NS * 4 + (size_t)NS * 8;
  unsigned char* base = smem_raw + (size_t)warp * ((per_warp + 15) & ~(size_t)15);
  long long* koff = reinterpret_cast<long long*>(base);
  float* qs = reinterpret_cast<float*>(base + (size_t)NS * 8);
  float* ws = qs + Dp;
  const bool vec = CH != 1;
  const int chunks = g.D / CH;

  for (long long row = (long long)blockIdx.x * kWarps + warp; row < n_rows;
       row += (long long)gridDim.x * kWarps) {
    const RowIdx r = decode_row(g, row);
    int start[3], hi[3];
    const bool inside = row_window(g, r, start, hi);
    if (!inside) {  // padded query of a variable-size batch
      for (int i = lane; i < g.D; i += 32) out[row * g.D + i] = from_f<T>(0.f);
      if (lse != nullptr && lane == 0) lse[row] = 0.f;
      continue;
    }
    const T* qrow = q + q_row_of(g, r) * g.D;
    for (int i = lane; i < g.D; i += 32) qs[i] = to_f<T>(qrow[i]);
    __syncwarp();
    float mx = -INFINITY;
    for (int s = lane; s < NS; s += 32) {
      const T* kr = slot_row<T>(g, r, start, hi, s, k, ke);
      float logit = -INFINITY;
      long long off = -1;
      if (kr != nullptr) {
        logit = g.scale * dot_smem<T>(qs, kr, g.D, vec);
        off = (s >= g.kvol) ? -2 - (long long)(kr - ke) : (long long)(kr - k);
      }
      ws[s] = logit;
      koff[s] = off;
      mx = fmaxf(mx, logit);
    }
    mx = warp_max(mx);
    float sum = 0.f;
    __syncwarp();
    for (int s = lane; s < NS; s += 32) {
      const float p = (koff[s] == -1) ? 0.f : __expf(ws[s] - mx);
      ws[s] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    __syncwarp();
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    if (lse != nullptr && lane == 0) lse[row] = sum > 0.f ? mx + logf(sum) : -INFINITY;

    const ChunkMap cm = chunk_map(chunks, lane);
    for (int c0 = 0; c0 < chunks; c0 += cm.cp) {
      const int c = c0 + cm.c;
      float acc[CH];
#pragma unroll
      for (int i = 0; i < CH; ++i) acc[i] = 0.f;
      if (c < chunks) {
        for (int s = cm.sg; s < NS; s += cm.G) {
          const long long off = koff[s];
          if (off == -1) continue;
          const T* vr = (off <= -2) ? ve + (-2 - off) : v + off;
          axpy_row<T, CH>(ws[s], vr + c * CH, acc);
        }
      }
      reduce_groups<CH>(acc, cm.cp);
      if (cm.sg == 0 && c < chunks) {
#pragma unroll
        for (int i = 0; i < CH; ++i) acc[i] *= inv;
        store_chunk<T, CH>(out + row * g.D + c * CH, acc);
      }
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------
// backward, query side: delta, dS and dQ
// ---------------------------------------------------------------------------
// delta = sum(dO * O) - dLSE;  P = exp(S - lse);  dS = P * (dO.V - delta);
// dQ = scale * sum dS * K.  delta is also written to scratch for the key-side
// kernels.  Shared memory per warp: q [D], dO [D], dS [NS], offsets [NS].
template <typename T, int CH>
__global__ void __launch_bounds__(kWarps * 32)
k_fused_bwd_q(Geo g, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
              const T* __restrict__ ke, const T* __restrict__ ve, const T* __restrict__ o,
              const float* __restrict__ lse, const T* __restrict__ dout,
              const float* __restrict__ dlse, T* __restrict__ dq, float* __restrict__ delta_out,
              long long n_rows) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int NS = g.kvol + g.n_extra;
  const int Dp = (g.D + 3) & ~3;
  const size_t per_warp = (size_t)Dp * 8 + (size_t)NS * 4 + (size_t)NS * 8;
  unsigned char* base = smem_raw + (size_t)warp * ((per_warp + 15) & ~(size_t)15);
  long long* koff = reinterpret_cast<long long*>(base);
  float* qs = reinterpret_cast<float*>(base + (size_t)NS * 8);
  float* dos = qs + Dp;
  float* ws = dos + Dp;
  const bool vec = CH != 1;
  const int chunks = g.D / CH;

  for (long long row = (long long)blockIdx.x * kWarps + warp; row < n_rows;
       row += (long long)gridDim.x * kWarps) {
    const RowIdx r = decode_row(g, row);
    int start[3], hi[3];
    const bool inside = row_window(g, r, start, hi);
    const long long qr = q_row_of(g, r);
    if (!inside) {
      for (int i = lane; i < g.D; i += 32) dq[qr * g.D + i] = from_f<T>(0.f);
      if (lane == 0) delta_out[row] = 0.f;
      continue;
    }
    float part = 0.f;
    for (int i = lane; i < g.D; i += 32) {
      const float d_o = to_f<T>(dout[row * g.D + i]);
      qs[i] = to_f<T>(q[qr * g.D + i]);
      dos[i] = d_o;
      part = fmaf(d_o, to_f<T>(o[row * g.D + i]), part);
    }
    const float delta = warp_sum(part) - (dlse != nullptr ? dlse[row] : 0.f);
    if (lane == 0) delta_out[row] = delta;
    const float l = lse[row];
    __syncwarp();
    for (int s = lane; s < NS; s += 32) {
      const T* kr = slot_row<T>(g, r, start, hi, s, k, ke);
      float ds = 0.f;
      long long off = -1;
      if (kr != nullptr) {
        const bool extra = s >= g.kvol;
        off = extra ? -2 - (long long)(kr - ke) : (long long)(kr - k);
        const T* vr = extra ? ve + (kr - ke) : v + (kr - k);
        const float p = __expf(g.scale * dot_smem<T>(qs, kr, g.D, vec) - l);
        ds = p * (dot_smem<T>(dos, vr, g.D, vec) - delta);
      }
      ws[s] = ds;
      koff[s] = off;
    }
    __syncwarp();
    const ChunkMap cm = chunk_map(chunks, lane);
    for (int c0 = 0; c0 < chunks; c0 += cm.cp) {
      const int c = c0 + cm.c;
      float acc[CH];
#pragma unroll
      for (int i = 0; i < CH; ++i) acc[i] = 0.f;
      if (c < chunks) {
        for (int s = cm.sg; s < NS; s += cm.G) {
          const long long off = koff[s];
          if (off == -1) continue;
          const T* kr = (off <= -2) ? ke + (-2 - off) : k + off;
          axpy_row<T, CH>(ws[s], kr + c * CH, acc);
        }
      }
      reduce_groups<CH>(acc, cm.cp);
      if (cm.sg == 0 && c < chunks) {
#pragma unroll
        for (int i = 0; i < CH; ++i) acc[i] *= g.scale;
        store_chunk<T, CH>(dq + qr * g.D + c * CH, acc);
      }
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------
// backward, key side: dK and dV of the window keys
// ---------------------------------------------------------------------------
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

// One warp per (key, kv head).  Pass 1 walks the candidate queries, keeps the
// ones whose window holds the key and stores (P, dS, row ids) in shared
// memory; pass 2 forms dV = sum P * dO and dK = scale * sum dS * Q.
// A key near a clamped edge is addressed by more queries than the kernel has
// slots (every edge query's window is pulled inward over it), so the lists are
// sized for a window of kKvWindow candidates and the candidates are walked
// window by window.
// Shared memory per warp: k [D], v [D], and P, dS, out-row, q-row of kKvWindow
// entries each.
constexpr int kKvWindow = 512;
template <typename T, int CH>
__global__ void __launch_bounds__(kWarps * 32)
k_fused_bwd_kv(Geo g, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
               const float* __restrict__ lse, const T* __restrict__ dout,
               const float* __restrict__ delta, T* __restrict__ dk, T* __restrict__ dv,
               long long n_rows) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cap = kKvWindow;
  const int Dp = (g.D + 3) & ~3;
  const size_t per_warp = (size_t)Dp * 8 + (size_t)cap * 16;
  unsigned char* base = smem_raw + (size_t)warp * ((per_warp + 15) & ~(size_t)15);
  float* ks = reinterpret_cast<float*>(base);
  float* vs = ks + Dp;
  float* ps = vs + Dp;
  float* dss = ps + cap;
  int* orow = reinterpret_cast<int*>(dss + cap);
  int* qrow = orow + cap;
  const bool vec = CH != 1;
  const int chunks = g.D / CH;
  // a query can sit up to K lattice steps from a key it addresses: an even
  // kernel pulled inward at the far edge does not reach the query itself
  const int C0 = 2 * g.K[0] + 1, C1 = 2 * g.K[1] + 1, C2 = 2 * g.K[2] + 1;
  const int n_cand = g.rep * C0 * C1 * C2;

  for (long long row = (long long)blockIdx.x * kWarps + warp; row < n_rows;
       row += (long long)gridDim.x * kWarps) {
    long long t = row;
    const int hk = (int)(t % g.Hkv); t /= g.Hkv;
    const int j2 = (int)(t % g.ke[2]); t /= g.ke[2];
    const int j1 = (int)(t % g.ke[1]); t /= g.ke[1];
    const int j0 = (int)(t % g.ke[0]); t /= g.ke[0];
    const int b = (int)t;
    int ext[3];
    sample_extent(g, b, ext);
    const int x0 = g.ko[0] + j0, x1 = g.ko[1] + j1, x2 = g.ko[2] + j2;
    for (int i = lane; i < g.D; i += 32) {
      ks[i] = to_f<T>(k[row * g.D + i]);
      vs[i] = to_f<T>(v[row * g.D + i]);
    }
    __syncwarp();
    const ChunkMap cm = chunk_map(chunks, lane);
    for (int cg = 0; cg < chunks; cg += cm.cp) {
      const int cc = cg + cm.c;
      float av[CH], ak[CH];
#pragma unroll
      for (int i = 0; i < CH; ++i) { av[i] = 0.f; ak[i] = 0.f; }
      // candidates are taken in windows of kKvWindow so that the lists always fit
      for (int w0 = 0; w0 < n_cand; w0 += kKvWindow) {
        const int w1 = w0 + kKvWindow < n_cand ? w0 + kKvWindow : n_cand;
        int count = 0;
        for (int c0 = w0; c0 < w1; c0 += 32) {
          const int c = c0 + lane;
          bool ok = c < w1;
          float p = 0.f, ds = 0.f;
          int orow_i = 0, qrow_i = 0;
          if (ok) {
            int u = c;
            const int m2 = u % C2 - g.K[2]; u /= C2;
            const int m1 = u % C1 - g.K[1]; u /= C1;
            const int m0 = u % C0 - g.K[0]; u /= C0;
            const int h = hk * g.rep + u;
            int o0, o1, o2;
            ok = inverse_slot(g, 0, ext[0], x0, m0, o0) >= 0 && inverse_slot(g, 1, ext[1], x1, m1, o1) >= 0 &&
                 inverse_slot(g, 2, ext[2], x2, m2, o2) >= 0;
            if (ok) {
              const long long ol = ((long long)o0 * g.out[1] + o1) * g.out[2] + o2;
              const long long ql = ((long long)(o0 * g.st[0]) * g.qe[1] + o1 * g.st[1]) * g.qe[2] + o2 * g.st[2];
              const long long orl = ((long long)b * g.n_out + ol) * g.Hq + h;
              const long long qrl = ((long long)b * g.n_q + ql) * g.Hq + h;
              orow_i = (int)orl;
              qrow_i = (int)qrl;
              p = __expf(g.scale * dot_smem<T>(ks, q + qrl * g.D, g.D, vec) - lse[orl]);
              ds = p * (dot_smem<T>(vs, dout + orl * g.D, g.D, vec) - delta[orl]);
            }
          }
          const unsigned ballot = __ballot_sync(0xffffffffu, ok);
          if (ok) {
            const int pos = count + __popc(ballot & ((1u << lane) - 1u));
            ps[pos] = p;
            dss[pos] = ds;
            orow[pos] = orow_i;
            qrow[pos] = qrow_i;
          }
          count += __popc(ballot);
        }
        __syncwarp();
        if (cc < chunks) {
          for (int s = cm.sg; s < count; s += cm.G) {
            axpy_row<T, CH>(ps[s], dout + (long long)orow[s] * g.D + cc * CH, av);
            axpy_row<T, CH>(dss[s], q + (long long)qrow[s] * g.D + cc * CH, ak);
          }
        }
        __syncwarp();
      }
      reduce_groups<CH>(av, cm.cp);
      reduce_groups<CH>(ak, cm.cp);
      if (cm.sg == 0 && cc < chunks) {
#pragma unroll
        for (int i = 0; i < CH; ++i) ak[i] *= g.scale;
        store_chunk<T, CH>(dv + row * g.D + cc * CH, av);
        store_chunk<T, CH>(dk + row * g.D + cc * CH, ak);
      }
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------
// backward, extra tokens: every query of the sample contributes
// ---------------------------------------------------------------------------
// One warp per (sample, token, kv head, query chunk); float accumulators are
// added into scratch with atomics and converted afterwards.  Lane i owns
// elements i, i+32, ... of the head dimension (at most kMaxPerLane of them).
constexpr int kMaxPerLane = 16;

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
k_fused_bwd_extra(Geo g, const T* __restrict__ q, const T* __restrict__ ke, const T* __restrict__ ve,
                  const float* __restrict__ lse, const T* __restrict__ dout,
                  const float* __restrict__ delta, float* __restrict__ acc_k, float* __restrict__ acc_v,
                  int q_chunk, int n_qchunks) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long n_items = (long long)g.B * g.n_extra * g.Hkv * n_qchunks;
  const int per = (g.D + 31) / 32;
  for (long long item = (long long)blockIdx.x * kWarps + warp; item < n_items;
       item += (long long)gridDim.x * kWarps) {
    long long t = item;
    const int qc = (int)(t % n_qchunks); t /= n_qchunks;
    const int hk = (int)(t % g.Hkv); t /= g.Hkv;
    const int e = (int)(t % g.n_extra); t /= g.n_extra;
    const int b = (int)t;
    int ext[3];
    sample_extent(g, b, ext);
    const long long erow = ((long long)b * g.n_extra + e) * g.Hkv + hk;
    float kr[kMaxPerLane], vr[kMaxPerLane], ak[kMaxPerLane], av[kMaxPerLane];
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      const bool in = i < per && d < g.D;
      kr[i] = in ? to_f<T>(ke[erow * g.D + d]) : 0.f;
      vr[i] = in ? to_f<T>(ve[erow * g.D + d]) : 0.f;
      ak[i] = 0.f;
      av[i] = 0.f;
    }
    const long long o_begin = (long long)qc * q_chunk;
    const long long o_end = o_begin + q_chunk < g.n_out ? o_begin + q_chunk : g.n_out;
    for (long long ol = o_begin; ol < o_end; ++ol) {
      const int o2 = (int)(ol % g.out[2]);
      const int o1 = (int)((ol / g.out[2]) % g.out[1]);
      const int o0 = (int)(ol / ((long long)g.out[2] * g.out[1]));
      if (g.qo[0] + o0 * g.st[0] >= ext[0] || g.qo[1] + o1 * g.st[1] >= ext[1] ||
          g.qo[2] + o2 * g.st[2] >= ext[2])
        continue;
      const long long ql = ((long long)(o0 * g.st[0]) * g.qe[1] + o1 * g.st[1]) * g.qe[2] + o2 * g.st[2];
      for (int hh = 0; hh < g.rep; ++hh) {
        const int h = hk * g.rep + hh;
        const long long orl = ((long long)b * g.n_out + ol) * g.Hq + h;
        const long long qrl = ((long long)b * g.n_q + ql) * g.Hq + h;
        float qv[kMaxPerLane], dv_[kMaxPerLane];
        float s = 0.f, dp = 0.f;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
          const int d = lane + 32 * i;
          const bool in = i < per && d < g.D;
          qv[i] = in ? to_f<T>(q[qrl * g.D + d]) : 0.f;
          dv_[i] = in ? to_f<T>(dout[orl * g.D + d]) : 0.f;
          s = fmaf(qv[i], kr[i], s);
          dp = fmaf(dv_[i], vr[i], dp);
        }
        s = warp_sum(s);
        dp = warp_sum(dp);
        const float p = __expf(g.scale * s - lse[orl]);
        const float ds = p * (dp - delta[orl]) * g.scale;
#pragma unroll
        for (int i = 0; i < kMaxPerLane; ++i) {
          av[i] = fmaf(p, dv_[i], av[i]);
          ak[i] = fmaf(ds, qv[i], ak[i]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < kMaxPerLane; ++i) {
      const int d = lane + 32 * i;
      if (i < per && d < g.D) {
        atomicAdd(acc_k + erow * g.D + d, ak[i]);
        atomicAdd(acc_v + erow * g.D + d, av[i]);
      }
    }
  }
}

template <typename T>
__global__ void k_cast_out(const float* __restrict__ src, T* __restrict__ dst, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = from_f<T>(src[i]);
}

int blocks_for_rows(long long rows) {
  long long blocks = (rows + kWarps - 1) / kWarps;
  const long long cap = 148LL * 64;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

template <typename K>
int opt_in_smem(K kernel, size_t bytes) {
  if (bytes > 227 * 1024) return set_error(NATTEN_B200_ERESOURCE,
      "kernel needs %zu bytes of shared memory per block (limit 232448)", bytes);
  if (bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return set_error(NATTEN_B200_ELAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  }
  return 0;
}

size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }

template <typename T, int CH>
int fwd_impl(const Geo& g, const FusedArgs& a, cudaStream_t s) {
  const int NS = g.kvol + g.n_extra;
  const int Dp = (g.D + 3) & ~3;
  const size_t smem = kWarps * align16((size_t)Dp * 4 + (size_t)NS * 12);
  if (int rc = opt_in_smem(k_fused_fwd<T, CH>, smem)) return rc;
  const long long rows = (long long)g.B * g.n_out * g.Hq;
  NB_LAUNCH("fused_fwd", s, k_fused_fwd<T, CH><<<blocks_for_rows(rows), kWarps * 32, smem, s>>>(
      g, (const T*)a.q, (const T*)a.k, (const T*)a.v, (const T*)a.k_extra, (const T*)a.v_extra,
      (T*)a.out, a.lse, rows));
  return check_launch("fused forward");
}

template <typename T, int CH>
int bwd_impl(const Geo& g, const FusedArgs& a, cudaStream_t s) {
  const int NS = g.kvol + g.n_extra;
  const int Dp = (g.D + 3) & ~3;
  const long long rows = (long long)g.B * g.n_out * g.Hq;
  float* delta = static_cast<float*>(a.scratch);
  const bool strided = g.n_out != g.n_q;
  if (strided) cudaMemsetAsync(a.dq, 0, (size_t)g.B * g.n_q * g.Hq * g.D * sizeof(T), s);
  {
    const size_t smem = kWarps * align16((size_t)Dp * 8 + (size_t)NS * 12);
    if (int rc = opt_in_smem(k_fused_bwd_q<T, CH>, smem)) return rc;
    NB_LAUNCH("fused_bwd_q", s, k_fused_bwd_q<T, CH><<<blocks_for_rows(rows), kWarps * 32, smem, s>>>(
        g, (const T*)a.q, (const T*)a.k, (const T*)a.v, (const T*)a.k_extra, (const T*)a.v_extra,
        (const T*)a.out, a.lse, (const T*)a.dout, a.dlse, (T*)a.dq, delta, rows));
  }
  {
    const size_t smem = kWarps * align16((size_t)Dp * 8 + (size_t)kKvWindow * 16);
    if (int rc = opt_in_smem(k_fused_bwd_kv<T, CH>, smem)) return rc;
    const long long krows = (long long)g.B * g.n_kv * g.Hkv;
    NB_LAUNCH("fused_bwd_kv", s, k_fused_bwd_kv<T, CH><<<blocks_for_rows(krows), kWarps * 32, smem, s>>>(
        g, (const T*)a.q, (const T*)a.k, (const T*)a.v, a.lse, (const T*)a.dout, delta,
        (T*)a.dk, (T*)a.dv, krows));
  }
  if (g.n_extra > 0) {
    if (g.D > 32 * kMaxPerLane)
      return set_error(NATTEN_B200_EINVAL, "extra-token gradient supports head_dim <= %d", 32 * kMaxPerLane);
    const long long n_e = (long long)g.B * g.n_extra * g.Hkv * g.D;
    float* acc_k = delta + ((rows + 3) & ~3LL);
    float* acc_v = acc_k + n_e;
    cudaMemsetAsync(acc_k, 0, (size_t)n_e * 2 * sizeof(float), s);
    const int q_chunk = 256;
    const int n_qchunks = (int)((g.n_out + q_chunk - 1) / q_chunk);
    const long long items = (long long)g.B * g.n_extra * g.Hkv * n_qchunks;
    NB_LAUNCH("fused_bwd_extra", s, k_fused_bwd_extra<T><<<blocks_for_rows(items), kWarps * 32, 0, s>>>(
        g, (const T*)a.q, (const T*)a.k_extra, (const T*)a.v_extra, a.lse, (const T*)a.dout, delta,
        acc_k, acc_v, q_chunk, n_qchunks));
    const int cb = (int)((n_e + 255) / 256 > 148 * 16 ? 148 * 16 : (n_e + 255) / 256);
    NB_LAUNCH("cast_out", s, k_cast_out<T><<<cb, 256, 0, s>>>(acc_k, (T*)a.dk_extra, n_e));
    NB_LAUNCH("cast_out", s, k_cast_out<T><<<cb, 256, 0, s>>>(acc_v, (T*)a.dv_extra, n_e));
  }
  return check_launch("fused backward");
}

template <typename T>
int fwd_dispatch(const Geo& g, const FusedArgs& a, cudaStream_t s) {
  if ((g.D * (int)sizeof(T)) % 16 == 0) return fwd_impl<T, Vec16<T>::n>(g, a, s);
  return fwd_impl<T, 1>(g, a, s);
}
template <typename T>
int bwd_dispatch(const Geo& g, const FusedArgs& a, cudaStream_t s) {
  if ((g.D * (int)sizeof(T)) % 16 == 0) return bwd_impl<T, Vec16<T>::n>(g, a, s);
  return bwd_impl<T, 1>(g, a, s);
}

}  // namespace

size_t fused_backward_scratch_simt(const Geo& g) {
  const long long rows = (long long)g.B * g.n_out * g.Hq;
  const long long n_e = (long long)g.B * g.n_extra * g.Hkv * g.D;
  return (size_t)(((rows + 3) & ~3LL) + 2 * n_e) * sizeof(float);
}

int run_fused_forward_simt(const Geo& g, int dtype, const FusedArgs& a, cudaStream_t s) {
  switch (dtype) {
    case NATTEN_B200_F32: return fwd_dispatch<float>(g, a, s);
    case NATTEN_B200_F16: return fwd_dispatch<__half>(g, a, s);
    case NATTEN_B200_BF16: return fwd_dispatch<__nv_bfloat16>(g, a, s);
  }
  return set_error(NATTEN_B200_EINVAL, "unsupported dtype %d", dtype);
}

int run_fused_backward_simt(const Geo& g, int dtype, const FusedArgs& a, cudaStream_t s) {
  switch (dtype) {
    case NATTEN_B200_F32: return bwd_dispatch<float>(g, a, s);
    case NATTEN_B200_F16: return bwd_dispatch<__half>(g, a, s);
    case NATTEN_B200_BF16: return bwd_dispatch<__nv_bfloat16>(g, a, s);
  }
  return set_error(NATTEN_B200_EINVAL, "unsupported dtype %d", dtype);
}

}  // namespace nb

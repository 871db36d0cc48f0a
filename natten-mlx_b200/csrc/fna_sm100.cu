// Tensor-core fused neighborhood attention, forward pass, for sm_100a.
//
// A persistent CTA walks (batch, kv head, head group, dilation class, query tile) work items.
// Dilation is removed up front: the queries p = i*d + g of one residue class g attend only
// to keys of the same class, so each class is a dilation-1 problem on a strided view and gets
// its own TMA tensor maps.  The 128 rows of a tile are (heads sharing the kv head) x (tile
// positions).  The keys every row of the tile can address form a box; the box is walked in
// chunks (ranges of box rows), and the chunks of all tiles of a CTA form one stream:
//   TMA warp     K/V chunks -> a ring of shared-memory stages (zero fill outside the tensor)
//   MMA warp     S = Q K^T of chunk j+1 (tcgen05.mma, operands in smem, S in a ring of TMEM
//                buffers), then O += P V of chunk j (A = P from TMEM, B = V MN-major)
//   4 softmax warps   S -> registers over the box rows the warp needs, window/causal mask as
//                additive offsets (or a bitmap for boxes without row structure), softmax in
//                base 2 against a lazily updated reference maximum, P (bf16/f16) -> TMEM over S
// and one chunk into the next tile the softmax warps scale the finished O by 1/l and write out
// and the log-sum-exp.  Math as in src/natten_mlx/_core/pure.py:155-255
// with the LSE of src/natten_mlx/functional.py:368-372.
#include <cuda.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <cstdio>
#include <map>
#include <mutex>
#include <vector>

#include "fna_sm100.cuh"
#include "sm100_ptx.cuh"

namespace nb {
namespace {

using namespace sm100;

constexpr int kMaxClasses = 16;
constexpr int kTileM = 128;
constexpr int kMaxCols = 384;            // S columns per chunk
constexpr int kMaxWords = kMaxCols / 32;
constexpr int kThreads = 192;            // 4 softmax warps, 1 TMA warp, 1 MMA warp
// Tensor maps of variable-size batches travel through a ring of slots in device memory that belongs to the
// library; a call's maps (four per (sample, dilation class) pair in the backward) must fit one slot.
constexpr int kMapSlots = 8;
constexpr size_t kMapSlotBytes = 256 * 1024;

struct alignas(64) TmaMaps {
  CUtensorMap q[kMaxClasses];
  CUtensorMap k[kMaxClasses];
  CUtensorMap v[kMaxClasses];
  CUtensorMap xk, xv;   // extra tokens [B, N_extra, Hkv, D]
};

// Backward: r1/r2 are the row operands of a tile (Q, dO | K, V), c1/c2 the
// chunk operands (K, V | Q, dO).
struct alignas(64) TmaMapsBwd {
  CUtensorMap r1[kMaxClasses];
  CUtensorMap r2[kMaxClasses];
  CUtensorMap c1[kMaxClasses];
  CUtensorMap c2[kMaxClasses];
  CUtensorMap xk, xv;   // extra tokens: chunk operands of the dQ kernel, row operands of the dK/dV kernel's extra-token items
};

struct FwdParams {
  int B, Hq, Hkv, rep, D;
  int rank;              // spatial rank of the tensors (tensor-map rank = rank + 2)
  int L[3], K[3], dl[3], ca[3];
  int Mr[3], Mc[3];                   // extents behind the memory strides of the row / chunk tensors (== L when dense)
  // queries on a stride lattice: the forward and dQ kernels tile output coordinates (row stride rst, position =
  // coordinate * rst), the dK/dV kernel walks them as chunk columns (cst); 1 everywhere without a stride.  Mq:
  // extents of the query tensor (dQ is laid out over positions, the statistics over outputs)
  int rst[3], cst[3], strided, Mq[3];
  int ro0, re0, co0, ce0;             // leading-axis slab: first global plane and plane count of the row / chunk tensors
  int T[3];              // query tile extents in class coordinates
  int hpt, P;            // heads per tile, positions per tile (hpt * P == 128)
  int box[3];            // key box extents
  int rp;                // 16 or 32: box rows padded to that many columns (box[2] == rp); 0: no row structure
  int chunk_axis, R, cchunks, n_chunks, inner, n_cols, n_pad, n_split, n_half;
  int dblk, ndblk, row_bytes, layout_type;
  int q_stages, kv_stages;
  int n_sbuf;                         // depth of the S/P (forward) or S+dP (backward) ring in tensor memory
  int ctas_per_sm, tmem_cols, ocol;   // TMEM: S/P at column 0, O at ocol
  // backward kernels: mode 1 = dQ (rows are queries), mode 2 = dK/dV (rows are keys)
  int mode, head_groups;
  int dp_col, acc_col, acc2_col;      // TMEM: dP at dp_col, dQ | dK at acc_col, dV at acc2_col
  const float* lse_in;                // saved log-sum-exp [rows of out] (natural log)
  const float* delta;                 // rowsum(dO * O) - dLSE [rows of out]
  void* out2;                         // dV (mode 2)
  // mode 2 on a slab: dK / dV rows of the first halo_lo and the last halo_hi planes of the K/V slab go to these
  // tensors ([batch, planes, rest of the layout]; memory of a neighbouring GPU) instead of out / out2
  int halo_lo, halo_hi;
  void *out_lo, *out2_lo, *out_hi, *out2_hi;
  int tiles[3];
  long long n_work;
  float scale_log2;
  uint32_t idesc_qk, idesc_pv;
  int is_bf16;
  // variable-size batches: per-sample extents on the device, and the tensor maps of every (sample, dilation class)
  // in global memory, `nmaps` per pair in the order of the parameter maps (q k v | r1 r2 c1 c2)
  const int* extents;
  const CUtensorMap* gmaps;
  int nmaps;
  // extra tokens: count, tokens per extra chunk (a chunk of xw tokens follows the chunks of the key box in the
  // forward and dQ kernels), number of such chunks
  int n_extra, xw, n_xchunks;
  // dK/dV kernel: the work items after n_work_main own the extra tokens (rows = a tile of 128 tokens, chunks = one
  // box of a dilation class's queries, xr[a] boxes per axis); their partial sums go to float32 accumulators
  long long n_work_main;
  int n_xtiles, xr[3];
  float *acc_k, *acc_v;
  void* out;
  float* lse;
  int* status;
  unsigned long long* prof;  // optional cycle counters of CTA 0 (diagnostic)
};

// ---------------------------------------------------------------------------
// host: planning
// ---------------------------------------------------------------------------
int ceil_div(int a, int b) { return (a + b - 1) / b; }

struct Plan {
  FwdParams p;
  size_t smem;
  bool ok;
  const char* why;
};

// Shared memory: [Q stages][K stages][V stages][bitmap][barriers + tmem slot]
size_t smem_needed(const FwdParams& p) {
  const size_t row_tiles = p.mode == 0 ? 1 : 2;   // forward: Q; backward: two row operands
  const size_t q = (size_t)p.q_stages * row_tiles * p.ndblk * kTileM * p.row_bytes;
  const size_t kv = (size_t)p.kv_stages * 2 * p.ndblk * p.n_pad * p.row_bytes;
  const size_t stats = p.mode == 2 ? (size_t)p.kv_stages * 2 * p.n_pad * 4 : 0;   // per-column lse / delta
  return 1024 /*alignment slack*/ + q + kv + stats + (size_t)kMaxWords * 128 * 4 + 2560 /*barriers, work items, window tables*/;
}

// Class entries i (global position i * d + g) of dilation class g that lie in planes [first, ...): the first one,
// and for an exclusive end plane the one past the last.
__host__ __device__ inline int slab_lo(int first, int g, int d) { return first <= g ? 0 : (first - g + d - 1) / d; }
__host__ __device__ inline int slab_hi(int end, int g, int d) { return end <= g ? 0 : (end - g + d - 1) / d; }

// Window of query i of a dilation class in class coordinates (the host twin of class_window()
// in the kernels): valid keys are [max(s, 0), e).
void host_class_window(int i, int g, int lg, int L, int K, int d, int& s, int& e) {
  if (d == 1) {
    s = window_start(i, L, K, 1);
  } else {
    const int start = window_start(i * d + g, L, K, d);
    s = (start - g) / d;
  }
  e = s + K < lg ? s + K : lg;
}

// Largest number of consecutive queries whose windows hold some key of a tile of T keys on one
// axis with a centred window: windows pulled inward at the two ends of the axis are also held
// by queries further in, so near the ends a key tile is addressed from more than T + K - 1
// queries (by up to K / 2 more when the tile starts within the first K keys).  Exact, by
// walking every tile of every dilation class.
int max_query_span(int L, int K, int d, int T) {
  int best = 0;
  for (int g = 0; g < d && g < L; ++g) {
    const int lg = (L - g + d - 1) / d;
    std::vector<int> lo(lg), hi(lg);           // per key: first query and one past the last query
    for (int x = 0; x < lg; ++x) { lo[x] = lg; hi[x] = 0; }
    for (int q = 0; q < lg; ++q) {
      int s, e;
      host_class_window(q, g, lg, L, K, d, s, e);
      for (int x = s < 0 ? 0 : s; x < e; ++x) {
        if (q < lo[x]) lo[x] = q;
        if (q + 1 > hi[x]) hi[x] = q + 1;
      }
    }
    for (int t = 0; t < lg; t += T) {
      int a = lg, b = 0;
      for (int x = t; x < t + T && x < lg; ++x) {
        if (lo[x] < a) a = lo[x];
        if (hi[x] > b) b = hi[x];
      }
      if (b - a > best) best = b - a;
    }
  }
  return best;
}

// Mean over the tiles of one axis of (box rows some row of the tile needs) / (box rows): tiles at
// the ends of an axis need fewer than the box holds, and the elementwise warps skip the rest.
// Rows are queries and the box holds keys (rows_are_q), or the other way round.  Class 0 stands
// for all dilation classes.
double mean_needed_fraction(int L, int K, int d, int T, int box, bool rows_are_q) {
  const int lg = (L + d - 1) / d;
  std::vector<int> lo(lg), hi(lg);
  for (int x = 0; x < lg; ++x) { lo[x] = lg; hi[x] = 0; }
  for (int q = 0; q < lg; ++q) {
    int s, e;
    host_class_window(q, 0, lg, L, K, d, s, e);
    if (s < 0) s = 0;
    if (rows_are_q) { lo[q] = s; hi[q] = e; continue; }
    for (int x = s; x < e; ++x) {
      if (q < lo[x]) lo[x] = q;
      if (q + 1 > hi[x]) hi[x] = q + 1;
    }
  }
  double sum = 0.0;
  int n = 0;
  for (int t = 0; t < lg; t += T, ++n) {
    int a = lg, b = 0;
    for (int x = t; x < t + T && x < lg; ++x) {
      if (lo[x] < a) a = lo[x];
      if (hi[x] > b) b = hi[x];
    }
    const int need = b - a < box ? b - a : box;
    sum += (double)(need > 0 ? need : 0) / box;
  }
  return n > 0 ? sum / n : 1.0;
}

// max_query_span over the extents the axis takes in this call: the global extent, or every distinct sample
// extent of a variable-size batch (results are kept: the planner asks for the same few values again and again).
int query_span(const Geo& g, int a, int T) {
  static std::mutex mu;
  static std::map<std::vector<int>, int> memo;
  auto one = [&](int L) {
    const std::vector<int> key = {L, g.K[a], g.dl[a], T};
    std::lock_guard<std::mutex> lock(mu);
    auto it = memo.find(key);
    if (it != memo.end()) return it->second;
    if (memo.size() > 65536) memo.clear();
    const int v = max_query_span(L, g.K[a], g.dl[a], T);
    memo.emplace(key, v);
    return v;
  };
  const int lead = 3 - g.rank;
  if (g.host_extents == nullptr || a < lead) return one(g.ge[a]);
  int best = 0;
  for (int b = 0; b < g.B; ++b) {
    const int v = one(g.host_extents[b * g.rank + (a - lead)]);
    if (v > best) best = v;
  }
  return best;
}

// Best query tile for a cap of `nmax` S columns per chunk; returns the cost
// (tiles x chunks x padded columns) or -1 when nothing fits.
// A pinned tile shape and chunk-width cap for one geometry and kernel (plan_hint entry point); zeros pin nothing.
struct PlanHint {
  int tile[3];
  int max_cols;
};

long long choose_tile(const Geo& g, FwdParams& p, int nmax, int mode, const PlanHint& hint) {
  int lgmax[3];
  for (int a = 0; a < 3; ++a) lgmax[a] = ceil_div(g.ge[a], g.dl[a]);
  // row class entries on the leading axis that lie in the local slab (all of them when unsharded)
  int nloc0 = 0;
  for (int g0 = 0; g0 < g.dl[0]; ++g0) {
    const int n = slab_hi(p.ro0 + p.re0, g0, g.dl[0]) - slab_lo(p.ro0, g0, g.dl[0]);
    if (n > nloc0) nloc0 = n;
  }
  // extents of the tile grid (rows) and of the chunk operand, in their own coordinates
  int lrow[3], lchunk[3];
  for (int a = 0; a < 3; ++a) {
    lrow[a] = ceil_div(lgmax[a], p.rst[a]);
    lchunk[a] = ceil_div(lgmax[a], p.cst[a]);
  }
  if (p.rst[0] != 1) nloc0 = lrow[0];
  long long best_cost = -1;
  double best_visited = 1.0;
  int want[3] = {0, 0, 0};                       // a pinned tile shape (plan_hint)
  if (hint.tile[2] > 0) { want[0] = hint.tile[0]; want[1] = hint.tile[1]; want[2] = hint.tile[2]; }
  for (int t2 = 1; t2 <= p.P; t2 *= 2)
    for (int t1 = 1; t1 * t2 <= p.P; t1 *= 2) {
      const int t0 = p.P / (t1 * t2);
      const int T[3] = {t0, t1, t2};
      bool skip = want[2] > 0 && (t0 != want[0] || t1 != want[1] || t2 != want[2]);
      int box[3];
      for (int a = 0; a < 3; ++a) {
        if (lrow[a] == 1 && T[a] != 1) skip = true;          // nothing to tile on a trivial axis
        // keys a query tile addresses: T + K - 1; queries that address a key tile: more near the
        // ends of the axis (see max_query_span)
        int need = g.ca[a] == 2 ? g.ge[a] : (T[a] - 1) * p.rst[a] + g.K[a];
        if (mode == 2 && g.ca[a] == 0) need = query_span(g, a, T[a]);
        if (mode == 2 && p.cst[a] != 1) need = ceil_div(need, p.cst[a]) + 1;     // queries on the stride lattice
        box[a] = need < lchunk[a] ? need : lchunk[a];
        if (box[a] > 256) skip = true;                        // TMA box limit
      }
      if (skip) continue;
      // box rows of at most 32 keys are padded to 16 or 32 columns, so that a
      // 16-column group of S never straddles two box rows
      const int rp = box[2] <= 16 ? 16 : (box[2] <= 32 ? 32 : 0);
      if (rp != 0) box[2] = rp;
      int ca, R;
      const long long v2 = box[2], v1 = (long long)box[1] * box[2], v0 = (long long)box[0] * v1;
      if (v0 <= nmax) { ca = 0; R = box[0]; }
      else if (v1 <= nmax) { ca = 0; R = (int)(nmax / v1); }
      else if (v2 <= nmax) { ca = 1; R = (int)(nmax / v2); }
      else continue;
      const int inner = ca == 0 ? (int)v1 : (int)v2;
      const int cch = ceil_div(box[ca], R);
      R = ceil_div(box[ca], cch);                             // even out the chunks
      const int nch = (ca == 1 ? box[0] : 1) * cch;
      int n_pad = (R * inner + 15) & ~15;
      if (n_pad > 256) n_pad = (n_pad + 31) & ~31;
      if (n_pad > nmax) continue;
      long long tiles = 1;
      for (int a = 0; a < 3; ++a) tiles *= ceil_div(a == 0 ? nloc0 : lrow[a], T[a]);
      // box rows (axes 0 and 1) that no row of a tile needs are skipped by the elementwise warps:
      // among tile shapes of equal cost the one with the fewest visited rows wins
      double visited = 1.0;
      for (int a = 0; a < 2; ++a)
        if (g.ge[a] > 1 && g.ca[a] == 0 && box[a] > 1)
          visited *= mean_needed_fraction(g.ge[a], g.K[a], g.dl[a], T[a], box[a], mode != 2);
      // +96: fixed per-chunk overhead; boxes without row structure go through per-row bitmaps, which cost the
      // elementwise warps about half as much again
      const long long cost = tiles * nch * (n_pad + 96) * (rp == 0 ? 3 : 2) / 2;
      if (best_cost < 0 || cost < best_cost || (cost == best_cost && visited < best_visited - 1e-9)) {
        best_cost = cost;
        best_visited = visited;
        for (int a = 0; a < 3; ++a) { p.T[a] = T[a]; p.box[a] = box[a]; p.tiles[a] = ceil_div(a == 0 ? nloc0 : lrow[a], T[a]); }
        p.chunk_axis = ca; p.R = R; p.cchunks = cch; p.n_chunks = nch; p.inner = inner;
        p.n_cols = R * inner; p.n_pad = n_pad; p.rp = rp;
      }
    }
  return best_cost;
}

Plan make_plan_uncached(const Geo& g, int dtype, int mode, const PlanHint& hint) {
  Plan pl{};
  pl.ok = false;
  FwdParams base{};
  if (dtype != NATTEN_B200_BF16 && dtype != NATTEN_B200_F16) { pl.why = "dtype is not bf16/f16"; return pl; }
  if (g.D != 32 && g.D != 64 && g.D != 128) { pl.why = "head_dim is not 32, 64 or 128"; return pl; }
  if (g.extents != nullptr && g.host_extents == nullptr) { pl.why = "per-sample extents without a host copy"; return pl; }
  const bool varlen = g.extents != nullptr;
  if (varlen) {
    const int lead = 3 - g.rank;
    for (int b = 0; b < g.B; ++b)
      for (int a = 0; a < g.rank; ++a) {
        const int e = g.host_extents[b * g.rank + a];
        if (e > g.ge[lead + a] || (long long)g.K[lead + a] * g.dl[lead + a] > e) {
          pl.why = "a sample extent is larger than the tensors or smaller than kernel_size * dilation";
          return pl;
        }
      }
  }
  if (!(g.scale > 0.f)) { pl.why = "scale is not positive"; return pl; }
  int ncls = 1;
  for (int a = 0; a < 3; ++a) {
    if (g.st[a] != 1 && g.dl[a] != 1) { pl.why = "stride and dilation on the same axis"; return pl; }
    if ((g.qe[a] != g.ge[a] || g.ke[a] != g.ge[a] || g.qo[a] != 0 || g.ko[a] != 0) && (a != 0 || g.rank != 3)) {
      pl.why = "slab on an axis other than the leading axis of a 3-D volume";
      return pl;
    }
    if ((g.qe[a] != g.ge[a] || g.ke[a] != g.ge[a]) && g.n_extra != 0) { pl.why = "extra tokens with a slab"; return pl; }
    ncls *= g.dl[a];
  }
  if (ncls > kMaxClasses) { pl.why = "more than 16 dilation classes"; return pl; }
  if (varlen && (size_t)g.B * ncls * 4 * sizeof(CUtensorMap) > kMapSlotBytes) {
    pl.why = "more (sample, dilation class) pairs than the tensor-map ring holds";
    return pl;
  }
  const bool strided = g.st[0] * g.st[1] * g.st[2] != 1;
  if (strided && (varlen || g.n_extra != 0 || g.pitched)) { pl.why = "stride with per-sample extents, extra tokens or mem_extent"; return pl; }
  for (int a = 0; a < 3; ++a)
    if (strided && (g.qe[a] != g.ge[a] || g.ke[a] != g.ge[a])) { pl.why = "stride with a slab"; return pl; }
  base.B = g.B; base.Hq = g.Hq; base.Hkv = g.Hkv; base.rep = g.rep; base.D = g.D; base.rank = g.rank;
  for (int a = 0; a < 3; ++a) { base.L[a] = g.ge[a]; base.K[a] = g.K[a]; base.dl[a] = g.dl[a]; base.ca[a] = g.ca[a]; }
  {
    // rows are queries (forward, dQ) or keys (dK/dV); the chunk operands are the other side
    const bool rows_are_q = mode != 2;
    const bool slab = g.qe[0] != g.ge[0] || g.ke[0] != g.ge[0];
    for (int a = 0; a < 3; ++a) {
      base.Mr[a] = slab ? (rows_are_q ? g.qe[a] : g.ke[a]) : g.me[a];
      base.Mc[a] = slab ? (rows_are_q ? g.ke[a] : g.qe[a]) : g.me[a];
      base.Mq[a] = slab ? g.qe[a] : g.me[a];      // the query tensor's own extents
      base.rst[a] = rows_are_q ? g.st[a] : 1;
      base.cst[a] = rows_are_q ? 1 : g.st[a];
      if (strided) {       // the query-side index space is the output's
        if (rows_are_q) base.Mr[a] = g.out[a];
        else base.Mc[a] = g.out[a];
      }
    }
    base.strided = strided ? 1 : 0;
    base.ro0 = rows_are_q ? g.qo[0] : g.ko[0];
    base.re0 = rows_are_q ? g.qe[0] : g.ke[0];
    base.co0 = rows_are_q ? g.ko[0] : g.qo[0];
    base.ce0 = rows_are_q ? g.ke[0] : g.qe[0];
  }
  base.mode = mode;
  base.hpt = mode == 2 ? 1 : ((g.rep % 4 == 0) ? 4 : (g.rep % 2 == 0 ? 2 : 1));
  base.head_groups = mode == 2 ? 1 : g.rep / base.hpt;
  base.P = kTileM / base.hpt;
  base.dblk = g.D == 32 ? 32 : 64;
  base.ndblk = g.D / base.dblk;
  base.row_bytes = base.dblk * 2;
  base.layout_type = g.D == 32 ? 4 : 2;

  // Two CTAs per SM (256 TMEM columns and half the shared memory each) let one
  // CTA's MMA/TMA phases run under the other's softmax; one CTA per SM allows
  // larger chunks.  Every feasible (CTAs, column cap) pair is costed.
  double best = -1.0;
  static const int caps[] = {384, 320, 256, 224, 192, 160, 128, 96, 64, 48, 32};
  const int max_cols = hint.max_cols;                       // cap on the chunk width (plan_hint), 0 = none
  // registers per thread of the kernels cap the CTAs per SM: forward 2, dQ 4, dK/dV 2
  const int max_ctas = mode == 1 ? 4 : 2;
  static const double overlap[5] = {0.0, 1.0, 1.7, 2.3, 2.8};
  for (int ctas = max_ctas; ctas >= 1; --ctas) {
    const int tmem_cols = ctas >= 3 ? 128 : 512 / ctas;   // a power of two per CTA
    const size_t smem_limit = (size_t)(232448 / ctas) - 1024;
    for (int cap : caps) {
      if (cap > kMaxCols || (max_cols >= 32 && cap > max_cols)) continue;
      // forward: S/P ring (>= 2 buffers) and two O buffers; backward: one or two S+dP buffers
      // and single accumulators
      const int acc_cols = mode == 1 ? g.D : 2 * g.D;
      for (int nb = 2; nb >= (mode == 0 ? 2 : 1); --nb) {
        const int s_regions = mode == 0 ? nb : 2 * nb;
        if (cap * s_regions > tmem_cols - acc_cols) continue;
        FwdParams p = base;
        const long long cost = choose_tile(g, p, cap, mode, hint);
        if (cost < 0) continue;
        p.q_stages = 2; p.kv_stages = 4; p.n_sbuf = nb;   // backward: up to four chunk-operand stages
        if (mode == 0) {
          // as many S/P buffers as tensor memory holds (a warp with little work in a chunk runs
          // ahead of the others by up to n_sbuf - 1 chunks), one more K/V stage than that
          p.n_sbuf = (tmem_cols - acc_cols) / p.n_pad;
          if (p.n_sbuf > 6) p.n_sbuf = 6;
          p.kv_stages = p.n_sbuf + 1 > 6 ? 6 : p.n_sbuf + 1;
        }

        while (p.kv_stages > 2 && smem_needed(p) > smem_limit) --p.kv_stages;
        if (smem_needed(p) > smem_limit) p.q_stages = 1;
        if (smem_needed(p) > smem_limit) continue;           // a single chunk stage would lose the prefetch
        // a second S+dP buffer hides the tensor-core round trip of a chunk
        const double eff = (double)cost / overlap[ctas] * (mode != 0 && nb == 1 ? 1.25 : 1.0);
        if (best < 0 || eff < best) {
          best = eff;
          p.ctas_per_sm = ctas; p.tmem_cols = tmem_cols; p.ocol = tmem_cols - 2 * g.D;
          p.dp_col = p.n_pad; p.acc_col = tmem_cols - acc_cols; p.acc2_col = tmem_cols - g.D;
          pl.p = p;
        }
      }
    }
  }
  if (best < 0) { pl.why = "no tile shape fits the key box into tensor and shared memory"; return pl; }
  FwdParams& p = pl.p;
  p.n_split = p.n_pad > 256 ? 2 : 1;
  p.n_half = p.n_pad / p.n_split;
  pl.smem = smem_needed(p);
  long long n_work = (long long)g.B * g.Hkv * p.head_groups * ncls * p.tiles[0] * p.tiles[1] * p.tiles[2];
  p.n_work_main = n_work;
  p.n_extra = g.n_extra;
  p.xw = p.n_xchunks = p.n_xtiles = 0;
  p.xr[0] = p.xr[1] = p.xr[2] = 1;
  if (g.n_extra > 0) {
    // forward / dQ: the extra tokens follow the key box as chunks of xw tokens (one TMA box: at most 256 rows)
    p.xw = p.n_pad < 256 ? p.n_pad : 256;
    p.n_xchunks = ceil_div(g.n_extra, p.xw);
    if (mode != 2) {
      p.xw = (ceil_div(g.n_extra, p.n_xchunks) + 15) & ~15;     // even out the chunks
    } else {
      // dK/dV: tiles of 128 extra tokens, each walking every box of every dilation class's queries
      p.n_xchunks = 0;
      p.n_xtiles = ceil_div(g.n_extra, kTileM);
      long long regions = 1;
      for (int a = 0; a < 3; ++a) {
        p.xr[a] = ceil_div(ceil_div(g.ge[a], g.dl[a]), p.box[a]);
        regions *= p.xr[a];
      }
      n_work += (long long)g.B * g.Hkv * p.n_xtiles * ncls * regions;
    }
  }
  if (n_work >= (1LL << 31)) { pl.why = "more than 2^31 tiles"; return pl; }
  p.n_work = n_work;
  p.scale_log2 = g.scale * 1.4426950408889634f;
  p.is_bf16 = dtype == NATTEN_B200_BF16;
  const int fmt = p.is_bf16 ? 1 : 0;
  p.idesc_qk = instr_desc(kTileM, p.n_half, fmt, 0, 0);
  p.idesc_pv = instr_desc(kTileM, g.D, fmt, 0, 1);
  pl.ok = true;
  pl.why = "";
  return pl;
}

// Plans depend on the geometry only; building one walks tile shapes, chunk widths and (for the
// dK/dV kernel) every key tile of every axis, which costs the host far more than a launch.
std::vector<int> plan_key(const Geo& g, int dtype, int mode) {
  std::vector<int> key = {dtype, mode, g.B, g.Hq, g.Hkv, g.D, g.rank, g.n_extra, g.extents != nullptr ? 1 : 0};
  int scale_bits;
  memcpy(&scale_bits, &g.scale, sizeof(int));
  key.push_back(scale_bits);
  for (int a = 0; a < 3; ++a)
    for (int v : {g.qe[a], g.ke[a], g.ge[a], g.me[a], g.qo[a], g.ko[a], g.K[a], g.st[a], g.dl[a], g.ca[a]}) key.push_back(v);
  key.push_back(g.host_extents != nullptr ? 1 : 0);
  if (g.extents != nullptr && g.host_extents != nullptr)   // the dK/dV query box depends on the sample extents
    for (int i = 0; i < g.B * g.rank; ++i) key.push_back(g.host_extents[i]);
  return key;
}

std::mutex g_plan_mu;
std::map<std::vector<int>, Plan> g_plan_cache;
std::map<std::vector<int>, PlanHint> g_plan_hints;

Plan make_plan(const Geo& g, int dtype, int mode = 0) {
  std::vector<int> key = plan_key(g, dtype, mode);
  std::lock_guard<std::mutex> lock(g_plan_mu);
  PlanHint hint{{0, 0, 0}, 0};
  auto h = g_plan_hints.find(key);
  if (h != g_plan_hints.end()) hint = h->second;
  auto it = g_plan_cache.find(key);
  if (it != g_plan_cache.end()) return it->second;
  if (g_plan_cache.size() > 4096) g_plan_cache.clear();   // many distinct per-sample sizes: start over rather than grow
  const Plan pl = make_plan_uncached(g, dtype, mode, hint);
  g_plan_cache.emplace(std::move(key), pl);
  return pl;
}

// Pins (or with zeros releases) the tile shape and chunk-width cap of one geometry and kernel.
int plan_hint_impl(const Geo& g, int dtype, int mode, const int tile[3], int max_cols) {
  const std::vector<int> key = plan_key(g, dtype, mode);
  PlanHint hint{{tile[0], tile[1], tile[2]}, max_cols};
  {
    std::lock_guard<std::mutex> lock(g_plan_mu);
    if (hint.tile[2] <= 0 && hint.max_cols <= 0) g_plan_hints.erase(key);
    else g_plan_hints[key] = hint;
    g_plan_cache.erase(key);
  }
  const Plan pl = make_plan(g, dtype, mode);
  if (!pl.ok) {
    std::lock_guard<std::mutex> lock(g_plan_mu);
    g_plan_hints.erase(key);
    g_plan_cache.erase(key);
    return set_error(NATTEN_B200_EINVAL, "plan_hint: no plan with this tile shape and chunk width: %s", pl.why);
  }
  return NATTEN_B200_OK;
}

// ---------------------------------------------------------------------------
// host: tensor maps
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    else
      (void)cudaGetLastError();
  });
  return fn;
}

// One map per dilation class for a [B, spatial..., heads, D] tensor.
// dims: (heads*D, axis rank-1, ..., axis 0, B); box_sp[a] is the box extent on
// normalised axis a (leading trivial axes of lower-rank tensors are skipped).
// `chunk_side`: the tensor is a chunk operand (its own slab range and strides) rather than a row operand.
// `mem_ext`, `step` and `div` describe tensors of the query side when the queries sit on a stride lattice: the
// extents behind the memory strides (default: Mr / Mc), the element step per axis on top of the dilation (the
// stride for the query tensor, which is laid out over positions) and the divisor of the class length (the stride:
// one entry per lattice point).
int encode_class_maps(CUtensorMap* maps, const void* base, const FwdParams& p, int heads, const int box_sp[3],
                      bool chunk_side = false, const int* mem_ext = nullptr, const int* step = nullptr,
                      const int* div = nullptr) {
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return set_error(NATTEN_B200_ENODEVICE, "cuTensorMapEncodeTiled is not available");
  const int lead = 3 - p.rank;
  const cuuint32_t trank = (cuuint32_t)(p.rank + 2);
  const int* ext = mem_ext != nullptr ? mem_ext : (chunk_side ? p.Mc : p.Mr);
  const int first0 = chunk_side ? p.co0 : p.ro0, count0 = chunk_side ? p.ce0 : p.re0;
  static const int ones[3] = {1, 1, 1};
  if (step == nullptr) step = ones;
  if (div == nullptr) div = ones;
  long long stride_el[3];  // elements between consecutive coordinates on each axis
  long long s = (long long)heads * p.D;
  for (int a = 2; a >= 0; --a) { stride_el[a] = s; s *= ext[a]; }
  const long long batch_el = s;
  int ci = 0;
  for (int g0 = 0; g0 < p.dl[0]; ++g0)
    for (int g1 = 0; g1 < p.dl[1]; ++g1)
      for (int g2 = 0; g2 < p.dl[2]; ++g2, ++ci) {
        const int gcls[3] = {g0, g1, g2};
        cuuint64_t dims[5];
        cuuint64_t strides[4];
        cuuint32_t box[5], estr[5] = {1, 1, 1, 1, 1};
        long long off = 0;
        dims[0] = (cuuint64_t)heads * p.D;
        box[0] = (cuuint32_t)p.dblk;
        int di = 1;
        for (int a = 2; a >= lead; --a, ++di) {
          long long n = ceil_div(ceil_div(p.L[a] - gcls[a], p.dl[a]), div[a]);
          long long first_plane = gcls[a];              // local plane of the class's first entry
          if (a == 0 && !p.strided) {                   // leading axis: only the entries inside the local planes
            const int lo = slab_lo(first0, g0, p.dl[0]), hi = slab_hi(first0 + count0, g0, p.dl[0]);
            n = hi - lo;
            first_plane = (long long)lo * p.dl[0] + g0 - first0;
            if (n <= 0) { n = 1; first_plane = 0; }     // a class without local entries: its tiles are dead
          }
          dims[di] = (cuuint64_t)n;
          strides[di - 1] = (cuuint64_t)(stride_el[a] * p.dl[a] * step[a] * 2);
          box[di] = (cuuint32_t)box_sp[a];
          off += first_plane * stride_el[a];
        }
        dims[di] = (cuuint64_t)p.B;
        strides[di - 1] = (cuuint64_t)(batch_el * 2);
        box[di] = 1;
        void* ptr = const_cast<char*>(static_cast<const char*>(base)) + off * 2;
        const CUresult r = enc(&maps[ci], p.is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                               trank, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               p.D == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return set_error(NATTEN_B200_ELAUNCH, "cuTensorMapEncodeTiled failed with code %d", (int)r);
      }
  return 0;
}

// Map of the extra tokens [B, N_extra, Hkv, D]: dims (Hkv * D, N_extra, B), box (dblk, rows, 1).  Rows past N_extra
// read as zeros.
int encode_extra_map(CUtensorMap* map, const void* base, const FwdParams& p, int heads, int n_extra, int rows) {
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return set_error(NATTEN_B200_ENODEVICE, "cuTensorMapEncodeTiled is not available");
  cuuint64_t dims[3] = {(cuuint64_t)heads * p.D, (cuuint64_t)n_extra, (cuuint64_t)p.B};
  cuuint64_t strides[2] = {(cuuint64_t)heads * p.D * 2, (cuuint64_t)n_extra * heads * p.D * 2};
  cuuint32_t box[3] = {(cuuint32_t)p.dblk, (cuuint32_t)rows, 1}, estr[3] = {1, 1, 1};
  const CUresult r = enc(map, p.is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         p.D == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(NATTEN_B200_ELAUNCH, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return 0;
}

// Variable-size batch: the class maps of one tensor for every sample, each with the sample's own bounds (strides
// stay those of the padded tensor), written to out[(b * ncls + cls) * nmaps + which].
int encode_sample_maps(std::vector<CUtensorMap>& out, int nmaps, int which, const void* base, const FwdParams& p, int heads,
                       const int box_sp[3], bool chunk_side, const int* host_extents) {
  int ncls = p.dl[0] * p.dl[1] * p.dl[2];
  const int lead = 3 - p.rank;
  const int* ext = chunk_side ? p.Mc : p.Mr;
  const long long batch_el = (long long)heads * p.D * ext[0] * ext[1] * ext[2];
  CUtensorMap tmp[kMaxClasses];
  for (int b = 0; b < p.B; ++b) {
    FwdParams pb = p;
    pb.B = 1;
    for (int a = 0; a < p.rank; ++a) pb.L[lead + a] = host_extents[b * p.rank + a];
    pb.ro0 = pb.co0 = 0;
    pb.re0 = pb.ce0 = pb.L[0];
    const char* sample = static_cast<const char*>(base) + (long long)b * batch_el * 2;
    if (int rc = encode_class_maps(tmp, sample, pb, heads, box_sp, chunk_side)) return rc;
    for (int c = 0; c < ncls; ++c) out[((size_t)b * ncls + c) * nmaps + which] = tmp[c];
  }
  return 0;
}

}  // namespace
}  // namespace nb

#include "fna_sm100_fwd_kernel.inc"
#include "fna_sm100_bwd_kernel.inc"
#include "fna_sm100_host.inc"

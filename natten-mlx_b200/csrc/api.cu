// C ABI of the library: argument checking, geometry normalisation and the
// choice between the CUDA-core and the tensor-core kernel families.
#include <stdarg.h>
#include <stdio.h>

#include <string.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "launch.cuh"
#include "fna_sm100.cuh"

#include <stddef.h>

// The ctypes mirror of the geometry struct relies on this layout.
static_assert(sizeof(natten_b200_geom) == 176, "natten_b200_geom layout changed");
static_assert(offsetof(natten_b200_geom, host_extents) == 168, "natten_b200_geom layout changed");
static_assert(offsetof(natten_b200_geom, mem_extent) == 152, "natten_b200_geom layout changed");
static_assert(offsetof(natten_b200_geom, scale) == 132, "natten_b200_geom layout changed");
static_assert(offsetof(natten_b200_geom, extents) == 144, "natten_b200_geom layout changed");

namespace nb {

static thread_local char g_error[512] = "";
static thread_local const char* g_path = "none";
static std::atomic<uint64_t> g_launches{0};

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return NATTEN_B200_OK;
  return set_error(NATTEN_B200_ELAUNCH, "%s: %s", what, cudaGetErrorString(e));
}

void set_last_path(const char* name) { g_path = name; }

// ---- per-kernel device timing (off by default) -----------------------------
namespace {
struct TraceSlot {
  const char* name;
  cudaEvent_t start, stop;
};
std::mutex g_trace_mutex;
std::atomic<int> g_trace_on{0};
std::vector<TraceSlot> g_trace;       // slots recorded since the last report
std::vector<TraceSlot> g_trace_pool;  // events kept for reuse
}  // namespace

LaunchScope::LaunchScope(const char* name, cudaStream_t stream) : stream_(stream), slot_(-1) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (!g_trace_on.load(std::memory_order_relaxed)) return;
  std::lock_guard<std::mutex> lock(g_trace_mutex);
  TraceSlot t{};
  if (!g_trace_pool.empty()) {
    t = g_trace_pool.back();
    g_trace_pool.pop_back();
  } else if (cudaEventCreate(&t.start) != cudaSuccess || cudaEventCreate(&t.stop) != cudaSuccess) {
    (void)cudaGetLastError();
    return;
  }
  t.name = name;
  cudaEventRecord(t.start, stream);
  g_trace.push_back(t);
  slot_ = (int)g_trace.size() - 1;
}

LaunchScope::~LaunchScope() {
  if (slot_ < 0) return;
  std::lock_guard<std::mutex> lock(g_trace_mutex);
  if (slot_ < (int)g_trace.size()) cudaEventRecord(g_trace[slot_].stop, stream_);
}

int make_geo(const natten_b200_geom* in, Geo* g) {
  if (in == nullptr) return set_error(NATTEN_B200_EINVAL, "geometry is null");
  if (in->rank < 1 || in->rank > 3) return set_error(NATTEN_B200_EINVAL, "rank must be 1, 2 or 3, got %d", in->rank);
  if (in->batch < 1 || in->heads_q < 1 || in->heads_kv < 1 || in->head_dim < 1)
    return set_error(NATTEN_B200_EINVAL, "batch, heads and head_dim must be positive");
  if (in->heads_q % in->heads_kv != 0)
    return set_error(NATTEN_B200_EINVAL, "heads_q (%d) must be divisible by heads_kv (%d)", in->heads_q, in->heads_kv);
  if (in->dtype < NATTEN_B200_F32 || in->dtype > NATTEN_B200_BF16)
    return set_error(NATTEN_B200_EINVAL, "unsupported dtype %d", in->dtype);
  if (in->n_extra < 0) return set_error(NATTEN_B200_EINVAL, "n_extra must be >= 0");
  g->B = in->batch; g->Hq = in->heads_q; g->Hkv = in->heads_kv; g->rep = in->heads_q / in->heads_kv;
  g->D = in->head_dim; g->rank = in->rank; g->scale = in->scale; g->n_extra = in->n_extra;
  g->extents = in->extents;
  g->host_extents = in->extents != nullptr ? in->host_extents : nullptr;
  const int lead = 3 - in->rank;
  for (int a = 0; a < 3; ++a) {
    g->qe[a] = g->ke[a] = g->ge[a] = 1;
    g->qo[a] = g->ko[a] = 0;
    g->K[a] = g->st[a] = g->dl[a] = 1;
    g->ca[a] = 0;
  }
  bool sharded = false;
  g->pitched = false;
  for (int i = 0; i < in->rank; ++i) g->pitched = g->pitched || in->mem_extent[i] != 0;
  for (int i = 0; i < in->rank; ++i) {
    const int a = lead + i;
    g->qe[a] = in->q_extent[i]; g->ke[a] = in->kv_extent[i]; g->ge[a] = in->global_extent[i];
    g->qo[a] = in->q_offset[i]; g->ko[a] = in->kv_offset[i];
    g->K[a] = in->kernel[i]; g->st[a] = in->stride[i]; g->dl[a] = in->dilation[i];
    g->ca[a] = in->causal[i];
    if (g->ca[a] < 0 || g->ca[a] > 2) return set_error(NATTEN_B200_EINVAL, "causal[%d] must be 0, 1 or 2", i);
    if (g->ca[a] == 2 && (in->kernel[i] != in->global_extent[i] || in->dilation[i] != 1 || in->stride[i] != 1 ||
                          in->extents != nullptr))
      return set_error(NATTEN_B200_EINVAL, "causal[%d] == 2 (whole axis) needs kernel == extent, dilation 1, stride 1", i);
    if (g->qe[a] < 1 || g->ke[a] < 1 || g->ge[a] < 1)
      return set_error(NATTEN_B200_EINVAL, "axis %d: extents must be positive", i);
    if (g->K[a] < 1) return set_error(NATTEN_B200_EINVAL, "kernel_size[%d] must be positive, got %d", i, g->K[a]);
    if (g->st[a] < 1 || g->st[a] > g->K[a])
      return set_error(NATTEN_B200_EINVAL, "stride[%d]=%d must be in [1, kernel_size[%d]=%d]", i, g->st[a], i, g->K[a]);
    if (g->dl[a] < 1) return set_error(NATTEN_B200_EINVAL, "dilation[%d] must be positive", i);
    if (g->K[a] > g->ge[a])
      return set_error(NATTEN_B200_EINVAL, "kernel_size[%d]=%d must be <= input spatial size %d", i, g->K[a], g->ge[a]);
    if ((long long)g->K[a] * g->dl[a] > g->ge[a])
      return set_error(NATTEN_B200_EINVAL, "dilation[%d] * kernel_size[%d] = %d exceeds input size %d", i, i,
                       g->K[a] * g->dl[a], g->ge[a]);
    if (g->qo[a] < 0 || g->ko[a] < 0 || g->qo[a] + g->qe[a] > g->ge[a] || g->ko[a] + g->ke[a] > g->ge[a])
      return set_error(NATTEN_B200_EINVAL, "axis %d: slab lies outside the global extent", i);
    if (g->qo[a] % g->st[a] != 0)
      return set_error(NATTEN_B200_EINVAL, "axis %d: q_offset must be a multiple of the stride", i);
    if (g->qe[a] != g->ge[a] || g->ke[a] != g->ge[a]) {
      sharded = true;
      // every key a local query can address must be inside the local key slab
      for (int p = g->qo[a]; p < g->qo[a] + g->qe[a]; p += g->st[a]) {
        int start, hi;
        axis_window(p, g->ge[a], g->K[a], g->dl[a], g->ca[a], start, hi);
        const int lo = start < 0 ? (start % g->dl[a] + g->dl[a]) % g->dl[a] : start;
        if (lo >= hi) continue;
        const int last = lo + ((hi - 1 - lo) / g->dl[a]) * g->dl[a];  // last key on the window's lattice
        if (lo < g->ko[a] || last >= g->ko[a] + g->ke[a])
          return set_error(NATTEN_B200_EINVAL,
                           "axis %d: query %d needs keys [%d, %d] but the local key slab is [%d, %d)", i, p, lo, last,
                           g->ko[a], g->ko[a] + g->ke[a]);
      }
    }
  }
  if (sharded && in->extents != nullptr)
    return set_error(NATTEN_B200_EINVAL, "per-sample extents cannot be combined with a sharded slab");
  for (int a = 0; a < 3; ++a) g->me[a] = g->ge[a];
  if (g->pitched) {
    if (sharded || in->extents != nullptr || in->n_extra != 0)
      return set_error(NATTEN_B200_EINVAL, "mem_extent cannot be combined with slabs, per-sample extents or extra tokens");
    for (int i = 0; i < in->rank; ++i) {
      if (in->mem_extent[i] < in->global_extent[i])
        return set_error(NATTEN_B200_EINVAL, "mem_extent[%d]=%d is smaller than the extent %d", i, in->mem_extent[i],
                         in->global_extent[i]);
      if (in->stride[i] != 1) return set_error(NATTEN_B200_EINVAL, "mem_extent needs stride 1");
      g->me[lead + i] = in->mem_extent[i];
    }
  }
  long long n_out = 1, n_q = 1, n_kv = 1, kvol = 1;
  for (int a = 0; a < 3; ++a) {
    g->out[a] = (g->qe[a] + g->st[a] - 1) / g->st[a];
    n_out *= g->out[a]; n_q *= g->qe[a]; n_kv *= g->ke[a]; kvol *= g->K[a];
  }
  g->n_out = n_out; g->n_q = n_q; g->n_kv = n_kv;
  if (kvol > (1 << 20)) return set_error(NATTEN_B200_EINVAL, "kernel volume %lld is too large", kvol);
  g->kvol = (int)kvol;
  const long long lim = 0x7fffffffLL;
  if (g->B * n_q * g->Hq > lim || g->B * n_kv * g->Hkv > lim || g->B * n_out * g->Hq > lim ||
      (long long)g->B * g->me[0] * g->me[1] * g->me[2] * g->Hq > lim)
    return set_error(NATTEN_B200_EINVAL, "problem has more than 2^31 rows");
  return NATTEN_B200_OK;
}

static bool any_null(std::initializer_list<const void*> ptrs) {
  for (const void* p : ptrs)
    if (p == nullptr) return true;
  return false;
}

// The kernels read and write rows through 16-byte vector accesses and TMA tensor maps, both of
// which need 16-byte aligned base addresses (null pointers of optional tensors pass).
static bool any_misaligned(std::initializer_list<const void*> ptrs) {
  for (const void* p : ptrs)
    if ((reinterpret_cast<uintptr_t>(p) & 15u) != 0) return true;
  return false;
}
static int reject_misaligned(const char* what) {
  return set_error(NATTEN_B200_EINVAL, "%s: tensor pointers must be 16-byte aligned", what);
}

}  // namespace nb

using namespace nb;

extern "C" {

int natten_b200_abi_version(void) { return NATTEN_B200_ABI_VERSION; }
const char* natten_b200_last_error(void) { return g_error; }
const char* natten_b200_last_path(void) { return g_path; }
uint64_t natten_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

void natten_b200_trace_enable(int on) { g_trace_on.store(on ? 1 : 0, std::memory_order_relaxed); }

size_t natten_b200_trace_report(char* buf, size_t cap) {
  std::lock_guard<std::mutex> lock(g_trace_mutex);
  std::map<std::string, std::pair<long long, double>> agg;
  for (TraceSlot& t : g_trace) {
    float ms = 0.f;
    if (cudaEventSynchronize(t.stop) == cudaSuccess && cudaEventElapsedTime(&ms, t.start, t.stop) == cudaSuccess) {
      auto& e = agg[t.name];
      e.first += 1;
      e.second += ms;
    } else {
      (void)cudaGetLastError();
    }
    g_trace_pool.push_back(t);
  }
  g_trace.clear();
  std::string out;
  char line[160];
  for (const auto& kv : agg) {
    snprintf(line, sizeof(line), "%s %lld %.6f\n", kv.first.c_str(), kv.second.first, kv.second.second);
    out += line;
  }
  if (buf != nullptr && cap > 0) {
    const size_t n = out.size() < cap - 1 ? out.size() : cap - 1;
    memcpy(buf, out.data(), n);
    buf[n] = '\0';
  }
  return out.size() + 1;
}

int natten_b200_axis_table(int32_t length, int32_t kernel, int32_t dilation, int32_t stride,
                           int32_t causal, int32_t* idx, uint8_t* valid, int32_t* start_out,
                           int32_t* pb) {
  if (length < 1 || kernel < 1 || dilation < 1 || stride < 1 || idx == nullptr || valid == nullptr)
    return set_error(NATTEN_B200_EINVAL, "axis_table: bad arguments");
  const int n = (length + stride - 1) / stride;
  for (int j = 0; j < n; ++j) {
    const int p = j * stride;
    int start, hi;
    axis_window(p, length, kernel, dilation, causal, start, hi);
    for (int s = 0; s < kernel; ++s) {
      const int raw = start + s * dilation;
      valid[j * kernel + s] = (raw >= 0 && raw < hi) ? 1 : 0;
      idx[j * kernel + s] = raw < 0 ? 0 : (raw > length - 1 ? length - 1 : raw);
    }
    if (start_out != nullptr) start_out[j] = start;
    if (pb != nullptr) pb[j] = pb_start(p, length, kernel, dilation);
  }
  return NATTEN_B200_OK;
}

static int reject_pitched(const Geo& g, const char* what) {
  return g.pitched ? set_error(NATTEN_B200_EINVAL, "%s: mem_extent is only taken by the fused entry points", what)
                   : NATTEN_B200_OK;
}

int natten_b200_qk_forward(const natten_b200_geom* gi, const void* q, const void* k,
                           const float* bias, void* logits, void* stream) {
  Geo g;
  if (int rc = make_geo(gi, &g)) return rc;
  if (int rc = reject_pitched(g, "qk_forward")) return rc;
  if (any_null({q, k, logits})) return set_error(NATTEN_B200_EINVAL, "qk_forward: null tensor");
  if (any_misaligned({q, k, logits})) return reject_misaligned("qk_forward");
  if (bias != nullptr) {
    for (int a = 0; a < 3; ++a)
      if (g.st[a] != 1 || g.ca[a]) return set_error(NATTEN_B200_EINVAL, "bias requires stride 1 and no causal axis");
  }
  return run_split(SplitOp::QkForward, g, gi->dtype, q, k, nullptr, bias, logits, nullptr, nullptr, (cudaStream_t)stream);
}

int natten_b200_qk_backward(const natten_b200_geom* gi, const void* q, const void* k,
                            const void* dlogits, void* dq, void* dk, float* dbias, void* stream) {
  Geo g;
  if (int rc = make_geo(gi, &g)) return rc;
  if (int rc = reject_pitched(g, "qk_backward")) return rc;
  if (any_null({q, k, dlogits, dq, dk})) return set_error(NATTEN_B200_EINVAL, "qk_backward: null tensor");
  if (any_misaligned({q, k, dlogits, dq, dk})) return reject_misaligned("qk_backward");
  return run_split(SplitOp::QkBackward, g, gi->dtype, q, k, dlogits, nullptr, dq, dk, dbias, (cudaStream_t)stream);
}

int natten_b200_qk_bias_av_forward(const natten_b200_geom* gi, const void* q, const void* k, const void* v,
                                   const float* bias, void* out, float* lse, void* stream) {
  Geo g;
  if (int rc = make_geo(gi, &g)) return rc;
  if (int rc = reject_pitched(g, "qk_bias_av_forward")) return rc;
  if (any_null({q, k, v, out})) return set_error(NATTEN_B200_EINVAL, "qk_bias_av_forward: null tensor");
  if (any_misaligned({q, k, v, out})) return reject_misaligned("qk_bias_av_forward");
  if (bias != nullptr) {
    for (int a = 0; a < 3; ++a)
      if (g.st[a] != 1 || g.ca[a]) return set_error(NATTEN_B200_EINVAL, "bias requires stride 1 and no causal axis");
  }
  if (!run_fused_rows(g, gi->dtype, q, k, v, bias, out, lse, (cudaStream_t)stream))
    return set_error(NATTEN_B200_EINVAL, "qk_bias_av_forward: head_dim %d is not served by the row kernels (8, 12 (float32), 16, 24, 32)",
                     g.D);
  return check_launch("qk_bias_av_forward");
}

int natten_b200_av_forward(const natten_b200_geom* gi, const void* attn, const void* v, void* out,
                           void* stream) {
  Geo g;
  if (int rc = make_geo(gi, &g)) return rc;
  if (int rc = reject_pitched(g, "av_forward")) return rc;
  if (any_null({attn, v, out})) return set_error(NATTEN_B200_EINVAL, "av_forward: null tensor");
  if (any_misaligned({attn, v, out})) return reject_misaligned("av_forward");
  return run_split(SplitOp::AvForward, g, gi->dtype, attn, v, nullptr, nullptr, out, nullptr, nullptr, (cudaStream_t)stream);
}

int natten_b200_av_backward(const natten_b200_geom* gi, const void* attn, const void* v,
                            const void* dout, void* dattn, void* dv, void* stream) {
  Geo g;
  if (int rc = make_geo(gi, &g)) return rc;
  if (int rc = reject_pitched(g, "av_backward")) return rc;
  if (any_null({attn, v, dout, dattn, dv})) return set_error(NATTEN_B200_EINVAL, "av_backward: null tensor");
  if (any_misaligned({attn, v, dout, dattn, dv})) return reject_misaligned("av_backward");
  return run_split(SplitOp::AvBackward, g, gi->dtype, attn, v, dout, nullptr, dattn, dv, nullptr, (cudaStream_t)stream);
}

int natten_b200_fused_forward(const natten_b200_geom* gi, const void* q, const void* k,
                              const void* v, const void* k_extra, const void* v_extra, void* out,
                              float* lse, void* stream) {
  Geo g;
  if (int rc = make_geo(gi, &g)) return rc;
  if (any_null({q, k, v, out})) return set_error(NATTEN_B200_EINVAL, "fused_forward: null tensor");
  if (any_misaligned({q, k, v, out, k_extra, v_extra})) return reject_misaligned("fused_forward");
  if (g.n_extra > 0 && any_null({k_extra, v_extra}))
    return set_error(NATTEN_B200_EINVAL, "fused_forward: n_extra > 0 needs k_extra and v_extra");
  FusedArgs a{};
  a.q = q; a.k = k; a.v = v; a.k_extra = k_extra; a.v_extra = v_extra; a.out = out; a.lse = lse;
  const bool tc = gi->path != NATTEN_B200_PATH_SIMT && sm100_forward_supported(g, gi->dtype);
  if (gi->path == NATTEN_B200_PATH_TCGEN05 && !tc)
    return set_error(NATTEN_B200_EINVAL, "fused_forward: shape not supported by the tcgen05 kernels: %s",
                     sm100_unsupported_reason(g, gi->dtype));
  if (tc) {
    set_last_path("tcgen05");
    return run_fused_forward_sm100(g, gi->dtype, a, (cudaStream_t)stream);
  }
  if (g.pitched)
    return set_error(NATTEN_B200_EINVAL, "fused_forward: mem_extent needs the tensor-core kernels, which do not take this shape: %s",
                     sm100_unsupported_reason(g, gi->dtype));
  set_last_path("simt");
  return run_fused_forward_simt(g, gi->dtype, a, (cudaStream_t)stream);
}

size_t natten_b200_fused_backward_scratch_bytes(const natten_b200_geom* gi) {
  Geo g;
  if (make_geo(gi, &g)) return 0;
  size_t n = fused_backward_scratch_simt(g);
  const size_t m = fused_backward_scratch_sm100(g, gi->dtype);
  return n > m ? n : m;
}

int natten_b200_fused_backward(const natten_b200_geom* gi, const void* q, const void* k,
                               const void* v, const void* k_extra, const void* v_extra,
                               const void* out, const float* lse, const void* dout,
                               const float* dlse, void* dq, void* dk, void* dv, void* dk_extra,
                               void* dv_extra, void* scratch, size_t scratch_bytes, void* stream) {
  Geo g;
  if (int rc = make_geo(gi, &g)) return rc;
  if (any_null({q, k, v, out, lse, dout, dq, dk, dv, scratch}))
    return set_error(NATTEN_B200_EINVAL, "fused_backward: null tensor");
  if (any_misaligned({q, k, v, out, dout, dq, dk, dv, k_extra, v_extra, dk_extra, dv_extra, scratch}))
    return reject_misaligned("fused_backward");
  if (g.n_extra > 0 && any_null({k_extra, v_extra, dk_extra, dv_extra}))
    return set_error(NATTEN_B200_EINVAL, "fused_backward: n_extra > 0 needs the extra-token tensors");
  if (scratch_bytes < natten_b200_fused_backward_scratch_bytes(gi))
    return set_error(NATTEN_B200_ERESOURCE, "fused_backward: scratch has %zu bytes, needs %zu", scratch_bytes,
                     natten_b200_fused_backward_scratch_bytes(gi));
  FusedArgs a{};
  a.q = q; a.k = k; a.v = v; a.k_extra = k_extra; a.v_extra = v_extra;
  a.out = const_cast<void*>(out); a.lse = const_cast<float*>(lse); a.dout = dout; a.dlse = dlse;
  a.dq = dq; a.dk = dk; a.dv = dv; a.dk_extra = dk_extra; a.dv_extra = dv_extra;
  a.scratch = scratch; a.scratch_bytes = scratch_bytes;
  const bool tc = gi->path != NATTEN_B200_PATH_SIMT && sm100_backward_supported(g, gi->dtype);
  if (gi->path == NATTEN_B200_PATH_TCGEN05 && !tc)
    return set_error(NATTEN_B200_EINVAL, "fused_backward: shape not supported by the tcgen05 kernels: %s",
                     sm100_unsupported_reason(g, gi->dtype));
  if (tc) {
    set_last_path("tcgen05");
    return run_fused_backward_sm100(g, gi->dtype, a, (cudaStream_t)stream);
  }
  if (g.pitched)
    return set_error(NATTEN_B200_EINVAL, "fused_backward: mem_extent needs the tensor-core kernels, which do not take this shape: %s",
                     sm100_unsupported_reason(g, gi->dtype));
  set_last_path("simt");
  return run_fused_backward_simt(g, gi->dtype, a, (cudaStream_t)stream);
}

int natten_b200_fused_backward_halo(const natten_b200_geom* gi, const void* q, const void* k,
                                    const void* v, const void* out, const float* lse, const void* dout,
                                    const float* dlse, void* dq, void* dk, void* dv, void* scratch,
                                    size_t scratch_bytes, const natten_b200_halo_out* halo, void* stream) {
  Geo g;
  if (int rc = make_geo(gi, &g)) return rc;
  if (halo == nullptr) return set_error(NATTEN_B200_EINVAL, "fused_backward_halo: halo is null");
  if (any_null({q, k, v, out, lse, dout, dq, dk, dv, scratch}))
    return set_error(NATTEN_B200_EINVAL, "fused_backward_halo: null tensor");
  if (any_misaligned({q, k, v, out, dout, dq, dk, dv, scratch, halo->dk_below, halo->dv_below, halo->dk_above, halo->dv_above}))
    return reject_misaligned("fused_backward_halo");
  if (g.n_extra != 0 || g.extents != nullptr)
    return set_error(NATTEN_B200_EINVAL, "fused_backward_halo: extra tokens and per-sample extents are not supported");
  if (g.rank != 3 || halo->planes_below < 0 || halo->planes_above < 0 || halo->planes_below + halo->planes_above > g.ke[0])
    return set_error(NATTEN_B200_EINVAL, "fused_backward_halo: needs a 3-D slab whose K/V planes include the halo planes");
  if ((halo->planes_below > 0 && any_null({halo->dk_below, halo->dv_below})) ||
      (halo->planes_above > 0 && any_null({halo->dk_above, halo->dv_above})))
    return set_error(NATTEN_B200_EINVAL, "fused_backward_halo: a halo destination is null");
  if (scratch_bytes < natten_b200_fused_backward_scratch_bytes(gi))
    return set_error(NATTEN_B200_ERESOURCE, "fused_backward_halo: scratch has %zu bytes, needs %zu", scratch_bytes,
                     natten_b200_fused_backward_scratch_bytes(gi));
  if (gi->path == NATTEN_B200_PATH_SIMT || !sm100_backward_supported(g, gi->dtype))
    return set_error(NATTEN_B200_EINVAL, "fused_backward_halo: needs the tensor-core kernels: %s",
                     sm100_unsupported_reason(g, gi->dtype));
  FusedArgs a{};
  a.q = q; a.k = k; a.v = v;
  a.out = const_cast<void*>(out); a.lse = const_cast<float*>(lse); a.dout = dout; a.dlse = dlse;
  a.dq = dq; a.dk = dk; a.dv = dv;
  a.scratch = scratch; a.scratch_bytes = scratch_bytes;
  a.halo_below = halo->planes_below; a.halo_above = halo->planes_above;
  a.dk_below = halo->dk_below; a.dv_below = halo->dv_below; a.dk_above = halo->dk_above; a.dv_above = halo->dv_above;
  set_last_path("tcgen05");
  return run_fused_backward_sm100(g, gi->dtype, a, (cudaStream_t)stream);
}

int natten_b200_kernel_status(void) { return sm100_read_status(); }

#ifdef NB_SM100_PROFILE
// Diagnostic builds only (not part of the ABI): where the tensor-core kernels put their cycle counters.
void natten_b200_profile_buffer(float* device_buffer) { sm100_set_profile_buffer(device_buffer); }
#endif

int natten_b200_plan_hint(const natten_b200_geom* gi, int32_t kernel, const int32_t* tile, int32_t max_cols) {
  Geo g;
  if (int rc = make_geo(gi, &g)) return rc;
  if (kernel < 0 || kernel > 2) return set_error(NATTEN_B200_EINVAL, "plan_hint: kernel must be 0 (forward), 1 (dQ) or 2 (dK/dV)");
  const int none[3] = {0, 0, 0};
  int t3[3] = {1, 1, 1};
  if (tile != nullptr)
    for (int i = 0; i < gi->rank; ++i) t3[3 - gi->rank + i] = tile[i];
  return sm100_plan_hint(g, gi->dtype, kernel, tile != nullptr ? t3 : none, max_cols);
}

int natten_b200_describe_plan(const natten_b200_geom* gi, char* buf, size_t cap) {
  Geo g;
  if (int rc = make_geo(gi, &g)) return rc;
  if (buf == nullptr || cap == 0) return set_error(NATTEN_B200_EINVAL, "describe_plan: null buffer");
  int n = sm100_describe_plan(g, gi->dtype, 0, buf, cap);
  for (int mode = 1; mode <= 2 && n > 0 && (size_t)n + 8 < cap; ++mode) {
    n += snprintf(buf + n, cap - n, mode == 1 ? " | dQ: " : " | dK/dV: ");
    n += sm100_describe_plan(g, gi->dtype, mode, buf + n, cap - n);
  }
  return NATTEN_B200_OK;
}

int natten_b200_merge_forward(int32_t dtype, int64_t rows, int32_t head_dim, const void* o0,
                              const float* l0, const void* o1, const float* l1, void* out,
                              float* lse, void* stream) {
  if (rows < 0 || head_dim < 1) return set_error(NATTEN_B200_EINVAL, "merge_forward: bad sizes");
  if (rows == 0) return NATTEN_B200_OK;
  if (any_null({o0, l0, o1, l1, out, lse})) return set_error(NATTEN_B200_EINVAL, "merge_forward: null tensor");
  if (any_misaligned({o0, o1, out})) return reject_misaligned("merge_forward");
  return run_merge_forward(dtype, rows, head_dim, o0, l0, o1, l1, out, lse, (cudaStream_t)stream);
}

int natten_b200_merge_backward(int32_t dtype, int64_t rows, int32_t head_dim, const void* o0,
                               const float* l0, const void* o1, const float* l1,
                               const void* dout, const float* dlse, void* do0, float* dl0,
                               void* do1, float* dl1, void* stream) {
  if (rows < 0 || head_dim < 1) return set_error(NATTEN_B200_EINVAL, "merge_backward: bad sizes");
  if (rows == 0) return NATTEN_B200_OK;
  if (any_null({o0, l0, o1, l1, dout, do0, dl0, do1, dl1}))
    return set_error(NATTEN_B200_EINVAL, "merge_backward: null tensor");
  if (any_misaligned({o0, o1, dout, do0, do1})) return reject_misaligned("merge_backward");
  return run_merge_backward(dtype, rows, head_dim, o0, l0, o1, l1, dout, dlse, do0, dl0, do1, dl1, (cudaStream_t)stream);
}

}  // extern "C"

// Host-side plumbing shared by the translation units: error state, launch
// counting and the prototypes of the per-family launchers.
#pragma once

#include "geom.cuh"

namespace nb {

// Records a message for natten_b200_last_error() and returns `code`.
int set_error(int code, const char* fmt, ...);
// Returns 0 or records the pending CUDA launch error.
int check_launch(const char* what);
void set_last_path(const char* name);

// Brackets one kernel launch: counts it and, while tracing is enabled, records
// CUDA events around it on the launch stream so that per-kernel device time
// can be read back with natten_b200_trace_report().
struct LaunchScope {
  LaunchScope(const char* name, cudaStream_t stream);
  ~LaunchScope();
  cudaStream_t stream_;
  int slot_;
};
#define NB_LAUNCH(name, stream, ...)          \
  do {                                        \
    ::nb::LaunchScope nb_scope_(name, stream); \
    __VA_ARGS__;                              \
  } while (0)

// Validates a public geometry and normalises it to three axes.
int make_geo(const natten_b200_geom* in, Geo* out);

enum class SplitOp { QkForward, QkBackward, AvForward, AvBackward };

int run_split(SplitOp op, const Geo& g, int dtype, const void* a, const void* b, const void* c,
              const float* bias, void* o0, void* o1, float* dbias, cudaStream_t s);
// Row-per-thread kernels for small head dims (split_rows.cu); false when the shape is not theirs.
bool run_split_rows(SplitOp op, const Geo& g, int dtype, const void* a, const void* b, const void* c,
                    const float* bias, void* o0, void* o1, cudaStream_t s);
bool run_bias_grad_rows(const Geo& g, int dtype, const void* dlogits, float* dbias, cudaStream_t s);
bool run_fused_rows(const Geo& g, int dtype, const void* q, const void* k, const void* v, const float* bias, void* out,
                    float* lse, cudaStream_t s);

struct FusedArgs {
  const void *q, *k, *v, *k_extra, *v_extra;
  // forward outputs / backward inputs
  void* out;
  float* lse;
  // backward only
  const void* dout;
  const float* dlse;
  void *dq, *dk, *dv, *dk_extra, *dv_extra;
  void* scratch;
  size_t scratch_bytes;
  // dK/dV of the leading / trailing planes of a K/V slab written elsewhere (another GPU's staging area): plane
  // counts and destinations laid out [batch, planes, rest of the K/V layout]; zeros when unused
  int halo_below = 0, halo_above = 0;
  void *dk_below = nullptr, *dv_below = nullptr, *dk_above = nullptr, *dv_above = nullptr;
};

int run_fused_forward_simt(const Geo& g, int dtype, const FusedArgs& a, cudaStream_t s);
int run_fused_backward_simt(const Geo& g, int dtype, const FusedArgs& a, cudaStream_t s);
size_t fused_backward_scratch_simt(const Geo& g);

int run_merge_forward(int dtype, long long rows, int D, const void* o0, const float* l0,
                      const void* o1, const float* l1, void* out, float* lse, cudaStream_t s);
int run_merge_backward(int dtype, long long rows, int D, const void* o0, const float* l0,
                       const void* o1, const float* l1, const void* dout, const float* dlse,
                       void* do0, float* dl0, void* do1, float* dl1, cudaStream_t s);

}  // namespace nb

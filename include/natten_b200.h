/*
 * natten_b200.h - C ABI of the B200 neighborhood-attention library.
 *
 * Every entry point takes plain device pointers and sizes; the caller owns all
 * memory (inputs, outputs and the scratch buffer the fused backward asks for).
 * Kernels are launched on the stream that is passed in (a cudaStream_t cast to
 * void*, NULL = the default stream) and the call returns without
 * synchronising.  Return value: 0 on success, a NATTEN_B200_E* code otherwise;
 * natten_b200_last_error() then holds a message for the calling thread.
 *
 * Tensor layout is "heads last": [batch, spatial..., heads, head_dim], dense.
 * Logits / attention weights are [batch, out..., heads_q, K_vol] with the slot
 * index row-major over the per-axis kernel slots; log-sum-exp is
 * [batch, out..., heads_q] float32.  out[a] = ceil(q_extent[a] / stride[a]).
 *
 * The functions replace the backend-module protocol that the reference's
 * dispatcher calls (src/natten_mlx/_core/ops.py:49-135) and the native entry
 * points of its compiled tier (src/natten_mlx/_core/_nanobind_ext.cpp:36-216).
 */
#ifndef NATTEN_B200_H
#define NATTEN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NATTEN_B200_ABI_VERSION 2

enum {
  NATTEN_B200_OK = 0,
  NATTEN_B200_EINVAL = 1,      /* bad geometry / null pointer / unsupported dtype */
  NATTEN_B200_ELAUNCH = 2,     /* CUDA reported an error at launch               */
  NATTEN_B200_ERESOURCE = 3,   /* needs more shared memory / scratch than exists */
  NATTEN_B200_ENODEVICE = 4    /* no CUDA device / driver entry point missing    */
};

enum { NATTEN_B200_F32 = 0, NATTEN_B200_F16 = 1, NATTEN_B200_BF16 = 2 };

/* Which kernel family the fused entry points may use. */
enum {
  NATTEN_B200_PATH_AUTO = 0,   /* tensor-core kernels when the shape qualifies   */
  NATTEN_B200_PATH_SIMT = 1,   /* CUDA-core kernels (any shape, any dtype)       */
  NATTEN_B200_PATH_TCGEN05 = 2 /* tensor-core kernels or NATTEN_B200_EINVAL      */
};

/*
 * Problem geometry.  Axis arrays are indexed 0..rank-1, leading axis first.
 *
 * For an unsharded call q_extent == kv_extent == global_extent and the
 * offsets are zero.  For a slab of a larger volume (leading-axis sharding with
 * K/V halo planes) the windows are evaluated in global coordinates:
 * local query index i is global q_offset + i, local key index j is global
 * kv_offset + j, and every key a local query can see must lie inside the
 * local key buffer.
 *
 * causal[a] == 2 makes every query see the whole axis (kernel[a] must equal
 * the extent, dilation and stride 1): the dense attention the reference
 * switches to when the kernel covers the extent
 * (src/natten_mlx/functional.py:141-187).
 *
 * extents, when not NULL, is a device array [batch, rank] int32 with the
 * valid extent of each sample inside the padded tensors (variable-size
 * batches); it replaces global_extent per sample, and queries outside it
 * produce zeros (CUDA-core kernels) or are left unwritten (tensor-core kernels:
 * hand them zero-filled outputs).  host_extents, when not NULL, is a host copy
 * of the same array: with it the fused entry points can serve a variable-size
 * batch on the tensor-core kernels in one launch per kernel (every sample gets
 * TMA tensor maps with its own bounds, built on the host, so that padding of
 * any content, NaN included, stays out of the arithmetic, as with the
 * reference's per-sample slices, src/natten_mlx/_core/pure.py:559-577);
 * without it such a batch runs on the CUDA-core kernels.  The host array is
 * read during the call only.
 *
 * mem_extent, when not all zero, says that every tensor of the call (q, k, v,
 * out, lse and the gradients) is the leading corner of a larger dense array
 * with spatial extents mem_extent >= global_extent: positions are as far
 * apart in memory as in that larger array, the window arithmetic and the
 * bounds use global_extent, and nothing outside the corner is read or
 * written.  This is how one sample of a padded variable-size batch is handed
 * to the tensor-core kernels (one call per sample, pointers at the sample, so
 * that padding of any content, NaN included, stays out of the arithmetic;
 * the reference slices the sample out, src/natten_mlx/_core/pure.py:559-577).
 * Only the fused entry points take it, only on the tensor-core kernels, and
 * not together with slabs, extents or extra tokens (NATTEN_B200_EINVAL).
 */
typedef struct natten_b200_geom {
  int32_t rank;             /* 1, 2 or 3                                          */
  int32_t batch;
  int32_t heads_q;
  int32_t heads_kv;         /* heads_q % heads_kv == 0; kv head = q head / ratio  */
  int32_t head_dim;
  int32_t dtype;            /* NATTEN_B200_F32 / F16 / BF16                       */
  int32_t q_extent[3];
  int32_t kv_extent[3];
  int32_t global_extent[3];
  int32_t q_offset[3];
  int32_t kv_offset[3];
  int32_t kernel[3];
  int32_t stride[3];
  int32_t dilation[3];
  int32_t causal[3];        /* 0 centred window, 1 causal window, 2 whole axis     */
  float scale;
  int32_t n_extra;          /* tokens in k_extra / v_extra, 0 if none            */
  int32_t path;             /* NATTEN_B200_PATH_*                                */
  const int32_t* extents;   /* device, [batch, rank], or NULL                     */
  int32_t mem_extent[3];    /* all zero: dense tensors; see above                 */
  int32_t reserved;         /* must be zero                                       */
  const int32_t* host_extents; /* host copy of extents, or NULL                    */
} natten_b200_geom;

int natten_b200_abi_version(void);
const char* natten_b200_last_error(void);

/* Name of the kernel family the last fused call on this thread used
 * ("simt" or "tcgen05"); for tests and benchmarks. */
const char* natten_b200_last_path(void);

/* Counts kernel launches issued by this library in this process. */
uint64_t natten_b200_launch_count(void);

/*
 * Per-kernel device timing, off by default.  While enabled every kernel the
 * library launches is bracketed by CUDA events on its launch stream.
 * natten_b200_trace_report waits for the recorded launches, writes one line
 * "kernel_name launches total_ms" per kernel into buf (NUL-terminated, at most
 * cap bytes), forgets them, and returns the size the full report needs.
 * Meant for one benchmarking thread; it takes the place of the reference's
 * env-gated wall-clock stage timing
 * (src/natten_mlx/extras/allin1/functional_metal.py:1242-1266).
 */
void natten_b200_trace_enable(int on);
size_t natten_b200_trace_report(char* buf, size_t cap);

/*
 * Host-side evaluation of the per-axis window table with the same integer code
 * the kernels use: for n_query = ceil(length/stride) queries at j*stride writes
 * idx[n_query*kernel] (neighbour coordinate clipped to [0,length-1]) and
 * valid[n_query*kernel] (0/1), start[n_query] (unclipped coordinate of slot 0,
 * nullable) and pb[n_query] (first relative-position-bias slot, nullable; only
 * meaningful when causal == 0).  Needs no GPU.
 * Replaces src/natten_mlx/_core/pure.py:52-73 and
 * src/natten_mlx/utils/window.py:65-103.
 */
int natten_b200_axis_table(int32_t length, int32_t kernel, int32_t dilation, int32_t stride,
                           int32_t causal, int32_t* idx, uint8_t* valid, int32_t* start,
                           int32_t* pb);

/*
 * Split QK: logits = scale * q . k_neighbour (+ bias), -inf at invalid slots.
 * bias (nullable, float32, [heads_q, prod(2*kernel[a]-1)]) is the relative
 * position bias of the allin1 ops and requires stride 1 and no causal axis.
 * Replaces na{1,2,3}d_qk_forward (src/natten_mlx/_core/ops.py:65-73;
 * src/natten_mlx/_core/pure.py:258-283, 320-359, 404-449) and the allin1
 * na{1,2}d_qk_rpb ops (src/natten_mlx/extras/allin1/__init__.py:40-79, 112-150).
 */
int natten_b200_qk_forward(const natten_b200_geom* g, const void* q, const void* k,
                           const float* bias, void* logits, void* stream);

/*
 * Gradients of split QK.  dq [q layout] and dk [k layout] are fully written
 * (queries off the stride lattice get zero).  dbias (nullable, float32, same
 * shape as bias) must be zero-filled by the caller; it is accumulated with
 * atomics.  Replaces na{1,2,3}d_qk_backward (src/natten_mlx/_core/ops.py:103-111;
 * src/natten_mlx/_core/pure.py:735-742, 757-764, 779-786).
 */
int natten_b200_qk_backward(const natten_b200_geom* g, const void* q, const void* k,
                            const void* dlogits, void* dq, void* dk, float* dbias, void* stream);

/*
 * out[B, out..., Hq, D] = softmax_slots(scale * q . k[neighbour] + bias) . v[neighbour], optionally with the
 * log-sum-exp lse[B, out..., Hq] (nullable): QK + relative position bias, softmax and AV in one launch, forward
 * only, one thread per (query, head) row, the logits never reach memory.  bias as in natten_b200_qk_forward
 * (nullable).  head_dim 8, 16, 24, 32, or 12 in float32 (NATTEN_B200_EINVAL otherwise).  The fused path of the
 * reference's DiNAT-style ops: natten2d_qkv_fused, src/natten_mlx/extras/allin1/functional_metal.py:2130-2170.
 */
int natten_b200_qk_bias_av_forward(const natten_b200_geom* g, const void* q, const void* k, const void* v,
                                   const float* bias, void* out, float* lse, void* stream);

/*
 * Split AV: out = sum over valid slots of attn * v_neighbour.
 * Replaces na{1,2,3}d_av_forward (src/natten_mlx/_core/ops.py:75-82;
 * src/natten_mlx/_core/pure.py:286-317, 362-401, 452-494) and the allin1
 * na{1,2}d_av_fused ops (src/natten_mlx/extras/allin1/__init__.py:82-109, 153-180).
 */
int natten_b200_av_forward(const natten_b200_geom* g, const void* attn, const void* v,
                           void* out, void* stream);

/*
 * Gradients of split AV: dattn (zero at invalid slots) and dv.
 * Replaces na{1,2,3}d_av_backward (src/natten_mlx/_core/ops.py:113-135;
 * src/natten_mlx/_core/pure.py:745-754, 767-776, 789-808).
 */
int natten_b200_av_backward(const natten_b200_geom* g, const void* attn, const void* v,
                            const void* dout, void* dattn, void* dv, void* stream);

/*
 * Fused attention: out = softmax(scale * q.k over the window and the extra
 * tokens) . v, lse = log-sum-exp of the same logits (float32, nullable).
 * k_extra / v_extra ([batch, n_extra, heads_kv, head_dim], nullable) are
 * tokens every query attends to.  Covers na{1,2,3}d_forward and
 * na{1,2,3}d_varlen_forward (src/natten_mlx/_core/ops.py:49-58;
 * src/natten_mlx/_core/pure.py:155-255, 497-519, 550-578, 617-647) and the
 * LSE / extra-token / GQA composition of the public functional
 * (src/natten_mlx/functional.py:29-33, 71-104, 251-294, 340-383, 430-473).
 */
int natten_b200_fused_forward(const natten_b200_geom* g, const void* q, const void* k,
                              const void* v, const void* k_extra, const void* v_extra,
                              void* out, float* lse, void* stream);

/*
 * Non-zero when a kernel launched by this library on the current device gave
 * up on one of its bounded waits since the last call (its results are then
 * invalid): 1 a tensor-core kernel, 2 natten_b200_peer_barrier.  0 otherwise.
 * Synchronises with the device.  Stands where the
 * reference turns a failed accelerated kernel into a silent fallback
 * (src/natten_mlx/_core/fast_metal.py:2003-2016): here it is reported instead.
 */
int natten_b200_kernel_status(void);


/* Writes a one-line description of the tensor-core tiling chosen for a
 * geometry (or why it is unsupported) into buf.  Needs no GPU.  Takes the
 * place of the reference's tuning tables (src/natten_mlx/_core/_forward_tuning.py:11-34). */
int natten_b200_describe_plan(const natten_b200_geom* g, char* buf, size_t cap);

/* Pins the tiling of one geometry for one tensor-core kernel (kernel: 0 forward, 1 dQ, 2 dK/dV):
 * tile = query/key tile extents per axis (rank entries, product = 128 / packed heads; NULL or
 * zeros = planner's choice) and max_cols = cap on the chunk width in S columns (0 = none).  The
 * hint stays until it is replaced; zeros release it.  NATTEN_B200_EINVAL when no plan exists with
 * the hint (the hint is then dropped).  This is the write side of the reference's tuning tables
 * (src/natten_mlx/_core/_forward_tuning.py:11-34, _softmax_tuning.py): a caller that measures
 * candidates on its own shapes (natten_mlx_b200.tune.tune_fused does) records the winner here. */
int natten_b200_plan_hint(const natten_b200_geom* g, int32_t kernel, const int32_t* tile, int32_t max_cols);

/* Bytes of scratch natten_b200_fused_backward needs for this geometry. */
size_t natten_b200_fused_backward_scratch_bytes(const natten_b200_geom* g);

/*
 * Gradients of fused attention from the saved out and lse.  dlse (nullable) is
 * the cotangent of lse.  dk_extra / dv_extra are required when n_extra > 0.
 * scratch: device buffer of at least natten_b200_fused_backward_scratch_bytes.
 * Covers na{1,2,3}d_backward and na{1,2,3}d_varlen_backward
 * (src/natten_mlx/_core/ops.py:93-101; src/natten_mlx/_core/pure.py:521-547,
 * 581-614, 650-688, 691-733).
 */
int natten_b200_fused_backward(const natten_b200_geom* g, const void* q, const void* k,
                               const void* v, const void* k_extra, const void* v_extra,
                               const void* out, const float* lse, const void* dout,
                               const float* dlse, void* dq, void* dk, void* dv,
                               void* dk_extra, void* dv_extra, void* scratch,
                               size_t scratch_bytes, void* stream);

/*
 * The fused backward for callers that cannot allocate device memory where the
 * backward runs (an allocator frozen while an execution plan is recorded or
 * replayed, a fixed-budget serving loop, a sandbox that only hands out
 * pre-registered buffers).  Same arguments and results as
 * natten_b200_fused_backward, minus the scratch buffer: the scratch lives in a
 * fixed array inside the library image (natten_b200_static_scratch_capacity()
 * bytes, 4 MiB, held by every GPU that loads the library until the process
 * exits).  A geometry whose natten_b200_fused_backward_scratch_bytes() exceeds
 * the capacity is refused with NATTEN_B200_ERESOURCE.  The call allocates
 * nothing: no cudaMalloc / cudaFree and no allocating library routine.
 * The first call on a device looks the array's device address up (with that
 * device current); make that first call before any stream capture.
 * All calls share the one array, whose contents are whatever the last call
 * left; the kernels rewrite or clear what they read, but two calls that overlap
 * on the GPU (different streams) race on it.
 * This entry point has no counterpart in the reference.
 */
size_t natten_b200_static_scratch_capacity(void);
int natten_b200_fused_backward_static_scratch(const natten_b200_geom* g, const void* q, const void* k,
                                              const void* v, const void* k_extra, const void* v_extra,
                                              const void* out, const float* lse, const void* dout,
                                              const float* dlse, void* dq, void* dk, void* dv,
                                              void* dk_extra, void* dv_extra, void* stream);

/*
 * Halo transport between the GPUs of one box for a volume sharded along its
 * leading axis (one process per GPU).  The reference is single-device and has
 * no counterpart; these two calls let the window of a query reach key/value
 * planes owned by the neighbouring rank, so that the sharded result equals
 * the reference's unsharded one (src/natten_mlx/functional.py:340-383).
 *
 * natten_b200_peer_copy2d copies `rows` rows of `width_bytes` bytes between
 * pitched buffers with plain 16-byte loads and stores; dst or src may be
 * another GPU's memory mapped into this process (CUDA IPC, symmetric memory).
 * Addresses, pitches and the width are multiples of 16 bytes.
 *
 * natten_b200_peer_barrier orders such copies between ranks on their streams:
 * flag_blocks (host array, `world` entries) holds the address, as mapped in
 * this process, of every rank's flag block (`world` zero-initialised uint32
 * words in peer-mapped memory).  The kernel publishes `epoch` in every peer's
 * block and waits until every peer has published an epoch >= it in this
 * rank's block; work queued on the stream after it sees what the peers wrote
 * before their barrier.  Epochs of successive barriers on one set of blocks
 * increase.  A wait longer than timeout_ms (0 = 10 s) gives up and sets
 * natten_b200_kernel_status() to 2 instead of spinning on.
 */
int natten_b200_peer_copy2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                            size_t width_bytes, size_t rows, void* stream);
/* The same copy through a copy engine (cudaMemcpy2DAsync) instead of a kernel: it occupies no SM, so it can run on a
 * second stream under a kernel that fills the GPU. */
int natten_b200_peer_copy2d_dma(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                                size_t width_bytes, size_t rows, void* stream);
int natten_b200_peer_barrier(const uint64_t* flag_blocks, int32_t world, int32_t rank, uint32_t epoch,
                             uint32_t timeout_ms, void* stream);

/*
 * The fused backward of one slab of a volume sharded along its leading axis, with the halo reduction of dK / dV
 * folded into the dK/dV kernel: gradients of the first planes_below and the last planes_above planes of the K/V
 * slab - planes another rank owns - are not written to dk / dv but stored by the kernel's epilogue, tile by tile,
 * straight into dk_below / dv_below and dk_above / dv_above, laid out [batch, planes, rest of the K/V layout]
 * (normally the owner's staging area in peer-mapped memory: plain 16-byte stores cross NVLink while the kernel
 * computes; natten_b200_peer_barrier then tells the owner that they have arrived).  Tensor-core kernels only
 * (bf16 / fp16 shapes they take; NATTEN_B200_EINVAL otherwise), no extra tokens, no per-sample extents.  The
 * other arguments are those of natten_b200_fused_backward.  No counterpart in the reference (single device).
 */
typedef struct natten_b200_halo_out {
  int32_t planes_below, planes_above;
  void *dk_below, *dv_below, *dk_above, *dv_above;
} natten_b200_halo_out;
int natten_b200_fused_backward_halo(const natten_b200_geom* g, const void* q, const void* k,
                                    const void* v, const void* out, const float* lse, const void* dout,
                                    const float* dlse, void* dq, void* dk, void* dv, void* scratch,
                                    size_t scratch_bytes, const natten_b200_halo_out* halo, void* stream);

/*
 * Merge two attention results over the same queries:
 * out = o0 - sigmoid(l1 - l0) * (o0 - o1), lse = l0 - logsigmoid(l0 - l1).
 * rows = number of (query, head) rows, o* are [rows, head_dim] in dtype,
 * l* and lse are float32 [rows].  Replaces merge_attentions
 * (src/natten_mlx/merge.py:56-68).
 */
int natten_b200_merge_forward(int32_t dtype, int64_t rows, int32_t head_dim, const void* o0,
                              const float* l0, const void* o1, const float* l1, void* out,
                              float* lse, void* stream);

/* Gradients of the merge: given dout [rows, head_dim] and dlse [rows]
 * (nullable) writes do0, do1 (dtype) and dl0, dl1 (float32). */
int natten_b200_merge_backward(int32_t dtype, int64_t rows, int32_t head_dim, const void* o0,
                               const float* l0, const void* o1, const float* l1,
                               const void* dout, const float* dlse, void* do0, float* dl0,
                               void* do1, float* dl1, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NATTEN_B200_H */

// Diagnostic: cost per tcgen05.mma instruction for the operand layouts and shapes the fused kernels issue.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --expt-relaxed-constexpr \
//        -o mma_issue_cost natten-mlx_b200/probe/mma_issue_cost.cu -lcuda && ./mma_issue_cost
//
// One thread of a CTA issues 64 rounds of a pattern back to back (operands are zeros in shared / tensor memory,
// only the timing matters), commits, and waits for completion with a bounded wait.  Patterns: the QK^T-like
// product (both operands in shared memory, N = chunk width, K = head dim), the P V-like product (A from tensor
// memory, B an MN-major shared-memory tile, N = head dim, 16 keys per instruction), both interleaved as in a
// forward chunk, a backward chunk (S, dP, then the two accumulating products), an N = 256 product as the
// reference point, and the P V-like product on two alternating accumulators.  Grids of 1, 148 and 296 CTAs
// (one and two CTAs per SM) show whether the streams of two CTAs of an SM slow each other down.
// Prints cycles per instruction at issue and at completion; the last three patterns commit and wait after every
// group of instructions and print cycles per round trip; the three after them issue whole forward chunks with two,
// three or no commits that nobody waits on and print cycles per chunk.
#include <cstdio>
#include <cstdlib>
#include <cuda.h>
#include <cuda_runtime.h>
#include "../csrc/sm100_ptx.cuh"
using namespace nb::sm100;

struct Args { int pattern; int reps; int RB; int layout; int npad; int D; long long* out; };

__global__ void __launch_bounds__(128) k_bench(Args a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar_s;
  __shared__ uint64_t bar_x[3];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  // zero 64 KB of operands
  for (int i = tid; i < 65536 / 16; i += 128) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0, 0, 0, 0);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  const uint32_t bar = smem_u32(&bar_s);
  if (tid == 0) { mbar_init(bar, 1); for (int i = 0; i < 3; ++i) mbar_init(smem_u32(&bar_x[i]), 1); abort_flag = 0; mbar_fence_init(); }
  __syncthreads();
  if (warp == 0) { tmem_alloc(smem_u32(&tmem_slot), 256); tmem_relinquish(); }
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = tmem_slot;
  if (tid == 0) {
    const int RB = a.RB;
    const uint64_t kk_desc0 = smem_desc(0, 16, 8 * RB, a.layout);
    const uint64_t mn_desc0 = smem_desc(0, a.npad * RB, 8 * RB, a.layout);
    const uint32_t a_lo = smem_u32(smem) >> 4, b_lo = (smem_u32(smem) + 16384) >> 4;
    const uint32_t idesc_s = instr_desc(128, a.npad, 1, 0, 0);
    const uint32_t idesc_256 = instr_desc(128, 256, 1, 0, 0);
    const uint32_t idesc_a = instr_desc(128, a.D, 1, 0, 1);
    const int ksteps = (RB / 2) / 16;   // D==dblk elements per row / 16
    const int n_kblk = a.npad / 16;
    uint32_t parity = 0;
    // warm
    mma_ss(tmem, kk_desc0 + a_lo, kk_desc0 + b_lo, idesc_s, 0);
    mma_commit(bar);
    for (uint32_t i = 0; i < 4000 && !mbar_try_wait(bar, parity); ++i) {}
    parity ^= 1;
    long long t0 = clock64();
    int n_mma = 0;
    for (int r = 0; r < a.reps; ++r) {
      if (a.pattern == 0 || a.pattern == 2) {          // QK-like: SS N=npad, ksteps k-steps
        for (int ks = 0; ks < ksteps; ++ks) { mma_ss(tmem, kk_desc0 + a_lo + 2 * ks, kk_desc0 + b_lo + 2 * ks, idesc_s, ks > 0); ++n_mma; }
      }
      if (a.pattern == 1 || a.pattern == 2) {          // PV-like: TS N=D, n_kblk blocks of 16 keys
        uint64_t bd = mn_desc0 + b_lo;
        for (int kk = 0; kk < n_kblk; ++kk) { mma_ts(tmem + 128, tmem + kk * 8, bd, idesc_a, 1); bd += RB; ++n_mma; }
      }
      if (a.pattern == 3) {                            // SS N=256 K=16 reference
        for (int ks = 0; ks < ksteps; ++ks) { mma_ss(tmem, kk_desc0 + a_lo + 2 * ks, kk_desc0 + b_lo + 2 * ks, idesc_256, ks > 0); ++n_mma; }
      }
      if (a.pattern == 4) {                            // PV-like with two alternating accumulators
        uint64_t bd = mn_desc0 + b_lo;
        for (int kk = 0; kk < n_kblk; ++kk) { mma_ts(tmem + 128 + (kk & 1) * 64, tmem + kk * 8, bd, idesc_a, 1); bd += RB; ++n_mma; }
      }
      if (a.pattern == 5) {                            // backward-like: 2 SS products + 2*n_kblk TS products
        for (int w = 0; w < 2; ++w)
          for (int ks = 0; ks < ksteps; ++ks) { mma_ss(tmem + w * a.npad, kk_desc0 + a_lo + 2 * ks, kk_desc0 + b_lo + 2 * ks, idesc_s, ks > 0); ++n_mma; }
        uint64_t bd = mn_desc0 + b_lo;
        for (int kk = 0; kk < n_kblk; ++kk) {
          mma_ts(tmem + 192, tmem + kk * 8, bd, idesc_a, 1);
          mma_ts(tmem + 224, tmem + a.npad + kk * 8, bd, idesc_a, 1);
          bd += RB; n_mma += 2;
        }
      }
    }
    if (a.pattern >= 9) {
      // a forward chunk with its commits (nobody waits on them): 9: one commit after the SS products and one after
      // the TS products; 10: a second commit behind the TS products; 11: no commits at all (= pattern 2)
      const uint32_t bar2 = smem_u32(&bar_x[0]), bar3 = smem_u32(&bar_x[1]), bar4 = smem_u32(&bar_x[2]);
      for (int r = 0; r < a.reps; ++r) {
        for (int ks = 0; ks < ksteps; ++ks) { mma_ss(tmem, kk_desc0 + a_lo + 2 * ks, kk_desc0 + b_lo + 2 * ks, idesc_s, ks > 0); ++n_mma; }
        if (a.pattern != 11) mma_commit(bar2);
        uint64_t bd = mn_desc0 + b_lo;
        for (int kk = 0; kk < n_kblk; ++kk) { mma_ts(tmem + 128, tmem + kk * 8, bd, idesc_a, 1); bd += RB; ++n_mma; }
        if (a.pattern != 11) mma_commit(bar3);
        if (a.pattern == 10) mma_commit(bar4);
      }
      n_mma = a.reps;      // reported per chunk
    } else if (a.pattern >= 6) {
      // round trips: a group of instructions, commit, wait for the barrier - the hand-over a chunk of the fused
      // kernels pays twice (6: one SS product; 7: the ksteps SS products of a chunk; 8: the n_kblk TS products)
      for (int r = 0; r < a.reps; ++r) {
        if (a.pattern == 6) { mma_ss(tmem, kk_desc0 + a_lo, kk_desc0 + b_lo, idesc_s, 0); ++n_mma; }
        if (a.pattern == 7)
          for (int ks = 0; ks < ksteps; ++ks) { mma_ss(tmem, kk_desc0 + a_lo + 2 * ks, kk_desc0 + b_lo + 2 * ks, idesc_s, ks > 0); ++n_mma; }
        if (a.pattern == 8) {
          uint64_t bd = mn_desc0 + b_lo;
          for (int kk = 0; kk < n_kblk; ++kk) { mma_ts(tmem + 128, tmem + kk * 8, bd, idesc_a, 1); bd += RB; ++n_mma; }
        }
        mma_commit(bar);
        bool got = false;
        for (uint32_t i = 0; i < 4000 && !got; ++i) got = mbar_try_wait(bar, parity);
        parity ^= 1;
      }
      n_mma = a.reps;      // reported per round trip
    }
    long long t_issue = clock64();
    mma_commit(bar);
    bool done = false;
    for (uint32_t i = 0; i < 4000 && !done; ++i) done = mbar_try_wait(bar, parity);
    long long t1 = clock64();
    if (blockIdx.x == 0) { a.out[0] = t_issue - t0; a.out[1] = t1 - t0; a.out[2] = n_mma; a.out[3] = done ? 1 : 0; }
  }
  tc_fence_before(); __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 256); }
}

int main() {
  long long* out; cudaMalloc(&out, 64);
  cudaFuncSetAttribute(k_bench, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  const char* names[] = {"SS QK-like", "TS PV-like", "QK+PV chunk", "SS N=256", "TS alt-acc", "bwd chunk",
                         "1 SS + commit + wait", "chunk SS + commit + wait", "chunk TS + commit + wait",
                         "chunk, 2 commits, no wait", "chunk, 3 commits, no wait", "chunk, no commits"};
  struct Cfg { int RB, layout, npad, D; } cfgs[] = {{64, 4, 96, 32}, {128, 2, 64, 64}, {128, 2, 128, 64}, {64, 4, 48, 32}, {32, 6, 96, 32}, {32, 6, 48, 32}, {32, 0, 96, 32}};
  for (auto c : cfgs)
    for (int grid : {1, 148, 296})
      for (int pat = 0; pat < 12; ++pat) {
        if (pat == 5 && (c.D != 32 || 2 * c.npad > 192)) continue;
        if (pat == 3 && c.npad != 96 && c.npad != 64) continue;
        Args a{pat, 64, c.RB, c.layout, c.npad, c.D, out};
        k_bench<<<grid, 128, 70 * 1024>>>(a);
        cudaError_t e = cudaDeviceSynchronize();
        long long h[4]; cudaMemcpy(h, out, 32, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) { printf("error %s\n", cudaGetErrorString(e)); return 1; }
        printf("RB=%d npad=%d D=%d grid=%3d %-12s: %lld MMAs, issue %.1f cyc/MMA, complete %.1f cyc/MMA done=%lld\n", c.RB, c.npad, c.D,
               grid, names[pat], h[2], (double)h[0] / h[2], (double)h[1] / h[2], h[3]);
      }
  return 0;
}

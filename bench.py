"""Benchmark of the neighborhood-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over one batch of synthetic input: a
fused forward + backward call for every variant of the workload.  The default
workload is the NAT-stage configuration: na2d bf16, B=32, 56x56, 4 heads,
D=32, kernel 7x7, dilation 1 and dilation 4 (two calls per step).

Prints ONE JSON line.  ``value`` is whole-job effective TFLOP/s (algorithmic
FLOPs: forward 4*B*H*N*K_vol*D, backward 2.5x that) with inputs resident in
HBM; ``e2e`` is the same metric through the public API with pinned HOST
buffers, host<->device copies inside the timed region.  ``roofline`` is for
the kernel with the largest share of device time, measured live with CUDA
events recorded by the library around each of its launches.

With ``--gpus N`` (launched by torchrun, one rank per GPU) the named batch is
sharded over the ranks (32 / N samples each: strong scaling, no data-path
collective, the batch x head shards are independent); time is the max over
ranks.  The line also carries the weak-scaling figure (every rank the whole
batch) and, under ``na3d_video``, the video volume sharded by heads and sharded
along T with the K/V halo exchange over NCCL.

``--impl reference`` times the CPU restatement of the reference's pure backend
(the MLX array library it needs does not install on Linux) on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _sub in ("natten-mlx_b200", "oracle"):
    _p = os.path.join(ROOT, _sub)
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402


# ---------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------
WORKLOADS = {
    # name: dict(rank, shape [B, spatial..., Hq, D], heads_kv, kernel, dilation variants, causal, dtype)
    "na2d_nat_stage": dict(shape=(32, 56, 56, 4, 32), heads_kv=4, kernel=(7, 7), dilations=[(1, 1), (4, 4)],
                           causal=(False, False), dtype="bf16",
                           label="na2d bf16 B=32 56x56 H=4 D=32 K=7x7 dilation {1,4} fwd+bwd"),
    "na3d_video": dict(shape=(2, 32, 96, 96, 16, 64), heads_kv=16, kernel=(3, 7, 7), dilations=[(1, 2, 2)],
                       causal=(True, False, False), dtype="bf16", cpu_shape=(1, 4, 32, 32, 2, 64),
                       label="na3d bf16 B=2 T=32 96x96 H=16 D=64 K=(3,7,7) causal-T dilation (1,2,2) fwd+bwd"),
    "na1d_parity": dict(shape=(2, 64, 4, 32), heads_kv=4, kernel=(7,), dilations=[(1,)], causal=(False,),
                        dtype="f32", label="na1d fp32 B=2 L=64 H=4 D=32 K=7 fwd+bwd"),
}
DTYPES = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


def kvol(w):
    v = 1
    for k in w["kernel"]:
        v *= k
    return v


def flops_fwd(w):
    b, hq, d = w["shape"][0], w["shape"][-2], w["shape"][-1]
    n = 1
    for e in w["shape"][1:-2]:
        n *= e
    return 4.0 * b * hq * n * kvol(w) * d


def flops_step(w):
    return 3.5 * flops_fwd(w) * len(w["dilations"])


def tensor_bytes(w, heads=None):
    n = 1
    for e in w["shape"][:-2]:
        n *= e
    esz = torch.tensor([], dtype=DTYPES[w["dtype"]]).element_size()
    return n * (heads if heads is not None else w["shape"][-2]) * w["shape"][-1] * esz


def lse_bytes(w):
    n = 1
    for e in w["shape"][:-1]:
        n *= e
    return n * 4


def algorithmic_bytes(w):
    """Compulsory HBM traffic per launch of each kernel (one variant)."""
    tq, tkv, tl = tensor_bytes(w), tensor_bytes(w, w["heads_kv"]), lse_bytes(w)
    fwd = tq + 2 * tkv + tq + tl                      # read q,k,v ; write out,lse
    bwd_q = tq + 2 * tkv + tq + tq + tl + tq + tl     # read q,k,v,out,dout,lse ; write dq,delta
    bwd_kv = tq + 2 * tkv + tq + 2 * tl + 2 * tkv     # read q,k,v,dout,lse,delta ; write dk,dv
    return {"fused_fwd": fwd, "fused_bwd_q": bwd_q, "fused_bwd_kv": bwd_kv,
            "fna_fwd_sm100": fwd, "fna_bwd_dq_sm100": bwd_q, "fna_bwd_dkv_sm100": bwd_kv,
            "fna_bwd_prep_sm100": 2 * tq + 2 * tl}


# dram__bytes_read.sum + dram__bytes_write.sum per launch, from an ncu capture of one forward+backward call of
# the default workload; workloads without a capture report null.
NCU_TRAFFIC = {"na2d_nat_stage": {"fna_fwd_sm100": 83.9e6, "fna_bwd_dq_sm100": 117.6e6, "fna_bwd_dkv_sm100": 130.6e6,
                                  "fna_bwd_prep_sm100": 51.4e6}}


def make_inputs(w, seed, device, pinned=False):
    """q, k, v and the output cotangent: iid N(0,1) from a fixed seed, cast to the dtype."""
    gen = torch.Generator().manual_seed(seed)
    dt = DTYPES[w["dtype"]]
    kv_shape = w["shape"][:-2] + (w["heads_kv"], w["shape"][-1])
    out = []
    for shape in (w["shape"], kv_shape, kv_shape, w["shape"]):
        t = torch.randn(shape, generator=gen, dtype=torch.float32).to(dt)
        t = t.pin_memory() if pinned else t.to(device)
        out.append(t)
    return out


# ---------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as fh:
            for line in fh:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1])); mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
# the reference arm / CPU baseline: the oracle on the host cores
# ---------------------------------------------------------------------------
def cpu_sample_workload(w, batch):
    """The bounded sample the CPU legs run: `batch` samples, or the workload's reduced `cpu_shape`."""
    if "cpu_shape" in w:
        return dict(w, shape=tuple(w["cpu_shape"]), heads_kv=min(w["heads_kv"], w["cpu_shape"][-2]))
    return dict(w, shape=(batch,) + tuple(w["shape"][1:]))


def cpu_sample_step(w, batch):
    """Forward + backward of every variant on the bounded sample with the CPU oracle (float32)."""
    import natten_oracle as oracle
    wb = cpu_sample_workload(w, batch)
    total = 0.0
    for vi, dil in enumerate(w["dilations"]):
        q, k, v, cot = (t.float() for t in make_inputs(wb, 1234 + vi, "cpu"))
        t0 = time.perf_counter()
        oracle.grads(lambda a, b, c: oracle.na(a, b, c, w["kernel"], 1, dil, w["causal"]), [q, k, v], cot)
        total += time.perf_counter() - t0
    return total


def cpu_sample_batch(w):
    # keep the K_vol-fold gather of the CPU path near a few hundred MB
    per_sample = tensor_bytes(dict(w, shape=(1,) + tuple(w["shape"][1:]), dtype="f32")) * kvol(w)
    return max(1, min(w["shape"][0], int(400e6 // max(per_sample, 1))))


def run_reference(args, w, rank, world):
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    batch = cpu_sample_batch(w)
    for _ in range(args.warmup):
        cpu_sample_step(w, batch)
    t = sum(cpu_sample_step(w, batch) for _ in range(args.steps))
    ms = t / args.steps * 1e3
    tflops = flops_step(cpu_sample_workload(w, batch)) / (ms * 1e-3) / 1e12
    sample = f"shape {cpu_sample_workload(w, batch)['shape']} of {w['shape']} per step, float32, both passes, every variant"
    line = {
        "impl": "reference", "metric": "na_fwd_bwd_effective_tflops", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["label"], "note": "CPU restatement of the reference's pure backend (torch CPU ops)"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------
def shard_batch(total, world, rank):
    """Samples [lo, hi) of a batch of `total` that rank `rank` of `world` owns (balanced contiguous split)."""
    return (total * rank) // world, (total * (rank + 1)) // world


class FusedRunner:
    """Device-resident fused forward + backward calls of one workload on this rank's shard, replayed from a CUDA graph
    (the launches of a step are a fixed sequence; at small per-GPU batches the host would otherwise be the limit)."""

    def __init__(self, w, dev, seed0=1234):
        from natten_mlx_b200._core import cuda as backend
        self.w, self.dev, self.backend = w, dev, backend
        self.one = (1,) * (len(w["shape"]) - 3)
        self.inputs = [make_inputs(w, seed0 + vi, dev) for vi in range(len(w["dilations"]))]
        self.graph = None

    def step_eager(self):
        w, be = self.w, self.backend
        res = None
        for (q, k, v, cot), dil in zip(self.inputs, w["dilations"]):
            out, lse = be.fused_forward(q, k, v, w["kernel"], self.one, dil, w["causal"], None)
            res = be.fused_backward(q, k, v, out, lse, cot, None, w["kernel"], self.one, dil, w["causal"], None)
        return res

    def capture(self):
        """Returns True when the step now replays from a graph (eager launches otherwise)."""
        try:
            side = torch.cuda.Stream(device=self.dev)
            side.wait_stream(torch.cuda.current_stream(self.dev))
            with torch.cuda.stream(side):
                for _ in range(2):
                    self.step_eager()
            torch.cuda.current_stream(self.dev).wait_stream(side)
            torch.cuda.synchronize(self.dev)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._keep = self.step_eager()
            self.graph = graph
        except Exception:                      # capture is an optimisation of the launch path, never a requirement
            self.graph = None
            torch.cuda.synchronize(self.dev)
        return self.graph is not None

    def step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self.step_eager()


def run_ours(args, w, rank, world, local_rank):
    import torch.distributed as dist
    import natten_mlx_b200 as nb
    from natten_mlx_b200 import _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device for the default arm (there is no CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    nvar = len(w["dilations"])
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            peaks = json.load(fh)
    except OSError:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured" if "hbm_gbs" in peaks else "fallback"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    last_stats = {}

    def timed(step_fn, steps, trace=False):
        """Mean device milliseconds per step: CUDA events around every step, L2 flushed before each, barrier +
        synchronize on both sides, maximum over the ranks.  Median and minimum of the steps go to `last_stats`."""
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        barrier()
        if trace:
            _lib.trace_report()
            _lib.trace_enable(True)
        for a, b in evs:
            flush.zero_()                       # evict L2 between timed iterations
            a.record()
            step_fn()
            b.record()
        barrier()
        if trace:
            _lib.trace_enable(False)
        each = sorted(a.elapsed_time(b) for a, b in evs)
        ms = sum(each)
        stats = [ms, each[len(each) // 2], each[0]]
        if world > 1:
            t = torch.tensor(stats, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            stats = [float(x) for x in t.tolist()]
        last_stats.update(median=stats[1], min=stats[2])      # of the steps of this call, max over the ranks
        return stats[0] / steps

    # ---- the workload: the named batch sharded over the ranks (strong scaling; at one GPU the whole batch)
    B = w["shape"][0]
    lo, hi = shard_batch(B, world, rank)
    w_loc = dict(w, shape=(hi - lo,) + tuple(w["shape"][1:]))
    main = FusedRunner(w_loc, dev, seed0=1234 + 16 * rank)
    tuned = {}
    for (q, k, v, cot), dil in zip(main.inputs, w["dilations"] if not args.no_tune else []):
        res = nb.tune.tune_fused(q, k, v, w["kernel"], dilation=dil, is_causal=w["causal"])
        tuned["x".join(str(d) for d in dil)] = {kn: {"tile": list(t), "max_cols": c} for kn, (t, c, _) in res.items()}
    for _ in range(max(args.warmup, 3)):
        main.step_eager()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count()
    ms_trace = timed(main.step_eager, args.steps, trace=True)      # eager launches with per-kernel events
    launches = _lib.launch_count() - launches0
    trace = _lib.trace_report()
    path = _lib.last_path()
    ms_eager = timed(main.step_eager, args.steps)
    graphed = main.capture()
    for _ in range(3):
        main.step()
    ms_plain = timed(main.step, args.steps)                        # the headline: same launches, replayed
    plain_stats = dict(last_stats)

    if args.short:
        if rank == 0:
            sampler.stop()
            name, (n, ms_total) = max(trace.items(), key=lambda kv: kv[1][1])
            print(json.dumps({"metric": "na_fwd_bwd_effective_tflops", "value": flops_step(w) / (ms_plain * 1e-3) / 1e12,
                              "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "ms_per_step": ms_plain,
                              "config": {"workload": w["label"], "short": True},
                              "kernels": {k: {"launches": n_, "ms_per_launch": t / n_} for k, (n_, t) in sorted(trace.items())},
                              "e2e": None, "cpu_baseline": None, "gpu_launches": int(launches)}))
        return

    # ---- end to end: pinned host buffers -> device -> public API forward + backward -> host, on the same shard
    host_in = [make_inputs(w_loc, 1234 + 16 * rank + vi, dev, pinned=True) for vi in range(nvar)]
    host_out = [[torch.empty_like(t).pin_memory() for t in (hi_[0], hi_[0], hi_[1], hi_[2])] for hi_ in host_in]
    h2d = sum(t.numel() * t.element_size() for hi_ in host_in for t in hi_)
    d2h = sum(t.numel() * t.element_size() for ho in host_out for t in ho)
    from natten_mlx_b200.host import HostPipeline
    pipes = [HostPipeline(w_loc["shape"], host_in[0][0].dtype, dev, w["kernel"], dilation=dil, is_causal=w["causal"],
                          heads_kv=w["heads_kv"], slabs=4) for dil in w["dilations"]]

    def step_e2e():
        for hi_, ho, pipe in zip(host_in, host_out, pipes):     # the variants share the streams and keep streaming
            pipe.run(hi_[0], hi_[1], hi_[2], hi_[3], ho[0], ho[1], ho[2], ho[3], wait=False)
        pipes[-1].join()

    for _ in range(2):
        step_e2e()
    ms_e2e = timed(step_e2e, args.steps)
    clocks = sampler.stop() if rank == 0 else None

    # ---- weak scaling for the record (every rank the whole named batch): N > 1 only
    weak = None
    if world > 1:
        wk = FusedRunner(w, dev, seed0=2234 + 16 * rank)
        for _ in range(3):
            wk.step_eager()
        wk.capture()
        for _ in range(2):
            wk.step()
        ms_weak = timed(wk.step, args.steps)
        weak = {"ms_per_step": ms_weak, "value": flops_step(w) * world / (ms_weak * 1e-3) / 1e12, "per_gpu_batch": B,
                "global_batch": B * world}
        del wk

    # ---- the video volume on the same ranks: sharded by heads (no collective) and along T (K/V halo exchange)
    video = run_video_legs(args, rank, world, dev, timed, barrier) if args.workload == "na2d_nat_stage" else None

    if rank != 0:
        return
    total_flops = flops_step(w)                    # the named batch, whatever the number of ranks
    value = total_flops / (ms_plain * 1e-3) / 1e12
    e2e_value = total_flops / (ms_e2e * 1e-3) / 1e12

    alg = algorithmic_bytes(w_loc)
    roofline = None
    if trace:
        name, (n, ms_total) = max(trace.items(), key=lambda kv: kv[1][1])
        per_launch_ms = ms_total / n
        share = ms_total / sum(v[1] for v in trace.values())
        if name in alg:
            achieved = alg[name] / (per_launch_ms * 1e-3) / 1e9
            traffic = NCU_TRAFFIC.get(args.workload, {}).get(name)
            roofline = {"bound": "hbm", "kernel": name, "achieved": achieved, "peak": hbm_peak, "unit": "GB/s",
                        "frac": achieved / hbm_peak,
                        "traffic": traffic * (hi - lo) / B if traffic is not None else None,   # scales with the batch
                        "peak_kind": peak_kind, "launch_ms": per_launch_ms, "share_of_device_time": share,
                        "algorithmic_bytes_per_launch": alg[name]}
    kernels = {k: {"launches": n, "ms_per_launch": ms / n} for k, (n, ms) in sorted(trace.items())}

    cpu = None
    if world == 1:
        torch.set_num_threads(os.cpu_count() or 1)
        batch = cpu_sample_batch(w)
        cpu_sample_step(w, batch)
        t_cpu, reps = 0.0, 0
        while t_cpu < 10.0 and reps < 20:
            t_cpu += cpu_sample_step(w, batch)
            reps += 1
        cpu_tflops = flops_step(cpu_sample_workload(w, batch)) * reps / t_cpu / 1e12
        cpu = {"value": cpu_tflops, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
               "sample": f"shape {cpu_sample_workload(w, batch)['shape']} of {w['shape']}, {reps} repetitions, float32 "
                         "CPU restatement of the reference's pure backend, forward+backward of every variant",
               "mlx_core_importable": mlx_importable()}

    line = {
        "metric": "na_fwd_bwd_effective_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_plain, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": w["dtype"], "data": "synthetic",
        "config": {"workload": w["label"], "calls_per_step": nvar, "per_gpu_batch": hi - lo,
                   "global_batch": B, "parallelism": f"batch of {B} sharded over {world} rank(s), no collective",
                   "l2": "256 MiB buffer written between timed iterations; separate inputs per variant",
                   "kernel_family": path, "flops_model": "fwd 4*B*H*N*K_vol*D, bwd 2.5x fwd",
                   "launch": "CUDA graph replay of the step's launches" if graphed else "eager launches",
                   "ms_per_step_median": plain_stats.get("median"), "ms_per_step_min": plain_stats.get("min"),
                   "ms_per_step_eager": ms_eager, "ms_per_step_eager_traced": ms_trace,
                   "ms_per_call_fwd_bwd": ms_plain / nvar,
                   "tuned_plans": tuned},
        "roofline": roofline, "kernels": kernels, "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d * world,
                "d2h_bytes_per_step": d2h * world,
                "per_rank": {"h2d_gb_per_s": h2d / (ms_e2e * 1e-3) / 1e9, "d2h_gb_per_s": d2h / (ms_e2e * 1e-3) / 1e9,
                             "note": "rank 0's bytes over the step time (max over ranks); the two directions overlap"}},
        "gpu_launches": int(launches), "clocks": clocks,
    }
    if weak is not None:
        line["weak_scaling"] = weak
    if video is not None:
        line["na3d_video"] = video
    print(json.dumps(line))


def mlx_importable():
    """Whether the array library of the reference is importable here (it is not on Linux images; when it is, the
    fixtures under tests/golden can be regenerated against it with tests/golden/make_golden.py)."""
    try:
        import importlib.util
        return importlib.util.find_spec("mlx.core") is not None
    except (ImportError, ValueError):
        return False


def run_video_legs(args, rank, world, dev, timed, barrier):
    """The 3-D video volume (bf16 B=2 T=32 96x96 16 heads D=64, kernel (3,7,7), causal along T, dilation (1,2,2)) on
    the same ranks, as extra figures of the line: the heads sharded over the ranks (no collective) and the volume
    sharded along T with the K/V halo exchange.  Forward + backward per step; returns rank 0's summary."""
    import torch.distributed as dist
    import natten_mlx_b200 as nb
    from natten_mlx_b200 import _lib, sharding

    w = WORKLOADS["na3d_video"]
    steps = max(3, min(args.steps, 5))
    out = {"workload": w["label"], "steps": steps}
    heads = w["shape"][-2]

    def traced(step_fn):
        for _ in range(2):
            step_fn()
        ms = timed(step_fn, steps, trace=True)
        kernels = {k: {"launches": n, "ms_per_launch": t / n} for k, (n, t) in sorted(_lib.trace_report().items())}
        ksum = sum(v["ms_per_launch"] * v["launches"] for v in kernels.values()) / steps
        return ms, kernels, ksum

    # (a) heads sharded: every rank the whole volume for heads [lo, hi)
    if heads % world == 0:
        hloc = heads // world
        w_h = dict(w, shape=tuple(w["shape"][:-2]) + (hloc, w["shape"][-1]), heads_kv=hloc)
        r = FusedRunner(w_h, dev, seed0=3234 + 16 * rank)
        ms, kernels, ksum = traced(r.step_eager)
        out["heads_sharded"] = {"ms_per_step": ms, "heads_per_gpu": hloc, "value": flops_step(w) / (ms * 1e-3) / 1e12,
                                "kernels_rank0": kernels, "kernel_ms_per_step_rank0": ksum}
        del r
        torch.cuda.empty_cache()
    # (b) sharded along T: K/V halo planes written into the neighbour's buffers by the library's copy kernel
    B, T = w["shape"][0], w["shape"][1]
    if world <= T:
        bounds = sharding.shard_bounds(T, world)
        lo, hi = bounds[rank], bounds[rank + 1]
        gen = torch.Generator().manual_seed(1240 + rank)
        local = (B, hi - lo) + tuple(w["shape"][2:])
        ks, dl, ca = w["kernel"], w["dilations"][0], w["causal"]
        mk = lambda: torch.randn(local, generator=gen, dtype=torch.float32).to(torch.bfloat16).to(dev)
        q, cot = mk().requires_grad_(True), mk()
        peer = world > 1 and sharding.peer_transport() is not None
        if peer:
            # K and V are produced straight into symmetric memory with room for the halo planes around them
            plans = sharding.all_plans(T, world, ks[0], dl[0], ca[0])
            (k, v), kv_lease = sharding.peer_kv_buffers(local, torch.bfloat16, plans, rank)
            k.copy_(mk())
            v.copy_(mk())
            k.requires_grad_(True)
            v.requires_grad_(True)
        else:
            k, v = mk().requires_grad_(True), mk().requires_grad_(True)

        def make_step(transport):
            def step():
                o = nb.na3d(q, k, v, kernel_size=ks, dilation=dl, is_causal=ca) if world == 1 else \
                    sharding.na_sharded(q, k, v, T, ks, dl, ca, transport=transport)
                return torch.autograd.grad(o, (q, k, v), cot)
            return step
        ms_p2p = traced(make_step("p2p"))[0] if world > 1 else None
        ms, kernels, ksum = traced(make_step("auto"))
        out["t_sharded"] = {"ms_per_step": ms, "planes_per_rank": [bounds[r + 1] - bounds[r] for r in range(world)],
                            "value": flops_step(w) / (ms * 1e-3) / 1e12, "kernels_rank0": kernels,
                            "kernel_ms_per_step_rank0": ksum, "ms_per_step_nccl_send_recv": ms_p2p,
                            "halo": "none (one rank)" if world == 1 else (
                                "K/V planes written into the neighbour's symmetric-memory K/V buffer by the library's copy "
                                "kernel between two flag barriers; dK/dV partials of the halo planes written into the "
                                "owner's staging area the same way and added in place" if peer else
                                "K/V planes and dK/dV partials by NCCL send/recv")}
    return out


# ---------------------------------------------------------------------------
# table workloads (the allin1 split 1-D path and the variable-size GQA batch with extra tokens): device-resident,
# single GPU, no CPU or end-to-end leg
# ---------------------------------------------------------------------------
TABLE_WORKLOADS = ("allin1_1d", "allin1_1d_long", "na2d_varlen_gqa")


def run_table_workload(args):
    import natten_mlx_b200 as nb
    from natten_mlx_b200 import _lib
    from natten_mlx_b200.extras.allin1 import na1d_av_fused, na1d_qk_rpb

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator().manual_seed(1236)
    rnd = lambda shape, dt: torch.randn(shape, generator=gen, dtype=torch.float32).to(dt).to(dev)
    kernel_bytes = None
    if args.workload in ("allin1_1d", "allin1_1d_long"):
        # q, k, v [8,L,4,12] fp32, rpb [4,9] ~ N(0,0.02), K=5, dilation 2, scale 0.288: QK+RPB -> softmax -> AV
        # (L = 4096 is the named configuration; the long variant, 16 times the length, takes launch latency out
        # of the per-kernel bandwidth figures)
        L = 4096 if args.workload == "allin1_1d" else 65536
        q, k, v = (rnd((8, L, 4, 12), torch.float32) for _ in range(3))
        rpb = rnd((4, 9), torch.float32) * 0.02
        label = f"allin1 fp32 na1d_qk_rpb -> softmax -> na1d_av_fused, B=8 L={L} H=4 D=12 K=5 dilation 2"
        tens = 8 * L * 4 * 12 * 4
        logit = 8 * L * 4 * 5 * 4
        byts = (2 * tens + logit) + 2 * logit + (logit + 2 * tens)       # QK ; softmax ; AV
        kernel_bytes = {"row_dot": 2 * tens + logit, "row_wsum": logit + 2 * tens, "row_fused": 4 * tens}
        flops = 2 * 4.0 * 8 * 4 * L * 5 * 12 / 2                         # 2*N*K*D for QK and again for AV

        def eager():
            with torch.no_grad():
                a = torch.softmax(na1d_qk_rpb(q, k, rpb, 5, 2, scale=0.288), dim=-1)
                return na1d_av_fused(a, v, 5, 2)
        # three launches of a few microseconds each: replayed from a CUDA graph (the eager time is reported too)
        for _ in range(3):
            eager()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_out = eager()
        step = graph.replay
        extra_cfg = {"launch": "CUDA graph replay of the three launches"}
        dtype = "f32"
        # the same result from the one-launch fused operator (no logits in memory), for the record
        from natten_mlx_b200.extras.allin1 import na1d_qkv_fused
        fused_fn = lambda: na1d_qkv_fused(q, k, v, rpb, 5, 2, scale=0.288)
        for _ in range(3):
            fused_fn()
        torch.cuda.synchronize()
        fgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(fgraph):
            fused_out = fused_fn()
    else:
        # B=16 padded to 128x128, per-sample H,W from {64,...,128}, 16 query / 4 KV heads, D=128, K=13, dilation 2,
        # 64 extra tokens, LSE returned and merged; forward + backward
        B, M, Hq, Hkv, D, NX = 16, 128, 16, 4, 128, 64
        sizes = (torch.randint(0, 9, (B, 2), generator=gen) * 8 + 64).to(torch.int32)
        bf = torch.bfloat16
        q = rnd((B, M, M, Hq, D), bf).requires_grad_(True)
        k, v = (rnd((B, M, M, Hkv, D), bf).requires_grad_(True) for _ in range(2))
        ak, av = (rnd((B, NX, Hkv, D), bf).requires_grad_(True) for _ in range(2))
        cot = rnd((B, M, M, Hq, D), bf)
        host_sizes = [tuple(int(x) for x in r) for r in sizes.tolist()]
        st = sizes.to(dev)
        tokens = sum(h * w_ for h, w_ in host_sizes)
        label = (f"na2d bf16 varlen B=16 max 128x128 ({tokens} tokens) 16q/4kv heads D=128 K=13x13 dilation 2, "
                 "64 extra tokens, lse+merge, fwd+bwd")
        flops = 3.5 * 4.0 * Hq * tokens * (169 + NX) * D
        byts = None

        def step():
            out = nb.na2d_varlen(q, k, v, st, 13, 2, additional_keys=ak, additional_values=av, host_sizes=host_sizes)
            return torch.autograd.grad(out, (q, k, v, ak, av), cot)
        eager = None
        # the tilings of the three tensor-core kernels are measured once for this geometry and pinned
        res = nb.tune.tune_fused(q.detach(), k.detach(), v.detach(), 13, 2, sizes=st, host_sizes=host_sizes,
                                 additional_keys=ak.detach(), additional_values=av.detach())
        extra_cfg = {"tuned": {kn: {"tile": list(t), "max_cols": c} for kn, (t, c, _) in res.items()}}
        dtype = "bf16"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(0)
    sampler.start()
    launches0 = _lib.launch_count()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    torch.cuda.synchronize()
    for a, b in evs:
        flush.zero_()
        a.record()
        step()
        b.record()
    torch.cuda.synchronize()
    ms = sum(a.elapsed_time(b) for a, b in evs) / args.steps
    launches = _lib.launch_count() - launches0
    if eager is not None:                    # the same step launched eagerly, for the record
        launches = 2 * args.steps            # graph replays bypass the library's launch counter
        for a, b in evs:
            flush.zero_()
            a.record()
            fgraph.replay()
            b.record()
        torch.cuda.synchronize()
        extra_cfg["fused_one_launch"] = {"ms_per_step": sum(a.elapsed_time(b) for a, b in evs) / args.steps,
                                         "algorithmic_bytes": 4 * tens,
                                         "max_abs_diff_to_split": float((fused_out - graph_out).abs().max())}
        for a, b in evs:
            flush.zero_()
            a.record()
            eager()
            b.record()
        torch.cuda.synchronize()
        extra_cfg["ms_per_step_eager"] = sum(a.elapsed_time(b) for a, b in evs) / args.steps
    clocks = sampler.stop()
    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
            peaks = json.load(fh)
    except OSError:
        pass
    # per-kernel device time of the library's launches (eager launches bracketed by events)
    run_eager = (lambda: (eager(), fused_fn())) if eager is not None else step
    _lib.trace_report()
    _lib.trace_enable(True)
    for _ in range(args.steps):
        flush.zero_()
        run_eager()
    torch.cuda.synchronize()
    _lib.trace_enable(False)
    kernels = {}
    for name, (n, ms_total) in sorted(_lib.trace_report().items()):
        kernels[name] = {"launches_per_step": n / args.steps, "ms_per_launch": ms_total / n}
        if kernel_bytes is not None and name in kernel_bytes:
            gbs = kernel_bytes[name] / (ms_total / n * 1e-3) / 1e9
            kernels[name].update(algorithmic_bytes=kernel_bytes[name], gb_per_s=gbs,
                                 frac_of_hbm_peak=gbs / float(peaks.get("hbm_gbs", 6650.0)))
    roofline = None
    if byts is not None:
        hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
        ach = byts / (ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": "whole step (3 launches)", "achieved": ach, "peak": hbm_peak, "unit": "GB/s",
                    "frac": ach / hbm_peak, "traffic": None, "peak_kind": "measured" if "hbm_gbs" in peaks else "fallback",
                    "algorithmic_bytes_per_step": byts}
    print(json.dumps({
        "metric": "na_fwd_bwd_effective_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": dict({"workload": label, "l2": "256 MiB buffer written between timed iterations",
                        "kernel_family": _lib.last_path()}, **extra_cfg),
        "roofline": roofline, "kernels": kernels, "cpu_baseline": None, "e2e": None, "gpu_launches": int(launches),
        "clocks": clocks}))


# ---------------------------------------------------------------------------
# the video volume sharded along T over the ranks (strong scaling, K/V halo exchange over NCCL)
# ---------------------------------------------------------------------------
def run_tshard(args, rank, world, local_rank):
    import torch.distributed as dist
    import natten_mlx_b200 as nb
    from natten_mlx_b200 import _lib, sharding

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    w = WORKLOADS["na3d_video"]
    B, T = w["shape"][0], w["shape"][1]
    bounds = sharding.shard_bounds(T, world)
    lo, hi = bounds[rank], bounds[rank + 1]
    gen = torch.Generator().manual_seed(1240 + rank)
    local = (B, hi - lo) + tuple(w["shape"][2:])
    q, k0, v0, cot = (torch.randn(local, generator=gen, dtype=torch.float32).to(torch.bfloat16).to(dev) for _ in range(4))
    ks, dl, ca = w["kernel"], w["dilations"][0], w["causal"]
    if world > 1 and sharding.peer_transport() is not None:
        # K and V are produced straight into symmetric memory with room for the halo planes around them
        (k, v), kv_lease = sharding.peer_kv_buffers(local, torch.bfloat16, sharding.all_plans(T, world, ks[0], dl[0], ca[0]), rank)
        k.copy_(k0)
        v.copy_(v0)
    else:
        k, v = k0, v0
    del k0, v0
    q, k, v = (t.requires_grad_(True) for t in (q, k, v))

    def make_step(transport):
        def step():
            if world == 1:
                out = nb.na3d(q, k, v, kernel_size=ks, dilation=dl, is_causal=ca)
            else:
                out = sharding.na_sharded(q, k, v, T, ks, dl, ca, transport=transport)
            return torch.autograd.grad(out, (q, k, v), cot)
        return step

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(step, trace):
        for _ in range(max(args.warmup, 3)):
            step()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        barrier()
        if trace:
            _lib.trace_report()
            _lib.trace_enable(True)               # per-kernel device times of this rank (events around each launch)
        count0 = _lib.launch_count()
        for a, b in evs:
            flush.zero_()
            if world > 1:
                dist.barrier()                    # every rank starts a step together: the halo exchange is inside it
            a.record()
            step()
            b.record()
        barrier()
        count = _lib.launch_count() - count0
        kernels = None
        if trace:
            _lib.trace_enable(False)
            kernels = {k: {"launches": n, "ms_per_launch": t / n} for k, (n, t) in sorted(_lib.trace_report().items())}
        ms = sum(a.elapsed_time(b) for a, b in evs) / args.steps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, kernels, count

    # the same step with NCCL send/recv as the transport, for comparison (untraced, before the measured run)
    ms_p2p = timed(make_step("p2p"), False)[0] if world > 1 else None
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms, kernels, launches = timed(make_step("auto"), True)
    transport = "none (one rank)" if world == 1 else (
        "the library's copy kernel into the neighbour's symmetric memory, flag barriers"
        if sharding.peer_transport() is not None else "NCCL send/recv")
    if _lib.kernel_status() != 0:
        raise RuntimeError("a bounded wait of a kernel ran out during the timed region")
    clocks = sampler.stop() if rank == 0 else None
    if rank != 0:
        return
    flops = flops_step(w)
    print(json.dumps({
        "metric": "na_fwd_bwd_effective_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["label"] + f", sharded along T over {world} rank(s)", "halo_transport": transport,
                   "ms_per_step_nccl_send_recv": ms_p2p,
                   "planes_per_rank": [bounds[r + 1] - bounds[r] for r in range(world)],
                   "l2": "256 MiB buffer written between timed iterations", "kernel_family": _lib.last_path()},
        "roofline": None, "kernels_rank0": kernels, "cpu_baseline": None, "e2e": None, "gpu_launches": int(launches),
        "clocks": clocks}))


# ---------------------------------------------------------------------------
# the variable-size GQA batch with extra tokens over several GPUs: whole samples per rank, balanced by token
# count, no collective on the data path
# ---------------------------------------------------------------------------
def run_varlen_sharded(args, rank, world, local_rank):
    import torch.distributed as dist
    import natten_mlx_b200 as nb
    from natten_mlx_b200 import _lib, sharding

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    B, M, Hq, Hkv, D, NX = 16, 128, 16, 4, 128, 64
    gen = torch.Generator().manual_seed(1236)
    sizes = (torch.randint(0, 9, (B, 2), generator=gen) * 8 + 64).to(torch.int32)     # the same draw as on one GPU
    host_all = [tuple(int(x) for x in r) for r in sizes.tolist()]
    parts = sharding.balance_by_tokens(host_all, world)
    mine = parts[rank]
    host_sizes = [host_all[i] for i in mine]
    n = len(mine)
    gen = torch.Generator().manual_seed(2236 + rank)
    bf = torch.bfloat16
    rnd = lambda shape: torch.randn(shape, generator=gen, dtype=torch.float32).to(bf).to(dev)
    q = rnd((n, M, M, Hq, D)).requires_grad_(True)
    k, v = (rnd((n, M, M, Hkv, D)).requires_grad_(True) for _ in range(2))
    ak, av = (rnd((n, NX, Hkv, D)).requires_grad_(True) for _ in range(2))
    cot = rnd((n, M, M, Hq, D))
    st = torch.tensor(host_sizes, dtype=torch.int32, device=dev)
    nb.tune.tune_fused(q.detach(), k.detach(), v.detach(), 13, 2, sizes=st, host_sizes=host_sizes,
                       additional_keys=ak.detach(), additional_values=av.detach())

    def step():
        out = nb.na2d_varlen(q, k, v, st, 13, 2, additional_keys=ak, additional_values=av, host_sizes=host_sizes)
        return torch.autograd.grad(out, (q, k, v, ak, av), cot)

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    dist.barrier()
    torch.cuda.synchronize()
    count0 = _lib.launch_count()
    for a, b in evs:
        flush.zero_()
        a.record()
        step()
        b.record()
    dist.barrier()
    torch.cuda.synchronize()
    launches = _lib.launch_count() - count0
    t = torch.tensor([sum(a.elapsed_time(b) for a, b in evs) / args.steps], device=dev)
    per_rank = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(per_rank, t)
    ms = max(float(x.item()) for x in per_rank)
    clocks = sampler.stop() if rank == 0 else None
    if _lib.kernel_status() != 0:
        raise RuntimeError("a bounded wait of a kernel ran out during the timed region")
    if rank != 0:
        return
    tokens = [sum(host_all[i][0] * host_all[i][1] for i in p) for p in parts]
    flops = 3.5 * 4.0 * Hq * sum(tokens) * (169 + NX) * D
    print(json.dumps({
        "metric": "na_fwd_bwd_effective_tflops", "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"na2d bf16 varlen B=16 max 128x128 ({sum(tokens)} tokens) 16q/4kv heads D=128 K=13x13 dilation 2, "
                               f"64 extra tokens, lse+merge, fwd+bwd; whole samples per rank, balanced by tokens, no collective",
                   "samples_per_rank": [len(p) for p in parts], "tokens_per_rank": tokens,
                   "ms_per_step_per_rank": [float(x.item()) for x in per_rank],
                   "l2": "256 MiB buffer written between timed iterations", "kernel_family": _lib.last_path()},
        "roofline": None, "cpu_baseline": None, "e2e": None, "gpu_launches": int(launches), "clocks": clocks}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--short", action="store_true",
                    help="device-resident legs only (no end-to-end, CPU or video legs; `e2e` and `cpu_baseline` are null): "
                         "for profilers, which should see few launches")
    ap.add_argument("--no-tune", action="store_true",
                    help="skip the measured tiling choice of the warm-up (keeps the launch sequence short for profilers)")
    ap.add_argument("--workload", default="na2d_nat_stage",
                    choices=sorted(WORKLOADS) + list(TABLE_WORKLOADS) + ["na3d_video_tshard"])
    args = ap.parse_args()
    if args.workload == "na3d_video_tshard":
        rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "the sharded workload has no reference arm"}))
            return
        if world > 1:
            import torch.distributed as dist
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        try:
            run_tshard(args, rank, world, local_rank)
        finally:
            if world > 1:
                import torch.distributed as dist
                dist.destroy_process_group()
        return
    if args.workload in TABLE_WORKLOADS:
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if args.impl == "reference":
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": "table workloads have no reference arm"}))
        elif args.workload == "na2d_varlen_gqa" and world > 1:
            import torch.distributed as dist
            local_rank = int(os.environ.get("LOCAL_RANK", "0"))
            torch.cuda.set_device(local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            try:
                run_varlen_sharded(args, int(os.environ.get("RANK", "0")), world, local_rank)
            finally:
                dist.destroy_process_group()
        elif int(os.environ.get("RANK", "0")) == 0:
            run_table_workload(args)
        return
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, w, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()

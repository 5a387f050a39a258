"""Benchmark of the hot path: weighted_laplace_sum forward at B=4, H=12, N=16384, D=Dv=64 (fp32).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one call of the operator on one batch of synthetic inputs (q, k ~ 2 N(0,1),
v ~ N(0,1), seed 0). Prints ONE JSON line. Metric: q.k pairs/s = P*D*N*M / time, whole job.

With N GPUs the 48 heads of the batch are split over the ranks (6 per GPU at 8): strong scaling,
no collective on the data path; time is the maximum over ranks of the CUDA-event time. The line
also carries the same figure with the results all-gathered to every rank (`with_gather`) and,
for comparison, the weak-scaling figure where every rank runs all 48 heads (`weak`).

--impl reference times the reference's own CPU-runnable path, the chunked compiled full-matrix
evaluation `_chunked(_normalized_compiled, "add_laplace", ...)` of its kernel_attention/attention.py,
imported unchanged from baseline/_ref/ (staged there by oracle/ref_python.py) on all host cores,
on a bounded sample of the workload per step. Where that folder is absent the restatement in
oracle/chunked_ref.py runs instead and the line says so (`cpu_baseline.kind`).

--workload ops prints a table of whole-operator device times at the other benchmark configurations
(reference protocol: 5 warm-up calls, 10 timed calls, CUDA events); with --with-ref-ext the
reference's own CUDA extensions (oracle/_ref, when built) are timed beside them on the same inputs.
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "quasi-linear-kernel-attention_b200"))

B, H, N, D, C = 4, 12, 16384, 64, 64
P = B * H
WORKLOAD = f"weighted_laplace_sum forward B={B} H={H} N=M={N} D={D} Dv={C} fp32 (q,k~2*N(0,1), v~N(0,1), seed 0)"


def algo_bytes(heads):
    """Every tensor once: q, k, v, out_w, out_u of `heads` heads."""
    return 4 * heads * (D * N + D * N + N * C + N * C + N)


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


# ------------------------------------------------------------------ CPU arm: the reference's chunked compiled path
class CpuArm:
    """One head, `m_sample` of the N queries against all N keys per call; pairs/s scale linearly in both."""

    def __init__(self, m_sample):
        torch.set_num_threads(host_cores())            # (a launcher may have exported OMP_NUM_THREADS=1)
        self.m = m_sample
        g = torch.Generator().manual_seed(0)
        self.q = torch.randn(1, D, m_sample, generator=g) * 2
        self.k = torch.randn(1, D, N, generator=g) * 2
        self.v = torch.randn(1, N, C, generator=g)
        self.kind, self.att = "port", None
        try:
            from oracle import ref_python
            self.att = ref_python.load(stub_extensions=True)
        except Exception as e:                         # the staged files are there but do not import
            self.note = f"reference import failed: {type(e).__name__}: {e}"
        if self.att is not None:
            self.kind = "reference"
        self.pairs = 1 * D * N * m_sample

    def call(self):
        with torch.no_grad():
            if self.att is not None:
                return self.att._chunked(self.att._normalized_compiled, "add_laplace", self.q, self.k, self.v, 1.0, None, D)
            from oracle import chunked_ref
            return chunked_ref.laplace_sum_chunked(self.q, self.k, self.v)

    def warm(self):
        """One untimed call: absorbs the inductor compile of the reference's chunk function (about a minute)."""
        try:
            self.call()
        except Exception as e:
            if self.att is None:
                raise
            self.att, self.kind = None, "port"          # e.g. no working C++ compiler for inductor on this host
            self.note = f"reference path failed ({type(e).__name__}); restatement timed instead"
            self.call()

    def timed(self):
        t0 = time.perf_counter()
        self.call()
        return time.perf_counter() - t0

    def describe(self, secs):
        what = ("the reference's _chunked(_normalized_compiled, 'add_laplace') imported unchanged (torch.compile, dynamic shapes)"
                if self.kind == "reference" else "oracle/chunked_ref.py, a restatement of the reference's chunked full-matrix path")
        s = f"1 head x {self.m} of {N} queries against all {N} keys, D={D}, C={C}; {secs:.2f} s per call; {what}; scaled by pairs"
        return s + (f"; {self.note}" if getattr(self, "note", None) else "")


def cpu_baseline(m_sample=4096, repeats=3):
    arm = CpuArm(m_sample)
    arm.warm()
    best = min(arm.timed() for _ in range(repeats))
    return {"value": arm.pairs / best, "unit": "pairs/s", "cores": torch.get_num_threads(), "kind": arm.kind,
            "sample": arm.describe(best)}


def run_reference(args, rank):
    if rank != 0:
        return
    arm = CpuArm(4096)
    arm.warm()
    for _ in range(max(0, args.warmup - 1)):
        arm.timed()
    times = [arm.timed() for _ in range(args.steps)]
    med = statistics.median(times)
    val = arm.pairs / med
    cb = {"value": val, "unit": "pairs/s", "cores": torch.get_num_threads(), "kind": arm.kind, "sample": arm.describe(med)}
    line = {"impl": "reference", "metric": "q.k pairs/s", "value": val, "unit": "pairs/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * med,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "note": "CPU host cores, bounded sample per step (1 head x 4096 queries), scaled by pairs"},
            "cpu_baseline": cb,
            "e2e": {"value": val, "unit": "pairs/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "50"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------ the training-step workload (not the headline)
def run_abs_fwd_bwd(args):
    """weighted_abs_sum_full forward + backward at B=8, H=12, N=4096, D=Dv=64 (the add_riesz training step of the
    reference's configurations): one GPU, device-resident inputs, one JSON line of the same shape without the host legs."""
    from weighted_abs_sum import weighted_abs_sum_full
    Pc, Dc, Nc, Cc = 8 * 12, 64, 4096, 64
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(0)
    q = (torch.randn(Pc, Dc, Nc, generator=g) * 0.5).to(dev).requires_grad_(True)
    k = (torch.randn(Pc, Dc, Nc, generator=g) * 0.5).to(dev).requires_grad_(True)
    v = torch.randn(Pc, Nc, Cc, generator=g).to(dev).requires_grad_(True)
    g_w = torch.randn(Pc, Nc, Cc, generator=g).to(dev)
    g_u = torch.randn(Pc, Nc, generator=g).to(dev)

    def step():
        q.grad = k.grad = v.grad = None
        out_w, out_u = weighted_abs_sum_full(q, k, v)
        torch.autograd.backward((out_w, out_u), (g_w, g_u))

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clocks:
        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            step()                                      # inputs and gradients (7 x 96 MiB + 2 x 1.5 MiB) exceed the 126 MB L2
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
    peak, which = measured_peaks()
    pairs = Pc * Dc * Nc * Nc
    # every tensor once: forward reads q, k, v and writes out_w, out_u; backward reads q, k, v, g_w, g_u and writes three gradients
    algo = 4 * Pc * ((Dc * Nc * 2 + Nc * Cc * 2 + Nc) + (Dc * Nc * 4 + Nc * Cc * 3 + Nc))
    achieved = algo / (ms * 1e-3) / 1e9
    line = {"metric": "q.k pairs/s", "value": pairs / (ms * 1e-3), "unit": "pairs/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "weighted_abs_sum_full forward+backward B=8 H=12 N=M=4096 D=64 Dv=64 fp32 (q,k~0.5*N(0,1), v,g~N(0,1), seed 0)",
                       "l2": "inputs larger than L2"},
            "clocks": clocks.summary(), "gpu_launches": 16 * args.steps,      # 6 kernels of the forward, 10 of the backward
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_source": which, "algorithmic_bytes": algo, "kernel": "whole forward+backward step"}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ operator table, optionally beside the reference's extensions
def run_ops_table(args):
    """Whole-operator device times at the benchmark configurations, the reference's protocol
    (Experiments/speed_and_memory/bench.py:83-121: 5 warm-up calls, 10 timed calls, one CUDA-event pair per call)."""
    import qlka_native
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    ref = {}
    if args.with_ref_ext:
        from oracle import build_ref
        ref = build_ref.load_ref()

    def timed(fn, warm=5, runs=10):
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(runs):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.mean(ts), statistics.pstdev(ts)

    def inputs(Pc, Dc, Nc, Cc, scale, uniform=False):
        g = torch.Generator(device="cuda").manual_seed(0)
        if uniform:
            q = (torch.rand(Pc, Dc, Nc, generator=g, device=dev) * 6 - 3)
            k = (torch.rand(Pc, Dc, Nc, generator=g, device=dev) * 6 - 3)
        else:
            q = torch.randn(Pc, Dc, Nc, generator=g, device=dev) * scale
            k = torch.randn(Pc, Dc, Nc, generator=g, device=dev) * scale
        v = torch.randn(Pc, Nc, Cc, generator=g, device=dev)
        g_w = torch.randn(Pc, Nc, Cc, generator=g, device=dev)
        g_u = torch.randn(Pc, Nc, generator=g, device=dev)
        return q, k, v, g_w, g_u

    configs = [   # name, (P, D, N, C), input scale, uniform inputs, operators
        ("c1 B=1 H=4 N=1024 D=Dv=32", (4, 32, 1024, 32), 1.0, False, ["laplace_fwd"]),
        ("c2 B=8 H=12 N=4096 D=Dv=64", (96, 64, 4096, 64), 0.5, False, ["abs_fwd", "abs_full_fwd", "abs_bwd", "abs_full_bwd"]),
        ("c3 B=4 H=12 N=16384 D=Dv=64", (48, 64, 16384, 64), 2.0, False, ["laplace_fwd", "abs_full_fwd"]),
        ("c5a B=1 H=16 N=65536 D=Dv=64", (16, 64, 65536, 64), 1.0, False, ["laplace_fwd", "abs_full_fwd"]),
        ("c5a B=1 H=16 N=262144 D=Dv=64", (16, 64, 262144, 64), 1.0, False, ["laplace_fwd", "abs_full_fwd"]),
        ("c5b B=256 H=1 N=600 D=Dv=64", (256, 64, 600, 64), 1.0, True, ["abs_full_fwd", "bump_three_calls", "bump_one_sort"]),
    ]
    rows = []
    for name, (Pc, Dc, Nc, Cc), scale, uniform, ops in configs:
        if args.ops_filter and args.ops_filter not in name:
            continue
        q, k, v, g_w, g_u = inputs(Pc, Dc, Nc, Cc, scale, uniform)
        for op in ops:
            ours = {
                "laplace_fwd": lambda: qlka_native.laplace_forward(q, k, v),
                "abs_fwd": lambda: qlka_native.abs_forward(q, k, v, full=False),
                "abs_full_fwd": lambda: qlka_native.abs_forward(q, k, v, full=True),
                "abs_bwd": lambda: qlka_native.abs_backward(q, k, v, g_w),
                "abs_full_bwd": lambda: qlka_native.abs_backward(q, k, v, g_w, g_u),
                "bump_three_calls": lambda: [qlka_native.abs_forward(q + s, k, v, full=True) for s in (0.0, 1.0, -1.0)],
                "bump_one_sort": lambda: qlka_native.abs_shifted_forward(q, k, v, (0.0, 1.0, -1.0), (-1.0, 0.5, 0.5)),
            }[op]
            theirs = None
            if ref and Nc <= 131072:               # the reference refuses longer sequences (binding.cpp:77-79)
                theirs = {
                    "laplace_fwd": lambda: ref["laplace"].weighted_laplace_sum_forward(q, k, v),
                    "abs_fwd": lambda: ref["abs"].weighted_abs_sum_forward(q, k, v, -1),
                    "abs_full_fwd": lambda: ref["abs"].weighted_abs_sum_full_forward(q, k, v, -1),
                    "abs_bwd": lambda: ref["abs"].weighted_abs_sum_backward(q, k, v, g_w),
                    "abs_full_bwd": lambda: ref["abs"].weighted_abs_sum_full_backward(q, k, v, g_w, g_u),
                    "bump_three_calls": lambda: [ref["abs"].weighted_abs_sum_full_forward(q + s, k, v, -1) for s in (0.0, 1.0, -1.0)],
                    "bump_one_sort": None,
                }[op]
            m, s = timed(ours)
            row = {"config": name, "op": op, "ours_ms": round(m, 4), "ours_std_ms": round(s, 4),
                   "pairs_per_s": Pc * Dc * Nc * Nc * (3 if op.startswith("bump") else 1) / (m * 1e-3)}
            if theirs is not None:
                m2, s2 = timed(theirs)
                row.update(ref_ext_ms=round(m2, 4), ref_ext_std_ms=round(s2, 4), speedup=round(m2 / m, 3))
            rows.append(row)
            print(json.dumps(row), file=sys.stderr, flush=True)
        del q, k, v, g_w, g_u
        torch.cuda.empty_cache()
    print(json.dumps({"workload": "ops", "protocol": "5 warm-up + 10 timed calls, CUDA events per call, mean and std",
                      "ref_ext": bool(ref), "gpu": torch.cuda.get_device_name(0), "rows": rows}), flush=True)


# ------------------------------------------------------------------ ours
def run_ours(args, rank, world, local_rank):
    import qlka_native
    import sharding
    from weighted_laplace_sum import weighted_laplace_sum

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    lo, hi = sharding.shard_range(P, rank, world)
    Ps = hi - lo                                                # heads of this rank
    g = torch.Generator().manual_seed(0)                        # the same 48 heads on every rank; a rank keeps its slice
    q_all = torch.randn(P, D, N, generator=g) * 2
    k_all = torch.randn(P, D, N, generator=g) * 2
    v_all = torch.randn(P, N, C, generator=g)
    q_h, k_h, v_h = q_all[lo:hi].clone().pin_memory(), k_all[lo:hi].clone().pin_memory(), v_all[lo:hi].clone().pin_memory()
    q, k, v = q_h.to(dev), k_h.to(dev), v_h.to(dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            return t.item()
        return ms

    def timed_loop(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / steps

    warm = max(args.warmup, 3)
    # the clock sampler runs from the warm-up to the end of the per-kernel timing: all of it is under load
    with ClockSampler(local_rank) as clocks:
        for _ in range(warm):
            weighted_laplace_sum(q, k, v)
        ms = timed_loop(lambda: weighted_laplace_sum(q, k, v), args.steps)     # one rank's inputs: 3 x Ps x 4 MiB, larger than L2 down to 8 GPUs
        # per-kernel split, same inputs, separate short loop
        stage = qlka_native.laplace_stage_times(q, k, v, reps=max(3, min(args.steps, 10)))
    clk = clocks.summary()

    # the same with the results gathered to every rank (NCCL all_gather of out_w and out_u)
    with_gather = None
    if world > 1 and P % world == 0:             # (all_gather_into_tensor wants equal slices)
        gw = torch.empty(P, N, C, device=dev)
        gu = torch.empty(P, N, device=dev)

        def step_gather():
            ow, ou = weighted_laplace_sum(q, k, v)
            torch.distributed.all_gather_into_tensor(gw, ow)
            torch.distributed.all_gather_into_tensor(gu, ou)

        for _ in range(2):
            step_gather()
        ms_g = timed_loop(step_gather, max(3, min(args.steps, 10)))
        with_gather = {"ms_per_step": ms_g, "value": float(P) * D * N * N / (ms_g * 1e-3), "unit": "pairs/s",
                       "gather_ms": ms_g - ms, "gathered_bytes_per_rank": 4 * P * N * (C + 1)}
        del gw, gu

    # weak scaling, for comparison: every rank runs all 48 heads
    weak = None
    if world > 1:
        qf, kf, vf = q_all.to(dev), k_all.to(dev), v_all.to(dev)
        for _ in range(2):
            weighted_laplace_sum(qf, kf, vf)
        ms_w = timed_loop(lambda: weighted_laplace_sum(qf, kf, vf), max(3, min(args.steps, 10)))
        weak = {"ms_per_step": ms_w, "value": float(P) * world * D * N * N / (ms_w * 1e-3), "unit": "pairs/s", "heads_per_gpu": P}
        del qf, kf, vf
    del q_all, k_all, v_all

    # end to end: pinned host buffers in, results back on the host, every step; each rank moves its own heads
    out_w_h = torch.empty(Ps, N, C).pin_memory()
    out_u_h = torch.empty(Ps, N).pin_memory()
    n_e2e = max(2, min(args.steps, 5))
    # the host-buffer entry of the library: heads stream through copy / compute / copy-back in chunks
    pipe = qlka_native.HostPipeline(Ps, D, N, N, C, chunk=max(1, Ps // 12), device=dev)
    ms_e2e = float("nan")
    if not args.no_e2e:
        pipe(q_h, k_h, v_h, out_w_h, out_u_h)
        ms_e2e = timed_loop(lambda: pipe(q_h, k_h, v_h, out_w_h, out_u_h), n_e2e)
    h2d = torch.tensor([4.0 * (q_h.numel() + k_h.numel() + v_h.numel())], device=dev, dtype=torch.float64)
    d2h = torch.tensor([4.0 * (out_w_h.numel() + out_u_h.numel())], device=dev, dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(h2d)
        torch.distributed.all_reduce(d2h)

    if rank != 0:
        return
    pairs = float(P) * D * N * N
    peak, which = measured_peaks()
    ab = algo_bytes(Ps)                                          # per launch: the heads one rank's kernels process
    achieved_op = ab / (ms * 1e-3) / 1e9
    # dominant kernel: the emitting pass of the walk; its launch time is measured live by the stage-timing entry point
    achieved = ab / (stage["walk_pass2_ms"] * 1e-3) / 1e9
    # DRAM traffic of one launch of the dominant kernel (from an ncu capture at 12 heads, scaled by the heads of a
    # launch: every array the kernel touches grows in proportion to them)
    traffic = WALK_DRAM_BYTES_PER_HEAD * Ps
    sm_clock = 1e6 * (clk.get("sm_max_mhz") or 1965.0)
    line = {
        "metric": "q.k pairs/s", "value": pairs / (ms * 1e-3), "unit": "pairs/s", "n_gpus": world,
        "steps": args.steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "heads_total": P, "heads_per_gpu": Ps,
                   "l2": f"inputs larger than L2 (3 x {Ps * D * N * 4 >> 20} MiB per rank and step)",
                   "sharding": "the batch*head dimension split across ranks, no data-path collective"},
        "clocks": clk,
        "e2e": {"value": pairs / (ms_e2e * 1e-3), "unit": "pairs/s", "ms_per_step": ms_e2e, "steps": n_e2e,
                "h2d_bytes_per_step": int(h2d.item()), "d2h_bytes_per_step": int(d2h.item())},
        "gpu_launches": 4 * args.steps,          # sort/rank, first walk pass, fold, second walk pass
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "peak_source": which, "algorithmic_bytes": ab,
                     "kernel": "laplace_pass2 (dominant kernel; launch time from CUDA events on the launching stream)",
                     "operator_achieved": achieved_op, "operator_frac": achieved_op / peak,
                     "stage_ms": stage,
                     # ceilings of this formulation that sit far below the HBM one (per launch, this rank's heads):
                     # issue slots of the packed fp32 recurrences and emission ((4 N + 2 M) C / 2 per segment), and the
                     # L2 floor: two 256-byte-row gathers and one row reduction per segment at the rates a bare
                     # gather / vector-reduction loop reaches on this GPU (17.2 and 6.1 TB/s, overlapped: 3.03 ms for 48 heads)
                     "fp32_floor_ms": 1e3 * Ps * D * (4 * N + 2 * N) * C / 2 / (148 * 128 * sm_clock),
                     "l2_floor_ms": L2_FLOOR_MS_PER_HEAD * Ps},
    }
    if with_gather:
        line["with_gather"] = with_gather
    if weak:
        line["weak"] = weak
    if not args.no_cpu and world == 1:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line), flush=True)


# figures from a profiler capture of the dominant kernel (dram__bytes_read + dram__bytes_write of one laplace_pass2 launch over
# 12 heads: 845.7 MB + 43.3 MB) and from a bare gather / reduction loop with the walk's access pattern (two row gathers and one
# row reduction per segment, 48 heads: 3.03 ms), both on a B200
WALK_DRAM_BYTES_PER_HEAD = (845.66e6 + 43.32e6) / 12
L2_FLOOR_MS_PER_HEAD = 3.034 / 48


def main():
    global B, P, WORKLOAD
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--batch", type=int, default=B, help="B of the workload (default: the benchmark's 4; smaller for profiler captures)")
    ap.add_argument("--workload", default="laplace_fwd", choices=["laplace_fwd", "abs_fwd_bwd", "ops"],
                    help="laplace_fwd: the headline benchmark (default); abs_fwd_bwd: the abs-sum training step, one GPU, device timing only; "
                         "ops: table of operator times at the other configurations")
    ap.add_argument("--with-ref-ext", action="store_true", help="ops table: time the reference's CUDA extensions (oracle/_ref) beside ours")
    ap.add_argument("--ops-filter", default="", help="ops table: only configurations whose name contains this text")
    args = ap.parse_args()
    if args.batch != B:
        B = args.batch
        P = B * H
        WORKLOAD = WORKLOAD.replace("B=4", f"B={B}")

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "abs_fwd_bwd":
        if rank == 0:
            run_abs_fwd_bwd(args)
        return
    if args.workload == "ops":
        if rank == 0:
            run_ops_table(args)
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()

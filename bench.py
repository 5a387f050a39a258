"""Benchmark of the hot path: weighted_laplace_sum forward at B=4, H=12, N=16384, D=Dv=64 (fp32).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one call of the operator on one batch of synthetic inputs (q, k ~ 2 N(0,1),
v ~ N(0,1), seed 0). Prints ONE JSON line. Metric: q.k pairs/s = P*D*N*M / time, whole job.
With N GPUs every rank runs the same per-GPU batch on its own heads (weak scaling, no
collective on the data path); time is the maximum over ranks of the CUDA-event time.

--impl reference times the reference's CPU-runnable path (chunked full-matrix evaluation,
restated in oracle/chunked_ref.py) on the host cores, on a bounded sample of the workload.
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
ALGO_BYTES = 4 * P * (D * N + D * N + N * C + N * C + N)      # every tensor once: q, k, v, out_w, out_u


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ------------------------------------------------------------------ CPU baseline (reference path restated)
def cpu_baseline(p_sample=1, m_sample=16384, repeats=1):
    from oracle import chunked_ref
    g = torch.Generator().manual_seed(0)
    q = torch.randn(p_sample, D, m_sample, generator=g) * 2
    k = torch.randn(p_sample, D, N, generator=g) * 2
    v = torch.randn(p_sample, N, C, generator=g)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        chunked_ref.laplace_sum_chunked(q, k, v)
        best = min(best, time.perf_counter() - t0)
    pairs = p_sample * D * N * m_sample
    return {"value": pairs / best, "unit": "pairs/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{p_sample} head(s) x {m_sample} of {N} queries against all {N} keys, D={D}, C={C}; "
                      f"{best:.2f} s; the reference's chunked full-matrix path (oracle/chunked_ref.py), scaled by pairs"}


def run_reference(args, rank):
    if rank != 0:
        return
    for _ in range(args.warmup and 1):
        cpu_baseline(1, 256)
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        cb = cpu_baseline(1, 1024)
        times.append(time.perf_counter() - t0)
    val = statistics.median([1 * D * N * 1024 / t for t in times])
    cb["value"] = val
    cb["sample"] = f"1 head x 1024 of {N} queries against all {N} keys per step (oracle/chunked_ref.py, the reference's chunked full-matrix path)"
    line = {"impl": "reference", "metric": "q.k pairs/s", "value": val, "unit": "pairs/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * statistics.median(times),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "note": "CPU host cores, bounded sample per step"},
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


# ------------------------------------------------------------------ ours
def run_ours(args, rank, world, local_rank):
    import qlka_native
    from weighted_laplace_sum import weighted_laplace_sum

    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(1000 * rank)             # rank r owns heads [r*P, (r+1)*P) of the job
    q_h = (torch.randn(P, D, N, generator=g) * 2).pin_memory()
    k_h = (torch.randn(P, D, N, generator=g) * 2).pin_memory()
    v_h = torch.randn(P, N, C, generator=g).pin_memory()
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

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # the clock sampler runs from the warm-up to the end of the per-kernel timing: all of it is under load
    with ClockSampler(local_rank) as clocks:
        for _ in range(max(args.warmup, 3)):
            weighted_laplace_sum(q, k, v)
        barrier()
        e0.record()
        for _ in range(args.steps):
            out_w, out_u = weighted_laplace_sum(q, k, v)     # inputs (3 x 192 MiB) exceed the 126 MB L2
        e1.record()
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
        # per-kernel split, same inputs, separate short loop
        stage = qlka_native.laplace_stage_times(q, k, v, reps=max(3, min(args.steps, 10)))
    clk = clocks.summary()

    # end to end: pinned host buffers in, results back on the host, every step
    out_w_h = torch.empty(P, N, C).pin_memory()
    out_u_h = torch.empty(P, N).pin_memory()
    n_e2e = max(2, min(args.steps, 5))

    # the host-buffer entry of the library: heads stream through copy / compute / copy-back in chunks
    pipe = qlka_native.HostPipeline(P, D, N, N, C, chunk=max(1, P // 12), device=dev)      # (12 chunks measured best: 12.9 ms against 13.5 ms for 6)

    def e2e_step():
        pipe(q_h, k_h, v_h, out_w_h, out_u_h)

    ms_e2e = float("nan")
    if not args.no_e2e:
        e2e_step()
        barrier()
        e0.record()
        for _ in range(n_e2e):
            e2e_step()
        e1.record()
        barrier()
        ms_e2e = max_over_ranks(e0.elapsed_time(e1)) / n_e2e

    if rank != 0:
        return
    pairs = float(P) * D * N * N * world
    peak, which = measured_peaks()
    achieved_op = ALGO_BYTES / (ms * 1e-3) / 1e9
    # dominant kernel: the walk (60 % of the device time, profiles/); its launch time is measured live
    achieved = ALGO_BYTES / (stage["walk_ms"] * 1e-3) / 1e9
    # DRAM traffic of one walk launch: dram__bytes_read + dram__bytes_write of an ncu capture at the benchmark size
    # (6.07 GB at B=4, profiles/laplace_forward_b4_h12_n16384_ncu.md); other batches scale it, every array grows with P
    traffic = 6.07e9 * B / 4
    line = {
        "metric": "q.k pairs/s", "value": pairs / (ms * 1e-3), "unit": "pairs/s", "n_gpus": world,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "heads_per_gpu": P, "l2": f"inputs larger than L2 (3 x {P * D * N * 4 >> 20} MiB per step)",
                   "sharding": "batch*head across ranks, no data-path collective"},
        "clocks": clk,
        "e2e": {"value": pairs / (ms_e2e * 1e-3), "unit": "pairs/s", "ms_per_step": ms_e2e, "steps": n_e2e,
                "h2d_bytes_per_step": 4 * (q_h.numel() + k_h.numel() + v_h.numel()),
                "d2h_bytes_per_step": 4 * (out_w_h.numel() + out_u_h.numel())},
        "gpu_launches": 2 * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic, "peak_source": which, "algorithmic_bytes": ALGO_BYTES,
                     "kernel": "laplace_walk (dominant kernel; launch time from CUDA events on the launching stream)",
                     "operator_achieved": achieved_op, "operator_frac": achieved_op / peak,
                     "stage_ms": stage},
    }
    if not args.no_cpu and world == 1:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line), flush=True)


def main():
    global B, P, WORKLOAD, ALGO_BYTES
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--batch", type=int, default=B, help="B of the workload (default: the benchmark's 4; smaller for profiler captures)")
    ap.add_argument("--workload", default="laplace_fwd", choices=["laplace_fwd", "abs_fwd_bwd"],
                    help="laplace_fwd: the headline benchmark (default); abs_fwd_bwd: the abs-sum training step, one GPU, device timing only")
    args = ap.parse_args()
    if args.batch != B:
        B = args.batch
        P = B * H
        WORKLOAD = WORKLOAD.replace("B=4", f"B={B}")
        ALGO_BYTES = 4 * P * (D * N + D * N + N * C + N * C + N)

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

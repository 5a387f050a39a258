"""Speed and memory sweep of kernel attention against softmax attention, with the reference's protocol
(Experiments/speed_and_memory/bench.py:22-42,83-121): B=4, H=12, D=C=64, N = 2^7 .. 2^17, CUDA events,
5 warm-up calls, 10 timed calls, mean and standard deviation, peak memory above the inputs; forward and
forward+backward for add_laplace (the reference times it forward only: it has no backward), add_riesz and softmax. Rows are appended to a CSV and
sizes already present in it are skipped (bench.py:128-131,141). The pykeops columns of the reference are
absent: this library has no keops backend.

    python quasi-linear-kernel-attention_b200/kernel_attention/speed_and_memory.py [--out results.csv] [--max_log2 17]
"""

import argparse
import csv
import os
import statistics
import sys

import torch
import torch.nn.functional as F

WARMUP, RUNS = 5, 10
B, H, D = 4, 12, 64


def measure(fn, backward):
    def step():
        out = fn()
        if backward:
            out.sum().backward()
    for _ in range(WARMUP):
        step()
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    times = []
    for _ in range(RUNS):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    return statistics.mean(times), statistics.pstdev(times), (torch.cuda.max_memory_allocated() - base) / 2 ** 20


def main():
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, here)
    from kernel_attention import TAU, attention
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="speed_and_memory.csv")
    ap.add_argument("--min_log2", type=int, default=7)
    ap.add_argument("--max_log2", type=int, default=17)
    a = ap.parse_args()
    done = set()
    if os.path.exists(a.out):
        done = {(r["method"], r["mode"], int(r["N"])) for r in csv.DictReader(open(a.out))}
    fields = ["method", "mode", "N", "ms_mean", "ms_std", "peak_mib"]
    new = not os.path.exists(a.out)
    with open(a.out, "a", newline="") as f:
        w = csv.DictWriter(f, fieldnames=fields)
        if new:
            w.writeheader()
        for lg in range(a.min_log2, a.max_log2 + 1):
            N = 1 << lg
            for method, modes in (("add_laplace", ("fwd", "fwd+bwd")), ("add_riesz", ("fwd", "fwd+bwd")), ("softmax", ("fwd", "fwd+bwd"))):
                for mode in modes:
                    if (method, mode, N) in done:
                        continue
                    bwd = mode == "fwd+bwd"
                    try:
                        q, k, v = (torch.randn(B, H, N, D, device="cuda", requires_grad=bwd) for _ in range(3))
                        if method == "softmax":
                            fn = lambda: F.scaled_dot_product_attention(q, k, v)
                        else:
                            fn = lambda: attention(q, k, v, method, TAU[method])
                        with torch.set_grad_enabled(bwd):
                            ms, sd, mib = measure(fn, bwd)
                        w.writerow(dict(method=method, mode=mode, N=N, ms_mean=f"{ms:.4f}", ms_std=f"{sd:.4f}", peak_mib=f"{mib:.1f}"))
                    except RuntimeError as e:          # out of memory or a size limit: record and go on
                        w.writerow(dict(method=method, mode=mode, N=N, ms_mean="nan", ms_std="nan", peak_mib=str(e)[:60]))
                    f.flush()
                    print(method, mode, N, flush=True)


if __name__ == "__main__":
    main()

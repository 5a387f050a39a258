"""Speed and memory sweep of kernel attention against softmax attention with the reference's protocol and
CSV layout (Experiments/speed_and_memory/bench.py:22-42, 83-121, 134-158): B=4, H=12, D=C=64,
N = 2^7 .. 2^17, fp32, CUDA events, 5 warm-up calls, 10 timed calls, mean and standard deviation, peak memory;
one row per (method, backend, dtype, B, H, D, C, N, mode, gpu), appended to --out, rows already there skipped.

Methods and backends:
  add_laplace / add_riesz   "qlka"        this library through `kernel_attention.attention` (fused native call
                                           forward, differentiable operators forward+backward; the reference times
                                           add_laplace forward only because its operator has no backward)
  add_laplace / add_riesz   "qlka-ops"    this library's operators inside the reference's own harness functions
                                           (layout change + .contiguous() + operator + normalisation in the timed region)
  add_laplace / add_riesz   "ref-ext"     the same harness functions over a build of the reference's CUDA extensions,
                                           only with --ref-ext-dir DIR (DIR/ref_laplace_ext/ref_laplace_ext.so and
                                           DIR/ref_abs_ext/ref_abs_ext.so); forward only, N <= 131072
  softmax                   "MEM_EFF" fp32, "FLASH" fp16   torch scaled_dot_product_attention
The reference's pykeops rows are absent: this library has no keops backend.

    python quasi-linear-kernel-attention_b200/kernel_attention/speed_and_memory.py [--sizes 128 1024 ...] [--out results.csv]
"""

import argparse
import csv
import datetime
import importlib.util
import math
import os
import socket
import sys

import torch
import torch.nn.functional as F
from torch.nn.attention import SDPBackend, sdpa_kernel

KEY = ["method", "backend", "dtype", "B", "H", "D", "C", "N", "mode", "gpu"]
FIELDS = KEY + ["time_mean_ms", "time_std_ms", "peak_mem_mb", "runs", "warmups", "hostname", "torch", "cuda", "cudnn", "date"]
LAPLACE_TAU = 0.5
SDPA = {"MEM_EFF": SDPBackend.EFFICIENT_ATTENTION, "FLASH": SDPBackend.FLASH_ATTENTION}
DTYPES = {"fp32": torch.float32, "fp16": torch.float16}


def _to_operator_layout(q, k, v, scale=1.0):
    """(B, H, S, D) -> q, k (P, D, S) and v (P, S, C), materialised, as the reference's harness does inside its timed region."""
    B, H, M, D = q.shape
    N, C = v.shape[2], v.shape[3]
    qs = (q * scale if scale != 1.0 else q).reshape(B * H, M, D).transpose(1, 2).contiguous()
    ks = (k * scale if scale != 1.0 else k).reshape(B * H, N, D).transpose(1, 2).contiguous()
    return qs, ks, v.reshape(B * H, N, C).contiguous()


def riesz_via_operator(abs_sum_full):
    """add_riesz attention with eps = 0 around an abs-sum operator returning (out_w, out_u)."""
    def fn(q, k, v):
        B, H, M, _ = q.shape
        qs, ks, vs = _to_operator_layout(q, k, v)
        qn, kn = qs.abs().sum(dim=1), ks.abs().sum(dim=1)
        dist_v, dist_1 = abs_sum_full(qs, ks, vs)
        num = torch.einsum("pn,pnc->pc", kn, vs).unsqueeze(1) + qn.unsqueeze(2) * vs.sum(dim=1).unsqueeze(1) - dist_v
        row = kn.sum(dim=1, keepdim=True) + qn * ks.shape[2] - dist_1
        return (num / row.clamp(min=1e-6).unsqueeze(2)).reshape(B, H, M, -1)
    return fn


def laplace_via_operator(laplace_sum):
    def fn(q, k, v):
        B, H, M, _ = q.shape
        qs, ks, vs = _to_operator_layout(q, k, v, 1.0 / LAPLACE_TAU)
        out_w, out_u = laplace_sum(qs, ks, vs)
        return (out_w / out_u.clamp(min=1e-6).unsqueeze(2)).reshape(B, H, M, -1)
    return fn


def _load_ext(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def build_methods(ref_ext_dir):
    """[(method, backend, dtype, attention function, has a backward, largest N)]"""
    from kernel_attention import TAU, attention
    from weighted_abs_sum import weighted_abs_sum_full
    from weighted_laplace_sum import weighted_laplace_sum
    rows = [("add_laplace", "qlka", "fp32", lambda q, k, v: attention(q, k, v, "add_laplace", LAPLACE_TAU), True, 262144),
            ("add_riesz", "qlka", "fp32", lambda q, k, v: attention(q, k, v, "add_riesz", TAU["add_riesz"]), True, 262144),
            ("add_laplace", "qlka-ops", "fp32", laplace_via_operator(weighted_laplace_sum), True, 262144),
            ("add_riesz", "qlka-ops", "fp32", riesz_via_operator(weighted_abs_sum_full), True, 262144)]
    if ref_ext_dir:
        lap = _load_ext(os.path.join(ref_ext_dir, "ref_laplace_ext", "ref_laplace_ext.so"), "ref_laplace_ext")
        ab = _load_ext(os.path.join(ref_ext_dir, "ref_abs_ext", "ref_abs_ext.so"), "ref_abs_ext")
        rows += [("add_laplace", "ref-ext", "fp32", laplace_via_operator(lap.weighted_laplace_sum_forward), False, 131072),
                 ("add_riesz", "ref-ext", "fp32", riesz_via_operator(lambda q, k, v: ab.weighted_abs_sum_full_forward(q, k, v, -1)), False, 131072)]

    def sdpa(backend):
        def fn(q, k, v):
            with sdpa_kernel(SDPA[backend]):
                return F.scaled_dot_product_attention(q, k, v)
        return fn
    rows += [("softmax", "MEM_EFF", "fp32", sdpa("MEM_EFF"), True, 1 << 30), ("softmax", "FLASH", "fp16", sdpa("FLASH"), True, 1 << 30)]
    return rows


def _event_ms(call):
    """Device time of one call, bracketed by a synchronise on both sides."""
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0.record()
    call()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1)


def measure(fn, dtype, shape, D, C, backward, warmups, runs):
    """(mean ms, std ms, peak MB) of fn on fresh random inputs; peak counts the inputs and the output gradient (twice
    when gradients are kept) plus whatever the first call allocates on top, as the reference's harness does."""
    make = lambda width, grad: torch.randn(*shape, width, dtype=dtype, device="cuda", requires_grad=grad)
    q, k, v, g_out = make(D, backward), make(D, backward), make(C, backward), make(C, False)
    held = sum(t.numel() * t.element_size() for t in (q, k, v, g_out)) * (2 if backward else 1)

    def call():
        for t in (q, k, v):
            t.grad = None
        with torch.set_grad_enabled(backward):
            result = fn(q, k, v)
            if backward:
                result.backward(g_out)

    try:
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        before = torch.cuda.memory_allocated()
        call()
        torch.cuda.synchronize()
        peak_mb = (torch.cuda.max_memory_allocated() - before + held) / 2 ** 20
        for _ in range(warmups):
            call()
        ms = torch.tensor([_event_ms(call) for _ in range(runs)])
        return ms.mean().item(), (ms.std().item() if runs > 1 else 0.0), peak_mb
    except (torch.OutOfMemoryError, RuntimeError) as e:       # out of memory, a size limit, or an SDPA backend that refuses the input
        print(f"    NaN: {type(e).__name__}: {str(e).splitlines()[0][:100]}")
        return math.nan, math.nan, math.nan


def main(argv=None):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--sizes", type=int, nargs="+", default=[2 ** i for i in range(7, 18)])
    ap.add_argument("--runs", type=int, default=10)
    ap.add_argument("--warmups", type=int, default=5)
    ap.add_argument("--B", type=int, default=4)
    ap.add_argument("--H", type=int, default=12)
    ap.add_argument("--D", type=int, default=64)
    ap.add_argument("--C", type=int, default=64)
    ap.add_argument("--out", default="speed_and_memory.csv")
    ap.add_argument("--ref-ext-dir", default="", help="folder with a build of the reference's two CUDA extensions to time beside this library")
    a = ap.parse_args(argv)

    methods = build_methods(a.ref_ext_dir)
    gpu = torch.cuda.get_device_name()
    versions = dict(torch=torch.__version__, cuda=torch.version.cuda, cudnn=torch.backends.cudnn.version())
    done = set()
    if os.path.exists(a.out):
        done = {tuple(r[c] for c in KEY) for r in csv.DictReader(open(a.out))}
    written = 0
    for N in a.sizes:
        for mode in ("fwd", "fwd+bwd"):
            for method, backend, dtype, fn, has_bwd, n_max in methods:
                if mode == "fwd+bwd" and not has_bwd:
                    continue
                row = dict(method=method, backend=backend, dtype=dtype, B=a.B, H=a.H, D=a.D, C=a.C, N=N, mode=mode, gpu=gpu)
                if tuple(str(row[c]) for c in KEY) in done:
                    continue
                if N > n_max:
                    mean = std = peak = math.nan
                else:
                    mean, std, peak = measure(fn, DTYPES[dtype], (a.B, a.H, N), a.D, a.C, mode == "fwd+bwd", a.warmups, a.runs)
                torch.cuda.empty_cache()
                row.update(time_mean_ms=round(mean, 4), time_std_ms=round(std, 4), peak_mem_mb=round(peak, 1), runs=a.runs,
                           warmups=a.warmups, hostname=socket.gethostname(), **versions,
                           date=datetime.datetime.now().isoformat(timespec="seconds"))
                new = not os.path.exists(a.out)
                with open(a.out, "a", newline="") as f:
                    w = csv.DictWriter(f, fieldnames=FIELDS)
                    if new:
                        w.writeheader()
                    w.writerow(row)
                written += 1
                print(f"{mode:<8} N={N:<6} {method:<11} {backend:<9} {dtype}  {mean:10.3f} +- {std:7.3f} ms  {peak:9.1f} MB", flush=True)
    return written


if __name__ == "__main__":
    main()

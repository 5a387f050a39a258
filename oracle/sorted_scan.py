"""TEST INFRASTRUCTURE ONLY - ctypes front end of oracle/sorted_scan.c (the CPU
O(N log N) restatement, double accumulation). Builds the shared object on first use.
Only tests, the smoke test and the CPU-baseline leg of the benchmark import this."""

import ctypes
import os
import subprocess

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libqlka_oracle.so")
_lib = None


def build(force=False):
    src = os.path.join(_HERE, "sorted_scan.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        os.makedirs(os.path.dirname(_SO), exist_ok=True)
        cc = "/usr/bin/gcc" if os.path.exists("/usr/bin/gcc") else "gcc"
        subprocess.check_call([cc, "-O2", "-fPIC", "-shared", "-fopenmp", "-o", _SO, src, "-lm"])
    return _SO


def _load():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _f32(x):
    return np.ascontiguousarray(x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else x, dtype=np.float32)


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _dims(q, k, v):
    P, D, M = q.shape
    return P, D, k.shape[2], M, v.shape[2]


def laplace_sum(q, k, v):
    q, k, v = _f32(q), _f32(k), _f32(v)
    P, D, N, M, C = _dims(q, k, v)
    ow = np.empty((P, M, C), np.float64)
    ou = np.empty((P, M), np.float64)
    rc = _load().oracle_laplace_forward(_ptr(q), _ptr(k), _ptr(v), _ptr(ow), _ptr(ou), P, D, N, M, C)
    assert rc == 0
    return torch.from_numpy(ow), torch.from_numpy(ou)


def abs_sum(q, k, v):
    q, k, v = _f32(q), _f32(k), _f32(v)
    P, D, N, M, C = _dims(q, k, v)
    ow = np.empty((P, M, C), np.float64)
    ou = np.empty((P, M), np.float64)
    rc = _load().oracle_abs_forward(_ptr(q), _ptr(k), _ptr(v), _ptr(ow), _ptr(ou), P, D, N, M, C)
    assert rc == 0
    return torch.from_numpy(ow), torch.from_numpy(ou)


def abs_sum_backward(q, k, v, g_w, g_u=None):
    q, k, v, g_w = _f32(q), _f32(k), _f32(v), _f32(g_w)
    P, D, N, M, C = _dims(q, k, v)
    gu = None if g_u is None else _f32(g_u)
    gq = np.empty((P, D, M), np.float64)
    gk = np.empty((P, D, N), np.float64)
    gv = np.empty((P, N, C), np.float64)
    rc = _load().oracle_abs_backward(_ptr(q), _ptr(k), _ptr(v), _ptr(g_w), None if gu is None else _ptr(gu),
                                     _ptr(gq), _ptr(gk), _ptr(gv), P, D, N, M, C)
    assert rc == 0
    return torch.from_numpy(gq), torch.from_numpy(gk), torch.from_numpy(gv)


def sgn_sum(q, k, v, g):
    q, k, v, g = _f32(q), _f32(k), _f32(v), _f32(g)
    P, D, N, M, C = _dims(q, k, v)
    out = np.empty((P, D, M), np.float64)
    rc = _load().oracle_sgn_forward(_ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(out), P, D, N, M, C)
    assert rc == 0
    return torch.from_numpy(out)

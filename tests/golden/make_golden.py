"""Generates the golden vectors in this folder from the reference's own Python code.

Run in a container that has the reference checkout (its path is the argument, or QLKA_REFERENCE_DIR):

    python tests/golden/make_golden.py /path/to/reference

The reference's `Experiments/kernel_attention/{kernels,attention}.py` are imported
unchanged; its two CUDA extension packages (which `attention.py` imports at module
level and which cannot run without a GPU) are replaced by empty stand-ins, so only the
naive full-matrix path (`impl="naive"`) and the chunked path (`_chunked(_normalized)`)
are exercised. Outputs:

  small_kernels.npz   kernel matrices and normalised attention of add_laplace /
                      add_riesz / add_bump on B=1,H=2,S=48,D=8 inputs, with and without
                      a key-keep mask, tau = 0.7
  c1_add_laplace.npz  add_laplace attention at B=1,H=4,N=1024,D=Dv=32, tau=1, seed 0:
                      the naive result and the chunked result
"""

import importlib
import os
import sys
import types

import numpy as np
import torch

ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("QLKA_REFERENCE_DIR")
if not ref:
    sys.exit("usage: python tests/golden/make_golden.py /path/to/reference   (or set QLKA_REFERENCE_DIR)")
for name in ("weighted_abs_sum", "weighted_laplace_sum"):
    stub = types.ModuleType(name)
    stub.weighted_abs_sum_full = None
    stub.weighted_laplace_sum = None
    sys.modules[name] = stub
sys.path.insert(0, os.path.join(ref, "Experiments"))
att = importlib.import_module("kernel_attention.attention")
ker = importlib.import_module("kernel_attention.kernels")
here = os.path.dirname(os.path.abspath(__file__))

# ---- small case: kernel matrices + attention, with and without mask
torch.manual_seed(1234)
B, H, S, D = 1, 2, 48, 8
q, k, v = torch.randn(B, H, S, D), torch.randn(B, H, S, D), torch.randn(B, H, S, D)
q[0, 0, :6, 0] = k[0, 0, :6, 0]              # exact ties in one feature dimension
keep = torch.rand(B, S) > 0.25
tau = 0.7
out = {"q": q.numpy(), "k": k.numpy(), "v": v.numpy(), "keep": keep.numpy(), "tau": np.float32(tau)}
P = B * H
qp, kp = q.transpose(2, 3).reshape(P, D, S), k.transpose(2, 3).reshape(P, D, S)
for name in ("add_laplace", "add_riesz", "add_bump"):
    out[f"A_{name}"] = ker.KERNELS[name](qp, kp, tau, None).numpy()
    out[f"A_{name}_masked"] = ker.KERNELS[name](qp, kp, tau, keep.repeat_interleave(H, dim=0)).numpy()
    out[f"att_{name}"] = att.attention(q, k, v, name, tau, None, impl="naive").numpy()
    out[f"att_{name}_masked"] = att.attention(q, k, v, name, tau, keep, impl="naive").numpy()
np.savez_compressed(os.path.join(here, "small_kernels.npz"), **out)

# ---- config 1: the reference's CPU-runnable add_laplace case
torch.manual_seed(0)
B, H, S, D = 1, 4, 1024, 32
tau = 1.0
q, k, v = torch.randn(B, H, S, D) / tau, torch.randn(B, H, S, D) / tau, torch.randn(B, H, S, D)
naive = att.attention(q, k, v, "add_laplace", tau, None, impl="naive")
P = B * H
chunked = att._chunked(att._normalized, "add_laplace", q.transpose(2, 3).reshape(P, D, S),
                       k.transpose(2, 3).reshape(P, D, S), v.reshape(P, S, D), tau, None, D).view(B, H, S, D)
np.savez_compressed(os.path.join(here, "c1_add_laplace.npz"),
                    q=q.numpy(), k=k.numpy(), v=v.numpy(), tau=np.float32(tau),
                    naive=naive.numpy(), chunked=chunked.numpy())
print("wrote", os.listdir(here))

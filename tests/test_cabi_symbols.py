"""CPU-only checks of the C ABI: the library loads, exports every function that
include/qlka.h declares, and its argument checks answer without touching a GPU."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import importlib.util
    spec = importlib.util.spec_from_file_location("qlka_build", os.path.join(ROOT, "quasi-linear-kernel-attention_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()
    import qlka_native
    return qlka_native.lib()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "qlka.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qlka_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_operator_set():
    names = declared_functions()
    for want in ("qlka_weighted_laplace_sum_forward", "qlka_weighted_abs_sum_forward", "qlka_weighted_abs_sum_backward",
                 "qlka_weighted_sgn_sum_forward", "qlka_status_string"):
        assert want in names


def test_every_declared_symbol_is_exported(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in include/qlka.h but not exported"


def test_dimension_checks_follow_the_reference(lib):
    n = ctypes.c_size_t(0)
    f = lib.qlka_laplace_forward_workspace_bytes
    assert f(2, 4, 100, 100, 8, ctypes.byref(n)) == 0 and n.value > 0
    assert f(0, 4, 100, 100, 8, ctypes.byref(n)) == 1           # sizes must be > 0
    assert f(2, 4, 100, 100, 129, ctypes.byref(n)) == 2         # C in [1, 128]
    assert f(2, 4, 262145, 100, 8, ctypes.byref(n)) == 3        # N, M <= 262144 (the reference: 131072)
    assert f(4096, 64, 16384, 16384, 8, ctypes.byref(n)) == 4   # P*D*max(N,M) must fit int32
    assert b"262144" in lib.qlka_status_string(3)
    assert b"int32" in lib.qlka_status_string(4)
    # forward calls refuse before any launch: bad path, pinned fused path, null pointers, short workspace
    fwd = lib.qlka_weighted_abs_sum_forward
    assert fwd(None, None, None, None, None, None, 0, 1, 1, 8, 8, 4, 7, None) == 5
    assert fwd(None, None, None, None, None, None, 0, 1, 1, 5000, 8, 4, 1, None) == 6
    assert fwd(None, None, None, None, None, None, 0, 1, 1, 8, 8, 4, -1, None) == 7
    assert lib.qlka_weighted_laplace_sum_forward(16, 16, 16, 16, 16, None, 0, 1, 1, 8, 8, 4, None) == 8


def test_workspace_grows_with_the_problem(lib):
    a, b = ctypes.c_size_t(0), ctypes.c_size_t(0)
    for name in ("laplace_forward", "abs_forward", "abs_backward", "sgn_forward"):
        f = getattr(lib, f"qlka_{name}_workspace_bytes")
        assert f(2, 4, 512, 512, 64, ctypes.byref(a)) == 0
        assert f(4, 4, 2048, 2048, 64, ctypes.byref(b)) == 0
        assert 0 < a.value < b.value
        assert a.value % 256 == 0


def test_ops_fail_loudly_without_cuda_tensors(lib):
    import torch
    from weighted_abs_sum import weighted_abs_sum
    from weighted_laplace_sum import weighted_laplace_sum
    q, k, v = torch.zeros(1, 2, 8), torch.zeros(1, 2, 8), torch.zeros(1, 8, 4)
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        weighted_laplace_sum(q, k, v)
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        weighted_abs_sum(q, k, v)
    with pytest.raises(ValueError):
        weighted_abs_sum(q, k, v, backend="nope")


def test_newer_entry_points_check_their_arguments(lib):
    n, m = ctypes.c_size_t(0), ctypes.c_size_t(0)
    # Laplace backward: same dimension rules, a workspace at least as large as the forward's records
    assert lib.qlka_laplace_backward_workspace_bytes(2, 4, 512, 300, 64, ctypes.byref(n)) == 0
    assert lib.qlka_laplace_forward_workspace_bytes(2, 4, 512, 300, 64, ctypes.byref(m)) == 0
    assert n.value >= m.value > 0
    assert lib.qlka_laplace_backward_workspace_bytes(2, 4, 512, 300, 0, ctypes.byref(n)) == 2
    assert lib.qlka_weighted_laplace_sum_backward(None, None, None, None, None, None, None, None, None, 0, 1, 1, 8, 8, 4, None) == 7
    # attention entry points: kind, head count, sequence limit of the fused bump, tau
    assert lib.qlka_laplace_attention_workspace_bytes(2, 3, 100, 16, 16, 0, ctypes.byref(n)) == 0 and n.value > 0
    assert lib.qlka_laplace_attention_workspace_bytes(2, 3, 100, 16, 16, 1, ctypes.byref(m)) == 0 and m.value > n.value
    assert lib.qlka_laplace_attention_workspace_bytes(0, 3, 100, 16, 16, 0, ctypes.byref(n)) == 1
    assert lib.qlka_abs_attention_workspace_bytes(2, 1, 1, 100, 16, 16, 0, ctypes.byref(n)) == 5          # kind is 0 or 1
    assert lib.qlka_abs_attention_workspace_bytes(1, 1, 1, 6000, 16, 16, 0, ctypes.byref(n)) == 10        # fused bump: 3 S <= 16384
    assert lib.qlka_abs_attention_workspace_bytes(0, 1, 1, 6000, 16, 16, 0, ctypes.byref(n)) == 0
    f = lib.qlka_abs_attention_forward
    assert f(0, None, None, None, None, ctypes.c_float(1.0), None, None, 0, 1, 1, 8, 4, 4, None) == 7     # null tensors
    assert f(0, 16, 16, 16, None, ctypes.c_float(0.0), 16, None, 0, 1, 1, 8, 4, 4, None) == 1             # tau must be > 0
    # shifted abs sum and the fixed-scratch Laplace entry refuse what they cannot hold
    assert lib.qlka_abs_shifted_forward_workspace_bytes(1, 1, 100, 6000, 8, 3, ctypes.byref(n)) == 10
    assert lib.qlka_abs_shifted_forward_workspace_bytes(1, 1, 100, 100, 8, 5, ctypes.byref(n)) == 1
    assert lib.qlka_noalloc_scratch_bytes() == 32 << 20


def test_row_matrices_must_be_16_byte_aligned(lib):
    """v, g_w, g, out_w, grad_v and the attention output are moved with 16-byte accesses; a pointer off that
    boundary is refused with its own status before anything is launched (the checks need no GPU)."""
    ok, off = 4096, 4096 + 4
    assert lib.qlka_weighted_laplace_sum_forward(ok, ok, off, ok, ok, None, 0, 1, 1, 8, 8, 4, None) == 12      # v
    assert lib.qlka_weighted_laplace_sum_forward(ok, ok, ok, off, ok, None, 0, 1, 1, 8, 8, 4, None) == 12      # out_w
    assert lib.qlka_weighted_laplace_sum_forward(off, off, ok, ok, off, None, 0, 1, 1, 8, 8, 4, None) == 8     # q, k, out_u: float alignment is enough
    assert lib.qlka_weighted_laplace_sum_forward_noalloc(ok, ok, off, ok, ok, 1, 1, 8, 8, 4, None) == 12
    assert lib.qlka_weighted_abs_sum_forward(ok, ok, ok, off, None, None, 0, 1, 1, 8, 8, 4, -1, None) == 12
    bwd = lib.qlka_weighted_abs_sum_backward
    assert bwd(ok, ok, ok, off, None, ok, ok, ok, None, 0, 1, 1, 8, 8, 4, None) == 12                          # g_w
    assert bwd(ok, ok, ok, ok, None, ok, ok, off, None, 0, 1, 1, 8, 8, 4, None) == 12                          # grad_v
    assert bwd(ok, ok, ok, ok, None, off, off, ok, None, 0, 1, 1, 8, 8, 4, None) == 8                          # grad_q, grad_k
    assert lib.qlka_weighted_laplace_sum_backward(ok, ok, off, ok, None, ok, ok, ok, None, 0, 1, 1, 8, 8, 4, None) == 12
    assert lib.qlka_weighted_sgn_sum_forward(ok, ok, ok, off, ok, None, 0, 1, 1, 8, 8, 4, None) == 12          # g
    assert lib.qlka_laplace_attention_forward(ok, ok, ok, None, ctypes.c_float(1.0), off, None, 0, 1, 1, 8, 4, 4, None) == 12
    assert lib.qlka_abs_attention_forward(0, ok, ok, off, None, ctypes.c_float(1.0), ok, None, 0, 1, 1, 8, 4, 4, None) == 12
    assert b"16-byte" in lib.qlka_status_string(12)

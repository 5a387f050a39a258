"""weighted_laplace_sum on the GPU (through the C ABI) against the CPU checkers."""

import os

import numpy as np
import pytest
import torch

from oracle import direct, sorted_scan
from util import make_inputs, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-4          # max|a-b| / max|b| against float64; the north-star bound is 1e-3
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

SHAPES = [
    (1, 1, 1, 1, 1), (2, 3, 7, 5, 4), (1, 2, 8, 9, 3), (2, 4, 100, 77, 32), (1, 3, 257, 300, 33),
    (1, 2, 64, 1000, 64), (1, 2, 1000, 3, 65), (2, 2, 600, 600, 64), (1, 2, 1024, 1024, 128),
    (1, 3, 2049, 1500, 16), (1, 2, 4096, 4096, 64), (3, 2, 5000, 7000, 8), (1, 2, 16384, 16384, 64),
]


@pytest.mark.parametrize("shape", SHAPES)
def test_forward_matches_oracle(shape):
    from weighted_laplace_sum import weighted_laplace_sum
    P, D, N, M, C = shape
    q, k, v = make_inputs(P, D, N, M, C, seed=N + M + C, scale=2.0)
    out_w, out_u = weighted_laplace_sum(q, k, v)
    torch.cuda.synchronize()
    ref_w, ref_u = sorted_scan.laplace_sum(q, k, v)
    assert out_w.shape == (P, M, C) and out_u.shape == (P, M)
    assert rel_err(out_w, ref_w) < TOL, f"out_w rel err {rel_err(out_w, ref_w)}"
    assert rel_err(out_u, ref_u) < TOL, f"out_u rel err {rel_err(out_u, ref_u)}"
    if N * M * D * P <= 1 << 24:
        dw, du = direct.laplace_sum(q, k, v)
        assert rel_err(out_w, dw) < TOL and rel_err(out_u, du) < TOL


def test_two_calls_agree_and_inputs_untouched():
    from weighted_laplace_sum import weighted_laplace_sum
    q, k, v = make_inputs(2, 4, 3000, 2500, 64, seed=5)
    q0, k0, v0 = q.clone(), k.clone(), v.clone()
    a = weighted_laplace_sum(q, k, v)
    b = weighted_laplace_sum(q, k, v)
    torch.cuda.synchronize()
    assert torch.equal(q, q0) and torch.equal(k, k0) and torch.equal(v, v0)
    assert rel_err(a[0], b[0].double()) < 1e-5 and rel_err(a[1], b[1].double()) < 1e-5     # atomics: order differs


def test_far_apart_keys_do_not_overflow():
    """Keys hundreds of units below every query: all exponent arguments stay <= 0."""
    from weighted_laplace_sum import weighted_laplace_sum
    q, k, v = make_inputs(1, 2, 300, 200, 8, seed=9, ties=False)
    k[0, 0, :50] -= 500.0
    q[0, 1, :20] += 300.0
    out_w, out_u = weighted_laplace_sum(q, k, v)
    ref_w, ref_u = sorted_scan.laplace_sum(q, k, v)
    assert torch.isfinite(out_w).all() and torch.isfinite(out_u).all()
    assert rel_err(out_w, ref_w) < TOL and rel_err(out_u, ref_u) < TOL


def test_config1_against_reference_golden():
    """B=1,H=4,N=1024,D=Dv=32 add_laplace attention against the reference's own output."""
    from kernel_attention import attention
    z = np.load(os.path.join(GOLD, "c1_add_laplace.npz"))
    q, k, v = (torch.from_numpy(z[n]).cuda() for n in ("q", "k", "v"))
    out = attention(q, k, v, "add_laplace", float(z["tau"]))
    assert rel_err(out, torch.from_numpy(z["naive"])) < TOL
    assert rel_err(out, torch.from_numpy(z["chunked"])) < TOL


def test_linearity_and_sampled_head_at_full_size():
    """B=4,H=12,N=16384,D=Dv=64 is too big for the checker as a whole: one head goes through the
    C restatement, and the full batch is checked through linearity in v."""
    from weighted_laplace_sum import weighted_laplace_sum
    P, D, N, C = 48, 64, 16384, 64
    g = torch.Generator().manual_seed(0)
    q = (torch.randn(P, D, N, generator=g) * 2).cuda()
    k = (torch.randn(P, D, N, generator=g) * 2).cuda()
    v1 = torch.randn(P, N, C, generator=g).cuda()
    v2 = torch.randn(P, N, C, generator=g).cuda()
    w1, u1 = weighted_laplace_sum(q, k, v1)
    w2, u2 = weighted_laplace_sum(q, k, v2)
    w3, u3 = weighted_laplace_sum(q, k, 2.0 * v1 - 0.5 * v2)
    assert rel_err(w3, (2.0 * w1.double() - 0.5 * w2.double())) < TOL
    assert rel_err(u3, u1.double()) < 1e-5
    p = 17
    ref_w, ref_u = sorted_scan.laplace_sum(q[p:p + 1], k[p:p + 1], v1[p:p + 1])
    assert rel_err(w1[p:p + 1], ref_w) < TOL and rel_err(u1[p:p + 1], ref_u) < TOL


def test_argument_errors():
    from weighted_laplace_sum import weighted_laplace_sum
    q, k, v = make_inputs(1, 2, 16, 16, 4, seed=1)
    with pytest.raises(RuntimeError, match="CUDA tensors"):
        weighted_laplace_sum(q.cpu(), k, v)
    with pytest.raises(RuntimeError, match="float32"):
        weighted_laplace_sum(q.double(), k.double(), v.double())
    with pytest.raises(RuntimeError, match="contiguous"):
        weighted_laplace_sum(q.transpose(1, 2).contiguous().transpose(1, 2), k, v)
    with pytest.raises(RuntimeError, match="same length"):
        weighted_laplace_sum(q, k, v[:, :8])
    with pytest.raises(RuntimeError, match=r"\[1, 128\]"):
        weighted_laplace_sum(q, k, torch.zeros(1, 16, 129, device="cuda"))


def test_host_pipeline_matches_device_call():
    """Pinned host buffers in and out, heads streamed in chunks (ragged last chunk)."""
    import qlka_native
    P, D, N, M, C = 7, 4, 1200, 900, 32
    q, k, v = make_inputs(P, D, N, M, C, seed=77, scale=2.0, device="cpu")
    q_h, k_h, v_h = q.pin_memory(), k.pin_memory(), v.pin_memory()
    out_w_h, out_u_h = torch.empty(P, M, C).pin_memory(), torch.empty(P, M).pin_memory()
    pipe = qlka_native.HostPipeline(P, D, N, M, C, chunk=3)
    for _ in range(2):
        pipe(q_h, k_h, v_h, out_w_h, out_u_h)
        torch.cuda.synchronize()
        ref_w, ref_u = qlka_native.laplace_forward(q.cuda(), k.cuda(), v.cuda())
        assert rel_err(out_w_h, ref_w.double()) < 1e-5 and rel_err(out_u_h, ref_u.double()) < 1e-5


@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("shape", [(1, 2, 50, 8, 8), (2, 3, 333, 16, 20), (1, 4, 1024, 32, 32), (2, 2, 700, 64, 33)])
def test_fused_attention_entry(shape, masked):
    """The one-call add_laplace attention on (B, H, S, D) against the float64 dense formula and the op-by-op route."""
    import qlka_native
    from kernel_attention import attention
    B, H, S, D, Dv = shape
    g = torch.Generator().manual_seed(S + D)
    q, k = (torch.randn(B, H, S, D, generator=g).cuda() for _ in range(2))
    v = torch.randn(B, H, S, Dv, generator=g).cuda()
    keep = None
    if masked:
        keep = (torch.rand(B, S, generator=g) > 0.3)
        keep[:, 0] = True
        keep = keep.cuda()
    out = qlka_native.laplace_attention(q, k, v, 0.5, keep)
    ref = direct.attention(q, k, v, "add_laplace", 0.5, keep)
    assert out.shape == (B, H, S, Dv)
    assert rel_err(out, ref) < TOL, f"rel err {rel_err(out, ref)}"
    assert rel_err(out, attention(q, k, v, "add_laplace", 0.5, keep).double()) < 1e-5     # same route without grad (atomics: order differs)
    with torch.enable_grad():
        qg = q.clone().requires_grad_(True)
        slow = attention(qg, k, v, "add_laplace", 0.5, keep)                      # op-by-op route
    assert rel_err(out, slow.double()) < 1e-5


def test_contiguous_view_at_an_odd_storage_offset():
    """A contiguous v whose storage offset puts it 4 bytes off a 16-byte boundary: the C ABI refuses such a row
    matrix with its own status (the kernels use 16-byte accesses), the Python operator copies it once instead."""
    import qlka_native
    from weighted_laplace_sum import weighted_laplace_sum
    q, k, v = make_inputs(2, 3, 500, 400, 64, seed=77)
    store = torch.empty(v.numel() + 1, device="cuda")
    v_off = store[1:].view_as(v)
    v_off.copy_(v)
    assert v_off.is_contiguous() and v_off.data_ptr() % 16 == 4
    lib = qlka_native.lib()
    out_w, out_u = torch.empty(2, 400, 64, device="cuda"), torch.empty(2, 400, device="cuda")
    st = lib.qlka_weighted_laplace_sum_forward_noalloc(q.data_ptr(), k.data_ptr(), v_off.data_ptr(), out_w.data_ptr(),
                                                       out_u.data_ptr(), 2, 3, 500, 400, 64, torch.cuda.current_stream().cuda_stream)
    assert st == 12
    a_w, a_u = weighted_laplace_sum(q, k, v_off)
    b_w, b_u = weighted_laplace_sum(q, k, v)
    assert rel_err(a_w, b_w.double()) < 1e-5 and rel_err(a_u, b_u.double()) < 1e-5

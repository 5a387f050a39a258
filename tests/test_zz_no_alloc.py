"""The entry point that brings its own scratch (for callers that may not allocate:
serving loops, hosts that own all device memory). Collected last on purpose.

Called through the C ABI, twice in a row with different problems, and compared with the
workspace entry point on the same inputs. The second call runs on scratch that still holds the
first call's records, which must not matter."""

import ctypes

import pytest
import torch

from util import make_inputs, rel_err

pytestmark = pytest.mark.gpu
TOL = 1e-4      # same bound as the other parity tests; the two entry points differ only by atomic order


def _call_noalloc(lib, q, k, v):
    P, D, M = q.shape
    N, C = k.shape[2], v.shape[2]
    out_w = torch.full((P, M, C), float("nan"), device="cuda")      # the call must overwrite every element
    out_u = torch.full((P, M), float("nan"), device="cuda")
    st = lib.qlka_weighted_laplace_sum_forward_noalloc(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), out_w.data_ptr(), out_u.data_ptr(),
        P, D, N, M, C, torch.cuda.current_stream().cuda_stream)
    assert st == 0, lib.qlka_status_string(st)
    return out_w, out_u


def test_matches_workspace_entry_point_on_two_calls_in_a_row():
    import qlka_native
    lib = qlka_native.lib()
    assert lib.qlka_noalloc_scratch_bytes() == 32 << 20
    first = make_inputs(2, 8, 1500, 1200, 64, seed=31, scale=2.0)
    second = make_inputs(3, 4, 700, 2100, 33, seed=32, scale=2.0)     # other sizes, padded channels
    for q, k, v in (first, second):
        got_w, got_u = _call_noalloc(lib, q, k, v)
        ref_w, ref_u = qlka_native.laplace_forward(q, k, v)
        torch.cuda.synchronize()
        assert torch.isfinite(got_w).all() and torch.isfinite(got_u).all()
        assert rel_err(got_w, ref_w.double()) < TOL
        assert rel_err(got_u, ref_u.double()) < TOL


def test_later_calls_leave_free_device_memory_unchanged():
    """The one claim of the entry point: once the scratch array exists (the first call on a device
    materialises it), a call takes no device memory - neither through the CUDA allocator nor
    through torch's. Outputs are preallocated so that the wrapper allocates nothing either."""
    import qlka_native
    lib = qlka_native.lib()
    q, k, v = make_inputs(2, 8, 1500, 1200, 64, seed=33, scale=2.0)
    P, D, M = q.shape
    N, C = k.shape[2], v.shape[2]
    out_w = torch.empty(P, M, C, device="cuda")
    out_u = torch.empty(P, M, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        st = lib.qlka_weighted_laplace_sum_forward_noalloc(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), out_w.data_ptr(), out_u.data_ptr(), P, D, N, M, C, stream)
        assert st == 0, lib.qlka_status_string(st)
        torch.cuda.synchronize()

    call()                                             # set-up call: may materialise the array and load kernels
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    for _ in range(3):
        call()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
    assert torch.cuda.memory_reserved() == reserved_before


def test_refuses_problems_beyond_the_fixed_scratch():
    import qlka_native
    lib = qlka_native.lib()
    dummy = torch.zeros(64, device="cuda")
    # B=4, H=12, N=16384, D=64 needs far more than 32 MiB of scratch: refused before any launch
    st = lib.qlka_weighted_laplace_sum_forward_noalloc(
        dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
        48, 64, 16384, 16384, 64, torch.cuda.current_stream().cuda_stream)
    assert st == 11
    assert b"32 MiB" in lib.qlka_status_string(st)
    with pytest.raises(RuntimeError, match="32 MiB"):
        q, k, v = make_inputs(48, 64, 2048, 2048, 8, seed=1)
        qlka_native.laplace_forward_noalloc(q, k, v)

"""ctypes binding of libqlka.so (the C ABI of include/qlka.h) for torch tensors.

torch is used for device memory and the current stream only; the kernels are the
library's. There is no fallback: a missing library or a non-CUDA tensor raises.
The tensor checks and their messages follow the reference's host code
(Weighted_Laplace_Sum/csrc/binding.cpp:66-79, Weighted_Abs_Sum/csrc/binding.cpp:69-84,
:251-262, :387-392).
"""

import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libqlka.so")
_lib = None

_vp, _sz, _i = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python {os.path.join(_HERE, 'build.py')}` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback for these operators.")
        L = ctypes.CDLL(LIB_PATH)
        L.qlka_status_string.restype = ctypes.c_char_p
        L.qlka_status_string.argtypes = [_i]
        L.qlka_last_cuda_error.restype = _i
        for name in ("laplace_forward", "laplace_backward", "abs_forward", "abs_backward", "sgn_forward"):
            f = getattr(L, f"qlka_{name}_workspace_bytes")
            f.restype, f.argtypes = _i, [_i] * 5 + [ctypes.POINTER(_sz)]
        L.qlka_sort_rank_workspace_bytes.restype = _i
        L.qlka_sort_rank_workspace_bytes.argtypes = [_i] * 4 + [ctypes.POINTER(_sz)]
        L.qlka_weighted_laplace_sum_forward.restype = _i
        L.qlka_weighted_laplace_sum_forward.argtypes = [_vp] * 5 + [_vp, _sz] + [_i] * 5 + [_vp]
        L.qlka_weighted_laplace_sum_backward.restype = _i
        L.qlka_weighted_laplace_sum_backward.argtypes = [_vp] * 8 + [_vp, _sz] + [_i] * 5 + [_vp]
        L.qlka_laplace_attention_workspace_bytes.restype = _i
        L.qlka_laplace_attention_workspace_bytes.argtypes = [_i] * 6 + [ctypes.POINTER(_sz)]
        L.qlka_laplace_attention_forward.restype = _i
        L.qlka_laplace_attention_forward.argtypes = [_vp] * 4 + [ctypes.c_float] + [_vp] + [_vp, _sz] + [_i] * 5 + [_vp]
        L.qlka_abs_attention_workspace_bytes.restype = _i
        L.qlka_abs_attention_workspace_bytes.argtypes = [_i] * 7 + [ctypes.POINTER(_sz)]
        L.qlka_abs_attention_forward.restype = _i
        L.qlka_abs_attention_forward.argtypes = [_i] + [_vp] * 4 + [ctypes.c_float] + [_vp] + [_vp, _sz] + [_i] * 5 + [_vp]
        L.qlka_laplace_forward_stage_ms.restype = _i
        L.qlka_laplace_forward_stage_ms.argtypes = [_vp] * 5 + [_vp, _sz] + [_i] * 5 + [_vp] + [ctypes.POINTER(ctypes.c_float)] * 3
        L.qlka_noalloc_scratch_bytes.restype = _sz
        L.qlka_weighted_laplace_sum_forward_noalloc.restype = _i
        L.qlka_weighted_laplace_sum_forward_noalloc.argtypes = [_vp] * 5 + [_i] * 5 + [_vp]
        L.qlka_weighted_abs_sum_forward.restype = _i
        L.qlka_weighted_abs_sum_forward.argtypes = [_vp] * 5 + [_vp, _sz] + [_i] * 6 + [_vp]
        L.qlka_abs_shifted_forward_workspace_bytes.restype = _i
        L.qlka_abs_shifted_forward_workspace_bytes.argtypes = [_i] * 6 + [ctypes.POINTER(_sz)]
        L.qlka_weighted_abs_sum_shifted_forward.restype = _i
        L.qlka_weighted_abs_sum_shifted_forward.argtypes = [_vp] * 5 + [ctypes.POINTER(ctypes.c_float)] * 2 + [_i] + [_vp, _sz] + [_i] * 5 + [_vp]
        L.qlka_weighted_abs_sum_backward.restype = _i
        L.qlka_weighted_abs_sum_backward.argtypes = [_vp] * 8 + [_vp, _sz] + [_i] * 5 + [_vp]
        L.qlka_weighted_sgn_sum_forward.restype = _i
        L.qlka_weighted_sgn_sum_forward.argtypes = [_vp] * 5 + [_vp, _sz] + [_i] * 5 + [_vp]
        L.qlka_sort_rank_records.restype = _i
        L.qlka_sort_rank_records.argtypes = [_vp] * 6 + [_vp, _sz] + [_i] * 5 + [_vp]
        _lib = L
    return _lib


def _raise(status):
    L = lib()
    msg = L.qlka_status_string(status).decode()
    if status == 9:
        msg += f" (cudaError {L.qlka_last_cuda_error()})"
    raise RuntimeError(msg)


def _check(cond, msg):
    if not cond:
        raise RuntimeError(msg)


def check_qkv(q, k, v, names="q, k and v"):
    _check(q.is_cuda and k.is_cuda and v.is_cuda, f"{names} must be CUDA tensors")
    _check(q.device == k.device == v.device, f"{names} must be on one device")
    _check(q.dtype == k.dtype == v.dtype == torch.float32, f"{names} must be float32")
    _check(q.dim() == 3 and k.dim() == 3 and v.dim() == 3, f"{names} must be 3D")
    _check(q.size(0) == k.size(0) == v.size(0), "batch size must match")
    _check(q.size(1) == k.size(1), "q and k must have the same feature dimension")
    _check(k.size(2) == v.size(1), "k and v must have the same length")
    _check(q.is_contiguous() and k.is_contiguous() and v.is_contiguous(), f"{names} must be contiguous")
    return q.size(0), q.size(1), k.size(2), q.size(2), v.size(2)      # P, D, N, M, C


def _aligned(t):
    """The row matrices must start on a 16-byte boundary (include/qlka.h); a contiguous view at an odd
    storage offset is copied once instead of being refused, as the reference accepts any contiguous tensor."""
    return t if t.data_ptr() % 16 == 0 else t.clone(memory_format=torch.contiguous_format)


def _check_like(t, name, shape, ref):
    _check(t.is_cuda and t.device == ref.device, f"{name} must be on q's CUDA device")
    _check(t.dtype == torch.float32, f"{name} must be float32")
    _check(tuple(t.shape) == tuple(shape), f"{name} must have shape {tuple(shape)}")
    _check(t.is_contiguous(), f"{name} must be contiguous")


def _workspace(fn, dims, device):
    n = _sz(0)
    st = fn(*dims, ctypes.byref(n))
    if st:
        _raise(st)
    return torch.empty(max(int(n.value), 256), dtype=torch.uint8, device=device), int(n.value)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def laplace_forward(q, k, v):
    P, D, N, M, C = dims = check_qkv(q, k, v)
    v = _aligned(v)
    L = lib()
    with torch.cuda.device(q.device):
        ws, n = _workspace(L.qlka_laplace_forward_workspace_bytes, dims, q.device)
        out_w = torch.empty(P, M, C, dtype=torch.float32, device=q.device)
        out_u = torch.empty(P, M, dtype=torch.float32, device=q.device)
        st = L.qlka_weighted_laplace_sum_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), out_w.data_ptr(), out_u.data_ptr(),
                                                 ws.data_ptr(), n, P, D, N, M, C, _stream())
    if st:
        _raise(st)
    return out_w, out_u


def laplace_forward_noalloc(q, k, v, out_w=None, out_u=None):
    """weighted Laplace sum through the entry point that uses the library's fixed scratch array
    instead of a workspace. The native call allocates nothing; pass preallocated `out_w` (P, M, C)
    and `out_u` (P, M) to keep this wrapper from allocating too. Raises if the problem needs more
    scratch than the array holds. Calls must not overlap on the GPU (they share the array)."""
    P, D, N, M, C = check_qkv(q, k, v)
    v = _aligned(v)
    L = lib()
    with torch.cuda.device(q.device):
        if out_w is None:
            out_w = torch.empty(P, M, C, dtype=torch.float32, device=q.device)
        if out_u is None:
            out_u = torch.empty(P, M, dtype=torch.float32, device=q.device)
        _check_like(out_w, "out_w", (P, M, C), q)
        _check_like(out_u, "out_u", (P, M), q)
        st = L.qlka_weighted_laplace_sum_forward_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), out_w.data_ptr(),
                                                         out_u.data_ptr(), P, D, N, M, C, _stream())
    if st:
        _raise(st)
    return out_w, out_u


class HostPipeline:
    """weighted Laplace sum for inputs and outputs in (pinned) host memory.

    The heads (dim 0 = P) are cut into chunks that flow through three CUDA streams - host-to-device
    copies, the operator, device-to-host copies - with two sets of device buffers, so that the PCIe
    transfers of one chunk overlap the kernels of the previous one and the read-back of the one
    before. Device buffers and the workspace are allocated once, at construction.
    """

    def __init__(self, P, D, N, M, C, chunk, device=None):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.dims = (P, D, N, M, C)
        self.chunk = max(1, min(chunk, P))
        L = lib()
        with torch.cuda.device(self.device):
            n = _sz(0)
            st = L.qlka_laplace_forward_workspace_bytes(self.chunk, D, N, M, C, ctypes.byref(n))
            if st:
                _raise(st)
            self.ws_bytes = int(n.value)
            f32 = dict(dtype=torch.float32, device=self.device)
            self.sets = [dict(q=torch.empty(self.chunk, D, M, **f32), k=torch.empty(self.chunk, D, N, **f32),
                              v=torch.empty(self.chunk, N, C, **f32), ow=torch.empty(self.chunk, M, C, **f32),
                              ou=torch.empty(self.chunk, M, **f32),
                              ws=torch.empty(max(self.ws_bytes, 256), dtype=torch.uint8, device=self.device),
                              loaded=torch.cuda.Event(), computed=torch.cuda.Event(), drained=torch.cuda.Event())
                         for _ in range(2)]
            self.s_in, self.s_run, self.s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()

    def _ranges(self, P):
        """Head ranges of the chunks: full chunks, then halves of what is left, so that the work that nothing overlaps
        (the kernels and the read-back of the last chunk) is that of a single head."""
        lo = 0
        while lo < P:
            left = P - lo
            n = self.chunk if left > self.chunk else max(1, left // 2)
            yield lo, lo + n
            lo += n

    def __call__(self, q_h, k_h, v_h, out_w_h, out_u_h):
        """Enqueue one pass over all heads; returns after everything has been enqueued. The caller
        synchronises (e.g. torch.cuda.synchronize()) before reading out_w_h / out_u_h."""
        P, D, N, M, C = self.dims
        L = lib()
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_run, self.s_out):
            s.wait_stream(cur)
        with torch.cuda.device(self.device):
            for i, (lo, hi) in enumerate(self._ranges(P)):
                b = self.sets[i % 2]
                n = hi - lo
                with torch.cuda.stream(self.s_in):
                    self.s_in.wait_event(b["computed"])          # the previous user of this buffer set has consumed its inputs
                    b["q"][:n].copy_(q_h[lo:hi], non_blocking=True)
                    b["k"][:n].copy_(k_h[lo:hi], non_blocking=True)
                    b["v"][:n].copy_(v_h[lo:hi], non_blocking=True)
                    b["loaded"].record(self.s_in)
                with torch.cuda.stream(self.s_run):
                    self.s_run.wait_event(b["loaded"])
                    self.s_run.wait_event(b["drained"])          # ... and its outputs have left the device
                    st = L.qlka_weighted_laplace_sum_forward(b["q"].data_ptr(), b["k"].data_ptr(), b["v"].data_ptr(),
                                                             b["ow"].data_ptr(), b["ou"].data_ptr(), b["ws"].data_ptr(),
                                                             self.ws_bytes, n, D, N, M, C, self.s_run.cuda_stream)
                    if st:
                        _raise(st)
                    b["computed"].record(self.s_run)
                with torch.cuda.stream(self.s_out):
                    self.s_out.wait_event(b["computed"])
                    out_w_h[lo:hi].copy_(b["ow"][:n], non_blocking=True)
                    out_u_h[lo:hi].copy_(b["ou"][:n], non_blocking=True)
                    b["drained"].record(self.s_out)
        for s in (self.s_in, self.s_run, self.s_out):
            cur.wait_stream(s)


def laplace_stage_times(q, k, v, reps=5):
    """Diagnostic: median device time (ms) of the sort/rank kernel, of the first walk pass (with its fold kernel)
    and of the second, emitting pass; `walk_ms` is the sum of the two passes."""
    P, D, N, M, C = dims = check_qkv(q, k, v)
    L = lib()
    rows = []
    with torch.cuda.device(q.device):
        ws, n = _workspace(L.qlka_laplace_forward_workspace_bytes, dims, q.device)
        out_w = torch.empty(P, M, C, dtype=torch.float32, device=q.device)
        out_u = torch.empty(P, M, dtype=torch.float32, device=q.device)
        for _ in range(reps):
            a, b, c = ctypes.c_float(0), ctypes.c_float(0), ctypes.c_float(0)
            st = L.qlka_laplace_forward_stage_ms(q.data_ptr(), k.data_ptr(), v.data_ptr(), out_w.data_ptr(), out_u.data_ptr(),
                                                 ws.data_ptr(), n, P, D, N, M, C, _stream(), ctypes.byref(a), ctypes.byref(b), ctypes.byref(c))
            if st:
                _raise(st)
            rows.append((a.value, b.value, c.value))
    med = [sorted(col)[len(col) // 2] for col in zip(*rows)]
    return {"sort_rank_ms": med[0], "walk_pass1_ms": med[1], "walk_pass2_ms": med[2], "walk_ms": med[1] + med[2]}


def abs_forward(q, k, v, full, path=-1):
    P, D, N, M, C = dims = check_qkv(q, k, v, "q, k, and v")
    v = _aligned(v)
    L = lib()
    with torch.cuda.device(q.device):
        ws, n = _workspace(L.qlka_abs_forward_workspace_bytes, dims, q.device)
        out_w = torch.empty(P, M, C, dtype=torch.float32, device=q.device)
        out_u = torch.empty(P, M, dtype=torch.float32, device=q.device) if full else None
        st = L.qlka_weighted_abs_sum_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), out_w.data_ptr(),
                                             out_u.data_ptr() if full else None,
                                             ws.data_ptr(), n, P, D, N, M, C, int(path), _stream())
    if st:
        _raise(st)
    return out_w, out_u


def abs_shifted_forward(q, k, v, shifts, weights, full=True):
    """sum_s weights[s] * abs_sum(q + shifts[s], k, v) from one sort of the keys: (out_w, out_u or None)."""
    P, D, N, M, C = check_qkv(q, k, v, "q, k, and v")
    v = _aligned(v)
    ns = len(shifts)
    _check(len(weights) == ns and 1 <= ns <= 4, "shifts and weights must have the same length, 1 to 4")
    L = lib()
    sh = (ctypes.c_float * ns)(*[float(x) for x in shifts])
    wg = (ctypes.c_float * ns)(*[float(x) for x in weights])
    with torch.cuda.device(q.device):
        n = _sz(0)
        st = L.qlka_abs_shifted_forward_workspace_bytes(P, D, N, M, C, ns, ctypes.byref(n))
        if st:
            _raise(st)
        ws = torch.empty(max(int(n.value), 256), dtype=torch.uint8, device=q.device)
        out_w = torch.empty(P, M, C, dtype=torch.float32, device=q.device)
        out_u = torch.empty(P, M, dtype=torch.float32, device=q.device) if full else None
        st = L.qlka_weighted_abs_sum_shifted_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), out_w.data_ptr(),
                                                     out_u.data_ptr() if full else None, sh, wg, ns,
                                                     ws.data_ptr(), int(n.value), P, D, N, M, C, _stream())
    if st:
        _raise(st)
    return out_w, out_u


def abs_backward(q, k, v, g_w, g_u=None):
    P, D, N, M, C = dims = check_qkv(q, k, v, "q, k, and v")
    _check_like(g_w, "g_w", (P, M, C), q)
    if g_u is not None:
        _check_like(g_u, "g_u", (P, M), q)
    v, g_w = _aligned(v), _aligned(g_w)
    L = lib()
    with torch.cuda.device(q.device):
        ws, n = _workspace(L.qlka_abs_backward_workspace_bytes, dims, q.device)
        gq = torch.empty(P, D, M, dtype=torch.float32, device=q.device)
        gk = torch.empty(P, D, N, dtype=torch.float32, device=q.device)
        gv = torch.empty(P, N, C, dtype=torch.float32, device=q.device)
        st = L.qlka_weighted_abs_sum_backward(q.data_ptr(), k.data_ptr(), v.data_ptr(), g_w.data_ptr(),
                                              None if g_u is None else g_u.data_ptr(),
                                              gq.data_ptr(), gk.data_ptr(), gv.data_ptr(),
                                              ws.data_ptr(), n, P, D, N, M, C, _stream())
    if st:
        _raise(st)
    return gq, gk, gv


ATTENTION_KINDS = {"add_laplace": -1, "add_riesz": 0, "add_bump": 1}


def fused_attention(kernel, q, k, v, tau, keep=None):
    """Normalised additive-kernel attention on (B, H, S, D) / (B, H, S, Dv) tensors in one native call (forward only)."""
    kind = ATTENTION_KINDS[kernel]
    _check(q.is_cuda and k.is_cuda and v.is_cuda, "q, k, and v must be CUDA tensors")
    _check(q.dtype == k.dtype == v.dtype == torch.float32, "q, k, and v must be float32")
    _check(q.dim() == 4 and k.shape == q.shape and v.dim() == 4 and v.shape[:3] == q.shape[:3],
           "expected q, k (B, H, S, D) and v (B, H, S, Dv)")
    q, k, v = q.contiguous(), k.contiguous(), _aligned(v.contiguous())
    B, H, S, D = q.shape
    Dv = v.shape[3]
    if keep is not None:
        _check(keep.shape == (B, S), "keep must be (B, S)")
        keep = keep.to(device=q.device, dtype=torch.float32).contiguous()
    L = lib()
    with torch.cuda.device(q.device):
        n = _sz(0)
        if kind < 0:
            st = L.qlka_laplace_attention_workspace_bytes(B, H, S, D, Dv, int(keep is not None), ctypes.byref(n))
        else:
            st = L.qlka_abs_attention_workspace_bytes(kind, B, H, S, D, Dv, int(keep is not None), ctypes.byref(n))
        if st:
            _raise(st)
        ws = torch.empty(max(int(n.value), 1), dtype=torch.uint8, device=q.device)
        out = torch.empty(B, H, S, Dv, dtype=torch.float32, device=q.device)
        kp = None if keep is None else keep.data_ptr()
        if kind < 0:
            st = L.qlka_laplace_attention_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), kp, float(tau), out.data_ptr(),
                                                  ws.data_ptr(), int(n.value), B, H, S, D, Dv, _stream())
        else:
            st = L.qlka_abs_attention_forward(kind, q.data_ptr(), k.data_ptr(), v.data_ptr(), kp, float(tau), out.data_ptr(),
                                              ws.data_ptr(), int(n.value), B, H, S, D, Dv, _stream())
    if st:
        _raise(st)
    return out


def laplace_attention(q, k, v, tau, keep=None):
    return fused_attention("add_laplace", q, k, v, tau, keep)


def laplace_backward(q, k, v, g_w, g_u=None):
    """Gradients (grad_q, grad_k, grad_v) of sum(out_w * g_w) + sum(out_u * g_u) of the Laplace sum."""
    P, D, N, M, C = dims = check_qkv(q, k, v, "q, k, and v")
    _check_like(g_w, "g_w", (P, M, C), q)
    if g_u is not None:
        _check_like(g_u, "g_u", (P, M), q)
    v, g_w = _aligned(v), _aligned(g_w)
    L = lib()
    with torch.cuda.device(q.device):
        ws, n = _workspace(L.qlka_laplace_backward_workspace_bytes, dims, q.device)
        gq = torch.empty(P, D, M, dtype=torch.float32, device=q.device)
        gk = torch.empty(P, D, N, dtype=torch.float32, device=q.device)
        gv = torch.empty(P, N, C, dtype=torch.float32, device=q.device)
        st = L.qlka_weighted_laplace_sum_backward(q.data_ptr(), k.data_ptr(), v.data_ptr(), g_w.data_ptr(),
                                                  None if g_u is None else g_u.data_ptr(),
                                                  gq.data_ptr(), gk.data_ptr(), gv.data_ptr(),
                                                  ws.data_ptr(), n, P, D, N, M, C, _stream())
    if st:
        _raise(st)
    return gq, gk, gv


def sgn_forward(q, k, v, g):
    P, D, N, M, C = dims = check_qkv(q, k, v, "q, k, and v")
    _check_like(g, "g", (P, M, C), q)
    v, g = _aligned(v), _aligned(g)
    L = lib()
    with torch.cuda.device(q.device):
        ws, n = _workspace(L.qlka_sgn_forward_workspace_bytes, dims, q.device)
        out = torch.empty(P, D, M, dtype=torch.float32, device=q.device)
        st = L.qlka_weighted_sgn_sum_forward(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), out.data_ptr(),
                                             ws.data_ptr(), n, P, D, N, M, C, _stream())
    if st:
        _raise(st)
    return out


def sort_rank_records(x, y, mode):
    """Diagnostic: the walk records of the sort/rank stage (see include/qlka.h)."""
    _check(x.is_cuda and y.is_cuda and x.dtype == y.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous(),
           "x and y must be contiguous float32 CUDA tensors")
    P, D, N = x.shape
    M = y.shape[2]
    L = lib()
    NBK = N // 8 + 1
    NP, MS = NBK * 8, (NBK + 1 + 3) // 4 * 4
    dev = x.device
    with torch.cuda.device(dev):
        n = _sz(0)
        st = L.qlka_sort_rank_workspace_bytes(P, D, N, M, ctypes.byref(n))
        if st:
            _raise(st)
        ws = torch.empty(int(n.value), dtype=torch.uint8, device=dev)
        xperm = torch.zeros(P * D, NP, dtype=torch.int32, device=dev)
        xval = torch.zeros(P * D, NP + 8, dtype=torch.float32, device=dev)
        yrec = torch.zeros(P * D, M + 1, 4, dtype=torch.int32, device=dev)
        mstart = torch.zeros(P * D, MS, dtype=torch.int32, device=dev)
        st = L.qlka_sort_rank_records(x.data_ptr(), y.data_ptr(), xperm.data_ptr(), xval.data_ptr(), yrec.data_ptr(),
                                      mstart.data_ptr(), ws.data_ptr(), int(n.value), P, D, N, M, int(mode), _stream())
    if st:
        _raise(st)
    return xperm, xval, yrec, mstart

/* C ABI of the sorted-scan kernel-attention operators for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers (float32, contiguous, all on the current
 * device), sizes and a CUDA stream, enqueues its kernels on that stream and returns at once
 * with a status code; nothing throws and no host synchronisation happens. Outputs are
 * written to caller-allocated buffers. Scratch memory is a caller-allocated workspace whose
 * size the matching *_workspace_bytes function reports; its contents are meaningless between
 * calls. Inputs are never modified.
 *
 * Shapes (row-major): q (P, D, M) queries, k (P, D, N) keys, v (P, N, C) values,
 * g_w / g (P, M, C), g_u (P, M), with P = batch * heads.
 *
 * Alignment: the row matrices - v, g_w, g, out_w, grad_v and the `out` of the attention entry
 * points - must start on a 16-byte boundary (the kernels move their rows with 16-byte copies and
 * vector reductions); anything else returns QLKA_ERR_ALIGNMENT before a kernel is launched.
 * q, k, g_u, out_u, grad_q and grad_k only need float alignment. The workspace needs 256 bytes.
 *
 * Limits shared by all entry points (those of the reference's check_qkv,
 * Weighted_Abs_Sum/csrc/binding.cpp:69-84 and Weighted_Laplace_Sum/csrc/binding.cpp:66-79):
 * P, D, N, M > 0, 1 <= C <= 128, P * D * max(N, M) <= INT32_MAX; N, M <= 262144 here (the reference
 * stops at 131072).
 */
#ifndef QLKA_H
#define QLKA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* qlka_stream_t;   /* a cudaStream_t */

enum qlka_status {
    QLKA_OK = 0,
    QLKA_ERR_BAD_SHAPE = 1,        /* a size is <= 0 */
    QLKA_ERR_C_RANGE = 2,          /* C outside [1, 128] */
    QLKA_ERR_LENGTH = 3,           /* N or M above 262144 */
    QLKA_ERR_INT32 = 4,            /* P * D * max(N, M) does not fit int32 */
    QLKA_ERR_PATH = 5,             /* path not in {-1, 0, 1} */
    QLKA_ERR_FUSED_UNAVAILABLE = 6,/* path == 1 pinned but max(N, M) > 4096 */
    QLKA_ERR_NULL = 7,             /* a required pointer is NULL */
    QLKA_ERR_WORKSPACE = 8,        /* workspace too small or misaligned (256 bytes) */
    QLKA_ERR_CUDA = 9,             /* a CUDA runtime call failed; see qlka_last_cuda_error */
    QLKA_ERR_UNSUPPORTED = 10,     /* a size inside the limits that this build has no kernel for */
    QLKA_ERR_NO_ALLOC_LIMIT = 11,  /* problem too large for the fixed scratch of the *_noalloc entry point */
    QLKA_ERR_ALIGNMENT = 12        /* a row matrix (v, g_w, g, out_w, grad_v, attention out) is not 16-byte aligned */
};

/* Human-readable text of a status code (static storage). */
const char* qlka_status_string(int status);
/* cudaError_t of the last failing runtime call made by this library on the calling thread. */
int qlka_last_cuda_error(void);

/* ---- weighted Laplace sum, forward ------------------------------------------------------
 * out_w[p,m,c] = sum_{d,n} exp(-|k[p,d,n] - q[p,d,m]|) v[p,n,c]     (P, M, C)
 * out_u[p,m]   = sum_{d,n} exp(-|k[p,d,n] - q[p,d,m]|)              (P, M)
 * Replaces weighted_laplace_sum_forward, Weighted_Laplace_Sum/csrc/binding.cpp:63-100
 * (Python: Weighted_Laplace_Sum/weighted_laplace_sum/__init__.py:4-13). */
int qlka_laplace_forward_workspace_bytes(int P, int D, int N, int M, int C, size_t* bytes);
int qlka_weighted_laplace_sum_forward(const float* q, const float* k, const float* v,
                                      float* out_w, float* out_u,
                                      void* workspace, size_t workspace_bytes,
                                      int P, int D, int N, int M, int C, qlka_stream_t stream);

/* The same operator for callers that cannot hand over a workspace and must not trigger an
 * allocation: latency-critical serving loops (cudaMalloc serialises the whole device) and hosts
 * whose own memory pool already owns all of HBM. (Nothing is claimed about recording the call into
 * a CUDA graph: that has not been tested.) The scratch is a fixed array of qlka_noalloc_scratch_bytes() (32 MiB) inside
 * the library image; every GPU that loads the library keeps that much reserved until the process
 * exits. Problems whose scratch would not fit are refused with QLKA_ERR_NO_ALLOC_LIMIT (roughly:
 * P*D*(N+M) above a few hundred thousand elements) - use the workspace variant for those. The call
 * allocates nothing and frees nothing once the array exists: with CUDA's default lazy module loading
 * the array is materialised by the first call on each device (which looks up its device address), or
 * at load time under CUDA_MODULE_LOADING=EAGER. So make one call per device at start-up, before the
 * host's own pool has taken the memory; that first call is the one that
 * can fail with QLKA_ERR_CUDA (out of memory), later ones leave free device memory untouched. All calls
 * share the one array: two calls whose kernels can overlap on the GPU (different streams, or
 * different host threads) corrupt each other, so serialise them. Nothing needs to be cleared
 * between calls. This entry point has no counterpart in the reference, whose operators allocate
 * through the torch caching allocator. */
size_t qlka_noalloc_scratch_bytes(void);
int qlka_weighted_laplace_sum_forward_noalloc(const float* q, const float* k, const float* v,
                                              float* out_w, float* out_u,
                                              int P, int D, int N, int M, int C, qlka_stream_t stream);

/* Diagnostic: the same call, but it waits for completion and reports the device time of the
 * sort/rank kernel, of the first walk pass (with the small fold kernel that follows it) and of the
 * second, emitting walk pass (CUDA events on `stream`), in milliseconds.
 * The reference has no counterpart; its benchmark times whole calls
 * (Experiments/speed_and_memory/bench.py:83-121). */
int qlka_laplace_forward_stage_ms(const float* q, const float* k, const float* v,
                                  float* out_w, float* out_u,
                                  void* workspace, size_t workspace_bytes,
                                  int P, int D, int N, int M, int C, qlka_stream_t stream,
                                  float* sort_ms, float* pass1_ms, float* pass2_ms);

/* ---- weighted Laplace sum, backward -----------------------------------------------------
 * Gradients of sum(out_w * g_w) + sum(out_u * g_u) (g_u NULL: first term only):
 * grad_q (P, D, M), grad_k (P, D, N), grad_v (P, N, C), from two more sort/rank runs and two
 * walks. exp(-|k - q|) has no derivative where a key equals a query; there both grad_q and
 * grad_k take the one-sided derivative +1 of the side the walk puts ties on (torch autograd
 * through exp(-abs(x)) takes 0 there). The reference has no counterpart: its Laplace operator
 * is forward only and training goes through the chunked PyTorch path
 * (Experiments/kernel_attention/attention.py:110-115). */
int qlka_laplace_backward_workspace_bytes(int P, int D, int N, int M, int C, size_t* bytes);
int qlka_weighted_laplace_sum_backward(const float* q, const float* k, const float* v,
                                       const float* g_w, const float* g_u /* nullable */,
                                       float* grad_q, float* grad_k, float* grad_v,
                                       void* workspace, size_t workspace_bytes,
                                       int P, int D, int N, int M, int C, qlka_stream_t stream);

/* ---- add_laplace attention on the caller's layout ---------------------------------------
 * out[b,h,i,:] = sum_j A_ij v[b,h,j,:] / max(sum_j A_ij, 1e-6),  A_ij = sum_d exp(-|q[b,h,i,d] - k[b,h,j,d]| / tau),
 * with q, k (B, H, S, D), v and out (B, H, S, Dv) contiguous and keep (B, S) an optional key-keep mask of 0 / 1 floats
 * (NULL: all keys kept). One call does what the reference spreads over attention() and _add_laplace
 * (Experiments/kernel_attention/attention.py:67-72, 95-126) around its operator: the layout change to (P, D, S) fused
 * with the division by tau and the zeroing of masked keys, the Laplace sum accumulated straight into `out`, and the
 * normalisation with the row sum corrected for the masked keys. Forward only. `masked` in the size query is 1 when a
 * keep mask will be passed. */
int qlka_laplace_attention_workspace_bytes(int B, int H, int S, int D, int Dv, int masked, size_t* bytes);
int qlka_laplace_attention_forward(const float* q, const float* k, const float* v, const float* keep /* nullable */,
                                   float tau, float* out, void* workspace, size_t workspace_bytes,
                                   int B, int H, int S, int D, int Dv, qlka_stream_t stream);

/* The same for the two kernels that go through the abs sum (forward only), kind 0 = add_riesz, kind 1 = add_bump:
 *   add_riesz  A_ij = |q_i|_1 + |k_j|_1 - |q_i - k_j|_1 + 1e-3   (Experiments/kernel_attention/attention.py:75-81)
 *   add_bump   A_ij = sum_d max(0, 1 - |q_id - k_jd|)             (:84-92; one sort for the three shifted abs sums,
 *              which limits it to 3 S <= 16384 - longer sequences get QLKA_ERR_UNSUPPORTED and go op by op)
 * with q and k divided by tau first; out = A v / max(row sum of A, 1e-6) over the kept keys. */
int qlka_abs_attention_workspace_bytes(int kind, int B, int H, int S, int D, int Dv, int masked, size_t* bytes);
int qlka_abs_attention_forward(int kind, const float* q, const float* k, const float* v, const float* keep /* nullable */,
                               float tau, float* out, void* workspace, size_t workspace_bytes,
                               int B, int H, int S, int D, int Dv, qlka_stream_t stream);

/* ---- weighted abs sum, forward ---------------------------------------------------------
 * out_w[p,m,c] = sum_{d,n} |k[p,d,n] - q[p,d,m]| v[p,n,c]           (P, M, C)
 * out_u[p,m]   = sum_{d,n} |k[p,d,n] - q[p,d,m]|                    (P, M), optional (NULL)
 * path: -1 auto, 0 global, 1 fused - kept for signature compatibility; the three values run
 * the same kernels here, but path == 1 with max(N, M) > 4096 is rejected as in the reference.
 * Replaces weighted_abs_sum_forward / weighted_abs_sum_full_forward,
 * Weighted_Abs_Sum/csrc/binding.cpp:132-239. */
int qlka_abs_forward_workspace_bytes(int P, int D, int N, int M, int C, size_t* bytes);
int qlka_weighted_abs_sum_forward(const float* q, const float* k, const float* v,
                                  float* out_w, float* out_u /* nullable */,
                                  void* workspace, size_t workspace_bytes,
                                  int P, int D, int N, int M, int C, int path, qlka_stream_t stream);

/* ---- weighted abs sum over shifted queries ---------------------------------------------
 * out = sum_s weights[s] * abs_sum(q + shifts[s], k, v) for 1 <= n_shifts <= 4 from ONE sort of the keys:
 * the shifted copies of the queries are ranked together and share their output rows. out_u likewise
 * (nullable). Needs N <= 16384 and n_shifts * M <= 16384. shifts and weights are host arrays.
 * With shifts (0, +1, -1) and weights (-1, 1/2, 1/2) this is the whole add_bump numerator and row sum,
 * which the reference assembles from three separate abs sums
 * (Experiments/kernel_attention/attention.py:84-92). Forward only. */
int qlka_abs_shifted_forward_workspace_bytes(int P, int D, int N, int M, int C, int n_shifts, size_t* bytes);
int qlka_weighted_abs_sum_shifted_forward(const float* q, const float* k, const float* v,
                                          float* out_w, float* out_u /* nullable */,
                                          const float* shifts, const float* weights, int n_shifts,
                                          void* workspace, size_t workspace_bytes,
                                          int P, int D, int N, int M, int C, qlka_stream_t stream);

/* ---- weighted abs sum, backward --------------------------------------------------------
 * Gradients of sum(out_w * g_w) + sum(out_u * g_u) (g_u NULL: first term only):
 * grad_q (P, D, M), grad_k (P, D, N), grad_v (P, N, C); a key equal to a query has
 * sub-gradient -1 for both. Replaces weighted_abs_sum_backward /
 * weighted_abs_sum_full_backward, Weighted_Abs_Sum/csrc/binding.cpp:246-380. */
int qlka_abs_backward_workspace_bytes(int P, int D, int N, int M, int C, size_t* bytes);
int qlka_weighted_abs_sum_backward(const float* q, const float* k, const float* v,
                                   const float* g_w, const float* g_u /* nullable */,
                                   float* grad_q, float* grad_k, float* grad_v,
                                   void* workspace, size_t workspace_bytes,
                                   int P, int D, int N, int M, int C, qlka_stream_t stream);

/* ---- weighted sgn sum ------------------------------------------------------------------
 * out[p,d,m] = sum_n sgn(k[p,d,n] - q[p,d,m]) <v[p,n,:], g[p,m,:]>, sgn(0) = +1   (P, D, M)
 * Replaces weighted_sgn_sum_forward, Weighted_Abs_Sum/csrc/binding.cpp:383-439. */
int qlka_sgn_forward_workspace_bytes(int P, int D, int N, int M, int C, size_t* bytes);
int qlka_weighted_sgn_sum_forward(const float* q, const float* k, const float* v, const float* g,
                                  float* out,
                                  void* workspace, size_t workspace_bytes,
                                  int P, int D, int N, int M, int C, qlka_stream_t stream);

/* ---- diagnostic: the sort/rank stage alone ---------------------------------------------
 * Sorts x (P, D, N) as the key stream and ranks y (P, D, M) against it, writing the walk
 * records: xperm (P*D, NP) uint32, xval (P*D, NP + 8) float, yrec (P*D, M + 1) 4 x uint32
 * {e0, e1, row, rank} (the last entry of a segment is a sentinel), mstart (P*D, MS) uint32, where NP = (N/8 + 1) * 8 and
 * MS = (N/8 + 2) rounded up to a multiple of 4. mode 0: Laplace records, 1: abs records.
 * Corresponds to sort_qk of the reference (Weighted_Laplace_Sum/csrc/binding.cpp:33-58);
 * exists so that tests can check the stage on its own. */
int qlka_sort_rank_workspace_bytes(int P, int D, int N, int M, size_t* bytes);
int qlka_sort_rank_records(const float* x, const float* y,
                           uint32_t* xperm, float* xval, uint32_t* yrec, uint32_t* mstart,
                           void* workspace, size_t workspace_bytes,
                           int P, int D, int N, int M, int mode, qlka_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* QLKA_H */

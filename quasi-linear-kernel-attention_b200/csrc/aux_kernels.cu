// Small streaming kernels around the walks: the pre-reductions and the rank-1 initial value
// of the abs sum (the reference uses ATen sum / bmm for the former,
// Weighted_Abs_Sum/csrc/binding.cpp:154-159,286-289,349-350, and abs_init for the latter,
// Weighted_Abs_Sum/csrc/abs_kernels.cu:23-70), and channel padding to a multiple of four
// (the reference pads odd C to even with constant_pad_nd, binding.cpp:87-89).
#include "qlka_common.cuh"

namespace qlka {

// out[p, l] = sum_d x[p, d, l]   (ABS: sum_d |x[p, d, l]|)
template <bool ABS>
__global__ void colsum_d_kernel(const float* __restrict__ x, float* __restrict__ out, const int D, const int L, const long long total) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long p = i / L, l = i % L;
    const float* src = x + p * D * L + l;
    float acc = 0.0f;
    for (int d = 0; d < D; d++) { const float t = src[(long long)d * L]; acc += ABS ? fabsf(t) : t; }
    out[i] = acc;
}

// Per p over rows r of w (P, R, C4) with optional row scalars s (P, R):
//   wsum[p, c] += sum_r w[r, c],  swsum[p, c] += sum_r s[r] w[r, c],  ssum[p] += sum_r s[r]
// (outputs must be zeroed; partial sums of a row tile are added atomically). grid (tiles, P).
constexpr int RS_THREADS = 256, RS_ROWS = 256;
__global__ void __launch_bounds__(RS_THREADS) rowstat_kernel(
    const float* __restrict__ w, const float* __restrict__ s,
    float* __restrict__ wsum, float* __restrict__ swsum, float* __restrict__ ssum,
    const int R, const int C4)
{
    __shared__ float red_w[RS_THREADS], red_k[RS_THREADS];
    const int chunks = (R + RS_ROWS - 1) / RS_ROWS;               // (p rides in blockIdx.x: a grid's y extent stops at 65535)
    const int p  = blockIdx.x / chunks;
    const int r0 = (blockIdx.x % chunks) * RS_ROWS, r1 = min(R, r0 + RS_ROWS);
    const int CW = C4 <= 32 ? 32 : (C4 <= 64 ? 64 : 128);
    const int c  = threadIdx.x % CW, lane_r = threadIdx.x / CW, nr = RS_THREADS / CW;
    float aw = 0.0f, ak = 0.0f, as = 0.0f;
    if (c < C4) {
        for (int r = r0 + lane_r; r < r1; r += nr) {
            const float x  = w[((long long)p * R + r) * C4 + c];
            const float sc = s ? s[(long long)p * R + r] : 0.0f;
            aw += x;
            ak = fmaf(sc, x, ak);
            if (c == 0) as += sc;
        }
    }
    red_w[threadIdx.x] = aw; red_k[threadIdx.x] = ak;
    __syncthreads();
    if (lane_r == 0 && c < C4) {
        for (int j = 1; j < nr; j++) { aw += red_w[j * CW + c]; ak += red_k[j * CW + c]; }
        atomicAdd(wsum + (long long)p * C4 + c, aw);
        if (swsum) atomicAdd(swsum + (long long)p * C4 + c, ak);
    }
    if (ssum && c == 0) atomicAdd(ssum + p, as);
}

// out[p] = sum_l x[p, l]; one CTA per p
__global__ void __launch_bounds__(256) vecsum_kernel(const float* __restrict__ x, float* __restrict__ out, const int L) {
    __shared__ float red[256];
    const int p = blockIdx.x;
    float acc = 0.0f;
    for (int l = threadIdx.x; l < L; l += 256) acc += x[(long long)p * L + l];
    red[threadIdx.x] = acc;
    __syncthreads();
    for (int off = 128; off > 0; off >>= 1) {
        if (threadIdx.x < off) red[threadIdx.x] += red[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[p] = red[0];
}

// out[p, m, c] = A * ktot[p, c] - (A * qsum[p, m] + Bq) * vsum[p, c];  out_u[p, m] = A * ksr[p] - Nk * (A * qsum[p, m] + Bq)
// (A = 1, Bq = 0 for the plain abs sum; a folded sum over shifted queries has A = sum of weights, Bq = D * sum w_s shift_s)
__global__ void abs_init_kernel(
    const float* __restrict__ ktot, const float* __restrict__ vsum, const float* __restrict__ qsum,
    const float* __restrict__ ksr, float* __restrict__ out, float* __restrict__ out_u,
    const int M, const int C4, const float Nk, const long long total4, const float A, const float Bq)
{
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total4) return;
    const int       q4 = C4 >> 2;
    const int       c  = (int)(i % q4) * 4;
    const long long pm = i / q4;
    const long long p  = pm / M;
    const float4 kt = *reinterpret_cast<const float4*>(ktot + p * C4 + c);
    const float4 vs = *reinterpret_cast<const float4*>(vsum + p * C4 + c);
    const float  qs = fmaf(A, qsum[pm], Bq);
    *reinterpret_cast<float4*>(out + pm * C4 + c) =
        make_float4(fmaf(-qs, vs.x, A * kt.x), fmaf(-qs, vs.y, A * kt.y), fmaf(-qs, vs.z, A * kt.z), fmaf(-qs, vs.w, A * kt.w));
    if (out_u && c == 0) out_u[pm] = A * ksr[p] - Nk * qs;
}

// dst (rows, C4) <- src (rows, C), zero filled
__global__ void pad_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, const int C, const int C4, const long long total) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long r = i / C4; const int c = (int)(i % C4);
    dst[i] = c < C ? src[r * C + c] : 0.0f;
}
// dst (rows, C) <- src (rows, C4)
__global__ void unpad_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, const int C, const int C4, const long long total) {
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long r = i / C; const int c = (int)(i % C);
    dst[i] = src[r * C4 + c];
}

// ---- the caller's side of add_laplace attention (Experiments/kernel_attention/attention.py:67-72, 95-126) ----
// dst[p, d, s] = src[p, s, d] * scale * (keep ? keep[p / H, s] : 1): the (B, H, S, D) -> (P, D, S) layout change of
// attention(), the division by tau and the zeroing of masked keys in one pass; 32 x 32 tiles through shared memory
__global__ void __launch_bounds__(256) transpose_scale_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                              const float* __restrict__ keep, const float scale,
                                                              const int S, const int D, const int H)
{
    __shared__ float tile[32][33];
    const int stiles = (S + 31) / 32;
    const int p  = blockIdx.x / stiles;
    const int s0 = (blockIdx.x % stiles) * 32, d0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;       // 32 x 8
    const float* sp = src + (long long)p * S * D;
    float*       dp = dst + (long long)p * D * S;
    #pragma unroll
    for (int r = ty; r < 32; r += 8) {
        const int s = s0 + r, d = d0 + tx;
        float x = 0.0f;
        if (s < S && d < D) {
            x = sp[(long long)s * D + d] * scale;
            if (keep) x *= keep[(long long)(p / H) * S + s];
        }
        tile[r][tx] = x;
    }
    __syncthreads();
    #pragma unroll
    for (int r = ty; r < 32; r += 8) {
        const int d = d0 + r, s = s0 + tx;
        if (d < D && s < S) dp[(long long)d * S + s] = tile[tx][r];
    }
}

// dst[p, s, :] = src[p, s, :] * keep[p / H, s]
__global__ void mask_rows_kernel(const float* __restrict__ src, float* __restrict__ dst, const float* __restrict__ keep,
                                 const int S, const int C, const int H, const long long total)
{
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long ps = i / C;
    const long long p = ps / S, s = ps % S;
    dst[i] = src[i] * keep[(p / H) * S + s];
}

// n_pad[b] = S - sum_s keep[b, s]; one CTA per b
__global__ void __launch_bounds__(256) npad_kernel(const float* __restrict__ keep, float* __restrict__ n_pad, const int S) {
    __shared__ float red[256];
    const int b = blockIdx.x;
    float acc = 0.0f;
    for (int s = threadIdx.x; s < S; s += 256) acc += keep[(long long)b * S + s];
    red[threadIdx.x] = acc;
    __syncthreads();
    for (int off = 128; off > 0; off >>= 1) {
        if (threadIdx.x < off) red[threadIdx.x] += red[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) n_pad[b] = (float)S - red[0];
}

// out[p, m, :] /= max(out_u[p, m] - n_pad[p / H] * sum_d f(qt[p, d, m]), clamp): the row normalisation of _add_laplace
// (BUMP = false, f(x) = exp(-|x|)) and of _add_bump (BUMP = true, f(x) = max(0, 1 - |x|)), with the row sum corrected for
// the masked keys (each sits at k = 0 with v = 0 and adds f(q_d) per dimension). One warp per row.
template <bool BUMP>
__global__ void __launch_bounds__(256) normalise_kernel(float* __restrict__ out, const float* __restrict__ out_u,
                                                        const float* __restrict__ qt, const float* __restrict__ n_pad,
                                                        const int M, const int D, const int C, const int H,
                                                        const float clamp, const long long rows)
{
    const long long row  = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int       lane = threadIdx.x & 31;
    if (row >= rows) return;
    const long long p = row / M, m = row % M;
    float den = out_u[row];
    if (n_pad) {
        const float np = n_pad[p / H];
        if (np != 0.0f) {
            float acc = 0.0f;
            for (int d = lane; d < D; d += 32) {
                const float x = fabsf(qt[(p * D + d) * M + m]);
                acc += BUMP ? fmaxf(0.0f, 1.0f - x) : __expf(-x);
            }
            #pragma unroll
            for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(FULL, acc, off);
            den -= np * acc;
        }
    }
    const float inv = 1.0f / fmaxf(den, clamp);
    float* o = out + row * C;
    for (int c = lane; c < C; c += 32) o[c] *= inv;
}

// The add_riesz epilogue (Experiments/kernel_attention/attention.py:75-81), in place on out = the weighted abs sum:
//   a = aq[p, m] + eps;  num = a * vsum[p, :] + akv[p, :] - out;  den = a * S + aksum[p] - out_u[p, m] - eps * n_pad[p / H]
//   out = num / max(den, clamp).   One warp per row.
__global__ void __launch_bounds__(256) riesz_epilogue_kernel(float* __restrict__ out, const float* __restrict__ out_u,
                                                             const float* __restrict__ aq, const float* __restrict__ vsum,
                                                             const float* __restrict__ akv, const float* __restrict__ aksum,
                                                             const float* __restrict__ n_pad,
                                                             const int M, const int C, const int C4, const int H,
                                                             const float eps, const float clamp, const long long rows)
{
    const long long row  = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int       lane = threadIdx.x & 31;
    if (row >= rows) return;
    const long long p = row / M;
    const float a   = aq[row] + eps;
    const float np  = n_pad ? n_pad[p / H] : 0.0f;
    const float den = a * (float)M + aksum[p] - out_u[row] - eps * np;
    const float inv = 1.0f / fmaxf(den, clamp);
    float* o = out + row * C;
    for (int c = lane; c < C; c += 32) o[c] = (fmaf(a, vsum[p * C4 + c], akv[p * C4 + c]) - o[c]) * inv;
}

static inline unsigned blocks_for(long long total, int threads) { return (unsigned)((total + threads - 1) / threads); }

cudaError_t launch_colsum_d(const float* x, float* out, int P, int D, int L, cudaStream_t st) {
    const long long total = (long long)P * L;
    colsum_d_kernel<false><<<blocks_for(total, 256), 256, 0, st>>>(x, out, D, L, total);
    return cudaGetLastError();
}
cudaError_t launch_abscolsum_d(const float* x, float* out, int P, int D, int L, cudaStream_t st) {
    const long long total = (long long)P * L;
    colsum_d_kernel<true><<<blocks_for(total, 256), 256, 0, st>>>(x, out, D, L, total);
    return cudaGetLastError();
}
cudaError_t launch_rowstat(const float* w, const float* s, float* wsum, float* swsum, float* ssum, int P, int R, int C4, cudaStream_t st) {
    const unsigned grid = (unsigned)((R + RS_ROWS - 1) / RS_ROWS) * (unsigned)P;
    rowstat_kernel<<<grid, RS_THREADS, 0, st>>>(w, s, wsum, swsum, ssum, R, C4);
    return cudaGetLastError();
}
cudaError_t launch_vecsum(const float* x, float* out, int P, int L, cudaStream_t st) {
    vecsum_kernel<<<P, 256, 0, st>>>(x, out, L);
    return cudaGetLastError();
}
cudaError_t launch_abs_init(const float* ktot, const float* vsum, const float* qsum, const float* ksr,
                            float* out, float* out_u, int P, int M, int C4, int Nk, float A, float Bq, cudaStream_t st) {
    const long long total4 = (long long)P * M * (C4 >> 2);
    abs_init_kernel<<<blocks_for(total4, 256), 256, 0, st>>>(ktot, vsum, qsum, ksr, out, out_u, M, C4, (float)Nk, total4, A, Bq);
    return cudaGetLastError();
}
cudaError_t launch_pad_rows(const float* src, float* dst, long long rows, int C, int C4, cudaStream_t st) {
    const long long total = rows * C4;
    pad_rows_kernel<<<blocks_for(total, 256), 256, 0, st>>>(src, dst, C, C4, total);
    return cudaGetLastError();
}
cudaError_t launch_unpad_rows(const float* src, float* dst, long long rows, int C, int C4, cudaStream_t st) {
    const long long total = rows * C;
    unpad_rows_kernel<<<blocks_for(total, 256), 256, 0, st>>>(src, dst, C, C4, total);
    return cudaGetLastError();
}

cudaError_t launch_transpose_scale(const float* src, float* dst, const float* keep, float scale, int P, int S, int D, int H, cudaStream_t st) {
    dim3 grid((unsigned)((S + 31) / 32) * (unsigned)P, (D + 31) / 32);
    transpose_scale_kernel<<<grid, 256, 0, st>>>(src, dst, keep, scale, S, D, H);
    return cudaGetLastError();
}
cudaError_t launch_mask_rows(const float* src, float* dst, const float* keep, int P, int S, int C, int H, cudaStream_t st) {
    const long long total = (long long)P * S * C;
    mask_rows_kernel<<<blocks_for(total, 256), 256, 0, st>>>(src, dst, keep, S, C, H, total);
    return cudaGetLastError();
}
cudaError_t launch_npad(const float* keep, float* n_pad, int B, int S, cudaStream_t st) {
    npad_kernel<<<B, 256, 0, st>>>(keep, n_pad, S);
    return cudaGetLastError();
}
cudaError_t launch_normalise(float* out, const float* out_u, const float* qt, const float* n_pad,
                             int P, int M, int D, int C, int H, float clamp, bool bump, cudaStream_t st) {
    const long long rows = (long long)P * M;
    if (bump) normalise_kernel<true><<<blocks_for(rows, 8), 256, 0, st>>>(out, out_u, qt, n_pad, M, D, C, H, clamp, rows);
    else      normalise_kernel<false><<<blocks_for(rows, 8), 256, 0, st>>>(out, out_u, qt, n_pad, M, D, C, H, clamp, rows);
    return cudaGetLastError();
}
cudaError_t launch_riesz_epilogue(float* out, const float* out_u, const float* aq, const float* vsum, const float* akv,
                                  const float* aksum, const float* n_pad, int P, int M, int C, int C4, int H,
                                  float eps, float clamp, cudaStream_t st) {
    const long long rows = (long long)P * M;
    riesz_epilogue_kernel<<<blocks_for(rows, 8), 256, 0, st>>>(out, out_u, aq, vsum, akv, aksum, n_pad, M, C, C4, H, eps, clamp, rows);
    return cudaGetLastError();
}

}  // namespace qlka

// Sort/rank kernel for segments of up to 16384 keys and queries: one CTA per segment sorts
// the keys and then the queries with a stable LSD radix sort that lives entirely in shared
// memory (8-bit digits, keys carried with their 16-bit index), ranks every query among the
// keys, and writes the walk records described in qlka_common.cuh.
//
// The reference does this step with two CUB segmented radix sorts through global memory
// (Weighted_Laplace_Sum/csrc/sort_utils.cu:23-81, Weighted_Abs_Sum/csrc/sort_utils.cu:18-75,
// called from sort_qk, Weighted_Laplace_Sum/csrc/binding.cpp:33-58) and searches the query
// ranges inside the walk kernels (laplace_kernels.cu:253-254, walk_common.cuh:23-30).
#include "qlka_common.cuh"

namespace qlka {

// ------------------------------------------------------------------ block radix sort
// Elements are held in registers, E per thread, in warp-blocked order: the element at
// array position warp*32*E + s*32 + lane sits in slot s of that lane. One pass ranks each
// element among equal digits of its own warp (match_any + per-warp counters, processed in
// array order so the pass is stable), scans the counters digit-major, and scatters through
// shared memory.
template <int THREADS, int E>
__device__ __forceinline__ void block_radix_sort(
    uint32_t (&key)[E], uint32_t (&idx)[E],
    uint32_t* __restrict__ skey, uint16_t* __restrict__ sidx,
    uint32_t* __restrict__ cnt, uint32_t* __restrict__ base, uint32_t* __restrict__ wsum)
{
    constexpr int W = THREADS / 32;
    const int      tid  = threadIdx.x;
    const int      warp = tid >> 5, lane = tid & 31;
    const uint32_t lt   = (1u << lane) - 1u;
    uint32_t*      mycnt = cnt + warp * 256;

    #pragma unroll 1
    for (int pass = 0; pass < 4; pass++) {
        const int shift = 8 * pass;
        for (int i = tid; i < W * 256; i += THREADS) cnt[i] = 0;
        __syncthreads();

        uint32_t rk[E];
        #pragma unroll
        for (int s = 0; s < E; s++) {
            const uint32_t d      = (key[s] >> shift) & 255u;
            const uint32_t peers  = __match_any_sync(FULL, d);
            const int      leader = __ffs(peers) - 1;
            uint32_t       old    = 0;
            if (lane == leader) { old = mycnt[d]; mycnt[d] = old + __popc(peers); }
            old   = __shfl_sync(FULL, old, leader);
            rk[s] = old + __popc(peers & lt);
            __syncwarp();
        }
        __syncthreads();

        // per digit: exclusive scan over warps, then exclusive scan of the digit totals
        uint32_t tot = 0, incl = 0;
        if (tid < 256) {
            uint32_t run = 0;
            #pragma unroll 4
            for (int w = 0; w < W; w++) { uint32_t c = cnt[w * 256 + tid]; cnt[w * 256 + tid] = run; run += c; }
            tot  = run;
            incl = tot;
            #pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                uint32_t t = __shfl_up_sync(FULL, incl, off);
                if (lane >= off) incl += t;
            }
            if (lane == 31) wsum[warp] = incl;
        }
        __syncthreads();
        if (tid < 256) {
            uint32_t pre = 0;
            for (int w = 0; w < warp; w++) pre += wsum[w];
            base[tid] = pre + incl - tot;
        }
        __syncthreads();

        #pragma unroll
        for (int s = 0; s < E; s++) {
            const uint32_t d   = (key[s] >> shift) & 255u;
            const uint32_t dst = base[d] + mycnt[d] + rk[s];
            skey[dst] = key[s];
            sidx[dst] = (uint16_t)idx[s];
        }
        __syncthreads();
        if (pass < 3) {
            #pragma unroll
            for (int s = 0; s < E; s++) {
                const int pos = warp * 32 * E + s * 32 + lane;
                key[s] = skey[pos];
                idx[s] = sidx[pos];
            }
        }
    }
}

template <int THREADS, int E>
__device__ __forceinline__ void load_segment(const float* __restrict__ src, const int n,
                                             uint32_t (&key)[E], uint32_t (&idx)[E])
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    #pragma unroll
    for (int s = 0; s < E; s++) {
        const int pos = warp * 32 * E + s * 32 + lane;
        key[s] = pos < n ? f2key(src[pos]) : 0xffffffffu;     // padding sorts last (stable: after any real key)
        idx[s] = pos;
    }
}

// ------------------------------------------------------------------ block scan of x_j = A_j x_{j-1} + B_j
// Inclusive, x_{-1} = 0, j = 0..n-1 in scan order; `elem(i, A, B)` gives the coefficients of
// scan position i and `store(i, x)` receives the result. Each thread owns a contiguous run.
template <int THREADS, class Elem, class Store>
__device__ __forceinline__ void block_affine_scan(const int n, float* __restrict__ wa, float* __restrict__ wb,
                                                  Elem elem, Store store)
{
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int per = (n + THREADS - 1) / THREADS;
    const int i0  = min(n, tid * per), i1 = min(n, i0 + per);

    float a = 1.0f, b = 0.0f;                     // composite of my run: x -> a x + b
    for (int i = i0; i < i1; i++) { float A, B; elem(i, A, B); a = A * a; b = A * b + B; }

    float ia = a, ib = b;                         // inclusive over lanes
    #pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        float pa = __shfl_up_sync(FULL, ia, off), pb = __shfl_up_sync(FULL, ib, off);
        if (lane >= off) { ib = ia * pb + ib; ia = ia * pa; }
    }
    __syncthreads();                              // wa/wb may still be read by a previous scan
    if (lane == 31) { wa[warp] = ia; wb[warp] = ib; }
    __syncthreads();
    float pb = 0.0f;                              // state entering my warp
    for (int w = 0; w < warp; w++) pb = wa[w] * pb + wb[w];
    float ea = __shfl_up_sync(FULL, ia, 1), eb = __shfl_up_sync(FULL, ib, 1);
    if (lane == 0) { ea = 1.0f; eb = 0.0f; }
    float x = ea * pb + eb;                       // state entering my run
    for (int i = i0; i < i1; i++) { float A, B; elem(i, A, B); x = A * x + B; store(i, x); }
}

__device__ __forceinline__ int lower_bound_f(const float* __restrict__ a, const int n, const float x) {
    int lo = 0, hi = n;
    while (lo < hi) { int mid = (lo + hi) >> 1; if (a[mid] < x) lo = mid + 1; else hi = mid; }
    return lo;
}
__device__ __forceinline__ int lower_bound_u(const uint32_t* __restrict__ a, const int n, const uint32_t x) {
    int lo = 0, hi = n;
    while (lo < hi) { int mid = (lo + hi) >> 1; if (a[mid] < x) lo = mid + 1; else hi = mid; }
    return lo;
}

// ------------------------------------------------------------------ the kernel
template <int THREADS, int E>
__global__ void __launch_bounds__(THREADS) sort_rank_small(const SortArgs a)
{
    constexpr int CAP = THREADS * E;
    constexpr int W   = THREADS / 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint32_t* skey = reinterpret_cast<uint32_t*>(smem_raw);
    float*    xs   = reinterpret_cast<float*>(skey + CAP);
    uint32_t* cnt  = reinterpret_cast<uint32_t*>(xs + CAP);
    uint32_t* base = cnt + W * 256;
    uint32_t* wsum = base + 256;
    float*    wa   = reinterpret_cast<float*>(wsum + 32);
    float*    wb   = wa + 32;
    uint16_t* sidx = reinterpret_cast<uint16_t*>(wb + 32);

    const int tid = threadIdx.x;
    const int seg = blockIdx.x;
    const int p   = seg / a.D;
    const int N = a.N, M = a.M;
    const int NP = npad(N), NBK = nblocks(N);

    uint32_t* xperm  = a.xperm + (long long)seg * NP;
    float*    xval   = a.xval + (long long)seg * xstride(N);
    uint4*    yrec   = a.yrec + (long long)seg * (M + 1);
    uint32_t* mstart = a.mstart + (long long)seg * mstride(N);
    float*    su0    = a.su0 ? a.su0 + (long long)seg * (N + 1) : nullptr;
    float*    su1    = a.su1 ? a.su1 + (long long)seg * (N + 1) : nullptr;

    uint32_t key[E], idx[E];

    // ---- keys
    load_segment<THREADS, E>(a.x + (long long)seg * N, N, key, idx);
    block_radix_sort<THREADS, E>(key, idx, skey, sidx, cnt, base, wsum);
    for (int j = tid; j < NP; j += THREADS) {
        if (j < N) xs[j] = key2f(skey[j]);
        xperm[j] = j < N ? (uint32_t)sidx[j] : 0u;
    }
    __syncthreads();

    auto dec = [&](int j) -> float { return (j > 0 && j < N) ? expf(-(xs[j] - xs[j - 1])) : 0.0f; };   // a_j
    if (a.mode != MODE_SGN) {
        for (int j = tid; j < NP + KB; j += THREADS) {
            float val;
            if (a.mode == MODE_LAPLACE) val = j < N ? dec(j) : 1.0f;
            else                        val = j < N ? xs[j] : 0.0f;
            xval[j] = val;
        }
    }

    // ---- scalar scans over the sorted keys (results in su0 / su1, read back per query below)
    if (a.scal == SCAL_UNIT && a.mode == MODE_LAPLACE) {
        // su0[j] = sum_{i<=j} exp(-(k_j - k_i)),  su1[j] = sum_{i>=j} exp(-(k_i - k_j))
        block_affine_scan<THREADS>(N, wa, wb,
            [&](int i, float& A, float& B) { A = dec(i); B = 1.0f; },
            [&](int i, float x) { su0[i] = x; });
        block_affine_scan<THREADS>(N, wa, wb,
            [&](int i, float& A, float& B) { A = dec(N - i); B = 1.0f; },      // position i <-> key N-1-i, decay a_{j+1}
            [&](int i, float x) { su1[N - 1 - i] = x; });
    } else if (a.scal == SCAL_UNIT) {
        // su0[j] = sum_{i<=j} k_i
        block_affine_scan<THREADS>(N, wa, wb,
            [&](int i, float& A, float& B) { A = 1.0f; B = xs[i]; },
            [&](int i, float x) { su0[i] = x; });
    } else if (a.scal == SCAL_PREFIX) {
        const float* us = a.us + (long long)p * N;
        block_affine_scan<THREADS>(N, wa, wb,
            [&](int i, float& A, float& B) { A = 1.0f; B = us[sidx[i]]; },
            [&](int i, float x) { su0[i] = x; });
    }
    __syncthreads();          // sidx / skey are about to be reused; the su arrays are complete

    // ---- queries
    load_segment<THREADS, E>(a.y + (long long)seg * M, M, key, idx);
    block_radix_sort<THREADS, E>(key, idx, skey, sidx, cnt, base, wsum);

    for (int m = tid; m < M; m += THREADS) {
        const float    y   = key2f(skey[m]);
        const uint32_t row = sidx[m];
        const int      r   = lower_bound_f(xs, N, y);
        float e0 = 0.0f, e1 = 0.0f;
        if (a.mode == MODE_LAPLACE) {
            e0 = r > 0 ? expf(-(y - xs[r - 1])) : 0.0f;
            e1 = r < N ? expf(-(xs[r] - y)) : 0.0f;
            if (a.scal == SCAL_UNIT) {
                float u = (r > 0 ? e0 * su0[r - 1] : 0.0f) + (r < N ? e1 * su1[r] : 0.0f);
                atomicAdd(a.out_u + (long long)p * M + row, u);
            }
        } else {
            if (a.mode == MODE_ABS) e0 = 2.0f * y;
            if (a.scal == SCAL_UNIT) {
                float pk = r > 0 ? su0[r - 1] : 0.0f;
                atomicAdd(a.out_u + (long long)p * M + row, 2.0f * (y * (float)r - pk));
            } else if (a.scal == SCAL_RANK) {
                e1 = a.uq[(long long)p * M + row] * (2.0f * (float)r - (float)N);
            } else if (a.scal == SCAL_PREFIX) {
                e1 = 2.0f * (r > 0 ? su0[r - 1] : 0.0f) - a.us_total[p];
            }
        }
        yrec[m] = make_uint4(__float_as_uint(e0), __float_as_uint(e1), row, (uint32_t)r);
        skey[m] = (uint32_t)r;                    // only this thread ever reads skey[m] above
    }
    if (tid == 0) yrec[M] = make_uint4(0u, 0u, 0u, 0xffffffffu);      // sentinel: a rank no key position has
    __syncthreads();
    for (int b = tid; b <= NBK; b += THREADS)
        mstart[b] = b == NBK ? (uint32_t)M : (uint32_t)lower_bound_u(skey, M, (uint32_t)(b * KB));
}

template <int THREADS, int E>
static cudaError_t launch_one(const SortArgs& a, cudaStream_t stream) {
    constexpr int CAP = THREADS * E;
    constexpr int W   = THREADS / 32;
    const size_t smem = (size_t)CAP * 4 * 2 + (size_t)W * 256 * 4 + 256 * 4 + 32 * 4 * 3 + (size_t)CAP * 2;
    auto kern = sort_rank_small<THREADS, E>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    kern<<<a.nseg, THREADS, smem, stream>>>(a);
    return cudaGetLastError();
}

// max(N, M) <= 16384
cudaError_t launch_sort_rank_small(const SortArgs& a, cudaStream_t stream) {
    const int mx = a.N > a.M ? a.N : a.M;
    if (mx <= 1024)  return launch_one<256, 4>(a, stream);
    if (mx <= 2048)  return launch_one<256, 8>(a, stream);
    if (mx <= 4096)  return launch_one<512, 8>(a, stream);
    if (mx <= 8192)  return launch_one<1024, 8>(a, stream);
    if (mx <= 16384) return launch_one<1024, 16>(a, stream);
    return cudaErrorInvalidValue;
}

}  // namespace qlka

// Sort/rank for segments longer than the shared-memory kernel holds (max(N, M) > 16384, up to
// 262144): the same walk records, produced by a few kernels that keep the segment in global
// memory (L2 resident per CTA) and stream it through shared memory a tile at a time.
//
//   seg_radix_pass   one CTA per segment, one launch per 8-bit digit: digit histogram of the whole
//                    segment, then tile by tile (16384 elements) the stable in-tile ranking of the
//                    shared-memory sort, a tile-local reorder in shared memory, and run-wise coalesced
//                    writes to the segment's output buffer at the running digit offsets.
//   key_scalars      per segment: sorted key values, permutation, per-key decays / key values and the
//                    scalar scans (unit column or prefix of a per-key scalar), tile by tile with a
//                    carried state.
//   rank_records     per sorted query: rank by binary search in the sorted keys, the record, the
//                    scalar side channel; then the per-block query starts.
//
// The reference covers these sizes with cub::DeviceSegmentedRadixSort (6-bit digits) for segments
// above 16384 (Weighted_Laplace_Sum/csrc/sort_utils.cu:62-81) and stops at 131072
// (Weighted_Laplace_Sum/csrc/binding.cpp:78); this path goes on to 262144.
#include "qlka_common.cuh"

namespace qlka {

constexpr int LT = 1024;            // threads
constexpr int LE = 16;              // elements per thread and tile
constexpr int LTILE = LT * LE;      // 16384
constexpr int LW = LT / 32;

__host__ __device__ inline long long large_pad(int n) { return ((long long)n + LTILE - 1) / LTILE * LTILE; }

// One 8-bit pass over every segment. pass 0 reads the float source (and creates the index payload),
// later passes read the previous pass's buffers.
__global__ void __launch_bounds__(LT, 1) seg_radix_pass(
    const float* __restrict__ src, const uint32_t* __restrict__ kin, const uint32_t* __restrict__ iin,
    uint32_t* __restrict__ kout, uint32_t* __restrict__ iout, const int n, const int shift, const int first)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint32_t* skey = reinterpret_cast<uint32_t*>(smem_raw);      // [LTILE]
    uint32_t* sidx = skey + LTILE;                               // [LTILE]
    uint32_t* cnt  = sidx + LTILE;                               // [LW][256]
    uint32_t* base = cnt + LW * 256;                             // [256] tile-local digit starts
    uint32_t* gofs = base + 256;                                 // [256] running digit offsets in the segment
    uint32_t* tot  = gofs + 256;                                 // [256]
    uint32_t* wsum = tot + 256;                                  // [32]

    const int       tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t  lt  = (1u << lane) - 1u;
    const long long npd = large_pad(n);
    const long long seg = blockIdx.x;
    src  += seg * n;
    kin  += seg * npd; iin += seg * npd; kout += seg * npd; iout += seg * npd;
    uint32_t* mycnt = cnt + warp * 256;

    auto key_at = [&](long long pos) -> uint32_t {
        return first ? (pos < n ? f2key(src[pos]) : 0xffffffffu) : kin[pos];
    };

    // ---- digit histogram of the segment -> exclusive offsets
    if (tid < 256) gofs[tid] = 0;
    __syncthreads();
    for (long long pos = tid; pos < npd; pos += LT) atomicAdd(&gofs[(key_at(pos) >> shift) & 255u], 1u);
    __syncthreads();
    {
        uint32_t c = 0, incl = 0;
        if (tid < 256) {
            c = gofs[tid]; incl = c;
            #pragma unroll
            for (int off = 1; off < 32; off <<= 1) { uint32_t t = __shfl_up_sync(FULL, incl, off); if (lane >= off) incl += t; }
            if (lane == 31) wsum[warp] = incl;
        }
        __syncthreads();
        if (tid < 256) { uint32_t pre = 0; for (int w = 0; w < warp; w++) pre += wsum[w]; gofs[tid] = pre + incl - c; }
        __syncthreads();
    }

    // ---- tiles in order
    for (long long t0 = 0; t0 < npd; t0 += LTILE) {
        uint32_t key[LE], idx[LE], rk[LE];
        #pragma unroll
        for (int s = 0; s < LE; s++) {
            const long long pos = t0 + warp * 32 * LE + s * 32 + lane;
            key[s] = key_at(pos);
            idx[s] = first ? (uint32_t)pos : iin[pos];
        }
        for (int i = tid; i < LW * 256; i += LT) cnt[i] = 0;
        __syncthreads();
        #pragma unroll
        for (int s = 0; s < LE; s++) {
            const uint32_t d     = (key[s] >> shift) & 255u;
            uint32_t       peers = FULL;
            #pragma unroll
            for (int bit = 0; bit < 8; bit++) {
                const uint32_t vote = __ballot_sync(FULL, (d >> bit) & 1u);
                peers &= ((d >> bit) & 1u) ? vote : ~vote;
            }
            const int leader = __ffs(peers) - 1;
            uint32_t  old    = 0;
            if (lane == leader) { old = mycnt[d]; mycnt[d] = old + __popc(peers); }
            old   = __shfl_sync(FULL, old, leader);
            rk[s] = old + __popc(peers & lt);
            __syncwarp();
        }
        __syncthreads();
        uint32_t c = 0, incl = 0;
        if (tid < 256) {
            uint32_t run = 0;
            #pragma unroll 4
            for (int w = 0; w < LW; w++) { uint32_t x = cnt[w * 256 + tid]; cnt[w * 256 + tid] = run; run += x; }
            c = run; incl = run; tot[tid] = run;
            #pragma unroll
            for (int off = 1; off < 32; off <<= 1) { uint32_t t = __shfl_up_sync(FULL, incl, off); if (lane >= off) incl += t; }
            if (lane == 31) wsum[warp] = incl;
        }
        __syncthreads();
        if (tid < 256) { uint32_t pre = 0; for (int w = 0; w < warp; w++) pre += wsum[w]; base[tid] = pre + incl - c; }
        __syncthreads();
        #pragma unroll
        for (int s = 0; s < LE; s++) {
            const uint32_t d   = (key[s] >> shift) & 255u;
            const uint32_t dst = base[d] + mycnt[d] + rk[s];
            skey[dst] = key[s];
            sidx[dst] = idx[s];
        }
        __syncthreads();
        // tile order is now digit-major: element i of digit d goes to gofs[d] + (i - base[d]), runs are contiguous
        for (int i = tid; i < LTILE; i += LT) {
            const uint32_t k = skey[i], d = (k >> shift) & 255u;
            const uint32_t dst = gofs[d] + (uint32_t)i - base[d];
            kout[dst] = k;
            iout[dst] = sidx[i];
        }
        __syncthreads();
        if (tid < 256) gofs[tid] += tot[tid];
        __syncthreads();
    }
}

// Sorted keys of every segment -> xs (float, [seg][N]), xperm, xval and the scalar scans su0 / su1.
// One CTA per segment, tiles of LT * LE keys, each thread a contiguous run of LE keys within the tile.
__global__ void __launch_bounds__(LT, 1) key_scalars(
    const uint32_t* __restrict__ ksorted, const uint32_t* __restrict__ isorted, float* __restrict__ xs_all, const SortArgs a)
{
    __shared__ float wa[32], wb[32], carry[2];
    const int       tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int       N = a.N, NP = npad(N);
    const long long seg = blockIdx.x, npd = large_pad(N);
    const int       p = (int)(seg / a.D);
    ksorted += seg * npd; isorted += seg * npd;
    float*    xs    = xs_all + seg * N;
    uint32_t* xperm = a.xperm + seg * NP;
    float*    xval  = a.xval + seg * xstride(N);
    float*    su0   = a.su0 + seg * (N + 1);
    float*    su1   = a.su1 + seg * (N + 1);

    for (int j = tid; j < NP + KB; j += LT) {
        if (j < N) xs[j] = key2f(ksorted[j]);
        if (j < NP) xperm[j] = j < N ? isorted[j] : 0u;
    }
    __syncthreads();
    auto dec = [&](int j) -> float { return (j > 0 && j < N) ? decay_of(xs[j] - xs[j - 1]) : 0.0f; };
    if (a.mode != MODE_SGN)
        for (int j = tid; j < NP + KB; j += LT)
            xval[j] = a.mode == MODE_LAPLACE ? (j < N ? dec(j) : 1.0f) : (j < N ? xs[j] : 0.0f);
    if (a.scal != SCAL_UNIT && a.scal != SCAL_PREFIX && a.scal != SCAL_SIGNED) return;

    // x_j = A_j x_{j-1} + B_j over the segment, forward (into su0) and, for the Laplace unit column,
    // backward (into su1); a tile at a time with the state carried in shared memory
    const bool   lap = a.mode == MODE_LAPLACE;
    const float* us  = (a.scal == SCAL_PREFIX || (a.scal == SCAL_SIGNED && a.us)) ? a.us + (long long)p * N : nullptr;
    for (int dir = 0; dir < (lap ? 2 : 1); dir++) {
        if (tid == 0) carry[0] = 0.0f;
        __syncthreads();
        for (long long t0 = 0; t0 < N; t0 += LTILE) {
            // scan position i (0-based in scan order) <-> key j = i (forward) or N-1-i (backward)
            float A[LE], B[LE];
            float ca = 1.0f, cb = 0.0f;
            #pragma unroll
            for (int k = 0; k < LE; k++) {
                const long long i = t0 + (long long)tid * LE + k;
                const int       j = dir ? N - 1 - (int)i : (int)i;
                if (i < N) {
                    A[k] = lap ? (dir ? dec(j + 1) : dec(j)) : 1.0f;
                    B[k] = us ? us[isorted[j]] : (lap ? 1.0f : xs[j]);
                } else { A[k] = 1.0f; B[k] = 0.0f; }
                ca = A[k] * ca; cb = fmaf(A[k], cb, B[k]);
            }
            float ia = ca, ib = cb;
            #pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                float pa = __shfl_up_sync(FULL, ia, off), pb = __shfl_up_sync(FULL, ib, off);
                if (lane >= off) { ib = fmaf(ia, pb, ib); ia = ia * pa; }
            }
            if (lane == 31) { wa[warp] = ia; wb[warp] = ib; }
            __syncthreads();
            float pb = carry[0];
            for (int w = 0; w < warp; w++) pb = fmaf(wa[w], pb, wb[w]);
            float ea = __shfl_up_sync(FULL, ia, 1), eb = __shfl_up_sync(FULL, ib, 1);
            if (lane == 0) { ea = 1.0f; eb = 0.0f; }
            float x = fmaf(ea, pb, eb);
            #pragma unroll
            for (int k = 0; k < LE; k++) {
                const long long i = t0 + (long long)tid * LE + k;
                if (i < N) {
                    x = fmaf(A[k], x, B[k]);
                    const int j = dir ? N - 1 - (int)i : (int)i;
                    (dir ? su1 : su0)[j] = x;
                }
            }
            __syncthreads();
            if (tid == LT - 1) carry[0] = x;          // state after the tile's last position (padding positions are identity)
            __syncthreads();
        }
    }
}

__device__ __forceinline__ int lower_bound_g(const float* __restrict__ a, const int n, const float x) {
    int lo = 0, hi = n;
    while (lo < hi) { int mid = (lo + hi) >> 1; if (__ldg(a + mid) < x) lo = mid + 1; else hi = mid; }
    return lo;
}

// one thread per sorted query
__global__ void __launch_bounds__(256) rank_records(
    const uint32_t* __restrict__ ysorted, const uint32_t* __restrict__ yidx, const float* __restrict__ xs_all, const SortArgs a)
{
    const int       N = a.N, M = a.M;
    const long long seg = blockIdx.y, mpd = large_pad(M);
    const int       m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m > M) return;
    uint4* yrec = a.yrec + seg * (M + 1);
    if (m == M) { yrec[M] = make_uint4(0u, 0u, 0u, 0xffffffffu); return; }
    const int    p   = (int)(seg / a.D);
    const float* xs  = xs_all + seg * N;
    const float* su0 = a.su0 + seg * (N + 1);
    const float* su1 = a.su1 + seg * (N + 1);
    const float    y   = key2f(ysorted[seg * mpd + m]);
    const uint32_t row = yidx[seg * mpd + m];       // (folded queries are not supported on this path; the host refuses them)
    const int      r   = lower_bound_g(xs, N, y);
    float e0 = 0.0f, e1 = 0.0f;
    if (a.mode == MODE_LAPLACE) {
        e0 = r > 0 ? expf(-(y - xs[r - 1])) : 0.0f;
        e1 = r < N ? expf(-(xs[r] - y)) : 0.0f;
        if (a.scal == SCAL_UNIT)
            atomicAdd(a.out_u + (long long)p * M + row, (r > 0 ? e0 * su0[r - 1] : 0.0f) + (r < N ? e1 * su1[r] : 0.0f));
        else if (a.scal == SCAL_SIGNED)
            a.out_s[seg * M + row] = (a.uq ? a.uq[(long long)p * M + row] : 1.0f)
                                   * ((r < N ? e1 * su1[r] : 0.0f) - (r > 0 ? e0 * su0[r - 1] : 0.0f));
    } else {
        if (a.mode == MODE_ABS) { e0 = 2.0f * y; e1 = a.rows_coef ? -2.0f : 0.0f; }
        if (a.scal == SCAL_UNIT)        atomicAdd(a.out_u + (long long)p * M + row, 2.0f * (y * (float)r - (r > 0 ? su0[r - 1] : 0.0f)));
        else if (a.scal == SCAL_RANK)   e1 = a.uq[(long long)p * M + row] * (2.0f * (float)r - (float)N);
        else if (a.scal == SCAL_PREFIX) e1 = 2.0f * (r > 0 ? su0[r - 1] : 0.0f) - a.us_total[p];
    }
    yrec[m] = make_uint4(__float_as_uint(e0), __float_as_uint(e1), row, (uint32_t)r);
}

// mstart[b] = first record whose rank is >= b * KB
__global__ void __launch_bounds__(256) block_starts(const SortArgs a)
{
    const int       N = a.N, M = a.M, NBK = nblocks(N);
    const long long seg = blockIdx.y;
    const int       b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b > NBK) return;
    const uint4* yrec = a.yrec + seg * (M + 1);
    uint32_t*    ms   = a.mstart + seg * mstride(N);
    if (b == NBK) { ms[b] = (uint32_t)M; return; }
    const uint32_t want = (uint32_t)(b * KB);
    int lo = 0, hi = M;
    while (lo < hi) { int mid = (lo + hi) >> 1; if (__ldg(&yrec[mid].w) < want) lo = mid + 1; else hi = mid; }
    ms[b] = (uint32_t)lo;
}

// scratch beyond the records: two ping-pong (key, index) buffers of the padded longer length, and the sorted keys
size_t sort_rank_large_scratch_bytes(int nseg, int N, int M) {
    const long long mx = large_pad(N > M ? N : M);
    return (size_t)nseg * mx * 4 * sizeof(uint32_t) + (size_t)nseg * N * sizeof(float) + 1024;
}

cudaError_t launch_sort_rank_large(const SortArgs& a, void* scratch, cudaStream_t stream)
{
    const long long mx  = large_pad(a.N > a.M ? a.N : a.M);
    uint32_t* k0 = static_cast<uint32_t*>(scratch);
    uint32_t* i0 = k0 + (size_t)a.nseg * mx;
    uint32_t* k1 = i0 + (size_t)a.nseg * mx;
    uint32_t* i1 = k1 + (size_t)a.nseg * mx;
    float*    xs = reinterpret_cast<float*>(i1 + (size_t)a.nseg * mx);
    const size_t smem = (size_t)LTILE * 8 + (size_t)LW * 1024 + 256 * 4 * 3 + 32 * 4;
    cudaError_t e = cudaFuncSetAttribute(seg_radix_pass, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;

    auto sort = [&](const float* src, int n) {       // result in (k1, i1), segment stride large_pad(n)
        seg_radix_pass<<<a.nseg, LT, smem, stream>>>(src, nullptr, nullptr, k0, i0, n, 0, 1);
        seg_radix_pass<<<a.nseg, LT, smem, stream>>>(src, k0, i0, k1, i1, n, 8, 0);
        seg_radix_pass<<<a.nseg, LT, smem, stream>>>(src, k1, i1, k0, i0, n, 16, 0);
        seg_radix_pass<<<a.nseg, LT, smem, stream>>>(src, k0, i0, k1, i1, n, 24, 0);
    };
    sort(a.x, a.N);
    key_scalars<<<a.nseg, LT, 0, stream>>>(k1, i1, xs, a);
    sort(a.y, a.M);
    rank_records<<<dim3((a.M + 1 + 255) / 256, a.nseg), 256, 0, stream>>>(k1, i1, xs, a);
    block_starts<<<dim3((nblocks(a.N) + 1 + 255) / 256, a.nseg), 256, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace qlka

// Sort/rank for segments longer than the shared-memory kernel holds (max(N, M) > 16384, up to
// 262144): the same walk records, produced by a few kernels that keep the segment in global
// memory (L2 resident per CTA) and stream it through shared memory a tile at a time.
//
//   seg_radix_pass   one CTA per segment, one launch per 8-bit digit: digit histogram of the whole
//                    segment (all four counted by the first launch), then tile by tile (8192 elements) the
//                    stable in-tile ranking of the shared-memory sort, a tile-local reorder in shared memory,
//                    and run-wise coalesced writes to the segment's output buffer at the running digit offsets.
//   key_scalars      per segment: sorted key values, permutation, per-key decays / key values, the
//                    scalar scans (unit column or prefix of a per-key scalar), tile by tile with a
//                    carried state, and a bucket index over the sorted keys for the rank search.
//   rank_queries     per query (the queries are never sorted): rank by a bucket lookup and a short binary
//                    search in the sorted keys, one count into the segment's rank histogram.
//   scan_starts      per segment: exclusive scan of the rank histogram = first record position of every
//                    rank; every eighth entry is the block start table of the walk.
//   place_records    per query: position from an atomic cursor on its rank's entry, the scalar side channel
//                    (coalesced, it is indexed by the query), the record written at its position.
//
// The reference covers these sizes with cub::DeviceSegmentedRadixSort (6-bit digits) for segments
// above 16384 (Weighted_Laplace_Sum/csrc/sort_utils.cu:62-81) and stops at 131072
// (Weighted_Laplace_Sum/csrc/binding.cpp:78); this path goes on to 262144.
#include "qlka_common.cuh"

namespace qlka {

constexpr int LE = 16;              // elements per thread and tile
constexpr int LTILE = 1024 * LE;    // 16384: the segments' (key, index) buffers are padded to a multiple of this

__host__ __device__ inline long long large_pad(int n) { return ((long long)n + LTILE - 1) / LTILE * LTILE; }

// One 8-bit pass over every segment: one CTA per segment, two CTAs per SM (so that one ranks a tile while
// the other waits for its loads), tiles of RT * RE elements. The first pass reads the float source, creates
// the index payload and counts the digits of all four passes in one sweep (the digit histogram of a whole
// segment does not depend on the order of its elements); the later passes find their histogram in ghist.
// The in-tile ranking is the (lane mask, count) table of the shared-memory sort (sort_rank.cu).
constexpr int RT = 512, RE = 16, RTILE = RT * RE, RW = RT / 32;
static_assert(LTILE % RTILE == 0, "the padded segment length must be a whole number of radix tiles");
constexpr size_t RADIX_SMEM = (size_t)RTILE * 8 + (size_t)RW * 256 * 4 + 256 * 4 * 3 + 32 * 4;

__global__ void __launch_bounds__(RT, 2) seg_radix_pass(
    const float* __restrict__ src, const uint32_t* __restrict__ kin, const uint32_t* __restrict__ iin,
    uint32_t* __restrict__ kout, uint32_t* __restrict__ iout, uint32_t* __restrict__ ghist, const int n, const int pass)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint32_t* skey = reinterpret_cast<uint32_t*>(smem_raw);      // [RTILE]
    uint32_t* sidx = skey + RTILE;                               // [RTILE]
    uint32_t* cnt  = sidx + RTILE;                               // [RW][256]
    uint32_t* base = cnt + RW * 256;                             // [256] tile-local digit starts
    uint32_t* gofs = base + 256;                                 // [256] running digit offsets in the segment
    uint32_t* tot  = gofs + 256;                                 // [256]
    uint32_t* wsum = tot + 256;                                  // [32]
    uint2*    tab  = reinterpret_cast<uint2*>(skey);             // [RW][256] ranking table, idle whenever the tile buffers are in use

    const int       tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t  lt  = (1u << lane) - 1u;
    const long long npd = large_pad(n);
    const long long seg = blockIdx.x;
    const int       shift = 8 * pass;
    const bool      first = pass == 0;
    src  += seg * n;
    kin  += seg * npd; iin += seg * npd; kout += seg * npd; iout += seg * npd;
    ghist += seg * 768;
    uint32_t* mycnt = cnt + warp * 256;
    uint2*    mytab = tab + warp * 256;

    // ---- digit histogram of the segment -> exclusive offsets
    if (first) {
        // digits 1 and 2 into 256 counters each; the top digit (sign and exponent: a handful of values) into eight
        // copies indexed by the lane, so that the lanes of a warp seldom add to one address
        uint32_t* h = skey;                                      // [256] [256] [8][256]
        if (tid < 256) gofs[tid] = 0;
        for (int i = tid; i < 2560; i += RT) h[i] = 0;
        __syncthreads();
        for (long long pos = tid; pos < npd; pos += RT) {
            const uint32_t k = pos < n ? f2key(src[pos]) : 0xffffffffu;
            atomicAdd(&gofs[k & 255u], 1u);
            atomicAdd(&h[(k >> 8) & 255u], 1u);
            atomicAdd(&h[256 + ((k >> 16) & 255u)], 1u);
            atomicAdd(&h[512 + (lane & 7) * 256 + (k >> 24)], 1u);
        }
        __syncthreads();
        for (int i = tid; i < 768; i += RT) {
            uint32_t c = h[i];
            if (i >= 512) for (int r = 1; r < 8; r++) c += h[i + r * 256];
            ghist[i] = c;
        }
    } else {
        if (tid < 256) gofs[tid] = ghist[(pass - 1) * 256 + tid];
    }
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
    for (long long t0 = 0; t0 < npd; t0 += RTILE) {
        uint32_t key[RE], idx[RE];
        #pragma unroll
        for (int s = 0; s < RE; s++) {
            const long long pos = t0 + warp * 32 * RE + s * 32 + lane;
            key[s] = first ? (pos < n ? f2key(src[pos]) : 0xffffffffu) : kin[pos];
            idx[s] = first ? (uint32_t)pos : iin[pos];
        }
        for (int i = tid; i < RW * 256; i += RT) tab[i] = make_uint2(0u, 0u);
        __syncthreads();
        #pragma unroll
        for (int s = 0; s < RE; s++) {
            uint2* slot = mytab + ((key[s] >> shift) & 255u);
            atomicOr(&slot->x, 1u << lane);
            __syncwarp();
            const uint2 mc = *slot;
            __syncwarp();
            if ((mc.x & lt) == 0u) *slot = make_uint2(0u, mc.y + __popc(mc.x));
            idx[s] |= (mc.y + __popc(mc.x & lt)) << 20;          // rank among the warp's equal digits (< 512) above the index (< 2^18)
            __syncwarp();
        }
        __syncthreads();
        uint32_t c = 0, incl = 0;
        if (tid < 256) {
            uint32_t run = 0;
            #pragma unroll 4
            for (int w = 0; w < RW; w++) { const uint32_t x = tab[w * 256 + tid].y; cnt[w * 256 + tid] = run; run += x; }
            c = run; incl = run; tot[tid] = run;
            #pragma unroll
            for (int off = 1; off < 32; off <<= 1) { uint32_t t = __shfl_up_sync(FULL, incl, off); if (lane >= off) incl += t; }
            if (lane == 31) wsum[warp] = incl;
        }
        __syncthreads();
        if (tid < 256) { uint32_t pre = 0; for (int w = 0; w < warp; w++) pre += wsum[w]; base[tid] = pre + incl - c; }
        __syncthreads();
        #pragma unroll
        for (int s = 0; s < RE; s++) {
            const uint32_t d   = (key[s] >> shift) & 255u;
            const uint32_t dst = base[d] + mycnt[d] + (idx[s] >> 20);
            skey[dst] = key[s];
            sidx[dst] = idx[s] & 0xfffffu;
        }
        __syncthreads();
        // tile order is now digit-major: element i of digit d goes to gofs[d] + (i - base[d]), runs are contiguous
        for (int i = tid; i < RTILE; i += RT) {
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
// One CTA per segment, tiles of ST * LE keys.
// Bucket index of the rank search: LNB(N) equal-width value buckets between the smallest and the largest key of a
// segment; bst[b] = number of keys in buckets below b, bst[LNB] = N. The bucket of a value is monotone in the value,
// so the rank of a query lies in [bst[b], bst[b + 1]] for its own bucket b.
__host__ __device__ inline int       large_nb(int n)      { return n / 4 + 1; }
__host__ __device__ inline long long large_bstride(int n) { return (long long)large_nb(n) + 3; }
struct BucketMap {
    float lo, scale; int nb;
    __device__ __forceinline__ BucketMap(const float smallest, const float largest, const int n) {
        lo = smallest; nb = large_nb(n);
        const float width = largest - smallest;
        scale = (width > 1e-30f && width < 1e30f) ? (float)nb / width : 0.0f;
    }
    __device__ __forceinline__ BucketMap(const float* __restrict__ xs, const int n) : BucketMap(__ldg(xs), __ldg(xs + n - 1), n) {}
    __device__ __forceinline__ int operator()(const float v) const { return (int)fminf(fmaxf((v - lo) * scale, 0.0f), (float)(nb - 1)); }
};

// The per-segment scan kernels (key_scalars, scan_starts) walk their segment tile by tile with a carried state, so a CTA has
// little in flight at any moment: 512 threads and two CTAs per SM, and the loads of a batch of iterations issued before its stores.
constexpr int ST = 512, STILE = ST * LE;

__global__ void __launch_bounds__(ST, 2) key_scalars(
    const uint32_t* __restrict__ ksorted, const uint32_t* __restrict__ isorted, float* __restrict__ xs_all,
    uint32_t* __restrict__ bst_all, const SortArgs a)
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

    // one sweep over the sorted keys: key values, permutation, per-key scalar (decay or key) and the bucket index, each key read
    // once together with its predecessor
    const bool lap = a.mode == MODE_LAPLACE;
    {
        const BucketMap bucket(key2f(ksorted[0]), key2f(ksorted[N - 1]), N);
        uint32_t* bst = bst_all + seg * large_bstride(N);
        constexpr int U = 4;
        for (int j0 = tid; j0 < NP + KB; j0 += ST * U) {
            uint32_t kj[U], kp[U], ij[U];
            #pragma unroll
            for (int u = 0; u < U; u++) {
                const int j = j0 + u * ST;
                kj[u] = j < N ? ksorted[j] : 0u;
                kp[u] = (j > 0 && j < N) ? ksorted[j - 1] : 0u;
                ij[u] = j < N ? isorted[j] : 0u;
            }
            #pragma unroll
            for (int u = 0; u < U; u++) {
                const int j = j0 + u * ST;
                if (j < N) {
                    const float x = key2f(kj[u]), xp = j > 0 ? key2f(kp[u]) : 0.0f;
                    xs[j] = x;
                    const int b = bucket(x), prev = j > 0 ? bucket(xp) : -1;
                    for (int t = prev + 1; t <= b; t++) bst[t] = (uint32_t)j;
                    if (j == N - 1) for (int t = b + 1; t <= bucket.nb; t++) bst[t] = (uint32_t)N;
                    if (a.mode != MODE_SGN) xval[j] = lap ? (j > 0 ? decay_of(x - xp) : 0.0f) : x;
                } else if (j < NP + KB && a.mode != MODE_SGN) {
                    xval[j] = lap ? 1.0f : 0.0f;
                }
                if (j < NP) xperm[j] = ij[u];
            }
        }
    }
    if (a.scal != SCAL_UNIT && a.scal != SCAL_PREFIX && a.scal != SCAL_SIGNED) return;
    __syncthreads();          // the scans read the decays back from xval instead of taking every exponential three times
    auto dec_at = [&](int j) -> float { return (j > 0 && j < N) ? xval[j] : 0.0f; };

    // x_j = A_j x_{j-1} + B_j over the segment, forward (into su0) and, for the Laplace unit column,
    // backward (into su1); a tile at a time with the state carried in shared memory
    const float* us  = (a.scal == SCAL_PREFIX || (a.scal == SCAL_SIGNED && a.us)) ? a.us + (long long)p * N : nullptr;
    // Every warp owns 32 * LE consecutive scan positions of the tile, lane l the positions k * 32 + l (so that each load
    // and store of a warp is one contiguous line); a row of 32 is scanned with shuffles, rows are chained through the
    // composite of the rows before, warps through shared memory, tiles through `carry`.
    for (int dir = 0; dir < (lap ? 2 : 1); dir++) {
        if (tid == 0) carry[0] = 0.0f;
        __syncthreads();
        float* dst = dir ? su1 : su0;
        for (long long t0 = 0; t0 < N; t0 += STILE) {
            // scan position i (0-based in scan order) <-> key j = i (forward) or N-1-i (backward)
            float ta[LE], tb[LE];                     // state at position (k, lane) = ta * (state entering the warp's chunk) + tb
            float ca = 1.0f, cb = 0.0f;               // the same for the end of the previous row
            const long long base = t0 + (long long)warp * 32 * LE;
            #pragma unroll
            for (int k = 0; k < LE; k++) {
                const long long i = base + k * 32 + lane;
                float ia = 1.0f, ib = 0.0f;
                if (i < N) {
                    const int j = dir ? N - 1 - (int)i : (int)i;
                    ia = lap ? (dir ? dec_at(j + 1) : dec_at(j)) : 1.0f;
                    ib = us ? us[isorted[j]] : (lap ? 1.0f : xs[j]);
                }
                #pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const float pa = __shfl_up_sync(FULL, ia, off), pb = __shfl_up_sync(FULL, ib, off);
                    if (lane >= off) { ib = fmaf(ia, pb, ib); ia = ia * pa; }
                }
                ta[k] = ia * ca;
                tb[k] = fmaf(ia, cb, ib);
                ca = __shfl_sync(FULL, ta[k], 31);
                cb = __shfl_sync(FULL, tb[k], 31);
            }
            if (lane == 0) { wa[warp] = ca; wb[warp] = cb; }
            __syncthreads();
            float x0 = carry[0];                       // state entering this warp's chunk
            for (int w = 0; w < warp; w++) x0 = fmaf(wa[w], x0, wb[w]);
            #pragma unroll
            for (int k = 0; k < LE; k++) {
                const long long i = base + k * 32 + lane;
                if (i < N) dst[dir ? N - 1 - (int)i : (int)i] = fmaf(ta[k], x0, tb[k]);
            }
            __syncthreads();
            if (tid == ST - 32) carry[0] = fmaf(ca, x0, cb);      // (lane 0 of the last warp) state after the tile; padding positions are identity
            __syncthreads();
        }
    }
}

// ---- queries: rank, count
__global__ void __launch_bounds__(256) rank_queries(
    const float* __restrict__ xs_all, const uint32_t* __restrict__ bst_all, uint32_t* __restrict__ rq_all,
    uint32_t* __restrict__ hist_all, const SortArgs a)
{
    const int       N = a.N, M = a.M;
    const unsigned  bps = (unsigned)(M + 1 + 255) / 256;       // blocks per segment (the segment index rides in blockIdx.x:
    const long long seg = blockIdx.x / bps;                    //  a grid's y extent stops at 65535)
    const int       m = (int)(blockIdx.x % bps) * 256 + threadIdx.x;
    if (m >= M) return;
    const float*    xs  = xs_all + seg * N;
    const uint32_t* bst = bst_all + seg * large_bstride(N);
    const BucketMap bucket(xs, N);
    const float y = a.y[seg * M + m];
    const int   b = bucket(y);
    int lo = (int)__ldg(bst + b), hi = (int)__ldg(bst + b + 1);
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (__ldg(xs + mid) < y) lo = mid + 1; else hi = mid; }
    rq_all[seg * M + m] = (uint32_t)lo;                         // number of keys strictly below the query
    atomicAdd(hist_all + seg * (N + 4) + lo, 1u);
}

// ---- exclusive scan of the rank histogram (N + 1 bins) in place; mstart[b] = start of rank b * KB
__global__ void __launch_bounds__(ST, 2) scan_starts(uint32_t* __restrict__ hist_all, const SortArgs a)
{
    __shared__ uint32_t wsum[32], carry;
    const int       tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int       N = a.N, NBK = nblocks(N);
    const long long seg = blockIdx.x;
    uint32_t* hist = hist_all + seg * (N + 4);
    uint32_t* ms   = a.mstart + seg * mstride(N);
    if (tid == 0) { carry = 0; ms[NBK] = (uint32_t)a.M; }
    __syncthreads();
    for (int t0 = 0; t0 <= N; t0 += ST * KB) {
        const int i0 = t0 + tid * KB;                           // a thread's run starts on a block boundary
        uint32_t c[KB], run = 0;
        #pragma unroll
        for (int k = 0; k < KB; k++) { c[k] = i0 + k <= N ? hist[i0 + k] : 0u; run += c[k]; }
        uint32_t incl = run;
        #pragma unroll
        for (int off = 1; off < 32; off <<= 1) { const uint32_t t = __shfl_up_sync(FULL, incl, off); if (lane >= off) incl += t; }
        if (lane == 31) wsum[warp] = incl;
        __syncthreads();
        uint32_t pre = carry + incl - run;
        for (int w = 0; w < warp; w++) pre += wsum[w];
        if (i0 <= N) ms[i0 / KB] = pre;                         // i0 / KB < NBK because i0 <= N
        #pragma unroll
        for (int k = 0; k < KB; k++) { if (i0 + k <= N) hist[i0 + k] = pre; pre += c[k]; }
        __syncthreads();
        if (tid == ST - 1) carry = pre;
        __syncthreads();
    }
}

// ---- records at their positions
__global__ void __launch_bounds__(256) place_records(
    const float* __restrict__ xs_all, const uint32_t* __restrict__ rq_all, uint32_t* __restrict__ hist_all, const SortArgs a)
{
    const int       N = a.N, M = a.M;
    const unsigned  bps = (unsigned)(M + 1 + 255) / 256;
    const long long seg = blockIdx.x / bps;
    const int       m = (int)(blockIdx.x % bps) * 256 + threadIdx.x;
    if (m > M) return;
    uint4* yrec = a.yrec + seg * (M + 1);
    if (m == M) { yrec[M] = make_uint4(0u, 0u, 0u, 0xffffffffu); return; }
    const int    p   = (int)(seg / a.D);
    const float* xs  = xs_all + seg * N;
    const float* su0 = a.su0 + seg * (N + 1);
    const float* su1 = a.su1 + seg * (N + 1);
    const float    y   = a.y[seg * M + m];                     // (folded queries are not supported on this path; the host refuses them)
    const int      r   = (int)rq_all[seg * M + m];
    const uint32_t pos = atomicAdd(hist_all + seg * (N + 4) + r, 1u);
    float e0 = 0.0f, e1 = 0.0f;
    if (a.mode == MODE_LAPLACE) {
        e0 = r > 0 ? __expf(-(y - __ldg(xs + r - 1))) : 0.0f;
        e1 = r < N ? __expf(-(__ldg(xs + r) - y)) : 0.0f;
        if (a.scal == SCAL_UNIT)
            atomicAdd(a.out_u + (long long)p * M + m, (r > 0 ? e0 * su0[r - 1] : 0.0f) + (r < N ? e1 * su1[r] : 0.0f));
        else if (a.scal == SCAL_SIGNED)
            a.out_s[seg * M + m] = (a.uq ? a.uq[(long long)p * M + m] : 1.0f)
                                 * ((r < N ? e1 * su1[r] : 0.0f) - (r > 0 ? e0 * su0[r - 1] : 0.0f));
    } else {
        if (a.mode == MODE_ABS) { e0 = 2.0f * y; e1 = a.rows_coef ? -2.0f : 0.0f; }
        if (a.scal == SCAL_UNIT)        atomicAdd(a.out_u + (long long)p * M + m, 2.0f * (y * (float)r - (r > 0 ? su0[r - 1] : 0.0f)));
        else if (a.scal == SCAL_RANK)   e1 = a.uq[(long long)p * M + m] * (2.0f * (float)r - (float)N);
        else if (a.scal == SCAL_PREFIX) e1 = 2.0f * (r > 0 ? su0[r - 1] : 0.0f) - a.us_total[p];
    }
    yrec[pos] = make_uint4(__float_as_uint(e0), __float_as_uint(e1), (uint32_t)m, (uint32_t)r);
}

// scratch beyond the records: two ping-pong (key, index) buffers of the padded key length, the sorted keys, the bucket
// index, the rank histogram and the rank of every query
size_t sort_rank_large_scratch_bytes(int nseg, int N, int M) {
    const long long np = large_pad(N);
    return (size_t)nseg * np * 4 * sizeof(uint32_t) + (size_t)nseg * N * sizeof(float)
         + (size_t)nseg * large_bstride(N) * sizeof(uint32_t) + (size_t)nseg * (N + 4) * sizeof(uint32_t)
         + (size_t)nseg * M * sizeof(uint32_t) + (size_t)nseg * 768 * sizeof(uint32_t) + 1024;
}

cudaError_t launch_sort_rank_large(const SortArgs& a, void* scratch, cudaStream_t stream)
{
    const long long np = large_pad(a.N);
    uint32_t* k0   = static_cast<uint32_t*>(scratch);
    uint32_t* i0   = k0 + (size_t)a.nseg * np;
    uint32_t* k1   = i0 + (size_t)a.nseg * np;
    uint32_t* i1   = k1 + (size_t)a.nseg * np;
    float*    xs   = reinterpret_cast<float*>(i1 + (size_t)a.nseg * np);
    uint32_t* bst  = reinterpret_cast<uint32_t*>(xs + (size_t)a.nseg * a.N);
    uint32_t* hist = bst + (size_t)a.nseg * large_bstride(a.N);
    uint32_t* rq   = hist + (size_t)a.nseg * (a.N + 4);
    uint32_t* gh   = rq + (size_t)a.nseg * a.M;                   // digit histograms of passes 1..3, written by pass 0
    const size_t smem = RADIX_SMEM;
    cudaError_t e = cudaFuncSetAttribute(seg_radix_pass, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(hist, 0, sizeof(uint32_t) * (size_t)a.nseg * (a.N + 4), stream);
    if (e != cudaSuccess) return e;

    // the keys: four 8-bit passes, result in (k1, i1), segment stride large_pad(N)
    seg_radix_pass<<<a.nseg, RT, smem, stream>>>(a.x, nullptr, nullptr, k0, i0, gh, a.N, 0);
    seg_radix_pass<<<a.nseg, RT, smem, stream>>>(a.x, k0, i0, k1, i1, gh, a.N, 1);
    seg_radix_pass<<<a.nseg, RT, smem, stream>>>(a.x, k1, i1, k0, i0, gh, a.N, 2);
    seg_radix_pass<<<a.nseg, RT, smem, stream>>>(a.x, k0, i0, k1, i1, gh, a.N, 3);
    key_scalars<<<a.nseg, ST, 0, stream>>>(k1, i1, xs, bst, a);
    // the queries: ranked where they are, ordered by rank with a counting sort
    const unsigned per_query = (unsigned)((a.M + 1 + 255) / 256) * (unsigned)a.nseg;
    rank_queries<<<per_query, 256, 0, stream>>>(xs, bst, rq, hist, a);
    scan_starts<<<a.nseg, ST, 0, stream>>>(hist, a);
    place_records<<<per_query, 256, 0, stream>>>(xs, rq, hist, a);
    return cudaGetLastError();
}

}  // namespace qlka

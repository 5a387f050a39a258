// Sort/rank kernel for segments of up to 16384 keys and queries: one CTA per segment sorts
// the keys in shared memory (by equal-width value buckets and a ranking inside each bucket,
// or, when the keys crowd into few buckets, with a stable LSD radix sort on 8-bit digits; keys
// carried with their 16-bit index), ranks every query among the keys (the queries are not
// sorted by value: the bucket starts as an index, a short binary search, then a counting sort
// by rank), and writes the walk records described in qlka_common.cuh.
//
// The reference does this step with two CUB segmented radix sorts through global memory
// (Weighted_Laplace_Sum/csrc/sort_utils.cu:23-81, Weighted_Abs_Sum/csrc/sort_utils.cu:18-75,
// called from sort_qk, Weighted_Laplace_Sum/csrc/binding.cpp:33-58) and searches the query
// ranges inside the walk kernels (laplace_kernels.cu:253-254, walk_common.cuh:23-30).
#include "qlka_common.cuh"

namespace qlka {

// Diagnostic build only (-DQLKA_PHASE_CLOCKS, see phase_clocks_main.cu): thread 0 of every CTA adds the cycles it spent
// between two marks to a global table, so that the kernel's phases can be weighed against each other.
#ifdef QLKA_PHASE_CLOCKS
__device__ unsigned long long g_phase_clocks[16];
#define PHASE_BEGIN() long long phase_t_ = clock64()
#define PHASE_MARK(i)                                                                                        \
    do {                                                                                                     \
        __syncthreads();                                                                                     \
        if (threadIdx.x == 0) { const long long t_ = clock64(); atomicAdd(&g_phase_clocks[i], (unsigned long long)(t_ - phase_t_)); phase_t_ = t_; } \
    } while (0)
#else
#define PHASE_BEGIN()
#define PHASE_MARK(i)
#endif

// ------------------------------------------------------------------ block radix sort
// Elements are held in registers, E per thread, in warp-blocked order: the element at
// array position warp*32*E + s*32 + lane sits in slot s of that lane. One pass ranks each
// element among equal digits of its own warp, step by step in array order so that the pass is
// stable, scans the per-warp digit counts digit-major, and scatters through shared memory.
// With E = 16 the ranking of a step goes through a per-warp table of (lane mask, count) pairs, one per
// digit: every lane ORs its bit into the mask of its digit, reads the pair back (the lanes that share
// the digit, and how many elements of the digit the warp saw in earlier steps), and the first of
// those lanes stores the pair back with the mask cleared and the count advanced. That is three
// shared-memory operations per step; eight ballots per step (the other way to find the lanes of
// equal digit) took 1.7 times as long there, and match.any longer still. The shorter segments
// (E < 16, several CTAs per SM) keep the ballots: the table would double their shared memory and
// cost them more in occupancy than the ranking gains (N = 600: 1.24 ms with ballots, 1.33 ms with the table).
// tab: W * 256 pairs (E = 16 only), any content on entry; cnt: W * 256 words.
template <int THREADS, int E>
__device__ __forceinline__ void block_radix_sort(
    uint32_t (&key)[E], uint32_t (&idx)[E],
    uint32_t* __restrict__ skey, uint16_t* __restrict__ sidx,
    uint32_t* __restrict__ cnt, uint32_t* __restrict__ base, uint32_t* __restrict__ wsum, uint2* __restrict__ tab)
{
    constexpr int W = THREADS / 32;
    const int      tid  = threadIdx.x;
    const int      warp = tid >> 5, lane = tid & 31;
    const uint32_t lt   = (1u << lane) - 1u;
    uint32_t*      mycnt = cnt + warp * 256;
    uint2*         mytab = tab + warp * 256;

    constexpr bool TABLE = E >= 16;
    if (TABLE) {
        for (int i = tid; i < W * 256; i += THREADS) tab[i] = make_uint2(0u, 0u);
        __syncthreads();
    }

    #pragma unroll 1
    for (int pass = 0; pass < 4; pass++) {
        const int shift = 8 * pass;
        if (TABLE) {
            #pragma unroll
            for (int s = 0; s < E; s++) {
                uint2* slot = mytab + ((key[s] >> shift) & 255u);
                atomicOr(&slot->x, 1u << lane);
                __syncwarp();
                const uint2 mc = *slot;
                __syncwarp();
                if ((mc.x & lt) == 0u) *slot = make_uint2(0u, mc.y + __popc(mc.x));
                idx[s] |= (mc.y + __popc(mc.x & lt)) << 16;      // rank among the warp's equal digits (< 32 E) rides on the index
                __syncwarp();
            }
        } else {
            for (int i = tid; i < W * 256; i += THREADS) cnt[i] = 0;
            __syncthreads();
            #pragma unroll
            for (int s0 = 0; s0 < E; s0 += 4) {
                // the peer masks of four steps first (independent votes), then their counter updates in order
                uint32_t peers[4];
                #pragma unroll
                for (int t = 0; t < 4; t++) peers[t] = FULL;
                #pragma unroll
                for (int bit = 0; bit < 8; bit++) {
                    #pragma unroll
                    for (int t = 0; t < 4; t++) {
                        const uint32_t b    = (key[s0 + t] >> (shift + bit)) & 1u;
                        const uint32_t vote = __ballot_sync(FULL, b);
                        peers[t] &= b ? vote : ~vote;
                    }
                }
                #pragma unroll
                for (int t = 0; t < 4; t++) {
                    const uint32_t d      = (key[s0 + t] >> shift) & 255u;
                    const int      leader = __ffs(peers[t]) - 1;
                    uint32_t       old    = 0;
                    if (lane == leader) { old = mycnt[d]; mycnt[d] = old + __popc(peers[t]); }
                    old         = __shfl_sync(FULL, old, leader);
                    idx[s0 + t] |= (old + __popc(peers[t] & lt)) << 16;
                    __syncwarp();
                }
            }
        }
        __syncthreads();

        // per digit: exclusive scan of the counts over warps (the table's counts go back to zero for the next
        // pass), then exclusive scan of the digit totals
        uint32_t tot = 0, incl = 0;
        if (tid < 256) {
            uint32_t run = 0;
            #pragma unroll 4
            for (int w = 0; w < W; w++) {
                uint32_t c;
                if (TABLE) { c = tab[w * 256 + tid].y; tab[w * 256 + tid].y = 0u; }
                else       { c = cnt[w * 256 + tid]; }
                cnt[w * 256 + tid] = run;
                run += c;
            }
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
        // fold the digit starts into the per-warp offsets (every thread's entries share one digit, THREADS being a
        // multiple of 256), so that the scatter below looks up one table, not two
        {
            const uint32_t bd = base[tid & 255];
            for (int i = tid; i < W * 256; i += THREADS) cnt[i] += bd;
        }
        __syncthreads();

        #pragma unroll
        for (int s = 0; s < E; s++) {
            const uint32_t d   = (key[s] >> shift) & 255u;
            const uint32_t dst = mycnt[d] + (idx[s] >> 16);
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

// ------------------------------------------------------------------ block scans
// x_j = A_j x_{j-1} + B_j, inclusive, x_{-1} = 0, over scan positions 0..n-1. Every thread owns
// the contiguous run [i0, i1) and passes the coefficients of its run in registers
// (for position i0 + k); on return the B array holds x at position i0 + k.
template <int THREADS, int E, bool REV, int OFF>
__device__ __forceinline__ void block_affine_scan(const int cnt, const float (&AA)[E + 1], float (&BX)[E],
                                                  float* __restrict__ wa, float* __restrict__ wb)
{
    // coefficient of run element k: A = AA[k + OFF]; BX holds B on entry and x on return
    // REV = false: positions ascend with k, thread and lane index. REV = true: the scan runs from the
    // last position to the first (k, lane and warp all descending); empty runs act as the identity.
    constexpr int W = THREADS / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float a = 1.0f, b = 0.0f;                     // composite of my run: x -> a x + b
    #pragma unroll
    for (int kk = 0; kk < E; kk++) {
        const int k = REV ? E - 1 - kk : kk;
        if (k < cnt) { a = AA[k + OFF] * a; b = fmaf(AA[k + OFF], b, BX[k]); }
    }
    float ia = a, ib = b;                         // inclusive over lanes, in scan order
    #pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        float pa = REV ? __shfl_down_sync(FULL, ia, off) : __shfl_up_sync(FULL, ia, off);
        float pb = REV ? __shfl_down_sync(FULL, ib, off) : __shfl_up_sync(FULL, ib, off);
        if (REV ? (lane + off < 32) : (lane >= off)) { ib = fmaf(ia, pb, ib); ia = ia * pa; }
    }
    __syncthreads();                              // wa/wb may still be read by a previous scan
    if (lane == (REV ? 0 : 31)) { wa[warp] = ia; wb[warp] = ib; }
    __syncthreads();
    float pb = 0.0f;                              // state entering my warp
    if (REV) { for (int w = W - 1; w > warp; w--) pb = fmaf(wa[w], pb, wb[w]); }
    else     { for (int w = 0; w < warp; w++)     pb = fmaf(wa[w], pb, wb[w]); }
    float ea = REV ? __shfl_down_sync(FULL, ia, 1) : __shfl_up_sync(FULL, ia, 1);
    float eb = REV ? __shfl_down_sync(FULL, ib, 1) : __shfl_up_sync(FULL, ib, 1);
    if (lane == (REV ? 31 : 0)) { ea = 1.0f; eb = 0.0f; }
    float x = fmaf(ea, pb, eb);                   // state entering my run
    #pragma unroll
    for (int kk = 0; kk < E; kk++) {
        const int k = REV ? E - 1 - kk : kk;
        if (k < cnt) { x = fmaf(AA[k + OFF], x, BX[k]); BX[k] = x; }
    }
}

// The same scan with the B terms read from and the results written to shared memory (position i0 + k of `src` / `dst`,
// which may be the same array): nothing but the coefficients stays in registers between the two sweeps over the run.
template <int THREADS, int E, bool REV, int OFF>
__device__ __forceinline__ void block_affine_scan_mem(const int cnt, const int i0, const float (&AA)[E + 1],
                                                      const float* __restrict__ src, float* __restrict__ dst,
                                                      float* __restrict__ wa, float* __restrict__ wb)
{
    constexpr int W = THREADS / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float a = 1.0f, b = 0.0f;
    #pragma unroll
    for (int kk = 0; kk < E; kk++) {
        const int k = REV ? E - 1 - kk : kk;
        if (k < cnt) { a = AA[k + OFF] * a; b = fmaf(AA[k + OFF], b, src[i0 + k]); }
    }
    float ia = a, ib = b;
    #pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        float pa = REV ? __shfl_down_sync(FULL, ia, off) : __shfl_up_sync(FULL, ia, off);
        float pb = REV ? __shfl_down_sync(FULL, ib, off) : __shfl_up_sync(FULL, ib, off);
        if (REV ? (lane + off < 32) : (lane >= off)) { ib = fmaf(ia, pb, ib); ia = ia * pa; }
    }
    __syncthreads();
    if (lane == (REV ? 0 : 31)) { wa[warp] = ia; wb[warp] = ib; }
    __syncthreads();
    float pb = 0.0f;
    if (REV) { for (int w = W - 1; w > warp; w--) pb = fmaf(wa[w], pb, wb[w]); }
    else     { for (int w = 0; w < warp; w++)     pb = fmaf(wa[w], pb, wb[w]); }
    float ea = REV ? __shfl_down_sync(FULL, ia, 1) : __shfl_up_sync(FULL, ia, 1);
    float eb = REV ? __shfl_down_sync(FULL, ib, 1) : __shfl_up_sync(FULL, ib, 1);
    if (lane == (REV ? 31 : 0)) { ea = 1.0f; eb = 0.0f; }
    float x = fmaf(ea, pb, eb);
    #pragma unroll
    for (int kk = 0; kk < E; kk++) {
        const int k = REV ? E - 1 - kk : kk;
        if (k < cnt) { x = fmaf(AA[k + OFF], x, src[i0 + k]); dst[i0 + k] = x; }
    }
}

// in-place exclusive prefix sum of h[0..n) (n <= THREADS * (E + 1)); returns nothing, h[i] <- sum_{j<i} h[j]
template <int THREADS, int E>
__device__ __forceinline__ void block_exclusive_sum(uint32_t* __restrict__ h, const int n, uint32_t* __restrict__ wsum)
{
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int per = (n + THREADS - 1) / THREADS;          // <= E + 1
    const int i0  = min(n, tid * per), i1 = min(n, i0 + per);
    uint32_t run = 0;
    for (int i = i0; i < i1; i++) run += h[i];
    uint32_t incl = run;
    #pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        uint32_t t = __shfl_up_sync(FULL, incl, off);
        if (lane >= off) incl += t;
    }
    __syncthreads();
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    uint32_t pre = incl - run;
    for (int w = 0; w < warp; w++) pre += wsum[w];
    for (int i = i0; i < i1; i++) { uint32_t c = h[i]; h[i] = pre; pre += c; }
}

// The sorted keys sit in shared memory with a word of padding after every 32 and another after every
// 1024, so that probe positions that differ by any power of two fall into different banks: a binary search
// over a power-of-two array otherwise probes addresses that are multiples of a large power of two,
// i.e. one bank, in its first ten steps.
__device__ __forceinline__ int skew(const int i) { return i + (i >> 5) + (i >> 10); }

__device__ __forceinline__ int lower_bound_f(const float* __restrict__ a, const int n, const float x) {
    int lo = 0, hi = n;
    while (lo < hi) { int mid = (lo + hi) >> 1; if (a[skew(mid)] < x) lo = mid + 1; else hi = mid; }
    return lo;
}

// ------------------------------------------------------------------ the kernel
// Phases: (1) sort of the keys (value buckets, or the radix sort above); (2) per-key decays and the scalar scans, each thread on a
// contiguous run of keys with the decays in registers; (3) the queries are not sorted by value:
// each is ranked against the sorted keys by binary search and the records are ordered by rank
// with a counting sort (shared-memory histogram over the N + 1 ranks, exclusive scan, atomic
// cursor), which also yields mstart for free; the records are then built in position order. Queries of
// equal rank come out in arbitrary order,
// which the walk does not care about.
// The kernel is compiled in four variants, so that each carries only the code of its own case (the whole kernel
// runs once per segment, straight through: instruction fetch is its most frequent stall, and dead branches cost):
//   VAR_LAP         Laplace records, optional unit-column side channel
//   VAR_LAP_SIGNED  Laplace records with the SCAL_SIGNED side channel (its scans run through shared memory)
//   VAR_ABS         abs / sgn records, the queries as given
//   VAR_ABS_FOLD    abs records over folded (shifted, weighted) query copies
enum SortVariant : int { VAR_LAP = 0, VAR_LAP_SIGNED = 1, VAR_ABS = 2, VAR_ABS_FOLD = 3 };

// Value buckets per segment (see phase (1) of the kernel): the more, the shorter the in-bucket ranking and the rank search.
// The 1024-thread kernel has its SM to itself and takes what its shared memory still holds (just under one bucket per
// element); the smaller ones stay at half their capacity, which keeps four CTAs on an SM.
__host__ __device__ constexpr int sort_buckets(int threads, int e) {
    return threads == 1024 ? threads * e - threads * e / 32 : threads * e / 2;
}

template <int THREADS, int E, int VAR>
__global__ void __launch_bounds__(THREADS, 1024 / THREADS) sort_rank_small(const SortArgs a)
{
    constexpr bool LAP = VAR == VAR_LAP || VAR == VAR_LAP_SIGNED, SIGNED = VAR == VAR_LAP_SIGNED, FOLD = VAR == VAR_ABS_FOLD;
    constexpr int CAP = THREADS * E;
    constexpr int W   = THREADS / 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint32_t* skey = reinterpret_cast<uint32_t*>(smem_raw);        // sort buffer, later the rank histogram (CAP + 1 + pad)
    float*    xs   = reinterpret_cast<float*>(skey + CAP + 32);    // sorted keys
    uint32_t* base = reinterpret_cast<uint32_t*>(xs + CAP + CAP / 32 + 32);
    uint32_t* wsum = base + 256;
    float*    wa   = reinterpret_cast<float*>(wsum + 32);
    float*    wb   = wa + 32;
    uint32_t* cnt  = reinterpret_cast<uint32_t*>(wb + 32);          // per-warp digit counters ...
    uint16_t* sidx = reinterpret_cast<uint16_t*>(cnt + W * 256);    // ... and the index payload; together >= 4 * CAP bytes
    float*    su0s = reinterpret_cast<float*>(cnt);                 // Laplace: forward unit scan, once both are idle
    uint16_t* bst  = sidx + CAP;                                    // bucket counters, then bucket starts: sort_buckets() + 1 entries (+ padding)
    uint2*    tab  = reinterpret_cast<uint2*>(xs);                  // (mask, count) table of the radix sort (E = 16), idle by the time xs is filled

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
    PHASE_BEGIN();
    // ---- (1) keys
    // NB equal-width value buckets between the smallest and the largest key; the bucket of a value is a monotone
    // function of it. They serve twice. Sorting: when no bucket holds more than RUN_LIMIT keys (any smooth
    // distribution), the keys are counted into their buckets, scattered to the buckets' ranges and ranked inside
    // their bucket by counting the smaller ones - one pass and a short loop per key instead of four radix passes;
    // otherwise (clustered keys, an outlier that stretches the range, infinities) the radix sort runs.
    // Rank search of phase (3): bst[b] = number of keys in buckets below b, so a query's rank lies in
    // [bst[b], bst[b + 1]] for its own bucket b and the binary search only covers that range.
    constexpr int      NB        = sort_buckets(THREADS, E);
    constexpr uint32_t RUN_LIMIT = 64;
    float blo, bsc;
    auto bucket = [&](const float val) -> int { return (int)fminf(fmaxf((val - blo) * bsc, 0.0f), (float)(NB - 1)); };
    bool by_radix;
    {
        uint32_t key[E], idx[E];
        load_segment<THREADS, E>(a.x + (long long)seg * N, N, key, idx);
        PHASE_MARK(0);
        const int warp = tid >> 5, lane = tid & 31;
        uint32_t* hw = reinterpret_cast<uint32_t*>(bst);           // the bucket counters: NB + 1 of 16 bits, two to a word
        {
            uint32_t kmin = 0xffffffffu, kmax = 0u;                // (the key order is the value order)
            #pragma unroll
            for (int s = 0; s < E; s++)
                if (warp * 32 * E + s * 32 + lane < N) { kmin = min(kmin, key[s]); kmax = max(kmax, key[s]); }
            #pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                kmin = min(kmin, __shfl_xor_sync(FULL, kmin, off));
                kmax = max(kmax, __shfl_xor_sync(FULL, kmax, off));
            }
            if (lane == 0) { base[warp] = kmin; base[32 + warp] = kmax; }
            for (int i = tid; i < NB / 2 + 1; i += THREADS) hw[i] = 0u;
            __syncthreads();
            kmin = lane < W ? base[lane] : 0xffffffffu;
            kmax = lane < W ? base[32 + lane] : 0u;
            #pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                kmin = min(kmin, __shfl_xor_sync(FULL, kmin, off));
                kmax = max(kmax, __shfl_xor_sync(FULL, kmax, off));
            }
            blo = key2f(kmin);
            const float bwd = key2f(kmax) - blo;
            bsc = (bwd > 1e-30f && bwd < 1e30f) ? (float)NB / bwd : 0.0f;
        }
        // count: the returned old value is the key's place among its bucket's keys (in arrival order)
        #pragma unroll
        for (int s = 0; s < E; s++) {
            if (warp * 32 * E + s * 32 + lane < N) {
                const uint32_t bk  = (uint32_t)bucket(key2f(key[s])), sh = (bk & 1u) * 16u;
                const uint32_t old = atomicAdd(&hw[bk >> 1], 1u << sh);            // (a bucket holds at most N <= 16384 keys: no carry)
                idx[s] = bk | (((old >> sh) & 0xffffu) << 16);
            }
        }
        __syncthreads();
        // bucket starts: exclusive scan of the NB + 1 counters in place (the last one counts nothing, so bst[NB] = N)
        {
            constexpr int PER = ((NB + 1 + THREADS - 1) / THREADS) | 1;      // odd: a thread's run of 16-bit counters starts in a bank of its own
            const int i0 = min(NB + 1, tid * PER), i1 = min(NB + 1, i0 + PER);
            uint32_t run = 0, big = 0;
            for (int i = i0; i < i1; i++) { const uint32_t c = bst[i]; run += c; big |= c > RUN_LIMIT; }
            uint32_t incl = run;
            #pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const uint32_t t = __shfl_up_sync(FULL, incl, off);
                if (lane >= off) incl += t;
            }
            if (lane == 31) wsum[warp] = incl;
            by_radix = __syncthreads_or((int)big) != 0;
            uint32_t pre = incl - run;
            for (int w = 0; w < warp; w++) pre += wsum[w];
            for (int i = i0; i < i1; i++) { const uint32_t c = bst[i]; bst[i] = (uint16_t)pre; pre += c; }
        }
        __syncthreads();
        if (!by_radix) {
            #pragma unroll
            for (int s = 0; s < E; s++) {
                const int pos = warp * 32 * E + s * 32 + lane;
                if (pos < N) {
                    const uint32_t dst = (uint32_t)bst[idx[s] & 0xffffu] + (idx[s] >> 16);
                    skey[dst] = key[s];
                    sidx[dst] = (uint16_t)pos;
                }
            }
            __syncthreads();
            // final place of the key at p: start of its bucket + the keys of the bucket that sort before it (equal keys in
            // the order of their original index, as the radix sort leaves them)
            uint16_t* sidx2 = reinterpret_cast<uint16_t*>(cnt);
            #pragma unroll 2
            for (int s = 0; s < E; s++) {
                const int pp = warp * 32 * E + s * 32 + lane;
                if (pp < N) {
                    const uint32_t k   = skey[pp], mine = sidx[pp];
                    const float    x   = key2f(k);
                    const int      bk  = bucket(x);
                    const int      lo  = bst[bk], hi = bst[bk + 1];
                    int            c   = 0;
                    for (int j = lo; j < hi; j++) {
                        const uint32_t kk = skey[j];
                        c += kk < k;
                        if (kk == k && j != pp) c += sidx[j] < mine;
                    }
                    xs[skew(lo + c)] = x;
                    sidx2[lo + c]    = (uint16_t)mine;
                }
            }
            __syncthreads();
            for (int j = tid; j < N; j += THREADS) sidx[j] = sidx2[j];
        } else {
            #pragma unroll
            for (int s = 0; s < E; s++) idx[s] = warp * 32 * E + s * 32 + lane;
            block_radix_sort<THREADS, E>(key, idx, skey, sidx, cnt, base, wsum, tab);
        }
    }
    PHASE_MARK(1);
    if (by_radix) {
        // sorted keys to floats; the bucket starts again, now from the sorted order: key j starts every bucket above its
        // predecessor's up to its own
        for (int j = tid; j < N; j += THREADS) {
            const float x = key2f(skey[j]);
            xs[skew(j)] = x;
            const int b = bucket(x), bp = j > 0 ? bucket(key2f(skey[j - 1])) : -1;
            for (int t = bp + 1; t <= b; t++) bst[t] = (uint16_t)j;
        }
        for (int t = bucket(key2f(skey[N - 1])) + 1 + tid; t <= NB; t += THREADS) bst[t] = (uint16_t)N;
    }
    __syncthreads();
    for (int j = tid; j < NP; j += THREADS) xperm[j] = j < N ? (uint32_t)sidx[j] : 0u;
    __syncthreads();
    PHASE_MARK(2);
    // ---- (2) per-key scalars; my run of keys is [i0, i0 + cntk). The run length is odd so that the
    // strided shared-memory accesses below are bank-conflict free; results leave through a staging
    // buffer (the idle sort buffer) so that the global stores are coalesced.
    {
        constexpr int R = E + 1;                                  // run capacity
        const int per = ((N + THREADS - 1) / THREADS) | 1;        // <= R
        const int i0  = min(N, tid * per), cntk = min(N, i0 + per) - i0;
        float*    stage = reinterpret_cast<float*>(skey);
        auto flush = [&](const float (&val)[R], float* __restrict__ dst) {
            __syncthreads();
            #pragma unroll
            for (int k = 0; k < R; k++) if (k < cntk) stage[i0 + k] = val[k];
            __syncthreads();
            for (int j = tid; j < N; j += THREADS) dst[j] = stage[j];
        };
        float dk[R + 1];                                          // dk[k] = decay a_{i0+k} = exp(-(k_j - k_{j-1})), a_0 = 0, a_N = 0
        if (LAP) {
            // the step decays in key order: to xval (coalesced) and to the staging buffer, from where every thread
            // picks up the R + 1 of its run (a rolled loop: the exponential is a long instruction sequence)
            #pragma unroll 2
            for (int j = tid; j < N; j += THREADS) {
                const float d = j > 0 ? decay_of(xs[skew(j)] - xs[skew(j - 1)]) : 0.0f;
                stage[j] = d;
                xval[j]  = d;
            }
            for (int j = N + tid; j < NP + KB; j += THREADS) xval[j] = 1.0f;
            __syncthreads();
            #pragma unroll
            for (int k = 0; k <= R; k++) {
                const int j = i0 + k;
                dk[k] = (k <= cntk && j < N) ? stage[j] : 0.0f;
            }
            float bx[R];
            if (SIGNED && a.scal == SCAL_SIGNED) {
                // su0[j] = sum_{i<=j} exp(-(k_j - k_i)) u_i,  su1[j] = sum_{i>=j} exp(-(k_i - k_j)) u_i with u the per-key scalar
                // (all ones without one). The scalars wait in the staging buffer, every thread touching only its own run,
                // because su0s overwrites the index payload; the backward scan runs in place there and leaves through it.
                {
                    const float* us = a.us ? a.us + (long long)p * N : nullptr;
                    __syncthreads();                  // every thread has picked its decays out of the staging buffer
                    #pragma unroll
                    for (int k = 0; k < R; k++) if (k < cntk) stage[i0 + k] = us ? us[sidx[i0 + k]] : 1.0f;
                }
                block_affine_scan_mem<THREADS, R, false, 0>(cntk, i0, dk, stage, su0s, wa, wb);
                block_affine_scan_mem<THREADS, R, true, 1>(cntk, i0, dk, stage, stage, wa, wb);
                __syncthreads();
                for (int j = tid; j < N; j += THREADS) su1[j] = stage[j];
            } else if (a.scal == SCAL_UNIT) {
                // su0[j] = sum_{i<=j} exp(-(k_j - k_i)),  su1[j] = sum_{i>=j} exp(-(k_i - k_j))
                #pragma unroll
                for (int k = 0; k < R; k++) bx[k] = 1.0f;
                block_affine_scan<THREADS, R, false, 0>(cntk, dk, bx, wa, wb);
                #pragma unroll
                for (int k = 0; k < R; k++) if (k < cntk) su0s[i0 + k] = bx[k];     // stays in shared memory
                // backward over the same runs: R_j = a_{j+1} R_{j+1} + 1
                #pragma unroll
                for (int k = 0; k < R; k++) bx[k] = 1.0f;
                block_affine_scan<THREADS, R, true, 1>(cntk, dk, bx, wa, wb);
                flush(bx, su1);
            }
        } else {
            if (a.mode == MODE_ABS)
                for (int j = tid; j < NP + KB; j += THREADS) xval[j] = j < N ? xs[skew(j)] : 0.0f;
            if (a.scal == SCAL_UNIT || a.scal == SCAL_PREFIX) {
                // su0[j] = sum_{i<=j} k_i   or   sum_{i<=j} us[row of key i]
                const float* us = a.scal == SCAL_PREFIX ? a.us + (long long)p * N : nullptr;
                float bx[R];
                #pragma unroll
                for (int k = 0; k <= R; k++) dk[k] = 1.0f;
                #pragma unroll
                for (int k = 0; k < R; k++) bx[k] = k < cntk ? (us ? us[sidx[i0 + k]] : xs[skew(i0 + k)]) : 0.0f;
                block_affine_scan<THREADS, R, false, 0>(cntk, dk, bx, wa, wb);
                flush(bx, su0);
            }
        }
    }
    __syncthreads();          // the su arrays are complete; skey becomes the rank histogram
    PHASE_MARK(3);
    // ---- (3) queries: rank, counting sort by rank, records
    uint32_t* hist = skey;                                         // N + 1 bins
    for (int i = tid; i <= N; i += THREADS) hist[i] = 0;
    __syncthreads();
    const int    MR   = FOLD ? a.fold : M;            // distinct query values (and output rows) per segment
    const float* ysrc = a.y + (long long)seg * MR;
    auto yval = [&](int m) -> float { return FOLD ? ysrc[m % MR] + a.shift[m / MR] : ysrc[m]; };
    uint32_t rp[E];                                   // rank, later rank | position << 16 (both <= 16384)
    // Slot s of a thread is query tid + ((s + rot) mod E) * THREADS with rot the segment index: the D segments of a head
    // run at the same time and all add into the same out_u row, and with a common visiting order their atomics would
    // queue up on the same sectors; the rotation spreads them over E different parts of the row.
    const int rot = seg & (E - 1);
    auto mq = [&](const int s) -> int { return tid + ((s + rot) & (E - 1)) * THREADS; };
    // QI searches in flight per thread (the probes are latency bound); the loop runs until the thread's longest is done
    constexpr int QI = E >= 8 ? 8 : 4;
    #pragma unroll
    for (int s0 = 0; s0 < E; s0 += QI) {
        int   lo[QI], hi[QI];
        float yq[QI];
        bool  open = false;
        #pragma unroll
        for (int t = 0; t < QI; t++) {
            const int m = mq(s0 + t);
            yq[t] = m < M ? yval(m) : 0.0f;
            const int b = bucket(yq[t]);
            lo[t] = bst[b]; hi[t] = bst[b + 1];
            open |= lo[t] < hi[t];
        }
        while (open) {
            open = false;
            #pragma unroll
            for (int t = 0; t < QI; t++) {
                if (lo[t] < hi[t]) {
                    const int mid = (lo[t] + hi[t]) >> 1;
                    if (xs[skew(mid)] < yq[t]) lo[t] = mid + 1; else hi[t] = mid;
                    open |= lo[t] < hi[t];
                }
            }
        }
        #pragma unroll
        for (int t = 0; t < QI; t++) rp[s0 + t] = (uint32_t)lo[t];       // number of keys strictly below the query
    }
    PHASE_MARK(4);
    #pragma unroll
    for (int s = 0; s < E; s++) if (mq(s) < M) atomicAdd(&hist[rp[s]], 1u);
    __syncthreads();
    block_exclusive_sum<THREADS, E>(hist, N + 1, wsum);
    __syncthreads();
    for (int b = tid; b <= NBK; b += THREADS) mstart[b] = b == NBK ? (uint32_t)M : hist[b * KB];     // b*KB <= N for b < NBK
    __syncthreads();
    #pragma unroll
    for (int s = 0; s < E; s++)
        if (mq(s) < M) rp[s] |= atomicAdd(&hist[rp[s]], 1u) << 16;       // final position of the record
    __syncthreads();
    PHASE_MARK(7);
    // The histogram is spent. Three steps from here, so that every access indexed by the query (its value, the
    // scalar side inputs, the out_u / out_s updates) is coalesced and every record leaves in position order as
    // full lines:
    //   A  each thread, for its own queries (rank and position in registers): the
    //      scalar side channel, whose atomics and stores are consecutive across the warp; the scan it looks up
    //      by rank that sits in scratch memory (su1 for Laplace, su0 otherwise) is first copied into the spent
    //      histogram's shared memory, because scattered 4-byte reads of global memory cost more than all the rest;
    //   B  the query's value and (index | rank << 16) go to shared memory at the record's position - the value into
    //      the forward-scan array, which step A was the last to read;
    //   C  in position order: weights from the two neighbouring keys, record written.
    constexpr bool lap = LAP;
    // e^{-gap} for the query weights: one ex2.approx (relative error ~ (2 + 1.2 gap) ulp; these weights enter each
    // output once, unlike the step decays, which multiply into every prefix state and are taken with expm1)
    auto wexp = [](const float gap) -> float { return __expf(-gap); };
    float yv[E];                                      // the thread's query values again, all loads in flight together
    #pragma unroll
    for (int s = 0; s < E; s++) {
        const int m = mq(s);
        yv[s] = m < M ? (FOLD ? __ldg(ysrc + m % MR) + a.shift[m / MR] : __ldg(ysrc + m)) : 0.0f;
    }
    if (a.scal == SCAL_UNIT || (SIGNED && a.scal == SCAL_SIGNED)) {
        float*       suq   = reinterpret_cast<float*>(skey);
        const float* susrc = lap ? su1 : su0;
        #pragma unroll 8
        for (int j = tid; j < N; j += THREADS) suq[j] = susrc[j];
        __syncthreads();
        #pragma unroll
        for (int s = 0; s < E; s++) {
            const int m = mq(s);
            if (m >= M) continue;
            const int   r   = (int)(rp[s] & 0xffffu);
            const float y   = yv[s];
            const int   row = FOLD ? m % MR : m;
            const float wq  = FOLD ? a.wgt[m / MR] : 1.0f;
            if (lap) {
                const float t0 = r > 0 ? wexp(y - xs[skew(r - 1)]) * su0s[r - 1] : 0.0f;
                const float t1 = r < N ? wexp(xs[skew(r)] - y) * suq[r] : 0.0f;
                if (a.scal == SCAL_UNIT) atomicAdd(a.out_u + (long long)p * MR + row, t0 + t1);
                else a.out_s[(long long)seg * M + m] = (a.uq ? a.uq[(long long)p * M + m] : 1.0f) * (t1 - t0);
            } else {
                atomicAdd(a.out_u + (long long)p * MR + row, wq * 2.0f * (y * (float)r - (r > 0 ? suq[r - 1] : 0.0f)));
            }
        }
    }
    __syncthreads();
    PHASE_MARK(8);
    uint32_t* who  = skey;
    float*    ypos = su0s;
    #pragma unroll
    for (int s = 0; s < E; s++) {
        const int m = mq(s);
        if (m < M) {
            const uint32_t pos = rp[s] >> 16;
            who[pos]  = (uint32_t)m | (rp[s] << 16);
            ypos[pos] = yv[s];
        }
    }
    __syncthreads();
    PHASE_MARK(5);
    #pragma unroll 4
    for (int pos = tid; pos < M; pos += THREADS) {
        const uint32_t w = who[pos];
        const int      m = (int)(w & 0xffffu), r = (int)(w >> 16);
        const float    y   = ypos[pos];
        const int      row = FOLD ? m % MR : m;
        const float    wq  = FOLD ? a.wgt[m / MR] : 1.0f;
        float e0 = 0.0f, e1 = 0.0f;
        if (lap) {
            e0 = r > 0 ? wexp(y - xs[skew(r - 1)]) : 0.0f;
            e1 = r < N ? wexp(xs[skew(r)] - y) : 0.0f;
        } else {
            if (a.mode == MODE_ABS) { e0 = 2.0f * y * wq; e1 = a.rows_coef ? -2.0f * wq : 0.0f; }      // row emission: e0 * PV + e1 * PK
            if (a.scal == SCAL_RANK)        e1 = a.uq[(long long)p * M + m] * (2.0f * (float)r - (float)N);
            else if (a.scal == SCAL_PREFIX) e1 = 2.0f * (r > 0 ? su0[r - 1] : 0.0f) - a.us_total[p];
        }
        yrec[pos] = make_uint4(__float_as_uint(e0), __float_as_uint(e1), (uint32_t)row, (uint32_t)r);
    }
    if (tid == 0) yrec[M] = make_uint4(0u, 0u, 0u, 0xffffffffu);      // sentinel: a rank no key position has
    PHASE_MARK(6);
}



template <int THREADS, int E, int VAR>
static cudaError_t launch_inst(const SortArgs& a, cudaStream_t stream) {
    constexpr int CAP = THREADS * E;
    constexpr int W   = THREADS / 32;
    const size_t smem = (size_t)CAP * 4 * 2 + 32 * 4 + (size_t)(CAP / 32 + 32) * 4 + (size_t)W * 256 * 4 + 256 * 4 + 32 * 4 * 3 + (size_t)CAP * 2
                      + (size_t)(sort_buckets(THREADS, E) + 8) * 2;
    auto kern = sort_rank_small<THREADS, E, VAR>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    kern<<<a.nseg, THREADS, smem, stream>>>(a);
    return cudaGetLastError();
}

template <int THREADS, int E>
static cudaError_t launch_one(const SortArgs& a, cudaStream_t stream) {
    if (a.mode == MODE_LAPLACE)
        return a.scal == SCAL_SIGNED ? launch_inst<THREADS, E, VAR_LAP_SIGNED>(a, stream) : launch_inst<THREADS, E, VAR_LAP>(a, stream);
    return a.fold ? launch_inst<THREADS, E, VAR_ABS_FOLD>(a, stream) : launch_inst<THREADS, E, VAR_ABS>(a, stream);
}

// max(N, M) <= 16384
cudaError_t launch_sort_rank_small(const SortArgs& a, cudaStream_t stream) {
    const int mx = a.N > a.M ? a.N : a.M;
    if (mx <= 1024)  return launch_one<256, 4>(a, stream);
    if (mx <= 2048)  return launch_one<256, 8>(a, stream);
    if (mx <= 4096)  return launch_one<256, 16>(a, stream);
    if (mx <= 8192)  return launch_one<512, 16>(a, stream);
    if (mx <= 16384) return launch_one<1024, 16>(a, stream);
    return cudaErrorInvalidValue;
}

}  // namespace qlka

// Shared definitions of the sorted-walk kernels (sm_100a).
//
// One "segment" is one (p = batch*head, d = feature dimension) pair: a stream of N sorted
// keys, each pointing at a row of C channels, and M queries that are merged into it.
// The sort/rank kernel turns a segment into four arrays ("walk records") in scratch
// memory; the walk kernels consume only those, never the raw keys:
//
//   xperm [seg][NP]        uint32  row index of the j-th smallest key (0 for j >= N)
//   xval  [seg][NP + KB]   float   per-key scalar: the step decay exp(-(k_j - k_{j-1}))
//                                  (Laplace, 0 for j = 0, 1 for j >= N) or the key value (abs)
//   yrec  [seg][M + 1]     uint4   per query in ascending order: {e0, e1, row, rank}, rank =
//                                  number of keys strictly below the query (ties count above);
//                                  entry M is a sentinel with rank 0xffffffff
//   mstart[seg][NBK + 1]   uint32  first query whose rank is >= b*KB, for every key block b
//
// with KB = 8 keys per block, NBK = N/KB + 1 blocks and NP = NBK*KB padded keys, so that at
// least one padded position follows the last key and every rank in [0, N] falls in a block.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace qlka {

constexpr int KB = 8;                       // keys per block of the walk
constexpr unsigned FULL = 0xffffffffu;

__host__ __device__ inline int       nblocks(int N)  { return N / KB + 1; }
__host__ __device__ inline int       npad(int N)     { return nblocks(N) * KB; }
__host__ __device__ inline long long xstride(int N)  { return (long long)npad(N) + KB; }
__host__ __device__ inline long long mstride(int N)  { return (long long)((nblocks(N) + 1 + 3) & ~3); }

enum SortMode : int { MODE_LAPLACE = 0, MODE_ABS = 1, MODE_SGN = 2 };
// scalar side channel of the sort/rank kernel
enum ScalMode : int {
    SCAL_NONE = 0,
    SCAL_UNIT = 1,      // accumulate the v == 1 column of the sum into out_u[p, row]
    SCAL_RANK = 2,      // e1 = uq[p, row] * (2 rank - N)
    SCAL_PREFIX = 3,    // e1 = 2 * (sum of us over keys below) - us_total[p]
    SCAL_SIGNED = 4     // Laplace: out_s[seg, row] = uq[p, row] * (e1 * R_r - e0 * L_{r-1}) with L, R the decayed prefix and
                        // suffix sums of the per-key scalar us[p, key row]; a null us or uq stands for all ones
};

struct SortArgs {
    const float* x;          // (P, D, N) keys to sort into the stream
    const float* y;          // (P, D, M) queries
    uint32_t*    xperm;
    float*       xval;
    uint4*       yrec;
    uint32_t*    mstart;
    float*       su0;        // [seg][N + 1] scratch for the scalar scans
    float*       su1;
    float*       out_u;      // (P, M)  SCAL_UNIT
    const float* uq;         // (P, M)  SCAL_RANK, SCAL_SIGNED
    const float* us;         // (P, N)  SCAL_PREFIX, SCAL_SIGNED
    const float* us_total;   // (P)     SCAL_PREFIX
    float*       out_s;      // (nseg, M)  SCAL_SIGNED
    int nseg, D, N, M, mode, scal;
    // folded queries (abs mode): the M queries are `M / fold` shifted copies of the `fold` values at y, copy s being
    // y + shift[s] with weight wgt[s]; records carry the weight and point at row m % fold. fold = 0: off.
    int   fold;
    float shift[4], wgt[4];
    int   rows_coef;          // abs mode: 1 = e1 is the key-sum coefficient -2 * weight of the row emission, 0 = e1 is a dot addend
};

struct WalkArgs {
    const float*    rows;     // (P, N, C4) rows the stream points at; C4 = channels padded to 4 (<= 64) or 8 floats
    const uint32_t* xperm;
    const float*    xval;
    const uint4*    yrec;
    const uint32_t* mstart;
    float*          ckpt;     // Laplace: [seg][NBK][C4] suffix checkpoints, written by the first pass
    float*          wck;      // Laplace: [seg][NBK]
    float*          agg;      // [seg * sps + stream][...] per-stream aggregates of the first pass (layout per walk)
    float*          out;      // emit rows: (P, M, C4), accumulated with vector reductions
    const float*    g;        // emit dot: (P, M, C4) matrix contracted with the walk state
    const float*    wtotal;   // emit dot, prefix walk: (P, C4) column sums of rows
    float*          out_s;    // emit dot: (P, D, M); plain stores in the prefix walk, added to in the Laplace walk
    float           sign;     // emit dot, prefix walk: output scale (+1 gradients, -1 public sgn op)
    int nseg, D, N, M, C4, sps, nitems;   // sps streams per segment, nitems work items of WALK_THREADS / LPS streams
    int Mrows;                // rows of `out` per p (= M unless the queries are folded)
};

__device__ __forceinline__ uint32_t f2key(float f) {
    uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key2f(uint32_t u) {
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

// exp(-gap) for gap >= 0, correctly rounded near 1: the step decays of dense keys are all within a few
// thousand ulps of 1 and thousands of them multiply into every prefix state, so their rounding error is
// what limits the accuracy of the Laplace recurrences; expf alone is off by up to 2 ulp there
__device__ __forceinline__ float decay_of(const float gap) {
    if (gap < 0.0625f) {
        // the usual case with thousands of keys: 1 - g + g^2/2 - ... - g^5/120 (the next term is below 1e-10 here); the
        // polynomial's own rounding is scaled by g, so the result is the exact value rounded once, to within 0.6 ulp
        float p = fmaf(gap, -1.0f / 120.0f, 1.0f / 24.0f);
        p = fmaf(gap, p, -1.0f / 6.0f);
        p = fmaf(gap, p, 0.5f);
        p = fmaf(gap, p, -1.0f);
        return fmaf(gap, p, 1.0f);
    }
    return gap < 0.5f ? 1.0f + expm1f(-gap) : expf(-gap);
}

// 16-byte vector reduction into global memory (no return value)
__device__ __forceinline__ void red_add4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                 :: "l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ float4 ldg4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

}  // namespace qlka

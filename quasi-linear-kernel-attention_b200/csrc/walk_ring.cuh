// Asynchronous row staging shared by the walk kernels.
//
// Every thread owns a private ring of DEPTH slots in shared memory; a slot holds the thread's
// CPL-channel slice of the KB rows of one key block. Rows are fetched with cp.async
// (global -> shared, no registers, L2 only) two blocks ahead of their use, one commit group
// per block, so the L2 latency of the row gather is hidden without extra warps. A thread only
// ever reads what it copied itself, so cp.async.wait_group is the only synchronisation the
// rows need. The per-key scalars of a block (9 floats) are staged once per stream by three of
// its lanes and read by all of them after a sub-warp barrier.
#pragma once
#include "qlka_common.cuh"

namespace qlka {

constexpr int WALK_THREADS = 256;
constexpr int RING_DEPTH   = 3;      // blocks in flight: the one in use and two prefetched
constexpr int SX_STRIDE    = 12;     // floats per staged scalar slot (9 used, 48 bytes)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

template <int CPL>
struct Vec {
    float x[CPL];
    __device__ __forceinline__ void zero() {
        #pragma unroll
        for (int c = 0; c < CPL; c++) x[c] = 0.0f;
    }
};

// address of this thread's float4 number h of row i in ring slot `slot`
template <int CPL>
__device__ __forceinline__ float4* ring_at(float4* ring, const int slot, const int i, const int h) {
    return ring + ((slot * KB + i) * (CPL / 4) + h) * WALK_THREADS + threadIdx.x;
}

// start the copies of key block b into ring slot `slot` and commit them as one group;
// pr = the block's eight row indices, tail = the block holds positions >= N (not copied)
template <int CPL>
__device__ __forceinline__ void ring_issue(float4* ring, float* sx_slot, const int slot, const int b,
                                           const uint4 p0, const uint4 p1, const float* __restrict__ rows,
                                           const float* __restrict__ xval, const int C4, const int N,
                                           const int ln, const bool stage_scalars)
{
    const int      j0    = b * KB;
    const uint32_t pr[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
    #pragma unroll
    for (int i = 0; i < KB; i++) {
        if (j0 + i < N) {
            const float* src = rows + (long long)pr[i] * C4;
            #pragma unroll
            for (int h = 0; h < CPL / 4; h++) cp_async16(ring_at<CPL>(ring, slot, i, h), src + 4 * h);
        }
    }
    if (stage_scalars) {
        if (ln == 0)      cp_async16(sx_slot, xval + j0);
        else if (ln == 1) cp_async16(sx_slot + 4, xval + j0 + 4);
        else if (ln == 2) cp_async4(sx_slot + 8, xval + j0 + 8);
    }
    cp_async_commit();
}

// this thread's slice of the block's rows, from its ring slot; rows at positions >= N read as zero
template <int CPL>
__device__ __forceinline__ void ring_read(float4* ring, const int slot, const int j0, const int N, Vec<CPL> (&v)[KB]) {
    #pragma unroll
    for (int i = 0; i < KB; i++) {
        #pragma unroll
        for (int h = 0; h < CPL / 4; h++) {
            const float4 t = *ring_at<CPL>(ring, slot, i, h);
            v[i].x[4 * h] = t.x; v[i].x[4 * h + 1] = t.y; v[i].x[4 * h + 2] = t.z; v[i].x[4 * h + 3] = t.w;
        }
    }
    if (j0 + KB > N) {
        #pragma unroll
        for (int i = 0; i < KB; i++) if (j0 + i >= N) v[i].zero();
    }
}

__device__ __forceinline__ void load_perm(const uint32_t* __restrict__ xperm, const int b, uint4& p0, uint4& p1) {
    p0 = __ldg(reinterpret_cast<const uint4*>(xperm + b * KB));
    p1 = __ldg(reinterpret_cast<const uint4*>(xperm + b * KB + 4));
}

}  // namespace qlka

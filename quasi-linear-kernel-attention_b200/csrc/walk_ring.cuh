// Asynchronous staging shared by the walk kernels.
//
// Every thread owns a private ring of RING_DEPTH slots in shared memory; a slot holds the
// thread's CPL-channel slice of the KB rows of one key block. Rows are fetched with cp.async
// (global -> shared, no registers, L2 only) two blocks ahead of their use, one commit group
// per block, so the L2 latency of the row gather is hidden without extra warps. A thread only
// ever reads the rows it copied itself, so cp.async.wait_group is all the rows need.
//
// Per stream (LPS lanes) and slot, two more things ride in the same commit group: the block's
// per-key scalars (9 floats, copied by lanes 0-2) and the first QCAP query records of the
// block (one 16-byte record per lane). Lane 3 adds the block's query range [m_lo, m_hi) with a
// plain store. These are read by all lanes of the stream after a sub-warp barrier, and a
// second sub-warp barrier after the reads lets the slot be refilled.
#pragma once
#include "qlka_common.cuh"

namespace qlka {

constexpr int WALK_THREADS = 256;
constexpr int RING_DEPTH   = 3;      // blocks in flight: the one in use and two prefetched
constexpr int SX_STRIDE    = 12;     // floats per staged scalar slot: 9 decays / keys, m_lo, m_hi

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

template <int CPL> __host__ __device__ constexpr int    ring_slot_f4()  { return KB * (CPL / 4) * WALK_THREADS; }
template <int CPL> __host__ __device__ constexpr size_t ring_bytes()    { return (size_t)RING_DEPTH * ring_slot_f4<CPL>() * sizeof(float4); }
// dynamic shared memory of a walk kernel: row ring | record slots | scalar slots
template <int LPS, int CPL> __host__ __device__ constexpr size_t walk_smem_bytes() {
    return ring_bytes<CPL>() + (size_t)(WALK_THREADS / LPS) * RING_DEPTH * LPS * sizeof(uint4)
         + (size_t)(WALK_THREADS / LPS) * RING_DEPTH * SX_STRIDE * sizeof(float);
}

// what one stream needs to stage its blocks
template <int LPS, int CPL>
struct Feeder {
    float4*         ring;      // + threadIdx.x
    uint4*          qs;        // this stream's record slots [RING_DEPTH][LPS]
    float*          sxs;       // this stream's scalar slots [RING_DEPTH][SX_STRIDE]
    const float*    rows;      // + p*N*C4 + lane channel offset
    const float*    xval;
    const uint32_t* xperm;
    const uint32_t* mstart;
    const uint4*    yrec;
    int             C4, N, ln;
    unsigned        gmask;
    bool            with_x, with_q;
    // prefetched one block before its issue
    uint4    p0, p1;
    uint32_t ms0, ms1;

    __device__ __forceinline__ void prefetch_index(const int b) {
        p0 = __ldg(reinterpret_cast<const uint4*>(xperm + b * KB));
        p1 = __ldg(reinterpret_cast<const uint4*>(xperm + b * KB + 4));
        if (with_q) { ms0 = __ldg(mstart + b); ms1 = __ldg(mstart + b + 1); }
    }

    // start the copies of key block b (whose indices were prefetched) into `slot`; one commit group
    __device__ __forceinline__ void issue(const int slot, const int b) {
        const int      j0    = b * KB;
        const uint32_t pr[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
        float4*        dst   = ring + slot * ring_slot_f4<CPL>();
        #pragma unroll
        for (int i = 0; i < KB; i++) {
            if (j0 + i < N) {
                const float* src = rows + (size_t)pr[i] * C4;
                #pragma unroll
                for (int h = 0; h < CPL / 4; h++) cp_async16(dst + (i * (CPL / 4) + h) * WALK_THREADS, src + 4 * h);
            }
        }
        float* sx = sxs + slot * SX_STRIDE;
        if (with_x) {
            if (ln == 0)      cp_async16(sx, xval + j0);
            else if (ln == 1) cp_async16(sx + 4, xval + j0 + 4);
            else if (ln == 2) cp_async4(sx + 8, xval + j0 + 8);
        }
        if (with_q) {
            if (ln == 3) { sx[9] = __uint_as_float(ms0); sx[10] = __uint_as_float(ms1); }
            const uint32_t n = min(ms1 - ms0, (uint32_t)LPS);
            if ((uint32_t)ln < n) cp_async16(qs + slot * LPS + ln, yrec + ms0 + ln);
        }
        cp_async_commit();
    }

    // this thread's slice of the block's rows from `slot`; rows at positions >= N read as zero
    __device__ __forceinline__ void read_rows(const int slot, const int j0, Vec<CPL> (&v)[KB]) const {
        const float4* src = ring + slot * ring_slot_f4<CPL>();
        #pragma unroll
        for (int i = 0; i < KB; i++) {
            #pragma unroll
            for (int h = 0; h < CPL / 4; h++) {
                const float4 t = src[(i * (CPL / 4) + h) * WALK_THREADS];
                v[i].x[4 * h] = t.x; v[i].x[4 * h + 1] = t.y; v[i].x[4 * h + 2] = t.z; v[i].x[4 * h + 3] = t.w;
            }
        }
        if (j0 + KB > N) {
            #pragma unroll
            for (int i = 0; i < KB; i++) if (j0 + i >= N) v[i].zero();
        }
    }
};

__device__ __forceinline__ int ring_next(const int cur) { return cur == RING_DEPTH - 1 ? 0 : cur + 1; }
__device__ __forceinline__ int ring_ahead2(const int cur) { return cur >= RING_DEPTH - 2 ? cur + 2 - RING_DEPTH : cur + 2; }

}  // namespace qlka

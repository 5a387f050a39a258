// Asynchronous staging shared by the walk kernels.
//
// Every thread owns a private ring of RING_DEPTH slots in shared memory; a slot holds the
// thread's CPL-channel slice of the KB rows of one key block. Rows are fetched with cp.async
// (global -> shared, no registers, L2 only) one block ahead of their use, one commit group
// per block, so the L2 latency of the row gather is hidden without extra warps. A thread only
// ever reads the rows it copied itself, so cp.async.wait_group is all the rows need.
//
// Per stream (LPS lanes) and slot, two more things ride in the same commit group: the block's
// per-key scalars (9 floats, copied by lanes 0-2) and up to LPS - 1 query records of the block
// (one 16-byte record per lane), closed by a sentinel record that a lane stores directly. Lane 3
// adds the block's query range [m_lo, m_hi). All of these are read by every lane of the stream
// after a sub-warp barrier; a sub-warp barrier at the top of the next iteration lets the slot
// be refilled. Shared memory is addressed with 32-bit shared-window addresses throughout.
#pragma once
#include "qlka_common.cuh"

namespace qlka {

#ifndef QLKA_WALK_THREADS
#define QLKA_WALK_THREADS 256
#endif
constexpr int WALK_THREADS = QLKA_WALK_THREADS;
#ifndef QLKA_RING_DEPTH
#define QLKA_RING_DEPTH 2
#endif
#ifndef QLKA_WALK_MIN_CTAS
#define QLKA_WALK_MIN_CTAS 2
#endif
constexpr int RING_DEPTH   = QLKA_RING_DEPTH;   // blocks in flight: the one in use and RING_DEPTH - 1 prefetched
constexpr int RING_AHEAD   = RING_DEPTH - 1;
constexpr int SX_STRIDE    = 12;     // floats per staged scalar slot: 8 decays / keys, the next one, pad, m_lo, m_hi

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(const uint32_t dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async4(const uint32_t dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

__device__ __forceinline__ float4 lds128(const uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128u(const uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128u(const uint32_t addr, const uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" :: "r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts64u(const uint32_t addr, const uint32_t a, const uint32_t b) {
    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" :: "r"(addr), "r"(a), "r"(b) : "memory");
}

template <int CPL>
struct Vec {
    float x[CPL];
    __device__ __forceinline__ void zero() {
        #pragma unroll
        for (int c = 0; c < CPL; c++) x[c] = 0.0f;
    }
};

template <int CPL> __host__ __device__ constexpr int    ring_slot_bytes() { return KB * (CPL / 4) * WALK_THREADS * 16; }
template <int CPL> __host__ __device__ constexpr size_t ring_bytes()      { return (size_t)RING_DEPTH * ring_slot_bytes<CPL>(); }
// dynamic shared memory of a walk kernel: row ring | record slots | scalar slots
template <int LPS, int CPL> __host__ __device__ constexpr size_t walk_smem_bytes() {
    return ring_bytes<CPL>() + (size_t)(WALK_THREADS / LPS) * RING_DEPTH * LPS * sizeof(uint4)
         + (size_t)(WALK_THREADS / LPS) * RING_DEPTH * SX_STRIDE * sizeof(float);
}

// what one stream needs to stage its blocks
template <int LPS, int CPL>
struct Feeder {
    uint32_t        ring_s;    // shared address of this thread's float4 in row 0 of slot 0
    uint32_t        qs_s;      // shared address of this stream's record slots [RING_DEPTH][LPS] x 16 B
    uint32_t        sx_s;      // shared address of this stream's scalar slots [RING_DEPTH][SX_STRIDE] x 4 B
    const float*    rows;      // + p*N*C4 + lane channel offset
    const float*    xval;
    const uint32_t* xperm;
    const uint32_t* mstart;
    const uint4*    yrec;
    uint32_t        row_bytes; // C4 * 4
    int             N, ln;
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
        const uint32_t dst   = ring_s + slot * ring_slot_bytes<CPL>();
        const char*    rb    = reinterpret_cast<const char*>(rows);
        if (j0 + KB <= N) {
            #pragma unroll
            for (int i = 0; i < KB; i++) {
                const char* src = rb + (size_t)pr[i] * row_bytes;
                #pragma unroll
                for (int h = 0; h < CPL / 4; h++) cp_async16(dst + (i * (CPL / 4) + h) * WALK_THREADS * 16, src + 16 * h);
            }
        } else {
            #pragma unroll
            for (int i = 0; i < KB; i++) {
                if (j0 + i < N) {
                    const char* src = rb + (size_t)pr[i] * row_bytes;
                    #pragma unroll
                    for (int h = 0; h < CPL / 4; h++) cp_async16(dst + (i * (CPL / 4) + h) * WALK_THREADS * 16, src + 16 * h);
                }
            }
        }
        const uint32_t sx = sx_s + slot * SX_STRIDE * 4;
        if (with_x) {
            if (ln == 0)      cp_async16(sx, xval + j0);
            else if (ln == 1) cp_async16(sx + 16, xval + j0 + 4);
            else if (ln == 2) cp_async4(sx + 32, xval + j0 + 8);
        }
        if (with_q) {
            // records 0 .. n-1 of the block, then a sentinel; n = min(count, LPS - 1)
            const uint32_t n = min(ms1 - ms0, (uint32_t)(LPS - 1));
            const uint32_t q = qs_s + (slot * LPS + ln) * 16;
            if ((uint32_t)ln < n)       cp_async16(q, yrec + ms0 + ln);
            else if ((uint32_t)ln == n) sts128u(q, make_uint4(0u, 0u, 0u, 0xffffffffu));
            if (ln == 3) sts64u(sx + 40, ms0, ms1);
        }
        cp_async_commit();
    }

    // Blocks are visited in steps t = 0 .. nblk-1, block of step t = bfirst + dir * t, slot of step t = t mod RING_DEPTH.
    // prologue: start the first RING_AHEAD blocks; step: start block t + RING_AHEAD, then wait for block t.
    __device__ __forceinline__ void prologue(const int bfirst, const int dir, const int nblk) {
        #pragma unroll
        for (int s = 0; s < RING_AHEAD; s++) {
            if (s < nblk) { prefetch_index(bfirst + dir * s); issue(s, bfirst + dir * s); }
            else cp_async_commit();
        }
        if (RING_AHEAD < nblk) prefetch_index(bfirst + dir * RING_AHEAD);
    }
    __device__ __forceinline__ void step(const int t, const int cur, const int bfirst, const int dir, const int nblk) {
        if (t + RING_AHEAD < nblk) issue(cur == 0 ? RING_DEPTH - 1 : cur - 1, bfirst + dir * (t + RING_AHEAD));
        else cp_async_commit();
        if (t + RING_AHEAD + 1 < nblk) prefetch_index(bfirst + dir * (t + RING_AHEAD + 1));
        cp_async_wait<RING_AHEAD>();
    }

    // this thread's slice of the block's rows from `slot`; rows at positions >= N read as zero
    __device__ __forceinline__ void read_rows(const int slot, const int j0, Vec<CPL> (&v)[KB]) const {
        const uint32_t src = ring_s + slot * ring_slot_bytes<CPL>();
        #pragma unroll
        for (int i = 0; i < KB; i++) {
            #pragma unroll
            for (int h = 0; h < CPL / 4; h++) {
                const float4 t = lds128(src + (i * (CPL / 4) + h) * WALK_THREADS * 16);
                v[i].x[4 * h] = t.x; v[i].x[4 * h + 1] = t.y; v[i].x[4 * h + 2] = t.z; v[i].x[4 * h + 3] = t.w;
            }
        }
        if (j0 + KB > N) {
            #pragma unroll
            for (int i = 0; i < KB; i++) if (j0 + i >= N) v[i].zero();
        }
    }

    // the block's nine scalars and its query range, from `slot`
    __device__ __forceinline__ void read_scalars(const int slot, float (&av)[KB + 1], uint32_t& m_lo, uint32_t& m_hi) const {
        const uint32_t sx = sx_s + slot * SX_STRIDE * 4;
        const float4 a0 = lds128(sx), a1 = lds128(sx + 16), a2 = lds128(sx + 32);
        av[0] = a0.x; av[1] = a0.y; av[2] = a0.z; av[3] = a0.w;
        av[4] = a1.x; av[5] = a1.y; av[6] = a1.z; av[7] = a1.w;
        av[8] = a2.x;
        m_lo = __float_as_uint(a2.z); m_hi = __float_as_uint(a2.w);
    }
};

__device__ __forceinline__ int ring_next(const int cur) { return cur == RING_DEPTH - 1 ? 0 : cur + 1; }

}  // namespace qlka

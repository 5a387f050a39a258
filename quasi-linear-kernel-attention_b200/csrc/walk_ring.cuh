// Asynchronous staging shared by the walk kernels.
//
// Every thread owns a private ring of RING_DEPTH slots in shared memory; a slot holds the
// thread's CPL-channel slice of the KB rows of one key block. Rows are fetched with cp.async
// (global -> shared, no registers, L2 only) one block ahead of their use, one commit group
// per block, so the L2 latency of the row gather is hidden without extra warps. A thread only
// ever reads the rows it copied itself, so cp.async.wait_group is all the rows need.
//
// Per stream (LPS lanes) and slot, two more things ride in the same commit group: the block's
// per-key scalars (12 floats of which 9 are used, copied by lanes 0-2) and the LPS query records
// from the block's first one on (one 16-byte record per lane; a block with fewer than LPS
// queries finds all of them there, followed by a record of a later block or the segment's
// sentinel). Both are read by every lane of the stream after a sub-warp barrier; a sub-warp
// barrier at the top of the next iteration lets the slot be refilled. The block's query range
// travels in registers. Shared memory is addressed with 32-bit shared-window addresses throughout.
//
// Walks that contract their state with a row of a second matrix per query (the dot emissions)
// need that row, whose index is only known once the query's record has arrived. Fetching it when
// the record is emitted puts one L2 round trip on every query of a stream; instead each thread
// copies its slice of the rows of up to G_SLOTS of the block's queries into a private third area
// as soon as the block's records are readable, and emits after the block's arithmetic.
//
// The dot of a query is a sum over the lanes of its stream. Warp shuffles inside the emission loop
// would split a warp that carries two or four streams (their loops have different trip counts) for good,
// so each lane parks its partial sum in shared memory - in the stream's part of the row slot in use,
// whose rows are in registers by then - and after the loop lane n adds up the partials of query n and
// writes the result: no shuffle, one writer per query, and the writes of a block go out together.
#pragma once
#include "qlka_common.cuh"

namespace qlka {

constexpr int WALK_THREADS  = 256;
constexpr int WALK_MIN_CTAS = 2;     // resident CTAs per SM the narrow (4 channels per lane) walks are compiled for
constexpr int RING_DEPTH    = 2;     // blocks in flight: the one in use and RING_DEPTH - 1 prefetched
constexpr int RING_AHEAD   = RING_DEPTH - 1;
constexpr int SX_STRIDE    = 12;     // floats per staged scalar slot: 8 decays / keys and the next four
constexpr int G_SLOTS      = 8;      // emit-side rows staged per batch (a power of two)

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
__device__ __forceinline__ uint32_t lds32u(const uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds32f(const uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts32f(const uint32_t addr, const float v) {
    asm volatile("st.shared.f32 [%0], %1;" :: "r"(addr), "f"(v) : "memory");
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

// d = a * b + c on two packed floats (one instruction on sm_100)
__device__ __forceinline__ void fma2(float& d0, float& d1, const float a0, const float a1, const float b0, const float b1,
                                     const float c0, const float c1) {
    asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
        "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void mul2(float& d0, float& d1, const float a0, const float a1, const float b0, const float b1) {
    asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "mul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

__device__ __forceinline__ void add2(float& d0, float& d1, const float a0, const float a1, const float b0, const float b1) {
    asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
        "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
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
// a first pass stages rows and per-key scalars only: row ring | scalar slots
template <int LPS, int CPL> __host__ __device__ constexpr size_t pass1_smem_bytes() {
    return ring_bytes<CPL>() + (size_t)(WALK_THREADS / LPS) * RING_DEPTH * SX_STRIDE * sizeof(float);
}
// the emit-side row area of the dot emissions follows: [G_SLOTS][CPL/4][WALK_THREADS] x 16 B
template <int CPL> __host__ __device__ constexpr size_t g_area_bytes() { return (size_t)G_SLOTS * (CPL / 4) * WALK_THREADS * 16; }

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
    int             N, M, ln;
    bool            with_x, with_q;
    uint32_t        g_s;       // dot emissions: shared address of this thread's float4 in emit-side slot 0
    const float*    grows;     //                + p*M*C4 + lane channel offset
    // prefetched one block before its issue
    uint4    p0, p1;
    uint32_t ms0, ms1;
    // query range [lo, hi) of the block in use and of the blocks in flight (all lanes load the same two words)
    uint32_t m_lo, m_hi, mq_lo[RING_AHEAD], mq_hi[RING_AHEAD];

    __device__ __forceinline__ void prefetch_index(const int b) {
        p0 = __ldg(reinterpret_cast<const uint4*>(xperm + b * KB));
        p1 = __ldg(reinterpret_cast<const uint4*>(xperm + b * KB + 4));
        if (with_q) { ms0 = __ldg(mstart + b); ms1 = __ldg(mstart + b + 1); }
    }

    // start the copies of key block b (whose indices were prefetched) into `slot`; one commit group
    __device__ __forceinline__ void issue(const int slot, const int b, const int ahead) {
        mq_lo[ahead] = ms0; mq_hi[ahead] = ms1;
        const int      j0    = b * KB;
        const uint32_t pr[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
        const uint32_t dst   = ring_s + slot * ring_slot_bytes<CPL>();
        const char*    rb    = reinterpret_cast<const char*>(rows);
        #pragma unroll
        for (int i = 0; i < KB; i++) {                 // (positions past the last key point at row 0; read_rows zeroes them)
            const char* src = rb + (size_t)pr[i] * row_bytes;
            #pragma unroll
            for (int h = 0; h < CPL / 4; h++) cp_async16(dst + (i * (CPL / 4) + h) * WALK_THREADS * 16, src + 16 * h);
        }
        const uint32_t sx = sx_s + slot * SX_STRIDE * 4;
        if (with_x && ln < 3) cp_async16(sx + 16 * ln, xval + j0 + 4 * ln);       // (the array is padded by KB floats)
        if (with_q) {
            // the LPS records from the block's first on (clamped to the segment's sentinel): a block with fewer than
            // LPS queries finds all of them here, followed by a record of a later block or the sentinel
            const uint32_t r = min(ms0 + (uint32_t)ln, (uint32_t)M);
            cp_async16(qs_s + (slot * LPS + ln) * 16, yrec + r);
        }
        cp_async_commit();
    }

    // Blocks are visited in steps t = 0 .. nblk-1, block of step t = bfirst + dir * t, slot of step t = t mod RING_DEPTH.
    // prologue: start the first RING_AHEAD blocks; step: start block t + RING_AHEAD, then wait for block t.
    __device__ __forceinline__ void prologue(const int bfirst, const int dir, const int nblk) {
        #pragma unroll
        for (int s = 0; s < RING_AHEAD; s++) {
            if (s < nblk) { prefetch_index(bfirst + dir * s); issue(s, bfirst + dir * s, s); }
            else cp_async_commit();
        }
        if (RING_AHEAD < nblk) prefetch_index(bfirst + dir * RING_AHEAD);
    }
    // first thing of every step: the oldest block in flight becomes the block in use
    __device__ __forceinline__ void advance_range() {
        m_lo = mq_lo[0]; m_hi = mq_hi[0];
        #pragma unroll
        for (int s = 0; s + 1 < RING_AHEAD; s++) { mq_lo[s] = mq_lo[s + 1]; mq_hi[s] = mq_hi[s + 1]; }
    }
    __device__ __forceinline__ void step_issue(const int t, const int cur, const int bfirst, const int dir, const int nblk) {
        if (t + RING_AHEAD < nblk) issue(cur == 0 ? RING_DEPTH - 1 : cur - 1, bfirst + dir * (t + RING_AHEAD), RING_AHEAD - 1);
        else cp_async_commit();
        if (t + RING_AHEAD + 1 < nblk) prefetch_index(bfirst + dir * (t + RING_AHEAD + 1));
    }
    __device__ __forceinline__ void step(const int t, const int cur, const int bfirst, const int dir, const int nblk) {
        advance_range();
        step_issue(t, cur, bfirst, dir, nblk);
        cp_async_wait<RING_AHEAD>();
    }

    // start the copies of this thread's slice of the emit-side rows of the staged records n0 .. n1-1 of `slot`
    // (n1 - n0 <= G_SLOTS; record n lands in emit-side slot n mod G_SLOTS); one commit group
    __device__ __forceinline__ void issue_g(const int slot, const uint32_t n0, const uint32_t n1) {
        const char* gb = reinterpret_cast<const char*>(grows);
        #pragma unroll
        for (int i = 0; i < G_SLOTS; i++) {
            const uint32_t n = n0 + i;
            if (n < n1) {
                const uint32_t row = lds32u(qs_s + (slot * LPS + n) * 16 + 8);
                const char*    src = gb + (size_t)row * row_bytes;
                #pragma unroll
                for (int h = 0; h < CPL / 4; h++)
                    cp_async16(g_s + ((n & (G_SLOTS - 1)) * (CPL / 4) + h) * WALK_THREADS * 16, src + 16 * h);
            }
        }
        cp_async_commit();
    }
    // Partial dots of query n of the block in `slot`: LPS floats inside the stream's share (LPS x 16 bytes) of row
    // (n mod 8) of the slot, at a word offset that puts the LPS lanes' reads of LPS different queries in different banks.
    __device__ __forceinline__ uint32_t part_addr(const int slot, const uint32_t n) const {
        return ring_s - ln * 16 + slot * ring_slot_bytes<CPL>() + (n & 7u) * (WALK_THREADS * 16) + ((n >> 3) * 32u + n) * 4u;
    }
    __device__ __forceinline__ void put_part(const int slot, const uint32_t n, const float acc) const {
        sts32f(part_addr(slot, n) + ln * 4, acc);
    }
    __device__ __forceinline__ float sum_parts(const int slot, const uint32_t n) const {
        const uint32_t p = part_addr(slot, n);
        float s0 = 0.0f, s1 = 0.0f;
        #pragma unroll
        for (int k = 0; k < LPS; k += 2) { s0 += lds32f(p + 4 * k); s1 += lds32f(p + 4 * k + 4); }
        return s0 + s1;
    }
    __device__ __forceinline__ void read_g(const uint32_t n, Vec<CPL>& gq) const {
        #pragma unroll
        for (int h = 0; h < CPL / 4; h++) {
            const float4 t = lds128(g_s + ((n & (G_SLOTS - 1)) * (CPL / 4) + h) * WALK_THREADS * 16);
            gq.x[4 * h] = t.x; gq.x[4 * h + 1] = t.y; gq.x[4 * h + 2] = t.z; gq.x[4 * h + 3] = t.w;
        }
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

    // the block's nine scalars, from `slot`
    __device__ __forceinline__ void read_scalars(const int slot, float (&av)[KB + 1]) const {
        const uint32_t sx = sx_s + slot * SX_STRIDE * 4;
        const float4 a0 = lds128(sx), a1 = lds128(sx + 16), a2 = lds128(sx + 32);
        av[0] = a0.x; av[1] = a0.y; av[2] = a0.z; av[3] = a0.w;
        av[4] = a1.x; av[5] = a1.y; av[6] = a1.z; av[7] = a1.w;
        av[8] = a2.x;
    }
};

// the key blocks [b0, b1) that stream s of the SPS streams of a segment owns (NBK blocks per segment)
__device__ __forceinline__ void stream_blocks(const int s, const int SPS, const int NBK, int& b0, int& b1) {
    b0 = (int)((long long)s * NBK / SPS);
    b1 = (int)((long long)(s + 1) * NBK / SPS);
}

__device__ __forceinline__ int ring_next(const int cur) { return cur == RING_DEPTH - 1 ? 0 : cur + 1; }

}  // namespace qlka

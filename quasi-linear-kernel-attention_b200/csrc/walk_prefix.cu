// Prefix walk: for every query m of every segment, with r its rank among the sorted keys,
// PV = sum of the rows of the r keys below it and PK = sum of key * row over the same keys:
//
//   EMIT_ROWS  out[p, row_m, :] += e0_m * PV + e1_m * PK       (vector reductions)
//              with e0 = 2 * query and e1 = -2 this is the walk term 2 (q PV - PK) of the abs sum; folded
//              queries (shifted, weighted copies that share a row) scale both by their weight
//              (Weighted_Abs_Sum/csrc/abs_kernels.cu:9-18; abs_chunk :78-199, abs_prefix :202-405)
//   EMIT_BOTH  both of the others over the same stream, rows and queries (grad_v and grad_k): one first pass and fold,
//              then the row emission and the dot emission as two second passes (one kernel doing both needs more than
//              the 128 registers that two resident CTAs leave a thread, and its spills cost more than the second walk)
//   EMIT_DOT   out_s[seg, row_m] = sign * ( <g[p, row_m, :], 2 PV - wtotal[p, :]> + e1_m )
//              the signed-rank walk behind grad_q, grad_k and the public sgn op
//              (Weighted_Abs_Sum/csrc/sgn_kernels.cu:8-15, sgn_prefix :17-192); one writer per
//              output element, plain stores.
//
// Same thread mapping and staging as the Laplace walk (LPS lanes per stream, CPL channels per
// lane, SPS independent streams per segment numbered over all segments, persistent CTAs, cp.async
// ring). The first launch sums each stream's rows into an aggregate table, a small kernel turns the
// table into exclusive prefix sums over each segment's streams, the last launch walks every stream
// forward from its incoming prefix and emits. With one stream per segment only the last one runs.
#include "walk_ring.cuh"

namespace qlka {

enum { EMIT_ROWS = 0, EMIT_DOT = 1, EMIT_BOTH = 2,       // BOTH (host level): row reductions and dots over the same stream and queries
       EMIT_ROWS_FIXED = 3 };                           // its row part: the key-sum coefficient is the constant -2, the record's e1 belongs to the dot

// floats per stream in the aggregate table: sum of the stream's rows | sum of key * row
__host__ __device__ inline int prefix_agg_stride(int C4) { return 2 * C4; }


// First launch (only with more than one stream per segment): every stream sums its rows (and key * row).
template <int LPS, int CPL, bool WITH_K>
__global__ void __launch_bounds__(WALK_THREADS, (CPL <= 4 ? 3 : 1)) prefix_pass1(const WalkArgs a)
{
    constexpr int STREAMS = WALK_THREADS / LPS;
    extern __shared__ __align__(16) float4 smem[];
    float4* ring   = smem;
    float*  sx_all = reinterpret_cast<float*>(reinterpret_cast<char*>(ring) + ring_bytes<CPL>());

    const int tid = threadIdx.x;
    const int st  = tid / LPS, ln = tid % LPS, c0 = ln * CPL;
    const int SPS = a.sps;
    const int N = a.N, C4 = a.C4;
    const int NBK = nblocks(N), NP = npad(N);
    const bool lane_on = c0 < C4;
    const int  c0l     = lane_on ? c0 : 0;
    const unsigned gmask = (LPS == 32) ? FULL : (((1u << LPS) - 1u) << ((tid & 31) & ~(LPS - 1)));
    const long long nstreams = (long long)a.nseg * SPS;

    Feeder<LPS, CPL> f;
    f.ring_s = smem_u32(ring + tid);
    f.qs_s   = 0;
    f.sx_s   = smem_u32(sx_all + st * RING_DEPTH * SX_STRIDE);
    f.row_bytes = (uint32_t)C4 * 4u; f.N = N; f.M = a.M; f.ln = ln; f.with_x = WITH_K; f.with_q = false;

    for (int item = blockIdx.x; item < a.nitems; item += gridDim.x) {
        const long long g  = (long long)item * STREAMS + st;
        const bool      on_s = g < nstreams;
        const long long gg = on_s ? g : 0;
        const int  sg = (int)(gg / SPS), s = (int)(gg - (long long)sg * SPS);
        const int  p  = sg / a.D;
        int b0, b1;
        stream_blocks(s, SPS, NBK, b0, b1);
        const int nblk = on_s ? b1 - b0 : 0;

        f.xperm = a.xperm + (long long)sg * NP;
        f.xval  = WITH_K ? a.xval + (long long)sg * xstride(N) : nullptr;
        f.rows  = a.rows + (long long)p * N * C4 + c0l;

        Vec<CPL> PV, PK;
        PV.zero(); PK.zero();
        __syncwarp(gmask);
        f.prologue(b0, 1, nblk);
        int cur = 0;
        for (int t = 0; t < nblk; t++) {
            const int b = b0 + t, j0 = b * KB;
            __syncwarp(gmask);
            f.step(t, cur, b0, 1, nblk);
            float kv[KB + 1];
            if (WITH_K) {
                __syncwarp(gmask);
                f.read_scalars(cur, kv);
            }
            Vec<CPL> v[KB];
            f.read_rows(cur, j0, v);
            #pragma unroll
            for (int i = 0; i < KB; i++) {
                #pragma unroll
                for (int c = 0; c < CPL; c += 2) {
                    add2(PV.x[c], PV.x[c + 1], PV.x[c], PV.x[c + 1], v[i].x[c], v[i].x[c + 1]);
                    if (WITH_K) fma2(PK.x[c], PK.x[c + 1], kv[i], kv[i], v[i].x[c], v[i].x[c + 1], PK.x[c], PK.x[c + 1]);
                }
            }
            cur = ring_next(cur);
        }
        cp_async_wait<0>();
        if (on_s && lane_on) {
            float* ag = a.agg + g * prefix_agg_stride(C4) + c0;
            #pragma unroll
            for (int c = 0; c < CPL; c += 4) {
                *reinterpret_cast<float4*>(ag + c) = make_float4(PV.x[c], PV.x[c + 1], PV.x[c + 2], PV.x[c + 3]);
                if (WITH_K) *reinterpret_cast<float4*>(ag + C4 + c) = make_float4(PK.x[c], PK.x[c + 1], PK.x[c + 2], PK.x[c + 3]);
            }
        }
    }
}

// Between the launches: per segment and channel, exclusive prefix sums of the stream aggregates, in place.
__global__ void __launch_bounds__(256) prefix_fold(float* __restrict__ agg, const int nseg, const int SPS, const int C4, const int with_k)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)nseg * C4) return;
    const int sg = (int)(i / C4), c = (int)(i - (long long)sg * C4);
    const int AGS = prefix_agg_stride(C4);
    float* ag = agg + (long long)sg * SPS * AGS;
    constexpr int CH = 16;                     // streams per chunk: their loads are issued together, then the serial part
    float pv = 0.0f, pk = 0.0f;
    for (int t0 = 0; t0 < SPS; t0 += CH) {
        float v[CH], k[CH];
        #pragma unroll
        for (int j = 0; j < CH; j++) {
            const float* at = ag + (long long)min(t0 + j, SPS - 1) * AGS;
            v[j] = at[c]; k[j] = with_k ? at[C4 + c] : 0.0f;
        }
        #pragma unroll
        for (int j = 0; j < CH; j++) {
            if (t0 + j < SPS) {
                float* at = ag + (long long)(t0 + j) * AGS;
                at[c] = pv; pv += v[j];
                if (with_k) { at[C4 + c] = pk; pk += k[j]; }
            }
        }
    }
}

// Last launch: the walk with emission, every stream starting from its incoming prefix sums.
template <int LPS, int CPL, int EMIT>
__global__ void __launch_bounds__(WALK_THREADS, (CPL <= 4 ? WALK_MIN_CTAS : 1)) prefix_pass2(const WalkArgs a)
{
    constexpr int  STREAMS = WALK_THREADS / LPS;
    constexpr bool WITH_K  = EMIT != EMIT_DOT;
    constexpr bool DO_ROWS = EMIT != EMIT_DOT, DO_DOT = EMIT == EMIT_DOT;
    extern __shared__ __align__(16) float4 smem[];
    float4* ring   = smem;
    uint4*  qs_all = reinterpret_cast<uint4*>(reinterpret_cast<char*>(ring) + ring_bytes<CPL>());
    float*  sx_all = reinterpret_cast<float*>(qs_all + STREAMS * RING_DEPTH * LPS);
    float4* g_area = reinterpret_cast<float4*>(sx_all + STREAMS * RING_DEPTH * SX_STRIDE);     // dot emissions only

    const int tid = threadIdx.x;
    const int st  = tid / LPS, ln = tid % LPS, c0 = ln * CPL;
    const int SPS = a.sps;
    const int N = a.N, M = a.M, C4 = a.C4;
    const int NBK = nblocks(N), NP = npad(N);
    const bool lane_on = c0 < C4;
    const int  c0l     = lane_on ? c0 : 0;
    const unsigned gmask = (LPS == 32) ? FULL : (((1u << LPS) - 1u) << ((tid & 31) & ~(LPS - 1)));
    const long long nstreams = (long long)a.nseg * SPS;
    const int AGS = prefix_agg_stride(C4);

    Feeder<LPS, CPL> f;
    f.ring_s = smem_u32(ring + tid);
    f.qs_s   = smem_u32(qs_all + st * RING_DEPTH * LPS);
    f.sx_s   = smem_u32(sx_all + st * RING_DEPTH * SX_STRIDE);
    f.row_bytes = (uint32_t)C4 * 4u; f.N = N; f.M = M; f.ln = ln; f.with_x = WITH_K; f.with_q = true;
    f.g_s = smem_u32(g_area + tid);

    // static round-robin over the work items (an atomic work counter was measured 10 % slower)
    for (int item = blockIdx.x; item < a.nitems; item += gridDim.x) {
        const long long g  = (long long)item * STREAMS + st;
        const bool      on_s = g < nstreams;
        const long long gg = on_s ? g : 0;
        const int  sg = (int)(gg / SPS), s = (int)(gg - (long long)sg * SPS);
        const int  p  = sg / a.D;
        const bool on = on_s && lane_on;
        int b0, b1;
        stream_blocks(s, SPS, NBK, b0, b1);
        const int nblk = on_s ? b1 - b0 : 0;

        f.xperm  = a.xperm + (long long)sg * NP;
        f.xval   = WITH_K ? a.xval + (long long)sg * xstride(N) : nullptr;
        f.rows   = a.rows + (long long)p * N * C4 + c0l;
        f.mstart = a.mstart + (long long)sg * mstride(N);
        f.yrec   = a.yrec + (long long)sg * (M + 1);

        Vec<CPL> PV, PK;
        PV.zero(); PK.zero();
        if (SPS > 1) {          // incoming prefix sums (prefix_fold left them in the aggregate table)
            const float* ag = a.agg + gg * AGS + c0l;
            #pragma unroll
            for (int c = 0; c < CPL; c += 4) {
                const float4 pv = ldg4(ag + c);
                PV.x[c] = pv.x; PV.x[c + 1] = pv.y; PV.x[c + 2] = pv.z; PV.x[c + 3] = pv.w;
                if (WITH_K) {
                    const float4 pk = ldg4(ag + C4 + c);
                    PK.x[c] = pk.x; PK.x[c + 1] = pk.y; PK.x[c + 2] = pk.z; PK.x[c + 3] = pk.w;
                }
            }
        }

        // emit-side constants
        Vec<CPL> wt;
        wt.zero();
        if (DO_DOT) {
            #pragma unroll
            for (int c = 0; c < CPL; c += 4) {
                const float4 t = ldg4(a.wtotal + (long long)p * C4 + c0l + c);
                wt.x[c] = t.x; wt.x[c + 1] = t.y; wt.x[c + 2] = t.z; wt.x[c + 3] = t.w;
            }
        }
        float*       out   = DO_ROWS ? a.out + (long long)p * a.Mrows * C4 + c0l : nullptr;
        const float* g_    = DO_DOT ? a.g + (long long)p * M * C4 + c0l : nullptr;
        float*       out_s = DO_DOT ? a.out_s + (long long)sg * M : nullptr;
        f.grows = g_;

        // ---------------- pass 2: forward with emission
        {
            __syncwarp(gmask);                         // every lane has left the previous item's slots
            f.prologue(b0, 1, nblk);
            int cur = 0;
            for (int t = 0; t < nblk; t++) {
                const int b = b0 + t, j0 = b * KB;
                float kv[KB + 1];
                uint32_t cnt;
                if (DO_DOT) {
                    // the block's copies have had a whole iteration; once its records are readable the emit-side rows
                    // of its first G_SLOTS queries start, ahead of the next block's copies, and land during the arithmetic
                    f.advance_range();
                    cp_async_wait<0>();
                    __syncwarp(gmask);
                    f.read_scalars(cur, kv);
                    cnt = f.m_hi - f.m_lo;
                    f.issue_g(cur, 0u, cnt < (uint32_t)LPS ? min(cnt, (uint32_t)G_SLOTS) : 0u);
                    f.step_issue(t, cur, b0, 1, nblk);
                } else {
                    __syncwarp(gmask);
                    f.step(t, cur, b0, 1, nblk);
                    __syncwarp(gmask);
                    f.read_scalars(cur, kv);      // (the key values are only staged and used by EMIT_ROWS)
                    cnt = f.m_hi - f.m_lo;
                }
                Vec<CPL> v[KB], kb[WITH_K ? KB : 1];
                f.read_rows(cur, j0, v);
                // prefix states before each key, in place of the rows
                #pragma unroll
                for (int i = 0; i < KB; i++) {
                    #pragma unroll
                    for (int c = 0; c < CPL; c += 2) {
                        const float t0 = v[i].x[c], t1 = v[i].x[c + 1];
                        v[i].x[c] = PV.x[c]; v[i].x[c + 1] = PV.x[c + 1];
                        add2(PV.x[c], PV.x[c + 1], PV.x[c], PV.x[c + 1], t0, t1);
                        if (WITH_K) {
                            kb[i].x[c] = PK.x[c]; kb[i].x[c + 1] = PK.x[c + 1];
                            fma2(PK.x[c], PK.x[c + 1], kv[i], kv[i], t0, t1, PK.x[c], PK.x[c + 1]);
                        }
                    }
                }
                auto load_g = [&](const uint4 rec, Vec<CPL>& gq) {      // the emit-side row slice of a record
                    const float* gr = g_ + (size_t)rec.z * C4;
                    #pragma unroll
                    for (int c = 0; c < CPL; c += 4) {
                        const float4 t4 = lane_on ? ldg4(gr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
                        gq.x[c] = t4.x; gq.x[c + 1] = t4.y; gq.x[c + 2] = t4.z; gq.x[c + 3] = t4.w;
                    }
                };
                auto emit_rows = [&](const uint4 rec, const Vec<CPL>& Pq, const Vec<CPL>& Kq) {
                    if (DO_ROWS) {
                        const float e0 = __uint_as_float(rec.x);
                        const float ek = EMIT == EMIT_ROWS ? __uint_as_float(rec.y) : -2.0f;     // (rec.y is the dot term's addend otherwise)
                        if (on) {
                            float* o = out + (size_t)rec.z * C4;
                            #pragma unroll
                            for (int c = 0; c < CPL; c += 4) {
                                float r0, r1, r2, r3;
                                mul2(r0, r1, ek, ek, Kq.x[c], Kq.x[c + 1]);
                                mul2(r2, r3, ek, ek, Kq.x[c + 2], Kq.x[c + 3]);
                                fma2(r0, r1, e0, e0, Pq.x[c], Pq.x[c + 1], r0, r1);
                                fma2(r2, r3, e0, e0, Pq.x[c + 2], Pq.x[c + 3], r2, r3);
                                red_add4(o + c, r0, r1, r2, r3);
                            }
                        }
                    }
                };
                auto dot_part = [&](const Vec<CPL>& Pq, const Vec<CPL>& gq) -> float {
                    float a0 = 0.0f, a1 = 0.0f;
                    #pragma unroll
                    for (int c = 0; c < CPL; c += 2) {
                        float t0, t1;
                        fma2(t0, t1, 2.0f, 2.0f, Pq.x[c], Pq.x[c + 1], -wt.x[c], -wt.x[c + 1]);
                        fma2(a0, a1, gq.x[c], gq.x[c + 1], t0, t1, a0, a1);
                    }
                    return a0 + a1;
                };
                if (DO_DOT) {
                    cp_async_wait<1>();               // the emit-side rows are in; the next block's copies may still fly
                    __syncwarp(gmask);                // every lane has its rows in registers: the slot may hold partial dots
                }
                if (cnt < (uint32_t)LPS) {
                    uint32_t qa  = f.qs_s + cur * LPS * 16;
                    uint4    rec = lds128u(qa);
                    uint32_t n = 0, nb = min(cnt, (uint32_t)G_SLOTS);      // records [0, nb) have their emit-side rows staged
                    #pragma unroll
                    for (int i = 0; i < KB; i++) {
                        while (rec.w == (uint32_t)(j0 + i)) {
                            qa += 16;
                            const uint4 nxt = lds128u(qa);
                            emit_rows(rec, v[i], kb[WITH_K ? i : 0]);
                            if (DO_DOT) {
                                if (n == nb) {                 // a block with more queries than slots: the next batch
                                    const uint32_t n1 = min(cnt, nb + (uint32_t)G_SLOTS);
                                    f.issue_g(cur, nb, n1);
                                    cp_async_wait<0>();
                                    nb = n1;
                                }
                                Vec<CPL> gq;
                                gq.zero();
                                if (lane_on) f.read_g(n, gq);
                                f.put_part(cur, n, dot_part(v[i], gq));
                            }
                            rec = nxt;
                            ++n;
                        }
                    }
                    if (DO_DOT) {
                        __syncwarp(gmask);
                        if ((uint32_t)ln < cnt) {             // lane n finishes query n of the block
                            const float sum = f.sum_parts(cur, (uint32_t)ln);
                            const uint4 r   = lds128u(f.qs_s + (cur * LPS + ln) * 16);
                            out_s[r.z] = a.sign * (sum + __uint_as_float(r.y));
                        }
                    }
                } else {
                    const uint4* yp  = f.yrec + f.m_lo;
                    uint32_t     n   = 0;
                    uint4        rec = __ldg(yp);
                    #pragma unroll
                    for (int i = 0; i < KB; i++) {
                        while (n < cnt && rec.w == (uint32_t)(j0 + i)) {
                            ++n;
                            const uint4 nxt = __ldg(yp + n);
                            emit_rows(rec, v[i], kb[WITH_K ? i : 0]);
                            if (DO_DOT) {
                                Vec<CPL> gq;
                                load_g(rec, gq);
                                float acc = dot_part(v[i], gq);
                                #pragma unroll
                                for (int off = LPS / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(gmask, acc, off);
                                if (ln == 0) out_s[rec.z] = a.sign * (acc + __uint_as_float(rec.y));
                            }
                            rec = nxt;
                        }
                    }
                }
                cur = ring_next(cur);
            }
        }
        cp_async_wait<0>();
    }
}

template <int LPS, int CPL, int EMIT>
static cudaError_t launch_pass2(const WalkArgs& a, int grid2, cudaStream_t stream) {
    auto k2 = prefix_pass2<LPS, CPL, EMIT>;
    const size_t smem2 = walk_smem_bytes<LPS, CPL>() + (EMIT == EMIT_DOT ? g_area_bytes<CPL>() : 0);
    cudaError_t e = cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    if (e != cudaSuccess) return e;
    k2<<<grid2, WALK_THREADS, smem2, stream>>>(a);
    return cudaGetLastError();
}

template <int LPS, int CPL>
static cudaError_t launch_pw(const WalkArgs& a, int emit, int grid1, int grid2, cudaStream_t stream) {
    if (a.sps > 1) {                                                   // (a lone stream per segment has nothing before it)
        const size_t smem1 = pass1_smem_bytes<LPS, CPL>();
        cudaError_t e;
        if (emit == EMIT_DOT) {
            auto k1 = prefix_pass1<LPS, CPL, false>;
            e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
            if (e != cudaSuccess) return e;
            k1<<<grid1, WALK_THREADS, smem1, stream>>>(a);
        } else {
            auto k1 = prefix_pass1<LPS, CPL, true>;
            e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
            if (e != cudaSuccess) return e;
            k1<<<grid1, WALK_THREADS, smem1, stream>>>(a);
        }
        prefix_fold<<<(unsigned)(((long long)a.nseg * a.C4 + 255) / 256), 256, 0, stream>>>(a.agg, a.nseg, a.sps, a.C4, emit == EMIT_DOT ? 0 : 1);
    }
    if (emit == EMIT_ROWS) return launch_pass2<LPS, CPL, EMIT_ROWS>(a, grid2, stream);
    if (emit == EMIT_DOT)  return launch_pass2<LPS, CPL, EMIT_DOT>(a, grid2, stream);
    cudaError_t e = launch_pass2<LPS, CPL, EMIT_ROWS_FIXED>(a, grid2, stream);       // EMIT_BOTH
    if (e != cudaSuccess) return e;
    return launch_pass2<LPS, CPL, EMIT_DOT>(a, grid2, stream);
}

int prefix_agg_stride_host(int C4) { return prefix_agg_stride(C4); }

// emit: EMIT_ROWS, EMIT_DOT or EMIT_BOTH; grid1 / grid2: CTAs of the first and of the emitting launches
cudaError_t launch_prefix_walk(const WalkArgs& a, int emit, int grid1, int grid2, cudaStream_t stream) {
    if (emit != EMIT_ROWS && emit != EMIT_DOT && emit != EMIT_BOTH) return cudaErrorInvalidValue;
    if (a.C4 <= 32)  return launch_pw<8, 4>(a, emit, grid1, grid2, stream);
    if (a.C4 <= 64)  return launch_pw<16, 4>(a, emit, grid1, grid2, stream);
    if (a.C4 <= 128) return launch_pw<16, 8>(a, emit, grid1, grid2, stream);
    return cudaErrorInvalidValue;
}

}  // namespace qlka

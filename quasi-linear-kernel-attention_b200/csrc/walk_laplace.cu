// Laplace walk: out[p, row_m, :] += e0_m * L_{r-1} + e1_m * R_r for every query m of every
// segment, where r is the query's rank, L the decayed prefix sum of the gathered rows and R
// the decayed suffix sum (recurrences of Weighted_Laplace_Sum/csrc/laplace_kernels.cu:5-13).
// Two more emissions serve the gradients of the sum, which the reference does not have (its
// training route is the chunked PyTorch path, Experiments/kernel_attention/attention.py:110-115):
//   LAP_DOT   out_s[seg, row_m] += <g[p, row_m, :], e1_m * R_r - e0_m * L_{r-1}>   (d/dquery of the sum,
//             contracted with the upstream gradient; one writer per element, added to the scalar
//             term that the sort/rank kernel stored there)
//   LAP_BOTH  the row reduction and the dot from one walk (grad_v and grad_k share stream and queries)
//
// Replaces the reference's laplace_chunk / laplace_scan / laplace_walk trio
// (laplace_kernels.cu:65-127, 134-188, 219-409) with two launches over independent work units:
//   * a "stream" is a contiguous run of key blocks of one segment; a segment is cut into SPS of them
//     (any number: the host picks it so that the persistent CTAs stay balanced) and the streams of all
//     segments are numbered consecutively. LPS lanes cooperate on one stream, each lane owning CPL
//     consecutive channels, so a row is one or two 16-byte copies per lane and a result is one or two
//     16-byte vector reductions; lanes never exchange rows. A CTA takes WALK_THREADS / LPS consecutive
//     streams per work item; nothing couples the streams of a CTA.
//   * rows, per-key decays and query records reach the lanes through the cp.async staging of
//     walk_ring.cuh, one block ahead of their use.
//   * laplace_pass1 walks every stream backwards once: the local suffix state at every block start goes
//     to the segment's checkpoint array, the stream's forward and backward aggregates and the decay
//     across it to the aggregate table.
//   * laplace_fold turns the aggregates of a segment's streams into the prefix state entering each stream
//     and the suffix state entering it from above (serial over the streams, parallel over channels).
//   * laplace_pass2 walks every stream forward from those states: per
//     block of 8 keys the suffix states are rebuilt in registers from the next checkpoint, the prefix
//     states overwrite the row registers, and the block's queries are emitted in rank order.
// The rows are therefore gathered twice (the reference gathers them three times) and every
// exponential was already taken by the sort/rank kernel.
#include "walk_ring.cuh"

namespace qlka {

enum { LAP_ROWS = 0, LAP_DOT = 1, LAP_BOTH = 2 };

// floats per stream in the aggregate table: forward aggregate | backward aggregate | decay forward, decay backward, pad
__host__ __device__ inline int lap_agg_stride(int C4) { return 2 * C4 + 4; }


template <int LPS, int CPL>
__global__ void __launch_bounds__(WALK_THREADS, (CPL <= 4 ? 3 : 1)) laplace_pass1(const WalkArgs a)
{
    constexpr int STREAMS = WALK_THREADS / LPS;
    extern __shared__ __align__(16) float4 smem[];
    float4* ring   = smem;                                                   // [RING_DEPTH][KB][CPL/4][WALK_THREADS]
    float*  sx_all = reinterpret_cast<float*>(reinterpret_cast<char*>(ring) + ring_bytes<CPL>());   // [STREAMS][RING_DEPTH][SX_STRIDE]

    const int tid = threadIdx.x;
    const int st  = tid / LPS, ln = tid % LPS, c0 = ln * CPL;
    const int SPS = a.sps;
    const int N = a.N, C4 = a.C4;
    const int NBK = nblocks(N), NP = npad(N);
    const bool lane_on = c0 < C4;
    const int  c0l     = lane_on ? c0 : 0;           // idle lanes shadow lane 0's loads and store nothing
    const unsigned gmask = (LPS == 32) ? FULL : (((1u << LPS) - 1u) << ((tid & 31) & ~(LPS - 1)));
    const long long nstreams = (long long)a.nseg * SPS;

    Feeder<LPS, CPL> f;
    f.ring_s = smem_u32(ring + tid);
    f.qs_s   = 0;                                  // no query records in this pass
    f.sx_s   = smem_u32(sx_all + st * RING_DEPTH * SX_STRIDE);
    f.row_bytes = (uint32_t)C4 * 4u; f.N = N; f.M = a.M; f.ln = ln; f.with_x = true; f.with_q = false;

    for (int item = blockIdx.x; item < a.nitems; item += gridDim.x) {
        const long long g  = (long long)item * STREAMS + st;         // this stream, in the numbering over all segments
        const bool      on_s = g < nstreams;
        const long long gg = on_s ? g : 0;
        const int  sg = (int)(gg / SPS), s = (int)(gg - (long long)sg * SPS);
        const int  p  = sg / a.D;
        const bool on = on_s && lane_on;
        int b0, b1;
        stream_blocks(s, SPS, NBK, b0, b1);
        const int nblk = on_s ? b1 - b0 : 0;

        f.xperm = a.xperm + (long long)sg * NP;
        f.xval  = a.xval + (long long)sg * xstride(N);
        f.rows  = a.rows + (long long)p * N * C4 + c0l;
        float* ck = a.ckpt + (long long)sg * NBK * C4 + c0l;
        float* wk = a.wck + (long long)sg * NBK;

        Vec<CPL> Rl, F;
        Rl.zero(); F.zero();
        float w = 1.0f, wprev = 1.0f;
        const float a_j1 = (on_s && b1 < NBK) ? __ldg(f.xval + b1 * KB) : 0.0f;   // decay from the next stream's first key
        __syncwarp(gmask);                         // every lane has left the previous item's slots
        f.prologue(b1 - 1, -1, nblk);
        int cur = 0;
        for (int t = 0; t < nblk; t++) {
            const int b = b1 - 1 - t, j0 = b * KB;
            __syncwarp(gmask);                     // every lane is done with the slot refilled below
            f.step(t, cur, b1 - 1, -1, nblk);
            __syncwarp(gmask);
            float av[KB + 1];
            f.read_scalars(cur, av);
            Vec<CPL> v[KB];
            f.read_rows(cur, j0, v);
            #pragma unroll
            for (int i = KB - 1; i >= 0; i--) {
                #pragma unroll
                for (int c = 0; c < CPL; c += 2) {
                    fma2(F.x[c], F.x[c + 1], w, w, v[i].x[c], v[i].x[c + 1], F.x[c], F.x[c + 1]);
                    fma2(Rl.x[c], Rl.x[c + 1], av[i + 1], av[i + 1], Rl.x[c], Rl.x[c + 1], v[i].x[c], v[i].x[c + 1]);
                }
                wprev = w;
                w *= av[i];
            }
            if (on) {                              // (streaming stores: the second pass reads them long after, once)
                #pragma unroll
                for (int c = 0; c < CPL; c += 4)
                    __stcs(reinterpret_cast<float4*>(ck + (long long)b * C4 + c), make_float4(Rl.x[c], Rl.x[c + 1], Rl.x[c + 2], Rl.x[c + 3]));
            }
            if (ln == 0) wk[b] = wprev * a_j1;
            cur = ring_next(cur);
        }
        cp_async_wait<0>();                        // (the trailing empty groups)
        if (on_s) {
            float* ag = a.agg + g * lap_agg_stride(C4);
            if (lane_on) {
                #pragma unroll
                for (int c = 0; c < CPL; c += 4) {
                    *reinterpret_cast<float4*>(ag + c0 + c)      = make_float4(F.x[c], F.x[c + 1], F.x[c + 2], F.x[c + 3]);
                    *reinterpret_cast<float4*>(ag + C4 + c0 + c) = make_float4(Rl.x[c], Rl.x[c + 1], Rl.x[c + 2], Rl.x[c + 3]);
                }
            }
            if (ln == 0) { ag[2 * C4] = w; ag[2 * C4 + 1] = wprev * a_j1; }
        }
    }
}

// Between the passes: per segment and channel, the aggregates of the SPS streams become the states entering each
// stream - in place, forward aggregate -> prefix state before the stream (L = decay * L + aggregate over the earlier
// streams), backward aggregate -> suffix state after it. One thread per (segment, channel), serial over the streams.
__global__ void __launch_bounds__(256) laplace_fold(float* __restrict__ agg, const int nseg, const int SPS, const int C4)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)nseg * C4) return;
    const int sg = (int)(i / C4), c = (int)(i - (long long)sg * C4);
    const int AGS = lap_agg_stride(C4);
    float* ag = agg + (long long)sg * SPS * AGS;
    constexpr int CH = 16;                     // streams per chunk: their loads are issued together, then the serial part
    float L = 0.0f;
    for (int t0 = 0; t0 < SPS; t0 += CH) {
        float fv[CH], af[CH];
        #pragma unroll
        for (int k = 0; k < CH; k++) {
            const float* at = ag + (long long)min(t0 + k, SPS - 1) * AGS;
            fv[k] = at[c]; af[k] = at[2 * C4];
        }
        #pragma unroll
        for (int k = 0; k < CH; k++) {
            if (t0 + k < SPS) { ag[(long long)(t0 + k) * AGS + c] = L; L = fmaf(af[k], L, fv[k]); }
        }
    }
    float R = 0.0f;
    for (int t0 = SPS - 1; t0 >= 0; t0 -= CH) {
        float bv[CH], ab[CH];
        #pragma unroll
        for (int k = 0; k < CH; k++) {
            const float* at = ag + (long long)max(t0 - k, 0) * AGS;
            bv[k] = at[C4 + c]; ab[k] = at[2 * C4 + 1];
        }
        #pragma unroll
        for (int k = 0; k < CH; k++) {
            if (t0 - k >= 0) { ag[(long long)(t0 - k) * AGS + C4 + c] = R; R = fmaf(ab[k], R, bv[k]); }
        }
    }
}

template <int LPS, int CPL, int EMIT>
__global__ void __launch_bounds__(WALK_THREADS, (CPL <= 4 ? WALK_MIN_CTAS : 1)) laplace_pass2(const WalkArgs a)
{
    constexpr bool DO_ROWS = EMIT != LAP_DOT, DO_DOT = EMIT != LAP_ROWS;
    constexpr int STREAMS = WALK_THREADS / LPS;
    extern __shared__ __align__(16) float4 smem[];
    float4* ring   = smem;                                                   // [RING_DEPTH][KB][CPL/4][WALK_THREADS]
    uint4*  qs_all = reinterpret_cast<uint4*>(reinterpret_cast<char*>(ring) + ring_bytes<CPL>());   // [STREAMS][RING_DEPTH][LPS]
    float*  sx_all = reinterpret_cast<float*>(qs_all + STREAMS * RING_DEPTH * LPS);       // [STREAMS][RING_DEPTH][SX_STRIDE]
    float4* g_area = reinterpret_cast<float4*>(sx_all + STREAMS * RING_DEPTH * SX_STRIDE);   // dot emissions only: [G_SLOTS][CPL/4][WALK_THREADS]

    const int tid = threadIdx.x;
    const int st  = tid / LPS, ln = tid % LPS, c0 = ln * CPL;
    const int SPS = a.sps;
    const int N = a.N, M = a.M, C4 = a.C4;
    const int NBK = nblocks(N), NP = npad(N);
    const bool lane_on = c0 < C4;
    const int  c0l     = lane_on ? c0 : 0;
    const unsigned gmask = (LPS == 32) ? FULL : (((1u << LPS) - 1u) << ((tid & 31) & ~(LPS - 1)));
    const long long nstreams = (long long)a.nseg * SPS;
    const int AGS = lap_agg_stride(C4);

    Feeder<LPS, CPL> f;
    f.ring_s = smem_u32(ring + tid);
    f.qs_s   = smem_u32(qs_all + st * RING_DEPTH * LPS);
    f.sx_s   = smem_u32(sx_all + st * RING_DEPTH * SX_STRIDE);
    f.row_bytes = (uint32_t)C4 * 4u; f.N = N; f.M = M; f.ln = ln; f.with_x = true; f.with_q = true;
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
        f.xval   = a.xval + (long long)sg * xstride(N);
        f.rows   = a.rows + (long long)p * N * C4 + c0l;
        f.mstart = a.mstart + (long long)sg * mstride(N);
        f.yrec   = a.yrec + (long long)sg * (M + 1);
        float*          out   = DO_ROWS ? a.out + (long long)p * a.Mrows * C4 + c0l : nullptr;
        const float*    g_    = DO_DOT ? a.g + (long long)p * M * C4 + c0l : nullptr;
        float*          out_s = DO_DOT ? a.out_s + (long long)sg * M : nullptr;
        f.grows = g_;
        const float* ck = a.ckpt + (long long)sg * NBK * C4 + c0l;
        const float* wk = a.wck + (long long)sg * NBK;

        // ---------------- incoming prefix and suffix state (laplace_fold left them in the aggregate table)
        Vec<CPL> L, Rin;
        {
            const float* ag = a.agg + gg * AGS + c0l;
            #pragma unroll
            for (int c = 0; c < CPL; c += 4) {
                const float4 fv = ldg4(ag + c), bv = ldg4(ag + C4 + c);
                L.x[c] = fv.x; L.x[c + 1] = fv.y; L.x[c + 2] = fv.z; L.x[c + 3] = fv.w;
                Rin.x[c] = bv.x; Rin.x[c + 1] = bv.y; Rin.x[c + 2] = bv.z; Rin.x[c + 3] = bv.w;
            }
        }

        // ---------------- forward with emission
        {
            __syncwarp(gmask);                         // every lane has left the previous item's slots
            f.prologue(b0, 1, nblk);
            // checkpoint of the block after the current one, fetched one iteration early
            Vec<CPL> cnext; cnext.zero();
            float    wnext = 0.0f;
            auto load_ckpt = [&](int bn) {
                if (bn < b1) {
                    wnext = wk[bn];
                    #pragma unroll
                    for (int c = 0; c < CPL; c += 4) {
                        const float4 t = __ldcs(reinterpret_cast<const float4*>(ck + (long long)bn * C4 + c));
                        cnext.x[c] = t.x; cnext.x[c + 1] = t.y; cnext.x[c + 2] = t.z; cnext.x[c + 3] = t.w;
                    }
                }
            };
            load_ckpt(b0 + 1);

            int cur = 0;
            for (int t = 0; t < nblk; t++) {
                const int b = b0 + t, j0 = b * KB;
                float av[KB + 1];
                uint32_t cnt;
                if (DO_DOT) {
                    // the block's copies have had a whole iteration; once its records are readable the emit-side rows
                    // of its first G_SLOTS queries start, ahead of the next block's copies, and land during the arithmetic
                    f.advance_range();
                    cp_async_wait<0>();
                    __syncwarp(gmask);
                    f.read_scalars(cur, av);
                    cnt = f.m_hi - f.m_lo;
                    f.issue_g(cur, 0u, cnt < (uint32_t)LPS ? min(cnt, (uint32_t)G_SLOTS) : 0u);
                } else {
                    __syncwarp(gmask);
                }

                // suffix state entering the block from above: corrected checkpoint, or the stream's incoming state
                Vec<CPL> Rn;
                if (b + 1 < b1) {
                    #pragma unroll
                    for (int c = 0; c < CPL; c++) Rn.x[c] = fmaf(wnext, Rin.x[c], cnext.x[c]);
                } else {
                    Rn = Rin;
                }
                load_ckpt(b + 2);

                if (DO_DOT) {
                    f.step_issue(t, cur, b0, 1, nblk);
                } else {
                    f.step(t, cur, b0, 1, nblk);
                    __syncwarp(gmask);
                    f.read_scalars(cur, av);
                    cnt = f.m_hi - f.m_lo;
                }
                Vec<CPL> v[KB];
                f.read_rows(cur, j0, v);

                Vec<CPL> Rb[KB];
                #pragma unroll
                for (int i = KB - 1; i >= 0; i--) {
                    #pragma unroll
                    for (int c = 0; c < CPL; c += 2) {
                        fma2(Rn.x[c], Rn.x[c + 1], av[i + 1], av[i + 1], Rn.x[c], Rn.x[c + 1], v[i].x[c], v[i].x[c + 1]);
                        Rb[i].x[c] = Rn.x[c]; Rb[i].x[c + 1] = Rn.x[c + 1];
                    }
                }
                // prefix state before each key, in place of the rows
                #pragma unroll
                for (int i = 0; i < KB; i++) {
                    #pragma unroll
                    for (int c = 0; c < CPL; c += 2) {
                        const float t0 = v[i].x[c], t1 = v[i].x[c + 1];
                        v[i].x[c] = L.x[c]; v[i].x[c + 1] = L.x[c + 1];
                        fma2(L.x[c], L.x[c + 1], av[i], av[i], L.x[c], L.x[c + 1], t0, t1);
                    }
                }
                // the block's queries, in rank order
                auto load_g = [&](const uint4 rec, Vec<CPL>& gq) {      // the emit-side row slice of a record
                    const float* gr = g_ + (size_t)rec.z * C4;
                    #pragma unroll
                    for (int c = 0; c < CPL; c += 4) {
                        const float4 t4 = lane_on ? ldg4(gr + c) : make_float4(0.f, 0.f, 0.f, 0.f);
                        gq.x[c] = t4.x; gq.x[c + 1] = t4.y; gq.x[c + 2] = t4.z; gq.x[c + 3] = t4.w;
                    }
                };
                auto emit_rows = [&](const uint4 rec, const Vec<CPL>& Lq, const Vec<CPL>& Rq) {
                    const float e0 = __uint_as_float(rec.x), e1 = __uint_as_float(rec.y);
                    if (DO_ROWS && on) {
                        float* o = out + (size_t)rec.z * C4;
                        #pragma unroll
                        for (int c = 0; c < CPL; c += 4) {
                            float r0, r1, r2, r3;
                            mul2(r0, r1, e1, e1, Rq.x[c], Rq.x[c + 1]);
                            mul2(r2, r3, e1, e1, Rq.x[c + 2], Rq.x[c + 3]);
                            fma2(r0, r1, e0, e0, Lq.x[c], Lq.x[c + 1], r0, r1);
                            fma2(r2, r3, e0, e0, Lq.x[c + 2], Lq.x[c + 3], r2, r3);
                            red_add4(o + c, r0, r1, r2, r3);
                        }
                    }
                };
                auto dot_part = [&](const uint4 rec, const Vec<CPL>& Lq, const Vec<CPL>& Rq, const Vec<CPL>& gq) -> float {
                    const float e0 = __uint_as_float(rec.x), e1 = __uint_as_float(rec.y);
                    float a0 = 0.0f, a1 = 0.0f;
                    #pragma unroll
                    for (int c = 0; c < CPL; c += 2) {
                        float t0, t1;
                        mul2(t0, t1, -e0, -e0, Lq.x[c], Lq.x[c + 1]);
                        fma2(t0, t1, e1, e1, Rq.x[c], Rq.x[c + 1], t0, t1);
                        fma2(a0, a1, gq.x[c], gq.x[c + 1], t0, t1, a0, a1);
                    }
                    return a0 + a1;
                };
                if (DO_DOT) {
                    cp_async_wait<1>();               // the emit-side rows are in; the next block's copies may still fly
                    __syncwarp(gmask);                // every lane has its rows in registers: the slot may hold partial dots
                }
                if (cnt < (uint32_t)LPS) {
                    // usual case: every record of the block sits in the staged slot, followed by a record of a later rank
                    uint32_t qa  = f.qs_s + cur * LPS * 16;
                    uint4    rec = lds128u(qa);
                    uint32_t n = 0, nb = min(cnt, (uint32_t)G_SLOTS);      // records [0, nb) have their emit-side rows staged
                    #pragma unroll
                    for (int i = 0; i < KB; i++) {
                        while (rec.w == (uint32_t)(j0 + i)) {
                            qa += 16;
                            const uint4 nxt = lds128u(qa);
                            emit_rows(rec, v[i], Rb[i]);
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
                                f.put_part(cur, n, dot_part(rec, v[i], Rb[i], gq));
                            }
                            rec = nxt;
                            ++n;
                        }
                    }
                    if (DO_DOT) {
                        __syncwarp(gmask);
                        if ((uint32_t)ln < cnt) {             // lane n finishes query n of the block
                            const float sum = f.sum_parts(cur, (uint32_t)ln);
                            atomicAdd(out_s + lds32u(f.qs_s + (cur * LPS + ln) * 16 + 8), sum);
                        }
                    }
                } else {
                    // more queries than the slot holds: read them from memory
                    const uint4* yp  = f.yrec + f.m_lo;
                    uint32_t     n   = 0;
                    uint4        rec = __ldg(yp);
                    #pragma unroll
                    for (int i = 0; i < KB; i++) {
                        while (n < cnt && rec.w == (uint32_t)(j0 + i)) {
                            ++n;
                            const uint4 nxt = __ldg(yp + n);        // at most the segment's sentinel
                            emit_rows(rec, v[i], Rb[i]);
                            if (DO_DOT) {
                                Vec<CPL> gq;
                                load_g(rec, gq);
                                float acc = dot_part(rec, v[i], Rb[i], gq);
                                #pragma unroll
                                for (int off = LPS / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(gmask, acc, off);
                                if (ln == 0) atomicAdd(out_s + rec.z, acc);
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
static cudaError_t launch_lap(const WalkArgs& a, int grid1, int grid2, cudaStream_t stream, cudaEvent_t mid) {
    auto k1 = laplace_pass1<LPS, CPL>;
    auto k2 = laplace_pass2<LPS, CPL, EMIT>;
    const size_t smem1 = pass1_smem_bytes<LPS, CPL>();
    const size_t smem2 = walk_smem_bytes<LPS, CPL>() + (EMIT != LAP_ROWS ? g_area_bytes<CPL>() : 0);
    cudaError_t e = cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    if (e != cudaSuccess) return e;
    k1<<<grid1, WALK_THREADS, smem1, stream>>>(a);
    laplace_fold<<<(unsigned)(((long long)a.nseg * a.C4 + 255) / 256), 256, 0, stream>>>(a.agg, a.nseg, a.sps, a.C4);
    if (mid) { e = cudaEventRecord(mid, stream); if (e != cudaSuccess) return e; }
    k2<<<grid2, WALK_THREADS, smem2, stream>>>(a);
    return cudaGetLastError();
}

template <int EMIT>
static cudaError_t launch_lap_c(const WalkArgs& a, int grid1, int grid2, cudaStream_t stream, cudaEvent_t mid) {
    if (a.C4 <= 32)  return launch_lap<8, 4, EMIT>(a, grid1, grid2, stream, mid);
    if (a.C4 <= 64)  return launch_lap<16, 4, EMIT>(a, grid1, grid2, stream, mid);
    if (a.C4 <= 128) return launch_lap<16, 8, EMIT>(a, grid1, grid2, stream, mid);
    return cudaErrorInvalidValue;
}

// lanes per stream for a padded channel count
int walk_lanes_per_stream(int C4) { return C4 <= 32 ? 8 : 16; }
int walk_threads() { return WALK_THREADS; }

int laplace_agg_stride(int C4) { return lap_agg_stride(C4); }

// emit: 0 = row reductions (the forward sum), 1 = dot, 2 = both; grid1 / grid2: CTAs of the two passes;
// mid: optional event recorded between the first pass (with the fold) and the second
cudaError_t launch_laplace_walk(const WalkArgs& a, int emit, int grid1, int grid2, cudaStream_t stream, cudaEvent_t mid) {
    if (emit == LAP_ROWS) return launch_lap_c<LAP_ROWS>(a, grid1, grid2, stream, mid);
    if (emit == LAP_DOT)  return launch_lap_c<LAP_DOT>(a, grid1, grid2, stream, mid);
    if (emit == LAP_BOTH) return launch_lap_c<LAP_BOTH>(a, grid1, grid2, stream, mid);
    return cudaErrorInvalidValue;
}

}  // namespace qlka

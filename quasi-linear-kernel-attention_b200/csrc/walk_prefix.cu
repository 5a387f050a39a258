// Prefix walk: for every query m of every segment, with r its rank among the sorted keys,
// PV = sum of the rows of the r keys below it and PK = sum of key * row over the same keys:
//
//   EMIT_ROWS  out[p, row_m, :] += e0_m * PV - 2 * PK          (vector reductions)
//              with e0 = 2 * query this is the walk term 2 (q PV - PK) of the abs sum
//              (Weighted_Abs_Sum/csrc/abs_kernels.cu:9-18; abs_chunk :78-199, abs_prefix :202-405)
//   EMIT_DOT   out_s[seg, row_m] = sign * ( <g[p, row_m, :], 2 PV - wtotal[p, :]> + e1_m )
//              the signed-rank walk behind grad_q, grad_k and the public sgn op
//              (Weighted_Abs_Sum/csrc/sgn_kernels.cu:8-15, sgn_prefix :17-192); one writer per
//              output element, plain stores.
//
// Same thread mapping as the Laplace walk (LPS lanes per stream, CPL channels per lane,
// SPS streams per segment, persistent CTAs). Pass 1 sums each stream's rows, a shared-memory
// scan turns the sums into each stream's incoming prefix, pass 2 walks forward and emits.
// With one stream per segment pass 1 and the scan are skipped.
#include "qlka_common.cuh"

namespace qlka {

constexpr int PWALK_THREADS = 256;
enum { EMIT_ROWS = 0, EMIT_DOT = 1 };

template <int CPL>
struct PVec { float x[CPL]; };

template <int CPL>
__device__ __forceinline__ void pload_row(PVec<CPL>& r, const float* __restrict__ p, const bool on) {
    #pragma unroll
    for (int c = 0; c < CPL; c += 4) {
        float4 t = on ? ldg4(p + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        r.x[c] = t.x; r.x[c + 1] = t.y; r.x[c + 2] = t.z; r.x[c + 3] = t.w;
    }
}

template <int LPS, int CPL, int EMIT>
__global__ void __launch_bounds__(PWALK_THREADS, (CPL <= 4 ? 2 : 1)) prefix_walk(const WalkArgs a)
{
    constexpr int  STREAMS = PWALK_THREADS / LPS;
    constexpr int  CW      = LPS * CPL;
    constexpr bool WITH_K  = EMIT == EMIT_ROWS;
    __shared__ float sV[STREAMS][CW];
    __shared__ float sK[WITH_K ? STREAMS : 1][WITH_K ? CW : 1];

    const int tid = threadIdx.x;
    const int st  = tid / LPS, ln = tid % LPS, c0 = ln * CPL;
    const int SPS = a.sps, SEGS = STREAMS / SPS;
    const int sl  = st / SPS, s = st % SPS;
    const int N = a.N, M = a.M, C4 = a.C4;
    const int NBK = nblocks(N), NP = npad(N);
    const bool lane_on = c0 < C4;
    const unsigned gmask = (LPS == 32) ? FULL : (((1u << LPS) - 1u) << ((tid & 31) & ~(LPS - 1)));

    for (int item = blockIdx.x; item < a.nitems; item += gridDim.x) {
        const int  seg    = item * SEGS + sl;
        const bool seg_on = seg < a.nseg;
        const bool on     = seg_on && lane_on;
        const int  p      = seg_on ? seg / a.D : 0;
        const int  b0     = seg_on ? (int)((long long)s * NBK / SPS) : 0;
        const int  b1     = seg_on ? (int)((long long)(s + 1) * NBK / SPS) : 0;

        const uint32_t* xperm  = a.xperm + (long long)(seg_on ? seg : 0) * NP;
        const float*    xval   = WITH_K ? a.xval + (long long)(seg_on ? seg : 0) * xstride(N) : nullptr;
        const uint4*    yrec   = a.yrec + (long long)(seg_on ? seg : 0) * M;
        const uint32_t* mstart = a.mstart + (long long)(seg_on ? seg : 0) * mstride(N);
        const float*    rows   = a.rows + (long long)p * N * C4 + c0;

        PVec<CPL> PV, PK;
        #pragma unroll
        for (int c = 0; c < CPL; c++) { PV.x[c] = 0.0f; PK.x[c] = 0.0f; }

        if (SPS > 1) {
            // ---------------- pass 1: stream sums
            for (int b = b0; b < b1; b++) {
                const int j0 = b * KB;
                float kv[KB];
                if (WITH_K) {
                    float4 t0 = ldg4(xval + j0), t1 = ldg4(xval + j0 + 4);
                    kv[0] = t0.x; kv[1] = t0.y; kv[2] = t0.z; kv[3] = t0.w;
                    kv[4] = t1.x; kv[5] = t1.y; kv[6] = t1.z; kv[7] = t1.w;
                }
                uint32_t pr[KB];
                {
                    uint4 t0 = __ldg(reinterpret_cast<const uint4*>(xperm + j0));
                    uint4 t1 = __ldg(reinterpret_cast<const uint4*>(xperm + j0 + 4));
                    pr[0] = t0.x; pr[1] = t0.y; pr[2] = t0.z; pr[3] = t0.w;
                    pr[4] = t1.x; pr[5] = t1.y; pr[6] = t1.z; pr[7] = t1.w;
                }
                PVec<CPL> v[KB];
                #pragma unroll
                for (int i = 0; i < KB; i++) pload_row<CPL>(v[i], rows + (long long)pr[i] * C4, on && (j0 + i < N));
                #pragma unroll
                for (int i = 0; i < KB; i++) {
                    #pragma unroll
                    for (int c = 0; c < CPL; c++) {
                        PV.x[c] += v[i].x[c];
                        if (WITH_K) PK.x[c] = fmaf(kv[i], v[i].x[c], PK.x[c]);
                    }
                }
            }
            #pragma unroll
            for (int c = 0; c < CPL; c++) {
                sV[st][c0 + c] = PV.x[c];
                if (WITH_K) sK[st][c0 + c] = PK.x[c];
            }
            __syncthreads();
            for (int i = tid; i < SEGS * CW; i += PWALK_THREADS) {
                const int g = i / CW, c = i % CW;
                float accv = 0.0f, acck = 0.0f;
                for (int t = 0; t < SPS; t++) {
                    const int q = g * SPS + t;
                    float fv = sV[q][c];
                    sV[q][c] = accv;
                    accv += fv;
                    if (WITH_K) { float fk = sK[q][c]; sK[q][c] = acck; acck += fk; }
                }
            }
            __syncthreads();
            #pragma unroll
            for (int c = 0; c < CPL; c++) {
                PV.x[c] = sV[st][c0 + c];
                if (WITH_K) PK.x[c] = sK[st][c0 + c];
            }
        }

        // emit-side constants
        PVec<CPL> wt;
        if (EMIT == EMIT_DOT) pload_row<CPL>(wt, a.wtotal + (long long)p * C4 + c0, on);
        float*       out   = EMIT == EMIT_ROWS ? a.out + (long long)p * M * C4 + c0 : nullptr;
        const float* g     = EMIT == EMIT_DOT ? a.g + (long long)p * M * C4 + c0 : nullptr;
        float*       out_s = EMIT == EMIT_DOT ? a.out_s + (long long)(seg_on ? seg : 0) * M : nullptr;

        // ---------------- pass 2: forward with emission
        for (int b = b0; b < b1; b++) {
            const int j0 = b * KB;
            float kv[KB];
            if (WITH_K) {
                float4 t0 = ldg4(xval + j0), t1 = ldg4(xval + j0 + 4);
                kv[0] = t0.x; kv[1] = t0.y; kv[2] = t0.z; kv[3] = t0.w;
                kv[4] = t1.x; kv[5] = t1.y; kv[6] = t1.z; kv[7] = t1.w;
            }
            uint32_t pr[KB];
            {
                uint4 t0 = __ldg(reinterpret_cast<const uint4*>(xperm + j0));
                uint4 t1 = __ldg(reinterpret_cast<const uint4*>(xperm + j0 + 4));
                pr[0] = t0.x; pr[1] = t0.y; pr[2] = t0.z; pr[3] = t0.w;
                pr[4] = t1.x; pr[5] = t1.y; pr[6] = t1.z; pr[7] = t1.w;
            }
            uint32_t       m  = __ldg(mstart + b);
            const uint32_t me = __ldg(mstart + b + 1);
            PVec<CPL> v[KB], kb[WITH_K ? KB : 1];
            #pragma unroll
            for (int i = 0; i < KB; i++) pload_row<CPL>(v[i], rows + (long long)pr[i] * C4, on && (j0 + i < N));
            // prefix states before each key, in place of the rows
            #pragma unroll
            for (int i = 0; i < KB; i++) {
                #pragma unroll
                for (int c = 0; c < CPL; c++) {
                    float t = v[i].x[c];
                    v[i].x[c] = PV.x[c];
                    PV.x[c] += t;
                    if (WITH_K) { kb[i].x[c] = PK.x[c]; PK.x[c] = fmaf(kv[i], t, PK.x[c]); }
                }
            }
            uint4 rec = m < me ? __ldg(yrec + m) : make_uint4(0, 0, 0, 0xffffffffu);
            #pragma unroll
            for (int i = 0; i < KB; i++) {
                while (m < me && rec.w == (uint32_t)(j0 + i)) {
                    const uint4 nxt = (m + 1 < me) ? __ldg(yrec + m + 1) : make_uint4(0, 0, 0, 0xffffffffu);
                    if (EMIT == EMIT_ROWS) {
                        const float e0 = __uint_as_float(rec.x);
                        if (on) {
                            float* o = out + (long long)rec.z * C4;
                            #pragma unroll
                            for (int c = 0; c < CPL; c += 4)
                                red_add4(o + c,
                                         fmaf(e0, v[i].x[c],     -2.0f * kb[WITH_K ? i : 0].x[c]),
                                         fmaf(e0, v[i].x[c + 1], -2.0f * kb[WITH_K ? i : 0].x[c + 1]),
                                         fmaf(e0, v[i].x[c + 2], -2.0f * kb[WITH_K ? i : 0].x[c + 2]),
                                         fmaf(e0, v[i].x[c + 3], -2.0f * kb[WITH_K ? i : 0].x[c + 3]));
                        }
                    } else {
                        PVec<CPL> gr;
                        pload_row<CPL>(gr, g + (long long)rec.z * C4, on);
                        float acc = 0.0f;
                        #pragma unroll
                        for (int c = 0; c < CPL; c++) acc = fmaf(gr.x[c], fmaf(2.0f, v[i].x[c], -wt.x[c]), acc);
                        #pragma unroll
                        for (int off = LPS / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(gmask, acc, off);
                        if (seg_on && ln == 0) out_s[rec.z] = a.sign * (acc + __uint_as_float(rec.y));
                    }
                    rec = nxt;
                    m++;
                }
            }
        }
        if (SPS > 1) __syncthreads();
    }
}

template <int LPS, int CPL, int EMIT>
static cudaError_t launch_pw(const WalkArgs& a, int grid, cudaStream_t stream) {
    prefix_walk<LPS, CPL, EMIT><<<grid, PWALK_THREADS, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_prefix_walk(const WalkArgs& a, int emit, int grid, cudaStream_t stream) {
    if (emit == EMIT_ROWS) {
        if (a.C4 <= 32)  return launch_pw<8, 4, EMIT_ROWS>(a, grid, stream);
        if (a.C4 <= 64)  return launch_pw<16, 4, EMIT_ROWS>(a, grid, stream);
        if (a.C4 <= 128) return launch_pw<16, 8, EMIT_ROWS>(a, grid, stream);
    } else {
        if (a.C4 <= 32)  return launch_pw<8, 4, EMIT_DOT>(a, grid, stream);
        if (a.C4 <= 64)  return launch_pw<16, 4, EMIT_DOT>(a, grid, stream);
        if (a.C4 <= 128) return launch_pw<16, 8, EMIT_DOT>(a, grid, stream);
    }
    return cudaErrorInvalidValue;
}

}  // namespace qlka

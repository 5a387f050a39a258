// Laplace walk: out[p, row_m, :] += e0_m * L_{r-1} + e1_m * R_r for every query m of every
// segment, where r is the query's rank, L the decayed prefix sum of the gathered rows and R
// the decayed suffix sum (recurrences of Weighted_Laplace_Sum/csrc/laplace_kernels.cu:5-13).
//
// Replaces the reference's laplace_chunk / laplace_scan / laplace_walk trio
// (laplace_kernels.cu:65-127, 134-188, 219-409) with one persistent kernel:
//   * LPS lanes cooperate on one "stream" (a contiguous run of key blocks of one segment),
//     each lane owning CPL consecutive channels, so a row is one or two 16-byte loads per
//     lane and a result is one or two 16-byte vector reductions; lanes never exchange data.
//   * pass 1 walks the stream backwards once: the local suffix state at every block start
//     goes to a per-CTA checkpoint buffer (L2 resident), the stream's forward and backward
//     aggregates to shared memory.
//   * a scan over the SPS streams of a segment (shared memory) gives every stream its
//     incoming prefix state and incoming suffix state.
//   * pass 2 walks forward: per block of 8 keys the suffix states are rebuilt in registers
//     from the next checkpoint, the prefix states overwrite the row registers, and the
//     block's queries (found through mstart, no searching) are emitted.
// The rows are therefore gathered twice (the reference gathers them three times) and every
// exponential was already taken by the sort/rank kernel.
#include "qlka_common.cuh"

namespace qlka {

constexpr int WALK_THREADS = 256;

template <int CPL>
struct Vec {
    float x[CPL];
    __device__ __forceinline__ void zero() {
        #pragma unroll
        for (int c = 0; c < CPL; c++) x[c] = 0.0f;
    }
};

template <int CPL>
__device__ __forceinline__ void load_row(Vec<CPL>& r, const float* __restrict__ p, const bool on) {
    #pragma unroll
    for (int c = 0; c < CPL; c += 4) {
        float4 t = on ? ldg4(p + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        r.x[c] = t.x; r.x[c + 1] = t.y; r.x[c + 2] = t.z; r.x[c + 3] = t.w;
    }
}

template <int LPS, int CPL>
__global__ void __launch_bounds__(WALK_THREADS, (CPL <= 4 ? 2 : 1)) laplace_walk(const WalkArgs a)
{
    constexpr int STREAMS = WALK_THREADS / LPS;
    constexpr int CW      = LPS * CPL;               // channel capacity of a stream
    __shared__ float sF[STREAMS][CW];                // forward aggregate  -> incoming prefix state
    __shared__ float sB[STREAMS][CW];                // backward aggregate -> incoming suffix state
    __shared__ float sAF[STREAMS], sAB[STREAMS];     // total decay across the stream (forward / backward)

    const int tid = threadIdx.x;
    const int st  = tid / LPS;                       // stream slot in this CTA
    const int ln  = tid % LPS;
    const int c0  = ln * CPL;
    const int SPS = a.sps, SEGS = STREAMS / SPS;
    const int sl  = st / SPS, s = st % SPS;          // segment slot, stream index within the segment
    const int N = a.N, M = a.M, C4 = a.C4;
    const int NBK = nblocks(N), NP = npad(N);
    const bool lane_on = c0 < C4;

    for (int item = blockIdx.x; item < a.nitems; item += gridDim.x) {
        const int  seg    = item * SEGS + sl;
        const bool seg_on = seg < a.nseg;
        const bool on     = seg_on && lane_on;
        const int  p      = seg_on ? seg / a.D : 0;
        const int  b0     = seg_on ? (int)((long long)s * NBK / SPS) : 0;
        const int  b1     = seg_on ? (int)((long long)(s + 1) * NBK / SPS) : 0;

        const uint32_t* xperm  = a.xperm + (long long)(seg_on ? seg : 0) * NP;
        const float*    xval   = a.xval + (long long)(seg_on ? seg : 0) * xstride(N);
        const uint4*    yrec   = a.yrec + (long long)(seg_on ? seg : 0) * M;
        const uint32_t* mstart = a.mstart + (long long)(seg_on ? seg : 0) * mstride(N);
        const float*    rows   = a.rows + (long long)p * N * C4 + c0;
        float*          out    = a.out + (long long)p * M * C4 + c0;
        const long long slot   = (long long)blockIdx.x * SEGS + sl;
        float*          ck     = a.ckpt + slot * NBK * C4 + c0;
        float*          wk     = a.wck + slot * NBK;

        // ---------------- pass 1: backward over the stream
        Vec<CPL> Rl, F;
        Rl.zero(); F.zero();
        float w = 1.0f, wprev = 1.0f;
        const float a_j1 = (seg_on && b1 < NBK) ? xval[b1 * KB] : 0.0f;   // decay from the next stream's first key
        for (int b = b1 - 1; b >= b0; b--) {
            const int j0 = b * KB;
            float av[KB + 1];
            {
                float4 t0 = ldg4(xval + j0), t1 = ldg4(xval + j0 + 4);
                av[0] = t0.x; av[1] = t0.y; av[2] = t0.z; av[3] = t0.w;
                av[4] = t1.x; av[5] = t1.y; av[6] = t1.z; av[7] = t1.w;
                av[8] = __ldg(xval + j0 + 8);
            }
            uint32_t pr[KB];
            {
                uint4 t0 = __ldg(reinterpret_cast<const uint4*>(xperm + j0));
                uint4 t1 = __ldg(reinterpret_cast<const uint4*>(xperm + j0 + 4));
                pr[0] = t0.x; pr[1] = t0.y; pr[2] = t0.z; pr[3] = t0.w;
                pr[4] = t1.x; pr[5] = t1.y; pr[6] = t1.z; pr[7] = t1.w;
            }
            Vec<CPL> v[KB];
            #pragma unroll
            for (int i = 0; i < KB; i++) load_row<CPL>(v[i], rows + (long long)pr[i] * C4, on && (j0 + i < N));
            #pragma unroll
            for (int i = KB - 1; i >= 0; i--) {
                #pragma unroll
                for (int c = 0; c < CPL; c++) {
                    F.x[c]  = fmaf(w, v[i].x[c], F.x[c]);
                    Rl.x[c] = fmaf(av[i + 1], Rl.x[c], v[i].x[c]);
                }
                wprev = w;
                w *= av[i];
            }
            if (on) {
                #pragma unroll
                for (int c = 0; c < CPL; c += 4)
                    *reinterpret_cast<float4*>(ck + (long long)b * C4 + c) = make_float4(Rl.x[c], Rl.x[c + 1], Rl.x[c + 2], Rl.x[c + 3]);
            }
            if (seg_on && ln == 0) wk[b] = wprev * a_j1;
        }
        #pragma unroll
        for (int c = 0; c < CPL; c++) { sF[st][c0 + c] = F.x[c]; sB[st][c0 + c] = Rl.x[c]; }
        if (ln == 0) { sAF[st] = w; sAB[st] = wprev * a_j1; }
        __syncthreads();

        // ---------------- scan over the streams of each segment
        for (int i = tid; i < SEGS * CW; i += WALK_THREADS) {
            const int g = i / CW, c = i % CW;
            float L = 0.0f;
            for (int t = 0; t < SPS; t++) {
                const int q = g * SPS + t;
                float f = sF[q][c];
                sF[q][c] = L;
                L = fmaf(sAF[q], L, f);
            }
            float R = 0.0f;
            for (int t = SPS - 1; t >= 0; t--) {
                const int q = g * SPS + t;
                float bb = sB[q][c];
                sB[q][c] = R;
                R = fmaf(sAB[q], R, bb);
            }
        }
        __syncthreads();

        // ---------------- pass 2: forward with emission
        Vec<CPL> L, Rin;
        #pragma unroll
        for (int c = 0; c < CPL; c++) { L.x[c] = sF[st][c0 + c]; Rin.x[c] = sB[st][c0 + c]; }

        for (int b = b0; b < b1; b++) {
            const int j0 = b * KB;
            float av[KB + 1];
            {
                float4 t0 = ldg4(xval + j0), t1 = ldg4(xval + j0 + 4);
                av[0] = t0.x; av[1] = t0.y; av[2] = t0.z; av[3] = t0.w;
                av[4] = t1.x; av[5] = t1.y; av[6] = t1.z; av[7] = t1.w;
                av[8] = __ldg(xval + j0 + 8);
            }
            uint32_t pr[KB];
            {
                uint4 t0 = __ldg(reinterpret_cast<const uint4*>(xperm + j0));
                uint4 t1 = __ldg(reinterpret_cast<const uint4*>(xperm + j0 + 4));
                pr[0] = t0.x; pr[1] = t0.y; pr[2] = t0.z; pr[3] = t0.w;
                pr[4] = t1.x; pr[5] = t1.y; pr[6] = t1.z; pr[7] = t1.w;
            }
            uint32_t m  = __ldg(mstart + b);
            const uint32_t me = __ldg(mstart + b + 1);
            Vec<CPL> v[KB];
            #pragma unroll
            for (int i = 0; i < KB; i++) load_row<CPL>(v[i], rows + (long long)pr[i] * C4, on && (j0 + i < N));

            // suffix state entering the block from above
            Vec<CPL> Rn;
            if (b + 1 < b1) {
                const float wn = wk[b + 1];          // written by lane 0 of this stream in pass 1 (before the barrier)
                #pragma unroll
                for (int c = 0; c < CPL; c += 4) {
                    float4 t = on ? *reinterpret_cast<const float4*>(ck + (long long)(b + 1) * C4 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
                    Rn.x[c]     = fmaf(wn, Rin.x[c], t.x);
                    Rn.x[c + 1] = fmaf(wn, Rin.x[c + 1], t.y);
                    Rn.x[c + 2] = fmaf(wn, Rin.x[c + 2], t.z);
                    Rn.x[c + 3] = fmaf(wn, Rin.x[c + 3], t.w);
                }
            } else {
                Rn = Rin;
            }
            Vec<CPL> Rb[KB];
            #pragma unroll
            for (int i = KB - 1; i >= 0; i--) {
                #pragma unroll
                for (int c = 0; c < CPL; c++) { Rn.x[c] = fmaf(av[i + 1], Rn.x[c], v[i].x[c]); Rb[i].x[c] = Rn.x[c]; }
            }
            // prefix state before each key, in place of the rows
            #pragma unroll
            for (int i = 0; i < KB; i++) {
                #pragma unroll
                for (int c = 0; c < CPL; c++) {
                    float t = v[i].x[c];
                    v[i].x[c] = L.x[c];
                    L.x[c] = fmaf(av[i], L.x[c], t);
                }
            }
            // the block's queries, in rank order
            uint4 rec = m < me ? __ldg(yrec + m) : make_uint4(0, 0, 0, 0xffffffffu);
            #pragma unroll
            for (int i = 0; i < KB; i++) {
                while (m < me && rec.w == (uint32_t)(j0 + i)) {
                    const uint4 nxt = (m + 1 < me) ? __ldg(yrec + m + 1) : make_uint4(0, 0, 0, 0xffffffffu);
                    const float e0 = __uint_as_float(rec.x), e1 = __uint_as_float(rec.y);
                    if (on) {
                        float* o = out + (long long)rec.z * C4;
                        #pragma unroll
                        for (int c = 0; c < CPL; c += 4)
                            red_add4(o + c,
                                     fmaf(e0, v[i].x[c],     e1 * Rb[i].x[c]),
                                     fmaf(e0, v[i].x[c + 1], e1 * Rb[i].x[c + 1]),
                                     fmaf(e0, v[i].x[c + 2], e1 * Rb[i].x[c + 2]),
                                     fmaf(e0, v[i].x[c + 3], e1 * Rb[i].x[c + 3]));
                    }
                    rec = nxt;
                    m++;
                }
            }
        }
        __syncthreads();        // shared aggregates are rewritten by the next item
    }
}

template <int LPS, int CPL>
static cudaError_t launch_lap(const WalkArgs& a, int grid, cudaStream_t stream) {
    laplace_walk<LPS, CPL><<<grid, WALK_THREADS, 0, stream>>>(a);
    return cudaGetLastError();
}

// streams per CTA for a channel count (C4 = channels rounded up to a multiple of 4)
int walk_lanes_per_stream(int C4) { return C4 <= 32 ? 8 : 16; }

cudaError_t launch_laplace_walk(const WalkArgs& a, int grid, cudaStream_t stream) {
    if (a.C4 <= 32)  return launch_lap<8, 4>(a, grid, stream);
    if (a.C4 <= 64)  return launch_lap<16, 4>(a, grid, stream);
    if (a.C4 <= 128) return launch_lap<16, 8>(a, grid, stream);
    return cudaErrorInvalidValue;
}

}  // namespace qlka

// Host side of the C ABI declared in include/qlka.h: argument checks that mirror the
// reference's TORCH_CHECKs, workspace carving, launch plans, and the kernel sequences of the
// four operators. No allocation, no synchronisation, no torch types.
#include "../../include/qlka.h"
#include "qlka_common.cuh"

#include <atomic>
#include <climits>

namespace qlka {
cudaError_t launch_sort_rank_small(const SortArgs& a, cudaStream_t stream);
cudaError_t launch_sort_rank_large(const SortArgs& a, void* scratch, cudaStream_t stream);
size_t      sort_rank_large_scratch_bytes(int nseg, int N, int M);
cudaError_t launch_laplace_walk(const WalkArgs& a, int emit, int grid1, int grid2, cudaStream_t stream, cudaEvent_t mid);
cudaError_t launch_prefix_walk(const WalkArgs& a, int emit, int grid1, int grid2, cudaStream_t stream);
int         walk_lanes_per_stream(int C4);
int         walk_threads();
int         laplace_agg_stride(int C4);
int         prefix_agg_stride_host(int C4);
cudaError_t launch_colsum_d(const float* x, float* out, int P, int D, int L, cudaStream_t st);
cudaError_t launch_rowstat(const float* w, const float* s, float* wsum, float* swsum, float* ssum, int P, int R, int C4, cudaStream_t st);
cudaError_t launch_vecsum(const float* x, float* out, int P, int L, cudaStream_t st);
cudaError_t launch_abs_init(const float* ktot, const float* vsum, const float* qsum, const float* ksr,
                            float* out, float* out_u, int P, int M, int C4, int Nk, float A, float Bq, cudaStream_t st);
cudaError_t launch_pad_rows(const float* src, float* dst, long long rows, int C, int C4, cudaStream_t st);
cudaError_t launch_unpad_rows(const float* src, float* dst, long long rows, int C, int C4, cudaStream_t st);
cudaError_t launch_transpose_scale(const float* src, float* dst, const float* keep, float scale, int P, int S, int D, int H, cudaStream_t st);
cudaError_t launch_mask_rows(const float* src, float* dst, const float* keep, int P, int S, int C, int H, cudaStream_t st);
cudaError_t launch_npad(const float* keep, float* n_pad, int B, int S, cudaStream_t st);
cudaError_t launch_normalise(float* out, const float* out_u, const float* qt, const float* n_pad,
                             int P, int M, int D, int C, int H, float clamp, bool bump, cudaStream_t st);
cudaError_t launch_abscolsum_d(const float* x, float* out, int P, int D, int L, cudaStream_t st);
cudaError_t launch_riesz_epilogue(float* out, const float* out_u, const float* aq, const float* vsum, const float* akv,
                                  const float* aksum, const float* n_pad, int P, int M, int C, int C4, int H,
                                  float eps, float clamp, cudaStream_t st);
}  // namespace qlka

using namespace qlka;

namespace {

thread_local int g_last_cuda = 0;

constexpr int SMALL_MAX = 16384;     // longest segment the shared-memory sort handles
constexpr int LENGTH_MAX = 262144;   // the reference stops at 131072 (binding.cpp:78); the global-memory sort goes on
constexpr int EMIT_ROWS = 0, EMIT_DOT = 1, EMIT_BOTH = 2;

#define CU(expr)                                                   \
    do {                                                           \
        cudaError_t e_ = (expr);                                   \
        if (e_ != cudaSuccess) { g_last_cuda = (int)e_; return QLKA_ERR_CUDA; } \
    } while (0)

int check_dims(int P, int D, int N, int M, int C) {
    if (P <= 0 || D <= 0 || N <= 0 || M <= 0) return QLKA_ERR_BAD_SHAPE;
    if (C < 1 || C > 128) return QLKA_ERR_C_RANGE;
    if (N > LENGTH_MAX || M > LENGTH_MAX) return QLKA_ERR_LENGTH;
    const long long mx = N > M ? N : M;
    if ((long long)P * D * mx > (long long)INT_MAX) return QLKA_ERR_INT32;
    return QLKA_OK;
}

// bump allocator over the workspace; with base == nullptr it only measures
struct Bump {
    char*  base;
    size_t off = 0;
    explicit Bump(void* b) : base(static_cast<char*>(b)) {}
    template <class T> T* take(size_t n) {
        off = (off + 255) & ~size_t(255);
        T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
        off += n * sizeof(T);
        return p;
    }
};

// SM count of the current device, looked up once per device (racing first calls store the same value)
int sm_count() {
    constexpr int MAX_DEV = 64;
    static std::atomic<int> cached[MAX_DEV];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return 148;      // B200; keeps workspace sizes defined without a device
    int n = cached[dev].load(std::memory_order_acquire);
    if (!n) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n, std::memory_order_release);
    }
    return n;
}

// How a walk over `nseg` segments of N keys is cut into streams, work items and CTAs. Streams are independent
// work units (the passes exchange their states through memory), so a segment may be cut into any number of them:
// more streams until the persistent CTAs of the second pass get about sixteen items each, as long as a stream
// keeps at least sixteen key blocks (the staging ring needs a few blocks to fill) - eight while there are fewer
// items than CTAs. The prefix walks need no first pass with one stream per segment, which pays as soon as whole
// segments alone give every CTA a few items.
struct WalkPlan { int sps, nitems, grid1, grid2; };

WalkPlan plan_walk(int nseg, int N, int C4, bool laplace) {
    const int lps      = walk_lanes_per_stream(C4);
    const int streams  = walk_threads() / lps;       // streams per CTA and work item
    const int sms      = sm_count();
    const int cap2     = sms * (C4 <= 64 ? 2 : 1);    // resident CTAs of the emitting pass (registers and shared memory)
    const int cap1     = sms * (C4 <= 64 ? 3 : 1);    // ... and of the lighter first pass
    const int nbk      = nblocks(N);
    auto items = [&](long long sps) { return (long long)(((long long)nseg * sps + streams - 1) / streams); };
    int sps = 1;
    if (laplace || items(1) < 2LL * cap2)
        while (items(sps) < 16LL * cap2 && nbk / (sps * 2) >= (items(sps) < cap2 ? 8 : 16) && sps < 4096) sps *= 2;
    WalkPlan w;
    w.sps    = sps;
    w.nitems = (int)items(sps);
    w.grid1  = w.nitems < cap1 ? w.nitems : cap1;
    w.grid2  = w.nitems < cap2 ? w.nitems : cap2;
    return w;
}

// per-stream aggregate table and (Laplace) per-segment checkpoint arrays of a planned walk
size_t walk_agg_floats(const WalkPlan& w, int nseg, int C4, bool laplace) {
    return (size_t)nseg * w.sps * (laplace ? laplace_agg_stride(C4) : prefix_agg_stride_host(C4));
}

// scratch of one sort/rank run over nseg segments of N keys and M queries
struct Records {
    uint32_t* xperm; float* xval; uint4* yrec; uint32_t* mstart; float* su0; float* su1;
    void* large;          // extra scratch of the global-memory sort, only when max(N, M) > SMALL_MAX
    void carve(Bump& b, int nseg, int N, int M) {
        large = (N > SMALL_MAX || M > SMALL_MAX) ? b.take<unsigned char>(sort_rank_large_scratch_bytes(nseg, N, M)) : nullptr;
        xperm  = b.take<uint32_t>((size_t)nseg * npad(N));
        xval   = b.take<float>((size_t)nseg * xstride(N));
        yrec   = b.take<uint4>((size_t)nseg * (M + 1));
        mstart = b.take<uint32_t>((size_t)nseg * mstride(N));
        su0    = b.take<float>((size_t)nseg * (N + 1));
        su1    = b.take<float>((size_t)nseg * (N + 1));
    }
};

SortArgs sort_args(const Records& r, const float* x, const float* y, int nseg, int D, int N, int M, int mode, int scal) {
    SortArgs s{};
    s.x = x; s.y = y;
    s.xperm = r.xperm; s.xval = r.xval; s.yrec = r.yrec; s.mstart = r.mstart; s.su0 = r.su0; s.su1 = r.su1;
    s.nseg = nseg; s.D = D; s.N = N; s.M = M; s.mode = mode; s.scal = scal;
    return s;
}

// the sort/rank stage: shared-memory kernel up to SMALL_MAX elements per segment, global-memory kernels above
cudaError_t launch_sort_rank(const SortArgs& s, const Records& r, cudaStream_t stream) {
    if (s.N <= SMALL_MAX && s.M <= SMALL_MAX) return launch_sort_rank_small(s, stream);
    return launch_sort_rank_large(s, r.large, stream);
}

WalkArgs walk_args(const Records& r, const float* rows, int nseg, int D, int N, int M, int C4) {
    WalkArgs a{};
    a.rows = rows; a.xperm = r.xperm; a.xval = r.xval; a.yrec = r.yrec; a.mstart = r.mstart;
    a.nseg = nseg; a.D = D; a.N = N; a.M = M; a.C4 = C4;
    a.sign = 1.0f;
    a.Mrows = M;
    return a;
}

// channels as the kernels see them: padded to the lane granularity of the walk (4 floats up to 64
// channels, 8 floats above, where a lane owns 8 channels)
inline int round4(int C) { return C <= 64 ? (C + 3) & ~3 : (C + 7) & ~7; }

// The row matrices (v, g_w, g, out_w, grad_v, the attention output) are read and written with 16-byte copies,
// loads and vector reductions: a pointer off that boundary would fault on the device, so it is refused here.
template <class... Ptr>
bool aligned16(Ptr... p) { return ((reinterpret_cast<uintptr_t>(p) | ...) & 15) == 0; }

bool ws_ok(const void* ws, size_t have, size_t need) {
    return need == 0 || (ws != nullptr && (reinterpret_cast<uintptr_t>(ws) & 255) == 0 && have >= need);
}

// ------------------------------------------------------------------ walks, a few heads at a time
// A walk gathers the rows of a head in 64 different orders and adds into its output rows; once the heads in flight no
// longer fit the L2 (long sequences) it pays to finish a few heads before starting the next ones, so every walk runs over
// chunks of whole heads whose row matrix stays under ROWS_BUDGET (one chunk up to B=4,H=12,N=16384,C=64 and well beyond;
// 15 heads at N=65536, 3 at N=262144 with 64 channels).
constexpr size_t ROWS_BUDGET = size_t(256) << 20;

int walk_chunk_heads(int P, int N, int C4) {
    size_t h = ROWS_BUDGET / ((size_t)N * C4 * sizeof(float));
    if (h < 1) h = 1;
    return (int)(h < (size_t)P ? h : (size_t)P);
}

// aggregate table of a prefix walk over P heads in chunks (the larger of the two chunk sizes that occur)
size_t prefix_agg_floats(int P, int D, int N, int C4) {
    const int heads = walk_chunk_heads(P, N, C4);
    size_t a = walk_agg_floats(plan_walk(heads * D, N, C4, false), heads * D, C4, false);
    if (const int rem = P % heads) {
        const size_t a2 = walk_agg_floats(plan_walk(rem * D, N, C4, false), rem * D, C4, false);
        if (a2 > a) a = a2;
    }
    return a;
}

// `w` describes the whole problem (pointers of head 0, nseg = P * D); every chunk gets its own plan
cudaError_t prefix_walk_chunked(WalkArgs w, int emit, int P, cudaStream_t stream)
{
    const int heads = walk_chunk_heads(P, w.N, w.C4);
    const WalkArgs all = w;
    for (int p0 = 0; p0 < P; p0 += heads) {
        const int       pc = heads < P - p0 ? heads : P - p0;
        const long long s0 = (long long)p0 * all.D;
        const WalkPlan  plan = plan_walk(pc * all.D, all.N, all.C4, false);
        w.rows   = all.rows + (size_t)p0 * all.N * all.C4;
        w.xperm  = all.xperm + s0 * npad(all.N);
        w.xval   = all.xval + s0 * xstride(all.N);
        w.yrec   = all.yrec + s0 * (all.M + 1);
        w.mstart = all.mstart + s0 * mstride(all.N);
        w.out    = all.out ? all.out + (size_t)p0 * all.Mrows * all.C4 : nullptr;
        w.g      = all.g ? all.g + (size_t)p0 * all.M * all.C4 : nullptr;
        w.wtotal = all.wtotal ? all.wtotal + (size_t)p0 * all.C4 : nullptr;
        w.out_s  = all.out_s ? all.out_s + s0 * all.M : nullptr;
        w.nseg = pc * all.D; w.sps = plan.sps; w.nitems = plan.nitems;
        cudaError_t e = launch_prefix_walk(w, emit, plan.grid1, plan.grid2, stream);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// The first walk pass leaves one suffix checkpoint per block of 8 keys and segment for the second pass: D / 8 times the
// size of the row matrix. So that this scratch does not grow with the batch, a chunk's checkpoints also stay under
// CKPT_BUDGET (the same chunks as the rows rule at D = 64).
constexpr size_t CKPT_BUDGET = size_t(2) << 30;

int laplace_chunk_heads(int P, int D, int N, int C4) {
    const size_t per_head = (size_t)D * nblocks(N) * C4 * sizeof(float);
    size_t h = CKPT_BUDGET / per_head;
    if (h < 1) h = 1;
    const int by_rows = walk_chunk_heads(P, N, C4);
    return (int)(h < (size_t)by_rows ? h : (size_t)by_rows);
}

struct LapWalkScratch {
    float *ckpt, *wck, *agg; int heads;
    void carve(Bump& b, int P, int D, int N, int C4) {
        heads = laplace_chunk_heads(P, D, N, C4);
        const int nseg_c = heads * D;
        ckpt = b.take<float>((size_t)nseg_c * nblocks(N) * C4);
        wck  = b.take<float>((size_t)nseg_c * nblocks(N));
        // the aggregate table of the larger of the two chunk sizes that occur (full chunks and the remainder)
        size_t a = walk_agg_floats(plan_walk(nseg_c, N, C4, true), nseg_c, C4, true);
        if (const int rem = P % heads) {
            const size_t a2 = walk_agg_floats(plan_walk(rem * D, N, C4, true), rem * D, C4, true);
            if (a2 > a) a = a2;
        }
        agg = b.take<float>(a);
    }
};

// rows (P, N, C4): the stream's rows; out (P, Mrows, C4) / g (P, M, C4) / out_s (P*D, M) as the emission needs them;
// mid: optional event between the passes of the first chunk (the stage timing of a single-chunk call)
cudaError_t laplace_walk_chunked(const Records& r, const LapWalkScratch& sc, const float* rows, float* out, const float* g, float* out_s,
                                 int emit, int P, int D, int N, int M, int C4, cudaStream_t stream, cudaEvent_t mid)
{
    for (int p0 = 0; p0 < P; p0 += sc.heads) {
        const int       pc = sc.heads < P - p0 ? sc.heads : P - p0, nseg = pc * D;
        const long long s0 = (long long)p0 * D;
        const WalkPlan  plan = plan_walk(nseg, N, C4, true);
        WalkArgs a{};
        a.rows = rows + (size_t)p0 * N * C4;
        a.xperm = r.xperm + s0 * npad(N); a.xval = r.xval + s0 * xstride(N);
        a.yrec = r.yrec + s0 * (M + 1);   a.mstart = r.mstart + s0 * mstride(N);
        a.ckpt = sc.ckpt; a.wck = sc.wck; a.agg = sc.agg;
        a.out   = out ? out + (size_t)p0 * M * C4 : nullptr;
        a.g     = g ? g + (size_t)p0 * M * C4 : nullptr;
        a.out_s = out_s ? out_s + s0 * M : nullptr;
        a.nseg = nseg; a.D = D; a.N = N; a.M = M; a.C4 = C4; a.sps = plan.sps; a.nitems = plan.nitems;
        a.sign = 1.0f; a.Mrows = M;
        cudaError_t e = launch_laplace_walk(a, emit, plan.grid1, plan.grid2, stream, p0 == 0 ? mid : nullptr);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// ------------------------------------------------------------------ Laplace forward
struct LaplaceWs {
    float* vpad; float* opad; Records rec; LapWalkScratch walk; size_t bytes;
    LaplaceWs(void* base, int P, int D, int N, int M, int C) {
        Bump b(base);
        const int C4 = round4(C), nseg = P * D;
        vpad = C4 != C ? b.take<float>((size_t)P * N * C4) : nullptr;
        opad = C4 != C ? b.take<float>((size_t)P * M * C4) : nullptr;
        rec.carve(b, nseg, N, M);
        walk.carve(b, P, D, N, C4);
        bytes = (b.off + 255) & ~size_t(255);
    }
};

// ------------------------------------------------------------------ Laplace backward
struct LaplaceBwdWs {
    float *vpad, *gpad, *gvpad; Records rec; LapWalkScratch walk; size_t bytes;
    LaplaceBwdWs(void* base, int P, int D, int N, int M, int C) {
        Bump b(base);
        const int C4 = round4(C), nseg = P * D;
        vpad  = C4 != C ? b.take<float>((size_t)P * N * C4) : nullptr;
        gpad  = C4 != C ? b.take<float>((size_t)P * M * C4) : nullptr;
        gvpad = C4 != C ? b.take<float>((size_t)P * N * C4) : nullptr;
        const int mx = N > M ? N : M;
        rec.carve(b, nseg, mx, mx);
        walk.carve(b, P, D, mx, C4);            // one scratch for both walks (stream of keys k, then stream of keys q): sized for the longer
        bytes = (b.off + 255) & ~size_t(255);
    }
};

// ------------------------------------------------------------------ abs forward
struct AbsFwdWs {
    float* vpad; float* opad; Records rec; float *qsum, *ksumd, *vsum, *ktot, *ksr, *agg; size_t bytes;
    AbsFwdWs(void* base, int P, int D, int N, int M, int C) {
        Bump b(base);
        const int C4 = round4(C), nseg = P * D;
        vpad = C4 != C ? b.take<float>((size_t)P * N * C4) : nullptr;
        opad = C4 != C ? b.take<float>((size_t)P * M * C4) : nullptr;
        rec.carve(b, nseg, N, M);
        qsum  = b.take<float>((size_t)P * M);
        ksumd = b.take<float>((size_t)P * N);
        vsum  = b.take<float>((size_t)P * C4 * 2 + P);     // vsum | ktot | ksr, zeroed together
        ktot  = vsum ? vsum + (size_t)P * C4 : nullptr;
        ksr   = vsum ? ktot + (size_t)P * C4 : nullptr;
        agg   = b.take<float>(prefix_agg_floats(P, D, N, C4));
        bytes = (b.off + 255) & ~size_t(255);
    }
};

// ------------------------------------------------------------------ abs backward / sgn
struct AbsBwdWs {
    float *vpad, *gpad, *gvpad; Records rec;
    float *qsumd, *ksumd, *sums /* vsum | gwsum | qtotg | gu_total */, *agg;
    size_t bytes;
    AbsBwdWs(void* base, int P, int D, int N, int M, int C) {
        Bump b(base);
        const int C4 = round4(C), nseg = P * D;
        vpad  = C4 != C ? b.take<float>((size_t)P * N * C4) : nullptr;
        gpad  = C4 != C ? b.take<float>((size_t)P * M * C4) : nullptr;
        gvpad = C4 != C ? b.take<float>((size_t)P * N * C4) : nullptr;
        const int mx = N > M ? N : M;
        rec.carve(b, nseg, mx, mx);
        qsumd = b.take<float>((size_t)P * M);
        ksumd = b.take<float>((size_t)P * N);
        sums  = b.take<float>((size_t)P * C4 * 3 + P);
        const size_t agg_k = prefix_agg_floats(P, D, N, C4), agg_q = prefix_agg_floats(P, D, M, C4);
        agg   = b.take<float>(agg_k > agg_q ? agg_k : agg_q);
        bytes = (b.off + 255) & ~size_t(255);
    }
};

}  // namespace

extern "C" {

const char* qlka_status_string(int status) {
    switch (status) {
        case QLKA_OK:                    return "ok";
        case QLKA_ERR_BAD_SHAPE:         return "N, M and D must be > 0";
        case QLKA_ERR_C_RANGE:           return "C (v.size(2)) must be in [1, 128]";
        case QLKA_ERR_LENGTH:            return "N and M must be <= 262144 (the reference: <= 131072)";
        case QLKA_ERR_INT32:             return "P*D*max(N,M) must fit int32 (cub sort offsets)";
        case QLKA_ERR_PATH:              return "path must be -1 (auto), 0 (global) or 1 (fused)";
        case QLKA_ERR_FUSED_UNAVAILABLE: return "fused path pinned but unavailable: needs max(N,M) <= 4096 and the bucket's shared memory to fit this device";
        case QLKA_ERR_NULL:              return "a required pointer is NULL";
        case QLKA_ERR_WORKSPACE:         return "workspace too small or not 256-byte aligned";
        case QLKA_ERR_CUDA:              return "a CUDA runtime call failed";
        case QLKA_ERR_UNSUPPORTED:       return "no kernel in this build for these sizes (shifted abs sum: N and n_shifts * M must be <= 16384)";
        case QLKA_ERR_NO_ALLOC_LIMIT:    return "problem needs more scratch than the fixed 32 MiB of the no-allocation entry point; use the workspace variant";
        case QLKA_ERR_ALIGNMENT:         return "v, g_w, g, out_w, grad_v and the attention output must be 16-byte aligned";
        default:                         return "unknown status";
    }
}

int qlka_last_cuda_error(void) { return g_last_cuda; }

// ---------------------------------------------------------------- Laplace
int qlka_laplace_forward_workspace_bytes(int P, int D, int N, int M, int C, size_t* bytes) {
    if (!bytes) return QLKA_ERR_NULL;
    int st = check_dims(P, D, N, M, C);
    if (st) return st;
    *bytes = LaplaceWs(nullptr, P, D, N, M, C).bytes;
    return QLKA_OK;
}

static int laplace_forward_impl(const float* q, const float* k, const float* v,
                                float* out_w, float* out_u, void* workspace, size_t workspace_bytes,
                                int P, int D, int N, int M, int C, cudaStream_t stream, cudaEvent_t* ev)
{
    int st = check_dims(P, D, N, M, C);
    if (st) return st;
    if (!q || !k || !v || !out_w || !out_u) return QLKA_ERR_NULL;
    if (!aligned16(v, out_w)) return QLKA_ERR_ALIGNMENT;
    LaplaceWs ws(workspace, P, D, N, M, C);
    if (!ws_ok(workspace, workspace_bytes, ws.bytes)) return QLKA_ERR_WORKSPACE;
    const int C4 = round4(C), nseg = P * D;

    const float* rows = v;
    float*       out  = out_w;
    if (C4 != C) {
        CU(launch_pad_rows(v, ws.vpad, (long long)P * N, C, C4, stream));
        rows = ws.vpad; out = ws.opad;
    }
    CU(cudaMemsetAsync(out, 0, sizeof(float) * (size_t)P * M * C4, stream));
    CU(cudaMemsetAsync(out_u, 0, sizeof(float) * (size_t)P * M, stream));
    if (ev) CU(cudaEventRecord(ev[0], stream));

    SortArgs s = sort_args(ws.rec, k, q, nseg, D, N, M, MODE_LAPLACE, SCAL_UNIT);
    s.out_u = out_u;
    CU(launch_sort_rank(s, ws.rec, stream));
    if (ev) CU(cudaEventRecord(ev[1], stream));

    CU(laplace_walk_chunked(ws.rec, ws.walk, rows, out, nullptr, nullptr, EMIT_ROWS, P, D, N, M, C4, stream, ev ? ev[2] : nullptr));
    if (ev) CU(cudaEventRecord(ev[3], stream));

    if (C4 != C) CU(launch_unpad_rows(out, out_w, (long long)P * M, C, C4, stream));
    return QLKA_OK;
}

int qlka_weighted_laplace_sum_forward(const float* q, const float* k, const float* v,
                                      float* out_w, float* out_u, void* workspace, size_t workspace_bytes,
                                      int P, int D, int N, int M, int C, qlka_stream_t stream_)
{
    return laplace_forward_impl(q, k, v, out_w, out_u, workspace, workspace_bytes, P, D, N, M, C,
                                reinterpret_cast<cudaStream_t>(stream_), nullptr);
}

int qlka_laplace_forward_stage_ms(const float* q, const float* k, const float* v,
                                  float* out_w, float* out_u, void* workspace, size_t workspace_bytes,
                                  int P, int D, int N, int M, int C, qlka_stream_t stream_,
                                  float* sort_ms, float* pass1_ms, float* pass2_ms)
{
    if (!sort_ms || !pass1_ms || !pass2_ms) return QLKA_ERR_NULL;
    cudaEvent_t ev[4];
    for (int i = 0; i < 4; i++) CU(cudaEventCreate(&ev[i]));
    int st = laplace_forward_impl(q, k, v, out_w, out_u, workspace, workspace_bytes, P, D, N, M, C,
                                  reinterpret_cast<cudaStream_t>(stream_), ev);
    if (st == QLKA_OK) {
        cudaError_t e = cudaEventSynchronize(ev[3]);
        if (e == cudaSuccess) e = cudaEventElapsedTime(sort_ms, ev[0], ev[1]);
        if (e == cudaSuccess) e = cudaEventElapsedTime(pass1_ms, ev[1], ev[2]);
        if (e == cudaSuccess) e = cudaEventElapsedTime(pass2_ms, ev[2], ev[3]);
        if (e != cudaSuccess) { g_last_cuda = (int)e; st = QLKA_ERR_CUDA; }
    }
    for (int i = 0; i < 4; i++) cudaEventDestroy(ev[i]);
    return st;
}

// ---------------------------------------------------------------- Laplace backward
int qlka_laplace_backward_workspace_bytes(int P, int D, int N, int M, int C, size_t* bytes) {
    if (!bytes) return QLKA_ERR_NULL;
    int st = check_dims(P, D, N, M, C);
    if (st) return st;
    *bytes = LaplaceBwdWs(nullptr, P, D, N, M, C).bytes;
    return QLKA_OK;
}

int qlka_weighted_laplace_sum_backward(const float* q, const float* k, const float* v,
                                       const float* g_w, const float* g_u,
                                       float* grad_q, float* grad_k, float* grad_v,
                                       void* workspace, size_t workspace_bytes,
                                       int P, int D, int N, int M, int C, qlka_stream_t stream_)
{
    int st = check_dims(P, D, N, M, C);
    if (st) return st;
    if (!q || !k || !v || !g_w || !grad_q || !grad_k || !grad_v) return QLKA_ERR_NULL;
    if (!aligned16(v, g_w, grad_v)) return QLKA_ERR_ALIGNMENT;
    LaplaceBwdWs ws(workspace, P, D, N, M, C);
    if (!ws_ok(workspace, workspace_bytes, ws.bytes)) return QLKA_ERR_WORKSPACE;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    const int C4 = round4(C), nseg = P * D;
    const bool full = g_u != nullptr;

    const float* vrows = v;
    const float* grows = g_w;
    float*       gv    = grad_v;
    if (C4 != C) {
        CU(launch_pad_rows(v, ws.vpad, (long long)P * N, C, C4, stream));
        CU(launch_pad_rows(g_w, ws.gpad, (long long)P * M, C, C4, stream));
        vrows = ws.vpad; grows = ws.gpad; gv = ws.gvpad;
    }
    CU(cudaMemsetAsync(gv, 0, sizeof(float) * (size_t)P * N * C4, stream));
    if (!full) {    // the walks add to grad_q and grad_k; with g_u the sort/rank kernel stores its term there first
        CU(cudaMemsetAsync(grad_q, 0, sizeof(float) * (size_t)nseg * M, stream));
        CU(cudaMemsetAsync(grad_k, 0, sizeof(float) * (size_t)nseg * N, stream));
    }
    {   // grad_q[d, m] = <g_w[m], e1 R_r - e0 L_{r-1}> + g_u[m] (e1 Ru_r - e0 Lu_{r-1}): queries q walk the key stream k
        SortArgs s = sort_args(ws.rec, k, q, nseg, D, N, M, MODE_LAPLACE, full ? SCAL_SIGNED : SCAL_NONE);
        s.uq = g_u; s.out_s = grad_q;
        CU(launch_sort_rank(s, ws.rec, stream));
        CU(laplace_walk_chunked(ws.rec, ws.walk, vrows, nullptr, grows, grad_q, EMIT_DOT, P, D, N, M, C4, stream, nullptr));
    }
    {   // roles swapped: queries k walk the stream q whose rows are g_w (and whose per-key scalar is g_u);
        // the row emission is grad_v, the dot with the v rows is grad_k
        SortArgs s = sort_args(ws.rec, q, k, nseg, D, M, N, MODE_LAPLACE, full ? SCAL_SIGNED : SCAL_NONE);
        s.us = g_u; s.out_s = grad_k;
        CU(launch_sort_rank(s, ws.rec, stream));
        CU(laplace_walk_chunked(ws.rec, ws.walk, grows, gv, vrows, grad_k, EMIT_BOTH, P, D, M, N, C4, stream, nullptr));
    }
    if (C4 != C) CU(launch_unpad_rows(gv, grad_v, (long long)P * N, C, C4, stream));
    return QLKA_OK;
}

// ---------------------------------------------------------------- add_laplace attention on (B, H, S, D)
namespace {
struct LaplaceAttnWs {
    float *qt, *kt, *vm, *out_u, *n_pad; void* inner; size_t inner_bytes, bytes;
    LaplaceAttnWs(void* base, int B, int H, int S, int D, int C, bool masked) {
        Bump b(base);
        const size_t P = (size_t)B * H;
        qt    = b.take<float>(P * D * S);
        kt    = b.take<float>(P * D * S);
        vm    = masked ? b.take<float>(P * S * C) : nullptr;
        out_u = b.take<float>(P * S);
        n_pad = masked ? b.take<float>((size_t)B) : nullptr;
        inner_bytes = LaplaceWs(nullptr, (int)P, D, S, S, C).bytes;
        inner = b.take<unsigned char>(inner_bytes);
        bytes = (b.off + 255) & ~size_t(255);
    }
};
}  // namespace

static int attn_check(int B, int H, int S, int D, int C) {
    if (B <= 0 || H <= 0) return QLKA_ERR_BAD_SHAPE;
    if ((long long)B * H > INT_MAX || D > 32 * 65535) return QLKA_ERR_INT32;
    return check_dims(B * H, D, S, S, C);
}

int qlka_laplace_attention_workspace_bytes(int B, int H, int S, int D, int Dv, int masked, size_t* bytes) {
    if (!bytes) return QLKA_ERR_NULL;
    int st = attn_check(B, H, S, D, Dv);
    if (st) return st;
    *bytes = LaplaceAttnWs(nullptr, B, H, S, D, Dv, masked != 0).bytes;
    return QLKA_OK;
}

int qlka_laplace_attention_forward(const float* q, const float* k, const float* v, const float* keep, float tau,
                                   float* out, void* workspace, size_t workspace_bytes,
                                   int B, int H, int S, int D, int Dv, qlka_stream_t stream_)
{
    int st = attn_check(B, H, S, D, Dv);
    if (st) return st;
    if (!q || !k || !v || !out) return QLKA_ERR_NULL;
    if (!aligned16(v, out)) return QLKA_ERR_ALIGNMENT;
    if (!(tau > 0.0f)) return QLKA_ERR_BAD_SHAPE;
    const bool masked = keep != nullptr;
    LaplaceAttnWs ws(workspace, B, H, S, D, Dv, masked);
    if (!ws_ok(workspace, workspace_bytes, ws.bytes)) return QLKA_ERR_WORKSPACE;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    const int P = B * H;

    CU(launch_transpose_scale(q, ws.qt, nullptr, 1.0f / tau, P, S, D, H, stream));
    CU(launch_transpose_scale(k, ws.kt, keep, 1.0f / tau, P, S, D, H, stream));
    const float* rows = v;
    if (masked) {
        CU(launch_mask_rows(v, ws.vm, keep, P, S, Dv, H, stream));
        CU(launch_npad(keep, ws.n_pad, B, S, stream));
        rows = ws.vm;
    }
    st = laplace_forward_impl(ws.qt, ws.kt, rows, out, ws.out_u, ws.inner, ws.inner_bytes, P, D, S, S, Dv, stream, nullptr);
    if (st) return st;
    CU(launch_normalise(out, ws.out_u, ws.qt, ws.n_pad, P, S, D, Dv, H, 1e-6f, false, stream));
    return QLKA_OK;
}

// ---------------------------------------------------------------- add_riesz / add_bump attention on (B, H, S, D)
static int abs_forward_impl(const float* q, const float* k, const float* v, float* out_w, float* out_u,
                            void* workspace, size_t workspace_bytes, int P, int D, int N, int M, int C,
                            int ns, const float* shifts, const float* weights, cudaStream_t stream);
namespace {
constexpr float BUMP_SHIFTS[3]  = {0.0f, 1.0f, -1.0f};     // max(0, 1 - |x|) = |x + 1| / 2 + |x - 1| / 2 - |x|
constexpr float BUMP_WEIGHTS[3] = {-1.0f, 0.5f, 0.5f};
struct AbsAttnWs {
    float *qt, *kt, *vm, *out_u, *n_pad, *aq, *ak, *sums /* vsum | akv | aksum */; void* inner; size_t inner_bytes, bytes;
    AbsAttnWs(void* base, int B, int H, int S, int D, int C, bool masked, bool bump) {
        Bump b(base);
        const size_t P = (size_t)B * H;
        qt    = b.take<float>(P * D * S);
        kt    = b.take<float>(P * D * S);
        vm    = masked ? b.take<float>(P * S * C) : nullptr;
        out_u = b.take<float>(P * S);
        n_pad = masked ? b.take<float>((size_t)B) : nullptr;
        aq    = bump ? nullptr : b.take<float>(P * S);
        ak    = bump ? nullptr : b.take<float>(P * S);
        sums  = bump ? nullptr : b.take<float>(P * C * 2 + P);
        inner_bytes = AbsFwdWs(nullptr, (int)P, D, S, bump ? 3 * S : S, C).bytes;
        inner = b.take<unsigned char>(inner_bytes);
        bytes = (b.off + 255) & ~size_t(255);
    }
};
}  // namespace

static int abs_attn_check(int kind, int B, int H, int S, int D, int C) {
    if (kind != 0 && kind != 1) return QLKA_ERR_PATH;
    int st = attn_check(B, H, S, D, C);
    if (st) return st;
    if (kind == 1 && 3LL * S > SMALL_MAX) return QLKA_ERR_UNSUPPORTED;     // the three shifted query copies share one shared-memory sort
    return QLKA_OK;
}

int qlka_abs_attention_workspace_bytes(int kind, int B, int H, int S, int D, int Dv, int masked, size_t* bytes) {
    if (!bytes) return QLKA_ERR_NULL;
    int st = abs_attn_check(kind, B, H, S, D, Dv);
    if (st) return st;
    *bytes = AbsAttnWs(nullptr, B, H, S, D, Dv, masked != 0, kind == 1).bytes;
    return QLKA_OK;
}

int qlka_abs_attention_forward(int kind, const float* q, const float* k, const float* v, const float* keep, float tau,
                               float* out, void* workspace, size_t workspace_bytes,
                               int B, int H, int S, int D, int Dv, qlka_stream_t stream_)
{
    int st = abs_attn_check(kind, B, H, S, D, Dv);
    if (st) return st;
    if (!q || !k || !v || !out) return QLKA_ERR_NULL;
    if (!aligned16(v, out)) return QLKA_ERR_ALIGNMENT;
    if (!(tau > 0.0f)) return QLKA_ERR_BAD_SHAPE;
    const bool masked = keep != nullptr, bump = kind == 1;
    AbsAttnWs ws(workspace, B, H, S, D, Dv, masked, bump);
    if (!ws_ok(workspace, workspace_bytes, ws.bytes)) return QLKA_ERR_WORKSPACE;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    const int P = B * H;

    CU(launch_transpose_scale(q, ws.qt, nullptr, 1.0f / tau, P, S, D, H, stream));
    CU(launch_transpose_scale(k, ws.kt, keep, 1.0f / tau, P, S, D, H, stream));
    const float* rows = v;
    if (masked) {
        CU(launch_mask_rows(v, ws.vm, keep, P, S, Dv, H, stream));
        CU(launch_npad(keep, ws.n_pad, B, S, stream));
        rows = ws.vm;
    }
    if (bump) {
        // numerator and row sum of the three shifted abs sums from one sort, then the row normalisation
        st = abs_forward_impl(ws.qt, ws.kt, rows, out, ws.out_u, ws.inner, ws.inner_bytes, P, D, S, S, Dv, 3, BUMP_SHIFTS, BUMP_WEIGHTS, stream);
        if (st) return st;
        CU(launch_normalise(out, ws.out_u, ws.qt, ws.n_pad, P, S, D, Dv, H, 1e-6f, true, stream));
    } else {
        // A_ij = |q_i|_1 + |k_j|_1 - |q_i - k_j|_1 + eps: rank-1 terms from column and row statistics, the abs sum from the walk
        float* vsum  = ws.sums;
        float* akv   = vsum + (size_t)P * Dv;
        float* aksum = akv + (size_t)P * Dv;
        CU(launch_abscolsum_d(ws.qt, ws.aq, P, D, S, stream));
        CU(launch_abscolsum_d(ws.kt, ws.ak, P, D, S, stream));
        CU(cudaMemsetAsync(ws.sums, 0, sizeof(float) * ((size_t)P * Dv * 2 + P), stream));
        CU(launch_rowstat(rows, ws.ak, vsum, akv, aksum, P, S, Dv, stream));
        st = abs_forward_impl(ws.qt, ws.kt, rows, out, ws.out_u, ws.inner, ws.inner_bytes, P, D, S, S, Dv, 0, nullptr, nullptr, stream);
        if (st) return st;
        CU(launch_riesz_epilogue(out, ws.out_u, ws.aq, vsum, akv, aksum, ws.n_pad, P, S, Dv, Dv, H, 1e-3f, 1e-6f, stream));
    }
    return QLKA_OK;
}

// ---------------------------------------------------------------- Laplace, fixed scratch
// Scratch for qlka_weighted_laplace_sum_forward_noalloc: lives in the library image, so every
// device that loads the library reserves QLKA_NOALLOC_SCRATCH_BYTES for as long as the process runs.
constexpr size_t QLKA_NOALLOC_SCRATCH_BYTES = size_t(32) << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[QLKA_NOALLOC_SCRATCH_BYTES];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not an address a kernel could
// use: the device address is looked up once per device (with that device current) and cached.
static int noalloc_scratch(void** out) {
    constexpr int MAX_DEV = 64;
    static std::atomic<void*> cached[MAX_DEV];
    int dev = 0;
    CU(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEV) return QLKA_ERR_UNSUPPORTED;
    void* ptr = cached[dev].load(std::memory_order_acquire);
    if (!ptr) {
        CU(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        cached[dev].store(ptr, std::memory_order_release);      // racing first calls store the same value
    }
    *out = ptr;
    return QLKA_OK;
}

size_t qlka_noalloc_scratch_bytes(void) { return QLKA_NOALLOC_SCRATCH_BYTES; }

int qlka_weighted_laplace_sum_forward_noalloc(const float* q, const float* k, const float* v,
                                              float* out_w, float* out_u,
                                              int P, int D, int N, int M, int C, qlka_stream_t stream_)
{
    int st = check_dims(P, D, N, M, C);
    if (st) return st;
    if (!q || !k || !v || !out_w || !out_u) return QLKA_ERR_NULL;
    if (!aligned16(v, out_w)) return QLKA_ERR_ALIGNMENT;
    if (LaplaceWs(nullptr, P, D, N, M, C).bytes > QLKA_NOALLOC_SCRATCH_BYTES) return QLKA_ERR_NO_ALLOC_LIMIT;
    void* scratch = nullptr;
    st = noalloc_scratch(&scratch);
    if (st) return st;
    // every byte of scratch that the kernels read is written earlier in the same call, and the
    // outputs are zeroed by the call itself, so what a previous call left behind is never seen
    return laplace_forward_impl(q, k, v, out_w, out_u, scratch, QLKA_NOALLOC_SCRATCH_BYTES, P, D, N, M, C,
                                reinterpret_cast<cudaStream_t>(stream_), nullptr);
}

// ---------------------------------------------------------------- abs forward
int qlka_abs_forward_workspace_bytes(int P, int D, int N, int M, int C, size_t* bytes) {
    if (!bytes) return QLKA_ERR_NULL;
    int st = check_dims(P, D, N, M, C);
    if (st) return st;
    *bytes = AbsFwdWs(nullptr, P, D, N, M, C).bytes;
    return QLKA_OK;
}

// ns == 0: the plain abs sum. ns >= 1: sum_s weights[s] * abs_sum(q + shifts[s]) from one sort of the keys.
static int abs_forward_impl(const float* q, const float* k, const float* v, float* out_w, float* out_u,
                            void* workspace, size_t workspace_bytes, int P, int D, int N, int M, int C,
                            int ns, const float* shifts, const float* weights, cudaStream_t stream)
{
    const int MQ = ns ? ns * M : M;                 // queries per segment
    AbsFwdWs ws(workspace, P, D, N, MQ, C);
    if (!ws_ok(workspace, workspace_bytes, ws.bytes)) return QLKA_ERR_WORKSPACE;
    const int C4 = round4(C), nseg = P * D;
    const bool full = out_u != nullptr;
    float A = 1.0f, Bq = 0.0f;
    if (ns) { A = 0.0f; for (int s = 0; s < ns; s++) { A += weights[s]; Bq += weights[s] * shifts[s] * (float)D; } }

    const float* rows = v;
    float*       out  = out_w;
    if (C4 != C) {
        CU(launch_pad_rows(v, ws.vpad, (long long)P * N, C, C4, stream));
        rows = ws.vpad; out = ws.opad;
    }
    // rank-1 part: out = k_total - qsum * vsum, out_u = ksum_raw - N * qsum (weighted over the shifts when folded)
    CU(launch_colsum_d(q, ws.qsum, P, D, M, stream));
    CU(launch_colsum_d(k, ws.ksumd, P, D, N, stream));
    CU(cudaMemsetAsync(ws.vsum, 0, sizeof(float) * ((size_t)P * C4 * 2 + P), stream));
    CU(launch_rowstat(rows, ws.ksumd, ws.vsum, ws.ktot, ws.ksr, P, N, C4, stream));
    CU(launch_abs_init(ws.ktot, ws.vsum, ws.qsum, ws.ksr, out, out_u, P, M, C4, N, A, Bq, stream));

    SortArgs s = sort_args(ws.rec, k, q, nseg, D, N, MQ, MODE_ABS, full ? SCAL_UNIT : SCAL_NONE);
    s.out_u = out_u; s.rows_coef = 1;
    if (ns) { s.fold = M; for (int i = 0; i < ns; i++) { s.shift[i] = shifts[i]; s.wgt[i] = weights[i]; } }
    CU(launch_sort_rank(s, ws.rec, stream));

    WalkArgs w = walk_args(ws.rec, rows, nseg, D, N, MQ, C4);
    w.out = out; w.Mrows = M; w.agg = ws.agg;
    CU(prefix_walk_chunked(w, EMIT_ROWS, P, stream));

    if (C4 != C) CU(launch_unpad_rows(out, out_w, (long long)P * M, C, C4, stream));
    return QLKA_OK;
}

int qlka_weighted_abs_sum_forward(const float* q, const float* k, const float* v,
                                  float* out_w, float* out_u, void* workspace, size_t workspace_bytes,
                                  int P, int D, int N, int M, int C, int path, qlka_stream_t stream_)
{
    int st = check_dims(P, D, N, M, C);
    if (st) return st;
    if (path < -1 || path > 1) return QLKA_ERR_PATH;
    if (path == 1 && (N > 4096 || M > 4096)) return QLKA_ERR_FUSED_UNAVAILABLE;
    if (!q || !k || !v || !out_w) return QLKA_ERR_NULL;
    if (!aligned16(v, out_w)) return QLKA_ERR_ALIGNMENT;
    return abs_forward_impl(q, k, v, out_w, out_u, workspace, workspace_bytes, P, D, N, M, C, 0, nullptr, nullptr,
                            reinterpret_cast<cudaStream_t>(stream_));
}

int qlka_abs_shifted_forward_workspace_bytes(int P, int D, int N, int M, int C, int n_shifts, size_t* bytes) {
    if (!bytes) return QLKA_ERR_NULL;
    if (n_shifts < 1 || n_shifts > 4) return QLKA_ERR_BAD_SHAPE;
    int st = check_dims(P, D, N, M, C);
    if (st) return st;
    if ((long long)n_shifts * M > SMALL_MAX || N > SMALL_MAX) return QLKA_ERR_UNSUPPORTED;
    *bytes = AbsFwdWs(nullptr, P, D, N, n_shifts * M, C).bytes;
    return QLKA_OK;
}

int qlka_weighted_abs_sum_shifted_forward(const float* q, const float* k, const float* v,
                                          float* out_w, float* out_u, const float* shifts, const float* weights, int n_shifts,
                                          void* workspace, size_t workspace_bytes,
                                          int P, int D, int N, int M, int C, qlka_stream_t stream_)
{
    if (n_shifts < 1 || n_shifts > 4) return QLKA_ERR_BAD_SHAPE;
    int st = check_dims(P, D, N, M, C);
    if (st) return st;
    if ((long long)n_shifts * M > SMALL_MAX || N > SMALL_MAX) return QLKA_ERR_UNSUPPORTED;
    if (!q || !k || !v || !out_w || !shifts || !weights) return QLKA_ERR_NULL;
    if (!aligned16(v, out_w)) return QLKA_ERR_ALIGNMENT;
    return abs_forward_impl(q, k, v, out_w, out_u, workspace, workspace_bytes, P, D, N, M, C, n_shifts, shifts, weights,
                            reinterpret_cast<cudaStream_t>(stream_));
}

// ---------------------------------------------------------------- abs backward
int qlka_abs_backward_workspace_bytes(int P, int D, int N, int M, int C, size_t* bytes) {
    if (!bytes) return QLKA_ERR_NULL;
    int st = check_dims(P, D, N, M, C);
    if (st) return st;
    *bytes = AbsBwdWs(nullptr, P, D, N, M, C).bytes;
    return QLKA_OK;
}

int qlka_weighted_abs_sum_backward(const float* q, const float* k, const float* v,
                                   const float* g_w, const float* g_u,
                                   float* grad_q, float* grad_k, float* grad_v,
                                   void* workspace, size_t workspace_bytes,
                                   int P, int D, int N, int M, int C, qlka_stream_t stream_)
{
    int st = check_dims(P, D, N, M, C);
    if (st) return st;
    if (!q || !k || !v || !g_w || !grad_q || !grad_k || !grad_v) return QLKA_ERR_NULL;
    if (!aligned16(v, g_w, grad_v)) return QLKA_ERR_ALIGNMENT;
    AbsBwdWs ws(workspace, P, D, N, M, C);
    if (!ws_ok(workspace, workspace_bytes, ws.bytes)) return QLKA_ERR_WORKSPACE;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    const int C4 = round4(C), nseg = P * D;
    const bool full = g_u != nullptr;

    const float* vrows = v;
    const float* grows = g_w;
    float*       gv    = grad_v;
    if (C4 != C) {
        CU(launch_pad_rows(v, ws.vpad, (long long)P * N, C, C4, stream));
        CU(launch_pad_rows(g_w, ws.gpad, (long long)P * M, C, C4, stream));
        vrows = ws.vpad; grows = ws.gpad; gv = ws.gvpad;
    }
    float* vsum     = ws.sums;
    float* gwsum    = vsum + (size_t)P * C4;
    float* qtotg    = gwsum + (size_t)P * C4;
    float* gu_total = qtotg + (size_t)P * C4;
    CU(launch_colsum_d(q, ws.qsumd, P, D, M, stream));
    CU(launch_colsum_d(k, ws.ksumd, P, D, N, stream));
    CU(cudaMemsetAsync(ws.sums, 0, sizeof(float) * ((size_t)P * C4 * 3 + P), stream));
    CU(launch_rowstat(vrows, nullptr, vsum, nullptr, nullptr, P, N, C4, stream));
    CU(launch_rowstat(grows, ws.qsumd, gwsum, qtotg, nullptr, P, M, C4, stream));
    if (full) CU(launch_vecsum(g_u, gu_total, P, M, stream));

    {   // grad_q: queries q walk the key stream k; prefix of v rows contracted with g_w rows
        SortArgs s = sort_args(ws.rec, k, q, nseg, D, N, M, MODE_SGN, full ? SCAL_RANK : SCAL_NONE);
        s.uq = g_u;
        CU(launch_sort_rank(s, ws.rec, stream));
        WalkArgs w = walk_args(ws.rec, vrows, nseg, D, N, M, C4);
        w.g = grows; w.wtotal = vsum; w.out_s = grad_q; w.agg = ws.agg;
        CU(prefix_walk_chunked(w, EMIT_DOT, P, stream));
    }
    {   // roles swapped: queries k walk the stream q whose rows are g_w
        SortArgs s = sort_args(ws.rec, q, k, nseg, D, M, N, MODE_ABS, full ? SCAL_PREFIX : SCAL_NONE);
        s.us = g_u; s.us_total = gu_total;
        CU(launch_sort_rank(s, ws.rec, stream));
        // one walk for both: grad_v = abs sum with keys q, weights g_w, evaluated at the keys k (row reductions on
        // top of its rank-1 initial value); grad_k = prefix of g_w rows contracted with v rows (+ the g_u term in e1)
        CU(launch_abs_init(qtotg, gwsum, ws.ksumd, nullptr, gv, nullptr, P, N, C4, M, 1.0f, 0.0f, stream));
        WalkArgs w = walk_args(ws.rec, grows, nseg, D, M, N, C4);
        w.g = vrows; w.wtotal = gwsum; w.out_s = grad_k; w.out = gv; w.agg = ws.agg;
        CU(prefix_walk_chunked(w, EMIT_BOTH, P, stream));
    }
    if (C4 != C) CU(launch_unpad_rows(gv, grad_v, (long long)P * N, C, C4, stream));
    return QLKA_OK;
}

// ---------------------------------------------------------------- sgn
int qlka_sgn_forward_workspace_bytes(int P, int D, int N, int M, int C, size_t* bytes) {
    return qlka_abs_backward_workspace_bytes(P, D, N, M, C, bytes);
}

int qlka_weighted_sgn_sum_forward(const float* q, const float* k, const float* v, const float* g,
                                  float* out, void* workspace, size_t workspace_bytes,
                                  int P, int D, int N, int M, int C, qlka_stream_t stream_)
{
    int st = check_dims(P, D, N, M, C);
    if (st) return st;
    if (!q || !k || !v || !g || !out) return QLKA_ERR_NULL;
    if (!aligned16(v, g)) return QLKA_ERR_ALIGNMENT;
    AbsBwdWs ws(workspace, P, D, N, M, C);
    if (!ws_ok(workspace, workspace_bytes, ws.bytes)) return QLKA_ERR_WORKSPACE;
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    const int C4 = round4(C), nseg = P * D;

    const float* vrows = v;
    const float* grows = g;
    if (C4 != C) {
        CU(launch_pad_rows(v, ws.vpad, (long long)P * N, C, C4, stream));
        CU(launch_pad_rows(g, ws.gpad, (long long)P * M, C, C4, stream));
        vrows = ws.vpad; grows = ws.gpad;
    }
    float* vsum = ws.sums;
    CU(cudaMemsetAsync(vsum, 0, sizeof(float) * (size_t)P * C4, stream));
    CU(launch_rowstat(vrows, nullptr, vsum, nullptr, nullptr, P, N, C4, stream));

    SortArgs s = sort_args(ws.rec, k, q, nseg, D, N, M, MODE_SGN, SCAL_NONE);
    CU(launch_sort_rank(s, ws.rec, stream));
    WalkArgs w = walk_args(ws.rec, vrows, nseg, D, N, M, C4);
    w.g = grows; w.wtotal = vsum; w.out_s = out; w.sign = -1.0f; w.agg = ws.agg;
    CU(prefix_walk_chunked(w, EMIT_DOT, P, stream));
    return QLKA_OK;
}

// ---------------------------------------------------------------- diagnostic
int qlka_sort_rank_workspace_bytes(int P, int D, int N, int M, size_t* bytes) {
    if (!bytes) return QLKA_ERR_NULL;
    int st = check_dims(P, D, N, M, 1);
    if (st) return st;
    *bytes = sizeof(float) * 2 * (size_t)P * D * (N + 1) + 1024
           + ((N > SMALL_MAX || M > SMALL_MAX) ? sort_rank_large_scratch_bytes(P * D, N, M) : 0);
    return QLKA_OK;
}

int qlka_sort_rank_records(const float* x, const float* y,
                           uint32_t* xperm, float* xval, uint32_t* yrec, uint32_t* mstart,
                           void* workspace, size_t workspace_bytes,
                           int P, int D, int N, int M, int mode, qlka_stream_t stream_)
{
    int st = check_dims(P, D, N, M, 1);
    if (st) return st;
    if (!x || !y || !xperm || !xval || !yrec || !mstart) return QLKA_ERR_NULL;
    if (mode != MODE_LAPLACE && mode != MODE_ABS) return QLKA_ERR_PATH;
    size_t need = 0;
    qlka_sort_rank_workspace_bytes(P, D, N, M, &need);
    if (!ws_ok(workspace, workspace_bytes, need)) return QLKA_ERR_WORKSPACE;
    Bump b(workspace);
    Records r;
    r.xperm = xperm; r.xval = xval; r.yrec = reinterpret_cast<uint4*>(yrec); r.mstart = mstart;
    r.su0 = b.take<float>((size_t)P * D * (N + 1));
    r.su1 = b.take<float>((size_t)P * D * (N + 1));
    r.large = (N > SMALL_MAX || M > SMALL_MAX) ? b.take<unsigned char>(sort_rank_large_scratch_bytes(P * D, N, M)) : nullptr;
    SortArgs s = sort_args(r, x, y, P * D, D, N, M, mode, SCAL_NONE);
    CU(launch_sort_rank(s, r, reinterpret_cast<cudaStream_t>(stream_)));
    return QLKA_OK;
}

}  // extern "C"

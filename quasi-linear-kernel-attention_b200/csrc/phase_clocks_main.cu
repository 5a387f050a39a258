// Diagnostic program, not part of the library: weighs the phases of the shared-memory sort/rank kernel.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -DQLKA_PHASE_CLOCKS -o sort_phase_clocks phase_clocks_main.cu
//   ./sort_phase_clocks [heads = 12] [D = 64] [N = M = 16384]
//
// Compiles sort_rank.cu with its phase marks switched on (every mark adds a block-wide barrier, so the
// instrumented kernel is a little slower than the shipped one), runs it on seeded Gaussian keys and queries
// scaled by 2 (the benchmark's distribution) in Laplace mode with the unit-column side channel, and prints
// the share of each phase in the cycles of thread 0, summed over all CTAs.
#include "sort_rank.cu"

#include <cstdio>
#include <cstdlib>

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); return 1; } } while (0)

__global__ void fill_gauss(float* x, long long n, unsigned long long seed, float scale) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= n) return;
    unsigned long long h = (unsigned long long)i * 0x9E3779B97F4A7C15ull + seed;
    h ^= h >> 30; h *= 0xBF58476D1CE4E5B9ull; h ^= h >> 27; h *= 0x94D049BB133111EBull; h ^= h >> 31;
    const float u1 = ((unsigned)(h >> 40) + 1.0f) * (1.0f / 16777217.0f), u2 = (unsigned)(h & 0xffffff) * (1.0f / 16777216.0f);
    x[i] = scale * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
}

int main(int argc, char** argv) {
    using namespace qlka;
    const int P = argc > 1 ? atoi(argv[1]) : 12, D = argc > 2 ? atoi(argv[2]) : 64, N = argc > 3 ? atoi(argv[3]) : 16384, M = N;
    if (N < 1 || N > 16384) { printf("N must be in [1, 16384]\n"); return 1; }
    const int nseg = P * D;
    SortArgs a{};
    float *x, *y, *out_u;
    CK(cudaMalloc(&x, sizeof(float) * (size_t)nseg * N));
    CK(cudaMalloc(&y, sizeof(float) * (size_t)nseg * M));
    CK(cudaMalloc(&out_u, sizeof(float) * (size_t)P * M));
    CK(cudaMalloc(&a.xperm, sizeof(uint32_t) * (size_t)nseg * npad(N)));
    CK(cudaMalloc(&a.xval, sizeof(float) * (size_t)nseg * xstride(N)));
    CK(cudaMalloc(&a.yrec, sizeof(uint4) * (size_t)nseg * (M + 1)));
    CK(cudaMalloc(&a.mstart, sizeof(uint32_t) * (size_t)nseg * mstride(N)));
    CK(cudaMalloc(&a.su0, sizeof(float) * (size_t)nseg * (N + 1)));
    CK(cudaMalloc(&a.su1, sizeof(float) * (size_t)nseg * (N + 1)));
    CK(cudaMemset(out_u, 0, sizeof(float) * (size_t)P * M));
    fill_gauss<<<(unsigned)(((long long)nseg * N + 255) / 256), 256>>>(x, (long long)nseg * N, 1, 2.0f);
    fill_gauss<<<(unsigned)(((long long)nseg * M + 255) / 256), 256>>>(y, (long long)nseg * M, 2, 2.0f);
    CK(cudaDeviceSynchronize());
    a.x = x; a.y = y; a.out_u = out_u;
    a.nseg = nseg; a.D = D; a.N = N; a.M = M; a.mode = MODE_LAPLACE; a.scal = SCAL_UNIT;

    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    for (int i = 0; i < 3; i++) CK(launch_sort_rank_small(a, 0));
    CK(cudaDeviceSynchronize());
    unsigned long long zero[16] = {};
    CK(cudaMemcpyToSymbol(g_phase_clocks, zero, sizeof(zero)));
    const int reps = 5;
    CK(cudaEventRecord(e0));
    for (int i = 0; i < reps; i++) CK(launch_sort_rank_small(a, 0));
    CK(cudaEventRecord(e1));
    CK(cudaDeviceSynchronize());
    float ms = 0.0f;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    unsigned long long clk[16];
    CK(cudaMemcpyFromSymbol(clk, g_phase_clocks, sizeof(clk)));
    // marks in the order the kernel passes them
    const int   order[9] = {0, 1, 2, 3, 4, 7, 8, 5, 6};
    const char* names[9] = {"load keys", "radix sort of the keys (4 passes)", "sorted keys to floats, xperm out, bucket index", "decays and scalar scans, xval / su out",
                            "rank search", "rank histogram, scan, mstart, positions", "scalar side channel (out_u / out_s)",
                            "values and indices to record positions", "records built and written"};
    double total = 0.0;
    for (int i = 0; i < 9; i++) total += (double)clk[order[i]];
    printf("%d segments of %d keys and %d queries: %.3f ms per launch (instrumented build)\n", nseg, N, M, ms / reps);
    for (int i = 0; i < 9; i++)
        printf("  %-44s %6.1f %%  %9.0f cycles per segment\n", names[i], 100.0 * clk[order[i]] / total, (double)clk[order[i]] / ((double)nseg * reps));
    return 0;
}

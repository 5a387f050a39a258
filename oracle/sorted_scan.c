/* TEST INFRASTRUCTURE ONLY - CPU restatement of the reference's sorted-scan algorithm.
 *
 * The product (the CUDA library) never links or calls this file; it exists so that the
 * tests can check the GPU results at sizes where the O(N^2) definition is too slow.
 *
 * The reference evaluates, per (p = batch*head, d = feature dim), the sums over keys on
 * either side of a query from prefix / suffix scans over the keys in ascending order:
 *
 *   Laplace  (Weighted_Laplace_Sum/csrc/laplace_kernels.cu:5-13): with sorted keys
 *            k_1 <= ... <= k_N,  L_j = exp(-(k_j - k_{j-1})) L_{j-1} + v_j  and
 *            R_j = exp(-(k_{j+1} - k_j)) R_{j+1} + v_j; a query with
 *            k_j < q <= k_{j+1} receives exp(-(q - k_j)) L_j + exp(-(k_{j+1} - q)) R_{j+1}
 *            (a key equal to the query counts on the R side).
 *   abs      (Weighted_Abs_Sum/csrc/abs_kernels.cu:9-18): prefix sums PV = sum_{k<q} v and
 *            PK = sum_{k<q} k v give sum_n |k_n - q| v_n = q (PV - SV) - (PK - SK) with the
 *            suffixes SV, SK taken as totals minus prefixes.
 *   sgn / abs backward (Weighted_Abs_Sum/csrc/sgn_kernels.cu:8-15,
 *            Weighted_Abs_Sum/csrc/binding.cpp:242-245): grad_q = sum_c g_w (2 PV - Vtot)
 *            + g_u (2 rank - N); grad_k the same with the roles of q and k swapped;
 *            grad_v the abs sum with q as keys and g_w as weights. A tie belongs to the
 *            ">=" side in both walks, i.e. sub-gradient -1.
 *
 * Everything is accumulated in double. Written from those formulas, not from the kernels.
 * Parity pin: tests/test_oracle.py checks this file against oracle/direct.py (fp64 O(N^2))
 * and, through it, against the reference's own Python outputs in tests/golden/.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

typedef struct { float key; int idx; } item_t;

static int cmp_item(const void* a, const void* b) {
    const item_t* x = (const item_t*)a; const item_t* y = (const item_t*)b;
    if (x->key < y->key) return -1;
    if (x->key > y->key) return 1;
    return (x->idx > y->idx) - (x->idx < y->idx);
}

/* ascending order of a[0..n) into it[] */
static void sort_items(const float* a, int n, item_t* it) {
    for (int i = 0; i < n; i++) { it[i].key = a[i]; it[i].idx = i; }
    qsort(it, (size_t)n, sizeof(item_t), cmp_item);
}

/* number of sorted keys strictly below x */
static int rank_below(const item_t* it, int n, float x) {
    int lo = 0, hi = n;
    while (lo < hi) { int mid = (lo + hi) >> 1; if (it[mid].key < x) lo = mid + 1; else hi = mid; }
    return lo;
}

int oracle_laplace_forward(const float* q, const float* k, const float* v,
                           double* out_w, double* out_u,
                           int P, int D, int N, int M, int C)
{
    memset(out_w, 0, sizeof(double) * (size_t)P * M * C);
    memset(out_u, 0, sizeof(double) * (size_t)P * M);
    int fail = 0;
    #pragma omp parallel for schedule(dynamic)
    for (int p = 0; p < P; p++) {
        item_t* it = (item_t*)malloc(sizeof(item_t) * (size_t)N);
        /* L[(j+1)*(C+1) + c]: state after key j (relative to key j); row 0 is the empty prefix.
           R[j*(C+1) + c]: state at key j (relative to key j); row N is the empty suffix. Channel C is v == 1. */
        const int C1 = C + 1;
        double* L = (double*)malloc(sizeof(double) * (size_t)(N + 1) * C1);
        double* R = (double*)malloc(sizeof(double) * (size_t)(N + 1) * C1);
        if (!it || !L || !R) { fail = 1; free(it); free(L); free(R); continue; }
        for (int d = 0; d < D; d++) {
            const float* kk = k + ((size_t)p * D + d) * N;
            const float* qq = q + ((size_t)p * D + d) * M;
            sort_items(kk, N, it);
            for (int c = 0; c < C1; c++) { L[c] = 0.0; R[(size_t)N * C1 + c] = 0.0; }
            for (int j = 0; j < N; j++) {
                double a = j ? exp(-((double)it[j].key - (double)it[j - 1].key)) : 0.0;
                const float* vr = v + ((size_t)p * N + it[j].idx) * C;
                for (int c = 0; c < C; c++) L[(size_t)(j + 1) * C1 + c] = a * L[(size_t)j * C1 + c] + vr[c];
                L[(size_t)(j + 1) * C1 + C] = a * L[(size_t)j * C1 + C] + 1.0;
            }
            for (int j = N - 1; j >= 0; j--) {
                double a = (j + 1 < N) ? exp(-((double)it[j + 1].key - (double)it[j].key)) : 0.0;
                const float* vr = v + ((size_t)p * N + it[j].idx) * C;
                for (int c = 0; c < C; c++) R[(size_t)j * C1 + c] = a * R[(size_t)(j + 1) * C1 + c] + vr[c];
                R[(size_t)j * C1 + C] = a * R[(size_t)(j + 1) * C1 + C] + 1.0;
            }
            for (int m = 0; m < M; m++) {
                float  x  = qq[m];
                int    j  = rank_below(it, N, x);            /* keys [0,j) are below x, keys [j,N) are >= x */
                double dq = j > 0 ? exp(-((double)x - (double)it[j - 1].key)) : 0.0;
                double dr = j < N ? exp(-((double)it[j].key - (double)x)) : 0.0;
                double* ow = out_w + ((size_t)p * M + m) * C;
                for (int c = 0; c < C; c++) ow[c] += dq * L[(size_t)j * C1 + c] + dr * R[(size_t)j * C1 + c];
                out_u[(size_t)p * M + m] += dq * L[(size_t)j * C1 + C] + dr * R[(size_t)j * C1 + C];
            }
        }
        free(it); free(L); free(R);
    }
    return fail;
}

/* prefix tables over the sorted stream: PW[(j)*(C+1)+c] = sum_{i<j} w_i[c], PKW = sum_{i<j} key_i w_i[c]; channel C is w == u_i
   (u == NULL -> 1). */
static void prefix_tables(const item_t* it, int n, const float* w, const float* u, int C, double* PW, double* PKW) {
    const int C1 = C + 1;
    for (int c = 0; c < C1; c++) { PW[c] = 0.0; PKW[c] = 0.0; }
    for (int j = 0; j < n; j++) {
        const float* wr = w + (size_t)it[j].idx * C;
        double key = it[j].key;
        for (int c = 0; c < C; c++) {
            PW[(size_t)(j + 1) * C1 + c]  = PW[(size_t)j * C1 + c] + wr[c];
            PKW[(size_t)(j + 1) * C1 + c] = PKW[(size_t)j * C1 + c] + key * wr[c];
        }
        double uu = u ? (double)u[it[j].idx] : 1.0;
        PW[(size_t)(j + 1) * C1 + C]  = PW[(size_t)j * C1 + C] + uu;
        PKW[(size_t)(j + 1) * C1 + C] = PKW[(size_t)j * C1 + C] + key * uu;
    }
}

int oracle_abs_forward(const float* q, const float* k, const float* v,
                       double* out_w, double* out_u,
                       int P, int D, int N, int M, int C)
{
    memset(out_w, 0, sizeof(double) * (size_t)P * M * C);
    memset(out_u, 0, sizeof(double) * (size_t)P * M);
    int fail = 0;
    #pragma omp parallel for schedule(dynamic)
    for (int p = 0; p < P; p++) {
        const int C1 = C + 1;
        item_t* it  = (item_t*)malloc(sizeof(item_t) * (size_t)N);
        double* PW  = (double*)malloc(sizeof(double) * (size_t)(N + 1) * C1);
        double* PKW = (double*)malloc(sizeof(double) * (size_t)(N + 1) * C1);
        if (!it || !PW || !PKW) { fail = 1; free(it); free(PW); free(PKW); continue; }
        for (int d = 0; d < D; d++) {
            const float* kk = k + ((size_t)p * D + d) * N;
            const float* qq = q + ((size_t)p * D + d) * M;
            sort_items(kk, N, it);
            prefix_tables(it, N, v + (size_t)p * N * C, NULL, C, PW, PKW);
            const double* TW = PW + (size_t)N * C1; const double* TK = PKW + (size_t)N * C1;
            for (int m = 0; m < M; m++) {
                double x = qq[m];
                int    j = rank_below(it, N, qq[m]);
                const double* pw = PW + (size_t)j * C1; const double* pk = PKW + (size_t)j * C1;
                double* ow = out_w + ((size_t)p * M + m) * C;
                for (int c = 0; c < C; c++) ow[c] += x * (pw[c] - (TW[c] - pw[c])) - (pk[c] - (TK[c] - pk[c]));
                out_u[(size_t)p * M + m] += x * (pw[C] - (TW[C] - pw[C])) - (pk[C] - (TK[C] - pk[C]));
            }
        }
        free(it); free(PW); free(PKW);
    }
    return fail;
}

/* grad_q (P,D,M), grad_k (P,D,N), grad_v (P,N,C); g_u may be NULL */
int oracle_abs_backward(const float* q, const float* k, const float* v,
                        const float* g_w, const float* g_u,
                        double* grad_q, double* grad_k, double* grad_v,
                        int P, int D, int N, int M, int C)
{
    memset(grad_v, 0, sizeof(double) * (size_t)P * N * C);
    int fail = 0;
    #pragma omp parallel for schedule(dynamic)
    for (int p = 0; p < P; p++) {
        const int C1 = C + 1;
        const int X  = N > M ? N : M;
        item_t* it  = (item_t*)malloc(sizeof(item_t) * (size_t)X);
        double* PW  = (double*)malloc(sizeof(double) * (size_t)(X + 1) * C1);
        double* PKW = (double*)malloc(sizeof(double) * (size_t)(X + 1) * C1);
        float*  zero_u = (float*)calloc((size_t)M, sizeof(float));
        if (!it || !PW || !PKW || !zero_u) { fail = 1; free(it); free(PW); free(PKW); free(zero_u); continue; }
        const float* vp = v + (size_t)p * N * C;
        const float* gp = g_w + (size_t)p * M * C;
        const float* up = g_u ? g_u + (size_t)p * M : zero_u;
        for (int d = 0; d < D; d++) {
            const float* kk = k + ((size_t)p * D + d) * N;
            const float* qq = q + ((size_t)p * D + d) * M;
            /* grad_q: stream = keys with weights v */
            sort_items(kk, N, it);
            prefix_tables(it, N, vp, NULL, C, PW, PKW);
            for (int m = 0; m < M; m++) {
                int j = rank_below(it, N, qq[m]);
                const double* pw = PW + (size_t)j * C1; const double* tw = PW + (size_t)N * C1;
                double acc = 0.0;
                for (int c = 0; c < C; c++) acc += (double)gp[(size_t)m * C + c] * (2.0 * pw[c] - tw[c]);
                acc += (double)up[m] * (2.0 * j - N);
                grad_q[((size_t)p * D + d) * M + m] = acc;
            }
            /* grad_k and grad_v: stream = queries with weights g_w (channel C carries g_u) */
            sort_items(qq, M, it);
            prefix_tables(it, M, gp, up, C, PW, PKW);
            const double* TW = PW + (size_t)M * C1; const double* TK = PKW + (size_t)M * C1;
            for (int n = 0; n < N; n++) {
                double x = kk[n];
                int    j = rank_below(it, M, kk[n]);
                const double* pw = PW + (size_t)j * C1; const double* pk = PKW + (size_t)j * C1;
                double acc = 0.0;
                for (int c = 0; c < C; c++) acc += (double)vp[(size_t)n * C + c] * (2.0 * pw[c] - TW[c]);
                acc += 2.0 * pw[C] - TW[C];
                grad_k[((size_t)p * D + d) * N + n] = acc;
                double* gv = grad_v + ((size_t)p * N + n) * C;
                for (int c = 0; c < C; c++) gv[c] += x * (pw[c] - (TW[c] - pw[c])) - (pk[c] - (TK[c] - pk[c]));
            }
        }
        free(it); free(PW); free(PKW); free(zero_u);
    }
    return fail;
}

/* out[p,d,m] = sum_n s(k-q) <v_n, g_m>, s(0) = +1 */
int oracle_sgn_forward(const float* q, const float* k, const float* v, const float* g,
                       double* out, int P, int D, int N, int M, int C)
{
    int fail = 0;
    #pragma omp parallel for schedule(dynamic)
    for (int p = 0; p < P; p++) {
        const int C1 = C + 1;
        item_t* it  = (item_t*)malloc(sizeof(item_t) * (size_t)N);
        double* PW  = (double*)malloc(sizeof(double) * (size_t)(N + 1) * C1);
        double* PKW = (double*)malloc(sizeof(double) * (size_t)(N + 1) * C1);
        if (!it || !PW || !PKW) { fail = 1; free(it); free(PW); free(PKW); continue; }
        for (int d = 0; d < D; d++) {
            const float* kk = k + ((size_t)p * D + d) * N;
            const float* qq = q + ((size_t)p * D + d) * M;
            sort_items(kk, N, it);
            prefix_tables(it, N, v + (size_t)p * N * C, NULL, C, PW, PKW);
            for (int m = 0; m < M; m++) {
                int j = rank_below(it, N, qq[m]);
                const double* pw = PW + (size_t)j * C1; const double* tw = PW + (size_t)N * C1;
                double acc = 0.0;
                for (int c = 0; c < C; c++) acc += (double)g[((size_t)p * M + m) * C + c] * (tw[c] - 2.0 * pw[c]);
                out[((size_t)p * D + d) * M + m] = acc;
            }
        }
        free(it); free(PW); free(PKW);
    }
    return fail;
}

/*
 * CPU oracle for the EMA scan, forward and backward.  TEST INFRASTRUCTURE ONLY: nothing on the
 * product path may link, import or call this file; it exists so that tests, the smoke check and
 * the CPU-baseline leg of the benchmark have an independent answer to compare against.
 *
 * It restates, in plain C, the sequential recurrences the reference project uses as its own
 * ground truth:
 *   - p-weighted loop   z_t = (1-p_t) z_{t-1} + p_t x_t      kernels/tests/ema/test_ema_scan_fwd.py:25-37
 *                                                            (same loop: main.py:120-131)
 *   - pre-scaled loop   z_t = (1-p_t) z_{t-1} + x_t          kernels/tests/ema_bwd/_ema_full_bwd.py:24-34
 * and the gradients autograd produces through those loops (the reference's backward test,
 * kernels/tests/ema_bwd/_ema_full_bwd.py:56-80), written as the closed-form adjoint recurrence
 *   lambda_t = dy_t + a_{t+1} lambda_{t+1}.
 * Parity is pinned: tests/test_oracle.py checks every function here against fixtures produced by
 * running the reference's loops and autograd (tests/golden/make_golden.py).
 *
 * Layout: x, y, dy, dx are dense [b, L, h, d]; decay is [b, L, h] (mode 0) or [h] (mode 1).
 * convention 0 ("north star"): decay holds a in (0,1); y_t = a y_{t-1} + (1-a) x_t;
 *                              gradients are d/dx and d/da.
 * convention 1 ("reference"):  decay holds A = log a <= 0 and x is the pre-scaled input u;
 *                              y_t = exp(A_t) y_{t-1} + u_t; gradients are d/du and d/dA.
 * acc64 != 0 carries the state in double (used to bound the rounding of the fp32 loops).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

/* Rows (b,h) are independent, so both passes run them on a small pthread pool (this image's gcc
 * has no OpenMP runtime).  ema_oracle_set_threads(0) restores the default: one per online core. */
static int g_threads = 0;

typedef void (*row_fn)(int64_t bi, int64_t hi, void *ctx);
typedef struct { row_fn fn; void *ctx; int64_t rows, h; int tid, nthreads; } row_job;

static void *row_worker(void *p) {
    row_job *j = (row_job *)p;
    for (int64_t r = j->tid; r < j->rows; r += j->nthreads) j->fn(r / j->h, r % j->h, j->ctx);
    return NULL;
}

static void for_each_row(int64_t b, int64_t h, row_fn fn, void *ctx) {
    int n = g_threads > 0 ? g_threads : (int)sysconf(_SC_NPROCESSORS_ONLN);
    const int64_t rows = b * h;
    if (n > rows) n = (int)rows;
    if (n < 1) n = 1;
    if (n > 256) n = 256;
    pthread_t th[256];
    row_job jobs[256];
    for (int i = 0; i < n; ++i) {
        jobs[i] = (row_job){fn, ctx, rows, h, i, n};
        if (i > 0) pthread_create(&th[i], NULL, row_worker, &jobs[i]);
    }
    row_worker(&jobs[0]);
    for (int i = 1; i < n; ++i) pthread_join(th[i], NULL);
}

void ema_oracle_set_threads(int n) { g_threads = n; }

static inline float decay_at(const float *decay, int mode, int64_t bi, int64_t t, int64_t hi,
                             int64_t L, int64_t h) {
    return mode ? decay[hi] : decay[(bi * L + t) * h + hi];
}

int ema_oracle_threads(void) {
    return g_threads > 0 ? g_threads : (int)sysconf(_SC_NPROCESSORS_ONLN);
}

typedef struct {
    const float *x, *decay, *dy;
    float *y, *chunk_states, *final_state, *dx, *ddecay;
    double *head_acc;
    int decay_mode, convention, acc64;
    int64_t b, L, h, d, chunk, C;
} ema_args;

static void fwd_row(int64_t bi, int64_t hi, void *ctx) {
    const ema_args *g = (const ema_args *)ctx;
    const int64_t L = g->L, h = g->h, d = g->d, chunk = g->chunk;
    double *z64 = (double *)calloc((size_t)(d > 0 ? d : 1), sizeof(double));
    float *z32 = (float *)calloc((size_t)(d > 0 ? d : 1), sizeof(float));
    for (int64_t t = 0; t < L; ++t) {
        if (g->chunk_states && t % chunk == 0) {
            float *cs = g->chunk_states + (((bi * h + hi) * g->C) + t / chunk) * d;
            for (int64_t c = 0; c < d; ++c) cs[c] = g->acc64 ? (float)z64[c] : z32[c];
        }
        const float dv = decay_at(g->decay, g->decay_mode, bi, t, hi, L, h);
        const float *xr = g->x + ((bi * L + t) * h + hi) * d;
        float *yr = g->y + ((bi * L + t) * h + hi) * d;
        if (g->acc64) {
            const double a = g->convention ? exp((double)dv) : (double)dv;
            const double p = g->convention ? 1.0 : 1.0 - (double)dv;
            for (int64_t c = 0; c < d; ++c) {
                z64[c] = a * z64[c] + p * (double)xr[c];
                yr[c] = (float)z64[c];
            }
        } else if (g->convention) {
            /* fp32 throughout, in the operation order of the reference's pre-scaled loop */
            const float p = 1.0f - expf(dv);
            for (int64_t c = 0; c < d; ++c) { z32[c] = (1.0f - p) * z32[c] + xr[c]; yr[c] = z32[c]; }
        } else {
            /* fp32 throughout, in the operation order of the reference's p-weighted loop */
            const float p = 1.0f - dv;
            for (int64_t c = 0; c < d; ++c) { z32[c] = (1.0f - p) * z32[c] + p * xr[c]; yr[c] = z32[c]; }
        }
    }
    if (g->final_state) {
        float *fs = g->final_state + (bi * h + hi) * d;
        for (int64_t c = 0; c < d; ++c) fs[c] = g->acc64 ? (float)z64[c] : z32[c];
    }
    free(z64);
    free(z32);
}

/* Forward.  chunk_states (optional) receives the state at the START of every chunk,
 * [b, h, ceil(L/chunk), d] fp32 (all zeros for chunk 0), the quantity the reference's
 * _ema_state_passing_fwd returns (kernels/ema_kernels/ema_state_pass.py:100-120);
 * final_state (optional) is [b, h, d]. */
int ema_oracle_fwd(const float *x, const float *decay, float *y, float *chunk_states,
                   float *final_state, int decay_mode, int convention, int acc64, int64_t b,
                   int64_t L, int64_t h, int64_t d, int64_t chunk) {
    if (b < 0 || L < 0 || h < 0 || d < 0) return -1;
    if (chunk_states && chunk <= 0) return -1;
    ema_args g = {x, decay, NULL, y, chunk_states, final_state, NULL, NULL, NULL, decay_mode,
                  convention, acc64, b, L, h, d, chunk, chunk > 0 ? (L + chunk - 1) / chunk : 0};
    for_each_row(b, h, fwd_row, &g);
    return 0;
}

static void bwd_row(int64_t bi, int64_t hi, void *ctx) {
    const ema_args *g = (const ema_args *)ctx;
    const int64_t L = g->L, h = g->h, d = g->d;
    const int conv = g->convention, acc64 = g->acc64;
    const size_t n = (size_t)(L * d > 0 ? L * d : 1);
    double *yprev = (double *)malloc(n * sizeof(double)); /* y_{t-1} for every t */
    double *lam = (double *)calloc((size_t)(d > 0 ? d : 1), sizeof(double));
    double *z = (double *)calloc((size_t)(d > 0 ? d : 1), sizeof(double));
    for (int64_t t = 0; t < L; ++t) {
        const float dv = decay_at(g->decay, g->decay_mode, bi, t, hi, L, h);
        const double a = conv ? exp((double)dv) : (double)dv;
        const double p = conv ? 1.0 : 1.0 - a;
        const float *xr = g->x + ((bi * L + t) * h + hi) * d;
        for (int64_t c = 0; c < d; ++c) {
            yprev[t * d + c] = z[c];
            z[c] = a * z[c] + p * (double)xr[c];
            if (!acc64) z[c] = (double)(float)z[c];
        }
    }
    double hsum = 0.0;
    for (int64_t t = L - 1; t >= 0; --t) {
        const float dv = decay_at(g->decay, g->decay_mode, bi, t, hi, L, h);
        const double a = conv ? exp((double)dv) : (double)dv;
        double a_next = 0.0;
        if (t + 1 < L) {
            const float dn = decay_at(g->decay, g->decay_mode, bi, t + 1, hi, L, h);
            a_next = conv ? exp((double)dn) : (double)dn;
        }
        const float *xr = g->x + ((bi * L + t) * h + hi) * d;
        const float *gr = g->dy + ((bi * L + t) * h + hi) * d;
        float *dxr = g->dx + ((bi * L + t) * h + hi) * d;
        double acc = 0.0;
        for (int64_t c = 0; c < d; ++c) {
            lam[c] = (double)gr[c] + a_next * lam[c];
            if (!acc64) lam[c] = (double)(float)lam[c];
            if (conv) {
                dxr[c] = (float)lam[c];
                acc += lam[c] * yprev[t * d + c];
            } else {
                dxr[c] = (float)((1.0 - a) * lam[c]);
                acc += lam[c] * (yprev[t * d + c] - (double)xr[c]);
            }
        }
        if (conv) acc *= a;
        if (g->decay_mode) hsum += acc;
        else g->ddecay[(bi * L + t) * h + hi] = (float)acc;
    }
    g->head_acc[bi * h + hi] = hsum;
    free(yprev);
    free(lam);
    free(z);
}

/* Backward.  dx is [b,L,h,d]; ddecay is [b,L,h] (mode 0) or [h] (mode 1).
 * convention 0: dx_t = (1-a_t) lambda_t,  da_t = sum_d lambda_t (y_{t-1} - x_t)
 * convention 1: du_t = lambda_t,          dA_t = exp(A_t) sum_d lambda_t y_{t-1}
 * The adjoint and the recomputed forward are carried in double when acc64, else rounded to float
 * every step; reductions over d (and over b,t for per-head decay) accumulate in double. */
int ema_oracle_bwd(const float *x, const float *decay, const float *dy, float *dx, float *ddecay,
                   int decay_mode, int convention, int acc64, int64_t b, int64_t L, int64_t h,
                   int64_t d) {
    if (b < 0 || L < 0 || h < 0 || d < 0) return -1;
    double *head_acc = (double *)calloc((size_t)(b * h > 0 ? b * h : 1), sizeof(double));
    ema_args g = {x, decay, dy, NULL, NULL, NULL, dx, ddecay, head_acc, decay_mode,
                  convention, acc64, b, L, h, d, 0, 0};
    for_each_row(b, h, bwd_row, &g);
    if (decay_mode) {
        for (int64_t hi = 0; hi < h; ++hi) {
            double s = 0.0;
            for (int64_t bi = 0; bi < b; ++bi) s += head_acc[bi * h + hi];
            ddecay[hi] = (float)s;
        }
    }
    free(head_acc);
    return 0;
}

/*
 * CPU restatement of the flash_dism hard path (test infrastructure, NOT product code).
 *
 * Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may
 * link or call this file.  The shipped library never routes through it.
 *
 * Every function restates, in plain C, what the reference defines:
 *   labels      dism_v3/python/flash_dism/reference/dism_v3_ref.py:159-162 (arg-max of x.E^T),
 *               dism_v3/python/flash_dism/kernels/interp_true.py:25-33 (lowest index wins ties)
 *   summary     dism_v3/tests/test_hard_summary.py:37-49, dism_v3/include/summary/hard.cuh:106-125
 *   boundary    dism_v3/tests/test_hard_chunk.py:14-36, dism_v3/src/hard_chunk.cu:19-69
 *   lengths     dism_v3/python/flash_dism/summary.py:8-16 (L = key coordinate - boundary)
 *   LUT         dism_v3/src/hard_forward.cu:9-25
 *   forward     dism_v3/python/flash_dism/reference/dism_v3_ref.py:36-66 with hard=True
 *   backward    dism_v3/python/flash_dism/reference/dism_v3_ref.py:69-132 with hard=True,
 *               dism_v3/docs/HARD_BACKWARD_QUADRATIC.md:60-91 (closed form of the tau gradient)
 *
 * Vectors are float arrays (already rounded to the storage type by the caller) laid out
 * [B,N,H,C]; labels are int32 [B,H,N]; hard flags are bytes [B,H]; accumulation is double.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define LOG_ZERO (-1000000.0f)

/* ---- discretiser ------------------------------------------------------------------ */
/* Canonical accumulation: acc = fl32(acc + fl32(x*e)) over d = 0..D-1, first maximum wins. */
void dism_oracle_labels(const float *x, const float *codebook, int B, int N, int H, int D, int V,
                        int32_t *out) {
    for (int b = 0; b < B; ++b)
        for (int n = 0; n < N; ++n)
            for (int h = 0; h < H; ++h) {
                const float *row = x + (((int64_t)b * N + n) * H + h) * D;
                float best = -INFINITY;
                int arg = 0;
                for (int v = 0; v < V; ++v) {
                    const float *e = codebook + ((int64_t)h * V + v) * D;
                    volatile float acc = 0.f;
                    for (int d = 0; d < D; ++d) {
                        volatile float p = row[d] * e[d];
                        acc = acc + p;
                    }
                    if (v == 0 || acc > best) { best = acc; arg = v; }
                }
                out[((int64_t)b * H + h) * N + n] = arg;
            }
}

/* ---- integer stages ---------------------------------------------------------------- */
/* Strip-local last mismatching key coordinate on the diagonal that ends at (32c+31, j). */
void dism_oracle_summary(const int32_t *iq, const int32_t *ik, const uint8_t *hard, int B, int H,
                         int N, int32_t *out) {
    int C = (N - 1) / 32;
    for (int bh = 0; bh < B * H; ++bh) {
        const int32_t *q = iq + (int64_t)bh * N, *k = ik + (int64_t)bh * N;
        int32_t *o = out + (int64_t)bh * C * N;
        for (int c = 0; c < C; ++c)
            for (int j = 0; j < N; ++j) {
                int32_t r = -1;
                if (hard[bh] && j <= 32 * c + 31)
                    for (int s = 0; s < 32 && j - s >= 0; ++s)
                        if (q[32 * c + 31 - s] != k[j - s]) { r = j - s; break; }
                o[(int64_t)c * N + j] = r;
            }
    }
}

/* boundary[c][j] = max(summary[c][j], boundary[c-1][j-32]); entries right of the strip's last
   row are -1 and are never read (the reference poisons them in its tests). */
void dism_oracle_chunk(const int32_t *summary, int BH, int N, int32_t *out) {
    int C = (N - 1) / 32;
    for (int bh = 0; bh < BH; ++bh) {
        const int32_t *s = summary + (int64_t)bh * C * N;
        int32_t *o = out + (int64_t)bh * C * N;
        for (int c = 0; c < C; ++c)
            for (int j = 0; j < N; ++j) {
                int32_t r = -1;
                if (j <= 32 * c + 31) {
                    r = s[(int64_t)c * N + j];
                    if (c && j >= 32) {
                        int32_t p = o[(int64_t)(c - 1) * N + j - 32];
                        if (p > r) r = p;
                    }
                }
                o[(int64_t)c * N + j] = r;
            }
    }
}

/* Dense match-length field of one (batch, head): L[i][j] for j <= i, 0 elsewhere. */
void dism_oracle_lengths(const int32_t *q, const int32_t *k, int N, int32_t *L) {
    for (int i = 0; i < N; ++i)
        for (int j = 0; j < N; ++j) {
            int32_t v = 0;
            if (j <= i && q[i] == k[j]) v = (i && j ? L[(int64_t)(i - 1) * N + j - 1] : 0) + 1;
            L[(int64_t)i * N + j] = v;
        }
}

/* Single longest earlier match of a symbol stream against itself (iq = ik = s): for every i the
   key j < i with the largest L(i,j), the most recent one on ties, -1 when no symbol matches;
   next[i] = s[j+1].  The reference defines L but no single winner; this tie-break is ours. */
void dism_oracle_longest(const int32_t *s, int N, int32_t *end, int32_t *len, int32_t *next) {
    int32_t *prev = calloc(N + 1, sizeof(int32_t)), *cur = calloc(N + 1, sizeof(int32_t));
    for (int i = 0; i < N; ++i) {
        int32_t best = 0, arg = -1;
        for (int j = 0; j < i; ++j) {
            cur[j + 1] = s[i] == s[j] ? prev[j] + 1 : 0;
            if (cur[j + 1] && cur[j + 1] >= best) { best = cur[j + 1]; arg = j; }
        }
        cur[i + 1] = i + 1; /* diagonal: excluded from the search, needed by the next row */
        cur[0] = 0;
        end[i] = arg; len[i] = best; next[i] = arg >= 0 ? s[arg + 1] : -1;
        int32_t *t = prev; prev = cur; cur = t;
    }
    free(prev); free(cur);
}

/* ---- LUT ----------------------------------------------------------------------------- */
void dism_oracle_lut(const float *tau, int H, int n, float *out) {
    for (int h = 0; h < H; ++h)
        for (int l = 0; l <= n; ++l) {
            float t = tau[h], r = LOG_ZERO;
            if (l > 0) {
                if (t == 0.f) r = log2f((float)l);
                else {
                    float a = fabsf(t);
                    r = (t > 0.f ? (float)l * t : t) * 1.4426950408889634f +
                        log2f(-expm1f(-(float)l * a)) - log2f(-expm1f(-a));
                }
            }
            out[(int64_t)h * (n + 1) + l] = r;
        }
}

/* natural log of W_l = sum_{s=1..l} exp(s tau), and g_l = d ln W_l / d tau, in double */
static void weight_tables(double tau, int n, double *logw, double *g) {
    logw[0] = -INFINITY; g[0] = 0.;
    double a = fabs(tau), lw1 = tau == 0. ? 0. : log(-expm1(-a));
    double s0 = 0., s1 = 0.; /* sum e^{-m a}, sum m e^{-m a}, m = 0..l-1 */
    for (int l = 1; l <= n; ++l) {
        double e = exp(-(double)(l - 1) * a);
        s0 += e; s1 += (double)(l - 1) * e;
        if (tau == 0.) { logw[l] = log((double)l); g[l] = 0.5 * (l + 1); continue; }
        logw[l] = (tau > 0 ? l * tau : tau) + log(-expm1(-(double)l * a)) - lw1;
        /* tau>0: W = e^{l tau} sum_m e^{-m tau}; weights of s = l-m.  tau<0: s = m+1. */
        g[l] = tau > 0 ? l - s1 / s0 : 1. + s1 / s0;
    }
}

/* ---- forward / backward ---------------------------------------------------------------- */
typedef struct {
    const float *sq, *sk, *v, *dout, *tau;
    const int32_t *iq, *ik;
    const uint8_t *hard;
    int B, N, H, R, DV;
    double *out, *lse2, *dsq, *dsk, *dv, *dtau_bh; /* dtau_bh: [B*H] partials */
    int backward;
    int next_task;
    pthread_mutex_t lock;
} Job;

static void run_head(Job *J, int bh) {
    int N = J->N, H = J->H, R = J->R, DV = J->DV, b = bh / H, h = bh % H;
    const int32_t *q = J->iq + (int64_t)bh * N, *k = J->ik + (int64_t)bh * N;
    int64_t stride_r = (int64_t)H * R, stride_v = (int64_t)H * DV;
    const float *sq = J->sq + ((int64_t)b * N * H + h) * R, *sk = J->sk + ((int64_t)b * N * H + h) * R;
    const float *v = J->v + ((int64_t)b * N * H + h) * DV;
    double *out = J->out ? J->out + ((int64_t)b * N * H + h) * DV : NULL;
    double *lse2 = J->lse2 ? J->lse2 + (int64_t)bh * N : NULL;
    if (!J->hard[bh]) {
        for (int i = 0; i < N; ++i) {
            if (out) memset(out + i * stride_v, 0, sizeof(double) * DV);
            if (lse2) lse2[i] = 0.;
        }
        if (J->backward) {
            J->dtau_bh[bh] = 0.;
            for (int i = 0; i < N; ++i) {
                memset(J->dsq + ((int64_t)b * N * H + h) * R + i * stride_r, 0, sizeof(double) * R);
                memset(J->dsk + ((int64_t)b * N * H + h) * R + i * stride_r, 0, sizeof(double) * R);
                memset(J->dv + ((int64_t)b * N * H + h) * DV + i * stride_v, 0, sizeof(double) * DV);
            }
        }
        return;
    }
    double *logw = malloc(sizeof(double) * (N + 1)), *g = malloc(sizeof(double) * (N + 1));
    weight_tables((double)J->tau[h], N, logw, g);
    int32_t *La = calloc(N + 1, sizeof(int32_t)), *Lb = calloc(N + 1, sizeof(int32_t));
    int32_t *hit = malloc(sizeof(int32_t) * N);
    double *acc = malloc(sizeof(double) * DV), *wts = malloc(sizeof(double) * N);
    const float *dO = J->backward ? J->dout + ((int64_t)b * N * H + h) * DV : NULL;
    double *dsq = NULL, *dsk = NULL, *dv = NULL, dtau = 0.;
    if (J->backward) {
        dsq = J->dsq + ((int64_t)b * N * H + h) * R;
        dsk = J->dsk + ((int64_t)b * N * H + h) * R;
        dv = J->dv + ((int64_t)b * N * H + h) * DV;
        for (int i = 0; i < N; ++i) {
            memset(dsq + i * stride_r, 0, sizeof(double) * R);
            memset(dsk + i * stride_r, 0, sizeof(double) * R);
            memset(dv + i * stride_v, 0, sizeof(double) * DV);
        }
    }
    for (int i = 0; i < N; ++i) {
        /* L(i,j) = (q_i == k_j) ? L(i-1,j-1) + 1 : 0; arrays are shifted by one so index 0 is 0 */
        int32_t qi = q[i];
        const int32_t *old = La;
        int32_t *cur = Lb;
        for (int j = 0; j <= i; ++j) cur[j + 1] = qi == k[j] ? old[j] + 1 : 0;
        int hits = 0;
        double zmax = 0.;
        for (int j = 0; j <= i; ++j)
            if (cur[j + 1]) {
                hit[hits++] = j;
                if (logw[cur[j + 1]] > zmax) zmax = logw[cur[j + 1]];
            }
        double den = exp(-zmax);
        for (int t = 0; t < hits; ++t) {
            wts[t] = exp(logw[cur[hit[t] + 1]] - zmax);
            den += wts[t];
        }
        for (int c = 0; c < DV; ++c) acc[c] = 0.;
        const float *sqi = sq + i * stride_r;
        double corr = 0.;
        for (int t = 0; t < hits; ++t) {
            int j = hit[t];
            const float *skj = sk + j * stride_r, *vj = v + j * stride_v;
            double s = 0.;
            for (int r = 0; r < R; ++r) s += (double)sqi[r] * skj[r];
            double p = wts[t] / den;
            for (int c = 0; c < DV; ++c) acc[c] += p * s * vj[c];
            if (J->backward) {
                const float *doi = dO + i * stride_v;
                double e = 0.;
                for (int c = 0; c < DV; ++c) e += (double)doi[c] * vj[c];
                corr += p * s * e;
                for (int c = 0; c < DV; ++c) dv[j * stride_v + c] += p * s * doi[c];
                for (int r = 0; r < R; ++r) {
                    dsq[i * stride_r + r] += p * e * skj[r];
                    dsk[j * stride_r + r] += p * e * sqi[r];
                }
            }
        }
        if (J->backward)
            for (int t = 0; t < hits; ++t) {
                int j = hit[t];
                const float *skj = sk + j * stride_r, *vj = v + j * stride_v, *doi = dO + i * stride_v;
                double s = 0., e = 0.;
                for (int r = 0; r < R; ++r) s += (double)sqi[r] * skj[r];
                for (int c = 0; c < DV; ++c) e += (double)doi[c] * vj[c];
                dtau += wts[t] / den * (s * e - corr) * g[cur[j + 1]];
            }
        if (out) for (int c = 0; c < DV; ++c) out[i * stride_v + c] = acc[c];
        if (lse2) lse2[i] = (zmax + log(den)) / 0.6931471805599453;
        La = cur; Lb = (int32_t *)old;
    }
    if (J->backward) J->dtau_bh[bh] = dtau;
    free(logw); free(g); free(La); free(Lb); free(hit); free(acc); free(wts);
}

static void *worker(void *arg) {
    Job *J = arg;
    for (;;) {
        pthread_mutex_lock(&J->lock);
        int t = J->next_task++;
        pthread_mutex_unlock(&J->lock);
        if (t >= J->B * J->H) return NULL;
        run_head(J, t);
    }
}

static void run_job(Job *J, int threads) {
    pthread_mutex_init(&J->lock, NULL);
    J->next_task = 0;
    if (threads <= 1) { worker(J); return; }
    pthread_t *ids = malloc(sizeof(pthread_t) * threads);
    for (int t = 0; t < threads; ++t) pthread_create(ids + t, NULL, worker, J);
    for (int t = 0; t < threads; ++t) pthread_join(ids[t], NULL);
    free(ids);
}

void dism_oracle_forward(const float *sq, const float *sk, const float *v, const int32_t *iq,
                         const int32_t *ik, const uint8_t *hard, const float *tau, int B, int N,
                         int H, int R, int DV, double *out, double *lse2, int threads) {
    Job J = {.sq = sq, .sk = sk, .v = v, .tau = tau, .iq = iq, .ik = ik, .hard = hard, .B = B,
             .N = N, .H = H, .R = R, .DV = DV, .out = out, .lse2 = lse2, .backward = 0};
    run_job(&J, threads);
}

/* dtau is the gradient with respect to the natural-log coefficient, summed over batch. */
void dism_oracle_backward(const float *sq, const float *sk, const float *v, const float *dout,
                          const int32_t *iq, const int32_t *ik, const uint8_t *hard,
                          const float *tau, int B, int N, int H, int R, int DV, double *dsq,
                          double *dsk, double *dv, double *dtau, int threads) {
    double *partial = calloc((size_t)B * H, sizeof(double));
    Job J = {.sq = sq, .sk = sk, .v = v, .dout = dout, .tau = tau, .iq = iq, .ik = ik,
             .hard = hard, .B = B, .N = N, .H = H, .R = R, .DV = DV, .dsq = dsq, .dsk = dsk,
             .dv = dv, .dtau_bh = partial, .backward = 1};
    run_job(&J, threads);
    for (int h = 0; h < H; ++h) {
        dtau[h] = 0.;
        for (int b = 0; b < B; ++b) dtau[h] += partial[b * H + h];
    }
    free(partial);
}

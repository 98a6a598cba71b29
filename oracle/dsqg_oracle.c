/* CPU oracle for DSQG attention in plain C -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A loop-nest restatement of the DWARF reference's DSQG math with double-precision
 * accumulation, used by the tests as a memory-light "ground truth" at sizes where the
 * PyTorch restatement (oracle/dsqg_oracle.py) would materialise tens of gigabytes.
 * Nothing shipped in dwarf_b200 links or calls this file.
 *
 * Reference statements followed (paths inside the DWARF repository):
 *   forward   kernels/dsqg_attention_v3.py:543-561 (_reference_v3), and the per-row
 *             form of the same math in kernels/dsqg_attention_v3.py:101-163
 *   backward  kernels/dsqg_attention_v3.py:236-271 (dQ, dpos_bias, dscale_embed) and
 *             kernels/dsqg_attention_v3.py:318-345 (dK, dV)
 *   gain      train/train_2048_condU.py:187 (out *= if_gain[h])
 *
 * Parity status: pinned through tests/test_oracle_golden.py, which checks these
 * functions against the committed outputs of the reference's own functions.
 *
 * Layout: q,k,v,out,dout,dq,dk,dv are [B,H,N,D] row-major float; pos_bias [J,H];
 * scale_embed [J,D] (may be NULL); head_gain [H] (may be NULL); offsets [J] ascending.
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

/* Minimal parallel-for over (batch, head) pairs with pthreads: each worker takes the
 * indices i = tid, tid + T, ...  Thread count = DSQG_ORACLE_THREADS or the online cores. */
typedef void (*bh_fn)(int bh, void *ctx);
typedef struct { bh_fn fn; void *ctx; int tid, T, n; } worker_arg;
static void *worker(void *p) {
    worker_arg *a = (worker_arg *)p;
    for (int i = a->tid; i < a->n; i += a->T) a->fn(i, a->ctx);
    return NULL;
}
static void parallel_for(int n, bh_fn fn, void *ctx) {
    long T = sysconf(_SC_NPROCESSORS_ONLN);
    const char *e = getenv("DSQG_ORACLE_THREADS");
    if (e) T = atol(e);
    if (T < 1) T = 1;
    if (T > n) T = n;
    if (T > 256) T = 256;
    pthread_t th[256]; worker_arg args[256];
    for (int t = 0; t < T; ++t) {
        args[t] = (worker_arg){fn, ctx, t, (int)T, n};
        if (t > 0) pthread_create(&th[t], NULL, worker, &args[t]);
    }
    if (T > 0) worker(&args[0]);
    for (int t = 1; t < T; ++t) pthread_join(th[t], NULL);
}

typedef struct {
    const float *q, *k, *v, *pos_bias, *scale_embed, *head_gain, *dout;
    const int32_t *offsets;
    int J, B, H, N, D;
    float *out, *lse, *dq, *dk, *dv;
    double *dpb_d, *dse_d, *dg_d;
} ctx_t;

static double dotd(const float *a, const float *b, int D) {
    double s = 0.0;
    for (int d = 0; d < D; ++d) s += (double)a[d] * (double)b[d];
    return s;
}

/* Forward.  lse may be NULL.  A row with no valid tap gives out = 0 and lse = -inf. */
static void fwd_bh(int bh, void *vc) {
    const ctx_t *c = (const ctx_t *)vc;
    const float *q = c->q, *k = c->k, *v = c->v, *pos_bias = c->pos_bias,
                *scale_embed = c->scale_embed, *head_gain = c->head_gain;
    const int32_t *offsets = c->offsets;
    const int J = c->J, H = c->H, N = c->N, D = c->D;
    float *out = c->out, *lse = c->lse;
    const double sc = 1.0 / sqrt((double)D);
    {
        const int h = bh % H;
        const float *qb = q + (size_t)bh * N * D, *kb = k + (size_t)bh * N * D,
                    *vb = v + (size_t)bh * N * D;
        double *s = (double *)malloc(sizeof(double) * (size_t)J);
        double *acc = (double *)malloc(sizeof(double) * (size_t)D);
        for (int n = 0; n < N; ++n) {
            double m = -INFINITY;
            for (int j = 0; j < J; ++j) {
                int src = n - offsets[j];
                if (src < 0) { s[j] = -INFINITY; continue; }
                double x = dotd(qb + (size_t)n * D, kb + (size_t)src * D, D) * sc + pos_bias[j * H + h];
                if (scale_embed) x += dotd(qb + (size_t)n * D, scale_embed + (size_t)j * D, D) * sc;
                s[j] = x;
                if (x > m) m = x;
            }
            double l = 0.0;
            for (int d = 0; d < D; ++d) acc[d] = 0.0;
            for (int j = 0; j < J; ++j) {
                if (s[j] == -INFINITY) continue;
                double p = exp(s[j] - m);
                l += p;
                const float *vr = vb + (size_t)(n - offsets[j]) * D;
                for (int d = 0; d < D; ++d) acc[d] += p * vr[d];
            }
            double g = head_gain ? head_gain[h] : 1.0;
            for (int d = 0; d < D; ++d)
                out[((size_t)bh * N + n) * D + d] = (float)(l > 0.0 ? g * acc[d] / l : 0.0);
            if (lse) lse[(size_t)bh * N + n] = (float)(l > 0.0 ? m + log(l) : -INFINITY);
        }
        free(s); free(acc);
    }
}

int dsqg_oracle_fwd(const float *q, const float *k, const float *v, const float *pos_bias,
                    const float *scale_embed, const float *head_gain, const int32_t *offsets,
                    int J, int B, int H, int N, int D, float *out, float *lse) {
    ctx_t c = {0};
    c.q = q; c.k = k; c.v = v; c.pos_bias = pos_bias; c.scale_embed = scale_embed;
    c.head_gain = head_gain; c.offsets = offsets; c.J = J; c.B = B; c.H = H; c.N = N; c.D = D;
    c.out = out; c.lse = lse;
    parallel_for(B * H, fwd_bh, &c);
    return 0;
}

/* Backward.  dse / dgain may be NULL when scale_embed / head_gain are NULL.
 * dpb [J,H], dse [J,D], dgain [H] are written (not accumulated into). */
static void bwd_bh(int bh, void *vc) {
    const ctx_t *c = (const ctx_t *)vc;
    const float *q = c->q, *k = c->k, *v = c->v, *pos_bias = c->pos_bias,
                *scale_embed = c->scale_embed, *head_gain = c->head_gain, *dout = c->dout;
    const int32_t *offsets = c->offsets;
    const int J = c->J, H = c->H, N = c->N, D = c->D;
    float *dq = c->dq, *dk = c->dk, *dv = c->dv;
    double *dpb_d = c->dpb_d, *dse_d = c->dse_d, *dg_d = c->dg_d;
    const double sc = 1.0 / sqrt((double)D);
    {
        const int h = bh % H;
        const size_t base = (size_t)bh * N * D;
        const float *qb = q + base, *kb = k + base, *vb = v + base, *dob = dout + base;
        double *dkd = (double *)calloc((size_t)N * D, sizeof(double));
        double *dvd = (double *)calloc((size_t)N * D, sizeof(double));
        double *s = (double *)malloc(sizeof(double) * (size_t)J);
        double *p = (double *)malloc(sizeof(double) * (size_t)J);
        double *dp = (double *)malloc(sizeof(double) * (size_t)J);
        double *o = (double *)malloc(sizeof(double) * (size_t)D);
        double *dqd = (double *)malloc(sizeof(double) * (size_t)D);
        const double g = head_gain ? head_gain[h] : 1.0;
        for (int n = 0; n < N; ++n) {
            const float *qr = qb + (size_t)n * D, *dor = dob + (size_t)n * D;
            double m = -INFINITY;
            for (int j = 0; j < J; ++j) {
                int src = n - offsets[j];
                if (src < 0) { s[j] = -INFINITY; continue; }
                double x = dotd(qr, kb + (size_t)src * D, D) * sc + pos_bias[j * H + h];
                if (scale_embed) x += dotd(qr, scale_embed + (size_t)j * D, D) * sc;
                s[j] = x;
                if (x > m) m = x;
            }
            double l = 0.0;
            for (int j = 0; j < J; ++j) { p[j] = (s[j] == -INFINITY) ? 0.0 : exp(s[j] - m); l += p[j]; }
            for (int d = 0; d < D; ++d) { o[d] = 0.0; dqd[d] = 0.0; }
            if (l > 0.0) {
                for (int j = 0; j < J; ++j) {
                    p[j] /= l;
                    if (p[j] == 0.0) continue;
                    const float *vr = vb + (size_t)(n - offsets[j]) * D;
                    for (int d = 0; d < D; ++d) o[d] += p[j] * vr[d];
                }
            } else {
                for (int j = 0; j < J; ++j) p[j] = 0.0;
            }
            /* out = g * o ; d(o) = g * dout ; dgain += dout . o */
            double delta = 0.0, dg = 0.0;
            for (int d = 0; d < D; ++d) { dg += (double)dor[d] * o[d]; }
            delta = g * dg;
            dg_d[bh] += dg;
            for (int j = 0; j < J; ++j) {
                int src = n - offsets[j];
                if (src < 0) continue;
                const float *kr = kb + (size_t)src * D, *vr = vb + (size_t)src * D;
                dp[j] = g * dotd(dor, vr, D);
                double ds = p[j] * (dp[j] - delta);
                dpb_d[(size_t)bh * J + j] += ds;
                for (int d = 0; d < D; ++d) {
                    dqd[d] += ds * sc * kr[d];
                    dkd[(size_t)src * D + d] += ds * sc * qr[d];
                    dvd[(size_t)src * D + d] += p[j] * g * dor[d];
                }
                if (scale_embed) {
                    const float *se = scale_embed + (size_t)j * D;
                    for (int d = 0; d < D; ++d) {
                        dqd[d] += ds * sc * se[d];
                        dse_d[((size_t)bh * J + j) * D + d] += ds * sc * qr[d];
                    }
                }
            }
            for (int d = 0; d < D; ++d) dq[base + (size_t)n * D + d] = (float)dqd[d];
        }
        for (size_t i = 0; i < (size_t)N * D; ++i) { dk[base + i] = (float)dkd[i]; dv[base + i] = (float)dvd[i]; }
        free(dkd); free(dvd); free(s); free(p); free(dp); free(o); free(dqd);
    }
}

int dsqg_oracle_bwd(const float *q, const float *k, const float *v, const float *pos_bias,
                    const float *scale_embed, const float *head_gain, const int32_t *offsets,
                    int J, int B, int H, int N, int D, const float *dout,
                    float *dq, float *dk, float *dv, float *dpb, float *dse, float *dgain) {
    const size_t BH = (size_t)B * H;
    double *dpb_d = (double *)calloc((size_t)BH * J, sizeof(double));
    double *dse_d = scale_embed ? (double *)calloc((size_t)BH * J * D, sizeof(double)) : NULL;
    double *dg_d = (double *)calloc(BH, sizeof(double));
    ctx_t c = {0};
    c.q = q; c.k = k; c.v = v; c.pos_bias = pos_bias; c.scale_embed = scale_embed;
    c.head_gain = head_gain; c.offsets = offsets; c.J = J; c.B = B; c.H = H; c.N = N; c.D = D;
    c.dout = dout; c.dq = dq; c.dk = dk; c.dv = dv; c.dpb_d = dpb_d; c.dse_d = dse_d; c.dg_d = dg_d;
    parallel_for((int)BH, bwd_bh, &c);
    for (int j = 0; j < J; ++j)
        for (int h = 0; h < H; ++h) {
            double t = 0.0;
            for (int b = 0; b < B; ++b) t += dpb_d[((size_t)b * H + h) * J + j];
            dpb[j * H + h] = (float)t;
        }
    if (scale_embed && dse)
        for (int j = 0; j < J; ++j)
            for (int d = 0; d < D; ++d) {
                double t = 0.0;
                for (size_t bh = 0; bh < BH; ++bh) t += dse_d[(bh * J + j) * D + d];
                dse[(size_t)j * D + d] = (float)t;
            }
    if (dgain)
        for (int h = 0; h < H; ++h) {
            double t = 0.0;
            for (int b = 0; b < B; ++b) t += dg_d[(size_t)b * H + h];
            dgain[h] = (float)t;
        }
    free(dpb_d); free(dse_d); free(dg_d);
    return 0;
}

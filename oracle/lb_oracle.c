/*
 * CPU restatement of Loopback's depth-attention residual read, its update write and their backward.
 *
 * TEST INFRASTRUCTURE, NOT PRODUCT. Only the tests, the smoke check and the CPU-baseline leg of the benchmark
 * may load this file's library; the CUDA library never calls it and has no CPU fallback.
 *
 * What it restates (reference project paths):
 *   update        d_s = hidden - x_before in the activation dtype            looped_transformer.py:544
 *   key scale     r = rsqrt(mean(d^2) + eps), fp32, from the stored update   looped_transformer.py:307-309, :406
 *   read          scores, two softmaxes, installed coefficients, output      looped_transformer.py:410-424
 *   prologue      base blend, coefficient/prior append and decay             looped_transformer.py:380-391
 *   first read    one source, no attention                                   looped_transformer.py:407-408
 *   backward      the analytic gradient of the read above (what autograd derives from those lines); its
 *                 factoring into per-source scalars follows the fused kernels' notes, fused_dattn.py:20-24
 *
 * Parity pin: oracle outputs are compared with tensors produced by the unmodified reference (imported from its
 * tree when the fixtures were generated) in tests/golden/ -- see tests/golden/make_golden.py.
 *
 * Every routine exists in a float ("f32": the arithmetic type of the reference read) and a double ("f64": error
 * attribution) flavour, generated from one body by including this file into itself.
 */
#ifndef LBO_BODY

#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define LBO_EXPORT __attribute__((visibility("default")))

/* round-to-nearest-even fp32 -> bf16 -> fp32, the rounding torch applies when a bf16 tensor is produced */
LBO_EXPORT float lbo_round_bf16(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) { u |= 0x00400000u; u &= 0xffff0000u; }   /* quiet NaN */
    else { u += 0x7fffu + ((u >> 16) & 1u); u &= 0xffff0000u; }
    memcpy(&x, &u, 4);
    return x;
}

LBO_EXPORT int lbo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

LBO_EXPORT void lbo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* The decay prior of read `step` (n = step + 1 entries) and its per-read companions, built the way the cell
 * builds it: append 1, multiply everything by (1 - beta) at the end of an iteration -- fp32 throughout.
 * looped_transformer.py:385-391 (prior), :414 (clamped log), :417 (mass). */
LBO_EXPORT void lbo_prior(int step, int num_blocks, double beta, float *c0, float *lc, float *mass) {
    int n = 0;
    float lam = (float)(1.0 - beta);
    for (int s = 0; s <= step; ++s) {
        c0[n++] = 1.0f;
        if (s % num_blocks == num_blocks - 1)
            for (int i = 0; i < n; ++i) c0[i] = lam * c0[i];
    }
    float m = 0.0f;
    for (int i = 0; i < n; ++i) {
        if (lc) lc[i] = logf(c0[i] < 1e-8f ? 1e-8f : c0[i]);
        m += c0[i];
    }
    if (mass) *mass = m;
}

#define LBO_BODY
#define REAL float
#define SUF(x) x##_f32
#define R_EXP expf
#define R_LOG logf
#define R_SQRT sqrtf
#include "lb_oracle.c"
#undef REAL
#undef SUF
#undef R_EXP
#undef R_LOG
#undef R_SQRT
#define REAL double
#define SUF(x) x##_f64
#define R_EXP exp
#define R_LOG log
#define R_SQRT sqrt
#include "lb_oracle.c"

#else /* LBO_BODY: the generic routines, compiled once per REAL */

/* Update write. v = h - x rounded once to the storage type (bf16_storage != 0: bf16; else REAL), then the key
 * scale from the ROUNDED update. looped_transformer.py:544, :406 with :307-309. */
LBO_EXPORT void SUF(lbo_write)(const REAL *h, const REAL *x, REAL *v, REAL *r, int64_t n_tok, int d, double eps,
                               int bf16_storage) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < n_tok; ++t) {
        const REAL *hp = h + t * d, *xp = x + t * d;
        REAL *vp = v + t * d;
        REAL ss = 0;
        for (int c = 0; c < d; ++c) {
            REAL u = hp[c] - xp[c];
            if (bf16_storage) u = (REAL)lbo_round_bf16((float)u);
            vp[c] = u;
            ss += u * u;
        }
        r[t] = (REAL)1 / R_SQRT(ss / (REAL)d + (REAL)eps);
    }
}

/* Boundary blend: base = proposal + beta (h0 - proposal) at the end of an iteration, else the proposal.
 * looped_transformer.py:380-381. In bf16 storage the blend is evaluated in bf16 steps like torch does. */
LBO_EXPORT void SUF(lbo_base)(const REAL *proposal, const REAL *h0, REAL *base, int64_t n_elem, double beta,
                              int at_boundary, int bf16_storage) {
#pragma omp parallel for schedule(static)
    for (int64_t k = 0; k < n_elem; ++k) {
        if (!at_boundary) { base[k] = proposal[k]; continue; }
        if (bf16_storage) {
            float df = lbo_round_bf16((float)(h0[k] - proposal[k]));
            float sc = lbo_round_bf16((float)beta * df);
            base[k] = (REAL)lbo_round_bf16((float)proposal[k] + sc);
        } else {
            base[k] = proposal[k] + (REAL)beta * (h0[k] - proposal[k]);
        }
    }
}

/* One read over n stored updates.
 *   V        [n][n_tok][d] (source i at V + i * src_stride), R [n][n_tok] key scales (R + i * n_tok)
 *   q [d], base [n_tok][d], cbar [n_tok][n] installed coefficients, c0 [n] the read's prior
 *   out [n_tok][d], tc [n_tok][n]; optional saves for the backward: p [n_tok][n], z [n_tok][n]
 * acc_bf16 != 0 reproduces the reference's accumulation in a bf16 activation dtype (coefficient delta, every term,
 * the running correction and the final sum each rounded to bf16); 0 accumulates in REAL and rounds nothing, which
 * is "the reference read evaluated in REAL on the same inputs".  looped_transformer.py:410-424. */
LBO_EXPORT void SUF(lbo_read_fwd)(const REAL *V, int64_t src_stride, const REAL *R, int n, const REAL *q,
                                  const REAL *base, const REAL *cbar, const float *c0, int64_t n_tok, int d,
                                  int acc_bf16, REAL *out, REAL *tc, REAL *p_save, REAL *z_save) {
    REAL lc[512], p0[512];
    REAL inv = (REAL)1 / R_SQRT((REAL)d);
    REAL mass = 0, mx0 = -INFINITY, s0 = 0;
    if (n > 512) return;
    for (int i = 0; i < n; ++i) {
        REAL c = (REAL)c0[i];
        lc[i] = R_LOG(c < (REAL)1e-8f ? (REAL)1e-8f : c);       /* :414 */
        mass += c;                                              /* :417 */
        if (lc[i] > mx0) mx0 = lc[i];
    }
    for (int i = 0; i < n; ++i) { p0[i] = R_EXP(lc[i] - mx0); s0 += p0[i]; }
    for (int i = 0; i < n; ++i) p0[i] /= s0;                    /* :415 */
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < n_tok; ++t) {
        REAL l[512], w[512];
        REAL mx = -INFINITY, sum = 0;
        for (int i = 0; i < n; ++i) {
            const REAL *vp = V + i * src_stride + t * d;
            REAL r = R[(int64_t)i * n_tok + t], dot = 0;
            for (int c = 0; c < d; ++c) dot += (vp[c] * r) * q[c];          /* key = v * r (:406), key . q (:413) */
            REAL z = dot * inv;
            if (z_save) z_save[t * n + i] = z;
            l[i] = z + lc[i];                                              /* :416 */
            if (l[i] > mx) mx = l[i];
        }
        for (int i = 0; i < n; ++i) { w[i] = R_EXP(l[i] - mx); sum += w[i]; }
        for (int i = 0; i < n; ++i) {
            REAL p = w[i] / sum;
            if (p_save) p_save[t * n + i] = p;
            REAL tci = (REAL)c0[i] + mass * (p - p0[i]);                    /* :418 */
            tc[t * n + i] = tci;
            w[i] = tci - cbar[t * n + i];                                   /* :419 */
            if (acc_bf16) w[i] = (REAL)lbo_round_bf16((float)w[i]);
        }
        const REAL *bp = base + t * d;
        REAL *op = out + t * d;
        for (int c = 0; c < d; ++c) {
            REAL corr = 0;
            for (int i = 0; i < n; ++i) {                                   /* :420-423 */
                REAL term = w[i] * V[i * src_stride + t * d + c];
                if (acc_bf16) {
                    term = (REAL)lbo_round_bf16((float)term);
                    corr = i ? (REAL)lbo_round_bf16((float)(corr + term)) : term;
                } else {
                    corr = i ? corr + term : term;
                }
            }
            REAL o = bp[c] + corr;                                          /* :424 */
            op[c] = acc_bf16 ? (REAL)lbo_round_bf16((float)o) : o;
        }
    }
}

/* Backward of one read, given g = dL/dout [n_tok][d] and gt = dL/dtc [n_tok][n] (may be NULL = zeros).
 * With p the scored softmax, z the scores and w = tc - cbar of the forward:
 *     gd_i = g . v_i          gp_i = mass (gd_i + gt_i)      S = sum_i p_i gp_i      dz_i = p_i (gp_i - S)
 *     dq      = sum_tok sum_i dz_i r_i v_i / sqrt(d)
 *     dV_i   += w_i g + dz_i r_i q / sqrt(d) + dr_i (-r_i^3 / d) v_i,     dr_i = dz_i z_i / r_i
 *     dcbar_i = -gd_i         dbase = g (the caller's)
 * dV [n][n_tok][d] is ADDED into (the caller zeroes it), dR_out (optional, [n][n_tok]) receives dr_i added,
 * dq [d] is overwritten. This is the derivative of looped_transformer.py:406-424 taken by hand; the grouping
 * into gd / gp / S / dz is the one described at fused_dattn.py:20-24. */
LBO_EXPORT void SUF(lbo_read_bwd)(const REAL *V, int64_t src_stride, const REAL *R, int n, const REAL *q,
                                  const REAL *cbar, const float *c0, const REAL *g, const REAL *gt,
                                  int64_t n_tok, int d, REAL *dq, REAL *dV, REAL *dcbar, REAL *dR_out) {
    REAL lc[512], p0[512];
    REAL inv = (REAL)1 / R_SQRT((REAL)d);
    REAL mass = 0, mx0 = -INFINITY, s0 = 0;
    if (n > 512) return;
    for (int i = 0; i < n; ++i) {
        REAL c = (REAL)c0[i];
        lc[i] = R_LOG(c < (REAL)1e-8f ? (REAL)1e-8f : c);
        mass += c;
        if (lc[i] > mx0) mx0 = lc[i];
    }
    for (int i = 0; i < n; ++i) { p0[i] = R_EXP(lc[i] - mx0); s0 += p0[i]; }
    for (int i = 0; i < n; ++i) p0[i] /= s0;
    int nthr = lbo_num_threads();
    double *dq_part = (double *)calloc((size_t)nthr * (size_t)d, sizeof(double));
#pragma omp parallel
    {
#ifdef _OPENMP
        double *mydq = dq_part + (size_t)omp_get_thread_num() * (size_t)d;
#else
        double *mydq = dq_part;
#endif
#pragma omp for schedule(static)
        for (int64_t t = 0; t < n_tok; ++t) {
            REAL z[512], p[512], gd[512];
            REAL mx = -INFINITY, sum = 0, S = 0;
            const REAL *gp_ = g + t * d;
            for (int i = 0; i < n; ++i) {
                const REAL *vp = V + i * src_stride + t * d;
                REAL r = R[(int64_t)i * n_tok + t], dot = 0, gdot = 0;
                for (int c = 0; c < d; ++c) { dot += (vp[c] * r) * q[c]; gdot += gp_[c] * vp[c]; }
                z[i] = dot * inv;
                gd[i] = gdot;
                if (z[i] + lc[i] > mx) mx = z[i] + lc[i];
            }
            for (int i = 0; i < n; ++i) { p[i] = R_EXP(z[i] + lc[i] - mx); sum += p[i]; }
            for (int i = 0; i < n; ++i) {
                p[i] /= sum;
                REAL gti = gt ? gt[t * n + i] : (REAL)0;
                S += p[i] * (mass * (gd[i] + gti));
            }
            for (int i = 0; i < n; ++i) {
                const REAL *vp = V + i * src_stride + t * d;
                REAL r = R[(int64_t)i * n_tok + t];
                REAL gti = gt ? gt[t * n + i] : (REAL)0;
                REAL dz = p[i] * (mass * (gd[i] + gti) - S);
                REAL w = (REAL)c0[i] + mass * (p[i] - p0[i]) - cbar[t * n + i];
                REAL dr = dz * z[i] / r;
                REAL kq = dz * r * inv, kr = dr * (-(r * r * r) / (REAL)d);
                REAL *dvp = dV + i * src_stride + t * d;
                for (int c = 0; c < d; ++c) {
                    dvp[c] += w * gp_[c] + kq * q[c] + kr * vp[c];
                    mydq[c] += (double)(kq * vp[c]);
                }
                if (dcbar) dcbar[t * n + i] = -gd[i];
                if (dR_out) dR_out[(int64_t)i * n_tok + t] += dr;
            }
        }
    }
    for (int c = 0; c < d; ++c) {
        double a = 0;
        for (int k = 0; k < nthr; ++k) a += dq_part[(size_t)k * (size_t)d + c];
        dq[c] = (REAL)a;
    }
    free(dq_part);
}

/* A whole K x R pass with the blocks replaced by x -> x + D_s (the benchmark's chain):
 *     x_0 = h0;  h = x_s + D_s;  d_s = write(h, x_s);  x_{s+1} = read_s(...)
 * and, when G != NULL, the backward of  loss = sum_s <x_{s+1}, G_s>  down to dq [N-1][d], dD [N][n_tok][d] and
 * dh0 [n_tok][d].  D and G are [N][n_tok][d]; states [N][n_tok][d] receives every read state; tc_last [n_tok][N].
 * Call sites restated: looped_transformer.py:513-546 (the model's loop over the shared blocks), :371-424 (cell).
 * Scratch is allocated here; sizes are the caller's responsibility (this is the CPU baseline's timed body). */
LBO_EXPORT int SUF(lbo_chain)(const REAL *h0, const REAL *D, const REAL *Q, const REAL *G, int64_t n_tok, int d,
                              int num_blocks, int num_loops, double beta, double eps, int bf16_storage,
                              REAL *states, REAL *tc_last, REAL *dq, REAL *dD, REAL *dh0) {
    int N = num_blocks * num_loops;
    int64_t td = n_tok * d;
    if (N > 512) return -1;
    REAL *V = (REAL *)malloc(sizeof(REAL) * (size_t)N * (size_t)td);
    REAL *R = (REAL *)malloc(sizeof(REAL) * (size_t)N * (size_t)n_tok);
    REAL *hbuf = (REAL *)malloc(sizeof(REAL) * (size_t)td);
    REAL *base = (REAL *)malloc(sizeof(REAL) * (size_t)td);
    /* installed coefficients of every read are kept for the backward: read s has s+1 of them per token */
    REAL **cbar = (REAL **)calloc((size_t)N, sizeof(REAL *));
    REAL **tcs = (REAL **)calloc((size_t)N, sizeof(REAL *));
    float c0[512];
    if (!V || !R || !hbuf || !base || !cbar || !tcs) return -2;
    for (int s = 0; s < N; ++s) {
        int n = s + 1, boundary = (s % num_blocks == num_blocks - 1);
        const REAL *x = s ? states + (int64_t)(s - 1) * td : h0;
        const REAL *Ds = D + (int64_t)s * td;
#pragma omp parallel for schedule(static)
        for (int64_t k = 0; k < td; ++k) {
            REAL u = x[k] + Ds[k];
            hbuf[k] = bf16_storage ? (REAL)lbo_round_bf16((float)u) : u;
        }
        SUF(lbo_write)(hbuf, x, V + (int64_t)s * td, R + (int64_t)s * n_tok, n_tok, d, eps, bf16_storage);
        SUF(lbo_base)(hbuf, h0, base, td, beta, boundary, bf16_storage);
        lbo_prior(s, num_blocks, beta, c0, NULL, NULL);
        cbar[s] = (REAL *)malloc(sizeof(REAL) * (size_t)n_tok * (size_t)n);
        tcs[s] = (REAL *)malloc(sizeof(REAL) * (size_t)n_tok * (size_t)n);
        REAL lam = boundary ? (REAL)(float)(1.0 - beta) : (REAL)1;
        for (int64_t t = 0; t < n_tok; ++t) {                       /* base_coeffs = cat(coeffs, 1) [* lam] */
            for (int i = 0; i < s; ++i) cbar[s][t * n + i] = lam * tcs[s - 1][t * s + i];
            cbar[s][t * n + s] = lam;
        }
        REAL *out = states + (int64_t)s * td;
        if (s == 0) {                                               /* first read: no attention (:407-408) */
            memcpy(out, base, sizeof(REAL) * (size_t)td);
            memcpy(tcs[0], cbar[0], sizeof(REAL) * (size_t)n_tok);
        } else {
            SUF(lbo_read_fwd)(V, td, R, n, Q + (int64_t)(s - 1) * d, base, cbar[s], c0, n_tok, d, bf16_storage,
                              out, tcs[s], NULL, NULL);
        }
    }
    if (tc_last) memcpy(tc_last, tcs[N - 1], sizeof(REAL) * (size_t)n_tok * (size_t)N);
    if (G) {
        REAL *dV = (REAL *)calloc((size_t)N * (size_t)td, sizeof(REAL));
        REAL *gout = (REAL *)malloc(sizeof(REAL) * (size_t)td);      /* dL/d x_{s+1} */
        REAL *gt = (REAL *)calloc((size_t)n_tok * (size_t)N, sizeof(REAL));
        REAL *dcb = (REAL *)malloc(sizeof(REAL) * (size_t)n_tok * (size_t)N);
        if (!dV || !gout || !gt || !dcb) return -2;
        memset(dh0, 0, sizeof(REAL) * (size_t)td);
        memset(gout, 0, sizeof(REAL) * (size_t)td);
        int have_gt = 0;
        for (int s = N - 1; s >= 0; --s) {
            int n = s + 1, boundary = (s % num_blocks == num_blocks - 1);
            REAL lam = boundary ? (REAL)(float)(1.0 - beta) : (REAL)1;
            const REAL *Gs = G + (int64_t)s * td;
#pragma omp parallel for schedule(static)
            for (int64_t k = 0; k < td; ++k) gout[k] += Gs[k];
            if (s >= 1) {
                lbo_prior(s, num_blocks, beta, c0, NULL, NULL);
                SUF(lbo_read_bwd)(V, td, R, n, Q + (int64_t)(s - 1) * d, cbar[s], c0, gout, have_gt ? gt : NULL,
                                  n_tok, d, dq + (int64_t)(s - 1) * d, dV, dcb, NULL);
                /* dL/d tc_{s-1} = lam * dcbar[:, :s]  (base_coeffs = lam * cat(tc_{s-1}, 1)) */
                for (int64_t t = 0; t < n_tok; ++t)
                    for (int i = 0; i < s; ++i) gt[t * s + i] = lam * dcb[t * n + i];
                have_gt = 1;
            }
            /* base = proposal + beta (h0 - proposal): dproposal = (1 - beta) g, dh0 = beta g at a boundary.
             * proposal = h = x_s + D_s; the update d_s = h - x_s sends dV[s] to h and -dV[s] to x_s. */
            REAL *dDs = dD + (int64_t)s * td;
            const REAL *dVs = dV + (int64_t)s * td;
#pragma omp parallel for schedule(static)
            for (int64_t k = 0; k < td; ++k) {
                REAL gb = gout[k];
                REAL dprop = boundary ? ((REAL)1 - (REAL)beta) * gb : gb;
                if (boundary) dh0[k] += (REAL)beta * gb;
                REAL dh = dprop + dVs[k];
                dDs[k] = dh;
                gout[k] = dh - dVs[k];                               /* dL/dx_s, the previous read's output */
            }
        }
#pragma omp parallel for schedule(static)
        for (int64_t k = 0; k < td; ++k) dh0[k] += gout[k];           /* x_0 = h0 */
        free(dV); free(gout); free(gt); free(dcb);
    }
    for (int s = 0; s < N; ++s) { free(cbar[s]); free(tcs[s]); }
    free(cbar); free(tcs); free(V); free(R); free(hbuf); free(base);
    return 0;
}

#endif /* LBO_BODY */

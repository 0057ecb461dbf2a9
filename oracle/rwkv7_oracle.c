/*
 * CPU oracle for the rwkv-rs WKV7 hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's tensor-op
 * definitions.  It is the checker for the CUDA kernels and the timed CPU
 * baseline; it is never linked into, loaded by or called from the product
 * library.
 *
 * PARITY UNPINNED: the reference ships no golden vectors, known-answer files or
 * fixtures for these operators (its tests compare a custom kernel with a
 * tensor-op path on unseeded random inputs), and the reference itself cannot be
 * compiled where this oracle was written (no Rust toolchain, Burn/CubeCL not
 * vendored).  The oracle is therefore pinned only by (1) a line-by-line reading
 * of the cited reference functions, (2) an independent fp64 torch restatement of
 * the same formulas, and (3) closed-form known answers; see tests/.
 *
 * Reference functions followed (paths inside the rwkv-rs repository):
 *   wkv7      crates/rwkv-nn/src/kernels/train/time_mixer/wkv7/mod.rs:179-242
 *             (wkv7_reference_with_state) cross-read with kernel.rs:60-196
 *             (index order, f32 accumulation, decay = exp(-exp(w)) :55-58)
 *   mix6      crates/rwkv-nn/src/kernels/train/time_mixer/mix6/mod.rs:111-156,
 *             kernel.rs:25-57
 *   addcmul   crates/rwkv-nn/src/kernels/template/addcmul/mod.rs:122-124,
 *             addcmul5 :165-175, kernel.rs:4-65
 *   token_shift_diff
 *             crates/rwkv-nn/src/kernels/template/token_shift_diff/mod.rs:114-155,
 *             :170-200, kernel.rs:16-45
 *   weight_prepare  crates/rwkv-nn/src/modules/time_mixer/weight_prepare.rs:252-287,
 *             crates/rwkv-nn/src/functions/normalize.rs:9-41, functions/lerp.rs:4-10
 *   gated_readout  crates/rwkv-nn/src/modules/time_mixer/gated_readout.rs:110-145
 *             (GroupNorm itself lives in Burn, which is not part of the reference
 *             tree: the published definition is restated, biased variance)
 *   channel_mixer  crates/rwkv-nn/src/kernels/train/channel_mixer/mod.rs:96-128
 *             (channel_mixer_reference)
 *   lm_head_ce  no reference implementation exists (lm_head_l2wrap_ce/mod.rs is
 *             empty); the specification is z = x W^T, lse = log sum exp z,
 *             loss = lse - z[target].
 *
 * Layouts: row-major contiguous.  Sequence tensors [B,T,H,N] index
 * ((b*T+t)*H+h)*N+n (kernel.rs:14-25); state [B,H,N,N] index
 * ((b*H+h)*N+i)*N+j with i the value row and j the key column (kernel.rs:27-37).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* A launcher may have set OMP_NUM_THREADS=1 for its workers (torchrun does); the timed CPU
 * baseline asks for the host's cores explicitly.  Returns the count now in force. */
int oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

/* ------------------------------------------------------------------ wkv7 -- */

/*
 * fp32 restatement with the accumulation order of the reference kernel
 * (kernel.rs:82-195): per token, per state row i:
 *   sa_i   = sum_j S[i][j] * a[j]             (S is S_{t-1}; j ascending, f32)
 *   S[i][j]= S[i][j]*d[j] + sa_i*b[j] + v[i]*k[j]      with d = exp(-exp(w))
 *   y[i]   = sum_j S[i][j] * r[j]             (S is S_t;     j ascending, f32)
 * s0 may be NULL (zero initial state, wkv7_pretrain_reference mod.rs:153-165);
 * s_out may be NULL (statetune drops the final state, forward.rs:522-526).
 */
void oracle_wkv7_f32(const float *r, const float *w, const float *k, const float *v,
                     const float *a, const float *b, const float *s0, float *y,
                     float *s_out, int64_t B, int64_t T, int64_t H, int64_t N) {
    const int64_t BH = B * H;
#pragma omp parallel
    {
        float *S = (float *)malloc(sizeof(float) * (size_t)(N * N));
        float *d = (float *)malloc(sizeof(float) * (size_t)N);
#pragma omp for schedule(dynamic, 1)
        for (int64_t bh = 0; bh < BH; ++bh) {
            const int64_t bi = bh / H, h = bh % H;
            if (s0)
                memcpy(S, s0 + bh * N * N, sizeof(float) * (size_t)(N * N));
            else
                memset(S, 0, sizeof(float) * (size_t)(N * N));
            for (int64_t t = 0; t < T; ++t) {
                const int64_t o = ((bi * T + t) * H + h) * N;
                const float *rt = r + o, *wt = w + o, *kt = k + o, *vt = v + o,
                            *at = a + o, *bt = b + o;
                for (int64_t j = 0; j < N; ++j) d[j] = expf(-expf(wt[j]));
                for (int64_t i = 0; i < N; ++i) {
                    float *Si = S + i * N;
                    float sa = 0.0f;
                    for (int64_t j = 0; j < N; ++j) sa += Si[j] * at[j];
                    const float vi = vt[i];
                    float acc = 0.0f;
                    for (int64_t j = 0; j < N; ++j) {
                        const float u = Si[j] * d[j] + sa * bt[j] + vi * kt[j];
                        Si[j] = u;
                        acc += u * rt[j];
                    }
                    y[o + i] = acc;
                }
            }
            if (s_out) memcpy(s_out + bh * N * N, S, sizeof(float) * (size_t)(N * N));
        }
        free(S);
        free(d);
    }
}

/*
 * fp64 restatement of the same definition (mod.rs:179-242): inputs are the
 * exact fp32 (or bf16-representable) values the kernel under test consumes, all
 * arithmetic in double.  This is the parity target for the CUDA kernels.
 */
void oracle_wkv7_f64(const float *r, const float *w, const float *k, const float *v,
                     const float *a, const float *b, const double *s0, double *y,
                     double *s_out, int64_t B, int64_t T, int64_t H, int64_t N) {
    const int64_t BH = B * H;
#pragma omp parallel
    {
        double *S = (double *)malloc(sizeof(double) * (size_t)(N * N));
        double *d = (double *)malloc(sizeof(double) * (size_t)N);
#pragma omp for schedule(dynamic, 1)
        for (int64_t bh = 0; bh < BH; ++bh) {
            const int64_t bi = bh / H, h = bh % H;
            if (s0)
                memcpy(S, s0 + bh * N * N, sizeof(double) * (size_t)(N * N));
            else
                memset(S, 0, sizeof(double) * (size_t)(N * N));
            for (int64_t t = 0; t < T; ++t) {
                const int64_t o = ((bi * T + t) * H + h) * N;
                for (int64_t j = 0; j < N; ++j) d[j] = exp(-exp((double)w[o + j]));
                for (int64_t i = 0; i < N; ++i) {
                    double *Si = S + i * N;
                    double sa = 0.0;
                    for (int64_t j = 0; j < N; ++j) sa += Si[j] * (double)a[o + j];
                    const double vi = (double)v[o + i];
                    double acc = 0.0;
                    for (int64_t j = 0; j < N; ++j) {
                        const double u =
                            Si[j] * d[j] + sa * (double)b[o + j] + vi * (double)k[o + j];
                        Si[j] = u;
                        acc += u * (double)r[o + j];
                    }
                    y[o + i] = acc;
                }
            }
            if (s_out) memcpy(s_out + bh * N * N, S, sizeof(double) * (size_t)(N * N));
        }
        free(S);
        free(d);
    }
}

/* -------------------------------------------------------- wkv7 training -- */

/*
 * Training forward (wkv7/kernel.rs:60-196,198-364 with forward.rs:368-375): the
 * recurrence above, also returning what the reference saves for its backward pass:
 * snapshots [B][H][T/chunk_len][N][N] = S after the last token of each chunk
 * (index order kernel.rs:40-53) and state_replacement [B][T][H][N] = sa_t.
 */
void oracle_wkv7_train_f64(const float *r, const float *w, const float *k, const float *v,
                           const float *a, const float *b, const double *s0, double *y,
                           double *s_out, double *snapshots, double *state_replacement, int64_t B,
                           int64_t T, int64_t H, int64_t N, int64_t chunk_len) {
    const int64_t BH = B * H, nchunks = T / chunk_len;
#pragma omp parallel
    {
        double *S = (double *)malloc(sizeof(double) * (size_t)(N * N));
        double *d = (double *)malloc(sizeof(double) * (size_t)N);
#pragma omp for schedule(dynamic, 1)
        for (int64_t bh = 0; bh < BH; ++bh) {
            const int64_t bi = bh / H, h = bh % H;
            if (s0) memcpy(S, s0 + bh * N * N, sizeof(double) * (size_t)(N * N));
            else memset(S, 0, sizeof(double) * (size_t)(N * N));
            for (int64_t t = 0; t < T; ++t) {
                const int64_t o = ((bi * T + t) * H + h) * N;
                for (int64_t j = 0; j < N; ++j) d[j] = exp(-exp((double)w[o + j]));
                for (int64_t i = 0; i < N; ++i) {
                    double *Si = S + i * N;
                    double sa = 0.0;
                    for (int64_t j = 0; j < N; ++j) sa += Si[j] * (double)a[o + j];
                    state_replacement[o + i] = sa;
                    const double vi = (double)v[o + i];
                    double acc = 0.0;
                    for (int64_t j = 0; j < N; ++j) {
                        const double u = Si[j] * d[j] + sa * (double)b[o + j] + vi * (double)k[o + j];
                        Si[j] = u;
                        acc += u * (double)r[o + j];
                    }
                    y[o + i] = acc;
                }
                if ((t + 1) % chunk_len == 0)
                    memcpy(snapshots + (bh * nchunks + t / chunk_len) * N * N, S, sizeof(double) * (size_t)(N * N));
            }
            if (s_out) memcpy(s_out + bh * N * N, S, sizeof(double) * (size_t)(N * N));
        }
        free(S);
        free(d);
    }
}

/*
 * Backward pass: exact reverse-mode differentiation of the recurrence, in double, with every
 * intermediate state kept (no rebuilding by inverse decay, which is how the reference's kernel
 * kernel.rs:395-690 saves memory).  Per token, with S the state before and S' after it:
 *   dS' += dy r^T; dr = S'^T dy; dv = dS' k; dk = dS'^T v; dsa = dS' b; db = dS'^T sa;
 *   dd_j = sum_i dS'_ij S_ij; dw = dd * (-exp(w) d); da = S^T dsa; dS = dS' diag(d) + dsa a^T.
 * grads are laid out like the inputs; ds0 [B][H][N][N]; dsT may be NULL (zero).
 */
void oracle_wkv7_backward_f64(const float *r, const float *w, const float *k, const float *v,
                              const float *a, const float *b, const double *s0, const double *dy,
                              const double *dsT, double *dr, double *dw, double *dk, double *dv,
                              double *da, double *db, double *ds0, int64_t B, int64_t T, int64_t H,
                              int64_t N) {
    const int64_t BH = B * H, NN = N * N;
#pragma omp parallel
    {
        double *states = (double *)malloc(sizeof(double) * (size_t)((T + 1) * NN));   /* S_0 .. S_T */
        double *sas = (double *)malloc(sizeof(double) * (size_t)(T * N));
        double *dS = (double *)malloc(sizeof(double) * (size_t)NN);
        double *d = (double *)malloc(sizeof(double) * (size_t)N);
        double *dsa = (double *)malloc(sizeof(double) * (size_t)N);
#pragma omp for schedule(dynamic, 1)
        for (int64_t bh = 0; bh < BH; ++bh) {
            const int64_t bi = bh / H, h = bh % H;
            if (s0) memcpy(states, s0 + bh * NN, sizeof(double) * (size_t)NN);
            else memset(states, 0, sizeof(double) * (size_t)NN);
            for (int64_t t = 0; t < T; ++t) {
                const int64_t o = ((bi * T + t) * H + h) * N;
                const double *S = states + t * NN;
                double *S1 = states + (t + 1) * NN;
                for (int64_t i = 0; i < N; ++i) {
                    double sa = 0.0;
                    for (int64_t j = 0; j < N; ++j) sa += S[i * N + j] * (double)a[o + j];
                    sas[t * N + i] = sa;
                    for (int64_t j = 0; j < N; ++j)
                        S1[i * N + j] = S[i * N + j] * exp(-exp((double)w[o + j])) + sa * (double)b[o + j] +
                                        (double)v[o + i] * (double)k[o + j];
                }
            }
            if (dsT) memcpy(dS, dsT + bh * NN, sizeof(double) * (size_t)NN);
            else memset(dS, 0, sizeof(double) * (size_t)NN);
            for (int64_t t = T - 1; t >= 0; --t) {
                const int64_t o = ((bi * T + t) * H + h) * N;
                const double *S = states + t * NN, *S1 = states + (t + 1) * NN;
                for (int64_t j = 0; j < N; ++j) d[j] = exp(-exp((double)w[o + j]));
                for (int64_t i = 0; i < N; ++i)
                    for (int64_t j = 0; j < N; ++j) dS[i * N + j] += dy[o + i] * (double)r[o + j];
                for (int64_t j = 0; j < N; ++j) {
                    double g_r = 0.0, g_k = 0.0, g_b = 0.0, g_d = 0.0;
                    for (int64_t i = 0; i < N; ++i) {
                        g_r += S1[i * N + j] * dy[o + i];
                        g_k += dS[i * N + j] * (double)v[o + i];
                        g_b += dS[i * N + j] * sas[t * N + i];
                        g_d += dS[i * N + j] * S[i * N + j];
                    }
                    dr[o + j] = g_r;
                    dk[o + j] = g_k;
                    db[o + j] = g_b;
                    dw[o + j] = g_d * (-exp((double)w[o + j]) * d[j]);
                }
                for (int64_t i = 0; i < N; ++i) {
                    double g_v = 0.0, g_sa = 0.0;
                    for (int64_t j = 0; j < N; ++j) {
                        g_v += dS[i * N + j] * (double)k[o + j];
                        g_sa += dS[i * N + j] * (double)b[o + j];
                    }
                    dv[o + i] = g_v;
                    dsa[i] = g_sa;
                }
                for (int64_t j = 0; j < N; ++j) {
                    double g_a = 0.0;
                    for (int64_t i = 0; i < N; ++i) g_a += S[i * N + j] * dsa[i];
                    da[o + j] = g_a;
                }
                for (int64_t i = 0; i < N; ++i)
                    for (int64_t j = 0; j < N; ++j)
                        dS[i * N + j] = dS[i * N + j] * d[j] + dsa[i] * (double)a[o + j];
            }
            if (ds0) memcpy(ds0 + bh * NN, dS, sizeof(double) * (size_t)NN);
        }
        free(states); free(sas); free(dS); free(d); free(dsa);
    }
}

/* ------------------------------------------------------------------ mix6 -- */

/*
 * mix6 (mix6/mod.rs:111-156): prev = x[b,t-1,c] (zero at t == 0, per batch row),
 * out_i = x + (prev - x) * mu_i[c] for the six branches, in the order
 * receptance, weight_decay, key, value, learning_rate, gate.  out is laid out
 * [6][B][T][C].  Computed in double from float inputs.
 */
void oracle_mix6_f64(const float *x, const float *const mu[6], double *out, int64_t B,
                     int64_t T, int64_t C) {
    const int64_t n = B * T * C;
#pragma omp parallel for schedule(static)
    for (int64_t bt = 0; bt < B * T; ++bt) {
        const int64_t t = bt % T;
        for (int64_t c = 0; c < C; ++c) {
            const int64_t e = bt * C + c;
            const double cur = (double)x[e];
            const double prev = (t == 0) ? 0.0 : (double)x[e - C];
            const double diff = prev - cur;
            for (int s = 0; s < 6; ++s) out[(int64_t)s * n + e] = cur + diff * (double)mu[s][c];
        }
    }
}

/* --------------------------------------------------------------- addcmul -- */

/* addcmul (addcmul/mod.rs:122-124): out = base + diff * scale[c].  nscale = 1
 * or 5 (addcmul5, mod.rs:165-175); out is [nscale][B*T][C]. */
void oracle_addcmul_f64(const float *base, const float *diff, const float *const *scale,
                        int nscale, double *out, int64_t BT, int64_t C) {
    const int64_t n = BT * C;
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < BT; ++row)
        for (int64_t c = 0; c < C; ++c) {
            const int64_t e = row * C + c;
            for (int s = 0; s < nscale; ++s)
                out[(int64_t)s * n + e] = (double)base[e] + (double)diff[e] * (double)scale[s][c];
        }
}

/* -------------------------------------------------- time-mixer epilogues -- */

static double sigmoid64(double x) { return 1.0 / (1.0 + exp(-x)); }
/* softplus with beta = 1: log(1 + e^z), evaluated without overflow */
static double softplus64(double z) { return (z > 0.0 ? z : 0.0) + log1p(exp(-fabs(z))); }

/*
 * Tail of WeightPrepare::forward (weight_prepare.rs:252-287).  rows = B*T*H head
 * rows of N channels; xi (param_key_removal) and alpha (param_key_replacement)
 * hold H*N values.  lr = sigmoid(lr_lora) (:252);
 *   replacement_key = k * (alpha * (lr - 1) + 1)                    (:254-257)
 *   weight_decay    = -softplus(-d) - 0.5                            (:272-274)
 *   removal_key_normalized = -(k*xi) / max(||k*xi||_2, 1e-12) per head   (:276-285, normalize.rs:32-40)
 *   replacement     = -removal_key_normalized * lr                   (:287)
 *   value           = vp + (vf - vp) * sigmoid(nu)   when vp != NULL  (:259-268, lerp.rs:9)
 */
void oracle_weight_prepare_f64(const float *k, const float *lr_lora, const float *d, const float *xi,
                               const float *alpha, const float *vp, const float *vf, const float *nu,
                               double *weight_decay, double *replacement_key, double *removal_key_normalized,
                               double *replacement, double *value, int64_t rows, int64_t H, int64_t N) {
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        const int64_t base = row * N, cbase = (row % H) * N;
        double ss = 0.0;
        for (int64_t n = 0; n < N; ++n) {
            const double rk = (double)k[base + n] * (double)xi[cbase + n];
            ss += rk * rk;
        }
        double denom = sqrt(ss);
        if (denom < 1e-12) denom = 1e-12;
        for (int64_t n = 0; n < N; ++n) {
            const int64_t e = base + n;
            const double lr = sigmoid64((double)lr_lora[e]);
            const double kappa = (double)k[e] * (double)xi[cbase + n] / denom;
            replacement_key[e] = (double)k[e] * ((double)alpha[cbase + n] * (lr - 1.0) + 1.0);
            weight_decay[e] = -softplus64(-(double)d[e]) - 0.5;
            removal_key_normalized[e] = -kappa;
            replacement[e] = kappa * lr;
            if (vp) value[e] = (double)vp[e] + ((double)vf[e] - (double)vp[e]) * sigmoid64((double)nu[e]);
        }
    }
}

/*
 * GatedReadout::forward between the gate LoRA and the output projection
 * (gated_readout.rs:123-141): GroupNorm with one group per head over the N
 * channels of the head (mean, biased variance, eps inside the square root,
 * per-channel gamma and beta), bonus = (sum_n r*k*rho[h,n]) * v, (norm + bonus) * gate.
 */
void oracle_gated_readout_f64(const float *y, const float *r, const float *k, const float *v,
                              const float *gate, const float *gamma, const float *beta, const float *rho,
                              double eps, double *out, int64_t rows, int64_t H, int64_t N) {
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        const int64_t base = row * N, cbase = (row % H) * N;
        double mean = 0.0, dot = 0.0;
        for (int64_t n = 0; n < N; ++n) {
            mean += (double)y[base + n];
            dot += (double)r[base + n] * (double)k[base + n] * (double)rho[cbase + n];
        }
        mean /= (double)N;
        double var = 0.0;
        for (int64_t n = 0; n < N; ++n) {
            const double dlt = (double)y[base + n] - mean;
            var += dlt * dlt;
        }
        var /= (double)N;
        const double rstd = 1.0 / sqrt(var + eps);
        for (int64_t n = 0; n < N; ++n) {
            const int64_t e = base + n;
            const double nrm = ((double)y[e] - mean) * rstd * (double)gamma[cbase + n] + (double)beta[cbase + n];
            out[e] = (nrm + dot * (double)v[e]) * (double)gate[e];
        }
    }
}

/* --------------------------------------------------------- channel mixer -- */

/*
 * channel_mixer_reference (channel_mixer/mod.rs:96-128): shifted = previous token
 * (zero at t == 0); key_input = x + (shifted - x) * key_scale[c];
 * hidden = relu(key_input . key_weight^T)^2 with key_weight [F][C];
 * out = hidden . value_weight^T with value_weight [C][F].  Double throughout.
 */
void oracle_channel_mixer_f64(const float *x, const float *key_scale, const float *key_weight,
                              const float *value_weight, double *out, int64_t B, int64_t T, int64_t C,
                              int64_t F) {
#pragma omp parallel
    {
        double *ki = (double *)malloc(sizeof(double) * (size_t)C);
        double *hid = (double *)malloc(sizeof(double) * (size_t)F);
#pragma omp for schedule(static)
        for (int64_t row = 0; row < B * T; ++row) {
            const int64_t t = row % T;
            for (int64_t c = 0; c < C; ++c) {
                const double cur = (double)x[row * C + c];
                const double prev = (t == 0) ? 0.0 : (double)x[(row - 1) * C + c];
                ki[c] = cur + (prev - cur) * (double)key_scale[c];
            }
            for (int64_t f = 0; f < F; ++f) {
                double acc = 0.0;
                for (int64_t c = 0; c < C; ++c) acc += ki[c] * (double)key_weight[f * C + c];
                acc = acc > 0.0 ? acc : 0.0;
                hid[f] = acc * acc;
            }
            for (int64_t c = 0; c < C; ++c) {
                double acc = 0.0;
                for (int64_t f = 0; f < F; ++f) acc += hid[f] * (double)value_weight[c * F + f];
                out[row * C + c] = acc;
            }
        }
        free(ki);
        free(hid);
    }
}

/* ------------------------------------------------------ token_shift_diff -- */

/*
 * token_shift_diff (token_shift_diff/mod.rs:65-81,114-155,170-200; kernel.rs:30-44):
 *   prev[b,0,:] = state[ids[b],:]; prev[b,t,:] = x[b,t-1,:];
 *   diff = prev - x;  state[ids[b],:] = x[b,T-1,:]; other rows unchanged;
 *   T == 0 leaves everything unchanged.  The subtraction of two floats is exact
 *   in double, so rounding the result to float gives the float result.
 * state is updated in place, as the reference kernel does.
 */
void oracle_token_shift_diff_f32(const float *x, float *state, const int64_t *ids,
                                 float *diff, int64_t B, int64_t T, int64_t C) {
    if (T == 0) return;
    for (int64_t bi = 0; bi < B; ++bi) {
        float *srow = state + ids[bi] * C;
        for (int64_t t = 0; t < T; ++t) {
            const float *cur = x + (bi * T + t) * C;
            const float *prev = (t == 0) ? srow : cur - C;
            float *o = diff + (bi * T + t) * C;
            for (int64_t c = 0; c < C; ++c) o[c] = prev[c] - cur[c];
        }
        memcpy(srow, x + (bi * T + T - 1) * C, sizeof(float) * (size_t)C);
    }
}

/* ------------------------------------------------------------ lm_head_ce -- */

/*
 * LM-head cross entropy (own specification; the reference file is empty):
 *   z[row][v] = sum_c x[row][c] * W[v][c]        (double accumulation)
 *   lse[row]  = log sum_v exp(z[row][v])
 *   loss[row] = lse[row] - z[row][target[row]]   (target < 0 -> loss 0, ignored)
 * W covers vocabulary rows [0, V).
 */
void oracle_lm_head_ce_f64(const float *x, const float *W, const int64_t *target,
                           double *lse, double *loss, int64_t R, int64_t C, int64_t V) {
#pragma omp parallel
    {
        double *z = (double *)malloc(sizeof(double) * (size_t)V);
#pragma omp for schedule(static)
        for (int64_t row = 0; row < R; ++row) {
            const float *xr = x + row * C;
            double m = -INFINITY;
            for (int64_t vv = 0; vv < V; ++vv) {
                const float *wr = W + vv * C;
                double acc = 0.0;
                for (int64_t c = 0; c < C; ++c) acc += (double)xr[c] * (double)wr[c];
                z[vv] = acc;
                if (acc > m) m = acc;
            }
            double s = 0.0;
            for (int64_t vv = 0; vv < V; ++vv) s += exp(z[vv] - m);
            lse[row] = m + log(s);
            const int64_t tg = target[row];
            loss[row] = (tg >= 0 && tg < V) ? lse[row] - z[tg] : 0.0;
        }
        free(z);
    }
}

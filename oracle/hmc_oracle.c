/*
 * CPU oracle for the HMC hot path of NVIDIA/mcmc-bnn-example.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C with double
 * accumulation, the arithmetic the reference performs in CUDA device code.
 * It is the checker the GPU library is compared with; nothing in the product
 * path links, loads or calls it.  Only the test-suite, the smoke check and the
 * benchmark's CPU-baseline leg may use it.
 *
 * Parity PINNED: the reference ships no tests, golden vectors or CPU code, so the
 * oracle is pinned against outputs of the reference's own FP32 kernel
 * (`leapfrog_step_kernel`, built unmodified from its headers by
 * oracle/ref_harness.cu and run on a B200); the captured vectors live in
 * tests/golden/ and tests/test_oracle_golden.py checks this file against them.
 *
 * Reference lines each function follows (paths inside the reference project):
 *   tanh with identity branch ............ include/mcmc/kernel_helpers.h:32-44
 *   leapfrog update + prior .............. include/mcmc/mcmc_step_ffma.h:106-152
 *   forward, loss, backward .............. include/mcmc/mcmc_step_ffma.h:225-370
 *   step scheduling (half first kick) .... include/mcmc/mcmc_step_ffma.h:395-427
 *   TF32 operand truncation .............. include/mcmc/mcmc_step_tc.h:362-396,529-555
 *   accept ratio ......................... include/mcmc/kernel_helpers.h:153-188
 *   driver loop, accept/reject, adaptation include/mcmc/main.h:191-283
 *   final loss evaluation ................ include/mcmc/main.h:78-115
 *   constants ............................ include/mcmc/global_params.h:27-58
 *
 * Parameter vector layout (P = D*H + 2H + 1 floats), as in the reference:
 *   W0[k][j] at k*H + j (input-major), b0[j] at D*H + j, W1[j] at D*H + H + j,
 *   b1 at D*H + 2H.   X is row-major [N][D], y is [N].
 *
 * Sign convention (reference): "loss" is a log-density that is maximised;
 * gradients are d(log p)/dw; momentum update is m += eps * grad.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

enum { ORACLE_LIK_STUDENT_T = 0, ORACLE_LIK_GAUSSIAN = 1 };

typedef struct {
  int32_t D;            /* input features (22) */
  int32_t H;            /* hidden units (40 or 128) */
  int32_t likelihood;   /* ORACLE_LIK_* */
  int32_t tf32;         /* 1: truncate the operands of both contractions to TF32 */
  double lik_scale;     /* Student-t scale, or Gaussian sigma */
  double lik_df;        /* Student-t degrees of freedom */
  double prior_scale;   /* sigma of the N(0, s^2) prior */
} oracle_model;

typedef struct {
  int32_t leapfrog_steps;
  int32_t adapt_steps;      /* iterations with step-size adaptation (reference: 100) */
  double eps0;              /* initial step size */
  double target_rate;       /* 0.2  */
  double decrement;         /* 0.1  */
  double increment;         /* 0.01 */
} oracle_sampler;

ORACLE_API int oracle_num_params(int D, int H) { return D * H + 2 * H + 1; }

/* log-normalisers; equal to the reference's hard-coded constants for its preset
 * (global_params.h:40-52): 5.63448313353184 and 6.21725589975271. */
ORACLE_API double oracle_lik_norm(const oracle_model* m) {
  const double pi = 3.14159265358979323846;
  if (m->likelihood == ORACLE_LIK_STUDENT_T)
    return log(fabs(m->lik_scale)) + 0.5 * log(m->lik_df) + 0.5 * log(pi) +
           lgamma(0.5 * m->lik_df) - lgamma(0.5 * (m->lik_df + 1.0));
  return 0.5 * log(2.0 * pi) + log(m->lik_scale);
}
ORACLE_API double oracle_prior_norm(const oracle_model* m) {
  const double pi = 3.14159265358979323846;
  return 0.5 * log(2.0 * pi) + log(m->prior_scale);
}

/* kernel_helpers.h:32-44 — tanh(x) as 2*sigmoid(2x)-1, returning x itself for
 * |x| below the cut-off.  The approximate PTX ops are replaced by exact math. */
ORACLE_API double oracle_tanh(double x) {
  const double cut = (double)0.0048176045529544353485f;
  return fabs(x) < cut ? x : tanh(x);
}

/* TF32 as the tensor core sees raw FP32 bits: the low 13 mantissa bits are
 * ignored (mcmc_step_tc.h:374,386,539,546 move FP32 bit patterns unchanged). */
static inline double tf32_trunc(double v) {
  float f = (float)v;
  uint32_t u;
  memcpy(&u, &f, 4);
  u &= 0xFFFFE000u;
  memcpy(&f, &u, 4);
  return (double)f;
}

/* Per-row log-likelihood and its derivative w.r.t. the prediction
 * (mcmc_step_ffma.h:289-301 for Student-t; the Gaussian case is the same
 * construction with the Gaussian density). */
static inline void lik_terms(const oracle_model* m, double norm, double y, double pred,
                             double* loss, double* dpred) {
  if (m->likelihood == ORACLE_LIK_STUDENT_T) {
    double d = (y - pred) / m->lik_scale;
    double d2 = d * d;
    *loss = -0.5 * (m->lik_df + 1.0) * log1p(d2 / m->lik_df) - norm;
    *dpred = (m->lik_df + 1.0) / m->lik_scale * d / (d2 + m->lik_df);
  } else {
    double d = (y - pred) / m->lik_scale;
    *loss = -0.5 * d * d - norm;
    *dpred = d / m->lik_scale;
  }
}

/*
 * log p(w | X, y) split into its two sums, and the full gradient
 * (likelihood + prior), rows [row0, row1) only (row sharding: the prior part
 * is added when add_prior != 0).
 *   row_loss   : optional [N] per-row log-likelihood (written for the rows visited)
 *   prior_loss : optional [P] per-parameter log-prior
 *   grad       : [P] doubles
 */
ORACLE_API void oracle_logp_grad_rows(const oracle_model* m, int64_t N, const float* X, const float* y,
                                      const float* w, int64_t row0, int64_t row1, int add_prior,
                                      double* loglik, double* logprior, double* grad,
                                      float* row_loss, float* prior_loss) {
  (void)N;
  const int D = m->D, H = m->H;
  const int P = oracle_num_params(D, H);
  const float* W0 = w;
  const float* b0 = w + D * H;
  const float* W1 = b0 + H;
  const double b1 = w[D * H + 2 * H];
  const double lnorm = oracle_lik_norm(m);
  double* W0e = (double*)malloc(sizeof(double) * D * H);
  for (int i = 0; i < D * H; ++i) W0e[i] = m->tf32 ? tf32_trunc(W0[i]) : (double)W0[i];

  int nthreads = 1;
#ifdef _OPENMP
  nthreads = omp_get_max_threads();
#endif
  double* gpart = (double*)calloc((size_t)nthreads * P, sizeof(double));
  double* lpart = (double*)calloc((size_t)nthreads, sizeof(double));

#pragma omp parallel
  {
    int tid = 0;
#ifdef _OPENMP
    tid = omp_get_thread_num();
#endif
    double* g = gpart + (size_t)tid * P;
    double* gW0 = g;
    double* gb0 = g + D * H;
    double* gW1 = gb0 + H;
    double* gb1 = g + D * H + 2 * H;
    double* h = (double*)malloc(sizeof(double) * H);
    double* xe = (double*)malloc(sizeof(double) * D);
    double ll = 0.0;
#pragma omp for schedule(static)
    for (int64_t r = row0; r < row1; ++r) {
      const float* x = X + r * D;
      for (int k = 0; k < D; ++k) xe[k] = m->tf32 ? tf32_trunc(x[k]) : (double)x[k];
      double pred = b1;
      for (int j = 0; j < H; ++j) {
        double z = b0[j];
        for (int k = 0; k < D; ++k) z += xe[k] * W0e[k * H + j];
        h[j] = oracle_tanh(z);
        pred += (double)W1[j] * h[j];
      }
      double loss, dy;
      lik_terms(m, lnorm, y[r], pred, &loss, &dy);
      if (row_loss) row_loss[r] = (float)loss;
      ll += loss;
      *gb1 += dy;
      for (int j = 0; j < H; ++j) {
        gW1[j] += dy * h[j];
        double dz = (1.0 - h[j] * h[j]) * ((double)W1[j] * dy); /* tanh_t::bwd */
        gb0[j] += dz;
        double dze = m->tf32 ? tf32_trunc(dz) : dz;
        for (int k = 0; k < D; ++k) gW0[k * H + j] += xe[k] * dze;
      }
    }
    lpart[tid] = ll;
    free(h);
    free(xe);
  }
  double ll = 0.0;
  for (int t = 0; t < nthreads; ++t) ll += lpart[t];
  for (int p = 0; p < P; ++p) {
    double s = 0.0;
    for (int t = 0; t < nthreads; ++t) s += gpart[(size_t)t * P + p];
    grad[p] = s;
  }
  *loglik = ll;
  /* prior: mcmc_step_ffma.h:113-118 */
  double lp = 0.0;
  if (add_prior) {
    const double pnorm = oracle_prior_norm(m);
    const double s2 = m->prior_scale * m->prior_scale;
    for (int p = 0; p < P; ++p) {
      double q = (double)w[p] / m->prior_scale;
      double l = -0.5 * q * q - pnorm;
      if (prior_loss) prior_loss[p] = (float)l;
      lp += l;
      grad[p] += -(double)w[p] / s2;
    }
  }
  *logprior = lp;
  free(gpart);
  free(lpart);
  free(W0e);
}

ORACLE_API void oracle_logp_grad(const oracle_model* m, int64_t N, const float* X, const float* y,
                                 const float* w, double* loglik, double* logprior, double* grad,
                                 float* row_loss, float* prior_loss) {
  oracle_logp_grad_rows(m, N, X, y, w, 0, N, 1, loglik, logprior, grad, row_loss, prior_loss);
}

/* log p(w) in double without rounding anything to float: for finite-difference
 * self-checks of the gradient. */
ORACLE_API double oracle_logp_f64(const oracle_model* m, int64_t N, const float* X, const float* y,
                                  const double* w) {
  const int D = m->D, H = m->H;
  const int P = oracle_num_params(D, H);
  const double lnorm = oracle_lik_norm(m), pnorm = oracle_prior_norm(m);
  double total = 0.0;
  for (int64_t r = 0; r < N; ++r) {
    double pred = w[D * H + 2 * H];
    for (int j = 0; j < H; ++j) {
      double z = w[D * H + j];
      for (int k = 0; k < D; ++k) z += (double)X[r * D + k] * w[k * H + j];
      pred += w[D * H + H + j] * tanh(z);
    }
    double loss, dy;
    lik_terms(m, lnorm, y[r], pred, &loss, &dy);
    total += loss;
  }
  for (int p = 0; p < P; ++p) {
    double q = w[p] / m->prior_scale;
    total += -0.5 * q * q - pnorm;
  }
  return total;
}

/*
 * One call of the reference's mcmc_step<T, L> (mcmc_step_ffma.h:395-427):
 * L leapfrog steps; the first momentum kick is a half kick
 * (MOM_CORRECTION = 2), the closing half kick is NOT applied here (it lives in
 * the accept ratio).  State vectors are stored as FP32 between steps, as the
 * reference stores them; arithmetic in between is double.
 *   loss_values : optional [N + P]: per-row log-lik then per-parameter log-prior
 *                 at w_next (the reference's OUTPUT_LOSS launch).
 */
ORACLE_API void oracle_mcmc_step(const oracle_model* m, int64_t N, const float* X, const float* y,
                                 int L, double eps, const float* w_prev, const float* mom_prev,
                                 const float* grad_prev, float* w_next, float* mom_next,
                                 float* grad_cur, float* loss_values, double* loglik,
                                 double* logprior) {
  const int P = oracle_num_params(m->D, m->H);
  float* w = (float*)malloc(sizeof(float) * P);
  float* mo = (float*)malloc(sizeof(float) * P);
  float* g = (float*)malloc(sizeof(float) * P);
  double* gd = (double*)malloc(sizeof(double) * P);
  memcpy(w, w_prev, sizeof(float) * P);
  memcpy(mo, mom_prev, sizeof(float) * P);
  memcpy(g, grad_prev, sizeof(float) * P);
  const float epsf = (float)eps;
  double ll = 0, lp = 0;
  for (int s = 0; s < L; ++s) {
    const double corr = (s == 0) ? 2.0 : 1.0;
    for (int p = 0; p < P; ++p) {
      mo[p] = (float)((double)mo[p] + (double)epsf * (double)g[p] / corr);
      w[p] = (float)((double)w[p] + (double)epsf * (double)mo[p]);
    }
    const int last = (s == L - 1);
    oracle_logp_grad(m, N, X, y, w, &ll, &lp, gd, (last && loss_values) ? loss_values : NULL,
                     (last && loss_values) ? loss_values + N : NULL);
    for (int p = 0; p < P; ++p) g[p] = (float)gd[p];
  }
  memcpy(w_next, w, sizeof(float) * P);
  memcpy(mom_next, mo, sizeof(float) * P);
  memcpy(grad_cur, g, sizeof(float) * P);
  if (loglik) *loglik = ll;
  if (logprior) *logprior = lp;
  free(w); free(mo); free(g); free(gd);
}

/*
 * The reference's driver loop (main.h:191-283) with the random draws injected:
 *   momenta [n_iter][P]  : the N(0,1) momentum of each iteration (main.h:207-216)
 *   log_u   [n_iter]     : log of the uniform accept draw (main.h:235-239)
 * Outputs (all optional except samples):
 *   samples [n_iter][P]  : the chain state after the accept/reject of each
 *                          iteration (main.h:277-283 stores these once past burn-in)
 *   log_acpt[n_iter]     : accept log-ratio (kernel_helpers.h:163-175), as double
 *   accepted[n_iter]     : 1/0
 *   eps_trace[n_iter]    : the step size USED by each iteration
 *   loglik_trace/logprior_trace [n_iter] : log-density parts of the state kept
 */
ORACLE_API void oracle_hmc_chain(const oracle_model* m, const oracle_sampler* s, int64_t N,
                                 const float* X, const float* y, int n_iter, const float* momenta,
                                 const float* log_u, float* samples, double* log_acpt,
                                 int32_t* accepted, double* eps_trace, double* loglik_trace,
                                 double* logprior_trace) {
  const int P = oracle_num_params(m->D, m->H);
  const int L = s->leapfrog_steps;
  float* w_cur = (float*)calloc(P, sizeof(float));       /* main.h:52,182: start at w = 0 */
  float* g_cur = (float*)calloc(P, sizeof(float));
  float* loss_cur = (float*)calloc((size_t)N + P, sizeof(float));
  float* w_new = (float*)calloc(P, sizeof(float));
  float* m_new = (float*)calloc(P, sizeof(float));
  float* g_new = (float*)calloc(P, sizeof(float));
  float* loss_new = (float*)calloc((size_t)N + P, sizeof(float));
  double* gd = (double*)calloc(P, sizeof(double));
  double ll_cur, lp_cur, ll_new, lp_new;
  /* bootstrap (main.h:191-202): log p and its gradient at the initial state */
  oracle_logp_grad(m, N, X, y, w_cur, &ll_cur, &lp_cur, gd, loss_cur, loss_cur + N);
  for (int p = 0; p < P; ++p) g_cur[p] = (float)gd[p];
  float eps = (float)s->eps0;
  for (int it = 0; it < n_iter; ++it) {
    const float* m0 = momenta + (size_t)it * P;
    if (eps_trace) eps_trace[it] = (double)eps;
    oracle_mcmc_step(m, N, X, y, L, (double)eps, w_cur, m0, g_cur, w_new, m_new, g_new, loss_new,
                     &ll_new, &lp_new);
    /* kernel_helpers.h:163-175: per-element loss differences, then the kinetic
     * difference with the closing half kick applied to the new momentum */
    double acc = 0.0;
    for (int64_t i = 0; i < N + P; ++i) acc += (double)loss_new[i] - (double)loss_cur[i];
    for (int p = 0; p < P; ++p) {
      double mf = (double)m_new[p] + (double)eps * (double)g_new[p] * 0.5;
      acc += 0.5 * ((double)m0[p] * (double)m0[p] - mf * mf);
    }
    const float h_log_acpt = (float)acc;
    const int ok = log_u[it] < h_log_acpt; /* main.h:242 */
    if (ok) {
      memcpy(w_cur, w_new, sizeof(float) * P);
      memcpy(g_cur, g_new, sizeof(float) * P);
      memcpy(loss_cur, loss_new, sizeof(float) * ((size_t)N + P));
      ll_cur = ll_new;
      lp_cur = lp_new;
    }
    if (log_acpt) log_acpt[it] = acc;
    if (accepted) accepted[it] = ok;
    if (loglik_trace) loglik_trace[it] = ll_cur;
    if (logprior_trace) logprior_trace[it] = lp_cur;
    /* main.h:266-276 */
    if (it < s->adapt_steps) {
      float lmr = h_log_acpt < 0.f ? h_log_acpt : 0.f;
      float dec = -(float)s->decrement / (1.f + (float)s->decrement);
      float inc = (float)s->increment;
      float adj = lmr < (float)log(s->target_rate) ? dec : inc;
      eps += eps * adj;
    }
    memcpy(samples + (size_t)it * P, w_cur, sizeof(float) * P);
  }
  free(w_cur); free(g_cur); free(loss_cur); free(w_new); free(m_new); free(g_new);
  free(loss_new); free(gd);
}

/* Network prediction b1 + W1 . tanh(W0^T x + b0) for every row, averaged over
 * S parameter samples (the posterior-mean prediction).  The reference only
 * evaluates losses over its stored samples (main.h:78-115); the forward pass
 * is the one of mcmc_step_ffma.h:225-281. */
ORACLE_API void oracle_predict_mean(const oracle_model* m, int64_t n, const float* Xs, int S,
                                    const float* samples, double* mean_pred) {
  const int D = m->D, H = m->H;
  const int P = oracle_num_params(D, H);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < n; ++r) {
    double acc = 0.0;
    for (int s = 0; s < S; ++s) {
      const float* w = samples + (size_t)s * P;
      double pred = w[D * H + 2 * H];
      for (int j = 0; j < H; ++j) {
        double z = w[D * H + j];
        for (int k = 0; k < D; ++k) {
          double a = Xs[r * D + k], b = w[k * H + j];
          if (m->tf32) { a = tf32_trunc(a); b = tf32_trunc(b); }
          z += a * b;
        }
        pred += (double)w[D * H + H + j] * oracle_tanh(z);
      }
      acc += pred;
    }
    mean_pred[r] = acc / (double)S;
  }
}

/* Mean log-likelihood and log-prior over stored samples: output_final_loss,
 * main.h:78-115 (running means on the host there; plain means here). */
ORACLE_API void oracle_final_loss(const oracle_model* m, int64_t N, const float* X, const float* y,
                                  int S, const float* samples, double* mean_loglik,
                                  double* mean_logprior) {
  const int P = oracle_num_params(m->D, m->H);
  double* gd = (double*)malloc(sizeof(double) * P);
  double a = 0, b = 0;
  for (int s = 0; s < S; ++s) {
    double ll, lp;
    oracle_logp_grad(m, N, X, y, samples + (size_t)s * P, &ll, &lp, gd, NULL, NULL);
    a += ll;
    b += lp;
  }
  *mean_loglik = a / S;
  *mean_logprior = b / S;
  free(gd);
}

/* ------------------------------------------------------------------------- *
 * FP32 host transcription of the same path, threaded over row blocks: the
 * timed CPU baseline (the reference has no CPU implementation of its model;
 * all of its arithmetic is CUDA device code).  Same math as above in float,
 * with the reference's tanh formula (kernel_helpers.h:36-43) on exp2f.
 * ------------------------------------------------------------------------- */
static inline float tanh_ref_f32(float x) {
  float e = exp2f(x * -2.88539008177792681472f);
  float sg = 1.0f / (1.0f + e);
  return fabsf(x) < 0.0048176045529544353485f ? x : sg * 2.f - 1.f;
}

#define PORT_MAX_H 128
#define PORT_MAX_D 32

/* gradient of the log-likelihood part + its sum, rows [0, N); prior added by caller */
static void port_f32_lik_grad(const oracle_model* m, int64_t N, const float* X, const float* y,
                              const float* w, float* grad, double* loglik) {
  const int D = m->D, H = m->H;
  const int P = oracle_num_params(D, H);
  const float lnorm = (float)oracle_lik_norm(m);
  const float* W0 = w;
  const float* b0 = w + D * H;
  const float* W1 = b0 + H;
  const float b1 = w[D * H + 2 * H];
  const int gauss = m->likelihood == ORACLE_LIK_GAUSSIAN;
  const float sc_r = (float)(1.0 / m->lik_scale), df = (float)m->lik_df;
  int nthreads = 1;
#ifdef _OPENMP
  nthreads = omp_get_max_threads();
#endif
  float* gpart = (float*)calloc((size_t)nthreads * P, sizeof(float));
  double* lpart = (double*)calloc((size_t)nthreads, sizeof(double));
#pragma omp parallel
  {
    int tid = 0;
#ifdef _OPENMP
    tid = omp_get_thread_num();
#endif
    float* g = gpart + (size_t)tid * P;
    float* gW0 = g;
    float* gb0 = g + D * H;
    float* gW1 = gb0 + H;
    float h[PORT_MAX_H], dz[PORT_MAX_H];
    double ll = 0.0;
    float gb1 = 0.f;
#pragma omp for schedule(static)
    for (int64_t r = 0; r < N; ++r) {
      const float* x = X + r * D;
      for (int j = 0; j < H; ++j) h[j] = b0[j];
      for (int k = 0; k < D; ++k) {
        const float xv = x[k];
        const float* wr = W0 + k * H;
        for (int j = 0; j < H; ++j) h[j] += xv * wr[j];
      }
      float pred = b1;
      for (int j = 0; j < H; ++j) {
        h[j] = tanh_ref_f32(h[j]);
        pred += W1[j] * h[j];
      }
      float d = (y[r] - pred) * sc_r, dy, loss;
      if (gauss) {
        loss = -0.5f * d * d - lnorm;
        dy = d * sc_r;
      } else {
        float d2 = d * d;
        loss = -0.5f * (df + 1.f) * log1pf(d2 / df) - lnorm;
        dy = (df + 1.f) * sc_r * d / (d2 + df);
      }
      ll += (double)loss;
      gb1 += dy;
      for (int j = 0; j < H; ++j) {
        gW1[j] += dy * h[j];
        dz[j] = (1.f - h[j] * h[j]) * (W1[j] * dy);
        gb0[j] += dz[j];
      }
      for (int k = 0; k < D; ++k) {
        const float xv = x[k];
        float* gr = gW0 + k * H;
        for (int j = 0; j < H; ++j) gr[j] += xv * dz[j];
      }
    }
    g[D * H + 2 * H] = gb1;
    lpart[tid] = ll;
  }
  double ll = 0;
  for (int t = 0; t < nthreads; ++t) ll += lpart[t];
  for (int p = 0; p < P; ++p) {
    float sacc = 0.f;
    for (int t = 0; t < nthreads; ++t) sacc += gpart[(size_t)t * P + p];
    grad[p] = sacc;
  }
  *loglik = ll;
  free(gpart);
  free(lpart);
}

/*
 * FP32 port of whole HMC iterations on one window (bootstrap + n_iter
 * iterations of L leapfrog steps, accept/reject with injected draws).
 * Returns the number of accepted proposals; `samples` optional [n_iter][P].
 * Used only for timing the CPU baseline and for a sanity cross-check with the
 * double oracle.
 */
ORACLE_API int oracle_port_f32_chain(const oracle_model* m, const oracle_sampler* s, int64_t N,
                                     const float* X, const float* y, int n_iter,
                                     const float* momenta, const float* log_u, float* samples,
                                     int nthreads) {
#ifdef _OPENMP
  if (nthreads > 0) omp_set_num_threads(nthreads);
#else
  (void)nthreads;
#endif
  if (m->H > PORT_MAX_H || m->D > PORT_MAX_D) return -1;
  const int P = oracle_num_params(m->D, m->H);
  const int L = s->leapfrog_steps;
  const float ps2 = (float)(1.0 / (m->prior_scale * m->prior_scale));
  const float pnorm = (float)oracle_prior_norm(m);
  float* w_cur = (float*)calloc(P, sizeof(float));
  float* g_cur = (float*)calloc(P, sizeof(float));
  float* w = (float*)calloc(P, sizeof(float));
  float* mo = (float*)calloc(P, sizeof(float));
  float* g = (float*)calloc(P, sizeof(float));
  double ll_cur, ll_new = 0, lp_cur = 0, lp_new = 0;
  port_f32_lik_grad(m, N, X, y, w_cur, g_cur, &ll_cur);
  for (int p = 0; p < P; ++p) {
    float q = w_cur[p] / (float)m->prior_scale;
    lp_cur += (double)(-0.5f * q * q - pnorm);
    g_cur[p] += -w_cur[p] * ps2;
  }
  float eps = (float)s->eps0;
  int n_acc = 0;
  for (int it = 0; it < n_iter; ++it) {
    const float* m0 = momenta + (size_t)it * P;
    memcpy(w, w_cur, sizeof(float) * P);
    memcpy(mo, m0, sizeof(float) * P);
    memcpy(g, g_cur, sizeof(float) * P);
    for (int st = 0; st < L; ++st) {
      const float corr = st == 0 ? 0.5f : 1.f;
      for (int p = 0; p < P; ++p) {
        mo[p] += eps * g[p] * corr;
        w[p] += eps * mo[p];
      }
      port_f32_lik_grad(m, N, X, y, w, g, &ll_new);
      lp_new = 0;
      for (int p = 0; p < P; ++p) {
        float q = w[p] / (float)m->prior_scale;
        lp_new += (double)(-0.5f * q * q - pnorm);
        g[p] += -w[p] * ps2;
      }
    }
    double acc = (ll_new - ll_cur) + (lp_new - lp_cur);
    for (int p = 0; p < P; ++p) {
      float mf = mo[p] + eps * g[p] * 0.5f;
      acc += 0.5 * ((double)m0[p] * m0[p] - (double)mf * mf);
    }
    const float la = (float)acc;
    if (log_u[it] < la) {
      memcpy(w_cur, w, sizeof(float) * P);
      memcpy(g_cur, g, sizeof(float) * P);
      ll_cur = ll_new;
      lp_cur = lp_new;
      ++n_acc;
    }
    if (it < s->adapt_steps) {
      float lmr = la < 0.f ? la : 0.f;
      float adj = lmr < (float)log(s->target_rate)
                      ? -(float)s->decrement / (1.f + (float)s->decrement)
                      : (float)s->increment;
      eps += eps * adj;
    }
    if (samples) memcpy(samples + (size_t)it * P, w_cur, sizeof(float) * P);
  }
  free(w_cur); free(g_cur); free(w); free(mo); free(g);
  return n_acc;
}

/* FP32 port: one gradient (likelihood + prior) — timed per-gradient baseline. */
ORACLE_API void oracle_port_f32_grad(const oracle_model* m, int64_t N, const float* X, const float* y,
                                     const float* w, float* grad, double* loglik, int nthreads) {
#ifdef _OPENMP
  if (nthreads > 0) omp_set_num_threads(nthreads);
#else
  (void)nthreads;
#endif
  const int P = oracle_num_params(m->D, m->H);
  const float ps2 = (float)(1.0 / (m->prior_scale * m->prior_scale));
  port_f32_lik_grad(m, N, X, y, w, grad, loglik);
  for (int p = 0; p < P; ++p) grad[p] += -w[p] * ps2;
}

ORACLE_API int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

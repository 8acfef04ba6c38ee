/*
 * mcmc_b200 — C-ABI of the B200 (sm_100a) HMC hot path for the two-layer
 * Bayesian MLP of NVIDIA/mcmc-bnn-example.
 *
 * The reference has no FFI layer: its boundary is the C++ header API under
 * include/mcmc/ (mcmc_step, log_acpt_prec, main_loop, Network, DeviceMatrix).
 * Every entry point below names the reference interface it stands in for
 * (paths inside the reference project).  All functions return an
 * MCMC_B200_* status; nothing aborts the process (the reference aborts in
 * include/mcmc/utils_cuda.h:30-46).  Plain pointers and sizes only.
 *
 * Conventions shared with the reference:
 *   - parameter vector of P = D*H + 2H + 1 floats: W0[k][j] at k*H + j, b0 at
 *     D*H, W1 at D*H + H, b1 at D*H + 2H (mcmc_step_ffma.h:35-44, :244);
 *   - X is row-major [N][D] FP32, y is [N] FP32;
 *   - "loss" is a log-density that is maximised, gradients are d(log p)/dw,
 *     the momentum update is m += eps * grad (mcmc_step_ffma.h:106-120).
 *
 * One host thread per context at a time.  Contexts are independent.
 */
#ifndef MCMC_B200_H_
#define MCMC_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MCMC_B200_OK 0
#define MCMC_B200_ERR_INVALID 1      /* bad argument or call order */
#define MCMC_B200_ERR_CUDA 2         /* a CUDA runtime/driver call failed */
#define MCMC_B200_ERR_NOMEM 3
#define MCMC_B200_ERR_TIMEOUT 4      /* a bounded device-side wait ran out */
#define MCMC_B200_ERR_NCCL 5
#define MCMC_B200_ERR_UNSUPPORTED 6  /* shape / mode not built */

#define MCMC_B200_LIK_STUDENT_T 0    /* global_params.h:39-45 */
#define MCMC_B200_LIK_GAUSSIAN 1

#define MCMC_B200_RNG_PHILOX 0       /* counter-based, keyed by (seed, global window, iteration): the default */
#define MCMC_B200_RNG_REFERENCE 1    /* the reference's own streams (main.h:207-216, :235-239), see below */

#define MCMC_B200_PREC_FP32 0        /* FFMA path; stands in for mcmc_step_ffma.h */
#define MCMC_B200_PREC_TF32 1        /* tcgen05 kind::tf32 path; stands in for mcmc_step_tc.h */

/* Everything the reference fixes at compile time in global_params.h:27-58. */
typedef struct mcmc_b200_config {
  int32_t D;               /* input features; 22 */
  int32_t H;               /* hidden units; 40 (or 128) */
  int32_t likelihood;      /* MCMC_B200_LIK_* */
  int32_t precision;       /* MCMC_B200_PREC_* */
  double lik_scale;        /* Student-t scale (100) or Gaussian sigma */
  double lik_df;           /* Student-t degrees of freedom (2.2) */
  double prior_scale;      /* sigma of the N(0, s^2) prior (200) */
  int32_t leapfrog_steps;  /* LEAPFROG_STEPS (1000) */
  int32_t burn_in;         /* BURN_IN_STEPS (100): iterations whose state is not stored */
  int32_t adapt_steps;     /* STEP_SIZE_ADAPT_STEPS (100) */
  int32_t sample_capacity; /* stored samples per window (SAMPLE_STEPS, 800); 0 = store none */
  double eps0;             /* STEP_SIZE_INIT (0.01) */
  double target_rate;      /* STEP_SIZE_TARGET_RATE (0.2) */
  double decrement;        /* STEP_SIZE_DECREMENT (0.1) */
  double increment;        /* STEP_SIZE_INCREMENT (0.01) */
  uint64_t seed;           /* SEED_INIT; keys the Philox streams */
  int32_t trace_iters;     /* first K iterations whose draws and energies are recorded */
  int32_t slices;          /* pieces each window is cut into per launch; 0 = chosen from the SM count
                              (fastest).  A fixed value makes a window's results bit-identical
                              however many windows share the context or the GPU. */
  int32_t rng_streams;     /* MCMC_B200_RNG_*: which random streams drive the chain */
} mcmc_b200_config;

/* Fills a config with the reference's shipped preset (global_params.h:27-58)
 * or with the Gaussian/N(0,1)/L=10/eps=1e-3 benchmark preset. */
void mcmc_b200_config_reference(mcmc_b200_config* cfg);
void mcmc_b200_config_baseline(mcmc_b200_config* cfg);

typedef struct mcmc_b200_ctx mcmc_b200_ctx;

/* Library-wide: last error text of the calling thread (also set by failed
 * create calls, where no context exists yet). */
const char* mcmc_b200_last_error(void);
/* 1 when the library was built with the tcgen05 kernels for sm_100a. */
int mcmc_b200_has_tf32(void);

/*
 * Context = the reference's per-process state (main.h:153-183: data, labels,
 * Network, loss buffers, prev_step_*, final_samples) for `n_windows`
 * independent windows of `rows` rows each, on CUDA device `device`.
 * Stands in for the allocations of main_loop (main.h:117-185).
 */
int mcmc_b200_create(const mcmc_b200_config* cfg, int device, int n_windows, int64_t rows,
                     mcmc_b200_ctx** out);
void mcmc_b200_destroy(mcmc_b200_ctx* ctx);

/* P for this context's model. */
int mcmc_b200_num_params(const mcmc_b200_ctx* ctx);

/*
 * Uploads one window's dataset.  Stands in for read_data + the H2D copies
 * (io.h:42-86) — the file parsing itself is not part of this library.
 * `global_window` keys the random streams, so a window gives the same chain
 * wherever it is placed.  x/y may be host or device pointers (is_device).
 * The library keeps its own repacked copy ([rows][24] floats: 22 features,
 * a constant 1 and y); the caller's buffers are not referenced afterwards.
 */
int mcmc_b200_set_window_data(mcmc_b200_ctx* ctx, int window, int64_t global_window,
                              const float* x, const float* y, int is_device);

/*
 * log p and its gradient at w, without touching the chain state: the
 * reference's loss-only idiom mcmc_step<T,1> with eps = 0 on a zeroed Network
 * (main.h:85-99) followed by get_loss_values (kernel_helpers.h:190-216).
 *   w        [P] host
 *   loglik   sum of per-row log-likelihoods      (loss_values[0..N))
 *   logprior sum of per-parameter log-priors     (loss_values[N..N+P))
 *   grad     [P] host, likelihood + prior gradient (grad_cur)
 *   row_loss optional [rows] host
 */
int mcmc_b200_potential_and_grad(mcmc_b200_ctx* ctx, int window, const float* w, double* loglik,
                                 double* logprior, float* grad, float* row_loss);

/*
 * L leapfrog steps on explicit host state: mcmc_step<T,L>
 * (mcmc_step_ffma.h:395-427 / mcmc_step_tc.h:679-696).  First kick is a half
 * kick with grad_prev, the closing half kick is NOT applied (it belongs to the
 * accept ratio, kernel_helpers.h:163-175).  All vectors [P] host.
 */
int mcmc_b200_leapfrog(mcmc_b200_ctx* ctx, int window, int L, float eps, const float* w_prev,
                       const float* mom_prev, const float* grad_prev, float* w_next,
                       float* mom_next, float* grad_cur, double* loglik, double* logprior);

/*
 * Runs `n_iter` further HMC iterations on every window of the context:
 * main_loop's sampling loop (main.h:204-287) with momentum draw, L leapfrog
 * steps, accept ratio, accept/reject, step-size adaptation and sample store
 * all on the device.  The first call also does the bootstrap evaluation at
 * w = 0 (main.h:191-202).  Returns after the device work has finished.
 */
int mcmc_b200_run_chain(mcmc_b200_ctx* ctx, int n_iter);
/* Same, but returns as soon as the work is queued on the context's stream. */
int mcmc_b200_run_chain_async(mcmc_b200_ctx* ctx, int n_iter);
int mcmc_b200_synchronize(mcmc_b200_ctx* ctx);
/* The CUDA stream (cudaStream_t) all of this context's work is queued on. */
void* mcmc_b200_stream(mcmc_b200_ctx* ctx);
/* Restarts every chain at w = 0, iteration 0 (the data stays). */
int mcmc_b200_reset_chain(mcmc_b200_ctx* ctx);

/* Iterations done so far, accepted proposals and the current step size. */
int mcmc_b200_chain_info(mcmc_b200_ctx* ctx, int window, int32_t* iterations, int32_t* accepted,
                         float* eps);
/* Current chain state [P] (prev_step_w, main.h:180) and its log-density parts. */
int mcmc_b200_get_state(mcmc_b200_ctx* ctx, int window, float* w, float* grad, double* loglik,
                        double* logprior);
/* Stored samples (final_samples, main.h:183,277-283): `count` vectors of P
 * floats starting at stored sample `first`, into host memory. */
int mcmc_b200_get_samples(mcmc_b200_ctx* ctx, int window, int first, int count, float* out);
/*
 * Trace of the first cfg.trace_iters iterations: what a parity test needs to
 * replay the chain on the CPU with the same draws.
 *   momenta  optional [count][P]: the N(0,1) momentum drawn for each iteration
 *   log_u    optional [count]   : log of the accept uniform
 *   log_acpt optional [count]   : accept log-ratio (kernel_helpers.h:163-175)
 *   accepted optional [count]
 *   eps      optional [count]   : step size used by the iteration
 */
int mcmc_b200_get_trace(mcmc_b200_ctx* ctx, int window, int first, int count, float* momenta,
                        float* log_u, double* log_acpt, int32_t* accepted, float* eps);

/*
 * Posterior-mean prediction: mean over stored samples [first, first+count) of
 * the network output for each of n rows of xs ([n][D] host).  The reference
 * evaluates only losses over its stored samples (output_final_loss,
 * main.h:78-115); this is the matching forward-only pass.
 */
int mcmc_b200_predict_mean(mcmc_b200_ctx* ctx, int window, const float* xs, int64_t n, int first,
                           int count, float* out);
/* Mean log-likelihood / log-prior over stored samples: output_final_loss
 * (main.h:78-115). */
int mcmc_b200_final_loss(mcmc_b200_ctx* ctx, int window, int first, int count, double* mean_loglik,
                         double* mean_logprior);

/*
 * Work partition of the persistent TF32 kernels, for inspection and tests (host
 * arithmetic only, needs no GPU).  A launch covers `windows` windows of
 * `tiles_per_window` 128-row tiles with at most max_ctas CTAs; CTA b owns the
 * segments seg_ptr[b] .. seg_ptr[b+1]-1, a segment is {window, first tile, end
 * tile, slot} (slot = index of this CTA's partial-gradient vector within the
 * window).  slices = 0: contiguous ranges balanced by cost (tiles plus a fixed
 * cost per segment); slices > 0: every window cut into that many fixed chunks
 * (results then do not depend on what else shares the launch).  The reference's
 * counterpart is the compile-time N_BLKS / N_WARP_SAMPLES grid arithmetic
 * (mcmc_step_ffma.h:40-52, mcmc_step_tc.h:145-155).  Either output array may be
 * null to query the counts only.
 */
int mcmc_b200_plan_work_table(int windows, int64_t tiles_per_window, int max_ctas, int slices,
                              int32_t* seg_ptr_out, int seg_ptr_capacity, int32_t* segs_out,
                              int segs_capacity, int32_t* n_ctas, int32_t* n_segs);

/*
 * Dataset text reader: the layout the reference's read_data scans
 * (io.h:42-80, sizes in global_params.h:61-65 there).  Whitespace-separated
 * tokens: total_cols header tokens (ignored), then `rows` rows of total_cols
 * tokens, of which the first skip_cols are ignored, the next one is the label,
 * the next D are the features and the rest is ignored.  Features are
 * multiplied by feature_scale (the reference scales by 0.001 in a separate
 * device pass, main.h:162-164).  x_out [rows][D] and y_out [rows] are host
 * arrays.  Host-only: needs no GPU.  The reference aborts on a missing file;
 * this returns MCMC_B200_ERR_INVALID with the reason in last_error.
 */
int mcmc_b200_read_table(const char* path, int64_t rows, int total_cols, int skip_cols, int D,
                         float feature_scale, float* x_out, float* y_out);

/*
 * Checkpoint / resume.  The reference keeps samples and chain state in device
 * memory only and loses them when the process ends (main.h:183,277-283,295).
 * A checkpoint is one host blob: a fixed header (configuration fingerprint,
 * iterations done) followed by every window's position, momentum, carried
 * gradient and energies, step size, counters, stored samples and trace.  The
 * dataset is NOT part of it: upload every window's data (same global window
 * ids) before loading.  Because every random draw is a pure function of
 * (seed, global window, iteration), a resumed chain continues bit-identically.
 *   size : bytes a save needs for this context
 *   save : synchronises the context, writes the blob to host_buf
 *   load : checks the header against this context's configuration, restores
 */
int mcmc_b200_checkpoint_size(mcmc_b200_ctx* ctx, uint64_t* bytes);
int mcmc_b200_checkpoint_save(mcmc_b200_ctx* ctx, void* host_buf, uint64_t bytes);
int mcmc_b200_checkpoint_load(mcmc_b200_ctx* ctx, const void* host_buf, uint64_t bytes);

/*
 * Row sharding of ONE window over several GPUs (one process per GPU): every
 * rank holds rows/nranks rows, and each leapfrog step sums the P-vector of
 * gradient partials (plus the log-likelihood) over ranks with one NCCL
 * allreduce.  The reference has no multi-GPU code; this is the mode its README
 * table implies.  Rank 0 makes the id, the caller broadcasts the 128 bytes.
 */
int mcmc_b200_nccl_unique_id(unsigned char id[128]);
int mcmc_b200_enable_row_sharding(mcmc_b200_ctx* ctx, const unsigned char id[128], int rank,
                                  int nranks);
/*
 * Replaces the NCCL call of a row-sharded context (after mcmc_b200_enable_row_sharding, before the chain
 * starts) by a one-shot all-reduce over peer memory: one launch per leapfrog step sums this rank's
 * partials, stores them into every rank's receive buffer with plain 8-byte stores over NVLink (buffers
 * exchanged as CUDA IPC handles over the communicator; every store carries the exchange's sequence number,
 * so no separate flag or fence is needed), and adds the ranks' contributions in rank order after a
 * bounded wait, so every rank holds identical bits.  An all-reduce of 7.7 KB is latency, not bandwidth:
 * this takes a few microseconds where the library call takes about 25 on 8 GPUs.  Needs peer access
 * between the GPUs (one process per GPU; never two ranks on one GPU: their kernels wait for one another).
 * A wait that runs out is reported as MCMC_B200_ERR_TIMEOUT by the next synchronising call.
 */
int mcmc_b200_enable_oneshot_allreduce(mcmc_b200_ctx* ctx);
/* Average device time in microseconds of the per-step reduction + all-reduce of a row-sharded context
 * (whichever of the two is enabled), from CUDA events around `reps` of them on the context's stream.
 * Collective: every rank calls it with the same reps. */
int mcmc_b200_time_allreduce(mcmc_b200_ctx* ctx, int reps, float* us_per_call);
/* Self-test of the one-shot all-reduce's bounded wait on ONE GPU: a fresh one-window context pretends to
 * be rank 0 of 2, the other rank never sends, the wait runs out after `polls` polls and the call returns
 * MCMC_B200_ERR_TIMEOUT; the context is an ordinary unsharded one again afterwards. */
int mcmc_b200_selftest_oneshot_timeout(mcmc_b200_ctx* ctx, int polls);

/*
 * Drop-in for mcmc::mcmc_step<float, L> on caller-owned DEVICE buffers
 * (mcmc_step_ffma.h:395-402).  Same argument meaning: x [N][D], y [N],
 * grad_prev = complete gradient at weights_prev; on return weights_next,
 * mom_next, the gradient at weights_next in grad_cur, grad_next zeroed,
 * loss_values[0..N) per-row log-likelihood and [N..N+P) per-parameter
 * log-prior.  Unlike the reference the caller's buffer roles are NOT rotated:
 * outputs always land in the buffers named here.  Queued on `stream`.
 * The context must have been created with n_windows = 1 and rows = N.
 */
int mcmc_b200_mcmc_step(mcmc_b200_ctx* ctx, const float* x, const float* y, const float* weights_prev,
                        float* weights_next, const float* mom_prev, float* mom_next,
                        const float* grad_prev, float* grad_cur, float* grad_next,
                        float* loss_values, int L, float eps, void* stream);
/*
 * mcmc_b200_mcmc_step keeps a repacked copy of the dataset and recognises the
 * dataset by its two POINTERS: it repacks on the first call and whenever x or
 * y is a different address, not when the contents behind the same addresses
 * change.  A caller that loads the next window into the same buffers (the
 * "sequential passes" of main.h:302-307) calls this first: the next mcmc_step
 * repacks.  The reference reads x and y afresh on every launch and needs no
 * such call (mcmc_step_ffma.h:76-104).
 */
int mcmc_b200_rebind_data(mcmc_b200_ctx* ctx);
/*
 * Drop-in for mcmc::log_acpt_prec (kernel_helpers.h:153-188) on DEVICE
 * buffers: sum(new_loss - prev_loss) over n_loss entries plus the kinetic
 * difference with the closing half kick; returns the scalar on the host
 * (synchronises `stream`, as the reference does).
 */
int mcmc_b200_log_acpt(mcmc_b200_ctx* ctx, const float* prev_loss, const float* new_loss,
                       int64_t n_loss, const float* prev_mom, const float* new_mom,
                       const float* grad_cur, float eps, void* stream, float* out);

/*
 * log p and its gradient at w without any device allocation.  Has no
 * counterpart in the reference (which allocates freely, main.h:156-183).
 *
 * For hosts that must not enter the CUDA allocator while they evaluate the
 * model: an application that has given all GPU memory to its own arena, or a
 * latency-critical loop where cudaMalloc/cudaFree would synchronise the device
 * and stall every stream.  No context is needed: the scratch (repacked dataset,
 * per-CTA gradient partials) is a fixed ~7.7 MB array inside the library image,
 * held by every GPU that loads the library until the process exits.
 *   limits : rows <= 65536, D = 22, H = 40, cfg->precision = FP32 (others are refused)
 *   x [rows][22], y [rows], w [P] : DEVICE pointers (inputs)
 *   grad [P], loglik_logprior [2] : DEVICE pointers (outputs: gradient; sum of
 *                                   log-likelihoods, sum of log-priors)
 * Runs on the current device, queued on `stream`; returns without waiting.
 * The first call on a device looks up the array's address (once per device);
 * make that call before any stream capture.  All calls on a GPU share the one
 * array, which keeps the last call's contents: calls that overlap on the GPU
 * (other streams, other threads) race — serialise them.
 */
int mcmc_b200_potential_and_grad_static(const mcmc_b200_config* cfg, const float* x, const float* y,
                                        int64_t rows, const float* w, float* grad,
                                        double* loglik_logprior, void* stream);

/*
 * Synthetic window generator (host code, no GPU): X ~ N(0,1), teacher weights
 * ~ N(0, 0.3^2), y = teacher(X) + N(0, 0.05^2), all from Philox streams keyed
 * by (seed, window).  Stands in for the reference's missing data file
 * (global_params.h:65).  teacher is optional [P].
 */
int mcmc_b200_synth_window(uint64_t seed, int64_t window, int64_t rows, int D, int H, float* x,
                           float* y, float* teacher);
/* Host evaluation of the library's random streams (for tests). */
float mcmc_b200_philox_normal(uint64_t seed, uint32_t window, uint32_t iteration, uint32_t stream,
                              uint32_t index);
void mcmc_b200_philox_raw(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]);

/*
 * The same generator evaluated ON THE DEVICE, for tests that compare the two:
 * n (1..4096, n*5+1 <= the context's padded row count) raw Philox blocks for
 * counters {ctr[0]+i, ctr[1], ctr[2], ctr[3]}, the n momentum normals the accept
 * kernel draws for (seed = key, window = ctr[2], iteration = ctr[1]) and that
 * iteration's accept uniform.  Replaces nothing in the reference, whose
 * streams are Thrust's and libstdc++'s minstd engines (main.h:207-216,235-239).
 */
int mcmc_b200_philox_device(mcmc_b200_ctx* ctx, const uint32_t ctr[4], const uint32_t key[2], int n,
                            uint32_t* raw_out, float* normals_out, float* uniform_out);

/*
 * The reference's random streams (cfg.rng_streams = MCMC_B200_RNG_REFERENCE), for a black-box comparison
 * with the reference binary.  With rel = 962 * iteration (961 momenta + 1 accept draw per iteration,
 * main.h:155,216,237):
 *   momentum p of an iteration : a fresh Thrust default_random_engine (minstd_rand), discard(seed + rel + p),
 *                                one thrust::normal_distribution<float>(0,1) draw, on the device (main.h:207-216);
 *   accept draw                : a fresh std::default_random_engine (minstd_rand0) seeded seed + rel + 961, one
 *                                std::uniform_real_distribution<float>(FLT_MIN, 1) draw, log() in double on
 *                                the host (main.h:235-239).
 * Both generators belong to libraries the reference does not pin (Thrust / CCCL, libstdc++); this library
 * CALLS them (the copies of this toolchain) rather than restating them.  Every window of a context gets the
 * same streams, as every run of the reference binary does.  The two functions below expose the streams for
 * tests: the raw engine value after discard(n) / after seed(s), the normal and the log-uniform built on them.
 * The normal needs a GPU (it is Thrust's device code path that the reference runs); the rest is host code.
 */
int mcmc_b200_refstream_momentum_device(mcmc_b200_ctx* ctx, uint64_t first_n, int count, float* out);
uint32_t mcmc_b200_refstream_engine(uint64_t n_discard);            /* Thrust minstd_rand after discard(n) */
uint32_t mcmc_b200_refstream_engine0(uint64_t seed);                /* libstdc++ minstd_rand0 seeded, first value */
float mcmc_b200_refstream_log_uniform(uint64_t seed);               /* log of the accept draw for that seed */

/*
 * Device micro-benchmarks behind the roofline figures (no counterpart in the reference): the rate at
 * which all SMs re-read an L2-resident buffer of `bytes` (one window of the benchmark workload is 5.4 MB
 * and stays in the L2 between leapfrog steps), and the MUFU pipe's rate for the activation (kind 0:
 * tanh.approx.f32, one operation per value; kind 1: ex2.approx + rcp.approx, the two operations of the
 * reference's tanh, kernel_helpers.h:32-44), in 10^9 values per second.  Timed with CUDA events.
 */
int mcmc_b200_microbench_l2_read(int device, int64_t bytes, double* gb_per_s);
int mcmc_b200_microbench_mufu(int device, int kind, double* gvalues_per_s);

/* Counters for benchmarks: kernels of this library launched on the context
 * since creation (or since the last reset of the counter). */
int64_t mcmc_b200_launch_count(mcmc_b200_ctx* ctx, int reset);
/* How the context's chain launches are cut: partial-gradient slots per window,
 * resident CTAs per SM of the gradient kernel, rows per tile.  Any may be null. */
int mcmc_b200_chain_geometry(mcmc_b200_ctx* ctx, int* slices, int* ctas_per_sm, int* tile_rows);

/*
 * Self-test of the device-side time-out route.  Every wait inside the kernels
 * is bounded (the reference's grid barrier spins without a limit,
 * mcmc_step_tc.h:597-612): a wait that runs out records a code in the
 * context's status word, the kernel finishes by itself, and the next
 * synchronising call returns MCMC_B200_ERR_TIMEOUT.  This call launches one
 * small kernel that waits, with the kernels' own wait routine and a limit of
 * limit_us microseconds (20 .. 1000000), on a barrier that nothing arms, and
 * returns what the context then reports: MCMC_B200_ERR_TIMEOUT when the route
 * works.  The status word is cleared on the way out: the context stays usable.
 */
int mcmc_b200_selftest_wait_timeout(mcmc_b200_ctx* ctx, int limit_us);

#ifdef __cplusplus
}
#endif
#endif /* MCMC_B200_H_ */

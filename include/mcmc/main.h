// Source-compatible mirror of the reference's sampler/model interface
// (include/mcmc/main.h, mcmc_step_ffma.h / mcmc_step_tc.h, kernel_helpers.h
// there), as thin inline wrappers over the C-ABI in mcmc_b200.h: a translation
// unit written against the reference (`#include "mcmc/main.h"`, then
// mcmc::main_loop<float>(), mcmc::mcmc_step<float, L>(...), mcmc::Network<float>,
// DeviceMatrix<float>, log_acpt_prec<...>) builds against this library.
//
// What a caller can observe differently from the reference:
//   * errors throw std::runtime_error instead of aborting the process;
//   * precision follows -DUSE_TC exactly as there (main.h:38-42): defined = the
//     TF32 tensor-core kernels, undefined = the FP32 kernels;
//   * after mcmc_step the caller's objects carry the names the reference's FFMA
//     variant leaves them with (L-1 rotations, mcmc_step_ffma.h:382-393) in both
//     precisions, so the TC-only replay of main.h:224-227 must not be done;
//     grad_prev's contents after the call are unspecified;
//   * mcmc_step recognises the dataset by the two pointers x.ptr() / y.ptr() and keeps a repacked
//     copy: a caller that refills the SAME DeviceMatrix objects with another window must call
//     mcmc::rebind_data() before the next mcmc_step (the reference re-reads x and y every launch);
//   * main_loop reads DATA_FNAME in the reference's text layout when that file
//     is present (mcmc_b200_read_table) and otherwise generates a synthetic
//     window (the reference's data file is not distributed); either way the
//     whole chain runs on the device.
#pragma once
#include <chrono>
#include <cstdio>
#include <stdexcept>
#include <string>
#include <vector>

#include "../mcmc_b200.h"
#include "global_params.h"
#include "utils_matrix.h"

namespace mcmc {

static constexpr int N_P_ALIGNED = (NUM_PARAMS + 3) / 4 * 4;

inline void check(int status, const char* what) {
  if (status != MCMC_B200_OK) throw std::runtime_error(std::string(what) + ": " + mcmc_b200_last_error());
}

// The library's reference preset with every constant of global_params.h applied on top (they are
// equal unless the header was configured on the command line).
inline mcmc_b200_config reference_config() {
  mcmc_b200_config cfg;
  mcmc_b200_config_reference(&cfg);
  cfg.D = FEAT_DIM[0];
  cfg.H = FEAT_DIM[1];
  cfg.lik_scale = STUDENT_T_SCALE;
  cfg.lik_df = STUDENT_T_DF;
  cfg.prior_scale = PRIOR_SCALE;
  cfg.leapfrog_steps = LEAPFROG_STEPS;
  cfg.burn_in = BURN_IN_STEPS;
  cfg.adapt_steps = STEP_SIZE_ADAPT_STEPS;
  cfg.sample_capacity = SAMPLE_STEPS;
  cfg.eps0 = STEP_SIZE_INIT;
  cfg.target_rate = STEP_SIZE_TARGET_RATE;
  cfg.decrement = STEP_SIZE_DECREMENT;
  cfg.increment = STEP_SIZE_INCREMENT;
#ifdef USE_TC
  cfg.precision = MCMC_B200_PREC_TF32;
#endif
  return cfg;
}

// One context per process for the explicit-buffer calls, as the reference keeps
// one set of kernels/attributes per process.
inline mcmc_b200_ctx* step_context() {
  static mcmc_b200_ctx* ctx = nullptr;
  if (!ctx) {
    mcmc_b200_config cfg = reference_config();
    cfg.sample_capacity = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    check(mcmc_b200_create(&cfg, dev, 1, N_SAMPLES, &ctx), "mcmc_b200_create");
  }
  return ctx;
}

template <typename T>
void set_dynamic_smem_max_size() {}  // the library sets its kernels' attributes itself

// Network<T> (main.h:48-76): seven views into one zeroed block.
template <typename T>
struct Network {
  explicit Network(const cudaStream_t& init_stream)
      : block(7, N_P_ALIGNED, T(0), init_stream),
        w_prev(1, N_P_ALIGNED, block.ptr()),
        w_next(1, N_P_ALIGNED, block.ptr() + N_P_ALIGNED * 3),
        mom_prev(1, N_P_ALIGNED, block.ptr() + N_P_ALIGNED * 1),
        mom_next(1, N_P_ALIGNED, block.ptr() + N_P_ALIGNED * 6),
        grad_prev(1, N_P_ALIGNED, block.ptr() + N_P_ALIGNED * 2),
        grad_cur(1, N_P_ALIGNED, block.ptr() + N_P_ALIGNED * 4),
        grad_next(1, N_P_ALIGNED, block.ptr() + N_P_ALIGNED * 5) {}
  DeviceMatrix<T> block;
  DeviceMatrix<T> w_prev, w_next, mom_prev, mom_next, grad_prev, grad_cur, grad_next;
  void do_swap_g() {
    grad_cur.swap(grad_next);
    grad_prev.swap(grad_next);
  }
  void do_swap() {
    w_prev.swap(w_next);
    mom_prev.swap(mom_next);
    do_swap_g();
  }
};

// mcmc::mcmc_step<T, LP_STEPS> (mcmc_step_ffma.h:395-402 / mcmc_step_tc.h:679-686)
template <typename T, int LP_STEPS = 1>
void mcmc_step(const DeviceMatrix<T>& x, const DeviceMatrix<T>& y, DeviceMatrix<T>& weights_prev,
               DeviceMatrix<T>& weights_next, DeviceMatrix<T>& mom_prev, DeviceMatrix<T>& mom_next,
               DeviceMatrix<T>& grad_prev, DeviceMatrix<T>& grad_cur, DeviceMatrix<T>& grad_next,
               DeviceMatrix<T>& loss_values, DeviceMatrix<int>* /*grid_sync_workspace*/, T eps,
               const cudaStream_t& stream) {
  static_assert(sizeof(T) == 4, "FP32 storage only");
  static_assert(LP_STEPS > 0, "LP_STEPS must be > 0");
  const T* w_in = weights_prev.ptr();
  const T* m_in = mom_prev.ptr();
  const T* g_in = grad_prev.ptr();
  // leave the caller's names where the reference's L-1 rotations leave them ...
  for (int i = 0; i < LP_STEPS - 1; ++i) {
    weights_prev.swap(weights_next);
    mom_prev.swap(mom_next);
    grad_cur.swap(grad_next);
    grad_prev.swap(grad_next);
  }
  // ... and put the results into the buffers those names now denote
  check(mcmc_b200_mcmc_step(step_context(), x.ptr(), y.ptr(), w_in, weights_next.ptr(), m_in, mom_next.ptr(),
                            g_in, grad_cur.ptr(), grad_next.ptr(), loss_values.ptr(), LP_STEPS, (float)eps,
                            (void*)stream),
        "mcmc_step");
}

// The next mcmc_step repacks x / y even when they are the same buffers as before (see the list above).
inline void rebind_data() { check(mcmc_b200_rebind_data(step_context()), "rebind_data"); }

}  // namespace mcmc

// log_acpt_prec<T, N_LOSS, N_MOM> (kernel_helpers.h:153-158); the scratch arguments are accepted and unused
template <typename T, int N_LOSS, int N_MOM, int TPB = 128>
T log_acpt_prec(T* /*log_acpt_out*/, const T* prev_loss_values, const T* new_loss_values, T* prev_mom_values,
                const T* new_mom_values, const T* grad_cur_ptr, T* /*loss_tmp*/, T*& /*tmp_storage*/,
                size_t& /*tmp_bytes*/, const T eps, const cudaStream_t& stream) {
  static_assert(N_MOM == NUM_PARAMS, "momentum length must be the model's parameter count");
  float out = 0.f;
  mcmc::check(mcmc_b200_log_acpt(mcmc::step_context(), prev_loss_values, new_loss_values,
                                 (int64_t)N_LOSS + N_MOM, prev_mom_values, new_mom_values, grad_cur_ptr,
                                 (float)eps, (void*)stream, &out),
              "log_acpt_prec");
  return (T)out;
}

namespace mcmc {

// main_loop<T> (main.h:117-308): the reference preset end to end on one window.
template <typename T>
void main_loop() {
  mcmc_b200_config cfg = reference_config();
  cfg.seed = SEED_INIT;
  int dev = 0;
  cudaGetDevice(&dev);
  mcmc_b200_ctx* ctx = nullptr;
  check(mcmc_b200_create(&cfg, dev, 1, N_SAMPLES, &ctx), "mcmc_b200_create");
  std::vector<float> x((size_t)N_SAMPLES * N_COLS), y(N_SAMPLES);
  // main.h:158-164: read the dataset, scale the features by 0.001
  if (FILE* probe = std::fopen(DATA_FNAME, "r")) {
    std::fclose(probe);
    std::printf("Reading dataset...\n");
    check(mcmc_b200_read_table(DATA_FNAME, N_SAMPLES, TOTAL_COLS, SKIP_COLS, N_COLS, 0.001f, x.data(), y.data()),
          "mcmc_b200_read_table");
    std::printf("Dataset read successfully\n");
  } else {
    std::printf("'%s' not found: using a synthetic window of the same shape\n", DATA_FNAME);
    check(mcmc_b200_synth_window(SEED_INIT, 0, N_SAMPLES, N_COLS, FEAT_DIM[1], x.data(), y.data(), nullptr),
          "mcmc_b200_synth_window");
    for (auto& v : x) v *= 0.001f;
  }
  check(mcmc_b200_set_window_data(ctx, 0, 0, x.data(), y.data(), 0), "mcmc_b200_set_window_data");
  const auto t0 = std::chrono::high_resolution_clock::now();
  check(mcmc_b200_run_chain(ctx, BURN_IN_STEPS + SAMPLE_STEPS), "mcmc_b200_run_chain");
  const auto t1 = std::chrono::high_resolution_clock::now();
  double ll = 0, lp = 0;
  check(mcmc_b200_final_loss(ctx, 0, 0, SAMPLE_STEPS, &ll, &lp), "mcmc_b200_final_loss");
  int32_t it = 0, acc = 0;
  float eps = 0;
  check(mcmc_b200_chain_info(ctx, 0, &it, &acc, &eps), "mcmc_b200_chain_info");
  const long long t_ms = std::chrono::duration_cast<std::chrono::milliseconds>(t1 - t0).count();
  std::printf("Final loss1: %g, loss2: %g, full loss: %g\n", ll, lp, ll + lp);
  std::printf("accepted %d of %d, final step size %g\n", acc, it, eps);
  std::printf("MCMC (%d burn in, %d sample steps, %d leap-frog steps) done in %lldms. "
              "Expected time for 200 sequential passes: %.3fh. Good bye!\n",
              BURN_IN_STEPS, SAMPLE_STEPS, LEAPFROG_STEPS, t_ms, 200 * (double(t_ms) / 3600000));
  mcmc_b200_destroy(ctx);
}

}  // namespace mcmc

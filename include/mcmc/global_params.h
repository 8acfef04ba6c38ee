// The reference's compile-time constants (include/mcmc/global_params.h:27-65
// there), kept under the same names so that code written against them builds.
// In this library they are only DEFAULTS: mcmc_b200_config carries every one of
// them at run time (mcmc_b200_config_reference fills in exactly these values).
#pragma once
#include <cstddef>

// The reference can only be reconfigured by editing its header (main.cu:28-31 ignores argv).  Here the
// chain lengths and the row count may also be given on the compiler command line
// (-DMCMC_LEAPFROG_STEPS=10 ...), which is how the short end-to-end test of main_loop is built.
#ifndef MCMC_BURN_IN_STEPS
#define MCMC_BURN_IN_STEPS 100
#endif
#ifndef MCMC_SAMPLE_STEPS
#define MCMC_SAMPLE_STEPS 800
#endif
#ifndef MCMC_LEAPFROG_STEPS
#define MCMC_LEAPFROG_STEPS 1000
#endif
#ifndef MCMC_N_SAMPLES
#define MCMC_N_SAMPLES 58368
#endif

// chain length and integrator (global_params.h:27-36)
static constexpr size_t SEED_INIT = 0;
static constexpr int BURN_IN_STEPS = MCMC_BURN_IN_STEPS, SAMPLE_STEPS = MCMC_SAMPLE_STEPS,
                     LEAPFROG_STEPS = MCMC_LEAPFROG_STEPS, OUTPUT_EVERY = 10;
static constexpr int STEP_SIZE_ADAPT_STEPS = BURN_IN_STEPS;
static constexpr double STEP_SIZE_INIT = 0.01, STEP_SIZE_TARGET_RATE = 0.2;
static constexpr double STEP_SIZE_DECREMENT = 0.1, STEP_SIZE_INCREMENT = 0.01;

// Student-t likelihood and Gaussian prior (global_params.h:39-52)
static constexpr double STUDENT_T_SCALE = 100.0, STUDENT_T_DF = 2.2, PRIOR_SCALE = 200.0;

// model 22 -> 40 -> 1 with the last two layers fused (global_params.h:55-58)
static constexpr int NUM_LAYERS = 2;
static constexpr int FEAT_DIM[] = {22, 40, 1};
static constexpr int NUM_PARAMS = FEAT_DIM[0] * FEAT_DIM[1] + 2 * FEAT_DIM[1] * FEAT_DIM[2] + FEAT_DIM[2];

// dataset file layout (global_params.h:61-65): 149 columns, 2 skipped, 1 label, 22 features
static constexpr int N_SAMPLES = MCMC_N_SAMPLES, N_COLS = FEAT_DIM[0], TOTAL_COLS = 149, SKIP_COLS = 2;
static constexpr const char* DATA_FNAME = "returns_and_features_for_mcmc.txt";

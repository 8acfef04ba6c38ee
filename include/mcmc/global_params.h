// The reference's compile-time constants (include/mcmc/global_params.h:27-65
// there), kept under the same names so that code written against them builds.
// In this library they are only DEFAULTS: mcmc_b200_config carries every one of
// them at run time.
#pragma once
#include <cstddef>

static constexpr size_t SEED_INIT = 0;
static constexpr int BURN_IN_STEPS = 100;
static constexpr int SAMPLE_STEPS = 800;
static constexpr int LEAPFROG_STEPS = 1000;
static constexpr int OUTPUT_EVERY = 10;
static constexpr double STEP_SIZE_INIT = 0.01;
static constexpr double STEP_SIZE_TARGET_RATE = 0.2;
static constexpr double STEP_SIZE_DECREMENT = 0.1;
static constexpr double STEP_SIZE_INCREMENT = 0.01;
static constexpr int STEP_SIZE_ADAPT_STEPS = BURN_IN_STEPS;
static constexpr double STUDENT_T_SCALE = 100.0;
static constexpr double STUDENT_T_DF = 2.2;
static constexpr double PRIOR_SCALE = 200.0;
static constexpr int NUM_LAYERS = 2;
static constexpr int FEAT_DIM[] = {22, 40, 1};
static constexpr int NUM_PARAMS = FEAT_DIM[0] * FEAT_DIM[1] + FEAT_DIM[1] + FEAT_DIM[1] * FEAT_DIM[2] + FEAT_DIM[2];
static constexpr int N_SAMPLES = 58368;
static constexpr int N_COLS = FEAT_DIM[0];
static constexpr int TOTAL_COLS = 149;
static constexpr int SKIP_COLS = 2;
static constexpr const char* DATA_FNAME = "returns_and_features_for_mcmc.txt";

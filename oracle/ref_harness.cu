// Harness around the reference's own, unmodified FP32 kernels.
//
// TEST INFRASTRUCTURE ONLY (like everything under oracle/).  It includes the
// reference's headers from the reference tree (-I<reference>/include, see the
// Makefile) and exposes three C entry points so that a Python test can run the
// reference's leapfrog_step_kernel / log_acpt_prec on a B200 and pin the CPU
// oracle against them.  Nothing of the reference is copied here.
//
// Only the FFMA variant is built: the reference's TF32 variant reads rows past
// the end of the dataset for N = 58368 (mcmc_step_tc.h:175-209) and waits in an
// unbounded spin (mcmc_step_tc.h:604-605), so it is never run.
//
// The reference fixes every shape at compile time (global_params.h): 58368
// rows, 22 features, 40 hidden units, Student-t(100, 2.2) likelihood,
// N(0, 200^2) prior.  The harness therefore works at exactly those.
#include <cuda_runtime.h>
#include <vector>

#include "mcmc/global_params.h"
#include "mcmc/kernel_helpers.h"
#include "mcmc/mcmc_step_ffma.h"
#include "mcmc/utils_cuda.h"
#include "mcmc/utils_matrix.h"

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {
template <typename T>
void h2d(DeviceMatrix<T>& m, const T* src, size_t n) {
  cudaMemcpy(m.ptr(), src, n * sizeof(T), cudaMemcpyHostToDevice);
}
template <typename T>
void d2h(T* dst, const DeviceMatrix<T>& m, size_t n) {
  cudaMemcpy(dst, m.ptr(), n * sizeof(T), cudaMemcpyDeviceToHost);
}
bool g_init = false;
void init_once() {
  if (!g_init) {
    mcmc::set_dynamic_smem_max_size<float>();
    g_init = true;
  }
}
}  // namespace

REF_API int ref_n_samples() { return N_SAMPLES; }
REF_API int ref_n_params() { return NUM_PARAMS; }

// mcmc_step<float, L> for L in {1, 2, 10} on host arrays.
//   x [N_SAMPLES*22], y [N_SAMPLES], state vectors [NUM_PARAMS],
//   loss_values [N_SAMPLES + NUM_PARAMS].
REF_API int ref_ffma_mcmc_step(const float* x, const float* y, int L, float eps, const float* w_prev,
                               const float* mom_prev, const float* grad_prev, float* w_next,
                               float* mom_next, float* grad_cur, float* loss_values) {
  using namespace mcmc;
  init_once();
  cudaStream_t stream = cudaStreamPerThread;
  DeviceMatrix<float> data(N_SAMPLES, N_COLS), labels(N_SAMPLES, 1);
  h2d(data, x, (size_t)N_SAMPLES * N_COLS);
  h2d(labels, y, (size_t)N_SAMPLES);
  const int NP = N_P_ALIGNED;
  DeviceMatrix<float> block(7, NP, 0.f, stream);
  DeviceMatrix<float> wp(1, NP, block.ptr()), mp(1, NP, block.ptr() + NP), gp(1, NP, block.ptr() + 2 * NP),
      wn(1, NP, block.ptr() + 3 * NP), gc(1, NP, block.ptr() + 4 * NP), gn(1, NP, block.ptr() + 5 * NP),
      mn(1, NP, block.ptr() + 6 * NP);
  DeviceMatrix<float> loss(1, N_SAMPLES + NUM_PARAMS, 0.f, stream);
  cudaStreamSynchronize(stream);
  h2d(wp, w_prev, NUM_PARAMS);
  h2d(mp, mom_prev, NUM_PARAMS);
  h2d(gp, grad_prev, NUM_PARAMS);
  if (L == 1) mcmc_step<float, 1>(data, labels, wp, wn, mp, mn, gp, gc, gn, loss, nullptr, eps, stream);
  else if (L == 2) mcmc_step<float, 2>(data, labels, wp, wn, mp, mn, gp, gc, gn, loss, nullptr, eps, stream);
  else if (L == 10) mcmc_step<float, 10>(data, labels, wp, wn, mp, mn, gp, gc, gn, loss, nullptr, eps, stream);
  else return 1;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return 2;
  d2h(w_next, wn, NUM_PARAMS);
  d2h(mom_next, mn, NUM_PARAMS);
  d2h(grad_cur, gc, NUM_PARAMS);
  d2h(loss_values, loss, (size_t)N_SAMPLES + NUM_PARAMS);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// log_acpt_prec<float, N_SAMPLES, NUM_PARAMS> on host arrays.
REF_API int ref_log_acpt(const float* prev_loss, const float* new_loss, const float* prev_mom,
                         const float* new_mom, const float* grad_cur, float eps, float* out) {
  init_once();
  cudaStream_t stream = cudaStreamPerThread;
  const size_t NL = (size_t)N_SAMPLES + NUM_PARAMS;
  DeviceMatrix<float> pl(1, NL), nl(1, NL), pm(1, NUM_PARAMS), nm(1, NUM_PARAMS), gc(1, NUM_PARAMS),
      tmp(1, N_SAMPLES + 2 * NUM_PARAMS), res(1, 4);
  h2d(pl, prev_loss, NL);
  h2d(nl, new_loss, NL);
  h2d(pm, prev_mom, NUM_PARAMS);
  h2d(nm, new_mom, NUM_PARAMS);
  h2d(gc, grad_cur, NUM_PARAMS);
  float* tmp_storage = nullptr;
  size_t tmp_bytes = 0;
  *out = log_acpt_prec<float, N_SAMPLES, NUM_PARAMS>(res.ptr(), pl.ptr(), nl.ptr(), pm.ptr(), nm.ptr(),
                                                      gc.ptr(), tmp.ptr(), tmp_storage, tmp_bytes, eps,
                                                      stream);
  if (tmp_storage) cudaFree(tmp_storage);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// Device time of the reference's FFMA path: `reps` calls of mcmc_step<float, 10> (ten launches of
// leapfrog_step_kernel each) on resident buffers, timed with CUDA events; returns the mean time of one
// leapfrog step (= one full-batch gradient) in microseconds through *us_per_step.
REF_API int ref_ffma_time_steps(const float* x, const float* y, float eps, int warmup, int reps,
                                float* us_per_step) {
  using namespace mcmc;
  init_once();
  cudaStream_t stream = cudaStreamPerThread;
  DeviceMatrix<float> data(N_SAMPLES, N_COLS), labels(N_SAMPLES, 1);
  h2d(data, x, (size_t)N_SAMPLES * N_COLS);
  h2d(labels, y, (size_t)N_SAMPLES);
  const int NP = N_P_ALIGNED;
  DeviceMatrix<float> block(7, NP, 0.f, stream);
  DeviceMatrix<float> wp(1, NP, block.ptr()), mp(1, NP, block.ptr() + NP), gp(1, NP, block.ptr() + 2 * NP),
      wn(1, NP, block.ptr() + 3 * NP), gc(1, NP, block.ptr() + 4 * NP), gn(1, NP, block.ptr() + 5 * NP),
      mn(1, NP, block.ptr() + 6 * NP);
  DeviceMatrix<float> loss(1, N_SAMPLES + NUM_PARAMS, 0.f, stream);
  cudaStreamSynchronize(stream);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  for (int r = 0; r < warmup + reps; ++r) {
    if (r == warmup) cudaEventRecord(e0, stream);
    cudaMemsetAsync(gc.ptr(), 0, NP * sizeof(float), stream);  // the step expects a zeroed grad_cur
    mcmc_step<float, 10>(data, labels, wp, wn, mp, mn, gp, gc, gn, loss, nullptr, eps, stream);
  }
  cudaEventRecord(e1, stream);
  if (cudaStreamSynchronize(stream) != cudaSuccess) return 2;
  float ms = 0.f;
  cudaEventElapsedTime(&ms, e0, e1);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  *us_per_step = ms * 1000.f / (10.f * reps);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// Two device micro-benchmarks that give the gradient kernels' rooflines their other denominators:
//   * L2 read bandwidth: one window of the benchmark workload is 5.4 MB and stays resident in the
//     126 MB L2 from one leapfrog step to the next, so for one-window launches the memory roofline is
//     the L2's, not HBM's;
//   * MUFU rate: the TF32 path evaluates one tanh per hidden unit and row on the MUFU pipe
//     (tanh.approx.f32; the reference's formula is ex2 + rcp, kernel_helpers.h:32-44, two MUFU
//     operations), which bounds rows/s independently of memory.
// Timed with CUDA events on the launching stream after warm-up launches.  Nothing on the sampling path
// calls these.
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/mcmc_b200.h"

void mcmc_b200_set_last_error(const std::string& msg);

namespace {

__global__ void __launch_bounds__(512) l2_read_kernel(const float4* __restrict__ buf, size_t n_vec, int passes,
                                                      float* sink) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (int p = 0; p < passes; ++p) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += stride) {
      float4 v;
      // ld.global.cg: cached in L2 only, so every pass goes back to the L2
      asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                   : "l"(buf + i));
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
  }
  if (acc.x + acc.y + acc.z + acc.w == 123.456f) *sink = acc.x;  // keeps the loads alive
}

// kind 0: tanh.approx.f32   1: ex2.approx + rcp.approx (the reference's tanh: two operations per value)
template <int KIND>
__global__ void __launch_bounds__(512) mufu_kernel(int iters, float seed, float* sink) {
  float v[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) v[k] = seed + 0.01f * (float)(threadIdx.x + k);
  for (int i = 0; i < iters; ++i) {
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (KIND == 0) {
        asm volatile("tanh.approx.f32 %0, %0;" : "+f"(v[k]));
      } else {
        asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(v[k]));
        asm volatile("rcp.approx.f32 %0, %0;" : "+f"(v[k]));
      }
    }
  }
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) s += v[k];
  if (s == 123.456f) *sink = s;
}

int fail_mb(const char* what, cudaError_t e) {
  mcmc_b200_set_last_error(std::string(what) + ": " + cudaGetErrorString(e));
  return MCMC_B200_ERR_CUDA;
}

}  // namespace

#define MB_CK(call)                                  \
  do {                                               \
    cudaError_t e_ = (call);                         \
    if (e_ != cudaSuccess) return fail_mb(#call, e_); \
  } while (0)

extern "C" __attribute__((visibility("default"))) int mcmc_b200_microbench_l2_read(int device, int64_t bytes,
                                                                                    double* gb_per_s) {
  if (!gb_per_s || bytes < (1 << 20) || bytes > (1LL << 32)) {
    mcmc_b200_set_last_error("bad arguments (1 MB .. 4 GB)");
    return MCMC_B200_ERR_INVALID;
  }
  MB_CK(cudaSetDevice(device));
  int sms = 0;
  MB_CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  float4* buf = nullptr;
  float* sink = nullptr;
  MB_CK(cudaMalloc(&buf, (size_t)bytes));
  MB_CK(cudaMalloc(&sink, 4));
  MB_CK(cudaMemset(buf, 0, (size_t)bytes));
  const size_t n_vec = (size_t)bytes / 16;
  // enough passes for about a gigabyte per launch
  const int passes = (int)((1LL << 30) / bytes) + 1;
  cudaEvent_t e0, e1;
  MB_CK(cudaEventCreate(&e0));
  MB_CK(cudaEventCreate(&e1));
  for (int w = 0; w < 3; ++w) l2_read_kernel<<<sms * 4, 512>>>(buf, n_vec, passes, sink);
  MB_CK(cudaEventRecord(e0));
  const int launches = 5;
  for (int r = 0; r < launches; ++r) l2_read_kernel<<<sms * 4, 512>>>(buf, n_vec, passes, sink);
  MB_CK(cudaEventRecord(e1));
  MB_CK(cudaEventSynchronize(e1));
  float ms = 0.f;
  MB_CK(cudaEventElapsedTime(&ms, e0, e1));
  *gb_per_s = (double)launches * passes * (double)bytes / (ms * 1e-3) / 1e9;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(buf);
  cudaFree(sink);
  return MCMC_B200_OK;
}

extern "C" __attribute__((visibility("default"))) int mcmc_b200_microbench_mufu(int device, int kind,
                                                                                 double* gops_per_s) {
  if (!gops_per_s || (kind != 0 && kind != 1)) {
    mcmc_b200_set_last_error("bad arguments");
    return MCMC_B200_ERR_INVALID;
  }
  MB_CK(cudaSetDevice(device));
  int sms = 0;
  MB_CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  float* sink = nullptr;
  MB_CK(cudaMalloc(&sink, 4));
  const int iters = 4096, blocks = sms * 4, threads = 512;
  cudaEvent_t e0, e1;
  MB_CK(cudaEventCreate(&e0));
  MB_CK(cudaEventCreate(&e1));
  auto launch = [&]() {
    if (kind == 0) mufu_kernel<0><<<blocks, threads>>>(iters, 0.3f, sink);
    else mufu_kernel<1><<<blocks, threads>>>(iters, 0.3f, sink);
  };
  for (int w = 0; w < 3; ++w) launch();
  MB_CK(cudaEventRecord(e0));
  const int launches = 5;
  for (int r = 0; r < launches; ++r) launch();
  MB_CK(cudaEventRecord(e1));
  MB_CK(cudaEventSynchronize(e1));
  float ms = 0.f;
  MB_CK(cudaEventElapsedTime(&ms, e0, e1));
  // values per second: one tanh.approx, or one ex2 + rcp pair, per value
  *gops_per_s = (double)launches * blocks * threads * (double)iters * 8.0 / (ms * 1e-3) / 1e9;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(sink);
  return MCMC_B200_OK;
}

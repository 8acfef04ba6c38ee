// Forward-only pass over (stored samples x rows): posterior-mean prediction and the mean losses over the
// stored samples.  The reference evaluates its stored samples one at a time through the full
// forward+backward kernel with eps = 0 (output_final_loss, include/mcmc/main.h:78-115, followed by two CUB
// reductions per sample, kernel_helpers.h:190-216); here one launch covers all samples and all rows and
// computes no gradient.
//
//   * FP32 FFMA with the reference's tanh (kernel_helpers.h:32-44): the result is the FP32 forward pass
//     whatever precision the chain was sampled in;
//   * a CTA owns 512 rows (4 per thread, held in registers for the whole launch) and walks through its
//     chunk of the samples; a sample's 961 parameters are staged in shared memory once per CTA and read as
//     16-byte broadcasts: 16 FMAs per load;
//   * PREDICT: per-row sums over the chunk's samples -> partial[chunk][row]; LOSS: per-sample sums over the
//     CTA's rows -> partial[tile][sample].  A second small launch adds the partials in a fixed order (and, for
//     LOSS, the log-prior of every sample).  Doubles, no atomics: bit-reproducible.
#include "chain.cuh"
#include "common.cuh"

namespace mcmc_b200 {

constexpr int FWD_THREADS = 128, FWD_RPT = 4, FWD_ROWS = FWD_THREADS * FWD_RPT;

template <int H, bool LOSS>
__global__ void __launch_bounds__(FWD_THREADS) forward_samples_kernel(const ForwardParams a) {
  constexpr int D = 22, P = D * H + 2 * H + 1;
  extern __shared__ __align__(16) float sw[];  // one sample: W0[k][j], b0, W1, b1
  __shared__ double red[FWD_THREADS / 32];
  const int tid = threadIdx.x;
  const long long row0 = (long long)blockIdx.x * FWD_ROWS;
  const int s0 = (int)((long long)blockIdx.y * a.count / gridDim.y);
  const int s1 = (int)((long long)(blockIdx.y + 1) * a.count / gridDim.y);
  // rows tid, tid + 128, ...: consecutive threads read consecutive rows
  float x[FWD_RPT][D], y[FWD_RPT];
  bool valid[FWD_RPT];
#pragma unroll
  for (int r = 0; r < FWD_RPT; ++r) {
    const long long row = row0 + r * FWD_THREADS + tid;
    valid[r] = row < a.n;
#pragma unroll
    for (int k = 0; k < D; ++k) x[r][k] = valid[r] ? a.x[row * a.x_stride + k] : 0.f;
    y[r] = (LOSS && valid[r]) ? a.y[row * a.y_stride] : 0.f;
  }
  double acc[FWD_RPT];
#pragma unroll
  for (int r = 0; r < FWD_RPT; ++r) acc[r] = 0.0;

  for (int s = s0; s < s1; ++s) {
    __syncthreads();
    for (int p = tid; p < P; p += FWD_THREADS) sw[p] = a.samples[(size_t)s * P + p];
    __syncthreads();
    float pred[FWD_RPT];
#pragma unroll
    for (int r = 0; r < FWD_RPT; ++r) pred[r] = sw[D * H + 2 * H];
#pragma unroll 1
    for (int j0 = 0; j0 < H; j0 += 4) {
      float z[FWD_RPT][4];
      const float4 b = *reinterpret_cast<const float4*>(sw + D * H + j0);
#pragma unroll
      for (int r = 0; r < FWD_RPT; ++r) { z[r][0] = b.x; z[r][1] = b.y; z[r][2] = b.z; z[r][3] = b.w; }
#pragma unroll
      for (int k = 0; k < D; ++k) {
        const float4 w = *reinterpret_cast<const float4*>(sw + k * H + j0);
#pragma unroll
        for (int r = 0; r < FWD_RPT; ++r) {
          z[r][0] = fmaf(x[r][k], w.x, z[r][0]);
          z[r][1] = fmaf(x[r][k], w.y, z[r][1]);
          z[r][2] = fmaf(x[r][k], w.z, z[r][2]);
          z[r][3] = fmaf(x[r][k], w.w, z[r][3]);
        }
      }
      const float4 w1 = *reinterpret_cast<const float4*>(sw + D * H + H + j0);
#pragma unroll
      for (int r = 0; r < FWD_RPT; ++r) {
        pred[r] = fmaf(w1.x, tanh_ref(z[r][0]), pred[r]);
        pred[r] = fmaf(w1.y, tanh_ref(z[r][1]), pred[r]);
        pred[r] = fmaf(w1.z, tanh_ref(z[r][2]), pred[r]);
        pred[r] = fmaf(w1.w, tanh_ref(z[r][3]), pred[r]);
      }
    }
    if (LOSS) {
      double l = 0.0;
#pragma unroll
      for (int r = 0; r < FWD_RPT; ++r) {
        float loss, dy;
        lik_terms(a.lik, y[r], pred[r], loss, dy);
        if (valid[r]) l += (double)loss;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
      if ((tid & 31) == 0) red[tid >> 5] = l;
      __syncthreads();
      if (tid == 0) {
        double t = red[0];
#pragma unroll
        for (int w = 1; w < FWD_THREADS / 32; ++w) t += red[w];
        a.partial[(size_t)blockIdx.x * a.count + s] = t;
      }
    } else {
#pragma unroll
      for (int r = 0; r < FWD_RPT; ++r) acc[r] += (double)pred[r];
    }
  }
  if (!LOSS) {
#pragma unroll
    for (int r = 0; r < FWD_RPT; ++r) {
      const long long row = row0 + r * FWD_THREADS + tid;
      if (valid[r]) a.partial[(size_t)blockIdx.y * a.n + row] = acc[r];
    }
  }
}

// PREDICT: out[row] = sum over chunks / count.  LOSS: per sample the sum over row tiles -> out_ll[s], the
// log-prior of the sample -> out_lp[s] (one CTA per sample).
__global__ void forward_finish_predict(const double* partial, int chunks, long long n, int count, float* out) {
  const long long row = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (row >= n) return;
  double t = 0.0;
  for (int c = 0; c < chunks; ++c) t += partial[(size_t)c * n + row];
  out[row] = (float)(t / (double)count);
}
__global__ void __launch_bounds__(128) forward_finish_loss(const double* partial, int tiles, int count,
                                                           const float* samples, int P, PriorParams prior,
                                                           double* out_ll, double* out_lp) {
  __shared__ double dsc[32];
  const int s = blockIdx.x;
  double t = 0.0;
  for (int k = threadIdx.x; k < tiles; k += blockDim.x) t += partial[(size_t)k * count + s];
  const double ll = block_sum_f64(t, dsc);
  double lp = 0.0;
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const float w = samples[(size_t)s * P + p];
    const float q = w * prior.inv_s;
    lp += (double)fmaf(-0.5f * q, q, -prior.norm);
  }
  lp = block_sum_f64(lp, dsc);
  if (threadIdx.x == 0) {
    out_ll[s] = ll;
    out_lp[s] = lp;
  }
}

int forward_row_tiles(long long n) { return (int)((n + FWD_ROWS - 1) / FWD_ROWS); }

template <int H>
static cudaError_t launch_forward_t(const ForwardParams& a, int chunks, bool loss, cudaStream_t st) {
  constexpr int P = 22 * H + 2 * H + 1;
  const size_t smem = sizeof(float) * ((P + 3) / 4 * 4);
  const dim3 grid(forward_row_tiles(a.n), chunks);
  if (loss) forward_samples_kernel<H, true><<<grid, FWD_THREADS, smem, st>>>(a);
  else forward_samples_kernel<H, false><<<grid, FWD_THREADS, smem, st>>>(a);
  return cudaGetLastError();
}

cudaError_t launch_forward_samples(int H, const ForwardParams& a, int chunks, bool loss, cudaStream_t st) {
  if (H == 40) return launch_forward_t<40>(a, chunks, loss, st);
  if (H == 128) return launch_forward_t<128>(a, chunks, loss, st);
  return cudaErrorInvalidValue;
}
cudaError_t launch_forward_finish_predict(const double* partial, int chunks, long long n, int count, float* out,
                                          cudaStream_t st) {
  forward_finish_predict<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(partial, chunks, n, count, out);
  return cudaGetLastError();
}
cudaError_t launch_forward_finish_loss(const double* partial, int tiles, int count, const float* samples, int P,
                                       const PriorParams& prior, double* out_ll, double* out_lp, cudaStream_t st) {
  forward_finish_loss<<<count, 128, 0, st>>>(partial, tiles, count, samples, P, prior, out_ll, out_lp);
  return cudaGetLastError();
}

}  // namespace mcmc_b200

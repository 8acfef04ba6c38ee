// FP32 (FFMA) fused leapfrog-update + forward + backward kernel.
//
// Stands in for leapfrog_step_kernel of the reference
// (include/mcmc/mcmc_step_ffma.h:154-379): same math, different mapping.
//   * grid = (slices, windows): many independent windows per launch, each
//     window's rows split over `slices` CTAs;
//   * rows arrive through the bulk-copy engine in double-buffered 64-row tiles
//     of the repacked [rows][24] dataset (contiguous, 16-byte aligned);
//   * a warp works on 16 rows at a time: lane = (hidden group of H/HS units,
//     row slot); each lane keeps R rows x H/HS pre-activations and its slice of
//     the dW0 accumulator in registers, so every lane does useful FMAs (the
//     reference maps 40 hidden units onto 64 lane slots);
//   * no atomics: lanes -> warp shuffles -> shared-memory tree -> one partial
//     vector per CTA; the next launch (or the accept kernel) sums the partials
//     of a window in a fixed order, so results are bit-reproducible.
#include "common.cuh"

namespace mcmc_b200 {

constexpr int FP32_THREADS = 128;
constexpr int FP32_WARPS = FP32_THREADS / 32;

template <int H, int HS, int R>
struct Fp32Geom {
  static constexpr int D = 22;
  static constexpr int HPL = H / HS;               // hidden units per lane
  static constexpr int HPLP = HPL <= 4 ? 4 : 8;    // padded for vector loads
  static constexpr int RS = 32 / HS;               // row slots per warp
  static constexpr int WARP_ROWS = RS * R;
  static constexpr int TILE = WARP_ROWS * FP32_WARPS;
  static constexpr int P = D * H + 2 * H + 1;
  static constexpr int PP = (P + 3) / 4 * 4;
  static constexpr int XS_FLOATS = 2 * TILE * KP;
  static constexpr int WS_FLOATS = KP * HS * HPLP;
  static constexpr int W1_FLOATS = (H + 3) / 4 * 4;
  static constexpr int RED_FLOATS = FP32_WARPS * PP;
  static constexpr size_t SMEM = sizeof(float) * (XS_FLOATS + WS_FLOATS + W1_FLOATS + RED_FLOATS);
  static_assert(H % HS == 0 && 32 % HS == 0, "hidden units must split evenly over lanes");
  static_assert(HPL <= 8, "too many hidden units per lane");
};

template <int H, int HS, int R>
__global__ void __launch_bounds__(FP32_THREADS, 2) grad_fp32_kernel(const GradParams g) {
  using G = Fp32Geom<H, HS, R>;
  constexpr int D = G::D, HPL = G::HPL, HPLP = G::HPLP, RS = G::RS;
  constexpr int WARP_ROWS = G::WARP_ROWS, TILE = G::TILE, PP = G::PP;
  constexpr uint32_t TILE_BYTES = TILE * KP * sizeof(float);

  extern __shared__ __align__(128) unsigned char smem_raw[];
  float* xs = reinterpret_cast<float*>(smem_raw);
  float* ws = xs + G::XS_FLOATS;
  float* w1s = ws + G::WS_FLOATS;
  float* red = w1s + G::W1_FLOATS;
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ float b1s;
  __shared__ double dsc[FP32_WARPS];

  const int tid = threadIdx.x;
  const int win = blockIdx.y;
  const int slice = blockIdx.x;
  const int S = gridDim.x;
  const int t0 = (int)((long long)slice * g.n_tiles / S);
  const int t1 = (int)((long long)(slice + 1) * g.n_tiles / S);
  const float* xw = g.xaug + (long long)(g.data_window0 + win) * g.window_stride;

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_fence_init();
  }
  for (int i = tid; i < G::WS_FLOATS; i += FP32_THREADS) ws[i] = 0.f;
  __syncthreads();
  if (tid == 0 && t0 < t1) {
    mbar_expect_tx(&bars[0], TILE_BYTES);
    bulk_g2s(xs, xw + (size_t)t0 * TILE * KP, TILE_BYTES, &bars[0]);
  }
  // fused leapfrog update; parameters land in the layout the lanes read
  for (int p = tid; p < G::P; p += FP32_THREADS) {
    const float w = leapfrog_param(g, win, p, slice == 0);
    if (p < D * H + H) {  // W0 rows 0..21 and the bias as row 22
      const int k = p / H, h = p - k * H;
      ws[(k * HS + h / HPL) * HPLP + (h % HPL)] = w;
    } else if (p < D * H + 2 * H) {
      w1s[p - (D * H + H)] = w;
    } else {
      b1s = w;
    }
  }
  __syncthreads();

  const int lane = tid & 31, warp = tid >> 5;
  const int hs = lane % HS, rs = lane / HS;
  float w1r[HPL];
#pragma unroll
  for (int j = 0; j < HPL; ++j) w1r[j] = w1s[hs * HPL + j];
  const float b1 = b1s;

  float acc[D + 1][HPL];  // dW0 rows 0..21 and db0 (row 22, x = 1)
#pragma unroll
  for (int k = 0; k <= D; ++k)
#pragma unroll
    for (int j = 0; j < HPL; ++j) acc[k][j] = 0.f;
  float dw1[HPL];
#pragma unroll
  for (int j = 0; j < HPL; ++j) dw1[j] = 0.f;
  float db1 = 0.f;
  double llacc = 0.0;
  bool ok = true;

  for (int t = t0; t < t1 && ok; ++t) {
    const int it = t - t0;
    const int stage = it & 1;
    if (tid == 0 && t + 1 < t1) {
      mbar_expect_tx(&bars[stage ^ 1], TILE_BYTES);
      bulk_g2s(xs + (stage ^ 1) * TILE * KP, xw + (size_t)(t + 1) * TILE * KP, TILE_BYTES,
               &bars[stage ^ 1]);
    }
    ok = mbar_wait(&bars[stage], (it >> 1) & 1, g.status, 101);
    const float* xt = xs + stage * TILE * KP + (warp * WARP_ROWS + rs) * KP;

    // ---- forward: z = [x, 1] . [W0; b0] ----
    float z[R][HPL];
    float yv[R];
#pragma unroll
    for (int i = 0; i < R; ++i)
#pragma unroll
      for (int j = 0; j < HPL; ++j) z[i][j] = 0.f;
#pragma unroll
    for (int kg = 0; kg < KP / 4; ++kg) {
      float4 xv[R];
#pragma unroll
      for (int i = 0; i < R; ++i)
        xv[i] = *reinterpret_cast<const float4*>(xt + i * RS * KP + kg * 4);
      if (kg == KP / 4 - 1) {
#pragma unroll
        for (int i = 0; i < R; ++i) yv[i] = xv[i].w;
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const int k = kg * 4 + kk;
        if (k > D) continue;
        float wv[HPLP];
        const float* wp = ws + (k * HS + hs) * HPLP;
#pragma unroll
        for (int q = 0; q < HPLP; q += 4) {
          if (q < HPL) {
            if (q + 4 <= HPL || HPLP == 4) {
              const float4 v = *reinterpret_cast<const float4*>(wp + q);
              wv[q] = v.x; wv[q + 1] = v.y; wv[q + 2] = v.z; wv[q + 3] = v.w;
            } else {
#pragma unroll
              for (int e = q; e < HPL; ++e) wv[e] = wp[e];
            }
          }
        }
#pragma unroll
        for (int i = 0; i < R; ++i) {
          const float xk = kk == 0 ? xv[i].x : kk == 1 ? xv[i].y : kk == 2 ? xv[i].z : xv[i].w;
#pragma unroll
          for (int j = 0; j < HPL; ++j) z[i][j] = fmaf(xk, wv[j], z[i][j]);
        }
      }
    }
    // ---- activation, output layer, loss, dZ ----
#pragma unroll
    for (int i = 0; i < R; ++i) {
      float pred = 0.f;
#pragma unroll
      for (int j = 0; j < HPL; ++j) {
        z[i][j] = tanh_ref(z[i][j]);
        pred = fmaf(w1r[j], z[i][j], pred);
      }
#pragma unroll
      for (int o = 1; o < HS; o <<= 1) pred += __shfl_xor_sync(0xffffffffu, pred, o);
      pred += b1;
      const int grow = t * TILE + warp * WARP_ROWS + i * RS + rs;
      const bool valid = grow < g.n_rows;
      float loss, dy;
      lik_terms(g.lik, yv[i], pred, loss, dy);
      if (!valid) { loss = 0.f; dy = 0.f; }
      if (hs == 0) {
        llacc += (double)loss;
        if (g.row_loss && valid) g.row_loss[(long long)win * g.row_loss_stride + grow] = loss;
      }
      db1 += dy;
#pragma unroll
      for (int j = 0; j < HPL; ++j) {
        const float h = z[i][j];
        dw1[j] = fmaf(dy, h, dw1[j]);
        z[i][j] = fmaf(-h, h, 1.f) * (w1r[j] * dy);  // tanh_t::bwd
      }
    }
    // ---- backward: dW0 (and db0 through the constant-1 column) ----
#pragma unroll
    for (int i = 0; i < R; ++i) {
#pragma unroll
      for (int kg = 0; kg < KP / 4; ++kg) {
        const float4 xv = *reinterpret_cast<const float4*>(xt + i * RS * KP + kg * 4);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const int k = kg * 4 + kk;
          if (k > D) continue;
          const float xk = kk == 0 ? xv.x : kk == 1 ? xv.y : kk == 2 ? xv.z : xv.w;
#pragma unroll
          for (int j = 0; j < HPL; ++j) acc[k][j] = fmaf(xk, z[i][j], acc[k][j]);
        }
      }
    }
    __syncthreads();
  }

  // ---- reduce: row slots -> warps -> CTA partial ----
#pragma unroll
  for (int o = HS; o < 32; o <<= 1) {
#pragma unroll
    for (int k = 0; k <= D; ++k)
#pragma unroll
      for (int j = 0; j < HPL; ++j) acc[k][j] += __shfl_xor_sync(0xffffffffu, acc[k][j], o);
#pragma unroll
    for (int j = 0; j < HPL; ++j) dw1[j] += __shfl_xor_sync(0xffffffffu, dw1[j], o);
    db1 += __shfl_xor_sync(0xffffffffu, db1, o);
    llacc += __shfl_xor_sync(0xffffffffu, llacc, o);
  }
  if (rs == 0) {
    float* r = red + warp * PP;
#pragma unroll
    for (int j = 0; j < HPL; ++j) {
      const int h = hs * HPL + j;
#pragma unroll
      for (int k = 0; k < D; ++k) r[k * H + h] = acc[k][j];
      r[D * H + h] = acc[D][j];
      r[D * H + H + h] = dw1[j];
    }
    if (hs == 0) {
      r[D * H + 2 * H] = db1;
      dsc[warp] = llacc;
    }
  }
  __syncthreads();
  float* po = g.partial_out + ((size_t)win * S + slice) * g.Pp;
  for (int p = tid; p < G::P; p += FP32_THREADS) {
    float s = red[p];
#pragma unroll
    for (int w = 1; w < FP32_WARPS; ++w) s += red[w * PP + p];
    po[p] = s;
  }
  if (tid == 0) {
    double s = dsc[0];
#pragma unroll
    for (int w = 1; w < FP32_WARPS; ++w) s += dsc[w];
    g.ll_out[(size_t)win * S + slice] = s;
  }
}

// ---- host side -----------------------------------------------------------
template <int H, int HS, int R>
static cudaError_t launch_fp32_t(const GradParams& g, int slices, int windows, cudaStream_t st) {
  using G = Fp32Geom<H, HS, R>;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(grad_fp32_kernel<H, HS, R>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G::SMEM);
    if (e != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  grad_fp32_kernel<H, HS, R><<<dim3(slices, windows), FP32_THREADS, G::SMEM, st>>>(g);
  return cudaGetLastError();
}

int fp32_tile_rows(int H) { return H == 40 ? Fp32Geom<40, 8, 4>::TILE : Fp32Geom<128, 32, 8>::TILE; }

cudaError_t launch_grad_fp32(int H, const GradParams& g, int slices, int windows, cudaStream_t st) {
  if (H == 40) return launch_fp32_t<40, 8, 4>(g, slices, windows, st);
  if (H == 128) return launch_fp32_t<128, 32, 8>(g, slices, windows, st);
  return cudaErrorInvalidValue;
}

int fp32_max_ctas_per_sm(int H) {
  int n = 0;
  if (H == 40) {
    cudaFuncSetAttribute(grad_fp32_kernel<40, 8, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)Fp32Geom<40, 8, 4>::SMEM);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, grad_fp32_kernel<40, 8, 4>, FP32_THREADS,
                                                  Fp32Geom<40, 8, 4>::SMEM);
  } else if (H == 128) {
    cudaFuncSetAttribute(grad_fp32_kernel<128, 32, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)Fp32Geom<128, 32, 8>::SMEM);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, grad_fp32_kernel<128, 32, 8>, FP32_THREADS,
                                                  Fp32Geom<128, 32, 8>::SMEM);
  }
  return n;
}

}  // namespace mcmc_b200

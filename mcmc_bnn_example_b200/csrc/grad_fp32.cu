// FP32 (FFMA) fused leapfrog-update + forward + backward kernel.
//
// Stands in for leapfrog_step_kernel of the reference
// (include/mcmc/mcmc_step_ffma.h:154-379): same math, different mapping.
//   * grid = (slices, windows): many independent windows per launch, each
//     window's rows split over `slices` CTAs;
//   * rows arrive through the bulk-copy engine in double-buffered 128-row tiles
//     of the repacked [rows][24] dataset (contiguous, 16-byte aligned);
//   * forward: a thread owns 8 rows x HPL hidden units (register tile), reads
//     its rows four features at a time and the weights as one vector per
//     feature; the output layer needs one shuffle reduction over the lanes that
//     share a row;
//   * backward: dZ goes through shared memory once, and the threads regroup:
//     a thread owns a 12-feature x HPL-hidden slice of dW0 for one sixteen-row
//     subset of the tile, so the dW0 accumulator costs 12*HPL registers instead
//     of 23*HPL (the reference keeps dW0 in shared memory and adds to it with
//     atomics, mcmc_step_ffma.h:346-367);
//   * no atomics: row subsets -> shared-memory tree -> one partial vector per
//     CTA; the next launch (or the accept kernel) sums the partials of a window
//     in a fixed order, so results are bit-reproducible.
#include "common.cuh"

namespace mcmc_b200 {

constexpr int FP32_TILE = 128;

template <int H, int HPL, int NT>
struct Fp32Geom {
  static constexpr int D = 22;
  static constexpr int CG = H / HPL;               // column (hidden-unit) groups
  static constexpr int Q4 = HPL / 4, R1 = HPL % 4; // a group's units: Q4 vectors of four + R1 singles
  static constexpr int RG = NT / CG;               // forward: row groups
  static constexpr int RPT = FP32_TILE / RG;       // forward: rows per thread
  static constexpr int KPT = 12;                   // backward: features per thread (two halves of 24)
  static constexpr int MT = 2 * CG;                // backward: accumulator slices
  static constexpr int RSUB = NT / MT;             // backward: row subsets
  static constexpr int RPS = FP32_TILE / RSUB;     // backward: rows per subset
  static constexpr int NW = NT / 32;
  static constexpr int P = D * H + 2 * H + 1;
  static constexpr int PP = (P + 3) / 4 * 4;
  static constexpr int XS_FLOATS = 2 * FP32_TILE * KP;
  static constexpr int ES_FLOATS = FP32_TILE * H;
  static constexpr int WS_FLOATS = (D + 1) * H;
  static constexpr int W1_FLOATS = (H + 3) / 4 * 4;
  static constexpr int RED_FLOATS = RSUB * PP;     // aliases the row tiles and dZ after the last tile
  static constexpr int BIG_FLOATS = XS_FLOATS + ES_FLOATS > RED_FLOATS ? XS_FLOATS + ES_FLOATS : RED_FLOATS;
  static constexpr size_t SMEM = sizeof(float) * (BIG_FLOATS + WS_FLOATS + W1_FLOATS);
  static_assert(H % HPL == 0 && NT % CG == 0 && FP32_TILE % RG == 0, "forward tiling");
  static_assert(NT % MT == 0 && FP32_TILE % RSUB == 0 && 32 % CG == 0, "backward tiling");
  static_assert(KP == 2 * KPT, "a repacked row is two halves of twelve floats");
  // unit j of group cg inside a block of H floats (one feature's weights, or one row of dZ):
  // vectors first ([Q4][CG][4]), then singles ([R1][CG]); a warp's vector loads are contiguous
  __host__ __device__ static constexpr int off(int cg, int j) {
    return j < 4 * Q4 ? (j / 4) * (CG * 4) + cg * 4 + (j % 4) : Q4 * CG * 4 + (j - 4 * Q4) * CG + cg;
  }
};

template <int H, int HPL, int NT>
__device__ __forceinline__ void load_units(const float* blk, int cg, float* v) {
  using G = Fp32Geom<H, HPL, NT>;
#pragma unroll
  for (int q = 0; q < G::Q4; ++q) {
    const float4 t = *reinterpret_cast<const float4*>(blk + q * (G::CG * 4) + cg * 4);
    v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
  }
#pragma unroll
  for (int r = 0; r < G::R1; ++r) v[4 * G::Q4 + r] = blk[G::Q4 * G::CG * 4 + r * G::CG + cg];
}
template <int H, int HPL, int NT>
__device__ __forceinline__ void store_units(float* blk, int cg, const float* v) {
  using G = Fp32Geom<H, HPL, NT>;
#pragma unroll
  for (int q = 0; q < G::Q4; ++q)
    *reinterpret_cast<float4*>(blk + q * (G::CG * 4) + cg * 4) =
        make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
#pragma unroll
  for (int r = 0; r < G::R1; ++r) blk[G::Q4 * G::CG * 4 + r * G::CG + cg] = v[4 * G::Q4 + r];
}

template <int H, int HPL, int NT, int MINB>
__global__ void __launch_bounds__(NT, MINB) grad_fp32_kernel(const GradParams g) {
  using G = Fp32Geom<H, HPL, NT>;
  constexpr int D = G::D, CG = G::CG, RG = G::RG, RPT = G::RPT, KPT = G::KPT, MT = G::MT;
  constexpr int RSUB = G::RSUB, RPS = G::RPS, NW = G::NW, PP = G::PP, TILE = FP32_TILE;
  constexpr uint32_t TILE_BYTES = TILE * KP * sizeof(float);

  extern __shared__ __align__(128) unsigned char smem_raw[];
  float* xs = reinterpret_cast<float*>(smem_raw);   // [2][TILE][24]
  float* es = xs + G::XS_FLOATS;                     // [TILE][H] dZ, unit layout of Fp32Geom::off
  float* red = xs;                                   // [RSUB][PP] after the last tile
  float* ws = xs + G::BIG_FLOATS;                    // [23][H] weights + hidden bias, same unit layout
  float* w1s = ws + G::WS_FLOATS;
  __shared__ __align__(8) uint64_t bars[2];
  __shared__ float b1s;
  __shared__ float red_w1[NW][H];
  __shared__ float red_db1[NW];
  __shared__ double red_ll[NW];

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
  __syncthreads();
  // The first row tile may be fetched ahead of the dependency wait only when no kernel directly before
  // this one in the stream wrote the dataset (inside a chain none does; right after a repack one did).
  const bool early_rows = g.data_fresh == 0;
  if (tid == 0 && t0 < t1 && early_rows) {
    mbar_expect_tx(&bars[0], TILE_BYTES);
    bulk_g2s(xs, xw + (size_t)t0 * TILE * KP, TILE_BYTES, &bars[0]);
  }
  pdl_trigger();
  pdl_wait();
  if (tid == 0 && t0 < t1 && !early_rows) {
    mbar_expect_tx(&bars[0], TILE_BYTES);
    bulk_g2s(xs, xw + (size_t)t0 * TILE * KP, TILE_BYTES, &bars[0]);
  }
  // fused leapfrog update; parameters land in the layout the lanes read
  for (int p = tid; p < G::P; p += NT) {
    const float w = leapfrog_param(g, win, p, slice == 0);
    if (p < D * H + H) {  // W0 rows 0..21 and the bias as row 22
      const int k = p / H, h = p - k * H;
      ws[k * H + G::off(h / HPL, h % HPL)] = w;
    } else if (p < D * H + 2 * H) {
      w1s[p - (D * H + H)] = w;
    } else {
      b1s = w;
    }
  }
  __syncthreads();

  const int lane = tid & 31, warp = tid >> 5;
  const int cg = tid % CG;          // hidden-unit group, the same in both phases
  const int rg = tid / CG;          // forward: rows rg, rg + RG, ...
  const int kh = (tid % MT) / CG;   // backward: feature half
  const int rsub = tid / MT;        // backward: rows rsub, rsub + RSUB, ...
  float w1r[HPL];
#pragma unroll
  for (int j = 0; j < HPL; ++j) w1r[j] = w1s[cg * HPL + j];
  const float b1 = b1s;

  // dW0 rows kh*12 .. kh*12+11 (row 22 = db0 through the constant-1 column), two features per register
  // pair: the backward FMAs are issued as packed f32x2 (half the issue slots)
  uint64_t acc2[KPT / 2][HPL];
#pragma unroll
  for (int k = 0; k < KPT / 2; ++k)
#pragma unroll
    for (int j = 0; j < HPL; ++j) acc2[k][j] = 0ull;
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
    const float* xt = xs + stage * TILE * KP;
    // ---- forward: z = [x, 1] . [W0; b0] for rows rg + i*RG ----
    float z[RPT][HPL];
    float yv[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i)
#pragma unroll
      for (int j = 0; j < HPL; ++j) z[i][j] = 0.f;
#pragma unroll
    for (int kg = 0; kg < KP / 4; ++kg) {
      float4 xv[RPT];
#pragma unroll
      for (int i = 0; i < RPT; ++i)
        xv[i] = *reinterpret_cast<const float4*>(xt + (i * RG + rg) * KP + kg * 4);
      if (kg == KP / 4 - 1) {
#pragma unroll
        for (int i = 0; i < RPT; ++i) yv[i] = xv[i].w;
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const int k = kg * 4 + kk;
        if (k > D) continue;
        float wv[HPL];
        load_units<H, HPL, NT>(ws + k * H, cg, wv);
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
          const float xk = kk == 0 ? xv[i].x : kk == 1 ? xv[i].y : kk == 2 ? xv[i].z : xv[i].w;
#pragma unroll
          for (int j = 0; j < HPL; ++j) z[i][j] = fmaf(xk, wv[j], z[i][j]);
        }
      }
    }
    // ---- activation, output layer, loss, dZ ----
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      float pred = 0.f;
#pragma unroll
      for (int j = 0; j < HPL; ++j) {
        z[i][j] = tanh_ref(z[i][j]);
        pred = fmaf(w1r[j], z[i][j], pred);
      }
#pragma unroll
      for (int o = 1; o < CG; o <<= 1) pred += __shfl_xor_sync(0xffffffffu, pred, o);
      pred += b1;
      const int row = i * RG + rg;
      const int grow = t * TILE + row;
      const bool valid = grow < g.n_rows;
      float loss, dy;
      lik_terms(g.lik, yv[i], pred, loss, dy);
      if (!valid) { loss = 0.f; dy = 0.f; }
      if (cg == 0) {
        llacc += (double)loss;
        db1 += dy;
        if (g.row_loss && valid) g.row_loss[(long long)win * g.row_loss_stride + grow] = loss;
      }
#pragma unroll
      for (int j = 0; j < HPL; ++j) {
        const float h = z[i][j];
        dw1[j] = fmaf(dy, h, dw1[j]);
        z[i][j] = fmaf(-h, h, 1.f) * (w1r[j] * dy);  // tanh_t::bwd
      }
      store_units<H, HPL, NT>(es + row * H, cg, z[i]);
    }
    __syncthreads();
    // ---- backward: dW0 (and db0 through the constant-1 column) for rows rsub + s*RSUB ----
#pragma unroll 4
    for (int s = 0; s < RPS; ++s) {
      const int row = s * RSUB + rsub;
      const float* xr = xt + row * KP + kh * KPT;
      uint64_t xk2[KPT / 2];
#pragma unroll
      for (int q = 0; q < KPT / 4; ++q) {
        const float4 v = *reinterpret_cast<const float4*>(xr + 4 * q);
        xk2[2 * q] = pack2(v.x, v.y);
        xk2[2 * q + 1] = pack2(v.z, v.w);
      }
      float ev[HPL];
      load_units<H, HPL, NT>(es + row * H, cg, ev);
#pragma unroll
      for (int j = 0; j < HPL; ++j) {
        const uint64_t e2 = pack2(ev[j], ev[j]);
#pragma unroll
        for (int k = 0; k < KPT / 2; ++k) acc2[k][j] = fma2(xk2[k], e2, acc2[k][j]);
      }
    }
    __syncthreads();
  }

  // ---- reduce: row subsets / row groups -> CTA partial ----
  {
    float* r = red + rsub * PP;
#pragma unroll
    for (int k = 0; k < KPT; ++k) {
      const int kk = kh * KPT + k;
      if (kk <= D) {  // feature 23 is y: not a gradient row
#pragma unroll
        for (int j = 0; j < HPL; ++j) {
          float lo, hi;
          unpack2(acc2[k / 2][j], lo, hi);
          r[kk * H + cg * HPL + j] = (k & 1) ? hi : lo;
        }
      }
    }
  }
  // dW1: the lanes of a warp that share a hidden group, then the warps
#pragma unroll
  for (int o = CG; o < 32; o <<= 1) {
#pragma unroll
    for (int j = 0; j < HPL; ++j) dw1[j] += __shfl_xor_sync(0xffffffffu, dw1[j], o);
  }
  if (lane < CG) {
#pragma unroll
    for (int j = 0; j < HPL; ++j) red_w1[warp][cg * HPL + j] = dw1[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    db1 += __shfl_xor_sync(0xffffffffu, db1, o);
    llacc += __shfl_xor_sync(0xffffffffu, llacc, o);
  }
  if (lane == 0) {
    red_db1[warp] = db1;
    red_ll[warp] = llacc;
  }
  __syncthreads();
  float* po = g.partial_out + ((size_t)win * S + slice) * g.Pp;
  for (int p = tid; p < G::P; p += NT) {
    float s;
    if (p < D * H + H) {
      s = red[p];
#pragma unroll
      for (int r = 1; r < RSUB; ++r) s += red[r * PP + p];
    } else if (p < D * H + 2 * H) {
      const int h = p - (D * H + H);
      s = red_w1[0][h];
#pragma unroll
      for (int w = 1; w < NW; ++w) s += red_w1[w][h];
    } else {
      s = red_db1[0];
#pragma unroll
      for (int w = 1; w < NW; ++w) s += red_db1[w];
    }
    po[p] = s;
  }
  if (tid == 0) {
    double s = red_ll[0];
#pragma unroll
    for (int w = 1; w < NW; ++w) s += red_ll[w];
    g.ll_out[(size_t)win * S + slice] = s;
  }
}

// ---- host side -----------------------------------------------------------
template <int H, int HPL, int NT, int MINB>
static cudaError_t launch_fp32_t(const GradParams& g, int slices, int windows, cudaStream_t st) {
  using G = Fp32Geom<H, HPL, NT>;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(grad_fp32_kernel<H, HPL, NT, MINB>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G::SMEM);
    if (e != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  return launch_chain_kernel(grad_fp32_kernel<H, HPL, NT, MINB>, dim3(slices, windows), dim3(NT), G::SMEM, st,
                             g);
}

int fp32_tile_rows(int H) { (void)H; return FP32_TILE; }

cudaError_t launch_grad_fp32(int H, const GradParams& g, int slices, int windows, cudaStream_t st) {
  if (H == 40) return launch_fp32_t<40, 5, 128, 3>(g, slices, windows, st);
  if (H == 128) return launch_fp32_t<128, 8, 256, 1>(g, slices, windows, st);
  return cudaErrorInvalidValue;
}

int fp32_max_ctas_per_sm(int H) {
  int n = 0;
  if (H == 40) {
    cudaFuncSetAttribute(grad_fp32_kernel<40, 5, 128, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)Fp32Geom<40, 5, 128>::SMEM);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, grad_fp32_kernel<40, 5, 128, 3>, 128,
                                                  Fp32Geom<40, 5, 128>::SMEM);
  } else if (H == 128) {
    cudaFuncSetAttribute(grad_fp32_kernel<128, 8, 256, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)Fp32Geom<128, 8, 256>::SMEM);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, grad_fp32_kernel<128, 8, 256, 1>, 256,
                                                  Fp32Geom<128, 8, 256>::SMEM);
  }
  return n;
}

}  // namespace mcmc_b200

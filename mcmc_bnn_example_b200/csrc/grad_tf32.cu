// TF32 tensor-core fused leapfrog-update + forward + backward kernel for
// sm_100a: tcgen05.mma kind::tf32 with accumulators in tensor memory, rows
// staged by TMA.
//
// Stands in for mcmc_step_kernel / leapfrog_step_single of the reference
// (include/mcmc/mcmc_step_tc.h:306-677), which issues warp-level
// mma.sync.m16n8k8 and exchanges fragments through shared memory.  Here:
//
//   forward   Z[128 rows x NF] = Xa[128 x 24] . W0a[24 x NF]
//             A = the TMA-staged row tile (K-major, 128-byte swizzle), B = the
//             per-step staged weights; row 22 of W0a is the hidden bias (Xa
//             has a constant-1 column), row 23 is zero (Xa column 23 carries y).
//             One tcgen05.ld gives each thread ONE FULL ROW of Z, so tanh, the
//             output layer, the loss and dZ need no cross-lane traffic at all
//             (the reference reduces and broadcasts across lanes,
//             mcmc_step_tc.h:426-432, :468-474).
//   backward  G[MB hidden x 24] += E^T[MB x 128 rows] . Xa[128 x 24]
//             E = (1 - h^2) * dL/dpred, written row-per-thread into shared
//             memory as the MN-major A operand; the SAME staged row tile is the
//             MN-major B operand.  G stays in tensor memory for every tile the
//             CTA owns and is read once at the end: dW0[k][j] = W1[j] * G[j][k],
//             db0[j] = W1[j] * G[j][22].  W1[j] is a per-output-row constant, so
//             it is applied after the reduction instead of per element.
//
// TF32 semantics: operands are raw FP32 bit patterns whose low 13 mantissa
// bits the tensor core ignores, as in the reference (mov.b32 of FP32 values,
// mcmc_step_tc.h:374,386,539,546).  tanh is tanh.approx.f32 (one MUFU op
// instead of the reference's ex2 + rcp), within the TF32 mode's tolerance.
//
// No atomics; every wait is bounded and reports through the status word.
#include <cuda.h>
#include <stdio.h>
#include <stdlib.h>
#include "common.cuh"
#include "chain.cuh"

namespace mcmc_b200 {

constexpr int TF32_THREADS = 128;

template <int H, int NST_>
struct Tf32Geom {
  static constexpr int D = 22;
  static constexpr int NST = NST_;                         // TMA stages
  static constexpr int NF = (H + 15) / 16 * 16;            // forward N (M = 128 needs N % 16 == 0)
  static constexpr int MB = H <= 64 ? 64 : 128;            // backward M
  static constexpr int NB = MB == 64 ? 24 : 32;            // backward N
  static constexpr int ATOMS = MB / 32;                    // 32-float swizzle atoms along M
  static constexpr int FWD_COLS = NF <= 64 ? 64 : 128;
  static constexpr int BWD_COL0 = FWD_COLS;
  static constexpr int TMEM_COLS = FWD_COLS + 32 <= 128 ? 128 : 256;
  static constexpr int TILE_BYTES = TF32_TILE * 128;       // 128 rows x 32 floats (24 real + 8 zero fill)
  static constexpr int XS_BYTES = NST * TILE_BYTES;          // K-major copies (forward A operand)
  static constexpr int XB_BYTES = NST * TILE_BYTES;          // MN-major copies (backward B operand)
  static constexpr int ES_BYTES = ATOMS * TILE_BYTES;
  static constexpr int W0S_BYTES = NF * 128;
  static constexpr int W1_BYTES = (H + 3) / 4 * 16;
  static constexpr int P = D * H + 2 * H + 1;
  static constexpr size_t SMEM = 1024 + XS_BYTES + XB_BYTES + ES_BYTES + W0S_BYTES + W1_BYTES;
  static_assert(H % 4 == 0, "hidden width must be a multiple of 4");
  static_assert(TF32_THREADS * (H + 1) * 4 <= ES_BYTES, "dW1 reduction scratch aliases the E buffer");
};

// ---- tcgen05 wrappers ----------------------------------------------------
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, float* v) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                 "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* tmap, int x, int y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// Shared-memory matrix descriptor (version 1).  Byte offsets are encoded
// without their 4 low bits.  Layout types used here:
//   2 = 128-byte swizzle of 16-byte chunks   (K-major operands)
//   1 = 128-byte swizzle of 32-byte chunks   (the only layout the tensor core
//       accepts for MN-major operands of 32-bit types)
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes, uint32_t layout_type) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) |
         ((uint64_t)layout_type << 61);
}
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                    uint32_t sbo_bytes) {
  return umma_desc(smem_addr, lbo_bytes, sbo_bytes, 2);
}
// MN-major, 32-byte-chunk swizzle: rows (K) of 128 bytes, groups of 4 rows 512 bytes apart,
// 32-float atoms along M/N `atom_stride` bytes apart
__device__ __forceinline__ uint64_t umma_desc_mn32(uint32_t smem_addr, uint32_t atom_stride) {
  return umma_desc(smem_addr, atom_stride, 512, 1);
}
// Instruction descriptor: F32 accumulate, TF32 x TF32, dense.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

template <int H, int NST>
__global__ void __launch_bounds__(TF32_THREADS)
grad_tf32_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap_mn,
                 const GradParams g, float* dbg) {
  using G = Tf32Geom<H, NST>;
  constexpr int D = G::D, NF = G::NF, MB = G::MB, NB = G::NB;
  constexpr uint32_t IDESC_FWD = umma_idesc_tf32(128, NF, 0, 0);
  constexpr uint32_t IDESC_BWD = umma_idesc_tf32(MB, NB, 1, 1);

  extern __shared__ unsigned char smem_raw[];
  unsigned char* base =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* xs = base;                   // [NST][128 rows][128 B], TMA-written, swizzled
  unsigned char* xb = xs + G::XS_BYTES;       // [NST][128 rows][128 B], same tiles, 32-byte-chunk swizzle
  unsigned char* es = xb + G::XB_BYTES;       // [ATOMS][128 rows][128 B], E operand, 32-byte-chunk swizzle
  unsigned char* w0s = es + G::ES_BYTES;      // [NF][128 B] weights, K-major, swizzled
  float* w1s = reinterpret_cast<float*>(w0s + G::W0S_BYTES);
  __shared__ __align__(8) uint64_t bar_tma[NST];
  __shared__ __align__(8) uint64_t bar_fwd, bar_bwd;
  __shared__ uint32_t tmem_slot;
  __shared__ float b1s;
  __shared__ float red_db1[4];
  __shared__ double red_ll[4];

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int win = blockIdx.y, slice = blockIdx.x, S = gridDim.x;
  const int t0 = (int)((long long)slice * g.n_tiles / S);
  const int t1 = (int)((long long)(slice + 1) * g.n_tiles / S);
  const int rows_pad = g.n_tiles * TF32_TILE;
  const int grow0 = (g.data_window0 + win) * rows_pad;  // first row of this window in the tensor map

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_slot)),
                 "r"((uint32_t)G::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    for (int s = 0; s < NST; ++s) mbar_init(&bar_tma[s], 1);
    mbar_init(&bar_fwd, 1);
    mbar_init(&bar_bwd, 1);
    mbar_fence_init();
  }
  // zero the weight operand (rows >= H, k >= 23 stay zero) and the E operand
  for (int i = tid; i < (G::W0S_BYTES + G::ES_BYTES) / 16; i += TF32_THREADS)
    reinterpret_cast<float4*>(es)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tmem_fwd = tmem;
  const uint32_t tmem_bwd = tmem + G::BWD_COL0;

  if (tid == 0) {
    for (int s = 0; s < NST && t0 + s < t1; ++s) {
      mbar_expect_tx(&bar_tma[s], 2 * G::TILE_BYTES);
      tma_load_2d(xs + s * G::TILE_BYTES, &tmap, 0, grow0 + (t0 + s) * TF32_TILE, &bar_tma[s]);
      tma_load_2d(xb + s * G::TILE_BYTES, &tmap_mn, 0, grow0 + (t0 + s) * TF32_TILE, &bar_tma[s]);
    }
  }
  // fused leapfrog update; W0 and b0 go into the swizzled K-major B operand:
  // element (n = hidden unit, k) at n*128 + ((k/4) ^ (n%8))*16 + (k%4)*4
  for (int p = tid; p < G::P; p += TF32_THREADS) {
    const float w = leapfrog_param(g, win, p, slice == 0);
    if (p < D * H + H) {
      const int k = p / H, n = p - k * H;
      *reinterpret_cast<float*>(w0s + n * 128 + (((k >> 2) ^ (n & 7)) << 4) + ((k & 3) << 2)) = w;
    } else if (p < D * H + 2 * H) {
      w1s[p - (D * H + H)] = w;
    } else {
      b1s = w;
    }
  }
  fence_proxy_async_smem();
  __syncthreads();

  const float b1 = b1s;
  float dw1[H];
#pragma unroll
  for (int j = 0; j < H; ++j) dw1[j] = 0.f;
  float db1 = 0.f;
  double llacc = 0.0;
  bool ok = true;
  const uint32_t es_addr = smem_u32(es);
  const uint32_t w0s_addr = smem_u32(w0s);

  if (tid == 0 && t0 < t1) {
    ok = mbar_wait(&bar_tma[0], 0, g.status, 201);
    tc_fence_after();
    const uint32_t xa = smem_u32(xs);
#pragma unroll
    for (int kb = 0; kb < 3; ++kb)
      tc_mma_tf32(tmem_fwd, umma_desc_sw128(xa + kb * 32, 16, 1024),
                  umma_desc_sw128(w0s_addr + kb * 32, 16, 1024), IDESC_FWD, kb > 0);
    tc_commit(&bar_fwd);
  }

  for (int t = t0; t < t1; ++t) {
    const int it = t - t0;
    const int stage = it % NST;
    // forward accumulator of this tile
    ok = ok && mbar_wait(&bar_fwd, it & 1, g.status, 202);
    if (tid == 0) {
      // the previous tile's backward MMAs have released their row tile and E:
      // refill that stage with the tile NST-1 ahead
      if (it > 0) ok = ok && mbar_wait(&bar_bwd, (it - 1) & 1, g.status, 203);
      const int tn = t + NST - 1;
      if (it > 0 && tn < t1 && ok) {
        const int sn = (it + NST - 1) % NST;
        mbar_expect_tx(&bar_tma[sn], 2 * G::TILE_BYTES);
        tma_load_2d(xs + sn * G::TILE_BYTES, &tmap, 0, grow0 + tn * TF32_TILE, &bar_tma[sn]);
        tma_load_2d(xb + sn * G::TILE_BYTES, &tmap_mn, 0, grow0 + tn * TF32_TILE, &bar_tma[sn]);
      }
    }
    tc_fence_after();
    float z[H];
    const uint32_t trow = tmem_fwd + ((uint32_t)(warp * 32) << 16);
#pragma unroll
    for (int c = 0; c < H; c += 8) tc_ld8(trow + c, z + c);
    tc_wait_ld();

    const unsigned char* xrow = xs + stage * G::TILE_BYTES + tid * 128;
    const float y = *reinterpret_cast<const float*>(xrow + (((COL_Y >> 2) ^ (tid & 7)) << 4) +
                                                    ((COL_Y & 3) << 2));
    if (dbg && blockIdx.x == 0 && blockIdx.y == 0 && it == 0) {
#pragma unroll
      for (int j = 0; j < H; ++j) dbg[tid * 64 + j] = z[j];
      dbg[tid * 64 + 63] = y;
      for (int c = 0; c < 32; ++c)
        dbg[12288 + tid * 32 + c] = reinterpret_cast<const float*>(xb + stage * G::TILE_BYTES)[tid * 32 + c];
    }
    float pred = b1;
#pragma unroll
    for (int j = 0; j < H; j += 4) {
      const float4 w1v = *reinterpret_cast<const float4*>(w1s + j);
      z[j] = tanh_fast(z[j]);
      z[j + 1] = tanh_fast(z[j + 1]);
      z[j + 2] = tanh_fast(z[j + 2]);
      z[j + 3] = tanh_fast(z[j + 3]);
      pred = fmaf(w1v.x, z[j], pred);
      pred = fmaf(w1v.y, z[j + 1], pred);
      pred = fmaf(w1v.z, z[j + 2], pred);
      pred = fmaf(w1v.w, z[j + 3], pred);
    }
    const int grow = t * TF32_TILE + tid;
    const bool valid = grow < g.n_rows;
    float loss, dy;
    lik_terms(g.lik, y, pred, loss, dy);
    if (!valid) { loss = 0.f; dy = 0.f; }
    llacc += (double)loss;
    if (g.row_loss && valid) g.row_loss[(long long)win * g.row_loss_stride + grow] = loss;
    db1 += dy;
#pragma unroll
    for (int j = 0; j < H; ++j) {
      const float h = z[j];
      dw1[j] = fmaf(dy, h, dw1[j]);
      z[j] = fmaf(-h, h, 1.f) * dy;  // E; the W1 factor is applied at read-out
    }
    // E row -> MN-major A operand (the previous backward MMAs are done with it)
    if (it > 0) ok = ok && mbar_wait(&bar_bwd, (it - 1) & 1, g.status, 204);
    unsigned char* erow = es + tid * 128;
#pragma unroll
    for (int c = 0; c < H / 4; ++c)
      *reinterpret_cast<float4*>(erow + (c >> 3) * G::TILE_BYTES + ((((c & 7) >> 1) ^ (tid & 3)) << 5) +
                                 ((c & 1) << 4)) =
          make_float4(z[4 * c], z[4 * c + 1], z[4 * c + 2], z[4 * c + 3]);
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && ok) {
      tc_fence_after();
      // next tile's forward first, so its epilogue can start while this
      // tile's backward MMAs run
      if (t + 1 < t1) {
        const int sn = (it + 1) % NST;
        ok = mbar_wait(&bar_tma[sn], ((it + 1) / NST) & 1, g.status, 205);
        tc_fence_after();
        if (ok) {
        const uint32_t xa = smem_u32(xs + sn * G::TILE_BYTES);
#pragma unroll
        for (int kb = 0; kb < 3; ++kb)
          tc_mma_tf32(tmem_fwd, umma_desc_sw128(xa + kb * 32, 16, 1024),
                      umma_desc_sw128(w0s_addr + kb * 32, 16, 1024), IDESC_FWD, kb > 0);
        tc_commit(&bar_fwd);
        }
      }
      const uint32_t xba = smem_u32(xb + stage * G::TILE_BYTES);
#pragma unroll
      for (int kb = 0; kb < TF32_TILE / 8; ++kb)
        tc_mma_tf32(tmem_bwd, umma_desc_mn32(es_addr + kb * 1024, G::TILE_BYTES),
                    umma_desc_mn32(xba + kb * 1024, G::TILE_BYTES), IDESC_BWD,
                    (it > 0 || kb > 0) ? 1u : 0u);
      tc_commit(&bar_bwd);
    }
  }

  // ---- read-out ----
  const int nt = t1 - t0;
  if (nt > 0 && ok) ok = mbar_wait(&bar_bwd, (nt - 1) & 1, g.status, 206);
  tc_fence_after();
  float* po = g.partial_out + ((size_t)win * S + slice) * g.Pp;
  {
    float gacc[NB];
    const uint32_t trow = tmem_bwd + ((uint32_t)(warp * 32) << 16);
#pragma unroll
    for (int c = 0; c < NB; c += 8) tc_ld8(trow + c, gacc + c);
    tc_wait_ld();
    if (dbg && blockIdx.x == 0 && blockIdx.y == 0) {
#pragma unroll
      for (int c = 0; c < NB; ++c) dbg[8192 + tid * 32 + c] = gacc[c];
    }
    // M = 64: accumulator row i lives in lane 32*(i/16) + i%16; M = 128: lane i
    const int hidx = (MB == 64) ? (lane < 16 ? warp * 16 + lane : -1) : tid;
    if (hidx >= 0 && hidx < H) {
      const float w1 = (nt > 0) ? w1s[hidx] : 0.f;
#pragma unroll
      for (int k = 0; k < D; ++k) po[k * H + hidx] = (nt > 0) ? w1 * gacc[k] : 0.f;
      po[D * H + hidx] = (nt > 0) ? w1 * gacc[COL_ONE] : 0.f;
    }
  }
  // dW1: per-thread partials -> shared memory (aliases E; all MMAs are done) -> column sums
  __syncthreads();
  float* sc = reinterpret_cast<float*>(es);
#pragma unroll
  for (int j = 0; j < H; ++j) sc[tid * (H + 1) + j] = dw1[j];
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
  for (int j = tid; j < H; j += TF32_THREADS) {
    float s = 0.f;
    for (int r = 0; r < TF32_THREADS; ++r) s += sc[r * (H + 1) + j];
    po[D * H + H + j] = s;
  }
  if (tid == 0) {
    po[D * H + 2 * H] = (red_db1[0] + red_db1[1]) + (red_db1[2] + red_db1[3]);
    g.ll_out[(size_t)win * S + slice] = (red_ll[0] + red_ll[1]) + (red_ll[2] + red_ll[3]);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                 "r"((uint32_t)G::TMEM_COLS)
                 : "memory");
  }
}

// ---- host side -----------------------------------------------------------
constexpr int TF32_NST = 2;

int tf32_supported(int H) { return H == 40; }

template <int H>
static cudaError_t launch_tf32_t(const void* tmap, const void* tmap_mn, const GradParams& g, int slices,
                                 int windows, float* dbg, cudaStream_t st) {
  using G = Tf32Geom<H, TF32_NST>;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(grad_tf32_kernel<H, TF32_NST>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G::SMEM);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(grad_tf32_kernel<H, TF32_NST>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  grad_tf32_kernel<H, TF32_NST><<<dim3(slices, windows), TF32_THREADS, G::SMEM, st>>>(
      *reinterpret_cast<const CUtensorMap*>(tmap), *reinterpret_cast<const CUtensorMap*>(tmap_mn), g, dbg);
  return cudaGetLastError();
}

cudaError_t launch_grad_tf32(int H, const void* tmap, const void* tmap_mn, const GradParams& g, int slices,
                             int windows, float* dbg, cudaStream_t st) {
  if (H == 40) return launch_tf32_t<40>(tmap, tmap_mn, g, slices, windows, dbg, st);
  return cudaErrorInvalidValue;
}

int tf32_max_ctas_per_sm(int H) {
  int n = 0;
  if (H == 40) {
    using G = Tf32Geom<40, TF32_NST>;
    cudaError_t e1 = cudaFuncSetAttribute(grad_tf32_kernel<40, TF32_NST>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G::SMEM);
    cudaFuncSetAttribute(grad_tf32_kernel<40, TF32_NST>, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    cudaError_t e2 = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, grad_tf32_kernel<40, TF32_NST>,
                                                                   TF32_THREADS, G::SMEM);
    if (getenv("MCMC_B200_DEBUG"))
      fprintf(stderr, "tf32 occupancy: attr=%d occ=%d n=%d smem=%zu\n", (int)e1, (int)e2, n, (size_t)G::SMEM);
    const int by_tmem = 512 / G::TMEM_COLS;
    if (n > by_tmem) n = by_tmem;
  }
  return n;
}

}  // namespace mcmc_b200

extern "C" __attribute__((visibility("default"))) void mcmc_b200_debug_occupancy() {
  using namespace mcmc_b200;
  cudaFuncAttributes a;
  cudaFuncGetAttributes(&a, grad_tf32_kernel<40, TF32_NST>);
  printf("tf32 kernel: regs %d static smem %zu maxDyn %d local %zu maxThreads %d carve %d\n", a.numRegs,
         a.sharedSizeBytes, a.maxDynamicSharedSizeBytes, a.localSizeBytes, a.maxThreadsPerBlock,
         a.preferredShmemCarveout);
  for (int kb = 8; kb <= 112; kb += 8) {
    int n = -1;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, grad_tf32_kernel<40, TF32_NST>, 128,
                                                                  (size_t)kb * 1024);
    printf("  dyn smem %d KB -> %d CTAs/SM (err %d)\n", kb, n, (int)e);
  }
}

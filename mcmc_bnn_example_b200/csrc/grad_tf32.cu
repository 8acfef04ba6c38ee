// TF32 tensor-core fused leapfrog-update + forward + backward kernel for
// sm_100a: tcgen05.mma kind::tf32 with accumulators AND the forward A operand
// in tensor memory, rows staged by TMA.
//
// Stands in for mcmc_step_kernel / leapfrog_step_single of the reference
// (include/mcmc/mcmc_step_tc.h:306-677), which issues warp-level
// mma.sync.m16n8k8 and exchanges fragments through shared memory.
//
// Shape of the kernel.  A kernel that allocates tensor memory gets one resident
// CTA per SM on this toolchain (the occupancy query says 1 whatever its other
// resources), so the kernel is persistent: one CTA per SM, three compute
// warpgroups (128 threads = the 128 rows of a tile each) plus one control warp
// whose lane 0 issues every MMA.  A CTA owns a contiguous range of the launch's
// (window, tile) list, cut into per-window segments by the host.
//
//   forward   Z[128 rows x NF] = Xa[128 x 24] . W0a[24 x NF]
//             Each thread copies ITS row of the staged tile into tensor memory
//             (tcgen05.st), which is the A operand; B = the per-segment staged
//             weights (K-major, 128-byte swizzle).  Row 22 of W0a is the hidden
//             bias (Xa has a constant-1 column), row 23 is zero (Xa column 23
//             carries y).  One tcgen05.ld gives each thread ONE FULL ROW of Z,
//             so tanh, the output layer, the loss and dZ need no cross-lane
//             traffic (the reference reduces and broadcasts across lanes,
//             mcmc_step_tc.h:426-432, :468-474).
//   backward  G[64 hidden x 24] += E^T[64 x 128 rows] . Xa[128 x 24]
//             E = (1 - h^2) * dL/dpred, written row-per-thread into shared
//             memory as the MN-major A operand; the TMA-staged row tile is the
//             MN-major B operand.  MN-major operands of a 32-bit type exist in
//             one layout only, the 128-byte swizzle of 32-byte chunks, so the
//             tile is staged in that layout (and that is why the forward takes
//             its A operand from tensor memory instead of a second copy of the
//             tile).  G stays in tensor memory for a whole segment and is read
//             once: dW0[k][j] = W1[j] * G[j][k], db0[j] = W1[j] * G[j][22] — W1[j]
//             is a per-output-row constant, applied after the reduction.
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
#include <utility>
#include "common.cuh"
#include "chain.cuh"
#include "tc05.cuh"

namespace mcmc_b200 {

constexpr int TF32_NWG = 3;                            // compute warpgroups
constexpr int TF32_THREADS = TF32_NWG * 128 + 128;      // + a control warpgroup (one warp per compute warpgroup, one idle)
// registers: 512 threads start with 128 each; the control warpgroup hands most of its share to the
// compute warpgroups (3 * 128 * 152 + 128 * 56 = 65536)
constexpr int TF32_COMPUTE_REGS = 152;
constexpr int TF32_CTRL_REGS = 56;
constexpr int TF32_NST = 3;                            // TMA stages per warpgroup

template <int H>
struct Tf32Geom {
  static constexpr int D = 22;
  static constexpr int NF = (H + 15) / 16 * 16;        // forward N (M = 128 needs N % 16 == 0)
  static constexpr int MB = 64;                        // backward M (hidden, padded)
  static constexpr int NB = 24;                        // backward N (features + 1 + y)
  static constexpr int TILE_BYTES = TF32_TILE * 128;   // 128 rows x 32 floats (24 real + 8 zero fill)
  static constexpr int XB_BYTES = TF32_NWG * TF32_NST * TILE_BYTES;
  // E operand, K-major: 4 atoms of 32 rows (K); in an atom hidden unit j is a 128-byte line.  Only
  // H of the MB lines are written; the lines H..MB-1 the tensor core also reads are whatever
  // follows (they only reach accumulator rows that are never read), so atoms are packed H lines apart.
  static constexpr int ES_ATOM_BYTES = H * 128;
  static constexpr int ES_WG_BYTES = 4 * ES_ATOM_BYTES;
  static constexpr int ES_BYTES = TF32_NWG * ES_WG_BYTES + (MB - H) * 128;
  static constexpr int W0S_BYTES = NF * 128;
  static constexpr int W1_BYTES = (H + 3) / 4 * 16;
  static constexpr int P = D * H + 2 * H + 1;
  static constexpr size_t SMEM = 1024 + XB_BYTES + ES_BYTES + W0S_BYTES + W1_BYTES;
  // tensor-memory columns: A operand and forward accumulator per warpgroup, one backward accumulator
  // (the forward accumulator is double-buffered: forward(n+1) runs while Z(n) is being consumed)
  static constexpr int A_COL0 = 0, A_STRIDE = 24;
  static constexpr int Z_COL0 = TF32_NWG * A_STRIDE, Z_STRIDE = NF;
  static constexpr int G_COL0 = Z_COL0 + 2 * TF32_NWG * Z_STRIDE, G_STRIDE = 24;
  static constexpr int TMEM_COLS = 512;
  static_assert(H % 8 == 0 && H <= 64, "hidden width must be a multiple of 8, at most 64");
  static_assert(G_COL0 + TF32_NWG * G_STRIDE <= TMEM_COLS, "tensor memory budget");
  static_assert(H > 32 && ((H - 32) & (H - 33)) == 0, "the dW1 butterfly handles 32 + a power of two units");
  static_assert(ES_ATOM_BYTES % 1024 == 0, "E atoms must keep the 1024-byte swizzle alignment");
};

// Experiments (built only with -DMCMC_B200_EXPERIMENTS): ABL(bit) skips a part of the pipeline when
// that bit is set in GradParams::ablate, PROF_MARK accumulates clock64 deltas per phase in thread 0 of
// each warpgroup of CTA 0.  In the production build both vanish at compile time.
#ifdef MCMC_B200_EXPERIMENTS
#define ABL(bit) ((g.ablate & (bit)) != 0)
#define PROF_DECL                                                                        \
  const bool prof = dbg && ABL(512) && blockIdx.x == 0 && wtid == 0;             \
  long long pacc[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};                                   \
  long long plast = clock64();
#define PROF_MARK(k)                                   \
  if (prof) {                                          \
    const long long now_ = clock64();                  \
    pacc[k] += now_ - plast;                           \
    plast = now_;                                      \
  }
#define PROF_FLUSH                                                                        \
  if (prof) {                                                                             \
    for (int k = 0; k < 10; ++k) dbg[12288 + wg * 16 + k] += (float)pacc[k];              \
    dbg[12288 + wg * 16 + 10] += (float)my_nt;                                            \
  }
#else
#define ABL(bit) false
#define PROF_DECL
#define PROF_MARK(k)
#define PROF_FLUSH
#endif

// One CTA's share of the cross-CTA sum inside a multi-step launch: parameters
// [blockIdx.x * per_cta, ...) summed over the n_slots partial vectors in a fixed order (one warp per
// parameter: lane l adds slots l, l+32, ..., then a shuffle tree).  Called by the 12 compute warps.
__device__ __forceinline__ void sum_partials_slice(const GradParams& g, const float* partial_out,
                                                   const double* ll_out, int tid) {
  const int nb = (int)gridDim.x;
  const int per_cta = (g.P + nb - 1) / nb;  // <= 12 (one per compute warp)
  const int q = tid >> 5, lane = tid & 31;
  const int p = (int)blockIdx.x * per_cta + q;
  if (q < per_cta && p < g.P) {
    const float* src = partial_out + p;
    float acc = 0.f;
#pragma unroll 5
    for (int sidx = lane; sidx < g.n_slots; sidx += 32) acc += __ldcg(src + (size_t)sidx * g.Pp);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) g.red[p] = (double)acc;
  }
  if (blockIdx.x == (unsigned)(nb - 1) && q == 11) {  // log-likelihood, and the padding of the sum vector
    double l = 0.0;
    for (int sidx = lane; sidx < g.n_slots; sidx += 32) l += __ldcg(ll_out + sidx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) {
      g.red[g.Pp] = l;
      for (int k = g.P; k < g.Pp; ++k) g.red[k] = 0.0;
    }
  }
}

// MULTI = several leapfrog steps of ONE window in one cooperative launch (GradParams::n_steps): after
// every step the CTAs meet at a grid-wide barrier, each CTA sums a few parameters' partials over all
// CTAs into GradParams::red, they meet again, and the next step's prologue reads the sums.  This is
// the reference's persistent-kernel structure (mcmc_step_kernel + sync_and_swap,
// mcmc_step_tc.h:597-677) with a bounded barrier and a fixed-order sum instead of atomics.
template <int H, bool MULTI>
__global__ void __launch_bounds__(TF32_THREADS, 1)
grad_tf32_kernel(const __grid_constant__ CUtensorMap tmap_mn, const GradParams g, float* dbg) {
  using G = Tf32Geom<H>;
  constexpr int D = G::D, NF = G::NF, MB = G::MB, NB = G::NB, NWG = TF32_NWG, NST = TF32_NST;
  constexpr uint32_t IDESC_FWD = umma_idesc_tf32(128, NF, 0, 0);
  constexpr uint32_t IDESC_BWD = umma_idesc_tf32(MB, NB, 0, 1);
  constexpr int NCOMPUTE = NWG * 128;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* base =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* xb = base;                   // [NWG][NST][128 rows][128 B], TMA-written, 32-byte-chunk swizzle
  unsigned char* es = xb + G::XB_BYTES;       // [NWG][4 atoms][H lines][128 B], E operand, K-major, 16-byte-chunk swizzle
  unsigned char* w0s = es + G::ES_BYTES;      // [NF][128 B] weights, K-major, 16-byte-chunk swizzle
  float* w1s = reinterpret_cast<float*>(w0s + G::W0S_BYTES);
  __shared__ __align__(8) uint64_t bar_tma[NWG][NST];
  __shared__ __align__(8) uint64_t bar_fwd[NWG], bar_bwd[NWG];
  __shared__ uint32_t tmem_slot;
  __shared__ float b1s;
  __shared__ float red_w1[NWG * 4][H];
  __shared__ float red_db1[NWG * 4];
  __shared__ double red_ll[NWG * 4];

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const bool is_ctrl = warp >= NWG * 4;
  const int wg = is_ctrl ? warp - NWG * 4 : warp >> 2;  // warpgroup this warp computes for / issues for
  const int wtid = tid & 127;         // row of the tile this thread owns
  const int wwarp = warp & 3;         // tensor-memory subpartition of this warp
  const int rows_pad = g.n_tiles * TF32_TILE;

  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&tmem_slot)),
                 "r"((uint32_t)G::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    for (int w = 0; w < NWG; ++w) {
      for (int s = 0; s < NST; ++s) mbar_init(&bar_tma[w][s], 1);
      mbar_init(&bar_fwd[w], 1);
      mbar_init(&bar_bwd[w], 1);
    }
    mbar_fence_init();
  }
  // zero the weight operand once (rows >= H and k >= 23 stay zero)
  for (int i = tid; i < G::W0S_BYTES / 16; i += TF32_THREADS)
    reinterpret_cast<float4*>(w0s)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tmem_g = tmem + G::G_COL0;
  const uint32_t w0s_addr = smem_u32(w0s);
  const int seg0 = g.seg_ptr[blockIdx.x], seg1 = g.seg_ptr[blockIdx.x + 1];  // host-written table
  bool ok = true;
  // (every CTA of a multi-step launch owns at least one segment: the host only uses it when all CTAs have tiles)
  const int nseg = seg1 - seg0;
  const int n_iters = MULTI ? g.n_steps * nseg : nseg;
  // everything above is private set-up; from here on the kernel reads what its predecessor wrote
  pdl_trigger();
  pdl_wait();

  // Every segment has three CTA-wide barriers, executed by both roles:
  //   S1 parameters staged   S2 all tiles of the segment done   S3 read-out done
  if (is_ctrl) {
    // =====================  control warpgroup (warps 12..15; warp 15 only keeps the barriers) ==========
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(TF32_CTRL_REGS));
    uint32_t c_issued = 0;  // tiles of this warpgroup whose MMAs have been issued (mbarrier phases follow it)
    bool alive = true;
    // a multi-step launch walks its segments once per step: ONE loop over (step, segment) pairs
    for (int it = 0; it < n_iters; ++it) {
      const int sg = MULTI ? seg0 + it % nseg : seg0 + it;
      const int4 seg = g.segs[sg];
      const int win = seg.x, t0 = seg.y, nt = seg.z - seg.y;
      const int grow0 = (g.data_window0 + win) * rows_pad;
      __syncthreads();  // S1
      if (wg < NWG) {
        // Order per tile n: forward(n+1) as soon as its rows are in tensor memory (the warpgroup stages
        // them at the START of tile n), backward(n) when E(n) is in shared memory, then — once those
        // MMAs have completed — the TMA refill of the row stage they read.
        const int cnt = (nt - wg + NWG - 1) / NWG;
        const uint32_t a_t = tmem + G::A_COL0 + wg * G::A_STRIDE;
        const uint32_t z_t0 = tmem + G::Z_COL0 + wg * 2 * G::Z_STRIDE;
        const uint32_t g_t = tmem_g + wg * G::G_STRIDE;
        // descriptors of K block 0 / row stage 0; the others differ only in the start address
        const uint64_t wdesc0 = umma_desc_k128(w0s_addr);
        const uint64_t adesc0 = umma_desc_k128(smem_u32(es + wg * G::ES_WG_BYTES));
        const uint64_t bdesc0 = umma_desc_mn32(smem_u32(xb + wg * NST * G::TILE_BYTES), G::TILE_BYTES);
        uint32_t stage = c_issued % NST;  // row stage of tile n, kept as a running counter
        auto issue_fwd = [&](uint32_t n) {
          named_sync(BAR_ROWS0 + wg, 160);
          if (lane == 0) {
            tc_fence_after();
            const uint32_t z_t = z_t0 + (n & 1) * G::Z_STRIDE;
            if (!ABL(32))
#pragma unroll
            for (int kb = 0; kb < 3; ++kb)
              tc_mma_tf32_ts(z_t, a_t + kb * 8, umma_desc_advance(wdesc0, kb * 2), IDESC_FWD, kb > 0);
            tc_commit(&bar_fwd[wg]);
          }
          __syncwarp();
        };
        if (cnt > 0) issue_fwd(c_issued);
        for (int i = 0; i < cnt; ++i) {
          const uint32_t n = c_issued + i;
          if (i + 1 < cnt) issue_fwd(n + 1);
          named_sync(BAR_E0 + wg, 160);
          if (lane == 0) {
            tc_fence_after();
            const uint64_t bd = umma_desc_advance(bdesc0, stage * (G::TILE_BYTES >> 4));
            if (!ABL(1))
#pragma unroll
            for (int kb = 0; kb < TF32_TILE / 8; ++kb)
              tc_mma_tf32_ss(g_t,
                             umma_desc_advance(adesc0, (kb >> 2) * (G::ES_ATOM_BYTES >> 4) + (kb & 3) * 2),
                             umma_desc_advance(bd, kb * 64), IDESC_BWD, (i == 0 && kb == 0) ? 0u : 1u);
            tc_commit(&bar_bwd[wg]);
            if (i + NST < cnt && !ABL(256)) {
              ok = ok && mbar_wait(&bar_bwd[wg], n & 1, g.status, 213);
              if (ok) {
                mbar_expect_tx(&bar_tma[wg][stage], G::TILE_BYTES);
                tma_load_2d(xb + (wg * NST + stage) * G::TILE_BYTES, &tmap_mn, 0,
                            grow0 + (t0 + wg + (i + NST) * NWG) * TF32_TILE, &bar_tma[wg][stage]);
              }
            }
          }
          stage = stage + 1 == NST ? 0 : stage + 1;
          __syncwarp();
        }
        c_issued += cnt;
      }
      __syncthreads();  // S2
      __syncthreads();  // S3
      if (MULTI && (it + 1) % nseg == 0) {
        // the two grid-wide barriers of a step: this role only keeps the CTA barriers inside them
        grid_barrier(g.grid_bar, 0u, false, alive, g.status, 0);
        if (it + 1 < n_iters) grid_barrier(g.grid_bar, 0u, false, alive, g.status, 0);
      }
    }
  } else {
    // =====================  compute warpgroups: one row per thread  =====================================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(TF32_COMPUTE_REGS));
    uint32_t n_done = 0;  // tiles this warpgroup has finished (mbarrier phases follow it)
    uint32_t st_stage = 0, st_phase = 0;  // row stage and mbarrier phase of the next tile to be staged
    const uint32_t lane_off = (uint32_t)(wwarp * 32) << 16;
    const uint32_t a_t = tmem + G::A_COL0 + wg * G::A_STRIDE + lane_off;
    const uint32_t z_t0 = tmem + G::Z_COL0 + wg * 2 * G::Z_STRIDE + lane_off;
    // E element (hidden j, row r): atom r/32 (= this warp), line j, 16-byte chunk (r%32)/4 ^ (j%8)
    uint32_t e_ptr[8];
#pragma unroll
    for (int c = 0; c < 8; ++c)
      e_ptr[c] = smem_u32(es + wg * G::ES_WG_BYTES + wwarp * G::ES_ATOM_BYTES) +
                 ((uint32_t)(((lane >> 2) ^ c) << 4)) + ((lane & 3) << 2);
    // rows r and r+4 of a staged tile keep their 32-byte chunks in the same banks: the upper four of
    // every eight rows read the two halves of a chunk in the opposite order
    const bool swap_halves = (wtid & 4) != 0;
    bool alive = true;

    for (int it = 0; it < n_iters; ++it) {
      const int sg = MULTI ? seg0 + it % nseg : seg0 + it;
      const int step = MULTI ? it / nseg : 0;
      const int4 seg = g.segs[sg];
      const int win = seg.x, t0 = seg.y, t1 = seg.z, slot = seg.w;
      const int nt = t1 - t0;
      const int grow0 = (g.data_window0 + win) * rows_pad;  // first row of this window in the tensor map
      const int my_nt = (nt - wg + NWG - 1) / NWG;          // tiles t0 + wg, t0 + wg + NWG, ...

      // ---- segment prologue: start the first row tiles, fused leapfrog update, stage W0a ----
      if (wtid == 0 && !ABL(256)) {
        for (int i = 0; i < NST && i < my_nt; ++i) {
          const uint32_t n = n_done + i;
          mbar_expect_tx(&bar_tma[wg][n % NST], G::TILE_BYTES);
          tma_load_2d(xb + (wg * NST + n % NST) * G::TILE_BYTES, &tmap_mn, 0,
                      grow0 + (t0 + wg + i * NWG) * TF32_TILE, &bar_tma[wg][n % NST]);
        }
      }
      // element (n = hidden unit, k) of the K-major B operand at n*128 + ((k/4) ^ (n%8))*16 + (k%4)*4
      const StepIo io = MULTI ? step_io(g, step) : step_io(g);
      for (int p = tid; p < G::P; p += NCOMPUTE) {
        const float w = leapfrog_param(g, io, win, p, slot == 0);
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
      __syncthreads();  // S1

      // output-layer weights live in registers for the whole segment
      float w1r[H];
#pragma unroll
      for (int j = 0; j < H; j += 4) {
        const float4 v = *reinterpret_cast<const float4*>(w1s + j);
        w1r[j] = v.x; w1r[j + 1] = v.y; w1r[j + 2] = v.z; w1r[j + 3] = v.w;
      }
      const float b1 = b1s;
      uint64_t dw1p[H / 2];  // dW1 accumulators, two hidden units per register pair
#pragma unroll
      for (int j = 0; j < H / 2; ++j) dw1p[j] = 0ull;
      float db1 = 0.f;
      double llacc = 0.0;

      // hands this thread's row of the landed tile to the tensor core (forward A operand); returns y
      auto stage_row = [&]() -> float {
        const uint32_t stage = st_stage, phase = st_phase;  // of the tile being staged
        st_stage = st_stage + 1 == NST ? 0 : st_stage + 1;
        st_phase ^= (st_stage == 0) ? 1u : 0u;
        if (!ABL(256)) ok = ok && mbar_wait(&bar_tma[wg][stage], phase, g.status, 201);
        // 32-byte chunk j of a row sits at position j ^ (row % 4)
        const unsigned char* xrow = xb + (wg * NST + stage) * G::TILE_BYTES + wtid * 128;
        float4 xr[6];
#pragma unroll
        for (int j = 0; j < 3; ++j) {
          const unsigned char* cp = xrow + ((j ^ (wtid & 3)) << 5);
          const float4 first = *reinterpret_cast<const float4*>(cp + (swap_halves ? 16 : 0));
          const float4 second = *reinterpret_cast<const float4*>(cp + (swap_halves ? 0 : 16));
          xr[2 * j].x = swap_halves ? second.x : first.x;
          xr[2 * j].y = swap_halves ? second.y : first.y;
          xr[2 * j].z = swap_halves ? second.z : first.z;
          xr[2 * j].w = swap_halves ? second.w : first.w;
          xr[2 * j + 1].x = swap_halves ? first.x : second.x;
          xr[2 * j + 1].y = swap_halves ? first.y : second.y;
          xr[2 * j + 1].z = swap_halves ? first.z : second.z;
          xr[2 * j + 1].w = swap_halves ? first.w : second.w;
        }
        if (!ABL(64))
#pragma unroll
        for (int j = 0; j < 3; ++j) tc_st8(a_t + j * 8, xr[2 * j], xr[2 * j + 1]);
        return xr[5].w;
      };
      // ... and tells the control warp once the stores have landed
      auto publish_row = [&]() {
        tc_wait_st();
        tc_fence_before();
        named_arrive(BAR_ROWS0 + wg, 160);
      };

      PROF_DECL
      float y = 0.f;
      if (my_nt > 0) {
        y = stage_row();
        publish_row();
      }
      PROF_MARK(9)
      for (int i = 0; i < my_nt; ++i) {
        const uint32_t n = n_done + i;
        const int t = t0 + wg + i * NWG;
        ok = ok && mbar_wait(&bar_fwd[wg], n & 1, g.status, 202);
        tc_fence_after();
        PROF_MARK(0)
        // forward(n) is done with the A operand: the next tile's rows go in now, so that forward(n+1)
        // (into the other accumulator buffer) has this whole tile's epilogue to complete
        float y_next = 0.f;
        if (i + 1 < my_nt) y_next = stage_row();
        PROF_MARK(1)
        const uint32_t z_t = z_t0 + (n & 1) * G::Z_STRIDE;
        float z[H];
        if (!ABL(128)) {
#pragma unroll
          for (int c = 0; c < H; c += 8) tc_ld8(z_t + c, z + c);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int c = 0; c < H; ++c) z[c] = 0.01f * c;
        }
        PROF_MARK(2)
        if (i + 1 < my_nt) publish_row();
        PROF_MARK(3)
        if (dbg && !ABL(512) && blockIdx.x == 0 && sg == seg0 && wg == 0 && i == 0) {
#pragma unroll
          for (int j = 0; j < H; ++j) dbg[wtid * 64 + j] = z[j];
          dbg[wtid * 64 + 63] = y;
        }
        float pred = b1;
        if (!ABL(8)) {
          float pred1 = 0.f;
#pragma unroll
          for (int j = 0; j < H; j += 2) {
            z[j] = tanh_fast(z[j]);
            z[j + 1] = tanh_fast(z[j + 1]);
            pred = fmaf(w1r[j], z[j], pred);
            pred1 = fmaf(w1r[j + 1], z[j + 1], pred1);
          }
          pred += pred1;
        }
        PROF_MARK(4)
        const int grow = t * TF32_TILE + wtid;
        const bool valid = grow < g.n_rows;
        float loss, dy;
        lik_terms(g.lik, y, pred, loss, dy);
        if (!valid) { loss = 0.f; dy = 0.f; }
        llacc += (double)loss;
        if (g.row_loss && valid) g.row_loss[(long long)win * g.row_loss_stride + grow] = loss;
        db1 += dy;
        if (!ABL(16)) {
          const uint64_t dy2 = pack2(dy, dy), one2 = pack2(1.f, 1.f);
#pragma unroll
          for (int j = 0; j < H; j += 2) {
            const uint64_t h2 = pack2(z[j], z[j + 1]);
            const uint64_t nh2 = pack2(-z[j], -z[j + 1]);
            dw1p[j >> 1] = fma2(dy2, h2, dw1p[j >> 1]);
            const uint64_t e2 = mul2(fma2(nh2, h2, one2), dy2);  // E; the W1 factor is applied at read-out
            unpack2(e2, z[j], z[j + 1]);
          }
        }
        PROF_MARK(5)
        // the previous tile's backward MMAs must be done with E before it is overwritten
        if (n > 0) ok = ok && mbar_wait(&bar_bwd[wg], (n - 1) & 1, g.status, 203);
        PROF_MARK(6)
        if (!ABL(4)) store_e_all(e_ptr, z, std::make_integer_sequence<int, H>{});
        fence_proxy_async_smem();
        named_arrive(BAR_E0 + wg, 160);
        y = y_next;
        PROF_MARK(7)
      }
      PROF_FLUSH
      n_done += my_nt;

      // ---- this warp's share of dW1 / db1 / log-lik ----
      if (n_done > 0) ok = ok && mbar_wait(&bar_bwd[wg], (n_done - 1) & 1, g.status, 204);
      tc_fence_after();
      {
        // column sums over the warp's 32 rows: a halving butterfly leaves hidden unit `lane` in lane `lane`
        // (units 0..31); the last H - 32 units take three halving steps and two plain ones
        float v[H];
#pragma unroll
        for (int j = 0; j < H; j += 2) unpack2(dw1p[j >> 1], v[j], v[j + 1]);
        const float s_lo = warp_column_sums(v, lane);
        constexpr int REST = H - 32;  // 8
        float* u = v + 32;
#pragma unroll
        for (int off = REST / 2; off > 0; off >>= 1) {
          const bool up = (lane & off) != 0;
#pragma unroll
          for (int i = 0; i < off; ++i) {
            const float send = up ? u[i] : u[i + off];
            const float keep = up ? u[i + off] : u[i];
            u[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
          }
        }
        float s_hi = u[0];
#pragma unroll
        for (int off = REST; off < 32; off <<= 1) s_hi += __shfl_xor_sync(0xffffffffu, s_hi, off);
        red_w1[warp][lane] = s_lo;
        if (lane < REST) red_w1[warp][32 + lane] = s_hi;
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
      __syncthreads();  // S2

      // ---- segment read-out: one partial gradient vector for (window, slot) ----
      float* po = (MULTI ? ((step & 1) ? g.partial_buf[1] : g.partial_buf[0]) : g.partial_out) + ((size_t)win * g.slices_out + slot) * g.Pp;
      if (warp < 4) {
        tc_fence_after();
        float gacc[NB];
        const uint32_t trow = tmem_g + ((uint32_t)(warp * 32) << 16);
#pragma unroll
        for (int c = 0; c < NB; c += 8) tc_ld8(trow + c, gacc + c);
        tc_wait_ld();
        // the other warpgroups' accumulators (those that had tiles in this segment)
#pragma unroll
        for (int w = 1; w < NWG; ++w) {
          if (w < nt) {
            float g2[NB];
#pragma unroll
            for (int c = 0; c < NB; c += 8) tc_ld8(trow + w * G::G_STRIDE + c, g2 + c);
            tc_wait_ld();
#pragma unroll
            for (int c = 0; c < NB; ++c) gacc[c] += g2[c];
          }
        }
        if (dbg && !ABL(512) && blockIdx.x == 0 && sg == seg0) {
#pragma unroll
          for (int c = 0; c < NB; ++c) dbg[8192 + tid * 32 + c] = gacc[c];
        }
        // M = 64: accumulator row i lives in lane 32*(i/16) + i%16
        const int hidx = lane < 16 ? warp * 16 + lane : -1;
        if (hidx >= 0 && hidx < H) {
          const float w1 = w1s[hidx];
#pragma unroll
          for (int k = 0; k < D; ++k) po[k * H + hidx] = w1 * gacc[k];
          po[D * H + hidx] = w1 * gacc[COL_ONE];
        }
        tc_fence_before();
      } else if (warp == 4) {
        for (int j = lane; j < H; j += 32) {
          float s = red_w1[0][j];
#pragma unroll
          for (int w = 1; w < NWG * 4; ++w) s += red_w1[w][j];
          po[D * H + H + j] = s;
        }
        if (lane == 0) {
          float s = 0.f;
          double l = 0.0;
          for (int w = 0; w < NWG * 4; ++w) { s += red_db1[w]; l += red_ll[w]; }
          po[D * H + 2 * H] = s;
          (MULTI ? ((step & 1) ? g.ll_buf[1] : g.ll_buf[0]) : g.ll_out)[(size_t)win * g.slices_out + slot] = l;
        }
      }
      __syncthreads();  // S3: read-out done before the next segment restages W0a / reuses the scratch
      if (MULTI && (it + 1) % nseg == 0) {
        // ---- all partial vectors of this step are written: sum them, a few parameters per CTA ----
        const unsigned int nb = gridDim.x;
        grid_barrier(g.grid_bar, (2u * step + 1u) * nb, tid == 0, alive, g.status, 401);
        sum_partials_slice(g, (step & 1) ? g.partial_buf[1] : g.partial_buf[0],
                           (step & 1) ? g.ll_buf[1] : g.ll_buf[0], tid);
        if (it + 1 < n_iters) grid_barrier(g.grid_bar, (2u * step + 2u) * nb, tid == 0, alive, g.status, 402);
      }
    }
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
int tf32_supported(int H) { return H == 40 || H == 128; }

template <int H>
static cudaError_t launch_tf32_t(const void* tmap_mn, const GradParams& g, int ctas, float* dbg,
                                 cudaStream_t st) {
  using G = Tf32Geom<H>;
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(grad_tf32_kernel<H, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)G::SMEM);
    if (e != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  return launch_chain_kernel(grad_tf32_kernel<H, false>, dim3(ctas), dim3(TF32_THREADS), G::SMEM, st,
                             *reinterpret_cast<const CUtensorMap*>(tmap_mn), g, dbg);
}

// Several leapfrog steps of one window in one COOPERATIVE launch (every CTA resident: the grid barrier
// inside relies on it).  Returns cudaErrorCooperativeLaunchTooLarge-like errors to the caller, which then
// falls back to one launch per step.
int tf32_multistep_max_ctas(int H) {
  if (H != 40) return 0;
  using G = Tf32Geom<40>;
  int dev = 0, coop = 0, sms = 0, per_sm = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (!coop) return 0;
  if (cudaFuncSetAttribute(grad_tf32_kernel<40, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)G::SMEM) != cudaSuccess)
    return 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, grad_tf32_kernel<40, true>, TF32_THREADS,
                                                    G::SMEM) != cudaSuccess)
    return 0;
  return per_sm * sms;
}

cudaError_t launch_grad_tf32_multistep(int H, const void* tmap_mn, const GradParams& g, int ctas,
                                       cudaStream_t st) {
  if (H != 40) return cudaErrorInvalidValue;
  using G = Tf32Geom<40>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas);
  cfg.blockDim = dim3(TF32_THREADS);
  cfg.dynamicSmemBytes = G::SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, grad_tf32_kernel<40, true>, *reinterpret_cast<const CUtensorMap*>(tmap_mn), g,
                            (float*)nullptr);
}

cudaError_t launch_grad_tf32(int H, const void* tmap_mn, const GradParams& g, int ctas, float* dbg,
                             cudaStream_t st) {
  if (H == 40) return launch_tf32_t<40>(tmap_mn, g, ctas, dbg, st);
  if (H == 128) return launch_grad_tf32_wide(tmap_mn, g, ctas, st);  // grad_tf32_wide.cu
  return cudaErrorInvalidValue;
}

}  // namespace mcmc_b200

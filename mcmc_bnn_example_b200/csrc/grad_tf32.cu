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
// warpgroups (128 threads = the 128 rows of a tile each) plus a control warpgroup:
// one warp per compute warpgroup, whose lane 0 issues that warpgroup's MMAs and
// TMA refills.  A CTA owns a contiguous range of the launch's (window, tile)
// list, cut into per-window segments by the host; a warpgroup's tiles of a
// segment use its three row stages round-robin from stage 0, and the tile loop
// is unrolled by three so that the stage is a compile-time constant.
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
//   backward  Gt[feature x hidden] += Xa^T[feature x rows] . E[rows x hidden]
//             E = (1 - h^2) * dL/dpred (stored negated, see below), written
//             row-per-thread into shared memory as the K-major B operand (one
//             128-byte line per hidden unit and 32 rows); the TMA-staged row
//             tile is the MN-major A operand.  MN-major operands of a 32-bit
//             type exist in one layout only, the 128-byte swizzle of 32-byte
//             chunks, so the tile is staged in that layout (and that is why the
//             forward takes its A operand from tensor memory instead of a
//             second copy of the tile).
//             The cost of a tcgen05.mma of this size is its issue, not its
//             arithmetic, and K is fixed at 8 rows per instruction.  One
//             instruction therefore covers TWO 32-row groups at once: M = 64 =
//             the 32-float rows of group a and of group a+1 (the second
//             32-float atom of the MN-major operand is simply the tile 32 rows
//             further down), N = 80 = the 40 lines of E for group a followed by
//             the 40 lines for group a+1.  The two diagonal blocks of the
//             64 x 80 result are the wanted sums, the off-diagonal blocks
//             (group a's rows against group a+1's E) are never read: 8
//             instructions per 128-row tile instead of 16, and no line of E is
//             fetched that is not used.  Gt stays in tensor memory for a whole
//             segment and is read once: dW0[k][j] = W1[j] * Gt[k][j],
//             db0[j] = W1[j] * Gt[22][j] — W1[j] is a per-column constant,
//             applied after the reduction.
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
#include <type_traits>
#include <utility>
#include "common.cuh"
#include "chain.cuh"
#include "tc05.cuh"

namespace mcmc_b200 {

constexpr int TF32_NWG = 3;                            // compute warpgroups
constexpr int TF32_THREADS = TF32_NWG * 128 + 128;      // + a control warpgroup (one warp per compute warpgroup, one idle)
// registers: 512 threads start with 128 each; the control warpgroup hands most of its share to the
// compute warpgroups (3 * 128 * 160 + 128 * 32 = 65536)
constexpr int TF32_COMPUTE_REGS = 160;
constexpr int TF32_CTRL_REGS = 32;
constexpr int TF32_NST = 3;                            // TMA stages per warpgroup

template <int H>
struct Tf32Geom {
  static constexpr int D = 22;
  static constexpr int NF = (H + 15) / 16 * 16;        // forward N (M = 128 needs N % 16 == 0)
  static constexpr int GM = 64;                        // backward M: two 32-float atoms of the row tile
  static constexpr int GN = 2 * H;                     // backward N: the hidden units of two 32-row groups
  static constexpr int TILE_BYTES = TF32_TILE * 128;   // 128 rows x 32 floats (24 real + 8 zero fill)
  static constexpr int GROUP_BYTES = 32 * 128;         // 32 rows of the staged tile
  static constexpr int XB_BYTES = TF32_NWG * TF32_NST * TILE_BYTES;
  // E operand, K-major: 4 atoms of 32 rows (K); in an atom hidden unit j is a 128-byte line
  static constexpr int ES_ATOM_BYTES = H * 128;
  static constexpr int ES_WG_BYTES = 4 * ES_ATOM_BYTES;
  static constexpr int ES_BYTES = TF32_NWG * ES_WG_BYTES;
  static constexpr int W0S_BYTES = NF * 128;
  static constexpr int W1_BYTES = (H + 3) / 4 * 16;
  static constexpr int P = D * H + 2 * H + 1;
  static constexpr size_t SMEM = 1024 + XB_BYTES + ES_BYTES + W0S_BYTES + W1_BYTES;
  // tensor-memory columns per warpgroup: forward A operand, forward accumulator (one buffer: forward(n+1)
  // is issued only after Z(n) has been read into registers), backward accumulator
  static constexpr int A_COL0 = 0, A_STRIDE = 24;
  static constexpr int Z_COL0 = TF32_NWG * A_STRIDE, Z_STRIDE = NF;
  static constexpr int G_COL0 = Z_COL0 + TF32_NWG * Z_STRIDE, G_STRIDE = GN;
  static constexpr int TMEM_COLS = 512;
  static_assert(H % 8 == 0 && H <= 64, "hidden width must be a multiple of 8, at most 64");
  static_assert(G_COL0 + TF32_NWG * G_STRIDE <= TMEM_COLS, "tensor memory budget");
  static_assert(H > 32 && ((H - 32) & (H - 33)) == 0, "the dW1 butterfly handles 32 + a power of two units");
  static_assert(ES_ATOM_BYTES % 1024 == 0, "E atoms must keep the 1024-byte swizzle alignment");
};

// E of one pair of hidden units (2J, 2J+1) of this thread's row, stored with the line offsets as immediates
template <int J>
__device__ __forceinline__ void store_e_pair(const uint32_t* e_ptr, const uint64_t* hp, uint64_t dy2,
                                             uint64_t ndy2, uint64_t* dw1p) {
  const uint64_t h2 = hp[J];
  const uint64_t t2 = mul2(dy2, h2);
  dw1p[J] = fma2(dy2, h2, dw1p[J]);
  float e0, e1;
  unpack2(fma2(t2, h2, ndy2), e0, e1);
  asm volatile("st.shared.f32 [%0+%2], %1;" ::"r"(e_ptr[(2 * J) & 7]), "f"(e0), "n"(2 * J * 128) : "memory");
  asm volatile("st.shared.f32 [%0+%2], %1;" ::"r"(e_ptr[(2 * J + 1) & 7]), "f"(e1), "n"((2 * J + 1) * 128) : "memory");
}
template <int... Js>
__device__ __forceinline__ void store_e_pairs(const uint32_t* e_ptr, const uint64_t* hp, uint64_t dy2,
                                              uint64_t ndy2, uint64_t* dw1p, std::integer_sequence<int, Js...>) {
  (store_e_pair<Js>(e_ptr, hp, dy2, ndy2, dw1p), ...);
}

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
grad_tf32_kernel(const __grid_constant__ CUtensorMap tmap_mn, const GradParams g) {
  using G = Tf32Geom<H>;
  constexpr int D = G::D, NF = G::NF, NWG = TF32_NWG, NST = TF32_NST;
  constexpr uint32_t IDESC_FWD = umma_idesc_tf32(128, NF, 0, 0);
  constexpr uint32_t IDESC_BWD = umma_idesc_tf32(G::GM, G::GN, 1, 0);  // A = Xa^T MN-major, B = E K-major
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
  __shared__ __align__(16) float red_g[KP][H];  // the second row group's half of Gt at read-out

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const bool is_ctrl = warp >= NWG * 4;
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
    // the warpgroup this warp issues for, in a form the compiler can see is the same in every lane
    const int wg = __shfl_sync(0xffffffffu, warp - NWG * 4, 0);
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
        // them at the START of tile n, after it has read Z(n)), backward(n) when E(n) is in shared
        // memory, then — once those MMAs have completed — the TMA refill of the row stage they read.
        const int cnt = (nt - wg + NWG - 1) / NWG;
        const uint32_t a_t = tmem + G::A_COL0 + wg * G::A_STRIDE;
        const uint32_t z_t = tmem + G::Z_COL0 + wg * G::Z_STRIDE;
        const uint32_t g_t = tmem_g + wg * G::G_STRIDE;
        // descriptors of K block 0 / row stage 0; the others differ only in the start address
        const uint64_t wdesc0 = umma_desc_k128(w0s_addr);
        const uint64_t edesc0 = umma_desc_k128(smem_u32(es + wg * G::ES_WG_BYTES));
        const uint64_t xdesc0 = umma_desc_mn32(smem_u32(xb + wg * NST * G::TILE_BYTES), G::GROUP_BYTES);
        uint32_t stage = 0;  // row stage of tile i of the segment: i % NST, kept as a running counter
        auto issue_fwd = [&]() {
          named_sync(BAR_ROWS0 + wg, 160);
          if (lane == 0) {
            tc_fence_after();
#pragma unroll
            for (int kb = 0; kb < 3; ++kb)
              tc_mma_tf32_ts(z_t, a_t + kb * 8, umma_desc_advance(wdesc0, kb * 2), IDESC_FWD, kb > 0);
            tc_commit(&bar_fwd[wg]);
          }
          __syncwarp();
        };
        if (cnt > 0) issue_fwd();
        for (int i = 0; i < cnt; ++i) {
          const uint32_t n = c_issued + i;
          if (i + 1 < cnt) issue_fwd();
          named_sync(BAR_E0 + wg, 160);
          if (lane == 0) {
            tc_fence_after();
            const uint64_t xd = umma_desc_advance(xdesc0, stage * (G::TILE_BYTES >> 4));
            // pair p = row groups 2p, 2p+1 (rows 64p .. 64p+63 of the tile); K block kb = 8 rows of each group
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const int p = q >> 2, kb = q & 3;
              tc_mma_tf32_ss(g_t, umma_desc_advance(xd, p * (2 * G::GROUP_BYTES >> 4) + kb * 64),
                             umma_desc_advance(edesc0, p * (2 * G::ES_ATOM_BYTES >> 4) + kb * 2), IDESC_BWD,
                             (i == 0 && q == 0) ? 0u : 1u);
            }
            tc_commit(&bar_bwd[wg]);
            if (i + NST < cnt) {
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
    // (through a shuffle: visibly the same in every lane, so barrier ids and mbarrier addresses derived from
    // it stay in uniform registers instead of being recomputed from the thread index at every use)
    const int wg = __shfl_sync(0xffffffffu, warp >> 2, 0);
    uint32_t n_done = 0;  // tiles this warpgroup has finished (mbarrier phases follow it)
    // Tile i of a segment (of this warpgroup) uses row stage i % NST, so that the stage is a compile-time
    // constant in the tile loop (unrolled by NST).  use_s[s] = uses of stage s in earlier segments: the k-th
    // use of a stage (k from 0) completes the phase of parity k & 1 of its barrier.
    uint32_t use_s[NST] = {0u, 0u, 0u};
    static_assert(NST == 3, "the tile loop is unrolled for three row stages");
    const uint32_t lane_off = (uint32_t)(wwarp * 32) << 16;
    const uint32_t a_t = pin(tmem + G::A_COL0 + wg * G::A_STRIDE + lane_off);
    const uint32_t z_t = pin(tmem + G::Z_COL0 + wg * G::Z_STRIDE + lane_off);
    // E element (hidden j, row r): atom r/32 (= this warp), line j, 16-byte chunk (r%32)/4 ^ (j%8)
    uint32_t e_ptr[8];
#pragma unroll
    for (int c = 0; c < 8; ++c)
      e_ptr[c] = pin(smem_u32(es + wg * G::ES_WG_BYTES + wwarp * G::ES_ATOM_BYTES) +
                     ((uint32_t)(((lane >> 2) ^ c) << 4)) + ((lane & 3) << 2));
    // This thread's row in a staged tile: 32-byte chunk j of row r sits at position j ^ (r % 4).  Rows r
    // and r+4 keep their chunks in the same banks, so the upper four of every eight rows read the two
    // 16-byte halves of a chunk in the opposite order (address ^ 16) and swap them back in registers.
    const bool swap_halves = pin((uint32_t)(wtid & 4)) != 0;
    const uint32_t xb_wg = smem_u32(xb + wg * NST * G::TILE_BYTES);
    uint32_t x_off[3];
#pragma unroll
    for (int j = 0; j < 3; ++j)
      x_off[j] = pin(xb_wg + (uint32_t)(wtid * 128 + ((j ^ (wtid & 3)) << 5) + ((wtid & 4) ? 16 : 0)));
    const int row_in_tile = (int)pin((uint32_t)wtid);
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
      if (wtid == 0) {
        for (int i = 0; i < NST && i < my_nt; ++i) {
          const uint32_t n = n_done + i;
          mbar_expect_tx(&bar_tma[wg][i], G::TILE_BYTES);
          tma_load_2d(xb + (wg * NST + i) * G::TILE_BYTES, &tmap_mn, 0,
                      grow0 + (t0 + wg + i * NWG) * TF32_TILE, &bar_tma[wg][i]);
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

      // The output-layer weights are the same for every thread: each is read once per segment and passed
      // through a shuffle, which tells the compiler that the value is warp-uniform, so that it can keep the 40
      // of them in uniform registers (63 per warp) next to Z (40 registers) and the dW1 accumulators (40).  Read
      // from shared memory per tile instead they cost ten 16-byte broadcast loads per row, 160 wavefronts per
      // tile on the busiest unit of the SM; kept in ordinary registers they cost spills.
      float w1u[H];
#pragma unroll
      for (int j = 0; j < H; ++j) w1u[j] = __shfl_sync(0xffffffffu, w1s[j], 0);
      const float b1 = b1s;
      uint64_t dw1p[H / 2];  // dW1 accumulators, two hidden units per register pair
#pragma unroll
      for (int j = 0; j < H / 2; ++j) dw1p[j] = 0ull;
      float db1 = 0.f;
      double llacc = 0.0;

      // One 16-byte half-pair of this thread's row of a landed tile: chunk j (features 8j .. 8j+7) goes into
      // the forward A operand in tensor memory; chunk 2 also carries y.
      auto stage_load = [&](uint32_t sb, int j, float4& p, float4& q) {
        const uint32_t a = sb + x_off[j];
        p = lds128(a);
        q = lds128(a ^ 16u);
      };
      auto stage_store = [&](int j, const float4& p, const float4& q) -> float {
        float4 lo, hi;
        lo.x = swap_halves ? q.x : p.x; lo.y = swap_halves ? q.y : p.y;
        lo.z = swap_halves ? q.z : p.z; lo.w = swap_halves ? q.w : p.w;
        hi.x = swap_halves ? p.x : q.x; hi.y = swap_halves ? p.y : q.y;
        hi.z = swap_halves ? p.z : q.z; hi.w = swap_halves ? p.w : q.w;
        tc_st8(a_t + j * 8, lo, hi);
        return hi.w;
      };
      // tells the control warp that this thread's row is in tensor memory
      auto publish_row = [&]() {
        tc_wait_st();
        tc_fence_before();
        named_arrive(BAR_ROWS0 + wg, 160);
      };
      float y = 0.f;
      if (my_nt > 0) {  // the segment's first tile: nothing to overlap the staging with
        mbar_wait_q(&bar_tma[wg][0], use_s[0] & 1, g.status, 201, ok);
#pragma unroll
        for (int j = 0; j < 3; ++j) {
          float4 p, q;
          stage_load(0u, j, p, q);
          y = stage_store(j, p, q);
        }
        publish_row();
      }
      // One tile.  HAS_NEXT: the warpgroup has another tile in this segment, whose rows are staged while
      // this tile's activations are computed (the last tile is the same code without that part, so that the
      // body has no data-dependent branch the instruction scheduler would have to stop at).
      // NS = row stage of the NEXT tile ((i + 1) % NST), kq = (i + 1) / NST: its use of that stage in this segment
      auto tile_body = [&](auto has_next_c, auto ns_c, int i, uint32_t kq) {
        constexpr bool HAS_NEXT = decltype(has_next_c)::value;
        constexpr uint32_t NS = decltype(ns_c)::value;
        const uint32_t n = n_done + i;
        const int t = t0 + wg + i * NWG;
        // forward(n) done (Z ready, A operand free) and, if there is one, the next tile's rows landed:
        // both barriers are polled before either answer is used, so their latencies overlap
        const uint32_t phase = (use_s[NS] + kq) & 1;
        const bool f_done = mbar_try_wait(&bar_fwd[wg], n & 1);
        const bool t_done = HAS_NEXT ? mbar_try_wait(&bar_tma[wg][NS], phase) : true;
        if (!f_done) ok = mbar_wait_slow(&bar_fwd[wg], n & 1, g.status, 202, ok);
        if (HAS_NEXT && !t_done) ok = mbar_wait_slow(&bar_tma[wg][NS], phase, g.status, 201, ok);
        tc_fence_after();
        // Z(n) starts moving into registers.  Once it is there forward(n+1) may overwrite the accumulator;
        // the control warp is told after the tanh pass, when the next tile's rows are in tensor memory too:
        // forward(n+1) still has the rest of this tile's epilogue to complete.
        float z[H];
#pragma unroll
        for (int c = 0; c < H; c += 8) tc_ld8(z_t + c, z + c);
        constexpr uint32_t sb = NS * G::TILE_BYTES;
        float4 sp, sq;
        if (HAS_NEXT) stage_load(sb, 0, sp, sq);
        tc_wait_ld();
        // hidden activations, kept as register pairs from here on (packed f32x2 arithmetic).  The tanh pass
        // is bound by the MUFU pipe (one warp instruction per 8 cycles): the staging of the next tile's row
        // (3 x {two loads, eight selects, one tensor-memory store}) is spread over it.
        uint64_t hp[H / 2];
        uint64_t pred2 = pack2(b1, 0.f);
        float y_next = 0.f;
#pragma unroll
        for (int j = 0; j < H; j += 4) {
          const float4 wv = make_float4(w1u[j], w1u[j + 1], w1u[j + 2], w1u[j + 3]);
          hp[j >> 1] = pack2(tanh_fast(z[j]), tanh_fast(z[j + 1]));
          hp[(j >> 1) + 1] = pack2(tanh_fast(z[j + 2]), tanh_fast(z[j + 3]));
          pred2 = fma2(pack2(wv.x, wv.y), hp[j >> 1], pred2);
          pred2 = fma2(pack2(wv.z, wv.w), hp[(j >> 1) + 1], pred2);
          if (HAS_NEXT) {
            constexpr int STEP = 12;  // hidden units between two staging steps
            if (j % STEP == 4) {
              y_next = stage_store(j / STEP, sp, sq);
              if (j / STEP < 2) stage_load(sb, j / STEP + 1, sp, sq);
            }
          }
        }
        float pred, pred1;
        unpack2(pred2, pred, pred1);
        pred += pred1;
        if (HAS_NEXT) publish_row();
        // the previous tile's backward MMAs must be done with E before it is overwritten (they were
        // issued a whole tile ago): polled here, used after the loss terms
        const bool b_done = n > 0 ? mbar_try_wait(&bar_bwd[wg], (n - 1) & 1) : true;
        const int grow = t * TF32_TILE + row_in_tile;
        const bool valid = grow < g.n_rows;
        float loss, dy;
        lik_terms(g.lik, y, pred, loss, dy);
        if (!valid) { loss = 0.f; dy = 0.f; }
        llacc += (double)loss;
        store_row_loss(g.row_loss, (long long)win * g.row_loss_stride + grow, loss, valid);
        db1 += dy;
        if (!b_done) ok = mbar_wait_slow(&bar_bwd[wg], (n - 1) & 1, g.status, 203, ok);
        {
          // with t = dy*h:  dW1 += t,  -E = t*h - dy  (E = (1 - h^2) dy; the sign and the W1 factor are
          // applied once per segment at read-out): three packed operations per pair of hidden units, each
          // pair stored as soon as it is ready so that the stores spread over the arithmetic
          const uint64_t dy2 = pack2(dy, dy), ndy2 = pack2(-dy, -dy);
          store_e_pairs(e_ptr, hp, dy2, ndy2, dw1p, std::make_integer_sequence<int, H / 2>{});
        }
        fence_proxy_async_smem();
        named_arrive(BAR_E0 + wg, 160);
        y = y_next;
      };
      // The loop is unrolled by the number of row stages, one inlined instance of the body per stage.  (Unrolling
      // also spreads the register copies the compiler places at the loop's back edge — the 20 dW1 pairs and
      // the other values carried from tile to tile — over several tiles; unrolled by eight the loop no longer
      // fits the instruction cache and runs 6 % slower.)
      {
        using S0 = std::integral_constant<uint32_t, 0>;
        using S1 = std::integral_constant<uint32_t, 1>;
        using S2 = std::integral_constant<uint32_t, 2>;
        uint32_t k = 0;
        for (int i = 0; i + 1 < my_nt; i += 3, ++k) {
          tile_body(std::true_type{}, S1{}, i, k);
          if (i + 2 < my_nt) tile_body(std::true_type{}, S2{}, i + 1, k);
          if (i + 3 < my_nt) tile_body(std::true_type{}, S0{}, i + 2, k + 1);
        }
        if (my_nt > 0) tile_body(std::false_type{}, S0{}, my_nt - 1, 0u);
      }
#pragma unroll
      for (int st = 0; st < NST; ++st) use_s[st] += (uint32_t)(my_nt - st + NST - 1) / NST;
      n_done += my_nt;

      // ---- this warp's share of dW1 / db1 / log-lik ----
      if (n_done > 0) mbar_wait_q(&bar_bwd[wg], (n_done - 1) & 1, g.status, 204, ok);
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
        // Gt accumulator row i = 32 * group + feature lives in lane 32 * (i / 16) + i % 16 (M = 64): warp w
        // holds, in its lanes 0..15, features 16 * (w & 1) + lane of row group w >> 1, whose hidden
        // units are columns H * (w >> 1) .. + H - 1
        tc_fence_after();
        const int grp = warp >> 1, k = (warp & 1) * 16 + lane;
        const uint32_t trow = tmem_g + ((uint32_t)(warp * 32) << 16) + grp * H;
        float gacc[H];
#pragma unroll
        for (int c = 0; c < H; c += 8) tc_ld8(trow + c, gacc + c);
        tc_wait_ld();
        // the other warpgroups' accumulators (those that had tiles in this segment)
#pragma unroll
        for (int w = 1; w < NWG; ++w) {
          if (w < nt) {
            float g2[H];
#pragma unroll
            for (int c = 0; c < H; c += 8) tc_ld8(trow + w * G::G_STRIDE + c, g2 + c);
            tc_wait_ld();
#pragma unroll
            for (int c = 0; c < H; ++c) gacc[c] += g2[c];
          }
        }
        const bool mine = lane < 16 && k <= COL_ONE;  // feature rows 0..21 and the constant-1 row (db0)
        if (grp == 1 && mine) {
#pragma unroll
          for (int c = 0; c < H; c += 4)
            *reinterpret_cast<float4*>(&red_g[k][c]) = make_float4(gacc[c], gacc[c + 1], gacc[c + 2], gacc[c + 3]);
        }
        named_sync(1, 128);
        if (grp == 0 && mine) {
          // dW0[k][j] = W1[j] * Gt[k][j]; E was stored negated
          float* dst = po + k * H;
#pragma unroll
          for (int c = 0; c < H; c += 4) {
            const float4 o = *reinterpret_cast<const float4*>(&red_g[k][c]);
            const float4 w1 = *reinterpret_cast<const float4*>(w1s + c);
            *reinterpret_cast<float4*>(dst + c) =
                make_float4(-w1.x * (gacc[c] + o.x), -w1.y * (gacc[c + 1] + o.y),
                            -w1.z * (gacc[c + 2] + o.z), -w1.w * (gacc[c + 3] + o.w));
          }
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
static cudaError_t launch_tf32_t(const void* tmap_mn, const GradParams& g, int ctas, cudaStream_t st) {
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
                             *reinterpret_cast<const CUtensorMap*>(tmap_mn), g);
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
  return cudaLaunchKernelEx(&cfg, grad_tf32_kernel<40, true>, *reinterpret_cast<const CUtensorMap*>(tmap_mn), g);
}

cudaError_t launch_grad_tf32(int H, const void* tmap_mn, const GradParams& g, int ctas, cudaStream_t st) {
  if (H == 40) return launch_tf32_t<40>(tmap_mn, g, ctas, st);
  if (H == 128) return launch_grad_tf32_wide(tmap_mn, g, ctas, st);  // grad_tf32_wide.cu
  return cudaErrorInvalidValue;
}

}  // namespace mcmc_b200

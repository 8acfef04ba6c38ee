// TF32 tensor-core fused leapfrog-update + forward + backward kernel for the
// wide model (22 -> 128 -> 1, 3073 parameters), sm_100a.
//
// Same math and the same building blocks as grad_tf32.cu (rows staged by TMA,
// forward A operand and both accumulators in tensor memory, E^T . Xa backward
// with E written K-major into shared memory, no atomics, bounded waits); what
// changes with 128 hidden units is where things fit:
//   * a row of Z is 128 values, more than a thread can hold, so the epilogue
//     makes two passes over Z in 32-column chunks.  Pass 1: tanh, the output
//     layer, and h written BACK to tensor memory in place of Z.  Then the
//     per-row loss and dL/dpred.  Pass 2: h again, E = (1 - h^2) dL/dpred to
//     shared memory, and dW1;
//   * dW1[j] = sum over rows of dL/dpred * h[j]: one accumulator per hidden unit and thread (64 register
//     pairs, packed fma), kept for a whole segment; the control warpgroup hands its registers to the
//     compute warpgroups for that (setmaxnreg: 216 / 64).  Once per segment each warp reduces the four
//     32-column chunks across its 32 rows with a halving butterfly (31 shuffles per chunk: every step a
//     lane sends one half of its values and keeps the other), which leaves column `lane` of the chunk in
//     lane `lane`.  (Reducing every tile instead, with four accumulators per thread, cost about 500
//     instructions per row.)
//   * E of one tile is 64 KB, so there are two tile pipelines per CTA (two
//     compute warpgroups + a control warpgroup, 384 threads) with two TMA
//     stages each, and one Z accumulator per pipeline (2 x 128 columns): the
//     next tile's forward MMAs are issued once the last chunk of h has been
//     read, and the next tile's rows are staged just before that;
//   * the backward is one M = 128 MMA per 8 rows: G[128 hidden x 24] in tensor
//     memory, accumulator row i in lane i.
// The reference has no kernel of this shape: its sizes are compile-time
// constants for 40 hidden units (global_params.h:55-58).
#include <cuda.h>
#include <utility>
#include "common.cuh"
#include "chain.cuh"
#include "tc05.cuh"

namespace mcmc_b200 {

constexpr int WIDE_NWG = 2;                          // tile pipelines = compute warpgroups
constexpr int WIDE_THREADS = WIDE_NWG * 128 + 128;   // + a control warpgroup (one warp per pipeline, two idle)
constexpr int WIDE_NST = 2;                          // TMA stages per pipeline
// registers: 384 threads start with 168 each; the control warpgroup hands most of its share to the two
// compute warpgroups (2 * 128 * 216 + 128 * 64 = 63,488 <= 384 * 168), which lets a thread keep one dW1
// accumulator per hidden unit (128) for a whole segment
constexpr int WIDE_COMPUTE_REGS = 216;
constexpr int WIDE_CTRL_REGS = 64;

struct WideGeom {
  // backward N: an M = 128 MMA needs N % 16 == 0, so the whole 32-float staged row (24 real columns +
  // 8 columns of TMA zero fill) is the B operand and the accumulator has 32 columns, 24 of them read
  static constexpr int H = 128, D = 22, NF = 128, MB = 128, NB = 32, NBR = 24, CH = 32, NCH = H / CH;
  static constexpr int TILE_BYTES = TF32_TILE * 128;
  static constexpr int XB_BYTES = WIDE_NWG * WIDE_NST * TILE_BYTES;
  static constexpr int ES_ATOM_BYTES = H * 128;       // 32 rows (K) x 128 hidden lines
  static constexpr int ES_WG_BYTES = 4 * ES_ATOM_BYTES;
  static constexpr int ES_BYTES = WIDE_NWG * ES_WG_BYTES;
  static constexpr int W0S_BYTES = NF * 128;
  static constexpr int W1_BYTES = H * 4;
  static constexpr int P = D * H + 2 * H + 1;
  static constexpr size_t SMEM = 1024 + XB_BYTES + ES_BYTES + W0S_BYTES + W1_BYTES;
  static constexpr int A_COL0 = 0, A_STRIDE = 24;
  static constexpr int Z_COL0 = WIDE_NWG * A_STRIDE, Z_STRIDE = NF;
  static constexpr int G_COL0 = Z_COL0 + WIDE_NWG * Z_STRIDE, G_STRIDE = NB;
  static constexpr int TMEM_COLS = 512;
  static_assert(G_COL0 + WIDE_NWG * G_STRIDE <= TMEM_COLS, "tensor memory budget");
};

__device__ __forceinline__ void tc_ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
        "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
      "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
      "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
      "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
      "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])),
      "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])),
      "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
      "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
      "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
      "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}

// E stores of one 32-column chunk: hidden unit 32*C + J is line 32*C + J of the atom (immediate offset)
template <int C, int J>
__device__ __forceinline__ void store_e_wide_one(const uint32_t* e_ptr, const float* v) {
  asm volatile("st.shared.f32 [%0+%2], %1;" ::"r"(e_ptr[J & 7]), "f"(v[J]), "n"((32 * C + J) * 128)
               : "memory");
}
template <int C, int... Js>
__device__ __forceinline__ void store_e_wide(const uint32_t* e_ptr, const float* v,
                                             std::integer_sequence<int, Js...>) {
  (store_e_wide_one<C, Js>(e_ptr, v), ...);
}

__global__ void __launch_bounds__(WIDE_THREADS, 1)
grad_tf32_wide_kernel(const __grid_constant__ CUtensorMap tmap_mn, const GradParams g) {
  using G = WideGeom;
  constexpr int D = G::D, H = G::H, NF = G::NF, MB = G::MB, NB = G::NB, NWG = WIDE_NWG, NST = WIDE_NST;
  constexpr int CH = G::CH, NCH = G::NCH;
  constexpr uint32_t IDESC_FWD = umma_idesc_tf32(128, NF, 0, 0);
  constexpr uint32_t IDESC_BWD = umma_idesc_tf32(MB, NB, 0, 1);
  constexpr int NCOMPUTE = NWG * 128;
  constexpr int NCWARPS = NWG * 4;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* base =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  unsigned char* xb = base;                   // [NWG][NST][128 rows][128 B], TMA-written, 32-byte-chunk swizzle
  unsigned char* es = xb + G::XB_BYTES;       // [NWG][4 atoms][128 lines][128 B], E operand, K-major
  unsigned char* w0s = es + G::ES_BYTES;      // [128][128 B] weights, K-major
  float* w1s = reinterpret_cast<float*>(w0s + G::W0S_BYTES);
  __shared__ __align__(8) uint64_t bar_tma[NWG][NST];
  __shared__ __align__(8) uint64_t bar_fwd[NWG], bar_bwd[NWG];
  __shared__ uint32_t tmem_slot;
  __shared__ float b1s;
  __shared__ float red_w1[NCWARPS][H];
  __shared__ float red_db1[NCWARPS];
  __shared__ double red_ll[NCWARPS];

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const bool is_ctrl = warp >= NCWARPS;
  // pipeline this warp computes for / issues for (through a shuffle: visibly the same in every lane, which
  // keeps the control warps' descriptor arithmetic in uniform registers)
  const int wg = __shfl_sync(0xffffffffu, is_ctrl ? warp - NCWARPS : warp >> 2, 0);
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
  // zero the weight operand once (k >= 23 stays zero)
  for (int i = tid; i < G::W0S_BYTES / 16; i += WIDE_THREADS)
    reinterpret_cast<float4*>(w0s)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tmem_g = tmem + G::G_COL0;
  const uint32_t w0s_addr = smem_u32(w0s);
  const int seg0 = g.seg_ptr[blockIdx.x], seg1 = g.seg_ptr[blockIdx.x + 1];  // host-written table
  bool ok = true;
  // everything above is private set-up; from here on the kernel reads what its predecessor wrote
  pdl_trigger();
  pdl_wait();

  // Every segment has three CTA-wide barriers, executed by both roles:
  //   S1 parameters staged   S2 all tiles of the segment done   S3 read-out done
  if (is_ctrl) {
    // =====================  control warpgroup (one warp per pipeline; the others keep the barriers) ====
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(WIDE_CTRL_REGS));
    uint32_t c_issued = 0;  // tiles of this pipeline whose MMAs have been issued (mbarrier phases follow it)
    for (int sg = seg0; sg < seg1; ++sg) {
      const int4 seg = g.segs[sg];
      const int win = seg.x, t0 = seg.y, nt = seg.z - seg.y;
      const int grow0 = (g.data_window0 + win) * rows_pad;
      __syncthreads();  // S1
      if (wg < NWG) {
        // Per tile n: forward(n+1) once its rows are in tensor memory and Z(n) has been consumed (the
        // warpgroup says so with one barrier), backward(n) when E(n) is in shared memory, then — once
        // those MMAs have completed — the TMA refill of the row stage they read.
        const int cnt = (nt - wg + NWG - 1) / NWG;
        const uint32_t a_t = tmem + G::A_COL0 + wg * G::A_STRIDE;
        const uint32_t z_t = tmem + G::Z_COL0 + wg * G::Z_STRIDE;
        const uint32_t g_t = tmem_g + wg * G::G_STRIDE;
        const uint64_t wdesc0 = umma_desc_k128(w0s_addr);
        const uint64_t adesc0 = umma_desc_k128(smem_u32(es + wg * G::ES_WG_BYTES));
        const uint64_t bdesc0 = umma_desc_mn32(smem_u32(xb + wg * NST * G::TILE_BYTES), G::TILE_BYTES);
        uint32_t stage = c_issued % NST;
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
            const uint64_t bd = umma_desc_advance(bdesc0, stage * (G::TILE_BYTES >> 4));
#pragma unroll
            for (int kb = 0; kb < TF32_TILE / 8; ++kb)
              tc_mma_tf32_ss(g_t,
                             umma_desc_advance(adesc0, (kb >> 2) * (G::ES_ATOM_BYTES >> 4) + (kb & 3) * 2),
                             umma_desc_advance(bd, kb * 64), IDESC_BWD, (i == 0 && kb == 0) ? 0u : 1u);
            tc_commit(&bar_bwd[wg]);
            if (i + NST < cnt) {
              ok = ok && mbar_wait(&bar_bwd[wg], n & 1, g.status, 313);
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
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(WIDE_COMPUTE_REGS));
    // =====================  compute warpgroups: one row per thread  =====================================
    uint32_t n_done = 0;  // tiles this pipeline has finished (mbarrier phases follow it)
    uint32_t st_stage = 0, st_phase = 0;  // row stage and mbarrier phase of the next tile to be staged
    const uint32_t lane_off = (uint32_t)(wwarp * 32) << 16;
    const uint32_t a_t = tmem + G::A_COL0 + wg * G::A_STRIDE + lane_off;
    const uint32_t z_t = tmem + G::Z_COL0 + wg * G::Z_STRIDE + lane_off;
    // E element (hidden j, row r): atom r/32 (= this warp), line j, 16-byte chunk (r%32)/4 ^ (j%8)
    uint32_t e_ptr[8];
#pragma unroll
    for (int c = 0; c < 8; ++c)
      e_ptr[c] = smem_u32(es + wg * G::ES_WG_BYTES + wwarp * G::ES_ATOM_BYTES) +
                 ((uint32_t)(((lane >> 2) ^ c) << 4)) + ((lane & 3) << 2);
    const bool swap_halves = (wtid & 4) != 0;

    for (int sg = seg0; sg < seg1; ++sg) {
      const int4 seg = g.segs[sg];
      const int win = seg.x, t0 = seg.y, t1 = seg.z, slot = seg.w;
      const int nt = t1 - t0;
      const int grow0 = (g.data_window0 + win) * rows_pad;
      const int my_nt = (nt - wg + NWG - 1) / NWG;

      // ---- segment prologue: start the first row tiles, fused leapfrog update, stage W0a ----
      if (wtid == 0) {
        for (int i = 0; i < NST && i < my_nt; ++i) {
          const uint32_t n = n_done + i;
          mbar_expect_tx(&bar_tma[wg][n % NST], G::TILE_BYTES);
          tma_load_2d(xb + (wg * NST + n % NST) * G::TILE_BYTES, &tmap_mn, 0,
                      grow0 + (t0 + wg + i * NWG) * TF32_TILE, &bar_tma[wg][n % NST]);
        }
      }
      // element (n = hidden unit, k) of the K-major B operand at n*128 + ((k/4) ^ (n%8))*16 + (k%4)*4
      for (int p = tid; p < G::P; p += NCOMPUTE) {
        const float w = leapfrog_param(g, win, p, slot == 0);
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

      const float b1 = b1s;
      const uint32_t w1s_addr = smem_u32(w1s);
      uint64_t dw1p[H / 2];  // dW1 of this thread's rows, two hidden units per register pair
#pragma unroll
      for (int j = 0; j < H / 2; ++j) dw1p[j] = 0ull;
      float db1 = 0.f;
      double llacc = 0.0;

      // hands this thread's row of the landed tile to the tensor core (forward A operand); returns y
      auto stage_row = [&]() -> float {
        const uint32_t stage = st_stage, phase = st_phase;
        st_stage = st_stage + 1 == NST ? 0 : st_stage + 1;
        st_phase ^= (st_stage == 0) ? 1u : 0u;
        mbar_wait_q(&bar_tma[wg][stage], phase, g.status, 301, ok);
        // 32-byte chunk j of a row sits at position j ^ (row % 4); rows r and r+4 keep their chunks in
        // the same banks, so the upper four of every eight rows read the two halves in the opposite order
        const uint32_t xrow = smem_u32(xb + (wg * NST + stage) * G::TILE_BYTES + wtid * 128);
        float4 xr[6];
#pragma unroll
        for (int j = 0; j < 3; ++j) {
          const uint32_t cp = xrow + ((j ^ (wtid & 3)) << 5);
          const float4 first = lds128(cp + (swap_halves ? 16 : 0));
          const float4 second = lds128(cp + (swap_halves ? 0 : 16));
          xr[2 * j].x = swap_halves ? second.x : first.x;
          xr[2 * j].y = swap_halves ? second.y : first.y;
          xr[2 * j].z = swap_halves ? second.z : first.z;
          xr[2 * j].w = swap_halves ? second.w : first.w;
          xr[2 * j + 1].x = swap_halves ? first.x : second.x;
          xr[2 * j + 1].y = swap_halves ? first.y : second.y;
          xr[2 * j + 1].z = swap_halves ? first.z : second.z;
          xr[2 * j + 1].w = swap_halves ? first.w : second.w;
        }
#pragma unroll
        for (int j = 0; j < 3; ++j) tc_st8(a_t + j * 8, xr[2 * j], xr[2 * j + 1]);
        return xr[5].w;
      };
      // ... and tells the control warp: the rows are in place AND this thread is done with Z
      auto publish_row = [&]() {
        tc_wait_st();
        tc_fence_before();
        named_arrive(BAR_ROWS0 + wg, 160);
      };

      float y = 0.f;
      if (my_nt > 0) {
        y = stage_row();
        publish_row();
      }
      for (int i = 0; i < my_nt; ++i) {
        const uint32_t n = n_done + i;
        const int t = t0 + wg + i * NWG;
        const bool has_next = i + 1 < my_nt;
        mbar_wait_q(&bar_fwd[wg], n & 1, g.status, 302, ok);
        tc_fence_after();
        // ---- pass 1: h = tanh(Z) back into tensor memory, output layer ----
        float pred = b1;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          float v[CH];
          tc_ld32(z_t + c * CH, v);
          tc_wait_ld();
          uint64_t pp0 = 0ull, pp1 = 0ull;  // packed f32x2 accumulators of the output layer
#pragma unroll
          for (int j = 0; j < CH; j += 4) {
            const float4 w1v = lds128(w1s_addr + (c * CH + j) * 4);  // broadcast read
            v[j] = tanh_fast(v[j]);
            v[j + 1] = tanh_fast(v[j + 1]);
            v[j + 2] = tanh_fast(v[j + 2]);
            v[j + 3] = tanh_fast(v[j + 3]);
            pp0 = fma2(pack2(w1v.x, w1v.y), pack2(v[j], v[j + 1]), pp0);
            pp1 = fma2(pack2(w1v.z, w1v.w), pack2(v[j + 2], v[j + 3]), pp1);
          }
          float q0, q1, q2, q3;
          unpack2(pp0, q0, q1);
          unpack2(pp1, q2, q3);
          pred += (q0 + q1) + (q2 + q3);
          tc_st32(z_t + c * CH, v);
        }
        tc_wait_st();
        // ---- loss and dL/dpred of this row ----
        const int grow = t * TF32_TILE + wtid;
        const bool valid = grow < g.n_rows;
        float loss, dy;
        lik_terms(g.lik, y, pred, loss, dy);
        if (!valid) { loss = 0.f; dy = 0.f; }
        llacc += (double)loss;
        store_row_loss(g.row_loss, (long long)win * g.row_loss_stride + grow, loss, valid);
        db1 += dy;
        // the previous tile's backward MMAs must be done with E before it is overwritten
        if (n > 0) mbar_wait_q(&bar_bwd[wg], (n - 1) & 1, g.status, 303, ok);
        // ---- pass 2: E to shared memory, dW1 ----
        float y_next = 0.f;
        const float ndy = -dy;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          float v[CH];
          tc_ld32(z_t + c * CH, v);
          tc_wait_ld();
          const uint64_t dy2 = pack2(dy, dy), ndy2 = pack2(ndy, ndy);
#pragma unroll
          for (int j = 0; j < CH; j += 2) {
            const uint64_t h2 = pack2(v[j], v[j + 1]);
            dw1p[(c * CH + j) >> 1] = fma2(dy2, h2, dw1p[(c * CH + j) >> 1]);
            // (1 - h^2) dy = dy - (h h) dy; the W1 factor is applied at read-out
            unpack2(fma2(mul2(h2, h2), ndy2, dy2), v[j], v[j + 1]);
          }
          if (c == 0) store_e_wide<0>(e_ptr, v, std::make_integer_sequence<int, CH>{});
          if (c == 1) store_e_wide<1>(e_ptr, v, std::make_integer_sequence<int, CH>{});
          if (c == 2) store_e_wide<2>(e_ptr, v, std::make_integer_sequence<int, CH>{});
          if (c == 3) store_e_wide<3>(e_ptr, v, std::make_integer_sequence<int, CH>{});
        }
        if (has_next) {
          // every chunk of h(n) has been read: the next tile's rows go in and the control warp may start
          // forward(n+1), which overwrites the accumulator
          y_next = stage_row();
          publish_row();
        }
        fence_proxy_async_smem();
        named_arrive(BAR_E0 + wg, 160);
        y = y_next;
      }
      n_done += my_nt;

      // ---- this warp's share of dW1 / db1 / log-lik ----
      if (my_nt > 0) mbar_wait_q(&bar_bwd[wg], (n_done - 1) & 1, g.status, 304, ok);
      tc_fence_after();
      // column sums over the warp's 32 rows, one 32-unit chunk at a time (halving butterfly: lane l ends with
      // hidden unit 32 c + l), once per segment
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        float v[CH];
#pragma unroll
        for (int j = 0; j < CH; j += 2) unpack2(dw1p[(c * CH + j) >> 1], v[j], v[j + 1]);
        red_w1[warp][c * CH + lane] = warp_column_sums(v, lane);
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
      float* po = g.partial_out + ((size_t)win * g.slices_out + slot) * g.Pp;
      if (warp < 4) {
        tc_fence_after();
        constexpr int NBR = G::NBR;
        float gacc[NBR];
#pragma unroll
        for (int c = 0; c < NBR; ++c) gacc[c] = 0.f;
        const uint32_t trow = tmem_g + ((uint32_t)(warp * 32) << 16);
#pragma unroll
        for (int w = 0; w < NWG; ++w) {
          if (w < nt) {  // the pipelines that had tiles in this segment
            float g2[NBR];
#pragma unroll
            for (int c = 0; c < NBR; c += 8) tc_ld8(trow + w * G::G_STRIDE + c, g2 + c);
            tc_wait_ld();
#pragma unroll
            for (int c = 0; c < NBR; ++c) gacc[c] += g2[c];
          }
        }
        // M = 128: accumulator row i (hidden unit i) lives in lane i
        const int hidx = warp * 32 + lane;
        const float w1 = w1s[hidx];
#pragma unroll
        for (int k = 0; k < D; ++k) po[k * H + hidx] = w1 * gacc[k];
        po[D * H + hidx] = w1 * gacc[COL_ONE];
        tc_fence_before();
      } else {
        const int j = tid - 128;  // the second warpgroup: one hidden unit per thread
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < NCWARPS; ++w) s += red_w1[w][j];
        po[D * H + H + j] = s;
        if (j == 0) {
          float sb = 0.f;
          double l = 0.0;
          for (int w = 0; w < NCWARPS; ++w) { sb += red_db1[w]; l += red_ll[w]; }
          po[D * H + 2 * H] = sb;
          g.ll_out[(size_t)win * g.slices_out + slot] = l;
        }
      }
      __syncthreads();  // S3: read-out done before the next segment restages W0a
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

cudaError_t launch_grad_tf32_wide(const void* tmap_mn, const GradParams& g, int ctas, cudaStream_t st) {
  static bool attr_done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(grad_tf32_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)WideGeom::SMEM);
    if (e != cudaSuccess) return e;
    attr_done[dev] = true;
  }
  return launch_chain_kernel(grad_tf32_wide_kernel, dim3(ctas), dim3(WIDE_THREADS), WideGeom::SMEM, st,
                             *reinterpret_cast<const CUtensorMap*>(tmap_mn), g);
}

}  // namespace mcmc_b200

// Shared device-side definitions of the HMC hot path: launch parameter
// blocks, the fused leapfrog prologue, likelihood terms and the PTX wrappers
// (mbarrier, bulk copies, tcgen05) used by the gradient kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <utility>

namespace mcmc_b200 {

// Rows of the repacked dataset: 22 features, a constant 1 (so that the hidden
// bias is row 22 of W0 and db0 is row 22 of dW0), and the target y.
constexpr int KP = 24;          // floats per repacked row (96 bytes)
constexpr int COL_ONE = 22;
constexpr int COL_Y = 23;
constexpr int MAX_SLICES = 1024;

enum GradMode : int {
  MODE_EVAL = 0,   // evaluate at w_in as it is (the reference's eps = 0 call, main.h:85-99)
  MODE_FIRST = 1,  // half kick with the carried gradient, drift (MOM_CORRECTION = 2)
  MODE_NEXT = 2    // full kick with the gradient of the previous step, drift
};

struct LikParams {
  int kind;          // 0 Student-t, 1 Gaussian
  float inv_scale;   // 1 / scale
  float df;          // Student-t degrees of freedom
  float norm;        // log-normaliser
  float g_scale;     // (df + 1) / scale  (Student-t)  |  1 / scale (Gaussian)
  float l_scale;     // -(df + 1) / 2     (Student-t)  |  -1/2      (Gaussian)
  float inv_df;
};

struct PriorParams {
  float neg_inv_s2;  // -1 / s^2   (PRIOR_SCALE_NEG_RECP2)
  float inv_s;       // 1 / s
  float norm;        // PRIOR_LOSS_NORMALIZATION
};

// One launch of a gradient kernel: grid = (slices, windows).
struct GradParams {
  // data
  const float* xaug;        // [windows][rows_pad][KP]
  long long window_stride;  // floats between windows in xaug
  int data_window0;         // first data window this launch covers
  int n_rows;               // valid rows per window
  int n_tiles;              // rows_pad / tile rows
  int P, Pp;                // parameters, padded to a multiple of 4
  // state in / out ([windows][Pp], indexed by blockIdx.y)
  const float* w_in;
  const float* m_in;
  float* w_out;
  float* m_out;
  const float* g_carried;   // MODE_FIRST
  const float* partial_in;  // MODE_NEXT: [windows][slices_in][Pp] likelihood-gradient partials
  int slices_in;            // slots per window in partial_in (stride, and count when nslot_in is null)
  const int* nslot_in;      // optional [windows]: slots of partial_in that are in use
  // persistent (one CTA per SM) kernels: which tile ranges this launch's CTAs own
  const int* seg_ptr;       // [ctas + 1] first segment of each CTA
  const int4* segs;         // {window, first tile, end tile, slot}
  int slices_out;           // slots per window in partial_out / ll_out
  const double* red_in;     // MODE_NEXT with row sharding: [windows][Pp + 4] all-reduced sums
  float* partial_out;       // [windows][slices][Pp]
  double* ll_out;           // [windows][slices]
  const float* eps;         // [windows] or null
  float eps_scalar;
  int mode;
  float* row_loss;          // optional [windows][rows_pad]
  long long row_loss_stride;
  LikParams lik;
  PriorParams prior;
  int* status;              // device error word (bounded waits that ran out)
  int data_fresh;           // 1: xaug was written by the launch directly before this one in the stream, so
                            // no row may be fetched ahead of the programmatic-dependency wait
  // several leapfrog steps in one cooperative launch (one window; grad_tf32.cu).  Step s reads
  // w_buf/m_buf[s & 1], writes [(s + 1) & 1] and partial_buf/ll_buf[s & 1]; `red` receives the summed
  // gradient after every step; grid_bar is a zeroed arrival counter
  int n_steps;
  int n_slots;              // CTAs that own tiles = partial vectors to sum
  float* w_buf[2];
  float* m_buf[2];
  float* partial_buf[2];
  double* ll_buf[2];
  double* red;
  unsigned int* grid_bar;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- reference tanh (kernel_helpers.h:32-44): 2*sigmoid(2x)-1 on ex2/rcp
// approximations, identity below the cut-off -------------------------------
__device__ __forceinline__ float tanh_ref(float x) {
  float e, d, s;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -2.88539008177792681472f));
  asm("add.ftz.f32 %0, %1, %2;" : "=f"(d) : "f"(1.f), "f"(e));
  asm("rcp.approx.f32 %0, %1;" : "=f"(s) : "f"(d));
  return fabsf(x) < 0.0048176045529544353485f ? x : fmaf(s, 2.f, -1.f);
}
// one MUFU op; absolute error about 5e-4, inside the TF32 mode's tolerance
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// per-row log-likelihood and d(log-lik)/d(prediction)
// (mcmc_step_ffma.h:289-301 for Student-t)
__device__ __forceinline__ void lik_terms(const LikParams& lk, float y, float pred, float& loss,
                                          float& dy) {
  float d = (y - pred) * lk.inv_scale;
  float d2 = d * d;
  if (lk.kind == 0) {
    loss = lk.l_scale * log1pf(d2 * lk.inv_df) - lk.norm;
    dy = __fdividef(d * lk.g_scale, d2 + lk.df);
  } else {
    loss = fmaf(lk.l_scale, d2, -lk.norm);
    dy = d * lk.g_scale;
  }
}

// Fused leapfrog update for parameter p of window `win`
// (apply_leapfrog_step, mcmc_step_ffma.h:106-120; load_weights_bias :122-152):
// every CTA of the window recomputes the same value from the same inputs in
// the same order, slice 0 stores it.
// The state vectors and sums are read with ld.global.cg: inside a multi-step launch they were written by
// other CTAs of the same kernel, and L1 is not coherent.
struct StepIo {            // what changes from one leapfrog step to the next
  const float* w_in;
  const float* m_in;
  float* w_out;
  float* m_out;
  const double* red_in;
  int mode;
};
__device__ __forceinline__ StepIo step_io(const GradParams& g) {
  return StepIo{g.w_in, g.m_in, g.w_out, g.m_out, g.red_in, g.mode};
}
// step s of a multi-step launch (chain_grad's buffer rotation)
__device__ __forceinline__ StepIo step_io(const GradParams& g, int s) {
  // (constant indices under a select: a dynamic index would move the parameter arrays to local memory)
  const bool odd = (s & 1) != 0;
  return StepIo{odd ? g.w_buf[1] : g.w_buf[0], odd ? g.m_buf[1] : g.m_buf[0],
                odd ? g.w_buf[0] : g.w_buf[1], odd ? g.m_buf[0] : g.m_buf[1],
                s == 0 ? nullptr : g.red, s == 0 ? MODE_FIRST : MODE_NEXT};
}
__device__ __forceinline__ float leapfrog_param(const GradParams& g, const StepIo& io, int win, int p,
                                                bool store) {
  const size_t o = (size_t)win * g.Pp + p;
  float w = __ldcg(io.w_in + o);
  if (io.mode == MODE_EVAL) return w;
  float grad;
  float kick;
  if (io.mode == MODE_FIRST) {
    grad = g.g_carried[o];
    kick = 0.5f;
  } else {
    if (io.red_in) {
      grad = (float)__ldcg(io.red_in + (size_t)win * (g.Pp + 4) + p);
    } else {
      const float* pi = g.partial_in + (size_t)win * g.slices_in * g.Pp + p;
      const int ns = g.nslot_in ? g.nslot_in[win] : g.slices_in;
      grad = 0.f;
      for (int s = 0; s < ns; ++s) grad += pi[(size_t)s * g.Pp];
    }
    grad = fmaf(w, g.prior.neg_inv_s2, grad);  // prior gradient at the previous point
    kick = 1.f;
  }
  const float eps = g.eps ? g.eps[win] : g.eps_scalar;
  float m = __ldcg(io.m_in + o);
  m = fmaf(eps * kick, grad, m);
  w = fmaf(eps, m, w);
  if (store) {
    io.w_out[o] = w;
    io.m_out[o] = m;
  }
  return w;
}
__device__ __forceinline__ float leapfrog_param(const GradParams& g, int win, int p, bool store) {
  return leapfrog_param(g, step_io(g), win, p, store);
}

// ---- mbarrier / bulk-copy wrappers --------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait that lets the hardware suspend the thread for up to `hint_ns` until the phase completes
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
// Bounded wait: the thread sleeps in hardware on the barrier in slices of 20 us and gives up after
// `slices` of them (default 2^16, about 1.3 s), records the code in the status word and returns false;
// the kernel then finishes with whatever it has, so a lost copy or MMA can never hang the GPU.
constexpr uint32_t MBAR_WAIT_SLICES = 1u << 16;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status, int code,
                                          uint32_t slices = MBAR_WAIT_SLICES) {
  if (mbar_try_wait(bar, parity)) return true;
  for (uint32_t i = 0; i < slices; ++i) {
    if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
  }
  if (status) atomicExch(status, code);
  return false;
}
// contiguous global -> shared copy through the bulk-copy engine
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(smem_u32(dst_smem)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// block-wide sum of doubles in a fixed order (deterministic); blockDim.x <= 1024
__device__ __forceinline__ double block_sum_f64(double v, double* scratch /* >= 32 */) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) scratch[w] = v;
  __syncthreads();
  double t = 0.0;
  const int nw = (blockDim.x + 31) >> 5;
  for (int i = 0; i < nw; ++i) t += scratch[i];
  return t;
}

// Packed FP32 pairs (sm_100 executes fma/mul on two floats per instruction)
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// ---- grid-wide barrier of a cooperative launch --------------------------------
// Every CTA of the grid is resident (the launch is cooperative), so the wait always ends; it is bounded
// all the same: after about 0.3 s the leader records `code`, and every later barrier of this CTA returns at
// once so that the kernel runs to its end (with results that the status word marks as invalid).
// `target` = arrivals expected in total at this barrier = (barriers passed so far + 1) * gridDim.x.
__device__ __forceinline__ bool grid_barrier(unsigned int* cnt, unsigned int target, bool leader, bool& alive,
                                             int* status, int code) {
  __shared__ int s_alive;
  __syncthreads();
  if (leader) {
    bool ok = alive;
    if (ok) {
      __threadfence();
      atomicAdd(cnt, 1u);
      unsigned int seen = 0;
      for (int it = 0; it < (1 << 19); ++it) {  // one L2 round trip per poll: about 0.3 s in all
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(cnt) : "memory");
        if (seen >= target) break;
      }
      ok = seen >= target;
      if (!ok && status) atomicExch(status, code);
      __threadfence();
    }
    s_alive = ok ? 1 : 0;
  }
  __syncthreads();
  alive = s_alive != 0;
  return alive;
}

// ---- programmatic dependent launch -----------------------------------------
// The chain is a string of short dependent launches (gradient, partial sum, accept).  A kernel
// launched with the programmatic-serialization attribute may start while its predecessor is still
// draining: its CTAs are scheduled as the predecessor's CTAs exit, do their private set-up (barriers,
// tensor-memory allocation, first row tiles — nothing the predecessor writes) and then block in
// pdl_wait() until the predecessor has completed and its writes are visible.  Every kernel of the
// chain calls pdl_trigger() (lets ITS successor start early) and pdl_wait() before it touches
// anything a predecessor produced, and writes global memory only after the wait.  Without the launch
// attribute both calls do nothing.  MCMC_B200_NO_PDL=1 turns the attribute off.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("MCMC_B200_NO_PDL");
    return !(e && e[0] == '1');
  }();
  return on;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chain_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                       cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace mcmc_b200

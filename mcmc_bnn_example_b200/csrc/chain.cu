// Per-iteration kernels of the HMC driver, one CTA per window:
//   * hmc_accept_kernel — the fixed-order sum of the gradient partials, the
//     prior terms, the closing half kick, the Hamiltonian difference, the
//     Philox accept draw, accept/reject, step-size adaptation, sample store and
//     the momentum draw of the next iteration.  It replaces the reference's
//     momentum-draw launch (main.h:207-216), log_acpt_prec (two launches, a
//     D2H copy and a stream synchronise, kernel_helpers.h:153-188), the host
//     accept draw (main.h:235-239), the six D2D copies (main.h:242-265), the
//     host step-size update (main.h:266-276) and the sample copy (:277-283):
//     no host round trip is left inside an iteration.
//   * repack_kernel — [N][22] + [N] -> [N_pad][24] rows {x, 1, y}.
//   * reduce_partials_kernel — row sharding: the vector that is all-reduced.
//   * log_acpt_kernel — the drop-in accept ratio on caller buffers.
#include <thrust/random.h>

#include "common.cuh"
#include "chain.cuh"
#include "philox.h"

namespace mcmc_b200 {

constexpr int ACC_THREADS = 256;

// One momentum draw of the reference's stream (main.h:207-213): a fresh Thrust engine advanced by n,
// one N(0,1) draw.  Thrust's own code does the work, as it does in the reference.
__device__ __forceinline__ float refstream_normal(unsigned long long n) {
  thrust::default_random_engine engine;
  engine.discard(n);
  thrust::normal_distribution<float> unit_normal(0.f, 1.f);
  return unit_normal(engine);
}
constexpr unsigned long long REF_DRAWS_PER_ITER = 962;  // 961 momenta + 1 accept draw (main.h:216,237)

__global__ void __launch_bounds__(ACC_THREADS) hmc_accept_kernel(const AcceptParams a) {
  __shared__ double dsc[32];
  __shared__ int s_accept;
  const int win = blockIdx.x;
  const int tid = threadIdx.x;
  const size_t o = (size_t)win * a.Pp;
  pdl_trigger();
  pdl_wait();
  const int iter = (a.mode == ACC_ITERATE) ? a.iter[win] : 0;
  const float eps = a.eps ? a.eps[win] : 0.f;
  const uint32_t gwin = a.gwin ? (uint32_t)a.gwin[win] : 0u;

  // log-likelihood of the proposal: fixed-order sum of the slice partials
  const int ns = a.nslot ? a.nslot[win] : a.slices;
  double ll_new;
  if (a.red_in) {
    ll_new = a.red_in[(size_t)win * (a.Pp + 4) + a.Pp];
  } else {
    ll_new = 0.0;
    for (int s = 0; s < ns; ++s) ll_new += a.ll_partial[(size_t)win * a.slices + s];
  }

  constexpr int MAXPT = 16;  // parameters per thread (P <= 4096)
  float wv[MAXPT], gv[MAXPT];
  double lp_loc = 0.0, dk_loc = 0.0;
  int n = 0;
  for (int p = tid; p < a.P; p += ACC_THREADS, ++n) {
    const float w = a.w_new[o + p];
    float g;
    if (a.red_in) {
      g = (float)a.red_in[(size_t)win * (a.Pp + 4) + p];
    } else {
      const float* pi = a.partial + (size_t)win * a.slices * a.Pp + p;
      g = 0.f;
      for (int s = 0; s < ns; ++s) g += pi[(size_t)s * a.Pp];
    }
    g = fmaf(w, a.prior.neg_inv_s2, g);
    const float q = w * a.prior.inv_s;
    const float pl = fmaf(-0.5f * q, q, -a.prior.norm);
    lp_loc += (double)pl;
    if (a.prior_loss_out) a.prior_loss_out[p] = pl;
    if (a.mode == ACC_ITERATE) {
      // closing half kick (kernel_helpers.h:169-172)
      const float mf = fmaf(eps * 0.5f, g, a.m_new[o + p]);
      const float m0 = a.m0[o + p];
      dk_loc += 0.5 * ((double)m0 * (double)m0 - (double)mf * (double)mf);
    }
    wv[n] = w;
    gv[n] = g;
  }
  const double lp_new = block_sum_f64(lp_loc, dsc);
  const double dk = (a.mode == ACC_ITERATE) ? block_sum_f64(dk_loc, dsc) : 0.0;

  if (a.mode == ACC_FINALIZE) {
    n = 0;
    for (int p = tid; p < a.P; p += ACC_THREADS, ++n) a.g_out[p] = gv[n];
    if (tid == 0) {
      // a bounded wait that ran out left the sums incomplete: say so in the result itself
      const bool bad = a.status_in && *a.status_in != 0;
      a.scalars_out[0] = bad ? (double)NAN : ll_new;
      a.scalars_out[1] = bad ? (double)NAN : lp_new;
    }
    return;
  }

  if (tid == 0) {
    int acc = 1;
    float eps_next = eps;
    if (a.mode == ACC_ITERATE) {
      const double la = (ll_new - a.ll_cur[win]) + (lp_new - a.lp_cur[win]) + dk;
      const float la_f = (float)la;
      const float log_u = a.ref_streams ? a.ref_log_u[iter % a.ref_cap]
                                        : logf(philox_accept_uniform(a.seed, gwin, (uint32_t)iter));
      acc = log_u < la_f;  // main.h:242; a NaN ratio rejects
      if (iter < a.adapt_steps) {  // main.h:266-276
        const float lmr = fminf(la_f, 0.f);
        const float adj = lmr < a.log_target ? a.dec_adj : a.inc_adj;
        eps_next = eps + eps * adj;
      }
      if (iter < a.trace_iters) {
        const size_t ti = (size_t)win * a.trace_iters + iter;
        a.tr_log_u[ti] = log_u;
        a.tr_log_acpt[ti] = la;
        a.tr_accept[ti] = acc;
        a.tr_eps[ti] = eps;
      }
      a.n_accept[win] += acc;
      a.iter[win] = iter + 1;
      a.eps[win] = eps_next;
    }
    if (acc) {
      a.ll_cur[win] = ll_new;
      a.lp_cur[win] = lp_new;
    }
    s_accept = acc;
  }
  __syncthreads();
  const int acc = s_accept;
  const int next_iter = (a.mode == ACC_ITERATE) ? iter + 1 : 0;
  const int store = (a.mode == ACC_ITERATE) ? iter - a.burn_in : -1;
  n = 0;
  for (int p = tid; p < a.P; p += ACC_THREADS, ++n) {
    float w_state;
    if (acc) {
      w_state = wv[n];
      a.w_cur[o + p] = wv[n];
      a.g_cur[o + p] = gv[n];
    } else {
      w_state = a.w_cur[o + p];
    }
    if (store >= 0 && store < a.sample_capacity)
      a.samples[((size_t)win * a.sample_capacity + store) * a.P + p] = w_state;
    // start of the next iteration: position, fresh momentum (main.h:207-218)
    const float m = a.ref_streams
                        ? refstream_normal(a.seed + REF_DRAWS_PER_ITER * (unsigned long long)next_iter + p)
                        : philox_normal(a.seed, gwin, (uint32_t)next_iter, STREAM_MOMENTUM, (uint32_t)p);
    a.w_start[o + p] = w_state;
    a.m_start[o + p] = m;
    a.m0[o + p] = m;
    if (next_iter < a.trace_iters)
      a.tr_mom[((size_t)win * a.trace_iters + next_iter) * a.P + p] = m;
  }
}

cudaError_t launch_accept(const AcceptParams& a, int windows, cudaStream_t st) {
  return launch_chain_kernel(hmc_accept_kernel, dim3(windows), dim3(ACC_THREADS), 0, st, a);
}

__global__ void refstream_momentum_kernel(unsigned long long first_n, int count, float* out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] = refstream_normal(first_n + i);
}
cudaError_t launch_refstream_momentum(unsigned long long first_n, int count, float* out, cudaStream_t st) {
  refstream_momentum_kernel<<<(count + 127) / 128, 128, 0, st>>>(first_n, count, out);
  return cudaGetLastError();
}

// ---- bounded-wait self-test ------------------------------------------------
// One CTA waits, with the gradient kernels' own mbar_wait, on a barrier that nothing ever arms: the wait
// runs out after `slices` slices of 20 us, records its code in the status word and the kernel returns by
// itself.  This is how the time-out route (status word -> MCMC_B200_ERR_TIMEOUT -> context still usable)
// is exercised without any fault, trap or unbounded wait (the reference's barrier spins without a limit,
// mcmc_step_tc.h:597-612).
__global__ void wait_probe_kernel(int* status, unsigned int slices) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(&bar, 0, status, 901, slices);
}
cudaError_t launch_wait_probe(int* status, unsigned int slices, cudaStream_t st) {
  wait_probe_kernel<<<1, 32, 0, st>>>(status, slices);
  return cudaGetLastError();
}

// ---- the device's random streams, for comparison with the host's ------------------------
// n raw Philox blocks for counters {ctr0 + i, ctr1, ctr2, ctr3}, and the n momentum normals / the accept
// uniform the accept kernel would draw for (seed, window, iteration): same functions, run on the device.
__global__ void philox_probe_kernel(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1,
                                    int n, uint32_t* raw, float* normals, float* uniform) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const Philox4 r = philox4x32_10(c0 + (uint32_t)i, c1, c2, c3, k0, k1);
  for (int q = 0; q < 4; ++q) raw[4 * i + q] = r.v[q];
  const uint64_t seed = ((uint64_t)k1 << 32) | k0;
  normals[i] = philox_normal(seed, c2, c1, STREAM_MOMENTUM, (uint32_t)i);
  if (i == 0) *uniform = philox_accept_uniform(seed, c2, c1);
}
cudaError_t launch_philox_probe(const uint32_t ctr[4], const uint32_t key[2], int n, uint32_t* raw, float* normals,
                                float* uniform, cudaStream_t st) {
  philox_probe_kernel<<<(n + 127) / 128, 128, 0, st>>>(ctr[0], ctr[1], ctr[2], ctr[3], key[0], key[1], n, raw,
                                                       normals, uniform);
  return cudaGetLastError();
}

// ---- dataset repack ------------------------------------------------------
__global__ void repack_kernel(const float* __restrict__ x, const float* __restrict__ y,
                              float* __restrict__ out, long long n_rows, long long rows_pad, int D) {
  const long long total = rows_pad * KP;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / KP;
    const int c = (int)(i - r * KP);
    float v = 0.f;
    if (r < n_rows) {
      if (c < D) v = x[r * D + c];
      else if (c == COL_ONE) v = 1.f;
      else if (c == COL_Y) v = y[r];
    }
    out[i] = v;
  }
}

cudaError_t launch_repack(const float* x, const float* y, float* out, long long n_rows,
                          long long rows_pad, int D, cudaStream_t st) {
  const long long total = rows_pad * KP;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  repack_kernel<<<blocks, 256, 0, st>>>(x, y, out, n_rows, rows_pad, D);
  return cudaGetLastError();
}

// ---- sum of a window's partial vectors, as doubles ------------------------------
// Used (a) when many CTAs touch one window (few windows per GPU): one small launch sums the
// slots once instead of every CTA of the next launch summing all of them in its prologue, and
// (b) for row sharding, where the result is what is all-reduced.  Fixed order: deterministic.
constexpr int RED_PARAMS = 32, RED_GROUPS = 32;  // every load of a thread is in flight at once
__global__ void __launch_bounds__(RED_PARAMS* RED_GROUPS)
reduce_partials_kernel(const float* __restrict__ partial, const double* __restrict__ ll_partial, int slices,
                       const int* __restrict__ nslot, int P, int Pp, double* __restrict__ red) {
  __shared__ float sg[RED_GROUPS][RED_PARAMS];
  __shared__ double sl[RED_GROUPS];
  const int win = blockIdx.y;
  const int ns = nslot ? nslot[win] : slices;
  const int pi = threadIdx.x % RED_PARAMS, gi = threadIdx.x / RED_PARAMS;
  const int p = blockIdx.x * RED_PARAMS + pi;
  double* r = red + (size_t)win * (Pp + 4);
  pdl_trigger();
  pdl_wait();
  float g = 0.f;
  if (p < P) {
    const float* src = partial + (size_t)win * slices * Pp + p;
#pragma unroll 8
    for (int s = gi; s < ns; s += RED_GROUPS) g += src[(size_t)s * Pp];
  }
  sg[gi][pi] = g;
  if (blockIdx.x == 0 && pi == 0) {
    double l = 0.0;
    for (int s = gi; s < ns; s += RED_GROUPS) l += ll_partial[(size_t)win * slices + s];
    sl[gi] = l;
  }
  __syncthreads();
  if (gi == 0) {
    if (p < P) {
      float t = sg[0][pi];
#pragma unroll
      for (int k = 1; k < RED_GROUPS; ++k) t += sg[k][pi];
      r[p] = (double)t;
    } else if (p < Pp) {
      r[p] = 0.0;
    }
    if (blockIdx.x == 0 && pi == 0) {
      double t = sl[0];
#pragma unroll
      for (int k = 1; k < RED_GROUPS; ++k) t += sl[k];
      r[Pp] = t;
      r[Pp + 1] = r[Pp + 2] = r[Pp + 3] = 0.0;
    }
  }
}

cudaError_t launch_reduce_partials(const float* partial, const double* ll_partial, int slices,
                                   const int* nslot, int P, int Pp, double* red, int windows,
                                   cudaStream_t st) {
  dim3 grid((Pp + RED_PARAMS - 1) / RED_PARAMS, windows);
  return launch_chain_kernel(reduce_partials_kernel, grid, dim3(RED_PARAMS * RED_GROUPS), 0, st, partial,
                             ll_partial, slices, nslot, P, Pp, red);
}

// ---- row sharding: this rank's sums and their all-reduce in ONE launch over peer memory ---------------
// The reference has no multi-GPU code; the mode its README table implies needs, per leapfrog step, the sum
// over ranks of P + 1 numbers.  A library all-reduce of 7.7 KB costs 12 us on 2 and about 25 us on 8 GPUs,
// more than the gradient evaluation itself.  Here CTA k owns parameters [32k, 32k + 32): it sums them
// over this rank's slots (as reduce_partials_kernel does) and stores each double into slot [rank] of
// EVERY rank's receive buffer with plain 8-byte stores over NVLink (peer pointers from CUDA IPC; no
// multicast, no bulk-copy engine).  Every 8-byte store carries 4 bytes of payload and the exchange's
// sequence number: an aligned 8-byte store arrives whole, so the receiver needs no separate flag and no
// fence, it simply re-reads a word until it shows the current sequence number (bounded), which costs one
// trip over the link instead of three.  Then the nranks contributions are added in rank order: every
// rank adds the same numbers in the same order, so the result is bit-identical everywhere, which the
// replicated accept decision relies on.  Receive buffers alternate between two halves (a rank can be at
// most one exchange ahead of the slowest).  Slices never wait for one another: no grid-wide barrier.
// One process per GPU: the ranks' kernels never share a GPU.
__device__ __forceinline__ void st_word(uint2* p, uint32_t payload, uint32_t seq) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(payload), "r"(seq) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__global__ void __launch_bounds__(RED_PARAMS* RED_GROUPS) oneshot_allreduce_kernel(const OneShotParams a) {
  static_assert(RED_PARAMS == ONESHOT_SLICE, "one CTA = one slice of 32 parameters");
  __shared__ float sg[RED_GROUPS][RED_PARAMS];
  __shared__ double sl[RED_GROUPS];
  const int pi = threadIdx.x % RED_PARAMS, gi = threadIdx.x / RED_PARAMS;
  const int p = blockIdx.x * RED_PARAMS + pi;
  const int vec = a.Pp + 4;
  pdl_trigger();
  pdl_wait();
  const uint32_t seq = *reinterpret_cast<volatile unsigned int*>(a.seq) + 1u;
  const int half = (int)(seq & 1u);
  const int ns = a.nslot ? a.nslot[0] : a.slices;
  // ---- this rank's sum of its slots ----
  float g = 0.f;
  if (p < a.P) {
    const float* src = a.partial + p;
#pragma unroll 8
    for (int s = gi; s < ns; s += RED_GROUPS) g += src[(size_t)s * a.Pp];
  }
  sg[gi][pi] = g;
  const bool ll_cta = (a.Pp / RED_PARAMS) == (int)blockIdx.x;  // the CTA whose slice holds element Pp
  if (ll_cta && pi == 0) {
    double l = 0.0;
    for (int s = gi; s < ns; s += RED_GROUPS) l += a.ll_partial[s];
    sl[gi] = l;
  }
  __syncthreads();
  if (gi == 0 && p < vec) {  // warp 0: one element of the vector per lane
    double mine = 0.0;
    if (p < a.P) {
      float t = sg[0][pi];
#pragma unroll
      for (int k = 1; k < RED_GROUPS; ++k) t += sg[k][pi];
      mine = (double)t;
    } else if (p == a.Pp) {
      double t = sl[0];
#pragma unroll
      for (int k = 1; k < RED_GROUPS; ++k) t += sl[k];
      mine = t;
    }
    // ---- to every rank (this one included): words [half][rank][p][0..1] ----
    const uint32_t lo = (uint32_t)__double_as_longlong(mine), hi = (uint32_t)(__double_as_longlong(mine) >> 32);
    const size_t w_mine = (((size_t)half * a.nranks + a.rank) * vec + p) * 2;
    for (int r = 0; r < a.nranks; ++r) {
      uint2* dst = a.peer_words[r] + w_mine;
      st_word(dst, lo, seq);
      st_word(dst + 1, hi, seq);
    }
    // ---- every rank's words for this element, in rank order (bounded wait on each) ----
    double t = 0.0;
    bool ok = true;
    for (int r = 0; r < a.nranks; ++r) {
      const uint2* src = a.local_words + (((size_t)half * a.nranks + r) * vec + p) * 2;
      uint2 w0 = ld_word(src), w1 = ld_word(src + 1);
      unsigned int it = 0;
      while (ok && (w0.y != seq || w1.y != seq)) {
        if (++it >= a.poll_limit) { ok = false; break; }
        w0 = ld_word(src);
        w1 = ld_word(src + 1);
      }
      t += __longlong_as_double((long long)(((unsigned long long)w1.x << 32) | w0.x));
    }
    if (!ok && a.status) atomicExch(a.status, 501);
    a.red[p] = (p < a.P || p == a.Pp) ? t : 0.0;
  }
  // ---- the launch's last CTA closes the exchange ----
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.done, 1u) == gridDim.x - 1) {
      *a.done = 0u;
      *a.seq = seq;
    }
  }
}
cudaError_t launch_oneshot_allreduce(const OneShotParams& p, cudaStream_t st) {
  const int n_sl = (p.Pp + 4 + ONESHOT_SLICE - 1) / ONESHOT_SLICE;
  return launch_chain_kernel(oneshot_allreduce_kernel, dim3(n_sl), dim3(RED_PARAMS * RED_GROUPS), 0, st, p);
}

// ---- drop-in accept ratio on caller buffers (kernel_helpers.h:153-188) ----
// Single CTA, fixed summation order, double accumulation.
__global__ void __launch_bounds__(1024) log_acpt_kernel(const float* __restrict__ prev_loss,
                                                        const float* __restrict__ new_loss,
                                                        long long n_loss,
                                                        const float* __restrict__ prev_mom,
                                                        const float* __restrict__ new_mom,
                                                        const float* __restrict__ grad_cur, int P,
                                                        float eps, float* __restrict__ out) {
  __shared__ double dsc[32];
  double acc = 0.0;
  for (long long i = threadIdx.x; i < n_loss; i += blockDim.x)
    acc += (double)new_loss[i] - (double)prev_loss[i];
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const float mf = fmaf(eps * 0.5f, grad_cur[p], new_mom[p]);
    const float m0 = prev_mom[p];
    acc += 0.5 * ((double)m0 * (double)m0 - (double)mf * (double)mf);
  }
  const double t = block_sum_f64(acc, dsc);
  if (threadIdx.x == 0) *out = (float)t;
}

cudaError_t launch_log_acpt(const float* prev_loss, const float* new_loss, long long n_loss,
                            const float* prev_mom, const float* new_mom, const float* grad_cur, int P,
                            float eps, float* out, cudaStream_t st) {
  log_acpt_kernel<<<1, 1024, 0, st>>>(prev_loss, new_loss, n_loss, prev_mom, new_mom, grad_cur, P,
                                      eps, out);
  return cudaGetLastError();
}

}  // namespace mcmc_b200

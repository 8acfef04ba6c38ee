// Launch parameter block of the accept kernel and the host-callable launchers
// shared between the translation units of the library.
#pragma once
#include "common.cuh"

namespace mcmc_b200 {

enum AcceptMode : int {
  ACC_BOOTSTRAP = 0,  // adopt the evaluated state as the chain's current state (main.h:191-202)
  ACC_ITERATE = 1,    // accept ratio, accept/reject, adaptation, store, next momentum
  ACC_FINALIZE = 2    // only assemble gradient and log-density sums for the caller
};

struct AcceptParams {
  int mode;
  int P, Pp;
  int slices;                // slots per window (stride, and count when nslot is null)
  const int* nslot;          // optional [windows]: slots in use
  const float* partial;      // [windows][slices][Pp] of the last gradient launch
  const double* ll_partial;  // [windows][slices]
  const double* red_in;      // row sharding: [windows][Pp + 4] all-reduced sums, else null
  const float* w_new;        // [windows][Pp] proposal position
  const float* m_new;        // [windows][Pp] proposal momentum (before the closing half kick)
  float* m0;                 // [windows][Pp] momentum drawn for the running iteration
  float* w_cur;              // [windows][Pp] chain state
  float* g_cur;              // [windows][Pp] full gradient at the chain state
  double* ll_cur;            // [windows]
  double* lp_cur;            // [windows]
  float* eps;                // [windows]
  int* iter;                 // [windows]
  int* n_accept;             // [windows]
  const long long* gwin;     // [windows] global window ids (random-stream keys)
  float* w_start;            // [windows][Pp] where the next iteration starts from
  float* m_start;            // [windows][Pp]
  float* samples;            // [windows][sample_capacity][P]
  int sample_capacity;
  int burn_in;
  int adapt_steps;
  float log_target, dec_adj, inc_adj;
  unsigned long long seed;
  // trace of the first trace_iters iterations
  int trace_iters;
  float* tr_mom;             // [windows][trace_iters][P]
  float* tr_log_u;           // [windows][trace_iters]
  double* tr_log_acpt;
  int* tr_accept;
  float* tr_eps;
  PriorParams prior;
  // ACC_FINALIZE outputs (single window)
  float* g_out;              // [P]
  float* prior_loss_out;     // optional [P]
  double* scalars_out;       // [2]: loglik, logprior
  const int* status_in;      // optional: device error word; when it is set the scalars come out as NaN
  // the reference's random streams instead of Philox (main.h:207-216, :235-239)
  int ref_streams;
  const float* ref_log_u;    // [ref_cap] host-computed log accept draws, indexed by iteration % ref_cap
  int ref_cap;
};

cudaError_t launch_accept(const AcceptParams& a, int windows, cudaStream_t st);
cudaError_t launch_repack(const float* x, const float* y, float* out, long long n_rows,
                          long long rows_pad, int D, cudaStream_t st);
cudaError_t launch_reduce_partials(const float* partial, const double* ll_partial, int slices,
                                   const int* nslot, int P, int Pp, double* red, int windows,
                                   cudaStream_t st);
// One-shot all-reduce over peer memory for row sharding (chain.cu): what every rank's launch needs
constexpr int ONESHOT_SLICE = 32;   // parameters per CTA
constexpr int ONESHOT_MAX_RANKS = 16;
struct OneShotParams {
  // this rank's partial vectors, as for reduce_partials
  const float* partial;
  const double* ll_partial;
  int slices;
  const int* nslot;
  int P, Pp;
  double* red;                  // [Pp + 4] result, identical bits on every rank
  int rank, nranks;
  // every rank's receive buffer (this rank's own at [rank]): [2 halves][nranks][Pp + 4][2] words of
  // {32 bits of payload, sequence number}
  uint2* peer_words[ONESHOT_MAX_RANKS];
  const uint2* local_words;
  unsigned int* seq;            // device counter of completed exchanges on this rank
  unsigned int* done;           // ticket of the CTAs of one launch
  unsigned int poll_limit;      // bounded wait: polls before giving up
  int* status;
};
cudaError_t launch_oneshot_allreduce(const OneShotParams& p, cudaStream_t st);
// forward-only pass over (samples x rows) (forward.cu)
struct ForwardParams {
  const float* x;          // rows, x_stride floats apart (22 for caller rows, 24 for the repacked dataset)
  long long x_stride;
  const float* y;          // LOSS only: targets, y_stride floats apart
  long long y_stride;
  long long n;             // rows
  const float* samples;    // [count][P]
  int count;
  LikParams lik;
  double* partial;         // PREDICT: [chunks][n]   LOSS: [row tiles][count]
};
int forward_row_tiles(long long n);
cudaError_t launch_forward_samples(int H, const ForwardParams& a, int chunks, bool loss, cudaStream_t st);
cudaError_t launch_forward_finish_predict(const double* partial, int chunks, long long n, int count, float* out,
                                          cudaStream_t st);
cudaError_t launch_forward_finish_loss(const double* partial, int tiles, int count, const float* samples, int P,
                                       const PriorParams& prior, double* out_ll, double* out_lp, cudaStream_t st);
cudaError_t launch_philox_probe(const uint32_t ctr[4], const uint32_t key[2], int n, uint32_t* raw, float* normals,
                                float* uniform, cudaStream_t st);
cudaError_t launch_refstream_momentum(unsigned long long first_n, int count, float* out, cudaStream_t st);
cudaError_t launch_wait_probe(int* status, unsigned int slices, cudaStream_t st);
cudaError_t launch_log_acpt(const float* prev_loss, const float* new_loss, long long n_loss,
                            const float* prev_mom, const float* new_mom, const float* grad_cur, int P,
                            float eps, float* out, cudaStream_t st);

// gradient kernels
cudaError_t launch_grad_fp32(int H, const GradParams& g, int slices, int windows, cudaStream_t st);
int fp32_max_ctas_per_sm(int H);
int fp32_tile_rows(int H);

// TF32 (tcgen05) path: persistent, one CTA per SM; `tmap_mn` is a CUtensorMap over the repacked
// dataset that stages a row tile with the 32-byte-chunk swizzle
cudaError_t launch_grad_tf32(int H, const void* tmap_mn, const GradParams& g, int ctas, cudaStream_t st);
int tf32_supported(int H);
int tf32_multistep_max_ctas(int H);
cudaError_t launch_grad_tf32_multistep(int H, const void* tmap_mn, const GradParams& g, int ctas,
                                       cudaStream_t st);
cudaError_t launch_grad_tf32_wide(const void* tmap_mn, const GradParams& g, int ctas, cudaStream_t st);
constexpr int TF32_TILE = 128;

}  // namespace mcmc_b200

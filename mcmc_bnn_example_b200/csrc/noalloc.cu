// mcmc_b200_potential_and_grad_static: log p and its gradient at w with NO
// device allocation anywhere on the call path.
//
// Who needs this.  Some hosts may not call cudaMalloc while they evaluate the
// model: a sampler embedded in a service whose GPU memory is owned entirely by
// the host application's own arena (a second allocator fragments or exhausts
// it), or a latency-critical loop in which cudaMalloc/cudaFree are off limits
// because they synchronise the whole device and stall every other stream.  The
// regular entry points keep their scratch in buffers that mcmc_b200_create
// allocates; this one keeps it in a fixed array that is part of the library
// image instead, so it needs no context and allocates nothing.
//
// The scratch (the repacked copy of the dataset and the per-CTA partial
// gradient vectors the FP32 gradient kernel writes before they are summed) lives
// in `g_static_scratch` below: about 7.7 MB that every GPU which loads this
// library holds until the process exits.  Limits that follow from its size:
// rows <= 65536, D = 22, H = 40, FP32 mode.  Larger requests are refused.
//
// One array per GPU, shared by all calls: it keeps the previous call's contents
// (everything a call reads it first overwrites, and the status word is cleared
// on every call), and two calls that overlap on the same GPU — different
// streams, or different host threads — race on it.  Serialise them.
//
// Errors after the call has returned: the call only queues work.  If a bounded
// device-side wait runs out, the kernel records it in the scratch's status word
// and the last kernel of the call writes NaN into both output scalars, so a
// caller that cannot query anything else still sees that the result is void.
#include <cuda_runtime.h>
#include <math.h>
#include <string.h>

#include <string>

#include "../../include/mcmc_b200.h"
#include "chain.cuh"
#include "common.cuh"

using namespace mcmc_b200;

namespace {

constexpr long long STATIC_MAX_ROWS = 65536;
constexpr int STATIC_MAX_SLOTS = 296;  // 2 CTAs on each of 148 SMs
constexpr int STATIC_P = 961, STATIC_PP = 964;
constexpr size_t XAUG_BYTES = (size_t)STATIC_MAX_ROWS * KP * sizeof(float);
constexpr size_t PARTIAL_BYTES = (size_t)STATIC_MAX_SLOTS * STATIC_PP * sizeof(float);
constexpr size_t LL_BYTES = (size_t)STATIC_MAX_SLOTS * sizeof(double);
constexpr size_t STATUS_BYTES = 256;
constexpr size_t SCRATCH_BYTES = XAUG_BYTES + PARTIAL_BYTES + LL_BYTES + STATUS_BYTES;

// In host code this name is only a handle for the runtime, NOT a device
// address: kernels get the address that cudaGetSymbolAddress returns.
static __device__ __align__(256) unsigned char g_static_scratch[SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
unsigned char* g_scratch_ptr[MAX_DEVICES] = {};
int g_num_sms[MAX_DEVICES] = {};


}  // namespace

// defined in api.cu: the library-wide last-error text
extern "C" const char* mcmc_b200_last_error(void);
void mcmc_b200_set_last_error(const std::string& msg);

static int fail_static(int code, const std::string& msg) {
  mcmc_b200_set_last_error(msg);
  return code;
}

extern "C" __attribute__((visibility("default"))) int mcmc_b200_potential_and_grad_static(
    const mcmc_b200_config* cfg, const float* x, const float* y, int64_t rows, const float* w, float* grad,
    double* loglik_logprior, void* stream) {
  if (!cfg || !x || !y || !w || !grad || !loglik_logprior || rows < 1)
    return fail_static(MCMC_B200_ERR_INVALID, "bad arguments");
  if (cfg->D != 22 || cfg->H != 40 || cfg->precision != MCMC_B200_PREC_FP32)
    return fail_static(MCMC_B200_ERR_UNSUPPORTED,
                       "the allocation-free entry point is built for D = 22, H = 40, FP32 mode only");
  if (rows > STATIC_MAX_ROWS)
    return fail_static(MCMC_B200_ERR_INVALID,
                       "rows exceeds the static scratch of the allocation-free entry point (max 65536)");
  if (cfg->lik_scale <= 0 || cfg->prior_scale <= 0)
    return fail_static(MCMC_B200_ERR_INVALID, "bad model constants");
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
    return fail_static(MCMC_B200_ERR_CUDA, "no current CUDA device");
  // Set-up, once per device, with that device current: the address of this
  // device's copy of the array.  It happens on the FIRST call on a device, so
  // that call should come before any stream capture.
  if (!g_scratch_ptr[dev]) {
    unsigned char* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
    if (e != cudaSuccess || !p)
      return fail_static(MCMC_B200_ERR_CUDA, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || sms < 1) return fail_static(MCMC_B200_ERR_CUDA, "cannot query the SM count");
    g_num_sms[dev] = sms;
    g_scratch_ptr[dev] = p;
  }
  unsigned char* base = g_scratch_ptr[dev];
  float* xaug = reinterpret_cast<float*>(base);
  float* partial = reinterpret_cast<float*>(base + XAUG_BYTES);
  double* llp = reinterpret_cast<double*>(base + XAUG_BYTES + PARTIAL_BYTES);
  int* status = reinterpret_cast<int*>(base + XAUG_BYTES + PARTIAL_BYTES + LL_BYTES);
  cudaStream_t st = (cudaStream_t)stream;

  const int tile = fp32_tile_rows(cfg->H);
  const long long rows_pad = (rows + TF32_TILE - 1) / TF32_TILE * TF32_TILE;
  const long long n_tiles = rows_pad / tile;
  long long slots = 2LL * g_num_sms[dev];
  if (slots > STATIC_MAX_SLOTS) slots = STATIC_MAX_SLOTS;
  if (slots > n_tiles) slots = n_tiles;

  // the status word must start at zero; everything else a call reads it first writes
  e = cudaMemsetAsync(status, 0, sizeof(int), st);
  if (e != cudaSuccess) return fail_static(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
  e = launch_repack(x, y, xaug, rows, rows_pad, cfg->D, st);
  if (e != cudaSuccess) return fail_static(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));

  const double pi = 3.14159265358979323846;
  GradParams g;
  memset(&g, 0, sizeof g);
  g.xaug = xaug;
  g.window_stride = rows_pad * KP;
  g.n_rows = (int)rows;
  g.n_tiles = (int)n_tiles;
  g.P = STATIC_P;
  g.Pp = STATIC_PP;
  g.w_in = w;
  g.mode = MODE_EVAL;
  g.slices_in = g.slices_out = (int)slots;
  g.partial_out = partial;
  g.ll_out = llp;
  g.status = status;
  g.data_fresh = 1;  // the repack above wrote xaug: the kernel fetches no row ahead of its dependency wait
  g.lik.kind = cfg->likelihood;
  g.lik.inv_scale = (float)(1.0 / cfg->lik_scale);
  if (cfg->likelihood == MCMC_B200_LIK_STUDENT_T) {
    g.lik.df = (float)cfg->lik_df;
    g.lik.inv_df = (float)(1.0 / cfg->lik_df);
    g.lik.norm = (float)(log(fabs(cfg->lik_scale)) + 0.5 * log(cfg->lik_df) + 0.5 * log(pi) +
                         lgamma(0.5 * cfg->lik_df) - lgamma(0.5 * (cfg->lik_df + 1.0)));
    g.lik.g_scale = (float)((cfg->lik_df + 1.0) / cfg->lik_scale);
    g.lik.l_scale = (float)(-0.5 * (cfg->lik_df + 1.0));
  } else {
    g.lik.norm = (float)(0.5 * log(2.0 * pi) + log(cfg->lik_scale));
    g.lik.g_scale = (float)(1.0 / cfg->lik_scale);
    g.lik.l_scale = -0.5f;
  }
  g.prior.neg_inv_s2 = (float)(-1.0 / (cfg->prior_scale * cfg->prior_scale));
  g.prior.inv_s = (float)(1.0 / cfg->prior_scale);
  g.prior.norm = (float)(0.5 * log(2.0 * pi) + log(cfg->prior_scale));
  e = launch_grad_fp32(cfg->H, g, (int)slots, 1, st);
  if (e != cudaSuccess) return fail_static(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));

  AcceptParams a;
  memset(&a, 0, sizeof a);
  a.mode = ACC_FINALIZE;
  a.P = STATIC_P;
  a.Pp = STATIC_PP;
  a.slices = (int)slots;
  a.partial = partial;
  a.ll_partial = llp;
  a.w_new = w;
  a.prior = g.prior;
  a.g_out = grad;
  a.scalars_out = loglik_logprior;
  a.status_in = status;  // a wait that ran out turns both scalars into NaN: the caller sees it in the result
  e = launch_accept(a, 1, st);
  if (e != cudaSuccess) return fail_static(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
  return MCMC_B200_OK;
}

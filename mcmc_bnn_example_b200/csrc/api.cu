// C-ABI of the library (declared in include/mcmc_b200.h): context and buffer
// management, launch sequencing of the gradient / accept kernels, CUDA-graph
// replay of whole HMC iterations, the optional NCCL allreduce for row sharding.
// Host-side counterpart of the reference's main_loop / Network / mcmc_step
// (include/mcmc/main.h:48-76, :117-308; mcmc_step_ffma.h:395-427).
#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <limits>
#include <random>
#include <string>
#include <vector>

#include <thrust/random.h>

#include "../../include/mcmc_b200.h"
#include "chain.cuh"
#include "common.cuh"
#include "philox.h"

using namespace mcmc_b200;

#define API extern "C" __attribute__((visibility("default")))

static thread_local std::string g_last_error;
// the one-launch-per-iteration path for single-window contexts: opt-in (MCMC_B200_MULTISTEP=1) while
// false, opt-out (MCMC_B200_NO_MULTISTEP=1) while true
static constexpr bool MULTISTEP_DEFAULT = false;

static int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}
// for the other translation units of the library
void mcmc_b200_set_last_error(const std::string& msg) { g_last_error = msg; }

#define CK(call)                                                                              \
  do {                                                                                        \
    cudaError_t e_ = (call);                                                                  \
    if (e_ != cudaSuccess)                                                                    \
      return fail(MCMC_B200_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e_));    \
  } while (0)

// ---- NCCL through dlopen: no link-time dependency, and the copy already
// loaded into the process (for instance by torch) is the one that is used ----
namespace {
struct NcclUniqueId { char internal[128]; };
typedef void* NcclComm;
struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitRank)(NcclComm*, int, NcclUniqueId, int) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, NcclComm, cudaStream_t) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  bool ok = false;
};
NcclApi g_nccl;

bool nccl_load(std::string* why) {
  if (g_nccl.ok) return true;
  const char* env = getenv("MCMC_B200_NCCL_LIB");
  const char* names[] = {env, "libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    if (!n) continue;
    g_nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (g_nccl.handle) break;
  }
  if (!g_nccl.handle) {
    *why = std::string("dlopen(libnccl.so.2) failed: ") + dlerror();
    return false;
  }
  g_nccl.GetUniqueId = (int (*)(NcclUniqueId*))dlsym(g_nccl.handle, "ncclGetUniqueId");
  g_nccl.CommInitRank = (int (*)(NcclComm*, int, NcclUniqueId, int))dlsym(g_nccl.handle, "ncclCommInitRank");
  g_nccl.AllReduce = (int (*)(const void*, void*, size_t, int, int, NcclComm, cudaStream_t))dlsym(
      g_nccl.handle, "ncclAllReduce");
  g_nccl.AllGather = (int (*)(const void*, void*, size_t, int, NcclComm, cudaStream_t))dlsym(g_nccl.handle,
                                                                                         "ncclAllGather");
  g_nccl.CommDestroy = (int (*)(NcclComm))dlsym(g_nccl.handle, "ncclCommDestroy");
  g_nccl.GetErrorString = (const char* (*)(int))dlsym(g_nccl.handle, "ncclGetErrorString");
  if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllReduce || !g_nccl.CommDestroy) {
    *why = "NCCL symbols missing";
    return false;
  }
  g_nccl.ok = true;
  return true;
}
constexpr int kNcclFloat64 = 8;
constexpr int kNcclChar = 0;
constexpr int kNcclSum = 0;
}  // namespace

struct mcmc_b200_ctx {
  mcmc_b200_config cfg;
  int device = 0, W = 0, P = 0, Pp = 0;
  long long rows = 0, rows_pad = 0;
  int num_sms = 0, ctas_per_sm = 1;
  bool use_red = false, use_red_x = false;  // sum partial slots with a separate small launch
  int slices = 1;      // CTAs per window in chain launches
  int slices_x = 1;    // CTAs for single-window explicit calls
  int tile_rows = 64;
  cudaStream_t stream = nullptr;
  // dataset
  float* xaug = nullptr;
  std::vector<char> window_set;
  CUtensorMap tmap_mn;
  bool tmap_ok = false;
  // persistent (TF32) kernel work tables: chain launches and single-window launches
  int *tab_seg_ptr = nullptr, *tab_nslot = nullptr, *xtab_seg_ptr = nullptr, *xtab_nslot = nullptr;
  int4 *tab_segs = nullptr, *xtab_segs = nullptr;
  int tab_ctas = 0, xtab_ctas = 0;
  // chain state
  float *wbuf[2] = {}, *mbuf[2] = {}, *w_cur = nullptr, *g_cur = nullptr, *m0 = nullptr;
  float* partial[2] = {};
  double* llp[2] = {};
  double *red = nullptr, *ll_cur = nullptr, *lp_cur = nullptr;
  float* eps = nullptr;
  int *iter = nullptr, *n_accept = nullptr;
  long long* gwin = nullptr;
  float* samples = nullptr;
  float *tr_mom = nullptr, *tr_log_u = nullptr, *tr_eps = nullptr;
  double* tr_log_acpt = nullptr;
  int* tr_accept = nullptr;
  int* status = nullptr;
  std::vector<long long> h_gwin;
  bool bootstrapped = false;
  int iters_done = 0;
  // explicit-state scratch (one window)
  float *xw[2] = {}, *xm[2] = {}, *xg = nullptr, *xpartial[2] = {}, *g_out = nullptr, *row_loss = nullptr;
  float* scalar_f = nullptr;
  double *xllp[2] = {}, *xred = nullptr, *scalars = nullptr;
  // bound dataset of the drop-in mcmc_step
  const float *bound_x = nullptr, *bound_y = nullptr;
  // graph of one HMC iteration
  cudaGraphExec_t graph_exec = nullptr;
  bool graph_tried = false;
  // row sharding
  NcclComm comm = nullptr;
  int nranks = 1, rank = 0;
  // ... with the one-shot all-reduce over peer memory instead of the NCCL call
  bool oneshot = false;
  void* os_block = nullptr;                 // this rank's receive buffer + flags (one allocation, IPC-exported)
  std::vector<void*> os_peer_blocks;        // the peers' blocks as mapped here (null at [rank])
  std::vector<void*> os_base;               // every rank's block as seen from here (own block at [rank])
  unsigned int *os_seq = nullptr, *os_done = nullptr;
  unsigned int os_poll_limit = 1u << 22;    // polls of about 0.1 us .. 1 us each
  long long launches = 0;
  // all L leapfrog steps of an iteration in one cooperative launch (one window, TF32, H = 40)
  bool multistep = false;
  unsigned int* grid_bar = nullptr;
  float* stage = nullptr;  // upload staging for one window: [rows][D] then [rows]
  // forward-only pass over the stored samples: scratch that grows on demand and is kept (no allocation per call)
  float* fwd_x = nullptr;
  float* fwd_out = nullptr;
  double* fwd_partial = nullptr;
  size_t fwd_x_cap = 0, fwd_out_cap = 0, fwd_partial_cap = 0;
  // the reference's random streams: host-computed log accept draws, indexed by iteration
  float* ref_log_u = nullptr;
  int ref_cap = 0, ref_filled = 0;
  std::vector<void*> allocs;
};

static int dalloc(mcmc_b200_ctx* c, void** p, size_t bytes, bool zero = true) {
  if (bytes == 0) bytes = 16;
  cudaError_t e = cudaMalloc(p, bytes);
  if (e != cudaSuccess) return fail(MCMC_B200_ERR_NOMEM, std::string("cudaMalloc: ") + cudaGetErrorString(e));
  c->allocs.push_back(*p);
  if (zero) {
    e = cudaMemset(*p, 0, bytes);
    if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, std::string("cudaMemset: ") + cudaGetErrorString(e));
  }
  return MCMC_B200_OK;
}
#define DA(ptr, bytes)                                                   \
  do {                                                                   \
    int r_ = dalloc(c, (void**)&(ptr), (bytes));                         \
    if (r_ != MCMC_B200_OK) { mcmc_b200_destroy(c); return r_; }         \
  } while (0)

API const char* mcmc_b200_last_error(void) { return g_last_error.c_str(); }
API int mcmc_b200_has_tf32(void) { return tf32_supported(40); }

API void mcmc_b200_config_reference(mcmc_b200_config* cfg) {
  memset(cfg, 0, sizeof(*cfg));
  cfg->D = 22; cfg->H = 40;
  cfg->likelihood = MCMC_B200_LIK_STUDENT_T;
  cfg->precision = MCMC_B200_PREC_FP32;
  cfg->lik_scale = 100.0; cfg->lik_df = 2.2; cfg->prior_scale = 200.0;
  cfg->leapfrog_steps = 1000; cfg->burn_in = 100; cfg->adapt_steps = 100; cfg->sample_capacity = 800;
  cfg->eps0 = 0.01; cfg->target_rate = 0.2; cfg->decrement = 0.1; cfg->increment = 0.01;
  cfg->seed = 0; cfg->trace_iters = 0; cfg->slices = 0;
  cfg->rng_streams = MCMC_B200_RNG_PHILOX;
}
API void mcmc_b200_config_baseline(mcmc_b200_config* cfg) {
  mcmc_b200_config_reference(cfg);
  cfg->likelihood = MCMC_B200_LIK_GAUSSIAN;
  cfg->lik_scale = 1.0; cfg->lik_df = 0.0; cfg->prior_scale = 1.0;
  cfg->leapfrog_steps = 10; cfg->burn_in = 0; cfg->adapt_steps = 0;
  cfg->eps0 = 1e-3;
}

static LikParams make_lik(const mcmc_b200_config& cfg) {
  LikParams l;
  const double pi = 3.14159265358979323846;
  l.kind = cfg.likelihood;
  l.inv_scale = (float)(1.0 / cfg.lik_scale);
  if (cfg.likelihood == MCMC_B200_LIK_STUDENT_T) {
    l.df = (float)cfg.lik_df;
    l.inv_df = (float)(1.0 / cfg.lik_df);
    l.norm = (float)(log(fabs(cfg.lik_scale)) + 0.5 * log(cfg.lik_df) + 0.5 * log(pi) +
                     lgamma(0.5 * cfg.lik_df) - lgamma(0.5 * (cfg.lik_df + 1.0)));
    l.g_scale = (float)((cfg.lik_df + 1.0) / cfg.lik_scale);
    l.l_scale = (float)(-0.5 * (cfg.lik_df + 1.0));
  } else {
    l.df = 0.f;
    l.inv_df = 0.f;
    l.norm = (float)(0.5 * log(2.0 * pi) + log(cfg.lik_scale));
    l.g_scale = (float)(1.0 / cfg.lik_scale);
    l.l_scale = -0.5f;
  }
  return l;
}
static PriorParams make_prior(const mcmc_b200_config& cfg) {
  PriorParams p;
  const double pi = 3.14159265358979323846;
  p.neg_inv_s2 = (float)(-1.0 / (cfg.prior_scale * cfg.prior_scale));
  p.inv_s = (float)(1.0 / cfg.prior_scale);
  p.norm = (float)(0.5 * log(2.0 * pi) + log(cfg.prior_scale));
  return p;
}

static int make_tensor_map(mcmc_b200_ctx* c) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                               CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                               CUtensorMapFloatOOBfill);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
  if (!fn || qres != cudaDriverEntryPointSuccess)
    return fail(MCMC_B200_ERR_CUDA, "cuTensorMapEncodeTiled not available");
  // [W * rows_pad][24] floats; the box is 32 floats wide so that a staged row
  // is a full 128-byte swizzle span: columns 24..31 are out of bounds and
  // arrive as zeros without being read.
  cuuint64_t gdim[2] = {(cuuint64_t)KP, (cuuint64_t)((long long)c->W * c->rows_pad)};
  cuuint64_t gstride[1] = {(cuuint64_t)(KP * sizeof(float))};
  cuuint32_t box[2] = {32, (cuuint32_t)TF32_TILE};
  cuuint32_t estr[2] = {1, 1};
  // 32-byte-chunk swizzle: the layout the tensor core wants for MN-major TF32 operands
  CUresult r = ((EncodeFn)fn)(&c->tmap_mn, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, c->xaug, gdim, gstride, box,
                              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char b[96];
    snprintf(b, sizeof b, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return fail(MCMC_B200_ERR_CUDA, b);
  }
  c->tmap_ok = true;
  return MCMC_B200_OK;
}

// Cuts the flattened (window, tile) list of a launch into one contiguous range per CTA and each
// range into per-window segments; slot = the segment's index among its window's segments.
static int build_work_table(mcmc_b200_ctx* c, int windows, long long tiles_per_window, int max_ctas,
                            int chunks_per_window, int** d_seg_ptr, int4** d_segs, int** d_nslot,
                            int* n_ctas, int* max_slots);

API int mcmc_b200_create(const mcmc_b200_config* cfg, int device, int n_windows, int64_t rows,
                         mcmc_b200_ctx** out) {
  if (!cfg || !out || n_windows < 1 || rows < 1) return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  if (cfg->D != 22) return fail(MCMC_B200_ERR_UNSUPPORTED, "only D = 22 is built");
  if (cfg->H != 40 && cfg->H != 128) return fail(MCMC_B200_ERR_UNSUPPORTED, "only H = 40 or 128 is built");
  if (cfg->precision == MCMC_B200_PREC_TF32 && !tf32_supported(cfg->H))
    return fail(MCMC_B200_ERR_UNSUPPORTED, "the TF32 path is not built for this hidden width");
  if (cfg->leapfrog_steps < 1 || cfg->lik_scale <= 0 || cfg->prior_scale <= 0)
    return fail(MCMC_B200_ERR_INVALID, "bad sampler/model constants");
  if (cfg->rng_streams != MCMC_B200_RNG_PHILOX && cfg->rng_streams != MCMC_B200_RNG_REFERENCE)
    return fail(MCMC_B200_ERR_INVALID, "rng_streams must be MCMC_B200_RNG_PHILOX or MCMC_B200_RNG_REFERENCE");
  if (n_windows > 65535) return fail(MCMC_B200_ERR_INVALID, "at most 65535 windows per context");
  {
    // the kernels index rows of the whole context with 32-bit integers (TMA coordinates, tile numbers)
    const long long rp = (rows + TF32_TILE - 1) / TF32_TILE * TF32_TILE;
    if (rows > 0x7fffffffLL - TF32_TILE || rp * (long long)n_windows > 0x7fffffffLL)
      return fail(MCMC_B200_ERR_INVALID, "rows per window x windows must stay below 2^31 rows per context");
  }
  int ndev = 0;
  cudaError_t e0 = cudaGetDeviceCount(&ndev);
  if (e0 != cudaSuccess || ndev == 0)
    return fail(MCMC_B200_ERR_CUDA, "no CUDA device: this library has no CPU path");
  if (device < 0 || device >= ndev) return fail(MCMC_B200_ERR_INVALID, "device ordinal out of range");
  CK(cudaSetDevice(device));
  cudaDeviceProp prop;
  CK(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(MCMC_B200_ERR_UNSUPPORTED, "kernels are built for sm_100a (B200) only");

  mcmc_b200_ctx* c = new mcmc_b200_ctx();
  c->cfg = *cfg;
  c->device = device;
  c->W = n_windows;
  c->rows = rows;
  c->rows_pad = (rows + TF32_TILE - 1) / TF32_TILE * TF32_TILE;
  c->P = cfg->D * cfg->H + 2 * cfg->H + 1;
  c->Pp = (c->P + 3) / 4 * 4;
  c->num_sms = prop.multiProcessorCount;
  const bool tf32 = cfg->precision == MCMC_B200_PREC_TF32;
  c->tile_rows = tf32 ? TF32_TILE : fp32_tile_rows(cfg->H);
  c->ctas_per_sm = tf32 ? 1 : fp32_max_ctas_per_sm(cfg->H);
  if (c->ctas_per_sm < 1) c->ctas_per_sm = 1;
  const long long n_tiles = c->rows_pad / c->tile_rows;
  c->window_set.assign(n_windows, 0);
  c->h_gwin.assign(n_windows, 0);
  cudaError_t es = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
  if (es != cudaSuccess) { delete c; return fail(MCMC_B200_ERR_CUDA, "cudaStreamCreate failed"); }
  if (tf32) {
    // persistent kernel: by default every CTA gets an equal share of the launch's tiles, so where a
    // window is cut depends on how many windows share the launch.  cfg.slices > 0 instead cuts every
    // window into that many fixed chunks (whole chunks per CTA): a window's result is then bit-identical
    // wherever and with whatever else it runs, at some cost in load balance.
    int r_ = build_work_table(c, n_windows, n_tiles, c->num_sms, cfg->slices, &c->tab_seg_ptr, &c->tab_segs,
                              &c->tab_nslot, &c->tab_ctas, &c->slices);
    if (r_ == MCMC_B200_OK)
      r_ = build_work_table(c, 1, n_tiles, c->num_sms, cfg->slices, &c->xtab_seg_ptr, &c->xtab_segs,
                            &c->xtab_nslot, &c->xtab_ctas, &c->slices_x);
    if (r_ != MCMC_B200_OK) { mcmc_b200_destroy(c); return r_; }
  } else {
    const long long capacity = (long long)c->num_sms * c->ctas_per_sm;
    // the fewest CTAs per window that keep the longest CTA as short as `cap` CTAs would: fewer partial
    // vectors to sum and fewer per-CTA prologues for the same critical path
    auto balanced = [&](long long cap) {
      if (cap < 1) cap = 1;
      if (cap > n_tiles) cap = n_tiles;
      if (cap > MAX_SLICES) cap = MAX_SLICES;
      const long long tiles_per_cta = (n_tiles + cap - 1) / cap;
      return (n_tiles + tiles_per_cta - 1) / tiles_per_cta;
    };
    long long s = cfg->slices > 0 ? cfg->slices : balanced(capacity / n_windows);
    if (s < 1) s = 1;
    if (s > n_tiles) s = n_tiles;
    if (s > MAX_SLICES) s = MAX_SLICES;
    c->slices = (int)s;
    long long sx = cfg->slices > 0 ? cfg->slices : balanced(capacity);
    if (sx > n_tiles) sx = n_tiles;
    if (sx > MAX_SLICES) sx = MAX_SLICES;
    if (sx < 1) sx = 1;
    c->slices_x = (int)sx;
  }

  // many slots per window (few windows per GPU): one small launch sums them once per step instead of
  // every CTA of the next launch summing all of them in its prologue
  c->use_red = c->slices > 4;
  c->use_red_x = c->slices_x > 4;
  {
    // one window on the whole GPU: run the L steps of an iteration as ONE cooperative launch (the CTAs
    // meet at a grid barrier after every step).  Needs every CTA resident, the sums in `red` (use_red) and
    // the free partition (a fixed `slices` asks for placement-independent bits: keep one launch per step).
    const char* off = getenv("MCMC_B200_NO_MULTISTEP");
    const char* on = getenv("MCMC_B200_MULTISTEP");
    const bool want = MULTISTEP_DEFAULT ? !(off && off[0] == '1') : (on && on[0] == '1');
    c->multistep = tf32 && n_windows == 1 && cfg->slices == 0 && c->use_red && cfg->leapfrog_steps >= 2 &&
                   want && c->tab_ctas > 0 && c->tab_ctas <= tf32_multistep_max_ctas(cfg->H) &&
                   (c->P + c->tab_ctas - 1) / c->tab_ctas <= 12;
  }
  const size_t W = n_windows, Pp = c->Pp, P = c->P;
  DA(c->xaug, W * c->rows_pad * KP * sizeof(float));
  for (int i = 0; i < 2; ++i) {
    DA(c->wbuf[i], W * Pp * 4);
    DA(c->mbuf[i], W * Pp * 4);
    DA(c->partial[i], W * c->slices * Pp * 4);
    DA(c->llp[i], W * c->slices * 8);
    DA(c->xw[i], Pp * 4);
    DA(c->xm[i], Pp * 4);
    DA(c->xpartial[i], (size_t)c->slices_x * Pp * 4);
    DA(c->xllp[i], (size_t)c->slices_x * 8);
  }
  DA(c->w_cur, W * Pp * 4);
  DA(c->g_cur, W * Pp * 4);
  DA(c->m0, W * Pp * 4);
  DA(c->red, W * (Pp + 4) * 8);
  DA(c->xred, (Pp + 4) * 8);
  DA(c->ll_cur, W * 8);
  DA(c->lp_cur, W * 8);
  DA(c->eps, W * 4);
  DA(c->iter, W * 4);
  DA(c->n_accept, W * 4);
  DA(c->gwin, W * 8);
  DA(c->status, 4);
  DA(c->grid_bar, 4);
  DA(c->xg, Pp * 4);
  DA(c->g_out, Pp * 4);
  DA(c->row_loss, (size_t)c->rows_pad * 4);
  DA(c->scalars, 4 * 8);
  DA(c->scalar_f, 16);
  if (cfg->sample_capacity > 0) {
    int r_ = dalloc(c, (void**)&c->samples, W * (size_t)cfg->sample_capacity * P * 4, false);
    if (r_ != MCMC_B200_OK) { mcmc_b200_destroy(c); return r_; }
  }
  if (cfg->trace_iters > 0) {
    const size_t K = cfg->trace_iters;
    DA(c->tr_mom, W * K * P * 4);
    DA(c->tr_log_u, W * K * 4);
    DA(c->tr_log_acpt, W * K * 8);
    DA(c->tr_accept, W * K * 4);
    DA(c->tr_eps, W * K * 4);
  }
  if (tf32) {
    int r_ = make_tensor_map(c);
    if (r_ != MCMC_B200_OK) { mcmc_b200_destroy(c); return r_; }
  }
  std::vector<float> e(W, (float)cfg->eps0);
  cudaMemcpy(c->eps, e.data(), W * 4, cudaMemcpyHostToDevice);
  *out = c;
  return MCMC_B200_OK;
}

// Host-only planner of the persistent kernels' work table: which (window, tile range, slot) segments each
// CTA owns.  Pure arithmetic (no CUDA): also exported for inspection and CPU tests.
static void plan_work_table(int windows, long long tiles_per_window, int max_ctas, int chunks_per_window,
                            std::vector<int>& seg_ptr, std::vector<int4>& segs, std::vector<int>& nslot) {
  const long long T = (long long)windows * tiles_per_window;
  seg_ptr.clear();
  segs.clear();
  nslot.assign(windows, 0);
  long long G;
  if (chunks_per_window > 0) {
    long long cpw = std::min<long long>(std::min<long long>(chunks_per_window, tiles_per_window), MAX_SLICES);
    const long long NC = (long long)windows * cpw;
    G = std::min<long long>(max_ctas, NC);
    seg_ptr.assign(G + 1, 0);
    for (long long b = 0; b < G; ++b) {
      seg_ptr[b] = (int)segs.size();
      for (long long ch = b * NC / G; ch < (b + 1) * NC / G; ++ch) {
        const long long w = ch / cpw, k = ch % cpw;
        segs.push_back(make_int4((int)w, (int)(k * tiles_per_window / cpw), (int)((k + 1) * tiles_per_window / cpw),
                                 (int)k));
        nslot[w] = (int)cpw;
      }
    }
  } else {
    // Contiguous ranges of the flattened (window, tile) list, balanced by COST rather than by tile
    // count: every segment a CTA starts (a new window inside its range) costs a fixed prologue + drain +
    // read-out, worth about `seg_cost` tiles.  A CTA whose range crosses a window boundary therefore
    // gets fewer tiles than one that stays inside a window.  The smallest per-CTA budget that covers
    // all tiles with at most max_ctas CTAs is found by bisection over a greedy walk.
    // measured with the current kernel (a tile is 0.53 us): 25-window step 0.5135 (8) -> 0.5063 (11) -> 0.5035 ms
    // (14), flat up to 24; 13 windows 0.284 -> 0.282; 50, 100 and 200 windows unchanged within 0.5 %
    const double seg_cost = 14.0;
    const long long tpw = tiles_per_window;
    const long long Gmax = std::max<long long>(1, std::min<long long>(max_ctas, T));
    auto walk = [&](double budget_per_cta, bool emit) -> long long {
      long long pos = 0, used = 0;
      while (pos < T) {
        if (emit) seg_ptr.push_back((int)segs.size());
        double budget = budget_per_cta;
        bool first = true;
        while (pos < T) {
          long long can = (long long)std::floor(budget - seg_cost + 1e-9);
          if (can < 1) {
            if (!first) break;
            can = 1;  // a CTA always takes at least one tile
          }
          const long long w = pos / tpw;
          const long long take = std::min(can, (w + 1) * tpw - pos);
          if (emit)
            segs.push_back(make_int4((int)w, (int)(pos - w * tpw), (int)(pos + take - w * tpw), nslot[w]++));
          pos += take;
          budget -= seg_cost + (double)take;
          first = false;
        }
        if (++used > 4 * Gmax + 16) break;  // cannot happen for a budget >= the lower bound
      }
      return used;
    };
    double lo = (double)T / (double)Gmax, hi = (double)T / (double)Gmax + seg_cost * ((double)(T / Gmax) / tpw + 3.0) + 2.0;
    while (walk(hi, false) > Gmax) hi *= 1.5;
    for (int it = 0; it < 48; ++it) {
      const double mid = 0.5 * (lo + hi);
      if (walk(mid, false) <= Gmax) hi = mid; else lo = mid;
    }
    G = walk(hi, true);
  }
  seg_ptr.resize(G + 1);
  seg_ptr[G] = (int)segs.size();
}

static int build_work_table(mcmc_b200_ctx* c, int windows, long long tiles_per_window, int max_ctas,
                            int chunks_per_window, int** d_seg_ptr, int4** d_segs, int** d_nslot,
                            int* n_ctas, int* max_slots) {
  std::vector<int> seg_ptr, nslot;
  std::vector<int4> segs;
  plan_work_table(windows, tiles_per_window, max_ctas, chunks_per_window, seg_ptr, segs, nslot);
  const long long G = (long long)seg_ptr.size() - 1;
  int ms = 1;
  for (int w = 0; w < windows; ++w) ms = std::max(ms, nslot[w]);
  int r = dalloc(c, (void**)d_seg_ptr, seg_ptr.size() * sizeof(int), false);
  if (r == MCMC_B200_OK) r = dalloc(c, (void**)d_segs, segs.size() * sizeof(int4), false);
  if (r == MCMC_B200_OK) r = dalloc(c, (void**)d_nslot, nslot.size() * sizeof(int), false);
  if (r != MCMC_B200_OK) return r;
  CK(cudaMemcpy(*d_seg_ptr, seg_ptr.data(), seg_ptr.size() * sizeof(int), cudaMemcpyHostToDevice));
  CK(cudaMemcpy(*d_segs, segs.data(), segs.size() * sizeof(int4), cudaMemcpyHostToDevice));
  CK(cudaMemcpy(*d_nslot, nslot.data(), nslot.size() * sizeof(int), cudaMemcpyHostToDevice));
  *n_ctas = (int)G;
  *max_slots = ms;
  return MCMC_B200_OK;
}

API int mcmc_b200_plan_work_table(int windows, int64_t tiles_per_window, int max_ctas, int slices,
                                  int32_t* seg_ptr_out, int seg_ptr_capacity, int32_t* segs_out,
                                  int segs_capacity, int32_t* n_ctas, int32_t* n_segs) {
  if (windows < 1 || tiles_per_window < 1 || max_ctas < 1 || slices < 0 || !n_ctas || !n_segs)
    return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  std::vector<int> seg_ptr, nslot;
  std::vector<int4> segs;
  plan_work_table(windows, tiles_per_window, max_ctas, slices, seg_ptr, segs, nslot);
  *n_ctas = (int32_t)seg_ptr.size() - 1;
  *n_segs = (int32_t)segs.size();
  if (seg_ptr_out) {
    if ((int)seg_ptr.size() > seg_ptr_capacity) return fail(MCMC_B200_ERR_INVALID, "seg_ptr_out too small");
    for (size_t i = 0; i < seg_ptr.size(); ++i) seg_ptr_out[i] = seg_ptr[i];
  }
  if (segs_out) {
    if ((int)segs.size() > segs_capacity) return fail(MCMC_B200_ERR_INVALID, "segs_out too small");
    for (size_t i = 0; i < segs.size(); ++i) {
      segs_out[4 * i] = segs[i].x;
      segs_out[4 * i + 1] = segs[i].y;
      segs_out[4 * i + 2] = segs[i].z;
      segs_out[4 * i + 3] = segs[i].w;
    }
  }
  return MCMC_B200_OK;
}

API void mcmc_b200_destroy(mcmc_b200_ctx* c) {
  if (!c) return;
  cudaSetDevice(c->device);
  if (c->stream) cudaStreamSynchronize(c->stream);
  if (c->graph_exec) cudaGraphExecDestroy(c->graph_exec);
  for (void* p : c->os_peer_blocks)
    if (p) cudaIpcCloseMemHandle(p);
  if (c->comm && g_nccl.ok) g_nccl.CommDestroy(c->comm);
  for (void* p : c->allocs) cudaFree(p);
  if (c->stream) cudaStreamDestroy(c->stream);
  delete c;
}

API int mcmc_b200_num_params(const mcmc_b200_ctx* c) { return c ? c->P : -1; }
API void* mcmc_b200_stream(mcmc_b200_ctx* c) { return c ? (void*)c->stream : nullptr; }

static int check_status(mcmc_b200_ctx* c) {
  int st = 0;
  CK(cudaMemcpyAsync(&st, c->status, 4, cudaMemcpyDeviceToHost, c->stream));
  CK(cudaStreamSynchronize(c->stream));
  if (st != 0) {
    cudaMemsetAsync(c->status, 0, 4, c->stream);
    char b[96];
    snprintf(b, sizeof b, "device-side wait ran out (code %d)", st);
    return fail(MCMC_B200_ERR_TIMEOUT, b);
  }
  return MCMC_B200_OK;
}

API int mcmc_b200_synchronize(mcmc_b200_ctx* c) {
  if (!c) return fail(MCMC_B200_ERR_INVALID, "null context");
  CK(cudaSetDevice(c->device));
  return check_status(c);
}

API int mcmc_b200_philox_device(mcmc_b200_ctx* c, const uint32_t ctr[4], const uint32_t key[2], int n,
                                uint32_t* raw_out, float* normals_out, float* uniform_out) {
  if (!c || !ctr || !key || n < 1 || n > 4096 || !raw_out || !normals_out || !uniform_out)
    return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  CK(cudaSetDevice(c->device));
  // scratch of this call: the single-window row-loss buffer is at least 128 floats and is free between calls
  if ((size_t)n * 5 + 1 > (size_t)c->rows_pad) return fail(MCMC_B200_ERR_INVALID, "n too large for this context");
  uint32_t* raw = reinterpret_cast<uint32_t*>(c->row_loss);
  float* normals = c->row_loss + 4 * (size_t)n;
  float* uni = normals + n;
  cudaError_t e = launch_philox_probe(ctr, key, n, raw, normals, uni, c->stream);
  c->launches++;
  if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
  CK(cudaMemcpyAsync(raw_out, raw, (size_t)n * 16, cudaMemcpyDeviceToHost, c->stream));
  CK(cudaMemcpyAsync(normals_out, normals, (size_t)n * 4, cudaMemcpyDeviceToHost, c->stream));
  CK(cudaMemcpyAsync(uniform_out, uni, 4, cudaMemcpyDeviceToHost, c->stream));
  CK(cudaStreamSynchronize(c->stream));
  return MCMC_B200_OK;
}

API int mcmc_b200_selftest_wait_timeout(mcmc_b200_ctx* c, int limit_us) {
  if (!c || limit_us < 20 || limit_us > 1000000) return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  CK(cudaSetDevice(c->device));
  cudaError_t e = launch_wait_probe(c->status, (unsigned int)(limit_us / 20), c->stream);
  c->launches++;
  if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
  return check_status(c);
}

API int mcmc_b200_set_window_data(mcmc_b200_ctx* c, int window, int64_t global_window, const float* x,
                                  const float* y, int is_device) {
  if (!c || !x || !y || window < 0 || window >= c->W) return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  CK(cudaSetDevice(c->device));
  const size_t nx = (size_t)c->rows * c->cfg.D, ny = (size_t)c->rows;
  const float *dx = x, *dy = y;
  if (!is_device) {
    if (!c->stage) {
      int r = dalloc(c, (void**)&c->stage, (nx + ny) * 4, false);
      if (r) return r;
    }
    CK(cudaMemcpyAsync(c->stage, x, nx * 4, cudaMemcpyHostToDevice, c->stream));
    CK(cudaMemcpyAsync(c->stage + nx, y, ny * 4, cudaMemcpyHostToDevice, c->stream));
    dx = c->stage;
    dy = c->stage + nx;
  }
  cudaError_t e = launch_repack(dx, dy, c->xaug + (size_t)window * c->rows_pad * KP, c->rows, c->rows_pad,
                                c->cfg.D, c->stream);
  c->launches++;
  if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
  c->h_gwin[window] = global_window;
  c->window_set[window] = 1;
  CK(cudaMemcpyAsync(c->gwin + window, &c->h_gwin[window], 8, cudaMemcpyHostToDevice, c->stream));
  CK(cudaStreamSynchronize(c->stream));  // the caller's buffers are free again on return
  if (window == 0) { c->bound_x = nullptr; c->bound_y = nullptr; }
  return MCMC_B200_OK;
}

// ---- launch helpers ------------------------------------------------------
static GradParams base_grad_params(mcmc_b200_ctx* c) {
  GradParams g;
  memset(&g, 0, sizeof g);
  g.xaug = c->xaug;
  g.window_stride = c->rows_pad * KP;
  g.n_rows = (int)c->rows;
  g.n_tiles = (int)(c->rows_pad / c->tile_rows);
  g.P = c->P;
  g.Pp = c->Pp;
  g.lik = make_lik(c->cfg);
  g.prior = make_prior(c->cfg);
  g.status = c->status;
  return g;
}

// `single` selects the single-window work table / slot count (explicit-state calls)
static int launch_grad(mcmc_b200_ctx* c, GradParams g, bool single, cudaStream_t st) {
  cudaError_t e;
  const int slots = single ? c->slices_x : c->slices;
  g.slices_in = slots;
  g.slices_out = slots;
  if (c->cfg.precision == MCMC_B200_PREC_TF32) {
    g.nslot_in = single ? c->xtab_nslot : c->tab_nslot;
    g.seg_ptr = single ? c->xtab_seg_ptr : c->tab_seg_ptr;
    g.segs = single ? c->xtab_segs : c->tab_segs;
    e = launch_grad_tf32(c->cfg.H, &c->tmap_mn, g, single ? c->xtab_ctas : c->tab_ctas, st);
  } else {
    e = launch_grad_fp32(c->cfg.H, g, slots, single ? 1 : c->W, st);
  }
  c->launches++;
  if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, std::string("gradient kernel launch: ") + cudaGetErrorString(e));
  return MCMC_B200_OK;
}

static int allreduce(mcmc_b200_ctx* c, double* buf, size_t count, cudaStream_t st) {
  int r = g_nccl.AllReduce(buf, buf, count, kNcclFloat64, kNcclSum, c->comm, st);
  if (r != 0)
    return fail(MCMC_B200_ERR_NCCL, std::string("ncclAllReduce: ") +
                                        (g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "error"));
  return MCMC_B200_OK;
}

// this rank's sums and their all-reduce over peer memory in one launch (row sharding, one window)
static size_t oneshot_block_bytes(const mcmc_b200_ctx* c) {
  return (size_t)2 * c->nranks * (c->Pp + 4) * 2 * sizeof(uint2);  // [2 halves][nranks][Pp + 4][2 words]
}
static int oneshot_allreduce(mcmc_b200_ctx* c, const float* partial, const double* llp, cudaStream_t st) {
  OneShotParams p;
  memset(&p, 0, sizeof p);
  p.partial = partial;
  p.ll_partial = llp;
  p.slices = c->slices;
  p.nslot = c->tab_nslot;
  p.P = c->P;
  p.Pp = c->Pp;
  p.red = c->red;
  p.rank = c->rank;
  p.nranks = c->nranks;
  for (int k = 0; k < c->nranks; ++k) p.peer_words[k] = reinterpret_cast<uint2*>(c->os_base[k]);
  p.local_words = reinterpret_cast<const uint2*>(c->os_block);
  p.seq = c->os_seq;
  p.done = c->os_done;
  p.poll_limit = c->os_poll_limit;
  p.status = c->status;
  cudaError_t e = launch_oneshot_allreduce(p, st);
  c->launches++;
  if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, std::string("one-shot all-reduce launch: ") + cudaGetErrorString(e));
  return MCMC_B200_OK;
}

static AcceptParams base_accept_params(mcmc_b200_ctx* c) {
  AcceptParams a;
  memset(&a, 0, sizeof a);
  a.P = c->P;
  a.Pp = c->Pp;
  a.prior = make_prior(c->cfg);
  a.seed = c->cfg.seed;
  a.ref_streams = c->cfg.rng_streams == MCMC_B200_RNG_REFERENCE;
  a.ref_log_u = c->ref_log_u;
  a.ref_cap = c->ref_cap > 0 ? c->ref_cap : 1;
  return a;
}

// ---- the reference's random streams (main.h:207-216, :235-239): the libraries' own engines ----------
constexpr uint64_t REF_DRAWS_PER_ITER = 962;  // 961 momenta + 1 accept draw per iteration (main.h:216,237)
static float refstream_log_uniform(uint64_t seed) {
  // main.h:235-239: a fresh engine per draw, U(FLT_MIN, 1), log() evaluated in double and narrowed
  std::default_random_engine engine;
  engine.seed((std::default_random_engine::result_type)seed);
  std::uniform_real_distribution<float> accept_draw(std::numeric_limits<float>::min(), 1.0f);
  return (float)log((double)accept_draw(engine));
}
API uint32_t mcmc_b200_refstream_engine(uint64_t n_discard) {
  thrust::default_random_engine engine;
  engine.discard(n_discard);
  return (uint32_t)engine();
}
API uint32_t mcmc_b200_refstream_engine0(uint64_t seed) {
  std::default_random_engine engine;
  engine.seed((std::default_random_engine::result_type)seed);
  return (uint32_t)engine();
}
API float mcmc_b200_refstream_log_uniform(uint64_t seed) { return refstream_log_uniform(seed); }

static void drop_graph(mcmc_b200_ctx* c);
// makes the log accept draws of iterations [0, upto) available on the device (absolute iteration index)
static int refstream_fill(mcmc_b200_ctx* c, int upto) {
  if (c->cfg.rng_streams != MCMC_B200_RNG_REFERENCE || upto <= c->ref_filled) return MCMC_B200_OK;
  if (upto > c->ref_cap) {
    const int cap = std::max(upto + 64, c->cfg.burn_in + c->cfg.sample_capacity + 64);
    float* nb = nullptr;
    int r = dalloc(c, (void**)&nb, (size_t)cap * 4, true);  // (the old buffer stays in the context's free list)
    if (r) return r;
    CK(cudaStreamSynchronize(c->stream));
    c->ref_log_u = nb;
    c->ref_cap = cap;
    c->ref_filled = 0;
    drop_graph(c);  // the captured accept launch holds the old pointer
  }
  std::vector<float> h((size_t)(upto - c->ref_filled));
  for (int it = c->ref_filled; it < upto; ++it)
    h[(size_t)(it - c->ref_filled)] = refstream_log_uniform(c->cfg.seed + REF_DRAWS_PER_ITER * (uint64_t)it + 961);
  CK(cudaMemcpyAsync(c->ref_log_u + c->ref_filled, h.data(), h.size() * 4, cudaMemcpyHostToDevice, c->stream));
  CK(cudaStreamSynchronize(c->stream));
  c->ref_filled = upto;
  return MCMC_B200_OK;
}

API int mcmc_b200_refstream_momentum_device(mcmc_b200_ctx* c, uint64_t first_n, int count, float* out) {
  if (!c || !out || count < 1 || (long long)count > c->rows_pad)
    return fail(MCMC_B200_ERR_INVALID, "bad arguments (count is limited to the context's padded row count)");
  CK(cudaSetDevice(c->device));
  cudaError_t e = launch_refstream_momentum(first_n, count, c->row_loss, c->stream);
  c->launches++;
  if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
  CK(cudaMemcpyAsync(out, c->row_loss, (size_t)count * 4, cudaMemcpyDeviceToHost, c->stream));
  CK(cudaStreamSynchronize(c->stream));
  return MCMC_B200_OK;
}

static void fill_chain_accept(mcmc_b200_ctx* c, AcceptParams& a, int mode, int L) {
  a.mode = mode;
  a.slices = c->slices;
  a.nslot = c->tab_nslot;
  const int last = (mode == ACC_BOOTSTRAP) ? 0 : (L - 1) & 1;
  a.partial = c->partial[last];
  a.ll_partial = c->llp[last];
  a.red_in = (c->comm || c->use_red || c->oneshot) ? c->red : nullptr;
  a.w_new = (mode == ACC_BOOTSTRAP) ? c->wbuf[0] : c->wbuf[L & 1];
  a.m_new = (mode == ACC_BOOTSTRAP) ? c->mbuf[0] : c->mbuf[L & 1];
  a.m0 = c->m0;
  a.w_cur = c->w_cur;
  a.g_cur = c->g_cur;
  a.ll_cur = c->ll_cur;
  a.lp_cur = c->lp_cur;
  a.eps = c->eps;
  a.iter = c->iter;
  a.n_accept = c->n_accept;
  a.gwin = c->gwin;
  a.w_start = c->wbuf[0];
  a.m_start = c->mbuf[0];
  a.samples = c->samples;
  a.sample_capacity = c->samples ? c->cfg.sample_capacity : 0;
  a.burn_in = c->cfg.burn_in;
  a.adapt_steps = c->cfg.adapt_steps;
  a.log_target = (float)log(c->cfg.target_rate);
  a.dec_adj = -(float)c->cfg.decrement / (1.f + (float)c->cfg.decrement);
  a.inc_adj = (float)c->cfg.increment;
  a.trace_iters = c->cfg.trace_iters;
  a.tr_mom = c->tr_mom;
  a.tr_log_u = c->tr_log_u;
  a.tr_log_acpt = c->tr_log_acpt;
  a.tr_accept = c->tr_accept;
  a.tr_eps = c->tr_eps;
}

// queue one gradient evaluation for all windows (+ the allreduce when sharded)
static int chain_grad(mcmc_b200_ctx* c, int mode, int s, cudaStream_t st) {
  GradParams g = base_grad_params(c);
  g.mode = mode;
  g.w_in = c->wbuf[s & 1];
  g.m_in = c->mbuf[s & 1];
  g.w_out = c->wbuf[(s + 1) & 1];
  g.m_out = c->mbuf[(s + 1) & 1];
  g.g_carried = c->g_cur;
  g.partial_in = c->partial[(s + 1) & 1];
  const bool red = c->comm || c->use_red || c->oneshot;
  g.red_in = (red && mode == MODE_NEXT) ? c->red : nullptr;
  g.partial_out = c->partial[s & 1];
  g.ll_out = c->llp[s & 1];
  g.eps = c->eps;
  int r = launch_grad(c, g, false, st);
  if (r) return r;
  if (c->oneshot) return oneshot_allreduce(c, c->partial[s & 1], c->llp[s & 1], st);
  if (red) {
    cudaError_t e = launch_reduce_partials(c->partial[s & 1], c->llp[s & 1], c->slices, c->tab_nslot, c->P,
                                           c->Pp, c->red, c->W, st);
    c->launches++;
    if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
    if (c->comm) {
      r = allreduce(c, c->red, (size_t)c->W * (c->Pp + 4), st);
      if (r) return r;
    }
  }
  return MCMC_B200_OK;
}

// All L gradient evaluations of one iteration in one cooperative launch (chain_grad's L launches folded
// into one; same buffers, same rotation).
static int chain_grad_multistep(mcmc_b200_ctx* c, cudaStream_t st) {
  GradParams g = base_grad_params(c);
  g.slices_in = g.slices_out = c->slices;
  g.nslot_in = c->tab_nslot;
  g.seg_ptr = c->tab_seg_ptr;
  g.segs = c->tab_segs;
  g.g_carried = c->g_cur;
  g.eps = c->eps;
  g.n_steps = c->cfg.leapfrog_steps;
  g.n_slots = c->slices;    // one window: the CTAs that own tiles of it, one partial vector each
  for (int i = 0; i < 2; ++i) {
    g.w_buf[i] = c->wbuf[i];
    g.m_buf[i] = c->mbuf[i];
    g.partial_buf[i] = c->partial[i];
    g.ll_buf[i] = c->llp[i];
  }
  g.red = c->red;
  g.grid_bar = c->grid_bar;
  CK(cudaMemsetAsync(c->grid_bar, 0, 4, st));
  cudaError_t e = launch_grad_tf32_multistep(c->cfg.H, &c->tmap_mn, g, c->tab_ctas, st);
  c->launches++;
  if (e != cudaSuccess)
    return fail(MCMC_B200_ERR_CUDA, std::string("multi-step gradient kernel launch: ") + cudaGetErrorString(e));
  return MCMC_B200_OK;
}

static int queue_iteration(mcmc_b200_ctx* c, cudaStream_t st) {
  const int L = c->cfg.leapfrog_steps;
  if (c->multistep) {
    int r = chain_grad_multistep(c, st);
    if (r) return r;
  } else {
    for (int s = 0; s < L; ++s) {
      int r = chain_grad(c, s == 0 ? MODE_FIRST : MODE_NEXT, s, st);
      if (r) return r;
    }
  }
  AcceptParams a = base_accept_params(c);
  fill_chain_accept(c, a, ACC_ITERATE, L);
  cudaError_t e = launch_accept(a, c->W, st);
  c->launches++;
  if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
  return MCMC_B200_OK;
}

static int bootstrap(mcmc_b200_ctx* c) {
  for (int w = 0; w < c->W; ++w)
    if (!c->window_set[w]) return fail(MCMC_B200_ERR_INVALID, "a window has no data yet");
  // main.h:52,182-185: the chain starts at w = 0
  const size_t n = (size_t)c->W * c->Pp * 4;
  CK(cudaMemsetAsync(c->wbuf[0], 0, n, c->stream));
  CK(cudaMemsetAsync(c->mbuf[0], 0, n, c->stream));
  CK(cudaMemsetAsync(c->iter, 0, (size_t)c->W * 4, c->stream));
  CK(cudaMemsetAsync(c->n_accept, 0, (size_t)c->W * 4, c->stream));
  std::vector<float> e(c->W, (float)c->cfg.eps0);
  CK(cudaMemcpyAsync(c->eps, e.data(), (size_t)c->W * 4, cudaMemcpyHostToDevice, c->stream));
  CK(cudaStreamSynchronize(c->stream));
  int r = chain_grad(c, MODE_EVAL, 0, c->stream);
  if (r) return r;
  AcceptParams a = base_accept_params(c);
  fill_chain_accept(c, a, ACC_BOOTSTRAP, 1);
  cudaError_t er = launch_accept(a, c->W, c->stream);
  c->launches++;
  if (er != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, cudaGetErrorString(er));
  c->bootstrapped = true;
  c->iters_done = 0;
  return MCMC_B200_OK;
}

// The captured iteration graph bakes in the launch sequence (with or without the partial-sum and
// all-reduce launches, one launch per step or one per iteration): whatever changes that sequence drops it.
static void drop_graph(mcmc_b200_ctx* c) {
  if (c->graph_exec) cudaGraphExecDestroy(c->graph_exec);
  c->graph_exec = nullptr;
  c->graph_tried = false;
}

API int mcmc_b200_reset_chain(mcmc_b200_ctx* c) {
  if (!c) return fail(MCMC_B200_ERR_INVALID, "null context");
  CK(cudaSetDevice(c->device));
  CK(cudaStreamSynchronize(c->stream));
  drop_graph(c);
  c->bootstrapped = false;
  c->iters_done = 0;
  return MCMC_B200_OK;
}

API int mcmc_b200_run_chain_async(mcmc_b200_ctx* c, int n_iter) {
  if (!c || n_iter < 0) return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  CK(cudaSetDevice(c->device));
  if (!c->bootstrapped) {
    int r = bootstrap(c);
    if (r) return r;
  }
  if (n_iter == 0) return MCMC_B200_OK;
  {
    int r = refstream_fill(c, c->iters_done + n_iter);
    if (r) return r;
  }
  // One HMC iteration (L gradient launches + the accept kernel) is captured
  // once and replayed: launch cost stays off the critical path.
  if (!c->graph_tried) {
    c->graph_tried = true;
    const long long launches_before = c->launches;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal);
    if (e == cudaSuccess) {
      int r = queue_iteration(c, c->stream);
      e = cudaStreamEndCapture(c->stream, &graph);
      if (r == MCMC_B200_OK && e == cudaSuccess && graph) {
        e = cudaGraphInstantiate(&c->graph_exec, graph, 0);
        if (e != cudaSuccess) c->graph_exec = nullptr;
      }
      if (graph) cudaGraphDestroy(graph);
    }
    cudaGetLastError();
    c->launches = launches_before;
  }
  const long long per_iter =
      c->multistep ? 2 : (long long)c->cfg.leapfrog_steps * ((c->comm || c->use_red || c->oneshot) ? 2 : 1) + 1;
  for (int i = 0; i < n_iter; ++i) {
    if (c->graph_exec) {
      CK(cudaGraphLaunch(c->graph_exec, c->stream));
      c->launches += per_iter;
    } else {
      int r = queue_iteration(c, c->stream);
      if (r) return r;
    }
  }
  c->iters_done += n_iter;
  return MCMC_B200_OK;
}

API int mcmc_b200_run_chain(mcmc_b200_ctx* c, int n_iter) {
  int r = mcmc_b200_run_chain_async(c, n_iter);
  if (r) return r;
  return check_status(c);
}

API int mcmc_b200_chain_info(mcmc_b200_ctx* c, int window, int32_t* iterations, int32_t* accepted,
                             float* eps) {
  if (!c || window < 0 || window >= c->W) return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  CK(cudaSetDevice(c->device));
  CK(cudaStreamSynchronize(c->stream));
  if (iterations) CK(cudaMemcpy(iterations, c->iter + window, 4, cudaMemcpyDeviceToHost));
  if (accepted) CK(cudaMemcpy(accepted, c->n_accept + window, 4, cudaMemcpyDeviceToHost));
  if (eps) CK(cudaMemcpy(eps, c->eps + window, 4, cudaMemcpyDeviceToHost));
  return MCMC_B200_OK;
}

API int mcmc_b200_get_state(mcmc_b200_ctx* c, int window, float* w, float* grad, double* loglik,
                            double* logprior) {
  if (!c || window < 0 || window >= c->W) return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  CK(cudaSetDevice(c->device));
  CK(cudaStreamSynchronize(c->stream));
  const size_t o = (size_t)window * c->Pp;
  if (w) CK(cudaMemcpy(w, c->w_cur + o, (size_t)c->P * 4, cudaMemcpyDeviceToHost));
  if (grad) CK(cudaMemcpy(grad, c->g_cur + o, (size_t)c->P * 4, cudaMemcpyDeviceToHost));
  if (loglik) CK(cudaMemcpy(loglik, c->ll_cur + window, 8, cudaMemcpyDeviceToHost));
  if (logprior) CK(cudaMemcpy(logprior, c->lp_cur + window, 8, cudaMemcpyDeviceToHost));
  return MCMC_B200_OK;
}

API int mcmc_b200_get_samples(mcmc_b200_ctx* c, int window, int first, int count, float* out) {
  if (!c || !out || window < 0 || window >= c->W || first < 0 || count < 0 || !c->samples ||
      first + count > c->cfg.sample_capacity)
    return fail(MCMC_B200_ERR_INVALID, "bad arguments or no sample storage");
  CK(cudaSetDevice(c->device));
  CK(cudaStreamSynchronize(c->stream));
  const size_t P = c->P;
  CK(cudaMemcpy(out, c->samples + ((size_t)window * c->cfg.sample_capacity + first) * P,
                (size_t)count * P * 4, cudaMemcpyDeviceToHost));
  return MCMC_B200_OK;
}

API int mcmc_b200_get_trace(mcmc_b200_ctx* c, int window, int first, int count, float* momenta,
                            float* log_u, double* log_acpt, int32_t* accepted, float* eps) {
  if (!c || window < 0 || window >= c->W || first < 0 || count < 0 ||
      first + count > c->cfg.trace_iters)
    return fail(MCMC_B200_ERR_INVALID, "bad arguments or trace not enabled");
  CK(cudaSetDevice(c->device));
  CK(cudaStreamSynchronize(c->stream));
  const size_t K = c->cfg.trace_iters, P = c->P, o = (size_t)window * K + first;
  if (momenta) CK(cudaMemcpy(momenta, c->tr_mom + o * P, (size_t)count * P * 4, cudaMemcpyDeviceToHost));
  if (log_u) CK(cudaMemcpy(log_u, c->tr_log_u + o, (size_t)count * 4, cudaMemcpyDeviceToHost));
  if (log_acpt) CK(cudaMemcpy(log_acpt, c->tr_log_acpt + o, (size_t)count * 8, cudaMemcpyDeviceToHost));
  if (accepted) CK(cudaMemcpy(accepted, c->tr_accept + o, (size_t)count * 4, cudaMemcpyDeviceToHost));
  if (eps) CK(cudaMemcpy(eps, c->tr_eps + o, (size_t)count * 4, cudaMemcpyDeviceToHost));
  return MCMC_B200_OK;
}

// ---- checkpoint / resume ------------------------------------------------------
// The reference keeps its samples in device memory and loses them, with the chain state, when the
// process ends (main.h:183,277-283,295).  Every random draw here is a pure function of (seed, global
// window, iteration), so a chain resumed from a checkpoint continues bit-identically.
namespace {
struct CkptHeader {
  char magic[8];          // "MCB2CKPT"
  uint32_t version, header_bytes;
  int32_t W, P, Pp, D, H, likelihood, precision, leapfrog_steps, burn_in, adapt_steps, sample_capacity,
      trace_iters, iters_done, slices, rng_streams;
  int64_t rows;
  uint64_t seed;
  uint64_t payload_bytes;
};
struct CkptField {
  void* dev;
  size_t bytes;
};
std::vector<CkptField> ckpt_fields(mcmc_b200_ctx* c) {
  const size_t W = c->W, Pp = c->Pp, P = c->P, S = c->cfg.sample_capacity, K = c->cfg.trace_iters;
  std::vector<CkptField> f = {
      {c->wbuf[0], W * Pp * 4}, {c->mbuf[0], W * Pp * 4}, {c->w_cur, W * Pp * 4}, {c->g_cur, W * Pp * 4},
      {c->m0, W * Pp * 4},      {c->ll_cur, W * 8},       {c->lp_cur, W * 8},     {c->eps, W * 4},
      {c->iter, W * 4},         {c->n_accept, W * 4},     {c->gwin, W * 8}};
  if (c->samples) f.push_back({c->samples, W * S * P * 4});
  if (K > 0) {
    f.push_back({c->tr_mom, W * K * P * 4});
    f.push_back({c->tr_log_u, W * K * 4});
    f.push_back({c->tr_log_acpt, W * K * 8});
    f.push_back({c->tr_accept, W * K * 4});
    f.push_back({c->tr_eps, W * K * 4});
  }
  return f;
}
CkptHeader ckpt_header(mcmc_b200_ctx* c) {
  CkptHeader h;
  memset(&h, 0, sizeof h);
  memcpy(h.magic, "MCB2CKPT", 8);
  h.version = 2;
  h.header_bytes = sizeof(CkptHeader);
  h.W = c->W; h.P = c->P; h.Pp = c->Pp; h.D = c->cfg.D; h.H = c->cfg.H;
  h.likelihood = c->cfg.likelihood; h.precision = c->cfg.precision;
  h.leapfrog_steps = c->cfg.leapfrog_steps; h.burn_in = c->cfg.burn_in; h.adapt_steps = c->cfg.adapt_steps;
  h.sample_capacity = c->cfg.sample_capacity; h.trace_iters = c->cfg.trace_iters;
  h.iters_done = c->iters_done; h.slices = c->slices; h.rng_streams = c->cfg.rng_streams;
  h.rows = c->rows; h.seed = c->cfg.seed;
  for (const CkptField& f : ckpt_fields(c)) h.payload_bytes += f.bytes;
  return h;
}
}  // namespace

API int mcmc_b200_checkpoint_size(mcmc_b200_ctx* c, uint64_t* bytes) {
  if (!c || !bytes) return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  const CkptHeader h = ckpt_header(c);
  *bytes = sizeof(CkptHeader) + h.payload_bytes;
  return MCMC_B200_OK;
}

API int mcmc_b200_checkpoint_save(mcmc_b200_ctx* c, void* host_buf, uint64_t bytes) {
  if (!c || !host_buf) return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  if (!c->bootstrapped) return fail(MCMC_B200_ERR_INVALID, "nothing to save: the chain has not started");
  CK(cudaSetDevice(c->device));
  int r = check_status(c);  // synchronises; a chain that timed out is not worth saving
  if (r) return r;
  const CkptHeader h = ckpt_header(c);
  if (bytes < sizeof(CkptHeader) + h.payload_bytes) return fail(MCMC_B200_ERR_INVALID, "buffer too small");
  memcpy(host_buf, &h, sizeof h);
  char* p = static_cast<char*>(host_buf) + sizeof h;
  for (const CkptField& f : ckpt_fields(c)) {
    CK(cudaMemcpy(p, f.dev, f.bytes, cudaMemcpyDeviceToHost));
    p += f.bytes;
  }
  return MCMC_B200_OK;
}

API int mcmc_b200_checkpoint_load(mcmc_b200_ctx* c, const void* host_buf, uint64_t bytes) {
  if (!c || !host_buf || bytes < sizeof(CkptHeader)) return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  CkptHeader h;
  memcpy(&h, host_buf, sizeof h);
  const CkptHeader want = ckpt_header(c);
  if (memcmp(h.magic, want.magic, 8) != 0 || h.version != want.version || h.header_bytes != sizeof h)
    return fail(MCMC_B200_ERR_INVALID, "not a checkpoint of this library version");
  if (h.W != want.W || h.P != want.P || h.Pp != want.Pp || h.D != want.D || h.H != want.H ||
      h.likelihood != want.likelihood || h.precision != want.precision ||
      h.leapfrog_steps != want.leapfrog_steps || h.burn_in != want.burn_in ||
      h.adapt_steps != want.adapt_steps || h.sample_capacity != want.sample_capacity ||
      h.trace_iters != want.trace_iters || h.rows != want.rows || h.seed != want.seed ||
      h.rng_streams != want.rng_streams ||
      h.payload_bytes != want.payload_bytes)
    return fail(MCMC_B200_ERR_INVALID, "checkpoint was written by a context with a different configuration");
  if (bytes < sizeof h + h.payload_bytes) return fail(MCMC_B200_ERR_INVALID, "truncated checkpoint");
  for (int w = 0; w < c->W; ++w)
    if (!c->window_set[w]) return fail(MCMC_B200_ERR_INVALID, "upload every window's data before resuming");
  CK(cudaSetDevice(c->device));
  CK(cudaStreamSynchronize(c->stream));
  const char* p = static_cast<const char*>(host_buf) + sizeof h;
  const std::vector<CkptField> fields = ckpt_fields(c);
  // the stored global window ids must be the ones this context was given: chains are keyed by them
  {
    size_t off = 0;
    for (const CkptField& f : fields) {
      if (f.dev == c->gwin) break;
      off += f.bytes;
    }
    if (memcmp(p + off, c->h_gwin.data(), (size_t)c->W * 8) != 0)
      return fail(MCMC_B200_ERR_INVALID, "checkpoint belongs to other global windows");
  }
  for (const CkptField& f : fields) {
    CK(cudaMemcpy(f.dev, p, f.bytes, cudaMemcpyHostToDevice));
    p += f.bytes;
  }
  c->bootstrapped = true;
  c->iters_done = h.iters_done;
  return MCMC_B200_OK;
}

// ---- explicit-state calls (one window) -------------------------------------
// L leapfrog steps from (w0, m0, g0) on device; results in xw/xm[L&1], g_out, scalars.
static int explicit_steps(mcmc_b200_ctx* c, int data_window, int L, float eps, const float* w0,
                          const float* m0, const float* g0, float* w_last, float* m_last,
                          float* g_out, float* row_loss, float* prior_loss, cudaStream_t st,
                          bool eval_only, bool data_fresh = false) {
  const int S = c->slices_x;
  for (int s = 0; s < L; ++s) {
    GradParams g = base_grad_params(c);
    g.data_window0 = data_window;
    g.data_fresh = (data_fresh && s == 0) ? 1 : 0;  // a repack was queued directly before the first launch
    g.mode = eval_only ? MODE_EVAL : (s == 0 ? MODE_FIRST : MODE_NEXT);
    g.w_in = s == 0 ? w0 : c->xw[s & 1];
    g.m_in = s == 0 ? m0 : c->xm[s & 1];
    const bool last = s == L - 1;
    g.w_out = (last && w_last) ? w_last : c->xw[(s + 1) & 1];
    g.m_out = (last && m_last) ? m_last : c->xm[(s + 1) & 1];
    g.g_carried = g0;
    g.partial_in = c->xpartial[(s + 1) & 1];
    const bool red = c->comm || c->use_red_x;
    g.red_in = (red && g.mode == MODE_NEXT) ? c->xred : nullptr;
    g.partial_out = c->xpartial[s & 1];
    g.ll_out = c->xllp[s & 1];
    g.eps = nullptr;
    g.eps_scalar = eps;
    g.row_loss = last ? row_loss : nullptr;
    g.row_loss_stride = 0;
    int r = launch_grad(c, g, true, st);
    if (r) return r;
    if (red) {
      cudaError_t e = launch_reduce_partials(c->xpartial[s & 1], c->xllp[s & 1], S, c->xtab_nslot, c->P, c->Pp,
                                             c->xred, 1, st);
      c->launches++;
      if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
      if (c->comm) {
        r = allreduce(c, c->xred, (size_t)(c->Pp + 4), st);
        if (r) return r;
      }
    }
  }
  AcceptParams a = base_accept_params(c);
  a.mode = ACC_FINALIZE;
  a.slices = S;
  a.nslot = c->xtab_nslot;
  a.partial = c->xpartial[(L - 1) & 1];
  a.ll_partial = c->xllp[(L - 1) & 1];
  a.red_in = (c->comm || c->use_red_x) ? c->xred : nullptr;
  a.w_new = eval_only ? w0 : ((w_last) ? w_last : c->xw[L & 1]);
  a.g_out = g_out;
  a.prior_loss_out = prior_loss;
  a.scalars_out = c->scalars;
  cudaError_t e = launch_accept(a, 1, st);
  c->launches++;
  if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
  return MCMC_B200_OK;
}

API int mcmc_b200_potential_and_grad(mcmc_b200_ctx* c, int window, const float* w, double* loglik,
                                     double* logprior, float* grad, float* row_loss) {
  if (!c || !w || window < 0 || window >= c->W) return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  if (!c->window_set[window]) return fail(MCMC_B200_ERR_INVALID, "window has no data yet");
  CK(cudaSetDevice(c->device));
  CK(cudaMemcpyAsync(c->xw[0], w, (size_t)c->P * 4, cudaMemcpyHostToDevice, c->stream));
  int r = explicit_steps(c, window, 1, 0.f, c->xw[0], c->xm[0], c->xg, nullptr, nullptr, c->g_out,
                         row_loss ? c->row_loss : nullptr, nullptr, c->stream, true);
  if (r) return r;
  double sc[2];
  CK(cudaMemcpyAsync(sc, c->scalars, 16, cudaMemcpyDeviceToHost, c->stream));
  if (grad) CK(cudaMemcpyAsync(grad, c->g_out, (size_t)c->P * 4, cudaMemcpyDeviceToHost, c->stream));
  if (row_loss)
    CK(cudaMemcpyAsync(row_loss, c->row_loss, (size_t)c->rows * 4, cudaMemcpyDeviceToHost, c->stream));
  r = check_status(c);
  if (r) return r;
  if (loglik) *loglik = sc[0];
  if (logprior) *logprior = sc[1];
  return MCMC_B200_OK;
}

API int mcmc_b200_leapfrog(mcmc_b200_ctx* c, int window, int L, float eps, const float* w_prev,
                           const float* mom_prev, const float* grad_prev, float* w_next,
                           float* mom_next, float* grad_cur, double* loglik, double* logprior) {
  if (!c || !w_prev || !mom_prev || !grad_prev || L < 1 || window < 0 || window >= c->W)
    return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  if (!c->window_set[window]) return fail(MCMC_B200_ERR_INVALID, "window has no data yet");
  CK(cudaSetDevice(c->device));
  const size_t n = (size_t)c->P * 4;
  CK(cudaMemcpyAsync(c->xw[0], w_prev, n, cudaMemcpyHostToDevice, c->stream));
  CK(cudaMemcpyAsync(c->xm[0], mom_prev, n, cudaMemcpyHostToDevice, c->stream));
  CK(cudaMemcpyAsync(c->xg, grad_prev, n, cudaMemcpyHostToDevice, c->stream));
  int r = explicit_steps(c, window, L, eps, c->xw[0], c->xm[0], c->xg, nullptr, nullptr, c->g_out, nullptr,
                         nullptr, c->stream, false);
  if (r) return r;
  double sc[2];
  CK(cudaMemcpyAsync(sc, c->scalars, 16, cudaMemcpyDeviceToHost, c->stream));
  if (w_next) CK(cudaMemcpyAsync(w_next, c->xw[L & 1], n, cudaMemcpyDeviceToHost, c->stream));
  if (mom_next) CK(cudaMemcpyAsync(mom_next, c->xm[L & 1], n, cudaMemcpyDeviceToHost, c->stream));
  if (grad_cur) CK(cudaMemcpyAsync(grad_cur, c->g_out, n, cudaMemcpyDeviceToHost, c->stream));
  r = check_status(c);
  if (r) return r;
  if (loglik) *loglik = sc[0];
  if (logprior) *logprior = sc[1];
  return MCMC_B200_OK;
}

API int mcmc_b200_mcmc_step(mcmc_b200_ctx* c, const float* x, const float* y, const float* weights_prev,
                            float* weights_next, const float* mom_prev, float* mom_next,
                            const float* grad_prev, float* grad_cur, float* grad_next,
                            float* loss_values, int L, float eps, void* stream) {
  if (!c || !x || !y || !weights_prev || !weights_next || !mom_prev || !mom_next || !grad_prev ||
      !grad_cur || L < 1)
    return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  if (c->W != 1) return fail(MCMC_B200_ERR_INVALID, "mcmc_step needs a context with one window");
  CK(cudaSetDevice(c->device));
  cudaStream_t st = (cudaStream_t)stream;
  bool repacked = false;
  if (x != c->bound_x || y != c->bound_y) {
    // first use of this dataset (or the first call after mcmc_b200_rebind_data): repack it
    // (io.h:82-85 is where the reference uploads it)
    cudaError_t e = launch_repack(x, y, c->xaug, c->rows, c->rows_pad, c->cfg.D, st);
    c->launches++;
    if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
    c->bound_x = x;
    c->bound_y = y;
    c->window_set[0] = 1;
    repacked = true;
  }
  int r = explicit_steps(c, 0, L, eps, weights_prev, mom_prev, grad_prev, weights_next, mom_next, grad_cur,
                         loss_values, loss_values ? loss_values + c->rows : nullptr, st, false, repacked);
  if (r) return r;
  if (grad_next) CK(cudaMemsetAsync(grad_next, 0, (size_t)c->P * 4, st));
  return MCMC_B200_OK;
}

API int mcmc_b200_rebind_data(mcmc_b200_ctx* c) {
  if (!c) return fail(MCMC_B200_ERR_INVALID, "null context");
  c->bound_x = nullptr;
  c->bound_y = nullptr;
  return MCMC_B200_OK;
}

API int mcmc_b200_log_acpt(mcmc_b200_ctx* c, const float* prev_loss, const float* new_loss,
                           int64_t n_loss, const float* prev_mom, const float* new_mom,
                           const float* grad_cur, float eps, void* stream, float* out) {
  if (!c || !prev_loss || !new_loss || !prev_mom || !new_mom || !grad_cur || !out)
    return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  CK(cudaSetDevice(c->device));
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = launch_log_acpt(prev_loss, new_loss, n_loss, prev_mom, new_mom, grad_cur, c->P, eps,
                                  c->scalar_f, st);
  c->launches++;
  if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
  CK(cudaMemcpyAsync(out, c->scalar_f, 4, cudaMemcpyDeviceToHost, st));
  CK(cudaStreamSynchronize(st));
  return MCMC_B200_OK;
}

// grows a cached scratch buffer (kept for the life of the context; the old one stays in the free list)
template <typename T>
static int fwd_reserve(mcmc_b200_ctx* c, T** buf, size_t* cap, size_t need) {
  if (need <= *cap) return MCMC_B200_OK;
  T* nb = nullptr;
  int r = dalloc(c, (void**)&nb, need * sizeof(T), false);
  if (r) return r;
  *buf = nb;
  *cap = need;
  return MCMC_B200_OK;
}
// sample chunks per row tile: enough CTAs for two waves of the GPU, at most one chunk per sample
static int fwd_chunks(const mcmc_b200_ctx* c, long long n, int count) {
  const long long tiles = forward_row_tiles(n);
  long long ch = (2LL * c->num_sms * 3 + tiles - 1) / tiles;
  ch = std::max<long long>(1, std::min<long long>(std::min<long long>(ch, count), 64));
  return (int)ch;
}

API int mcmc_b200_predict_mean(mcmc_b200_ctx* c, int window, const float* xs, int64_t n, int first,
                               int count, float* out) {
  if (!c || !xs || !out || n < 1 || window < 0 || window >= c->W || first < 0 || count < 1 ||
      !c->samples || first + count > c->cfg.sample_capacity)
    return fail(MCMC_B200_ERR_INVALID, "bad arguments or no sample storage");
  CK(cudaSetDevice(c->device));
  const int chunks = fwd_chunks(c, n, count);
  int r = fwd_reserve(c, &c->fwd_x, &c->fwd_x_cap, (size_t)n * c->cfg.D);
  if (r == MCMC_B200_OK) r = fwd_reserve(c, &c->fwd_out, &c->fwd_out_cap, (size_t)n);
  if (r == MCMC_B200_OK) r = fwd_reserve(c, &c->fwd_partial, &c->fwd_partial_cap, (size_t)chunks * n);
  if (r) return r;
  CK(cudaMemcpyAsync(c->fwd_x, xs, (size_t)n * c->cfg.D * 4, cudaMemcpyHostToDevice, c->stream));
  ForwardParams a;
  memset(&a, 0, sizeof a);
  a.x = c->fwd_x;
  a.x_stride = c->cfg.D;
  a.n = n;
  a.samples = c->samples + ((size_t)window * c->cfg.sample_capacity + first) * c->P;
  a.count = count;
  a.lik = make_lik(c->cfg);
  a.partial = c->fwd_partial;
  cudaError_t e = launch_forward_samples(c->cfg.H, a, chunks, false, c->stream);
  if (e == cudaSuccess) e = launch_forward_finish_predict(c->fwd_partial, chunks, n, count, c->fwd_out, c->stream);
  c->launches += 2;
  if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
  CK(cudaMemcpyAsync(out, c->fwd_out, (size_t)n * 4, cudaMemcpyDeviceToHost, c->stream));
  CK(cudaStreamSynchronize(c->stream));
  return MCMC_B200_OK;
}

API int mcmc_b200_final_loss(mcmc_b200_ctx* c, int window, int first, int count, double* mean_loglik,
                             double* mean_logprior) {
  if (!c || window < 0 || window >= c->W || first < 0 || count < 1 || !c->samples ||
      first + count > c->cfg.sample_capacity)
    return fail(MCMC_B200_ERR_INVALID, "bad arguments or no sample storage");
  if (!c->window_set[window]) return fail(MCMC_B200_ERR_INVALID, "window has no data yet");
  CK(cudaSetDevice(c->device));
  // all samples against the window's rows in one launch (FP32 forward pass, no gradient)
  const int tiles = forward_row_tiles(c->rows);
  const int chunks = fwd_chunks(c, c->rows, count);
  int r = fwd_reserve(c, &c->fwd_partial, &c->fwd_partial_cap, (size_t)tiles * count + 2 * (size_t)count);
  if (r) return r;
  const float* xw = c->xaug + (size_t)window * c->rows_pad * KP;
  const float* smp = c->samples + ((size_t)window * c->cfg.sample_capacity + first) * c->P;
  ForwardParams a;
  memset(&a, 0, sizeof a);
  a.x = xw;
  a.x_stride = KP;
  a.y = xw + COL_Y;
  a.y_stride = KP;
  a.n = c->rows;
  a.samples = smp;
  a.count = count;
  a.lik = make_lik(c->cfg);
  a.partial = c->fwd_partial;
  double* d_ll = c->fwd_partial + (size_t)tiles * count;
  double* d_lp = d_ll + count;
  cudaError_t e = launch_forward_samples(c->cfg.H, a, chunks, true, c->stream);
  if (e == cudaSuccess)
    e = launch_forward_finish_loss(c->fwd_partial, tiles, count, smp, c->P, make_prior(c->cfg), d_ll, d_lp, c->stream);
  c->launches += 2;
  if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
  std::vector<double> h(2 * (size_t)count);
  CK(cudaMemcpyAsync(h.data(), d_ll, h.size() * 8, cudaMemcpyDeviceToHost, c->stream));
  CK(cudaStreamSynchronize(c->stream));
  double sa = 0, sb = 0;
  for (int s = 0; s < count; ++s) { sa += h[s]; sb += h[count + s]; }  // main.h:100-113: running means
  if (mean_loglik) *mean_loglik = sa / count;
  if (mean_logprior) *mean_logprior = sb / count;
  return MCMC_B200_OK;
}

API int mcmc_b200_nccl_unique_id(unsigned char id[128]) {
  std::string why;
  if (!nccl_load(&why)) return fail(MCMC_B200_ERR_NCCL, why);
  NcclUniqueId u;
  int r = g_nccl.GetUniqueId(&u);
  if (r != 0) return fail(MCMC_B200_ERR_NCCL, "ncclGetUniqueId failed");
  memcpy(id, u.internal, 128);
  return MCMC_B200_OK;
}

API int mcmc_b200_enable_row_sharding(mcmc_b200_ctx* c, const unsigned char id[128], int rank, int nranks) {
  if (!c || !id || nranks < 1 || rank < 0 || rank >= nranks) return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  if (c->bootstrapped) return fail(MCMC_B200_ERR_INVALID, "enable row sharding before the chain starts");
  std::string why;
  if (!nccl_load(&why)) return fail(MCMC_B200_ERR_NCCL, why);
  CK(cudaSetDevice(c->device));
  NcclUniqueId u;
  memcpy(u.internal, id, 128);
  int r = g_nccl.CommInitRank(&c->comm, nranks, u, rank);
  if (r != 0) {
    c->comm = nullptr;
    return fail(MCMC_B200_ERR_NCCL, std::string("ncclCommInitRank: ") +
                                        (g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "error"));
  }
  c->rank = rank;
  c->nranks = nranks;
  c->multistep = false;  // every step's sums cross GPUs: one launch + one all-reduce per step
  drop_graph(c);         // a graph captured before this call has neither the sums nor the all-reduce in it
  return MCMC_B200_OK;
}

// Sets up the peer-memory all-reduce on top of an existing row-sharding communicator: one allocation per
// rank (receive slots + flags), its CUDA IPC handle gathered over the communicator, every peer's block
// mapped into this process.  `fake_peers` (self-test only): no communicator, the "peers" are further
// blocks of THIS GPU that nothing ever writes.
static int oneshot_setup(mcmc_b200_ctx* c, bool fake_peers) {
  if (c->nranks > ONESHOT_MAX_RANKS) return fail(MCMC_B200_ERR_INVALID, "too many ranks for the one-shot all-reduce");
  const size_t block = oneshot_block_bytes(c);
  int r = dalloc(c, &c->os_block, fake_peers ? block * c->nranks : block, true);
  if (r) return r;
  r = dalloc(c, (void**)&c->os_seq, 8, true);
  if (r) return r;
  c->os_done = c->os_seq + 1;
  std::vector<char*> base(c->nranks, nullptr);
  c->os_peer_blocks.assign(c->nranks, nullptr);
  if (fake_peers) {
    for (int k = 0; k < c->nranks; ++k) base[k] = static_cast<char*>(c->os_block) + (size_t)k * block;
  } else {
    cudaIpcMemHandle_t mine;
    CK(cudaIpcGetMemHandle(&mine, c->os_block));
    char* dh = nullptr;
    r = dalloc(c, (void**)&dh, sizeof(mine) * c->nranks, true);
    if (r) return r;
    CK(cudaMemcpy(dh + sizeof(mine) * c->rank, &mine, sizeof(mine), cudaMemcpyHostToDevice));
    if (!g_nccl.AllGather) return fail(MCMC_B200_ERR_NCCL, "ncclAllGather missing");
    int nr = g_nccl.AllGather(dh + sizeof(mine) * c->rank, dh, sizeof(mine), kNcclChar, c->comm, c->stream);
    if (nr != 0) return fail(MCMC_B200_ERR_NCCL, "ncclAllGather of the IPC handles failed");
    CK(cudaStreamSynchronize(c->stream));
    std::vector<cudaIpcMemHandle_t> all(c->nranks);
    CK(cudaMemcpy(all.data(), dh, sizeof(mine) * c->nranks, cudaMemcpyDeviceToHost));
    for (int k = 0; k < c->nranks; ++k) {
      if (k == c->rank) { base[k] = static_cast<char*>(c->os_block); continue; }
      void* p = nullptr;
      cudaError_t e = cudaIpcOpenMemHandle(&p, all[k], cudaIpcMemLazyEnablePeerAccess);
      if (e != cudaSuccess)
        return fail(MCMC_B200_ERR_CUDA, std::string("cudaIpcOpenMemHandle (peer access between the GPUs is "
                                                    "required): ") + cudaGetErrorString(e));
      c->os_peer_blocks[k] = p;
      base[k] = static_cast<char*>(p);
    }
  }
  c->os_base.assign(base.begin(), base.end());
  if (!fake_peers) {
    // nobody may send before every rank has zeroed and mapped its block: one tiny all-reduce as the barrier
    int nr = g_nccl.AllReduce(c->red, c->red, 1, kNcclFloat64, kNcclSum, c->comm, c->stream);
    if (nr != 0) return fail(MCMC_B200_ERR_NCCL, "set-up barrier failed");
    CK(cudaStreamSynchronize(c->stream));
  }
  c->oneshot = true;
  c->multistep = false;
  drop_graph(c);
  return MCMC_B200_OK;
}

API int mcmc_b200_enable_oneshot_allreduce(mcmc_b200_ctx* c) {
  if (!c) return fail(MCMC_B200_ERR_INVALID, "null context");
  if (!c->comm) return fail(MCMC_B200_ERR_INVALID, "call mcmc_b200_enable_row_sharding first");
  if (c->bootstrapped) return fail(MCMC_B200_ERR_INVALID, "enable it before the chain starts");
  if (c->oneshot) return MCMC_B200_OK;
  if (c->W != 1) return fail(MCMC_B200_ERR_INVALID, "row sharding is for contexts with one window");
  CK(cudaSetDevice(c->device));
  return oneshot_setup(c, false);
}

API int mcmc_b200_selftest_oneshot_timeout(mcmc_b200_ctx* c, int polls) {
  if (!c || polls < 1 || polls > (1 << 24)) return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  if (c->comm || c->oneshot || c->bootstrapped || c->W != 1)
    return fail(MCMC_B200_ERR_INVALID, "needs a fresh one-window context without row sharding");
  CK(cudaSetDevice(c->device));
  // two "ranks" of which only this one ever sends: the wait for the other one must run out
  c->nranks = 2;
  c->rank = 0;
  int r = oneshot_setup(c, true);
  if (r) return r;
  c->os_poll_limit = (unsigned int)polls;
  CK(cudaMemsetAsync(c->partial[0], 0, (size_t)c->slices * c->Pp * 4, c->stream));
  r = oneshot_allreduce(c, c->partial[0], c->llp[0], c->stream);
  // back to an unsharded context whatever happened
  c->oneshot = false;
  c->nranks = 1;
  c->os_poll_limit = 1u << 22;
  drop_graph(c);
  if (r) return r;
  return check_status(c);
}

API int mcmc_b200_time_allreduce(mcmc_b200_ctx* c, int reps, float* us_per_call) {
  if (!c || reps < 1 || !us_per_call) return fail(MCMC_B200_ERR_INVALID, "bad arguments");
  if (!c->comm) return fail(MCMC_B200_ERR_INVALID, "row sharding is not enabled");
  CK(cudaSetDevice(c->device));
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  auto once = [&]() -> int {
    if (c->oneshot) return oneshot_allreduce(c, c->partial[0], c->llp[0], c->stream);
    cudaError_t e = launch_reduce_partials(c->partial[0], c->llp[0], c->slices, c->tab_nslot, c->P, c->Pp, c->red,
                                           c->W, c->stream);
    c->launches++;
    if (e != cudaSuccess) return fail(MCMC_B200_ERR_CUDA, cudaGetErrorString(e));
    return allreduce(c, c->red, (size_t)c->W * (c->Pp + 4), c->stream);
  };
  for (int i = 0; i < 5; ++i) { int r = once(); if (r) return r; }
  CK(cudaEventRecord(e0, c->stream));
  for (int i = 0; i < reps; ++i) { int r = once(); if (r) return r; }
  CK(cudaEventRecord(e1, c->stream));
  CK(cudaEventSynchronize(e1));
  float ms = 0.f;
  CK(cudaEventElapsedTime(&ms, e0, e1));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  *us_per_call = 1e3f * ms / reps;
  return check_status(c);
}

API int64_t mcmc_b200_launch_count(mcmc_b200_ctx* c, int reset) {
  if (!c) return -1;
  long long v = c->launches;
  if (reset) c->launches = 0;
  return v;
}

API int mcmc_b200_chain_geometry(mcmc_b200_ctx* c, int* slices, int* ctas_per_sm, int* tile_rows) {
  if (!c) return fail(MCMC_B200_ERR_INVALID, "null context");
  if (slices) *slices = c->slices;
  if (ctas_per_sm) *ctas_per_sm = c->ctas_per_sm;
  if (tile_rows) *tile_rows = c->tile_rows;
  return MCMC_B200_OK;
}

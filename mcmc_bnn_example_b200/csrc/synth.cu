// Host-side helpers exported through the C-ABI: the synthetic window generator
// that stands in for the reference's data file (include/mcmc/global_params.h:65,
// include/mcmc/io.h:42-86 — the file is not distributed with the reference) and
// host evaluation of the library's Philox streams.  No GPU is needed for these.
#include <math.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <vector>

#include "../../include/mcmc_b200.h"
#include "philox.h"

using namespace mcmc_b200;

#define API extern "C" __attribute__((visibility("default")))

namespace {

// normals [i0, i1) of a stream, four per Philox block
void fill_normals(uint64_t seed, uint32_t window, uint32_t stream, long long i0, long long i1, float scale,
                  float* out) {
  const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  long long i = i0;
  while (i < i1) {
    const uint32_t blk = (uint32_t)(i >> 2);
    Philox4 r = philox4x32_10(blk, 0u, window, stream, k0, k1);
    float n[4];
    philox_box_muller(r.v[0], r.v[1], &n[0], &n[1]);
    philox_box_muller(r.v[2], r.v[3], &n[2], &n[3]);
    for (int l = (int)(i & 3); l < 4 && i < i1; ++l, ++i) out[i] = scale * n[l];
  }
}

template <typename F>
void parallel_for(long long n, long long grain, F f) {
  unsigned hw = std::thread::hardware_concurrency();
  if (hw == 0) hw = 1;
  long long nt = std::min<long long>(hw, (n + grain - 1) / grain);
  if (nt <= 1) { f(0, n); return; }
  std::vector<std::thread> th;
  long long chunk = ((n + nt - 1) / nt + 3) & ~3LL;  // keep Philox blocks whole
  for (long long t = 0; t < nt; ++t) {
    long long a = t * chunk, b = std::min(n, a + chunk);
    if (a >= b) break;
    th.emplace_back([=] { f(a, b); });
  }
  for (auto& t : th) t.join();
}

}  // namespace

API int mcmc_b200_synth_window(uint64_t seed, int64_t window, int64_t rows, int D, int H, float* x, float* y,
                               float* teacher) {
  if (!x || !y || rows < 1 || D < 1 || H < 1 || (long long)rows * D >= (1LL << 34)) return MCMC_B200_ERR_INVALID;
  const uint32_t win = (uint32_t)window;
  const int P = D * H + 2 * H + 1;
  std::vector<float> tw(P);
  fill_normals(seed, win, STREAM_SYNTH_TEACHER, 0, P, 0.3f, tw.data());
  if (teacher) memcpy(teacher, tw.data(), sizeof(float) * P);
  parallel_for((long long)rows * D, 1 << 16,
               [&](long long a, long long b) { fill_normals(seed, win, STREAM_SYNTH_X, a, b, 1.0f, x); });
  parallel_for(rows, 1 << 14,
               [&](long long a, long long b) { fill_normals(seed, win, STREAM_SYNTH_NOISE, a, b, 0.05f, y); });
  // y = teacher(x) + noise, teacher forward in double
  parallel_for(rows, 1 << 12, [&](long long a, long long b) {
    for (long long r = a; r < b; ++r) {
      double pred = tw[D * H + 2 * H];
      for (int j = 0; j < H; ++j) {
        double z = tw[D * H + j];
        for (int k = 0; k < D; ++k) z += (double)x[r * D + k] * (double)tw[k * H + j];
        pred += (double)tw[D * H + H + j] * tanh(z);
      }
      y[r] = (float)(pred + (double)y[r]);
    }
  });
  return MCMC_B200_OK;
}

API float mcmc_b200_philox_normal(uint64_t seed, uint32_t window, uint32_t iteration, uint32_t stream,
                                  uint32_t index) {
  return philox_normal(seed, window, iteration, stream, index);
}

API void mcmc_b200_philox_raw(const uint32_t ctr[4], const uint32_t key[2], uint32_t out[4]) {
  Philox4 r = philox4x32_10(ctr[0], ctr[1], ctr[2], ctr[3], key[0], key[1]);
  for (int i = 0; i < 4; ++i) out[i] = r.v[i];
}

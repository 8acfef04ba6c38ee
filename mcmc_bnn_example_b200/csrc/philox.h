// Counter-based Philox4x32-10 generator shared by host and device code.
//
// The reference draws its momentum from a Thrust minstd engine on the device
// and its accept uniform from a libstdc++ minstd0 engine on the host
// (include/mcmc/main.h:207-216, :235-239), re-seeded per element / per
// iteration.  This library replaces both with one stateless generator keyed by
// (seed, window, iteration): any draw can be recomputed anywhere, so chains are
// independent of how windows are placed on GPUs and can be resumed exactly.
//
// Counter layout:   ctr = {index, iteration, window, stream}
// Key:              key = {seed_lo, seed_hi}
// Streams: 0 = momentum normals, 1 = accept uniform, 2 = synthetic X,
//          3 = synthetic teacher weights, 4 = synthetic noise.
#pragma once
#include <stdint.h>
#include <math.h>

#if defined(__CUDACC__)
#define PHILOX_HD __host__ __device__ __forceinline__
#else
#define PHILOX_HD static inline
#endif

namespace mcmc_b200 {

enum PhiloxStream : uint32_t {
  STREAM_MOMENTUM = 0,
  STREAM_ACCEPT = 1,
  STREAM_SYNTH_X = 2,
  STREAM_SYNTH_TEACHER = 3,
  STREAM_SYNTH_NOISE = 4
};

struct Philox4 {
  uint32_t v[4];
};

PHILOX_HD void philox_mulhilo(uint32_t a, uint32_t b, uint32_t* hi, uint32_t* lo) {
#if defined(__CUDA_ARCH__)
  *hi = __umulhi(a, b);
  *lo = a * b;
#else
  uint64_t p = (uint64_t)a * (uint64_t)b;
  *hi = (uint32_t)(p >> 32);
  *lo = (uint32_t)p;
#endif
}

// Philox4x32 with 10 rounds (Salmon et al., "Parallel random numbers: as easy
// as 1, 2, 3", SC'11): multipliers 0xD2511F53 / 0xCD9E8D57, Weyl key
// increments 0x9E3779B9 / 0xBB67AE85.
PHILOX_HD Philox4 philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0,
                                uint32_t k1) {
  for (int r = 0; r < 10; ++r) {
    uint32_t hi0, lo0, hi1, lo1;
    philox_mulhilo(0xD2511F53u, c0, &hi0, &lo0);
    philox_mulhilo(0xCD9E8D57u, c2, &hi1, &lo1);
    uint32_t n0 = hi1 ^ c1 ^ k0;
    uint32_t n1 = lo1;
    uint32_t n2 = hi0 ^ c3 ^ k1;
    uint32_t n3 = lo0;
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  Philox4 out;
  out.v[0] = c0; out.v[1] = c1; out.v[2] = c2; out.v[3] = c3;
  return out;
}

// (0, 1]: never returns 0 so that log() is finite.
PHILOX_HD float philox_u01(uint32_t x) { return ((float)(x >> 8) + 1.0f) * (1.0f / 16777216.0f); }

// Two standard normals from two 32-bit words (Box-Muller).
PHILOX_HD void philox_box_muller(uint32_t a, uint32_t b, float* n0, float* n1) {
  float u1 = philox_u01(a);
  float u2 = philox_u01(b);
  float r = sqrtf(-2.0f * logf(u1));
  float s, c;
#if defined(__CUDA_ARCH__)
  sincospif(2.0f * u2, &s, &c);
#else
  const float two_pi = 6.28318530717958647692f;
  s = sinf(two_pi * u2);
  c = cosf(two_pi * u2);
#endif
  *n0 = r * c;
  *n1 = r * s;
}

// The i-th standard normal of (seed, window, iteration, stream).  Four normals
// share one Philox block: index i uses block i/4, lane i%4.
PHILOX_HD float philox_normal(uint64_t seed, uint32_t window, uint32_t iteration, uint32_t stream,
                              uint32_t i) {
  Philox4 r = philox4x32_10(i >> 2, iteration, window, stream, (uint32_t)seed, (uint32_t)(seed >> 32));
  float n0, n1;
  if ((i & 2u) == 0) philox_box_muller(r.v[0], r.v[1], &n0, &n1);
  else philox_box_muller(r.v[2], r.v[3], &n0, &n1);
  return (i & 1u) ? n1 : n0;
}

// The accept uniform of (seed, window, iteration), in (0, 1].
PHILOX_HD float philox_accept_uniform(uint64_t seed, uint32_t window, uint32_t iteration) {
  Philox4 r = philox4x32_10(0u, iteration, window, STREAM_ACCEPT, (uint32_t)seed, (uint32_t)(seed >> 32));
  return philox_u01(r.v[0]);
}

}  // namespace mcmc_b200

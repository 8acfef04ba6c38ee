// tcgen05 / tensor-memory / TMA wrappers and descriptor builders shared by the TF32 kernels
// (grad_tf32.cu: 40 hidden units, grad_tf32_wide.cu: 128).
#pragma once
#include <cuda.h>
#include <utility>
#include "common.cuh"

namespace mcmc_b200 {

// ---- tcgen05 wrappers ----------------------------------------------------
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem desc] . B[smem desc]
__device__ __forceinline__ void tc_mma_tf32_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem desc]
__device__ __forceinline__ void tc_mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, float* v) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                 "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tc_st8(uint32_t taddr, const float4& a, const float4& b) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr),
               "r"(__float_as_uint(a.x)), "r"(__float_as_uint(a.y)), "r"(__float_as_uint(a.z)),
               "r"(__float_as_uint(a.w)), "r"(__float_as_uint(b.x)), "r"(__float_as_uint(b.y)),
               "r"(__float_as_uint(b.z)), "r"(__float_as_uint(b.w))
               : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* tmap, int x, int y,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
      "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// Shared-memory matrix descriptor (version 1).  Byte offsets are encoded
// without their 4 low bits.  Layout types used here:
//   2 = 128-byte swizzle of 16-byte chunks   (K-major operands)
//   1 = 128-byte swizzle of 32-byte chunks   (the only layout the tensor core
//       accepts for MN-major operands of 32-bit types)
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                              uint32_t sbo_bytes, uint32_t layout_type) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) |
         ((uint64_t)layout_type << 61);
}
// K-major, 16-byte-chunk swizzle: rows (M/N) of 128 bytes, groups of 8 rows 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t smem_addr) {
  return umma_desc(smem_addr, 16, 1024, 2);
}
// MN-major, 32-byte-chunk swizzle: rows (K) of 128 bytes, groups of 4 rows 512 bytes apart,
// 32-float atoms along M/N `atom_stride` bytes apart
__device__ __forceinline__ uint64_t umma_desc_mn32(uint32_t smem_addr, uint32_t atom_stride) {
  return umma_desc(smem_addr, atom_stride, 512, 1);
}
// Moves a descriptor's start address by `units` x 16 bytes (the address field is the low 14 bits; the
// operands here never carry out of it): one 32-bit add instead of rebuilding the descriptor per MMA.
__device__ __forceinline__ uint64_t umma_desc_advance(uint64_t d, uint32_t units) {
  return (d & 0xFFFFFFFF00000000ull) | (uint64_t)((uint32_t)d + units);
}
// Instruction descriptor: F32 accumulate, TF32 x TF32, dense.
__host__ __device__ constexpr uint32_t umma_idesc_tf32(int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)a_mn_major << 15) |
         ((uint32_t)b_mn_major << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// E element stores with the line offset as an immediate (no address arithmetic per store)
template <int J>
__device__ __forceinline__ void store_e_one(const uint32_t* e_ptr, const float* z) {
  asm volatile("st.shared.f32 [%0+%2], %1;" ::"r"(e_ptr[J & 7]), "f"(z[J]), "n"(J * 128) : "memory");
}
template <int... Js>
__device__ __forceinline__ void store_e_all(const uint32_t* e_ptr, const float* z,
                                            std::integer_sequence<int, Js...>) {
  (store_e_one<Js>(e_ptr, z), ...);
}

// Pins a loop-invariant per-thread value in a register: a value that went through a shuffle cannot be
// recomputed from the thread index at every use (which is what the compiler otherwise does with the
// address constants of the tile loop when registers are tight, at some 100 instructions per tile).
__device__ __forceinline__ uint32_t pin(uint32_t v) { return __shfl_sync(0xffffffffu, v, threadIdx.x & 31); }

__device__ __forceinline__ float4 lds128(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

// Optional per-row loss output as a predicated store (no branch in the tile body)
__device__ __forceinline__ void store_row_loss(float* base, long long idx, float loss, bool valid) {
  const uint32_t on = (base != nullptr && valid) ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %2, 0;\n\t@p st.global.f32 [%0], %1;\n\t}" ::"l"(base + idx), "f"(loss),
      "r"(on)
      : "memory");
}

// The slow side of a bounded wait, out of line so that the five waits of a tile cost one test each.
// `ok` is false once any wait of this thread has run out: later waits then return at once instead of
// running out one after the other.
static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, int* status, int code, bool ok) {
  if (!ok) return false;
  for (uint32_t i = 0; i < MBAR_WAIT_SLICES; ++i) {
    if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
  }
  if (status) atomicExch(status, code);
  return false;
}
__device__ __forceinline__ void mbar_wait_q(uint64_t* bar, uint32_t parity, int* status, int code, bool& ok) {
  if (!mbar_try_wait(bar, parity)) ok = mbar_wait_slow(bar, parity, status, code, ok);
}

// Named hardware barriers hand work from a warpgroup (128 arriving threads) to its control warp
// (32 waiting threads): a few tens of cycles, no polling.  Ids 1..NWG are the warpgroups' own barriers.
constexpr int BAR_ROWS0 = 4;   // + wg: rows of a tile are in tensor memory
constexpr int BAR_E0 = 8;      // + wg: E of a tile is in shared memory
__device__ __forceinline__ void named_arrive(int id, int count) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// Sum of v[j] over the 32 lanes of the warp, for every j = 0..31: lane l returns the sum for j = l.
// Step `off` (16, 8, 4, 2, 1): a lane whose bit `off` is clear keeps the lower half of its remaining values
// and sends the upper half to lane ^ off, which does the opposite.
__device__ __forceinline__ float warp_column_sums(float* v, int lane) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const bool up = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < off; ++i) {
      const float send = up ? v[i] : v[i + off];
      const float keep = up ? v[i + off] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
    }
  }
  return v[0];
}

}  // namespace mcmc_b200

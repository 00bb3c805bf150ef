// Pieces shared by the fast tensor-core GEMM kernels (gemm_tc_fast.cu, gemm_tc_skinny.cu):
// the magic-number conversion constants, the exact fix-up of a K-tile accumulator and the
// one-lane barrier wait.
#pragma once

#include "fxp_common.cuh"
#include "tc_common.cuh"

namespace fxpr {

static __device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

static constexpr uint32_t kMagicBits = 0x4B400000u;      // 1.5 * 2^23
static constexpr uint32_t kExpBits = 0x4B000000u;        // exponent pattern of [2^23, 2^24)

static __device__ __forceinline__ float tmem_ld1(uint32_t taddr) {
  uint32_t r;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  return __uint_as_float(r);
}

// Rare path, entered by a whole warp (tcgen05.ld is warp-collective): for `ncols`
// columns of one K-tile accumulator, find this lane's out-of-range partials and record
// (a) the raw value the fast path added for them and (b) the reference conversion's
// result.  Rolled loop, no register arrays: small code, off the hot path.
static __device__ __noinline__ void fixup_tile(uint32_t taddr, int ncols, float scale, int int_bits,
                                        uint32_t* corr_raw, long long* corr_q) {
  const float magic = __uint_as_float(kMagicBits);
#pragma unroll 1
  for (int i = 0; i < ncols; ++i) {
    const float f = tmem_ld1(taddr + i);
    const uint32_t b = __float_as_uint(__fmaf_rn(f, scale, magic));
    if (((b ^ kExpBits) >> 23) != 0) {
      corr_raw[i] += b - kMagicBits;
      corr_q[i] += (int_bits == 64) ? float_to_fixed<64>(f, scale) : (long long)float_to_fixed<32>(f, scale);
    }
  }
}

// One lane polls, the warp follows: 32x fewer mbarrier probes than every lane spinning.
static __device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int lane) {
  int ok = 1;
  if (lane == 0) ok = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

}  // namespace fxpr

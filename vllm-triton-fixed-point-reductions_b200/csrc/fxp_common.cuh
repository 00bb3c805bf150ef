// Device helpers shared by every kernel: Q-format casts, deterministic exp2/log,
// typed loads/stores, integer warp reductions.
//
// The float -> fixed conversion follows fxpr_vllm/_triton/fxp.py:92-108 of the
// reference: one fp32 multiply by 2^frac, then cvt.rni.sat (int16/int32) or a
// float clamp followed by cvt.rni.s64 (int64).  All "exact" float arithmetic
// here uses explicit round-to-nearest intrinsics so no fused multiply-add can be
// formed and a CPU that does single IEEE operations reproduces every bit.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fxpr_b200.h"

namespace fxpr {

// ---- host-side error plumbing ------------------------------------------------
void set_last_error(const char* what, cudaError_t err);
int check_launch(const char* what);

inline int ceil_div_i(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }

// ---- programmatic dependent launch ------------------------------------------------
// Decode steps are chains of short kernels, each waiting for the one before it.  Launched with
// the programmatic-stream-serialization attribute, a kernel's CTAs may start (barrier setup,
// tensor-memory allocation, descriptor prefetch) while the previous kernel is still running;
// pdl_wait() then blocks until every earlier kernel of the stream has completed and its writes
// are visible.  Rules every such kernel keeps: no global-memory access that depends on (or is
// read by) an earlier kernel before pdl_wait(), and every CTA calls pdl_wait().  Without the
// attribute both instructions do nothing.  FXPR_NO_PDL=1 in the environment turns the
// attribute off.
bool pdl_enabled();

__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// cudaLaunchKernelEx with the attribute (and an optional cluster width along x).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, unsigned cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- integer type by width -----------------------------------------------------
template <int BITS> struct IntOf;
template <> struct IntOf<16> { using type = int16_t; };
template <> struct IntOf<32> { using type = int32_t; };
template <> struct IntOf<64> { using type = long long; };

// ---- PTX conversions -------------------------------------------------------------
__device__ __forceinline__ int32_t cvt_rni_sat_s32(float x) {
  int32_t r;
  asm("cvt.rni.sat.s32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ int16_t cvt_rni_sat_s16(float x) {
  short r;
  asm("cvt.rni.sat.s16.f32 %0, %1;" : "=h"(r) : "f"(x));
  return (int16_t)r;
}
__device__ __forceinline__ long long cvt_rni_s64(float x) {
  long long r;
  asm("cvt.rni.s64.f32 %0, %1;" : "=l"(r) : "f"(x));
  return r;
}

// Quantise an fp32 value: rint-half-even of x * scale, saturated to BITS.
template <int BITS>
__device__ __forceinline__ typename IntOf<BITS>::type float_to_fixed(float x, float scale) {
  const float s = __fmul_rn(x, scale);
  if constexpr (BITS == 32) {
    return cvt_rni_sat_s32(s);
  } else if constexpr (BITS == 16) {
    return cvt_rni_sat_s16(s);
  } else {
    // No .sat form for s64 <- f32 in the reference's recipe: clamp in float first.
    // fmaxf drops a NaN, so NaN ends at qmin.
    const float c = fminf(fmaxf(s, -9223372036854775808.0f), 9223372036854775807.0f);
    return cvt_rni_s64(c);
  }
}

// Same, accumulator-friendly: always returns a 64-bit value.
__device__ __forceinline__ long long float_to_fixed_any(float x, float scale, int bits) {
  if (bits == 32) return (long long)float_to_fixed<32>(x, scale);
  if (bits == 16) return (long long)float_to_fixed<16>(x, scale);
  return float_to_fixed<64>(x, scale);
}

// Wrap a 64-bit running sum to the accumulator width (plain += in that type).
__device__ __forceinline__ long long wrap_to_bits(long long v, int bits) {
  if (bits == 32) return (long long)(int32_t)v;
  if (bits == 16) return (long long)(int16_t)v;
  return v;
}

template <typename I>
__device__ __forceinline__ float fixed_to_float(I q, float inv_scale) {
  float f;
  if constexpr (sizeof(I) == 8) f = __ll2float_rn((long long)q);
  else f = __int2float_rn((int)q);
  return __fmul_rn(f, inv_scale);
}

// ---- typed element access ----------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<double>(double v) { return __double2float_rn(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ double from_f32<double>(float v) { return (double)v; }

// silu(g) * u on values the io dtype holds, rounded back to it (the SiLU*mul kernels and the
// GEMM epilogue that fuses them share this, so their bits agree)
template <typename T>
__device__ __forceinline__ T silu_mul_io(float g, float u) {
  const float sg = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
  return from_f32<T>(__fmul_rn(sg, u));
}

// ---- deterministic 2^t -----------------------------------------------------------
// n = rint(t), f = t - n (exact), degree-7 Horner polynomial of 2^f with separate
// multiply and add, exact scaling by 2^n.  t < -125 or NaN -> 0; t > 127 -> +inf.
// Coefficients are fp32((ln 2)^k / k!) written as bit patterns.
__device__ __forceinline__ float exp2_det(float t) {
  if (!(t >= -125.0f)) return 0.0f;
  if (t > 127.0f) return __int_as_float(0x7f800000);
  const float n = rintf(t);
  const float f = __fsub_rn(t, n);
  float p = __int_as_float(0x377fe5fe);                            // c7
  p = __fadd_rn(__fmul_rn(p, f), __int_as_float(0x39218489));      // c6
  p = __fadd_rn(__fmul_rn(p, f), __int_as_float(0x3aaec3ff));      // c5
  p = __fadd_rn(__fmul_rn(p, f), __int_as_float(0x3c1d955b));      // c4
  p = __fadd_rn(__fmul_rn(p, f), __int_as_float(0x3d635847));      // c3
  p = __fadd_rn(__fmul_rn(p, f), __int_as_float(0x3e75fdf0));      // c2
  p = __fadd_rn(__fmul_rn(p, f), __int_as_float(0x3f317218));      // c1
  p = __fadd_rn(__fmul_rn(p, f), __int_as_float(0x3f800000));      // c0
  const float two_n = __int_as_float(((int)n + 127) << 23);
  return __fmul_rn(p, two_n);
}

// log2(e) as the fp32 the host oracle uses (1.4426950408889634 rounded).
#define FXPR_LOG2E_F32 __int_as_float(0x3fb8aa3b)

// ---- two fp32 lanes per instruction (add/sub/mul/fma .f32x2: IEEE round-to-nearest per lane) ----
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_sub(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// exp2_det of two non-positive (or NaN) arguments at once, for callers that only use the
// result through float_to_fixed with at most 32 fraction bits.  Same operations on every lane as
// exp2_det, with two differences that cannot change a rounded Q value: arguments below -126 (and
// NaN) are clamped to -126 instead of returning 0 (2^-126 * 2^32 still rounds to 0), and
// n = rint(t) is taken from the mantissa of t + 1.5 * 2^23 (exact for |t| < 2^22), whose low bits
// also give the exponent field of 2^n without a float-to-int conversion.
__device__ __forceinline__ uint64_t exp2_det_nonpos_pair(float t0, float t1) {
  const float m = __uint_as_float(0x4B400000u);
  const uint64_t magic = f2_pack(m, m);
  const uint64_t t = f2_pack(fmaxf(t0, -126.0f), fmaxf(t1, -126.0f));
  const uint64_t r = f2_add(t, magic);               // bits: 0x4B400000 + n
  const uint64_t n = f2_sub(r, magic);
  const uint64_t f = f2_sub(t, n);
#define FXPR_C2(bits) f2_pack(__int_as_float(bits), __int_as_float(bits))
  uint64_t p = FXPR_C2(0x377fe5fe);
  p = f2_add(f2_mul(p, f), FXPR_C2(0x39218489));
  p = f2_add(f2_mul(p, f), FXPR_C2(0x3aaec3ff));
  p = f2_add(f2_mul(p, f), FXPR_C2(0x3c1d955b));
  p = f2_add(f2_mul(p, f), FXPR_C2(0x3d635847));
  p = f2_add(f2_mul(p, f), FXPR_C2(0x3e75fdf0));
  p = f2_add(f2_mul(p, f), FXPR_C2(0x3f317218));
  p = f2_add(f2_mul(p, f), FXPR_C2(0x3f800000));
#undef FXPR_C2
  // (0x4B400000 + n + 127) << 23 keeps only n + 127 in the exponent field
  const uint32_t lo = ((uint32_t)r + 127u) << 23, hi = ((uint32_t)(r >> 32) + 127u) << 23;
  const uint64_t two_n = ((uint64_t)hi << 32) | lo;
  return f2_mul(p, two_n);
}

// ---- deterministic natural log of a positive, normal fp32 ---------------------------
// fp64 with + - * / only: v = m 2^e, m in [sqrt(1/2), sqrt(2)); s = (m-1)/(m+1);
// log m = 2 s (1 + s^2/3 + ... + s^18/19).  Result rounded to fp32.
__device__ __forceinline__ float log_det(float v) {
  const double a = (double)v;
  long long bits = __double_as_longlong(a);
  int e = (int)((bits >> 52) & 0x7ff) - 1022;
  double m = __longlong_as_double((bits & 0x800fffffffffffffLL) | 0x3fe0000000000000LL);
  if (m < 0x1.6a09e667f3bcdp-1) {
    m = __dmul_rn(m, 2.0);
    e -= 1;
  }
  const double s = __ddiv_rn(__dsub_rn(m, 1.0), __dadd_rn(m, 1.0));
  const double s2 = __dmul_rn(s, s);
  double p = 0x1.af286bca1af28p-5;                                // 1/19
  p = __dadd_rn(__dmul_rn(p, s2), 0x1.e1e1e1e1e1e1ep-5);           // 1/17
  p = __dadd_rn(__dmul_rn(p, s2), 0x1.1111111111111p-4);           // 1/15
  p = __dadd_rn(__dmul_rn(p, s2), 0x1.3b13b13b13b14p-4);           // 1/13
  p = __dadd_rn(__dmul_rn(p, s2), 0x1.745d1745d1746p-4);           // 1/11
  p = __dadd_rn(__dmul_rn(p, s2), 0x1.c71c71c71c71cp-4);           // 1/9
  p = __dadd_rn(__dmul_rn(p, s2), 0x1.2492492492492p-3);           // 1/7
  p = __dadd_rn(__dmul_rn(p, s2), 0x1.999999999999ap-3);           // 1/5
  p = __dadd_rn(__dmul_rn(p, s2), 0x1.5555555555555p-2);           // 1/3
  p = __dadd_rn(__dmul_rn(p, s2), 1.0);
  double r = __dmul_rn(__dmul_rn(2.0, s), p);
  r = __dadd_rn(r, __dmul_rn((double)e, 0x1.62e42fefa39efp-1));
  return __double2float_rn(r);
}

// ---- warp / block integer reductions (order-free, hence deterministic) ---------------
__device__ __forceinline__ long long warp_sum_i64(long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max_f32(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide int64 sum; `red` holds >= 32 entries of shared memory.  All threads
// get the total.
__device__ __forceinline__ long long block_sum_i64(long long v, long long* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum_i64(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  long long t = (lane < nwarps) ? red[lane] : 0;
  t = warp_sum_i64(t);
  return t;
}
__device__ __forceinline__ float block_max_f32(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max_f32(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? red[lane] : -__int_as_float(0x7f800000);
  t = warp_max_f32(t);
  return t;
}

}  // namespace fxpr

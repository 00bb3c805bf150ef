// Elementwise float <-> Q-format casts as 128-bit vectorised, grid-stride HBM
// streaming kernels.  Semantics: fxpr_vllm/_triton/fxp.py:92-113 and
// fxpr_vllm/_triton/casts.py:21-54 of the reference (rint half-to-even,
// saturating; int -> fp32 round-to-nearest, multiply by 2^-frac, narrow).
#include "fxp_common.cuh"

namespace fxpr {

static constexpr int kCastThreads = 256;
static constexpr int kCastCtasPerSm = 8;

template <typename T, int N>
struct alignas(sizeof(T) * N >= 16 ? 16 : sizeof(T) * N) Pack {
  T v[N];
};

// Access shape: a lane moves E consecutive elements per access, chosen so that neither its
// load nor its store exceeds 16 bytes, and the lanes of a warp are contiguous -- every load
// and store instruction covers one unbroken span (fp32 -> int64: 256 B loads, 512 B stores).
// U independent accesses per thread and step keep several loads in flight.  E == 1 is the
// fallback for unaligned pointers.
template <typename TIn, typename TOut>
struct CastShape {
  static constexpr int kIn = 16 / (int)sizeof(TIn), kOut = 16 / (int)sizeof(TOut);
  static constexpr int E = kIn < kOut ? kIn : kOut;
};
static constexpr int kCastU = 4;

template <typename TIn, int BITS, int E>
__global__ void __launch_bounds__(kCastThreads)
float_to_fixed_kernel(const TIn* __restrict__ x, typename IntOf<BITS>::type* __restrict__ y,
                      int64_t n, float scale) {
  using TOut = typename IntOf<BITS>::type;
  const int64_t per_block = (int64_t)blockDim.x * E * kCastU;
  for (int64_t base = (int64_t)blockIdx.x * per_block; base < n; base += (int64_t)gridDim.x * per_block) {
    Pack<TIn, E> in[kCastU];
#pragma unroll
    for (int u = 0; u < kCastU; ++u) {
      const int64_t i = base + ((int64_t)u * blockDim.x + threadIdx.x) * E;
      if (i + E <= n) in[u] = *reinterpret_cast<const Pack<TIn, E>*>(x + i);
    }
#pragma unroll
    for (int u = 0; u < kCastU; ++u) {
      const int64_t i = base + ((int64_t)u * blockDim.x + threadIdx.x) * E;
      if (i + E <= n) {
        Pack<TOut, E> out;
#pragma unroll
        for (int j = 0; j < E; ++j) out.v[j] = float_to_fixed<BITS>(to_f32<TIn>(in[u].v[j]), scale);
        *reinterpret_cast<Pack<TOut, E>*>(y + i) = out;
      } else {
        for (int64_t j = i; j < n; ++j) y[j] = float_to_fixed<BITS>(to_f32<TIn>(x[j]), scale);   // ragged tail
      }
    }
  }
}

template <typename TIn, typename TOut, int E>
__global__ void __launch_bounds__(kCastThreads)
fixed_to_float_kernel(const TIn* __restrict__ x, TOut* __restrict__ y, int64_t n, float inv_scale) {
  const int64_t per_block = (int64_t)blockDim.x * E * kCastU;
  for (int64_t base = (int64_t)blockIdx.x * per_block; base < n; base += (int64_t)gridDim.x * per_block) {
    Pack<TIn, E> in[kCastU];
#pragma unroll
    for (int u = 0; u < kCastU; ++u) {
      const int64_t i = base + ((int64_t)u * blockDim.x + threadIdx.x) * E;
      if (i + E <= n) in[u] = *reinterpret_cast<const Pack<TIn, E>*>(x + i);
    }
#pragma unroll
    for (int u = 0; u < kCastU; ++u) {
      const int64_t i = base + ((int64_t)u * blockDim.x + threadIdx.x) * E;
      if (i + E <= n) {
        Pack<TOut, E> out;
#pragma unroll
        for (int j = 0; j < E; ++j) out.v[j] = from_f32<TOut>(fixed_to_float<TIn>(in[u].v[j], inv_scale));
        *reinterpret_cast<Pack<TOut, E>*>(y + i) = out;
      } else {
        for (int64_t j = i; j < n; ++j) y[j] = from_f32<TOut>(fixed_to_float<TIn>(x[j], inv_scale));
      }
    }
  }
}

static int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 148;
  }
  return cached[dev];
}

static int cast_grid(int64_t n, int vec) {
  vec *= kCastU;
  int64_t want = (n + (int64_t)kCastThreads * vec - 1) / ((int64_t)kCastThreads * vec);
  int64_t cap = (int64_t)num_sms() * kCastCtasPerSm;
  return (int)(want < cap ? (want < 1 ? 1 : want) : cap);
}

static bool aligned16(const void* a, const void* b) {
  return (((uintptr_t)a | (uintptr_t)b) & 15) == 0;
}

template <typename TIn, int BITS>
static int launch_f2x(const void* x, void* y, int64_t n, float scale, cudaStream_t s) {
  using TOut = typename IntOf<BITS>::type;
  constexpr int VEC = CastShape<TIn, TOut>::E;
  if (aligned16(x, y)) {
    float_to_fixed_kernel<TIn, BITS, VEC><<<cast_grid(n, VEC), kCastThreads, 0, s>>>(
        (const TIn*)x, (TOut*)y, n, scale);
  } else {
    float_to_fixed_kernel<TIn, BITS, 1><<<cast_grid(n, 1), kCastThreads, 0, s>>>(
        (const TIn*)x, (TOut*)y, n, scale);
  }
  return check_launch("float_to_fixed");
}

template <typename TIn>
static int dispatch_f2x(const void* x, void* y, int bits, int64_t n, float scale, cudaStream_t s) {
  switch (bits) {
    case 16: return launch_f2x<TIn, 16>(x, y, n, scale, s);
    case 32: return launch_f2x<TIn, 32>(x, y, n, scale, s);
    case 64: return launch_f2x<TIn, 64>(x, y, n, scale, s);
  }
  return FXPR_ERR_BAD_ARG;
}

template <typename TIn, typename TOut>
static int launch_x2f(const void* x, void* y, int64_t n, float inv, cudaStream_t s) {
  constexpr int VEC = CastShape<TIn, TOut>::E;
  if (aligned16(x, y)) {
    fixed_to_float_kernel<TIn, TOut, VEC><<<cast_grid(n, VEC), kCastThreads, 0, s>>>(
        (const TIn*)x, (TOut*)y, n, inv);
  } else {
    fixed_to_float_kernel<TIn, TOut, 1><<<cast_grid(n, 1), kCastThreads, 0, s>>>(
        (const TIn*)x, (TOut*)y, n, inv);
  }
  return check_launch("fixed_to_float");
}

template <typename TIn>
static int dispatch_x2f(const void* x, void* y, int float_bits, int64_t n, float inv, cudaStream_t s) {
  switch (float_bits) {
    case 16: return launch_x2f<TIn, __half>(x, y, n, inv, s);
    case 32: return launch_x2f<TIn, float>(x, y, n, inv, s);
    case 64: return launch_x2f<TIn, double>(x, y, n, inv, s);
  }
  return FXPR_ERR_BAD_ARG;
}

}  // namespace fxpr

using namespace fxpr;

extern "C" int fxpr_float_to_fixed(const void* x, int x_dtype, void* y, int int_bits,
                                   int frac_bits, int64_t n, void* stream) {
  if (n < 0 || frac_bits < 0 || frac_bits >= 64) return FXPR_ERR_BAD_ARG;
  if (int_bits != 16 && int_bits != 32 && int_bits != 64) return FXPR_ERR_BAD_ARG;
  if (n == 0) return FXPR_OK;
  if (!x || !y) return FXPR_ERR_BAD_ARG;
  const float scale = (float)(1ull << frac_bits);
  cudaStream_t s = (cudaStream_t)stream;
  switch (x_dtype) {
    case FXPR_F16: return dispatch_f2x<__half>(x, y, int_bits, n, scale, s);
    case FXPR_F32: return dispatch_f2x<float>(x, y, int_bits, n, scale, s);
    case FXPR_F64: return dispatch_f2x<double>(x, y, int_bits, n, scale, s);
  }
  return FXPR_ERR_UNSUPPORTED;
}

extern "C" int fxpr_fixed_to_float(const void* x, int int_bits, void* y, int float_bits,
                                   int frac_bits, int64_t n, void* stream) {
  if (n < 0 || frac_bits < 0 || frac_bits >= 64) return FXPR_ERR_BAD_ARG;
  if (float_bits != 16 && float_bits != 32 && float_bits != 64) return FXPR_ERR_BAD_ARG;
  if (n == 0) return FXPR_OK;
  if (!x || !y) return FXPR_ERR_BAD_ARG;
  const float inv = 1.0f / (float)(1ull << frac_bits);
  cudaStream_t s = (cudaStream_t)stream;
  switch (int_bits) {
    case 16: return dispatch_x2f<int16_t>(x, y, float_bits, n, inv, s);
    case 32: return dispatch_x2f<int32_t>(x, y, float_bits, n, inv, s);
    case 64: return dispatch_x2f<long long>(x, y, float_bits, n, inv, s);
  }
  return FXPR_ERR_UNSUPPORTED;
}

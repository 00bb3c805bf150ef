// RMSNorm (+ fused residual add) whose sum of squares is an int64 sum of
// Q-format integers, so the result cannot depend on how the row is split over
// threads, warps or CTAs.
//
// Float steps follow fxpr_vllm/_triton/rms_norm.py:38-64 of the reference
// (fp32 add of the residual, residual rounded to the IO dtype before the second
// pass, y = (x * w) * rrms evaluated left to right); the reference's fp32
// tree-sum (rms_norm.py:41-50) is replaced by sum(Q(x^2)).  mean, sqrt and the
// reciprocal are single IEEE round-to-nearest operations.
//
// One CTA per row.  The row is read from HBM once: the values the second pass
// needs are parked in shared memory as fp32 (rows too long for shared memory
// are re-read instead).  128-bit loads/stores when the row length allows.
#include "fxp_common.cuh"

namespace fxpr {

template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) RowPack {
  T v[VEC];
};

template <typename T, int VEC, bool RESIDUAL, bool CACHE>
__global__ void __launch_bounds__(256)
rms_norm_kernel(const T* __restrict__ x, T* __restrict__ residual, const T* __restrict__ w,
                T* __restrict__ y, int hidden, float eps, float scale, float inv_scale) {
  extern __shared__ __align__(16) float row_cache[];
  __shared__ long long red[32];
  pdl_launch_dependents();
  pdl_wait();

  const int64_t base = (int64_t)blockIdx.x * hidden;
  const T* xr = x + base;
  T* rr = RESIDUAL ? residual + base : nullptr;
  T* yr = y + base;
  const int nvec = hidden / VEC;  // launcher guarantees hidden % VEC == 0

  long long acc = 0;
  for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
    RowPack<T, VEC> xv = *reinterpret_cast<const RowPack<T, VEC>*>(xr + c * VEC);
    RowPack<T, VEC> rv;
    if (RESIDUAL) rv = *reinterpret_cast<const RowPack<T, VEC>*>(rr + c * VEC);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      float v = to_f32<T>(xv.v[j]);
      if (RESIDUAL) {
        v = __fadd_rn(v, to_f32<T>(rv.v[j]));
        rv.v[j] = from_f32<T>(v);
      }
      acc += float_to_fixed<64>(__fmul_rn(v, v), scale);
      if (CACHE) row_cache[c * VEC + j] = RESIDUAL ? to_f32<T>(rv.v[j]) : v;
    }
    if (RESIDUAL) *reinterpret_cast<RowPack<T, VEC>*>(rr + c * VEC) = rv;
  }

  const long long total = block_sum_i64(acc, red);
  const float sum = fixed_to_float<long long>(total, inv_scale);
  const float mean = fmaxf(__fdiv_rn(sum, (float)hidden), 0.0f);
  const float rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));

  for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
    RowPack<T, VEC> wv = *reinterpret_cast<const RowPack<T, VEC>*>(w + c * VEC);
    RowPack<T, VEC> src;
    if (!CACHE) {
      // Same thread wrote these residual elements in pass 1, so it sees them.
      src = *reinterpret_cast<const RowPack<T, VEC>*>((RESIDUAL ? (const T*)rr : xr) + c * VEC);
    }
    RowPack<T, VEC> out;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float v = CACHE ? row_cache[c * VEC + j] : to_f32<T>(src.v[j]);
      out.v[j] = from_f32<T>(__fmul_rn(__fmul_rn(v, to_f32<T>(wv.v[j])), rrms));
    }
    *reinterpret_cast<RowPack<T, VEC>*>(yr + c * VEC) = out;
  }
}

// Row-parallel layers under tensor parallelism: the input is the all-reduced INTEGER
// accumulator tensor of the GEMM.  One kernel does what gemm_fxp_epilogue followed by
// rms_norm_fxp_residual do -- x = T(fp32(acc) * 2^-f + bias), residual <- T(x + residual),
// y = residual * w * rrms with the integer sum of squares -- with the same roundings in the
// same order, so the bits are those of the two-kernel sequence (and of TP = 1).
template <typename T, typename ACC>
__global__ void __launch_bounds__(256)
rms_norm_from_int_kernel(const ACC* __restrict__ acc_in, const T* __restrict__ bias, T* __restrict__ residual,
                         const T* __restrict__ w, T* __restrict__ y, int hidden, float eps, float gemm_inv_scale,
                         float scale, float inv_scale) {
  extern __shared__ __align__(16) float row_cache[];
  __shared__ long long red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t base = (int64_t)blockIdx.x * hidden;
  const ACC* ar = acc_in + base;
  T* rr = residual + base;
  T* yr = y + base;
  long long acc = 0;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float x = fixed_to_float<ACC>(ar[c], gemm_inv_scale);
    if (bias) x = __fadd_rn(x, to_f32<T>(bias[c]));
    const float xr = to_f32<T>(from_f32<T>(x));             // the GEMM output as the io dtype holds it
    const float v = __fadd_rn(xr, to_f32<T>(rr[c]));
    const T rt = from_f32<T>(v);
    rr[c] = rt;
    acc += float_to_fixed<64>(__fmul_rn(v, v), scale);
    row_cache[c] = to_f32<T>(rt);
  }
  const long long total = block_sum_i64(acc, red);
  const float sum = fixed_to_float<long long>(total, inv_scale);
  const float mean = fmaxf(__fdiv_rn(sum, (float)hidden), 0.0f);
  const float rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
  for (int c = threadIdx.x; c < hidden; c += blockDim.x)
    yr[c] = from_f32<T>(__fmul_rn(__fmul_rn(row_cache[c], to_f32<T>(w[c])), rrms));
}

static constexpr int kMaxCacheBytes = 64 * 1024;

template <typename T>
static int launch_rms_from_int(const void* acc, int int_bits, const void* bias, void* r, const void* w, void* y,
                               int64_t rows, int hidden, float eps, float gemm_inv, float scale, float inv,
                               cudaStream_t s) {
  const size_t cache_bytes = (size_t)hidden * sizeof(float);
  if (cache_bytes > (size_t)kMaxCacheBytes) return FXPR_ERR_UNSUPPORTED;
  int threads = 32;
  while (threads < 256 && threads * 2 <= hidden) threads *= 2;
#define FXPR_RMS_INT(ACC)                                                                               \
  do {                                                                                                  \
    auto k = rms_norm_from_int_kernel<T, ACC>;                                                          \
    if (cache_bytes > 48 * 1024) {                                                                      \
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxCacheBytes); \
      if (e != cudaSuccess) { set_last_error("rms_norm_from_int smem attribute", e); return FXPR_ERR_CUDA; } \
    }                                                                                                   \
    cudaError_t le = launch_pdl(k, dim3((unsigned)rows), dim3(threads), cache_bytes, s, 1u, (const ACC*)acc, \
                                (const T*)bias, (T*)r, (const T*)w, (T*)y, hidden, eps, gemm_inv, scale, inv); \
    if (le != cudaSuccess) { set_last_error("rms_norm_from_int launch", le); return FXPR_ERR_CUDA; }   \
  } while (0)
  if (int_bits == 64) FXPR_RMS_INT(long long);
  else if (int_bits == 32) FXPR_RMS_INT(int32_t);
  else FXPR_RMS_INT(int16_t);
#undef FXPR_RMS_INT
  return check_launch("rms_norm_from_int");
}

template <typename T, int VEC, bool RESIDUAL>
static int launch_rms(const void* x, void* r, const void* w, void* y, int64_t rows, int hidden,
                      float eps, float scale, float inv, cudaStream_t s) {
  const int nvec = hidden / VEC;
  int threads = 32;
  while (threads < 256 && threads * 2 <= nvec) threads *= 2;
  const size_t cache_bytes = (size_t)hidden * sizeof(float);
  if (cache_bytes <= (size_t)kMaxCacheBytes) {
    auto k = rms_norm_kernel<T, VEC, RESIDUAL, true>;
    if (cache_bytes > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           kMaxCacheBytes);
      if (e != cudaSuccess) { set_last_error("rms_norm smem attribute", e); return FXPR_ERR_CUDA; }
    }
    cudaError_t le = launch_pdl(k, dim3((unsigned)rows), dim3(threads), cache_bytes, s, 1u, (const T*)x, (T*)r,
                                (const T*)w, (T*)y, hidden, eps, scale, inv);
    if (le != cudaSuccess) { set_last_error("rms_norm launch", le); return FXPR_ERR_CUDA; }
  } else {
    cudaError_t le = launch_pdl(rms_norm_kernel<T, VEC, RESIDUAL, false>, dim3((unsigned)rows), dim3(threads), 0, s,
                                1u, (const T*)x, (T*)r, (const T*)w, (T*)y, hidden, eps, scale, inv);
    if (le != cudaSuccess) { set_last_error("rms_norm launch", le); return FXPR_ERR_CUDA; }
  }
  return check_launch("rms_norm");
}

template <typename T>
static int dispatch_rms(const void* x, void* r, const void* w, void* y, int64_t rows, int hidden,
                        float eps, float scale, float inv, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  const bool vec_ok = (hidden % V == 0) &&
                      ((((uintptr_t)x | (uintptr_t)r | (uintptr_t)w | (uintptr_t)y) & 15) == 0);
  if (vec_ok) {
    return r ? launch_rms<T, V, true>(x, r, w, y, rows, hidden, eps, scale, inv, s)
             : launch_rms<T, V, false>(x, r, w, y, rows, hidden, eps, scale, inv, s);
  }
  return r ? launch_rms<T, 1, true>(x, r, w, y, rows, hidden, eps, scale, inv, s)
           : launch_rms<T, 1, false>(x, r, w, y, rows, hidden, eps, scale, inv, s);
}

}  // namespace fxpr

using namespace fxpr;

extern "C" int fxpr_rms_norm(const void* x, void* residual, const void* weight, void* y, int dtype,
                             int64_t rows, int64_t hidden, float eps, int frac_bits,
                             void* stream) {
  if (rows < 0 || hidden < 0 || frac_bits < 0 || frac_bits >= 63) return FXPR_ERR_BAD_ARG;
  if (rows == 0 || hidden == 0) return FXPR_OK;
  if (!x || !weight || !y) return FXPR_ERR_BAD_ARG;
  if (hidden > (int64_t)1 << 30 || rows > 0x7fffffffLL) return FXPR_ERR_BAD_ARG;
  const float scale = (float)(1ull << frac_bits);
  const float inv = 1.0f / scale;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case FXPR_F32: return dispatch_rms<float>(x, residual, weight, y, rows, (int)hidden, eps, scale, inv, s);
    case FXPR_F16: return dispatch_rms<__half>(x, residual, weight, y, rows, (int)hidden, eps, scale, inv, s);
    case FXPR_BF16: return dispatch_rms<__nv_bfloat16>(x, residual, weight, y, rows, (int)hidden, eps, scale, inv, s);
  }
  return FXPR_ERR_UNSUPPORTED;
}

extern "C" int fxpr_rms_norm_from_int(const void* acc, int int_bits, const void* bias, void* residual,
                                      const void* weight, void* y, int dtype, int64_t rows, int64_t hidden,
                                      float eps, int gemm_frac_bits, int frac_bits, void* stream) {
  if (rows < 0 || hidden < 0 || frac_bits < 0 || frac_bits >= 63 || gemm_frac_bits < 0 || gemm_frac_bits >= 63)
    return FXPR_ERR_BAD_ARG;
  if (int_bits != 16 && int_bits != 32 && int_bits != 64) return FXPR_ERR_BAD_ARG;
  if (rows == 0 || hidden == 0) return FXPR_OK;
  if (!acc || !residual || !weight || !y) return FXPR_ERR_BAD_ARG;
  if (hidden > (int64_t)1 << 30 || rows > 0x7fffffffLL) return FXPR_ERR_BAD_ARG;
  const float scale = (float)(1ull << frac_bits);
  const float inv = 1.0f / scale;
  const float gemm_inv = 1.0f / (float)(1ull << gemm_frac_bits);
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case FXPR_F32: return launch_rms_from_int<float>(acc, int_bits, bias, residual, weight, y, rows, (int)hidden, eps, gemm_inv, scale, inv, s);
    case FXPR_F16: return launch_rms_from_int<__half>(acc, int_bits, bias, residual, weight, y, rows, (int)hidden, eps, gemm_inv, scale, inv, s);
    case FXPR_BF16: return launch_rms_from_int<__nv_bfloat16>(acc, int_bits, bias, residual, weight, y, rows, (int)hidden, eps, gemm_inv, scale, inv, s);
  }
  return FXPR_ERR_UNSUPPORTED;
}

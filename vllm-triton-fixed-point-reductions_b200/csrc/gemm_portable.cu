// Portable fixed-point GEMM on CUDA cores: any dtype, any strides, any shape.
//
// It is the route for operands the tensor-core kernel cannot take (fp32 inputs,
// leading dimensions that break TMA's 16-byte rule, very small N or K) and the
// cross-check for that kernel.  Which route a problem takes depends only on
// (dtype, N, K, strides) -- never on M -- so a row's bits never depend on the
// batch it arrives in.
//
// Semantics: fxpr_vllm/_triton/gemm.py:183-204 of the reference.  Per K-tile
// the fp32 partial is formed by adding products in ascending k with separate
// multiply and add (bit-reproducible on a CPU), quantised with float_to_fixed and
// added as an integer; the epilogue converts once, adds the bias in fp32 and
// rounds to the IO dtype.  The K tail is zero padding (adds nothing).
#include "fxp_common.cuh"

namespace fxpr {

static constexpr int kPT = 64;   // output tile edge
static constexpr int kPK = 16;   // k chunk staged in shared memory

template <typename T>
__global__ void __launch_bounds__(256)
gemm_portable_kernel(const T* __restrict__ a, const T* __restrict__ b, const T* __restrict__ bias,
                     T* __restrict__ c, void* __restrict__ c_int, float* __restrict__ partials,
                     int M, int N, int K, int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn,
                     int64_t c_sm, int int_bits, float scale, float inv_scale, int k_tile) {
  __shared__ float sa[kPK][kPT + 1];
  __shared__ float sb[kPK][kPT + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * kPT, n0 = blockIdx.x * kPT;
  long long acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0;

  const int tiles = (K + k_tile - 1) / k_tile;
  for (int t = 0; t < tiles; ++t) {
    float p[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) p[i][j] = 0.0f;
    const int k_lo = t * k_tile, k_hi = min(K, k_lo + k_tile);
    for (int kc = k_lo; kc < k_hi; kc += kPK) {
      const int kn = min(kPK, k_hi - kc);
      __syncthreads();
      for (int idx = threadIdx.x; idx < kPK * kPT; idx += 256) {
        const int kk = idx / kPT, mm = idx % kPT;  // A: consecutive threads walk m
        float v = 0.0f;
        if (kk < kn && m0 + mm < M) v = to_f32<T>(a[(int64_t)(m0 + mm) * a_sm + (int64_t)(kc + kk) * a_sk]);
        sa[kk][mm] = v;
      }
      for (int idx = threadIdx.x; idx < kPK * kPT; idx += 256) {
        const int kk = idx / kPT, nn = idx % kPT;  // B: consecutive threads walk n
        float v = 0.0f;
        if (kk < kn && n0 + nn < N) v = to_f32<T>(b[(int64_t)(kc + kk) * b_sk + (int64_t)(n0 + nn) * b_sn]);
        sb[kk][nn] = v;
      }
      __syncthreads();
      for (int kk = 0; kk < kn; ++kk) {
        float av[4], bv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty + 16 * i];
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tx + 16 * j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) p[i][j] = __fadd_rn(p[i][j], __fmul_rn(av[i], bv[j]));
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[i][j] += float_to_fixed_any(p[i][j], scale, int_bits);
        if (partials) {
          const int m = m0 + ty + 16 * i, n = n0 + tx + 16 * j;
          if (m < M && n < N) partials[((int64_t)t * M + m) * N + n] = p[i][j];
        }
      }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty + 16 * i, n = n0 + tx + 16 * j;
      if (m >= M || n >= N) continue;
      const long long q = wrap_to_bits(acc[i][j], int_bits);
      if (c_int) {
        const int64_t o = (int64_t)m * N + n;
        if (int_bits == 64) ((long long*)c_int)[o] = q;
        else if (int_bits == 32) ((int32_t*)c_int)[o] = (int32_t)q;
        else ((int16_t*)c_int)[o] = (int16_t)q;
      }
      if (c) {
        float v = fixed_to_float<long long>(q, inv_scale);
        if (bias) v = __fadd_rn(v, to_f32<T>(bias[n]));
        c[(int64_t)m * c_sm + n] = from_f32<T>(v);
      }
    }
}

// c = T(fp32(c_int) * 2^-frac + bias)
template <typename T, typename I>
__global__ void __launch_bounds__(256)
epilogue_from_int_kernel(const I* __restrict__ c_int, const T* __restrict__ bias, T* __restrict__ c,
                         int64_t M, int64_t N, int64_t c_sm, float inv_scale) {
  const int64_t total = M * N;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / N, n = i - m * N;
    float v = fixed_to_float<I>(c_int[i], inv_scale);
    if (bias) v = __fadd_rn(v, to_f32<T>(bias[n]));
    c[m * c_sm + n] = from_f32<T>(v);
  }
}

template <typename T>
int gemm_portable_launch(const void* a, const void* b, const void* bias, void* c, void* c_int,
                         float* partials, int64_t M, int64_t N, int64_t K, int64_t a_sm,
                         int64_t a_sk, int64_t b_sk, int64_t b_sn, int64_t c_sm, int int_bits,
                         int frac_bits, int k_tile, cudaStream_t s) {
  const float scale = (float)(1ull << frac_bits);
  dim3 grid((unsigned)ceil_div_i(N, kPT), (unsigned)ceil_div_i(M, kPT));
  gemm_portable_kernel<T><<<grid, 256, 0, s>>>((const T*)a, (const T*)b, (const T*)bias, (T*)c, c_int,
                                             partials, (int)M, (int)N, (int)K, a_sm, a_sk, b_sk,
                                             b_sn, c_sm, int_bits, scale, 1.0f / scale, k_tile);
  return check_launch("gemm_portable");
}

int gemm_portable(const void* a, const void* b, const void* bias, void* c, void* c_int,
                  float* partials, int dtype, int64_t M, int64_t N, int64_t K, int64_t a_sm,
                  int64_t a_sk, int64_t b_sk, int64_t b_sn, int64_t c_sm, int int_bits,
                  int frac_bits, int k_tile, cudaStream_t s) {
  switch (dtype) {
    case FXPR_F32:
      return gemm_portable_launch<float>(a, b, bias, c, c_int, partials, M, N, K, a_sm, a_sk, b_sk, b_sn, c_sm, int_bits, frac_bits, k_tile, s);
    case FXPR_F16:
      return gemm_portable_launch<__half>(a, b, bias, c, c_int, partials, M, N, K, a_sm, a_sk, b_sk, b_sn, c_sm, int_bits, frac_bits, k_tile, s);
    case FXPR_BF16:
      return gemm_portable_launch<__nv_bfloat16>(a, b, bias, c, c_int, partials, M, N, K, a_sm, a_sk, b_sk, b_sn, c_sm, int_bits, frac_bits, k_tile, s);
  }
  return FXPR_ERR_UNSUPPORTED;
}

template <typename T>
static int epilogue_dispatch(const void* c_int, int int_bits, const void* bias, void* c, int64_t M,
                             int64_t N, int64_t c_sm, float inv, cudaStream_t s) {
  const int64_t total = M * N;
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  if (int_bits == 64)
    epilogue_from_int_kernel<T, long long><<<grid, 256, 0, s>>>((const long long*)c_int, (const T*)bias, (T*)c, M, N, c_sm, inv);
  else if (int_bits == 32)
    epilogue_from_int_kernel<T, int32_t><<<grid, 256, 0, s>>>((const int32_t*)c_int, (const T*)bias, (T*)c, M, N, c_sm, inv);
  else
    epilogue_from_int_kernel<T, int16_t><<<grid, 256, 0, s>>>((const int16_t*)c_int, (const T*)bias, (T*)c, M, N, c_sm, inv);
  return check_launch("gemm_epilogue_from_int");
}

}  // namespace fxpr

using namespace fxpr;

extern "C" int fxpr_gemm_epilogue_from_int(const void* c_int, int int_bits, const void* bias,
                                           void* c, int dtype, int64_t M, int64_t N, int64_t c_sm,
                                           int frac_bits, void* stream) {
  if (M < 0 || N < 0 || frac_bits < 0 || frac_bits >= 64) return FXPR_ERR_BAD_ARG;
  if (int_bits != 16 && int_bits != 32 && int_bits != 64) return FXPR_ERR_BAD_ARG;
  if (M == 0 || N == 0) return FXPR_OK;
  if (!c_int || !c) return FXPR_ERR_BAD_ARG;
  const float inv = 1.0f / (float)(1ull << frac_bits);
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case FXPR_F32: return epilogue_dispatch<float>(c_int, int_bits, bias, c, M, N, c_sm, inv, s);
    case FXPR_F16: return epilogue_dispatch<__half>(c_int, int_bits, bias, c, M, N, c_sm, inv, s);
    case FXPR_BF16: return epilogue_dispatch<__nv_bfloat16>(c_int, int_bits, bias, c, M, N, c_sm, inv, s);
  }
  return FXPR_ERR_UNSUPPORTED;
}

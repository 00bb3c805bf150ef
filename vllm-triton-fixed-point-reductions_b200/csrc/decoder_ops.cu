// Element-wise steps either side of the attention kernel in a decoder layer, fused so that a
// decode step is a dozen launches per layer instead of fifty:
//
//   fxpr_rope_kv_write  split a fused QKV activation, apply rotate-half RoPE to Q and K in
//                       fp32, write Q to its own tensor and K/V straight into the paged
//                       cache (num_blocks, 2, page, kv_heads, head_dim).  In the reference
//                       plugin the cache write is vLLM's reshape_and_cache_flash
//                       (fxpr_vllm/attention_backend.py:253-277) and RoPE a separate vLLM op.
//   fxpr_silu_mul       act = silu(gate) * up on a fused [T, 2F] gate/up activation.
//
// No reductions here: every output element depends on one or two input elements, so these
// kernels cannot affect batch / split / tensor-parallel invariance.
#include "fxp_common.cuh"

namespace fxpr {

template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_write_kernel(const T* __restrict__ qkv, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                     const int64_t* __restrict__ pos, const int64_t* __restrict__ seq_ids,
                     const int32_t* __restrict__ block_table, int64_t bt_stride, T* __restrict__ q_out,
                     T* __restrict__ kv_cache, int q_heads, int kv_heads, int head_dim, int page,
                     int64_t kv_sblock, int64_t kv_skv, int64_t kv_sslot, int64_t kv_shead) {
  // grid: (token, slice of the work): blockIdx.y strides over the head items so that a decode
  // step (64 tokens) still fills the GPU
  pdl_launch_dependents();
  pdl_wait();
  const int64_t tok = blockIdx.x;
  const int part = blockIdx.y, parts = gridDim.y;
  const int half = head_dim / 2;
  const int64_t p = pos[tok];
  const int64_t blk = block_table[seq_ids[tok] * bt_stride + p / page];
  const int64_t slot = p % page;
  const T* row = qkv + tok * (int64_t)(q_heads + 2 * kv_heads) * head_dim;
  const float* cs = cos_t + p * half;
  const float* sn = sin_t + p * half;
  T* kdst = kv_cache + blk * kv_sblock + slot * kv_sslot;
  T* vdst = kdst + kv_skv;
  const int rope_heads = q_heads + kv_heads;
  // rotated heads: one (i, i + half) pair per item
  for (int idx = part * blockDim.x + threadIdx.x; idx < rope_heads * half; idx += parts * blockDim.x) {
    const int h = idx / half, i = idx % half;
    const float x1 = to_f32<T>(row[h * head_dim + i]);
    const float x2 = to_f32<T>(row[h * head_dim + half + i]);
    const float c = cs[i], s = sn[i];
    const T o1 = from_f32<T>(__fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s)));
    const T o2 = from_f32<T>(__fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s)));
    if (h < q_heads) {
      T* d = q_out + (tok * q_heads + h) * (int64_t)head_dim;
      d[i] = o1; d[half + i] = o2;
    } else {
      T* d = kdst + (int64_t)(h - q_heads) * kv_shead;
      d[i] = o1; d[half + i] = o2;
    }
  }
  // V heads: plain copy
  const T* vrow = row + (int64_t)rope_heads * head_dim;
  for (int idx = part * blockDim.x + threadIdx.x; idx < kv_heads * head_dim; idx += parts * blockDim.x) {
    const int h = idx / head_dim, i = idx % head_dim;
    vdst[(int64_t)h * kv_shead + i] = vrow[idx];
  }
}

template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) ActPack {
  T v[VEC];
};

// VEC elements (16 bytes when aligned) per lane and access, lanes contiguous.
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t rows, int64_t f) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t fv = f / VEC;                      // launcher guarantees f % VEC == 0
  const int64_t n = rows * fv;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / fv, c = (idx % fv) * VEC;
    const ActPack<T, VEC> g = *reinterpret_cast<const ActPack<T, VEC>*>(gu + r * 2 * f + c);
    const ActPack<T, VEC> u = *reinterpret_cast<const ActPack<T, VEC>*>(gu + r * 2 * f + f + c);
    ActPack<T, VEC> o;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      o.v[j] = silu_mul_io<T>(to_f32<T>(g.v[j]), to_f32<T>(u.v[j]));
    }
    *reinterpret_cast<ActPack<T, VEC>*>(out + r * f + c) = o;
  }
}

// gate and up interleaved by column: gu[r, 2 j] = gate_j, gu[r, 2 j + 1] = up_j
template <typename T>
__global__ void __launch_bounds__(256)
silu_mul_pairs_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t rows, int64_t f) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t n = rows * f;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x) {
    const ActPack<T, 2> p = *reinterpret_cast<const ActPack<T, 2>*>(gu + 2 * idx);
    out[idx] = silu_mul_io<T>(to_f32<T>(p.v[0]), to_f32<T>(p.v[1]));
  }
}

template <typename T>
static void launch_silu(const void* gu, void* out, int64_t rows, int64_t f, cudaStream_t s) {
  constexpr int V = 16 / (int)sizeof(T);
  const bool vec = (f % V == 0) && ((((uintptr_t)gu | (uintptr_t)out) & 15) == 0);
  const int64_t n = rows * (vec ? f / V : f);
  const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (vec) (void)launch_pdl(silu_mul_kernel<T, V>, dim3(grid), dim3(256), 0, s, 1u, (const T*)gu, (T*)out, rows, f);
  else (void)launch_pdl(silu_mul_kernel<T, 1>, dim3(grid), dim3(256), 0, s, 1u, (const T*)gu, (T*)out, rows, f);
}

}  // namespace fxpr

using namespace fxpr;

extern "C" int fxpr_rope_kv_write(const void* qkv, int dtype, const float* cos_table, const float* sin_table,
                                  const int64_t* positions, const int64_t* seq_ids,
                                  const int32_t* block_table, int64_t bt_stride, void* q_out, void* kv_cache,
                                  int64_t tokens, int q_heads, int kv_heads, int head_dim, int page_size,
                                  int64_t kv_sblock, int64_t kv_skv, int64_t kv_sslot, int64_t kv_shead,
                                  void* stream) {
  if (tokens < 0 || q_heads < 0 || kv_heads <= 0 || head_dim <= 0 || (head_dim & 1) || page_size <= 0)
    return FXPR_ERR_BAD_ARG;
  if (tokens == 0) return FXPR_OK;
  if (!qkv || !cos_table || !sin_table || !positions || !seq_ids || !block_table || !q_out || !kv_cache)
    return FXPR_ERR_BAD_ARG;
  if (tokens > 0x7fffffffLL) return FXPR_ERR_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  // enough CTAs for ~4 per SM at decode sizes, one per token for long prefills
  const int work = (q_heads + kv_heads) * (head_dim / 2);
  int parts = (work + 255) / 256;
  while (parts > 1 && tokens * parts > 148 * 8) parts = (parts + 1) / 2;
  const dim3 grid((unsigned)tokens, (unsigned)parts);
#define FXPR_ROPE(TT)                                                                                  \
  (void)launch_pdl(rope_kv_write_kernel<TT>, grid, dim3(256), 0, s, 1u,                                \
      (const TT*)qkv, cos_table, sin_table, positions, seq_ids, block_table, bt_stride, (TT*)q_out,    \
      (TT*)kv_cache, q_heads, kv_heads, head_dim, page_size, kv_sblock, kv_skv, kv_sslot, kv_shead)
  switch (dtype) {
    case FXPR_BF16: FXPR_ROPE(__nv_bfloat16); break;
    case FXPR_F16: FXPR_ROPE(__half); break;
    case FXPR_F32: FXPR_ROPE(float); break;
    default: return FXPR_ERR_UNSUPPORTED;
  }
#undef FXPR_ROPE
  return check_launch("rope_kv_write");
}

extern "C" int fxpr_silu_mul(const void* gate_up, int dtype, void* out, int64_t rows, int64_t f, void* stream) {
  if (rows < 0 || f < 0) return FXPR_ERR_BAD_ARG;
  if (rows == 0 || f == 0) return FXPR_OK;
  if (!gate_up || !out) return FXPR_ERR_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case FXPR_BF16: launch_silu<__nv_bfloat16>(gate_up, out, rows, f, s); break;
    case FXPR_F16: launch_silu<__half>(gate_up, out, rows, f, s); break;
    case FXPR_F32: launch_silu<float>(gate_up, out, rows, f, s); break;
    default: return FXPR_ERR_UNSUPPORTED;
  }
  return check_launch("silu_mul");
}

extern "C" int fxpr_silu_mul_pairs(const void* gate_up, int dtype, void* out, int64_t rows, int64_t f,
                                   void* stream) {
  if (rows < 0 || f < 0) return FXPR_ERR_BAD_ARG;
  if (rows == 0 || f == 0) return FXPR_OK;
  if (!gate_up || !out) return FXPR_ERR_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t n = rows * f;
  const unsigned grid = (unsigned)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
#define FXPR_SILU_PAIRS(TT)                                                                         \
  (void)launch_pdl(silu_mul_pairs_kernel<TT>, dim3(grid), dim3(256), 0, s, 1u, (const TT*)gate_up,  \
                   (TT*)out, rows, f)
  switch (dtype) {
    case FXPR_BF16: FXPR_SILU_PAIRS(__nv_bfloat16); break;
    case FXPR_F16: FXPR_SILU_PAIRS(__half); break;
    case FXPR_F32: FXPR_SILU_PAIRS(float); break;
    default: return FXPR_ERR_UNSUPPORTED;
  }
#undef FXPR_SILU_PAIRS
  return check_launch("silu_mul_pairs");
}

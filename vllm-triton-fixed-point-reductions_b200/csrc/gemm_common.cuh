// Argument bundle and entry points shared by the GEMM kernels and their dispatcher.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace fxpr {

struct GemmArgs {
  const void* a; const void* b; const void* bias; void* c; void* c_int; float* partials;
  int dtype; int64_t M, N, K; int64_t a_sm, a_sk, b_sk, b_sn, c_sm;
  int int_bits, frac_bits, k_tile, split_k;
  void* scratch; int64_t scratch_bytes; int32_t* status; int flags;
  unsigned long long* best = nullptr;   // fxpr_gemm_argmax: per-row (value, column) keys, see tc_common.cuh
  int64_t n_offset = 0;
};

// Tensor-core (tcgen05 / TMEM / TMA) kernel.
bool gemm_tc_supported(const GemmArgs& g);
int gemm_tc(const GemmArgs& g, cudaStream_t s);
int64_t gemm_tc_scratch_bytes(int64_t M, int64_t N, int int_bits, int split_k);

// CUDA-core kernel (any dtype / strides).
int gemm_portable(const void* a, const void* b, const void* bias, void* c, void* c_int,
                  float* partials, int dtype, int64_t M, int64_t N, int64_t K, int64_t a_sm,
                  int64_t a_sk, int64_t b_sk, int64_t b_sn, int64_t c_sm, int int_bits,
                  int frac_bits, int k_tile, cudaStream_t s);

}  // namespace fxpr

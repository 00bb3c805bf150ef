// Tensor-parallel row-parallel layers: cross-rank integer sum + GEMM epilogue + residual add +
// RMSNorm in ONE kernel over peer memory (NVLink loads and stores, no library collective).
//
// Every rank holds, in one peer-mapped allocation, its K-shard's integer accumulators
// acc [rows, hidden], the replicated residual and output rows, and a flag block.  Rows are
// divided among the ranks; a rank
//   1. tells every peer "my accumulators of this call are complete" (ready flag),
//   2. waits for all ready flags, PULLS its rows of every rank's accumulators (plain loads over
//      NVLink), adds them as integers (order-free: any rank count gives the same bits),
//   3. does what rms_norm_from_int_kernel does on the sum (same roundings, same order),
//   4. PUSHES its rows of the new residual and of the normalised output to every rank,
//   5. tells every peer "my rows have landed" (done flag) and leaves once all done flags are in,
//      so the next kernel of the stream sees complete tensors and may overwrite acc.
// Flags carry a call counter kept on the device, so a captured graph can replay the kernel.
// Every wait is bounded; when it runs out the kernel writes FXPR_ERR_TIMEOUT to the status word
// and returns without touching peer memory again.  No multicast, no multimem.
//
// The reference has no counterpart (its plugin leaves the reduce to vLLM's float all-reduce,
// vllm/model_executor/layers/linear.py); ncclAllReduce on the integer tensor stays the default.
#include <algorithm>
#include <cstring>
#include <type_traits>

#include "fxp_common.cuh"

namespace fxpr {

static constexpr int kTpMaxWorld = 8;
static constexpr int kTpThreads = 512;
static constexpr int kTpFlagWords = 32;       // ready[0..7] | done at 16 + [0..7]
static constexpr int kTpDone = 16;

struct TpPeers {
  const void* acc[kTpMaxWorld];
  void* residual[kTpMaxWorld];
  void* y[kTpMaxWorld];
  uint32_t* flags[kTpMaxWorld];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// four consecutive accumulators of a peer (system-scope loads: never a stale cached copy)
__device__ __forceinline__ void ld_peer4(const long long* p, unsigned long long (&v)[4]) {
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(v[0]), "=l"(v[1]) : "l"(p) : "memory");
  asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(v[2]), "=l"(v[3]) : "l"(p + 2) : "memory");
}
__device__ __forceinline__ void ld_peer4(const int32_t* p, uint32_t (&v)[4]) {
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "l"(p) : "memory");
}

// Spin until *flag has reached `epoch` (wrap-safe), at most `timeout` clocks.
__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch, long long timeout) {
  if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const long long t0 = clock64();
  while ((int32_t)(ld_acquire_sys(flag) - epoch) < 0) {
    if (clock64() - t0 > timeout) return false;
  }
  return true;
}

template <typename T, typename ACC>
__global__ void __launch_bounds__(kTpThreads)
tp_reduce_norm_kernel(const TpPeers peers, uint32_t* __restrict__ ctl, int world, int rank, int rows,
                      int rows_per_rank, int hidden, const T* __restrict__ bias, const T* __restrict__ w,
                      float eps, float gemm_inv_scale, float scale, float inv_scale, long long timeout,
                      int32_t* status, int local_residual) {
  using UACC = typename std::conditional<sizeof(ACC) == 8, unsigned long long, uint32_t>::type;
  extern __shared__ __align__(16) float row_cache[];
  __shared__ long long red[32];
  __shared__ int s_abort;
  __shared__ int s_last;

  pdl_launch_dependents();
  pdl_wait();
  // written once per call by the last CTA of the previous launch, after everything else
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(ctl) + 1;
  uint32_t* my_flags = peers.flags[rank];
  const int row = rank * rows_per_rank + (int)blockIdx.x;
  const bool has_row = (int)blockIdx.x < rows_per_rank && row < rows;
  if (threadIdx.x == 0) { s_abort = 0; s_last = 0; }
  // 1. this rank's accumulators were finished by the previous kernel of the stream
  if (blockIdx.x == 0 && (int)threadIdx.x < world) st_release_sys(peers.flags[threadIdx.x] + rank, epoch);
  __syncthreads();
  // 2. every rank's accumulators are ready
  if ((int)threadIdx.x < world && !wait_flag(my_flags + threadIdx.x, epoch, timeout)) {
    atomicExch(status, FXPR_ERR_TIMEOUT);
    s_abort = 1;
  }
  __syncthreads();
  const bool run = !s_abort;

  if (run && has_row) {
    const int64_t base = (int64_t)row * hidden;
    T* rr = reinterpret_cast<T*>(peers.residual[rank]) + base;
    long long sq = 0;
    for (int c = 4 * (int)threadIdx.x; c < hidden; c += 4 * kTpThreads) {
      UACC part[kTpMaxWorld][4];
#pragma unroll
      for (int p = 0; p < kTpMaxWorld; ++p)
        if (p < world) ld_peer4(reinterpret_cast<const ACC*>(peers.acc[p]) + base + c, part[p]);
      UACC sum[4] = {0, 0, 0, 0};
#pragma unroll
      for (int p = 0; p < kTpMaxWorld; ++p)
        if (p < world) {
#pragma unroll
          for (int j = 0; j < 4; ++j) sum[j] += part[p][j];    // wraps like the integer all-reduce
        }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float x = fixed_to_float<ACC>((ACC)sum[j], gemm_inv_scale);
        if (bias) x = __fadd_rn(x, to_f32<T>(bias[c + j]));
        const float xr = to_f32<T>(from_f32<T>(x));           // the GEMM output as the io dtype holds it
        const float v = __fadd_rn(xr, to_f32<T>(rr[c + j]));
        const T rt = from_f32<T>(v);
        sq += float_to_fixed<64>(__fmul_rn(v, v), scale);
        row_cache[c + j] = to_f32<T>(rt);
      }
    }
    const long long total = block_sum_i64(sq, red);
    const float sumf = fixed_to_float<long long>(total, inv_scale);
    const float mean = fmaxf(__fdiv_rn(sumf, (float)hidden), 0.0f);
    const float rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    // 4. the row goes to every rank (this one included)
    for (int c = 4 * (int)threadIdx.x; c < hidden; c += 4 * kTpThreads) {
      __align__(16) T rv[4];
      __align__(16) T yv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        rv[j] = from_f32<T>(row_cache[c + j]);
        yv[j] = from_f32<T>(__fmul_rn(__fmul_rn(row_cache[c + j], to_f32<T>(w[c + j])), rrms));
      }
#pragma unroll
      for (int p = 0; p < kTpMaxWorld; ++p)
        if (p < world) {
          T* rp = reinterpret_cast<T*>(peers.residual[p]) + base + c;
          T* yp = reinterpret_cast<T*>(peers.y[p]) + base + c;
          const bool res_too = !local_residual || p == rank;   // a row-sharded residual stays at home
          if (sizeof(T) == 2) {
            if (res_too) *reinterpret_cast<uint2*>(rp) = *reinterpret_cast<const uint2*>(rv);
            *reinterpret_cast<uint2*>(yp) = *reinterpret_cast<const uint2*>(yv);
          } else {
            if (res_too) *reinterpret_cast<uint4*>(rp) = *reinterpret_cast<const uint4*>(rv);
            *reinterpret_cast<uint4*>(yp) = *reinterpret_cast<const uint4*>(yv);
          }
        }
    }
  }
  // 5. pushes visible system-wide before the done flag
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(ctl + 1, 1u);
    s_last = prev + 1 == gridDim.x;
  }
  __syncthreads();
  if (!s_last) return;
  // last CTA of this rank: all its rows are out
  __threadfence();
  if (run && (int)threadIdx.x < world) st_release_sys(peers.flags[threadIdx.x] + kTpDone + rank, epoch);
  if (run && (int)threadIdx.x < world && !wait_flag(my_flags + kTpDone + threadIdx.x, epoch, timeout))
    atomicExch(status, FXPR_ERR_TIMEOUT);
  __syncthreads();
  if (threadIdx.x == 0) {
    ctl[1] = 0;
    *reinterpret_cast<volatile uint32_t*>(ctl) = epoch;
  }
}

template <typename T>
static int launch_tp(const TpPeers& peers, void* ctl, int world, int rank, int int_bits, const void* bias,
                     const void* w, int64_t rows, int hidden, float eps, float gemm_inv, float scale, float inv,
                     long long timeout, int32_t* status, int local_residual, cudaStream_t s) {
  const int rows_per = (int)((rows + world - 1) / world);
  const int mine = (int)std::max<int64_t>(0, std::min<int64_t>(rows_per, rows - (int64_t)rank * rows_per));
  const unsigned grid = (unsigned)std::max(1, mine);
  const size_t smem = (size_t)hidden * sizeof(float);
#define FXPR_TP_LAUNCH(ACC)                                                                           \
  do {                                                                                                \
    auto k = tp_reduce_norm_kernel<T, ACC>;                                                           \
    if (smem > 48 * 1024) {                                                                           \
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024); \
      if (e != cudaSuccess) { set_last_error("tp_reduce_norm smem attribute", e); return FXPR_ERR_CUDA; } \
    }                                                                                                 \
    cudaError_t le = launch_pdl(k, dim3(grid), dim3(kTpThreads), smem, s, 1u, peers, (uint32_t*)ctl, world, rank, \
                                (int)rows, rows_per, hidden, (const T*)bias, (const T*)w, eps, gemm_inv, scale,  \
                                inv, timeout, status, local_residual);                                \
    if (le != cudaSuccess) { set_last_error("tp_reduce_norm launch", le); return FXPR_ERR_CUDA; }     \
  } while (0)
  if (int_bits == 64) FXPR_TP_LAUNCH(long long);
  else FXPR_TP_LAUNCH(int32_t);
#undef FXPR_TP_LAUNCH
  return check_launch("tp_reduce_norm");
}

}  // namespace fxpr

using namespace fxpr;

extern "C" int fxpr_tp_buffer_bytes(int64_t max_rows, int64_t hidden, int int_bits, int dtype,
                                    int64_t* acc_offset, int64_t* residual_offset, int64_t* y_offset,
                                    int64_t* flags_offset, int64_t* total) {
  if (max_rows <= 0 || hidden <= 0 || (int_bits != 32 && int_bits != 64)) return FXPR_ERR_BAD_ARG;
  const int64_t io = dtype == FXPR_F32 ? 4 : 2;
  auto up = [](int64_t v) { return (v + 255) / 256 * 256; };
  const int64_t acc = 0;
  const int64_t res = up(acc + max_rows * hidden * (int_bits / 8));
  const int64_t y = up(res + max_rows * hidden * io);
  const int64_t fl = up(y + max_rows * hidden * io);
  if (acc_offset) *acc_offset = acc;
  if (residual_offset) *residual_offset = res;
  if (y_offset) *y_offset = y;
  if (flags_offset) *flags_offset = fl;
  if (total) *total = fl + 256;
  return FXPR_OK;
}

extern "C" int fxpr_tp_alloc(int64_t bytes, void** ptr, void* handle64) {
  if (bytes <= 0 || !ptr || !handle64) return FXPR_ERR_BAD_ARG;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) { set_last_error("tp buffer cudaMalloc", e); return FXPR_ERR_CUDA; }
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    set_last_error("tp buffer export", e);
    cudaFree(p);
    return FXPR_ERR_CUDA;
  }
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, sizeof(h));
  *ptr = p;
  return FXPR_OK;
}

extern "C" int fxpr_tp_open(const void* handle64, void** ptr) {
  if (!handle64 || !ptr) return FXPR_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) { set_last_error("tp buffer open", e); return FXPR_ERR_CUDA; }
  return FXPR_OK;
}

extern "C" int fxpr_tp_close(void* ptr) {
  if (!ptr) return FXPR_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) { set_last_error("tp buffer close", e); return FXPR_ERR_CUDA; }
  return FXPR_OK;
}

extern "C" int fxpr_tp_free(void* ptr) {
  if (!ptr) return FXPR_OK;
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) { set_last_error("tp buffer free", e); return FXPR_ERR_CUDA; }
  return FXPR_OK;
}

extern "C" int fxpr_tp_reduce_norm(const void* const* peer_bases, int world, int rank, void* ctl,
                                   int64_t acc_offset, int64_t residual_offset, int64_t y_offset,
                                   int64_t flags_offset, int int_bits, const void* bias, const void* weight,
                                   int dtype, int64_t rows, int64_t hidden, float eps, int gemm_frac_bits,
                                   int frac_bits, int64_t timeout_cycles, int flags, int32_t* status,
                                   void* stream) {
  if (!peer_bases || !ctl || !weight || !status) return FXPR_ERR_BAD_ARG;
  if (world < 1 || world > kTpMaxWorld || rank < 0 || rank >= world) return FXPR_ERR_BAD_ARG;
  if (rows < 0 || hidden <= 0 || frac_bits < 0 || frac_bits >= 63 || gemm_frac_bits < 0 || gemm_frac_bits >= 63)
    return FXPR_ERR_BAD_ARG;
  if (int_bits != 32 && int_bits != 64) return FXPR_ERR_UNSUPPORTED;
  if (hidden % 4 || hidden * 4 > 64 * 1024 || rows > 0x7fffffffLL / hidden) return FXPR_ERR_UNSUPPORTED;
  if (timeout_cycles <= 0) timeout_cycles = 2000000000LL;       // about a second
  TpPeers peers;
  for (int p = 0; p < kTpMaxWorld; ++p) {
    const char* b = p < world ? (const char*)peer_bases[p] : nullptr;
    if (p < world && !b) return FXPR_ERR_BAD_ARG;
    peers.acc[p] = b ? b + acc_offset : nullptr;
    peers.residual[p] = b ? (void*)(b + residual_offset) : nullptr;
    peers.y[p] = b ? (void*)(b + y_offset) : nullptr;
    peers.flags[p] = b ? (uint32_t*)(b + flags_offset) : nullptr;
  }
  const float scale = (float)(1ull << frac_bits);
  const float inv = 1.0f / scale;
  const float gemm_inv = 1.0f / (float)(1ull << gemm_frac_bits);
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case FXPR_F32: return launch_tp<float>(peers, ctl, world, rank, int_bits, bias, weight, rows, (int)hidden, eps, gemm_inv, scale, inv, timeout_cycles, status, (flags & FXPR_TP_LOCAL_RESIDUAL) ? 1 : 0, s);
    case FXPR_F16: return launch_tp<__half>(peers, ctl, world, rank, int_bits, bias, weight, rows, (int)hidden, eps, gemm_inv, scale, inv, timeout_cycles, status, (flags & FXPR_TP_LOCAL_RESIDUAL) ? 1 : 0, s);
    case FXPR_BF16: return launch_tp<__nv_bfloat16>(peers, ctl, world, rank, int_bits, bias, weight, rows, (int)hidden, eps, gemm_inv, scale, inv, timeout_cycles, status, (flags & FXPR_TP_LOCAL_RESIDUAL) ? 1 : 0, s);
  }
  return FXPR_ERR_UNSUPPORTED;
}

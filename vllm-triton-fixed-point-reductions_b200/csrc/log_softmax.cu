// Row-wise log-softmax with an integer (int64 Q-format) sum of exponentials.
//
//   m = max_i x_i (exact)          e_i = exp2_det((x_i - m) * log2 e)
//   S = sum_i Q(e_i)  (int64)      y_i = (x_i - m) - log_det(fp32(S) * 2^-frac)
//
// The reference has no such kernel (its README lists sampler files that are
// absent); this is the order-free replacement for the float log_softmax of
// vLLM's Sampler.compute_logprobs.
//
// A row is split over a thread-block cluster of 1..16 CTAs; each CTA keeps its
// slice in shared memory, so HBM is read once and written once.  The row maximum
// and the integer sum are exchanged through distributed shared memory (max and
// integer add are order-free).  Two kernels: log_softmax_bulk_kernel for 16-byte
// aligned rows with slices of at most 8192 elements (persistent clusters, bulk
// asynchronous copies), log_softmax_kernel for everything else; rows too long for
// 16 x shared memory re-read the slice there.
#include <cooperative_groups.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>

#include "fxp_common.cuh"

namespace cg = cooperative_groups;

namespace fxpr {

static constexpr int kLsmThreads = 256;
static constexpr int kLsmMaxSliceBytes = 200 * 1024;

template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) LsPack {
  T v[VEC];
};

// slice: elements [begin, end) of the row handled by this CTA; `begin` is a
// multiple of VEC so vector accesses stay aligned.
template <typename T, int VEC, bool CACHE>
__global__ void __launch_bounds__(kLsmThreads)
log_softmax_kernel(const T* __restrict__ x, float* __restrict__ y, int cols, int slice_len,
                   float scale, float inv_scale, bool wide_q) {
  extern __shared__ __align__(16) float slice[];
  __shared__ long long red_i[32];
  __shared__ float red_f[32];
  __shared__ float xchg_max;        // read by peer CTAs
  __shared__ long long xchg_sum;    // read by peer CTAs
  __shared__ float bc_log;

  cg::cluster_group cluster = cg::this_cluster();
  const unsigned csize = cluster.num_blocks();
  const unsigned crank = cluster.block_rank();
  const int64_t row = blockIdx.x / csize;
  const int begin = (int)crank * slice_len;
  const int end = min(cols, begin + slice_len);
  const int len = max(0, end - begin);
  const T* xr = x + row * (int64_t)cols + begin;
  float* yr = y + row * (int64_t)cols + begin;
  const int nvec = len / VEC;
  const float ninf = -__int_as_float(0x7f800000);

  // ---- phase 1: load the slice, local maximum --------------------------------
  float lmax = ninf;
  for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
    LsPack<T, VEC> p = *reinterpret_cast<const LsPack<T, VEC>*>(xr + c * VEC);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      const float v = to_f32<T>(p.v[j]);
      if (CACHE) slice[c * VEC + j] = v;
      lmax = fmaxf(lmax, v);
    }
  }
  for (int i = nvec * VEC + threadIdx.x; i < len; i += blockDim.x) {
    const float v = to_f32<T>(xr[i]);
    if (CACHE) slice[i] = v;
    lmax = fmaxf(lmax, v);
  }
  lmax = block_max_f32(lmax, red_f);
  if (threadIdx.x == 0) xchg_max = lmax;
  cluster.sync();
  float gmax = ninf;
  for (unsigned r = 0; r < csize; ++r) gmax = fmaxf(gmax, *cluster.map_shared_rank(&xchg_max, r));

  // ---- phase 2: integer sum of exponentials ------------------------------------
  unsigned long long acc = 0;
  auto add_one = [&](float v) {
    const float e = exp2_det(__fmul_rn(__fsub_rn(v, gmax), FXPR_LOG2E_F32));
    // e is in [0, 1]: it fits 32 bits unless frac_bits > 30.
    if (wide_q) acc += (unsigned long long)float_to_fixed<64>(e, scale);
    else acc += (unsigned long long)(long long)float_to_fixed<32>(e, scale);
  };
  // two logits per instruction (packed sub/mul/add round each lane as the scalar forms do)
  const uint64_t gmax2 = f2_pack(gmax, gmax), log2e2 = f2_pack(FXPR_LOG2E_F32, FXPR_LOG2E_F32);
  auto add_two = [&](float a, float b) {
    float t0, t1, e0, e1;
    f2_unpack(f2_mul(f2_sub(f2_pack(a, b), gmax2), log2e2), t0, t1);
    f2_unpack(exp2_det_nonpos_pair(t0, t1), e0, e1);
    if (wide_q) acc += (unsigned long long)float_to_fixed<64>(e0, scale) + (unsigned long long)float_to_fixed<64>(e1, scale);
    else acc += (unsigned long long)(long long)float_to_fixed<32>(e0, scale) + (unsigned long long)(long long)float_to_fixed<32>(e1, scale);
  };
  if (CACHE) {
    // four independent exp chains per thread and iteration (the polynomial is a long
    // dependent chain; integer addition makes the visiting order irrelevant)
    const int n4 = len / 4;
    for (int c = threadIdx.x; c < n4; c += blockDim.x) {
      const float4 v = *reinterpret_cast<const float4*>(slice + c * 4);
      add_two(v.x, v.y); add_two(v.z, v.w);
    }
    for (int i = n4 * 4 + threadIdx.x; i < len; i += blockDim.x) add_one(slice[i]);
  } else {
    for (int i = threadIdx.x; i < len; i += blockDim.x) add_one(to_f32<T>(xr[i]));
  }
  const long long lsum = block_sum_i64((long long)acc, red_i);
  if (threadIdx.x == 0) xchg_sum = lsum;
  cluster.sync();
  if (threadIdx.x == 0) {
    long long total = 0;
    for (unsigned r = 0; r < csize; ++r) total += *cluster.map_shared_rank(&xchg_sum, r);
    bc_log = log_det(fixed_to_float<long long>(total, inv_scale));
  }
  __syncthreads();
  const float lg = bc_log;

  // ---- phase 3: write the slice ---------------------------------------------------
  const bool y_vec = (((uintptr_t)yr) & 15) == 0;
  if (CACHE && y_vec) {
    const int n4 = len / 4;
    for (int c = threadIdx.x; c < n4; c += blockDim.x) {
      float4 v = *reinterpret_cast<const float4*>(slice + c * 4);
      v.x = __fsub_rn(__fsub_rn(v.x, gmax), lg);
      v.y = __fsub_rn(__fsub_rn(v.y, gmax), lg);
      v.z = __fsub_rn(__fsub_rn(v.z, gmax), lg);
      v.w = __fsub_rn(__fsub_rn(v.w, gmax), lg);
      *reinterpret_cast<float4*>(yr + c * 4) = v;
    }
    for (int i = n4 * 4 + threadIdx.x; i < len; i += blockDim.x)
      yr[i] = __fsub_rn(__fsub_rn(slice[i], gmax), lg);
  } else {
    for (int i = threadIdx.x; i < len; i += blockDim.x) {
      const float v = CACHE ? slice[i] : to_f32<T>(xr[i]);
      yr[i] = __fsub_rn(__fsub_rn(v, gmax), lg);
    }
  }
  // Peers may still be reading this CTA's exchange slots.
  cluster.sync();
}

// ---- bulk-copy variant ------------------------------------------------------------
// The slice travels global -> shared memory as bulk asynchronous copies (one per 4 KB, each
// with its own mbarrier) issued by one thread at kernel start, so no registers are tied up by
// loads in flight and six CTAs (192 KB of slices) share an SM.  The row maximum and the integer
// sum are PUSHED into every peer's shared memory before a cluster barrier, so after the barrier
// each CTA reads only its own memory and may exit without a trailing cluster barrier.
// Same per-element arithmetic as the kernels above, hence the same bits.
static constexpr int kLsmBulkRows = 8;                       // 4 KB pieces per slice
static constexpr int kLsmPiece = kLsmThreads * 16;           // bytes: one 16-byte vector per thread

__device__ __forceinline__ void cluster_arrive_relaxed() {
  asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t peer_shared(const void* local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
  return r;
}
// Bounded: a bulk copy of mapped memory always completes; the limit only keeps a fault elsewhere
// from turning into a hang.
__device__ __forceinline__ bool lsm_wait(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < (1 << 20); ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}

template <typename T>
__global__ void __launch_bounds__(kLsmThreads, 6)
log_softmax_bulk_kernel(const T* __restrict__ x, float* __restrict__ y, int64_t rows, int cols,
                        int slice_len, float scale, float inv_scale, bool wide_q) {
  constexpr int VEC = 16 / sizeof(T);
  extern __shared__ __align__(128) uint8_t lsm_slice[];
  __shared__ __align__(8) uint64_t bars[kLsmBulkRows];
  __shared__ float red_f[kLsmThreads / 32];
  __shared__ long long red_i[kLsmThreads / 32];
  __shared__ float xchg_max[16];            // written by peer CTAs
  __shared__ long long xchg_sum[16];        // written by peer CTAs

  uint32_t csize, crank;
  asm("mov.u32 %0, %%cluster_nctarank;" : "=r"(csize));
  asm("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t nclusters = gridDim.x / csize;
  const int begin = (int)crank * slice_len;
  const int len = max(0, min(cols, begin + slice_len) - begin);   // multiple of VEC
  const int nvec = len / VEC;
  const int npieces = (nvec + kLsmThreads - 1) / kLsmThreads;
  const int total_bytes = len * (int)sizeof(T);
  const float ninf = -__int_as_float(0x7f800000);
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(lsm_slice);

  // global -> shared memory: thread r < npieces copies 4 KB piece r and arms its barrier
  auto issue_load = [&](int64_t row) {
    const int r = (int)threadIdx.x;
    if (r < npieces) {
      const uint8_t* src = reinterpret_cast<const uint8_t*>(x + row * (int64_t)cols + begin);
      const int bytes = min(kLsmPiece, total_bytes - r * kLsmPiece);
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                   ::"r"(bar0 + 8 * r), "r"(bytes) : "memory");
      asm volatile(
          "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
          ::"r"(dst + r * kLsmPiece), "l"(src + (size_t)r * kLsmPiece), "r"(bytes),
            "r"(bar0 + 8 * r) : "memory");
    }
  };

  cluster_arrive_relaxed();                 // "this CTA runs": awaited before the first remote store
  int64_t row = blockIdx.x / csize;
  if ((int)threadIdx.x < npieces) {         // each issuing thread initialises the barrier it arms
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0 + 8 * threadIdx.x));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (row < rows) issue_load(row);
  __syncthreads();                          // barriers initialised before anyone polls them
  cluster_wait_acquire();                   // every CTA of the cluster has started

  const LsPack<T, VEC>* vecs = reinterpret_cast<const LsPack<T, VEC>*>(lsm_slice);
  const bool magic_ok = scale <= 2097152.0f;
  const float magic = __uint_as_float(0x4B400000u);
  const uint64_t log2e2 = f2_pack(FXPR_LOG2E_F32, FXPR_LOG2E_F32);
  const uint64_t scale2 = f2_pack(scale, scale), magic2 = f2_pack(magic, magic);

  // A cluster walks rows cluster_id, cluster_id + nclusters, ...; while it works on one row the
  // next row's slice is pulled into L2, so the copy into shared memory that follows is short.
  for (uint32_t parity = 0; row < rows; row += nclusters, parity ^= 1) {
    float* yr = y + row * (int64_t)cols + begin;
    if (threadIdx.x < npieces && row + nclusters < rows) {
      const uint8_t* nxt = reinterpret_cast<const uint8_t*>(x + (row + nclusters) * (int64_t)cols + begin)
                           + (size_t)threadIdx.x * kLsmPiece;
      const int bytes = min(kLsmPiece, total_bytes - (int)threadIdx.x * kLsmPiece);
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(nxt), "r"(bytes) : "memory");
    }

    // ---- phase 1: maximum, piece by piece as the copies land -------------------------------
    float lmax = ninf;
    bool ok = true;
    for (int r = 0; r < npieces; ++r) {
      ok = lsm_wait(bar0 + 8 * r, parity) && ok;
      const int c = r * kLsmThreads + (int)threadIdx.x;
      if (c < nvec) {
        const LsPack<T, VEC> pk = vecs[c];
#pragma unroll
        for (int j = 0; j < VEC; ++j) lmax = fmaxf(lmax, to_f32<T>(pk.v[j]));
      }
    }
    lmax = warp_max_f32(lmax);
    if (lane == 0) red_f[warp] = lmax;
    const int failed = __syncthreads_or(!ok);
    if (warp == 0) {
      float v = lane < kLsmThreads / 32 ? red_f[lane] : ninf;
      v = warp_max_f32(v);
      if (lane < (int)csize)
        asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(peer_shared(&xchg_max[crank], lane)), "f"(v) : "memory");
    }
    cluster_arrive_release();
    cluster_wait_acquire();
    const float gmax = warp_max_f32(lane < (int)csize ? xchg_max[lane] : ninf);

    // ---- phase 2: integer sum of exponentials ---------------------------------------------
    // e is in [0, 1]: for frac_bits <= 21 its Q-format value is the low mantissa of
    // fma(e, 2^f, 1.5 * 2^23) (exactly rint-half-even, as cvt.rni gives), so the raw bit patterns
    // are summed in 32 bits and count * MAGIC is taken out once (at most 32 terms of <= 2^21).
    unsigned long long acc = 0;
    uint32_t acc32 = 0, cnt = 0;
    const uint64_t gmax2 = f2_pack(gmax, gmax);
#pragma unroll 2
    for (int r = 0; r < npieces; ++r) {
      const int c = r * kLsmThreads + (int)threadIdx.x;
      if (c < nvec) {
        const LsPack<T, VEC> pk = vecs[c];
#pragma unroll
        for (int j = 0; j < VEC; j += 2) {
          float t0, t1;
          f2_unpack(f2_mul(f2_sub(f2_pack(to_f32<T>(pk.v[j]), to_f32<T>(pk.v[j + 1])), gmax2), log2e2), t0, t1);
          const uint64_t e2 = exp2_det_nonpos_pair(t0, t1);
          if (magic_ok) {
            const uint64_t q = f2_fma(e2, scale2, magic2);
            acc32 += (uint32_t)q + (uint32_t)(q >> 32);
          } else {
            float e0, e1;
            f2_unpack(e2, e0, e1);
            if (wide_q) acc += (unsigned long long)float_to_fixed<64>(e0, scale) + (unsigned long long)float_to_fixed<64>(e1, scale);
            else acc += (unsigned long long)(long long)float_to_fixed<32>(e0, scale) + (unsigned long long)(long long)float_to_fixed<32>(e1, scale);
          }
        }
        cnt += VEC;
      }
    }
    if (magic_ok) acc = (unsigned long long)(uint32_t)(acc32 - cnt * 0x4B400000u);
    const long long wsum = warp_sum_i64((long long)acc);
    if (lane == 0) red_i[warp] = wsum;
    __syncthreads();
    if (warp == 0) {
      long long v = lane < kLsmThreads / 32 ? red_i[lane] : 0;
      v = warp_sum_i64(v);
      if (lane < (int)csize)
        asm volatile("st.shared::cluster.s64 [%0], %1;" ::"r"(peer_shared(&xchg_sum[crank], lane)), "l"(v) : "memory");
    }
    cluster_arrive_release();
    cluster_wait_acquire();
    const long long total = warp_sum_i64(lane < (int)csize ? xchg_sum[lane] : 0);
    float lg = log_det(fixed_to_float<long long>(total, inv_scale));   // once per warp, no block barrier
    if (failed) lg = __int_as_float(0x7fc00000);
    const uint64_t lg2 = f2_pack(lg, lg);

    // ---- phase 3: write the slice --------------------------------------------------------------
#pragma unroll 4
    for (int r = 0; r < npieces; ++r) {
      const int c = r * kLsmThreads + (int)threadIdx.x;
      if (c < nvec) {
        const LsPack<T, VEC> pk = vecs[c];
#pragma unroll
        for (int j4 = 0; j4 < VEC / 4; ++j4) {
          float4 o;
          f2_unpack(f2_sub(f2_sub(f2_pack(to_f32<T>(pk.v[j4 * 4 + 0]), to_f32<T>(pk.v[j4 * 4 + 1])), gmax2), lg2), o.x, o.y);
          f2_unpack(f2_sub(f2_sub(f2_pack(to_f32<T>(pk.v[j4 * 4 + 2]), to_f32<T>(pk.v[j4 * 4 + 3])), gmax2), lg2), o.z, o.w);
          *reinterpret_cast<float4*>(yr + c * VEC + j4 * 4) = o;
        }
      }
    }
    if (row + nclusters < rows) {
      __syncthreads();                      // every thread is done reading the slice
      issue_load(row + nclusters);
    }
  }
}

template <typename T>
static int launch_lsm(const void* x, float* y, int64_t rows, int cols, float scale, float inv,
                      bool wide_q, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  int csize = 1;
  auto slice_of = [&](int c) {
    int sl = (cols + c - 1) / c;
    return ((sl + 15) / 16) * 16;  // multiple of 16 elements: aligned for every dtype
  };
  // up to 16 CTAs per row (16 needs the non-portable cluster attribute): 32 KB slices
  // keep ~6 CTAs resident per SM, so loads, exp work and stores of different rows overlap
  while (csize < 16 && (size_t)slice_of(csize) * 4 > 32 * 1024) csize *= 2;
  int slice_len = slice_of(csize);
  const bool cache = (size_t)slice_len * 4 <= (size_t)kLsmMaxSliceBytes;
  const bool vec_ok = (cols % V == 0) && ((((uintptr_t)x) & 15) == 0);
  const size_t smem = cache ? (size_t)slice_len * 4 : 0;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows * csize));
  cfg.blockDim = dim3(kLsmThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = csize;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;

  const T* xp = (const T*)x;
  cudaError_t e;
  // 16-byte aligned rows whose slices fit eight 4 KB pieces take the bulk-copy kernel (y rows are
  // 16-byte aligned whenever x rows are: cols % V == 0 with V >= 4)
  if (vec_ok && slice_len <= 32 * kLsmThreads && ((((uintptr_t)y) & 15) == 0) && cols % 4 == 0) {
    auto k = log_softmax_bulk_kernel<T>;
    if (csize > 8) {
      e = cudaFuncSetAttribute(k, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
      if (e != cudaSuccess) { set_last_error("log_softmax cluster attribute", e); return FXPR_ERR_CUDA; }
    }
    cfg.dynamicSmemBytes = (size_t)slice_len * sizeof(T);
    // as many clusters as the device keeps resident at once; each walks several rows
    static std::mutex mu;
    static std::map<std::tuple<int, int, size_t>, int> resident;
    int dev = 0;
    cudaGetDevice(&dev);
    int ncl = 0;
    {
      std::lock_guard<std::mutex> lk(mu);
      auto key = std::make_tuple(dev, csize, (size_t)cfg.dynamicSmemBytes);
      auto it = resident.find(key);
      if (it == resident.end()) {
        cfg.gridDim = dim3((unsigned)csize);
        e = cudaOccupancyMaxActiveClusters(&ncl, k, &cfg);
        if (e != cudaSuccess || ncl < 1) { (void)cudaGetLastError(); ncl = 0; }
        resident[key] = ncl;
      } else {
        ncl = it->second;
      }
    }
    const int64_t nclusters = ncl > 0 ? std::min<int64_t>(rows, ncl) : rows;
    cfg.gridDim = dim3((unsigned)(nclusters * csize));
    e = cudaLaunchKernelEx(&cfg, k, xp, y, rows, cols, slice_len, scale, inv, wide_q);
    if (e != cudaSuccess) { set_last_error("log_softmax launch", e); return FXPR_ERR_CUDA; }
    return check_launch("log_softmax");
  }
#define FXPR_LSM_LAUNCH(VV, CC)                                                              \
  do {                                                                                       \
    auto k = log_softmax_kernel<T, VV, CC>;                                                  \
    if (smem > 48 * 1024) {                                                                  \
      e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize,               \
                               kLsmMaxSliceBytes);                                           \
      if (e != cudaSuccess) { set_last_error("log_softmax smem attribute", e); return FXPR_ERR_CUDA; } \
    }                                                                                        \
    if (csize > 8) {                                                                         \
      e = cudaFuncSetAttribute(k, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);        \
      if (e != cudaSuccess) { set_last_error("log_softmax cluster attribute", e); return FXPR_ERR_CUDA; } \
    }                                                                                        \
    e = cudaLaunchKernelEx(&cfg, k, xp, y, cols, slice_len, scale, inv, wide_q);             \
  } while (0)
  if (cache) {
    if (vec_ok) FXPR_LSM_LAUNCH(V, true); else FXPR_LSM_LAUNCH(1, true);
  } else {
    if (vec_ok) FXPR_LSM_LAUNCH(V, false); else FXPR_LSM_LAUNCH(1, false);
  }
#undef FXPR_LSM_LAUNCH
  if (e != cudaSuccess) { set_last_error("log_softmax launch", e); return FXPR_ERR_CUDA; }
  return check_launch("log_softmax");
}

}  // namespace fxpr

using namespace fxpr;

extern "C" int fxpr_log_softmax(const void* x, int x_dtype, float* y, int64_t rows, int64_t cols,
                                int frac_bits, void* stream) {
  if (rows < 0 || cols < 0 || frac_bits < 0 || frac_bits > 32) return FXPR_ERR_BAD_ARG;
  if (rows == 0 || cols == 0) return FXPR_OK;
  if (!x || !y) return FXPR_ERR_BAD_ARG;
  if (cols > (int64_t)1 << 30 || rows * 16 > 0x7fffffffLL) return FXPR_ERR_BAD_ARG;
  const float scale = (float)(1ull << frac_bits);
  const float inv = 1.0f / scale;
  const bool wide_q = frac_bits > 30;
  cudaStream_t s = (cudaStream_t)stream;
  switch (x_dtype) {
    case FXPR_F32: return launch_lsm<float>(x, y, rows, (int)cols, scale, inv, wide_q, s);
    case FXPR_F16: return launch_lsm<__half>(x, y, rows, (int)cols, scale, inv, wide_q, s);
    case FXPR_BF16: return launch_lsm<__nv_bfloat16>(x, y, rows, (int)cols, scale, inv, wide_q, s);
  }
  return FXPR_ERR_UNSUPPORTED;
}

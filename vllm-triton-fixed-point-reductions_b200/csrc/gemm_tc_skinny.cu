// Tensor-core fixed-point GEMM for decode shapes (M <= 64 rows of activations against a
// large weight matrix): the operands swap roles.  The 128-row side of tcgen05.mma carries
// 128 output COLUMNS (weights), its N side the (padded) 64 activation rows:
//
//     D^T[n, m] = sum_k W[k, n] * X[m, k]        M_mma = 128 (n), N_mma = 64 (m), K = 16
//
// so no tensor work is spent on padding rows, a K-tile's accumulator is 128 x 64 instead of
// 128 x 128 (a quarter of the conversion work per byte of weights), and TMEM holds EIGHT
// accumulators: k_tile 64 runs four groups of two (a 128-deep super-stage per hand-off, as
// in gemm_tc_fast.cu), k_tile 128 eight groups of one.  Four 48 KB shared-memory stages.
// The kernel is bound by streaming the weights from HBM once.
//
// Numerics are those of the other tensor-core kernels: one fp32 partial per K-tile and
// output element from tcgen05.mma (kind::f16, fp32 accumulate, fresh accumulator per
// K-tile), rint-half-even conversion to Q-format on the FP32 pipe with the exact fix-up for
// out-of-range partials, wrap-around integer sums; split-K through per-split partial planes.
// An output element's bits do not depend on M, on the route or on the split count.
#include <cooperative_groups.h>
#include <cuda.h>

#include "fxp_common.cuh"
#include "gemm_common.cuh"
#include "tc_common.cuh"
#include "gemm_tc_fast_common.cuh"

namespace cg = cooperative_groups;

namespace fxpr {

static constexpr int kSkMP = 64;                          // activation rows per tile (MMA N)
static constexpr int kSkWarps = 2 + 8;                    // producer, issuer, 8 epilogue warps
static constexpr int kSkStages = 4;
static constexpr int kSkWBytes = 2 * 128 * kBK * 2;       // weights: two 64-deep halves, 128 columns
static constexpr int kSkXBytes = 2 * kSkMP * kBK * 2;     // activations: two 64-deep halves, 64 rows
static constexpr int kSkSSBytes = kSkWBytes + kSkXBytes;  // 48 KB per super-stage
static constexpr int kSkGroups = 8;                       // barrier slots (groups in use: 4 or 8)

// CLUSTER: split-K as a thread-block cluster (grid = splits x tiles, one item per CTA): the
// ranks leave their integer partials in their own shared memory and every rank sums a slice of
// the rows over its peers through distributed shared memory -- no global scratch, no fences.
template <typename T, bool CLUSTER>
__global__ void __launch_bounds__(kSkWarps * 32, 1)
gemm_tc_skinny_kernel(const __grid_constant__ CUtensorMap tma_w, const __grid_constant__ CUtensorMap tma_x,
                      const TcParams p, const int zero /* always 0: keeps the side arrays in local memory */) {
  constexpr int STAGES = kSkStages;
  constexpr int MP = kSkMP;
  constexpr int EPIW = 8;
  constexpr int kCols = MP / (EPIW / 4);                 // 32 activation rows per epilogue thread
  constexpr int kBarOffset = STAGES * kSkSSBytes;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kBarOffset;
  const uint32_t full0 = bar_base, empty0 = bar_base + 8u * STAGES;
  const uint32_t tfull0 = bar_base + 8u * (2 * STAGES), tempty0 = tfull0 + 8u * kSkGroups;
  constexpr int kMisc = 8 * (2 * STAGES + 2 * kSkGroups);
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem_gen + kBarOffset + kMisc);
  volatile int* abort_flag = (volatile int*)(smem_gen + kBarOffset + kMisc + 8);
  const uint32_t epi_bar = bar_base + kMisc + 16u;
  volatile int* s_last = (volatile int*)(smem_gen + kBarOffset + kMisc + 24);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  pdl_launch_dependents();                               // the next kernel may start its own setup
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8u * s, 1); mbar_init(empty0 + 8u * s, 1); }
    for (int b = 0; b < kSkGroups; ++b) { mbar_init(tfull0 + 8u * b, 1); mbar_init(tempty0 + 8u * b, EPIW); }
    mbar_init(epi_bar, EPIW);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32((const void*)tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Barriers, tensor memory and descriptors are set up; from here on the kernel reads what
  // earlier kernels of the stream wrote -- except, when the caller vouches for it
  // (FXPR_GEMM_WEIGHTS_STATIC), the weights: the producer warp then requests the weight boxes of
  // its first stages BEFORE it waits, so their HBM latency (~2.7 us cold) passes while the
  // previous kernel finishes.
  if (warp != 0) pdl_wait();

  const int tiles_n = p.tiles_n;                         // 128-column tiles; one row tile (M <= 64)
  const int items = tiles_n * p.split_k;
  // item = tile * split_k + split.  Persistent: CTA b takes items b, b + grid, ...  Cluster:
  // CTA (x, y) takes the single item (tile y, split x).
  const int first_item = CLUSTER ? (int)(blockIdx.y * p.split_k + blockIdx.x) : (int)blockIdx.x;
  const int item_step = CLUSTER ? items : (int)gridDim.x;
  const int k_tiles_total = (p.K + p.k_tile - 1) / p.k_tile;
  const bool pairs = p.k_tile == 64;                     // two K-tiles per super-stage
  const int ngroup = pairs ? 4 : 8;
  const uint32_t group_cols = pairs ? 2u * MP : (uint32_t)MP;

  if (warp == 0) {
    // ------------------------------ TMA producer --------------------------------
    const bool wk = p.b_kmajor != 0;                     // weights given as an (N, K) row-major view
    // A stage is free again when the MMAs that read it are done, which is also when their
    // accumulator group is full: the issuer signals both with ONE commit (a tcgen05.commit costs
    // ~260 clocks of the issuing thread), so super-stage j waits for the group barrier of
    // super-stage j - STAGES.
    int stage = 0; int wgrp = 0; uint32_t wphase = 0; int issued = 0;
    // boxes of super-stage ss of an item into shared-memory stage st: weights and/or activations
    auto issue_boxes = [&](int item, int ss, int st, bool arm, bool weights, bool acts) {
      const int n0 = (item / p.split_k) * 128;
      const int ks = item % p.split_k;
      const int n_kt = (k_tiles_total - ks + p.split_k - 1) / p.split_k;
      const int ka = pairs ? (ks + (2 * ss) * p.split_k) * 64 : (ks + ss * p.split_k) * 128;
      const int kb = pairs ? ka + p.split_k * 64 : ka + 64;
      const bool two = pairs ? (2 * ss + 1 < n_kt) : true;
      const uint32_t fb = full0 + 8u * st;
      const uint32_t sw = smem_base + st * kSkSSBytes;
      const uint32_t sx = sw + kSkWBytes;
      if (lane == 0) {
        if (arm) mbar_expect_tx(fb, two ? kSkSSBytes : kSkSSBytes / 2);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (h == 1 && !two) break;
          const int kk = h ? kb : ka;
          if (weights) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
              tma_load_2d(sw + h * (kSkWBytes / 2) + j * 8192, &tma_w, fb, wk ? kk : n0 + j * 64, wk ? n0 + j * 64 : kk);
          }
          if (acts) tma_load_2d(sx + h * (kSkXBytes / 2), &tma_x, fb, kk, 0);
        }
      }
      __syncwarp();
    };
    auto n_ss_of = [&](int item) {
      const int ks = item % p.split_k;
      const int n_kt = (k_tiles_total - ks + p.split_k - 1) / p.split_k;
      return pairs ? (n_kt + 1) >> 1 : n_kt;
    };
    // weights of the first item's first stages, then the dependency wait, then their activations
    int early = 0;
    if (p.w_static && first_item < items) {
      early = min(STAGES, n_ss_of(first_item));
      for (int ss = 0; ss < early; ++ss) issue_boxes(first_item, ss, ss, true, true, false);
    }
    pdl_wait();
    for (int ss = 0; ss < early; ++ss) issue_boxes(first_item, ss, ss, false, false, true);
    for (int item = first_item; item < items; item += item_step) {
      const int n_ss = n_ss_of(item);
      for (int ss = 0; ss < n_ss; ++ss) {
        if (item == first_item && ss < early) {      // already requested above
          ++issued;
          if (++stage == STAGES) stage = 0;
          continue;
        }
        if (issued >= STAGES) {
          if (!__all_sync(0xffffffffu, mbar_wait(tfull0 + 8u * wgrp, wphase, abort_flag))) goto producer_done;
          if (++wgrp == ngroup) { wgrp = 0; wphase ^= 1; }
        }
        ++issued;
        issue_boxes(item, ss, stage, true, true, true);
        if (++stage == STAGES) stage = 0;
      }
    }
  producer_done:;
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ----------------------------------
    // Weights are the 128-row operand: MN-major for a (K, N) row-major matrix, K-major for
    // an (N, K).t() view.  Activations are the K-major 64-row operand.
    const uint64_t wdesc0 = p.b_kmajor ? make_smem_desc(smem_base, 16, 1024) : make_smem_desc(smem_base, 8192, 1024);
    const uint64_t xdesc0 = make_smem_desc(smem_base + kSkWBytes, 16, 1024);
    const uint64_t wks = p.b_kmajor ? 2 : 128;           // (32 B | 2048 B) >> 4 per 16-deep k step
    constexpr uint64_t kStep = kSkSSBytes >> 4;
    constexpr uint64_t kHalfW = (kSkWBytes / 2) >> 4, kHalfX = (kSkXBytes / 2) >> 4;
    const uint32_t idesc = p.idesc;
    int stage = 0; uint32_t phase = 0; int grp = 0; uint32_t gphase = 1;
    for (int item = first_item; item < items; item += item_step) {
      const int ks = item % p.split_k;
      const int n_kt = (k_tiles_total - ks + p.split_k - 1) / p.split_k;
      const int n_ss = pairs ? (n_kt + 1) >> 1 : n_kt;
      for (int ss = 0; ss < n_ss; ++ss) {
        const bool two = pairs ? (2 * ss + 1 < n_kt) : true;
        {
          const bool r1 = mbar_wait(tempty0 + 8u * grp, gphase, abort_flag);
          const bool r2 = mbar_wait(full0 + 8u * stage, phase, abort_flag);
          if (!__all_sync(0xffffffffu, r1 && r2)) goto issuer_done;
        }
        tc_fence_after();
        const uint32_t d0 = tmem_base + (uint32_t)grp * group_cols;
        const uint32_t d1 = pairs ? d0 + MP : d0;
        const uint64_t wd = wdesc0 + (uint64_t)stage * kStep;
        const uint64_t xd = xdesc0 + (uint64_t)stage * kStep;
        if (lane == 0) {
#pragma unroll
          for (int i = 0; i < 4; ++i) umma_f16(d0, wd + i * wks, xd + i * 2, idesc, i ? 1u : 0u);
          if (two) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              umma_f16(d1, wd + kHalfW + i * wks, xd + kHalfX + i * 2, idesc, (i || !pairs) ? 1u : 0u);
          }
          umma_commit(tfull0 + 8u * grp);              // stage consumed AND accumulator group full
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
        if (++grp == ngroup) { grp = 0; gphase ^= 1; }
      }
    }
  issuer_done:;
  } else {
#include "gemm_tc_skinny_epilogue.inl"
  }

  if constexpr (CLUSTER) {
    // ------------------------------ cluster merge ---------------------------------
    // The epilogue warps left this split's integer partials in shared memory ([64 rows][128
    // columns] int64 over the first stages, which no copy or MMA touches any more).  Rank r sums
    // rows [r * 64 / S, (r + 1) * 64 / S) over all ranks and writes the outputs.  Every thread
    // of every CTA reaches both cluster barriers, also after a timed-out wait.
    cg::cluster_group cluster = cg::this_cluster();
    __syncthreads();
    cluster.sync();
    if (warp >= 2 && !*abort_flag) {
      const int S = p.split_k, rank = (int)blockIdx.x;
      const long long* red = reinterpret_cast<const long long*>(smem_gen);
      const int rows_per = (MP + S - 1) / S, mr0 = rank * rows_per;   // any S <= 8; the last rank may get fewer
      const int tile = (int)blockIdx.y;
      const T* bias = (const T*)p.bias;
      // Two neighbouring columns per thread and step: one 16-byte read per rank.  (Reads over
      // distributed shared memory are paced per request, ~100 clocks per warp request whatever
      // its width -- issuing more of them at once made the merge slower -- so wider requests are
      // what shortens it.)
      const long long* peer[8];
      for (int rr = 0; rr < S; ++rr) peer[rr] = cluster.map_shared_rank(red, rr);
      for (int idx = (int)threadIdx.x - 64; idx < rows_per * 64; idx += EPIW * 32) {
        const int m = mr0 + idx / 64, nl = (idx % 64) * 2, n = tile * 128 + nl;
        if (m >= MP || m >= p.M || n >= p.N) continue;
        long long q0 = 0, q1 = 0;
        for (int rr = 0; rr < S; ++rr) {
          const longlong2 v = *reinterpret_cast<const longlong2*>(peer[rr] + m * 128 + nl);
          q0 += v.x;
          q1 += v.y;
        }
        if (p.int_bits != 64) { q0 = (long long)(int32_t)q0; q1 = (long long)(int32_t)q1; }
        const bool two = n + 1 < p.N;
        if (p.silu_mul) {
          // the (gate, up) pair of output column n / 2
          if (!two) continue;
          float g = fixed_to_float<long long>(q0, p.inv_scale), u = fixed_to_float<long long>(q1, p.inv_scale);
          if (bias) { g = __fadd_rn(g, to_f32<T>(bias[n])); u = __fadd_rn(u, to_f32<T>(bias[n + 1])); }
          ((T*)p.c)[(int64_t)m * p.c_sm + (n >> 1)] =
              silu_mul_io<T>(to_f32<T>(from_f32<T>(g)), to_f32<T>(from_f32<T>(u)));
          continue;
        }
        if (p.c_int) {
          if (p.int_bits == 64) {
            ((long long*)p.c_int)[(int64_t)m * p.N + n] = q0;
            if (two) ((long long*)p.c_int)[(int64_t)m * p.N + n + 1] = q1;
          } else {
            ((int32_t*)p.c_int)[(int64_t)m * p.N + n] = (int32_t)q0;
            if (two) ((int32_t*)p.c_int)[(int64_t)m * p.N + n + 1] = (int32_t)q1;
          }
        }
        if (p.c) {
          float v0 = fixed_to_float<long long>(q0, p.inv_scale), v1 = fixed_to_float<long long>(q1, p.inv_scale);
          if (bias) {
            v0 = __fadd_rn(v0, to_f32<T>(bias[n]));
            if (two) v1 = __fadd_rn(v1, to_f32<T>(bias[n + 1]));
          }
          T* dst = (T*)p.c + (int64_t)m * p.c_sm + n;
          dst[0] = from_f32<T>(v0);
          if (two) dst[1] = from_f32<T>(v1);
        }
      }
    }
    cluster.sync();                                  // peers may still be reading this CTA's partials
  }

  // ------------------------------ teardown ----------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // let copies that are still in flight land before shared memory is released
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) { __nanosleep(1000); }
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, FXPR_ERR_TIMEOUT);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// The skinny route takes what the fast route takes (int32 / int64 sums, frac_bits <= 21,
// k_tile 64 or 128, at most 510 K-tiles per item) when all rows fit one 64-row tile.
bool gemm_tc_fast_supported(const GemmArgs& g, int split_k);

bool gemm_tc_skinny_supported(const GemmArgs& g, int split_k) {
  return g.M <= kSkMP && g.partials == nullptr && gemm_tc_fast_supported(g, split_k);
}

template <typename T>
static int launch_skinny_cluster(const CUtensorMap& mw, const CUtensorMap& mx, TcParams& p, cudaStream_t s) {
  constexpr int kSmem = kSkStages * kSkSSBytes + 256 + 1024;
  auto k = gemm_tc_skinny_kernel<T, true>;
  static bool attr_done_dev[64] = {};            // function attributes are per device
  int dev_id = 0;
  cudaGetDevice(&dev_id);
  bool& attr_done = attr_done_dev[dev_id & 63];
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) { set_last_error("gemm_tc_skinny smem attribute", e); return FXPR_ERR_CUDA; }
    attr_done = true;
  }
  p.tiles_m = 1;
  p.tiles_n = (p.N + 127) / 128;
  cudaError_t e = launch_pdl(k, dim3((unsigned)p.split_k, (unsigned)p.tiles_n, 1), dim3(kSkWarps * 32), kSmem, s,
                             (unsigned)p.split_k, mw, mx, p, 0);
  if (e != cudaSuccess) { set_last_error("gemm_tc_skinny cluster launch", e); return FXPR_ERR_CUDA; }
  return check_launch("gemm_tc_skinny");
}

template <typename T>
static int launch_skinny(const CUtensorMap& mw, const CUtensorMap& mx, TcParams& p, int sms, cudaStream_t s) {
  constexpr int kSmem = kSkStages * kSkSSBytes + 256 + 1024;
  auto k = gemm_tc_skinny_kernel<T, false>;
  static bool attr_done_dev[64] = {};            // function attributes are per device
  int dev_id = 0;
  cudaGetDevice(&dev_id);
  bool& attr_done = attr_done_dev[dev_id & 63];
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) { set_last_error("gemm_tc_skinny smem attribute", e); return FXPR_ERR_CUDA; }
    attr_done = true;
  }
  p.tiles_m = 1;
  p.tiles_n = (p.N + 127) / 128;
  const int64_t items = (int64_t)p.tiles_n * p.split_k;
  const int grid = (int)(items < sms ? items : sms);
  cudaError_t e = launch_pdl(k, dim3((unsigned)grid), dim3(kSkWarps * 32), kSmem, s, 1u, mw, mx, p, 0);
  if (e != cudaSuccess) { set_last_error("gemm_tc_skinny launch", e); return FXPR_ERR_CUDA; }
  return check_launch("gemm_tc_skinny");
}

// mw: the weight tensor map of gemm_tc() (64-row boxes in either layout).
int gemm_tc_skinny(const GemmArgs& g, TcParams& p, const CUtensorMap& mw, cudaStream_t s) {
  const int sms = tc_device_sms();
  if (sms < 0) return FXPR_ERR_ARCH;
  CUtensorMap mx;
  if (!tc_make_map(&mx, g.dtype, g.a, g.M, g.K, g.a_sm, kSkMP)) {
    set_last_error("cuTensorMapEncodeTiled(X)", cudaErrorInvalidValue);
    return FXPR_ERR_CUDA;
  }
  // M = 128 weight columns, N = 64 activation rows; bit 15: the 128-row operand is MN-major
  p.idesc = make_idesc(g.dtype == FXPR_BF16 ? 1 : 0, 0, kSkMP, 128) | (p.b_kmajor ? 0u : (1u << 15));
  // 2 to 8 splits run as a thread-block cluster (merge through distributed shared memory);
  // larger split counts use the partial planes in the caller's scratch.  Same bits either way.
  const bool cluster = p.split_k >= 2 && p.split_k <= 8 && (p.N + 127) / 128 <= 65535 &&
                       !(g.flags & FXPR_GEMM_NO_CLUSTER);
  if (cluster) {
    if (g.dtype == FXPR_BF16) return launch_skinny_cluster<__nv_bfloat16>(mw, mx, p, s);
    return launch_skinny_cluster<__half>(mw, mx, p, s);
  }
  if (g.dtype == FXPR_BF16) return launch_skinny<__nv_bfloat16>(mw, mx, p, sms, s);
  return launch_skinny<__half>(mw, mx, p, sms, s);
}

}  // namespace fxpr

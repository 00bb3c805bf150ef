// Fixed-point GEMM on the 5th-generation tensor cores (sm_100a): TMA-fed
// tcgen05.mma with fp32 accumulators in tensor memory, one FRESH accumulator per
// K-tile, read back by the epilogue warps (tcgen05.ld), rounded to Q-format and
// summed as integers in registers.  Semantics: fxpr_vllm/_triton/gemm.py:183-204
// (persistent kernel) and :273-325 (split-K with integer atomics and a
// last-arriver epilogue) of the reference.
//
// CTA = 10 warps, one CTA per SM, persistent over (output tile, k-split) items:
//   warp 0      TMA producer: A [128 x 64] and B [64 x BN] bf16/fp16 tiles, 128-byte
//               swizzle, STAGES-deep mbarrier ring
//   warp 1      MMA issuer: per K-tile k_tile/16 tcgen05.mma (M=128, N=BN, K=16) into
//               one of two TMEM accumulator buffers, tcgen05.commit to free smem
//               stages and to publish the finished K-tile
//   warps 2..9  epilogue: warp w reads TMEM lanes 32*(w%4).. (a row per thread) and
//               half of the BN columns; converts and accumulates while the MMA warp
//               works on the next K-tile in the other TMEM buffer
// Because every K-tile is quantised before it is added, the integer sum does not
// depend on tile order, split-K, grid size or which CTA ran what.
//
// Every wait is bounded: after ~2 s a waiter raises an abort flag, writes the status
// word, lets in-flight copies land, frees TMEM and returns.
#include <cuda.h>

#include <type_traits>

#include "fxp_common.cuh"
#include "gemm_common.cuh"
#include "tc_common.cuh"

namespace fxpr {

// ---------------------------------------------------------------------------------
// kernel
// ---------------------------------------------------------------------------------
template <typename T, int BN, bool ACC64, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               const TcParams p) {
  using L = SmemLayout<BN, STAGES>;
  using AccT = typename std::conditional<ACC64, long long, int32_t>::type;
  constexpr int kColsPerThread = BN / 2;      // two epilogue warps share a lane quarter
  constexpr int kTmemCols = 2 * BN;            // two accumulator buffers (power of two >= 32)

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // SW128 tiles need 1 KB alignment
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem_gen + L::kBarOffset + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = (volatile int*)(smem_gen + L::kBarOffset + 8 * (2 * STAGES + 4) + 8);
  const uint32_t epi_bar = bar_base + 8u * (2 * STAGES + 4) + 16u;   // epilogue-warps-only barrier
  volatile int* s_last = (volatile int*)(smem_gen + L::kBarOffset + 8 * (2 * STAGES + 4) + 24);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), kEpiWarps); }
    mbar_init(epi_bar, kEpiWarps);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32((const void*)tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_mn = p.tiles_m * p.tiles_n;
  const int items = tiles_mn * p.split_k;
  const int k_tiles_total = (p.K + p.k_tile - 1) / p.k_tile;
  const int chunks = p.k_tile / kBK;

  auto tile_coords = [&](int tile, int& pm, int& pn) {
    const int in_group = kGroupM * p.tiles_n;
    const int g = tile / in_group;
    const int first = g * kGroupM;
    const int gsz = min(p.tiles_m - first, kGroupM);
    pm = first + (tile % in_group) % gsz;
    pn = (tile % in_group) / gsz;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer --------------------------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        int pm, pn; tile_coords(item / p.split_k, pm, pn);
        const int ks = item % p.split_k;
        for (int kt = ks; kt < k_tiles_total && ok; kt += p.split_k) {
          for (int ch = 0; ch < chunks; ++ch) {
            if (!mbar_wait(empty_bar(stage), phase ^ 1, abort_flag)) { ok = false; break; }
            const uint32_t sa = smem_base + stage * L::kStageBytes;
            const uint32_t sb = sa + L::kABytes;
            const int k0 = kt * p.k_tile + ch * kBK;
            mbar_expect_tx(full_bar(stage), L::kStageBytes);
            tma_load_2d(sa, &tma_a, full_bar(stage), k0, pm * kBM);
            if (p.b_kmajor) {
              // B stored (N, K): rows = n, 64 k contiguous; boxes of 64 rows keep the
              // tensor-map box <= 256 and the layout identical to A's
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * (64 * kBK * 2), &tma_b, full_bar(stage), k0, pn * BN + j * 64);
            } else {
              // B stored (K, N): boxes of 64 n (128 B) x 64 k rows
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + j * (64 * kBK * 2), &tma_b, full_bar(stage), pn * BN + j * 64, k0);
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ----------------------------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; int buf = 0; uint32_t tphase[2] = {0, 0}; bool ok = true;
      // A: K-major, 8-row groups 1024 B apart, +32 B per 16-wide k step.  B K-major: same.
      // B N-major: 64-column slabs 8192 B apart (leading offset), 8-k-row groups 1024 B
      // apart, +2048 B per 16-deep k step.
      const uint64_t adesc0 = make_smem_desc(smem_base, 16, 1024);
      const uint64_t bdesc0 = p.b_kmajor ? make_smem_desc(smem_base + L::kABytes, 16, 1024)
                                         : make_smem_desc(smem_base + L::kABytes, 8192, 1024);
      const uint64_t b_kstep = p.b_kmajor ? 2 : 128;
      constexpr uint64_t kStageStep = L::kStageBytes >> 4;
      const uint32_t idesc = p.idesc;
      for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int ks = item % p.split_k;
        for (int kt = ks; kt < k_tiles_total && ok; kt += p.split_k) {
          if (!mbar_wait(tempty_bar(buf), tphase[buf] ^ 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
          for (int ch = 0; ch < chunks; ++ch) {
            if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            // descriptors differ from stage 0 / k 0 only in the 14-bit address field
            const uint64_t ad = adesc0 + (uint64_t)stage * kStageStep;
            const uint64_t bd = bdesc0 + (uint64_t)stage * kStageStep;
            umma_f16(d_tmem, ad, bd, idesc, ch ? 1u : 0u);
            umma_f16(d_tmem, ad + 2, bd + b_kstep, idesc, 1u);
            umma_f16(d_tmem, ad + 4, bd + 2 * b_kstep, idesc, 1u);
            umma_f16(d_tmem, ad + 6, bd + 3 * b_kstep, idesc, 1u);
            umma_commit(empty_bar(stage));   // frees the smem stage when these MMAs finish
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (!ok) break;
          umma_commit(tfull_bar(buf));       // K-tile accumulator complete
          tphase[buf] ^= 1; buf ^= 1;
        }
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------------
    const int ew = warp - 2;
    const int quarter = warp & 3;              // TMEM lane quarter this warp may touch
    const int half = ew >> 2;                  // which half of the BN columns
    const int row_in_tile = quarter * 32 + lane;
    const int col0 = half * kColsPerThread;
    int buf = 0; uint32_t tphase[2] = {0, 0}; bool ok = true;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    uint32_t epi_phase = 0;
    // barrier over the 8 epilogue warps with a bounded wait (a plain bar.sync could
    // hang if one warp had given up on an earlier wait)
    auto epi_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(epi_bar);
      const bool done = mbar_wait(epi_bar, epi_phase, abort_flag);
      epi_phase ^= 1;
      return done;
    };

    for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const int tile = item / p.split_k, ks = item % p.split_k;
      int pm, pn; tile_coords(tile, pm, pn);
      const int row = pm * kBM + row_in_tile;
      const int ncol0 = pn * BN + col0;
      AccT acc[kColsPerThread];
#pragma unroll
      for (int i = 0; i < kColsPerThread; ++i) acc[i] = 0;

      for (int kt = ks; kt < k_tiles_total && ok; kt += p.split_k) {
        if (!mbar_wait(tfull_bar(buf), tphase[buf], abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t t_addr = tmem_base + lane_addr + (uint32_t)(buf * BN + col0);
#pragma unroll
        for (int c = 0; c < kColsPerThread / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(t_addr + c * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float f = __uint_as_float(v[i]);
            if constexpr (ACC64) {
              acc[c * 32 + i] += float_to_fixed<64>(f, p.scale);
            } else {
              acc[c * 32 + i] += (p.int_bits == 16) ? (int32_t)float_to_fixed<16>(f, p.scale)
                                                    : float_to_fixed<32>(f, p.scale);
            }
          }
          if (p.partials && row < p.M) {
            float* dst = p.partials + ((int64_t)kt * p.M + row) * p.N + ncol0 + c * 32;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (ncol0 + c * 32 + i < p.N) dst[i] = __uint_as_float(v[i]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(buf));
        tphase[buf] ^= 1; buf ^= 1;
      }
      if (!ok) break;

      // ---- tile epilogue ----
      const bool row_ok = row < p.M;
      if (p.split_k > 1) {
        // Every split leaves its integer partial tile in its own plane of the scratch,
        // column-major inside the tile (a warp's 32 rows are 32 consecutive words); the
        // split that arrives last adds the other planes to its registers.  Integer sums
        // do not depend on which split that is.
        const int64_t plane_elems = (int64_t)kBM * BN;
        const int64_t plane_stride = (int64_t)p.tiles_m * p.tiles_n * plane_elems;
        AccT* planes = (AccT*)p.acc_scratch + (int64_t)tile * plane_elems + (int64_t)col0 * kBM + row_in_tile;
        {
          AccT* dst = planes + ks * plane_stride;
#pragma unroll
          for (int i = 0; i < kColsPerThread; ++i) __stcg(dst + i * kBM, acc[i]);
        }
        __threadfence();
        // all 8 epilogue warps must have stored before the tile counts as arrived
        if (!epi_sync()) { ok = false; break; }
        if (threadIdx.x == 64) *s_last = (atomicAdd(p.locks + tile, 1) == p.split_k - 1) ? 1 : 0;
        if (!epi_sync()) { ok = false; break; }
        const bool last = *s_last != 0;
        if (last) {
          __threadfence();
          if (row_ok) {
            for (int s2 = 0; s2 < p.split_k; ++s2) {
              if (s2 == ks) continue;
              const AccT* src = planes + s2 * plane_stride;
#pragma unroll
              for (int i = 0; i < kColsPerThread; ++i) acc[i] += __ldcg(src + i * kBM);
            }
          }
          if (threadIdx.x == 64) p.locks[tile] = 0;
        }
        if (!epi_sync()) { ok = false; break; }   // s_last may be rewritten only after everyone read it
        if (!last) continue;
      }
      if (!row_ok) continue;

      if (p.c_int) {
        if (p.int_bits == 64) {
          long long* dst = (long long*)p.c_int + (int64_t)row * p.N + ncol0;
#pragma unroll
          for (int i = 0; i < kColsPerThread; ++i) if (ncol0 + i < p.N) dst[i] = (long long)acc[i];
        } else if (p.int_bits == 32) {
          int32_t* dst = (int32_t*)p.c_int + (int64_t)row * p.N + ncol0;
#pragma unroll
          for (int i = 0; i < kColsPerThread; ++i) if (ncol0 + i < p.N) dst[i] = (int32_t)acc[i];
        } else {
          int16_t* dst = (int16_t*)p.c_int + (int64_t)row * p.N + ncol0;
#pragma unroll
          for (int i = 0; i < kColsPerThread; ++i) if (ncol0 + i < p.N) dst[i] = (int16_t)acc[i];
        }
      }
      if (p.c) {
        T* dst = (T*)p.c + (int64_t)row * p.c_sm + ncol0;
        const T* bias = (const T*)p.bias;
#pragma unroll
        for (int g = 0; g < kColsPerThread / 8; ++g) {
          alignas(16) T out[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int col = ncol0 + g * 8 + i;
            long long q = (long long)acc[g * 8 + i];
            if (!ACC64 && p.int_bits == 16) q = (long long)(int16_t)q;
            float v = fixed_to_float<long long>(q, p.inv_scale);
            if (bias && col < p.N) v = __fadd_rn(v, to_f32<T>(bias[col]));
            out[i] = from_f32<T>(v);
          }
          const int colg = ncol0 + g * 8;
          if (p.c_vec_ok && colg + 8 <= p.N) {
            *reinterpret_cast<uint4*>(dst + g * 8) = *reinterpret_cast<const uint4*>(out);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) if (colg + i < p.N) dst[g * 8 + i] = out[i];
          }
        }
      }
    }
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
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)ptr;
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] (cols contiguous), box [box_rows, 64 cols], 128 B swizzle.
bool tc_make_map(CUtensorMap* m, int dtype, const void* base, int64_t rows, int64_t cols,
                     int64_t row_stride_elems, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_stride_elems * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, dtype == FXPR_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                  2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

int tc_device_sms() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!cached[dev]) {
    int n = 0, major = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cached[dev] = (major == 10 && n > 0) ? n : -1;
  }
  return cached[dev];
}

bool gemm_tc_supported(const GemmArgs& g) {
  if (g.dtype != FXPR_F16 && g.dtype != FXPR_BF16) return false;
  if (g.K < 1 || g.k_tile < 64 || g.k_tile % 64 != 0) return false;
  if (g.a_sk != 1 || (g.a_sm % 8) != 0 || ((uintptr_t)g.a & 15)) return false;
  const bool b_nmajor = (g.b_sn == 1) && (g.b_sk % 8 == 0) && g.b_sk >= g.N;
  const bool b_kmajor = (g.b_sk == 1) && (g.b_sn % 8 == 0) && g.b_sn >= g.K;
  if (!(b_nmajor || b_kmajor) || ((uintptr_t)g.b & 15)) return false;
  // very small problems stay on the CUDA-core kernel; the rule looks at N and K only
  if (g.N < 64 || g.K < 64) return false;
  return true;
}

// Split-K scratch: [tile counters | split_k planes of integer partial tiles].  The counter
// region has one fixed size so that a buffer reused for problems of different shapes never
// shows plane contents as counters; only the counters must be zero before the first use,
// and every launch leaves them zero.  Problems with more tiles than counters run unsplit
// (they fill the GPU many times over; the result is the same bits).
static constexpr int64_t kLockBytes = 256 * 1024;
static constexpr int64_t kMaxSplitTiles = kLockBytes / 4;
static int64_t tc_lock_bytes(int64_t, int64_t) { return kLockBytes; }

int64_t gemm_tc_scratch_bytes(int64_t M, int64_t N, int int_bits, int split_k) {
  const int64_t rows = ((M + 255) / 256) * 256;       // the two-SM kernel works on 256-row pair tiles
  const int64_t cols = ((N + 255) / 256) * 256;
  const int64_t planes = (int64_t)(split_k < 1 ? 1 : split_k) * rows * cols * (int_bits == 64 ? 8 : 4);
  return tc_lock_bytes(M, N) + ((planes + 255) / 256) * 256;
}

template <typename T, int BN, bool ACC64, int STAGES>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, TcParams& p, int sms, cudaStream_t s) {
  using L = SmemLayout<BN, STAGES>;
  auto k = gemm_tc_kernel<T, BN, ACC64, STAGES>;
  static bool attr_done_dev[64] = {};            // function attributes are per device
  int dev_id = 0;
  cudaGetDevice(&dev_id);
  bool& attr_done = attr_done_dev[dev_id & 63];
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) { set_last_error("gemm_tc smem attribute", e); return FXPR_ERR_CUDA; }
    attr_done = true;
  }
  p.tiles_m = (p.M + kBM - 1) / kBM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int64_t items = (int64_t)p.tiles_m * p.tiles_n * p.split_k;
  const int grid = (int)(items < sms ? items : sms);
  k<<<grid, kThreads, L::kTotal, s>>>(ma, mb, p);
  return check_launch("gemm_tc");
}

bool gemm_tc_fast_supported(const GemmArgs& g, int split_k);
bool gemm_tc_skinny_supported(const GemmArgs& g, int split_k);
bool gemm_tc_n256_supported(const GemmArgs& g, int split_k);
int gemm_tc_n256(const GemmArgs& g, TcParams& p, const CUtensorMap& ma, const CUtensorMap& mb, cudaStream_t s);
int gemm_tc_skinny(const GemmArgs& g, TcParams& p, const CUtensorMap& mw, cudaStream_t s);
int gemm_tc_fast(const GemmArgs& g, TcParams& p, const CUtensorMap& ma, const CUtensorMap& mb,
                 cudaStream_t s);
bool gemm_tc_pair_supported(const GemmArgs& g, int split_k);
int gemm_tc_pair(const GemmArgs& g, TcParams& p, const CUtensorMap& ma, const CUtensorMap& mb,
                 int bn, cudaStream_t s);

int gemm_tc(const GemmArgs& g, cudaStream_t s) {
  const int sms = tc_device_sms();
  if (sms < 0) return FXPR_ERR_ARCH;
  const bool b_kmajor = !((g.b_sn == 1) && (g.b_sk % 8 == 0));
  const bool acc64 = g.int_bits == 64;
  const int BN = acc64 ? 128 : 256;

  CUtensorMap ma, mb;
  if (!tc_make_map(&ma, g.dtype, g.a, g.M, g.K, g.a_sm, kBM)) {
    set_last_error("cuTensorMapEncodeTiled(A)", cudaErrorInvalidValue);
    return FXPR_ERR_CUDA;
  }
  const bool okb = b_kmajor ? tc_make_map(&mb, g.dtype, g.b, g.N, g.K, g.b_sn, 64)
                            : tc_make_map(&mb, g.dtype, g.b, g.K, g.N, g.b_sk, 64);
  if (!okb) {
    set_last_error("cuTensorMapEncodeTiled(B)", cudaErrorInvalidValue);
    return FXPR_ERR_CUDA;
  }

  TcParams p;
  p.bias = g.bias; p.c = g.c; p.c_int = g.c_int; p.partials = g.partials;
  p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K; p.c_sm = g.c_sm;
  p.k_tile = g.k_tile; p.int_bits = g.int_bits;
  p.scale = (float)(1ull << g.frac_bits); p.inv_scale = 1.0f / p.scale;
  p.b_kmajor = b_kmajor ? 1 : 0;
  p.idesc = make_idesc(g.dtype == FXPR_BF16 ? 1 : 0, b_kmajor ? 0 : 1, BN, kBM);
  p.c_vec_ok = (g.c && (((uintptr_t)g.c & 15) == 0) && (g.c_sm % 8 == 0)) ? 1 : 0;
  p.status = g.status;
  p.silu_mul = 0;
  p.best = nullptr; p.n_offset = 0;
  p.w_static = (g.flags & FXPR_GEMM_WEIGHTS_STATIC) ? 1 : 0;
  const int k_tiles = (int)((g.K + g.k_tile - 1) / g.k_tile);
  p.split_k = g.split_k < 1 ? 1 : (g.split_k > k_tiles ? k_tiles : g.split_k);
  p.acc_scratch = nullptr; p.locks = nullptr;
  if (((g.M + kBM - 1) / kBM) * ((g.N + 127) / 128) > kMaxSplitTiles) p.split_k = 1;
  if (p.split_k > 1) {
    const int64_t need = gemm_tc_scratch_bytes(g.M, g.N, g.int_bits, p.split_k);
    if (!g.scratch || g.scratch_bytes < need) return FXPR_ERR_SCRATCH;
    if ((uintptr_t)g.scratch & 15) return FXPR_ERR_BAD_ARG;
    p.locks = (int32_t*)g.scratch;
    p.acc_scratch = (char*)g.scratch + tc_lock_bytes(g.M, g.N);
  }

  // decode shapes: weights on the 128-row side of the MMA (same bits, see gemm_tc_skinny.cu)
  if (!(g.flags & (FXPR_GEMM_FORCE_EXACT_TC | FXPR_GEMM_NO_SKINNY)) && gemm_tc_skinny_supported(g, p.split_k)) {
    p.silu_mul = (g.flags & FXPR_GEMM_SILU_MUL) ? 1 : 0;
    if (g.best) {
      if (p.split_k != 1 || p.silu_mul) return FXPR_ERR_UNSUPPORTED;
      p.best = g.best; p.n_offset = (unsigned int)g.n_offset;
    }
    return gemm_tc_skinny(g, p, mb, s);
  }
  if (g.best) return FXPR_ERR_UNSUPPORTED;                          // only the decode-shape kernel
  if (g.flags & FXPR_GEMM_SILU_MUL) return FXPR_ERR_UNSUPPORTED;   // only the decode-shape kernel fuses it
  // 128 x 256 tiles: measured +6 % at k_tile 128 (two 64-deep stages per accumulator) and -12 %
  // at k_tile 64 (one MMA group per hand-off with only two accumulators in TMEM), same bits;
  // so they are the default for k_tile 128 only.  The flags force either shape.
  if ((g.flags & FXPR_GEMM_PAIR) && !(g.flags & FXPR_GEMM_FORCE_EXACT_TC) && gemm_tc_pair_supported(g, p.split_k)) {
    int bn = (g.N >= 256) ? 256 : 128;
    if (g.flags & FXPR_GEMM_TILE_N128) bn = 128;
    return gemm_tc_pair(g, p, ma, mb, bn, s);
  }
  const bool want_n256 = (g.flags & FXPR_GEMM_TILE_N256) || (g.k_tile == 128 && !(g.flags & FXPR_GEMM_TILE_N128));
  if (want_n256 && !(g.flags & FXPR_GEMM_FORCE_EXACT_TC) && gemm_tc_n256_supported(g, p.split_k))
    return gemm_tc_n256(g, p, ma, mb, s);
  if (!(g.flags & FXPR_GEMM_FORCE_EXACT_TC) && gemm_tc_fast_supported(g, p.split_k)) {
    return gemm_tc_fast(g, p, ma, mb, s);
  }

  if (g.dtype == FXPR_BF16) {
    return acc64 ? launch_tc<__nv_bfloat16, 128, true, 6>(ma, mb, p, sms, s)
                 : launch_tc<__nv_bfloat16, 256, false, 4>(ma, mb, p, sms, s);
  }
  return acc64 ? launch_tc<__half, 128, true, 6>(ma, mb, p, sms, s)
               : launch_tc<__half, 256, false, 4>(ma, mb, p, sms, s);
}

}  // namespace fxpr

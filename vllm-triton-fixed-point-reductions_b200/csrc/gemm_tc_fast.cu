// Fast route of the tensor-core fixed-point GEMM (sm_100a): same TMA / tcgen05.mma
// main loop as gemm_tc.cu, but an epilogue built for the real bottleneck -- one
// fp32 partial has to be rounded to Q-format and integer-added for every 2*k_tile
// flops, i.e. ~64 elements per clock per SM at k_tile = 64.
//
//   * rounding runs on the FP32 pipe: r = fma(p, 2^f, 1.5*2^23) has rint-half-even of
//     p*2^f in its mantissa whenever |p*2^f| < 2^22, so float_as_int(r) = MAGIC + q.
//     The raw bit patterns are summed in int32 and MAGIC * (#tiles) is subtracted once.
//   * a one-instruction-per-two-partials screen (OR of the raw fp32 bits, test bit 30,
//     i.e. "some |p| >= 2") sends a K-tile to an exact fix-up that uses the reference's
//     cvt.rni conversion (fxpr_vllm/_triton/fxp.py:92-108) for every out-of-range
//     partial, so results equal the plain conversion for every input.
//   * int64 semantics with 32-bit registers: in-range addends are < 2^22, so up to 510
//     K-tiles cannot overflow int32; out-of-range addends go to per-thread side arrays
//     in local memory that are touched only on that rare path.
//
// Tile 128 x 128, one persistent CTA per SM.  Warp 0 = TMA producer, warp 1 = MMA issuer,
// then 16 epilogue warps (TMEM lane quarter x 32-column group).  The single-lane roles are
// latency-bound: an mbarrier probe, a tcgen05 fence, an MMA issue and a commit each take
// 50-100 cycles of the issuing thread, so the pipeline hands over 128 of K at a time
// ("super-stage": for k_tile 64 a pair of K-tiles into two TMEM buffers, each with a fresh
// accumulator; for k_tile 128 one K-tile): one full/empty and one tensor-full/empty
// hand-off per 8 MMAs.  Every index (stage, TMEM group, barrier phase) is a function of the
// running super-stage number, so the roles need no communication beyond the barriers.
//
// Measured with clock64 stamps of CTA 0 at 4096^3, k_tile 64:
// a super-stage takes ~1700 cycles against 512 cycles of tensor work; the issuer spends
// ~1250 of them between "operands landed" and "committed" (MMA issue is paced at 65-80
// cycles per MMA when nothing else runs and ~125 when the 16 epilogue warps convert), the
// rest waiting for the epilogue to hand the TMEM group back.  Tried and measured slower or
// equal: two issuer warps (one per TMEM group; correct, -10 %), four single-buffer groups
// for k_tile 128 (equal), software-pipelined or pairwise TMEM loads in the epilogue
// (-6 % / -11 %), no TMA copies at all (equal: shared-memory bandwidth is not the limit).
// Split-K: per-split integer partial planes, summed by the last arriver.  All waits bounded.
#include <cuda.h>

#include "fxp_common.cuh"
#include "gemm_common.cuh"
#include "tc_common.cuh"
#include "gemm_tc_fast_common.cuh"

namespace fxpr {

static constexpr int kRoleWarps = 2;     // warp 0: TMA producer, warp 1: MMA issuer
static constexpr int kSSBytesA = 2 * kBM * kBK * 2;      // two 64-deep halves of A

// A "super-stage" is 128 deep in K: for k_tile = 128 it is one K-tile (one TMEM buffer),
// for k_tile = 64 it is a PAIR of K-tiles whose accumulators go to the two buffers of a
// TMEM group.  One full/empty hand-off and one tfull/tempty hand-off per super-stage.
template <typename T, int BN, int EPIW, bool DUMP>
__global__ void __launch_bounds__((kRoleWarps + EPIW) * 32, 1)
gemm_tc_fast_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const TcParams p, const int zero /* always 0: keeps the side arrays in local memory */) {
  constexpr int STAGES = 3;                            // super-stages in flight
  constexpr int kSSBytesB = 2 * BN * kBK * 2;
  constexpr int kSSBytes = kSSBytesA + kSSBytesB;      // 64 KB at BN = 128
  constexpr int kBarOffset = STAGES * kSSBytes;
  constexpr int NGROUP = 2;                            // TMEM groups of two BN-column buffers
  constexpr int kCols = BN / (EPIW / 4);               // columns per epilogue thread
  static_assert(BN == 128, "two groups of two buffers need 4 * BN <= 512 TMEM columns");

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kBarOffset;
  const uint32_t full0 = bar_base, empty0 = bar_base + 8u * STAGES;
  const uint32_t tfull0 = bar_base + 8u * (2 * STAGES), tempty0 = tfull0 + 8u * NGROUP;
  constexpr int kMisc = 8 * (2 * STAGES + 2 * NGROUP);
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem_gen + kBarOffset + kMisc);
  volatile int* abort_flag = (volatile int*)(smem_gen + kBarOffset + kMisc + 8);
  const uint32_t epi_bar = bar_base + kMisc + 16u;
  volatile int* s_last = (volatile int*)(smem_gen + kBarOffset + kMisc + 24);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8u * s, 1); mbar_init(empty0 + 8u * s, 1); }
    for (int b = 0; b < NGROUP; ++b) { mbar_init(tfull0 + 8u * b, 1); mbar_init(tempty0 + 8u * b, EPIW); }
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

  const int tiles_mn = p.tiles_m * p.tiles_n;
  const int items = tiles_mn * p.split_k;
  const int k_tiles_total = (p.K + p.k_tile - 1) / p.k_tile;
  const bool pairs = p.k_tile == 64;                   // two K-tiles per super-stage

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
    // All 32 lanes run the loop (uniform control flow lets the compiler keep addresses
    // and descriptors in uniform registers); lane 0 alone issues the copies.
    {
      const bool bk = p.b_kmajor != 0;
      int stage = 0; uint32_t phase = 1;               // "empty" waits start one phase ahead
      int gss = 0;
      for (int item = blockIdx.x; item < items; item += gridDim.x) {
        int pm, pn; tile_coords(item / p.split_k, pm, pn);
        const int m0 = pm * kBM, n0 = pn * BN;
        const int ks = item % p.split_k;
        const int n_kt = (k_tiles_total - ks + p.split_k - 1) / p.split_k;
        const int n_ss = pairs ? (n_kt + 1) >> 1 : n_kt;
        for (int ss = 0; ss < n_ss; ++ss) {
          // K offsets of the two 64-deep halves: consecutive for k_tile = 128, the two
          // K-tiles of the pair (split_k apart) for k_tile = 64
          const int ka = pairs ? (ks + (2 * ss) * p.split_k) * 64 : (ks + ss * p.split_k) * 128;
          const int kb = pairs ? ka + p.split_k * 64 : ka + 64;
          const bool two = pairs ? (2 * ss + 1 < n_kt) : true;
          if (!__all_sync(0xffffffffu, mbar_wait(empty0 + 8u * stage, phase, abort_flag))) goto producer_done;
          const uint32_t fb = full0 + 8u * stage;
          const uint32_t sa = smem_base + stage * kSSBytes;
          const uint32_t sb = sa + kSSBytesA;
          if (lane == 0) {
            mbar_expect_tx(fb, two ? kSSBytes : kSSBytes / 2);
            tma_load_2d(sa, &tma_a, fb, ka, m0);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, &tma_b, fb, bk ? ka : n0 + j * 64, bk ? n0 + j * 64 : ka);
            if (two) {
              tma_load_2d(sa + kSSBytesA / 2, &tma_a, fb, kb, m0);
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                tma_load_2d(sb + kSSBytesB / 2 + j * 8192, &tma_b, fb, bk ? kb : n0 + j * 64, bk ? n0 + j * 64 : kb);
            }
          }
          __syncwarp();
          ++gss;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    producer_done:;
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ----------------------------------
    // One lane feeds the tensor core and its loop is latency-bound (each mbarrier probe,
    // fence, MMA issue and commit costs 50-100 cycles), so it does as little as possible
    // per 8 MMAs: two waits, one fence, two commits.  Descriptors are built once; only
    // their 14-bit address field (bytes >> 4) advances.  All lanes run the loop (uniform
    // control flow, operands in uniform registers); lane 0 issues.
    {
      const uint64_t adesc0 = make_smem_desc(smem_base, 16, 1024);
      const uint64_t bdesc0 = p.b_kmajor ? make_smem_desc(smem_base + kSSBytesA, 16, 1024)
                                         : make_smem_desc(smem_base + kSSBytesA, 8192, 1024);
      const uint64_t bks = p.b_kmajor ? 2 : 128;        // (32 B | 2048 B) >> 4 per 16-deep k step
      constexpr uint64_t kStep = kSSBytes >> 4;
      constexpr uint64_t kHalfA = (kSSBytesA / 2) >> 4, kHalfB = (kSSBytesB / 2) >> 4;
      const uint32_t idesc = p.idesc;
      int stage = 0; uint32_t phase = 0; int grp = 0; uint32_t gphase = 1;
      int gss = 0;
      for (int item = blockIdx.x; item < items; item += gridDim.x) {
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
          const uint32_t d0 = tmem_base + (uint32_t)(grp * 2 * BN);
          const uint32_t d1 = pairs ? d0 + BN : d0;       // second half: other buffer, or accumulate on
          const uint64_t ad = adesc0 + (uint64_t)stage * kStep;
          const uint64_t bd = bdesc0 + (uint64_t)stage * kStep;
          if (lane == 0) {
          umma_f16(d0, ad, bd, idesc, 0u);
          umma_f16(d0, ad + 2, bd + bks, idesc, 1u);
          umma_f16(d0, ad + 4, bd + 2 * bks, idesc, 1u);
          umma_f16(d0, ad + 6, bd + 3 * bks, idesc, 1u);
          if (two) {
            umma_f16(d1, ad + kHalfA, bd + kHalfB, idesc, pairs ? 0u : 1u);
            umma_f16(d1, ad + kHalfA + 2, bd + kHalfB + bks, idesc, 1u);
            umma_f16(d1, ad + kHalfA + 4, bd + kHalfB + 2 * bks, idesc, 1u);
            umma_f16(d1, ad + kHalfA + 6, bd + kHalfB + 3 * bks, idesc, 1u);
          }
          umma_commit(empty0 + 8u * stage);            // frees the super-stage when these finish
          umma_commit(tfull0 + 8u * grp);              // accumulator(s) of this super-stage complete
          }
          __syncwarp();
          ++gss;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          grp ^= 1; if (grp == 0) gphase ^= 1;
        }
      }
    issuer_done:;
    }
  } else {
#include "gemm_tc_fast_epilogue.inl"
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

template <typename T, int BN, int EPIW, bool DUMP>
static int launch_fast(const CUtensorMap& ma, const CUtensorMap& mb, TcParams& p, int sms, cudaStream_t s) {
  constexpr int kSmem = 3 * (kSSBytesA + 2 * BN * kBK * 2) + 256 + 1024;
  auto k = gemm_tc_fast_kernel<T, BN, EPIW, DUMP>;
  static bool attr_done_dev[64] = {};            // function attributes are per device
  int dev_id = 0;
  cudaGetDevice(&dev_id);
  bool& attr_done = attr_done_dev[dev_id & 63];
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) { set_last_error("gemm_tc_fast smem attribute", e); return FXPR_ERR_CUDA; }
    attr_done = true;
  }
  p.tiles_m = (p.M + kBM - 1) / kBM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int64_t items = (int64_t)p.tiles_m * p.tiles_n * p.split_k;
  const int grid = (int)(items < sms ? items : sms);
  k<<<grid, (kRoleWarps + EPIW) * 32, kSmem, s>>>(ma, mb, p, 0);
  return check_launch("gemm_tc_fast");
}

// The fast route covers int32 / int64 accumulation while no item has more than 510
// K-tiles (in-range addends are < 2^22, so their int32 sum cannot overflow) and the
// "|p| < 2" screen implies "|p * 2^f| < 2^22" (f <= 21).
bool gemm_tc_fast_supported(const GemmArgs& g, int split_k) {
  if (g.int_bits == 16) return false;
  if (g.frac_bits > 21) return false;
  if (g.k_tile != 64 && g.k_tile != 128) return false;
  const int64_t k_tiles = (g.K + g.k_tile - 1) / g.k_tile;
  const int64_t per_item = (k_tiles + split_k - 1) / split_k;
  return per_item <= 510;
}

int gemm_tc_fast(const GemmArgs& g, TcParams& p, const CUtensorMap& ma, const CUtensorMap& mb,
                 cudaStream_t s) {
  const int sms = tc_device_sms();
  if (sms < 0) return FXPR_ERR_ARCH;
  p.idesc = make_idesc(g.dtype == FXPR_BF16 ? 1 : 0, p.b_kmajor ? 0 : 1, 128, kBM);
  const bool dump = p.partials != nullptr;
#define FXPR_FAST(TT)                                                                              \
  do {                                                                                             \
    if (dump) return launch_fast<TT, 128, 16, true>(ma, mb, p, sms, s);                            \
    return launch_fast<TT, 128, 16, false>(ma, mb, p, sms, s);                                     \
  } while (0)
  if (g.dtype == FXPR_BF16) FXPR_FAST(__nv_bfloat16);
  FXPR_FAST(__half);
#undef FXPR_FAST
}

}  // namespace fxpr

// 128 x 256 output tiles for the tensor-core fixed-point GEMM (sm_100a).
//
// Why a second tile shape: the single thread that issues tcgen05.mma needs about the same
// time for a 128x128x16 MMA (64 tensor-pipe clocks) as for its issue slot plus its share of
// the barrier probes and commits, so with 128-column tiles the tensor pipe idles during that
// overhead (gemm_tc_fast.cu, measured).  A 128x256x16 MMA keeps the pipe busy for 128 clocks
// per issue: half as many MMAs, probes and commits per flop.
//
// One K-tile accumulator is 128 lanes x 256 columns, so TMEM holds exactly two of them: the
// MMA warp fills one while the 16 epilogue warps drain the other.  Shared-memory stages are
// 64 deep (A 128x64, B 64x256: 48 KB), four of them; a K-tile of 64 is one stage, a K-tile of
// 128 two stages into the same accumulator.  Each epilogue thread owns one row and 64
// columns: 64 accumulator registers, TMEM read 8 columns at a time to stay inside the
// 96-register budget of an 18-warp CTA.
//
// Numerics, conversion (magic-number rounding with the exact fix-up), split-K planes and the
// bounded waits are those of gemm_tc_fast.cu; outputs are bit-identical to it.
#include <cuda.h>

#include "fxp_common.cuh"
#include "gemm_common.cuh"
#include "tc_common.cuh"
#include "gemm_tc_fast_common.cuh"

namespace fxpr {

static constexpr int kWdBN = 256;
static constexpr int kWdWarps = 2 + 16;
static constexpr int kWdStages = 4;
static constexpr int kWdABytes = kBM * kBK * 2;           // 16 KB
static constexpr int kWdBBytes = kWdBN * kBK * 2;         // 32 KB: four 64-column slabs
static constexpr int kWdStageBytes = kWdABytes + kWdBBytes;

__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld_regs8(uint32_t (&r)[8]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
               :: "memory");
}

template <typename T>
__global__ void __launch_bounds__(kWdWarps * 32, 1)
gemm_tc_n256_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const TcParams p, const int zero /* always 0: keeps the side arrays in local memory */) {
  constexpr int STAGES = kWdStages;
  constexpr int BN = kWdBN;
  constexpr int EPIW = 16;
  constexpr int kCols = BN / (EPIW / 4);                 // 64 columns per epilogue thread
  constexpr int kBarOffset = STAGES * kWdStageBytes;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kBarOffset;
  const uint32_t full0 = bar_base, empty0 = bar_base + 8u * STAGES;
  const uint32_t tfull0 = bar_base + 8u * (2 * STAGES), tempty0 = tfull0 + 16u;
  constexpr int kMisc = 8 * (2 * STAGES + 4);
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem_gen + kBarOffset + kMisc);
  volatile int* abort_flag = (volatile int*)(smem_gen + kBarOffset + kMisc + 8);
  const uint32_t epi_bar = bar_base + kMisc + 16u;
  volatile int* s_last = (volatile int*)(smem_gen + kBarOffset + kMisc + 24);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8u * s, 1); mbar_init(empty0 + 8u * s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8u * b, 1); mbar_init(tempty0 + 8u * b, EPIW); }
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
  const int halves = p.k_tile / 64;                      // stages per K-tile: 1 or 2

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
    const bool bk = p.b_kmajor != 0;
    int stage = 0; uint32_t phase = 1;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
      int pm, pn; tile_coords(item / p.split_k, pm, pn);
      const int m0 = pm * kBM, n0 = pn * BN;
      const int ks = item % p.split_k;
      const int n_kt = (k_tiles_total - ks + p.split_k - 1) / p.split_k;
      for (int i = 0; i < n_kt; ++i) {
        const int kt = ks + i * p.split_k;
        for (int h = 0; h < halves; ++h) {
          const int k0 = kt * p.k_tile + h * 64;
          if (!__all_sync(0xffffffffu, mbar_wait(empty0 + 8u * stage, phase, abort_flag))) goto producer_done;
          const uint32_t fb = full0 + 8u * stage;
          const uint32_t sa = smem_base + stage * kWdStageBytes;
          const uint32_t sb = sa + kWdABytes;
          if (lane == 0) {
            mbar_expect_tx(fb, kWdStageBytes);
            tma_load_2d(sa, &tma_a, fb, k0, m0);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, &tma_b, fb, bk ? k0 : n0 + j * 64, bk ? n0 + j * 64 : k0);
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  producer_done:;
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ----------------------------------
    const uint64_t adesc0 = make_smem_desc(smem_base, 16, 1024);
    const uint64_t bdesc0 = p.b_kmajor ? make_smem_desc(smem_base + kWdABytes, 16, 1024)
                                       : make_smem_desc(smem_base + kWdABytes, 8192, 1024);
    const uint64_t bks = p.b_kmajor ? 2 : 128;           // (32 B | 2048 B) >> 4 per 16-deep k step
    constexpr uint64_t kStep = kWdStageBytes >> 4;
    const uint32_t idesc = p.idesc;
    int stage = 0; uint32_t phase = 0; int buf = 0; uint32_t bphase = 1;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
      const int ks = item % p.split_k;
      const int n_kt = (k_tiles_total - ks + p.split_k - 1) / p.split_k;
      for (int i = 0; i < n_kt; ++i) {
        const uint32_t d = tmem_base + (uint32_t)(buf * BN);
        for (int h = 0; h < halves; ++h) {
          bool ok1 = true;
          if (h == 0) ok1 = mbar_wait(tempty0 + 8u * buf, bphase, abort_flag);
          const bool ok2 = mbar_wait(full0 + 8u * stage, phase, abort_flag);
          if (!__all_sync(0xffffffffu, ok1 && ok2)) goto issuer_done;
          tc_fence_after();
          const uint64_t ad = adesc0 + (uint64_t)stage * kStep;
          const uint64_t bd = bdesc0 + (uint64_t)stage * kStep;
          if (lane == 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) umma_f16(d, ad + 2 * q, bd + q * bks, idesc, (h || q) ? 1u : 0u);
            umma_commit(empty0 + 8u * stage);
            if (h == halves - 1) umma_commit(tfull0 + 8u * buf);
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        buf ^= 1; if (buf == 0) bphase ^= 1;
      }
    }
  issuer_done:;
  } else {
#include "gemm_tc_n256_epilogue.inl"
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

bool gemm_tc_fast_supported(const GemmArgs& g, int split_k);

// Same conditions as the 128-column route, plus enough 256-column tiles to be worth it.
bool gemm_tc_n256_supported(const GemmArgs& g, int split_k) {
  return g.partials == nullptr && g.N >= 256 && gemm_tc_fast_supported(g, split_k);
}

template <typename T>
static int launch_n256(const CUtensorMap& ma, const CUtensorMap& mb, TcParams& p, int sms, cudaStream_t s) {
  constexpr int kSmem = kWdStages * kWdStageBytes + 256 + 1024;
  auto k = gemm_tc_n256_kernel<T>;
  static bool attr_done_dev[64] = {};            // function attributes are per device
  int dev_id = 0;
  cudaGetDevice(&dev_id);
  bool& attr_done = attr_done_dev[dev_id & 63];
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
    if (e != cudaSuccess) { set_last_error("gemm_tc_n256 smem attribute", e); return FXPR_ERR_CUDA; }
    attr_done = true;
  }
  p.tiles_m = (p.M + kBM - 1) / kBM;
  p.tiles_n = (p.N + kWdBN - 1) / kWdBN;
  const int64_t items = (int64_t)p.tiles_m * p.tiles_n * p.split_k;
  const int grid = (int)(items < sms ? items : sms);
  k<<<grid, kWdWarps * 32, kSmem, s>>>(ma, mb, p, 0);
  return check_launch("gemm_tc_n256");
}

// ma, mb: the tensor maps of gemm_tc() (A: 128-row boxes, B: 64-row boxes in either layout).
int gemm_tc_n256(const GemmArgs& g, TcParams& p, const CUtensorMap& ma, const CUtensorMap& mb, cudaStream_t s) {
  const int sms = tc_device_sms();
  if (sms < 0) return FXPR_ERR_ARCH;
  p.idesc = make_idesc(g.dtype == FXPR_BF16 ? 1 : 0, p.b_kmajor ? 0 : 1, kWdBN, kBM);
  if (g.dtype == FXPR_BF16) return launch_n256<__nv_bfloat16>(ma, mb, p, sms, s);
  return launch_n256<__half>(ma, mb, p, sms, s);
}

}  // namespace fxpr

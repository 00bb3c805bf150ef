// Wide-tile route of the tensor-core fixed-point GEMM (sm_100a) with a lean epilogue.
//
// The fixed-point contract (fxpr_vllm/_triton/gemm.py:183-195 of the reference) gives every
// K-tile a fresh fp32 accumulator that has to be rounded to Q-format and integer-added
// before the next one may reuse its tensor memory, so the kernel is bound by the number of
// instructions its epilogue warps issue per accumulator element, not by the tensor pipe.
// This kernel spends as few as it can:
//
//   * 8 epilogue warps instead of 16: half as many warps poll barriers, run loop control
//     and compute addresses; each thread owns one output row and BN/2 columns.
//   * tcgen05.ld of 16 columns into one of two register sets; the load of the next chunk
//     is in flight while the current one is converted.
//   * the conversion r = fma(p, 2^f, 1.5 * 2^23) is done two elements at a time with
//     fma.rn.f32x2 (one issue slot for two partials), the raw bit patterns are summed with
//     32-bit integer adds and n_ktiles * bits(1.5 * 2^23) is subtracted once per tile;
//     the OR of the raw partials screens for |p| >= 2 (exact fix-up of that K-tile with
//     cvt.rni, as in gemm_tc_fast.cu -- same bits for every input).
//   * the accumulator goes back to the MMA warp as soon as the last chunk has left tensor
//     memory and passed the screen, before that chunk is converted.
//
// Tile 128 x BN with BN = 256 (two accumulators in tensor memory, four 48 KB stages) or
// BN = 128 (four accumulators, six 32 KB stages); shared-memory stages are 64 deep, a
// K-tile of 128 is two stages into one accumulator.  Warp 0 = TMA producer, warp 1 =
// tcgen05.mma issuer.  Split-K planes, bounded waits and the persistent grouped-M tile
// order are those of gemm_tc_fast.cu; outputs are bit-identical to it.
#include <cuda.h>

#include "fxp_common.cuh"
#include "gemm_common.cuh"
#include "tc_common.cuh"
#include "gemm_tc_fast_common.cuh"

namespace fxpr {

static constexpr int kLnFirstEpi = 2;

// {lo, hi} = fma.rn(a, s, m) on both halves: one instruction for two partials
__device__ __forceinline__ void fma2_bits(uint32_t a0, uint32_t a1, uint64_t s2, uint64_t m2,
                                          uint32_t& r0, uint32_t& r1) {
  uint64_t a, d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "r"(a0), "r"(a1));
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(s2), "l"(m2));
  asm("mov.b64 {%0, %1}, %2;" : "=r"(r0), "=r"(r1) : "l"(d));
}

// tcgen05.ld of 8 / 16 / 32 columns and the matching wait that names the loaded registers
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
__device__ __forceinline__ void tmem_wait_ld_regs32(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :: "memory");
}
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, uint32_t (&r)[8]) { tmem_ld8(taddr, r); }
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_ldn(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld32(taddr, r); }
__device__ __forceinline__ void tmem_wait_ldn(uint32_t (&r)[8]) { tmem_wait_ld_regs8(r); }
__device__ __forceinline__ void tmem_wait_ldn(uint32_t (&r)[16]) { tmem_wait_ld_regs(r); }
__device__ __forceinline__ void tmem_wait_ldn(uint32_t (&r)[32]) { tmem_wait_ld_regs32(r); }

template <int BN> struct LeanCfg {
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kNBuf = 512 / BN;
  static constexpr int kSmem = kStages * kStageBytes + 256 + 1024;
};

template <typename T, int BN, int EPIW, int CH, bool F2, bool PIPE, bool DUMP>
__global__ void __launch_bounds__((kLnFirstEpi + EPIW) * 32, 1)
gemm_tc_lean_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const TcParams p, const int zero /* always 0: keeps the side arrays in local memory */) {
  using Cfg = LeanCfg<BN>;
  constexpr int STAGES = Cfg::kStages;
  constexpr int NBUF = Cfg::kNBuf;
  constexpr int kCols = BN / (EPIW / 4);                // columns per epilogue thread
  constexpr int NCH = kCols / CH;
  constexpr int kBarOffset = STAGES * Cfg::kStageBytes;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kBarOffset;
  const uint32_t full0 = bar_base, empty0 = bar_base + 8u * STAGES;
  const uint32_t tfull0 = bar_base + 8u * (2 * STAGES), tempty0 = tfull0 + 8u * NBUF;
  constexpr int kMisc = 8 * (2 * STAGES + 2 * NBUF);
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem_gen + kBarOffset + kMisc);
  volatile int* abort_flag = (volatile int*)(smem_gen + kBarOffset + kMisc + 8);
  const uint32_t epi_bar = bar_base + kMisc + 16u;
  volatile int* s_last = (volatile int*)(smem_gen + kBarOffset + kMisc + 24);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8u * s, 1); mbar_init(empty0 + 8u * s, 1); }
    for (int b = 0; b < NBUF; ++b) { mbar_init(tfull0 + 8u * b, 1); mbar_init(tempty0 + 8u * b, EPIW); }
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
  const int halves = p.k_tile / 64;                     // stages per K-tile: 1 or 2

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
          const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
          const uint32_t sb = sa + Cfg::kABytes;
          if (lane == 0) {
            mbar_expect_tx(fb, Cfg::kStageBytes);
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
    const uint64_t bdesc0 = p.b_kmajor ? make_smem_desc(smem_base + Cfg::kABytes, 16, 1024)
                                       : make_smem_desc(smem_base + Cfg::kABytes, 8192, 1024);
    const uint64_t bks = p.b_kmajor ? 2 : 128;          // (32 B | 2048 B) >> 4 per 16-deep k step
    constexpr uint64_t kStep = Cfg::kStageBytes >> 4;
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
            if (p.dbg != 3) {
#pragma unroll
            for (int q = 0; q < 4; ++q) umma_f16(d, ad + 2 * q, bd + q * bks, idesc, (h || q) ? 1u : 0u);
            }
            umma_commit(empty0 + 8u * stage);
            if (h == halves - 1) umma_commit(tfull0 + 8u * buf);
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (++buf == NBUF) { buf = 0; bphase ^= 1; }
      }
    }
  issuer_done:;
  } else if (warp >= kLnFirstEpi) {
    // ------------------------------ epilogue warps -------------------------------
    // Warp w owns tensor-memory lanes 32 * (w % 4) .. (one output row per thread) and kCols
    // consecutive columns.
    const int quarter = warp & 3;
    const int cgroup = (warp - kLnFirstEpi) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    const int col0 = cgroup * kCols;
    const uint32_t lane_addr = ((uint32_t)(quarter * 32) << 16) + (uint32_t)col0;
    const float scale = p.scale;
    uint64_t scale2, magic_pos2, magic_neg2;
    asm("mov.b64 %0, {%1, %1};" : "=l"(scale2) : "r"(__float_as_uint(scale)));
    asm("mov.b64 %0, {%1, %1};" : "=l"(magic_pos2) : "r"(kMagicBits));
    asm("mov.b64 %0, {%1, %1};" : "=l"(magic_neg2) : "r"(kMagicBits | 0x80000000u));
    int buf = 0; uint32_t bphase = 0; uint32_t epi_phase = 0; bool ok = true;
    auto epi_sync = [&]() -> bool {   // bounded barrier over the epilogue warps only
      __syncwarp();
      if (lane == 0) mbar_arrive(epi_bar);
      const bool done = warp_wait(epi_bar, epi_phase, abort_flag, lane);
      epi_phase ^= 1;
      return done;
    };

    // Side arrays in local memory: the integer sums the float accumulators are flushed into
    // every `flush_every` K-tiles, and the exact conversions of out-of-range partials.
    uint32_t acc_i[kCols];
    long long corr_q[kCols];
    bool corr_used = false;
    const int flush_every = p.flush_every;               // even; 2^(21 - f) K-tiles

    for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const int tile = item / p.split_k, ks = item % p.split_k;
      int pm, pn; tile_coords(tile, pm, pn);
      const int row = pm * kBM + row_in_tile;
      const int ncol0 = pn * BN + col0;
      const int n_kt = (k_tiles_total - ks + p.split_k - 1) / p.split_k;
      // Float accumulators, two per 64-bit register.  Even K-tiles add MAGIC + q, odd ones
      // -MAGIC + q, so the running value alternates between S and MAGIC + S (S = the integer
      // sum so far); both are exactly representable while |S| < 2^22, so every add is exact.
      uint64_t acc2[kCols / 2];
#pragma unroll
      for (int i = 0; i < kCols / 2; ++i) acc2[i] = 0;
      corr_used = false;
      bool flushed = false;
      int since = 0;

      for (int kt = 0; kt < n_kt; ++kt) {
        if (!warp_wait(tfull0 + 8u * buf, bphase, abort_flag, lane)) { ok = false; break; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + lane_addr + (uint32_t)(buf * BN);
        const uint64_t m2 = (since & 1) ? magic_neg2 : magic_pos2;
        uint32_t v[PIPE ? 2 : 1][CH];
        if (p.dbg == 2) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(tempty0 + 8u * buf);
          if (++buf == NBUF) { buf = 0; bphase ^= 1; }
          continue;
        }
        tmem_ldn(taddr, v[0]);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          uint32_t (&cur)[CH] = v[PIPE ? (c & 1) : 0];
          tmem_wait_ldn(cur);
          if (PIPE && c + 1 < NCH) tmem_ldn(taddr + (c + 1) * CH, v[PIPE ? ((c + 1) & 1) : 0]);
          if (c + 1 == NCH) {
            // every partial of this accumulator is in registers: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8u * buf);
          }
          if (DUMP) {
            if (row < p.M) {
              const int ktg = ks + kt * p.split_k;
              float* dst = p.partials + ((int64_t)ktg * p.M + row) * p.N + ncol0 + c * CH;
#pragma unroll
              for (int i = 0; i < CH; ++i)
                if (ncol0 + c * CH + i < p.N) dst[i] = __uint_as_float(cur[i]);
            }
          }
          // Screen: bit 30 of the OR of the raw fp32 bits stays clear only if every |p| < 2,
          // i.e. |p * 2^f| < 2^(f+1).  A thread that sees it set converts the out-of-range
          // partials of this chunk with the reference's cvt.rni (fxp.py:92-108) into corr_q
          // and replaces them by 0 before the fast path runs, so the float accumulators
          // only ever see in-range values.
          uint32_t screen = 0;
#pragma unroll
          for (int i = 0; i < CH; i += 2) screen |= cur[i] | cur[i + 1];
          if (screen & 0x40000000u) {
            if (!corr_used) {
#pragma unroll 1
              for (int z = 0; z < kCols; ++z) corr_q[z + zero] = 0;
              corr_used = true;
            }
#pragma unroll
            for (int i = 0; i < CH; ++i) {
              const float f = __uint_as_float(cur[i]);
              if (!(fabsf(f) < 2.0f)) {
                corr_q[c * CH + i + zero] += (p.int_bits == 64) ? float_to_fixed<64>(f, scale)
                                                               : (long long)float_to_fixed<32>(f, scale);
                cur[i] = 0;
              }
            }
          }
#pragma unroll
          for (int i = 0; i < CH; i += 2) {
            uint64_t a, r;
            asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "r"(cur[i]), "r"(cur[i + 1]));
            asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(scale2), "l"(m2));
            asm("add.rn.f32x2 %0, %1, %2;" : "=l"(acc2[(c * CH + i) / 2]) : "l"(acc2[(c * CH + i) / 2]), "l"(r));
          }
          if (!PIPE && c + 1 < NCH) tmem_ldn(taddr + (c + 1) * CH, v[0]);
        }
        if (++buf == NBUF) { buf = 0; bphase ^= 1; }
        if (++since == flush_every) {
          // |S| could reach 2^22 with the next K-tile: move it to the integer sums
          if (!flushed) {
#pragma unroll 1
            for (int z = 0; z < kCols; ++z) acc_i[z + zero] = 0;
            flushed = true;
          }
#pragma unroll
          for (int i = 0; i < kCols / 2; ++i) {
            uint32_t lo, hi;
            asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(acc2[i]));
            acc_i[2 * i + zero] += (uint32_t)__float2int_rz(__uint_as_float(lo));
            acc_i[2 * i + 1 + zero] += (uint32_t)__float2int_rz(__uint_as_float(hi));
            acc2[i] = 0;
          }
          since = 0;
        }
      }
      if (!ok) break;

      if (since & 1) {   // an odd number of K-tiles since the last flush: take MAGIC out again
#pragma unroll
        for (int i = 0; i < kCols / 2; ++i)
          asm("add.rn.f32x2 %0, %1, %2;" : "=l"(acc2[i]) : "l"(acc2[i]), "l"(magic_neg2));
      }
      auto total = [&](int i) -> long long {
        uint32_t lo, hi;
        asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(acc2[i >> 1]));
        uint32_t raw = (uint32_t)__float2int_rz(__uint_as_float((i & 1) ? hi : lo));
        if (flushed) raw += acc_i[i + zero];
        // the in-range part is < 2^31 in magnitude: the wrapped 32-bit sum is its value
        long long t = (long long)(int32_t)raw;
        if (corr_used) t += corr_q[i + zero];
        return p.int_bits == 64 ? t : (long long)(int32_t)t;
      };

      // Split-K: every split leaves its integer partial tile in its own plane of the scratch
      // (column-major inside the tile, so a warp's 32 rows are 32 consecutive words and every
      // store and load is one full line); the split that arrives last adds the planes of the
      // others to its registers.  Integer addition is commutative and associative: which
      // split comes last cannot change the sum.
      const bool row_ok = row < p.M;
      bool do_store = true;
      const int64_t plane_elems = (int64_t)kBM * BN;
      const int64_t plane_stride = (int64_t)p.tiles_m * p.tiles_n * plane_elems;
      const int64_t plane_off = (int64_t)tile * plane_elems + (int64_t)col0 * kBM + row_in_tile;
      if (p.split_k > 1) {
        if (p.int_bits == 64) {
          long long* dst = (long long*)p.acc_scratch + ks * plane_stride + plane_off;
#pragma unroll
          for (int i = 0; i < kCols; ++i) __stcg(dst + i * kBM, total(i));
        } else {
          int* dst = (int*)p.acc_scratch + ks * plane_stride + plane_off;
#pragma unroll
          for (int i = 0; i < kCols; ++i) __stcg(dst + i * kBM, (int)total(i));
        }
        __threadfence();
        if (!epi_sync()) { ok = false; break; }
        if (threadIdx.x == kLnFirstEpi * 32) *s_last = (atomicAdd(p.locks + tile, 1) == p.split_k - 1) ? 1 : 0;
        if (!epi_sync()) { ok = false; break; }
        do_store = *s_last != 0;
        if (do_store) __threadfence();
      }

      if (do_store && row_ok) {
        T* cdst = p.c ? (T*)p.c + (int64_t)row * p.c_sm + ncol0 : nullptr;
        const T* bias = (const T*)p.bias;
#pragma unroll
        for (int g = 0; g < kCols / 8; ++g) {
          long long q8[8];
          const int colg = ncol0 + g * 8;
#pragma unroll
          for (int i = 0; i < 8; ++i) q8[i] = total(g * 8 + i);
          if (p.split_k > 1) {
            for (int s2 = 0; s2 < p.split_k; ++s2) {
              if (s2 == ks) continue;
              if (p.int_bits == 64) {
                const long long* src = (const long long*)p.acc_scratch + s2 * plane_stride + plane_off + (int64_t)g * 8 * kBM;
#pragma unroll
                for (int i = 0; i < 8; ++i) q8[i] += __ldcg(src + i * kBM);
              } else {
                const int* src = (const int*)p.acc_scratch + s2 * plane_stride + plane_off + (int64_t)g * 8 * kBM;
#pragma unroll
                for (int i = 0; i < 8; ++i) q8[i] += (long long)__ldcg(src + i * kBM);
              }
            }
            if (p.int_bits != 64) {
#pragma unroll
              for (int i = 0; i < 8; ++i) q8[i] = (long long)(int32_t)q8[i];
            }
          }
          if (p.c_int) {
            if (p.int_bits == 64) {
              long long* dst = (long long*)p.c_int + (int64_t)row * p.N + colg;
#pragma unroll
              for (int i = 0; i < 8; ++i) if (colg + i < p.N) dst[i] = q8[i];
            } else {
              int32_t* dst = (int32_t*)p.c_int + (int64_t)row * p.N + colg;
#pragma unroll
              for (int i = 0; i < 8; ++i) if (colg + i < p.N) dst[i] = (int32_t)q8[i];
            }
          }
          if (cdst) {
            alignas(16) T out[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float v8 = fixed_to_float<long long>(q8[i], p.inv_scale);
              if (bias && colg + i < p.N) v8 = __fadd_rn(v8, to_f32<T>(bias[colg + i]));
              out[i] = from_f32<T>(v8);
            }
            if (p.c_vec_ok && colg + 8 <= p.N) {
              *reinterpret_cast<uint4*>(cdst + g * 8) = *reinterpret_cast<const uint4*>(out);
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i) if (colg + i < p.N) cdst[g * 8 + i] = out[i];
            }
          }
        }
      }
      if (p.split_k > 1) {
        if (do_store && threadIdx.x == kLnFirstEpi * 32) p.locks[tile] = 0;
        if (!epi_sync()) { ok = false; break; }    // s_last is rewritten only after all have read it
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
    tmem_dealloc(tmem_base, 512);
  }
}

bool gemm_tc_fast_supported(const GemmArgs& g, int split_k);

// Same numeric conditions as gemm_tc_fast.cu (int32 / int64 sums, f <= 21, at most 510
// K-tiles per item).
bool gemm_tc_lean_supported(const GemmArgs& g, int split_k) {
  return g.N >= 128 && gemm_tc_fast_supported(g, split_k);
}

template <typename T, int BN, int EPIW, int CH, bool F2, bool PIPE, bool DUMP>
static int launch_lean(const CUtensorMap& ma, const CUtensorMap& mb, TcParams& p, int sms, cudaStream_t s) {
  using Cfg = LeanCfg<BN>;
  auto k = gemm_tc_lean_kernel<T, BN, EPIW, CH, F2, PIPE, DUMP>;
  static bool attr_done_dev[64] = {};            // function attributes are per device
  int dev_id = 0;
  cudaGetDevice(&dev_id);
  bool& attr_done = attr_done_dev[dev_id & 63];
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem);
    if (e != cudaSuccess) { set_last_error("gemm_tc_lean smem attribute", e); return FXPR_ERR_CUDA; }
    attr_done = true;
  }
  p.tiles_m = (p.M + kBM - 1) / kBM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int64_t items = (int64_t)p.tiles_m * p.tiles_n * p.split_k;
  const int grid = (int)(items < sms ? items : sms);
  k<<<grid, (kLnFirstEpi + EPIW) * 32, Cfg::kSmem, s>>>(ma, mb, p, 0);
  return check_launch("gemm_tc_lean");
}

// ma, mb: the tensor maps of gemm_tc() (A: 128-row boxes, B: 64-row boxes in either layout).
int gemm_tc_lean(const GemmArgs& g, TcParams& p, const CUtensorMap& ma, const CUtensorMap& mb,
                 int bn, cudaStream_t s) {
  const int sms = tc_device_sms();
  if (sms < 0) return FXPR_ERR_ARCH;
  p.idesc = make_idesc(g.dtype == FXPR_BF16 ? 1 : 0, p.b_kmajor ? 0 : 1, bn, kBM);
  const bool dump = p.partials != nullptr;
  const int var = (g.flags >> 10) & 15;    // experiment selector
  p.dbg = (g.flags >> 14) & 3;
  // in-range partials are < 2^(f+1) after scaling; the float accumulators hold |S| < 2^22
  p.flush_every = g.frac_bits >= 20 ? 2 : (1 << (21 - g.frac_bits > 9 ? 9 : 21 - g.frac_bits));
  if (g.dtype == FXPR_BF16 && !dump && var) {
    using TT = __nv_bfloat16;
    if (bn == 128) switch (var) {
      case 1: return launch_lean<TT, 128, 16, 16, true, false, false>(ma, mb, p, sms, s);
      case 2: return launch_lean<TT, 128, 16, 8, true, true, false>(ma, mb, p, sms, s);
      case 3: return launch_lean<TT, 128, 8, 16, true, true, false>(ma, mb, p, sms, s);
      case 4: return launch_lean<TT, 128, 8, 32, true, false, false>(ma, mb, p, sms, s);
      case 5: return launch_lean<TT, 128, 8, 16, true, false, false>(ma, mb, p, sms, s);
      case 6: return launch_lean<TT, 128, 16, 32, true, false, false>(ma, mb, p, sms, s);
      default: break;
    } else switch (var) {
      case 1: return launch_lean<TT, 256, 16, 16, true, false, false>(ma, mb, p, sms, s);
      case 2: return launch_lean<TT, 256, 16, 8, true, true, false>(ma, mb, p, sms, s);
      case 3: return launch_lean<TT, 256, 8, 16, true, true, false>(ma, mb, p, sms, s);
      case 4: return launch_lean<TT, 256, 8, 32, true, false, false>(ma, mb, p, sms, s);
      case 5: return launch_lean<TT, 256, 8, 16, true, false, false>(ma, mb, p, sms, s);
      case 6: return launch_lean<TT, 256, 16, 32, true, false, false>(ma, mb, p, sms, s);
      default: break;
    }
  }
#define FXPR_LEAN(TT)                                                                  \
  do {                                                                                 \
    if (bn == 256) {                                                                   \
      if (dump) return launch_lean<TT, 256, 8, 8, true, true, true>(ma, mb, p, sms, s);   \
      return launch_lean<TT, 256, 8, 8, true, true, false>(ma, mb, p, sms, s);            \
    }                                                                                  \
    if (dump) return launch_lean<TT, 128, 8, 16, true, true, true>(ma, mb, p, sms, s);    \
    return launch_lean<TT, 128, 8, 16, true, true, false>(ma, mb, p, sms, s);             \
  } while (0)
  if (g.dtype == FXPR_BF16) FXPR_LEAN(__nv_bfloat16);
  FXPR_LEAN(__half);
#undef FXPR_LEAN
}

}  // namespace fxpr

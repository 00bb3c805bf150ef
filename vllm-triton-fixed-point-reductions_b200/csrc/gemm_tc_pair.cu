// Two-SM route of the tensor-core fixed-point GEMM (sm_100a): tcgen05.mma with
// cta_group::2 on clusters of two CTAs.
//
// Why: measured with an idle epilogue, the single-CTA kernels are bound by operand traffic
// from L2 into shared memory, not by the tensor pipe -- a 128 x 128 tile pulls 32 KB per
// 64-deep stage (2.1 GB for a 4096^3 problem, ~200 us), a 128 x 256 tile 48 KB (1.6 GB,
// ~140 us), against 82 us of tensor work.  A CTA pair computes a 256 x BN tile with ONE
// instruction stream: each CTA loads its own 128 rows of A and its own half of the BN columns
// of B, the tensor cores of both SMs read both halves of B, and each CTA's tensor memory
// receives its 128 rows x BN columns of the accumulator.  Per CTA that is 32 KB per stage
// for a 128 x 256 accumulator (1.07 GB in all), and one MMA-issuing thread per two SMs.
//
// Roles per CTA (18 warps): warp 0 = TMA producer (both CTAs, each for its own shared
// memory; the copies of both complete on the leader's "full" barrier), warp 1 = MMA issuer
// (leader CTA only; its commits arrive on the barriers of both CTAs), warps 2-17 = epilogue
// (each CTA drains its own tensor memory; the follower's warps arrive on the leader's
// "accumulator free" barrier through the cluster address space).  Every copy names one
// destination and one barrier; only tcgen05.commit signals both CTAs at once.
//
// Barriers: full[stage] (leader), done[stage] (both CTAs: "the MMAs that read this stage
// have finished" -- the producer refills the stage on it and, for the last stage of a
// K-tile, the epilogue reads the accumulator on it: one commit per stage serves both),
// tempty[buffer] (the CTA's 16 epilogue warps have drained the buffer; the follower's idle
// warp 1 forwards its completion to the leader's as ONE remote arrival.  Measured at 4096^3,
// K-tile 128: sixteen remote arrivals per K-tile 259 us, the forwarding warp 212 us, a
// shared-memory counter whose last arriver signals 236 us).
//
// Numerics, the magic-number conversion with its exact fix-up, split-K planes, bounded
// waits and the persistent grouped tile order are those of gemm_tc_fast.cu; results are
// bit-identical to it (the fixed-point contract: fxpr_vllm/_triton/gemm.py:183-204).
#include <cuda.h>

#include "fxp_common.cuh"
#include "gemm_common.cuh"
#include "tc_common.cuh"
#include "gemm_tc_fast_common.cuh"

namespace fxpr {

static constexpr int kPrEpiW = 16;
static constexpr int kPrFirstEpi = 2;
static constexpr int kPrThreads = (kPrFirstEpi + kPrEpiW) * 32;
static constexpr int kPrGroupM = 4;        // pair-tile rows (256 each) per L2 group

// ---- cluster / cta_group::2 PTX ---------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cta address -> shared::cluster address of the same offset in CTA `rank`
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load whose completion bytes are counted on a barrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair once every MMA
// this thread issued so far is done.  One instruction for both: a tcgen05.commit costs the
// issuing thread ~260 clocks here (measured with no MMA in flight), so commits are rationed.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(both) : "memory");
}
__device__ __forceinline__ void tmem_ld8p(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld8p(uint32_t (&r)[8]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
               :: "memory");
}
__device__ __forceinline__ void tmem_ldp(uint32_t taddr, uint32_t (&r)[8]) { tmem_ld8p(taddr, r); }
__device__ __forceinline__ void tmem_ldp(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld16(taddr, r); }
__device__ __forceinline__ void tmem_wait_ldp(uint32_t (&r)[8]) { tmem_wait_ld8p(r); }
__device__ __forceinline__ void tmem_wait_ldp(uint32_t (&r)[16]) { tmem_wait_ld_regs(r); }

// Non-blocking probe.  mbarrier.try_wait may park the thread for a hardware time limit, and a
// parked thread is woken promptly only by arrivals from its own CTA; most barriers here are
// completed from the peer CTA, so the waits of this kernel poll with test_wait instead.
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
__device__ __forceinline__ bool mbar_wait_poll(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_test_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (!mbar_test_wait(bar, parity)) {
    if ((++spins & 255) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitCycles) { *abort_flag = 1; return false; }
    }
  }
  return true;
}
__device__ __forceinline__ bool warp_wait_poll(uint32_t bar, uint32_t parity, volatile int* abort_flag, int lane) {
  int ok = 1;
  if (lane == 0) ok = mbar_wait_poll(bar, parity, abort_flag) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

template <int BN> struct PairCfg {
  static constexpr int kStages = BN == 256 ? 6 : 8;
  static constexpr int kABytes = kBM * kBK * 2;             // this CTA's 128 rows of A
  static constexpr int kBBytes = (BN / 2) * kBK * 2;        // this CTA's half of the B columns
  static constexpr int kStageBytes = kABytes + kBBytes;     // 32 KB / 24 KB
  static constexpr int kNBuf = 512 / BN;
  static constexpr int kSmem = kStages * kStageBytes + 256 + 1024;
  static constexpr int kChunk = BN == 256 ? 8 : 16;         // columns per tcgen05.ld
};

template <typename T, int BN, bool DUMP>
__global__ void __launch_bounds__(kPrThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const TcParams p, const int zero /* always 0: keeps the side arrays in local memory */) {
  using Cfg = PairCfg<BN>;
  constexpr int STAGES = Cfg::kStages;
  constexpr int NBUF = Cfg::kNBuf;
  constexpr int CH = Cfg::kChunk;
  constexpr int kCols = BN / (kPrEpiW / 4);               // columns per epilogue thread
  constexpr int NCH = kCols / CH;
  constexpr int kBarOffset = STAGES * Cfg::kStageBytes;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + kBarOffset;
  const uint32_t full0 = bar_base, done0 = bar_base + 8u * STAGES;
  const uint32_t tempty0 = bar_base + 8u * (2 * STAGES);
  constexpr int kMisc = 8 * (2 * STAGES + NBUF);
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem_gen + kBarOffset + kMisc);
  volatile int* abort_flag = (volatile int*)(smem_gen + kBarOffset + kMisc + 8);
  const uint32_t epi_bar = bar_base + kMisc + 16u;
  volatile int* s_last = (volatile int*)(smem_gen + kBarOffset + kMisc + 24);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                 // 0 = leader
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    // full: one arrive (the leader's producer) plus the bytes of both CTAs; done: one commit;
    // tempty: this CTA's epilogue warps, plus in the leader one arrival forwarded from the follower
    for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8u * s, 1); mbar_init(done0 + 8u * s, 1); }
    for (int b = 0; b < NBUF; ++b) mbar_init(tempty0 + 8u * b, rank == 0 ? kPrEpiW + 1 : kPrEpiW);
    mbar_init(epi_bar, kPrEpiW);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32((const void*)tmem_slot), 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                      // the peer's barriers exist from here on
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_mn = p.tiles_m * p.tiles_n;              // pair tiles: 256 rows x BN columns
  const int items = tiles_mn * p.split_k;
  const int k_tiles_total = (p.K + p.k_tile - 1) / p.k_tile;
  const int halves = p.k_tile / 64;                        // stages per K-tile: 1 or 2

  auto tile_coords = [&](int tile, int& pm, int& pn) {
    const int in_group = kPrGroupM * p.tiles_n;
    const int g = tile / in_group;
    const int first = g * kPrGroupM;
    const int gsz = min(p.tiles_m - first, kPrGroupM);
    pm = first + (tile % in_group) % gsz;
    pn = (tile % in_group) / gsz;
  };

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ----------------------
    const bool bk = p.b_kmajor != 0;
    int stage = 0; uint32_t phase = 1;
    for (int item = pair_id; item < items; item += num_pairs) {
      int pm, pn; tile_coords(item / p.split_k, pm, pn);
      const int m0 = pm * 256 + (int)rank * kBM;
      const int n0 = pn * BN + (int)rank * (BN / 2);
      const int ks = item % p.split_k;
      const int n_kt = (k_tiles_total - ks + p.split_k - 1) / p.split_k;
      for (int i = 0; i < n_kt; ++i) {
        const int kt = ks + i * p.split_k;
        for (int h = 0; h < halves; ++h) {
          const int k0 = kt * p.k_tile + h * 64;
          if (!__all_sync(0xffffffffu, mbar_wait_poll(done0 + 8u * stage, phase, abort_flag))) goto producer_done;
          const uint32_t fb_local = full0 + 8u * stage;
          const uint32_t fb = mapa_u32(fb_local, 0);       // the leader's barrier counts both CTAs' bytes
          const uint32_t sa = smem_base + stage * Cfg::kStageBytes;
          const uint32_t sb = sa + Cfg::kABytes;
          if (lane == 0) {
            if (rank == 0) mbar_expect_tx(fb_local, 2 * Cfg::kStageBytes);
            tma_load_2d_pair(sa, &tma_a, fb, k0, m0);
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)
              tma_load_2d_pair(sb + j * 8192, &tma_b, fb, bk ? k0 : n0 + j * 64, bk ? n0 + j * 64 : k0);
          }
          __syncwarp();
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  producer_done:;
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader only) ----------------------
    if (rank == 0) {
      const uint64_t adesc0 = make_smem_desc(smem_base, 16, 1024);
      const uint64_t bdesc0 = p.b_kmajor ? make_smem_desc(smem_base + Cfg::kABytes, 16, 1024)
                                         : make_smem_desc(smem_base + Cfg::kABytes, 8192, 1024);
      const uint64_t bks = p.b_kmajor ? 2 : 128;          // (32 B | 2048 B) >> 4 per 16-deep k step
      constexpr uint64_t kStep = Cfg::kStageBytes >> 4;
      const uint32_t idesc = p.idesc;
      int stage = 0; uint32_t phase = 0; int buf = 0; uint32_t bphase = 1;
      for (int item = pair_id; item < items; item += num_pairs) {
        const int ks = item % p.split_k;
        const int n_kt = (k_tiles_total - ks + p.split_k - 1) / p.split_k;
        for (int i = 0; i < n_kt; ++i) {
          const uint32_t d = tmem_base + (uint32_t)(buf * BN);
          for (int h = 0; h < halves; ++h) {
            bool ok1 = true;
            if (h == 0) ok1 = mbar_wait_poll(tempty0 + 8u * buf, bphase, abort_flag);
            const bool ok2 = mbar_wait_poll(full0 + 8u * stage, phase, abort_flag);
            if (!__all_sync(0xffffffffu, ok1 && ok2)) goto issuer_done;
            tc_fence_after();
            const uint64_t ad = adesc0 + (uint64_t)stage * kStep;
            const uint64_t bd = bdesc0 + (uint64_t)stage * kStep;
            if (lane == 0) {
#pragma unroll
              for (int q = 0; q < 4; ++q) umma_f16_pair(d, ad + 2 * q, bd + q * bks, idesc, (h || q) ? 1u : 0u);
              // in both CTAs: the stage may be refilled and, after the last stage of a K-tile,
              // the accumulator may be read, once these MMAs are done
              umma_commit_pair(done0 + 8u * stage);
            }
            __syncwarp();
            if (++stage == STAGES) { stage = 0; phase ^= 1; }
          }
          if (++buf == NBUF) { buf = 0; bphase ^= 1; }
        }
      }
    } else {
      // follower: forward "my epilogue has drained the buffer" to the leader
      const uint32_t tempty_leader0 = mapa_u32(tempty0, 0);
      int buf = 0; uint32_t fphase = 0;
      for (int item = pair_id; item < items; item += num_pairs) {
        const int ks = item % p.split_k;
        const int n_kt = (k_tiles_total - ks + p.split_k - 1) / p.split_k;
        for (int i = 0; i < n_kt; ++i) {
          if (!__all_sync(0xffffffffu, mbar_wait_poll(tempty0 + 8u * buf, fphase, abort_flag))) goto issuer_done;
          if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8u * buf);
          __syncwarp();
          if (++buf == NBUF) { buf = 0; fphase ^= 1; }
        }
      }
    }
  issuer_done:;
  } else {
    // ------------------------------ epilogue warps (both CTAs) --------------------
    // Warp w owns tensor-memory lanes 32 * (w % 4) .. (one output row per thread) and kCols
    // consecutive columns of this CTA's 128 x BN accumulator.
    const int quarter = warp & 3;
    const int cgroup = (warp - kPrFirstEpi) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    const int col0 = cgroup * kCols;
    const uint32_t lane_addr = ((uint32_t)(quarter * 32) << 16) + (uint32_t)col0;
    const float scale = p.scale;
    uint64_t scale2, magic2;
    asm("mov.b64 %0, {%1, %1};" : "=l"(scale2) : "r"(__float_as_uint(scale)));
    asm("mov.b64 %0, {%1, %1};" : "=l"(magic2) : "r"(kMagicBits));
    auto release_buffer = [&](int b) {     // this warp has drained accumulator buffer b
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8u * b);
    };
    int buf = 0; uint32_t epi_phase = 0; bool ok = true;
    int dstage = halves - 1; uint32_t dphase = 0;          // done-barrier of the K-tile's last stage
    auto epi_sync = [&]() -> bool {   // bounded barrier over this CTA's epilogue warps
      __syncwarp();
      if (lane == 0) mbar_arrive(epi_bar);
      const bool done = warp_wait(epi_bar, epi_phase, abort_flag, lane);
      epi_phase ^= 1;
      return done;
    };

    // Rare-path corrections (local memory, zeroed on first use): wrap-sum of the raw values
    // the fast add contributed for out-of-range partials, and the exact int64 sum of what
    // the reference conversion gives for them.
    uint32_t corr_raw[kCols];
    long long corr_q[kCols];
    bool corr_used = false;

    for (int item = pair_id; item < items && ok; item += num_pairs) {
      const int tile = item / p.split_k, ks = item % p.split_k;
      int pm, pn; tile_coords(tile, pm, pn);
      const int row = pm * 256 + (int)rank * kBM + row_in_tile;
      const int ncol0 = pn * BN + col0;
      const int n_kt = (k_tiles_total - ks + p.split_k - 1) / p.split_k;
      uint32_t acc[kCols];
#pragma unroll
      for (int i = 0; i < kCols; ++i) acc[i] = 0;
      corr_used = false;

      for (int kt = 0; kt < n_kt; ++kt) {
        if (!warp_wait_poll(done0 + 8u * dstage, dphase, abort_flag, lane)) { ok = false; break; }
        dstage += halves; if (dstage >= STAGES) { dstage -= STAGES; dphase ^= 1; }
        tc_fence_after();
        const uint32_t taddr = tmem_base + lane_addr + (uint32_t)(buf * BN);
        // r = fma(p, 2^f, MAGIC) two partials per instruction, raw bit patterns added as
        // integers; the OR of the raw fp32 bits is the range screen (bit 30 clear: every
        // |p| < 2, hence |p * 2^f| < 2^22 for f <= 21).  The next chunk's tcgen05.ld is in
        // flight while the current one is converted.
        uint32_t v[2][CH];
        uint32_t screen = 0;
        tmem_ldp(taddr, v[0]);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          uint32_t (&cur)[CH] = v[c & 1];
          tmem_wait_ldp(cur);
          if (c + 1 < NCH) tmem_ldp(taddr + (c + 1) * CH, v[(c + 1) & 1]);
#pragma unroll
          for (int i = 0; i < CH; i += 2) {
            uint64_t a, r;
            uint32_t r0, r1;
            asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "r"(cur[i]), "r"(cur[i + 1]));
            asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(scale2), "l"(magic2));
            asm("mov.b64 {%0, %1}, %2;" : "=r"(r0), "=r"(r1) : "l"(r));
            acc[c * CH + i] += r0;
            acc[c * CH + i + 1] += r1;
            screen |= cur[i] | cur[i + 1];
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
        }
        if (__any_sync(0xffffffffu, (screen & 0x40000000u) != 0)) {
          // exact fix-up of this K-tile (rare): see fixup_tile
          if (!corr_used) {
#pragma unroll 1
            for (int z = 0; z < kCols; ++z) { corr_raw[z + zero] = 0; corr_q[z + zero] = 0; }
            corr_used = true;
          }
          fixup_tile(taddr, kCols, scale, p.int_bits, &corr_raw[zero], &corr_q[zero]);
        }
        release_buffer(buf);
        if (++buf == NBUF) buf = 0;
      }
      if (!ok) break;

      // every K-tile added MAGIC once
      const uint32_t bias_bits = (uint32_t)n_kt * kMagicBits;
      auto total = [&](int i) -> long long {
        uint32_t raw = acc[i] - bias_bits;
        long long t;
        if (corr_used) {
          // the in-range part is < 2^31 in magnitude, so it is the sign extension of the
          // wrapped sum once the out-of-range raw values are taken out again
          raw -= corr_raw[i + zero];
          t = (long long)(int32_t)raw + corr_q[i + zero];
        } else {
          t = (long long)(int32_t)raw;
        }
        return p.int_bits == 64 ? t : (long long)(int32_t)t;
      };

      // Split-K: every split leaves its integer partial tile in its own plane of the scratch
      // (column-major inside this CTA's 128 x BN tile, so every store and load is a full
      // line); the split that arrives last adds the planes of the others to its registers.
      // Integer addition is commutative and associative: which split comes last cannot
      // change the sum.
      const bool row_ok = row < p.M;
      bool do_store = true;
      const int cta_tile = tile * 2 + (int)rank;
      const int64_t plane_elems = (int64_t)kBM * BN;
      const int64_t plane_stride = (int64_t)tiles_mn * 2 * plane_elems;
      const int64_t plane_off = (int64_t)cta_tile * plane_elems + (int64_t)col0 * kBM + row_in_tile;
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
        if (threadIdx.x == kPrFirstEpi * 32) *s_last = (atomicAdd(p.locks + cta_tile, 1) == p.split_k - 1) ? 1 : 0;
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
        if (do_store && threadIdx.x == kPrFirstEpi * 32) p.locks[cta_tile] = 0;
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
  // Neither CTA may leave while the other can still signal its barriers or while MMAs that
  // read its shared memory are in flight (the last tfull commit covers those).
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

bool gemm_tc_fast_supported(const GemmArgs& g, int split_k);

// Same numeric conditions as gemm_tc_fast.cu; worth it once a pair tile has two real row blocks.
bool gemm_tc_pair_supported(const GemmArgs& g, int split_k) {
  return g.M > 128 && g.N >= 128 && gemm_tc_fast_supported(g, split_k);
}

template <typename T, int BN, bool DUMP>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, TcParams& p, int sms, cudaStream_t s) {
  using Cfg = PairCfg<BN>;
  auto k = gemm_tc_pair_kernel<T, BN, DUMP>;
  static bool attr_done_dev[64] = {};            // function attributes are per device
  int dev_id = 0;
  cudaGetDevice(&dev_id);
  bool& attr_done = attr_done_dev[dev_id & 63];
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem);
    if (e != cudaSuccess) { set_last_error("gemm_tc_pair smem attribute", e); return FXPR_ERR_CUDA; }
    attr_done = true;
  }
  p.tiles_m = (p.M + 255) / 256;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int64_t items = (int64_t)p.tiles_m * p.tiles_n * p.split_k;
  const int pairs = (int)(items < sms / 2 ? items : sms / 2);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
  cfg.blockDim = dim3(kPrThreads, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, k, ma, mb, (const TcParams)p, 0);
  if (e != cudaSuccess) { set_last_error("gemm_tc_pair launch", e); return FXPR_ERR_CUDA; }
  return check_launch("gemm_tc_pair");
}

// ma, mb: the tensor maps of gemm_tc() (A: 128-row boxes, B: 64-row boxes in either layout).
int gemm_tc_pair(const GemmArgs& g, TcParams& p, const CUtensorMap& ma, const CUtensorMap& mb,
                 int bn, cudaStream_t s) {
  const int sms = tc_device_sms();
  if (sms < 0) return FXPR_ERR_ARCH;
  p.idesc = make_idesc(g.dtype == FXPR_BF16 ? 1 : 0, p.b_kmajor ? 0 : 1, bn, 256);
  const bool dump = p.partials != nullptr;
#define FXPR_PAIR(TT)                                                              \
  do {                                                                             \
    if (bn == 256) {                                                               \
      if (dump) return launch_pair<TT, 256, true>(ma, mb, p, sms, s);              \
      return launch_pair<TT, 256, false>(ma, mb, p, sms, s);                       \
    }                                                                              \
    if (dump) return launch_pair<TT, 128, true>(ma, mb, p, sms, s);                \
    return launch_pair<TT, 128, false>(ma, mb, p, sms, s);                         \
  } while (0)
  if (g.dtype == FXPR_BF16) FXPR_PAIR(__nv_bfloat16);
  FXPR_PAIR(__half);
#undef FXPR_PAIR
}

}  // namespace fxpr

// Prefill attention on the 5th-generation tensor cores (sm_100a): TMA-fed tcgen05.mma with
// the score tile and the per-tile P.V partial in tensor memory.
//
// Semantics: the fused kernel of the reference, fxpr_vllm/_triton/attention.py:127-301 --
// pass A finds the exact row maxima of s = (q.k) * scale * log2(e) (+ soft-cap, ALiBi, masks),
// pass B recomputes s, forms w = exp2(s - max), sums Q(w) into an integer denominator and,
// per 64-key tile, Q(P.V) with P = w rounded to the io dtype into an integer numerator
// (:259-290); out = num / max(den, 1e-6).  Key tiles are 64 wide from key 0.
//
// Bit compatibility: a tcgen05.mma kind::f16 chain of 16-deep steps in ascending k gives the
// same fp32 bits as the mma.sync.m16n8k16 chain of attention_mma.cu (measured on a B200:
// every element of 128 x 128 x {64, 128} products identical), ex2.approx and the roundings
// are the same instructions, so this kernel's outputs equal that kernel's bit for bit --
// which keeps "a token's bits do not depend on whether it was computed in a prefill block or
// a decode step" (the decode kernel stays on mma.sync) and is what the tests assert.
//
// One CTA = 128 query rows of one KV head: a row is a (token, query head of the GQA group)
// pair, so a K/V tile is fetched once for the whole group.  18 warps:
//   warp 0      producer: Q (once) and the K / V tiles of the paged cache by TMA, one box of
//               16 keys x 64 head dims per page and half head (a 16-key group never straddles
//               a page: page sizes are multiples of 16), 128-byte swizzle, 4-stage ring
//   warp 1      tcgen05.mma issuer: S = Q.K^T (128 x 64, 8 steps) into one of two tensor-memory
//               buffers; P.V (128 x 128, 4 steps, fresh accumulator per tile) into one of two
//               others, P read from shared memory where the softmax warps put it
//   warps 2-17  softmax / conversion: thread = one row and a quarter of the columns (four
//               warps per scheduler hide the tensor-memory, MUFU and ALU latencies).  Pass A: row
//               maxima straight from tensor memory (a row lives in one lane: no shuffles).
//               Pass B: weights, integer denominator, P -> shared memory (K-major, swizzled,
//               the A operand of P.V); then the P.V partial of the previous tile is rounded to
//               Q-format on the FP32 pipe (r = fma(v, 2^f, 1.5 * 2^23), raw bits summed in
//               32-bit registers, exponent screen, exact fix-up from tensor memory) while the
//               tensor core works on the next tile.
// KV splits are not handled here (the dispatcher sends them to attention_mma.cu: same bits).
// Every wait is bounded; on a time-out the CTA sets the status word and leaves.
#include <algorithm>
#include <cuda.h>

#include "attention_common.cuh"
#include "fxp_common.cuh"
#include "tc_common.cuh"
#include "gemm_tc_fast_common.cuh"

namespace fxpr {

static constexpr int kTcTileN = 64;            // keys per tile (attention.py:32-36)
static constexpr int kTcRows = 128;            // query rows per CTA = tensor-memory lanes
static constexpr int kTcColGroups = 4;         // softmax threads per row: each owns 64/4 keys and HD/4 output columns
static constexpr int kTcSoftWarps = 4 * kTcColGroups;
static constexpr int kTcFirstSoft = 2;         // warp 0: TMA producer, warp 1: MMA issuer
static constexpr int kTcThreads = (kTcFirstSoft + kTcSoftWarps) * 32;
static constexpr int kTcStages = 4;

struct TcAttnShape {
  int rows_per_token;      // GQA group size
  int tokens_per_block;    // 128 / rows_per_token
  int num_q_blocks;
  int page_size;
  int group_shift;         // log2 of the keys per TMA box: 6 when pages are multiples of 64 tokens, else 4
  int page_mask;           // page_size - 1 when the page size is a power of two, else 0
  uint32_t idesc_s, idesc_pv;
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z,
                                            int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// generic-proxy writes to shared memory become visible to the tensor core (async proxy)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ float ex2_approx_tc(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <typename T> __device__ __forceinline__ uint32_t pack2_tc(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2_tc<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2_tc<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Wait used by the 16 softmax warps: one lane polls and sleeps between probes, so that the
// waiting warps leave the issue slots to the two single-lane role warps that they wait for.
__device__ __forceinline__ bool warp_wait_relaxed(uint32_t bar, uint32_t parity, volatile int* abort_flag, int lane) {
  int ok = 1;
  if (lane == 0 && !mbar_try_wait(bar, parity)) {
    const long long t0 = clock64();
    int spins = 0;
    while (!mbar_try_wait(bar, parity)) {
      __nanosleep(40);
      if ((++spins & 63) == 0) {
        if (*abort_flag) { ok = 0; break; }
        if (clock64() - t0 > kWaitCycles) { *abort_flag = 1; ok = 0; break; }
      }
    }
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

template <typename T, int HD>
__global__ void __launch_bounds__(kTcThreads, 1)
attn_tc_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const AttnParams p, const TcAttnShape sh,
                       int32_t* status, const int zero /* always 0: keeps the side arrays in local memory */) {
  static_assert(HD == 128, "head size 128");
  constexpr int kQBytes = kTcRows * HD * 2;                // 32 KB: two 64-dim slabs of 128 rows x 128 B
  constexpr int kKBytes = kTcTileN * HD * 2;               // 16 KB: two slabs of 64 keys x 128 B
  constexpr int kStageBytes = 2 * kKBytes;                 // K then V
  constexpr int kPBytes = kTcRows * kTcTileN * 2;          // 16 KB: 128 rows x 128 B
  constexpr int kBarOffset = kQBytes + kTcStages * kStageBytes + 2 * kPBytes;
  constexpr int CG = kTcColGroups;
  constexpr int KT = kTcTileN / CG;                        // keys per softmax thread and tile
  constexpr int kHalfCols = HD / CG;                       // P.V columns per thread
  static_assert(KT == 16 && kHalfCols == 32, "one 16-column and one 32-column tensor-memory load per tile");
  constexpr uint32_t kColS = 0, kColPV = 128;              // tensor-memory columns: S[2] x 64, PV[2] x 128

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_s = smem_base, stage0 = smem_base + kQBytes, p_s0 = stage0 + kTcStages * kStageBytes;
  const uint32_t bar_base = smem_base + kBarOffset;
  // barriers: qfull | full[4] empty[4] | sfull[2] sfree[2] | pready[2] | pvfull[2] pvfree[2] | sync | qfree
  const uint32_t qfull = bar_base, full0 = bar_base + 8, empty0 = full0 + 8 * kTcStages;
  const uint32_t sfull0 = empty0 + 8 * kTcStages, sfree0 = sfull0 + 16, pready0 = sfree0 + 16;
  const uint32_t pvfull0 = pready0 + 16, pvfree0 = pvfull0 + 16, soft_bar = pvfree0 + 16;
  const uint32_t qfree = soft_bar + 8;
  constexpr int kMisc = 8 * (1 + 2 * kTcStages + 10 + 2);
  volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem_gen + kBarOffset + kMisc);
  volatile int* abort_flag = (volatile int*)(smem_gen + kBarOffset + kMisc + 8);
  float* rmax_s = (float*)(smem_gen + kBarOffset + kMisc + 16);                 // [CG][128]
  long long* den_s = (long long*)(smem_gen + kBarOffset + kMisc + 16 + 2048);   // [CG][128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- work items ---------------------------------------------------------------------
  // Persistent CTAs: CTA b takes the work items b, b + gridDim.x, ... of the padded space
  // (request, row block, KV head), later row blocks (more keys) first.  Every role walks the
  // same list and keeps its ring positions and barrier phases running from one item to the
  // next, so the producer fetches the next item's Q and first keys and the MMA warp starts its
  // scores while the softmax warps still convert and store the current item's output.
  const int hkv = p.num_kv_heads;
  const int G = sh.rows_per_token;
  const int items_per_req = sh.num_q_blocks * hkv;
  const int total_items = items_per_req * p.num_reqs;
  struct Item { int live, req, kvh, q_start, q_len, tok0, seq_len, ctx, t0, t1; };
  auto decode_item = [&](int w) -> Item {
    Item I;
    I.req = w / items_per_req;
    const int rem = w - I.req * items_per_req;
    const int qb = sh.num_q_blocks - 1 - rem / hkv;
    I.kvh = rem % hkv;
    I.q_start = p.qsl[I.req];
    I.q_len = p.qsl[I.req + 1] - I.q_start;
    I.tok0 = qb * sh.tokens_per_block;
    I.live = I.tok0 < I.q_len;
    I.seq_len = I.live ? p.seq_lens[I.req] : 0;
    I.ctx = I.seq_len - I.q_len;
    const int tok_end = min(I.q_len, I.tok0 + sh.tokens_per_block);
    const int hi_key = p.causal ? min(I.seq_len, I.ctx + tok_end) : I.seq_len;
    const int lo_key = p.window > 0 ? max(0, I.ctx + I.tok0 - p.window + 1) : 0;
    I.t0 = lo_key / kTcTileN;
    I.t1 = max(I.t0, (hi_key + kTcTileN - 1) / kTcTileN);
    return I;
  };

  if (threadIdx.x == 32) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  if (threadIdx.x == 0) {
    mbar_init(qfull, 1);
    mbar_init(qfree, 1);
    for (int s = 0; s < kTcStages; ++s) { mbar_init(full0 + 8u * s, 1); mbar_init(empty0 + 8u * s, 1); }
    for (int b = 0; b < 2; ++b) {
      mbar_init(sfull0 + 8u * b, 1); mbar_init(sfree0 + 8u * b, kTcSoftWarps);
      mbar_init(pready0 + 8u * b, kTcSoftWarps);
      mbar_init(pvfull0 + 8u * b, 1); mbar_init(pvfree0 + 8u * b, kTcSoftWarps);
    }
    mbar_init(soft_bar, kTcSoftWarps);
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

  if (warp == 0) {
    // ------------------------------ K / V producer (TMA) ------------------------------
    // One box per 16-token page piece and half head (2 KB).  Measured on a B200: an SM keeps
    // only ~15 bytes per clock of such pieces in flight, whether they are fetched as TMA
    // boxes, as 16-byte cp.async copies from two or four warps, or as both at once; that,
    // not the tensor core or the conversion work, bounds this kernel at 16-token pages
    // (48 KB per 128 x 64 tile over the two passes).  The boxes of a tile are issued from 16
    // lanes in one instruction: issued one by one they cost the issuing thread ~80 clocks
    // each.  Nothing is copied, and the block table is not read, past the end of the
    // sequence; V rows there are cleared by the MMA warp before P.V.
    int stage = 0; uint32_t phase = 1;
    uint32_t q_phase = 1;                                    // qfree: the first wait passes
    // Block-table entries are read 32 at a time (lane L: the 16-key group L of an 8-tile
    // block), one block ahead of their use, and handed round by shuffle.
    int page_shift = -1;
    for (int b = 4; b < 31; ++b) if ((1 << b) == sh.page_size) page_shift = b;
    for (int w = blockIdx.x; w < total_items; w += gridDim.x) {
    const Item I = decode_item(w);
    if (!I.live) continue;
    const int kvh = I.kvh, seq_len = I.seq_len, t0 = I.t0, t1 = I.t1;
    const int32_t* bt = p.block_table + (int64_t)I.req * p.bt_stride;
    // Q rows: box {64 dims, G heads, 128 / G tokens} -> row = token * G + head.  Tokens past
    // this request's (they belong to the next one, or lie beyond the tensor: zeros) are rows
    // whose every key is masked and that are never stored.  The buffer is free once the MMA
    // warp's last score MMA of the previous item has completed.
    if (!__all_sync(0xffffffffu, mbar_wait(qfree, q_phase, abort_flag))) goto producer_done;
    q_phase ^= 1;
    if (lane == 0) {
      mbar_expect_tx(qfull, kQBytes);
      tma_load_3d(q_s, &map_q, qfull, 0, kvh * G, I.q_start + I.tok0);
      tma_load_3d(q_s + kQBytes / 2, &map_q, qfull, 64, kvh * G, I.q_start + I.tok0);
    }
    __syncwarp();
    auto load_entries = [&](int tb) -> int {
      const int n = tb * kTcTileN + lane * 16;
      return (tb < t1 && n < seq_len) ? bt[page_shift >= 0 ? (n >> page_shift) : (n / sh.page_size)] : 0;
    };
    for (int pass = 0; pass < 2; ++pass) {
      int cur = load_entries(t0);
      for (int tb = t0; tb < t1; tb += 8) {
        const int nxt = load_entries(tb + 8);
        for (int tt = 0; tt < 8 && tb + tt < t1; ++tt) {
          const int t = tb + tt;
          if (!__all_sync(0xffffffffu, mbar_wait(empty0 + 8u * stage, phase, abort_flag))) goto producer_done;
          const uint32_t fb = full0 + 8u * stage;
          const uint32_t ks = stage0 + stage * kStageBytes;
          // boxes hold group_keys keys (16, or the whole tile when pages are multiples of 64
          // tokens); only groups that start inside the sequence are copied
          // (shifts and masks only: this single warp's loop latency is on the critical path)
          const int gs = sh.group_shift, gk = 1 << gs;
          int groups = (seq_len - t * kTcTileN + gk - 1) >> gs;
          groups = min(groups, kTcTileN >> gs);
          if (lane == 0) mbar_expect_tx(fb, (uint32_t)((groups << (gs + 8)) << pass));
          __syncwarp();
          // lane = group * 4 + {K low half, K high half, V low half, V high half}
          const int g = (lane >> 2) & 3, sel = lane & 3;
          const int blk = __shfl_sync(0xffffffffu, cur, tt * 4 + (gs == 4 ? g : 0));
          if (lane < 16 && g < groups && (pass || sel < 2)) {
            const int n = t * kTcTileN + (g << gs);
            const int slot = sh.page_mask ? (n & sh.page_mask) : (n % sh.page_size);
            const uint32_t dst = ks + (uint32_t)((sel >> 1) * kKBytes + (sel & 1) * 8192 + (g << (gs + 7)));
            tma_load_4d(dst, (sel >> 1) ? &map_v : &map_k, fb, (sel & 1) * 64, kvh, slot, blk);
          }
          __syncwarp();
          if (++stage == kTcStages) { stage = 0; phase ^= 1; }
        }
        cur = nxt;
      }
    }
    }
  producer_done:;
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ----------------------------------------
    // S_t = Q . K_t^T: both operands K-major (head dim contiguous), two 64-dim slabs
    auto issue_s = [&](int stage, int sbuf) {
      const uint32_t d = tmem_base + kColS + (uint32_t)(sbuf * 64);
      const uint64_t qd = make_smem_desc(q_s, 16, 1024);
      const uint64_t kd = make_smem_desc(stage0 + stage * kStageBytes, 16, 1024);
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t ao = (uint64_t)((kk >> 2) * (kQBytes / 2) + (kk & 3) * 32) >> 4;
          const uint64_t bo = (uint64_t)((kk >> 2) * (kKBytes / 2) + (kk & 3) * 32) >> 4;
          umma_f16(d, qd + ao, kd + bo, sh.idesc_s, kk ? 1u : 0u);
        }
        umma_commit(sfull0 + 8u * sbuf);
      }
      __syncwarp();
    };
    int stage = 0; uint32_t phase = 0;
    int it = 0;                                              // S tiles issued so far (all items, both passes)
    int jg = 0;                                              // P.V tiles issued so far (all items)
    uint32_t q_phase = 0;
    for (int w = blockIdx.x; w < total_items; w += gridDim.x) {
    const Item I = decode_item(w);
    if (!I.live) continue;
    const int seq_len = I.seq_len, t0 = I.t0, t1 = I.t1, n_tiles = I.t1 - I.t0;
    bool okq = mbar_wait(qfull, q_phase, abort_flag);
    if (!__all_sync(0xffffffffu, okq)) goto issuer_done;
    q_phase ^= 1;
    {
      // pass A: scores only
      for (int t = t0; t < t1; ++t, ++it) {
        const int sb = it & 1; const uint32_t sph = ((it >> 1) & 1) ^ 1;
        const bool a = mbar_wait(full0 + 8u * stage, phase, abort_flag);
        const bool b = mbar_wait(sfree0 + 8u * sb, sph, abort_flag);
        if (!__all_sync(0xffffffffu, a && b)) goto issuer_done;
        tc_fence_after();
        issue_s(stage, sb);
        if (lane == 0) umma_commit(empty0 + 8u * stage);
        __syncwarp();
        if (++stage == kTcStages) { stage = 0; phase ^= 1; }
      }
      // pass B: S runs one tile ahead of P.V
      int s_stage = stage; uint32_t s_phase = phase;         // ring position of the next S tile
      auto issue_s_next = [&]() -> bool {
        const int sb = it & 1; const uint32_t sph = ((it >> 1) & 1) ^ 1;
        const bool a = mbar_wait(full0 + 8u * s_stage, s_phase, abort_flag);
        const bool b = mbar_wait(sfree0 + 8u * sb, sph, abort_flag);
        if (!__all_sync(0xffffffffu, a && b)) return false;
        tc_fence_after();
        issue_s(s_stage, sb);
        ++it;
        if (++s_stage == kTcStages) { s_stage = 0; s_phase ^= 1; }
        return true;
      };
      if (n_tiles > 0 && !issue_s_next()) goto issuer_done;
      if (n_tiles <= 1 && lane == 0) umma_commit(qfree);     // the item's last score MMA is issued
      __syncwarp();
      for (int j = 0; j < n_tiles; ++j, ++jg) {
        if (j + 1 < n_tiles) {
          if (!issue_s_next()) goto issuer_done;
          if (j + 2 == n_tiles && lane == 0) umma_commit(qfree);
          __syncwarp();
        }
        const int b = jg & 1; const uint32_t ph = (jg >> 1) & 1;
        const bool r1 = mbar_wait(pready0 + 8u * b, ph, abort_flag);
        const bool r2 = mbar_wait(pvfree0 + 8u * b, ph ^ 1, abort_flag);
        if (!__all_sync(0xffffffffu, r1 && r2)) goto issuer_done;
        tc_fence_after();
        {
          // Keys at or past the end of the sequence: their V rows were not copied (or come
          // from slots nobody wrote) and 0 * NaN would poison the accumulator, so the rows
          // are cleared.  Only the last tile of a sequence has any.
          const int r0 = seq_len - (t0 + j) * kTcTileN;
          if (r0 < kTcTileN) {
            const uint32_t vs = stage0 + stage * kStageBytes + kKBytes;
            for (int idx = lane; idx < (kTcTileN - r0) * 16; idx += 32) {
              const int rr = r0 + (idx >> 4), cc = idx & 15;
              const uint32_t addr = vs + (uint32_t)((cc >> 3) * 8192 + rr * 128 + (cc & 7) * 16);
              asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0) : "memory");
            }
            fence_proxy_async_smem();
            __syncwarp();
          }
        }
        // PV_j = P_j . V_j: P K-major (keys contiguous), V MN-major (head dim contiguous)
        const uint32_t d = tmem_base + kColPV + (uint32_t)(b * HD);
        const uint64_t pd = make_smem_desc(p_s0 + b * kPBytes, 16, 1024);
        const uint64_t vd = make_smem_desc(stage0 + stage * kStageBytes + kKBytes, 8192, 1024);
        if (lane == 0) {
#pragma unroll
          for (int kk = 0; kk < kTcTileN / 16; ++kk)
            umma_f16(d, pd + (uint64_t)(kk * 2), vd + (uint64_t)(kk * 128), sh.idesc_pv, kk ? 1u : 0u);
          umma_commit(pvfull0 + 8u * b);
          umma_commit(empty0 + 8u * stage);
        }
        __syncwarp();
        if (++stage == kTcStages) { stage = 0; phase ^= 1; }
      }
    }
    }
  issuer_done:;
  } else if (warp >= kTcFirstSoft) {
    // ------------------------------ softmax / conversion warps ------------------------
    const int quarter = warp & 3;
    const int half = (warp - kTcFirstSoft) >> 2;                        // which quarter of the columns
    const int row = quarter * 32 + lane;                     // tensor-memory lane = query row
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    const float ninf = -__int_as_float(0x7f800000);
    const bool plain_scores = !(p.cap_log2 > 0.0f) && p.alibi == nullptr;
    const float magic = __uint_as_float(kMagicBits);
    uint32_t soft_phase = 0;
    bool ok = true;
    auto soft_sync = [&]() -> bool {                         // bounded barrier over these 8 warps
      __syncwarp();
      if (lane == 0) mbar_arrive(soft_bar);
      const bool done = warp_wait_relaxed(soft_bar, soft_phase, abort_flag, lane);
      soft_phase ^= 1;
      return done;
    };
    int it = 0;                                              // S tiles consumed so far (all items, both passes)
    int jg = 0;                                              // P.V tiles of the items before this one
    for (int w = blockIdx.x; w < total_items && ok; w += gridDim.x) {
    const Item I = decode_item(w);
    if (!I.live) continue;
    const int kvh = I.kvh, q_start = I.q_start, q_len = I.q_len, tok0 = I.tok0, seq_len = I.seq_len, ctx = I.ctx;
    const int t0 = I.t0, t1 = I.t1, n_tiles = I.t1 - I.t0;
    const int tok = tok0 + row / G, head = kvh * G + row % G;
    const bool valid = tok < q_len;
    const int pos = ctx + tok;
    const int kend = valid ? (p.causal ? min(seq_len, pos + 1) : seq_len) : 0;
    const int kbeg = valid ? (p.window > 0 ? max(0, pos - p.window + 1) : 0) : 0;
    const float slope = (p.alibi && valid) ? p.alibi[head] : 0.0f;
    // scores of this thread's 32 keys of tile t, in log2 space, masked (attention.py:103-121, 249-254)
    auto load_scores = [&](int it, int t, float (&s)[KT]) -> bool {
      const int sb = it & 1; const uint32_t sph = (it >> 1) & 1;
      if (!warp_wait_relaxed(sfull0 + 8u * sb, sph, abort_flag, lane)) return false;
      tc_fence_after();
      uint32_t v[KT];
      tmem_ld16(tmem_base + lane_sel + kColS + (uint32_t)(sb * 64 + half * KT), v);
      tmem_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sfree0 + 8u * sb);          // the buffer may take the tile after next
      const int n0 = t * kTcTileN + half * KT;
      if (plain_scores && n0 >= kbeg && n0 + KT <= kend) {
#pragma unroll
        for (int i = 0; i < KT; ++i) s[i] = __fmul_rn(__uint_as_float(v[i]), p.ss_log2);
      } else {
#pragma unroll
        for (int i = 0; i < KT; ++i) {
          const int n = n0 + i;
          float x = __fmul_rn(__uint_as_float(v[i]), p.ss_log2);
          if (p.cap_log2 > 0.0f) x = __fmul_rn(p.cap_log2, tanhf(__fdiv_rn(x, p.cap_log2)));
          if (p.alibi) x = __fadd_rn(x, __fmul_rn(slope, __fsub_rn((float)n, (float)pos)));
          s[i] = (n >= kbeg && n < kend) ? x : ninf;
        }
      }
      return true;
    };

    // =============================== pass A: row maxima ===============================
    float rmax = ninf;
    for (int t = t0; t < t1 && ok; ++t, ++it) {
      float s[KT];
      if (!load_scores(it, t, s)) { ok = false; break; }
      // max is exact and order-free: a tree keeps the dependency chain short
#pragma unroll
      for (int w = KT / 2; w > 0; w >>= 1)
#pragma unroll
        for (int i = 0; i < w; ++i) s[i] = fmaxf(s[i], s[i + w]);
      rmax = fmaxf(rmax, s[0]);
    }
    rmax_s[half * kTcRows + row] = rmax;
    if (ok && !soft_sync()) ok = false;
    float gmax = rmax_s[row];
#pragma unroll
    for (int c = 1; c < CG; ++c) gmax = fmaxf(gmax, rmax_s[c * kTcRows + row]);
    if (gmax == ninf) gmax = 0.0f;                           // rows without keys: exp2 gives 0, not NaN

    // =============================== pass B ===========================================
    uint32_t den32 = 0, den32b = 0;                         // two chains: integer adds commute
    uint32_t acc[kHalfCols];
#pragma unroll
    for (int i = 0; i < kHalfCols; ++i) acc[i] = 0;
    uint32_t corr_raw[kHalfCols];                            // rare path, local memory
    long long corr_q[kHalfCols];
    bool corr_used = false;

    // round the P.V partial of tile j (this thread's 64 columns) to Q-format and add it
    auto convert_pv = [&](int j) -> bool {                  // j counts over all items
      const int b = j & 1; const uint32_t ph = (j >> 1) & 1;
      if (!warp_wait_relaxed(pvfull0 + 8u * b, ph, abort_flag, lane)) return false;
      tc_fence_after();
      const uint32_t taddr = tmem_base + lane_sel + kColPV + (uint32_t)(b * HD + half * kHalfCols);
      uint32_t screen = 0, screen_b = 0;
      {
        uint32_t v[32];
        tmem_ld32(taddr, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const uint32_t ra = __float_as_uint(__fmaf_rn(__uint_as_float(v[i]), p.scale, magic));
          const uint32_t rb = __float_as_uint(__fmaf_rn(__uint_as_float(v[i + 1]), p.scale, magic));
          acc[i] += ra;
          acc[i + 1] += rb;
          screen |= ra ^ kExpBits;
          screen_b |= rb ^ kExpBits;
        }
      }
      if (__any_sync(0xffffffffu, ((screen | screen_b) >> 23) != 0)) {
        // some partial left the fast range: exact conversion of the offending elements
        if (!corr_used) {
#pragma unroll 1
          for (int z = 0; z < kHalfCols; ++z) { corr_raw[z + zero] = 0; corr_q[z + zero] = 0; }
          corr_used = true;
        }
        fixup_tile(taddr, kHalfCols, p.scale, p.int_bits, &corr_raw[zero], &corr_q[zero]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pvfree0 + 8u * b);
      return true;
    };

    for (int j = 0; j < n_tiles && ok; ++j, ++it) {
      const int t = t0 + j;
      float s[KT];
      if (!load_scores(it, t, s)) { ok = false; break; }
      // weights, integer denominator, P in the io dtype -> shared memory (A operand of P.V):
      // row = 128 bytes of 64 keys, 16-byte chunks XOR-swizzled with the row number
      const int b = (jg + j) & 1;
      const uint32_t prow = p_s0 + b * kPBytes + (uint32_t)row * 128u;
#pragma unroll
      for (int c = 0; c < KT / 8; ++c) {
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float s0 = s[c * 8 + e * 2], s1 = s[c * 8 + e * 2 + 1];
          const float w0 = (s0 == ninf) ? 0.0f : ex2_approx_tc(__fsub_rn(s0, gmax));
          const float w1 = (s1 == ninf) ? 0.0f : ex2_approx_tc(__fsub_rn(s1, gmax));
          den32 += __float_as_uint(__fmaf_rn(w0, p.scale, magic));
          den32b += __float_as_uint(__fmaf_rn(w1, p.scale, magic));
          pk[e] = pack2_tc<T>(w0, w1);
        }
        const uint32_t chunk = (uint32_t)(half * (KT / 8) + c);
        const uint32_t addr = prow + ((chunk ^ (uint32_t)(row & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]) : "memory");
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pready0 + 8u * b);
      if (j > 0 && !convert_pv(jg + j - 1)) { ok = false; break; }
    }
    if (ok && n_tiles > 0 && !convert_pv(jg + n_tiles - 1)) ok = false;
    jg += n_tiles;

    // =============================== output ===========================================
    // KT weights per tile went through the fast add in this thread
    const long long den_half = (long long)(int32_t)(den32 + den32b - (uint32_t)KT * (uint32_t)n_tiles * kMagicBits);
    den_s[half * kTcRows + row] = den_half;
    if (ok && !soft_sync()) ok = false;
    if (ok && valid) {
      long long dsum = den_s[row];
#pragma unroll
      for (int c = 1; c < CG; ++c) dsum += den_s[c * kTcRows + row];
      const float dn = fmaxf(fixed_to_float<long long>(wrap_to_bits(dsum, p.int_bits), p.inv_scale), 1.0e-6f);
      T* op = (T*)p.o + (int64_t)(q_start + tok) * p.o_st + (int64_t)head * p.o_sh + half * kHalfCols;
      const uint32_t bias_bits = (uint32_t)n_tiles * kMagicBits;
#pragma unroll
      for (int g8 = 0; g8 < kHalfCols / 8; ++g8) {
        alignas(16) T out[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = g8 * 8 + i;
          uint32_t raw = acc[c] - bias_bits;
          float num;
          if (corr_used) {
            raw -= corr_raw[c + zero];
            const long long tot = (long long)(int32_t)raw + corr_q[c + zero];
            num = fixed_to_float<long long>(wrap_to_bits(tot, p.int_bits), p.inv_scale);
          } else {
            // the sum fits 32 bits: the same value through the cheaper 32-bit conversion
            num = fixed_to_float<int>((int)raw, p.inv_scale);
          }
          out[i] = from_f32<T>(__fdiv_rn(num, dn));
        }
        *reinterpret_cast<uint4*>(op + g8 * 8) = *reinterpret_cast<const uint4*>(out);
      }
    }
    }
  }

  // ------------------------------ teardown ----------------------------------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // let copies that are still in flight land before shared memory is released
    const long long tw = clock64();
    while (clock64() - tw < 200000) { __nanosleep(1000); }
    if (threadIdx.x == 0 && status) atomicExch(status, FXPR_ERR_TIMEOUT);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFnA)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFnA encode_fn() {
  static EncodeTiledFnA fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFnA)ptr;
  }
  return fn;
}

// The prefill kernel takes head size 128, bf16/fp16, 32- or 64-bit sums with at most 16
// fraction bits, no KV split, a sequence short enough for the 32-bit fast sums, and strides
// a tensor map can express (multiples of 16 bytes, below 2^40).
bool attention_tc_supported(const AttnParams& p, int dtype, int max_query_len, bool force_exact) {
  if (force_exact || p.num_splits != 1) return false;
  if (dtype != FXPR_F16 && dtype != FXPR_BF16) return false;
  if (p.head_dim != 128 || p.page_size % 16 != 0) return false;
  const int G = p.num_heads / p.num_kv_heads;
  if (G != 1 && G != 2 && G != 4 && G != 8 && G != 16) return false;
  if ((int64_t)max_query_len * G <= 16) return false;      // decode shapes: attention_mma.cu
  if (p.int_bits != 32 && p.int_bits != 64) return false;
  if (p.scale > 65536.0f) return false;
  const int64_t max_keys = p.bt_stride * (int64_t)p.page_size;
  if ((max_keys + kTcTileN - 1) / kTcTileN > 500) return false;
  const int64_t strides[] = {p.q_st, p.q_sh, p.o_st, p.o_sh, p.kv_sblock, p.kv_sslot, p.kv_shead};
  for (int64_t st : strides) if (st % 8 != 0 || st <= 0 || st >= (1ll << 38)) return false;
  if (((uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v | (uintptr_t)p.o) & 15) return false;
  if (p.num_reqs > 65535) return false;
  return encode_fn() != nullptr;
}

int attention_tc(const AttnParams& p, int dtype, int max_query_len, int32_t* status, cudaStream_t s) {
  EncodeTiledFnA fn = encode_fn();
  if (!fn) return FXPR_ERR_CUDA;
  const int G = p.num_heads / p.num_kv_heads;
  TcAttnShape sh;
  sh.rows_per_token = G;
  sh.tokens_per_block = kTcRows / G;
  sh.num_q_blocks = (max_query_len + sh.tokens_per_block - 1) / sh.tokens_per_block;
  sh.page_size = p.page_size;
  sh.group_shift = (p.page_size % 64 == 0) ? 6 : 4;
  sh.page_mask = (p.page_size & (p.page_size - 1)) == 0 ? p.page_size - 1 : 0;
  const int fmt = dtype == FXPR_BF16 ? 1 : 0;
  sh.idesc_s = make_idesc(fmt, 0, kTcTileN, kTcRows);
  sh.idesc_pv = make_idesc(fmt, 1, p.head_dim, kTcRows);
  if ((int64_t)sh.num_q_blocks * p.num_kv_heads > 0x7fffffffLL) return FXPR_ERR_UNSUPPORTED;

  const CUtensorMapDataType dt = dtype == FXPR_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap mq, mk, mv;
  {
    // q [tokens, heads, dims]
    cuuint64_t dims[3] = {(cuuint64_t)p.head_dim, (cuuint64_t)p.num_heads, (cuuint64_t)p.total_q};
    cuuint64_t strides[2] = {(cuuint64_t)p.q_sh * 2, (cuuint64_t)p.q_st * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)sh.tokens_per_block};
    cuuint32_t es[3] = {1, 1, 1};
    if (fn(&mq, dt, 3, const_cast<void*>(p.q), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      set_last_error("cuTensorMapEncodeTiled(Q)", cudaErrorInvalidValue);
      return FXPR_ERR_CUDA;
    }
  }
  for (int which = 0; which < 2; ++which) {
    // cache plane [blocks, slots, kv heads, dims]; the number of blocks is not known here and
    // only bounds the coordinates, which come from the block table
    cuuint64_t dims[4] = {(cuuint64_t)p.head_dim, (cuuint64_t)p.num_kv_heads, (cuuint64_t)p.page_size,
                          (cuuint64_t)1 << 31};
    cuuint64_t strides[3] = {(cuuint64_t)p.kv_shead * 2, (cuuint64_t)p.kv_sslot * 2, (cuuint64_t)p.kv_sblock * 2};
    cuuint32_t box[4] = {64, 1, (cuuint32_t)(1 << sh.group_shift), 1};
    cuuint32_t es[4] = {1, 1, 1, 1};
    if (fn(which ? &mv : &mk, dt, 4, const_cast<void*>(which ? p.v : p.k), dims, strides, box, es,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
      set_last_error("cuTensorMapEncodeTiled(KV)", cudaErrorInvalidValue);
      return FXPR_ERR_CUDA;
    }
  }

  constexpr int kSmem = kTcRows * 128 * 2 + kTcStages * 2 * kTcTileN * 128 * 2 + 2 * kTcRows * kTcTileN * 2 +
                        8 * (1 + 2 * kTcStages + 10 + 2) + 16 + 2048 + 4096 + 1024;
  // persistent CTAs, one per SM (204 KB of shared memory each), walking the padded item list
  int dev_now = 0, sms = 0;
  cudaGetDevice(&dev_now);
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev_now) != cudaSuccess || sms < 1) sms = 148;
  const int64_t total_items = (int64_t)sh.num_q_blocks * p.num_kv_heads * p.num_reqs;
  if (total_items > 0x7fffffffLL) return FXPR_ERR_UNSUPPORTED;
  dim3 grid((unsigned)std::min<int64_t>(total_items, sms), 1, 1);
#define FXPR_TC_ATTN(TT)                                                                              \
  do {                                                                                                \
    auto k = attn_tc_prefill_kernel<TT, 128>;                                                         \
    static bool attr_done_dev[64] = {};                                                               \
    int dev_id = 0;                                                                                   \
    cudaGetDevice(&dev_id);                                                                           \
    if (!attr_done_dev[dev_id & 63]) {                                                                \
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);    \
      if (e != cudaSuccess) { set_last_error("attention_tc smem attribute", e); return FXPR_ERR_CUDA; } \
      attr_done_dev[dev_id & 63] = true;                                                              \
    }                                                                                                 \
    k<<<grid, kTcThreads, kSmem, s>>>(mq, mk, mv, p, sh, status, 0);                                  \
  } while (0)
  if (dtype == FXPR_BF16) FXPR_TC_ATTN(__nv_bfloat16);
  else FXPR_TC_ATTN(__half);
#undef FXPR_TC_ATTN
  return check_launch("attention_tc");
}

}  // namespace fxpr

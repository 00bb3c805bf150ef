// Kernel and launcher of the tensor-core attention route (included by attention_mma.cu).
//
// Template: T = io dtype, HD = head size (64 | 128), NW = warps per CTA (16 query rows
// each), STASH = keep this CTA's fp32 scores in shared memory between the two passes
// (decode), ACC64 = 64-bit integer accumulators, FAST = second pass with magic-number
// rounding on the FP32 pipe and 32-bit wrap-around accumulators (same bits, see
// attention_mma_pass_b_fast.inl).
// Grid: x = KV split (= rank in the cluster), y = q_block * num_kv_heads + kv_head,
// z = request.

template <typename T, int HD, int NW, bool STASH, bool ACC64, bool FAST>
__global__ void __launch_bounds__(NW * 32, FAST ? 3 : 1)
attn_mma_kernel(const AttnParams p, const MmaAttnShape sh) {
  constexpr int RC = HD / 8;                       // 16-byte chunks per K/V/Q row
  constexpr int BM = 16 * NW;                      // query rows per CTA
  constexpr int NT = NW * 32;
  constexpr int kTileBytes = kTileN * HD * 2;
  constexpr int kStageBytes = STASH ? kTileBytes : 2 * kTileBytes;   // K | K+V
  constexpr int NSTAGE = STASH ? 3 : 2;
  using AccT = typename IntOf<ACC64 ? 64 : 32>::type;

  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* q_s = smem;                                            // BM x HD io elements
  uint8_t* stage_s = q_s + BM * HD * 2;                           // NSTAGE stages
  float* rmax_s = reinterpret_cast<float*>(stage_s + NSTAGE * kStageBytes);       // [BM]
  long long* den_s = reinterpret_cast<long long*>(rmax_s + BM);                   // [BM]
  float* stash_s = reinterpret_cast<float*>(den_s + BM);                          // decode only
  long long* wv_s = reinterpret_cast<long long*>(stage_s);        // [BM][HD], reuses the stages
  pdl_launch_dependents();
  pdl_wait();

  cg::cluster_group cluster = cg::this_cluster();
  const int S = gridDim.x;
  const int rank = blockIdx.x;
  const int hkv = p.num_kv_heads;
  const int qb = blockIdx.y / hkv, kvh = blockIdx.y % hkv;
  const int req = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  const int q_start = p.qsl[req], q_len = p.qsl[req + 1] - q_start;
  const int G = sh.rows_per_token;
  const int tok0 = qb * sh.tokens_per_block;
  if (tok0 >= q_len) return;                       // same decision in every CTA of the cluster
  const int seq_len = p.seq_lens[req];
  const int ctx = seq_len - q_len;
  const int tok_end = min(q_len, tok0 + sh.tokens_per_block);
  const int32_t* bt = p.block_table + (int64_t)req * p.bt_stride;

  // ---- key range of this row block, dealt to the cluster ranks in whole tiles ----------
  const int hi_key = p.causal ? min(seq_len, ctx + tok_end) : seq_len;
  const int lo_key = p.window > 0 ? max(0, ctx + tok0 - p.window + 1) : 0;
  const int t_first = lo_key / kTileN;
  const int t_last = max(t_first, (hi_key + kTileN - 1) / kTileN);
  const int per_rank = (t_last - t_first + S - 1) / S;
  const int t0 = min(t_last, t_first + rank * per_rank);
  const int t1 = min(t_last, t0 + per_rank);

  // the stash is sized from the block table's width on the host; never index past it
  if (STASH && per_rank * kTileN > sh.stash_keys) {
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, FXPR_ERR_SCRATCH);
    return;
  }

  // ---- the two rows this thread owns in the MMA accumulator layout ------------------
  int r_tok[2], r_head[2], r_kend[2], r_kbeg[2]; bool r_valid[2]; float r_slope[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + g + 8 * h;
    r_tok[h] = tok0 + r / G;
    r_head[h] = kvh * G + r % G;
    r_valid[h] = r_tok[h] < q_len;
    const int pos = ctx + r_tok[h];
    r_kend[h] = p.causal ? min(seq_len, pos + 1) : seq_len;
    r_kbeg[h] = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    r_slope[h] = (p.alibi && r_valid[h]) ? p.alibi[r_head[h]] : 0.0f;
    if (!r_valid[h]) { r_kend[h] = 0; r_kbeg[h] = 0; }
  }

  // ---- Q rows -> shared memory (zero rows beyond the block's tokens) ----------------------
  for (int idx = threadIdx.x; idx < BM * RC; idx += NT) {
    const int r = idx / RC, c = idx % RC;
    const int tok = tok0 + r / G;
    const bool v = tok < q_len;
    const T* src = (const T*)p.q + (int64_t)(q_start + (v ? tok : 0)) * p.q_st +
                   (int64_t)(kvh * G + r % G) * p.q_sh + c * 8;
    cp_async16(smem_addr(q_s) + swz<RC>(r, c), src, v);
  }
  cp_async_commit();

  const T* kbase = (const T*)p.k + (int64_t)kvh * p.kv_shead;
  const T* vbase = (const T*)p.v + (int64_t)kvh * p.kv_shead;

  // stage one 64-key tile of K and/or V: 16-byte cp.async per (key, chunk); rows past the
  // sequence are zero-filled and never touch the block table.  The block table is looked
  // up once per 16 keys and the four page offsets stay in scalars (a dynamically indexed
  // array would live in local memory).
  auto issue_kv = [&](int t, uint32_t dst_k, uint32_t dst_v, bool want_k, bool want_v) {
    auto page_of = [&](int q4) -> int64_t {
      const int n = t * kTileN + q4 * 16;
      return (n < seq_len) ? (int64_t)bt[n / p.page_size] * p.kv_sblock +
                                 (int64_t)(n % p.page_size) * p.kv_sslot
                           : 0;
    };
    const int64_t po0 = page_of(0), po1 = page_of(1), po2 = page_of(2), po3 = page_of(3);
#pragma unroll
    for (int it = 0; it < kTileN * RC / NT; ++it) {
      const int idx = threadIdx.x + it * NT;
      const int key = idx / RC, c = idx % RC;
      const bool v = t * kTileN + key < seq_len;
      const int q4 = key >> 4;
      const int64_t po = q4 == 0 ? po0 : (q4 == 1 ? po1 : (q4 == 2 ? po2 : po3));
      const int64_t off = v ? po + (int64_t)(key & 15) * p.kv_sslot + c * 8 : 0;
      const uint32_t so = swz<RC>(key, c);
      if (want_k) cp_async16(dst_k + so, kbase + off, v);
      if (want_v) cp_async16(dst_v + so, vbase + off, v);
    }
  };
  auto issue_tile = [&](const T* base, int t, uint32_t dst) {
    if (base == kbase) issue_kv(t, dst, 0, true, false);
    else issue_kv(t, 0, dst, false, true);
  };

  const uint32_t stage0 = smem_addr(stage_s);
  const uint32_t qs_addr = smem_addr(q_s);
  const float ninf = -__int_as_float(0x7f800000);

  // ldmatrix addresses: the XOR swizzle only depends on lane bits, so each fragment address is
  // a per-lane base (a handful of variants selected by compile-time loop indices) plus a
  // compile-time offset; nothing is recomputed per load.
  const int r7 = lane & 7, l15 = lane & 15, c1 = lane >> 4;
  uint32_t kbase_l[2];                              // K rows j*8 + r7, chunk (kk2*4 + (lane>>3)) ^ r7
  {
    const int lo = (lane >> 3) ^ (r7 & 3), hi = r7 >> 2;
    const int base = (r7 * RC + lo) * 16;
    kbase_l[0] = (uint32_t)(base + (hi ? 64 : 0));  // kk2 even
    kbase_l[1] = (uint32_t)(base - (hi ? 64 : 0));  // kk2 odd
  }
  uint32_t qbase_l[2][2];                           // Q rows warp*16 + l15, chunk (kk2*4 + 2a + c1) ^ r7
#pragma unroll
  for (int par = 0; par < 2; ++par)
#pragma unroll
    for (int a2 = 0; a2 < 2; ++a2) {
      const int lo = c1 ^ (r7 & 1), mid = a2 ^ ((r7 >> 1) & 1), hi = r7 >> 2;
      qbase_l[par][a2] = (uint32_t)(((warp * 16 + l15) * RC + lo + 2 * mid) * 16 + (hi ? (par ? -64 : 64) : 0));
    }
  uint32_t vbase_l[4];                              // V rows kk*16 + l15, chunk (jn2*2 + c1) ^ r7
#pragma unroll
  for (int q = 0; q < 4; ++q)
    vbase_l[q] = (uint32_t)((l15 * RC + (c1 ^ (r7 & 1))) * 16 + ((q ^ (r7 >> 1)) * 32));
  // address of the V fragment for k-step kk (16 keys) and head-dim pair jn2
  auto v_frag = [&](uint32_t v_addr, int kk, int jn2) -> uint32_t {
    return v_addr + vbase_l[jn2 & 3] + (uint32_t)(kk * 16 * RC * 16 + (jn2 >> 2) * 128);
  };

  const bool plain_scores = !(p.cap_log2 > 0.0f) && p.alibi == nullptr;

  // scores of one tile for this warp's 16 rows: s[j][e], j = 8-key group, e = C-fragment slot
  auto qk_tile = [&](uint32_t k_addr, int t, float (&s)[8][4]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
#pragma unroll
    for (int kk2 = 0; kk2 < HD / 32; ++kk2) {
      uint32_t a0[4], a1[4];
      ldsm_x4(qs_addr + qbase_l[kk2 & 1][0] + kk2 * 64, a0[0], a0[1], a0[2], a0[3]);
      ldsm_x4(qs_addr + qbase_l[kk2 & 1][1] + kk2 * 64, a1[0], a1[1], a1[2], a1[3]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(k_addr + kbase_l[kk2 & 1] + (uint32_t)(j * 8 * RC * 16 + kk2 * 64), b0, b1, b2, b3);
        mma16816<T>(s[j], a0, b0, b1);
        mma16816<T>(s[j], a1, b2, b3);
      }
    }
    // scale to log2 space, soft-cap, ALiBi, masks (attention.py:103-121, 249-254).  A tile
    // that lies inside the key range of all 16 rows of the warp needs the scale only.
    const int tile_lo = t * kTileN, tile_hi = tile_lo + kTileN;
    const bool inside = tile_lo >= max(r_kbeg[0], r_kbeg[1]) && tile_hi <= min(r_kend[0], r_kend[1]);
    if (plain_scores && __all_sync(0xffffffffu, inside)) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = __fmul_rn(s[j][e], p.ss_log2);
      return;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const int n = t * kTileN + j * 8 + 2 * t4 + (e & 1);
        float v = __fmul_rn(s[j][e], p.ss_log2);
        if (p.cap_log2 > 0.0f) v = __fmul_rn(p.cap_log2, tanhf(__fdiv_rn(v, p.cap_log2)));
        if (p.alibi) v = __fadd_rn(v, __fmul_rn(r_slope[h], __fsub_rn((float)n, (float)(ctx + r_tok[h]))));
        s[j][e] = (n >= r_kbeg[h] && n < r_kend[h]) ? v : ninf;
      }
  };

  const int srows = sh.stash_rows;                 // rows kept in the stash: <= 8, or 16
  const int slanes = srows <= 8 ? 4 * srows : 32;
  const int svals = srows <= 8 ? 2 : 4;

#include "attention_mma_passes.inl"
}

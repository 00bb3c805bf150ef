// Decode kernel of the tensor-core attention route: at most 16 query rows per KV head
// ((tokens of the step) x (GQA group)), so one 16-row MMA tile per CTA.  The CTA's NW
// warps COOPERATE on every 64-key tile instead of owning tiles:
//   pass A  warp w computes Q.K^T for keys [64/NW * w, ...) of the tile, keeps the row
//           maxima and parks the fp32 scores in the shared-memory stash;
//   pass B  every warp rebuilds all 64 weights of the tile from the stash (the integer
//           denominator is taken by the warp that owns the keys), and computes P.V for its
//           own HD/NW slice of the head dimension over all 64 keys -- the same four
//           m16n8k16 k-steps in the same order as the prefill kernel, so a token's bits do
//           not depend on which kernel served it.
// K is streamed once (pass A), V once (pass B); KV splits are cluster ranks merged through
// distributed shared memory exactly as in attn_mma_kernel.

// ROWS8: at most 8 of the 16 tile rows are real (e.g. one token x GQA group of 4): the
// second half of every accumulator fragment is known to be masked and is skipped.
template <typename T, int HD, int NW, bool ACC64, bool ROWS8, int NSTAGE = 2, int MINB = 4>
__global__ void __launch_bounds__(NW * 32, MINB)
attn_decode_kernel(const AttnParams p, const MmaAttnShape sh) {
  constexpr int RC = HD / 8;
  constexpr int NT = NW * 32;
  constexpr int kTileBytes = kTileN * HD * 2;
  constexpr int JW = 8 / NW;                       // 8-key groups per warp in pass A
  constexpr int DW = HD / 8 / NW;                  // 8-wide head-dim groups per warp in pass B
  static_assert((NW == 2 || NW == 4 || NW == 8) && (HD / 8 / NW) % 2 == 0, "warps must divide the 8 key groups and the HD/16 pairs");
  constexpr int NE = ROWS8 ? 2 : 4;                // live slots of a C fragment
  constexpr int NH = ROWS8 ? 1 : 2;                // live row halves
  using AccT = typename IntOf<ACC64 ? 64 : 32>::type;

  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int QR = ROWS8 ? 8 : 16;               // Q rows kept in shared memory (rows 8..15 of the MMA tile are zero registers)
  uint8_t* q_s = smem;                                            // QR x HD
  uint8_t* stage_s = q_s + QR * HD * 2;
  float* rmax_s = reinterpret_cast<float*>(stage_s + NSTAGE * kTileBytes);        // [NW][16]
  long long* den_s = reinterpret_cast<long long*>(rmax_s + NW * 16);              // [NW][16]
  float* stash_s = reinterpret_cast<float*>(den_s + NW * 16);
  long long* wv_s = reinterpret_cast<long long*>(stage_s);        // [16][HD], reuses the stages

  pdl_launch_dependents();
  pdl_wait();
  cg::cluster_group cluster = cg::this_cluster();
  const int S = gridDim.x, rank = blockIdx.x;
  const int hkv = p.num_kv_heads;
  const int qb = blockIdx.y / hkv, kvh = blockIdx.y % hkv;
  const int req = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  const int q_start = p.qsl[req], q_len = p.qsl[req + 1] - q_start;
  const int G = sh.rows_per_token;
  const int tok0 = qb * sh.tokens_per_block;
  if (tok0 >= q_len) return;
  const int seq_len = p.seq_lens[req];
  const int ctx = seq_len - q_len;
  const int tok_end = min(q_len, tok0 + sh.tokens_per_block);
  const int32_t* bt = p.block_table + (int64_t)req * p.bt_stride;

  const int hi_key = p.causal ? min(seq_len, ctx + tok_end) : seq_len;
  const int lo_key = p.window > 0 ? max(0, ctx + tok0 - p.window + 1) : 0;
  const int t_first = lo_key / kTileN;
  const int t_last = max(t_first, (hi_key + kTileN - 1) / kTileN);
  const int per_rank = (t_last - t_first + S - 1) / S;
  const int t0 = min(t_last, t_first + rank * per_rank);
  const int t1 = min(t_last, t0 + per_rank);
  if (per_rank * kTileN > sh.stash_keys) {          // the host sizes the stash from the block-table width
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, FXPR_ERR_SCRATCH);
    return;                                          // the same decision in every CTA of the cluster
  }

  int r_tok[2], r_kend[2], r_kbeg[2]; float r_slope[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = g + 8 * h;
    r_tok[h] = tok0 + r / G;
    const bool valid = r_tok[h] < q_len;
    const int pos = ctx + r_tok[h];
    r_kend[h] = valid ? (p.causal ? min(seq_len, pos + 1) : seq_len) : 0;
    r_kbeg[h] = valid ? (p.window > 0 ? max(0, pos - p.window + 1) : 0) : 0;
    r_slope[h] = (p.alibi && valid) ? p.alibi[kvh * G + r % G] : 0.0f;
  }

  for (int idx = threadIdx.x; idx < QR * RC; idx += NT) {
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
  // Every warp stages exactly the shared-memory bytes it will read itself, so the main loops
  // need no CTA-wide barrier: a warp waits for its own cp.async groups and runs ahead of (or
  // behind) its siblings.  Pass A: warp w reads keys [16w, 16w+16) of a tile (all of the head
  // dimension) -- one 16-key page group, one block-table entry.  Pass B: warp w reads all 64
  // keys but only its HD/NW slice of the head dimension.  The tile layout in shared memory
  // (64 rows x RC chunks, XOR swizzle) is the same in both passes.  Rows past the sequence
  // are zero-filled and never touch the block table.
  static_assert(NW == 4, "one 16-key page group per warp in pass A");
  const int pshift = sh.page_shift;
  auto page_offset = [&](int n) -> int64_t {         // element offset of key n's row (head 0)
    const int blk = pshift >= 0 ? (n >> pshift) : n / p.page_size;
    const int slot = pshift >= 0 ? (n & (p.page_size - 1)) : n % p.page_size;
    return (int64_t)bt[blk] * p.kv_sblock + (int64_t)slot * p.kv_sslot;
  };
  constexpr int KCP = 16 * RC / 32;                  // copies per lane: 16 keys x RC chunks
  const int ka_c = lane % RC, ka_key0 = lane / RC;   // pass A: chunk column, first key (step 32 / RC)
  auto issue_k = [&](int t, uint32_t dst) {
    const int n0 = t * kTileN + warp * 16;
    const int n_left = seq_len - n0;                 // keys of this warp's group that exist
    const int64_t off = n_left > 0 ? page_offset(n0) : 0;
#pragma unroll
    for (int it = 0; it < KCP; ++it) {
      const int key = ka_key0 + it * (32 / RC);
      const bool v = key < n_left;
      const T* src = v ? kbase + off + (int64_t)key * p.kv_sslot + ka_c * 8 : kbase;
      cp_async16(dst + swz<RC>(warp * 16 + key, ka_c), src, v);
    }
  };
  constexpr int WC = RC / NW;                        // chunk columns per warp in pass B
  constexpr int VCP = kTileN * WC / 32;              // copies per lane
  const int vb_c = warp * WC + lane % WC, vb_key0 = lane / WC;
  auto issue_v = [&](int t, uint32_t dst) {
    int64_t my_off = 0;
    if (lane < 4) {
      const int n = t * kTileN + lane * 16;
      if (n < seq_len) my_off = page_offset(n);
    }
    int64_t page_off[4];
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) page_off[q4] = __shfl_sync(0xffffffffu, my_off, q4);
    const int n_left = seq_len - t * kTileN;
#pragma unroll
    for (int it = 0; it < VCP; ++it) {
      const int key = vb_key0 + it * (32 / WC);      // (32 / WC) divides 16: it selects the page group statically
      const bool v = key < n_left;
      const T* src = v ? vbase + page_off[(it * (32 / WC)) >> 4] + (int64_t)(key & 15) * p.kv_sslot + vb_c * 8 : vbase;
      cp_async16(dst + swz<RC>(key, vb_c), src, v);
    }
  };

  const uint32_t stage0 = smem_addr(stage_s);
  const uint32_t qs_addr = smem_addr(q_s);
  const float ninf = -__int_as_float(0x7f800000);
  const int srows = sh.stash_rows;
  const int slanes = srows <= 8 ? 4 * srows : 32;
  const int svals = srows <= 8 ? 2 : 4;
  const bool small_q = p.int_bits >= 32 && p.scale <= 16777216.0f;   // Q(w) <= 2^24 per key, 64 keys per tile

  // =============================== pass A =============================================
  float rmax[2] = {ninf, ninf};
  {
    cp_async_wait<0>();
    __syncthreads();                                 // Q is in shared memory for every warp
    int issued = t0;
#pragma unroll 1
    for (int s = 0; s < NSTAGE - 1; ++s) {
      if (issued < t1) { issue_k(issued, stage0 + (issued - t0) % NSTAGE * kTileBytes); ++issued; }
      cp_async_commit();
    }
#pragma unroll 1
    for (int t = t0; t < t1; ++t) {
      cp_async_wait<NSTAGE - 2>();
      __syncwarp();                                  // this warp's rows of tile t landed; its rows of t-1 are free
      if (issued < t1) { issue_k(issued, stage0 + (issued - t0) % NSTAGE * kTileBytes); ++issued; }
      cp_async_commit();
      const uint32_t k_addr = stage0 + (t - t0) % NSTAGE * kTileBytes;
      float s[JW][4];
#pragma unroll
      for (int jj = 0; jj < JW; ++jj) { s[jj][0] = s[jj][1] = s[jj][2] = s[jj][3] = 0.0f; }
#pragma unroll
      for (int kk2 = 0; kk2 < HD / 32; ++kk2) {
        uint32_t a0[4], a1[4];
        if (ROWS8) {
          // eight live rows: one load brings rows 0..7 of four 8-wide k chunks
          ldsm_x4(qs_addr + swz<RC>(lane & 7, kk2 * 4 + (lane >> 3)), a0[0], a0[2], a1[0], a1[2]);
          a0[1] = a0[3] = a1[1] = a1[3] = 0u;
        } else {
          ldsm_x4(qs_addr + swz<RC>(lane & 15, kk2 * 4 + (lane >> 4)), a0[0], a0[1], a0[2], a0[3]);
          ldsm_x4(qs_addr + swz<RC>(lane & 15, kk2 * 4 + 2 + (lane >> 4)), a1[0], a1[1], a1[2], a1[3]);
        }
#pragma unroll
        for (int jj = 0; jj < JW; ++jj) {
          const int j = warp * JW + jj;
          uint32_t b0, b1, b2, b3;
          ldsm_x4(k_addr + swz<RC>(j * 8 + (lane & 7), kk2 * 4 + (lane >> 3)), b0, b1, b2, b3);
          mma16816<T>(s[jj], a0, b0, b1);
          mma16816<T>(s[jj], a1, b2, b3);
        }
      }
#pragma unroll
      for (int jj = 0; jj < JW; ++jj) {
        const int j = warp * JW + jj;
#pragma unroll
        for (int e = 0; e < NE; ++e) {
          const int h = e >> 1;
          const int n = t * kTileN + j * 8 + 2 * t4 + (e & 1);
          float v = __fmul_rn(s[jj][e], p.ss_log2);
          if (p.cap_log2 > 0.0f) v = __fmul_rn(p.cap_log2, tanhf(__fdiv_rn(v, p.cap_log2)));
          if (p.alibi) v = __fadd_rn(v, __fmul_rn(r_slope[h], __fsub_rn((float)n, (float)(ctx + r_tok[h]))));
          s[jj][e] = (n >= r_kbeg[h] && n < r_kend[h]) ? v : ninf;
        }
        rmax[0] = fmaxf(rmax[0], fmaxf(s[jj][0], s[jj][1]));
        if (!ROWS8) rmax[1] = fmaxf(rmax[1], fmaxf(s[jj][2], s[jj][3]));
        if (lane < slanes) {
          float* d = stash_s + ((size_t)((t - t0) * 8 + j) * slanes + lane) * svals;
          *reinterpret_cast<float2*>(d) = make_float2(s[jj][0], s[jj][1]);
          if (!ROWS8) *reinterpret_cast<float2*>(d + 2) = make_float2(s[jj][2], s[jj][3]);
        }
      }
    }
    cp_async_wait<0>();
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 1));
    rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 2));
    if (t4 == 0) rmax_s[warp * 16 + g + 8 * h] = rmax[h];
  }
  // Pass B's first V tiles are requested now, so their latency overlaps the cluster-wide
  // exchange of the maxima (every warp is done with pass A's stages after this barrier).
  __syncthreads();
  int issued_b = t0;
#pragma unroll 1
  for (int s = 0; s < NSTAGE - 1; ++s) {
    if (issued_b < t1) { issue_v(issued_b, stage0 + (issued_b - t0) % NSTAGE * kTileBytes); ++issued_b; }
    cp_async_commit();
  }
  cluster.sync();                                    // also orders the stash writes before pass B
  float gmax[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float m = ninf;
    for (int r = 0; r < S; ++r) {
      const float* rm = cluster.map_shared_rank(rmax_s, r);
#pragma unroll
      for (int w = 0; w < NW; ++w) m = fmaxf(m, rm[w * 16 + g + 8 * h]);
    }
    gmax[h] = (m == ninf) ? 0.0f : m;
  }

  // =============================== pass B =============================================
  long long den[2] = {0, 0};
  AccT acc[DW][4];
#pragma unroll
  for (int j = 0; j < DW; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0; }
  {
    int issued = issued_b;
#pragma unroll 1
    for (int t = t0; t < t1; ++t) {
      cp_async_wait<NSTAGE - 2>();
      __syncwarp();
      if (issued < t1) { issue_v(issued, stage0 + (issued - t0) % NSTAGE * kTileBytes); ++issued; }
      cp_async_commit();
      const uint32_t v_addr = stage0 + (t - t0) % NSTAGE * kTileBytes;
      uint32_t pa[4][4];
      uint32_t den_tile[2] = {0u, 0u};                 // w <= 1, so a tile's Q(w) sum fits 32 bits (f <= 24)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float sv[4] = {ninf, ninf, ninf, ninf};
        if (lane < slanes) {
          const float* d = stash_s + ((size_t)((t - t0) * 8 + j) * slanes + lane) * svals;
          const float2 lo2 = *reinterpret_cast<const float2*>(d);
          sv[0] = lo2.x; sv[1] = lo2.y;
          if (!ROWS8) { const float2 hi2 = *reinterpret_cast<const float2*>(d + 2); sv[2] = hi2.x; sv[3] = hi2.y; }
        }
        float w[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int e = 0; e < NE; ++e)
          w[e] = (sv[e] == ninf) ? 0.0f : ex2_approx(__fsub_rn(sv[e], gmax[e >> 1]));
        if (j / JW == warp) {                          // the warp that owns these keys counts them
#pragma unroll
          for (int e = 0; e < NE; ++e) {
            if (small_q) den_tile[e >> 1] += (uint32_t)float_to_fixed_any(w[e], p.scale, p.int_bits);
            else den[e >> 1] += float_to_fixed_any(w[e], p.scale, p.int_bits);
          }
        }
        pa[j >> 1][(j & 1) * 2 + 0] = pack2_io<T>(w[0], w[1]);
        pa[j >> 1][(j & 1) * 2 + 1] = ROWS8 ? 0u : pack2_io<T>(w[2], w[3]);
      }
      den[0] += (long long)den_tile[0];
      if (!ROWS8) den[1] += (long long)den_tile[1];
#pragma unroll
      for (int jj2 = 0; jj2 < DW / 2; ++jj2) {
        const int jn2 = warp * (DW / 2) + jj2;           // pair of 8-wide head-dim groups
        float pv0[4] = {0.f, 0.f, 0.f, 0.f}, pv1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(v_addr + swz<RC>(kk * 16 + (lane & 15), jn2 * 2 + (lane >> 4)), b0, b1, b2, b3);
          mma16816<T>(pv0, pa[kk], b0, b1);
          mma16816<T>(pv1, pa[kk], b2, b3);
        }
#pragma unroll
        for (int e = 0; e < NE; ++e) {
          if (ACC64) {
            acc[jj2 * 2][e] += (AccT)float_to_fixed<64>(pv0[e], p.scale);
            acc[jj2 * 2 + 1][e] += (AccT)float_to_fixed<64>(pv1[e], p.scale);
          } else {
            acc[jj2 * 2][e] += (AccT)float_to_fixed_any(pv0[e], p.scale, p.int_bits);
            acc[jj2 * 2 + 1][e] += (AccT)float_to_fixed_any(pv1[e], p.scale, p.int_bits);
          }
        }
      }
    }
    cp_async_wait<0>();
  }

  // =============================== merge ==============================================
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    den[h] += __shfl_xor_sync(0xffffffffu, den[h], 1);
    den[h] += __shfl_xor_sync(0xffffffffu, den[h], 2);
  }
  __syncthreads();                                   // stages are free: reuse them for wv_s
#pragma unroll
  for (int h = 0; h < NH; ++h) {
    const int r = g + 8 * h;
    if (t4 == 0) den_s[warp * 16 + r] = den[h];
#pragma unroll
    for (int jj = 0; jj < DW; ++jj) {
      const int d = (warp * DW + jj) * 8 + 2 * t4;
      wv_s[(size_t)r * HD + d] = (long long)acc[jj][2 * h];
      wv_s[(size_t)r * HD + d + 1] = (long long)acc[jj][2 * h + 1];
    }
  }
  // One denominator per row and CTA (not one per warp): reads over distributed shared memory are
  // paced per request, so the merge below asks for as few and as wide ones as it can.
  __syncthreads();
  long long den_row = 0;
  if (threadIdx.x < 16) {
#pragma unroll
    for (int w = 0; w < NW; ++w) den_row += den_s[w * 16 + threadIdx.x];
  }
  __syncthreads();
  if (threadIdx.x < 16) den_s[threadIdx.x] = den_row;
  cluster.sync();
  {
    // Every rank merges its own slice of the head dimension (integer sums over the ranks are
    // order-free), so the peers' shared memory is needed only for a short, parallel read.
    const int rows_here = min(16, (tok_end - tok0) * G);
    const int cpr = (HD + S - 1) / S;                // columns per rank
    const int c0 = rank * cpr;
    const int ncol = max(0, min(HD, c0 + cpr) - c0);
    const bool pairs = ((cpr | ncol) & 1) == 0;      // then c0 is even too: 16-byte reads
    const int per_row = pairs ? ncol / 2 : ncol;
    for (int idx = threadIdx.x; idx < rows_here * per_row; idx += NT) {
      const int r = idx / per_row, d = c0 + (pairs ? 2 : 1) * (idx % per_row);
      long long dsum = 0, w0 = 0, w1 = 0;
      for (int rr = 0; rr < S; ++rr) {
        dsum += cluster.map_shared_rank(den_s, rr)[r];
        const long long* wp = cluster.map_shared_rank(wv_s, rr) + (size_t)r * HD + d;
        if (pairs) {
          const longlong2 v = *reinterpret_cast<const longlong2*>(wp);
          w0 += v.x;
          w1 += v.y;
        } else {
          w0 += wp[0];
        }
      }
      const float dn = fmaxf(fixed_to_float<long long>(wrap_to_bits(dsum, p.int_bits), p.inv_scale), 1.0e-6f);
      const int tok = tok0 + r / G, head = kvh * G + r % G;
      T* op = (T*)p.o + (int64_t)(q_start + tok) * p.o_st + (int64_t)head * p.o_sh;
      op[d] = from_f32<T>(__fdiv_rn(fixed_to_float<long long>(wrap_to_bits(w0, p.int_bits), p.inv_scale), dn));
      if (pairs)
        op[d + 1] = from_f32<T>(__fdiv_rn(fixed_to_float<long long>(wrap_to_bits(w1, p.int_bits), p.inv_scale), dn));
    }
  }
  cluster.sync();
}

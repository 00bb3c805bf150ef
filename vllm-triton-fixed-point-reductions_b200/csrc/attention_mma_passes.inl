// Body of attn_mma_kernel after set-up: pass A (row maxima, optional score stash),
// cluster-wide maximum, pass B (integer denominator and numerator), cluster-wide integer
// merge and the final divide.  Included inside the kernel.

  // =============================== pass A =============================================
  float rmax[2] = {ninf, ninf};
  {
    int issued = t0;
#pragma unroll 1
    for (int s = 0; s < NSTAGE - 1; ++s) {
      if (issued < t1) { issue_tile(kbase, issued, stage0 + (issued - t0) % NSTAGE * kStageBytes); ++issued; }
      cp_async_commit();
    }
#pragma unroll 1
    for (int t = t0; t < t1; ++t) {
      cp_async_wait<NSTAGE - 2>();
      __syncthreads();                               // tile t (and Q) landed; stage of t-1 is free
      if (issued < t1) { issue_tile(kbase, issued, stage0 + (issued - t0) % NSTAGE * kStageBytes); ++issued; }
      cp_async_commit();
      float s[8][4];
      qk_tile(stage0 + (t - t0) % NSTAGE * kStageBytes, t, s);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        rmax[0] = fmaxf(rmax[0], fmaxf(s[j][0], s[j][1]));
        rmax[1] = fmaxf(rmax[1], fmaxf(s[j][2], s[j][3]));
      }
      if (STASH) {
        if (lane < slanes) {
          float* dst = stash_s + ((size_t)((t - t0) * 8) * slanes + lane) * svals;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float* d = dst + (size_t)j * slanes * svals;
            d[0] = s[j][0]; d[1] = s[j][1];
            if (svals == 4) { d[2] = s[j][2]; d[3] = s[j][3]; }
          }
        }
      }
    }
    cp_async_wait<0>();
  }
  // row maximum: across the 4 lanes that share a row, then across the cluster
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 1));
    rmax[h] = fmaxf(rmax[h], __shfl_xor_sync(0xffffffffu, rmax[h], 2));
    if (t4 == 0) rmax_s[warp * 16 + g + 8 * h] = rmax[h];
  }
  cluster.sync();
  float gmax[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float m = ninf;
    for (int r = 0; r < S; ++r) m = fmaxf(m, cluster.map_shared_rank(rmax_s, r)[warp * 16 + g + 8 * h]);
    gmax[h] = (m == ninf) ? 0.0f : m;               // rows without keys: exp2 gives 0, not NaN
  }

  if constexpr (FAST) {
#include "attention_mma_pass_b_fast.inl"
  } else {
  // =============================== pass B =============================================
  long long den[2] = {0, 0};
  AccT acc[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j) { acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0; }
  {
    // STASH: a stage holds one V tile.  Otherwise a stage holds K then V.
    auto issue_b = [&](int t) {
      const uint32_t dst = stage0 + (t - t0) % NSTAGE * kStageBytes;
      if (STASH) issue_kv(t, 0, dst, false, true);
      else issue_kv(t, dst, dst + kTileBytes, true, true);
    };
    __syncthreads();                                 // everyone is done with pass A's stages
    int issued = t0;
#pragma unroll 1
    for (int s = 0; s < NSTAGE - 1; ++s) {
      if (issued < t1) { issue_b(issued); ++issued; }
      cp_async_commit();
    }
#pragma unroll 1
    for (int t = t0; t < t1; ++t) {
      cp_async_wait<NSTAGE - 2>();
      __syncthreads();
      if (issued < t1) { issue_b(issued); ++issued; }
      cp_async_commit();
      const uint32_t st = stage0 + (t - t0) % NSTAGE * kStageBytes;
      float s[8][4];
      if (STASH) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = ninf; }
        if (lane < slanes) {
          const float* src = stash_s + ((size_t)((t - t0) * 8) * slanes + lane) * svals;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float* d = src + (size_t)j * slanes * svals;
            s[j][0] = d[0]; s[j][1] = d[1];
            if (svals == 4) { s[j][2] = d[2]; s[j][3] = d[3]; }
          }
        }
      } else {
        qk_tile(st, t, s);
      }
      // weights, integer denominator, P in the io dtype as the A operand of P.V
      uint32_t pa[4][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          w[e] = (s[j][e] == ninf) ? 0.0f : ex2_approx(__fsub_rn(s[j][e], gmax[e >> 1]));
          den[e >> 1] += float_to_fixed_any(w[e], p.scale, p.int_bits);
        }
        pa[j >> 1][(j & 1) * 2 + 0] = pack2_io<T>(w[0], w[1]);
        pa[j >> 1][(j & 1) * 2 + 1] = pack2_io<T>(w[2], w[3]);
      }
      const uint32_t v_addr = STASH ? st : st + kTileBytes;
#pragma unroll
      for (int jn2 = 0; jn2 < HD / 16; ++jn2) {
        float pv0[4] = {0.f, 0.f, 0.f, 0.f}, pv1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4_t(v_frag(v_addr, kk, jn2), b0, b1, b2, b3);
          mma16816<T>(pv0, pa[kk], b0, b1);
          mma16816<T>(pv1, pa[kk], b2, b3);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (ACC64) {
            acc[jn2 * 2][e] += (AccT)float_to_fixed<64>(pv0[e], p.scale);
            acc[jn2 * 2 + 1][e] += (AccT)float_to_fixed<64>(pv1[e], p.scale);
          } else {
            acc[jn2 * 2][e] += (AccT)float_to_fixed_any(pv0[e], p.scale, p.int_bits);
            acc[jn2 * 2 + 1][e] += (AccT)float_to_fixed_any(pv1[e], p.scale, p.int_bits);
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
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + g + 8 * h;
    if (t4 == 0) den_s[r] = den[h];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) {
      wv_s[(size_t)r * HD + j * 8 + 2 * t4] = (long long)acc[j][2 * h];
      wv_s[(size_t)r * HD + j * 8 + 2 * t4 + 1] = (long long)acc[j][2 * h + 1];
    }
  }
  }
  cluster.sync();
  if (rank == 0) {
    // integer sums over the ranks are order-free; rank 0 converts once and stores
    const int rows_here = min(BM, (tok_end - tok0) * G);
    for (int idx = threadIdx.x; idx < rows_here * HD; idx += NT) {
      const int r = idx / HD, d = idx % HD;
      long long dsum = 0, wsum = 0;
      for (int rr = 0; rr < S; ++rr) {
        dsum += cluster.map_shared_rank(den_s, rr)[r];
        wsum += cluster.map_shared_rank(wv_s, rr)[(size_t)r * HD + d];
      }
      const float dn = fmaxf(fixed_to_float<long long>(wrap_to_bits(dsum, p.int_bits), p.inv_scale), 1.0e-6f);
      const float num = fixed_to_float<long long>(wrap_to_bits(wsum, p.int_bits), p.inv_scale);
      const int tok = tok0 + r / G, head = kvh * G + r % G;
      T* op = (T*)p.o + (int64_t)(q_start + tok) * p.o_st + (int64_t)head * p.o_sh;
      op[d] = from_f32<T>(__fdiv_rn(num, dn));
    }
  }
  cluster.sync();                                    // peers' shared memory stays alive until rank 0 is done

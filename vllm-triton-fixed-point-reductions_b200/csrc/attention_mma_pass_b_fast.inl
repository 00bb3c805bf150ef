// Second pass of attn_mma_kernel with the float -> Q-format conversions on the FP32 pipe
// (included inside the kernel when FAST; requires frac_bits <= 16, int_bits 32 or 64, at
// most kFastMaxTiles key tiles per CTA, no score stash).
//
//   r = fma(v, 2^f, 1.5 * 2^23): for |v * 2^f| < 2^22 the low mantissa bits of r are exactly
//   rint_half_even(v * 2^f), so bits(r) = MAGIC + q and the raw bit patterns can be summed
//   as 32-bit integers; count * MAGIC is taken out once at the end.
//
// Weights are in [0, 1], always in range.  A P.V partial is in range while |pv| < 2^(22-f);
// the exponent field of r tells (it is 150 exactly when in range), so the screen costs one
// logic operation per element.  A tile that fails the screen (warp-uniform decision) is
// recomputed in place, recording what the fast add contributed for the offending
// elements and what the reference conversion gives for them.  The result is bit-identical
// to the cvt.rni.sat path.
    __syncthreads();                                 // everyone is done with pass A's stages
    uint32_t acc32[HD / 8][4];
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) { acc32[j][0] = acc32[j][1] = acc32[j][2] = acc32[j][3] = 0; }
    uint32_t den32[2] = {0, 0};
    long long den[2];
    uint32_t corr_raw[HD / 2];                       // rare path, local memory
    long long corr_q[HD / 2];
    bool corr_used = false;
    const float magic = __uint_as_float(kAttnMagicBits);
    {
      auto issue_b = [&](int t) {
        const uint32_t dst = stage0 + (t - t0) % NSTAGE * kStageBytes;
        issue_kv(t, dst, dst + kTileBytes, true, true);
      };
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
        qk_tile(st, t, s);
        // weights, integer denominator, P in the io dtype as the A operand of P.V
        uint32_t pa[4][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float w[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            w[e] = (s[j][e] == ninf) ? 0.0f : ex2_approx(__fsub_rn(s[j][e], gmax[e >> 1]));
            den32[e >> 1] += __float_as_uint(__fmaf_rn(w[e], p.scale, magic));
          }
          pa[j >> 1][(j & 1) * 2 + 0] = pack2_io<T>(w[0], w[1]);
          pa[j >> 1][(j & 1) * 2 + 1] = pack2_io<T>(w[2], w[3]);
        }
        const uint32_t v_addr = st + kTileBytes;
        uint32_t screen = 0;
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
            const uint32_t r0 = __float_as_uint(__fmaf_rn(pv0[e], p.scale, magic));
            const uint32_t r1 = __float_as_uint(__fmaf_rn(pv1[e], p.scale, magic));
            acc32[jn2 * 2][e] += r0;
            acc32[jn2 * 2 + 1][e] += r1;
            screen |= (r0 ^ kAttnExpBits) | (r1 ^ kAttnExpBits);
          }
        }
        if (__any_sync(0xffffffffu, (screen >> 23) != 0)) {
          if (!corr_used) {
#pragma unroll 1
            for (int z = 0; z < HD / 2; ++z) { corr_raw[z] = 0; corr_q[z] = 0; }
            corr_used = true;
          }
          // recompute this tile's partials (same MMA sequence, same bits); for every element
          // outside the fast range record what the fast add contributed and what the
          // reference conversion gives.  Rolled loop: the arrays stay in local memory.
#pragma unroll 1
          for (int jn2 = 0; jn2 < HD / 16; ++jn2) {
            float pv[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              uint32_t b0, b1, b2, b3;
              ldsm_x4_t(v_addr + swz<RC>(kk * 16 + (lane & 15), jn2 * 2 + (lane >> 4)), b0, b1, b2, b3);   // runtime jn2: no table lookup
              mma16816<T>(pv[0], pa[kk], b0, b1);
              mma16816<T>(pv[1], pa[kk], b2, b3);
            }
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float f = pv[u][e];
                const uint32_t bb = __float_as_uint(__fmaf_rn(f, p.scale, magic));
                if (((bb ^ kAttnExpBits) >> 23) != 0) {
                  const int idx = (jn2 * 2 + u) * 4 + e;
                  corr_raw[idx] += bb - kAttnMagicBits;
                  corr_q[idx] += float_to_fixed_any(f, p.scale, p.int_bits);
                }
              }
          }
        }
      }
      cp_async_wait<0>();
    }

    // ---- back to exact integers ------------------------------------------------------
    const uint32_t n_tiles_done = (uint32_t)(t1 - t0);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      // 16 weights per row, thread and tile went through the fast add
      den[h] = (long long)(int32_t)(den32[h] - 16u * n_tiles_done * kAttnMagicBits);
      den[h] += __shfl_xor_sync(0xffffffffu, den[h], 1);
      den[h] += __shfl_xor_sync(0xffffffffu, den[h], 2);
    }
    __syncthreads();                                 // stages are free: reuse them for wv_s
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = warp * 16 + g + 8 * h;
      if (t4 == 0) den_s[r] = den[h];
#pragma unroll
      for (int j = 0; j < HD / 8; ++j) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int e = 2 * h + c;
          uint32_t raw = acc32[j][e] - n_tiles_done * kAttnMagicBits;
          long long tot;
          if (corr_used) {
            raw -= corr_raw[j * 4 + e];
            tot = (long long)(int32_t)raw + corr_q[j * 4 + e];
          } else {
            tot = (long long)(int32_t)raw;
          }
          wv_s[(size_t)r * HD + j * 8 + 2 * t4 + c] = tot;
        }
      }
    }

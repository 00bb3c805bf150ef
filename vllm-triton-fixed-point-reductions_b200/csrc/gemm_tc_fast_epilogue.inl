// Epilogue-warp body of gemm_tc_fast_kernel (included inside the kernel: it uses the
// kernel's template parameters and locals).  Warp w owns TMEM lanes 32*(w%4).. (one
// output row per thread) and kCols consecutive columns.
{
  const int quarter = warp & 3;
  const int cgroup = (warp - kRoleWarps) >> 2;
  const int row_in_tile = quarter * 32 + lane;
  const int col0 = cgroup * kCols;
  const uint32_t lane_addr = ((uint32_t)(quarter * 32) << 16) + (uint32_t)col0;
  const float magic = __uint_as_float(kMagicBits);
  const float scale = p.scale;
  int grp = 0; uint32_t gphase = 0; uint32_t epi_phase = 0; bool ok = true;
  int gss = 0;
  auto epi_sync = [&]() -> bool {   // bounded barrier over the epilogue warps only
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

  for (int item = blockIdx.x; item < items && ok; item += gridDim.x) {
    const int tile = item / p.split_k, ks = item % p.split_k;
    int pm, pn; tile_coords(tile, pm, pn);
    const int row = pm * kBM + row_in_tile;
    const int ncol0 = pn * BN + col0;
    const int n_kt = (k_tiles_total - ks + p.split_k - 1) / p.split_k;
    uint32_t acc[kCols];
#pragma unroll
    for (int i = 0; i < kCols; ++i) acc[i] = 0;
    corr_used = false;

    const int n_ss = pairs ? (n_kt + 1) >> 1 : n_kt;
    for (int ss = 0; ss < n_ss; ++ss) {
      if (!warp_wait(tfull0 + 8u * grp, gphase, abort_flag, lane)) { ok = false; break; }
      tc_fence_after();
      const int nbuf = (pairs && 2 * ss + 1 < n_kt) ? 2 : 1;
      // Hot path: r = fma(p, 2^f, MAGIC) on the FP32 pipe, raw bit patterns added as
      // integers, and the OR of the raw fp32 bits as a screen: bit 30 stays clear only if
      // every |p| < 2, which (f <= 21) implies |p * 2^f| < 2^22.
      // Measured on B200: this plain order (load 16 columns, wait, convert) beats both a
      // software-pipelined order (next load in flight during the conversion: -6 %) and a
      // pairwise order (both K-tiles of a pair per step, one three-input add: -11 %).
      static_assert(kCols == 32, "two 16-column chunks per accumulator buffer");
      const uint32_t ta0 = tmem_base + lane_addr + (uint32_t)((grp * 2) * BN);
      const uint32_t ta1 = ta0 + BN;
      uint32_t va[16], vb[16];
      uint32_t screen0 = 0, screen1 = 0;
      auto convert = [&](const uint32_t (&v)[16], int c, uint32_t& screen, int h) {
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          acc[c * 16 + i] += __float_as_uint(__fmaf_rn(__uint_as_float(v[i]), scale, magic));
          acc[c * 16 + i + 1] += __float_as_uint(__fmaf_rn(__uint_as_float(v[i + 1]), scale, magic));
          screen |= v[i] | v[i + 1];
        }
        if (DUMP) {
          if (row < p.M) {
            const int kt = pairs ? ks + (2 * ss + h) * p.split_k : ks + ss * p.split_k;
            float* dst = p.partials + ((int64_t)kt * p.M + row) * p.N + ncol0 + c * 16;
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (ncol0 + c * 16 + i < p.N) dst[i] = __uint_as_float(v[i]);
          }
        }
      };
      tmem_ld16(ta0, va); tmem_wait_ld_regs(va); convert(va, 0, screen0, 0);
      tmem_ld16(ta0 + 16, vb); tmem_wait_ld_regs(vb); convert(vb, 1, screen0, 0);
      if (nbuf == 2) {
        tmem_ld16(ta1, va); tmem_wait_ld_regs(va); convert(va, 0, screen1, 1);
        tmem_ld16(ta1 + 16, vb); tmem_wait_ld_regs(vb); convert(vb, 1, screen1, 1);
      }
      if (__any_sync(0xffffffffu, ((screen0 | screen1) & 0x40000000u) != 0)) {
        // exact fix-up for the K-tile(s) that failed the screen (rare): see fixup_tile
        if (!corr_used) {
#pragma unroll 1
          for (int z = 0; z < kCols; ++z) { corr_raw[z + zero] = 0; corr_q[z + zero] = 0; }
          corr_used = true;
        }
        if (__any_sync(0xffffffffu, (screen0 & 0x40000000u) != 0))
          fixup_tile(ta0, kCols, scale, p.int_bits, &corr_raw[zero], &corr_q[zero]);
        if (__any_sync(0xffffffffu, (screen1 & 0x40000000u) != 0))
          fixup_tile(ta1, kCols, scale, p.int_bits, &corr_raw[zero], &corr_q[zero]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8u * grp);
      ++gss;
      grp ^= 1; if (grp == 0) gphase ^= 1;
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

    const bool row_ok = row < p.M;
    bool do_store = true;
    // Split-K: every split leaves its integer partial tile in its own plane of the scratch
    // (column-major inside the tile, so a warp's 32 rows are 32 consecutive words and every
    // store and load is one full line); the split that arrives last adds the planes of the
    // others to its registers.  Integer addition is commutative and associative: which
    // split comes last cannot change the sum.
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
      if (threadIdx.x == kRoleWarps * 32) *s_last = (atomicAdd(p.locks + tile, 1) == p.split_k - 1) ? 1 : 0;
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
            float v = fixed_to_float<long long>(q8[i], p.inv_scale);
            if (bias && colg + i < p.N) v = __fadd_rn(v, to_f32<T>(bias[colg + i]));
            out[i] = from_f32<T>(v);
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
      if (do_store && threadIdx.x == kRoleWarps * 32) p.locks[tile] = 0;
      if (!epi_sync()) { ok = false; break; }    // s_last is rewritten only after all have read it
    }
  }
}

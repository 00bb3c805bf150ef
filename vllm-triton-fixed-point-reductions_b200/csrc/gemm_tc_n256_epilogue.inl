// Epilogue-warp body of gemm_tc_n256_kernel (included inside the kernel).  Warp w owns TMEM
// lanes 32*(w%4).. (one output row per thread) and 64 consecutive columns.
{
  const int quarter = warp & 3;
  const int cgroup = (warp - 2) >> 2;
  const int row_in_tile = quarter * 32 + lane;
  const int col0 = cgroup * kCols;
  const uint32_t lane_addr = ((uint32_t)(quarter * 32) << 16) + (uint32_t)col0;
  const float magic = __uint_as_float(kMagicBits);
  const float scale = p.scale;
  int buf = 0; uint32_t bphase = 0; uint32_t epi_phase = 0; bool ok = true;
  auto epi_sync = [&]() -> bool {   // bounded barrier over the epilogue warps only
    __syncwarp();
    if (lane == 0) mbar_arrive(epi_bar);
    const bool done = warp_wait(epi_bar, epi_phase, abort_flag, lane);
    epi_phase ^= 1;
    return done;
  };

  // Rare-path corrections (local memory, zeroed on first use), as in gemm_tc_fast_epilogue.inl
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

    for (int kt = 0; kt < n_kt; ++kt) {
      if (!warp_wait(tfull0 + 8u * buf, bphase, abort_flag, lane)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + lane_addr + (uint32_t)(buf * BN);
      // r = fma(p, 2^f, MAGIC) on the FP32 pipe, raw bit patterns added as integers; the OR of
      // the raw fp32 bits is the range screen (bit 30 clear: every |p| < 2)
      uint32_t screen = 0;
#pragma unroll
      for (int c = 0; c < kCols / 8; ++c) {
        uint32_t v[8];
        tmem_ld8(taddr + c * 8, v);
        tmem_wait_ld_regs8(v);
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          acc[c * 8 + i] += __float_as_uint(__fmaf_rn(__uint_as_float(v[i]), scale, magic));
          acc[c * 8 + i + 1] += __float_as_uint(__fmaf_rn(__uint_as_float(v[i + 1]), scale, magic));
          screen |= v[i] | v[i + 1];
        }
      }
      if (__any_sync(0xffffffffu, (screen & 0x40000000u) != 0)) {
        if (!corr_used) {
#pragma unroll 1
          for (int z = 0; z < kCols; ++z) { corr_raw[z + zero] = 0; corr_q[z + zero] = 0; }
          corr_used = true;
        }
        fixup_tile(taddr, kCols, scale, p.int_bits, &corr_raw[zero], &corr_q[zero]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8u * buf);
      buf ^= 1; if (buf == 0) bphase ^= 1;
    }
    if (!ok) break;

    const uint32_t bias_bits = (uint32_t)n_kt * kMagicBits;   // every K-tile added MAGIC once
    auto total = [&](int i) -> long long {
      uint32_t raw = acc[i] - bias_bits;
      long long t;
      if (corr_used) {
        raw -= corr_raw[i + zero];
        t = (long long)(int32_t)raw + corr_q[i + zero];
      } else {
        t = (long long)(int32_t)raw;
      }
      return p.int_bits == 64 ? t : (long long)(int32_t)t;
    };

    // Split-K: per-split integer partial planes (column-major inside the tile), summed by the
    // last arriver.
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
      if (threadIdx.x == 64) *s_last = (atomicAdd(p.locks + tile, 1) == p.split_k - 1) ? 1 : 0;
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
      if (do_store && threadIdx.x == 64) p.locks[tile] = 0;
      if (!epi_sync()) { ok = false; break; }    // s_last is rewritten only after all have read it
    }
  }
}

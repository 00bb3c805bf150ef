// Epilogue-warp body of gemm_tc_skinny_kernel (included inside the kernel).  Warp w owns
// TMEM lanes 32*(w%4).. -- one output COLUMN n per thread -- and kCols consecutive TMEM
// columns, which are activation rows m.  Same conversion as gemm_tc_fast_epilogue.inl.
{
  const int quarter = warp & 3;
  const int cgroup = (warp - 2) >> 2;
  const int n_in_tile = quarter * 32 + lane;
  const int m0 = cgroup * kCols;
  const uint32_t lane_addr = ((uint32_t)(quarter * 32) << 16) + (uint32_t)m0;
  const float magic = __uint_as_float(kMagicBits);
  const float scale = p.scale;
  int grp = 0; uint32_t gphase = 0; uint32_t epi_phase = 0; bool ok = true;
  auto epi_sync = [&]() -> bool {   // bounded barrier over the epilogue warps only
    __syncwarp();
    if (lane == 0) mbar_arrive(epi_bar);
    const bool done = warp_wait(epi_bar, epi_phase, abort_flag, lane);
    epi_phase ^= 1;
    return done;
  };

  // Rare-path corrections (local memory, zeroed on first use), as in the wide kernel.
  uint32_t corr_raw[kCols];
  long long corr_q[kCols];
  bool corr_used = false;

  for (int item = first_item; item < items && ok; item += item_step) {
    const int tile = item / p.split_k, ks = item % p.split_k;
    const int n = tile * 128 + n_in_tile;
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
      static_assert(kCols == 32, "two 16-column chunks per accumulator buffer");
      const uint32_t ta0 = tmem_base + lane_addr + (uint32_t)grp * group_cols;
      const uint32_t ta1 = ta0 + MP;
      uint32_t va[16], vb[16];
      uint32_t screen0 = 0, screen1 = 0;
      auto convert = [&](const uint32_t (&v)[16], int c, uint32_t& screen) {
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          acc[c * 16 + i] += __float_as_uint(__fmaf_rn(__uint_as_float(v[i]), scale, magic));
          acc[c * 16 + i + 1] += __float_as_uint(__fmaf_rn(__uint_as_float(v[i + 1]), scale, magic));
          screen |= v[i] | v[i + 1];
        }
      };
      // both halves of a buffer are requested before the one wait
      tmem_ld16(ta0, va); tmem_ld16(ta0 + 16, vb); tmem_wait_ld_regs2(va, vb);
      convert(va, 0, screen0); convert(vb, 1, screen0);
      if (nbuf == 2) {
        tmem_ld16(ta1, va); tmem_ld16(ta1 + 16, vb); tmem_wait_ld_regs2(va, vb);
        convert(va, 0, screen1); convert(vb, 1, screen1);
      }
      if (__any_sync(0xffffffffu, ((screen0 | screen1) & 0x40000000u) != 0)) {
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
      if (++grp == ngroup) { grp = 0; gphase ^= 1; }
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

    // Split-K: per-split integer partial planes, column-major inside the 128 x 64 tile (the
    // warp's 32 output columns are 32 consecutive words); the last arriver adds the others.
    if constexpr (CLUSTER) {
      if (p.split_k > 1) {
        // this split's partials go to shared memory; the cluster merge after the role branches
        // sums them over the ranks and writes the outputs
        long long* red = reinterpret_cast<long long*>(smem_gen);
#pragma unroll
        for (int i = 0; i < kCols; ++i) red[(m0 + i) * 128 + n_in_tile] = total(i);
        continue;
      }
    }
    bool do_store = true;
    const int64_t plane_elems = (int64_t)128 * MP;
    const int64_t plane_stride = (int64_t)tiles_n * plane_elems;
    const int64_t plane_off = (int64_t)tile * plane_elems + (int64_t)m0 * 128 + n_in_tile;
    if (p.split_k > 1) {
      if (p.int_bits == 64) {
        long long* dst = (long long*)p.acc_scratch + ks * plane_stride + plane_off;
#pragma unroll
        for (int i = 0; i < kCols; ++i) __stcg(dst + i * 128, total(i));
      } else {
        int* dst = (int*)p.acc_scratch + ks * plane_stride + plane_off;
#pragma unroll
        for (int i = 0; i < kCols; ++i) __stcg(dst + i * 128, (int)total(i));
      }
      __threadfence();
      if (!epi_sync()) { ok = false; break; }
      if (threadIdx.x == 64) *s_last = (atomicAdd(p.locks + tile, 1) == p.split_k - 1) ? 1 : 0;
      if (!epi_sync()) { ok = false; break; }
      do_store = *s_last != 0;
      if (do_store) __threadfence();
    }

    if (do_store) {
      long long q[kCols];
#pragma unroll
      for (int i = 0; i < kCols; ++i) q[i] = total(i);
      if (p.split_k > 1) {
        // all 32 loads of a plane are in flight together (the sums are order-free)
        for (int s2 = 0; s2 < p.split_k; ++s2) {
          if (s2 == ks) continue;
          if (p.int_bits == 64) {
            const long long* src = (const long long*)p.acc_scratch + s2 * plane_stride + plane_off;
#pragma unroll
            for (int i = 0; i < kCols; ++i) q[i] += __ldcg(src + i * 128);
          } else {
            const int* src = (const int*)p.acc_scratch + s2 * plane_stride + plane_off;
#pragma unroll
            for (int i = 0; i < kCols; ++i) q[i] += (long long)__ldcg(src + i * 128);
          }
        }
        if (p.int_bits != 64) {
#pragma unroll
          for (int i = 0; i < kCols; ++i) q[i] = (long long)(int32_t)q[i];
        }
      }
      if (p.silu_mul) {
        // columns come in (gate, up) pairs held by neighbouring lanes: the even lane combines the
        // two outputs as the io dtype holds them and writes column n / 2 of the [M, N / 2] result
        const T* bias = (const T*)p.bias;
        const float bias_f = (bias && n < p.N) ? to_f32<T>(bias[n]) : 0.0f;
#pragma unroll
        for (int i = 0; i < kCols; ++i) {
          float v = fixed_to_float<long long>(q[i], p.inv_scale);
          if (bias) v = __fadd_rn(v, bias_f);
          const float mine = to_f32<T>(from_f32<T>(v));
          const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
          const int m = m0 + i;
          if (!(lane & 1) && n + 1 < p.N && m < p.M)
            ((T*)p.c)[(int64_t)m * p.c_sm + (n >> 1)] = silu_mul_io<T>(mine, other);
        }
      } else if (n < p.N) {
        const T* bias = (const T*)p.bias;
        const float bias_f = bias ? to_f32<T>(bias[n]) : 0.0f;
#pragma unroll
        for (int i = 0; i < kCols; ++i) {           // fully unrolled: the arrays stay in registers
          const int m = m0 + i;
          if (m >= p.M) continue;
          if (p.c_int) {
            if (p.int_bits == 64) ((long long*)p.c_int)[(int64_t)m * p.N + n] = q[i];
            else ((int32_t*)p.c_int)[(int64_t)m * p.N + n] = (int32_t)q[i];
          }
          if (p.c) {
            float v = fixed_to_float<long long>(q[i], p.inv_scale);
            if (bias) v = __fadd_rn(v, bias_f);
            ((T*)p.c)[(int64_t)m * p.c_sm + n] = from_f32<T>(v);
          }
        }
      }
      if (p.best) {
        // Greedy sampling without a pass over the logits: per row, the best (value, column) key
        // over this warp's 32 columns by recursive halving -- after the exchange with the lane at
        // distance d a lane keeps half of the rows it held -- then one atomic maximum per row.
        const T* bias = (const T*)p.bias;
        const float bias_f = (bias && n < p.N) ? to_f32<T>(bias[n]) : 0.0f;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          unsigned long long key[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float v = fixed_to_float<long long>(q[half * 16 + i], p.inv_scale);
            if (bias) v = __fadd_rn(v, bias_f);
            v = to_f32<T>(from_f32<T>(v));                       // the logit as the io dtype holds it
            key[i] = n < p.N ? argmax_key(v, p.n_offset + (unsigned int)n) : 0ull;
          }
#pragma unroll
          for (int step = 0; step < 4; ++step) {
            const int d = 16 >> step, cnt = 8 >> step;
            const bool upper = (lane & d) != 0;                  // keeps rows [cnt, 2 cnt) of what it holds
#pragma unroll
            for (int i = 0; i < cnt; ++i) {
              const unsigned long long send = upper ? key[i] : key[cnt + i];
              const unsigned long long recv = __shfl_xor_sync(0xffffffffu, send, d);
              const unsigned long long mine = upper ? key[cnt + i] : key[i];
              key[i] = mine > recv ? mine : recv;
            }
          }
          const unsigned long long other = __shfl_xor_sync(0xffffffffu, key[0], 1);
          const unsigned long long top = key[0] > other ? key[0] : other;
          const int row = half * 16 + ((lane & 16) ? 8 : 0) + ((lane & 8) ? 4 : 0) + ((lane & 4) ? 2 : 0) +
                          ((lane & 2) ? 1 : 0);
          if (!(lane & 1) && m0 + row < p.M && top != 0ull) atomicMax(p.best + m0 + row, top);
        }
      }
    }
    if (p.split_k > 1) {
      if (do_store && threadIdx.x == 64) p.locks[tile] = 0;
      if (!epi_sync()) { ok = false; break; }    // s_last is rewritten only after all have read it
    }
  }
}

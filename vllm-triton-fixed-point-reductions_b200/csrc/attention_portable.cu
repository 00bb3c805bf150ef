// Portable unified (prefill + decode) paged attention on CUDA cores: any dtype,
// head size and page size.  One warp owns one (query token, head, kv-split).
//
// Semantics: fxpr_vllm/_triton/attention.py of the reference -- score
// post-processing :103-121, masks :199-215, exact row maximum first :233-257,
// then w = exp2(s - max), integer denominator sum(Q(w)) and integer numerator
// sum over 64-key (32 for fp32) tiles of Q(P.V) :259-290, out = num / max(den, 1e-6)
// :292-301; split path :306-652 (per-split maxima, integer atomics, last arriver).
//
// Differences, all bit-neutral or documented: key tiles always start at key 0
// (with a sliding window the reference starts them at a query-block dependent
// offset, which makes its bits depend on batching); fully masked tiles are
// skipped (they add integer zeros); float sums run in a fixed ascending order
// with separate multiply and add and exp2 is the deterministic polynomial, so a
// CPU reproduces every bit.
#include "attention_common.cuh"
#include "fxp_common.cuh"

namespace fxpr {


static constexpr int kAttnWarps = 4;

template <typename T, int BN>
__global__ void __launch_bounds__(kAttnWarps * 32)
attn_portable_kernel(const AttnParams p, const int phase /*0 fused, 1 split-max, 2 split-dv*/) {
  extern __shared__ float smem[];
  constexpr int KPL = BN / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int D = p.head_dim;
  float* q_s = smem + (size_t)warp * (D + BN);
  float* w_s = q_s + D;

  const int S = p.num_splits;
  const int64_t gw = (int64_t)blockIdx.x * kAttnWarps + warp;
  const int64_t total = p.total_q * p.num_heads * S;
  if (gw >= total) return;
  const int split = (int)(gw % S);
  const int head = (int)((gw / S) % p.num_heads);
  const int64_t tok = gw / ((int64_t)S * p.num_heads);
  const int kvh = head / (p.num_heads / p.num_kv_heads);

  // request owning this token: last r with qsl[r] <= tok
  int lo_r = 0, hi_r = p.num_reqs;
  while (hi_r - lo_r > 1) {
    const int mid = (lo_r + hi_r) >> 1;
    if ((int64_t)p.qsl[mid] <= tok) lo_r = mid; else hi_r = mid;
  }
  const int req = lo_r;
  const int q_start = p.qsl[req], q_end = p.qsl[req + 1];
  if (tok < q_start || tok >= q_end) return;  // token past the last request
  const int q_len = q_end - q_start;
  const int seq_len = p.seq_lens[req];
  const int pos = seq_len - q_len + (int)(tok - q_start);
  const int key_end = p.causal ? min(seq_len, pos + 1) : seq_len;
  const int key_begin = p.window > 0 ? max(0, pos - p.window + 1) : 0;

  const int t_first = key_begin / BN;
  const int t_last = max(t_first, (key_end + BN - 1) / BN);
  const int per_split = (t_last - t_first + S - 1) / S;
  const int t0 = min(t_last, t_first + split * per_split);
  const int t1 = min(t_last, t0 + per_split);

  const T* qp = (const T*)p.q + tok * p.q_st + (int64_t)head * p.q_sh;
  for (int d = lane; d < D; d += 32) q_s[d] = to_f32<T>(qp[d]);
  __syncwarp();

  const int32_t* bt = p.block_table + (int64_t)req * p.bt_stride;
  const float slope = p.alibi ? p.alibi[head] : 0.0f;
  const float ninf = -__int_as_float(0x7f800000);

  // score of key n for this row, or -inf when masked
  auto score = [&](int n) -> float {
    if (n < key_begin || n >= key_end) return ninf;
    const int phys = bt[n / p.page_size];
    const T* kp = (const T*)p.k + (int64_t)phys * p.kv_sblock +
                  (int64_t)(n % p.page_size) * p.kv_sslot + (int64_t)kvh * p.kv_shead;
    float s = 0.0f;
    for (int d = 0; d < D; ++d) s = __fadd_rn(s, __fmul_rn(q_s[d], to_f32<T>(kp[d])));
    s = __fmul_rn(s, p.ss_log2);
    if (p.cap_log2 > 0.0f) s = __fmul_rn(p.cap_log2, tanhf(__fdiv_rn(s, p.cap_log2)));
    if (p.alibi) s = __fadd_rn(s, __fmul_rn(slope, __fsub_rn((float)n, (float)pos)));
    return s;
  };

  float gmax = ninf;
  if (phase != 2) {
    for (int t = t0; t < t1; ++t)
#pragma unroll
      for (int i = 0; i < KPL; ++i) gmax = fmaxf(gmax, score(t * BN + lane + 32 * i));
    gmax = warp_max_f32(gmax);
    if (phase == 1) {
      if (lane == 0) p.partial_max[(tok * p.num_heads + head) * S + split] = gmax;
      return;
    }
  } else {
    const float* pm = p.partial_max + (tok * p.num_heads + head) * S;
    for (int s = lane; s < S; s += 32) gmax = fmaxf(gmax, pm[s]);
    gmax = warp_max_f32(gmax);
  }
  if (gmax == ninf) gmax = 0.0f;

  // ---- pass 2: integer denominator and numerator -----------------------------------
  long long den = 0;
  long long wv[8];  // D <= 256: lane owns dims lane + 32 j
#pragma unroll
  for (int j = 0; j < 8; ++j) wv[j] = 0;
  const int nd = (D + 31) / 32;

  for (int t = t0; t < t1; ++t) {
#pragma unroll
    for (int i = 0; i < KPL; ++i) {
      const int n = t * BN + lane + 32 * i;
      const float s = score(n);
      const float w = (s == ninf) ? 0.0f : exp2_det(__fsub_rn(s, gmax));
      den += float_to_fixed_any(w, p.scale, p.int_bits);
      w_s[lane + 32 * i] = to_f32<T>(from_f32<T>(w));  // numerator sees the IO-rounded weight
    }
    __syncwarp();
    float pv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) pv[j] = 0.0f;
    const int n_hi = min(BN, seq_len - t * BN);
    for (int jn = 0; jn < n_hi; ++jn) {
      const int n = t * BN + jn;
      const int phys = bt[n / p.page_size];
      const T* vp = (const T*)p.v + (int64_t)phys * p.kv_sblock +
                    (int64_t)(n % p.page_size) * p.kv_sslot + (int64_t)kvh * p.kv_shead;
      const float wj = w_s[jn];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int d = lane + 32 * j;
        if (j < nd && d < D) pv[j] = __fadd_rn(pv[j], __fmul_rn(wj, to_f32<T>(vp[d])));
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < nd) wv[j] += float_to_fixed_any(pv[j], p.scale, p.int_bits);
    __syncwarp();
  }
  den = warp_sum_i64(den);

  T* op = (T*)p.o + tok * p.o_st + (int64_t)head * p.o_sh;
  if (phase == 0) {
    const float dn = fmaxf(fixed_to_float<long long>(wrap_to_bits(den, p.int_bits), p.inv_scale), 1.0e-6f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int d = lane + 32 * j;
      if (j < nd && d < D) {
        const float num = fixed_to_float<long long>(wrap_to_bits(wv[j], p.int_bits), p.inv_scale);
        op[d] = from_f32<T>(__fdiv_rn(num, dn));
      }
    }
    return;
  }

  // split path: integer atomics are commutative, so arrival order is irrelevant
  const int64_t th = tok * p.num_heads + head;
  unsigned long long* td = (unsigned long long*)p.total_denom + th;
  unsigned long long* tw = (unsigned long long*)p.total_wv + th * D;
  if (lane == 0) atomicAdd(td, (unsigned long long)den);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int d = lane + 32 * j;
    if (j < nd && d < D) atomicAdd(tw + d, (unsigned long long)wv[j]);
  }
  __threadfence();
  __syncwarp();
  int arrived = 0;
  if (lane == 0) arrived = atomicAdd(p.locks + th, 1);
  arrived = __shfl_sync(0xffffffffu, arrived, 0);
  if (arrived != S - 1) return;
  __threadfence();
  const long long den_all = (long long)atomicAdd(td, 0ull);
  const float dn = fmaxf(fixed_to_float<long long>(wrap_to_bits(den_all, p.int_bits), p.inv_scale), 1.0e-6f);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int d = lane + 32 * j;
    if (j < nd && d < D) {
      const long long wv_all = (long long)atomicAdd(tw + d, 0ull);
      const float num = fixed_to_float<long long>(wrap_to_bits(wv_all, p.int_bits), p.inv_scale);
      op[d] = from_f32<T>(__fdiv_rn(num, dn));
    }
  }
}

template <typename T, int BN>
static int attn_portable_launch(const AttnParams& p, cudaStream_t s) {
  const int64_t warps = p.total_q * p.num_heads * p.num_splits;
  const unsigned grid = (unsigned)((warps + kAttnWarps - 1) / kAttnWarps);
  const size_t smem = (size_t)kAttnWarps * (p.head_dim + BN) * sizeof(float);
  if (p.num_splits <= 1) {
    attn_portable_kernel<T, BN><<<grid, kAttnWarps * 32, smem, s>>>(p, 0);
  } else {
    attn_portable_kernel<T, BN><<<grid, kAttnWarps * 32, smem, s>>>(p, 1);
    attn_portable_kernel<T, BN><<<grid, kAttnWarps * 32, smem, s>>>(p, 2);
  }
  return check_launch("attention_portable");
}

int attention_portable(const AttnParams& p, int dtype, cudaStream_t s) {
  if (p.head_dim > 256) return FXPR_ERR_UNSUPPORTED;
  switch (dtype) {
    case FXPR_F32: return attn_portable_launch<float, 32>(p, s);
    case FXPR_F16: return attn_portable_launch<__half, 64>(p, s);
    case FXPR_BF16: return attn_portable_launch<__nv_bfloat16, 64>(p, s);
  }
  return FXPR_ERR_UNSUPPORTED;
}

}  // namespace fxpr

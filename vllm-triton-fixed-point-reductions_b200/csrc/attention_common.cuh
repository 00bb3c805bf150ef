// Launch parameters shared by the attention kernels and their dispatcher.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace fxpr {

struct AttnParams {
  const void* q; const void* k; const void* v; void* o;
  const int32_t* qsl; const int32_t* seq_lens; const int32_t* block_table; const float* alibi;
  int64_t total_q; int num_reqs, num_heads, num_kv_heads, head_dim, page_size;
  int64_t q_st, q_sh, o_st, o_sh, kv_sblock, kv_sslot, kv_shead, bt_stride;
  int causal, window, int_bits, num_splits;
  float ss_log2, cap_log2, scale, inv_scale;
  float* partial_max;          // [T, H, S]
  long long* total_denom;      // [T, H]
  long long* total_wv;         // [T, H, D]
  int32_t* locks;              // [T, H]
  int32_t* status;             // optional device status word (bounded waits, capacity refusals)
};

// Scratch carve-up for the split path: [partial_max | total_denom | total_wv | locks],
// each region 256-byte aligned.
struct AttnScratchLayout {
  int64_t off_pmax, off_denom, off_wv, off_locks, zero_begin, zero_bytes, total;
};

inline AttnScratchLayout attn_scratch_layout(int64_t total_q, int heads, int head_dim, int splits) {
  auto up = [](int64_t v) { return (v + 255) / 256 * 256; };
  AttnScratchLayout l;
  const int64_t th = total_q * heads;
  l.off_pmax = 0;
  l.off_denom = up(th * splits * (int64_t)sizeof(float));
  l.off_wv = l.off_denom + up(th * 8);
  l.off_locks = l.off_wv + up(th * head_dim * 8);
  l.total = l.off_locks + up(th * 4);
  l.zero_begin = l.off_denom;
  l.zero_bytes = l.total - l.off_denom;
  return l;
}

int attention_portable(const AttnParams& p, int dtype, cudaStream_t s);
int attention_mma(const AttnParams& p, int dtype, int max_query_len, bool force_exact, cudaStream_t s);
bool attention_mma_supported(const AttnParams& p, int dtype);
// tcgen05 / TMEM / TMA prefill kernel (attention_tc.cu)
bool attention_tc_supported(const AttnParams& p, int dtype, int max_query_len, bool force_exact);
int attention_tc(const AttnParams& p, int dtype, int max_query_len, int32_t* status, cudaStream_t s);

}  // namespace fxpr

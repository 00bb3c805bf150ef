// C-ABI entry points for the GEMM and attention paths: argument checking and
// routing.  Routing depends only on dtype, head/page geometry, N, K and strides
// -- never on the number of rows/tokens or on the split count -- so one logical
// operation always runs the same float instruction sequence and its bits do not
// depend on batching.
#include "attention_common.cuh"
#include "fxp_common.cuh"
#include "gemm_common.cuh"

using namespace fxpr;

static int default_k_tile(int dtype) {
  // fxpr_vllm/_triton/gemm.py:26-30: 128 for 16-bit inputs, 64 for fp32
  return dtype == FXPR_F32 ? 64 : 128;
}

extern "C" int64_t fxpr_gemm_scratch_bytes(int64_t M, int64_t N, int int_bits, int split_k) {
  if (split_k <= 1 || M <= 0 || N <= 0) return 0;
  return gemm_tc_scratch_bytes(M, N, int_bits, split_k);
}

static int gemm_entry(const void* a, const void* b, const void* bias, void* c, void* c_int,
                      int dtype, int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk,
                      int64_t b_sk, int64_t b_sn, int64_t c_sm, int int_bits, int frac_bits,
                      int k_tile, int split_k, int flags, void* scratch, int64_t scratch_bytes,
                      float* partials_out, int32_t* status_word, void* stream,
                      unsigned long long* best, int64_t n_offset) {
  if (M < 0 || N < 0 || K < 0) return FXPR_ERR_BAD_ARG;
  if (int_bits != 16 && int_bits != 32 && int_bits != 64) return FXPR_ERR_BAD_ARG;
  if (frac_bits < 0 || frac_bits >= 63) return FXPR_ERR_BAD_ARG;
  if (M == 0 || N == 0) return FXPR_OK;  // gemm.py:626-627
  if ((K > 0 && (!a || !b)) || (!c && !c_int)) return FXPR_ERR_BAD_ARG;
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return FXPR_ERR_BAD_ARG;
  if (dtype != FXPR_F16 && dtype != FXPR_BF16 && dtype != FXPR_F32) return FXPR_ERR_UNSUPPORTED;
  if (k_tile <= 0) k_tile = default_k_tile(dtype);
  if (split_k < 1) split_k = 1;
  if (split_k > 1 && partials_out) return FXPR_ERR_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;

  GemmArgs g;
  g.a = a; g.b = b; g.bias = bias; g.c = c; g.c_int = c_int; g.partials = partials_out;
  g.dtype = dtype; g.M = M; g.N = N; g.K = K;
  g.a_sm = a_sm; g.a_sk = a_sk; g.b_sk = b_sk; g.b_sn = b_sn; g.c_sm = c_sm;
  g.int_bits = int_bits; g.frac_bits = frac_bits; g.k_tile = k_tile; g.split_k = split_k;
  g.scratch = scratch; g.scratch_bytes = scratch_bytes; g.status = status_word; g.flags = flags;
  g.best = best; g.n_offset = n_offset;

  if (best) {
    if (!c || c_int || partials_out || n_offset < 0 || n_offset + N > 0xffffffffLL) return FXPR_ERR_BAD_ARG;
    if ((flags & FXPR_GEMM_FORCE_PORTABLE) || !gemm_tc_supported(g)) return FXPR_ERR_UNSUPPORTED;
    cudaError_t e = cudaMemsetAsync(best, 0, (size_t)M * sizeof(unsigned long long), s);
    if (e != cudaSuccess) { set_last_error("gemm_argmax memset", e); return FXPR_ERR_CUDA; }
  }
  if (flags & FXPR_GEMM_SILU_MUL) {
    if (!c || c_int || partials_out || (N & 1)) return FXPR_ERR_BAD_ARG;
    if ((flags & FXPR_GEMM_FORCE_PORTABLE) || !gemm_tc_supported(g)) return FXPR_ERR_UNSUPPORTED;
  }
  if (!(flags & FXPR_GEMM_FORCE_PORTABLE) && gemm_tc_supported(g)) return gemm_tc(g, s);
  return gemm_portable(a, b, bias, c, c_int, partials_out, dtype, M, N, K, a_sm, a_sk, b_sk, b_sn,
                       c_sm, int_bits, frac_bits, k_tile, s);
}

extern "C" int fxpr_gemm(const void* a, const void* b, const void* bias, void* c, void* c_int,
                         int dtype, int64_t M, int64_t N, int64_t K, int64_t a_sm, int64_t a_sk,
                         int64_t b_sk, int64_t b_sn, int64_t c_sm, int int_bits, int frac_bits,
                         int k_tile, int split_k, int flags, void* scratch, int64_t scratch_bytes,
                         float* partials_out, int32_t* status_word, void* stream) {
  return gemm_entry(a, b, bias, c, c_int, dtype, M, N, K, a_sm, a_sk, b_sk, b_sn, c_sm, int_bits, frac_bits,
                    k_tile, split_k, flags, scratch, scratch_bytes, partials_out, status_word, stream,
                    nullptr, 0);
}

extern "C" int fxpr_gemm_argmax(const void* a, const void* b, const void* bias, void* c, uint64_t* best,
                                int64_t n_offset, int dtype, int64_t M, int64_t N, int64_t K,
                                int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int64_t c_sm,
                                int int_bits, int frac_bits, int k_tile, int flags, int32_t* status_word,
                                void* stream) {
  if (!best) return FXPR_ERR_BAD_ARG;
  return gemm_entry(a, b, bias, c, nullptr, dtype, M, N, K, a_sm, a_sk, b_sk, b_sn, c_sm, int_bits, frac_bits,
                    k_tile, 1, flags, nullptr, 0, nullptr, status_word, stream,
                    reinterpret_cast<unsigned long long*>(best), n_offset);
}

extern "C" int64_t fxpr_attention_scratch_bytes(int64_t total_q_tokens, int num_heads, int head_dim,
                                                int int_bits, int num_splits) {
  (void)int_bits;
  if (num_splits <= 1 || total_q_tokens <= 0) return 0;
  return attn_scratch_layout(total_q_tokens, num_heads, head_dim, num_splits).total;
}

extern "C" int fxpr_attention(const void* q, const void* k_cache, const void* v_cache, void* o,
                              const int32_t* query_start_loc, const int32_t* seq_lens,
                              const int32_t* block_table, const float* alibi, int dtype,
                              int64_t total_q_tokens, int num_reqs, int num_heads, int num_kv_heads,
                              int head_dim, int page_size, int64_t q_st, int64_t q_sh, int64_t o_st,
                              int64_t o_sh, int64_t kv_sblock, int64_t kv_sslot, int64_t kv_shead,
                              int64_t bt_stride, int max_query_len, int flags, double softmax_scale,
                              double logit_softcap, int window, int int_bits, int frac_bits,
                              int num_splits, void* scratch, int64_t scratch_bytes,
                              int32_t* status_word, void* stream) {
  if (total_q_tokens < 0 || num_reqs < 0 || num_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 ||
      page_size <= 0 || window < 0)
    return FXPR_ERR_BAD_ARG;
  if (num_heads % num_kv_heads != 0) return FXPR_ERR_BAD_ARG;  // attention.py:743-744
  if (int_bits != 16 && int_bits != 32 && int_bits != 64) return FXPR_ERR_BAD_ARG;
  if (frac_bits < 0 || frac_bits >= 63) return FXPR_ERR_BAD_ARG;
  if (num_reqs == 0 || total_q_tokens == 0) return FXPR_OK;  // attention.py:745-746
  if (!q || !k_cache || !v_cache || !o || !query_start_loc || !seq_lens || !block_table)
    return FXPR_ERR_BAD_ARG;
  if (dtype != FXPR_F16 && dtype != FXPR_BF16 && dtype != FXPR_F32) return FXPR_ERR_UNSUPPORTED;
  if (num_splits < 1) num_splits = 1;
  cudaStream_t s = (cudaStream_t)stream;

  AttnParams p;
  p.q = q; p.k = k_cache; p.v = v_cache; p.o = o;
  p.qsl = query_start_loc; p.seq_lens = seq_lens; p.block_table = block_table; p.alibi = alibi;
  p.total_q = total_q_tokens; p.num_reqs = num_reqs; p.num_heads = num_heads;
  p.num_kv_heads = num_kv_heads; p.head_dim = head_dim; p.page_size = page_size;
  p.q_st = q_st; p.q_sh = q_sh; p.o_st = o_st; p.o_sh = o_sh;
  p.kv_sblock = kv_sblock; p.kv_sslot = kv_sslot; p.kv_shead = kv_shead; p.bt_stride = bt_stride;
  p.causal = (flags & FXPR_ATTN_CAUSAL) ? 1 : 0; p.window = window; p.int_bits = int_bits;
  p.num_splits = num_splits;
  // attention.py:748-750: scores live in log2 space
  p.ss_log2 = (float)(softmax_scale * 1.4426950408889634);
  p.cap_log2 = (float)(logit_softcap * 1.4426950408889634);
  p.scale = (float)(1ull << frac_bits);
  p.inv_scale = 1.0f / p.scale;
  p.partial_max = nullptr; p.total_denom = nullptr; p.total_wv = nullptr; p.locks = nullptr;
  p.status = status_word;

  // The tensor-core route merges its splits through distributed shared memory and needs
  // no scratch; only the CUDA-core route uses the caller's buffer.
  if (!(flags & FXPR_ATTN_FORCE_PORTABLE) && attention_mma_supported(p, dtype)) {
    const bool exact = (flags & FXPR_ATTN_EXACT_CONVERT) != 0;
    // prefill blocks without a KV split: tcgen05 kernel (same bits as the mma.sync kernel)
    if (!(flags & FXPR_ATTN_NO_TCGEN05) && attention_tc_supported(p, dtype, max_query_len, exact))
      return attention_tc(p, dtype, max_query_len, status_word, s);
    return attention_mma(p, dtype, max_query_len, exact, s);
  }
  if (num_splits > 1) {
    const AttnScratchLayout l = attn_scratch_layout(total_q_tokens, num_heads, head_dim, num_splits);
    if (!scratch || scratch_bytes < l.total) return FXPR_ERR_SCRATCH;
    if (((uintptr_t)scratch & 15) != 0) return FXPR_ERR_BAD_ARG;
    char* base = (char*)scratch;
    p.partial_max = (float*)(base + l.off_pmax);
    p.total_denom = (long long*)(base + l.off_denom);
    p.total_wv = (long long*)(base + l.off_wv);
    p.locks = (int32_t*)(base + l.off_locks);
    cudaError_t e = cudaMemsetAsync(base + l.zero_begin, 0, (size_t)l.zero_bytes, s);
    if (e != cudaSuccess) { set_last_error("attention scratch memset", e); return FXPR_ERR_CUDA; }
  }

  return attention_portable(p, dtype, s);
}

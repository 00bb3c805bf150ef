// Split-KV attention for callers that cannot allocate device memory.
//
// fxpr_attention() needs a scratch buffer for its split path (per-split row maxima,
// integer totals, arrival counters) and expects the caller to bring one.  Some
// callers have nowhere to get it from: a serving process that handed the whole
// HBM budget to its KV cache at start-up and has no allocator of its own on this
// code path, a plain C host without torch's caching allocator, or a latency-critical
// loop that must not risk the implicit device synchronisation of cudaMalloc/cudaFree.
// For them this file keeps the scratch in a fixed device array that is part of the
// library image: every GPU that loads the library holds these bytes until the
// process exits, so the size is kept modest and larger problems are refused.
#include <stdio.h>

#include "attention_common.cuh"
#include "fxp_common.cuh"

namespace fxpr {
void set_last_error_text(const char* text);
}

namespace {

constexpr long long kStaticScratchBytes = 4ll << 20;  // 4 MiB per GPU

// Device-resident scratch.  In HOST code this name is only a stand-in for the
// symbol, not a device address; the address is looked up once per device below.
static __device__ __align__(256) unsigned char g_attn_scratch[kStaticScratchBytes];

void* g_scratch_addr[64] = {nullptr};

// Once per device, with that device current: resolve the array's device address.
int static_scratch_ptr(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { fxpr::set_last_error("cudaGetDevice", e); return FXPR_ERR_CUDA; }
  if (dev < 0 || dev >= 64) return FXPR_ERR_BAD_ARG;
  if (!g_scratch_addr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_attn_scratch);
    if (e != cudaSuccess || !ptr) {
      fxpr::set_last_error("cudaGetSymbolAddress(static attention scratch)", e);
      return FXPR_ERR_CUDA;
    }
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return FXPR_OK;
}

}  // namespace

extern "C" int64_t fxpr_attention_static_scratch_capacity(void) { return kStaticScratchBytes; }

extern "C" int fxpr_attention_static_scratch(
    const void* q, const void* k_cache, const void* v_cache, void* o,
    const int32_t* query_start_loc, const int32_t* seq_lens, const int32_t* block_table,
    const float* alibi, int dtype, int64_t total_q_tokens, int num_reqs, int num_heads,
    int num_kv_heads, int head_dim, int page_size, int64_t q_st, int64_t q_sh, int64_t o_st,
    int64_t o_sh, int64_t kv_sblock, int64_t kv_sslot, int64_t kv_shead, int64_t bt_stride,
    int max_query_len, int flags, double softmax_scale, double logit_softcap, int window,
    int int_bits, int frac_bits, int num_splits, int32_t* status_word, void* stream) {
  void* scratch = nullptr;
  int64_t need = 0;
  // Only the CUDA-core route of fxpr_attention touches scratch memory (its split path keeps
  // per-split maxima, integer totals and arrival counters there); the tensor-core route
  // merges its splits inside a thread-block cluster.  So decide the route first, with the
  // rule fxpr_attention itself applies, and size, refuse and resolve the array only when
  // the call will really use it.
  bool uses_scratch = false;
  if (num_splits > 1 && total_q_tokens > 0 && num_reqs > 0 && num_heads > 0 && num_kv_heads > 0 &&
      head_dim > 0 && page_size > 0 && num_heads % num_kv_heads == 0) {
    fxpr::AttnParams rp{};
    rp.q = q; rp.k = k_cache; rp.v = v_cache;
    rp.num_reqs = num_reqs; rp.num_heads = num_heads; rp.num_kv_heads = num_kv_heads;
    rp.head_dim = head_dim; rp.page_size = page_size;
    rp.q_st = q_st; rp.q_sh = q_sh; rp.kv_sblock = kv_sblock; rp.kv_sslot = kv_sslot; rp.kv_shead = kv_shead;
    uses_scratch = (flags & FXPR_ATTN_FORCE_PORTABLE) || !fxpr::attention_mma_supported(rp, dtype);
  }
  if (uses_scratch) {
    need = fxpr::attn_scratch_layout(total_q_tokens, num_heads, head_dim, num_splits).total;
    if (need > kStaticScratchBytes) {
      char msg[200];
      snprintf(msg, sizeof(msg),
               "fxpr_attention_static_scratch: problem needs %lld bytes of scratch, the built-in "
               "buffer holds %lld; use fxpr_attention with caller-owned scratch",
               (long long)need, kStaticScratchBytes);
      fxpr::set_last_error_text(msg);
      return FXPR_ERR_SCRATCH;
    }
    const int rc = static_scratch_ptr(&scratch);
    if (rc != FXPR_OK) return rc;
  }
  // The existing entry point clears the regions that must start at zero
  // (cudaMemsetAsync on the caller's stream; no allocation) and launches.
  return fxpr_attention(q, k_cache, v_cache, o, query_start_loc, seq_lens, block_table, alibi, dtype,
                        total_q_tokens, num_reqs, num_heads, num_kv_heads, head_dim, page_size, q_st,
                        q_sh, o_st, o_sh, kv_sblock, kv_sslot, kv_shead, bt_stride, max_query_len,
                        flags, softmax_scale, logit_softcap, window, int_bits, frac_bits, num_splits,
                        scratch, scratch ? kStaticScratchBytes : 0, status_word, stream);
}

// Unified prefill + decode paged attention on tensor cores for fp16/bf16, head size
// 64/128, page sizes that are multiples of 16 and GQA groups of 1/2/4/8/16.
//
// Semantics: fxpr_vllm/_triton/attention.py of the reference (scores in log2 space
// :103-121, masks :199-215, exact row maximum first :233-257, w = exp2(s - max),
// integer denominator sum(Q(w)) and integer numerator sum over 64-key tiles of Q(P.V)
// :259-290, out = num / max(den, 1e-6) :292-301, split merge :618-652).
//
// B200 design:
//   * One CTA works on one KV head and a block of query rows; a row is a (token, query
//     head of the GQA group) pair, so K/V tiles are fetched once for all heads of the
//     group (the reference runs one program per query head).
//   * KV splits are the CTAs of one thread-block cluster: row maxima and the integer
//     partial sums are exchanged through distributed shared memory, so the split path
//     needs no global scratch, no atomics, and K and V are read exactly once.
//   * Decode (<= 16 rows per KV head) stashes the fp32 scores of its key slice in shared
//     memory during the max pass, so the second pass streams V only.  Prefill recomputes
//     Q.K^T in the second pass like the reference.
//   * 64-key tiles start at key 0 for every row block and split count, QK^T and P.V use
//     mma.sync.m16n8k16 with a fixed k order and each output row depends only on its own
//     query row, so a token's bits are the same in any batch, block or split.
//   * K/V pages are staged with 16-byte cp.async into XOR-swizzled shared memory.
#include <cooperative_groups.h>

#include "attention_common.cuh"
#include "fxp_common.cuh"

namespace cg = cooperative_groups;

namespace fxpr {

static constexpr int kTileN = 64;              // keys per tile (attention.py:32-36)

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;                // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ uint32_t pack2_io(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2_io<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2_io<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows hold
// ROW_CHUNKS chunks; XOR swizzle keeps ldmatrix and cp.async bank-conflict free.
template <int ROW_CHUNKS>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  return (uint32_t)((row * ROW_CHUNKS + (chunk ^ (row & 7))) * 16);
}

struct MmaAttnShape {
  int rows_per_token;      // GQA group size (power of two <= 16)
  int tokens_per_block;    // 16 * NW / rows_per_token
  int num_q_blocks;        // ceil(max_query_len / tokens_per_block)
  int stash_keys;          // keys of score stash per CTA (0 = recompute)
  int stash_rows;          // rows kept per key in the stash: <= 8, or 16
  int page_shift;          // log2(page_size) when it is a power of two, else -1
};

// Magic-number rounding of the second pass (attention_mma_pass_b_fast.inl)
static constexpr uint32_t kAttnMagicBits = 0x4B400000u;   // 1.5 * 2^23
static constexpr uint32_t kAttnExpBits = 0x4B000000u;     // sign 0, exponent 150: r in [2^23, 2^24)
static constexpr int kFastMaxTiles = 500;                 // 500 * 2^22 < 2^31: the 32-bit sums cannot wrap twice

#include "attention_mma_kernel.inl"
#include "attention_mma_decode.inl"

static int stash_bytes_per_key(int stash_rows) { return stash_rows <= 8 ? stash_rows * 4 : 64; }

template <typename T, int HD, int NW, bool STASH, bool ACC64, bool FAST = false>
static int launch_mma(const AttnParams& p, const MmaAttnShape& sh, cudaStream_t s) {
  constexpr int BM = 16 * NW;
  constexpr int kTileBytes = kTileN * HD * 2;
  constexpr int kStage = STASH ? kTileBytes : 2 * kTileBytes;
  constexpr int NSTAGE = STASH ? 3 : 2;
  size_t smem = (size_t)BM * HD * 2 + (size_t)NSTAGE * kStage + BM * 4 + BM * 8;
  if (STASH) smem += (size_t)sh.stash_keys * stash_bytes_per_key(sh.stash_rows);
  auto k = attn_mma_kernel<T, HD, NW, STASH, ACC64, FAST>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
  if (e != cudaSuccess) { set_last_error("attention_mma smem attribute", e); return FXPR_ERR_CUDA; }
  if (p.num_splits > 8) {
    e = cudaFuncSetAttribute(k, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) { set_last_error("attention_mma cluster attribute", e); return FXPR_ERR_CUDA; }
  }
  e = launch_pdl(k, dim3((unsigned)p.num_splits, (unsigned)(sh.num_q_blocks * p.num_kv_heads), (unsigned)p.num_reqs),
                 dim3(NW * 32), smem, s, (unsigned)p.num_splits, p, sh);
  if (e != cudaSuccess) { set_last_error("attention_mma launch", e); return FXPR_ERR_CUDA; }
  return check_launch("attention_mma");
}

template <typename T, int HD, int NW, bool ACC64, bool ROWS8, int NSTAGE = 2, int MINB = 4>
static int launch_decode(const AttnParams& p, const MmaAttnShape& sh, cudaStream_t s) {
  constexpr int kTileBytes = kTileN * HD * 2;
  const size_t smem = (size_t)(ROWS8 ? 8 : 16) * HD * 2 + NSTAGE * (size_t)kTileBytes + NW * 16 * 4 + NW * 16 * 8 +
                      (size_t)sh.stash_keys * stash_bytes_per_key(sh.stash_rows);
  auto k = attn_decode_kernel<T, HD, NW, ACC64, ROWS8, NSTAGE, MINB>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
  if (e != cudaSuccess) { set_last_error("attention_decode smem attribute", e); return FXPR_ERR_CUDA; }
  if (p.num_splits > 8) {
    e = cudaFuncSetAttribute(k, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) { set_last_error("attention_decode cluster attribute", e); return FXPR_ERR_CUDA; }
  }
  e = launch_pdl(k, dim3((unsigned)p.num_splits, (unsigned)(sh.num_q_blocks * p.num_kv_heads), (unsigned)p.num_reqs),
                 dim3(NW * 32), smem, s, (unsigned)p.num_splits, p, sh);
  if (e != cudaSuccess) { set_last_error("attention_decode launch", e); return FXPR_ERR_CUDA; }
  return check_launch("attention_decode");
}

static bool pow2_le16(int v) { return v == 1 || v == 2 || v == 4 || v == 8 || v == 16; }

bool attention_mma_supported(const AttnParams& p, int dtype) {
  if (dtype != FXPR_F16 && dtype != FXPR_BF16) return false;
  if (p.head_dim != 64 && p.head_dim != 128) return false;
  if (p.page_size % 16 != 0) return false;
  if (!pow2_le16(p.num_heads / p.num_kv_heads)) return false;
  // 16-byte cp.async: every row start must be 16-byte aligned
  const int64_t strides[] = {p.q_st, p.q_sh, p.kv_sblock, p.kv_sslot, p.kv_shead};
  for (int64_t st : strides) if (st % 8 != 0) return false;
  if (((uintptr_t)p.q | (uintptr_t)p.k | (uintptr_t)p.v) & 15) return false;
  if (p.num_kv_heads > 4096 || p.num_reqs > 65535) return false;
  return true;
}

int attention_mma(const AttnParams& p_in, int dtype, int max_query_len, bool force_exact, cudaStream_t s) {
  AttnParams p = p_in;
  if (p.num_splits > 16) p.num_splits = 16;        // cluster size limit; results do not depend on it
  if (p.num_splits < 1) p.num_splits = 1;
  const int G = p.num_heads / p.num_kv_heads;
  const int mq = max_query_len < 1 ? 1 : max_query_len;
  MmaAttnShape sh;
  sh.rows_per_token = G;
  sh.page_shift = -1;
  for (int b = 0; b < 30; ++b) if ((1 << b) == p.page_size) sh.page_shift = b;
  const bool small = (int64_t)mq * G <= 16;         // decode-like: one 16-row tile per KV head
  const int NW = small ? 1 : 4;
  sh.tokens_per_block = 16 * NW / G;
  sh.num_q_blocks = (mq + sh.tokens_per_block - 1) / sh.tokens_per_block;
  if ((int64_t)sh.num_q_blocks * p.num_kv_heads > 65535) return FXPR_ERR_UNSUPPORTED;
  const int rows = mq * G < 16 ? mq * G : 16;
  sh.stash_rows = rows <= 8 ? rows : 16;
  // upper bound on the keys one CTA can see: the block table's width
  const int64_t max_keys = p.bt_stride * (int64_t)p.page_size;
  const int64_t tiles = (max_keys + kTileN - 1) / kTileN;
  const int64_t per_rank = (tiles + p.num_splits - 1) / p.num_splits;
  sh.stash_keys = (int)(per_rank * kTileN);
  const bool stash = small && (int64_t)sh.stash_keys * stash_bytes_per_key(sh.stash_rows) <= 150 * 1024;
  if (!stash) sh.stash_keys = 0;
  const bool acc64 = p.int_bits == 64;
  // fast second pass (same bits): scale <= 2^16, 32- or 64-bit sums, bounded tiles per CTA
  const bool fast = !force_exact && p.scale <= 65536.0f && (p.int_bits == 32 || p.int_bits == 64) &&
                    per_rank <= kFastMaxTiles;

#define FXPR_ATTN(TT, HDV)                                                                      \
  do {                                                                                          \
    if (small && stash && sh.stash_rows <= 8)                                                   \
      return acc64 ? launch_decode<TT, HDV, 4, true, true>(p, sh, s)                     \
                   : launch_decode<TT, HDV, 4, false, true>(p, sh, s);                   \
    if (small && stash) return acc64 ? launch_decode<TT, HDV, 4, true, false>(p, sh, s)  \
                                     : launch_decode<TT, HDV, 4, false, false>(p, sh, s);\
    if (small) return acc64 ? launch_mma<TT, HDV, 1, false, true>(p, sh, s)                     \
                            : launch_mma<TT, HDV, 1, false, false>(p, sh, s);                   \
    if (fast) return launch_mma<TT, HDV, 4, false, false, true>(p, sh, s);                      \
    return acc64 ? launch_mma<TT, HDV, 4, false, true>(p, sh, s)                                \
                 : launch_mma<TT, HDV, 4, false, false>(p, sh, s);                              \
  } while (0)
  if (dtype == FXPR_BF16) {
    if (p.head_dim == 128) FXPR_ATTN(__nv_bfloat16, 128);
    FXPR_ATTN(__nv_bfloat16, 64);
  }
  if (p.head_dim == 128) FXPR_ATTN(__half, 128);
  FXPR_ATTN(__half, 64);
#undef FXPR_ATTN
}

}  // namespace fxpr

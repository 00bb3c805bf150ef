/*
 * fxpr_b200 -- C ABI of the B200 (sm_100a) fixed-point reduction kernels.
 *
 * Every entry point takes raw DEVICE pointers, plain sizes/strides, the Q-format
 * and a CUDA stream (a cudaStream_t passed as void*), launches on that stream,
 * never synchronises, never allocates (unless its comment says so) and returns
 * FXPR_OK or a negative status.  The library owns no memory: outputs and scratch
 * are the caller's (in the Python host layer they are torch tensors, so the
 * caching allocator and CUDA-graph capture keep working).
 *
 * Each entry replaces one launcher of the reference plugin fxpr_vllm (a pure
 * Python/Triton project, so the "FFI" it replaces is the Python call of a
 * `*_run` launcher from fxpr_vllm/_lib.py); the file:line beside each
 * declaration names that launcher.
 */
#ifndef FXPR_B200_H_
#define FXPR_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
#define FXPR_OK               0
#define FXPR_ERR_BAD_ARG     -1  /* null pointer, negative size, bad bit width    -> ValueError   */
#define FXPR_ERR_UNSUPPORTED -2  /* dtype / layout not implemented                -> TypeError    */
#define FXPR_ERR_SCRATCH     -3  /* scratch buffer missing or too small           -> RuntimeError */
#define FXPR_ERR_CUDA        -4  /* a CUDA runtime/driver call failed             -> RuntimeError */
#define FXPR_ERR_TIMEOUT     -5  /* a bounded device-side wait gave up            -> RuntimeError */
#define FXPR_ERR_ARCH        -6  /* device is not compute capability 10.x         -> RuntimeError */

/* ---- element types ----------------------------------------------------- */
#define FXPR_F16  0
#define FXPR_BF16 1
#define FXPR_F32  2
#define FXPR_F64  3

/* ---- gemm flags -------------------------------------------------------- */
#define FXPR_GEMM_FORCE_PORTABLE 1  /* route to the CUDA-core kernel (sequential-k partials) */
#define FXPR_GEMM_FORCE_EXACT_TC 2  /* tensor-core kernel with the plain cvt.rni epilogue */
#define FXPR_GEMM_NO_SKINNY      8  /* M <= 64: use the 128-row-tile kernel anyway (tests: same bits) */
#define FXPR_GEMM_NO_CLUSTER     16 /* M <= 64 split-K: partial planes in the scratch instead of a cluster merge (tests) */
#define FXPR_GEMM_TILE_N256       64 /* force 128 x 256 output tiles (same bits) */
#define FXPR_GEMM_TILE_N128       128 /* force 128 x 128 output tiles (same bits) */
#define FXPR_GEMM_SILU_MUL        1024 /* B's columns are (gate_j, up_j) pairs; c is [M, N/2] = silu(gate) * up, computed from the GEMM outputs as the io dtype holds them (same bits as fxpr_gemm + fxpr_silu_mul_pairs); M <= 64 on the tensor-core decode route with c_int == NULL, else FXPR_ERR_UNSUPPORTED */
#define FXPR_GEMM_WEIGHTS_STATIC  2048 /* the caller vouches that b was complete before this launch was enqueued behind its predecessor (model weights): the decode-shape kernel may then fetch its first weight tiles while the previous kernel of the stream is still running (programmatic dependent launch) */
#define FXPR_GEMM_PAIR            512 /* two-SM kernel (gemm_tc_pair.cu): 256 x BN tiles on CTA pairs, tcgen05 cta_group::2; same bits, opt-in */

/* ---- attention flags --------------------------------------------------- */
#define FXPR_ATTN_CAUSAL         1
#define FXPR_ATTN_FORCE_PORTABLE 2  /* route to the CUDA-core kernel (sequential partials) */
#define FXPR_ATTN_EXACT_CONVERT  4  /* tensor-core route with cvt.rni.sat conversions only (tests: same bits as the default) */
#define FXPR_ATTN_NO_TCGEN05     8  /* prefill on the mma.sync kernel instead of the tcgen05 one (tests: same bits) */

int fxpr_version(void);
const char* fxpr_status_string(int status);

/* Last CUDA error text recorded by this library on the calling thread ("" if none). */
const char* fxpr_last_error(void);

/*
 * y[i] = saturate(rint_half_even(fp32(x[i]) * 2^frac_bits)) as int{16,32,64}.
 * x_dtype in {FXPR_F16, FXPR_F32, FXPR_F64}; n elements, both contiguous.
 * Replaces float_to_fixed_run, fxpr_vllm/_triton/casts.py:57-89
 * (device math fxpr_vllm/_triton/fxp.py:92-108).
 */
int fxpr_float_to_fixed(const void* x, int x_dtype, void* y, int int_bits,
                        int frac_bits, int64_t n, void* stream);

/*
 * y[i] = T(fp32(x[i]) * 2^-frac_bits), x int{16,32,64}, T = fp{16,32,64}.
 * Replaces fixed_to_float_run, fxpr_vllm/_triton/casts.py:92-126.
 */
int fxpr_fixed_to_float(const void* x, int int_bits, void* y, int float_bits,
                        int frac_bits, int64_t n, void* stream);

/*
 * RMSNorm over rows of a contiguous [rows, hidden] matrix, optional fused
 * residual add (residual != NULL: residual <- T(x + residual) in place, and the
 * rounded sum is what gets normalised).  The sum of squares is an int64 sum of
 * Q(frac_bits) integers; mean, 1/sqrt and the scaling are single IEEE
 * operations.  dtype in {FXPR_F16, FXPR_BF16, FXPR_F32}; weight has that dtype.
 * Replaces _common_launch, fxpr_vllm/_triton/rms_norm.py:78-134 (whose kernel
 * sums in fp32, rms_norm.py:38-50).
 */
int fxpr_rms_norm(const void* x, void* residual, const void* weight, void* y,
                  int dtype, int64_t rows, int64_t hidden, float eps,
                  int frac_bits, void* stream);

/*
 * The step after a tensor-parallel row-parallel GEMM in one kernel: acc is the
 * all-reduced integer accumulator tensor [rows, hidden] (int{int_bits}, Q(gemm_frac_bits),
 * as fxpr_gemm's c_int), and the kernel does what fxpr_gemm_epilogue_from_int followed by
 * fxpr_rms_norm with a residual do, with the same roundings in the same order:
 * x = T(fp32(acc) * 2^-gemm_frac_bits + bias), residual <- T(x + residual) in place,
 * y = RMSNorm(residual) with the integer sum of squares (Q(frac_bits), int64).
 * bias may be NULL.  Rows longer than 16384 elements return FXPR_ERR_UNSUPPORTED (use
 * the two calls).  No counterpart in the reference (its plugin leaves the reduce to
 * vLLM's float all-reduce, vllm/model_executor/layers/linear.py).
 */
int fxpr_rms_norm_from_int(const void* acc, int int_bits, const void* bias,
                           void* residual, const void* weight, void* y, int dtype,
                           int64_t rows, int64_t hidden, float eps,
                           int gemm_frac_bits, int frac_bits, void* stream);

/*
 * Tensor-parallel row-parallel layers without a library collective: the cross-rank integer
 * sum, fxpr_rms_norm_from_int's arithmetic and the distribution of the result as ONE kernel
 * per rank over peer-mapped memory (plain loads and stores over NVLink; no multicast).  Same
 * bits as ncclAllReduce(sum) on the accumulators followed by fxpr_rms_norm_from_int, for any
 * rank count.  No counterpart in the reference (vLLM's float all-reduce follows its
 * quant_method.apply, vllm/model_executor/layers/linear.py); the integer ncclAllReduce of
 * fxpr_vllm/tp.py stays the default exchange.
 *
 * Each rank owns one buffer: accumulators [max_rows, hidden] int{int_bits} | residual
 * [max_rows, hidden] | output [max_rows, hidden] (io dtype) | 32 flag words, at the offsets
 * fxpr_tp_buffer_bytes reports.  fxpr_tp_alloc makes a zeroed cudaMalloc buffer on the current
 * device and its 64-byte CUDA IPC handle; fxpr_tp_open maps a peer's handle into the current
 * device's context (lazy peer access); fxpr_tp_close / fxpr_tp_free undo them.
 *
 * fxpr_tp_reduce_norm: peer_bases[world] are the buffers as mapped in THIS process
 * (peer_bases[rank] is the local one); ctl points to two zero-initialised 32-bit words in local
 * device memory that the kernel owns (call counter, CTA arrivals).  Before the call this
 * rank's accumulators [rows, hidden] are complete in its buffer (same stream) and its residual
 * rows are current; after it every rank's residual and output regions hold all rows.  Rank r
 * reduces rows [r * ceil(rows / world), ...).  All ranks must issue the same sequence of calls.
 * Waits last at most timeout_cycles SM clocks (<= 0: about a second); when one runs out the
 * kernel writes FXPR_ERR_TIMEOUT to *status and stops touching peer memory; the buffers must
 * then be re-created.  int_bits 32 or 64; hidden a multiple of 4, at most 16384.  flags:
 * FXPR_TP_LOCAL_RESIDUAL -- the new residual rows are written to this rank's buffer only (for
 * callers that keep the residual row-sharded: a rank only ever reads the residual of its own rows).
 */
#define FXPR_TP_LOCAL_RESIDUAL 1
int fxpr_tp_buffer_bytes(int64_t max_rows, int64_t hidden, int int_bits, int dtype,
                         int64_t* acc_offset, int64_t* residual_offset, int64_t* y_offset,
                         int64_t* flags_offset, int64_t* total);
int fxpr_tp_alloc(int64_t bytes, void** ptr, void* handle64);
int fxpr_tp_open(const void* handle64, void** ptr);
int fxpr_tp_close(void* ptr);
int fxpr_tp_free(void* ptr);
int fxpr_tp_reduce_norm(const void* const* peer_bases, int world, int rank, void* ctl,
                        int64_t acc_offset, int64_t residual_offset, int64_t y_offset,
                        int64_t flags_offset, int int_bits, const void* bias, const void* weight,
                        int dtype, int64_t rows, int64_t hidden, float eps, int gemm_frac_bits,
                        int frac_bits, int64_t timeout_cycles, int flags, int32_t* status,
                        void* stream);

/*
 * Row-wise log-softmax of a contiguous [rows, cols] matrix into fp32:
 * y = (x - max) - log(sum_int64(Q(exp(x - max)))).  x_dtype in
 * {FXPR_F16, FXPR_BF16, FXPR_F32}.  No counterpart in the reference (the
 * sampler files its README lists are absent); hook point is vLLM's
 * Sampler.compute_logprobs.
 */
int fxpr_log_softmax(const void* x, int x_dtype, float* y, int64_t rows,
                     int64_t cols, int frac_bits, void* stream);

/*
 * Bytes of scratch fxpr_gemm needs for this problem (0 when split_k <= 1):
 * tile counters followed by one plane of integer partial tiles per split.
 * The buffer must be zero-filled once before its first use; after that it may
 * be reused, without clearing, for calls of any shape that it is large enough
 * for (calls that share a buffer must be ordered on one stream).
 * Replaces _get_splitk_scratch, fxpr_vllm/_triton/gemm.py:86-107.
 */
int64_t fxpr_gemm_scratch_bytes(int64_t M, int64_t N, int int_bits, int split_k);

/*
 * C[M,N] = T( fp32( sum_t Q( fp32dot(A[:, tile t], B[tile t, :]) ) ) * 2^-frac + bias ).
 * a: (M,K) element strides a_sm,a_sk.  b: (K,N) strides b_sk,b_sn.  c: (M,N)
 * row stride c_sm, unit column stride; may be NULL when only c_int is wanted.
 * c_int: optional contiguous [M,N] int{int_bits} receiving the integer
 * accumulators (for the tensor-parallel reduce and for tests).
 * k_tile: conversion granularity (0 = reference default: 128 for f16/bf16, 64
 * for f32).  split_k: 0/1 = none, else the K-tiles are dealt round-robin to
 * split_k CTAs per output tile; each leaves an integer partial tile in the
 * scratch and the last to arrive adds them up (order-free, needs scratch).
 * partials_out: optional fp32 [ceil(K/k_tile), M, N] dump of the per-tile
 * float partials (tests only; must be NULL when split_k > 1).
 * status_word: optional device int the tensor-core kernel sets to
 * FXPR_ERR_TIMEOUT if one of its bounded mbarrier waits gave up (the output is
 * then undefined); the host reads it when it next synchronises.
 * Replaces gemm_fxp_run, fxpr_vllm/_triton/gemm.py:612-763.
 */
int fxpr_gemm(const void* a, const void* b, const void* bias, void* c, void* c_int,
              int dtype, int64_t M, int64_t N, int64_t K,
              int64_t a_sm, int64_t a_sk, int64_t b_sk, int64_t b_sn, int64_t c_sm,
              int int_bits, int frac_bits, int k_tile, int split_k, int flags,
              void* scratch, int64_t scratch_bytes, float* partials_out,
              int32_t* status_word, void* stream);

/*
 * c = T(fp32(c_int) * 2^-frac + bias): the GEMM epilogue applied to integer
 * accumulators that were summed across tensor-parallel ranks.  c_int is a
 * contiguous [M,N] int{int_bits}.  Same formula as gemm.py:195-204.
 */
int fxpr_gemm_epilogue_from_int(const void* c_int, int int_bits, const void* bias,
                                void* c, int dtype, int64_t M, int64_t N,
                                int64_t c_sm, int frac_bits, void* stream);

/*
 * Bytes of scratch fxpr_attention needs (any contents; the call initialises
 * what it uses).  Replaces the per-call torch.full/zeros of
 * fxpr_vllm/_triton/attention.py:838-851.
 */
int64_t fxpr_attention_scratch_bytes(int64_t total_q_tokens, int num_heads,
                                     int head_dim, int int_bits, int num_splits);

/*
 * Unified prefill + decode attention over a paged KV cache with integer
 * softmax denominator and P.V numerator.
 * q,o: [T, Hq, D] (token/head strides in elements, unit stride in D).
 * kv_cache: [num_blocks, 2, page, Hkv, D] given as separate K and V base
 * pointers plus block/slot/head strides (elements).  query_start_loc [R+1],
 * seq_lens [R], block_table [R, bt_stride] int32.  alibi: fp32 [Hq] slopes
 * already multiplied by log2(e), or NULL.  softmax_scale is the plain scale
 * (the call multiplies by log2(e)).  logit_softcap 0 = off, window 0 = off.
 * num_splits >= 1 (the host picks it).  status_word: optional device int set
 * non-zero by a kernel that gave up on a bounded wait.
 * Replaces unified_attention_fxp_run, fxpr_vllm/_triton/attention.py:692-953.
 */
int fxpr_attention(const void* q, const void* k_cache, const void* v_cache, void* o,
                   const int32_t* query_start_loc, const int32_t* seq_lens,
                   const int32_t* block_table, const float* alibi,
                   int dtype, int64_t total_q_tokens, int num_reqs, int num_heads,
                   int num_kv_heads, int head_dim, int page_size,
                   int64_t q_st, int64_t q_sh, int64_t o_st, int64_t o_sh,
                   int64_t kv_sblock, int64_t kv_sslot, int64_t kv_shead,
                   int64_t bt_stride, int max_query_len, int flags,
                   double softmax_scale, double logit_softcap, int window,
                   int int_bits, int frac_bits, int num_splits,
                   void* scratch, int64_t scratch_bytes, int32_t* status_word,
                   void* stream);

/*
 * fxpr_attention for callers that cannot allocate device memory.  It has no
 * counterpart in the reference (whose launcher allocates scratch with torch on
 * every call).  Same arguments as fxpr_attention without scratch/scratch_bytes:
 * the split path's scratch lives in a fixed device array inside the library,
 * fxpr_attention_static_scratch_capacity() bytes (4 MiB) on every GPU that
 * loads the library, held until the process exits.  Meant for hosts with no
 * allocator on this path: a server that gave all of HBM to its KV cache, a C
 * caller without torch, a loop that must avoid cudaMalloc's implicit
 * synchronisation.  It calls no cudaMalloc/cudaFree and no allocating library.
 *   - Only the CUDA-core route uses scratch at all (fp32 inputs, head sizes
 *     other than 64/128, pages that are not a multiple of 16 tokens, or
 *     FXPR_ATTN_FORCE_PORTABLE); the tensor-core route merges its splits inside a
 *     thread-block cluster and never touches the array, whatever the sizes.
 *   - Calls on the CUDA-core route whose scratch need
 *     (fxpr_attention_scratch_bytes) exceeds the capacity are refused with
 *     FXPR_ERR_SCRATCH and a message in fxpr_last_error(); nothing is launched.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call
 *     before any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents;
 *     each call clears what must start at zero on the given stream.  Two calls
 *     whose kernels can overlap on the GPU (different streams) race on it:
 *     serialise them.
 */
int64_t fxpr_attention_static_scratch_capacity(void);
int fxpr_attention_static_scratch(
                   const void* q, const void* k_cache, const void* v_cache, void* o,
                   const int32_t* query_start_loc, const int32_t* seq_lens,
                   const int32_t* block_table, const float* alibi,
                   int dtype, int64_t total_q_tokens, int num_reqs, int num_heads,
                   int num_kv_heads, int head_dim, int page_size,
                   int64_t q_st, int64_t q_sh, int64_t o_st, int64_t o_sh,
                   int64_t kv_sblock, int64_t kv_sslot, int64_t kv_shead,
                   int64_t bt_stride, int max_query_len, int flags,
                   double softmax_scale, double logit_softcap, int window,
                   int int_bits, int frac_bits, int num_splits,
                   int32_t* status_word, void* stream);

/*
 * fxpr_gemm for at most 64 rows that also leaves, per row, the arg-max of the outputs (greedy
 * sampling straight from the lm_head without a pass over the logits; no reference counterpart):
 * best[m] (zeroed by the call) becomes the maximum over columns n of the key
 * (order-preserving bits of c[m, n] as the io dtype holds it) << 32 | (0xFFFFFFFF - (n_offset + n)),
 * so the winning column is 0xFFFFFFFF - (best[m] & 0xFFFFFFFF): the largest output, the
 * smallest column among equals (torch.argmax's rule).  Keys of column shards (vocab-parallel
 * lm_head: n_offset = first column of the shard) combine by a plain integer maximum.  c is
 * still written.  Tensor-core decode route only (split_k 1), else FXPR_ERR_UNSUPPORTED.
 */
int fxpr_gemm_argmax(const void* a, const void* b, const void* bias, void* c, uint64_t* best,
                     int64_t n_offset, int dtype, int64_t M, int64_t N, int64_t K, int64_t a_sm,
                     int64_t a_sk, int64_t b_sk, int64_t b_sn, int64_t c_sm, int int_bits,
                     int frac_bits, int k_tile, int flags, int32_t* status_word, void* stream);

/*
 * Decoder-layer element-wise steps around the attention call (no reductions).
 *
 * fxpr_rope_kv_write: qkv is [tokens, (q_heads + 2 kv_heads) * head_dim] (Q heads, K heads,
 * V heads).  Rotate-half RoPE in fp32 with cos/sin tables [max_pos, head_dim / 2]; rotated Q
 * goes to q_out [tokens, q_heads, head_dim], rotated K and V go into the paged cache at
 * block_table[seq_ids[t], positions[t] / page_size], slot positions[t] % page_size.  The
 * cache strides are in elements (block, K-to-V plane, slot, head).  Replaces vLLM's
 * reshape_and_cache_flash call of fxpr_vllm/attention_backend.py:253-277 plus the RoPE op
 * before it.
 * fxpr_silu_mul: out[r, c] = silu(gate_up[r, c]) * gate_up[r, f + c] for a fused [rows, 2 f]
 * activation (vLLM's SiluAndMul).  fxpr_silu_mul_pairs: the same for a [rows, 2 f] activation
 * whose columns are (gate_j, up_j) pairs, the layout FXPR_GEMM_SILU_MUL expects of its weights.
 */
int fxpr_rope_kv_write(const void* qkv, int dtype, const float* cos_table, const float* sin_table,
                       const int64_t* positions, const int64_t* seq_ids,
                       const int32_t* block_table, int64_t bt_stride, void* q_out,
                       void* kv_cache, int64_t tokens, int q_heads, int kv_heads,
                       int head_dim, int page_size, int64_t kv_sblock, int64_t kv_skv,
                       int64_t kv_sslot, int64_t kv_shead, void* stream);
int fxpr_silu_mul(const void* gate_up, int dtype, void* out, int64_t rows, int64_t f,
                  void* stream);
int fxpr_silu_mul_pairs(const void* gate_up, int dtype, void* out, int64_t rows, int64_t f,
                        void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FXPR_B200_H_ */

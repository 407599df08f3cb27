/*
 * b200_decode.h — C ABI of libb200decode.so
 *
 * The drop-in boundary of the B200-native decode hot path.
 * Every entry point takes raw DEVICE pointers, int64 shapes/strides counted in
 * ELEMENTS (not bytes), plain scalars and the CUDA stream to launch on.  No
 * torch types cross this boundary.  Every function returns B200_OK (0) or a
 * negative b200_status; nothing here aborts the process, allocates device
 * memory behind the caller's back, synchronises the host with the device or
 * reads device metadata on the host, so every call is CUDA-graph capturable
 * (the reference contract: src/engine/model_runner.cpp:141-210).
 *
 * Each declaration cites the reference interface it replaces (paths relative
 * to the ScaleLLM tree @ffee4ffd).  INTEGRATION.md shows the reference-side
 * binding (C++ shim with the reference's own signatures, and the ctypes stub).
 */
#ifndef B200_DECODE_H_
#define B200_DECODE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define B200_API
#else
#define B200_API __attribute__((visibility("default")))
#endif

/* Opaque cudaStream_t (CUstream).  0 / NULL = legacy default stream. */
typedef void* b200_stream_t;

typedef enum b200_status {
  B200_OK = 0,
  B200_ERR_INVALID_ARG = -1,  /* bad shape / alignment / null pointer          */
  B200_ERR_UNSUPPORTED = -2,  /* valid in the reference, not implemented here  */
  B200_ERR_CUDA = -3,         /* a CUDA runtime/driver call failed             */
  B200_ERR_WORKSPACE = -4     /* caller's workspace too small                  */
} b200_status;

/* Element types of activations / caches. */
typedef enum b200_dtype {
  B200_BF16 = 0,
  B200_FP16 = 1,
  B200_FP32 = 2 /* elementwise + norm kernels only */
} b200_dtype;

/* Library ABI version (bumped on any signature change). */
B200_API int b200_abi_version(void);

/* Human readable description of the last error on the calling thread. */
B200_API const char* b200_last_error(void);

/* Number of kernels this library launched on the calling thread since the
 * last reset (bench.py's "gpu_launches" claim is read from here). */
B200_API int64_t b200_launch_count(void);
B200_API void b200_launch_count_reset(void);

/* ------------------------------------------------------------------------ *
 * A4  RMSNorm                       src/kernels/layernorm_kernels.h:6-19
 *     out = T(x * rsqrt(mean(x^2) + eps)) * w          (layernorm_kernels.cu:15-41)
 *     residual form: r = r + x (stored), then the same on r   (:125-155)
 *     in/out/residual: [rows, n] contiguous; weight: [n].
 * ------------------------------------------------------------------------ */
B200_API int b200_rms_norm(void* out, const void* in, const void* weight,
                           int64_t rows, int64_t n, float eps, int dtype,
                           b200_stream_t stream);

B200_API int b200_rms_norm_residual(void* out, void* residual, const void* in,
                                    const void* weight, int64_t rows, int64_t n,
                                    float eps, int dtype, b200_stream_t stream);

/* ------------------------------------------------------------------------ *
 * A3  Rotary embedding, in place    src/kernels/pos_embedding_kernels.h:7-13
 *     q: [n_tokens, n_heads, head_dim]   (token stride q_stride, heads dense)
 *     k: [n_tokens, n_kv_heads, head_dim](token stride k_stride, heads dense)
 *     positions: [n_tokens] int32
 *     cos_sin:  [max_pos, rotary_dim] = [cos(rotary_dim/2) | sin(rotary_dim/2)]
 *     every multiply / add rounded to the element type (pos_embedding_kernels.cu:24-29)
 * ------------------------------------------------------------------------ */
B200_API int b200_rope_inplace(void* q, void* k, const int32_t* positions,
                               const void* cos_sin, int64_t n_tokens,
                               int64_t n_heads, int64_t n_kv_heads,
                               int64_t head_dim, int64_t rotary_dim,
                               int64_t q_stride, int64_t k_stride,
                               int interleaved, int dtype, b200_stream_t stream);

/* Debug / test hook (host arithmetic only): the work partition b200_paged_attn_decode would use.
 * out[8] = {impl (0 simt, 1 mma, 2 stream), n_splits, tiles per warp, padded tiles per
 * (sequence, row block, kv head), number of those, row blocks, total tiles, block-table window}. */
B200_API int b200_debug_attn_plan(int64_t batch, int max_q_len, int max_kv_len, int n_heads,
                                  int n_kv_heads, int head_dim, int block_size, int64_t* out);

/* ------------------------------------------------------------------------ *
 * A2  KV-cache slot write           src/kernels/kv_cache_kernels.h:6-11
 *     cache[slot_ids[t], h, :] = {k,v}[t, h, :]        (bit exact)
 *     k,v: [n_tokens, n_kv_heads, head_dim], token strides k_stride/v_stride
 *     caches: [n_slots, n_kv_heads, head_dim] contiguous
 * ------------------------------------------------------------------------ */
B200_API int b200_kv_write(const int32_t* slot_ids, const void* k, const void* v,
                           void* k_cache, void* v_cache, int64_t n_tokens,
                           int64_t n_kv_heads, int64_t head_dim,
                           int64_t k_stride, int64_t v_stride, int dtype,
                           b200_stream_t stream);

/* Fusion of A3 + A2 (ScaleAttnHandler::apply_pos_emb + append_kv_cache,
 * src/layers/attention/scale_attn_handler.cpp:31-42,71-84): rotates q and k in
 * place AND scatters rotated k plus v into the cache in one pass.  Results are
 * bit-identical to b200_rope_inplace followed by b200_kv_write. */
B200_API int b200_rope_kv_write(void* q, void* k, const void* v,
                                const int32_t* positions, const void* cos_sin,
                                const int32_t* slot_ids, void* k_cache,
                                void* v_cache, int64_t n_tokens, int64_t n_heads,
                                int64_t n_kv_heads, int64_t head_dim,
                                int64_t rotary_dim, int64_t q_stride,
                                int64_t k_stride, int64_t v_stride,
                                int interleaved, int dtype, b200_stream_t stream);

/* Gather (test/debug helper; KVCache::get_kv_cache, src/memory/kv_cache.cpp:60-98):
 * {k,v}_out[t] = cache[slot_ids[t]]. */
B200_API int b200_kv_gather(const int32_t* slot_ids, const void* k_cache,
                            const void* v_cache, void* k_out, void* v_out,
                            int64_t n_tokens, int64_t n_kv_heads,
                            int64_t head_dim, int dtype, b200_stream_t stream);

/* ------------------------------------------------------------------------ *
 * A5  Activations                   src/kernels/activation_kernels.h:6-14
 *     silu:      out[r, i] = T(x / (1 + exp(-x)))            in: [rows, n], row stride in_stride
 *     silu_mul:  out[r, i] = T(silu(in[r, i])) * in[r, n+i]   in: [rows, 2n] contiguous
 *     (two roundings, activation_kernels.cu:44-50,84-95)
 * ------------------------------------------------------------------------ */
B200_API int b200_silu(void* out, const void* in, int64_t rows, int64_t n,
                       int64_t in_stride, int dtype, b200_stream_t stream);

B200_API int b200_silu_mul(void* out, const void* in, int64_t rows, int64_t n,
                           int dtype, b200_stream_t stream);

/* silu(gate) * up with gate and up given as separate strided views — the exact
 * op pair Llama's MLP issues (src/models/meta/llama.h:61-64): kernel::silu then
 * a torch multiply.  gate/up: [rows, n] with row strides; out contiguous. */
B200_API int b200_silu_mul_strided(void* out, const void* gate, const void* up,
                                   int64_t rows, int64_t n, int64_t gate_stride,
                                   int64_t up_stride, int dtype,
                                   b200_stream_t stream);
/* Adjacent operators of the same reference link target (:kernels), so that a link-time swap also
 * resolves for the reference's Gemma / GPT-2 / Phi models — bit-identical to the reference kernels,
 * not on the benchmarked path:
 *   gemma_rms_norm  out = (T)(x * rstd * (1.0 + w))           src/kernels/layernorm_kernels.cu:66-123
 *   layer_norm      out = (T)((x - mean) * rstd * w (+ b))     src/kernels/layernorm_kernels.cu:185-260
 *   gelu            act 1 = gelu_new, 2 = gelu_fast (tanh.approx), optionally * up
 *                                                             src/kernels/activation_kernels.cu:13-41,108-145 */
B200_API int b200_gemma_rms_norm(void* out, const void* in, const void* weight, int64_t rows,
                                 int64_t n, float eps, int dtype, b200_stream_t stream);
B200_API int b200_layer_norm(void* out, const void* in, const void* weight, const void* bias /*nullable*/,
                             int64_t rows, int64_t n, float eps, int dtype, b200_stream_t stream);
B200_API int b200_gelu(void* out, const void* in, int64_t rows, int64_t n, int64_t in_stride, int act,
                       int with_mul, int dtype, b200_stream_t stream);


/* ------------------------------------------------------------------------ *
 * A1  Paged-KV variable-length attention (decode-shaped)
 *                                   src/kernels/attention/attn_api.h:12-27
 *     O = softmax(mask(softcap(Q K^T * sm_scale) + alibi)) V per sequence,
 *     causal with diagonal kv_len - q_len, slot lookup
 *     block_table[block_cu_lens[b] + (idx >> log2(bs))] + (idx & (bs-1))
 *     (block_table holds FIRST-SLOT ids: block_id * block_size;
 *      src/kernels/attention/kernel/sm80_kernel_mha.cuh:148-152, src/engine/batch.cpp:206-209)
 *
 *     out, q:  [n_tokens, n_heads, head_dim], strides (q_stride_t, q_stride_h, 1)
 *     caches:  [n_slots, n_kv_heads, head_dim], strides (kv_stride_s, kv_stride_h, 1)
 *     head_dim in {64, 128, 256} (tensor-core kernels) or {32, 96} (CUDA-core kernel; the
 *     reference pads these into its 64 / 128 tiles, common/static_dispatch.h:16-46); bf16 / fp16
 *     q_cu_lens, kv_cu_lens, block_cu_lens: [batch+1] int32;  block_table int32
 *     alibi_slopes: [n_heads] float32 or NULL
 *     sliding_window < 0 disables the local mask; logits_soft_cap == 0 disables it.
 *     workspace: device scratch for split-KV partials, at least
 *     b200_paged_attn_workspace_bytes(...) bytes, 16-byte aligned (may be NULL
 *     when that function returns 0).
 *     Every query token of a sequence is processed as its own work item, which is
 *     the right shape for decode / speculative decode (max_q_len <= ~8); large
 *     q_len (prefill) is correct but not the tuned path.
 * ------------------------------------------------------------------------ */
B200_API int64_t b200_paged_attn_workspace_bytes(int64_t batch, int64_t max_q_len,
                                                 int64_t max_kv_len,
                                                 int64_t n_heads,
                                                 int64_t n_kv_heads,
                                                 int64_t head_dim);

B200_API int b200_paged_attn_decode(
    void* out, const void* q, const void* k_cache, const void* v_cache,
    const int32_t* q_cu_lens, const int32_t* kv_cu_lens,
    const int32_t* block_table, const int32_t* block_cu_lens,
    const float* alibi_slopes, int64_t batch, int64_t n_heads,
    int64_t n_kv_heads, int64_t head_dim, int64_t n_slots, int64_t q_stride_t,
    int64_t q_stride_h, int64_t o_stride_t, int64_t o_stride_h,
    int64_t kv_stride_s, int64_t kv_stride_h, int block_size, int max_q_len,
    int max_kv_len, float sm_scale, float logits_soft_cap, int sliding_window,
    void* workspace, int64_t workspace_bytes, int dtype, b200_stream_t stream);

/* ------------------------------------------------------------------------ *
 * A6/A7  int4 weight x bf16 activation matmul (W4A16)
 *     replaces marlin::awq_repack / gptq_repack + marlin::gptq_gemm
 *     (src/kernels/quantization/marlin.h:17-37) behind the qlinear plugins
 *     (src/layers/quantization/qlinear_awq_marlin_impl.cpp:99-125,332-365).
 *
 *     C[M,N] = A[M,K] * W,   W[k,n] = bf16_mul( bf16(q[k,n]) - bf16(z[k/g,n]), s[k/g,n] )
 *     (exact subtract, one bf16 rounding in the multiply: marlin/numeric_conversion.h:144-167,221-240),
 *     fp32 accumulate, fp32 cross-CTA reduction, one final rounding to bf16.
 *
 *     Checkpoint formats accepted by the prepack calls (device pointers):
 *       AWQ : qweight [K, N/8] int32, nibbles along N in order [0,2,4,6,1,3,5,7];
 *             qzeros [K/g, N/8] int32 same packing; scales [K/g, N] bf16
 *             (tests/kernels/quant_utils.py:177-197)
 *       GPTQ: qweight [K/8, N] int32, nibbles along K in natural order
 *             (quant_utils.py:101-115); symmetric zero point 8 when qzeros == NULL
 *             (qlinear_gptq_marlin_impl.cpp:18-20), else qzeros [K/g, N/8] int32
 *             natural order with the GPTQ-v1 "+1" convention applied iff
 *             zeros_plus_one != 0 (src/layers/quantization/qlinear_impl.cpp:44,86);
 *             g_idx (act-order) is not supported: B200_ERR_UNSUPPORTED.
 *     group_size g in {32, 64, 128, -1(=K)};  K % 128 == 0, N % 128 == 0.
 *
 *     The prepacked buffer is an opaque tile-blob layout private to this
 *     library (DESIGN.md "W4 tile blob"); size from b200_w4a16_packed_bytes.
 * ------------------------------------------------------------------------ */
B200_API int64_t b200_w4a16_packed_bytes(int64_t K, int64_t N, int group_size);

B200_API int b200_w4a16_prepack_awq(void* packed, const int32_t* qweight,
                                    const int32_t* qzeros, const void* scales,
                                    int64_t K, int64_t N, int group_size,
                                    b200_stream_t stream);

B200_API int b200_w4a16_prepack_gptq(void* packed, const int32_t* qweight,
                                     const int32_t* qzeros, const void* scales,
                                     int64_t K, int64_t N, int group_size,
                                     int zeros_plus_one, b200_stream_t stream);

/* GPTQ act-order (desc_act): the rows of the packed weight are the checkpoint's rows sorted by
 * quant group — perm = argsort(g_idx), g_idx_sorted = g_idx[perm] (qlinear_gptq_marlin_impl.cpp:43-56,
 * marlin/gptq_repack.cu:17); the caller feeds the GEMM activations with the same column order
 * (b200_permute_cols, the reference's permute_cols_kernel marlin/gptq_gemm.cu:66-104).  Whole K
 * only (is_k_full): every group then has exactly group_size rows. */
B200_API int b200_w4a16_prepack_gptq_actorder(void* packed, const int32_t* qweight,
                                              const int32_t* qzeros, const void* scales,
                                              const int32_t* perm, const int32_t* g_idx_sorted,
                                              int64_t K, int64_t N, int group_size,
                                              int zeros_plus_one, b200_stream_t stream);
/* The operator-level drop-in for marlin::awq_repack(q_weight, out, num_bits) /
 * gptq_repack(q_weight, perm, out, num_bits) (src/kernels/quantization/marlin.h:30-37): `out` has
 * the byte count of q_weight (K * N / 2) and receives the nibble part of every tile blob, tile
 * (nt, kt) at byte (nt * K/128 + kt) * 8192; perm = act-order row order or NULL. */
B200_API int b200_w4a16_repack_awq(void* out, const int32_t* qweight, int64_t K, int64_t N,
                                   b200_stream_t stream);
B200_API int b200_w4a16_repack_gptq(void* out, const int32_t* qweight, const int32_t* perm,
                                    int64_t K, int64_t N, b200_stream_t stream);
/* ... and for what marlin::gptq_gemm receives beside it (marlin.h:17-28): scales [K/g, N] and
 * zero points [K/g, N/8] ALREADY in Marlin's column order (the layer permuted them,
 * qlinear_awq_marlin_impl.cpp:62-124); zeros_marlin NULL = symmetric, zero point 8 (has_zp
 * false).  Writes the full tile blobs b200_w4a16_gemm streams (b200_w4a16_packed_bytes). */
B200_API int b200_w4a16_assemble_marlin(void* packed, const void* nibbles, const void* scales_marlin,
                                        const int32_t* zeros_marlin, int64_t K, int64_t N,
                                        int group_size, b200_stream_t stream);
/* out[r, j] = in[r, perm[j]], bf16 / fp16 rows (strides in elements): the activation side of
 * act-order, permute_cols_kernel marlin/gptq_gemm.cu:66-104. */
B200_API int b200_permute_cols(void* out, const void* in, const int32_t* perm, int64_t rows,
                               int64_t cols, int64_t in_stride, int64_t out_stride, int dtype,
                               b200_stream_t stream);
/* Inverse of the prepack (debug / parity): W_out[K,N] bf16 = dequantised weights. */
B200_API int b200_w4a16_dequant(void* w_out, const void* packed, int64_t K,
                                int64_t N, int group_size, b200_stream_t stream);

/* Workspace of b200_w4a16_gemm: the fp32 stream-K partials of one chunk of <= 128 rows
 * (slots x min(M,128) x N floats).  No initialisation contract: it is fully overwritten before
 * it is read (unlike Marlin's zeroed lock workspace, marlin.h:24, which has no counterpart here). */
B200_API int64_t b200_w4a16_workspace_bytes(int64_t M, int64_t N, int64_t K);

/* A: [M, K] bf16 row stride lda;  C: [M, N] bf16 row stride ldc; bias: [N] bf16 or NULL.
 * Two launches: the stream-K GEMM (fp32 partials into the workspace) and a reduction pass. */
B200_API int b200_w4a16_gemm(void* C, const void* A, const void* packed,
                             const void* bias, int64_t M, int64_t N, int64_t K,
                             int64_t lda, int64_t ldc, int group_size,
                             void* workspace, int64_t workspace_bytes,
                             b200_stream_t stream);

/* "Partials" mode (B200-native fusion of the GEMM's cross-CTA reduction into its consumer).
 * The GEMM is stream-K: the (n tile, k tile) units are cut into equal contiguous shares, one per
 * CTA, and every CTA writes the fp32 partial of each tile it touches to
 * partials[slot][M][N], slot = its rank among that tile's contributors.  The consumer
 * (b200_rms_norm_residual_splitk, b200_ar_allreduce_splitk, or the reduction pass of
 * b200_w4a16_gemm) recomputes the same partition from (N, K), sums each tile's slots in slot
 * order and rounds once to the element type — exactly what a GEMM epilogue would have stored.
 * Replaces the o_proj / down_proj + residual add + RMSNorm sequence of
 * models/meta/llama.h:170-177.  b200_w4a16_splitk_splits returns the slot count the partials
 * buffer must have for a [K, N] weight on the current device (<= 8).  M <= 128. */
B200_API int b200_w4a16_splitk_splits(int64_t M, int64_t N, int64_t K);
B200_API int b200_w4a16_gemm_splitk(float* partials, const void* A, const void* packed, int64_t M,
                                    int64_t N, int64_t K, int64_t lda, int group_size, int splits,
                                    b200_stream_t stream);
/* C[M, N] bf16 (row stride ldc) = bf16(sum_slots partials) (+ bias): the plain reduction pass. */
B200_API int b200_w4a16_reduce_partials(void* C, const float* partials, int splits, int64_t gemm_k,
                                        const void* bias, int64_t M, int64_t N, int64_t ldc,
                                        b200_stream_t stream);
/* residual += T(sum_slots partials); out = rms_norm(residual) * weight.
 * partials: [splits, rows, n] fp32 from a GEMM with reduction dimension gemm_k. */
B200_API int b200_rms_norm_residual_splitk(void* out, void* residual, const float* partials,
                                           int splits, int64_t gemm_k, const void* weight,
                                           int64_t rows, int64_t n, float eps, int dtype,
                                           b200_stream_t stream);

/* Fused consumers of the qkv / gate_up GEMM partials (same partition rules as above):
 *   b200_rope_kv_write_splitk: qkv[T, (H + 2 Hkv) D] = T(sum_slots partials), then exactly
 *     b200_rope_kv_write on its q | k | v column blocks (q, k rotated in place, rotated k and v
 *     scattered to their cache slots).  Replaces qkv_proj's epilogue + apply_rotary_pos_emb +
 *     set_kv_cache (models/meta/llama.h:123-133).
 *   b200_silu_mul_splitk: out[rows, inter] = silu(T(gate)) * T(up), gate | up the two halves of the
 *     gate_up GEMM row (models/meta/llama.h:61-64, activation.cpp:101-103 rounding). */
B200_API int b200_rope_kv_write_splitk(void* qkv, const float* partials, int splits, int64_t gemm_k,
                                       const int32_t* positions, const void* cos_sin,
                                       const int32_t* slot_ids, void* k_cache, void* v_cache,
                                       int64_t n_tokens, int64_t n_heads, int64_t n_kv_heads,
                                       int64_t head_dim, int64_t rotary_dim, int interleaved,
                                       int dtype, b200_stream_t stream);
B200_API int b200_silu_mul_splitk(void* out, const float* partials, int splits, int64_t gemm_k,
                                  int64_t rows, int64_t inter, int dtype, b200_stream_t stream);

/* Debug / test hook (host arithmetic only, no device): the stream-K partition the GEMM and its
 * consumers use for a [K, N] weight split over `ctas` CTAs with `nsub` (1 or 2) weight tiles per
 * partition tile.  plan_out[5] = {units, ctas used, k tiles, partition tiles, slots};
 * first_owner_out / contrib_out (optional, one entry per partition tile) = first contributing CTA
 * and number of contributors of that tile (the slot a CTA writes is its index minus first_owner). */
B200_API int b200_debug_w4a16_plan(int64_t N, int64_t K, int ctas, int nsub, int32_t* plan_out,
                                   int32_t* first_owner_out, int32_t* contrib_out);

/* ------------------------------------------------------------------------ *
 * A8  Dense bf16 linear, decode-sized batches
 *     replaces F::linear -> cuBLASLt of ColumnParallelLinearImpl / RowParallelLinearImpl::forward
 *     (src/layers/linear/parallel_linear.cpp:256-263,294-308) and lm_head
 *     (src/models/meta/llama.h:259-265): C[M, N] = A[M, K] W[N, K]^T (+ bias), bf16 in / out,
 *     fp32 accumulation, one rounding.  W is the nn.Linear weight as the checkpoint stores it
 *     ([N, K] row-major, row stride ldw elements); N %% 8 == 0, K %% 64 == 0; any M (one pass over
 *     W per 128 rows).  workspace: b200_dense_workspace_bytes (fp32 stream-K partials).
 * ------------------------------------------------------------------------ */
B200_API int64_t b200_dense_workspace_bytes(int64_t M, int64_t N, int64_t K);
B200_API int b200_dense_gemm(void* C, const void* A, const void* W, const void* bias /*nullable [N]*/,
                             int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldw, int64_t ldc,
                             void* workspace, int64_t workspace_bytes, b200_stream_t stream);
/* Partials mode, same contract as b200_w4a16_gemm_splitk (the reduction, and whatever follows it in
 * the layer — RoPE + KV write, residual + RMSNorm, SiLU*mul, the TP all-reduce — runs in the
 * consumer): partials [b200_dense_splitk_splits()][M][N] fp32, M <= 128, N and K multiples of 128;
 * the stream-K partition is the int4 GEMM's for the same (N, K), so every b200_*_splitk consumer
 * takes these partials unchanged. */
B200_API int b200_dense_splitk_splits(int64_t M, int64_t N, int64_t K);
B200_API int b200_dense_gemm_splitk(float* partials, const void* A, const void* W, int64_t M, int64_t N,
                                    int64_t K, int64_t lda, int64_t ldw, int splits, b200_stream_t stream);

/* Debug hook: when non-NULL, every b200_w4a16_gemm CTA records clock64() milestones into
 * device_buffer[blockIdx.x * 16 + slot] (long long).  Pass NULL to disable (default). */
B200_API void b200_debug_set_trace(void* device_buffer);

/* ------------------------------------------------------------------------ *
 * Greedy sampling tail (the step driver's last kernel):
 *     out[r] = argmax_j logits[r, j]   (first index of the maximum, NaN counts as the maximum:
 *     torch.argmax semantics, which the reference's greedy path uses, src/sampling/sampler.cpp).
 * ------------------------------------------------------------------------ */
B200_API int b200_argmax(int64_t* out, const void* logits, int64_t rows, int64_t n, int64_t stride,
                         int dtype, b200_stream_t stream);

/* The logits processors of the sampling tail, in place on logits [batch, vocab] (contiguous), with
 * the semantics and rounding points of src/kernels/sampling/penalty_kernels.cu:9-33,52-75,107-140
 * and softmax_kernels.cu:11-54 (declared in src/kernels/sampling/sampling_kernels.h:7-29):
 *   temperature   logits[b, :] *= (t[b] == 0 ? 1 : 1 / t[b])
 *   repetition    for the lens[b] unique ids of row b: x < 0 ? x * p[b] : x / p[b]
 *   freq/presence for ids with count > 0: x -= count * freq[b]; x -= presence[b]
 *   softmax       exp(x - max) stored in T, summed from the stored values, / (sum + 1e-6)
 * token_ids int64 [batch, max_len], token_counts / token_ids_lens int32. */
B200_API int b200_apply_temperature(void* logits, const void* temperatures, int64_t batch,
                                    int64_t vocab, int dtype, b200_stream_t stream);
B200_API int b200_apply_repetition_penalty(void* logits, const int64_t* token_ids,
                                           const int32_t* token_ids_lens, const void* penalties,
                                           int64_t batch, int64_t vocab, int64_t max_len, int dtype,
                                           b200_stream_t stream);
B200_API int b200_apply_frequency_presence_penalty(void* logits, const int64_t* token_ids,
                                                   const int32_t* token_counts,
                                                   const int32_t* token_ids_lens,
                                                   const void* frequency_penalties,
                                                   const void* presence_penalties, int64_t batch,
                                                   int64_t vocab, int64_t max_len, int dtype,
                                                   b200_stream_t stream);
B200_API int b200_softmax(void* logits, int64_t batch, int64_t vocab, int dtype, b200_stream_t stream);
/* top-k / top-p filter, in place: replaces TopKTopPLogitsProcessor::forward
 * (src/sampling/logits_processor.h:243-276: sort descending, mask sorted positions >= top_k[b], softmax of
 * the rest, mask positions whose exclusive cumulative probability exceeds top_p[b], scatter back — a
 * [batch, vocab] sort and four more library launches) by one launch that finds the cut with a radix
 * histogram and writes -inf over everything outside it.  top_k [batch] int64 (<= 0: no top-k limit),
 * top_p [batch] float (>= 1: no top-p limit); either may be NULL.  logits [batch, vocab] bf16 / fp16, row
 * stride in elements.  Of equal logits straddling the cut the lowest vocabulary indices are kept. */
B200_API int b200_topk_topp_filter(void* logits, const int64_t* top_k /*nullable*/, const float* top_p /*nullable*/,
                                   int64_t batch, int64_t vocab, int64_t stride, int dtype, b200_stream_t stream);

/* ------------------------------------------------------------------------ *
 * A9  Tensor-parallel all-reduce over NVLink peer memory
 *     replaces ProcessGroupNCCL::allreduce (src/model_parallel/process_group.cpp:135-153)
 *     for the <= 1 MiB row-parallel reductions of the decode step (two-shot row-partitioned
 *     push protocol above two ranks, one-shot pull at two; csrc/allreduce.cu).
 *
 *     One communicator per GPU.  One process per GPU: every rank calls
 *     b200_ar_create (allocates its symmetric buffer + flags and returns an IPC
 *     handle blob), exchanges the blobs out of band (torch.distributed
 *     all_gather in this repo), then calls b200_ar_open_peers with all ranks'
 *     blobs in rank order.  All ranks in one process, one thread per GPU (the
 *     reference engine): b200_ar_create_all.
 * ------------------------------------------------------------------------ */
typedef struct b200_ar_comm b200_ar_comm;
#define B200_AR_HANDLE_BYTES 128

B200_API int b200_ar_create(b200_ar_comm** comm, int rank, int world_size,
                            int64_t max_bytes, void* handle_out /*[B200_AR_HANDLE_BYTES]*/);
B200_API int b200_ar_open_peers(b200_ar_comm* comm,
                                const void* all_handles /*[world][B200_AR_HANDLE_BYTES]*/);
/* All ranks in ONE process, one thread per GPU — the reference engine's model:
 * ProcessGroup::create_process_groups -> ncclCommInitAll (process_group.cpp:98-118).  Creates
 * comms[r] on devices[r] for r = 0..world_size-1 and maps every peer's region through CUDA peer
 * access (no IPC, no handle exchange); all or nothing.  Each communicator is then used from the
 * thread that has its device current, exactly like the IPC form. */
B200_API int b200_ar_create_all(b200_ar_comm** comms /*[world_size] out*/, const int* devices,
                                int world_size, int64_t max_bytes);
/* In-place sum of data[count] (bf16/fp16/fp32) over all ranks, on `stream`. */
B200_API int b200_ar_allreduce(b200_ar_comm* comm, void* data, int64_t count,
                               int dtype, b200_stream_t stream);
/* All-gather along the last dimension: in [rows, row_bytes] per rank -> out [rows, world *
 * row_bytes] with rank r's row at byte offset r * row_bytes — what
 * gather_from_model_parallel_region builds with allgather + cat(dim=-1)
 * (src/model_parallel/model_parallel.cpp:13-31).  Bit exact; rows * row_bytes <= max_bytes,
 * row_bytes % 16 == 0; shares the communicator's epoch with the all-reduces (every rank must
 * issue the same sequence of collectives). */
B200_API int b200_ar_allgather(b200_ar_comm* comm, void* out, const void* in, int64_t rows,
                               int64_t row_bytes, b200_stream_t stream);
/* Same reduction, but this rank's input is the producing GEMM's stream-K partials
 * [splits][count] fp32 (b200_w4a16_gemm_splitk of a [gemm_k, n] weight, count = rows * n): the
 * copy-in stage sums each tile's slots and rounds once, so the row-parallel GEMM needs no
 * reduction pass of its own.  out: [count] bf16/fp16. */
B200_API int b200_ar_allreduce_splitk(b200_ar_comm* comm, void* out, const float* partials,
                                      int splits, int64_t gemm_k, int64_t n, int64_t count,
                                      int dtype, b200_stream_t stream);
/* ... and with the consumer fused as well: residual += T(all-reduced row); out = rms_norm(residual)
 * * weight, one launch for the row-parallel GEMM's reduction, the TP all-reduce, the residual add
 * and the RMSNorm (models/meta/llama.h:170-177 under tensor parallelism).  Two-shot form (default
 * above two ranks): rows <= 128, n <= 8192; one-shot form: rows <= 64, n <= 4096. */
B200_API int b200_ar_allreduce_splitk_norm(b200_ar_comm* comm, void* out, void* residual,
                                           const float* partials, int splits, int64_t gemm_k,
                                           const void* weight, int64_t rows, int64_t n, float eps,
                                           int dtype, b200_stream_t stream);
/* Greedy sampling over a column-parallel (vocabulary-sharded) lm_head without gathering the
 * logits: out[r] = argmax over all ranks' columns of row r, exactly what
 * torch.argmax(gather_from_model_parallel_region(logits), -1) gives (lm_head gather_output=true,
 * src/models/meta/llama.h:259-265 -> model_parallel.cpp:13-31, then the greedy sampler): first
 * index of the maximum, NaN counts as the maximum.  logits: this rank's [rows, n_local] shard
 * (row stride `stride` elements), global column = rank * n_local + local column.  One launch: an
 * 8-byte candidate per rank and row crosses NVLink.  rows <= 128.  Shares the communicator's
 * epoch with the other collectives. */
B200_API int b200_ar_argmax(b200_ar_comm* comm, int64_t* out, const void* logits, int64_t rows,
                            int64_t n_local, int64_t stride, int dtype, b200_stream_t stream);
B200_API int b200_ar_destroy(b200_ar_comm* comm);

/* ------------------------------------------------------------------------ *
 * Sequence mixers and residual arrangements beyond the Llama layer (hyper.cu, latent_attn.cu,
 * delta_rule.cu, moe.cu).  The reference has no counterpart for these; each entry states its own
 * arithmetic.  "T" is the activation type named by `dtype`; everything marked fp32 is float on the
 * device whatever T is.  All strides count elements.  Step metadata as in the attention entry
 * (q_cu_lens / kv_cu_lens / block_tables of first-slot ids / cu_block_lens), plus
 *   token_seq   [rows]  index of the step's sequence a packed row belongs to
 *   state_slots [n_seq] recurrent-state slot of every sequence of the step
 * A portion whose first row has position 0 starts from zero state instead of reading its slot.
 * ------------------------------------------------------------------------ */
/* X[row, s, :] = table[tokens[row], :] for all S residual streams (X fp32 [rows, S, W]). */
B200_API int b200_embed_streams(float* X, const void* table, const int32_t* tokens, int64_t rows, int64_t W,
                                int64_t S, int64_t vocab, int dtype, b200_stream_t stream);
/* u = sum_s collapse[s] X[row, s, :] (collapse NULL: plain sum); out = u * rsqrt(mean(u^2) + eps) *
 * (offset + weight), written as T and, when out32 is given, also as fp32.  S <= 8. */
B200_API int b200_hc_norm(void* out, float* out32 /*nullable*/, const float* X, const float* collapse /*nullable*/,
                          const float* weight, int64_t rows, int64_t W, int64_t S, float eps, float offset,
                          int dtype, b200_stream_t stream);
/* out_t = n_t + (n_{t-1} - n_t) * mu; n_{t-1} of a portion's first row comes from state[slot]
 * (fp32 [n_slots, W]), which then receives the portion's last n. */
B200_API int b200_token_shift(void* out, const float* n32, const float* mu, float* state, const int32_t* q_cu_lens,
                              const int32_t* positions, const int32_t* token_seq, const int32_t* state_slots,
                              int64_t rows, int64_t W, int dtype, b200_stream_t stream);
/* X[row, t, :] <- sum_s mix[s, t] X[row, s, :] + out_coef[t] * y[row, :] * sigmoid(gate[row, :] + gate_bias)
 * (gate NULL: no gate; mix NULL: identity; out_coef NULL: ones). */
B200_API int b200_gated_hc_update(float* X, const void* y, int64_t ldy, const void* gate /*nullable*/, int64_t ldg,
                                  const float* gate_bias /*nullable*/, const float* mix /*nullable*/,
                                  const float* out_coef /*nullable*/, int64_t rows, int64_t W, int64_t S,
                                  int dtype, b200_stream_t stream);
/* out[rows, n] = act(in[:, :n]) * in[:, n:2n]; act 0 = SiLU, 1 = GELU in its tanh form with tanhf. */
B200_API int b200_gated_act(void* out, const void* in, int64_t rows, int64_t n, int64_t ld_in, int act, int dtype,
                            b200_stream_t stream);
/* out[t, h * d + i] = in[h, t, i] (* sigmoid(gate[t, h * d + i]) when gate is given). */
B200_API int b200_heads_to_rows(void* out, const void* in, const void* gate /*nullable*/, int64_t ldg, int64_t rows,
                                int64_t H, int64_t d, int dtype, b200_stream_t stream);
/* Latent attention, per token: cache[slot] = [rmsnorm(dkv[:rank]) * c_norm_weight | rope(dkv[rank:rank+rd])]
 * and rope in place on columns [dim, dim + rd) of each of q's H heads of width dim + rd.  The first `dims`
 * entries of a rotary part rotate as interleaved pairs (2i, 2i+1), or with half_pairs as pairs (i, i + dims/2),
 * by positions * inv_freq[i]; cos and sin are multiplied by `mult`. */
B200_API int b200_latent_prepare(void* q, int64_t ldq, const void* dkv, int64_t ld_dkv, void* cache, int64_t ldc,
                                 const float* c_norm_weight, const float* inv_freq, float mult,
                                 const int32_t* positions, const int32_t* slots, int64_t rows, int64_t H,
                                 int64_t dim, int64_t rd, int64_t dims, int64_t rank, float eps, int half_pairs,
                                 int dtype, b200_stream_t stream);
/* out[h, t, :rank] = sum_j softmax_j((q_absorbed[h, t] . c_j + q_rot[t, h] . kr_j) * scale) c_j over the
 * cached rows j <= position of t (paged), with window > 0 only over the rows with position - j < window.
 * q_absorbed: fp32 or T, [H, rows, rank] by strides. */
B200_API int b200_latent_attn(void* out, int64_t out_head_stride, int64_t out_token_stride, const void* q_absorbed,
                              int64_t qa_head_stride, int64_t qa_token_stride, int qa_is_fp32, const void* q,
                              int64_t ldq, const void* cache, int64_t ldc, const int32_t* q_cu_lens,
                              const int32_t* kv_cu_lens, const int32_t* block_tables, const int32_t* cu_block_lens,
                              const int32_t* token_seq, int64_t rows, int64_t H, int64_t dim, int64_t rd,
                              int64_t rank, int64_t block_size, float scale, int64_t window, int n_splits,
                              void* workspace, int64_t workspace_bytes, int dtype, b200_stream_t stream);
/* n_splits >= 1 (bf16 only): tensor-core form, the keys of every row cut into n_splits ranges that run as
 * separate CTAs and are merged by a second kernel (n_splits > 1 needs the workspace below); n_splits = 0: the
 * CUDA-core form (any dtype, fp32 arithmetic throughout). */
B200_API int64_t b200_latent_attn_workspace_bytes(int64_t rows, int64_t H, int64_t rank, int64_t n_splits);
/* Generalised delta rule over each sequence's tokens of the step (see delta_rule.cu); r, k, v, removal and gate
 * logits are column blocks [H * d] of matrices with row stride ld, the decay logits have row stride ld_decay;
 * state fp32 [n_slots, H, d, d]. */
B200_API int b200_delta_rule(void* out, int64_t ldo, const void* r, const void* k, const void* v,
                             const void* decay_logits, const void* removal_logits, const void* gate_logits,
                             int64_t ld, int64_t ld_decay, const float* decay_bias, const float* removal_bias,
                             const float* norm_weight, float* state, const int32_t* q_cu_lens,
                             const int32_t* positions, const int32_t* state_slots, int64_t n_seq, int64_t H,
                             int64_t d, float decay_scale, float key_eps, float eps, int dtype,
                             b200_stream_t stream);
/* Mixture of experts (see moe.cu). */
B200_API int b200_moe_route(int32_t* expert_ids, float* weights, const void* h, int64_t ldh,
                            const float* router_weight, int64_t rows, int64_t W, int64_t E, int64_t top, int dtype,
                            b200_stream_t stream);
B200_API int b200_moe_plan(int32_t* offsets, int32_t* sorted_pair, int32_t* pos_of_pair, const int32_t* expert_ids,
                           int64_t n_pairs, int64_t E, b200_stream_t stream);
B200_API int b200_grouped_gemm(void* C, int64_t ldc, const void* A, int64_t lda, const int32_t* sorted_pair /*nullable*/,
                               const float* pair_scale /*nullable*/, int64_t top, const void* weights,
                               const int32_t* offsets, int64_t n_rows, int64_t E, int64_t N, int64_t K, int dtype,
                               b200_stream_t stream);
/* The same product for few rows per expert (decoding): the weights are streamed once per 8 rows of an expert. */
B200_API int b200_grouped_gemv(void* C, int64_t ldc, const void* A, int64_t lda, const int32_t* sorted_pair /*nullable*/,
                               const float* pair_scale /*nullable*/, int64_t top, const void* weights,
                               const int32_t* offsets, int64_t n_rows, int64_t E, int64_t N, int64_t K, int dtype,
                               b200_stream_t stream);
/* xs[pos] = pair_scale[pair] * h[pair / top] in sorted order: the input of a library grouped GEMM. */
B200_API int b200_moe_gather(void* xs, const void* h, int64_t ldh, const int32_t* sorted_pair,
                             const float* pair_scale /*nullable*/, int64_t top, int64_t n_pairs, int64_t W, int dtype,
                             b200_stream_t stream);
/* out[row] = scale * sum_k Y[pos_of_pair[row, k]] (+ addend[row], a result that every token gets). */
B200_API int b200_moe_combine(void* out, const void* Y, int64_t ldy, const int32_t* pos_of_pair, int64_t rows,
                              int64_t W, int64_t top, float scale, const void* addend /*nullable*/, int64_t ld_add,
                              int dtype, b200_stream_t stream);
/* Experts chosen by the token id, not by a router: expert_ids[row, k] = table[tokens[row], k] (table int32
 * [vocab, top]). */
B200_API int b200_moe_table_route(int32_t* expert_ids, const int32_t* table, const int32_t* tokens, int64_t rows,
                                  int64_t top, int64_t vocab, int64_t E, b200_stream_t stream);

/* ---------------------------------------------------------------------------
 * Decoders with a normalised sublayer RESULT, a depth-weighted average of layer results, a minimal gated
 * recurrence and differential sliding-window attention (postnorm.cu, mingru.cu, diff_attn.cu).  The reference
 * has no such operators; each entry states its arithmetic.  Conventions as in the block above.
 * ------------------------------------------------------------------------ */
/* x[row] = scale * table[tok] + pair_table[(mul_prev * prev + mul_cur * tok) mod buckets] (row `buckets` of the
 * pair table when prev_tokens[row] < 0 or prev_tokens is NULL; no pair term when pair_table is NULL);
 * x fp32 [rows, W], h (nullable) the same rows as T. */
B200_API int b200_bigram_embed(float* x, void* h /*nullable*/, const void* table, const void* pair_table /*nullable*/,
                               const int32_t* tokens, const int32_t* prev_tokens /*nullable*/, int64_t rows,
                               int64_t W, int64_t vocab, int64_t buckets, int64_t mul_prev, int64_t mul_cur,
                               float scale, int dtype, b200_stream_t stream);
/* r = x_in + mult * y / sqrt(mean_group(y^2) + eps) * weight, the row cut into `groups` equal consecutive parts.
 * Without hist: x_out = r.  With hist (fp32 [n_hist, hist_stride], slice j = the result of stage j):
 * hist[n_hist - 1] = r and x_out = sum_j coef[j] hist[j].  h_out (nullable): x_out as T.  x_out may be x_in. */
B200_API int b200_postnorm_residual(float* x_out, void* h_out /*nullable*/, const float* x_in, const void* y,
                                    int64_t ldy, const float* weight, int64_t rows, int64_t W, int64_t groups,
                                    float mult, float eps, float* hist /*nullable*/, int64_t hist_stride,
                                    int64_t n_hist, const float* coef /*nullable*/, int dtype, b200_stream_t stream);
/* The partition b200_dense_gemm_splitk uses for an [N, K] weight, as six integers a fused consumer is given
 * (returns the number of partial slots, 0 if the shape has no such partition). */
B200_API int b200_dense_splitk_plan(int64_t N, int64_t K, int32_t* plan6);
/* b200_postnorm_residual / b200_glu_clamped fed by the split-K partials [n_slots][rows][W or 2 n] of the matrix
 * product that made their input (its reduction pass folded in: the sum is rounded to T first). */
B200_API int b200_postnorm_residual_splitk(float* x_out, void* h_out /*nullable*/, const float* x_in,
                                           const float* partials, int64_t n_slots, const int32_t* plan6,
                                           const float* weight, int64_t rows, int64_t W, int64_t groups, float mult,
                                           float eps, float* hist /*nullable*/, int64_t hist_stride, int64_t n_hist,
                                           const float* coef /*nullable*/, int dtype, b200_stream_t stream);
B200_API int b200_glu_clamped_splitk(void* out, const float* partials, int64_t n_slots, const int32_t* plan6,
                                     int64_t rows, int64_t n, float limit, float slope, int dtype,
                                     b200_stream_t stream);
/* out (T) = x / sqrt(mean_group(x^2) + eps) * weight for fp32 rows x [rows, W]. */
B200_API int b200_group_rms_norm(void* out, const float* x, const float* weight, int64_t rows, int64_t W,
                                 int64_t groups, float eps, int dtype, b200_stream_t stream);
/* out[rows, n] = g sigmoid(slope g) (u + 1) with g = min(in[:, :n], limit), u = clamp(in[:, n:2n], -limit, limit). */
B200_API int b200_glu_clamped(void* out, const void* in, int64_t rows, int64_t n, int64_t ld_in, float limit,
                              float slope, int dtype, b200_stream_t stream);
/* out[r, c] = gelu_tanh(in[r, c]) * table[tokens[r], col0 + c] for c < n. */
B200_API int b200_token_gated_gelu(void* out, const void* in, int64_t ld_in, const void* table, int64_t ld_table,
                                   int64_t col0, const int32_t* tokens, int64_t rows, int64_t n, int64_t vocab,
                                   int dtype, b200_stream_t stream);
/* The per-token term and its post-norm in one launch, for few rows: y = P (gelu_tanh(G h) * table[tok, col0 : col0 +
 * side_dim]) with G [side_dim, W], P given TRANSPOSED as [side_dim, W], and h [rows, W] of type T (intermediate results rounded to T like
 * matrix products), then b200_postnorm_residual's arithmetic on y. */
B200_API int b200_token_side_postnorm(float* x_out, void* h_out /*nullable*/, const float* x_in, const void* h,
                                      const void* gate_weight, const void* proj_weight, const void* table,
                                      int64_t ld_table, int64_t col0, const int32_t* tokens, int64_t vocab,
                                      int64_t side_dim, const float* weight, int64_t rows, int64_t W, int64_t groups,
                                      float mult, float eps, float* hist /*nullable*/, int64_t hist_stride,
                                      int64_t n_hist, const float* coef /*nullable*/, int dtype, b200_stream_t stream);
/* Minimal gated recurrent unit over each sequence's tokens of the step (see mingru.cu): proj = [z | x | g] column
 * blocks of `width`, state fp32 [n_slots, width]. */
B200_API int b200_mingru_scan(void* out, int64_t ldo, const void* proj, int64_t ld, const float* z_bias /*nullable*/,
                              const float* x_bias /*nullable*/, float* state, const int32_t* q_cu_lens,
                              const int32_t* positions, const int32_t* state_slots, int64_t n_seq, int64_t width,
                              int dtype, b200_stream_t stream);
/* The same scan with every portion cut into chunks of chunk_len tokens that run side by side (two kernels: the
 * chunks' (A, B) with S_end = A S_start + B, then every chunk from the fold of those before it).  q_max: the longest
 * portion of the step; workspace: fp32, at least ..._workspace_floats. */
B200_API int64_t b200_mingru_chunked_workspace_floats(int64_t n_seq, int64_t width, int64_t q_max, int64_t chunk_len);
B200_API int b200_mingru_scan_chunked(void* out, int64_t ldo, const void* proj, int64_t ld,
                                      const float* z_bias /*nullable*/, const float* x_bias /*nullable*/, float* state,
                                      const int32_t* q_cu_lens, const int32_t* positions, const int32_t* state_slots,
                                      int64_t n_seq, int64_t width, int64_t q_max, int64_t chunk_len, float* workspace,
                                      int64_t workspace_floats, int dtype, b200_stream_t stream);
/* Differential attention, per token (see diff_attn.cu): RMS norm + rotation of the H * 2 query maps into q_out
 * (fp32 [rows, H, 2, dim]) and, when k_in is given, of the G * 2 key maps into k_cache[slot] ([slots, G, 2 * dim])
 * with v_in copied to v_cache[slot] ([slots, G, vdim]).  q_in / k_in / v_in: rows of stride ld. */
B200_API int b200_diff_attn_prepare(float* q_out, const void* q_in, const void* k_in /*nullable*/,
                                    const void* v_in /*nullable*/, int64_t ld, void* k_cache, void* v_cache,
                                    const float* q_norm_weight, const float* k_norm_weight,
                                    const float* inv_freq, float rot_mult, const int32_t* positions,
                                    const int32_t* slots, int64_t rows, int64_t H, int64_t G, int64_t dim,
                                    int64_t vdim, int64_t rot_dims, float eps, int dtype, b200_stream_t stream);
/* out[row, h * vdim + c] = the normalised, gated difference of the two maps' attention results (diff_attn.cu).
 * window 0: every earlier key is visible; gate (nullable): logits [rows, >= H] of stride ldg. */
B200_API int b200_diff_attn(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache,
                            const void* gate /*nullable*/, int64_t ldg, const int32_t* q_cu_lens,
                            const int32_t* kv_cu_lens, const int32_t* block_tables, const int32_t* cu_block_lens,
                            const int32_t* token_seq, int64_t rows, int64_t H, int64_t G, int64_t dim,
                            int64_t vdim, int64_t block_size, float scale, int64_t window, int64_t keep_first,
                            float lambda, float out_scale, float eps, int dtype, b200_stream_t stream);
/* The same result for prompt portions in bf16 on the tensor cores: CTAs of 16 to 64 consecutive tokens of one
 * sequence walk tiles of 32 keys (diff_attn.cu).  dim and vdim multiples of 16, at most 128 (..._supported tells);
 * q_max: the longest portion of the step. */
B200_API int b200_diff_attn_prefill_supported(int64_t dim, int64_t vdim, int dtype);
B200_API int b200_diff_attn_prefill(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache,
                                    const void* gate /*nullable*/, int64_t ldg, const int32_t* q_cu_lens,
                                    const int32_t* kv_cu_lens, const int32_t* block_tables,
                                    const int32_t* cu_block_lens, int64_t n_seq, int64_t q_max, int64_t H, int64_t G,
                                    int64_t dim, int64_t vdim, int64_t block_size, float scale, int64_t window,
                                    int64_t keep_first, float lambda, float out_scale, float eps, int dtype,
                                    b200_stream_t stream);
/* Single tokens in bf16 on the tensor cores: the 16 rows of a tile are the query heads of one key/value group, so
 * the group's keys are read once for all of them (same head sizes as ..._prefill_supported).  n_splits > 1: every
 * row's keys are shared out over that many CTAs and merged by a second kernel through the workspace (fp32, rows * H *
 * n_splits * (4 + 2 vdim) floats). */
B200_API int b200_diff_attn_decode_tc(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache,
                                      const void* gate /*nullable*/, int64_t ldg, const int32_t* q_cu_lens,
                                      const int32_t* kv_cu_lens, const int32_t* block_tables,
                                      const int32_t* cu_block_lens, const int32_t* token_seq, int64_t rows, int64_t H,
                                      int64_t G, int64_t dim, int64_t vdim, int64_t block_size, float scale,
                                      int64_t window, int64_t keep_first, float lambda, float out_scale, float eps,
                                      int64_t n_splits, float* workspace /*nullable*/, int64_t workspace_floats,
                                      int dtype, b200_stream_t stream);

/* ---------------------------------------------------------------------------
 * Decoders that normalise AFTER the residual sum with one gain per row, attend with unit-length queries and keys
 * under a distance bias and a learned sink, and cap their logits (postnorm.cu, sink_attn.cu).  The reference has
 * no such operators; each entry states its arithmetic.  Conventions as in the blocks above.
 * ------------------------------------------------------------------------ */
/* s = alpha x_in + y ; x_out = s / sqrt(mean(s^2) + eps) * weight[i * weight_stride] (stride 0: one number for the
 * row) ; h_out (nullable) = x_out as T.  x fp32 [rows, W]; y T with row stride ldy. */
B200_API int b200_sumnorm_residual(float* x_out, void* h_out /*nullable*/, const float* x_in, const void* y,
                                   int64_t ldy, const float* weight, int64_t weight_stride, int64_t rows, int64_t W,
                                   float alpha, float eps, int dtype, b200_stream_t stream);
/* The same fed by the split-K partials [n_slots][rows][W] of the matrix product that makes y (plan6:
 * b200_dense_splitk_plan); their sum is rounded to T first. */
B200_API int b200_sumnorm_residual_splitk(float* x_out, void* h_out /*nullable*/, const float* x_in,
                                          const float* partials, int64_t n_slots, const int32_t* plan6,
                                          const float* weight, int64_t weight_stride, int64_t rows, int64_t W,
                                          float alpha, float eps, int dtype, b200_stream_t stream);
/* out = cap * tanh(in / cap), elementwise (may be in place). */
B200_API int b200_softcap(void* out, const void* in, int64_t total, float cap, int dtype, b200_stream_t stream);
/* Per token: q_out[row, h] = q_in[row, h] / rms * (1 + temp_coef ln(floor((pos + 1) / temp_every) + 1)) as fp32
 * (temp_every 0: no temperature); with k_in / v_in (column blocks of the same matrix, row stride ld):
 * k_cache[slot, g] = k_in[row, g] / rms and v_cache[slot] = v_in[row], or with v_other (row stride ld_other)
 * (1 - lam) v_in[row] + lam v_other[row].  rms over the head's dim channels, eps inside the root. */
B200_API int b200_sink_attn_prepare(float* q_out, const void* q_in, const void* k_in /*nullable*/,
                                    const void* v_in /*nullable*/, int64_t ld, const void* v_other /*nullable*/,
                                    int64_t ld_other, float lam, void* k_cache, void* v_cache,
                                    const int32_t* positions, const int32_t* slots, int64_t rows, int64_t H, int64_t G,
                                    int64_t dim, int64_t vdim, float eps, float temp_coef, int64_t temp_every,
                                    int dtype, b200_stream_t stream);
/* out[row, h] = sum_j p_j v_j over the cached rows j <= position i of the row (paged), p_j = exp(s_j) /
 * (exp(sink[h]) + sum_j' exp(s_j')), s_j = scale q . k_j - r1[h] ln(1 + r2[h] (i - j)).  r1 / r2 (both or
 * neither) and sink are fp32 [H], nullable.  q fp32 [rows, H, dim]; caches [slots, G, dim] and [slots, G, vdim]
 * of type `dtype`; CUDA cores, any sizes. */
B200_API int b200_sink_attn(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache,
                            const float* r1 /*nullable*/, const float* r2 /*nullable*/,
                            const float* sink /*nullable*/, const int32_t* q_cu_lens, const int32_t* kv_cu_lens,
                            const int32_t* block_tables, const int32_t* cu_block_lens, const int32_t* token_seq,
                            int64_t rows, int64_t H, int64_t G, int64_t dim, int64_t vdim, int64_t block_size,
                            float scale, int dtype, b200_stream_t stream);
/* The same for bf16 on the tensor cores, tiles of 16 consecutive tokens of a sequence: dim and vdim multiples of
 * 16, at most 128 (..._supported tells); q_max: the longest portion of the step. */
B200_API int b200_sink_attn_prefill_supported(int64_t dim, int64_t vdim, int dtype);
B200_API int b200_sink_attn_prefill(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache,
                                    const float* r1 /*nullable*/, const float* r2 /*nullable*/,
                                    const float* sink /*nullable*/, const int32_t* q_cu_lens,
                                    const int32_t* kv_cu_lens, const int32_t* block_tables,
                                    const int32_t* cu_block_lens, int64_t n_seq, int64_t q_max, int64_t H, int64_t G,
                                    int64_t dim, int64_t vdim, int64_t block_size, float scale, int dtype,
                                    b200_stream_t stream);

/* Single tokens in bf16 on the tensor cores: the 16 rows of a tile are the query heads of one key/value group, so
 * the group's keys are read once for all of them (same head sizes as ..._prefill_supported).  n_splits > 1: every
 * row's keys are shared out over that many CTAs and merged by a second kernel through the workspace (fp32, rows * H *
 * n_splits * (2 + vdim) floats). */
B200_API int b200_sink_attn_decode_tc(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache,
                                      const float* r1 /*nullable*/, const float* r2 /*nullable*/,
                                      const float* sink /*nullable*/, const int32_t* q_cu_lens,
                                      const int32_t* kv_cu_lens, const int32_t* block_tables,
                                      const int32_t* cu_block_lens, const int32_t* token_seq, int64_t rows, int64_t H,
                                      int64_t G, int64_t dim, int64_t vdim, int64_t block_size, float scale,
                                      int64_t n_splits, float* workspace /*nullable*/, int64_t workspace_floats,
                                      int dtype, b200_stream_t stream);

/* ---- sigmoid attention inside blocks of positions with a head mix, gated delta rule with short input filters,
 * softmax router with group limits and pass-through outputs, branch norms (sigmoid_attn.cu, delta_rule.cu, moe.cu,
 * postnorm.cu).  The reference has no such operators; each entry states its arithmetic. ---- */
/* Per token: q_out[row, h] = turn(q_in[row, h] + q_bias) as fp32; k_cache[slot, g] = turn(k_in[row, g] + k_bias);
 * v_cache[slot] = v_in[row] + v_bias.  turn: the first rot_dims channels of a head, channel t with t + rot_dims / 2,
 * by the angle position * inv_freq[t] (fp32).  q_in / k_in / v_in: column blocks of one matrix (row stride ld);
 * biases fp32, nullable. */
B200_API int b200_sigmoid_attn_prepare(float* q_out, const void* q_in, const void* k_in, const void* v_in, int64_t ld,
                                       const float* q_bias /*nullable*/, const float* k_bias /*nullable*/,
                                       const float* v_bias /*nullable*/, void* k_cache, void* v_cache,
                                       const float* inv_freq /*nullable when rot_dims == 0*/,
                                       const int32_t* positions, const int32_t* slots, int64_t rows, int64_t H,
                                       int64_t G, int64_t dim, int64_t vdim, int64_t rot_dims, int dtype,
                                       b200_stream_t stream);
/* out[row, h] = sum_j a'_hj v_j over the cached rows j <= position i of the row with floor(j / size) = floor(i / size)
 * (size 0: all j <= i); a_hj = sigmoid(cap tanh(scale q_h . k_j / cap) + head_bias[h]) (cap 0: no cap), not normalised;
 * a'_hj = sum_g head_mix[h, g] a_gj (head_mix fp32 [H, H], nullable: a' = a).  q fp32 [rows, H, dim]; caches
 * [slots, G, dim] and [slots, G, vdim] of type `dtype`.  rows_per_cta: a hint (the longest portion of the step): CTAs
 * take up to 8 consecutive rows and share the key tiles among them.  n_splits > 1 (single rows only): every row's key
 * tiles are shared out over that many CTAs whose sums a second kernel adds up through the workspace (fp32, rows *
 * n_splits * H * vdim floats).  CUDA cores, any sizes with H * vdim <= 8192. */
B200_API int b200_sigmoid_attn(void* out, int64_t ldo, const float* q, const void* k_cache, const void* v_cache,
                               const float* head_bias /*nullable*/, const float* head_mix /*nullable*/,
                               const int32_t* q_cu_lens, const int32_t* kv_cu_lens, const int32_t* block_tables,
                               const int32_t* cu_block_lens, const int32_t* token_seq, int64_t rows, int64_t H,
                               int64_t G, int64_t dim, int64_t vdim, int64_t block_size, float scale, float cap,
                               int64_t size, int64_t rows_per_cta, int64_t n_splits, float* workspace /*nullable*/,
                               int64_t workspace_floats, int dtype, b200_stream_t stream);
/* The same for prompt portions in bf16 on the tensor cores: tiles of 16 consecutive tokens of a sequence x all heads
 * (dim and vdim multiples of 16 and shared memory for the heads' queries and one key tile: ..._supported tells);
 * q_max: the longest portion of the step. */
B200_API int b200_sigmoid_attn_prefill_supported(int64_t H, int64_t G, int64_t dim, int64_t vdim, int has_mix,
                                                 int dtype);
B200_API int b200_sigmoid_attn_prefill(void* out, int64_t ldo, const float* q, const void* k_cache,
                                       const void* v_cache, const float* head_bias /*nullable*/,
                                       const float* head_mix /*nullable*/, const int32_t* q_cu_lens,
                                       const int32_t* kv_cu_lens, const int32_t* block_tables,
                                       const int32_t* cu_block_lens, int64_t n_seq, int64_t q_max, int64_t H,
                                       int64_t G, int64_t dim, int64_t vdim, int64_t block_size, float scale,
                                       float cap, int64_t size, int dtype, b200_stream_t stream);
/* Inputs of the gated delta rule for every row: x = silu(filter(x_in)) with causal per-channel filters [channels, taps]
 * (last column: the current token; lags before the step come from filter_state [n_slots, taps - 1, 2 G dim + H vdim],
 * lags before position 0 are zero); q, k [rows, G, dim] made unit length per head (eps unit_eps under the root), q also
 * times dim^(-1/2); v [rows, H, vdim]; decay[row, h, c] = exp(-exp(a_log[h]) softplus(decay_in + dt_bias));
 * beta[row, h] = sigmoid(beta_in).  q_in, k_in, v_in, beta_in: column blocks of one matrix (row stride ld).  Then
 * filter_state takes the last taps - 1 inputs of every sequence.  All outputs fp32. */
B200_API int b200_gated_delta_prepare(float* q_out, float* k_out, float* v_out, float* decay_out, float* beta_out,
                                      const void* q_in, const void* k_in, const void* v_in, const void* beta_in,
                                      int64_t ld, const void* decay_in, int64_t ld_decay, const float* q_filter,
                                      const float* k_filter, const float* v_filter, const float* a_log,
                                      const float* dt_bias, float* filter_state, const int32_t* q_cu_lens,
                                      const int32_t* positions, const int32_t* token_seq, const int32_t* state_slots,
                                      int64_t rows, int64_t n_seq, int64_t H, int64_t G, int64_t dim, int64_t vdim,
                                      int64_t taps, float unit_eps, int dtype, b200_stream_t stream);
/* Per (sequence, head), over the sequence's rows in order, S [dim, vdim] fp32 in state[slot, h] (zero where the
 * portion starts at position 0):  S <- diag(decay) S ; u = beta (v - S^T k) ; S <- S + k u^T ; o = S^T q ;
 * out[row, h] = o / rms(o) * norm_weight[vdim] * sigmoid(gate_logits[row, h]).  Head h reads q / k head h / (H / G).
 * dim <= 128 with vdim <= 256, or dim <= 256 with vdim <= 128.  raw_workspace (nullable; fp32 [rows, H * vdim], rows =
 * the step's packed rows): the walk stores the plain read-outs there and a second, token-parallel launch applies the
 * norm and the gate (long portions: one barrier per token instead of two). */
B200_API int b200_gated_delta_scan(void* out, int64_t ldo, const float* q, const float* k, const float* v,
                                   const float* decay, const float* beta, const void* gate_logits, int64_t ld_gate,
                                   const float* norm_weight, float* state, const int32_t* q_cu_lens,
                                   const int32_t* positions, const int32_t* state_slots, int64_t n_seq, int64_t H,
                                   int64_t G, int64_t dim, int64_t vdim, float eps, float* raw_workspace /*nullable*/,
                                   int64_t rows, int dtype, b200_stream_t stream);
/* p = softmax(router_weight h) over E outputs (fp32); choice score c = p + correction (nullable); the outputs form
 * n_groups equal runs of neighbours and only the keep_groups runs with the largest max c can be chosen; the `top`
 * largest c are chosen; weights = chosen p / (their sum + weight_eps).  extra_weight (nullable, fp32 [W]):
 * extra_out[row] = sigmoid(extra_weight . h). */
B200_API int b200_moe_route_softmax(int32_t* expert_ids, float* weights, float* extra_out /*nullable*/, const void* h,
                                    int64_t ldh, const float* router_weight, const float* correction /*nullable*/,
                                    const float* extra_weight /*nullable*/, int64_t rows, int64_t W, int64_t E,
                                    int64_t top, int64_t n_groups, int64_t keep_groups, float weight_eps, int dtype,
                                    b200_stream_t stream);
/* out[row] = sum_k pair_weights[row, k] * (expert_ids[row, k] < n_real ? Y[pos_of_pair[row, k]] : h[row])
 * (+ addend_gate[row] * addend[row]; gate nullable: 1). */
B200_API int b200_moe_combine_weighted(void* out, const void* Y, int64_t ldy, const int32_t* pos_of_pair,
                                       const int32_t* expert_ids, const float* pair_weights, int64_t n_real,
                                       const void* h, int64_t ldh, int64_t rows, int64_t W, int64_t top,
                                       const void* addend /*nullable*/, int64_t ld_add,
                                       const float* addend_gate /*nullable*/, int dtype, b200_stream_t stream);
/* m = 1/2 (a / rms(a) * weight_a + b / rms(b) * weight_b), or m = a / rms(a) * weight_a without b, or m = a without
 * weight_a;  x_out = x_in + m / rms(m) * weight;  h_out (nullable) = x_out / rms(x_out) * weight_next as T, or x_out
 * as T without weight_next.  x fp32 [rows, W]; a, b of type T with row strides lda, ldb. */
B200_API int b200_branch_norm_residual(float* x_out, void* h_out /*nullable*/, const float* x_in, const void* a,
                                       int64_t lda, const void* b /*nullable*/, int64_t ldb,
                                       const float* weight_a /*nullable*/, const float* weight_b /*nullable*/,
                                       const float* weight, const float* weight_next /*nullable*/, int64_t rows,
                                       int64_t W, float eps, int dtype, b200_stream_t stream);
/* out [rows, n] = max(in, 0)^2 for the first n columns of rows with stride ld_in. */
B200_API int b200_relu_squared(void* out, const void* in, int64_t rows, int64_t n, int64_t ld_in, int dtype,
                               b200_stream_t stream);

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* B200_DECODE_H_ */

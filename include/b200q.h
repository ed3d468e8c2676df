/*
 * b200q.h -- C ABI of libb200q.so: hand-written sm_100a CUDA kernels for the quantized
 * single-token decode path (q4/q8 group-wise matvec family, fused gate/up + SwiGLU MLP,
 * q4/q8 paged-KV GQA decode attention, block-table gather).
 *
 * Every entry point is what the matching operator of manishklach/mlx-metal-kernels hands to
 * `mx.fast.metal_kernel(...)(inputs=..., output_shapes=..., grid=..., threadgroup=...)`: raw
 * device buffers plus the integers the reference packs into its `meta` array.  The reference
 * site each one replaces is cited as path:line within that project.
 *
 * Conventions
 *   - all pointers are DEVICE pointers on the current CUDA device; the library never
 *     allocates, frees or keeps them.  Outputs and workspaces are caller-allocated.
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).  Calls are
 *     asynchronous and stream-ordered.
 *   - dtype codes: B200Q_F16, B200Q_BF16, B200Q_F32.
 *   - return value: B200Q_OK (0) or a negative B200Q_ERR_* code; nothing aborts or traps.
 *     Execution errors of an already-launched kernel surface at the caller's next sync.
 *   - weights: q4 = two codes per byte, low nibble = even k, rows of ceil(K/2) bytes;
 *     q8 = one byte per code; scales/zeros [rows, ceil(K/group)] row-major.  Dequantisation
 *     is (code - zero) * scale, or code * scale when zeros is NULL
 *     (ops/quant_ops.py:205-212).
 */
#ifndef B200Q_H_
#define B200Q_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { B200Q_F16 = 0, B200Q_BF16 = 1, B200Q_F32 = 2 };

enum {
    B200Q_OK = 0,
    B200Q_ERR_BAD_ARG = -1,      /* null pointer, non-positive size, unknown dtype/bits */
    B200Q_ERR_UNSUPPORTED = -2,  /* shape outside what the kernels implement (e.g. head_dim > 128) */
    B200Q_ERR_LAUNCH = -3,       /* cudaGetLastError() after the launch was not cudaSuccess */
    B200Q_ERR_WORKSPACE = -4,    /* workspace pointer NULL or smaller than *_workspace_bytes() */
    B200Q_ERR_DEVICE_WAIT = -5,  /* reported by b200q_device_status(): a bounded device wait gave up */
    B200Q_ERR_STATIC_SCRATCH = -6 /* b200q_paged_gqa_decode_static: problem exceeds the built-in scratch array */
};

int b200q_version(void);
const char* b200q_strerror(int code);

/* Reads (and, if reset != 0, clears) the device-side status word.  Kernels record an event there instead of
 * trapping: 1-5 a bounded wait (on a shared-memory barrier or on a peer's flag) ran out, 6 b200q_rope_kv_append
 * met a position outside the rotary table (the row was left unrotated), 7 it met a position whose block-table
 * entry is unassigned (nothing was appended).  The largest event seen is returned.  Synchronises `stream`.
 * 0 = no event. */
int b200q_device_status(int reset, void* stream);

/* Runtime tuning knob (benchmark sweeps and tests; defaults are chosen per shape when unset/0).  Keys:
 *   "gemv.ts"            1 = every matvec the tcgen05 kernel supports goes to it, -1 = none, 0 = by batch
 *   "gemv.ts_min_batch"  smallest batch the tcgen05 kernel takes when "gemv.ts" is 0
 *   "gemv.fuse_norm"     1 = the tcgen05 kernel computes a requested rmsnorm in its own prologue even when the caller
 *                        gave a buffer for the normalised rows (default: a launch of the row kernel in front of it)
 *   "gemv.force_generic" 1 = always the one-warp-per-row kernel that follows the reference arithmetic literally
 *   "gemv.stage_k", "gemv.stages", "gemv.smem_kb", "gemv.interleave"   ring geometry, shared-memory budget and row
 *                        dealing of the mma.sync kernel
 *   "ts.stages", "ts.smem_kb", "ts.split", "ts.big"     ring depth, shared-memory budget, K split, shape of the tcgen05 kernel
 *   "ts.slow_reduce"     1 = the partial sums of a K split always travel through the first CTA's weight ring
 *   "ts.tp_world"        number of equal row shards the matrices of this process are split into (tensor parallelism):
 *                        the tcgen05 kernel then splits K, and the attention picks its kernel, as the unsharded call
 *                        would, which keeps a shard's rows bit-identical to the unsharded result
 *   "attn.ctas_per_sm", "attn.min_pages"                grid sizing of the split-KV attention kernel
 *   "attn.cluster"       1 = the one-kernel cluster form of the attention whenever it applies, -1 = never, 0 = small batches
 *   "attn.cluster_size"  CTAs per cluster of that form: 4, 8 (default) or 16
 *   "attn.force_simple"  1 = always the one-warp-per-head attention kernel
 *   "peer.spin_limit", "tp.spin_limit"   flag probes after which b200q_peer_allgather / the wait of an exchange fused
 *                        into a kernel gives up and records event 5 (default 2^22; tests shorten it)
 *   "no_pdl"             1 = launch without programmatic dependent launch */
int b200q_set_tuning(const char* key, int value);

/* Group-wise dequantisation, bit-exact: out = cast(fp32(code - zero) * scale) with two
 * separately rounded fp32 operations.  Replaces kernels/dequant_q4.metal, dequant_q8.metal as
 * launched by dequant_q4 / dequant_q8 (ops/quant_ops.py:215-253, 279-316).
 * codes [M, ceil(K/2)] (bits=4) or [M, K] (bits=8); zeros may be NULL; out [M, K]. */
int b200q_dequant(int bits, const uint8_t* codes, const void* scales, const void* zeros, void* out,
                  int64_t M, int64_t K, int group_size, int scale_dtype, int out_dtype, void* stream);

/* y[b, n] = sum_k x[b, k] * (code[n, k] - zero[n, k/G]) * scale[n, k/G], fp32 accumulation,
 * saturated to the finite range of act_dtype.  One implementation serves the reference's
 * `metal`, `metal_parallel` and `metal_tiled` launches of q4/q8_matvec_decode
 * (ops/quant_ops.py:407-506, 529-631; kernels/q{4,8}_matvec_decode{,_parallel,_tiled}.metal).
 * If `residual` is not NULL the result is cast(residual + cast(y)), the residual_add that
 * follows the down projection in quantized_mlp_block (ops/mlp_block_ops.py:360-361;
 * kernels/residual_add.metal).  x [B, K], y and residual [B, N] in act_dtype. */
int b200q_qmatvec(int bits, const void* x, const uint8_t* codes, const void* scales, const void* zeros,
                  const void* residual, void* y, int B, int64_t N, int64_t K, int group_size,
                  int act_dtype, int scale_dtype, void* stream);

/* The same matvec with the RMSNorm (and residual add) that precedes it fused in: the rows fed to the
 * projection are rmsnorm(x + residual_in) (residual_in may be NULL).  Replaces rms_norm followed by the
 * QKV matvec of llama_layer_decode_step (ops/llama_layer_ops.py:255-259,
 * ops/quantized_decode_block_ops.py:113-131).  z_out / normed_out are written when not NULL. */
int b200q_norm_qmatvec(int bits, const void* x, const void* residual_in, const void* norm_weight, int norm_w_dtype,
                       float eps, void* z_out, void* normed_out, const uint8_t* codes, const void* scales,
                       const void* zeros, const void* residual, void* y, int B, int64_t N, int64_t K,
                       int group_size, int act_dtype, int scale_dtype, void* stream);

/* Gate and up projections of the same rows in one launch, with the SwiGLU that follows them:
 * gate = Wg x, up = Wu x (each rounded to act_dtype), act = cast(silu(gate) * up),
 * silu(g) = g / (1 + exp(-g)).  Any of gate_out / up_out / act_out may be NULL.  Replaces
 * q4/q8_gate_up_matvec_tiled (ops/quant_ops.py:634-738; kernels/q{4,8}_gate_up_matvec_tiled.metal)
 * plus fused_swiglu (ops/activation_ops.py:118-153; kernels/fused_swiglu.metal).
 *
 * Optional fused prologue (norm_weight != NULL): the rows fed to the projections are
 * rmsnorm(x + residual_in) as in quantized_mlp_block (ops/mlp_block_ops.py:339-340;
 * kernels/residual_add.metal, kernels/rms_norm.metal); z_out = cast(x + residual_in) and
 * normed_out = cast(z * rsqrt(mean(z^2) + eps) * norm_weight) are written when not NULL.
 * residual_in may be NULL (z = x); norm_weight [K] is read in norm_w_dtype. */
int b200q_gate_up_swiglu(int bits, const void* x, const uint8_t* gate_codes, const uint8_t* up_codes,
                         const void* gate_scales, const void* up_scales, const void* gate_zeros,
                         const void* up_zeros, void* gate_out, void* up_out, void* act_out,
                         const void* residual_in, const void* norm_weight, int norm_w_dtype, float eps,
                         void* z_out, void* normed_out, int rows, int64_t N, int64_t K, int group_size,
                         int act_dtype, int scale_dtype, void* stream);

/* out = cast(silu(gate) * up) on [rows, dim].  Replaces kernels/swiglu.metal and
 * kernels/fused_swiglu.metal (ops/activation_ops.py:91-153). */
int b200q_swiglu(const void* gate, const void* up, void* out, int64_t rows, int64_t dim, int dtype, void* stream);

/* out = cast(float(x) + float(residual)).  Replaces kernels/residual_add.metal
 * (ops/fused_ops.py:155-180). */
int b200q_residual_add(const void* x, const void* residual, void* out, int64_t n, int dtype, void* stream);

/* z = cast(x + residual) (residual may be NULL: z = x), y = cast(z * rsqrt(mean(z^2) + eps) * w).
 * z_out may be NULL.  Replaces kernels/rms_norm.metal and kernels/rmsnorm_residual.metal
 * (ops/norm_ops.py:55-85, ops/fused_ops.py:212-241).  x [rows, D]; weight [D] in w_dtype. */
int b200q_rmsnorm_residual(const void* x, const void* residual, const void* weight, void* y, void* z_out,
                           int64_t rows, int64_t D, float eps, int dtype, int w_dtype, void* stream);

/* page_ids[b] = block_table[b, positions[b] / page_size]; offsets[b] = positions[b] % page_size.
 * Replaces kernels/block_table_lookup.metal (ops/paged_kv_ops.py:155-182). */
int b200q_block_table_lookup(const int32_t* block_table, const int32_t* positions, int32_t* page_ids,
                             int32_t* offsets, int B, int max_blocks, int page_size, void* stream);

/* Paged quantized-KV GQA decode attention.  For every (b, hq): hkv = hq / (Hq/Hkv); over the
 * valid tokens j < min(lengths[b], max_blocks*page_size) whose block-table entry is >= 0,
 * out = softmax(scale * q . Khat_j) . Vhat_j with Khat = fp16((code - 128|8) * k_scale).
 * A sequence with no valid token writes zeros.  Replaces
 * kernels/q{4,8}_paged_gqa_decode_attention.metal as launched by
 * _metal_q{8,4}_paged_gqa_decode_attention (ops/paged_quantized_kv_ops.py:549-629).
 *   q, out      [B, Hq, D] in q_dtype (the reference's [B,1,Hq,D])
 *   k/v codes   [num_pages, page_size, Hkv, D] (bits=8) or [.., ceil(D/2)] (bits=4)
 *   k/v scales  [num_pages, page_size, Hkv, ceil(D/group)] in scale_dtype
 *   block_table [B, max_blocks] int32, lengths [B] int32
 *   workspace   b200q_paged_gqa_workspace_bytes(B, Hq, Hkv, D) bytes of scratch (split-KV partials)
 */
size_t b200q_paged_gqa_workspace_bytes(int B, int Hq, int Hkv, int D);
int b200q_paged_gqa_decode(int bits, const void* q, const uint8_t* k_codes, const uint8_t* v_codes,
                           const void* k_scales, const void* v_scales, const int32_t* block_table,
                           const int32_t* lengths, void* out, void* workspace, size_t workspace_bytes,
                           int B, int Hq, int Hkv, int D, int page_size, int64_t num_pages, int max_blocks,
                           int group_size, float scale, int q_dtype, int scale_dtype, void* stream);

/* The same attention restricted to a sliding window with optional attention sinks: of the valid tokens
 * j < L = min(lengths[b], max_blocks*page_size) only j < sink_tokens and j >= L - window_size take part
 * (the decode row of the reference's "sliding_window" / "sliding_window_sink" masks,
 * build_sparse_attention_mask, ops/sparse_attention_ops.py:85-105, with the query at position L - 1).
 * The reference has this over a quantized cache only as a pure-MLX scaffold
 * (reference_sparse_paged_quantized_kv_gqa_decode_attention, ops/paged_quantized_kv_ops.py:669-714, and
 * ops/quantized_kv_cache_ops.py:544-603, whose Metal backend raises NotImplementedError); here the split-KV
 * kernel skips the pages that hold no attended position, so the cost follows sink_tokens + window_size, not
 * the context length.  window_size must be > 0; sink_tokens >= 0.  Other arguments as above. */
int b200q_paged_gqa_decode_window(int bits, const void* q, const uint8_t* k_codes, const uint8_t* v_codes,
                                  const void* k_scales, const void* v_scales, const int32_t* block_table,
                                  const int32_t* lengths, void* out, void* workspace, size_t workspace_bytes,
                                  int B, int Hq, int Hkv, int D, int page_size, int64_t num_pages, int max_blocks,
                                  int group_size, float scale, int q_dtype, int scale_dtype, int sink_tokens,
                                  int window_size, void* stream);

/* The same attention under a block-sparse mask: with L = min(lengths[b], max_blocks*page_size) the query sits at
 * position L - 1 and key j < L takes part iff block_mask[(L-1)/block_size][j/block_size] != 0 (the decode row of the
 * reference's "block_sparse" pattern, build_sparse_attention_mask, ops/sparse_attention_ops.py:98-107; its causal
 * bound j <= L - 1 holds for every cached token).  The reference has this over a quantized cache only as the pure-MLX
 * scaffold of ops/paged_quantized_kv_ops.py:669-714.
 *   block_mask   [n_qblocks, n_kblocks] bytes in device memory; a row or column index beyond it counts as masked
 *   page_scratch B*(max_blocks+1) int32 of device scratch, or NULL.  With scratch and block_size a multiple of
 *                page_size, one small kernel compacts every sequence's attended pages into a private block table and
 *                the dense kernels above run on it (cost follows the attended pages); otherwise the one-warp-per-head
 *                kernel tests every token.
 * A sequence whose mask row hides every key writes zeros (the reference scaffold degenerates to a uniform average
 * over all keys there).  Other arguments as b200q_paged_gqa_decode. */
int b200q_paged_gqa_decode_block_sparse(int bits, const void* q, const uint8_t* k_codes, const uint8_t* v_codes,
                                        const void* k_scales, const void* v_scales, const int32_t* block_table,
                                        const int32_t* lengths, void* out, void* workspace, size_t workspace_bytes,
                                        const uint8_t* block_mask, int n_qblocks, int n_kblocks, int block_size,
                                        int32_t* page_scratch, int B, int Hq, int Hkv, int D, int page_size,
                                        int64_t num_pages, int max_blocks, int group_size, float scale, int q_dtype,
                                        int scale_dtype, void* stream);

/* Decode attention over an UNQUANTISED paged cache with grouped query heads: K/V pages
 * [num_pages, page_size, Hkv, D] in `dtype` (B200Q_F16 or B200Q_BF16, also the type of q and out), D <= 128,
 * fp32 scores and sums.  Replaces kernels/paged_decode_attention{,_threadgroup,_d64,_d128}.metal as launched by
 * paged_decode_attention (ops/paged_kv_ops.py:307-360; Hq == Hkv there) and serves
 * reference_paged_gqa_decode_attention's shapes (ops/gqa_ops.py:307-340; Hq a multiple of Hkv).  Tokens whose
 * block-table entry is negative take no part; a sequence with no valid token writes zeros.
 * workspace: b200q_paged_fp16_gqa_workspace_bytes(B, Hq, Hkv, max_blocks) bytes (0 when one CTA per head suffices). */
size_t b200q_paged_fp16_gqa_workspace_bytes(int B, int Hq, int Hkv, int max_blocks);
int b200q_paged_fp16_gqa_decode(const void* q, const void* k_pages, const void* v_pages, const int32_t* block_table,
                                const int32_t* lengths, void* out, void* workspace, size_t workspace_bytes, int B, int Hq,
                                int Hkv, int D, int page_size, int64_t num_pages, int max_blocks, float scale, int dtype,
                                void* stream);

/* The same attention for callers that cannot allocate device memory at all.  (No counterpart in the
 * reference: its runtime allocates every kernel output itself.)  Some hosts of this library may not
 * call cudaMalloc: a plugin running inside another runtime's memory budget, a worker that must not
 * touch the allocator while a CUDA graph is being captured, or a process whose device memory was
 * handed out entirely at start-up.  They still own q, the cache and `out`, but have nowhere to put
 * the split-KV partial results that b200q_paged_gqa_decode keeps in its `workspace` argument.  This
 * entry point keeps them in a fixed array of b200q_paged_gqa_static_scratch_bytes() (8 MiB) that is
 * part of the library image: every GPU that loads the library holds those 8 MiB until the process
 * exits.  It allocates nothing and calls no allocating routine.
 *   - Limit: returns B200Q_ERR_STATIC_SCRATCH when
 *     b200q_paged_gqa_workspace_bytes(B, Hq, Hkv, D) exceeds the array (for 32 query heads of
 *     head_dim 128 over 8 kv heads that is a batch of 200 sequences); use the workspace variant then.
 *   - The first call on each device looks up the array's device address (with that device current)
 *     and remembers it.  Make that first call outside any stream capture.
 *   - Every call on a device shares the one array.  Nothing in it has to start at zero: each call
 *     writes every partial result it later reads, so leftovers of the previous call are never seen.
 *     Two calls whose kernels overlap on the GPU (different streams, or graphs replayed
 *     concurrently) would overwrite each other's partials: keep calls on one device stream-ordered.
 *   - Dense attention only (there is no windowed form of this entry point).  Shapes that run the
 *     one-warp-per-head kernel (head_dim != 128, bf16 q, page sizes other than 16 ...) use no scratch and are
 *     never refused for size.
 * Arguments and results are those of b200q_paged_gqa_decode without workspace / workspace_bytes. */
size_t b200q_paged_gqa_static_scratch_bytes(void);
int b200q_paged_gqa_decode_static(int bits, const void* q, const uint8_t* k_codes, const uint8_t* v_codes,
                                  const void* k_scales, const void* v_scales, const int32_t* block_table,
                                  const int32_t* lengths, void* out, int B, int Hq, int Hkv, int D,
                                  int page_size, int64_t num_pages, int max_blocks, int group_size, float scale,
                                  int q_dtype, int scale_dtype, void* stream);

/* Decode-layer glue: split a fused QKV row [B, (Hq + 2 Hkv) * D] (fp16), apply the interleaved-pair
 * rotary embedding at positions[b] to q and k (tables cos/sin [table_len, D/2] fp32, as
 * reference_apply_rope, ops/rope_ops.py:61-75, after reference_gqa_qkv_split_rope,
 * ops/gqa_ops.py:148-160), write q_out [B, Hq, D], and append k / v - quantised with the cache rule
 * of ops/paged_quantized_kv_ops.py:146-175 - to page block_table[b, pos / page_size], slot
 * pos % page_size.  The reference has no quantised append (its update kernels copy the whole cache,
 * kernels/paged_kv_cache_update.metal); this is the in-place form the decode stack needs.
 * A position outside [0, table_len) leaves q / k unrotated, and a position whose block-table entry is negative
 * or >= num_pages appends nothing; both are recorded in the status word (b200q_device_status events 6 and 7). */
int b200q_rope_kv_append(const void* qkv, const float* cos_table, const float* sin_table,
                         const int32_t* positions, const int32_t* block_table, void* q_out, uint8_t* k_codes,
                         uint8_t* v_codes, void* k_scales, void* v_scales, int bits, int B, int Hq, int Hkv,
                         int D, int page_size, int64_t num_pages, int max_blocks, int group_size, int table_len,
                         void* stream);

/* b200q_rope_kv_append followed by b200q_paged_gqa_decode over the cache that now holds the new token, as one entry
 * point: the attention stage of llama_layer_decode_step (ops/llama_layer_ops.py:262-330: reference_gqa_qkv_split_rope,
 * cache update, GQA decode attention) on a paged quantized cache.  fp16 rows and fp16 cache scales.  For small batches
 * (batch x kv heads up to a quarter of the SM count) the whole stage is ONE kernel: a thread-block cluster per
 * (sequence, kv head) rotates q, appends the head's k / v to the page of positions[b], walks the sequence's pages and
 * merges its partial results through distributed shared memory - no workspace traffic and no merge launch.  Larger
 * batches run the two stages back to back; q_scratch [B, Hq, D] then receives the rotated queries (it may be NULL only
 * when the one-kernel form is known to apply) and workspace is that of b200q_paged_gqa_decode.  lengths[b] must already
 * count the new token (positions[b] + 1).  The result equals the two separate calls to within fp32 merge order. */
int b200q_rope_append_paged_gqa_decode(const void* qkv, const float* cos_table, const float* sin_table,
                                       const int32_t* positions, int table_len, int bits, uint8_t* k_codes, uint8_t* v_codes,
                                       void* k_scales, void* v_scales, const int32_t* block_table, const int32_t* lengths,
                                       void* out, void* q_scratch, void* workspace, size_t workspace_bytes, int B, int Hq,
                                       int Hkv, int D, int page_size, int64_t num_pages, int max_blocks, int group_size,
                                       float scale, void* stream);

/* Kernel launches the attention stage takes on the current device for head_dim 128 / page size 16 caches: 1 when the
 * cluster kernel applies (with or without the append), else 2 (split-KV + merge) plus 1 for the append.  For callers
 * that report launch counts; no counterpart in the reference. */
int b200q_attention_stage_launches(int B, int Hkv, int with_append);

/* Symmetric group-wise quantisation of KV rows with the rule of the reference cache
 * (_quantize_group_symmetric_8 / _4, ops/paged_quantized_kv_ops.py:146-153, 168-175, as applied by quantize_kv_pages,
 * :194-292): per group of `group_size` values along D, scale = max(max|v|, 1e-8) / (127 | 7) in fp32 (stored fp16),
 * code = clip(rint(v / scale), -127|-7, 127|7) + (128 | 8).  values [rows, D] in in_dtype (fp16 / bf16);
 * codes [rows, D] (bits=8) or [rows, ceil(D/2)] (bits=4, low nibble = even d); scales [rows, ceil(D/group)] fp16. */
int b200q_quantize_kv(int bits, const void* values, uint8_t* codes, void* scales, int64_t rows, int D, int group_size,
                      int in_dtype, void* stream);

/* Tensor-parallel glue (no counterpart in the reference, which is single-device): all-gather of an
 * activation shard over NVLink peer memory.  `local` [rows, row_bytes_local] is this rank's shard;
 * peer_full[r] / peer_flags[r] are HOST arrays of `world` device pointers: rank r's full buffer
 * [rows, world * row_bytes_local] and its flag array (uint32[world], zero-initialised once) as mapped on
 * THIS GPU (symmetric memory; entry `rank` is the local copy).  `epoch` is a device uint32 owned by this rank,
 * zero-initialised once, one per full buffer; all ranks must call in the same order.  One small kernel
 * stores the shard into column block `rank` of every rank's full buffer, publishes a sequence number and
 * waits (bounded; b200q_device_status() reports B200Q_ERR_DEVICE_WAIT-class events) until all shards of
 * this call have arrived.  row_bytes_local must be a multiple of 16.  Stream-ordered, capturable. */
int b200q_peer_allgather(const void* local, void* const* peer_full, uint32_t* const* peer_flags, uint32_t* epoch,
                         int rank, int world, int rows, int64_t row_bytes_local, void* stream);

/* The same exchange fused into the kernels (no stand-alone launch): an exchange buffer is registered once
 * under a slot number (0..15) - pointers as for b200q_peer_allgather, plus `counter`, a device uint32 owned by
 * this rank and zero-initialised once.  b200q_tp_next(in_slot, out_slot) then applies to the NEXT call of
 * b200q_qmatvec / b200q_norm_qmatvec / b200q_gate_up_swiglu / b200q_paged_gqa_decode made by this thread
 * (-1 = none):
 *   out_slot: the kernel stores its result rows (for gate/up: the SwiGLU rows) into column block `rank` of
 *             every rank's full buffer instead of (y / act_out / out may then be NULL) or besides the local
 *             output, and its last CTA publishes the sequence number;
 *   in_slot:  the kernel's input `x` is this rank's view of that slot's full buffer; the kernel waits (bounded)
 *             for all source ranks before reading it.
 * b200q_rope_append_paged_gqa_decode honours out_slot as b200q_paged_gqa_decode does.
 * Only the tensor-core matvec kernels and the split-KV / cluster attention kernels support this (B200Q_ERR_UNSUPPORTED
 * otherwise); batch rows <= 16.  The sharded result equals the unsharded one bit for bit. */
int b200q_tp_register(int slot, void* const* peer_full, uint32_t* const* peer_flags, uint32_t* epoch, uint32_t* counter,
                      int rank, int world);
int b200q_tp_next(int in_slot, int out_slot);

/* Packet form of a registered exchange slot (packets != 0): the slot's full buffers then hold one 32-bit word per
 * 16-bit element - the element in the low half, the low bits of the exchange's sequence number in the high half -
 * so they are TWICE the size of the plain rows, must start zeroed, and are read only by kernels called with this
 * slot as in_slot (the pointer passed as `x` is the packet buffer).  A writer kernel stores each element and its
 * "arrived" mark in one 4-byte peer store; a reader polls the packets it loads (bounded, event 5).  No system-scope
 * fence, flag word or counter crosses NVLink: an exchange costs one one-way store latency.  The flag pointers given
 * to b200q_tp_register are unused in this form.  Results are the same bits as in the plain form.  Readers of a packet
 * buffer take batches of up to 4 rows (B200Q_ERR_UNSUPPORTED above that). */
int b200q_tp_set_packets(int slot, int packets);

/* Diagnostics (no counterpart in the reference): one CTA waits on a shared-memory barrier that nothing arrives on, with
 * the bounded wait the matvec and attention kernels use, for `limit` probes (1..65536).  The wait runs out, the kernel
 * returns, b200q_device_status() then reports event 1 and *probes_out (device uint32, may be NULL) holds `limit`.
 * Lets a caller check that an expired device wait reaches the host as a status instead of a hang. */
int b200q_wait_expiry_selftest(unsigned limit, uint32_t* probes_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H_ */

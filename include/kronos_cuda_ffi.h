/*
 * kronos_cuda_ffi.h — C ABI of the B200 (sm_100a) backend for kronos-2t's quantized
 * decode / prefill hot path.
 *
 * Conventions follow the reference's include/kronos_ffi.h:12-30 and
 * src/ffi/mobile_ffi.rs:32-41,159-168: opaque handles, int32_t 0 / -1 returns,
 * `*_last_error()` returns a NUL-terminated string that stays valid until the next
 * mutating call on the same handle, NULL handles are tolerated, nothing unwinds
 * across the boundary.  One caller at a time per handle (the reference's forward
 * methods are `&mut self`).
 *
 * Matrices are passed in the byte formats the reference stores in .k2tb/.k2tm files;
 * the backend copies them into HBM (repacked for coalesced streaming) and owns that
 * memory.  Host buffers only need to live for the duration of the call.
 *
 * There is no CPU fallback: every entry point fails with an error when no CUDA
 * device is usable.
 */
#ifndef KRONOS_CUDA_FFI_H
#define KRONOS_CUDA_FFI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct KronosCudaContext KronosCudaContext;
typedef struct KronosCudaMatrix KronosCudaMatrix;

/* Matrix kinds use the tags of the .k2tb container (src/model/real_llm.rs:3805-3823,
 * matrix tags in save_bipolar 3705-3895). */
#define KRONOS_CUDA_MATRIX_BIPOLAR 0u /* FusedBipolarLutMatrix, src/kernels/simd_lut.rs:1754-1836 */
#define KRONOS_CUDA_MATRIX_NF      2u /* NfSdotMatrix (bits 5,4,3; 2 = E8Q2), simd_lut.rs:4796-5226 */

/* Upload flag: reorder gate_up rows from [gate; up] into 64-row [gate_64(ic), up_64(ic)] blocks,
 * as Nibble4SdotMatrix::from_bipolar_with_perm (simd_lut.rs:3297-3327) and
 * NfSdotMatrix::to_gate_up_interleaved (5500-5524) do for the CPU path. */
#define KRONOS_CUDA_UPLOAD_GATE_UP_INTERLEAVE 1u

/* A weight matrix exactly as the reference holds it after loading a .k2tb file.
 * Replaces the `&LinearBackend` borrows of LayerBorrow (src/backend/metal_gpu.rs:428-439),
 * extended to bipolar matrices.
 *   BIPOLAR: bits = planes (4..6); data0 = interleaved planes
 *            [stripes][cols/8][planes][16]; data1 = bf16 scales [stripes][cols/64][16] (bytes, LE).
 *   NF:      bits = 5,4,3 or 2 (E8Q2); data0 = pair_stream; data1 = tail_stream (len1 may be 0);
 *            codebook = the 16 stored int8 centroids; scale_group_chunks = 64-col chunks per scale. */
typedef struct KronosCudaMatrixDesc {
    uint32_t kind;
    uint32_t rows;
    uint32_t cols;
    uint32_t bits;
    uint32_t scale_group_chunks;
    int8_t codebook[16];
    const uint8_t *data0;
    size_t len0;
    const uint8_t *data1;
    size_t len1;
} KronosCudaMatrixDesc;

/* ---- context ------------------------------------------------------------------------------ */

/* Opens CUDA device `device` and creates the stream all calls of this context are ordered on.
 * Returns NULL when the device cannot be used (see kronos_cuda_last_error(NULL)).
 * Counterpart of MetalLlamaEngine's device/queue acquisition in try_new (metal_gpu.rs:1196-1206). */
KronosCudaContext *kronos_cuda_context_create(int32_t device);
void kronos_cuda_context_destroy(KronosCudaContext *ctx);
/* Last error of `ctx`, or of the last failed context_create when ctx is NULL. */
const char *kronos_cuda_last_error(const KronosCudaContext *ctx);
/* Blocks until everything queued on the context's stream has finished. */
int32_t kronos_cuda_synchronize(KronosCudaContext *ctx);
/* Number of kernels this context has launched so far (own kernels only). */
uint64_t kronos_cuda_launch_count(const KronosCudaContext *ctx);
/* Routes subsequent launches of this context onto an existing cudaStream_t (NULL = the context's
 * own stream).  Lets a host harness time calls with events it records on its own stream. */
int32_t kronos_cuda_set_stream(KronosCudaContext *ctx, void *cuda_stream);

/* ---- matrices ----------------------------------------------------------------------------- */

/* Copies a matrix to HBM in the backend's streaming layout.  Replaces the buffer wrapping of
 * MetalLlamaEngine::try_new (metal_gpu.rs:1094-1172) and, for bipolar matrices,
 * RealLlamaEngine::repack_sdot (real_llm.rs:3657-3702). */
KronosCudaMatrix *kronos_cuda_matrix_upload(KronosCudaContext *ctx, const KronosCudaMatrixDesc *desc,
                                            uint32_t flags);
/* A second, independent HBM copy of an uploaded matrix (device-to-device).  Benchmarks rotate over
 * such copies so that consecutive launches never find their weights in L2.  No counterpart in the
 * reference. */
KronosCudaMatrix *kronos_cuda_matrix_clone(KronosCudaContext *ctx, const KronosCudaMatrix *m);
void kronos_cuda_matrix_free(KronosCudaContext *ctx, KronosCudaMatrix *m);
/* Bytes the matrix occupies in the reference's file format (the "algorithmic" weight bytes)
 * and in HBM. */
size_t kronos_cuda_matrix_file_bytes(const KronosCudaMatrix *m);
size_t kronos_cuda_matrix_device_bytes(const KronosCudaMatrix *m);

/* Host-only diagnostic: writes the HBM image kronos_cuda_matrix_upload would copy (code planes, then
 * bf16 scales) into `out` and returns its size in bytes; with out == NULL or cap too small nothing is
 * written.  Needs no GPU.  Returns 0 for a malformed descriptor.  No counterpart in the reference. */
size_t kronos_cuda_matrix_image(const KronosCudaMatrixDesc *desc, uint32_t flags, uint8_t *out, size_t cap);

/* ---- kernels, host buffers (copies to and from the device happen inside the call) ---------- */

/* Int8ChunkActivation::populate_fwht / populate_rmsnorm_fwht (simd_lut.rs:2954-2991):
 * optional (x*inv_rms)*norm_w, signed FWHT-64 with global chunk index chunk0 + c, per-chunk int8.
 * x[n_tok][cols]; norm_w[cols] or NULL; inv_rms[n_tok] or NULL (required with norm_w);
 * q[n_tok][cols], scales[n_tok][cols/64], sums[n_tok][cols/64]. */
int32_t kronos_cuda_fwht_quant(KronosCudaContext *ctx, const float *x, size_t n_tok, size_t cols,
                               const float *norm_w, const float *inv_rms, uint64_t chunk0,
                               int8_t *q, float *scales, int32_t *sums);

/* nibble4_sdot_stripe_range_raw (simd_lut.rs:3536-3582) / nf_sdot_stripe_range_raw (5687-5760) for
 * n_tok = 1 and the batch forms (4101-4331, 6689-7029) for any n_tok >= 1 (up to 15 tokens run as weight passes
 * of 4 tokens inside the call; 16 and more in one launch whose integer dots run on the tensor cores - the same results
 * either way; a call that asks for int_dots always takes the passes), over all rows:
 * out[t*out_stride + r] = sum over chunks of fmaf((float)dot*xs, w_scale, acc), ascending chunks,
 * chunks with xs == 0 skipped.  int_dots (optional, [n_tok][rows][cols/64]) receives the exact
 * int32 chunk dots (bipolar: 2*sum(u*q) - (2^B-1)*xsum; NF: sum(cb[idx]*q)). xsum may be NULL for NF. */
int32_t kronos_cuda_gemv(KronosCudaContext *ctx, const KronosCudaMatrix *m, const int8_t *xq,
                         const float *xs, const int32_t *xsum, size_t n_tok, float *out,
                         size_t out_stride, int32_t *int_dots);

/* DenseMoeRouter::route_sorted (src/model/sparse_moe.rs:86-182): logits = W x_norm (+ bias), scoring 0 = softmax over all
 * experts, 1 = softmax over the selected logits, 2 = sigmoid; the top_k experts by score (the earlier expert wins ties),
 * optionally renormalised (norm_topk), returned in ascending expert order.  Host buffers: router_w[n_experts][hidden],
 * router_bias[n_experts] or NULL, x_norm[hidden]; route_ids / route_w receive min(top_k, n_experts) entries.  Returns that
 * count, -1 on error.  Non-finite inputs still yield ids inside [0, n_experts) (unranked slots are expert i, weight 0). */
int32_t kronos_cuda_moe_route(KronosCudaContext *ctx, const float *router_w, const float *router_bias, const float *x_norm,
                              uint32_t n_experts, uint32_t hidden, uint32_t top_k, int32_t norm_topk, uint32_t scoring,
                              uint32_t *route_ids, float *route_w);

/* LinearBackend::forward for the Nibble4 / NfSdot arms (real_llm.rs:825-858) fed by
 * Int8ChunkActivation::populate_fwht: y[t] = W * rotate_quantize(x[t]).  x[n_tok][cols] fp32 in,
 * out[n_tok][rows] fp32.  This is the host-buffer call the benchmark's end-to-end number uses. */
int32_t kronos_cuda_linear(KronosCudaContext *ctx, const KronosCudaMatrix *m, const float *x,
                           size_t n_tok, float *out);
/* The same call without the final wait: copies and kernels are queued on the context's stream and the call returns.
 * x and out must stay valid (and should be page-locked, or the copies are staged synchronously) until
 * kronos_cuda_synchronize(ctx), which also reports a device-side failure of any queued call.  Calls queue in order,
 * so independent projections (a host that evaluates several matrices before it needs any result) overlap their
 * copies with one another's kernels.  No counterpart in the reference (its CPU LinearBackend::forward is synchronous). */
int32_t kronos_cuda_linear_async(KronosCudaContext *ctx, const KronosCudaMatrix *m, const float *x,
                                 size_t n_tok, float *out);

/* ---- kernels, device buffers (no copies; pointers are device addresses on ctx's device) ---- */

int32_t kronos_cuda_fwht_quant_dev(KronosCudaContext *ctx, const float *d_x, size_t n_tok, size_t cols,
                                   const float *d_norm_w, const float *d_inv_rms, uint64_t chunk0,
                                   int8_t *d_q, float *d_scales, int32_t *d_sums);
int32_t kronos_cuda_gemv_dev(KronosCudaContext *ctx, const KronosCudaMatrix *m, const int8_t *d_xq,
                             const float *d_xs, const int32_t *d_xsum, size_t n_tok, float *d_out,
                             size_t out_stride, int32_t *d_int_dots);

/* ---- whole-token engine ------------------------------------------------------------------------ */

typedef struct KronosCudaEngine KronosCudaEngine;

/* LlamaConfig scalars the device forward needs (src/model/real_llm.rs:91-457), as MetalLlamaEngine::try_new
 * receives them through `cfg`, plus the KV format (kv_bits: 8 = int8 Hadamard cache, 4 = NF4 Hadamard cache as
 * selected by RealLlamaEngine::set_kv_bits, real_llm.rs:1731-1735). */
typedef struct KronosCudaEngineConfig {
    /* sizeof(KronosCudaEngineConfig) as the caller compiled it: kronos_cuda_engine_create refuses any other value, so
     * a binding written against an older or shorter layout fails with a message instead of being read past its end. */
    uint32_t struct_size;
    uint32_t hidden_size, num_layers, num_attention_heads, num_key_value_heads, head_dim,
             intermediate_size, vocab_size, max_seq_len;
    float rms_norm_eps;
    int32_t qk_norm_after_rope;
    uint32_t kv_bits;
    /* MoeGeometry (metal_gpu.rs:443-456), all zero for a dense model: experts per MoE layer, routes per token,
     * renormalise the top-k weights, expert MLP width, NF bits (2..5) and scale group of the expert matrices, bytes of
     * one .k2tm expert record (nf_expert_byte_layout, moe_800b.rs:1330-1383).  moe_norm_topk: bit 0 = renormalise the
     * top-k weights, bits 8.. = MoeRouterScoring tag (sparse_moe.rs:28-53: 0 softmax over all experts, 1 top-k softmax,
     * 2 sigmoid).  Shared experts are not accepted. */
    uint32_t moe_num_experts, moe_top_k, moe_norm_topk, moe_d_ff, moe_bits, moe_scale_group_chunks;
    uint64_t moe_expert_bytes;
    /* Tensor parallelism over the GPUs of one node, one process (and one engine) per rank; all zero / tp_size <= 1 for a
     * single device.  No counterpart in the reference.  The sizes above are then the rank's LOCAL ones: its query / kv
     * heads, its MLP columns (intermediate_size) and its lm_head rows (vocab_size); vocab_total is the whole vocabulary;
     * o_chunk0 / down_chunk0 are the global indices of the first 64-column chunk of this rank's slice of o_proj's and
     * down_proj's input, so that the activations are rotated with their global block index.  The matrices passed to
     * kronos_cuda_engine_create are the rank's slices in the ordinary file formats (kronos_2t_b200/tp.py cuts them). */
    uint32_t tp_size, tp_rank, o_chunk0, down_chunk0, vocab_total;
    /* Expert parallelism for sparse-MoE models (no counterpart in the reference): ep_size ranks, one engine each; every
     * rank keeps the dense tensors (attention, norms, lm_head, router) whole and only the experts e with
     * e % ep_size == ep_rank.  A token's routed experts run on their owners; the ranks' partial weighted sums are added
     * in rank order inside the norm kernel that follows the MoE block (the exchange of kronos_cuda_engine_tp_handle /
     * _tp_attach, with ep_size handles).  Zero / ep_size <= 1 for one device; not combined with tp_size > 1. */
    uint32_t ep_size, ep_rank;
    /* Sliding-window + attention-sink KV ring (RealLlamaEngine::set_kv_sliding_window, real_llm.rs:1764-1790, as try_new
     * receives kv_window / kv_sinks, metal_gpu.rs:1196-1206): kv_window = 0 keeps the full causal context; otherwise
     * (>= 8) a token attends to the first kv_sinks positions and the last kv_window - kv_sinks ones, and cache rows live
     * in a ring (QuantKvRawPtrs::slot_of_pos, real_llm.rs:1116-1122).  kronos_cuda_engine_reconfigure_kv changes both. */
    uint32_t kv_window, kv_sinks;
    /* KRONOS_CUDA_ENGINE_* bits */
    uint32_t flags;
} KronosCudaEngineConfig;

/* flags: contexts longer than 512 positions are attended in the reference's summation order by default (logits and
 * greedy streams identical to the CPU path at any length).  With this bit the split-KV kernel serves them instead:
 * exact scores, partial sums merged in split order, so outputs agree with the CPU path to fp32 rounding only - faster
 * at long contexts, not bit-identical.  No counterpart in the reference. */
#define KRONOS_CUDA_ENGINE_SPLIT_KV_ATTENTION 1u

/* One decoder layer as borrowed from the host engine: counterpart of LayerBorrow
 * (src/backend/metal_gpu.rs:428-439).  Optional vectors are NULL when absent.  qkv_proj is the row
 * concatenation [q; k; v], gate_up_proj = [gate; up] (not interleaved), as stored in .k2tb files. */
typedef struct KronosCudaLayerDesc {
    const float *input_norm, *post_attn_norm;      /* [hidden] */
    const float *qkv_bias;                         /* [q_dim + 2 kv_dim] or NULL */
    const float *q_norm, *k_norm;                  /* [head_dim] or NULL */
    KronosCudaMatrixDesc qkv_proj, o_proj, gate_up_proj, down_proj;
    /* MoeLayerBorrow (metal_gpu.rs:418-426); moe_router_w == NULL for a dense layer.  On a MoE layer the FFN is the
     * router [moe_num_experts][hidden] fp32 (+ optional bias) and moe_num_experts expert records (.k2tm record layout:
     * codebooks at 0 / 16, gate_up pair_stream at 64, down pair_stream at the next multiple of 64) stored back to back
     * in moe_shard; gate_up_proj / down_proj then describe the layer's SHARED expert (SharedMoeExpert with NF matrices,
     * sparse_moe.rs:223-315: gate_up [2 inter][hidden], gate rows first, down [hidden][inter]) or have rows = 0 when
     * the layer has none, and moe_shared_gate_w is its sigmoid gate weight [hidden] or NULL. */
    const float *moe_router_w, *moe_router_bias;
    const uint8_t *moe_shard;
    size_t moe_shard_len;
    const float *moe_shared_gate_w;
} KronosCudaLayerDesc;

/* MetalLlamaEngine::try_new (metal_gpu.rs:1196-1206): copies every tensor to HBM, allocates the KV cache
 * for max_seq_len positions and the per-token workspace.  rope_cos_sin = build_rope_table()'s
 * [max_seq_len][head_dim] rows (cos half, sin half; real_llm.rs:9212-9236).  embed_bf16 = untied
 * embedding table [vocab][hidden] (all vocab_total rows on every rank under tensor parallelism) or NULL for
 * tied embeddings (the lm_head row, rotated back: embed_token_into, real_llm.rs:8063-8097).  Returns NULL on error (kronos_cuda_last_error(ctx)). */
KronosCudaEngine *kronos_cuda_engine_create(KronosCudaContext *ctx, const KronosCudaEngineConfig *cfg,
                                            const float *rope_cos_sin, const KronosCudaLayerDesc *layers,
                                            size_t n_layers, const float *final_norm,
                                            const KronosCudaMatrixDesc *lm_head, const uint16_t *embed_bf16);
void kronos_cuda_engine_destroy(KronosCudaEngine *engine);

/* MetalLlamaEngine::forward_tokens (metal_gpu.rs:1619-1627): runs n_tok tokens whose embeddings the
 * host supplies (embeds[n_tok][hidden]) at positions pos_start.., writes the logits of the last token
 * to last_logits[vocab] and, if all_logits is not NULL, of every token to all_logits[n_tok][vocab]. */
int32_t kronos_cuda_engine_forward_tokens(KronosCudaEngine *engine, const float *embeds, size_t n_tok,
                                          size_t pos_start, float *all_logits, float *last_logits);
/* Same with token ids; the embedding lookup runs on the device (RealLlamaEngine::forward_token /
 * forward_prompt, real_llm.rs:6455, 7407-7448). */
int32_t kronos_cuda_engine_forward_token_ids(KronosCudaEngine *engine, const uint32_t *tokens, size_t n_tok,
                                             size_t pos_start, float *all_logits, float *last_logits);
/* RealLlamaEngine::generate_greedy's decode loop (real_llm.rs:7879-7913) with the argmax on the device:
 * feeds first_token at pos_start, then n_steps times takes the argmax (first maximum) as the next
 * token.  out_tokens[n_steps] receives the chosen tokens; last_logits (optional) the logits that
 * produced the last one.  One CUDA graph replay per step, no host round trip inside the loop. */
int32_t kronos_cuda_engine_decode_greedy(KronosCudaEngine *engine, uint32_t first_token, size_t pos_start,
                                         size_t n_steps, uint32_t *out_tokens, float *last_logits);
/* kv_cache_bytes (metal_gpu.rs:1454-1617 family): bytes of KV cache held for `positions` positions. */
size_t kronos_cuda_engine_kv_bytes(const KronosCudaEngine *engine, size_t positions);
/* KV blobs in the reference's position-major export format (export_kv_positions / import_kv_positions, real_llm.rs:6213-6291;
 * KvSlotPtrs::export / import, src/model/kv_blob.rs:47-110): per position, per (layer, kv head): key row, key scale(s),
 * value row, value scale(s); kv_bytes_per_pos = 2 * layers * kv_heads * (row + scale bytes) (12,240 / 6,120 B for the 135M
 * shape with the int8 / NF4 cache).  A blob exported by the CPU engine imports here and vice versa (same kv_bits).
 * kv_export writes positions [lo, hi) and returns the byte count (-1 on error); kv_import restores positions [0, n).
 * Truncating a context needs no call: the host just continues at an earlier pos_start (truncate_context, 6294-6296). */
size_t kronos_cuda_engine_kv_bytes_per_pos(const KronosCudaEngine *engine);
int64_t kronos_cuda_engine_kv_export(KronosCudaEngine *engine, size_t lo, size_t hi, uint8_t *out, size_t cap);
int32_t kronos_cuda_engine_kv_import(KronosCudaEngine *engine, const uint8_t *data, size_t len, size_t n);
/* RealLlamaEngine::set_kv_bits / set_kv_sliding_window (real_llm.rs:1731-1790) as they reach a device backend
 * (MetalLlamaEngine::reconfigure_kv, metal_gpu.rs:1561): rebuilds the cache in format kv_bits (8 / 4) and geometry -
 * window = 0: the full causal context; otherwise the sliding-window + sink ring of QuantizedKvCache::new_with_opts
 * (real_llm.rs:1235-1257), taken only when 8 <= window and window + 512 < max_seq_len (else the full context is kept, as
 * in the reference), sinks capped at window / 2, sinks + (window - sinks + 512) cache rows per (layer, kv head).  With a
 * window every token is attended by causal_gqa_group_q4_or_window's arithmetic (real_llm.rs:8794-8988), bit for bit.
 * The cache contents are lost; the host continues at position 0.  Not combined with tensor / expert parallelism. */
int32_t kronos_cuda_engine_reconfigure_kv(KronosCudaEngine *engine, uint32_t kv_bits, size_t window, size_t sinks);
/* kv_sliding_window (real_llm.rs:1793-1803): returns 1 and the effective (window, sinks) when a ring is active, else 0. */
int32_t kronos_cuda_engine_kv_sliding_window(const KronosCudaEngine *engine, size_t *window, size_t *sinks);
/* Cache rows per (layer, kv head): max_seq_len, or sinks + ring length. */
size_t kronos_cuda_engine_kv_rows(const KronosCudaEngine *engine);
/* can_truncate_kv_to (real_llm.rs:1806-1821): may a host that stands at cur_pos continue at the earlier target_len
 * (speculative rollback, truncate_context) without reading ring rows that later positions have overwritten? */
int32_t kronos_cuda_engine_can_truncate_kv_to(const KronosCudaEngine *engine, size_t cur_pos, size_t target_len);
/* KV prefix snapshots (KvPrefixSnapshot::Q8 / Q4 with RealLlamaEngine::save_kv_prefix / restore_kv_prefix_slice,
 * real_llm.rs:5821-6155; the Metal backend's twin, metal_gpu.rs:1454-1617): a head-major copy of the first min(n, cur_pos)
 * cache rows of every (layer, kv head) - of the whole ring when a sliding window is active - for prompt caches and
 * speculative rollback.  Blob: 32-byte header ("K2TKVPFX", kv_bits, slots_per_head, heads, head_dim, 0, 0 as u32) followed by
 * the snapshot's four vectors in field order (key rows, value rows, key scales, value scales).  restore copies the first
 * min(slots_per_head, copy_slots) rows back (copy_slots = SIZE_MAX: all); the host then continues at its own position. */
size_t kronos_cuda_engine_kv_prefix_bytes(const KronosCudaEngine *engine, size_t n, size_t cur_pos);
int64_t kronos_cuda_engine_save_kv_prefix(KronosCudaEngine *engine, size_t n, size_t cur_pos, uint8_t *out, size_t cap);
int32_t kronos_cuda_engine_restore_kv_prefix(KronosCudaEngine *engine, const uint8_t *data, size_t len, size_t copy_slots);
/* Bytes of weights (reference file format) one decode step streams: all layer matrices + lm_head. */
size_t kronos_cuda_engine_weight_bytes(const KronosCudaEngine *engine);
/* Diagnostic: hidden state [hidden] after the last forwarded token (before the final norm). */
int32_t kronos_cuda_engine_read_hidden(KronosCudaEngine *engine, float *hidden);
/* Tensor parallel set-up (after create, before the first forward call; every rank in the same order):
 *   tp_handle: writes this rank's 64-byte inter-process handle (cudaIpcMemHandle_t) of its exchange buffer;
 *   tp_attach: takes the handles of all tp_size ranks (this rank's own entry is ignored), maps the peers' buffers and
 *              enables the exchanges: the partial outputs of o_proj and down_proj are summed over the ranks in rank
 *              order, the logits slices are concatenated, every rank ends a step with the same logits and next token.
 * The caller makes sure (a process-group barrier) that all ranks have attached before any of them runs a step.
 * With tied embeddings every rank also needs the whole lm_head for the token lookup: set_embedding_matrix uploads it. */
int32_t kronos_cuda_engine_tp_handle(KronosCudaEngine *engine, uint8_t handle[64]);
int32_t kronos_cuda_engine_tp_attach(KronosCudaEngine *engine, const uint8_t *handles /* [tp_size][64] */, size_t n_handles);
/* Also the route for an untied embedding table stored as an NF4 matrix (embed_nf4, real_llm.rs:1553, 8084-8087). */
int32_t kronos_cuda_engine_set_embedding_matrix(KronosCudaEngine *engine, const KronosCudaMatrixDesc *table);
/* tp_attach for a host that drives every rank from ONE process (one engine per GPU, the single-caller contract of
 * MetalLlamaEngine kept): `engines` = the tp_size (or ep_size) engines in rank order, this engine's own entry included;
 * peer access between their devices is enabled as needed.  Every engine of the group makes this call.
 * Waits for a peer are bounded: a rank whose peers never write (a peer was destroyed, or never ran the matching call)
 * gives up after KRONOS_CUDA_PEER_WAIT_POLLS polls per kernel (environment, default 4194304), its calls return -1
 * ("gave up waiting for a peer rank") and the context stays in that state: destroy and recreate the group. */
int32_t kronos_cuda_engine_tp_attach_local(KronosCudaEngine *engine, KronosCudaEngine *const *engines, size_t n_engines);
/* Diagnostic: routes of the last forwarded token through MoE layer `layer` (route_sorted, sparse_moe.rs:86-182):
 * up to 32 (expert id, weight) pairs in ascending expert order; returns their number (0 for a dense layer). */
size_t kronos_cuda_engine_read_routes(KronosCudaEngine *engine, uint32_t layer, uint32_t *experts, float *weights);
/* Diagnostic: attention output of the last layer for the last forwarded token, before o_proj:
 * [num_attention_heads * head_dim] (the `attn` vector of forward_token, real_llm.rs:6651-6700). */
int32_t kronos_cuda_engine_read_attention(KronosCudaEngine *engine, float *attention);
/* Same for an NF4 Hadamard cache (kv_bits = 4): packed indices [head_dim / 2] (byte 16h+i of a 64-value group
 * = columns 32h+i low nibble, 32h+16+i high nibble) and one bf16 scale per 64 values [head_dim / 64]
 * (store_hadamard_q4_head_raw, real_llm.rs:8646-8701). */
int32_t kronos_cuda_engine_read_kv_q4(KronosCudaEngine *engine, uint32_t layer, uint32_t kv_head, size_t position,
                                      uint8_t *k_q4, uint16_t *k_s16, uint8_t *v_q4, uint16_t *v_s16);
/* Diagnostic: phase trace of the whole-token decode kernel (the last step of the last decode_greedy call that
 * used it): global-timer readings in ns taken by CTA 0 at the start of the step, then around every phase
 * (activation prologue done / GEMV done / grid barrier passed; the attention phase has two marks).  Returns
 * the number of marks written (0 when that kernel is not in use).  No counterpart in the reference. */
size_t kronos_cuda_engine_decode_trace(KronosCudaEngine *engine, uint64_t *marks_ns, size_t cap);
/* Per-kernel-class timing of one greedy decode step (the CUDA counterpart of the Metal backend's KRONOS_DECODE_PROF
 * table, src/backend/metal_gpu.rs:963-1027): the step for `token` is launched kernel by kernel with a timing event after
 * every kernel, `reps` times (positions pos, pos + 1, ...), without programmatic overlap, so each kernel is timed alone on
 * a warm device.  Writes a text table (kernel class | launches per step | us per step | avg us | share) into table[cap]
 * (NUL-terminated, truncated to cap) and returns its full length, -1 on error.  The KV cache rows at pos .. pos + reps - 1
 * are overwritten.  With KRONOS_CUDA_DECODE_PROF=1 in the environment kronos_cuda_engine_decode_greedy prints this
 * table for its last position to stderr. */
int64_t kronos_cuda_engine_profile_step(KronosCudaEngine *engine, uint32_t token, size_t pos, uint32_t reps, char *table, size_t cap);
/* Diagnostic: 32 words the kernels of layer 0 leave when KRONOS_CUDA_ATTN_TRACE=1 was set at engine creation (SM clock
 * readings of query head 0 at the phase boundaries of the attention kernel).  No counterpart in the reference. */
size_t kronos_cuda_engine_debug_words(KronosCudaEngine *engine, uint64_t *out, size_t cap);
/* Diagnostic: one KV cache entry (layer, kv head, position): k_q8/v_q8[head_dim] rotated int8 values and
 * their fp32 scales - the contents of the reference's k_q8 / k_scales / v_q8 / v_scales slot
 * (KvCache, real_llm.rs:8303-8365). */
int32_t kronos_cuda_engine_read_kv(KronosCudaEngine *engine, uint32_t layer, uint32_t kv_head, size_t position,
                                   int8_t *k_q8, float *k_scale, int8_t *v_q8, float *v_scale);

/* ---- .k2tb compiled-model container ---------------------------------------------------------- */

/* Reader / writer of the reference's dense cache file (RealLlamaEngine::save_bipolar / load_bipolar,
 * real_llm.rs:3705-3895, 3902-4186; magics K2TBIPOLAR1, K2TKRONOS2/3/4/6).  Host code, no GPU needed.  The descriptors
 * handed out point into storage owned by the handle and stay valid until kronos_cuda_k2tb_close; they are exactly what
 * kronos_cuda_engine_create takes, so a cached model runs with no recompile.  Shapes (heads, head_dim, ...) are not in
 * the file: they come from the model's config.json as in the reference.  VQ2 / Q2c matrices are rejected.  The sparse-MoE
 * core (K2TKRONOS5, RealLlamaEngine::load_moe_from_files, real_llm.rs:5166-5519) opens through the same call (version 5);
 * its expert records live in the .k2tm shard below.  Errors: NULL / -1 and kronos_cuda_k2tb_last_error() (per thread). */
typedef struct KronosCudaK2tb KronosCudaK2tb;
KronosCudaK2tb *kronos_cuda_k2tb_open(const char *path);
void kronos_cuda_k2tb_close(KronosCudaK2tb *file);
const char *kronos_cuda_k2tb_last_error(void);
/* version = 1, 2, 3, 4 or 6; mode_words = the six RealWeightMode words (real_llm.rs:3805-3829). */
int32_t kronos_cuda_k2tb_info(const KronosCudaK2tb *file, uint32_t *version, uint64_t mode_words[6], size_t *n_layers);
/* Layer l as a KronosCudaLayerDesc; qkv_bias_len = elements of the bias (0 = none).  A MoE layer of a K2TKRONOS5 core gets
 * its router (moe_router_w / moe_router_bias); the caller adds moe_shard / moe_shard_len from kronos_cuda_k2tm_layer.  Fails
 * (message in kronos_cuda_k2tb_last_error) for layers with an o_proj bias or a shared expert, which the engine does not run. */
int32_t kronos_cuda_k2tb_layer(const KronosCudaK2tb *file, size_t l, KronosCudaLayerDesc *out, size_t *qkv_bias_len);
/* K2TKRONOS5 only: NF bits and scale group (64-column chunks per scale) of the expert matrices. */
int32_t kronos_cuda_k2tb_moe_info(const KronosCudaK2tb *file, uint64_t *expert_bits, uint64_t *expert_scale_group_chunks);
/* 1 when layer l is a MoE layer (then: its slot in the expert shard, router experts and hidden), 0 for a dense layer. */
int32_t kronos_cuda_k2tb_moe_layer(const KronosCudaK2tb *file, size_t l, uint64_t *moe_slot_idx, uint64_t *experts, uint64_t *hidden);

/* The .k2tm expert shard (K2tmShardHeader, src/model/moe_800b.rs:790-854; open_k2tm, src/model/sparse_moe.rs:685): mapped
 * read-only.  info: the header's seven words (layers, experts per layer, d_model, d_ff, scale_group_chunks, aligned expert
 * bytes, bits).  layer: the records of MoE slot `moe_slot_idx` (experts x aligned bytes, from expert_byte_offset(slot, 0)) -
 * what KronosCudaLayerDesc.moe_shard / moe_shard_len take; valid until kronos_cuda_k2tm_close. */
typedef struct KronosCudaK2tm KronosCudaK2tm;
KronosCudaK2tm *kronos_cuda_k2tm_open(const char *path);
void kronos_cuda_k2tm_close(KronosCudaK2tm *shard);
int32_t kronos_cuda_k2tm_info(const KronosCudaK2tm *shard, uint64_t words[7]);
int32_t kronos_cuda_k2tm_layer(const KronosCudaK2tm *shard, size_t moe_slot_idx, const uint8_t **records, size_t *len);
int32_t kronos_cuda_k2tb_head(const KronosCudaK2tb *file, const float **final_norm, size_t *final_norm_len,
                              KronosCudaMatrixDesc *lm_head, const uint16_t **embed_bf16, size_t *embed_bf16_len,
                              const float **embed_f32, size_t *embed_f32_len);
/* The untied embedding table quantized to NF4 (embed_nf4, real_llm.rs:1553; containers of version >= 4): 1 and the matrix
 * when the file holds one, 0 when it does not.  Hand it to kronos_cuda_engine_set_embedding_matrix (embed_bf16 = NULL at
 * engine creation): the engine then embeds a token as embed_token_into does (8084-8087), row decode + inverse rotation. */
int32_t kronos_cuda_k2tb_embed_nf4(const KronosCudaK2tb *file, KronosCudaMatrixDesc *table);
/* Writes a container the reference's load_bipolar reads: the version follows save_bipolar's rule (6 with q/k norms, 4 with
 * an NF4 embedding table, 3 with a qkv bias or a bf16 embedding table, 2 with NF matrices, else 1).  hidden / qkv_rows /
 * head_dim give the lengths of the per-layer vectors; embed_nf4 may be NULL. */
int32_t kronos_cuda_k2tb_save(const char *path, const uint64_t mode_words[6], const KronosCudaLayerDesc *layers, size_t n_layers,
                              size_t hidden, size_t qkv_rows, size_t head_dim, const float *final_norm,
                              const KronosCudaMatrixDesc *lm_head, const uint16_t *embed_bf16, size_t embed_bf16_len,
                              const KronosCudaMatrixDesc *embed_nf4);

/* ---- no-allocation variant ------------------------------------------------------------------- */

/* Widest matrix (columns) kronos_cuda_linear_noalloc accepts, and the bytes of device memory its
 * static scratch occupies on every GPU that loads the library, until the process exits. */
#define KRONOS_CUDA_NOALLOC_MAX_COLS 32768u
#define KRONOS_CUDA_NOALLOC_SCRATCH_BYTES (4u * 32768u + 2u * 4u * (32768u / 64u) * 4u)

/* Same result as kronos_cuda_linear, for callers that must not allocate on the decode path (a host
 * with a fixed device-memory plan, a real-time loop, a process under a memory cap): inputs and
 * outputs are DEVICE buffers (d_x[n_tok][cols] fp32, d_out[n_tok][rows] fp32), launches are queued on
 * the context's stream and the call returns without synchronizing.  It calls no cudaMalloc / cudaFree
 * and no allocating library routine: the quantized activations between its two kernels live in a
 * fixed __device__ array inside the library (KRONOS_CUDA_NOALLOC_SCRATCH_BYTES per GPU).
 *   - Matrices wider than KRONOS_CUDA_NOALLOC_MAX_COLS columns are rejected with an error.
 *   - All calls on a device share that array: calls that overlap on the GPU (other streams, other
 *     contexts) race; calls on one stream are safe. Nothing in it needs clearing between calls.
 *   - The first call on a device looks the array's device address up (cudaGetSymbolAddress); make
 *     that first call before starting any stream capture.
 * This entry point has no counterpart in the reference. */
int32_t kronos_cuda_linear_noalloc(KronosCudaContext *ctx, const KronosCudaMatrix *m, const float *d_x,
                                   size_t n_tok, float *d_out);

#ifdef __cplusplus
}
#endif
#endif

/*
 * k2t_oracle.h — CPU restatement of the kronos-2t quantized decode path.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the checker the CUDA backend is
 * compared against (and the timed CPU baseline of the benchmark).  Nothing in
 * the product path links, imports or calls it.
 *
 * Parity status: PARITY UNPINNED.  The reference is a Rust crate and no Rust
 * toolchain exists in the build environment, and the reference ships no golden
 * vectors for this path (its own tests compare two implementations with each
 * other).  The oracle is therefore pinned only by (a) the structural constants
 * the reference publishes (codebooks, E8Q2 templates, SplitMix64 constants,
 * record sizes, published model byte counts) and (b) the reference's own
 * cross-implementation equalities, all of which tests/ re-checks.
 *
 * Where the reference's aarch64 (NEON) and portable fallbacks differ, the
 * NEON arithmetic is followed: exact int32 dot per 64-column chunk, then
 * f = fmaf((float)dot * sx, w_scale, f) in ascending chunk order.
 *
 * Every function names the reference source it restates
 * (path within the reference project : line).
 */
#ifndef K2T_ORACLE_H
#define K2T_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- src/kernels/hadamard.rs ------------------------------------------- */
/* rademacher_sign_masks_64 (hadamard.rs:29-44): 0 or 0x80000000 per element. */
void k2o_rademacher_masks(uint64_t block_idx, uint32_t out[64]);
/* fwht64_signed_inplace_scalar (hadamard.rs:71-99). block0 = index of data[0]'s block. */
void k2o_fwht64(float *data, size_t n, uint64_t block0);
/* ifwht64_signed_inplace_scalar (hadamard.rs:200-228). */
void k2o_ifwht64(float *data, size_t n, uint64_t block0);

/* ---- src/kernels/simd_lut.rs:1375-1388 --------------------------------- */
uint16_t k2o_f32_to_bf16(float v);
float    k2o_bf16_to_f32(uint16_t b);

/* ---- Int8ChunkActivation (simd_lut.rs:2921-3256) ----------------------- */
/* populate_scalar (3235-3255): no rotation. */
void k2o_act_populate(const float *x, size_t cols, int8_t *q, float *scales, int32_t *sums);
/* populate_fwht / populate_rmsnorm_fwht via populate_chunk_fwht_scalar (3133-3196).
 * norm_w may be NULL (then inv_rms is ignored). chunk0 = global chunk index of x[0]. */
void k2o_act_populate_fwht(const float *x, size_t cols, const float *norm_w, float inv_rms,
                           uint64_t chunk0, int8_t *q, float *scales, int32_t *sums);

/* dot_f32_neon_16 (src/model/real_llm.rs:931-963): 16 fma lanes, NEON combine order. */
float k2o_dot_f32(const float *a, const float *b, size_t n);
/* rms_norm's inv_rms (real_llm.rs:9858-9860). */
float k2o_inv_rms(const float *x, size_t n, float eps);

/* ---- bipolar bit-plane matrices ---------------------------------------- */
size_t k2o_bipolar_data_bytes(size_t rows, size_t cols, size_t planes);
size_t k2o_bipolar_scale_count(size_t rows, size_t cols);
/* compile_hadamard_gptq_bipolar with hessian=None (src/model/compiler.rs:912-1107)
 * followed by FusedBipolarLutMatrix::pack_interleaved (simd_lut.rs:1772-1794). */
void k2o_bipolar_quantize_rtn(const float *weights, size_t rows, size_t cols, size_t planes,
                              size_t threads, uint8_t *interleaved, uint16_t *bf16_scales);
/* pack_interleaved alone, from row-major codes u[rows*cols]. */
void k2o_bipolar_pack(const uint8_t *u_grid, size_t rows, size_t cols, size_t planes, uint8_t *interleaved);
/* unpack_row_codes (1804-1820) / dequantize_row_rotated (1823-1835). */
void k2o_bipolar_unpack_row(const uint8_t *interleaved, size_t rows, size_t cols, size_t planes,
                            size_t r, uint8_t *codes);
void k2o_bipolar_dequant_row(const uint8_t *interleaved, const uint16_t *bf16_scales, size_t rows,
                             size_t cols, size_t planes, size_t r, float *out);

/* Nibble4SdotMatrix::from_bipolar_with_perm (simd_lut.rs:3297-3400). */
size_t k2o_nibble4_pair_bytes(size_t rows, size_t cols, size_t planes);
size_t k2o_nibble4_tail_bytes(size_t rows, size_t cols, size_t planes);
void k2o_nibble4_from_bipolar(const uint8_t *interleaved, const uint16_t *bf16_scales, size_t rows,
                              size_t cols, size_t planes, int interleave_gate_up,
                              uint8_t *pair_stream, uint8_t *tail_stream);
/* Nibble4SdotMatrix::dequantize_row_rotated (3441-3481). */
void k2o_nibble4_dequant_row(const uint8_t *pair_stream, const uint8_t *tail_stream, size_t rows,
                             size_t cols, size_t planes, size_t r, float *out);
/* sdot_one_stripe_neon (3763-3868) in scalar form over the Nibble4 records.
 * n_tok tokens share the weights (sdot_batch_tile_neon, 4228-4331: same per-(row,token) order).
 * xq[n_tok][cols], xs/xsum[n_tok][nc]; out[t*out_stride + r].
 * int_dots (optional) receives dot = 2a - max_odd*sum per [t][row][chunk]. threads>=1. */
void k2o_nibble4_gemv(const uint8_t *pair_stream, const uint8_t *tail_stream, size_t rows, size_t cols,
                      size_t planes, const int8_t *xq, const float *xs, const int32_t *xsum,
                      size_t n_tok, float *out, size_t out_stride, int32_t *int_dots, size_t threads);
/* Definition-level GEMV straight from the file format (codes via unpack_row_codes):
 * used to cross-check the Nibble4 path. Single token. */
void k2o_bipolar_gemv_def(const uint8_t *interleaved, const uint16_t *bf16_scales, size_t rows,
                          size_t cols, size_t planes, const int8_t *xq, const float *xs,
                          const int32_t *xsum, float *out, int32_t *int_dots);

/* ---- NF5/NF4/NF3/E8Q2 codebook matrices -------------------------------- */
extern const int8_t K2O_NF5_DEFAULT_POS[16];   /* simd_lut.rs:4338-4340 */
extern const int8_t K2O_NF4_DEFAULT[16];       /* 4343-4345 */
extern const int8_t K2O_NF3_DEFAULT[16];       /* 4348-4350 */
extern const int8_t K2O_E8Q2_EVEN_TEMPLATES[28][4]; /* 4354-4383 */
/* nf_expand_codebook32 (4636-4647). */
void k2o_nf_expand_codebook32(size_t bits, const int8_t codebook[16], int8_t out[32]);
/* e8q2_decode_8d (4436-4459). */
void k2o_e8q2_decode_8d(uint8_t tpl, uint8_t sgn, int8_t out[8]);
/* stripe_chunk_bytes / pair_total_bytes / tail_total_bytes (4818-4841). */
size_t k2o_nf_chunk_bytes(size_t bits);
size_t k2o_nf_pair_stream_bytes(size_t rows, size_t cols, size_t bits, size_t sgc);
size_t k2o_nf_tail_stream_bytes(size_t rows, size_t cols, size_t bits, size_t sgc);
size_t k2o_nf_scale_count(size_t rows, size_t cols, size_t sgc);
/* fit_empirical_nf_codebook (compiler.rs:1404-1528). returns mu_top. */
float k2o_nf_fit_codebook(const float *weights, size_t rows, size_t cols, size_t bits, size_t sgc,
                          int8_t codebook[16]);
/* compile_hadamard_gptq_nf with hessian=None, bits 3..5 (compiler.rs:1530-1860):
 * writes row-major indices and stripe-major bf16 scales [stripes][nsg][16]. */
/* NfSdotMatrix::from_bf16_u16_embeddings_nf4 (simd_lut.rs:5230-5495): bf16 table [rows][cols] -> NF4 streams (default codebook) */
void k2o_nf4_embed_from_bf16(const uint16_t *bf16, size_t rows, size_t cols, size_t sgc, size_t threads,
                             uint8_t *pair_stream, uint8_t *tail_stream);
void k2o_nf_quantize_rtn(const float *weights, size_t rows, size_t cols, size_t bits, size_t sgc,
                         size_t threads, int8_t codebook[16], uint8_t *flat_idx, uint16_t *bf16_scales);
/* NfSdotMatrix::from_indices (simd_lut.rs:4850-5023). */
void k2o_nf_pack(const uint8_t *flat_idx, const uint16_t *bf16_scales, size_t rows, size_t cols,
                 size_t bits, size_t sgc, uint8_t *pair_stream, uint8_t *tail_stream);
/* NfSdotMatrix::from_e8q2_codes (5118-5226): tpl/sgn are [rows][cols/8]. */
void k2o_e8q2_pack(const uint8_t *tpl, const uint8_t *sgn, const uint16_t *bf16_scales, size_t rows,
                   size_t cols, size_t sgc, uint8_t *pair_stream, uint8_t *tail_stream);
/* to_gate_up_interleaved (5500-5524). */
void k2o_nf_gate_up_interleave(const uint8_t *pair_stream, size_t rows, size_t cols, size_t bits,
                               size_t sgc, uint8_t *out_pair_stream);
/* dequantize_row_rotated (5560-5635). */
void k2o_nf_dequant_row(const uint8_t *pair_stream, const uint8_t *tail_stream, const int8_t codebook[16],
                        size_t rows, size_t cols, size_t bits, size_t sgc, size_t r, float *out);
/* nf_sdot_one_stripe_neon (6071-6181) / nf_sdot_batch_tile_neon (6689-7029) in scalar form,
 * index unpack as in the scalar pair-stream kernel (6459-6539). Same calling shape as k2o_nibble4_gemv. */
void k2o_nf_gemv(const uint8_t *pair_stream, const uint8_t *tail_stream, const int8_t codebook[16],
                 size_t rows, size_t cols, size_t bits, size_t sgc, const int8_t *xq, const float *xs,
                 size_t n_tok, float *out, size_t out_stride, int32_t *int_dots, size_t threads);

/* ---- dense Llama/Qwen decode step (k2t_model.cpp) ---------------------------------------------- */
/* A matrix in the reference's storage (same fields as the descriptors the device backend takes):
 * kind 0 = FusedBipolar (data0 interleaved planes, data1 bf16 scales), kind 2 = NF (pair/tail streams). */
typedef struct K2oMatrixDesc {
    uint32_t kind, rows, cols, bits, scale_group_chunks;
    int8_t codebook[16];
    const uint8_t *data0; size_t len0;
    const uint8_t *data1; size_t len1;
} K2oMatrixDesc;
/* LlamaConfig scalars the decode step needs (src/model/real_llm.rs:91-457). */
typedef struct K2oConfig {
    uint32_t hidden, layers, n_q, n_kv, head_dim, inter, vocab, max_seq;
    float eps;
    int32_t qk_norm_after_rope;
    uint32_t kv_bits;   /* 8 = int8 Hadamard cache, 4 = NF4 Hadamard cache (set_kv_bits, real_llm.rs:1731-1735) */
    /* Tensor-parallel rank view (no counterpart in the reference, which runs on one device): the model holds n_q / n_kv
     * LOCAL heads, inter LOCAL MLP columns and vocab LOCAL lm_head rows; the activations of the row-parallel projections
     * are rotated with their GLOBAL chunk index: o_proj input chunk c is global chunk o_chunk0 + c, down_proj input chunk c
     * is down_chunk0 + c.  All zero for the whole model. */
    uint32_t o_chunk0, down_chunk0;
} K2oConfig;
typedef struct K2oModel K2oModel;
K2oModel *k2o_model_new(const K2oConfig *cfg, const float *rope_table);
/* RealLlamaEngine::set_kv_bits / set_kv_sliding_window (real_llm.rs:1731-1790): rebuilds the cache in the given format and,
 * when 8 <= window and window + 512 < max_seq, as a ring of sinks + (window - sinks + 512) rows per (layer, kv head);
 * resets the position.  Returns 1 when a window is active, 0 when the full causal context is kept, -1 on error. */
int k2o_model_set_kv_window(K2oModel *m, uint32_t kv_bits, size_t window, size_t sinks);
/* KvPrefixSnapshot (save_kv_prefix / restore_kv_prefix_slice, real_llm.rs:5876-6155) as one blob: 32-byte header ("K2TKVPFX",
 * kv_bits, slots_per_head, heads, head_dim, 0, 0) + key rows, value rows, key scales, value scales, head-major.  save returns
 * the byte count (out == NULL: only the count); restore copies min(slots_per_head, copy_slots) rows and sets the position. */
size_t k2o_model_save_kv_prefix(const K2oModel *m, size_t n, uint8_t *out);
int k2o_model_restore_kv_prefix(K2oModel *m, const uint8_t *data, size_t len, size_t copy_slots, size_t total_pos);
/* causal_gqa_attention_q8 (real_llm.rs:8951-8988) over a stand-alone int8 Hadamard cache: k_q8 / v_q8 [n_kv][seq_len][head_dim],
 * scales [n_kv][seq_len], q [n_q][head_dim] (fp32, before rotation), out [n_q][head_dim]. */
void k2o_attention_q8(size_t head_dim, size_t n_q, size_t n_kv, size_t seq_len, const int8_t *k_q8, const float *k_scale,
                      const int8_t *v_q8, const float *v_scale, const float *q, float attn_scale, float *out);
/* cache rows per (layer, kv head) */
size_t k2o_model_kv_rows(const K2oModel *m);
/* can_truncate_kv_to (real_llm.rs:1806-1821): may the context be cut back to target_len without ring aliasing? */
int k2o_model_can_truncate_kv_to(const K2oModel *m, size_t target_len);
void k2o_model_free(K2oModel *m);
int k2o_model_set_layer(K2oModel *m, uint32_t l, const float *input_norm, const float *post_norm, const float *qkv_bias,
                        const float *q_norm, const float *k_norm, const K2oMatrixDesc *qkv, const K2oMatrixDesc *o,
                        const K2oMatrixDesc *gate_up, const K2oMatrixDesc *down);
/* Makes layer l a sparse-MoE layer (its dense gate_up / down are ignored): router [n_experts][hidden] fp32 (+ optional
 * bias), top_k with optional renormalisation (DenseMoeRouter::route_sorted, sparse_moe.rs:86-206; norm_topk bit 0 = renormalise,
 * bits 8.. = MoeRouterScoring tag: 0 softmax over all experts, 1 top-k softmax, 2 sigmoid), experts
 * as .k2tm records (nf_expert_byte_layout / pack_nf_expert_record, moe_800b.rs:1330-1407): record e of `shard` starts at
 * e * expert_bytes.  Forward = SparseMoeRuntime::forward_layer_single (sparse_moe.rs:961-1084) with the zero-copy NF
 * expert (MmapNfExpertView::forward_swiglu_zero_copy, moe_800b.rs:1440-1563). */
int k2o_model_set_moe(K2oModel *m, uint32_t l, const float *router_w, const float *router_bias, uint32_t n_experts,
                      uint32_t top_k, int norm_topk, uint32_t d_ff, uint32_t bits, uint32_t scale_group_chunks,
                      const uint8_t *shard, size_t expert_bytes);
/* Routes of the last token through MoE layer l: up to 32 (expert, weight) pairs sorted by expert id; returns k. */
/* Expert-parallel emulation (the reference runs on one device): from now on the MoE blocks of `m` add only the routed
 * experts e with e % ep_size == ep_rank, so k2o_model_ffn_part returns one rank's partial sum. */
/* shared expert of a sparse-MoE layer (SharedMoeExpert, Nf backend, sparse_moe.rs:223-315): gate_up [2 inter][hidden] (gate
 * rows first), down [hidden][inter], optional sigmoid gate weight [hidden] */
int k2o_model_set_moe_shared(K2oModel *m, uint32_t l, const K2oMatrixDesc *gate_up, const K2oMatrixDesc *down, const float *gate_w);
void k2o_model_set_ep(K2oModel *m, uint32_t ep_size, uint32_t ep_rank);
uint32_t k2o_model_last_routes(const K2oModel *m, uint32_t l, uint32_t *experts, float *weights);
/* .k2tm record geometry (NfExpertByteLayout): returns aligned_expert_bytes, fills the pair-stream offsets / sizes. */
size_t k2o_nf_expert_layout(size_t d_model, size_t d_ff, size_t bits, size_t sgc, size_t *gu_pair_off, size_t *gu_pair_bytes,
                            size_t *dn_pair_off, size_t *dn_pair_bytes);
int k2o_model_set_head(K2oModel *m, const float *final_norm, const K2oMatrixDesc *lm_head, const uint16_t *embed_bf16);
int k2o_model_set_embedding_matrix(K2oModel *m, const K2oMatrixDesc *table);   /* embed_nf4: NF rows instead of bf16 */
void k2o_model_reset(K2oModel *m);
size_t k2o_model_pos(const K2oModel *m);
void k2o_model_set_pos(K2oModel *m, size_t pos);
/* embed_token_into (real_llm.rs:8063-8097). */
void k2o_model_embed(const K2oModel *m, uint32_t token, float *out);
/* forward_token, generic path (6485-6790), int8 Hadamard KV; advances pos by one. */
/* The three pieces of a token's forward pass, for a tensor-parallel emulation that sums the ranks' partial outputs in
 * rank order between them (with one rank they compose to k2o_model_forward_embedding):
 *   attn_part: hidden[h] -> this rank's o_proj output (input norm, qkv, RoPE, KV store at the current position, attention
 *              over the local heads, o_proj over the local columns);
 *   ffn_part:  hidden[h] -> this rank's down_proj output (post-attention norm, local gate_up, SwiGLU, local down);
 *   head_part: hidden[h] -> logits of this rank's lm_head rows (final norm, lm_head);  advance: position += 1. */
int k2o_model_attn_part(K2oModel *m, uint32_t layer, const float *hidden, float *out, size_t threads);
int k2o_model_ffn_part(K2oModel *m, uint32_t layer, const float *hidden, float *out, size_t threads);
int k2o_model_head_part(K2oModel *m, const float *hidden, float *logits, size_t threads);
void k2o_model_advance(K2oModel *m);
int k2o_model_forward_embedding(K2oModel *m, const float *embedding, float *logits, size_t threads);
int k2o_model_forward_token(K2oModel *m, uint32_t token, float *logits, size_t threads);
/* hidden state after every layer of the last step, [layers][hidden]. */
const float *k2o_model_tap_hidden(const K2oModel *m);
/* Attention output (before o_proj) of the last layer for the last token: [n_q * head_dim]. */
const float *k2o_model_tap_attention(const K2oModel *m);
/* NF4 Hadamard cache (kv_bits = 4): packed indices [head_dim / 2] and bf16 scales [head_dim / 64] of one slot. */
int k2o_model_read_kv_q4(const K2oModel *m, uint32_t layer, uint32_t kv_head, size_t pos, uint8_t *k_q4, uint16_t *k_s16,
                         uint8_t *v_q4, uint16_t *v_s16);
/* store_hadamard_q4_head_raw (real_llm.rs:8646-8701) on one head: packed NF4 indices and one bf16 scale per 64 values. */
void k2o_kv_quant_head_q4(const float *src, size_t head_dim, uint8_t *q4, uint16_t *s16);
uint8_t k2o_nf4_nearest_idx(float y);
/* KV blob of positions [lo, hi) in the position-major export format (KvSlotPtrs::export, src/model/kv_blob.rs:63-81): per
 * position, per (layer, kv head): key row, key scale(s), value row, value scale(s).  Returns the byte count; with out ==
 * NULL only the count.  k2o_model_kv_import restores positions [0, n) and sets the position to n. */
size_t k2o_model_kv_export(const K2oModel *m, size_t lo, size_t hi, uint8_t *out);
int k2o_model_kv_import(K2oModel *m, const uint8_t *data, size_t len, size_t n);
/* One KV cache slot (layer, kv head, position): int8 rotated values [head_dim] and fp32 scales. */
int k2o_model_read_kv(const K2oModel *m, uint32_t layer, uint32_t kv_head, size_t pos, int8_t *k_q8, float *k_scale,
                      int8_t *v_q8, float *v_scale);
uint32_t k2o_argmax(const float *v, size_t n);                                   /* argmax_scalar 9914-9924 */
void k2o_build_rope_table(size_t max_seq, size_t head_dim, double theta, float *table);   /* 9212-9236 */
float k2o_exp_poly(float x);                                                     /* exp_f32_neon 9430-9454 */
void k2o_swiglu(const float *gate, const float *up, size_t n, float *out);       /* swiglu_activate_neon 9811-9842 */
void k2o_rope_heads(float *buf, size_t heads, size_t head_dim, const float *rope_row);    /* 9287-9326 */
void k2o_head_rms_norm(float *buf, size_t heads, size_t head_dim, const float *w, float eps); /* 8167-8178 */
void k2o_kv_quant_head(const float *src, size_t head_dim, int8_t *q, float *scale);       /* 8303-8365 */

#ifdef __cplusplus
}
#endif
#endif

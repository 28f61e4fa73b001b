// Launchers of the per-token kernels around the GEMVs (k2t_model_kernels.cu).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>

#include "k2t_layout.h"
#include "k2t_tp.h"

namespace k2t {

struct EmbedArgs {               // tied embedding = row of the lm_head matrix (device layout), or a bf16 table
    const uint8_t *plane[3];
    const uint16_t *scales;
    const uint16_t *embed_bf16;  // [vocab][hidden] or null
    const uint32_t *token;       // device, [n_tok]
    float *hidden;
    uint32_t fmt, nc, rows_pad, sgc, sgc_shift;
    uint32_t cell[3];
    int32_t max_odd;
    int8_t codebook[32];
};

// Sliding-window + attention-sink KV ring (QuantizedKvCache::new_with_opts, src/model/real_llm.rs:1235-1257): all zero =
// full causal context, cache row = position.  Otherwise a token attends to positions [0, sinks) and the last
// window - sinks ones, and position p >= sinks lives in row sinks + (p - sinks) % ring_len.
struct KvRing {
    uint32_t window, sinks, ring_len;
#ifdef __CUDACC__
    __host__ __device__
#endif
    uint32_t slot_of_pos(uint32_t p) const { return (ring_len == 0 || p < sinks) ? p : sinks + (p - sinks) % ring_len; }      // slot_of_pos, 1116-1122
#ifdef __CUDACC__
    __host__ __device__
#endif
    uint32_t active_len(uint32_t seq_len) const { return (window > 0 && seq_len > window) ? window : seq_len; }              // active_kv_len, 8597-8603
#ifdef __CUDACC__
    __host__ __device__
#endif
    uint32_t active_pos(uint32_t idx, uint32_t seq_len) const {                                                              // active_kv_pos, 8605-8612
        return (window > 0 && seq_len > window && idx >= sinks) ? (seq_len - (window - sinks)) + (idx - sinks) : idx;
    }
};

struct QkvPostArgs {
    const float *qkv;            // [n_q + 2 n_kv][head_dim]
    const float *bias, *q_norm, *k_norm;     // null when absent
    const float *rope;           // [max_seq][head_dim]: cos(hd/2), sin(hd/2)
    const uint32_t *pos;         // device
    uint32_t pos_offset;         // token of the batch: position = *pos + pos_offset
    int8_t *q_i8; float *q_scale;            // rotated int8 queries, one scale per head
    int8_t *k_q8, *v_q8; float *k_scale, *v_scale;   // cache: [layer][kv head][max_seq][head_dim] / [..][max_seq]
    uint32_t n_q, n_kv, head_dim, max_seq, layer;
    uint32_t kv_bits;            // 8: int8 rows + fp32 scale; 4: packed NF4 rows + bf16 scale per 64 values
    float eps;
    int32_t qk_norm_after_rope;
    KvRing ring;                 // where the position's cache row lives
    int8_t *v_t;                 // optional second copy of the int8 value rows, transposed in 16-position blocks (see ExactAttnArgs)
};

// Contexts up to this many positions are attended by the single fused kernel; longer ones by the three-kernel path in
// the same (CPU) summation order, or - on request - by the split-KV kernels (fp32-rounding agreement).
#define ATTN_EXACT_CTX 512u

struct AttnArgs {
    const int8_t *q_i8; const float *q_scale;
    const int8_t *k_q8, *v_q8; const float *k_scale, *v_scale;
    const uint32_t *pos;         // device: position of the current token (context = pos + 1)
    uint32_t pos_offset;         // token of the batch: position = *pos + pos_offset
    float *part_m, *part_l, *part_o;         // [n_q][n_split], [n_q][n_split], [n_q][n_split][head_dim]
    float *attn_out;             // optional fp32 attention output [n_q][head_dim] (tests), may be null
    int8_t *out_q; float *out_scales; int32_t *out_sums;   // activation of o_proj
    uint32_t out_chunk0;         // global index of the first o_proj input chunk of this rank (tensor parallel), else 0
    uint32_t n_kv, group, head_dim, max_seq, layer, n_split;
    uint32_t kv_bits;            // 8 or 4 (see QkvPostArgs)
    float attn_scale;
    uint32_t *err_flag;          // set to 1 when a bounded wait for a staged tile gives up
};

struct ExactAttnArgs {           // attention in the reference's summation order at any context length (k2t_attn_exact.cu)
    const int8_t *q_i8; const float *q_scale;              // rotated int8 queries of qkv_post_kernel
    const int8_t *k_q8, *v_q8; const float *k_scale, *v_scale;
    const uint32_t *pos;         // device: position of the current token (context = pos + 1)
    uint32_t pos_offset;
    float *sc;                   // scratch: scores [n_q][sc_stride]
    float *bmax;                 // scratch: maximum of every 128-position block [n_q][blk_stride]
    float *attn_out;             // optional fp32 attention output [n_q][head_dim], may be null
    int8_t *out_q; float *out_scales; int32_t *out_sums;   // activation of o_proj
    uint32_t out_chunk0;
    uint32_t n_kv, group, head_dim, max_seq, layer;
    uint32_t sc_stride, blk_stride;
    uint32_t ctx_cap;            // longest context the launch is sized for (a multiple of 4, at most sc_stride)
    uint32_t n_tok;              // tokens of the launch (set by the launcher)
    uint32_t kv_bits;
    float attn_scale;
    uint32_t *err_flag;
    unsigned long long *trace;   // optional diagnostic: SM clock readings of query head 0 at the phase boundaries (8 words)
    KvRing ring;                 // sliding window: active positions and their cache rows; scores then follow causal_gqa_group_q4_or_window for both cache formats
    // int8 cache without a window: a second copy of the value rows laid out for the chains, per (layer, kv head)
    // [position / 16][dimension][16 positions], bytes stored with the sign bit flipped (b ^ 0x80).  A 256-position tile is
    // one contiguous run, and dimension d's chain reads sixteen positions per 16-byte load straight from the landed tile -
    // no transposing pass through shared memory.  Null: the kernel transposes the row-major rows itself.
    const int8_t *v_t;
};

struct FusedAttnArgs {           // one layer's attention from the fused qkv vector to the o_proj activation
    const float *qkv;            // [n_q + 2 n_kv][head_dim]
    const float *bias, *q_norm, *k_norm;     // null when absent
    const float *rope;           // [max_seq][head_dim]
    const uint32_t *pos;         // device (stand-alone kernel; the whole-token kernel passes the position itself)
    uint32_t pos_offset;         // token of the batch: position = *pos + pos_offset
    int8_t *k_q8, *v_q8; float *k_scale, *v_scale;
    float *attn_tap;             // optional fp32 attention output [n_q][head_dim]
    int8_t *out_q; float *out_scales; int32_t *out_sums;
    uint32_t out_chunk0;         // global index of the first o_proj input chunk of this rank (tensor parallel), else 0
    uint32_t *err_flag;          // set when the bounded wait for the value rows gives up
    uint32_t n_q, n_kv, head_dim, max_seq, layer;
    uint32_t kv_bits;            // 8: int8 rows [head_dim] + fp32 scale per slot; 4: NF4 rows [head_dim / 2] + bf16 scale per 64 values
    float eps, attn_scale;
    int32_t qk_norm_after_rope;
    unsigned long long *trace;   // optional diagnostic: SM clock readings of query head 0 at the phase boundaries (16 words)
    uint32_t early;              // 1: the launch before this one wrote nothing this kernel prefetches (position word, cache rows of
                                 // earlier positions), so those loads are issued before the dependency wait
    int8_t *v_t;                 // optional block-transposed copy of the value rows (ExactAttnArgs.v_t): the new row is stored there too
};

struct RouterArgs {              // DenseMoeRouter::route_sorted, softmax scoring (sparse_moe.rs:86-182)
    const float *w, *bias;       // [n_experts][hidden], [n_experts] or null
    const float *x;              // normalised hidden state (fp32, not rotated)
    uint32_t n_experts, hidden, top_k;
    int32_t norm_topk;
    uint32_t scoring;            // MoeRouterScoring tag: 0 softmax over all experts, 1 top-k softmax, 2 sigmoid
    uint32_t *route_ids;         // out: [top_k] expert ids, ascending
    float *route_w;              // out: [top_k]
    float *logits;               // scratch: [n_experts] router logits (device)
    uint32_t *done;              // scratch: CTAs that have written their logits (zero between launches)
    // batches (grid.y = token t): x + t * hidden, route_ids / route_w + t * route_stride, logits + t * n_experts, done + t
    uint32_t route_stride;
    uint32_t staged;             // set by the launcher: the CTA's router rows are bulk-copied to shared memory before the dependency wait
    uint32_t *err_flag;          // device error word (1 = a bounded wait for a bulk copy gave up); may be null
};

// pdl: launch as a programmatic dependent of the previous kernel in the stream (see pdl_wait in k2t_device.cuh).
// n_tok: tokens of the batch (per-token vectors are contiguous: [n_tok][n])
cudaError_t launch_embed(cudaStream_t s, const EmbedArgs &a, uint32_t n_tok, bool pdl);
cudaError_t launch_rmsnorm_quant(cudaStream_t s, float *hidden, const float *delta, const float *w, uint32_t n, float eps,
                                 int8_t *q, float *scales, int32_t *sums, uint32_t n_tok, bool pdl);
// n_tok consecutive tokens (positions *pos + pos_offset + t): qkv [n_tok][n_q + 2 n_kv][head_dim], q_i8 [n_tok][n_q][head_dim], q_scale [n_tok][n_q]
cudaError_t launch_qkv_post(cudaStream_t s, const QkvPostArgs &a, bool pdl, uint32_t n_tok = 1);
cudaError_t launch_attention(cudaStream_t s, const AttnArgs &a, bool pdl);     // two kernels
// any context length in the reference's summation order: two kernels (after launch_qkv_post).  n_tok consecutive tokens of a
// batch are attended side by side (token t sees the positions up to its own): per-token query slots as above, scores
// [n_tok][n_q][sc_stride], block maxima [n_tok][n_q][blk_stride], o_proj activation rows [n_tok][n_q * head_dim] (scales and
// sums [n_tok][n_q * head_dim / 64]); attn_out (optional) receives the last token's output.
cudaError_t launch_attention_exact(cudaStream_t s, const ExactAttnArgs &a, bool pdl, uint32_t n_tok = 1);
// longest context launch_attention_exact can serve (its value weights live in shared memory)
size_t attention_exact_max_ctx(uint32_t head_dim, uint32_t kv_bits);
// contexts of up to ATTN_EXACT_CTX positions: qkv_post + attention in one kernel (leaves longer contexts untouched)
cudaError_t launch_attention_fused(cudaStream_t s, const FusedAttnArgs &a, bool pdl);
// chunk0: global index of the first down_proj input chunk of this rank (tensor parallel), else 0
cudaError_t launch_swiglu_quant(cudaStream_t s, const float *gate_up, uint32_t inter, int8_t *q, float *scales, int32_t *sums,
                                float *dbg, uint32_t chunk0, uint32_t n_tok, bool pdl);
// scratch: ARGMAX_SCRATCH_WORDS zeroed 32-bit words of device memory (per-CTA candidates and the arrival counter)
constexpr uint32_t ARGMAX_SCRATCH_WORDS = 2 * 256 + 4;
cudaError_t launch_argmax_step(cudaStream_t s, const float *logits, uint32_t n, uint32_t *token, uint32_t *pos,
                               uint32_t *history, uint32_t *step, float *scratch, bool pdl);
// x_norm (optional): also write the normalised fp32 vector (the MoE router reads it)
cudaError_t launch_rmsnorm_quant_x(cudaStream_t s, float *hidden, const float *delta, const float *w, uint32_t n, float eps,
                                   int8_t *q, float *scales, int32_t *sums, float *x_norm, uint32_t n_tok, bool pdl);
// the same with the tensor-parallel exchange of `delta` (each rank's partial projection output) folded in: tp.tp > 1,
// tp_done = a zeroed device word; n_tok * n floats must fit a slot of the exchange buffer
cudaError_t launch_rmsnorm_quant_tp(cudaStream_t s, float *hidden, const float *delta, const float *w, uint32_t n, float eps,
                                    int8_t *q, float *scales, int32_t *sums, float *x_norm, uint32_t n_tok, bool pdl,
                                    const TpLink &tp, uint32_t *tp_done);
cudaError_t launch_moe_router(cudaStream_t s, const RouterArgs &a, bool pdl, uint32_t n_tok = 1);
// SwiGLU of n_slot expert outputs [n_slot][2 * d_ff] with the scalar-path exp (moe_800b.rs:1498-1517), then rotation + int8
cudaError_t launch_expert_swiglu_quant(cudaStream_t s, const float *gate_up, uint32_t d_ff, uint32_t n_slot, int8_t *q, float *scales,
                                       int32_t *sums, bool pdl);
// out[i] = sum over slots, in slot order, of route_w[s] * expert_out[s][i]   (sparse_moe.rs:1046-1048)
cudaError_t launch_moe_combine(cudaStream_t s, const float *expert_out, const float *route_w, uint32_t n_slot, uint32_t n, float *out,
                               bool pdl, const uint32_t *route_ids = nullptr, const uint8_t *const *owned = nullptr, uint32_t n_experts = 0,
                               uint32_t n_tok = 1, uint32_t route_stride = 0, const float *base = nullptr, const float *base_scale = nullptr);
// sigmoid gate of a shared expert, one value per token of the batch
cudaError_t launch_shared_gate(cudaStream_t s, const float *gate_w, const float *x_norm, uint32_t n, uint32_t n_tok, float *scale, bool pdl);
cudaError_t launch_advance_pos(cudaStream_t s, uint32_t *pos, uint32_t by, bool pdl);
// rebuilds the block-transposed value copy from the row-major int8 value rows (after rows were imported from the host)
cudaError_t launch_vt_rebuild(cudaStream_t s, const int8_t *v_q8, int8_t *v_t, size_t heads, uint32_t rows_per_head, uint32_t head_dim);
// one thread that waits about `ns` nanoseconds (bounded): lets a host queue work behind it (measurement only)
cudaError_t launch_delay(cudaStream_t s, uint64_t ns);

}  // namespace k2t

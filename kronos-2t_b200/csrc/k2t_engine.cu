// Whole-token engine behind the C ABI: counterpart of MetalLlamaEngine (src/backend/metal_gpu.rs:929-969,
// try_new 1196, forward_tokens 1619) for dense Llama/Qwen layers with bit-plane or NF projections and the
// int8 Hadamard KV cache.  One decode step = 10 kernels per layer + 3; the greedy loop and the token-id
// forward replay a captured CUDA graph (position, token and step counter live in device memory).
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <map>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "k2t_context.h"
#include "k2t_decode_mega.h"
#include "k2t_gemv_fused.h"
#include "k2t_model_kernels.h"
#include "k2t_prologue.cuh"
#include "k2t_tp.h"

using namespace k2t;

struct EngineLayer {
    float *input_norm = nullptr, *post_norm = nullptr, *qkv_bias = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    KronosCudaMatrix *qkv = nullptr, *o = nullptr, *gate_up = nullptr, *down = nullptr;
    // sparse-MoE FFN (router + expert records) instead of gate_up / down
    bool moe = false;
    float *router_w = nullptr, *router_bias = nullptr;
    k2t::DeviceMatrix gu_dm{}, dn_dm{};                                // geometry (and image base) of the first expert this rank holds: template of the expert launches
    uint8_t *d_experts = nullptr;                                     // ONE allocation: the device images of all experts of the layer this rank holds
    const uint8_t **d_gu_bases = nullptr, **d_dn_bases = nullptr;     // device tables: image base of every expert
    k2t::ExpertCodebook *d_gu_books = nullptr, *d_dn_books = nullptr; // device tables: decode tables of every expert
    int gu_fmt = -1, dn_fmt = -1;                                     // kernel format of the layer's experts
    uint32_t expert0 = 0;                                             // first expert held by this rank (expert parallelism)
    uint32_t *d_route_ids = nullptr;                                  // [max_batch][32] routes of the last batch
    float *d_route_w = nullptr;
    // shared expert of a MoE layer (SharedMoeExpert, sparse_moe.rs:223-315): its matrices live in gate_up / down above
    uint32_t sh_inter = 0;
    float *sh_gate_w = nullptr;
};

struct KronosCudaEngine {
    KronosCudaContext *ctx = nullptr;
    KronosCudaEngineConfig cfg{};
    std::vector<EngineLayer> layers;
    KronosCudaMatrix *lm_head = nullptr;
    float *final_norm = nullptr, *rope = nullptr;
    uint16_t *embed_bf16 = nullptr;
    // workspace
    float *hidden = nullptr, *proj = nullptr, *qkv = nullptr, *gate_up = nullptr, *logits = nullptr;
    int8_t *act_q = nullptr, *q_i8 = nullptr;
    float *attn_tap = nullptr;                // attention output of the last layer (diagnostic)
    float *act_s = nullptr, *q_scale = nullptr, *part_m = nullptr, *part_l = nullptr, *part_o = nullptr;
    float *attn_sc = nullptr, *attn_bmax = nullptr;      // long contexts in CPU order: scores [n_q][kv_stride], block maxima [n_q][kv_stride / 128]
    bool split_kv = false;                    // long contexts by the split-KV kernels instead (config flag, or the cache is too long for the exact path)
    int32_t *act_m = nullptr;
    int8_t *k_q8 = nullptr, *v_q8 = nullptr;
    int8_t *v_t = nullptr;      // int8 cache without a window: the value rows once more, transposed in 16-position blocks for the value chains
    float *k_scale = nullptr, *v_scale = nullptr;
    uint32_t *d_token = nullptr, *d_pos = nullptr, *d_step = nullptr, *d_history = nullptr;
    uint32_t n_split = 32;
    uint32_t max_batch = 256;                 // tokens per prompt batch: their projections run on the tensor cores in one weight pass (k2t_gemm_tc.cu), their attention side by side; every per-token buffer holds this many rows (KRONOS_CUDA_PROMPT_BATCH, 16..512)
    uint32_t ctx_bound = 0;                   // prompt batches (launched eagerly, position known on the host): no token of the batch sees more positions; 0 = size launches for the whole cache
    uint32_t kv_stride = 0;                   // cache rows per (layer, kv head): the rows the geometry needs (max_seq_len, or sinks + ring) rounded up to 32, so every 32-row tile of rows and scales starts on 16 bytes
    k2t::KvRing ring{};                       // sliding-window + sink ring (all zero: row = position)
    uint32_t kv_rows = 0;                     // rows in use per (layer, kv head)
    // sparse-MoE workspace: normalised hidden state, per-route expert buffers
    float *x_norm = nullptr, *moe_gu = nullptr, *moe_out = nullptr, *router_logits = nullptr;
    uint32_t *router_done = nullptr;
    int8_t *moe_q = nullptr; float *moe_s = nullptr; int32_t *moe_m = nullptr;
    // shared-expert workspace, [max_batch] rows each: gate_up outputs, the down projection's activation, outputs, gate values
    uint32_t sh_inter_max = 0;
    float *sh_gu = nullptr, *sh_out = nullptr, *sh_scale = nullptr;
    int8_t *sh_q = nullptr; float *sh_s = nullptr; int32_t *sh_m = nullptr;
    bool has_moe = false;
    // tensor parallel: exchange buffer (data[2][tp][slot] floats + flags[tp]) and the peers' mappings
    k2t::TpLink tp{};
    float *tp_buf = nullptr;
    uint32_t *tp_done = nullptr;              // CTAs of the current fused exchange that have finished (device word)
    std::vector<void *> tp_peers;            // mappings opened with cudaIpcOpenMemHandle
    bool tp_ready = false;
    float *logits_local = nullptr;            // this rank's logits slice [max_batch][vocab_size]
    KronosCudaMatrix *embed_matrix = nullptr; // whole lm_head for the token lookup (tied embeddings under tp)
    uint32_t last_row = 0;                    // row of `hidden` that holds the last forwarded token (prompt batches)
    bool pdl = true;                          // kernels of a step overlap their prologues with the predecessor's tail
    bool fused = false;                       // single-token steps: norm / SwiGLU / embedding run as prologues of the GEMV that consumes them (KRONOS_CUDA_FUSED=1)
    const float *final_hidden = nullptr;      // where the last step left the residual stream of its last token
    size_t weight_bytes = 0;
    std::vector<void *> allocs;
    // whole-token decode kernel (contexts up to ATTN_EXACT_CTX positions)
    bool mega_ok = false;
    std::string mega_why;                     // why the kernel is not used, when it is not
    float *hidden2 = nullptr;
    k2t::MegaLayer *d_mega_layers = nullptr;
    k2t::MegaMatrix *d_mega_head = nullptr;
    uint32_t *d_barrier = nullptr;
    unsigned long long *d_trace = nullptr;    // phase trace of the last step of the last decode-kernel call
    uint32_t mega_warp_smem = 0, mega_kmax = 0;
    size_t mega_smem = 0;
    cudaGraphExec_t graphs[4] = {nullptr, nullptr, nullptr, nullptr};      // [greedy ? 0 : 1][long context ? 1 : 0] -> 2 * ids + long
    cudaStream_t graph_stream = nullptr;      // the stream the graphs were captured on
    // per-kernel-class timing of one step (kronos_cuda_engine_profile_step): while prof_on, every launch is followed
    // by an event record, so a captured step carries one event node per kernel
    bool prof_on = false;
    std::vector<std::pair<const char *, cudaEvent_t>> prof_marks;
#ifdef K2T_TIMELINE
    std::vector<const char *> tl_labels[4];     // launch labels of the four captured step graphs, in launch order
    std::vector<const char *> *tl_cur = nullptr;
#endif
    unsigned long long *d_dbg = nullptr;      // 32 diagnostic words (phase clocks of the attention kernel, layer 0)
    float *argmax_scratch = nullptr;          // candidates and arrival counter of the argmax kernel
    bool attn_trace = false;
};

namespace {

template <typename T>
bool dev_alloc(KronosCudaEngine *e, T *&p, size_t count, const T *host = nullptr) {
    void *raw = nullptr;
    const size_t bytes = std::max<size_t>(count, 1) * sizeof(T);
    if (!cuda_ok(e->ctx, cudaMalloc(&raw, bytes), "cudaMalloc(engine)")) return false;
    e->allocs.push_back(raw);
    p = static_cast<T *>(raw);
    if (host) return cuda_ok(e->ctx, cudaMemcpyAsync(p, host, count * sizeof(T), cudaMemcpyHostToDevice, e->ctx->stream), "upload");
    return cuda_ok(e->ctx, cudaMemsetAsync(p, 0, bytes, e->ctx->stream), "clear");
}


void dev_free(KronosCudaEngine *e, void *p) {
    if (!p) return;
    for (size_t i = 0; i < e->allocs.size(); ++i)
        if (e->allocs[i] == p) { e->allocs.erase(e->allocs.begin() + i); break; }
    cudaFree(p);
}

// (Re)builds the KV cache: format `bits` (8 / 4) and geometry - the full causal context, or the sliding-window ring of
// QuantizedKvCache::new_with_opts (real_llm.rs:1235-1257): taken only when 8 <= window and window + 512 < max_seq_len, sinks
// capped at window / 2, ring = window - sinks + 512 rows of slack for batches.  Also the scratch sized by the cache rows.
bool alloc_kv(KronosCudaEngine *e, uint32_t bits, uint32_t window, uint32_t sinks) {
    KronosCudaContext *ctx = e->ctx;
    KronosCudaEngineConfig &c = e->cfg;
    if (bits != 8 && bits != 4) return fail(ctx, "kv_bits must be 8 (int8 Hadamard cache) or 4 (NF4 Hadamard cache)");
    for (void *p : {(void *)e->k_q8, (void *)e->v_q8, (void *)e->v_t, (void *)e->k_scale, (void *)e->v_scale, (void *)e->attn_sc, (void *)e->attn_bmax}) dev_free(e, p);
    e->k_q8 = e->v_q8 = e->v_t = nullptr; e->k_scale = e->v_scale = e->attn_sc = e->attn_bmax = nullptr;
    c.kv_bits = bits;
    if (window >= 8 && (uint64_t)window + 512u < c.max_seq_len) {
        e->ring.window = window;
        e->ring.sinks = std::min(sinks, window / 2);
        e->ring.ring_len = (window - e->ring.sinks) + 512u;
        e->kv_rows = e->ring.sinks + e->ring.ring_len;
    } else {
        e->ring = KvRing{};
        e->kv_rows = c.max_seq_len;
    }
    c.kv_window = e->ring.window; c.kv_sinks = e->ring.sinks;
    e->kv_stride = (e->kv_rows + 31u) & ~31u;
    const uint32_t hd = c.head_dim, n_q = c.num_attention_heads;
    // contexts beyond 512 positions: in the CPU's order unless the split-KV kernels were asked for (they know no window) or
    // the value weights of the longest context would not fit the values kernel's shared memory
    const uint32_t longest = e->ring.window ? e->ring.window : e->kv_stride;
    e->split_kv = e->ring.window == 0 && ((c.flags & KRONOS_CUDA_ENGINE_SPLIT_KV_ATTENTION) != 0 || longest > attention_exact_max_ctx(hd, bits));
    if (e->ring.window && longest > attention_exact_max_ctx(hd, bits)) return fail(ctx, "kv_window is longer than the attention kernel can hold");
    const size_t slots = (size_t)c.num_layers * c.num_key_value_heads * e->kv_stride;
    const bool ok = dev_alloc(e, e->attn_sc, (size_t)e->max_batch * n_q * e->kv_stride) && dev_alloc(e, e->attn_bmax, (size_t)e->max_batch * n_q * ((e->kv_stride + 127) / 128)) &&
                    dev_alloc(e, e->k_q8, bits == 4 ? slots * hd / 2 : slots * hd) && dev_alloc(e, e->v_q8, bits == 4 ? slots * hd / 2 : slots * hd) &&
                    dev_alloc(e, e->k_scale, bits == 4 ? (slots * (hd / 64) + 1) / 2 : slots) &&      // NF4: bf16 per 64 values
                    dev_alloc(e, e->v_scale, bits == 4 ? (slots * (hd / 64) + 1) / 2 : slots);
    // unwritten NF4 rows hold index 8 in both nibbles, as in the reference's fresh cache (vec![0x88; ..], real_llm.rs:1278-1279)
    const bool filled = !ok || bits != 4 ||
                        (cuda_ok(ctx, cudaMemsetAsync(e->k_q8, 0x88, slots * hd / 2, ctx->stream), "fill cache") &&
                         cuda_ok(ctx, cudaMemsetAsync(e->v_q8, 0x88, slots * hd / 2, ctx->stream), "fill cache"));
    for (cudaGraphExec_t &g : e->graphs) if (g) { cudaGraphExecDestroy(g); g = nullptr; }      // captured cache pointers are stale
    // the transposed copy of the value rows (zero rows = 0x80 there); not for the NF4 cache, windows or the split-KV kernels
    bool vt_ok = true;
    if (ok && bits == 8 && e->ring.window == 0 && !e->split_kv)
        vt_ok = dev_alloc(e, e->v_t, slots * hd) && cuda_ok(ctx, cudaMemsetAsync(e->v_t, 0x80, slots * hd, ctx->stream), "fill cache");
    return ok && filled && vt_ok;
}

// after value rows came from the host (imported blobs, restored snapshots): bring the transposed copy up to date
bool sync_vt(KronosCudaEngine *e) {
    if (!e->v_t) return true;
    const KronosCudaEngineConfig &c = e->cfg;
    return cuda_ok(e->ctx, launch_vt_rebuild(e->ctx->stream, e->v_q8, e->v_t, (size_t)c.num_layers * c.num_key_value_heads, e->kv_stride, c.head_dim), "rebuild value copy");
}

// y[t] = W x[t] for the n_tok tokens of the batch (activations [n_tok][cols] in act_*; one weight pass for up to 4 tokens)
bool count(KronosCudaEngine *e, cudaError_t err, const char *what, uint32_t n = 1);


bool gemv_from(KronosCudaEngine *e, const KronosCudaMatrix *m, const int8_t *q, const float *sc, const int32_t *sums, float *out, const char *what,
               uint32_t n_tok) {
    uint32_t launched = 0;
    cudaError_t err = launch_gemv_batch(e->ctx->stream, m->dm, q, sc, sums, n_tok, out, m->dm.geom.rows, nullptr, e->ctx->sm_count, e->ctx->d_err, &launched, e->pdl);
    return count(e, err, what, launched);
}
bool gemv(KronosCudaEngine *e, const KronosCudaMatrix *m, float *out, const char *what, uint32_t n_tok = 1, size_t act_tok0 = 0) {
    const size_t cols = m->dm.geom.cols, nc = cols / 64;
    return gemv_from(e, m, e->act_q + act_tok0 * cols, e->act_s + act_tok0 * nc, e->act_m + act_tok0 * nc, out, what, n_tok);
}

bool count(KronosCudaEngine *e, cudaError_t err, const char *what, uint32_t n) {
    e->ctx->launches += n;
#ifdef K2T_TIMELINE
    if (e->tl_cur) for (uint32_t i = 0; i < n; ++i) e->tl_cur->push_back(what);
#endif
    if (e->prof_on && err == cudaSuccess) {
        cudaEvent_t ev = nullptr;
        if (!cuda_ok(e->ctx, cudaEventCreate(&ev), "profile event") || !cuda_ok(e->ctx, cudaEventRecord(ev, e->ctx->stream), "profile event"))
            return false;
        e->prof_marks.emplace_back(what, ev);
    }
    return cuda_ok(e->ctx, err, what);
}

void fill_embed_args(const KronosCudaEngine *e, EmbedArgs &a);

// tensor parallel: x <- sum over ranks of x (rank order), and the concatenation of the ranks' slices; no-ops on one device
bool tp_gather(KronosCudaEngine *e, const float *slice, float *all, uint32_t n) {
    if (!e->tp_ready) return fail(e->ctx, "tensor-parallel engine used before kronos_cuda_engine_tp_attach");
    return count(e, launch_tp_exchange(e->ctx->stream, e->tp, slice, all, n, n, e->pdl), "tp gather");
}


// Residual add + RMSNorm + activation of the next projection.  Under tensor parallelism `delta` is this rank's partial
// output of a row-parallel projection: the kernel exchanges and sums the ranks' partials itself.
// `partial`: delta holds this rank's share only (row-parallel projection under tensor parallelism, routed experts under
// Context the attention launches beyond 512 positions are sized for (grid of the scores kernel, shared memory of the values
// kernel): the cache's capacity (a captured decode step is replayed at any position), or, for a prompt batch whose last
// position the host knows, that position rounded up - two values CTAs fit an SM then, and no scores CTA starts for nothing.
uint32_t attn_ctx_cap(const KronosCudaEngine *e) {
    const uint32_t full = e->ring.window ? (e->ring.window + 3u) & ~3u : e->kv_stride;
    if (e->ctx_bound == 0) return full;
    return std::min(full, (e->ctx_bound + 127u) & ~127u);
}

// expert parallelism).
bool norm_quant(KronosCudaEngine *e, const float *delta, const float *w, float *x_norm, uint32_t T, bool pdl, bool partial) {
    const KronosCudaEngineConfig &c = e->cfg;
    if (partial && delta != nullptr) {
        if (!e->tp_ready) return fail(e->ctx, "tensor-parallel engine used before kronos_cuda_engine_tp_attach");
        return count(e, launch_rmsnorm_quant_tp(e->ctx->stream, e->hidden, delta, w, c.hidden_size, c.rms_norm_eps, e->act_q, e->act_s, e->act_m, x_norm, T, pdl,
                                                e->tp, e->tp_done), "rmsnorm");
    }
    return count(e, launch_rmsnorm_quant_x(e->ctx->stream, e->hidden, delta, w, c.hidden_size, c.rms_norm_eps, e->act_q, e->act_s, e->act_m, x_norm, T, pdl), "rmsnorm");
}

enum class Tail { Greedy, LastLogits, AllLogits, None };

bool enqueue_attention(KronosCudaEngine *e, uint32_t l, uint32_t t, uint32_t T, bool long_ctx);
bool enqueue_attention_batch(KronosCudaEngine *e, uint32_t l, uint32_t T);

// One token with the small operators folded into the GEMVs (k2t_gemv_fused.cu): per dense layer
//   [residual + norm -> qkv]  [attention]  [o]  [residual + norm -> gate_up]  [SwiGLU -> down]
// five kernels instead of eight; per sparse-MoE layer norm, router, expert gate_up, [SwiGLU -> expert down], the weighted
// sum of the experts riding in the next residual prologue.  The residual stream alternates between two buffers (every
// CTA of a fused GEMV reads the old one while CTA 0 writes the new one).
bool enqueue_fused_step(KronosCudaEngine *e, bool embed, Tail tail, bool long_ctx) {
    const KronosCudaEngineConfig &c = e->cfg;
    cudaStream_t s = e->ctx->stream;
    const uint32_t h = c.hidden_size, inter = c.intermediate_size;
    float *cur = e->hidden, *other = e->hidden2;
    const float *pend = nullptr;              // projection output not yet added to the residual stream
    const EngineLayer *pend_moe = nullptr;    // ... or the routed experts' outputs of that layer
    auto residual_norm = [&](FusedPro &p, const float *w, bool first) {
        p = FusedPro{};
        p.n = h; p.chunk0 = 0; p.eps = c.rms_norm_eps; p.norm_w = w;
        if (first && embed) {
            p.mode = PRO_EMBED_NORM;
            fill_embed_args(e, p.embed);
            p.x_out = cur;
            return;
        }
        p.mode = PRO_NORM;
        p.x_in = cur;
        if (pend_moe != nullptr) {
            p.moe_out = e->moe_out; p.route_w = pend_moe->d_route_w; p.n_slot = std::min(c.moe_top_k, c.moe_num_experts);
        } else {
            p.delta = pend;
        }
        if (p.delta != nullptr || p.n_slot > 0) { p.x_out = other; std::swap(cur, other); }
        pend = nullptr; pend_moe = nullptr;
    };
    const bool pdl = e->pdl;
    for (uint32_t l = 0; l < c.num_layers; ++l) {
        const EngineLayer &L = e->layers[l];
        FusedPro p;
        residual_norm(p, L.input_norm, l == 0);
        if (!count(e, launch_gemv_fused(s, L.qkv->dm, p, e->qkv, e->ctx->sm_count, e->ctx->d_err, pdl && (l > 0)), "gemv qkv (+norm)")) return false;
        if (!enqueue_attention(e, l, 0, 1, long_ctx)) return false;
        if (!gemv(e, L.o, e->proj, "gemv o")) return false;
        pend = e->proj;
        if (L.moe) {
            // norm kernel (x_norm for the router + the experts' activation), router, expert gate_up, [SwiGLU -> expert down]
            if (!count(e, launch_rmsnorm_quant_x(s, cur, pend, L.post_norm, h, c.rms_norm_eps, e->act_q, e->act_s, e->act_m, e->x_norm, 1, pdl), "rmsnorm")) return false;
            pend = nullptr;        // added in place by the norm kernel
            const uint32_t k = std::min(c.moe_top_k, c.moe_num_experts), dff = c.moe_d_ff;
            RouterArgs ra{};
            ra.w = L.router_w; ra.bias = L.router_bias; ra.x = e->x_norm;
            ra.n_experts = c.moe_num_experts; ra.hidden = h; ra.top_k = k; ra.norm_topk = (int32_t)(c.moe_norm_topk & 1u); ra.scoring = c.moe_norm_topk >> 8;
            ra.route_ids = L.d_route_ids; ra.route_w = L.d_route_w; ra.logits = e->router_logits; ra.done = e->router_done; ra.err_flag = e->ctx->d_err;
            if (!count(e, launch_moe_router(s, ra, pdl), "router")) return false;
            if (!count(e, launch_gemv_experts(s, L.gu_dm, L.gu_fmt, L.d_gu_books, L.d_gu_bases, ra.route_ids, k, e->act_q, e->act_s, e->act_m, 0, 0,
                                              e->moe_gu, (size_t)2 * dff, e->ctx->sm_count, e->ctx->d_err, pdl, c.moe_num_experts), "expert gate_up")) return false;
            FusedPro ps{};
            ps.mode = PRO_SWIGLU; ps.n = dff; ps.chunk0 = 0; ps.swiglu_exp_cr = 1; ps.gate_up = e->moe_gu;
            if (!count(e, launch_gemv_fused_experts(s, L.dn_dm, L.dn_fmt, L.d_dn_books, L.d_dn_bases, ra.route_ids, k, c.moe_num_experts, ps,
                                                    (size_t)2 * dff, e->moe_out, h, e->ctx->sm_count, e->ctx->d_err, pdl), "expert down (+swiglu)")) return false;
            pend_moe = &L;
            continue;
        }
        residual_norm(p, L.post_norm, false);
        if (!count(e, launch_gemv_fused(s, L.gate_up->dm, p, e->gate_up, e->ctx->sm_count, e->ctx->d_err, pdl), "gemv gate_up (+norm)")) return false;
        FusedPro ps{};
        ps.mode = PRO_SWIGLU; ps.n = inter; ps.chunk0 = c.down_chunk0; ps.gate_up = e->gate_up;
        if (!count(e, launch_gemv_fused(s, L.down->dm, ps, e->proj, e->ctx->sm_count, e->ctx->d_err, pdl), "gemv down (+swiglu)")) return false;
        pend = e->proj;
    }
    FusedPro p;
    residual_norm(p, e->final_norm, false);
    e->final_hidden = cur;
    if (!count(e, launch_gemv_fused(s, e->lm_head->dm, p, e->logits, e->ctx->sm_count, e->ctx->d_err, pdl), "gemv lm_head (+norm)")) return false;
    if (tail == Tail::Greedy) return count(e, launch_argmax_step(s, e->logits, c.vocab_size, e->d_token, e->d_pos, e->d_history, e->d_step, e->argmax_scratch, pdl), "argmax");
    return count(e, launch_advance_pos(s, e->d_pos, 1, pdl), "advance");
}

// Attention of all T tokens of a batch for layer l in three launches: bias / norm / RoPE / cache rows / int8 queries of every
// token, then scores and values of the T tokens side by side (token t sees the positions up to its own, the rows of the
// tokens before it in the batch included: they are in the cache by then).  Same arithmetic as the single-token kernels.
bool enqueue_attention_batch(KronosCudaEngine *e, uint32_t l, uint32_t T) {
    const KronosCudaEngineConfig &c = e->cfg;
    cudaStream_t s = e->ctx->stream;
    const EngineLayer &L = e->layers[l];
    const uint32_t hd = c.head_dim;
    QkvPostArgs qa{};
    qa.qkv = e->qkv; qa.bias = L.qkv_bias; qa.q_norm = L.q_norm; qa.k_norm = L.k_norm; qa.rope = e->rope;
    qa.pos = e->d_pos; qa.pos_offset = 0;
    qa.q_i8 = e->q_i8; qa.q_scale = e->q_scale; qa.k_q8 = e->k_q8; qa.v_q8 = e->v_q8; qa.k_scale = e->k_scale; qa.v_scale = e->v_scale;
    qa.n_q = c.num_attention_heads; qa.n_kv = c.num_key_value_heads; qa.head_dim = hd; qa.max_seq = e->kv_stride; qa.layer = l;
    qa.eps = c.rms_norm_eps; qa.qk_norm_after_rope = c.qk_norm_after_rope; qa.kv_bits = c.kv_bits; qa.ring = e->ring; qa.v_t = e->v_t;
    if (!count(e, launch_qkv_post(s, qa, e->pdl, T), "qkv_post")) return false;
    ExactAttnArgs xa{};
    xa.q_i8 = e->q_i8; xa.q_scale = e->q_scale; xa.k_q8 = e->k_q8; xa.v_q8 = e->v_q8; xa.k_scale = e->k_scale; xa.v_scale = e->v_scale;
    xa.pos = e->d_pos; xa.pos_offset = 0;
    xa.sc = e->attn_sc; xa.bmax = e->attn_bmax; xa.attn_out = l + 1 == c.num_layers ? e->attn_tap : nullptr;
    xa.out_q = e->act_q; xa.out_scales = e->act_s; xa.out_sums = e->act_m; xa.out_chunk0 = c.o_chunk0;
    xa.n_kv = c.num_key_value_heads; xa.group = c.num_attention_heads / c.num_key_value_heads; xa.head_dim = hd;
    xa.max_seq = e->kv_stride; xa.layer = l; xa.sc_stride = e->kv_stride; xa.blk_stride = (e->kv_stride + 127) / 128;
    xa.ctx_cap = attn_ctx_cap(e); xa.ring = e->ring;
    xa.kv_bits = c.kv_bits; xa.attn_scale = 1.0f / sqrtf((float)hd); xa.err_flag = e->ctx->d_err; xa.trace = nullptr; xa.v_t = e->v_t;
    return count(e, launch_attention_exact(s, xa, e->pdl, T), "attention", 2);
}

// Attention of token t of a batch of T for layer l: the output becomes row t of the o_proj activation.
bool enqueue_attention(KronosCudaEngine *e, uint32_t l, uint32_t t, uint32_t T, bool long_ctx) {
    const KronosCudaEngineConfig &c = e->cfg;
    cudaStream_t s = e->ctx->stream;
    const EngineLayer &L = e->layers[l];
    const uint32_t hd = c.head_dim, q_dim = c.num_attention_heads * hd, qkv_rows = q_dim + 2 * c.num_key_value_heads * hd;
        float *qkv_t = e->qkv + (size_t)t * qkv_rows;
        int8_t *oq = e->act_q + (size_t)t * q_dim;
        float *os = e->act_s + (size_t)t * (q_dim / 64);
        int32_t *om = e->act_m + (size_t)t * (q_dim / 64);
        float *tap = (l + 1 == c.num_layers && t + 1 == T) ? e->attn_tap : nullptr;
        if (!long_ctx && e->ring.window == 0) {       // contexts of up to ATTN_EXACT_CTX positions: one kernel, CPU summation order
            FusedAttnArgs fa{};
            fa.qkv = qkv_t; fa.bias = L.qkv_bias; fa.q_norm = L.q_norm; fa.k_norm = L.k_norm; fa.rope = e->rope;
            fa.pos = e->d_pos; fa.pos_offset = t;
            fa.k_q8 = e->k_q8; fa.v_q8 = e->v_q8; fa.k_scale = e->k_scale; fa.v_scale = e->v_scale;
            fa.attn_tap = tap;
            fa.out_q = oq; fa.out_scales = os; fa.out_sums = om; fa.err_flag = e->ctx->d_err;
            fa.n_q = c.num_attention_heads; fa.n_kv = c.num_key_value_heads; fa.head_dim = hd; fa.max_seq = e->kv_stride; fa.layer = l;
            fa.eps = c.rms_norm_eps; fa.attn_scale = 1.0f / sqrtf((float)hd); fa.qk_norm_after_rope = c.qk_norm_after_rope;
            fa.kv_bits = c.kv_bits; fa.out_chunk0 = c.o_chunk0;
            fa.trace = (e->attn_trace && l == 0) ? e->d_dbg : nullptr;
            fa.v_t = e->v_t;
            fa.early = T == 1 ? 1u : 0u;        // in a batch the launch before is the attention of the token before: it wrote a row this one reads
            if (!count(e, launch_attention_fused(s, fa, e->pdl), "attention")) return false;
        } else {
            QkvPostArgs qa{};
            qa.qkv = qkv_t; qa.bias = L.qkv_bias; qa.q_norm = L.q_norm; qa.k_norm = L.k_norm; qa.rope = e->rope;
            qa.pos = e->d_pos; qa.pos_offset = t;
            qa.q_i8 = e->q_i8; qa.q_scale = e->q_scale; qa.k_q8 = e->k_q8; qa.v_q8 = e->v_q8; qa.k_scale = e->k_scale; qa.v_scale = e->v_scale;
            qa.n_q = c.num_attention_heads; qa.n_kv = c.num_key_value_heads; qa.head_dim = hd; qa.max_seq = e->kv_stride; qa.layer = l;
            qa.eps = c.rms_norm_eps; qa.qk_norm_after_rope = c.qk_norm_after_rope; qa.kv_bits = c.kv_bits; qa.ring = e->ring; qa.v_t = e->v_t;
            if (!count(e, launch_qkv_post(s, qa, e->pdl), "qkv_post")) return false;
            if (!e->split_kv) {
                ExactAttnArgs xa{};
                xa.q_i8 = e->q_i8; xa.q_scale = e->q_scale; xa.k_q8 = e->k_q8; xa.v_q8 = e->v_q8; xa.k_scale = e->k_scale; xa.v_scale = e->v_scale;
                xa.pos = e->d_pos; xa.pos_offset = t;
                xa.sc = e->attn_sc; xa.bmax = e->attn_bmax; xa.attn_out = tap;
                xa.out_q = oq; xa.out_scales = os; xa.out_sums = om; xa.out_chunk0 = c.o_chunk0;
                xa.n_kv = c.num_key_value_heads; xa.group = c.num_attention_heads / c.num_key_value_heads; xa.head_dim = hd;
                xa.max_seq = e->kv_stride; xa.layer = l; xa.sc_stride = e->kv_stride; xa.blk_stride = (e->kv_stride + 127) / 128;
                xa.ctx_cap = attn_ctx_cap(e); xa.ring = e->ring;
                xa.kv_bits = c.kv_bits; xa.attn_scale = 1.0f / sqrtf((float)hd); xa.err_flag = e->ctx->d_err;
                xa.trace = (e->attn_trace && l == 0) ? e->d_dbg + 16 : nullptr; xa.v_t = e->v_t;
                return count(e, launch_attention_exact(s, xa, e->pdl), "attention", 2);
            }
            AttnArgs aa{};
            aa.q_i8 = e->q_i8; aa.q_scale = e->q_scale; aa.k_q8 = e->k_q8; aa.v_q8 = e->v_q8; aa.k_scale = e->k_scale; aa.v_scale = e->v_scale;
            aa.pos = e->d_pos; aa.pos_offset = t;
            aa.part_m = e->part_m; aa.part_l = e->part_l; aa.part_o = e->part_o; aa.attn_out = tap;
            aa.out_q = oq; aa.out_scales = os; aa.out_sums = om; aa.out_chunk0 = c.o_chunk0;
            aa.n_kv = c.num_key_value_heads; aa.group = c.num_attention_heads / c.num_key_value_heads; aa.head_dim = hd;
            aa.max_seq = e->kv_stride; aa.layer = l; aa.n_split = e->n_split; aa.attn_scale = 1.0f / sqrtf((float)hd); aa.kv_bits = c.kv_bits;
            aa.err_flag = e->ctx->d_err;
            if (!count(e, launch_attention(s, aa, e->pdl), "attention", 2)) return false;
        }
    return true;
}

// Queues the kernels of a batch of T <= 4 consecutive tokens on the context's stream (T = 1: one decode step).
// `embed`: look the T tokens of d_token up first (otherwise `hidden` already holds the T embeddings).  Every
// projection reads its weights once for the whole batch (small-N GEMM); attention runs token by token because
// token t attends to the keys of the tokens before it in the same batch.  `tail`: Greedy = lm_head + argmax for
// the (single) token; LastLogits = lm_head for the last token of the batch; AllLogits = for all T; None = no lm_head.
// The position word is advanced by T at the end (by the argmax kernel when Greedy).
bool enqueue_batch(KronosCudaEngine *e, uint32_t T, bool embed, Tail tail, bool long_ctx) {
    const KronosCudaEngineConfig &c = e->cfg;
    cudaStream_t s = e->ctx->stream;
    const uint32_t h = c.hidden_size, hd = c.head_dim, q_dim = c.num_attention_heads * hd, inter = c.intermediate_size;
    const uint32_t qkv_rows = q_dim + 2 * c.num_key_value_heads * hd;
    (void)qkv_rows; (void)hd;
    if (T == 1 && e->fused && tail != Tail::None) return enqueue_fused_step(e, embed, tail, long_ctx);
    e->final_hidden = nullptr;
    if (embed) {
        EmbedArgs a{};
        fill_embed_args(e, a);
        if (!count(e, launch_embed(s, a, T, false), "embed")) return false;
    }
    for (uint32_t l = 0; l < c.num_layers; ++l) {
        const EngineLayer &L = e->layers[l];
        // the FFN output of the layer before: partial sums under tensor parallelism, and after a MoE block under expert parallelism
        const bool ffn_partial = c.tp_size > 1 || (c.ep_size > 1 && l > 0 && e->layers[l - 1].moe);
        if (!norm_quant(e, l == 0 ? nullptr : e->proj, L.input_norm, nullptr, T, e->pdl && (embed || l > 0), ffn_partial)) return false;
        if (!gemv(e, L.qkv, e->qkv, "gemv qkv", T)) return false;
        if (T > 1 && !e->split_kv) {
            if (!enqueue_attention_batch(e, l, T)) return false;
        } else {
            for (uint32_t t = 0; t < T; ++t)
                if (!enqueue_attention(e, l, t, T, long_ctx)) return false;
        }
        if (!gemv(e, L.o, e->proj, "gemv o", T)) return false;        // under tp: partial sums, exchanged by the norm kernel that follows
        if (L.moe) {
            // SparseMoeRuntime::forward_layer_single (sparse_moe.rs:961-1084) for every token of the batch in five launches
            // (forward_layer_coalesced_batch, 1090-1352, gives each token the same sums: its routes are visited in ascending
            // expert order either way): routes of all tokens, then the expert projections over the (token, route) pairs -
            // slot = token * k + route; two tokens that picked the same expert read its image twice, the second time from L2.
            if (!norm_quant(e, e->proj, L.post_norm, e->x_norm, T, e->pdl, c.tp_size > 1)) return false;
            const uint32_t k = std::min(c.moe_top_k, c.moe_num_experts), dff = c.moe_d_ff;
            // shared expert (every token; under expert parallelism rank 0's partial sum carries it): two plain projections
            // around the experts' SwiGLU kernel, and its sigmoid gate
            const bool shared = L.gate_up != nullptr && (c.ep_size <= 1 || c.ep_rank == 0);
            if (shared) {
                if (!gemv(e, L.gate_up, e->sh_gu, "shared gate_up", T)) return false;
                if (!count(e, launch_expert_swiglu_quant(s, e->sh_gu, L.sh_inter, T, e->sh_q, e->sh_s, e->sh_m, e->pdl), "shared swiglu")) return false;
                if (!gemv_from(e, L.down, e->sh_q, e->sh_s, e->sh_m, e->sh_out, "shared down", T)) return false;
                if (L.sh_gate_w && !count(e, launch_shared_gate(s, L.sh_gate_w, e->x_norm, h, T, e->sh_scale, e->pdl), "shared gate")) return false;
            }
            RouterArgs ra{};
            ra.w = L.router_w; ra.bias = L.router_bias; ra.x = e->x_norm;
            ra.n_experts = c.moe_num_experts; ra.hidden = h; ra.top_k = k; ra.norm_topk = (int32_t)(c.moe_norm_topk & 1u); ra.scoring = c.moe_norm_topk >> 8;
            ra.route_ids = L.d_route_ids; ra.route_w = L.d_route_w; ra.logits = e->router_logits; ra.done = e->router_done; ra.route_stride = 32; ra.err_flag = e->ctx->d_err;
            if (!count(e, launch_moe_router(s, ra, e->pdl, T), "router")) return false;
            if (!count(e, launch_gemv_experts(s, L.gu_dm, L.gu_fmt, L.d_gu_books, L.d_gu_bases, L.d_route_ids, T * k, e->act_q, e->act_s, e->act_m, h, h / 64,
                                              e->moe_gu, (size_t)2 * dff, e->ctx->sm_count, e->ctx->d_err, e->pdl, c.moe_num_experts, k, 32, k), "expert gate_up")) return false;
            if (!count(e, launch_expert_swiglu_quant(s, e->moe_gu, dff, T * k, e->moe_q, e->moe_s, e->moe_m, e->pdl), "expert swiglu")) return false;
            if (!count(e, launch_gemv_experts(s, L.dn_dm, L.dn_fmt, L.d_dn_books, L.d_dn_bases, L.d_route_ids, T * k, e->moe_q, e->moe_s, e->moe_m, dff, dff / 64,
                                              e->moe_out, h, e->ctx->sm_count, e->ctx->d_err, e->pdl, c.moe_num_experts, k, 32, 1), "expert down")) return false;
            if (!count(e, launch_moe_combine(s, e->moe_out, L.d_route_w, k, h, e->proj, e->pdl, L.d_route_ids, c.ep_size > 1 ? L.d_dn_bases : nullptr,
                                             c.moe_num_experts, T, 32, shared ? e->sh_out : nullptr, shared && L.sh_gate_w ? e->sh_scale : nullptr), "moe combine")) return false;
            continue;
        }
        if (!norm_quant(e, e->proj, L.post_norm, nullptr, T, e->pdl, c.tp_size > 1)) return false;
        if (!gemv(e, L.gate_up, e->gate_up, "gemv gate_up", T)) return false;
        if (!count(e, launch_swiglu_quant(s, e->gate_up, inter, e->act_q, e->act_s, e->act_m, nullptr, c.down_chunk0, T, e->pdl), "swiglu")) return false;
        if (!gemv(e, L.down, e->proj, "gemv down", T)) return false;
    }
    // the last residual is folded into `hidden` by the final norm even when no logits are wanted
    if (!norm_quant(e, e->proj, e->final_norm, nullptr, T, e->pdl, c.tp_size > 1 || (c.ep_size > 1 && e->layers.back().moe))) return false;
    const uint32_t vocab_all = c.tp_size > 1 ? c.vocab_total : c.vocab_size;
    float *lg = c.tp_size > 1 ? e->logits_local : e->logits;        // under tp: this rank's slice, then gathered into `logits`
    if (tail == Tail::AllLogits || tail == Tail::Greedy) {
        if (!gemv(e, e->lm_head, lg, "gemv lm_head", T)) return false;
        for (uint32_t t = 0; t < T && c.tp_size > 1; ++t)
            if (!tp_gather(e, lg + (size_t)t * c.vocab_size, e->logits + (size_t)t * vocab_all, c.vocab_size)) return false;
    } else if (tail == Tail::LastLogits) {
        if (!gemv(e, e->lm_head, lg, "gemv lm_head", 1, T - 1)) return false;
        if (c.tp_size > 1 && !tp_gather(e, lg, e->logits, c.vocab_size)) return false;
    }
    if (tail == Tail::Greedy) return count(e, launch_argmax_step(s, e->logits, vocab_all, e->d_token, e->d_pos, e->d_history, e->d_step, e->argmax_scratch, e->pdl), "argmax");
    return count(e, launch_advance_pos(s, e->d_pos, T, e->pdl), "advance");
}

bool set_u32(KronosCudaEngine *e, uint32_t *dst, uint32_t v) {
    return cuda_ok(e->ctx, cudaMemcpyAsync(dst, &v, 4, cudaMemcpyHostToDevice, e->ctx->stream), "set scalar") &&
           cuda_ok(e->ctx, cudaStreamSynchronize(e->ctx->stream), "set scalar sync");
}

// Captures one step into an executable graph (first use on the current stream).
bool ensure_graphs(KronosCudaEngine *e, size_t warm_pos) {
    KronosCudaContext *ctx = e->ctx;
    if (e->graphs[0] && e->graph_stream == ctx->stream) return true;
    for (cudaGraphExec_t &g : e->graphs) if (g) { cudaGraphExecDestroy(g); g = nullptr; }
    // eager steps first: loads every kernel and sets its attributes outside a capture, where an error is also
    // easier to attribute.  They run token 0 at the position the caller is about to run for real: the only cache row
    // they touch is that position's, which the real step rewrites before anything attends to it, so a prompt already
    // in the cache (and, with a sliding window, every live row of the ring) stays as it is.  Callers set position and
    // token before every replay.
    const int variants = 2;
    const uint32_t wp = (uint32_t)std::min<size_t>(warm_pos, e->cfg.max_seq_len - 1);
    for (int long_ctx = 0; long_ctx < variants; ++long_ctx)
        if (!set_u32(e, e->d_pos, wp) || !set_u32(e, e->d_token, 0) || !enqueue_batch(e, 1, true, Tail::Greedy, long_ctx != 0) ||
            !sync_and_check(ctx, "engine warm-up step"))
            return false;
    const uint64_t launches_before = ctx->launches;
    for (int which = 0; which < 4; ++which) {
        cudaGraph_t graph = nullptr;
        if (!cuda_ok(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal), "begin capture")) return false;
#ifdef K2T_TIMELINE
        e->tl_labels[which].clear();
        e->tl_cur = &e->tl_labels[which];
#endif
        const bool ok = enqueue_batch(e, 1, true, which < 2 ? Tail::Greedy : Tail::LastLogits, (which & 1) != 0);
#ifdef K2T_TIMELINE
        e->tl_cur = nullptr;
#endif
        cudaError_t err = cudaStreamEndCapture(ctx->stream, &graph);
        if (!ok || !cuda_ok(ctx, err, "end capture")) { if (graph) cudaGraphDestroy(graph); return false; }
        cudaGraphExec_t exec = nullptr;
        err = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (!cuda_ok(ctx, err, "graph instantiate")) return false;
        e->graphs[which] = exec;
    }
    ctx->launches = launches_before;          // captured, not launched
    e->graph_stream = ctx->stream;
    return true;
}

// the graph of one step: greedy (argmax on the device) or logits only, for the context length this position gives
cudaGraphExec_t step_graph(const KronosCudaEngine *e, bool greedy, size_t pos) {
    return e->graphs[(greedy ? 0 : 2) + ((pos + 1 > ATTN_EXACT_CTX || e->ring.window) ? 1 : 0)];
}
uint32_t step_launches(const KronosCudaEngine *e, size_t pos) {
    if (e->fused) {      // lm_head + argmax; per layer qkv, attention (1 or 3 kernels), o, and gate_up / down or norm / router / two expert GEMVs
        uint32_t n = 2;
        for (const EngineLayer &L : e->layers) n += ((pos + 1 > ATTN_EXACT_CTX || e->ring.window) ? 3 : 1) + (L.moe ? 6 : 4);
        return n;
    }
    uint32_t n = 1 + 2 + 1 + (e->cfg.tp_size > 1 ? 1 : 0);
    for (const EngineLayer &L : e->layers) {     // MoE FFN: 6 kernels for 4 (+ 3 or 4 of a shared expert); the tensor-parallel sums ride in the norm kernels
        n += ((pos + 1 > ATTN_EXACT_CTX || e->ring.window) ? 10 : 8) + (L.moe ? 2 : 0);
        if (L.moe && L.gate_up && (e->cfg.ep_size <= 1 || e->cfg.ep_rank == 0)) n += 3 + (L.sh_gate_w ? 1 : 0);
    }
    return n;
}

constexpr uint32_t TRACE_CAP = 2048;

// Builds the device-side tables of the whole-token decode kernel.  Leaves mega_ok false (with the reason in
// mega_why) when the model does not fit the kernel; the per-operator path then serves every call.
bool setup_mega(KronosCudaEngine *e) {
    KronosCudaContext *ctx = e->ctx;
    const KronosCudaEngineConfig &c = e->cfg;
    // Off unless KRONOS_CUDA_MEGA=1: at the model sizes measured so far a grid barrier costs as much as a kernel
    // boundary of the CUDA-graph path (about 2 us) and the phases between them are latency-bound, so the graph of
    // per-operator kernels decodes faster; the kernel is kept for its phase trace and as the base for further work.
    const char *want = std::getenv("KRONOS_CUDA_MEGA");
    if (!want || want[0] != '1') { e->mega_why = "not requested (KRONOS_CUDA_MEGA=1 enables it)"; return true; }
    if (c.num_attention_heads > (uint32_t)ctx->sm_count) { e->mega_why = "more query heads than SMs"; return true; }
    if (e->has_moe) { e->mega_why = "sparse-MoE layers are served by the per-operator path"; return true; }
    if (e->ring.window) { e->mega_why = "a sliding KV window is served by the per-operator path"; return true; }
    if (c.tp_size > 1 || c.ep_size > 1) { e->mega_why = "tensor- and expert-parallel ranks are served by the per-operator path"; return true; }
    uint32_t warp_smem = 0;
    auto fill = [&](const KronosCudaMatrix *m, MegaMatrix &mm) {
        const int fmt = fill_gemv_args(m->dm, true, mm.g);
        mm.fmt = (uint32_t)fmt;
        mm.g.err_flag = ctx->d_err;
        const uint32_t np = (mm.g.nc + 31) / 32, n_rb = (mm.g.rows + 3) / 4;
        uint32_t wk = 1;
        while (wk < 8 && wk * 2 <= np && n_rb * wk < 8u * (uint32_t)ctx->sm_count) wk *= 2;
        mm.wk = wk;
        warp_smem = std::max(warp_smem, gemv_warp_smem_bytes(fmt));
    };
    std::vector<MegaLayer> layers(c.num_layers);
    for (uint32_t l = 0; l < c.num_layers; ++l) {
        const EngineLayer &L = e->layers[l];
        fill(L.qkv, layers[l].qkv); fill(L.o, layers[l].o); fill(L.gate_up, layers[l].gate_up); fill(L.down, layers[l].down);
        layers[l].input_norm = L.input_norm; layers[l].post_norm = L.post_norm; layers[l].qkv_bias = L.qkv_bias;
        layers[l].q_norm = L.q_norm; layers[l].k_norm = L.k_norm;
    }
    MegaMatrix head;
    fill(e->lm_head, head);
    e->mega_warp_smem = (warp_smem + 127u) & ~127u;
    e->mega_kmax = std::max(std::max(c.hidden_size, c.num_attention_heads * c.head_dim), c.intermediate_size);
    e->mega_smem = decode_mega_smem(e->mega_warp_smem, e->mega_kmax);
    cudaError_t chk = decode_mega_check(e->mega_smem, ctx->sm_count);
    if (chk != cudaSuccess) {
        cudaGetLastError();
        e->mega_why = std::string("kernel does not fit one CTA per SM: ") + cudaGetErrorString(chk);
        return true;
    }
    if (!dev_alloc(e, e->d_barrier, 1) || !dev_alloc(e, e->d_trace, TRACE_CAP + 1) ||
        !dev_alloc(e, e->d_mega_layers, layers.size(), layers.data()) || !dev_alloc(e, e->d_mega_head, 1, &head) ||
        !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "decode kernel tables"))      // the host vectors go out of scope
        return false;
    e->mega_ok = true;
    return true;
}

void fill_embed_args(const KronosCudaEngine *e, EmbedArgs &a) {
    const KronosCudaMatrix *src = e->embed_matrix ? e->embed_matrix : e->lm_head;
    const MatrixGeom &g = src->dm.geom;
    for (int k = 0; k < 3; ++k) { a.plane[k] = src->dm.d_base + g.plane_off[k]; a.cell[k] = g.cell[k]; }
    a.scales = reinterpret_cast<const uint16_t *>(src->dm.d_base + g.scale_off);
    a.embed_bf16 = e->embed_bf16; a.token = e->d_token; a.hidden = e->hidden;
    a.fmt = g.fmt; a.nc = g.nc; a.rows_pad = g.rows_pad; a.sgc = g.sgc; a.max_odd = g.max_odd;
    a.sgc_shift = 32;
    for (uint32_t sh = 0; sh < 4; ++sh) if ((1u << sh) == g.sgc) a.sgc_shift = sh;
    for (int i = 0; i < 32; ++i) a.codebook[i] = g.codebook32[i];
}

// n_steps greedy tokens in one cooperative launch (contexts up to ATTN_EXACT_CTX positions)
bool decode_mega(KronosCudaEngine *e, uint32_t first_token, uint32_t pos_start, uint32_t n_steps) {
    KronosCudaContext *ctx = e->ctx;
    const KronosCudaEngineConfig &c = e->cfg;
    MegaArgs a{};
    a.layers = e->d_mega_layers; a.head = e->d_mega_head;
    a.n_layers = c.num_layers; a.hidden = c.hidden_size; a.n_q = c.num_attention_heads; a.n_kv = c.num_key_value_heads;
    a.head_dim = c.head_dim; a.inter = c.intermediate_size; a.vocab = c.vocab_size; a.max_seq = e->kv_stride; a.kv_bits = c.kv_bits;
    a.eps = c.rms_norm_eps; a.attn_scale = 1.0f / sqrtf((float)c.head_dim); a.qk_norm_after_rope = c.qk_norm_after_rope;
    a.final_norm = e->final_norm; a.rope = e->rope;
    fill_embed_args(e, a.embed);
    a.hidden_a = e->hidden2; a.hidden_b = e->hidden; a.proj = e->proj; a.qkv = e->qkv; a.gate_up = e->gate_up; a.logits = e->logits;
    a.attn_tap = e->attn_tap; a.act_q = e->act_q; a.act_s = e->act_s; a.act_m = e->act_m;
    a.k_q8 = e->k_q8; a.v_q8 = e->v_q8; a.k_scale = e->k_scale; a.v_scale = e->v_scale; a.v_t = e->v_t;
    a.token = e->d_token; a.pos = e->d_pos; a.step = e->d_step; a.history = e->d_history;
    a.barrier = e->d_barrier; a.err_flag = ctx->d_err;
    a.first_token = first_token; a.pos0 = pos_start; a.n_steps = n_steps;
    a.warp_smem = e->mega_warp_smem; a.kmax = e->mega_kmax;
    a.trace = e->d_trace; a.trace_cap = TRACE_CAP;
    if (!cuda_ok(ctx, cudaMemsetAsync(e->d_barrier, 0, 4, ctx->stream), "clear barrier")) return false;
    ctx->launches += 1;
    return cuda_ok(ctx, launch_decode_mega(ctx->stream, a, e->mega_smem, ctx->sm_count), "decode kernel launch");
}


// Uploads the experts of one MoE layer from its .k2tm records (nf_expert_byte_layout, moe_800b.rs:1330-1383).
// Returns an error text, empty on success.
std::string setup_moe_layer(KronosCudaEngine *e, EngineLayer &L, const KronosCudaLayerDesc &d) {
    KronosCudaContext *ctx = e->ctx;
    const KronosCudaEngineConfig &c = e->cfg;
    const uint32_t E = c.moe_num_experts, h = c.hidden_size, dff = c.moe_d_ff, bits = c.moe_bits, sgc = std::max(1u, c.moe_scale_group_chunks);
    if (E < 2 || E > 256 || c.moe_top_k == 0 || c.moe_top_k > 32) return "MoE geometry: 2..256 experts and 1..32 routes per token are supported";
    if (bits < 2 || bits > 5 || dff == 0 || dff % 64 || (2 * dff) % 32 || h % 32) return "MoE geometry: NF bits 2..5, d_ff a multiple of 64";
    static const size_t chunk_bytes[6] = {0, 0, 256, 384, 512, 640};
    const size_t cb = chunk_bytes[bits];
    const size_t gu_chunks = h / 64, gu_sg = (gu_chunks + sgc - 1) / sgc, dn_chunks = dff / 64, dn_sg = (dn_chunks + sgc - 1) / sgc;
    const size_t gu_bytes = (size_t)(2 * dff / 32) * (gu_sg * 64 + gu_chunks * 2 * cb), dn_bytes = (size_t)(h / 32) * (dn_sg * 64 + dn_chunks * 2 * cb);
    const size_t gu_off = 64, dn_off = (gu_off + gu_bytes + 63) / 64 * 64, rec = (dn_off + dn_bytes + 16383) / 16384 * 16384;
    if (rec != c.moe_expert_bytes) return "moe_expert_bytes does not match the record layout of this geometry";
    if (!d.moe_shard || d.moe_shard_len < (size_t)E * rec) return "expert shard is shorter than moe_num_experts records";
    if (!dev_alloc(e, L.router_w, (size_t)E * h, d.moe_router_w)) return ctx->err;
    if (d.moe_router_bias && !dev_alloc(e, L.router_bias, E, d.moe_router_bias)) return ctx->err;
    std::vector<const uint8_t *> gu_bases(E, nullptr), dn_bases(E, nullptr);
    std::vector<ExpertCodebook> gu_books(E), dn_books(E);
    L.expert0 = c.ep_size > 1 ? c.ep_rank : 0;         // the first expert this rank holds: geometry template of the expert kernels
    // every expert of the layer has the same shapes, so the same image sizes: one device allocation and one upload per
    // layer (12,288 single allocations took 25 s for the 48 x 128 experts of the 30B-A3B shape), images repacked on the
    // host by a few threads
    std::vector<uint32_t> owned;
    for (uint32_t x = 0; x < E; ++x)
        if (c.ep_size <= 1 || x % c.ep_size == c.ep_rank) owned.push_back(x);
    auto desc_of = [&](uint32_t x, bool down) {
        const uint8_t *r = d.moe_shard + (size_t)x * rec;
        KronosCudaMatrixDesc m{};
        m.kind = KRONOS_CUDA_MATRIX_NF; m.bits = bits; m.scale_group_chunks = sgc;
        if (!down) { m.rows = 2 * dff; m.cols = h; std::memcpy(m.codebook, r, 16); m.data0 = r + gu_off; m.len0 = gu_bytes; }
        else { m.rows = h; m.cols = dff; std::memcpy(m.codebook, r + 16, 16); m.data0 = r + dn_off; m.len0 = dn_bytes; }
        return m;
    };
    MatrixGeom g_gu, g_dn;
    std::string why;
    {
        const KronosCudaMatrixDesc m0 = desc_of(owned[0], false), m1 = desc_of(owned[0], true);
        if (!matrix_geometry(m0, g_gu, why) || !matrix_geometry(m1, g_dn, why)) return "expert matrices: " + why;
    }
    const size_t img_gu = (g_gu.image_bytes() + 255) & ~(size_t)255, img_dn = (g_dn.image_bytes() + 255) & ~(size_t)255, img = img_gu + img_dn;
    std::vector<uint8_t> host;
    try { host.resize(owned.size() * img); } catch (...) { return "out of host memory for the expert images"; }
    std::vector<MatrixGeom> geo_gu(owned.size()), geo_dn(owned.size());
    std::vector<std::string> errs(owned.size());
    {
        const unsigned n_thr = std::max(1u, std::min(16u, std::thread::hardware_concurrency()));
        std::vector<std::thread> pool;
        for (unsigned t = 0; t < n_thr; ++t)
            pool.emplace_back([&, t] {
                for (size_t i = t; i < owned.size(); i += n_thr) {
                    const KronosCudaMatrixDesc m0 = desc_of(owned[i], false), m1 = desc_of(owned[i], true);
                    if (!matrix_geometry(m0, geo_gu[i], errs[i]) || !matrix_geometry(m1, geo_dn[i], errs[i])) continue;
                    repack_matrix(m0, geo_gu[i], false, host.data() + i * img, 1);
                    repack_matrix(m1, geo_dn[i], false, host.data() + i * img + img_gu, 1);
                }
            });
        for (std::thread &th : pool) th.join();
    }
    for (size_t i = 0; i < owned.size(); ++i)
        if (!errs[i].empty()) return "expert " + std::to_string(owned[i]) + ": " + errs[i];
    if (!dev_alloc(e, L.d_experts, host.size(), host.data()) || !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "expert upload")) return ctx->err;
    bool first = true;
    for (size_t i = 0; i < owned.size(); ++i) {
        const uint32_t x = owned[i];
        DeviceMatrix gu{geo_gu[i], L.d_experts + i * img, img_gu}, dn{geo_dn[i], L.d_experts + i * img + img_gu, img_dn};
        // every expert of a layer decodes with one kernel: NF4 falls back to the general decode for all of them as soon
        // as one codebook does not fit the two-table form
        const int fg = expert_codebook(gu, gu_books[x]), fd = expert_codebook(dn, dn_books[x]);
        if (fg < 0 || fd < 0) return "expert matrices in an unsupported format";
        L.gu_fmt = first ? fg : (L.gu_fmt == fg ? fg : (int)FMT_COUNT);
        L.dn_fmt = first ? fd : (L.dn_fmt == fd ? fd : (int)FMT_COUNT);
        if (first) { L.gu_dm = gu; L.dn_dm = dn; }
        first = false;
        gu_bases[x] = gu.d_base; dn_bases[x] = dn.d_base;
    }
    if (!dev_alloc(e, L.d_gu_books, E, gu_books.data()) || !dev_alloc(e, L.d_dn_books, E, dn_books.data()) ||
        !dev_alloc(e, L.d_gu_bases, E, gu_bases.data()) || !dev_alloc(e, L.d_dn_bases, E, dn_bases.data()) ||
        !dev_alloc(e, L.d_route_ids, (size_t)e->max_batch * 32) || !dev_alloc(e, L.d_route_w, (size_t)e->max_batch * 32) ||
        !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "MoE tables"))
        return ctx->err;
    e->has_moe = true;
    // one token streams the router and the routed experts
    e->weight_bytes += (size_t)E * h * 4 + (size_t)std::min(c.moe_top_k, E) * (gu_bytes + dn_bytes + 32);
    return std::string();
}

}  // namespace

extern "C" {

void kronos_cuda_engine_destroy(KronosCudaEngine *e) {
    if (!e) return;
    cudaSetDevice(e->ctx->device);
    cudaStreamSynchronize(e->ctx->stream);
    for (cudaGraphExec_t g : e->graphs) if (g) cudaGraphExecDestroy(g);
    for (EngineLayer &L : e->layers)
    {
        for (KronosCudaMatrix *m : {L.qkv, L.o, L.gate_up, L.down})
            if (m) kronos_cuda_matrix_free(e->ctx, m);
    }
    if (e->lm_head) kronos_cuda_matrix_free(e->ctx, e->lm_head);
    if (e->embed_matrix) kronos_cuda_matrix_free(e->ctx, e->embed_matrix);
    for (void *p : e->tp_peers) cudaIpcCloseMemHandle(p);
    for (void *p : e->allocs) cudaFree(p);
    delete e;
}

KronosCudaEngine *kronos_cuda_engine_create(KronosCudaContext *ctx, const KronosCudaEngineConfig *cfg, const float *rope,
                                            const KronosCudaLayerDesc *layers, size_t n_layers, const float *final_norm,
                                            const KronosCudaMatrixDesc *lm_head, const uint16_t *embed_bf16) {
    if (!ctx) return nullptr;
    ctx->err.clear();
    if (!cfg || !rope || !layers || !final_norm || !lm_head) { fail(ctx, "engine_create: NULL argument"); return nullptr; }
    const KronosCudaEngineConfig &c = *cfg;
    if (c.struct_size != sizeof(KronosCudaEngineConfig)) {
        fail(ctx, "engine_create: config.struct_size is " + std::to_string(c.struct_size) + ", this library's KronosCudaEngineConfig has " +
                      std::to_string(sizeof(KronosCudaEngineConfig)) + " bytes (binding out of date?)");
        return nullptr;
    }
    if (n_layers != c.num_layers || c.num_layers == 0) { fail(ctx, "engine_create: n_layers does not match the config"); return nullptr; }
    if (c.head_dim != 64 && c.head_dim != 128) { fail(ctx, "engine_create: head_dim must be 64 or 128"); return nullptr; }
    if (c.hidden_size % 64 || c.intermediate_size % 64 || c.hidden_size == 0) { fail(ctx, "engine_create: hidden and intermediate sizes must be multiples of 64"); return nullptr; }
    if (c.num_key_value_heads == 0 || c.num_attention_heads % c.num_key_value_heads || c.num_attention_heads / c.num_key_value_heads > 8) {
        fail(ctx, "engine_create: query heads must be a multiple (at most 8x) of the kv heads"); return nullptr; }
    if (c.kv_bits != 8 && c.kv_bits != 4) { fail(ctx, "engine_create: kv_bits must be 8 (int8 Hadamard cache) or 4 (NF4 Hadamard cache)"); return nullptr; }
    if (c.max_seq_len == 0) { fail(ctx, "engine_create: max_seq_len is 0"); return nullptr; }
    if (c.tp_size > 1) {
        if (c.tp_size > TP_MAX || c.tp_rank >= c.tp_size) { fail(ctx, "engine_create: tp_size up to 8 and tp_rank below it"); return nullptr; }
        if (c.vocab_total != c.vocab_size * c.tp_size || c.vocab_size % 4) { fail(ctx, "engine_create: vocab_total must be tp_size equal lm_head slices"); return nullptr; }
    }
    if (c.ep_size > 1) {
        if (c.tp_size > 1) { fail(ctx, "engine_create: expert parallelism is not combined with tensor parallelism"); return nullptr; }
        if (c.ep_size > TP_MAX || c.ep_rank >= c.ep_size || c.ep_size > c.moe_num_experts) { fail(ctx, "engine_create: ep_size up to 8 (and at most the experts), ep_rank below it"); return nullptr; }
    }
    if (!make_current(ctx)) return nullptr;
    const uint32_t h = c.hidden_size, hd = c.head_dim, q_dim = c.num_attention_heads * hd, kv_dim = c.num_key_value_heads * hd;
    const uint32_t qkv_rows = q_dim + 2 * kv_dim, inter = c.intermediate_size;
    KronosCudaEngine *e = new (std::nothrow) KronosCudaEngine();
    if (!e) { fail(ctx, "engine_create: out of host memory"); return nullptr; }
    e->ctx = ctx; e->cfg = c;
    {   // split-KV attention runs one warp per (kv head, split): enough splits to put about eight warps on every SM,
        // at most 128 (a split is at least one 32-position tile of a context above ATTN_EXACT_CTX)
        const uint32_t want = (8u * (uint32_t)ctx->sm_count + c.num_key_value_heads - 1) / c.num_key_value_heads;
        e->n_split = std::min(128u, std::max(32u, (want + 3u) & ~3u));
    }
    if (const char *v = std::getenv("KRONOS_CUDA_PROMPT_BATCH")) {                  // tokens per prompt batch (default 256: 1.7B-shape prompts 13.5k / 18.8k / 21.8k tok/s at 64 / 128 / 256)
        const uint32_t n = (uint32_t)std::strtoul(v, nullptr, 10);
        e->max_batch = std::min(512u, std::max(16u, (n + 15u) & ~15u));
    }
    if (const char *v = std::getenv("KRONOS_CUDA_PDL")) e->pdl = v[0] != '0';     // measurement switch (default on)
    if (const char *v = std::getenv("KRONOS_CUDA_ATTN_TRACE")) e->attn_trace = v[0] == '1';
    if (const char *v = std::getenv("KRONOS_CUDA_FUSED")) e->fused = v[0] == '1';     // measurement switch
    if (c.tp_size > 1 || c.ep_size > 1) e->fused = false;       // the exchanges of the parallel modes live in the norm kernel
    e->layers.resize(c.num_layers);
    auto bad = [&](const std::string &why) { std::string keep = why; kronos_cuda_engine_destroy(e); fail(ctx, keep); return (KronosCudaEngine *)nullptr; };
    auto shape_ok = [](const KronosCudaMatrixDesc &d, uint32_t rows, uint32_t cols) { return d.rows == rows && d.cols == cols; };
    for (uint32_t l = 0; l < c.num_layers; ++l) {
        const KronosCudaLayerDesc &d = layers[l];
        EngineLayer &L = e->layers[l];
        if (!d.input_norm || !d.post_attn_norm) return bad("engine_create: a layer has no norm weights");
        L.moe = d.moe_router_w != nullptr;
        if (!shape_ok(d.qkv_proj, qkv_rows, h) || !shape_ok(d.o_proj, h, q_dim) ||
            (!L.moe && (!shape_ok(d.gate_up_proj, 2 * inter, h) || !shape_ok(d.down_proj, h, inter))))
            return bad("engine_create: layer " + std::to_string(l) + " has a projection whose shape does not match the config");
        if (!dev_alloc(e, L.input_norm, h, d.input_norm) || !dev_alloc(e, L.post_norm, h, d.post_attn_norm)) return bad(ctx->err);
        if (d.qkv_bias && !dev_alloc(e, L.qkv_bias, qkv_rows, d.qkv_bias)) return bad(ctx->err);
        if (d.q_norm && !dev_alloc(e, L.q_norm, hd, d.q_norm)) return bad(ctx->err);
        if (d.k_norm && !dev_alloc(e, L.k_norm, hd, d.k_norm)) return bad(ctx->err);
        L.qkv = kronos_cuda_matrix_upload(ctx, &d.qkv_proj, 0);
        L.o = L.qkv ? kronos_cuda_matrix_upload(ctx, &d.o_proj, 0) : nullptr;
        if (!L.o) return bad("engine_create: layer " + std::to_string(l) + ": " + ctx->err);
        e->weight_bytes += L.qkv->dm.geom.file_bytes + L.o->dm.geom.file_bytes;
        if (L.moe) {
            const std::string why = setup_moe_layer(e, L, d);
            if (!why.empty()) return bad("engine_create: layer " + std::to_string(l) + ": " + why);
            if (d.gate_up_proj.rows > 0 || d.down_proj.rows > 0) {         // the layer's shared expert
                const uint32_t sh = d.down_proj.cols;
                if (d.gate_up_proj.kind != KRONOS_CUDA_MATRIX_NF || d.down_proj.kind != KRONOS_CUDA_MATRIX_NF || sh == 0 || sh % 64 != 0 ||
                    !shape_ok(d.gate_up_proj, 2 * sh, h) || !shape_ok(d.down_proj, h, sh))
                    return bad("engine_create: layer " + std::to_string(l) + ": the shared expert must be two NF matrices [2 inter][hidden] and [hidden][inter]");
                L.gate_up = kronos_cuda_matrix_upload(ctx, &d.gate_up_proj, 0);
                L.down = L.gate_up ? kronos_cuda_matrix_upload(ctx, &d.down_proj, 0) : nullptr;
                if (!L.down) return bad("engine_create: layer " + std::to_string(l) + ": shared expert: " + ctx->err);
                if (d.moe_shared_gate_w && !dev_alloc(e, L.sh_gate_w, h, d.moe_shared_gate_w)) return bad(ctx->err);
                L.sh_inter = sh;
                e->sh_inter_max = std::max(e->sh_inter_max, sh);
                e->weight_bytes += L.gate_up->dm.geom.file_bytes + L.down->dm.geom.file_bytes;
                e->fused = false;               // the fused-prologue path has no shared-expert form
            }
            continue;
        }
        L.gate_up = kronos_cuda_matrix_upload(ctx, &d.gate_up_proj, 0);
        L.down = L.gate_up ? kronos_cuda_matrix_upload(ctx, &d.down_proj, 0) : nullptr;
        if (!L.down) return bad("engine_create: layer " + std::to_string(l) + ": " + ctx->err);
        e->weight_bytes += L.gate_up->dm.geom.file_bytes + L.down->dm.geom.file_bytes;
    }
    if (!shape_ok(*lm_head, c.vocab_size, h)) return bad("engine_create: lm_head shape does not match the config");
    e->lm_head = kronos_cuda_matrix_upload(ctx, lm_head, 0);
    if (!e->lm_head) return bad("engine_create: lm_head: " + ctx->err);
    e->weight_bytes += e->lm_head->dm.geom.file_bytes;
    const uint32_t act_n = std::max(std::max(h, q_dim), inter), n_q = c.num_attention_heads;
    bool ok = dev_alloc(e, e->final_norm, h, final_norm) && dev_alloc(e, e->rope, (size_t)c.max_seq_len * hd, rope) &&
              (embed_bf16 == nullptr || dev_alloc(e, e->embed_bf16, (size_t)(c.tp_size > 1 ? c.vocab_total : c.vocab_size) * h, embed_bf16)) &&   // every rank keeps the whole table
              // per-token vectors hold max_batch tokens (prompt batches), [token][n]
              dev_alloc(e, e->hidden, (size_t)e->max_batch * h) && dev_alloc(e, e->hidden2, h) && dev_alloc(e, e->proj, (size_t)e->max_batch * h) &&
              dev_alloc(e, e->qkv, (size_t)e->max_batch * qkv_rows) && dev_alloc(e, e->gate_up, (size_t)e->max_batch * 2 * inter) &&
              dev_alloc(e, e->logits, (size_t)e->max_batch * (c.tp_size > 1 ? c.vocab_total : c.vocab_size)) && dev_alloc(e, e->act_q, (size_t)e->max_batch * act_n) &&
              dev_alloc(e, e->act_s, (size_t)e->max_batch * act_n / 64) && dev_alloc(e, e->act_m, (size_t)e->max_batch * act_n / 64) &&
              dev_alloc(e, e->q_i8, (size_t)e->max_batch * q_dim) && dev_alloc(e, e->attn_tap, q_dim) && dev_alloc(e, e->q_scale, (size_t)e->max_batch * n_q) &&
              dev_alloc(e, e->part_m, (size_t)n_q * e->n_split) && dev_alloc(e, e->part_l, (size_t)n_q * e->n_split) &&
              dev_alloc(e, e->part_o, (size_t)n_q * e->n_split * hd) &&
              alloc_kv(e, c.kv_bits, c.kv_window, c.kv_sinks) &&
              dev_alloc(e, e->d_token, e->max_batch) && dev_alloc(e, e->d_pos, 1) && dev_alloc(e, e->d_step, 1) &&
              dev_alloc(e, e->d_history, c.max_seq_len) && dev_alloc(e, e->d_dbg, 32) && dev_alloc(e, e->argmax_scratch, ARGMAX_SCRATCH_WORDS);
    const uint32_t xg = c.tp_size > 1 ? c.tp_size : c.ep_size, xr = c.tp_size > 1 ? c.tp_rank : c.ep_rank;     // exchange group
    if (ok && xg > 1) {
        if (e->has_moe && c.tp_size > 1) return bad("engine_create: sparse-MoE layers are not combined with tensor parallelism");
        const size_t slot = std::max<size_t>((size_t)e->max_batch * h, c.vocab_size), floats = 2 * (size_t)xg * slot;
        void *raw = nullptr;
        // floats | 256 bytes of flags | (value, call number) words of the fused sums: [2][tp][max_batch * hidden] x 8 bytes
        const size_t ll_slot = (size_t)e->max_batch * h, total = floats * 4 + 256 + 2 * (size_t)xg * ll_slot * 8;
        ok = cuda_ok(ctx, cudaMalloc(&raw, total), "cudaMalloc(tp exchange)");
        if (ok) {
            e->allocs.push_back(raw);
            e->tp_buf = static_cast<float *>(raw);
            e->tp.ll_slot = (uint32_t)ll_slot;
            e->tp.peer_ll[xr] = reinterpret_cast<unsigned long long *>(static_cast<uint8_t *>(raw) + floats * 4 + 256);
            e->tp.wait_polls = TP_WAIT_POLLS_DEFAULT;
            if (const char *v = std::getenv("KRONOS_CUDA_PEER_WAIT_POLLS")) e->tp.wait_polls = (uint32_t)std::strtoul(v, nullptr, 10);
            ok = cuda_ok(ctx, cudaMemsetAsync(raw, 0, total, ctx->stream), "clear tp exchange") &&
                 dev_alloc(e, e->tp.epoch, 1) && dev_alloc(e, e->tp_done, 1) && dev_alloc(e, e->logits_local, (size_t)e->max_batch * c.vocab_size);
            e->tp.tp = xg; e->tp.rank = xr; e->tp.slot = (uint32_t)slot; e->tp.err = ctx->d_err;
            e->tp.peer_data[xr] = e->tp_buf;
            e->tp.peer_flags[xr] = reinterpret_cast<uint32_t *>(e->tp_buf + floats);
        }
    }
    if (ok && e->has_moe) {
        const uint32_t k = std::min(c.moe_top_k, c.moe_num_experts), dff = c.moe_d_ff;
        ok = dev_alloc(e, e->x_norm, (size_t)e->max_batch * h) && dev_alloc(e, e->router_logits, (size_t)e->max_batch * 256) && dev_alloc(e, e->router_done, e->max_batch) &&
             dev_alloc(e, e->moe_gu, (size_t)e->max_batch * k * 2 * dff) && dev_alloc(e, e->moe_out, (size_t)e->max_batch * k * h) &&
             dev_alloc(e, e->moe_q, (size_t)e->max_batch * k * dff) && dev_alloc(e, e->moe_s, (size_t)e->max_batch * k * dff / 64) &&
             dev_alloc(e, e->moe_m, (size_t)e->max_batch * k * dff / 64);
        if (ok && e->sh_inter_max > 0) {
            const size_t si = e->sh_inter_max;
            ok = dev_alloc(e, e->sh_gu, (size_t)e->max_batch * 2 * si) && dev_alloc(e, e->sh_out, (size_t)e->max_batch * h) && dev_alloc(e, e->sh_scale, e->max_batch) &&
                 dev_alloc(e, e->sh_q, (size_t)e->max_batch * si) && dev_alloc(e, e->sh_s, (size_t)e->max_batch * si / 64) && dev_alloc(e, e->sh_m, (size_t)e->max_batch * si / 64);
        }
    }
    if (!ok || !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "engine_create sync")) return bad(ctx->err);
    if (!setup_mega(e)) return bad(ctx->err);
    return e;
}

size_t kronos_cuda_engine_kv_bytes(const KronosCudaEngine *e, size_t positions) {
    if (!e) return 0;
    // int8 keys and values plus one fp32 scale each per (layer, kv head, position): the reference's
    // 2 * layers * n_kv * (head_dim + 4) bytes per position (real_llm.rs:10223)
    const size_t hd = e->cfg.head_dim, per_head = e->cfg.kv_bits == 4 ? hd / 2 + 2 * (hd / 64) : hd + 4;   // NF4: packed + bf16 per 64
    return positions * 2 * (size_t)e->cfg.num_layers * e->cfg.num_key_value_heads * per_head;
}
size_t kronos_cuda_engine_weight_bytes(const KronosCudaEngine *e) { return e ? e->weight_bytes : 0; }
int64_t kronos_cuda_engine_profile_step(KronosCudaEngine *e, uint32_t token, size_t pos, uint32_t reps, char *table, size_t cap);

int32_t kronos_cuda_engine_read_hidden(KronosCudaEngine *e, float *hidden) {
    if (!e || !hidden) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!make_current(ctx)) return -1;
    // the final norm kernel has already folded the last down_proj into the residual stream
    const float *src = e->final_hidden ? e->final_hidden : e->hidden + (size_t)e->last_row * e->cfg.hidden_size;
    if (!cuda_ok(ctx, cudaMemcpyAsync(hidden, src, (size_t)e->cfg.hidden_size * 4,
                                      cudaMemcpyDeviceToHost, ctx->stream), "read hidden") ||
        !sync_and_check(ctx, "read hidden"))
        return -1;
    return 0;
}

int32_t kronos_cuda_engine_tp_handle(KronosCudaEngine *e, uint8_t handle[64]) {
    if (!e || !handle) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!e->tp_buf) return fail(ctx, "tp_handle: the engine was created with tp_size <= 1 and ep_size <= 1"), -1;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaIpcMemHandle_t hnd;
    if (!make_current(ctx) || !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "tp_handle") ||      // the buffer is cleared by now
        !cuda_ok(ctx, cudaIpcGetMemHandle(&hnd, e->tp_buf), "cudaIpcGetMemHandle"))
        return -1;
    std::memcpy(handle, &hnd, 64);
    return 0;
}

int32_t kronos_cuda_engine_tp_attach(KronosCudaEngine *e, const uint8_t *handles, size_t n_handles) {
    if (!e) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!e->tp_buf) return fail(ctx, "tp_attach: the engine was created with tp_size <= 1 and ep_size <= 1"), -1;
    if (!handles || n_handles != e->tp.tp) return fail(ctx, "tp_attach: one handle per rank is needed"), -1;
    if (e->tp_ready) return fail(ctx, "tp_attach: already attached"), -1;
    if (!make_current(ctx)) return -1;
    const size_t floats = 2 * (size_t)e->tp.tp * e->tp.slot;
    for (uint32_t r = 0; r < e->tp.tp; ++r) {
        if (r == e->tp.rank) continue;
        cudaIpcMemHandle_t hnd;
        std::memcpy(&hnd, handles + (size_t)r * 64, 64);
        void *p = nullptr;
        if (!cuda_ok(ctx, cudaIpcOpenMemHandle(&p, hnd, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")) return -1;
        e->tp_peers.push_back(p);
        e->tp.peer_data[r] = static_cast<float *>(p);
        e->tp.peer_flags[r] = reinterpret_cast<uint32_t *>(static_cast<float *>(p) + floats);
        e->tp.peer_ll[r] = reinterpret_cast<unsigned long long *>(static_cast<uint8_t *>(p) + floats * 4 + 256);
    }
    e->tp_ready = true;
    return 0;
}

int32_t kronos_cuda_engine_tp_attach_local(KronosCudaEngine *e, KronosCudaEngine *const *engines, size_t n_engines) {
    if (!e) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!e->tp_buf) return fail(ctx, "tp_attach_local: the engine was created with tp_size <= 1 and ep_size <= 1"), -1;
    if (!engines || n_engines != e->tp.tp) return fail(ctx, "tp_attach_local: one engine per rank is needed"), -1;
    if (e->tp_ready) return fail(ctx, "tp_attach_local: already attached"), -1;
    if (!make_current(ctx)) return -1;
    const size_t floats = 2 * (size_t)e->tp.tp * e->tp.slot;
    for (uint32_t r = 0; r < e->tp.tp; ++r) {
        if (r == e->tp.rank) continue;
        const KronosCudaEngine *o = engines[r];
        if (!o || !o->tp_buf || o->tp.tp != e->tp.tp || o->tp.rank != r || o->tp.slot != e->tp.slot || o->tp.ll_slot != e->tp.ll_slot)
            return fail(ctx, "tp_attach_local: engine " + std::to_string(r) + " is not rank " + std::to_string(r) + " of the same group"), -1;
        if (o->ctx->device != ctx->device) {
            cudaError_t pe = cudaDeviceEnablePeerAccess(o->ctx->device, 0);
            if (pe == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
            else if (!cuda_ok(ctx, pe, "cudaDeviceEnablePeerAccess")) return -1;
        }
        e->tp.peer_data[r] = o->tp_buf;
        e->tp.peer_flags[r] = reinterpret_cast<uint32_t *>(o->tp_buf + floats);
        e->tp.peer_ll[r] = reinterpret_cast<unsigned long long *>(reinterpret_cast<uint8_t *>(o->tp_buf) + floats * 4 + 256);
    }
    e->tp_ready = true;
    return 0;
}

int32_t kronos_cuda_engine_set_embedding_matrix(KronosCudaEngine *e, const KronosCudaMatrixDesc *whole) {
    if (!e) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!whole || whole->cols != e->cfg.hidden_size) return fail(ctx, "set_embedding_matrix: the matrix must have hidden_size columns"), -1;
    if (e->embed_matrix) { kronos_cuda_matrix_free(ctx, e->embed_matrix); e->embed_matrix = nullptr; }
    e->embed_matrix = kronos_cuda_matrix_upload(ctx, whole, 0);
    for (cudaGraphExec_t &g : e->graphs) if (g) { cudaGraphExecDestroy(g); g = nullptr; }      // captured embed arguments are stale
    return e->embed_matrix ? 0 : -1;
}

size_t kronos_cuda_engine_read_routes(KronosCudaEngine *e, uint32_t layer, uint32_t *experts, float *weights) {
    if (!e || !experts || !weights || layer >= e->cfg.num_layers || !e->layers[layer].moe) return 0;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!make_current(ctx)) return 0;
    const EngineLayer &L = e->layers[layer];
    const size_t k = std::min(e->cfg.moe_top_k, e->cfg.moe_num_experts);
    if (!cuda_ok(ctx, cudaMemcpyAsync(experts, L.d_route_ids + e->last_row * 32, k * 4, cudaMemcpyDeviceToHost, ctx->stream), "read routes") ||
        !cuda_ok(ctx, cudaMemcpyAsync(weights, L.d_route_w + e->last_row * 32, k * 4, cudaMemcpyDeviceToHost, ctx->stream), "read routes") ||
        !sync_and_check(ctx, "read routes"))
        return 0;
    return k;
}

int32_t kronos_cuda_engine_read_attention(KronosCudaEngine *e, float *attention) {
    if (!e || !attention) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!make_current(ctx)) return -1;
    const size_t n = (size_t)e->cfg.num_attention_heads * e->cfg.head_dim;
    if (!cuda_ok(ctx, cudaMemcpyAsync(attention, e->attn_tap, n * 4, cudaMemcpyDeviceToHost, ctx->stream), "read attention") ||
        !sync_and_check(ctx, "read attention"))
        return -1;
    return 0;
}

size_t kronos_cuda_engine_decode_trace(KronosCudaEngine *e, uint64_t *marks_ns, size_t cap) {
    if (!e || !e->mega_ok || !marks_ns) return 0;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!make_current(ctx)) return 0;
    std::vector<unsigned long long> buf(TRACE_CAP + 1);
    if (!cuda_ok(ctx, cudaMemcpyAsync(buf.data(), e->d_trace, buf.size() * 8, cudaMemcpyDeviceToHost, ctx->stream), "read trace") ||
        !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "read trace"))
        return 0;
    const size_t n = std::min<size_t>(std::min<size_t>(buf[TRACE_CAP], TRACE_CAP), cap);
    for (size_t i = 0; i < n; ++i) marks_ns[i] = buf[i];
    return n;
}

int32_t kronos_cuda_engine_read_kv(KronosCudaEngine *e, uint32_t layer, uint32_t kv_head, size_t position, int8_t *k_q8,
                                   float *k_scale, int8_t *v_q8, float *v_scale) {
    if (!e) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!k_q8 || !k_scale || !v_q8 || !v_scale) return fail(ctx, "read_kv: NULL buffer"), -1;
    if (layer >= e->cfg.num_layers || kv_head >= e->cfg.num_key_value_heads || position >= e->cfg.max_seq_len)
        return fail(ctx, "read_kv: index out of range"), -1;
    if (e->cfg.kv_bits != 8) return fail(ctx, "read_kv: the engine holds an NF4 cache (use read_kv_q4)"), -1;
    if (!make_current(ctx)) return -1;
    const size_t slot = ((size_t)layer * e->cfg.num_key_value_heads + kv_head) * e->kv_stride + e->ring.slot_of_pos((uint32_t)position), hd = e->cfg.head_dim;
    cudaStream_t s = ctx->stream;
    if (!cuda_ok(ctx, cudaMemcpyAsync(k_q8, e->k_q8 + slot * hd, hd, cudaMemcpyDeviceToHost, s), "read_kv") ||
        !cuda_ok(ctx, cudaMemcpyAsync(v_q8, e->v_q8 + slot * hd, hd, cudaMemcpyDeviceToHost, s), "read_kv") ||
        !cuda_ok(ctx, cudaMemcpyAsync(k_scale, e->k_scale + slot, 4, cudaMemcpyDeviceToHost, s), "read_kv") ||
        !cuda_ok(ctx, cudaMemcpyAsync(v_scale, e->v_scale + slot, 4, cudaMemcpyDeviceToHost, s), "read_kv"))
        return -1;
    return sync_and_check(ctx, "read_kv") ? 0 : -1;
}

int32_t kronos_cuda_engine_read_kv_q4(KronosCudaEngine *e, uint32_t layer, uint32_t kv_head, size_t position, uint8_t *k_q4,
                                      uint16_t *k_s16, uint8_t *v_q4, uint16_t *v_s16) {
    if (!e) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!k_q4 || !k_s16 || !v_q4 || !v_s16) return fail(ctx, "read_kv_q4: NULL buffer"), -1;
    if (layer >= e->cfg.num_layers || kv_head >= e->cfg.num_key_value_heads || position >= e->cfg.max_seq_len)
        return fail(ctx, "read_kv_q4: index out of range"), -1;
    if (e->cfg.kv_bits != 4) return fail(ctx, "read_kv_q4: the engine holds an int8 cache (use read_kv)"), -1;
    if (!make_current(ctx)) return -1;
    const size_t slot = ((size_t)layer * e->cfg.num_key_value_heads + kv_head) * e->kv_stride + e->ring.slot_of_pos((uint32_t)position), hd = e->cfg.head_dim;
    const size_t nb = hd / 64;
    cudaStream_t s = ctx->stream;
    if (!cuda_ok(ctx, cudaMemcpyAsync(k_q4, reinterpret_cast<uint8_t *>(e->k_q8) + slot * hd / 2, hd / 2, cudaMemcpyDeviceToHost, s), "read_kv_q4") ||
        !cuda_ok(ctx, cudaMemcpyAsync(v_q4, reinterpret_cast<uint8_t *>(e->v_q8) + slot * hd / 2, hd / 2, cudaMemcpyDeviceToHost, s), "read_kv_q4") ||
        !cuda_ok(ctx, cudaMemcpyAsync(k_s16, reinterpret_cast<uint16_t *>(e->k_scale) + slot * nb, nb * 2, cudaMemcpyDeviceToHost, s), "read_kv_q4") ||
        !cuda_ok(ctx, cudaMemcpyAsync(v_s16, reinterpret_cast<uint16_t *>(e->v_scale) + slot * nb, nb * 2, cudaMemcpyDeviceToHost, s), "read_kv_q4"))
        return -1;
    return sync_and_check(ctx, "read_kv_q4") ? 0 : -1;
}

// ---- KV blobs: the reference's position-major export format (KvSlotPtrs::export / import, src/model/kv_blob.rs:47-110):
// for every position, for every (layer, kv head): key row, key scale(s), value row, value scale(s).
static size_t kv_row_bytes(const KronosCudaEngine *e) { return e->cfg.kv_bits == 4 ? e->cfg.head_dim / 2 : e->cfg.head_dim; }
static size_t kv_scale_bytes(const KronosCudaEngine *e) { return e->cfg.kv_bits == 4 ? 2 * (e->cfg.head_dim / 64) : 4; }

size_t kronos_cuda_engine_kv_bytes_per_pos(const KronosCudaEngine *e) {
    return e ? 2 * (size_t)e->cfg.num_layers * e->cfg.num_key_value_heads * (kv_row_bytes(e) + kv_scale_bytes(e)) : 0;
}

int64_t kronos_cuda_engine_kv_export(KronosCudaEngine *e, size_t lo, size_t hi, uint8_t *out, size_t cap) {
    if (!e) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (lo > hi || hi > e->cfg.max_seq_len) return fail(ctx, "kv_export: position range out of bounds"), -1;
    const size_t n = hi - lo, heads = (size_t)e->cfg.num_layers * e->cfg.num_key_value_heads, db = kv_row_bytes(e), sb = kv_scale_bytes(e);
    const size_t total = n * kronos_cuda_engine_kv_bytes_per_pos(e);
    if (n == 0) return 0;
    if (!out || cap < total) return fail(ctx, "kv_export: output buffer too small"), -1;
    if (!make_current(ctx)) return -1;
    const size_t S = e->kv_stride;
    cudaStream_t st = ctx->stream;
    if (e->ring.ring_len > 0) {           // ring: fetch every row of the (small) cache and pick each position's row
        const size_t R = e->kv_rows;
        std::vector<uint8_t> kd(heads * R * db), vd(heads * R * db), ks(heads * R * sb), vs(heads * R * sb);
        if (!cuda_ok(ctx, cudaMemcpy2DAsync(kd.data(), R * db, e->k_q8, S * db, R * db, heads, cudaMemcpyDeviceToHost, st), "kv_export") ||
            !cuda_ok(ctx, cudaMemcpy2DAsync(vd.data(), R * db, e->v_q8, S * db, R * db, heads, cudaMemcpyDeviceToHost, st), "kv_export") ||
            !cuda_ok(ctx, cudaMemcpy2DAsync(ks.data(), R * sb, e->k_scale, S * sb, R * sb, heads, cudaMemcpyDeviceToHost, st), "kv_export") ||
            !cuda_ok(ctx, cudaMemcpy2DAsync(vs.data(), R * sb, e->v_scale, S * sb, R * sb, heads, cudaMemcpyDeviceToHost, st), "kv_export") ||
            !sync_and_check(ctx, "kv_export"))
            return -1;
        uint8_t *w = out;
        for (size_t p = lo; p < hi; ++p) {
            const size_t r = e->ring.slot_of_pos((uint32_t)p);
            for (size_t h = 0; h < heads; ++h) {
                std::memcpy(w, kd.data() + (h * R + r) * db, db); w += db;
                std::memcpy(w, ks.data() + (h * R + r) * sb, sb); w += sb;
                std::memcpy(w, vd.data() + (h * R + r) * db, db); w += db;
                std::memcpy(w, vs.data() + (h * R + r) * sb, sb); w += sb;
            }
        }
        return (int64_t)total;
    }
    std::vector<uint8_t> kd(heads * n * db), vd(heads * n * db), ks(heads * n * sb), vs(heads * n * sb);
    if (!cuda_ok(ctx, cudaMemcpy2DAsync(kd.data(), n * db, reinterpret_cast<uint8_t *>(e->k_q8) + lo * db, S * db, n * db, heads, cudaMemcpyDeviceToHost, st), "kv_export") ||
        !cuda_ok(ctx, cudaMemcpy2DAsync(vd.data(), n * db, reinterpret_cast<uint8_t *>(e->v_q8) + lo * db, S * db, n * db, heads, cudaMemcpyDeviceToHost, st), "kv_export") ||
        !cuda_ok(ctx, cudaMemcpy2DAsync(ks.data(), n * sb, reinterpret_cast<uint8_t *>(e->k_scale) + lo * sb, S * sb, n * sb, heads, cudaMemcpyDeviceToHost, st), "kv_export") ||
        !cuda_ok(ctx, cudaMemcpy2DAsync(vs.data(), n * sb, reinterpret_cast<uint8_t *>(e->v_scale) + lo * sb, S * sb, n * sb, heads, cudaMemcpyDeviceToHost, st), "kv_export") ||
        !sync_and_check(ctx, "kv_export"))
        return -1;
    uint8_t *w = out;
    for (size_t p = 0; p < n; ++p)
        for (size_t h = 0; h < heads; ++h) {
            std::memcpy(w, kd.data() + (h * n + p) * db, db); w += db;
            std::memcpy(w, ks.data() + (h * n + p) * sb, sb); w += sb;
            std::memcpy(w, vd.data() + (h * n + p) * db, db); w += db;
            std::memcpy(w, vs.data() + (h * n + p) * sb, sb); w += sb;
        }
    return (int64_t)total;
}

int32_t kronos_cuda_engine_kv_import(KronosCudaEngine *e, const uint8_t *data, size_t len, size_t n) {
    if (!e) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (n > e->cfg.max_seq_len) return fail(ctx, "kv_import: more positions than max_seq_len"), -1;
    if (n == 0) return 0;
    if (!data || len < n * kronos_cuda_engine_kv_bytes_per_pos(e)) return fail(ctx, "kv_import: blob is shorter than n positions"), -1;
    if (!make_current(ctx)) return -1;
    const size_t heads = (size_t)e->cfg.num_layers * e->cfg.num_key_value_heads, db = kv_row_bytes(e), sb = kv_scale_bytes(e), S = e->kv_stride;
    if (e->ring.ring_len > 0) {           // ring: positions go to their rows in order (a later position overwrites the row it shares)
        const size_t R = e->kv_rows;
        std::vector<uint8_t> kd(heads * R * db), vd(heads * R * db), ks(heads * R * sb), vs(heads * R * sb);
        const uint8_t *rd = data;
        for (size_t p = 0; p < n; ++p) {
            const size_t row = e->ring.slot_of_pos((uint32_t)p);
            for (size_t h = 0; h < heads; ++h) {
                std::memcpy(kd.data() + (h * R + row) * db, rd, db); rd += db;
                std::memcpy(ks.data() + (h * R + row) * sb, rd, sb); rd += sb;
                std::memcpy(vd.data() + (h * R + row) * db, rd, db); rd += db;
                std::memcpy(vs.data() + (h * R + row) * sb, rd, sb); rd += sb;
            }
        }
        cudaStream_t st = ctx->stream;
        if (!cuda_ok(ctx, cudaMemcpy2DAsync(e->k_q8, S * db, kd.data(), R * db, R * db, heads, cudaMemcpyHostToDevice, st), "kv_import") ||
            !cuda_ok(ctx, cudaMemcpy2DAsync(e->v_q8, S * db, vd.data(), R * db, R * db, heads, cudaMemcpyHostToDevice, st), "kv_import") ||
            !cuda_ok(ctx, cudaMemcpy2DAsync(e->k_scale, S * sb, ks.data(), R * sb, R * sb, heads, cudaMemcpyHostToDevice, st), "kv_import") ||
            !cuda_ok(ctx, cudaMemcpy2DAsync(e->v_scale, S * sb, vs.data(), R * sb, R * sb, heads, cudaMemcpyHostToDevice, st), "kv_import") ||
            !sync_vt(e) || !sync_and_check(ctx, "kv_import"))
            return -1;
        return 0;
    }
    std::vector<uint8_t> kd(heads * n * db), vd(heads * n * db), ks(heads * n * sb), vs(heads * n * sb);
    const uint8_t *r = data;
    for (size_t p = 0; p < n; ++p)
        for (size_t h = 0; h < heads; ++h) {
            std::memcpy(kd.data() + (h * n + p) * db, r, db); r += db;
            std::memcpy(ks.data() + (h * n + p) * sb, r, sb); r += sb;
            std::memcpy(vd.data() + (h * n + p) * db, r, db); r += db;
            std::memcpy(vs.data() + (h * n + p) * sb, r, sb); r += sb;
        }
    cudaStream_t st = ctx->stream;
    if (!cuda_ok(ctx, cudaMemcpy2DAsync(e->k_q8, S * db, kd.data(), n * db, n * db, heads, cudaMemcpyHostToDevice, st), "kv_import") ||
        !cuda_ok(ctx, cudaMemcpy2DAsync(e->v_q8, S * db, vd.data(), n * db, n * db, heads, cudaMemcpyHostToDevice, st), "kv_import") ||
        !cuda_ok(ctx, cudaMemcpy2DAsync(e->k_scale, S * sb, ks.data(), n * sb, n * sb, heads, cudaMemcpyHostToDevice, st), "kv_import") ||
        !cuda_ok(ctx, cudaMemcpy2DAsync(e->v_scale, S * sb, vs.data(), n * sb, n * sb, heads, cudaMemcpyHostToDevice, st), "kv_import") ||
        !sync_vt(e) || !sync_and_check(ctx, "kv_import"))
        return -1;
    return 0;
}

int32_t kronos_cuda_engine_reconfigure_kv(KronosCudaEngine *e, uint32_t kv_bits, size_t window, size_t sinks) {
    if (!e) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!make_current(ctx) || !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "reconfigure_kv")) return -1;
    if (e->cfg.tp_size > 1 || e->cfg.ep_size > 1) {
        if (window != 0) return fail(ctx, "reconfigure_kv: a sliding window is not combined with tensor / expert parallelism"), -1;
    }
    if (!alloc_kv(e, kv_bits, (uint32_t)std::min<size_t>(window, 0xffffffffu), (uint32_t)std::min<size_t>(sinks, 0xffffffffu)) ||
        !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "reconfigure_kv"))
        return -1;
    if (e->ring.window) e->mega_ok = false;
    return 0;
}

int32_t kronos_cuda_engine_kv_sliding_window(const KronosCudaEngine *e, size_t *window, size_t *sinks) {
    if (!e) return -1;
    if (window) *window = e->ring.window;
    if (sinks) *sinks = e->ring.sinks;
    return e->ring.window ? 1 : 0;
}

size_t kronos_cuda_engine_kv_rows(const KronosCudaEngine *e) { return e ? e->kv_rows : 0; }

int32_t kronos_cuda_engine_can_truncate_kv_to(const KronosCudaEngine *e, size_t cur_pos, size_t target_len) {
    if (!e) return 0;
    if (target_len >= cur_pos) return 1;
    if (e->ring.ring_len > 0) {
        const size_t live = e->ring.window - e->ring.sinks, slack = e->ring.ring_len > live ? e->ring.ring_len - live : 0;
        return (target_len <= e->ring.sinks || cur_pos - target_len <= slack) ? 1 : 0;
    }
    return 1;
}

// ---- KV prefix snapshots (KvPrefixSnapshot::Q8 / Q4, RealLlamaEngine::save_kv_prefix / restore_kv_prefix_slice,
// real_llm.rs:5821-6155): head-major copies of the first rows of every (layer, kv head) - the first n positions, or the
// whole ring when a sliding window is active.  Blob = 32-byte header {"K2TKVPFX", kv_bits, slots_per_head, heads, head_dim,
// 0, 0} + the snapshot's four vectors in field order: key rows, value rows, key scales, value scales.
static const char KV_PREFIX_MAGIC[8] = {'K', '2', 'T', 'K', 'V', 'P', 'F', 'X'};

size_t kronos_cuda_engine_kv_prefix_bytes(const KronosCudaEngine *e, size_t n, size_t cur_pos) {
    if (!e) return 0;
    const size_t len = std::min(n, cur_pos), slots = e->ring.ring_len > 0 ? e->kv_rows : std::min<size_t>(len, e->kv_rows);
    const size_t heads = (size_t)e->cfg.num_layers * e->cfg.num_key_value_heads;
    return 32 + 2 * heads * slots * (kv_row_bytes(e) + kv_scale_bytes(e));
}

int64_t kronos_cuda_engine_save_kv_prefix(KronosCudaEngine *e, size_t n, size_t cur_pos, uint8_t *out, size_t cap) {
    if (!e) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    const size_t total = kronos_cuda_engine_kv_prefix_bytes(e, n, cur_pos);
    if (!out || cap < total) return fail(ctx, "save_kv_prefix: output buffer too small"), -1;
    if (!make_current(ctx)) return -1;
    const size_t len = std::min(n, cur_pos), slots = e->ring.ring_len > 0 ? e->kv_rows : std::min<size_t>(len, e->kv_rows);
    const size_t heads = (size_t)e->cfg.num_layers * e->cfg.num_key_value_heads, db = kv_row_bytes(e), sb = kv_scale_bytes(e), S = e->kv_stride;
    std::memcpy(out, KV_PREFIX_MAGIC, 8);
    const uint32_t hdr[6] = {e->cfg.kv_bits, (uint32_t)slots, (uint32_t)heads, e->cfg.head_dim, 0u, 0u};
    std::memcpy(out + 8, hdr, 24);
    if (slots == 0) return (int64_t)total;
    uint8_t *kd = out + 32, *vd = kd + heads * slots * db, *ks = vd + heads * slots * db, *vs = ks + heads * slots * sb;
    cudaStream_t st = ctx->stream;
    if (!cuda_ok(ctx, cudaMemcpy2DAsync(kd, slots * db, e->k_q8, S * db, slots * db, heads, cudaMemcpyDeviceToHost, st), "save_kv_prefix") ||
        !cuda_ok(ctx, cudaMemcpy2DAsync(vd, slots * db, e->v_q8, S * db, slots * db, heads, cudaMemcpyDeviceToHost, st), "save_kv_prefix") ||
        !cuda_ok(ctx, cudaMemcpy2DAsync(ks, slots * sb, e->k_scale, S * sb, slots * sb, heads, cudaMemcpyDeviceToHost, st), "save_kv_prefix") ||
        !cuda_ok(ctx, cudaMemcpy2DAsync(vs, slots * sb, e->v_scale, S * sb, slots * sb, heads, cudaMemcpyDeviceToHost, st), "save_kv_prefix") ||
        !sync_and_check(ctx, "save_kv_prefix"))
        return -1;
    return (int64_t)total;
}

int32_t kronos_cuda_engine_restore_kv_prefix(KronosCudaEngine *e, const uint8_t *data, size_t len, size_t copy_slots) {
    if (!e) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!data || len < 32 || std::memcmp(data, KV_PREFIX_MAGIC, 8) != 0) return fail(ctx, "restore_kv_prefix: not a KV prefix snapshot"), -1;
    uint32_t hdr[6];
    std::memcpy(hdr, data + 8, 24);
    const size_t slots = hdr[1], heads = (size_t)e->cfg.num_layers * e->cfg.num_key_value_heads, db = kv_row_bytes(e), sb = kv_scale_bytes(e), S = e->kv_stride;
    if (hdr[0] != e->cfg.kv_bits || hdr[2] != heads || hdr[3] != e->cfg.head_dim) return fail(ctx, "restore_kv_prefix: the snapshot was taken from a cache of another format or shape"), -1;
    if (len < 32 + 2 * heads * slots * (db + sb)) return fail(ctx, "restore_kv_prefix: snapshot is shorter than its header says"), -1;
    const size_t cp = std::min(slots, copy_slots);
    if (cp > e->kv_rows) return fail(ctx, "restore_kv_prefix: the snapshot holds more rows than the cache"), -1;
    if (cp == 0) return 0;
    if (!make_current(ctx)) return -1;
    const uint8_t *kd = data + 32, *vd = kd + heads * slots * db, *ks = vd + heads * slots * db, *vs = ks + heads * slots * sb;
    cudaStream_t st = ctx->stream;
    if (!cuda_ok(ctx, cudaMemcpy2DAsync(e->k_q8, S * db, kd, slots * db, cp * db, heads, cudaMemcpyHostToDevice, st), "restore_kv_prefix") ||
        !cuda_ok(ctx, cudaMemcpy2DAsync(e->v_q8, S * db, vd, slots * db, cp * db, heads, cudaMemcpyHostToDevice, st), "restore_kv_prefix") ||
        !cuda_ok(ctx, cudaMemcpy2DAsync(e->k_scale, S * sb, ks, slots * sb, cp * sb, heads, cudaMemcpyHostToDevice, st), "restore_kv_prefix") ||
        !cuda_ok(ctx, cudaMemcpy2DAsync(e->v_scale, S * sb, vs, slots * sb, cp * sb, heads, cudaMemcpyHostToDevice, st), "restore_kv_prefix") ||
        !sync_vt(e) || !sync_and_check(ctx, "restore_kv_prefix"))
        return -1;
    return 0;
}

static int32_t forward_common(KronosCudaEngine *e, const float *embeds, const uint32_t *tokens, size_t n_tok, size_t pos_start,
                              float *all_logits, float *last_logits) {
    if (!e) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if ((!embeds && !tokens) || !last_logits) return fail(ctx, "forward: NULL buffer"), -1;
    if (n_tok == 0) return fail(ctx, "forward: n_tok is 0"), -1;
    if (pos_start + n_tok > e->cfg.max_seq_len) return fail(ctx, "forward: sequence would exceed max_seq_len"), -1;
    if (!make_current(ctx)) return -1;
    if (tokens)
        for (size_t t = 0; t < n_tok; ++t)
            if (tokens[t] >= (e->cfg.tp_size > 1 ? e->cfg.vocab_total : e->cfg.vocab_size)) return fail(ctx, "forward: token id out of range"), -1;
    const size_t h = e->cfg.hidden_size, v = e->cfg.tp_size > 1 ? e->cfg.vocab_total : e->cfg.vocab_size;
    if (tokens && n_tok == 1) {         // one decode step: the captured graph
        if (!ensure_graphs(e, pos_start) || !set_u32(e, e->d_pos, (uint32_t)pos_start)) return -1;
        if (!cuda_ok(ctx, cudaMemcpyAsync(e->d_token, tokens, 4, cudaMemcpyHostToDevice, ctx->stream), "copy token") ||
            !cuda_ok(ctx, cudaGraphLaunch(step_graph(e, false, pos_start), ctx->stream), "graph launch"))
            return -1;
        ctx->launches += step_launches(e, pos_start);
        e->last_row = 0;
        if (!cuda_ok(ctx, cudaMemcpyAsync(last_logits, e->logits, v * 4, cudaMemcpyDeviceToHost, ctx->stream), "copy logits") ||
            !sync_and_check(ctx, "forward"))
            return -1;
        if (all_logits) std::memcpy(all_logits, last_logits, v * 4);
        return 0;
    }
    // prompt: batches of up to max_batch tokens (forward_prompt / forward_batch_sdot_impl, real_llm.rs:7407-7448, 7450-7860):
    // every projection as one tensor-core weight pass over the batch, the attention of the batch's tokens side by side
    if (!set_u32(e, e->d_pos, (uint32_t)pos_start)) return -1;
    for (size_t t0 = 0, T_done = 0; t0 < n_tok; t0 += T_done) {
        uint32_t T = (uint32_t)std::min<size_t>(e->max_batch, n_tok - t0);
        const size_t p0 = pos_start + t0;
        if (e->split_kv && p0 < ATTN_EXACT_CTX && p0 + T > ATTN_EXACT_CTX) T = (uint32_t)(ATTN_EXACT_CTX - p0);    // split-KV kernels: a batch stays on one side of the attention switch
        const bool last = t0 + T == n_tok;
        if (tokens) {
            if (!cuda_ok(ctx, cudaMemcpyAsync(e->d_token, tokens + t0, T * 4, cudaMemcpyHostToDevice, ctx->stream), "copy tokens")) return -1;
        } else {
            if (!cuda_ok(ctx, cudaMemcpyAsync(e->hidden, embeds + t0 * h, (size_t)T * h * 4, cudaMemcpyHostToDevice, ctx->stream), "copy embeddings")) return -1;
        }
        const Tail tail = all_logits ? Tail::AllLogits : (last ? Tail::LastLogits : Tail::None);
        e->ctx_bound = (uint32_t)(pos_start + t0 + T);
        const bool queued = enqueue_batch(e, T, tokens != nullptr, tail, pos_start + t0 + T > ATTN_EXACT_CTX);
        e->ctx_bound = 0;
        if (!queued) return -1;
        e->last_row = T - 1;
        T_done = T;
        if (all_logits && !cuda_ok(ctx, cudaMemcpyAsync(all_logits + t0 * v, e->logits, (size_t)T * v * 4, cudaMemcpyDeviceToHost, ctx->stream), "copy logits")) return -1;
        if (!all_logits && last && !cuda_ok(ctx, cudaMemcpyAsync(last_logits, e->logits, v * 4, cudaMemcpyDeviceToHost, ctx->stream), "copy logits")) return -1;
        // the token / embedding staging buffers are reused by the next batch: the copies above are stream-ordered
    }
    if (!sync_and_check(ctx, "forward")) return -1;
    if (all_logits) std::memcpy(last_logits, all_logits + (n_tok - 1) * v, v * 4);
    return 0;
}

int32_t kronos_cuda_engine_forward_tokens(KronosCudaEngine *e, const float *embeds, size_t n_tok, size_t pos_start,
                                          float *all_logits, float *last_logits) {
    return forward_common(e, embeds, nullptr, n_tok, pos_start, all_logits, last_logits);
}

int32_t kronos_cuda_engine_forward_token_ids(KronosCudaEngine *e, const uint32_t *tokens, size_t n_tok, size_t pos_start,
                                             float *all_logits, float *last_logits) {
    return forward_common(e, nullptr, tokens, n_tok, pos_start, all_logits, last_logits);
}

int32_t kronos_cuda_engine_decode_greedy(KronosCudaEngine *e, uint32_t first_token, size_t pos_start, size_t n_steps,
                                         uint32_t *out_tokens, float *last_logits) {
    if (!e) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!out_tokens) return fail(ctx, "decode_greedy: out_tokens is NULL"), -1;
    const size_t vocab_all = e->cfg.tp_size > 1 ? e->cfg.vocab_total : e->cfg.vocab_size;
    if (first_token >= vocab_all) return fail(ctx, "decode_greedy: token id out of range"), -1;
    if (pos_start + n_steps > e->cfg.max_seq_len) return fail(ctx, "decode_greedy: sequence would exceed max_seq_len"), -1;
    if (n_steps == 0) return 0;
    if (!make_current(ctx)) return -1;
    e->last_row = 0;
    if (e->mega_ok && pos_start + n_steps <= ATTN_EXACT_CTX) {
        if (!decode_mega(e, first_token, (uint32_t)pos_start, (uint32_t)n_steps)) return -1;
        if (!cuda_ok(ctx, cudaMemcpyAsync(out_tokens, e->d_history, n_steps * 4, cudaMemcpyDeviceToHost, ctx->stream), "copy tokens")) return -1;
        if (last_logits && !cuda_ok(ctx, cudaMemcpyAsync(last_logits, e->logits, vocab_all * 4, cudaMemcpyDeviceToHost, ctx->stream), "copy logits")) return -1;
        return sync_and_check(ctx, "decode_greedy") ? 0 : -1;
    }
    if (!ensure_graphs(e, pos_start)) return -1;
    const uint32_t init[3] = {first_token, (uint32_t)pos_start, 0u};
    if (!cuda_ok(ctx, cudaMemcpyAsync(e->d_token, &init[0], 4, cudaMemcpyHostToDevice, ctx->stream), "set token") ||
        !cuda_ok(ctx, cudaMemcpyAsync(e->d_pos, &init[1], 4, cudaMemcpyHostToDevice, ctx->stream), "set pos") ||
        !cuda_ok(ctx, cudaMemcpyAsync(e->d_step, &init[2], 4, cudaMemcpyHostToDevice, ctx->stream), "set step") ||
        !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "decode_greedy setup"))
        return -1;
#ifdef K2T_TIMELINE
    // KRONOS_CUDA_TIMELINE=<file>: stamps of every kernel of these steps (see pdl_wait), one line of labels, then one line
    // of nanosecond stamps per step.  All steps must use the same graph variant.
    const char *tl_path = std::getenv("KRONOS_CUDA_TIMELINE");
    unsigned long long *tl_dev = nullptr;
    const size_t tl_cap = 1 << 18;
    if (tl_path) {
        if (!cuda_ok(ctx, cudaMalloc(&tl_dev, (tl_cap + 2) * 8), "timeline buffer")) return -1;
        const unsigned long long head[2] = {0, tl_cap};
        cudaMemcpy(tl_dev, head, 16, cudaMemcpyHostToDevice);
        for (auto set : timeline_setters()) set(tl_dev);
    }
#endif
    for (size_t i = 0; i < n_steps; ++i) {
        if (!cuda_ok(ctx, cudaGraphLaunch(step_graph(e, true, pos_start + i), ctx->stream), "graph launch")) return -1;
        ctx->launches += step_launches(e, pos_start + i);
    }
    if (!cuda_ok(ctx, cudaMemcpyAsync(out_tokens, e->d_history, n_steps * 4, cudaMemcpyDeviceToHost, ctx->stream), "copy tokens")) return -1;
    if (last_logits && !cuda_ok(ctx, cudaMemcpyAsync(last_logits, e->logits, vocab_all * 4, cudaMemcpyDeviceToHost, ctx->stream), "copy logits")) return -1;
    if (!sync_and_check(ctx, "decode_greedy")) return -1;
#ifdef K2T_TIMELINE
    if (tl_path) {
        for (auto set : timeline_setters()) set(nullptr);
        std::vector<unsigned long long> h(tl_cap + 2);
        cudaMemcpy(h.data(), tl_dev, h.size() * 8, cudaMemcpyDeviceToHost);
        cudaFree(tl_dev);
        const int which = (pos_start + 1 > ATTN_EXACT_CTX || e->ring.window) ? 1 : 0;
        const std::vector<const char *> &lab = e->tl_labels[which];
        const size_t n = std::min<size_t>(h[0], tl_cap);
        std::sort(h.begin() + 2, h.begin() + 2 + n);
        if (FILE *f = std::fopen(tl_path, "a")) {
            std::fprintf(f, "steps %zu stamps %zu labels %zu\n", n_steps, n, lab.size());
            for (const char *l : lab) std::fprintf(f, "%s|", l);
            std::fprintf(f, "\n");
            for (size_t i = 0; i < n; ++i) std::fprintf(f, "%llu%c", h[2 + i] - h[2], (i + 1) % std::max<size_t>(1, lab.size()) == 0 ? '\n' : ' ');
            std::fprintf(f, "\n");
            std::fclose(f);
        }
    }
#endif
    if (const char *v = std::getenv("KRONOS_CUDA_DECODE_PROF")) {
        if (v[0] == '1') {              // the step that produced the last token, once more, kernel by kernel (same cache row, same result)
            std::vector<char> table(1 << 14);
            const uint32_t tok = n_steps >= 2 ? out_tokens[n_steps - 2] : first_token;
            if (kronos_cuda_engine_profile_step(e, tok, pos_start + n_steps - 1, 1, table.data(), table.size()) >= 0)
                std::fprintf(stderr, "[kronos_cuda decode profile, position %zu]\n%s", pos_start + n_steps - 1, table.data());
        }
    }
    return 0;
}

int64_t kronos_cuda_engine_profile_step(KronosCudaEngine *e, uint32_t token, size_t pos, uint32_t reps, char *table, size_t cap) {
    if (!e) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!table || cap == 0) return fail(ctx, "profile_step: no output buffer"), -1;
    reps = std::max(1u, reps);
    if (pos + reps > e->cfg.max_seq_len) return fail(ctx, "profile_step: positions beyond max_seq_len"), -1;
    if (!make_current(ctx) || !ensure_graphs(e, pos)) return -1;          // warm: every kernel loaded, attributes set
    // The step is launched kernel by kernel with a timing event after each one (and one in front), without programmatic
    // overlap, so the time between two events is the kernel between them, run alone on a warm device.  A bounded delay
    // kernel keeps the stream busy while the host queues the step, so the gaps between events hold no launch latency.
    const bool pdl_was = e->pdl;
    const bool long_ctx = pos + reps > ATTN_EXACT_CTX;
    std::map<std::string, std::pair<double, uint32_t>> acc;
    std::vector<std::string> order;
    double total = 0.0;
    cudaEvent_t first = nullptr;
    bool ok = cuda_ok(ctx, cudaEventCreate(&first), "profile event");
    const uint32_t init[3] = {token, (uint32_t)pos, 0u};
    ok = ok && cuda_ok(ctx, cudaMemcpyAsync(e->d_token, &init[0], 4, cudaMemcpyHostToDevice, ctx->stream), "set token") &&
         cuda_ok(ctx, cudaMemcpyAsync(e->d_pos, &init[1], 4, cudaMemcpyHostToDevice, ctx->stream), "set pos") &&
         cuda_ok(ctx, cudaMemcpyAsync(e->d_step, &init[2], 4, cudaMemcpyHostToDevice, ctx->stream), "set step") &&
         cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "profile setup");
    for (uint32_t r = 0; ok && r < reps; ++r) {
        e->pdl = false;
        e->prof_on = true;
        e->prof_marks.clear();
        const uint64_t delay_ns = 1000000ull + 8000ull * step_launches(e, pos + r);
        ok = cuda_ok(ctx, launch_delay(ctx->stream, delay_ns), "delay kernel") && cuda_ok(ctx, cudaEventRecord(first, ctx->stream), "profile event") &&
             enqueue_batch(e, 1, true, Tail::Greedy, long_ctx);
        e->pdl = pdl_was;
        e->prof_on = false;
        ok = ok && sync_and_check(ctx, "profile step");
        cudaEvent_t prev = first;
        for (auto &mk : e->prof_marks) {
            float ms = 0.0f;
            if (ok && !cuda_ok(ctx, cudaEventElapsedTime(&ms, prev, mk.second), "event time")) ok = false;
            if (ok) {
                auto it = acc.find(mk.first);
                if (it == acc.end()) { acc[mk.first] = {0.0, 0u}; order.push_back(mk.first); it = acc.find(mk.first); }
                it->second.first += ms * 1e3; it->second.second += 1;
                total += ms * 1e3;
            }
            prev = mk.second;
        }
        for (auto &mk : e->prof_marks) cudaEventDestroy(mk.second);
        e->prof_marks.clear();
    }
    e->pdl = pdl_was;
    e->prof_on = false;
    for (auto &mk : e->prof_marks) cudaEventDestroy(mk.second);
    e->prof_marks.clear();
    if (first) cudaEventDestroy(first);
    if (!ok) return -1;
    std::string out = "kernel class | launches per step | us per step | avg us | share\n";
    char line[256];
    for (const std::string &k : order) {
        const auto &v = acc[k];
        std::snprintf(line, sizeof line, "%s | %.1f | %.1f | %.2f | %.1f%%\n", k.c_str(), (double)v.second / reps, v.first / reps, v.first / v.second,
                      100.0 * v.first / std::max(total, 1e-9));
        out += line;
    }
    std::snprintf(line, sizeof line, "total | | %.1f | |\n", total / reps);
    out += line;
    const size_t n = std::min(out.size(), cap - 1);
    std::memcpy(table, out.data(), n);
    table[n] = 0;
    return (int64_t)out.size();
}

size_t kronos_cuda_engine_debug_words(KronosCudaEngine *e, uint64_t *out, size_t cap) {
    if (!e || !out) return 0;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!make_current(ctx)) return 0;
    unsigned long long buf[32];
    if (!cuda_ok(ctx, cudaMemcpyAsync(buf, e->d_dbg, sizeof buf, cudaMemcpyDeviceToHost, ctx->stream), "read debug words") ||
        !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "read debug words"))
        return 0;
    const size_t n = std::min<size_t>(32, cap);
    for (size_t i = 0; i < n; ++i) out[i] = buf[i];
    return n;
}

}  // extern "C"

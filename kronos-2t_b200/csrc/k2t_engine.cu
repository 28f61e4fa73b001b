// Whole-token engine behind the C ABI: counterpart of MetalLlamaEngine (src/backend/metal_gpu.rs:929-969,
// try_new 1196, forward_tokens 1619) for dense Llama/Qwen layers with bit-plane or NF projections and the
// int8 Hadamard KV cache.  One decode step = 10 kernels per layer + 3; the greedy loop and the token-id
// forward replay a captured CUDA graph (position, token and step counter live in device memory).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <new>
#include <vector>

#include "k2t_context.h"
#include "k2t_model_kernels.h"

using namespace k2t;

struct EngineLayer {
    float *input_norm = nullptr, *post_norm = nullptr, *qkv_bias = nullptr, *q_norm = nullptr, *k_norm = nullptr;
    KronosCudaMatrix *qkv = nullptr, *o = nullptr, *gate_up = nullptr, *down = nullptr;
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
    int32_t *act_m = nullptr;
    int8_t *k_q8 = nullptr, *v_q8 = nullptr;
    float *k_scale = nullptr, *v_scale = nullptr;
    uint32_t *d_token = nullptr, *d_pos = nullptr, *d_step = nullptr, *d_history = nullptr;
    uint32_t n_split = 32;
    size_t weight_bytes = 0;
    std::vector<void *> allocs;
    cudaGraphExec_t graph_greedy = nullptr, graph_ids = nullptr;
    cudaStream_t graph_stream = nullptr;      // the stream the graphs were captured on
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

bool gemv(KronosCudaEngine *e, const KronosCudaMatrix *m, float *out) {
    uint32_t launched = 0;
    cudaError_t err = launch_gemv(e->ctx->stream, m->dm, e->act_q, e->act_s, e->act_m, 1, out, m->dm.geom.rows, nullptr,
                                  e->ctx->sm_count, e->ctx->d_err, &launched);
    e->ctx->launches += launched;
    return cuda_ok(e->ctx, err, "engine gemv");
}

bool count(KronosCudaEngine *e, cudaError_t err, const char *what, uint32_t n = 1) {
    e->ctx->launches += n;
    return cuda_ok(e->ctx, err, what);
}

// Queues the kernels of one token on the context's stream.  `embed`: look d_token up first.
// `greedy`: finish with argmax (next token, history, step, position); otherwise only advance the position.
bool enqueue_step(KronosCudaEngine *e, bool embed, bool greedy) {
    const KronosCudaEngineConfig &c = e->cfg;
    cudaStream_t s = e->ctx->stream;
    const uint32_t h = c.hidden_size, hd = c.head_dim, q_dim = c.num_attention_heads * hd;
    if (embed) {
        const MatrixGeom &g = e->lm_head->dm.geom;
        EmbedArgs a{};
        for (int k = 0; k < 3; ++k) { a.plane[k] = e->lm_head->dm.d_base + g.plane_off[k]; a.pitch[k] = g.pitch[k]; a.cell[k] = g.cell[k]; }
        a.scales = reinterpret_cast<const uint16_t *>(e->lm_head->dm.d_base + g.scale_off);
        a.embed_bf16 = e->embed_bf16; a.token = e->d_token; a.hidden = e->hidden;
        a.fmt = g.fmt; a.nc = g.nc; a.nsg_pad = g.nsg_pad; a.sgc = g.sgc; a.max_odd = g.max_odd;
        a.sgc_shift = 32;
        for (uint32_t sh = 0; sh < 4; ++sh) if ((1u << sh) == g.sgc) a.sgc_shift = sh;
        for (int i = 0; i < 32; ++i) a.codebook[i] = g.codebook32[i];
        if (!count(e, launch_embed(s, a), "embed")) return false;
    }
    for (uint32_t l = 0; l < c.num_layers; ++l) {
        const EngineLayer &L = e->layers[l];
        if (!count(e, launch_rmsnorm_quant(s, e->hidden, l == 0 ? nullptr : e->proj, L.input_norm, h, c.rms_norm_eps, e->act_q, e->act_s, e->act_m), "rmsnorm")) return false;
        if (!gemv(e, L.qkv, e->qkv)) return false;
        QkvPostArgs qa{};
        qa.qkv = e->qkv; qa.bias = L.qkv_bias; qa.q_norm = L.q_norm; qa.k_norm = L.k_norm; qa.rope = e->rope; qa.pos = e->d_pos;
        qa.q_i8 = e->q_i8; qa.q_scale = e->q_scale; qa.k_q8 = e->k_q8; qa.v_q8 = e->v_q8; qa.k_scale = e->k_scale; qa.v_scale = e->v_scale;
        qa.n_q = c.num_attention_heads; qa.n_kv = c.num_key_value_heads; qa.head_dim = hd; qa.max_seq = c.max_seq_len; qa.layer = l;
        qa.eps = c.rms_norm_eps; qa.qk_norm_after_rope = c.qk_norm_after_rope;
        if (!count(e, launch_qkv_post(s, qa), "qkv_post")) return false;
        AttnArgs aa{};
        aa.q_i8 = e->q_i8; aa.q_scale = e->q_scale; aa.k_q8 = e->k_q8; aa.v_q8 = e->v_q8; aa.k_scale = e->k_scale; aa.v_scale = e->v_scale;
        aa.pos = e->d_pos; aa.part_m = e->part_m; aa.part_l = e->part_l; aa.part_o = e->part_o; aa.attn_out = l + 1 == c.num_layers ? e->attn_tap : nullptr;
        aa.out_q = e->act_q; aa.out_scales = e->act_s; aa.out_sums = e->act_m;
        aa.n_kv = c.num_key_value_heads; aa.group = c.num_attention_heads / c.num_key_value_heads; aa.head_dim = hd;
        aa.max_seq = c.max_seq_len; aa.layer = l; aa.n_split = e->n_split; aa.attn_scale = 1.0f / sqrtf((float)hd);
        if (!count(e, launch_attention(s, aa), "attention", 2)) return false;
        if (!gemv(e, L.o, e->proj)) return false;
        if (!count(e, launch_rmsnorm_quant(s, e->hidden, e->proj, L.post_norm, h, c.rms_norm_eps, e->act_q, e->act_s, e->act_m), "rmsnorm")) return false;
        if (!gemv(e, L.gate_up, e->gate_up)) return false;
        if (!count(e, launch_swiglu_quant(s, e->gate_up, c.intermediate_size, e->act_q, e->act_s, e->act_m, nullptr), "swiglu")) return false;
        if (!gemv(e, L.down, e->proj)) return false;
    }
    if (!count(e, launch_rmsnorm_quant(s, e->hidden, e->proj, e->final_norm, h, c.rms_norm_eps, e->act_q, e->act_s, e->act_m), "rmsnorm")) return false;
    if (!gemv(e, e->lm_head, e->logits)) return false;
    (void)q_dim;
    if (greedy) return count(e, launch_argmax_step(s, e->logits, c.vocab_size, e->d_token, e->d_pos, e->d_history, e->d_step), "argmax");
    return count(e, launch_advance_pos(s, e->d_pos), "advance");
}

bool set_u32(KronosCudaEngine *e, uint32_t *dst, uint32_t v) {
    return cuda_ok(e->ctx, cudaMemcpyAsync(dst, &v, 4, cudaMemcpyHostToDevice, e->ctx->stream), "set scalar") &&
           cuda_ok(e->ctx, cudaStreamSynchronize(e->ctx->stream), "set scalar sync");
}

// Captures one step into an executable graph (first use on the current stream).
bool ensure_graphs(KronosCudaEngine *e) {
    KronosCudaContext *ctx = e->ctx;
    if (e->graph_greedy && e->graph_stream == ctx->stream) return true;
    if (e->graph_greedy) { cudaGraphExecDestroy(e->graph_greedy); e->graph_greedy = nullptr; }
    if (e->graph_ids) { cudaGraphExecDestroy(e->graph_ids); e->graph_ids = nullptr; }
    // one eager step first (position 0, token 0; callers set both before every replay): loads every kernel
    // and sets its attributes outside a capture, where an error is also easier to attribute
    if (!set_u32(e, e->d_pos, 0) || !set_u32(e, e->d_token, 0) || !enqueue_step(e, true, true) ||
        !sync_and_check(ctx, "engine warm-up step"))
        return false;
    const uint64_t launches_before = ctx->launches;
    for (int which = 0; which < 2; ++which) {
        cudaGraph_t graph = nullptr;
        if (!cuda_ok(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal), "begin capture")) return false;
        const bool ok = enqueue_step(e, true, which == 0);
        cudaError_t err = cudaStreamEndCapture(ctx->stream, &graph);
        if (!ok || !cuda_ok(ctx, err, "end capture")) { if (graph) cudaGraphDestroy(graph); return false; }
        cudaGraphExec_t exec = nullptr;
        err = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (!cuda_ok(ctx, err, "graph instantiate")) return false;
        (which == 0 ? e->graph_greedy : e->graph_ids) = exec;
    }
    ctx->launches = launches_before;          // captured, not launched
    e->graph_stream = ctx->stream;
    return true;
}

uint32_t launches_per_step(const KronosCudaEngine *e) { return 1 + e->cfg.num_layers * 10 + 2 + 1; }

}  // namespace

extern "C" {

void kronos_cuda_engine_destroy(KronosCudaEngine *e) {
    if (!e) return;
    cudaSetDevice(e->ctx->device);
    cudaStreamSynchronize(e->ctx->stream);
    if (e->graph_greedy) cudaGraphExecDestroy(e->graph_greedy);
    if (e->graph_ids) cudaGraphExecDestroy(e->graph_ids);
    for (EngineLayer &L : e->layers)
        for (KronosCudaMatrix *m : {L.qkv, L.o, L.gate_up, L.down})
            if (m) kronos_cuda_matrix_free(e->ctx, m);
    if (e->lm_head) kronos_cuda_matrix_free(e->ctx, e->lm_head);
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
    if (n_layers != c.num_layers || c.num_layers == 0) { fail(ctx, "engine_create: n_layers does not match the config"); return nullptr; }
    if (c.head_dim != 64 && c.head_dim != 128) { fail(ctx, "engine_create: head_dim must be 64 or 128"); return nullptr; }
    if (c.hidden_size % 64 || c.intermediate_size % 64 || c.hidden_size == 0) { fail(ctx, "engine_create: hidden and intermediate sizes must be multiples of 64"); return nullptr; }
    if (c.num_key_value_heads == 0 || c.num_attention_heads % c.num_key_value_heads || c.num_attention_heads / c.num_key_value_heads > 8) {
        fail(ctx, "engine_create: query heads must be a multiple (at most 8x) of the kv heads"); return nullptr; }
    if (c.kv_bits != 8) { fail(ctx, "engine_create: only the int8 Hadamard KV cache (kv_bits = 8) is implemented"); return nullptr; }
    if (c.max_seq_len == 0) { fail(ctx, "engine_create: max_seq_len is 0"); return nullptr; }
    if (!make_current(ctx)) return nullptr;
    const uint32_t h = c.hidden_size, hd = c.head_dim, q_dim = c.num_attention_heads * hd, kv_dim = c.num_key_value_heads * hd;
    const uint32_t qkv_rows = q_dim + 2 * kv_dim, inter = c.intermediate_size;
    KronosCudaEngine *e = new (std::nothrow) KronosCudaEngine();
    if (!e) { fail(ctx, "engine_create: out of host memory"); return nullptr; }
    e->ctx = ctx; e->cfg = c;
    e->layers.resize(c.num_layers);
    auto bad = [&](const std::string &why) { std::string keep = why; kronos_cuda_engine_destroy(e); fail(ctx, keep); return (KronosCudaEngine *)nullptr; };
    auto shape_ok = [](const KronosCudaMatrixDesc &d, uint32_t rows, uint32_t cols) { return d.rows == rows && d.cols == cols; };
    for (uint32_t l = 0; l < c.num_layers; ++l) {
        const KronosCudaLayerDesc &d = layers[l];
        EngineLayer &L = e->layers[l];
        if (!d.input_norm || !d.post_attn_norm) return bad("engine_create: a layer has no norm weights");
        if (!shape_ok(d.qkv_proj, qkv_rows, h) || !shape_ok(d.o_proj, h, q_dim) || !shape_ok(d.gate_up_proj, 2 * inter, h) ||
            !shape_ok(d.down_proj, h, inter))
            return bad("engine_create: layer " + std::to_string(l) + " has a projection whose shape does not match the config");
        if (!dev_alloc(e, L.input_norm, h, d.input_norm) || !dev_alloc(e, L.post_norm, h, d.post_attn_norm)) return bad(ctx->err);
        if (d.qkv_bias && !dev_alloc(e, L.qkv_bias, qkv_rows, d.qkv_bias)) return bad(ctx->err);
        if (d.q_norm && !dev_alloc(e, L.q_norm, hd, d.q_norm)) return bad(ctx->err);
        if (d.k_norm && !dev_alloc(e, L.k_norm, hd, d.k_norm)) return bad(ctx->err);
        L.qkv = kronos_cuda_matrix_upload(ctx, &d.qkv_proj, 0);
        L.o = L.qkv ? kronos_cuda_matrix_upload(ctx, &d.o_proj, 0) : nullptr;
        L.gate_up = L.o ? kronos_cuda_matrix_upload(ctx, &d.gate_up_proj, 0) : nullptr;
        L.down = L.gate_up ? kronos_cuda_matrix_upload(ctx, &d.down_proj, 0) : nullptr;
        if (!L.down) return bad("engine_create: layer " + std::to_string(l) + ": " + ctx->err);
        for (KronosCudaMatrix *m : {L.qkv, L.o, L.gate_up, L.down}) {
            if (m->dm.geom.fmt == FMT_NF5 || m->dm.geom.fmt == FMT_E8Q2) return bad("engine_create: NF5 / E8Q2 projections are not implemented");
            e->weight_bytes += m->dm.geom.file_bytes;
        }
    }
    if (!shape_ok(*lm_head, c.vocab_size, h)) return bad("engine_create: lm_head shape does not match the config");
    e->lm_head = kronos_cuda_matrix_upload(ctx, lm_head, 0);
    if (!e->lm_head) return bad("engine_create: lm_head: " + ctx->err);
    if (e->lm_head->dm.geom.fmt == FMT_NF5 || e->lm_head->dm.geom.fmt == FMT_E8Q2) return bad("engine_create: NF5 / E8Q2 lm_head is not implemented");
    e->weight_bytes += e->lm_head->dm.geom.file_bytes;
    const size_t slots = (size_t)c.num_layers * c.num_key_value_heads * c.max_seq_len;
    const uint32_t act_n = std::max(std::max(h, q_dim), inter), n_q = c.num_attention_heads;
    bool ok = dev_alloc(e, e->final_norm, h, final_norm) && dev_alloc(e, e->rope, (size_t)c.max_seq_len * hd, rope) &&
              (embed_bf16 == nullptr || dev_alloc(e, e->embed_bf16, (size_t)c.vocab_size * h, embed_bf16)) &&
              dev_alloc(e, e->hidden, h) && dev_alloc(e, e->proj, h) && dev_alloc(e, e->qkv, qkv_rows) &&
              dev_alloc(e, e->gate_up, (size_t)2 * inter) && dev_alloc(e, e->logits, c.vocab_size) &&
              dev_alloc(e, e->act_q, act_n) && dev_alloc(e, e->act_s, act_n / 64) && dev_alloc(e, e->act_m, act_n / 64) &&
              dev_alloc(e, e->q_i8, q_dim) && dev_alloc(e, e->attn_tap, q_dim) && dev_alloc(e, e->q_scale, n_q) &&
              dev_alloc(e, e->part_m, (size_t)n_q * e->n_split) && dev_alloc(e, e->part_l, (size_t)n_q * e->n_split) &&
              dev_alloc(e, e->part_o, (size_t)n_q * e->n_split * hd) &&
              dev_alloc(e, e->k_q8, slots * hd) && dev_alloc(e, e->v_q8, slots * hd) &&
              dev_alloc(e, e->k_scale, slots) && dev_alloc(e, e->v_scale, slots) &&
              dev_alloc(e, e->d_token, 1) && dev_alloc(e, e->d_pos, 1) && dev_alloc(e, e->d_step, 1) &&
              dev_alloc(e, e->d_history, c.max_seq_len);
    if (!ok || !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "engine_create sync")) return bad(ctx->err);
    return e;
}

size_t kronos_cuda_engine_kv_bytes(const KronosCudaEngine *e, size_t positions) {
    if (!e) return 0;
    // int8 keys and values plus one fp32 scale each per (layer, kv head, position): the reference's
    // 2 * layers * n_kv * (head_dim + 4) bytes per position (real_llm.rs:10223)
    return positions * 2 * (size_t)e->cfg.num_layers * e->cfg.num_key_value_heads * (e->cfg.head_dim + 4);
}
size_t kronos_cuda_engine_weight_bytes(const KronosCudaEngine *e) { return e ? e->weight_bytes : 0; }

int32_t kronos_cuda_engine_read_hidden(KronosCudaEngine *e, float *hidden) {
    if (!e || !hidden) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!make_current(ctx)) return -1;
    // the final norm kernel has already folded the last down_proj into the residual stream
    if (!cuda_ok(ctx, cudaMemcpyAsync(hidden, e->hidden, (size_t)e->cfg.hidden_size * 4, cudaMemcpyDeviceToHost, ctx->stream), "read hidden") ||
        !sync_and_check(ctx, "read hidden"))
        return -1;
    return 0;
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

int32_t kronos_cuda_engine_read_kv(KronosCudaEngine *e, uint32_t layer, uint32_t kv_head, size_t position, int8_t *k_q8,
                                   float *k_scale, int8_t *v_q8, float *v_scale) {
    if (!e) return -1;
    KronosCudaContext *ctx = e->ctx;
    ctx->err.clear();
    if (!k_q8 || !k_scale || !v_q8 || !v_scale) return fail(ctx, "read_kv: NULL buffer"), -1;
    if (layer >= e->cfg.num_layers || kv_head >= e->cfg.num_key_value_heads || position >= e->cfg.max_seq_len)
        return fail(ctx, "read_kv: index out of range"), -1;
    if (!make_current(ctx)) return -1;
    const size_t slot = ((size_t)layer * e->cfg.num_key_value_heads + kv_head) * e->cfg.max_seq_len + position, hd = e->cfg.head_dim;
    cudaStream_t s = ctx->stream;
    if (!cuda_ok(ctx, cudaMemcpyAsync(k_q8, e->k_q8 + slot * hd, hd, cudaMemcpyDeviceToHost, s), "read_kv") ||
        !cuda_ok(ctx, cudaMemcpyAsync(v_q8, e->v_q8 + slot * hd, hd, cudaMemcpyDeviceToHost, s), "read_kv") ||
        !cuda_ok(ctx, cudaMemcpyAsync(k_scale, e->k_scale + slot, 4, cudaMemcpyDeviceToHost, s), "read_kv") ||
        !cuda_ok(ctx, cudaMemcpyAsync(v_scale, e->v_scale + slot, 4, cudaMemcpyDeviceToHost, s), "read_kv"))
        return -1;
    return sync_and_check(ctx, "read_kv") ? 0 : -1;
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
    if (tokens) {
        for (size_t t = 0; t < n_tok; ++t)
            if (tokens[t] >= e->cfg.vocab_size) return fail(ctx, "forward: token id out of range"), -1;
        if (!ensure_graphs(e)) return -1;
    }
    if (!set_u32(e, e->d_pos, (uint32_t)pos_start)) return -1;
    const size_t h = e->cfg.hidden_size, v = e->cfg.vocab_size;
    for (size_t t = 0; t < n_tok; ++t) {
        if (tokens) {
            if (!cuda_ok(ctx, cudaMemcpyAsync(e->d_token, tokens + t, 4, cudaMemcpyHostToDevice, ctx->stream), "copy token")) return -1;
            if (!cuda_ok(ctx, cudaGraphLaunch(e->graph_ids, ctx->stream), "graph launch")) return -1;
            ctx->launches += launches_per_step(e);
        } else {
            if (!cuda_ok(ctx, cudaMemcpyAsync(e->hidden, embeds + t * h, h * 4, cudaMemcpyHostToDevice, ctx->stream), "copy embedding")) return -1;
            if (!enqueue_step(e, false, false)) return -1;
        }
        float *dst = all_logits ? all_logits + t * v : (t + 1 == n_tok ? last_logits : nullptr);
        if (dst && !cuda_ok(ctx, cudaMemcpyAsync(dst, e->logits, v * 4, cudaMemcpyDeviceToHost, ctx->stream), "copy logits")) return -1;
        if (tokens && !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "forward sync")) return -1;   // the token word is reused
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
    if (first_token >= e->cfg.vocab_size) return fail(ctx, "decode_greedy: token id out of range"), -1;
    if (pos_start + n_steps > e->cfg.max_seq_len) return fail(ctx, "decode_greedy: sequence would exceed max_seq_len"), -1;
    if (n_steps == 0) return 0;
    if (!make_current(ctx) || !ensure_graphs(e)) return -1;
    const uint32_t init[3] = {first_token, (uint32_t)pos_start, 0u};
    if (!cuda_ok(ctx, cudaMemcpyAsync(e->d_token, &init[0], 4, cudaMemcpyHostToDevice, ctx->stream), "set token") ||
        !cuda_ok(ctx, cudaMemcpyAsync(e->d_pos, &init[1], 4, cudaMemcpyHostToDevice, ctx->stream), "set pos") ||
        !cuda_ok(ctx, cudaMemcpyAsync(e->d_step, &init[2], 4, cudaMemcpyHostToDevice, ctx->stream), "set step") ||
        !cuda_ok(ctx, cudaStreamSynchronize(ctx->stream), "decode_greedy setup"))
        return -1;
    for (size_t i = 0; i < n_steps; ++i) {
        if (!cuda_ok(ctx, cudaGraphLaunch(e->graph_greedy, ctx->stream), "graph launch")) return -1;
        ctx->launches += launches_per_step(e);
    }
    if (!cuda_ok(ctx, cudaMemcpyAsync(out_tokens, e->d_history, n_steps * 4, cudaMemcpyDeviceToHost, ctx->stream), "copy tokens")) return -1;
    if (last_logits && !cuda_ok(ctx, cudaMemcpyAsync(last_logits, e->logits, (size_t)e->cfg.vocab_size * 4, cudaMemcpyDeviceToHost, ctx->stream), "copy logits")) return -1;
    return sync_and_check(ctx, "decode_greedy") ? 0 : -1;
}

}  // extern "C"

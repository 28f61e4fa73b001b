// k2t_model.cpp — CPU restatement of the kronos-2t dense Llama/Qwen decode step.
// TEST INFRASTRUCTURE ONLY (see k2t_oracle.h).  PARITY UNPINNED: no reference binary exists to run.
//
// Follows RealLlamaEngine::forward_token, generic per-op path (src/model/real_llm.rs:6485-6790), for
// engines whose projections are bit-plane (Nibble4) or NF matrices and whose KV cache is the int8
// Hadamard cache.  Where aarch64 and portable code differ the aarch64 arithmetic is followed:
// polynomial exp (9430-9454) in SwiGLU and softmax bodies, fused multiply-adds where NEON uses them.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <memory>
#include <vector>

#include "k2t_oracle.h"

namespace {

inline float bits_f32(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }

// exp_f32_neon (real_llm.rs:9430-9454), one lane.
inline float exp_poly(float x_raw) {
    float x = std::fmin(std::fmax(x_raw, -87.33654f), 88.0f);
    float kf = std::nearbyintf(x * 1.44269504088896340736f);
    float r = std::fmaf(-kf, 1.4286068e-6f, std::fmaf(-kf, 0.69314575f, x));
    float y = std::fmaf(1.9875691e-4f, r, 1.3982e-3f);
    y = std::fmaf(y, r, 8.333452e-3f);
    y = std::fmaf(y, r, 4.1665796e-2f);
    y = std::fmaf(y, r, 1.6666666e-1f);
    y = std::fmaf(y, r, 0.5f);
    y = std::fmaf(y, r, 1.0f);
    y = std::fmaf(y, r, 1.0f);
    int32_t ki = (int32_t)kf;
    return y * bits_f32((uint32_t)(ki + 127) << 23);
}

struct Mat {
    uint32_t kind = 0, rows = 0, cols = 0, bits = 0, sgc = 1;
    int8_t codebook[16] = {0};
    std::vector<uint8_t> a, b;   // bipolar: Nibble4 pair/tail streams; NF: pair/tail streams
    // bipolar source kept for tied-embedding row dequantization
    void gemv(const int8_t *q, const float *xs, const int32_t *xsum, float *out, size_t threads) const {
        if (kind == 0)
            k2o_nibble4_gemv(a.data(), b.data(), rows, cols, bits, q, xs, xsum, 1, out, rows, nullptr, threads);
        else
            k2o_nf_gemv(a.data(), b.data(), codebook, rows, cols, bits, sgc, q, xs, 1, out, rows, nullptr, threads);
    }
    void dequant_row(size_t r, float *out) const {
        if (kind == 0) k2o_nibble4_dequant_row(a.data(), b.data(), rows, cols, bits, r, out);
        else k2o_nf_dequant_row(a.data(), b.data(), codebook, rows, cols, bits, sgc, r, out);
    }
};

bool load_mat(Mat &m, const K2oMatrixDesc *d) {
    if (!d) return false;
    m.kind = d->kind; m.rows = d->rows; m.cols = d->cols; m.bits = d->bits; m.sgc = d->scale_group_chunks ? d->scale_group_chunks : 1;
    std::memcpy(m.codebook, d->codebook, 16);
    if (d->kind == 0) {   // FusedBipolar -> Nibble4 (repack_sdot, real_llm.rs:3657-3702; no gate_up interleave: a row permutation)
        m.a.resize(std::max<size_t>(1, k2o_nibble4_pair_bytes(d->rows, d->cols, d->bits)));
        m.b.resize(std::max<size_t>(1, k2o_nibble4_tail_bytes(d->rows, d->cols, d->bits)));
        k2o_nibble4_from_bipolar(d->data0, reinterpret_cast<const uint16_t *>(d->data1), d->rows, d->cols, d->bits, 0,
                                 m.a.data(), m.b.data());
    } else if (d->kind == 2) {
        m.a.assign(d->data0, d->data0 + d->len0);
        m.b.assign(d->data1, d->data1 + d->len1);
        if (m.a.empty()) m.a.resize(1);
        if (m.b.empty()) m.b.resize(1);
    } else {
        return false;
    }
    return true;
}

struct Expert { Mat gu, dn; };
struct Moe {
    bool on = false;
    uint32_t n_experts = 0, top_k = 0, d_ff = 0;
    bool norm_topk = false;
    uint32_t scoring = 0;               // MoeRouterScoring tag: 0 softmax, 1 top-k softmax, 2 sigmoid (sparse_moe.rs:28-53)
    std::vector<float> router_w, router_bias;
    std::vector<Expert> experts;
    // shared expert (SharedMoeExpert, Nf backend, sparse_moe.rs:223-315): runs for every token, optional sigmoid gate
    bool has_shared = false;
    Mat sh_gu, sh_dn;
    std::vector<float> sh_gate;
    uint32_t ep_size = 1, ep_rank = 0;   // expert-parallel emulation: only experts e % ep_size == ep_rank contribute (tests)
    uint32_t last_k = 0;                 // routes of the last token (tests)
    uint32_t last_e[32] = {0};
    float last_w[32] = {0};
};
struct Layer {
    std::vector<float> input_norm, post_norm, qkv_bias, q_norm, k_norm;
    Mat qkv, o, gate_up, down;
    Moe moe;
};

}  // namespace

struct K2oModel {
    K2oConfig cfg;
    std::vector<float> rope;          // [max_seq][head_dim]: cos(hd/2), sin(hd/2)
    std::vector<Layer> layers;
    std::vector<float> final_norm;
    Mat lm_head;
    std::vector<uint16_t> embed_bf16; // empty = tied (row of lm_head, inverse rotated)
    Mat embed_nf;                     // untied table quantized to NF4 (embed_nf4, real_llm.rs:1553): its rows, inverse rotated
    bool has_embed_nf = false;
    // int8 Hadamard KV cache (QuantizedKvCache, real_llm.rs:1093-1412): [layer][kv head][pos][hd] + scale per (head,pos)
    std::vector<int8_t> k_q8, v_q8;
    std::vector<float> k_sc, v_sc;
    // NF4 Hadamard KV cache (kv_bits = 4): packed indices [..][hd / 2], bf16 scale per 64-value group [..][hd / 64]
    std::vector<uint8_t> k_q4, v_q4;
    std::vector<uint16_t> k_s16, v_s16;
    size_t pos = 0;
    // taps of the last forward (for tests)
    std::vector<float> tap_hidden;    // hidden state after every layer [layers][hidden]
    std::vector<float> tap_attn;      // attention output of the last layer, last token [n_q * head_dim]

    // sliding-window + sink ring (QuantizedKvCache::new_with_opts, real_llm.rs:1235-1257; zero = full causal context)
    size_t window = 0, sinks = 0, ring_len = 0;
    size_t cap = 0;                   // cache rows per (layer, kv head): max_seq, or sinks + ring_len

    // QuantKvRawPtrs::slot_of_pos (real_llm.rs:1116-1122)
    size_t slot_of_pos(size_t p) const { return (ring_len == 0 || p < sinks) ? p : sinks + ((p - sinks) % ring_len); }
    size_t kv_slot(size_t l, size_t h, size_t p) const { return (l * cfg.n_kv + h) * cap + slot_of_pos(p); }
    // active_kv_len / active_kv_pos (real_llm.rs:8597-8612)
    size_t active_len(size_t seq_len) const { return (window > 0 && seq_len > window) ? window : seq_len; }
    size_t active_pos(size_t idx, size_t seq_len) const {
        return (window > 0 && seq_len > window && idx >= sinks) ? (seq_len - (window - sinks)) + (idx - sinks) : idx;
    }
    void alloc_cache() {
        const size_t slots = (size_t)cfg.layers * cfg.n_kv * cap, hd = cfg.head_dim;
        k_q8.clear(); v_q8.clear(); k_sc.clear(); v_sc.clear(); k_q4.clear(); v_q4.clear(); k_s16.clear(); v_s16.clear();
        if (cfg.kv_bits == 8) {
            k_q8.assign(slots * hd, 0); v_q8.assign(slots * hd, 0); k_sc.assign(slots, 0.0f); v_sc.assign(slots, 0.0f);
        } else {
            k_q4.assign(slots * hd / 2, 0x88); v_q4.assign(slots * hd / 2, 0x88); k_s16.assign(slots * hd / 64, 0); v_s16.assign(slots * hd / 64, 0);
        }
    }
};

namespace {

void rms_norm(const float *x, const float *w, size_t n, float eps, float *out) {
    float inv = k2o_inv_rms(x, n, eps);
    for (size_t i = 0; i < n; ++i) out[i] = (x[i] * inv) * w[i];
}

void head_rms_norm(float *buf, size_t heads, size_t hd, const float *w, float eps) {   // apply_per_head_rms_norm 8167-8178
    const float inv_hd = 1.0f / (float)hd;
    for (size_t h = 0; h < heads; ++h) {
        float *v = buf + h * hd;
        float inv = 1.0f / std::sqrt(k2o_dot_f32(v, v, hd) * inv_hd + eps);
        for (size_t i = 0; i < hd; ++i) v[i] = (v[i] * inv) * w[i];
    }
}

void rope_heads(float *buf, size_t heads, size_t hd, const float *row) {    // apply_llama_rope_head64/128_neon 9287-9326
    const size_t half = hd / 2;
    for (size_t h = 0; h < heads; ++h) {
        float *v = buf + h * hd;
        for (size_t i = 0; i < half; ++i) {
            float x0 = v[i], x1 = v[half + i], c = row[i], s = row[half + i];
            float a = x0 * c, b = x1 * s, d = x1 * c, e = x0 * s;
            v[i] = a - b;
            v[half + i] = d + e;
        }
    }
}

// store_hadamard_q8_head{64,128}_raw (8303-8365): rotate with block index 0 (,1), one scale per head.
void quant_head(const float *src, size_t hd, int8_t *q, float *scale) {
    float rot[128];
    std::memcpy(rot, src, hd * sizeof(float));
    k2o_fwht64(rot, hd, 0);
    float mx = 0.0f;
    for (size_t i = 0; i < hd; ++i) mx = std::max(mx, std::fabs(rot[i]));
    if (mx <= 1.1920929e-07f) { std::memset(q, 0, hd); *scale = 0.0f; return; }
    float inv = 127.0f / mx;
    for (size_t i = 0; i < hd; ++i) q[i] = (int8_t)(int32_t)std::nearbyintf(rot[i] * inv);
    *scale = mx / 127.0f;
}

// causal_gqa_group_q8 (8471-8594) for one query head; aarch64 arithmetic.
void attend_head(const K2oModel &m, size_t l, size_t kvh, const float *q_head, size_t seq_len, float attn_scale,
                 std::vector<float> &sc, float *out) {
    const size_t hd = m.cfg.head_dim;
    int8_t qi[128];
    float qs;
    quant_head(q_head, hd, qi, &qs);
    const float qas = qs * attn_scale;
    const int8_t *K = m.k_q8.data() + m.kv_slot(l, kvh, 0) * hd;
    const int8_t *V = m.v_q8.data() + m.kv_slot(l, kvh, 0) * hd;
    const float *ks = m.k_sc.data() + m.kv_slot(l, kvh, 0);
    const float *vs = m.v_sc.data() + m.kv_slot(l, kvh, 0);
    sc.resize(seq_len);
    // scores: 256-position tiles; groups of 8 use dot*(ks*qas), the tile remainder (dot*ks)*qas (8992-9057)
    for (size_t t0 = 0; t0 < seq_len; t0 += 256) {
        size_t t1 = std::min(seq_len, t0 + 256), n8 = t0 + ((t1 - t0) / 8) * 8;
        for (size_t t = t0; t < t1; ++t) {
            int32_t dot = 0;
            for (size_t i = 0; i < hd; ++i) dot += (int32_t)qi[i] * (int32_t)K[t * hd + i];
            sc[t] = t < n8 ? (float)dot * (ks[t] * qas) : ((float)dot * ks[t]) * qas;
        }
    }
    float mx = -INFINITY;
    for (size_t t = 0; t < seq_len; ++t) mx = std::max(mx, sc[t]);
    // softmax_unnorm_neon (9603-9632): 4 lanes accumulate, pairwise horizontal add, libm exp for the tail.
    // The tail's f32::exp is the platform libm's expf in the reference; libms differ in the last bit on a small
    // fraction of inputs, so the correctly rounded value (double exp rounded to float) stands in for it here.
    float acc[4] = {0, 0, 0, 0};
    size_t t = 0;
    for (; t + 4 <= seq_len; t += 4)
        for (int j = 0; j < 4; ++j) { float e = exp_poly(sc[t + j] - mx); sc[t + j] = e; acc[j] += e; }
    float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    for (; t < seq_len; ++t) { float e = (float)std::exp((double)(sc[t] - mx)); sc[t] = e; sum += e; }
    const float inv = 1.0f / sum;
    float o[128] = {0};
    for (size_t tt = 0; tt < seq_len; ++tt) {      // attn_values_head*_q8_accum_neon (9121-9162)
        float w = (sc[tt] * inv) * vs[tt];
        if (w == 0.0f) continue;
        for (size_t i = 0; i < hd; ++i) o[i] = std::fmaf((float)V[tt * hd + i], w, o[i]);
    }
    k2o_ifwht64(o, hd, 0);
    std::memcpy(out, o, hd * sizeof(float));
}

const int8_t NF4_CB[16] = {-127, -96, -75, -58, -44, -31, -18, -6, 6, 18, 31, 44, 58, 75, 96, 127};   // simd_lut.rs:4343

// nf4_nearest_idx (8615-8644): nearest default centroid by magnitude thresholds, sign picks the half.
uint8_t nf4_nearest_idx(float y) {
    const float a = std::fabs(y);
    const int p = a < 37.5f ? (a < 12.0f ? 0 : a < 24.5f ? 1 : 2) : a < 85.5f ? (a < 51.0f ? 3 : a < 66.5f ? 4 : 5) : a < 111.5f ? 6 : 7;
    return (uint8_t)(y >= 0.0f ? 8 + p : 7 - p);
}

inline uint16_t bf16_rne(float v) {      // f32_to_bf16 (simd_lut.rs:1375-1382)
    uint32_t bits;
    std::memcpy(&bits, &v, 4);
    if ((bits & 0x7F800000u) == 0x7F800000u && (bits & 0x007FFFFFu) != 0) return (uint16_t)((bits >> 16) | 0x0040u);
    return (uint16_t)((bits + 0x00007FFFu + ((bits >> 16) & 1u)) >> 16);
}
inline float bf16_f32(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; std::memcpy(&f, &u, 4); return f; }

// store_hadamard_q4_head_raw (8646-8701): per 64-value group a least-squares scale over the first assignment,
// rounded to bf16, then the final assignment; byte i of half h packs columns 32h+i (low) and 32h+16+i (high).
void quant_head_q4(const float *src, size_t hd, uint8_t *q4, uint16_t *s16) {
    float rot[128];
    std::memcpy(rot, src, hd * sizeof(float));
    k2o_fwht64(rot, hd, 0);
    for (size_t g = 0; g < hd / 64; ++g) {
        const float *blk = rot + g * 64;
        float max_abs = 0.0f;
        for (size_t i = 0; i < 64; ++i) { float a = std::fabs(blk[i]); if (a > max_abs) max_abs = a; }
        if (max_abs < 1e-30f) { s16[g] = 0; std::memset(q4 + g * 32, 0x88, 32); continue; }
        const float inv0 = 127.0f / max_abs;
        float num = 0.0f, den = 0.0f;
        for (size_t i = 0; i < 64; ++i) {
            const float c = (float)NF4_CB[nf4_nearest_idx(blk[i] * inv0)];
            num += blk[i] * c;
            den += c * c;
        }
        const float refined = (den > 1e-12f && num > 0.0f) ? num / den : max_abs / 127.0f;
        const uint16_t sb = bf16_rne(refined);
        const float s_final = bf16_f32(sb);
        const float inv_final = s_final > 1e-30f ? 1.0f / s_final : 0.0f;
        s16[g] = sb;
        for (size_t h = 0; h < 2; ++h)
            for (size_t i = 0; i < 16; ++i) {
                const uint8_t lo = nf4_nearest_idx(blk[h * 32 + i] * inv_final), hi = nf4_nearest_idx(blk[h * 32 + 16 + i] * inv_final);
                q4[g * 32 + h * 16 + i] = (uint8_t)(lo | (hi << 4));
            }
    }
}

// causal_gqa_group_q4_or_window (8794-8988) with bits == 4, no window, for one query head; aarch64 arithmetic
// (integer dots, fma value accumulation, softmax_unnorm_neon).
void attend_head_q4(const K2oModel &m, size_t l, size_t kvh, const float *q_head, size_t seq_len, float attn_scale,
                    std::vector<float> &sc, float *out) {
    const size_t hd = m.cfg.head_dim, gph = hd / 64, half = hd / 2;
    int8_t qi[128];
    float qs;
    quant_head(q_head, hd, qi, &qs);
    const float q_s = qs * attn_scale;
    const size_t slot0 = m.kv_slot(l, kvh, 0);
    sc.resize(seq_len);
    for (size_t t = 0; t < seq_len; ++t) {
        float total = 0.0f;
        for (size_t g = 0; g < gph; ++g) {
            const float ks = bf16_f32(m.k_s16[(slot0 + t) * gph + g]);
            const uint8_t *kp = m.k_q4.data() + (slot0 + t) * half + g * 32;
            int32_t dot = 0;
            for (size_t h = 0; h < 2; ++h)
                for (size_t i = 0; i < 16; ++i) {
                    const uint8_t b = kp[h * 16 + i];
                    dot += (int32_t)NF4_CB[b & 15] * qi[g * 64 + h * 32 + i] + (int32_t)NF4_CB[b >> 4] * qi[g * 64 + h * 32 + 16 + i];
                }
            total += ((float)dot * ks) * q_s;
        }
        sc[t] = total;
    }
    float mx = -INFINITY;
    for (size_t t = 0; t < seq_len; ++t) mx = std::max(mx, sc[t]);
    float acc[4] = {0, 0, 0, 0};
    size_t t = 0;
    for (; t + 4 <= seq_len; t += 4)
        for (int j = 0; j < 4; ++j) { float e = exp_poly(sc[t + j] - mx); sc[t + j] = e; acc[j] += e; }
    float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    for (; t < seq_len; ++t) { float e = (float)std::exp((double)(sc[t] - mx)); sc[t] = e; sum += e; }
    const float inv = 1.0f / sum;
    float o[128] = {0};
    for (size_t tt = 0; tt < seq_len; ++tt) {
        const float p_norm = sc[tt] * inv;
        if (p_norm == 0.0f) continue;
        for (size_t g = 0; g < gph; ++g) {
            const float w = p_norm * bf16_f32(m.v_s16[(slot0 + tt) * gph + g]);
            if (w == 0.0f) continue;
            const uint8_t *vp = m.v_q4.data() + (slot0 + tt) * half + g * 32;
            for (size_t h = 0; h < 2; ++h)
                for (size_t i = 0; i < 16; ++i) {
                    const uint8_t b = vp[h * 16 + i];
                    float &lo = o[g * 64 + h * 32 + i], &hi = o[g * 64 + h * 32 + 16 + i];
                    lo = std::fmaf((float)NF4_CB[b & 15], w, lo);
                    hi = std::fmaf((float)NF4_CB[b >> 4], w, hi);
                }
        }
    }
    k2o_ifwht64(o, hd, 0);
    std::memcpy(out, o, hd * sizeof(float));
}

// causal_gqa_group_q4_or_window (8794-8988) with a sliding window configured, either cache format: the active positions
// are the sinks and the last window - sinks positions (all positions while the context is shorter than the window), rows
// come from their ring slots; scores add ((dot_g * ks) * q_s) per 64-value group for BOTH formats (the int8 cache uses the
// slot's one scale for every group), values accumulate one fma per element in active-index order.
void attend_head_window(const K2oModel &m, size_t l, size_t kvh, const float *q_head, size_t seq_len, float attn_scale,
                        std::vector<float> &sc, float *out) {
    const size_t hd = m.cfg.head_dim, gph = hd / 64, half = hd / 2, act = m.active_len(seq_len);
    const bool q4 = m.cfg.kv_bits == 4;
    int8_t qi[128];
    float qs;
    quant_head(q_head, hd, qi, &qs);
    const float q_s = qs * attn_scale;
    sc.resize(act);
    for (size_t idx = 0; idx < act; ++idx) {
        const size_t slot = m.kv_slot(l, kvh, m.active_pos(idx, seq_len));
        float total = 0.0f;
        for (size_t g = 0; g < gph; ++g) {
            int32_t dot = 0;
            float ks;
            if (q4) {
                ks = bf16_f32(m.k_s16[slot * gph + g]);
                const uint8_t *kp = m.k_q4.data() + slot * half + g * 32;
                for (size_t h = 0; h < 2; ++h)
                    for (size_t i = 0; i < 16; ++i) {
                        const uint8_t b = kp[h * 16 + i];
                        dot += (int32_t)NF4_CB[b & 15] * qi[g * 64 + h * 32 + i] + (int32_t)NF4_CB[b >> 4] * qi[g * 64 + h * 32 + 16 + i];
                    }
            } else {
                ks = m.k_sc[slot];
                const int8_t *kp = m.k_q8.data() + slot * hd + g * 64;
                for (size_t i = 0; i < 64; ++i) dot += (int32_t)kp[i] * (int32_t)qi[g * 64 + i];
            }
            total += ((float)dot * ks) * q_s;
        }
        sc[idx] = total;
    }
    float mx = -INFINITY;
    for (size_t t = 0; t < act; ++t) mx = std::max(mx, sc[t]);
    float acc[4] = {0, 0, 0, 0};
    size_t t = 0;
    for (; t + 4 <= act; t += 4)
        for (int j = 0; j < 4; ++j) { float e = exp_poly(sc[t + j] - mx); sc[t + j] = e; acc[j] += e; }
    float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    for (; t < act; ++t) { float e = (float)std::exp((double)(sc[t] - mx)); sc[t] = e; sum += e; }
    const float inv = 1.0f / sum;
    float o[128] = {0};
    for (size_t idx = 0; idx < act; ++idx) {
        const float p_norm = sc[idx] * inv;
        if (p_norm == 0.0f) continue;
        const size_t slot = m.kv_slot(l, kvh, m.active_pos(idx, seq_len));
        if (q4) {
            for (size_t g = 0; g < gph; ++g) {
                const float w = p_norm * bf16_f32(m.v_s16[slot * gph + g]);
                if (w == 0.0f) continue;
                const uint8_t *vp = m.v_q4.data() + slot * half + g * 32;
                for (size_t h = 0; h < 2; ++h)
                    for (size_t i = 0; i < 16; ++i) {
                        const uint8_t b = vp[h * 16 + i];
                        float &lo = o[g * 64 + h * 32 + i], &hi = o[g * 64 + h * 32 + 16 + i];
                        lo = std::fmaf((float)NF4_CB[b & 15], w, lo);
                        hi = std::fmaf((float)NF4_CB[b >> 4], w, hi);
                    }
            }
        } else {
            const float w = p_norm * m.v_sc[slot];
            if (w == 0.0f) continue;
            const int8_t *vp = m.v_q8.data() + slot * hd;
            for (size_t i = 0; i < hd; ++i) o[i] = std::fmaf((float)vp[i], w, o[i]);
        }
    }
    k2o_ifwht64(o, hd, 0);
    std::memcpy(out, o, hd * sizeof(float));
}

}  // namespace

// causal_gqa_attention_q8 (real_llm.rs:8951-8988) for a stand-alone cache: n_kv heads of `seq_len` cached positions,
// k_q8 / v_q8 [n_kv][seq_len][head_dim], scales [n_kv][seq_len]; q [n_q][head_dim] fp32 in, out [n_q][head_dim].  Lets the
// reference's own attention accuracy test run against this restatement without a model around it.
void k2o_attention_q8(size_t head_dim, size_t n_q, size_t n_kv, size_t seq_len, const int8_t *k_q8, const float *k_scale,
                      const int8_t *v_q8, const float *v_scale, const float *q, float attn_scale, float *out) {
    K2oModel m;
    m.cfg = K2oConfig{};
    m.cfg.head_dim = (uint32_t)head_dim; m.cfg.n_kv = (uint32_t)n_kv; m.cfg.n_q = (uint32_t)n_q; m.cfg.layers = 1; m.cfg.kv_bits = 8;
    m.cfg.max_seq = (uint32_t)seq_len;
    m.cap = seq_len;
    m.k_q8.assign(k_q8, k_q8 + n_kv * seq_len * head_dim);
    m.v_q8.assign(v_q8, v_q8 + n_kv * seq_len * head_dim);
    m.k_sc.assign(k_scale, k_scale + n_kv * seq_len);
    m.v_sc.assign(v_scale, v_scale + n_kv * seq_len);
    std::vector<float> sc;
    const size_t group = n_q / n_kv;
    for (size_t qh = 0; qh < n_q; ++qh) attend_head(m, 0, qh / group, q + qh * head_dim, seq_len, attn_scale, sc, out + qh * head_dim);
}

namespace {

// The platform expf of the reference's scalar paths, replaced by the correctly rounded value (see attend_head).
inline float exp_cr(float x) { return (float)std::exp((double)x); }

// select_topk_by_score (sparse_moe.rs:185-206): insertion with strict '>' (the earlier expert wins ties), descending.
void select_topk(const float *scores, size_t n, size_t k, uint32_t *ids, float *vals) {
    size_t len = 0;
    for (size_t e = 0; e < n; ++e) {
        const float sc = scores[e];
        if (len < k) {
            size_t pos = len;
            while (pos > 0 && sc > vals[pos - 1]) { ids[pos] = ids[pos - 1]; vals[pos] = vals[pos - 1]; --pos; }
            ids[pos] = (uint32_t)e; vals[pos] = sc; ++len;
        } else if (sc > vals[k - 1]) {
            size_t pos = k - 1;
            while (pos > 0 && sc > vals[pos - 1]) { ids[pos] = ids[pos - 1]; vals[pos] = vals[pos - 1]; --pos; }
            ids[pos] = (uint32_t)e; vals[pos] = sc;
        }
    }
}

struct Act {
    std::vector<int8_t> q;
    std::vector<float> s;
    std::vector<int32_t> m;
    // fwht64_signed_inplace + populate (exec_hidden_proj!, 6521-6562); chunk0 = global index of the first chunk
    void populate(const float *x, size_t cols, uint64_t chunk0 = 0) {
        q.resize(cols); s.resize(cols / 64); m.resize(cols / 64);
        k2o_act_populate_fwht(x, cols, nullptr, 1.0f, chunk0, q.data(), s.data(), m.data());
    }
};

// SparseMoeRuntime::forward_layer_single (sparse_moe.rs:961-1084), zero-copy NF experts, optional NF shared expert.
void moe_forward(Moe &M, const float *x_norm, size_t h, float *out, size_t threads) {
    const size_t E = M.n_experts, k = std::min<size_t>(std::min<size_t>(M.top_k, E), 32);
    std::vector<float> logits(E);
    for (size_t e = 0; e < E; ++e) {
        float v = k2o_dot_f32(M.router_w.data() + e * h, x_norm, h);      // dot_f32_moe_neon = the 16-lane fma order
        if (!M.router_bias.empty()) v += M.router_bias[e];
        logits[e] = v;
    }
    uint32_t ids[32];
    float w[32];
    if (M.scoring == 1) {                              // TopkSoftmax: top-k raw logits, then a k-way softmax
        select_topk(logits.data(), E, k, ids, w);
        float max_z = -INFINITY, sum = 0.0f;
        for (size_t i = 0; i < k; ++i) max_z = std::max(max_z, w[i]);
        for (size_t i = 0; i < k; ++i) { w[i] = exp_cr(w[i] - max_z); sum += w[i]; }
        const float inv = sum > 0.0f ? 1.0f / sum : 1.0f / (float)k;
        for (size_t i = 0; i < k; ++i) w[i] *= inv;
    } else {
        if (M.scoring == 2) {                          // Sigmoid
            for (size_t e = 0; e < E; ++e) logits[e] = 1.0f / (1.0f + exp_cr(-logits[e]));
        } else {                                       // Softmax over all experts
            float max_z = -INFINITY, sum = 0.0f;
            for (size_t e = 0; e < E; ++e) max_z = std::max(max_z, logits[e]);
            for (size_t e = 0; e < E; ++e) { logits[e] = exp_cr(logits[e] - max_z); sum += logits[e]; }
            const float inv_all = sum > 0.0f ? 1.0f / sum : 1.0f / (float)E;
            for (size_t e = 0; e < E; ++e) logits[e] *= inv_all;
        }
        select_topk(logits.data(), E, k, ids, w);
        if (M.norm_topk) {
            float top_sum = 0.0f;
            for (size_t i = 0; i < k; ++i) top_sum += w[i];
            if (top_sum > 0.0f) { const float inv_top = 1.0f / top_sum; for (size_t i = 0; i < k; ++i) w[i] *= inv_top; }
        }
    }
    for (size_t i = 1; i < k; ++i) {                  // insertion sort by ascending expert id
        const uint32_t ce = ids[i]; const float cw = w[i];
        size_t j = i;
        while (j > 0 && ids[j - 1] > ce) { ids[j] = ids[j - 1]; w[j] = w[j - 1]; --j; }
        ids[j] = ce; w[j] = cw;
    }
    M.last_k = (uint32_t)k;
    for (size_t i = 0; i < k; ++i) { M.last_e[i] = ids[i]; M.last_w[i] = w[i]; }
    Act act_in, act_mid;
    act_in.populate(x_norm, h);
    std::vector<float> gu(2 * (size_t)M.d_ff), sw(M.d_ff), eo(h);
    std::fill(out, out + h, 0.0f);
    if (M.has_shared && (M.ep_size <= 1 || M.ep_rank == 0)) {      // SharedMoeExpert::forward_single (254-314); under the expert-parallel emulation rank 0 holds it
        const size_t inter = M.sh_dn.cols;
        float scale = 1.0f;
        if (!M.sh_gate.empty()) scale = 1.0f / (1.0f + exp_cr(-k2o_dot_f32(M.sh_gate.data(), x_norm, h)));      // gate_scale (241-249)
        std::vector<float> sgu(2 * inter), ssw(inter);
        M.sh_gu.gemv(act_in.q.data(), act_in.s.data(), act_in.m.data(), sgu.data(), threads);
        for (size_t j = 0; j < inter; ++j) {
            const float g = sgu[j], u = sgu[inter + j];
            ssw[j] = (g / (1.0f + exp_cr(-g))) * u;
        }
        Act sh_mid;
        sh_mid.populate(ssw.data(), inter);
        M.sh_dn.gemv(sh_mid.q.data(), sh_mid.s.data(), sh_mid.m.data(), out, threads);
        if (std::fabs(scale - 1.0f) > 1.1920929e-07f)
            for (size_t j = 0; j < h; ++j) out[j] *= scale;
    }
    for (size_t i = 0; i < k; ++i) {
        if (M.ep_size > 1 && ids[i] % M.ep_size != M.ep_rank) continue;      // another rank's expert
        const Expert &X = M.experts[ids[i]];
        X.gu.gemv(act_in.q.data(), act_in.s.data(), act_in.m.data(), gu.data(), threads);
        for (size_t j = 0; j < M.d_ff; ++j) {          // moe_800b.rs:1498-1505: scalar libm exp, gate = rows [0, d_ff), up = the rest
            const float g = gu[j], u = gu[M.d_ff + j];
            sw[j] = (g / (1.0f + exp_cr(-g))) * u;
        }
        act_mid.populate(sw.data(), M.d_ff);
        X.dn.gemv(act_mid.q.data(), act_mid.s.data(), act_mid.m.data(), eo.data(), threads);
        for (size_t j = 0; j < h; ++j) out[j] += w[i] * eo[j];
    }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

extern "C" {

size_t k2o_nf_expert_layout(size_t d_model, size_t d_ff, size_t bits, size_t sgc, size_t *gu_pair_off, size_t *gu_pair_bytes,
                            size_t *dn_pair_off, size_t *dn_pair_bytes) {
    sgc = std::max<size_t>(sgc, 1);
    const size_t cb = k2o_nf_chunk_bytes(bits);
    const size_t gu_chunks = d_model / 64, gu_sg = (gu_chunks + sgc - 1) / sgc, gu_pairs = 2 * d_ff / 32;
    const size_t dn_chunks = d_ff / 64, dn_sg = (dn_chunks + sgc - 1) / sgc, dn_pairs = d_model / 32;
    const size_t gub = gu_pairs * (gu_sg * 64 + gu_chunks * 2 * cb), dnb = dn_pairs * (dn_sg * 64 + dn_chunks * 2 * cb);
    const size_t gu_off = 64, dn_off = align_up(gu_off + gub, 64);
    if (gu_pair_off) *gu_pair_off = gu_off;
    if (gu_pair_bytes) *gu_pair_bytes = gub;
    if (dn_pair_off) *dn_pair_off = dn_off;
    if (dn_pair_bytes) *dn_pair_bytes = dnb;
    return align_up(dn_off + dnb, 16384);             // K2TM_VM_PAGE_BYTES
}

int k2o_model_set_moe(K2oModel *m, uint32_t l, const float *router_w, const float *router_bias, uint32_t n_experts,
                      uint32_t top_k, int norm_topk, uint32_t d_ff, uint32_t bits, uint32_t sgc, const uint8_t *shard,
                      size_t expert_bytes) {
    if (!m || l >= m->layers.size() || !router_w || !shard || n_experts < 2 || top_k == 0 || d_ff % 64 || bits < 2 || bits > 5) return -1;
    const size_t h = m->cfg.hidden;
    if ((2 * (size_t)d_ff) % 32 || h % 32) return -1;
    size_t gu_off, gub, dn_off, dnb;
    if (k2o_nf_expert_layout(h, d_ff, bits, sgc, &gu_off, &gub, &dn_off, &dnb) != expert_bytes) return -1;
    Moe &M = m->layers[l].moe;
    M.on = true; M.n_experts = n_experts; M.top_k = top_k; M.d_ff = d_ff; M.norm_topk = (norm_topk & 1) != 0;
    M.scoring = (uint32_t)norm_topk >> 8;             // bits 8.. of the flag word carry the scoring tag
    M.router_w.assign(router_w, router_w + (size_t)n_experts * h);
    if (router_bias) M.router_bias.assign(router_bias, router_bias + n_experts); else M.router_bias.clear();
    M.experts.resize(n_experts);
    for (uint32_t e = 0; e < n_experts; ++e) {
        const uint8_t *rec = shard + (size_t)e * expert_bytes;
        K2oMatrixDesc d{};
        d.kind = 2; d.bits = bits; d.scale_group_chunks = sgc ? sgc : 1;
        d.rows = 2 * d_ff; d.cols = (uint32_t)h; std::memcpy(d.codebook, rec, 16);
        d.data0 = rec + gu_off; d.len0 = gub; d.data1 = nullptr; d.len1 = 0;
        if (!load_mat(M.experts[e].gu, &d)) return -1;
        d.rows = (uint32_t)h; d.cols = d_ff; std::memcpy(d.codebook, rec + 16, 16);
        d.data0 = rec + dn_off; d.len0 = dnb;
        if (!load_mat(M.experts[e].dn, &d)) return -1;
    }
    return 0;
}

int k2o_model_set_moe_shared(K2oModel *m, uint32_t l, const K2oMatrixDesc *gate_up, const K2oMatrixDesc *down, const float *gate_w) {
    if (!m || l >= m->layers.size() || !m->layers[l].moe.on || !gate_up || !down) return -1;
    Moe &M = m->layers[l].moe;
    if (!load_mat(M.sh_gu, gate_up) || !load_mat(M.sh_dn, down)) return -1;
    const size_t h = m->cfg.hidden;
    if (M.sh_gu.cols != h || M.sh_dn.rows != h || M.sh_gu.rows != 2 * M.sh_dn.cols) return -1;
    if (gate_w) M.sh_gate.assign(gate_w, gate_w + h); else M.sh_gate.clear();
    M.has_shared = true;
    return 0;
}

void k2o_model_set_ep(K2oModel *m, uint32_t ep_size, uint32_t ep_rank) {
    if (!m) return;
    for (Layer &L : m->layers) { L.moe.ep_size = ep_size ? ep_size : 1; L.moe.ep_rank = ep_rank; }
}

uint32_t k2o_model_last_routes(const K2oModel *m, uint32_t l, uint32_t *experts, float *weights) {
    if (!m || l >= m->layers.size() || !m->layers[l].moe.on) return 0;
    const Moe &M = m->layers[l].moe;
    for (uint32_t i = 0; i < M.last_k; ++i) { experts[i] = M.last_e[i]; weights[i] = M.last_w[i]; }
    return M.last_k;
}

K2oModel *k2o_model_new(const K2oConfig *cfg, const float *rope_table) {
    if (!cfg || !rope_table) return nullptr;
    if (cfg->head_dim != 64 && cfg->head_dim != 128) return nullptr;
    auto m = std::make_unique<K2oModel>();
    m->cfg = *cfg;
    m->rope.assign(rope_table, rope_table + (size_t)cfg->max_seq * cfg->head_dim);
    m->layers.resize(cfg->layers);
    if (m->cfg.kv_bits == 0) m->cfg.kv_bits = 8;
    if (m->cfg.kv_bits != 8 && m->cfg.kv_bits != 4) return nullptr;
    m->cap = cfg->max_seq;
    m->alloc_cache();
    return m.release();
}

// set_kv_sliding_window (real_llm.rs:1764-1790) + QuantizedKvCache::new_with_opts (1235-1257): a window is taken only when
// 8 <= window and window + 512 < max_seq; sinks are capped at window / 2; the ring keeps 512 rows of slack for batches.
int k2o_model_set_kv_window(K2oModel *m, uint32_t kv_bits, size_t window, size_t sinks) {
    if (!m || (kv_bits != 8 && kv_bits != 4)) return -1;
    m->cfg.kv_bits = kv_bits;
    if (window >= 8 && window + 512 < m->cfg.max_seq) {
        m->window = window;
        m->sinks = std::min(sinks, window / 2);
        m->ring_len = (window - m->sinks) + 512;
        m->cap = m->sinks + m->ring_len;
    } else {
        m->window = m->sinks = m->ring_len = 0;
        m->cap = m->cfg.max_seq;
    }
    m->alloc_cache();
    m->pos = 0;
    return m->window > 0 ? 1 : 0;
}
size_t k2o_model_kv_rows(const K2oModel *m) { return m ? m->cap : 0; }
// can_truncate_kv_to (real_llm.rs:1806-1821)
int k2o_model_can_truncate_kv_to(const K2oModel *m, size_t target_len) {
    if (!m || target_len >= m->pos) return 1;
    if (m->ring_len > 0) {
        const size_t live = m->window - m->sinks, slack = m->ring_len > live ? m->ring_len - live : 0;
        return (target_len <= m->sinks || (m->pos - target_len) <= slack) ? 1 : 0;
    }
    return 1;
}

void k2o_model_free(K2oModel *m) { delete m; }

int k2o_model_set_layer(K2oModel *m, uint32_t l, const float *input_norm, const float *post_norm, const float *qkv_bias,
                        const float *q_norm, const float *k_norm, const K2oMatrixDesc *qkv, const K2oMatrixDesc *o,
                        const K2oMatrixDesc *gate_up, const K2oMatrixDesc *down) {
    if (!m || l >= m->layers.size()) return -1;
    const K2oConfig &c = m->cfg;
    Layer &L = m->layers[l];
    L.input_norm.assign(input_norm, input_norm + c.hidden);
    L.post_norm.assign(post_norm, post_norm + c.hidden);
    size_t qkv_rows = (size_t)(c.n_q + 2 * c.n_kv) * c.head_dim;
    if (qkv_bias) L.qkv_bias.assign(qkv_bias, qkv_bias + qkv_rows); else L.qkv_bias.clear();
    if (q_norm) L.q_norm.assign(q_norm, q_norm + c.head_dim); else L.q_norm.clear();
    if (k_norm) L.k_norm.assign(k_norm, k_norm + c.head_dim); else L.k_norm.clear();
    if (!load_mat(L.qkv, qkv) || !load_mat(L.o, o)) return -1;
    if (L.qkv.rows != qkv_rows || L.qkv.cols != c.hidden || L.o.rows != c.hidden || L.o.cols != c.n_q * c.head_dim) return -1;
    if (!gate_up && !down) return 0;                    // a sparse-MoE layer: k2o_model_set_moe supplies the FFN
    if (!load_mat(L.gate_up, gate_up) || !load_mat(L.down, down)) return -1;
    if (L.gate_up.rows != 2 * c.inter || L.gate_up.cols != c.hidden || L.down.rows != c.hidden || L.down.cols != c.inter) return -1;
    return 0;
}

int k2o_model_set_head(K2oModel *m, const float *final_norm, const K2oMatrixDesc *lm_head, const uint16_t *embed_bf16) {
    if (!m || !final_norm || !load_mat(m->lm_head, lm_head)) return -1;
    m->final_norm.assign(final_norm, final_norm + m->cfg.hidden);
    if (embed_bf16) m->embed_bf16.assign(embed_bf16, embed_bf16 + (size_t)m->cfg.vocab * m->cfg.hidden);
    else m->embed_bf16.clear();
    return (m->lm_head.rows == m->cfg.vocab && m->lm_head.cols == m->cfg.hidden) ? 0 : -1;
}

void k2o_model_reset(K2oModel *m) { if (m) m->pos = 0; }
size_t k2o_model_pos(const K2oModel *m) { return m ? m->pos : 0; }
void k2o_model_set_pos(K2oModel *m, size_t pos) { if (m) m->pos = pos; }

// embed_token_into (real_llm.rs:8063-8097)
void k2o_model_embed(const K2oModel *m, uint32_t token, float *out) {
    const size_t h = m->cfg.hidden;
    if (!m->embed_bf16.empty()) {
        for (size_t i = 0; i < h; ++i) out[i] = k2o_bf16_to_f32(m->embed_bf16[(size_t)token * h + i]);
        return;
    }
    if (m->has_embed_nf) m->embed_nf.dequant_row(token, out);
    else m->lm_head.dequant_row(token, out);
    k2o_ifwht64(out, h, 0);
}

// the NF4-compressed untied table (compress_untied_embeddings_nf4, real_llm.rs:1825-1844): replaces the bf16 rows
int k2o_model_set_embedding_matrix(K2oModel *m, const K2oMatrixDesc *table) {
    if (!m || !table || !load_mat(m->embed_nf, table)) return -1;
    if (m->embed_nf.cols != m->cfg.hidden) return -1;
    m->has_embed_nf = true;
    m->embed_bf16.clear();
    return 0;
}

const float *k2o_model_tap_hidden(const K2oModel *m) { return m->tap_hidden.data(); }
const float *k2o_model_tap_attention(const K2oModel *m) { return m->tap_attn.data(); }
size_t k2o_model_kv_export(const K2oModel *m, size_t lo, size_t hi, uint8_t *out) {
    if (!m || lo > hi || hi > m->cfg.max_seq) return 0;
    const bool q4 = m->cfg.kv_bits == 4;
    const size_t hd = m->cfg.head_dim, heads = (size_t)m->cfg.layers * m->cfg.n_kv, db = q4 ? hd / 2 : hd, sb = q4 ? 2 * (hd / 64) : 4;
    const size_t total = (hi - lo) * 2 * heads * (db + sb);
    if (!out) return total;
    const uint8_t *kd = q4 ? m->k_q4.data() : reinterpret_cast<const uint8_t *>(m->k_q8.data());
    const uint8_t *vd = q4 ? m->v_q4.data() : reinterpret_cast<const uint8_t *>(m->v_q8.data());
    const uint8_t *ks = q4 ? reinterpret_cast<const uint8_t *>(m->k_s16.data()) : reinterpret_cast<const uint8_t *>(m->k_sc.data());
    const uint8_t *vs = q4 ? reinterpret_cast<const uint8_t *>(m->v_s16.data()) : reinterpret_cast<const uint8_t *>(m->v_sc.data());
    for (size_t p = lo; p < hi; ++p)
        for (size_t h = 0; h < heads; ++h) {
            const size_t slot = h * m->cap + m->slot_of_pos(p);
            std::memcpy(out, kd + slot * db, db); out += db;
            std::memcpy(out, ks + slot * sb, sb); out += sb;
            std::memcpy(out, vd + slot * db, db); out += db;
            std::memcpy(out, vs + slot * sb, sb); out += sb;
        }
    return total;
}

int k2o_model_kv_import(K2oModel *m, const uint8_t *data, size_t len, size_t n) {
    if (!m || !data || n > m->cfg.max_seq || len < k2o_model_kv_export(m, 0, n, nullptr)) return -1;
    const bool q4 = m->cfg.kv_bits == 4;
    const size_t hd = m->cfg.head_dim, heads = (size_t)m->cfg.layers * m->cfg.n_kv, db = q4 ? hd / 2 : hd, sb = q4 ? 2 * (hd / 64) : 4;
    uint8_t *kd = q4 ? m->k_q4.data() : reinterpret_cast<uint8_t *>(m->k_q8.data());
    uint8_t *vd = q4 ? m->v_q4.data() : reinterpret_cast<uint8_t *>(m->v_q8.data());
    uint8_t *ks = q4 ? reinterpret_cast<uint8_t *>(m->k_s16.data()) : reinterpret_cast<uint8_t *>(m->k_sc.data());
    uint8_t *vs = q4 ? reinterpret_cast<uint8_t *>(m->v_s16.data()) : reinterpret_cast<uint8_t *>(m->v_sc.data());
    for (size_t p = 0; p < n; ++p)
        for (size_t h = 0; h < heads; ++h) {
            const size_t slot = h * m->cap + m->slot_of_pos(p);
            std::memcpy(kd + slot * db, data, db); data += db;
            std::memcpy(ks + slot * sb, data, sb); data += sb;
            std::memcpy(vd + slot * db, data, db); data += db;
            std::memcpy(vs + slot * sb, data, sb); data += sb;
        }
    m->pos = n;
    return 0;
}

// KvPrefixSnapshot::Q8 / Q4 (save_kv_prefix / restore_kv_prefix_slice, real_llm.rs:5876-6155) as one blob: 32-byte header
// ("K2TKVPFX", kv_bits, slots_per_head, heads, head_dim, 0, 0) + key rows, value rows, key scales, value scales, head-major.
size_t k2o_model_save_kv_prefix(const K2oModel *m, size_t n, uint8_t *out) {
    if (!m) return 0;
    const size_t len = std::min(n, m->pos), slots = m->ring_len > 0 ? m->cap : len;
    const size_t heads = (size_t)m->cfg.layers * m->cfg.n_kv, hd = m->cfg.head_dim;
    const bool q4 = m->cfg.kv_bits == 4;
    const size_t db = q4 ? hd / 2 : hd, sb = q4 ? 2 * (hd / 64) : 4, total = 32 + 2 * heads * slots * (db + sb);
    if (!out) return total;
    std::memcpy(out, "K2TKVPFX", 8);
    const uint32_t hdr[6] = {m->cfg.kv_bits, (uint32_t)slots, (uint32_t)heads, (uint32_t)hd, 0u, 0u};
    std::memcpy(out + 8, hdr, 24);
    uint8_t *kd = out + 32, *vd = kd + heads * slots * db, *ks = vd + heads * slots * db, *vs = ks + heads * slots * sb;
    const uint8_t *K = q4 ? m->k_q4.data() : reinterpret_cast<const uint8_t *>(m->k_q8.data());
    const uint8_t *V = q4 ? m->v_q4.data() : reinterpret_cast<const uint8_t *>(m->v_q8.data());
    const uint8_t *KS = q4 ? reinterpret_cast<const uint8_t *>(m->k_s16.data()) : reinterpret_cast<const uint8_t *>(m->k_sc.data());
    const uint8_t *VS = q4 ? reinterpret_cast<const uint8_t *>(m->v_s16.data()) : reinterpret_cast<const uint8_t *>(m->v_sc.data());
    for (size_t h = 0; h < heads; ++h) {
        std::memcpy(kd + h * slots * db, K + h * m->cap * db, slots * db);
        std::memcpy(vd + h * slots * db, V + h * m->cap * db, slots * db);
        std::memcpy(ks + h * slots * sb, KS + h * m->cap * sb, slots * sb);
        std::memcpy(vs + h * slots * sb, VS + h * m->cap * sb, slots * sb);
    }
    return total;
}
int k2o_model_restore_kv_prefix(K2oModel *m, const uint8_t *data, size_t len, size_t copy_slots, size_t total_pos) {
    if (!m || !data || len < 32 || std::memcmp(data, "K2TKVPFX", 8) != 0) return -1;
    uint32_t hdr[6];
    std::memcpy(hdr, data + 8, 24);
    const size_t slots = hdr[1], heads = (size_t)m->cfg.layers * m->cfg.n_kv, hd = m->cfg.head_dim;
    const bool q4 = m->cfg.kv_bits == 4;
    const size_t db = q4 ? hd / 2 : hd, sb = q4 ? 2 * (hd / 64) : 4;
    if (hdr[0] != m->cfg.kv_bits || hdr[2] != heads || hdr[3] != hd || len < 32 + 2 * heads * slots * (db + sb)) return -1;
    const size_t cp = std::min(slots, copy_slots);
    if (cp > m->cap) return -1;
    const uint8_t *kd = data + 32, *vd = kd + heads * slots * db, *ks = vd + heads * slots * db, *vs = ks + heads * slots * sb;
    uint8_t *K = q4 ? m->k_q4.data() : reinterpret_cast<uint8_t *>(m->k_q8.data());
    uint8_t *V = q4 ? m->v_q4.data() : reinterpret_cast<uint8_t *>(m->v_q8.data());
    uint8_t *KS = q4 ? reinterpret_cast<uint8_t *>(m->k_s16.data()) : reinterpret_cast<uint8_t *>(m->k_sc.data());
    uint8_t *VS = q4 ? reinterpret_cast<uint8_t *>(m->v_s16.data()) : reinterpret_cast<uint8_t *>(m->v_sc.data());
    for (size_t h = 0; h < heads; ++h) {
        std::memcpy(K + h * m->cap * db, kd + h * slots * db, cp * db);
        std::memcpy(V + h * m->cap * db, vd + h * slots * db, cp * db);
        std::memcpy(KS + h * m->cap * sb, ks + h * slots * sb, cp * sb);
        std::memcpy(VS + h * m->cap * sb, vs + h * slots * sb, cp * sb);
    }
    m->pos = total_pos;
    return 0;
}

int k2o_model_read_kv_q4(const K2oModel *m, uint32_t layer, uint32_t kv_head, size_t pos, uint8_t *k_q4, uint16_t *k_s16,
                         uint8_t *v_q4, uint16_t *v_s16) {
    if (!m || m->cfg.kv_bits != 4 || layer >= m->cfg.layers || kv_head >= m->cfg.n_kv || pos >= m->cfg.max_seq) return -1;
    const size_t slot = m->kv_slot(layer, kv_head, pos), hd = m->cfg.head_dim;
    std::memcpy(k_q4, m->k_q4.data() + slot * hd / 2, hd / 2);
    std::memcpy(v_q4, m->v_q4.data() + slot * hd / 2, hd / 2);
    std::memcpy(k_s16, m->k_s16.data() + slot * (hd / 64), hd / 64 * 2);
    std::memcpy(v_s16, m->v_s16.data() + slot * (hd / 64), hd / 64 * 2);
    return 0;
}
void k2o_kv_quant_head_q4(const float *src, size_t head_dim, uint8_t *q4, uint16_t *s16) { quant_head_q4(src, head_dim, q4, s16); }
uint8_t k2o_nf4_nearest_idx(float y) { return nf4_nearest_idx(y); }

int k2o_model_read_kv(const K2oModel *m, uint32_t layer, uint32_t kv_head, size_t pos, int8_t *k_q8, float *k_scale,
                      int8_t *v_q8, float *v_scale) {
    if (!m || m->cfg.kv_bits != 8 || layer >= m->cfg.layers || kv_head >= m->cfg.n_kv || pos >= m->cfg.max_seq) return -1;
    const size_t slot = m->kv_slot(layer, kv_head, pos), hd = m->cfg.head_dim;
    std::memcpy(k_q8, m->k_q8.data() + slot * hd, hd);
    std::memcpy(v_q8, m->v_q8.data() + slot * hd, hd);
    *k_scale = m->k_sc[slot];
    *v_scale = m->v_sc[slot];
    return 0;
}

// One decode step from an embedding vector (what the device boundary receives); logits[vocab].
int k2o_model_attn_part(K2oModel *m, uint32_t l, const float *hidden, float *out, size_t threads) {
    if (!m || l >= m->layers.size() || m->pos >= m->cfg.max_seq) return -1;
    const K2oConfig &c = m->cfg;
    const size_t h = c.hidden, hd = c.head_dim, q_dim = (size_t)c.n_q * hd, kv_dim = (size_t)c.n_kv * hd;
    const size_t group = c.n_q / c.n_kv, pos = m->pos;
    const float attn_scale = 1.0f / std::sqrt((float)hd);
    const float *rope_row = m->rope.data() + pos * hd;
    Layer &L = m->layers[l];
    std::vector<float> norm(h), qkv(q_dim + 2 * kv_dim), attn(q_dim), sc;
    Act act;
    rms_norm(hidden, L.input_norm.data(), h, c.eps, norm.data());
    act.populate(norm.data(), h);
    L.qkv.gemv(act.q.data(), act.s.data(), act.m.data(), qkv.data(), threads);
    if (!L.qkv_bias.empty()) for (size_t i = 0; i < qkv.size(); ++i) qkv[i] = std::fmaf(L.qkv_bias[i], 1.0f, qkv[i]);
    float *q = qkv.data(), *k = q + q_dim, *v = k + kv_dim;
    // apply_qk_norm_rope (8139-8165)
    if (c.qk_norm_after_rope) { rope_heads(q, c.n_q, hd, rope_row); rope_heads(k, c.n_kv, hd, rope_row); }
    if (!L.q_norm.empty()) head_rms_norm(q, c.n_q, hd, L.q_norm.data(), c.eps);
    if (!L.k_norm.empty()) head_rms_norm(k, c.n_kv, hd, L.k_norm.data(), c.eps);
    if (!c.qk_norm_after_rope) { rope_heads(q, c.n_q, hd, rope_row); rope_heads(k, c.n_kv, hd, rope_row); }
    for (size_t kvh = 0; kvh < c.n_kv; ++kvh) {
        size_t slot = m->kv_slot(l, kvh, pos);
        if (c.kv_bits == 4) {
            quant_head_q4(k + kvh * hd, hd, m->k_q4.data() + slot * hd / 2, m->k_s16.data() + slot * (hd / 64));
            quant_head_q4(v + kvh * hd, hd, m->v_q4.data() + slot * hd / 2, m->v_s16.data() + slot * (hd / 64));
        } else {
            quant_head(k + kvh * hd, hd, m->k_q8.data() + slot * hd, &m->k_sc[slot]);
            quant_head(v + kvh * hd, hd, m->v_q8.data() + slot * hd, &m->v_sc[slot]);
        }
    }
    for (size_t qh = 0; qh < c.n_q; ++qh)
        (m->window > 0 ? attend_head_window : c.kv_bits == 4 ? attend_head_q4 : attend_head)(*m, l, qh / group, q + qh * hd, pos + 1, attn_scale, sc,
                                                                                           attn.data() + qh * hd);
    if (l + 1 == c.layers) m->tap_attn = attn;
    act.populate(attn.data(), q_dim, c.o_chunk0);
    L.o.gemv(act.q.data(), act.s.data(), act.m.data(), out, threads);
    return 0;
}

int k2o_model_ffn_part(K2oModel *m, uint32_t l, const float *hidden, float *out, size_t threads) {
    if (!m || l >= m->layers.size()) return -1;
    const K2oConfig &c = m->cfg;
    const size_t h = c.hidden, inter = c.inter;
    Layer &L = m->layers[l];
    std::vector<float> norm(h);
    rms_norm(hidden, L.post_norm.data(), h, c.eps, norm.data());
    if (L.moe.on) {                                     // real_llm.rs:6709-6714
        moe_forward(L.moe, norm.data(), h, out, threads);
        return 0;
    }
    Act act;
    std::vector<float> gu(2 * inter), sw(inter);
    act.populate(norm.data(), h);
    L.gate_up.gemv(act.q.data(), act.s.data(), act.m.data(), gu.data(), threads);
    for (size_t i = 0; i < inter; ++i) {               // swiglu_activate_neon (9811-9842): inter is a multiple of 8
        float g = gu[i], u = gu[inter + i];
        sw[i] = (g / (1.0f + exp_poly(-g))) * u;
    }
    act.populate(sw.data(), inter, c.down_chunk0);
    L.down.gemv(act.q.data(), act.s.data(), act.m.data(), out, threads);
    return 0;
}

int k2o_model_head_part(K2oModel *m, const float *hidden, float *logits, size_t threads) {
    if (!m) return -1;
    const size_t h = m->cfg.hidden;
    std::vector<float> norm(h);
    Act act;
    rms_norm(hidden, m->final_norm.data(), h, m->cfg.eps, norm.data());
    act.populate(norm.data(), h);
    m->lm_head.gemv(act.q.data(), act.s.data(), act.m.data(), logits, threads);
    return 0;
}

void k2o_model_advance(K2oModel *m) { if (m) m->pos += 1; }

int k2o_model_forward_embedding(K2oModel *m, const float *embedding, float *logits, size_t threads) {
    if (!m || m->pos >= m->cfg.max_seq) return -1;
    const size_t h = m->cfg.hidden;
    std::vector<float> hidden(embedding, embedding + h), proj(h);
    m->tap_hidden.assign((size_t)m->cfg.layers * h, 0.0f);
    for (uint32_t l = 0; l < m->cfg.layers; ++l) {
        if (k2o_model_attn_part(m, l, hidden.data(), proj.data(), threads) != 0) return -1;
        for (size_t i = 0; i < h; ++i) hidden[i] = std::fmaf(proj[i], 1.0f, hidden[i]);   // add_inplace = axpy(1.0)
        if (k2o_model_ffn_part(m, l, hidden.data(), proj.data(), threads) != 0) return -1;
        for (size_t i = 0; i < h; ++i) hidden[i] = std::fmaf(proj[i], 1.0f, hidden[i]);
        std::memcpy(m->tap_hidden.data() + (size_t)l * h, hidden.data(), h * sizeof(float));
    }
    if (k2o_model_head_part(m, hidden.data(), logits, threads) != 0) return -1;
    m->pos += 1;
    return 0;
}

int k2o_model_forward_token(K2oModel *m, uint32_t token, float *logits, size_t threads) {
    if (!m || token >= m->cfg.vocab) return -1;
    std::vector<float> e(m->cfg.hidden);
    k2o_model_embed(m, token, e.data());
    return k2o_model_forward_embedding(m, e.data(), logits, threads);
}

// argmax_scalar (9914-9924): first maximum.
uint32_t k2o_argmax(const float *v, size_t n) {
    size_t best = 0;
    float bv = -INFINITY;
    for (size_t i = 0; i < n; ++i) if (v[i] > bv) { bv = v[i]; best = i; }
    return (uint32_t)best;
}

// build_rope_table (9212-9236).
void k2o_build_rope_table(size_t max_seq, size_t head_dim, double theta, float *table) {
    const size_t half = head_dim / 2;
    std::vector<float> inv_freq(half);
    for (size_t i = 0; i < half; ++i) inv_freq[i] = (float)(1.0 / std::pow(theta, (double)(2 * i) / (double)head_dim));
    for (size_t p = 0; p < max_seq; ++p)
        for (size_t i = 0; i < half; ++i) {
            float ang = (float)p * inv_freq[i];
            table[p * head_dim + i] = std::cos(ang);
            table[p * head_dim + half + i] = std::sin(ang);
        }
}

// exposed pieces for kernel-level parity tests
float k2o_exp_poly(float x) { return exp_poly(x); }
void k2o_swiglu(const float *gate, const float *up, size_t n, float *out) {
    for (size_t i = 0; i < n; ++i) out[i] = (gate[i] / (1.0f + exp_poly(-gate[i]))) * up[i];
}
void k2o_rope_heads(float *buf, size_t heads, size_t head_dim, const float *rope_row) { rope_heads(buf, heads, head_dim, rope_row); }
void k2o_head_rms_norm(float *buf, size_t heads, size_t head_dim, const float *w, float eps) { head_rms_norm(buf, heads, head_dim, w, eps); }
void k2o_kv_quant_head(const float *src, size_t head_dim, int8_t *q, float *scale) { quant_head(src, head_dim, q, scale); }

}  // extern "C"

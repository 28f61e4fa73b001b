// .k2tb dense compiled-model container: reader and writer (reference: RealLlamaEngine::save_bipolar,
// src/model/real_llm.rs:3705-3895, and load_bipolar / CacheReader, 45-87, 3902-4186).  Little-endian.
//   magic (K2TBIPOLAR1 / K2TKRONOS2 / 3 / 4 / 6, 11 characters + '\n'; the version picks the optional fields)
//   6 x u64 mode words, u64 n_layers
//   per layer: f32s input_norm, f32s post_attn_norm, (v>=3) f32s qkv_bias, (v>=6) f32s q_norm, f32s k_norm,
//              matrices qkv, o, gate_up, down
//   f32s final_norm, matrix lm_head, f32s embed_f32, (v>=3) u16s embed_bf16, (v>=4) u64 flag [+ NF matrix]
//   f32s / u16s = u64 count + data.  Matrix (v>=2: leading u64 tag; v1: always bipolar):
//     tag 0 bipolar: rows, cols, planes, u64 len + interleaved bytes, u64 n + bf16 scales
//     tag 2 NF:      rows, cols, bits, scale_group_chunks, 16-byte codebook, u64 len + pair_stream, u64 len + tail_stream
//   Tags 1 (VQ2) and 3 (Q2c) are other weight formats of the reference and are rejected here.
// Host code only: the arrays are copied out of the file image into aligned storage owned by the handle, and the
// descriptors handed out point into that storage.
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "../../include/kronos_cuda_ffi.h"

namespace {

struct OwnedMatrix {
    KronosCudaMatrixDesc d{};
    std::vector<uint8_t> a, b;
    void fix() { d.data0 = a.empty() ? nullptr : a.data(); d.len0 = a.size(); d.data1 = b.empty() ? nullptr : b.data(); d.len1 = b.size(); }
};
struct OwnedLayer {
    std::vector<float> input_norm, post_norm, qkv_bias, q_norm, k_norm;
    OwnedMatrix qkv, o, gate_up, down;
};

struct Reader {
    const uint8_t *p;
    size_t n, pos = 0;
    std::string err;
    bool need(size_t k) { if (pos + k > n || pos + k < pos) { if (err.empty()) err = "file is truncated"; return false; } return true; }
    bool u64(uint64_t &v) { if (!need(8)) return false; std::memcpy(&v, p + pos, 8); pos += 8; return true; }
    template <typename T> bool arr(std::vector<T> &out, uint64_t max_count) {
        uint64_t c;
        if (!u64(c)) return false;
        if (c > max_count || !need((size_t)c * sizeof(T))) { if (err.empty()) err = "array length exceeds the file"; return false; }
        out.resize((size_t)c);
        if (c) std::memcpy(out.data(), p + pos, (size_t)c * sizeof(T));
        pos += (size_t)c * sizeof(T);
        return true;
    }
    bool matrix(OwnedMatrix &m, bool tagged) {
        uint64_t tag = 0, rows, cols, bits, sgc = 1;
        if (tagged && !u64(tag)) return false;
        if (tag != 0 && tag != 2) { err = tag == 1 ? "VQ2 matrices are not supported" : tag == 3 ? "Q2c matrices are not supported" : "unknown matrix tag"; return false; }
        if (!u64(rows) || !u64(cols) || !u64(bits)) return false;
        if (tag == 2 && !u64(sgc)) return false;
        if (rows == 0 || cols == 0 || rows > 0xFFFFFFFFull || cols > 0xFFFFFFFFull || bits > 64 || sgc > 64) { err = "implausible matrix header"; return false; }
        m.d.kind = tag == 0 ? KRONOS_CUDA_MATRIX_BIPOLAR : KRONOS_CUDA_MATRIX_NF;
        m.d.rows = (uint32_t)rows; m.d.cols = (uint32_t)cols; m.d.bits = (uint32_t)bits; m.d.scale_group_chunks = (uint32_t)sgc;
        if (tag == 2) { if (!need(16)) return false; std::memcpy(m.d.codebook, p + pos, 16); pos += 16; }
        if (!arr(m.a, n)) return false;
        if (tag == 0) {
            std::vector<uint16_t> sc;
            if (!arr(sc, n)) return false;
            m.b.resize(sc.size() * 2);
            if (!sc.empty()) std::memcpy(m.b.data(), sc.data(), m.b.size());
        } else if (!arr(m.b, n)) return false;
        m.fix();
        return true;
    }
};

}  // namespace

struct KronosCudaK2tb {
    int version = 0;
    uint64_t mode[6] = {0};
    std::vector<OwnedLayer> layers;
    std::vector<float> final_norm, embed_f32;
    std::vector<uint16_t> embed_bf16;
    OwnedMatrix lm_head, embed_nf4;
    bool has_embed_nf4 = false;
};

namespace {
thread_local std::string g_k2tb_error;

bool parse(const uint8_t *bytes, size_t n, KronosCudaK2tb &f, std::string &err) {
    static const struct { const char *magic; int version; } MAGICS[] = {
        {"K2TBIPOLAR1\n", 1}, {"K2TKRONOS2\n", 2}, {"K2TKRONOS3\n", 3}, {"K2TKRONOS4\n", 4}, {"K2TKRONOS6\n", 6}};
    size_t mlen = 0;
    for (const auto &m : MAGICS) {
        const size_t l = std::strlen(m.magic);
        if (n >= l && std::memcmp(bytes, m.magic, l) == 0) { f.version = m.version; mlen = l; }
    }
    if (!f.version) {
        err = (n >= 11 && std::memcmp(bytes, "K2TKRONOS5\n", 11) == 0) ? "a sparse-MoE core (K2TKRONOS5) is read by the MoE loader, not this one"
                                                                        : "not a .k2tb file (unknown magic)";
        return false;
    }
    Reader r{bytes, n, mlen, {}};
    uint64_t n_layers = 0;
    for (int i = 0; i < 6; ++i) if (!r.u64(f.mode[i])) { err = r.err; return false; }
    if (!r.u64(n_layers) || n_layers == 0 || n_layers > 4096) { err = r.err.empty() ? "implausible layer count" : r.err; return false; }
    f.layers.resize((size_t)n_layers);
    const bool tagged = f.version >= 2;
    for (OwnedLayer &L : f.layers) {
        bool ok = r.arr(L.input_norm, n) && r.arr(L.post_norm, n);
        if (ok && f.version >= 3) ok = r.arr(L.qkv_bias, n);
        if (ok && f.version >= 6) ok = r.arr(L.q_norm, n) && r.arr(L.k_norm, n);
        ok = ok && r.matrix(L.qkv, tagged) && r.matrix(L.o, tagged) && r.matrix(L.gate_up, tagged) && r.matrix(L.down, tagged);
        if (!ok) { err = r.err; return false; }
    }
    bool ok = r.arr(f.final_norm, n) && r.matrix(f.lm_head, tagged) && r.arr(f.embed_f32, n);
    if (ok && f.version >= 3) ok = r.arr(f.embed_bf16, n);
    if (ok && f.version >= 4) {
        uint64_t flag = 0;
        ok = r.u64(flag);
        if (ok && flag) { f.has_embed_nf4 = true; ok = r.matrix(f.embed_nf4, true); }
    }
    if (!ok) { err = r.err; return false; }
    if (r.pos != n) { err = "trailing bytes after the last field"; return false; }
    return true;
}

struct Writer {
    FILE *f;
    bool ok = true;
    void raw(const void *p, size_t n) { if (ok && n && std::fwrite(p, 1, n, f) != n) ok = false; }
    void u64(uint64_t v) { raw(&v, 8); }
    void f32s(const float *p, size_t n) { u64(p ? n : 0); if (p) raw(p, n * 4); }
    bool matrix(const KronosCudaMatrixDesc &d, bool tagged, std::string &err) {
        if (d.kind == KRONOS_CUDA_MATRIX_BIPOLAR) {
            if (tagged) u64(0);
            u64(d.rows); u64(d.cols); u64(d.bits);
            u64(d.len0); raw(d.data0, d.len0);
            u64(d.len1 / 2); raw(d.data1, d.len1);
        } else if (d.kind == KRONOS_CUDA_MATRIX_NF) {
            if (!tagged) { err = "an NF matrix needs a version 2+ container"; return false; }
            u64(2); u64(d.rows); u64(d.cols); u64(d.bits); u64(d.scale_group_chunks);
            raw(d.codebook, 16);
            u64(d.len0); raw(d.data0, d.len0);
            u64(d.len1); raw(d.data1, d.len1);
        } else { err = "unsupported matrix kind"; return false; }
        return true;
    }
};

}  // namespace

extern "C" {

const char *kronos_cuda_k2tb_last_error(void) { return g_k2tb_error.c_str(); }

KronosCudaK2tb *kronos_cuda_k2tb_open(const char *path) {
    g_k2tb_error.clear();
    if (!path) { g_k2tb_error = "k2tb_open: NULL path"; return nullptr; }
    FILE *fp = std::fopen(path, "rb");
    if (!fp) { g_k2tb_error = std::string("k2tb_open: cannot open ") + path; return nullptr; }
    std::vector<uint8_t> bytes;
    uint8_t buf[1 << 16];
    size_t got;
    while ((got = std::fread(buf, 1, sizeof buf, fp)) > 0) bytes.insert(bytes.end(), buf, buf + got);
    std::fclose(fp);
    std::unique_ptr<KronosCudaK2tb> f(new KronosCudaK2tb());
    std::string err;
    if (!parse(bytes.data(), bytes.size(), *f, err)) { g_k2tb_error = "k2tb_open: " + err; return nullptr; }
    return f.release();
}

void kronos_cuda_k2tb_close(KronosCudaK2tb *f) { delete f; }

int32_t kronos_cuda_k2tb_info(const KronosCudaK2tb *f, uint32_t *version, uint64_t mode_words[6], size_t *n_layers) {
    if (!f) return -1;
    if (version) *version = (uint32_t)f->version;
    if (mode_words) std::memcpy(mode_words, f->mode, sizeof f->mode);
    if (n_layers) *n_layers = f->layers.size();
    return 0;
}

int32_t kronos_cuda_k2tb_layer(const KronosCudaK2tb *f, size_t l, KronosCudaLayerDesc *out, size_t *qkv_bias_len) {
    if (!f || !out || l >= f->layers.size()) return -1;
    const OwnedLayer &L = f->layers[l];
    std::memset(out, 0, sizeof *out);
    out->input_norm = L.input_norm.data(); out->post_attn_norm = L.post_norm.data();
    out->qkv_bias = L.qkv_bias.empty() ? nullptr : L.qkv_bias.data();
    out->q_norm = L.q_norm.empty() ? nullptr : L.q_norm.data();
    out->k_norm = L.k_norm.empty() ? nullptr : L.k_norm.data();
    out->qkv_proj = L.qkv.d; out->o_proj = L.o.d; out->gate_up_proj = L.gate_up.d; out->down_proj = L.down.d;
    if (qkv_bias_len) *qkv_bias_len = L.qkv_bias.size();
    return 0;
}

int32_t kronos_cuda_k2tb_head(const KronosCudaK2tb *f, const float **final_norm, size_t *final_norm_len, KronosCudaMatrixDesc *lm_head,
                              const uint16_t **embed_bf16, size_t *embed_bf16_len, const float **embed_f32, size_t *embed_f32_len) {
    if (!f) return -1;
    if (final_norm) *final_norm = f->final_norm.data();
    if (final_norm_len) *final_norm_len = f->final_norm.size();
    if (lm_head) *lm_head = f->lm_head.d;
    if (embed_bf16) *embed_bf16 = f->embed_bf16.empty() ? nullptr : f->embed_bf16.data();
    if (embed_bf16_len) *embed_bf16_len = f->embed_bf16.size();
    if (embed_f32) *embed_f32 = f->embed_f32.empty() ? nullptr : f->embed_f32.data();
    if (embed_f32_len) *embed_f32_len = f->embed_f32.size();
    return 0;
}

int32_t kronos_cuda_k2tb_save(const char *path, const uint64_t mode_words[6], const KronosCudaLayerDesc *layers, size_t n_layers,
                              size_t hidden, size_t qkv_rows, size_t head_dim, const float *final_norm, const KronosCudaMatrixDesc *lm_head,
                              const uint16_t *embed_bf16, size_t embed_bf16_len) {
    g_k2tb_error.clear();
    if (!path || !mode_words || !layers || !n_layers || !final_norm || !lm_head) { g_k2tb_error = "k2tb_save: NULL argument"; return -1; }
    bool any_nf = lm_head->kind == KRONOS_CUDA_MATRIX_NF, any_bias = false, any_qk = false;
    for (size_t l = 0; l < n_layers; ++l) {
        const KronosCudaLayerDesc &d = layers[l];
        if (d.moe_router_w) { g_k2tb_error = "k2tb_save: sparse-MoE layers belong to the K2TKRONOS5 core format"; return -1; }
        for (const KronosCudaMatrixDesc *m : {&d.qkv_proj, &d.o_proj, &d.gate_up_proj, &d.down_proj}) any_nf |= m->kind == KRONOS_CUDA_MATRIX_NF;
        any_bias |= d.qkv_bias != nullptr;
        any_qk |= d.q_norm != nullptr || d.k_norm != nullptr;
    }
    // version choice of save_bipolar (real_llm.rs:3831-3846)
    const int version = any_qk ? 6 : (any_bias || embed_bf16_len) ? 3 : any_nf ? 2 : 1;
    FILE *fp = std::fopen(path, "wb");
    if (!fp) { g_k2tb_error = std::string("k2tb_save: cannot create ") + path; return -1; }
    Writer w{fp};
    const char *magic = version == 6 ? "K2TKRONOS6\n" : version == 3 ? "K2TKRONOS3\n" : version == 2 ? "K2TKRONOS2\n" : "K2TBIPOLAR1\n";
    w.raw(magic, std::strlen(magic));
    for (int i = 0; i < 6; ++i) w.u64(mode_words[i]);
    w.u64(n_layers);
    std::string err;
    bool ok = true;
    for (size_t l = 0; l < n_layers && ok; ++l) {
        const KronosCudaLayerDesc &d = layers[l];
        w.f32s(d.input_norm, hidden); w.f32s(d.post_attn_norm, hidden);
        if (version >= 3) w.f32s(d.qkv_bias, qkv_rows);
        if (version >= 6) { w.f32s(d.q_norm, head_dim); w.f32s(d.k_norm, head_dim); }
        for (const KronosCudaMatrixDesc *m : {&d.qkv_proj, &d.o_proj, &d.gate_up_proj, &d.down_proj}) ok = ok && w.matrix(*m, version >= 2, err);
    }
    if (ok) {
        w.f32s(final_norm, hidden);
        ok = w.matrix(*lm_head, version >= 2, err);
        w.f32s(nullptr, 0);                                      // embed_f32 (empty: tied or bf16 table)
        if (version >= 3) { w.u64(embed_bf16 ? embed_bf16_len : 0); if (embed_bf16) w.raw(embed_bf16, embed_bf16_len * 2); }
        if (version >= 4) w.u64(0);                              // no NF4-quantized embedding table
    }
    const bool closed = std::fclose(fp) == 0;
    if (!ok || !w.ok || !closed) { g_k2tb_error = "k2tb_save: " + (err.empty() ? std::string("write failed") : err); return -1; }
    return 0;
}

}  // extern "C"

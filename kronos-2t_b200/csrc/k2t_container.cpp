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
// Sparse-MoE models come as two files (RealLlamaEngine::load_moe_from_files, real_llm.rs:5166-5519):
//   the core, magic K2TKRONOS5: 6 x u64 mode words, u64 expert_bits, u64 expert_scale_group_chunks, u64 n_layers;
//     per layer: f32s input_norm, post_attn_norm, qkv_bias, o_bias, q_norm, k_norm (empty = absent), matrices qkv, o, u64 is_moe;
//       MoE layer: u64 moe_slot_idx, u64 experts, u64 hidden, f32s router weights, f32s router bias,
//                  u64 has_shared [+ u64 inter, f32s gate_weight, matrices gate_up, down],
//                  u64 has_lookahead [+ u64 future_layer, u64 d_model, u64 rank, f32s u, f32s v];
//       dense layer: matrices gate_up, down;
//     f32s final_norm, matrix lm_head, f32s embed_f32, u16s embed_bf16, u64 flag [+ NF matrix];
//   the expert shard (.k2tm, K2tmShardHeader, src/model/moe_800b.rs:790-854): a 16 KiB header page - magic
//     "K2TM800B_V1\0", at byte 16 seven u64: layers, experts per layer, d_model, d_ff, scale_group_chunks, aligned expert
//     bytes, bits - then layers x experts records of aligned_expert_bytes each (expert_byte_offset = 16384 + (layer *
//     experts + expert) * aligned bytes).  The shard is mapped read-only, not copied.
// Host code only: the arrays are copied out of the file image into aligned storage owned by the handle, and the
// descriptors handed out point into that storage.
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "../../include/kronos_cuda_ffi.h"

namespace {

struct OwnedMatrix {
    KronosCudaMatrixDesc d{};
    std::vector<uint8_t> a, b;
    void fix() { d.data0 = a.empty() ? nullptr : a.data(); d.len0 = a.size(); d.data1 = b.empty() ? nullptr : b.data(); d.len1 = b.size(); }
};
struct OwnedLayer {
    std::vector<float> input_norm, post_norm, qkv_bias, o_bias, q_norm, k_norm;
    OwnedMatrix qkv, o, gate_up, down;
    // sparse-MoE layer of a K2TKRONOS5 core
    bool moe = false, has_shared = false, has_lookahead = false;
    uint64_t moe_slot = 0, router_experts = 0, router_hidden = 0;
    std::vector<float> router_w, router_bias;
    std::vector<float> shared_gate_w;          // shared expert: its matrices are kept in gate_up / down
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
    uint64_t expert_bits = 0, expert_sgc = 0;      // K2TKRONOS5 only
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
        {"K2TBIPOLAR1\n", 1}, {"K2TKRONOS2\n", 2}, {"K2TKRONOS3\n", 3}, {"K2TKRONOS4\n", 4}, {"K2TKRONOS5\n", 5}, {"K2TKRONOS6\n", 6}};
    size_t mlen = 0;
    for (const auto &m : MAGICS) {
        const size_t l = std::strlen(m.magic);
        if (n >= l && std::memcmp(bytes, m.magic, l) == 0) { f.version = m.version; mlen = l; }
    }
    if (!f.version) { err = "not a .k2tb file (unknown magic)"; return false; }
    Reader r{bytes, n, mlen, {}};
    uint64_t n_layers = 0;
    for (int i = 0; i < 6; ++i) if (!r.u64(f.mode[i])) { err = r.err; return false; }
    if (f.version == 5) {          // sparse-MoE core: its own field order (load_moe_from_files, real_llm.rs:5166-5519)
        if (!r.u64(f.expert_bits) || !r.u64(f.expert_sgc) || !r.u64(n_layers) || n_layers == 0 || n_layers > 4096) {
            err = r.err.empty() ? "implausible layer count" : r.err;
            return false;
        }
        if (f.expert_sgc == 0) f.expert_sgc = 1;
        f.layers.resize((size_t)n_layers);
        for (OwnedLayer &L : f.layers) {
            uint64_t is_moe = 0;
            bool ok = r.arr(L.input_norm, n) && r.arr(L.post_norm, n) && r.arr(L.qkv_bias, n) && r.arr(L.o_bias, n) && r.arr(L.q_norm, n) && r.arr(L.k_norm, n) &&
                      r.matrix(L.qkv, true) && r.matrix(L.o, true) && r.u64(is_moe);
            if (ok && is_moe) {
                L.moe = true;
                uint64_t flag = 0;
                ok = r.u64(L.moe_slot) && r.u64(L.router_experts) && r.u64(L.router_hidden) && r.arr(L.router_w, n) && r.arr(L.router_bias, n) && r.u64(flag);
                if (ok && L.router_w.size() != L.router_experts * L.router_hidden) { r.err = "router weights do not match experts x hidden"; ok = false; }
                if (ok && flag) {          // shared expert: inter, optional gate weight, gate_up and down as NF matrices (5097-5114)
                    L.has_shared = true;
                    uint64_t inter;
                    ok = r.u64(inter) && r.arr(L.shared_gate_w, n) && r.matrix(L.gate_up, true) && r.matrix(L.down, true);
                    if (ok && (L.gate_up.d.kind != KRONOS_CUDA_MATRIX_NF || L.down.d.kind != KRONOS_CUDA_MATRIX_NF || L.down.d.cols != inter ||
                               L.gate_up.d.rows != 2 * inter)) { r.err = "the shared expert must be two NF matrices of its intermediate size"; ok = false; }
                }
                ok = ok && r.u64(flag);
                if (ok && flag) {          // lookahead projector (expert prefetch of the CPU pager): read past it
                    L.has_lookahead = true;
                    uint64_t a, b, c;
                    std::vector<float> u, v;
                    ok = r.u64(a) && r.u64(b) && r.u64(c) && r.arr(u, n) && r.arr(v, n);
                }
            } else if (ok) {
                ok = r.matrix(L.gate_up, true) && r.matrix(L.down, true);
            }
            if (!ok) { err = r.err; return false; }
        }
        uint64_t flag = 0;
        bool ok = r.arr(f.final_norm, n) && r.matrix(f.lm_head, true) && r.arr(f.embed_f32, n) && r.arr(f.embed_bf16, n) && r.u64(flag);
        if (ok && flag) { f.has_embed_nf4 = true; ok = r.matrix(f.embed_nf4, true); }
        if (!ok) { err = r.err; return false; }
        if (r.pos != n) { err = "trailing bytes after the last field"; return false; }
        return true;
    }
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
    if (!L.o_bias.empty()) { g_k2tb_error = "k2tb_layer: the layer carries an o_proj bias, which the device engine does not apply"; return -1; }
    if (L.moe) {
        // a shared expert rides in gate_up_proj / down_proj (filled above; rows = 0 without one)
        out->moe_shared_gate_w = L.has_shared && !L.shared_gate_w.empty() ? L.shared_gate_w.data() : nullptr;
        out->moe_router_w = L.router_w.data();
        out->moe_router_bias = L.router_bias.empty() ? nullptr : L.router_bias.data();
        // moe_shard / moe_shard_len come from the expert shard: kronos_cuda_k2tm_layer(shard, moe slot)
    }
    return 0;
}

int32_t kronos_cuda_k2tb_moe_info(const KronosCudaK2tb *f, uint64_t *expert_bits, uint64_t *expert_scale_group_chunks) {
    if (!f || f->version != 5) return -1;
    if (expert_bits) *expert_bits = f->expert_bits;
    if (expert_scale_group_chunks) *expert_scale_group_chunks = f->expert_sgc;
    return 0;
}

int32_t kronos_cuda_k2tb_moe_layer(const KronosCudaK2tb *f, size_t l, uint64_t *moe_slot_idx, uint64_t *experts, uint64_t *hidden) {
    if (!f || l >= f->layers.size()) return -1;
    const OwnedLayer &L = f->layers[l];
    if (!L.moe) return 0;
    if (moe_slot_idx) *moe_slot_idx = L.moe_slot;
    if (experts) *experts = L.router_experts;
    if (hidden) *hidden = L.router_hidden;
    return 1;
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

int32_t kronos_cuda_k2tb_embed_nf4(const KronosCudaK2tb *f, KronosCudaMatrixDesc *table) {
    if (!f) return -1;
    if (!f->has_embed_nf4) return 0;
    if (table) *table = f->embed_nf4.d;
    return 1;
}

struct KronosCudaK2tm {
    void *map = nullptr;
    size_t len = 0;
    uint64_t w[7] = {0};      // layers, experts per layer, d_model, d_ff, scale_group_chunks, aligned expert bytes, bits
};

KronosCudaK2tm *kronos_cuda_k2tm_open(const char *path) {
    g_k2tb_error.clear();
    if (!path) { g_k2tb_error = "k2tm_open: NULL path"; return nullptr; }
    const int fd = ::open(path, O_RDONLY);
    if (fd < 0) { g_k2tb_error = std::string("k2tm_open: cannot open ") + path; return nullptr; }
    struct stat st;
    if (::fstat(fd, &st) != 0 || st.st_size < 16384 || (st.st_size % 16384) != 0) {       // open_k2tm (sparse_moe.rs:685): whole 16 KiB pages
        ::close(fd);
        g_k2tb_error = "k2tm_open: the file is not a whole number of 16 KiB pages";
        return nullptr;
    }
    void *map = ::mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (map == MAP_FAILED) { g_k2tb_error = "k2tm_open: mmap failed"; return nullptr; }
    std::unique_ptr<KronosCudaK2tm> h(new KronosCudaK2tm());
    h->map = map; h->len = (size_t)st.st_size;
    const uint8_t *page = static_cast<const uint8_t *>(map);
    auto bad = [&](const char *why) { g_k2tb_error = std::string("k2tm_open: ") + why; ::munmap(map, (size_t)st.st_size); h->map = nullptr; return (KronosCudaK2tm *)nullptr; };
    if (std::memcmp(page, "K2TM800B_V1\0", 12) != 0) return bad("bad k2tm header magic");
    std::memcpy(h->w, page + 16, 56);
    const uint64_t L = h->w[0], E = h->w[1], rec = h->w[5];
    if (L == 0 || E == 0 || rec == 0 || rec % 16384 || L > 4096 || E > 65536) return bad("implausible shard header");
    if (16384 + L * E * rec != (uint64_t)st.st_size) return bad("file size does not match layers x experts x record bytes");
    return h.release();
}

void kronos_cuda_k2tm_close(KronosCudaK2tm *h) {
    if (!h) return;
    if (h->map) ::munmap(h->map, h->len);
    delete h;
}

int32_t kronos_cuda_k2tm_info(const KronosCudaK2tm *h, uint64_t words[7]) {
    if (!h || !words) return -1;
    std::memcpy(words, h->w, sizeof h->w);
    return 0;
}

int32_t kronos_cuda_k2tm_layer(const KronosCudaK2tm *h, size_t moe_slot_idx, const uint8_t **records, size_t *len) {
    if (!h || !records || !len || moe_slot_idx >= h->w[0]) return -1;
    *records = static_cast<const uint8_t *>(h->map) + 16384 + moe_slot_idx * h->w[1] * h->w[5];      // expert_byte_offset(slot, 0)
    *len = (size_t)(h->w[1] * h->w[5]);
    return 0;
}

int32_t kronos_cuda_k2tb_save(const char *path, const uint64_t mode_words[6], const KronosCudaLayerDesc *layers, size_t n_layers,
                              size_t hidden, size_t qkv_rows, size_t head_dim, const float *final_norm, const KronosCudaMatrixDesc *lm_head,
                              const uint16_t *embed_bf16, size_t embed_bf16_len, const KronosCudaMatrixDesc *embed_nf4) {
    g_k2tb_error.clear();
    if (embed_nf4 && (embed_nf4->kind != KRONOS_CUDA_MATRIX_NF || embed_nf4->bits != 4)) { g_k2tb_error = "k2tb_save: the embedding table must be an NF4 matrix"; return -1; }
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
    const int version = any_qk ? 6 : embed_nf4 ? 4 : (any_bias || embed_bf16_len) ? 3 : any_nf ? 2 : 1;
    FILE *fp = std::fopen(path, "wb");
    if (!fp) { g_k2tb_error = std::string("k2tb_save: cannot create ") + path; return -1; }
    Writer w{fp};
    const char *magic = version == 6 ? "K2TKRONOS6\n" : version == 4 ? "K2TKRONOS4\n" : version == 3 ? "K2TKRONOS3\n" : version == 2 ? "K2TKRONOS2\n" : "K2TBIPOLAR1\n";
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
        if (version >= 4) {                                      // the NF4-quantized untied embedding table, if any
            w.u64(embed_nf4 ? 1 : 0);
            if (embed_nf4) ok = ok && w.matrix(*embed_nf4, true, err);
        }
    }
    const bool closed = std::fclose(fp) == 0;
    if (!ok || !w.ok || !closed) { g_k2tb_error = "k2tb_save: " + (err.empty() ? std::string("write failed") : err); return -1; }
    return 0;
}

}  // extern "C"

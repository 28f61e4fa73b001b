// Host-side repack of reference-format matrices into the device cell-plane layout (k2t_layout.h).
// Input formats: FusedBipolarLutMatrix (src/kernels/simd_lut.rs:1761-1794) and NfSdotMatrix
// pair_stream / tail_stream (simd_lut.rs:4850-5023, E8Q2 5118-5226) exactly as stored in .k2tb/.k2tm.
#include "k2t_layout.h"

#include <algorithm>
#include <cstring>
#include <thread>

namespace k2t {
namespace {

constexpr uint32_t STRIPE = 16;

inline size_t nf_chunk_bytes(uint32_t bits) { return bits == 5 ? 640 : bits == 4 ? 512 : bits == 3 ? 384 : 256; }

// Reader of one matrix in the reference layouts: code / index / scale of (row, column).
struct FileView {
    const KronosCudaMatrixDesc &d;
    uint32_t nc, nsg, num_stripes, num_pairs;
    size_t cb, pair_tot;

    explicit FileView(const KronosCudaMatrixDesc &desc) : d(desc) {
        nc = d.cols / 64;
        num_stripes = (d.rows + STRIPE - 1) / STRIPE;
        num_pairs = num_stripes / 2;
        uint32_t sgc = d.kind == KRONOS_CUDA_MATRIX_NF ? d.scale_group_chunks : 1;
        nsg = (nc + sgc - 1) / sgc;
        cb = nf_chunk_bytes(d.bits);
        pair_tot = (size_t)nsg * 64 + (size_t)nc * 2 * cb;
    }

    // ---- bit-planes: data[((s*(cols/8) + o)*B + p)*16 + lane], bit k of the byte = column 8o+k
    uint32_t bp_code(uint32_t r, uint32_t col) const {
        size_t s = r / STRIPE, lane = r % STRIPE, o = col / 8, k = col % 8;
        const uint8_t *base = d.data0 + ((s * (d.cols / 8) + o) * d.bits) * STRIPE + lane;
        uint32_t u = 0;
        for (uint32_t p = 0; p < d.bits; ++p) u |= ((uint32_t)(base[p * STRIPE] >> k) & 1u) << p;
        return u;
    }
    uint16_t bp_scale(uint32_t r, uint32_t c) const {
        size_t i = (((size_t)(r / STRIPE) * nc + c) * STRIPE + r % STRIPE) * 2;
        return (uint16_t)(d.data1[i] | (d.data1[i + 1] << 8));
    }

    // ---- NF: (data, scales) of (stripe, chunk) inside pair_stream / tail_stream
    void nf_ptrs(uint32_t stripe, uint32_t c, const uint8_t *&data, const uint8_t *&sc) const {
        uint32_t sgc = d.scale_group_chunks, sg = c / sgc, sub_c = c % sgc, c_start = sg * sgc;
        if (stripe < num_pairs * 2) {
            uint32_t side = stripe & 1;
            const uint8_t *sgp = d.data0 + (size_t)(stripe / 2) * pair_tot + (size_t)sg * 64 + (size_t)c_start * 2 * cb;
            sc = sgp + side * 32;
            data = sgp + 64 + (size_t)sub_c * 2 * cb + side * cb;
        } else {
            const uint8_t *sgp = d.data1 + (size_t)sg * 32 + (size_t)c_start * cb;
            sc = sgp;
            data = sgp + 32 + (size_t)sub_c * cb;
        }
    }
    uint16_t nf_scale(uint32_t r, uint32_t c) const {
        const uint8_t *data, *sc;
        nf_ptrs(r / STRIPE, c, data, sc);
        uint32_t lane = r % STRIPE;
        return (uint16_t)(sc[lane * 2] | (sc[lane * 2 + 1] << 8));
    }
    // index of (lane, sub_col) in one chunk block, bits 3..5
    uint32_t nf_index(const uint8_t *blk, uint32_t lane, uint32_t sub_col) const {
        uint32_t g = lane / 4, j = lane % 4;
        if (d.bits == 3) {
            uint32_t kp = sub_col / 32, k32 = sub_col % 32, which = k32 / 4, t = k32 % 4, b = j * 4 + t;
            const uint8_t *p = blk + kp * 192 + g * 48;
            uint32_t v0 = p[b], v1 = p[16 + b], v2 = p[32 + b];
            switch (which) {
                case 0: return v0 & 7;
                case 1: return (v0 >> 3) & 7;
                case 2: return ((v0 >> 6) & 3) | (((v2 >> 6) & 1) << 2);
                case 3: return v1 & 7;
                case 4: return (v1 >> 3) & 7;
                case 5: return ((v1 >> 6) & 3) | (((v2 >> 7) & 1) << 2);
                case 6: return v2 & 7;
                default: return (v2 >> 3) & 7;
            }
        }
        uint32_t k = sub_col / 16, w = sub_col % 16, sub4 = w / 4, t = w % 4, b = j * 4 + t;
        uint32_t byte = blk[k * 128 + g * 32 + (sub4 / 2) * 16 + b];
        uint32_t idx = (sub4 & 1) ? (byte >> 4) : (byte & 0x0F);
        if (d.bits == 5) {
            uint32_t hb = blk[512 + g * 32 + (k / 2) * 16 + b];
            uint32_t sh = ((k & 1) == 0) ? 4 + sub4 : sub4;
            idx |= ((hb >> sh) & 1u) << 4;
        }
        return idx;
    }
    // E8Q2 (template, sign) bytes of 8-column block `eb8` (0..7) of a chunk
    void e8_codes(const uint8_t *blk, uint32_t lane, uint32_t eb8, uint8_t &tpl, uint8_t &sgn) const {
        uint32_t g = lane / 4, j = lane % 4, kp = eb8 / 4, eb = eb8 % 4;
        size_t off = kp * 128 + g * 32 + eb * 4 + j;
        tpl = blk[off];
        sgn = blk[off + 16];
    }
};

inline void put_u16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)(v & 0xFF); p[1] = (uint8_t)(v >> 8); }

}  // namespace

bool matrix_geometry(const KronosCudaMatrixDesc &d, MatrixGeom &g, std::string &err) {
    std::memset(&g, 0, sizeof g);
    if (d.rows == 0 || d.cols == 0 || d.cols % 64 != 0) { err = "matrix: cols must be a positive multiple of 64"; return false; }
    g.rows = d.rows; g.cols = d.cols; g.nc = d.cols / 64;
    const size_t ns = (d.rows + STRIPE - 1) / STRIPE;
    if (d.kind == KRONOS_CUDA_MATRIX_BIPOLAR) {
        if (d.bits < 4 || d.bits > 6) { err = "bipolar matrix: planes must be 4, 5 or 6"; return false; }
        g.fmt = (Format)(FMT_BP4 + (d.bits - 4));
        g.sgc = 1; g.nsg = g.nc; g.max_odd = (1 << d.bits) - 1;
        g.cell[0] = 16; g.cell[1] = 16; g.cell[2] = 8 * (d.bits - 4);
        size_t want0 = ns * (d.cols / 8) * d.bits * STRIPE, want1 = ns * g.nc * STRIPE * 2;
        if (d.len0 != want0 || d.len1 != want1 || !d.data0 || !d.data1) { err = "bipolar matrix: plane/scale byte counts do not match rows x cols"; return false; }
        g.file_bytes = want0 + want1;
    } else if (d.kind == KRONOS_CUDA_MATRIX_NF) {
        if (d.bits < 2 || d.bits > 5) { err = "NF matrix: bits must be 2..5"; return false; }
        if (d.scale_group_chunks < 1 || d.scale_group_chunks > 8) { err = "NF matrix: scale_group_chunks must be 1..8"; return false; }
        g.fmt = d.bits == 4 ? FMT_NF4 : d.bits == 3 ? FMT_NF3 : d.bits == 5 ? FMT_NF5 : FMT_E8Q2;
        g.sgc = d.scale_group_chunks; g.nsg = (g.nc + g.sgc - 1) / g.sgc; g.max_odd = 0;
        g.cell[0] = 16; g.cell[1] = d.bits >= 4 ? 16 : d.bits == 3 ? 8 : 0; g.cell[2] = d.bits == 5 ? 8 : 0;
        size_t cb = nf_chunk_bytes(d.bits);
        size_t want0 = (ns / 2) * ((size_t)g.nsg * 64 + (size_t)g.nc * 2 * cb);
        size_t want1 = (ns & 1) * ((size_t)g.nsg * 32 + (size_t)g.nc * cb);
        if (d.len0 != want0 || d.len1 != want1 || (want0 && !d.data0) || (want1 && !d.data1)) { err = "NF matrix: pair/tail stream byte counts do not match rows x cols"; return false; }
        if (d.bits == 5) {
            for (int m = 0; m < 16; ++m) { g.codebook32[15 - m] = (int8_t)(-d.codebook[m]); g.codebook32[16 + m] = d.codebook[m]; }
        } else if (d.bits == 3) {
            std::memcpy(g.codebook32, d.codebook, 16);
        } else if (d.bits == 4) {
            // rank of every centroid in ascending order (stable), sorted device codebook
            for (int i = 0; i < 16; ++i) {
                int rank = 0;
                for (int j = 0; j < 16; ++j)
                    if (d.codebook[j] < d.codebook[i] || (d.codebook[j] == d.codebook[i] && j < i)) ++rank;
                g.nf4_rank[i] = (uint8_t)rank;
                g.codebook32[rank] = d.codebook[i];
            }
            // two-table decode: value = hi[l] + off for ranks 8..15, = off - lo[l] for ranks 0..7, tables in 0..127
            int max_lo = g.codebook32[7], min_lo = g.codebook32[0], min_hi = g.codebook32[8], max_hi = g.codebook32[15];
            int off_min = std::max(max_lo, max_hi - 127), off_max = std::min(min_hi, min_lo + 127);
            if (off_min <= off_max) {
                int off = std::min(std::max(0, off_min), off_max);
                g.nf4_split_ok = 1;
                g.nf4_offset = off;
                for (int l = 0; l < 8; ++l) {
                    g.nf4_hi[l] = (uint8_t)(g.codebook32[8 + l] - off);
                    g.nf4_lo[l] = (uint8_t)(off - g.codebook32[l]);
                }
            }
        }
        g.file_bytes = want0 + want1 + 16;
    } else {
        err = "matrix: unsupported kind (only bipolar=0 and NF=2)";
        return false;
    }
    g.rows_pad = (g.rows + 3u) & ~3u;
    g.np = (g.nc + 31u) / 32u;
    size_t off = 0;
    for (int k = 0; k < 3; ++k) {
        g.plane_off[k] = off;
        off += (size_t)g.rows_pad * g.nc * g.cell[k];      // a multiple of 16: rows_pad is a multiple of 4, cells are 8 or 16 bytes
    }
    g.scale_off = off;
    off += (size_t)g.np * g.rows_pad * 64;
    g.image_total = off + 16;
    return true;
}

void repack_matrix(const KronosCudaMatrixDesc &d, const MatrixGeom &g, bool interleave, uint8_t *out,
                   unsigned threads) {
    std::memset(out, 0, g.image_bytes());
    const FileView fv(d);
    const uint32_t inter = d.rows / 2;
    // destination row -> source row (gate_up interleave puts gate block ic at rows [128ic, +64), up block at [128ic+64, +64))
    auto src_row = [&](uint32_t r) -> uint32_t {
        if (!interleave) return r;
        uint32_t blk = r / 128, w = r % 128;
        return w < 64 ? blk * 64 + w : inter + blk * 64 + (w - 64);
    };

    auto do_rows = [&](uint32_t r_lo, uint32_t r_hi) {
        for (uint32_t r_dst = r_lo; r_dst < r_hi; ++r_dst) {
            const uint32_t r = src_row(r_dst), lane = r % STRIPE;
            for (uint32_t c = 0; c < g.nc; ++c) {
                uint8_t *c0 = out + g.cell_off(0, r_dst, c);
                uint8_t *c1 = out + g.cell_off(1, r_dst, c);
                uint8_t *c2 = out + g.cell_off(2, r_dst, c);
                if (d.kind == KRONOS_CUDA_MATRIX_BIPOLAR) {
                    put_u16(out + g.scale_off_of(r_dst, c), fv.bp_scale(r, c));
                    for (uint32_t col = 0; col < 64; ++col) {
                        uint32_t u = fv.bp_code(r, c * 64 + col);
                        uint32_t k = col % 8, cc = col % 32;
                        uint8_t *half = col < 32 ? c0 : c1;
                        half[(cc / 8) * 4 + (k % 4)] |= (uint8_t)((u & 0x0F) << (k < 4 ? 0 : 4));
                        if (d.bits == 5) {
                            uint32_t bit = 8 * (col % 4) + cc / 4;
                            c2[(col / 32) * 4 + bit / 8] |= (uint8_t)(((u >> 4) & 1) << (bit % 8));
                        } else if (d.bits == 6) {
                            uint32_t bit = 8 * (col % 4) + 2 * ((col % 16) / 4);
                            c2[(col / 16) * 4 + bit / 8] |= (uint8_t)(((u >> 4) & 3) << (bit % 8));
                        }
                    }
                    continue;
                }
                const uint8_t *blk, *sc;
                fv.nf_ptrs(r / STRIPE, c, blk, sc);
                put_u16(out + g.scale_off_of(r_dst, c), fv.nf_scale(r, c));     // every chunk of a group writes the group's scale (a group may sit in two tiles)
                if (d.bits == 2) {
                    for (uint32_t eb8 = 0; eb8 < 8; ++eb8) {
                        uint8_t tpl, sgn;
                        fv.e8_codes(blk, lane, eb8, tpl, sgn);
                        c0[2 * eb8] = tpl;
                        c0[2 * eb8 + 1] = sgn;
                    }
                } else if (d.bits == 3) {
                    auto word_ptr = [&](uint32_t w) { return w < 4 ? c0 + w * 4 : c1 + (w - 4) * 4; };
                    for (uint32_t col = 0; col < 64; ++col) {
                        uint32_t idx = fv.nf_index(blk, lane, col);
                        if (col < 48) {
                            uint32_t nib = col % 8;
                            word_ptr(col / 8)[nib / 2] |= (uint8_t)(idx << (4 * (nib % 2)));
                        } else {
                            uint32_t t = col - 48, nib = t % 8;
                            for (uint32_t j = 0; j < 3; ++j)
                                word_ptr(3 * (t / 8) + j)[nib / 2] |= (uint8_t)(((idx >> j) & 1) << (4 * (nib % 2) + 3));
                        }
                    }
                } else {  // 4 or 5 bits
                    for (uint32_t col = 0; col < 64; ++col) {
                        uint32_t idx = fv.nf_index(blk, lane, col);
                        if (d.bits == 4) idx = g.nf4_rank[idx];
                        uint32_t nib = col % 8, cc = col % 32;
                        uint8_t *half = col < 32 ? c0 : c1;
                        half[(cc / 8) * 4 + nib / 2] |= (uint8_t)((idx & 0x0F) << (4 * (nib % 2)));
                        if (d.bits == 5) {
                            uint32_t bit = 8 * (col % 4) + cc / 4;
                            c2[(col / 32) * 4 + bit / 8] |= (uint8_t)(((idx >> 4) & 1) << (bit % 8));
                        }
                    }
                }
            }
        }
    };

    threads = std::max(1u, std::min(threads, d.rows));
    if (threads == 1 || (size_t)d.rows * d.cols < (1u << 20)) { do_rows(0, d.rows); return; }
    std::vector<std::thread> pool;
    uint32_t per = (d.rows + threads - 1) / threads;
    for (unsigned t = 0; t < threads; ++t) {
        uint32_t lo = t * per, hi = std::min(d.rows, lo + per);
        if (lo >= hi) break;
        pool.emplace_back(do_rows, lo, hi);
    }
    for (auto &th : pool) th.join();
}

}  // namespace k2t

// k2t_oracle.cpp — CPU restatement of the kronos-2t quantized kernels.
// TEST INFRASTRUCTURE ONLY (see k2t_oracle.h).  PARITY UNPINNED: no reference
// binary or golden vector exists to run against; fidelity rests on restating
// the cited reference lines and on the structural checks in tests/.
//
// Build with -ffp-contract=off: every fused multiply-add below is an explicit
// fmaf(), everything else rounds after each operation like the reference.
#include "k2t_oracle.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

namespace {

constexpr size_t STRIPE = 16;   // SIMD_ROW_STRIPE, simd_lut.rs:15
constexpr size_t BLK = 64;      // HADAMARD_BLOCK, hadamard.rs:14

inline float bits_f32(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }
inline uint32_t f32_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }

inline void masks64(uint64_t b, uint32_t *m) {
    // SplitMix64 stream seeded per block (hadamard.rs:29-44).
    uint64_t state = 0x9E3779B97F4A7C15ull + b * 0xBF58476D1CE4E5B9ull;
    for (int i = 0; i < 64; ++i) {
        state += 0x9E3779B97F4A7C15ull;
        uint64_t z = state;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        m[i] = (z & 1) ? 0x80000000u : 0u;
    }
}

inline void butterflies64(float *v) {
    // natural-order in-place Walsh-Hadamard, h = 1..32 (hadamard.rs:84-98).
    for (size_t h = 1; h < BLK; h <<= 1)
        for (size_t i = 0; i < BLK; i += 2 * h)
            for (size_t j = i; j < i + h; ++j) {
                float a = v[j], b = v[j + h];
                v[j] = a + b;
                v[j + h] = a - b;
            }
}

inline void fwht_block(float *v, uint64_t b) {
    uint32_t m[64];
    masks64(b, m);
    for (int i = 0; i < 64; ++i) v[i] = bits_f32(f32_bits(v[i]) ^ m[i]) * 0.125f;
    butterflies64(v);
}

inline void ifwht_block(float *v, uint64_t b) {
    uint32_t m[64];
    masks64(b, m);
    butterflies64(v);
    for (int i = 0; i < 64; ++i) v[i] = bits_f32(f32_bits(v[i] * 0.125f) ^ m[i]);
}

inline uint16_t to_bf16(float v) {
    uint32_t bits = f32_bits(v);
    if ((bits & 0x7F800000u) == 0x7F800000u && (bits & 0x007FFFFFu) != 0)
        return (uint16_t)((bits >> 16) | 0x0040u);
    uint32_t bias = 0x00007FFFu + ((bits >> 16) & 1u);
    return (uint16_t)((bits + bias) >> 16);
}
inline float from_bf16(uint16_t b) { return bits_f32((uint32_t)b << 16); }

// Quantize one already-rotated (or plain) 64-block: simd_lut.rs:3176-3195 / 3236-3254.
inline void quant_block(const float *blk, int8_t *q, float *scale, int32_t *sum) {
    float max_abs = 0.0f;
    for (int i = 0; i < 64; ++i) max_abs = std::max(max_abs, std::fabs(blk[i]));
    if (max_abs <= 1.1920929e-07f) {  // f32::EPSILON
        std::memset(q, 0, 64);
        *scale = 0.0f;
        *sum = 0;
        return;
    }
    float inv = 127.0f / max_abs;
    int32_t s = 0;
    for (int i = 0; i < 64; ++i) {
        int32_t qv = (int32_t)std::nearbyintf(blk[i] * inv);  // default rounding mode = ties-to-even
        s += qv;
        q[i] = (int8_t)qv;
    }
    *scale = max_abs / 127.0f;
    *sum = s;
}

template <class F>
void parallel_ranges(size_t n, size_t threads, F fn) {
    threads = std::max<size_t>(1, std::min(threads, n));
    if (threads == 1) { fn(0, n); return; }
    std::vector<std::thread> pool;
    size_t per = (n + threads - 1) / threads;
    for (size_t t = 0; t < threads; ++t) {
        size_t lo = t * per, hi = std::min(n, lo + per);
        if (lo >= hi) break;
        pool.emplace_back([=] { fn(lo, hi); });
    }
    for (auto &th : pool) th.join();
}

}  // namespace

extern "C" {

void k2o_rademacher_masks(uint64_t block_idx, uint32_t out[64]) { masks64(block_idx, out); }

void k2o_fwht64(float *data, size_t n, uint64_t block0) {
    for (size_t b = 0; b < n / BLK; ++b) fwht_block(data + b * BLK, block0 + b);
}
void k2o_ifwht64(float *data, size_t n, uint64_t block0) {
    for (size_t b = 0; b < n / BLK; ++b) ifwht_block(data + b * BLK, block0 + b);
}

uint16_t k2o_f32_to_bf16(float v) { return to_bf16(v); }
float k2o_bf16_to_f32(uint16_t b) { return from_bf16(b); }

void k2o_act_populate(const float *x, size_t cols, int8_t *q, float *scales, int32_t *sums) {
    for (size_t c = 0; c < cols / BLK; ++c) quant_block(x + c * BLK, q + c * BLK, scales + c, sums + c);
}

void k2o_act_populate_fwht(const float *x, size_t cols, const float *norm_w, float inv_rms,
                           uint64_t chunk0, int8_t *q, float *scales, int32_t *sums) {
    for (size_t c = 0; c < cols / BLK; ++c) {
        float blk[64];
        const float *xc = x + c * BLK;
        if (norm_w) {
            const float *wc = norm_w + c * BLK;
            for (int i = 0; i < 64; ++i) blk[i] = (xc[i] * inv_rms) * wc[i];  // two roundings, this order
        } else {
            std::memcpy(blk, xc, sizeof blk);
        }
        fwht_block(blk, chunk0 + c);
        quant_block(blk, q + c * BLK, scales + c, sums + c);
    }
}

float k2o_dot_f32(const float *a, const float *b, size_t n) {
    // Four 4-lane fma accumulators over 16-element strides, combined
    // (acc0+acc1)+(acc2+acc3) lane-wise, then a pairwise horizontal add; scalar tail.
    float acc[16] = {0};
    size_t i = 0;
    for (; i + 16 <= n; i += 16)
        for (int l = 0; l < 16; ++l) acc[l] = std::fmaf(a[i + l], b[i + l], acc[l]);
    float v[4];
    for (int l = 0; l < 4; ++l) v[l] = (acc[l] + acc[4 + l]) + (acc[8 + l] + acc[12 + l]);
    float sum = (v[0] + v[1]) + (v[2] + v[3]);
    for (; i < n; ++i) sum += a[i] * b[i];
    return sum;
}

float k2o_inv_rms(const float *x, size_t n, float eps) {
    float mean_sq = k2o_dot_f32(x, x, n) / (float)n;
    return 1.0f / std::sqrt(mean_sq + eps);
}

/* ======================= bipolar bit-planes ============================== */

size_t k2o_bipolar_data_bytes(size_t rows, size_t cols, size_t planes) {
    return ((rows + STRIPE - 1) / STRIPE) * (cols / 8) * planes * STRIPE;
}
size_t k2o_bipolar_scale_count(size_t rows, size_t cols) {
    return ((rows + STRIPE - 1) / STRIPE) * (cols / BLK) * STRIPE;
}

void k2o_bipolar_pack(const uint8_t *u, size_t rows, size_t cols, size_t planes, uint8_t *data) {
    size_t opr = cols / 8;
    std::memset(data, 0, k2o_bipolar_data_bytes(rows, cols, planes));
    for (size_t r = 0; r < rows; ++r) {
        size_t s = r / STRIPE, lane = r % STRIPE;
        for (size_t o = 0; o < opr; ++o) {
            const uint8_t *oct = u + r * cols + o * 8;
            size_t base = (s * opr + o) * planes * STRIPE + lane;
            for (size_t p = 0; p < planes; ++p) {
                uint8_t byte = 0;
                for (int k = 0; k < 8; ++k) byte |= (uint8_t)(((oct[k] >> p) & 1) << k);
                data[base + p * STRIPE] = byte;
            }
        }
    }
}

void k2o_bipolar_unpack_row(const uint8_t *data, size_t rows, size_t cols, size_t planes, size_t r,
                            uint8_t *codes) {
    (void)rows;
    size_t opr = cols / 8, s = r / STRIPE, lane = r % STRIPE;
    for (size_t o = 0; o < opr; ++o) {
        size_t base = (s * opr + o) * planes * STRIPE + lane;
        uint8_t *dst = codes + o * 8;
        std::memset(dst, 0, 8);
        for (size_t p = 0; p < planes; ++p) {
            uint8_t byte = data[base + p * STRIPE];
            for (int k = 0; k < 8; ++k) dst[k] |= (uint8_t)(((byte >> k) & 1) << p);
        }
    }
}

void k2o_bipolar_dequant_row(const uint8_t *data, const uint16_t *sc, size_t rows, size_t cols,
                             size_t planes, size_t r, float *out) {
    std::vector<uint8_t> codes(cols);
    k2o_bipolar_unpack_row(data, rows, cols, planes, r, codes.data());
    int max_odd = (1 << planes) - 1;
    size_t nc = cols / BLK;
    size_t sc_base = (r / STRIPE) * nc * STRIPE + r % STRIPE;
    for (size_t c = 0; c < nc; ++c) {
        float delta = from_bf16(sc[sc_base + c * STRIPE]);
        for (size_t i = 0; i < BLK; ++i)
            out[c * BLK + i] = (float)(2 * (int)codes[c * BLK + i] - max_odd) * delta;
    }
}

void k2o_bipolar_quantize_rtn(const float *weights, size_t rows, size_t cols, size_t planes,
                              size_t threads, uint8_t *interleaved, uint16_t *scales) {
    // quantize_stripe_batch_bipolar with u_slice = None (compiler.rs:1000-1076):
    // per row: rotate; per 64-chunk: 12-ratio grid search of a bf16 step size.
    static const float ratios[12] = {0.62f, 0.67f, 0.72f, 0.77f, 0.82f, 0.87f,
                                     0.92f, 0.97f, 1.02f, 1.07f, 1.12f, 1.18f};
    const int max_odd = (1 << planes) - 1;
    const float max_u_f = (float)max_odd, half_off = 0.5f * max_u_f;
    const size_t nc = cols / BLK;
    std::vector<uint8_t> flat(rows * cols, 0);
    std::fill(scales, scales + k2o_bipolar_scale_count(rows, cols), (uint16_t)0);
    parallel_ranges(rows, threads, [&](size_t lo, size_t hi) {
        std::vector<float> work(cols);
        for (size_t r = lo; r < hi; ++r) {
            std::memcpy(work.data(), weights + r * cols, cols * sizeof(float));
            k2o_fwht64(work.data(), cols, 0);
            for (size_t c = 0; c < nc; ++c) {
                const float *sub = work.data() + c * BLK;
                float max_abs = 0.0f;
                for (size_t i = 0; i < BLK; ++i) max_abs = std::max(max_abs, std::fabs(sub[i]));
                uint8_t best_u[64] = {0};
                uint16_t best_bf16 = 0;
                if (max_abs > 1e-12f) {
                    float best_loss = INFINITY;
                    for (float rat : ratios) {
                        uint16_t d_bf16 = to_bf16((max_abs * rat) / max_u_f);
                        float delta = from_bf16(d_bf16);
                        if (!(delta > 0.0f)) continue;
                        float inv_2delta = 0.5f / delta;
                        uint8_t cand[64];
                        float loss = 0.0f;
                        for (size_t j = 0; j < BLK; ++j) {
                            float wj = sub[j];
                            float t = std::roundf(wj * inv_2delta + half_off);  // half away from zero
                            t = std::min(std::max(t, 0.0f), max_u_f);
                            int u_idx = (int)t;
                            cand[j] = (uint8_t)u_idx;
                            float diff = wj - (float)(2 * u_idx - max_odd) * delta;
                            loss += diff * diff;
                        }
                        if (loss < best_loss) {
                            best_loss = loss;
                            best_bf16 = d_bf16;
                            std::memcpy(best_u, cand, 64);
                        }
                    }
                    scales[((r / STRIPE) * nc + c) * STRIPE + r % STRIPE] = best_bf16;
                    std::memcpy(flat.data() + r * cols + c * BLK, best_u, 64);
                }
                // max_abs <= 1e-12: the reference leaves codes 0 and scale 0 for the chunk.
            }
        }
    });
    k2o_bipolar_pack(flat.data(), rows, cols, planes, interleaved);
}

static inline size_t n4_pair_rec(size_t hp) { return 1024 + 256 * hp + 64; }
static inline size_t n4_tail_rec(size_t hp) { return 512 + 128 * hp + 32; }

size_t k2o_nibble4_pair_bytes(size_t rows, size_t cols, size_t planes) {
    size_t ns = (rows + STRIPE - 1) / STRIPE;
    return (ns / 2) * (cols / BLK) * n4_pair_rec(planes - 4);
}
size_t k2o_nibble4_tail_bytes(size_t rows, size_t cols, size_t planes) {
    size_t ns = (rows + STRIPE - 1) / STRIPE;
    return (ns & 1) * (cols / BLK) * n4_tail_rec(planes - 4);
}

void k2o_nibble4_from_bipolar(const uint8_t *data, const uint16_t *sc, size_t rows, size_t cols,
                              size_t planes, int interleave_gate_up, uint8_t *pair_stream,
                              uint8_t *tail_stream) {
    const size_t hp = planes - 4, nc = cols / BLK;
    const size_t ns = (rows + STRIPE - 1) / STRIPE, num_pairs = ns / 2;
    const size_t p_rec = n4_pair_rec(hp), t_rec = n4_tail_rec(hp);
    std::memset(pair_stream, 0, k2o_nibble4_pair_bytes(rows, cols, planes));
    if (ns & 1) std::memset(tail_stream, 0, k2o_nibble4_tail_bytes(rows, cols, planes));
    const size_t inter = rows / 2;
    std::vector<uint8_t> codes(cols);
    for (size_t orig_r = 0; orig_r < rows; ++orig_r) {
        k2o_bipolar_unpack_row(data, rows, cols, planes, orig_r, codes.data());
        size_t r = orig_r;
        if (interleave_gate_up) {  // [gate;up] -> 64-row [gate_64(ic), up_64(ic)] blocks (3315-3327)
            if (orig_r < inter) r = (orig_r / 64) * 128 + orig_r % 64;
            else { size_t ur = orig_r - inter; r = (ur / 64) * 128 + 64 + ur % 64; }
        }
        size_t orig_stripe = orig_r / STRIPE, orig_lane = orig_r % STRIPE;
        size_t stripe = r / STRIPE, lane = r % STRIPE, g = lane / 4, j = lane % 4;
        bool in_pair = stripe < num_pairs * 2;
        size_t p = stripe / 2, side = stripe & 1;
        for (size_t c = 0; c < nc; ++c) {
            uint16_t s16 = sc[(orig_stripe * nc + c) * STRIPE + orig_lane];
            uint8_t *rec;
            size_t data_off, hi_off, sc_off;
            if (in_pair) {
                rec = pair_stream + (p * nc + c) * p_rec;
                data_off = side * 512; hi_off = 1024 + side * 128 * hp; sc_off = 1024 + 256 * hp + side * 32;
            } else {
                rec = tail_stream + c * t_rec;
                data_off = 0; hi_off = 512; sc_off = 512 + 128 * hp;
            }
            rec[sc_off + lane * 2] = (uint8_t)(s16 & 0xFF);
            rec[sc_off + lane * 2 + 1] = (uint8_t)(s16 >> 8);
            for (size_t sub_col = 0; sub_col < 64; ++sub_col) {
                uint8_t u = codes[c * BLK + sub_col];
                size_t k = sub_col / 16, w = sub_col % 16, half = w / 8, sub = w / 4, t = w % 4;
                size_t byte = data_off + k * 128 + g * 32 + half * 16 + j * 4 + t;
                uint8_t lo = u & 0x0F;
                rec[byte] |= ((w % 8) < 4) ? lo : (uint8_t)(lo << 4);
                if (hp == 1) {
                    size_t hb = hi_off + (k / 2) * 64 + g * 16 + j * 4 + t;
                    size_t bit = ((k & 1) == 0) ? 4 + sub : sub;
                    rec[hb] |= (uint8_t)(((u >> 4) & 1) << bit);
                } else if (hp == 2) {
                    static const int sh[4] = {4, 6, 2, 0};
                    size_t hb = hi_off + k * 64 + g * 16 + j * 4 + t;
                    rec[hb] |= (uint8_t)(((u >> 4) & 3) << sh[sub]);
                }
            }
        }
    }
}

// (data, hi planes, scales) of (stripe, chunk): stripe_chunk_ptrs, simd_lut.rs:3413-3438.
static inline void n4_ptrs(const uint8_t *pair_stream, const uint8_t *tail_stream, size_t num_pairs,
                           size_t nc, size_t hp, size_t stripe, size_t c, const uint8_t **d,
                           const uint8_t **h, const uint8_t **s) {
    if (stripe < num_pairs * 2) {
        const uint8_t *base = pair_stream + ((stripe / 2) * nc + c) * n4_pair_rec(hp);
        size_t side = stripe & 1;
        *d = base + side * 512; *h = base + 1024 + side * 128 * hp; *s = base + 1024 + 256 * hp + side * 32;
    } else {
        const uint8_t *base = tail_stream + c * n4_tail_rec(hp);
        *d = base; *h = base + 512; *s = base + 512 + 128 * hp;
    }
}

// Code of (lane, sub_col) inside one (stripe, chunk) record.
static inline int n4_code(const uint8_t *d, const uint8_t *h, size_t hp, size_t lane, size_t sub_col) {
    size_t g = lane / 4, j = lane % 4;
    size_t k = sub_col / 16, w = sub_col % 16, sub = w / 4, t = w % 4;
    uint8_t byte = d[k * 128 + g * 32 + (w / 8) * 16 + j * 4 + t];
    int u = ((w % 8) < 4) ? (byte & 0x0F) : (byte >> 4);
    if (hp == 1) {
        uint8_t hb = h[(k / 2) * 64 + g * 16 + j * 4 + t];
        size_t bit = ((k & 1) == 0) ? 4 + sub : sub;
        u |= ((hb >> bit) & 1) << 4;
    } else if (hp == 2) {
        static const int sh[4] = {4, 6, 2, 0};
        uint8_t hb = h[k * 64 + g * 16 + j * 4 + t];
        u |= ((hb >> sh[sub]) & 3) << 4;
    }
    return u;
}

void k2o_nibble4_dequant_row(const uint8_t *pair_stream, const uint8_t *tail_stream, size_t rows,
                             size_t cols, size_t planes, size_t r, float *out) {
    const size_t hp = planes - 4, nc = cols / BLK, ns = (rows + STRIPE - 1) / STRIPE;
    const int max_odd = (1 << planes) - 1;
    size_t stripe = r / STRIPE, lane = r % STRIPE;
    for (size_t c = 0; c < nc; ++c) {
        const uint8_t *d, *h, *s;
        n4_ptrs(pair_stream, tail_stream, ns / 2, nc, hp, stripe, c, &d, &h, &s);
        float delta = from_bf16((uint16_t)(s[lane * 2] | (s[lane * 2 + 1] << 8)));
        for (size_t i = 0; i < BLK; ++i)
            out[c * BLK + i] = (float)(2 * n4_code(d, h, hp, lane, i) - max_odd) * delta;
    }
}

void k2o_nibble4_gemv(const uint8_t *pair_stream, const uint8_t *tail_stream, size_t rows, size_t cols,
                      size_t planes, const int8_t *xq, const float *xs, const int32_t *xsum,
                      size_t n_tok, float *out, size_t out_stride, int32_t *int_dots, size_t threads) {
    const size_t hp = planes - 4, nc = cols / BLK, ns = (rows + STRIPE - 1) / STRIPE;
    const int max_odd = (1 << planes) - 1;
    parallel_ranges(ns, threads, [&](size_t s_lo, size_t s_hi) {
        std::vector<float> f(n_tok * STRIPE);
        uint8_t codes[STRIPE][64];
        for (size_t s = s_lo; s < s_hi; ++s) {
            std::fill(f.begin(), f.end(), 0.0f);
            size_t row0 = s * STRIPE, valid = std::min(STRIPE, rows - row0);
            for (size_t c = 0; c < nc; ++c) {
                const uint8_t *d, *h, *sp;
                n4_ptrs(pair_stream, tail_stream, ns / 2, nc, hp, s, c, &d, &h, &sp);
                for (size_t lane = 0; lane < STRIPE; ++lane)
                    for (size_t i = 0; i < 64; ++i) codes[lane][i] = (uint8_t)n4_code(d, h, hp, lane, i);
                for (size_t t = 0; t < n_tok; ++t) {
                    float sx = xs[t * nc + c];
                    const int8_t *q = xq + t * cols + c * BLK;
                    int32_t off = max_odd * xsum[t * nc + c];
                    for (size_t lane = 0; lane < valid; ++lane) {
                        int32_t a = 0;
                        for (size_t i = 0; i < 64; ++i) a += (int32_t)codes[lane][i] * (int32_t)q[i];
                        int32_t dot = 2 * a - off;
                        if (int_dots) int_dots[(t * rows + row0 + lane) * nc + c] = dot;
                        if (sx == 0.0f) continue;  // chunk skipped (3781-3783)
                        float ws = from_bf16((uint16_t)(sp[lane * 2] | (sp[lane * 2 + 1] << 8)));
                        f[t * STRIPE + lane] = std::fmaf((float)dot * sx, ws, f[t * STRIPE + lane]);
                    }
                }
            }
            for (size_t t = 0; t < n_tok; ++t)
                for (size_t lane = 0; lane < valid; ++lane) out[t * out_stride + row0 + lane] = f[t * STRIPE + lane];
        }
    });
}

void k2o_bipolar_gemv_def(const uint8_t *data, const uint16_t *sc, size_t rows, size_t cols, size_t planes,
                          const int8_t *xq, const float *xs, const int32_t *xsum, float *out,
                          int32_t *int_dots) {
    const size_t nc = cols / BLK;
    const int max_odd = (1 << planes) - 1;
    std::vector<uint8_t> codes(cols);
    for (size_t r = 0; r < rows; ++r) {
        k2o_bipolar_unpack_row(data, rows, cols, planes, r, codes.data());
        float f = 0.0f;
        size_t sc_base = (r / STRIPE) * nc * STRIPE + r % STRIPE;
        for (size_t c = 0; c < nc; ++c) {
            int32_t a = 0;
            for (size_t i = 0; i < BLK; ++i) a += (int32_t)codes[c * BLK + i] * (int32_t)xq[c * BLK + i];
            int32_t dot = 2 * a - max_odd * xsum[c];
            if (int_dots) int_dots[r * nc + c] = dot;
            if (xs[c] == 0.0f) continue;
            f = std::fmaf((float)dot * xs[c], from_bf16(sc[sc_base + c * STRIPE]), f);
        }
        out[r] = f;
    }
}

/* ======================= NF / E8Q2 codebooks ============================= */

const int8_t K2O_NF5_DEFAULT_POS[16] = {3, 8, 13, 19, 24, 30, 36, 42, 49, 56, 64, 72, 82, 93, 107, 127};
const int8_t K2O_NF4_DEFAULT[16] = {-127, -96, -75, -58, -44, -31, -18, -6, 6, 18, 31, 44, 58, 75, 96, 127};
const int8_t K2O_NF3_DEFAULT[16] = {-127, -79, -45, -14, 14, 45, 79, 127, 0, 0, 0, 0, 0, 0, 0, 0};
const int8_t K2O_E8Q2_EVEN_TEMPLATES[28][4] = {
    {0, 0, 0, 0},   {32, 32, 0, 0},  {32, 0, 32, 0},  {32, 0, 0, 32},  {0, 32, 32, 0},   {0, 32, 0, 32},
    {0, 0, 32, 32}, {64, 0, 0, 0},   {0, 64, 0, 0},   {0, 0, 64, 0},   {0, 0, 0, 64},    {32, 32, 32, 32},
    {32, 0, 0, 0},  {0, 32, 0, 0},   {0, 0, 32, 0},   {0, 0, 0, 32},   {32, 32, 32, 0},  {32, 32, 0, 32},
    {32, 0, 32, 32}, {0, 32, 32, 32}, {96, 0, 0, 0},  {0, 96, 0, 0},   {0, 0, 96, 0},    {0, 0, 0, 96},
    {64, 32, 32, 32}, {32, 64, 32, 32}, {32, 32, 64, 32}, {32, 32, 32, 64}};

void k2o_nf_expand_codebook32(size_t bits, const int8_t cb[16], int8_t out[32]) {
    std::memset(out, 0, 32);
    if (bits == 5) {
        for (int m = 0; m < 16; ++m) { out[15 - m] = (int8_t)(-cb[m]); out[16 + m] = cb[m]; }
    } else {
        std::memcpy(out, cb, 16);
    }
}

void k2o_e8q2_decode_8d(uint8_t tpl, uint8_t sgn, int8_t out[8]) {
    bool even_coset = (__builtin_popcount((unsigned)(tpl ^ sgn)) & 1) != 0;
    if (even_coset) {
        unsigned tu = tpl & 0x0F, tv = tpl >> 4;
        unsigned ui = (tu < 12 && tv >= 12) ? 16 + tu : tu;
        unsigned vi = (tv < 12 && tu >= 12) ? 16 + tv : tv;
        for (int i = 0; i < 4; ++i) {
            int8_t mu = K2O_E8Q2_EVEN_TEMPLATES[ui][i], mv = K2O_E8Q2_EVEN_TEMPLATES[vi][i];
            out[i] = ((sgn >> i) & 1) ? (int8_t)-mu : mu;
            out[4 + i] = ((sgn >> (4 + i)) & 1) ? (int8_t)-mv : mv;
        }
    } else {
        for (int i = 0; i < 8; ++i) {
            int8_t mag = ((tpl >> i) & 1) ? 48 : 16;
            out[i] = ((sgn >> i) & 1) ? (int8_t)-mag : mag;
        }
    }
}

size_t k2o_nf_chunk_bytes(size_t bits) {
    switch (bits) { case 5: return 640; case 4: return 512; case 3: return 384; case 2: return 256; }
    return 0;
}
static inline size_t nf_nsg(size_t cols, size_t sgc) { return (cols / BLK + sgc - 1) / sgc; }
static inline size_t nf_pair_tot(size_t cols, size_t bits, size_t sgc) {
    return nf_nsg(cols, sgc) * 64 + (cols / BLK) * 2 * k2o_nf_chunk_bytes(bits);
}
static inline size_t nf_tail_tot(size_t cols, size_t bits, size_t sgc) {
    return nf_nsg(cols, sgc) * 32 + (cols / BLK) * k2o_nf_chunk_bytes(bits);
}
size_t k2o_nf_pair_stream_bytes(size_t rows, size_t cols, size_t bits, size_t sgc) {
    return (((rows + STRIPE - 1) / STRIPE) / 2) * nf_pair_tot(cols, bits, sgc);
}
size_t k2o_nf_tail_stream_bytes(size_t rows, size_t cols, size_t bits, size_t sgc) {
    return (((rows + STRIPE - 1) / STRIPE) & 1) * nf_tail_tot(cols, bits, sgc);
}
size_t k2o_nf_scale_count(size_t rows, size_t cols, size_t sgc) {
    return ((rows + STRIPE - 1) / STRIPE) * nf_nsg(cols, sgc) * STRIPE;
}

float k2o_nf_fit_codebook(const float *weights, size_t rows, size_t cols, size_t bits, size_t sgc_in,
                          int8_t codebook[16]) {
    constexpr size_t HIST_BINS = 2000;
    const float Z_MAX = 5.0f;
    const float BIN_W = Z_MAX / (float)HIST_BINS;
    const int8_t *def_cb = bits == 5 ? K2O_NF5_DEFAULT_POS : bits == 4 ? K2O_NF4_DEFAULT : K2O_NF3_DEFAULT;
    const float def_top = bits == 5 ? 3.2500f : bits == 4 ? 2.7326f : 2.1520f;
    const size_t nc = cols / BLK, sgc = std::max<size_t>(sgc_in, 1), nsg = (nc + sgc - 1) / sgc;
    const size_t step = std::max<size_t>(rows / 512, 1);
    std::vector<uint64_t> hist(HIST_BINS, 0);
    uint64_t total = 0;
    std::vector<float> row(cols);
    for (size_t r = 0; r < rows; r += step) {
        std::memcpy(row.data(), weights + r * cols, cols * sizeof(float));
        k2o_fwht64(row.data(), cols, 0);
        for (size_t sg = 0; sg < nsg; ++sg) {
            size_t col_s = sg * sgc * BLK, col_e = std::min((sg + 1) * sgc * BLK, cols);
            float sum_sq = 0.0f;
            for (size_t i = col_s; i < col_e; ++i) sum_sq += row[i] * row[i];
            float rms = std::sqrt(sum_sq / (float)(col_e - col_s));
            if (rms <= 1e-12f) continue;
            float inv_rms = 1.0f / rms;
            for (size_t i = col_s; i < col_e; ++i) {
                float z = std::fabs(row[i]) * inv_rms;
                size_t bin = std::min((size_t)(z / BIN_W), HIST_BINS - 1);
                hist[bin] += 1;
                total += 1;
            }
        }
    }
    if (total < 256) { std::memcpy(codebook, def_cb, 16); return def_top; }

    const size_t half = (size_t)1 << (bits - 1);
    std::vector<double> mu;
    if (bits == 5) mu = {0.068, 0.205, 0.343, 0.483, 0.626, 0.773, 0.925, 1.084,
                         1.252, 1.432, 1.628, 1.845, 2.092, 2.382, 2.743, 3.250};
    else if (bits == 4) mu = {0.1284, 0.3881, 0.6568, 0.9424, 1.2562, 1.6180, 2.0690, 2.7326};
    else mu = {0.2451, 0.7560, 1.3439, 2.1520};
    const double bw = (double)BIN_W;
    for (int it = 0; it < 24; ++it) {
        std::vector<size_t> bounds(half + 1, 0);
        bounds[half] = HIST_BINS;
        for (size_t m = 0; m + 1 < half; ++m) {
            double mid = 0.5 * (mu[m] + mu[m + 1]);
            size_t b = (size_t)std::round(mid / bw);
            bounds[m + 1] = std::min(std::max(b, bounds[m]), HIST_BINS);
        }
        for (size_t m = 0; m < half; ++m) {
            double w_sum = 0.0; uint64_t c_sum = 0;
            for (size_t b = bounds[m]; b < bounds[m + 1]; ++b)
                if (hist[b] > 0) { w_sum += (double)hist[b] * (((double)b + 0.5) * bw); c_sum += hist[b]; }
            if (c_sum > 0) mu[m] = w_sum / (double)c_sum;
        }
        for (size_t m = 1; m < half; ++m)
            if (mu[m] <= mu[m - 1] + 1e-4) mu[m] = mu[m - 1] + 0.05;
    }
    double mu_top = std::max(mu[half - 1], 0.5);
    std::vector<int> q_pos(half);
    for (size_t m = 0; m < half; ++m) {
        int v = (int)std::round(127.0 * mu[m] / mu_top);
        q_pos[m] = std::min(std::max(v, 1), 127);
    }
    q_pos[half - 1] = 127;
    for (size_t m = half - 1; m-- > 0;)
        if (q_pos[m] >= q_pos[m + 1]) q_pos[m] = std::max(q_pos[m + 1] - 1, 1);
    for (size_t m = 1; m < half; ++m)
        if (q_pos[m] <= q_pos[m - 1]) q_pos[m] = std::min(q_pos[m - 1] + 1, 127);
    std::memset(codebook, 0, 16);
    if (bits == 5) {
        for (size_t m = 0; m < 16; ++m) codebook[m] = (int8_t)q_pos[m];
    } else {
        for (size_t m = 0; m < half; ++m) {
            codebook[half - 1 - m] = (int8_t)(-q_pos[m]);
            codebook[half + m] = (int8_t)q_pos[m];
        }
    }
    return (float)mu_top;
}

void k2o_nf_quantize_rtn(const float *weights, size_t rows, size_t cols, size_t bits, size_t sgc,
                         size_t threads, int8_t codebook[16], uint8_t *flat_idx, uint16_t *scales) {
    // quantize_stripe_batch_nf with u_slice = None (compiler.rs:1624-1860).
    static const float ratios[11] = {0.74f, 0.80f, 0.86f, 0.91f, 0.96f, 1.00f, 1.04f, 1.09f, 1.15f, 1.22f, 1.30f};
    const float mu_top = k2o_nf_fit_codebook(weights, rows, cols, bits, sgc, codebook);
    const size_t nc = cols / BLK, nsg = (nc + sgc - 1) / sgc;
    const size_t half = (size_t)1 << (bits - 1), levels = (size_t)1 << bits;
    int8_t cb32[32];
    k2o_nf_expand_codebook32(bits, codebook, cb32);
    float cb_f[32] = {0};
    for (size_t k = 0; k < levels; ++k) cb_f[k] = (float)cb32[k];
    float pos_th[15] = {0};
    for (size_t m = 0; m + 1 < half; ++m) pos_th[m] = 0.5f * (cb_f[half + m] + cb_f[half + m + 1]);
    std::fill(scales, scales + k2o_nf_scale_count(rows, cols, sgc), (uint16_t)0);

    // Nearest centroid by magnitude thresholds. The reference walks a fixed binary tree
    // (1655-1707); with ascending thresholds that equals counting the thresholds <= |w|/delta.
    auto nearest = [&](float w, float inv_delta) -> size_t {
        float aw = std::fabs(w) * inv_delta;
        size_t lo = 0, n = half;  // magnitude index in [0, half)
        while (n > 1) {
            size_t h = n / 2;
            if (aw < pos_th[lo + h - 1]) n = h; else { lo += h; n -= h; }
        }
        return (w >= 0.0f) ? half + lo : half - 1 - lo;
    };

    parallel_ranges(rows, threads, [&](size_t lo, size_t hi) {
        std::vector<float> work(cols);
        std::vector<uint8_t> best_idx(sgc * BLK), cand(sgc * BLK);
        for (size_t r = lo; r < hi; ++r) {
            std::memcpy(work.data(), weights + r * cols, cols * sizeof(float));
            k2o_fwht64(work.data(), cols, 0);
            for (size_t sg = 0; sg < nsg; ++sg) {
                size_t col_s = sg * sgc * BLK, col_e = std::min((sg * sgc + sgc), nc) * BLK;
                size_t glen = col_e - col_s;
                const float *sub = work.data() + col_s;
                float sum_sq = 0.0f;
                for (size_t i = 0; i < glen; ++i) sum_sq += sub[i] * sub[i];
                float rms = std::sqrt(sum_sq / (float)glen);
                size_t sc_i = ((r / STRIPE) * nsg + sg) * STRIPE + r % STRIPE;
                if (rms <= 1e-12f) {
                    std::memset(flat_idx + r * cols + col_s, (int)(half - 1), glen);
                    scales[sc_i] = 0;
                    continue;
                }
                float base_delta = rms * (mu_top / 127.0f);
                float best_loss = INFINITY;
                uint16_t best_bf16 = 0;
                auto eval = [&](uint16_t d_bf16) {
                    float delta = from_bf16(d_bf16);
                    if (!(delta > 0.0f)) return;
                    float inv_delta = 1.0f / delta, loss = 0.0f;
                    for (size_t j = 0; j < glen; ++j) {
                        size_t k = nearest(sub[j], inv_delta);
                        cand[j] = (uint8_t)k;
                        float diff = sub[j] - cb_f[k] * delta;
                        loss += diff * diff;
                    }
                    if (loss < best_loss) {
                        best_loss = loss;
                        best_bf16 = d_bf16;
                        std::memcpy(best_idx.data(), cand.data(), glen);
                    }
                };
                for (float rat : ratios) eval(to_bf16(base_delta * rat));
                // least-squares refit of the bf16 scale on the chosen centroids (1800-1821)
                float dot_wc = 0.0f, dot_cc = 0.0f;
                for (size_t j = 0; j < glen; ++j) {
                    float cv = cb_f[best_idx[j]];
                    dot_wc += sub[j] * cv;
                    dot_cc += cv * cv;
                }
                if (dot_cc > 1e-12f && dot_wc > 0.0f) {
                    uint16_t ls = to_bf16(dot_wc / dot_cc);
                    if (ls != best_bf16) eval(ls);
                }
                scales[sc_i] = best_bf16;
                std::memcpy(flat_idx + r * cols + col_s, best_idx.data(), glen);
            }
        }
    });
}

}  // extern "C"

namespace {
// One (stripe, chunk) block of packed indices: closure pack_one_stripe_chunk, simd_lut.rs:4884-4960.
void nf_pack_chunk(const uint8_t *flat, size_t rows, size_t cols, size_t bits, size_t stripe, size_t c,
                   uint8_t *dst) {
    const size_t r_base = stripe * STRIPE, c_col = c * BLK;
    auto idx_at = [&](size_t lane, size_t sub_col) -> uint8_t {
        size_t r = r_base + lane;
        return r < rows ? flat[r * cols + c_col + sub_col] : (uint8_t)0;
    };
    if (bits == 4 || bits == 5) {
        for (size_t k = 0; k < 4; ++k)
            for (size_t lane = 0; lane < 16; ++lane)
                for (size_t t = 0; t < 4; ++t) {
                    size_t g = lane / 4, j = lane % 4;
                    size_t b0 = k * 128 + g * 32 + j * 4 + t;
                    dst[b0] = (uint8_t)((idx_at(lane, k * 16 + t) & 0x0F) | ((idx_at(lane, k * 16 + 4 + t) & 0x0F) << 4));
                    dst[b0 + 16] = (uint8_t)((idx_at(lane, k * 16 + 8 + t) & 0x0F) | ((idx_at(lane, k * 16 + 12 + t) & 0x0F) << 4));
                }
        if (bits == 5)
            for (size_t lane = 0; lane < 16; ++lane)
                for (size_t kp = 0; kp < 2; ++kp)
                    for (size_t t = 0; t < 4; ++t) {
                        size_t g = lane / 4, j = lane % 4, k0 = kp * 2, k1 = k0 + 1;
                        uint8_t v = 0;
                        for (size_t q = 0; q < 4; ++q) {
                            v |= (uint8_t)(((idx_at(lane, k0 * 16 + 4 * q + t) >> 4) & 1) << (4 + q));
                            v |= (uint8_t)(((idx_at(lane, k1 * 16 + 4 * q + t) >> 4) & 1) << q);
                        }
                        dst[512 + g * 32 + kp * 16 + j * 4 + t] = v;
                    }
    } else {  // 3-bit: eight indices in three bytes
        for (size_t kp = 0; kp < 2; ++kp)
            for (size_t lane = 0; lane < 16; ++lane)
                for (size_t t = 0; t < 4; ++t) {
                    size_t g = lane / 4, j = lane % 4, b = j * 4 + t;
                    uint8_t i[8];
                    for (size_t q = 0; q < 8; ++q) i[q] = idx_at(lane, kp * 32 + 4 * q + t) & 7;
                    uint8_t *blk = dst + kp * 192 + g * 48;
                    blk[b] = (uint8_t)(i[0] | (i[1] << 3) | ((i[2] & 3) << 6));
                    blk[16 + b] = (uint8_t)(i[3] | (i[4] << 3) | ((i[5] & 3) << 6));
                    blk[32 + b] = (uint8_t)(i[6] | (i[7] << 3) | (((i[2] >> 2) & 1) << 6) | (((i[5] >> 2) & 1) << 7));
                }
    }
}

void e8_pack_chunk(const uint8_t *tpl, const uint8_t *sgn, size_t rows, size_t cols, size_t stripe,
                   size_t c, uint8_t *dst) {
    const size_t bpr = cols / 8, r_base = stripe * STRIPE;
    for (size_t kp = 0; kp < 2; ++kp)
        for (size_t lane = 0; lane < 16; ++lane)
            for (size_t eb = 0; eb < 4; ++eb) {
                size_t g = lane / 4, j = lane % 4, r = r_base + lane;
                uint8_t tp = 0, sg = 1;  // padding rows decode to zeros
                if (r < rows) { tp = tpl[r * bpr + c * 8 + kp * 4 + eb]; sg = sgn[r * bpr + c * 8 + kp * 4 + eb]; }
                uint8_t *blk = dst + kp * 128 + g * 32;
                blk[eb * 4 + j] = tp;
                blk[16 + eb * 4 + j] = sg;
            }
}

template <class PackChunk>
void nf_pack_streams(const uint16_t *sc, size_t rows, size_t cols, size_t bits, size_t sgc,
                     uint8_t *pair_stream, uint8_t *tail_stream, PackChunk pack_chunk) {
    const size_t ns = (rows + STRIPE - 1) / STRIPE, num_pairs = ns / 2, nc = cols / BLK;
    const size_t nsg = (nc + sgc - 1) / sgc, cb = k2o_nf_chunk_bytes(bits);
    const size_t pair_tot = nf_pair_tot(cols, bits, sgc);
    std::memset(pair_stream, 0, num_pairs * pair_tot);
    for (size_t p = 0; p < num_pairs; ++p) {
        size_t cur = p * pair_tot;
        for (size_t sg = 0; sg < nsg; ++sg) {
            for (size_t side = 0; side < 2; ++side)
                for (size_t lane = 0; lane < STRIPE; ++lane) {
                    uint16_t v = sc[((2 * p + side) * nsg + sg) * STRIPE + lane];
                    pair_stream[cur + side * 32 + lane * 2] = (uint8_t)(v & 0xFF);
                    pair_stream[cur + side * 32 + lane * 2 + 1] = (uint8_t)(v >> 8);
                }
            cur += 64;
            for (size_t c = sg * sgc; c < std::min(sg * sgc + sgc, nc); ++c) {
                pack_chunk(2 * p, c, pair_stream + cur);
                pack_chunk(2 * p + 1, c, pair_stream + cur + cb);
                cur += 2 * cb;
            }
        }
    }
    if (ns & 1) {
        std::memset(tail_stream, 0, nf_tail_tot(cols, bits, sgc));
        size_t st = num_pairs * 2, cur = 0;
        for (size_t sg = 0; sg < nsg; ++sg) {
            for (size_t lane = 0; lane < STRIPE; ++lane) {
                uint16_t v = sc[(st * nsg + sg) * STRIPE + lane];
                tail_stream[cur + lane * 2] = (uint8_t)(v & 0xFF);
                tail_stream[cur + lane * 2 + 1] = (uint8_t)(v >> 8);
            }
            cur += 32;
            for (size_t c = sg * sgc; c < std::min(sg * sgc + sgc, nc); ++c) {
                pack_chunk(st, c, tail_stream + cur);
                cur += cb;
            }
        }
    }
}

// (data, scales) of (stripe, chunk): NfSdotMatrix::stripe_chunk_ptrs, simd_lut.rs:5526-5557.
inline void nf_ptrs(const uint8_t *pair_stream, const uint8_t *tail_stream, size_t num_pairs, size_t cols,
                    size_t bits, size_t sgc, size_t stripe, size_t c, const uint8_t **d, const uint8_t **s) {
    const size_t cb = k2o_nf_chunk_bytes(bits), sg = c / sgc, sub_c = c % sgc, c_start = sg * sgc;
    if (stripe < num_pairs * 2) {
        size_t side = stripe & 1;
        const uint8_t *sgp = pair_stream + (stripe / 2) * nf_pair_tot(cols, bits, sgc) + sg * 64 + c_start * 2 * cb;
        *s = sgp + side * 32;
        *d = sgp + 64 + sub_c * 2 * cb + side * cb;
    } else {
        const uint8_t *sgp = tail_stream + sg * 32 + c_start * cb;
        *s = sgp;
        *d = sgp + 32 + sub_c * cb;
    }
}

// Signed int8 weight values of one lane for the 64 columns of a chunk.
inline void nf_decode_lane(const uint8_t *d, size_t bits, const int8_t cb32[32], size_t lane, int8_t w[64]) {
    const size_t g = lane / 4, j = lane % 4;
    if (bits == 2) {
        for (size_t kp = 0; kp < 2; ++kp)
            for (size_t eb = 0; eb < 4; ++eb) {
                size_t off = kp * 128 + g * 32 + eb * 4 + j;
                k2o_e8q2_decode_8d(d[off], d[off + 16], w + kp * 32 + eb * 8);
            }
    } else if (bits == 3) {
        for (size_t kp = 0; kp < 2; ++kp)
            for (size_t t = 0; t < 4; ++t) {
                const uint8_t *blk = d + kp * 192 + g * 48;
                size_t b = j * 4 + t;
                uint8_t v0 = blk[b], v1 = blk[16 + b], v2 = blk[32 + b];
                uint8_t i[8] = {(uint8_t)(v0 & 7), (uint8_t)((v0 >> 3) & 7),
                                (uint8_t)(((v0 >> 6) & 3) | (((v2 >> 6) & 1) << 2)),
                                (uint8_t)(v1 & 7), (uint8_t)((v1 >> 3) & 7),
                                (uint8_t)(((v1 >> 6) & 3) | (((v2 >> 7) & 1) << 2)),
                                (uint8_t)(v2 & 7), (uint8_t)((v2 >> 3) & 7)};
                for (size_t q = 0; q < 8; ++q) w[kp * 32 + 4 * q + t] = cb32[i[q]];
            }
    } else {
        for (size_t sub_col = 0; sub_col < 64; ++sub_col) {
            size_t k = sub_col / 16, ww = sub_col % 16, sub4 = ww / 4, t = ww % 4, b = j * 4 + t;
            uint8_t byte = d[k * 128 + g * 32 + (sub4 / 2) * 16 + b];
            unsigned idx = (sub4 & 1) ? (byte >> 4) : (byte & 0x0F);
            if (bits == 5) {
                uint8_t hb = d[512 + g * 32 + (k / 2) * 16 + b];
                size_t sh = ((k & 1) == 0) ? 4 + sub4 : sub4;
                idx |= ((hb >> sh) & 1u) << 4;
            }
            w[sub_col] = cb32[idx];
        }
    }
}
}  // namespace

extern "C" {

void k2o_nf_pack(const uint8_t *flat_idx, const uint16_t *sc, size_t rows, size_t cols, size_t bits,
                 size_t sgc, uint8_t *pair_stream, uint8_t *tail_stream) {
    nf_pack_streams(sc, rows, cols, bits, sgc, pair_stream, tail_stream,
                    [&](size_t stripe, size_t c, uint8_t *dst) { nf_pack_chunk(flat_idx, rows, cols, bits, stripe, c, dst); });
}

// NfSdotMatrix::build_nf4_from_bf16_getter (simd_lut.rs:5262-5495): the untied bf16 embedding table as 4-bit rows in the
// rotated domain, default NF4 codebook.  Per row and scale group: scale0 = max|v| / top, indices at scale0, the least-squares
// scale of those indices (bf16), indices again at that scale.  Lanes past the last row hold index 8 and scale 0.
void k2o_nf4_embed_from_bf16(const uint16_t *bf16, size_t rows, size_t cols, size_t sgc, size_t threads,
                             uint8_t *pair_stream, uint8_t *tail_stream) {
    if (sgc == 0) sgc = 1;
    const size_t nc = cols / BLK, nsg = (nc + sgc - 1) / sgc, rows_pad = (rows + STRIPE - 1) / STRIPE * STRIPE;
    int8_t cb32[32];
    k2o_nf_expand_codebook32(4, K2O_NF4_DEFAULT, cb32);
    float pos_th[7];
    for (size_t m = 0; m < 7; ++m) pos_th[m] = 0.5f * ((float)cb32[8 + m] + (float)cb32[9 + m]);
    const float cb_top = std::max((float)cb32[15], 1.0f);
    auto quant4 = [&](float w, float inv_delta) -> uint8_t {           // the reference's fixed comparison tree (5277-5293)
        const float aw = std::fabs(w) * inv_delta;
        size_t mag;
        if (aw < pos_th[3]) mag = aw < pos_th[1] ? (aw >= pos_th[0] ? 1 : 0) : 2 + (aw >= pos_th[2] ? 1 : 0);
        else if (aw < pos_th[5]) mag = 4 + (aw >= pos_th[4] ? 1 : 0);
        else mag = 6 + (aw >= pos_th[6] ? 1 : 0);
        return (uint8_t)(w >= 0.0f ? 8 + mag : 7 - mag);
    };
    std::vector<uint8_t> idx(rows_pad * cols, (uint8_t)8);
    std::vector<uint16_t> sc(k2o_nf_scale_count(rows_pad, cols, sgc), (uint16_t)0);
    parallel_ranges(rows, threads, [&](size_t lo, size_t hi) {
        std::vector<float> buf(cols);
        for (size_t r = lo; r < hi; ++r) {
            for (size_t c = 0; c < cols; ++c) buf[c] = from_bf16(bf16[r * cols + c]);
            k2o_fwht64(buf.data(), cols, 0);
            for (size_t sg = 0; sg < nsg; ++sg) {
                const size_t col0 = sg * sgc * BLK, col1 = std::min(col0 + sgc * BLK, cols);
                const size_t sc_i = ((r / STRIPE) * nsg + sg) * STRIPE + r % STRIPE;
                float max_abs = 0.0f;
                for (size_t c = col0; c < col1; ++c) if (std::fabs(buf[c]) > max_abs) max_abs = std::fabs(buf[c]);
                if (max_abs <= 1e-12f) { sc[sc_i] = 0; continue; }      // indices stay 8
                const float inv0 = cb_top / max_abs;
                float dot_wq = 0.0f, dot_qq = 0.0f;
                for (size_t c = col0; c < col1; ++c) {
                    const float qf = (float)cb32[quant4(buf[c], inv0)];
                    dot_wq += buf[c] * qf;
                    dot_qq += qf * qf;
                }
                const uint16_t d16 = k2o_f32_to_bf16(dot_qq > 0.0f ? std::max(dot_wq / dot_qq, 0.0f) : max_abs / cb_top);
                const float delta = from_bf16(d16), inv = delta > 1e-12f ? 1.0f / delta : 0.0f;
                for (size_t c = col0; c < col1; ++c) idx[r * cols + c] = quant4(buf[c], inv);
                sc[sc_i] = d16;
            }
        }
    });
    k2o_nf_pack(idx.data(), sc.data(), rows_pad, cols, 4, sgc, pair_stream, tail_stream);
}

void k2o_e8q2_pack(const uint8_t *tpl, const uint8_t *sgn, const uint16_t *sc, size_t rows, size_t cols,
                   size_t sgc, uint8_t *pair_stream, uint8_t *tail_stream) {
    nf_pack_streams(sc, rows, cols, 2, sgc, pair_stream, tail_stream,
                    [&](size_t stripe, size_t c, uint8_t *dst) { e8_pack_chunk(tpl, sgn, rows, cols, stripe, c, dst); });
}

void k2o_nf_gate_up_interleave(const uint8_t *pair_stream, size_t rows, size_t cols, size_t bits,
                               size_t sgc, uint8_t *out) {
    const size_t nc_i = rows / 128, blk64 = 2 * nf_pair_tot(cols, bits, sgc);
    for (size_t ic = 0; ic < nc_i; ++ic) {
        std::memcpy(out + (ic * 2) * blk64, pair_stream + ic * blk64, blk64);
        std::memcpy(out + (ic * 2 + 1) * blk64, pair_stream + (nc_i + ic) * blk64, blk64);
    }
}

void k2o_nf_dequant_row(const uint8_t *pair_stream, const uint8_t *tail_stream, const int8_t codebook[16],
                        size_t rows, size_t cols, size_t bits, size_t sgc, size_t r, float *out) {
    const size_t ns = (rows + STRIPE - 1) / STRIPE, nc = cols / BLK, stripe = r / STRIPE, lane = r % STRIPE;
    int8_t cb32[32];
    k2o_nf_expand_codebook32(bits, codebook, cb32);
    for (size_t c = 0; c < nc; ++c) {
        const uint8_t *d, *s;
        nf_ptrs(pair_stream, tail_stream, ns / 2, cols, bits, sgc, stripe, c, &d, &s);
        float delta = from_bf16((uint16_t)(s[lane * 2] | (s[lane * 2 + 1] << 8)));
        int8_t w[64];
        nf_decode_lane(d, bits, cb32, lane, w);
        for (size_t i = 0; i < 64; ++i) out[c * BLK + i] = (float)w[i] * delta;
    }
}

void k2o_nf_gemv(const uint8_t *pair_stream, const uint8_t *tail_stream, const int8_t codebook[16],
                 size_t rows, size_t cols, size_t bits, size_t sgc, const int8_t *xq, const float *xs,
                 size_t n_tok, float *out, size_t out_stride, int32_t *int_dots, size_t threads) {
    const size_t ns = (rows + STRIPE - 1) / STRIPE, nc = cols / BLK;
    int8_t cb32[32];
    k2o_nf_expand_codebook32(bits, codebook, cb32);
    parallel_ranges(ns, threads, [&](size_t s_lo, size_t s_hi) {
        std::vector<float> f(n_tok * STRIPE);
        int8_t w[STRIPE][64];
        for (size_t s = s_lo; s < s_hi; ++s) {
            std::fill(f.begin(), f.end(), 0.0f);
            size_t row0 = s * STRIPE, valid = std::min(STRIPE, rows - row0);
            for (size_t c = 0; c < nc; ++c) {
                const uint8_t *d, *sp;
                nf_ptrs(pair_stream, tail_stream, ns / 2, cols, bits, sgc, s, c, &d, &sp);
                for (size_t lane = 0; lane < STRIPE; ++lane) nf_decode_lane(d, bits, cb32, lane, w[lane]);
                for (size_t t = 0; t < n_tok; ++t) {
                    float sx = xs[t * nc + c];
                    const int8_t *q = xq + t * cols + c * BLK;
                    for (size_t lane = 0; lane < valid; ++lane) {
                        int32_t a = 0;
                        for (size_t i = 0; i < 64; ++i) a += (int32_t)w[lane][i] * (int32_t)q[i];
                        if (int_dots) int_dots[(t * rows + row0 + lane) * nc + c] = a;
                        if (sx == 0.0f) continue;  // 6105-6108
                        float ws = from_bf16((uint16_t)(sp[lane * 2] | (sp[lane * 2 + 1] << 8)));
                        f[t * STRIPE + lane] = std::fmaf((float)a * sx, ws, f[t * STRIPE + lane]);
                    }
                }
            }
            for (size_t t = 0; t < n_tok; ++t)
                for (size_t lane = 0; lane < valid; ++lane) out[t * out_stride + row0 + lane] = f[t * STRIPE + lane];
        }
    });
}

}  // extern "C"

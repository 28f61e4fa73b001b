// Device helpers shared by the per-token kernels and the whole-token decode kernel.
#pragma once
#include "k2t_device.cuh"
#include "k2t_fwht.cuh"
#include "k2t_model_kernels.h"

namespace k2t {

// exp_f32_neon (src/model/real_llm.rs:9430-9454), one lane, same operations in the same order.
__device__ __forceinline__ float exp_poly(float x_raw) {
    const float x = fminf(fmaxf(x_raw, -87.33654f), 88.0f);
    const float kf = rintf(__fmul_rn(x, 1.44269504088896340736f));
    const float r = __fmaf_rn(-kf, 1.4286068e-6f, __fmaf_rn(-kf, 0.69314575f, x));
    float y = __fmaf_rn(1.9875691e-4f, r, 1.3982e-3f);
    y = __fmaf_rn(y, r, 8.333452e-3f);
    y = __fmaf_rn(y, r, 4.1665796e-2f);
    y = __fmaf_rn(y, r, 1.6666666e-1f);
    y = __fmaf_rn(y, r, 0.5f);
    y = __fmaf_rn(y, r, 1.0f);
    y = __fmaf_rn(y, r, 1.0f);
    const int ki = (int)kf;
    return __fmul_rn(y, __int_as_float((ki + 127) << 23));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
    return v;
}

// ------------------------------------------------------------------------------------------------
// embedding (embed_token_into, real_llm.rs:8063-8097)
// ------------------------------------------------------------------------------------------------
// weight value (rotated domain) of element `col` (0..63) of cell (row, c)
__device__ __forceinline__ float cell_value(const EmbedArgs &a, uint32_t row, uint32_t c, uint32_t col) {
    // pass-tile addressing (k2t_layout.h): tile p = c / 32 holds n cells per row
    const uint32_t p = c / 32, n = tile_chunks(a.nc, p);
    const size_t cell = (size_t)row * n + c % 32;
    const uint8_t *p0 = a.plane[0] + tile_code_off(a.rows_pad, a.cell[0], p) + cell * a.cell[0];
    const uint8_t *p1 = a.plane[1] + tile_code_off(a.rows_pad, a.cell[1], p) + cell * a.cell[1];
    const uint8_t *p2 = a.plane[2] + tile_code_off(a.rows_pad, a.cell[2], p) + cell * a.cell[2];
    const uint8_t *sp = reinterpret_cast<const uint8_t *>(a.scales) + tile_scale_off(a.rows_pad, p) + (size_t)row * tile_scale_pitch(a.nc, a.sgc, p) +
                        (size_t)(c / a.sgc - (32u * p) / a.sgc) * 2;
    const float delta = bf16_bits_to_f32(*reinterpret_cast<const uint16_t *>(sp));
    if (a.fmt == FMT_BP4 || a.fmt == FMT_BP5 || a.fmt == FMT_BP6) {
        const uint8_t *half = col < 32 ? p0 : p1;
        const uint32_t cc = col % 32, k = col % 8;
        uint32_t u = (half[(cc / 8) * 4 + (k % 4)] >> (k < 4 ? 0 : 4)) & 0x0F;
        if (a.fmt == FMT_BP5) {
            const uint32_t bit = 8 * (col % 4) + cc / 4;
            u |= ((p2[(col / 32) * 4 + bit / 8] >> (bit % 8)) & 1u) << 4;
        } else if (a.fmt == FMT_BP6) {
            const uint32_t bit = 8 * (col % 4) + 2 * ((col % 16) / 4);
            u |= ((p2[(col / 16) * 4 + bit / 8] >> (bit % 8)) & 3u) << 4;
        }
        return __fmul_rn((float)(2 * (int)u - a.max_odd), delta);
    }
    if (a.fmt == FMT_E8Q2) {      // e8q2_decode_8d on the (template, sign) pair of the column's 8-column block
        const uint32_t blk = col / 8, i = col % 8, tpl = p0[2 * blk], sgn = p0[2 * blk + 1];
        int mag;
        if ((__popc(tpl ^ sgn) & 1) != 0) {
            const uint32_t tu = tpl & 15u, tv = tpl >> 4;
            const uint32_t ui = (tu < 12u && tv >= 12u) ? 16u + tu : tu, vi = (tv < 12u && tu >= 12u) ? 16u + tv : tv;
            mag = (int)((E8Q2_TEMPLATE_WORDS[i < 4 ? ui : vi] >> (8 * (i % 4))) & 0xFFu);
        } else {
            mag = ((tpl >> i) & 1u) ? 48 : 16;
        }
        return __fmul_rn((float)(((sgn >> i) & 1u) ? -mag : mag), delta);
    }
    uint32_t idx;
    if (a.fmt == FMT_NF3) {
        auto word = [&](uint32_t w) { return w < 4 ? reinterpret_cast<const uint32_t *>(p0)[w] : reinterpret_cast<const uint32_t *>(p1)[w - 4]; };
        if (col < 48) idx = (word(col / 8) >> (4 * (col % 8))) & 7u;
        else {
            const uint32_t t = col - 48;
            idx = 0;
            for (uint32_t j = 0; j < 3; ++j) idx |= ((word(3 * (t / 8) + j) >> (4 * (t % 8) + 3)) & 1u) << j;
        }
    } else {
        const uint8_t *half = col < 32 ? p0 : p1;
        const uint32_t cc = col % 32, nib = col % 8;
        idx = (half[(cc / 8) * 4 + nib / 2] >> (4 * (nib % 2))) & 0x0F;
        if (a.fmt == FMT_NF5) {
            const uint32_t bit = 8 * (col % 4) + cc / 4;
            idx |= ((p2[(col / 32) * 4 + bit / 8] >> (bit % 8)) & 1u) << 4;
        }
    }
    return __fmul_rn((float)a.codebook[idx], delta);
}


// split-KV attention: positions per split = the context divided over the splits, in whole 32-position tiles
__device__ __forceinline__ uint32_t split_span(uint32_t ctx, uint32_t n_split) {
    return (((ctx + n_split - 1) / n_split) + 31u) & ~31u;
}

// ------------------------------------------------------------------------------------------------
// NF4 Hadamard KV cache (kv_bits = 4): store_hadamard_q4_head_raw / nf4_nearest_idx (real_llm.rs:8615-8701)
// ------------------------------------------------------------------------------------------------
__constant__ float NF4_KV_CENTROIDS[16] = {-127.f, -96.f, -75.f, -58.f, -44.f, -31.f, -18.f, -6.f, 6.f, 18.f, 31.f, 44.f, 58.f, 75.f, 96.f, 127.f};
// two-table decode of four packed indices at once (see cell_dot in k2t_gemv_core.cuh): centroid = hi[idx & 7] for
// idx >= 8, -lo[idx] below; a selector nibble with bit 3 set yields the replicated sign bit of a non-negative byte = 0
constexpr uint32_t NF4_KV_HI0 = 0x2C1F1206u, NF4_KV_HI1 = 0x7F604B3Au, NF4_KV_LO0 = 0x3A4B607Fu, NF4_KV_LO1 = 0x06121F2Cu;

__device__ __forceinline__ uint32_t nf4_nearest_idx(float y) {
    const float a = fabsf(y);
    const uint32_t p = a < 37.5f ? (a < 12.0f ? 0u : a < 24.5f ? 1u : 2u) : a < 85.5f ? (a < 51.0f ? 3u : a < 66.5f ? 4u : 5u) : a < 111.5f ? 6u : 7u;
    return y >= 0.0f ? 8u + p : 7u - p;
}
__device__ __forceinline__ uint16_t bf16_rne_bits(float v) {        // f32_to_bf16 (simd_lut.rs:1375-1382)
    const uint32_t bits = __float_as_uint(v);
    if ((bits & 0x7F800000u) == 0x7F800000u && (bits & 0x007FFFFFu) != 0) return (uint16_t)((bits >> 16) | 0x0040u);
    return (uint16_t)((bits + 0x00007FFFu + ((bits >> 16) & 1u)) >> 16);
}

// One 64-value group held by a warp (lane l: rotated elements 2l, 2l+1) -> 32 packed bytes + bf16 scale.  The
// least-squares sums run sequentially in element order, as on the CPU (lane 0: numerator, lane 1: denominator).
// s_val / s_c: 64 floats each, s_idx: 64 bytes of per-warp scratch.  Lane j returns byte j; *scale_bits = the scale.
__device__ __forceinline__ uint32_t warp_quant64_q4(float v0, float v1, uint32_t lane, float *s_val, float *s_c, uint8_t *s_idx,
                                                    uint16_t *scale_bits) {
    const float max_abs = warp_max(fmaxf(fabsf(v0), fabsf(v1)));
    if (max_abs < 1e-30f) { *scale_bits = 0; return 0x88u; }
    const float inv0 = __fdiv_rn(127.0f, max_abs);
    s_val[2 * lane] = v0; s_val[2 * lane + 1] = v1;
    s_c[2 * lane] = NF4_KV_CENTROIDS[nf4_nearest_idx(__fmul_rn(v0, inv0))];
    s_c[2 * lane + 1] = NF4_KV_CENTROIDS[nf4_nearest_idx(__fmul_rn(v1, inv0))];
    __syncwarp();
    float acc = 0.0f;
    if (lane == 0) {
#pragma unroll 8
        for (int i = 0; i < 64; ++i) acc = __fadd_rn(acc, __fmul_rn(s_val[i], s_c[i]));
    } else if (lane == 1) {
#pragma unroll 8
        for (int i = 0; i < 64; ++i) acc = __fadd_rn(acc, __fmul_rn(s_c[i], s_c[i]));
    }
    const float num = __shfl_sync(0xffffffffu, acc, 0), den = __shfl_sync(0xffffffffu, acc, 1);
    const float refined = (den > 1e-12f && num > 0.0f) ? __fdiv_rn(num, den) : __fdiv_rn(max_abs, 127.0f);
    const uint16_t sb = bf16_rne_bits(refined);
    const float s_final = bf16_bits_to_f32(sb);
    const float inv_final = s_final > 1e-30f ? __fdiv_rn(1.0f, s_final) : 0.0f;
    *scale_bits = sb;
    s_idx[2 * lane] = (uint8_t)nf4_nearest_idx(__fmul_rn(v0, inv_final));
    s_idx[2 * lane + 1] = (uint8_t)nf4_nearest_idx(__fmul_rn(v1, inv_final));
    __syncwarp();
    const uint32_t h = lane / 16, i = lane % 16;       // byte j = 16h + i packs columns 32h+i (low) and 32h+16+i (high)
    const uint32_t byte = (uint32_t)s_idx[h * 32 + i] | ((uint32_t)s_idx[h * 32 + 16 + i] << 4);
    __syncwarp();
    return byte;
}

// ------------------------------------------------------------------------------------------------
// One query head, from the fused qkv vector to the int8 activation of o_proj, by one CTA of 256 threads, for
// contexts of up to ATTN_EXACT_CTX positions: bias, qk-norm, RoPE, rotation + int8 of the head's query and
// of its kv head's key and value (6609-6650, 8139-8178, 8303-8365, 9287-9326; the first query head of a
// group stores them in the cache), then causal_gqa_group_q8 (8471-8594) in the CPU's order - scores, maximum,
// exp (polynomial body in groups of 4, correctly rounded exp for the remainder), the 4-accumulator sum, one
// position-ascending fma chain per dimension - then the inverse rotation, the forward rotation with the
// global chunk index and the quantization for o_proj (7059-7084).  Bit for bit the CPU result.
// ------------------------------------------------------------------------------------------------
constexpr uint32_t ATTN_THREADS = 256;

struct AttnSmem {
    float *sc;                 // [ATTN_EXACT_CTX]
    int8_t *vbuf;              // [ATTN_EXACT_CTX][head_dim <= 128] cached value rows (one bulk copy)
    uint8_t *vt;               // [head_dim][ATTN_EXACT_CTX] the same rows transposed (value_rows_transpose); null: the chain reads vbuf bytes
    uint64_t *bar;             // mbarrier of that copy
    // kv_bits = 4 only
    float *wg;                 // [2][ATTN_EXACT_CTX] value weights per 64-value group
    float *cbf;                // [16] centroids as floats
    float *qs_val, *qs_c;      // [3][64] quantizer scratch per head warp
    uint8_t *qs_idx;           // [3][64]
    uint8_t *hq4;              // [2][64] packed key / value of the current position
    uint16_t *hs16;            // [2][2] their group scales
    float *head;               // [3][128] q / k / v head being processed
    int8_t *hq;                // [3][128] their int8 form
    float *hs;                 // [3] scales
    float *o;                  // [128]
    float *red;                // [32 words]
    float *inv;                // [1]
};
__host__ __device__ inline size_t attn_round(size_t v) { return (v + 127) & ~(size_t)127; }
constexpr uint32_t ATTN_VT_BYTES = 128 * ATTN_EXACT_CTX;
__host__ __device__ inline size_t attn_smem_bytes(bool staged = false) {
    return (staged ? ATTN_VT_BYTES : 0) + attn_round(2 * ATTN_EXACT_CTX * 4) + 128 + 2 * attn_round(3 * 64 * 4) + attn_round(3 * 64) + 128 + 128 +
           attn_round(ATTN_EXACT_CTX * 4) + attn_round(ATTN_EXACT_CTX * 128) + 128 + attn_round(3 * 128 * 4) + attn_round(3 * 128) + 128 +
           attn_round(128 * 4) + 128 + 128;
}
__device__ __forceinline__ AttnSmem attn_carve(uint8_t *base, bool staged = false) {
    AttnSmem s;
    size_t off = 0;
    s.vt = staged ? base : nullptr;
    if (staged) off += ATTN_VT_BYTES;
    s.sc = reinterpret_cast<float *>(base + off); off += attn_round(ATTN_EXACT_CTX * 4);
    s.vbuf = reinterpret_cast<int8_t *>(base + off); off += attn_round(ATTN_EXACT_CTX * 128);
    s.bar = reinterpret_cast<uint64_t *>(base + off); off += 128;
    s.wg = reinterpret_cast<float *>(base + off); off += attn_round(2 * ATTN_EXACT_CTX * 4);
    s.cbf = reinterpret_cast<float *>(base + off); off += 128;
    s.qs_val = reinterpret_cast<float *>(base + off); off += attn_round(3 * 64 * 4);
    s.qs_c = reinterpret_cast<float *>(base + off); off += attn_round(3 * 64 * 4);
    s.qs_idx = reinterpret_cast<uint8_t *>(base + off); off += attn_round(3 * 64);
    s.hq4 = reinterpret_cast<uint8_t *>(base + off); off += 128;
    s.hs16 = reinterpret_cast<uint16_t *>(base + off); off += 128;
    s.head = reinterpret_cast<float *>(base + off); off += attn_round(3 * 128 * 4);
    s.hq = reinterpret_cast<int8_t *>(base + off); off += attn_round(3 * 128);
    s.hs = reinterpret_cast<float *>(base + off); off += 128;
    s.o = reinterpret_cast<float *>(base + off); off += attn_round(128 * 4);
    s.red = reinterpret_cast<float *>(base + off); off += 128;
    s.inv = reinterpret_cast<float *>(base + off); off += 128;
    return s;
}


// ------------------------------------------------------------------------------------------------
// Transposed value tile.  The position-ascending fma chain of a dimension wants that dimension's bytes of consecutive
// positions side by side: one 16-byte shared-memory load then feeds sixteen chain steps (byte -> float by prmt + one
// subtraction), where the row-major cache rows cost a byte load per step.  Warps that are not on the chain transpose
// 16-position blocks in registers (4x4 byte transposes, eight prmt each).  Layout: row d (dimension) holds `stride`
// bytes; the 16-byte chunk of positions 16b..16b+15 sits at chunk index b ^ swz(d), swz(d) = (d ^ (d >> 3)) & 7, which
// keeps both sides free of bank conflicts (eight consecutive dimensions read eight different chunks; the eight lanes
// of a store phase, dimensions 4 apart, also do).  int8 rows are stored with the sign bit flipped (b ^ 0x80), NF4 rows as
// one byte per value holding 4 * index (the byte offset of its centroid in the fp32 table).
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t vt_swz(uint32_t d) { return (d ^ (d >> 3)) & 7u; }
__device__ __forceinline__ uint32_t lds_u32(uint32_t saddr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(saddr));
    return v;
}
__device__ __forceinline__ uint4 lds_u32x4(uint32_t saddr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(saddr));
    return v;
}
__device__ __forceinline__ void sts_u32x4(uint32_t saddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(saddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// w[0..3] = four positions x four dimensions (byte i of w[j] = dimension i of position j)  ->  t[i] = dimension i, positions 0..3
__device__ __forceinline__ void transpose4x4_bytes(const uint32_t w[4], uint32_t t[4]) {
    const uint32_t a = prmt(w[0], w[1], 0x5140u), b = prmt(w[2], w[3], 0x5140u);
    const uint32_t c = prmt(w[0], w[1], 0x7362u), d = prmt(w[2], w[3], 0x7362u);
    t[0] = prmt(a, b, 0x5410u); t[1] = prmt(a, b, 0x7632u);
    t[2] = prmt(c, d, 0x5410u); t[3] = prmt(c, d, 0x7632u);
}
// One warp transposes 16-position blocks blk0, blk0 + blk_step, ... < n_blk of the row-major rows at shared address
// `rows` (ROW bytes each: head_dim int8, or head_dim / 2 packed NF4 pairs) into the tile at `tile` (see above; block b of
// the source becomes chunk (b + chunk0) of the tile rows).  A lane takes one word column of the rows: head_dim / 4 lanes
// per block for int8, head_dim / 8 for NF4, so a warp works on 32 / that many blocks at a time.
template <int HD, bool KV4>
__device__ __forceinline__ void value_rows_transpose(uint32_t rows, uint32_t tile, uint32_t stride, uint32_t n_blk, uint32_t unit0,
                                                     uint32_t unit_step, uint32_t lane, uint32_t chunk0 = 0) {
    constexpr uint32_t ROW = KV4 ? HD / 2 : HD, LPB = ROW / 4, BPU = 32 / LPB, NOUT = KV4 ? 8 : 4;
    const uint32_t col = lane % LPB;
    // the NOUT tile rows this lane writes (dimension, swizzle) do not change from block to block
    uint32_t out_row[NOUT], out_swz[NOUT];
#pragma unroll
    for (uint32_t k = 0; k < NOUT; ++k) {
        uint32_t d;
        if (KV4) {      // bytes 4 col .. 4 col + 3 of a row: low nibbles = dimensions D .. D + 3, high nibbles = D + 16 .. D + 19
            const uint32_t B0 = 4 * col, D = (B0 / 32) * 64 + ((B0 / 16) % 2) * 32 + B0 % 16;
            d = D + 16 * (k / 4) + k % 4;
        } else {
            d = 4 * col + k;
        }
        out_row[k] = tile + d * stride;
        out_swz[k] = vt_swz(d);
    }
    // two units per round, the loads of both ahead of the byte shuffles of either: one unit alone is a chain of latencies
    // (sixteen loads, three levels of prmt, four stores: about 330 cycles for 90 instructions)
    auto load = [&](uint32_t b, uint32_t (&w)[16]) {
        const uint32_t src = rows + 16 * b * ROW + 4 * col;
#define K2T_LD_ROW(j) asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(w[j]) : "r"(src), "n"((j) * ROW))
        K2T_LD_ROW(0); K2T_LD_ROW(1); K2T_LD_ROW(2); K2T_LD_ROW(3); K2T_LD_ROW(4); K2T_LD_ROW(5); K2T_LD_ROW(6); K2T_LD_ROW(7);
        K2T_LD_ROW(8); K2T_LD_ROW(9); K2T_LD_ROW(10); K2T_LD_ROW(11); K2T_LD_ROW(12); K2T_LD_ROW(13); K2T_LD_ROW(14); K2T_LD_ROW(15);
#undef K2T_LD_ROW
    };
    auto emit = [&](uint32_t b, const uint32_t (&w)[16]) {
        const uint32_t chunk = b + chunk0, hi = (chunk & ~7u) << 4, lo = chunk & 7u;
#pragma unroll
        for (uint32_t half = 0; half < (KV4 ? 2u : 1u); ++half) {
            uint32_t t[4][4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t x[4], r[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    x[j] = KV4 ? (half ? (w[4 * q + j] >> 2) & 0x3C3C3C3Cu : (w[4 * q + j] << 2) & 0x3C3C3C3Cu) : w[4 * q + j] ^ 0x80808080u;
                transpose4x4_bytes(x, r);
#pragma unroll
                for (int i = 0; i < 4; ++i) t[i][q] = r[i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
                sts_u32x4(out_row[4 * half + i] + hi + ((lo ^ out_swz[4 * half + i]) << 4), t[i][0], t[i][1], t[i][2], t[i][3]);
        }
    };
    for (uint32_t u = unit0; u * BPU < n_blk; u += 2 * unit_step) {
        const uint32_t b0 = u * BPU + lane / LPB, b1 = (u + unit_step) * BPU + lane / LPB;
        const bool on0 = b0 < n_blk, on1 = b1 < n_blk;
        uint32_t w0[16], w1[16];
        if (on0) load(b0, w0);
        if (on1) load(b1, w1);
        if (on0) emit(b0, w0);
        if (on1) emit(b1, w1);
    }
}
// The softmax denominator's body (softmax_unnorm_neon's four-lane accumulator): lane i < 4 of the calling warp adds the
// terms 4k + i, k ascending - four chains that share one instruction stream, sixty-four positions requested ahead, so
// the loop runs at the latency of a dependent add - then (a0 + a1) + (a2 + a3).  `sa` = shared address of the terms,
// n4 = their count (a multiple of 4).  The result is valid in lane 0.
__device__ __forceinline__ float softmax_body_sum(uint32_t sa, uint32_t n4, uint32_t lane) {
    float acc = 0.0f;
    if (lane < 4) {
        const uint32_t base = sa + 4 * lane;
        uint32_t t = 0;
        float A[16], B[16];
#define K2T_LD_TERM(u) asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v[u]) : "r"(at), "n"(16 * (u)))
        auto load16 = [&](float (&v)[16], uint32_t t0) {
            const uint32_t at = base + 4 * t0;
            K2T_LD_TERM(0); K2T_LD_TERM(1); K2T_LD_TERM(2); K2T_LD_TERM(3); K2T_LD_TERM(4); K2T_LD_TERM(5); K2T_LD_TERM(6); K2T_LD_TERM(7);
            K2T_LD_TERM(8); K2T_LD_TERM(9); K2T_LD_TERM(10); K2T_LD_TERM(11); K2T_LD_TERM(12); K2T_LD_TERM(13); K2T_LD_TERM(14); K2T_LD_TERM(15);
        };
#undef K2T_LD_TERM
        auto add16 = [&](const float (&v)[16]) {
#pragma unroll
            for (int u = 0; u < 16; ++u) acc = __fadd_rn(acc, v[u]);
        };
        if (n4 >= 64) {
            load16(A, 0);
            for (;;) {          // A holds positions t .. t + 63
                if (t + 128 > n4) { add16(A); t += 64; break; }
                load16(B, t + 64); add16(A); t += 64;
                if (t + 128 > n4) { add16(B); t += 64; break; }
                load16(A, t + 64); add16(B); t += 64;
            }
        }
        for (; t < n4; t += 4) {
            float v;
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(base + 4 * t));
            acc = __fadd_rn(acc, v);
        }
    }
    acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 1));          // lane 0: a0 + a1, lane 2: a2 + a3
    acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 2));
    return acc;
}

// Sixteen chain steps of dimension d from one 16-byte chunk of its tile row: o = fma(value, weight, o), positions ascending.
// `n` < 16 stops after n steps (selects, no branches).  KV4: `cbfa` = shared address of the 16 fp32 centroids.
template <bool KV4>
__device__ __forceinline__ float value_chain16(float o, const uint4 x, const float4 w0, const float4 w1, const float4 w2, const float4 w3,
                                               uint32_t cbfa, uint32_t n = 16) {
    const uint32_t xs[4] = {x.x, x.y, x.z, x.w};
    const float ws[16] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w, w2.x, w2.y, w2.z, w2.w, w3.x, w3.y, w3.z, w3.w};
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        float v;
        if (KV4) {
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(cbfa + prmt(xs[k / 4], 0u, 0x4440u + (k % 4))));
        } else {
            // 0x4B000000 | (b ^ 0x80) is the float 2^23 + 128 + (int8)b: subtracting 2^23 + 128 converts without the conversion unit
            v = __fsub_rn(__uint_as_float(prmt(xs[k / 4], 0x4B000000u, 0x7440u + (k % 4))), 8388736.0f);
        }
        const float r = __fmaf_rn(v, ws[k], o);
        o = (uint32_t)k < n ? r : o;
    }
    return o;
}

#define ATTN_MARK(i) do { if (A.trace != nullptr && qh == 0 && threadIdx.x == 0) A.trace[i] = (unsigned long long)clock64(); } while (0)

template <int HD, bool KV4, bool STAGED>
__device__ __noinline__ void attention_head_cta(const FusedAttnArgs &A, uint32_t qh, uint32_t pos, const AttnSmem &s, int pdl_mode) {
    // pdl_mode: 0 = not a programmatic dependent (whole-token kernel), 1 = the caller has waited for the predecessor,
    // 2 = the wait is in here, after the prefetch of everything older launches wrote.  In modes 1 and 2 the successor
    // is released before the value chain, not at the start: CTAs that sit on an SM waiting for their predecessor slow
    // the warps running there (this kernel's phases took a third longer with the next projection's CTAs resident from
    // the start), and the successor needs only a microsecond or two of lead for its first weight stages.
    constexpr int QW = HD / 4, NB = HD / 64;
    constexpr uint32_t NT = ATTN_THREADS, NW = ATTN_THREADS / 32;
    constexpr uint32_t ROW = KV4 ? HD / 2 : HD;            // bytes of one cached key / value row
    // The work areas arrive as generic pointers; telling the compiler that they are shared memory turns every access into
    // a shared-memory instruction (generic loads of shared memory cost several times the latency: the value chain below
    // ran at 40 cycles per position with them).
    __builtin_assume(__isShared(s.sc)); __builtin_assume(__isShared(s.vbuf)); __builtin_assume(__isShared(s.head));
    __builtin_assume(__isShared(s.hq)); __builtin_assume(__isShared(s.hs)); __builtin_assume(__isShared(s.o));
    __builtin_assume(__isShared(s.red)); __builtin_assume(__isShared(s.inv)); __builtin_assume(__isShared(s.bar));
    __builtin_assume(__isShared(s.wg)); __builtin_assume(__isShared(s.cbf)); __builtin_assume(__isShared(s.qs_val));
    __builtin_assume(__isShared(s.qs_c)); __builtin_assume(__isShared(s.qs_idx)); __builtin_assume(__isShared(s.hq4));
    __builtin_assume(__isShared(s.hs16));
    if (STAGED) __builtin_assume(__isShared(s.vt));
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t group = A.n_q / A.n_kv, kvh = qh / group, ctx = pos + 1, layer = A.layer;
    const size_t slot0 = ((size_t)layer * A.n_kv + kvh) * A.max_seq;
    const uint8_t *K = reinterpret_cast<const uint8_t *>(A.k_q8) + slot0 * ROW, *V = reinterpret_cast<const uint8_t *>(A.v_q8) + slot0 * ROW;
    // scales: one fp32 per slot (int8 cache) or NB bf16 per slot (NF4 cache)
    const float *ks = A.k_scale + slot0, *vs = A.v_scale + slot0;
    const uint16_t *ks16 = reinterpret_cast<const uint16_t *>(A.k_scale) + slot0 * NB, *vs16 = reinterpret_cast<const uint16_t *>(A.v_scale) + slot0 * NB;
    // ---- everything that does not depend on the current token is requested first, so that its L2 latency
    // overlaps the head preparation.  First of all (its fences would otherwise wait for the loads below) the
    // cached value rows [0, pos): they are contiguous, so one bulk copy into shared memory, completion on an
    // mbarrier; then this lane's head inputs, and the key rows and scales of this thread's (at most two)
    // cached positions.
    const uint32_t vbar = (uint32_t)__cvta_generic_to_shared(s.bar);
    ATTN_MARK(0);
    if (tid == NT - 32 && pos > 0) {       // a warp that has nothing to do during the head preparation: its fences delay nobody
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(vbar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async;" ::: "memory");       // barrier init, and the cache rows other CTAs / kernels stored
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(vbar), "r"(pos * ROW) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"((uint32_t)__cvta_generic_to_shared(s.vbuf)), "l"(V), "r"(pos * ROW), "r"(vbar) : "memory");
    }
    if (KV4 && tid < 16) s.cbf[tid] = NF4_KV_CENTROIDS[tid];
    constexpr int HV = HD / 32;                            // head elements per lane (warps 0..2)
    const uint32_t my_head = warp == 0 ? qh : warp == 1 ? A.n_q + kvh : A.n_q + A.n_kv + kvh;
    float hv[HV], hb[HV], rc[HV], rs[HV];                  // head values, their bias, rope cos / sin of the lane's pair
    FwhtSigns sg_head[NB], sg_out_inv, sg_out_fwd;         // rotation signs: of the head's blocks (warps 0..2), of the output chunk (warps < NB)
#pragma unroll
    for (int b = 0; b < NB; ++b) sg_head[b] = fwht_signs(b, lane);
    sg_out_inv = fwht_signs(warp, lane);
    sg_out_fwd = fwht_signs(A.out_chunk0 + qh * NB + warp, lane);
    if (warp < 3) {
#pragma unroll
        for (int k = 0; k < HV; ++k) {
            const uint32_t i = lane + 32 * k;
            hb[k] = A.bias != nullptr ? __ldg(A.bias + (size_t)my_head * HD + i) : 0.0f;
            rc[k] = __ldg(A.rope + (size_t)pos * HD + (i % (HD / 2)));
            rs[k] = __ldg(A.rope + (size_t)pos * HD + HD / 2 + (i % (HD / 2)));
        }
    }
    constexpr int PT = ATTN_EXACT_CTX / ATTN_THREADS;     // positions per thread
    constexpr int KR = ROW / 16;                           // int4 per key row
    int4 kreg[PT][KR];
    float ksr[PT][KV4 ? NB : 1], vsr[PT][KV4 ? NB : 1];
#pragma unroll
    for (int k = 0; k < PT; ++k) {
        const uint32_t t = tid + k * NT;
        const bool cached = t < pos;
#pragma unroll
        for (int i = 0; i < KR; ++i)
            kreg[k][i] = cached ? __ldcg(reinterpret_cast<const int4 *>(K + (size_t)t * ROW) + i) : make_int4(0, 0, 0, 0);
        if (KV4) {
#pragma unroll
            for (int g = 0; g < NB; ++g) {
                ksr[k][g] = cached ? bf16_bits_to_f32(__ldcg(ks16 + (size_t)t * NB + g)) : 0.0f;
                vsr[k][g] = cached ? bf16_bits_to_f32(__ldcg(vs16 + (size_t)t * NB + g)) : 0.0f;
            }
        } else {
            ksr[k][0] = cached ? __ldcg(ks + t) : 0.0f;
            vsr[k][0] = cached ? __ldcg(vs + t) : 0.0f;
        }
    }
    // Everything above reads what earlier steps (or a launch at least two back) wrote; the projection output below is the
    // predecessor's.
    if (pdl_mode == 2) pdl_wait();
    ATTN_MARK(1);
    if (warp < 3) {
#pragma unroll
        for (int k = 0; k < HV; ++k) {
            hv[k] = __ldcg(A.qkv + (size_t)my_head * HD + lane + 32 * k);
            if (A.bias != nullptr) hv[k] = __fadd_rn(hv[k], hb[k]);
        }
    }
    // ---- the three heads of this CTA: warp 0 = query qh, warp 1 = key kvh, warp 2 = value kvh
    if (warp < 3) {
        float *sh = s.head + warp * 128;
#pragma unroll
        for (int k = 0; k < HV; ++k) sh[lane + 32 * k] = hv[k];
        __syncwarp();
        const float *norm_w = warp == 0 ? A.q_norm : (warp == 1 ? A.k_norm : nullptr);
        auto do_rope = [&]() {       // element i pairs with i +- hd/2: x0' = x0 c - x1 s, x1' = x1 c + x0 s
            float nv[HV];
#pragma unroll
            for (int k = 0; k < HV; ++k) {
                const uint32_t i = lane + 32 * k;
                const float me = sh[i], other = sh[i < HD / 2 ? i + HD / 2 : i - HD / 2];
                nv[k] = i < HD / 2 ? __fsub_rn(__fmul_rn(me, rc[k]), __fmul_rn(other, rs[k]))
                                   : __fadd_rn(__fmul_rn(me, rc[k]), __fmul_rn(other, rs[k]));
            }
            __syncwarp();
#pragma unroll
            for (int k = 0; k < HV; ++k) sh[lane + 32 * k] = nv[k];
            __syncwarp();
        };
        auto do_norm = [&]() {
            float ss = 0.0f;
            if (lane < 16)
                for (uint32_t i = lane; i < HD; i += 16) ss = __fmaf_rn(sh[i], sh[i], ss);
            ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, 4));
            ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, 8));
            ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, 1));
            ss = __fadd_rn(ss, __shfl_down_sync(0xffffffffu, ss, 2));
            ss = __shfl_sync(0xffffffffu, ss, 0);
            const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(ss, __fdiv_rn(1.0f, (float)HD)), A.eps)));
            for (uint32_t i = lane; i < HD; i += 32) sh[i] = __fmul_rn(__fmul_rn(sh[i], inv), __ldg(norm_w + i));
            __syncwarp();
        };
        if (warp < 2) {
#pragma unroll 1
            for (int step = 0; step < 2; ++step) {       // rolled: one copy of each in the code
                if ((step == 0) == (A.qk_norm_after_rope != 0)) do_rope();
                else if (norm_w != nullptr) do_norm();
            }
        }
        float v0[NB], v1[NB], mx = 0.0f;
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            v0[b] = sh[b * 64 + 2 * lane];
            v1[b] = sh[b * 64 + 2 * lane + 1];
            warp_fwht64(v0[b], v1[b], sg_head[b], lane);
            mx = fmaxf(mx, fmaxf(fabsf(v0[b]), fabsf(v1[b])));
        }
        const bool store = warp > 0 && qh % group == 0;     // one CTA of the group writes the cache entry
        if (KV4 && warp > 0) {       // NF4 key / value: per 64-value group a refined bf16 scale and packed indices
            uint8_t *cache = const_cast<uint8_t *>(warp == 1 ? K : V) + (size_t)pos * ROW;
            uint16_t *cache_s = const_cast<uint16_t *>(warp == 1 ? ks16 : vs16) + (size_t)pos * NB;
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                uint16_t sb;
                const uint32_t byte = warp_quant64_q4(v0[b], v1[b], lane, s.qs_val + warp * 64, s.qs_c + warp * 64, s.qs_idx + warp * 64, &sb);
                s.hq4[(warp - 1) * 64 + b * 32 + lane] = (uint8_t)byte;
                if (store) cache[b * 32 + lane] = (uint8_t)byte;
                if (lane == 0) {
                    s.hs16[(warp - 1) * 2 + b] = sb;
                    if (store) cache_s[b] = sb;
                }
            }
        } else {                     // int8 with one scale for the whole head (queries always)
            mx = warp_max(mx);
            const bool zero = mx <= 1.1920929e-07f;
            const float inv = zero ? 0.0f : __fdiv_rn(127.0f, mx), scale = zero ? 0.0f : __fdiv_rn(mx, 127.0f);
            int8_t *cache = reinterpret_cast<int8_t *>(const_cast<uint8_t *>(warp == 1 ? K : V)) + (size_t)pos * HD;
            // value rows also go to the block-transposed copy the long-context chains read (ExactAttnArgs.v_t)
            int8_t *vt = (store && warp == 2 && A.v_t != nullptr) ? A.v_t + slot0 * HD + (size_t)(pos / 16) * HD * 16 + pos % 16 : nullptr;
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                const int q0 = zero ? 0 : __float2int_rn(__fmul_rn(v0[b], inv)), q1 = zero ? 0 : __float2int_rn(__fmul_rn(v1[b], inv));
                const char2 pk = make_char2((signed char)q0, (signed char)q1);
                reinterpret_cast<char2 *>(s.hq + warp * 128 + b * 64)[lane] = pk;
                if (store) reinterpret_cast<char2 *>(cache + b * 64)[lane] = pk;
                if (vt != nullptr) {
                    vt[(b * 64 + 2 * lane) * 16] = (int8_t)(q0 ^ 0x80);
                    vt[(b * 64 + 2 * lane + 1) * 16] = (int8_t)(q1 ^ 0x80);
                }
            }
            if (lane == 0) {
                s.hs[warp] = scale;
                if (store) const_cast<float *>(warp == 1 ? ks : vs)[pos] = scale;
            }
        }
    }
    ATTN_MARK(2);
    __syncthreads();
    ATTN_MARK(3);
    // ---- scores (positions < pos from the prefetched cache rows, position pos from shared memory)
    const float qas = __fmul_rn(s.hs[0], A.attn_scale);
    int qw[QW];
    if (KV4) {
        // a packed word holds columns (i, 16+i, i+1, 16+i+1 | i+2, 16+i+2, i+3, 16+i+3) of a 32-column half in its
        // eight nibbles: the query bytes are gathered in that order once
#pragma unroll
        for (int g = 0; g < NB; ++g)
#pragma unroll
            for (int w = 0; w < 8; ++w) {
                const int8_t *qb = s.hq + g * 64 + (w / 4) * 32 + 4 * (w % 4);
#pragma unroll
                for (int u = 0; u < 2; ++u)
                    qw[g * 16 + 2 * w + u] = (int)((uint32_t)(uint8_t)qb[2 * u] | ((uint32_t)(uint8_t)qb[16 + 2 * u] << 8) |
                                                   ((uint32_t)(uint8_t)qb[2 * u + 1] << 16) | ((uint32_t)(uint8_t)qb[16 + 2 * u + 1] << 24));
            }
    } else {
#pragma unroll
        for (int i = 0; i < QW; ++i) qw[i] = reinterpret_cast<const int *>(s.hq)[i];
    }
    float mx = -INFINITY, scr[PT];
#pragma unroll
    for (int k = 0; k < PT; ++k) {
        const uint32_t t = tid + k * NT;
        scr[k] = -INFINITY;
        if (t < ctx) {
            if (KV4) {        // causal_gqa_group_q4_or_window (8794-8988): total += ((dot * ks_g) * q_s) per 64-value group
                float total = 0.0f;
#pragma unroll
                for (int g = 0; g < NB; ++g) {
                    int up = 0, dn = 0;
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const int4 v = t < pos ? kreg[k][2 * g + i] : reinterpret_cast<const int4 *>(s.hq4 + g * 32)[i];
                        const uint32_t xw[4] = {(uint32_t)v.x, (uint32_t)v.y, (uint32_t)v.z, (uint32_t)v.w};
#pragma unroll
                        for (int w = 0; w < 4; ++w) {
                            const uint32_t x = xw[w], y = x ^ 0x88888888u;
                            const int q0 = qw[g * 16 + 2 * (4 * i + w)], q1 = qw[g * 16 + 2 * (4 * i + w) + 1];
                            up = dp4a_us(prmt(NF4_KV_HI0, NF4_KV_HI1, y), q0, up);
                            dn = dp4a_us(prmt(NF4_KV_LO0, NF4_KV_LO1, x), q0, dn);
                            up = dp4a_us(prmt(NF4_KV_HI0, NF4_KV_HI1, y >> 16), q1, up);
                            dn = dp4a_us(prmt(NF4_KV_LO0, NF4_KV_LO1, x >> 16), q1, dn);
                        }
                    }
                    const float ksg = t < pos ? ksr[k][g] : bf16_bits_to_f32(s.hs16[g]);
                    total = __fadd_rn(total, __fmul_rn(__fmul_rn((float)(up - dn), ksg), qas));
                }
                scr[k] = total;
            } else {
                int dot = 0;
#pragma unroll
                for (int i = 0; i < QW / 4; ++i) {
                    const int4 v = t < pos ? kreg[k][i] : reinterpret_cast<const int4 *>(s.hq + 128)[i];
                    dot = __dp4a(v.x, qw[4 * i], dot); dot = __dp4a(v.y, qw[4 * i + 1], dot);
                    dot = __dp4a(v.z, qw[4 * i + 2], dot); dot = __dp4a(v.w, qw[4 * i + 3], dot);
                }
                // 256-position tiles: whole groups of 8 use dot*(ks*qas), the tile remainder (dot*ks)*qas (8992-9057)
                const uint32_t tile0 = t & ~255u, tile_n = min(ctx, tile0 + 256u) - tile0;
                const float kst = t < pos ? ksr[k][0] : s.hs[1];
                scr[k] = (t - tile0 < (tile_n & ~7u)) ? __fmul_rn((float)dot, __fmul_rn(kst, qas))
                                                       : __fmul_rn(__fmul_rn((float)dot, kst), qas);
            }
            mx = fmaxf(mx, scr[k]);
        }
    }
    mx = warp_max(mx);
    if (lane == 0) s.red[warp] = mx;
    __syncthreads();
    ATTN_MARK(4);
#pragma unroll
    for (int i = 0; i < (int)NW; ++i) mx = fmaxf(mx, s.red[i]);
    // softmax_unnorm (9603-9632): polynomial exp for whole groups of 4 positions, libm exp for the rest
    // (correctly rounded: double exp rounded to float; those run while warp 0 sums the body)
    const uint32_t n4 = ctx & ~3u;
#pragma unroll
    for (int k = 0; k < PT; ++k) {
        const uint32_t t = tid + k * NT;
        if (t < n4) s.sc[t] = exp_poly(__fsub_rn(scr[k], mx));
    }
    __syncthreads();
    ATTN_MARK(5);
    // warp 0 sums the body while at most three other threads evaluate the remainder's exps and warps 1.. transpose the
    // cached value rows for the chain below
    float acc = 0.0f;
    bool copy_failed = false;
    if (warp == 0) acc = softmax_body_sum((uint32_t)__cvta_generic_to_shared(s.sc), n4, lane);
    ATTN_MARK(6);
    {
        // the remainder's exps (at most three positions; thread 0 gets to its own, if any, after the sum)
        float tail_x = 0.0f;
        uint32_t tail_t = 0xffffffffu;
#pragma unroll
        for (int k = 0; k < PT; ++k) {
            const uint32_t t = tid + k * NT;
            if (t >= n4 && t < ctx) { tail_t = t; tail_x = __fsub_rn(scr[k], mx); }
        }
        if (tail_t != 0xffffffffu) s.sc[tail_t] = (float)exp((double)tail_x);
    }
    if (STAGED && warp > 0 && pos > 0) {           // bounded wait for the bulk copy of the value rows, then the transposition
        uint32_t ok = 0;
        for (uint32_t spin = 0; spin < (1u << 22) && !ok; ++spin) ok = mbar_try_wait(vbar, 0);
        copy_failed = !ok;
        if (ok)
            value_rows_transpose<HD, KV4>((uint32_t)__cvta_generic_to_shared(s.vbuf), (uint32_t)__cvta_generic_to_shared(s.vt), ATTN_EXACT_CTX,
                                          (pos + 15) / 16, warp - 1, NW - 1, lane);
    }
    __syncthreads();
    ATTN_MARK(7);
    if (tid == 0) {
        for (uint32_t t = n4; t < ctx; ++t) acc = __fadd_rn(acc, s.sc[t]);
        *s.inv = __fdiv_rn(1.0f, acc);
    }
    __syncthreads();
    ATTN_MARK(8);
    const float inv = *s.inv;
#pragma unroll
    for (int k = 0; k < PT; ++k) {
        const uint32_t t = tid + k * NT;
        if (t < ctx) {
            const float p_norm = __fmul_rn(s.sc[t], inv);
            if (KV4) {
#pragma unroll
                for (int g = 0; g < NB; ++g)
                    s.wg[g * ATTN_EXACT_CTX + t] = __fmul_rn(p_norm, t < pos ? vsr[k][g] : bf16_bits_to_f32(s.hs16[2 + g]));
            } else {
                s.sc[t] = __fmul_rn(p_norm, t < pos ? vsr[k][0] : s.hs[2]);
            }
        }
    }
    // ---- values: thread i < HD = dimension i runs the position-ascending chain over the staged rows
    __syncthreads();                       // weights complete
    if (pdl_mode != 0) pdl_trigger();
    ATTN_MARK(9);
    float o = 0.0f;
    if (pos > 0 && !STAGED) {              // bounded wait for the bulk copy (the transposers have waited already where there is a tile)
        uint32_t ok = 0;
        for (uint32_t spin = 0; spin < (1u << 22) && !ok; ++spin)
            asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(vbar) : "memory");
        copy_failed = !ok;
    }
    copy_failed = __syncthreads_or(copy_failed) != 0;      // the same verdict in every thread (there are barriers below)
    if (copy_failed && tid == 0 && A.err_flag != nullptr) atomicExch(A.err_flag, 1u);
    ATTN_MARK(10);
    if (STAGED) {
        if (tid < HD && !copy_failed) {
            const uint32_t row = (uint32_t)__cvta_generic_to_shared(s.vt) + tid * ATTN_EXACT_CTX, fd = vt_swz(tid);
            const uint32_t wa = (uint32_t)__cvta_generic_to_shared(KV4 ? s.wg + (tid / 64) * ATTN_EXACT_CTX : s.sc);
            const uint32_t cbfa = (uint32_t)__cvta_generic_to_shared(s.cbf);
            const uint32_t n_full = pos / 16, rem = pos % 16;
            auto chunk_at = [&](uint32_t b) { return row + (((b & ~7u) | ((b ^ fd) & 7u)) << 4); };
            uint4 x = make_uint4(0, 0, 0, 0);
            float4 w0 = make_float4(0, 0, 0, 0), w1 = w0, w2 = w0, w3 = w0;
            if (pos > 0) {
                x = lds_u32x4(chunk_at(0));
                w0 = lds_f32x4(wa); w1 = lds_f32x4(wa + 16); w2 = lds_f32x4(wa + 32); w3 = lds_f32x4(wa + 48);
            }
            for (uint32_t b = 0; b < n_full; ++b) {
                // the next block's bytes and weights are requested before this block's sixteen steps (the last request may
                // read the partial block or, at pos = 512, one chunk of the next row: in bounds, unused)
                const uint32_t nb = b + 1 < ATTN_EXACT_CTX / 16 ? b + 1 : b;
                const uint4 xn = lds_u32x4(chunk_at(nb));
                const float4 n0 = lds_f32x4(wa + 64 * nb), n1 = lds_f32x4(wa + 64 * nb + 16), n2 = lds_f32x4(wa + 64 * nb + 32), n3 = lds_f32x4(wa + 64 * nb + 48);
                o = value_chain16<KV4>(o, x, w0, w1, w2, w3, cbfa);
                x = xn; w0 = n0; w1 = n1; w2 = n2; w3 = n3;
            }
            if (rem != 0) o = value_chain16<KV4>(o, x, w0, w1, w2, w3, cbfa, rem);
            // the current position: its value row is still in the head area
            if (KV4) {
                const uint32_t g = tid / 64, e = tid % 64, r = e % 32;
                const uint32_t byte_off = g * 32 + (e / 32) * 16 + (r % 16), shift = r < 16 ? 0u : 4u;
                o = __fmaf_rn(s.cbf[(s.hq4[64 + byte_off] >> shift) & 15u], s.wg[g * ATTN_EXACT_CTX + pos], o);
            } else {
                const uint32_t b = reinterpret_cast<const uint8_t *>(s.hq)[256 + tid];
                o = __fmaf_rn(__fsub_rn(__uint_as_float(b ^ 0x4B000080u), 8388736.0f), s.sc[pos], o);
            }
        }
    } else if (tid < HD && !copy_failed) {
        // a zero weight skips the position (as the CPU loop does): select, not branch.  Eight positions are
        // loaded before their fma chain starts, so the chain runs at fma latency, not shared-memory latency.
        if (KV4) {
            const uint32_t g = tid / 64, e = tid % 64, r = e % 32;
            const uint32_t byte_off = g * 32 + (e / 32) * 16 + (r % 16), shift = r < 16 ? 0u : 4u;
            const float *wp = s.wg + g * ATTN_EXACT_CTX;
            const uint8_t *vp = reinterpret_cast<const uint8_t *>(s.vbuf) + byte_off;
            // plain fma for every position (a zero weight adds +-0: same bits as the CPU's skip), next eight positions
            // loaded while the current eight run
            uint32_t j = 0;
            float w[8], c[8], wn[8], cn[8];
            if (pos >= 8) {
#pragma unroll
                for (int u = 0; u < 8; ++u) { w[u] = wp[u]; c[u] = s.cbf[(vp[u * ROW] >> shift) & 15u]; }
            }
            for (; j + 16 <= pos; j += 8) {
#pragma unroll
                for (int u = 0; u < 8; ++u) { wn[u] = wp[j + 8 + u]; cn[u] = s.cbf[(vp[(j + 8 + u) * ROW] >> shift) & 15u]; }
#pragma unroll
                for (int u = 0; u < 8; ++u) o = __fmaf_rn(c[u], w[u], o);
#pragma unroll
                for (int u = 0; u < 8; ++u) { w[u] = wn[u]; c[u] = cn[u]; }
            }
            if (j + 8 <= pos) {
#pragma unroll
                for (int u = 0; u < 8; ++u) o = __fmaf_rn(c[u], w[u], o);
                j += 8;
            }
            for (; j < pos; ++j) o = __fmaf_rn(s.cbf[(vp[j * ROW] >> shift) & 15u], wp[j], o);
            // the current position: its value row is still in shared memory
            o = __fmaf_rn(s.cbf[(s.hq4[64 + byte_off] >> shift) & 15u], wp[pos], o);
        } else {
            // int8 -> fp32 without the conversion unit (a quarter-rate pipe that would bound this loop): for a byte b,
            // 0x4B000000 | (b ^ 0x80) is the float 2^23 + (int8)b + 128, so subtracting 2^23 + 128 gives (float)(int8)b exactly.
            // The CPU loop skips positions whose weight is zero; the plain fma gives the same bits (w >= 0 and the values
            // are finite: o + (+-0) = o, and +0 + (-0) = +0), so the chain is one fma per position.
            // Every thread reads the byte of its own dimension; sixteen positions (and their weights) are loaded while the
            // sixteen before them run through the chain, so the chain never waits for shared memory (measured 8.3 cycles
            // per position against 4.5 for the bare fma chain; a variant that fetched words for four positions and
            // handed them round by shuffle ran at 18 or more).
            const float *wp = s.sc;
            const uint8_t *vb = reinterpret_cast<const uint8_t *>(s.vbuf);
            auto to_f32 = [](uint32_t b) { return __fsub_rn(__uint_as_float(b ^ 0x4B000080u), 8388736.0f); };
            const uint32_t vt = (uint32_t)__cvta_generic_to_shared(vb) + tid, wa = (uint32_t)__cvta_generic_to_shared(wp);
            uint32_t j = 0;
            if (pos >= 16) {
                uint32_t cur[16], nxt[16];
                float4 wc[4], wn[4];
#pragma unroll
                for (int u = 0; u < 16; ++u) cur[u] = lds_u8(vt + u * HD);
#pragma unroll
                for (int u = 0; u < 4; ++u) wc[u] = lds_f32x4(wa + 16 * u);
                for (; j + 32 <= pos; j += 16) {
#pragma unroll
                    for (int u = 0; u < 16; ++u) nxt[u] = lds_u8(vt + (j + 16 + u) * HD);
#pragma unroll
                    for (int u = 0; u < 4; ++u) wn[u] = lds_f32x4(wa + 4 * (j + 16) + 16 * u);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        o = __fmaf_rn(to_f32(cur[4 * u + 0]), wc[u].x, o);
                        o = __fmaf_rn(to_f32(cur[4 * u + 1]), wc[u].y, o);
                        o = __fmaf_rn(to_f32(cur[4 * u + 2]), wc[u].z, o);
                        o = __fmaf_rn(to_f32(cur[4 * u + 3]), wc[u].w, o);
                    }
#pragma unroll
                    for (int u = 0; u < 16; ++u) cur[u] = nxt[u];
#pragma unroll
                    for (int u = 0; u < 4; ++u) wc[u] = wn[u];
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    o = __fmaf_rn(to_f32(cur[4 * u + 0]), wc[u].x, o);
                    o = __fmaf_rn(to_f32(cur[4 * u + 1]), wc[u].y, o);
                    o = __fmaf_rn(to_f32(cur[4 * u + 2]), wc[u].z, o);
                    o = __fmaf_rn(to_f32(cur[4 * u + 3]), wc[u].w, o);
                }
                j += 16;
            }
            for (; j < pos; ++j) o = __fmaf_rn(to_f32(vb[(size_t)j * HD + tid]), wp[j], o);
            // the current position: its value row is still in shared memory
            o = __fmaf_rn(to_f32(reinterpret_cast<const uint8_t *>(s.hq)[256 + tid]), wp[pos], o);
        }
    }
    ATTN_MARK(11);
    __syncthreads();
    ATTN_MARK(12);
    if (tid < HD) s.o[tid] = o;
    __syncthreads();
    if (warp < NB) {
        const uint32_t b = warp;
        float x0 = s.o[b * 64 + 2 * lane], x1 = s.o[b * 64 + 2 * lane + 1];
        warp_ifwht64(x0, x1, sg_out_inv, lane);
        if (A.attn_tap != nullptr) reinterpret_cast<float2 *>(A.attn_tap + (size_t)qh * HD + b * 64)[lane] = make_float2(x0, x1);
        const uint32_t c = qh * NB + b;
        warp_fwht64(x0, x1, sg_out_fwd, lane);
        int q0, q1, sum;
        float sc;
        warp_quant64(x0, x1, q0, q1, sc, sum);
        reinterpret_cast<char2 *>(A.out_q + (size_t)c * 64)[lane] = make_char2((signed char)q0, (signed char)q1);
        if (lane == 0) { A.out_scales[c] = sc; A.out_sums[c] = sum; }
    }
    ATTN_MARK(13);
    // the barrier's memory is initialised again by the next call on this shared memory (the whole-token kernel)
    if (tid == NT - 32 && pos > 0) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(vbar) : "memory");
}

// runtime dispatch on head_dim / cache format
template <bool STAGED>
__device__ __forceinline__ void attention_head_dispatch(const FusedAttnArgs &A, uint32_t qh, uint32_t pos, const AttnSmem &s, int pdl_mode = 0) {
    if (A.kv_bits == 4) {
        if (A.head_dim == 64) attention_head_cta<64, true, STAGED>(A, qh, pos, s, pdl_mode);
        else attention_head_cta<128, true, STAGED>(A, qh, pos, s, pdl_mode);
    } else {
        if (A.head_dim == 64) attention_head_cta<64, false, STAGED>(A, qh, pos, s, pdl_mode);
        else attention_head_cta<128, false, STAGED>(A, qh, pos, s, pdl_mode);
    }
}

}  // namespace k2t

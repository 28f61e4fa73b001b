// Quantized GEMV (batch 1) and small-N GEMM (2..4 tokens per pass) for bit-plane (b4/b5/b6) and
// codebook (NF4/NF3) matrices.
//
// Arithmetic contract (reference: sdot_one_stripe_neon, src/kernels/simd_lut.rs:3763-3868, and
// nf_sdot_one_stripe_neon, 6071-6181; batch forms 4228-4331 / 6689-7029):
//   per row r and 64-column chunk c:  a = sum_i code_i * q_i           (exact int32)
//       bit-plane: dot = 2a - (2^B-1) * xsum[c]      NF: dot = a
//   f = 0;  for c ascending, skipping chunks with xs[c] == 0:
//       f = fmaf((float)dot * xs[c], w_scale[r, c / sgc], f)
// The integer dots are computed by all lanes in parallel; the fp32 chain runs per row in ascending
// chunk order, so outputs are bit-identical to the reference order.
//
// Mapping.  A lane owns a CELL (one row x one 64-column chunk) at a time.  In a warp, lane l works on
// chunk 32p + l of the current pass p, so the int8 activations of that chunk (64 B), their scale and
// their sum stay in the lane's registers while the warp walks down its rows: the inner loop touches
// no shared memory for activations.  Warps are independent (one warp per CTA, persistent grid): warp
// w owns the 4-row blocks w, w + W, w + 2W, ... and works through them 8 blocks (32 rows) at a time.
//
// Weight streaming.  Each warp runs its own bulk-copy pipeline: a stage receives the cells of one
// 4-row block for one pass (16-byte half cells of columns 0..31 and 32..63, the extra-bit plane and
// the bf16 scales; the pass-tiled image makes each of them ONE contiguous run, so a stage is three or
// four `cp.async.bulk` copies) and signals an mbarrier with the byte count.  NSTAGE stages per warp keep 9..13 KiB per warp in flight without holding a register; the
// stage is refilled right after its four rows have been reduced.  Cells are 16 bytes apart in a
// stage, so the 128-bit shared-memory reads of a warp are conflict-free.
//
// Chain.  Every cell parks (v, w_scale) in a [32 rows][32 chunks] shared-memory tile; after the
// eight blocks of a pass, lane i continues the fp32 chain of row i over the 32 chunks of that pass
// (f stays in a register between passes), which keeps the reference's ascending-chunk order.
#pragma once
#include "k2t_device.cuh"
#include "k2t_kernels.h"

namespace k2t {

struct GemvArgs {
    const uint8_t *plane[3];  // code planes in pass tiles (k2t_layout.h)
    const uint16_t *scales;   // scale plane in pass tiles
    const int8_t *xq;
    const float *xs;
    const int32_t *xsum;
    float *out;
    int32_t *int_dots;
    uint32_t *err_flag;       // set to 1 when a bounded mbarrier wait gives up
    size_t out_stride;
    uint32_t rows, rows_pad, cols, nc, nsg, sgc, sgc_shift, n_tok;  // sgc_shift: log2(sgc) or 32
    int32_t max_odd;
    int32_t nf4_offset;
    uint32_t cb[8];    // expanded codebook, 4 centroids per word (NF4: sorted ascending)
    uint32_t tab[4];   // NF4 two-table decode: hi[0..3], hi[4..7], lo[0..3], lo[4..7]
    uint32_t pdl;      // host side only: launch as a programmatic dependent
};

constexpr int FMT_NF4G = FMT_COUNT;   // NF4 with a codebook the two-table decode cannot represent

// bytes per cell in each code plane, and the words of a cell a lane holds (plane 0, 1, 2 in order)
template <int FMT> struct Cell { static constexpr int B0 = 16, B1 = 16, B2 = 0; };
template <> struct Cell<FMT_BP5> { static constexpr int B0 = 16, B1 = 16, B2 = 8; };
template <> struct Cell<FMT_BP6> { static constexpr int B0 = 16, B1 = 16, B2 = 16; };
template <> struct Cell<FMT_NF3> { static constexpr int B0 = 16, B1 = 8, B2 = 0; };
template <> struct Cell<FMT_NF5> { static constexpr int B0 = 16, B1 = 16, B2 = 8; };
template <> struct Cell<FMT_E8Q2> { static constexpr int B0 = 16, B1 = 0, B2 = 0; };

__device__ __forceinline__ uint32_t *e8q2_templates_smem() {
    __shared__ uint32_t tab[32];
    return tab;
}
// four flag bits (bit i -> byte i) as a byte mask 0xFF / 0x00
__device__ __forceinline__ uint32_t spread4(uint32_t bits4) { return ((bits4 * 0x00204081u) & 0x01010101u) * 0xFFu; }

template <int FMT>
struct Raw {
    uint32_t w[(Cell<FMT>::B0 + Cell<FMT>::B1 + Cell<FMT>::B2) / 4];
};

// Expands a cell into 16 words of four weight bytes each: u[j] holds columns 4j..4j+3 of the chunk.
// Bit-plane formats give unsigned codes 0..63, NF formats signed centroids.
template <int FMT>
__device__ __forceinline__ void decode(const Raw<FMT> &w, const uint32_t (&cb)[8], uint32_t (&u)[16]) {
    if (FMT == FMT_BP4 || FMT == FMT_BP5 || FMT == FMT_BP6) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            u[2 * i] = w.w[i] & 0x0F0F0F0Fu;
            u[2 * i + 1] = (w.w[i] >> 4) & 0x0F0F0F0Fu;
        }
        if (FMT == FMT_BP5) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {   // plane-4 bit of column 4j+b sits at bit j of byte b
                uint32_t h0 = j <= 4 ? (w.w[8] << (4 - j)) : (w.w[8] >> (j - 4));
                uint32_t h1 = j <= 4 ? (w.w[9] << (4 - j)) : (w.w[9] >> (j - 4));
                u[j] = lop3_or_and(u[j], h0, 0x10101010u);
                u[8 + j] = lop3_or_and(u[8 + j], h1, 0x10101010u);
            }
        }
        if (FMT == FMT_BP6) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {   // planes 4,5 of column 16v+4f+b sit at bits 2f,2f+1 of byte b
                uint32_t h = w.w[8 + v];
                u[4 * v + 0] = lop3_or_and(u[4 * v + 0], h << 4, 0x30303030u);
                u[4 * v + 1] = lop3_or_and(u[4 * v + 1], h << 2, 0x30303030u);
                u[4 * v + 2] = lop3_or_and(u[4 * v + 2], h, 0x30303030u);
                u[4 * v + 3] = lop3_or_and(u[4 * v + 3], h >> 2, 0x30303030u);
            }
        }
    } else if (FMT == FMT_NF4 || FMT == FMT_NF4G) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {      // word i = eight consecutive 4-bit indices (columns 8i..8i+7)
            uint32_t x = w.w[i];
            uint32_t lo3 = x & 0x77777777u, hb = x & 0x88888888u, hs = hb << 4;
            uint32_t lo3h = lo3 >> 16;
            uint32_t m0 = prmt(hs, hb, 0xD9C8u), m1 = prmt(hs, hb, 0xFBEAu);   // byte masks: index bit 3
            u[2 * i] = lop3_select(prmt(cb[0], cb[1], lo3), prmt(cb[2], cb[3], lo3), m0);
            u[2 * i + 1] = lop3_select(prmt(cb[0], cb[1], lo3h), prmt(cb[2], cb[3], lo3h), m1);
        }
    } else if (FMT == FMT_NF3) {
#pragma unroll
        for (int i = 0; i < 6; ++i) {      // columns 8i..8i+7: index in the low 3 bits of each nibble
            uint32_t s = w.w[i] & 0x77777777u;
            u[2 * i] = prmt(cb[0], cb[1], s);
            u[2 * i + 1] = prmt(cb[0], cb[1], s >> 16);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {      // columns 48+8h..: index bit j = bit 3 of the nibbles of W[3h+j]
            uint32_t s = (w.w[3 * h] >> 3) & 0x11111111u;
            s = lop3_or_and(s, w.w[3 * h + 1] >> 2, 0x22222222u);
            s = lop3_or_and(s, w.w[3 * h + 2] >> 1, 0x44444444u);
            u[12 + 2 * h] = prmt(cb[0], cb[1], s);
            u[13 + 2 * h] = prmt(cb[0], cb[1], s >> 16);
        }
    } else if (FMT == FMT_NF5) {
        // 32-entry codebook: bits 0..3 in the nibbles of words 0..7 (as NF4), bit 4 of column 4j+b at bit j of byte b of
        // word 8 (columns 0..31) / 9 (columns 32..63), as for b5
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t x = w.w[i];
            const uint32_t lo3 = x & 0x77777777u, hb = x & 0x88888888u, hs = hb << 4, lo3h = lo3 >> 16;
            const uint32_t m0 = prmt(hs, hb, 0xD9C8u), m1 = prmt(hs, hb, 0xFBEAu);          // byte masks: index bit 3
            const uint32_t hw = w.w[8 + i / 4];
            const int j0 = 2 * (i % 4), j1 = j0 + 1;
            const uint32_t t0 = ((j0 <= 4 ? (hw << (4 - j0)) : (hw >> (j0 - 4))) & 0x10101010u) >> 4;
            const uint32_t t1 = ((j1 <= 4 ? (hw << (4 - j1)) : (hw >> (j1 - 4))) & 0x10101010u) >> 4;
            const uint32_t b0 = t0 * 0xFFu, b1 = t1 * 0xFFu;                                   // byte masks: index bit 4
            const uint32_t a0 = lop3_select(prmt(cb[0], cb[1], lo3), prmt(cb[2], cb[3], lo3), m0);
            const uint32_t c0 = lop3_select(prmt(cb[4], cb[5], lo3), prmt(cb[6], cb[7], lo3), m0);
            const uint32_t a1 = lop3_select(prmt(cb[0], cb[1], lo3h), prmt(cb[2], cb[3], lo3h), m1);
            const uint32_t c1 = lop3_select(prmt(cb[4], cb[5], lo3h), prmt(cb[6], cb[7], lo3h), m1);
            u[2 * i] = lop3_select(a0, c0, b0);
            u[2 * i + 1] = lop3_select(a1, c1, b1);
        }
    } else if (FMT == FMT_E8Q2) {
        // e8q2_decode_8d (simd_lut.rs:4385-4459): byte 2b = template, 2b+1 = signs of columns 8b..8b+7
        const uint32_t *tab = e8q2_templates_smem();
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            const uint32_t pair = (w.w[b / 2] >> (16 * (b % 2))) & 0xFFFFu, tpl = pair & 0xFFu, sgn = pair >> 8;
            const bool even = (__popc(tpl ^ sgn) & 1) != 0;
            const uint32_t tu = tpl & 15u, tv = tpl >> 4;
            const uint32_t ui = (tu < 12u && tv >= 12u) ? 16u + tu : tu, vi = (tv < 12u && tu >= 12u) ? 16u + tv : tv;
            // odd coset: magnitude 16 or 48 per column; even coset: two template entries (indices stay below 28 for
            // every byte pair the packer emits; masked so that a stray pair cannot read outside the table)
            const uint32_t mu = even ? tab[ui & 31u] : ((spread4(tu) & 0x20202020u) + 0x10101010u);
            const uint32_t mv = even ? tab[vi & 31u] : ((spread4(tv) & 0x20202020u) + 0x10101010u);
            const uint32_t su = spread4(sgn & 15u), sv = spread4(sgn >> 4);
            u[2 * b] = __vsub4(mu & ~su, mu & su);          // per byte: +m or -m
            u[2 * b + 1] = __vsub4(mv & ~sv, mv & sv);
        }
    }
}

template <int FMT> __device__ __forceinline__ constexpr bool is_bitplane() {
    return FMT == FMT_BP4 || FMT == FMT_BP5 || FMT == FMT_BP6;
}

template <int FMT>
__device__ __forceinline__ int dot16(const uint32_t (&u)[16], const int (&q)[16]) {
    int a0 = 0, a1 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (is_bitplane<FMT>()) { a0 = dp4a_us(u[2 * i], q[2 * i], a0); a1 = dp4a_us(u[2 * i + 1], q[2 * i + 1], a1); }
        else { a0 = dp4a_ss(u[2 * i], q[2 * i], a0); a1 = dp4a_ss(u[2 * i + 1], q[2 * i + 1], a1); }
    }
    return a0 + a1;
}

// Integer sum(code * q) of one cell against the lane's activation chunk, single token.
// b4 keeps high nibbles in place (x16) in a second accumulator; NF4 looks the eight largest and the
// eight smallest centroids up in two non-negative 8-entry tables: a prmt selector nibble with bit 3
// set yields the replicated sign bit of the table byte, i.e. 0 here, so `x ^ 0x88888888` selects the
// upper half where bit 3 is set and `x` the lower half where it is clear, with no masks or blends.
template <int FMT>
__device__ __forceinline__ int cell_dot(const Raw<FMT> &w, const GemvArgs &a, const int (&q)[16], int xsum_c) {
    if (FMT == FMT_BP4) {
        int lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            lo = dp4a_us(w.w[i] & 0x0F0F0F0Fu, q[2 * i], lo);
            hi = dp4a_us(w.w[i] & 0xF0F0F0F0u, q[2 * i + 1], hi);
        }
        return lo + (hi >> 4);   // hi is an exact multiple of 16
    } else if (FMT == FMT_NF4) {
        int up = 0, dn = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t x = w.w[i], y = x ^ 0x88888888u;
            up = dp4a_us(prmt(a.tab[0], a.tab[1], y), q[2 * i], up);
            dn = dp4a_us(prmt(a.tab[2], a.tab[3], x), q[2 * i], dn);
            up = dp4a_us(prmt(a.tab[0], a.tab[1], y >> 16), q[2 * i + 1], up);
            dn = dp4a_us(prmt(a.tab[2], a.tab[3], __umulhi(x, 65536u)), q[2 * i + 1], dn);   // >> 16 on the FMA pipe
        }
        return up - dn + a.nf4_offset * xsum_c;
    } else {
        uint32_t u[16];
        decode<FMT>(w, a.cb, u);
        return dot16<FMT>(u, q);
    }
}

__device__ __forceinline__ uint32_t scale_group_of(const GemvArgs &a, uint32_t c) {
    return a.sgc_shift < 32 ? c >> a.sgc_shift : c / a.sgc;
}

__host__ __device__ inline uint32_t up16(uint32_t x) { return (x + 15u) & ~15u; }

constexpr int RS = 4;           // rows per stage (one 4-row block, one pass)
constexpr int NSTAGE = 2;       // stages per warp
constexpr int SCALE_PITCH = 80; // bytes reserved per row for the scales of a pass (32 bf16 + alignment slack)
constexpr uint32_t WAIT_LIMIT = 1u << 22;

template <int FMT> struct Stage {
    static constexpr uint32_t OFF0 = 0;
    static constexpr uint32_t OFF1 = RS * 32 * Cell<FMT>::B0;
    static constexpr uint32_t OFF2 = OFF1 + RS * 32 * Cell<FMT>::B1;
    static constexpr uint32_t OFFS = OFF2 + RS * 32 * Cell<FMT>::B2;
    static constexpr uint32_t BYTES = OFFS + RS * SCALE_PITCH;
    static constexpr uint32_t NPL = 1 + (Cell<FMT>::B1 ? 1 : 0) + (Cell<FMT>::B2 ? 1 : 0) + 1;   // code planes + scales
};

// shared memory of one warp: stages, v tile float [NT][32][33], w_scale tile bf16 [32][34], mbarriers
// GB row blocks (GB x RS = 32 rows) share one fp32-chain step: lane i runs row i.  The kernel is latency-bound and its
// throughput follows the warps an SM can hold (measured on a 2048 x 49152 b4 launch: 14.2 / 12.6 / 10.1 / 9.6 us with
// 8 / 10 / 12 / 14 warps per SM), which shared memory per warp decides; halving the group (a smaller tile, 17 warps)
// was measured slower all the same (10.1 us; NF4 17.8 instead of 12.5 us): the chain steps double.
constexpr uint32_t GB = 8, GROUP_ROWS = GB * RS;
constexpr uint32_t TILE_V = GROUP_ROWS * 33 * 4, TILE_WS = GROUP_ROWS * 34 * 2;
template <int FMT> __host__ __device__ constexpr uint32_t warp_smem(uint32_t nt) {
    return ((NSTAGE * Stage<FMT>::BYTES + nt * TILE_V + TILE_WS + 128) + 127u) & ~127u;
}

template <int FMT>
__device__ __forceinline__ void read_cell(Raw<FMT> &o, const uint8_t *st, uint32_t rr, uint32_t lane,
                                          uint32_t p0, uint32_t p1, uint32_t p2) {
    const uint4 a = *reinterpret_cast<const uint4 *>(st + Stage<FMT>::OFF0 + rr * p0 + lane * 16);
    o.w[0] = a.x; o.w[1] = a.y; o.w[2] = a.z; o.w[3] = a.w;
    if (Cell<FMT>::B1 == 16) {
        const uint4 b = *reinterpret_cast<const uint4 *>(st + Stage<FMT>::OFF1 + rr * p1 + lane * 16);
        o.w[4] = b.x; o.w[5] = b.y; o.w[6] = b.z; o.w[7] = b.w;
    } else if (Cell<FMT>::B1 == 8) {
        const uint2 b = *reinterpret_cast<const uint2 *>(st + Stage<FMT>::OFF1 + rr * p1 + lane * 8);
        o.w[4] = b.x; o.w[5] = b.y;
    }
    if (Cell<FMT>::B2 == 8) {
        const uint2 h = *reinterpret_cast<const uint2 *>(st + Stage<FMT>::OFF2 + rr * p2 + lane * 8);
        o.w[8] = h.x; o.w[9] = h.y;
    } else if (Cell<FMT>::B2 == 16) {
        const uint4 h = *reinterpret_cast<const uint4 *>(st + Stage<FMT>::OFF2 + rr * p2 + lane * 16);
        o.w[8] = h.x; o.w[9] = h.y; o.w[10] = h.z; o.w[11] = h.w;
    }
}


// blockDim.x = 32 * WK.  WK = 1: every warp is on its own.  WK > 1 (long rows, few of them): the WK
// warps of a CTA share the CTA's row blocks and split the passes (warp w takes passes w, w + WK, ...);
// the fp32 chain is handed from pass to pass through shared memory in pass order.
//
// The body is a device function so that the stand-alone kernel (one team per CTA) and the whole-token
// decode kernel (several teams per CTA, many matrices per launch) share it.  A TEAM is the WK warps that
// split the passes of their row blocks; `gw` / `nw` are the team's index and the number of teams, `wid`
// the warp's index in the team, `wsm` the warp's own shared-memory region (warp_smem bytes, 128-byte
// aligned), `s_f` the team's [NT][32] hand-off array, `bar_id` the named barrier of the team (0 = the whole CTA).  The activations come through
// xq / xs / xsum (global memory when !MEGA, read through the read-only L1 path: every warp of an SM reads the
// same few KB, and sending each of those reads to L2 makes its slices a hot spot - measured 19 us instead of
// 11 us for a 2048 x 49152 b4 launch; any address space otherwise); `ps` carries the
// stage cursor and mbarrier parities from one call to the next (the mbarriers are initialised once by the caller).
struct PipeState { uint32_t stage = 0, phase = 0; };

__device__ __forceinline__ void team_sync(uint32_t bar_id, uint32_t WK) {
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(32u * WK) : "memory");
}

__device__ __forceinline__ void gemv_init_barriers(uint8_t *wsm) {     // one lane per warp, once per kernel
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(wsm);
    for (int s = 0; s < NSTAGE; ++s) mbar_init(bar0 + 8 * s, 1);
    fence_mbar_init();
    fence_proxy_async();
}

struct NoHook { __device__ __forceinline__ void operator()() const {} };

// `hook` runs once per warp right after the first weight stages have been requested and before any activation is read:
// a kernel that builds its activation itself (k2t_gemv_fused.cu) waits for its predecessor and fills the shared-memory
// activation there, CTA-wide, while its weights are already on their way.
template <int FMT, int NT, bool DOTS, bool MEGA, typename Hook>
__device__ __forceinline__ void gemv_body(const GemvArgs &a, const int8_t *xq, const float *xs, const int32_t *xsum_p, float *out,
                                          uint8_t *wsm, float *s_f, uint32_t gw, uint32_t nw, uint32_t wid, uint32_t WK,
                                          uint32_t bar_id, PipeState &ps, Hook hook) {
    using St = Stage<FMT>;
    const uint32_t lane = threadIdx.x & 31;
    if (FMT == FMT_E8Q2) {          // every warp fills the (same) table itself, so no CTA-wide barrier is needed
        uint32_t *tab = e8q2_templates_smem();
        tab[lane] = lane < 28 ? E8Q2_TEMPLATE_WORDS[lane] : 0u;
        __syncwarp();
    }
    const uint32_t n_rb = (a.rows + RS - 1) / RS;              // 4-row blocks of the matrix
    const uint32_t J = gw < n_rb ? (n_rb - gw + nw - 1) / nw : 0;   // blocks of this CTA: gw, gw + nw, ...
    const uint32_t np = (a.nc + 31) / 32;
    const uint32_t my_np = wid < np ? (np - wid + WK - 1) / WK : 0; // passes of this warp: wid, wid + WK, ...
    const uint32_t rounds = (np + WK - 1) / WK;
    // warp region: mbarriers (first 128 B, so that the stages keep their 128-byte alignment and a quarter-warp's
    // 128-bit reads stay within one 128-byte line), stages, v tile, w_scale tile
    uint8_t *stages = wsm + 128;
    float *s_v = reinterpret_cast<float *>(wsm + 128 + NSTAGE * St::BYTES);
    uint16_t *s_ws = reinterpret_cast<uint16_t *>(wsm + 128 + NSTAGE * St::BYTES + NT * TILE_V);
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(wsm);
    const uint32_t stage_sa = (uint32_t)__cvta_generic_to_shared(stages);

    // ---- producer role of this lane: lane k < NPL copies plane k (the last one: the scales) of every unit - the
    // four rows of a block are one contiguous run in a pass tile.  What does not depend on the unit is fixed here.
    const uint32_t my_k = lane;
    const bool my_role = lane < St::NPL, my_scale = my_k == St::NPL - 1;
    const uint32_t my_cell = my_scale ? 0u : (my_k == 0 ? (uint32_t)Cell<FMT>::B0 : my_k == 1 ? (uint32_t)Cell<FMT>::B1 : (uint32_t)Cell<FMT>::B2);
    const uint8_t *my_base = my_scale ? reinterpret_cast<const uint8_t *>(a.scales) : a.plane[my_role ? my_k : 0];
    const uint32_t my_soff = my_scale ? St::OFFS : (my_k == 0 ? St::OFF0 : my_k == 1 ? St::OFF1 : St::OFF2);
    constexpr uint32_t CELL_SUM = Cell<FMT>::B0 + Cell<FMT>::B1 + Cell<FMT>::B2;

    // producer cursor: 32-row group, own pass index, block in group; the tile geometry is recomputed only when the
    // pass changes (never, for a matrix of one pass)
    uint32_t pj0 = 0, ppi = 0, pjj = 0;
    uint32_t c_pass = 0xffffffffu, c_pitch = 0, c_total = 0;
    const uint8_t *c_src = my_base;
    auto issue = [&](uint32_t stage) {
        if (pj0 >= J || my_np == 0) return;                     // nothing left: the stage stays idle
        const uint32_t p = wid + ppi * WK;
        if (p != c_pass) {
            const uint32_t n = tile_chunks(a.nc, p), sp = tile_scale_pitch(a.nc, a.sgc, p);
            c_pass = p;
            c_pitch = my_scale ? sp : n * my_cell;              // bytes of one row of this lane's plane in tile p
            c_total = RS * (sp + n * CELL_SUM);
            c_src = my_base + (my_scale ? tile_scale_off(a.rows_pad, p) : tile_code_off(a.rows_pad, my_cell, p));
        }
        const uint32_t row0 = (gw + (pj0 + pjj) * nw) * RS;
        const uint32_t bar = bar0 + 8 * stage;
        if (lane == 0) { fence_proxy_async(); mbar_expect_tx(bar, c_total); }
        __syncwarp();
        if (my_role) bulk_g2s(stage_sa + stage * St::BYTES + my_soff, c_src + (size_t)row0 * c_pitch, RS * c_pitch, bar);
        const uint32_t in_group = min(GB, J - pj0);
        if (++pjj == in_group) { pjj = 0; if (++ppi == my_np) { ppi = 0; pj0 += GB; } }
    };
    // the first unit goes to the stage the consumer reads first (the cursor persists across calls)
#pragma unroll
    for (int s = 0; s < NSTAGE; ++s) issue((ps.stage + s) % NSTAGE);
    // weights are on their way; the activations (and the output buffer) belong to the preceding kernels
    if (!MEGA) { pdl_wait(); pdl_trigger(); }
    hook();

    // Teams of the stand-alone kernels pass the fp32 chain from pass to pass by TURN: a counter behind the hand-off array
    // holds the number of chain steps done; the warp that owns pass p of group g waits for g * np + p, runs its step and
    // publishes the next number.  Unlike a team barrier per step this lets the other warps go on with the dot products of
    // their next pass while one warp is on the chain (the steps themselves stay serial: each starts from its predecessor's sum):
    // a 3584 x 18944 b5 launch (ten passes, teams of four) 16.6 -> 14.7 us.
    volatile uint32_t *s_turn = reinterpret_cast<volatile uint32_t *>(s_f + NT * 32);
    const bool by_turn = !MEGA && WK > 1 && rounds > 1;       // one round: nothing to overlap, and a barrier costs the waiting warps no issue slots
    if (by_turn) {
        if (wid == 0 && lane == 0) *s_turn = 0;
        team_sync(bar_id, WK);
    }

    // ---- consumer
    int q[NT][16];
    float sx[NT];
    int xsum[NT];
    uint32_t nz[NT];
    uint32_t stage = ps.stage, phase = ps.phase;
    bool failed = false;                                         // a wait gave up: keep the barriers in step, skip waiting
    const uint32_t slot_j = lane / RS, slot_r = lane % RS;       // chain: lane -> (block in group, row in block)
    for (uint32_t j0 = 0; j0 < J; j0 += GB) {
        const uint32_t in_group = min(GB, J - j0);
        for (uint32_t r = 0; r < rounds; ++r) {
            const uint32_t p = r * WK + wid;
            const bool has = p < np;
            const uint32_t c = p * 32 + lane, n = has ? min(32u, a.nc - p * 32) : 0;
            const bool act = lane < n;
            if (has) {
                if (my_np > 1 || j0 == 0) {       // this lane's activation chunk(s) for the pass, kept in registers
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        const bool on = act && (uint32_t)t < a.n_tok;
                        sx[t] = on ? (MEGA ? xs[(size_t)t * a.nc + c] : __ldg(xs + (size_t)t * a.nc + c)) : 0.0f;
                        xsum[t] = (on && xsum_p != nullptr) ? (MEGA ? xsum_p[(size_t)t * a.nc + c] : __ldg(xsum_p + (size_t)t * a.nc + c)) : 0;
#pragma unroll
                        for (int jq = 0; jq < 4; ++jq) {
                            const int4 *src4 = reinterpret_cast<const int4 *>(xq + (size_t)t * a.cols + (size_t)c * 64) + jq;
                            const int4 v = on ? (MEGA ? *src4 : __ldg(src4)) : make_int4(0, 0, 0, 0);
                            q[t][4 * jq] = v.x; q[t][4 * jq + 1] = v.y; q[t][4 * jq + 2] = v.z; q[t][4 * jq + 3] = v.w;
                        }
                        nz[t] = __ballot_sync(0xffffffffu, sx[t] != 0.0f);
                    }
                }
                // stage geometry of this pass
                const uint32_t p0 = n * Cell<FMT>::B0, p1 = n * Cell<FMT>::B1, p2 = n * Cell<FMT>::B2;
                const uint32_t ps = tile_scale_pitch(a.nc, a.sgc, p);
                const uint32_t ws_off = (scale_group_of(a, act ? c : p * 32) - scale_group_of(a, p * 32)) * 2;

                for (uint32_t jj = 0; jj < in_group; ++jj) {
                    const uint32_t row0 = (gw + (j0 + jj) * nw) * RS;
                    const uint32_t nrows = min((uint32_t)RS, a.rows - row0);
                    if (!failed) {                 // wait for the stage (bounded)
                        uint32_t ok = 0;
                        for (uint32_t spin = 0; spin < WAIT_LIMIT && !ok; ++spin) ok = mbar_try_wait(bar0 + 8 * stage, (phase >> stage) & 1u);
                        if (__any_sync(0xffffffffu, !ok)) {
                            if (lane == 0) atomicExch(a.err_flag, 1u);
                            failed = true;
                        }
                    }
                    phase ^= 1u << stage;
                    const uint8_t *st = stages + stage * St::BYTES;
                    // all four rows are read and reduced unconditionally (stale bytes of absent rows are
                    // harmless): no branches, so the four independent dot chains interleave
                    Raw<FMT> w[RS];
                    uint16_t wsb[RS];
#pragma unroll
                    for (uint32_t rr = 0; rr < RS; ++rr) {
                        read_cell<FMT>(w[rr], st, rr, lane, p0, p1, p2);
                        wsb[rr] = *reinterpret_cast<const uint16_t *>(st + St::OFFS + rr * ps + ws_off);
                    }
                    if (NT == 1) {
                        int dot[RS];
#pragma unroll
                        for (uint32_t rr = 0; rr < RS; ++rr) {
                            const int acc = cell_dot<FMT>(w[rr], a, q[0], xsum[0]);
                            dot[rr] = is_bitplane<FMT>() ? 2 * acc - a.max_odd * xsum[0] : acc;
                        }
#pragma unroll
                        for (uint32_t rr = 0; rr < RS; ++rr) {
                            if (act && rr < nrows) {
                                s_v[(jj * RS + rr) * 33 + lane] = __fmul_rn(__int2float_rn(dot[rr]), sx[0]);
                                s_ws[(jj * RS + rr) * 34 + lane] = wsb[rr];
                                if (DOTS) a.int_dots[(size_t)(row0 + rr) * a.nc + c] = dot[rr];
                            }
                        }
                    } else {
#pragma unroll
                        for (uint32_t rr = 0; rr < RS; ++rr) {
                            uint32_t ub[16];
                            decode<FMT>(w[rr], a.cb, ub);
                            if (act && rr < nrows) s_ws[(jj * RS + rr) * 34 + lane] = wsb[rr];
#pragma unroll
                            for (int t = 0; t < NT; ++t) {
                                const int acc = dot16<FMT>(ub, q[t]);
                                const int dot = is_bitplane<FMT>() ? 2 * acc - a.max_odd * xsum[t] : acc;
                                if (act && rr < nrows) {
                                    s_v[t * (GROUP_ROWS * 33) + (jj * RS + rr) * 33 + lane] = __fmul_rn(__int2float_rn(dot), sx[t]);
                                    if (DOTS && (uint32_t)t < a.n_tok) a.int_dots[((size_t)t * a.rows + row0 + rr) * a.nc + c] = dot;
                                }
                            }
                        }
                    }
                    __syncwarp();                  // every lane has read the stage: refill it
                    issue(stage);
                    stage = stage + 1 == NSTAGE ? 0 : stage + 1;
                }
                __syncwarp();
            }
            // fp32 chain over the chunks of the passes of this round, in pass order: warp k continues
            // where warp k-1 stopped (f travels through s_f); lane -> row slot
            if (by_turn && has) {           // wait for this pass's turn on the chain (bounded)
                const uint32_t turn = (j0 / GB) * np + p;
                uint32_t spin = 0;
                while (*s_turn != turn && ++spin < WAIT_LIMIT) {}
                if (spin >= WAIT_LIMIT && lane == 0) atomicExch(a.err_flag, 1u);
                __threadfence_block();
            }
            for (uint32_t k = by_turn ? wid : 0; k < (by_turn ? wid + 1 : WK); ++k) {
                if (k == wid && has && slot_j < in_group) {
                    const uint32_t row = (gw + (j0 + slot_j) * nw) * RS + slot_r;
#pragma unroll
                    for (int t = 0; t < NT; ++t) {
                        const float *vv = s_v + t * (GROUP_ROWS * 33) + lane * 33;
                        const uint16_t *wv = s_ws + lane * 34;
                        float ft = p == 0 ? 0.0f : s_f[t * 32 + lane];
                        if (nz[t] == (n == 32 ? 0xffffffffu : (1u << n) - 1u)) {
#pragma unroll 8
                            for (uint32_t l = 0; l < n; ++l) ft = __fmaf_rn(vv[l], bf16_bits_to_f32(wv[l]), ft);
                        } else {
                            for (uint32_t l = 0; l < n; ++l)
                                if ((nz[t] >> l) & 1u) ft = __fmaf_rn(vv[l], bf16_bits_to_f32(wv[l]), ft);
                        }
                        if (p + 1 == np) { if (row < a.rows && (uint32_t)t < a.n_tok) out[(size_t)t * a.out_stride + row] = ft; }
                        else s_f[t * 32 + lane] = ft;
                    }
                }
                if (by_turn) {
                    __syncwarp();
                    if (has && lane == 0) { __threadfence_block(); *s_turn = (j0 / GB) * np + p + 1; }
                } else if (WK > 1) team_sync(bar_id, WK);
                else __syncwarp();
            }
        }
    }
    ps.stage = stage; ps.phase = phase;
}

template <int FMT, int NT, bool DOTS, bool MEGA>
__device__ __forceinline__ void gemv_body(const GemvArgs &a, const int8_t *xq, const float *xs, const int32_t *xsum_p, float *out,
                                          uint8_t *wsm, float *s_f, uint32_t gw, uint32_t nw, uint32_t wid, uint32_t WK,
                                          uint32_t bar_id, PipeState &ps) {
    gemv_body<FMT, NT, DOTS, MEGA>(a, xq, xs, xsum_p, out, wsm, s_f, gw, nw, wid, WK, bar_id, ps, NoHook{});
}

}  // namespace k2t

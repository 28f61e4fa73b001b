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
// their sum stay in the lane's registers while the warp walks down the rows of its tile: the inner
// loop touches no shared memory for activations.  A warp step reads 32 cells x 32 B = 1 KiB of
// contiguous weights with 128-bit loads (cells are stored row-major, [row][chunk]); loads are issued
// in register batches of UB rows, the next batch in flight while the current one is reduced, and the
// UB cells of a batch are independent, which gives the lane UB-way instruction-level parallelism.
// Every cell parks (v, w_scale) in a shared-memory tile [row][chunk]; when the tile is complete, lane
// i of the tile's first warp runs the fp32 chain of row i over all chunks.  With `wk` warps per tile
// the passes are dealt round-robin to the warps (K split), with `tr` rows per tile the rows are.
#include "k2t_device.cuh"
#include "k2t_kernels.h"

namespace k2t {

struct GemvArgs {
    const uint8_t *pa;        // plane A  [rows][nc] cells
    const uint8_t *pb;        // plane B  [rows][nc] cells (formats with more than 4 bits, NF3)
    const uint16_t *scales;   // [rows][nsg] bf16
    const int8_t *xq;
    const float *xs;
    const int32_t *xsum;
    float *out;
    int32_t *int_dots;
    size_t out_stride;
    uint32_t rows, cols, nc, nsg, sgc, sgc_shift, n_tok;   // sgc_shift: log2(sgc) or 32
    uint32_t tr, wk, tpc;     // rows per tile, warps per tile, tiles per CTA
    int32_t max_odd;
    int32_t nf4_offset;
    uint32_t cb[8];    // expanded codebook, 4 centroids per word (NF4: sorted ascending)
    uint32_t tab[4];   // NF4 two-table decode: hi[0..3], hi[4..7], lo[0..3], lo[4..7]
};

constexpr int FMT_NF4G = FMT_COUNT;   // NF4 with a codebook the two-table decode cannot represent

template <int FMT> struct CellWords { static constexpr int A = 8, B = 0; };
template <> struct CellWords<FMT_BP5> { static constexpr int A = 8, B = 2; };
template <> struct CellWords<FMT_BP6> { static constexpr int A = 8, B = 4; };
template <> struct CellWords<FMT_NF3> { static constexpr int A = 4, B = 2; };

template <int FMT>
struct Raw {          // the words of one cell: plane A words first, then plane B words
    uint32_t w[CellWords<FMT>::A + CellWords<FMT>::B];
};

template <int FMT>
__device__ __forceinline__ void load_cell(Raw<FMT> &o, const uint8_t *ca, const uint8_t *cb) {
    constexpr int A = CellWords<FMT>::A, B = CellWords<FMT>::B;
    uint4 a = ldg_stream(reinterpret_cast<const uint4 *>(ca));
    o.w[0] = a.x; o.w[1] = a.y; o.w[2] = a.z; o.w[3] = a.w;
    if (A == 8) {
        uint4 b = ldg_stream(reinterpret_cast<const uint4 *>(ca) + 1);
        o.w[4] = b.x; o.w[5] = b.y; o.w[6] = b.z; o.w[7] = b.w;
    }
    if (B == 2) {
        uint2 h = ldg_stream(reinterpret_cast<const uint2 *>(cb));
        o.w[A] = h.x; o.w[A + 1] = h.y;
    }
    if (B == 4) {
        uint4 h = ldg_stream(reinterpret_cast<const uint4 *>(cb));
        o.w[A] = h.x; o.w[A + 1] = h.y; o.w[A + 2] = h.z; o.w[A + 3] = h.w;
    }
}

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
            up = dp4a_us(prmt(a.tab[0], a.tab[1], __umulhi(y, 65536u)), q[2 * i + 1], up);   // >> 16 on the FMA pipe
            dn = dp4a_us(prmt(a.tab[2], a.tab[3], __umulhi(x, 65536u)), q[2 * i + 1], dn);
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

__host__ __device__ inline size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }

// rows of a register batch: about 32 words of cells per buffer, two buffers
template <int FMT> struct Batch { static constexpr int UB = 32 / (CellWords<FMT>::A + CellWords<FMT>::B); };
template <> struct Batch<FMT_NF3> { static constexpr int UB = 4; };

struct SmemPlan { size_t nz, tile, tile_stride, total; };
__host__ __device__ inline SmemPlan smem_plan(uint32_t nt, uint32_t nc, uint32_t tr, uint32_t tpc) {
    SmemPlan p;
    const uint32_t np = (nc + 31) / 32;
    p.nz = 0;                                                   // [nt][np] masks of chunks with xs != 0
    p.tile = align16((size_t)nt * np * 4);
    p.tile_stride = (size_t)nt * tr * (nc + 1) * 8;             // float2 [nt][tr][nc + 1] per tile
    p.total = p.tile + p.tile_stride * tpc;
    return p;
}

template <int FMT, int NT>
__global__ void __launch_bounds__(256) gemv_kernel(const GemvArgs a) {
    constexpr int UB = Batch<FMT>::UB;
    constexpr int CA = CellWords<FMT>::A * 4, CB = CellWords<FMT>::B * 4;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t np = (a.nc + 31) / 32;
    const SmemPlan sp = smem_plan(NT, a.nc, a.tr, a.tpc);
    uint32_t *s_nz = reinterpret_cast<uint32_t *>(smem + sp.nz);

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t tl = warp / a.wk, kw = warp % a.wk;
    const uint32_t tile = blockIdx.x * a.tpc + tl;
    const uint32_t row0 = tile * a.tr;
    const uint32_t trv = row0 < a.rows ? min(a.tr, a.rows - row0) : 0;      // valid rows of this tile
    const uint32_t stride = a.nc + 1;
    float2 *s_tile = reinterpret_cast<float2 *>(smem + sp.tile + sp.tile_stride * tl);

    for (uint32_t p = kw; p < np; p += a.wk) {
        const uint32_t c = p * 32 + lane;
        const bool act = c < a.nc;
        // this lane's activation chunk(s): 64 int8 per token, kept in registers for the whole tile
        int q[NT][16];
        float sx[NT];
        int xsum[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const bool on = act && (uint32_t)t < a.n_tok;
            sx[t] = on ? __ldg(a.xs + (size_t)t * a.nc + c) : 0.0f;
            xsum[t] = (on && a.xsum != nullptr) ? __ldg(a.xsum + (size_t)t * a.nc + c) : 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int4 v = on ? __ldg(reinterpret_cast<const int4 *>(a.xq + (size_t)t * a.cols + (size_t)c * 64) + j) : make_int4(0, 0, 0, 0);
                q[t][4 * j] = v.x; q[t][4 * j + 1] = v.y; q[t][4 * j + 2] = v.z; q[t][4 * j + 3] = v.w;
            }
            const uint32_t nz = __ballot_sync(0xffffffffu, sx[t] != 0.0f);
            if (tl == 0 && lane == 0) s_nz[t * np + p] = nz;
        }

        const uint8_t *ca = a.pa + ((size_t)row0 * a.nc + c) * CA;
        const uint8_t *cb = a.pb + ((size_t)row0 * a.nc + c) * CB;
        const size_t sa = (size_t)a.nc * CA, sb = (size_t)a.nc * CB;
        const uint16_t *wsp = a.scales + (size_t)row0 * a.nsg + scale_group_of(a, act ? c : 0);

        Raw<FMT> cur[UB], nxt[UB];
        uint16_t cur_ws[UB], nxt_ws[UB];
#pragma unroll
        for (int u = 0; u < UB; ++u)
            if (act && (uint32_t)u < trv) {
                load_cell<FMT>(cur[u], ca + u * sa, cb + u * sb);
                cur_ws[u] = __ldg(wsp + (size_t)u * a.nsg);
            }
        for (uint32_t i0 = 0; i0 < trv; i0 += UB) {
#pragma unroll
            for (int u = 0; u < UB; ++u) {
                const uint32_t i = i0 + UB + u;
                if (act && i < trv) {
                    load_cell<FMT>(nxt[u], ca + (size_t)i * sa, cb + (size_t)i * sb);
                    nxt_ws[u] = __ldg(wsp + (size_t)i * a.nsg);
                }
            }
#pragma unroll
            for (int u = 0; u < UB; ++u) {
                const uint32_t i = i0 + u;
                if (act && i < trv) {
                    const float ws = bf16_bits_to_f32(cur_ws[u]);
                    if (NT == 1) {
                        const int acc = cell_dot<FMT>(cur[u], a, q[0], xsum[0]);
                        const int dot = is_bitplane<FMT>() ? 2 * acc - a.max_odd * xsum[0] : acc;
                        s_tile[(size_t)i * stride + c] = make_float2(__fmul_rn(__int2float_rn(dot), sx[0]), ws);
                        if (a.int_dots != nullptr) a.int_dots[(size_t)(row0 + i) * a.nc + c] = dot;
                    } else {
                        uint32_t ub[16];
                        decode<FMT>(cur[u], a.cb, ub);
#pragma unroll
                        for (int t = 0; t < NT; ++t) {
                            const int acc = dot16<FMT>(ub, q[t]);
                            const int dot = is_bitplane<FMT>() ? 2 * acc - a.max_odd * xsum[t] : acc;
                            s_tile[((size_t)t * a.tr + i) * stride + c] = make_float2(__fmul_rn(__int2float_rn(dot), sx[t]), ws);
                            if (a.int_dots != nullptr && (uint32_t)t < a.n_tok)
                                a.int_dots[((size_t)t * a.rows + row0 + i) * a.nc + c] = dot;
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < UB; ++u) { cur[u] = nxt[u]; cur_ws[u] = nxt_ws[u]; }
        }
    }
    __syncthreads();

    // ordered fp32 chain: lane i of the tile's first warp owns row i (token t)
    if (kw == 0) {
        for (uint32_t item = lane; item < NT * trv; item += 32) {
            const uint32_t t = item / trv, i = item % trv;
            if (t >= a.n_tok) continue;
            const float2 *vv = s_tile + ((size_t)t * a.tr + i) * stride;
            float f = 0.0f;
            for (uint32_t p = 0; p < np; ++p) {
                const uint32_t nz = s_nz[t * np + p];
                const uint32_t c_end = min(32u, a.nc - p * 32);
#pragma unroll 8
                for (uint32_t l = 0; l < c_end; ++l) {
                    const float2 v = vv[p * 32 + l];
                    if ((nz >> l) & 1u) f = __fmaf_rn(v.x, v.y, f);
                }
            }
            a.out[(size_t)t * a.out_stride + row0 + i] = f;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static const size_t kSmemBudget = 196 * 1024;

template <typename K>
static cudaError_t allow_big_smem(K kernel, size_t smem) {
    if (smem <= 48 * 1024) return cudaSuccess;
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
}

template <int FMT, int NT>
static cudaError_t launch_one(cudaStream_t stream, const GemvArgs &a, size_t smem, uint32_t grid) {
    cudaError_t e = allow_big_smem(gemv_kernel<FMT, NT>, smem);
    if (e != cudaSuccess) return e;
    gemv_kernel<FMT, NT><<<grid, 32 * a.wk * a.tpc, smem, stream>>>(a);
    return cudaGetLastError();
}

template <int FMT>
static cudaError_t launch_fmt(cudaStream_t stream, const GemvArgs &a, uint32_t nt, size_t smem, uint32_t grid) {
    switch (nt) {
        case 1: return launch_one<FMT, 1>(stream, a, smem, grid);
        case 2: return launch_one<FMT, 2>(stream, a, smem, grid);
        default: return launch_one<FMT, 4>(stream, a, smem, grid);
    }
}

uint32_t gemv_max_tokens(const DeviceMatrix &) { return 4; }

cudaError_t launch_gemv(cudaStream_t stream, const DeviceMatrix &m, const int8_t *xq, const float *xs,
                        const int32_t *xsum, uint32_t n_tok, float *out, size_t out_stride, int32_t *int_dots,
                        int sm_count, uint32_t *launches) {
    const MatrixGeom &g = m.geom;
    if (launches) *launches = 0;
    if (n_tok == 0) return cudaSuccess;
    if (n_tok > 4 || g.fmt == FMT_NF5 || g.fmt == FMT_E8Q2) return cudaErrorNotSupported;
    const uint32_t nt = n_tok <= 1 ? 1 : n_tok <= 2 ? 2 : 4;
    GemvArgs a;
    a.pa = m.d_a; a.pb = m.d_b; a.scales = m.d_scales; a.xq = xq; a.xs = xs; a.xsum = xsum; a.out = out; a.int_dots = int_dots;
    a.out_stride = out_stride;
    a.rows = g.rows; a.cols = g.cols; a.nc = g.nc; a.nsg = g.nsg; a.sgc = g.sgc; a.n_tok = n_tok;
    a.sgc_shift = 32;
    for (uint32_t sh = 0; sh < 4; ++sh) if ((1u << sh) == g.sgc) a.sgc_shift = sh;
    a.max_odd = g.max_odd; a.nf4_offset = g.nf4_offset;
    for (int i = 0; i < 8; ++i) {
        const uint8_t *b = reinterpret_cast<const uint8_t *>(g.codebook32) + 4 * i;
        a.cb[i] = (uint32_t)b[0] | ((uint32_t)b[1] << 8) | ((uint32_t)b[2] << 16) | ((uint32_t)b[3] << 24);
    }
    for (int i = 0; i < 2; ++i) {
        const uint8_t *h = g.nf4_hi + 4 * i, *l = g.nf4_lo + 4 * i;
        a.tab[i] = (uint32_t)h[0] | ((uint32_t)h[1] << 8) | ((uint32_t)h[2] << 16) | ((uint32_t)h[3] << 24);
        a.tab[2 + i] = (uint32_t)l[0] | ((uint32_t)l[1] << 8) | ((uint32_t)l[2] << 16) | ((uint32_t)l[3] << 24);
    }
    // tiling: K split over up to 4 warps (one 32-chunk pass each), rows per tile as large as still
    // leaves about 16 warps per SM
    const uint32_t np = (g.nc + 31) / 32;
    a.wk = np < 4 ? np : 4;
    const uint32_t want_warps = 16u * (uint32_t)sm_count;
    a.tr = 32;
    while (a.tr > 4 && ((g.rows + a.tr - 1) / a.tr) * a.wk < want_warps) a.tr /= 2;
    a.tpc = a.wk >= 4 ? 1 : 4 / a.wk;
    size_t smem = smem_plan(nt, g.nc, a.tr, a.tpc).total;
    while (smem > kSmemBudget && a.tpc > 1) { a.tpc /= 2; smem = smem_plan(nt, g.nc, a.tr, a.tpc).total; }
    while (smem > kSmemBudget && a.tr > 1) { a.tr /= 2; smem = smem_plan(nt, g.nc, a.tr, a.tpc).total; }
    if (smem > kSmemBudget) return cudaErrorInvalidValue;
    const uint32_t tiles = (g.rows + a.tr - 1) / a.tr;
    const uint32_t grid = (tiles + a.tpc - 1) / a.tpc;
    const bool nf4_fast = g.fmt == FMT_NF4 && g.nf4_split_ok && (g.nf4_offset == 0 || xsum != nullptr);
    cudaError_t e;
    switch (g.fmt) {
        case FMT_BP4: e = launch_fmt<FMT_BP4>(stream, a, nt, smem, grid); break;
        case FMT_BP5: e = launch_fmt<FMT_BP5>(stream, a, nt, smem, grid); break;
        case FMT_BP6: e = launch_fmt<FMT_BP6>(stream, a, nt, smem, grid); break;
        case FMT_NF4: e = nf4_fast ? launch_fmt<FMT_NF4>(stream, a, nt, smem, grid) : launch_fmt<FMT_NF4G>(stream, a, nt, smem, grid); break;
        case FMT_NF3: e = launch_fmt<FMT_NF3>(stream, a, nt, smem, grid); break;
        default: return cudaErrorNotSupported;
    }
    if (e == cudaSuccess && launches) *launches = 1;
    return e;
}

}  // namespace k2t

// Quantized GEMV (batch 1) and small-N GEMM (2..8 tokens) for bit-plane (b4/b5/b6) and codebook
// (NF4/NF3) matrices.
//
// Arithmetic contract (reference: sdot_one_stripe_neon, src/kernels/simd_lut.rs:3763-3868, and
// nf_sdot_one_stripe_neon, 6071-6181; batch forms 4228-4331 / 6689-7029):
//   per row r and 64-column chunk c:  a = sum_i code_i * q_i           (exact int32)
//       bit-plane: dot = 2a - (2^B-1) * xsum[c]      NF: dot = a
//   f = 0;  for c ascending, skipping chunks with xs[c] == 0:
//       f = fmaf((float)dot * xs[c], w_scale[r, c / sgc], f)
// The integer dots are computed by all lanes in parallel; the fp32 chain always runs per row in
// ascending chunk order, so outputs are bit-identical to the reference order.
//
// Batch-1 kernel (gemv1_kernel).  One row group (8 rows) is served by W warps = 4W quarter-warps;
// quarter-warp j owns the j-th contiguous slice of the chunks and its 8 lanes are the 8 rows, so each
// 128-bit access of a quarter-warp covers one 128-byte line and each quarter-warp streams one
// contiguous byte range.  Lanes park (v, w_scale) per chunk in a private shared-memory column; the
// fp32 chain then runs slice after slice, handed from quarter-warp to quarter-warp with a shuffle and
// from warp to warp through shared memory, which keeps the reference's ascending-chunk order exactly.
// Activations (int8, <= 18.5 KiB) are staged once per CTA in shared memory and read as broadcasts.
#include "k2t_device.cuh"
#include "k2t_kernels.h"

namespace k2t {

struct GemvArgs {
    const uint8_t *rec;
    const uint16_t *scales;   // [group][nsg][8] bf16
    const int8_t *xq;
    const float *xs;
    const int32_t *xsum;
    float *out;
    int32_t *int_dots;
    size_t out_stride;
    uint32_t rows, cols, nc, nsg, sgc, sgc_shift, ngroups, rec_bytes, n_tok, gpb, wpg;   // sgc_shift: log2(sgc) or 32
    int32_t max_odd;
    int32_t nf4_offset;
    uint32_t cb[8];    // expanded codebook, 4 centroids per word (NF4: sorted ascending)
    uint32_t tab[4];   // NF4 two-table decode: hi[0..3], hi[4..7], lo[0..3], lo[4..7]
};

constexpr int FMT_NF4G = FMT_COUNT;   // NF4 with a codebook the two-table decode cannot represent

template <int FMT> struct RawWords { static constexpr int N = 8; };
template <> struct RawWords<FMT_BP5> { static constexpr int N = 10; };
template <> struct RawWords<FMT_BP6> { static constexpr int N = 12; };
template <> struct RawWords<FMT_NF3> { static constexpr int N = 6; };

template <int FMT>
struct Raw {          // the words one lane loads for one (group, chunk) record
    uint32_t w[RawWords<FMT>::N];
};

template <int FMT>
__device__ __forceinline__ void load_raw(Raw<FMT> &o, const uint8_t *rec, uint32_t r) {
    const uint4 *p = reinterpret_cast<const uint4 *>(rec);
    uint4 a = ldg_stream(p + r);
    o.w[0] = a.x; o.w[1] = a.y; o.w[2] = a.z; o.w[3] = a.w;
    if (FMT == FMT_NF3) {
        uint2 h = ldg_stream(reinterpret_cast<const uint2 *>(rec + 128) + r);
        o.w[4] = h.x; o.w[5] = h.y;
        return;
    }
    uint4 b = ldg_stream(p + 8 + r);
    o.w[4] = b.x; o.w[5] = b.y; o.w[6] = b.z; o.w[7] = b.w;
    if (FMT == FMT_BP5) {
        uint2 h = ldg_stream(reinterpret_cast<const uint2 *>(rec + 256) + r);
        o.w[8] = h.x; o.w[9] = h.y;
    }
    if (FMT == FMT_BP6) {
        uint4 h = ldg_stream(p + 16 + r);
        o.w[8] = h.x; o.w[9] = h.y; o.w[10] = h.z; o.w[11] = h.w;
    }
}

// Expands a record into 16 words of four weight bytes each: u[j] holds columns 4j..4j+3 of the chunk.
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

template <int FMT>
__device__ __forceinline__ int dot16(const uint32_t (&u)[16], const int4 *q) {
    int acc = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int4 v = q[i];
        if (FMT == FMT_BP4 || FMT == FMT_BP5 || FMT == FMT_BP6) {
            acc = dp4a_us(u[4 * i], v.x, acc); acc = dp4a_us(u[4 * i + 1], v.y, acc);
            acc = dp4a_us(u[4 * i + 2], v.z, acc); acc = dp4a_us(u[4 * i + 3], v.w, acc);
        } else {
            acc = dp4a_ss(u[4 * i], v.x, acc); acc = dp4a_ss(u[4 * i + 1], v.y, acc);
            acc = dp4a_ss(u[4 * i + 2], v.z, acc); acc = dp4a_ss(u[4 * i + 3], v.w, acc);
        }
    }
    return acc;
}

// Integer sum(code * q) of one record against one 64-column activation chunk, single token.
// b4 keeps high nibbles in place (x16) in a second accumulator; NF4 looks the eight largest and the
// eight smallest centroids up in two non-negative 8-entry tables: a prmt selector nibble with bit 3
// set yields the replicated sign bit of the table byte, i.e. 0 here, so `x ^ 0x88888888` selects the
// upper half where bit 3 is set and `x` the lower half where it is clear, with no masks or blends.
template <int FMT>
__device__ __forceinline__ int cell_dot(const Raw<FMT> &w, const GemvArgs &a, const int4 *q4, int xsum_c) {
    if (FMT == FMT_BP4) {
        int lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int4 v = q4[i];
            lo = dp4a_us(w.w[2 * i] & 0x0F0F0F0Fu, v.x, lo);
            hi = dp4a_us(w.w[2 * i] & 0xF0F0F0F0u, v.y, hi);
            lo = dp4a_us(w.w[2 * i + 1] & 0x0F0F0F0Fu, v.z, lo);
            hi = dp4a_us(w.w[2 * i + 1] & 0xF0F0F0F0u, v.w, hi);
        }
        return lo + (hi >> 4);   // hi is an exact multiple of 16
    } else if (FMT == FMT_NF4) {
        int up = 0, dn = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int4 v = q4[i];
            uint32_t x0 = w.w[2 * i], x1 = w.w[2 * i + 1];
            uint32_t y0 = x0 ^ 0x88888888u, y1 = x1 ^ 0x88888888u;
            up = dp4a_us(prmt(a.tab[0], a.tab[1], y0), v.x, up);
            dn = dp4a_us(prmt(a.tab[2], a.tab[3], x0), v.x, dn);
            up = dp4a_us(prmt(a.tab[0], a.tab[1], __umulhi(y0, 65536u)), v.y, up);   // >> 16 on the FMA pipe
            dn = dp4a_us(prmt(a.tab[2], a.tab[3], __umulhi(x0, 65536u)), v.y, dn);
            up = dp4a_us(prmt(a.tab[0], a.tab[1], y1), v.z, up);
            dn = dp4a_us(prmt(a.tab[2], a.tab[3], x1), v.z, dn);
            up = dp4a_us(prmt(a.tab[0], a.tab[1], __umulhi(y1, 65536u)), v.w, up);
            dn = dp4a_us(prmt(a.tab[2], a.tab[3], __umulhi(x1, 65536u)), v.w, dn);
        }
        return up - dn + a.nf4_offset * xsum_c;
    } else {
        uint32_t u[16];
        decode<FMT>(w, a.cb, u);
        return dot16<FMT>(u, q4);
    }
}

__device__ __forceinline__ uint32_t scale_group_of(const GemvArgs &a, uint32_t c) {
    return a.sgc_shift < 32 ? c >> a.sgc_shift : c / a.sgc;
}

template <int FMT> __device__ __forceinline__ constexpr bool is_bitplane() {
    return FMT == FMT_BP4 || FMT == FMT_BP5 || FMT == FMT_BP6;
}

__host__ __device__ inline size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }

// ------------------------------------------------------------------------------------------------
// batch-1 kernel
// ------------------------------------------------------------------------------------------------
// Weight records travel global -> shared memory with cp.async (16-byte LDGSTS, L1 bypass).  Every
// quarter-warp owns a ring of NBATCH batches of BATCH slots; a slot holds one record plus the 16-byte
// granule with the eight bf16 scales of its rows.  One commit group per batch, retired strictly
// oldest-first by `cp.async.wait_group NBATCH-1`.  Unlike loads into registers, whose completion is
// tracked by a handful of per-warp scoreboards shared between old and new requests, this keeps
// (NBATCH-1)*BATCH .. NBATCH*BATCH records per quarter-warp in flight for the whole stream and costs
// no registers.
constexpr int BATCH = 2;
constexpr int NBATCH = 3;

template <int FMT> __host__ __device__ constexpr uint32_t slot_bytes() { return RawWords<FMT>::N * 32 + 16; }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int FMT>
__device__ __forceinline__ void read_slot(Raw<FMT> &o, const uint8_t *slot, uint32_t r) {
    const uint4 *p = reinterpret_cast<const uint4 *>(slot);
    uint4 a = p[r];
    o.w[0] = a.x; o.w[1] = a.y; o.w[2] = a.z; o.w[3] = a.w;
    if (FMT == FMT_NF3) {
        uint2 h = reinterpret_cast<const uint2 *>(slot + 128)[r];
        o.w[4] = h.x; o.w[5] = h.y;
        return;
    }
    uint4 b = p[8 + r];
    o.w[4] = b.x; o.w[5] = b.y; o.w[6] = b.z; o.w[7] = b.w;
    if (FMT == FMT_BP5) {
        uint2 h = reinterpret_cast<const uint2 *>(slot + 256)[r];
        o.w[8] = h.x; o.w[9] = h.y;
    }
    if (FMT == FMT_BP6) {
        uint4 h = p[16 + r];
        o.w[8] = h.x; o.w[9] = h.y; o.w[10] = h.z; o.w[11] = h.w;
    }
}

struct Smem1 { size_t xa, f, v, ring, total; };
__host__ __device__ inline Smem1 smem1_plan(uint32_t cols, uint32_t nc, uint32_t threads, uint32_t n_max, uint32_t slot) {
    Smem1 p;
    p.xa = align16(cols);                                   // {xs, xsum} pairs after the int8 activations
    p.f = p.xa + align16((size_t)nc * 8);                   // chain hand-off between the warps of a group
    p.v = p.f + align16((size_t)(threads / 32) * 8 * 4);
    p.ring = p.v + (size_t)n_max * threads * 8;             // private (v, w_scale) columns
    p.total = p.ring + (size_t)(threads / 8) * NBATCH * BATCH * slot;
    return p;
}

// blockDim.x = 32 * wpg * gpb: gpb row groups per CTA, each served by wpg warps (4*wpg K-slices).
template <int FMT>
__global__ void __launch_bounds__(256) gemv1_kernel(const GemvArgs a) {
    constexpr uint32_t SLOT = slot_bytes<FMT>();
    constexpr uint32_t GRANULES = RawWords<FMT>::N * 2;     // 16-byte pieces of one record
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t threads = blockDim.x;
    const uint32_t W = a.wpg, n_sl = 4 * W;
    const uint32_t base = a.nc / n_sl, rem = a.nc % n_sl;
    const uint32_t n_max = base + (rem != 0);               // CTA-uniform trip count
    const Smem1 sp = smem1_plan(a.cols, a.nc, threads, n_max, SLOT);
    int8_t *s_xq = reinterpret_cast<int8_t *>(smem);
    float2 *s_xa = reinterpret_cast<float2 *>(smem + sp.xa);   // .x = activation scale, .y = bits of the int32 chunk sum
    float *s_f = reinterpret_cast<float *>(smem + sp.f);
    float2 *s_v = reinterpret_cast<float2 *>(smem + sp.v);

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, r = lane & 7, q = lane >> 3;
    const uint32_t gl = warp / W, wg = warp % W;
    const uint32_t g = blockIdx.x * a.gpb + gl;
    const bool live = g < a.ngroups;
    const uint32_t sl = wg * 4 + q;                             // this quarter-warp's slice of the chunks
    const uint32_t c0 = sl * base + min(sl, rem);
    const uint32_t n_i = live ? base + (sl < rem) : 0;
    const uint8_t *rec = a.rec + ((size_t)g * a.nc + c0) * a.rec_bytes + r * 16;
    const uint16_t *ws_g = a.scales + (size_t)g * a.nsg * 8;
    uint8_t *ring = smem + sp.ring + (size_t)(tid >> 3) * (NBATCH * BATCH) * SLOT;
    const uint32_t ring_sa = (uint32_t)__cvta_generic_to_shared(ring) + r * 16;

    auto issue_batch = [&](uint32_t i0, uint32_t slot0) {     // records i0..i0+BATCH-1 -> slots slot0..
#pragma unroll
        for (uint32_t k = 0; k < BATCH; ++k) {
            const uint32_t i = i0 + k;
            if (i < n_i) {
                const uint8_t *src = rec + (size_t)i * a.rec_bytes;
                const uint32_t dst = ring_sa + (slot0 + k) * SLOT;
#pragma unroll
                for (uint32_t j = 0; j < (GRANULES + 7) / 8; ++j)
                    if (j * 8 + r < GRANULES) cp_async16(dst + j * 128, src + j * 128);
                if (r == 0) cp_async16(dst + GRANULES * 16, ws_g + (size_t)scale_group_of(a, c0 + i) * 8);
            }
        }
        cp_async_commit();          // one group per batch, possibly empty: keeps the group count in step
    };

    // the first NBATCH batches go out before anything else: their latency covers the staging below
#pragma unroll
    for (uint32_t b = 0; b < NBATCH; ++b) issue_batch(b * BATCH, b * BATCH);

    for (uint32_t i = tid; i < a.cols / 16; i += threads)
        reinterpret_cast<int4 *>(s_xq)[i] = __ldg(reinterpret_cast<const int4 *>(a.xq) + i);
    for (uint32_t i = tid; i < a.nc; i += threads)
        s_xa[i] = make_float2(__ldg(a.xs + i), __int_as_float(a.xsum != nullptr ? __ldg(a.xsum + i) : 0));
    __syncthreads();

    const uint32_t row = g * 8 + r;
    float2 *my_v = s_v + tid;
    uint32_t slot0 = 0;
    for (uint32_t i0 = 0; i0 < n_max; i0 += BATCH) {
        cp_async_wait<NBATCH - 1>();                // this thread's share of the oldest batch has landed
        __syncwarp();                               // ... and so have the scale granules lane 0 fetched
#pragma unroll
        for (uint32_t k = 0; k < BATCH; ++k) {
            const uint32_t i = i0 + k;
            if (i < n_i) {
                const uint8_t *slot = ring + (slot0 + k) * SLOT;
                Raw<FMT> w;
                read_slot<FMT>(w, slot, r);
                const float ws = bf16_bits_to_f32(reinterpret_cast<const uint16_t *>(slot + GRANULES * 16)[r]);
                const uint32_t c = c0 + i;
                const float2 xa = s_xa[c];
                const int xsum_c = __float_as_int(xa.y);
                const int acc = cell_dot<FMT>(w, a, reinterpret_cast<const int4 *>(s_xq + (size_t)c * 64), xsum_c);
                const int dot = is_bitplane<FMT>() ? 2 * acc - a.max_odd * xsum_c : acc;
                my_v[(size_t)i * threads] = make_float2(__fmul_rn(__int2float_rn(dot), xa.x), ws);
                if (a.int_dots != nullptr && row < a.rows) a.int_dots[(size_t)row * a.nc + c] = dot;
            }
        }
        __syncwarp();                               // every lane is done with the batch before it is refilled
        issue_batch(i0 + NBATCH * BATCH, slot0);
        slot0 = slot0 + BATCH == NBATCH * BATCH ? 0 : slot0 + BATCH;
    }
    cp_async_wait<0>();

    // ordered fp32 chain: slice after slice, quarter-warp to quarter-warp by shuffle, warp to warp via s_f
    float f = 0.0f;
    for (uint32_t round = 0; round < W; ++round) {
        if (wg == round) {
            if (round > 0) f = s_f[gl * 8 + r];
#pragma unroll
            for (uint32_t qq = 0; qq < 4; ++qq) {
                if (q == qq)
                    for (uint32_t i = 0; i < n_i; ++i) {
                        const float2 t = my_v[(size_t)i * threads];
                        if (s_xa[c0 + i].x != 0.0f) f = __fmaf_rn(t.x, t.y, f);
                    }
                const float up = __shfl_up_sync(0xffffffffu, f, 8);
                if (q == qq + 1) f = up;
            }
            if (q == 3 && live) {
                if (round + 1 == W) { if (row < a.rows) a.out[row] = f; }
                else s_f[gl * 8 + r] = f;
            }
        }
        if (W > 1) __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------------
// 2..8-token kernel: weights decoded once per record, reused for every token
// ------------------------------------------------------------------------------------------------
struct SmemPlan { size_t xq, xs, xsum, ws, v, total; };
__host__ __device__ inline SmemPlan smem_plan(uint32_t nt, uint32_t cols, uint32_t nc, uint32_t nsg, uint32_t gpb) {
    SmemPlan p;
    p.xq = 0;
    p.xs = align16((size_t)nt * cols);
    p.xsum = p.xs + align16((size_t)nt * nc * 4);
    p.ws = p.xsum + align16((size_t)nt * nc * 4);
    p.v = p.ws + align16((size_t)gpb * 8 * nsg * 2);
    p.total = p.v + (size_t)nt * gpb * nc * 8 * 4;
    return p;
}

template <int FMT, int NT>
__global__ void __launch_bounds__(256) gemm_small_kernel(const GemvArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    const SmemPlan sp = smem_plan(NT, a.cols, a.nc, a.nsg, a.gpb);
    int8_t *s_xq = reinterpret_cast<int8_t *>(smem + sp.xq);
    float *s_xs = reinterpret_cast<float *>(smem + sp.xs);
    int32_t *s_xsum = reinterpret_cast<int32_t *>(smem + sp.xsum);
    uint16_t *s_ws = reinterpret_cast<uint16_t *>(smem + sp.ws);
    float *s_v = reinterpret_cast<float *>(smem + sp.v);

    const uint32_t tid = threadIdx.x, r = tid & 7, qw = tid >> 3;
    const uint32_t g0 = blockIdx.x * a.gpb;
    const uint32_t ng = min(a.gpb, a.ngroups - g0);
    const uint32_t total = ng * a.nc;
    const uint8_t *rec0 = a.rec + (size_t)g0 * a.nc * a.rec_bytes;

    uint32_t L = qw;
    Raw<FMT> cur;
    if (L < total) load_raw<FMT>(cur, rec0 + (size_t)L * a.rec_bytes, r);

    {
        const uint32_t vec_per_tok = a.cols / 16;
        for (uint32_t i = tid; i < NT * vec_per_tok; i += 256) {
            uint32_t t = i / vec_per_tok, k = i % vec_per_tok;
            int4 v = make_int4(0, 0, 0, 0);
            if (t < a.n_tok) v = reinterpret_cast<const int4 *>(a.xq + (size_t)t * a.cols)[k];
            reinterpret_cast<int4 *>(s_xq + (size_t)t * a.cols)[k] = v;
        }
        for (uint32_t i = tid; i < NT * a.nc; i += 256) {
            uint32_t t = i / a.nc;
            s_xs[i] = t < a.n_tok ? a.xs[i] : 0.0f;
            s_xsum[i] = (t < a.n_tok && a.xsum != nullptr) ? a.xsum[i] : 0;
        }
        const uint32_t n_ws = ng * 8 * a.nsg;                       // [group][sg][row], contiguous for the CTA
        const uint16_t *ws_src = a.scales + (size_t)g0 * 8 * a.nsg;
        for (uint32_t i = tid; i < n_ws; i += 256) s_ws[i] = ws_src[i];
    }
    __syncthreads();

    uint32_t c = L % a.nc, gl = L / a.nc;
    while (L < total) {
        const uint32_t Ln = L + 32;
        Raw<FMT> nxt;
        if (Ln < total) load_raw<FMT>(nxt, rec0 + (size_t)Ln * a.rec_bytes, r);
        uint32_t u[16];
        decode<FMT>(cur, a.cb, u);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const int4 *q = reinterpret_cast<const int4 *>(s_xq + (size_t)t * a.cols + (size_t)c * 64);
            int acc = dot16<FMT>(u, q);
            int dot = is_bitplane<FMT>() ? 2 * acc - a.max_odd * s_xsum[t * a.nc + c] : acc;
            s_v[((size_t)(t * a.gpb + gl) * a.nc + c) * 8 + r] = __fmul_rn(__int2float_rn(dot), s_xs[t * a.nc + c]);
            if (a.int_dots != nullptr && t < (int)a.n_tok) {
                uint32_t row = (g0 + gl) * 8 + r;
                if (row < a.rows) a.int_dots[((size_t)t * a.rows + row) * a.nc + c] = dot;
            }
        }
        cur = nxt;
        L = Ln;
        c += 32;
        while (c >= a.nc) { c -= a.nc; ++gl; }
    }
    __syncthreads();

    for (uint32_t idx = tid; idx < NT * ng * 8; idx += 256) {
        const uint32_t rr = idx & 7, gli = (idx >> 3) % ng, t = idx / (8 * ng);
        const uint32_t row = (g0 + gli) * 8 + rr;
        if (row >= a.rows || t >= a.n_tok) continue;
        const float *vv = s_v + ((size_t)(t * a.gpb + gli) * a.nc) * 8 + rr;
        const uint16_t *wsr = s_ws + (size_t)gli * a.nsg * 8 + rr;
        const float *sx = s_xs + (size_t)t * a.nc;
        float f = 0.0f;
        uint32_t cc = 0;
        for (uint32_t sg = 0; sg < a.nsg; ++sg) {
            const float ws = bf16_bits_to_f32(wsr[(size_t)sg * 8]);
            const uint32_t c_end = min(cc + a.sgc, a.nc);
            for (; cc < c_end; ++cc)
                if (sx[cc] != 0.0f) f = __fmaf_rn(vv[(size_t)cc * 8], ws, f);
        }
        a.out[(size_t)t * a.out_stride + row] = f;
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

template <int FMT>
static cudaError_t launch_gemv1(cudaStream_t stream, const GemvArgs &a, uint32_t grid) {
    const uint32_t threads = 32 * a.wpg * a.gpb, n_sl = 4 * a.wpg;
    const uint32_t n_max = a.nc / n_sl + (a.nc % n_sl != 0);
    const size_t smem = smem1_plan(a.cols, a.nc, threads, n_max, slot_bytes<FMT>()).total;
    if (smem > kSmemBudget) return cudaErrorInvalidValue;
    cudaError_t e = allow_big_smem(gemv1_kernel<FMT>, smem);
    if (e != cudaSuccess) return e;
    gemv1_kernel<FMT><<<grid, threads, smem, stream>>>(a);
    return cudaGetLastError();
}

template <int FMT, int NT>
static cudaError_t launch_small_one(cudaStream_t stream, const GemvArgs &a, size_t smem, uint32_t grid) {
    cudaError_t e = allow_big_smem(gemm_small_kernel<FMT, NT>, smem);
    if (e != cudaSuccess) return e;
    gemm_small_kernel<FMT, NT><<<grid, 256, smem, stream>>>(a);
    return cudaGetLastError();
}

template <int FMT>
static cudaError_t launch_small(cudaStream_t stream, const GemvArgs &a, uint32_t nt, size_t smem, uint32_t grid) {
    switch (nt) {
        case 2: return launch_small_one<FMT, 2>(stream, a, smem, grid);
        case 4: return launch_small_one<FMT, 4>(stream, a, smem, grid);
        default: return launch_small_one<FMT, 8>(stream, a, smem, grid);
    }
}

static uint32_t round_tokens(uint32_t n) { return n <= 1 ? 1 : n <= 2 ? 2 : n <= 4 ? 4 : 8; }

uint32_t gemv_max_tokens(const DeviceMatrix &m) {
    for (uint32_t nt = 8; nt > 1; nt >>= 1)
        if (smem_plan(nt, m.geom.cols, m.geom.nc, m.geom.nsg, 1).total <= kSmemBudget) return nt;
    return 1;
}

cudaError_t launch_gemv(cudaStream_t stream, const DeviceMatrix &m, const int8_t *xq, const float *xs,
                        const int32_t *xsum, uint32_t n_tok, float *out, size_t out_stride, int32_t *int_dots,
                        int sm_count, uint32_t *launches) {
    const MatrixGeom &g = m.geom;
    if (launches) *launches = 0;
    if (n_tok == 0) return cudaSuccess;
    if (n_tok > 8 || g.fmt == FMT_NF5 || g.fmt == FMT_E8Q2) return cudaErrorNotSupported;
    GemvArgs a;
    a.rec = m.d_rec; a.scales = m.d_scales; a.xq = xq; a.xs = xs; a.xsum = xsum; a.out = out; a.int_dots = int_dots;
    a.out_stride = out_stride;
    a.rows = g.rows; a.cols = g.cols; a.nc = g.nc; a.nsg = g.nsg; a.sgc = g.sgc; a.ngroups = g.ngroups;
    a.sgc_shift = 32;
    for (uint32_t sh = 0; sh < 4; ++sh) if ((1u << sh) == g.sgc) a.sgc_shift = sh;
    a.rec_bytes = g.rec_bytes; a.n_tok = n_tok; a.max_odd = g.max_odd; a.nf4_offset = g.nf4_offset;
    for (int i = 0; i < 8; ++i) {
        const uint8_t *b = reinterpret_cast<const uint8_t *>(g.codebook32) + 4 * i;
        a.cb[i] = (uint32_t)b[0] | ((uint32_t)b[1] << 8) | ((uint32_t)b[2] << 16) | ((uint32_t)b[3] << 24);
    }
    for (int i = 0; i < 2; ++i) {
        const uint8_t *h = g.nf4_hi + 4 * i, *l = g.nf4_lo + 4 * i;
        a.tab[i] = (uint32_t)h[0] | ((uint32_t)h[1] << 8) | ((uint32_t)h[2] << 16) | ((uint32_t)h[3] << 24);
        a.tab[2 + i] = (uint32_t)l[0] | ((uint32_t)l[1] << 8) | ((uint32_t)l[2] << 16) | ((uint32_t)l[3] << 24);
    }
    cudaError_t e;
    if (n_tok == 1) {
        // warps per row group: enough warps to keep ~24 per SM busy, at least one chunk per K-slice
        const uint32_t want_warps = 24u * (uint32_t)sm_count;
        uint32_t W = 1;
        while (W < 8 && g.ngroups * W < want_warps && 8 * W <= g.nc) W *= 2;
        a.wpg = W;
        a.gpb = W >= 4 ? 1 : 4 / W;
        const uint32_t grid = (g.ngroups + a.gpb - 1) / a.gpb;
        const bool nf4_fast = g.fmt == FMT_NF4 && g.nf4_split_ok && (g.nf4_offset == 0 || xsum != nullptr);
        switch (g.fmt) {
            case FMT_BP4: e = launch_gemv1<FMT_BP4>(stream, a, grid); break;
            case FMT_BP5: e = launch_gemv1<FMT_BP5>(stream, a, grid); break;
            case FMT_BP6: e = launch_gemv1<FMT_BP6>(stream, a, grid); break;
            case FMT_NF4: e = nf4_fast ? launch_gemv1<FMT_NF4>(stream, a, grid) : launch_gemv1<FMT_NF4G>(stream, a, grid); break;
            case FMT_NF3: e = launch_gemv1<FMT_NF3>(stream, a, grid); break;
            default: return cudaErrorNotSupported;
        }
    } else {
        const uint32_t nt = round_tokens(n_tok);
        uint32_t gpb = 1;
        for (uint32_t cand : {4u, 2u}) {
            if ((g.ngroups + cand - 1) / cand >= (uint32_t)(2 * sm_count) &&
                smem_plan(nt, g.cols, g.nc, g.nsg, cand).total <= 64 * 1024) { gpb = cand; break; }
        }
        a.gpb = gpb; a.wpg = 1;
        const size_t smem = smem_plan(nt, g.cols, g.nc, g.nsg, gpb).total;
        if (smem > kSmemBudget) return cudaErrorInvalidValue;
        const uint32_t grid = (g.ngroups + gpb - 1) / gpb;
        switch (g.fmt) {
            case FMT_BP4: e = launch_small<FMT_BP4>(stream, a, nt, smem, grid); break;
            case FMT_BP5: e = launch_small<FMT_BP5>(stream, a, nt, smem, grid); break;
            case FMT_BP6: e = launch_small<FMT_BP6>(stream, a, nt, smem, grid); break;
            case FMT_NF4: e = launch_small<FMT_NF4G>(stream, a, nt, smem, grid); break;
            case FMT_NF3: e = launch_small<FMT_NF3>(stream, a, nt, smem, grid); break;
            default: return cudaErrorNotSupported;
        }
    }
    if (e == cudaSuccess && launches) *launches = 1;
    return e;
}

}  // namespace k2t

// Quantized GEMV / small-N GEMM for bit-plane (b4/b5/b6) and codebook (NF4/NF3) matrices.
//
// Arithmetic contract (reference: sdot_one_stripe_neon, src/kernels/simd_lut.rs:3763-3868, and
// nf_sdot_one_stripe_neon, 6071-6181; batch forms 4228-4331 / 6689-7029):
//   per row r and 64-column chunk c:  a = sum_i code_i * q_i           (exact int32)
//       bit-plane: dot = 2a - (2^B-1) * xsum[c]      NF: dot = a
//   f = 0;  for c ascending, skipping chunks with xs[c] == 0:
//       f = fmaf((float)dot * xs[c], w_scale[r, c / sgc], f)
// The integer part is computed in parallel by all lanes; the fp32 chain is then run per row in
// ascending chunk order by one lane, so outputs are bit-identical to the reference order.
//
// Work decomposition: a CTA owns `gpb` consecutive 8-row groups and all K.  A quarter-warp
// (8 lanes = 8 rows) handles one (group, chunk) record per step; the four quarter-warps of a warp
// take four consecutive records, i.e. 1 KiB (b4) of contiguous weights per warp step, each
// 128-bit load of a quarter-warp covering one 128-byte line.  Activations (int8, <= 18.5 KiB)
// sit in shared memory and are read as quarter-warp broadcasts.
#include "k2t_device.cuh"
#include "k2t_kernels.h"

namespace k2t {

struct GemvArgs {
    const uint8_t *rec;
    const uint16_t *scales;
    const int8_t *xq;
    const float *xs;
    const int32_t *xsum;
    float *out;
    int32_t *int_dots;
    size_t out_stride;
    uint32_t rows, cols, nc, nsg, sgc, ngroups, rec_bytes, n_tok, gpb;
    int32_t max_odd;
    uint32_t cb[8];   // expanded codebook, 4 centroids per word
};

struct Raw {          // the bytes one lane loads for one (group, chunk) record
    uint4 a, b, c;
};

template <int FMT>
__device__ __forceinline__ Raw load_raw(const uint8_t *rec, uint32_t r) {
    Raw w;
    const uint4 *p = reinterpret_cast<const uint4 *>(rec);
    w.a = ldg_stream(p + r);
    w.b = make_uint4(0, 0, 0, 0);
    w.c = make_uint4(0, 0, 0, 0);
    if (FMT == FMT_BP4 || FMT == FMT_BP5 || FMT == FMT_BP6 || FMT == FMT_NF4 || FMT == FMT_NF5) w.b = ldg_stream(p + 8 + r);
    if (FMT == FMT_BP5 || FMT == FMT_NF5) {
        uint2 h = ldg_stream(reinterpret_cast<const uint2 *>(rec + 256) + r);
        w.c.x = h.x; w.c.y = h.y;
    }
    if (FMT == FMT_BP6) w.c = ldg_stream(p + 16 + r);
    if (FMT == FMT_NF3) {
        uint2 h = ldg_stream(reinterpret_cast<const uint2 *>(rec + 128) + r);
        w.c.x = h.x; w.c.y = h.y;
    }
    return w;
}

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) {
    return i == 0 ? v.x : i == 1 ? v.y : i == 2 ? v.z : v.w;
}

// Expands a record into 16 words of four weight bytes each: u[j] holds columns 4j..4j+3 of the chunk.
// Bit-plane formats give unsigned codes 0..63, NF formats signed centroids.
template <int FMT>
__device__ __forceinline__ void decode(const Raw &w, const uint32_t (&cb)[8], uint32_t (&u)[16]) {
    if (FMT == FMT_BP4 || FMT == FMT_BP5 || FMT == FMT_BP6) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t x = word_of(w.a, i), y = word_of(w.b, i);
            u[2 * i] = x & 0x0F0F0F0Fu;
            u[2 * i + 1] = (x >> 4) & 0x0F0F0F0Fu;
            u[8 + 2 * i] = y & 0x0F0F0F0Fu;
            u[8 + 2 * i + 1] = (y >> 4) & 0x0F0F0F0Fu;
        }
        if (FMT == FMT_BP5) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {   // plane-4 bit of column 4j+b sits at bit j of byte b
                uint32_t h0 = j <= 4 ? (w.c.x << (4 - j)) : (w.c.x >> (j - 4));
                uint32_t h1 = j <= 4 ? (w.c.y << (4 - j)) : (w.c.y >> (j - 4));
                u[j] = lop3_or_and(u[j], h0, 0x10101010u);
                u[8 + j] = lop3_or_and(u[8 + j], h1, 0x10101010u);
            }
        }
        if (FMT == FMT_BP6) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {   // planes 4,5 of column 16v+4f+b sit at bits 2f,2f+1 of byte b
                uint32_t h = word_of(w.c, v);
                u[4 * v + 0] = lop3_or_and(u[4 * v + 0], h << 4, 0x30303030u);
                u[4 * v + 1] = lop3_or_and(u[4 * v + 1], h << 2, 0x30303030u);
                u[4 * v + 2] = lop3_or_and(u[4 * v + 2], h, 0x30303030u);
                u[4 * v + 3] = lop3_or_and(u[4 * v + 3], h >> 2, 0x30303030u);
            }
        }
    } else if (FMT == FMT_NF4) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {      // word i = eight consecutive 4-bit indices (columns 8i..8i+7)
            uint32_t x = i < 4 ? word_of(w.a, i) : word_of(w.b, i - 4);
            uint32_t lo3 = x & 0x77777777u, hb = x & 0x88888888u, hs = hb << 4;
            uint32_t lo3h = lo3 >> 16;
            uint32_t m0 = prmt(hs, hb, 0xD9C8u), m1 = prmt(hs, hb, 0xFBEAu);   // byte masks: index bit 3
            u[2 * i] = lop3_select(prmt(cb[0], cb[1], lo3), prmt(cb[2], cb[3], lo3), m0);
            u[2 * i + 1] = lop3_select(prmt(cb[0], cb[1], lo3h), prmt(cb[2], cb[3], lo3h), m1);
        }
    } else if (FMT == FMT_NF3) {
        uint32_t W[6] = {w.a.x, w.a.y, w.a.z, w.a.w, w.c.x, w.c.y};
#pragma unroll
        for (int i = 0; i < 6; ++i) {      // columns 8i..8i+7: index in the low 3 bits of each nibble
            uint32_t s = W[i] & 0x77777777u;
            u[2 * i] = prmt(cb[0], cb[1], s);
            u[2 * i + 1] = prmt(cb[0], cb[1], s >> 16);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {      // columns 48+8h..: index bit j = bit 3 of the nibbles of W[3h+j]
            uint32_t s = (W[3 * h] >> 3) & 0x11111111u;
            s = lop3_or_and(s, W[3 * h + 1] >> 2, 0x22222222u);
            s = lop3_or_and(s, W[3 * h + 2] >> 1, 0x44444444u);
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

__host__ __device__ inline size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }

struct SmemPlan {
    size_t xq, xs, xsum, ws, v, total;
};
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
__global__ void __launch_bounds__(256) gemv_kernel(const GemvArgs a) {
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

    // first weight record is requested before anything else so HBM latency overlaps the staging below
    uint32_t L = qw;
    Raw cur;
    if (L < total) cur = load_raw<FMT>(rec0 + (size_t)L * a.rec_bytes, r);

    // stage activations (tokens beyond n_tok are zero and skipped) and this CTA's weight scales
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
        const uint32_t n_ws = ng * 8 * a.nsg;                       // bf16 count, contiguous for the CTA
        const uint16_t *ws_src = a.scales + (size_t)g0 * 8 * a.nsg;
        for (uint32_t i = tid; i < n_ws; i += 256) s_ws[i] = ws_src[i];
    }
    __syncthreads();

    while (L < total) {
        const uint32_t Ln = L + 32;
        Raw nxt;
        if (Ln < total) nxt = load_raw<FMT>(rec0 + (size_t)Ln * a.rec_bytes, r);
        uint32_t u[16];
        decode<FMT>(cur, a.cb, u);
        const uint32_t c = L % a.nc, gl = L / a.nc;
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const int4 *q = reinterpret_cast<const int4 *>(s_xq + (size_t)t * a.cols + (size_t)c * 64);
            int acc = dot16<FMT>(u, q);
            int dot = (FMT == FMT_BP4 || FMT == FMT_BP5 || FMT == FMT_BP6)
                          ? 2 * acc - a.max_odd * s_xsum[t * a.nc + c] : acc;
            s_v[((size_t)(t * a.gpb + gl) * a.nc + c) * 8 + r] = __fmul_rn(__int2float_rn(dot), s_xs[t * a.nc + c]);
            if (a.int_dots != nullptr && t < (int)a.n_tok) {
                uint32_t row = (g0 + gl) * 8 + r;
                if (row < a.rows) a.int_dots[((size_t)t * a.rows + row) * a.nc + c] = dot;
            }
        }
        cur = nxt;
        L = Ln;
    }
    __syncthreads();

    // ordered fp32 chain: one lane per (token, row)
    for (uint32_t idx = tid; idx < NT * ng * 8; idx += 256) {
        const uint32_t rr = idx & 7, gl = (idx >> 3) % ng, t = idx / (8 * ng);
        const uint32_t row = (g0 + gl) * 8 + rr;
        if (row >= a.rows || t >= a.n_tok) continue;
        const float *vv = s_v + ((size_t)(t * a.gpb + gl) * a.nc) * 8 + rr;
        const uint16_t *wsr = s_ws + (size_t)(gl * 8 + rr) * a.nsg;
        const float *sx = s_xs + (size_t)t * a.nc;
        float f = 0.0f;
        uint32_t c = 0;
        for (uint32_t sg = 0; sg < a.nsg; ++sg) {
            const float ws = bf16_bits_to_f32(wsr[sg]);
            const uint32_t c_end = min(c + a.sgc, a.nc);
            for (; c < c_end; ++c)
                if (sx[c] != 0.0f) f = __fmaf_rn(vv[(size_t)c * 8], ws, f);
        }
        a.out[(size_t)t * a.out_stride + row] = f;
    }
}

template <int FMT, int NT>
static cudaError_t launch_one(cudaStream_t stream, const GemvArgs &a, size_t smem, uint32_t grid) {
    static bool configured = false;   // per instantiation; the attribute is process-wide for the function
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemv_kernel<FMT, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    gemv_kernel<FMT, NT><<<grid, 256, smem, stream>>>(a);
    return cudaGetLastError();
}

template <int FMT>
static cudaError_t launch_fmt(cudaStream_t stream, const GemvArgs &a, uint32_t nt, size_t smem, uint32_t grid) {
    switch (nt) {
        case 1: return launch_one<FMT, 1>(stream, a, smem, grid);
        case 2: return launch_one<FMT, 2>(stream, a, smem, grid);
        case 4: return launch_one<FMT, 4>(stream, a, smem, grid);
        default: return launch_one<FMT, 8>(stream, a, smem, grid);
    }
}

static uint32_t round_tokens(uint32_t n) { return n <= 1 ? 1 : n <= 2 ? 2 : n <= 4 ? 4 : 8; }
static const size_t kSmemBudget = 196 * 1024;

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
    const uint32_t nt = round_tokens(n_tok);
    // groups per CTA: as many as keep >= 2 CTAs per SM and fit shared memory
    uint32_t gpb = 1;
    for (uint32_t cand : {4u, 2u}) {
        if ((g.ngroups + cand - 1) / cand >= (uint32_t)(2 * sm_count) &&
            smem_plan(nt, g.cols, g.nc, g.nsg, cand).total <= 64 * 1024) { gpb = cand; break; }
    }
    const size_t smem = smem_plan(nt, g.cols, g.nc, g.nsg, gpb).total;
    if (smem > kSmemBudget) return cudaErrorInvalidValue;
    GemvArgs a;
    a.rec = m.d_rec; a.scales = m.d_scales; a.xq = xq; a.xs = xs; a.xsum = xsum; a.out = out; a.int_dots = int_dots;
    a.out_stride = out_stride;
    a.rows = g.rows; a.cols = g.cols; a.nc = g.nc; a.nsg = g.nsg; a.sgc = g.sgc; a.ngroups = g.ngroups;
    a.rec_bytes = g.rec_bytes; a.n_tok = n_tok; a.gpb = gpb; a.max_odd = g.max_odd;
    for (int i = 0; i < 8; ++i) {
        const uint8_t *b = reinterpret_cast<const uint8_t *>(g.codebook32) + 4 * i;
        a.cb[i] = (uint32_t)b[0] | ((uint32_t)b[1] << 8) | ((uint32_t)b[2] << 16) | ((uint32_t)b[3] << 24);
    }
    const uint32_t grid = (g.ngroups + gpb - 1) / gpb;
    cudaError_t e;
    switch (g.fmt) {
        case FMT_BP4: e = launch_fmt<FMT_BP4>(stream, a, nt, smem, grid); break;
        case FMT_BP5: e = launch_fmt<FMT_BP5>(stream, a, nt, smem, grid); break;
        case FMT_BP6: e = launch_fmt<FMT_BP6>(stream, a, nt, smem, grid); break;
        case FMT_NF4: e = launch_fmt<FMT_NF4>(stream, a, nt, smem, grid); break;
        case FMT_NF3: e = launch_fmt<FMT_NF3>(stream, a, nt, smem, grid); break;
        default: return cudaErrorNotSupported;
    }
    if (e == cudaSuccess && launches) *launches = 1;
    return e;
}

}  // namespace k2t

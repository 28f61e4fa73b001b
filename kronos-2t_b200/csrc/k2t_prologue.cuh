// CTA-wide builders of a GEMV's int8 activation in shared memory: the small operators of a decode step that sit between
// two projections, computed by every CTA of the consuming GEMV for itself (a few KB of fp32 from L2, nothing to exchange),
// as the workers of the reference's forward_token_sdot_megakernel do (src/model/real_llm.rs:6927-6953 residual + RMSNorm +
// rotation + int8 in front of qkv / gate_up / lm_head, 6723-6730 SwiGLU in front of down).  Arithmetic and summation orders
// are those of rmsnorm_quant_kernel / swiglu_quant_kernel / embed_kernel / moe_combine_kernel, so the results are theirs
// bit for bit.
#pragma once
#include "k2t_model_device.cuh"

namespace k2t {

enum ProMode : uint32_t { PRO_NORM = 1, PRO_SWIGLU = 2, PRO_EMBED_NORM = 3 };

struct FusedPro {
    uint32_t mode;
    uint32_t n;                  // activation length = columns of the matrix
    uint32_t chunk0;             // global index of the activation's first 64-value chunk (sign masks of the rotation)
    float eps;
    // PRO_NORM: x = x_in + delta, RMSNorm with norm_w.  delta = a projection output [n] (may be null), or - n_slot > 0 -
    // the weighted sum of n_slot expert outputs moe_out[slot][n] in slot order (moe_combine_kernel's arithmetic).
    const float *x_in, *delta, *norm_w;
    const float *moe_out, *route_w;
    uint32_t n_slot;
    uint32_t swiglu_exp_cr;      // PRO_SWIGLU: 1 = correctly rounded exp (expert records), 0 = the NEON polynomial
    float *x_out;                // PRO_NORM / PRO_EMBED_NORM: CTA 0 stores x here (a buffer other than x_in), or null
    float *x_norm_out;           // PRO_NORM: CTA 0 also stores the normalised fp32 vector (router input), or null
    const float *gate_up;        // PRO_SWIGLU: [2 n], gate then up
    EmbedArgs embed;             // PRO_EMBED_NORM: x = embedding row of *embed.token
};

struct ActSmem {                 // all in shared memory
    float *x;                    // [n] fp32 staging (PRO_NORM / PRO_EMBED_NORM)
    int8_t *xq;                  // [n]
    float *xs;                   // [n / 64]
    int32_t *xm;                 // [n / 64]
    float *inv;                  // [1]
};
__host__ __device__ inline size_t pro_round(size_t v) { return (v + 127) & ~(size_t)127; }
__host__ __device__ inline size_t act_smem_bytes(uint32_t mode, uint32_t n) {
    return (mode == PRO_SWIGLU ? 0 : pro_round((size_t)n * 4)) + pro_round(n) + 2 * pro_round((size_t)n / 64 * 4) + 128;
}
__device__ __forceinline__ ActSmem act_carve(uint8_t *base, uint32_t mode, uint32_t n) {
    ActSmem s;
    size_t off = 0;
    s.x = reinterpret_cast<float *>(base); off += mode == PRO_SWIGLU ? 0 : pro_round((size_t)n * 4);
    s.xq = reinterpret_cast<int8_t *>(base + off); off += pro_round(n);
    s.xs = reinterpret_cast<float *>(base + off); off += pro_round((size_t)n / 64 * 4);
    s.xm = reinterpret_cast<int32_t *>(base + off); off += pro_round((size_t)n / 64 * 4);
    s.inv = reinterpret_cast<float *>(base + off);
    return s;
}

// rotation + int8 of chunk c (values v0, v1 of this lane) into the shared activation
__device__ __forceinline__ void pro_store_chunk(const ActSmem &s, float v0, float v1, uint32_t c, uint32_t chunk0, uint32_t lane) {
    warp_fwht64(v0, v1, chunk0 + c, lane);
    int q0, q1, sum;
    float sc;
    warp_quant64(v0, v1, q0, q1, sc, sum);
    reinterpret_cast<char2 *>(s.xq + (size_t)c * 64)[lane] = make_char2((signed char)q0, (signed char)q1);
    if (lane == 0) { s.xs[c] = sc; s.xm[c] = sum; }
}

// s.x holds n fp32 values: RMSNorm (sum of squares in the CPU's 16-accumulator order, see rmsnorm_quant_kernel) +
// rotation + int8.  Ends with a CTA barrier: the activation is complete.
__device__ __forceinline__ void cta_norm_quant(const ActSmem &s, const FusedPro &p) {
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5, n = p.n, nc = n / 64;
    if (warp == 0) {
        float acc = 0.0f;
        if (lane < 16) {
#pragma unroll 8
            for (uint32_t i = lane; i < n; i += 16) { const float v = s.x[i]; acc = __fmaf_rn(v, v, acc); }
        }
        float t = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 4));
        t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 8));
        t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 1));
        t = __fadd_rn(t, __shfl_down_sync(0xffffffffu, t, 2));
        if (lane == 0) *s.inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(t, (float)n), p.eps)));
    }
    __syncthreads();
    const float inv = *s.inv;
    const bool tap = p.x_norm_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
    // two chunks per round: their shuffle chains are independent and interleave
    for (uint32_t c = warp; c < nc; c += 2 * nwarp) {
        const uint32_t c2 = c + nwarp;
        const bool two = c2 < nc;
        float2 a = reinterpret_cast<const float2 *>(s.x + (size_t)c * 64)[lane];
        float2 b = two ? reinterpret_cast<const float2 *>(s.x + (size_t)c2 * 64)[lane] : make_float2(0.0f, 0.0f);
        const float2 wa = __ldg(reinterpret_cast<const float2 *>(p.norm_w + (size_t)c * 64) + lane);
        const float2 wb = two ? __ldg(reinterpret_cast<const float2 *>(p.norm_w + (size_t)c2 * 64) + lane) : make_float2(0.0f, 0.0f);
        a.x = __fmul_rn(__fmul_rn(a.x, inv), wa.x); a.y = __fmul_rn(__fmul_rn(a.y, inv), wa.y);
        b.x = __fmul_rn(__fmul_rn(b.x, inv), wb.x); b.y = __fmul_rn(__fmul_rn(b.y, inv), wb.y);
        if (tap) {
            reinterpret_cast<float2 *>(p.x_norm_out + (size_t)c * 64)[lane] = a;
            if (two) reinterpret_cast<float2 *>(p.x_norm_out + (size_t)c2 * 64)[lane] = b;
        }
        warp_fwht64(a.x, a.y, p.chunk0 + c, lane);
        warp_fwht64(b.x, b.y, p.chunk0 + c2, lane);
        int qa0, qa1, sa, qb0, qb1, sb;
        float sca, scb;
        warp_quant64(a.x, a.y, qa0, qa1, sca, sa);
        warp_quant64(b.x, b.y, qb0, qb1, scb, sb);
        reinterpret_cast<char2 *>(s.xq + (size_t)c * 64)[lane] = make_char2((signed char)qa0, (signed char)qa1);
        if (two) reinterpret_cast<char2 *>(s.xq + (size_t)c2 * 64)[lane] = make_char2((signed char)qb0, (signed char)qb1);
        if (lane == 0) {
            s.xs[c] = sca; s.xm[c] = sa;
            if (two) { s.xs[c2] = scb; s.xm[c2] = sb; }
        }
    }
    __syncthreads();
}

// x = x_in + delta into s.x (CTA 0 also stores it to x_out), then norm + quant
__device__ __forceinline__ void cta_residual_norm_quant(const ActSmem &s, const FusedPro &p) {
    const bool keep = p.x_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
    for (uint32_t i = threadIdx.x; i < p.n / 4; i += blockDim.x) {
        float4 v = __ldcg(reinterpret_cast<const float4 *>(p.x_in) + i);
        if (p.n_slot > 0) {          // sum over the routes in slot order: acc = acc + w * out (separate multiply and add)
            float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (uint32_t sl = 0; sl < p.n_slot; ++sl) {
                const float w = __ldcg(p.route_w + sl);
                const float4 o = __ldcg(reinterpret_cast<const float4 *>(p.moe_out + (size_t)sl * p.n) + i);
                acc.x = __fadd_rn(acc.x, __fmul_rn(w, o.x)); acc.y = __fadd_rn(acc.y, __fmul_rn(w, o.y));
                acc.z = __fadd_rn(acc.z, __fmul_rn(w, o.z)); acc.w = __fadd_rn(acc.w, __fmul_rn(w, o.w));
            }
            v.x = __fadd_rn(v.x, acc.x); v.y = __fadd_rn(v.y, acc.y); v.z = __fadd_rn(v.z, acc.z); v.w = __fadd_rn(v.w, acc.w);
        } else if (p.delta != nullptr) {
            const float4 d = __ldcg(reinterpret_cast<const float4 *>(p.delta) + i);
            v.x = __fadd_rn(v.x, d.x); v.y = __fadd_rn(v.y, d.y); v.z = __fadd_rn(v.z, d.z); v.w = __fadd_rn(v.w, d.w);
        }
        reinterpret_cast<float4 *>(s.x)[i] = v;
        if (keep) reinterpret_cast<float4 *>(p.x_out)[i] = v;
    }
    __syncthreads();
    cta_norm_quant(s, p);
}

// x = embedding row of the current token (embed_kernel), then norm + quant
__device__ __forceinline__ void cta_embed_norm_quant(const ActSmem &s, const FusedPro &p) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const EmbedArgs &e = p.embed;
    const uint32_t tok = __ldcg(e.token);
    const bool keep = p.x_out != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
    for (uint32_t c = warp; c < e.nc; c += nwarp) {
        float v0, v1;
        if (e.embed_bf16 != nullptr) {
            const uint16_t *row = e.embed_bf16 + (size_t)tok * e.nc * 64 + (size_t)c * 64;
            v0 = bf16_bits_to_f32(row[2 * lane]);
            v1 = bf16_bits_to_f32(row[2 * lane + 1]);
        } else {
            v0 = cell_value(e, tok, c, 2 * lane);
            v1 = cell_value(e, tok, c, 2 * lane + 1);
            warp_ifwht64(v0, v1, c, lane);
        }
        reinterpret_cast<float2 *>(s.x + (size_t)c * 64)[lane] = make_float2(v0, v1);
        if (keep) reinterpret_cast<float2 *>(p.x_out + (size_t)c * 64)[lane] = make_float2(v0, v1);
    }
    __syncthreads();
    cta_norm_quant(s, p);
}

__device__ __forceinline__ float swiglu_one(float g, float u, bool cr) {
    const float e = cr ? (float)exp((double)-g) : exp_poly(-g);
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, e)), u);
}

// SwiGLU of gate_up[2 n] + rotation + int8 (swiglu_quant_kernel / expert_swiglu_quant_kernel); two chunks per round
__device__ __forceinline__ void cta_swiglu_quant(const ActSmem &s, const FusedPro &p, const float *gate_up) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5, n = p.n, nc = n / 64;
    const bool cr = p.swiglu_exp_cr != 0;
    for (uint32_t c = warp; c < nc; c += 2 * nwarp) {
        const uint32_t c2 = c + nwarp;
        const bool two = c2 < nc;
        const float2 ga = __ldcg(reinterpret_cast<const float2 *>(gate_up + (size_t)c * 64) + lane);
        const float2 ua = __ldcg(reinterpret_cast<const float2 *>(gate_up + n + (size_t)c * 64) + lane);
        const float2 gb = two ? __ldcg(reinterpret_cast<const float2 *>(gate_up + (size_t)c2 * 64) + lane) : make_float2(0.0f, 0.0f);
        const float2 ub = two ? __ldcg(reinterpret_cast<const float2 *>(gate_up + n + (size_t)c2 * 64) + lane) : make_float2(0.0f, 0.0f);
        float a0 = swiglu_one(ga.x, ua.x, cr), a1 = swiglu_one(ga.y, ua.y, cr);
        float b0 = swiglu_one(gb.x, ub.x, cr), b1 = swiglu_one(gb.y, ub.y, cr);
        warp_fwht64(a0, a1, p.chunk0 + c, lane);
        warp_fwht64(b0, b1, p.chunk0 + c2, lane);
        int qa0, qa1, sa, qb0, qb1, sb;
        float sca, scb;
        warp_quant64(a0, a1, qa0, qa1, sca, sa);
        warp_quant64(b0, b1, qb0, qb1, scb, sb);
        reinterpret_cast<char2 *>(s.xq + (size_t)c * 64)[lane] = make_char2((signed char)qa0, (signed char)qa1);
        if (two) reinterpret_cast<char2 *>(s.xq + (size_t)c2 * 64)[lane] = make_char2((signed char)qb0, (signed char)qb1);
        if (lane == 0) {
            s.xs[c] = sca; s.xm[c] = sa;
            if (two) { s.xs[c2] = scb; s.xm[c2] = sb; }
        }
    }
    __syncthreads();
}

__device__ __forceinline__ void cta_build_activation(const ActSmem &s, const FusedPro &p, const float *gate_up) {
    if (p.mode == PRO_NORM) cta_residual_norm_quant(s, p);
    else if (p.mode == PRO_SWIGLU) cta_swiglu_quant(s, p, gate_up);
    else cta_embed_norm_quant(s, p);
}

}  // namespace k2t

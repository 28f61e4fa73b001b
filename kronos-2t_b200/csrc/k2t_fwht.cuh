// Warp-level signed FWHT-64 + int8 chunk quantization.
//
// One warp owns one 64-element block: lane l holds elements 2l and 2l+1.  The butterfly
// order is the natural-order Walsh-Hadamard of fwht64_signed_inplace_scalar
// (src/kernels/hadamard.rs:71-99): stage h pairs element j with j+h, the low element
// becomes a+b and the high one a-b.  Stage h=1 is in-lane, stages 2..32 exchange with lane
// l ^ (h/2).  Each output is produced by exactly the additions of the scalar code, in the
// same order, so results are bit-identical to the reference (floating-point add is commutative).
#pragma once
#include "k2t_device.cuh"

namespace k2t {

// The two sign words of a lane (elements 2l, 2l+1 of `block`).  They depend on nothing a kernel computes, so kernels on a
// latency chain fetch them before they wait for their predecessor (the SplitMix64 rounds cost about a hundred cycles).
struct FwhtSigns { uint32_t s0, s1; };
__device__ __forceinline__ FwhtSigns fwht_signs(uint64_t block, uint32_t lane) {
    return FwhtSigns{rademacher_sign(block, 2 * lane), rademacher_sign(block, 2 * lane + 1)};
}

// In: v0/v1 = elements 2l, 2l+1 of the block (already RMS-normalised if wanted).
// Out: rotated values  (1/8) * H64 * D_block * x.
__device__ __forceinline__ void warp_fwht64(float &v0, float &v1, const FwhtSigns sg, uint32_t lane) {
    v0 = __fmul_rn(__uint_as_float(__float_as_uint(v0) ^ sg.s0), 0.125f);
    v1 = __fmul_rn(__uint_as_float(__float_as_uint(v1) ^ sg.s1), 0.125f);
    float a = __fadd_rn(v0, v1), b = __fsub_rn(v0, v1);
    v0 = a; v1 = b;
#pragma unroll
    for (uint32_t m = 1; m < 32; m <<= 1) {
        float o0 = __shfl_xor_sync(0xffffffffu, v0, m);
        float o1 = __shfl_xor_sync(0xffffffffu, v1, m);
        bool hi = (lane & m) != 0;   // this lane holds the `b` element of the pair
        v0 = hi ? __fsub_rn(o0, v0) : __fadd_rn(v0, o0);
        v1 = hi ? __fsub_rn(o1, v1) : __fadd_rn(v1, o1);
    }
}

__device__ __forceinline__ void warp_fwht64(float &v0, float &v1, uint64_t block, uint32_t lane) {
    warp_fwht64(v0, v1, fwht_signs(block, lane), lane);
}

// Inverse: butterflies, then *0.125, then sign (ifwht64_signed_inplace_scalar, hadamard.rs:200-228).
__device__ __forceinline__ void warp_ifwht64(float &v0, float &v1, const FwhtSigns sg, uint32_t lane) {
    float a = __fadd_rn(v0, v1), b = __fsub_rn(v0, v1);
    v0 = a; v1 = b;
#pragma unroll
    for (uint32_t m = 1; m < 32; m <<= 1) {
        float o0 = __shfl_xor_sync(0xffffffffu, v0, m);
        float o1 = __shfl_xor_sync(0xffffffffu, v1, m);
        bool hi = (lane & m) != 0;
        v0 = hi ? __fsub_rn(o0, v0) : __fadd_rn(v0, o0);
        v1 = hi ? __fsub_rn(o1, v1) : __fadd_rn(v1, o1);
    }
    v0 = __uint_as_float(__float_as_uint(__fmul_rn(v0, 0.125f)) ^ sg.s0);
    v1 = __uint_as_float(__float_as_uint(__fmul_rn(v1, 0.125f)) ^ sg.s1);
}
__device__ __forceinline__ void warp_ifwht64(float &v0, float &v1, uint64_t block, uint32_t lane) {
    warp_ifwht64(v0, v1, fwht_signs(block, lane), lane);
}

// Per-chunk int8 quantization of one rotated block held by a warp
// (populate_chunk_fwht_scalar, src/kernels/simd_lut.rs:3176-3195):
// max|v| <= f32::EPSILON -> zeros; else q = rne(v * (127/max)), scale = max/127, sum = sum(q).
// Returns the two int8 values of this lane; scale and sum are valid in every lane.
__device__ __forceinline__ void warp_quant64(float v0, float v1, int &q0, int &q1, float &scale, int &sum) {
    float mx = fmaxf(fabsf(v0), fabsf(v1));
#pragma unroll
    for (uint32_t m = 16; m > 0; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
    if (mx <= 1.1920929e-07f) {
        q0 = q1 = 0; scale = 0.0f; sum = 0;
        return;
    }
    float inv = __fdiv_rn(127.0f, mx);
    q0 = __float2int_rn(__fmul_rn(v0, inv));
    q1 = __float2int_rn(__fmul_rn(v1, inv));
    int s = q0 + q1;
#pragma unroll
    for (uint32_t m = 16; m > 0; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
    sum = s;
    scale = __fdiv_rn(mx, 127.0f);
}

}  // namespace k2t
